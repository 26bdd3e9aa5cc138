/*
 * CPU oracle for the duckdb-ann GPU search path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic the reference performs on its
 * CPU path.  Only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark may link or call it; the CUDA library never does.
 *
 * Parity status.  The reference holds no stored golden vectors for its FAISS
 * or diskann-vector results (libfaiss 1.13.2 and diskann-vector 0.45.0 are
 * third-party and not vendored), so for the large seeded configurations this
 * oracle is "parity unpinned".  It IS pinned on every known answer the
 * reference's own tests contain (squared-L2 2.0 / 0.020000001, inner product
 * 1.0, IVFFlat ids 1,2,7, batch distances 0.0 / 0.5, SQ8 nearest neighbour
 * unchanged); those fixtures live in tests/golden/.
 *
 * Conventions (reference file:line, paths relative to the reference root):
 *   - batch L2 is the SQUARED distance, batch IP is the NEGATED dot product
 *     (src/ann_search.cpp:702-720, rust_lib/src/distance.rs:15-25,
 *      faiss-metal/shaders/diskann_distance.metal:148,192).
 *   - FAISS-style search returns squared L2 ascending / raw dot descending,
 *     sorted best first, missing slots = (+inf | -inf, -1)
 *     (faiss-metal/src/MetalIndexFlat.mm:294-369, test/sql/faiss_basic.test:37-63,105-110).
 *   - IVFFlat: assign to the nearest centroid under the index metric, ids are
 *     the global add order, search probes the nprobe nearest centroids and
 *     returns the exact top-k of their union
 *     (faiss-metal/src/MetalIndexIVFFlat.mm:102-120, 122-256).
 *   - SQ8: per-dimension min / (max-min) scale, code = round(clamp(norm*255)),
 *     dequantise (code/255)*scale+min (rust_lib/src/provider.rs:161-210, 138-147).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* metric codes of the batch-distance ABI: 0 = L2, anything else = IP
 * (src/metal_diskann_bridge.mm:167). */
/* metric codes of the FAISS-shaped API: 0 = inner product, 1 = L2. */
enum { ORACLE_METRIC_IP = 0, ORACLE_METRIC_L2 = 1 };

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Lets the caller use every host core even when the environment said otherwise
 * (torchrun exports OMP_NUM_THREADS=1 to its children). */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* Batch distance: the scalar loop of ComputeDistancesCPU, same operation     */
/* order, float accumulator (src/ann_search.cpp:702-720).                     */
/* ------------------------------------------------------------------------- */
static float batch_one_f32(const float *q, const float *c, int64_t dim, int metric) {
    float sum = 0.0f;
    if (metric == 0) {
        for (int64_t j = 0; j < dim; j++) {
            float diff = q[j] - c[j];
            sum += diff * diff;
        }
    } else {
        for (int64_t j = 0; j < dim; j++) {
            sum += q[j] * c[j];
        }
        sum = -sum;
    }
    return sum;
}

static double batch_one_f64(const float *q, const float *c, int64_t dim, int metric) {
    double sum = 0.0;
    if (metric == 0) {
        for (int64_t j = 0; j < dim; j++) {
            double diff = (double)q[j] - (double)c[j];
            sum += diff * diff;
        }
    } else {
        for (int64_t j = 0; j < dim; j++) {
            sum += (double)q[j] * (double)c[j];
        }
        sum = -sum;
    }
    return sum;
}

/* exact == 0: float accumulation in the reference's order; exact != 0: double. */
ORACLE_API int oracle_batch_distances(const float *query, const float *candidates, int64_t n, int64_t dim,
                                      int metric, int exact, float *out) {
    if (!query || !candidates || !out || n <= 0 || dim <= 0) return -1; /* bridge.mm:157-159 */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const float *c = candidates + i * dim;
        out[i] = exact ? (float)batch_one_f64(query, c, dim, metric) : batch_one_f32(query, c, dim, metric);
    }
    return 0;
}

/* query_map[i] picks the query of candidate i
 * (faiss-metal/shaders/diskann_distance.metal:64-105, src/metal_diskann_bridge.mm:255-323). */
ORACLE_API int oracle_multi_batch_distances(const float *queries, const float *candidates,
                                            const uint32_t *query_map, int64_t total_n, int64_t nq, int64_t dim,
                                            int metric, int exact, float *out) {
    if (!queries || !candidates || !query_map || !out || total_n <= 0 || nq <= 0 || dim <= 0) return -1;
    for (int64_t i = 0; i < total_n; i++)
        if ((int64_t)query_map[i] >= nq) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total_n; i++) {
        const float *q = queries + (int64_t)query_map[i] * dim;
        const float *c = candidates + i * dim;
        out[i] = exact ? (float)batch_one_f64(q, c, dim, metric) : batch_one_f32(q, c, dim, metric);
    }
    return 0;
}

/* Same arithmetic with the candidate rows named by id into a resident table
 * (the gather DiskProvider does at rust_lib/src/disk_provider.rs:420-424,592-600
 * folded into the distance call). */
ORACLE_API int oracle_batch_distances_by_id(const float *table, int64_t num, int64_t dim, const float *queries,
                                            int64_t nq, const uint32_t *ids, const uint32_t *query_map,
                                            int64_t total_n, int metric, int exact, float *out) {
    if (!table || !queries || !ids || !out || total_n <= 0 || nq <= 0 || dim <= 0) return -1;
    for (int64_t i = 0; i < total_n; i++) {
        if ((int64_t)ids[i] >= num) return -1;
        if (query_map && (int64_t)query_map[i] >= nq) return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total_n; i++) {
        const float *q = queries + (query_map ? (int64_t)query_map[i] : 0) * dim;
        const float *c = table + (int64_t)ids[i] * dim;
        out[i] = exact ? (float)batch_one_f64(q, c, dim, metric) : batch_one_f32(q, c, dim, metric);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* SQ8 (rust_lib/src/provider.rs:161-210 quantise, :138-147 dequantise).      */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_sq8_train(const float *x, int64_t n, int64_t dim, float *mins, float *scale) {
    if (!x || n <= 0 || dim <= 0) return -1;
    for (int64_t d = 0; d < dim; d++) {
        mins[d] = 3.402823466e+38f;   /* f32::MAX */
        scale[d] = -3.402823466e+38f; /* holds max for now (f32::MIN) */
    }
    for (int64_t i = 0; i < n; i++) {
        const float *row = x + i * dim;
        for (int64_t d = 0; d < dim; d++) {
            float v = row[d];
            if (v < mins[d]) mins[d] = v;
            if (v > scale[d]) scale[d] = v;
        }
    }
    for (int64_t d = 0; d < dim; d++) {
        float range = scale[d] - mins[d];
        scale[d] = range > 0.0f ? range : 1.0f;
    }
    return 0;
}

ORACLE_API int oracle_sq8_encode(const float *x, int64_t n, int64_t dim, const float *mins, const float *scale,
                                 uint8_t *codes) {
    if (!x || !codes || n <= 0 || dim <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        for (int64_t d = 0; d < dim; d++) {
            float normalized = (x[i * dim + d] - mins[d]) / scale[d];
            float r = roundf(normalized * 255.0f); /* Rust f32::round: half away from zero */
            if (r < 0.0f) r = 0.0f;
            if (r > 255.0f) r = 255.0f;
            codes[i * dim + d] = (uint8_t)r;
        }
    }
    return 0;
}

ORACLE_API int oracle_sq8_decode(const uint8_t *codes, int64_t n, int64_t dim, const float *mins,
                                 const float *scale, float *x) {
    if (!x || !codes || n <= 0 || dim <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++)
        for (int64_t d = 0; d < dim; d++)
            x[i * dim + d] = ((float)codes[i * dim + d] / 255.0f) * scale[d] + mins[d];
    return 0;
}

/* Asymmetric distance: fp32 query against the dequantised row, distance as in
 * compute_distance (rust_lib/src/distance.rs:15-25) on the dequantised vector. */
ORACLE_API int oracle_sq8_batch_distances_by_id(const uint8_t *codes, int64_t num, int64_t dim, const float *mins,
                                                const float *scale, const float *queries, int64_t nq,
                                                const uint32_t *ids, const uint32_t *query_map, int64_t total_n,
                                                int metric, int exact, float *out) {
    if (!codes || !queries || !ids || !out || total_n <= 0 || nq <= 0 || dim <= 0) return -1;
    for (int64_t i = 0; i < total_n; i++) {
        if ((int64_t)ids[i] >= num) return -1;
        if (query_map && (int64_t)query_map[i] >= nq) return -1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total_n; i++) {
        const float *q = queries + (query_map ? (int64_t)query_map[i] : 0) * dim;
        const uint8_t *c = codes + (int64_t)ids[i] * dim;
        if (exact) {
            double sum = 0.0;
            for (int64_t d = 0; d < dim; d++) {
                float xh = ((float)c[d] / 255.0f) * scale[d] + mins[d];
                if (metric == 0) {
                    double diff = (double)q[d] - (double)xh;
                    sum += diff * diff;
                } else {
                    sum += (double)q[d] * (double)xh;
                }
            }
            out[i] = (float)(metric == 0 ? sum : -sum);
        } else {
            float sum = 0.0f;
            for (int64_t d = 0; d < dim; d++) {
                float xh = ((float)c[d] / 255.0f) * scale[d] + mins[d];
                if (metric == 0) {
                    float diff = q[d] - xh;
                    sum += diff * diff;
                } else {
                    sum += q[d] * xh;
                }
            }
            out[i] = metric == 0 ? sum : -sum;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* k-selection: a bounded heap on (key, id); smaller key is better; ties go   */
/* to the smaller id so the oracle's order is deterministic.                  */
/* ------------------------------------------------------------------------- */
typedef struct {
    double key;
    int64_t id;
} hitem;

static int worse(const hitem *a, const hitem *b) { /* a is worse than b */
    return a->key > b->key || (a->key == b->key && a->id > b->id);
}

static void heap_push(hitem *h, int64_t *n, int64_t k, double key, int64_t id) {
    hitem it = {key, id};
    if (*n < k) {
        int64_t i = (*n)++;
        h[i] = it;
        while (i > 0) {
            int64_t p = (i - 1) / 2;
            if (worse(&h[i], &h[p])) {
                hitem t = h[i]; h[i] = h[p]; h[p] = t; i = p;
            } else break;
        }
    } else if (worse(&h[0], &it)) {
        h[0] = it;
        int64_t i = 0;
        for (;;) {
            int64_t l = 2 * i + 1, r = l + 1, m = i;
            if (l < k && worse(&h[l], &h[m])) m = l;
            if (r < k && worse(&h[r], &h[m])) m = r;
            if (m == i) break;
            hitem t = h[i]; h[i] = h[m]; h[m] = t; i = m;
        }
    }
}

static int cmp_hitem(const void *a, const void *b) {
    const hitem *x = (const hitem *)a, *y = (const hitem *)b;
    if (worse(x, y)) return 1;
    if (worse(y, x)) return -1;
    return 0;
}

/* Writes k slots best first; unfilled slots get (sentinel, -1)
 * (faiss-metal/src/MetalIndexFlat.mm:352-368). */
static void heap_emit(hitem *h, int64_t n, int64_t k, int metric, float *D, int64_t *I) {
    qsort(h, (size_t)n, sizeof(hitem), cmp_hitem);
    float sentinel = metric == ORACLE_METRIC_L2 ? INFINITY : -INFINITY;
    for (int64_t j = 0; j < k; j++) {
        if (j < n) {
            D[j] = (float)(metric == ORACLE_METRIC_L2 ? h[j].key : -h[j].key);
            I[j] = h[j].id;
        } else {
            D[j] = sentinel;
            I[j] = -1;
        }
    }
}

/* key: smaller is better.  L2 -> squared distance; IP -> negated dot. */
static double pair_key(const float *q, const float *x, int64_t d, int metric) {
    double s = 0.0;
    if (metric == ORACLE_METRIC_L2) {
        for (int64_t j = 0; j < d; j++) {
            double t = (double)q[j] - (double)x[j];
            s += t * t;
        }
        return s;
    }
    for (int64_t j = 0; j < d; j++) s += (double)q[j] * (double)x[j];
    return -s;
}

/* ------------------------------------------------------------------------- */
/* Flat exact search (faiss::IndexFlat semantics as the reference uses them:  */
/* faiss-metal/src/MetalIndexFlat.mm:294-369).  Distances in double.          */
/* ------------------------------------------------------------------------- */
ORACLE_API int oracle_flat_search(const float *xb, int64_t n, int64_t d, const float *xq, int64_t nq, int64_t k,
                                  int metric, float *D, int64_t *I) {
    if (k <= 0 || d <= 0 || nq < 0 || n < 0) return -1;
    int64_t kk = k < n ? k : n;
#pragma omp parallel
    {
        hitem *h = (hitem *)malloc(sizeof(hitem) * (size_t)(kk > 0 ? kk : 1));
#pragma omp for schedule(dynamic, 1)
        for (int64_t qi = 0; qi < nq; qi++) {
            int64_t cnt = 0;
            const float *q = xq + qi * d;
            if (kk > 0)
                for (int64_t i = 0; i < n; i++) heap_push(h, &cnt, kk, pair_key(q, xb + i * d, d, metric), i);
            heap_emit(h, cnt, k, metric, D + qi * k, I + qi * k);
        }
        free(h);
    }
    return 0;
}

/* All pair keys of a query against the whole database, in double, written as
 * user-facing distances (squared L2 or raw dot).  Used by the tests to judge
 * tolerance ties at the k-th / (k+1)-th boundary. */
ORACLE_API int oracle_all_distances(const float *xb, int64_t n, int64_t d, const float *q, int metric, double *out) {
    if (!xb || !q || !out || n < 0 || d <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        double key = pair_key(q, xb + i * d, d, metric);
        out[i] = metric == ORACLE_METRIC_L2 ? key : -key;
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* IVFFlat                                                                    */
/* ------------------------------------------------------------------------- */
/* Nearest centroid under the index metric
 * (faiss-metal/src/MetalIndexIVFFlat.mm:55-66,102-120). */
ORACLE_API int oracle_ivf_assign(const float *x, int64_t n, int64_t d, const float *centroids, int64_t nlist,
                                 int metric, int64_t *assign) {
    if (!x || !centroids || !assign || n < 0 || d <= 0 || nlist <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        double best = INFINITY;
        int64_t bi = 0;
        for (int64_t c = 0; c < nlist; c++) {
            double key = pair_key(x + i * d, centroids + c * d, d, metric);
            if (key < best) { best = key; bi = c; }
        }
        assign[i] = bi;
    }
    return 0;
}

/* Seeded Lloyd k-means.  K-means is outside the search hot path; the oracle
 * only needs SOME centroids, which are then handed unchanged to both the
 * oracle search and the GPU index (the reference trains once with FAISS and
 * copies the centroids to the GPU index, faiss-metal/src/MetalIndexIVFFlat.mm:291-296). */
static uint64_t splitmix(uint64_t *s) {
    uint64_t z = (*s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

ORACLE_API int oracle_kmeans(const float *x, int64_t n, int64_t d, int64_t nlist, int niter, uint64_t seed,
                             float *centroids) {
    if (!x || !centroids || n < nlist || nlist <= 0 || d <= 0) return -1;
    /* initial centroids: a seeded sample of distinct rows (partial Fisher-Yates) */
    int64_t *perm = (int64_t *)malloc(sizeof(int64_t) * (size_t)n);
    for (int64_t i = 0; i < n; i++) perm[i] = i;
    uint64_t s = seed;
    for (int64_t i = 0; i < nlist; i++) {
        int64_t j = i + (int64_t)(splitmix(&s) % (uint64_t)(n - i));
        int64_t t = perm[i]; perm[i] = perm[j]; perm[j] = t;
        memcpy(centroids + i * d, x + perm[i] * d, sizeof(float) * (size_t)d);
    }
    free(perm);
    int64_t *assign = (int64_t *)malloc(sizeof(int64_t) * (size_t)n);
    double *sums = (double *)malloc(sizeof(double) * (size_t)(nlist * d));
    int64_t *cnt = (int64_t *)malloc(sizeof(int64_t) * (size_t)nlist);
    for (int it = 0; it < niter; it++) {
        oracle_ivf_assign(x, n, d, centroids, nlist, ORACLE_METRIC_L2, assign);
        memset(sums, 0, sizeof(double) * (size_t)(nlist * d));
        memset(cnt, 0, sizeof(int64_t) * (size_t)nlist);
        for (int64_t i = 0; i < n; i++) {
            int64_t c = assign[i];
            cnt[c]++;
            for (int64_t j = 0; j < d; j++) sums[c * d + j] += x[i * d + j];
        }
        for (int64_t c = 0; c < nlist; c++) {
            if (cnt[c] == 0) continue; /* keep an empty cluster's centroid where it was */
            for (int64_t j = 0; j < d; j++) centroids[c * d + j] = (float)(sums[c * d + j] / (double)cnt[c]);
        }
    }
    free(assign); free(sums); free(cnt);
    return 0;
}

/* IVFFlat search over lists given in CSR form: rows of list c are
 * list_rows[list_off[c] .. list_off[c+1]) (indices into xb, which are also the
 * labels: global add order, MetalIndexIVFFlat.mm:112).  probes_out (nq x nprobe,
 * may be NULL) receives the probed list numbers, nearest first, -1 padded. */
ORACLE_API int oracle_ivf_search(const float *xb, int64_t n, int64_t d, const float *centroids, int64_t nlist,
                                 const int64_t *list_off, const int64_t *list_rows, const float *xq, int64_t nq,
                                 int64_t k, int64_t nprobe, int metric, float *D, int64_t *I, int64_t *probes_out) {
    (void)n;
    if (k <= 0 || d <= 0 || nlist <= 0 || nprobe <= 0) return -1;
    if (nprobe > nlist) nprobe = nlist;
#pragma omp parallel
    {
        hitem *h = (hitem *)malloc(sizeof(hitem) * (size_t)k);
        hitem *ph = (hitem *)malloc(sizeof(hitem) * (size_t)nprobe);
#pragma omp for schedule(dynamic, 1)
        for (int64_t qi = 0; qi < nq; qi++) {
            const float *q = xq + qi * d;
            int64_t pc = 0;
            for (int64_t c = 0; c < nlist; c++) heap_push(ph, &pc, nprobe, pair_key(q, centroids + c * d, d, metric), c);
            qsort(ph, (size_t)pc, sizeof(hitem), cmp_hitem);
            int64_t cnt = 0;
            for (int64_t p = 0; p < pc; p++) {
                int64_t c = ph[p].id;
                if (probes_out) probes_out[qi * nprobe + p] = c;
                for (int64_t r = list_off[c]; r < list_off[c + 1]; r++) {
                    int64_t row = list_rows[r];
                    heap_push(h, &cnt, k, pair_key(q, xb + row * d, d, metric), row);
                }
            }
            if (probes_out)
                for (int64_t p = pc; p < nprobe; p++) probes_out[qi * nprobe + p] = -1;
            heap_emit(h, cnt, k, metric, D + qi * k, I + qi * k);
        }
        free(h); free(ph);
    }
    return 0;
}

/* IVFFlat search with the probe lists GIVEN (nq x nprobe, -1 = skip).  Lets a
 * test hold the coarse step fixed when the nprobe-th and (nprobe+1)-th centroid
 * distances of a query lie within tolerance of each other. */
ORACLE_API int oracle_ivf_search_given_probes(const float *xb, int64_t d, const int64_t *list_off,
                                              const int64_t *list_rows, const float *xq, int64_t nq, int64_t k,
                                              int64_t nprobe, const int64_t *probes, int metric, float *D,
                                              int64_t *I) {
    if (k <= 0 || d <= 0 || nprobe <= 0) return -1;
#pragma omp parallel
    {
        hitem *h = (hitem *)malloc(sizeof(hitem) * (size_t)k);
#pragma omp for schedule(dynamic, 1)
        for (int64_t qi = 0; qi < nq; qi++) {
            const float *q = xq + qi * d;
            int64_t cnt = 0;
            for (int64_t p = 0; p < nprobe; p++) {
                int64_t c = probes[qi * nprobe + p];
                if (c < 0) continue;
                for (int64_t r = list_off[c]; r < list_off[c + 1]; r++) {
                    int64_t row = list_rows[r];
                    heap_push(h, &cnt, k, pair_key(q, xb + row * d, d, metric), row);
                }
            }
            heap_emit(h, cnt, k, metric, D + qi * k, I + qi * k);
        }
        free(h);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Fast fp32 paths: what a CPU build of the reference executes per query      */
/* (FAISS CPU scans with SIMD fp32 and a heap; OpenMP over queries).  Used    */
/* only as the timed CPU baseline.                                            */
/* ------------------------------------------------------------------------- */
static inline float key_f32(const float *q, const float *x, int64_t d, int metric) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int64_t j = 0;
    if (metric == ORACLE_METRIC_L2) {
        for (; j + 4 <= d; j += 4) {
            float a = q[j] - x[j], b = q[j + 1] - x[j + 1], c = q[j + 2] - x[j + 2], e = q[j + 3] - x[j + 3];
            s0 += a * a; s1 += b * b; s2 += c * c; s3 += e * e;
        }
        for (; j < d; j++) { float a = q[j] - x[j]; s0 += a * a; }
        return (s0 + s1) + (s2 + s3);
    }
    for (; j + 4 <= d; j += 4) {
        s0 += q[j] * x[j]; s1 += q[j + 1] * x[j + 1]; s2 += q[j + 2] * x[j + 2]; s3 += q[j + 3] * x[j + 3];
    }
    for (; j < d; j++) s0 += q[j] * x[j];
    return -((s0 + s1) + (s2 + s3));
}

ORACLE_API int oracle_ivf_search_fast(const float *xb, int64_t d, const float *centroids, int64_t nlist,
                                      const int64_t *list_off, const int64_t *list_rows, const float *xq,
                                      int64_t nq, int64_t k, int64_t nprobe, int metric, float *D, int64_t *I) {
    if (k <= 0 || d <= 0 || nlist <= 0 || nprobe <= 0) return -1;
    if (nprobe > nlist) nprobe = nlist;
#pragma omp parallel
    {
        hitem *h = (hitem *)malloc(sizeof(hitem) * (size_t)k);
        hitem *ph = (hitem *)malloc(sizeof(hitem) * (size_t)nprobe);
#pragma omp for schedule(dynamic, 1)
        for (int64_t qi = 0; qi < nq; qi++) {
            const float *q = xq + qi * d;
            int64_t pc = 0;
            for (int64_t c = 0; c < nlist; c++)
                heap_push(ph, &pc, nprobe, (double)key_f32(q, centroids + c * d, d, metric), c);
            int64_t cnt = 0;
            for (int64_t p = 0; p < pc; p++) {
                int64_t c = ph[p].id;
                for (int64_t r = list_off[c]; r < list_off[c + 1]; r++) {
                    int64_t row = list_rows[r];
                    heap_push(h, &cnt, k, (double)key_f32(q, xb + row * d, d, metric), row);
                }
            }
            heap_emit(h, cnt, k, metric, D + qi * k, I + qi * k);
        }
        free(h); free(ph);
    }
    return 0;
}

/* Select the k best of a precomputed (nq x n) fp32 key block, merging into
 * running (nq x k) results.  With a BLAS product feeding it this is the
 * blocked sgemm + heap form of a CPU flat search; ids are offset by id0. */
ORACLE_API int oracle_select_block(const float *keys, int64_t nq, int64_t n, int64_t id0, int64_t k, float *runD,
                                   int64_t *runI) {
    if (!keys || !runD || !runI || k <= 0) return -1;
#pragma omp parallel
    {
        hitem *h = (hitem *)malloc(sizeof(hitem) * (size_t)k);
#pragma omp for schedule(static)
        for (int64_t qi = 0; qi < nq; qi++) {
            int64_t cnt = 0;
            for (int64_t j = 0; j < k; j++)
                if (runI[qi * k + j] >= 0) heap_push(h, &cnt, k, (double)runD[qi * k + j], runI[qi * k + j]);
            const float *row = keys + qi * n;
            double thr = cnt == k ? h[0].key : INFINITY;
            for (int64_t i = 0; i < n; i++) {
                if ((double)row[i] < thr || cnt < k) {
                    heap_push(h, &cnt, k, (double)row[i], id0 + i);
                    if (cnt == k) thr = h[0].key;
                }
            }
            qsort(h, (size_t)cnt, sizeof(hitem), cmp_hitem);
            for (int64_t j = 0; j < k; j++) {
                if (j < cnt) { runD[qi * k + j] = (float)h[j].key; runI[qi * k + j] = h[j].id; }
                else { runD[qi * k + j] = INFINITY; runI[qi * k + j] = -1; }
            }
        }
        free(h);
    }
    return 0;
}
