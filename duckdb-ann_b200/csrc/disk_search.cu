// Lock-step batched graph search over a ".diskann" index image whose vectors live in GPU memory.
//
// This is the caller side of the batch-distance path: the search loop of
// DiskProvider::search_batch (rust_lib/src/disk_provider.rs:470-652; the in-memory provider has
// the same loop, rust_lib/src/provider.rs:333-427), restated in C++ because the image has no Rust
// toolchain.  Every iteration each active query pops its best unexpanded candidate, the
// not-yet-visited neighbours of all those candidates are concatenated, and ONE batch-distance call
// scores them.  The reference gathers the neighbour ROWS on the host and hands them to
// diskann_metal_multi_batch_distances (:592-610); here the table was loaded into HBM once
// (diskann_cuda_load_index) and the call takes the neighbour IDS
// (diskann_cuda_batch_distances_by_id_device), so nothing but ids and distances crosses PCIe.
// The graph itself (adjacency, entry points) stays on the host, as in the reference.
//
// Differences from the reference loop, on purpose: every distance comes from the GPU (the
// reference scores batches below MIN_GPU_WORK and the entry points with its CPU distance
// functions; this library has no CPU distance path), and a single query takes the same loop.
#include <algorithm>
#include <queue>
#include <unordered_set>

#include "common.cuh"
#include "cuda_diskann_bridge.h"

using anncuda::DeviceGuard;

namespace {

thread_local std::string t_search_error;
int fail(const char *what) {
    t_search_error = what;
    const char *inner = diskann_cuda_last_error();
    if (inner && *inner) t_search_error += std::string(": ") + inner;
    return -1;
}

struct Pinned {
    void *ptr = nullptr;
    size_t cap = 0;
    int ensure(size_t bytes) {
        if (bytes <= cap) return 0;
        if (ptr) cudaFreeHost(ptr);
        ptr = nullptr;
        cap = 0;
        size_t want = 4096;
        while (want < bytes) want <<= 1;
        if (cudaMallocHost(&ptr, want) != cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
        cap = want;
        return 0;
    }
    void release() {
        if (ptr) cudaFreeHost(ptr);
        ptr = nullptr;
        cap = 0;
    }
};

}  // namespace

struct diskann_cuda_searcher {
    int device = 0;
    diskann_cuda_index_info info{};
    diskann_cuda_table *vectors = nullptr, *sq8 = nullptr;
    bool use_sq8 = false;
    std::vector<uint32_t> entry_points, adjacency;  // host copies of the graph
    cudaStream_t stream = nullptr;
    anncuda::GrowBuf d_queries, d_ids, d_map, d_out;
    Pinned h_ids, h_map, h_out;
    std::mutex mu;  // one batch search at a time per searcher (the buffers above are shared)
    // what the last search did
    uint64_t iterations = 0, pairs_scored = 0, distance_calls = 0;
    // optional trace of the id batches of the last search (for workload generation)
    bool trace = false;
    std::vector<uint32_t> trace_ids, trace_map;
    std::vector<uint64_t> trace_offsets;
};

extern "C" {

const char *diskann_cuda_searcher_last_error(void) { return t_search_error.c_str(); }

int diskann_cuda_searcher_open(int device, const void *image, size_t len, int use_sq8, diskann_cuda_searcher **out) {
    if (!out) return fail("null output handle");
    *out = nullptr;
    if (!image) return fail("null image");
    auto *s = new diskann_cuda_searcher();
    s->device = device;
    if (diskann_cuda_load_index(device, image, len, &s->info, &s->vectors, &s->sq8)) {
        delete s;
        return fail("loading the index image failed");
    }
    s->use_sq8 = use_sq8 != 0;
    if (s->use_sq8 && !s->sq8) {
        diskann_cuda_unregister(s->vectors);
        delete s;
        return fail("the image carries no SQ8 trailer");
    }
    const auto *bytes = static_cast<const unsigned char *>(image);
    const auto *ep = reinterpret_cast<const uint32_t *>(bytes + s->info.entry_points_offset);
    s->entry_points.assign(ep, ep + s->info.num_entry_points);
    const auto *adj = reinterpret_cast<const uint32_t *>(bytes + s->info.adjacency_offset);
    s->adjacency.assign(adj, adj + (size_t)s->info.num_vectors * s->info.max_degree);
    DeviceGuard g(device);
    if (!g.ok || cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        diskann_cuda_unregister(s->vectors);
        if (s->sq8) diskann_cuda_unregister(s->sq8);
        delete s;
        return fail("could not create the search stream");
    }
    *out = s;
    return 0;
}

void diskann_cuda_searcher_close(diskann_cuda_searcher *s) {
    if (!s) return;
    DeviceGuard g(s->device);
    if (s->stream) cudaStreamSynchronize(s->stream);
    for (anncuda::GrowBuf *b : {&s->d_queries, &s->d_ids, &s->d_map, &s->d_out}) b->release();
    for (Pinned *p : {&s->h_ids, &s->h_map, &s->h_out}) p->release();
    if (s->stream) cudaStreamDestroy(s->stream);
    if (s->vectors) diskann_cuda_unregister(s->vectors);
    if (s->sq8) diskann_cuda_unregister(s->sq8);
    delete s;
}

int diskann_cuda_searcher_info(const diskann_cuda_searcher *s, diskann_cuda_index_info *info) {
    if (!s || !info) return fail("invalid arguments");
    *info = s->info;
    return 0;
}

void diskann_cuda_searcher_set_trace(diskann_cuda_searcher *s, int on) {
    if (s) s->trace = on != 0;
}

int diskann_cuda_searcher_stats(const diskann_cuda_searcher *s, uint64_t *iterations, uint64_t *pairs_scored,
                                uint64_t *distance_calls) {
    if (!s) return fail("null searcher");
    if (iterations) *iterations = s->iterations;
    if (pairs_scored) *pairs_scored = s->pairs_scored;
    if (distance_calls) *distance_calls = s->distance_calls;
    return 0;
}

int64_t diskann_cuda_searcher_trace(const diskann_cuda_searcher *s, uint32_t *ids, uint32_t *query_map, uint64_t *offsets,
                                    int64_t max_pairs, int64_t max_batches) {
    if (!s) return fail("null searcher");
    const int64_t nb = (int64_t)s->trace_offsets.size() - 1;
    if (nb < 0) return 0;
    if (ids && query_map && offsets) {
        if ((int64_t)s->trace_ids.size() > max_pairs || nb > max_batches) return fail("trace buffers too small");
        std::copy(s->trace_ids.begin(), s->trace_ids.end(), ids);
        std::copy(s->trace_map.begin(), s->trace_map.end(), query_map);
        std::copy(s->trace_offsets.begin(), s->trace_offsets.end(), offsets);
    }
    return nb;
}

int diskann_cuda_searcher_search_batch(diskann_cuda_searcher *s, const float *queries, int nq, int k, int l_search,
                                       uint64_t *out_ids, float *out_distances, int *out_counts) {
    if (!s || nq < 0 || (nq > 0 && (!queries || !out_ids || !out_distances || !out_counts))) return fail("invalid arguments");
    std::lock_guard<std::mutex> lock(s->mu);
    s->iterations = s->pairs_scored = s->distance_calls = 0;
    s->trace_ids.clear();
    s->trace_map.clear();
    s->trace_offsets.assign(1, 0);
    const uint32_t num = s->info.num_vectors;
    for (int q = 0; q < nq; q++) out_counts[q] = 0;
    if (nq == 0 || num == 0 || k <= 0) return 0;  // disk_provider.rs:477-479
    const int dim = (int)s->info.dimension, degree = (int)s->info.max_degree;
    const int k_stride = k;  // the output arrays are nq x k as the caller passed k
    k = (int)std::min<uint32_t>((uint32_t)k, num);
    const size_t l = (size_t)std::max(l_search, k);  // :485-486
    const int metric = (int)s->info.metric;         // bridge code: 0 = L2, else IP (negated dot)
    const diskann_cuda_table *table = s->use_sq8 ? s->sq8 : s->vectors;

    DeviceGuard guard(s->device);
    if (!guard.ok) return fail("cudaSetDevice failed");
    const size_t max_pairs = (size_t)nq * std::max<size_t>((size_t)degree, s->entry_points.size());
    if (s->d_queries.ensure((size_t)nq * dim * 4) || s->d_ids.ensure(max_pairs * 4) || s->d_map.ensure(max_pairs * 4) ||
        s->d_out.ensure(max_pairs * 4) || s->h_ids.ensure(max_pairs * 4) || s->h_map.ensure(max_pairs * 4) ||
        s->h_out.ensure(max_pairs * 4))
        return fail("out of memory for the search buffers");
    if (cudaMemcpyAsync(s->d_queries.ptr, queries, (size_t)nq * dim * 4, cudaMemcpyHostToDevice, s->stream) != cudaSuccess)
        return fail("query upload failed");
    auto *h_ids = static_cast<uint32_t *>(s->h_ids.ptr), *h_map = static_cast<uint32_t *>(s->h_map.ptr);
    auto *h_out = static_cast<float *>(s->h_out.ptr);

    // ids and map in, distances out: one batch-distance launch on the table in HBM
    auto score = [&](size_t total) -> int {
        if (cudaMemcpyAsync(s->d_ids.ptr, h_ids, total * 4, cudaMemcpyHostToDevice, s->stream) != cudaSuccess ||
            cudaMemcpyAsync(s->d_map.ptr, h_map, total * 4, cudaMemcpyHostToDevice, s->stream) != cudaSuccess)
            return fail("id upload failed");
        if (diskann_cuda_batch_distances_by_id_device(table, s->d_queries.as<float>(), nq, s->d_ids.as<uint32_t>(),
                                                      s->d_map.as<uint32_t>(), (int)total, metric, s->d_out.as<float>(),
                                                      s->stream))
            return fail("batch distance call failed");
        if (cudaMemcpyAsync(h_out, s->d_out.ptr, total * 4, cudaMemcpyDeviceToHost, s->stream) != cudaSuccess ||
            cudaStreamSynchronize(s->stream) != cudaSuccess)
            return fail("reading the distances back failed");
        s->distance_calls++;
        s->pairs_scored += total;
        if (s->trace) {
            s->trace_ids.insert(s->trace_ids.end(), h_ids, h_ids + total);
            s->trace_map.insert(s->trace_map.end(), h_map, h_map + total);
            s->trace_offsets.push_back(s->trace_ids.size());
        }
        return 0;
    };

    // per-query state (:495-510): visited set, min-heap of candidates, sorted result list of at most l
    struct Cand {
        float dist;
        uint32_t id;
        bool operator>(const Cand &o) const { return dist > o.dist || (dist == o.dist && id > o.id); }
    };
    struct QState {
        std::unordered_set<uint32_t> visited;
        std::priority_queue<Cand, std::vector<Cand>, std::greater<Cand>> candidates;
        std::vector<Cand> result;
        bool active = true;
    };
    std::vector<QState> states((size_t)nq);
    // insert_result (:655-678)
    auto insert_result = [&](QState &st, float dist, uint32_t id) {
        if (st.result.size() < l || dist < st.result.back().dist) {
            auto pos = std::lower_bound(st.result.begin(), st.result.end(), dist,
                                        [](const Cand &c, float d) { return c.dist < d; });
            st.result.insert(pos, Cand{dist, id});
            if (st.result.size() > l) st.result.resize(l);
            st.candidates.push(Cand{dist, id});
        }
    };

    // seed: the entry points of every query (:512-527), scored in one call
    size_t total = 0;
    for (int q = 0; q < nq; q++)
        for (uint32_t ep : s->entry_points)
            if (ep < num && states[(size_t)q].visited.insert(ep).second) {
                h_ids[total] = ep;
                h_map[total++] = (uint32_t)q;
            }
    if (total && score(total)) return -1;
    for (size_t i = 0; i < total; i++) {
        QState &st = states[h_map[i]];
        st.candidates.push(Cand{h_out[i], h_ids[i]});
        st.result.push_back(Cand{h_out[i], h_ids[i]});
    }
    for (QState &st : states)
        std::stable_sort(st.result.begin(), st.result.end(), [](const Cand &a, const Cand &b) { return a.dist < b.dist; });

    for (;;) {
        bool any_active = false;
        total = 0;
        // phase 1 (:546-581): pop the best candidate of every active query, collect its unvisited neighbours
        for (int q = 0; q < nq; q++) {
            QState &st = states[(size_t)q];
            if (!st.active) continue;
            if (st.candidates.empty()) {
                st.active = false;
                continue;
            }
            const Cand c = st.candidates.top();
            st.candidates.pop();
            if (st.result.size() >= l && c.dist > st.result[l - 1].dist) {
                st.active = false;
                continue;
            }
            any_active = true;
            const uint32_t *nb = s->adjacency.data() + (size_t)c.id * degree;
            for (int j = 0; j < degree; j++) {
                const uint32_t v = nb[j];
                if (v >= num) continue;  // unused slot
                if (!st.visited.insert(v).second) continue;
                h_ids[total] = v;
                h_map[total++] = (uint32_t)q;
            }
        }
        if (!any_active) break;
        s->iterations++;
        if (total == 0) continue;
        // phase 2 (:590-610): one distance call for the neighbours of all queries
        if (score(total)) return -1;
        for (size_t i = 0; i < total; i++) insert_result(states[h_map[i]], h_out[i], h_ids[i]);
    }

    for (int q = 0; q < nq; q++) {
        const QState &st = states[(size_t)q];
        const int cnt = (int)std::min<size_t>((size_t)k, st.result.size());
        out_counts[q] = cnt;
        for (int j = 0; j < cnt; j++) {
            out_ids[(size_t)q * k_stride + j] = st.result[(size_t)j].id;
            out_distances[(size_t)q * k_stride + j] = st.result[(size_t)j].dist;
        }
    }
    return 0;
}

}  // extern "C"
