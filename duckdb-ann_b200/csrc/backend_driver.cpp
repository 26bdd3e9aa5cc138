// Command-line driver for the C++ plugin surface: builds a CPU-side index holder,
// converts it with duckdb::GetGpuBackend().CpuToGpu(), searches the way
// FaissIndex::Search does (src/faiss_index.cpp:708-762: one query per call, labels
// -1 skipped) and as one batch, converts back with GpuToCpu() and checks that the
// rows survived bit for bit.  The GPU tests run it and compare its output file with
// the CPU oracle.
//
//   backend_driver info
//   backend_driver flat|ivf <in.bin> <out.bin>
//   backend_driver storage <in.bin> <out.bin> f16|bf16        CudaIndexFlat with reduced-precision rows
//       (faiss_metal::StorageType, MetalIndexFlat.h:38-60): same in.bin / out.bin as `flat`; the JSON line says
//       whether the storage flags read back, reconstruct returns the same row twice, and GpuToCpu hands out
//       exactly the rows reconstruct shows.
//   backend_driver glue <in.bin> <out.bin> [cpu|gpu|auto]     the FaissIndex glue of faiss_index_glue.hpp:
//       in.bin : int64 {d, n, nq, k, metric, n0, ntomb}, float xb[n*d], float xq[nq*d], int64 tomb[ntomb]
//       builds from the first n0 rows, searches (one query per call and as ONE batch), appends the rest,
//       marks `tomb` deleted, searches again.  out.bin: for both phases D_single, I_single, D_batch, I_batch
//       (nq*k each; slots a query could not fill hold label -1).
// in.bin : int64 {d, n, nq, k, metric, nlist, nprobe}, float xb[n*d], float xq[nq*d],
//          for ivf: float centroids[nlist*d], int64 assign[n]
// out.bin: float D_batch[nq*k], int64 I_batch[nq*k], float D_single[nq*k], int64 I_single[nq*k]
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>

#ifndef FAISS_AVAILABLE
#define FAISS_AVAILABLE
#endif
#include "faiss_index_glue.hpp"
#include "gpu_backend.hpp"
#include "gpu_backend_cuda.hpp"

template <class T>
static bool read_vec(FILE *f, std::vector<T> &v, size_t n) {
    v.resize(n);
    return n == 0 || fread(v.data(), sizeof(T), n, f) == n;
}

static void write_results(FILE *o, const std::vector<std::vector<std::pair<faiss::idx_t, float>>> &res, int64_t nq, int64_t k) {
    std::vector<float> D((size_t)(nq * k), 0.f);
    std::vector<int64_t> I((size_t)(nq * k), -1);
    for (int64_t q = 0; q < nq && q < (int64_t)res.size(); q++)
        for (size_t j = 0; j < res[(size_t)q].size(); j++) {
            I[(size_t)(q * k) + j] = res[(size_t)q][j].first;
            D[(size_t)(q * k) + j] = res[(size_t)q][j].second;
        }
    fwrite(D.data(), 4, D.size(), o);
    fwrite(I.data(), 8, I.size(), o);
}

// CudaIndexFlat(device, d, metric, StorageType): the index answers for the rows it keeps (rounded to fp16 / bf16).
static int run_storage(int argc, char **argv) {
    if (argc < 5) return 2;
    const bool bf16 = strcmp(argv[4], "bf16") == 0;
    FILE *f = fopen(argv[2], "rb");
    if (!f) return 2;
    int64_t h[7];
    if (fread(h, 8, 7, f) != 7) return 2;
    const int64_t d = h[0], n = h[1], nq = h[2], k = h[3];
    const faiss::MetricType metric = h[4] == 1 ? faiss::METRIC_L2 : faiss::METRIC_INNER_PRODUCT;
    std::vector<float> xb, xq;
    if (!read_vec(f, xb, (size_t)(n * d)) || !read_vec(f, xq, (size_t)(nq * d))) return 2;
    fclose(f);
    try {
        using faiss_cuda::StorageType;
        const StorageType st = bf16 ? StorageType::BFloat16 : StorageType::Float16;
        faiss_cuda::CudaIndexFlat gpu(0, (int)d, metric, st);
        gpu.add(n, xb.data());
        const int flags_ok = gpu.getStorageType() == st && gpu.isBFloat16Storage() == bf16 && gpu.isFloat16Storage() == !bf16 &&
                             gpu.ntotal == n;
        std::vector<float> D((size_t)(nq * k)), D1((size_t)(nq * k));
        std::vector<int64_t> I((size_t)(nq * k)), I1((size_t)(nq * k));
        gpu.search(nq, xq.data(), k, D.data(), I.data());
        for (int64_t q = 0; q < nq; q++) gpu.search(1, xq.data() + q * d, k, D1.data() + q * k, I1.data() + q * k);
        // GpuToCpu: a CPU IndexFlat over the rounded rows, the same values reconstruct returns
        std::unique_ptr<faiss::Index> back = duckdb::GetGpuBackend().GpuToCpu(&gpu);
        auto *bf = dynamic_cast<faiss::IndexFlat *>(back.get());
        int roundtrip_ok = bf && back->ntotal == n;
        std::vector<float> one((size_t)d), again((size_t)d);
        float worst = 0.f;
        for (int64_t r = 0; roundtrip_ok && r < n; r += (n > 64 ? n / 64 : 1)) {
            gpu.reconstruct(r, one.data());
            gpu.reconstruct(r, again.data());
            roundtrip_ok = memcmp(one.data(), again.data(), (size_t)d * 4) == 0 &&
                           memcmp(one.data(), bf->get_xb() + r * d, (size_t)d * 4) == 0;
            for (int64_t c = 0; c < d; c++) {
                const float e = one[(size_t)c] - xb[(size_t)(r * d + c)];
                worst = e > worst ? e : (-e > worst ? -e : worst);
            }
        }
        FILE *o = fopen(argv[3], "wb");
        if (!o) return 2;
        fwrite(D.data(), 4, D.size(), o);
        fwrite(I.data(), 8, I.size(), o);
        fwrite(D1.data(), 4, D1.size(), o);
        fwrite(I1.data(), 8, I1.size(), o);
        fclose(o);
        printf("{\"backend\": \"%s\", \"flags_ok\": %d, \"roundtrip_ok\": %d, \"worst_rounding\": %g}\n",
               duckdb::GetGpuBackend().BackendName().c_str(), flags_ok, roundtrip_ok, (double)worst);
        return 0;
    } catch (const std::exception &e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}

// FaissIndex::Search / SearchBatch over the GPU backend, with an append and deletions in between.
static int run_glue(int argc, char **argv) {
    using duckdb_glue::FaissGpuMode;
    FaissGpuMode mode = FaissGpuMode::AUTO;
    if (argc >= 5 && strcmp(argv[4], "gpu") == 0) mode = FaissGpuMode::GPU;
    if (argc >= 5 && strcmp(argv[4], "cpu") == 0) mode = FaissGpuMode::CPU;
    FILE *f = fopen(argv[2], "rb");
    if (!f) return 2;
    int64_t h[7];
    if (fread(h, 8, 7, f) != 7) return 2;
    const int64_t d = h[0], n = h[1], nq = h[2], k = h[3], n0 = h[5], ntomb = h[6];
    const faiss::MetricType metric = h[4] == 1 ? faiss::METRIC_L2 : faiss::METRIC_INNER_PRODUCT;
    std::vector<float> xb, xq;
    std::vector<int64_t> tomb;
    if (!read_vec(f, xb, (size_t)(n * d)) || !read_vec(f, xq, (size_t)(nq * d)) || !read_vec(f, tomb, (size_t)ntomb)) return 2;
    fclose(f);
    auto *flat = new faiss::IndexFlat(d, metric);
    flat->add(n0, xb.data());
    duckdb_glue::FaissIndexGlue index(std::unique_ptr<faiss::Index>(flat), mode);
    index.EnsureGpuIndex();  // Finalize (src/faiss_index.cpp:364)
    const int on_gpu_after_build = index.OnGpu();
    FILE *o = fopen(argv[3], "wb");
    if (!o) return 2;
    auto search_both = [&] {
        std::vector<std::vector<std::pair<faiss::idx_t, float>>> single;
        for (int64_t q = 0; q < nq; q++) single.push_back(index.Search(xq.data() + q * d, (int32_t)d, (int32_t)k));
        write_results(o, single, nq, k);
        write_results(o, index.SearchBatch(xq.data(), nq, (int32_t)d, (int32_t)k), nq, k);
    };
    search_both();
    index.Append(n - n0, xb.data() + n0 * d);  // drops the GPU copy (src/faiss_index.cpp:469)
    const int on_gpu_after_append = index.OnGpu();
    for (int64_t t : tomb) index.Delete(t);
    search_both();  // the first of these searches uploads the index again
    fclose(o);
    const int wrong_dim = index.Search(xq.data(), (int32_t)d + 1, (int32_t)k).empty();  // test/sql/faiss_basic.test:265-269
    printf("{\"on_gpu_after_build\": %d, \"on_gpu_after_append\": %d, \"on_gpu_at_end\": %d, \"gpu_uploads\": %d, "
           "\"wrong_dimension_is_empty\": %d}\n",
           on_gpu_after_build, on_gpu_after_append, (int)index.OnGpu(), index.GpuUploads(), wrong_dim);
    return 0;
}

int main(int argc, char **argv) {
    try {
        duckdb::GpuBackend &backend = duckdb::GetGpuBackend();
        if (argc >= 2 && strcmp(argv[1], "info") == 0) {
            printf("{\"available\": %s, \"backend\": \"%s\", \"device\": \"%s\"}\n", backend.IsAvailable() ? "true" : "false",
                   backend.BackendName().c_str(), backend.DeviceInfo().c_str());
            return 0;
        }
        if (argc < 4) {
            fprintf(stderr, "usage: %s info | flat|ivf in.bin out.bin | storage in.bin out.bin f16|bf16 | glue in.bin out.bin [cpu|gpu|auto]\n", argv[0]);
            return 2;
        }
        if (strcmp(argv[1], "glue") == 0) return run_glue(argc, argv);
        if (strcmp(argv[1], "storage") == 0) return run_storage(argc, argv);
        const bool ivf = strcmp(argv[1], "ivf") == 0;
        FILE *f = fopen(argv[2], "rb");
        if (!f) return 2;
        int64_t h[7];
        if (fread(h, 8, 7, f) != 7) return 2;
        const int64_t d = h[0], n = h[1], nq = h[2], k = h[3], nlist = h[5], nprobe = h[6];
        const faiss::MetricType metric = h[4] == 1 ? faiss::METRIC_L2 : faiss::METRIC_INNER_PRODUCT;
        std::vector<float> xb, xq, cent;
        std::vector<int64_t> assign;
        if (!read_vec(f, xb, (size_t)(n * d)) || !read_vec(f, xq, (size_t)(nq * d))) return 2;
        if (ivf && (!read_vec(f, cent, (size_t)(nlist * d)) || !read_vec(f, assign, (size_t)n))) return 2;
        fclose(f);

        std::unique_ptr<faiss::Index> cpu;
        if (!ivf) {
            auto *flat = new faiss::IndexFlat(d, metric);
            flat->add(n, xb.data());
            cpu.reset(flat);
        } else {
            auto *quantizer = new faiss::IndexFlat(d, metric);
            quantizer->add(nlist, cent.data());
            auto *idx = new faiss::IndexIVFFlat(quantizer, (size_t)d, (size_t)nlist, metric);
            idx->own_fields = true;
            idx->nprobe = (size_t)nprobe;
            for (int64_t i = 0; i < n; i++)
                idx->invlists->add_entries((size_t)assign[i], 1, &i, reinterpret_cast<const uint8_t *>(xb.data() + i * d));
            idx->ntotal = n;
            cpu.reset(idx);
        }
        std::unique_ptr<faiss::Index> gpu = backend.CpuToGpu(cpu.get());
        if (gpu->ntotal != n || gpu->d != d) {
            fprintf(stderr, "converted index has ntotal=%lld d=%d\n", (long long)gpu->ntotal, gpu->d);
            return 1;
        }
        std::vector<float> D((size_t)(nq * k)), D1((size_t)(nq * k));
        std::vector<int64_t> I((size_t)(nq * k)), I1((size_t)(nq * k));
        gpu->search(nq, xq.data(), k, D.data(), I.data());
        for (int64_t q = 0; q < nq; q++) gpu->search(1, xq.data() + q * d, k, D1.data() + q * k, I1.data() + q * k);

        // searchAsync (MetalIndexFlat.h:71-76): one token per query, all in flight, then waited
        // on in reverse order; the answers are those of the synchronous calls
        int async_ok = 1;
        // CpuToGpu hands out a CudaIndexFlat for an IndexFlat on one device (a CudaShardedIndex,
        // which has no tokens, when several devices are configured)
        if (auto *gf = dynamic_cast<faiss_cuda::CudaIndexFlat *>(gpu.get())) {
            std::vector<float> D2((size_t)(nq * k));
            std::vector<int64_t> I2((size_t)(nq * k));
            std::vector<faiss_cuda::CudaSearchToken> tokens;
            for (int64_t q = 0; q < nq; q++)
                tokens.push_back(gf->searchAsync(1, xq.data() + q * d, k, D2.data() + q * k, I2.data() + q * k));
            for (int64_t q = nq - 1; q >= 0; q--) tokens[(size_t)q].wait();
            for (auto &t : tokens) async_ok = async_ok && t.isReady();
            async_ok = async_ok && memcmp(D2.data(), D1.data(), D1.size() * 4) == 0 &&
                       memcmp(I2.data(), I1.data(), I1.size() * 8) == 0;
        }

        // round trip: every row comes back bit for bit
        std::unique_ptr<faiss::Index> back = backend.GpuToCpu(gpu.get());
        int roundtrip_ok = back->ntotal == n;
        if (!ivf) {
            auto *bf = dynamic_cast<faiss::IndexFlat *>(back.get());
            roundtrip_ok = roundtrip_ok && bf && memcmp(bf->get_xb(), xb.data(), xb.size() * 4) == 0;
            std::vector<float> one((size_t)d);
            if (n > 0) {
                gpu->reconstruct(n - 1, one.data());
                roundtrip_ok = roundtrip_ok && memcmp(one.data(), xb.data() + (n - 1) * d, (size_t)d * 4) == 0;
            }
        } else {
            auto *bi = dynamic_cast<faiss::IndexIVFFlat *>(back.get());
            roundtrip_ok = roundtrip_ok && bi && bi->nprobe == (size_t)nprobe;
            auto *ci = dynamic_cast<faiss::IndexIVFFlat *>(cpu.get());
            for (size_t l = 0; roundtrip_ok && l < (size_t)nlist; l++) {
                const size_t sz = ci->invlists->list_size(l);
                roundtrip_ok = bi->invlists->list_size(l) == sz &&
                               (sz == 0 || (memcmp(bi->invlists->get_ids(l), ci->invlists->get_ids(l), sz * 8) == 0 &&
                                            memcmp(bi->invlists->get_codes(l), ci->invlists->get_codes(l), sz * d * 4) == 0));
            }
        }
        // unsupported type -> std::runtime_error (gpu_backend_metal.mm:58-59)
        int rejects_unknown = 0;
        struct Other : faiss::Index {
            void add(faiss::idx_t, const float *) override {}
            void search(faiss::idx_t, const float *, faiss::idx_t, float *, faiss::idx_t *,
                        const faiss::SearchParameters *) const override {}
            void reset() override {}
        } other;
        try {
            backend.CpuToGpu(&other);
        } catch (const std::runtime_error &) {
            rejects_unknown = 1;
        }
        FILE *o = fopen(argv[3], "wb");
        if (!o) return 2;
        fwrite(D.data(), 4, D.size(), o);
        fwrite(I.data(), 8, I.size(), o);
        fwrite(D1.data(), 4, D1.size(), o);
        fwrite(I1.data(), 8, I1.size(), o);
        fclose(o);
        auto *sharded = dynamic_cast<faiss_cuda::CudaShardedIndex *>(gpu.get());
        printf("{\"backend\": \"%s\", \"roundtrip_ok\": %d, \"rejects_unknown\": %d, \"async_ok\": %d, \"shards\": %d}\n",
               backend.BackendName().c_str(), roundtrip_ok, rejects_unknown, async_ok, sharded ? sharded->shardCount() : 1);
        return 0;
    } catch (const std::exception &e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
