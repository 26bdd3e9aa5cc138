// CUDA (sm_100a) implementations of faiss::Index for the GpuBackend plugin: the
// counterparts of faiss_metal::MetalIndexFlat / MetalIndexIVFFlat
// (faiss-metal/include/faiss-metal/MetalIndexFlat.h:47-101,
//  faiss-metal/include/faiss-metal/MetalIndexIVFFlat.h:25-76).
// Each class owns a handle of the C ABI in ann_cuda.h and forwards to it; C-ABI
// errors surface as std::runtime_error, which FaissIndex catches
// (src/faiss_index.cpp:122,146).
#pragma once

#include <faiss/Index.h>
#include <faiss/IndexFlat.h>
#include <faiss/IndexIVFFlat.h>

#include <memory>

struct ann_cuda_index;
struct ann_cuda_search_token;

namespace faiss_cuda {

// Move-only handle of one in-flight search (the role of faiss_metal::MetalSearchToken,
// faiss-metal/include/faiss-metal/MetalIndexFlat.h:15-36).
class CudaSearchToken {
public:
    CudaSearchToken(CudaSearchToken &&o) noexcept : token_(o.token_) { o.token_ = nullptr; }
    CudaSearchToken &operator=(CudaSearchToken &&o) noexcept;
    ~CudaSearchToken();
    CudaSearchToken(const CudaSearchToken &) = delete;
    CudaSearchToken &operator=(const CudaSearchToken &) = delete;

    void wait();           // blocks, then the caller's distances / labels are filled; throws on a device error
    bool isReady() const;  // non-blocking

private:
    friend class CudaIndexFlat;
    explicit CudaSearchToken(ann_cuda_search_token *t) : token_(t) {}
    ann_cuda_search_token *token_ = nullptr;
};

class CudaIndexFlat : public faiss::Index {
public:
    CudaIndexFlat(int device, int d, faiss::MetricType metric = faiss::METRIC_L2);
    ~CudaIndexFlat() override;
    CudaIndexFlat(const CudaIndexFlat &) = delete;
    CudaIndexFlat &operator=(const CudaIndexFlat &) = delete;

    void add(faiss::idx_t n, const float *x) override;
    void search(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances, faiss::idx_t *labels,
                const faiss::SearchParameters *params = nullptr) const override;
    void reset() override;
    void reconstruct(faiss::idx_t key, float *recons) const override;

    // Enqueues the search and returns; token.wait() fills distances / labels
    // (MetalIndexFlat.h:71-76).  x may be reused as soon as this returns.
    CudaSearchToken searchAsync(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances, faiss::idx_t *labels,
                                const faiss::SearchParameters *params = nullptr) const;

    // Copies rows [first, first + n) to host memory (the role of getVectorsData()).
    void getRows(faiss::idx_t first, faiss::idx_t n, float *rows) const;
    ann_cuda_index *handle() const { return handle_; }

private:
    ann_cuda_index *handle_ = nullptr;
};

class CudaIndexIVFFlat : public faiss::Index {
public:
    CudaIndexIVFFlat(int device, int d, size_t nlist, faiss::MetricType metric = faiss::METRIC_L2);
    ~CudaIndexIVFFlat() override;
    CudaIndexIVFFlat(const CudaIndexIVFFlat &) = delete;
    CudaIndexIVFFlat &operator=(const CudaIndexIVFFlat &) = delete;

    void train(faiss::idx_t n, const float *x) override;
    void add(faiss::idx_t n, const float *x) override;
    void search(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances, faiss::idx_t *labels,
                const faiss::SearchParameters *params = nullptr) const override;
    void reset() override;
    void reconstruct(faiss::idx_t key, float *recons) const override;

    size_t getNlist() const;
    size_t getNprobe() const;
    void setNprobe(size_t nprobe);
    ann_cuda_index *handle() const { return handle_; }

private:
    friend std::unique_ptr<CudaIndexIVFFlat> index_cpu_to_cuda_ivf(int device, const faiss::IndexIVFFlat *cpu_index);
    ann_cuda_index *handle_ = nullptr;
};

// Conversions (faiss-metal/src/MetalIndexFlat.mm:504-535,
// faiss-metal/src/MetalIndexIVFFlat.mm:283-356).
std::unique_ptr<CudaIndexFlat> index_cpu_to_cuda(int device, const faiss::IndexFlat *cpu_index);
std::unique_ptr<faiss::IndexFlat> index_cuda_to_cpu(const CudaIndexFlat *cuda_index);
std::unique_ptr<CudaIndexIVFFlat> index_cpu_to_cuda_ivf(int device, const faiss::IndexIVFFlat *cpu_index);
std::unique_ptr<faiss::IndexIVFFlat> index_cuda_to_cpu_ivf(const CudaIndexIVFFlat *cuda_index);

}  // namespace faiss_cuda
