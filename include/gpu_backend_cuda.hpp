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

#include <cstdint>
#include <memory>
#include <vector>

struct ann_cuda_index;
struct ann_cuda_search_token;
struct ann_cuda_sharded_index;

// The classes are part of the library's interface: their type information is exported even
// though the library is built with hidden visibility (dynamic_cast across the boundary).
#if defined(__GNUC__)
#define ANN_CUDA_CLASS __attribute__((visibility("default")))
#else
#define ANN_CUDA_CLASS
#endif

namespace faiss_cuda {

// Move-only handle of one in-flight search (the role of faiss_metal::MetalSearchToken,
// faiss-metal/include/faiss-metal/MetalIndexFlat.h:15-36).
class ANN_CUDA_CLASS CudaSearchToken {
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

// Row storage precision of CudaIndexFlat: faiss_metal::StorageType
// (faiss-metal/include/faiss-metal/MetalIndexFlat.h:38-43), same values.
enum class StorageType : uint8_t {
    Float32 = 0,
    Float16 = 1,   // rows rounded to fp16 when added, 2 bytes per element
    BFloat16 = 2,  // rows rounded to bf16 when added, 2 bytes per element
};

class ANN_CUDA_CLASS CudaIndexFlat : public faiss::Index {
public:
    CudaIndexFlat(int device, int d, faiss::MetricType metric = faiss::METRIC_L2);
    // MetalIndexFlat(resources, d, metric, storage) (MetalIndexFlat.h:60): queries stay fp32, the search
    // answers for the rounded rows.
    CudaIndexFlat(int device, int d, faiss::MetricType metric, StorageType storage);
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

    // Copies rows [first, first + n) to host memory (the role of getVectorsData()); a reduced-precision
    // store hands out its rounded rows widened to fp32.
    void getRows(faiss::idx_t first, faiss::idx_t n, float *rows) const;
    // MetalIndexFlat.h:83-90
    bool isFloat16Storage() const { return getStorageType() == StorageType::Float16; }
    bool isBFloat16Storage() const { return getStorageType() == StorageType::BFloat16; }
    StorageType getStorageType() const;
    ann_cuda_index *handle() const { return handle_; }

private:
    ann_cuda_index *handle_ = nullptr;
};

class ANN_CUDA_CLASS CudaIndexIVFFlat : public faiss::Index {
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

// One Flat (nlist = 0) or IVFFlat index spread over several GPUs of the box, searched from the one
// process that owns it through the ordinary faiss::Index calls.  No counterpart in the reference
// (single device); it is what CudaGpuBackend::CpuToGpu returns when ANN_CUDA_DEVICES names more
// than one device.  Flat: contiguous row ranges; IVFFlat: list l on shard l % shards.
class ANN_CUDA_CLASS CudaShardedIndex : public faiss::Index {
public:
    CudaShardedIndex(const std::vector<int> &devices, int d, size_t nlist, faiss::MetricType metric = faiss::METRIC_L2);
    ~CudaShardedIndex() override;
    CudaShardedIndex(const CudaShardedIndex &) = delete;
    CudaShardedIndex &operator=(const CudaShardedIndex &) = delete;

    void train(faiss::idx_t n, const float *x) override;
    void add(faiss::idx_t n, const float *x) override;
    void search(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances, faiss::idx_t *labels,
                const faiss::SearchParameters *params = nullptr) const override;
    void reset() override;
    void reconstruct(faiss::idx_t key, float *recons) const override;

    bool isIVF() const { return nlist_ > 0; }
    size_t getNlist() const { return nlist_; }
    size_t getNprobe() const { return nprobe_; }
    void setNprobe(size_t nprobe);
    int shardCount() const;
    ann_cuda_sharded_index *handle() const { return handle_; }

private:
    ann_cuda_sharded_index *handle_ = nullptr;
    size_t nlist_ = 0, nprobe_ = 1;
};

// Conversions (faiss-metal/src/MetalIndexFlat.mm:504-535,
// faiss-metal/src/MetalIndexIVFFlat.mm:283-356).
std::unique_ptr<CudaIndexFlat> index_cpu_to_cuda(int device, const faiss::IndexFlat *cpu_index,
                                                 StorageType storage = StorageType::Float32);
std::unique_ptr<faiss::IndexFlat> index_cuda_to_cpu(const CudaIndexFlat *cuda_index);
std::unique_ptr<CudaIndexIVFFlat> index_cpu_to_cuda_ivf(int device, const faiss::IndexIVFFlat *cpu_index);
std::unique_ptr<faiss::IndexIVFFlat> index_cuda_to_cpu_ivf(const CudaIndexIVFFlat *cuda_index);
// ... and the same onto / back from several devices
std::unique_ptr<CudaShardedIndex> index_cpu_to_cuda_sharded(const std::vector<int> &devices, const faiss::IndexFlat *cpu_index);
std::unique_ptr<CudaShardedIndex> index_cpu_to_cuda_sharded_ivf(const std::vector<int> &devices,
                                                               const faiss::IndexIVFFlat *cpu_index);
std::unique_ptr<faiss::Index> index_cuda_sharded_to_cpu(const CudaShardedIndex *cuda_index);

}  // namespace faiss_cuda
