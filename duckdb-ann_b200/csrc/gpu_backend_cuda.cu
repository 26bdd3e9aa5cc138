// CudaGpuBackend and the faiss::Index subclasses it hands out.
//
// Counterpart of the reference's src/gpu_backend_metal.mm (backend) and of the
// index classes in faiss-metal/src/MetalIndexFlat.mm / MetalIndexIVFFlat.mm; all
// device work goes through the C ABI in ann_cuda.h.
#include "gpu_backend_cuda.hpp"

#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

#include "ann_cuda.h"

#ifndef FAISS_AVAILABLE
#define FAISS_AVAILABLE
#endif
#include "gpu_backend.hpp"

#if defined(__GNUC__)
#define ANN_CUDA_EXPORT __attribute__((visibility("default")))
#else
#define ANN_CUDA_EXPORT
#endif

namespace faiss_cuda {

namespace {
[[noreturn]] void fail(const char *what) {
    throw std::runtime_error(std::string(what) + ": " + ann_cuda_last_error());
}
int metric_code(faiss::MetricType m) {
    if (m == faiss::METRIC_L2) return ANN_CUDA_METRIC_L2;
    if (m == faiss::METRIC_INNER_PRODUCT) return ANN_CUDA_METRIC_INNER_PRODUCT;
    throw std::runtime_error("CUDA GPU backend supports METRIC_L2 and METRIC_INNER_PRODUCT only");
}
}  // namespace

// ---------------------------------------------------------------- CudaIndexFlat
ANN_CUDA_EXPORT CudaIndexFlat::CudaIndexFlat(int device, int d, faiss::MetricType metric) : faiss::Index(d, metric) {
    if (ann_cuda_flat_create(device, d, metric_code(metric), &handle_)) fail("CudaIndexFlat");
    is_trained = true;
}
ANN_CUDA_EXPORT CudaIndexFlat::CudaIndexFlat(int device, int d, faiss::MetricType metric, StorageType storage)
    : faiss::Index(d, metric) {
    if (ann_cuda_flat_create_storage(device, d, metric_code(metric), (int)storage, &handle_)) fail("CudaIndexFlat");
    is_trained = true;
}
ANN_CUDA_EXPORT StorageType CudaIndexFlat::getStorageType() const {
    const int s = ann_cuda_index_storage(handle_);
    return s == ANN_CUDA_STORAGE_F16 ? StorageType::Float16 : s == ANN_CUDA_STORAGE_BF16 ? StorageType::BFloat16 : StorageType::Float32;
}
ANN_CUDA_EXPORT CudaIndexFlat::~CudaIndexFlat() { ann_cuda_index_free(handle_); }

ANN_CUDA_EXPORT void CudaIndexFlat::add(faiss::idx_t n, const float *x) {
    if (ann_cuda_index_add(handle_, n, x)) fail("CudaIndexFlat::add");
    ntotal = ann_cuda_index_ntotal(handle_);
}
ANN_CUDA_EXPORT void CudaIndexFlat::search(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances,
                                           faiss::idx_t *labels, const faiss::SearchParameters *) const {
    if (k <= 0) throw std::runtime_error("k must be > 0");
    if (ann_cuda_index_search(handle_, n, x, k, distances, labels)) fail("CudaIndexFlat::search");
}
ANN_CUDA_EXPORT void CudaIndexFlat::reset() {
    if (ann_cuda_index_reset(handle_)) fail("CudaIndexFlat::reset");
    ntotal = 0;
}
ANN_CUDA_EXPORT CudaSearchToken CudaIndexFlat::searchAsync(faiss::idx_t n, const float *x, faiss::idx_t k,
                                                           float *distances, faiss::idx_t *labels,
                                                           const faiss::SearchParameters *) const {
    ann_cuda_search_token *t = nullptr;
    if (ann_cuda_index_search_async(handle_, n, x, k, distances, labels, &t)) fail("CudaIndexFlat::searchAsync");
    return CudaSearchToken(t);
}
ANN_CUDA_EXPORT CudaSearchToken &CudaSearchToken::operator=(CudaSearchToken &&o) noexcept {
    if (this != &o) {
        ann_cuda_search_token_free(token_);
        token_ = o.token_;
        o.token_ = nullptr;
    }
    return *this;
}
ANN_CUDA_EXPORT CudaSearchToken::~CudaSearchToken() { ann_cuda_search_token_free(token_); }
ANN_CUDA_EXPORT void CudaSearchToken::wait() {
    if (token_ && ann_cuda_search_token_wait(token_)) fail("CudaSearchToken::wait");
}
ANN_CUDA_EXPORT bool CudaSearchToken::isReady() const { return !token_ || ann_cuda_search_token_ready(token_) == 1; }

ANN_CUDA_EXPORT void CudaIndexFlat::reconstruct(faiss::idx_t key, float *recons) const {
    if (ann_cuda_index_reconstruct(handle_, key, recons)) fail("CudaIndexFlat::reconstruct");
}
ANN_CUDA_EXPORT void CudaIndexFlat::getRows(faiss::idx_t first, faiss::idx_t n, float *rows) const {
    if (ann_cuda_flat_get_rows(handle_, first, n, rows)) fail("CudaIndexFlat::getRows");
}

// ---------------------------------------------------------------- CudaIndexIVFFlat
ANN_CUDA_EXPORT CudaIndexIVFFlat::CudaIndexIVFFlat(int device, int d, size_t nlist, faiss::MetricType metric)
    : faiss::Index(d, metric) {
    if (ann_cuda_ivfflat_create(device, d, (int64_t)nlist, metric_code(metric), &handle_)) fail("CudaIndexIVFFlat");
    is_trained = false;
}
ANN_CUDA_EXPORT CudaIndexIVFFlat::~CudaIndexIVFFlat() { ann_cuda_index_free(handle_); }

ANN_CUDA_EXPORT void CudaIndexIVFFlat::train(faiss::idx_t n, const float *x) {
    if (ann_cuda_ivfflat_train(handle_, n, x)) fail("CudaIndexIVFFlat::train");
    is_trained = true;
}
ANN_CUDA_EXPORT void CudaIndexIVFFlat::add(faiss::idx_t n, const float *x) {
    if (!is_trained) throw std::runtime_error("add: index must be trained first");
    if (ann_cuda_index_add(handle_, n, x)) fail("CudaIndexIVFFlat::add");
    ntotal = ann_cuda_index_ntotal(handle_);
}
ANN_CUDA_EXPORT void CudaIndexIVFFlat::search(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances,
                                              faiss::idx_t *labels, const faiss::SearchParameters *) const {
    if (!is_trained) throw std::runtime_error("search: index must be trained first");
    if (k <= 0) throw std::runtime_error("k must be > 0");
    if (ann_cuda_index_search(handle_, n, x, k, distances, labels)) fail("CudaIndexIVFFlat::search");
}
ANN_CUDA_EXPORT void CudaIndexIVFFlat::reset() {
    if (ann_cuda_index_reset(handle_)) fail("CudaIndexIVFFlat::reset");
    ntotal = 0;
}
ANN_CUDA_EXPORT void CudaIndexIVFFlat::reconstruct(faiss::idx_t key, float *recons) const {
    if (ann_cuda_index_reconstruct(handle_, key, recons)) fail("CudaIndexIVFFlat::reconstruct");
}
ANN_CUDA_EXPORT size_t CudaIndexIVFFlat::getNlist() const { return (size_t)ann_cuda_ivfflat_nlist(handle_); }
ANN_CUDA_EXPORT size_t CudaIndexIVFFlat::getNprobe() const { return (size_t)ann_cuda_ivfflat_get_nprobe(handle_); }
ANN_CUDA_EXPORT void CudaIndexIVFFlat::setNprobe(size_t nprobe) {
    if (ann_cuda_ivfflat_set_nprobe(handle_, (int64_t)nprobe)) fail("CudaIndexIVFFlat::setNprobe");
}

// ---------------------------------------------------------------- conversions
ANN_CUDA_EXPORT std::unique_ptr<CudaIndexFlat> index_cpu_to_cuda(int device, const faiss::IndexFlat *cpu, StorageType storage) {
    std::unique_ptr<CudaIndexFlat> gpu(storage == StorageType::Float32
                                           ? new CudaIndexFlat(device, cpu->d, cpu->metric_type)
                                           : new CudaIndexFlat(device, cpu->d, cpu->metric_type, storage));
    if (cpu->ntotal > 0) {
        if (ann_cuda_index_reserve(gpu->handle(), cpu->ntotal)) fail("index_cpu_to_cuda");
        gpu->add(cpu->ntotal, cpu->get_xb());
    }
    return gpu;
}

ANN_CUDA_EXPORT std::unique_ptr<faiss::IndexFlat> index_cuda_to_cpu(const CudaIndexFlat *gpu) {
    std::unique_ptr<faiss::IndexFlat> cpu(new faiss::IndexFlat(gpu->d, gpu->metric_type));
    if (gpu->ntotal > 0) {
        std::vector<float> rows((size_t)gpu->ntotal * gpu->d);
        gpu->getRows(0, gpu->ntotal, rows.data());
        cpu->add(gpu->ntotal, rows.data());
    }
    return cpu;
}

ANN_CUDA_EXPORT std::unique_ptr<CudaIndexIVFFlat> index_cpu_to_cuda_ivf(int device, const faiss::IndexIVFFlat *cpu) {
    if (!cpu->is_trained) throw std::runtime_error("CPU IndexIVFFlat must be trained");
    auto *quantizer = dynamic_cast<const faiss::IndexFlat *>(cpu->quantizer);
    if (!quantizer) throw std::runtime_error("IndexIVFFlat quantizer must be IndexFlat");
    if ((size_t)quantizer->ntotal != cpu->nlist) throw std::runtime_error("quantizer size does not match nlist");
    std::unique_ptr<CudaIndexIVFFlat> gpu(new CudaIndexIVFFlat(device, cpu->d, cpu->nlist, cpu->metric_type));
    if (ann_cuda_ivfflat_set_centroids(gpu->handle_, quantizer->get_xb())) fail("index_cpu_to_cuda_ivf");
    gpu->is_trained = true;
    if (ann_cuda_index_reserve(gpu->handle_, cpu->ntotal)) fail("index_cpu_to_cuda_ivf");
    const faiss::InvertedLists *lists = cpu->invlists;
    for (size_t c = 0; c < cpu->nlist; c++) {
        const size_t n = lists->list_size(c);
        if (n == 0) continue;
        const faiss::idx_t *ids = lists->get_ids(c);
        const uint8_t *codes = lists->get_codes(c);
        const int rc = ann_cuda_ivfflat_add_list(gpu->handle_, (int64_t)c, (int64_t)n, ids,
                                                 reinterpret_cast<const float *>(codes));
        lists->release_ids(c, ids);
        lists->release_codes(c, codes);
        if (rc) fail("index_cpu_to_cuda_ivf");
    }
    gpu->ntotal = cpu->ntotal;
    gpu->setNprobe(cpu->nprobe);
    return gpu;
}

ANN_CUDA_EXPORT std::unique_ptr<faiss::IndexIVFFlat> index_cuda_to_cpu_ivf(const CudaIndexIVFFlat *gpu) {
    if (!gpu->is_trained) throw std::runtime_error("CUDA index must be trained");
    const int d = gpu->d;
    const size_t nlist = gpu->getNlist();
    std::vector<float> cent(nlist * (size_t)d);
    if (ann_cuda_ivfflat_get_centroids(gpu->handle(), cent.data())) fail("index_cuda_to_cpu_ivf");
    auto *quantizer = new faiss::IndexFlat(d, gpu->metric_type);
    quantizer->add((faiss::idx_t)nlist, cent.data());
    std::unique_ptr<faiss::IndexIVFFlat> cpu(new faiss::IndexIVFFlat(quantizer, d, nlist, gpu->metric_type));
    cpu->own_fields = true;
    cpu->is_trained = true;
    cpu->nprobe = gpu->getNprobe();
    std::vector<faiss::idx_t> ids;
    std::vector<float> rows;
    for (size_t c = 0; c < nlist; c++) {
        const int64_t n = ann_cuda_ivfflat_list_size(gpu->handle(), (int64_t)c);
        if (n < 0) fail("index_cuda_to_cpu_ivf");
        if (n == 0) continue;
        ids.resize((size_t)n);
        rows.resize((size_t)n * d);
        if (ann_cuda_ivfflat_get_list(gpu->handle(), (int64_t)c, ids.data(), rows.data())) fail("index_cuda_to_cpu_ivf");
        cpu->invlists->add_entries(c, (size_t)n, ids.data(), reinterpret_cast<const uint8_t *>(rows.data()));
    }
    cpu->ntotal = gpu->ntotal;
    return cpu;
}

// ---------------------------------------------------------------- CudaShardedIndex
ANN_CUDA_EXPORT CudaShardedIndex::CudaShardedIndex(const std::vector<int> &devices, int d, size_t nlist,
                                                   faiss::MetricType metric)
    : faiss::Index(d, metric), nlist_(nlist) {
    if (ann_cuda_sharded_create(devices.data(), (int)devices.size(), d, metric_code(metric), (int64_t)nlist, &handle_))
        fail("CudaShardedIndex");
    is_trained = nlist == 0;
}
ANN_CUDA_EXPORT CudaShardedIndex::~CudaShardedIndex() { ann_cuda_sharded_free(handle_); }
ANN_CUDA_EXPORT int CudaShardedIndex::shardCount() const { return ann_cuda_sharded_shard_count(handle_); }
ANN_CUDA_EXPORT void CudaShardedIndex::train(faiss::idx_t n, const float *x) {
    if (!isIVF()) return;
    if (ann_cuda_sharded_train(handle_, n, x)) fail("CudaShardedIndex::train");
    is_trained = true;
}
ANN_CUDA_EXPORT void CudaShardedIndex::add(faiss::idx_t n, const float *x) {
    if (!is_trained) throw std::runtime_error("add: index must be trained first");
    if (ann_cuda_sharded_add(handle_, n, x)) fail("CudaShardedIndex::add");
    ntotal = ann_cuda_sharded_ntotal(handle_);
}
ANN_CUDA_EXPORT void CudaShardedIndex::search(faiss::idx_t n, const float *x, faiss::idx_t k, float *distances,
                                              faiss::idx_t *labels, const faiss::SearchParameters *) const {
    if (!is_trained) throw std::runtime_error("search: index must be trained first");
    if (k <= 0) throw std::runtime_error("k must be > 0");
    if (ann_cuda_sharded_search(handle_, n, x, k, distances, labels)) fail("CudaShardedIndex::search");
}
ANN_CUDA_EXPORT void CudaShardedIndex::reset() {
    if (ann_cuda_sharded_reset(handle_)) fail("CudaShardedIndex::reset");
    ntotal = 0;
}
ANN_CUDA_EXPORT void CudaShardedIndex::reconstruct(faiss::idx_t key, float *recons) const {
    if (ann_cuda_sharded_reconstruct(handle_, key, recons)) fail("CudaShardedIndex::reconstruct");
}
ANN_CUDA_EXPORT void CudaShardedIndex::setNprobe(size_t nprobe) {
    if (!isIVF()) return;
    nprobe_ = nprobe < 1 ? 1 : (nprobe > nlist_ ? nlist_ : nprobe);  // MetalIndexIVFFlat.mm:275-279
    if (ann_cuda_sharded_set_nprobe(handle_, (int64_t)nprobe_)) fail("CudaShardedIndex::setNprobe");
}

ANN_CUDA_EXPORT std::unique_ptr<CudaShardedIndex> index_cpu_to_cuda_sharded(const std::vector<int> &devices,
                                                                            const faiss::IndexFlat *cpu) {
    std::unique_ptr<CudaShardedIndex> gpu(new CudaShardedIndex(devices, cpu->d, 0, cpu->metric_type));
    if (cpu->ntotal > 0) gpu->add(cpu->ntotal, cpu->get_xb());  // one add: equal contiguous row ranges
    return gpu;
}

ANN_CUDA_EXPORT std::unique_ptr<CudaShardedIndex> index_cpu_to_cuda_sharded_ivf(const std::vector<int> &devices,
                                                                                const faiss::IndexIVFFlat *cpu) {
    if (!cpu->is_trained) throw std::runtime_error("CPU IndexIVFFlat must be trained");
    auto *quantizer = dynamic_cast<const faiss::IndexFlat *>(cpu->quantizer);
    if (!quantizer) throw std::runtime_error("IndexIVFFlat quantizer must be IndexFlat");
    if ((size_t)quantizer->ntotal != cpu->nlist) throw std::runtime_error("quantizer size does not match nlist");
    std::unique_ptr<CudaShardedIndex> gpu(new CudaShardedIndex(devices, cpu->d, cpu->nlist, cpu->metric_type));
    if (ann_cuda_sharded_set_centroids(gpu->handle(), quantizer->get_xb())) fail("index_cpu_to_cuda_sharded_ivf");
    gpu->is_trained = true;
    const faiss::InvertedLists *lists = cpu->invlists;
    for (size_t c = 0; c < cpu->nlist; c++) {
        const size_t n = lists->list_size(c);
        if (n == 0) continue;
        const faiss::idx_t *ids = lists->get_ids(c);
        const uint8_t *codes = lists->get_codes(c);
        const int rc = ann_cuda_sharded_add_list(gpu->handle(), (int64_t)c, (int64_t)n, ids, reinterpret_cast<const float *>(codes));
        lists->release_ids(c, ids);
        lists->release_codes(c, codes);
        if (rc) fail("index_cpu_to_cuda_sharded_ivf");
    }
    gpu->ntotal = cpu->ntotal;
    gpu->setNprobe(cpu->nprobe);
    return gpu;
}

ANN_CUDA_EXPORT std::unique_ptr<faiss::Index> index_cuda_sharded_to_cpu(const CudaShardedIndex *gpu) {
    const int d = gpu->d;
    if (!gpu->isIVF()) {
        std::unique_ptr<faiss::IndexFlat> cpu(new faiss::IndexFlat(d, gpu->metric_type));
        if (gpu->ntotal > 0) {
            std::vector<float> rows((size_t)gpu->ntotal * d);
            if (ann_cuda_sharded_get_rows(gpu->handle(), 0, gpu->ntotal, rows.data())) fail("index_cuda_sharded_to_cpu");
            cpu->add(gpu->ntotal, rows.data());
        }
        return cpu;
    }
    if (!gpu->is_trained) throw std::runtime_error("CUDA index must be trained");
    const size_t nlist = gpu->getNlist();
    const int shards = gpu->shardCount();
    std::vector<float> cent(nlist * (size_t)d);
    if (ann_cuda_ivfflat_get_centroids(ann_cuda_sharded_shard(gpu->handle(), 0), cent.data())) fail("index_cuda_sharded_to_cpu");
    auto *quantizer = new faiss::IndexFlat(d, gpu->metric_type);
    quantizer->add((faiss::idx_t)nlist, cent.data());
    std::unique_ptr<faiss::IndexIVFFlat> cpu(new faiss::IndexIVFFlat(quantizer, d, nlist, gpu->metric_type));
    cpu->own_fields = true;
    cpu->is_trained = true;
    cpu->nprobe = gpu->getNprobe();
    std::vector<faiss::idx_t> ids;
    std::vector<float> rows;
    for (size_t c = 0; c < nlist; c++) {
        const ann_cuda_index *owner = ann_cuda_sharded_shard(gpu->handle(), (int)(c % (size_t)shards));
        const int64_t n = ann_cuda_ivfflat_list_size(owner, (int64_t)c);
        if (n < 0) fail("index_cuda_sharded_to_cpu");
        if (n == 0) continue;
        ids.resize((size_t)n);
        rows.resize((size_t)n * d);
        if (ann_cuda_ivfflat_get_list(owner, (int64_t)c, ids.data(), rows.data())) fail("index_cuda_sharded_to_cpu");
        cpu->invlists->add_entries(c, (size_t)n, ids.data(), reinterpret_cast<const uint8_t *>(rows.data()));
    }
    cpu->ntotal = gpu->ntotal;
    return cpu;
}

}  // namespace faiss_cuda

// ---------------------------------------------------------------- the backend
namespace duckdb {

class ANN_CUDA_EXPORT CudaGpuBackend : public GpuBackend {
public:
    // Availability is a flag; the constructor never throws (gpu_backend_metal.mm:17-24).
    CudaGpuBackend() {
        available_ = ann_cuda_available() != 0;
        const int count = ann_cuda_device_count();
        // ANN_CUDA_DEVICES = "0,1,2,3" or "all": indexes are spread over these devices (one process,
        // one host thread and stream per device).  Otherwise ANN_CUDA_DEVICE (one device, default 0).
        if (const char *many = std::getenv("ANN_CUDA_DEVICES")) {
            const std::string list(many);
            if (list == "all") {
                for (int i = 0; i < count; i++) devices_.push_back(i);
            } else {
                size_t pos = 0;
                while (pos < list.size()) {
                    size_t end = list.find(',', pos);
                    if (end == std::string::npos) end = list.size();
                    const std::string item = list.substr(pos, end - pos);
                    if (!item.empty()) {
                        const int dev = std::atoi(item.c_str());
                        if (dev >= 0 && dev < count) devices_.push_back(dev);
                    }
                    pos = end + 1;
                }
            }
        }
        // ANN_CUDA_STORAGE = f16 | bf16: flat indexes on one device keep their rows in 16 bits (the CPU index the
        // extension holds stays the source of truth in fp32; searches answer for the rounded rows)
        if (const char *st = std::getenv("ANN_CUDA_STORAGE")) {
            if (std::string(st) == "f16") storage_ = faiss_cuda::StorageType::Float16;
            if (std::string(st) == "bf16") storage_ = faiss_cuda::StorageType::BFloat16;
        }
        if (devices_.empty()) {
            const char *env = std::getenv("ANN_CUDA_DEVICE");
            int device = env ? std::atoi(env) : 0;
            if (device < 0 || device >= count) device = 0;
            devices_.push_back(device);
        }
    }
    bool IsAvailable() const override { return available_; }
    std::string DeviceInfo() const override {
        if (!available_) return "CUDA: not available";
        char buf[256];
        if (ann_cuda_device_info(buf, sizeof buf)) return "CUDA GPU";
        std::string info(buf);
        if (devices_.size() > 1) info += " [indexes sharded over " + std::to_string(devices_.size()) + " devices]";
        return info;
    }
    std::string BackendName() const override { return "cuda"; }

    std::unique_ptr<faiss::Index> CpuToGpu(faiss::Index *cpu_index) override {
        if (!available_) throw std::runtime_error("CUDA GPU backend not available");
        const bool sharded = devices_.size() > 1;
        // IVFFlat first: it also contains an IndexFlat quantizer (gpu_backend_metal.mm:47-51)
        if (auto *ivf = dynamic_cast<faiss::IndexIVFFlat *>(cpu_index)) {
            if (sharded) return faiss_cuda::index_cpu_to_cuda_sharded_ivf(devices_, ivf);
            return faiss_cuda::index_cpu_to_cuda_ivf(devices_[0], ivf);
        }
        if (auto *flat = dynamic_cast<faiss::IndexFlat *>(cpu_index)) {
            if (sharded) return faiss_cuda::index_cpu_to_cuda_sharded(devices_, flat);
            return faiss_cuda::index_cpu_to_cuda(devices_[0], flat, storage_);
        }
        throw std::runtime_error("CUDA GPU supports IndexFlat and IndexIVFFlat. Got an unsupported index type.");
    }
    std::unique_ptr<faiss::Index> GpuToCpu(faiss::Index *gpu_index) override {
        if (auto *sh = dynamic_cast<faiss_cuda::CudaShardedIndex *>(gpu_index)) return faiss_cuda::index_cuda_sharded_to_cpu(sh);
        if (auto *ivf = dynamic_cast<faiss_cuda::CudaIndexIVFFlat *>(gpu_index)) return faiss_cuda::index_cuda_to_cpu_ivf(ivf);
        if (auto *flat = dynamic_cast<faiss_cuda::CudaIndexFlat *>(gpu_index)) return faiss_cuda::index_cuda_to_cpu(flat);
        throw std::runtime_error("Index is not a CUDA index -- cannot convert to CPU");
    }

private:
    bool available_ = false;
    std::vector<int> devices_;
    faiss_cuda::StorageType storage_ = faiss_cuda::StorageType::Float32;
};

ANN_CUDA_EXPORT GpuBackend &GetGpuBackend() {
    static CudaGpuBackend instance;
    return instance;
}

}  // namespace duckdb
