// The GPU-related slice of the extension's FaissIndex, restated over GetGpuBackend() so that the
// glue a maintainer adds on the reference side can be compiled and tested here without DuckDB:
//   EnsureGpuIndex / InvalidateGpuIndex      src/faiss_index.cpp:108-153
//   Search (request_k, tombstones, -1 slots)  src/faiss_index.cpp:708-762
// and the two changes that make SQL reach the batched GPU path:
//   * after an invalidation (Append, MergeIndexes, Vacuum: src/faiss_index.cpp:469, 835, 897) the
//     next search uploads the index again - the reference drops the GPU copy and then searches on
//     the CPU until the next load, although its README promises a rebuild on the next search;
//   * SearchBatch: ONE search(n, ...) call for a batch of queries, instead of the per-query loops
//     of ann_search_batch / ann_search_table (src/ann_search.cpp:324-331, 614-620).
// Everything DuckDB-specific (storage, catalog, row ids) is left out: labels are returned as they
// are.  Errors are std::runtime_error where the reference throws InvalidInputException.
#pragma once

#include <cstdint>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_set>
#include <utility>
#include <vector>

#ifndef FAISS_AVAILABLE
#define FAISS_AVAILABLE
#endif
#include "gpu_backend.hpp"

namespace duckdb_glue {

enum class FaissGpuMode : uint8_t { CPU, GPU, AUTO };  // src/include/faiss_index.hpp:8

class FaissIndexGlue {
public:
    FaissIndexGlue(std::unique_ptr<faiss::Index> cpu_index, FaissGpuMode mode, std::string index_type = "Flat")
        : faiss_index_(std::move(cpu_index)), mode_(mode), index_type_(std::move(index_type)),
          dimension_(faiss_index_ ? faiss_index_->d : 0) {}

    // Finalize / LoadFromStorage call this once the CPU index is complete.
    void EnsureGpuIndex() {
        std::lock_guard<std::mutex> lock(gpu_mu_);
        EnsureGpuIndexLocked();
    }
    void InvalidateGpuIndex() {
        std::lock_guard<std::mutex> lock(gpu_mu_);
        gpu_index_.reset();
        gpu_stale_ = true;
    }

    // Append (src/faiss_index.cpp:430-470): rows go to the CPU index, the GPU copy is dropped.
    void Append(faiss::idx_t n, const float *x) {
        faiss_index_->add(n, x);
        InvalidateGpuIndex();
    }
    // Delete marks a label; Search asks for that many more results and skips it (:713-718, :753).
    void Delete(faiss::idx_t label) { deleted_labels_.insert(label); }

    std::vector<std::pair<faiss::idx_t, float>> Search(const float *query, int32_t dimension, int32_t k) {
        auto all = SearchBatch(query, 1, dimension, k);
        return all.empty() ? std::vector<std::pair<faiss::idx_t, float>>() : std::move(all[0]);
    }

    // One search(n, ...) for all queries; per query the first k labels that are neither -1 nor deleted.
    std::vector<std::vector<std::pair<faiss::idx_t, float>>> SearchBatch(const float *queries, int64_t n, int32_t dimension,
                                                                         int32_t k) {
        std::vector<std::vector<std::pair<faiss::idx_t, float>>> results;
        if (!faiss_index_ || dimension != dimension_ || n <= 0) return results;
        int64_t request_k = (int64_t)k + (int64_t)deleted_labels_.size();
        if (request_k > faiss_index_->ntotal) request_k = faiss_index_->ntotal;
        if (request_k <= 0) return results;
        faiss::Index *search_index = SearchIndex();
        std::vector<float> distances((size_t)(n * request_k));
        std::vector<faiss::idx_t> labels((size_t)(n * request_k));
        search_index->search(n, queries, request_k, distances.data(), labels.data());
        results.resize((size_t)n);
        for (int64_t q = 0; q < n; q++) {
            auto &out = results[(size_t)q];
            out.reserve((size_t)k);
            for (int64_t i = 0; i < request_k && (int32_t)out.size() < k; i++) {
                const faiss::idx_t label = labels[(size_t)(q * request_k + i)];
                if (label < 0) continue;  // unfilled slot
                if (deleted_labels_.count(label)) continue;
                out.emplace_back(label, distances[(size_t)(q * request_k + i)]);
            }
        }
        return results;
    }

    bool OnGpu() const { return gpu_index_ != nullptr; }
    int GpuUploads() const { return gpu_uploads_; }
    faiss::Index *CpuIndex() const { return faiss_index_.get(); }

private:
    // The index a search runs on: the GPU copy, uploaded again first if an update dropped it.
    faiss::Index *SearchIndex() {
        std::lock_guard<std::mutex> lock(gpu_mu_);
        if (!gpu_index_ && gpu_stale_) EnsureGpuIndexLocked();
        return gpu_index_ ? gpu_index_.get() : faiss_index_.get();
    }
    void EnsureGpuIndexLocked() {
        if (mode_ == FaissGpuMode::CPU || !faiss_index_ || gpu_index_) return;
        duckdb::GpuBackend &backend = duckdb::GetGpuBackend();
        gpu_stale_ = false;
        if (mode_ == FaissGpuMode::GPU) {  // explicit: an unavailable or unsuitable GPU is an error
            if (!backend.IsAvailable()) throw std::runtime_error("mode='gpu' requested but no GPU backend available");
            try {
                gpu_index_ = backend.CpuToGpu(faiss_index_.get());
            } catch (std::runtime_error &e) {
                throw std::runtime_error(std::string("mode='gpu' requested but index type unsupported on GPU: ") + e.what());
            }
            gpu_uploads_++;
            return;
        }
        // AUTO: the reference's heuristic (:129-148)
        if (!backend.IsAvailable()) return;
        if (index_type_ == "HNSW" || index_type_ == "hnsw") return;
        if (faiss_index_->ntotal < 256) return;
        if (dimension_ < 128) return;
        try {
            gpu_index_ = backend.CpuToGpu(faiss_index_.get());
            gpu_uploads_++;
        } catch (std::runtime_error &) {
            // AUTO mode falls back to the CPU index without a word
        }
    }

    std::unique_ptr<faiss::Index> faiss_index_;
    std::unique_ptr<faiss::Index> gpu_index_;
    FaissGpuMode mode_;
    std::string index_type_;
    int dimension_;
    std::unordered_set<faiss::idx_t> deleted_labels_;
    std::mutex gpu_mu_;
    bool gpu_stale_ = false;
    int gpu_uploads_ = 0;
};

}  // namespace duckdb_glue
