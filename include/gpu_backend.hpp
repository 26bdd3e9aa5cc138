// GPU backend plugin interface of the FAISS index type.
//
// This is the boundary the extension's FaissIndex talks to
// (src/include/gpu_backend.hpp:12-33 in the reference): the class name, the five
// virtuals, their signatures and GetGpuBackend() are kept as they are there so
// that src/faiss_index.cpp:108-153 and src/faiss_fn_gpu.cpp:33-46 compile against
// this header unchanged.
#pragma once

#ifdef FAISS_AVAILABLE

#include <faiss/Index.h>

#include <memory>
#include <string>

namespace duckdb {

class GpuBackend {
public:
    virtual ~GpuBackend() = default;

    // True when a usable device is present.  Never throws.
    virtual bool IsAvailable() const = 0;

    // Human-readable device description, shown by faiss_gpu_info().
    virtual std::string DeviceInfo() const = 0;

    // Short backend name ("cuda" here; the reference has "metal" and "cpu").
    virtual std::string BackendName() const = 0;

    // Copies a CPU index to the GPU and returns the GPU index; the CPU index is only
    // read.  Throws std::runtime_error on failure or for unsupported index types.
    virtual std::unique_ptr<faiss::Index> CpuToGpu(faiss::Index *cpu_index) = 0;

    // Copies a GPU index back into a new CPU index.  Throws on failure.
    virtual std::unique_ptr<faiss::Index> GpuToCpu(faiss::Index *gpu_index) = 0;
};

// Process-wide backend singleton.  Exactly one translation unit defines it: this
// library does when built with FAISS_CUDA_ENABLED.
GpuBackend &GetGpuBackend();

}  // namespace duckdb

#endif  // FAISS_AVAILABLE
