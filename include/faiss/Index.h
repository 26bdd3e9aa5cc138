// Stand-in for <faiss/Index.h>; see README.md in this directory.
#pragma once
#include <faiss/MetricType.h>

#include <stdexcept>

namespace faiss {

struct SearchParameters {
    virtual ~SearchParameters() {}
};

struct Index {
    int d;
    idx_t ntotal;
    bool verbose;
    bool is_trained;
    MetricType metric_type;
    float metric_arg;

    explicit Index(idx_t d = 0, MetricType metric = METRIC_L2)
        : d((int)d), ntotal(0), verbose(false), is_trained(true), metric_type(metric), metric_arg(0) {}
    virtual ~Index() {}

    virtual void train(idx_t /*n*/, const float * /*x*/) {}
    virtual void add(idx_t n, const float *x) = 0;
    virtual void search(idx_t n, const float *x, idx_t k, float *distances, idx_t *labels,
                        const SearchParameters *params = nullptr) const = 0;
    virtual void reset() = 0;
    virtual void reconstruct(idx_t /*key*/, float * /*recons*/) const {
        throw std::runtime_error("reconstruct not implemented for this type of index");
    }
};

}  // namespace faiss
