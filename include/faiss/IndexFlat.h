// Stand-in for <faiss/IndexFlat.h>; see README.md in this directory.
#pragma once
#include <faiss/Index.h>

#include <cstring>
#include <vector>

namespace faiss {

// Row storage only.  The real class also searches on the CPU; this one refuses to.
struct IndexFlat : Index {
    std::vector<float> xb;

    explicit IndexFlat(idx_t d = 0, MetricType metric = METRIC_L2) : Index(d, metric) {}

    void add(idx_t n, const float *x) override {
        xb.insert(xb.end(), x, x + n * d);
        ntotal += n;
    }
    void search(idx_t, const float *, idx_t, float *, idx_t *, const SearchParameters * = nullptr) const override {
        throw std::runtime_error("faiss stand-in: no CPU search; link libfaiss for a CPU index");
    }
    void reset() override {
        xb.clear();
        ntotal = 0;
    }
    void reconstruct(idx_t key, float *recons) const override {
        if (key < 0 || key >= ntotal) throw std::runtime_error("reconstruct: key out of range");
        std::memcpy(recons, xb.data() + key * d, sizeof(float) * d);
    }
    float *get_xb() { return xb.data(); }
    const float *get_xb() const { return xb.data(); }
};

struct IndexFlatL2 : IndexFlat {
    explicit IndexFlatL2(idx_t d = 0) : IndexFlat(d, METRIC_L2) {}
};
struct IndexFlatIP : IndexFlat {
    explicit IndexFlatIP(idx_t d = 0) : IndexFlat(d, METRIC_INNER_PRODUCT) {}
};

}  // namespace faiss
