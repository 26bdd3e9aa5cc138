// Stand-in for <faiss/IndexIVFFlat.h> and <faiss/invlists/InvertedLists.h>; see
// README.md in this directory.
#pragma once
#include <faiss/IndexFlat.h>

#include <cstddef>
#include <cstdint>
#include <vector>

namespace faiss {

struct InvertedLists {
    size_t nlist;
    size_t code_size;
    InvertedLists(size_t nlist, size_t code_size) : nlist(nlist), code_size(code_size) {}
    virtual ~InvertedLists() {}
    virtual size_t list_size(size_t list_no) const = 0;
    virtual const uint8_t *get_codes(size_t list_no) const = 0;
    virtual const idx_t *get_ids(size_t list_no) const = 0;
    virtual void release_codes(size_t, const uint8_t *) const {}
    virtual void release_ids(size_t, const idx_t *) const {}
    virtual size_t add_entries(size_t list_no, size_t n_entry, const idx_t *ids, const uint8_t *code) = 0;
};

struct ArrayInvertedLists : InvertedLists {
    std::vector<std::vector<uint8_t>> codes;
    std::vector<std::vector<idx_t>> ids;
    ArrayInvertedLists(size_t nlist, size_t code_size) : InvertedLists(nlist, code_size), codes(nlist), ids(nlist) {}
    size_t list_size(size_t l) const override { return ids[l].size(); }
    const uint8_t *get_codes(size_t l) const override { return codes[l].data(); }
    const idx_t *get_ids(size_t l) const override { return ids[l].data(); }
    size_t add_entries(size_t l, size_t n, const idx_t *i, const uint8_t *c) override {
        size_t o = ids[l].size();
        ids[l].insert(ids[l].end(), i, i + n);
        codes[l].insert(codes[l].end(), c, c + n * code_size);
        return o;
    }
};

// Container for a trained IVFFlat index: quantizer (an IndexFlat of centroids),
// inverted lists of raw fp32 rows.  No CPU training, assignment or search here.
struct IndexIVFFlat : Index {
    Index *quantizer;
    size_t nlist;
    size_t nprobe;
    InvertedLists *invlists;
    bool own_invlists;
    bool own_fields;
    size_t code_size;

    IndexIVFFlat(Index *quantizer, size_t d, size_t nlist, MetricType metric = METRIC_L2)
        : Index((idx_t)d, metric), quantizer(quantizer), nlist(nlist), nprobe(1),
          invlists(new ArrayInvertedLists(nlist, d * sizeof(float))), own_invlists(true), own_fields(false),
          code_size(d * sizeof(float)) {
        is_trained = quantizer && quantizer->ntotal == (idx_t)nlist;
    }
    ~IndexIVFFlat() override {
        if (own_invlists) delete invlists;
        if (own_fields) delete quantizer;
    }
    void add(idx_t, const float *) override {
        throw std::runtime_error("faiss stand-in: no CPU assignment; use invlists->add_entries");
    }
    void search(idx_t, const float *, idx_t, float *, idx_t *, const SearchParameters * = nullptr) const override {
        throw std::runtime_error("faiss stand-in: no CPU search; link libfaiss for a CPU index");
    }
    void reset() override {
        for (size_t l = 0; l < nlist; l++) {
            static_cast<ArrayInvertedLists *>(invlists)->ids[l].clear();
            static_cast<ArrayInvertedLists *>(invlists)->codes[l].clear();
        }
        ntotal = 0;
    }
};

}  // namespace faiss
