// One index spread over several GPUs of a box, inside ONE process: the form of multi-GPU search
// that fits behind the reference's plugin surface, where a single process calls
// GetGpuBackend().CpuToGpu(index) once and then search() on what it got back
// (src/faiss_index.cpp:108-149, 729-737; src/include/gpu_backend.hpp:25-29).  The reference itself
// has no multi-GPU path.
//
// Flat: the rows are cut into contiguous ranges, one per shard; labels are global positions
// (label offset of a shard = rows of the shards before it).  IVFFlat: inverted list l lives on
// shard l % shards, the coarse quantiser is replicated.  A search hands the queries to every
// shard (one persistent host thread and one stream per shard), each shard runs the ordinary
// device search of index.cu, its (distance, label) lists are copied into the merging GPU's own
// memory with cudaMemcpyPeerAsync (NVLink when peer access is available; no kernel ever reads
// another GPU's memory), and the merge kernel of merge.cu selects the final k there.
#include <condition_variable>
#include <functional>
#include <memory>
#include <thread>

#include "ann_cuda.h"
#include "common.cuh"
#include "kernels.h"

using namespace anncuda;

namespace {

constexpr int64_t kShardQueryBlock = 16384;  // queries per pass: bounds the staging buffers

// A host thread bound to one shard; runs the tasks it is handed, one at a time.
class ShardWorker {
public:
    ShardWorker() : thread_([this] { loop(); }) {}
    ~ShardWorker() {
        {
            std::lock_guard<std::mutex> lock(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        thread_.join();
    }
    void post(std::function<int()> task) {
        std::lock_guard<std::mutex> lock(mu_);
        task_ = std::move(task);
        has_task_ = true;
        done_ = false;
        cv_.notify_all();
    }
    int wait(std::string *error) {
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [this] { return done_; });
        if (rc_ && error && error->empty()) *error = error_;
        return rc_;
    }

private:
    void loop() {
        for (;;) {
            std::function<int()> task;
            {
                std::unique_lock<std::mutex> lock(mu_);
                cv_.wait(lock, [this] { return has_task_ || stop_; });
                if (stop_) return;
                task = std::move(task_);
                has_task_ = false;
            }
            const int rc = task();
            {
                std::lock_guard<std::mutex> lock(mu_);
                rc_ = rc;
                error_ = rc ? ann_cuda_last_error() : "";  // the error text is per thread: carry it over
                done_ = true;
            }
            cv_.notify_all();
        }
    }
    std::mutex mu_;
    std::condition_variable cv_;
    std::function<int()> task_;
    bool has_task_ = false, done_ = true, stop_ = false;
    int rc_ = 0;
    std::string error_;
    std::thread thread_;
};

struct Shard {
    int device = 0;
    ann_cuda_index *ix = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t done = nullptr;
    GrowBuf xq, out_d, out_i;
    std::unique_ptr<ShardWorker> worker;
};

}  // namespace

struct ann_cuda_sharded_index {
    bool ivf = false;
    int d = 0, metric = ANN_CUDA_METRIC_L2;
    int64_t nlist = 0;
    std::vector<Shard> shards;
    // merging GPU = the first shard's device
    cudaStream_t merge_stream = nullptr;
    GrowBuf parts_d, parts_i, merged_d, merged_i;
    mutable std::mutex mu;  // searches and updates of one sharded index are serialised

    int merge_device() const { return shards[0].device; }

    // Runs fn(shard number) on every shard's own thread and waits for all of them.
    int on_every_shard(const std::function<int(int)> &fn) const {
        for (size_t g = 0; g < shards.size(); g++) shards[g].worker->post([&fn, g] { return fn((int)g); });
        int rc = 0;
        std::string error;
        for (const Shard &s : shards)
            if (s.worker->wait(&error)) rc = -1;
        if (rc) set_error("%s", error.c_str());
        return rc;
    }
    int64_t rows_before(int g) const {
        int64_t n = 0;
        for (int j = 0; j < g; j++) n += ann_cuda_index_ntotal(shards[j].ix);
        return n;
    }
};

namespace {

void free_shards(ann_cuda_sharded_index *s) {
    for (Shard &sh : s->shards) {
        sh.worker.reset();
        DeviceGuard g(sh.device);
        if (sh.ix) ann_cuda_index_free(sh.ix);
        if (sh.stream) cudaStreamSynchronize(sh.stream);
        sh.xq.release();
        sh.out_d.release();
        sh.out_i.release();
        if (sh.done) cudaEventDestroy(sh.done);
        if (sh.stream) cudaStreamDestroy(sh.stream);
    }
    if (!s->shards.empty()) {
        DeviceGuard g(s->merge_device());
        for (GrowBuf *b : {&s->parts_d, &s->parts_i, &s->merged_d, &s->merged_i}) b->release();
        if (s->merge_stream) cudaStreamDestroy(s->merge_stream);
    }
}

}  // namespace

extern "C" {

int ann_cuda_sharded_create(const int *devices, int ndev, int d, int metric, int64_t nlist, ann_cuda_sharded_index **out) {
    if (!out) return set_error("null output handle");
    *out = nullptr;
    if (!devices || ndev <= 0 || ndev > 64) return set_error("a sharded index needs 1 to 64 devices");
    auto *s = new ann_cuda_sharded_index();
    s->ivf = nlist > 0;
    s->d = d;
    s->metric = metric;
    s->nlist = nlist;
    s->shards.resize((size_t)ndev);
    int rc = 0;
    for (int g = 0; g < ndev && rc == 0; g++) {
        Shard &sh = s->shards[(size_t)g];
        sh.device = devices[g];
        rc = s->ivf ? ann_cuda_ivfflat_create(sh.device, d, nlist, metric, &sh.ix)
                    : ann_cuda_flat_create(sh.device, d, metric, &sh.ix);
        if (rc == 0 && s->ivf) rc = ann_cuda_ivfflat_set_shard(sh.ix, g, ndev);
        if (rc) break;
        DeviceGuard guard(sh.device);
        if (cudaStreamCreateWithFlags(&sh.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&sh.done, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            rc = set_error("could not create the stream of shard %d on device %d", g, sh.device);
            break;
        }
        // direct copies into the merging GPU's memory; without peer access the copy is staged by the driver
        if (g > 0 && sh.device != devices[0]) {
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, sh.device, devices[0]) == cudaSuccess && can) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(devices[0], 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            }
        }
        sh.worker.reset(new ShardWorker());
    }
    if (rc == 0) {
        DeviceGuard guard(devices[0]);
        if (cudaStreamCreateWithFlags(&s->merge_stream, cudaStreamNonBlocking) != cudaSuccess) {
            cudaGetLastError();
            rc = set_error("could not create the merge stream on device %d", devices[0]);
        }
    }
    if (rc) {
        const std::string keep = ann_cuda_last_error();
        free_shards(s);
        delete s;
        return set_error("%s", keep.c_str());
    }
    *out = s;
    return 0;
}

void ann_cuda_sharded_free(ann_cuda_sharded_index *s) {
    if (!s) return;
    free_shards(s);
    delete s;
}

int ann_cuda_sharded_shard_count(const ann_cuda_sharded_index *s) { return s ? (int)s->shards.size() : -1; }

ann_cuda_index *ann_cuda_sharded_shard(const ann_cuda_sharded_index *s, int i) {
    if (!s || i < 0 || i >= (int)s->shards.size()) {
        set_error("no such shard");
        return nullptr;
    }
    return s->shards[(size_t)i].ix;
}

int64_t ann_cuda_sharded_ntotal(const ann_cuda_sharded_index *s) {
    if (!s) return -1;
    if (s->ivf) return ann_cuda_index_ntotal(s->shards[0].ix);  // every shard counts all rows (labels are global)
    return s->rows_before((int)s->shards.size());
}

int ann_cuda_sharded_add(ann_cuda_sharded_index *s, int64_t n, const float *x) {
    if (!s || n < 0 || (n > 0 && !x)) return set_error("invalid arguments");
    if (n == 0) return 0;
    std::lock_guard<std::mutex> lock(s->mu);
    const int G = (int)s->shards.size();
    if (s->ivf)  // every shard assigns all rows and keeps those of its own lists
        return s->on_every_shard([&](int g) { return ann_cuda_index_add(s->shards[(size_t)g].ix, n, x); });
    if (ann_cuda_sharded_ntotal(s) > 0)  // ranges stay contiguous: later rows go behind the last shard's
        return ann_cuda_index_add(s->shards[(size_t)G - 1].ix, n, x);
    // first add: equal contiguous ranges (they differ by at most one row)
    return s->on_every_shard([&](int g) {
        const int64_t base = n / G, rem = n % G;
        const int64_t begin = g * base + std::min<int64_t>(g, rem), cnt = base + (g < rem ? 1 : 0);
        return cnt > 0 ? ann_cuda_index_add(s->shards[(size_t)g].ix, cnt, x + begin * s->d) : 0;
    });
}

int ann_cuda_sharded_set_centroids(ann_cuda_sharded_index *s, const float *centroids) {
    if (!s || !s->ivf || !centroids) return set_error("invalid arguments");
    std::lock_guard<std::mutex> lock(s->mu);
    return s->on_every_shard([&](int g) { return ann_cuda_ivfflat_set_centroids(s->shards[(size_t)g].ix, centroids); });
}

int ann_cuda_sharded_train(ann_cuda_sharded_index *s, int64_t n, const float *x) {
    if (!s || !s->ivf || !x) return set_error("invalid arguments");
    std::vector<float> cent((size_t)s->nlist * s->d);
    {
        std::lock_guard<std::mutex> lock(s->mu);
        // k-means once, on the first shard; the other shards receive the same centroids
        if (ann_cuda_ivfflat_train(s->shards[0].ix, n, x) || ann_cuda_ivfflat_get_centroids(s->shards[0].ix, cent.data()))
            return -1;
    }
    return ann_cuda_sharded_set_centroids(s, cent.data());
}

int ann_cuda_sharded_add_list(ann_cuda_sharded_index *s, int64_t list_no, int64_t n, const int64_t *ids, const float *rows) {
    if (!s || !s->ivf) return set_error("invalid arguments");
    std::lock_guard<std::mutex> lock(s->mu);
    // the owner stores the rows, the others only advance their row count
    for (Shard &sh : s->shards)
        if (ann_cuda_ivfflat_add_list(sh.ix, list_no, n, ids, rows)) return -1;
    return 0;
}

int ann_cuda_sharded_set_nprobe(ann_cuda_sharded_index *s, int64_t nprobe) {
    if (!s || !s->ivf) return set_error("not an IVFFlat index");
    std::lock_guard<std::mutex> lock(s->mu);
    for (Shard &sh : s->shards)
        if (ann_cuda_ivfflat_set_nprobe(sh.ix, nprobe)) return -1;
    return 0;
}

int ann_cuda_sharded_reset(ann_cuda_sharded_index *s) {
    if (!s) return set_error("null index");
    std::lock_guard<std::mutex> lock(s->mu);
    for (Shard &sh : s->shards)
        if (ann_cuda_index_reset(sh.ix)) return -1;
    return 0;
}

int ann_cuda_sharded_reconstruct(const ann_cuda_sharded_index *s, int64_t key, float *recons) {
    if (!s || !recons) return set_error("invalid arguments");
    std::lock_guard<std::mutex> lock(s->mu);
    if (s->ivf) {  // the label may sit in any list: ask the shards in turn
        for (const Shard &sh : s->shards)
            if (ann_cuda_index_reconstruct(sh.ix, key, recons) == 0) return 0;
        return set_error("reconstruct: key %lld not found", (long long)key);
    }
    int64_t first = 0;
    for (const Shard &sh : s->shards) {
        const int64_t cnt = ann_cuda_index_ntotal(sh.ix);
        if (key >= first && key < first + cnt) return ann_cuda_index_reconstruct(sh.ix, key - first, recons);
        first += cnt;
    }
    return set_error("reconstruct: key %lld out of range", (long long)key);
}

int ann_cuda_sharded_get_rows(const ann_cuda_sharded_index *s, int64_t first, int64_t n, float *rows) {
    if (!s || s->ivf || !rows || first < 0 || n < 0) return set_error("invalid arguments");
    std::lock_guard<std::mutex> lock(s->mu);
    int64_t begin = 0;
    for (const Shard &sh : s->shards) {
        const int64_t cnt = ann_cuda_index_ntotal(sh.ix);
        const int64_t a = std::max(first, begin), b = std::min(first + n, begin + cnt);
        if (a < b && ann_cuda_flat_get_rows(sh.ix, a - begin, b - a, rows + (a - first) * s->d)) return -1;
        begin += cnt;
    }
    if (first + n > begin) return set_error("get_rows: range past the last row");
    return 0;
}

int ann_cuda_sharded_search(const ann_cuda_sharded_index *s, int64_t n, const float *x, int64_t k, float *distances,
                            int64_t *labels) {
    if (!s || n < 0 || (n > 0 && (!x || !distances || !labels))) return set_error("invalid arguments");
    if (k <= 0) return set_error("k must be > 0");
    if (n == 0) return 0;
    std::lock_guard<std::mutex> lock(s->mu);
    auto *ms = const_cast<ann_cuda_sharded_index *>(s);  // scratch buffers; guarded by mu
    const int G = (int)s->shards.size();
    const int mdev = s->merge_device();
    std::vector<int64_t> offset((size_t)G, 0);
    if (!s->ivf)
        for (int g = 0; g < G; g++) offset[(size_t)g] = s->rows_before(g);
    for (int64_t q0 = 0; q0 < n; q0 += kShardQueryBlock) {
        const int64_t nb = std::min(kShardQueryBlock, n - q0);
        const size_t part_d = (size_t)nb * k * 4, part_i = (size_t)nb * k * 8;
        {
            DeviceGuard guard(mdev);
            if (ms->parts_d.ensure(part_d * G) || ms->parts_i.ensure(part_i * G) || ms->merged_d.ensure(part_d) ||
                ms->merged_i.ensure(part_i))
                return -1;
        }
        // every shard, on its own thread and stream: queries in, local search, results over to the merging GPU
        const int rc = s->on_every_shard([&](int g) {
            Shard &sh = ms->shards[(size_t)g];
            DeviceGuard guard(sh.device);
            if (!guard.ok) return set_error("cudaSetDevice(%d) failed", sh.device);
            if (sh.xq.ensure((size_t)nb * s->d * 4) || sh.out_d.ensure(part_d) || sh.out_i.ensure(part_i)) return -1;
            ANN_CUDA_TRY(cudaMemcpyAsync(sh.xq.ptr, x + q0 * s->d, (size_t)nb * s->d * 4, cudaMemcpyHostToDevice, sh.stream));
            if (ann_cuda_index_search_device(sh.ix, nb, sh.xq.as<float>(), k, sh.out_d.as<float>(), sh.out_i.as<int64_t>(),
                                             offset[(size_t)g], sh.stream))
                return -1;
            ANN_CUDA_TRY(cudaMemcpyPeerAsync(static_cast<char *>(ms->parts_d.ptr) + part_d * g, mdev, sh.out_d.ptr, sh.device,
                                             part_d, sh.stream));
            ANN_CUDA_TRY(cudaMemcpyPeerAsync(static_cast<char *>(ms->parts_i.ptr) + part_i * g, mdev, sh.out_i.ptr, sh.device,
                                             part_i, sh.stream));
            ANN_CUDA_TRY(cudaEventRecord(sh.done, sh.stream));
            return 0;
        });
        if (rc) return -1;
        {
            DeviceGuard guard(mdev);
            for (const Shard &sh : s->shards) ANN_CUDA_TRY(cudaStreamWaitEvent(ms->merge_stream, sh.done, 0));
            const float *res_d = ms->parts_d.as<float>();
            const int64_t *res_i = ms->parts_i.as<int64_t>();
            if (G > 1) {
                if (ann_cuda_merge_topk_device(mdev, ms->parts_d.as<float>(), ms->parts_i.as<int64_t>(), G, nb, k, s->metric,
                                               ms->merged_d.as<float>(), ms->merged_i.as<int64_t>(), ms->merge_stream))
                    return -1;
                res_d = ms->merged_d.as<float>();
                res_i = ms->merged_i.as<int64_t>();
            }
            ANN_CUDA_TRY(cudaMemcpyAsync(distances + q0 * k, res_d, part_d, cudaMemcpyDeviceToHost, ms->merge_stream));
            ANN_CUDA_TRY(cudaMemcpyAsync(labels + q0 * k, res_i, part_i, cudaMemcpyDeviceToHost, ms->merge_stream));
            ANN_CUDA_TRY(cudaStreamSynchronize(ms->merge_stream));
        }
        // a shard whose kernel gave up on a bounded wait fails the whole search
        for (const Shard &sh : s->shards)
            if (ann_cuda_index_search_status(sh.ix, sh.stream)) return -1;
    }
    return 0;
}

}  // extern "C"
