// segment_sched.cpp — collective-free scheduler that spreads independent work units (audio
// segments, beam groups, decode streams, utterances) over the GPUs of one box.
//
// One host worker thread per device, each with its own CUDA stream.  Units are first split into
// contiguous ranges (b200_sched_partition); a worker that drains its range steals from the others
// through their atomic cursors — the same shape as the reference's `-p N` loop with its shared
// atomic next-slice counter.  A unit whose callback fails is queued once more for a different
// worker; a second failure marks it failed.  Nothing here exchanges data between devices.
#include <atomic>
#include <chrono>
#include <deque>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/b200_fattn.h"

struct b200_sched {
    std::vector<int> devices;          // empty in host-only mode
    std::vector<cudaStream_t> streams;  // one per worker (null in host-only mode)
    int n_workers = 0;
    bool host_only = false;
};

extern "C" {

B200_API void b200_sched_partition(int n_units, int n_workers, int w, int* first, int* count) {
    if (n_workers <= 0 || w < 0 || w >= n_workers || n_units < 0) {
        if (first) *first = 0;
        if (count) *count = 0;
        return;
    }
    const int base = n_units / n_workers, rem = n_units % n_workers;
    const int f = w * base + (w < rem ? w : rem);
    if (first) *first = f;
    if (count) *count = base + (w < rem ? 1 : 0);
}

B200_API int b200_sched_create(const int* devices, int n_devices, int n_host_workers, b200_sched** out) {
    if (!out) return B200_E_NULL;
    *out = nullptr;
    if (n_devices < 0 || (n_devices == 0 && n_host_workers <= 0)) return B200_E_SHAPE;
    b200_sched* s = new (std::nothrow) b200_sched();
    if (!s) return B200_E_STATE;
    if (n_devices == 0) {
        s->host_only = true;
        s->n_workers = n_host_workers;
        s->streams.assign(n_host_workers, nullptr);
        *out = s;
        return B200_OK;
    }
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess || visible <= 0) {
        cudaGetLastError();
        delete s;
        return B200_E_NO_DEVICE;
    }
    int prev = 0;
    cudaGetDevice(&prev);
    for (int i = 0; i < n_devices; i++) {
        const int d = devices ? devices[i] : i;
        if (d < 0 || d >= visible) {
            for (size_t j = 0; j < s->streams.size(); j++) {
                cudaSetDevice(s->devices[j]);
                cudaStreamDestroy(s->streams[j]);
            }
            cudaSetDevice(prev);
            delete s;
            return B200_E_NO_DEVICE;
        }
        cudaStream_t st = nullptr;
        if (cudaSetDevice(d) != cudaSuccess || cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
            cudaGetLastError();
            cudaSetDevice(prev);
            delete s;
            return B200_E_CUDA;
        }
        s->devices.push_back(d);
        s->streams.push_back(st);
    }
    cudaSetDevice(prev);
    s->n_workers = n_devices;
    *out = s;
    return B200_OK;
}

B200_API void b200_sched_destroy(b200_sched* s) {
    if (!s) return;
    if (!s->host_only) {
        int prev = 0;
        cudaGetDevice(&prev);
        for (size_t i = 0; i < s->streams.size(); i++) {
            cudaSetDevice(s->devices[i]);
            cudaStreamDestroy(s->streams[i]);
        }
        cudaSetDevice(prev);
    }
    delete s;
}

namespace {
struct UnitAsBatch {
    b200_unit_fn fn;
    void* user;
};
int unit_as_batch(void* user, int device, int first_unit, int n_units, void* cuda_stream) {
    (void)n_units;   // always 1: b200_sched_run hands out single units
    UnitAsBatch* u = (UnitAsBatch*)user;
    return u->fn(u->user, device, first_unit, cuda_stream);
}
}  // namespace

B200_API int b200_sched_run(b200_sched* s, int n_units, b200_unit_fn fn, void* user, int* unit_device) {
    if (!s || !fn) return B200_E_NULL;
    UnitAsBatch u{fn, user};
    return b200_sched_run_batched(s, n_units, 1, 1, unit_as_batch, &u, unit_device);
}

B200_API int b200_sched_run_batched(b200_sched* s, int n_units, int max_batch, int steal, b200_batch_fn fn, void* user,
                                    int* unit_device) {
    if (!s || !fn) return B200_E_NULL;
    if (n_units < 0 || max_batch < 1) return B200_E_SHAPE;
    const int W = s->n_workers;
    std::vector<std::atomic<int>> cursor(W);
    std::vector<int> range_end(W);
    for (int w = 0; w < W; w++) {
        int f = 0, c = 0;
        b200_sched_partition(n_units, W, w, &f, &c);
        cursor[w].store(f);
        range_end[w] = f + c;
    }
    std::vector<int> done_by(n_units, -1);
    std::atomic<int> outstanding(n_units), failed(0), cuda_error(0), alive(W);
    std::mutex mu;
    struct Run {
        int first, count, failed_by;
    };
    std::deque<Run> retry;  // runs whose callback failed once, with the worker that failed them
    std::vector<std::atomic<int>> dead(W);   // workers that could not bind their device
    for (int w = 0; w < W; w++) dead[w].store(0);

    // A run of up to max_batch consecutive units: from the worker's own range first, then (if stealing is on) from
    // the other ranges in ring order.  A run never crosses a range border, so what a worker is handed is always a
    // contiguous slice of one static share.
    auto next_fresh = [&](int w, int* count) -> int {
        for (int k = 0; k < W; k++) {
            const int v = (w + k) % W;
            if (k > 0 && !steal && !dead[v].load(std::memory_order_relaxed)) continue;   // a dead worker's share is always up for grabs
            if (cursor[v].load(std::memory_order_relaxed) >= range_end[v]) continue;
            const int u = cursor[v].fetch_add(max_batch);
            if (u < range_end[v]) {
                *count = range_end[v] - u < max_batch ? range_end[v] - u : max_batch;
                return u;
            }
        }
        return -1;
    };

    auto worker = [&](int w) {
        const int dev = s->host_only ? -1 : s->devices[w];
        if (!s->host_only && cudaSetDevice(dev) != cudaSuccess) {
            // this worker cannot run; the others steal its range
            cuda_error.store(1);
            cudaGetLastError();
            dead[w].store(1);
            alive.fetch_sub(1);
            return;
        }
        while (outstanding.load() > 0) {
            int count = 0;
            int unit = next_fresh(w, &count);
            bool is_retry = false;
            if (unit < 0) {
                std::lock_guard<std::mutex> lk(mu);
                for (auto it = retry.begin(); it != retry.end(); ++it) {
                    if (it->failed_by != w || alive.load() == 1) {
                        unit = it->first, count = it->count;
                        retry.erase(it);
                        is_retry = true;
                        break;
                    }
                }
            }
            if (unit < 0) {
                std::this_thread::sleep_for(std::chrono::microseconds(50));
                continue;
            }
            const int rc = fn(user, dev, unit, count, (void*)s->streams[w]);
            if (rc == 0) {
                for (int u = unit; u < unit + count; u++) done_by[u] = w;
                outstanding.fetch_sub(count);
            } else if (!is_retry) {
                std::lock_guard<std::mutex> lk(mu);
                retry.push_back(Run{unit, count, w});
            } else {
                failed.fetch_add(count);
                outstanding.fetch_sub(count);
            }
        }
        if (!s->host_only && cudaStreamSynchronize(s->streams[w]) != cudaSuccess) {
            cuda_error.store(1);
            cudaGetLastError();
        }
    };

    std::vector<std::thread> threads;
    threads.reserve(W);
    for (int w = 0; w < W; w++) threads.emplace_back(worker, w);
    for (auto& t : threads) t.join();
    if (unit_device)
        for (int u = 0; u < n_units; u++) unit_device[u] = done_by[u];
    if (cuda_error.load()) return B200_E_CUDA;
    return failed.load();
}

}  // extern "C"
