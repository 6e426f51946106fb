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

B200_API int b200_sched_run(b200_sched* s, int n_units, b200_unit_fn fn, void* user, int* unit_device) {
    if (!s || !fn) return B200_E_NULL;
    if (n_units < 0) return B200_E_SHAPE;
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
    std::deque<std::pair<int, int>> retry;  // (unit, worker that failed it)

    auto next_fresh = [&](int w) -> int {
        for (int k = 0; k < W; k++) {  // own range first, then victims in ring order
            const int v = (w + k) % W;
            if (cursor[v].load(std::memory_order_relaxed) >= range_end[v]) continue;
            const int u = cursor[v].fetch_add(1);
            if (u < range_end[v]) return u;
        }
        return -1;
    };

    auto worker = [&](int w) {
        const int dev = s->host_only ? -1 : s->devices[w];
        if (!s->host_only && cudaSetDevice(dev) != cudaSuccess) {
            // this worker cannot run; the others steal its range
            cuda_error.store(1);
            cudaGetLastError();
            alive.fetch_sub(1);
            return;
        }
        while (outstanding.load() > 0) {
            int unit = next_fresh(w);
            bool is_retry = false;
            if (unit < 0) {
                std::lock_guard<std::mutex> lk(mu);
                for (auto it = retry.begin(); it != retry.end(); ++it) {
                    if (it->second != w || alive.load() == 1) {
                        unit = it->first;
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
            const int rc = fn(user, dev, unit, (void*)s->streams[w]);
            if (rc == 0) {
                done_by[unit] = w;
                outstanding.fetch_sub(1);
            } else if (!is_retry) {
                std::lock_guard<std::mutex> lk(mu);
                retry.emplace_back(unit, w);
            } else {
                failed.fetch_add(1);
                outstanding.fetch_sub(1);
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
