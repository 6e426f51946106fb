// slice_batch.cpp — forming per-GPU batches out of independent units (audio slices, decode streams).
//
// The reference processes one slice per operator call (CrispasrBackend::encode_slice / decode_slice,
// examples/cli/crispasr_backend.h:181-230; the producer/consumer pipeline of examples/cli/crispasr_run.cpp:1765-1881
// keeps at most two slices in flight) and pads to buckets with a -inf mask when lengths differ
// (src/canary_ctc.cpp:370-382).  On a B200 a one-slice launch leaves most SMs idle (a one-segment decode step runs at
// under a fifth of the memory roofline that 64 segments per launch reach), so the units of one GPU share launches:
// they are concatenated on the batch dimension ne[3], and a per-unit (q_len, kv_len) table - ext->q_len / ext->kv_len
// of the operator - replaces the padding mask, so padding costs neither arithmetic nor memory traffic.
//
// Two pieces:
//  * b200_batch_pack: orders pending units by length and cuts them into launches (at most max_units each, and no
//    unit shorter than (1 - max_pad) of the longest in its launch), which bounds the padded size of the operand
//    buffers the caller has to provide.
//  * b200_batch: the slot table of a resident batch (decode streams come and go, caches grow by one row per step):
//    host arrays in pinned memory, mirrored to the device with one asynchronous copy when they changed.
#include <algorithm>
#include <cstring>
#include <new>
#include <numeric>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/b200_fattn.h"

struct b200_batch {
    int capacity = 0;
    bool has_device = false;
    int device = -1;
    int32_t* h_tab = nullptr;   // [2][capacity]: q_len, kv_len (pinned when a device is present)
    int32_t* d_tab = nullptr;   // device mirror
    std::vector<int> unit;      // unit id per slot, -1 = free
    int n_active = 0;
    bool dirty = true;
};

extern "C" {

B200_API int b200_batch_pack(const int32_t* q_len, const int32_t* kv_len, int n_units, int max_units, float max_pad,
                             int32_t* order, int32_t* group_end, int* n_groups) {
    if (!q_len || !kv_len || !order || !group_end || !n_groups) return B200_E_NULL;
    if (n_units < 0 || max_units <= 0 || !(max_pad >= 0.0f) || max_pad > 1.0f) return B200_E_SHAPE;
    for (int i = 0; i < n_units; i++)
        if (q_len[i] < 0 || kv_len[i] < 0) return B200_E_SHAPE;
    std::iota(order, order + n_units, 0);
    // longest first; ties by the other length, then by index so the result is reproducible
    std::stable_sort(order, order + n_units, [&](int32_t x, int32_t y) {
        if (kv_len[x] != kv_len[y]) return kv_len[x] > kv_len[y];
        return q_len[x] > q_len[y];
    });
    int g = 0, start = 0;
    for (int i = 0; i <= n_units; i++) {
        bool cut = i == n_units || i - start == max_units;
        if (!cut && i > start) {
            // the group's padded extents are those of its first (longest) unit
            const float kv0 = (float)kv_len[order[start]];
            int qmax = q_len[order[i]], qmin = q_len[order[i]];   // with the candidate included
            for (int j = start; j < i; j++) qmax = std::max(qmax, (int)q_len[order[j]]), qmin = std::min(qmin, (int)q_len[order[j]]);
            if ((float)kv_len[order[i]] < (1.0f - max_pad) * kv0) cut = true;
            if ((float)qmin < (1.0f - max_pad) * (float)qmax) cut = true;
        }
        if (cut && i > start) {
            group_end[g++] = i;
            start = i;
        }
    }
    *n_groups = g;
    return B200_OK;
}

B200_API int b200_batch_create(int capacity, b200_batch** out) {
    if (!out) return B200_E_NULL;
    *out = nullptr;
    if (capacity <= 0 || capacity > 65535) return B200_E_SHAPE;
    b200_batch* b = new (std::nothrow) b200_batch();
    if (!b) return B200_E_STATE;
    b->capacity = capacity;
    b->unit.assign(capacity, -1);
    int count = 0;
    const size_t bytes = (size_t)2 * capacity * sizeof(int32_t);
    if (cudaGetDeviceCount(&count) == cudaSuccess && count > 0 && cudaGetDevice(&b->device) == cudaSuccess &&
        cudaMallocHost((void**)&b->h_tab, bytes) == cudaSuccess) {
        if (cudaMalloc((void**)&b->d_tab, bytes) != cudaSuccess) {
            cudaGetLastError();
            cudaFreeHost(b->h_tab);
            delete b;
            return B200_E_CUDA;
        }
        b->has_device = true;
    } else {
        cudaGetLastError();   // host-only table (no GPU): everything but b200_batch_tables works
        b->h_tab = new (std::nothrow) int32_t[2 * (size_t)capacity];
        if (!b->h_tab) {
            delete b;
            return B200_E_STATE;
        }
    }
    memset(b->h_tab, 0, bytes);
    *out = b;
    return B200_OK;
}

B200_API void b200_batch_destroy(b200_batch* b) {
    if (!b) return;
    if (b->has_device) {
        cudaFree(b->d_tab);
        cudaFreeHost(b->h_tab);
    } else {
        delete[] b->h_tab;
    }
    delete b;
}

B200_API int b200_batch_add(b200_batch* b, int unit_id, int q_len, int kv_len) {
    if (!b) return B200_E_NULL;
    if (unit_id < 0 || q_len < 0 || kv_len < 0) return B200_E_SHAPE;
    for (int s = 0; s < b->capacity; s++) {
        if (b->unit[s] >= 0) continue;
        b->unit[s] = unit_id;
        b->h_tab[s] = q_len, b->h_tab[b->capacity + s] = kv_len;
        b->n_active++;
        b->dirty = true;
        return s;   // the lowest free slot: launches stay as narrow as the live units allow
    }
    return B200_E_LIMIT;
}

B200_API int b200_batch_set(b200_batch* b, int slot, int q_len, int kv_len) {
    if (!b) return B200_E_NULL;
    if (slot < 0 || slot >= b->capacity || q_len < 0 || kv_len < 0) return B200_E_SHAPE;
    if (b->unit[slot] < 0) return B200_E_STATE;
    b->h_tab[slot] = q_len, b->h_tab[b->capacity + slot] = kv_len;
    b->dirty = true;
    return B200_OK;
}

B200_API int b200_batch_advance(b200_batch* b, int kv_delta) {
    if (!b) return B200_E_NULL;
    for (int s = 0; s < b->capacity; s++)
        if (b->unit[s] >= 0) b->h_tab[b->capacity + s] = std::max(0, b->h_tab[b->capacity + s] + kv_delta);
    b->dirty = true;
    return B200_OK;
}

B200_API int b200_batch_remove(b200_batch* b, int slot) {
    if (!b) return B200_E_NULL;
    if (slot < 0 || slot >= b->capacity) return B200_E_SHAPE;
    if (b->unit[slot] < 0) return B200_E_STATE;
    b->unit[slot] = -1;
    b->h_tab[slot] = 0, b->h_tab[b->capacity + slot] = 0;   // a free slot inside the span costs nothing: zero rows, zero keys
    b->n_active--;
    b->dirty = true;
    return B200_OK;
}

B200_API int b200_batch_span(const b200_batch* b, int* n_slots, int* n_active, int* max_q_len, int* max_kv_len) {
    if (!b) return B200_E_NULL;
    int span = 0, mq = 0, mk = 0;
    for (int s = 0; s < b->capacity; s++)
        if (b->unit[s] >= 0) {
            span = s + 1;
            mq = std::max(mq, (int)b->h_tab[s]);
            mk = std::max(mk, (int)b->h_tab[b->capacity + s]);
        }
    if (n_slots) *n_slots = span;
    if (n_active) *n_active = b->n_active;
    if (max_q_len) *max_q_len = mq;
    if (max_kv_len) *max_kv_len = mk;
    return B200_OK;
}

B200_API int b200_batch_unit(const b200_batch* b, int slot) {
    if (!b || slot < 0 || slot >= b->capacity) return -1;
    return b->unit[slot];
}

B200_API int b200_batch_lengths(const b200_batch* b, int slot, int* q_len, int* kv_len) {
    if (!b) return B200_E_NULL;
    if (slot < 0 || slot >= b->capacity) return B200_E_SHAPE;
    if (q_len) *q_len = b->h_tab[slot];
    if (kv_len) *kv_len = b->h_tab[b->capacity + slot];
    return B200_OK;
}

B200_API int b200_batch_tables(b200_batch* b, void* cuda_stream, const int32_t** q_len_dev, const int32_t** kv_len_dev) {
    if (!b || !q_len_dev || !kv_len_dev) return B200_E_NULL;
    if (!b->has_device) return B200_E_NO_DEVICE;
    if (b->dirty) {
        // one copy of both tables; the pinned source may be edited again only after the stream has passed this point
        // (the callers' pattern - edit between steps, launch, synchronise or record an event per step - does that)
        if (cudaMemcpyAsync(b->d_tab, b->h_tab, (size_t)2 * b->capacity * sizeof(int32_t), cudaMemcpyHostToDevice,
                            (cudaStream_t)cuda_stream) != cudaSuccess) {
            cudaGetLastError();
            return B200_E_CUDA;
        }
        b->dirty = false;
    }
    *q_len_dev = b->d_tab;
    *kv_len_dev = b->d_tab + b->capacity;
    return B200_OK;
}

}  // extern "C"
