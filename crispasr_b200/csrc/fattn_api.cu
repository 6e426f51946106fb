// fattn_api.cu — the C-ABI of include/b200_fattn.h for the attention operator: operand
// validation (ggml shape rules, returned as codes, never asserts), kernel choice, workspace
// sizing, launch, and the host-buffer round trip.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "fattn_common.cuh"
#include "fattn_tc5.cuh"

namespace b200 {

namespace {

thread_local char g_cuda_err[256] = "";
thread_local int g_last_kernel = B200_KERNEL_NONE;
std::atomic<int> g_override{B200_KERNEL_NONE};   // process-wide A/B knob, read once per plan

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
    return B200_E_CUDA;
}

struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    bool ok = false;
};

// Properties of the current device, cached per device ordinal.
int device_info(DeviceInfo* out) {
    static std::mutex mu;
    static DeviceInfo cache[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaGetDevice");
        return B200_E_NO_DEVICE;
    }
    if (dev < 0 || dev >= 64) return B200_E_NO_DEVICE;
    std::lock_guard<std::mutex> lk(mu);
    if (!cache[dev].ok) {
        int sm = 0, major = 0;
        if ((e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
            (e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) {
            cuda_fail(e, "cudaDeviceGetAttribute");
            return B200_E_NO_DEVICE;
        }
        cache[dev].sm_count = sm;
        cache[dev].cc_major = major;
        cache[dev].ok = true;
    }
    *out = cache[dev];
    return out->cc_major == 10 ? B200_OK : B200_E_NO_DEVICE;
}

size_t type_size(int t) {
    switch (t) {
        case B200_TYPE_F32: return 4;
        case B200_TYPE_F16: return 2;
        case B200_TYPE_Q8_0: return 34;
        default: return 0;
    }
}

bool is_vec16(const b200_tensor* t) {
    return ((uintptr_t)t->data % 16 == 0) && t->nb[1] % 16 == 0 && t->nb[2] % 16 == 0 && t->nb[3] % 16 == 0;
}

View make_view(const b200_tensor* t) {
    View v;
    v.p = (const uint8_t*)t->data;
    v.nb1 = (int64_t)t->nb[1];
    v.nb2 = (int64_t)t->nb[2];
    v.nb3 = (int64_t)t->nb[3];
    v.type = t->type;
    v.vec16 = is_vec16(t) ? 1 : 0;
    return v;
}

// Type, nb[0], alignment and stride-granularity rules of one operand.
int check_operand(const b200_tensor* t, bool allow_f32, bool allow_f16, bool allow_q8) {
    if (!t->data) return B200_E_NULL;
    const size_t es = type_size(t->type);
    if (es == 0) return B200_E_TYPE;
    if (t->type == B200_TYPE_F32 && !allow_f32) return B200_E_TYPE;
    if (t->type == B200_TYPE_F16 && !allow_f16) return B200_E_TYPE;
    if (t->type == B200_TYPE_Q8_0 && !allow_q8) return B200_E_TYPE;
    if (t->nb[0] != es) return B200_E_STRIDE;
    const size_t align = t->type == B200_TYPE_F32 ? 4 : 2;
    if ((uintptr_t)t->data % align) return B200_E_ALIGN;
    for (int i = 1; i < 4; i++)
        if (t->nb[i] % align) return B200_E_STRIDE;
    for (int i = 0; i < 4; i++)
        if (t->ne[i] <= 0) return B200_E_SHAPE;
    if (t->type == B200_TYPE_Q8_0 && t->ne[0] % 32) return B200_E_SHAPE;
    return B200_OK;
}

struct Plan {
    FattnArgs args;
    int kernel;
    size_t ws_bytes;
    bool cast_kv;      // K/V are first converted to contiguous F16 in the workspace (prefill on the tcgen05 kernel)
    bool cast_r;       // the same for the rel-pos table R
    size_t cast_each;  // bytes of one converted K or V tensor, rounded up to 256
    size_t cast_r_bytes;
};

bool kv_is_tma_ready(const FattnArgs& a) {
    return a.k.type == B200_TYPE_F16 && a.v.type == B200_TYPE_F16 && a.k.vec16 && a.v.vec16;
}
bool r_is_tma_ready(const FattnArgs& a) { return !a.relpos || (a.r.type == B200_TYPE_F16 && a.r.vec16); }

FattnArgs with_f16_r(const FattnArgs& a, const void* rbuf) {
    FattnArgs c = a;
    c.r.p = (const uint8_t*)rbuf;
    c.r.type = B200_TYPE_F16;
    c.r.nb1 = (int64_t)a.hd * 2;
    c.r.nb2 = c.r.nb1 * (2 * a.Tq - 1);
    c.r.nb3 = c.r.nb2 * a.H;
    c.r.vec16 = 1;
    return c;
}

// The operand block as the tcgen05 kernel would see it after K/V have been converted to contiguous F16.
FattnArgs with_f16_kv(const FattnArgs& a, const void* kbuf, const void* vbuf) {
    FattnArgs c = a;
    const int Bk = a.B / a.bq;
    (void)Bk;
    for (int which = 0; which < 2; which++) {
        View& v = which ? c.v : c.k;
        v.p = (const uint8_t*)(which ? vbuf : kbuf);
        v.type = B200_TYPE_F16;
        v.nb1 = (int64_t)a.hd * 2;
        v.nb2 = v.nb1 * a.Lk;
        v.nb3 = v.nb2 * a.Hkv;
        v.vec16 = 1;
    }
    return c;
}

// Validates the operands against the op contract and fills the kernel argument block.
// `need_device` = false keeps the call free of CUDA (supports / plan on a CPU-only host assume 148 SMs).
int make_plan(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v, const b200_tensor* mask,
              const b200_tensor* dst, const b200_fattn_params* p, const b200_fattn_ext* ext, bool need_device,
              Plan* plan) {
    if (!q || !k || !v || !dst || !p) return B200_E_NULL;
    int rc;
    if ((rc = check_operand(q, true, true, false))) return rc;
    if ((rc = check_operand(k, true, true, true))) return rc;
    if ((rc = check_operand(v, true, true, true))) return rc;
    if ((rc = check_operand(dst, true, false, false))) return rc;
    if (k->type != v->type) return B200_E_TYPE;

    const int64_t hd = q->ne[0], Tq = q->ne[1], H = q->ne[2], B = q->ne[3];
    const int64_t Lk = k->ne[1], Hkv = k->ne[2], Bk = k->ne[3];
    if (k->ne[0] != hd || v->ne[0] != hd) return v->ne[0] != hd && k->ne[0] == hd ? B200_E_UNSUPPORTED : B200_E_SHAPE;
    if (v->ne[1] != Lk || v->ne[2] != Hkv || v->ne[3] != Bk) return B200_E_SHAPE;
    if (H % Hkv || B % Bk) return B200_E_SHAPE;
    if (dst->ne[0] != hd || dst->ne[1] != H || dst->ne[2] != Tq || dst->ne[3] != B) return B200_E_SHAPE;
    if (dst->nb[1] != (uint64_t)hd * 4 || dst->nb[2] != (uint64_t)hd * H * 4 ||
        dst->nb[3] != (uint64_t)hd * H * Tq * 4)
        return B200_E_STRIDE;
    // output rows are written with 128-bit stores where the row length allows it (head_dim 64 / 128 on the
    // tensor-core kernels), so the base must be 16-byte aligned for those head dims
    if ((hd == 64 || hd == 128) && (uintptr_t)dst->data % 16) return B200_E_ALIGN;
    if (hd > 128) return B200_E_UNSUPPORTED;
    if (Tq > INT32_MAX / 2 || Lk > INT32_MAX / 2 || H > 65535 || B > 65535) return B200_E_LIMIT;
    if (!std::isfinite(p->scale) || !std::isfinite(p->max_bias) || !std::isfinite(p->logit_softcap))
        return B200_E_SHAPE;

    FattnArgs& a = plan->args;
    memset(&a, 0, sizeof(a));
    if (mask) {
        if ((rc = check_operand(mask, false, true, false))) return rc;
        // one mask value per logical key: the rows of K, or the entries of the index lists when keys are gathered
        const int64_t n_logical = (ext && ext->kv_index) ? ext->kv_index_stride : Lk;
        if (mask->ne[0] != n_logical || mask->ne[1] < Tq) return B200_E_SHAPE;
        if (mask->ne[2] != 1 && mask->ne[2] != H) return B200_E_SHAPE;
        if (mask->ne[3] != 1 && mask->ne[3] != B) return B200_E_SHAPE;
        a.mask = make_view(mask);
        a.mask_ne2 = (int)mask->ne[2];
        a.mask_ne3 = (int)mask->ne[3];
        a.has_mask = 1;
    } else {
        a.mask_ne2 = a.mask_ne3 = 1;
    }
    a.q = make_view(q);
    a.k = make_view(k);
    a.v = make_view(v);
    a.dst = (float*)dst->data;
    a.hd = (int)hd, a.Tq = (int)Tq, a.H = (int)H, a.B = (int)B;
    a.Lk = (int)Lk, a.Hkv = (int)Hkv, a.gqa = (int)(H / Hkv), a.bq = (int)(B / Bk);
    a.relscale = p->scale;
    a.softcap = p->logit_softcap;
    a.scale = p->logit_softcap != 0.0f ? p->scale / p->logit_softcap : p->scale;
    if (p->max_bias > 0.0f) {
        a.n2 = 1 << (int)floorf(log2f((float)H));
        a.m0 = powf(2.0f, -p->max_bias / (float)a.n2);
        a.m1 = powf(2.0f, -(p->max_bias / 2.0f) / (float)a.n2);
    }
    if (ext) {
        const bool fused_bias = ext->pos_bias_u != nullptr || ext->pos_bias_v != nullptr;
        if (fused_bias && (!ext->pos_bias_u || !ext->pos_bias_v || ext->q_v || !ext->r)) return B200_E_NULL;
        if (!fused_bias && (ext->q_v != nullptr) != (ext->r != nullptr)) return B200_E_NULL;
        if (ext->r) {
            const b200_tensor *qv = fused_bias ? q : ext->q_v, *r = ext->r;
            if ((rc = check_operand(qv, true, true, false))) return rc;
            if ((rc = check_operand(r, true, true, false))) return rc;
            for (int i = 0; i < 4; i++)
                if (qv->ne[i] != q->ne[i]) return B200_E_SHAPE;
            if (Lk != Tq) return B200_E_SHAPE;
            if (r->ne[0] != hd || r->ne[1] != 2 * Tq - 1 || r->ne[2] != H) return B200_E_SHAPE;
            if (r->ne[3] != 1 && r->ne[3] != B) return B200_E_SHAPE;
            if (fused_bias) {
                const b200_tensor* bb[2] = {ext->pos_bias_u, ext->pos_bias_v};
                for (int i = 0; i < 2; i++) {
                    if (!bb[i]->data) return B200_E_NULL;
                    if (bb[i]->type != B200_TYPE_F32) return B200_E_TYPE;
                    if (bb[i]->ne[0] != hd || bb[i]->ne[1] != H || bb[i]->ne[2] != 1 || bb[i]->ne[3] != 1) return B200_E_SHAPE;
                    if (bb[i]->nb[0] != 4 || bb[i]->nb[1] != (uint64_t)hd * 4) return B200_E_STRIDE;
                    if (((uintptr_t)bb[i]->data & 3) != 0) return B200_E_ALIGN;
                }
                a.bias_u = (const float*)ext->pos_bias_u->data;
                a.bias_v = (const float*)ext->pos_bias_v->data;
            }
            a.qv = make_view(qv);
            a.r = make_view(r);
            a.r_ne3 = (int)r->ne[3];
            a.relpos = 1;
            a.relpos_f32 = ext->relpos_bias_f32 ? 1 : 0;
        }
        a.causal = ext->causal ? 1 : 0;
        a.n_past = ext->n_past;
        a.kv_len = ext->kv_len;
        a.q_len = ext->q_len;
        if (ext->kv_index) {
            if (!ext->kv_len) return B200_E_NULL;   // the lists' lengths
            if (ext->kv_index_stride <= 0 || ext->kv_index_stride > INT32_MAX / 2) return B200_E_SHAPE;
            if ((uintptr_t)ext->kv_index % 4) return B200_E_ALIGN;
            a.kv_index = ext->kv_index;
            a.kv_index_stride = ext->kv_index_stride;
        }
    }

    int sm_count = 148;
    if (need_device) {
        DeviceInfo di;
        if ((rc = device_info(&di))) return rc;
        sm_count = di.sm_count;
    }

    // kernel choice
    int kernel = B200_KERNEL_TILE_MMA;
    const bool decode_ok = !a.relpos && Tq * (H / Hkv) <= 16;
    // index lists: the decode kernel only; a mask must be one the F16 ring can stage (16-byte aligned rows, no ALiBi)
    if (a.kv_index && (!decode_ok || a.causal || a.softcap != 0.0f || a.q_len || (a.has_mask && (!a.mask.vec16 || a.n2 != 0))))
        return B200_E_UNSUPPORTED;
    if (a.kv_index && a.has_mask && (a.k.type != B200_TYPE_F16 || !a.k.vec16 || !a.v.vec16 || (a.hd != 32 && a.hd != 64 && a.hd != 128)))
        return B200_E_UNSUPPORTED;
    const bool tc5_ok = tc5_supported(a);
    const int override_k = g_override.load(std::memory_order_relaxed);
    if (decode_ok) kernel = B200_KERNEL_DECODE_SPLIT;
    else if (tc5_ok) kernel = B200_KERNEL_PREFILL_TC5;
    if (override_k == B200_KERNEL_TILE_MMA && !a.kv_index) kernel = B200_KERNEL_TILE_MMA;   // index lists exist in the decode kernel only
    if (override_k == B200_KERNEL_DECODE_SPLIT && decode_ok) kernel = B200_KERNEL_DECODE_SPLIT;
    if (override_k == B200_KERNEL_PREFILL_TC5 && tc5_ok) kernel = B200_KERNEL_PREFILL_TC5;
    plan->cast_kv = plan->cast_r = false;
    plan->cast_each = plan->cast_r_bytes = 0;
    if (kernel == B200_KERNEL_TILE_MMA && override_k != B200_KERNEL_TILE_MMA && !decode_ok && (a.hd == 64 || a.hd == 128) &&
        !tc5_ok) {
        // F32 / Q8_0 / unaligned K/V: a conversion pre-pass into the workspace puts the call on the tcgen05 kernel
        FattnArgs c = kv_is_tma_ready(a) ? a : with_f16_kv(a, (const void*)256, (const void*)256);
        if (!r_is_tma_ready(a)) c = with_f16_r(c, (const void*)256);
        if (tc5_supported(c)) {
            kernel = B200_KERNEL_PREFILL_TC5;
            plan->cast_kv = !kv_is_tma_ready(a);
            plan->cast_r = !r_is_tma_ready(a);
            if (plan->cast_kv) plan->cast_each = ((size_t)a.hd * 2 * a.Lk * a.Hkv * (a.B / a.bq) + 255) / 256 * 256;
            if (plan->cast_r) plan->cast_r_bytes = ((size_t)a.hd * 2 * (2 * a.Tq - 1) * a.H * a.r_ne3 + 255) / 256 * 256;
        }
    }
    plan->kernel = kernel;
    a.n_splits = 1;
    plan->ws_bytes = 2 * plan->cast_each + plan->cast_r_bytes;
    if (kernel == B200_KERNEL_DECODE_SPLIT) {
        a.n_splits = decode_split_choose(a, a.B, sm_count);
        // splits that merge inside thread-block clusters never touch a workspace
        plan->ws_bytes = decode_uses_cluster_merge(a) ? 0 : decode_split_ws_bytes(a.B, a.Hkv, a.n_splits, a.hd);
    }
    return B200_OK;
}

// ---- per-launch tracing: an NVTX range around the enqueue and a CUDA event pair around the kernels ----
// Off by default.  b200_trace_enable(n) creates a ring of n event pairs on the current device up front, so a traced
// launch allocates nothing; launches on other devices, and launches made while a stream is being captured into a
// CUDA graph, are not traced (an event record of this kind cannot be captured with timing).
struct TraceSlot {
    cudaEvent_t begin = nullptr, end = nullptr;
    b200_trace_record rec;
    bool used = false;
};
struct Trace {
    std::mutex mu;
    std::vector<TraceSlot> ring;
    size_t next = 0, count = 0;   // count = slots holding unread records (oldest at next - count)
    int device = -1;
    std::atomic<int> on{0};
} g_trace;

const char* kernel_label(int k) {
    switch (k) {
        case B200_KERNEL_TILE_MMA: return "b200_fattn:tile_mma";
        case B200_KERNEL_DECODE_SPLIT: return "b200_fattn:decode_split";
        case B200_KERNEL_PREFILL_TC5: return "b200_fattn:prefill_tc5";
        default: return "b200_fattn";
    }
}

int do_launch_untraced(Plan& plan, void* workspace, size_t ws_bytes, cudaStream_t st);

int do_launch(Plan& plan, void* workspace, size_t ws_bytes, cudaStream_t st) {
    if (!g_trace.on.load(std::memory_order_relaxed)) return do_launch_untraced(plan, workspace, ws_bytes, st);
    int dev = -1;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != g_trace.device || cudaStreamIsCapturing(st, &cap) != cudaSuccess ||
        cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return do_launch_untraced(plan, workspace, ws_bytes, st);
    }
    std::lock_guard<std::mutex> lk(g_trace.mu);
    if (g_trace.ring.empty()) return do_launch_untraced(plan, workspace, ws_bytes, st);
    TraceSlot& slot = g_trace.ring[g_trace.next];
    const FattnArgs& a = plan.args;
    nvtxRangePushA(kernel_label(plan.kernel));
    cudaEventRecord(slot.begin, st);
    const int rc = do_launch_untraced(plan, workspace, ws_bytes, st);
    cudaEventRecord(slot.end, st);
    nvtxRangePop();
    if (rc == B200_OK) {
        slot.rec = b200_trace_record{plan.kernel, a.n_splits, a.hd, a.Tq, a.Lk, a.H, a.Hkv, a.B, a.k.type, -1.0f};
        slot.used = true;
        g_trace.next = (g_trace.next + 1) % g_trace.ring.size();
        if (g_trace.count < g_trace.ring.size()) g_trace.count++;   // a full ring drops its oldest record
    }
    return rc;
}

int do_launch_untraced(Plan& plan, void* workspace, size_t ws_bytes, cudaStream_t st) {
    FattnArgs& a = plan.args;
    if (plan.cast_kv || plan.cast_r) {
        if (!workspace || ws_bytes < plan.ws_bytes || (uintptr_t)workspace % 256) return B200_E_WORKSPACE;
        FattnArgs c = a;
        int ce = 0;
        if (plan.cast_kv) {
            void* kbuf = workspace;
            void* vbuf = (uint8_t*)workspace + plan.cast_each;
            const int Bk = a.B / a.bq;
            ce = launch_kv_pair_to_f16(a.k, kbuf, a.v, vbuf, a.hd, a.Lk, a.Hkv, Bk, st);
            c = with_f16_kv(c, kbuf, vbuf);
        }
        if (ce == 0 && plan.cast_r) {
            void* rbuf = (uint8_t*)workspace + 2 * plan.cast_each;
            ce = launch_kv_to_f16(a.r, rbuf, a.hd, 2 * a.Tq - 1, a.H, a.r_ne3, st);
            c = with_f16_r(c, rbuf);
        }
        if (ce != 0) return cuda_fail((cudaError_t)ce, "operand conversion launch");
        const int rc = launch_prefill_tc5(c, st, g_cuda_err, sizeof(g_cuda_err));
        if (rc != B200_OK) return rc;
        g_last_kernel = plan.kernel;
        return B200_OK;
    }
    if (plan.ws_bytes) {
        if (!workspace || ws_bytes < plan.ws_bytes || (uintptr_t)workspace % 256) return B200_E_WORKSPACE;
        const int hdp = a.hd <= 32 ? 32 : (a.hd <= 64 ? 64 : 128);
        const size_t units = (size_t)a.B * a.Hkv * a.n_splits;
        const size_t o = ((units * 16 * hdp * sizeof(float) + 255) / 256) * 256;
        a.ws_o = (float*)workspace;
        a.ws_ml = (float*)((uint8_t*)workspace + o);
    }
    int e = 0;
    switch (plan.kernel) {
        case B200_KERNEL_DECODE_SPLIT: e = launch_decode_split(a, st); break;
        case B200_KERNEL_PREFILL_TC5: {
            const int rc = launch_prefill_tc5(a, st, g_cuda_err, sizeof(g_cuda_err));
            if (rc != B200_OK) return rc;
            break;
        }
        default: e = launch_tile_mma(a, st); break;
    }
    if (e != 0) return cuda_fail((cudaError_t)e, "kernel launch");
    g_last_kernel = plan.kernel;
    return B200_OK;
}

// ---- per-thread staging arena of the host-buffer entry point ----
struct Arena {
    uint8_t* base = nullptr;
    size_t cap = 0;
    int device = -1;
    cudaStream_t stream = nullptr, stream2 = nullptr;
    ~Arena() { release(); }
    void release() {
        if (base) cudaFree(base);
        if (stream) cudaStreamDestroy(stream);
        if (stream2) cudaStreamDestroy(stream2);
        base = nullptr, cap = 0, stream = nullptr, stream2 = nullptr, device = -1;
    }
};
thread_local Arena g_arena;

// Bytes spanned by a strided tensor (offset of the last element + one element/block).
size_t span_bytes(const b200_tensor* t) {
    size_t last = 0;
    const int64_t n0 = t->type == B200_TYPE_Q8_0 ? t->ne[0] / 32 : t->ne[0];
    last += (size_t)(n0 - 1) * t->nb[0];
    for (int i = 1; i < 4; i++) last += (size_t)(t->ne[i] - 1) * t->nb[i];
    return last + t->nb[0];
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

B200_API const char* b200_version(void) { return "b200-fattn 0.1 (sm_100a)"; }

B200_API const char* b200_strerror(int code) {
    switch (code) {
        case B200_OK: return "ok";
        case B200_E_NULL: return "a required pointer is NULL";
        case B200_E_TYPE: return "operand type not allowed by the flash_attn_ext contract";
        case B200_E_SHAPE: return "operand shapes disagree";
        case B200_E_STRIDE: return "stride not allowed (nb[0] must be the element size; dst must be contiguous)";
        case B200_E_ALIGN: return "operand base pointer is misaligned for its type";
        case B200_E_UNSUPPORTED: return "legal operator form without a kernel in this library";
        case B200_E_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case B200_E_CUDA: return "CUDA call failed (see b200_last_cuda_error)";
        case B200_E_NO_DEVICE: return "no sm_100 CUDA device is current";
        case B200_E_LIMIT: return "size exceeds a fixed limit of this entry point";
        case B200_E_STATE: return "object used in the wrong state";
        case B200_E_DEVICE_WAIT: return "a bounded device-side wait ran out";
        default: return "unknown error code";
    }
}

B200_API const char* b200_last_cuda_error(void) { return g_cuda_err; }
B200_API int b200_last_kernel(void) { return g_last_kernel; }

B200_API int b200_device_status(void) {
    int st_tc5 = 0, st_mma = 0;
    int e = tc5_read_status(&st_tc5);
    if (e == 0) e = mma_read_status(&st_mma);
    if (e != 0) return cuda_fail((cudaError_t)e, "cudaMemcpyFromSymbol(status)");
    return (st_tc5 | st_mma) ? B200_E_DEVICE_WAIT : B200_OK;
}

B200_API int b200_device_status_reset(void) {
    int e = tc5_reset_status();
    if (e == 0) e = mma_reset_status();
    if (e != 0) return cuda_fail((cudaError_t)e, "cudaMemcpyToSymbol(status)");
    return B200_OK;
}

B200_API int b200_trace_enable(int capacity) {
    if (capacity < 0 || capacity > (1 << 16)) return B200_E_LIMIT;
    std::lock_guard<std::mutex> lk(g_trace.mu);
    g_trace.on.store(0);
    for (TraceSlot& sl : g_trace.ring) {
        if (sl.begin) cudaEventDestroy(sl.begin);
        if (sl.end) cudaEventDestroy(sl.end);
    }
    g_trace.ring.clear();
    g_trace.next = g_trace.count = 0;
    g_trace.device = -1;
    if (capacity == 0) return B200_OK;
    DeviceInfo di;
    const int rc = device_info(&di);
    if (rc != B200_OK) return rc;
    cudaGetDevice(&g_trace.device);
    g_trace.ring.resize((size_t)capacity);
    for (TraceSlot& sl : g_trace.ring) {
        cudaError_t e = cudaEventCreate(&sl.begin);
        if (e == cudaSuccess) e = cudaEventCreate(&sl.end);
        if (e != cudaSuccess) {
            for (TraceSlot& x : g_trace.ring) {
                if (x.begin) cudaEventDestroy(x.begin);
                if (x.end) cudaEventDestroy(x.end);
            }
            g_trace.ring.clear();
            return cuda_fail(e, "cudaEventCreate(trace)");
        }
    }
    g_trace.on.store(1);
    return B200_OK;
}

B200_API int b200_trace_read(b200_trace_record* out, int max_records, int* n_out) {
    if (!n_out || (max_records > 0 && !out)) return B200_E_NULL;
    *n_out = 0;
    std::lock_guard<std::mutex> lk(g_trace.mu);
    const size_t n = g_trace.ring.size();
    if (n == 0) return B200_OK;
    size_t idx = (g_trace.next + n - g_trace.count) % n;   // oldest unread
    while (g_trace.count > 0 && *n_out < max_records) {
        TraceSlot& sl = g_trace.ring[idx];
        cudaError_t e = cudaEventSynchronize(sl.end);
        float ms = -1.0f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, sl.begin, sl.end);
        if (e != cudaSuccess) return cuda_fail(e, "trace event");
        out[*n_out] = sl.rec;
        out[*n_out].ms = ms;
        (*n_out)++;
        sl.used = false;
        idx = (idx + 1) % n;
        g_trace.count--;
    }
    return B200_OK;
}

B200_API int b200_test_empty_launch(void* cuda_stream) {
    const int e = launch_empty((cudaStream_t)cuda_stream);
    if (e != 0) return cuda_fail((cudaError_t)e, "empty launch");
    return B200_OK;
}

B200_API int b200_test_bounded_wait(int polls, void* cuda_stream) {
    if (polls < 1 || polls > (1 << 20)) return B200_E_LIMIT;
    DeviceInfo di;
    const int rc = device_info(&di);
    if (rc != B200_OK) return rc;
    const int e = launch_bounded_wait_probe(polls, (cudaStream_t)cuda_stream);
    if (e != 0) return cuda_fail((cudaError_t)e, "bounded-wait probe launch");
    return B200_OK;
}

B200_API int b200_set_decode_splits(int n_splits) {
    if (n_splits < 0 || n_splits > 64) return B200_E_LIMIT;
    decode_split_force(n_splits);
    return B200_OK;
}

B200_API int b200_set_kernel_override(int kernel) {
    if (kernel < B200_KERNEL_NONE || kernel > B200_KERNEL_PREFILL_TC5) return B200_E_SHAPE;
    g_override.store(kernel, std::memory_order_relaxed);
    return B200_OK;
}

B200_API int b200_beam_cells_to_index(const int32_t* cell_pos, const uint32_t* cell_seq_bits, int n_cells,
                                      const int32_t* tok_seq, const int32_t* tok_pos, int n_tokens,
                                      int32_t* index_out, int stride, int32_t* len_out) {
    if (!cell_pos || !cell_seq_bits || !tok_seq || !tok_pos || !index_out || !len_out) return B200_E_NULL;
    if (n_cells < 0 || n_tokens < 0 || stride <= 0) return B200_E_SHAPE;
    for (int j = 0; j < n_tokens; j++) {
        if (tok_seq[j] < 0 || tok_seq[j] >= 32) return B200_E_SHAPE;
        int32_t* row = index_out + (size_t)j * stride;
        int n = 0;
        for (int i = 0; i < n_cells; i++) {
            // visible iff the cell carries the token's sequence id and is not ahead of the token
            if (((cell_seq_bits[i] >> tok_seq[j]) & 1u) && cell_pos[i] <= tok_pos[j]) {
                if (n == stride) return B200_E_LIMIT;
                row[n++] = i;
            }
        }
        len_out[j] = n;
        for (int i = n; i < stride; i++) row[i] = 0;   // never read (beyond kv_len), kept in range all the same
    }
    return B200_OK;
}

B200_API int b200_beam_cells_to_union(const int32_t* cell_pos, const uint32_t* cell_seq_bits, int n_cells,
                                      const int32_t* tok_seq, const int32_t* tok_pos, int n_tokens,
                                      int32_t* index_out, int stride, int32_t* len_out, uint16_t* mask_out) {
    if (!cell_pos || !cell_seq_bits || !tok_seq || !tok_pos || !index_out || !len_out || !mask_out) return B200_E_NULL;
    if (n_cells < 0 || n_tokens < 0 || stride <= 0) return B200_E_SHAPE;
    for (int j = 0; j < n_tokens; j++)
        if (tok_seq[j] < 0 || tok_seq[j] >= 32) return B200_E_SHAPE;
    int n = 0;
    for (int i = 0; i < n_cells; i++) {
        bool any = false;
        for (int j = 0; j < n_tokens && !any; j++) any = ((cell_seq_bits[i] >> tok_seq[j]) & 1u) && cell_pos[i] <= tok_pos[j];
        if (!any) continue;   // a cell no token of this step can see (free, or ahead of every token): not in the list
        if (n == stride) return B200_E_LIMIT;
        index_out[n] = i;
        for (int j = 0; j < n_tokens; j++) {
            const bool visible = ((cell_seq_bits[i] >> tok_seq[j]) & 1u) && cell_pos[i] <= tok_pos[j];
            mask_out[(size_t)j * stride + n] = visible ? 0x0000u : 0xFC00u;   // F16 0 / -inf, the reference's values
        }
        n++;
    }
    for (int i = n; i < stride; i++) {
        index_out[i] = 0;
        for (int j = 0; j < n_tokens; j++) mask_out[(size_t)j * stride + i] = 0xFC00u;
    }
    *len_out = n;
    return B200_OK;
}

B200_API int b200_mask_classify(const uint16_t* mask, int Lk, int Tq, int64_t row_stride, int* kind, int* n_past,
                                int* kv_len) {
    if (!mask || !kind) return B200_E_NULL;
    if (Lk <= 0 || Tq <= 0 || row_stride < Lk) return B200_E_SHAPE;
    *kind = B200_MASK_GENERAL;
    // per row: the number of leading zeros (0x0000 / 0x8000) followed by -inf (0xFC00) to the end, or -1
    int first = -1;
    bool same = true, step = true;
    for (int i = 0; i < Tq; i++) {
        const uint16_t* row = mask + (int64_t)i * row_stride;
        int z = 0;
        while (z < Lk && (row[z] & 0x7FFFu) == 0) z++;
        for (int j = z; j < Lk; j++)
            if (row[j] != 0xFC00u) return B200_OK;   // a finite bias, or a hole: general
        if (i == 0) first = z;
        if (z != first) same = false;
        // causal with n_past = first - 1: row i shows min(Lk, first + i) keys
        if (z != (first + i < Lk ? first + i : Lk)) step = false;
    }
    if (same) {
        if (first == Lk) *kind = B200_MASK_NONE;
        else {
            *kind = B200_MASK_TAIL;
            if (kv_len) *kv_len = first;
        }
    } else if (step && first >= 1) {
        *kind = B200_MASK_CAUSAL;
        if (n_past) *n_past = first - 1;
    }
    return B200_OK;
}

B200_API int b200_fattn_supports(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                 const b200_tensor* mask, const b200_tensor* dst, const b200_fattn_params* params,
                                 const b200_fattn_ext* ext, int* why) {
    Plan plan;
    const int rc = make_plan(q, k, v, mask, dst, params, ext, false, &plan);
    if (why) *why = rc;
    return rc == B200_OK ? 1 : 0;
}

B200_API int b200_fattn_plan(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                             const b200_tensor* mask, const b200_tensor* dst, const b200_fattn_params* params,
                             const b200_fattn_ext* ext, int* kernel, int* n_splits) {
    Plan plan;
    const int rc = make_plan(q, k, v, mask, dst, params, ext, false, &plan);
    if (rc != B200_OK) return rc;
    if (kernel) *kernel = plan.kernel;
    if (n_splits) *n_splits = plan.args.n_splits;
    return B200_OK;
}

B200_API int b200_fattn_workspace_bytes(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                        const b200_tensor* mask, const b200_tensor* dst,
                                        const b200_fattn_params* params, const b200_fattn_ext* ext, size_t* bytes) {
    if (!bytes) return B200_E_NULL;
    Plan plan;
    const int rc = make_plan(q, k, v, mask, dst, params, ext, false, &plan);
    if (rc != B200_OK) return rc;
    *bytes = plan.ws_bytes;
    return B200_OK;
}

B200_API int b200_fattn_launch(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                               const b200_tensor* mask, const b200_tensor* dst, const b200_fattn_params* params,
                               const b200_fattn_ext* ext, void* workspace, size_t workspace_bytes,
                               void* cuda_stream) {
    Plan plan;
    // The split count must match b200_fattn_workspace_bytes, which assumes 148 SMs; the device is
    // only queried to refuse non-sm_100 parts.
    int rc = make_plan(q, k, v, mask, dst, params, ext, false, &plan);
    if (rc != B200_OK) return rc;
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    return do_launch(plan, workspace, workspace_bytes, (cudaStream_t)cuda_stream);
}

B200_API int b200_fattn_forward_host(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                     const b200_tensor* mask, const b200_tensor* dst,
                                     const b200_fattn_params* params, const b200_fattn_ext* ext) {
    Plan plan;
    int rc = make_plan(q, k, v, mask, dst, params, ext, false, &plan);
    if (rc != B200_OK) return rc;
    if (ext && ext->kv_index) return B200_E_UNSUPPORTED;   // index lists address a device-resident pool; nothing to stage
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    int dev = 0;
    cudaGetDevice(&dev);

    // operands to stage: q, k, v, [mask], [q_v, r, pos_bias_u, pos_bias_v], [kv_len]; then dst and workspace
    constexpr int NIN = 8;
    const b200_tensor* in[NIN] = {q, k, v, mask, ext ? ext->q_v : nullptr, ext ? ext->r : nullptr,
                                  ext ? ext->pos_bias_u : nullptr, ext ? ext->pos_bias_v : nullptr};
    size_t off[NIN], total = 0;
    auto bump = [&](size_t n) {
        const size_t o = total;
        total += (n + 255) / 256 * 256;
        return o;
    };
    for (int i = 0; i < NIN; i++) off[i] = in[i] ? bump(span_bytes(in[i])) : 0;
    const size_t kvlen_off = (ext && ext->kv_len) ? bump((size_t)q->ne[3] * 4) : 0;
    const size_t qlen_off = (ext && ext->q_len) ? bump((size_t)q->ne[3] * 4) : 0;
    const size_t dst_bytes = (size_t)dst->ne[0] * dst->ne[1] * dst->ne[2] * dst->ne[3] * 4;
    const size_t dst_off = bump(dst_bytes);

    // Batch entries are independent, so the call is pipelined over chunks of the batch dimension on two
    // streams: the H2D copy of chunk i+1 overlaps the kernel and the D2H copy of chunk i (separate copy
    // engines).  Chunking needs the batch dimension outermost in every batched operand; otherwise one chunk.
    const int64_t B = q->ne[3];
    auto batch_outermost = [](const b200_tensor* t) {
        b200_tensor one = *t;
        one.ne[3] = 1;
        return t->ne[3] == 1 || t->nb[3] >= span_bytes(&one);
    };
    bool chunkable = B >= 2 && k->ne[3] == B;
    for (int i = 0; i < NIN && chunkable; i++)
        if (in[i] && in[i]->ne[3] != 1 && (in[i]->ne[3] != B || !batch_outermost(in[i]))) chunkable = false;
    static const int max_chunks = [] {  // B200_HOST_CHUNKS=1..16 overrides the default pipeline depth
        const char* e = getenv("B200_HOST_CHUNKS");
        const int n = e ? atoi(e) : 0;
        return n >= 1 && n <= 16 ? n : 4;
    }();
    const int n_chunks = chunkable ? (int)(B < max_chunks ? B : max_chunks) : 1;
    // Workspace of one chunk: a smaller batch may be split over more KV ranges than the whole call would be,
    // so the split-decode workspace is sized for the chunk batches, not taken from the full plan.
    size_t ws_need = plan.ws_bytes;
    if (plan.kernel == B200_KERNEL_DECODE_SPLIT) {
        for (int c = 0; c < n_chunks; c++) {
            const int64_t b0 = B * c / n_chunks;
            const int nb = (int)(B * (c + 1) / n_chunks - b0);
            // the split count depends on operand alignment: describe the operands where the chunk will find them
            // (arena offsets behind a notional 1 MiB-aligned base), not where the host buffers are
            FattnArgs ca = plan.args;
            View* views[4] = {&ca.q, &ca.k, &ca.v, &ca.mask};
            for (int i = 0; i < 4; i++) {
                if (!in[i]) continue;
                b200_tensor t = *in[i];
                t.data = (void*)(uintptr_t)(((size_t)1 << 20) + off[i] +
                                            (n_chunks > 1 && in[i]->ne[3] != 1 ? (size_t)b0 * in[i]->nb[3] : 0));
                *views[i] = make_view(&t);
            }
            const int ns = decode_split_choose(ca, nb, di.sm_count);
            const size_t w = decode_split_ws_bytes(nb, plan.args.Hkv, ns, plan.args.hd);
            if (w > ws_need) ws_need = w;
        }
    }
    const size_t ws_each = (ws_need + 255) / 256 * 256;
    const size_t ws_off = bump(2 * ws_each);  // one per stream in flight

    Arena& ar = g_arena;
    cudaError_t e;
    if (ar.device != dev) ar.release();
    if (!ar.stream) {
        if ((e = cudaStreamCreateWithFlags(&ar.stream, cudaStreamNonBlocking)) != cudaSuccess)
            return cuda_fail(e, "cudaStreamCreate");
        ar.device = dev;
    }
    if (ar.cap < total) {
        if (ar.base) cudaFree(ar.base);
        ar.base = nullptr, ar.cap = 0;
        if ((e = cudaMalloc((void**)&ar.base, total)) != cudaSuccess) return cuda_fail(e, "cudaMalloc(arena)");
        ar.cap = total;
    }
    if (!ar.stream2 && (e = cudaStreamCreateWithFlags(&ar.stream2, cudaStreamNonBlocking)) != cudaSuccess)
        return cuda_fail(e, "cudaStreamCreate");

    cudaStream_t streams[2] = {ar.stream, ar.stream2};

    // Everything below enqueues asynchronous work that reads and writes the caller's host buffers.  Whatever goes
    // wrong, the call leaves through ONE exit that first waits for both streams, so the caller may free or reuse
    // its buffers as soon as it has the return code, and the event is always destroyed.
    b200_tensor dt[NIN];
    cudaEvent_t shared_ready = nullptr;
    auto enqueue_all = [&]() -> int {
        cudaError_t e;
        // operands without a batch dimension (ne[3] == 1) are copied once, ahead of everything, on stream 0
        for (int i = 0; i < NIN; i++) {
            if (!in[i]) continue;
            dt[i] = *in[i];
            dt[i].data = ar.base + off[i];
            if (n_chunks == 1 || in[i]->ne[3] == 1) {
                if ((e = cudaMemcpyAsync(dt[i].data, in[i]->data, span_bytes(in[i]), cudaMemcpyHostToDevice, streams[0])) !=
                    cudaSuccess)
                    return cuda_fail(e, "cudaMemcpyAsync(H2D)");
            }
        }
        if (ext && ext->kv_len &&
            (e = cudaMemcpyAsync(ar.base + kvlen_off, ext->kv_len, (size_t)B * 4, cudaMemcpyHostToDevice, streams[0])) !=
                cudaSuccess)
            return cuda_fail(e, "cudaMemcpyAsync(kv_len)");
        if (ext && ext->q_len &&
            (e = cudaMemcpyAsync(ar.base + qlen_off, ext->q_len, (size_t)B * 4, cudaMemcpyHostToDevice, streams[0])) !=
                cudaSuccess)
            return cuda_fail(e, "cudaMemcpyAsync(q_len)");
        if (n_chunks > 1) {
            if ((e = cudaEventCreateWithFlags(&shared_ready, cudaEventDisableTiming)) != cudaSuccess)
                return cuda_fail(e, "cudaEventCreate");
            if ((e = cudaEventRecord(shared_ready, streams[0])) != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
            if ((e = cudaStreamWaitEvent(streams[1], shared_ready, 0)) != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
        }
        for (int c = 0; c < n_chunks; c++) {
            const int64_t b0 = B * c / n_chunks, b1 = B * (c + 1) / n_chunks, nb = b1 - b0;
            cudaStream_t st = streams[c & 1];
            b200_tensor ct[NIN];
            for (int i = 0; i < NIN; i++) {
                if (!in[i]) continue;
                ct[i] = dt[i];
                if (n_chunks > 1 && in[i]->ne[3] != 1) {
                    ct[i].data = (uint8_t*)dt[i].data + (size_t)b0 * in[i]->nb[3];
                    ct[i].ne[3] = nb;
                    b200_tensor hview = *in[i];
                    hview.ne[3] = nb;
                    if ((e = cudaMemcpyAsync(ct[i].data, (const uint8_t*)in[i]->data + (size_t)b0 * in[i]->nb[3], span_bytes(&hview),
                                             cudaMemcpyHostToDevice, st)) != cudaSuccess)
                        return cuda_fail(e, "cudaMemcpyAsync(H2D chunk)");
                }
            }
            b200_fattn_ext dext;
            memset(&dext, 0, sizeof(dext));
            if (ext) {
                dext = *ext;
                dext.q_v = ext->q_v ? &ct[4] : nullptr;
                dext.r = ext->r ? &ct[5] : nullptr;
                dext.pos_bias_u = ext->pos_bias_u ? &ct[6] : nullptr;
                dext.pos_bias_v = ext->pos_bias_v ? &ct[7] : nullptr;
                dext.kv_len = ext->kv_len ? (const int32_t*)(ar.base + kvlen_off) + b0 : nullptr;
                dext.q_len = ext->q_len ? (const int32_t*)(ar.base + qlen_off) + b0 : nullptr;
            }
            b200_tensor cdst = *dst;
            cdst.ne[3] = nb;
            cdst.data = ar.base + dst_off + (size_t)b0 * dst->nb[3];
            Plan cplan;
            int rc_c = make_plan(&ct[0], &ct[1], &ct[2], mask ? &ct[3] : nullptr, &cdst, params, ext ? &dext : nullptr, false, &cplan);
            if (rc_c != B200_OK) return rc_c;
            if (cplan.ws_bytes > ws_each) return B200_E_WORKSPACE;
            rc_c = do_launch(cplan, cplan.ws_bytes ? ar.base + ws_off + (size_t)(c & 1) * ws_each : nullptr, cplan.ws_bytes, st);
            if (rc_c != B200_OK) return rc_c;
            if ((e = cudaMemcpyAsync((uint8_t*)dst->data + (size_t)b0 * dst->nb[3], cdst.data, (size_t)nb * dst->nb[3],
                                     cudaMemcpyDeviceToHost, st)) != cudaSuccess)
                return cuda_fail(e, "cudaMemcpyAsync(D2H)");
        }
        return B200_OK;
    };
    const int rc_enqueue = enqueue_all();
    const cudaError_t e0 = cudaStreamSynchronize(streams[0]), e1 = cudaStreamSynchronize(streams[1]);
    if (shared_ready) cudaEventDestroy(shared_ready);
    if (rc_enqueue != B200_OK) return rc_enqueue;
    if (e0 != cudaSuccess) return cuda_fail(e0, "cudaStreamSynchronize");
    if (e1 != cudaSuccess) return cuda_fail(e1, "cudaStreamSynchronize");
    return B200_OK;
}

B200_API void b200_host_arena_release(void) { g_arena.release(); }

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free variant of the split-KV decode launch.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run the operator:
// a decode loop that sits inside a real-time audio callback, an embedder whose memory budget is
// fixed at start-up and audited, or a process that hands the library a stream but owns no
// allocator of its own.  b200_fattn_launch needs a caller-provided workspace for the split-KV
// partials; this entry point instead keeps that scratch in a fixed array that is part of the
// loaded module, so a call needs nothing but its operands.
//
// The array costs kStaticScratchBytes of device memory on every GPU that loads the library, from
// load until the process exits.  All calls share it and it is never cleared: the decode kernel
// writes every partial (O, m, l) of every split before the merge kernel reads any, so nothing has
// to start at zero, but the previous call's bytes are still there.  Two calls that can overlap
// on the GPU (different streams, or different host threads) race on the array; issue them on one
// stream or serialise them.
// ------------------------------------------------------------------------------------------
namespace b200 {
namespace {
// 8 MiB.  A launch fits when B * Hkv * n_splits * (16 * hdp * 4 + 128) bytes <= 8 MiB (hdp = head_dim rounded up to
// 32 / 64 / 128): e.g. 8 streams x 8 KV heads x head_dim 128 with up to 15 splits, or one Whisper segment
// (20 heads, head_dim 64) with up to 64.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address the kernels can use comes from cudaGetSymbolAddress, once per device, with that device current.
int static_scratch_ptr(void** out) {
    static std::mutex mu;
    static void* ptrs[64] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaGetDevice");
        return B200_E_NO_DEVICE;
    }
    if (dev < 0 || dev >= 64) return B200_E_NO_DEVICE;
    std::lock_guard<std::mutex> lk(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        if (!p || (uintptr_t)p % 256) return B200_E_ALIGN;
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return B200_OK;
}
}  // namespace
}  // namespace b200

extern "C" B200_API int b200_fattn_launch_static(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                                  const b200_tensor* mask, const b200_tensor* dst,
                                                  const b200_fattn_params* params, const b200_fattn_ext* ext,
                                                  void* cuda_stream) {
    Plan plan;
    int rc = make_plan(q, k, v, mask, dst, params, ext, false, &plan);
    if (rc != B200_OK) return rc;
    if (plan.kernel != B200_KERNEL_DECODE_SPLIT) return B200_E_UNSUPPORTED;  // only the split-KV decode form
    if (plan.ws_bytes > kStaticScratchBytes) return B200_E_LIMIT;
    DeviceInfo di;
    if ((rc = device_info(&di))) return rc;
    void* scratch = nullptr;
    if ((rc = static_scratch_ptr(&scratch))) return rc;
    return do_launch(plan, scratch, kStaticScratchBytes, (cudaStream_t)cuda_stream);
}

extern "C" B200_API size_t b200_fattn_static_scratch_bytes(void) { return b200::kStaticScratchBytes; }
