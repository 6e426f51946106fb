// fattn_common.cuh — argument block shared by the attention kernels, and small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_fattn.h"

namespace b200 {

// One operand as the kernels see it: base pointer plus byte strides of dims 1..3.
struct View {
    const uint8_t* p;
    int64_t nb1, nb2, nb3;
    int32_t type;    // b200_type
    int32_t vec16;   // base and all strides are multiples of 16 bytes: 128-bit loads are legal
};

struct FattnArgs {
    View q, k, v, mask, qv, r;
    float* dst;  // contiguous [hd, H, Tq, B]
    int32_t hd, Tq, H, B;
    int32_t Lk, Hkv, gqa, bq;  // bq = B / Bk
    int32_t mask_ne2, mask_ne3, r_ne3, has_mask;
    float scale;      // already divided by softcap when softcap != 0
    float softcap;    // 0 = off
    float relscale;   // the caller's scale (bias uses it undivided)
    float m0, m1;     // ALiBi bases
    int32_t n2;       // ALiBi head split; 0 = max_bias off
    int32_t causal, n_past;
    const int32_t* kv_len;
    const int32_t* q_len;      // [B] valid query rows per batch entry; nullptr = Tq
    const int32_t* kv_index;   // [B][kv_index_stride] cache row of each logical key; nullptr = identity
    int32_t kv_index_stride;
    int32_t relpos, relpos_f32;
    int32_t cluster_merge;  // split-KV: the splits of one (batch, kv-head) form a thread-block cluster and merge through distributed shared memory
    const float* bias_u;  // [hd, H] fp32 added to Q on load (content scores); nullptr = off
    const float* bias_v;  // the same for the Q of the relative-position bias
    // split-KV
    int32_t n_splits;
    float* ws_o;   // [B][Hkv][n_splits][16][hd]
    float* ws_ml;  // [B][Hkv][n_splits][16][2]
};

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float alibi_slope(const FattnArgs& a, int h) {
    if (a.n2 == 0) return 1.0f;
    return h < a.n2 ? powf(a.m0, (float)(h + 1)) : powf(a.m1, (float)(2 * (h - a.n2) + 1));
}

// Valid query rows of batch entry b (ext->q_len clamped to [0, Tq]; Tq without the table).
__device__ __forceinline__ int q_rows_of(const FattnArgs& a, int b) {
    if (!a.q_len) return a.Tq;
    const int v = a.q_len[b];
    return v < 0 ? 0 : (v > a.Tq ? a.Tq : v);
}

// n_past of the implicit causal rule (key k visible to query q iff k <= n_past + q).  A batched launch that gives
// both per-entry tables places an entry's q_len new tokens at the end of its kv_len keys; otherwise the scalar applies.
__device__ __forceinline__ int n_past_of(const FattnArgs& a, int len_b, int tq_b) {
    return (a.q_len && a.kv_len) ? len_b - tq_b : a.n_past;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Eight Q elements [c0, c0+8) of one row plus eight fp32 bias values, as packed f16: the sum is formed in fp32
// and rounded once (an F32 add followed by the conversion to F16). F16 and F32 rows only; c0 + 8 <= head_dim.
__device__ __forceinline__ uint4 load8_plus_bias_as_half(const uint8_t* rowp, int type, int c0, bool vec16,
                                                         const float* bias8) {
    float f[8];
    if (type == B200_TYPE_F16) {
        uint32_t w[4];
        if (vec16) {
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(rowp + 2 * c0));
            w[0] = u.x, w[1] = u.y, w[2] = u.z, w[3] = u.w;
        } else {
            const uint16_t* h = reinterpret_cast<const uint16_t*>(rowp + 2 * c0);
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] = h[2 * i] | ((uint32_t)h[2 * i + 1] << 16);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = p.x, f[2 * i + 1] = p.y;
        }
    } else if (vec16) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(rowp + 4 * c0));
        const float4 y = __ldg(reinterpret_cast<const float4*>(rowp + 4 * c0 + 16));
        f[0] = x.x, f[1] = x.y, f[2] = x.z, f[3] = x.w, f[4] = y.x, f[5] = y.y, f[6] = y.z, f[7] = y.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) f[i] = *reinterpret_cast<const float*>(rowp + 4 * (c0 + i));
    }
#pragma unroll
    for (int i = 0; i < 8; i++) f[i] = __fadd_rn(f[i], __ldg(bias8 + i));
    uint4 out;
    out.x = pack_half2(f[0], f[1]), out.y = pack_half2(f[2], f[3]);
    out.z = pack_half2(f[4], f[5]), out.w = pack_half2(f[6], f[7]);
    return out;
}

// Raises a kernel's dynamic shared memory limit once per (kernel instantiation, device): the attribute call is
// kept out of the steady-state launch path (and out of stream captures after the first launch).
// `done` is a static flag array owned by the calling launcher instantiation (one per kernel instantiation).
template <typename Kern>
inline cudaError_t set_smem_once(Kern kern, size_t smem, bool (&done)[64]) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
    return e;
}

// Launchers implemented per kernel family; each returns a cudaError_t-compatible int (0 = ok).
int launch_tile_mma(const FattnArgs& a, cudaStream_t st);
int launch_decode_split(const FattnArgs& a, cudaStream_t st);
// Converts K or V (F32 / Q8_0 / unaligned F16, any strides) to contiguous F16 [hd, Lk, Hkv, Bk] at `dst`.
int launch_kv_to_f16(const View& src, void* dst, int hd, int Lk, int Hkv, int Bk, cudaStream_t st);
// K and V of one call in one launch.
int launch_kv_pair_to_f16(const View& k, void* kdst, const View& v, void* vdst, int hd, int Lk, int Hkv, int Bk, cudaStream_t st);
size_t decode_split_ws_bytes(int B, int Hkv, int n_splits, int hd);
int decode_split_choose(const FattnArgs& a, int B, int sm_count);
void decode_split_force(int n_splits);  // 0 = automatic
bool decode_cluster_merge_ok(const FattnArgs& a);
// True when a launch with these arguments (n_splits set) merges its splits inside thread-block clusters: it then
// neither reads nor writes a workspace.
bool decode_uses_cluster_merge(const FattnArgs& a);
// Status word of the mma.sync kernels' bounded waits (0 = no wait ever ran out). cudaError_t-compatible returns.
int mma_read_status(int* status);
int mma_reset_status();
// Test hook: a one-warp kernel that waits, for at most `polls` polls, on an mbarrier nobody completes, then sets the
// status word and returns.
int launch_bounded_wait_probe(int polls, cudaStream_t st);
// Measurement hook: one empty one-warp kernel on the stream (the launch-latency floor of a kernel per layer).
int launch_empty(cudaStream_t st);

}  // namespace b200
