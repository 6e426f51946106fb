// fattn_mma.cu — the general tiled attention kernel and the split-KV decode kernel.
//
// Both kernels stage K/V tiles as fp16 in XOR-swizzled shared memory (F16 rows are copied,
// F32 rows are rounded, Q8_0 blocks are dequantised as fp32(d)*q and rounded to fp16), run
// Q.K^T and P.V on the mma.sync m16n8k16 tensor path with fp32 accumulators and keep the
// online softmax in fp32 registers.
//
//  * fattn_tile_mma_kernel  — 64 query rows x 64 keys per step, one (q-tile, head, batch) per
//    CTA.  Covers every operand form of the op contract: explicit F16 mask ([Lk,Tq,1|H,1|B]),
//    implicit causal mask, per-batch kv_len, softcap, ALiBi, GQA, generic strides, and the
//    fused FastConformer relative-position bias (per-warp band GEMM + diagonal gather).
//  * fattn_decode_split_kernel — for <= 16 query rows per KV head (single-token decode with
//    GQA, beams sharing a cross-attention cache): one (split, kv-head, batch) per CTA streams its
//    share of the keys once, the four warps own 16-key slices of each tile, and partial
//    (O, m, l) go to the workspace; fattn_merge_kernel combines splits with a log-sum-exp merge.
#include <atomic>
#include <cstdlib>
#include "fattn_common.cuh"

namespace b200 {

int decode_ctas_per_sm(const FattnArgs& a, bool cluster = false);   // resident CTAs of the split kernel per SM for these operands, as a cluster launch with its receive area if asked (defined below)

__device__ int g_mma_status = 0;  // 0 ok, 1 = a bounded wait of a kernel in this file ran out
#ifdef B200_Q8T_TRACE
__device__ long long g_q8t_trace[16];
#define Q8T_TRACE(k) do { if (blockIdx.x == 0 && blockIdx.y == 3 && blockIdx.z == B200_Q8T_TRACE && threadIdx.x == 0) g_q8t_trace[k] = clock64(); } while (0)
#else
#define Q8T_TRACE(k) do { } while (0)
#endif

namespace {

constexpr int kThreads = 128;

template <int HD>
__device__ __forceinline__ int swz(int row, int ch) {
    if (HD >= 64) return ch ^ (row & 7);
    return ch ^ ((row >> 1) & 3);
}

template <int HD>
__device__ __forceinline__ uint32_t tile_addr(const __half* sm, int row, int ch) {
    return smem_u32(sm) + (uint32_t)((row * (HD / 8) + swz<HD>(row, ch)) * 16);
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Same product with the accumulator rows g+8 in caller-chosen registers: when those rows are padding (all zeros in
// A and in C) a few shared zero registers stand in for them and the real accumulator needs half the registers.
__device__ __forceinline__ void mma16816_lo(float& c0, float& c1, float& z0, float& z1, const uint32_t (&a)[4], uint32_t b0,
                                            uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x on the exponential unit, one instruction (exp2f adds a range fix-up that P in f16 does not need; -inf -> 0).
__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Eight consecutive elements [c0, c0+8) of one row, converted to fp16 (zero beyond hd).
__device__ __forceinline__ uint4 load8_as_half(const uint8_t* rowp, int type, int c0, int hd, bool vec16) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (c0 >= hd) return out;
    if (type == B200_TYPE_F16) {
        if (vec16 && c0 + 8 <= hd) return __ldg(reinterpret_cast<const uint4*>(rowp + 2 * c0));
        __half tmp[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            tmp[i] = (c0 + i < hd) ? *reinterpret_cast<const __half*>(rowp + 2 * (c0 + i)) : __float2half(0.0f);
        out = *reinterpret_cast<uint4*>(tmp);
    } else if (type == B200_TYPE_F32) {
        float f[8];
        if (vec16 && c0 + 8 <= hd) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(rowp + 4 * c0));
            const float4 b = __ldg(reinterpret_cast<const float4*>(rowp + 4 * c0 + 16));
            f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++)
                f[i] = (c0 + i < hd) ? *reinterpret_cast<const float*>(rowp + 4 * (c0 + i)) : 0.0f;
        }
        out.x = pack_half2(f[0], f[1]);
        out.y = pack_half2(f[2], f[3]);
        out.z = pack_half2(f[4], f[5]);
        out.w = pack_half2(f[6], f[7]);
    } else {  // Q8_0: 34-byte blocks {fp16 d; int8 q[32]}; rows are only 2-byte aligned
        const uint8_t* blk = rowp + 34 * (c0 >> 5);
        const float d = __half2float(*reinterpret_cast<const __half*>(blk));
        const uint16_t* qs = reinterpret_cast<const uint16_t*>(blk + 2 + (c0 & 31));
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint16_t w = qs[i];
            f[2 * i] = d * (float)(int8_t)(w & 0xFF);
            f[2 * i + 1] = d * (float)(int8_t)(w >> 8);
        }
        out.x = pack_half2(f[0], f[1]);
        out.y = pack_half2(f[2], f[3]);
        out.z = pack_half2(f[4], f[5]);
        out.w = pack_half2(f[6], f[7]);
    }
    return out;
}

// Rows [row0, row0+NROWS) of a strided 2-D slice -> swizzled fp16 tile; rows outside
// [row_lo, row_hi) are zero-filled.
// `index` (may be null) maps a logical row to the row of `base` that holds it, clamped to [0, pool_rows).
template <int HD, int NROWS>
__device__ __forceinline__ void load_tile(__half* sm, const uint8_t* base, int64_t nb1, int type, bool vec16,
                                          int row0, int row_lo, int row_hi, int hd, int tid, const int32_t* index = nullptr,
                                          int pool_rows = 0) {
    constexpr int CPR = HD / 8;
    for (int idx = tid; idx < NROWS * CPR; idx += kThreads) {
        const int row = idx / CPR, ch = idx % CPR;
        const int grow = row0 + row;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (grow >= row_lo && grow < row_hi) {
            const int src = index ? min(max(__ldg(index + grow), 0), pool_rows - 1) : grow;
            val = load8_as_half(base + (int64_t)src * nb1, type, ch * 8, hd, vec16);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm) + (row * CPR + swz<HD>(row, ch)) * 16) = val;
    }
}

// The same for a Q tile with an fp32 bias row [hd] added before the rounding to fp16 (F16 / F32 rows).
template <int HD, int NROWS>
__device__ __forceinline__ void load_tile_bias(__half* sm, const uint8_t* base, int64_t nb1, int type, bool vec16,
                                               int row0, int row_hi, int hd, const float* bias, int tid) {
    constexpr int CPR = HD / 8;
    for (int idx = tid; idx < NROWS * CPR; idx += kThreads) {
        const int row = idx / CPR, ch = idx % CPR, c0 = ch * 8;
        const int grow = row0 + row;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (grow < row_hi && c0 < hd) {
            const uint8_t* rowp = base + (int64_t)grow * nb1;
            if (c0 + 8 <= hd) {
                val = load8_plus_bias_as_half(rowp, type, c0, vec16, bias + c0);
            } else {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    f[i] = 0.0f;
                    if (c0 + i < hd) {
                        const float x = type == B200_TYPE_F16
                                            ? __half2float(*reinterpret_cast<const __half*>(rowp + 2 * (c0 + i)))
                                            : *reinterpret_cast<const float*>(rowp + 4 * (c0 + i));
                        f[i] = __fadd_rn(x, __ldg(bias + c0 + i));
                    }
                }
                val.x = pack_half2(f[0], f[1]), val.y = pack_half2(f[2], f[3]);
                val.z = pack_half2(f[4], f[5]), val.w = pack_half2(f[6], f[7]);
            }
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm) + (row * CPR + swz<HD>(row, ch)) * 16) = val;
    }
}

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    return v;
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    return v;
}

// Valid keys of batch entry b: kv_len[b] clamped to the number of logical keys (the rows of K, or the width of the
// index lists when keys are addressed through ext->kv_index).
__device__ __forceinline__ int clamp_len(const FattnArgs& a, int b) {
    const int cap = a.kv_index ? a.kv_index_stride : a.Lk;
    if (!a.kv_len) return cap;
    const int v = a.kv_len[b];
    return v < 0 ? 0 : (v > cap ? cap : v);
}

// ------------------------------------------------------------------------------------------
// General tiled kernel
// ------------------------------------------------------------------------------------------
constexpr int kXStride = 88;  // floats per row of the per-warp bias band buffer (80 used)

template <int HD, bool RELPOS>
__global__ void __launch_bounds__(kThreads) fattn_tile_mma_kernel(const FattnArgs a) {
    constexpr int BM = 64, BN = 64;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);
    __half* sK = sQ + BM * HD;
    __half* sV = sK + BN * HD;
    __half* sQv = sV + BN * HD;                             // RELPOS only
    __half* sR = sQv + BM * HD;                             // RELPOS only, 128 rows
    float* sX = reinterpret_cast<float*>(sR + 128 * HD);    // RELPOS only, [4][16][kXStride]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int q0 = blockIdx.x * BM, h = blockIdx.y, b = blockIdx.z;
    const int hk = h / a.gqa, bk = b / a.bq;
    const float ninf = -INFINITY;
    const int tq_b = q_rows_of(a, b);   // rows at or beyond it are padding of a batched launch: zeros, no work
    if (q0 >= tq_b) {
        for (int idx = tid; idx < BM * a.hd; idx += kThreads) {
            const int iq = q0 + idx / a.hd;
            if (iq < a.Tq) a.dst[(((int64_t)b * a.Tq + iq) * a.H + h) * a.hd + idx % a.hd] = 0.0f;
        }
        return;
    }

    if (RELPOS && a.bias_u != nullptr) {
        // untied position biases folded into the load: Q_u = Q + bias_u, Q_v = Q + bias_v (q_v aliases q)
        const uint8_t* qb = a.q.p + (int64_t)h * a.q.nb2 + (int64_t)b * a.q.nb3;
        load_tile_bias<HD, BM>(sQ, qb, a.q.nb1, a.q.type, a.q.vec16, q0, a.Tq, a.hd, a.bias_u + (int64_t)h * a.hd, tid);
        load_tile_bias<HD, BM>(sQv, qb, a.q.nb1, a.q.type, a.q.vec16, q0, a.Tq, a.hd, a.bias_v + (int64_t)h * a.hd, tid);
    } else {
        load_tile<HD, BM>(sQ, a.q.p + (int64_t)h * a.q.nb2 + (int64_t)b * a.q.nb3, a.q.nb1, a.q.type, a.q.vec16, q0, 0,
                          a.Tq, a.hd, tid);
        if (RELPOS)
            load_tile<HD, BM>(sQv, a.qv.p + (int64_t)h * a.qv.nb2 + (int64_t)b * a.qv.nb3, a.qv.nb1, a.qv.type,
                              a.qv.vec16, q0, 0, a.Tq, a.hd, tid);
    }

    const uint8_t* kbase = a.k.p + (int64_t)hk * a.k.nb2 + (int64_t)bk * a.k.nb3;
    const uint8_t* vbase = a.v.p + (int64_t)hk * a.v.nb2 + (int64_t)bk * a.v.nb3;
    const uint8_t* rbase = RELPOS ? a.r.p + (int64_t)h * a.r.nb2 + (int64_t)(a.r_ne3 > 1 ? b : 0) * a.r.nb3 : nullptr;
    const uint8_t* mbase =
        a.has_mask ? a.mask.p + (int64_t)(h % a.mask_ne2) * a.mask.nb2 + (int64_t)(b % a.mask_ne3) * a.mask.nb3
                   : nullptr;

    const int len_b = clamp_len(a, b);
    int kmax = len_b;
    // causal bound: key k is visible to query q iff k <= n_past + q; in a batched launch with per-entry lengths the
    // new tokens are the last q_len rows of the entry's kv_len keys
    const int n_past = n_past_of(a, len_b, tq_b);
    if (a.causal) {
        const int last_q = min(q0 + BM, tq_b) - 1;
        kmax = min(kmax, n_past + last_q + 1);
    }
    const float slope = alibi_slope(a, h);

    float m_run[2] = {ninf, ninf}, l_run[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    for (int k0 = 0; k0 < kmax; k0 += BN) {
        __syncthreads();
        load_tile<HD, BN>(sK, kbase, a.k.nb1, a.k.type, a.k.vec16, k0, 0, len_b, a.hd, tid);
        load_tile<HD, BN>(sV, vbase, a.v.nb1, a.v.type, a.v.vec16, k0, 0, len_b, a.hd, tid);
        if (RELPOS)
            load_tile<HD, 128>(sR, rbase, a.r.nb1, a.r.type, a.r.vec16, a.Tq - 1 + k0 - q0 - 63, 0, 2 * a.Tq - 1,
                               a.hd, tid);
        __syncthreads();

        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t af[4];
            ldsm_x4(af, tile_addr<HD>(sQ, warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
            for (int np = 0; np < BN / 16; np++) {
                uint32_t bf[4];
                ldsm_x4(bf, tile_addr<HD>(sK, np * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
                mma16816(s[2 * np], af, bf[0], bf[1]);
                mma16816(s[2 * np + 1], af, bf[2], bf[3]);
            }
        }

        float* xw = sX + warp * 16 * kXStride;
        if (RELPOS) {
            // Band GEMM of this warp: X[i][jj] = Q_v[16w+i] . R[rb0 + jj], jj in [0,80), where
            // rb0 = (Tq-1) + k0 - (q0+16w+15) is local row 16*(3-w) of the 128-row R tile;
            // the bias of (row i, key j) is X[i][j + 15 - i].
            float x[10][4];
#pragma unroll
            for (int i = 0; i < 10; i++) x[i][0] = x[i][1] = x[i][2] = x[i][3] = 0.0f;
            const int rrow0 = 16 * (3 - warp);
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) {
                uint32_t af[4];
                ldsm_x4(af, tile_addr<HD>(sQv, warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
                for (int np = 0; np < 5; np++) {
                    uint32_t bf[4];
                    ldsm_x4(bf, tile_addr<HD>(sR, rrow0 + np * 16 + (lane & 7) + ((lane >> 4) << 3),
                                              ks * 2 + ((lane >> 3) & 1)));
                    mma16816(x[2 * np], af, bf[0], bf[1]);
                    mma16816(x[2 * np + 1], af, bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 10; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float val = x[nt][e] * a.relscale;
                    if (!a.relpos_f32) val = __half2float(__float2half_rn(val));
                    xw[(g + ((e >> 1) << 3)) * kXStride + nt * 8 + 2 * t + (e & 1)] = val;
                }
            __syncwarp();
        }

        // scale, softcap, bias, mask, bounds; then to the log2 domain
        float rmax[2] = {ninf, ninf};
#pragma unroll
        for (int nt = 0; nt < BN / 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = g + ((e >> 1) << 3);
                const int j = nt * 8 + 2 * t + (e & 1);
                const int iq = q0 + warp * 16 + i, ik = k0 + j;
                float val = s[nt][e] * a.scale;
                if (a.softcap != 0.0f) val = a.softcap * tanhf(val);
                if (RELPOS) val += xw[i * kXStride + j + 15 - i];
                const bool valid = ik < len_b && (!a.causal || ik <= n_past + iq);
                if (mbase && valid && iq < a.Tq)
                    val += slope * __half2float(*reinterpret_cast<const __half*>(mbase + (int64_t)iq * a.mask.nb1 +
                                                                                 (int64_t)ik * 2));
                val = valid ? val * kLog2e : ninf;
                s[nt][e] = val;
                rmax[e >> 1] = fmaxf(rmax[e >> 1], val);
            }

        float alpha[2], muse[2];
#pragma unroll
        for (int rI = 0; rI < 2; rI++) {
            const float mnew = fmaxf(m_run[rI], quad_max(rmax[rI]));
            muse[rI] = mnew == ninf ? 0.0f : mnew;
            alpha[rI] = exp2f(m_run[rI] - muse[rI]);
            m_run[rI] = mnew;
            l_run[rI] *= alpha[rI];
        }
#pragma unroll
        for (int nt = 0; nt < BN / 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = fast_ex2(s[nt][e] - muse[e >> 1]);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            o[i][0] *= alpha[0];
            o[i][1] *= alpha[0];
            o[i][2] *= alpha[1];
            o[i][3] *= alpha[1];
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; kk++) {
            uint32_t pf[4];
            pf[0] = pack_half2(s[2 * kk][0], s[2 * kk][1]);
            pf[1] = pack_half2(s[2 * kk][2], s[2 * kk][3]);
            pf[2] = pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pf[3] = pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < HD / 16; np++) {
                uint32_t bf[4];
                ldsm_x4_t(bf, tile_addr<HD>(sV, kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
                mma16816(o[2 * np], pf, bf[0], bf[1]);
                mma16816(o[2 * np + 1], pf, bf[2], bf[3]);
            }
        }
    }

    const float l0 = quad_sum(l_run[0]), l1 = quad_sum(l_run[1]);
    const float inv0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
#pragma unroll
    for (int rI = 0; rI < 2; rI++) {
        const int iq = q0 + warp * 16 + g + rI * 8;
        if (iq >= a.Tq) continue;
        float* out = a.dst + (((int64_t)b * a.Tq + iq) * a.H + h) * a.hd;
        const float inv = rI ? inv1 : inv0;
        const bool live = iq < tq_b;   // padding rows get literal zeros, whatever their Q rows held
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++) {
            const int c = nt * 8 + 2 * t;
            if (c < a.hd) out[c] = live ? o[nt][2 * rI] * inv : 0.0f;
            if (c + 1 < a.hd) out[c + 1] = live ? o[nt][2 * rI + 1] * inv : 0.0f;
        }
    }
}

template <int HD, bool RELPOS>
int launch_tile_t(const FattnArgs& a, cudaStream_t st) {
    size_t smem = (size_t)(64 + 64 + 64) * HD * sizeof(__half);
    if (RELPOS) smem += (size_t)(64 + 128) * HD * sizeof(__half) + 4 * 16 * kXStride * sizeof(float);
    auto kern = fattn_tile_mma_kernel<HD, RELPOS>;
    static bool smem_set[64] = {false};
    cudaError_t e = set_smem_once(kern, smem, smem_set);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((a.Tq + 63) / 64, a.H, a.B);
    kern<<<grid, kThreads, smem, st>>>(a);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// Split-KV decode kernel
// ------------------------------------------------------------------------------------------
constexpr int kDecRows = 16;
constexpr int kDecBN = 64;
constexpr int kDecQ8Stages = 2;   // raw Q8_0 tile stages per warp; small footprint: four CTAs per SM hide the latency

// How a decode CTA brings K/V tiles into shared memory.
enum DecodeMode {
    kDecSync = 0,    // element loads + conversion (F32 K/V, unaligned or gapped layouts)
    kDecAsyncF16 = 1,  // cp.async 16-byte copies of F16 rows into a multi-stage ring
    kDecAsyncQ8 = 2,   // bulk copy of the raw Q8_0 byte range of a tile, then a shared-to-shared dequantise (head_dim 32)
    kDecRegQ8 = 3      // bulk copy of the raw Q8_0 bytes, dequantised in registers (head_dim 64 / 128)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;  // src-size 0 zero-fills the 16 destination bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// cp.async copy of rows [row0, row0+64) x HD halves into a swizzled fp16 tile; rows >= row_hi are zero-filled.
// IDX: logical row `grow` lives in cache row index[grow] (clamped to the pool): the gather of ext->kv_index.
template <int HD, bool IDX = false>
__device__ __forceinline__ void issue_tile_f16(__half* sm, const uint8_t* base, int64_t nb1, int row0, int row_hi, int tid,
                                               const int32_t* index = nullptr, int pool_rows = 0) {
    constexpr int CPR = HD / 8;
#pragma unroll
    for (int it = 0; it < kDecBN * CPR / kThreads; it++) {
        const int idx = tid + it * kThreads;
        const int row = idx / CPR, ch = idx % CPR;
        const int grow = row0 + row;
        const bool valid = grow < row_hi;
        int src = grow;
        if (IDX && valid) src = min(max(__ldg(index + grow), 0), pool_rows - 1);
        cp_async16(tile_addr<HD>(sm, row, ch), base + (valid ? (int64_t)src * nb1 + ch * 16 : 0), valid);
    }
}

// The same copy for a gathered tile whose cache rows were looked up one tile ahead: `pre[it]` is the cache row of
// this thread's it-th 16-byte piece (see load_tile_index), so the copies do not wait for the list.
template <int HD>
__device__ __forceinline__ void load_tile_index(int (&pre)[kDecBN * (HD / 8) / kThreads], const int32_t* index, int row0, int row_hi,
                                                int tid) {
    constexpr int CPR = HD / 8;
#pragma unroll
    for (int it = 0; it < kDecBN * CPR / kThreads; it++) {
        const int grow = row0 + (tid + it * kThreads) / CPR;
        pre[it] = grow < row_hi ? __ldg(index + grow) : 0;   // clamped where it is used: nothing here waits for the load
    }
}
template <int HD>
__device__ __forceinline__ void issue_tile_f16_pre(__half* sm, const uint8_t* base, int64_t nb1, int row0, int row_hi, int tid,
                                                   const int (&pre)[kDecBN * (HD / 8) / kThreads], int pool_rows) {
    constexpr int CPR = HD / 8;
#pragma unroll
    for (int it = 0; it < kDecBN * CPR / kThreads; it++) {
        const int idx = tid + it * kThreads;
        const int row = idx / CPR, ch = idx % CPR;
        const bool valid = row0 + row < row_hi;
        cp_async16(tile_addr<HD>(sm, row, ch), base + (valid ? (int64_t)min(max(pre[it], 0), pool_rows - 1) * nb1 + ch * 16 : 0), valid);
    }
}

// ---- bulk copies (one instruction per contiguous range) with a per-warp mbarrier per stage ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: a copy that never lands ends the wait after about a second.  Called by all lanes of a warp on the warp's
// own barrier; the result is warp-uniform (a phase one lane saw complete is complete).  On expiry the device status
// word is set (b200_device_status reports B200_E_DEVICE_WAIT) and the caller stops consuming tiles.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = 1u << 22) {
    bool ok = false;
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) {
            ok = true;
            break;
        }
        if (it > 64) __nanosleep(64);
    }
    ok = __any_sync(0xffffffffu, ok);
    if (!ok && (threadIdx.x & 31) == 0) atomicExch(&g_mma_status, 1);
    return ok;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// Raw bytes of this warp's 16 Q8_0 rows [row0 + 16*warp, +16) of a 64-row K tile and V tile: two contiguous,
// 16-byte aligned ranges of at most 16 * (HD/32*34) bytes, one bulk copy each, issued by lane 0.  Only the bytes of
// rows below row_hi are requested (rounded up to 16: the same footprint as 16-byte chunk copies; the rest of the
// stage keeps old bytes, which the dequantiser replaces by zeros).  Each warp copies, dequantises and multiplies
// only its own keys.
template <int HD>
__device__ __forceinline__ void issue_tile_q8raw(uint8_t* smK, uint8_t* smV, const uint8_t* kbase, const uint8_t* vbase, int row0,
                                                 int row_hi, int warp, uint32_t bar) {
    constexpr int RB = HD / 32 * 34;
    const int r0 = row0 + 16 * warp;
    const int n = min(16, max(0, row_hi - r0));
    const uint32_t bytes = (uint32_t)((n * RB + 15) / 16 * 16);
    mbar_expect_tx(bar, 2 * bytes);
    if (bytes) {
        bulk_g2s(smem_u32(smK) + 16 * warp * RB, kbase + (int64_t)r0 * RB, bytes, bar);
        bulk_g2s(smem_u32(smV) + 16 * warp * RB, vbase + (int64_t)r0 * RB, bytes, bar);
    }
}

// Raw Q8_0 tile (64 rows of HD/32 blocks) in shared memory -> swizzled fp16 tile. x = fp16(d * q): the product of
// an 11-bit and a 7-bit significand is exact before the single rounding, i.e. equal to fp32(d)*q rounded to fp16.
template <int HD>
__device__ __forceinline__ void dequant_tile_q8(const uint8_t* raw, __half* sm, int rows_valid, int warp, int lane) {
    constexpr int NBLK = HD / 32, RB = NBLK * 34;
    // this warp's 16 rows x NBLK blocks, one block per lane and step
#pragma unroll
    for (int idx0 = 0; idx0 < 16 * NBLK; idx0 += 32) {
        const int idx = idx0 + lane;
        if (16 * NBLK < 32 && idx >= 16 * NBLK) break;   // head_dim 32: one block per row, half of the lanes idle
        const int row = 16 * warp + idx / NBLK, blk = idx % NBLK;
        const uint16_t* src = reinterpret_cast<const uint16_t*>(raw + row * RB + blk * 34);
        if (row >= rows_valid) {  // rows past the valid length read as zeros whatever the copy brought in
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++)
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm) + (row * (HD / 8) + swz<HD>(row, blk * 4 + c4)) * 16) =
                    make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        const __half2 d2 = __half2half2(*reinterpret_cast<const __half*>(src));
        const __half2 bias = __float2half2_rn(1152.0f);
        // The 32 quants start 2 bytes into the block. Read aligned 32-bit words and realign with a funnel shift:
        // block offset = 0 mod 4 -> word 0 holds {d, q0, q1} and the quants straddle words (shift 16);
        // block offset = 2 mod 4 -> the quants start on the next word boundary (shift 0).
        const uint32_t o = (uint32_t)(row * RB + blk * 34);
        const uint32_t sh = (o >> 1) & 1u;
        const uint32_t* W = reinterpret_cast<const uint32_t*>(raw + (o & ~3u) + 4u * sh);
        uint32_t w[9];
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = W[i];
        w[8] = sh ? 0u : W[8];
        const uint32_t fs = 16u * (1u - sh);
        uint32_t out[16];
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
            const uint32_t win = __funnelshift_r(w[kk], w[kk + 1], fs) ^ 0x80808080u;  // four int8 -> biased uint8
            // halves 0x64xx = 1024 + xx; minus 1152 gives the signed value exactly; times d rounds once
            const uint32_t h01 = __byte_perm(win, 0x64646464u, 0x4140), h23 = __byte_perm(win, 0x64646464u, 0x4342);
            const __half2 v01 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&h01), bias), d2);
            const __half2 v23 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&h23), bias), d2);
            out[2 * kk] = *reinterpret_cast<const uint32_t*>(&v01);
            out[2 * kk + 1] = *reinterpret_cast<const uint32_t*>(&v23);
        }
#pragma unroll
        for (int c4 = 0; c4 < 4; c4++)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sm) + (row * (HD / 8) + swz<HD>(row, blk * 4 + c4)) * 16) =
                make_uint4(out[4 * c4], out[4 * c4 + 1], out[4 * c4 + 2], out[4 * c4 + 3]);
    }
}

// PLAIN: no explicit mask, no softcap, no causal bound: only kv_len limits the keys (its own instantiation).
// LOW (with STAGE_MASK or PLAIN): at most 8 live rows, so rows g+8 of every fragment are padding and skipped.
// ---- split merge inside a thread-block cluster ------------------------------------------------------------------
// When the splits of one (batch entry, kv-head) are launched as one cluster (n_splits <= 8), no workspace and no
// merge kernel are needed: every CTA leaves its partial (O scaled to its own row maxima, m, l) in its shared
// memory, the cluster meets at its hardware barrier, and each CTA finishes a slice of the output rows by reading
// all peers' partials through distributed shared memory.  A second barrier keeps every CTA's shared memory alive
// until its peers are done reading.
__device__ __forceinline__ uint32_t peer_addr(const void* p, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(p)), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_peer_v4(uint32_t remote, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(remote), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void st_peer_v2(uint32_t remote, float x, float y) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" :: "r"(remote), "f"(x), "f"(y) : "memory");
}
// A split kernel launched as clusters says "this CTA runs" at its start; the write-out waits for that phase before its
// first store into a peer's shared memory.
__device__ __forceinline__ void cluster_announce(const FattnArgs& a) {
    if (a.n_splits > 1 && a.cluster_merge) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}

// Row rr of a KV head's packed query rows is (query position iq, head hq) with rr = iq * gqa + (hq - hk * gqa).  One
// query head per KV head, or one new token per step, need no division - and a decode CTA runs this code once, at
// instruction-fetch pace.
__device__ __forceinline__ void row_to_query(const FattnArgs& a, int hk, int rr, int& iq, int& hq) {
    if (a.gqa == 1) iq = rr, hq = hk;
    else if (a.Tq == 1) iq = 0, hq = hk * a.gqa + rr;
    else iq = rr / a.gqa, hq = hk * a.gqa + rr % a.gqa;
}

// Receive area of the merge inside a cluster: shared memory of its own behind a kernel's stages (a peer may push while
// this CTA is still in its key loop): [n_splits][slots] 16-byte column groups this CTA owns (rows * hd / 4 of them over the
// cluster, rounded up per split), then [8][16] (M, L).
// `rows` = the launch's query rows per KV head (Tq * gqa).
__host__ __device__ constexpr size_t cluster_push_bytes(int hd, int rows) { return (size_t)(rows * (hd / 4) + 8) * 16 + 8 * kDecRows * 8; }

// Write-out shared by the split-KV decode kernels.  `slab` holds the four warps' partial O [4][16][HD + 4], each scaled
// to its own warp's running maximum s_m[w][row] with row sum s_l[w][row]; the CTA has passed a barrier since they were
// written.  One warp per live row, one 16-byte column group per lane, the log-sum-exp merge of the four partials on
// the way; the result goes
//   * n_splits == 1: to dst, divided by the row sum;
//   * workspace form: to this split's [16][HD] partial and (M, L) pairs, for the merge kernel;
//   * cluster form: the column groups of the R x HD result are dealt round-robin to the CTAs of the cluster; every CTA
//     stores its partial of a group into the OWNER's receive area (and its (M, L) into everybody's), one cluster
//     barrier later each owner merges what it received from its own shared memory and writes the rows.  One barrier and
//     no remote load on the critical path; the first form of this merge (barrier, every CTA pulls 3 n_splits values per
//     element from its peers, barrier) took 4.0 k of a 13.7 k clk CTA at 8 streams of the Q8_0 cache, this one 2.0 k.
// A CTA with two or three tiles shares its SM with few others, but at the usual 256-stream size three neighbours are
// in their key loops and every dependent step of a tail waits for an issue slot, so the chain is kept short: no
// separate pass for the common maximum, no index division per element.
template <int HD>
__device__ __forceinline__ void decode_write_out(const FattnArgs& a, const float* slab, const float (*s_m)[kDecRows],
                                                 const float (*s_l)[kDecRows], uint8_t* recv, int R, int b, int hk, int split,
                                                 int tq_b, int tid) {
    constexpr int STRIDE = HD + 4, G = HD / 4;
    const int warp = tid >> 5, lane = tid & 31;
    const float ninf = -INFINITY;
    const bool push = a.n_splits > 1 && a.cluster_merge;
    float4* recv_o = reinterpret_cast<float4*>(recv);
    float2* recv_ml = reinterpret_cast<float2*>(recv_o + (R * G + 8));
    const int n_groups = R * G, slots = (n_groups + a.n_splits - 1) / a.n_splits;
    if (push) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // every CTA of the cluster has started
    for (int rr = warp; rr < R; rr += 4) {
        const float m0 = s_m[0][rr], m1 = s_m[1][rr], m2 = s_m[2][rr], m3 = s_m[3][rr];
        const float l0 = s_l[0][rr], l1 = s_l[1][rr], l2 = s_l[2][rr], l3 = s_l[3][rr];
        const float M = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        const float w0 = m0 == ninf ? 0.0f : fast_ex2(m0 - M), w1 = m1 == ninf ? 0.0f : fast_ex2(m1 - M);
        const float w2 = m2 == ninf ? 0.0f : fast_ex2(m2 - M), w3 = m3 == ninf ? 0.0f : fast_ex2(m3 - M);
        const float L = (w0 * l0 + w1 * l1) + (w2 * l2 + w3 * l3);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane < G) {
            const float4 x0 = *reinterpret_cast<const float4*>(slab + (0 * kDecRows + rr) * STRIDE + 4 * lane);
            const float4 x1 = *reinterpret_cast<const float4*>(slab + (1 * kDecRows + rr) * STRIDE + 4 * lane);
            const float4 x2 = *reinterpret_cast<const float4*>(slab + (2 * kDecRows + rr) * STRIDE + 4 * lane);
            const float4 x3 = *reinterpret_cast<const float4*>(slab + (3 * kDecRows + rr) * STRIDE + 4 * lane);
            // a warp that saw no live key holds zeros and weight 0
            v.x = (w0 * x0.x + w1 * x1.x) + (w2 * x2.x + w3 * x3.x), v.y = (w0 * x0.y + w1 * x1.y) + (w2 * x2.y + w3 * x3.y);
            v.z = (w0 * x0.z + w1 * x1.z) + (w2 * x2.z + w3 * x3.z), v.w = (w0 * x0.w + w1 * x1.w) + (w2 * x2.w + w3 * x3.w);
        }
        if (a.n_splits == 1) {
            int iq, hq;
            row_to_query(a, hk, rr, iq, hq);
            const float inv = (L > 0.0f && iq < tq_b) ? 1.0f / L : 0.0f;
            float* drow = a.dst + (((int64_t)b * a.Tq + iq) * a.H + hq) * a.hd;
            if (lane < G) {
                if (a.hd == HD) {
                    *reinterpret_cast<float4*>(drow + 4 * lane) = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
                } else {   // a head dim padded up to HD: the row is a.hd floats long
                    const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (4 * lane + j < a.hd) drow[4 * lane + j] = vv[j] * inv;
                }
            }
        } else if (a.cluster_merge) {
            if (lane < G) {
                const int grp = rr * G + lane;   // owner grp % n_splits, its slot grp / n_splits
                st_peer_v4(peer_addr(recv_o + split * slots + grp / a.n_splits, grp % a.n_splits), v);
            }
            if (lane < a.n_splits) st_peer_v2(peer_addr(recv_ml + split * kDecRows + rr, lane), M, L);
        } else {
            const int64_t unit = ((int64_t)b * a.Hkv + hk) * a.n_splits + split;
            if (lane < G) *reinterpret_cast<float4*>(a.ws_o + unit * kDecRows * HD + rr * HD + 4 * lane) = v;   // live rows only: the merge kernel reads no others
            if (lane == 0) a.ws_ml[(unit * kDecRows + rr) * 2] = M, a.ws_ml[(unit * kDecRows + rr) * 2 + 1] = L;
        }
    }
    if (push) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        for (int pos = tid; pos * a.n_splits + split < n_groups; pos += kThreads) {
            const int grp = pos * a.n_splits + split, rr = grp / G, cg = grp % G;
            float2 ml[8];
            float M = ninf;
#pragma unroll
            for (int s = 0; s < 8; s++) {
                ml[s] = make_float2(ninf, 0.0f);
                if (s < a.n_splits) ml[s] = recv_ml[s * kDecRows + rr];
                M = fmaxf(M, ml[s].x);
            }
            float L = 0.0f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < 8; s++) {
                if (s < a.n_splits && ml[s].x != ninf) {   // a split that saw no live key holds zeros
                    const float w = fast_ex2(ml[s].x - M);
                    const float4 x = recv_o[s * slots + pos];
                    L = fmaf(w, ml[s].y, L);
                    acc.x = fmaf(w, x.x, acc.x), acc.y = fmaf(w, x.y, acc.y), acc.z = fmaf(w, x.z, acc.z), acc.w = fmaf(w, x.w, acc.w);
                }
            }
            int iq, hq;
            row_to_query(a, hk, rr, iq, hq);
            const float inv = (L > 0.0f && iq < tq_b) ? 1.0f / L : 0.0f;
            *reinterpret_cast<float4*>(a.dst + (((int64_t)b * a.Tq + iq) * a.H + hq) * HD + 4 * cg) =
                make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);   // the cluster form is offered for a.hd == HD only
        }
    }
}

// IDX (F16 ring; PLAIN or STAGE_MASK): keys are gathered through ext->kv_index (one list per batch entry); an explicit
// mask is then indexed by the logical key, like the list.
template <int HD, int MODE, bool STAGE_MASK = false, bool PLAIN = false, bool LOW = false, bool IDX = false>
__global__ void __launch_bounds__(kThreads, MODE == kDecAsyncQ8 ? 4 : 1) fattn_decode_split_kernel(const FattnArgs a) {
    constexpr int NR = LOW ? 1 : 2, NE = 2 * NR;   // live row halves / accumulator elements per n-tile
    constexpr int TILE_HALVES = kDecBN * HD;              // one fp16 K or V tile
    constexpr int RAW_BYTES = kDecBN * (HD / 32 * 34);    // one raw Q8_0 K or V tile
    constexpr int NS = MODE == kDecSync ? 1 : (MODE == kDecAsyncF16 ? (HD >= 128 ? 3 : 4) : kDecQ8Stages);
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);              // [16][HD]
    // fp16 tiles: NS stages (async F16) or one pair (sync, Q8)
    __half* sKV = sQ + kDecRows * HD;
    constexpr int F16_STAGES = MODE == kDecAsyncF16 ? NS : 1;
    constexpr int F16_TILES = MODE == kDecAsyncQ8 ? 1 : F16_STAGES * 2;   // Q8: K and V take turns in one fp16 tile
    uint8_t* sRaw = reinterpret_cast<uint8_t*>(sKV + F16_TILES * TILE_HALVES);  // Q8: NS stages of raw K|V
    // F16 ring + explicit mask with 16-byte aligned rows: the mask values of a tile (R rows x 64 keys) travel with
    // the K/V tile through the same cp.async stage, so the softmax reads them from shared memory instead of
    // stalling on global loads issued right before their use.
    constexpr bool stage_mask = STAGE_MASK;   // separate instantiation: the maskless kernel carries none of it
    __half* sMask = reinterpret_cast<__half*>(sRaw);   // [NS][R][64] (F16 ring mode has no raw stages)
    __shared__ float s_m[4][kDecRows], s_l[4][kDecRows];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int bk = b / a.bq;
    const int R = a.Tq * a.gqa;  // <= 16; row rr -> (iq = rr / gqa, head hk*gqa + rr % gqa)
    const float ninf = -INFINITY;
    cluster_announce(a);

    const uint8_t* kbase = a.k.p + (int64_t)hk * a.k.nb2 + (int64_t)bk * a.k.nb3;
    const uint8_t* vbase = a.v.p + (int64_t)hk * a.v.nb2 + (int64_t)bk * a.v.nb3;
    const int32_t* index = a.kv_index ? a.kv_index + (int64_t)b * a.kv_index_stride : nullptr;   // this entry's key list

    __shared__ __align__(8) uint64_t s_q8bar[4][kDecQ8Stages];   // Q8_0: one barrier per (warp, raw stage)
    if (MODE == kDecAsyncQ8) {
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < kDecQ8Stages; i++) mbar_init(smem_u32(&s_q8bar[warp][i]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
    }
    // Launched with programmatic stream serialisation: everything above (kernel parameters, this CTA's own shared
    // memory) ran while the previous kernel of the stream drained; from here on that kernel has completed and flushed
    // (a no-op under an ordinary launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int len_b = clamp_len(a, b);
    const int tq_b = q_rows_of(a, b);   // query rows at or beyond it give zeros
    int kmax = tq_b > 0 ? len_b : 0;    // an entry without live rows reads no keys
    const int n_past = n_past_of(a, len_b, tq_b);
    if (a.causal) kmax = min(kmax, n_past + tq_b);
    const int n_tiles = (kmax + kDecBN - 1) / kDecBN;
    const int tps = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int tile_lo = split * tps, tile_hi = min(n_tiles, tile_lo + tps);
    // staged mask: the row of the mask this thread copies pieces of (the head and batch broadcasts are remainders by
    // run-time values: computed once, not per tile)
    const int n_logical = a.kv_index ? a.kv_index_stride : a.Lk;   // a mask row holds one value per logical key
    const uint8_t* mask_row = nullptr;
    if (stage_mask && tid < R * 8) {
        int iq, hq;
        row_to_query(a, hk, tid >> 3, iq, hq);
        mask_row = a.mask.p + (int64_t)iq * a.mask.nb1 + (int64_t)(hq % a.mask_ne2) * a.mask.nb2 + (int64_t)(b % a.mask_ne3) * a.mask.nb3;
    }
    int pre_rows[kDecBN * (HD / 8) / kThreads];   // gathered keys: this thread's cache rows of the next tile to be issued
    if (IDX && tile_lo < tile_hi) load_tile_index<HD>(pre_rows, index, tile_lo * kDecBN, len_b, tid);
    auto issue = [&](int tile) {
        if (MODE == kDecAsyncQ8) {
            if (tile < tile_hi && lane == 0) {
                const int stage = (tile - tile_lo) % NS;
                issue_tile_q8raw<HD>(sRaw + stage * 2 * RAW_BYTES, sRaw + stage * 2 * RAW_BYTES + RAW_BYTES, kbase, vbase,
                                     tile * kDecBN, len_b, warp, smem_u32(&s_q8bar[warp][stage]));
            }
            return;
        }
        if (tile < tile_hi) {
            const int stage = (tile - tile_lo) % NS;
            if (IDX) {
                // tiles are issued in order: the list entries of this one were requested when the previous one was issued
                issue_tile_f16_pre<HD>(sKV + stage * 2 * TILE_HALVES, kbase, a.k.nb1, tile * kDecBN, len_b, tid, pre_rows, a.Lk);
                issue_tile_f16_pre<HD>(sKV + stage * 2 * TILE_HALVES + TILE_HALVES, vbase, a.v.nb1, tile * kDecBN, len_b, tid, pre_rows, a.Lk);
                if (tile + 1 < tile_hi) load_tile_index<HD>(pre_rows, index, (tile + 1) * kDecBN, len_b, tid);
            } else {
                issue_tile_f16<HD, false>(sKV + stage * 2 * TILE_HALVES, kbase, a.k.nb1, tile * kDecBN, len_b, tid);
                issue_tile_f16<HD, false>(sKV + stage * 2 * TILE_HALVES + TILE_HALVES, vbase, a.v.nb1, tile * kDecBN, len_b, tid);
            }
            if (stage_mask && tid < R * 8) {
                const int rr = tid >> 3, ch = tid & 7;
                const int key0 = tile * kDecBN + ch * 8;
                const int nbytes = max(0, min(8, n_logical - key0)) * 2;          // the rest reads as 0
                const uint8_t* src = mask_row + (int64_t)(nbytes ? key0 : 0) * 2;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(sMask + ((stage * R + rr) * kDecBN + ch * 8))),
                             "l"(src), "r"(nbytes)
                             : "memory");
            }
        }
        cp_async_commit();
    };
    if (MODE != kDecSync) {
#pragma unroll
        for (int s0 = 0; s0 < NS - 1; s0++) issue(tile_lo + s0);
    }

    // Q rows (tiny): one 8-element chunk per loop step
    for (int idx = tid; idx < kDecRows * (HD / 8); idx += kThreads) {
        const int rr = idx / (HD / 8), ch = idx % (HD / 8);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (rr < R) {
            int iq, hq;
            row_to_query(a, hk, rr, iq, hq);
            val = load8_as_half(a.q.p + (int64_t)iq * a.q.nb1 + (int64_t)hq * a.q.nb2 + (int64_t)b * a.q.nb3,
                                a.q.type, ch * 8, a.hd, a.q.vec16);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sQ) + (rr * (HD / 8) + swz<HD>(rr, ch)) * 16) = val;
    }
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) ldsm_x4(qf[ks], tile_addr<HD>(sQ, lane & 15, ks * 2 + (lane >> 4)));

    // per-thread row metadata for rows g and g+8
    int row_iq[2] = {0, 0};
    float row_slope[2] = {1.0f, 1.0f};
    const uint8_t* row_mask[2] = {nullptr, nullptr};
#pragma unroll
    for (int rI = 0; rI < 2 && !PLAIN && !STAGE_MASK; rI++) {
        const int rr = g + rI * 8;
        row_iq[rI] = rr / a.gqa;
        const int hq = hk * a.gqa + rr % a.gqa;
        row_slope[rI] = alibi_slope(a, hq);
        row_mask[rI] = (a.has_mask && rr < R)
                           ? a.mask.p + (int64_t)row_iq[rI] * a.mask.nb1 + (int64_t)(hq % a.mask_ne2) * a.mask.nb2 +
                                 (int64_t)(b % a.mask_ne3) * a.mask.nb3
                           : nullptr;
    }

    float m_run[2] = {ninf, ninf}, l_run[2] = {0.0f, 0.0f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

    for (int tile = tile_lo; tile < tile_hi; tile++) {
        const int k0 = tile * kDecBN;
        const __half *sK, *sV;
        if (MODE == kDecSync) {
            __syncthreads();
            load_tile<HD, kDecBN>(sKV, kbase, a.k.nb1, a.k.type, a.k.vec16, k0, 0, len_b, a.hd, tid, index, a.Lk);
            load_tile<HD, kDecBN>(sKV + TILE_HALVES, vbase, a.v.nb1, a.v.type, a.v.vec16, k0, 0, len_b, a.hd, tid, index, a.Lk);
            __syncthreads();
            sK = sKV, sV = sKV + TILE_HALVES;
        } else if (MODE == kDecAsyncF16) {
            cp_async_wait<NS - 2>();
            __syncthreads();             // tile `tile` has landed for every thread; stage of tile-1 is free
            issue(tile + NS - 1);
            const int stage = (tile - tile_lo) % NS;
            sK = sKV + stage * 2 * TILE_HALVES, sV = sK + TILE_HALVES;
        } else {
            // Warp-local pipeline: a warp only ever touches its own 16 keys of a tile (raw bytes, fp16 rows, MMA
            // operands), so the key loop needs no CTA-wide barrier and the four warps drift apart freely - one
            // waits for its copy while another dequantises or multiplies.
            const int stage = (tile - tile_lo) % NS;
            if (!mbar_wait_bounded(smem_u32(&s_q8bar[warp][stage]), (uint32_t)((tile - tile_lo) / NS) & 1u)) break;
            __syncwarp();                // this warp's raw rows landed; its previous fp16 rows have been consumed
            dequant_tile_q8<HD>(sRaw + stage * 2 * RAW_BYTES, sKV, len_b - k0, warp, lane);
            __syncwarp();
            sK = sKV, sV = sKV;          // V is dequantised into the same rows once the scores are in registers
        }

        // this warp's 16 keys: k0 + 16*warp ..
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t bf[4];
            ldsm_x4(bf, tile_addr<HD>(sK, warp * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
            mma16816(s[0], qf[ks], bf[0], bf[1]);
            mma16816(s[1], qf[ks], bf[2], bf[3]);
        }
        if (MODE == kDecAsyncQ8) {
            __syncwarp();                // every lane has read its K fragments
            const int stage = (tile - tile_lo) % NS;
            dequant_tile_q8<HD>(sRaw + stage * 2 * RAW_BYTES + RAW_BYTES, sKV, len_b - k0, warp, lane);
            __syncwarp();
            issue(tile + NS - 1);        // overwrites the raw stage of tile-1, which this warp dequantised an iteration ago
        }
        float rmax[2] = {ninf, ninf};
        // common case (no mask, no softcap, every key of the tile visible to every row): one multiply per score
        const bool plain_tile = STAGE_MASK ? false : PLAIN ? (k0 + kDecBN <= len_b)
                                      : (!a.has_mask && a.softcap == 0.0f && k0 + kDecBN <= len_b && (!a.causal || k0 + kDecBN <= n_past + 1));
        if (plain_tile) {
            const float c = a.scale * kLog2e;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    s[nt][e] *= c;
                    rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
                }
        } else if (PLAIN) {   // last tile of the valid range
            const float c = a.scale * kLog2e;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    const int ik = k0 + warp * 16 + nt * 8 + 2 * t + (e & 1);
                    s[nt][e] = ik < len_b ? s[nt][e] * c : ninf;
                    rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
                }
        } else if (STAGE_MASK) {
            // this instantiation is only launched without softcap, ALiBi and causal bound: logit = s*scale + mask
            const float c = a.scale * kLog2e;
            const __half* mt = sMask + ((tile - tile_lo) % NS) * R * kDecBN + warp * 16 + 2 * t;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int rI = 0; rI < NR; rI++) {
                    const int rr = g + rI * 8, ik = k0 + warp * 16 + nt * 8 + 2 * t;
                    float2 m2 = make_float2(0.0f, 0.0f);
                    if (rr < R) m2 = __half22float2(*reinterpret_cast<const __half2*>(mt + rr * kDecBN + nt * 8));
                    const float v0 = ik < len_b ? fmaf(s[nt][2 * rI], c, m2.x * kLog2e) : ninf;
                    const float v1 = ik + 1 < len_b ? fmaf(s[nt][2 * rI + 1], c, m2.y * kLog2e) : ninf;
                    s[nt][2 * rI] = v0, s[nt][2 * rI + 1] = v1;
                    rmax[rI] = fmaxf(rmax[rI], fmaxf(v0, v1));
                }
        } else
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int rI = e >> 1;
                const int ik = k0 + warp * 16 + nt * 8 + 2 * t + (e & 1);
                float val = s[nt][e] * a.scale;
                if (a.softcap != 0.0f) val = a.softcap * tanhf(val);
                const bool valid = ik < len_b && (!a.causal || ik <= n_past + row_iq[rI]);
                if (row_mask[rI] && valid)
                    val += row_slope[rI] * __half2float(*reinterpret_cast<const __half*>(row_mask[rI] + (int64_t)ik * 2));
                val = valid ? val * kLog2e : ninf;
                s[nt][e] = val;
                rmax[rI] = fmaxf(rmax[rI], val);
            }
        // Lazy rescale: m_run is a reference, not the exact running maximum - it is only raised (and O, l rescaled)
        // when a row's tile maximum outgrew it by 2^8, so P <= 256 stays inside f16 and most tiles skip the rescale.
        float alpha[2] = {1.0f, 1.0f}, muse[2] = {0.0f, 0.0f};
#pragma unroll
        for (int rI = 0; rI < NR; rI++) {
            const float mt = quad_max(rmax[rI]);
            const float mnew = (mt > m_run[rI] + 8.0f) ? mt : m_run[rI];   // -inf + 8 = -inf: the first finite maximum is taken
            muse[rI] = mnew == ninf ? 0.0f : mnew;
            alpha[rI] = (mnew == m_run[rI]) ? 1.0f : exp2f(m_run[rI] - muse[rI]);
            m_run[rI] = mnew;
            l_run[rI] *= alpha[rI];
        }
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (e >= NE) {
                    s[nt][e] = 0.0f;   // padding rows: P = 0
                    continue;
                }
                const float p = fast_ex2(s[nt][e] - muse[e >> 1]);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
        uint32_t pf[4];
        pf[0] = pack_half2(s[0][0], s[0][1]);
        pf[1] = pack_half2(s[0][2], s[0][3]);
        pf[2] = pack_half2(s[1][0], s[1][1]);
        pf[3] = pack_half2(s[1][2], s[1][3]);
        // the running maxima settle after a few tiles: the accumulator is only rescaled when some row of the warp moved
        if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < HD / 8; i++) o[i][0] *= alpha[0], o[i][1] *= alpha[0], o[i][2] *= alpha[1], o[i][3] *= alpha[1];
        }
#pragma unroll
        for (int np = 0; np < HD / 16; np++) {
            uint32_t bf[4];
            ldsm_x4_t(bf, tile_addr<HD>(sV, warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), np * 2 + (lane >> 4)));
            mma16816(o[2 * np], pf, bf[0], bf[1]);
            mma16816(o[2 * np + 1], pf, bf[2], bf[3]);
        }
    }
    if (MODE == kDecAsyncF16) cp_async_wait<0>();

    // the merge kernel (if any) may start launching: it waits for this grid's completion before reading anything
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- merge the four warps' (m, l, O) in shared memory ----
    constexpr int SLAB_STRIDE = HD + 4;
    float* slab = reinterpret_cast<float*>(smem_raw);   // [4][16][SLAB_STRIDE]
    {
        const float lq[2] = {quad_sum(l_run[0]), quad_sum(l_run[1])};
        if (t == 0) {   // static shared memory: written before the barrier that retires the tiles
            s_m[warp][g] = m_run[0], s_m[warp][g + 8] = m_run[1];
            s_l[warp][g] = lq[0], s_l[warp][g + 8] = lq[1];
        }
    }
    __syncthreads();  // all warps are done with the K/V tiles; the warps' (m, l) are visible
    // Each warp parks its partial O as it is, scaled to its OWN running maximum, in its own padded slab (the slabs start
    // at the base of dynamic shared memory - Q and the tiles are dead by now): a thread's accumulators of one n-tile are
    // two consecutive dims of rows g and g + 8, one 8-byte store each; rows at or beyond R are never read.
    // (Shared-memory atomics on one [16][HD] array serialised the four warps and cost about 15 us per launch when a
    // CTA has a single tile.)
#pragma unroll
    for (int rI = 0; rI < NR; rI++) {
        if (g + rI * 8 >= R) continue;
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++)
            *reinterpret_cast<float2*>(slab + (warp * kDecRows + g + rI * 8) * SLAB_STRIDE + nt * 8 + 2 * t) =
                make_float2(o[nt][2 * rI], o[nt][2 * rI + 1]);
    }
    __syncthreads();
    decode_write_out<HD>(a, slab, s_m, s_l, reinterpret_cast<uint8_t*>(sRaw) + (MODE == kDecAsyncQ8 ? NS * 2 * RAW_BYTES : (stage_mask ? NS * R * kDecBN * (int)sizeof(__half) : 0)), R, b, hk, split, tq_b, tid);
}

// ------------------------------------------------------------------------------------------
// Split-KV decode over a Q8_0 cache, dequantised in registers
// ------------------------------------------------------------------------------------------
// The raw 34-byte blocks go from HBM to shared memory by bulk copies and from there straight into MMA operand
// registers: no fp16 staging tile (16 KB of the 25 KB of shared-memory traffic per warp and tile of the staged
// form, which kept the shared-memory pipe 70 % busy), no barrier of any kind inside the key loop.
// A thread's operand bytes are made contiguous by permuting the contraction index inside each 32-element block,
// which is free as long as both operands of a product use the same order:
//   Q.K^T (contraction over dims): per block, k-step A takes dims {4t..4t+3}, k-step B dims {16+4t..16+4t+3}
//     of thread t -> one 32-bit word of quants per k-step and key; Q fragments are read in the same order.
//   P.V (output dims): n-tile j of a block holds dims {4g + j}, so the four bytes at dims 4g..4g+3 of one key are
//     thread g's column values for the block's four n-tiles; the epilogue undoes the mapping.
// int8 -> f16: byte b -> half 0x6400 | (b ^ 0x80) = 1024 + (q + 128); minus 1152 is q exactly; times d rounds once:
// fp16(d*q), bit-identical to the staged dequantiser and to the reference's dequantise-then-cast.
constexpr int kDecRegStages = 3;

// PLAIN: no explicit mask, no softcap, no causal bound (single-token decode): only kv_len limits the keys.  A separate
// instantiation, so the common case carries none of the general path's registers and code.
// LOW (with PLAIN): at most 8 live rows (Tq * gqa <= 8), so rows g+8 of every fragment are padding and their softmax
// arithmetic is skipped.
template <int HD, bool PLAIN, bool LOW = false>
__global__ void __launch_bounds__(kThreads, 4) fattn_decode_q8reg_kernel(const FattnArgs a) {
    constexpr int NR = LOW ? 1 : 2, NE = 2 * NR;   // live row halves / accumulator elements per n-tile
    constexpr int NBLK = HD / 32, RB = NBLK * 34;
    constexpr int RAW_BYTES = kDecBN * RB;   // one raw K or V tile
    constexpr int NS = kDecRegStages;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);                                  // [16][HD], 16-byte chunks swizzled
    uint8_t* sRaw = smem_raw + kDecRows * HD * sizeof(__half);                          // NS stages of raw K | V
    __shared__ float s_m[4][kDecRows], s_l[4][kDecRows];
    __shared__ __align__(8) uint64_t s_bar[4][NS];                                      // one barrier per (warp, stage)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int bk = b / a.bq;
    const int R = a.Tq * a.gqa;  // <= 16; row rr -> (iq = rr / gqa, head hk*gqa + rr % gqa)
    const float ninf = -INFINITY;
    cluster_announce(a);

    // launched with programmatic stream serialisation: the previous kernel of the stream has completed and flushed
    // before anything is read or written (a no-op under an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int len_b = clamp_len(a, b);
    const int tq_b = q_rows_of(a, b);   // query rows at or beyond it give zeros
    int kmax = tq_b > 0 ? len_b : 0;    // an entry without live rows reads no keys
    const int n_past = n_past_of(a, len_b, tq_b);
    if (a.causal) kmax = min(kmax, n_past + tq_b);
    const int n_tiles = (kmax + kDecBN - 1) / kDecBN;
    const int tps = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int tile_lo = split * tps, tile_hi = min(n_tiles, tile_lo + tps);
    const uint8_t* kbase = a.k.p + (int64_t)hk * a.k.nb2 + (int64_t)bk * a.k.nb3;
    const uint8_t* vbase = a.v.p + (int64_t)hk * a.v.nb2 + (int64_t)bk * a.v.nb3;

    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NS; i++) mbar_init(smem_u32(&s_bar[warp][i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    auto issue = [&](int tile) {
        if (tile < tile_hi && lane == 0) {
            const int stage = (tile - tile_lo) % NS;
            issue_tile_q8raw<HD>(sRaw + stage * 2 * RAW_BYTES, sRaw + stage * 2 * RAW_BYTES + RAW_BYTES, kbase, vbase, tile * kDecBN,
                                 len_b, warp, smem_u32(&s_bar[warp][stage]));
        }
    };
#pragma unroll
    for (int s0 = 0; s0 < NS; s0++) issue(tile_lo + s0);

    // Q rows (tiny): one 8-element chunk per loop step
    for (int idx = tid; idx < kDecRows * (HD / 8); idx += kThreads) {
        const int rr = idx / (HD / 8), ch = idx % (HD / 8);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (rr < R) {
            int iq, hq;
            row_to_query(a, hk, rr, iq, hq);
            val = load8_as_half(a.q.p + (int64_t)iq * a.q.nb1 + (int64_t)hq * a.q.nb2 + (int64_t)b * a.q.nb3,
                                a.q.type, ch * 8, a.hd, a.q.vec16);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sQ) + (rr * (HD / 8) + swz<HD>(rr, ch)) * 16) = val;
    }
    __syncthreads();
    // Q fragments in the permuted contraction order: k-step A of block blk uses dims 32blk + {4t..4t+3},
    // k-step B dims 32blk + 16 + {4t..4t+3}; rows g and g+8.  qf[blk][ks] = {a0, a1, a2, a3}.
    uint32_t qf[NBLK][2][4];
#pragma unroll
    for (int blk = 0; blk < NBLK; blk++)
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            const int ch = 4 * blk + 2 * ks + (t >> 1);   // 16-byte chunk holding dims 32blk + 16ks + 4t .. +3
#pragma unroll
            for (int rI = 0; rI < 2; rI++) {
                const int rr = g + 8 * rI;
                const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(sQ) +
                                                                 (rr * (HD / 8) + swz<HD>(rr, ch)) * 16 + (t & 1) * 8);
                qf[blk][ks][rI] = w.x, qf[blk][ks][2 + rI] = w.y;
            }
        }

    // per-thread row metadata for rows g and g+8 (general path only)
    int row_iq[2] = {0, 0};
    float row_slope[2] = {1.0f, 1.0f};
    const uint8_t* row_mask[2] = {nullptr, nullptr};
#pragma unroll
    for (int rI = 0; rI < 2 && !PLAIN; rI++) {
        const int rr = g + rI * 8;
        row_iq[rI] = rr / a.gqa;
        const int hq = hk * a.gqa + rr % a.gqa;
        row_slope[rI] = alibi_slope(a, hq);
        row_mask[rI] = (a.has_mask && rr < R)
                           ? a.mask.p + (int64_t)row_iq[rI] * a.mask.nb1 + (int64_t)(hq % a.mask_ne2) * a.mask.nb2 +
                                 (int64_t)(b % a.mask_ne3) * a.mask.nb3
                           : nullptr;
    }

    float m_run[2] = {ninf, ninf}, l_run[2] = {0.0f, 0.0f};
    float o[HD / 8][4];   // n-tile 4*blk + j, column n <-> dim 32blk + 4n + j
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float zpad[4][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};   // LOW: stand-ins for the padding rows of O (stay 0)
    const __half2 bias = __float2half2_rn(1152.0f);
    auto cvt2 = [&](uint32_t packed, __half2 d2) {   // {0x64 q1' 0x64 q0'} -> {d*q0, d*q1}
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&packed), bias), d2);
        return *reinterpret_cast<const uint32_t*>(&v);
    };

    for (int tile = tile_lo; tile < tile_hi; tile++) {
        const int k0 = tile * kDecBN;
        const int stage = (tile - tile_lo) % NS;
        if (!mbar_wait_bounded(smem_u32(&s_bar[warp][stage]), (uint32_t)((tile - tile_lo) / NS) & 1u)) break;
        const uint8_t* rawK = sRaw + stage * 2 * RAW_BYTES + 16 * warp * RB;   // this warp's 16 keys
        const uint8_t* rawV = rawK + RAW_BYTES;
        const int rows_valid = len_b - (k0 + 16 * warp);   // keys at or beyond it hold stale bytes: their scale reads as 0
        const bool all_live = rows_valid >= 16;            // warp-uniform: the common case needs no per-key test

        // ---- S = Q.K^T for this warp's 16 keys ----
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const int key = nt * 8 + g;
            const uint8_t* rowp = rawK + key * RB;
            const bool live = all_live || key < rows_valid;
#pragma unroll
            for (int blk = 0; blk < NBLK; blk++) {
                const uint8_t* bp = rowp + blk * 34;
                const uint16_t dbits = live ? *reinterpret_cast<const uint16_t*>(bp) : (uint16_t)0;
                const __half2 d2 = __half2half2(__ushort_as_half(dbits));
                // quants at bp + 2: words at byte offsets 4t and 16 + 4t of the block's 32 quants; block starts are
                // 2 mod 4 for even blk (rows are multiples of 4 bytes), so those words are read as two halves there
                uint32_t wA, wB;
                if (blk & 1) {
                    wA = *reinterpret_cast<const uint32_t*>(bp + 2 + 4 * t);
                    wB = *reinterpret_cast<const uint32_t*>(bp + 2 + 16 + 4 * t);
                } else {
                    const uint16_t* hp = reinterpret_cast<const uint16_t*>(bp + 2 + 4 * t);
                    wA = hp[0] | ((uint32_t)hp[1] << 16);
                    wB = hp[8] | ((uint32_t)hp[9] << 16);
                }
                wA ^= 0x80808080u, wB ^= 0x80808080u;
                mma16816(s[nt], qf[blk][0], cvt2(__byte_perm(wA, 0x64646464u, 0x5140), d2), cvt2(__byte_perm(wA, 0x64646464u, 0x7362), d2));
                mma16816(s[nt], qf[blk][1], cvt2(__byte_perm(wB, 0x64646464u, 0x5140), d2), cvt2(__byte_perm(wB, 0x64646464u, 0x7362), d2));
            }
        }

        float rmax[2] = {ninf, ninf};
        // common case (no mask, no softcap, every key of the tile visible to every row): one multiply per score
        const bool plain_tile = PLAIN ? (k0 + kDecBN <= len_b)
                                      : (!a.has_mask && a.softcap == 0.0f && k0 + kDecBN <= len_b && (!a.causal || k0 + kDecBN <= n_past + 1));
        if (plain_tile) {
            const float c = a.scale * kLog2e;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    s[nt][e] *= c;
                    rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
                }
        } else if (PLAIN) {   // last tile of the valid range
            const float c = a.scale * kLog2e;
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < NE; e++) {
                    const int ik = k0 + warp * 16 + nt * 8 + 2 * t + (e & 1);
                    s[nt][e] = ik < len_b ? s[nt][e] * c : ninf;
                    rmax[e >> 1] = fmaxf(rmax[e >> 1], s[nt][e]);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int rI = e >> 1;
                    const int ik = k0 + warp * 16 + nt * 8 + 2 * t + (e & 1);
                    float val = s[nt][e] * a.scale;
                    if (a.softcap != 0.0f) val = a.softcap * tanhf(val);
                    const bool valid = ik < len_b && (!a.causal || ik <= n_past + row_iq[rI]);
                    if (row_mask[rI] && valid)
                        val += row_slope[rI] * __half2float(*reinterpret_cast<const __half*>(row_mask[rI] + (int64_t)ik * 2));
                    val = valid ? val * kLog2e : ninf;
                    s[nt][e] = val;
                    rmax[rI] = fmaxf(rmax[rI], val);
                }
        }
        // Lazy rescale: m_run is a reference, not the exact running maximum - it is only raised (and O, l rescaled)
        // when a row's tile maximum outgrew it by 2^8, so P <= 256 stays inside f16 and most tiles skip the rescale.
        float alpha[2] = {1.0f, 1.0f}, muse[2] = {0.0f, 0.0f};
#pragma unroll
        for (int rI = 0; rI < NR; rI++) {
            const float mt = quad_max(rmax[rI]);
            const float mnew = (mt > m_run[rI] + 8.0f) ? mt : m_run[rI];   // -inf + 8 = -inf: the first finite maximum is taken
            muse[rI] = mnew == ninf ? 0.0f : mnew;
            alpha[rI] = (mnew == m_run[rI]) ? 1.0f : exp2f(m_run[rI] - muse[rI]);
            m_run[rI] = mnew;
            l_run[rI] *= alpha[rI];
        }
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (e >= NE) {
                    s[nt][e] = 0.0f;   // padding rows: P = 0
                    continue;
                }
                const float p = fast_ex2(s[nt][e] - muse[e >> 1]);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
        uint32_t pf[4];
        pf[0] = pack_half2(s[0][0], s[0][1]);
        pf[1] = pack_half2(s[0][2], s[0][3]);
        pf[2] = pack_half2(s[1][0], s[1][1]);
        pf[3] = pack_half2(s[1][2], s[1][3]);
        // the running maxima settle after a few tiles: the accumulator is only rescaled when some row of the warp moved
        if (__any_sync(0xffffffffu, alpha[0] != 1.0f || alpha[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < HD / 8; i++) {
                o[i][0] *= alpha[0], o[i][1] *= alpha[0];
                if (!LOW) o[i][2] *= alpha[1], o[i][3] *= alpha[1];
            }
        }

        // ---- O += P.V: keys 2t, 2t+1 (b0) and 2t+8, 2t+9 (b1); this thread's bytes are dims 4g..4g+3 of each block ----
#pragma unroll
        for (int blk = 0; blk < NBLK; blk++) {
            uint32_t w[4];
            uint16_t db[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int key = 2 * t + (i & 1) + 8 * (i >> 1);
                const uint8_t* bp = rawV + key * RB + blk * 34;
                db[i] = *reinterpret_cast<const uint16_t*>(bp);
                if (!all_live && key >= rows_valid) db[i] = (uint16_t)0;   // a dead key's scale may be any bit pattern: 0 * NaN
                if (blk & 1) {
                    w[i] = *reinterpret_cast<const uint32_t*>(bp + 2 + 4 * g);
                } else {
                    const uint16_t* hp = reinterpret_cast<const uint16_t*>(bp + 2 + 4 * g);
                    w[i] = hp[0] | ((uint32_t)hp[1] << 16);
                }
                w[i] ^= 0x80808080u;
            }
            const uint32_t d01b = db[0] | ((uint32_t)db[1] << 16), d23b = db[2] | ((uint32_t)db[3] << 16);
            const __half2 d01 = *reinterpret_cast<const __half2*>(&d01b), d23 = *reinterpret_cast<const __half2*>(&d23b);
            // pair the two keys of an operand register: x = {k0.j, k1.j, k0.j', k1.j'}
            const uint32_t x01a = __byte_perm(w[0], w[1], 0x5140), x01b = __byte_perm(w[0], w[1], 0x7362);
            const uint32_t x23a = __byte_perm(w[2], w[3], 0x5140), x23b = __byte_perm(w[2], w[3], 0x7362);
            if (LOW) mma16816_lo(o[4 * blk + 0][0], o[4 * blk + 0][1], zpad[0][0], zpad[0][1], pf, cvt2(__byte_perm(x01a, 0x64646464u, 0x5140), d01), cvt2(__byte_perm(x23a, 0x64646464u, 0x5140), d23));
            else mma16816(o[4 * blk + 0], pf, cvt2(__byte_perm(x01a, 0x64646464u, 0x5140), d01), cvt2(__byte_perm(x23a, 0x64646464u, 0x5140), d23));
            if (LOW) mma16816_lo(o[4 * blk + 1][0], o[4 * blk + 1][1], zpad[1][0], zpad[1][1], pf, cvt2(__byte_perm(x01a, 0x64646464u, 0x7362), d01), cvt2(__byte_perm(x23a, 0x64646464u, 0x7362), d23));
            else mma16816(o[4 * blk + 1], pf, cvt2(__byte_perm(x01a, 0x64646464u, 0x7362), d01), cvt2(__byte_perm(x23a, 0x64646464u, 0x7362), d23));
            if (LOW) mma16816_lo(o[4 * blk + 2][0], o[4 * blk + 2][1], zpad[2][0], zpad[2][1], pf, cvt2(__byte_perm(x01b, 0x64646464u, 0x5140), d01), cvt2(__byte_perm(x23b, 0x64646464u, 0x5140), d23));
            else mma16816(o[4 * blk + 2], pf, cvt2(__byte_perm(x01b, 0x64646464u, 0x5140), d01), cvt2(__byte_perm(x23b, 0x64646464u, 0x5140), d23));
            if (LOW) mma16816_lo(o[4 * blk + 3][0], o[4 * blk + 3][1], zpad[3][0], zpad[3][1], pf, cvt2(__byte_perm(x01b, 0x64646464u, 0x7362), d01), cvt2(__byte_perm(x23b, 0x64646464u, 0x7362), d23));
            else mma16816(o[4 * blk + 3], pf, cvt2(__byte_perm(x01b, 0x64646464u, 0x7362), d01), cvt2(__byte_perm(x23b, 0x64646464u, 0x7362), d23));
        }
        __syncwarp();       // every lane is done with this stage's bytes
        issue(tile + NS);   // the next tile that lives in this stage: NS-1 tiles stay in flight during the arithmetic
    }

    // the merge kernel (if any) may start launching: it waits for this grid's completion before reading anything
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- merge the four warps' (m, l, O) in shared memory ----
    constexpr int SLAB_STRIDE = HD + 4;
    float* slab = reinterpret_cast<float*>(smem_raw);   // [4][16][SLAB_STRIDE]
    {
        const float lq[2] = {quad_sum(l_run[0]), quad_sum(l_run[1])};
        if (t == 0) {   // static shared memory: written before the barrier that retires the tiles
            s_m[warp][g] = m_run[0], s_m[warp][g + 8] = m_run[1];
            s_l[warp][g] = lq[0], s_l[warp][g + 8] = lq[1];
        }
    }
    __syncthreads();  // all warps are done with the raw stages (the merge slabs alias them); the warps' (m, l) are visible
    // Each warp parks its partial O as it is, scaled to its OWN running maximum, in its own padded slab (the slabs start
    // at the base of dynamic shared memory - Q and the raw stages are dead by now): the four n-tiles of a block give a
    // thread four consecutive dims of rows g and g + 8 (dim = 32 blk + 4 (2t + e) + n-tile), one 16-byte store each;
    // rows at or beyond R are never read.
#pragma unroll
    for (int rI = 0; rI < NR; rI++) {
        if (g + rI * 8 >= R) continue;
#pragma unroll
        for (int blk = 0; blk < HD / 32; blk++)
#pragma unroll
            for (int e = 0; e < 2; e++)
                *reinterpret_cast<float4*>(slab + (warp * kDecRows + g + rI * 8) * SLAB_STRIDE + 32 * blk + 4 * (2 * t + e)) =
                    make_float4(o[4 * blk + 0][2 * rI + e], o[4 * blk + 1][2 * rI + e], o[4 * blk + 2][2 * rI + e], o[4 * blk + 3][2 * rI + e]);
    }
    __syncthreads();
    decode_write_out<HD>(a, slab, s_m, s_l, sRaw + NS * 2 * RAW_BYTES, R, b, hk, split, tq_b, tid);
}

// ------------------------------------------------------------------------------------------
// Split-KV decode over a Q8_0 cache with the KEYS on the M side of the MMA (at most 8 query rows, plain form)
// ------------------------------------------------------------------------------------------
// The register kernel above multiplies 16 query rows (at most 8 of them real) with 8 keys per MMA and has to apply the
// block scale to every operand register of K and V (hsub2 + hmul2 per register: half of its instructions).  This
// variant transposes both products - S^T = K.Q^T and O^T = V^T.P^T, m16 = keys / output dims, n8 = the query rows - so
// that a block scale belongs to an accumulator ROW of the thread that loaded the block:
//   * scores: the quants go into the MMA as the exact halves 1152 + q (0x6400 | (b ^ 0x80), no subtract, no multiply),
//     one accumulator per 32-element block; then s += d * (acc - 1152 * sum_block(Q)), the block sum of the query row
//     being a per-thread constant.  fp32(d) * (integer dot) is the oracle's own arithmetic (x = fp32(d) * q), one
//     rounding closer to it than fp16(d * q) operands;
//   * P.V: the V block scale moves onto P (two half2 multiplies per block instead of eight), the quants go in as exact
//     integers q (one subtract, no multiply).  P <= 2^4 here (the lazy-rescale bound is 4 instead of 8), so P * d stays
//     inside f16 for every representable block scale (d <= 65504 / 127);
//   * half as many MMAs (no padding rows), no quad shuffles in the common tile: the running maximum is only reduced
//     across the warp when some key outgrew it.
// P comes out of the score MMA as (key, row) accumulators and is needed as the (key, row) B operand of the second
// product: one movmatrix.trans per 8 keys.  Staging (per-warp bulk copies of raw bytes, per-warp mbarriers, 3 stages),
// split / merge forms and the epilogue are those of the kernel above.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

__device__ __forceinline__ void mma16832_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// S8: the score product runs on the int8 tensor path.  The K quants are the A operand as they lie in the cache (no
// byte permutes, no bias, no conversion at all); the query row is split once per CTA into two int8 planes per
// 32-element block, q = dq*(hi + lo/254) with hi = round(x/dq), lo = round((x - dq*hi)*254/dq), dq = max|x|/127, which
// keeps an absolute error of dq/508 = 1.5e-5 of the block maximum per element (F16 itself resolves 4.9e-4 of a
// value).  Per block two k32 MMAs give exact int32 dots, combined as 254*hi + lo, converted once and scaled by
// fp32(d_k)*dq/254.  This empties the integer ALU pipe of the K side, which bounds the F16 form of this kernel.
template <int HD, bool S8>
__global__ void __launch_bounds__(kThreads, 4) fattn_decode_q8t_kernel(const FattnArgs a) {
    constexpr int NBLK = HD / 32, RB = NBLK * 34;
    constexpr int RAW_BYTES = kDecBN * RB;   // one raw K or V tile
    constexpr int NS = kDecRegStages;
    constexpr float kGrow = 4.0f;            // lazy-rescale bound in log2 units: P <= 16
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __half* sQ = reinterpret_cast<__half*>(smem_raw);                                  // [16][HD], 16-byte chunks swizzled
    uint8_t* sRaw = smem_raw + kDecRows * HD * sizeof(__half);                          // NS stages of raw K | V
    __shared__ float s_m[4][kDecRows], s_l[4][kDecRows];
    __shared__ __align__(8) uint64_t s_bar[4][NS];                                      // one barrier per (warp, stage)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    Q8T_TRACE(0);
    const int bk = b / a.bq;
    const int R = a.Tq * a.gqa;  // <= 8; row rr -> (iq = rr / gqa, head hk*gqa + rr % gqa)
    const float ninf = -INFINITY;
    cluster_announce(a);

    const uint8_t* kbase = a.k.p + (int64_t)hk * a.k.nb2 + (int64_t)bk * a.k.nb3;
    const uint8_t* vbase = a.v.p + (int64_t)hk * a.v.nb2 + (int64_t)bk * a.v.nb3;

    // A CTA of this kernel shares its SM with three others in their key loops, where a lone thread gets an issue slot
    // every few tens of clocks: the set-up below is spread over lanes so that its chain of dependent instructions is
    // short - lane i initialises barrier i, lanes 2s and 2s+1 request the K and the V bytes of stage s.
    Q8T_TRACE(14);
    if (lane < NS) {
        mbar_init(smem_u32(&s_bar[warp][lane]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    Q8T_TRACE(15);
    // Launched with programmatic stream serialisation: everything above (kernel parameters, this CTA's own shared
    // memory) ran while the previous kernel of the stream drained; from here on that kernel has completed and flushed
    // (a no-op under an ordinary launch).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    Q8T_TRACE(1);
    const int len_b = clamp_len(a, b);
    const int tq_b = q_rows_of(a, b);
    const int kmax = tq_b > 0 ? len_b : 0;
    const int n_tiles = (kmax + kDecBN - 1) / kDecBN;
    const int tps = (n_tiles + a.n_splits - 1) / a.n_splits;
    const int tile_lo = split * tps, tile_hi = min(n_tiles, tile_lo + tps);
    // lanes 2s (K) and 2s+1 (V) of a warp copy the raw bytes of the warp's 16 keys of tile `tile0 + s`; lane 2s also
    // announces both copies to the stage's barrier.  Copies stop at the stream's length (whole 16-byte units).
    auto issue_lanes = [&](int tile0, int n_stages) {
        const int s_ = lane >> 1, tile = tile0 + s_;
        if (s_ < n_stages && tile < tile_hi) {
            const int stage = (tile - tile_lo) % NS;
            const int r0 = tile * kDecBN + 16 * warp;
            const int n = min(16, max(0, len_b - r0));
            const uint32_t bytes = (uint32_t)((n * RB + 15) / 16 * 16);
            const uint32_t bar = smem_u32(&s_bar[warp][stage]);
            if ((lane & 1) == 0) mbar_expect_tx(bar, 2 * bytes);
            if (bytes) {
                const uint32_t dst = smem_u32(sRaw + stage * 2 * RAW_BYTES + (lane & 1) * RAW_BYTES) + 16 * warp * RB;
                bulk_g2s(dst, ((lane & 1) ? vbase : kbase) + (int64_t)r0 * RB, bytes, bar);
            }
        }
    };
    auto issue = [&](int tile) { issue_lanes(tile, 1); };
    issue_lanes(tile_lo, NS);
    Q8T_TRACE(2);
    // Q rows (tiny): the eight rows this kernel has, one 8-element chunk per thread; rows >= R are zero.  A single
    // new token per stream (the usual decode step) needs no division by the group size.
    static_assert(8 * (HD / 8) <= kThreads, "one chunk per thread");
    if (tid < 8 * (HD / 8)) {
        const int rr = tid / (HD / 8), ch = tid % (HD / 8);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (rr < R) {
            int iq, hq;
            row_to_query(a, hk, rr, iq, hq);
            val = load8_as_half(a.q.p + (int64_t)iq * a.q.nb1 + (int64_t)hq * a.q.nb2 + (int64_t)b * a.q.nb3,
                                a.q.type, ch * 8, a.hd, a.q.vec16);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sQ) + (rr * (HD / 8) + swz<HD>(rr, ch)) * 16) = val;
    }
    __syncthreads();
    // S8: the two int8 planes and the block scales of the 8 query rows, built once by 8 * NBLK threads in shared memory
    // behind the f16 rows (the raw stages are not touched: their copies are already in flight)
    // (rows 8..15 of the f16 Q tile do not exist in this kernel: the planes take their 16 * HD bytes; the block scales
    // borrow the first 8 * NBLK floats of s_l, which is not used before the epilogue - four CTAs per SM leave no room
    // for more static shared memory)
    int8_t* s_qhi = reinterpret_cast<int8_t*>(sQ) + 8 * HD * sizeof(__half);
    int8_t* s_qlo = s_qhi + 8 * HD;
    float* s_qd = &s_l[0][0];
    if (S8) {
        if (tid < 8 * NBLK) {
            const int rr = tid / NBLK, blk = tid % NBLK;
            float x[32];
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(sQ) + (rr * (HD / 8) + swz<HD>(rr, 4 * blk + c4)) * 16);
                const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
                    x[c4 * 8 + 2 * i] = f2.x, x[c4 * 8 + 2 * i + 1] = f2.y;
                }
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
            const float dq = amax / 127.0f, inv = dq > 0.0f ? 1.0f / dq : 0.0f;
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const float hi = rintf(x[i] * inv);
                const float lo = fminf(fmaxf(rintf((x[i] - dq * hi) * inv * 254.0f), -127.0f), 127.0f);
                s_qhi[rr * HD + blk * 32 + i] = (int8_t)hi, s_qlo[rr * HD + blk * 32 + i] = (int8_t)lo;
            }
            s_qd[rr * NBLK + blk] = dq * (1.0f / 254.0f);
        }
        __syncthreads();
    }
    // Q as the B operand of S^T = K.Q^T: column n = query row g.  F16 form: per (block, k-step) the thread's four
    // contraction indices are dims 32blk + 16ks + {4t..4t+3} (the same permutation the K bytes are read in): one 8-byte
    // read.  S8 form: per block, k = 4t..4t+3 (b0) and 16+4t..16+4t+3 (b1) of both planes, no permutation.
    uint32_t qb[NBLK][2][2];
#pragma unroll
    for (int blk = 0; blk < NBLK; blk++)
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            if (S8) {
                // ks = plane (0 = hi, 1 = lo); [.][0] = k 4t.., [.][1] = k 16+4t..
                const int8_t* plane = (ks ? s_qlo : s_qhi) + g * HD;
                qb[blk][ks][0] = *reinterpret_cast<const uint32_t*>(plane + blk * 32 + 4 * t);
                qb[blk][ks][1] = *reinterpret_cast<const uint32_t*>(plane + blk * 32 + 16 + 4 * t);
            } else {
                const int ch = 4 * blk + 2 * ks + (t >> 1);
                const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(sQ) + (g * (HD / 8) + swz<HD>(g, ch)) * 16 + (t & 1) * 8);
                qb[blk][ks][0] = w.x, qb[blk][ks][1] = w.y;
            }
        }
    // F16 form: -1152 * (sum of the query row's f16 values over a block); S8 form: the row's block scale dq / 254 -
    // for this thread's accumulator columns (rows 2t, 2t+1)
    if (!S8) {
        // the 8 * NBLK block sums of the query rows, once per CTA: four threads per (row, block), one 16-byte chunk each
        // (s_l is free until the epilogue)
        const int pair = tid >> 2, c4 = tid & 3;
        float sum = 0.0f;
        if (pair < 8 * NBLK) {
            const int rr = pair / NBLK, blk = pair % NBLK;
            const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(sQ) + (rr * (HD / 8) + swz<HD>(rr, 4 * blk + c4)) * 16);
            const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[i]));
                sum += f2.x + f2.y;
            }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (pair < 8 * NBLK && c4 == 0) s_qd[pair] = -1152.0f * sum;
        __syncthreads();
    }
    Q8T_TRACE(3);
    float negc[NBLK][2];
#pragma unroll
    for (int blk = 0; blk < NBLK; blk++)
#pragma unroll
        for (int j = 0; j < 2; j++) negc[blk][j] = s_qd[(2 * t + j) * NBLK + blk];

    float m_run[2] = {ninf, ninf}, l_run[2] = {0.0f, 0.0f};   // rows 2t, 2t+1; m_run is the same on the 8 lanes that share t
    float o[NBLK][2][4];   // [block][m-tile]: c0/c1 = dim 32blk+4g+2mt of rows 2t/2t+1, c2/c3 = dim +1
#pragma unroll
    for (int blk = 0; blk < NBLK; blk++)
#pragma unroll
        for (int mt = 0; mt < 2; mt++) o[blk][mt][0] = o[blk][mt][1] = o[blk][mt][2] = o[blk][mt][3] = 0.0f;
    const __half2 bias = __float2half2_rn(1152.0f);
    const float c = a.scale * kLog2e;

    Q8T_TRACE(4);
    for (int tile = tile_lo; tile < tile_hi; tile++) {
        const int k0 = tile * kDecBN;
        const int stage = (tile - tile_lo) % NS;
        if (!mbar_wait_bounded(smem_u32(&s_bar[warp][stage]), (uint32_t)((tile - tile_lo) / NS) & 1u)) break;
        if (tile == tile_lo) Q8T_TRACE(5);
        if (tile == tile_lo + 1) Q8T_TRACE(6);
        const uint8_t* rawK = sRaw + stage * 2 * RAW_BYTES + 16 * warp * RB;   // this warp's 16 keys
        const uint8_t* rawV = rawK + RAW_BYTES;
        const int rows_valid = len_b - (k0 + 16 * warp);   // keys at or beyond it hold stale bytes: their scale reads as 0
        const bool all_live = rows_valid >= 16;

        // ---- S^T = K.Q^T: keys g and g+8 of this warp's 16, query rows 2t and 2t+1 ----
        float st[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint8_t* rowp[2] = {rawK + g * RB, rawK + (g + 8) * RB};
        const bool live[2] = {all_live || g < rows_valid, all_live || g + 8 < rows_valid};
#pragma unroll
        for (int blk = 0; blk < NBLK; blk++) {
            if (S8) {
                // the K bytes are the A operand as they lie: words at quants 4t..4t+3 and 16+4t.. of keys g and g+8
                uint32_t af[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint8_t* bp = rowp[i & 1] + blk * 34 + 2 + 16 * (i >> 1) + 4 * t;
                    if (blk & 1) {
                        af[i] = *reinterpret_cast<const uint32_t*>(bp);
                    } else {
                        const uint16_t* hp = reinterpret_cast<const uint16_t*>(bp);
                        af[i] = hp[0] | ((uint32_t)hp[1] << 16);
                    }
                }
                int ahi[4] = {0, 0, 0, 0}, alo[4] = {0, 0, 0, 0};
                mma16832_s8(ahi, af, qb[blk][0][0], qb[blk][0][1]);
                mma16832_s8(alo, af, qb[blk][1][0], qb[blk][1][1]);
                const uint16_t d0b = live[0] ? *reinterpret_cast<const uint16_t*>(rowp[0] + blk * 34) : (uint16_t)0;
                const uint16_t d1b = live[1] ? *reinterpret_cast<const uint16_t*>(rowp[1] + blk * 34) : (uint16_t)0;
                const float d0 = __half2float(__ushort_as_half(d0b)), d1 = __half2float(__ushort_as_half(d1b));
                // exact integer dot of the block: 254 * hi + lo (|.| < 2^28), then one conversion and the two scales
                st[0] = fmaf(d0 * negc[blk][0], (float)(ahi[0] * 254 + alo[0]), st[0]);
                st[1] = fmaf(d0 * negc[blk][1], (float)(ahi[1] * 254 + alo[1]), st[1]);
                st[2] = fmaf(d1 * negc[blk][0], (float)(ahi[2] * 254 + alo[2]), st[2]);
                st[3] = fmaf(d1 * negc[blk][1], (float)(ahi[3] * 254 + alo[3]), st[3]);
                continue;
            }
            // the accumulators start at -1152 * sum_block(Q): the products of the biased halves land on the integer dot
            float acc[4] = {negc[blk][0], negc[blk][1], negc[blk][0], negc[blk][1]};
#pragma unroll
            for (int ks = 0; ks < 2; ks++) {
                uint32_t w[2];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint8_t* bp = rowp[i] + blk * 34 + 2 + 16 * ks + 4 * t;   // block starts are 2 mod 4 for even blk
                    if (blk & 1) {
                        w[i] = *reinterpret_cast<const uint32_t*>(bp);
                    } else {
                        const uint16_t* hp = reinterpret_cast<const uint16_t*>(bp);
                        w[i] = hp[0] | ((uint32_t)hp[1] << 16);
                    }
                    w[i] ^= 0x80808080u;
                }
                const uint32_t af[4] = {__byte_perm(w[0], 0x64646464u, 0x5140), __byte_perm(w[1], 0x64646464u, 0x5140),
                                        __byte_perm(w[0], 0x64646464u, 0x7362), __byte_perm(w[1], 0x64646464u, 0x7362)};
                mma16816(acc, af, qb[blk][ks][0], qb[blk][ks][1]);
            }
            // the scale is read whether or not the key is live (stale bytes of a finished stage are harmless here: dead
            // scores are replaced by -inf below), so the common tile has no branch around the load
            const float d0 = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rowp[0] + blk * 34)));
            const float d1 = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(rowp[1] + blk * 34)));
            st[0] = fmaf(d0, acc[0], st[0]);
            st[1] = fmaf(d0, acc[1], st[1]);
            st[2] = fmaf(d1, acc[2], st[2]);
            st[3] = fmaf(d1, acc[3], st[3]);
        }
        // scale to the log2 domain; keys beyond the valid length are masked (last tile of a stream only)
#pragma unroll
        for (int e = 0; e < 4; e++) st[e] *= c;
        if (!all_live) {
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (!live[e >> 1]) st[e] = ninf;
        }

        // ---- lazy running maximum: only when some key outgrew the reference by 2^4 is it reduced over the warp ----
        const float lm[2] = {fmaxf(st[0], st[2]), fmaxf(st[1], st[3])};
        if (__any_sync(0xffffffffu, lm[0] > m_run[0] + kGrow || lm[1] > m_run[1] + kGrow)) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                float rm = lm[j];
                rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, 4));
                rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, 8));
                rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, 16));
                const float mnew = (rm > m_run[j] + kGrow) ? rm : m_run[j];   // -inf + 4 = -inf: the first finite maximum is taken
                if (mnew != m_run[j]) {
                    const float alpha = exp2f(m_run[j] - mnew);   // m_run = -inf -> 0
                    l_run[j] *= alpha;
#pragma unroll
                    for (int blk = 0; blk < NBLK; blk++)
#pragma unroll
                        for (int mt = 0; mt < 2; mt++) o[blk][mt][j] *= alpha, o[blk][mt][2 + j] *= alpha;
                    m_run[j] = mnew;
                }
            }
        }
        const float muse[2] = {m_run[0] == ninf ? 0.0f : m_run[0], m_run[1] == ninf ? 0.0f : m_run[1]};
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            p[e] = fast_ex2(st[e] - muse[e & 1]);
            l_run[e & 1] += p[e];
        }
        // P^T as the B operand of O^T = V^T.P^T: (key g, rows 2t,2t+1) -> (keys 2t,2t+1, row g)
        const uint32_t pb0 = movmatrix_trans(pack_half2(p[0], p[1]));
        const uint32_t pb1 = movmatrix_trans(pack_half2(p[2], p[3]));
        const __half2 pb0h = *reinterpret_cast<const __half2*>(&pb0), pb1h = *reinterpret_cast<const __half2*>(&pb1);

        // ---- O^T += V^T.P^T: keys 2t, 2t+1 (low k half) and 2t+8, 2t+9; this thread's bytes are dims 4g..4g+3 of each block ----
#pragma unroll
        for (int blk = 0; blk < NBLK; blk++) {
            uint32_t w[4];
            uint16_t db[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int key = 2 * t + (i & 1) + 8 * (i >> 1);
                const uint8_t* bp = rawV + key * RB + blk * 34;
                db[i] = (all_live || key < rows_valid) ? *reinterpret_cast<const uint16_t*>(bp) : (uint16_t)0;
                if (blk & 1) {
                    w[i] = *reinterpret_cast<const uint32_t*>(bp + 2 + 4 * g);
                } else {
                    const uint16_t* hp = reinterpret_cast<const uint16_t*>(bp + 2 + 4 * g);
                    w[i] = hp[0] | ((uint32_t)hp[1] << 16);
                }
                w[i] ^= 0x80808080u;
            }
            // the block scales ride on P: P'[key] = P[key] * d(key, blk)
            const uint32_t d01b = db[0] | ((uint32_t)db[1] << 16), d23b = db[2] | ((uint32_t)db[3] << 16);
            const __half2 q0 = __hmul2(pb0h, *reinterpret_cast<const __half2*>(&d01b));
            const __half2 q1 = __hmul2(pb1h, *reinterpret_cast<const __half2*>(&d23b));
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&q0), b1 = *reinterpret_cast<const uint32_t*>(&q1);
            // pair the two keys of an operand register: x = {k0.j, k1.j, k0.j', k1.j'}
            const uint32_t x01a = __byte_perm(w[0], w[1], 0x5140), x01b = __byte_perm(w[0], w[1], 0x7362);
            const uint32_t x23a = __byte_perm(w[2], w[3], 0x5140), x23b = __byte_perm(w[2], w[3], 0x7362);
            auto exact = [&](uint32_t packed) {   // {0x64 q1' 0x64 q0'} -> {q0, q1} as f16 integers
                const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&packed), bias);
                return *reinterpret_cast<const uint32_t*>(&v);
            };
            const uint32_t a_lo[4] = {exact(__byte_perm(x01a, 0x64646464u, 0x5140)), exact(__byte_perm(x01a, 0x64646464u, 0x7362)),
                                      exact(__byte_perm(x23a, 0x64646464u, 0x5140)), exact(__byte_perm(x23a, 0x64646464u, 0x7362))};
            mma16816(o[blk][0], a_lo, b0, b1);
            const uint32_t a_hi[4] = {exact(__byte_perm(x01b, 0x64646464u, 0x5140)), exact(__byte_perm(x01b, 0x64646464u, 0x7362)),
                                      exact(__byte_perm(x23b, 0x64646464u, 0x5140)), exact(__byte_perm(x23b, 0x64646464u, 0x7362))};
            mma16816(o[blk][1], a_hi, b0, b1);
        }
        __syncwarp();       // every lane is done with this stage's bytes
        issue(tile + NS);
    }

    Q8T_TRACE(7);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- merge the four warps' (m, l, O) in shared memory (same slabs as the kernel above) ----
    constexpr int SLAB_STRIDE = HD + 4;
    float* slab = reinterpret_cast<float*>(smem_raw);   // [4][16][SLAB_STRIDE]
    float lq[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        float v = l_run[j];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        lq[j] = v;
    }
    if (g == 0) {
        s_m[warp][2 * t] = m_run[0], s_m[warp][2 * t + 1] = m_run[1];
        s_l[warp][2 * t] = lq[0], s_l[warp][2 * t + 1] = lq[1];
    }
    if (lane < 8) s_m[warp][8 + lane] = ninf, s_l[warp][8 + lane] = 0.0f;   // rows 8..15 do not exist in this form
    __syncthreads();  // the warps' (m, l) are visible, and all warps are done with the raw stages (the merge slabs alias them)
    Q8T_TRACE(8);
    // Each warp parks its accumulators as they are (scaled to its OWN running maximum): a thread's accumulators of one
    // block are four consecutive dims (4g .. 4g+3) of rows 2t and 2t+1, one 16-byte store per (block, row), conflict-free
    // (quarter-warps cover eight different 16-byte slots of a 128-byte line); rows at or beyond R are never read.
#pragma unroll
    for (int j = 0; j < 2; j++) {
        if (2 * t + j >= R) continue;
#pragma unroll
        for (int blk = 0; blk < NBLK; blk++)
            *reinterpret_cast<float4*>(slab + (warp * kDecRows + 2 * t + j) * SLAB_STRIDE + 32 * blk + 4 * g) =
                make_float4(o[blk][0][j], o[blk][0][2 + j], o[blk][1][j], o[blk][1][2 + j]);
    }
    Q8T_TRACE(12);
    __syncthreads();
    Q8T_TRACE(9);
    Q8T_TRACE(13);
    decode_write_out<HD>(a, slab, s_m, s_l, sRaw + NS * 2 * RAW_BYTES, R, b, hk, split, tq_b, tid);
    Q8T_TRACE(10);
}

// One warp per (batch, kv-head, row): log-sum-exp merge of the split partials.
template <int HD>
__global__ void __launch_bounds__(kThreads) fattn_merge_kernel(const FattnArgs a) {
    // Launched with programmatic stream serialisation: its CTAs may become resident while the split kernel drains;
    // nothing of the workspace is read before the split grid has completed and flushed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp_global = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int R = a.Tq * a.gqa;   // live rows per (batch, kv head); one warp each
    const int total = a.B * a.Hkv * R;
    if (warp_global >= total) return;
    const int rr = warp_global % R;
    const int hk = (warp_global / R) % a.Hkv;
    const int b = warp_global / (R * a.Hkv);
    const int64_t unit0 = ((int64_t)b * a.Hkv + hk) * a.n_splits;
    // One pass, sixteen splits per round: every load of a round is issued before the first is used (one memory
    // round trip per round), and the running (M, L, acc) are rescaled when a round raises the maximum.
    float M = -INFINITY, L = 0.0f;
    float acc[HD / 32];
#pragma unroll
    for (int i = 0; i < HD / 32; i++) acc[i] = 0.0f;
    for (int s0 = 0; s0 < a.n_splits; s0 += 16) {
        float2 ml[16];
        float po[16][HD / 32];
#pragma unroll
        for (int u = 0; u < 16; u++) {
            const int s = min(s0 + u, a.n_splits - 1);
            ml[u] = *reinterpret_cast<const float2*>(a.ws_ml + ((unit0 + s) * kDecRows + rr) * 2);
            const float* p = a.ws_o + ((unit0 + s) * kDecRows + rr) * HD;
#pragma unroll
            for (int i = 0; i < HD / 32; i++) po[u][i] = p[lane + 32 * i];
        }
        float Mr = M;
#pragma unroll
        for (int u = 0; u < 16; u++)
            if (s0 + u < a.n_splits) Mr = fmaxf(Mr, ml[u].x);
        if (Mr > M) {
            const float scale_old = (M == -INFINITY) ? 0.0f : exp2f(M - Mr);
            L *= scale_old;
#pragma unroll
            for (int i = 0; i < HD / 32; i++) acc[i] *= scale_old;
            M = Mr;
        }
#pragma unroll
        for (int u = 0; u < 16; u++) {
            if (s0 + u >= a.n_splits || ml[u].x == -INFINITY) continue;
            const float w = exp2f(ml[u].x - M);
            L += w * ml[u].y;
#pragma unroll
            for (int i = 0; i < HD / 32; i++) acc[i] += w * po[u][i];
        }
    }
    int iq, hq;
    row_to_query(a, hk, rr, iq, hq);
    float* out = a.dst + (((int64_t)b * a.Tq + iq) * a.H + hq) * a.hd;
    const float inv = (L > 0.0f && iq < q_rows_of(a, b)) ? 1.0f / L : 0.0f;
#pragma unroll
    for (int i = 0; i < HD / 32; i++) {
        const int c = lane + 32 * i;
        if (c < a.hd) out[c] = acc[i] * inv;
    }
}

// Merge kernel with programmatic stream serialisation (its launch overlaps the tail of the split kernel; the
// kernel itself waits for the split grid before it reads the workspace).
template <int HD>
cudaError_t launch_merge(const FattnArgs& a, cudaStream_t st) {
    const int warps = a.B * a.Hkv * a.Tq * a.gqa;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((warps + 3) / 4);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, fattn_merge_kernel<HD>, a);
}

// The splits of one (batch entry, kv-head) of the Q8_0 register kernel run as one thread-block cluster when there
// are at most 8 of them (the portable cluster size): they merge through distributed shared memory and the merge
// kernel is not launched.  The F16 kernel takes the same form: one to eight segments per launch measured 4-14 %
// faster for cross-attention (1500 keys) and +9 % / +4 % at four / eight segments of the pooled self-attention
// (2304 cells); where twelve workspace splits beat eight cluster splits (one segment of the latter) the cost model
// below keeps the merge kernel.
// B200_DECODE_CLUSTER_MERGE=0 keeps the workspace + merge-kernel form everywhere.
bool cluster_merge_enabled() {
    static const bool enabled = [] {
        const char* e = getenv("B200_DECODE_CLUSTER_MERGE");
        return !(e && e[0] == '0');
    }();
    return enabled;
}

bool use_cluster_merge(const FattnArgs& a) {
    // only while the whole grid is resident at once (2 to 4 CTAs on each of 148 SMs): with several waves the cluster
    // barriers hold finished CTAs on their SMs and the form measured 10 % slower than the merge kernel
    return decode_cluster_merge_ok(a) && a.n_splits > 1 && a.n_splits <= 8 &&
           (long)a.n_splits * a.Hkv * a.B <= (long)decode_ctas_per_sm(a, true) * 148;
}

template <typename Kern>
void launch_split(Kern kern, dim3 grid, size_t smem, cudaStream_t st, const FattnArgs& a) {
    // Programmatic stream serialisation: the grid may become resident while the previous kernel of the stream drains
    // (its CTAs wait on the device before they touch memory), which hides the launch latency between the layers of a
    // decode step (+0.8 % on the 64-segment decode launches, +1 % at 32 streams).
    FattnArgs ac = a;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int n = 0;
    // also for the cluster form: with the pushed merge an early-resident cluster measures +3 to +4 % (8 / 16 streams
    // of the Q8_0 cache, 1 / 4 Whisper segments); with the pulled merge, whose CTAs stayed resident through two cluster
    // barriers, it had measured 8.7 against 8.0 us per layer
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
    if (use_cluster_merge(a)) {
        ac.cluster_merge = 1;
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = grid.x, attr[n].val.clusterDim.y = 1, attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kern, ac);   // errors are picked up by the caller's cudaGetLastError
}

template <int HD, int MODE>
int launch_decode_m(const FattnArgs& a, cudaStream_t st) {
    constexpr int NS = MODE == kDecSync ? 1 : (MODE == kDecAsyncF16 ? (HD >= 128 ? 3 : 4) : kDecQ8Stages);
    constexpr int F16_STAGES = MODE == kDecAsyncF16 ? NS : 1;
    constexpr int F16_TILES = MODE == kDecAsyncQ8 ? 1 : F16_STAGES * 2;
    size_t smem = (size_t)(kDecRows + F16_TILES * kDecBN) * HD * sizeof(__half);
    if (MODE == kDecAsyncQ8) smem += (size_t)NS * 2 * kDecBN * (HD / 32 * 34);
    // the attribute is raised once, to the largest size this instantiation can ask for (mask staging for 16 rows)
    const size_t smem_attr = smem + (MODE == kDecAsyncF16 ? (size_t)NS * kDecRows * kDecBN * sizeof(__half) : 0) + cluster_push_bytes(HD, kDecRows);
    const bool staged_mask = MODE == kDecAsyncF16 && a.has_mask && a.mask.vec16 && a.softcap == 0.0f && !a.causal && a.n2 == 0;
    if (staged_mask) smem += (size_t)NS * (a.Tq * a.gqa) * kDecBN * sizeof(__half);
    if (use_cluster_merge(a)) smem += cluster_push_bytes(HD, a.Tq * a.gqa);   // the receive area of the merge inside a cluster, behind everything else
    dim3 grid(a.n_splits, a.Hkv, a.B);
    cudaError_t e;
    const bool low = a.Tq * a.gqa <= 8;
    if (staged_mask && a.kv_index && low) {   // a shared index list plus a compact membership mask over its entries
        auto kern = fattn_decode_split_kernel<HD, MODE, MODE == kDecAsyncF16, false, MODE == kDecAsyncF16, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (staged_mask && a.kv_index) {
        auto kern = fattn_decode_split_kernel<HD, MODE, MODE == kDecAsyncF16, false, false, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (staged_mask && low) {
        auto kern = fattn_decode_split_kernel<HD, MODE, MODE == kDecAsyncF16, false, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (staged_mask) {
        auto kern = fattn_decode_split_kernel<HD, MODE, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (MODE == kDecAsyncF16 && a.kv_index && low) {   // index lists come without mask / softcap / causal bound
        auto kern = fattn_decode_split_kernel<HD, MODE, false, MODE == kDecAsyncF16, MODE == kDecAsyncF16, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (MODE == kDecAsyncF16 && a.kv_index) {
        auto kern = fattn_decode_split_kernel<HD, MODE, false, MODE == kDecAsyncF16, false, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (MODE == kDecAsyncF16 && !a.has_mask && a.softcap == 0.0f && !a.causal && low) {
        auto kern = fattn_decode_split_kernel<HD, MODE, false, MODE == kDecAsyncF16, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (MODE == kDecAsyncF16 && !a.has_mask && a.softcap == 0.0f && !a.causal) {
        auto kern = fattn_decode_split_kernel<HD, MODE, false, MODE == kDecAsyncF16>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else {
        auto kern = fattn_decode_split_kernel<HD, MODE, false, false>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (a.n_splits > 1 && !use_cluster_merge(a)) e = launch_merge<HD>(a, st);
    return (int)e;
}

// Which staging mode the operands allow.
int decode_mode(const FattnArgs& a, int hdp) {
    if (a.hd != hdp) return kDecSync;  // zero-padded head dims take the element path
    if (a.k.type == B200_TYPE_F16 && a.k.vec16 && a.v.vec16) return kDecAsyncF16;
    if (a.k.type == B200_TYPE_Q8_0) {
        const int64_t rb = a.hd / 32 * 34;
        const bool contiguous_rows = a.k.nb1 == rb && a.v.nb1 == rb;
        const bool aligned = ((uintptr_t)a.k.p % 16 == 0) && ((uintptr_t)a.v.p % 16 == 0) && a.k.nb2 % 16 == 0 &&
                             a.k.nb3 % 16 == 0 && a.v.nb2 % 16 == 0 && a.v.nb3 % 16 == 0;
        // the last 16-byte chunk of a tile may reach past row Lk-1 by < 16 bytes only if rows*rb is not a
        // multiple of 16; chunks are issued per tile of 64 rows (64*rb is a multiple of 16) and chunks that
        // start at or beyond row kv_len are zero-filled, so reads stay inside rows [0, Lk) when Lk*rb % 16 == 0
        // or the head slab continues behind row Lk-1 (nb2 > Lk*rb).
        const bool tail_ok = ((int64_t)a.Lk * rb) % 16 == 0 || a.k.nb2 >= ((int64_t)a.Lk * rb + 15) / 16 * 16;
        if (!a.kv_index && contiguous_rows && aligned && tail_ok && a.v.nb2 >= ((int64_t)a.Lk * rb + 15) / 16 * 16)   // gathered rows are not contiguous: element path
            return (a.hd == 64 || a.hd == 128) ? kDecRegQ8 : kDecAsyncQ8;
    }
    return kDecSync;
}

template <int HD>
int launch_decode_q8reg(const FattnArgs& a, cudaStream_t st) {
    // a cluster launch carries the receive area of the merge behind the stages; the attribute is raised once, to that size
    const size_t smem_main = (size_t)kDecRows * HD * sizeof(__half) + (size_t)kDecRegStages * 2 * kDecBN * (HD / 32 * 34);
    const size_t smem_attr = smem_main + cluster_push_bytes(HD, kDecRows);
    const size_t smem = smem_main + (use_cluster_merge(a) ? cluster_push_bytes(HD, a.Tq * a.gqa) : 0);
    dim3 grid(a.n_splits, a.Hkv, a.B);
    cudaError_t e;
    // B200_DECODE_Q8T=0 keeps the rows-on-M register kernel, =1 (default) the keys-on-M kernel with F16 score MMAs, =2
    // the keys-on-M kernel with int8 score MMAs (measured equal at 256 streams, 5 % slower at 8: its set-up; A/B runs)
    static const int keys_on_m = [] {
        const char* e = getenv("B200_DECODE_Q8T");
        return (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
    }();
    if (keys_on_m == 2 && !a.has_mask && a.softcap == 0.0f && !a.causal && a.Tq * a.gqa <= 8) {
        auto kern = fattn_decode_q8t_kernel<HD, true>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (keys_on_m == 1 && !a.has_mask && a.softcap == 0.0f && !a.causal && a.Tq * a.gqa <= 8) {
        auto kern = fattn_decode_q8t_kernel<HD, false>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (!a.has_mask && a.softcap == 0.0f && !a.causal && a.Tq * a.gqa <= 8) {
        auto kern = fattn_decode_q8reg_kernel<HD, true, true>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else if (!a.has_mask && a.softcap == 0.0f && !a.causal) {
        auto kern = fattn_decode_q8reg_kernel<HD, true, false>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    } else {
        auto kern = fattn_decode_q8reg_kernel<HD, false, false>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem_attr, smem_set);
        if (e != cudaSuccess) return (int)e;
        launch_split(kern, grid, smem, st, a);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (a.n_splits > 1 && !use_cluster_merge(a)) e = launch_merge<HD>(a, st);
    return (int)e;
}

template <int HD>
int launch_decode_t(const FattnArgs& a, cudaStream_t st) {
    switch (decode_mode(a, HD)) {
        case kDecRegQ8:
            if constexpr (HD == 64 || HD == 128) return launch_decode_q8reg<HD>(a, st);
            else return launch_decode_m<HD, kDecAsyncQ8>(a, st);
        case kDecAsyncF16: return launch_decode_m<HD, kDecAsyncF16>(a, st);
        case kDecAsyncQ8: return launch_decode_m<HD, kDecAsyncQ8>(a, st);
        default: return launch_decode_m<HD, kDecSync>(a, st);
    }
}

// K or V of any supported type / stride -> contiguous F16 [hd, Lk, Hkv, Bk] (the operand form of the tcgen05 kernels).
// blockIdx.y selects the tensor: K and V of one call are converted by one launch.
__global__ void kv_to_f16_kernel(const View src0, uint8_t* dst0, const View src1, uint8_t* dst1, int hd, int Lk, int Hkv, int Bk) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the attention kernel may start its set-up
    const View& src = blockIdx.y ? src1 : src0;
    uint8_t* dst = blockIdx.y ? dst1 : dst0;
    const int cpr = hd / 8;
    const int64_t total = (int64_t)Bk * Hkv * Lk * cpr;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int ch = (int)(i % cpr);
        const int64_t row = i / cpr;  // ((b*Hkv + h)*Lk + k)
        const int k = (int)(row % Lk);
        const int h = (int)((row / Lk) % Hkv);
        const int b = (int)(row / ((int64_t)Lk * Hkv));
        const uint8_t* rowp = src.p + (int64_t)k * src.nb1 + (int64_t)h * src.nb2 + (int64_t)b * src.nb3;
        *reinterpret_cast<uint4*>(dst + (row * cpr + ch) * 16) = load8_as_half(rowp, src.type, ch * 8, hd, src.vec16 != 0);
    }
}

}  // namespace

int launch_kv_to_f16(const View& src, void* dst, int hd, int Lk, int Hkv, int Bk, cudaStream_t st) {
    const int64_t total = (int64_t)Bk * Hkv * Lk * (hd / 8);
    const int blocks = (int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256);
    kv_to_f16_kernel<<<dim3(blocks, 1), 256, 0, st>>>(src, (uint8_t*)dst, src, (uint8_t*)dst, hd, Lk, Hkv, Bk);
    return (int)cudaGetLastError();
}

int launch_kv_pair_to_f16(const View& k, void* kdst, const View& v, void* vdst, int hd, int Lk, int Hkv, int Bk, cudaStream_t st) {
    const int64_t total = (int64_t)Bk * Hkv * Lk * (hd / 8);
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    kv_to_f16_kernel<<<dim3(blocks, 2), 256, 0, st>>>(k, (uint8_t*)kdst, v, (uint8_t*)vdst, hd, Lk, Hkv, Bk);
    return (int)cudaGetLastError();
}

int launch_tile_mma(const FattnArgs& a, cudaStream_t st) {
    const int hdp = a.hd <= 32 ? 32 : (a.hd <= 64 ? 64 : 128);
    if (a.relpos) {
        if (hdp == 32) return launch_tile_t<32, true>(a, st);
        if (hdp == 64) return launch_tile_t<64, true>(a, st);
        return launch_tile_t<128, true>(a, st);
    }
    if (hdp == 32) return launch_tile_t<32, false>(a, st);
    if (hdp == 64) return launch_tile_t<64, false>(a, st);
    return launch_tile_t<128, false>(a, st);
}

int launch_decode_split(const FattnArgs& a, cudaStream_t st) {
    const int hdp = a.hd <= 32 ? 32 : (a.hd <= 64 ? 64 : 128);
    if (hdp == 32) return launch_decode_t<32>(a, st);
    if (hdp == 64) return launch_decode_t<64>(a, st);
    return launch_decode_t<128>(a, st);
}

size_t decode_split_ws_bytes(int B, int Hkv, int n_splits, int hd) {
    if (n_splits <= 1) return 0;
    const int hdp = hd <= 32 ? 32 : (hd <= 64 ? 64 : 128);
    const size_t units = (size_t)B * Hkv * n_splits;
    const size_t o = units * kDecRows * hdp * sizeof(float);
    const size_t ml = units * kDecRows * 2 * sizeof(float);
    return ((o + 255) / 256) * 256 + ((ml + 255) / 256) * 256;
}

bool decode_uses_cluster_merge(const FattnArgs& a) { return use_cluster_merge(a); }

#ifdef B200_Q8T_TRACE
extern "C" __attribute__((visibility("default"))) int b200_dbg_q8t_trace(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_q8t_trace, sizeof(long long) * 16);
}
#endif

int mma_read_status(int* status) {
    int v = 0;
    const cudaError_t e = cudaMemcpyFromSymbol(&v, g_mma_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    *status = v;
    return 0;
}

int mma_reset_status() {
    const int zero = 0;
    return (int)cudaMemcpyToSymbol(g_mma_status, &zero, sizeof(int));
}

namespace {
// One warp arms nothing and waits on its own mbarrier for at most `polls` polls: the wait must run out, set the
// status word and let the kernel return.  Exercises the failure path of mbar_wait_bounded without a fault.
__global__ void bounded_wait_probe_kernel(uint32_t polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    mbar_wait_bounded(smem_u32(&bar), 0u, polls);
}
}  // namespace

namespace {
__global__ void empty_kernel() {}
}  // namespace

int launch_empty(cudaStream_t st) {
    empty_kernel<<<1, 32, 0, st>>>();
    return (int)cudaGetLastError();
}

int launch_bounded_wait_probe(int polls, cudaStream_t st) {
    bounded_wait_probe_kernel<<<1, 32, 0, st>>>((uint32_t)polls);
    return (int)cudaGetLastError();
}

bool decode_cluster_merge_ok(const FattnArgs& a) {
    return cluster_merge_enabled() && (a.k.type == B200_TYPE_Q8_0 || a.k.type == B200_TYPE_F16) && (a.hd == 64 || a.hd == 128);
}

// CTAs of the split kernel that fit on one SM for these operands (shared memory of the staging form; registers
// allow four).
int decode_ctas_per_sm(const FattnArgs& a, bool cluster) {
    const int hdp = a.hd <= 32 ? 32 : (a.hd <= 64 ? 64 : 128);
    size_t smem;
    switch (decode_mode(a, hdp)) {
        case kDecRegQ8: smem = (size_t)kDecRows * hdp * 2 + (size_t)kDecRegStages * 2 * kDecBN * (hdp / 32 * 34); break;
        case kDecAsyncF16: {
            const int ns = hdp >= 128 ? 3 : 4;
            smem = (size_t)(kDecRows + ns * 2 * kDecBN) * hdp * 2;
            if (a.has_mask && a.mask.vec16) smem += (size_t)ns * (a.Tq * a.gqa) * kDecBN * 2;
            break;
        }
        case kDecAsyncQ8: smem = (size_t)(kDecRows + kDecBN) * hdp * 2 + (size_t)kDecQ8Stages * 2 * kDecBN * (hdp / 32 * 34); break;
        default: smem = (size_t)(kDecRows + 2 * kDecBN) * hdp * 2; break;
    }
    if (cluster) smem += cluster_push_bytes(hdp, a.Tq * a.gqa);   // the receive area of the merge
    const int n = (int)((size_t)227 * 1024 / (smem + 640 + 1024));   // static shared memory of the kernels, 1 KB the system keeps per CTA
    return n < 1 ? 1 : (n > 4 ? 4 : n);
}

// Split count of the KV range for `B` batch entries of these operands.  A small cost model in units of one 64-key
// tile of one CTA: a split costs its tiles plus 1.5 (set-up, epilogue) plus its share of the merge (1.0 through the
// workspace and the merge kernel, 0.5 inside a cluster), the grid runs in whole waves while it is at most four waves
// long, and a merge kernel adds its launch latency (1.5) and 0.2 per split it has to read (0.1 inside a cluster).  The candidates it separates were measured on the Q8_0
// kernel (9 tiles): 16 streams 3 splits 47.3 k vs 5 splits 38.0 k stream-steps/s; 32 streams 2 vs 3 splits 58.3 k
// vs 54.3 k; 64 streams 1 vs 2 splits 80.9 k vs 68.7 k.
static std::atomic<int> g_forced_splits{0};
void decode_split_force(int n_splits) { g_forced_splits.store(n_splits, std::memory_order_relaxed); }

int decode_split_choose(const FattnArgs& a, int B, int sm_count) {
    const int forced = g_forced_splits.load(std::memory_order_relaxed);
    static const int per_sm_env = [] {  // B200_DECODE_CTAS_PER_SM=1..16 overrides the resident-CTA estimate
        const char* e = getenv("B200_DECODE_CTAS_PER_SM");
        const int n = e ? atoi(e) : 0;
        return n >= 1 && n <= 16 ? n : 0;
    }();
    const int tiles = ((a.kv_index ? a.kv_index_stride : a.Lk) + kDecBN - 1) / kDecBN;
    if (tiles <= 1) return 1;
    if (forced) return forced < tiles ? forced : tiles;
    const double units = (double)B * a.Hkv;
    const double cap = (double)(per_sm_env ? per_sm_env : decode_ctas_per_sm(a)) * sm_count;
    const double cap_cluster = (double)(per_sm_env ? per_sm_env : decode_ctas_per_sm(a, true)) * sm_count;   // with the receive area of the merge
    const bool cluster_ok = decode_cluster_merge_ok(a);
    int best = 1;
    double best_cost = 0.0;
    for (int n = 1; n <= tiles && n <= 64; n++) {
        const int tps = (tiles + n - 1) / n;
        if ((tiles + tps - 1) / tps != n) continue;   // some split would get no tile
        const double w = units * n / cap;
        const double waves = w <= 4.0 ? ceil(w) : w + 0.5;
        const bool cluster = cluster_ok && n > 1 && n <= 8 && units * n <= cap_cluster;
        double cost = waves * (tps + 1.5 + (n == 1 ? 0.0 : (cluster ? 0.5 : 1.0)));
        // the merge reads n partials per output row.  F16 kernel (100 KB CTAs, merge kernel launched under its tail):
        // merge kernel 0.8 + 0.2 n, cluster 1.0 + 0.1 n, fitted to one segment of Whisper cross-attention (24 tiles:
        // 8 cluster splits 5.54 k segment-steps/s, 12 workspace splits 4.67 k) and of the pooled self-attention (36
        // tiles: 12 workspace splits 3.95 k, 18: 3.61 k, 6 / 8 cluster splits 3.91 / 3.83 k) and to 2 / 4 / 8 segments.
        // Q8_0 kernel through the workspace: 3.0 + 0.2 n (32 streams: one split 80.0 k stream-steps/s, two 71.9 k)
        const bool f16 = a.k.type == B200_TYPE_F16;
        if (n > 1) cost += cluster ? (f16 ? 1.0 : 0.0) + 0.1 * n : (f16 ? 0.8 : 3.0) + 0.2 * n;
        if (n == 1 || cost < best_cost - 1e-9) best = n, best_cost = cost;
    }
    return best;
}

}  // namespace b200
