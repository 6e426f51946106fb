// fattn_tc5.cu — prefill attention on the Blackwell tensor path: TMA-staged K/V tiles, tcgen05.mma
// with accumulators in tensor memory (TMEM), fp32 online softmax by one thread per query row.
//
// One CTA = one 128-row query tile of one (head, batch entry); 192 threads:
//   warps 0-3  softmax / correction / epilogue: thread r owns query row r (TMEM lane r)
//   warp  4    TMA producer (one lane): K and V tiles of 128 keys, 128-byte swizzled
//   warp  5    TMEM allocator and the single tcgen05.mma issuing thread
// TMEM (256 columns per CTA, so two CTAs share an SM and fill each other's softmax bubbles):
//   cols [0,128)       S = Q.K^T tile, fp32            (128 lanes x 128 keys)
//   cols [0,64)        P = exp2(S - m), f16x2 packed    (aliases S once the row has been read)
//   cols [128,128+HD)  O accumulator, fp32
// Shared memory: Q tile (written once by the softmax warps, converted to f16, swizzled by hand so
// both F32 and F16 Q with any strides work), NSTG K tiles and NSTG V tiles (TMA, SWIZZLE_128B).
// Per KV tile: S = Q.K^T (SS MMA, both operands K-major) -> softmax threads read S, write P to TMEM
// -> O += P.V (TS MMA: A = P from TMEM, B = V from shared memory, MN-major).
// The rescale of O by exp2(m_old - m_new) is lazy: it only happens when a row's maximum grew by
// more than 2^8, so P stays within f16 range and the common case touches O only in the MMA.
//
// Every mbarrier wait is bounded: when a wait runs out the CTA raises a flag, all roles leave their
// loops, in-flight copies are drained (bounded), TMEM is released and a device status word is set.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "fattn_tc5.cuh"

namespace b200 {

__device__ int g_tc5_status = 0;  // 0 ok, 1 = a bounded wait ran out in some CTA

#ifdef B200_TC5_TRACE
__device__ long long g_tc5_trace[3][64][8];
#ifndef B200_TC5_TRACE_Z
#define B200_TC5_TRACE_Z 0
#endif
#define TC5_TRACE(role, j, k) do { if (blockIdx.x == 1 && blockIdx.y == 3 && blockIdx.z == B200_TC5_TRACE_Z && (j) < 64) g_tc5_trace[role][j][k] = clock64(); } while (0)
#else
#define TC5_TRACE(role, j, k) do { } while (0)
#endif

namespace {

constexpr int kTile = 128;              // query rows per CTA and keys per step
constexpr int kPanelBytes = 128 * 128;  // 128 rows x 64 f16
constexpr int kThreadsTc5 = 192;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: P <= 256 stays well inside f16 range

// ---- PTX wrappers -----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test.  The answer takes about 120 clocks to come back even when the phase completed long ago, so a
// wait whose barrier is normally complete is probed early (the result is consumed after other work) and only falls
// back to the polling wait when the probe said no.
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait. Returns false when the CTA is aborting (this wait or another one ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t it = 0; it < kWaitLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 256) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    atomicExch(&g_tc5_status, 1);
    return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Tensor store shared -> global as its own bulk group; the caller waits for the group's reads of shared memory
// before the CTA ends.  The innermost coordinate times the element size must be a multiple of 16 bytes, and no
// coordinate may be negative.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Shared-memory matrix descriptor, SWIZZLE_128B, descriptor version 1 (sm_100).
//   K-major operand : rows of 128 bytes, 8-row groups 1024 bytes apart  -> LBO = 16 B (unused), SBO = 1024 B
//   MN-major operand: 64-element chunks `lbo` bytes apart, 8-k groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;   // version
    d |= (uint64_t)2 << 61;   // SWIZZLE_128B
    return d;
}

// The two 32-bit words of a descriptor.  Only the low word carries the address (bits 0-13, in 16-byte units),
// so stepping through an operand is one 32-bit add: the issuing thread's instruction latency, not the tensor
// pipe, bounds how fast small MMAs can be issued.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ constexpr uint32_t smem_desc_hi(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// Instruction descriptor for kind::f16: F16 A/B, F32 accumulate, M = 128.
__host__ __device__ constexpr uint32_t idesc_f16(int n, bool b_mn_major) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTile >> 4) << 24);
}

__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32 pairs (one issue slot for two lanes of work on sm_100) and the three-input maximum.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Eight Q elements [c0, c0+8) of one row as packed f16 (F32 rows are rounded to nearest even).
__device__ __forceinline__ uint4 q_chunk(const uint8_t* rowp, int type, int c0, bool vec16) {
    uint4 out;
    if (type == B200_TYPE_F16) {
        if (vec16) return __ldg(reinterpret_cast<const uint4*>(rowp + 2 * c0));
        const uint16_t* h = reinterpret_cast<const uint16_t*>(rowp + 2 * c0);
        out.x = h[0] | ((uint32_t)h[1] << 16), out.y = h[2] | ((uint32_t)h[3] << 16);
        out.z = h[4] | ((uint32_t)h[5] << 16), out.w = h[6] | ((uint32_t)h[7] << 16);
        return out;
    }
    float f[8];
    if (vec16) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(rowp + 4 * c0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(rowp + 4 * c0 + 16));
        f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) f[i] = *reinterpret_cast<const float*>(rowp + 4 * (c0 + i));
    }
    out.x = pack_half2(f[0], f[1]), out.y = pack_half2(f[2], f[3]);
    out.z = pack_half2(f[4], f[5]), out.w = pack_half2(f[6], f[7]);
    return out;
}

// {hi, lo} -> packed f16x2 with lo in the low half
__device__ __forceinline__ uint32_t cvt_f16x2(float lo, float hi) {
    uint32_t y;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(y) : "f"(hi), "f"(lo));
    return y;
}
// Maximum of 64 score columns held in two 32-register chunks; columns >= n_valid (tile-relative) are skipped.
__device__ __forceinline__ float row_max64(const uint32_t (&sreg)[2][32], int col0, int n_valid) {
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float s0 = (col0 + q2 * 32 + i < n_valid) ? __uint_as_float(sreg[q2][i]) : -INFINITY;
            const float s1 = (col0 + q2 * 32 + i + 1 < n_valid) ? __uint_as_float(sreg[q2][i + 1]) : -INFINITY;
            mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], s0, s1);
        }
    return max3(fmaxf(mx[0], mx[1]), mx[2], mx[3]);
}

// 64 score columns -> 32 packed f16x2 probabilities exp2(s*c - m); updates the running raw maximum and the
// row sum (f16x2 partial sums of four pairs, widened to fp32).
template <bool MASKED>
__device__ __forceinline__ void softmax64(const uint32_t (&sreg)[2][32], uint32_t (&preg)[32], float c, float m_use,
                                          int col0, int n_valid, float& mx_io, float& lsum_io) {
    // Per pair of columns: one three-input max, one packed FMA, two MUFU, one packed add, one f16x2 convert.
    float mx[8];
    uint64_t ls[4] = {0ull, 0ull, 0ull, 0ull};   // four packed pairs of fp32 partial sums
    const uint64_t c2 = pack2(c, c), nm2 = pack2(-m_use, -m_use);
#pragma unroll
    for (int i = 0; i < 8; i++) mx[i] = -INFINITY;
#pragma unroll
    for (int q2 = 0; q2 < 2; q2++) {
        if (MASKED && col0 + q2 * 32 >= n_valid) {   // a 32-column chunk beyond the last key: P = 0 without the exponentials
#pragma unroll
            for (int i = 0; i < 16; i++) preg[q2 * 16 + i] = 0u;
            continue;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float s0 = __uint_as_float(sreg[q2][i]), s1 = __uint_as_float(sreg[q2][i + 1]);
            if (MASKED) {
                if (col0 + q2 * 32 + i >= n_valid) s0 = -INFINITY;
                if (col0 + q2 * 32 + i + 1 >= n_valid) s1 = -INFINITY;
            }
            mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], s0, s1);
            float t0, t1;
            unpack2(fma2(pack2(s0, s1), c2, nm2), t0, t1);
            const float p0 = ex2(t0), p1 = ex2(t1);
            ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
            preg[q2 * 16 + (i >> 1)] = cvt_f16x2(p0, p1);
        }
    }
    mx_io = max3(mx_io, max3(fmaxf(mx[0], mx[1]), mx[2], mx[3]), max3(fmaxf(mx[4], mx[5]), mx[6], mx[7]));
    float l0, l1;
    unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), l0, l1);
    lsum_io += l0 + l1;
}

// One 32-column chunk of the same arithmetic with the accumulators kept by the caller (mx[8], ls[4] live across the
// four chunks of a tile): lets the TMEM load of a later chunk run under the exponentials of an earlier one.
template <bool MASKED>
__device__ __forceinline__ void softmax32(const uint32_t (&sreg)[32], uint32_t* preg16, uint64_t c2, uint64_t nm2, int col0, int n_valid,
                                          float (&mx)[8], uint64_t (&ls)[4]) {
    if (MASKED && col0 >= n_valid) {
#pragma unroll
        for (int i = 0; i < 16; i++) preg16[i] = 0u;
        return;
    }
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        float s0 = __uint_as_float(sreg[i]), s1 = __uint_as_float(sreg[i + 1]);
        if (MASKED) {
            if (col0 + i >= n_valid) s0 = -INFINITY;
            if (col0 + i + 1 >= n_valid) s1 = -INFINITY;
        }
        mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], s0, s1);
        float t0, t1;
        unpack2(fma2(pack2(s0, s1), c2, nm2), t0, t1);
        const float p0 = ex2(t0), p1 = ex2(t1);
        ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
        preg16[i >> 1] = cvt_f16x2(p0, p1);
    }
}

// 64 consecutive F16 mask values starting at `mptr` as eight 16-byte loads, all in flight at once (2-byte loads
// where the address is not 16-byte aligned); values at or beyond `avail` (the end of the mask row) read as 0 and
// are never touched in memory.
__device__ __forceinline__ void load_mask64(uint4 (&mv)[8], const uint8_t* mptr, int avail) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
        if (q * 8 + 8 <= avail && ((reinterpret_cast<uintptr_t>(mptr) & 15) == 0)) {
            mv[q] = __ldg(reinterpret_cast<const uint4*>(mptr + q * 16));
        } else {   // the end of the row, or a row that does not start on a 16-byte boundary (mask rows hold exactly Lk values)
            uint16_t hv[8];
#pragma unroll
            for (int i = 0; i < 8; i++)
                hv[i] = (q * 8 + i < avail) ? __ldg(reinterpret_cast<const uint16_t*>(mptr + (q * 8 + i) * 2)) : (uint16_t)0;
            mv[q] = make_uint4(hv[0] | ((uint32_t)hv[1] << 16), hv[2] | ((uint32_t)hv[3] << 16), hv[4] | ((uint32_t)hv[5] << 16),
                               hv[6] | ((uint32_t)hv[7] << 16));
        }
    }
}
// Mask value pair (columns i, i+1 of the 64, i even) of a block loaded by load_mask64.
__device__ __forceinline__ float2 mask_pair(const uint4 (&mv)[8], int i) {
    const uint4& v = mv[i >> 3];
    const int u = (i & 7) >> 1;
    const uint32_t w = u == 0 ? v.x : (u == 1 ? v.y : (u == 2 ? v.z : v.w));
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// Explicit F16 mask: turns 64 raw scores into log2-domain logits t = s*c + mask*log2(e) in place (mask -inf stays
// -inf).  `mptr` points at the mask value of the first of the 64 columns, `avail` is how many mask columns exist
// from there to the end of the mask row (loads never go past it).
__device__ __forceinline__ void apply_mask64(uint32_t (&sreg)[2][32], const uint8_t* mptr, int avail, float c) {
    uint4 mv[8];
    load_mask64(mv, mptr, avail);
#pragma unroll
    for (int i = 0; i < 64; i += 2) {
        const float2 m2 = mask_pair(mv, i);
        sreg[i >> 5][i & 31] = __float_as_uint(fmaf(__uint_as_float(sreg[i >> 5][i & 31]), c, m2.x * kLog2e));
        sreg[i >> 5][(i + 1) & 31] = __float_as_uint(fmaf(__uint_as_float(sreg[i >> 5][(i + 1) & 31]), c, m2.y * kLog2e));
    }
}

// Explicit mask, fused form: 64 raw scores and their 64 mask values -> probabilities in one pass,
// x = s*c + (mask*log2(e) - m) with two packed FMAs per pair (folding the mask into the scores first and subtracting the
// maximum afterwards costs four scalar operations more per pair, and this path is bound by instruction issue).  The
// running maximum is tracked on x; the caller adds m back.  Columns >= n_valid (tile-relative) are dead.
template <bool MASKED>
__device__ __forceinline__ void softmax64_masked(const uint32_t (&sreg)[2][32], const uint4 (&mv)[8], uint32_t (&preg)[32], float c,
                                                 float m_use, int col0, int n_valid, float& mx_io, float& lsum_io) {
    float mx[8];
    uint64_t ls[4] = {0ull, 0ull, 0ull, 0ull};
    const uint64_t c2 = pack2(c, c), l2e2 = pack2(kLog2e, kLog2e), nm2 = pack2(-m_use, -m_use);
#pragma unroll
    for (int i = 0; i < 8; i++) mx[i] = -INFINITY;
#pragma unroll
    for (int i = 0; i < 64; i += 2) {
        const float2 m2 = mask_pair(mv, i);
        float x0, x1;
        unpack2(fma2(pack2(__uint_as_float(sreg[i >> 5][i & 31]), __uint_as_float(sreg[i >> 5][(i + 1) & 31])), c2,
                     fma2(pack2(m2.x, m2.y), l2e2, nm2)), x0, x1);
        if (MASKED) {
            if (col0 + i >= n_valid) x0 = -INFINITY;
            if (col0 + i + 1 >= n_valid) x1 = -INFINITY;
        }
        mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], x0, x1);
        const float p0 = ex2(x0), p1 = ex2(x1);
        ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
        preg[i >> 1] = cvt_f16x2(p0, p1);
    }
    mx_io = max3(mx_io, max3(fmaxf(mx[0], mx[1]), mx[2], mx[3]), max3(fmaxf(mx[4], mx[5]), mx[6], mx[7]));
    float l0, l1;
    unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), l0, l1);
    lsum_io += l0 + l1;
}

// One query row (HD elements) -> f16, written into the 128-byte swizzled operand tile: row r, 16-byte chunk c of
// panel p at p*16384 + r*128 + ((c ^ (r & 7)) * 16).  The type is tested once and all loads of the row are issued
// before the first store, so the row costs one memory round trip instead of HD/8.
template <int HD>
__device__ __forceinline__ void load_q_row(uint8_t* tile, int r, const uint8_t* rowp, int type, bool vec16, bool valid) {
    uint4 v[HD / 8];
    if (!valid) {
#pragma unroll
        for (int c = 0; c < HD / 8; c++) v[c] = make_uint4(0u, 0u, 0u, 0u);
    } else if (type == B200_TYPE_F16 && vec16) {
#pragma unroll
        for (int c = 0; c < HD / 8; c++) v[c] = __ldg(reinterpret_cast<const uint4*>(rowp) + c);
    } else if (type == B200_TYPE_F32 && vec16) {
#pragma unroll
        for (int c0 = 0; c0 < HD / 8; c0 += 4) {  // 4 chunks = 8 float4 in flight
            float4 f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __ldg(reinterpret_cast<const float4*>(rowp) + c0 * 2 + i);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v[c0 + i].x = pack_half2(f[2 * i].x, f[2 * i].y), v[c0 + i].y = pack_half2(f[2 * i].z, f[2 * i].w);
                v[c0 + i].z = pack_half2(f[2 * i + 1].x, f[2 * i + 1].y), v[c0 + i].w = pack_half2(f[2 * i + 1].z, f[2 * i + 1].w);
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < HD / 8; c++) v[c] = q_chunk(rowp, type, c * 8, false);
    }
    uint8_t* dst_row = tile + r * 128;
#pragma unroll
    for (int c = 0; c < HD / 8; c++)
        *reinterpret_cast<uint4*>(dst_row + (c >> 3) * kPanelBytes + (((c & 7) ^ (r & 7)) << 4)) = v[c];
}

struct Tc5Smem {
    // offsets from the 1024-byte aligned base of dynamic shared memory
    template <int HD, int NSTG>
    static constexpr int tile_bytes() { return kPanelBytes * (HD / 64); }
};

// Coalesced forms of the two per-row transfers of a CTA.  A thread that moves its own row makes every warp instruction
// touch 32 rows (32 sectors for 16 bytes each); here a warp instruction covers whole rows, the row pointers travel by
// shuffle from the lanes that own them (lane i of warp w owns row 32w + i).
//
// F32 query rows -> f16 operand tile: per instruction RPI = 128 / HD rows, lane l reads float4 number l % (HD/4) of row
// l / (HD/4), converts and writes 8 bytes into the swizzled tile.  A null row pointer gives a zero row.
template <int HD>
__device__ __forceinline__ void load_q_rows_f32_coalesced(uint8_t* tile, int warp, int lane, const uint8_t* my_rowp) {
    constexpr int F4 = HD / 4, RPI = 32 / F4;   // float4 per row; rows per warp instruction
    const uint32_t plo = (uint32_t)reinterpret_cast<uintptr_t>(my_rowp), phi = (uint32_t)(reinterpret_cast<uintptr_t>(my_rowp) >> 32);
    const int c = lane % F4, sub = lane / F4;
#pragma unroll
    for (int batch = 0; batch < 32 / RPI / 16; batch++) {
        float4 f[16];
#pragma unroll
        for (int k = 0; k < 16; k++) {
            const int src = (batch * 16 + k) * RPI + sub;
            const uintptr_t p = (uintptr_t)__shfl_sync(0xffffffffu, plo, src) | ((uintptr_t)__shfl_sync(0xffffffffu, phi, src) << 32);
            f[k] = p ? __ldg(reinterpret_cast<const float4*>(p) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < 16; k++) {
            const int row = warp * 32 + (batch * 16 + k) * RPI + sub;
            const int cc = c >> 1;   // 16-byte chunk of the f16 row
            *reinterpret_cast<uint2*>(tile + (cc >> 3) * kPanelBytes + row * 128 + (((cc & 7) ^ (row & 7)) << 4) + (c & 1) * 8) =
                make_uint2(pack_half2(f[k].x, f[k].y), pack_half2(f[k].z, f[k].w));
        }
    }
}

// The same for F16 query rows: a row is HD / 8 16-byte chunks, 256 / HD rows per warp instruction, copied as they are.
template <int HD>
__device__ __forceinline__ void load_q_rows_f16_coalesced(uint8_t* tile, int warp, int lane, const uint8_t* my_rowp) {
    constexpr int C16 = HD / 8, RPI = 32 / C16;
    const uint32_t plo = (uint32_t)reinterpret_cast<uintptr_t>(my_rowp), phi = (uint32_t)(reinterpret_cast<uintptr_t>(my_rowp) >> 32);
    const int cc = lane % C16, sub = lane / C16;
    uint4 v[32 / RPI];
#pragma unroll
    for (int k = 0; k < 32 / RPI; k++) {
        const int src = k * RPI + sub;
        const uintptr_t p = (uintptr_t)__shfl_sync(0xffffffffu, plo, src) | ((uintptr_t)__shfl_sync(0xffffffffu, phi, src) << 32);
        v[k] = p ? __ldg(reinterpret_cast<const uint4*>(p) + cc) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int k = 0; k < 32 / RPI; k++) {
        const int row = warp * 32 + k * RPI + sub;
        *reinterpret_cast<uint4*>(tile + (cc >> 3) * kPanelBytes + row * 128 + (((cc & 7) ^ (row & 7)) << 4)) = v[k];
    }
}

// Output rows: each thread parks its scaled row in its warp's staging area (chunks swizzled by the row), then the warp
// writes whole rows.  `stage` is this warp's 32 * HD floats; a null row pointer skips the row.
template <int HD>
__device__ __forceinline__ void store_o_rows_coalesced(float* stage, int lane, float* my_out) {
    constexpr int F4 = HD / 4, RPI = 32 / F4;
    __syncwarp();
    const uint32_t plo = (uint32_t)reinterpret_cast<uintptr_t>(my_out), phi = (uint32_t)(reinterpret_cast<uintptr_t>(my_out) >> 32);
    const int c = lane % F4, sub = lane / F4;
#pragma unroll 4
    for (int k = 0; k < 32 / RPI; k++) {
        const int row = k * RPI + sub;
        const uintptr_t p = (uintptr_t)__shfl_sync(0xffffffffu, plo, row) | ((uintptr_t)__shfl_sync(0xffffffffu, phi, row) << 32);
        const float4 v = *reinterpret_cast<const float4*>(stage + row * HD + ((c ^ (row & 7)) << 2));
        if (p) *(reinterpret_cast<float4*>(p) + c) = v;
    }
}

// EARLY (head_dim 64 without explicit mask; A/B variants, both measured slower than EARLY = 0 and opt-in):
//   1  a softmax thread pulls its whole 128-column score row into registers at the start of a tile and says so
//      (s_read); the MMA thread issues S[j+1] right then instead of after P[j], so the next score tile is computed
//      under the exponentials of the current one.  With 168 registers per thread the row spills: 0.6x.
//   2  the score columns are released after the SECOND 64-column half is in registers (no extra registers); a half
//      that outgrew the reference maximum is redone from registers and the other half's probabilities are scaled.
//      The score MMAs and the P.V MMAs are issued from two warps on two schedulers, each refilling the K (V) slots
//      its own MMAs free.  Tile period of a traced CTA about equal to EARLY = 0; whole launches 0.79x.
// QMODE / OTMA: how the query tile comes in and the output tile goes out (see q_tma below).  Template parameters, not
// run-time flags: every path compiled into one kernel costs the others (the raw F32 form behind a flag took 5 % off the
// F16-Q encoder launches and 9 % off the T = 407 prefill).
template <int HD, int NSTG, bool HASMASK, int EARLY = 0, int QMODE = 0, bool OTMA = false>
__global__ void __launch_bounds__(kThreadsTc5, 2)
fattn_prefill_tc5_kernel(const FattnArgs a, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQ,
                         const __grid_constant__ CUtensorMap tmO) {
    constexpr int q_tma = QMODE;
    constexpr bool o_tma = OTMA;
    constexpr int PANELS = HD / 64;
    constexpr int TILE_BYTES = kPanelBytes * PANELS;
    constexpr uint32_t IDESC_S = idesc_f16(kTile, false);
    constexpr uint32_t IDESC_PV = idesc_f16(HD, true);

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
    const uint32_t sQ = smem_base;
    const uint32_t sK = sQ + TILE_BYTES;
    const uint32_t sV = sK + NSTG * TILE_BYTES;
    const uint32_t sBar = sV + NSTG * TILE_BYTES;  // 8-byte slots
    const uint32_t bar_k_full = sBar, bar_k_empty = sBar + 8 * NSTG, bar_v_full = sBar + 16 * NSTG,
                   bar_v_empty = sBar + 24 * NSTG, bar_s_full = sBar + 32 * NSTG, bar_p_ready = bar_s_full + 8,
                   bar_o_done = bar_s_full + 16, bar_pv_done = bar_s_full + 24, bar_s_read = bar_s_full + 32,
                   bar_s_drain = bar_s_full + 40, bar_q_full = bar_s_full + 48, bar_q_conv = bar_s_full + 56;
    uint8_t* misc = smem_gen + (1 + 2 * NSTG) * TILE_BYTES + 32 * NSTG + 64;
    // q_tma: 0 = the softmax warps load and convert the Q tile; 1 = F16 rows by one tensor copy into the operand tile;
    // 2 = F32 rows by tensor copies into stages that are not needed yet, converted from there by the softmax warps.
    // head_dim 128 (the form that is launched): the raw tile (64 KB) takes the K and the V stage, so the first K tile
    // waits for the conversion too - still ahead of a register pass, whose global loads a CTA next to one in its key
    // loop issues at a few tens of clocks per instruction (T = 407 GQA prefill with an F32 Q: 4807 -> 5034 streams/s).
    // head_dim 64 (the raw tile in the two V stages) measured 1459 against 1481 segments/s for the register pass on the
    // encoder and is not launched.
    constexpr bool RAW_OK = QMODE == 2 && EARLY == 0 && ((HD == 64 && NSTG == 2) || (HD == 128 && NSTG == 1));
    static_assert(QMODE != 2 || RAW_OK, "the raw form needs stages to park the tile in");
    constexpr int RAW_OFF = HD == 64 ? (1 + NSTG) * TILE_BYTES : TILE_BYTES;   // V stages / K stage onwards
    constexpr bool q_raw = RAW_OK;
    // head_dim 64 leaves 64 spare TMEM columns: P gets its own, so S of the next tile can be issued before P.V
    constexpr bool SEP_P = (HD == 64);
    volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(misc);
    volatile int* s_abort = reinterpret_cast<volatile int*>(misc + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // launched with programmatic stream serialisation: nothing is read or written before the previous kernel of the
    // stream (e.g. the K/V conversion pass) has completed and flushed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Causal launches hand out the query tiles with the most KV tiles first (longest-processing-time order over
    // the whole grid: the tile index becomes the slowest-varying coordinate, reversed), which shortens the tail of
    // short prefills; otherwise consecutive CTAs are the query tiles of one head, which share K/V in L2.
    // GQA packing: the grid runs over KV heads, and a CTA's 128 rows are (query position, head of the group) pairs -
    // packed row q0 + r is query (q0 + r) / gqa of head hk*gqa + (q0 + r) % gqa.  The heads of a group share their
    // K/V tiles, and a short causal prefill covers fewer, fuller tiles (gqa = 1: the plain one-head tile).
    int q0 = blockIdx.x * kTile, hk = blockIdx.y, b = blockIdx.z;
    if (a.causal) {
        const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z), hb = gridDim.y * gridDim.z;
        q0 = (gridDim.x - 1 - lin / hb) * kTile;
        hk = (lin % hb) % gridDim.y, b = (lin % hb) / gridDim.y;
    }
    const int bk = b / a.bq;
    const int rows_total = a.Tq * a.gqa;   // packed rows of this (kv head, batch entry)
    const int tq_b = q_rows_of(a, b);      // query rows at or beyond it are padding of a batched launch: zeros
    const int rows_live = tq_b * a.gqa;

    int len_b = a.Lk;
    if (a.kv_len) {
        const int v = a.kv_len[b];
        len_b = v < 0 ? 0 : (v > a.Lk ? a.Lk : v);
    }
    const int n_past = n_past_of(a, len_b, tq_b);
    int kmax = q0 < rows_live ? len_b : 0;   // a tile of padding rows reads no keys
    if (a.causal) kmax = min(kmax, n_past + min((q0 + kTile - 1) / a.gqa + 1, tq_b));
    const int n_tiles = kmax > 0 ? (kmax + kTile - 1) / kTile : 0;

    if (n_tiles == 0) {  // nothing to attend to: zeros
        if (tid < kTile && q0 + tid < rows_total) {
            const int iq = (q0 + tid) / a.gqa, h = hk * a.gqa + (q0 + tid) % a.gqa;
            float4* out = reinterpret_cast<float4*>(a.dst + (((int64_t)b * a.Tq + iq) * a.H + h) * HD);
#pragma unroll
            for (int i = 0; i < HD / 4; i++) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        return;
    }

    // ---- set-up ----
    if (tid == 0) TC5_TRACE(2, 60, 0);
    if (tid == 4 * 32) {
        for (int i = 0; i < NSTG; i++) {
            mbar_init(bar_k_full + 8 * i, 1);
            mbar_init(bar_k_empty + 8 * i, 1);
            mbar_init(bar_v_full + 8 * i, 1);
            mbar_init(bar_v_empty + 8 * i, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_p_ready, 4);   // one arrival per softmax warp
        mbar_init(bar_o_done, 1);
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_s_read, 4);    // one arrival per softmax warp
        mbar_init(bar_s_drain, 1);
        mbar_init(bar_q_full, 1);
        mbar_init(bar_q_conv, 4);    // one arrival per softmax warp
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (q_raw) {
            // HD / 32 panels of 128 rows x 32 floats, rows in packed order like the F16 box
            mbar_arrive_expect_tx(bar_q_full, (HD / 32) * kPanelBytes);
#pragma unroll
            for (int p = 0; p < HD / 32; p++)
                tma_load_4d(sQ + RAW_OFF + p * kPanelBytes, &tmQ, bar_q_full, p * 32, hk * a.gqa, q0 / a.gqa, b);
        } else if (q_tma) {
            // F16 query rows go straight into the operand layout: one copy instead of a pass through the softmax warps'
            // registers, which a CTA sharing its SM with another one in its key loop executes at a few tens of clocks
            // per instruction.  The box is [64 columns, the gqa heads of the group, 128 / gqa tokens]: its rows land in
            // packed order (token-major, head of the group minor).  Tokens at or beyond Tq read as zeros.
            mbar_arrive_expect_tx(bar_q_full, TILE_BYTES);
#pragma unroll
            for (int p = 0; p < PANELS; p++) tma_load_4d(sQ + p * kPanelBytes, &tmQ, bar_q_full, p * 64, hk * a.gqa, q0 / a.gqa, b);
        }
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
        // the first NSTG tiles need no empty-slot wait: start their copies before the CTA-wide set-up barrier
        for (int j = 0; j < NSTG && j < n_tiles; j++) {
            if (q_raw && HD == 128) continue;   // the K stage holds raw Q rows for now
            mbar_arrive_expect_tx(bar_k_full + 8 * j, TILE_BYTES);
#pragma unroll
            for (int p = 0; p < PANELS; p++)
                tma_load_4d(sK + j * TILE_BYTES + p * kPanelBytes, &tmK, bar_k_full + 8 * j, p * 64, j * kTile, hk, bk);
            if (q_raw) continue;   // the V stages hold the raw Q tile for now
            mbar_arrive_expect_tx(bar_v_full + 8 * j, TILE_BYTES);
#pragma unroll
            for (int p = 0; p < PANELS; p++)
                tma_load_4d(sV + j * TILE_BYTES + p * kPanelBytes, &tmV, bar_v_full + 8 * j, p * 64, j * kTile, hk, bk);
        }
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(s_tmem_base))),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        if (lane == 0) TC5_TRACE(2, 61, 0);
    }
    if (warp < 4 && !q_tma) {
        // Q tile -> shared memory (thread r writes row r)
        const int r = tid;
        const int iq = (q0 + r) / a.gqa, h = hk * a.gqa + (q0 + r) % a.gqa;
        const uint8_t* rowp = a.q.p + (int64_t)iq * a.q.nb1 + (int64_t)h * a.q.nb2 + (int64_t)b * a.q.nb3;
        if (a.q.type == B200_TYPE_F32 && a.q.vec16) load_q_rows_f32_coalesced<HD>(smem_gen, warp, lane, q0 + r < rows_total ? rowp : nullptr);
        else if (a.q.type == B200_TYPE_F16 && a.q.vec16) load_q_rows_f16_coalesced<HD>(smem_gen, warp, lane, q0 + r < rows_total ? rowp : nullptr);
        else load_q_row<HD>(smem_gen, r, rowp, a.q.type, a.q.vec16 != 0, q0 + r < rows_total);
        fence_proxy_async();
        if (tid == 0) TC5_TRACE(2, 61, 1);
    }
    if (tid == 4 * 32) TC5_TRACE(2, 61, 2);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;
    if (tid == 0) TC5_TRACE(2, 60, 1);
    const uint32_t tmem_S = tmem_base;            // cols [0,128)
    const uint32_t tmem_P = SEP_P ? tmem_base + kTile + HD : tmem_base;  // f16x2: cols [192,256) (hd 64) or aliasing S [0,64)
    const uint32_t tmem_O = tmem_base + kTile;    // cols [128,128+HD)
    if constexpr (RAW_OK) {
        if (q_raw && warp < 4) {
            // raw F32 row r (panels of 128-byte swizzled rows) -> F16 row r of the operand tile: HD / 4 loads, HD / 2
            // conversions, HD / 8 stores per thread, all from shared memory
            if (mbar_wait(bar_q_full, 0, s_abort)) {
                const int r = tid;
                const uint8_t* raw = smem_gen + RAW_OFF + r * 128;
                uint8_t* qrow = smem_gen + r * 128;
#pragma unroll
                for (int c = 0; c < HD / 8; c++) {   // F16 chunk c = columns 8c .. 8c+7 = F32 chunks 2c, 2c+1 of raw panel c / 4
                    const int f0 = (2 * c) & 7;
                    const float4 x0 = *reinterpret_cast<const float4*>(raw + (c >> 2) * kPanelBytes + ((f0 ^ (r & 7)) << 4));
                    const float4 x1 = *reinterpret_cast<const float4*>(raw + (c >> 2) * kPanelBytes + (((f0 + 1) ^ (r & 7)) << 4));
                    *reinterpret_cast<uint4*>(qrow + (c >> 3) * kPanelBytes + (((c & 7) ^ (r & 7)) << 4)) =
                        make_uint4(pack_half2(x0.x, x0.y), pack_half2(x0.z, x0.w), pack_half2(x1.x, x1.y), pack_half2(x1.z, x1.w));
                }
                fence_proxy_async();   // the operand tile is read, and the V stages are overwritten, through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_q_conv);
            }
        }
    }

    if (EARLY != 2 && warp == 4) {
        // ================= TMA producer =================
        if (lane == 0) {
            bool ok = true;
            int issued_k = (q_raw && HD == 128) ? 0 : min(NSTG, n_tiles), issued_v = q_raw ? 0 : min(NSTG, n_tiles);
            if (q_raw) {
                ok = mbar_wait(bar_q_conv, 0, s_abort);
                for (int j = 0; j < NSTG && j < n_tiles && ok; j++) {
                    if (HD == 128) {
                        mbar_arrive_expect_tx(bar_k_full + 8 * j, TILE_BYTES);
#pragma unroll
                        for (int p = 0; p < PANELS; p++)
                            tma_load_4d(sK + j * TILE_BYTES + p * kPanelBytes, &tmK, bar_k_full + 8 * j, p * 64, j * kTile, hk, bk);
                        issued_k = j + 1;
                    }
                    mbar_arrive_expect_tx(bar_v_full + 8 * j, TILE_BYTES);
#pragma unroll
                    for (int p = 0; p < PANELS; p++)
                        tma_load_4d(sV + j * TILE_BYTES + p * kPanelBytes, &tmV, bar_v_full + 8 * j, p * 64, j * kTile, hk, bk);
                    issued_v = j + 1;
                }
            }
            for (int j = NSTG; j < n_tiles && ok; j++) {
                const int slot = j % NSTG, use = j / NSTG;
                const int k0 = j * kTile;
                ok = mbar_wait(bar_k_empty + 8 * slot, (use - 1) & 1, s_abort);
                if (!ok) break;
                TC5_TRACE(2, j, 0);
                mbar_arrive_expect_tx(bar_k_full + 8 * slot, TILE_BYTES);
#pragma unroll
                for (int p = 0; p < PANELS; p++)
                    tma_load_4d(sK + slot * TILE_BYTES + p * kPanelBytes, &tmK, bar_k_full + 8 * slot, p * 64, k0, hk, bk);
                issued_k = j + 1;
                ok = mbar_wait(bar_v_empty + 8 * slot, (use - 1) & 1, s_abort);
                if (!ok) break;
                TC5_TRACE(2, j, 1);
                mbar_arrive_expect_tx(bar_v_full + 8 * slot, TILE_BYTES);
#pragma unroll
                for (int p = 0; p < PANELS; p++)
                    tma_load_4d(sV + slot * TILE_BYTES + p * kPanelBytes, &tmV, bar_v_full + 8 * slot, p * 64, k0, hk, bk);
                issued_v = j + 1;
            }
            if (!ok) {
                // drain: wait (bounded) for the copies this thread still has in flight
                if (q_tma)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_q_full, 0); ++it) __nanosleep(256);
                for (int j = max(0, issued_k - NSTG); j < issued_k; j++)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_k_full + 8 * (j % NSTG), (j / NSTG) & 1); ++it) __nanosleep(256);
                for (int j = max(0, issued_v - NSTG); j < issued_v; j++)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_v_full + 8 * (j % NSTG), (j / NSTG) & 1); ++it) __nanosleep(256);
            }
        }
    } else if (EARLY == 2 && warp == 4) {
        // ================= K loader + score-MMA issuer (half-tile release variant) =================
        // An issuing thread costs the other warps of its scheduler issue slots (60-80 clk per tcgen05 instruction), and
        // a tile ends when the slowest softmax warp is done: the two products are issued from two schedulers, and each
        // issuer refills the operand slots its own MMAs free (their completion lies a tile back: no real wait).
        if (lane == 0) {
            const uint32_t q_lo = smem_desc_lo(sQ, 16), k_lo = smem_desc_lo(sK, 16);
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            bool ok = true;
            int issued_k = min(NSTG, n_tiles);
            for (int j = 0; j < n_tiles && ok; j++) {   // S[j]
                const int slot = j % NSTG, use = j / NSTG;
                // K[j+1] goes into the slot S[j-1] read (NSTG = 2); the softmax warps are already working on that product
                const int jn = j + NSTG - 1;
                if (j > 0 && jn < n_tiles) {
                    const int ns = jn % NSTG, nu = jn / NSTG;
                    ok = mbar_wait(bar_k_empty + 8 * ns, (nu - 1) & 1, s_abort);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_k_full + 8 * ns, TILE_BYTES);
#pragma unroll
                    for (int p = 0; p < PANELS; p++)
                        tma_load_4d(sK + ns * TILE_BYTES + p * kPanelBytes, &tmK, bar_k_full + 8 * ns, p * 64, jn * kTile, hk, bk);
                    issued_k = jn + 1;
                }
                ok = mbar_wait(bar_k_full + 8 * slot, use & 1, s_abort);
                if (ok && j > 0) ok = mbar_wait(bar_s_read, (j - 1) & 1, s_abort);   // every softmax warp holds S[j-1] in registers
                if (!ok) break;
                if (j > 0) TC5_TRACE(1, j - 1, 0);
                tc_fence_after();
                const uint32_t kd = k_lo + slot * (TILE_BYTES >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t off16 = (uint32_t)(((ks >> 2) * kPanelBytes + (ks & 3) * 32) >> 4);
                    mma_ss(tmem_S, desc64(q_lo + off16, desc_hi), desc64(kd + off16, desc_hi), IDESC_S, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full);
                tc_commit(bar_k_empty + 8 * slot);
                if (j > 0) TC5_TRACE(1, j - 1, 1);
            }
            if (!ok) {   // no score MMA and no K copy of this CTA may still be running when the CTA ends
                tc_commit(bar_s_drain);
                for (uint32_t it = 0; it < 65536 && !mbar_try_wait(bar_s_drain, 0); ++it) __nanosleep(256);
                for (int j = max(0, issued_k - NSTG); j < issued_k; j++)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_k_full + 8 * (j % NSTG), (j / NSTG) & 1); ++it) __nanosleep(256);
            }
        }
    } else if (EARLY == 2 && warp == 5) {
        // ================= V loader + P.V-MMA issuer (half-tile release variant) =================
        if (lane == 0) {
            const uint32_t v_lo = smem_desc_lo(sV, kPanelBytes);
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            bool ok = true;
            int issued_v = min(NSTG, n_tiles);
            for (int j = 0; j < n_tiles && ok; j++) {
                const int slot = j % NSTG, use = j / NSTG;
                // V[j+1] goes into the slot P.V[j-1] read; that product was issued a tile ago
                const int jn = j + NSTG - 1;
                if (j > 0 && jn < n_tiles) {
                    const int ns = jn % NSTG, nu = jn / NSTG;
                    ok = mbar_wait(bar_v_empty + 8 * ns, (nu - 1) & 1, s_abort);
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar_v_full + 8 * ns, TILE_BYTES);
#pragma unroll
                    for (int p = 0; p < PANELS; p++)
                        tma_load_4d(sV + ns * TILE_BYTES + p * kPanelBytes, &tmV, bar_v_full + 8 * ns, p * 64, jn * kTile, hk, bk);
                    issued_v = jn + 1;
                }
                ok = mbar_wait(bar_v_full + 8 * slot, use & 1, s_abort);
                TC5_TRACE(1, j, 2);
                if (ok) ok = mbar_wait(bar_p_ready, j & 1, s_abort);
                if (!ok) break;
                TC5_TRACE(1, j, 3);
                tc_fence_after();
                const uint32_t vd = v_lo + slot * (TILE_BYTES >> 4);
                mma_ts(tmem_O, tmem_P, desc64(vd, desc_hi), IDESC_PV, j > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < kTile / 16; ks++) mma_ts(tmem_O, tmem_P + ks * 8, desc64(vd + ks * (2048 >> 4), desc_hi), IDESC_PV, 1u);
                tc_commit(bar_v_empty + 8 * slot);
                tc_commit(bar_pv_done);
                if (j + 1 == n_tiles) tc_commit(bar_o_done);
                TC5_TRACE(1, j, 4);
            }
            if (!ok) {
                tc_commit(bar_o_done);
                for (uint32_t it = 0; it < 65536 && !mbar_try_wait(bar_o_done, 0); ++it) __nanosleep(256);
                for (int j = max(0, issued_v - NSTG); j < issued_v; j++)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_v_full + 8 * (j % NSTG), (j / NSTG) & 1); ++it) __nanosleep(256);
            }
        }
    } else if (warp == 5) {
        // ================= MMA issuer =================
        // Order: S[0]; then per tile j: (barriers of tile j+1 are awaited while the softmax of tile j runs)
        // wait P[j] -> PV[j] -> S[j+1], back to back, so the softmax threads of the next tile wake as early
        // as the tensor pipe allows.  S[j+1] overwrites the columns P[j] lives in; tcgen05.mma executes in
        // issue order, so PV[j] has consumed P[j] before S[j+1] writes.
        if (lane == 0) {
            const uint32_t q_lo = smem_desc_lo(sQ, 16), k_lo = smem_desc_lo(sK, 16), v_lo = smem_desc_lo(sV, kPanelBytes);
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            bool ok = mbar_wait(bar_k_full, 0, s_abort);
            if (ok && q_tma) ok = mbar_wait(q_raw ? bar_q_conv : bar_q_full, 0, s_abort);
            if (ok) {
                TC5_TRACE(1, 0, 0);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t off = (ks >> 2) * kPanelBytes + (ks & 3) * 32;
                    mma_ss(tmem_S, smem_desc(sQ + off, 16, 1024), smem_desc(sK + off, 16, 1024), IDESC_S, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full);
                tc_commit(bar_k_empty);
                TC5_TRACE(1, 0, 1);
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                const int slot = j % NSTG, use = j / NSTG;
                const int nslot = (j + 1) % NSTG, nuse = (j + 1) / NSTG;
                const bool more = j + 1 < n_tiles;
                if (EARLY) {
                    // the score columns are free once all four softmax warps hold tile j in registers
                    if (more) ok = mbar_wait(bar_k_full + 8 * nslot, nuse & 1, s_abort);
                    if (ok) ok = mbar_wait(bar_s_read, j & 1, s_abort);
                    if (!ok) break;
                    if (j > 0) TC5_TRACE(1, j, 0);
                    if (more) {
                        tc_fence_after();
                        const uint32_t kd = k_lo + nslot * (TILE_BYTES >> 4);
#pragma unroll
                        for (int ks = 0; ks < HD / 16; ks++) {
                            const uint32_t off16 = (uint32_t)(((ks >> 2) * kPanelBytes + (ks & 3) * 32) >> 4);
                            mma_ss(tmem_S, desc64(q_lo + off16, desc_hi), desc64(kd + off16, desc_hi), IDESC_S, ks > 0 ? 1u : 0u);
                        }
                        tc_commit(bar_s_full);
                        tc_commit(bar_k_empty + 8 * nslot);
                    }
                    if (j > 0) TC5_TRACE(1, j, 1);
                    ok = mbar_wait(bar_v_full + 8 * slot, use & 1, s_abort);
                } else {
                    ok = mbar_wait(bar_v_full + 8 * slot, use & 1, s_abort);
                    if (ok && more) ok = mbar_wait(bar_k_full + 8 * nslot, nuse & 1, s_abort);
                }
                if (!ok) break;
                TC5_TRACE(1, j, 2);
                ok = mbar_wait(bar_p_ready, j & 1, s_abort);
                if (!ok) break;
                TC5_TRACE(1, j, 3);
                tc_fence_after();
                // Descriptors differ only in the low word (address in 16-byte units): one add per MMA.  The issuing
                // thread's latency, about 50 clocks per MMA and 100 per commit, is what the softmax threads wait for.
                auto issue_next_s = [&]() {
                    const uint32_t kd = k_lo + nslot * (TILE_BYTES >> 4);
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++) {
                        const uint32_t off16 = (uint32_t)(((ks >> 2) * kPanelBytes + (ks & 3) * 32) >> 4);
                        mma_ss(tmem_S, desc64(q_lo + off16, desc_hi), desc64(kd + off16, desc_hi), IDESC_S, ks > 0 ? 1u : 0u);
                    }
                    tc_commit(bar_s_full);
                };
                // with P in its own columns the next S goes first: the softmax threads wake after 4 MMAs, not 12
                if (SEP_P && more && !EARLY) issue_next_s();
                const uint32_t vd = v_lo + slot * (TILE_BYTES >> 4);
                mma_ts(tmem_O, tmem_P, desc64(vd, desc_hi), IDESC_PV, j > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < kTile / 16; ks++) mma_ts(tmem_O, tmem_P + ks * 8, desc64(vd + ks * (2048 >> 4), desc_hi), IDESC_PV, 1u);
                if (SEP_P) {
                    if (more && !EARLY) tc_commit(bar_k_empty + 8 * nslot);   // after the P.V MMAs: off the softmax threads' critical path
                    tc_commit(bar_v_empty + 8 * slot);
                    tc_commit(bar_pv_done);
                } else {
                    tc_commit(bar_v_empty + 8 * slot);
                    if (more) {
                        issue_next_s();
                        tc_commit(bar_k_empty + 8 * nslot);
                    }
                }
                if (!more) tc_commit(bar_o_done);
                TC5_TRACE(1, j, 4);
            }
            if (!ok) {
                // make sure no MMA of this CTA is still running before TMEM is released
                tc_commit(bar_o_done);
                for (uint32_t it = 0; it < 65536 && !mbar_try_wait(bar_o_done, 0); ++it) __nanosleep(256);
            }
        }
    } else {
        // ================= softmax / correction / epilogue =================
        const int r = tid;
        const bool row_live = q0 + r < rows_live;
        const bool row_zero = !row_live && q0 + r < rows_total;   // a padding row inside the tensor: its dst row is zero-filled
        const int iq_dst = (q0 + r) / a.gqa;
        const int iq = row_live ? iq_dst : a.Tq, h = hk * a.gqa + (q0 + r) % a.gqa;   // dead rows: iq = Tq
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const float c = a.scale * kLog2e;
        int kend = len_b;
        if (a.causal) kend = min(kend, n_past + iq + 1);
        float m_ref = -INFINITY, l_run = 0.0f;
        bool ok = true;
        // explicit mask row of this query ([Lk, Tq, 1|H, 1|B] F16); rows past Tq reuse row 0
        const uint8_t* mrow = HASMASK ? a.mask.p + (int64_t)(iq < a.Tq ? iq : 0) * a.mask.nb1 +
                                            (int64_t)(h % a.mask_ne2) * a.mask.nb2 + (int64_t)(b % a.mask_ne3) * a.mask.nb3
                                      : nullptr;
        const float c_exp = HASMASK ? 1.0f : c;   // with a mask the scores are moved to the log2 domain by apply_mask64
        if constexpr (EARLY == 1) {
            const uint64_t c2 = pack2(c, c);
            for (int j = 0; j < n_tiles; j++) {
                ok = mbar_wait(bar_s_full, j & 1, s_abort);
                if (!ok) break;
                if (tid == 0) TC5_TRACE(0, j, 0);
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) tmem_ld32(tmem_S + lane_base + q4 * 32, s[q4]);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_s_read);   // the tile is in registers: its columns may be overwritten
                if (tid == 0) TC5_TRACE(0, j, 3);
                const int n_valid = kend - j * kTile;     // columns >= n_valid of this row are masked
                const bool full = __all_sync(0xffffffffu, n_valid >= kTile);
                if (j == 0) {
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float x0 = (i < n_valid) ? __uint_as_float(s[0][i]) : -INFINITY;
                        const float x1 = (i + 1 < n_valid) ? __uint_as_float(s[0][i + 1]) : -INFINITY;
                        m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], x0, x1);
                    }
                    m_ref = max3(fmaxf(m4[0], m4[1]), m4[2], m4[3]) * c;
                }
                float lsum = 0.0f;
                bool pv_waited = false;
                for (int attempt = 0; attempt < 2; attempt++) {
                    const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
                    const uint64_t nm2 = pack2(-m_use, -m_use);
                    uint64_t ls[4] = {0ull, 0ull, 0ull, 0ull};
                    float mx[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) mx[i] = -INFINITY;
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        uint32_t preg[16];
                        if (full) {
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                const float s0 = __uint_as_float(s[q4][i]), s1 = __uint_as_float(s[q4][i + 1]);
                                mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], s0, s1);
                                float t0, t1;
                                unpack2(fma2(pack2(s0, s1), c2, nm2), t0, t1);
                                const float p0 = ex2(t0), p1 = ex2(t1);
                                ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
                                preg[i >> 1] = cvt_f16x2(p0, p1);
                            }
                        } else if (q4 * 32 >= n_valid) {
#pragma unroll
                            for (int i = 0; i < 16; i++) preg[i] = 0u;
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                float s0 = __uint_as_float(s[q4][i]), s1 = __uint_as_float(s[q4][i + 1]);
                                if (q4 * 32 + i >= n_valid) s0 = -INFINITY;
                                if (q4 * 32 + i + 1 >= n_valid) s1 = -INFINITY;
                                mx[(i >> 1) & 7] = max3(mx[(i >> 1) & 7], s0, s1);
                                float t0, t1;
                                unpack2(fma2(pack2(s0, s1), c2, nm2), t0, t1);
                                const float p0 = ex2(t0), p1 = ex2(t1);   // -inf -> 0
                                ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
                                preg[i >> 1] = cvt_f16x2(p0, p1);
                            }
                        }
                        if (q4 == 0 && j > 0 && !pv_waited) {
                            // the first 32 probabilities are in registers: only now must P[j-1] have been consumed
                            ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                            tc_fence_after();
                            pv_waited = true;
                        }
                        tmem_st16(tmem_P + lane_base + q4 * 16, preg);
                    }
                    if (!ok) break;
                    {
                        float l0, l1;
                        unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), l0, l1);
                        lsum = l0 + l1;
                    }
                    const float m_tile = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) * c;
                    if (!__any_sync(0xffffffffu, m_tile > m_ref + kRescaleThreshold)) break;
                    // some row of this warp outgrew its reference maximum: rescale O and l (O is at rest: pv_done was
                    // awaited above), then redo P from the registers
                    const float m_new = fmaxf(m_ref, m_tile);
                    const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_ref - m_new);
                    l_run *= alpha;
                    if (j > 0) {
                        tmem_wait_st();
#pragma unroll
                        for (int q4 = 0; q4 < HD / 32; q4++) {
                            uint32_t oreg[32];
                            tmem_ld32(tmem_O + lane_base + q4 * 32, oreg);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; i++) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                            tmem_st32(tmem_O + lane_base + q4 * 32, oreg);
                        }
                    }
                    m_ref = m_new;
                }
                if (!ok) break;
                l_run += lsum;
                if (tid == 0) TC5_TRACE(0, j, 1);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p_ready);
                if (tid == 0) TC5_TRACE(0, j, 2);
            }
        } else if constexpr (EARLY == 2) {
            // Half-tile release: the score columns are handed back (s_read) as soon as the second 64-column half is in
            // registers, so the tensor pipe computes S[j+1] under the exponentials of that half and the next tile's
            // scores are waiting when this loop comes round.  Nothing is read from the score columns afterwards: a
            // half that outgrew the reference maximum is redone from the registers it still sits in, and when that
            // is the second half the first half's probabilities (finite: they passed their own check) are scaled.
            for (int j = 0; j < n_tiles; j++) {
                ok = mbar_wait(bar_s_full, j & 1, s_abort);
                if (!ok) break;
                if (tid == 0) TC5_TRACE(0, j, 0);
                tc_fence_after();
                const int n_valid = kend - j * kTile;  // columns >= n_valid of this row are masked
                const bool full_tile = __all_sync(0xffffffffu, n_valid >= kTile);
                uint32_t preg[2][32];
                float lsum = 0.0f;
                bool pv_waited = false;
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    uint32_t sreg[2][32];
                    tmem_ld32(tmem_S + lane_base + hh * 64, sreg[0]);
                    tmem_ld32(tmem_S + lane_base + hh * 64 + 32, sreg[1]);
                    tmem_wait_ld();
                    if (hh == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_s_read);
                        if (lane == 0) TC5_TRACE(2, j, 2 + warp);
                    }
                    if (tid == 0) TC5_TRACE(0, j, 3 + 2 * hh);
                    if (HASMASK) apply_mask64(sreg, mrow + (int64_t)(j * kTile + hh * 64) * 2, a.Lk - (j * kTile + hh * 64), c);
                    if (j == 0 && hh == 0) m_ref = row_max64(sreg, 0, full_tile ? 2 * kTile : n_valid) * c_exp;
                    for (int attempt = 0; attempt < 2; attempt++) {
                        const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
                        float mx = -INFINITY, ls = 0.0f;
                        if (full_tile) softmax64<false>(sreg, preg[hh], c_exp, m_use, 0, 0, mx, ls);
                        else softmax64<true>(sreg, preg[hh], c_exp, m_use, hh * 64, n_valid, mx, ls);
                        const float m_tile = mx * c_exp;
                        if (attempt == 1 || !__any_sync(0xffffffffu, m_tile > m_ref + kRescaleThreshold)) {
                            lsum += ls;
                            break;
                        }
                        if (j > 0 && !pv_waited) {  // O must be at rest: P.V of the previous tile has completed
                            ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                            if (!ok) break;
                            tc_fence_after();
                            pv_waited = true;
                        }
                        const float m_new = fmaxf(m_ref, m_tile);
                        const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_ref - m_new);
                        l_run *= alpha;
                        lsum *= alpha;
                        if (hh == 1) {
                            const __half2 a2 = __float2half2_rn(alpha);
#pragma unroll
                            for (int i = 0; i < 32; i++) {
                                const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&preg[0][i]), a2);
                                preg[0][i] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                        }
                        if (j > 0) {
#pragma unroll
                            for (int q4 = 0; q4 < HD / 32; q4++) {
                                uint32_t oreg[32];
                                tmem_ld32(tmem_O + lane_base + q4 * 32, oreg);
                                tmem_wait_ld();
#pragma unroll
                                for (int i = 0; i < 32; i++) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                                tmem_st32(tmem_O + lane_base + q4 * 32, oreg);
                            }
                        }
                        m_ref = m_new;
                    }
                    if (!ok) break;
                    if (tid == 0) TC5_TRACE(0, j, 4 + 2 * hh);
                }
                if (!ok) break;
                l_run += lsum;
                if (j > 0 && !pv_waited) {  // P[j-1] must have been consumed before P[j] overwrites it
                    ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                    if (!ok) break;
                    tc_fence_after();
                }
                if (tid == 0) TC5_TRACE(0, j, 1);
                tmem_st32(tmem_P + lane_base, preg[0]);
                tmem_st32(tmem_P + lane_base + 32, preg[1]);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p_ready);
                if (tid == 0) TC5_TRACE(0, j, 2);
            }
        } else
        for (int j = 0; j < n_tiles; j++) {
            ok = mbar_wait(bar_s_full, j & 1, s_abort);
            if (!ok) break;
            if (tid == 0) TC5_TRACE(0, j, 0);
            tc_fence_after();
            const int n_valid = kend - j * kTile;  // columns >= n_valid of this row are masked
            const bool full_tile = __all_sync(0xffffffffu, n_valid >= kTile);
            if (j == 0) {
                // First tile: a first reference maximum.  Without a mask the maximum of the row's first 32 scores
                // is enough - it is rarely more than 2^8 below the row's real maximum, and when it is (or when those
                // columns are masked) the lazy-rescale check below redoes the tile against the exact maximum.
                float mx = -INFINITY;
                if (HASMASK) {
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        uint32_t sreg[2][32];
                        tmem_ld32(tmem_S + lane_base + hh * 64, sreg[0]);
                        tmem_ld32(tmem_S + lane_base + hh * 64 + 32, sreg[1]);
                        tmem_wait_ld();
                        apply_mask64(sreg, mrow + (int64_t)(j * kTile + hh * 64) * 2, a.Lk - (j * kTile + hh * 64), c);
                        mx = fmaxf(mx, row_max64(sreg, hh * 64, full_tile ? 2 * kTile : n_valid));
                    }
                } else {
                    uint32_t s0[32];
                    tmem_ld32(tmem_S + lane_base, s0);
                    tmem_wait_ld();
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float x0 = (i < n_valid) ? __uint_as_float(s0[i]) : -INFINITY;
                        const float x1 = (i + 1 < n_valid) ? __uint_as_float(s0[i + 1]) : -INFINITY;
                        m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], x0, x1);
                    }
                    mx = max3(fmaxf(m4[0], m4[1]), m4[2], m4[3]);
                }
                m_ref = mx * c_exp;  // c > 0
            }
            uint32_t preg[2][32];
            float lsum = 0.0f;
            bool pv_waited = false;
            uint32_t pv_probe = 0;   // early answer to "has P.V of the previous tile completed" (it normally has by mid-tile)
            for (int attempt = 0; attempt < 2; attempt++) {
                // P = exp2(S*c - m_ref), rounded to f16x2; the tile maximum is tracked in the same pass and
                // only checked afterwards (lazy rescale).
                const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
                float mx = -INFINITY;
                lsum = 0.0f;
                if constexpr (!HASMASK) {
                    // rolling 32-column chunks: the load of chunk k+2 is issued into the registers chunk k has just
                    // left and completes under the exponentials of chunk k+1
                    float mx8[8];
                    uint64_t ls4[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                    for (int i = 0; i < 8; i++) mx8[i] = -INFINITY;
                    const uint64_t c2 = pack2(c_exp, c_exp), nm2 = pack2(-m_use, -m_use);
                    uint32_t sA[32], sB[32];
                    // a partial tile (the last one, or the diagonal of a causal call) puts -inf into the dead columns
                    // first and skips chunks that are dead for the whole warp: one copy of the arithmetic serves both
                    auto chunk = [&](uint32_t (&sx)[32], uint32_t* p16, int col0) {
                        if (!full_tile) {
                            if (__all_sync(0xffffffffu, col0 >= n_valid)) {
#pragma unroll
                                for (int i = 0; i < 16; i++) p16[i] = 0u;
                                return;
                            }
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (col0 + i >= n_valid) sx[i] = 0xFF800000u;
                        }
                        softmax32<false>(sx, p16, c2, nm2, 0, 0, mx8, ls4);
                    };
                    tmem_ld32(tmem_S + lane_base, sA);
                    tmem_ld32(tmem_S + lane_base + 32, sB);
                    tmem_wait_ld();
                    chunk(sA, preg[0], 0);
                    tmem_ld32(tmem_S + lane_base + 64, sA);
                    if (SEP_P && j > 0 && !pv_waited && !pv_probe) pv_probe = mbar_test(bar_pv_done, (j - 1) & 1);
                    chunk(sB, preg[0] + 16, 32);
                    tmem_wait_ld();
                    tmem_ld32(tmem_S + lane_base + 96, sB);
                    chunk(sA, preg[1], 64);
                    tmem_wait_ld();
                    chunk(sB, preg[1] + 16, 96);
                    mx = max3(max3(fmaxf(mx8[0], mx8[1]), mx8[2], mx8[3]), max3(fmaxf(mx8[4], mx8[5]), mx8[6], mx8[7]), mx);
                    float l0, l1;
                    unpack2(add2(add2(ls4[0], ls4[1]), add2(ls4[2], ls4[3])), l0, l1);
                    lsum = l0 + l1;
                } else
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    uint32_t sreg[2][32];
                    tmem_ld32(tmem_S + lane_base + hh * 64, sreg[0]);
                    tmem_ld32(tmem_S + lane_base + hh * 64 + 32, sreg[1]);
                    if (SEP_P && hh == 1 && j > 0 && !pv_waited && !pv_probe) pv_probe = mbar_test(bar_pv_done, (j - 1) & 1);
                    tmem_wait_ld();
                    if (tid == 0) TC5_TRACE(0, j, 3 + 2 * hh);
                    if constexpr (HASMASK) {
                        uint4 mv[8];
                        load_mask64(mv, mrow + (int64_t)(j * kTile + hh * 64) * 2, a.Lk - (j * kTile + hh * 64));
                        if (full_tile) softmax64_masked<false>(sreg, mv, preg[hh], c, m_use, 0, 0, mx, lsum);
                        else softmax64_masked<true>(sreg, mv, preg[hh], c, m_use, hh * 64, n_valid, mx, lsum);
                    } else {
                        if (full_tile) softmax64<false>(sreg, preg[hh], c_exp, m_use, 0, 0, mx, lsum);
                        else softmax64<true>(sreg, preg[hh], c_exp, m_use, hh * 64, n_valid, mx, lsum);
                    }
                    if (tid == 0) TC5_TRACE(0, j, 4 + 2 * hh);
                }
                if (tid == 0 && attempt == 1) TC5_TRACE(0, j, 7);
                const float m_tile = HASMASK ? mx + m_use : mx * c_exp;   // (the masked form tracks the maximum of x = logit - m)
                const bool grow = m_tile > m_ref + kRescaleThreshold;
                if (!__any_sync(0xffffffffu, grow)) break;
                // some row of this warp outgrew its reference maximum: rescale O and l, then redo P
                if (SEP_P && j > 0 && !pv_waited) {  // O must be at rest: P.V of the previous tile has completed
                    ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                    if (!ok) break;
                    tc_fence_after();
                    pv_waited = true;
                }
                const float m_new = fmaxf(m_ref, m_tile);
                const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_ref - m_new);
                l_run *= alpha;
                if (j > 0) {
#pragma unroll
                    for (int q4 = 0; q4 < HD / 32; q4++) {
                        uint32_t oreg[32];
                        tmem_ld32(tmem_O + lane_base + q4 * 32, oreg);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                        tmem_st32(tmem_O + lane_base + q4 * 32, oreg);
                    }
                }
                m_ref = m_new;
            }
            if (!ok) break;
            l_run += lsum;
            if (SEP_P && j > 0 && !pv_waited) {  // P[j-1] must have been consumed before P[j] overwrites it
                if (!pv_probe) ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                if (!ok) break;
                tc_fence_after();
            }
            if (tid == 0) TC5_TRACE(0, j, 1);
            tmem_st32(tmem_P + lane_base, preg[0]);
            tmem_st32(tmem_P + lane_base + 32, preg[1]);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_ready);
            if (tid == 0) TC5_TRACE(0, j, 2);
        }
        if (ok) ok = mbar_wait(bar_o_done, 0, s_abort);
        if (tid == 0) TC5_TRACE(2, 60, 2);
        if (ok) {
            tc_fence_after();
            // dead rows are written as literal zeros (whatever the padding row of Q held never reaches dst), rows
            // outside the tensor not at all.  The K/V stages are free once the last MMA has completed: they stage O.
            const float inv = row_live && l_run > 0.0f ? 1.0f / l_run : 0.0f;
            float* out = (row_live || row_zero) ? a.dst + (((int64_t)b * a.Tq + iq_dst) * a.H + h) * HD : nullptr;
            float* stage = reinterpret_cast<float*>(smem_gen + TILE_BYTES) + warp * 32 * HD;
            if (o_tma) {
                // A warp's 32 packed rows x 32 columns are a box [32 columns, gqa heads, 32 / gqa tokens] of
                // dst [hd, H, Tq, B]; the warp parks them as 128-byte rows with the 16-byte chunks swizzled by the row (the
                // copy's own pattern, conflict-free for the stores) and one lane hands each panel to a tensor store,
                // which also clips the tokens beyond Tq.
#pragma unroll
                for (int q4 = 0; q4 < HD / 32; q4++) {
                    uint32_t oreg[32];
                    tmem_ld32(tmem_O + lane_base + q4 * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(stage + q4 * 32 * 32 + lane * 32 + (((i >> 2) ^ (lane & 7)) << 2)) =
                            row_live ? make_float4(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv,
                                                   __uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && q0 + warp * 32 < rows_total) {
#pragma unroll
                    for (int q4 = 0; q4 < HD / 32; q4++)
                        tma_store_4d(&tmO, smem_u32(stage + q4 * 32 * 32), q4 * 32, hk * a.gqa, (q0 + warp * 32) / a.gqa, b);
                    tma_store_commit_and_wait_read();
                }
            } else {
#pragma unroll
                for (int q4 = 0; q4 < HD / 32; q4++) {
                    uint32_t oreg[32];
                    tmem_ld32(tmem_O + lane_base + q4 * 32, oreg);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(stage + lane * HD + ((((q4 * 32 + i) >> 2) ^ (lane & 7)) << 2)) =
                            row_live ? make_float4(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv,
                                                   __uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                store_o_rows_coalesced<HD>(stage, lane, out);
            }
        }
    }

    // ---- teardown ----
    if (tid == 0) TC5_TRACE(2, 60, 3);
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------------
// Relative-position variant (FastConformer, head_dim 128): logits = scale*Q_u.K^T + f16(scale * relshift(Q_v.R^T)).
//
// Per 128x128 tile the bias needs X = Q_v[128 x hd] . R_band[256 x hd]^T with R_band = R rows
// [rb, rb+256), rb = (Tq-1) + k0 - q0 - 127; the bias of (row i, key j) is X[i][j - i + 127] (the rel-shift).
// X is one more accumulator in TMEM (256 columns; S 128, O 128 -> all 512 columns, one CTA per SM).
// A tcgen05.ld reads the same columns for every lane, so the per-row shift cannot be done in the load:
// each softmax thread loads the 96 columns its warp can need for half a tile, rounds scale*x to f16 (the
// reference's rounding point), parks them in its own row of a shared-memory buffer and reads 64 of them
// back from its row-dependent offset.  Only the thread itself touches its row: no barrier is involved.
// Consecutive KV tiles share half of the band, so R arrives in 128-row half-blocks through a 2-slot ring
// (half-block m = rows rb_0 + 128m ..; tile j uses half-blocks j and j+1).
// MMA order: X[0] S[0] | per tile j: X[j+1] as soon as the softmax threads have drained X[j]; then, once
// P[j] is in TMEM, PV[j] and S[j+1].
// ------------------------------------------------------------------------------------------------------
constexpr int kBncStride = 128;  // bytes per bounce row: a ring of 64 f16 values

constexpr int kThreadsRelpos = 320;  // 8 softmax warps (two threads per query row), TMA warp, MMA warp

template <bool HASMASK>
__global__ void __launch_bounds__(kThreadsRelpos, 1)
fattn_prefill_tc5_relpos_kernel(const FattnArgs a, const __grid_constant__ CUtensorMap tmK,
                                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmR) {
    constexpr int HD = 128;
    constexpr int TILE_BYTES = 2 * kPanelBytes;  // 128 rows x 128 halves
    constexpr uint32_t IDESC_S = idesc_f16(kTile, false);
    constexpr uint32_t IDESC_X = idesc_f16(2 * kTile, false);  // N = 256: the whole band in one instruction
    constexpr uint32_t IDESC_PV = idesc_f16(HD, true);

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
    const uint32_t sQ = smem_base, sQv = sQ + TILE_BYTES, sK = sQv + TILE_BYTES, sV = sK + TILE_BYTES,
                   sR = sV + TILE_BYTES, sBnc = sR + 2 * TILE_BYTES, sBar = sBnc + 2 * kTile * kBncStride;
    const uint32_t bar_k_full = sBar, bar_k_empty = sBar + 8, bar_v_full = sBar + 16, bar_v_empty = sBar + 24,
                   bar_r_full = sBar + 32 /* [2] */, bar_r_empty = sBar + 48 /* [2] */, bar_s_full = sBar + 64,
                   bar_x_full = sBar + 72, bar_x_free = sBar + 80, bar_p_ready = sBar + 88, bar_o_done = sBar + 96,
                   bar_pair = sBar + 104 /* [4]: the two warps that share 32 TMEM lanes */;
    uint8_t* misc = smem_gen + 6 * TILE_BYTES + 2 * kTile * kBncStride + 136;
    volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(misc);
    volatile int* s_abort = reinterpret_cast<volatile int*>(misc + 4);
    volatile float* s_xchg = reinterpret_cast<volatile float*>(misc + 8);   // [2][128]: row maximum exchange of a thread pair

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q0 = blockIdx.x * kTile, h = blockIdx.y, b = blockIdx.z;
    const int hk = h / a.gqa, bk = b / a.bq;
    const int rb3 = a.r_ne3 > 1 ? b : 0;

    int len_b = a.Lk;
    if (a.kv_len) {
        const int v = a.kv_len[b];
        len_b = v < 0 ? 0 : (v > a.Lk ? a.Lk : v);
    }
    const int tq_b = q_rows_of(a, b);   // query rows at or beyond it are padding of a batched launch: zeros
    const int n_tiles = (len_b > 0 && q0 < tq_b) ? (len_b + kTile - 1) / kTile : 0;
    if (n_tiles == 0) {
        if (tid < kTile && q0 + tid < a.Tq) {
            float4* out = reinterpret_cast<float4*>(a.dst + (((int64_t)b * a.Tq + q0 + tid) * a.H + h) * HD);
#pragma unroll
            for (int i = 0; i < HD / 4; i++) out[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    const int rb0 = a.Tq - 1 - q0 - 127;  // first R row of half-block 0 (may be negative: TMA zero-fills)

    // half-block m of R -> ring slot m % 2.  The ring is laid out panel-major, [panel 0: slot 0 | slot 1][panel 1:
    // slot 0 | slot 1] (16 KB each), so that per 64-column panel the 256 rows of both slots are contiguous and the
    // band GEMM can address them as one N = 256 operand.
    auto load_r = [&](int m) {
        const int slot = m & 1;
        mbar_arrive_expect_tx(bar_r_full + 8 * slot, TILE_BYTES);
        tma_load_4d(sR + slot * kPanelBytes, &tmR, bar_r_full + 8 * slot, 0, rb0 + kTile * m, h, rb3);
        tma_load_4d(sR + 2 * kPanelBytes + slot * kPanelBytes, &tmR, bar_r_full + 8 * slot, 64, rb0 + kTile * m, h, rb3);
    };
    auto load_kv = [&](int j, bool is_v) {
        const uint32_t bar = is_v ? bar_v_full : bar_k_full;
        const uint32_t dst = is_v ? sV : sK;
        mbar_arrive_expect_tx(bar, TILE_BYTES);
        tma_load_4d(dst, is_v ? &tmV : &tmK, bar, 0, j * kTile, hk, bk);
        tma_load_4d(dst + kPanelBytes, is_v ? &tmV : &tmK, bar, 64, j * kTile, hk, bk);
    };

    // ---- set-up ----
    if (tid == 8 * 32) {
        for (int i = 0; i < 17; i++) {
            const uint32_t bar = sBar + 8 * i;
            mbar_init(bar, (bar == bar_x_free || bar == bar_p_ready) ? 8 : (bar >= bar_pair ? 64 : 1));   // 8 = one arrival per softmax warp
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmR)) : "memory");
        load_r(0);
        load_r(1);
        load_kv(0, false);
        load_kv(0, true);
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(s_tmem_base))),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < 8) {
        // Q_u and Q_v tiles -> shared memory: thread (r, ch) converts and stores half of each row
        const int r = tid & 127, ch = tid >> 7;
        const int iq = q0 + r;
#pragma unroll
        for (int which = 0; which < 2; which++) {
            const View& qv = which ? a.qv : a.q;
            const uint8_t* rowp = qv.p + (int64_t)iq * qv.nb1 + (int64_t)h * qv.nb2 + (int64_t)b * qv.nb3;
            const float* bias = which ? a.bias_v : a.bias_u;  // untied position biases folded into the load
            uint4 v[HD / 16];
            if (bias != nullptr) {
#pragma unroll
                for (int c = 0; c < HD / 16; c++) {
                    const int c0 = (ch * (HD / 16) + c) * 8;
                    v[c] = (iq < a.Tq) ? load8_plus_bias_as_half(rowp, qv.type, c0, qv.vec16 != 0, bias + h * HD + c0)
                                       : make_uint4(0u, 0u, 0u, 0u);
                }
            } else {
#pragma unroll
                for (int c = 0; c < HD / 16; c++)
                    v[c] = (iq < a.Tq) ? q_chunk(rowp, qv.type, (ch * (HD / 16) + c) * 8, qv.vec16 != 0) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int c = 0; c < HD / 16; c++) {
                const int cc = ch * (HD / 16) + c;
                *reinterpret_cast<uint4*>(smem_gen + which * TILE_BYTES + r * 128 + (cc >> 3) * kPanelBytes + (((cc & 7) ^ (r & 7)) << 4)) = v[c];
            }
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;
    const uint32_t tmem_S = tmem_base, tmem_P = tmem_base, tmem_O = tmem_base + 128, tmem_X = tmem_base + 256;

    if (warp == 8) {
        // ================= TMA producer =================
        if (lane == 0) {
            bool ok = true;
            for (int j = 1; j < n_tiles && ok; j++) {
                // half-block j+1 goes into the slot half-block j-1 leaves once X[j-1] has been computed
                ok = mbar_wait(bar_r_empty + 8 * ((j + 1) & 1), (((j - 1) >> 1)) & 1, s_abort);
                if (!ok) break;
                load_r(j + 1);
                ok = mbar_wait(bar_k_empty, (j - 1) & 1, s_abort);
                if (!ok) break;
                load_kv(j, false);
                ok = mbar_wait(bar_v_empty, (j - 1) & 1, s_abort);
                if (!ok) break;
                load_kv(j, true);
            }
            if (!ok) {  // drain: bounded wait for copies still in flight
                for (uint32_t it = 0; it < 65536; ++it) __nanosleep(64);
            }
        }
    } else if (warp == 9) {
        // ================= MMA issuer =================
        if (lane == 0) {
            // X[j] = Q_v . [ring slot 0 | ring slot 1]^T as ONE N=256 MMA per k-step (A is fetched once instead of
            // twice).  Slot 0 holds half-block j for even j and half-block j+1 for odd j, so for odd j the two
            // 128-column halves of X come out swapped; the softmax threads account for that in their column base.
            auto issue_x = [&](int j) {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    // per panel: rows 0..127 of the B operand are slot 0, rows 128..255 slot 1 (contiguous 32 KB)
                    const uint32_t off = (ks >> 2) * kPanelBytes + (ks & 3) * 32;
                    const uint32_t roff = (ks >> 2) * 2 * kPanelBytes + (ks & 3) * 32;
                    mma_ss(tmem_X, smem_desc(sQv + off, 16, 1024), smem_desc(sR + roff, 16, 1024), IDESC_X, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_x_full);
                tc_commit(bar_r_empty + 8 * (j & 1));
            };
            auto issue_s = [&]() {
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const uint32_t off = (ks >> 2) * kPanelBytes + (ks & 3) * 32;
                    mma_ss(tmem_S, smem_desc(sQ + off, 16, 1024), smem_desc(sK + off, 16, 1024), IDESC_S, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full);
                tc_commit(bar_k_empty);
            };
            bool ok = mbar_wait(bar_r_full, 0, s_abort) && mbar_wait(bar_r_full + 8, 0, s_abort) &&
                      mbar_wait(bar_k_full, 0, s_abort);
            if (ok) {
                tc_fence_after();
                issue_x(0);
                issue_s();
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                const bool more = j + 1 < n_tiles;
                if (more) {
                    // X[j+1] needs half-block j+2 (slot j%2, its (j+2)/2-th use) and the X columns drained
                    ok = mbar_wait(bar_r_full + 8 * (j & 1), ((j + 2) >> 1) & 1, s_abort) &&
                         mbar_wait(bar_x_free, j & 1, s_abort);
                    if (!ok) break;
                    TC5_TRACE(1, j, 0);
                    tc_fence_after();
                    issue_x(j + 1);
                    TC5_TRACE(1, j, 1);
                }
                ok = mbar_wait(bar_v_full, j & 1, s_abort);
                if (ok && more) ok = mbar_wait(bar_k_full, (j + 1) & 1, s_abort);
                if (ok) ok = mbar_wait(bar_p_ready, j & 1, s_abort);
                if (!ok) break;
                TC5_TRACE(1, j, 2);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kTile / 16; ks++)
                    mma_ts(tmem_O, tmem_P + ks * 8, smem_desc(sV + ks * 2048, kPanelBytes, 1024), IDESC_PV,
                           (j > 0 || ks > 0) ? 1u : 0u);
                tc_commit(bar_v_empty);
                if (more) issue_s();
                else tc_commit(bar_o_done);
                TC5_TRACE(1, j, 3);
            }
            if (!ok) {
                tc_commit(bar_o_done);
                for (uint32_t it = 0; it < 65536 && !mbar_try_wait(bar_o_done, 0); ++it) __nanosleep(256);
            }
        }
    } else {
        // ================= softmax / bias / epilogue: thread (r, ch) owns columns [64ch, 64ch+64) of row r ========
        // Eight softmax warps: warps w and w+4 see the same 32 TMEM lanes. The two threads of a row agree on the
        // running maximum through shared memory and a 64-thread named barrier once per tile; each keeps a partial
        // row sum and owns half of the O columns.
        const int r = tid & 127, ch = tid >> 7;
        const int iq = q0 + r;
        const uint32_t my_pair_bar = bar_pair + 8 * (warp & 3);
        uint32_t pair_phase = 0;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const float bscale = a.relscale;   // == a.scale: the tcgen05 path is not taken with a softcap
        const uint64_t bscale2 = pack2(bscale, bscale);
        const int shift = 31 - lane;       // band offset of this row inside the warp's columns
        // Bounce ring of this thread: 64 f16 values (two 32-column chunks) = 32 words.
        uint8_t* const bnc_gen = smem_gen + (sBnc - smem_base) + tid * kBncStride;
        // rotation in words: 16-byte stores of the same logical chunk by the 8 lanes of a quarter-warp, and 4-byte
        // loads of logical word (const - lane/2) by all 32 lanes, both hit 32 distinct banks (found by enumeration)
        const uint32_t rot = 4u * ((lane + 3u * (lane >> 3)) & 7u);
        const uint32_t x_col0 = 96 - 32 * (warp & 3) + 64 * ch;   // first X column this thread's warp can need
        float m_ref = -INFINITY, l_run = 0.0f;
        bool ok = true;
        // Explicit F16 mask added on top of the bias (bucket padding of src/canary_ctc.cpp:370-382, the local-attention
        // window of src/core/fastconformer.h:887-895): this thread's row of [Lk, Tq, 1|H, 1|B];
        // rows past Tq (the padding rows of the last query tile) read row 0.
        const uint8_t* mrow = HASMASK ? a.mask.p + (int64_t)(iq < a.Tq ? iq : 0) * a.mask.nb1 +
                                            (int64_t)(h % a.mask_ne2) * a.mask.nb2 + (int64_t)(b % a.mask_ne3) * a.mask.nb3
                                      : nullptr;
        // Publish a value, meet the partner warp at the pair barrier (bounded wait), read the partner's value.
        // One slot per thread is enough: the partner's next write comes after its wait for the next S tile, which the
        // tensor pipe only produces after the P*V product that needed this thread's later arrival on bar_p_ready.
        auto exchange = [&](float mine) {
            s_xchg[ch * 128 + r] = mine;
            mbar_arrive(my_pair_bar);
            ok = mbar_wait(my_pair_bar, pair_phase, s_abort);
            pair_phase ^= 1;
            return s_xchg[(ch ^ 1) * 128 + r];
        };
        for (int j = 0; j < n_tiles; j++) {
            // ---- phase A: the 64 bias values of this half row, fp32 registers holding f16-rounded numbers ----
            ok = mbar_wait(bar_x_full, j & 1, s_abort);
            if (!ok) break;
            if (tid == 0) TC5_TRACE(0, j, 0);
            tc_fence_after();
            float u[2][32];
            auto bounce_chunk = [&](const uint32_t (&xr)[32], int k) {
                // scale*x rounded to f16 (the reference's cast of its mask), 32 values = 16 words, into ring half k&1
                uint32_t w[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    float x0, x1;
                    unpack2(mul2(pack2(__uint_as_float(xr[2 * i]), __uint_as_float(xr[2 * i + 1])), bscale2), x0, x1);
                    w[i] = cvt_f16x2(x0, x1);
                }
#pragma unroll
                for (int i = 0; i < 16; i += 4)
                    *reinterpret_cast<uint4*>(bnc_gen + ((((k & 1) * 16 + i + rot) & 31) << 2)) = make_uint4(w[i], w[i + 1], w[i + 2], w[i + 3]);
            };
            auto read_quarter = [&](int qq) {  // half-row columns [32qq, 32qq+32): ring halves shift .. shift+31 of chunks qq, qq+1
                const uint32_t h0 = (uint32_t)(qq * 32 + shift);
                const uint32_t fs = (h0 & 1u) * 16u;
                uint32_t prev = *reinterpret_cast<const uint32_t*>(bnc_gen + ((((h0 >> 1) + rot) & 31) << 2));
#pragma unroll
                for (int p2 = 0; p2 < 16; p2++) {
                    const uint32_t next = *reinterpret_cast<const uint32_t*>(bnc_gen + ((((h0 >> 1) + p2 + 1 + rot) & 31) << 2));
                    const uint32_t pk = __funnelshift_r(prev, next, fs);
                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&pk));
                    u[qq][2 * p2] = f2.x, u[qq][2 * p2 + 1] = f2.y;
                    prev = next;
                }
            };
            {
                const uint32_t xswap = (j & 1) ? 128u : 0u;  // odd tiles: the two 128-column halves of X are swapped
                uint32_t xa[3][32];
#pragma unroll
                for (int k = 0; k < 3; k++) tmem_ld32(tmem_X + lane_base + ((x_col0 + k * 32 + xswap) & 255u), xa[k]);
                tmem_wait_ld();
                // the X columns are free the moment every warp holds its 96 values in registers: X[j+1] is computed
                // under the rest of this tile instead of after the extraction
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_x_free);
                bounce_chunk(xa[0], 0);
                bounce_chunk(xa[1], 1);
                read_quarter(0);
                bounce_chunk(xa[2], 2);
                read_quarter(1);
            }
            if (tid == 0) TC5_TRACE(0, j, 1);
            uint4 mv[8];
            if (HASMASK) load_mask64(mv, mrow + (int64_t)(j * kTile + ch * 64) * 2, a.Lk - (j * kTile + ch * 64));   // in flight during the wait for S

            // ---- phase B: u = S*scale + bias (natural units), row maximum ----
            ok = mbar_wait(bar_s_full, j & 1, s_abort);
            if (!ok) break;
            if (tid == 0) TC5_TRACE(0, j, 2);
            tc_fence_after();
            const int n_valid = len_b - j * kTile;
            const bool full_tile = n_valid >= kTile;   // uniform over the CTA: only the last tile is partial
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            {
                uint32_t sreg[2][32];
                tmem_ld32(tmem_S + lane_base + ch * 64, sreg[0]);
                tmem_ld32(tmem_S + lane_base + ch * 64 + 32, sreg[1]);
                tmem_wait_ld();
#pragma unroll
                for (int q2 = 0; q2 < 2; q2++)
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float u0, u1;
                        unpack2(fma2(pack2(__uint_as_float(sreg[q2][i]), __uint_as_float(sreg[q2][i + 1])), bscale2,
                                     pack2(u[q2][i], u[q2][i + 1])), u0, u1);
                        if (HASMASK) {
                            const float2 m2 = mask_pair(mv, q2 * 32 + i);
                            u0 += m2.x, u1 += m2.y;
                        }
                        if (!full_tile) {
                            if (ch * 64 + q2 * 32 + i >= n_valid) u0 = -INFINITY;
                            if (ch * 64 + q2 * 32 + i + 1 >= n_valid) u1 = -INFINITY;
                        }
                        u[q2][i] = u0, u[q2][i + 1] = u1;
                        mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], u0, u1);
                    }
            }
            if (tid == 0) TC5_TRACE(0, j, 3);
            const float mx_half = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            // after this barrier both threads of the row have read their S columns: P stores may alias them
            const float m_tile = fmaxf(mx_half, exchange(mx_half)) * kLog2e;
            if (!ok) break;
            // lazy rescale: O and l are only touched when a row outgrew its reference maximum by 2^8; both warps of a
            // pair see the same row maxima and take the same branch
            const bool grow = m_tile > m_ref + kRescaleThreshold;  // also true for -inf -> finite
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_ref, m_tile);
                const float alpha = (m_ref == -INFINITY) ? 0.0f : ex2(m_ref - m_new);
                l_run *= alpha;
                if (j > 0) {
#pragma unroll
                    for (int q4 = 0; q4 < 2; q4++) {
                        uint32_t oreg[32];
                        tmem_ld32(tmem_O + lane_base + ch * 64 + q4 * 32, oreg);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                        tmem_st32(tmem_O + lane_base + ch * 64 + q4 * 32, oreg);
                    }
                }
                m_ref = m_new;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
            // P = exp2(u*log2(e) - m_ref) from registers; masked columns hold -inf and give 0
            uint64_t ls[4] = {0ull, 0ull, 0ull, 0ull};
            const uint64_t l2e2 = pack2(kLog2e, kLog2e), nm2 = pack2(-m_use, -m_use);
            uint32_t preg[32];
#pragma unroll
            for (int q2 = 0; q2 < 2; q2++)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float t0, t1;
                    unpack2(fma2(pack2(u[q2][i], u[q2][i + 1]), l2e2, nm2), t0, t1);
                    const float p0 = ex2(t0), p1 = ex2(t1);
                    ls[(i >> 1) & 3] = add2(ls[(i >> 1) & 3], pack2(p0, p1));
                    preg[q2 * 16 + (i >> 1)] = cvt_f16x2(p0, p1);
                }
            tmem_st32(tmem_P + lane_base + ch * 32, preg);
            {
                float l0, l1;
                unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), l0, l1);
                l_run += l0 + l1;
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_ready);
            if (tid == 0) TC5_TRACE(0, j, 4);
        }
        if (ok) ok = mbar_wait(bar_o_done, 0, s_abort);
        if (ok) {
            tc_fence_after();
            const float l_tot = l_run + exchange(l_run);   // a failed wait has set the abort flag: the host reports it
            const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            float* out = a.dst + (((int64_t)b * a.Tq + iq) * a.H + h) * HD + ch * 64;
#pragma unroll
            for (int q4 = 0; q4 < 2; q4++) {
                uint32_t oreg[32];
                tmem_ld32(tmem_O + lane_base + ch * 64 + q4 * 32, oreg);
                tmem_wait_ld();
                if (iq < tq_b) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(out + q4 * 32 + i) =
                            make_float4(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv,
                                        __uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv);
                } else if (iq < a.Tq) {   // padding row of a batched launch: literal zeros
#pragma unroll
                    for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(out + q4 * 32 + i) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}


// ---- host side ----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// K/V as a rank-4 F16 tensor [hd, Lk, Hkv, Bk] with the caller's byte strides; box = 64 x 128 x 1 x 1.
bool encode_kv_map(CUtensorMap* m, const View& v, int hd, int Lk, int Hkv, int Bk) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)Lk, (cuuint64_t)Hkv, (cuuint64_t)Bk};
    const cuuint64_t strides[3] = {(cuuint64_t)v.nb1, (cuuint64_t)v.nb2, (cuuint64_t)v.nb3};
    const cuuint32_t box[4] = {64, (cuuint32_t)kTile, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<uint8_t*>(v.p), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Q as a rank-4 F16 or F32 tensor [hd, H, Tq, B] (head stride nb2, token stride nb1); box = 128 bytes of columns x the gqa
// heads of a group x 128 / gqa tokens: the rows of a box are the packed rows of a query tile.
bool encode_q_map(CUtensorMap* m, const FattnArgs& a) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)a.hd, (cuuint64_t)a.H, (cuuint64_t)a.Tq, (cuuint64_t)a.B};
    const cuuint64_t strides[3] = {(cuuint64_t)a.q.nb2, (cuuint64_t)a.q.nb1, (cuuint64_t)a.q.nb3};
    const bool f32 = a.q.type == B200_TYPE_F32;   // 128-byte box rows either way: 64 halves or 32 floats
    const cuuint32_t box[4] = {f32 ? 32u : 64u, (cuuint32_t)a.gqa, (cuuint32_t)(kTile / a.gqa), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<uint8_t*>(a.q.p), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// dst as a rank-4 F32 tensor [hd, H, Tq, B] (contiguous); box = 32 columns x gqa heads x 32 / gqa tokens: a warp's
// 32 packed rows.
bool encode_o_map(CUtensorMap* m, const FattnArgs& a) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)a.hd, (cuuint64_t)a.H, (cuuint64_t)a.Tq, (cuuint64_t)a.B};
    const cuuint64_t strides[3] = {(cuuint64_t)a.hd * 4, (cuuint64_t)a.hd * 4 * a.H, (cuuint64_t)a.hd * 4 * a.H * a.Tq};
    const cuuint32_t box[4] = {32, (cuuint32_t)a.gqa, (cuuint32_t)(32 / a.gqa), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.dst, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// R as a rank-4 F16 tensor [hd, 2T-1, H, 1|B]; box = 64 columns x 128 rows.
bool encode_r_map(CUtensorMap* m, const FattnArgs& a) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const int64_t nb3 = a.r_ne3 > 1 ? a.r.nb3 : a.r.nb2 * a.H;
    const cuuint64_t dims[4] = {(cuuint64_t)a.hd, (cuuint64_t)(2 * a.Tq - 1), (cuuint64_t)a.H, (cuuint64_t)a.r_ne3};
    const cuuint64_t strides[3] = {(cuuint64_t)a.r.nb1, (cuuint64_t)a.r.nb2, (cuuint64_t)nb3};
    const cuuint32_t box[4] = {64, (cuuint32_t)kTile, 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<uint8_t*>(a.r.p), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_relpos(const FattnArgs& a, cudaStream_t st, char* errbuf, size_t errlen) {
    CUtensorMap tmK, tmV, tmR;
    if (!encode_kv_map(&tmK, a.k, a.hd, a.Lk, a.Hkv, a.B / a.bq) || !encode_kv_map(&tmV, a.v, a.hd, a.Lk, a.Hkv, a.B / a.bq) ||
        !encode_r_map(&tmR, a)) {
        snprintf(errbuf, errlen, "cuTensorMapEncodeTiled failed for K/V/R");
        return B200_E_CUDA;
    }
    const size_t smem = 1024 + (size_t)6 * 2 * kPanelBytes + (size_t)2 * kTile * kBncStride + 136 + 8 + 2 * 128 * sizeof(float) + 16;
    cudaError_t e;
    dim3 grid((a.Tq + kTile - 1) / kTile, a.H, a.B);
    if (a.has_mask) {
        auto kern = fattn_prefill_tc5_relpos_kernel<true>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem, smem_set);
        if (e == cudaSuccess) {
            kern<<<grid, kThreadsRelpos, smem, st>>>(a, tmK, tmV, tmR);
            e = cudaGetLastError();
        }
    } else {
        auto kern = fattn_prefill_tc5_relpos_kernel<false>;
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, smem, smem_set);
        if (e == cudaSuccess) {
            kern<<<grid, kThreadsRelpos, smem, st>>>(a, tmK, tmV, tmR);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        snprintf(errbuf, errlen, "tcgen05 rel-pos prefill launch: %s", cudaGetErrorString(e));
        return B200_E_CUDA;
    }
    return B200_OK;
}

// Launch that may begin while the previous kernel of the stream drains, if that kernel allows it
// (griddepcontrol.launch_dependents: the K/V conversion pre-pass does).  The kernels wait for the predecessor's
// completion (griddepcontrol.wait) before they read anything it may have written.
template <typename Kern, typename... Args>
cudaError_t launch_pdl(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

#include "fattn_tc5_pair.cuh"
#include "fattn_tc5_split.cuh"

// B200_PREFILL_SPLIT=1 selects the split-row kernel (eight softmax warps, scores released at once) for head_dim 64
// without explicit mask.
bool split_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200_PREFILL_SPLIT");
        return e && e[0] == '1';
    }();
    return on;
}

bool split_supported(const FattnArgs& a) { return split_enabled() && a.hd == 64 && !a.has_mask && !a.relpos; }

int launch_split(const FattnArgs& a, cudaStream_t st, char* errbuf, size_t errlen) {
    CUtensorMap tmK, tmV;
    if (!encode_kv_map(&tmK, a.k, a.hd, a.Lk, a.Hkv, a.B / a.bq) || !encode_kv_map(&tmV, a.v, a.hd, a.Lk, a.Hkv, a.B / a.bq)) {
        snprintf(errbuf, errlen, "cuTensorMapEncodeTiled failed for K/V");
        return B200_E_CUDA;
    }
    const size_t smem = 1024 + (size_t)5 * kPanelBytes + 64 + 72 + 8 + 2048 + 16;
    dim3 grid((a.Tq * a.gqa + kTile - 1) / kTile, a.Hkv, a.B);
    auto kern = fattn_prefill_tc5_split_kernel;
    static bool smem_set[64] = {false};
    cudaError_t e = set_smem_once(kern, smem, smem_set);
    if (e == cudaSuccess) e = launch_pdl(kern, grid, kThreadsSplit, smem, st, a, tmK, tmV);
    if (e != cudaSuccess) {
        snprintf(errbuf, errlen, "tcgen05 split-row prefill launch: %s", cudaGetErrorString(e));
        return B200_E_CUDA;
    }
    return B200_OK;
}

// The paired-tile persistent kernel takes head_dim 64 without explicit mask and without causal bound.
// B200_PREFILL_PAIR=1 selects it (the one-tile kernel is the default); B200_PREFILL_POLY=n (2..16) moves every n-th pair of
// exponentials of the paired kernel to the FMA pipe (0 = none).
int pair_mode() {
    static const int mode = [] {
        const char* e = getenv("B200_PREFILL_PAIR");
        if (!(e && e[0] == '1')) return -1;   // opt-in while it measures slower than the one-tile kernel
        const char* p = getenv("B200_PREFILL_POLY");
        const int n = p ? atoi(p) : 0;
        return (n == 2 || n == 3 || n == 4 || n == 8) ? n : 0;
    }();
    return mode;
}

bool pair_supported(const FattnArgs& a) {
    return pair_mode() >= 0 && a.hd == 64 && !a.has_mask && !a.causal && !a.relpos;
}

int launch_pair(const FattnArgs& a, cudaStream_t st, char* errbuf, size_t errlen) {
    CUtensorMap tmK, tmV;
    if (!encode_kv_map(&tmK, a.k, a.hd, a.Lk, a.Hkv, a.B / a.bq) || !encode_kv_map(&tmV, a.v, a.hd, a.Lk, a.Hkv, a.B / a.bq)) {
        snprintf(errbuf, errlen, "cuTensorMapEncodeTiled failed for K/V");
        return B200_E_CUDA;
    }
    const int n_pairs = (a.Tq * a.gqa + 2 * kTile - 1) / (2 * kTile);
    const int64_t n_items64 = (int64_t)n_pairs * a.Hkv * a.B;
    if (n_items64 > INT32_MAX) return B200_E_LIMIT;
    const int n_items = (int)n_items64;
    static const int chunk_env = [] {   // B200_PAIR_CHUNK=n: items per CTA (default 4)
        const char* e = getenv("B200_PAIR_CHUNK");
        const int n = e ? atoi(e) : 0;
        return n >= 1 && n <= 1024 ? n : 4;
    }();
    const int chunk = chunk_env;
    static const int stagger = [] {   // B200_PAIR_STAGGER=clocks: delay of slot 1's first tile (default 1200)
        const char* e = getenv("B200_PAIR_STAGGER");
        const int n = e ? atoi(e) : -1;
        return n >= 0 && n <= 100000 ? n : 1200;
    }();
    dim3 grid((n_items + chunk - 1) / chunk);
    cudaError_t e;
    auto go = [&](auto kern) {
        static bool smem_set[64] = {false};
        e = set_smem_once(kern, kPairSmem, smem_set);
        if (e == cudaSuccess) e = launch_pdl(kern, grid, kPairThreads, kPairSmem, st, a, tmK, tmV, n_pairs, n_items, chunk, stagger);
    };
    switch (pair_mode()) {
        case 2: go(fattn_prefill_tc5_pair_kernel<2>); break;
        case 3: go(fattn_prefill_tc5_pair_kernel<3>); break;
        case 4: go(fattn_prefill_tc5_pair_kernel<4>); break;
        case 8: go(fattn_prefill_tc5_pair_kernel<8>); break;
        default: go(fattn_prefill_tc5_pair_kernel<0>); break;
    }
    if (e != cudaSuccess) {
        snprintf(errbuf, errlen, "tcgen05 paired prefill launch: %s", cudaGetErrorString(e));
        return B200_E_CUDA;
    }
    return B200_OK;
}

// B200_PREFILL_EARLY=1 or 2 selects an early-score order in the one-tile head_dim 64 kernel (A/B runs; off by default).
int early_scores_mode() {
    static const int mode = [] {
        const char* e = getenv("B200_PREFILL_EARLY");   // 0 (default), 1 or 2: see the kernel's EARLY parameter
        const int v = e ? atoi(e) : 0;
        return (v == 1 || v == 2) ? v : 0;
    }();
    return mode;
}

// One instantiation per kernel: its own "shared-memory attribute raised" flags per device.
template <auto Kern, typename... Args>
cudaError_t launch_inst(dim3 grid, size_t smem, cudaStream_t st, Args... args) {
    static bool smem_set[64] = {false};
    cudaError_t e = set_smem_once(Kern, smem, smem_set);
    if (e == cudaSuccess) e = launch_pdl(Kern, grid, kThreadsTc5, smem, st, args...);
    return e;
}

template <int HD, int NSTG>
int launch_t(const FattnArgs& a_in, cudaStream_t st, char* errbuf, size_t errlen) {
    const FattnArgs& a = a_in;
    CUtensorMap tmK, tmV;
    if (!encode_kv_map(&tmK, a.k, a.hd, a.Lk, a.Hkv, a.B / a.bq) || !encode_kv_map(&tmV, a.v, a.hd, a.Lk, a.Hkv, a.B / a.bq)) {
        snprintf(errbuf, errlen, "cuTensorMapEncodeTiled failed for K/V");
        return B200_E_CUDA;
    }
    constexpr int TILE_BYTES = kPanelBytes * (HD / 64);
    const size_t smem = 1024 + (size_t)(1 + 2 * NSTG) * TILE_BYTES + 32 * NSTG + 64 + 8;
    // F16 query rows, 16-byte aligned: the Q tile is one tensor copy (B200_PREFILL_QTMA=0: through registers)
    static const bool q_tma_on = [] {
        const char* e = getenv("B200_PREFILL_QTMA");
        return !(e && e[0] == '0');
    }();
    constexpr bool RAW_INST = HD == 128 && NSTG == 1;   // the raw F32 form exists (and pays) at head_dim 128 only
    CUtensorMap tmQ = tmK;
    int q_tma = 0;
    const bool gqa_box = a.gqa >= 1 && a.gqa <= 32 && 32 % a.gqa == 0;   // a warp's 32 packed rows are whole tokens
    const bool early = HD == 64 && !a.has_mask && early_scores_mode() != 0;   // the A/B variants move their tiles through the threads
    if (q_tma_on && !early && a.q.type == B200_TYPE_F16 && a.q.vec16 && gqa_box && !a.bias_u &&
        a.q.nb1 % 16 == 0 && a.q.nb2 % 16 == 0 && a.q.nb3 % 16 == 0 && a.q.nb1 > 0 && a.q.nb2 > 0 && a.q.nb3 > 0)
        q_tma = encode_q_map(&tmQ, a) ? 1 : 0;
    else if (q_tma_on && RAW_INST && a.q.type == B200_TYPE_F32 && a.q.vec16 && gqa_box && !a.bias_u &&
             early_scores_mode() == 0 && a.q.nb1 % 16 == 0 && a.q.nb2 % 16 == 0 && a.q.nb3 % 16 == 0 && a.q.nb1 > 0 && a.q.nb2 > 0 &&
             a.q.nb3 > 0)
        q_tma = encode_q_map(&tmQ, a) ? 2 : 0;   // F32 rows: raw tile into stages not needed yet, converted from shared memory
    // a warp's rows of the output are a box of dst, written by tensor stores (B200_PREFILL_OTMA=0: by the threads)
    static const bool o_tma_on = [] {
        const char* e = getenv("B200_PREFILL_OTMA");
        return !(e && e[0] == '0');
    }();
    CUtensorMap tmO = tmK;
    int o_tma = 0;
    if (o_tma_on && !early && gqa_box && (uintptr_t)a.dst % 16 == 0) o_tma = encode_o_map(&tmO, a) ? 1 : 0;
    cudaError_t e;
    dim3 grid((a.Tq * a.gqa + kTile - 1) / kTile, a.Hkv, a.B);   // packed (query, group head) rows per KV head
    // launch_inst is instantiated per kernel (the kernels share one function-pointer type, so a generic lambda would
    // share its "attribute set" flags between them)
    auto args = [&](auto launch) { e = launch(grid, smem, st, a, tmK, tmV, tmQ, tmO); };
    constexpr int QRAW = RAW_INST ? 2 : 0;
#define B200_GO(...) args(launch_inst<fattn_prefill_tc5_kernel<__VA_ARGS__>, FattnArgs, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap>)
    if (HD == 64 && !a.has_mask && early_scores_mode() == 2) {
        B200_GO(HD, NSTG, false, HD == 64 ? 2 : 0);
    } else if (HD == 64 && !a.has_mask && early_scores_mode() == 1) {
        B200_GO(HD, NSTG, false, HD == 64 ? 1 : 0);
    } else if (a.has_mask) {
        if (q_tma == 2) { if (o_tma) B200_GO(HD, NSTG, true, 0, QRAW, true); else B200_GO(HD, NSTG, true, 0, QRAW, false); }
        else if (q_tma == 1) { if (o_tma) B200_GO(HD, NSTG, true, 0, 1, true); else B200_GO(HD, NSTG, true, 0, 1, false); }
        else { if (o_tma) B200_GO(HD, NSTG, true, 0, 0, true); else B200_GO(HD, NSTG, true, 0, 0, false); }
    } else {
        if (q_tma == 2) { if (o_tma) B200_GO(HD, NSTG, false, 0, QRAW, true); else B200_GO(HD, NSTG, false, 0, QRAW, false); }
        else if (q_tma == 1) { if (o_tma) B200_GO(HD, NSTG, false, 0, 1, true); else B200_GO(HD, NSTG, false, 0, 1, false); }
        else { if (o_tma) B200_GO(HD, NSTG, false, 0, 0, true); else B200_GO(HD, NSTG, false, 0, 0, false); }
    }
#undef B200_GO
    if (e != cudaSuccess) {
        snprintf(errbuf, errlen, "tcgen05 prefill launch: %s", cudaGetErrorString(e));
        return B200_E_CUDA;
    }
    return B200_OK;
}

}  // namespace

bool tc5_supported(const FattnArgs& a) {
    if (a.hd != 64 && a.hd != 128) return false;
    if (a.k.type != B200_TYPE_F16 || a.v.type != B200_TYPE_F16) return false;
    if (!a.k.vec16 || !a.v.vec16) return false;
    if (a.softcap != 0.0f || a.n2 != 0) return false;
    if (!(a.scale > 0.0f)) return false;
    // explicit masks: any 2-byte aligned layout (rows that are not 16-byte aligned are read with 2-byte loads)
    if (a.relpos) {
        // fused bias: head_dim 128, F16 R with TMA-legal strides, no causal mask, bias rounded to F16
        if (a.hd != 128 || a.causal || a.relpos_f32) return false;
        if (a.r.type != B200_TYPE_F16 || !a.r.vec16 || a.r.nb1 <= 0 || a.r.nb2 <= 0) return false;
    }
    const int64_t lim = (int64_t)1 << 40;
    if (a.k.nb1 <= 0 || a.k.nb2 <= 0 || a.k.nb3 <= 0 || a.v.nb1 <= 0 || a.v.nb2 <= 0 || a.v.nb3 <= 0) return false;
    if (a.k.nb1 >= lim || a.k.nb2 >= lim || a.k.nb3 >= lim || a.v.nb1 >= lim || a.v.nb2 >= lim || a.v.nb3 >= lim) return false;
    return true;
}

int launch_prefill_tc5(const FattnArgs& a, cudaStream_t st, char* errbuf, size_t errlen) {
    if (a.relpos) return launch_relpos(a, st, errbuf, errlen);
    if (pair_supported(a)) return launch_pair(a, st, errbuf, errlen);
    if (split_supported(a)) return launch_split(a, st, errbuf, errlen);
    if (a.hd == 64) return launch_t<64, 2>(a, st, errbuf, errlen);
    return launch_t<128, 1>(a, st, errbuf, errlen);
}

#ifdef B200_TC5_TRACE
extern "C" __attribute__((visibility("default"))) int b200_dbg_trace(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_tc5_trace, sizeof(long long) * 3 * 64 * 8);
}
#endif

int tc5_read_status(int* status) {
    int v = 0;
    const cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc5_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    *status = v;
    return 0;
}

int tc5_reset_status() {
    const int zero = 0;
    return (int)cudaMemcpyToSymbol(g_tc5_status, &zero, sizeof(int));
}

}  // namespace b200
