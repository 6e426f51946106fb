// Split-row tcgen05 prefill kernel, head_dim 64, no explicit mask.  Included by fattn_tc5.cu (uses its PTX wrappers).
//
// Same tile as the one-tile kernel (128 query rows x 128 keys per step, two CTAs per SM, S 128 + O 64 + P 64 TMEM
// columns), but EIGHT softmax warps: warps w and w+4 see the same 32 TMEM lanes and thread (r, ch) owns columns
// [64ch, 64ch+64) of row r.  What that buys at head_dim 64, where 16384 exponentials per tile (1024 clk of the
// SM's exponential unit) outweigh 512 clk of MMA:
//   * a thread's half row is 64 registers, so the WHOLE score tile sits in registers right after one TMEM load and the
//     score columns are handed back at once (s_read): the tensor pipe computes S[j+1] under the exponentials of tile
//     j, and no softmax warp ever waits for the MMA thread between two tiles;
//   * the row maximum is known (one pass over the registers, one exchange with the partner thread through shared
//     memory) before the first exponential, so there is no "redo the tile" path;
//   * four softmax warps per scheduler (two per CTA) instead of two keep the exponential unit fed while others sit
//     in a TMEM load, the exchange or a store.
// Everything else (TMA ring, P in its own columns, lazy rescale of O, zero rows for padding, GQA packing, causal
// order) is the one-tile kernel's.
#pragma once

constexpr int kThreadsSplit = 320;   // 8 softmax warps, TMA warp, MMA warp

__global__ void __launch_bounds__(kThreadsSplit, 2)
fattn_prefill_tc5_split_kernel(const FattnArgs a, const __grid_constant__ CUtensorMap tmK,
                               const __grid_constant__ CUtensorMap tmV) {
    constexpr int HD = 64, NSTG = 2;
    constexpr int TILE_BYTES = kPanelBytes;
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
                   bar_pair = bar_s_full + 40;   // [4]
    uint8_t* misc = smem_gen + (1 + 2 * NSTG) * TILE_BYTES + 32 * NSTG + 72;
    volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(misc);
    volatile int* s_abort = reinterpret_cast<volatile int*>(misc + 4);
    volatile float* s_xchg = reinterpret_cast<volatile float*>(misc + 8);   // [2 tile parities][2 halves][128 rows]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    int q0 = blockIdx.x * kTile, hk = blockIdx.y, b = blockIdx.z;
    if (a.causal) {   // longest query tiles first over the whole grid
        const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z), hb = gridDim.y * gridDim.z;
        q0 = (gridDim.x - 1 - lin / hb) * kTile;
        hk = (lin % hb) % gridDim.y, b = (lin % hb) / gridDim.y;
    }
    const int bk = b / a.bq;
    const int rows_total = a.Tq * a.gqa;
    const int tq_b = q_rows_of(a, b);
    const int rows_live = tq_b * a.gqa;
    int len_b = a.Lk;
    if (a.kv_len) {
        const int v = a.kv_len[b];
        len_b = v < 0 ? 0 : (v > a.Lk ? a.Lk : v);
    }
    const int n_past = n_past_of(a, len_b, tq_b);
    int kmax = q0 < rows_live ? len_b : 0;
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
    if (tid == 8 * 32) {
        for (int i = 0; i < NSTG; i++) {
            mbar_init(bar_k_full + 8 * i, 1);
            mbar_init(bar_k_empty + 8 * i, 1);
            mbar_init(bar_v_full + 8 * i, 1);
            mbar_init(bar_v_empty + 8 * i, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_p_ready, 8);   // one arrival per softmax warp
        mbar_init(bar_o_done, 1);
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_s_read, 8);
        for (int i = 0; i < 4; i++) mbar_init(bar_pair + 8 * i, 2);   // the two warps that share 32 TMEM lanes
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
        for (int j = 0; j < NSTG && j < n_tiles; j++) {
            mbar_arrive_expect_tx(bar_k_full + 8 * j, TILE_BYTES);
            tma_load_4d(sK + j * TILE_BYTES, &tmK, bar_k_full + 8 * j, 0, j * kTile, hk, bk);
            mbar_arrive_expect_tx(bar_v_full + 8 * j, TILE_BYTES);
            tma_load_4d(sV + j * TILE_BYTES, &tmV, bar_v_full + 8 * j, 0, j * kTile, hk, bk);
        }
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(s_tmem_base))),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp < 8) {
        // Q tile -> shared memory: thread (r, ch) converts 16-byte chunks 4ch .. 4ch+3 of row r
        const int r = tid & 127, ch = tid >> 7;
        const int iq = (q0 + r) / a.gqa, h = hk * a.gqa + (q0 + r) % a.gqa;
        const uint8_t* rowp = a.q.p + (int64_t)iq * a.q.nb1 + (int64_t)h * a.q.nb2 + (int64_t)b * a.q.nb3;
        uint4 v[4];
        if (q0 + r >= rows_total) {
#pragma unroll
            for (int c = 0; c < 4; c++) v[c] = make_uint4(0u, 0u, 0u, 0u);
        } else if (a.q.type == B200_TYPE_F32 && a.q.vec16) {
            float4 f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __ldg(reinterpret_cast<const float4*>(rowp) + ch * 8 + i);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v[i].x = pack_half2(f[2 * i].x, f[2 * i].y), v[i].y = pack_half2(f[2 * i].z, f[2 * i].w);
                v[i].z = pack_half2(f[2 * i + 1].x, f[2 * i + 1].y), v[i].w = pack_half2(f[2 * i + 1].z, f[2 * i + 1].w);
            }
        } else if (a.q.type == B200_TYPE_F16 && a.q.vec16) {
#pragma unroll
            for (int c = 0; c < 4; c++) v[c] = __ldg(reinterpret_cast<const uint4*>(rowp) + ch * 4 + c);
        } else {
#pragma unroll
            for (int c = 0; c < 4; c++) v[c] = q_chunk(rowp, a.q.type, (ch * 4 + c) * 8, false);
        }
        uint8_t* dst_row = smem_gen + r * 128;
#pragma unroll
        for (int c = 0; c < 4; c++) *reinterpret_cast<uint4*>(dst_row + ((((ch * 4 + c) & 7) ^ (r & 7)) << 4)) = v[c];
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;
    const uint32_t tmem_S = tmem_base;                  // cols [0,128)
    const uint32_t tmem_O = tmem_base + kTile;          // cols [128,192)
    const uint32_t tmem_P = tmem_base + kTile + HD;     // f16x2: cols [192,256)

    if (warp == 8) {
        // ================= TMA producer =================
        if (lane == 0) {
            bool ok = true;
            int issued_k = min(NSTG, n_tiles), issued_v = min(NSTG, n_tiles);
            for (int j = NSTG; j < n_tiles; j++) {
                const int slot = j % NSTG, use = j / NSTG;
                const int k0 = j * kTile;
                ok = mbar_wait(bar_k_empty + 8 * slot, (use - 1) & 1, s_abort);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_k_full + 8 * slot, TILE_BYTES);
                tma_load_4d(sK + slot * TILE_BYTES, &tmK, bar_k_full + 8 * slot, 0, k0, hk, bk);
                issued_k = j + 1;
                ok = mbar_wait(bar_v_empty + 8 * slot, (use - 1) & 1, s_abort);
                if (!ok) break;
                mbar_arrive_expect_tx(bar_v_full + 8 * slot, TILE_BYTES);
                tma_load_4d(sV + slot * TILE_BYTES, &tmV, bar_v_full + 8 * slot, 0, k0, hk, bk);
                issued_v = j + 1;
            }
            if (!ok) {   // drain: wait (bounded) for the copies this thread still has in flight
                for (int j = max(0, issued_k - NSTG); j < issued_k; j++)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_k_full + 8 * (j % NSTG), (j / NSTG) & 1); ++it) __nanosleep(256);
                for (int j = max(0, issued_v - NSTG); j < issued_v; j++)
                    for (uint32_t it = 0; it < 4096 && !mbar_try_wait(bar_v_full + 8 * (j % NSTG), (j / NSTG) & 1); ++it) __nanosleep(256);
            }
        }
    } else if (warp == 9) {
        // ================= MMA issuer =================
        // S[0]; then per tile j: S[j+1] as soon as every softmax warp holds S[j] in registers (s_read), P.V[j] when
        // P[j] is stored.  The tensor pipe executes in issue order.
        if (lane == 0) {
            const uint32_t q_lo = smem_desc_lo(sQ, 16), k_lo = smem_desc_lo(sK, 16), v_lo = smem_desc_lo(sV, kPanelBytes);
            constexpr uint32_t desc_hi = smem_desc_hi(1024);
            auto issue_s = [&](int slot) {
                const uint32_t kd = k_lo + slot * (TILE_BYTES >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++)
                    mma_ss(tmem_S, desc64(q_lo + ks * 2, desc_hi), desc64(kd + ks * 2, desc_hi), IDESC_S, ks > 0 ? 1u : 0u);
                tc_commit(bar_s_full);
                tc_commit(bar_k_empty + 8 * slot);
            };
            bool ok = mbar_wait(bar_k_full, 0, s_abort);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                const int slot = j % NSTG, use = j / NSTG;
                const int nslot = (j + 1) % NSTG, nuse = (j + 1) / NSTG;
                const bool more = j + 1 < n_tiles;
                if (more) ok = mbar_wait(bar_k_full + 8 * nslot, nuse & 1, s_abort);
                if (ok) ok = mbar_wait(bar_s_read, j & 1, s_abort);
                if (!ok) break;
                if (more) {
                    tc_fence_after();
                    issue_s(nslot);
                }
                ok = mbar_wait(bar_v_full + 8 * slot, use & 1, s_abort);
                if (ok) ok = mbar_wait(bar_p_ready, j & 1, s_abort);
                if (!ok) break;
                tc_fence_after();
                const uint32_t vd = v_lo + slot * (TILE_BYTES >> 4);
                mma_ts(tmem_O, tmem_P, desc64(vd, desc_hi), IDESC_PV, j > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < kTile / 16; ks++) mma_ts(tmem_O, tmem_P + ks * 8, desc64(vd + ks * (2048 >> 4), desc_hi), IDESC_PV, 1u);
                tc_commit(bar_v_empty + 8 * slot);
                tc_commit(bar_pv_done);
                if (!more) tc_commit(bar_o_done);
            }
            if (!ok) {   // make sure no MMA of this CTA is still running before TMEM is released
                tc_commit(bar_o_done);
                for (uint32_t it = 0; it < 65536 && !mbar_try_wait(bar_o_done, 0); ++it) __nanosleep(256);
            }
        }
    } else {
        // ================= softmax / correction / epilogue =================
        const int r = tid & 127, ch = tid >> 7;
        const bool row_live = q0 + r < rows_live;
        const bool row_zero = !row_live && q0 + r < rows_total;
        const int iq_dst = (q0 + r) / a.gqa;
        const int iq = row_live ? iq_dst : a.Tq, h = hk * a.gqa + (q0 + r) % a.gqa;   // dead rows: iq = Tq
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t my_pair_bar = bar_pair + 8 * (warp & 3);
        uint32_t pair_phase = 0;
        const float c = a.scale * kLog2e;
        const uint64_t c2 = pack2(c, c);
        int kend = len_b;
        if (a.causal) kend = min(kend, n_past + iq + 1);
        float m_ref = -INFINITY, l_run = 0.0f;
        bool ok = true;
        // Publish a value, meet the partner warp (bounded wait), read the partner's value.  The slots alternate with
        // `slot`: a thread's next write to the same slot lies two meetings ahead, after the partner has read this one.
        auto exchange = [&](float mine, int slot) {
            s_xchg[(slot & 1) * 256 + ch * 128 + r] = mine;
            __syncwarp();
            if (lane == 0) mbar_arrive(my_pair_bar);
            ok = mbar_wait(my_pair_bar, pair_phase, s_abort);
            pair_phase ^= 1;
            return s_xchg[(slot & 1) * 256 + (ch ^ 1) * 128 + r];
        };
        for (int j = 0; j < n_tiles; j++) {
            ok = mbar_wait(bar_s_full, j & 1, s_abort);
            if (!ok) break;
            if (tid == 0) TC5_TRACE(0, j, 0);
            tc_fence_after();
            uint32_t sreg[2][32];
            tmem_ld32(tmem_S + lane_base + ch * 64, sreg[0]);
            tmem_ld32(tmem_S + lane_base + ch * 64 + 32, sreg[1]);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s_read);   // this warp's part of the tile is in registers
            if (tid == 0) TC5_TRACE(0, j, 3);
            const int n_valid = kend - j * kTile - ch * 64;   // this thread's columns >= n_valid are masked
            if (!__all_sync(0xffffffffu, n_valid >= 64)) {
#pragma unroll
                for (int i = 0; i < 64; i++)
                    if (i >= n_valid) sreg[i >> 5][i & 31] = 0xFF800000u;   // -inf
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 64; i += 2)
                mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(sreg[i >> 5][i & 31]), __uint_as_float(sreg[i >> 5][(i + 1) & 31]));
            const float mx_half = max3(fmaxf(mx[0], mx[1]), mx[2], mx[3]) * c;
            const float m_tile = fmaxf(mx_half, exchange(mx_half, j));
            if (!ok) break;
            if (tid == 0) TC5_TRACE(0, j, 4);
            bool pv_waited = false;
            // lazy rescale: O and l are only touched when a row outgrew its reference maximum by 2^8; the two warps of
            // a pair see the same row maxima and take the same branch
            if (__any_sync(0xffffffffu, m_tile > m_ref + kRescaleThreshold)) {
                if (j > 0) {   // O must be at rest: P.V of the previous tile has completed
                    ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                    if (!ok) break;
                    tc_fence_after();
                    pv_waited = true;
                }
                const float m_new = fmaxf(m_ref, m_tile);
                const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_ref - m_new);
                l_run *= alpha;
                if (j > 0) {   // eight columns at a time: the score row stays in registers meanwhile
#pragma unroll 1
                    for (int q8 = 0; q8 < 4; q8++) {
                        uint32_t o[8];
                        const uint32_t addr = tmem_O + lane_base + ch * 32 + q8 * 8;
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                     : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                                     : "r"(addr)
                                     : "memory");
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(addr), "r"(o[0]),
                                     "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                                     : "memory");
                    }
                }
                m_ref = m_new;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
            const uint64_t nm2 = pack2(-m_use, -m_use);
            uint64_t ls[2] = {0ull, 0ull};
            uint32_t preg[32];
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                float t0, t1;
                unpack2(fma2(pack2(__uint_as_float(sreg[i >> 5][i & 31]), __uint_as_float(sreg[i >> 5][(i + 1) & 31])), c2, nm2), t0, t1);
                const float p0 = ex2(t0), p1 = ex2(t1);   // -inf -> 0
                ls[(i >> 1) & 1] = add2(ls[(i >> 1) & 1], pack2(p0, p1));
                preg[i >> 1] = cvt_f16x2(p0, p1);
            }
            {
                float l0, l1;
                unpack2(add2(ls[0], ls[1]), l0, l1);
                l_run += l0 + l1;
            }
            if (j > 0 && !pv_waited) {  // P[j-1] must have been consumed before P[j] overwrites it
                ok = mbar_wait(bar_pv_done, (j - 1) & 1, s_abort);
                if (!ok) break;
                tc_fence_after();
            }
            if (tid == 0) TC5_TRACE(0, j, 1);
            tmem_st32(tmem_P + lane_base + ch * 32, preg);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_ready);
            if (tid == 0) TC5_TRACE(0, j, 2);
        }
        if (ok) ok = mbar_wait(bar_o_done, 0, s_abort);
        if (ok) {
            tc_fence_after();
            const float l_tot = l_run + exchange(l_run, n_tiles);   // a failed wait has set the abort flag: the host reports it
            const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            float* out = a.dst + (((int64_t)b * a.Tq + iq_dst) * a.H + h) * HD + ch * 32;
            uint32_t oreg[32];
            tmem_ld32(tmem_O + lane_base + ch * 32, oreg);
            tmem_wait_ld();
            if (row_live) {
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(out + i) = make_float4(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv,
                                                                      __uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv);
            } else if (row_zero) {   // literal zeros: whatever the padding row of Q held never reaches dst
#pragma unroll
                for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(out + i) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}
