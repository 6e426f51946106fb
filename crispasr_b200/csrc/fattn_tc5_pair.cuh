// fattn_tc5_pair.cuh — persistent paired-tile prefill kernel for head_dim 64 (included by fattn_tc5.cu inside its
// anonymous namespace, after the PTX wrappers).
//
// At head_dim 64 a 128x128 score tile costs 512 clocks of tensor pipe but 1024 clocks of the exponential unit, so the
// kernel lives or dies by how busy the softmax warps keep that unit.  The one-tile kernel above puts two independent
// CTAs on an SM; a trace of it shows each softmax warp spending a quarter of every tile on things that are not
// exponentials (tensor-memory round trips that are not overlapped, the wait for the next score tile) and every CTA
// paying a prologue (Q conversion, first K/V copies) and an epilogue that the other CTA only partly covers.  This
// kernel is the fusion of those two CTAs into ONE persistent CTA per SM:
//
//   * an item is a PAIR of 128-row query tiles of one (KV head, batch entry); the two tiles ("slots") share every K/V
//     tile in shared memory, so K/V travel from L2 once per 256 query rows;
//   * 384 threads: warps 0-3 softmax of slot 0, warps 4-7 softmax of slot 1 (thread r of a slot owns query row r, all
//     128 score columns of a tile live in its registers), warp 8 TMA producer, warp 9 issues the score MMAs, warp 11
//     the P.V MMAs, warp 10 converts the NEXT item's Q tiles into the second Q buffer while the current item runs.  Register budgets are moved with
//     setmaxnreg: 200 per softmax thread, 96 for the rest;
//   * tensor memory, all 512 columns: S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384) P0 [384,448) P1 [448,512).
//     A softmax thread pulls its whole score row into registers at the start of a tile and says so (s_read); P has its
//     own columns; so the MMA thread issues S_t[j+1] right then, under the slot's exponentials of tile j, and the
//     softmax warps never wait for the tensor pipe between two tiles (the registers are the second score buffer);
//   * a CTA walks `chunk` consecutive items (the pairs of one head first, so its K/V stay in L2); K/V tiles stream through
//     one ring across item borders, the next item's first score tiles are computed while the softmax warps write the
//     previous item's output, and barriers, tensor memory and tensor maps are set up once per chunk instead of once per
//     128 rows; the grid is ceil(items / chunk) CTAs, one resident per SM, handed out by the hardware as SMs free up;
//   * the row maximum is taken from registers before the exponentials (same instruction count as tracking it in the
//     same pass), so a tile is never computed twice; O and l are rescaled lazily (only when a row outgrew its reference
//     maximum by 2^8);
//   * POLY > 0 sends every POLY-th pair of exponentials to a cubic on the FMA pipe instead of the exponential unit.
//
// Scope: head_dim 64, F16 K/V through TMA, no explicit mask, no causal bound; per-entry kv_len and q_len, GQA packing
// (rows of a tile are (query, head-of-group) pairs) as in the one-tile kernel, which keeps every other form.
// Every mbarrier wait is bounded; on expiry the CTA raises its abort flag, all roles leave their loops, tensor memory
// is released and the device status word is set.

#ifdef B200_TC5_TRACE
#define PAIR_TRACE(role, j, k) do { if (blockIdx.x == 1 && (j) < 64) g_tc5_trace[role][j][k] = clock64(); } while (0)
#else
#define PAIR_TRACE(role, j, k) do { } while (0)
#endif

constexpr int kPairThreads = 384;
constexpr int kPairStages = 3;                        // K and V ring depth (16 KB per tile)
constexpr int kPairTile = kPanelBytes;                // bytes of one 128 x 64 f16 tile
constexpr int kPairBars = 4 * kPairStages + 14;       // k/v full/empty, q_full/q_empty[2], s_full/p_ready/pv_done/o_done/s_read[2]
constexpr size_t kPairSmem = 1024 + (size_t)(4 + 2 * kPairStages) * kPairTile + 8 * kPairBars + 64;

struct PairItem {
    int q0, hk, b, bk, len_b, n_tiles, rows_total, rows_live;
    bool active, live1;
};

__device__ __forceinline__ PairItem pair_item(const FattnArgs& a, int item, int n_pairs) {
    PairItem it;
    const int pair = item % n_pairs, hb = item / n_pairs;
    it.hk = hb % a.Hkv, it.b = hb / a.Hkv, it.bk = it.b / a.bq;
    it.q0 = pair * 2 * kTile;
    it.rows_total = a.Tq * a.gqa;
    it.rows_live = q_rows_of(a, it.b) * a.gqa;
    it.len_b = a.Lk;
    if (a.kv_len) {
        const int v = a.kv_len[it.b];
        it.len_b = v < 0 ? 0 : (v > a.Lk ? a.Lk : v);
    }
    it.n_tiles = (it.len_b + kTile - 1) / kTile;
    it.active = it.n_tiles > 0 && it.q0 < it.rows_live;
    it.live1 = it.active && it.q0 + kTile < it.rows_live;
    return it;
}

// 2^x for a pair on the FMA pipe: x = n + f with n = round(x) (magic-number add), 2^f by a cubic on [-0.5, 0.5]
// (relative error 7.5e-5, below the F16 rounding of P), the exponent added to the bit pattern.  x is clamped to
// >= -126 so the exponent arithmetic cannot wrap; -inf (a masked column) must not come here.
__device__ __forceinline__ void exp2_poly_pair(float x0, float x1, float& p0, float& p1) {
    const float magic = 12582912.0f;   // 1.5 * 2^23: the low mantissa bits of x + magic hold round(x)
    x0 = fmaxf(x0, -126.0f), x1 = fmaxf(x1, -126.0f);
    const uint64_t x2 = pack2(x0, x1);
    const uint64_t r2 = add2(x2, pack2(magic, magic));
    const uint64_t n2 = add2(r2, pack2(-magic, -magic));
    const uint64_t f2 = fma2(n2, pack2(-1.0f, -1.0f), x2);
    // minimax cubic for 2^f on [-0.5, 0.5]: relative error 7.5e-5
    uint64_t q = fma2(pack2(0.05517167f, 0.05517167f), f2, pack2(0.24261113f, 0.24261113f));
    q = fma2(q, f2, pack2(0.69326097f, 0.69326097f));
    q = fma2(q, f2, pack2(0.99992806f, 0.99992806f));
    float q0, q1, r0, r1;
    unpack2(q, q0, q1);
    unpack2(r2, r0, r1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(r0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(r1) << 23));
}

template <int POLY>
__global__ void __launch_bounds__(kPairThreads, 1)
fattn_prefill_tc5_pair_kernel(const FattnArgs a, const __grid_constant__ CUtensorMap tmK,
                              const __grid_constant__ CUtensorMap tmV, const int n_pairs, const int n_items, const int chunk, const int stagger) {
    constexpr int HD = 64;
    constexpr uint32_t IDESC_S = idesc_f16(kTile, false);
    constexpr uint32_t IDESC_PV = idesc_f16(HD, true);
    constexpr int NS = kPairStages;

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
    const uint32_t sQ = smem_base;                         // [buffer 2][slot 2] tiles
    const uint32_t sK = sQ + 4 * kPairTile;
    const uint32_t sV = sK + NS * kPairTile;
    const uint32_t sBar = sV + NS * kPairTile;
    const uint32_t bar_k_full = sBar, bar_k_empty = sBar + 8 * NS, bar_v_full = sBar + 16 * NS, bar_v_empty = sBar + 24 * NS;
    const uint32_t bar_q_full = sBar + 32 * NS, bar_q_empty = bar_q_full + 16, bar_s_full = bar_q_full + 32,
                   bar_p_ready = bar_q_full + 48, bar_pv_done = bar_q_full + 64, bar_o_done = bar_q_full + 80,
                   bar_s_read = bar_q_full + 96;
    uint8_t* misc = smem_gen + (4 + 2 * NS) * kPairTile + 8 * kPairBars;
    volatile uint32_t* s_tmem_base = reinterpret_cast<volatile uint32_t*>(misc);
    volatile int* s_abort = reinterpret_cast<volatile int*>(misc + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // This CTA's items: `chunk` consecutive ones.  The grid is not persistent on purpose: SMs differ in speed by more than
    // a quarter on this part (a static split of the items over 148 resident CTAs finished between 1.64 and 2.08 ms), so
    // the hardware's CTA scheduler does the load balancing, at chunk granularity.
    const int item_lo = blockIdx.x * chunk, item_hi = min(n_items, item_lo + chunk);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // programmatic launch: the previous kernel of the stream has completed
#ifdef B200_TC5_TRACE
    if (tid == 0 && blockIdx.x < 192) {
        long long tnow;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tnow));
        (&g_tc5_trace[2][0][0])[blockIdx.x * 2] = tnow;
        if (blockIdx.x < 8) (&g_tc5_trace[1][40][0])[blockIdx.x * 2] = clock64();
    }
#endif

    // ---- set-up, once per SM ----
    if (tid == 8 * 32) {
        for (int i = 0; i < kPairBars; i++) {
            const uint32_t bar = sBar + 8 * i;
            uint32_t count = 1;
            // q_full: one arrival (the Q-loader warp)
            if (bar >= bar_p_ready && bar < bar_pv_done) count = 4;     // one arrival per softmax warp of the slot
            if (bar >= bar_s_read) count = 4;
            mbar_init(bar, count);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmK)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmV)) : "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(s_tmem_base))),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem_base;

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;" ::: "memory");
        if (warp == 10) {
            // ================= Q loader: the next item's two query tiles -> the free Q buffer =================
            const int lt = lane;   // eight rows each
            bool ok = true;
            int ka = 0;
            for (int item = item_lo; item < item_hi && ok; item++) {
                const PairItem it = pair_item(a, item, n_pairs);
                if (!it.active) continue;
                const int buf = ka & 1, use = ka >> 1;
                if (lane == 0) PAIR_TRACE(1, 16 + ka, 0);
                if (use > 0) ok = mbar_wait(bar_q_empty + 8 * buf, (use - 1) & 1, s_abort);
                if (!ok) break;
                if (lane == 0) PAIR_TRACE(1, 16 + ka, 1);
#pragma unroll 1
                for (int rr = 0; rr < 8; rr++) {
                    const int r = lt + 32 * rr, slot = r >> 7, row = r & 127;
                    const int pr = it.q0 + r;                       // packed (query, head-of-group) row
                    const int iq = pr / a.gqa, h = it.hk * a.gqa + pr % a.gqa;
                    load_q_row<HD>(smem_gen + (buf * 2 + slot) * kPairTile, row,
                                   a.q.p + (int64_t)iq * a.q.nb1 + (int64_t)h * a.q.nb2 + (int64_t)it.b * a.q.nb3, a.q.type,
                                   a.q.vec16 != 0, pr < it.rows_total);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_q_full + 8 * buf);
                if (lane == 0) PAIR_TRACE(1, 16 + ka, 2);
                ka++;
            }
        } else if (warp == 8) {
            // ================= TMA producer: one K/V ring across all items =================
            if (lane == 0) {
                bool ok = true;
                int g = 0;
                for (int item = item_lo; item < item_hi && ok; item++) {
                    const PairItem it = pair_item(a, item, n_pairs);
                    if (!it.active) continue;
                    for (int j = 0; j < it.n_tiles && ok; j++, g++) {
                        const int slot = g % NS, use = g / NS;
                        if (use > 0) ok = mbar_wait(bar_k_empty + 8 * slot, (use - 1) & 1, s_abort);
                        if (!ok) break;
                        mbar_arrive_expect_tx(bar_k_full + 8 * slot, kPairTile);
                        tma_load_4d(sK + slot * kPairTile, &tmK, bar_k_full + 8 * slot, 0, j * kTile, it.hk, it.bk);
                        if (use > 0) ok = mbar_wait(bar_v_empty + 8 * slot, (use - 1) & 1, s_abort);
                        if (!ok) break;
                        mbar_arrive_expect_tx(bar_v_full + 8 * slot, kPairTile);
                        tma_load_4d(sV + slot * kPairTile, &tmV, bar_v_full + 8 * slot, 0, j * kTile, it.hk, it.bk);
                    }
                }
                if (!ok) {   // drain: give copies in flight time to land before the CTA's shared memory goes away
                    for (uint32_t itn = 0; itn < 16384; ++itn) __nanosleep(64);
                }
            }
        } else if (warp == 9) {
            // ================= score issuer: S_t[j] = Q_t . K[j]^T =================
            // Two threads issue the tensor-core work, this one the score tiles and warp 11 the P.V products: one
            // thread doing both took 4 k clocks per pair of tiles (about 65 per MMA or commit, twice that per barrier
            // test) and was what the softmax warps waited for.
            if (lane == 0) {
                constexpr uint32_t desc_hi = smem_desc_hi(1024);
                const uint32_t tS[2] = {tmem_base, tmem_base + 128};
                bool ok = true;
                int g = 0, ka = 0;
                int cnt[2] = {0, 0};     // score tiles each slot has taken into registers so far (phase of s_read)
                bool any_mma = false;
                auto issue_s = [&](int t, uint32_t q_addr, int kslot) {
                    const uint32_t qd = smem_desc_lo(q_addr, 16), kd = smem_desc_lo(sK + kslot * kPairTile, 16);
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++)
                        mma_ss(tS[t], desc64(qd + ks * 2, desc_hi), desc64(kd + ks * 2, desc_hi), IDESC_S, ks > 0 ? 1u : 0u);
                    tc_commit(bar_s_full + 8 * t);
                };
                for (int item = item_lo; item < item_hi && ok; item++) {
                    const PairItem it = pair_item(a, item, n_pairs);
                    if (!it.active) continue;
                    const int buf = ka & 1, n = it.n_tiles;
                    const uint32_t q_addr[2] = {sQ + (buf * 2) * kPairTile, sQ + (buf * 2 + 1) * kPairTile};
                    ok = mbar_wait(bar_q_full + 8 * buf, (ka >> 1) & 1, s_abort);
                    for (int j = 0; j < n && ok; j++, g++) {
                        // tile j of the item: the slot's score columns are free once its four warps hold tile j-1 in
                        // registers (s_read), long before its P is ready - so the next score tile is computed under
                        // the slot's exponentials and a softmax warp never waits for the tensor pipe between tiles
                        const int slot = g % NS;
                        ok = mbar_wait(bar_k_full + 8 * slot, (g / NS) & 1, s_abort);
                        if (ka == 0) PAIR_TRACE(1, j, 0);
#pragma unroll
                        for (int t = 0; t < 2; t++) {
                            if (!ok || (t == 1 && !it.live1)) continue;
                            if (cnt[t] > 0) ok = mbar_wait(bar_s_read + 8 * t, (cnt[t] - 1) & 1, s_abort);   // the slot's previous tile (of this or the last item)
                            if (!ok) continue;
                            cnt[t]++;
                            tc_fence_after();
                            issue_s(t, q_addr[t], slot);
                            any_mma = true;
                            if (ka == 0) PAIR_TRACE(1, j, 1 + t);
                        }
                        if (!ok) break;
                        tc_commit(bar_k_empty + 8 * slot);
                        if (j + 1 == n) tc_commit(bar_q_empty + 8 * buf);   // the item's last score tiles have been issued
                    }
                    ka++;
                }
                if (!ok && any_mma) {
                    tc_commit(bar_q_empty);
                    for (uint32_t itn = 0; itn < 65536; ++itn) __nanosleep(64);   // no MMA of this CTA may still run when tensor memory is released
                }
            }
        } else {
            // ================= P.V issuer: O_t += P_t[j] . V[j] =================
            if (lane == 0) {
                constexpr uint32_t desc_hi = smem_desc_hi(1024);
                const uint32_t tO[2] = {tmem_base + 256, tmem_base + 320}, tP[2] = {tmem_base + 384, tmem_base + 448};
                bool ok = true;
                int g = 0, ka = 0;
                int cnt[2] = {0, 0};     // P tiles consumed per slot (phase of p_ready)
                bool any_mma = false;
                for (int item = item_lo; item < item_hi && ok; item++) {
                    const PairItem it = pair_item(a, item, n_pairs);
                    if (!it.active) continue;
                    const int n = it.n_tiles;
                    for (int j = 0; j < n && ok; j++, g++) {
                        const int slot = g % NS;
                        const bool more = j + 1 < n;
                        ok = mbar_wait(bar_v_full + 8 * slot, (g / NS) & 1, s_abort);
                        if (!ok) break;
                        const uint32_t vd = smem_desc_lo(sV + slot * kPairTile, kPanelBytes);
#pragma unroll
                        for (int t = 0; t < 2; t++) {
                            if (t == 1 && !it.live1) continue;
                            ok = mbar_wait(bar_p_ready + 8 * t, cnt[t] & 1, s_abort);
                            if (!ok) break;
                            cnt[t]++;
                            if (ka == 0) PAIR_TRACE(1, j, 3 + 2 * t);
                            tc_fence_after();
#pragma unroll
                            for (int ks = 0; ks < kTile / 16; ks++)
                                mma_ts(tO[t], tP[t] + ks * 8, desc64(vd + ks * (2048 >> 4), desc_hi), IDESC_PV, (j > 0 || ks > 0) ? 1u : 0u);
                            any_mma = true;
                            tc_commit(bar_pv_done + 8 * t);
                            if (!more) tc_commit(bar_o_done + 8 * t);
                            if (ka == 0) PAIR_TRACE(1, j, 4 + 2 * t);
                        }
                        if (!ok) break;
                        tc_commit(bar_v_empty + 8 * slot);
                    }
                    ka++;
                }
                if (!ok && any_mma) {
                    tc_commit(bar_v_empty);
                    for (uint32_t itn = 0; itn < 65536; ++itn) __nanosleep(64);
                }
            }
        }
    } else {
        // ================= softmax / correction / epilogue: slot t = warp / 4, thread r owns query row r of the slot =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;" ::: "memory");
        const int t = warp >> 2, r = tid & 127;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t tS = tmem_base + 128 * t + lane_base, tO = tmem_base + 256 + 64 * t + lane_base,
                       tP = tmem_base + 384 + 64 * t + lane_base;
        const float c = a.scale * kLog2e;
        const uint64_t c2 = pack2(c, c);
        bool ok = true;
        int cnt = 0, items_done = 0;   // score tiles / items this slot has processed (barrier phases)
        // The two slots share the exponential unit.  Started together they stay in lockstep: both compute (each at half
        // the unit's rate), then both wait (the unit idles).  Slot 1 therefore starts its first tile `stagger` clocks late
        // (about half a tile of exponentials): from then on one slot's loads, barriers and stores fall into the other
        // slot's exponentials, and since both slots do the same work per tile the offset persists across tiles and items.
        if (t == 1 && stagger > 0) {
            const long long t_go = clock64() + stagger;
            while (clock64() < t_go) __nanosleep(200);
        }
        for (int item = item_lo; item < item_hi && ok; item++) {
            const PairItem it = pair_item(a, item, n_pairs);
            const int pr = it.q0 + t * kTile + r;                    // packed row of this thread
            const int iq = pr / a.gqa, h = it.hk * a.gqa + pr % a.gqa;
            float* out = a.dst + (((int64_t)it.b * a.Tq + iq) * a.H + h) * HD;
            if (!it.active || (t == 1 && !it.live1)) {
                // no key, or a tile of padding rows: zeros for the rows that exist in dst, no tensor-core work
                if (pr < it.rows_total) {
#pragma unroll
                    for (int i = 0; i < HD / 4; i++) reinterpret_cast<float4*>(out)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                continue;
            }
            const bool row_live = pr < it.rows_live, row_zero = !row_live && pr < it.rows_total;
            float m_ref = -INFINITY, l_run = 0.0f;
            if (tid == 0) PAIR_TRACE(0, 16 + items_done, 0);
            for (int j = 0; j < it.n_tiles; j++, cnt++) {
                const bool tr = (r == 0) && items_done == 0;
                if (tr && t == 0) PAIR_TRACE(0, j, 7);
                ok = mbar_wait(bar_s_full + 8 * t, cnt & 1, s_abort);
                if (!ok) break;
                if (tr && t == 0) PAIR_TRACE(0, j, 0);
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) tmem_ld32(tS + q4 * 32, s[q4]);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_s_read + 8 * t);   // the tile is in registers: its columns may be overwritten
                if (tr && t == 0) PAIR_TRACE(0, j, 1);
                const int n_valid = it.len_b - j * kTile;   // the same for every row: columns >= n_valid are beyond the last key
                const bool full = n_valid >= kTile;
                if (j == 0) {
                    // first tile of an item: a first reference maximum from the row's first 32 scores - rarely more than
                    // 2^8 below the row's real maximum, and when it is the check below raises it and redoes the tile
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float x0 = (i < n_valid) ? __uint_as_float(s[0][i]) : -INFINITY;
                        const float x1 = (i + 1 < n_valid) ? __uint_as_float(s[0][i + 1]) : -INFINITY;
                        m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], x0, x1);
                    }
                    m_ref = max3(fmaxf(m4[0], m4[1]), m4[2], m4[3]) * c;
                }
                if (tr && t == 0) PAIR_TRACE(0, j, 2);
                bool pv_waited = (j == 0);   // the slot's previous P.V must have completed before P or O is written
                if (tr && t == 0) PAIR_TRACE(0, j, 3);
                // ---- P = exp2(S*c - m_ref) -> f16x2 -> tensor memory, 32 columns at a time.  The row maximum is tracked
                // in the same pass (the three-input maximum and the exponential sit on different pipes and overlap) and
                // only checked afterwards; a row that outgrew its reference by 2^8 raises it, rescales l and O, and the
                // tile is redone from the registers. ----
                float lsum = 0.0f;
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
                                float t0, t1, p0, p1;
                                unpack2(fma2(pack2(s0, s1), c2, nm2), t0, t1);
                                if (POLY > 0 && ((i >> 1) % (POLY > 0 ? POLY : 1)) == 0) {
                                    exp2_poly_pair(t0, t1, p0, p1);
                                } else {
                                    p0 = ex2(t0), p1 = ex2(t1);
                                }
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
                        if (!pv_waited) {
                            // the first 32 probabilities are in registers: only now must P[j-1] have been consumed
                            ok = mbar_wait(bar_pv_done + 8 * t, (cnt - 1) & 1, s_abort);
                            tc_fence_after();
                            pv_waited = true;
                        }
                        tmem_st16(tP + q4 * 16, preg);
                    }
                    if (!ok) break;
                    {
                        float l0, l1;
                        unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), l0, l1);
                        lsum = l0 + l1;
                    }
                    const float m_tile = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])) * c;   // c > 0
                    if (!__any_sync(0xffffffffu, m_tile > m_ref + kRescaleThreshold)) break;
                    const float m_new = fmaxf(m_ref, m_tile);
                    const float alpha = (m_new == -INFINITY) ? 1.0f : ex2(m_ref - m_new);
                    l_run *= alpha;
                    if (j > 0) {
                        tmem_wait_st();
#pragma unroll
                        for (int q4 = 0; q4 < HD / 32; q4++) {
                            uint32_t oreg[32];
                            tmem_ld32(tO + q4 * 32, oreg);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; i++) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
                            tmem_st32(tO + q4 * 32, oreg);
                        }
                    }
                    m_ref = m_new;
                }
                if (!ok) break;
                l_run += lsum;
                if (tr && t == 0) PAIR_TRACE(0, j, 4);
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_p_ready + 8 * t);
                if (tr && t == 0) PAIR_TRACE(0, j, 5);
            }
            if (!ok) break;
            if (tid == 0) PAIR_TRACE(0, 16 + items_done, 1);
            ok = mbar_wait(bar_o_done + 8 * t, items_done & 1, s_abort);
            if (!ok) break;
            if (tid == 0) PAIR_TRACE(0, 16 + items_done, 2);
            items_done++;
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
#pragma unroll
            for (int q4 = 0; q4 < HD / 32; q4++) {
                uint32_t oreg[32];
                tmem_ld32(tO + q4 * 32, oreg);
                tmem_wait_ld();
                if (row_live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4*>(out + q4 * 32 + i) =
                            make_float4(__uint_as_float(oreg[i]) * inv, __uint_as_float(oreg[i + 1]) * inv,
                                        __uint_as_float(oreg[i + 2]) * inv, __uint_as_float(oreg[i + 3]) * inv);
                } else if (row_zero) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(out + q4 * 32 + i) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            if (tid == 0) PAIR_TRACE(0, 16 + items_done - 1, 3);
            tc_fence_before();   // the reads of O are ordered before this thread's next arrival, which the next item's first P.V waits for
        }
    }

    // ---- teardown ----
#ifdef B200_TC5_TRACE
    if (tid == 0 && blockIdx.x < 192) {
        long long tnow;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tnow));
        (&g_tc5_trace[2][0][0])[blockIdx.x * 2 + 1] = tnow;
        if (blockIdx.x < 8) (&g_tc5_trace[1][40][0])[blockIdx.x * 2 + 1] = clock64();
    }
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}
