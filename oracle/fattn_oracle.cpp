// fattn_oracle.cpp — CPU restatement of GGML_OP_FLASH_ATTN_EXT and its neighbours.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is compared
// against and the "port" CPU baseline that bench.py times; the product library never
// links, loads or calls it.
//
// PARITY UNPINNED at the operator boundary: the reference's own arithmetic for this op
// lives in the un-vendored ggml submodule (CrispStrobe/ggml, branch sync/upstream-v0.17,
// pin a0f7289d ~ ggml v0.17.0: ggml/src/ggml-cpu/ops.cpp
// ggml_compute_forward_flash_attn_ext_f16), which is an empty directory in the reference
// tree, and no reference test holds golden outputs of the op.  What IS pinned, against
// in-tree reference code and the gguf-py library the reference's converters call:
//   * the plain multi-head attention of tests/test-core-cross-attn.cpp:99-137,
//   * the Q8_0 block format (gguf-py quants, call site models/convert-arkasr-to-gguf.py:304-305)
//     and the round-trip bound of tests/test-kv-quant-roundtrip.cpp:192-195,
//   * the rel-shift algebra of tools/dev/tiledbd_parity.cpp:28-32,57-66 and
//     src/core/fastconformer.h:98-102,118-130,876-918,
//   * the mask rules of src/crispasr.cpp:3467-3499 and src/voxtral.cpp:1187-1194.
//
// Rounding policy (the oracle of record): operands are taken in their storage type
// (Q rounded to F16 unless q_round_f16 == 0; K/V F16, F32 or Q8_0 with x = fp32(d)*q);
// mask values are read as F16; scores, softmax and P.V accumulate in fp32 (or fp64 when
// gold == 1); Q is never re-quantised against Q8_0 K; output fp32.

#include "../include/b200_fattn.h"

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- IEEE binary16 <-> binary32, round-to-nearest-even, bit-exact on every host ----
inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | man << 13;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | man << 13;
    } else {
        bits = sign | (exp + 127 - 15) << 23 | man << 13;
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  // rounds to inf
    if (x < 0x33000001u) return sign;                         // rounds to zero
    int exp = (int)(x >> 23) - 127;
    uint32_t man = (x & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t half_exp;
    if (exp < -14) {
        shift = 13 + (-14 - exp);
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(exp + 15);
    }
    uint32_t res = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (res & 1))) res++;
    if (half_exp == 0) return (uint16_t)(sign | res);  // subnormal (res may carry into exp=1: still right)
    res += (half_exp - 1) << 10;                       // res has the implicit bit at 0x400
    return (uint16_t)(sign | res);
}

inline float round_f16(float f) { return f16_to_f32(f32_to_f16(f)); }

struct Q80Block {
    uint16_t d;
    int8_t q[32];
};
static_assert(sizeof(Q80Block) == 34, "Q8_0 block is 34 bytes");

// Element c of the row that starts at `row` (type t).
inline float load_elem(const uint8_t* row, int type, int64_t c) {
    switch (type) {
        case B200_TYPE_F32: {
            float f;
            std::memcpy(&f, row + 4 * c, 4);
            return f;
        }
        case B200_TYPE_F16: {
            uint16_t h;
            std::memcpy(&h, row + 2 * c, 2);
            return f16_to_f32(h);
        }
        default: {  // Q8_0
            const uint8_t* blk = row + 34 * (c / 32);
            uint16_t d;
            std::memcpy(&d, blk, 2);
            return f16_to_f32(d) * (float)(int8_t)blk[2 + (c % 32)];
        }
    }
}

inline void load_row(const uint8_t* row, int type, int64_t n, float* out) {
    for (int64_t c = 0; c < n; c++) out[c] = load_elem(row, type, c);
}

inline const uint8_t* tptr(const b200_tensor* t, int64_t i1, int64_t i2, int64_t i3) {
    return (const uint8_t*)t->data + (uint64_t)i1 * t->nb[1] + (uint64_t)i2 * t->nb[2] + (uint64_t)i3 * t->nb[3];
}

// ALiBi slope of head h (ggml convention; zero max_bias gives 1).
inline float alibi_slope(float max_bias, int64_t n_head, int64_t h) {
    if (max_bias <= 0.0f) return 1.0f;
    const uint32_t n2 = 1u << (uint32_t)std::floor(std::log2((double)n_head));
    const float m0 = std::pow(2.0f, -max_bias / (float)n2);
    const float m1 = std::pow(2.0f, -(max_bias / 2.0f) / (float)n2);
    return (uint64_t)h < n2 ? std::pow(m0, (float)(h + 1)) : std::pow(m1, (float)(2 * (h - n2) + 1));
}

// Options of one oracle run.  The first three select the oracle of record (gold = fp64 accumulation).  q_as_q8_0
// and acc_f16 are DIAGNOSTIC switches: they restate two things the upstream CPU kernel is believed to do
// (unverifiable here, its source being absent) so that the distance they would move a result can be measured:
//   q_as_q8_0: against a Q8_0 K the query row is itself quantised to Q8_0 blocks and every block's dot product is
//              an integer sum times the two block scales (the vec-dot pairing of a quantised K);
//   acc_f16:   with F16 V the output row is accumulated key by key in F16 by a streaming softmax
//              (acc = f16(acc*ms); acc = f16(acc + v*vs)), instead of fp32 after a two-pass softmax.
// rows/n_rows restrict the computation to a subset of query rows (others are left untouched in dst).
struct OrcOptions {
    int gold = 0, q_round_f16 = 1, n_threads = 0;
    int q_as_q8_0 = 0, acc_f16 = 0;
    const int32_t* rows = nullptr;
    int n_rows = 0;
};

template <typename acc_t>
int flash_attn_impl(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v, const b200_tensor* mask,
                    const b200_tensor* dst, const b200_fattn_params* p, const b200_fattn_ext* ext, const OrcOptions& opt) {
    const int q_round_f16 = opt.q_round_f16, n_threads = opt.n_threads;
    const bool q_q8 = opt.q_as_q8_0 && k->type == B200_TYPE_Q8_0;
    const bool acc16 = opt.acc_f16 && v->type == B200_TYPE_F16;
    const int64_t hd = q->ne[0], Tq = q->ne[1], H = q->ne[2], B = q->ne[3];
    const int64_t Lk = k->ne[1], Hkv = k->ne[2], Bk = k->ne[3];
    const int64_t hdv = v->ne[0];
    if (k->ne[0] != hd || v->ne[1] != Lk || v->ne[2] != Hkv || v->ne[3] != Bk) return B200_E_SHAPE;
    if (Hkv <= 0 || H % Hkv || Bk <= 0 || B % Bk) return B200_E_SHAPE;
    if (dst->ne[0] != hdv || dst->ne[1] != H || dst->ne[2] != Tq || dst->ne[3] != B) return B200_E_SHAPE;
    if (mask && (mask->type != B200_TYPE_F16 || mask->ne[0] != Lk || mask->ne[1] < Tq)) return B200_E_SHAPE;
    const int64_t gqa = H / Hkv, bq = B / Bk;
    const b200_tensor* qv = ext ? ext->q_v : nullptr;
    const b200_tensor* r = ext ? ext->r : nullptr;
    if ((qv != nullptr) != (r != nullptr)) return B200_E_NULL;
    if (r && (Lk != Tq || r->ne[0] != hd || r->ne[1] != 2 * Tq - 1 || r->ne[2] != H)) return B200_E_SHAPE;
    const bool causal = ext && ext->causal;
    const int64_t n_past = ext ? ext->n_past : 0;
    const int32_t* kv_len = ext ? ext->kv_len : nullptr;
    const bool bias_f32 = ext && ext->relpos_bias_f32;
    const float scale = p->logit_softcap != 0.0f ? p->scale / p->logit_softcap : p->scale;
    const float ninf = -std::numeric_limits<float>::infinity();

#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#else
    (void)n_threads;
#endif

    int err = 0;
    // One (batch, kv head) at a time: K, V (and R) of that head are converted to fp32 once.
    for (int64_t b = 0; b < B && !err; b++) {
        const int64_t len_b = kv_len ? std::min<int64_t>(std::max<int64_t>(kv_len[b], 0), Lk) : Lk;
        for (int64_t hk = 0; hk < Hkv; hk++) {
            std::vector<float> Kf((size_t)Lk * hd), Vf((size_t)Lk * hdv);
#pragma omp parallel for schedule(static)
            for (int64_t ik = 0; ik < Lk; ik++) {
                load_row(tptr(k, ik, hk, b / bq), k->type, hd, &Kf[(size_t)ik * hd]);
                load_row(tptr(v, ik, hk, b / bq), v->type, hdv, &Vf[(size_t)ik * hdv]);
            }
            for (int64_t g = 0; g < gqa; g++) {
                const int64_t h = hk * gqa + g;
                const float slope = alibi_slope(p->max_bias, H, h);
                std::vector<float> Rf;
                if (r) {
                    Rf.resize((size_t)r->ne[1] * hd);
#pragma omp parallel for schedule(static)
                    for (int64_t ir = 0; ir < r->ne[1]; ir++)
                        load_row(tptr(r, ir, h, r->ne[3] > 1 ? b : 0), r->type, hd, &Rf[(size_t)ir * hd]);
                }
#pragma omp parallel
                {
                    std::vector<float> qrow(hd), qvrow(hd), s(Lk);
                    std::vector<acc_t> o(hdv);
                    std::vector<int8_t> qq(hd);          // q_as_q8_0: the query row as Q8_0 quants ...
                    std::vector<float> qd(hd / 32 + 1);  // ... and block scales (rounded to F16 like stored blocks)
                    std::vector<uint16_t> o16(hdv);      // acc_f16: the F16 accumulator
                    const int64_t n_iter = opt.rows ? opt.n_rows : Tq;
#pragma omp for schedule(dynamic, 4)
                    for (int64_t it = 0; it < n_iter; it++) {
                        const int64_t iq = opt.rows ? opt.rows[it] : it;
                        if (iq < 0 || iq >= Tq) continue;
                        load_row(tptr(q, iq, h, b), q->type, hd, qrow.data());
                        if (q_round_f16)
                            for (int64_t c = 0; c < hd; c++) qrow[c] = round_f16(qrow[c]);
                        if (q_q8) {
                            for (int64_t blk = 0; blk < hd / 32; blk++) {
                                float amax = 0.0f;
                                for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(qrow[blk * 32 + i]));
                                const float d = amax / 127.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
                                for (int i = 0; i < 32; i++) qq[blk * 32 + i] = (int8_t)std::round(qrow[blk * 32 + i] * id);
                                qd[blk] = round_f16(d);
                            }
                        }
                        if (qv) {
                            load_row(tptr(qv, iq, h, b), qv->type, hd, qvrow.data());
                            if (q_round_f16)
                                for (int64_t c = 0; c < hd; c++) qvrow[c] = round_f16(qvrow[c]);
                        }
                        const uint8_t* mrow =
                            mask ? tptr(mask, iq, h % mask->ne[2], b % mask->ne[3]) : nullptr;
                        int64_t kend = len_b;
                        if (causal) kend = std::min<int64_t>(kend, n_past + iq + 1);
                        float mx = ninf;
                        for (int64_t ik = 0; ik < kend; ik++) {
                            const float* kr = &Kf[(size_t)ik * hd];
                            acc_t acc = 0;
                            if (q_q8) {
                                // per block: integer dot of the quants, times both block scales, summed in fp32
                                const uint8_t* krow = tptr(k, ik, hk, b / bq);
                                float sumf = 0.0f;
                                for (int64_t blk = 0; blk < hd / 32; blk++) {
                                    const uint8_t* kb = krow + 34 * blk;
                                    uint16_t dk;
                                    std::memcpy(&dk, kb, 2);
                                    int sumi = 0;
                                    for (int i = 0; i < 32; i++) sumi += (int)qq[blk * 32 + i] * (int)(int8_t)kb[2 + i];
                                    sumf += (float)sumi * (qd[blk] * f16_to_f32(dk));
                                }
                                acc = (acc_t)sumf;
                            } else {
#pragma omp simd reduction(+ : acc)
                                for (int64_t c = 0; c < hd; c++) acc += (acc_t)qrow[c] * (acc_t)kr[c];
                            }
                            float sv = (float)acc * scale;
                            if (p->logit_softcap != 0.0f) sv = p->logit_softcap * std::tanh(sv);
                            if (r) {
                                const float* rr = &Rf[(size_t)(Tq - 1 + ik - iq) * hd];
                                acc_t bacc = 0;
#pragma omp simd reduction(+ : bacc)
                                for (int64_t c = 0; c < hd; c++) bacc += (acc_t)qvrow[c] * (acc_t)rr[c];
                                const float bias = (float)bacc * p->scale;
                                sv += bias_f32 ? bias : round_f16(bias);
                            }
                            if (mrow) {
                                uint16_t mh;
                                std::memcpy(&mh, mrow + 2 * ik, 2);
                                sv += slope * f16_to_f32(mh);
                            }
                            s[ik] = sv;
                            mx = std::max(mx, sv);
                        }
                        float* out = (float*)((uint8_t*)dst->data + (uint64_t)h * dst->nb[1] +
                                              (uint64_t)iq * dst->nb[2] + (uint64_t)b * dst->nb[3]);
                        if (mx == ninf) {  // every key masked (or no key): zeros
                            for (int64_t c = 0; c < hdv; c++) out[c] = 0.0f;
                            continue;
                        }
                        if (acc16) {
                            // streaming softmax in key order with an F16 output accumulator
                            std::fill(o16.begin(), o16.end(), (uint16_t)0);
                            float M = ninf, S = 0.0f;
                            for (int64_t ik = 0; ik < kend; ik++) {
                                const float sv = s[ik];
                                if (sv == ninf) continue;
                                float ms = 1.0f, vs = 1.0f;
                                if (sv > M) {
                                    ms = std::exp(M - sv);   // exp(-inf) = 0 on the first key
                                    M = sv;
                                    for (int64_t c = 0; c < hdv; c++) o16[c] = f32_to_f16(f16_to_f32(o16[c]) * ms);
                                } else {
                                    vs = std::exp(sv - M);
                                }
                                const float* vr = &Vf[(size_t)ik * hdv];
                                for (int64_t c = 0; c < hdv; c++) o16[c] = f32_to_f16(f16_to_f32(o16[c]) + vr[c] * vs);
                                S = S * ms + vs;
                            }
                            for (int64_t c = 0; c < hdv; c++) out[c] = f16_to_f32(o16[c]) / S;
                            continue;
                        }
                        std::fill(o.begin(), o.end(), (acc_t)0);
                        acc_t sum = 0;
                        for (int64_t ik = 0; ik < kend; ik++) {
                            const float pv = s[ik] == ninf ? 0.0f : std::exp(s[ik] - mx);
                            if (pv == 0.0f) continue;
                            sum += (acc_t)pv;
                            const float* vr = &Vf[(size_t)ik * hdv];
#pragma omp simd
                            for (int64_t c = 0; c < hdv; c++) o[c] += (acc_t)pv * (acc_t)vr[c];
                        }
                        const acc_t inv = (acc_t)1 / sum;
                        for (int64_t c = 0; c < hdv; c++) out[c] = (float)(o[c] * inv);
                    }
                }
            }
        }
    }
    return err;
}

}  // namespace

extern "C" {

// The operator. Host pointers everywhere (ext->kv_len included). gold != 0 accumulates in fp64.
B200_API int orc_flash_attn_ext(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                const b200_tensor* mask, const b200_tensor* dst, const b200_fattn_params* params,
                                const b200_fattn_ext* ext, int gold, int q_round_f16, int n_threads) {
    if (!q || !k || !v || !dst || !params) return B200_E_NULL;
    if (k->type != v->type) return B200_E_TYPE;
    OrcOptions opt;
    opt.gold = gold, opt.q_round_f16 = q_round_f16, opt.n_threads = n_threads;
    if (gold) return flash_attn_impl<double>(q, k, v, mask, dst, params, ext, opt);
    return flash_attn_impl<float>(q, k, v, mask, dst, params, ext, opt);
}

// The same with every option: `flags` bit 0 = gold, bit 1 = do NOT round Q to F16, bit 2 = q_as_q8_0 (diagnostic),
// bit 3 = acc_f16 (diagnostic); `rows` (may be NULL) lists the query rows to compute, other rows of dst are left alone.
B200_API int orc_flash_attn_ext_opt(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                    const b200_tensor* mask, const b200_tensor* dst, const b200_fattn_params* params,
                                    const b200_fattn_ext* ext, int flags, int n_threads, const int32_t* rows, int n_rows) {
    if (!q || !k || !v || !dst || !params) return B200_E_NULL;
    if (k->type != v->type) return B200_E_TYPE;
    OrcOptions opt;
    opt.gold = flags & 1, opt.q_round_f16 = !(flags & 2), opt.q_as_q8_0 = (flags >> 2) & 1, opt.acc_f16 = (flags >> 3) & 1;
    opt.n_threads = n_threads, opt.rows = rows, opt.n_rows = rows ? n_rows : 0;
    if (opt.gold) return flash_attn_impl<double>(q, k, v, mask, dst, params, ext, opt);
    return flash_attn_impl<float>(q, k, v, mask, dst, params, ext, opt);
}

// Q8_0 row quantisation as gguf-py quants.Q8_0.quantize_blocks does it (the library the
// reference's converters call): d = max|x|/127 kept in fp32 for the division, stored as fp16;
// q = round-half-away-from-zero(x * (1/d)), 1/d := 0 when d == 0.
B200_API void orc_quantize_q8_0(const float* x, uint8_t* out, int64_t n) {
    for (int64_t b = 0; b < n / 32; b++) {
        const float* xb = x + 32 * b;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(xb[i]));
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint8_t* blk = out + 34 * b;
        const uint16_t dh = f32_to_f16(d);
        std::memcpy(blk, &dh, 2);
        for (int i = 0; i < 32; i++) {
            const float t = xb[i] * id;
            // gguf-py np_roundf: floor(|t|) + floor(2*(|t| - floor(|t|))), sign restored == roundf
            blk[2 + i] = (uint8_t)(int8_t)std::round(t);
        }
    }
}

B200_API void orc_dequantize_q8_0(const uint8_t* in, float* x, int64_t n) {
    for (int64_t i = 0; i < n; i++) x[i] = load_elem(in, B200_TYPE_Q8_0, i);
}

B200_API void orc_f32_to_f16(const float* x, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = f32_to_f16(x[i]);
}
B200_API void orc_f16_to_f32(const uint16_t* x, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = f16_to_f32(x[i]);
}

// Sinusoidal relative-position table of src/core/fastconformer.h:118-130:
// row p in [0, 2T-2] holds position T-1-p; pe[p*d + 2i] = sin(pos*div_i), pe[p*d + 2i+1] = cos(pos*div_i).
B200_API void orc_make_pos_enc(int d_model, int T, float* pe) {
    const int n_pos = 2 * T - 1;
    for (int p = 0; p < n_pos; p++) {
        const float pos = (float)(T - 1 - p);
        for (int i = 0; i < d_model / 2; i++) {
            const float div = std::exp(-std::log(10000.0f) * (float)(2 * i) / (float)d_model);
            pe[(size_t)p * d_model + 2 * i] = std::sin(pos * div);
            pe[(size_t)p * d_model + 2 * i + 1] = std::cos(pos * div);
        }
    }
}

// The materialised bias-as-mask of src/core/fastconformer.h:880-918:
// BD_raw[r,q,h] = sum_c R[c,r,h] * Q_v[c,q,h]; BD[k,q,h] = BD_raw[k-q+T-1, q, h];
// out[k,q,h] = f16(scale * BD[k,q,h]).  out is contiguous [T, T, H] F16 (k fastest).
B200_API int orc_relpos_mask(const b200_tensor* q_v, const b200_tensor* r, float scale, int q_round_f16,
                             uint16_t* out) {
    const int64_t hd = q_v->ne[0], T = q_v->ne[1], H = q_v->ne[2];
    if (r->ne[0] != hd || r->ne[1] != 2 * T - 1 || r->ne[2] != H) return B200_E_SHAPE;
    for (int64_t h = 0; h < H; h++) {
        std::vector<float> Rf((size_t)r->ne[1] * hd);
        for (int64_t ir = 0; ir < r->ne[1]; ir++) load_row(tptr(r, ir, h, 0), r->type, hd, &Rf[(size_t)ir * hd]);
#pragma omp parallel for schedule(static)
        for (int64_t iq = 0; iq < T; iq++) {
            std::vector<float> qrow(hd);
            load_row(tptr(q_v, iq, h, 0), q_v->type, hd, qrow.data());
            if (q_round_f16)
                for (int64_t c = 0; c < hd; c++) qrow[c] = round_f16(qrow[c]);
            for (int64_t ik = 0; ik < T; ik++) {
                const float* rr = &Rf[(size_t)(T - 1 + ik - iq) * hd];
                float acc = 0;
#pragma omp simd reduction(+ : acc)
                for (int64_t c = 0; c < hd; c++) acc += qrow[c] * rr[c];
                out[((size_t)h * T + iq) * T + ik] = f32_to_f16(acc * scale);
            }
        }
    }
    return 0;
}

// Whisper beam mask rule of src/crispasr.cpp:3480-3488: for token j (sequence seq[j], position
// pos[j]) cell i is masked iff the cell does not carry seq[j] or cell_pos[i] > pos[j].
// cell_seq_bits[i] is a bitset of the sequence ids held by cell i. out is [n_kv, n_tokens] F16.
B200_API void orc_whisper_beam_mask(const int32_t* cell_pos, const uint32_t* cell_seq_bits, int n_kv,
                                    const int32_t* tok_seq, const int32_t* tok_pos, int n_tokens, uint16_t* out) {
    for (int j = 0; j < n_tokens; j++)
        for (int i = 0; i < n_kv; i++) {
            const bool masked = !((cell_seq_bits[i] >> tok_seq[j]) & 1u) || cell_pos[i] > tok_pos[j];
            out[(size_t)j * n_kv + i] = masked ? 0xFC00u : 0x0000u;
        }
}

// LLM causal mask rule of src/voxtral.cpp:1187-1194: mask[q][k] = -inf iff k > n_past + q.
B200_API void orc_causal_mask(int Lk, int T, int n_past, uint16_t* out) {
    for (int qi = 0; qi < T; qi++)
        for (int ki = 0; ki < Lk; ki++) out[(size_t)qi * Lk + ki] = ki > n_past + qi ? 0xFC00u : 0x0000u;
}

B200_API int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
