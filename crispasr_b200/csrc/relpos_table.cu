// relpos_table.cu — the relative-position table R of the FastConformer attention block, built on the device and
// cached per (layer, T).
//
// The reference forms it on every graph build: pos_enc = make_pos_enc(d, T) on the host
// (src/core/fastconformer.h:118-130: row p in [0, 2T-2] holds position T-1-p, pe[p][2i] = sin(pos*div_i),
// pe[p][2i+1] = cos(pos*div_i), div_i = exp(-ln(1e4)*2i/d)), uploaded, then R = MUL_MAT(attn_pos_w, pos_enc)
// (:843), reshaped [hd, H, 2T-1] and permuted to [hd, 2T-1, H] (:851).  R depends on the layer's weight and on T
// only, so this file computes it once per (layer, T), straight into the F16 head-major layout the fused
// attention kernels read ([hd, 2T-1, H] contiguous), and hands out the cached table afterwards.
//
//   R[c, p, h] = f16( sum_k attn_pos_w[k, h*hd + c] * pe[k, p] )      (fp32 products and sums, one rounding)
//
// The sinusoid is generated inside the GEMM's operand load (no pos_enc tensor exists), the product is a plain
// shared-memory tiled fp32 GEMM on the FMA pipe: 2*(2T-1)*d*d FLOP once per (layer, T) (31 GFLOP at T = 7500,
// d = 1024) against 461 GFLOP of attention per utterance-layer, so it is nowhere near the hot loop and fp32
// keeps it within one F16 rounding of the reference's F32 mul_mat.
#include <cmath>
#include <mutex>
#include <new>
#include <vector>

#include "fattn_common.cuh"

struct b200_relpos_cache {
    struct Entry {
        int T = 0;
        int n_heads = 0, d_model = 0;
        const void* weight = nullptr;   // the weight pointer the entry was built from (part of the key)
        uint8_t* data = nullptr;        // cudaMalloc'ed [hd, 2T-1, H] F16
        uint64_t stamp = 0;             // last use, for eviction
    };
    std::vector<std::vector<Entry>> layers;
    int max_per_layer = 0;
    int device = -1;
    uint64_t clock = 0;
    size_t bytes = 0;
    std::mutex mu;
};

namespace b200 {
namespace {

constexpr int kBM = 64, kBN = 64, kBK = 16;
constexpr int kMaxDiv = 1024;   // d_model / 2 frequencies at most (d_model <= 2048)

// The d/2 frequencies div_i = expf(-logf(10000.0f) * (float)(2 * i) / (float)d_model), evaluated on the HOST with the
// reference's own expression (src/core/fastconformer.h:124) and handed to the kernel by value: an exponential that
// is one ulp off turns into an angle error of up to 7499 * 6e-8 = 4.5e-4 rad at the far end of a 10-minute
// utterance, i.e. a whole F16 ulp of R; with the host's value the device forms the same fp32 angle as the reference.
struct DivTable {
    float v[kMaxDiv];
};

// One 64 (positions) x 64 (output features) tile of R per CTA, 256 threads, 4 x 4 outputs per thread.
// A = pe [2T-1, d] generated on the fly, B = W [d_out, d_in] (row o contiguous over the input feature k).
template <typename WT>
__global__ void __launch_bounds__(256) relpos_table_kernel(const WT* __restrict__ w, int64_t w_row_stride, int d, int T, int hd,
                                                           __half* __restrict__ r_out, const __grid_constant__ DivTable div_tab) {
    __shared__ float sA[kBK][kBM + 4];
    __shared__ float sB[kBK][kBN + 4];
    const int n_pos = 2 * T - 1;
    const int p0 = blockIdx.x * kBM, o0 = blockIdx.y * kBN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < d; k0 += kBK) {
        // A tile: 64 positions x 16 features = 1024 values, 4 per thread
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int idx = tid + it * 256;
            const int kk = idx & 15, pp = idx >> 4;
            const int p = p0 + pp, k = k0 + kk;
            float val = 0.0f;
            if (p < n_pos && k < d) {
                const float pos = (float)(T - 1 - p);
                const float ang = __fmul_rn(pos, div_tab.v[k >> 1]);
                val = (k & 1) ? cosf(ang) : sinf(ang);
            }
            sA[kk][pp] = val;
        }
        // B tile: 64 output features x 16 input features
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int idx = tid + it * 256;
            const int kk = idx & 15, oo = idx >> 4;
            const int o = o0 + oo, k = k0 + kk;
            sB[kk][oo] = (o < d && k < d) ? (float)w[(int64_t)o * w_row_stride + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kBK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = sB[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int p = p0 + ty * 4 + i;
        if (p >= n_pos) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int o = o0 + tx * 4 + j;
            if (o >= d) continue;
            const int h = o / hd, c = o % hd;
            r_out[((int64_t)h * n_pos + p) * hd + c] = __float2half_rn(acc[i][j]);
        }
    }
}

int check_weight(const b200_tensor* w, int n_heads, int T) {
    if (!w || !w->data) return B200_E_NULL;
    if (w->type != B200_TYPE_F32 && w->type != B200_TYPE_F16) return B200_E_TYPE;
    const size_t es = w->type == B200_TYPE_F32 ? 4 : 2;
    if (w->nb[0] != es || w->nb[1] % es) return B200_E_STRIDE;
    if ((uintptr_t)w->data % es) return B200_E_ALIGN;
    if (w->ne[0] <= 0 || w->ne[0] != w->ne[1] || w->ne[2] != 1 || w->ne[3] != 1) return B200_E_SHAPE;
    if (n_heads <= 0 || w->ne[0] % n_heads || w->ne[0] % 2 || T <= 0 || T > (1 << 20)) return B200_E_SHAPE;
    if (w->ne[0] > 2 * kMaxDiv) return B200_E_LIMIT;
    return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" {

B200_API int b200_relpos_table(const b200_tensor* attn_pos_w, int n_heads, int T, void* r_out, size_t r_bytes, void* cuda_stream) {
    int rc = b200::check_weight(attn_pos_w, n_heads, T);
    if (rc != B200_OK) return rc;
    if (!r_out) return B200_E_NULL;
    const int d = (int)attn_pos_w->ne[0], hd = d / n_heads;
    const size_t need = (size_t)d * (2 * (size_t)T - 1) * 2;
    if (r_bytes < need) return B200_E_WORKSPACE;
    if ((uintptr_t)r_out % 16) return B200_E_ALIGN;
    dim3 grid((2 * T - 1 + b200::kBM - 1) / b200::kBM, (d + b200::kBN - 1) / b200::kBN);
    cudaStream_t st = (cudaStream_t)cuda_stream;
    b200::DivTable div;
    for (int i = 0; i < d / 2; i++) div.v[i] = expf(-logf(10000.0f) * (float)(2 * i) / (float)d);
    for (int i = d / 2; i < b200::kMaxDiv; i++) div.v[i] = 0.0f;
    if (attn_pos_w->type == B200_TYPE_F32)
        b200::relpos_table_kernel<float><<<grid, 256, 0, st>>>((const float*)attn_pos_w->data, (int64_t)(attn_pos_w->nb[1] / 4), d, T, hd,
                                                                 (__half*)r_out, div);
    else
        b200::relpos_table_kernel<__half><<<grid, 256, 0, st>>>((const __half*)attn_pos_w->data, (int64_t)(attn_pos_w->nb[1] / 2), d, T,
                                                                  hd, (__half*)r_out, div);
    return cudaGetLastError() == cudaSuccess ? B200_OK : B200_E_CUDA;
}

B200_API int b200_relpos_cache_create(int n_layers, int max_entries_per_layer, b200_relpos_cache** out) {
    if (!out) return B200_E_NULL;
    *out = nullptr;
    if (n_layers <= 0 || max_entries_per_layer <= 0) return B200_E_SHAPE;
    b200_relpos_cache* c = new (std::nothrow) b200_relpos_cache();
    if (!c) return B200_E_STATE;
    c->layers.resize(n_layers);
    c->max_per_layer = max_entries_per_layer;
    if (cudaGetDevice(&c->device) != cudaSuccess) {
        cudaGetLastError();
        delete c;
        return B200_E_NO_DEVICE;
    }
    *out = c;
    return B200_OK;
}

B200_API void b200_relpos_cache_destroy(b200_relpos_cache* c) {
    if (!c) return;
    for (auto& layer : c->layers)
        for (auto& e : layer)
            if (e.data) cudaFree(e.data);
    delete c;
}

B200_API size_t b200_relpos_cache_bytes(const b200_relpos_cache* c) { return c ? c->bytes : 0; }

B200_API int b200_relpos_cache_get(b200_relpos_cache* c, int layer, int T, const b200_tensor* attn_pos_w, int n_heads,
                                   void* cuda_stream, b200_tensor* r, int* was_hit) {
    if (!c || !r) return B200_E_NULL;
    if (layer < 0 || layer >= (int)c->layers.size()) return B200_E_SHAPE;
    int rc = b200::check_weight(attn_pos_w, n_heads, T);
    if (rc != B200_OK) return rc;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != c->device) return B200_E_STATE;   // tables live on the cache's device
    const int d = (int)attn_pos_w->ne[0], hd = d / n_heads;
    std::lock_guard<std::mutex> lk(c->mu);
    auto& entries = c->layers[layer];
    b200_relpos_cache::Entry* e = nullptr;
    for (auto& x : entries)
        if (x.T == T && x.n_heads == n_heads && x.d_model == d && x.weight == attn_pos_w->data) e = &x;
    const bool hit = e != nullptr;
    if (!hit) {
        const size_t bytes = (size_t)d * (2 * (size_t)T - 1) * 2;
        uint8_t* buf = nullptr;
        if (cudaMalloc((void**)&buf, bytes) != cudaSuccess) {
            cudaGetLastError();
            return B200_E_CUDA;
        }
        rc = b200_relpos_table(attn_pos_w, n_heads, T, buf, bytes, cuda_stream);
        if (rc != B200_OK) {
            cudaFree(buf);
            return rc;
        }
        if ((int)entries.size() >= c->max_per_layer) {
            // evict the least recently used table of this layer (cudaFree waits for work that may still read it)
            size_t victim = 0;
            for (size_t i = 1; i < entries.size(); i++)
                if (entries[i].stamp < entries[victim].stamp) victim = i;
            c->bytes -= (size_t)entries[victim].d_model * (2 * (size_t)entries[victim].T - 1) * 2;
            cudaFree(entries[victim].data);
            entries.erase(entries.begin() + victim);
        }
        entries.emplace_back();
        e = &entries.back();
        e->T = T, e->n_heads = n_heads, e->d_model = d, e->weight = attn_pos_w->data, e->data = buf;
        c->bytes += bytes;
    }
    e->stamp = ++c->clock;
    r->data = e->data;
    r->type = B200_TYPE_F16;
    r->reserved = 0;
    r->ne[0] = hd, r->ne[1] = 2 * (int64_t)T - 1, r->ne[2] = n_heads, r->ne[3] = 1;
    r->nb[0] = 2, r->nb[1] = (uint64_t)hd * 2, r->nb[2] = r->nb[1] * (uint64_t)(2 * (int64_t)T - 1), r->nb[3] = r->nb[2] * n_heads;
    if (was_hit) *was_hit = hit ? 1 : 0;
    return B200_OK;
}

}  // extern "C"
