// kv_slab.cu — KV-cache slabs and the append (row quantise-on-write) kernels.
//
// Layout: one arena per cache, holding 2*n_layers slabs (K then V per layer), each slab starting
// on a 1024-byte boundary.  Inside a slab rows are head-major, ggml view [hd, max_ctx, n_kv, n_streams]:
//   nb1 = row bytes (hd*2 for F16, hd/32*34 for Q8_0), nb2 = ctx_rows*nb1, nb3 = n_kv*nb2,
// with ctx_rows = max_ctx rounded up to a multiple of 32 so that every head's row range starts on a
// 16-byte boundary for both row sizes (a Q8_0 row of head_dim 128 is 136 bytes).
#include <cstdio>
#include <new>

#include "fattn_common.cuh"

struct b200_kv_cache {
    b200_kv_config cfg;
    uint8_t* arena;   // cudaMalloc'ed
    uint8_t* base;    // arena rounded up to 1024
    size_t slab_bytes;
    size_t row_bytes;
    int64_t ctx_rows;
    int device;
};

namespace b200 {
namespace {

// F32 rows -> F16 rows. One thread per element pair.
__global__ void kv_append_f16_kernel(const uint8_t* src, int64_t snb1, int64_t snb2, int64_t snb3, uint8_t* dst,
                                     int64_t dnb1, int64_t dnb2, int64_t dnb3, int hd, int n_new, int n_kv,
                                     int n_streams, const int32_t* pos, int pos0, int ctx_rows) {
    const int64_t total = (int64_t)n_streams * n_kv * n_new * (hd / 2);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c2 = (int)(i % (hd / 2));
        const int row = (int)((i / (hd / 2)) % n_new);
        const int h = (int)((i / ((int64_t)(hd / 2) * n_new)) % n_kv);
        const int s = (int)(i / ((int64_t)(hd / 2) * n_new * n_kv));
        const int p = (pos ? pos[s] : pos0) + row;
        if (p < 0 || p >= ctx_rows) continue;  // out-of-range rows are dropped, never written
        const float2 x = *reinterpret_cast<const float2*>(src + row * snb1 + h * snb2 + s * snb3 + (int64_t)c2 * 8);
        *reinterpret_cast<__half2*>(dst + p * dnb1 + h * dnb2 + s * dnb3 + (int64_t)c2 * 4) = __floats2half2_rn(x.x, x.y);
    }
}

// F32 rows -> Q8_0 blocks, bit-identical to gguf-py quantize_blocks: d = amax/127 (fp32), stored as
// fp16; q = roundf(x * (1/d)) with 1/d = 0 for d == 0.  One warp per block, one lane per element.
__global__ void kv_append_q8_0_kernel(const uint8_t* src, int64_t snb1, int64_t snb2, int64_t snb3, uint8_t* dst,
                                      int64_t dnb1, int64_t dnb2, int64_t dnb3, int hd, int n_new, int n_kv,
                                      int n_streams, const int32_t* pos, int pos0, int ctx_rows) {
    const int lane = threadIdx.x & 31;
    const int nblk = hd / 32;
    const int64_t total = (int64_t)n_streams * n_kv * n_new * nblk;
    const int64_t warp0 = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t i = warp0; i < total; i += nwarps) {
        const int blk = (int)(i % nblk);
        const int row = (int)((i / nblk) % n_new);
        const int h = (int)((i / ((int64_t)nblk * n_new)) % n_kv);
        const int s = (int)(i / ((int64_t)nblk * n_new * n_kv));
        const int p = (pos ? pos[s] : pos0) + row;
        if (p < 0 || p >= ctx_rows) continue;
        const float x = *reinterpret_cast<const float*>(src + row * snb1 + h * snb2 + s * snb3 + (int64_t)(blk * 32 + lane) * 4);
        float amax = fabsf(x);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        const int q = (int)roundf(__fmul_rn(x, id));
        uint8_t* out = dst + p * dnb1 + h * dnb2 + s * dnb3 + (int64_t)blk * 34;
        // pack two int8 per 16-bit store (blocks are only 2-byte aligned)
        const int qn = __shfl_down_sync(0xffffffffu, q, 1);
        if ((lane & 1) == 0)
            *reinterpret_cast<uint16_t*>(out + 2 + lane) = (uint16_t)((q & 0xFF) | ((qn & 0xFF) << 8));
        if (lane == 0) *reinterpret_cast<__half*>(out) = __float2half_rn(d);
    }
}

}  // namespace
}  // namespace b200

extern "C" {

B200_API int b200_kv_create(const b200_kv_config* cfg, b200_kv_cache** out) {
    if (!cfg || !out) return B200_E_NULL;
    *out = nullptr;
    if (cfg->type != B200_TYPE_F16 && cfg->type != B200_TYPE_Q8_0) return B200_E_TYPE;
    if (cfg->head_dim <= 0 || cfg->head_dim % 32 || cfg->head_dim > 128) return B200_E_UNSUPPORTED;
    if (cfg->n_kv_heads <= 0 || cfg->n_layers <= 0 || cfg->max_ctx <= 0 || cfg->n_streams <= 0) return B200_E_SHAPE;
    b200_kv_cache* kv = new (std::nothrow) b200_kv_cache();
    if (!kv) return B200_E_CUDA;
    kv->cfg = *cfg;
    kv->row_bytes = cfg->type == B200_TYPE_F16 ? (size_t)cfg->head_dim * 2 : (size_t)cfg->head_dim / 32 * 34;
    kv->ctx_rows = ((int64_t)cfg->max_ctx + 31) / 32 * 32;
    const size_t raw = kv->row_bytes * kv->ctx_rows * cfg->n_kv_heads * cfg->n_streams;
    kv->slab_bytes = (raw + 1023) / 1024 * 1024;
    const size_t total = kv->slab_bytes * 2 * cfg->n_layers + 1024;
    if (cudaGetDevice(&kv->device) != cudaSuccess) {
        delete kv;
        return B200_E_NO_DEVICE;
    }
    if (cudaMalloc((void**)&kv->arena, total) != cudaSuccess) {
        cudaGetLastError();
        delete kv;
        return B200_E_CUDA;
    }
    kv->base = (uint8_t*)(((uintptr_t)kv->arena + 1023) / 1024 * 1024);
    // a cleared cache reads as zeros (whisper clears kv_pad at init, src/crispasr.cpp:1506)
    if (cudaMemset(kv->arena, 0, total) != cudaSuccess) {
        cudaFree(kv->arena);
        delete kv;
        return B200_E_CUDA;
    }
    *out = kv;
    return B200_OK;
}

B200_API void b200_kv_destroy(b200_kv_cache* kv) {
    if (!kv) return;
    if (kv->arena) cudaFree(kv->arena);
    delete kv;
}

B200_API size_t b200_kv_bytes(const b200_kv_cache* kv) { return kv ? kv->slab_bytes * 2 * kv->cfg.n_layers : 0; }

B200_API int b200_kv_view(const b200_kv_cache* kv, int layer, int64_t n_rows, b200_tensor* k, b200_tensor* v) {
    if (!kv || !k || !v) return B200_E_NULL;
    if (layer < 0 || layer >= kv->cfg.n_layers || n_rows <= 0 || n_rows > kv->ctx_rows) return B200_E_SHAPE;
    for (int which = 0; which < 2; which++) {
        b200_tensor* t = which ? v : k;
        t->data = kv->base + kv->slab_bytes * (2 * (size_t)layer + which);
        t->type = kv->cfg.type;
        t->reserved = 0;
        t->ne[0] = kv->cfg.head_dim, t->ne[1] = n_rows, t->ne[2] = kv->cfg.n_kv_heads, t->ne[3] = kv->cfg.n_streams;
        t->nb[0] = kv->cfg.type == B200_TYPE_F16 ? 2 : 34;
        t->nb[1] = kv->row_bytes;
        t->nb[2] = kv->row_bytes * kv->ctx_rows;
        t->nb[3] = t->nb[2] * kv->cfg.n_kv_heads;
    }
    return B200_OK;
}

B200_API int b200_kv_append(b200_kv_cache* kv, int layer, const b200_tensor* k_new, const b200_tensor* v_new,
                            const int32_t* pos, int32_t pos0, void* cuda_stream) {
    if (!kv || !k_new || !v_new) return B200_E_NULL;
    if (layer < 0 || layer >= kv->cfg.n_layers) return B200_E_SHAPE;
    b200_tensor kd, vd;
    b200_kv_view(kv, layer, kv->ctx_rows, &kd, &vd);
    for (int which = 0; which < 2; which++) {
        const b200_tensor* s = which ? v_new : k_new;
        const b200_tensor* d = which ? &vd : &kd;
        if (!s->data) return B200_E_NULL;
        if (s->type != B200_TYPE_F32) return B200_E_TYPE;
        if (s->nb[0] != 4) return B200_E_STRIDE;
        if ((uintptr_t)s->data % 8 || s->nb[1] % 8 || s->nb[2] % 8 || s->nb[3] % 8) return B200_E_ALIGN;
        if (s->ne[0] != kv->cfg.head_dim || s->ne[2] != kv->cfg.n_kv_heads || s->ne[3] != kv->cfg.n_streams)
            return B200_E_SHAPE;
        const int n_new = (int)s->ne[1];
        if (n_new <= 0 || n_new > kv->ctx_rows) return B200_E_SHAPE;
        if (!pos && (pos0 < 0 || pos0 + n_new > kv->ctx_rows)) return B200_E_SHAPE;
        const int64_t work = (int64_t)kv->cfg.n_streams * kv->cfg.n_kv_heads * n_new * kv->cfg.head_dim;
        cudaStream_t st = (cudaStream_t)cuda_stream;
        if (kv->cfg.type == B200_TYPE_F16) {
            const int64_t threads = work / 2;
            const int blocks = (int)((threads + 255) / 256 > 148 * 16 ? 148 * 16 : (threads + 255) / 256);
            b200::kv_append_f16_kernel<<<blocks, 256, 0, st>>>(
                (const uint8_t*)s->data, (int64_t)s->nb[1], (int64_t)s->nb[2], (int64_t)s->nb[3], (uint8_t*)d->data,
                (int64_t)d->nb[1], (int64_t)d->nb[2], (int64_t)d->nb[3], kv->cfg.head_dim, n_new, kv->cfg.n_kv_heads,
                kv->cfg.n_streams, pos, pos0, (int)kv->ctx_rows);
        } else {
            const int64_t threads = work;  // one lane per element
            const int blocks = (int)((threads + 255) / 256 > 148 * 16 ? 148 * 16 : (threads + 255) / 256);
            b200::kv_append_q8_0_kernel<<<blocks, 256, 0, st>>>(
                (const uint8_t*)s->data, (int64_t)s->nb[1], (int64_t)s->nb[2], (int64_t)s->nb[3], (uint8_t*)d->data,
                (int64_t)d->nb[1], (int64_t)d->nb[2], (int64_t)d->nb[3], kv->cfg.head_dim, n_new, kv->cfg.n_kv_heads,
                kv->cfg.n_streams, pos, pos0, (int)kv->ctx_rows);
        }
        if (cudaGetLastError() != cudaSuccess) return B200_E_CUDA;
    }
    return B200_OK;
}

B200_API int b200_kv_copy_stream(b200_kv_cache* kv, int dst_stream, int src_stream, int64_t n_rows, void* cuda_stream) {
    if (!kv) return B200_E_NULL;
    if (dst_stream < 0 || src_stream < 0 || dst_stream >= kv->cfg.n_streams || src_stream >= kv->cfg.n_streams)
        return B200_E_SHAPE;
    if (n_rows < 0 || n_rows > kv->ctx_rows) return B200_E_SHAPE;
    if (dst_stream == src_stream || n_rows == 0) return B200_OK;
    const size_t head_pitch = kv->row_bytes * kv->ctx_rows;
    const size_t stream_pitch = head_pitch * kv->cfg.n_kv_heads;
    for (int slab = 0; slab < 2 * kv->cfg.n_layers; slab++) {
        uint8_t* base = kv->base + kv->slab_bytes * slab;
        // one 2-D copy per slab: n_kv_heads rows of n_rows*row_bytes bytes, head_pitch apart
        if (cudaMemcpy2DAsync(base + stream_pitch * dst_stream, head_pitch, base + stream_pitch * src_stream, head_pitch,
                              (size_t)n_rows * kv->row_bytes, kv->cfg.n_kv_heads, cudaMemcpyDeviceToDevice,
                              (cudaStream_t)cuda_stream) != cudaSuccess) {
            cudaGetLastError();
            return B200_E_CUDA;
        }
    }
    return B200_OK;
}

}  // extern "C"
