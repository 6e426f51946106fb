/*
 * b200_fattn.h — C-ABI of the B200-native fused attention path.
 *
 * This library implements exactly one operator of the CrispASR/ggml stack,
 * GGML_OP_FLASH_ATTN_EXT, plus the two pieces of host plumbing that feed it
 * (a KV-cache slab allocator and a per-GPU segment scheduler).  Every entry
 * point is plain C: pointers, sizes and enums, no C++ or torch types.
 *
 * Tensor descriptors use ggml conventions throughout: ne[0] is the fastest
 * dimension, nb[i] is the stride of dimension i in BYTES, nb[0] is the size of
 * one element (or of one quantised block), `data` is a DEVICE pointer unless an
 * entry point says otherwise.
 *
 * Operator contract (reference call sites: src/crispasr.cpp:2821,3220,3280;
 * src/core/attention.h:478,572,992; src/core/fastconformer.h:933;
 * src/core/cross_attn.h:148; src/canary.cpp:971,994):
 *
 *   Q    [hd,  Tq, H,   B]  F32 or F16, nb[0] == element size
 *   K    [hd,  Lk, Hkv, Bk] F16, F32 or Q8_0 (34-byte blocks of 32), H % Hkv == 0, B % Bk == 0
 *   V    [hdv, Lk, Hkv, Bk] same type as K (hdv == hd in this library)
 *   mask [Lk,  Tq, 1|H, 1|B] F16 or NULL; 0 = attend, -inf = masked, any finite value = additive bias
 *   dst  [hdv, H,  Tq,  B]  F32, contiguous; 16-byte aligned base for head_dim 64 / 128 (else B200_E_ALIGN)
 *
 *   s[k]   = scale * sum_c Q[c,q,h,b] * K[c,k,h/(H/Hkv),b/(B/Bk)]
 *   s[k]   = softcap * tanh(s[k] / softcap)                (only when logit_softcap != 0)
 *   s[k]  += slope(h) * mask[k,q,h%mask.ne2,b%mask.ne3]    (slope == 1 when max_bias == 0)
 *   dst[:,h,q,b] = sum_k softmax_k(s)[k] * V[:,k,...]      (fp32 softmax, fp32 accumulation)
 *
 * Q is rounded to F16 before the dot product (it is the tensor-core operand
 * type); K/V quantised blocks are dequantised as fp32(d) * q.  A row whose keys
 * are all masked yields zeros.
 */
#ifndef B200_FATTN_H
#define B200_FATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200_API
#else
#define B200_API __attribute__((visibility("default")))
#endif

/* Numeric ids equal ggml's GGML_TYPE_* / gguf-py GGMLQuantizationType (F32=0, F16=1, Q8_0=8). */
typedef enum b200_type {
    B200_TYPE_F32 = 0,
    B200_TYPE_F16 = 1,
    B200_TYPE_Q8_0 = 8,
} b200_type;

/* Mirrors the fields of `struct ggml_tensor` the operator reads (data, type, ne, nb). */
typedef struct b200_tensor {
    void* data;
    int32_t type; /* b200_type */
    int32_t reserved;
    int64_t ne[4];
    uint64_t nb[4];
} b200_tensor;

/* op_params of ggml_flash_attn_ext(ctx, q, k, v, mask, scale, max_bias, logit_softcap)
 * (+ ggml_flash_attn_ext_set_prec). prec_f32 is accepted and ignored: softmax and
 * accumulation are always fp32. */
typedef struct b200_fattn_params {
    float scale;
    float max_bias;
    float logit_softcap;
    int32_t prec_f32;
} b200_fattn_params;

/* Optional fused extensions. A NULL pointer or an all-zero struct is the plain ggml op. */
typedef struct b200_fattn_ext {
    /* FastConformer relative-position bias, replacing the materialised F16 mask that
     * src/core/fastconformer.h:880-918 builds (MUL_MAT(R,Q_v) -> rel_shift -> scale -> cast F16):
     *   bias[k,q,h] = f16( scale * sum_c q_v[c,q,h] * r[c, (Tq-1) + k - q, h] )
     * q_v has the shape and type rules of Q; r is [hd, 2*Tq-1, H, 1|B] F16 or F32. Requires
     * Lk == Tq and either q_v or the two position biases below. May be combined with `mask` (added after the bias) and kv_len. */
    const b200_tensor* q_v;
    const b200_tensor* r;
    /* Untied position biases folded into the Q load, replacing the two ggml_add passes of
     * src/core/fastconformer.h:846-847 (Q_u = Q + pos_bias_u, Q_v = Q + pos_bias_v): both are F32
     * [hd, H] contiguous. Given together with `r` and a NULL q_v, the op reads Q once and uses
     * f16(Q + pos_bias_u) for the content scores and f16(Q + pos_bias_v) for the bias (the sums are
     * formed in fp32 and rounded once, as the reference's F32 add followed by the op's F16 conversion).
     * With a non-NULL q_v they must be NULL. */
    const b200_tensor* pos_bias_u;
    const b200_tensor* pos_bias_v;
    /* Implicit causal mask of src/voxtral.cpp:1187-1194: key k is masked iff k > n_past + q. */
    int32_t causal;
    int32_t n_past;
    /* Device array [B] of valid key counts per batch entry (keys >= kv_len[b] are masked); NULL = Lk.
     * Read on the device at run time, so a captured launch follows a growing cache. */
    const int32_t* kv_len;
    /* If non-zero the relative-position bias is NOT rounded to F16 (diagnostic; the reference rounds). */
    int32_t relpos_bias_f32;
    /* Index lists instead of a dense membership mask.  Replaces, for the decoder self-attention over whisper's
     * unified cell pool, the F16 mask that src/crispasr.cpp:3467-3499 fills (cell i visible to token j iff the cell
     * carries j's sequence id and cell.pos <= pos_j) and with it the scan of every pooled cell by every beam:
     * kv_index is a device array [B][kv_index_stride]; logical key i of batch entry b is row kv_index[b][i] of
     * K and V (rows of batch entry b / (B/Bk), so the beams of one segment are batch entries that share its pool),
     * for i < kv_len[b] (kv_len is then required; kv_len[b] <= kv_index_stride).  Entries are clamped to
     * [0, Lk).  Two ways to use it: one list per beam (every beam a batch entry with Tq = 1, no mask:
     * b200_beam_cells_to_index), or one list per segment holding the UNION of the cells its beams can see, the beams
     * as the Tq query rows, and a compact F16 `mask` [kv_index_stride, Tq] over the list's entries that says which
     * beam sees which entry (b200_beam_cells_to_union) - every live cell is then read once for all beams.  With
     * kv_index the mask has one value per list entry (mask.ne[0] == kv_index_stride) and 16-byte aligned rows.
     * Only for launches that b200_fattn_plan maps to B200_KERNEL_DECODE_SPLIT, without the causal flag, softcap or
     * ALiBi; the masked form needs an F16 pool with 16-byte aligned rows; otherwise B200_E_UNSUPPORTED. */
    int32_t kv_index_stride;
    const int32_t* kv_index;
    /* Device array [B] of valid query rows per batch entry (rows >= q_len[b] are not computed; their dst rows are
     * zero-filled); NULL = Tq.  With kv_len this is the per-unit (q_len, kv_len) table of a batched launch over
     * independent units of different lengths (b200_batch_*): no padding mask, no work for the padding. */
    const int32_t* q_len;
} b200_fattn_ext;

/* Error codes (negative). 0 is success. Nothing in this library aborts or throws. */
enum {
    B200_OK = 0,
    B200_E_NULL = -1,        /* a required pointer is NULL */
    B200_E_TYPE = -2,        /* operand type not supported by the op contract */
    B200_E_SHAPE = -3,       /* shapes disagree (head dims, Lk, GQA ratio, mask dims, dst dims) */
    B200_E_STRIDE = -4,      /* nb[0] is not the element size, or a stride is not a multiple of it */
    B200_E_ALIGN = -5,       /* base pointer alignment below what the element type needs */
    B200_E_UNSUPPORTED = -6, /* legal ggml op that this library has no kernel for (e.g. head_dim 160) */
    B200_E_WORKSPACE = -7,   /* workspace NULL or smaller than b200_fattn_workspace_bytes */
    B200_E_CUDA = -8,        /* a CUDA runtime/driver call failed; see b200_last_cuda_error */
    B200_E_NO_DEVICE = -9,   /* no CUDA device, or the device is not compute capability 10.x */
    B200_E_LIMIT = -10,      /* a size exceeds a documented fixed limit of the entry point */
    B200_E_STATE = -11,      /* object used in the wrong state (scheduler/allocator) */
    B200_E_DEVICE_WAIT = -12 /* a bounded device-side wait ran out; reported via the status word */
};

/* Which kernel family a launch used (b200_fattn_plan / b200_last_kernel). */
enum {
    B200_KERNEL_NONE = 0,
    B200_KERNEL_TILE_MMA = 1,   /* general tiled kernel, mma.sync tensor path, every operand form */
    B200_KERNEL_DECODE_SPLIT = 2, /* split-KV streaming kernel for <=16 query rows per KV head + LSE merge */
    B200_KERNEL_PREFILL_TC5 = 3 /* TMA + tcgen05.mma + TMEM prefill kernel (F16 K/V) */
};

/* Force a kernel family for A/B tests (B200_KERNEL_NONE restores automatic choice). Process-wide: an atomic that
 * every plan reads once.  Do not change it between the b200_fattn_workspace_bytes and b200_fattn_launch calls
 * of one operator call (the launch would find its workspace too small and return B200_E_WORKSPACE). */
B200_API int b200_set_kernel_override(int kernel);
/* Force the split count of the split-KV decode kernel (1..64, clamped to the number of 64-key tiles; 0 restores
 * the automatic choice). For A/B tests and tuning. Process-wide atomic, same rule as above. */
B200_API int b200_set_decode_splits(int n_splits);

B200_API const char* b200_strerror(int code);
B200_API const char* b200_version(void);
/* Text of the last CUDA error seen by the calling thread ("" if none). */
B200_API const char* b200_last_cuda_error(void);

/*
 * b200_fattn_supports — replaces ggml_backend_dev_supports_op(dev, op) for
 * GGML_OP_FLASH_ATTN_EXT (asked by the scheduler at src/crispasr.cpp:1977).
 * Returns 1 if b200_fattn_launch will accept these operands, 0 if not; never
 * touches the device. `why` (may be NULL) receives the negative code on refusal.
 */
B200_API int b200_fattn_supports(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                 const b200_tensor* mask, const b200_tensor* dst,
                                 const b200_fattn_params* params, const b200_fattn_ext* ext, int* why);

/*
 * b200_fattn_plan — which kernel would run and how many KV splits it would use.
 * Pure function of the descriptors. Returns 0 or a negative code.
 */
B200_API int b200_fattn_plan(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                             const b200_tensor* mask, const b200_tensor* dst,
                             const b200_fattn_params* params, const b200_fattn_ext* ext,
                             int* kernel, int* n_splits);

/*
 * b200_fattn_workspace_bytes — scratch the launch needs (split-KV partial O/m/l, or the F16
 * copies of K/V/R that the conversion pre-pass of the tensor-core prefill writes).
 * Mirrors ggml's per-op work buffer sizing (the reference sizes it inside
 * ggml_backend_sched_alloc_graph, src/voxtral.cpp:1196-1198). May return 0 bytes: one split,
 * or splits that merge inside thread-block clusters (small decode batches: at most eight splits of a resident grid).
 */
B200_API int b200_fattn_workspace_bytes(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                        const b200_tensor* mask, const b200_tensor* dst,
                                        const b200_fattn_params* params, const b200_fattn_ext* ext,
                                        size_t* bytes);

/*
 * b200_fattn_launch — replaces the backend's GGML_OP_FLASH_ATTN_EXT compute
 * (reached through ggml_backend_sched_graph_compute, src/crispasr.cpp:273,
 * src/parakeet.cpp:997, src/voxtral.cpp:1209).  Enqueues the kernels on
 * `cuda_stream` (a cudaStream_t, NULL = legacy default stream) of the CURRENT
 * device and returns without synchronising.  Allocates nothing; `workspace`
 * must be a device buffer of at least b200_fattn_workspace_bytes (256-byte
 * aligned) and may be NULL when that size is 0.  Returns 0 or a negative code.
 */
B200_API int b200_fattn_launch(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                               const b200_tensor* mask, const b200_tensor* dst,
                               const b200_fattn_params* params, const b200_fattn_ext* ext,
                               void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * b200_fattn_forward_host — the same operator for callers that hold HOST
 * buffers, i.e. the ggml_backend_tensor_set -> graph_compute -> tensor_get
 * round trip of src/voxtral.cpp:1196-1223 in one call.  All `data` pointers
 * (and ext->kv_len) are host pointers; operands are staged through a per-thread
 * device arena that grows on demand, copied in, computed and copied back, and
 * the call returns after the result is in `dst->data`.  Batch entries (ne[3]) are
 * independent, so the call is pipelined over up to four chunks of the batch on two
 * streams (environment variable B200_HOST_CHUNKS = 1..16 changes the depth): the
 * upload of one chunk overlaps the kernel and the download of the previous one.
 * Pinned host buffers are needed for that overlap to happen.
 */
B200_API int b200_fattn_forward_host(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                     const b200_tensor* mask, const b200_tensor* dst,
                                     const b200_fattn_params* params, const b200_fattn_ext* ext);
/* Frees the calling thread's staging arena of b200_fattn_forward_host. */
B200_API void b200_host_arena_release(void);

/*
 * b200_fattn_launch_static — no counterpart in the reference (ggml always sizes a work buffer for the
 * op): the split-KV decode launch for callers that cannot allocate device memory — code running inside a
 * real-time audio callback, embedders with a fixed, audited memory budget, hosts that pass a stream but
 * own no allocator.  Same operands and semantics as b200_fattn_launch, no workspace argument: the split
 * partials live in a fixed array inside the loaded module (b200_fattn_static_scratch_bytes() = 8 MiB, held
 * on every GPU that loads the library until the process exits).  The call itself allocates and frees
 * nothing.  Accepts only operand forms that b200_fattn_plan maps to B200_KERNEL_DECODE_SPLIT
 * (else B200_E_UNSUPPORTED) whose b200_fattn_workspace_bytes fits the array (else B200_E_LIMIT).
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current); make that first call before starting any stream capture.  Every call shares the one
 * array and finds the previous call's contents in it (the kernels overwrite all they read, nothing
 * needs clearing); calls that may overlap on the GPU race on it, so keep them on one stream.
 */
B200_API int b200_fattn_launch_static(const b200_tensor* q, const b200_tensor* k, const b200_tensor* v,
                                      const b200_tensor* mask, const b200_tensor* dst,
                                      const b200_fattn_params* params, const b200_fattn_ext* ext,
                                      void* cuda_stream);
B200_API size_t b200_fattn_static_scratch_bytes(void);

/*
 * b200_device_status — every wait inside the kernels (on an mbarrier that a TMA copy or a tensor-core
 * commit completes) is bounded; a CTA whose wait runs out stops, releases its tensor memory and sets a
 * status word on the device.  This reads that word on the current device: B200_OK, or
 * B200_E_DEVICE_WAIT if any launch since load hit the limit (its output is then undefined).  Call it
 * after synchronising the stream(s) of interest.  No reference counterpart (ggml aborts instead).
 */
B200_API int b200_device_status(void);
/* Clears the status word of the current device (it is sticky otherwise).  Call with no launch in flight. */
B200_API int b200_device_status_reset(void);
/*
 * b200_test_bounded_wait — test hook for the failure path above, in the only form that is safe on a shared
 * GPU: launches a one-warp kernel that waits on an mbarrier which nothing ever completes, with a limit of
 * `polls` polls (1 .. 2^20).  The wait runs out, the kernel sets the status word and returns normally; the
 * context stays usable.  After synchronising, b200_device_status must report B200_E_DEVICE_WAIT.
 */
B200_API int b200_test_bounded_wait(int polls, void* cuda_stream);
/* Measurement hook: enqueues one empty one-warp kernel.  A stream (or captured graph) of these gives the
 * launch-latency floor per layer that the short decode launches are compared with. */
B200_API int b200_test_empty_launch(void* cuda_stream);

/*
 * Per-launch tracing, off by default.  The reference's counterparts are its debug taps and per-op timing buckets
 * (src/core/attention.h:786-806 dumps tensors around the FA call; src/qwen3_tts.cpp:196-273 accumulates wall time
 * per op class).  b200_trace_enable(n > 0) creates a ring of n CUDA event pairs on the current device; from then on
 * every b200_fattn_launch / b200_fattn_launch_static / chunk of b200_fattn_forward_host on that device is wrapped
 * in an NVTX range named after its kernel family and bracketed by an event pair on its stream.  b200_trace_read
 * waits for the recorded launches and returns their records oldest first (a full ring overwrites its oldest
 * record).  Launches made while the stream is being captured into a CUDA graph are not traced.
 * b200_trace_enable(0) turns tracing off and frees the events.  Tracing serialises concurrent launches on a lock.
 */
typedef struct b200_trace_record {
    int32_t kernel;   /* B200_KERNEL_* */
    int32_t n_splits;
    int32_t head_dim, q_len, kv_len, n_heads, n_kv_heads, n_batch;
    int32_t kv_type;  /* b200_type */
    float ms;         /* device time between the two events: all kernels of the launch (pre-pass, merge) included */
} b200_trace_record;
B200_API int b200_trace_enable(int capacity);
B200_API int b200_trace_read(b200_trace_record* out, int max_records, int* n_out);

/* The kernel family the calling thread's most recent successful launch used. */
B200_API int b200_last_kernel(void);

/* ------------------------------------------------------------------------------------------
 * KV-cache slabs.  Replaces the cache tensors of core_attn (layout (hd, max_ctx, n_kv, n_layers),
 * src/core/attention.h:593-595) and whisper's kv_self / kv_cross buffers
 * (src/crispasr.cpp:1471-1516): one contiguous, 1024-byte aligned slab per layer and per K/V,
 * head-major rows, so that every (layer, kv-head) row range is a single flat byte range that
 * TMA boxes (F16) or 128-bit streaming loads (Q8_0) can cover.
 * ------------------------------------------------------------------------------------------ */
typedef struct b200_kv_cache b200_kv_cache; /* opaque */

typedef struct b200_kv_config {
    int32_t type;     /* B200_TYPE_F16 or B200_TYPE_Q8_0 */
    int32_t head_dim; /* 64 or 128 (multiple of 32) */
    int32_t n_kv_heads;
    int32_t n_layers;
    int32_t max_ctx;  /* rows per (layer, head, stream) */
    int32_t n_streams; /* independent sequences / beams sharing the geometry (ne[3]) */
} b200_kv_config;

/* Allocates 2 * n_layers slabs on the current device. Returns 0 or a negative code. */
B200_API int b200_kv_create(const b200_kv_config* cfg, b200_kv_cache** out);
B200_API void b200_kv_destroy(b200_kv_cache* kv);
B200_API size_t b200_kv_bytes(const b200_kv_cache* kv);
/* Fills K and V descriptors viewing rows [0, n_rows) of `layer` for all heads and streams
 * (the view_3d of src/core/attention.h:887-895). */
B200_API int b200_kv_view(const b200_kv_cache* kv, int layer, int64_t n_rows, b200_tensor* k, b200_tensor* v);
/*
 * b200_kv_append — replaces core_attn::kv_cache_write (src/core/attention.h:342-378) and the
 * write branch at :840-867 (ggml_cpy for F16, ggml_set_rows for quantised caches): converts
 * F32 rows k_new/v_new [hd, n_new, n_kv_heads, n_streams] (device, generic strides) to the cache
 * type and stores them at rows pos[s] .. pos[s]+n_new-1 of each stream s (`pos` is a device
 * array [n_streams], or NULL meaning `pos0` for all).  Asynchronous on `cuda_stream`.
 */
B200_API int b200_kv_append(b200_kv_cache* kv, int layer, const b200_tensor* k_new, const b200_tensor* v_new,
                            const int32_t* pos, int32_t pos0, void* cuda_stream);

/*
 * b200_kv_copy_stream — replaces core_attn::kv_snapshot_pool save/restore (src/core/attention.h:198-320), the
 * device-to-device blits that branched beam search uses to fork a hypothesis: copies rows [0, n_rows) of every
 * layer and head from stream `src_stream` to stream `dst_stream` of the same cache (one 2-D copy per slab),
 * asynchronously on `cuda_stream`.  Beams that only share a prefix need no copy at all: they can read the same
 * stream with different kv_len / masks.
 */
B200_API int b200_kv_copy_stream(b200_kv_cache* kv, int dst_stream, int src_stream, int64_t n_rows, void* cuda_stream);

/*
 * b200_beam_cells_to_index — host helper for ext->kv_index: turns whisper's cell pool
 * (src/crispasr.cpp:1194-1217: per cell a position and a set of sequence ids; find_slot :1517-1564 hands cells
 * out, beam reshuffles are seq-id edits :8193-8235) into one index list per token.  cell_pos[n_cells] and
 * cell_seq_bits[n_cells] (bit s set = the cell carries sequence id s; an empty cell has no bit set) describe the
 * pool; token j belongs to sequence tok_seq[j] at position tok_pos[j] and sees exactly the cells
 * {i : bit tok_seq[j] of cell_seq_bits[i] set and cell_pos[i] <= tok_pos[j]} — the complement of the reference's
 * -inf rule (:3480-3488).  index_out is [n_tokens][stride] (host), filled in ascending cell order; len_out[j]
 * receives the count.  Returns B200_E_LIMIT if a list does not fit `stride`.  Pure host function.
 */
B200_API int b200_beam_cells_to_index(const int32_t* cell_pos, const uint32_t* cell_seq_bits, int n_cells,
                                      const int32_t* tok_seq, const int32_t* tok_pos, int n_tokens,
                                      int32_t* index_out, int stride, int32_t* len_out);
/* The shared form: ONE list (index_out[stride], ascending cell order, *len_out entries) of the cells that at least one
 * of the n_tokens tokens can see, and the compact mask mask_out[n_tokens][stride] over its entries (F16 bits: 0 where
 * the reference's mask has 0, -inf where it has -inf or beyond the list).  The step then reads every live cell once
 * for all beams instead of scanning the whole pool (reference) or once per beam (b200_beam_cells_to_index). */
B200_API int b200_beam_cells_to_union(const int32_t* cell_pos, const uint32_t* cell_seq_bits, int n_cells,
                                      const int32_t* tok_seq, const int32_t* tok_pos, int n_tokens,
                                      int32_t* index_out, int stride, int32_t* len_out, uint16_t* mask_out);

/*
 * b200_mask_classify — host helper for adapters whose runtime fills its F16 mask on the host before uploading it
 * (the causal prefill mask of src/voxtral.cpp:1187-1194, the bucket padding mask of src/canary_ctc.cpp:370-382): says
 * whether the mask [Lk, Tq] (row_stride elements between query rows) is one of the shapes the operator takes as a
 * parameter instead of as a tensor.  An explicit mask costs the kernels a load, a conversion and a fold per score;
 * the parameters cost nothing per element and skip dead tiles.
 *   B200_MASK_GENERAL  pass the mask as it is (any value other than 0 / -0 / -inf, or any other pattern)
 *   B200_MASK_NONE     every entry is 0: pass no mask
 *   B200_MASK_CAUSAL   entry (query i, key j) is 0 for j <= n_past + i and -inf beyond: pass ext.causal = 1 and
 *                      ext.n_past = *n_past (no mask)
 *   B200_MASK_TAIL     keys >= *kv_len are -inf for every query row, the rest 0: pass ext.kv_len (no mask)
 * Returns B200_OK or an argument error.
 */
#define B200_MASK_GENERAL 0
#define B200_MASK_NONE 1
#define B200_MASK_CAUSAL 2
#define B200_MASK_TAIL 3
B200_API int b200_mask_classify(const uint16_t* mask, int Lk, int Tq, int64_t row_stride, int* kind, int* n_past,
                                int* kv_len);

/* ------------------------------------------------------------------------------------------
 * Relative-position table of the FastConformer attention block.  Replaces make_pos_enc
 * (src/core/fastconformer.h:118-130), its upload, and R = MUL_MAT(attn_pos_w, pos_enc) with the
 * reshape/permute that follows (:843, :851): R depends on the layer's weight and on T only, so it is built
 * once per (layer, T) on the device, in the F16 [hd, 2T-1, H] layout that ext->r of the fused attention
 * takes, and reused for every utterance of that length bucket.
 * ------------------------------------------------------------------------------------------ */
/* Builds R for one weight: attn_pos_w is the device tensor [d_in, d_out] (ggml order: ne[0] = input
 * feature, contiguous) F32 or F16 with d_in == d_out == n_heads * hd.  Writes (2T-1) * d F16 values,
 * head-major ([hd, 2T-1, H] contiguous), to r_out (device, 16-byte aligned, r_bytes >= that).  Asynchronous. */
B200_API int b200_relpos_table(const b200_tensor* attn_pos_w, int n_heads, int T, void* r_out, size_t r_bytes,
                               void* cuda_stream);
typedef struct b200_relpos_cache b200_relpos_cache; /* opaque; tables live on the device current at creation */
B200_API int b200_relpos_cache_create(int n_layers, int max_entries_per_layer, b200_relpos_cache** out);
B200_API void b200_relpos_cache_destroy(b200_relpos_cache* c);
B200_API size_t b200_relpos_cache_bytes(const b200_relpos_cache* c);
/* Fills `r` with the descriptor of the table for (layer, T, this weight pointer), building it on a miss (one
 * device allocation and one launch on `cuda_stream`; a hit does no device work).  Each layer keeps at most
 * max_entries_per_layer tables and evicts the least recently used one.  Use the table on the stream it was
 * built on, or order the streams yourself.  `was_hit` may be NULL. */
B200_API int b200_relpos_cache_get(b200_relpos_cache* c, int layer, int T, const b200_tensor* attn_pos_w, int n_heads,
                                   void* cuda_stream, b200_tensor* r, int* was_hit);

/* ------------------------------------------------------------------------------------------
 * Segment scheduler.  Replaces the `-p N` worker instances with an atomic next-slice cursor
 * (examples/cli/crispasr_run.cpp:1882-1930) and whisper_full_parallel (src/crispasr.cpp:8755-8880)
 * for the attention path: independent units (audio segments, beams groups, streams, utterances)
 * are handed to one host worker thread per GPU; there is no inter-GPU exchange.
 * ------------------------------------------------------------------------------------------ */
typedef struct b200_sched b200_sched; /* opaque */

/* Called on a worker thread with its device current: process unit `unit` on `cuda_stream`.
 * Return 0, or non-zero to report failure (the unit is retried once on another worker, then
 * recorded as failed — the deferred-retry rule of crispasr_run.cpp:1819-1844). */
typedef int (*b200_unit_fn)(void* user, int device, int unit, void* cuda_stream);

/* devices == NULL means devices 0..n_devices-1. n_devices == 0 builds a host-only scheduler
 * (workers run without touching CUDA; used by CPU tests) with `n_host_workers` threads. */
B200_API int b200_sched_create(const int* devices, int n_devices, int n_host_workers, b200_sched** out);
B200_API void b200_sched_destroy(b200_sched* s);
/* Runs units [0, n_units): a contiguous range per worker first, then stealing from the shared
 * cursor.  Blocks until every unit has finished or failed twice.  `unit_device` (may be NULL,
 * else [n_units]) receives the worker index that completed each unit, -1 for a failed unit.
 * Returns the number of failed units (>= 0) or a negative code. */
B200_API int b200_sched_run(b200_sched* s, int n_units, b200_unit_fn fn, void* user, int* unit_device);
/*
 * b200_sched_run_batched — the same scheduler for callers that batch: the callback receives a RUN of up to
 * `max_batch` consecutive units (never crossing the border of a worker's static share) and processes it as one
 * batch, i.e. one kernel launch per layer over all units of the run (units concatenated on ne[3], ragged lengths
 * through ext->kv_len / ext->q_len; see b200_batch_* below).  This is what lets several slices of
 * CrispasrBackend::encode_slice / decode_slice (examples/cli/crispasr_backend.h:181-230) share a launch per GPU
 * instead of one launch each.  max_batch >= the share size hands each worker its whole share at once;
 * `steal` = 0 keeps every unit on the worker that owns it statically (resident per-device inputs), non-zero lets
 * idle workers take runs from the others.  A run whose callback fails is retried once, whole, on another worker.
 * Every worker synchronises its stream before the call returns.  Returns the number of failed units.
 */
typedef int (*b200_batch_fn)(void* user, int device, int first_unit, int n_units, void* cuda_stream);
B200_API int b200_sched_run_batched(b200_sched* s, int n_units, int max_batch, int steal, b200_batch_fn fn, void* user,
                                    int* unit_device);
/* Static part of the partition: first unit and count owned by worker `w` of `n_workers`. */
B200_API void b200_sched_partition(int n_units, int n_workers, int w, int* first, int* count);

/* ------------------------------------------------------------------------------------------
 * Slice batcher.  The reference runs one slice per operator call (CrispasrBackend::encode_slice /
 * decode_slice, examples/cli/crispasr_backend.h:181-230; the encode/decode pipeline of
 * examples/cli/crispasr_run.cpp:1765-1881 holds at most two slices) and pads different lengths to a bucket
 * with a -inf mask (src/canary_ctc.cpp:370-382).  Here the units of one GPU share launches: they are
 * concatenated on ne[3] and a per-unit (q_len, kv_len) table (ext->q_len / ext->kv_len) replaces the padding
 * mask, so padding costs no arithmetic and no memory traffic.
 * ------------------------------------------------------------------------------------------ */
/* Orders `n_units` pending units by length (longest first) and cuts them into launches of at most `max_units`
 * in which no unit's kv_len (q_len) is below (1 - max_pad) of the launch's longest: the padded operand buffers
 * of a launch are then at most 1 / (1 - max_pad) times the sum of its units.  order[n_units] receives unit
 * indices in launch order, group_end[g] the end (exclusive) of launch g in `order` (n_units entries suffice),
 * n_groups the launch count.  Pure host function. */
B200_API int b200_batch_pack(const int32_t* q_len, const int32_t* kv_len, int n_units, int max_units, float max_pad,
                             int32_t* order, int32_t* group_end, int* n_groups);
/* Slot table of a resident batch on the current device (decode streams join and leave, caches grow by a row per
 * step).  Slot s is batch entry s of the launch: ne[3] of Q/K/V/dst = the span returned by b200_batch_span. */
typedef struct b200_batch b200_batch; /* opaque */
B200_API int b200_batch_create(int capacity, b200_batch** out);
B200_API void b200_batch_destroy(b200_batch* b);
/* Places unit `unit_id` (>= 0) in the lowest free slot; returns the slot or B200_E_LIMIT. */
B200_API int b200_batch_add(b200_batch* b, int unit_id, int q_len, int kv_len);
B200_API int b200_batch_set(b200_batch* b, int slot, int q_len, int kv_len);
/* kv_len += kv_delta for every occupied slot: one decode step of all resident streams. */
B200_API int b200_batch_advance(b200_batch* b, int kv_delta);
/* Frees a slot; inside the span it stays in the launch with zero rows and zero keys (no work, zero output). */
B200_API int b200_batch_remove(b200_batch* b, int slot);
/* Span (highest occupied slot + 1), occupied slots, and the longest q_len / kv_len among them (any may be NULL). */
B200_API int b200_batch_span(const b200_batch* b, int* n_slots, int* n_active, int* max_q_len, int* max_kv_len);
B200_API int b200_batch_unit(const b200_batch* b, int slot); /* unit id, or -1 for a free slot */
B200_API int b200_batch_lengths(const b200_batch* b, int slot, int* q_len, int* kv_len);
/* Device arrays [capacity] for ext->q_len and ext->kv_len; uploads the tables with one asynchronous copy on
 * `cuda_stream` if they changed since the last call.  Edit the table again only after work enqueued behind that
 * copy no longer needs the old values in the pinned source (i.e. after the copy itself has run). */
B200_API int b200_batch_tables(b200_batch* b, void* cuda_stream, const int32_t** q_len_dev, const int32_t** kv_len_dev);

#ifdef __cplusplus
}
#endif
#endif /* B200_FATTN_H */
