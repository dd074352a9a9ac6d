/*
 * tq_b200.h — C ABI of the B200 (sm_100a) TurboQuant packed-KV library.
 *
 * Every entry point is extern "C", takes plain pointers and sizes, returns an
 * int32 status (0 = ok, negative = error, see TQ_ERR_*) and never throws.  The
 * caller owns all device buffers and passes the CUDA stream to launch on; kernels
 * are asynchronous on that stream.  The compute entry points (tq_pack, tq_decode_*,
 * tq_dequant, tq_key_norm_sum, tq_gather_wait) allocate nothing.  The calls that
 * allocate are: tq_ctx_create / tq_ctx_destroy (the device copy of the codec
 * tables), tq_peer_buffer_create / tq_peer_buffer_destroy (device memory that other
 * processes can map), and - only while tq_profile_enable is on - the decode calls,
 * which then create the CUDA events they record.  A tq_ctx is bound to one device
 * and may be used from one host thread at a time; one process may hold contexts on
 * several devices.
 *
 * The functions replace these pieces of the reference (paths relative to the
 * reference project root):
 *
 *   tq_ctx_create       PackedMSELayer.lazy_initialization / _build_codebook_tensors
 *                       src/turboquant/runtime/packed_qmse_cache.py:226-283
 *   tq_pack             PackedMSELayer.initialize_from_dense, _encode_group,
 *                       _encode_keys_qjl_group, and the quantize_decode=True branch of
 *                       _update_lazy + PackedTensorMSE.append / PackedQJL.append
 *                       src/turboquant/runtime/packed_qmse_cache.py:285-310,332-402,626-668,81-92,135-140
 *   tq_decode_attn      fused_attention + _tile_attention_kernel + cross-tile reduce +
 *                       dense-tail merge + un-rotation
 *                       src/turboquant/runtime/triton_kernels.py:84-198,238-368
 *                       (and, for batch > 1, chunked_turboquant_attention,
 *                       src/turboquant/runtime/attention.py:215-304)
 *   tq_dequant          _decode_group / _decode_keys_qjl_group / triton_decode_group
 *                       src/turboquant/runtime/packed_qmse_cache.py:312-330,404-435
 *                       src/turboquant/runtime/triton_kernels.py:36-55,227-236
 *   tq_key_norm_mean    the per-layer mean key norm of build_packed_mse_cache
 *                       src/turboquant/runtime/packed_qmse_cache.py:918-920
 */
#ifndef TQ_B200_H
#define TQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_OK 0
#define TQ_ERR_ARG (-1)          /* null pointer, negative size, misaligned buffer */
#define TQ_ERR_UNSUPPORTED (-2)  /* head_dim != 128, bits outside 2..4, too many query heads per KV head */
#define TQ_ERR_CUDA (-3)         /* a CUDA runtime call failed; see tq_last_cuda_error */
#define TQ_ERR_WORKSPACE (-4)    /* workspace smaller than tq_decode_workspace_bytes */

#define TQ_DTYPE_F32 0
#define TQ_DTYPE_F16 1
#define TQ_DTYPE_BF16 2

#define TQ_HEAD_DIM 128
#define TQ_MAX_GROUPS 8 /* query heads per KV head */

typedef struct tq_ctx tq_ctx;
typedef struct tq_gather_desc tq_gather_desc; /* KV-head sharding, defined below */
typedef void *tq_stream; /* a cudaStream_t */

/* Codec set-up, all pointers to HOST memory, row-major float32.
 *   rot_k, rot_v : [128][128] orthogonal rotations R; encode computes u @ R^T.
 *                  For Q_mse (use_qjl = 0) pass the same matrix for both.
 *   qjl          : [128][128] Gaussian projection S (NULL when use_qjl = 0).
 *   centers_k/v  : 2^key_bits / 2^bits Lloyd-Max centres; bounds_k/v one fewer.
 *                  key_bits = bits - 1 when use_qjl, else bits. */
typedef struct {
    int32_t head_dim; /* must be 128 */
    int32_t bits;     /* 2, 3 or 4: total bits per coordinate */
    int32_t use_qjl;  /* 1 = Q_prod keys (bits-1 Lloyd-Max + 1-bit QJL residual sketch) */
    const float *rot_k;
    const float *rot_v;
    const float *qjl;
    const float *centers_k;
    const float *bounds_k;
    const float *centers_v;
    const float *bounds_v;
} tq_codec_desc;

/* The packed cache of one layer: six device streams, token axis innermost but one.
 * Row (b, h) of a stream starts at element offset (b*stride_b + h*stride_h) tokens;
 * a token is key_bits*16 bytes of k_codes, bits*16 bytes of v_codes, 16 bytes of
 * k_signs, one fp16 for each norm stream.  With stride_h == capacity == n_tokens and
 * stride_b == kv_heads*capacity, the first n_tokens of every row are byte-for-byte the
 * reference's PackedTensorMSE.packed_indices / norms and PackedQJL tensors.
 * All stream pointers must be 16-byte aligned and stride_b, stride_h multiples of 8. */
typedef struct {
    uint8_t *k_codes;
    uint16_t *k_norms;  /* fp16 bit patterns */
    uint8_t *k_signs;   /* NULL unless use_qjl */
    uint16_t *k_rnorms; /* NULL unless use_qjl */
    uint8_t *v_codes;
    uint16_t *v_norms;
    int32_t batch;
    int32_t kv_heads;
    int32_t capacity; /* tokens allocated per (b, h) row */
    int64_t stride_b; /* in tokens */
    int64_t stride_h; /* in tokens */
    const int32_t *seq_start; /* optional DEVICE array [batch]: the decode calls attend tokens
                                 [seq_start[b], seq_len) of batch entry b instead of [0, seq_len)
                                 - a left-padded batch, the only mask shape a decoder-only generation
                                 loop produces; NULL = every row from token 0.  What the reference's
                                 chunked path gets by adding the attention-mask slice to its logits
                                 (src/turboquant/runtime/attention.py:253-255,278-283). */
} tq_cache_desc;

/* A dense [batch, heads, tokens, 128] tensor with arbitrary outer strides (in elements);
 * the last axis is contiguous. */
typedef struct {
    const void *data;
    int32_t dtype; /* TQ_DTYPE_* */
    int64_t stride_b;
    int64_t stride_h;
    int64_t stride_t;
} tq_dense_desc;

int32_t tq_abi_version(void);
const char *tq_last_cuda_error(void);

/* Allocates the device copy of the codec tables on `device` (the only allocating calls). */
int32_t tq_ctx_create(tq_ctx **out, int32_t device, const tq_codec_desc *codec);
int32_t tq_ctx_destroy(tq_ctx *ctx);

/* Quantise n_tokens new tokens of K and V and write them at token positions
 * [pos0, pos0 + n_tokens) of every (b, h) row of the cache: prefill packing
 * (pos0 = 0) and the O(1) in-place append of a decoded token (n_tokens = 1). */
int32_t tq_pack(tq_ctx *ctx, const tq_dense_desc *k, const tq_dense_desc *v, int32_t n_tokens,
                const tq_cache_desc *cache, int32_t pos0, tq_stream stream);

/* Bytes of scratch tq_decode_attn needs for this shape. */
size_t tq_decode_workspace_bytes(int32_t batch, int32_t q_heads, int32_t n_splits);
/* A split count that fills the GPU for this shape (>= 1). */
int32_t tq_decode_suggest_splits(tq_ctx *ctx, int32_t batch, int32_t kv_heads, int32_t seq_len);

/* One decode step of attention straight from the packed cache.
 *   q     : [batch, q_heads, 128] contiguous, dtype q_dtype (one query token per sequence)
 *   out   : [batch, q_heads, 128] contiguous, same dtype (== [batch, 1, q_heads, 128])
 *   seq_len tokens of every cache row are attended; softmax scale is 1/sqrt(128).
 *   tail_k/tail_v (optional, may be NULL): n_tail un-quantised tokens
 *   [batch, kv_heads, n_tail, 128] attended after the packed ones (quantize_decode = False).
 * fp32 queries take an fp32-exact CUDA-core kernel; fp16/bf16 queries take the
 * tensor-core kernel. */
int32_t tq_decode_attn(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                       const tq_cache_desc *cache, int32_t seq_len, const tq_dense_desc *tail_k,
                       const tq_dense_desc *tail_v, int32_t n_tail, int32_t n_splits,
                       void *workspace, size_t workspace_bytes, void *out, tq_stream stream);

/* tq_decode_attn for fp16 / bf16 queries without a dense tail, with the result written
 * UNROUNDED as float32 [batch, q_heads, 128]: the same kernels, only the final cast to the query
 * dtype is left out.  For callers that go on in fp32 and for measuring the kernels' own error
 * apart from the rounding of the output (no reference counterpart: the reference's fused path
 * always casts to the query dtype, src/turboquant/runtime/triton_kernels.py:368). */
int32_t tq_decode_attn_f32out(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                              const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits,
                              void *workspace, size_t workspace_bytes, float *out, tq_stream stream);

/* One whole decode step for callers whose tensors live in HOST memory (pinned for the copies
 * to be asynchronous): copy the query and the new token's key / value to the device, append
 * the token at position `pos` of every cache row, attend over pos + 1 tokens, copy the
 * output back.  Replaces, per layer and step, the reference's PackedMSELayer.update +
 * turboquant_attention_forward (src/turboquant/runtime/packed_qmse_cache.py:600-679,
 * src/turboquant/runtime/attention.py:28-72).  q_host / out_host: [batch, q_heads, 128];
 * k_host / v_host: [batch, kv_heads, 128]; all contiguous, of `dtype`.  The work is queued on
 * `stream`; out_host is valid once the stream has been synchronised. */
size_t tq_decode_step_workspace_bytes(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t n_splits);
int32_t tq_decode_step_host(tq_ctx *ctx, const void *q_host, const void *k_host, const void *v_host,
                            int32_t dtype, int32_t q_heads, const tq_cache_desc *cache, int32_t pos,
                            int32_t n_splits, void *workspace, size_t workspace_bytes, void *out_host,
                            tq_stream stream);

/* The same step with every operand in DEVICE memory and the cache length read from device
 * memory when the kernels run, so that one recorded launch sequence (a CUDA graph of a whole
 * model's decode step) can be replayed for every token: append k_new / v_new
 * [batch, kv_heads, 128] at token *pos_dev of every row, attend with q [batch, q_heads, 128]
 * over *pos_dev + 1 tokens, write out [batch, q_heads, 128].  The caller advances *pos_dev
 * between steps (in stream order).  An append past the cache's capacity is dropped and
 * reported by tq_device_status (4).  16-bit dtypes and at most 8 query heads per KV head;
 * other shapes return TQ_ERR_UNSUPPORTED.  Replaces the per-token PackedMSELayer.update +
 * turboquant_attention_forward pair and the host bookkeeping between them
 * (src/turboquant/runtime/packed_qmse_cache.py:600-679, src/turboquant/runtime/attention.py:28-72,
 * src/turboquant/runtime/generation.py:140-170).  Workspace: tq_decode_workspace_bytes.
 * With gather != NULL (KV-head sharding, see tq_gather_desc below; gather->seq_dev must be set)
 * the outputs of all ranks are exchanged by the combine kernel, the call also queues the wait,
 * and out receives the gathered [batch, q_heads_total, 128] output. */
int32_t tq_decode_step_dev(tq_ctx *ctx, const void *q, const void *k_new, const void *v_new, int32_t dtype,
                           int32_t q_heads, const tq_cache_desc *cache, const int32_t *pos_dev,
                           int32_t n_splits, void *workspace, size_t workspace_bytes, void *out,
                           const tq_gather_desc *gather, tq_stream stream);

/* Dequantise tokens [pos0, pos0 + n_tokens) of the keys (which = 0) or values (which = 1)
 * into a dense [batch, kv_heads, n_tokens, 128] tensor of dtype out->dtype. */
int32_t tq_dequant(tq_ctx *ctx, const tq_cache_desc *cache, int32_t which, int32_t pos0,
                   int32_t n_tokens, const tq_dense_desc *out, tq_stream stream);

/* Sum of the L2 norms of all key vectors of a dense tensor, accumulated into
 * *sum_out (a device float64 the caller zeroes); mean = sum / (batch*heads*tokens). */
int32_t tq_key_norm_sum(const tq_dense_desc *k, int32_t batch, int32_t heads, int32_t n_tokens,
                        double *sum_out, tq_stream stream);

/* ---- KV-head sharding over the GPUs of one box (no counterpart in the reference, which is
 * single-GPU).  Rank r serves kv_heads / world KV heads and their query heads; the only exchange
 * per decode step is the per-head attention outputs.  tq_decode_attn_gather fuses that exchange
 * into the combine kernel: every block stores its finished rows straight into the gathered-output
 * buffer of EVERY rank (plain stores to peer memory over NVLink) and then adds the number of rows
 * it stored to this rank's word in every rank's flag block, with a release reduction at system
 * scope (the waiting side reads the words with acquire loads).
 * tq_gather_wait (one small kernel, stream-ordered before the consumer of the gathered output)
 * waits - with a time limit, reporting through tq_device_status (5) instead of hanging - until
 * every rank's word has reached step * batch * (q_heads_total / world): all rows of the step are
 * in place.  The words only ever grow, so a descriptor serves steps 1, 2, 3, ... of ONE shape.
 *
 * Buffers come from tq_peer_buffer_create (device memory that other processes on the box can
 * map): exchange the 64-byte handles by any host-side means and map the peers' buffers with
 * tq_peer_buffer_open.  A rank needs: two gathered-output buffers (steps alternate between them,
 * so a fast rank never overwrites what a slow rank still reads) of batch * q_heads_total * 128
 * elements each, and one flag block of TQ_MAX_PEERS uint32 (zero-initialised); plus a local
 * zero-initialised uint32 counter. */
#define TQ_MAX_PEERS 8
struct tq_gather_desc {
    int32_t world, rank;
    int32_t q_heads_total;          /* query heads of the whole model (all ranks) */
    uint32_t seq;                   /* step sequence number: 1, 2, 3, ... (the same on all ranks); unused with seq_dev */
    void *out[TQ_MAX_PEERS];        /* out[r]: the first of rank r's two gathered-output buffers (as mapped here) */
    int64_t out_stride;             /* bytes from a rank's first buffer to its second; step s uses buffer s & 1 */
    uint32_t *flags[TQ_MAX_PEERS];  /* flags[r]: rank r's flag block (as mapped here); word [rank] counts OUR rows there */
    uint32_t *counter;              /* local scratch word, zero between calls (used by tq_gather_wait with seq_dev) */
    uint32_t *seq_dev;              /* optional local device word holding the LAST completed sequence number
                                       (zero-initialised): the step then takes its number from the device,
                                       tq_gather_wait advances it, and a recorded launch sequence can be replayed */
    int32_t out_local_only;         /* non-zero: the copy that tq_gather_wait / tq_decode_step_host_gather make for the
                                       caller (out_final / out_host) holds only THIS rank's heads
                                       [batch, q_heads_total / world, 128] instead of the whole gathered output; the
                                       gathered buffers themselves are always complete */
};

int32_t tq_peer_buffer_create(size_t bytes, void **dev_ptr, void *handle64_out);
int32_t tq_peer_buffer_open(const void *handle64, void **dev_ptr);
int32_t tq_peer_buffer_close(void *dev_ptr);
int32_t tq_peer_buffer_destroy(void *dev_ptr);

/* tq_decode_attn without a dense tail, for 16-bit queries, with the output rows
 * [batch, q_heads, 128] of this rank written at head offset rank * q_heads into every rank's
 * gathered buffer [batch, q_heads_total, 128]. */
int32_t tq_decode_attn_gather(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                              const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits,
                              void *workspace, size_t workspace_bytes, const tq_gather_desc *gather,
                              tq_stream stream);
/* tq_decode_step_host for a KV-head shard: q_host [batch, q_heads, 128] and k_host / v_host
 * [batch, kv_heads, 128] are this rank's heads, out_host receives the gathered output of all
 * ranks [batch, q_heads_total, 128] (or, with gather->out_local_only, this rank's heads only).  All four buffers must be page-locked host memory mapped
 * into the device's address space (or device memory); 16-bit dtypes only.  Queues the append,
 * the attention, the exchange and the wait. */
int32_t tq_decode_step_host_gather(tq_ctx *ctx, const void *q_host, const void *k_host, const void *v_host,
                                   int32_t dtype, int32_t q_heads, const tq_cache_desc *cache, int32_t pos,
                                   int32_t n_splits, void *workspace, size_t workspace_bytes,
                                   const tq_gather_desc *gather, void *out_host, tq_stream stream);
/* Stream-ordered wait for all ranks' flags of the step (see above).  With out_final != NULL the
 * gathered output [batch, q_heads_total, 128] is then copied from this rank's buffer of the step
 * into out_final (device memory), which is what a caller needs when the step number lives on the
 * device and it cannot know which of the two buffers was used. */
int32_t tq_gather_wait(tq_ctx *ctx, const tq_gather_desc *gather, int32_t batch, int32_t dtype, void *out_final,
                       tq_stream stream);

/* ---- Sequence split: more ranks than KV heads (no counterpart in the reference).  `parts` ranks
 * share a group of KV heads; rank r belongs to group r / parts and is part r % parts of it, holding
 * a disjoint part of the cached tokens of the group's heads (which tokens is up to the caller:
 * attention does not depend on their order).  Per step every rank calls tq_decode_attn_parts with
 * the group's query heads q [batch, q_heads, 128] (the same on every part of a group) and ITS
 * tokens: the kernels attend them and store the unfinished partial (max, sum, acc[128], fp32) of
 * every row into every rank's partial-exchange buffer - the two buffers of tq_gather_desc.out,
 * here of tq_parts_exchange_bytes(batch, q_heads_total, parts) bytes each, with
 * q_heads_total = q_heads * world / parts.  seq_len may be 0 (a part that holds no token yet).
 * tq_decode_parts_finish then waits (bounded, status 5) until the partials of all ranks are in,
 * merges the parts of every row, un-rotates and writes out [batch, q_heads_total, 128] - on every
 * rank, so no second exchange is needed.  heads_per_block (1..8, a divisor of q_heads_total) only
 * groups the finishing kernel's work.  Host-numbered steps only (gather->seq_dev must be NULL);
 * 16-bit dtypes; a descriptor serves steps of one shape. */
size_t tq_parts_exchange_bytes(int32_t batch, int32_t q_heads_total, int32_t parts);
int32_t tq_decode_attn_parts(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                             const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits, void *workspace,
                             size_t workspace_bytes, const tq_gather_desc *gather, int32_t parts, tq_stream stream);
int32_t tq_decode_parts_finish(tq_ctx *ctx, const tq_gather_desc *gather, int32_t batch, int32_t dtype,
                               int32_t parts, int32_t heads_per_block, void *out, tq_stream stream);

/* Decode attention for callers that cannot allocate (no counterpart in the reference).
 * Same computation and arguments as tq_decode_attn without a dense tail, but the scratch
 * lives in an 8 MiB array built into the library instead of a caller workspace: use it from
 * hosts that are not allowed to call an allocator while running (a server that owns all
 * device memory through its own pool, a plug-in hook barred from allocating).  Shapes that
 * need more than tq_static_scratch_bytes() of scratch return TQ_ERR_WORKSPACE.  The first
 * call on a device resolves the array's address and should happen before any stream capture.
 * All calls share the array: calls that overlap on the GPU race and must be serialised.
 * The context's device must be current. */
size_t tq_static_scratch_bytes(void);
int32_t tq_decode_attn_static(tq_ctx *ctx, const void *q, int32_t q_dtype, int32_t q_heads,
                              const tq_cache_desc *cache, int32_t seq_len, int32_t n_splits, void *out,
                              tq_stream stream);

/* How long tq_gather_wait polls for its peers before it gives up (milliseconds of the GPU's
 * wall clock, 1 .. 60000; 2000 when never set).  The value is read when the wait is queued. */
int32_t tq_set_wait_limit_ms(tq_ctx *ctx, int32_t limit_ms);

/* Device-side status (no reference counterpart).  Kernels never spin without a limit: a
 * wait on an asynchronous copy that runs out sets a status word instead of hanging.  This
 * call synchronises with the device and returns that word: 0 = no kernel ever gave up;
 * 1 = a decode kernel's wait ran out; 2 = a decode kernel found that its shared-memory layout
 * does not fit and did not run; 3 = the encoder's wait ran out; 4 = an append addressed a
 * token past the cache's capacity and was dropped; 5 = tq_gather_wait gave up waiting for a peer;
 * 6 = (bounds-checked build only) a kernel was about to read or write outside a buffer and did not.
 * The word is sticky for the context. */
int32_t tq_device_status(tq_ctx *ctx, int32_t *status_out);

/* Measurement hooks (no reference counterpart; used by the benchmark).  While enabled, each
 * tq_decode_attn call brackets its main kernel (the one that streams the packed cache)
 * with CUDA events on the launch stream and counts every kernel the library launches.
 * tq_profile_read synchronises those events, returns the summed main-kernel time and
 * the counts, and resets them. */
int32_t tq_profile_enable(tq_ctx *ctx, int32_t on);
int32_t tq_profile_read(tq_ctx *ctx, double *main_kernel_ms, int64_t *main_kernel_launches,
                        int64_t *all_launches);

#ifdef __cplusplus
}
#endif
#endif /* TQ_B200_H */
