/* irontensor_b200 -- C ABI of the B200 (sm_100a) attention path for the IronTensor library.
 *
 * This is what a CUDA device behind IronTensor's op layer binds to.  Every entry point names the
 * reference interface it stands in for (paths relative to the reference project's root).
 * Conventions:
 *   - plain C: opaque handles, raw pointers, sizes; no C++ or torch types.
 *   - every call returns an it_status (0 = OK, negative = error); it_last_error() gives the text
 *     of the calling thread's most recent failure.  Nothing throws, nothing aborts.
 *   - tensor arguments are DEVICE pointers owned by the caller, contiguous row-major
 *     [batch, heads, seq, head_dim] (the layout of src/ops/flash_attention.rs:65-70).
 *   - compute calls only enqueue work on `stream` and return; results are valid after
 *     it_stream_sync / it_event_wait, like work encoded into the reference's CommandBatch.
 *   - compute calls allocate nothing: scratch comes from the caller's workspace.
 *   - there is no CPU fallback: without a CUDA device it_ctx_create fails.
 */
#ifndef IRONTENSOR_B200_H
#define IRONTENSOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct it_ctx it_ctx;       /* one per process and GPU; stands in for MetalContext (src/device.rs:10-37) */
typedef struct it_stream it_stream; /* ordered work queue; stands in for a thread's CommandBatch (src/command_batch.rs:49-53) */
typedef struct it_event it_event;   /* completion marker; stands in for the async command buffer handle (src/command_batch.rs:228-275) */
typedef struct it_host_step it_host_step; /* buffers and streams of it_host_step_run */

typedef int32_t it_status;
enum {
  IT_OK = 0,
  IT_ERR_INVALID_ARG = -1,       /* null pointer, negative size, undersized workspace */
  IT_ERR_UNSUPPORTED_SHAPE = -2, /* head_dim outside 1..128 (assert at src/ops/flash_attention.rs:98) */
  IT_ERR_PRECISION = -3,         /* dtype not handled (asserts at src/ops/flash_attention.rs:78-80) */
  IT_ERR_ALIGNMENT = -4,         /* a tensor pointer is not 16-byte aligned */
  IT_ERR_CUDA = -5,              /* a CUDA runtime or driver call failed */
  IT_ERR_TIMEOUT = -6            /* a bounded wait inside a kernel ran out (see it_attention_status_poll) */
};

/* Storage precision of the tensors; arithmetic is fp32 either way (src/precision.rs:1-6;
 * bf16 follows "read BF16, compute FP32, write BF16", src/shaders/bf16_ops.metal:8). */
typedef enum { IT_F32 = 0, IT_BF16 = 1 } it_dtype;

/* ---- context, streams, events ------------------------------------------------------------- */

/* MetalContext::new / ::global (src/device.rs:17-29).  Fails with IT_ERR_CUDA when the device
 * does not exist or is not an sm_100 part. */
it_status it_ctx_create(int device, it_ctx** out);
it_status it_ctx_destroy(it_ctx* ctx);
/* Text of the calling thread's last error (never null). */
const char* it_last_error(void);

/* CommandBatch::begin (src/command_batch.rs:174-182): a new in-order queue.
 * Every stream object (created or wrapped) holds one 4-byte work-item counter out of a pool of 4096 that the
 * context allocates once: the bf16 forward for head_dim 64 and for head_dim 128 below 5120 keys starts one CTA
 * per SM when it has more work items than SMs, zeroes the counter in front of the launch and lets the CTAs draw
 * their next items from it.  Launches through one stream object run one after the other, so one counter is
 * enough; a stream object created when the pool is empty gets none and its forwards start one CTA per item
 * (same results).  A forward captured into a CUDA graph keeps the counter of the stream object it was captured
 * through: do not run that graph beside other forwards of the same stream object on another stream. */
it_status it_stream_create(it_ctx* ctx, it_stream** out);
/* Adopts an existing cudaStream_t (0 = the legacy default stream) without owning it. */
it_status it_stream_wrap(it_ctx* ctx, void* cuda_stream, it_stream** out);
it_status it_stream_destroy(it_ctx* ctx, it_stream* stream);
/* CommandBatch::sync / ::end (src/command_batch.rs:191-226): block until the queue drains.  Returns
 * IT_ERR_TIMEOUT (without clearing anything) when the device status word is set, see
 * it_attention_status_poll; so does it_event_wait. */
it_status it_stream_sync(it_ctx* ctx, it_stream* stream);

/* CommandBatch::commit_async / is_async_complete / wait_for_completion
 * (src/command_batch.rs:228-275). */
it_status it_event_create(it_ctx* ctx, it_event** out);
it_status it_event_destroy(it_ctx* ctx, it_event* ev);
it_status it_event_record(it_ctx* ctx, it_stream* stream, it_event* ev);
it_status it_event_query(it_ctx* ctx, it_event* ev, int32_t* done);
it_status it_event_wait(it_ctx* ctx, it_event* ev);
/* Device time between two recorded, completed events (the profiler hook of
 * src/profile/timer.rs:27-36, measured on the GPU instead of the host). */
it_status it_event_elapsed_ms(it_ctx* ctx, it_event* start, it_event* stop, float* ms);

/* ---- buffers ------------------------------------------------------------------------------ */

/* Tensor::zeros' allocation (src/tensor.rs:63-84); zero bytes allocate one byte as there. */
it_status it_buf_alloc(it_ctx* ctx, size_t bytes, void** out_dev);
it_status it_buf_free(it_ctx* ctx, void* dev);
/* Page-locked host memory for uploads/downloads that overlap with compute. */
it_status it_host_alloc(it_ctx* ctx, size_t bytes, void** out_host);
it_status it_host_free(it_ctx* ctx, void* host);
/* Tensor::from_f32_slice (src/tensor.rs:90-118) and Tensor::as_f32_slice (src/tensor.rs:136-148):
 * the reference's buffers are unified memory; here the copies are explicit and stream-ordered. */
it_status it_buf_upload(it_ctx* ctx, it_stream* stream, void* dst_dev, const void* src_host, size_t bytes);
it_status it_buf_download(it_ctx* ctx, it_stream* stream, void* dst_host, const void* src_dev, size_t bytes);
it_status it_buf_memset_async(it_ctx* ctx, it_stream* stream, void* dev, int value, size_t bytes);

/* ---- attention ---------------------------------------------------------------------------- */

/* flash_attention(q, k, v, causal) (src/ops/flash_attention.rs:76-193; kernels
 * src/shaders/flash_attention.metal:45-163 and :167-223).  O = softmax(mask(Q K^T / sqrt(D))) V.
 * Adds what the reference lacks: bf16 tensors, and lse[B,H,S] (fp32, natural log of the row's sum
 * of exp(scaled scores); may be null).  seq == 0 or batch*heads == 0 is a no-op returning IT_OK. */
it_status it_flash_attention_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t heads,
                                 int32_t seq, int32_t head_dim, int32_t causal, const void* q, const void* k,
                                 const void* v, void* o, float* lse);

/* Scratch size for it_flash_attention_bwd with the same dtype and shape. */
it_status it_flash_attention_bwd_workspace_bytes(it_dtype dtype, int32_t batch, int32_t heads, int32_t seq,
                                                 int32_t head_dim, size_t* out_bytes);

/* attention_backward_recompute(grad_output, q, k, v) (src/train/helpers.rs:120-193).  The
 * reference recomputes P from Q,K alone through eight S x S intermediates; this call recomputes
 * it tile by tile from the forward's lse, so it also takes o and lse (what the training cache of
 * src/train/cache.rs:10-15 gains).  The reference is always causal (helpers.rs:152); `causal`
 * must match the forward that produced o and lse.  workspace: device memory of at least
 * it_flash_attention_bwd_workspace_bytes, 256-byte aligned; its contents are overwritten. */
it_status it_flash_attention_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t heads,
                                 int32_t seq, int32_t head_dim, int32_t causal, const void* q, const void* k,
                                 const void* v, const void* o, const void* d_o, const float* lse, void* dq,
                                 void* dk, void* dv, void* workspace, size_t workspace_bytes);

/* attention(q, k, v, causal) on [batch, seq, heads, head_dim] tensors (src/ops/attention.rs:286-377), and
 * its backward in the same layout.  The reference gets from this layout to the flash-attention one and
 * back with transpose kernels (src/ops/transpose.rs:277-395; three before and one after each forward,
 * src/train/forward.rs:125-127,141; one before and three after each backward, src/train/backward.rs:102,
 * 114-116).  Here the kernels read and write the [B,S,H,D] tensors in place through strided TMA
 * descriptors, so those copies disappear.  Same math, dispatch, workspace size
 * (it_flash_attention_bwd_workspace_bytes with the same B, H, S, D) and error codes as the [B,H,S,D] entry
 * points; lse stays [batch, heads, seq].  K/V with another sequence length than Q (which the reference
 * allows when not causal): it_attention_cross_fwd below. */
it_status it_attention_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq, int32_t heads,
                           int32_t head_dim, int32_t causal, const void* q, const void* k, const void* v, void* o,
                           float* lse);
it_status it_attention_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq, int32_t heads,
                           int32_t head_dim, int32_t causal, const void* q, const void* k, const void* v, const void* o,
                           const void* d_o, const float* lse, void* dq, void* dk, void* dv, void* workspace,
                           size_t workspace_bytes);

/* attention(q, k, v, causal = false) with a key/value length different from the query length: the reference reads
 * kv_seq_len from K (src/ops/attention.rs:304) and only its causal branch requires it to equal q_seq_len (:349-352).
 * q, o: [batch, seq_q, heads, head_dim]; k, v: [batch, seq_kv, heads, head_dim]; lse [batch, heads, seq_q] (may be
 * null).  Never causal.  seq_q == seq_kv is it_attention_fwd with causal = 0 (tensor-core kernels for bf16);
 * otherwise the CUDA-core kernels run (fp32 as in the reference, or bf16), since a query and a key length that
 * differ occur in the reference only outside its training path.  The reference has no backward for this op. */
it_status it_attention_cross_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq_q,
                                 int32_t seq_kv, int32_t heads, int32_t head_dim, const void* q, const void* k,
                                 const void* v, void* o, float* lse);

/* Grouped-query attention on [batch, seq, heads, head_dim] queries and [batch, seq, kv_heads, head_dim]
 * keys/values, kv_heads dividing heads; query head h reads K/V head h / (heads / kv_heads).  The reference
 * expands K and V to `heads` heads with repeat_kv before its attention and sums the expanded gradients
 * back with repeat_kv_backward after it (src/ops/repeat_kv.rs:68-149, 151-232; kernels
 * src/shaders/repeat_kv.metal:19-47, 49-88; call sites src/train/forward.rs:117-118,
 * src/train/backward.rs:121-122).  Here the head mapping is a coordinate of the K/V tensor maps and the
 * backward accumulates dK/dV over the group's query heads in tensor memory, so neither the expanded
 * copies nor the expanded gradients exist.  o, d_o, dq: [batch, seq, heads, head_dim]; dk, dv:
 * [batch, seq, kv_heads, head_dim]; lse: [batch, heads, seq].  Workspace size:
 * it_flash_attention_bwd_workspace_bytes with the QUERY head count.  kv_heads == heads is it_attention_*. */
it_status it_attention_gqa_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq,
                               int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t causal, const void* q,
                               const void* k, const void* v, void* o, float* lse);
it_status it_attention_gqa_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq,
                               int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t causal, const void* q,
                               const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                               void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes);

/* Rotary position embedding of Q [batch, seq, heads, head_dim] and K [batch, seq, kv_heads, head_dim] in ONE
 * launch (the reference runs rope() once per tensor: src/ops/rope.rs:22-75, kernel src/shaders/rope.metal:22-61;
 * call sites src/train/forward.rs:111-112).  theta_i = 1 / base^(2i / head_dim), angle = (position +
 * position_offset) * theta_i; pairs (2i, 2i+1) are rotated.  inverse != 0 applies the backward rotation
 * (rope_backward, src/shaders/backward/rope.metal:25-62).  head_dim must be even.  kv_heads may be 0 (K is
 * then not touched).  In place (q_out == q_in) is allowed.  F32 as in the reference, or BF16. */
it_status it_rope_qk(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq, int32_t heads,
                     int32_t kv_heads, int32_t head_dim, float rope_base, int32_t position_offset, int32_t inverse,
                     const void* q_in, const void* k_in, void* q_out, void* k_out);

/* it_attention_gqa_bwd with the backward of the rotary embedding folded in: q and k are the ROTATED tensors
 * the forward attended over, dq and dk come back as gradients of the un-rotated ones.  The reference runs
 * rope_backward as two more passes after its attention backward (src/train/backward.rs:129,132); here the
 * rotation is applied where dQ and dK leave the chip (the fp32 -> bf16 pass of dQ, the dK epilogue), so
 * those passes and their 4 x tensor bytes of traffic do not exist.  dv is not affected. */
it_status it_attention_gqa_bwd_rope(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq,
                                    int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t causal,
                                    float rope_base, int32_t position_offset, const void* q, const void* k,
                                    const void* v, const void* o, const void* d_o, const float* lse, void* dq,
                                    void* dk, void* dv, void* workspace, size_t workspace_bytes);

/* Attention for ONE new token per sequence against a key/value cache.  (The reference has no cache: its
 * generator re-runs the whole forward for every generated token, src/inference/generator.rs:146-200, and
 * lists "Inference-optimized KV cache" as future work, docs/PRESENTATION.md:576.)  q, o: [batch, heads,
 * head_dim]; k_cache, v_cache: [batch, max_len, kv_heads, head_dim] (the [B,S,H,D] layout the projections
 * produce, so appending a token writes one row), of which the first kv_len positions are valid and include
 * the new token's own key and value; kv_heads divides heads.  o equals the last row of causal attention
 * over those kv_len tokens (src/shaders/flash_attention.metal:167-223 with q = kv_len - 1); lse ([batch,
 * heads], natural log, may be null) as in it_flash_attention_fwd.  The keys are split over CTAs and merged
 * when batch * kv_heads alone cannot fill the GPU; each cache row is read once per group of query heads.
 * head_dim a multiple of 8.  workspace: it_attention_decode_workspace_bytes, 256-byte aligned. */
it_status it_attention_decode_workspace_bytes(int32_t batch, int32_t heads, int32_t head_dim, size_t* out_bytes);
it_status it_attention_decode(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t heads,
                              int32_t kv_heads, int32_t head_dim, int32_t kv_len, int32_t max_len, const void* q,
                              const void* k_cache, const void* v_cache, void* o, float* lse, void* workspace,
                              size_t workspace_bytes);

/* The projections around attention (src/train/forward.rs:101-103,146; src/train/backward.rs:91,139-147) in bf16:
 * linear_forward, y = x W^T with x [n, in], W [out, in] (src/train/helpers.rs:48-53: matmul_mps_nt), and
 * linear_backward, dx = dy W and dW = dy^T x (helpers.rs:61-76: matmul, matmul_mps_tn).  The reference runs
 * them on MPS in fp32, converting bf16 weights first (ensure_fp32); here x, W, dy, y, dx are bf16, the
 * accumulation is fp32 in tensor memory, and dW comes back in fp32 as the reference's gradients do.  The
 * three transposition cases are descriptor bits of one tcgen05 kernel, nothing is transposed in memory.  in and
 * out must be multiples of 8.  dx or dw may be null (not computed). */
it_status it_linear_fwd(it_ctx* ctx, it_stream* stream, int32_t n, int32_t in_dim, int32_t out_dim, const void* x,
                        const void* w, void* y);
it_status it_linear_bwd(it_ctx* ctx, it_stream* stream, int32_t n, int32_t in_dim, int32_t out_dim, const void* dy,
                        const void* x, const void* w, void* dx, float* dw);

/* A projection whose result is a SUM OVER GPUs, with the reduce-scatter done by the GEMM itself.  With the heads of a layer
 * split over `world` GPUs, the output projection (src/train/forward.rs:146: attn [n, heads*D] @ Wo^T) and the gradient of
 * the layer's input (src/train/backward.rs:139-147) are sums over ranks of partial products; the reference is single-device
 * and has neither.  kind 0: a [n, in] times W [out, in]^T -> [n, out];  kind 1: a [n, out] times W [out, in] -> [n, in]
 * (bf16, fp32 accumulation, as it_linear_fwd / the dx of it_linear_bwd).  Instead of storing its partial product the
 * kernel ADDS row block [r*rows_per_rank, (r+1)*rows_per_rank) into c_of_rank[r] as the tiles leave tensor memory
 * (TMA reduce-adds of bf16 in whole 128-byte lines, over NVLink for r != this rank), so the exchange runs under the GEMM's own math and after all
 * ranks' calls rank r holds the finished sum of its row block; an all-gather of the row blocks makes it an all-reduce.
 * c_of_rank[r]: the [n, width] bf16 result buffer of rank r as a pointer THIS process may store to (peer mapping of a
 * symmetric allocation; c_of_rank[own rank] is local memory).  The caller zeroes its own row block and synchronises
 * the ranks before the call (no add may arrive before the zeroing) and after it (all adds have landed) -- with a
 * collective barrier over the same ranks.  The summed product's width must be a multiple of 64 and rows_per_rank of
 * 128; world <= 8.  Sums of
 * bf16 partials are rounded to bf16 at every add, like a bf16 all-reduce. */
it_status it_linear_scatter_add(it_ctx* ctx, it_stream* stream, int32_t kind, int32_t n, int32_t in_dim, int32_t out_dim,
                                const void* a, const void* w, void* const* c_of_rank, int32_t world, int32_t rows_per_rank);

/* The Q, K and V projections and the rotary embedding of Q and K as ONE kernel: x [batch*seq, hidden] times the
 * stacked weights w_qkv = [Wq; Wk; Wv] ([(heads + 2*kv_heads)*head_dim, hidden]), the rotation applied in the
 * GEMM's epilogue, q_out [batch, seq, heads, head_dim], k_out and v_out [batch, seq, kv_heads, head_dim] written
 * in the layout it_attention_gqa_* read.  The reference runs three linear_forward calls on the same input and
 * rope() twice (src/train/forward.rs:101-103,111-112).  rope_base 0 leaves Q and K un-rotated.  bf16; head_dim
 * 32, 64, 96 or 128; hidden a multiple of 8.  workspace (it_qkv_rope_workspace_bytes, 256-byte aligned; may be
 * null when rope_base is 0) holds the cosine/sine table of the call.  With k_out and v_out both null, q_out is
 * ONE packed buffer [batch, seq, (heads + 2*kv_heads)*head_dim] holding q_rope | k_rope | v per token: the layout
 * it_attention_packed_* read, and whose gradient it_linear_bwd takes as a single dy. */
it_status it_qkv_rope_workspace_bytes(int32_t seq, int32_t head_dim, size_t* out_bytes);
it_status it_qkv_rope_fwd(it_ctx* ctx, it_stream* stream, int32_t batch, int32_t seq, int32_t hidden, int32_t heads,
                          int32_t kv_heads, int32_t head_dim, float rope_base, int32_t position_offset, const void* x,
                          const void* w_qkv, void* q_out, void* k_out, void* v_out, void* workspace,
                          size_t workspace_bytes);

/* Attention on the packed projection output: qkv [batch, seq, (heads + 2*kv_heads)*head_dim] = q | k | v per token
 * (what it_qkv_rope_fwd writes with k_out = v_out = null), o and d_o [batch, seq, heads, head_dim], dqkv in the
 * layout of qkv.  Same kernels as it_attention_gqa_*: the column ranges are tensor-map strides.  With the
 * projections on both sides this removes every layout step of the reference's layer (views, transposes, repeat_kv,
 * the concatenation of the three gradients before the weight GEMMs): forward = it_qkv_rope_fwd, it_attention_packed_fwd,
 * it_linear_fwd (Wo); backward = it_linear_bwd (Wo), it_attention_packed_bwd, it_linear_bwd (stacked [Wq; Wk; Wv]).
 * rope_base as in it_attention_gqa_bwd_rope (0: none).  bf16, head_dim 64 or 128, seq >= 128. */
it_status it_attention_packed_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq,
                                  int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t causal, const void* qkv,
                                  void* o, float* lse);
it_status it_attention_packed_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch, int32_t seq,
                                  int32_t heads, int32_t kv_heads, int32_t head_dim, int32_t causal, float rope_base,
                                  int32_t position_offset, const void* qkv, const void* o, const void* d_o,
                                  const float* lse, void* dqkv, void* workspace, size_t workspace_bytes);

/* Forward + backward for tensors that live in page-locked HOST memory (the reference's buffers are unified memory, so
 * its ops never copy: src/tensor.rs:73; on a discrete GPU a caller with host data pays the host link both ways).  One
 * call enqueues the whole step: the (batch x head) slices are taken `group_slices` at a time, each group on one of
 * `n_streams` streams in rotation: upload q, k, v, dO -> it_flash_attention_fwd -> it_flash_attention_bwd -> download
 * o, dq, dk, dv (and lse when hlse is not null), so that one group's upload, another's kernels and a third's download run
 * at the same time on the two copy engines and the SMs.  With the loop inside the library the host spends microseconds
 * per group, so groups can be small and the first upload and last download, which nothing overlaps, short.
 * it_host_step_create allocates the device buffers (per stream: eight group-sized tensors, lse and the backward's
 * workspace), streams and events once; it_host_step_run allocates nothing.  All host pointers: [n_slices, S, D]
 * (lse [n_slices, S]) of the dtype given at creation, page-locked (it_host_alloc) for the copies to overlap.  The groups
 * start after the work enqueued on `stream` so far, and `stream` continues after the last download; nothing is waited
 * for on the host: it_stream_sync(stream) before reading the results (it reports a device time-out).  copies_only != 0
 * enqueues the same copies without the kernels (what the host link alone costs).  One run at a time per it_host_step. */
it_status it_host_step_create(it_ctx* ctx, it_dtype dtype, int32_t group_slices, int32_t seq, int32_t head_dim,
                              int32_t causal, int32_t n_streams, it_host_step** out);
it_status it_host_step_run(it_host_step* step, it_stream* stream, int32_t n_slices, const void* q, const void* k,
                           const void* v, const void* d_o, void* o, float* lse, void* dq, void* dk, void* dv,
                           int32_t copies_only);
it_status it_host_step_destroy(it_host_step* step);

/* Backward for callers that cannot allocate device memory.  (No counterpart in the reference:
 * there every op allocates its own buffers, src/tensor.rs:63-84.)
 *
 * Who needs it: a host that runs inside someone else's CUDA context and was handed only tensor
 * pointers and a stream -- for instance a plugin called from a real-time or sandboxed process
 * whose policy forbids cudaMalloc after start-up, or code running while another component owns
 * the allocator and any allocation could stall or fail.  Such a caller has nowhere to take
 * it_flash_attention_bwd's workspace from.  Here the scratch is a fixed array of
 * IT_NOALLOC_SCRATCH_BYTES that is part of the library image: every GPU that loads the library
 * holds that much memory until the process exits, whether or not this call is ever made.
 *
 * Same arguments, results and dispatch as it_flash_attention_bwd, minus the workspace.  Differences:
 *   - the shape is refused with IT_ERR_UNSUPPORTED_SHAPE when its scratch need
 *     (it_flash_attention_bwd_workspace_bytes) exceeds IT_NOALLOC_SCRATCH_BYTES;
 *   - this call makes no cudaMalloc / cudaFree and calls nothing that allocates device memory; the
 *     first call on a device may still make the CUDA runtime load this library's kernels, which is
 *     the runtime's own one-time work -- from the second call on nothing is allocated at all;
 *   - the first call on each device looks up the array's device address (a symbol lookup, once per
 *     device and process): make that first call outside any stream capture.  The address is kept for
 *     the life of the process, so it does not survive a cudaDeviceReset by the host application;
 *   - all calls on one GPU share the one array, and it keeps the previous call's contents; the call
 *     clears what has to start from zero itself.  Two calls whose kernels can overlap on the GPU
 *     (different streams, no ordering between them) race on it: order them. */
#define IT_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)
it_status it_flash_attention_bwd_noalloc(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t batch,
                                         int32_t heads, int32_t seq, int32_t head_dim, int32_t causal,
                                         const void* q, const void* k, const void* v, const void* o,
                                         const void* d_o, const float* lse, void* dq, void* dk, void* dv);

/* Kernels never spin without bound: a wait that runs out (one second of wall-clock time on the device's
 * global timer, which keeps counting while the context is descheduled or serialised by a tool) records a
 * code in the context's device status word and the kernel winds down.  While the word is non-zero EVERY
 * later launch of this library on the context, on any stream, returns at once without computing, so the
 * outputs of those launches are not written: the C entry points still return IT_OK (they only enqueue),
 * and it_stream_sync, it_event_wait and it_ctx_check_status report IT_ERR_TIMEOUT.
 * it_attention_status_poll drains `stream`, returns the word in *device_status (0 = clean) and CLEARS it,
 * after which launches compute again.  Returns IT_ERR_TIMEOUT when the word was non-zero.
 * (The reference never checks command-buffer errors; src/command_batch.rs:191-226.) */
it_status it_attention_status_poll(it_ctx* ctx, it_stream* stream, int32_t* device_status);
/* Reads the status word without draining a caller's stream and without clearing it: IT_OK when zero,
 * IT_ERR_TIMEOUT otherwise; *device_status (may be null) gets the word.  For hosts that synchronise by
 * other means (their own events, a blocking copy) before they read results. */
it_status it_ctx_check_status(it_ctx* ctx, int32_t* device_status);

/* How many kernels this library has launched on this context since it was created. */
it_status it_ctx_launch_count(it_ctx* ctx, uint64_t* out);

/* Device-side timers around the two main kernels, the counterpart of the reference's
 * OpCategory::FlashAttention timer (src/ops/flash_attention.rs:77, src/profile/timer.rs:27-36),
 * which measures host encode time.  enable = 1: each it_flash_attention_bwd call records a CUDA event before
 * and after its main kernel on the call's stream; 2: the forward kernel of it_flash_attention_fwd as well; 3: the
 * backward's prepare and finish passes too.  Every bracket is two event records in the stream: a few
 * microseconds each, visible on the smallest shapes (12 us of a 50 us step), which is why the levels exist.
 * it_ctx_kernel_ms waits for the most recent such pair and returns the time between them
 * (which = 0: forward kernel, 1: backward main kernel, 2: backward prepare pass, 3: backward finish pass; 2 and 3
 * exist for the tensor-core backward only).  it_ctx_kernel_tag gives the reference's profiler tag for what a timer
 * covers: its composed backward reports attn_bwd/recompute, /grad_v, /grad_p and /grad_qk (src/train/helpers.rs:
 * 126-183), all of which are inside the one main kernel here. */
it_status it_ctx_enable_kernel_timing(it_ctx* ctx, int32_t enable);
it_status it_ctx_kernel_ms(it_ctx* ctx, int32_t which, float* ms);
const char* it_ctx_kernel_tag(int32_t which);

/* ---- self tests (no reference counterpart; they pin the hardware descriptors the kernels use) */

/* One 128x128x128 bf16 MMA through the given operand path, result fp32 [128,128] row-major.
 *   variant 0: A, B both K-major in shared memory (TMA)             a[128(M),128(K)], b[128(N),128(K)]
 *   variant 1: A from tensor memory, B N-major in shared memory     a[M,K], b[128(K),128(N)]
 *   variant 2: A K-major written by threads (swizzled), B N-major   a[M,K], b[K,N]
 *   variant 3: A M-major written by threads (swizzled), B N-major   a[M,K], b[K,N]
 * In every variant out = a * (b as K x N). */
it_status it_selftest_umma(it_ctx* ctx, it_stream* stream, int32_t variant, const void* a_bf16,
                           const void* b_bf16, float* out);
/* Launches one CTA that waits `limit_ms` on a barrier nothing arrives on, so that the bounded-wait
 * path can be checked: afterwards it_attention_status_poll reports a non-zero word. */
it_status it_selftest_wait_timeout(it_ctx* ctx, it_stream* stream, int32_t limit_ms);

#ifdef __cplusplus
}
#endif
#endif /* IRONTENSOR_B200_H */
