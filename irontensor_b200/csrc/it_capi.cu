// C ABI of the B200 attention path (declared in include/irontensor_b200.h): context, streams,
// events, buffers, and the attention forward / backward dispatch onto the sm_100a kernels.
// Host-side validation mirrors the reference's asserts (src/ops/flash_attention.rs:78-104) but
// returns status codes instead of panicking.
#include "../../include/irontensor_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <cmath>
#include <mutex>
#include <new>

#include "fa_bwd_sm100.cuh"
#include <algorithm>
#include <vector>
#include <type_traits>

#include "fa_fwd_sm100.cuh"
#include "fa_decode.cuh"
#include "fa_fwd_pp_sm100.cuh"
#include "fa_fwd_f32_sm100.cuh"
#include "gemm_sm100.cuh"
#include "fa_generic.cuh"
#include "selftest_sm100.cuh"

namespace {

thread_local char g_err[512] = "";

it_status fail(it_status code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return code;
}

#define IT_CUDA(expr)                                                                              \
  do {                                                                                             \
    cudaError_t e_ = (expr);                                                                       \
    if (e_ != cudaSuccess) return fail(IT_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_));      \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

struct it_ctx {
  int device = 0;
  int sm_count = 0;
  int* d_status = nullptr;      // device status word written by kernels whose waits run out
  int* h_status = nullptr;      // pinned mirror
  cudaStream_t status_stream = nullptr;   // reads the status word without touching a caller's stream
  std::mutex status_mutex;      // h_status and status_stream are shared by every thread using the context
  EncodeTiledFn encode = nullptr;
  int timing = 0;               // events around: 1 the backward main kernel; 2 the forward kernel too; 3 the backward's prepare and finish passes too
  // [forward | backward main | backward prepare | backward finish][start | stop]; the prepare pass starts where the
  // previous timer stopped only in time, not in events: three pairs share the boundaries prepare|main|finish
  cudaEvent_t ev[4][2] = {};
  bool ev_valid[4] = {false, false, false, false};
  std::atomic<uint64_t> launches{0};
  // Work-item counters of the forward kernel that walks its items in a loop: one int per live stream object (launches
  // on one stream run one after the other, so a stream needs one counter), handed out from a pool allocated with the
  // context so that wrapping a stream calls nothing a stream capture forbids.
  static constexpr int WORK_SLOTS = 4096;
  int* d_work_pool = nullptr;
  std::mutex work_mutex;
  std::vector<int> work_free;
  int work_next = 0;
};
struct it_stream {
  cudaStream_t s = nullptr;
  bool owned = false;
  int* d_work = nullptr;     // this stream's work-item counter; null when the pool ran out (the launcher then starts one CTA per item)
  bool work_used = false;    // a launch has drawn from the counter
};
namespace {
int* take_work_slot(it_ctx* ctx) {
  std::lock_guard<std::mutex> lock(ctx->work_mutex);
  if (ctx->d_work_pool == nullptr) return nullptr;
  if (!ctx->work_free.empty()) {
    const int i = ctx->work_free.back();
    ctx->work_free.pop_back();
    return ctx->d_work_pool + i;
  }
  return ctx->work_next < it_ctx::WORK_SLOTS ? ctx->d_work_pool + ctx->work_next++ : nullptr;
}
void give_work_slot(it_ctx* ctx, it_stream* stream) {
  if (ctx == nullptr || stream->d_work == nullptr) return;
  if (stream->work_used) cudaStreamSynchronize(stream->s);   // a kernel in flight may still draw from the counter
  std::lock_guard<std::mutex> lock(ctx->work_mutex);
  ctx->work_free.push_back(static_cast<int>(stream->d_work - ctx->d_work_pool));
  stream->d_work = nullptr;
}
}  // namespace
struct it_event {
  cudaEvent_t e = nullptr;
};
// Device buffers, streams and events of it_host_step_*: everything a forward + backward over host-resident tensors
// needs, allocated once.
struct it_host_step {
  it_ctx* ctx = nullptr;
  it_dtype dtype = IT_BF16;
  int32_t group_slices = 0, S = 0, D = 0, causal = 1, n_streams = 0;
  size_t tensor_bytes = 0, lse_bytes = 0, ws_bytes = 0;   // per group
  static constexpr int MAX_STREAMS = 4;
  it_stream streams[MAX_STREAMS];
  cudaEvent_t done[MAX_STREAMS] = {};
  cudaEvent_t start = nullptr;
  uint8_t* dev[MAX_STREAMS] = {};   // per stream: q, k, v, dO, o, dq, dk, dv, lse, workspace
};

namespace {

// Copies the device status word to the host on the context's own stream.  Called after a caller's
// stream or event has been waited for, so every kernel that could have written the word is done.
it_status read_device_status(it_ctx* ctx, int* out) {
  std::lock_guard<std::mutex> lock(ctx->status_mutex);
  IT_CUDA(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->status_stream));
  IT_CUDA(cudaStreamSynchronize(ctx->status_stream));
  *out = *ctx->h_status;
  return IT_OK;
}

it_status fail_if_device_status(it_ctx* ctx) {
  int st = 0;
  it_status rc = read_device_status(ctx, &st);
  if (rc != IT_OK) return rc;
  if (st != 0)
    return fail(IT_ERR_TIMEOUT,
                "a bounded wait inside a kernel ran out (device status %d): results of launches since then are "
                "invalid, and further launches on this context do nothing until it_attention_status_poll clears it",
                st);
  return IT_OK;
}

// A bf16 attention tensor viewed by TMA as a 4-D tensor (head_dim, seq, heads, batch) with the
// layout's strides; one box = 128 rows x 64 columns of one (batch, head) slice, written to shared
// memory with the 128-byte swizzle.  Rows past `seq` read as zero.
it_status make_tmap(it_ctx* ctx, CUtensorMap* map, const void* base, int64_t B, int64_t H, int64_t S, int64_t D,
                    const it::TensorStrides& st, int box_rows) {
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(H),
                              static_cast<cuuint64_t>(B)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st.row) * 2, static_cast<cuuint64_t>(st.head) * 2,
                                 static_cast<cuuint64_t>(st.batch) * 2};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = ctx->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(IT_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
  return IT_OK;
}

// [B,H,S,D] (flash_attention) and [B,S,H,D] (attention) as strides in elements.
it::TensorStrides strides_bhsd(int64_t H, int64_t S, int64_t D) { return it::TensorStrides{D, S * D, H * S * D, static_cast<int>(H)}; }
it::TensorStrides strides_bshd(int64_t H, int64_t S, int64_t D) { return it::TensorStrides{H * D, D, S * H * D, static_cast<int>(H)}; }
// A K/V tensor with Hkv = H / group heads, indexed by the query slice (see TensorStrides).
it::TensorStrides strides_kv(bool bshd, int64_t H, int64_t Hkv, int64_t S, int64_t D) {
  it::TensorStrides t = bshd ? strides_bshd(Hkv, S, D) : strides_bhsd(Hkv, S, D);
  t.heads = static_cast<int>(H);
  t.group = static_cast<int>(H / Hkv);
  return t;
}

// theta_i = 1.0f / pow(base, float(2i) / float(head_dim)), every step in fp32 as the shader computes it
// (src/shaders/rope.metal:41-43), so a CPU check that calls the same powf multiplies positions by the
// same frequencies bit for bit.
it::RopeFreqs make_rope_freqs(int D, float base, int position_offset, bool enabled) {
  it::RopeFreqs f;
  for (int i = 0; i < 64; ++i)
    f.inv_freq[i] = (enabled && 2 * i < D) ? 1.0f / powf(base, static_cast<float>(2 * i) / static_cast<float>(D)) : 0.f;
  f.enabled = enabled ? 1 : 0;
  f.position_offset = position_offset;
  return f;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

it_status check_common(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H, int32_t S, int32_t D) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (dtype != IT_F32 && dtype != IT_BF16) return fail(IT_ERR_PRECISION, "dtype %d is not F32 or BF16", (int)dtype);
  if (B < 0 || H < 0 || S < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  if (D < 1 || D > 128) return fail(IT_ERR_UNSUPPORTED_SHAPE, "head_dim must be in 1..128, got %d", D);
  if (static_cast<int64_t>(B) * H > 65535)
    return fail(IT_ERR_UNSUPPORTED_SHAPE, "batch*heads must be <= 65535, got %lld", (long long)B * H);
  return IT_OK;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may be set up while the kernel in front of it
// in the stream still runs, and waits in griddepcontrol.wait for that kernel's completion before it touches its results.
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

// The tensor-core kernels take bf16 tensors with head_dim 64 or 128 and at least one full tile.
bool use_sm100_path(it_dtype dtype, int32_t S, int32_t D) {
  return dtype == IT_BF16 && (D == 64 || D == 128) && S >= 128;
}

int round_dp(int D) { return D <= 16 ? 16 : D <= 32 ? 32 : D <= 64 ? 64 : 128; }

template <typename ST>
it_status launch_fwd_generic(it_ctx* ctx, cudaStream_t s, int BH, int S, int D, int causal, const void* q, const void* k,
                        const void* v, void* o, float* lse, const it::TensorStrides& st, const it::TensorStrides& skv,
                        int Skv = -1) {
  if (Skv < 0) Skv = S;   // self-attention; a different key/value length only comes from it_attention_cross_fwd
  if (sizeof(ST) == 4 && D <= 64 && (D & 3) == 0 && S >= 128 && Skv == S && getenv("IT_F32_CUDA_CORES") == nullptr) {
    // fp32 tensors with at least one full 128-row tile: the tensor-core kernel (operands split into three bf16 terms).
    // Shorter sequences -- the per-token calls of generation without a key/value cache -- stay on the latency kernel below.
    using T = it::FwdF32Traits;
    static std::atomic<bool> attr_set[16];
    if (!attr_set[ctx->device & 15]) {
      IT_CUDA(cudaFuncSetAttribute(it::fa_fwd_f32_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
      attr_set[ctx->device & 15] = true;
    }
    it::FwdF32Params p;
    p.q = static_cast<const float*>(q);
    p.k = static_cast<const float*>(k);
    p.v = static_cast<const float*>(v);
    p.o = static_cast<float*>(o);
    p.lse = lse;
    p.st = st;
    p.st_kv = skv;
    p.status = ctx->d_status;
    p.S = S;
    p.D = D;
    p.causal = causal;
    p.scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;
    it::fa_fwd_f32_sm100_kernel<<<static_cast<unsigned>(BH) * ((S + 127) / 128), T::THREADS, T::SMEM_BYTES, s>>>(p);
    ctx->launches += 1;
    IT_CUDA(cudaGetLastError());
    return IT_OK;
  }
  const float scale = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;   // exp2 domain
  const dim3 grid((S + 63) / 64, BH);
  const ST *qq = static_cast<const ST*>(q), *kk = static_cast<const ST*>(k), *vv = static_cast<const ST*>(v);
  ST* oo = static_cast<ST*>(o);
  if (sizeof(ST) == 4 && S <= 2048 && (D & 3) == 0) {   // fp32, short to medium sequences: the latency path
    const int smem = (16 * D + 4 * 32 * (D + 4) + 4 * 4 * 32) * 4;
    const dim3 g16((S + 15) / 16, BH);
    const float *qf = reinterpret_cast<const float*>(q), *kf = reinterpret_cast<const float*>(k),
                *vf = reinterpret_cast<const float*>(v);
    float* of = reinterpret_cast<float*>(o);
    // Four rows per warp (128 threads) or two (256 threads).  A launch with no more CTAs than SMs (the
    // per-token calls of no-KV-cache generation) is a chain of dependent steps in every warp, and halving
    // the rows per warp shortens it (6.7 against 7.3 us per call at batch 1, 4 heads, 20..119 keys); a launch
    // with several CTAs per SM is bound by issue and shared-memory loads, where four rows per warp reuse
    // each K chunk twice as often (53 against 64 us at batch 16, 4 heads, 256 keys).
    const int rw = (static_cast<long long>(g16.x) * g16.y <= ctx->sm_count) ? 2 : 4;
    const unsigned nt = 32u * (16u / static_cast<unsigned>(rw));
    if (D <= 32) {
      if (rw == 2) IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<1, 2>, g16, dim3(nt), smem, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
      else IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<1, 4>, g16, dim3(nt), smem, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
    } else if (D <= 64 && static_cast<long long>(g16.x) * g16.y > 4LL * ctx->sm_count) {
      // Many CTAs per SM (the reference's TINY training shape, batch 16 x 4 heads x 256 keys): the kernel is
      // bound by its shared-memory loads, and 32-row CTAs with eight rows per warp use every K chunk and V
      // row for twice as many rows (49 against 53 us on that shape).
      const int smem32 = (32 * D + 4 * 32 * (D + 4) + 32 * 32) * 4;
      const dim3 g32((S + 31) / 32, BH);
      IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<2, 8, 32>, g32, dim3(128), smem32, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
    } else if (D <= 64) {
      if (rw == 2) IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<2, 2>, g16, dim3(nt), smem, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
      else IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<2, 4>, g16, dim3(nt), smem, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
    } else {
      static std::atomic<bool> attr_set[16];   // zero-initialised; setting an attribute twice is harmless
      if (!attr_set[ctx->device & 15]) {
        IT_CUDA(cudaFuncSetAttribute(it::fa_fwd_rows_f32_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (16 * 128 + 4 * 32 * 132 + 512) * 4));
        IT_CUDA(cudaFuncSetAttribute(it::fa_fwd_rows_f32_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (16 * 128 + 4 * 32 * 132 + 512) * 4));
        attr_set[ctx->device & 15] = true;
      }
      if (rw == 2) IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<4, 2>, g16, dim3(nt), smem, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
      else IT_CUDA(launch_dependent(it::fa_fwd_rows_f32_kernel<4, 4>, g16, dim3(nt), smem, s, qf, kf, vf, of, lse, S, Skv, D, causal, scale, st, skv));
    }
    ctx->launches += 1;
    IT_CUDA(cudaGetLastError());
    return IT_OK;
  }
  switch (round_dp(D)) {
    case 16: it::fa_fwd_generic_kernel<ST, 16><<<grid, 256, 0, s>>>(qq, kk, vv, oo, lse, S, Skv, D, causal, scale, st, skv); break;
    case 32: it::fa_fwd_generic_kernel<ST, 32><<<grid, 256, 0, s>>>(qq, kk, vv, oo, lse, S, Skv, D, causal, scale, st, skv); break;
    case 64: it::fa_fwd_generic_kernel<ST, 64><<<grid, 256, 0, s>>>(qq, kk, vv, oo, lse, S, Skv, D, causal, scale, st, skv); break;
    default: it::fa_fwd_generic_kernel<ST, 128><<<grid, 256, 0, s>>>(qq, kk, vv, oo, lse, S, Skv, D, causal, scale, st, skv); break;
  }
  ctx->launches += 1;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

template <typename ST>
it_status launch_bwd_generic(it_ctx* ctx, cudaStream_t s, int BH, int S, int D, int causal, const void* q, const void* k,
                        const void* v, const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                        float* delta, const it::TensorStrides& st, const it::TensorStrides& skv, const it::RopeFreqs& rf) {
  const float scale = 1.0f / sqrtf(static_cast<float>(D));
  const ST *qq = static_cast<const ST*>(q), *kk = static_cast<const ST*>(k), *vv = static_cast<const ST*>(v);
  const ST *oo = static_cast<const ST*>(o), *dd = static_cast<const ST*>(d_o);
  const long long rows = static_cast<long long>(BH) * S;
  it::fa_bwd_generic_delta_kernel<ST><<<static_cast<unsigned>((rows + 3) / 4), 128, 0, s>>>(oo, dd, delta, rows, S, D, st);
  const dim3 grid((S + 3) / 4, BH), grid_kv((S + 3) / 4, BH / skv.group);
  it::fa_bwd_generic_kernel<ST, 0><<<grid, 128, 0, s>>>(qq, kk, vv, dd, lse, delta, static_cast<ST*>(dq), static_cast<ST*>(dk),
                                                        static_cast<ST*>(dv), S, D, causal, scale, st, skv, rf);
  it::fa_bwd_generic_kernel<ST, 1><<<grid_kv, 128, 0, s>>>(qq, kk, vv, dd, lse, delta, static_cast<ST*>(dq), static_cast<ST*>(dk),
                                                           static_cast<ST*>(dv), S, D, causal, scale, st, skv, rf);
  ctx->launches += 3;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

// The two tensor-core forward kernels: one query tile per CTA with the softmax groups alternating over key
// tiles (long sequences: the tensor core never waits for a softmax), or two query tiles per CTA sharing
// each K/V tile (short sequences: half as many CTA start-ups per unit of work).
template <int D, bool PP>
it_status launch_fwd_sm100(it_ctx* ctx, it_stream* stream, int B, int H, int S, int causal, const void* q, const void* k,
                           const void* v, void* o, float* lse, const it::TensorStrides& stv,
                           const it::TensorStrides& skv, const it::TensorStrides& sq) {
  const int BH = B * H;
  const int Hkv = H / skv.group;
  cudaStream_t s = stream->s;
  using T = std::conditional_t<PP, it::FwdPPTraits<D>, it::FwdTraits<D>>;
  auto kernel = PP ? it::fa_fwd_pp_sm100_kernel<D> : it::fa_fwd_sm100_kernel<D>;
  CUtensorMap mq, mk, mv;
  it_status st;
  if ((st = make_tmap(ctx, &mq, q, B, H, S, D, sq, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mk, k, B, Hkv, S, D, skv, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mv, v, B, Hkv, S, D, skv, 128)) != IT_OK) return st;
  static std::atomic<bool> attr_set[16];   // zero-initialised; setting an attribute twice is harmless
  if (!attr_set[ctx->device & 15]) {
    IT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
    attr_set[ctx->device & 15] = true;
  }
  it::FwdParams p;
  p.st = stv;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.status = ctx->d_status;
  p.S = S;
  p.BH = BH;
  p.causal = causal;
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;
  p.kv_group = skv.group;
  // Slices whose work items the two-query-tile kernel hands out together (heaviest pairs of all of them first): as many
  // as have 40 MB of K and V at head_dim 128, 96 MB at head_dim 64, in groups of equal size.  Measured on B200 (causal): at
  // head_dim 128 larger groups lose once K and V of the whole launch exceed L2 (B32 H16 S4096: 2.12 ms at 40 MB, 2.18 at
  // 96 MB, 2.41 ungrouped; B64 H16 S1024: 0.39 / 0.43 / 0.48 ms); at head_dim 64, where a tile is half as many bytes, 96 MB
  // is about 1 % ahead.  Equal groups matter more than the size: with 64 slices in groups of 20, 20, 20, 4 the last group's
  // heaviest items ran at the very end with few CTAs left to share them (B4 H16 S8192 D64: 0.916 ms, 0.850 in four groups
  // of 16).  IT_FWD_GROUP_MB in the environment overrides the size (A/B runs).
  long long group_mb = (D == 64) ? 96 : 40;
  if (const char* e = getenv("IT_FWD_GROUP_MB")) group_mb = std::max(1, atoi(e));
  {
    // equal groups: a short last group would put its heaviest items at the very end of the launch, with few CTAs left to share them
    const long long gs_max = std::clamp<long long>((group_mb << 20) / (4LL * S * D), 1, BH);
    const long long n_groups = (BH + gs_max - 1) / gs_max;
    p.group_slices = static_cast<int>((BH + n_groups - 1) / n_groups);
  }
  p.dec_tiles_per_split = 0;
  p.dec_n_splits = 1;
  p.dec_part_o = nullptr;
  p.dec_part_ml = nullptr;
  const int n_ctas_per_slice = (S + T::BM * T::QT_PER_CTA - 1) / (T::BM * T::QT_PER_CTA);
  long long grid = static_cast<long long>(n_ctas_per_slice) * BH;
  p.work_counter = nullptr;
  if (!PP && grid > ctx->sm_count) {
    // One CTA per SM; each draws its next work item from a counter (one per stream: launches on a stream run one
    // after the other), zeroed in front of the launch.  IT_FWD_ONE_ITEM_PER_CTA=1 launches one CTA per item instead.
    const char* one = getenv("IT_FWD_ONE_ITEM_PER_CTA");
    if (stream->d_work != nullptr && (one == nullptr || one[0] != '1')) {
      IT_CUDA(cudaMemsetAsync(stream->d_work, 0, sizeof(int), s));
      stream->work_used = true;
      p.work_counter = stream->d_work;
      grid = ctx->sm_count;
    }
  }
  if (ctx->timing >= 2) IT_CUDA(cudaEventRecord(ctx->ev[0][0], s));
  IT_CUDA(launch_dependent(kernel, static_cast<unsigned>(grid), T::THREADS, T::SMEM_BYTES, s, mq, mk, mv, p));
  if (ctx->timing >= 2) {
    IT_CUDA(cudaEventRecord(ctx->ev[0][1], s));
    ctx->ev_valid[0] = true;
  }
  ctx->launches += 1;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

struct BwdWorkspace {
  size_t dq_accum_off, lse2_off, delta_off, total;
  int S_pad;
};
BwdWorkspace bwd_workspace_layout(it_dtype dtype, int64_t BH, int64_t S, int64_t D) {
  BwdWorkspace w{};
  auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
  if (use_sm100_path(dtype, static_cast<int32_t>(S), static_cast<int32_t>(D))) {
    w.S_pad = static_cast<int>((S + 127) / 128 * 128);
    w.dq_accum_off = 0;
    w.lse2_off = up(static_cast<size_t>(BH) * S * D * 4);
    w.delta_off = w.lse2_off + up(static_cast<size_t>(BH) * w.S_pad * 4);
    w.total = w.delta_off + up(static_cast<size_t>(BH) * w.S_pad * 4);
  } else {
    w.S_pad = static_cast<int>(S);
    w.delta_off = 0;
    w.total = up(static_cast<size_t>(BH) * S * 4);
  }
  if (w.total == 0) w.total = 256;
  return w;
}

template <int D>
it_status launch_bwd_sm100(it_ctx* ctx, cudaStream_t s, int B, int H, int S, int causal, const void* q, const void* k,
                           const void* v, const void* o, const void* d_o, const float* lse, void* dq, void* dk,
                           void* dv, uint8_t* ws, const BwdWorkspace& w, const it::TensorStrides& stv,
                           const it::TensorStrides& skv, const it::RopeFreqs& rf, const it::TensorStrides& sq) {
  const int BH = B * H;
  const int Hkv = H / skv.group;
  using T = it::BwdTraits<D>;
  CUtensorMap mq, mk, mv, mdo;
  it_status st;
  if ((st = make_tmap(ctx, &mq, q, B, H, S, D, sq, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mk, k, B, Hkv, S, D, skv, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mv, v, B, Hkv, S, D, skv, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mdo, d_o, B, H, S, D, stv, 128)) != IT_OK) return st;
  // fp32 dQ accumulator [BH, S, D]: boxes of 32 columns x 128 rows for the TMA reduce-add
  CUtensorMap mdq;
  {
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(BH)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 4, static_cast<cuuint64_t>(S) * D * 4};
    const cuuint32_t box[3] = {32, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = ctx->encode(&mdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ws + w.dq_accum_off, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(IT_ERR_CUDA, "cuTensorMapEncodeTiled (dQ accumulator) failed with %d", static_cast<int>(r));
  }
  static std::atomic<bool> attr_set[16];   // zero-initialised; setting an attribute twice is harmless
  if (!attr_set[ctx->device & 15]) {
    IT_CUDA(cudaFuncSetAttribute(it::fa_bwd_sm100_kernel<D, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 it::BwdTraits<D, 1>::SMEM_BYTES));
    if constexpr (D == 64)
      IT_CUDA(cudaFuncSetAttribute(it::fa_bwd_sm100_kernel<D, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   it::BwdTraits<D, 2>::SMEM_BYTES));
    attr_set[ctx->device & 15] = true;
  }
  float* dq_accum = reinterpret_cast<float*>(ws + w.dq_accum_off);
  float* lse2 = reinterpret_cast<float*>(ws + w.lse2_off);
  float* delta = reinterpret_cast<float*>(ws + w.delta_off);
  const size_t n_dq = static_cast<size_t>(BH) * S * D;
  const long long rows_pad = static_cast<long long>(BH) * w.S_pad;
  if (ctx->timing >= 3) IT_CUDA(cudaEventRecord(ctx->ev[2][0], s));
  IT_CUDA(launch_dependent(it::fa_bwd_prepare_kernel<D>, static_cast<unsigned>((rows_pad / 8 + 7) / 8), 256, 0, s,   // 8 rows per warp, 8 warps
                           static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), lse, lse2, delta, dq_accum, S,
                           w.S_pad, BH, stv));
  it::BwdParams p;
  p.st = stv;
  p.st_kv = skv;
  p.lse2_pad = lse2;
  p.delta_pad = delta;
  p.dq_accum = dq_accum;
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.status = ctx->d_status;
  p.S = S;
  p.S_pad = w.S_pad;
  p.BH = BH;
  p.causal = causal;
  p.scale = 1.0f / sqrtf(static_cast<float>(D));
  p.scale_log2 = p.scale * 1.4426950408889634f;
  const int n_kt = (S + 127) / 128;
  // At head_dim 64 a CTA can own two key tiles (tensor memory holds four accumulators of 64 columns): half as many
  // CTAs, so half as many start-ups and epilogues for the same work.  Taken when the launch has CTAs to spare (more
  // than two per SM with one key tile each); a launch that does not even fill the GPU is a latency case and keeps
  // the shorter CTAs.  IT_BWD_KEY_TILES=1 or 2 in the environment overrides the choice (the tests run both forms).
  const char* force = getenv("IT_BWD_KEY_TILES");
  const bool two_tiles = (D == 64) && n_kt >= 2 &&
                         (force != nullptr ? force[0] == '2' : static_cast<long long>(n_kt) * B * Hkv > 2LL * ctx->sm_count);
  if (ctx->timing >= 3) {
    IT_CUDA(cudaEventRecord(ctx->ev[2][1], s));
    ctx->ev_valid[2] = true;
  }
  if (ctx->timing) IT_CUDA(cudaEventRecord(ctx->ev[1][0], s));
  if constexpr (D == 64) {
    if (two_tiles)
      IT_CUDA(launch_dependent(it::fa_bwd_sm100_kernel<D, 2>, static_cast<unsigned>((n_kt + 1) / 2) * B * Hkv, T::THREADS,
                               it::BwdTraits<D, 2>::SMEM_BYTES, s, mq, mk, mv, mdo, mdq, p, rf));
  }
  if (!two_tiles)
    IT_CUDA(launch_dependent(it::fa_bwd_sm100_kernel<D, 1>, static_cast<unsigned>(n_kt) * B * Hkv, T::THREADS, T::SMEM_BYTES, s,
                             mq, mk, mv, mdo, mdq, p, rf));
  if (ctx->timing) {
    IT_CUDA(cudaEventRecord(ctx->ev[1][1], s));
    ctx->ev_valid[1] = true;
  }
  if (ctx->timing >= 3) IT_CUDA(cudaEventRecord(ctx->ev[3][0], s));
  const size_t n4 = n_dq / 4;
  IT_CUDA(launch_dependent(it::fa_bwd_finish_kernel, static_cast<unsigned>((n4 + 255) / 256), 256, 0, s,
                           static_cast<const float*>(dq_accum), static_cast<__nv_bfloat16*>(dq), n4, p.scale, S, D, sq, rf));
  if (ctx->timing >= 3) {
    IT_CUDA(cudaEventRecord(ctx->ev[3][1], s));
    ctx->ev_valid[3] = true;
  }
  ctx->launches += 3;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

constexpr int kDecodeMaxSplits = 64;

// C[M,N] = op(A) op(B) in bf16 with fp32 accumulation.  layout 0: A [M,K], B [N,K]; 1: A [M,K], B [K,N];
// 2: A [K,M], B [K,N].  Row-major, pitches in elements.
struct QkvEpilogue {
  void *q, *k, *v;
  int seq, heads, kv_heads, head_dim;
  const float2* rope_table;
  long long ld_q, ld_kv;
};
struct ScatterEpilogue {
  void* const* c_of_rank;
  int world, rows_per_rank;
};

template <int LAYOUT, bool QKV = false, bool RS = false>
it_status launch_gemm(it_ctx* ctx, cudaStream_t s, int M, int N, int K, const void* a, long long lda, const void* b,
                      long long ldb, void* c, long long ldc, bool c_is_f32, const QkvEpilogue* epi = nullptr,
                      const ScatterEpilogue* rs = nullptr) {
  using T = it::GemmTraits;
  CUtensorMap ma, mb;
  it_status st;
  const int a_rows = (LAYOUT == 2) ? K : M, a_cols = (LAYOUT == 2) ? M : K;
  const int b_rows = (LAYOUT == 0) ? N : K, b_cols = (LAYOUT == 0) ? K : N;
  const it::TensorStrides sa{lda, lda * a_rows, lda * a_rows, 1}, sb{ldb, ldb * b_rows, ldb * b_rows, 1};
  if ((st = make_tmap(ctx, &ma, a, 1, 1, a_rows, a_cols, sa, (LAYOUT == 2) ? T::BK : T::BM)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mb, b, 1, 1, b_rows, b_cols, sb, (LAYOUT == 0) ? T::BN : T::BK)) != IT_OK) return st;
  static std::atomic<bool> attr_set[16];   // zero-initialised; setting an attribute twice is harmless
  if (!attr_set[ctx->device & 15]) {
    IT_CUDA(cudaFuncSetAttribute(it::gemm_bf16_sm100_kernel<LAYOUT, QKV, RS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 T::SMEM_BYTES));
    attr_set[ctx->device & 15] = true;
  }
  it::GemmParams p;
  p.c = c;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.c_is_f32 = c_is_f32 ? 1 : 0;
  p.status = ctx->d_status;
  p.q = p.k = p.v = nullptr;
  p.seq = p.heads = p.kv_heads = p.head_dim = 0;
  p.ld_q = p.ld_kv = 0;
  p.rope_table = nullptr;
  p.rs_world = 0;
  p.rs_rows = 1;
  static const it::GemmScatterMaps no_maps{};
  it::GemmScatterMaps rs_maps;
  if (RS) {
    p.rs_world = rs->world;
    p.rs_rows = rs->rows_per_rank;
    const it::TensorStrides sc{ldc, ldc * M, ldc * M, 1};
    for (int i = 0; i < rs->world; ++i)
      if ((st = make_tmap(ctx, &rs_maps.c_of_rank[i], rs->c_of_rank[i], 1, 1, M, N, sc, T::BM)) != IT_OK) return st;
    for (int i = rs->world; i < 8; ++i) rs_maps.c_of_rank[i] = rs_maps.c_of_rank[0];
  }
  if (epi != nullptr) {
    p.q = static_cast<__nv_bfloat16*>(epi->q);
    p.k = static_cast<__nv_bfloat16*>(epi->k);
    p.v = static_cast<__nv_bfloat16*>(epi->v);
    p.seq = epi->seq;
    p.heads = epi->heads;
    p.kv_heads = epi->kv_heads;
    p.head_dim = epi->head_dim;
    p.rope_table = epi->rope_table;
    p.ld_q = epi->ld_q;
    p.ld_kv = epi->ld_kv;
  }
  const int n_tiles = ((M + T::BM - 1) / T::BM) * ((N + T::BN - 1) / T::BN);
  const int grid = std::min(n_tiles, ctx->sm_count);
  it::gemm_bf16_sm100_kernel<LAYOUT, QKV, RS><<<grid, T::THREADS, T::SMEM_BYTES, s>>>(ma, mb, p, RS ? rs_maps : no_maps);
  ctx->launches += 1;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

it_status check_linear(it_ctx* ctx, it_stream* stream, int32_t n, int32_t in_dim, int32_t out_dim) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (n < 0 || in_dim < 0 || out_dim < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  if ((in_dim & 7) || (out_dim & 7))
    return fail(IT_ERR_UNSUPPORTED_SHAPE, "in and out dimensions must be multiples of 8, got %d and %d", in_dim, out_dim);
  return IT_OK;
}

// Decode on the tensor-core pipeline (bf16, head_dim 64 or 128): the group's query heads are the rows of
// one query tile, the cache is streamed by TMA.  See fa_fwd_pp_sm100.cuh, DECODE.
template <int D>
it_status launch_decode_sm100(it_ctx* ctx, cudaStream_t s, int B, int H, int Hkv, int kv_len, int max_len, const void* q,
                              const void* kc, const void* vc, void* o, float* lse, float* ws) {
  using T = it::FwdPPTraits<D>;
  const int G = H / Hkv;
  const int n_tiles = (kv_len + T::BN - 1) / T::BN;
  const long long base_ctas = static_cast<long long>(B) * Hkv;
  // one CTA per SM runs at a time: split the keys until the GPU is covered, but keep at least four tiles per CTA
  long long want = (ctx->sm_count + base_ctas - 1) / base_ctas;
  want = std::max(1LL, std::min<long long>({want, std::max(1, n_tiles / 4), kDecodeMaxSplits}));
  const int tiles_per_split = static_cast<int>((n_tiles + want - 1) / want);
  const int n_splits = (n_tiles + tiles_per_split - 1) / tiles_per_split;
  CUtensorMap mq, mk, mv;
  it_status st;
  const it::TensorStrides sq{D, static_cast<long long>(G) * D, static_cast<long long>(H) * D, Hkv};
  const it::TensorStrides sc{static_cast<long long>(Hkv) * D, D, static_cast<long long>(max_len) * Hkv * D, Hkv};
  if ((st = make_tmap(ctx, &mq, q, B, Hkv, G, D, sq, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mk, kc, B, Hkv, kv_len, D, sc, 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mv, vc, B, Hkv, kv_len, D, sc, 128)) != IT_OK) return st;
  auto kernel = it::fa_fwd_pp_sm100_kernel<D, true>;
  static std::atomic<bool> attr_set[16];   // zero-initialised; setting an attribute twice is harmless
  if (!attr_set[ctx->device & 15]) {
    IT_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES));
    attr_set[ctx->device & 15] = true;
  }
  it::FwdParams p;
  p.st = it::TensorStrides{D, D, static_cast<long long>(H) * D, H};
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.status = ctx->d_status;
  p.S = kv_len;
  p.BH = B * H;
  p.causal = 0;
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;
  p.kv_group = G;
  p.group_slices = 1;
  p.work_counter = nullptr;
  p.dec_tiles_per_split = tiles_per_split;
  p.dec_n_splits = n_splits;
  p.dec_part_o = ws;
  p.dec_part_ml = ws + static_cast<size_t>(B) * H * n_splits * D;
  IT_CUDA(launch_dependent(kernel, static_cast<unsigned>(base_ctas * n_splits), T::THREADS, T::SMEM_BYTES, s, mq, mk, mv, p));
  ctx->launches += 1;
  if (n_splits > 1) {
    IT_CUDA(launch_dependent(it::fa_decode_merge_kernel<__nv_bfloat16>, static_cast<unsigned>(B * H), 128, 0, s,
                             static_cast<const float*>(p.dec_part_o), static_cast<const float*>(p.dec_part_ml),
                             static_cast<__nv_bfloat16*>(o), lse, n_splits, D));
    ctx->launches += 1;
  }
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

template <typename ST>
it_status launch_decode(it_ctx* ctx, cudaStream_t s, int B, int H, int Hkv, int D, int kv_len, int max_len,
                               const void* q, const void* kc, const void* vc, void* o, float* lse, float* ws) {
  const int G = H / Hkv;
  const int chunks = (G + it::DEC_GC - 1) / it::DEC_GC;
  const long long base_ctas = static_cast<long long>(B) * Hkv * chunks;
  // enough CTAs for about four per SM, no split shorter than 256 keys, at most kDecodeMaxSplits
  long long want = (4LL * ctx->sm_count + base_ctas - 1) / base_ctas;
  want = std::max(1LL, std::min<long long>({want, (kv_len + 255) / 256, kDecodeMaxSplits}));
  int split_len = static_cast<int>((kv_len + want - 1) / want);
  split_len = (split_len + it::DEC_TK - 1) / it::DEC_TK * it::DEC_TK;
  const int n_splits = (kv_len + split_len - 1) / split_len;
  it::DecodeParams p;
  p.H = H;
  p.Hkv = Hkv;
  p.D = D;
  p.kv_len = kv_len;
  p.cache_batch_stride = static_cast<long long>(max_len) * Hkv * D;
  p.n_splits = n_splits;
  p.split_len = split_len;
  p.scale_log2 = (1.0f / sqrtf(static_cast<float>(D))) * 1.4426950408889634f;
  const int pad = 16 / static_cast<int>(sizeof(ST));
  const size_t smem = static_cast<size_t>(it::DEC_GC) * D * 4 + 2ull * it::DEC_TK * (D + pad) * sizeof(ST) +
                      static_cast<size_t>(it::DEC_GC) * it::DEC_TK * 4 + 3 * it::DEC_GC * 4;
  static std::atomic<bool> attr_set[16];   // zero-initialised; setting an attribute twice is harmless
  if (!attr_set[ctx->device & 15]) {
    IT_CUDA(cudaFuncSetAttribute(it::fa_decode_split_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    attr_set[ctx->device & 15] = true;
  }
  float* part_o = ws;
  float* part_ml = ws + static_cast<size_t>(B) * H * n_splits * D;
  const dim3 grid(n_splits, B * Hkv, chunks);
  it::fa_decode_split_kernel<ST><<<grid, it::DEC_THREADS, smem, s>>>(
      static_cast<const ST*>(q), static_cast<const ST*>(kc), static_cast<const ST*>(vc), static_cast<ST*>(o), lse, part_o,
      part_ml, p);
  ctx->launches += 1;
  if (n_splits > 1) {
    it::fa_decode_merge_kernel<ST><<<B * H, 128, 0, s>>>(part_o, part_ml, static_cast<ST*>(o), lse, n_splits, D);
    ctx->launches += 1;
  }
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

}  // namespace

extern "C" {

const char* it_last_error(void) { return g_err; }

it_status it_ctx_create(int device, it_ctx** out) {
  if (out == nullptr) return fail(IT_ERR_INVALID_ARG, "out is null");
  *out = nullptr;
  int count = 0;
  IT_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count) return fail(IT_ERR_CUDA, "CUDA device %d not present (%d visible)", device, count);
  IT_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  IT_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(IT_ERR_CUDA, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                prop.minor);
  it_ctx* c = new (std::nothrow) it_ctx;
  if (c == nullptr) return fail(IT_ERR_CUDA, "out of host memory");
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    delete c;
    return fail(IT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  c->encode = reinterpret_cast<EncodeTiledFn>(fn);
  if (cudaMalloc(&c->d_status, sizeof(int)) != cudaSuccess || cudaMemset(c->d_status, 0, sizeof(int)) != cudaSuccess ||
      cudaMalloc(&c->d_work_pool, it_ctx::WORK_SLOTS * sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&c->h_status, sizeof(int)) != cudaSuccess ||
      cudaStreamCreateWithFlags(&c->status_stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete c;
    return fail(IT_ERR_CUDA, "could not allocate the status word");
  }
  *out = c;
  return IT_OK;
}

it_status it_ctx_destroy(it_ctx* ctx) {
  if (ctx == nullptr) return IT_OK;
  cudaSetDevice(ctx->device);
  cudaFree(ctx->d_status);
  cudaFree(ctx->d_work_pool);
  cudaFreeHost(ctx->h_status);
  if (ctx->status_stream != nullptr) cudaStreamDestroy(ctx->status_stream);
  for (int a = 0; a < 4; ++a)
    for (int b = 0; b < 2; ++b)
      if (ctx->ev[a][b] != nullptr) cudaEventDestroy(ctx->ev[a][b]);
  delete ctx;
  return IT_OK;
}

it_status it_stream_create(it_ctx* ctx, it_stream** out) {
  if (ctx == nullptr || out == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaSetDevice(ctx->device));
  it_stream* s = new (std::nothrow) it_stream;
  if (s == nullptr) return fail(IT_ERR_CUDA, "out of host memory");
  cudaError_t e = cudaStreamCreateWithFlags(&s->s, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete s;
    return fail(IT_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
  }
  s->owned = true;
  s->d_work = take_work_slot(ctx);
  *out = s;
  return IT_OK;
}

it_status it_stream_wrap(it_ctx* ctx, void* cuda_stream, it_stream** out) {
  if (ctx == nullptr || out == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  it_stream* s = new (std::nothrow) it_stream;
  if (s == nullptr) return fail(IT_ERR_CUDA, "out of host memory");
  s->s = static_cast<cudaStream_t>(cuda_stream);
  s->owned = false;
  s->d_work = take_work_slot(ctx);
  *out = s;
  return IT_OK;
}

it_status it_stream_destroy(it_ctx* ctx, it_stream* stream) {
  if (stream == nullptr) return IT_OK;
  if (ctx != nullptr) cudaSetDevice(ctx->device);
  give_work_slot(ctx, stream);
  if (stream->owned) cudaStreamDestroy(stream->s);
  delete stream;
  return IT_OK;
}

it_status it_stream_sync(it_ctx* ctx, it_stream* stream) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaStreamSynchronize(stream->s));
  return fail_if_device_status(ctx);
}

it_status it_event_create(it_ctx* ctx, it_event** out) {
  if (ctx == nullptr || out == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaSetDevice(ctx->device));
  it_event* ev = new (std::nothrow) it_event;
  if (ev == nullptr) return fail(IT_ERR_CUDA, "out of host memory");
  cudaError_t e = cudaEventCreate(&ev->e);
  if (e != cudaSuccess) {
    delete ev;
    return fail(IT_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e));
  }
  *out = ev;
  return IT_OK;
}

it_status it_event_destroy(it_ctx* ctx, it_event* ev) {
  (void)ctx;
  if (ev == nullptr) return IT_OK;
  cudaEventDestroy(ev->e);
  delete ev;
  return IT_OK;
}

it_status it_event_record(it_ctx* ctx, it_stream* stream, it_event* ev) {
  if (ctx == nullptr || stream == nullptr || ev == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaEventRecord(ev->e, stream->s));
  return IT_OK;
}

it_status it_event_query(it_ctx* ctx, it_event* ev, int32_t* done) {
  if (ctx == nullptr || ev == nullptr || done == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  cudaError_t e = cudaEventQuery(ev->e);
  if (e == cudaSuccess) {
    *done = 1;
  } else if (e == cudaErrorNotReady) {
    *done = 0;
  } else {
    return fail(IT_ERR_CUDA, "cudaEventQuery: %s", cudaGetErrorString(e));
  }
  return IT_OK;
}

it_status it_event_wait(it_ctx* ctx, it_event* ev) {
  if (ctx == nullptr || ev == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaEventSynchronize(ev->e));
  return fail_if_device_status(ctx);
}

it_status it_event_elapsed_ms(it_ctx* ctx, it_event* start, it_event* stop, float* ms) {
  if (ctx == nullptr || start == nullptr || stop == nullptr || ms == nullptr)
    return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaEventElapsedTime(ms, start->e, stop->e));
  return IT_OK;
}

it_status it_buf_alloc(it_ctx* ctx, size_t bytes, void** out_dev) {
  if (ctx == nullptr || out_dev == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaSetDevice(ctx->device));
  IT_CUDA(cudaMalloc(out_dev, bytes == 0 ? 1 : bytes));
  return IT_OK;
}

it_status it_buf_free(it_ctx* ctx, void* dev) {
  if (ctx == nullptr) return fail(IT_ERR_INVALID_ARG, "null context");
  if (dev != nullptr) IT_CUDA(cudaFree(dev));
  return IT_OK;
}

it_status it_host_alloc(it_ctx* ctx, size_t bytes, void** out_host) {
  if (ctx == nullptr || out_host == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaSetDevice(ctx->device));
  IT_CUDA(cudaMallocHost(out_host, bytes == 0 ? 1 : bytes));
  return IT_OK;
}

it_status it_host_free(it_ctx* ctx, void* host) {
  if (ctx == nullptr) return fail(IT_ERR_INVALID_ARG, "null context");
  if (host != nullptr) IT_CUDA(cudaFreeHost(host));
  return IT_OK;
}

it_status it_buf_upload(it_ctx* ctx, it_stream* stream, void* dst_dev, const void* src_host, size_t bytes) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (bytes == 0) return IT_OK;
  if (dst_dev == nullptr || src_host == nullptr) return fail(IT_ERR_INVALID_ARG, "null buffer");
  IT_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, stream->s));
  return IT_OK;
}

it_status it_buf_download(it_ctx* ctx, it_stream* stream, void* dst_host, const void* src_dev, size_t bytes) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (bytes == 0) return IT_OK;
  if (dst_host == nullptr || src_dev == nullptr) return fail(IT_ERR_INVALID_ARG, "null buffer");
  IT_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, stream->s));
  return IT_OK;
}

it_status it_buf_memset_async(it_ctx* ctx, it_stream* stream, void* dev, int value, size_t bytes) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (bytes == 0) return IT_OK;
  if (dev == nullptr) return fail(IT_ERR_INVALID_ARG, "null buffer");
  IT_CUDA(cudaMemsetAsync(dev, value, bytes, stream->s));
  return IT_OK;
}

static it_status check_kv_heads(int32_t H, int32_t Hkv) {
  if (Hkv < 1 || Hkv > H || H % Hkv != 0)
    return fail(IT_ERR_INVALID_ARG, "kv_heads must divide heads: heads %d, kv_heads %d", H, Hkv);
  return IT_OK;
}

static it_status attention_fwd_impl(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H, int32_t Hkv,
                                    int32_t S, int32_t D, int32_t causal, const void* q, const void* k, const void* v,
                                    void* o, float* lse, bool bshd, long long qkv_row = 0) {
  it_status st = check_common(ctx, stream, dtype, B, H, S, D);
  if (st != IT_OK) return st;
  if (H > 0 && (st = check_kv_heads(H, Hkv)) != IT_OK) return st;
  const int BH = B * H;
  if (S == 0 || BH == 0) return IT_OK;   // src/ops/flash_attention.rs:102-104, src/ops/attention.rs:313-315
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(IT_ERR_ALIGNMENT, "q, k, v and o must be 16-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  const it::TensorStrides sv = bshd ? strides_bshd(H, S, D) : strides_bhsd(H, S, D);
  it::TensorStrides skv = strides_kv(bshd, H, Hkv, S, D);
  it::TensorStrides sq = sv;
  if (qkv_row != 0) {   // q, k and v are column ranges of one [batch, seq, qkv_row] buffer
    if (!use_sm100_path(dtype, S, D))
      return fail(IT_ERR_UNSUPPORTED_SHAPE, "the packed layout needs bf16, head_dim 64 or 128 and seq >= 128");
    sq.row = skv.row = qkv_row;
    sq.batch = skv.batch = qkv_row * S;
  }
  if (use_sm100_path(dtype, S, D)) {
    // Crossover measured on B200 (causal, head_dim 128): the two-tile kernel wins by 3 % at S = 4096, the one-tile kernel by
    // 1.5 % at 6144 and 6-10 % from 8192 on; the two-tile kernel takes head_dim 64 at every length.
    // IT_FWD_KERNEL=pp|two in the environment overrides the choice (A/B runs).
    const char* force = getenv("IT_FWD_KERNEL");
    const bool pp = (force != nullptr) ? (force[0] == 'p') : ((D == 128) && (S >= 5120));
    if (D == 128)
      return pp ? launch_fwd_sm100<128, true>(ctx, stream, B, H, S, causal != 0, q, k, v, o, lse, sv, skv, sq)
                : launch_fwd_sm100<128, false>(ctx, stream, B, H, S, causal != 0, q, k, v, o, lse, sv, skv, sq);
    return pp ? launch_fwd_sm100<64, true>(ctx, stream, B, H, S, causal != 0, q, k, v, o, lse, sv, skv, sq)
              : launch_fwd_sm100<64, false>(ctx, stream, B, H, S, causal != 0, q, k, v, o, lse, sv, skv, sq);
  }
  return dtype == IT_F32 ? launch_fwd_generic<float>(ctx, stream->s, BH, S, D, causal != 0, q, k, v, o, lse, sv, skv)
                         : launch_fwd_generic<__nv_bfloat16>(ctx, stream->s, BH, S, D, causal != 0, q, k, v, o, lse, sv, skv);
}

it_status it_flash_attention_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H, int32_t S,
                                 int32_t D, int32_t causal, const void* q, const void* k, const void* v, void* o,
                                 float* lse) {
  return attention_fwd_impl(ctx, stream, dtype, B, H, H, S, D, causal, q, k, v, o, lse, false);
}

it_status it_attention_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H, int32_t D,
                           int32_t causal, const void* q, const void* k, const void* v, void* o, float* lse) {
  return attention_fwd_impl(ctx, stream, dtype, B, H, H, S, D, causal, q, k, v, o, lse, true);
}

it_status it_attention_gqa_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H,
                               int32_t Hkv, int32_t D, int32_t causal, const void* q, const void* k, const void* v,
                               void* o, float* lse) {
  return attention_fwd_impl(ctx, stream, dtype, B, H, Hkv, S, D, causal, q, k, v, o, lse, true);
}

it_status it_attention_cross_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t Sq, int32_t Skv, int32_t H,
                                 int32_t D, const void* q, const void* k, const void* v, void* o, float* lse) {
  if (Sq == Skv) return attention_fwd_impl(ctx, stream, dtype, B, H, H, Sq, D, 0, q, k, v, o, lse, true);
  it_status st = check_common(ctx, stream, dtype, B, H, Sq, D);
  if (st != IT_OK) return st;
  if (Skv < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  if (B == 0 || Sq == 0 || Skv == 0 || H == 0) return IT_OK;   // src/ops/attention.rs:313-315: the zeroed output is the caller's
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(IT_ERR_ALIGNMENT, "q, k, v and o must be 16-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  const it::TensorStrides sq = strides_bshd(H, Sq, D), skv = strides_bshd(H, Skv, D);
  return dtype == IT_F32 ? launch_fwd_generic<float>(ctx, stream->s, B * H, Sq, D, 0, q, k, v, o, lse, sq, skv, Skv)
                         : launch_fwd_generic<__nv_bfloat16>(ctx, stream->s, B * H, Sq, D, 0, q, k, v, o, lse, sq, skv, Skv);
}

it_status it_flash_attention_bwd_workspace_bytes(it_dtype dtype, int32_t B, int32_t H, int32_t S, int32_t D,
                                                 size_t* out_bytes) {
  if (out_bytes == nullptr) return fail(IT_ERR_INVALID_ARG, "out_bytes is null");
  if (dtype != IT_F32 && dtype != IT_BF16) return fail(IT_ERR_PRECISION, "dtype %d is not F32 or BF16", (int)dtype);
  if (B < 0 || H < 0 || S < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  if (D < 1 || D > 128) return fail(IT_ERR_UNSUPPORTED_SHAPE, "head_dim must be in 1..128, got %d", D);
  *out_bytes = bwd_workspace_layout(dtype, static_cast<int64_t>(B) * H, S, D).total;
  return IT_OK;
}

static it_status attention_bwd_impl(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H, int32_t Hkv,
                                    int32_t S, int32_t D, int32_t causal, const void* q, const void* k, const void* v,
                                    const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                                    void* workspace, size_t workspace_bytes, bool bshd,
                                    const it::RopeFreqs& rf = make_rope_freqs(0, 1.f, 0, false), long long qkv_row = 0) {
  it_status st = check_common(ctx, stream, dtype, B, H, S, D);
  if (st != IT_OK) return st;
  if (H > 0 && (st = check_kv_heads(H, Hkv)) != IT_OK) return st;
  const int BH = B * H;
  if (S == 0 || BH == 0) return IT_OK;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || d_o == nullptr || lse == nullptr ||
      dq == nullptr || dk == nullptr || dv == nullptr)
    return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv))
    return fail(IT_ERR_ALIGNMENT, "tensors must be 16-byte aligned");
  const BwdWorkspace w = bwd_workspace_layout(dtype, BH, S, D);
  if (workspace == nullptr || workspace_bytes < w.total)
    return fail(IT_ERR_INVALID_ARG, "workspace of %zu bytes needed, %zu given", w.total, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(IT_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const it::TensorStrides sv = bshd ? strides_bshd(H, S, D) : strides_bhsd(H, S, D);
  it::TensorStrides skv = strides_kv(bshd, H, Hkv, S, D);
  it::TensorStrides sq = sv;
  if (qkv_row != 0) {   // q, k, v (and dq, dk, dv) are column ranges of one [batch, seq, qkv_row] buffer each
    if (!use_sm100_path(dtype, S, D))
      return fail(IT_ERR_UNSUPPORTED_SHAPE, "the packed layout needs bf16, head_dim 64 or 128 and seq >= 128");
    sq.row = skv.row = qkv_row;
    sq.batch = skv.batch = qkv_row * S;
  }
  if (use_sm100_path(dtype, S, D)) {
    return D == 128
               ? launch_bwd_sm100<128>(ctx, stream->s, B, H, S, causal != 0, q, k, v, o, d_o, lse, dq, dk, dv, ws, w, sv, skv, rf, sq)
               : launch_bwd_sm100<64>(ctx, stream->s, B, H, S, causal != 0, q, k, v, o, d_o, lse, dq, dk, dv, ws, w, sv, skv, rf, sq);
  }
  float* delta = reinterpret_cast<float*>(ws + w.delta_off);
  return dtype == IT_F32
             ? launch_bwd_generic<float>(ctx, stream->s, BH, S, D, causal != 0, q, k, v, o, d_o, lse, dq, dk, dv, delta, sv, skv, rf)
             : launch_bwd_generic<__nv_bfloat16>(ctx, stream->s, BH, S, D, causal != 0, q, k, v, o, d_o, lse, dq, dk, dv, delta,
                                                 sv, skv, rf);
}

it_status it_flash_attention_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H, int32_t S,
                                 int32_t D, int32_t causal, const void* q, const void* k, const void* v, const void* o,
                                 const void* d_o, const float* lse, void* dq, void* dk, void* dv, void* workspace,
                                 size_t workspace_bytes) {
  return attention_bwd_impl(ctx, stream, dtype, B, H, H, S, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, workspace,
                            workspace_bytes, false);
}

it_status it_attention_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H, int32_t D,
                           int32_t causal, const void* q, const void* k, const void* v, const void* o, const void* d_o,
                           const float* lse, void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes) {
  return attention_bwd_impl(ctx, stream, dtype, B, H, H, S, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, workspace,
                            workspace_bytes, true);
}

it_status it_attention_gqa_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H,
                               int32_t Hkv, int32_t D, int32_t causal, const void* q, const void* k, const void* v,
                               const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                               void* workspace, size_t workspace_bytes) {
  return attention_bwd_impl(ctx, stream, dtype, B, H, Hkv, S, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, workspace,
                            workspace_bytes, true);
}

it_status it_attention_packed_fwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H,
                                  int32_t Hkv, int32_t D, int32_t causal, const void* qkv, void* o, float* lse) {
  if (qkv == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (dtype != IT_BF16) return fail(IT_ERR_PRECISION, "the packed layout is bf16 only");
  const long long row = (static_cast<long long>(H) + 2LL * Hkv) * D;
  const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(qkv);
  return attention_fwd_impl(ctx, stream, dtype, B, H, Hkv, S, D, causal, base, base + static_cast<long long>(H) * D,
                            base + (static_cast<long long>(H) + Hkv) * D, o, lse, true, row);
}

static it_status check_rope(int32_t D, float base) {
  if (D < 2 || D > 128 || (D & 1)) return fail(IT_ERR_UNSUPPORTED_SHAPE, "rotary embedding needs an even head_dim in 2..128, got %d", D);
  if (!(base > 0.f)) return fail(IT_ERR_INVALID_ARG, "rotary base must be positive");
  return IT_OK;
}

it_status it_attention_gqa_bwd_rope(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H,
                                    int32_t Hkv, int32_t D, int32_t causal, float rope_base, int32_t position_offset,
                                    const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                    const float* lse, void* dq, void* dk, void* dv, void* workspace,
                                    size_t workspace_bytes) {
  it_status st = check_rope(D, rope_base);
  if (st != IT_OK) return st;
  return attention_bwd_impl(ctx, stream, dtype, B, H, Hkv, S, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, workspace,
                            workspace_bytes, true, make_rope_freqs(D, rope_base, position_offset, true));
}

it_status it_attention_packed_bwd(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H,
                                  int32_t Hkv, int32_t D, int32_t causal, float rope_base, int32_t position_offset,
                                  const void* qkv, const void* o, const void* d_o, const float* lse, void* dqkv,
                                  void* workspace, size_t workspace_bytes) {
  if (qkv == nullptr || dqkv == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (dtype != IT_BF16) return fail(IT_ERR_PRECISION, "the packed layout is bf16 only");
  it_status st;
  if (rope_base != 0.f && (st = check_rope(D, rope_base)) != IT_OK) return st;
  const long long row = (static_cast<long long>(H) + 2LL * Hkv) * D;
  const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(qkv);
  __nv_bfloat16* gbase = static_cast<__nv_bfloat16*>(dqkv);
  const long long ko = static_cast<long long>(H) * D, vo = (static_cast<long long>(H) + Hkv) * D;
  return attention_bwd_impl(ctx, stream, dtype, B, H, Hkv, S, D, causal, base, base + ko, base + vo, o, d_o, lse, gbase,
                            gbase + ko, gbase + vo, workspace, workspace_bytes, true,
                            make_rope_freqs(D, rope_base == 0.f ? 1.f : rope_base, position_offset, rope_base != 0.f), row);
}

it_status it_rope_qk(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t S, int32_t H, int32_t Hkv,
                     int32_t D, float rope_base, int32_t position_offset, int32_t inverse, const void* q_in,
                     const void* k_in, void* q_out, void* k_out) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (dtype != IT_F32 && dtype != IT_BF16) return fail(IT_ERR_PRECISION, "dtype %d is not F32 or BF16", (int)dtype);
  if (B < 0 || S < 0 || H < 0 || Hkv < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  it_status st = check_rope(D, rope_base);
  if (st != IT_OK) return st;
  if (static_cast<int64_t>(B) * S == 0 || H + Hkv == 0) return IT_OK;
  if (H > 0 && (q_in == nullptr || q_out == nullptr)) return fail(IT_ERR_INVALID_ARG, "null q tensor");
  if (Hkv > 0 && (k_in == nullptr || k_out == nullptr)) return fail(IT_ERR_INVALID_ARG, "null k tensor");
  IT_CUDA(cudaSetDevice(ctx->device));
  const it::RopeFreqs rf = make_rope_freqs(D, rope_base, position_offset, true);
  const int half = D / 2;
  const int n_heads = H + Hkv;
  const int threads = half * std::max(1, std::min(n_heads, 256 / half));
  const unsigned grid = static_cast<unsigned>(static_cast<int64_t>(B) * S);
  const void* kin = Hkv > 0 ? k_in : nullptr;
#define IT_ROPE_LAUNCH(ST, INV)                                                                                   \
  it::rope_qk_kernel<ST, INV><<<grid, threads, 0, stream->s>>>(static_cast<const ST*>(q_in), static_cast<const ST*>(kin), \
                                                               static_cast<ST*>(q_out), static_cast<ST*>(k_out), S, H, Hkv, D, rf)
  if (dtype == IT_F32) {
    if (inverse) IT_ROPE_LAUNCH(float, true); else IT_ROPE_LAUNCH(float, false);
  } else {
    if (inverse) IT_ROPE_LAUNCH(__nv_bfloat16, true); else IT_ROPE_LAUNCH(__nv_bfloat16, false);
  }
#undef IT_ROPE_LAUNCH
  ctx->launches += 1;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

it_status it_attention_decode_workspace_bytes(int32_t B, int32_t H, int32_t D, size_t* out_bytes) {
  if (out_bytes == nullptr) return fail(IT_ERR_INVALID_ARG, "out_bytes is null");
  if (B < 0 || H < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  if (D < 1 || D > 128) return fail(IT_ERR_UNSUPPORTED_SHAPE, "head_dim must be in 1..128, got %d", D);
  const size_t n = static_cast<size_t>(B) * H * kDecodeMaxSplits * (static_cast<size_t>(D) + 2) * sizeof(float);
  *out_bytes = (n + 255) / 256 * 256 + 256;
  return IT_OK;
}

it_status it_attention_decode(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H, int32_t Hkv,
                              int32_t D, int32_t kv_len, int32_t max_len, const void* q, const void* k_cache,
                              const void* v_cache, void* o, float* lse, void* workspace, size_t workspace_bytes) {
  it_status st = check_common(ctx, stream, dtype, B, H, 0, D);
  if (st != IT_OK) return st;
  if (H > 0 && (st = check_kv_heads(H, Hkv)) != IT_OK) return st;
  if (kv_len < 1 || max_len < kv_len) return fail(IT_ERR_INVALID_ARG, "need 1 <= kv_len <= max_len, got %d, %d", kv_len, max_len);
  if (D % 8 != 0) return fail(IT_ERR_UNSUPPORTED_SHAPE, "decode needs head_dim a multiple of 8, got %d", D);
  if (B == 0 || H == 0) return IT_OK;
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || o == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(o))
    return fail(IT_ERR_ALIGNMENT, "q, caches and o must be 16-byte aligned");
  size_t need = 0;
  it_attention_decode_workspace_bytes(B, H, D, &need);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(IT_ERR_INVALID_ARG, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(IT_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  float* ws = static_cast<float*>(workspace);
  if (dtype == IT_BF16 && (D == 64 || D == 128) && H / Hkv <= 128 && kv_len >= 256)
    return D == 128 ? launch_decode_sm100<128>(ctx, stream->s, B, H, Hkv, kv_len, max_len, q, k_cache, v_cache, o, lse, ws)
                    : launch_decode_sm100<64>(ctx, stream->s, B, H, Hkv, kv_len, max_len, q, k_cache, v_cache, o, lse, ws);
  return dtype == IT_F32 ? launch_decode<float>(ctx, stream->s, B, H, Hkv, D, kv_len, max_len, q, k_cache, v_cache, o, lse, ws)
                         : launch_decode<__nv_bfloat16>(ctx, stream->s, B, H, Hkv, D, kv_len, max_len, q, k_cache, v_cache, o,
                                                        lse, ws);
}

it_status it_linear_fwd(it_ctx* ctx, it_stream* stream, int32_t n, int32_t in_dim, int32_t out_dim, const void* x,
                        const void* w, void* y) {
  it_status st = check_linear(ctx, stream, n, in_dim, out_dim);
  if (st != IT_OK) return st;
  if (n == 0 || out_dim == 0) return IT_OK;
  if (x == nullptr || w == nullptr || y == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return fail(IT_ERR_ALIGNMENT, "x, w and y must be 16-byte aligned");
  if (in_dim == 0) {
    IT_CUDA(cudaMemsetAsync(y, 0, static_cast<size_t>(n) * out_dim * 2, stream->s));
    return IT_OK;
  }
  IT_CUDA(cudaSetDevice(ctx->device));
  return launch_gemm<0>(ctx, stream->s, n, out_dim, in_dim, x, in_dim, w, in_dim, y, out_dim, false);
}

it_status it_linear_scatter_add(it_ctx* ctx, it_stream* stream, int32_t kind, int32_t n, int32_t in_dim, int32_t out_dim,
                                const void* a, const void* w, void* const* c_of_rank, int32_t world, int32_t rows_per_rank) {
  it_status st = check_linear(ctx, stream, n, in_dim, out_dim);
  if (st != IT_OK) return st;
  if (kind != 0 && kind != 1) return fail(IT_ERR_INVALID_ARG, "kind must be 0 (a W^T) or 1 (a W)");
  if (world < 1 || world > 8) return fail(IT_ERR_INVALID_ARG, "world must be in 1..8, got %d", world);
  if (rows_per_rank < 1 || static_cast<int64_t>(rows_per_rank) * world < n)
    return fail(IT_ERR_INVALID_ARG, "rows_per_rank * world must cover the %d rows", n);
  if (c_of_rank == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  // kind 0: a [n, in] W [out, in] -> [n, out];  kind 1: a [n, out] W [out, in] -> [n, in]
  const int k_dim = kind == 0 ? in_dim : out_dim, c_cols = kind == 0 ? out_dim : in_dim;
  if (n == 0 || c_cols == 0 || k_dim == 0) return IT_OK;   // nothing to add
  if (c_cols % 64 != 0 || rows_per_rank % 128 != 0)
    return fail(IT_ERR_UNSUPPORTED_SHAPE,
                "the summed product's width must be a multiple of 64 and rows_per_rank a multiple of 128, got %d and %d", c_cols,
                rows_per_rank);
  if (a == nullptr || w == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(a) || !aligned16(w)) return fail(IT_ERR_ALIGNMENT, "tensors must be 16-byte aligned");
  for (int r = 0; r < world; ++r) {
    if (c_of_rank[r] == nullptr) return fail(IT_ERR_INVALID_ARG, "null result pointer for rank %d", r);
    if (!aligned16(c_of_rank[r])) return fail(IT_ERR_ALIGNMENT, "result pointers must be 16-byte aligned");
  }
  IT_CUDA(cudaSetDevice(ctx->device));
  const ScatterEpilogue rs{c_of_rank, world, rows_per_rank};
  return kind == 0 ? launch_gemm<0, false, true>(ctx, stream->s, n, out_dim, in_dim, a, in_dim, w, in_dim, nullptr, out_dim, false, nullptr, &rs)
                   : launch_gemm<1, false, true>(ctx, stream->s, n, in_dim, out_dim, a, out_dim, w, in_dim, nullptr, in_dim, false, nullptr, &rs);
}

it_status it_qkv_rope_workspace_bytes(int32_t S, int32_t D, size_t* out_bytes) {
  if (out_bytes == nullptr) return fail(IT_ERR_INVALID_ARG, "out_bytes is null");
  if (S < 0 || D < 2 || D > 128 || (D & 1)) return fail(IT_ERR_INVALID_ARG, "bad seq or head_dim");
  *out_bytes = (static_cast<size_t>(S) * (D / 2) * sizeof(float2) + 255) / 256 * 256 + 256;
  return IT_OK;
}

it_status it_qkv_rope_fwd(it_ctx* ctx, it_stream* stream, int32_t B, int32_t S, int32_t hidden, int32_t H, int32_t Hkv,
                          int32_t D, float rope_base, int32_t position_offset, const void* x, const void* w_qkv,
                          void* q_out, void* k_out, void* v_out, void* workspace, size_t workspace_bytes) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null context or stream");
  if (B < 0 || S < 0 || hidden < 1 || H < 1) return fail(IT_ERR_INVALID_ARG, "bad dimension");
  it_status st = check_kv_heads(H, Hkv);
  if (st != IT_OK) return st;
  if (D != 32 && D != 64 && D != 96 && D != 128)
    return fail(IT_ERR_UNSUPPORTED_SHAPE, "head_dim must be 32, 64, 96 or 128 for the fused projection, got %d", D);
  if (hidden & 7) return fail(IT_ERR_UNSUPPORTED_SHAPE, "hidden must be a multiple of 8, got %d", hidden);
  if (rope_base != 0.f && (st = check_rope(D, rope_base)) != IT_OK) return st;
  const long long n = static_cast<long long>(B) * S;
  if (n == 0) return IT_OK;
  if (n > 0x7fffffffLL) return fail(IT_ERR_UNSUPPORTED_SHAPE, "too many tokens");
  const bool packed = (k_out == nullptr && v_out == nullptr);   // q_out is then [batch, seq, (heads + 2 kv_heads) * head_dim]
  if (x == nullptr || w_qkv == nullptr || q_out == nullptr || (!packed && (k_out == nullptr || v_out == nullptr)))
    return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(x) || !aligned16(w_qkv) || !aligned16(q_out) || !aligned16(k_out) || !aligned16(v_out))
    return fail(IT_ERR_ALIGNMENT, "tensors must be 16-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  const float2* table = nullptr;
  if (rope_base != 0.f) {
    size_t need = 0;
    it_qkv_rope_workspace_bytes(S, D, &need);
    if (workspace == nullptr || workspace_bytes < need)
      return fail(IT_ERR_INVALID_ARG, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(IT_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    const int cells = S * (D / 2);
    it::rope_table_kernel<<<(cells + 255) / 256, 256, 0, stream->s>>>(static_cast<float2*>(workspace), S, D / 2,
                                                                      make_rope_freqs(D, rope_base, position_offset, true));
    ctx->launches += 1;
    table = static_cast<const float2*>(workspace);
  }
  const int out_dim = (H + 2 * Hkv) * D;
  QkvEpilogue epi{q_out, k_out, v_out, S, H, Hkv, D, table, static_cast<long long>(H) * D, static_cast<long long>(Hkv) * D};
  if (packed) {
    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(q_out);
    epi.k = base + static_cast<long long>(H) * D;
    epi.v = base + (static_cast<long long>(H) + Hkv) * D;
    epi.ld_q = epi.ld_kv = out_dim;
  }
  return launch_gemm<0, true>(ctx, stream->s, static_cast<int>(n), out_dim, hidden, x, hidden, w_qkv, hidden, nullptr, 0,
                              false, &epi);
}

it_status it_linear_bwd(it_ctx* ctx, it_stream* stream, int32_t n, int32_t in_dim, int32_t out_dim, const void* dy,
                        const void* x, const void* w, void* dx, float* dw) {
  it_status st = check_linear(ctx, stream, n, in_dim, out_dim);
  if (st != IT_OK) return st;
  if (in_dim == 0 || (n == 0 && out_dim == 0)) return IT_OK;
  if ((dx && !aligned16(dx)) || (dw && !aligned16(dw))) return fail(IT_ERR_ALIGNMENT, "tensors must be 16-byte aligned");
  if (n == 0 || out_dim == 0) {   // empty sums: dy and x (n == 0) or dy and w (out_dim == 0) are empty and may be null
    IT_CUDA(cudaSetDevice(ctx->device));
    if (dx && n) IT_CUDA(cudaMemsetAsync(dx, 0, static_cast<size_t>(n) * in_dim * 2, stream->s));
    if (dw && out_dim) IT_CUDA(cudaMemsetAsync(dw, 0, static_cast<size_t>(out_dim) * in_dim * 4, stream->s));
    return IT_OK;
  }
  if (dy == nullptr || x == nullptr || w == nullptr) return fail(IT_ERR_INVALID_ARG, "null tensor");
  if (!aligned16(dy) || !aligned16(x) || !aligned16(w)) return fail(IT_ERR_ALIGNMENT, "tensors must be 16-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  if (dx != nullptr &&
      (st = launch_gemm<1>(ctx, stream->s, n, in_dim, out_dim, dy, out_dim, w, in_dim, dx, in_dim, false)) != IT_OK)
    return st;
  if (dw != nullptr &&
      (st = launch_gemm<2>(ctx, stream->s, out_dim, in_dim, n, dy, out_dim, x, in_dim, dw, in_dim, true)) != IT_OK)
    return st;
  return IT_OK;
}

// Scratch for it_flash_attention_bwd_noalloc: part of the module image on every GPU that loads it.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[IT_NOALLOC_SCRATCH_BYTES];
static std::mutex g_noalloc_mutex;
static void* g_noalloc_ptr[64] = {};   // device address of the array, per device ordinal

it_status it_flash_attention_bwd_noalloc(it_ctx* ctx, it_stream* stream, it_dtype dtype, int32_t B, int32_t H,
                                         int32_t S, int32_t D, int32_t causal, const void* q, const void* k,
                                         const void* v, const void* o, const void* d_o, const float* lse, void* dq,
                                         void* dk, void* dv) {
  it_status st = check_common(ctx, stream, dtype, B, H, S, D);
  if (st != IT_OK) return st;
  if (S == 0 || B * H == 0) return IT_OK;
  const size_t need = bwd_workspace_layout(dtype, static_cast<int64_t>(B) * H, S, D).total;
  if (need > IT_NOALLOC_SCRATCH_BYTES)
    return fail(IT_ERR_UNSUPPORTED_SHAPE,
                "this shape needs %zu bytes of scratch; the built-in scratch of the allocation-free backward holds %u",
                need, static_cast<unsigned>(IT_NOALLOC_SCRATCH_BYTES));
  if (ctx->device < 0 || ctx->device >= 64) return fail(IT_ERR_INVALID_ARG, "device ordinal %d out of range", ctx->device);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[ctx->device] == nullptr) {
      // once per device, with that device current
      IT_CUDA(cudaSetDevice(ctx->device));
      void* p = nullptr;
      IT_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
      if (p == nullptr) return fail(IT_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
      g_noalloc_ptr[ctx->device] = p;
    }
    scratch = g_noalloc_ptr[ctx->device];
  }
  // The regular entry point clears the dQ accumulator and rewrites the per-row arrays on every call,
  // so nothing left in the array by an earlier call is read.
  return it_flash_attention_bwd(ctx, stream, dtype, B, H, S, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, scratch,
                                IT_NOALLOC_SCRATCH_BYTES);
}

it_status it_host_step_destroy(it_host_step* hs) {
  if (hs == nullptr) return IT_OK;
  if (hs->ctx != nullptr) cudaSetDevice(hs->ctx->device);
  for (int i = 0; i < it_host_step::MAX_STREAMS; ++i) {
    if (hs->streams[i].s != nullptr) {
      cudaStreamSynchronize(hs->streams[i].s);
      give_work_slot(hs->ctx, &hs->streams[i]);
      cudaStreamDestroy(hs->streams[i].s);
    }
    if (hs->done[i] != nullptr) cudaEventDestroy(hs->done[i]);
    if (hs->dev[i] != nullptr) cudaFree(hs->dev[i]);
  }
  if (hs->start != nullptr) cudaEventDestroy(hs->start);
  delete hs;
  return IT_OK;
}

it_status it_host_step_create(it_ctx* ctx, it_dtype dtype, int32_t group_slices, int32_t S, int32_t D, int32_t causal,
                              int32_t n_streams, it_host_step** out) {
  if (ctx == nullptr || out == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  *out = nullptr;
  if (dtype != IT_F32 && dtype != IT_BF16) return fail(IT_ERR_PRECISION, "dtype %d is not F32 or BF16", (int)dtype);
  if (group_slices < 1 || group_slices > 65535 || S < 1) return fail(IT_ERR_INVALID_ARG, "bad group size or sequence length");
  if (D < 1 || D > 128) return fail(IT_ERR_UNSUPPORTED_SHAPE, "head_dim must be in 1..128, got %d", D);
  if (n_streams < 1 || n_streams > it_host_step::MAX_STREAMS)
    return fail(IT_ERR_INVALID_ARG, "n_streams must be in 1..%d", it_host_step::MAX_STREAMS);
  IT_CUDA(cudaSetDevice(ctx->device));
  it_host_step* hs = new (std::nothrow) it_host_step;
  if (hs == nullptr) return fail(IT_ERR_CUDA, "out of host memory");
  hs->ctx = ctx;
  hs->dtype = dtype;
  hs->group_slices = group_slices;
  hs->S = S;
  hs->D = D;
  hs->causal = causal != 0;
  hs->n_streams = n_streams;
  auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
  hs->tensor_bytes = up(static_cast<size_t>(group_slices) * S * D * (dtype == IT_F32 ? 4 : 2));
  hs->lse_bytes = up(static_cast<size_t>(group_slices) * S * 4);
  hs->ws_bytes = bwd_workspace_layout(dtype, group_slices, S, D).total;
  const size_t per_stream = 8 * hs->tensor_bytes + hs->lse_bytes + hs->ws_bytes;
  cudaError_t e = cudaEventCreateWithFlags(&hs->start, cudaEventDisableTiming);
  for (int i = 0; i < n_streams && e == cudaSuccess; ++i) {
    e = cudaStreamCreateWithFlags(&hs->streams[i].s, cudaStreamNonBlocking);
    if (e == cudaSuccess) hs->streams[i].d_work = take_work_slot(ctx);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&hs->done[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&hs->dev[i]), per_stream);
  }
  if (e != cudaSuccess) {
    it_host_step_destroy(hs);
    return fail(IT_ERR_CUDA, "it_host_step_create: %s", cudaGetErrorString(e));
  }
  *out = hs;
  return IT_OK;
}

it_status it_host_step_run(it_host_step* hs, it_stream* stream, int32_t n_slices, const void* hq, const void* hk,
                           const void* hv, const void* hdo, void* ho, float* hlse, void* hdq, void* hdk, void* hdv,
                           int32_t copies_only) {
  if (hs == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  if (n_slices < 0) return fail(IT_ERR_INVALID_ARG, "negative dimension");
  if (n_slices == 0) return IT_OK;
  if (hq == nullptr || hk == nullptr || hv == nullptr || hdo == nullptr || ho == nullptr || hdq == nullptr || hdk == nullptr ||
      hdv == nullptr)
    return fail(IT_ERR_INVALID_ARG, "null tensor");
  it_ctx* ctx = hs->ctx;
  IT_CUDA(cudaSetDevice(ctx->device));
  const size_t esz = hs->dtype == IT_F32 ? 4 : 2;
  const size_t slice_bytes = static_cast<size_t>(hs->S) * hs->D * esz;
  // the groups start after what the caller's stream has enqueued so far (the host tensors may be results of it)
  IT_CUDA(cudaEventRecord(hs->start, stream->s));
  int used = 0;
  for (int32_t b0 = 0, g = 0; b0 < n_slices; b0 += hs->group_slices, ++g) {
    const int32_t n = std::min(hs->group_slices, n_slices - b0);
    const int si = g % hs->n_streams;
    used = std::max(used, si + 1);
    it_stream* st = &hs->streams[si];
    uint8_t* base = hs->dev[si];
    uint8_t* d[8];
    for (int i = 0; i < 8; ++i) d[i] = base + i * hs->tensor_bytes;   // q k v dO o dq dk dv
    float* dlse = reinterpret_cast<float*>(base + 8 * hs->tensor_bytes);
    void* ws = base + 8 * hs->tensor_bytes + hs->lse_bytes;
    const size_t bytes = n * slice_bytes, off = b0 * slice_bytes;
    if (g < hs->n_streams) IT_CUDA(cudaStreamWaitEvent(st->s, hs->start, 0));
    const void* src[4] = {hq, hk, hv, hdo};
    for (int i = 0; i < 4; ++i)
      IT_CUDA(cudaMemcpyAsync(d[i], static_cast<const uint8_t*>(src[i]) + off, bytes, cudaMemcpyHostToDevice, st->s));
    if (!copies_only) {
      it_status rc = it_flash_attention_fwd(ctx, st, hs->dtype, 1, n, hs->S, hs->D, hs->causal, d[0], d[1], d[2], d[4], dlse);
      if (rc != IT_OK) return rc;
      rc = it_flash_attention_bwd(ctx, st, hs->dtype, 1, n, hs->S, hs->D, hs->causal, d[0], d[1], d[2], d[4], d[3], dlse, d[5],
                                  d[6], d[7], ws, hs->ws_bytes);
      if (rc != IT_OK) return rc;
    }
    void* dst[4] = {ho, hdq, hdk, hdv};
    const int from[4] = {4, 5, 6, 7};
    for (int i = 0; i < 4; ++i)
      IT_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(dst[i]) + off, d[from[i]], bytes, cudaMemcpyDeviceToHost, st->s));
    if (hlse != nullptr)
      IT_CUDA(cudaMemcpyAsync(hlse + static_cast<size_t>(b0) * hs->S, dlse, static_cast<size_t>(n) * hs->S * 4,
                              cudaMemcpyDeviceToHost, st->s));
  }
  for (int i = 0; i < used; ++i) {   // the caller's stream continues when every group has been downloaded
    IT_CUDA(cudaEventRecord(hs->done[i], hs->streams[i].s));
    IT_CUDA(cudaStreamWaitEvent(stream->s, hs->done[i], 0));
  }
  return IT_OK;
}

it_status it_attention_status_poll(it_ctx* ctx, it_stream* stream, int32_t* device_status) {
  if (ctx == nullptr || stream == nullptr || device_status == nullptr)
    return fail(IT_ERR_INVALID_ARG, "null argument");
  IT_CUDA(cudaStreamSynchronize(stream->s));
  int word = 0;
  it_status rc = read_device_status(ctx, &word);
  if (rc != IT_OK) return rc;
  *device_status = word;
  if (*device_status != 0) {
    IT_CUDA(cudaMemsetAsync(ctx->d_status, 0, sizeof(int), stream->s));
    IT_CUDA(cudaStreamSynchronize(stream->s));
    return fail(IT_ERR_TIMEOUT, "a bounded wait inside a kernel ran out (device status %d)", *device_status);
  }
  return IT_OK;
}

it_status it_ctx_check_status(it_ctx* ctx, int32_t* device_status) {
  if (ctx == nullptr) return fail(IT_ERR_INVALID_ARG, "null context");
  int word = 0;
  it_status rc = read_device_status(ctx, &word);
  if (rc != IT_OK) return rc;
  if (device_status != nullptr) *device_status = word;
  return word == 0 ? IT_OK : fail_if_device_status(ctx);
}

it_status it_ctx_enable_kernel_timing(it_ctx* ctx, int32_t enable) {
  if (ctx == nullptr) return fail(IT_ERR_INVALID_ARG, "null context");
  IT_CUDA(cudaSetDevice(ctx->device));
  if (enable && ctx->ev[0][0] == nullptr) {
    for (int a = 0; a < 4; ++a)
      for (int b = 0; b < 2; ++b) IT_CUDA(cudaEventCreate(&ctx->ev[a][b]));
  }
  ctx->timing = enable < 0 ? 0 : (enable > 3 ? 3 : enable);
  return IT_OK;
}

it_status it_ctx_kernel_ms(it_ctx* ctx, int32_t which, float* ms) {
  if (ctx == nullptr || ms == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  if (which < 0 || which > 3)
    return fail(IT_ERR_INVALID_ARG, "which must be 0 (forward), 1 (backward main), 2 (backward prepare) or 3 (backward finish)");
  if (!ctx->ev_valid[which]) return fail(IT_ERR_INVALID_ARG, "no timed launch of that kernel yet");
  IT_CUDA(cudaEventSynchronize(ctx->ev[which][1]));
  IT_CUDA(cudaEventElapsedTime(ms, ctx->ev[which][0], ctx->ev[which][1]));
  return IT_OK;
}

const char* it_ctx_kernel_tag(int32_t which) {
  // The reference's profiler names (src/ops/flash_attention.rs:77; src/train/helpers.rs:126-183) for what each timer covers.
  switch (which) {
    case 0: return "FlashAttention";
    case 1: return "attn_bwd/recompute+grad_v+grad_p+grad_qk";
    case 2: return "attn_bwd/prepare";
    case 3: return "attn_bwd/finish";
    default: return "";
  }
}

it_status it_ctx_launch_count(it_ctx* ctx, uint64_t* out) {
  if (ctx == nullptr || out == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  *out = ctx->launches.load();
  return IT_OK;
}

it_status it_selftest_umma(it_ctx* ctx, it_stream* stream, int32_t variant, const void* a_bf16, const void* b_bf16,
                           float* out) {
  if (ctx == nullptr || stream == nullptr || a_bf16 == nullptr || b_bf16 == nullptr || out == nullptr)
    return fail(IT_ERR_INVALID_ARG, "null argument");
  if (variant < 0 || variant > 3) return fail(IT_ERR_INVALID_ARG, "variant must be 0..3");
  if (!aligned16(a_bf16) || !aligned16(b_bf16)) return fail(IT_ERR_ALIGNMENT, "operands must be 16-byte aligned");
  IT_CUDA(cudaSetDevice(ctx->device));
  CUtensorMap ma, mb;
  it_status st;
  if ((st = make_tmap(ctx, &ma, a_bf16, 1, 1, 128, 128, strides_bhsd(1, 128, 128), 128)) != IT_OK) return st;
  if ((st = make_tmap(ctx, &mb, b_bf16, 1, 1, 128, 128, strides_bhsd(1, 128, 128), 128)) != IT_OK) return st;
  const int smem = 4 * 128 * 128 + 64;
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(a_bf16);
#define IT_SELFTEST_CASE(V)                                                                                     \
  case V:                                                                                                       \
    IT_CUDA(cudaFuncSetAttribute(it::umma_selftest_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    it::umma_selftest_kernel<V><<<1, 128, smem, stream->s>>>(ma, mb, a, out, ctx->d_status);                    \
    break;
  switch (variant) {
    IT_SELFTEST_CASE(0)
    IT_SELFTEST_CASE(1)
    IT_SELFTEST_CASE(2)
    IT_SELFTEST_CASE(3)
  }
#undef IT_SELFTEST_CASE
  ctx->launches += 1;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

it_status it_selftest_wait_timeout(it_ctx* ctx, it_stream* stream, int32_t limit_ms) {
  if (ctx == nullptr || stream == nullptr) return fail(IT_ERR_INVALID_ARG, "null argument");
  if (limit_ms < 1 || limit_ms > 1000) return fail(IT_ERR_INVALID_ARG, "limit_ms must be in 1..1000");
  IT_CUDA(cudaSetDevice(ctx->device));
  it::wait_timeout_selftest_kernel<<<1, 32, 0, stream->s>>>(ctx->d_status,
                                                           static_cast<unsigned long long>(limit_ms) * 1000000ull);
  ctx->launches += 1;
  IT_CUDA(cudaGetLastError());
  return IT_OK;
}

}  // extern "C"
