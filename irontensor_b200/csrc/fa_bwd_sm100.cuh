// Fused attention backward (dQ, dK, dV from Q, K, V, O, dO, LSE) for bf16 inputs on sm_100a.
//
// Replaces the reference project's 13-step composed backward (src/train/helpers.rs:142-182: five
// batched GEMMs, four transposes, scale, mask, softmax, softmax-backward, eight S x S
// intermediates per head) with three launches and no S x S traffic:
//   1. fa_bwd_prepare_kernel : delta = rowsum(dO * O) (equal to the reference's rowsum(dP * P),
//                              src/shaders/backward/softmax.metal:35-38) and LSE*log2(e), both
//                              padded to a multiple of 128 rows per head.
//   2. fa_bwd_sm100_kernel   : one CTA per 128-key tile of one (batch, head); loops over the query
//                              tiles that can see it.  Everything is computed transposed so that
//                              keys sit on TMEM lanes:
//                                S^T = K Q^T          P^T = 2^(S^T*c - LSE*log2e)
//                                dP^T = V dO^T        dS^T = P^T o (dP^T - delta)
//                                dV += P^T dO         dK += dS^T Q         dQ_i = dS K
//                              P^T feeds its MMA straight from TMEM; dS^T goes to shared memory once
//                              and is read K-major by the dK MMA and M-major by the dQ MMA.  dQ
//                              tiles go TMEM -> registers -> swizzled shared memory -> TMA
//                              reduce-add into an fp32 workspace (whole-line reductions in L2;
//                              per-thread 16-byte atomics cost a third of the kernel's time).
//   3. fa_bwd_finish_kernel  : dQ = bf16(workspace * 1/sqrt(D)).
// Warp roles in (2): warp 0 TMA producer, warp 1 MMA issuer, warp 2 TMEM allocation, warp 3 dQ reduce issuer,
// warps 4-7 and 8-11 two math groups (P^T, dS^T; a thread owns one key row and one half of the 128
// query columns), warps 12-15 dQ drain.  Per query tile the tensor core sees, in order:
//   dP^T(n) | [P^T(n) ready] dV(n), S^T(n+1) | [dS^T(n) ready] dQ(n), dK(n) | [dQ(n) drained] dP^T(n+1) ...
// so the math groups work on dS^T(n) while dV(n) and S^T(n+1) run, and on P^T(n+1) while dQ(n), dK(n)
// run; dQ is issued before dK so that its drain overlaps the dK MMA.
// TMEM columns (512): S^T [0,128) with P^T written over it (queries 0-63 packed in [0,32), 64-127 in
// [64,96): each math group overwrites only columns it has already read), dP^T and dQ (aliased) [128,256),
// dV [256,256+D), dK [384,384+D).
#pragma once
#include "rope.cuh"
#include "sm100_ptx.cuh"

namespace it {

// KT: key tiles a CTA owns (1, or 2 at head_dim 64 where tensor memory has room for two dV and two dK accumulators).
template <int D, int KT = 1>
struct BwdTraits {
  static_assert(KT == 1 || (KT == 2 && D == 64), "two key tiles per CTA need four accumulators of D columns beside S^T and dP^T");
  static constexpr int BM = 128;   // keys per tile (TMEM lanes)
  static constexpr int BN = 128;   // query rows per inner tile
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int BLOCK_BYTES = 128 * 128;
  static constexpr int NBLK = D / 64;
  static constexpr int SMEM_K = 0;                          // KT tiles
  static constexpr int SMEM_V = SMEM_K + KT * TILE_BYTES;   // KT tiles
  static constexpr int SMEM_Q = SMEM_V + KT * TILE_BYTES;   // 2 stages
  static constexpr int SMEM_DO = SMEM_Q + 2 * TILE_BYTES;   // 1 stage: dO(n) is free again well before dP^T(n+1)
  static constexpr int SMEM_DS = SMEM_DO + TILE_BYTES;      // [2 blocks][128 keys][64 q] bf16
  static constexpr int SMEM_DQS = SMEM_DS + 2 * BLOCK_BYTES;   // dQ staging: [2][128 rows][32 fp32], 128B swizzle
  static constexpr int SMEM_LSE = SMEM_DQS + 2 * BLOCK_BYTES;  // [2 stages][128] fp32
  static constexpr int SMEM_DELTA = SMEM_LSE + 2 * 512;        // [2 stages][128] fp32
  static constexpr int SMEM_BAR = SMEM_DELTA + 2 * 512;
  static constexpr int NUM_BARS = 20;
  static constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = SMEM_MISC + 16;
  static constexpr int THREADS = 512;
  static constexpr uint32_t TMEM_COLS = 512;
  // dV and dK of the CTA's key tile t sit at COL_DV + t * D and COL_DK + t * D
  static constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DQ = 128, COL_DV = 256, COL_DK = 384;
};

struct BwdParams {
  ptx::TensorStrides st;   // layout of q, o, dO and dq
  ptx::TensorStrides st_kv;  // layout of k, v, dk, dv: heads / group heads (grouped-query attention), group 1 otherwise
  const float* lse2_pad;   // [BH, S_pad] LSE * log2(e), +inf in the padding
  const float* delta_pad;  // [BH, S_pad] rowsum(dO*O), 0 in the padding
  float* dq_accum;         // [BH, S, D] fp32, zeroed by the caller
  __nv_bfloat16* dk;       // [BH, S, D]
  __nv_bfloat16* dv;       // [BH, S, D]
  int* status;
  int S;
  int S_pad;
  int BH;
  int causal;
  float scale;             // 1/sqrt(D)
  float scale_log2;        // scale * log2(e)
};

// ------------------------------------------------------------------ (1) prepare
// One warp per eight consecutive rows of one (batch, head): delta and LSE*log2e into the padded arrays, and
// the rows' slices of the fp32 dQ accumulator cleared (saves a separate pass over those 4*D bytes per
// row).  A row is read by 16 lanes (16 bytes per lane at head_dim 128, 8 at 64), so a warp covers two
// rows per load; all eight loads of a lane are issued before the first is used (with one row per warp
// the kernel ran at 70 % of the HBM rate for want of bytes in flight, and 4-byte loads at head_dim 64
// kept half as many bytes in flight as at 128).
template <int D>
__global__ void fa_bwd_prepare_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                      const float* __restrict__ lse, float* __restrict__ lse2_pad,
                                      float* __restrict__ delta_pad, float* __restrict__ dq_accum, int S, int S_pad,
                                      int BH, ptx::TensorStrides st) {
  constexpr int NP = 4;            // passes; a pass covers two rows, one per half-warp
  constexpr int RW = 2 * NP;       // rows per warp; S_pad is a multiple of 128, so they share a head
  constexpr int EL = D / 16;       // elements per lane and row: 8 (D = 128) or 4 (D = 64)
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15, half = lane >> 4;
  ptx::grid_dep_wait();     // O and LSE come from the kernel in front (the forward); the accumulator it clears may still be read
  ptx::grid_dep_launch();   // the main kernel may set itself up meanwhile; it waits for this pass before its first load
  const long long row0 = ((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * RW;
  if (row0 >= static_cast<long long>(BH) * S_pad) return;
  const int bh = static_cast<int>(row0 / S_pad);
  const int s0 = static_cast<int>(row0 % S_pad);
  uint4 a[NP], b[NP];
#pragma unroll
  for (int r = 0; r < NP; ++r) {
    a[r] = make_uint4(0u, 0u, 0u, 0u);
    b[r] = make_uint4(0u, 0u, 0u, 0u);
    const int s_ = s0 + 2 * r + half;
    if (s_ < S) {
      const size_t base = static_cast<size_t>(st.slice(bh) + static_cast<long long>(s_) * st.row);
      if (EL == 8) {
        a[r] = reinterpret_cast<const uint4*>(o + base)[sub];
        b[r] = reinterpret_cast<const uint4*>(d_o + base)[sub];
      } else {
        const uint2 ta = reinterpret_cast<const uint2*>(o + base)[sub];
        const uint2 tb = reinterpret_cast<const uint2*>(d_o + base)[sub];
        a[r].x = ta.x, a[r].y = ta.y;
        b[r].x = tb.x, b[r].y = tb.y;
      }
    }
  }
  float lse_r = 0.f;
  if (lane < RW && s0 + lane < S) lse_r = lse[static_cast<size_t>(bh) * S + s0 + lane];
#pragma unroll
  for (int r = 0; r < NP; ++r) {
    const int s_ = s0 + 2 * r + half;
    if (s_ < S) {
      float* acc_row = dq_accum + (static_cast<size_t>(bh) * S + s_) * D;   // the accumulator is always [BH, S, D]
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      if (EL == 8) {   // 512 bytes per row: two 256-byte halves, each written by the 16 lanes at once
        reinterpret_cast<float4*>(acc_row)[sub] = z;
        reinterpret_cast<float4*>(acc_row)[16 + sub] = z;
      } else {
        reinterpret_cast<float4*>(acc_row)[sub] = z;
      }
    }
  }
  float acc[NP];
#pragma unroll
  for (int r = 0; r < NP; ++r) {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a[r]);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b[r]);
    acc[r] = 0.f;
#pragma unroll
    for (int i = 0; i < EL / 2; ++i) {
      const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
      acc[r] = fmaf(fa.x, fb.x, acc[r]);
      acc[r] = fmaf(fa.y, fb.y, acc[r]);
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) {
#pragma unroll
    for (int r = 0; r < NP; ++r) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
  }
  // row s0 + j (j < 8) was summed in pass j / 2 by half-warp j & 1: bring it to lane j
  float d = 0.f;
#pragma unroll
  for (int r = 0; r < NP; ++r) {
    const float t = __shfl_sync(0xffffffffu, acc[r], (lane & 1) * 16);
    if ((lane >> 1) == r) d = t;
  }
  if (lane < RW) {
    const bool valid = s0 + lane < S;
    delta_pad[row0 + lane] = valid ? d : 0.f;
    lse2_pad[row0 + lane] = valid ? lse_r * 1.4426950408889634f : INFINITY;
  }
}

// ------------------------------------------------------------------ (3) finish
// With freqs.enabled the gradient is rotated back through the rotary embedding on its way out
// (src/shaders/backward/rope.metal:25-62), so dq is the gradient of the un-rotated queries.
__global__ void fa_bwd_finish_kernel(const float* __restrict__ dq_accum, __nv_bfloat16* __restrict__ dq,
                                     size_t n_vec4, float scale, int S, int D, ptx::TensorStrides st,
                                     const __grid_constant__ RopeFreqs freqs) {
  ptx::grid_dep_wait();   // every reduce-add of the main kernel has landed
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec4) return;
  float4 v = reinterpret_cast<const float4*>(dq_accum)[i];
  const size_t e = i * 4;                       // element index in the [BH, S, D] accumulator
  const size_t row = e / D;
  const int d = static_cast<int>(e - row * D);
  const int bh = static_cast<int>(row / S);
  const int s_ = static_cast<int>(row - static_cast<size_t>(bh) * S);
  if (freqs.enabled) {
    float c, sn;
    rope_sincos(freqs, s_ + freqs.position_offset, d >> 1, &c, &sn);
    const float a0 = v.x * c + v.y * sn, a1 = v.y * c - v.x * sn;
    rope_sincos(freqs, s_ + freqs.position_offset, (d >> 1) + 1, &c, &sn);
    const float b0 = v.z * c + v.w * sn, b1 = v.w * c - v.z * sn;
    v = make_float4(a0, a1, b0, b1);
  }
  uint2 w;
  w.x = ptx::pack_bf16(v.x * scale, v.y * scale);
  w.y = ptx::pack_bf16(v.z * scale, v.w * scale);
  *reinterpret_cast<uint2*>(dq + st.slice(bh) + static_cast<long long>(s_) * st.row + d) = w;
}

// ------------------------------------------------------------------ (2) main kernel
template <int D, int KT = 1>
__global__ void __launch_bounds__(512, 1)
fa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ CUtensorMap tmap_dq, const BwdParams prm,
                    const __grid_constant__ RopeFreqs freqs) {
  using T = BwdTraits<D, KT>;
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::SMEM_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [2]
  uint64_t* q_empty = bars + 3;    // [2]
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 7;
  uint64_t* st_full = bars + 9;
  uint64_t* dpt_full = bars + 10;
  uint64_t* p_full = bars + 11;
  uint64_t* ds_full = bars + 12;
  uint64_t* dq_full = bars + 13;
  uint64_t* dq_empty = bars + 14;
  uint64_t* dkv_done = bars + 15;
  uint64_t* dqs_free = bars + 16;  // [2] staging buffer may be rewritten
  uint64_t* dqs_full = bars + 18;  // [2] staging buffer holds a chunk
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + T::SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = prm.S;
  const int n_q_tiles = (S + T::BN - 1) / T::BN;
  // Head-major order in groups of four slices (grouped_tile_order): the CTAs resident at one time belong
  // to four (batch, head) slices, so their Q/dO streams and the fp32 dQ accumulator they add into stay in
  // L2.  Key tile 0 comes first: under the causal mask it sees every query tile and has the most work.
  const int n_k_tiles = (S + T::BM - 1) / T::BM;
  // A CTA owns one key tile of one K/V head and loops over the query heads of that head's group
  // (grouped-query attention: dK and dV are the sums over the group, accumulated in TMEM, so the
  // reference's repeat_kv_backward pass, src/shaders/repeat_kv.metal:49-88, does not exist here).
  const int G = prm.st_kv.group;
  const int kv_heads = prm.st.heads / G;
  // With KT = 2 the CTA owns the key tiles 2*ktp and 2*ktp + 1 (the second may not exist): half as many CTAs, and so
  // half as many start-ups and epilogues, for the same work -- at a thousand keys those are half of a CTA's life.
  const int n_kp = (n_k_tiles + KT - 1) / KT;
  int bhk, ktp;   // batch * kv_heads + kv_head, index of the CTA's key tiles
  grouped_tile_order(static_cast<int>(blockIdx.x), n_kp, static_cast<int>(gridDim.x) / n_kp, &bhk, &ktp);
  const int kt = ktp * KT;                                    // first key tile
  const int nk_cta = min(KT, n_k_tiles - kt);                 // key tiles this CTA owns
  const int hkv = bhk % kv_heads, bt = bhk / kv_heads;        // TMA coordinates of the K/V slice
  const int bh0 = bt * prm.st.heads + hkv * G;                // first query slice of the group
  const int i0 = prm.causal ? kt : 0;
  // An iteration = (query head of the group, query tile, one of the CTA's key tiles), in that nesting; under the causal
  // mask key tile kt + t takes part from query tile kt + t on.
  const int per_head = prm.causal ? (n_q_tiles - kt) * nk_cta - (nk_cta * (nk_cta - 1)) / 2 : n_q_tiles * nk_cta;
  const int n_iter = per_head * G;
  // (g, qi, t) of the next iteration; every role walks the same sequence, starting at (0, i0, 0)
  auto advance = [&](int& g_, int& qi_, int& t_) {
    ++t_;
    if (t_ >= nk_cta || (prm.causal && qi_ < kt + t_)) {
      t_ = 0;
      if (++qi_ == n_q_tiles) {
        qi_ = i0;
        ++g_;
      }
    }
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if (smem_addr(smem) & 1023u) {
      *abort_flag = 1;
      atomicCAS(prm.status, 0, DEV_ERR_SMEM_ALIGN);
    }
    // An earlier CTA of this (or a previous) launch gave up on a wait: do not start, so that a
    // launch that cannot make progress drains quickly instead of timing out CTA by CTA.
    if (*reinterpret_cast<volatile int*>(prm.status) != 0) *abort_flag = 1;
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(do_full, 1);
    mbar_init(do_empty, 1);
    mbar_init(st_full, 1);
    mbar_init(dpt_full, 1);
    mbar_init(p_full, 256);
    mbar_init(ds_full, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 128);
    mbar_init(dkv_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&dqs_free[i], 1);
      mbar_init(&dqs_full[i], 128);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  // Loads of query tile `qi` of the group's query head `g_` for iteration `n`: Q with the rows' LSE*log2e and delta on
  // one barrier, dO on another.  Only the producer thread (thread 0) calls it.
  auto load_q_do = [&](int n, int qi, int g_) -> bool {
    const int st = n & 1;
    const uint32_t ph = (n >> 1) & 1;
    const int hd = hkv * G + g_;   // query head
    if (!mbar_wait_parked(&q_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) return false;
    mbar_arrive_expect_tx(&q_full[st], T::TILE_BYTES + 1024);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_Q + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_q, &q_full[st], b * 64, qi * T::BN, hd, bt);
    const size_t row0 = static_cast<size_t>(bh0 + g_) * prm.S_pad + static_cast<size_t>(qi) * T::BN;
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];" ::"r"(
            smem_addr(smem + T::SMEM_LSE + st * 512)),
        "l"(reinterpret_cast<uint64_t>(prm.lse2_pad + row0)), "r"(smem_addr(&q_full[st]))
        : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], 512, [%2];" ::"r"(
            smem_addr(smem + T::SMEM_DELTA + st * 512)),
        "l"(reinterpret_cast<uint64_t>(prm.delta_pad + row0)), "r"(smem_addr(&q_full[st]))
        : "memory");
    if (!mbar_wait_parked(do_empty, (n & 1) ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) return false;
    mbar_arrive_expect_tx(do_full, T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_DO + b * T::BLOCK_BYTES, &tmap_do, do_full, b * 64, qi * T::BN, hd, bt);
    return true;
  };
  // The first loads go out before the CTA-wide set-up (tensor-memory allocation, barrier, register hand-over), so
  // their round trip to memory runs under it: a short-sequence CTA lives for a handful of tiles and this wait is a
  // visible part of its life.  Nothing is loaded into a CTA that is not going to run.
  if (threadIdx.x == 0 && *abort_flag == 0 && n_iter > 0) {
    grid_dep_wait();   // LSE*log2e, delta and the cleared dQ accumulator come from the prepare pass in front
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
    prefetch_tensormap(&tmap_do);
    prefetch_tensormap(&tmap_dq);
    mbar_arrive_expect_tx(kv_full, nk_cta * 2 * T::TILE_BYTES);
    for (int t = 0; t < nk_cta; ++t)
      for (int b = 0; b < T::NBLK; ++b) {
        tma_load_4d(smem + T::SMEM_K + t * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_k, kv_full, b * 64, (kt + t) * T::BM, hkv, bt);
        tma_load_4d(smem + T::SMEM_V + t * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_v, kv_full, b * 64, (kt + t) * T::BM, hkv, bt);
      }
    load_q_do(0, i0, 0);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dep_wait();     // (thread 0 has been through it; the others write to memory the prepare pass wrote as well)
  grid_dep_launch();   // the finish pass may be set up; it waits for this kernel to complete before it reads
  const uint32_t tmem_base = *tmem_slot;
  const bool bad_start = (*abort_flag != 0);

  // Register budget: the control warpgroup (warps 0-3) keeps 96 per thread; what it gives up lets
  // the dQ drain warpgroup (warps 12-15) hold a whole 128 x D fp32 tile in registers, so that tile
  // leaves TMEM in one go.  128*96 + 256*128 + 128*160 = 65536 <= 65536.
  const bool run = !bad_start && n_iter > 0;
  static_assert(128 * 96 + 256 * 128 + 128 * 160 <= 512 * 128, "setmaxnreg budget exceeds the registers the CTA is launched with");
  if (warp < 4) {
    setmaxnreg_dec<96>();
    if (!run) {
      // nothing to do
    } else if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      // (K, V and the first query tile's loads were issued by this thread before the CTA-wide set-up barrier.)
      if (lane == 0) {
        int g = 0, qi = i0, t = 0;   // iteration 0
        for (int n = 1; n < n_iter; ++n) {
          advance(g, qi, t);
          if (!load_q_do(n, qi, g)) break;   // (with two key tiles a query tile is fetched once per key tile; the second comes from L2)
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (one thread)
      if (lane == 0) {
        constexpr uint32_t IDESC_SS = make_idesc(128, 128, false, false);   // S^T, dP^T
        constexpr uint32_t IDESC_ND = make_idesc(128, D, false, true);      // dV, dK (B N-major)
        constexpr uint32_t IDESC_DQ = make_idesc(128, D, true, true);       // dQ (A M-major, B N-major)
        const uint32_t k_addr = smem_addr(smem + T::SMEM_K);
        const uint32_t v_addr = smem_addr(smem + T::SMEM_V);
        const uint32_t q_addr = smem_addr(smem + T::SMEM_Q);
        const uint32_t do_addr = smem_addr(smem + T::SMEM_DO);
        const uint32_t ds_addr = smem_addr(smem + T::SMEM_DS);
        auto kmajor_off = [](int kk) -> uint32_t { return (kk >> 2) * T::BLOCK_BYTES + (kk & 3) * 32; };
        // A barrier probe takes a few hundred cycles while the tensor core streams operands out of shared
        // memory, and the queue in front of the tensor core is short, so a probe between two bursts is a
        // gap in the MMA stream.  Every burst therefore runs `mid` half-way through: a non-blocking probe
        // of the barrier the NEXT burst depends on, whose answer is read when this burst has been issued.
        auto none = [] {};
        auto issue_st = [&](int st, int t, auto mid) {   // S^T = K * Q^T   (t: which of the CTA's key tiles)
          const uint64_t da = make_sdesc(k_addr + t * T::TILE_BYTES, 16, 1024);
          const uint64_t db = make_sdesc(q_addr + st * T::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            if (kk == D / 32) mid();
            umma_ss(tmem_base + T::COL_ST, sdesc_advance(da, kmajor_off(kk)), sdesc_advance(db, kmajor_off(kk)),
                    IDESC_SS, kk > 0);
          }
          umma_commit(st_full);
        };
        auto issue_dpt = [&](int t, auto mid) {   // dP^T = V * dO^T
          const uint64_t da = make_sdesc(v_addr + t * T::TILE_BYTES, 16, 1024);
          const uint64_t db = make_sdesc(do_addr, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            if (kk == D / 32) mid();
            umma_ss(tmem_base + T::COL_DPT, sdesc_advance(da, kmajor_off(kk)), sdesc_advance(db, kmajor_off(kk)),
                    IDESC_SS, kk > 0);
          }
          umma_commit(dpt_full);
        };
        auto issue_dv = [&](int t, bool first, auto mid) {   // dV += P^T * dO   (A from TMEM, B = dO N-major)
          const uint64_t db = make_sdesc(do_addr, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            if (kk == 4) mid();
            umma_ts(tmem_base + T::COL_DV + t * D, tmem_base + T::COL_ST + (kk >> 2) * 64 + (kk & 3) * 8,
                    sdesc_advance(db, kk * 2048), IDESC_ND, (!first || kk > 0) ? 1u : 0u);
          }
        };
        auto issue_dk = [&](int st, int t, bool first, auto mid) {   // dK += dS^T * Q   (A = dS^T K-major, B = Q N-major)
          const uint64_t da = make_sdesc(ds_addr, 16, 1024);
          const uint64_t db = make_sdesc(q_addr + st * T::TILE_BYTES, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            if (kk == 4) mid();
            umma_ss(tmem_base + T::COL_DK + t * D, sdesc_advance(da, kmajor_off(kk)), sdesc_advance(db, kk * 2048), IDESC_ND,
                    (!first || kk > 0) ? 1u : 0u);
          }
        };
        auto issue_dq = [&](int t) {   // dQ = dS * K   (A = dS M-major from the same buffer, B = K N-major)
          const uint64_t da = make_sdesc(ds_addr, T::BLOCK_BYTES, 1024);
          const uint64_t db = make_sdesc(k_addr + t * T::TILE_BYTES, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tmem_base + T::COL_DQ, sdesc_advance(da, kk * 2048), sdesc_advance(db, kk * 2048), IDESC_DQ,
                    kk > 0);
        };
        auto need = [&](bool ready, uint64_t* bar, uint32_t parity, int code) {
          return ready || mbar_wait_parked(bar, parity, abort_flag, prm.status, code);
        };
        bool ok = mbar_wait_parked(kv_full, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (ok) ok = mbar_wait_parked(&q_full[0], 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (ok) {
          tc_fence_after();
          issue_st(0, 0, none);
        }
        bool r_do = false, r_dq = false, r_p = false, r_q = false, r_ds = false;   // answers of the early probes
        int g_c = 0, qi_c = i0, t_c = 0;     // this iteration's query head, query tile and key tile
        bool started[KT] = {};               // has the key tile's dV / dK accumulation begun?
        for (int n = 0; n < n_iter && ok; ++n) {
          const int t = t_c;
          advance(g_c, qi_c, t_c);           // t_c: the next iteration's key tile
          const bool first = !started[t];
          started[t] = true;
          const int st = n & 1;
          const uint32_t par = n & 1;
          const bool more = (n + 1 < n_iter);
          const int st_n = (n + 1) & 1;
          const uint32_t ph_n = ((n + 1) >> 1) & 1;
          ok = need(r_do, do_full, par, DEV_ERR_TIMEOUT_LOAD);
          // dQ(n-1) must have left TMEM before dP^T(n) overwrites those columns
          if (ok && n > 0) ok = need(r_dq, dq_empty, (n - 1) & 1, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          issue_dpt(t, [&] { r_p = mbar_test_wait(p_full, par); });
          ok = need(r_p, p_full, par, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          issue_dv(t, first, [&] { r_q = more && mbar_test_wait(&q_full[st_n], ph_n); });
          umma_commit(do_empty);
          r_ds = false;
          if (more) {
            ok = need(r_q, &q_full[st_n], ph_n, DEV_ERR_TIMEOUT_LOAD);
            if (!ok) break;
            tc_fence_after();
            issue_st(st_n, t_c, [&] { r_ds = mbar_test_wait(ds_full, par); });
          }
          ok = need(r_ds, ds_full, par, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          issue_dq(t);
          umma_commit(dq_full);
          issue_dk(st, t, first, [&] {
            r_do = more && mbar_test_wait(do_full, par ^ 1);
            r_dq = more && mbar_test_wait(dq_empty, par);
          });
          umma_commit(&q_empty[st]);
        }
        if (ok) umma_commit(dkv_done);
      }
    } else if (warp == 3) {
      // ------------------------------------------------------------ dQ reduce issuer (one thread)
      // Adds each staged 128 x 32 chunk of a dQ tile into the fp32 accumulator (TMA reduce-add) and hands the
      // staging buffers back to the drain warps.  A thread of its own: the drain warps then never wait for a
      // reduce to be issued or for its read of shared memory to finish.
      if (lane == 0) {
        bool ok = true;
        int g = 0;
        int g_q = 0, qi = i0, t_q = 0;
        for (int n = 0; n < n_iter && ok; ++n, advance(g_q, qi, t_q)) {
          const int bh_q = bh0 + g_q;
#pragma unroll
          for (int c = 0; c < D / 32; ++c, ++g) {
            const int buf = g & 1;
            if (!mbar_wait(&dqs_full[buf], static_cast<uint32_t>(g >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX)) {
              ok = false;
              break;
            }
            tma_reduce_add_3d(&tmap_dq, smem + T::SMEM_DQS + buf * T::BLOCK_BYTES, c * 32, qi * T::BN, bh_q);
            bulk_commit_group();
            if (g >= 1) {   // the previous chunk's reduce has read the other buffer: hand it back
              bulk_wait_group_read<1>();
              mbar_arrive(&dqs_free[buf ^ 1]);
            }
          }
        }
        bulk_wait_group_all();   // shared memory must outlive the reads; results complete before exit
      }
    }
  } else if (warp < 12) {
    if (run) {
      // ------------------------------------------------------------ P^T and dS^T math, dK/dV epilogue
      const int half = (warp - 4) >> 2;                 // which 64 of the 128 query columns
      const int lane_base = (warp & 3) * 32;
      const int k_local = lane_base + lane;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
      const uint32_t t_st = t_lane + T::COL_ST + half * 64;
      const uint32_t t_dpt = t_lane + T::COL_DPT + half * 64;
      const float sl2 = prm.scale_log2;
      uint8_t* ds_row = smem + T::SMEM_DS + half * T::BLOCK_BYTES + k_local * 128;
      const int swz = k_local & 7;
      bool ok = true;
      uint32_t ra[16], rb[16];
      uint32_t p_keep[32];   // this thread's 64 P^T values, packed bf16, kept between the two phases
      int g_m = 0, qi = i0, t_m = 0;
      for (int n = 0; n < n_iter; ++n, advance(g_m, qi, t_m)) {
        const int st = n & 1;
        const bool diag = prm.causal && (qi == kt + t_m);   // the key tile's own query tile: keys after the query are masked
        const float* lse_s = reinterpret_cast<const float*>(smem + T::SMEM_LSE + st * 512) + half * 64;
        const float* dl_s = reinterpret_cast<const float*>(smem + T::SMEM_DELTA + st * 512) + half * 64;
        // lse/delta for this query tile ride on the Q barrier
        ok = mbar_wait_parked(&q_full[st], (n >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (ok) ok = mbar_wait_parked(st_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // phase A: P^T = 2^(S^T * scale*log2e - LSE*log2e); the next 16 columns load while these are computed
        auto phase_a = [&](const uint32_t (&r)[16], int c) {
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(lse_s + c * 16 + i);
            float p0 = ex2(fmaf(__uint_as_float(r[i + 0]), sl2, -l4.x));
            float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), sl2, -l4.y));
            float p2 = ex2(fmaf(__uint_as_float(r[i + 2]), sl2, -l4.z));
            float p3 = ex2(fmaf(__uint_as_float(r[i + 3]), sl2, -l4.w));
            if (diag) {   // key after the query: masked
              const int qc = half * 64 + c * 16 + i;
              if (k_local > qc + 0) p0 = 0.f;
              if (k_local > qc + 1) p1 = 0.f;
              if (k_local > qc + 2) p2 = 0.f;
              if (k_local > qc + 3) p3 = 0.f;
            }
            p_keep[c * 8 + (i >> 1)] = pack_bf16(p0, p1);
            p_keep[c * 8 + (i >> 1) + 1] = pack_bf16(p2, p3);
          }
        };
        tmem_ld_x16(t_st, ra);
        tmem_wait_ld();
        tmem_ld_x16(t_st + 16, rb);
        phase_a(ra, 0);
        tmem_wait_ld();
        tmem_ld_x16(t_st + 32, ra);
        phase_a(rb, 1);
        tmem_wait_ld();
        tmem_ld_x16(t_st + 48, rb);
        phase_a(ra, 2);
        tmem_wait_ld();
        phase_a(rb, 3);
        tmem_st_x32(t_st, p_keep);   // 64 queries -> 32 packed columns at the start of this group's own range
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full);
        // phase B: dS^T = P^T o (dP^T - delta), bf16, swizzled into shared memory
        ok = mbar_wait_parked(dpt_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        auto phase_b = [&](const uint32_t (&r)[16], int c) {
          uint32_t dsp[8];
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const float4 d4 = *reinterpret_cast<const float4*>(dl_s + c * 16 + i);
            const uint32_t pa = p_keep[c * 8 + (i >> 1)], pb = p_keep[c * 8 + (i >> 1) + 1];
            const float p0 = __uint_as_float(pa << 16), p1 = __uint_as_float(pa & 0xFFFF0000u);
            const float p2 = __uint_as_float(pb << 16), p3 = __uint_as_float(pb & 0xFFFF0000u);
            dsp[i >> 1] = pack_bf16(p0 * (__uint_as_float(r[i + 0]) - d4.x), p1 * (__uint_as_float(r[i + 1]) - d4.y));
            dsp[(i >> 1) + 1] = pack_bf16(p2 * (__uint_as_float(r[i + 2]) - d4.z), p3 * (__uint_as_float(r[i + 3]) - d4.w));
          }
          // 16 query columns = two 16-byte chunks of this key row
          *reinterpret_cast<uint4*>(ds_row + (((2 * c) ^ swz) << 4)) = make_uint4(dsp[0], dsp[1], dsp[2], dsp[3]);
          *reinterpret_cast<uint4*>(ds_row + (((2 * c + 1) ^ swz) << 4)) = make_uint4(dsp[4], dsp[5], dsp[6], dsp[7]);
        };
        tmem_ld_x16(t_dpt, ra);
        tmem_wait_ld();
        tmem_ld_x16(t_dpt + 16, rb);
        phase_b(ra, 0);
        tmem_wait_ld();
        tmem_ld_x16(t_dpt + 32, ra);
        phase_b(rb, 1);
        tmem_wait_ld();
        tmem_ld_x16(t_dpt + 48, rb);
        phase_b(ra, 2);
        tmem_wait_ld();
        phase_b(rb, 3);
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(ds_full);
      }
      if (ok) {
        ok = mbar_wait_parked(dkv_done, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        // each math group writes one half of the head dimension of its key row's dV and dK
        tc_fence_after();
        constexpr int HC = D / 2;
#pragma unroll 1
        for (int tw = 0; tw < 2 * nk_cta; ++tw) {   // dV then dK of each of the CTA's key tiles
          const int t = tw >> 1, which = tw & 1;
          const int k_row = (kt + t) * T::BM + k_local;
          const long long out_off = prm.st_kv.slice(bh0) + static_cast<long long>(k_row) * prm.st_kv.row + half * HC;
          __nv_bfloat16* dv_row = prm.dv + out_off;
          __nv_bfloat16* dk_row = prm.dk + out_off;
          const uint32_t col = (which ? T::COL_DK : T::COL_DV) + t * D + half * HC;
          const float f = which ? prm.scale : 1.0f;
          __nv_bfloat16* orow = which ? dk_row : dv_row;
#pragma unroll 1
          for (int c = 0; c < HC / 16; ++c) {
            tmem_ld_x16(t_lane + col + c * 16, ra);
            tmem_wait_ld();
            if (which && freqs.enabled) {   // dK leaves through the inverse rotary rotation of its key position
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                float cs, sn;
                rope_sincos(freqs, k_row + freqs.position_offset, (half * HC + c * 16) / 2 + j, &cs, &sn);
                const float g0 = __uint_as_float(ra[2 * j]), g1 = __uint_as_float(ra[2 * j + 1]);
                ra[2 * j] = __float_as_uint(g0 * cs + g1 * sn);
                ra[2 * j + 1] = __float_as_uint(g1 * cs - g0 * sn);
              }
            }
            if (k_row < S) {
#pragma unroll
              for (int v4 = 0; v4 < 2; ++v4) {
                uint4 w;
                w.x = pack_bf16(__uint_as_float(ra[v4 * 8 + 0]) * f, __uint_as_float(ra[v4 * 8 + 1]) * f);
                w.y = pack_bf16(__uint_as_float(ra[v4 * 8 + 2]) * f, __uint_as_float(ra[v4 * 8 + 3]) * f);
                w.z = pack_bf16(__uint_as_float(ra[v4 * 8 + 4]) * f, __uint_as_float(ra[v4 * 8 + 5]) * f);
                w.w = pack_bf16(__uint_as_float(ra[v4 * 8 + 6]) * f, __uint_as_float(ra[v4 * 8 + 7]) * f);
                *reinterpret_cast<uint4*>(orow + c * 16 + v4 * 8) = w;
              }
            }
          }
        }
      }
    }
  } else {
    setmaxnreg_inc<160>();
    if (run) {
      // ------------------------------------------------------------ dQ drain: TMEM -> registers -> smem -> TMA reduce-add
      // The tile is read out of TMEM in one go (so dP^T of the next query tile can start at once),
      // then goes 32 columns at a time through two staging buffers.  Hand-offs use mbarriers with
      // bounded waits (no named barriers: a role that gives up must never leave another one blocked).
      const int lane_base = (warp & 3) * 32;
      const int row = lane_base + lane;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + T::COL_DQ;
      const int swz = row & 7;
      bool ok = true;
      uint32_t r[D / 32][32];
      int g = 0;   // chunks handled so far
      for (int n = 0; n < n_iter && ok; ++n) {
        ok = mbar_wait_parked(dq_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld_x32(t_lane + c * 32, r[c]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(dq_empty);
#pragma unroll
        for (int c = 0; c < D / 32; ++c, ++g) {
          const int buf = g & 1;
          const uint32_t use = static_cast<uint32_t>(g >> 1);
          uint8_t* stage = smem + T::SMEM_DQS + buf * T::BLOCK_BYTES;
          // the reduce that read this buffer two chunks ago must be done with it
          ok = mbar_wait_parked(&dqs_free[buf], (use & 1) ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          uint8_t* dst = stage + row * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(dst + ((ch ^ swz) << 4)) =
                make_uint4(r[c][ch * 4 + 0], r[c][ch * 4 + 1], r[c][ch * 4 + 2], r[c][ch * 4 + 3]);
          fence_proxy_async_smem();
          mbar_arrive(&dqs_full[buf]);   // the reduce issuer (warp 3) takes it from here
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*abort_flag) {
      for (int i = 0; i < 50; ++i) __nanosleep(20000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace it
