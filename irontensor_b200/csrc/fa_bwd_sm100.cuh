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
//                              tiles are added into an fp32 workspace with vector atomics.
//   3. fa_bwd_finish_kernel  : dQ = bf16(workspace * 1/sqrt(D)).
// Warp roles in (2): warp 0 TMA producer, warp 1 MMA issuer, warp 2 TMEM allocation,
// warps 4-7 softmax/dS math (one thread per key row), warps 8-11 dQ drain.
// TMEM columns (512): S^T/P^T [0,128)  dP^T and dQ (aliased) [128,256)  dV [256,256+D)  dK [384,384+D).
#pragma once
#include "sm100_ptx.cuh"

namespace it {

template <int D>
struct BwdTraits {
  static constexpr int BM = 128;   // keys per CTA tile (TMEM lanes)
  static constexpr int BN = 128;   // query rows per inner tile
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int BLOCK_BYTES = 128 * 128;
  static constexpr int NBLK = D / 64;
  static constexpr int SMEM_K = 0;
  static constexpr int SMEM_V = SMEM_K + TILE_BYTES;
  static constexpr int SMEM_Q = SMEM_V + TILE_BYTES;        // 2 stages
  static constexpr int SMEM_DO = SMEM_Q + 2 * TILE_BYTES;   // 2 stages
  static constexpr int SMEM_DS = SMEM_DO + 2 * TILE_BYTES;  // [2 blocks][128 keys][64 q] bf16
  static constexpr int SMEM_LSE = SMEM_DS + 2 * BLOCK_BYTES;   // [2 stages][128] fp32
  static constexpr int SMEM_DELTA = SMEM_LSE + 2 * 512;        // [2 stages][128] fp32
  static constexpr int SMEM_BAR = SMEM_DELTA + 2 * 512;
  static constexpr int NUM_BARS = 16;
  static constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = SMEM_MISC + 16;
  static constexpr int THREADS = 384;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DQ = 128, COL_DV = 256, COL_DK = 384;
};

struct BwdParams {
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
// One warp per (bh, row): delta and LSE*log2e into the padded arrays.
template <int D>
__global__ void fa_bwd_prepare_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                      const float* __restrict__ lse, float* __restrict__ lse2_pad,
                                      float* __restrict__ delta_pad, int S, int S_pad, int BH) {
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= static_cast<long long>(BH) * S_pad) return;
  const int bh = static_cast<int>(row / S_pad);
  const int s = static_cast<int>(row % S_pad);
  if (s >= S) {
    if (lane == 0) {
      lse2_pad[row] = INFINITY;
      delta_pad[row] = 0.f;
    }
    return;
  }
  const size_t base = (static_cast<size_t>(bh) * S + s) * D;
  float acc = 0.f;
  if (D == 128) {
    const uint2 a = reinterpret_cast<const uint2*>(o + base)[lane];
    const uint2 b = reinterpret_cast<const uint2*>(d_o + base)[lane];
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
      acc = fmaf(fa.x, fb.x, acc);
      acc = fmaf(fa.y, fb.y, acc);
    }
  } else {
    const __nv_bfloat162 a = reinterpret_cast<const __nv_bfloat162*>(o + base)[lane];
    const __nv_bfloat162 b = reinterpret_cast<const __nv_bfloat162*>(d_o + base)[lane];
    const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    acc = fmaf(fa.x, fb.x, fa.y * fb.y);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    delta_pad[row] = acc;
    lse2_pad[row] = lse[static_cast<size_t>(bh) * S + s] * 1.4426950408889634f;
  }
}

// ------------------------------------------------------------------ (3) finish
__global__ void fa_bwd_finish_kernel(const float* __restrict__ dq_accum, __nv_bfloat16* __restrict__ dq,
                                     size_t n_vec4, float scale) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec4) return;
  const float4 v = reinterpret_cast<const float4*>(dq_accum)[i];
  uint2 w;
  w.x = ptx::pack_bf16(v.x * scale, v.y * scale);
  w.y = ptx::pack_bf16(v.z * scale, v.w * scale);
  reinterpret_cast<uint2*>(dq)[i] = w;
}

// ------------------------------------------------------------------ (2) main kernel
template <int D>
__global__ void __launch_bounds__(384, 1)
fa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const BwdParams prm) {
  using T = BwdTraits<D>;
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::SMEM_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [2]
  uint64_t* q_empty = bars + 3;    // [2]
  uint64_t* do_full = bars + 5;    // [2]
  uint64_t* do_empty = bars + 7;   // [2]
  uint64_t* st_full = bars + 9;
  uint64_t* dpt_full = bars + 10;
  uint64_t* p_full = bars + 11;
  uint64_t* ds_full = bars + 12;
  uint64_t* dq_full = bars + 13;
  uint64_t* dq_empty = bars + 14;
  uint64_t* dkv_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + T::SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = prm.S;
  const int n_q_tiles = (S + T::BN - 1) / T::BN;
  // Key tile 0 sees every query tile (most work under the causal mask): schedule it first.
  const int kt = static_cast<int>(blockIdx.x) / prm.BH;
  const int bh = static_cast<int>(blockIdx.x) % prm.BH;
  const int i0 = prm.causal ? kt : 0;
  const int n_iter = n_q_tiles - i0;

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
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 1);
    }
    mbar_init(st_full, 1);
    mbar_init(dpt_full, 1);
    mbar_init(p_full, 128);
    mbar_init(ds_full, 128);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 128);
    mbar_init(dkv_done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool bad_start = (*abort_flag != 0);

  if (!bad_start && n_iter > 0) {
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        prefetch_tensormap(&tmap_do);
        mbar_arrive_expect_tx(kv_full, 2 * T::TILE_BYTES);
        for (int b = 0; b < T::NBLK; ++b) {
          tma_load_3d(smem + T::SMEM_K + b * T::BLOCK_BYTES, &tmap_k, kv_full, b * 64, kt * T::BM, bh);
          tma_load_3d(smem + T::SMEM_V + b * T::BLOCK_BYTES, &tmap_v, kv_full, b * 64, kt * T::BM, bh);
        }
        for (int n = 0; n < n_iter; ++n) {
          const int st = n & 1;
          const uint32_t ph = (n >> 1) & 1;
          const int qi = i0 + n;
          if (!mbar_wait(&q_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) break;
          mbar_arrive_expect_tx(&q_full[st], T::TILE_BYTES + 1024);
          for (int b = 0; b < T::NBLK; ++b)
            tma_load_3d(smem + T::SMEM_Q + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_q, &q_full[st], b * 64,
                        qi * T::BN, bh);
          const size_t row0 = static_cast<size_t>(bh) * prm.S_pad + static_cast<size_t>(qi) * T::BN;
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
          if (!mbar_wait(&do_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) break;
          mbar_arrive_expect_tx(&do_full[st], T::TILE_BYTES);
          for (int b = 0; b < T::NBLK; ++b)
            tma_load_3d(smem + T::SMEM_DO + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_do, &do_full[st], b * 64,
                        qi * T::BN, bh);
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
        auto issue_st = [&](int st) {   // S^T = K * Q^T
          const uint64_t da = make_sdesc(k_addr, 16, 1024);
          const uint64_t db = make_sdesc(q_addr + st * T::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            umma_ss(tmem_base + T::COL_ST, sdesc_advance(da, kmajor_off(kk)), sdesc_advance(db, kmajor_off(kk)),
                    IDESC_SS, kk > 0);
          umma_commit(st_full);
        };
        auto issue_dpt = [&](int st) {   // dP^T = V * dO^T
          const uint64_t da = make_sdesc(v_addr, 16, 1024);
          const uint64_t db = make_sdesc(do_addr + st * T::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            umma_ss(tmem_base + T::COL_DPT, sdesc_advance(da, kmajor_off(kk)), sdesc_advance(db, kmajor_off(kk)),
                    IDESC_SS, kk > 0);
          umma_commit(dpt_full);
        };
        auto issue_dv = [&](int st, bool first) {   // dV += P^T * dO   (A from TMEM, B = dO N-major)
          const uint64_t db = make_sdesc(do_addr + st * T::TILE_BYTES, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(tmem_base + T::COL_DV, tmem_base + T::COL_ST + kk * 8, sdesc_advance(db, kk * 2048), IDESC_ND,
                    (!first || kk > 0) ? 1u : 0u);
        };
        auto issue_dk = [&](int st, bool first) {   // dK += dS^T * Q   (A = dS^T K-major, B = Q N-major)
          const uint64_t da = make_sdesc(ds_addr, 16, 1024);
          const uint64_t db = make_sdesc(q_addr + st * T::TILE_BYTES, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tmem_base + T::COL_DK, sdesc_advance(da, kmajor_off(kk)), sdesc_advance(db, kk * 2048), IDESC_ND,
                    (!first || kk > 0) ? 1u : 0u);
        };
        auto issue_dq = [&]() {   // dQ = dS * K   (A = dS M-major from the same buffer, B = K N-major)
          const uint64_t da = make_sdesc(ds_addr, T::BLOCK_BYTES, 1024);
          const uint64_t db = make_sdesc(k_addr, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tmem_base + T::COL_DQ, sdesc_advance(da, kk * 2048), sdesc_advance(db, kk * 2048), IDESC_DQ,
                    kk > 0);
        };
        bool ok = mbar_wait(kv_full, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (ok) {
          tc_fence_after();
          issue_st(0);
        }
        for (int n = 0; n < n_iter && ok; ++n) {
          const int st = n & 1;
          const uint32_t ph = (n >> 1) & 1;
          ok = mbar_wait(&do_full[st], ph, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
          if (!ok) break;
          if (n > 0) {   // dQ(n-1) must have left TMEM before dP^T(n) overwrites those columns
            ok = mbar_wait(dq_empty, (n - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
            if (!ok) break;
          }
          tc_fence_after();
          issue_dpt(st);
          ok = mbar_wait(p_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          issue_dv(st, n == 0);
          umma_commit(&do_empty[st]);
          if (n + 1 < n_iter) {
            const int st_n = (n + 1) & 1;
            const uint32_t ph_n = ((n + 1) >> 1) & 1;
            ok = mbar_wait(&q_full[st_n], ph_n, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
            if (!ok) break;
            tc_fence_after();
            issue_st(st_n);
          }
          ok = mbar_wait(ds_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          issue_dk(st, n == 0);
          issue_dq();
          umma_commit(&q_empty[st]);
          umma_commit(dq_full);
        }
        if (ok) umma_commit(dkv_done);
      }
    } else if (warp >= 4 && warp < 8) {
      // ------------------------------------------------------------ P^T and dS^T math, dK/dV epilogue
      const int lane_base = (warp & 3) * 32;
      const int k_local = lane_base + lane;
      const int k_row = kt * T::BM + k_local;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
      const float sl2 = prm.scale_log2;
      uint8_t* ds_row = smem + T::SMEM_DS + k_local * 128;
      const int swz = k_local & 7;
      bool ok = true;
      uint32_t r[32];
      uint32_t p_keep[64];   // P^T row, packed bf16, kept between the two phases
      for (int n = 0; n < n_iter; ++n) {
        const int st = n & 1;
        const int qi = i0 + n;
        const bool diag = prm.causal && (qi == kt);
        const float* lse_s = reinterpret_cast<const float*>(smem + T::SMEM_LSE + st * 512);
        const float* dl_s = reinterpret_cast<const float*>(smem + T::SMEM_DELTA + st * 512);
        // lse/delta for this query tile ride on the Q barrier
        ok = mbar_wait(&q_full[st], (n >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (ok) ok = mbar_wait(st_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // phase A: P^T = 2^(S^T * scale*log2e - LSE*log2e)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_x32(t_lane + T::COL_ST + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 l2 = *reinterpret_cast<const float2*>(lse_s + c * 32 + i);
            float p0 = ex2(fmaf(__uint_as_float(r[i]), sl2, -l2.x));
            float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), sl2, -l2.y));
            if (diag) {   // key after the query: masked
              if (k_local > c * 32 + i) p0 = 0.f;
              if (k_local > c * 32 + i + 1) p1 = 0.f;
            }
            p_keep[c * 16 + (i >> 1)] = pack_bf16(p0, p1);
          }
          tmem_st_x16(t_lane + T::COL_ST + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&p_keep[c * 16]));
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full);
        // phase B: dS^T = P^T o (dP^T - delta), bf16, swizzled into shared memory
        ok = mbar_wait(dpt_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_x32(t_lane + T::COL_DPT + c * 32, r);
          tmem_wait_ld();
          uint32_t dsp[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 dl = *reinterpret_cast<const float2*>(dl_s + c * 32 + i);
            const uint32_t pp = p_keep[c * 16 + (i >> 1)];
            const float p0 = __uint_as_float(pp << 16);
            const float p1 = __uint_as_float(pp & 0xFFFF0000u);
            dsp[i >> 1] = pack_bf16(p0 * (__uint_as_float(r[i]) - dl.x), p1 * (__uint_as_float(r[i + 1]) - dl.y));
          }
          // 32 query columns = four 16-byte chunks of this key row, in 64-column block (c >> 1)
          uint8_t* blk = ds_row + (c >> 1) * T::BLOCK_BYTES;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const int chunk = (c & 1) * 4 + ch;
            *reinterpret_cast<uint4*>(blk + ((chunk ^ swz) << 4)) =
                make_uint4(dsp[ch * 4 + 0], dsp[ch * 4 + 1], dsp[ch * 4 + 2], dsp[ch * 4 + 3]);
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(ds_full);
      }
      if (ok) {
        ok = mbar_wait(dkv_done, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
        __nv_bfloat16* dv_row = prm.dv + (static_cast<size_t>(bh) * S + k_row) * D;
        __nv_bfloat16* dk_row = prm.dk + (static_cast<size_t>(bh) * S + k_row) * D;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          const uint32_t col = which ? T::COL_DK : T::COL_DV;
          const float f = which ? prm.scale : 1.0f;
          __nv_bfloat16* orow = which ? dk_row : dv_row;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld_x32(t_lane + col + c * 32, r);
            tmem_wait_ld();
            if (k_row < S) {
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                uint4 w;
                w.x = pack_bf16(__uint_as_float(r[v4 * 8 + 0]) * f, __uint_as_float(r[v4 * 8 + 1]) * f);
                w.y = pack_bf16(__uint_as_float(r[v4 * 8 + 2]) * f, __uint_as_float(r[v4 * 8 + 3]) * f);
                w.z = pack_bf16(__uint_as_float(r[v4 * 8 + 4]) * f, __uint_as_float(r[v4 * 8 + 5]) * f);
                w.w = pack_bf16(__uint_as_float(r[v4 * 8 + 6]) * f, __uint_as_float(r[v4 * 8 + 7]) * f);
                *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = w;
              }
            }
          }
        }
      }
    } else if (warp >= 8) {
      // ------------------------------------------------------------ dQ drain: TMEM -> fp32 atomics
      const int lane_base = (warp & 3) * 32;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + T::COL_DQ;
      bool ok = true;
      uint32_t r[32];
      for (int n = 0; n < n_iter; ++n) {
        const int q_row = (i0 + n) * T::BN + lane_base + lane;
        ok = mbar_wait(dq_full, n & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        float* dst = prm.dq_accum + (static_cast<size_t>(bh) * S + q_row) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld_x32(t_lane + c * 32, r);
          tmem_wait_ld();
          if (c == D / 32 - 1) {   // last read done: the columns may be overwritten
            tc_fence_before();
            mbar_arrive(dq_empty);
          }
          if (q_row < S) {
#pragma unroll
            for (int v4 = 0; v4 < 8; ++v4)
              atomicAdd(reinterpret_cast<float4*>(dst + c * 32 + v4 * 4),
                        make_float4(__uint_as_float(r[v4 * 4 + 0]), __uint_as_float(r[v4 * 4 + 1]),
                                    __uint_as_float(r[v4 * 4 + 2]), __uint_as_float(r[v4 * 4 + 3])));
          }
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
