// Causal / full attention forward for FP32 tensors on the sm_100a tensor cores.
//
// The reference's own precision is fp32 (src/ops/flash_attention.rs:76-193; kernels
// src/shaders/flash_attention.metal:45-163 and :167-223), and its results are held to 1e-4.  The tensor
// cores multiply bf16, so every fp32 operand is split into three bf16 terms,
//     x = x_hi + x_mid + x_lo,   x_hi = bf16(x), x_mid = bf16(x - x_hi), x_lo = bf16(x - x_hi - x_mid),
// (the two subtractions are exact in fp32; the three terms carry 24 mantissa bits) and a product of two split
// operands is the sum of the six term products of order above 2^-24:
//     a b ~= a_hi b_hi + a_hi b_mid + a_mid b_hi + a_hi b_lo + a_mid b_mid + a_lo b_hi,
// six tcgen05.mma into one fp32 accumulator.  Q K^T and P V are done that way; the softmax between them is
// the same fp32 online softmax as in the bf16 kernels.  Measured against the scalar fp32 restatement of the reference kernels: at most 6e-6 on O and 4e-6 on LSE.
//
// One CTA owns one 128-row query tile of one (batch, head) slice and walks the key tiles:
//   warps 0-3 : softmax, one thread per query row: S from TMEM, P = 2^(s*c - m) split into three packed bf16
//               planes and written back to TMEM (the A operand of the P V MMAs), final O / l and LSE
//   warps 4-7 : loaders: fp32 rows of Q, K, V from global memory into registers, split, and stored as three
//               bf16 planes each in the 128-byte-swizzled layout the MMA descriptors read; the next key
//               tile's rows are fetched into registers while the current tile is being worked on
//   warp 8    : tensor-memory allocation, and the one thread that issues the MMAs
// head_dim <= 64 and a multiple of 4 (columns past head_dim are zero planes).  Tensor memory: S [0,128),
// P planes [128,320), O [320,384).  Shared memory: three planes each of Q, K and V, 16 KB a plane.
#pragma once
#include "sm100_ptx.cuh"

namespace it {

struct FwdF32Traits {
  static constexpr int BM = 128, BN = 128, DP = 64;      // query rows, keys per tile, padded head_dim
  static constexpr int PLANE_BYTES = 128 * 128;          // [128 rows][64 bf16], 128-byte swizzle
  static constexpr int SMEM_Q = 0;                       // 3 planes
  static constexpr int SMEM_K = SMEM_Q + 3 * PLANE_BYTES;
  static constexpr int SMEM_V = SMEM_K + 3 * PLANE_BYTES;
  static constexpr int SMEM_BAR = SMEM_V + 3 * PLANE_BYTES;
  static constexpr int NUM_BARS = 6;
  static constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = SMEM_MISC + 16;
  static constexpr int THREADS = 288;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t COL_S = 0, COL_P = 128, COL_O = 320;
};

struct FwdF32Params {
  const float* q;
  const float* k;
  const float* v;
  float* o;
  float* lse;              // [BH, S] or null
  ptx::TensorStrides st;   // layout of q and o
  ptx::TensorStrides st_kv;
  int* status;
  int S;
  int D;
  int causal;
  float scale_log2;        // 1/sqrt(D) * log2(e)
};

// The three bf16 terms of two fp32 values, each packed (first value in the low half).
__device__ __forceinline__ void split3_bf16x2(float a, float b, uint32_t* hi, uint32_t* mid, uint32_t* lo) {
  const uint32_t h = ptx::pack_bf16(a, b);
  const float ra = a - __uint_as_float(h << 16), rb = b - __uint_as_float(h & 0xFFFF0000u);
  const uint32_t m = ptx::pack_bf16(ra, rb);
  const float sa = ra - __uint_as_float(m << 16), sb = rb - __uint_as_float(m & 0xFFFF0000u);
  *hi = h;
  *mid = m;
  *lo = ptx::pack_bf16(sa, sb);
}

__global__ void __launch_bounds__(288, 1) fa_fwd_f32_sm100_kernel(const FwdF32Params prm) {
  using T = FwdF32Traits;
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::SMEM_BAR);
  uint64_t* q_ready = bars + 0;   // 128 loader arrivals
  uint64_t* k_ready = bars + 1;   // 128
  uint64_t* v_ready = bars + 2;   // 128
  uint64_t* s_full = bars + 3;    // MMA commit: S(j) complete (and the K planes free)
  uint64_t* p_full = bars + 4;    // 128 softmax arrivals: P(j) planes in tensor memory
  uint64_t* pv_done = bars + 5;   // MMA commit: O += P(j) V(j) complete (V planes and P planes free)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + T::SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = prm.S, D = prm.D;
  const int n_qt = (S + T::BM - 1) / T::BM;
  const int bh = static_cast<int>(blockIdx.x) / n_qt;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x) % n_qt;   // most keys first
  const int n_kt = (S + T::BN - 1) / T::BN;
  const int n_kv = prm.causal ? min(qt + 1, n_kt) : n_kt;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if (smem_addr(smem) & 1023u) {
      *abort_flag = 1;
      atomicCAS(prm.status, 0, DEV_ERR_SMEM_ALIGN);
    }
    if (*reinterpret_cast<volatile int*>(prm.status) != 0) *abort_flag = 1;
    mbar_init(q_ready, 128);
    mbar_init(k_ready, 128);
    mbar_init(v_ready, 128);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool run = (*abort_flag == 0);

  if (!run) {
    // nothing to do
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------ loaders
    const int t = threadIdx.x - 128;
    // A thread owns float4 column c4 of rows r0, r0 + rstep, ...: with 16 float4 per row (head_dim 64) eight rows per
    // pass of the 128 loaders, sixteen passes per tile.  Shorter rows leave the upper lanes of each group idle.
    const int nd4 = D >> 2;                       // float4 per row
    constexpr int MAXV = 16;                      // float4 per thread and tile
    const int c4 = t & 15, r0 = t >> 4;           // 16 lanes per row, rows r0 + 8 * i
    const bool col_ok = c4 < nd4;
    // fp32 rows of tile `tile` of a tensor into registers (rows past S read as zero)
    auto fetch = [&](const float* base, long long row_stride, int tile, float4 (&r)[MAXV]) {
      const float* p = base + static_cast<long long>(tile * 128 + r0) * row_stride + 4 * c4;
      const int s0 = tile * 128 + r0;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        r[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (col_ok && s0 + 8 * i < S) r[i] = __ldg(reinterpret_cast<const float4*>(p + static_cast<long long>(8 * i) * row_stride));
      }
    };
    // split and store as three swizzled bf16 planes
    auto store_planes = [&](uint8_t* planes, const float4 (&r)[MAXV]) {
      if (!col_ok) return;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int row = r0 + 8 * i;
        {
          uint32_t h0, m0, l0, h1, m1, l1;
          split3_bf16x2(r[i].x, r[i].y, &h0, &m0, &l0);
          split3_bf16x2(r[i].z, r[i].w, &h1, &m1, &l1);
          const uint32_t off = swz128_offset(row, c4 * 4);
          *reinterpret_cast<uint2*>(planes + off) = make_uint2(h0, h1);
          *reinterpret_cast<uint2*>(planes + T::PLANE_BYTES + off) = make_uint2(m0, m1);
          *reinterpret_cast<uint2*>(planes + 2 * T::PLANE_BYTES + off) = make_uint2(l0, l1);
        }
      }
    };
    if (D < T::DP) {   // columns past head_dim: zero in every plane, written once
      for (int i = t; i < 9 * T::PLANE_BYTES / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the loaders only; nothing else has started on these buffers
    }
    const float* qb = prm.q + prm.st.slice(bh);
    const float* kb = prm.k + prm.st_kv.slice(bh);
    const float* vb = prm.v + prm.st_kv.slice(bh);
    float4 rk[MAXV], rv[MAXV];
    fetch(qb, prm.st.row, qt, rk);
    fetch(kb, prm.st_kv.row, 0, rv);
    store_planes(smem + T::SMEM_Q, rk);
    fence_proxy_async_smem();
    mbar_arrive(q_ready);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) rk[i] = rv[i];
    fetch(vb, prm.st_kv.row, 0, rv);
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (j > 0) {   // S(j-1) has been computed: the K planes may be rewritten
        ok = mbar_wait(s_full, (j - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      store_planes(smem + T::SMEM_K, rk);
      fence_proxy_async_smem();
      mbar_arrive(k_ready);
      if (j + 1 < n_kv) fetch(kb, prm.st_kv.row, j + 1, rk);
      if (j > 0) {   // P(j-1) V(j-1) is complete: the V planes may be rewritten
        ok = mbar_wait(pv_done, (j - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      store_planes(smem + T::SMEM_V, rv);
      fence_proxy_async_smem();
      mbar_arrive(v_ready);
      if (j + 1 < n_kv) fetch(vb, prm.st_kv.row, j + 1, rv);
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
      constexpr uint32_t IDESC_PV = make_idesc(128, T::DP, false, true);
      const uint32_t q_addr = smem_addr(smem + T::SMEM_Q), k_addr = smem_addr(smem + T::SMEM_K),
                     v_addr = smem_addr(smem + T::SMEM_V);
      // term pairs (a plane, b plane) of order above 2^-24: hi hi, hi mid, mid hi, hi lo, mid mid, lo hi
      constexpr int TA[6] = {0, 0, 1, 0, 1, 2};
      constexpr int TB[6] = {0, 1, 0, 2, 1, 0};
      bool ok = mbar_wait(q_ready, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
      for (int j = 0; j < n_kv && ok; ++j) {
        ok = mbar_wait(k_ready, j & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int term = 0; term < 6; ++term) {
          const uint64_t da = make_sdesc(q_addr + TA[term] * T::PLANE_BYTES, 16, 1024);
          const uint64_t db = make_sdesc(k_addr + TB[term] * T::PLANE_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < T::DP / 16; ++kk)
            umma_ss(tmem_base + T::COL_S, sdesc_advance(da, kk * 32), sdesc_advance(db, kk * 32), IDESC_S,
                    (term > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(s_full);
        ok = mbar_wait(p_full, j & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
        if (ok) ok = mbar_wait(v_ready, j & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int term = 0; term < 6; ++term) {
          const uint64_t db = make_sdesc(v_addr + TB[term] * T::PLANE_BYTES, T::PLANE_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < T::BN / 16; ++kk)
            umma_ts(tmem_base + T::COL_O, tmem_base + T::COL_P + TA[term] * 64 + kk * 8, sdesc_advance(db, kk * 2048), IDESC_PV,
                    (j > 0 || term > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 0-3)
    const int lane_base = warp * 32;
    const int q_row = qt * T::BM + lane_base + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
    const float sl2 = prm.scale_log2;
    const int k_limit = prm.causal ? min(S - 1, q_row) : (S - 1);   // last visible key index
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    uint32_t r[32];   // 32 columns of this thread's row at a time: two passes over S (maximum, then P) keep the code small
    for (int j = 0; j < n_kv; ++j) {
      ok = mbar_wait(s_full, j & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool edge = (prm.causal && j == qt) || ((j + 1) * T::BN > S);   // diagonal or ragged last tile
      const int vis = edge ? k_limit - j * T::BN : 127;                     // columns 0..vis are visible
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_x32(t_lane + T::COL_S + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float a0 = (c * 32 + i <= vis) ? __uint_as_float(r[i]) : -INFINITY;
          const float a1 = (c * 32 + i + 1 <= vis) ? __uint_as_float(r[i + 1]) : -INFINITY;
          mx = fmax3(mx, a0, a1);
        }
      }
      float m_new = mx * sl2;
      if (m_new == -INFINITY) m_new = 0.f;   // a row past S: nothing visible, keep everything finite
      if (j > 0) {   // P(j-1) V(j-1) must be complete before O is rescaled or the P planes are rewritten
        ok = mbar_wait(pv_done, (j - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
      }
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m_used + 8.0f)) {   // rare: raise the reference, rescale O
        const float m_next = fmaxf(m_used, m_new);
        const float f = ex2(m_used - m_next);
        l_sum *= f;
        m_used = m_next;
        uint32_t tmp[16];
#pragma unroll 1
        for (int c = 0; c < T::DP / 16; ++c) {
          tmem_ld_x16(t_lane + T::COL_O + c * 16, tmp);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) tmp[i] = __float_as_uint(__uint_as_float(tmp[i]) * f);
          tmem_st_x16(t_lane + T::COL_O + c * 16, tmp);
        }
        tmem_wait_st();
      }
      // P = 2^(s*c - m) in fp32, summed in fp32, handed to the tensor core as three bf16 planes
      const float neg_m = -m_used;
      float l0 = 0.f, l1 = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t ph[16], pm[16], pl[16];
        tmem_ld_x32(t_lane + T::COL_S + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2(fmaf(__uint_as_float(r[i]), sl2, neg_m));
          float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), sl2, neg_m));
          if (c * 32 + i > vis) p0 = 0.f;
          if (c * 32 + i + 1 > vis) p1 = 0.f;
          l0 += p0;
          l1 += p1;
          split3_bf16x2(p0, p1, &ph[i >> 1], &pm[i >> 1], &pl[i >> 1]);
        }
        tmem_st_x16(t_lane + T::COL_P + c * 16, ph);
        tmem_st_x16(t_lane + T::COL_P + 64 + c * 16, pm);
        tmem_st_x16(t_lane + T::COL_P + 128 + c * 16, pl);
      }
      l_sum += l0 + l1;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok) {
      ok = mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l_sum;
      float* orow = prm.o + prm.st.slice(bh) + static_cast<long long>(q_row) * prm.st.row;
#pragma unroll 1
      for (int c = 0; c < T::DP / 32; ++c) {
        tmem_ld_x32(t_lane + T::COL_O + c * 32, r);
        tmem_wait_ld();
        if (q_row < S) {
#pragma unroll
          for (int c4 = 0; c4 < 8; ++c4)
            if (c * 32 + c4 * 4 < D)
              reinterpret_cast<float4*>(orow)[c * 8 + c4] =
                  make_float4(__uint_as_float(r[c4 * 4]) * inv_l, __uint_as_float(r[c4 * 4 + 1]) * inv_l,
                              __uint_as_float(r[c4 * 4 + 2]) * inv_l, __uint_as_float(r[c4 * 4 + 3]) * inv_l);
        }
      }
      if (q_row < S) {
        if (prm.lse != nullptr) prm.lse[static_cast<size_t>(bh) * S + q_row] = (m_used + lg2(l_sum)) * 0.6931471805599453f;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    if (*abort_flag)
      for (int i = 0; i < 50; ++i) __nanosleep(20000);
    tc_fence_after();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace it
