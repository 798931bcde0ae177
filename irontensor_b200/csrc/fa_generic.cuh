// CUDA-core attention kernels with fp32 arithmetic: the path for fp32 tensors (the reference's
// FP32 mode, src/ops/flash_attention.rs:76-193) and for bf16 shapes the tensor-core kernels do not
// take (head_dim other than 64/128, sequences shorter than one 128-row tile).  Any S >= 1, any
// 1 <= D <= 128, causal or full.  Storage type ST is float or __nv_bfloat16; math is fp32, the
// exponentials in the exp2 domain (ex2.approx / lg2.approx, relative error 2^-22), which keeps the
// fp32 mode within 1e-4 (measured: 2e-6) of the reference's scalar kernels.
//
// Forward: a CTA owns 64 query rows of one (batch, head); four threads share a row, each holding
// a quarter of the head dimension of q and of the output accumulator.  Keys and values stream
// through shared memory in tiles; scores for 16 keys at a time are completed with two shuffles,
// then folded into an online softmax (same recurrence as src/shaders/flash_attention.metal:27-41).
// Backward: one warp per query row (dQ) and one warp per key row (dK, dV), P recomputed from the
// forward's LSE, delta = rowsum(dO*O).  No atomics, so results are bit-reproducible.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

#include "layout.cuh"
#include "rope.cuh"

namespace it {

__device__ __forceinline__ float g_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float g_lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename ST> __device__ __forceinline__ float ld_as_f32(const ST* p);
template <> __device__ __forceinline__ float ld_as_f32<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_as_f32<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename ST> __device__ __forceinline__ void st_from_f32(ST* p, float v);
template <> __device__ __forceinline__ void st_from_f32<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_from_f32<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

// DP: head_dim rounded up to 16, 32, 64 or 128.  BN keys per shared-memory tile.
template <typename ST, int DP>
__global__ void __launch_bounds__(256)
fa_fwd_generic_kernel(const ST* __restrict__ q, const ST* __restrict__ k, const ST* __restrict__ v,
                      ST* __restrict__ o, float* __restrict__ lse, int S, int Skv, int D, int causal, float scale_log2,
                      TensorStrides st, TensorStrides skv) {
  // S query rows against Skv keys; a causal launch has Skv == S (src/ops/attention.rs:349-352).
  constexpr int BM = 64;
  constexpr int BN = (DP >= 128) ? 32 : 64;
  constexpr int NCH = DP / 16;              // float4 chunks per thread
  __shared__ __align__(16) float sK[BN * DP];
  __shared__ __align__(16) float sV[BN * DP];

  const int tid = threadIdx.x;
  const int t4 = tid & 3;
  const int r_local = tid >> 2;
  const int n_rt = (S + BM - 1) / BM;
  const int rt = n_rt - 1 - static_cast<int>(blockIdx.x);     // heaviest row tiles first
  const int bh = blockIdx.y;
  const int row = rt * BM + r_local;
  const bool row_ok = row < S;
  const size_t base = static_cast<size_t>(st.slice(bh));
  const size_t RS = static_cast<size_t>(st.row);
  const size_t kbase = static_cast<size_t>(skv.slice(bh));   // the K/V head this query head reads
  const size_t KRS = static_cast<size_t>(skv.row);

  float4 qv[NCH], acc[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int d0 = 4 * (t4 + 4 * j);
    float tmp[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      tmp[e] = (row_ok && d0 + e < D) ? ld_as_f32(q + base + static_cast<size_t>(row) * RS + d0 + e) : 0.f;
    qv[j] = make_float4(tmp[0], tmp[1], tmp[2], tmp[3]);
    acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m_run = -INFINITY, l_run = 0.f;

  const int row_hi = min(S, (rt + 1) * BM) - 1;               // last valid row of this CTA
  const int k_end = causal ? (row_hi + 1) : Skv;              // keys [0, k_end)
  for (int k0 = 0; k0 < k_end; k0 += BN) {
    const int nk = min(BN, k_end - k0);
    __syncthreads();
    for (int i = tid; i < BN * DP; i += 256) {
      const int kk = i / DP, d = i % DP;
      const bool okk = (kk < nk) && (d < D);
      const size_t g = kbase + static_cast<size_t>(k0 + kk) * KRS + d;
      sK[i] = okk ? ld_as_f32(k + g) : 0.f;
      sV[i] = okk ? ld_as_f32(v + g) : 0.f;
    }
    __syncthreads();
    for (int g0 = 0; g0 < nk; g0 += 16) {
      float sc[16];
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const float4* kr = reinterpret_cast<const float4*>(sK + (g0 + kk) * DP);
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const float4 kv = kr[t4 + 4 * j];
          a = fmaf(qv[j].x, kv.x, a);
          a = fmaf(qv[j].y, kv.y, a);
          a = fmaf(qv[j].z, kv.z, a);
          a = fmaf(qv[j].w, kv.w, a);
        }
        a += __shfl_xor_sync(0xffffffffu, a, 1);
        a += __shfl_xor_sync(0xffffffffu, a, 2);
        const int kidx = k0 + g0 + kk;
        const bool vis = (g0 + kk < nk) && (!causal || kidx <= row);
        sc[kk] = vis ? a * scale_log2 : -INFINITY;
      }
      float gmax = sc[0];
#pragma unroll
      for (int kk = 1; kk < 16; ++kk) gmax = fmaxf(gmax, sc[kk]);
      const float m_new = fmaxf(m_run, gmax);
      // Nothing visible to this row yet: keep the state at (-inf, 0) without producing NaN.
      const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = g_ex2(m_run - m_ref);
      l_run *= corr;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        acc[j].x *= corr; acc[j].y *= corr; acc[j].z *= corr; acc[j].w *= corr;
      }
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const float p = g_ex2(sc[kk] - m_ref);
        l_run += p;
        const float4* vr = reinterpret_cast<const float4*>(sV + (g0 + kk) * DP);
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const float4 vv = vr[t4 + 4 * j];
          acc[j].x = fmaf(p, vv.x, acc[j].x);
          acc[j].y = fmaf(p, vv.y, acc[j].y);
          acc[j].z = fmaf(p, vv.z, acc[j].z);
          acc[j].w = fmaf(p, vv.w, acc[j].w);
        }
      }
      m_run = m_new;
    }
  }
  if (row_ok) {
    const float inv = 1.0f / l_run;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int d0 = 4 * (t4 + 4 * j);
      const float tmp[4] = {acc[j].x * inv, acc[j].y * inv, acc[j].z * inv, acc[j].w * inv};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (d0 + e < D) st_from_f32(o + base + static_cast<size_t>(row) * RS + d0 + e, tmp[e]);
    }
    if (lse != nullptr && t4 == 0)
      lse[static_cast<size_t>(bh) * S + row] = (m_run + g_lg2(l_run)) * 0.6931471805599453f;
  }
}

// fp32 tensors with D a multiple of 4 and short to medium sequences: the latency path (the greedy
// no-KV-cache inference pattern re-runs it once per generated token, and the reference's TINY model
// sits at S = 256).  A CTA owns RB (16 or 32) consecutive query rows of one head, RW (two, four or eight) per warp.  Keys and
// values stream through shared memory 32 at a time (cp.async, double buffered, rows padded by four
// floats so that lane-per-key float4 reads are conflict free).  Scores: one key per lane, each K
// chunk read once and used for all of the warp's rows; softmax: online, warp-reduced per tile (the
// recurrence of src/shaders/flash_attention.metal:27-41); output: lanes over the head dimension,
// the tile's probabilities parked in shared memory and read back four keys at a time, V read from
// shared memory.  NJ = ceil(D / 32) output elements per lane.
template <int NJ, int RW, int RB = 16>
__global__ void __launch_bounds__(32 * (RB / RW))
fa_fwd_rows_f32_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       float* __restrict__ o, float* __restrict__ lse, int S, int Skv, int D, int causal, float scale_log2,
                       TensorStrides st, TensorStrides skv) {
  constexpr int TK = 32, NT = 32 * (RB / RW);   // RB rows per CTA: RB / RW warps, RW rows each
  // Launched as a programmatic dependent: a chain of per-token calls (generation without a key/value cache) then pays
  // each call's launch latency under the previous call's execution.  The inputs may be what the kernel in front wrote.
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  extern __shared__ __align__(16) float sm[];
  const int DS = D + 4;                       // padded row stride (floats)
  float* sQ = sm;                             // [RB][D]
  float* sK = sQ + RB * D;                    // [2][TK][DS]
  float* sV = sK + 2 * TK * DS;               // [2][TK][DS]
  float* sP = sV + 2 * TK * DS;               // [warps][RW][TK] probabilities of the current tile
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nd4 = D >> 2;
  const int n_rb = (S + RB - 1) / RB;
  const int rb = n_rb - 1 - static_cast<int>(blockIdx.x);    // longest rows first
  const int bh = blockIdx.y;
  const int r0 = rb * RB;
  const size_t base = static_cast<size_t>(st.slice(bh));
  const size_t RS = static_cast<size_t>(st.row);
  const size_t kbase = static_cast<size_t>(skv.slice(bh));   // the K/V head this query head reads
  const size_t KRS = static_cast<size_t>(skv.row);
  const int k_end_cta = causal ? min(S, r0 + RB) : Skv;
  const int n_tiles = (k_end_cta + TK - 1) / TK;

  auto load_tile = [&](int tile, int buf) {
    const int k0 = tile * TK;
    float* dk = sK + buf * TK * DS;
    float* dv = sV + buf * TK * DS;
    for (int idx = tid; idx < TK * nd4; idx += NT) {
      const int key = idx / nd4, c = idx - key * nd4;
      float* pk = dk + key * DS + 4 * c;
      float* pv = dv + key * DS + 4 * c;
      if (k0 + key < k_end_cta) {
        const size_t g = kbase + static_cast<size_t>(k0 + key) * KRS + 4 * c;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(pk))), "l"(k + g));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(pv))), "l"(v + g));
      } else {   // rows past the end: zeros, so that 0 * V stays 0
        *reinterpret_cast<float4*>(pk) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(pv) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  load_tile(0, 0);
  for (int idx = tid; idx < RB * nd4; idx += NT) {
    const int rr = idx / nd4, c = idx - rr * nd4;
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r0 + rr < S) val = reinterpret_cast<const float4*>(q + base + static_cast<size_t>(r0 + rr) * RS)[c];
    reinterpret_cast<float4*>(sQ + rr * D)[c] = val;
  }

  float m_run[RW], l_run[RW], acc[RW][NJ];
  int lim[RW];                                  // last visible key of each of this warp's rows
  int lim_max = -1;
#pragma unroll
  for (int w = 0; w < RW; ++w) {
    const int row = r0 + warp * RW + w;
    m_run[w] = -INFINITY;
    l_run[w] = 0.f;
    lim[w] = (row < S) ? (causal ? row : Skv - 1) : -1;
    lim_max = max(lim_max, lim[w]);
#pragma unroll
    for (int jj = 0; jj < NJ; ++jj) acc[w][jj] = 0.f;
  }

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) {
      load_tile(tile + 1, buf ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int k0 = tile * TK;
    if (k0 <= lim_max) {   // some row of this warp sees a key of the tile
      const float4* kp = reinterpret_cast<const float4*>(sK + buf * TK * DS + lane * DS);
      const float4* qp = reinterpret_cast<const float4*>(sQ + warp * RW * D);
      float dot[RW], dot2[RW];
#pragma unroll
      for (int w = 0; w < RW; ++w) dot[w] = dot2[w] = 0.f;
#pragma unroll 4
      for (int c = 0; c < nd4; ++c) {
        const float4 kv = kp[c];
#pragma unroll
        for (int w = 0; w < RW; ++w) {
          const float4 qv = qp[w * nd4 + c];
          dot[w] = fmaf(qv.x, kv.x, dot[w]);
          dot2[w] = fmaf(qv.y, kv.y, dot2[w]);
          dot[w] = fmaf(qv.z, kv.z, dot[w]);
          dot2[w] = fmaf(qv.w, kv.w, dot2[w]);
        }
      }
      float* pw = sP + warp * RW * TK;
      float p[RW];
#pragma unroll
      for (int w = 0; w < RW; ++w) {
        const float s2 = (k0 + lane <= lim[w]) ? (dot[w] + dot2[w]) * scale_log2 : -INFINITY;
        float tmax = s2;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
        const float m_new = fmaxf(m_run[w], tmax);
        const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;   // nothing visible yet: stay at (-inf, 0)
        p[w] = g_ex2(s2 - m_ref);
        pw[w * TK + lane] = p[w];
        float psum = p[w];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, off);
        const float corr = g_ex2(m_run[w] - m_ref);
        l_run[w] = l_run[w] * corr + psum;
#pragma unroll
        for (int jj = 0; jj < NJ; ++jj) acc[w][jj] *= corr;
        m_run[w] = m_new;
      }
      __syncwarp();
      const float* vp = sV + buf * TK * DS + lane;
#pragma unroll 2
      for (int kk = 0; kk < TK; kk += 4) {
        float4 p4[RW];
#pragma unroll
        for (int w = 0; w < RW; ++w) p4[w] = *reinterpret_cast<const float4*>(pw + w * TK + kk);   // broadcast read
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float vv[NJ];
#pragma unroll
          for (int jj = 0; jj < NJ; ++jj) vv[jj] = (lane + 32 * jj < D) ? vp[(kk + e) * DS + 32 * jj] : 0.f;
#pragma unroll
          for (int w = 0; w < RW; ++w) {
            const float pk = e == 0 ? p4[w].x : e == 1 ? p4[w].y : e == 2 ? p4[w].z : p4[w].w;
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) acc[w][jj] = fmaf(pk, vv[jj], acc[w][jj]);
          }
        }
      }
      __syncwarp();   // the warp's probability buffer is rewritten by the next tile
    }
    __syncthreads();   // everyone is done with this buffer before the next load overwrites it
  }
#pragma unroll
  for (int w = 0; w < RW; ++w) {
    const int row = r0 + warp * RW + w;
    if (row < S) {
      const float inv = 1.0f / l_run[w];
#pragma unroll
      for (int jj = 0; jj < NJ; ++jj) {
        const int d = lane + 32 * jj;
        if (d < D) o[base + static_cast<size_t>(row) * RS + d] = acc[w][jj] * inv;
      }
      if (lse != nullptr && lane == 0)
        lse[static_cast<size_t>(bh) * S + row] = (m_run[w] + g_lg2(l_run[w])) * 0.6931471805599453f;
    }
  }
}

// delta[bh, s] = sum_d dO * O, one warp per row.
template <typename ST>
__global__ void fa_bwd_generic_delta_kernel(const ST* __restrict__ o, const ST* __restrict__ d_o,
                                            float* __restrict__ delta, long long rows, int S, int D, TensorStrides st) {
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  const int bh = static_cast<int>(row / S);
  const long long off = st.slice(bh) + (row - static_cast<long long>(bh) * S) * st.row;
  float a = 0.f;
  for (int d = lane; d < D; d += 32) a = fmaf(ld_as_f32(o + off + d), ld_as_f32(d_o + off + d), a);
#pragma unroll
  for (int off2 = 16; off2 > 0; off2 >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off2);
  if (lane == 0) delta[row] = a;
}

// MODE 0: one warp per query row -> dQ.   MODE 1: one warp per key row of a K/V head -> dK, dV, summed
// over the query heads of its group (the reference's repeat_kv_backward, src/shaders/repeat_kv.metal:49-88,
// folded in).  Lanes split the head dimension (lane, lane+32, ...); the two dot products per
// (query, key) pair are completed with a butterfly over the warp.  blockIdx.y is the query slice
// (MODE 0) or the K/V slice batch * kv_heads + kv_head (MODE 1).
template <typename ST, int MODE>
__global__ void __launch_bounds__(128)
fa_bwd_generic_kernel(const ST* __restrict__ q, const ST* __restrict__ k, const ST* __restrict__ v,
                      const ST* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta,
                      ST* __restrict__ dq, ST* __restrict__ dk, ST* __restrict__ dv, int S, int D, int causal,
                      float scale, TensorStrides st, TensorStrides skv, const __grid_constant__ RopeFreqs freqs) {
  const int lane = threadIdx.x & 31;
  const int r = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5);
  if (r >= S) return;
  const int G = (MODE == 0) ? 1 : skv.group;
  const int kv_heads = skv.heads / skv.group;
  // first query slice this warp works on: its own (MODE 0), or the first of the K/V head's group (MODE 1)
  const int bh0 = (MODE == 0) ? static_cast<int>(blockIdx.y)
                              : (static_cast<int>(blockIdx.y) / kv_heads) * skv.heads +
                                    (static_cast<int>(blockIdx.y) % kv_heads) * skv.group;
  const size_t kbase = static_cast<size_t>(skv.slice(bh0));
  const size_t KRS = static_cast<size_t>(skv.row);
  const size_t RS = static_cast<size_t>(st.row);
  float a0[4], a1[4], g0[4], g1[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane + 32 * j;
    const bool in = d < D;
    if (MODE == 0) {
      const size_t off = static_cast<size_t>(st.slice(bh0)) + static_cast<size_t>(r) * RS + d;
      a0[j] = in ? ld_as_f32(q + off) : 0.f;     // q_i
      a1[j] = in ? ld_as_f32(d_o + off) : 0.f;   // dO_i
    } else {
      const size_t off = kbase + static_cast<size_t>(r) * KRS + d;
      a0[j] = in ? ld_as_f32(k + off) : 0.f;     // k_j
      a1[j] = in ? ld_as_f32(v + off) : 0.f;     // v_j
    }
    g0[j] = 0.f;
    g1[j] = 0.f;
  }
  const int lo = (MODE == 0) ? 0 : (causal ? r : 0);
  const int hi = (MODE == 0) ? (causal ? r + 1 : S) : S;
  for (int g = 0; g < G; ++g) {
    const int bh = bh0 + g;
    const size_t base = static_cast<size_t>(st.slice(bh));
    const float* lse_h = lse + static_cast<size_t>(bh) * S;
    const float* dl_h = delta + static_cast<size_t>(bh) * S;
    const float lse_r = (MODE == 0) ? lse_h[r] : 0.f;
    const float dl_r = (MODE == 0) ? dl_h[r] : 0.f;
    for (int x = lo; x < hi; ++x) {
      float b0[4], b1[4];
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int d = lane + 32 * j;
        const bool in = d < D;
        if (MODE == 0) {
          const size_t off = kbase + static_cast<size_t>(x) * KRS + d;
          b0[j] = in ? ld_as_f32(k + off) : 0.f;   // k_x
          b1[j] = in ? ld_as_f32(v + off) : 0.f;   // v_x
        } else {
          const size_t off = base + static_cast<size_t>(x) * RS + d;
          b0[j] = in ? ld_as_f32(q + off) : 0.f;   // q_x
          b1[j] = in ? ld_as_f32(d_o + off) : 0.f; // dO_x
        }
        s = fmaf(a0[j], b0[j], s);
        dp = fmaf(a1[j], b1[j], dp);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, off);
        dp += __shfl_xor_sync(0xffffffffu, dp, off);
      }
      const float lse_x = (MODE == 0) ? lse_r : lse_h[x];
      const float dl_x = (MODE == 0) ? dl_r : dl_h[x];
      const float p = g_ex2(fmaf(s, scale * 1.4426950408889634f, -lse_x * 1.4426950408889634f));
      const float ds = p * (dp - dl_x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        g0[j] = fmaf(ds, b0[j], g0[j]);            // dq += ds * k_x   or   dk += ds * q_x
        if (MODE == 1) g1[j] = fmaf(p, b1[j], g1[j]);   // dv += p * dO_x
      }
    }
  }
  if (freqs.enabled) {
    // dQ and dK leave through the inverse rotary rotation of their row's position
    // (src/shaders/backward/rope.metal:25-62); the two elements of a pair sit in neighbouring lanes.
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = lane + 32 * j;
      const float other = __shfl_xor_sync(0xffffffffu, g0[j], 1);
      if (d < D) {
        float c, sn;
        rope_sincos(freqs, r + freqs.position_offset, d >> 1, &c, &sn);
        g0[j] = (d & 1) ? (g0[j] * c - other * sn) : (g0[j] * c + other * sn);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane + 32 * j;
    if (d < D) {
      if (MODE == 0) {
        st_from_f32(dq + static_cast<size_t>(st.slice(bh0)) + static_cast<size_t>(r) * RS + d, g0[j] * scale);
      } else {
        const size_t off = kbase + static_cast<size_t>(r) * KRS + d;
        st_from_f32(dk + off, g0[j] * scale);
        st_from_f32(dv + off, g1[j]);
      }
    }
  }
}

}  // namespace it
