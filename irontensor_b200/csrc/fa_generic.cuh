// CUDA-core attention kernels with fp32 arithmetic: the path for fp32 tensors (the reference's
// FP32 mode, src/ops/flash_attention.rs:76-193) and for bf16 shapes the tensor-core kernels do not
// take (head_dim other than 64/128, sequences shorter than one 128-row tile).  Any S >= 1, any
// 1 <= D <= 128, causal or full.  Storage type ST is float or __nv_bfloat16; math is fp32 with
// libm-accurate expf/logf so the fp32 mode stays within 1e-4 of the reference's scalar kernels.
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

namespace it {

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
                      ST* __restrict__ o, float* __restrict__ lse, int S, int D, int causal, float scale) {
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
  const size_t base = static_cast<size_t>(bh) * S * D;

  float4 qv[NCH], acc[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int d0 = 4 * (t4 + 4 * j);
    float tmp[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      tmp[e] = (row_ok && d0 + e < D) ? ld_as_f32(q + base + static_cast<size_t>(row) * D + d0 + e) : 0.f;
    qv[j] = make_float4(tmp[0], tmp[1], tmp[2], tmp[3]);
    acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m_run = -INFINITY, l_run = 0.f;

  const int row_hi = min(S, (rt + 1) * BM) - 1;               // last valid row of this CTA
  const int k_end = causal ? (row_hi + 1) : S;                // keys [0, k_end)
  for (int k0 = 0; k0 < k_end; k0 += BN) {
    const int nk = min(BN, k_end - k0);
    __syncthreads();
    for (int i = tid; i < BN * DP; i += 256) {
      const int kk = i / DP, d = i % DP;
      const bool okk = (kk < nk) && (d < D);
      const size_t g = base + static_cast<size_t>(k0 + kk) * D + d;
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
        sc[kk] = vis ? a * scale : -INFINITY;
      }
      float gmax = sc[0];
#pragma unroll
      for (int kk = 1; kk < 16; ++kk) gmax = fmaxf(gmax, sc[kk]);
      const float m_new = fmaxf(m_run, gmax);
      // Nothing visible to this row yet: keep the state at (-inf, 0) without producing NaN.
      const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = expf(m_run - m_ref);
      l_run *= corr;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        acc[j].x *= corr; acc[j].y *= corr; acc[j].z *= corr; acc[j].w *= corr;
      }
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const float p = expf(sc[kk] - m_ref);
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
        if (d0 + e < D) st_from_f32(o + base + static_cast<size_t>(row) * D + d0 + e, tmp[e]);
    }
    if (lse != nullptr && t4 == 0) lse[static_cast<size_t>(bh) * S + row] = m_run + logf(l_run);
  }
}

// delta[bh, s] = sum_d dO * O, one warp per row.
template <typename ST>
__global__ void fa_bwd_generic_delta_kernel(const ST* __restrict__ o, const ST* __restrict__ d_o,
                                            float* __restrict__ delta, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  float a = 0.f;
  for (int d = lane; d < D; d += 32) a = fmaf(ld_as_f32(o + row * D + d), ld_as_f32(d_o + row * D + d), a);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
  if (lane == 0) delta[row] = a;
}

// MODE 0: one warp per query row -> dQ.   MODE 1: one warp per key row -> dK, dV.
// Lanes split the head dimension (lane, lane+32, ...); the two dot products per (query, key)
// pair are completed with a butterfly over the warp.
template <typename ST, int MODE>
__global__ void __launch_bounds__(128)
fa_bwd_generic_kernel(const ST* __restrict__ q, const ST* __restrict__ k, const ST* __restrict__ v,
                      const ST* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta,
                      ST* __restrict__ dq, ST* __restrict__ dk, ST* __restrict__ dv, int S, int D, int causal,
                      float scale) {
  const int lane = threadIdx.x & 31;
  const int r = static_cast<int>((static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5);
  const int bh = blockIdx.y;
  if (r >= S) return;
  const size_t base = static_cast<size_t>(bh) * S * D;
  const float* lse_h = lse + static_cast<size_t>(bh) * S;
  const float* dl_h = delta + static_cast<size_t>(bh) * S;
  float a0[4], a1[4], g0[4], g1[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane + 32 * j;
    const bool in = d < D;
    const size_t off = base + static_cast<size_t>(r) * D + d;
    if (MODE == 0) {
      a0[j] = in ? ld_as_f32(q + off) : 0.f;     // q_i
      a1[j] = in ? ld_as_f32(d_o + off) : 0.f;   // dO_i
    } else {
      a0[j] = in ? ld_as_f32(k + off) : 0.f;     // k_j
      a1[j] = in ? ld_as_f32(v + off) : 0.f;     // v_j
    }
    g0[j] = 0.f;
    g1[j] = 0.f;
  }
  const int lo = (MODE == 0) ? 0 : (causal ? r : 0);
  const int hi = (MODE == 0) ? (causal ? r + 1 : S) : S;
  const float lse_r = (MODE == 0) ? lse_h[r] : 0.f;
  const float dl_r = (MODE == 0) ? dl_h[r] : 0.f;
  for (int x = lo; x < hi; ++x) {
    float b0[4], b1[4];
    float s = 0.f, dp = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = lane + 32 * j;
      const bool in = d < D;
      const size_t off = base + static_cast<size_t>(x) * D + d;
      if (MODE == 0) {
        b0[j] = in ? ld_as_f32(k + off) : 0.f;   // k_x
        b1[j] = in ? ld_as_f32(v + off) : 0.f;   // v_x
        s = fmaf(a0[j], b0[j], s);
        dp = fmaf(a1[j], b1[j], dp);
      } else {
        b0[j] = in ? ld_as_f32(q + off) : 0.f;   // q_x
        b1[j] = in ? ld_as_f32(d_o + off) : 0.f; // dO_x
        s = fmaf(a0[j], b0[j], s);
        dp = fmaf(a1[j], b1[j], dp);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, off);
      dp += __shfl_xor_sync(0xffffffffu, dp, off);
    }
    const float lse_x = (MODE == 0) ? lse_r : lse_h[x];
    const float dl_x = (MODE == 0) ? dl_r : dl_h[x];
    const float p = expf(s * scale - lse_x);
    const float ds = p * (dp - dl_x);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (MODE == 0) {
        g0[j] = fmaf(ds, b0[j], g0[j]);          // dq += ds * k_x
      } else {
        g0[j] = fmaf(ds, b0[j], g0[j]);          // dk += ds * q_x
        g1[j] = fmaf(p, b1[j], g1[j]);           // dv += p * dO_x
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane + 32 * j;
    if (d < D) {
      const size_t off = base + static_cast<size_t>(r) * D + d;
      if (MODE == 0) {
        st_from_f32(dq + off, g0[j] * scale);
      } else {
        st_from_f32(dk + off, g0[j] * scale);
        st_from_f32(dv + off, g1[j]);
      }
    }
  }
}

}  // namespace it
