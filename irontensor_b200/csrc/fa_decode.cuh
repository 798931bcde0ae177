// Attention for one new token per sequence against a key/value cache ("decode"): q [batch, heads, D],
// caches [batch, max_len, kv_heads, D], the first kv_len positions valid.
//
// The reference has no key/value cache: its generator re-runs the whole forward for every token
// (src/inference/generator.rs:146-200) and lists the cache as future work (docs/PRESENTATION.md:576).
// The result here equals the last row of its causal attention over the kv_len tokens
// (src/shaders/flash_attention.metal:167-223 with q = kv_len - 1), computed from the cache alone.
//
// The op is bound by reading the cache once (2 * kv_len * kv_heads * D elements per batch entry), so:
//   * a CTA serves ALL query heads of one K/V head (grouped-query attention: the cache rows are read once
//     per group, not once per query head), in chunks of at most 8 heads;
//   * the keys are split over several CTAs when batch * kv_heads alone cannot fill the GPU (split-KV);
//     each split leaves an unnormalised partial output and its (max, sum), and a small second kernel
//     merges them (the same online-softmax recurrence as flash_attention.metal:27-41, across splits);
//   * K and V tiles of 64 keys go through shared memory with rows padded so that both the lane-per-key
//     score pass (16-byte reads down a column of rows) and the lane-per-dimension output pass are free
//     of bank conflicts; several CTAs per SM hide the load latency.
// CUDA cores, fp32 math in the exp2 domain; bf16 or fp32 storage; D a multiple of 8, at most 128.
// This file is the general path.  bf16 caches with head_dim 64 or 128 and at least 256 positions go through
// the tensor-core pipeline instead (fa_fwd_pp_sm100.cuh, DECODE), which streams the cache by TMA and is
// several times faster; both leave the same partial results for fa_decode_merge_kernel.
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace it {

constexpr int DEC_TK = 64;      // keys per shared-memory tile
constexpr int DEC_GC = 8;       // query heads per CTA at most
constexpr int DEC_THREADS = 128;

template <typename ST> struct DecVec;   // 16 bytes of storage as floats
template <> struct DecVec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
};
template <> struct DecVec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};
__device__ __forceinline__ float dec_ld(const float* p) { return *p; }
__device__ __forceinline__ float dec_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void dec_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void dec_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float dec_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct DecodeParams {
  int H, Hkv, D;
  int kv_len;          // valid cache positions
  long long cache_batch_stride;   // elements between batch entries of a cache (max_len * Hkv * D)
  int n_splits;
  int split_len;       // keys per split, a multiple of DEC_TK
  float scale_log2;    // 1/sqrt(D) * log2(e)
};

// grid: (n_splits, batch * Hkv, head chunks of the group).  Dynamic shared memory:
//   q [GC][D] fp32 | K tile [TK][D + pad] ST | V tile [TK][D + pad] ST | p [GC][TK] fp32 | corr, m, l [GC] fp32
template <typename ST>
__global__ void __launch_bounds__(DEC_THREADS)
fa_decode_split_kernel(const ST* __restrict__ q, const ST* __restrict__ k_cache, const ST* __restrict__ v_cache,
                       ST* __restrict__ o, float* __restrict__ lse, float* __restrict__ part_o,
                       float* __restrict__ part_ml, const DecodeParams prm) {
  constexpr int VN = DecVec<ST>::N;
  constexpr int PAD = 16 / sizeof(ST);   // 16 bytes: row stride = 4 banks mod 32 -> conflict free
  extern __shared__ __align__(16) uint8_t dec_smem[];
  const int D = prm.D, RS = D + PAD;
  float* s_q = reinterpret_cast<float*>(dec_smem);
  ST* s_k = reinterpret_cast<ST*>(s_q + DEC_GC * D);
  ST* s_v = s_k + DEC_TK * RS;
  float* s_p = reinterpret_cast<float*>(s_v + DEC_TK * RS);
  float* s_corr = s_p + DEC_GC * DEC_TK;
  float* s_m = s_corr + DEC_GC;
  float* s_l = s_m + DEC_GC;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = prm.H / prm.Hkv;
  const int b = static_cast<int>(blockIdx.y) / prm.Hkv, hk = static_cast<int>(blockIdx.y) % prm.Hkv;
  const int g0 = static_cast<int>(blockIdx.z) * DEC_GC;           // first head of this chunk within the group
  const int gc = min(DEC_GC, G - g0);                             // heads in this chunk
  const int h0 = hk * G + g0;                                     // first query head
  const int sp = blockIdx.x;
  const int k_begin = sp * prm.split_len;
  const int k_end = min(prm.kv_len, k_begin + prm.split_len);

  for (int i = tid; i < gc * D; i += DEC_THREADS)
    s_q[i] = dec_ld(q + (static_cast<size_t>(b) * prm.H + h0) * D + i) * prm.scale_log2;
  if (tid < DEC_GC) {
    s_m[tid] = -INFINITY;
    s_l[tid] = 0.f;
  }
  float acc[DEC_GC];
#pragma unroll
  for (int g = 0; g < DEC_GC; ++g) acc[g] = 0.f;
  const size_t row_stride = static_cast<size_t>(prm.Hkv) * D;
  const ST* kb = k_cache + static_cast<size_t>(b) * prm.cache_batch_stride + static_cast<size_t>(hk) * D;
  const ST* vb = v_cache + static_cast<size_t>(b) * prm.cache_batch_stride + static_cast<size_t>(hk) * D;
  const int vec_per_row = D / VN;

  for (int k0 = k_begin; k0 < k_end; k0 += DEC_TK) {
    const int nk = min(DEC_TK, k_end - k0);
    __syncthreads();   // the previous tile's consumers are done (and s_q, s_m, s_l are set on the first pass)
    // eight 16-byte loads per thread are issued before the first is stored: the tile load is latency bound otherwise
    constexpr int LB = 4;
    for (int i0 = tid; i0 < DEC_TK * vec_per_row; i0 += DEC_THREADS * LB) {
      uint4 kk[LB], vv[LB];
#pragma unroll
      for (int u = 0; u < LB; ++u) {
        const int i = i0 + u * DEC_THREADS;
        const int key = i / vec_per_row, c = i - key * vec_per_row;
        kk[u] = make_uint4(0u, 0u, 0u, 0u);
        vv[u] = kk[u];
        if (i < DEC_TK * vec_per_row && key < nk) {
          kk[u] = *reinterpret_cast<const uint4*>(kb + static_cast<size_t>(k0 + key) * row_stride + c * VN);
          vv[u] = *reinterpret_cast<const uint4*>(vb + static_cast<size_t>(k0 + key) * row_stride + c * VN);
        }
      }
#pragma unroll
      for (int u = 0; u < LB; ++u) {
        const int i = i0 + u * DEC_THREADS;
        if (i < DEC_TK * vec_per_row) {
          const int key = i / vec_per_row, c = i - key * vec_per_row;
          *reinterpret_cast<uint4*>(s_k + key * RS + c * VN) = kk[u];
          *reinterpret_cast<uint4*>(s_v + key * RS + c * VN) = vv[u];
        }
      }
    }
    __syncthreads();
    // scores: thread = (key, every other head)
    {
      const int key = tid & (DEC_TK - 1);
      for (int g = tid >> 6; g < gc; g += DEC_THREADS / DEC_TK) {
        const float* qg = s_q + g * D;
        const ST* kr = s_k + key * RS;
        float a0 = 0.f, a1 = 0.f;
        for (int c = 0; c < vec_per_row; ++c) {
          float f[VN];
          DecVec<ST>::load(kr + c * VN, f);
#pragma unroll
          for (int e = 0; e < VN; e += 2) {
            a0 = fmaf(f[e], qg[c * VN + e], a0);
            a1 = fmaf(f[e + 1], qg[c * VN + e + 1], a1);
          }
        }
        s_p[g * DEC_TK + key] = (key < nk) ? (a0 + a1) : -INFINITY;
      }
    }
    __syncthreads();
    // online softmax per head: warp w owns heads w, w + 4; a lane owns keys lane and lane + 32
    for (int g = warp; g < gc; g += DEC_THREADS / 32) {
      const float x0 = s_p[g * DEC_TK + lane], x1 = s_p[g * DEC_TK + lane + 32];
      float mx = fmaxf(x0, x1);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_old = s_m[g];
      const float m_new = fmaxf(m_old, mx);           // finite: a tile holds at least one valid key
      const float p0 = dec_ex2(x0 - m_new), p1 = dec_ex2(x1 - m_new);
      float sum = p0 + p1;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      const float corr = dec_ex2(m_old - m_new);      // 0 on the first tile (m_old = -inf)
      s_p[g * DEC_TK + lane] = p0;
      s_p[g * DEC_TK + lane + 32] = p1;
      if (lane == 0) {
        s_corr[g] = corr;
        s_m[g] = m_new;
        s_l[g] = s_l[g] * corr + sum;
      }
    }
    __syncthreads();
    // output: thread = one dimension, all heads of the chunk
    if (tid < D) {
#pragma unroll
      for (int g = 0; g < DEC_GC; ++g)
        if (g < gc) acc[g] *= s_corr[g];
      for (int key = 0; key < nk; ++key) {
        const float v = dec_ld(s_v + key * RS + tid);
#pragma unroll
        for (int g = 0; g < DEC_GC; ++g)
          if (g < gc) acc[g] = fmaf(s_p[g * DEC_TK + key], v, acc[g]);
      }
    }
  }
  __syncthreads();
  if (tid < D) {
    for (int g = 0; g < gc; ++g) {
      const size_t bh = static_cast<size_t>(b) * prm.H + h0 + g;
      if (prm.n_splits == 1) {
        dec_st(o + bh * D + tid, acc[g] / s_l[g]);
      } else {
        part_o[(bh * prm.n_splits + sp) * D + tid] = acc[g];
      }
    }
  }
  if (tid < gc) {
    const size_t bh = static_cast<size_t>(b) * prm.H + h0 + tid;
    if (prm.n_splits == 1) {
      if (lse != nullptr) lse[bh] = (s_m[tid] + log2f(s_l[tid])) * 0.6931471805599453f;
    } else {
      part_ml[(bh * prm.n_splits + sp) * 2] = s_m[tid];
      part_ml[(bh * prm.n_splits + sp) * 2 + 1] = s_l[tid];
    }
  }
}

// One CTA per (batch, head): merges the splits' partial results.  A split past kv_len has (m, l) = (-inf, 0).
template <typename ST>
__global__ void fa_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       ST* __restrict__ o, float* __restrict__ lse, int n_splits, int D) {
  ptx::grid_dep_wait();     // the partial results come from the kernel in front
  ptx::grid_dep_launch();
  const size_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_ml[(bh * n_splits + s) * 2]);
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(bh * n_splits + s) * 2];
    if (ms == -INFINITY) continue;
    const float w = dec_ex2(ms - m);
    l = fmaf(part_ml[(bh * n_splits + s) * 2 + 1], w, l);
    if (d < D) acc = fmaf(part_o[(bh * n_splits + s) * D + d], w, acc);
  }
  if (d < D) dec_st(o + bh * D + d, acc / l);
  if (d == 0 && lse != nullptr) lse[bh] = (m + log2f(l)) * 0.6931471805599453f;
}

}  // namespace it
