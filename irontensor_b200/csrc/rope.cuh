// Rotary position embedding on [batch, seq, heads, head_dim] tensors, and its inverse.
//
// Follows the reference's rope_f32 / rope_backward_f32 (src/shaders/rope.metal:22-61,
// src/shaders/backward/rope.metal:25-62): for position p and dimension pair i,
//   theta_i = 1 / base^(2i / head_dim),  angle = float(p) * theta_i,
//   forward  (x0, x1) -> (x0 cos - x1 sin,  x0 sin + x1 cos)
//   backward (g0, g1) -> (g0 cos + g1 sin, -g0 sin + g1 cos)      (the transpose of the rotation).
// The reference runs the forward once for Q and once for K, and the backward once for dQ and once
// for dK.  Here Q and K are rotated by ONE launch (rope_qk_kernel), and the backward rotation is not
// a pass at all: the attention backward applies it where dQ and dK leave the chip (the fp32 -> bf16
// finish pass of dQ, the dK epilogue), see fa_bwd_sm100.cuh and fa_generic.cuh.
// Rotating K "on load" inside the attention kernels was rejected: every K tile is loaded once per
// query tile (S/128 times), every Q tile once per key tile in the backward, so the rotation would be
// redone that many times on shared-memory tiles of kernels that are shared-memory bound.
// theta_i comes from the host as a table computed in fp32 exactly as the shader does (powf, then one
// division), so that a CPU check multiplies the position by bit-identical frequencies.
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace it {

struct RopeFreqs {
  float inv_freq[64];   // theta_i for i < head_dim / 2 (head_dim <= 128)
  int enabled;          // 0: no rotation
  int position_offset;  // position of sequence index 0 (KV-cache continuation, rope.metal:16)
};

__device__ __forceinline__ void rope_sincos(const RopeFreqs& f, int position, int pair, float* c, float* s) {
  const float angle = static_cast<float>(position) * f.inv_freq[pair];
  *c = cosf(angle);
  *s = sinf(angle);
}

__device__ __forceinline__ float rope_ld(const float* p) { return *p; }
__device__ __forceinline__ float rope_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void rope_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void rope_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One CTA per (batch, position); thread t owns dimension pair t % (D/2) and walks the heads of Q
// and then of K (which may have fewer heads) with stride blockDim / (D/2), so each thread computes
// its sine and cosine once.  INVERSE applies the backward rotation.  In place is fine.
template <typename ST, bool INVERSE>
__global__ void __launch_bounds__(256)
rope_qk_kernel(const ST* __restrict__ q_in, const ST* __restrict__ k_in, ST* __restrict__ q_out, ST* __restrict__ k_out,
               int S, int H, int Hkv, int D, const __grid_constant__ RopeFreqs freqs) {
  const int half = D >> 1;
  const int pair = threadIdx.x % half;
  const int lane_head = threadIdx.x / half;
  const int heads_per_pass = blockDim.x / half;
  const long long bs = blockIdx.x;                 // batch * S + position
  const int pos = static_cast<int>(bs % S) + freqs.position_offset;
  float c, s;
  rope_sincos(freqs, pos, pair, &c, &s);
  if (INVERSE) s = -s;
  const int n_heads = H + (k_in != nullptr ? Hkv : 0);
  for (int hh = lane_head; hh < n_heads; hh += heads_per_pass) {
    const bool is_q = hh < H;
    const ST* src = is_q ? q_in + (bs * H + hh) * D : k_in + (bs * Hkv + (hh - H)) * D;
    ST* dst = is_q ? q_out + (bs * H + hh) * D : k_out + (bs * Hkv + (hh - H)) * D;
    const float x0 = rope_ld(src + 2 * pair), x1 = rope_ld(src + 2 * pair + 1);
    rope_st(dst + 2 * pair, x0 * c - x1 * s);
    rope_st(dst + 2 * pair + 1, x0 * s + x1 * c);
  }
}

// (cos, sin) of every (sequence index, dimension pair): [S][D/2] float2.  Built once per call by kernels
// that would otherwise evaluate the same sine and cosine in every column tile (the fused QKV projection).
__global__ void rope_table_kernel(float2* __restrict__ table, int S, int half, const __grid_constant__ RopeFreqs freqs) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S * half) return;
  float c, s;
  rope_sincos(freqs, i / half + freqs.position_offset, i % half, &c, &s);
  table[i] = make_float2(c, s);
}

}  // namespace it
