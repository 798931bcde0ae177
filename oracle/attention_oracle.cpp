// CPU oracle for causal scaled-dot-product attention (forward with LSE, composed backward).
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the smoke test and the
// benchmark's cpu_baseline leg compare the CUDA path against.  Nothing in the product
// (irontensor_b200/) links, loads or calls it.
//
// It is a restatement, in plain scalar C++, of the arithmetic the reference performs on this path
// (paths are relative to the reference project's root):
//   * forward, seq_len <= 256 : src/shaders/flash_attention.metal:167-223 (exact two-pass softmax)
//   * forward, seq_len  > 256 : src/shaders/flash_attention.metal:27-41,45-163 (online softmax over
//                               32-key blocks); the host picks between them at
//                               src/ops/flash_attention.rs:130
//   * backward                : src/train/helpers.rs:142-182 (13-step composition) with the scalar
//                               kernels it dispatches: gemm.metal:95-119, elementwise.metal:31-41,
//                               attention.metal:163-207, softmax.metal:14-111,
//                               backward/softmax.metal:22-90
//   * bf16 rounding           : src/precision.rs:24-29
//   * rotary embedding        : src/shaders/rope.metal:22-61, src/shaders/backward/rope.metal:25-62
//   * repeat_kv and backward  : src/shaders/repeat_kv.metal:19-88
// The same operation order is kept per output element (fp32, sums in index order, no FMA
// contraction: build with -ffp-contract=off), so that on inputs both can run, this file and the
// reference's own shader source compiled as C++ (oracle/ref_shim) agree exactly (IEEE ==).
// The rotary embedding and repeat_kv are pinned the same way (same libm powf / cosf / sinf as the
// compiled shader source; Apple's own pow, cos and sin cannot run here).
// Parity status: the forward and the scalar-kernel backward composition are pinned that way; the
// production backward's five GEMMs run in Apple's closed MPS library, whose summation order is
// unknown, so bit-level parity with THAT is unpinned (the reference itself only asserts 1e-3 there).
//
// Additions the reference does not have, derived from its state variables:
//   * LSE = row_max + logf(row_sum) (natural log of the scaled scores), from the softmax state of
//     flash_attention.metal:84-85,154-155 / :192,206-213.
//   * private arrays sized by head_dim (the tiled shader sizes them 64 and overruns for D > 64,
//     flash_attention.metal:78,88).
//   * a non-causal backward (the reference's backward masks unconditionally, helpers.rs:152).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float fmax2(float a, float b) { return a < b ? b : a; }

// flash_attention.metal:167-223 -- one query row, exact softmax.
void fwd_row_small(const float* Q, const float* K, const float* V, float* O, float* lse,
                   int S, int D, int q_pos, float scale, bool causal,
                   float* q_vec, float* scores) {
  for (int d = 0; d < D; ++d) q_vec[d] = Q[(size_t)q_pos * D + d];
  const int k_end = causal ? q_pos + 1 : S;
  float max_score = -INFINITY;
  for (int kp = 0; kp < k_end; ++kp) {
    float score = 0.0f;
    const float* krow = K + (size_t)kp * D;
    for (int d = 0; d < D; ++d) score += q_vec[d] * krow[d];
    score *= scale;
    scores[kp] = score;
    max_score = fmax2(max_score, score);
  }
  float sum_exp = 0.0f;
  for (int kp = 0; kp < k_end; ++kp) {
    float e = expf(scores[kp] - max_score);
    scores[kp] = e;
    sum_exp += e;
  }
  const float inv_sum = 1.0f / sum_exp;
  for (int d = 0; d < D; ++d) {
    float acc = 0.0f;
    for (int kp = 0; kp < k_end; ++kp) acc += scores[kp] * V[(size_t)kp * D + d];
    O[(size_t)q_pos * D + d] = acc * inv_sum;
  }
  if (lse) lse[q_pos] = max_score + logf(sum_exp);
}

// flash_attention.metal:45-163 with online_softmax_update (:27-41) -- one query row, 32-key blocks.
void fwd_row_tiled(const float* Q, const float* K, const float* V, float* O, float* lse,
                   int S, int D, int q_pos, float scale, bool causal,
                   float* q_vec, float* o_vec) {
  constexpr int BLOCK_N = 32;
  for (int d = 0; d < D; ++d) q_vec[d] = Q[(size_t)q_pos * D + d];
  for (int d = 0; d < D; ++d) o_vec[d] = 0.0f;
  float row_max = -INFINITY, row_sum = 0.0f;
  const int k_end = causal ? q_pos + 1 : S;
  float sc[BLOCK_N];
  for (int k0 = 0; k0 < k_end; k0 += BLOCK_N) {
    const int nk = std::min(k0 + BLOCK_N, k_end) - k0;
    float blk_max = -INFINITY;
    for (int i = 0; i < nk; ++i) {
      const int kp = k0 + i;
      const float* krow = K + (size_t)kp * D;
      float score = 0.0f;
      for (int d = 0; d < D; ++d) score += q_vec[d] * krow[d];
      score *= scale;
      if (causal && kp > q_pos) score = -INFINITY;
      sc[i] = score;
      blk_max = fmax2(blk_max, score);
    }
    float blk_sum = 0.0f;
    for (int i = 0; i < nk; ++i) {
      float e = expf(sc[i] - blk_max);
      sc[i] = e;
      blk_sum += e;
    }
    const float new_max = fmax2(row_max, blk_max);
    const float old_corr = expf(row_max - new_max);
    const float new_corr = expf(blk_max - new_max);
    const float new_sum = row_sum * old_corr + blk_sum * new_corr;
    for (int d = 0; d < D; ++d) o_vec[d] *= old_corr;
    const float blk_corr = expf(blk_max - new_max);
    for (int i = 0; i < nk; ++i) {
      const float w = sc[i] * blk_corr;
      const float* vrow = V + (size_t)(k0 + i) * D;
      for (int d = 0; d < D; ++d) o_vec[d] += w * vrow[d];
    }
    row_max = new_max;
    row_sum = new_sum;
  }
  const float inv_sum = 1.0f / row_sum;
  for (int d = 0; d < D; ++d) O[(size_t)q_pos * D + d] = o_vec[d] * inv_sum;
  if (lse) lse[q_pos] = row_max + logf(row_sum);
}

// gemm.metal:95-119 : C[m,n] = sum_k A[m,k]*B[k,n], k ascending, one fp32 accumulator per element.
// Loop nest is reordered for cache use; every element still sees the same sequence of adds.
void gemm_rowmajor(const float* A, const float* B, float* C, int M, int K, int N) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* c = C + (size_t)m * N;
    for (int n = 0; n < N; ++n) c[n] = 0.0f;
    const float* a = A + (size_t)m * K;
    for (int k = 0; k < K; ++k) {
      const float av = a[k];
      const float* b = B + (size_t)k * N;
      for (int n = 0; n < N; ++n) c[n] += av * b[n];
    }
  }
}

// attention.metal:163-184
void transpose2d(const float* in, float* out, int m, int n) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) out[(size_t)j * m + i] = in[(size_t)i * n + j];
}

// softmax.metal:14-44 (dim < 256) and :49-111 (dim >= 256: 256 lanes stride the row, then a
// halving tree over the lane partials); kernel choice at src/ops/softmax.rs:196.
void softmax_row(const float* in, float* out, int dim) {
  constexpr int T = 256;
  if (dim < T) {
    float mx = in[0];
    for (int i = 1; i < dim; ++i) mx = fmax2(mx, in[i]);
    float sum = 0.0f;
    for (int i = 0; i < dim; ++i) { float e = expf(in[i] - mx); out[i] = e; sum += e; }
    const float inv = 1.0f / sum;
    for (int i = 0; i < dim; ++i) out[i] *= inv;
    return;
  }
  float lane[T];
  for (int t = 0; t < T; ++t) {
    float m = -INFINITY;
    for (int i = t; i < dim; i += T) m = fmax2(m, in[i]);
    lane[t] = m;
  }
  for (int s = T / 2; s > 0; s >>= 1)
    for (int t = 0; t < s; ++t) lane[t] = fmax2(lane[t], lane[t + s]);
  const float gmax = lane[0];
  for (int t = 0; t < T; ++t) {
    float acc = 0.0f;
    for (int i = t; i < dim; i += T) { float e = expf(in[i] - gmax); out[i] = e; acc += e; }
    lane[t] = acc;
  }
  for (int s = T / 2; s > 0; s >>= 1)
    for (int t = 0; t < s; ++t) lane[t] += lane[t + s];
  const float inv = 1.0f / lane[0];
  for (int i = 0; i < dim; ++i) out[i] *= inv;
}

// backward/softmax.metal:22-45 (dim < 256) and :50-90 (dim >= 256); choice at
// src/ops/backward/softmax.rs:45.
void softmax_backward_row(const float* gy, const float* y, float* gx, int dim) {
  constexpr int T = 256;
  float dot;
  if (dim < T) {
    dot = 0.0f;
    for (int i = 0; i < dim; ++i) dot += gy[i] * y[i];
  } else {
    float lane[T];
    for (int t = 0; t < T; ++t) {
      float acc = 0.0f;
      for (int i = t; i < dim; i += T) acc += gy[i] * y[i];
      lane[t] = acc;
    }
    for (int s = T / 2; s > 0; s >>= 1)
      for (int t = 0; t < s; ++t) lane[t] += lane[t + s];
    dot = lane[0];
  }
  for (int i = 0; i < dim; ++i) gx[i] = y[i] * (gy[i] - dot);
}

// src/train/helpers.rs:142-182 for one (batch, head) slice.
void bwd_one_head(const float* Q, const float* K, const float* V, const float* dO,
                  float* dQ, float* dK, float* dV, int S, int D, float scale, bool causal,
                  std::vector<float>& w0, std::vector<float>& w1, std::vector<float>& w2,
                  std::vector<float>& t0) {
  const size_t SS = (size_t)S * S, SD = (size_t)S * D;
  w0.resize(SS); w1.resize(SS); w2.resize(SS); t0.resize(std::max(SS, SD));
  float* scores = w0.data();   // later reused for dS
  float* P = w1.data();
  float* tmp = w2.data();      // P^T, dP, dS^T in turn
  float* tr = t0.data();       // K^T / V^T
  // :145-148 scores = Q @ K^T
  transpose2d(K, tr, S, D);
  gemm_rowmajor(Q, tr, scores, S, D, S);
  // :151-152 scale (elementwise.metal:31), then mask (attention.metal:186: col > row -> -inf)
#pragma omp parallel for schedule(static)
  for (int r = 0; r < S; ++r) {
    float* row = scores + (size_t)r * S;
    for (int c = 0; c < S; ++c) {
      float x = row[c] * scale;
      if (causal && c > r) x = -INFINITY;
      row[c] = x;
    }
  }
  // :155 P = softmax(rows)
#pragma omp parallel for schedule(static)
  for (int r = 0; r < S; ++r) softmax_row(scores + (size_t)r * S, P + (size_t)r * S, S);
  // :161-162 dV = P^T @ dO
  transpose2d(P, tmp, S, S);
  gemm_rowmajor(tmp, dO, dV, S, S, D);
  // :167-168 dP = dO @ V^T
  transpose2d(V, tr, S, D);
  gemm_rowmajor(dO, tr, tmp, S, D, S);
  // :171 dS = softmax_backward(dP, P)   (into `scores`)
  float* dS = scores;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < S; ++r)
    softmax_backward_row(tmp + (size_t)r * S, P + (size_t)r * S, dS + (size_t)r * S, S);
  // :176-177 dQ = (dS @ K) * scale
  gemm_rowmajor(dS, K, dQ, S, S, D);
  for (size_t i = 0; i < SD; ++i) dQ[i] = dQ[i] * scale;
  // :180-182 dK = (dS^T @ Q) * scale
  transpose2d(dS, tmp, S, S);
  gemm_rowmajor(tmp, Q, dK, S, S, D);
  for (size_t i = 0; i < SD; ++i) dK[i] = dK[i] * scale;
}

}  // namespace

extern "C" {

// src/precision.rs:24-29 : round-to-nearest-even on the upper 16 bits, no NaN special case.
void oracle_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t bits;
    std::memcpy(&bits, src + i, 4);
    const uint32_t round = ((bits >> 16) & 1u) + 0x7FFFu;
    dst[i] = (uint16_t)((bits + round) >> 16);
  }
}

void oracle_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t bits = (uint32_t)src[i] << 16;
    std::memcpy(dst + i, &bits, 4);
  }
}

// Forward over [B,H,S,D] fp32 row-major (src/ops/flash_attention.rs:76-193).
// kernel: 0 = the host's own choice (S <= 256 exact, else tiled), 1 = force exact, 2 = force tiled.
// lse may be null.  bh_begin/bh_end select a range of (batch*head) slices (for bounded samples).
// Returns 0, or -1 for arguments the reference asserts on.
int oracle_attention_fwd(int B, int H, int S, int D, int causal, int kernel,
                         const float* q, const float* k, const float* v, float* o, float* lse,
                         int bh_begin, int bh_end) {
  if (B < 0 || H < 0 || S < 0 || D < 1 || D > 128) return -1;   // flash_attention.rs:98
  if (S == 0) return 0;                                          // flash_attention.rs:102-104
  const float scale = 1.0f / sqrtf((float)D);                    // flash_attention.rs:109
  const bool small = kernel == 1 || (kernel == 0 && S <= 256);   // flash_attention.rs:130
  if (bh_end < 0) bh_end = B * H;
  const int64_t rows = (int64_t)(bh_end - bh_begin) * S;
#pragma omp parallel
  {
    std::vector<float> qv(D), aux(small ? S : D);
#pragma omp for schedule(dynamic, 16)
    for (int64_t r = 0; r < rows; ++r) {
      const int bh = bh_begin + (int)(r / S), qp = (int)(r % S);
      const size_t base = (size_t)bh * S * D;
      float* l = lse ? lse + (size_t)bh * S : nullptr;
      if (small)
        fwd_row_small(q + base, k + base, v + base, o + base, l, S, D, qp, scale, causal != 0,
                      qv.data(), aux.data());
      else
        fwd_row_tiled(q + base, k + base, v + base, o + base, l, S, D, qp, scale, causal != 0,
                      qv.data(), aux.data());
    }
  }
  return 0;
}

// Backward over [B,H,S,D] fp32 (src/train/helpers.rs:120-193).  Inputs are dO,Q,K,V only, as in
// the reference; P is recomputed.  Needs ~4*S*S floats of scratch (one head at a time).
int oracle_attention_bwd(int B, int H, int S, int D, int causal,
                         const float* q, const float* k, const float* v, const float* d_o,
                         float* dq, float* dk, float* dv, int bh_begin, int bh_end) {
  if (B < 0 || H < 0 || S < 0 || D < 1 || D > 128) return -1;
  if (S == 0) return 0;
  const float scale = 1.0f / sqrtf((float)D);                    // helpers.rs:135
  if (bh_end < 0) bh_end = B * H;
  std::vector<float> w0, w1, w2, t0;
  for (int bh = bh_begin; bh < bh_end; ++bh) {
    const size_t base = (size_t)bh * S * D;
    bwd_one_head(q + base, k + base, v + base, d_o + base, dq + base, dk + base, dv + base,
                 S, D, scale, causal != 0, w0, w1, w2, t0);
  }
  return 0;
}

// Rotary position embedding of one [B,S,H,D] fp32 tensor (src/shaders/rope.metal:22-61), or, with
// backward != 0, the transposed rotation of src/shaders/backward/rope.metal:25-62.  Every value is
// computed as the shader computes it: theta = 1.0f / powf(base, float(2i) / float(D)) in fp32,
// angle = float(position) * theta, one cosf and one sinf per element pair.
int oracle_rope(int B, int S, int H, int D, float base, int position_offset, int backward,
                const float* in, float* out) {
  if (B < 0 || S < 0 || H < 0 || D < 0 || (D & 1)) return -1;   // src/ops/rope.rs:38-42
  const int64_t rows = (int64_t)B * S * H;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const int seq_pos = (int)((r / H) % S);
    const uint32_t position = (uint32_t)seq_pos + (uint32_t)position_offset;
    const float* x = in + r * D;
    float* y = out + r * D;
    for (int pair = 0; pair < D / 2; ++pair) {
      const float dim_idx = (float)(pair * 2);
      const float theta = 1.0f / powf(base, dim_idx / (float)D);
      const float angle = (float)position * theta;
      const float c = cosf(angle), sn = sinf(angle);
      const float x0 = x[2 * pair], x1 = x[2 * pair + 1];
      if (backward) {
        y[2 * pair] = x0 * c + x1 * sn;
        y[2 * pair + 1] = -x0 * sn + x1 * c;
      } else {
        y[2 * pair] = x0 * c - x1 * sn;
        y[2 * pair + 1] = x0 * sn + x1 * c;
      }
    }
  }
  return 0;
}

// repeat_kv (src/shaders/repeat_kv.metal:19-47): in [B,S,Hkv,D] -> out [B,S,H,D], output head h
// reads head h / (H / Hkv).  backward != 0 (:49-88): in [B,S,H,D] -> out [B,S,Hkv,D], the group's
// gradients summed in head order starting from 0.0f.
int oracle_repeat_kv(int B, int S, int H, int Hkv, int D, int backward, const float* in, float* out) {
  if (Hkv < 1 || H % Hkv != 0) return -1;                        // src/ops/repeat_kv.rs:77-80
  const int rep = H / Hkv;
  const int64_t bs = (int64_t)B * S;
  for (int64_t t = 0; t < bs; ++t) {
    if (backward) {
      for (int kvh = 0; kvh < Hkv; ++kvh)
        for (int d = 0; d < D; ++d) {
          float sum = 0.0f;
          for (int r = 0; r < rep; ++r) sum += in[(t * H + kvh * rep + r) * D + d];
          out[(t * Hkv + kvh) * D + d] = sum;
        }
    } else {
      for (int h = 0; h < H; ++h)
        for (int d = 0; d < D; ++d) out[(t * H + h) * D + d] = in[(t * Hkv + h / rep) * D + d];
    }
  }
  return 0;
}

// Launchers such as torchrun export OMP_NUM_THREADS=1; the timed CPU legs ask for all cores again.
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
