// Runs the reference project's OWN shader sources on the CPU.  TEST INFRASTRUCTURE ONLY.
//
// The .metal files are included, unmodified and where they lie (REF_ROOT, passed by the
// Makefile); nothing of them is copied into this repository.  Each is wrapped in a namespace so
// that their same-named parameter structs do not collide.  One-thread-per-element kernels are
// driven by looping the thread ids; the two 256-lane threadgroup kernels (softmax_fast_f32,
// softmax_backward_fast_f32) are driven by 256 host threads meeting at a std::barrier.
//
// Exports (C ABI, same signatures as oracle/attention_oracle.cpp):
//   ref_attention_fwd : flash_attention_small_f32 / flash_attention_forward_f32, chosen as
//                       src/ops/flash_attention.rs:130 chooses; LSE is NOT produced (the
//                       reference has none).
//   ref_attention_bwd : the composition of src/train/helpers.rs:142-182 built from the scalar
//                       kernels gemm_f32_batched, scale_f32, causal_mask_3d_f32, softmax[_fast]_f32,
//                       softmax_backward[_fast]_f32, transpose_3d_f32.
//   ref_rope, ref_rope_backward : rope_f32 (src/shaders/rope.metal:22-61) and rope_backward_f32
//                       (src/shaders/backward/rope.metal:25-62) on [batch, seq, heads, head_dim],
//                       grids as src/ops/rope.rs dispatches them (one thread per rotation pair).
//   ref_repeat_kv, ref_repeat_kv_backward : repeat_kv_f32 / repeat_kv_backward_f32
//                       (src/shaders/repeat_kv.metal:19-88), one thread per output element.
#include <metal_stdlib>
#include <cstring>
#include <algorithm>

#define IT_STR2(x) #x
#define IT_STR(x) IT_STR2(x)
#define IT_REF(path) IT_STR(REF_ROOT/path)

namespace ref_fa {
#include IT_REF(src/shaders/flash_attention.metal)
}
namespace ref_sm {
#include IT_REF(src/shaders/softmax.metal)
}
#undef SOFTMAX_THREADS
namespace ref_smb {
#include IT_REF(src/shaders/backward/softmax.metal)
}
namespace ref_gemm {
#include IT_REF(src/shaders/gemm.metal)
}
namespace ref_attn {
#include IT_REF(src/shaders/attention.metal)
}
namespace ref_ew {
#include IT_REF(src/shaders/elementwise.metal)
}
namespace ref_rope_f {
#include IT_REF(src/shaders/rope.metal)
}
namespace ref_rope_b {
#include IT_REF(src/shaders/backward/rope.metal)
}
namespace ref_rkv {
#include IT_REF(src/shaders/repeat_kv.metal)
}
// The shader keywords are macros in the shim; drop them before any host code follows.
#undef kernel
#undef device
#undef constant
#undef thread
#undef threadgroup

namespace {

// Tiled kernel with private arrays of 64: only valid for D <= 64 (the shader's own limit).
void run_fwd(const float* q, const float* k, const float* v, float* o, int B, int H, int S, int D,
             int causal, int which) {
  ref_fa::FlashAttentionParams p;
  p.batch_size = B; p.num_heads = H; p.seq_len = S; p.head_dim = D;
  p.scale = 1.0f / sqrtf((float)D);
  p.causal = causal ? 1u : 0u;
  const bool small = which == 1 || (which == 0 && S <= 256);
  if (small) {
    for (uint z = 0; z < (uint)(B * H); ++z)
      for (uint x = 0; x < (uint)S; ++x) ref_fa::flash_attention_small_f32(q, k, v, o, p, uint3{x, 0, z});
  } else {
    const uint nblk = (S + 31) / 32;
    for (uint z = 0; z < (uint)(B * H); ++z)
      for (uint bx = 0; bx < nblk; ++bx)
        for (uint t = 0; t < 32; ++t)
          ref_fa::flash_attention_forward_f32(q, k, v, o, p, uint3{t, 0, 0}, uint3{bx, 0, z},
                                              uint3{32, 1, 1});
  }
}

void gemm(const float* A, const float* Bm, float* C, uint M, uint K, uint N) {
  ref_gemm::GemmParams gp;
  std::memset(&gp, 0, sizeof gp);
  gp.M = M; gp.N = N; gp.K = K;
  const uint one = 1;
  for (uint r = 0; r < M; ++r)
    for (uint c = 0; c < N; ++c) ref_gemm::gemm_f32_batched(A, Bm, C, gp, one, uint3{c, r, 0});
}

void transpose(const float* in, float* out, uint m, uint n) {
  ref_attn::Transpose3DParams tp{1, m, n};
  for (uint j = 0; j < n; ++j)
    for (uint i = 0; i < m; ++i) ref_attn::transpose_3d_f32(in, out, tp, uint3{i, j, 0});
}

// 256 host threads emulate one threadgroup at a time over all rows.
template <class F>
void run_threadgroups(uint rows, F body) {
  constexpr uint T = 256;
  std::barrier<> bar(T);
  metal::shim_barrier() = &bar;
  std::vector<std::thread> th;
  for (uint t = 0; t < T; ++t)
    th.emplace_back([&, t] {
      for (uint r = 0; r < rows; ++r) {
        body(r, t);
        bar.arrive_and_wait();   // the next row reuses the static threadgroup arrays
      }
    });
  for (auto& x : th) x.join();
  metal::shim_barrier() = nullptr;
}

void softmax_rows(const float* in, float* out, uint rows, uint dim) {
  ref_sm::SoftmaxParams sp{rows, dim};
  if (dim >= 256)   // src/ops/softmax.rs:196
    run_threadgroups(rows, [&](uint r, uint t) { ref_sm::softmax_fast_f32(in, out, sp, r, t); });
  else
    for (uint r = 0; r < rows; ++r) ref_sm::softmax_f32(in, out, sp, r);
}

void softmax_bwd_rows(const float* gy, const float* y, float* gx, uint rows, uint dim) {
  ref_smb::SoftmaxParams sp{rows, dim};
  if (dim >= 256)   // src/ops/backward/softmax.rs:45
    run_threadgroups(rows, [&](uint r, uint t) { ref_smb::softmax_backward_fast_f32(gy, y, gx, sp, r, t); });
  else
    for (uint r = 0; r < rows; ++r) ref_smb::softmax_backward_f32(gy, y, gx, sp, r);
}

}  // namespace

extern "C" {

int ref_attention_fwd(int B, int H, int S, int D, int causal, int kernel,
                      const float* q, const float* k, const float* v, float* o) {
  const bool small = kernel == 1 || (kernel == 0 && S <= 256);
  if (D > 128 || (!small && D > 64) || (small && S > 512)) return -1;   // the shaders' array sizes
  if (S == 0) return 0;
  run_fwd(q, k, v, o, B, H, S, D, causal, kernel);
  return 0;
}

int ref_attention_bwd(int B, int H, int S, int D,
                      const float* q, const float* k, const float* v, const float* d_o,
                      float* dq, float* dk, float* dv) {
  const uint s = S, d = D;
  const float scale = 1.0f / sqrtf((float)D);
  const size_t SS = (size_t)S * S, SD = (size_t)S * D;
  std::vector<float> kt(SD), scores(SS), scaled(SS), masked(SS), P(SS), Pt(SS), vt(SD), dP(SS),
      dS(SS), dSt(SS), tmp(SD);
  for (int bh = 0; bh < B * H; ++bh) {
    const float *Q = q + bh * SD, *K = k + bh * SD, *V = v + bh * SD, *dO = d_o + bh * SD;
    const uint one = 1, nss = (uint)SS, nsd = (uint)SD;
    transpose(K, kt.data(), s, d);
    gemm(Q, kt.data(), scores.data(), s, d, s);
    for (uint i = 0; i < nss; ++i) ref_ew::scale_f32(scores.data(), scaled.data(), scale, nss, i);
    for (uint r = 0; r < s; ++r)
      for (uint c = 0; c < s; ++c)
        ref_attn::causal_mask_3d_f32(scaled.data(), masked.data(), one, s, uint3{c, r, 0});
    softmax_rows(masked.data(), P.data(), s, s);
    transpose(P.data(), Pt.data(), s, s);
    gemm(Pt.data(), dO, dv + bh * SD, s, s, d);
    transpose(V, vt.data(), s, d);
    gemm(dO, vt.data(), dP.data(), s, d, s);
    softmax_bwd_rows(dP.data(), P.data(), dS.data(), s, s);
    gemm(dS.data(), K, tmp.data(), s, s, d);
    for (uint i = 0; i < nsd; ++i) ref_ew::scale_f32(tmp.data(), dq + bh * SD, scale, nsd, i);
    transpose(dS.data(), dSt.data(), s, s);
    gemm(dSt.data(), Q, tmp.data(), s, s, d);
    for (uint i = 0; i < nsd; ++i) ref_ew::scale_f32(tmp.data(), dk + bh * SD, scale, nsd, i);
  }
  return 0;
}

int ref_rope(int B, int S, int H, int D, float base, int position_offset, int backward, const float* in,
             float* out) {
  if (D & 1) return -1;
  const uint b = B, s = S, h = H, d = D;
  if (backward) {
    ref_rope_b::RoPEParams p{b, s, h, d, base, (uint)position_offset};
    for (uint z = 0; z < b * h; ++z)
      for (uint y = 0; y < s; ++y)
        for (uint x = 0; x < d / 2; ++x) ref_rope_b::rope_backward_f32(in, out, p, uint3{x, y, z});
  } else {
    ref_rope_f::RoPEParams p{b, s, h, d, base, (uint)position_offset};
    for (uint z = 0; z < b * h; ++z)
      for (uint y = 0; y < s; ++y)
        for (uint x = 0; x < d / 2; ++x) ref_rope_f::rope_f32(in, out, p, uint3{x, y, z});
  }
  return 0;
}

// forward: in [B,S,Hkv,D] -> out [B,S,H,D]; backward: in [B,S,H,D] -> out [B,S,Hkv,D]
int ref_repeat_kv(int B, int S, int H, int Hkv, int D, int backward, const float* in, float* out) {
  if (Hkv < 1 || H % Hkv != 0) return -1;
  ref_rkv::RepeatKVParams p{(uint)B, (uint)S, (uint)H, (uint)Hkv, (uint)D, (uint)(H / Hkv)};
  const uint heads_out = backward ? Hkv : H;
  for (uint z = 0; z < (uint)(B * S); ++z)
    for (uint y = 0; y < heads_out; ++y)
      for (uint x = 0; x < (uint)D; ++x) {
        if (backward) ref_rkv::repeat_kv_backward_f32(in, out, p, uint3{x, y, z});
        else ref_rkv::repeat_kv_f32(in, out, p, uint3{x, y, z});
      }
  return 0;
}

}  // extern "C"
