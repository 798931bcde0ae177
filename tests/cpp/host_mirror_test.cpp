// Exercises include/irontensor_b200.hpp the way the reference's own unit tests exercise its ops
// (src/ops/flash_attention.rs:242-349, src/ops/attention.rs:624-711, src/train/helpers.rs:437-494):
// closed-form inputs, GPU op, comparison with a CPU loop written in the test.
#include <cmath>
#include <cstdio>
#include <vector>

#include "irontensor_b200.hpp"

using it::Precision;
using it::Tensor;

static int failures = 0;
#define EXPECT(cond, ...)                         \
  do {                                            \
    if (!(cond)) {                                \
      std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
      std::printf(__VA_ARGS__);                   \
      std::printf("\n");                          \
      ++failures;                                 \
    }                                             \
  } while (0)

// Plain fp64 attention on [B,H,S,D] with its gradients (the math of src/train/helpers.rs:142-182).
struct CpuResult { std::vector<double> o, dq, dk, dv; };
static CpuResult cpu_attention(const std::vector<float>& q, const std::vector<float>& k, const std::vector<float>& v,
                               const std::vector<float>& d_o, size_t BH, size_t S, size_t D, bool causal) {
  CpuResult r;
  r.o.assign(q.size(), 0), r.dq.assign(q.size(), 0), r.dk.assign(q.size(), 0), r.dv.assign(q.size(), 0);
  const double scale = 1.0 / std::sqrt(static_cast<double>(D));
  std::vector<double> p(S), dp(S);
  for (size_t bh = 0; bh < BH; ++bh) {
    const size_t base = bh * S * D;
    for (size_t i = 0; i < S; ++i) {
      const size_t kend = causal ? i + 1 : S;
      double m = -INFINITY, l = 0;
      for (size_t j = 0; j < kend; ++j) {
        double s = 0;
        for (size_t d = 0; d < D; ++d) s += static_cast<double>(q[base + i * D + d]) * k[base + j * D + d];
        p[j] = s * scale;
        m = std::max(m, p[j]);
      }
      for (size_t j = 0; j < kend; ++j) { p[j] = std::exp(p[j] - m); l += p[j]; }
      double dot = 0;
      for (size_t j = 0; j < kend; ++j) {
        p[j] /= l;
        double g = 0;
        for (size_t d = 0; d < D; ++d) {
          r.o[base + i * D + d] += p[j] * v[base + j * D + d];
          g += static_cast<double>(d_o[base + i * D + d]) * v[base + j * D + d];
        }
        dp[j] = g;
        dot += g * p[j];
      }
      for (size_t j = 0; j < kend; ++j) {
        const double ds = p[j] * (dp[j] - dot);
        for (size_t d = 0; d < D; ++d) {
          r.dv[base + j * D + d] += p[j] * d_o[base + i * D + d];
          r.dq[base + i * D + d] += ds * k[base + j * D + d] * scale;
          r.dk[base + j * D + d] += ds * q[base + i * D + d] * scale;
        }
      }
    }
  }
  return r;
}

template <class U>
static double max_abs_diff(const std::vector<float>& a, const std::vector<U>& b) {
  double m = 0;
  for (size_t i = 0; i < a.size(); ++i) m = std::max(m, std::fabs(static_cast<double>(a[i]) - static_cast<double>(b[i])));
  return m;
}

int main() {
  try {
    // --- flash attention against the CPU loop and against attention() in the other layout
    {
      const size_t B = 2, H = 4, S = 32, D = 16, n = B * H * S * D;
      std::vector<float> x(n), dummy(n, 0.f);
      for (size_t i = 0; i < n; ++i) x[i] = std::sin(static_cast<float>(i) * 0.1f) * 0.5f;
      const Tensor t = Tensor::from_f32_slice(x, {B, H, S, D});
      for (int causal = 0; causal < 2; ++causal) {
        it::CommandBatch::begin();
        const Tensor o = it::flash_attention(t, t, t, causal != 0);
        it::CommandBatch::end();
        const CpuResult ref = cpu_attention(x, x, x, dummy, B * H, S, D, causal != 0);
        EXPECT(o.shape() == t.shape(), "output shape");
        EXPECT(max_abs_diff(o.to_host_f32(), ref.o) < 1e-4, "flash vs cpu, causal=%d: %g", causal, max_abs_diff(o.to_host_f32(), ref.o));
        // the same data in [B,S,H,D] through attention()
        std::vector<float> xs(n);
        for (size_t b = 0; b < B; ++b)
          for (size_t h = 0; h < H; ++h)
            for (size_t s = 0; s < S; ++s)
              for (size_t d = 0; d < D; ++d) xs[((b * S + s) * H + h) * D + d] = x[((b * H + h) * S + s) * D + d];
        const Tensor ts = Tensor::from_f32_slice(xs, {B, S, H, D});
        const std::vector<float> os = it::attention(ts, ts, ts, causal != 0).to_host_f32();
        const std::vector<float> of = o.to_host_f32();
        double m = 0;
        for (size_t b = 0; b < B; ++b)
          for (size_t h = 0; h < H; ++h)
            for (size_t s = 0; s < S; ++s)
              for (size_t d = 0; d < D; ++d)
                m = std::max(m, std::fabs(static_cast<double>(os[((b * S + s) * H + h) * D + d]) - of[((b * H + h) * S + s) * D + d]));
        EXPECT(m < 1e-6, "attention() vs flash_attention(), causal=%d: %g", causal, m);
      }
    }
    // --- longer sequence, head_dim 32
    {
      const size_t B = 1, H = 2, S = 128, D = 32, n = B * H * S * D;
      std::vector<float> x(n), dummy(n, 0.f);
      for (size_t i = 0; i < n; ++i) x[i] = std::sin(static_cast<float>(i) * 0.01f) * 0.3f;
      const Tensor t = Tensor::from_f32_slice(x, {B, H, S, D});
      const Tensor o = it::flash_attention(t, t, t, true);
      EXPECT(max_abs_diff(o.to_host_f32(), cpu_attention(x, x, x, dummy, B * H, S, D, true).o) < 1e-4, "longer sequence");
      EXPECT(o.lse && o.lse->shape() == std::vector<size_t>({B, H, S}), "lse shape");
    }
    // --- output shape only (B2 H8 S64 D64), and the empty sequence
    {
      const Tensor t = Tensor::zeros({2, 8, 64, 64});
      EXPECT(it::flash_attention(t, t, t, true).shape() == std::vector<size_t>({2, 8, 64, 64}), "shape");
      const Tensor e = Tensor::zeros({2, 2, 0, 8});
      EXPECT(it::flash_attention(e, e, e, true).numel() == 0, "empty sequence");
    }
    // --- backward, with and without the cached forward, fp32 and bf16
    {
      const size_t B = 2, H = 4, S = 16, D = 8, n = B * H * S * D;
      std::vector<float> go(n), q(n), k(n), v(n);
      for (size_t i = 0; i < n; ++i) {
        go[i] = static_cast<float>(i % 17) * 0.01f - 0.08f;
        q[i] = static_cast<float>(i % 13) * 0.01f - 0.06f;
        k[i] = static_cast<float>(i % 11) * 0.01f - 0.05f;
        v[i] = static_cast<float>(i % 7) * 0.01f - 0.03f;
      }
      const CpuResult ref = cpu_attention(q, k, v, go, B * H, S, D, true);
      const std::vector<size_t> shp = {B, H, S, D};
      const Tensor tq = Tensor::from_f32_slice(q, shp), tk = Tensor::from_f32_slice(k, shp),
                   tv = Tensor::from_f32_slice(v, shp), tgo = Tensor::from_f32_slice(go, shp);
      for (int cached = 0; cached < 2; ++cached) {
        Tensor dq, dk, dv;
        if (cached) {
          const Tensor o = it::flash_attention(tq, tk, tv, true);
          std::tie(dq, dk, dv) = it::attention_backward_recompute(tgo, tq, tk, tv, &o);
        } else {
          std::tie(dq, dk, dv) = it::attention_backward_recompute(tgo, tq, tk, tv);
        }
        it::CommandBatch::commit_async();
        it::CommandBatch::wait_for_completion();
        EXPECT(it::CommandBatch::is_async_complete(), "async completion");
        EXPECT(max_abs_diff(dq.to_host_f32(), ref.dq) < 1e-4, "dQ cached=%d", cached);
        EXPECT(max_abs_diff(dk.to_host_f32(), ref.dk) < 1e-4, "dK cached=%d", cached);
        EXPECT(max_abs_diff(dv.to_host_f32(), ref.dv) < 1e-4, "dV cached=%d", cached);
      }
    }
    {
      const size_t B = 1, H = 2, S = 256, D = 64, n = B * H * S * D;   // bf16: the tensor-core kernels
      std::vector<float> go(n), q(n), k(n), v(n);
      for (size_t i = 0; i < n; ++i) {
        q[i] = it::bf16_to_f32(it::f32_to_bf16(std::sin(static_cast<float>(i) * 0.37f)));
        k[i] = it::bf16_to_f32(it::f32_to_bf16(std::cos(static_cast<float>(i) * 0.11f)));
        v[i] = it::bf16_to_f32(it::f32_to_bf16(std::sin(static_cast<float>(i) * 0.05f + 1.f)));
        go[i] = it::bf16_to_f32(it::f32_to_bf16(std::cos(static_cast<float>(i) * 0.23f)));
      }
      const CpuResult ref = cpu_attention(q, k, v, go, B * H, S, D, true);
      const std::vector<size_t> shp = {B, H, S, D};
      const Tensor tq = Tensor::from_f32_as_bf16(q, shp), tk = Tensor::from_f32_as_bf16(k, shp),
                   tv = Tensor::from_f32_as_bf16(v, shp), tgo = Tensor::from_f32_as_bf16(go, shp);
      const Tensor o = it::flash_attention(tq, tk, tv, true);
      EXPECT(o.precision() == Precision::BF16, "bf16 output precision");
      auto [dq, dk, dv] = it::attention_backward_recompute(tgo, tq, tk, tv, &o);
      it::CommandBatch::poll_device_status();
      EXPECT(max_abs_diff(o.to_host_f32(), ref.o) < 2e-2, "bf16 O %g", max_abs_diff(o.to_host_f32(), ref.o));
      EXPECT(max_abs_diff(dq.to_host_f32(), ref.dq) < 2e-2, "bf16 dQ %g", max_abs_diff(dq.to_host_f32(), ref.dq));
      EXPECT(max_abs_diff(dk.to_host_f32(), ref.dk) < 2e-2, "bf16 dK %g", max_abs_diff(dk.to_host_f32(), ref.dk));
      EXPECT(max_abs_diff(dv.to_host_f32(), ref.dv) < 2e-2, "bf16 dV %g", max_abs_diff(dv.to_host_f32(), ref.dv));
      // the same tensors in [B,S,H,D] through attention() / attention_backward(): no transposes on the device
      auto to_bshd = [&](const auto& x) {
        auto y = x;
        for (size_t b = 0; b < B; ++b) for (size_t h = 0; h < H; ++h) for (size_t s = 0; s < S; ++s) for (size_t d = 0; d < D; ++d)
          y[((b * S + s) * H + h) * D + d] = x[((b * H + h) * S + s) * D + d];
        return y;
      };
      const std::vector<size_t> shp2 = {B, S, H, D};
      const Tensor sq = Tensor::from_f32_as_bf16(to_bshd(q), shp2), sk = Tensor::from_f32_as_bf16(to_bshd(k), shp2),
                   sv = Tensor::from_f32_as_bf16(to_bshd(v), shp2), sgo = Tensor::from_f32_as_bf16(to_bshd(go), shp2);
      const Tensor so = it::attention(sq, sk, sv, true);
      auto [sdq, sdk, sdv] = it::attention_backward(sgo, sq, sk, sv, so, true);
      it::CommandBatch::poll_device_status();
      EXPECT(max_abs_diff(so.to_host_f32(), to_bshd(o.to_host_f32())) == 0.0, "[B,S,H,D] O equals [B,H,S,D] O");
      EXPECT(max_abs_diff(sdk.to_host_f32(), to_bshd(dk.to_host_f32())) == 0.0, "[B,S,H,D] dK equals [B,H,S,D] dK");
      EXPECT(max_abs_diff(sdv.to_host_f32(), to_bshd(dv.to_host_f32())) == 0.0, "[B,S,H,D] dV equals [B,H,S,D] dV");
      EXPECT(max_abs_diff(sdq.to_host_f32(), to_bshd(ref.dq)) < 2e-2, "[B,S,H,D] dQ");
    }
    // --- grouped queries, rotary embedding, key/value cache: against the plain ops on expanded / full tensors
    {
      const size_t B = 1, S = 48, H = 4, Hkv = 2, D = 16;
      std::vector<float> q(B * S * H * D), k(B * S * Hkv * D), v(k.size()), go(q.size());
      for (size_t i = 0; i < q.size(); ++i) { q[i] = std::sin(0.37f * i); go[i] = std::cos(0.23f * i); }
      for (size_t i = 0; i < k.size(); ++i) { k[i] = std::cos(0.11f * i); v[i] = std::sin(0.05f * i + 1.f); }
      auto expand = [&](const std::vector<float>& x) {   // repeat_kv: [B,S,Hkv,D] -> [B,S,H,D]
        std::vector<float> y(B * S * H * D);
        for (size_t bs = 0; bs < B * S; ++bs) for (size_t h = 0; h < H; ++h) for (size_t d = 0; d < D; ++d)
          y[(bs * H + h) * D + d] = x[(bs * Hkv + h / (H / Hkv)) * D + d];
        return y;
      };
      const Tensor tq = Tensor::from_f32_slice(q, {B, S, H, D}), tk = Tensor::from_f32_slice(k, {B, S, Hkv, D}),
                   tv = Tensor::from_f32_slice(v, {B, S, Hkv, D}), tgo = Tensor::from_f32_slice(go, {B, S, H, D});
      const Tensor o = it::attention_gqa(tq, tk, tv, true);
      const Tensor ke = Tensor::from_f32_slice(expand(k), {B, S, H, D}), ve = Tensor::from_f32_slice(expand(v), {B, S, H, D});
      const Tensor oe = it::attention(tq, ke, ve, true);
      EXPECT(max_abs_diff(o.to_host_f32(), oe.to_host_f32()) < 1e-6, "attention_gqa equals attention on expanded K/V");
      auto [dq, dk, dv] = it::attention_gqa_backward(tgo, tq, tk, tv, o, true);
      auto [dqe, dke, dve] = it::attention_backward(tgo, tq, ke, ve, oe, true);
      EXPECT(max_abs_diff(dq.to_host_f32(), dqe.to_host_f32()) < 1e-5, "grouped dQ");
      std::vector<float> fold(B * S * Hkv * D, 0.f);   // repeat_kv_backward
      const std::vector<float> dkeh = dke.to_host_f32();
      for (size_t bs = 0; bs < B * S; ++bs) for (size_t h = 0; h < H; ++h) for (size_t d = 0; d < D; ++d)
        fold[(bs * Hkv + h / (H / Hkv)) * D + d] += dkeh[(bs * H + h) * D + d];
      EXPECT(max_abs_diff(dk.to_host_f32(), fold) < 1e-5, "grouped dK is the sum over the group");
      // rotary: position 0 is the identity, inverse(forward) is the identity
      auto [qr, kr] = it::rope_qk(tq, tk);
      const std::vector<float> qrh = qr.to_host_f32();
      double m0 = 0;
      for (size_t i = 0; i < H * D; ++i) m0 = std::max(m0, std::fabs(static_cast<double>(qrh[i]) - q[i]));
      EXPECT(m0 == 0.0, "rope at position 0 is the identity");
      auto [qb, kb] = it::rope_qk(qr, kr, 10000.f, 0, true);
      EXPECT(max_abs_diff(qb.to_host_f32(), q) < 1e-5 && max_abs_diff(kb.to_host_f32(), k) < 1e-5, "rope inverse");
      // key/value cache: the new token's output equals the last row of the full causal attention
      std::vector<float> q_last(H * D);
      for (size_t i = 0; i < H * D; ++i) q_last[i] = q[((S - 1) * H) * D + i];
      const Tensor dec = it::attention_decode(Tensor::from_f32_slice(q_last, {B, H, D}), tk, tv, S);
      const std::vector<float> oh = o.to_host_f32();
      std::vector<float> want(oh.begin() + (S - 1) * H * D, oh.begin() + S * H * D);
      EXPECT(max_abs_diff(dec.to_host_f32(), want) < 1e-5, "decode equals the last row");
    }
    // --- projections: y = x W^T against a plain loop, and the fused Q/K/V front end against it
    {
      const size_t n = 96, in = 64, H = 2, Hkv = 1, D = 32, out = (H + 2 * Hkv) * D, B = 2, S = 48;
      std::vector<float> x(n * in), w(out * in);
      for (size_t i = 0; i < x.size(); ++i) x[i] = it::bf16_to_f32(it::f32_to_bf16(std::sin(0.13f * i)));
      for (size_t i = 0; i < w.size(); ++i) w[i] = it::bf16_to_f32(it::f32_to_bf16(0.1f * std::cos(0.07f * i)));
      std::vector<double> ref(n * out, 0.0);
      for (size_t r = 0; r < n; ++r) for (size_t c = 0; c < out; ++c) for (size_t kk = 0; kk < in; ++kk)
        ref[r * out + c] += static_cast<double>(x[r * in + kk]) * w[c * in + kk];
      const Tensor tx = Tensor::from_f32_as_bf16(x, {n, in}), tw = Tensor::from_f32_as_bf16(w, {out, in});
      const Tensor y = it::linear_forward(tx, tw);
      EXPECT(max_abs_diff(y.to_host_f32(), ref) < 2e-2, "linear_forward");
      auto [q, k, v] = it::qkv_rope_forward(tx.view({B, S, in}), tw, H, Hkv, D, 0.f);   // no rotation: pure layout
      const std::vector<float> qh = q.to_host_f32(), vh = v.to_host_f32(), yh = y.to_host_f32();
      double mq = 0, mv = 0;
      for (size_t r = 0; r < n; ++r) {
        for (size_t c = 0; c < H * D; ++c) mq = std::max(mq, std::fabs(static_cast<double>(qh[r * H * D + c]) - yh[r * out + c]));
        for (size_t c = 0; c < Hkv * D; ++c)
          mv = std::max(mv, std::fabs(static_cast<double>(vh[r * Hkv * D + c]) - yh[r * out + (H + Hkv) * D + c]));
      }
      EXPECT(mq == 0.0 && mv == 0.0, "fused projection without rotation equals the plain projection, column ranges split");
      auto [dx, dw] = it::linear_backward(y, tx, tw);
      EXPECT(dx.shape() == std::vector<size_t>({n, in}) && dw.shape() == std::vector<size_t>({out, in}) &&
                 dw.precision() == Precision::FP32, "linear_backward shapes");
    }
    // --- the reference's asserts
    {
      const Tensor a = Tensor::zeros({2, 4, 32, 16}), b = Tensor::zeros({2, 4, 33, 16});
      bool threw = false;
      try { it::flash_attention(a, b, a, true); } catch (const std::logic_error& e) { threw = std::string(e.what()).find("same shape") != std::string::npos; }
      EXPECT(threw, "shape mismatch must throw");
      threw = false;
      try { it::flash_attention(a.view({8, 32, 16}), a.view({8, 32, 16}), a.view({8, 32, 16}), true); } catch (const std::logic_error&) { threw = true; }
      EXPECT(threw, "3-D input must throw");
    }
  } catch (const std::exception& e) {
    std::printf("FAIL: exception %s\n", e.what());
    return 2;
  }
  std::printf(failures == 0 ? "host mirror: all checks passed\n" : "host mirror: %d check(s) failed\n", failures);
  return failures == 0 ? 0 : 1;
}
