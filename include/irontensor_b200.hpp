// C++ host-side mirror of the reference's attention interface over the C ABI (irontensor_b200.h).
//
// The reference is a Rust crate; with no Rust toolchain to build against, this header is the
// compiled-language host layer: same names, argument meaning and error behaviour as
//   Precision, Tensor            src/precision.rs:1-29, src/tensor.rs:11-300
//   CommandBatch                 src/command_batch.rs:167-391
//   flash_attention              src/ops/flash_attention.rs:76-193     [B,H,S,D]
//   attention                    src/ops/attention.rs:286-377          [B,S,H,D]
//   attention_backward_recompute src/train/helpers.rs:120-193          [B,H,S,D]
//   attention_gqa / rope_qk / attention_decode: the callers' steps around attention folded in (see each)
// Where the reference panics (assert!), these throw std::logic_error with the same message; failures of
// the library itself throw it::Error carrying the status code.  Header-only; link libirontensor_b200.so.
// No CPU fallback: every operation needs the CUDA library and a device.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "irontensor_b200.h"

namespace it {

struct Error : std::runtime_error {
  it_status status;
  Error(it_status s, const std::string& what) : std::runtime_error(what), status(s) {}
};
inline void check(it_status s) {
  if (s != IT_OK) throw Error(s, it_last_error());
}
inline void require(bool cond, const char* msg) {
  if (!cond) throw std::logic_error(msg);
}

enum class Precision { FP32, BF16 };
inline size_t byte_size(Precision p) { return p == Precision::FP32 ? 4 : 2; }

// src/precision.rs:24-29
inline uint16_t f32_to_bf16(float x) {
  uint32_t bits;
  std::memcpy(&bits, &x, 4);
  const uint32_t round = ((bits >> 16) & 1u) + 0x7FFFu;
  return static_cast<uint16_t>((bits + round) >> 16);
}
inline float bf16_to_f32(uint16_t x) {
  const uint32_t bits = static_cast<uint32_t>(x) << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// One context per device for the whole process and one stream per (thread, context) (MetalContext::global,
// src/device.rs:27-29; the thread-local CommandBatch, src/command_batch.rs:49-53).  global() is the context of
// the default device (0 until set_default_device); global(d) that of device d.
// Ownership rule, as for the reference's thread-local batch: work is ordered only within the calling thread's
// stream.  A Tensor (zeros() and uploads are enqueued, not finished, when they return) may be handed to another
// thread only after CommandBatch::sync() on the thread that produced it.
class Context {
 public:
  static void set_default_device(int device) { default_device() = device; }
  static Context& global(int device = -1) {
    static std::mutex m;
    static std::map<int, std::unique_ptr<Context>> all;
    if (device < 0) device = default_device();
    std::lock_guard<std::mutex> lock(m);
    auto& slot = all[device];
    if (!slot) slot.reset(new Context(device));
    return *slot;
  }
  it_ctx* raw() const { return ctx_; }
  it_stream* stream() {
    thread_local std::map<it_ctx*, it_stream*> mine;   // streams live as long as the process, like the contexts
    it_stream*& s = mine[ctx_];
    if (s == nullptr) check(it_stream_create(ctx_, &s));
    return s;
  }
  ~Context() { it_ctx_destroy(ctx_); }

 private:
  explicit Context(int device) { check(it_ctx_create(device, &ctx_)); }
  static int& default_device() {
    static int d = 0;
    return d;
  }
  it_ctx* ctx_ = nullptr;
};

struct CommandBatch {
  static void begin() { active() = true; }
  static bool is_active() { return active(); }
  static void sync() { check(it_stream_sync(Context::global().raw(), Context::global().stream())); }
  static void end() {
    sync();
    active() = false;
  }
  static void commit_async() {
    it_event*& ev = pending();
    if (ev == nullptr) check(it_event_create(Context::global().raw(), &ev));
    check(it_event_record(Context::global().raw(), Context::global().stream(), ev));
    recorded() = true;
    active() = false;
  }
  static bool is_async_complete() {
    if (!recorded()) return true;
    int32_t done = 0;
    check(it_event_query(Context::global().raw(), pending(), &done));
    return done != 0;
  }
  static void wait_for_completion() {
    if (!recorded()) return;
    check(it_event_wait(Context::global().raw(), pending()));
    recorded() = false;
  }
  // Raises it::Error(IT_ERR_TIMEOUT) if a kernel's bounded wait ran out since the last poll.
  static void poll_device_status() {
    int32_t st = 0;
    check(it_attention_status_poll(Context::global().raw(), Context::global().stream(), &st));
  }

 private:
  static bool& active() {
    thread_local bool a = false;
    return a;
  }
  static bool& recorded() {
    thread_local bool r = false;
    return r;
  }
  static it_event*& pending() {
    thread_local it_event* e = nullptr;
    return e;
  }
};

// Device buffer + shape + precision (src/tensor.rs:11-15).  view() shares the buffer, like the
// reference's retained MTLBuffer (src/tensor.rs:183-198).
class Tensor {
 public:
  Tensor() = default;
  static Tensor zeros(const std::vector<size_t>& shape, Precision p = Precision::FP32) {
    Tensor t(shape, p);
    check(it_buf_memset_async(Context::global().raw(), Context::global().stream(), t.ptr(), 0, t.byte_size()));
    return t;
  }
  static Tensor empty(const std::vector<size_t>& shape, Precision p) { return Tensor(shape, p); }
  static Tensor from_f32_slice(const std::vector<float>& data, const std::vector<size_t>& shape) {
    Tensor t(shape, Precision::FP32);
    require(data.size() == t.numel(), "Data length does not match shape");
    check(it_buf_upload(Context::global().raw(), Context::global().stream(), t.ptr(), data.data(), t.byte_size()));
    CommandBatch::sync();   // `data` may go away after the call
    return t;
  }
  static Tensor from_f32_as_bf16(const std::vector<float>& data, const std::vector<size_t>& shape) {
    Tensor t(shape, Precision::BF16);
    require(data.size() == t.numel(), "Data length does not match shape");
    std::vector<uint16_t> bits(data.size());
    for (size_t i = 0; i < data.size(); ++i) bits[i] = f32_to_bf16(data[i]);
    check(it_buf_upload(Context::global().raw(), Context::global().stream(), t.ptr(), bits.data(), t.byte_size()));
    CommandBatch::sync();
    return t;
  }
  const std::vector<size_t>& shape() const { return shape_; }
  Precision precision() const { return precision_; }
  size_t numel() const {
    size_t n = 1;
    for (size_t d : shape_) n *= d;
    return n;
  }
  size_t byte_size() const { return numel() * it::byte_size(precision_); }
  void* ptr() const { return buf_ ? buf_->dev : nullptr; }
  // Values on the host as fp32, whatever the storage precision (as_f32_slice, src/tensor.rs:136-148;
  // the reference aliases unified memory, here the stream is drained and the bytes are copied).
  std::vector<float> to_host_f32() const {
    std::vector<float> out(numel());
    if (numel() == 0) return out;
    if (precision_ == Precision::FP32) {
      check(it_buf_download(Context::global().raw(), Context::global().stream(), out.data(), ptr(), byte_size()));
      CommandBatch::sync();
    } else {
      std::vector<uint16_t> bits(numel());
      check(it_buf_download(Context::global().raw(), Context::global().stream(), bits.data(), ptr(), byte_size()));
      CommandBatch::sync();
      for (size_t i = 0; i < bits.size(); ++i) out[i] = bf16_to_f32(bits[i]);
    }
    return out;
  }
  Tensor view(const std::vector<size_t>& new_shape) const {
    Tensor t = *this;
    t.shape_ = new_shape;
    require(t.numel() == numel(), "Cannot view tensor with a different number of elements");
    return t;
  }
  // Side output of flash_attention: per-row log-sum-exp [B,H,S], fp32 (the reference has none).
  std::shared_ptr<Tensor> lse;

 private:
  struct Buf {
    void* dev = nullptr;
    ~Buf() {
      if (dev) it_buf_free(Context::global().raw(), dev);
    }
  };
  Tensor(const std::vector<size_t>& shape, Precision p) : shape_(shape), precision_(p), buf_(std::make_shared<Buf>()) {
    check(it_buf_alloc(Context::global().raw(), byte_size(), &buf_->dev));
  }
  std::vector<size_t> shape_;
  Precision precision_ = Precision::FP32;
  std::shared_ptr<Buf> buf_;
};

inline it_dtype dtype_code(Precision p) { return p == Precision::FP32 ? IT_F32 : IT_BF16; }

// Scratch for the calls that need a workspace: one grow-only buffer per thread (and so per stream), reused by
// every call, so that an op neither allocates nor drains the stream in the steady state.  Growing drains the
// stream once before the smaller buffer is released.
inline void* thread_workspace(size_t bytes) {
  thread_local Tensor ws;
  if (ws.byte_size() < bytes || ws.ptr() == nullptr) {
    if (ws.ptr() != nullptr) check(it_stream_sync(Context::global().raw(), Context::global().stream()));
    ws = Tensor::empty({bytes / 4 + 64}, Precision::FP32);
  }
  return ws.ptr();
}

// src/ops/flash_attention.rs:76-193
inline Tensor flash_attention(const Tensor& q, const Tensor& k, const Tensor& v, bool causal) {
  require(q.precision() == k.precision() && q.precision() == v.precision(), "Q, K and V must have the same precision");
  require(q.shape().size() == 4, "Q must be 4D [batch, heads, seq, head_dim]");
  require(k.shape().size() == 4, "K must be 4D [batch, heads, seq, head_dim]");
  require(v.shape().size() == 4, "V must be 4D [batch, heads, seq, head_dim]");
  require(q.shape() == k.shape(), "Q and K must have same shape");
  require(q.shape() == v.shape(), "Q and V must have same shape");
  const auto& s = q.shape();
  require(s[3] <= 128, "head_dim must be <= 128");
  Tensor out = Tensor::zeros(s, q.precision());
  out.lse = std::make_shared<Tensor>(Tensor::zeros({s[0], s[1], s[2]}, Precision::FP32));
  if (s[2] == 0 || s[0] * s[1] == 0) return out;
  check(it_flash_attention_fwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                               static_cast<int32_t>(s[0]), static_cast<int32_t>(s[1]), static_cast<int32_t>(s[2]),
                               static_cast<int32_t>(s[3]), causal ? 1 : 0, q.ptr(), k.ptr(), v.ptr(), out.ptr(),
                               static_cast<float*>(out.lse->ptr())));
  return out;
}

// src/train/helpers.rs:120-193.  The reference takes (grad_output, q, k, v) and is always causal; pass
// the forward's result (`o`, carrying `o.lse`) to skip re-running the forward.
inline std::tuple<Tensor, Tensor, Tensor> attention_backward_recompute(const Tensor& grad_output, const Tensor& q,
                                                                       const Tensor& k, const Tensor& v,
                                                                       const Tensor* o = nullptr, bool causal = true) {
  const auto& s = q.shape();
  require(s.size() == 4, "Q must be 4D [batch, heads, seq, head_dim]");
  require(grad_output.shape() == s && k.shape() == s && v.shape() == s, "shape mismatch");
  require(grad_output.precision() == q.precision() && k.precision() == q.precision() && v.precision() == q.precision(),
          "all tensors must have the same precision");
  Tensor dq = Tensor::zeros(s, q.precision()), dk = Tensor::zeros(s, q.precision()), dv = Tensor::zeros(s, q.precision());
  if (s[2] == 0 || s[0] * s[1] == 0) return {dq, dk, dv};
  Tensor fwd;
  if (o == nullptr || !o->lse) {
    fwd = flash_attention(q, k, v, causal);
    o = &fwd;
  }
  size_t ws_bytes = 0;
  check(it_flash_attention_bwd_workspace_bytes(dtype_code(q.precision()), static_cast<int32_t>(s[0]),
                                               static_cast<int32_t>(s[1]), static_cast<int32_t>(s[2]),
                                               static_cast<int32_t>(s[3]), &ws_bytes));
  void* const ws = thread_workspace(ws_bytes);
  check(it_flash_attention_bwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                               static_cast<int32_t>(s[0]), static_cast<int32_t>(s[1]), static_cast<int32_t>(s[2]),
                               static_cast<int32_t>(s[3]), causal ? 1 : 0, q.ptr(), k.ptr(), v.ptr(), o->ptr(),
                               grad_output.ptr(), static_cast<const float*>(o->lse->ptr()), dq.ptr(), dk.ptr(), dv.ptr(),
                               ws, ws_bytes));
  return {dq, dk, dv};
}

// src/ops/attention.rs:286-377: [batch, seq, heads, head_dim] in and out.  The kernels read and write
// this layout in place, so the transposes the reference runs around its GEMMs are gone.  K/V may have
// another sequence length than Q when not causal (src/ops/attention.rs:304,349-352).  The result carries
// `.lse` ([batch, heads, seq]) for attention_backward.
inline Tensor attention(const Tensor& q, const Tensor& k, const Tensor& v, bool causal) {
  require(q.shape().size() == 4, "Q must be 4D [batch, seq, heads, dim]");
  require(k.shape().size() == 4, "K must be 4D [batch, seq, heads, dim]");
  require(v.shape().size() == 4, "V must be 4D [batch, seq, heads, dim]");
  require(q.precision() == k.precision() && q.precision() == v.precision(), "Q, K and V must have the same precision");
  const size_t B = q.shape()[0], S = q.shape()[1], H = q.shape()[2], D = q.shape()[3];
  require(k.shape()[0] == B && v.shape()[0] == B, "Batch size mismatch");
  require(k.shape()[2] == H && v.shape()[2] == H, "Num heads mismatch");
  require(k.shape()[3] == D && v.shape()[3] == D, "Head dim mismatch");
  require(v.shape()[1] == k.shape()[1], "K and V seq_len must match");
  Tensor out = Tensor::zeros({B, S, H, D}, q.precision());
  out.lse = std::make_shared<Tensor>(Tensor::zeros({B, H, S}, Precision::FP32));
  if (B == 0 || S == 0 || k.shape()[1] == 0) return out;
  if (causal) require(k.shape()[1] == S, "Causal attention requires Q and K to have same seq_len");
  if (k.shape()[1] != S) {
    check(it_attention_cross_fwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                                 static_cast<int32_t>(B), static_cast<int32_t>(S), static_cast<int32_t>(k.shape()[1]),
                                 static_cast<int32_t>(H), static_cast<int32_t>(D), q.ptr(), k.ptr(), v.ptr(), out.ptr(),
                                 static_cast<float*>(out.lse->ptr())));
    return out;
  }
  check(it_attention_fwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                         static_cast<int32_t>(B), static_cast<int32_t>(S), static_cast<int32_t>(H), static_cast<int32_t>(D),
                         causal ? 1 : 0, q.ptr(), k.ptr(), v.ptr(), out.ptr(), static_cast<float*>(out.lse->ptr())));
  return out;
}

// Gradients for attention(), all tensors [batch, seq, heads, head_dim]; `o` is attention()'s result.
inline std::tuple<Tensor, Tensor, Tensor> attention_backward(const Tensor& grad_output, const Tensor& q, const Tensor& k,
                                                             const Tensor& v, const Tensor& o, bool causal = true) {
  const auto& s = q.shape();
  require(s.size() == 4 && grad_output.shape() == s && k.shape() == s && v.shape() == s && o.shape() == s, "shape mismatch");
  require(static_cast<bool>(o.lse), "o must come from attention()");
  Tensor dq = Tensor::zeros(s, q.precision()), dk = Tensor::zeros(s, q.precision()), dv = Tensor::zeros(s, q.precision());
  if (s[1] == 0 || s[0] * s[2] == 0) return {dq, dk, dv};
  size_t ws_bytes = 0;
  check(it_flash_attention_bwd_workspace_bytes(dtype_code(q.precision()), static_cast<int32_t>(s[0]),
                                               static_cast<int32_t>(s[2]), static_cast<int32_t>(s[1]),
                                               static_cast<int32_t>(s[3]), &ws_bytes));
  void* const ws = thread_workspace(ws_bytes);
  check(it_attention_bwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                         static_cast<int32_t>(s[0]), static_cast<int32_t>(s[1]), static_cast<int32_t>(s[2]),
                         static_cast<int32_t>(s[3]), causal ? 1 : 0, q.ptr(), k.ptr(), v.ptr(), o.ptr(), grad_output.ptr(),
                         static_cast<const float*>(o.lse->ptr()), dq.ptr(), dk.ptr(), dv.ptr(), ws, ws_bytes));
  return {dq, dk, dv};
}

// Grouped-query attention: q [batch, seq, heads, head_dim], k and v [batch, seq, kv_heads, head_dim].  Equal to
// attention(q, repeat_kv(k), repeat_kv(v), causal) of the reference (src/train/forward.rs:117-139;
// repeat_kv_gpu, src/ops/repeat_kv.rs:68-149) without the expanded copies.
inline Tensor attention_gqa(const Tensor& q, const Tensor& k, const Tensor& v, bool causal = true) {
  require(q.shape().size() == 4 && k.shape().size() == 4 && v.shape().size() == 4, "Q, K and V must be 4D");
  require(k.shape() == v.shape(), "K and V must have the same shape");
  const size_t B = q.shape()[0], S = q.shape()[1], H = q.shape()[2], D = q.shape()[3], Hkv = k.shape()[2];
  require(k.shape()[0] == B && k.shape()[1] == S && k.shape()[3] == D, "K/V must be [batch, seq, kv_heads, head_dim]");
  require(Hkv >= 1 && H % Hkv == 0, "num_heads must be divisible by num_kv_heads");   // src/ops/repeat_kv.rs:77-80
  Tensor out = Tensor::zeros({B, S, H, D}, q.precision());
  out.lse = std::make_shared<Tensor>(Tensor::zeros({B, H, S}, Precision::FP32));
  if (B * S * H == 0) return out;
  check(it_attention_gqa_fwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                             static_cast<int32_t>(B), static_cast<int32_t>(S), static_cast<int32_t>(H),
                             static_cast<int32_t>(Hkv), static_cast<int32_t>(D), causal ? 1 : 0, q.ptr(), k.ptr(), v.ptr(),
                             out.ptr(), static_cast<float*>(out.lse->ptr())));
  return out;
}

// (dQ, dK, dV) for attention_gqa(); dK, dV come back summed over each group (repeat_kv_backward,
// src/ops/repeat_kv.rs:151-232, folded in).  With rope_base > 0, q and k are the ROTATED tensors the
// forward attended over and dQ, dK are gradients of the un-rotated ones (the reference's two
// rope_backward passes, src/train/backward.rs:129,132, folded in).
inline std::tuple<Tensor, Tensor, Tensor> attention_gqa_backward(const Tensor& grad_output, const Tensor& q, const Tensor& k,
                                                                 const Tensor& v, const Tensor& o, bool causal = true,
                                                                 float rope_base = 0.f, int position_offset = 0) {
  const auto& s = q.shape();
  require(s.size() == 4 && grad_output.shape() == s && o.shape() == s && k.shape() == v.shape(), "shape mismatch");
  require(static_cast<bool>(o.lse), "o must come from attention_gqa()");
  const int32_t B = static_cast<int32_t>(s[0]), S = static_cast<int32_t>(s[1]), H = static_cast<int32_t>(s[2]),
                D = static_cast<int32_t>(s[3]), Hkv = static_cast<int32_t>(k.shape()[2]);
  Tensor dq = Tensor::zeros(s, q.precision()), dk = Tensor::zeros(k.shape(), q.precision()), dv = Tensor::zeros(k.shape(), q.precision());
  if (s[0] * s[1] * s[2] == 0) return {dq, dk, dv};
  size_t ws_bytes = 0;
  check(it_flash_attention_bwd_workspace_bytes(dtype_code(q.precision()), B, H, S, D, &ws_bytes));
  void* const ws = thread_workspace(ws_bytes);
  if (rope_base > 0.f) {
    check(it_attention_gqa_bwd_rope(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()), B, S, H, Hkv,
                                    D, causal ? 1 : 0, rope_base, position_offset, q.ptr(), k.ptr(), v.ptr(), o.ptr(),
                                    grad_output.ptr(), static_cast<const float*>(o.lse->ptr()), dq.ptr(), dk.ptr(), dv.ptr(),
                                    ws, ws_bytes));
  } else {
    check(it_attention_gqa_bwd(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()), B, S, H, Hkv, D,
                               causal ? 1 : 0, q.ptr(), k.ptr(), v.ptr(), o.ptr(), grad_output.ptr(),
                               static_cast<const float*>(o.lse->ptr()), dq.ptr(), dk.ptr(), dv.ptr(), ws, ws_bytes));
  }
  return {dq, dk, dv};
}

// rope(q) and rope(k) (src/ops/rope.rs:22-75; src/train/forward.rs:111-112) as one launch; k may have fewer
// heads.  `inverse` gives the backward rotation.
inline std::pair<Tensor, Tensor> rope_qk(const Tensor& q, const Tensor& k, float base = 10000.f, int position_offset = 0,
                                         bool inverse = false) {
  require(q.shape().size() == 4 && k.shape().size() == 4, "Input must be 4D [batch, seq_len, num_heads, head_dim]");
  require(q.shape()[3] % 2 == 0, "head_dim must be even for RoPE");
  require(k.shape()[0] == q.shape()[0] && k.shape()[1] == q.shape()[1] && k.shape()[3] == q.shape()[3], "q and k must agree");
  Tensor qo = Tensor::empty(q.shape(), q.precision()), ko = Tensor::empty(k.shape(), q.precision());
  check(it_rope_qk(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()),
                   static_cast<int32_t>(q.shape()[0]), static_cast<int32_t>(q.shape()[1]), static_cast<int32_t>(q.shape()[2]),
                   static_cast<int32_t>(k.shape()[2]), static_cast<int32_t>(q.shape()[3]), base, position_offset, inverse ? 1 : 0,
                   q.ptr(), k.ptr(), qo.ptr(), ko.ptr()));
  return {qo, ko};
}

// One new token per sequence against a key/value cache: q [batch, heads, head_dim], caches [batch, max_len,
// kv_heads, head_dim] with the first kv_len positions valid.  (The reference's generator recomputes the whole
// forward per token, src/inference/generator.rs:146-200.)
inline Tensor attention_decode(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, size_t kv_len) {
  require(q.shape().size() == 3 && k_cache.shape().size() == 4 && k_cache.shape() == v_cache.shape(), "shape mismatch");
  const int32_t B = static_cast<int32_t>(q.shape()[0]), H = static_cast<int32_t>(q.shape()[1]),
                D = static_cast<int32_t>(q.shape()[2]), max_len = static_cast<int32_t>(k_cache.shape()[1]),
                Hkv = static_cast<int32_t>(k_cache.shape()[2]);
  Tensor out = Tensor::zeros(q.shape(), q.precision());
  out.lse = std::make_shared<Tensor>(Tensor::zeros({q.shape()[0], q.shape()[1]}, Precision::FP32));
  size_t ws_bytes = 0;
  check(it_attention_decode_workspace_bytes(B, H, D, &ws_bytes));
  void* const ws = thread_workspace(ws_bytes);
  check(it_attention_decode(Context::global().raw(), Context::global().stream(), dtype_code(q.precision()), B, H, Hkv, D,
                            static_cast<int32_t>(kv_len), max_len, q.ptr(), k_cache.ptr(), v_cache.ptr(), out.ptr(),
                            static_cast<float*>(out.lse->ptr()), ws, ws_bytes));
  return out;
}

// output = input @ weight.T for BF16 tensors: input [n, in], weight [out, in] (src/train/helpers.rs:48-53).
inline Tensor linear_forward(const Tensor& input, const Tensor& weight) {
  require(input.precision() == Precision::BF16 && weight.precision() == Precision::BF16, "linear_forward takes BF16 tensors");
  require(input.shape().size() == 2 && weight.shape().size() == 2 && input.shape()[1] == weight.shape()[1],
          "inner dimensions must match");
  Tensor y = Tensor::empty({input.shape()[0], weight.shape()[0]}, Precision::BF16);
  check(it_linear_fwd(Context::global().raw(), Context::global().stream(), static_cast<int32_t>(input.shape()[0]),
                      static_cast<int32_t>(input.shape()[1]), static_cast<int32_t>(weight.shape()[0]), input.ptr(), weight.ptr(),
                      y.ptr()));
  return y;
}

// (grad_input BF16 [n, in], grad_weight FP32 [out, in]) = (grad_output @ weight, grad_output.T @ input)
// (src/train/helpers.rs:61-76; the reference returns FP32 gradients).
inline std::pair<Tensor, Tensor> linear_backward(const Tensor& grad_output, const Tensor& input, const Tensor& weight) {
  require(grad_output.shape().size() == 2 && input.shape().size() == 2 && weight.shape().size() == 2, "2D tensors expected");
  const size_t n = grad_output.shape()[0], out = grad_output.shape()[1], in = input.shape()[1];
  require(input.shape()[0] == n && weight.shape()[0] == out && weight.shape()[1] == in, "shape mismatch");
  Tensor dx = Tensor::empty({n, in}, Precision::BF16), dw = Tensor::empty({out, in}, Precision::FP32);
  check(it_linear_bwd(Context::global().raw(), Context::global().stream(), static_cast<int32_t>(n), static_cast<int32_t>(in),
                      static_cast<int32_t>(out), grad_output.ptr(), input.ptr(), weight.ptr(), dx.ptr(),
                      static_cast<float*>(dw.ptr())));
  return {dx, dw};
}

// q_rope, k_rope, v from x [batch, seq, hidden] and the stacked weights [Wq; Wk; Wv] in one kernel
// (src/train/forward.rs:101-103,111-112).  rope_base 0: no rotation.
inline std::tuple<Tensor, Tensor, Tensor> qkv_rope_forward(const Tensor& x, const Tensor& w_qkv, size_t heads, size_t kv_heads,
                                                           size_t head_dim, float rope_base = 10000.f, int position_offset = 0) {
  require(x.shape().size() == 3 && w_qkv.shape().size() == 2, "x must be [batch, seq, hidden], w_qkv 2D");
  const size_t B = x.shape()[0], S = x.shape()[1], hidden = x.shape()[2];
  require(w_qkv.shape()[0] == (heads + 2 * kv_heads) * head_dim && w_qkv.shape()[1] == hidden,
          "w_qkv must be [Wq; Wk; Wv] stacked by rows");
  Tensor q = Tensor::empty({B, S, heads, head_dim}, Precision::BF16), k = Tensor::empty({B, S, kv_heads, head_dim}, Precision::BF16),
         v = Tensor::empty({B, S, kv_heads, head_dim}, Precision::BF16);
  size_t ws_bytes = 0;
  check(it_qkv_rope_workspace_bytes(static_cast<int32_t>(S), static_cast<int32_t>(head_dim), &ws_bytes));
  void* const ws = thread_workspace(ws_bytes);
  check(it_qkv_rope_fwd(Context::global().raw(), Context::global().stream(), static_cast<int32_t>(B), static_cast<int32_t>(S),
                        static_cast<int32_t>(hidden), static_cast<int32_t>(heads), static_cast<int32_t>(kv_heads),
                        static_cast<int32_t>(head_dim), rope_base, position_offset, x.ptr(), w_qkv.ptr(), q.ptr(), k.ptr(), v.ptr(),
                        ws, ws_bytes));
  return {q, k, v};
}

}  // namespace it
