"""Host-side mirror of the reference's attention interface, on top of the C ABI.

Same names, argument meaning and error behaviour as the reference (paths relative to its root):
  Precision, Tensor            src/precision.rs:1-29, src/tensor.rs:11-300
  CommandBatch                 src/command_batch.rs:167-391
  flash_attention              src/ops/flash_attention.rs:76-193     [B,H,S,D]
  attention                    src/ops/attention.rs:286-377          [B,S,H,D]
  attention_backward_recompute src/train/helpers.rs:120-193          [B,H,S,D]
Where the reference asserts (panics), these raise AssertionError with the same message.

torch is used for plumbing only: device memory, the current CUDA stream and pinned host buffers.
All arithmetic runs in libirontensor_b200.so; if that library cannot be loaded, or no CUDA device
is present, every op raises -- there is no fallback.
"""
import ctypes
import enum
import threading

import numpy as np

from . import _lib, synth


class Precision(enum.Enum):
    FP32 = 0
    BF16 = 1

    def byte_size(self):
        return 4 if self is Precision.FP32 else 2


_state = threading.local()
_ctx_lock = threading.Lock()
_ctxs = {}


def _torch():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("irontensor_b200 needs a CUDA device (sm_100a); none is visible and there is no fallback")
    return torch


class _Context:
    """Per-device library context (the reference's MetalContext::global, src/device.rs:15-29)."""

    def __init__(self, device):
        self.lib = _lib.load()
        self.device = device
        h = ctypes.c_void_p()
        _lib.check(self.lib.it_ctx_create(device, ctypes.byref(h)))
        self.handle = h
        self._streams = {}

    def stream(self):
        """it_stream wrapping torch's current stream on this device."""
        torch = _torch()
        raw_stream = torch.cuda.current_stream(self.device).cuda_stream
        s = self._streams.get(raw_stream)
        if s is None:
            s = ctypes.c_void_p()
            _lib.check(self.lib.it_stream_wrap(self.handle, ctypes.c_void_p(raw_stream), ctypes.byref(s)))
            self._streams[raw_stream] = s
        return s

    def launch_count(self):
        n = ctypes.c_uint64()
        _lib.check(self.lib.it_ctx_launch_count(self.handle, ctypes.byref(n)))
        return n.value

    def enable_kernel_timing(self, on=True):
        """False / 0: off; True / 1: the backward main kernel; 2: the forward kernel too; 3: the backward's prepare and
        finish passes as well."""
        _lib.check(self.lib.it_ctx_enable_kernel_timing(self.handle, int(on)))

    def kernel_tag(self, which):
        """The reference's profiler tag for what timer `which` covers (FlashAttention, attn_bwd/...)."""
        return self.lib.it_ctx_kernel_tag(which).decode()

    def kernel_ms(self, which):
        """Device time of the most recent forward (0), backward-main (1), backward-prepare (2) or backward-finish (3) kernel."""
        ms = ctypes.c_float()
        _lib.check(self.lib.it_ctx_kernel_ms(self.handle, which, ctypes.byref(ms)))
        return ms.value

    def check_status(self):
        """Raises ITError(IT_ERR_TIMEOUT) if a kernel's bounded wait ran out on this context (every later launch
        is then a no-op and its outputs are garbage).  Does not drain a stream and does not clear the word;
        call it after the results have been waited for.  poll_status() clears."""
        _lib.check(self.lib.it_ctx_check_status(self.handle, None))

    def poll_status(self):
        """Drains the current stream; raises ITError(IT_ERR_TIMEOUT) if a kernel's wait ran out."""
        st = ctypes.c_int32()
        rc = self.lib.it_attention_status_poll(self.handle, self.stream(), ctypes.byref(st))
        _lib.check(rc)
        return st.value


def context(device=None):
    torch = _torch()
    if device is None:
        device = torch.cuda.current_device()
    with _ctx_lock:
        c = _ctxs.get(device)
        if c is None:
            c = _Context(device)
            _ctxs[device] = c
        return c


class CommandBatch:
    """The reference batches encoded work per thread and flushes on sync (src/command_batch.rs:167-391).
    Here work is enqueued on the thread's current CUDA stream as soon as an op is called; these
    functions keep the same call sites meaningful.  sync, end and wait_for_completion raise ITError(IT_ERR_TIMEOUT)
    when a kernel's bounded wait ran out (it_stream_sync / it_event_wait report the device status word)."""

    @staticmethod
    def begin():
        _state.active = True

    @staticmethod
    def is_active():
        return getattr(_state, "active", False)

    @staticmethod
    def sync():
        c = context()
        _lib.check(c.lib.it_stream_sync(c.handle, c.stream()))

    @staticmethod
    def end():
        CommandBatch.sync()
        _state.active = False

    @staticmethod
    def commit_async():
        c = context()
        ev = ctypes.c_void_p()
        _lib.check(c.lib.it_event_create(c.handle, ctypes.byref(ev)))
        _lib.check(c.lib.it_event_record(c.handle, c.stream(), ev))
        old = getattr(_state, "pending", None)
        if old is not None:
            c.lib.it_event_destroy(c.handle, old)
        _state.pending = ev
        _state.active = False

    @staticmethod
    def is_async_complete():
        ev = getattr(_state, "pending", None)
        if ev is None:
            return True
        c = context()
        done = ctypes.c_int32()
        _lib.check(c.lib.it_event_query(c.handle, ev, ctypes.byref(done)))
        return bool(done.value)

    @staticmethod
    def wait_for_completion():
        ev = getattr(_state, "pending", None)
        if ev is None:
            return
        c = context()
        _lib.check(c.lib.it_event_wait(c.handle, ev))
        c.lib.it_event_destroy(c.handle, ev)
        _state.pending = None


class Tensor:
    """Device-resident tensor: buffer + shape + precision (src/tensor.rs:11-15).

    The reference's buffers are unified memory, so `as_f32_slice` aliases GPU memory
    (src/tensor.rs:136-148); here it synchronises the stream and copies device -> host."""

    def __init__(self, data, shape, precision):
        self._data = data            # flat torch CUDA tensor (float32 or bfloat16)
        self._shape = list(shape)
        self._precision = precision
        self.lse = None              # side output of flash_attention: Tensor [B,H,S] fp32

    # -- constructors (src/tensor.rs:63-118, 205-240)
    @staticmethod
    def zeros(shape, precision=Precision.FP32):
        torch = _torch()
        dt = torch.float32 if precision is Precision.FP32 else torch.bfloat16
        n = int(np.prod(shape)) if len(shape) else 1
        return Tensor(torch.zeros(max(n, 1), dtype=dt, device="cuda")[:n], shape, precision)

    @staticmethod
    def from_f32_slice(data, shape):
        torch = _torch()
        a = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        n = int(np.prod(shape))
        assert a.size == n, f"Data length {a.size} does not match shape {list(shape)} (numel={n})"
        return Tensor(torch.from_numpy(a).to("cuda", non_blocking=False), shape, Precision.FP32)

    @staticmethod
    def from_bf16_slice(bits, shape):
        torch = _torch()
        a = np.ascontiguousarray(bits, dtype=np.uint16).reshape(-1)
        n = int(np.prod(shape))
        assert a.size == n, f"Data length {a.size} does not match shape {list(shape)} (numel={n})"
        t = torch.from_numpy(a.view(np.int16)).to("cuda").view(torch.bfloat16)
        return Tensor(t, shape, Precision.BF16)

    @staticmethod
    def from_f32_as_bf16(data, shape):
        return Tensor.from_bf16_slice(synth.f32_to_bf16_bits(np.asarray(data, dtype=np.float32).reshape(-1)), shape)

    @staticmethod
    def empty(shape, precision=Precision.FP32):
        """Uninitialised storage, for outputs a kernel overwrites completely."""
        torch = _torch()
        dt = torch.float32 if precision is Precision.FP32 else torch.bfloat16
        n = int(np.prod(shape)) if len(shape) else 1
        return Tensor(torch.empty(max(n, 1), dtype=dt, device="cuda")[:n], shape, precision)

    # -- explicit, stream-ordered copies to and from page-locked host memory
    def upload_from(self, host):
        """Asynchronous host -> device copy of a pinned torch tensor with the same byte size."""
        c = context()
        assert host.is_pinned() and host.numel() * host.element_size() == self.byte_size()
        _lib.check(c.lib.it_buf_upload(c.handle, c.stream(), self.data_ptr(), host.data_ptr(), self.byte_size()))
        return self

    def download_to(self, host):
        """Asynchronous device -> host copy into a pinned torch tensor with the same byte size."""
        c = context()
        assert host.is_pinned() and host.numel() * host.element_size() == self.byte_size()
        _lib.check(c.lib.it_buf_download(c.handle, c.stream(), host.data_ptr(), self.data_ptr(), self.byte_size()))
        return host

    # -- accessors
    def shape(self):
        return list(self._shape)

    def precision(self):
        return self._precision

    def numel(self):
        return int(np.prod(self._shape)) if self._shape else 1

    def byte_size(self):
        return self.numel() * self._precision.byte_size()

    def is_bf16(self):
        return self._precision is Precision.BF16

    def is_f32(self):
        return self._precision is Precision.FP32

    def data_ptr(self):
        return self._data.data_ptr()

    def torch(self):
        return self._data.view(self._shape)

    def as_f32_slice(self):
        assert self._precision is Precision.FP32, "Tensor is not FP32"
        host = self._data.cpu().numpy()      # drains the stream
        context(self._data.device.index).check_status()   # a kernel that gave up leaves garbage here: raise instead
        return host

    def as_bf16_slice(self):
        assert self._precision is Precision.BF16, "Tensor is not BF16"
        torch = _torch()
        host = self._data.view(torch.int16).cpu().numpy().view(np.uint16)
        context(self._data.device.index).check_status()
        return host

    def to_f32_host(self):
        """Values as fp32 on the host, whatever the storage precision."""
        if self._precision is Precision.FP32:
            return self.as_f32_slice().reshape(self._shape)
        return synth.bf16_bits_to_f32(self.as_bf16_slice()).reshape(self._shape)

    def view(self, new_shape):
        n = int(np.prod(new_shape))
        assert n == self.numel(), f"Cannot view tensor with {self.numel()} elements as shape {list(new_shape)}"
        t = Tensor(self._data, new_shape, self._precision)
        return t

    def to_bf16(self):
        if self._precision is Precision.BF16:
            return Tensor(self._data.clone(), self._shape, Precision.BF16)
        return Tensor.from_f32_as_bf16(self.as_f32_slice(), self._shape)

    def to_f32(self):
        torch = _torch()
        return Tensor(self._data.to(torch.float32), self._shape, Precision.FP32)


def _dtype_code(p):
    return _lib.IT_F32 if p is Precision.FP32 else _lib.IT_BF16


class raw:
    """Thin typed wrappers over the two compute entry points, taking raw device pointers."""

    @staticmethod
    def fwd(dtype, B, H, S, D, causal, q, k, v, o, lse, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_flash_attention_fwd(c.handle, c.stream(), dtype, B, H, S, D, int(causal), q, k, v, o, lse))

    @staticmethod
    def fwd_bshd(dtype, B, S, H, D, causal, q, k, v, o, lse, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_fwd(c.handle, c.stream(), dtype, B, S, H, D, int(causal), q, k, v, o, lse))

    @staticmethod
    def bwd_bshd(dtype, B, S, H, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, ws, ws_bytes, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_bwd(c.handle, c.stream(), dtype, B, S, H, D, int(causal), q, k, v, o, d_o, lse,
                                          dq, dk, dv, ws, ws_bytes))

    @staticmethod
    def fwd_gqa(dtype, B, S, H, Hkv, D, causal, q, k, v, o, lse, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_gqa_fwd(c.handle, c.stream(), dtype, B, S, H, Hkv, D, int(causal), q, k, v, o, lse))

    @staticmethod
    def bwd_gqa(dtype, B, S, H, Hkv, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, ws, ws_bytes, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_gqa_bwd(c.handle, c.stream(), dtype, B, S, H, Hkv, D, int(causal), q, k, v, o, d_o,
                                              lse, dq, dk, dv, ws, ws_bytes))

    @staticmethod
    def rope_qk(dtype, B, S, H, Hkv, D, base, position_offset, inverse, q_in, k_in, q_out, k_out, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_rope_qk(c.handle, c.stream(), dtype, B, S, H, Hkv, D, float(base), int(position_offset),
                                    int(inverse), q_in, k_in, q_out, k_out))

    @staticmethod
    def bwd_gqa_rope(dtype, B, S, H, Hkv, D, causal, base, position_offset, q, k, v, o, d_o, lse, dq, dk, dv, ws, ws_bytes,
                     ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_gqa_bwd_rope(c.handle, c.stream(), dtype, B, S, H, Hkv, D, int(causal), float(base),
                                                   int(position_offset), q, k, v, o, d_o, lse, dq, dk, dv, ws, ws_bytes))

    @staticmethod
    def decode_workspace_bytes(B, H, D):
        out = ctypes.c_size_t(0)
        _lib.check(_lib.load().it_attention_decode_workspace_bytes(B, H, D, ctypes.byref(out)))
        return out.value

    @staticmethod
    def decode(dtype, B, H, Hkv, D, kv_len, max_len, q, k_cache, v_cache, o, lse, ws, ws_bytes, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_decode(c.handle, c.stream(), dtype, B, H, Hkv, D, kv_len, max_len, q, k_cache,
                                             v_cache, o, lse, ws, ws_bytes))

    @staticmethod
    def linear_fwd(n, in_dim, out_dim, x, w, y, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_linear_fwd(c.handle, c.stream(), n, in_dim, out_dim, x, w, y))

    @staticmethod
    def qkv_rope_fwd(B, S, hidden, H, Hkv, D, base, position_offset, x, w_qkv, q, k, v, ctx=None):
        c = ctx or context()
        n = ctypes.c_size_t(0)
        _lib.check(c.lib.it_qkv_rope_workspace_bytes(S, D, ctypes.byref(n)))
        ws = _workspace(n.value)
        _lib.check(c.lib.it_qkv_rope_fwd(c.handle, c.stream(), B, S, hidden, H, Hkv, D, float(base), int(position_offset), x,
                                         w_qkv, q, k, v, ws.data_ptr(), ws.numel()))

    @staticmethod
    def packed_fwd(B, S, H, Hkv, D, causal, qkv, o, lse, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_packed_fwd(c.handle, c.stream(), _lib.IT_BF16, B, S, H, Hkv, D, int(causal), qkv, o, lse))

    @staticmethod
    def packed_bwd(B, S, H, Hkv, D, causal, base, position_offset, qkv, o, d_o, lse, dqkv, ws, ws_bytes, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_attention_packed_bwd(c.handle, c.stream(), _lib.IT_BF16, B, S, H, Hkv, D, int(causal), float(base),
                                                 int(position_offset), qkv, o, d_o, lse, dqkv, ws, ws_bytes))

    @staticmethod
    def linear_bwd(n, in_dim, out_dim, dy, x, w, dx, dw, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_linear_bwd(c.handle, c.stream(), n, in_dim, out_dim, dy, x, w, dx, dw))

    @staticmethod
    def linear_scatter_add(kind, n, in_dim, out_dim, a, w, c_of_rank, rows_per_rank, ctx=None):
        """kind 0: a W^T, kind 1: a W; row block r of the product is added into c_of_rank[r] (device pointers this
        process may store to, one per rank).  See it_linear_scatter_add."""
        c = ctx or context()
        arr = (ctypes.c_void_p * len(c_of_rank))(*[int(p) for p in c_of_rank])
        _lib.check(c.lib.it_linear_scatter_add(c.handle, c.stream(), kind, n, in_dim, out_dim, a, w, arr, len(c_of_rank),
                                               rows_per_rank))

    @staticmethod
    def bwd_workspace_bytes(dtype, B, H, S, D):
        n = ctypes.c_size_t()
        _lib.check(_lib.load().it_flash_attention_bwd_workspace_bytes(dtype, B, H, S, D, ctypes.byref(n)))
        return n.value

    @staticmethod
    def bwd(dtype, B, H, S, D, causal, q, k, v, o, d_o, lse, dq, dk, dv, ws, ws_bytes, ctx=None):
        c = ctx or context()
        _lib.check(c.lib.it_flash_attention_bwd(c.handle, c.stream(), dtype, B, H, S, D, int(causal), q, k, v, o, d_o,
                                                lse, dq, dk, dv, ws, ws_bytes))


_workspaces = {}


def _workspace(nbytes):
    """Grow-only scratch buffer per device (the ops allocate outputs like the reference does; the
    C ABI itself never allocates)."""
    torch = _torch()
    # one buffer per (device, stream): calls on different streams may run at the same time
    key = (torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        w = torch.empty(max(nbytes, 256), dtype=torch.uint8, device="cuda")
        _workspaces[key] = w
    return w


def flash_attention(q, k, v, causal):
    """FlashAttention forward on [batch, heads, seq, head_dim] (src/ops/flash_attention.rs:76-193).

    Accepts FP32 tensors like the reference and additionally BF16 (all three alike).  The per-row
    log-sum-exp the fused backward needs is attached to the result as `.lse`."""
    p = q.precision()
    assert p in (Precision.FP32, Precision.BF16)
    assert k.precision() is p and v.precision() is p, "Q, K and V must have the same precision"
    qs, ks, vs = q.shape(), k.shape(), v.shape()
    assert len(qs) == 4, "Q must be 4D [batch, heads, seq, head_dim]"
    assert len(ks) == 4, "K must be 4D [batch, heads, seq, head_dim]"
    assert len(vs) == 4, "V must be 4D [batch, heads, seq, head_dim]"
    assert qs == ks, "Q and K must have same shape"
    assert qs == vs, "Q and V must have same shape"
    B, H, S, D = qs
    assert D <= 128, "head_dim must be <= 128"
    if S == 0 or B * H == 0:
        out = Tensor.zeros([B, H, S, D], p)
        out.lse = Tensor.zeros([B, H, S], Precision.FP32)
        return out
    out = Tensor.empty([B, H, S, D], p)     # the kernel writes every element
    out.lse = Tensor.empty([B, H, S], Precision.FP32)
    raw.fwd(_dtype_code(p), B, H, S, D, causal, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
            out.lse.data_ptr())
    return out


def attention(q, k, v, causal):
    """Scaled dot-product attention on [batch, seq, heads, head_dim] (src/ops/attention.rs:286-377).

    Same math as flash_attention.  The kernels read and write this layout in place (strided TMA
    descriptors), so the transposes the reference runs around its attention are gone.  Accepts FP32
    like the reference, and BF16.  The result carries `.lse` ([batch, heads, seq]) for
    attention_backward.  K/V may have another sequence length when not causal, as in the reference
    (src/ops/attention.rs:304,349-352); that case runs on the CUDA-core kernels."""
    p = q.precision()
    assert k.precision() is p and v.precision() is p
    qs, ks, vs = q.shape(), k.shape(), v.shape()
    assert len(qs) == 4, "Q must be 4D [batch, seq, heads, dim]"
    assert len(ks) == 4, "K must be 4D [batch, seq, heads, dim]"
    assert len(vs) == 4, "V must be 4D [batch, seq, heads, dim]"
    B, Sq, H, D = qs
    assert ks[0] == B and vs[0] == B, "Batch size mismatch"
    assert ks[2] == H and vs[2] == H, "Num heads mismatch"
    assert ks[3] == D and vs[3] == D, "Head dim mismatch"
    assert vs[1] == ks[1], "K and V seq_len must match"
    if B == 0 or Sq == 0 or ks[1] == 0:
        return Tensor.zeros([B, Sq, H, D], p)
    if causal:
        assert ks[1] == Sq, "Causal attention requires Q and K to have same seq_len"      # src/ops/attention.rs:349-352
    out = Tensor.empty([B, Sq, H, D], p)
    out.lse = Tensor.empty([B, H, Sq], Precision.FP32)
    if ks[1] != Sq:
        c = context()
        _lib.check(c.lib.it_attention_cross_fwd(c.handle, c.stream(), _dtype_code(p), B, Sq, ks[1], H, D, q.data_ptr(),
                                                k.data_ptr(), v.data_ptr(), out.data_ptr(), out.lse.data_ptr()))
        return out
    raw.fwd_bshd(_dtype_code(p), B, Sq, H, D, causal, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                 out.lse.data_ptr())
    return out


def attention_backward(grad_output, q, k, v, o, causal=True):
    """(dQ, dK, dV) for attention(): every tensor is [batch, seq, heads, head_dim]; `o` is attention()'s
    result (with its `.lse`).  The layout-fused counterpart of attention_backward_recompute: the reference
    transposes the gradient in and the three gradients out (src/train/backward.rs:102,114-116)."""
    p = q.precision()
    B, S, H, D = q.shape()
    for t in (grad_output, k, v, o):
        assert t.precision() is p and t.shape() == [B, S, H, D], "shape or precision mismatch"
    assert o.lse is not None, "o must come from attention()"
    if S == 0 or B * H == 0:
        return Tensor.zeros([B, S, H, D], p), Tensor.zeros([B, S, H, D], p), Tensor.zeros([B, S, H, D], p)
    dq, dk, dv = Tensor.empty([B, S, H, D], p), Tensor.empty([B, S, H, D], p), Tensor.empty([B, S, H, D], p)
    code = _dtype_code(p)
    nbytes = raw.bwd_workspace_bytes(code, B, H, S, D)
    ws = _workspace(nbytes)
    raw.bwd_bshd(code, B, S, H, D, causal, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), grad_output.data_ptr(),
                 o.lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel())
    return dq, dk, dv


def attention_gqa(q, k, v, causal=True):
    """Grouped-query attention: q [batch, seq, heads, head_dim], k and v [batch, seq, kv_heads, head_dim] with
    kv_heads dividing heads.  Equal to attention(q, repeat_kv(k), repeat_kv(v), causal) of the reference
    (src/train/forward.rs:117-139; repeat_kv_gpu, src/ops/repeat_kv.rs:68-149) without the expanded copies:
    query head h reads K/V head h // (heads // kv_heads).  The result carries `.lse` for attention_gqa_backward."""
    p = q.precision()
    assert k.precision() is p and v.precision() is p
    assert len(q.shape()) == 4 and len(k.shape()) == 4 and len(v.shape()) == 4, "Q, K and V must be 4D"
    B, S, H, D = q.shape()
    assert k.shape() == v.shape(), "K and V must have the same shape"
    Hkv = k.shape()[2]
    assert k.shape() == [B, S, Hkv, D], "K/V must be [batch, seq, kv_heads, head_dim]"
    assert Hkv >= 1 and H % Hkv == 0, "num_heads must be divisible by num_kv_heads"   # src/ops/repeat_kv.rs:77-80
    out = Tensor.empty([B, S, H, D], p)
    out.lse = Tensor.empty([B, H, S], Precision.FP32)
    if B * S * H == 0:
        return out
    raw.fwd_gqa(_dtype_code(p), B, S, H, Hkv, D, causal, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                out.lse.data_ptr())
    return out


def rope(input, base=10000.0, position_offset=0):
    """Rotary position embedding of one [batch, seq, heads, head_dim] tensor (src/ops/rope.rs:22-75)."""
    assert len(input.shape()) == 4, "Input must be 4D [batch, seq_len, num_heads, head_dim]"
    B, S, H, D = input.shape()
    assert D % 2 == 0, "head_dim must be even for RoPE"
    out = Tensor.empty([B, S, H, D], input.precision())
    raw.rope_qk(_dtype_code(input.precision()), B, S, H, 0, D, base, position_offset, False, input.data_ptr(), None,
                out.data_ptr(), None)
    return out


def rope_qk(q, k, base=10000.0, position_offset=0, inverse=False):
    """rope(q) and rope(k) (src/train/forward.rs:111-112) as one launch; k may have fewer heads.  `inverse`
    gives the backward rotation (rope_backward, src/ops/backward/rope.rs)."""
    B, S, H, D = q.shape()
    Hkv = k.shape()[2]
    assert k.shape() == [B, S, Hkv, D] and k.precision() is q.precision() and D % 2 == 0
    qo, ko = Tensor.empty([B, S, H, D], q.precision()), Tensor.empty([B, S, Hkv, D], q.precision())
    raw.rope_qk(_dtype_code(q.precision()), B, S, H, Hkv, D, base, position_offset, inverse, q.data_ptr(), k.data_ptr(),
                qo.data_ptr(), ko.data_ptr())
    return qo, ko


def attention_gqa_backward(grad_output, q, k, v, o, causal=True, rope_base=None, position_offset=0):
    """(dQ, dK, dV) for attention_gqa(): dQ like q, dK and dV like k and v, i.e. already summed over the query
    heads of each group (the reference's repeat_kv_backward after its attention backward,
    src/train/backward.rs:102-122; src/ops/repeat_kv.rs:151-232).  With `rope_base`, q and k are the rotated
    tensors the forward attended over and dQ, dK come back as gradients of the un-rotated ones: the
    reference's two rope_backward passes (src/train/backward.rs:129,132) folded into this call."""
    p = q.precision()
    B, S, H, D = q.shape()
    Hkv = k.shape()[2]
    assert grad_output.shape() == [B, S, H, D] and o.shape() == [B, S, H, D]
    assert k.shape() == [B, S, Hkv, D] and v.shape() == [B, S, Hkv, D] and H % Hkv == 0
    assert o.lse is not None, "o must come from attention_gqa()"
    dq, dk, dv = Tensor.empty([B, S, H, D], p), Tensor.empty([B, S, Hkv, D], p), Tensor.empty([B, S, Hkv, D], p)
    if B * S * H == 0:
        return dq, dk, dv
    code = _dtype_code(p)
    nbytes = raw.bwd_workspace_bytes(code, B, H, S, D)
    ws = _workspace(nbytes)
    args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), grad_output.data_ptr(), o.lse.data_ptr(), dq.data_ptr(),
            dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel())
    if rope_base is None:
        raw.bwd_gqa(code, B, S, H, Hkv, D, causal, *args)
    else:
        raw.bwd_gqa_rope(code, B, S, H, Hkv, D, causal, rope_base, position_offset, *args)
    return dq, dk, dv


def attention_decode(q, k_cache, v_cache, kv_len):
    """Attention of one new token per sequence against a key/value cache: q [batch, heads, head_dim], caches
    [batch, max_len, kv_heads, head_dim] whose first `kv_len` positions are valid (the new token's key and value
    included).  Equals the last row of the causal attention the reference's generator recomputes from scratch for
    every token (src/inference/generator.rs:146-200).  The result carries `.lse` ([batch, heads])."""
    p = q.precision()
    assert k_cache.precision() is p and v_cache.precision() is p
    assert len(q.shape()) == 3 and len(k_cache.shape()) == 4 and k_cache.shape() == v_cache.shape()
    B, H, D = q.shape()
    Bc, max_len, Hkv, Dc = k_cache.shape()
    assert Bc == B and Dc == D and H % Hkv == 0 and 1 <= kv_len <= max_len
    out = Tensor.empty([B, H, D], p)
    out.lse = Tensor.empty([B, H], Precision.FP32)
    nbytes = raw.decode_workspace_bytes(B, H, D)
    ws = _workspace(nbytes)
    raw.decode(_dtype_code(p), B, H, Hkv, D, kv_len, max_len, q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
               out.data_ptr(), out.lse.data_ptr(), ws.data_ptr(), ws.numel())
    return out


def linear_forward(input, weight):
    """output = input @ weight.T (src/train/helpers.rs:48-53) for BF16 tensors: input [n, in], weight [out, in]."""
    assert input.precision() is Precision.BF16 and weight.precision() is Precision.BF16, "linear_forward takes BF16 tensors"
    n, k = input.shape()
    out_dim, k2 = weight.shape()
    assert k == k2, "inner dimensions must match"
    y = Tensor.empty([n, out_dim], Precision.BF16)
    raw.linear_fwd(n, k, out_dim, input.data_ptr(), weight.data_ptr(), y.data_ptr())
    return y


def qkv_rope_forward(x, w_qkv, heads, kv_heads, head_dim, rope_base=10000.0, position_offset=0, packed=False):
    """q_rope, k_rope, v from x [batch, seq, hidden] and the stacked weights [Wq; Wk; Wv] in one kernel: the three
    projections of src/train/forward.rs:101-103 and the two rope() calls of :111-112, written directly in the
    [batch, seq, heads, head_dim] layout attention_gqa reads.  rope_base None: no rotation.  packed=True returns ONE
    tensor [batch, seq, (heads + 2*kv_heads)*head_dim] (q_rope | k_rope | v per token) for attention_packed."""
    assert x.precision() is Precision.BF16 and w_qkv.precision() is Precision.BF16
    B, S, hidden = x.shape()
    assert w_qkv.shape() == [(heads + 2 * kv_heads) * head_dim, hidden], "w_qkv must be [Wq; Wk; Wv] stacked by rows"
    if packed:
        qkv = Tensor.empty([B, S, (heads + 2 * kv_heads) * head_dim], Precision.BF16)
        raw.qkv_rope_fwd(B, S, hidden, heads, kv_heads, head_dim, 0.0 if rope_base is None else rope_base, position_offset,
                         x.data_ptr(), w_qkv.data_ptr(), qkv.data_ptr(), None, None)
        return qkv
    q = Tensor.empty([B, S, heads, head_dim], Precision.BF16)
    k = Tensor.empty([B, S, kv_heads, head_dim], Precision.BF16)
    v = Tensor.empty([B, S, kv_heads, head_dim], Precision.BF16)
    raw.qkv_rope_fwd(B, S, hidden, heads, kv_heads, head_dim, 0.0 if rope_base is None else rope_base, position_offset,
                     x.data_ptr(), w_qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr())
    return q, k, v


def attention_packed(qkv, heads, kv_heads, head_dim, causal=True):
    """Grouped-query attention on the packed projection output [batch, seq, (heads + 2*kv_heads)*head_dim]
    (qkv_rope_forward(..., packed=True)).  Returns O [batch, seq, heads, head_dim] with `.lse`."""
    B, S, W = qkv.shape()
    assert qkv.precision() is Precision.BF16 and W == (heads + 2 * kv_heads) * head_dim
    out = Tensor.empty([B, S, heads, head_dim], Precision.BF16)
    out.lse = Tensor.empty([B, heads, S], Precision.FP32)
    raw.packed_fwd(B, S, heads, kv_heads, head_dim, causal, qkv.data_ptr(), out.data_ptr(), out.lse.data_ptr())
    return out


def attention_packed_backward(grad_output, qkv, o, heads, kv_heads, head_dim, causal=True, rope_base=None, position_offset=0):
    """Gradient of attention_packed with respect to the packed tensor, in the same layout (dq | dk | dv per token, dk and dv
    summed over each group, dq and dk rotated back when rope_base is given): ready to be the one `grad_output` of
    linear_backward for the stacked weights [Wq; Wk; Wv]."""
    B, S, W = qkv.shape()
    assert grad_output.shape() == [B, S, heads, head_dim] and o.lse is not None
    dqkv = Tensor.empty([B, S, W], Precision.BF16)
    nbytes = raw.bwd_workspace_bytes(_lib.IT_BF16, B, heads, S, head_dim)
    ws = _workspace(nbytes)
    raw.packed_bwd(B, S, heads, kv_heads, head_dim, causal, 0.0 if rope_base is None else rope_base, position_offset,
                   qkv.data_ptr(), o.data_ptr(), grad_output.data_ptr(), o.lse.data_ptr(), dqkv.data_ptr(), ws.data_ptr(), ws.numel())
    return dqkv


def linear_backward(grad_output, input, weight):
    """(grad_input, grad_weight) = (grad_output @ weight, grad_output.T @ input) (src/train/helpers.rs:61-76);
    grad_input BF16 [n, in], grad_weight FP32 [out, in] (the reference returns FP32 gradients)."""
    n, out_dim = grad_output.shape()
    k = input.shape()[1]
    assert input.shape() == [n, k] and weight.shape() == [out_dim, k]
    dx = Tensor.empty([n, k], Precision.BF16)
    dw = Tensor.empty([out_dim, k], Precision.FP32)
    raw.linear_bwd(n, k, out_dim, grad_output.data_ptr(), input.data_ptr(), weight.data_ptr(), dx.data_ptr(), dw.data_ptr())
    return dx, dw


def attention_backward_recompute(grad_output, q, k, v, o=None, lse=None, causal=True):
    """(dQ, dK, dV) on [batch, heads, seq, head_dim] (src/train/helpers.rs:120-193).

    The reference takes (grad_output, q, k, v) and is always causal.  Pass the forward's `o` and
    `lse` (flash_attention's result and its `.lse`) to skip the recomputation; without them the
    forward is run again here, which is what "recompute" means for the fused path."""
    p = q.precision()
    for t in (grad_output, k, v):
        assert t.precision() is p, "all tensors must have the same precision"
    B, H, S, D = q.shape()
    for t in (grad_output, k, v):
        assert t.shape() == [B, H, S, D], "shape mismatch"
    if S == 0 or B * H == 0:
        return Tensor.zeros([B, H, S, D], p), Tensor.zeros([B, H, S, D], p), Tensor.zeros([B, H, S, D], p)
    dq, dk, dv = Tensor.empty([B, H, S, D], p), Tensor.empty([B, H, S, D], p), Tensor.empty([B, H, S, D], p)
    if o is None or lse is None:
        o = flash_attention(q, k, v, causal)
        lse = o.lse
    code = _dtype_code(p)
    nbytes = raw.bwd_workspace_bytes(code, B, H, S, D)
    ws = _workspace(nbytes)
    raw.bwd(code, B, H, S, D, causal, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), grad_output.data_ptr(),
            lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel())
    return dq, dk, dv


class HostAttentionStep:
    """Forward + backward for tensors that live in page-locked HOST memory (it_host_step_* of the C ABI).

    The reference's tensors are unified memory, so its ops never copy; on a discrete GPU a caller with host data
    pays the host link both ways.  The library hides most of it: the (batch*head) slices are cut into `chunks`
    groups, and each group runs upload -> forward -> backward -> download on one of `n_streams` streams in rotation,
    so one group's upload, another's kernels and a third's download proceed at the same time on the two copy
    engines and the SMs.  The loop over the groups runs inside the library (one call per step), so groups can be
    small.  Device buffers, streams and events are allocated once, in the constructor."""

    def __init__(self, n_slices, S, D, precision=Precision.BF16, causal=True, chunks=4, n_streams=3):
        self.ctx = context()
        self.n_slices, self.S, self.D, self.precision = n_slices, S, D, precision
        chunks = max(1, min(chunks, n_slices))
        self.group = -(-n_slices // chunks)
        h = ctypes.c_void_p()
        _lib.check(self.ctx.lib.it_host_step_create(self.ctx.handle, _dtype_code(precision), self.group, S, D, int(causal),
                                                    max(1, min(n_streams, chunks, 4)), ctypes.byref(h)))
        self.handle = h

    def run(self, hq, hk, hv, hdo, ho, hdq, hdk, hdv, hlse=None, copies_only=False):
        """All arguments: pinned torch tensors [n_slices, S, D] (hlse [n_slices, S], optional).  Enqueues the whole step;
        torch's current stream continues only after every group's download has finished.  Nothing is waited for
        here: drain the stream and check the device status (CommandBatch.sync(), context().poll_status()) before
        reading the host tensors.  copies_only=True enqueues the same uploads and downloads on the same streams
        without the kernels (what the host link alone costs)."""
        for t in (hq, hk, hv, hdo, ho, hdq, hdk, hdv):
            assert t.is_pinned() and t.numel() == self.n_slices * self.S * self.D
        _lib.check(self.ctx.lib.it_host_step_run(self.handle, self.ctx.stream(), self.n_slices, hq.data_ptr(), hk.data_ptr(),
                                                 hv.data_ptr(), hdo.data_ptr(), ho.data_ptr(),
                                                 None if hlse is None else hlse.data_ptr(), hdq.data_ptr(), hdk.data_ptr(),
                                                 hdv.data_ptr(), int(copies_only)))

    def __del__(self):
        try:
            self.ctx.lib.it_host_step_destroy(self.handle)
        except Exception:
            pass
