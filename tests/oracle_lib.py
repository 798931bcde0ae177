"""ctypes access to the CPU oracle (oracle/liboracle_attention.so) and, where it was built, to the
reference project's own shader sources compiled as C++ (oracle/_ref/libref_attention.so).

Test infrastructure: imported by tests/, __graft_entry__.smoke() and bench.py's CPU legs only."""
import ctypes
import os
import subprocess
import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ODIR = os.path.join(_ROOT, "oracle")
_f32p = ctypes.POINTER(ctypes.c_float)
_lib = None
_ref = None


def build():
    subprocess.run(["make", "-C", _ODIR, "-s"], check=True)


def oracle():
    global _lib
    if _lib is None:
        path = os.path.join(_ODIR, "liboracle_attention.so")
        if not os.path.exists(path):
            build()
        _lib = ctypes.CDLL(path)
        _lib.oracle_attention_fwd.argtypes = [ctypes.c_int] * 6 + [_f32p] * 5 + [ctypes.c_int] * 2
        _lib.oracle_attention_bwd.argtypes = [ctypes.c_int] * 5 + [_f32p] * 7 + [ctypes.c_int] * 2
        _lib.oracle_f32_to_bf16.argtypes = [_f32p, ctypes.POINTER(ctypes.c_uint16), ctypes.c_int64]
    return _lib


def reference():
    """The compiled reference shaders, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None:
        path = os.path.join(_ODIR, "_ref", "libref_attention.so")
        if not os.path.exists(path):
            return None
        _ref = ctypes.CDLL(path)
        _ref.ref_attention_fwd.argtypes = [ctypes.c_int] * 6 + [_f32p] * 4
        _ref.ref_attention_bwd.argtypes = [ctypes.c_int] * 4 + [_f32p] * 7
    return _ref


def _p(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fwd(q, k, v, causal=True, kernel=0, want_lse=True, bh_range=None):
    """q,k,v: [B,H,S,D] fp32.  Returns (O, LSE)."""
    q, k, v = _c(q), _c(k), _c(v)
    B, H, S, D = q.shape
    o = np.zeros_like(q)
    lse = np.zeros((B, H, S), np.float32) if want_lse else None
    b0, b1 = bh_range if bh_range else (0, -1)
    rc = oracle().oracle_attention_fwd(B, H, S, D, int(causal), kernel, _p(q), _p(k), _p(v), _p(o), _p(lse), b0, b1)
    if rc != 0:
        raise ValueError("oracle rejected the arguments")
    return o, lse


def bwd(q, k, v, d_o, causal=True, bh_range=None):
    """Returns (dQ, dK, dV) following the reference's composed backward."""
    q, k, v, d_o = _c(q), _c(k), _c(v), _c(d_o)
    B, H, S, D = q.shape
    dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
    b0, b1 = bh_range if bh_range else (0, -1)
    rc = oracle().oracle_attention_bwd(B, H, S, D, int(causal), _p(q), _p(k), _p(v), _p(d_o), _p(dq), _p(dk), _p(dv), b0, b1)
    if rc != 0:
        raise ValueError("oracle rejected the arguments")
    return dq, dk, dv


def f32_to_bf16_bits(x):
    x = _c(x)
    out = np.zeros(x.shape, np.uint16)
    oracle().oracle_f32_to_bf16(_p(x), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), x.size)
    return out


def ref_fwd(q, k, v, causal=True, kernel=0):
    r = reference()
    q, k, v = _c(q), _c(k), _c(v)
    B, H, S, D = q.shape
    o = np.zeros_like(q)
    rc = r.ref_attention_fwd(B, H, S, D, int(causal), kernel, _p(q), _p(k), _p(v), _p(o))
    if rc != 0:
        raise ValueError("shape outside what the reference shaders can run")
    return o


def ref_bwd(q, k, v, d_o):
    r = reference()
    q, k, v, d_o = _c(q), _c(k), _c(v), _c(d_o)
    B, H, S, D = q.shape
    dq, dk, dv = np.zeros_like(q), np.zeros_like(q), np.zeros_like(q)
    r.ref_attention_bwd(B, H, S, D, _p(q), _p(k), _p(v), _p(d_o), _p(dq), _p(dk), _p(dv))
    return dq, dk, dv


def gqa_expand(x, heads):
    """repeat_kv of the reference (src/shaders/repeat_kv.metal:19-47): [B,S,Hkv,D] -> [B,S,H,D], output head h
    reads K/V head h // (H // Hkv)."""
    return np.repeat(x, heads // x.shape[2], axis=2)


def gqa_fwd(q, k, v, causal=True):
    """Oracle for grouped-query attention on [B,S,H,D] / [B,S,Hkv,D]: the reference's composition
    repeat_kv -> transpose -> attention -> transpose (src/train/forward.rs:117-141).  Returns O [B,S,H,D], LSE [B,H,S]."""
    H = q.shape[2]
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    o, lse = fwd(t(q), t(gqa_expand(k, H)), t(gqa_expand(v, H)), causal)
    return np.ascontiguousarray(o.transpose(0, 2, 1, 3)), lse


def gqa_bwd(q, k, v, d_o, causal=True):
    """Oracle backward for the same composition, ending in repeat_kv_backward (src/shaders/repeat_kv.metal:49-88:
    the expanded gradients of a group summed in head order).  Returns dQ [B,S,H,D], dK, dV [B,S,Hkv,D]."""
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    dq, dk, dv = bwd(t(q), t(gqa_expand(k, H)), t(gqa_expand(v, H)), t(d_o), causal)
    def fold(g):   # [B,H,S,D] -> [B,S,Hkv,D]
        acc = np.zeros((B, Hkv, S, D), np.float32)
        g5 = g.reshape(B, Hkv, H // Hkv, S, D)
        for r in range(H // Hkv):
            acc += g5[:, :, r]
        return np.ascontiguousarray(acc.transpose(0, 2, 1, 3))
    return np.ascontiguousarray(dq.transpose(0, 2, 1, 3)), fold(dk), fold(dv)


def rope(x, base=10000.0, position_offset=0, inverse=False):
    """CPU restatement of rope_f32 / rope_backward_f32 (src/shaders/rope.metal:22-61,
    src/shaders/backward/rope.metal:25-62) on [B,S,H,D], fp32 arithmetic: theta_i = 1 / base^(2i/D),
    angle = float(position) * theta_i.  theta is rounded once from double, as the library's table is."""
    x = np.asarray(x, np.float32)
    B, S, H, D = x.shape
    i = np.arange(D // 2)
    theta = (1.0 / np.power(np.float64(base), (2.0 * i) / D)).astype(np.float32)
    pos = (np.arange(S) + position_offset).astype(np.float32)
    ang = (pos[:, None] * theta[None, :]).astype(np.float32)          # [S, D/2], the fp32 product
    c, s = np.cos(ang).astype(np.float32)[None, :, None, :], np.sin(ang).astype(np.float32)[None, :, None, :]
    if inverse:
        s = -s
    x0, x1 = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = x0 * c - x1 * s
    out[..., 1::2] = x0 * s + x1 * c
    return out
