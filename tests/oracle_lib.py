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
    """Builds the oracle; the reference's shaders too when a checkout is at $IRONTENSOR_REF_ROOT or in a
    "reference" directory beside this repository."""
    ref = os.environ.get("IRONTENSOR_REF_ROOT") or os.path.join(os.path.dirname(_ROOT), "reference")
    cmd = ["make", "-C", _ODIR, "-s"]
    if os.path.isdir(os.path.join(ref, "src", "shaders")):
        cmd.append("REF_ROOT=" + ref)
    subprocess.run(cmd, check=True)


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
        _lib.oracle_rope.argtypes = [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, _f32p, _f32p]
        _lib.oracle_repeat_kv.argtypes = [ctypes.c_int] * 6 + [_f32p, _f32p]
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
        _ref.ref_rope.argtypes = [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, _f32p, _f32p]
        _ref.ref_repeat_kv.argtypes = [ctypes.c_int] * 6 + [_f32p, _f32p]
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


def cross_fwd(q, k, v):
    """Non-causal attention of q [B,H,Sq,D] over k, v [B,H,Skv,D] with Sq != Skv, which the reference's attention()
    accepts (src/ops/attention.rs:304,349-352).  Without a mask every query row is independent of the other query
    rows, so the oracle's equal-length forward is run on chunks of at most Skv query rows padded to Skv with zeros."""
    q, k, v = _c(q), _c(k), _c(v)
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    o = np.zeros_like(q)
    lse = np.zeros((B, H, Sq), np.float32)
    for r0 in range(0, Sq, Skv):
        n = min(Skv, Sq - r0)
        qp = np.zeros((B, H, Skv, D), np.float32)
        qp[:, :, :n] = q[:, :, r0:r0 + n]
        oc, lc = fwd(qp, k, v, causal=False)
        o[:, :, r0:r0 + n] = oc[:, :, :n]
        lse[:, :, r0:r0 + n] = lc[:, :, :n]
    return o, lse


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


def _rope_call(fn, x, base, position_offset, inverse):
    x = _c(x)
    B, S, H, D = x.shape
    out = np.zeros_like(x)
    if fn(B, S, H, D, float(base), int(position_offset), int(bool(inverse)), _p(x), _p(out)) != 0:
        raise ValueError("head_dim must be even")
    return out


def rope(x, base=10000.0, position_offset=0, inverse=False):
    """Rotary embedding of [B,S,H,D] (inverse: the backward rotation) by the C++ oracle."""
    return _rope_call(oracle().oracle_rope, x, base, position_offset, inverse)


def ref_rope(x, base=10000.0, position_offset=0, inverse=False):
    """The same through the reference's own rope.metal / backward/rope.metal compiled as C++."""
    return _rope_call(reference().ref_rope, x, base, position_offset, inverse)


def _repeat_call(fn, x, heads, kv_heads, backward):
    x = _c(x)
    B, S, _, D = x.shape
    out = np.zeros((B, S, kv_heads if backward else heads, D), np.float32)
    if fn(B, S, heads, kv_heads, D, int(backward), _p(x), _p(out)) != 0:
        raise ValueError("num_heads must be divisible by num_kv_heads")
    return out


def repeat_kv(x, heads, backward=False, kv_heads=None):
    """repeat_kv ([B,S,Hkv,D] -> [B,S,H,D]) or its backward ([B,S,H,D] -> [B,S,Hkv,D]) by the C++ oracle."""
    return _repeat_call(oracle().oracle_repeat_kv, x, heads, kv_heads if backward else x.shape[2], backward)


def ref_repeat_kv(x, heads, backward=False, kv_heads=None):
    return _repeat_call(reference().ref_repeat_kv, x, heads, kv_heads if backward else x.shape[2], backward)


# Grouped-query attention as the reference composes it is restated in oracle/layer_oracle.py.
import importlib.util as _ilu
_spec = _ilu.spec_from_file_location("layer_oracle", os.path.join(_ODIR, "layer_oracle.py"))
_layer = _ilu.module_from_spec(_spec)
_spec.loader.exec_module(_layer)
gqa_expand = _layer.gqa_expand


def gqa_fwd(q, k, v, causal=True):
    return _layer.gqa_fwd(fwd, q, k, v, causal)


def gqa_bwd(q, k, v, d_o, causal=True):
    return _layer.gqa_bwd(bwd, q, k, v, d_o, causal)
