"""Grouped-query attention as the reference composes it around its attention op (numpy): repeat_kv, attention,
repeat_kv_backward.  TEST INFRASTRUCTURE ONLY, like attention_oracle.cpp: imported by tests/ (through
tests/oracle_lib.py); nothing in the product loads it.

Each function cites the reference shader it follows (paths relative to the reference project's root).  They take the
attention oracle's forward / backward as arguments so that this file has no dependency of its own.
Parity status: pinned.  repeat_kv is a copy and its backward an in-order sum; tests/test_oracle.py holds gqa_expand and
the fold below bit-for-bit to the reference's own repeat_kv shaders compiled as C++ (oracle/ref_shim) and to the
golden vectors made from them.  The rotary embedding is restated in attention_oracle.cpp (oracle_rope)."""
import numpy as np


def gqa_expand(x, heads):
    """repeat_kv of the reference (src/shaders/repeat_kv.metal:19-47): [B,S,Hkv,D] -> [B,S,H,D], output head h
    reads K/V head h // (H // Hkv)."""
    return np.repeat(x, heads // x.shape[2], axis=2)


def gqa_fwd(fwd, q, k, v, causal=True):
    """Oracle for grouped-query attention on [B,S,H,D] / [B,S,Hkv,D]: the reference's composition
    repeat_kv -> transpose -> attention -> transpose (src/train/forward.rs:117-141).  Returns O [B,S,H,D], LSE [B,H,S]."""
    H = q.shape[2]
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    o, lse = fwd(t(q), t(gqa_expand(k, H)), t(gqa_expand(v, H)), causal)
    return np.ascontiguousarray(o.transpose(0, 2, 1, 3)), lse


def gqa_bwd(bwd, q, k, v, d_o, causal=True):
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
