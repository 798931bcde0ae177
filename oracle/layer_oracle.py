"""CPU restatements (numpy) of the reference's steps either side of attention: repeat_kv and its backward,
rotary position embedding and its backward.  TEST INFRASTRUCTURE ONLY, like attention_oracle.cpp: imported by
tests/ (through tests/oracle_lib.py); nothing in the product loads it.

Each function cites the reference shader it follows (paths relative to the reference project's root).  They take the
attention oracle's forward / backward as arguments so that this file has no dependency of its own.
Parity status: repeat_kv is a copy / an in-order sum and is exact; the rotary angles use Metal's pow, cos and sin in
the reference, which cannot run here, so bit-level parity of rope is unpinned (checked against the reference's unit-test
properties, src/ops/rope.rs:128-250, and to 1e-5 against the library)."""
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
