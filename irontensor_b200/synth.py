"""Seeded synthetic attention inputs.

A counter-based generator: element `i` of tensor `tensor_id` under `seed` depends only on
(seed, tensor_id, i), so any (batch*head) shard can be produced on any rank, or on the CPU, and be
identical everywhere.  splitmix64 of the counter gives two 24-bit uniforms, Box-Muller turns them
into one N(0,1) sample.  bf16 values are produced with the reference's rounding rule
(round-to-nearest-even on the upper 16 bits, src/precision.rs:24-29 of the reference project).
"""
import numpy as np

TENSOR_Q, TENSOR_K, TENSOR_V, TENSOR_DO = 0, 1, 2, 3
BASE_SEED = 0x1A7E5EED

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def normal(seed, tensor_id, start, count, scale=1.0):
    """`count` fp32 N(0,1)*scale samples for linear indices [start, start+count)."""
    with np.errstate(over="ignore"):
        idx = np.arange(start, start + count, dtype=np.uint64)
        key = _splitmix64(np.uint64(seed) * np.uint64(4) + np.uint64(tensor_id))
        bits = _splitmix64(idx ^ key)
    u1 = ((bits >> np.uint64(40)).astype(np.float64) + 1.0) / 16777216.0      # (0, 1]
    u2 = ((bits >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) / 16777216.0
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * scale).astype(np.float32)


def f32_to_bf16_bits(x):
    """fp32 array -> uint16 bf16 bit patterns (RNE, no NaN special case)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rnd = ((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((bits + rnd) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x):
    """fp32 array rounded to the nearest bf16 value, returned as fp32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def attention_inputs(seed, B, H, S, D, bf16=False, qk_scale=1.0, with_do=True, bh_begin=0, bh_end=None):
    """Q, K, V (and dO) of shape [bh_end-bh_begin, S, D] as fp32 (bf16-representable if `bf16`)."""
    if bh_end is None:
        bh_end = B * H
    n = (bh_end - bh_begin) * S * D
    start = bh_begin * S * D
    out = []
    for tid, sc in ((TENSOR_Q, qk_scale), (TENSOR_K, qk_scale), (TENSOR_V, 1.0), (TENSOR_DO, 1.0)):
        if tid == TENSOR_DO and not with_do:
            break
        t = normal(seed, tid, start, n, sc)
        if bf16:
            t = round_bf16(t)
        out.append(t.reshape(bh_end - bh_begin, S, D))
    return out
