"""CPU tests of the oracle itself: against the golden vectors produced by the reference's own
shader sources, against those sources directly where oracle/_ref was built, against an independent
fp64 formulation and finite differences, and of the bf16 rounding rule."""
import math
import os

import numpy as np
import pytest

import oracle_lib as ol
from irontensor_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def seeded(seed, B, H, S, D, with_do=True):
    return [t.reshape(B, H, S, D) for t in synth.attention_inputs(seed, B, H, S, D, with_do=with_do)]


# ---------------------------------------------------------------- golden vectors (bit-exact)
def test_golden_flash_kat1():
    g = gold("flash_kat1")
    assert np.array_equal(ol.fwd(g["q"], g["k"], g["v"], True)[0], g["o_causal"])
    assert np.array_equal(ol.fwd(g["q"], g["k"], g["v"], False)[0], g["o_full"])


def test_golden_flash_kat2():
    g = gold("flash_kat2")
    assert np.array_equal(ol.fwd(g["q"], g["k"], g["v"], True)[0], g["o_causal"])


def test_golden_backward_kat():
    g = gold("bwd_kat")
    dq, dk, dv = ol.bwd(g["q"], g["k"], g["v"], g["d_o"])
    assert np.array_equal(dq, g["dq"]) and np.array_equal(dk, g["dk"]) and np.array_equal(dv, g["dv"])
    assert np.array_equal(ol.fwd(g["q"], g["k"], g["v"], True)[0], g["o_causal"])


def test_golden_tiled_kernel_seeded():
    g = gold("tiled_seeded")
    q, k, v = seeded(int(g["seed"]), 1, 2, 300, 64, with_do=False)
    assert np.array_equal(ol.fwd(q, k, v, True)[0], g["o_causal"])
    assert np.array_equal(ol.fwd(q, k, v, False)[0], g["o_full"])


def test_golden_decode_prefix_seeded():
    g = gold("decode_seeded")
    q, k, v = seeded(int(g["seed"]), 1, 4, 119, 64, with_do=False)
    assert np.array_equal(ol.fwd(q, k, v, True)[0], g["o_causal"])


def test_golden_backward_seeded():
    g = gold("bwd_seeded")
    q, k, v, d_o = seeded(int(g["seed"]), 1, 2, 40, 16)
    for got, name in zip(ol.bwd(q, k, v, d_o), ("dq", "dk", "dv")):
        assert np.array_equal(got, g[name]), name


# ---------------------------------------------------------------- the reference's sources, live
needs_ref = pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (no reference tree)")


@needs_ref
@pytest.mark.parametrize("shape,kernel", [((2, 4, 32, 16), 0), ((1, 2, 40, 16), 2), ((1, 2, 257, 64), 0),
                                          ((2, 2, 33, 128), 1), ((1, 4, 20, 64), 0), ((1, 1, 256, 64), 0)])
@pytest.mark.parametrize("causal", [True, False])
def test_forward_equals_reference_sources(shape, kernel, causal):
    q, k, v = seeded(21, *shape, with_do=False)
    assert np.array_equal(ol.fwd(q, k, v, causal, kernel)[0], ol.ref_fwd(q, k, v, causal, kernel))


@needs_ref
@pytest.mark.parametrize("shape", [(2, 4, 16, 8), (1, 2, 40, 16), (1, 1, 130, 32)])
def test_backward_equals_reference_sources(shape):
    q, k, v, d_o = seeded(22, *shape)
    for a, b in zip(ol.bwd(q, k, v, d_o), ol.ref_bwd(q, k, v, d_o)):
        assert np.array_equal(a, b)


@needs_ref
def test_backward_equals_reference_sources_threadgroup_softmax():
    # S >= 256 makes the reference pick its 256-lane softmax kernels (src/ops/softmax.rs:196).
    q, k, v, d_o = seeded(23, 1, 1, 256, 16)
    for a, b in zip(ol.bwd(q, k, v, d_o), ol.ref_bwd(q, k, v, d_o)):
        assert np.array_equal(a, b)


# ---------------------------------------------------------------- independent math
def sdpa_f64(q, k, v, d_o, causal):
    q, k, v, d_o = (x.astype(np.float64) for x in (q, k, v, d_o))
    S, D = q.shape[-2:]
    s = q @ np.swapaxes(k, -1, -2) / np.sqrt(D)
    if causal:
        s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    p = e / l
    o = p @ v
    lse = (m + np.log(l))[..., 0]
    dv = np.swapaxes(p, -1, -2) @ d_o
    dp = d_o @ np.swapaxes(v, -1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True))
    dq = ds @ k / np.sqrt(D)
    dk = np.swapaxes(ds, -1, -2) @ q / np.sqrt(D)
    return o, lse, dq, dk, dv


@pytest.mark.parametrize("shape", [(1, 2, 50, 24), (2, 2, 300, 64), (1, 1, 64, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_oracle_matches_fp64_math(shape, causal):
    q, k, v, d_o = seeded(31, *shape)
    o, lse = ol.fwd(q, k, v, causal)
    dq, dk, dv = ol.bwd(q, k, v, d_o, causal)
    ro, rlse, rdq, rdk, rdv = sdpa_f64(q, k, v, d_o, causal)
    assert np.abs(o - ro).max() < 2e-6
    assert np.abs(lse - rlse).max() < 5e-6
    for a, b in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert np.abs(a - b).max() < 2e-5


def test_small_and_tiled_forward_agree():
    q, k, v = seeded(32, 1, 2, 200, 64, with_do=False)
    o1, l1 = ol.fwd(q, k, v, True, kernel=1)
    o2, l2 = ol.fwd(q, k, v, True, kernel=2)
    assert np.abs(o1 - o2).max() < 1e-6 and np.abs(l1 - l2).max() < 2e-6


def test_backward_against_finite_differences():
    # d/dx of L = sum(O * dO) by central differences in fp64 on a tiny case.
    q, k, v, d_o = seeded(33, 1, 1, 6, 4)
    _, _, rdq, rdk, rdv = sdpa_f64(q, k, v, d_o, True)
    dq, dk, dv = ol.bwd(q, k, v, d_o, True)
    eps = 1e-5

    def loss(qq, kk, vv):
        return (sdpa_f64(qq, kk, vv, d_o, True)[0] * d_o).sum()

    for name, got in (("q", dq), ("k", dk), ("v", dv)):
        base = {"q": q.astype(np.float64), "k": k.astype(np.float64), "v": v.astype(np.float64)}
        num = np.zeros_like(base[name])
        it = np.nditer(num, flags=["multi_index"])
        for _ in it:
            idx = it.multi_index
            hi = {n: a.copy() for n, a in base.items()}
            lo = {n: a.copy() for n, a in base.items()}
            hi[name][idx] += eps
            lo[name][idx] -= eps
            num[idx] = (loss(hi["q"], hi["k"], hi["v"]) - loss(lo["q"], lo["k"], lo["v"])) / (2 * eps)
        assert np.abs(got - num).max() < 1e-4, name


def test_sequence_zero_and_bad_head_dim():
    z = np.zeros((2, 2, 0, 8), np.float32)
    o, lse = ol.fwd(z, z, z)
    assert o.shape == (2, 2, 0, 8)
    big = np.zeros((1, 1, 4, 129), np.float32)
    with pytest.raises(ValueError):
        ol.fwd(big, big, big)


# ---------------------------------------------------------------- bf16 rule and the generator
def test_bf16_rounding_rule():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.1415927, 1e-40, 65504.0, np.inf, -np.inf], np.float32)
    bits = ol.f32_to_bf16_bits(x)
    assert np.array_equal(bits, synth.f32_to_bf16_bits(x))
    # ties go to even: 1.00390625 = 0x3F808000 -> 0x3F80 ; 1.01171875 = 0x3F818000 -> 0x3F82
    assert bits[1] == 0x3F80 and bits[2] == 0x3F82
    assert bits[7] == 0x7F80 and bits[8] == 0xFF80
    r = synth.bf16_bits_to_f32(bits)
    assert np.all(np.abs(r[:5] - x[:5]) <= np.abs(x[:5]) * 2.0 ** -8)
    rng = np.random.default_rng(0)
    y = rng.standard_normal(100000).astype(np.float32)
    assert np.array_equal(ol.f32_to_bf16_bits(y), synth.f32_to_bf16_bits(y))
    import torch
    assert np.array_equal(synth.round_bf16(y), torch.from_numpy(y).to(torch.bfloat16).float().numpy())


def test_generator_is_counter_based():
    full = synth.attention_inputs(5, 2, 3, 16, 8)
    part = synth.attention_inputs(5, 2, 3, 16, 8, bh_begin=2, bh_end=5)
    for a, b in zip(full, part):
        assert np.array_equal(a[2:5], b)
    q = full[0]
    assert abs(q.mean()) < 0.1 and abs(q.std() - 1.0) < 0.1
    assert not np.array_equal(full[0], full[1])
    h = synth.attention_inputs(5, 2, 3, 16, 8, bf16=True, qk_scale=0.5)
    assert np.array_equal(h[0], synth.round_bf16(h[0]))


def test_rope_oracle_against_reference_unit_values():
    """The reference's own checks for rope (src/ops/rope.rs tests): position 0 is the identity, the rotation keeps
    the norm of every pair, a quarter turn maps (1, 0) to (0, 1), and backward(forward(x)) = x."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 7, 3, 8)).astype(np.float32)
    y = ol.rope(x)
    assert np.array_equal(y[:, 0], x[:, 0])                                    # position 0: angle 0
    n_in = x[..., 0::2] ** 2 + x[..., 1::2] ** 2
    n_out = y[..., 0::2] ** 2 + y[..., 1::2] ** 2
    assert np.abs(n_in - n_out).max() < 1e-5
    assert np.abs(ol.rope(y, inverse=True) - x).max() < 1e-5
    # pair 0 has theta = 1: at position p the angle is p radians
    e = np.zeros((1, 3, 1, 4), np.float32)
    e[..., 0] = 1.0
    r = ol.rope(e)
    for p in range(3):
        assert abs(r[0, p, 0, 0] - math.cos(p)) < 1e-6 and abs(r[0, p, 0, 1] - math.sin(p)) < 1e-6
    # position offset shifts the angle
    assert np.allclose(ol.rope(e, position_offset=2)[0, 0, 0, :2], [math.cos(2), math.sin(2)], atol=1e-6)


# ---------------------------------------------------------------- rotary embedding and repeat_kv: pinned
def test_golden_rope_vectors():
    """oracle_rope against the outputs of the reference's rope_f32 / rope_backward_f32 (compiled as C++) on the inputs
    of the reference's own tests (src/ops/rope.rs:128-250) and at positions near 8192: bit for bit, since both call
    the same libm powf, cosf and sinf in the same order."""
    g = gold("rope_kat")
    assert np.array_equal(ol.rope(g["simple_in"]), g["simple_out"])
    assert np.array_equal(ol.rope(g["zero_in"]), g["zero_out"])
    assert np.array_equal(g["zero_out"], g["zero_in"])                       # test_rope_position_zero
    assert np.array_equal(ol.rope(g["larger_in"]), g["larger_out"])
    assert np.array_equal(ol.rope(g["larger_out"], inverse=True), g["larger_back"])
    assert np.abs(g["larger_back"] - g["larger_in"]).max() < 1e-6            # backward undoes forward
    assert np.array_equal(ol.rope(g["offset_in"], position_offset=10), g["offset_out"])
    assert np.array_equal(ol.rope(g["long_in"], position_offset=8188), g["long_out"])


def test_golden_repeat_kv_vectors():
    """oracle_repeat_kv and the numpy forms the grouped-query oracle uses (gqa_expand, the in-order fold) against the
    outputs of the reference's repeat_kv_f32 / repeat_kv_backward_f32 on its own test inputs
    (src/ops/repeat_kv.rs:308-440): bit for bit."""
    g = gold("repeat_kv_kat")
    assert np.array_equal(ol.repeat_kv(g["simple_in"], 8), g["simple_out"])
    assert np.array_equal(ol.gqa_expand(g["simple_in"], 8), g["simple_out"])
    assert np.array_equal(ol.repeat_kv(g["backward_in"], 8, backward=True, kv_heads=2), g["backward_out"])
    assert np.array_equal(ol.repeat_kv(g["norepeat_in"], 4), g["norepeat_out"])
    assert np.array_equal(g["norepeat_out"], g["norepeat_in"])
    mid = ol.repeat_kv(g["roundtrip_in"], 4)
    assert np.array_equal(mid, g["roundtrip_mid"])
    assert np.array_equal(ol.repeat_kv(mid, 4, backward=True, kv_heads=2), g["roundtrip_out"])
    assert np.array_equal(g["roundtrip_out"], 2 * g["roundtrip_in"])          # each head was repeated twice


def test_gqa_fold_equals_repeat_kv_backward():
    """The group sum inside the grouped-query oracle (oracle/layer_oracle.py:gqa_bwd) is the reference's
    repeat_kv_backward: same summation order, so equal bits on random data."""
    rng = np.random.default_rng(9)
    B, S, H, Hkv, D = 2, 5, 6, 2, 8
    g = rng.standard_normal((B, S, H, D)).astype(np.float32)
    want = ol.repeat_kv(g, H, backward=True, kv_heads=Hkv)
    acc = np.zeros((B, S, Hkv, D), np.float32)
    g5 = g.reshape(B, S, Hkv, H // Hkv, D)
    for r in range(H // Hkv):
        acc += g5[:, :, :, r]
    assert np.array_equal(acc, want)


@pytest.mark.skipif(ol.reference() is None, reason="oracle/_ref not built (needs the reference tree)")
def test_rope_and_repeat_kv_equal_the_compiled_reference_shaders():
    rng = np.random.default_rng(21)
    for (B, S, H, D, off) in [(1, 3, 2, 4, 0), (2, 33, 3, 64, 7), (1, 17, 2, 128, 8000), (1, 5, 1, 2, 0)]:
        x = rng.standard_normal((B, S, H, D)).astype(np.float32)
        for base in (10000.0, 500000.0):
            assert np.array_equal(ol.rope(x, base, off), ol.ref_rope(x, base, off))
            assert np.array_equal(ol.rope(x, base, off, inverse=True), ol.ref_rope(x, base, off, inverse=True))
    for (B, S, H, Hkv, D) in [(1, 2, 4, 1, 8), (2, 3, 6, 3, 5), (1, 4, 8, 8, 16)]:
        x = rng.standard_normal((B, S, Hkv, D)).astype(np.float32)
        assert np.array_equal(ol.repeat_kv(x, H), ol.ref_repeat_kv(x, H))
        gx = rng.standard_normal((B, S, H, D)).astype(np.float32)
        assert np.array_equal(ol.repeat_kv(gx, H, backward=True, kv_heads=Hkv),
                              ol.ref_repeat_kv(gx, H, backward=True, kv_heads=Hkv))
