"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the golden
vectors produced by the reference's own shader sources.

Tolerances
  fp32 tensors : max-abs <= 1e-4 on O, LSE, dQ, dK, dV (as stated for the path).
  bf16 tensors : max-abs <= 2e-2 against the fp32 oracle (as stated for the path); LSE, which stays fp32, 1e-4.
                 Relative L2: the stated 1e-3 is unattainable for a result STORED in bf16 -- rounding the oracle's own
                 output to bf16 gives 1.48e-3 for a uniform mantissa ((2^-8/sqrt(3))/sqrt(7/3)), 1.5e-3..1.7e-3 on these
                 data (gpu_util.err_stats returns it as `floor`).  On top of the floor the kernels add what every bf16
                 tensor-core attention adds: P and dS are rounded to bf16 (2^-9 relative) before their MMAs, and dS
                 carries P's rounding as well.  The bounds are per tensor, about 10 % above the worst value measured
                 over every bf16 case of this file (BF16_REL_L2), so that a regression of any one tensor shows.
                 With IT_ERR_STATS_FILE set, the worst figures of the run are written there as JSON.
"""
import ctypes
import math
import os

import numpy as np
import pytest

import gpu_util as gu
import oracle_lib as ol
from irontensor_b200 import _lib, raw, synth

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
F32_TOL = 1e-4
BF16_MAX_ABS = 2e-2
# raw relative-L2 bound per tensor (measured worst: O 2.3e-3, dV 2.4e-3, dQ and dK 3.1e-3)
BF16_REL_L2 = {"O": 2.5e-3, "dV": 2.6e-3, "dQ": 3.4e-3, "dK": 3.4e-3}
_worst = {}


def seeded(seed, B, H, S, D, bf16=False, qk_scale=1.0):
    return [t.reshape(B, H, S, D) for t in synth.attention_inputs(seed, B, H, S, D, bf16=bf16, qk_scale=qk_scale)]


def check_f32(got, want, name):
    err = float(np.abs(np.asarray(got, np.float64) - want).max())
    assert not np.isnan(got).any(), f"{name}: NaN in output"
    assert err <= F32_TOL, f"{name}: max-abs {err:.3e} > {F32_TOL}"


def check_bf16(got, want, name, rel_scale=1.0):
    """`name` ends in the tensor's kind (O, dQ, dK, dV), which selects the relative-L2 bound."""
    assert not np.isnan(got).any(), f"{name}: NaN in output"
    kind = name.split()[-1]
    mx, rel, floor = gu.err_stats(got, want)
    own = math.sqrt(max(rel * rel - floor * floor, 0.0))
    w = _worst.setdefault(kind, {"max_abs": 0.0, "rel_l2": 0.0, "rel_l2_beyond_floor": 0.0})
    w["max_abs"], w["rel_l2"], w["rel_l2_beyond_floor"] = max(w["max_abs"], mx), max(w["rel_l2"], rel), max(w["rel_l2_beyond_floor"], own)
    if os.environ.get("IT_ERR_STATS_FILE"):
        import json
        with open(os.environ["IT_ERR_STATS_FILE"], "w") as f:
            json.dump(_worst, f)
    assert mx <= BF16_MAX_ABS, f"{name}: max-abs {mx:.3e} > {BF16_MAX_ABS}"
    bound = BF16_REL_L2[kind] * rel_scale
    assert rel <= bound, f"{name}: rel-L2 {rel:.3e} > {bound:.1e} (bf16 storage floor {floor:.3e}, beyond it {own:.3e})"


# ---------------------------------------------------------------- hardware self tests
@pytest.mark.parametrize("variant", [0, 1, 2, 3])
def test_umma_operand_paths(it_ctx, variant):
    import torch
    rng = np.random.default_rng(variant)
    a = synth.round_bf16(rng.standard_normal((128, 128)).astype(np.float32))
    b = synth.round_bf16(rng.standard_normal((128, 128)).astype(np.float32))
    ta, tb = gu.to_dev(a, True), gu.to_dev(b, True)
    out = torch.full((128, 128), float("nan"), device="cuda")
    _lib.check(it_ctx.lib.it_selftest_umma(it_ctx.handle, it_ctx.stream(), variant, ta.data_ptr(), tb.data_ptr(),
                                           out.data_ptr()))
    assert it_ctx.poll_status() == 0
    want = a.astype(np.float64) @ (b.T if variant == 0 else b).astype(np.float64)
    assert np.abs(out.cpu().numpy() - want).max() < 1e-3


def test_bounded_wait_reports_timeout(it_ctx):
    """A wait that runs out (a 20 ms wait on a barrier nothing arrives on: nothing faults) sets the status word.
    Until it is cleared every host-side drain reports it -- it_stream_sync, it_ctx_check_status, CommandBatch.sync,
    Tensor.as_*_slice -- and launches do nothing, so a host layer can never hand out the garbage silently."""
    import torch
    from irontensor_b200 import CommandBatch, Precision, Tensor, flash_attention
    from irontensor_b200._lib import ITError
    _lib.check(it_ctx.lib.it_selftest_wait_timeout(it_ctx.handle, it_ctx.stream(), 20))
    assert it_ctx.lib.it_stream_sync(it_ctx.handle, it_ctx.stream()) == _lib.IT_ERR_TIMEOUT
    word = ctypes.c_int32()
    assert it_ctx.lib.it_ctx_check_status(it_ctx.handle, ctypes.byref(word)) == _lib.IT_ERR_TIMEOUT and word.value == 6
    with pytest.raises(ITError):
        CommandBatch.sync()
    # a launch while the word is set returns at once: its output keeps the poison, and reading it raises
    x = Tensor.from_f32_as_bf16(np.ones(128 * 64, np.float32), [1, 1, 128, 64])
    out = flash_attention(x, x, x, True)
    out._data.fill_(float("nan"))
    raw.fwd(_lib.IT_BF16, 1, 1, 128, 64, True, x.data_ptr(), x.data_ptr(), x.data_ptr(), out.data_ptr(), out.lse.data_ptr(),
            ctx=it_ctx)
    torch.cuda.synchronize()
    assert torch.isnan(out._data.float()).all()
    with pytest.raises(ITError):
        out.as_bf16_slice()
    st = ctypes.c_int32()
    rc = it_ctx.lib.it_attention_status_poll(it_ctx.handle, it_ctx.stream(), ctypes.byref(st))
    assert rc == _lib.IT_ERR_TIMEOUT and st.value == 6
    assert b"ran out" in it_ctx.lib.it_last_error()
    # the word is cleared and the context stays usable
    assert it_ctx.poll_status() == 0
    q, k, v, _ = seeded(1, 1, 1, 128, 64, bf16=True)
    o, _ = gu.run_fwd(it_ctx, q, k, v, True, True)
    assert not np.isnan(o).any()


# ---------------------------------------------------------------- golden vectors (reference's shaders)
def test_golden_forward_vectors(it_ctx):
    g = np.load(os.path.join(GOLD, "flash_kat1.npz"))
    check_f32(gu.run_fwd(it_ctx, g["q"], g["k"], g["v"], True)[0], g["o_causal"], "kat1 causal")
    check_f32(gu.run_fwd(it_ctx, g["q"], g["k"], g["v"], False)[0], g["o_full"], "kat1 full")
    g = np.load(os.path.join(GOLD, "flash_kat2.npz"))
    check_f32(gu.run_fwd(it_ctx, g["q"], g["k"], g["v"], True)[0], g["o_causal"], "kat2 causal")
    g = np.load(os.path.join(GOLD, "tiled_seeded.npz"))
    q, k, v, _ = seeded(int(g["seed"]), 1, 2, 300, 64)
    check_f32(gu.run_fwd(it_ctx, q, k, v, True)[0], g["o_causal"], "tiled causal")
    check_f32(gu.run_fwd(it_ctx, q, k, v, False)[0], g["o_full"], "tiled full")
    g = np.load(os.path.join(GOLD, "decode_seeded.npz"))
    q, k, v, _ = seeded(int(g["seed"]), 1, 4, 119, 64)
    check_f32(gu.run_fwd(it_ctx, q, k, v, True)[0], g["o_causal"], "decode prefix 119")


def test_golden_backward_vectors(it_ctx):
    g = np.load(os.path.join(GOLD, "bwd_kat.npz"))
    o, lse, dq, dk, dv = gu.run_fwd_bwd(it_ctx, g["q"], g["k"], g["v"], g["d_o"], True)
    check_f32(o, g["o_causal"], "bwd_kat O")
    for got, name in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        check_f32(got, g[name], "bwd_kat " + name)
    g = np.load(os.path.join(GOLD, "bwd_seeded.npz"))
    q, k, v, d_o = seeded(int(g["seed"]), 1, 2, 40, 16)
    o, lse, dq, dk, dv = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True)
    for got, name in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        check_f32(got, g[name], "bwd_seeded " + name)


# ---------------------------------------------------------------- fp32 path vs the oracle
@pytest.mark.parametrize("S", [1, 31, 32, 33, 255, 256, 257, 1000])
@pytest.mark.parametrize("D", [16, 64, 128])
def test_fp32_forward_backward_edges(it_ctx, S, D):
    if S == 1000 and D != 64:
        pytest.skip("one long case is enough")
    B, H = (1, 3)
    q, k, v, d_o = seeded(100 + S, B, H, S, D)
    o, lse, dq, dk, dv = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True)
    ro, rlse = ol.fwd(q, k, v, True)
    rdq, rdk, rdv = ol.bwd(q, k, v, d_o, True)
    for got, want, name in ((o, ro, "O"), (lse, rlse, "LSE"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        check_f32(got, want, f"S{S} D{D} {name}")


@pytest.mark.parametrize("shape", [(2, 2, 50, 24), (1, 2, 100, 40), (1, 1, 7, 1), (1, 2, 130, 100)])
def test_fp32_full_attention_odd_head_dims(it_ctx, shape):
    q, k, v, d_o = seeded(7, *shape)
    o, lse, dq, dk, dv = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, False)
    ro, rlse = ol.fwd(q, k, v, False)
    rdq, rdk, rdv = ol.bwd(q, k, v, d_o, False)
    for got, want, name in ((o, ro, "O"), (lse, rlse, "LSE"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        check_f32(got, want, f"{shape} {name}")


def test_config1_tiny_fp32_forward(it_ctx):
    q, k, v, _ = seeded(synth.BASE_SEED + 1, 16, 4, 256, 64)
    o, lse = gu.run_fwd(it_ctx, q, k, v, True)
    ro, rlse = ol.fwd(q, k, v, True)
    check_f32(o, ro, "C1 O")
    check_f32(lse, rlse, "C1 LSE")


def test_config5_greedy_prefix_lengths_fp32(it_ctx):
    worst = 0.0
    for S in range(20, 120):
        q, k, v, _ = seeded(synth.BASE_SEED + S, 1, 4, S, 64)
        o, lse = gu.run_fwd(it_ctx, q, k, v, True)
        ro, rlse = ol.fwd(q, k, v, True)
        worst = max(worst, float(np.abs(o - ro).max()), float(np.abs(lse - rlse).max()))
        assert not np.isnan(o).any()
    assert worst <= F32_TOL, worst


# ---------------------------------------------------------------- bf16 path vs the oracle
@pytest.mark.parametrize("shape,causal", [
    ((1, 1, 128, 64), True), ((1, 2, 256, 128), True), ((2, 3, 384, 128), True), ((1, 2, 300, 64), True),
    ((1, 2, 129, 128), True), ((1, 3, 1000, 64), True), ((1, 2, 512, 128), False), ((1, 2, 200, 64), False),
    ((1, 2, 64, 64), True), ((1, 2, 100, 32), True), ((1, 5, 640, 64), True),
])
def test_bf16_forward_backward(it_ctx, shape, causal):
    q, k, v, d_o = seeded(40, *shape, bf16=True)
    o, lse, dq, dk, dv = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, causal, bf16=True)
    ro, rlse = ol.fwd(q, k, v, causal)
    rdq, rdk, rdv = ol.bwd(q, k, v, d_o, causal)
    assert np.abs(lse - rlse).max() <= 1e-4
    for got, want, name in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        check_bf16(got, want, f"{shape} causal={causal} {name}")


def test_config2_tiny_bf16_forward_backward(it_ctx):
    q, k, v, d_o = seeded(synth.BASE_SEED + 2, 16, 4, 256, 64, bf16=True)
    o, lse, dq, dk, dv = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True, bf16=True)
    ro, rlse = ol.fwd(q, k, v, True)
    rdq, rdk, rdv = ol.bwd(q, k, v, d_o, True)
    assert np.abs(lse - rlse).max() <= 1e-4
    for got, want, name in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        check_bf16(got, want, "C2 " + name)


def _full_size_slices(it_ctx, B, H, S, D, seed, qk_scale, slices):
    """Runs the full-size config on the GPU; checks the listed (batch*head) slices against the
    oracle and returns the GPU outputs (torch) for the property checks."""
    import torch
    BH = B * H
    dev = []
    for tid, sc in ((synth.TENSOR_Q, qk_scale), (synth.TENSOR_K, qk_scale), (synth.TENSOR_V, 1.0), (synth.TENSOR_DO, 1.0)):
        t = torch.empty((BH, S, D), dtype=torch.bfloat16, device="cuda")
        step = max(1, BH // 8)
        for b0 in range(0, BH, step):   # generate in pieces to bound host memory
            b1 = min(BH, b0 + step)
            x = synth.normal(seed, tid, b0 * S * D, (b1 - b0) * S * D, sc)
            t[b0:b1] = torch.from_numpy(synth.f32_to_bf16_bits(x).view(np.int16)).cuda().view(torch.bfloat16).view(b1 - b0, S, D)
        dev.append(t)
    tq, tk, tv, tdo = dev
    o = torch.full_like(tq, float("nan"))
    lse = torch.full((BH, S), float("nan"), dtype=torch.float32, device="cuda")
    raw.fwd(_lib.IT_BF16, B, H, S, D, True, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), lse.data_ptr(), ctx=it_ctx)
    g = [torch.full_like(tq, float("nan")) for _ in range(3)]
    n = raw.bwd_workspace_bytes(_lib.IT_BF16, B, H, S, D)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    raw.bwd(_lib.IT_BF16, B, H, S, D, True, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), tdo.data_ptr(),
            lse.data_ptr(), g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), ws.data_ptr(), n, ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    for t in (o, lse, *g):
        assert not torch.isnan(t).any()
    for bh in slices:
        hq, hk, hv, hdo = (gu.to_host(t[bh])[None, None] for t in (tq, tk, tv, tdo))
        ro, rlse = ol.fwd(hq, hk, hv, True)
        rdq, rdk, rdv = ol.bwd(hq, hk, hv, hdo, True)
        assert np.abs(lse[bh].cpu().numpy() - rlse[0, 0]).max() <= 1e-4
        for got, want, name in ((o, ro, "O"), (g[0], rdq, "dQ"), (g[1], rdk, "dK"), (g[2], rdv, "dV")):
            check_bf16(gu.to_host(got[bh]), want[0, 0], f"slice {bh} {name}")
    return tq, tk, tv, tdo, o, lse, g


def test_config3_gpt_small_width_bf16(it_ctx):
    # slices on both sides of the boundaries of the CTA order's groups of four, spread over the 384, and the tail
    _full_size_slices(it_ctx, 32, 12, 1024, 64, synth.BASE_SEED + 3, 1.0, slices=[0, 3, 4, 97, 191, 192, 290, 376, 383])


def test_config4_long_context_bf16(it_ctx):
    import torch
    B, H, S, D = 4, 16, 8192, 128
    # Slices either side of a boundary of the backward's groups of four (3 | 4), inside the forward's tail group of
    # eight (56, 63), and in the middle: an index slip in the CTA -> (slice, tile) maps would hit some and not others.
    tq, tk, tv, tdo, o, lse, g = _full_size_slices(it_ctx, B, H, S, D, synth.BASE_SEED + 4, 0.5, slices=[0, 3, 4, 31, 56, 63])
    # size-independent properties on the whole tensor ------------------------------------------
    # (1) the shard of a contiguous (batch*head) range equals the same range of the full run, bit for bit
    b0, b1 = 16, 24
    o2 = torch.empty_like(o[b0:b1])
    lse2 = torch.empty_like(lse[b0:b1])
    raw.fwd(_lib.IT_BF16, 1, b1 - b0, S, D, True, tq[b0:b1].data_ptr(), tk[b0:b1].data_ptr(), tv[b0:b1].data_ptr(),
            o2.data_ptr(), lse2.data_ptr(), ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    assert torch.equal(o2, o[b0:b1]) and torch.equal(lse2, lse[b0:b1])
    # ... and so does the backward of an 8-slice shard (the launch one of eight GPUs runs): dK and dV bit for bit,
    # dQ (summed by reduce-adds in arrival order) within the bf16 tolerance
    g2 = [torch.full_like(o2, float("nan")) for _ in range(3)]
    n2 = raw.bwd_workspace_bytes(_lib.IT_BF16, 1, b1 - b0, S, D)
    ws2 = torch.empty(n2, dtype=torch.uint8, device="cuda")
    raw.bwd(_lib.IT_BF16, 1, b1 - b0, S, D, True, tq[b0:b1].data_ptr(), tk[b0:b1].data_ptr(), tv[b0:b1].data_ptr(),
            o2.data_ptr(), tdo[b0:b1].data_ptr(), lse2.data_ptr(), g2[0].data_ptr(), g2[1].data_ptr(), g2[2].data_ptr(),
            ws2.data_ptr(), n2, ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    assert torch.equal(g2[1], g[1][b0:b1]) and torch.equal(g2[2], g[2][b0:b1])
    assert (g2[0].float() - g[0][b0:b1].float()).abs().max().item() <= BF16_MAX_ABS
    del g2, ws2
    # (2) O is linear in V: doubling V doubles O exactly (a power of two commutes with rounding)
    v2 = (tv[b0:b1].float() * 2).to(torch.bfloat16)
    o3 = torch.empty_like(o2)
    raw.fwd(_lib.IT_BF16, 1, b1 - b0, S, D, True, tq[b0:b1].data_ptr(), tk[b0:b1].data_ptr(), v2.data_ptr(),
            o3.data_ptr(), lse2.data_ptr(), ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    assert torch.equal(o3.float(), o2.float() * 2)
    # (3) with V = 1 every output is a probability-weighted mean of ones
    ones = torch.ones_like(tv[b0:b1])
    raw.fwd(_lib.IT_BF16, 1, b1 - b0, S, D, True, tq[b0:b1].data_ptr(), tk[b0:b1].data_ptr(), ones.data_ptr(),
            o3.data_ptr(), lse2.data_ptr(), ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    assert (o3.float() - 1).abs().max().item() <= 2 ** -7
    # (4) dV columns sum: sum_k dV[k,:] = sum_q dO[q,:] because every row of P sums to one
    lhs = g[2][b0:b1].float().sum(1)
    rhs = tdo[b0:b1].float().sum(1)
    assert ((lhs - rhs).abs().max() / rhs.abs().max()).item() < 2e-2


@pytest.mark.parametrize("shape", [(1, 2, 32768, 128), (1, 1, 65536, 128), (1, 2, 40000, 64)])
def test_sequences_beyond_the_bench_size(it_ctx, shape):
    """Sequences of 32K-64K keys (hundreds of key tiles per query tile): checked through properties that
    need no O(S^2) oracle run, plus the first rows against an fp32 softmax (causal rows see only their prefix)."""
    import torch
    B, H, S, D = shape
    gen = torch.Generator(device="cuda").manual_seed(synth.BASE_SEED + S)
    q, k, v, d_o = [torch.randn(B, H, S, D, device="cuda", generator=gen).mul_(0.5 if i < 2 else 1.0).to(torch.bfloat16)
                    for i in range(4)]
    o = torch.full_like(q, float("nan"))
    lse = torch.full((B, H, S), float("nan"), device="cuda")
    ones = torch.ones_like(v)
    raw.fwd(_lib.IT_BF16, B, H, S, D, True, q.data_ptr(), k.data_ptr(), ones.data_ptr(), o.data_ptr(), lse.data_ptr(),
            ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    assert (o.float() - 1).abs().max().item() <= 2 ** -7
    raw.fwd(_lib.IT_BF16, B, H, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
            ctx=it_ctx)
    g = [torch.full_like(q, float("nan")) for _ in range(3)]
    n = raw.bwd_workspace_bytes(_lib.IT_BF16, B, H, S, D)
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    raw.bwd(_lib.IT_BF16, B, H, S, D, True, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(),
            lse.data_ptr(), g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), ws.data_ptr(), n, ctx=it_ctx)
    assert it_ctx.poll_status() == 0
    for t in (o, lse, *g):
        assert not torch.isnan(t).any().item()
    lhs, rhs = g[2].float().sum(2), d_o.float().sum(2)
    assert ((lhs - rhs).abs().max() / rhs.abs().max()).item() < 1e-3
    R = 256
    s = torch.einsum("bhqd,bhkd->bhqk", q[:, :, :R].float(), k[:, :, :R].float()) / D ** 0.5
    s = s.masked_fill(torch.ones(R, R, device="cuda").triu(1).bool(), float("-inf"))
    want = torch.softmax(s, -1) @ v[:, :, :R].float()
    assert (o[:, :, :R].float() - want).abs().max().item() <= 2e-2
    assert (lse[:, :, :R] - torch.logsumexp(s, -1)).abs().max().item() <= 1e-3


def test_causality_and_determinism(it_ctx):
    q, k, v, d_o = seeded(55, 1, 2, 512, 128, bf16=True)
    o1, l1 = gu.run_fwd(it_ctx, q, k, v, True, True)
    o2, l2 = gu.run_fwd(it_ctx, q, k, v, True, True)
    assert np.array_equal(o1, o2) and np.array_equal(l1, l2)
    k2, v2 = k.copy(), v.copy()
    k2[:, :, 300:] += 1.0
    v2[:, :, 300:] -= 2.0
    o3, l3 = gu.run_fwd(it_ctx, q, synth.round_bf16(k2), synth.round_bf16(v2), True, True)
    assert np.array_equal(o3[:, :, :300], o1[:, :, :300]) and np.array_equal(l3[:, :, :300], l1[:, :, :300])
    assert not np.array_equal(o3[:, :, 300:], o1[:, :, 300:])


def test_sharding_uneven_heads_matches_whole(it_ctx):
    # 6 head-slices over 4 ranks (ceil split 2,2,2,0) give the same bytes as one launch
    from irontensor_b200.sharding import shard_range
    q, k, v, d_o = seeded(56, 1, 6, 256, 64, bf16=True)
    whole = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True, True)
    parts = []
    for r in range(4):
        b0, b1 = shard_range(6, 4, r)
        if b1 > b0:
            parts.append(gu.run_fwd_bwd(it_ctx, q[:, b0:b1], k[:, b0:b1], v[:, b0:b1], d_o[:, b0:b1], True, True))
    for i in (0, 1, 3, 4):   # O, LSE, dK, dV are reproducible bit for bit
        assert np.array_equal(np.concatenate([p[i] for p in parts], axis=1), whole[i])
    dq_parts = np.concatenate([p[2] for p in parts], axis=1)   # dQ is summed with atomics: order may differ
    assert np.abs(dq_parts - whole[2]).max() <= 2e-2


# ---------------------------------------------------------------- argument checking
def test_error_codes(it_ctx):
    import torch
    lib, h, s = it_ctx.lib, it_ctx.handle, it_ctx.stream()
    t = torch.zeros(2 * 128 * 64 + 64, dtype=torch.bfloat16, device="cuda")
    p = t.data_ptr()
    lse = torch.zeros(256, device="cuda").data_ptr()
    assert lib.it_flash_attention_fwd(h, s, 7, 1, 2, 128, 64, 1, p, p, p, p, lse) == _lib.IT_ERR_PRECISION
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_BF16, 1, 2, 128, 129, 1, p, p, p, p, lse) == _lib.IT_ERR_UNSUPPORTED_SHAPE
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_BF16, 1, 2, 128, 0, 1, p, p, p, p, lse) == _lib.IT_ERR_UNSUPPORTED_SHAPE
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_BF16, 1, 2, 128, 64, 1, None, p, p, p, lse) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_BF16, 1, -2, 128, 64, 1, p, p, p, p, lse) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_BF16, 1, 2, 128, 64, 1, p + 2, p, p, p, lse) == _lib.IT_ERR_ALIGNMENT
    assert lib.it_flash_attention_fwd(None, s, _lib.IT_BF16, 1, 2, 128, 64, 1, p, p, p, p, lse) == _lib.IT_ERR_INVALID_ARG
    assert b"null" in lib.it_last_error()
    # seq == 0 and batch*heads == 0 are no-ops (src/ops/flash_attention.rs:102-104 of the reference)
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_BF16, 1, 2, 0, 64, 1, None, None, None, None, None) == _lib.IT_OK
    assert lib.it_flash_attention_fwd(h, s, _lib.IT_F32, 0, 2, 16, 64, 1, None, None, None, None, None) == _lib.IT_OK
    n = raw.bwd_workspace_bytes(_lib.IT_BF16, 1, 2, 128, 64)
    ws = torch.zeros(n, dtype=torch.uint8, device="cuda").data_ptr()
    args = (h, s, _lib.IT_BF16, 1, 2, 128, 64, 1, p, p, p, p, p, lse, p, p, p)
    assert lib.it_flash_attention_bwd(*args, ws, n - 1) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_flash_attention_bwd(*args, None, n) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_flash_attention_bwd(*args, ws + 16, n) == _lib.IT_ERR_ALIGNMENT
    # linear_backward with no rows: dy [0,out] and x [0,in] are empty (null from a C caller), dW is a sum over nothing
    dw = torch.full((16, 8), float("nan"), device="cuda")
    assert lib.it_linear_bwd(h, s, 0, 8, 16, None, None, p, None, dw.data_ptr()) == _lib.IT_OK
    torch.cuda.synchronize()
    assert torch.equal(dw, torch.zeros_like(dw))
    # ... and with no output features: dx [n,in] is a sum over nothing, w [0,in] and dy [n,0] may be null
    dx = torch.full((4, 8), 1.0, dtype=torch.bfloat16, device="cuda")
    assert lib.it_linear_bwd(h, s, 4, 8, 0, None, p, None, dx.data_ptr(), None) == _lib.IT_OK
    torch.cuda.synchronize()
    assert torch.equal(dx, torch.zeros_like(dx))
    assert lib.it_linear_bwd(h, s, 4, 8, 16, None, p, p, dx.data_ptr(), None) == _lib.IT_ERR_INVALID_ARG
    assert it_ctx.poll_status() == 0


# ---------------------------------------------------------------- the mirrored op interface
def test_ops_mirror_reference_interface(it_ctx):
    from irontensor_b200 import CommandBatch, Precision, Tensor, attention, attention_backward_recompute, flash_attention
    B, H, S, D = 2, 4, 32, 16
    g = np.load(os.path.join(GOLD, "flash_kat1.npz"))
    q = Tensor.from_f32_slice(g["q"].reshape(-1), [B, H, S, D])
    CommandBatch.begin()
    out = flash_attention(q, q, q, True)
    CommandBatch.sync()
    assert out.shape() == [B, H, S, D] and out.precision() is Precision.FP32
    assert np.abs(out.as_f32_slice().reshape(B, H, S, D) - g["o_causal"]).max() <= F32_TOL
    CommandBatch.end()
    # attention() takes [B,S,H,D] (src/ops/attention.rs:279-285) and must agree with flash_attention
    x = np.ascontiguousarray(g["q"].transpose(0, 2, 1, 3))
    qs = Tensor.from_f32_slice(x.reshape(-1), [B, S, H, D])
    std = attention(qs, qs, qs, False).as_f32_slice().reshape(B, S, H, D).transpose(0, 2, 1, 3)
    assert np.abs(std - g["o_full"]).max() <= F32_TOL
    # backward with and without the cached forward results
    gb = np.load(os.path.join(GOLD, "bwd_kat.npz"))
    shp = list(gb["q"].shape)
    tq, tk, tv, tdo = (Tensor.from_f32_slice(gb[n].reshape(-1), shp) for n in ("q", "k", "v", "d_o"))
    for cached in (False, True):
        if cached:
            o = flash_attention(tq, tk, tv, True)
            grads = attention_backward_recompute(tdo, tq, tk, tv, o=o, lse=o.lse)
        else:
            grads = attention_backward_recompute(tdo, tq, tk, tv)
        CommandBatch.commit_async()
        CommandBatch.wait_for_completion()
        assert CommandBatch.is_async_complete()
        for t, name in zip(grads, ("dq", "dk", "dv")):
            assert np.abs(t.as_f32_slice().reshape(shp) - gb[name]).max() <= F32_TOL
    # the reference's asserts
    with pytest.raises(AssertionError, match="same shape"):
        flash_attention(q, Tensor.zeros([B, H, S + 1, D]), q, True)
    with pytest.raises(AssertionError, match="4D"):
        flash_attention(q.view([B * H, S, D]), q.view([B * H, S, D]), q.view([B * H, S, D]), True)
    with pytest.raises(AssertionError, match="precision"):
        flash_attention(q, q.to_bf16(), q, True)
    z = flash_attention(Tensor.zeros([2, 2, 0, 8]), Tensor.zeros([2, 2, 0, 8]), Tensor.zeros([2, 2, 0, 8]), True)
    assert z.shape() == [2, 2, 0, 8]
    # bf16 tensors through the same ops
    qb = q.to_bf16()
    ob = flash_attention(qb, qb, qb, True)
    assert ob.precision() is Precision.BF16
    ref = ol.fwd(synth.round_bf16(g["q"]), synth.round_bf16(g["k"]), synth.round_bf16(g["v"]), True)[0]
    assert np.abs(ob.to_f32_host() - ref).max() <= BF16_MAX_ABS


def test_host_step_overlapped_chunks_match_device_resident(it_ctx):
    """HostAttentionStep (pinned host tensors, chunked over streams) gives the bytes of one device-resident run."""
    import torch
    from irontensor_b200 import HostAttentionStep, Precision
    BH, S, D = 10, 256, 64     # 10 slices in 4 chunks: 3,3,3,1
    q, k, v, d_o = seeded(77, 1, BH, S, D, bf16=True)
    whole = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True, True)
    host_in = [gu.to_dev(x[0], True).cpu().pin_memory() for x in (q, k, v, d_o)]
    host_out = [torch.empty_like(host_in[0]).pin_memory() for _ in range(4)]
    step = HostAttentionStep(BH, S, D, Precision.BF16, causal=True, chunks=4)
    for _ in range(2):   # twice: buffers and streams are reused
        step.run(*host_in, *host_out)
        torch.cuda.synchronize()
    assert it_ctx.poll_status() == 0
    got = [gu.to_host(t) for t in host_out]   # O, dQ, dK, dV
    assert np.array_equal(got[0], whole[0][0])
    assert np.abs(got[1] - whole[2][0]).max() <= 2e-2     # dQ: reduction order may differ
    assert np.array_equal(got[2], whole[3][0]) and np.array_equal(got[3], whole[4][0])
    # fp32 tensors (the reference's own precision), an uneven last group, and the log-sum-exp downloaded as well
    BH, S, D = 5, 70, 32
    q, k, v, d_o = seeded(78, 1, BH, S, D)
    whole = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True, False)
    host_in = [torch.from_numpy(np.ascontiguousarray(x[0])).pin_memory() for x in (q, k, v, d_o)]
    host_out = [torch.empty_like(host_in[0]).pin_memory() for _ in range(4)]
    host_lse = torch.empty((BH, S), dtype=torch.float32).pin_memory()
    step = HostAttentionStep(BH, S, D, Precision.FP32, causal=True, chunks=3)      # groups of 2, 2, 1
    step.run(*host_in, *host_out, hlse=host_lse)
    torch.cuda.synchronize()
    assert it_ctx.poll_status() == 0
    for got_t, want in zip(host_out, (whole[0][0], whole[2][0], whole[3][0], whole[4][0])):
        assert np.array_equal(got_t.numpy(), want)
    assert np.array_equal(host_lse.numpy(), whole[1][0])
    # the copies alone leave the status clean and touch nothing but the host tensors
    step.run(*host_in, *host_out, copies_only=True)
    torch.cuda.synchronize()
    assert it_ctx.poll_status() == 0


def test_forward_on_a_stream_object_without_a_work_counter(it_ctx):
    """The context hands each stream object one work-item counter out of a pool of 4096.  A stream object wrapped when
    the pool is empty has none: its forwards start one CTA per work item and give the same bits; destroying stream
    objects hands their counters back."""
    import torch
    B, H, S, D = 6, 8, 1024, 64                      # 192 slices x 4 pairs of query tiles: more items than SMs
    q, k, v, _ = seeded(811, B, H, S, D, bf16=True)
    tq, tk, tv = (gu.to_dev(x, True) for x in (q, k, v))
    ref_o, ref_lse = torch.empty_like(tq), torch.empty((B, H, S), device="cuda")
    raw.fwd(_lib.IT_BF16, B, H, S, D, True, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), ref_o.data_ptr(), ref_lse.data_ptr(), ctx=it_ctx)
    lib, cur = it_ctx.lib, torch.cuda.current_stream().cuda_stream
    wrapped = []
    try:
        for _ in range(4200):
            h = ctypes.c_void_p()
            _lib.check(lib.it_stream_wrap(it_ctx.handle, ctypes.c_void_p(cur), ctypes.byref(h)))
            wrapped.append(h)
        for h in (wrapped[0], wrapped[-1]):          # one with a counter, one without
            o, lse = torch.full_like(tq, float("nan")), torch.full((B, H, S), float("nan"), device="cuda")
            _lib.check(lib.it_flash_attention_fwd(it_ctx.handle, h, _lib.IT_BF16, B, H, S, D, 1, tq.data_ptr(), tk.data_ptr(),
                                                  tv.data_ptr(), o.data_ptr(), lse.data_ptr()))
            torch.cuda.synchronize()
            assert torch.equal(o, ref_o) and torch.equal(lse, ref_lse)
    finally:
        for h in wrapped:
            lib.it_stream_destroy(it_ctx.handle, h)
    assert it_ctx.poll_status() == 0


def test_kernel_timers_and_profiler_tags(it_ctx):
    """The device-side timers that stand in for the reference's profiler categories (OpCategory::FlashAttention,
    src/ops/flash_attention.rs:77; attn_bwd/* in src/train/helpers.rs:126-183): levels 1 to 3 bracket more kernels."""
    assert it_ctx.kernel_tag(0) == "FlashAttention"
    assert it_ctx.kernel_tag(1).startswith("attn_bwd/") and "grad_qk" in it_ctx.kernel_tag(1)
    assert it_ctx.kernel_tag(2) == "attn_bwd/prepare" and it_ctx.kernel_tag(3) == "attn_bwd/finish"
    q, k, v, d_o = seeded(5, 1, 2, 256, 64, bf16=True)
    it_ctx.enable_kernel_timing(3)
    try:
        gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True, True)
        times = [it_ctx.kernel_ms(w) for w in range(4)]
        assert all(0.0 < t < 50.0 for t in times), times
    finally:
        it_ctx.enable_kernel_timing(0)


@pytest.mark.parametrize("shape,bf16", [((2, 3, 256, 64), True), ((1, 2, 300, 128), True), ((2, 4, 32, 16), False),
                                        ((1, 3, 100, 40), False), ((2, 2, 64, 64), True)])
def test_bshd_layout_matches_bhsd(it_ctx, shape, bf16):
    """attention()/attention_backward() on [B,S,H,D] (strided TMA, no transposes) against the [B,H,S,D] path."""
    import torch
    from irontensor_b200 import Precision, Tensor, attention, attention_backward
    B, H, S, D = shape
    q, k, v, d_o = seeded(81, B, H, S, D, bf16=bf16)
    want = gu.run_fwd_bwd(it_ctx, q, k, v, d_o, True, bf16)                    # O, LSE, dQ, dK, dV in [B,H,S,D]
    mk = Tensor.from_f32_as_bf16 if bf16 else Tensor.from_f32_slice
    tq, tk, tv, tdo = (mk(np.ascontiguousarray(x.transpose(0, 2, 1, 3)).reshape(-1), [B, S, H, D]) for x in (q, k, v, d_o))
    o = attention(tq, tk, tv, True)
    dq, dk, dv = attention_backward(tdo, tq, tk, tv, o, True)
    assert it_ctx.poll_status() == 0
    back = lambda t: t.to_f32_host().reshape(B, S, H, D).transpose(0, 2, 1, 3)
    assert np.array_equal(back(o), want[0])
    assert np.array_equal(o.lse.to_f32_host().reshape(B, H, S), want[1])
    assert np.array_equal(back(dk), want[3]) and np.array_equal(back(dv), want[4])
    if bf16 and S >= 128 and D in (64, 128):
        assert np.abs(back(dq) - want[2]).max() <= 2e-2      # reduction order of the fp32 accumulator
    else:
        assert np.array_equal(back(dq), want[2])
    # non-causal forward against the oracle, in this layout
    o2 = attention(tq, tk, tv, False)
    ref = ol.fwd(q, k, v, False)[0]
    tol = BF16_MAX_ABS if bf16 else F32_TOL
    assert np.abs(back(o2) - ref).max() <= tol


@pytest.mark.parametrize("B,Sq,Skv,H,D,bf16", [(2, 5, 37, 3, 16, False), (1, 200, 64, 2, 64, False), (2, 1, 77, 4, 32, False),
                                               (1, 70, 300, 2, 128, True), (1, 128, 384, 2, 64, True), (1, 300, 40, 2, 40, True)])
def test_attention_with_another_key_length(it_ctx, B, Sq, Skv, H, D, bf16):
    """attention(q, k, v, causal=False) with K/V of another sequence length than Q, which the reference accepts
    (src/ops/attention.rs:304; only the causal branch asserts equal lengths, :349-352), against the oracle; and the
    causal call with unequal lengths raises the reference's assertion."""
    from irontensor_b200 import Tensor, attention
    rng = np.random.default_rng(1000 * Sq + Skv)
    rnd = lambda *shape: synth.round_bf16(rng.standard_normal(shape).astype(np.float32)) if bf16 else rng.standard_normal(shape).astype(np.float32)
    q, k, v = rnd(B, Sq, H, D), rnd(B, Skv, H, D), rnd(B, Skv, H, D)
    mk = Tensor.from_f32_as_bf16 if bf16 else Tensor.from_f32_slice
    tq, tk, tv = mk(q.reshape(-1), [B, Sq, H, D]), mk(k.reshape(-1), [B, Skv, H, D]), mk(v.reshape(-1), [B, Skv, H, D])
    out = attention(tq, tk, tv, False)
    assert it_ctx.poll_status() == 0
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    ro, rlse = ol.cross_fwd(t(q), t(k), t(v))
    got = out.to_f32_host().reshape(B, Sq, H, D).transpose(0, 2, 1, 3)
    assert np.abs(got - ro).max() <= (BF16_MAX_ABS if bf16 else F32_TOL)
    assert np.abs(out.lse.to_f32_host().reshape(B, H, Sq) - rlse).max() <= F32_TOL
    with pytest.raises(AssertionError, match="same seq_len"):
        attention(tq, tk, tv, True)


@pytest.mark.parametrize("S,causal,qk_scale", [(4096, True, 1.0), (4100, True, 1.0), (4225, False, 1.0), (4352, True, 3.0),
                                               (4480, False, 3.0)])
def test_bf16_long_sequence_forward(it_ctx, S, causal, qk_scale, monkeypatch):
    """Both bf16 forward kernels at head_dim 128 on long sequences (the launcher picks by length; IT_FWD_KERNEL forces one):
    one query tile per CTA with the two softmax groups alternating over key tiles, and two query tiles per work item
    with one CTA per SM walking the items.  Against the oracle: ragged lengths, odd and even tile counts, no mask, and
    scores spread widely enough that the reference maximum is raised (O rescaled) many times."""
    q, k, v, _ = seeded(90 + S, 1, 2, S, 128, bf16=True, qk_scale=qk_scale)
    ro, rlse = ol.fwd(q, k, v, causal)
    for kernel in ("pp", "two"):
        monkeypatch.setenv("IT_FWD_KERNEL", kernel)
        o, lse = gu.run_fwd(it_ctx, q, k, v, causal, bf16=True)
        assert np.abs(lse - rlse).max() <= 1e-4 * max(1.0, qk_scale ** 2), kernel
        check_bf16(o, ro, f"S={S} causal={causal} {kernel} O")


@pytest.mark.parametrize("B,H,S,D,causal", [(8, 12, 1024, 64, True), (5, 8, 1000, 64, True), (6, 10, 640, 128, True),
                                            (40, 4, 256, 64, False), (3, 7, 2176, 64, True)])
def test_forward_walking_work_items_matches_one_item_per_cta(it_ctx, B, H, S, D, causal, monkeypatch):
    """More work items than SMs: the two-query-tile forward starts one CTA per SM and each walks items drawn from
    the stream's counter.  An item's arithmetic does not depend on who runs it or after what, so O and LSE must
    equal, bit for bit, what one CTA per item produces (IT_FWD_ONE_ITEM_PER_CTA=1); repeated launches on the same
    stream re-zero the counter; a few slices are checked against the oracle as well."""
    import torch
    q, k, v, _ = seeded(700 + S + D, B, H, S, D, bf16=True)
    monkeypatch.setenv("IT_FWD_KERNEL", "two")
    monkeypatch.setenv("IT_FWD_ONE_ITEM_PER_CTA", "1")
    o1, lse1 = gu.run_fwd(it_ctx, q, k, v, causal, bf16=True)
    monkeypatch.delenv("IT_FWD_ONE_ITEM_PER_CTA")
    for _ in range(3):
        o2, lse2 = gu.run_fwd(it_ctx, q, k, v, causal, bf16=True)
        assert np.array_equal(o1, o2) and np.array_equal(lse1, lse2)
    for b, h in ((0, 0), (B - 1, H - 1), (B // 2, H // 3)):
        ro, rlse = ol.fwd(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], causal)
        assert np.abs(lse2[b:b + 1, h:h + 1] - rlse).max() <= 1e-4
        check_bf16(o2[b:b + 1, h:h + 1], ro, f"slice ({b},{h}) O")


@pytest.mark.parametrize("shape,bf16,causal", [
    ((2, 40, 4, 2, 16), False, True), ((1, 100, 6, 2, 40), False, True), ((1, 300, 8, 1, 64), False, False),
    ((1, 256, 4, 2, 64), True, True), ((2, 384, 8, 2, 128), True, True), ((1, 300, 4, 1, 128), True, False),
    ((1, 100, 4, 2, 64), True, True), ((1, 4224, 4, 2, 128), True, True),
])
def test_grouped_query_attention(it_ctx, shape, bf16, causal):
    """attention_gqa / attention_gqa_backward (K/V with fewer heads, no expanded copies, dK/dV summed over the
    group inside the kernels) against the reference's composition repeat_kv -> attention -> repeat_kv_backward."""
    from irontensor_b200 import Tensor, attention_gqa, attention_gqa_backward
    B, S, H, Hkv, D = shape
    q4, _, _, do4 = seeded(120, B, H, S, D, bf16=bf16)
    _, k4, v4, _ = seeded(121, B, Hkv, S, D, bf16=bf16)
    to_bshd = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    q, k, v, d_o = (to_bshd(x) for x in (q4, k4, v4, do4))
    mk = Tensor.from_f32_as_bf16 if bf16 else Tensor.from_f32_slice
    tq, tk, tv, tdo = mk(q.reshape(-1), [B, S, H, D]), mk(k.reshape(-1), [B, S, Hkv, D]), mk(v.reshape(-1), [B, S, Hkv, D]), \
        mk(d_o.reshape(-1), [B, S, H, D])
    o = attention_gqa(tq, tk, tv, causal)
    dq, dk, dv = attention_gqa_backward(tdo, tq, tk, tv, o, causal)
    assert it_ctx.poll_status() == 0
    ro, rlse = ol.gqa_fwd(q, k, v, causal)
    rdq, rdk, rdv = ol.gqa_bwd(q, k, v, d_o, causal)
    assert np.abs(o.lse.to_f32_host() - rlse).max() <= 1e-4
    for got, want, name in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        g = got.to_f32_host()
        assert g.shape == want.shape
        if bf16:
            # dK and dV are sums over the group's H // Hkv query heads: their magnitude, and with it the size of a
            # bf16 rounding step, grows like the square root of the group size
            scale = math.sqrt(H // Hkv) if name in ("dK", "dV") else 1.0
            check_bf16(g / scale, want / scale, f"{shape} {name}")
        else:
            assert np.abs(g - want).max() <= F32_TOL, f"{shape} {name}: {np.abs(g - want).max()}"


@pytest.mark.parametrize("shape,bf16,offset", [((1, 2, 1, 4), False, 0), ((2, 16, 8, 64), False, 0), ((1, 8, 4, 32), False, 10),
                                               ((2, 300, 6, 128), False, 0), ((1, 100, 4, 64), True, 3)])
def test_rope_matches_reference_math(it_ctx, shape, bf16, offset):
    """rope() and the one-launch rope_qk() against the CPU restatement of rope_f32 (src/shaders/rope.metal:22-61); the
    shapes are those of the reference's tests (src/ops/rope.rs:128-250: simple, position zero, larger, with offset)."""
    from irontensor_b200 import Tensor, rope, rope_qk
    B, S, H, D = shape
    x = seeded(140, B, H, S, D, bf16=bf16)[0].transpose(0, 2, 1, 3).copy()     # [B,S,H,D]
    mk = Tensor.from_f32_as_bf16 if bf16 else Tensor.from_f32_slice
    tol = 2e-2 if bf16 else 1e-5
    y = rope(mk(x.reshape(-1), [B, S, H, D]), 10000.0, offset).to_f32_host()
    assert np.abs(y - ol.rope(x, 10000.0, offset)).max() <= tol
    if offset == 0 and not bf16:
        assert np.array_equal(y[:, 0], x[:, 0])                               # position 0 is the identity
    Hkv = max(1, H // 2)
    k = x[:, :, :Hkv].copy()
    qo, ko = rope_qk(mk(x.reshape(-1), [B, S, H, D]), mk(k.reshape(-1), [B, S, Hkv, D]), 10000.0, offset)
    assert np.abs(qo.to_f32_host() - ol.rope(x, 10000.0, offset)).max() <= tol
    assert np.abs(ko.to_f32_host() - ol.rope(k, 10000.0, offset)).max() <= tol
    back, _ = rope_qk(qo, ko, 10000.0, offset, inverse=True)
    assert np.abs(back.to_f32_host() - x).max() <= (4e-2 if bf16 else 1e-5)


@pytest.mark.parametrize("shape,bf16", [((1, 40, 4, 2, 16), False), ((1, 300, 4, 4, 64), False), ((1, 256, 4, 2, 64), True),
                                        ((1, 384, 4, 1, 128), True)])
def test_attention_backward_with_rope_folded_in(it_ctx, shape, bf16):
    """rope -> grouped-query attention -> backward with the rotary backward folded into the kernels' output paths,
    against the reference's chain rope, repeat_kv, attention, attention backward, repeat_kv_backward, rope_backward
    (src/train/forward.rs:111-139, src/train/backward.rs:102-132)."""
    from irontensor_b200 import Tensor, attention_gqa, attention_gqa_backward, rope_qk
    B, S, H, Hkv, D = shape
    base, offset = 10000.0, 0
    q4, _, _, do4 = seeded(150, B, H, S, D, bf16=bf16)
    _, k4, v4, _ = seeded(151, B, Hkv, S, D, bf16=bf16)
    to_bshd = lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3))
    q, k, v, d_o = (to_bshd(a) for a in (q4, k4, v4, do4))
    mk = Tensor.from_f32_as_bf16 if bf16 else Tensor.from_f32_slice
    tq, tk, tv, tdo = mk(q.reshape(-1), [B, S, H, D]), mk(k.reshape(-1), [B, S, Hkv, D]), mk(v.reshape(-1), [B, S, Hkv, D]), \
        mk(d_o.reshape(-1), [B, S, H, D])
    tqr, tkr = rope_qk(tq, tk, base, offset)
    o = attention_gqa(tqr, tkr, tv, True)
    dq, dk, dv = attention_gqa_backward(tdo, tqr, tkr, tv, o, True, rope_base=base, position_offset=offset)
    assert it_ctx.poll_status() == 0
    # oracle: rotate what the device rotated (its stored, rounded q_rope/k_rope), so that only the backward is compared
    qr, kr = tqr.to_f32_host(), tkr.to_f32_host()
    rdq, rdk, rdv = ol.gqa_bwd(qr, kr, v, d_o, True)
    rdq, rdk = ol.rope(rdq, base, offset, inverse=True), ol.rope(rdk, base, offset, inverse=True)
    for got, want, name in ((dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        g = got.to_f32_host()
        if bf16:
            scale = math.sqrt(H // Hkv) if name in ("dK", "dV") else 1.0
            check_bf16(g / scale, want / scale, f"{shape} {name}")
        else:
            assert np.abs(g - want).max() <= F32_TOL, f"{shape} {name}: {np.abs(g - want).max()}"


@pytest.mark.parametrize("shape,bf16", [((2, 4, 4, 64, 100, 128), False), ((1, 8, 2, 128, 1000, 1024), False),
                                        ((3, 6, 2, 64, 777, 800), True), ((2, 32, 4, 128, 5000, 5000), True),
                                        ((1, 16, 1, 128, 4096, 4096), True), ((16, 4, 4, 64, 64, 256), True),
                                        ((1, 2, 2, 40, 333, 400), False), ((1, 128, 1, 64, 600, 640), True),
                                        ((1, 160, 1, 64, 300, 300), True), ((2, 24, 2, 128, 257, 300), True)])
def test_kv_cache_decode_equals_last_row_of_causal_attention(it_ctx, shape, bf16):
    """attention_decode (one new token against a K/V cache, grouped heads, keys split over CTAs) against the
    last row of the oracle's causal attention over the same kv_len tokens."""
    from irontensor_b200 import Tensor, attention_decode
    B, H, Hkv, D, L, max_len = shape
    q4, _, _, _ = seeded(160, B, H, L, D, bf16=bf16)          # [B,H,L,D]; only the last row matters
    _, k4, v4, _ = seeded(161, B, Hkv, L, D, bf16=bf16)
    mk = Tensor.from_f32_as_bf16 if bf16 else Tensor.from_f32_slice
    kc = np.zeros((B, max_len, Hkv, D), np.float32)
    vc = np.full((B, max_len, Hkv, D), 7.0, np.float32)       # positions past kv_len must not be read into the result
    kc[:, :L] = k4.transpose(0, 2, 1, 3)
    vc[:, :L] = v4.transpose(0, 2, 1, 3)
    q_last = np.ascontiguousarray(q4[:, :, L - 1])            # [B,H,D]
    out = attention_decode(mk(q_last.reshape(-1), [B, H, D]), mk(kc.reshape(-1), [B, max_len, Hkv, D]),
                           mk(vc.reshape(-1), [B, max_len, Hkv, D]), L)
    assert it_ctx.poll_status() == 0
    G = H // Hkv
    ro, rlse = ol.fwd(q4, np.repeat(k4, G, axis=1), np.repeat(v4, G, axis=1), True)
    tol = BF16_MAX_ABS if bf16 else F32_TOL
    assert np.abs(out.to_f32_host() - ro[:, :, L - 1]).max() <= tol
    assert np.abs(out.lse.to_f32_host() - rlse[:, :, L - 1]).max() <= 1e-4


def test_kv_cache_decode_over_a_generation(it_ctx):
    """The reference's greedy generation pattern (config 5: B1 H4 D64, sequence lengths 20..119, one full forward per
    token, src/inference/generator.rs:146-200) served from a cache: every step's decode output equals the last row of
    the full forward at that length."""
    from irontensor_b200 import Tensor, attention_decode, flash_attention
    B, H, D, L0, L1 = 1, 4, 64, 20, 120
    q, k, v, _ = seeded(synth.BASE_SEED + 5, B, H, L1, D)
    kc = Tensor.from_f32_slice(np.ascontiguousarray(k.transpose(0, 2, 1, 3)).reshape(-1), [B, L1, H, D])
    vc = Tensor.from_f32_slice(np.ascontiguousarray(v.transpose(0, 2, 1, 3)).reshape(-1), [B, L1, H, D])
    worst = 0.0
    for L in range(L0, L1):
        full = flash_attention(*(Tensor.from_f32_slice(np.ascontiguousarray(x[:, :, :L]).reshape(-1), [B, H, L, D]) for x in (q, k, v)), True)
        want = full.to_f32_host()[:, :, L - 1]
        got = attention_decode(Tensor.from_f32_slice(np.ascontiguousarray(q[:, :, L - 1]).reshape(-1), [B, H, D]), kc, vc, L)
        worst = max(worst, float(np.abs(got.to_f32_host() - want).max()))
    assert it_ctx.poll_status() == 0
    assert worst <= F32_TOL, worst


@pytest.mark.parametrize("n,k,out", [(128, 64, 256), (300, 200, 264), (1000, 1024, 768), (130, 72, 40), (4096, 2048, 512), (64, 8, 8)])
def test_projection_gemms_match_fp32_matmul(it_ctx, n, k, out):
    """linear_forward / linear_backward (src/train/helpers.rs:48-76) on the tcgen05 GEMM, the three transposition
    cases, against fp32 matmuls of the same bf16-rounded operands (what the reference computes after ensure_fp32).
    Sizes cover edge tiles in M, N and K."""
    from irontensor_b200 import Tensor, linear_backward, linear_forward
    x = synth.round_bf16(synth.normal(170, synth.TENSOR_Q, 0, n * k, 1.0)).reshape(n, k)
    w = synth.round_bf16(synth.normal(170, synth.TENSOR_K, 0, out * k, 0.05)).reshape(out, k)
    dy = synth.round_bf16(synth.normal(170, synth.TENSOR_DO, 0, n * out, 1.0)).reshape(n, out)
    tx, tw, tdy = (Tensor.from_f32_as_bf16(a.reshape(-1), list(a.shape)) for a in (x, w, dy))
    y = linear_forward(tx, tw).to_f32_host()
    dx, dw = linear_backward(tdy, tx, tw)
    assert it_ctx.poll_status() == 0
    x64, w64, dy64 = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    for got, want, name, exact_store in ((y, x64 @ w64.T, "y", False), (dx.to_f32_host(), dy64 @ w64, "dx", False),
                                         (dw.to_f32_host(), dy64.T @ x64, "dW", True)):
        err = np.abs(got - want).max()
        scale = np.abs(want).max() + 1e-30
        # bf16 results carry half an ulp (2^-9 relative) of storage rounding; the fp32 dW only accumulation error
        assert err <= (2e-5 if exact_store else 4.5e-3) * scale, f"{name} n={n} k={k} out={out}: {err} vs scale {scale}"


@pytest.mark.parametrize("B,S,hidden,H,Hkv,D,base", [(2, 100, 256, 4, 2, 64, 10000.0), (1, 300, 512, 8, 8, 128, 10000.0),
                                                      (3, 50, 64, 2, 1, 32, 500.0), (1, 130, 200, 3, 3, 96, None)])
def test_fused_qkv_projection_with_rotary_epilogue(it_ctx, B, S, hidden, H, Hkv, D, base):
    """qkv_rope_forward (one GEMM over [Wq; Wk; Wv] whose epilogue rotates Q and K and writes the attention layout)
    against the reference's chain: three fp32 projections, then rope on Q and K (src/train/forward.rs:101-112)."""
    from irontensor_b200 import Tensor, qkv_rope_forward
    n, out = B * S, (H + 2 * Hkv) * D
    x = synth.round_bf16(synth.normal(180, synth.TENSOR_Q, 0, n * hidden, 1.0)).reshape(B, S, hidden)
    w = synth.round_bf16(synth.normal(180, synth.TENSOR_K, 0, out * hidden, 0.05)).reshape(out, hidden)
    q, k, v = qkv_rope_forward(Tensor.from_f32_as_bf16(x.reshape(-1), [B, S, hidden]), Tensor.from_f32_as_bf16(w.reshape(-1), [out, hidden]),
                               H, Hkv, D, base, 3)
    assert it_ctx.poll_status() == 0
    y = (x.reshape(n, hidden).astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    rq = y[:, :H * D].reshape(B, S, H, D)
    rk = y[:, H * D:(H + Hkv) * D].reshape(B, S, Hkv, D)
    rv = y[:, (H + Hkv) * D:].reshape(B, S, Hkv, D)
    if base is not None:
        rq, rk = ol.rope(rq, base, 3), ol.rope(rk, base, 3)
    for got, want, name in ((q, rq, "q"), (k, rk, "k"), (v, rv, "v")):
        g = got.to_f32_host()
        assert g.shape == want.shape
        err = np.abs(g - want).max()
        assert err <= 4.5e-3 * np.abs(want).max(), f"{name}: {err}"


@pytest.mark.parametrize("B,S,hidden,H,Hkv,D", [(2, 256, 128, 4, 2, 64), (1, 384, 256, 4, 4, 128), (1, 130, 64, 2, 1, 64)])
def test_packed_layer_equals_the_separate_tensor_path(it_ctx, B, S, hidden, H, Hkv, D):
    """The whole layer on ONE packed q|k|v buffer (fused projection -> attention -> attention backward with the rotary
    backward folded in -> one linear_backward for the stacked weights) against the same ops on separate tensors with
    the gradients concatenated by hand: identical forward, gradients within the dQ accumulation-order tolerance."""
    from irontensor_b200 import (Tensor, attention_gqa, attention_gqa_backward, attention_packed, attention_packed_backward,
                                 linear_backward, qkv_rope_forward)
    n, W = B * S, (H + 2 * Hkv) * D
    x = synth.round_bf16(synth.normal(190, synth.TENSOR_Q, 0, n * hidden, 1.0)).reshape(B, S, hidden)
    w = synth.round_bf16(synth.normal(190, synth.TENSOR_K, 0, W * hidden, 0.08)).reshape(W, hidden)
    d_o = synth.round_bf16(synth.normal(190, synth.TENSOR_DO, 0, n * H * D, 1.0)).reshape(B, S, H, D)
    tx, tw = Tensor.from_f32_as_bf16(x.reshape(-1), [B, S, hidden]), Tensor.from_f32_as_bf16(w.reshape(-1), [W, hidden])
    tdo = Tensor.from_f32_as_bf16(d_o.reshape(-1), [B, S, H, D])
    base = 10000.0
    # separate tensors
    q, k, v = qkv_rope_forward(tx, tw, H, Hkv, D, base)
    o = attention_gqa(q, k, v, True)
    dq, dk, dv = attention_gqa_backward(tdo, q, k, v, o, True, rope_base=base)
    cat = np.concatenate([dq.to_f32_host().reshape(n, H * D), dk.to_f32_host().reshape(n, Hkv * D),
                          dv.to_f32_host().reshape(n, Hkv * D)], axis=1)
    dx_ref, dw_ref = linear_backward(Tensor.from_f32_as_bf16(cat.reshape(-1), [n, W]), tx.view([n, hidden]), tw)
    # packed
    qkv = qkv_rope_forward(tx, tw, H, Hkv, D, base, packed=True)
    o2 = attention_packed(qkv, H, Hkv, D, True)
    dqkv = attention_packed_backward(tdo, qkv, o2, H, Hkv, D, True, rope_base=base)
    dx, dw = linear_backward(dqkv.view([n, W]), tx.view([n, hidden]), tw)
    assert it_ctx.poll_status() == 0
    packed_host = qkv.to_f32_host().reshape(n, W)
    assert np.array_equal(packed_host[:, :H * D], q.to_f32_host().reshape(n, H * D))
    assert np.array_equal(packed_host[:, H * D:(H + Hkv) * D], k.to_f32_host().reshape(n, Hkv * D))
    assert np.array_equal(packed_host[:, (H + Hkv) * D:], v.to_f32_host().reshape(n, Hkv * D))
    assert np.array_equal(o2.to_f32_host(), o.to_f32_host()) and np.array_equal(o2.lse.to_f32_host(), o.lse.to_f32_host())
    g = dqkv.to_f32_host().reshape(n, W)
    assert np.array_equal(g[:, H * D:], cat[:, H * D:])                     # dk | dv: bit for bit
    assert np.abs(g[:, :H * D] - cat[:, :H * D]).max() <= 2e-2              # dq: order of the fp32 reduce-adds
    assert np.abs(dx.to_f32_host() - dx_ref.to_f32_host()).max() <= 4.5e-3 * np.abs(dx_ref.to_f32_host()).max() + 2e-2
    assert np.abs(dw.to_f32_host() - dw_ref.to_f32_host()).max() <= 2e-2 * np.abs(dw_ref.to_f32_host()).max()


def test_randomised_shapes_against_the_oracle(it_ctx):
    """Twenty seeded random shapes (ragged lengths around the 128-row tiles, odd batch and head counts, grouped heads,
    both head dims of the tensor-core path and a few of the CUDA-core path, causal or not) through attention_gqa and
    its backward, against the oracle composition.  Catches index arithmetic that the hand-picked shapes miss."""
    from irontensor_b200 import Tensor, attention_gqa, attention_gqa_backward
    rng = np.random.default_rng(20251)
    for case in range(20):
        D = int(rng.choice([64, 128, 128, 64, 32, 80]))
        Hkv = int(rng.integers(1, 4))
        G = int(rng.choice([1, 1, 2, 3, 4]))
        H = Hkv * G
        B = int(rng.integers(1, 3))
        S = int(rng.choice([rng.integers(1, 130), rng.integers(128, 400), rng.integers(250, 700)]))
        causal = bool(rng.integers(0, 2))
        bf16 = True
        q4, _, _, do4 = seeded(300 + case, B, H, S, D, bf16=bf16)
        _, k4, v4, _ = seeded(400 + case, B, Hkv, S, D, bf16=bf16)
        to_bshd = lambda a: np.ascontiguousarray(a.transpose(0, 2, 1, 3))
        q, k, v, d_o = (to_bshd(a) for a in (q4, k4, v4, do4))
        tq, tk, tv, tdo = (Tensor.from_f32_as_bf16(a.reshape(-1), list(a.shape)) for a in (q, k, v, d_o))
        o = attention_gqa(tq, tk, tv, causal)
        dq, dk, dv = attention_gqa_backward(tdo, tq, tk, tv, o, causal)
        assert it_ctx.poll_status() == 0
        ro, rlse = ol.gqa_fwd(q, k, v, causal)
        rdq, rdk, rdv = ol.gqa_bwd(q, k, v, d_o, causal)
        tag = f"case {case}: B{B} S{S} H{H} Hkv{Hkv} D{D} causal={causal}"
        assert np.abs(o.lse.to_f32_host() - rlse).max() <= 1e-4, tag
        for got, want, name in ((o, ro, "O"), (dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
            # the 2e-2 bound on the absolute error is meant for values of order one: half a bf16 rounding step of an
            # entry of magnitude 8 is already 3e-2 (short causal rows give such entries), so tensors whose largest entry exceeds 2 are
            # brought to that range first; the relative L2 bounds are unaffected by the scaling
            scale = max(1.0, float(np.abs(want).max()) / 2.0)
            check_bf16(got.to_f32_host() / scale, want / scale, f"{tag} {name}")
