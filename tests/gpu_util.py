"""Helpers for the GPU parity tests: run the C ABI on torch-held device memory, compare with the oracle."""
import ctypes

import numpy as np

from irontensor_b200 import _lib, raw, synth


def to_dev(a, bf16):
    import torch
    a = np.ascontiguousarray(a, dtype=np.float32)
    if bf16:
        bits = synth.f32_to_bf16_bits(a.reshape(-1)).view(np.int16)
        return torch.from_numpy(bits).cuda().view(torch.bfloat16).view(a.shape)
    return torch.from_numpy(a).cuda()


def to_host(t):
    import torch
    if t.dtype == torch.bfloat16:
        bits = t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        return synth.bf16_bits_to_f32(bits.reshape(-1)).reshape(tuple(t.shape))
    return t.cpu().numpy()


def run_fwd(ctx, q, k, v, causal=True, bf16=False, poison=True):
    """q,k,v: numpy [B,H,S,D] fp32 (already bf16-representable when bf16).  Returns (O, LSE) as numpy fp32."""
    import torch
    B, H, S, D = q.shape
    dq, dk, dv = (to_dev(x, bf16) for x in (q, k, v))
    o = torch.empty_like(dq)
    lse = torch.empty((B, H, S), dtype=torch.float32, device="cuda")
    if poison:   # every element must be overwritten by the kernel
        o.fill_(float("nan"))
        lse.fill_(float("nan"))
    raw.fwd(_lib.IT_BF16 if bf16 else _lib.IT_F32, B, H, S, D, causal, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            o.data_ptr(), lse.data_ptr(), ctx=ctx)
    assert ctx.poll_status() == 0
    return to_host(o), lse.cpu().numpy()


def run_fwd_bwd(ctx, q, k, v, d_o, causal=True, bf16=False):
    """Forward then backward through the C ABI.  Returns (O, LSE, dQ, dK, dV) as numpy fp32."""
    import torch
    B, H, S, D = q.shape
    code = _lib.IT_BF16 if bf16 else _lib.IT_F32
    tq, tk, tv, tdo = (to_dev(x, bf16) for x in (q, k, v, d_o))
    o = torch.full_like(tq, float("nan"))
    lse = torch.full((B, H, S), float("nan"), dtype=torch.float32, device="cuda")
    raw.fwd(code, B, H, S, D, causal, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), lse.data_ptr(), ctx=ctx)
    g = [torch.full_like(tq, float("nan")) for _ in range(3)]
    nbytes = raw.bwd_workspace_bytes(code, B, H, S, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    raw.bwd(code, B, H, S, D, causal, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), tdo.data_ptr(),
            lse.data_ptr(), g[0].data_ptr(), g[1].data_ptr(), g[2].data_ptr(), ws.data_ptr(), nbytes, ctx=ctx)
    assert ctx.poll_status() == 0
    return (to_host(o), lse.cpu().numpy()) + tuple(to_host(x) for x in g)


def err_stats(got, want):
    """max-abs error, relative L2 error, and the relative L2 error that rounding `want` to bf16
    alone would give (the floor for any bf16-stored result)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    nrm = np.linalg.norm(want) + 1e-300
    floor = np.linalg.norm(synth.round_bf16(want.astype(np.float32)).astype(np.float64) - want) / nrm
    return float(np.abs(got - want).max()), float(np.linalg.norm(got - want) / nrm), float(floor)
