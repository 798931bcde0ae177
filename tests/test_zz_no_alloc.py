"""The allocation-free backward (it_flash_attention_bwd_noalloc) against the regular entry point.

Some hosts may not allocate device memory when they call into this library: a plugin running in a
sandboxed or real-time process that forbids cudaMalloc after start-up, or a caller that was handed
nothing but tensor pointers and a stream.  They cannot supply it_flash_attention_bwd's workspace,
so this variant keeps its scratch in a fixed array inside the library.  The test calls it through
the C ABI twice in a row (the array is shared and keeps the previous call's contents, so a second
call must not be disturbed by the first) and compares with the regular entry point.

Collected last on purpose, so that a run that stops at the first failure has already run
everything else.  It must pass on its own in a fresh process and after the other tests."""
import numpy as np
import pytest

import gpu_util as gu
from irontensor_b200 import _lib, raw, synth

pytestmark = pytest.mark.gpu


def _run(it_ctx, shape, bf16, causal, seed, check_no_alloc=False):
    import torch
    B, H, S, D = shape
    code = _lib.IT_BF16 if bf16 else _lib.IT_F32
    q, k, v, d_o = [t.reshape(B, H, S, D) for t in synth.attention_inputs(seed, B, H, S, D, bf16=bf16)]
    tq, tk, tv, tdo = (gu.to_dev(x, bf16) for x in (q, k, v, d_o))
    o = torch.empty_like(tq)
    lse = torch.empty((B, H, S), dtype=torch.float32, device="cuda")
    raw.fwd(code, B, H, S, D, causal, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), lse.data_ptr(), ctx=it_ctx)
    # regular entry point, caller-supplied workspace
    ref = [torch.full_like(tq, float("nan")) for _ in range(3)]
    n = raw.bwd_workspace_bytes(code, B, H, S, D)
    assert n <= _lib.IT_NOALLOC_SCRATCH_BYTES
    ws = torch.empty(n, dtype=torch.uint8, device="cuda")
    raw.bwd(code, B, H, S, D, causal, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), o.data_ptr(), tdo.data_ptr(),
            lse.data_ptr(), ref[0].data_ptr(), ref[1].data_ptr(), ref[2].data_ptr(), ws.data_ptr(), n, ctx=it_ctx)
    # allocation-free entry point: no workspace argument
    got = [torch.full_like(tq, float("nan")) for _ in range(3)]
    torch.cuda.synchronize()
    free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
    _lib.check(it_ctx.lib.it_flash_attention_bwd_noalloc(
        it_ctx.handle, it_ctx.stream(), code, B, H, S, D, int(causal), tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
        o.data_ptr(), tdo.data_ptr(), lse.data_ptr(), got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr()))
    assert it_ctx.poll_status() == 0
    if check_no_alloc:
        # The device's free memory (cudaMemGetInfo, which sees every allocation of the process, not only torch's)
        # is what it was before the call: nothing was allocated and kept, nor allocated and freed through torch.
        assert torch.cuda.memory_reserved() == reserved_before
        assert torch.cuda.mem_get_info()[0] == free_before
    return [gu.to_host(t) for t in ref], [gu.to_host(t) for t in got]


def test_noalloc_backward_matches_regular_entry_twice_in_a_row(it_ctx):
    # call 1: bf16 tensor-core path (scratch = fp32 dQ accumulator + two per-row arrays)
    # call 2: a different, smaller fp32 shape right after it, reusing the same built-in array
    # call 3: the first shape again, after the array was overwritten by call 2
    # The first call on a device may make the CUDA runtime load kernels; from the second call on the device's free
    # memory must not move at all.
    for i, (shape, bf16, causal, seed) in enumerate((((2, 4, 384, 64), True, True, 71), ((1, 3, 100, 40), False, False, 72),
                                                     ((2, 4, 384, 64), True, True, 71))):
        ref, got = _run(it_ctx, shape, bf16, causal, seed, check_no_alloc=(i > 0))
        for r, g, name in zip(ref, got, ("dQ", "dK", "dV")):
            assert not np.isnan(g).any(), name
            if bf16 and name == "dQ":
                # dQ tiles are summed with atomics; the order, and so the last bit, may differ
                assert np.abs(g - r).max() <= 2e-2, name
            else:
                assert np.array_equal(g, r), name


def test_noalloc_backward_at_the_edge_of_its_scratch(it_ctx):
    """A shape whose scratch need is exactly the built-in array runs and matches the regular entry point; one
    that needs 256 bytes more (the next step of the workspace granularity) is refused."""
    import torch
    B, H, S, D = 512, 64, 64, 8          # bf16, short rows: scratch = one fp32 per row = 512*64*64*4 bytes = 8 MiB
    assert raw.bwd_workspace_bytes(_lib.IT_BF16, B, H, S, D) == _lib.IT_NOALLOC_SCRATCH_BYTES
    ref, got = _run(it_ctx, (B, H, S, D), True, True, 73)
    for r, g, name in zip(ref, got, ("dQ", "dK", "dV")):
        assert not np.isnan(g).any(), name
        assert np.array_equal(g, r), name
    B, H = 1, 32769                       # 64 rows more
    assert raw.bwd_workspace_bytes(_lib.IT_BF16, B, H, S, D) == _lib.IT_NOALLOC_SCRATCH_BYTES + 256
    p = torch.zeros(64, dtype=torch.bfloat16, device="cuda").data_ptr()
    rc = it_ctx.lib.it_flash_attention_bwd_noalloc(it_ctx.handle, it_ctx.stream(), _lib.IT_BF16, B, H, S, D, 1,
                                                   p, p, p, p, p, p, p, p, p)
    assert rc == _lib.IT_ERR_UNSUPPORTED_SHAPE


def test_noalloc_backward_rejects_shapes_beyond_its_scratch(it_ctx):
    import torch
    B, H, S, D = 4, 16, 8192, 128       # needs 256 MiB of scratch
    p = torch.zeros(64, dtype=torch.bfloat16, device="cuda").data_ptr()
    rc = it_ctx.lib.it_flash_attention_bwd_noalloc(it_ctx.handle, it_ctx.stream(), _lib.IT_BF16, B, H, S, D, 1,
                                                   p, p, p, p, p, p, p, p, p)
    assert rc == _lib.IT_ERR_UNSUPPORTED_SHAPE
    msg = it_ctx.lib.it_last_error()
    assert b"scratch" in msg and str(_lib.IT_NOALLOC_SCRATCH_BYTES).encode() in msg
    assert it_ctx.poll_status() == 0
