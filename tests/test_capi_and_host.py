"""CPU tests of the boundary and host logic: the C-ABI library loads and exports everything the
header declares, sharding covers every slice once, and the N>1 timing reduction works (gloo)."""
import os
import re
import subprocess
import sys
import textwrap

import pytest

from irontensor_b200 import _lib
from irontensor_b200.sharding import shard_range

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    with open(os.path.join(ROOT, "include", "irontensor_b200.h")) as f:
        return set(re.findall(r"(?:it_status|const char\*)\s+(it_[a-z0-9_]+)\s*\(", f.read()))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = declared_symbols()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(_lib.SIGNATURES) | {"it_last_error"} == declared


def test_argument_checks_that_need_no_gpu():
    import ctypes
    lib = _lib.load()
    n = ctypes.c_size_t()
    assert lib.it_flash_attention_bwd_workspace_bytes(_lib.IT_BF16, 4, 16, 8192, 128, ctypes.byref(n)) == _lib.IT_OK
    # dQ accumulator + two padded per-row arrays
    assert n.value >= 64 * 8192 * 128 * 4 + 2 * 64 * 8192 * 4
    assert lib.it_flash_attention_bwd_workspace_bytes(_lib.IT_F32, 2, 2, 100, 64, ctypes.byref(n)) == _lib.IT_OK
    assert n.value >= 2 * 2 * 100 * 4
    assert lib.it_flash_attention_bwd_workspace_bytes(_lib.IT_F32, 2, 2, 100, 129, ctypes.byref(n)) == _lib.IT_ERR_UNSUPPORTED_SHAPE
    assert lib.it_flash_attention_bwd_workspace_bytes(9, 2, 2, 100, 64, ctypes.byref(n)) == _lib.IT_ERR_PRECISION
    assert lib.it_flash_attention_bwd_workspace_bytes(_lib.IT_F32, 2, 2, 100, 64, None) == _lib.IT_ERR_INVALID_ARG
    assert b"null" in lib.it_last_error()
    assert lib.it_stream_sync(None, None) == _lib.IT_ERR_INVALID_ARG


def test_no_device_means_error_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import ctypes
    h = ctypes.c_void_p()
    assert _lib.load().it_ctx_create(0, ctypes.byref(h)) == _lib.IT_ERR_CUDA
    from irontensor_b200 import Tensor
    with pytest.raises(RuntimeError, match="no fallback"):
        Tensor.zeros([1, 1, 4, 8])


@pytest.mark.parametrize("n,world", [(64, 1), (64, 2), (64, 8), (384, 8), (6, 4), (3, 8), (0, 4)])
def test_shard_ranges_partition_the_slices(n, world):
    seen = []
    for r in range(world):
        b0, b1 = shard_range(n, world, r)
        assert 0 <= b0 <= b1 <= n
        seen.extend(range(b0, b1))
    assert seen == list(range(n))
    if n == 6 and world == 4:
        assert [shard_range(6, 4, r) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 6)]
    with pytest.raises(ValueError):
        shard_range(n, world, world)


def test_product_code_does_not_touch_the_oracle():
    """Nothing under irontensor_b200/ may import, load or call the CPU checker."""
    pkg = os.path.join(ROOT, "irontensor_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                with open(os.path.join(dirpath, fn)) as f:
                    text = f.read()
                assert "oracle" not in text.lower(), f"{fn} mentions the oracle"


def test_two_rank_max_reduction_over_gloo(tmp_path):
    """The N>1 bench path: ranks take disjoint shards, the reported time is the max over ranks."""
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch, torch.distributed as dist
        from irontensor_b200.sharding import shard_range
        dist.init_process_group("gloo")
        r, w = dist.get_rank(), dist.get_world_size()
        b0, b1 = shard_range(64, w, r)
        t = torch.tensor([float(10 + 5 * r), float(b1 - b0)], dtype=torch.float64)
        mx = t.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        assert mx[0].item() == 10 + 5 * (w - 1) and sm[1].item() == 64
        dist.barrier()
        if r == 0: print("OK", mx[0].item())
        dist.destroy_process_group()
    """))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "OK 15.0" in out.stdout
