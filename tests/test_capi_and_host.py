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
    assert set(_lib.SIGNATURES) | {"it_last_error", "it_ctx_kernel_tag"} == declared


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


def test_head_shards_keep_groups_together():
    from irontensor_b200.sharding import head_shard, qkv_weight_rows
    for H, Hkv, W in ((16, 16, 4), (32, 8, 8), (12, 4, 3), (8, 2, 4), (6, 3, 2)):
        seen_q, seen_kv = [], []
        for r in range(W):
            qb, qe, kb, ke = head_shard(H, Hkv, W, r)
            assert (qe - qb) == (ke - kb) * (H // Hkv)
            for h in range(qb, qe):
                assert kb <= h // (H // Hkv) < ke          # the K/V head a query head reads is on the same rank
            seen_q += list(range(qb, qe))
            seen_kv += list(range(kb, ke))
            (q0, q1), (k0, k1), (v0, v1) = qkv_weight_rows(H, Hkv, 64, W, r)
            assert (q0, q1, k0, k1) == (qb * 64, qe * 64, kb * 64, ke * 64) and (v0, v1) == (k0, k1)
        assert seen_q == list(range(H)) and seen_kv == list(range(Hkv))
    with pytest.raises(ValueError):
        head_shard(10, 4, 2, 0)


def test_head_parallel_projections_sum_to_the_full_layer_over_gloo(tmp_path):
    """Two ranks, heads split between them: each projects with its rows of Wq/Wk/Wv, attends over its heads, multiplies by
    its columns of Wo, and the all-reduce of the partial outputs equals the unsharded layer (fp64 on CPU; the GPU
    kernels are exercised by the gpu tests, this covers the sharding arithmetic and the one collective)."""
    script = tmp_path / "tp.py"
    script.write_text(textwrap.dedent(f"""
        import sys
        sys.path.insert(0, {ROOT!r})
        import numpy as np, torch, torch.distributed as dist
        from irontensor_b200.sharding import head_shard, qkv_weight_rows, out_projection_all_reduce
        dist.init_process_group("gloo")
        r, w = dist.get_rank(), dist.get_world_size()
        S, hidden, H, Hkv, D = 12, 32, 4, 2, 8
        rng = np.random.default_rng(3)                      # same data on every rank
        x = rng.standard_normal((S, hidden)); wq = rng.standard_normal((H * D, hidden)); wk = rng.standard_normal((Hkv * D, hidden))
        wv = rng.standard_normal((Hkv * D, hidden)); wo = rng.standard_normal((hidden, H * D))
        def attend(q, k, v):                                # q [S,h,D], k/v [S,hk,D], causal, grouped
            g = q.shape[1] // k.shape[1]
            out = np.zeros_like(q)
            for h in range(q.shape[1]):
                s = q[:, h] @ k[:, h // g].T / np.sqrt(D)
                s = np.where(np.tril(np.ones((S, S), bool)), s, -np.inf)
                p = np.exp(s - s.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
                out[:, h] = p @ v[:, h // g]
            return out
        full = attend((x @ wq.T).reshape(S, H, D), (x @ wk.T).reshape(S, Hkv, D), (x @ wv.T).reshape(S, Hkv, D)).reshape(S, H * D) @ wo.T
        (q0, q1), (k0, k1), (v0, v1) = qkv_weight_rows(H, Hkv, D, w, r)
        qb, qe, kb, ke = head_shard(H, Hkv, w, r)
        mine = attend((x @ wq[q0:q1].T).reshape(S, qe - qb, D), (x @ wk[k0:k1].T).reshape(S, ke - kb, D),
                      (x @ wv[v0:v1].T).reshape(S, ke - kb, D)).reshape(S, (qe - qb) * D)
        partial = torch.from_numpy(mine @ wo[:, q0:q1].T)
        total = out_projection_all_reduce(partial)
        assert np.abs(total.numpy() - full).max() < 1e-10
        dist.barrier()
        if r == 0: print("OK")
        dist.destroy_process_group()
    """))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                         capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "OK" in out.stdout


def test_workspace_size_functions_of_the_widened_rows():
    import ctypes
    lib = _lib.load()
    n = ctypes.c_size_t()
    assert lib.it_attention_decode_workspace_bytes(32, 32, 128, ctypes.byref(n)) == _lib.IT_OK
    assert n.value >= 32 * 32 * 64 * (128 + 2) * 4                    # 64 splits of (D + 2) floats per (batch, head)
    assert lib.it_attention_decode_workspace_bytes(1, 1, 129, ctypes.byref(n)) == _lib.IT_ERR_UNSUPPORTED_SHAPE
    assert lib.it_attention_decode_workspace_bytes(1, 1, 64, None) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_qkv_rope_workspace_bytes(8192, 128, ctypes.byref(n)) == _lib.IT_OK
    assert n.value >= 8192 * 64 * 8                                   # one (cos, sin) pair per position and dimension pair
    assert lib.it_qkv_rope_workspace_bytes(16, 63, ctypes.byref(n)) == _lib.IT_ERR_INVALID_ARG
    # entry points that need a context refuse a null one before touching the GPU
    assert lib.it_linear_fwd(None, None, 8, 8, 8, None, None, None) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_rope_qk(None, None, _lib.IT_F32, 1, 1, 1, 1, 8, 10000.0, 0, 0, None, None, None, None) == _lib.IT_ERR_INVALID_ARG
    assert lib.it_attention_decode(None, None, _lib.IT_BF16, 1, 1, 1, 64, 1, 1, None, None, None, None, None, None, 0) == _lib.IT_ERR_INVALID_ARG
