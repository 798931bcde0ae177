"""Tests that need two GPUs on the box (skipped otherwise): the projection GEMM whose epilogue does the reduce-scatter
over peer memory, against the same product summed by an NCCL all-reduce.  Ranks are child processes under torchrun."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _gpus():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("world", [2, 4])
def test_gemm_with_fused_reduce_scatter_equals_all_reduce(tmp_path, world):
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "rs.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import torch, torch.distributed as dist
        from irontensor_b200 import context, raw
        from irontensor_b200.sharding import SummedProjection
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        try:
            ctx = context(rank)
            for kind, n, in_dim, out_dim in ((0, 1024, 256, 512), (1, 2048, 384, 640), (0, 512 * world, 64, 128)):
                k_dim, width = (in_dim, out_dim) if kind == 0 else (out_dim, in_dim)
                gen = torch.Generator(device="cuda").manual_seed(100 + rank)      # every rank has its own partial
                a = torch.randn((n, k_dim), generator=gen, device="cuda").to(torch.bfloat16)
                w = (torch.randn((out_dim, in_dim), generator=gen, device="cuda") * 0.1).to(torch.bfloat16)
                sp = SummedProjection(n, width)
                got = sp.run(kind, a.data_ptr(), w.data_ptr(), in_dim, out_dim).clone()
                ctx.poll_status()
                # reference: the exact partial in fp64, summed over ranks in fp64
                part = (a.double() @ (w.double().t() if kind == 0 else w.double()))
                dist.all_reduce(part)
                err = (got.double() - part).norm() / part.norm()
                assert err < 6e-3, (kind, n, float(err))
                # every rank holds the same bits
                mine = got.view(torch.int16).to(torch.int64).sum()
                lo, hi = mine.clone(), mine.clone()
                dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                assert lo.item() == hi.item()
                # a second run on the same buffer starts from zero again
                got2 = sp.run(kind, a.data_ptr(), w.data_ptr(), in_dim, out_dim)
                assert ((got2.double() - part).norm() / part.norm()) < 6e-3
                del sp
            dist.barrier()
            torch.cuda.synchronize()
            if rank == 0:
                print("OK")
        finally:
            dist.destroy_process_group()
    """))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "OK" in out.stdout
