"""Two ranks on two GPUs: the expert-parallel step (all-to-all dispatch and return over peer memory) gives, for each
rank's tokens, the output of the one-GPU step over the same experts - the same bits where both take the same kernels,
within 2 bf16 ulp where the one-GPU step is small enough for the ungrouped kernels - and the same bits run after run
and under graph replay. Skipped where
fewer than two GPUs are visible. NVLS is off and only plain peer stores are used."""
import os
import socket
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from crownest_b200 import _lib, workloads
    res = "ok"
    try:
        dev = f"cuda:{rank}"
        for name, cls, kw, tokens in (("nvfp4", workloads.MoeDecode, dict(experts=64, topk=6), 8), ("nvfp4-64", workloads.MoeDecode, dict(experts=64, topk=6), 64),
                                      ("mul1", workloads.Mul1MoeDecode, dict(experts=8, topk=4, hidden=1024, inter=512), 5)):
            ep = cls(tokens, device=dev, rank=rank, world=world, **kw)
            one = cls(tokens, device=dev, rank=0, world=1, **kw)  # every expert on this GPU
            one.x.copy_(ep.x), one.logits.copy_(ep.logits)
            want = one.step().clone()
            got = ep.step().clone()
            torch.cuda.synchronize()
            g32, w32 = got.float(), want.float()
            rel = float((g32 - w32).norm() / w32.norm())
            at = torch.maximum(w32.abs(), w32.pow(2).mean().sqrt() / 64)
            ulps = float(((g32 - w32).abs() / torch.exp2(torch.floor(torch.log2(at)) - 7)).max())
            if rel > 1e-3 or ulps > 2:
                res = f"{name}: expert-parallel output differs from the one-GPU step (rel L2 {rel:.3e}, {ulps:.1f} bf16 ulp)"
                break
            want = got
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    ep.step()
            for it in range(3):
                ep.y.zero_()
                g.replay()
                torch.cuda.synchronize()
                if not torch.equal(ep.y.view(torch.int16), want.view(torch.int16)):
                    res = f"{name}: replay {it} differs"
            if _lib.device_status() != 0:
                res = f"{name}: device status"
            if res != "ok":
                break
            del g
    except Exception as e:  # noqa: BLE001 - reported to the parent
        import traceback
        res = f"{type(e).__name__}: {e} {traceback.format_exc()[-600:]}"
    out.put((rank, res))
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


def test_expert_parallel_step_matches_the_one_gpu_step():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
