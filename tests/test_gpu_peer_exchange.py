"""Two ranks on two GPUs: the peer-memory exchange of the tensor-parallel stack gives the bits of the NCCL all-gather
path, replay after replay. Skipped where fewer than two GPUs are visible."""
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


def _worker(rank, world, port, out, protocol):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from crownest_b200 import _lib, dense
    res = "ok"
    try:
        # the fused form once with the QKV output exchanged too (four exchanges per layer), else with q kept local
        gq = protocol == "peer-lines"
        a = dense.DenseStack(layers=3, device=f"cuda:{rank}", seed=5, rank=rank, world=world, exchange="nccl", gather_q=gq)
        b = dense.DenseStack(layers=3, device=f"cuda:{rank}", seed=5, rank=rank, world=world, exchange=protocol, gather_q=gq)
        assert b.peer is not None
        x = torch.randn((1, a.hidden), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
        a.x.copy_(x), b.x.copy_(x)
        ya = a.run_layers(1).clone()
        b.capture(1)
        for it in range(3):
            b.graph.replay()
            torch.cuda.synchronize()
            for name in ("q", "o", "h", "y"):
                va, vb = getattr(a, name), getattr(b, name)
                if name in a.local_only:  # not exchanged: every rank holds its own slice only
                    lo, hi = dense.tp_rows(va.shape[1], rank, world)
                    va, vb = va[:, lo:hi].contiguous(), vb[:, lo:hi].contiguous()
                if not torch.equal(va.view(torch.int16), vb.view(torch.int16)):
                    res = f"replay {it}: vector {name} differs from the all-gather path"
            # a rank's copy of a peer's slice lives until that peer's next exchange of the vector: nobody starts the next
            # replay before everybody has looked at this one
            dist.barrier()
        if not torch.equal(ya.view(torch.int16), b.y.view(torch.int16)):
            res = "output differs"
        if _lib.device_status() != 0:
            res = f"device status {_lib.device_status()}"
    except Exception as e:  # noqa: BLE001 - reported to the parent
        res = f"{type(e).__name__}: {e}"
    out.put((rank, res))
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


# lines stored by the GEMV itself / lines pushed by the exchange kernel / data followed by a flag
@pytest.mark.parametrize("protocol", ["peer", "peer-lines", "peer-flags"])
def test_peer_exchange_matches_the_all_gather(protocol):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, protocol)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
