"""The multi-rank host logic on CPU: two gloo ranks. Tensor parallel: row ranges + all-gather give the
one-rank result bit for bit. Expert parallel: every expert has one owner, and the ranks' partial sums
add up to the one-rank layer output."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT

sys.path.insert(0, ROOT)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from crownest_b200 import dense, synth
    rows, k = 96, 512
    rng = np.random.default_rng(11)
    w = synth.nvfp4_matrix(rows, k, rng)
    rb = k // 64 * 36
    for m in (1, 3):
        x = rng.standard_normal((m, k)).astype(np.float32)
        lo, hi = dense.tp_rows(rows, rank, world)
        part = oracle.nvfp4_gemv(w[lo * rb:hi * rb], hi - lo, k, 0.5, x, threads=1, path=0)
        full = torch.zeros((m, rows), dtype=torch.float32)
        dense.gather_rows(torch.from_numpy(np.ascontiguousarray(part)), full, m, world)
        ref = oracle.nvfp4_gemv(w, rows, k, 0.5, x, threads=1, path=0)
        if not np.array_equal(full.numpy().view(np.uint32), ref.view(np.uint32)):
            out.put((rank, f"tp gather differs at m={m}"))
            dist.destroy_process_group()
            return
    out.put((rank, "ok"))
    dist.destroy_process_group()


def _ep_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from crownest_b200 import synth, workloads
    hidden, inter, experts, k, tokens_per_rank = 256, 256, 8, 3, 2
    rng = np.random.default_rng(5)
    rb = hidden // 64 * 36
    gu = [synth.nvfp4_matrix(2 * inter, hidden, rng) for _ in range(experts)]
    dn = [synth.nvfp4_matrix(hidden, inter, rng) for _ in range(experts)]
    # dispatch: every rank's rows and logits, gathered (the same generator on both ranks stands in for the exchange)
    x_all = rng.standard_normal((world * tokens_per_rank, hidden)).astype(np.float32)
    logits_all = rng.standard_normal((world * tokens_per_rank, experts)).astype(np.float32)
    mine_x = torch.from_numpy(x_all[rank * tokens_per_rank:(rank + 1) * tokens_per_rank].copy())
    got = torch.empty((world * tokens_per_rank, hidden))
    dist.all_gather_into_tensor(got, mine_x)
    assert np.array_equal(got.numpy(), x_all)
    ids, wts = oracle.route_softmax_topk(logits_all, k)
    tokens = x_all.shape[0]

    def expert_out(c):
        e = ids.reshape(-1)[c]
        g, u = gu[e][: inter * rb], gu[e][inter * rb:]
        return oracle.nvfp4_ffn(g, u, dn[e], hidden, inter, [0.25, 0.25, 0.5], x_all[c // k: c // k + 1], threads=1, path=0)[0]

    ye = np.zeros((tokens * k, hidden), np.float32)
    w_local = wts.copy()
    for c in range(tokens * k):
        if workloads.ep_owner(int(ids.reshape(-1)[c]), experts, world) == rank:
            ye[c] = expert_out(c)
        else:
            w_local.reshape(-1)[c] = 0.0  # a null table entry: the combo adds nothing on this rank
    part = torch.from_numpy(oracle.moe_acc_combo(ye, w_local, None))
    dist.all_reduce(part)  # combine (gloo has no reduce-scatter: all-reduce, then the rank's own rows)
    own = part[rank * tokens_per_rank:(rank + 1) * tokens_per_rank].numpy()
    ye_full = np.stack([expert_out(c) for c in range(tokens * k)])
    ref = oracle.moe_acc_combo(ye_full, wts, None)[rank * tokens_per_rank:(rank + 1) * tokens_per_rank]
    err = np.linalg.norm(own - ref) / np.linalg.norm(ref)
    owners = [workloads.ep_owner(e, experts, world) for e in range(experts)]
    ok = err < 1e-6 and sorted(set(owners)) == list(range(world)) and all(owners.count(r) == experts // world for r in range(world))
    out.put((rank, "ok" if ok else f"ep combine rel err {err}, owners {owners}"))
    dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_tp_worker, _ep_worker])
def test_two_gloo_ranks(worker):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(res) == [(0, "ok"), (1, "ok")], res
