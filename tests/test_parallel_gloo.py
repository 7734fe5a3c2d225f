"""The multi-rank host logic on CPU: two gloo ranks. Tensor parallel: row ranges + all-gather give the
one-rank result bit for bit. Expert parallel: every expert has one owner, and the all-to-all dispatch and return
with the device's placement rule reproduce the one-rank layer output bit for bit. The tensor-parallel line exchange:
numbering, buffer choice and acceptance rule of the kernels, restated on the host."""
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
    """The all-to-all of the expert-parallel step with the placement rule of cn_ep_dispatch (`peer.ep_slots`): every rank
    routes its own tokens, sends each combo's row to the expert's owner in slot order, the owner computes and sends the
    result back to row `combo` of the source, and the source combines in pick order - bit for bit the one-rank result."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    from crownest_b200 import peer, synth
    hidden, inter, experts, k, tokens = 256, 256, 8, 3, 3
    rng = np.random.default_rng(5)
    rb = hidden // 64 * 36
    gu = [synth.nvfp4_matrix(2 * inter, hidden, rng) for _ in range(experts)]
    dn = [synth.nvfp4_matrix(hidden, inter, rng) for _ in range(experts)]
    x_all = rng.standard_normal((world, tokens, hidden)).astype(np.float32)
    logits_all = rng.standard_normal((world, tokens, experts)).astype(np.float32)
    x, logits = x_all[rank], logits_all[rank]
    ids, wts = oracle.route_softmax_topk(logits, k)
    cap = tokens * k

    def ffn(e, row):
        g, u = gu[e][: inter * rb], gu[e][inter * rb:]
        return oracle.nvfp4_ffn(g, u, dn[e], hidden, inter, [0.25, 0.25, 0.5], row[None], threads=1, path=0)[0]

    # dispatch: per destination the rows in slot order, padded to cap, with {expert, source combo}
    slots = peer.ep_slots(ids, experts, world)
    send_x = torch.zeros((world, cap, hidden))
    send_meta = torch.full((world, cap, 2), -1, dtype=torch.int64)
    for r, combos in enumerate(slots):
        for slot, c in enumerate(combos):
            e = int(ids.reshape(-1)[c])
            assert peer.ep_owner(e, experts, world) == r
            send_x[r, slot] = torch.from_numpy(x[c // k])
            send_meta[r, slot] = torch.tensor([e, int(c)])
    recv_x, recv_meta = torch.empty_like(send_x), torch.empty_like(send_meta)
    dist.all_to_all_single(recv_x, send_x)
    dist.all_to_all_single(recv_meta, send_meta)
    # the owner's experts over its inbox; every result goes back to row `source combo` of the source rank
    back = torch.zeros((world, cap, hidden))
    mine = 0
    for s_rank in range(world):
        for slot in range(cap):
            e, c = (int(v) for v in recv_meta[s_rank, slot])
            if e < 0:
                continue
            assert peer.ep_owner(e, experts, world) == rank
            back[s_rank, c] = torch.from_numpy(ffn(e, recv_x[s_rank, slot].numpy()))
            mine += 1
    ret = torch.empty_like(back)
    dist.all_to_all_single(ret, back)
    eo = ret.sum(0).numpy()  # every combo has exactly one owner: one non-zero contribution per row
    got = oracle.moe_acc_combo(eo, wts, None)
    ref = oracle.moe_acc_combo(np.stack([ffn(int(ids.reshape(-1)[c]), x[c // k]) for c in range(cap)]), wts, None)
    counts = torch.tensor([mine])
    dist.all_reduce(counts)
    owners = [peer.ep_owner(e, experts, world) for e in range(experts)]
    ok = (np.array_equal(got.view(np.uint32), ref.view(np.uint32)) and int(counts) == world * cap
          and all(owners.count(r) == experts // world for r in range(world))
          and all(list(ids.reshape(-1)[c]) == sorted(ids.reshape(-1)[c]) for c in slots))
    out.put((rank, "ok" if ok else f"expert-parallel exchange differs from the one-rank result (combos handled {int(counts)})"))
    dist.destroy_process_group()


def _lines_worker(rank, world, port, out):
    """The tensor-parallel line exchange on the host: every rank's slice of a vector travels as 16-byte lines that carry
    the exchange number into the buffer the kernels would pick; the receiver accepts a slice only when every half line
    carries the number it expects. Over several steps, with a vector exchanged an odd and an even number of times per
    step, the gathered vector equals the all-gather, a buffer still holding the previous exchange is never accepted, and
    a peer that is one exchange ahead writes into the other buffer."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from crownest_b200 import dense
    n = 64
    rng = np.random.default_rng(100 + rank)
    res = "ok"
    for per_step in (3, 4):
        bufs = [[np.zeros((world, n // world // 4, 4), np.uint32) for _ in range(2)] for _ in range(world)]  # [rank][buffer][source]
        tag, last_buf = 0, None
        for epoch in range(1, 4):
            tag = 0
            for occ in range(per_step):
                tag += 1
                number, buf = dense.line_number(epoch, tag), dense.line_buffer(epoch, occ, per_step)
                if buf == last_buf:
                    res = "two consecutive exchanges in one buffer"
                last_buf = buf
                mine = rng.integers(0, 1 << 16, n // world, dtype=np.uint16)
                lo, hi = dense.tp_rows(n, rank, world)
                # before the peers' lines arrive the buffer holds an older exchange (or zeros): never accepted
                stale = bufs[rank][buf][(rank + 1) % world]
                if dense.unpack_lines(stale, number) is not None:
                    res = "a stale buffer was accepted"
                lines = torch.from_numpy(dense.pack_lines(mine, number).astype(np.int64))
                everyone = [torch.zeros_like(lines) for _ in range(world)]
                dist.all_gather(everyone, lines)  # stands in for the stores into the peers' line buffers
                full = np.zeros(n, np.uint16)
                for src in range(world):
                    bufs[rank][buf][src] = everyone[src].numpy().astype(np.uint32)
                    got = mine if src == rank else dense.unpack_lines(bufs[rank][buf][src], number)
                    if got is None:
                        res = "a complete slice was refused"
                        got = np.zeros(n // world, np.uint16)
                    a, b = dense.tp_rows(n, src, world)
                    full[a:b] = got
                ref = [torch.zeros(n // world, dtype=torch.int32) for _ in range(world)]
                dist.all_gather(ref, torch.from_numpy(mine.astype(np.int32)))
                if not np.array_equal(full, torch.cat(ref).numpy().astype(np.uint16)):
                    res = f"gathered vector differs (per step {per_step}, step {epoch}, exchange {occ})"
                # a half-written line (the second half still from two exchanges ago) is not a line yet
                torn = bufs[rank][buf][(rank + 1) % world].copy()
                torn[0, 3] = dense.line_number(epoch - 1, tag) if epoch > 1 else 0
                if dense.unpack_lines(torn, number) is not None:
                    res = "a torn line was accepted"
    out.put((rank, res))
    dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_tp_worker, _ep_worker, _lines_worker])
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
