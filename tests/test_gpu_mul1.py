"""Parity of the CUDA MUL1 (EXL3 trellis) path with the CPU checker: bit-exact decoded weights,
GEMV / FFN / MoE outputs within rel L2 <= 1e-3 of the exact-order f32 CPU reference."""
import hashlib
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from conftest import GOLDEN
from crownest_b200 import moe, mul1, ops, synth
from oracle import testkit as tk
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16

dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("K,k,n", [(3.0, 256, 128), (2.0, 384, 256), (3.5, 256, 128), (4.0, 128, 128), (8.0, 64, 64), (1.5, 64, 32)])
def test_decoded_weights_are_bit_exact(K, k, n):
    rng = np.random.default_rng(int(K * 10))
    tr = rng.integers(0, 65536, size=oracle.mul1_trellis_bytes(k, n, K) // 2, dtype=np.uint16)
    got = mul1.reconstruct(dev(tr.view(np.int16)), k, n, K).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.mul1_reconstruct(tr, k, n, K))


def test_quantizer_record_decodes_to_the_exllamav3_digest():
    # the reference's golden: sha256 of exllamav3's own reconstruct output (converter/tests/fixtures)
    for line in open(os.path.join(GOLDEN, "exl3-mul1-decode.tsv")):
        if not line.startswith("q-k3\t"):
            continue
        f = line.rstrip("\n").split("\t")
        hidden, inter = int(f[3]), int(f[4])
        raw = np.fromfile(os.path.join(GOLDEN, f[1]), np.uint8)
        tb = oracle.mul1_trellis_bytes(hidden, inter, 3.0)
        for i, (k, n) in enumerate([(hidden, inter), (hidden, inter), (inter, hidden)]):
            tr = raw[i * tb:(i + 1) * tb].view(np.int16)
            got = mul1.reconstruct(dev(tr), k, n, 3.0).cpu().numpy()
            assert hashlib.sha256(got.tobytes()).hexdigest() == f[5 + i]


def expert_parts(rec, hidden, inter, K):
    tb = oracle.mul1_trellis_bytes(hidden, inter, K)
    at, out = 3 * tb, []
    for nbytes in (2 * hidden, 2 * inter, 2 * hidden, 2 * inter, 2 * inter, 2 * hidden):
        out.append(rec[at:at + nbytes].view(np.uint16))
        at += nbytes
    return tb, out


@pytest.mark.parametrize("K,hidden,inter", [(3.0, 512, 256), (3.0, 4096, 1536), (2.0, 256, 384), (3.5, 256, 128), (4.0, 128, 256)])
@pytest.mark.parametrize("t", [1, 3])
def test_gemv_matches_the_cpu_reference(K, hidden, inter, t):
    rec = tk.mul1_record(7, hidden, inter, K)
    tb, (gs, gv, us, uv, ds, dv) = expert_parts(rec, hidden, inter, K)
    rng = np.random.default_rng(2)
    slots = 2
    d_rec = [dev(rec), dev(rec.copy())]
    ptrs = torch.tensor([r.data_ptr() for r in d_rec], dtype=torch.int64, device="cuda")
    plan = mul1.Mul1Plan(hidden, inter, K, slots=slots, tokens=t)
    for which, (k, n, tro, su, sv) in enumerate([(hidden, inter, 0, gs, gv), (hidden, inter, tb, us, uv), (inter, hidden, 2 * tb, ds, dv)]):
        x = rng.uniform(-2, 2, size=(slots, t, k)).astype(np.float32)
        y = plan.run_slots(which, ptrs, dev(x)).cpu().numpy()
        for s in range(slots):
            ref = oracle.mul1_gemv(rec[tro:tro + tb], su, sv, k, n, K, x[s], threads=8)
            check_close(y[s], ref, f"mul1 gemv K={K} which={which} slot {s}", bf16_out=False)
    plan.free()


def test_null_slots_are_skipped_and_rows_are_batch_invariant():
    hidden, inter, K = 512, 256, 3.0
    rec = dev(tk.mul1_record(3, hidden, inter, K))
    plan = mul1.Mul1Plan(hidden, inter, K, slots=3, tokens=4)
    x = torch.randn((3, 4, hidden), device="cuda")
    ptrs = torch.tensor([rec.data_ptr(), 0, rec.data_ptr()], dtype=torch.int64, device="cuda")
    y = torch.full((3, 4, inter), float("nan"), device="cuda")
    plan.run_slots(0, ptrs, x, y)
    assert torch.isnan(y[1]).all() and torch.isfinite(y[0]).all() and torch.isfinite(y[2]).all()
    # one row at a time gives the same bits as four rows at once
    one = mul1.Mul1Plan(hidden, inter, K, slots=1, tokens=1)
    for t in range(4):
        y1 = one.run_slots(0, ptrs[:1], x[0, t:t + 1].contiguous())
        assert torch.equal(y1.view(torch.int32).reshape(-1), y[0, t].view(torch.int32))
    plan.free(), one.free()


@pytest.mark.parametrize("limit", [0.0, 10.0])
def test_expert_ffn_matches_the_cpu_reference(limit):
    hidden, inter, K = 1024, 512, 3.0
    recs = [tk.mul1_record(20 + i, hidden, inter, K) for i in range(3)]
    d = [dev(r) for r in recs]
    ptrs = torch.tensor([r.data_ptr() for r in d], dtype=torch.int64, device="cuda")
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((3, 2, hidden)) * 0.3).astype(np.float32)
    plan = mul1.Mul1Plan(hidden, inter, K, slots=3, tokens=2)
    y = plan.ffn(ptrs, dev(x), limit=limit).cpu().numpy()
    for s in range(3):
        ref = oracle.mul1_expert_ffn(recs[s], hidden, inter, K, x[s], limit=limit, threads=8)
        check_close(y[s], ref, f"mul1 ffn slot {s}", bf16_out=False)
    plan.free()


@pytest.mark.parametrize("tokens", [1, 4, 16])
def test_moe_step_over_mul1_experts_matches_the_cpu_reference(tokens):
    # the benchmark's EXL3 shape: hidden 4096 <-> inter 1536, 64 experts, top-4, K = 3. Only the experts the routing picks
    # get a record (4 / ~15 / ~41 of them); the other table entries are null and nothing may touch them
    hidden, inter, K, experts, topk = 4096, 1536, 3.0, 64, 4
    rng = np.random.default_rng(40 + tokens)
    xb, xf = synth.activations(tokens, hidden, rng)
    xf = (xf * np.float32(0.25)).astype(np.float32)
    xb = synth.bf16_bits(xf)
    xf = synth.bf16_to_f32(xb)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    ids, wts = moe.route_softmax_topk(dev(logits), topk)
    rids, rw = oracle.route_softmax_topk(logits, topk)
    assert np.array_equal(ids.cpu().numpy(), rids)
    picked = sorted(set(int(e) for e in rids.reshape(-1)))
    recs = {e: tk.mul1_record(0x1640 + 9 * e, hidden, inter, K) for e in picked}
    d = {e: dev(r) for e, r in recs.items()}
    table = torch.tensor([d[e].data_ptr() if e in d else 0 for e in range(experts)], dtype=torch.int64, device="cuda")
    plan = mul1.Mul1Plan(hidden, inter, K, slots=tokens * topk, tokens=1)
    y = plan.moe(table, ids, wts, to_dev_bf16(xb), limit=10.0)
    ye = np.zeros((tokens * topk, hidden), np.float32)
    for c in range(tokens * topk):
        ye[c] = oracle.mul1_expert_ffn(recs[rids.reshape(-1)[c]], hidden, inter, K, xf[c // topk: c // topk + 1], limit=10.0, threads=8)[0]
    ref = oracle.moe_combine(ye, rw, None)
    # f32 in / out: the 1e-3 contract proper
    yf = plan.moe(table, ids, wts, dev(xf), limit=10.0)
    check_close(yf.cpu().numpy(), ref, f"mul1 moe f32 tokens={tokens}", bf16_out=False)
    # bf16 in / out (ulp taken no lower than rms / 64: the combine cancels)
    check_close(from_dev_bf16(y), ref, f"mul1 moe tokens={tokens}", ulp_floor=1.0 / 64)
    plan.free()


@pytest.mark.parametrize("tokens,experts,topk", [(32, 6, 3), (40, 5, 4), (10, 6, 3)])
def test_moe_step_with_bundled_rows_matches_the_cpu_reference(tokens, experts, topk):
    """At least two combo slots per expert: the combos are sorted by expert and run as groups of up to four rows that share
    one decode of the expert (one, two, three and four-row groups and unused row slots all occur)."""
    hidden, inter, K = 1024, 512, 3.0
    rng = np.random.default_rng(7 + tokens)
    recs = [tk.mul1_record(0x2000 + 5 * e, hidden, inter, K) for e in range(experts)]
    d = [dev(r) for r in recs]
    table = torch.tensor([r.data_ptr() for r in d], dtype=torch.int64, device="cuda")
    x = (rng.standard_normal((tokens, hidden)) * 0.25).astype(np.float32)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    ids, wts = moe.route_softmax_topk(dev(logits), topk)
    rids, rw = oracle.route_softmax_topk(logits, topk)
    assert np.array_equal(ids.cpu().numpy(), rids)
    plan = mul1.Mul1Plan(hidden, inter, K, slots=tokens * topk, tokens=1)
    y = plan.moe(table, ids, wts, dev(x), limit=10.0)
    ye = np.zeros((tokens * topk, hidden), np.float32)
    for c in range(tokens * topk):
        ye[c] = oracle.mul1_expert_ffn(recs[rids.reshape(-1)[c]], hidden, inter, K, x[c // topk: c // topk + 1], limit=10.0, threads=8)[0]
    ref = oracle.moe_combine(ye, rw, None)
    check_close(y.cpu().numpy(), ref, f"mul1 moe bundled tokens={tokens}", bf16_out=False)
    y2 = plan.moe(table, ids, wts, dev(x), limit=10.0)
    assert torch.equal(y.view(torch.int32), y2.view(torch.int32))
    plan.free()
