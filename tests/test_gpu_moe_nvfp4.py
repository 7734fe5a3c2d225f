"""Parity of the routers and of the routed NVFP4 expert step (through the C ABI) with the CPU checker:
routing indices bit-exact, layer outputs within rel L2 <= 1e-3 / 2 bf16 ulp of the f32 reference."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import moe, ops, synth
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16


@pytest.mark.parametrize("tokens,experts,k", [(1, 512, 10), (8, 512, 10), (64, 512, 10), (16, 64, 4), (5, 288, 8), (3, 7, 3)])
def test_softmax_router_indices_are_bit_exact(tokens, experts, k):
    rng = np.random.default_rng(experts + tokens)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    if tokens > 2:
        logits[1, experts - 1] = logits[1, 0] = logits[1].max() + 1  # a tie at the top: lowest index first
    ids, w = moe.route_softmax_topk(torch.from_numpy(logits).cuda(), k)
    rids, rw = oracle.route_softmax_topk(logits, k)
    assert np.array_equal(ids.cpu().numpy(), rids)
    assert np.max(np.abs(w.cpu().numpy() - rw)) <= 1e-6
    assert np.allclose(w.cpu().numpy().sum(1), 1, atol=1e-6)


@pytest.mark.parametrize("tokens,experts,k,scale", [(64, 288, 8, 2.5), (16, 64, 4, 1.0), (4, 5, 2, 2.5)])
def test_sigmoid_router_indices_are_bit_exact(tokens, experts, k, scale):
    rng = np.random.default_rng(7 * experts)
    logits = (rng.standard_normal((tokens, experts)) * 2).astype(np.float32)
    bias = (rng.uniform(-0.09, 0.09, size=experts)).astype(np.float32)
    ids, w = moe.route_sigmoid_topk(torch.from_numpy(logits).cuda(), torch.from_numpy(bias).cuda(), k, scale)
    rids, rw = oracle.route_sigmoid_topk(logits, bias, k, scale)
    assert np.array_equal(ids.cpu().numpy(), rids)
    assert np.max(np.abs(w.cpu().numpy() - rw)) <= 1e-6


def test_sigmoid_router_ties_and_nan():
    l = torch.tensor([[0.0, 1.0, 1.0, float("nan"), 1.0, -1.0, 1.0], [float("nan")] * 7], device="cuda")
    ids, _ = moe.route_sigmoid_topk(l, None, 3, 1.0)
    assert ids.cpu().numpy().tolist() == [[1, 2, 4], [0, 1, 2]]


def test_sort_groups_combos_by_expert_stably():
    from crownest_b200._lib import check, lib
    rng = np.random.default_rng(3)
    ids = rng.integers(0, 512, size=640).astype(np.int32)
    ids[5] = -1
    d = torch.from_numpy(ids).cuda()
    order = torch.empty(640, dtype=torch.int32, device="cuda")
    check(lib().cn_moe_sort(d.data_ptr(), order.data_ptr(), 640, 512, torch.cuda.current_stream().cuda_stream))
    key = np.where(ids < 0, 512, ids)
    assert order.cpu().numpy().tolist() == np.argsort(key, kind="stable").tolist()


def make_experts(hidden, inter, experts, rng, only=None):
    """gate|up slabs and down matrices per expert; with `only`, just for those experts (None elsewhere)."""
    want = range(experts) if only is None else sorted(set(int(e) for e in only))
    gu, dn = [None] * experts, [None] * experts
    for e in want:
        gu[e] = synth.nvfp4_matrix(2 * inter, hidden, rng)
        dn[e] = synth.nvfp4_matrix(hidden, inter, rng)
    return gu, dn


def cpu_moe(x, ids, wts, gu, dn, hidden, inter, gs_gu, gs_dn, shared=None, shared_gs=None, limit=0.0):
    """the reference's moe_cpu order (engine/src/glm5_moe.rs:319-346) on NVFP4 experts"""
    tokens, k = ids.shape
    ye = np.zeros((tokens * k, hidden), np.float32)
    rb = hidden // 64 * 36
    for c in range(tokens * k):
        e = ids.reshape(-1)[c]
        g, u = gu[e][: inter * rb], gu[e][inter * rb:]
        ye[c] = oracle.nvfp4_ffn(g, u, dn[e], hidden, inter, [gs_gu, gs_gu, gs_dn], x[c // k: c // k + 1], limit=limit, threads=4, path=1)[0]
    ys = None
    if shared is not None:
        si = shared[0].size // rb
        ys = oracle.nvfp4_ffn(shared[0], shared[1], shared[2], hidden, si, list(shared_gs), x, limit=limit, threads=4, path=1)
    return oracle.moe_acc_combo(ye, wts, ys)


@pytest.mark.parametrize("tokens", [1, 8, 64])
def test_moe_step_matches_the_cpu_reference(tokens):
    # the benchmark's MoE shape: hidden 2048, 512 experts, intermediate 512, one shared expert, softmax top-10. Only the
    # experts the routing picks get weights (the others are null table entries that nothing may touch): 10 / ~75 / ~370
    hidden, inter, experts, k = 2048, 512, 512, 10
    rng = np.random.default_rng(100 + tokens)
    xb, xf = synth.activations(tokens, hidden, rng)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    rids, rw = oracle.route_softmax_topk(logits, k)
    gu, dn = make_experts(hidden, inter, experts, rng, only=rids.reshape(-1))
    shared = [synth.nvfp4_matrix(inter, hidden, rng), synth.nvfp4_matrix(inter, hidden, rng), synth.nvfp4_matrix(hidden, inter, rng)]
    gs_gu, gs_dn, sgs = np.float32(0.03), np.float32(0.05), [np.float32(0.03), np.float32(0.04), np.float32(0.05)]
    dev = lambda a: None if a is None else torch.from_numpy(a).cuda()
    w = moe.GpuMoeWeights(hidden, inter, experts, gs_gu, gs_dn, gate_up=[dev(a) for a in gu], down=[dev(a) for a in dn],
                          shared=[dev(a) for a in shared], shared_gs=sgs)
    plan = moe.GpuMoePlan(hidden, inter, experts, k, max_tokens=64, shared_inter=inter)
    y = plan.run(w, dev(logits), to_dev_bf16(xb))
    ids, wts = plan.read_routing()
    assert np.array_equal(ids, rids)
    ref = cpu_moe(xf, rids, rw, gu, dn, hidden, inter, gs_gu, gs_dn, shared, sgs)
    check_close(from_dev_bf16(y), ref, f"moe tokens={tokens}", ulp_floor=1.0 / 64)
    # run to run: same bits
    y2 = plan.run(w, dev(logits), to_dev_bf16(xb))
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    plan.free()


def test_moe_f32_separate_gate_up_clamp_and_missing_experts():
    hidden, inter, experts, k = 1024, 256, 12, 4
    rng = np.random.default_rng(5)
    rb = hidden // 64 * 36
    gu, dn = make_experts(hidden, inter, experts, rng)
    gate = [a[: inter * rb].copy() for a in gu]
    up = [a[inter * rb:].copy() for a in gu]
    x = rng.standard_normal((3, hidden)).astype(np.float32)
    logits = rng.standard_normal((3, experts)).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).cuda()
    rids, rw = oracle.route_sigmoid_topk(logits, None, k, 2.5)
    w = moe.GpuMoeWeights(hidden, inter, experts, 0.2, 0.3, gate=[dev(a) for a in gate], up=[dev(a) for a in up], gs_up=0.2,
                          down=[dev(a) for a in dn])
    plan = moe.GpuMoePlan(hidden, inter, experts, k, max_tokens=8)
    y = plan.run(w, dev(logits), dev(x), router="sigmoid", scale=2.5, limit=10.0)
    ref = cpu_moe(x, rids, rw, gu, dn, hidden, inter, np.float32(0.2), np.float32(0.3), limit=10.0)
    check_close(y.cpu().numpy(), ref, "moe f32 clamp", bf16_out=False)
    # experts 0..5 not resident (null table entries): their combos add nothing
    w2 = moe.GpuMoeWeights(hidden, inter, experts, 0.2, 0.3, gate=[None if e < 6 else dev(gate[e]) for e in range(experts)],
                           up=[None if e < 6 else dev(up[e]) for e in range(experts)], gs_up=0.2,
                           down=[None if e < 6 else dev(dn[e]) for e in range(experts)])
    y2 = plan.run(w2, dev(logits), dev(x), router="sigmoid", scale=2.5, limit=10.0)
    rw2 = np.where(rids < 6, 0.0, rw).astype(np.float32)
    ref2 = cpu_moe(x, rids, rw2, gu, dn, hidden, inter, np.float32(0.2), np.float32(0.3), limit=10.0)
    check_close(y2.cpu().numpy(), ref2, "moe partial residency", bf16_out=False)
    plan.free()


@pytest.mark.parametrize("hidden,inter,experts,k,tokens", [(1024, 256, 24, 4, 40), (2048, 512, 16, 6, 33), (768, 1280, 9, 3, 50)])
def test_grouped_experts_with_f32_rows_and_short_rows(hidden, inter, experts, k, tokens):
    """More than 96 combos: the experts run over groups of rows that share an expert. f32 activations ride as two f16
    planes; k = 256 / 512 / 768 / 1280 cover the stage shapes for short and ragged rows; several rows per expert."""
    rng = np.random.default_rng(hidden + tokens)
    gu, dn = make_experts(hidden, inter, experts, rng)
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    dev = lambda a: torch.from_numpy(a).cuda()
    rids, rw = oracle.route_softmax_topk(logits, k)
    w = moe.GpuMoeWeights(hidden, inter, experts, 0.2, 0.3, gate_up=[dev(a) for a in gu], down=[dev(a) for a in dn])
    plan = moe.GpuMoePlan(hidden, inter, experts, k, max_tokens=tokens)
    y = plan.run(w, dev(logits), dev(x))
    ref = cpu_moe(x, rids, rw, gu, dn, hidden, inter, np.float32(0.2), np.float32(0.3))
    check_close(y.cpu().numpy(), ref, "grouped moe f32", bf16_out=False)
    # bf16 rows through the one-row and four-row group kernels, against the same reference fed the rounded rows
    xb = synth.bf16_bits(x)
    yb = plan.run(w, dev(logits), to_dev_bf16(xb))
    refb = cpu_moe(synth.bf16_to_f32(xb), rids, rw, gu, dn, hidden, inter, np.float32(0.2), np.float32(0.3))
    check_close(from_dev_bf16(yb), refb, "grouped moe bf16", ulp_floor=1.0 / 64)
    yb2 = plan.run(w, dev(logits), to_dev_bf16(xb))
    assert torch.equal(yb.view(torch.int16), yb2.view(torch.int16))
    from crownest_b200 import device_status
    assert device_status() == 0
    plan.free()
