"""The persistent GEMV chain (cn_nvfp4_seq_*) against the CPU checker and against the per-projection launches:
every step within rel L2 <= 1e-3 / 2 bf16 ulp of the f32 CPU reference fed with the same (bf16) inputs, the same bits run
after run, and shapes whose tiles do not divide evenly among the CTAs (cut tiles handed over between CTAs)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import CrownestError, dense, device_status, ops, synth
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16


def _mat(rows, k, rng, gs):
    w = synth.nvfp4_matrix(rows, k, rng)
    return w, ops.Fp4.from_host(w, rows, k, gs)


@pytest.mark.parametrize("hidden,inter,rows_a", [(2048, 4096, 1000), (5120, 17408, 7168), (2304, 2048, 37)])
def test_chain_of_dependent_steps_matches_the_cpu_reference(hidden, inter, rows_a):
    """a: x -> [rows_a], then the FFN: h = act(gate x, up x), y = down h; each checked from its own device input."""
    rng = np.random.default_rng(hidden + inter)
    gs = [np.float32(v) for v in (0.7, 0.02, 0.03, 0.05)]
    wa, fa = _mat(rows_a, hidden, rng, gs[0])
    wg, fg = _mat(inter, hidden, rng, gs[1])
    wu, fu = _mat(inter, hidden, rng, gs[2])
    wd, fd = _mat(hidden, inter, rng, gs[3])
    xb, xf = synth.activations(1, hidden, rng)
    x = to_dev_bf16(xb)
    a = torch.full((1, rows_a), float("nan"), dtype=torch.bfloat16, device="cuda")
    h = torch.full((1, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    y = torch.full((1, hidden), float("nan"), dtype=torch.float32, device="cuda")
    seq = ops.GemvSeq()
    s0 = seq.gemv(fa, x, a)
    s1 = seq.gemv_gu(fg, fu, x, h, after=s0)
    seq.gemv(fd, h, y, after=s1)
    seq.build()
    seq.run()
    torch.cuda.synchronize()
    assert device_status() == 0
    check_close(from_dev_bf16(a), oracle.nvfp4_gemv(wa, rows_a, hidden, gs[0], xf, threads=8, path=1), "chain step 0")
    g = oracle.nvfp4_gemv(wg, inter, hidden, gs[1], xf, threads=8, path=1)
    u = oracle.nvfp4_gemv(wu, inter, hidden, gs[2], xf, threads=8, path=1)
    href = np.vectorize(oracle.lib().cn_o_silu_mul)(g, u).astype(np.float32)
    check_close(from_dev_bf16(h), href, "chain gate/up", ulp_floor=1.0 / 64)
    hdev = from_dev_bf16(h)  # the down step is checked from the device's own (bf16) h
    yref = oracle.nvfp4_gemv(wd, hidden, inter, gs[3], hdev, threads=8, path=1)
    check_close(y.cpu().numpy(), yref, "chain down", bf16_out=False)
    # replay: counters carry over from run to run, the bits do not change
    a0, h0, y0 = a.clone(), h.clone(), y.clone()
    for _ in range(3):
        a.fill_(0), h.fill_(0), y.fill_(0)
        seq.run()
    torch.cuda.synchronize()
    assert torch.equal(a.view(torch.int16), a0.view(torch.int16)) and torch.equal(h.view(torch.int16), h0.view(torch.int16))
    assert torch.equal(y.view(torch.int32), y0.view(torch.int32))
    assert device_status() == 0
    seq.free()


def test_fused_stack_matches_the_per_projection_launches():
    cfg = dict(hidden=5120, qkv=7168, inter=17408, layers=3)
    a = dense.DenseStack(cfg=cfg, seed=3)
    b = dense.DenseStack(cfg=cfg, seed=3).fuse("token")
    c = dense.DenseStack(cfg=cfg, seed=3).fuse("layer")
    d = dense.DenseStack(cfg=cfg, seed=3).fuse("gemv")
    x = torch.randn((1, 5120), generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    for st in (a, b, c, d):
        st.x.copy_(x)
        st.run_layers(1)
    torch.cuda.synchronize()
    assert device_status() == 0
    for name in ("q", "o", "h", "y"):
        ra = from_dev_bf16(getattr(a, name))
        for other in (b, c, d):
            rb = from_dev_bf16(getattr(other, name))
            # two summation orders of the same f32 products: a bf16 ulp apart at most
            assert np.max(np.abs(ra - rb) / np.maximum(np.abs(ra), np.sqrt(np.mean(ra * ra)) / 64)) <= 2.0 ** -7, name
    assert torch.equal(b.y.view(torch.int16), c.y.view(torch.int16))  # same shares per step -> same bits
    g2 = d.capture(1)  # one launch per projection, replayed: the same bits every time
    y1 = d.y.clone()
    for _ in range(3):
        g2.replay()
    torch.cuda.synchronize()
    assert torch.equal(d.y.view(torch.int16), y1.view(torch.int16))
    # under graph capture, replayed
    g = b.capture(1)
    y0 = b.y.clone()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(b.y.view(torch.int16), y0.view(torch.int16)) and device_status() == 0


def test_chain_refuses_shapes_it_does_not_take():
    rng = np.random.default_rng(1)
    _, f = _mat(64, 1024, rng, 1.0)
    seq = ops.GemvSeq()
    seq.gemv(f, torch.zeros((1, 1024), dtype=torch.bfloat16, device="cuda"), torch.zeros((1, 64), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(CrownestError, match="at least 2048"):
        seq.build()
