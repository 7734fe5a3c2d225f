"""Parity of the CUDA NVFP4 GEMV (through the C ABI) with the CPU checker on the same seeded inputs.

Tolerances (the stated contract): bit-exact dequantised weights; GEMV outputs within relative
L2 <= 1e-3 and max abs error <= 2 bf16 ulp of the fp32-accumulated CPU reference; rows of a
small-M call bit-identical to one-row calls.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import CrownestError, device_status, ops, synth

REL_L2 = 1e-3
BF16_ULPS = 2


def bf16_ulp(v):
    """spacing of bf16 at |v| (8 significand bits)"""
    a = np.maximum(np.abs(v.astype(np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


def check_close(got_f32, ref_f32, what, bf16_out=True, rel_l2=REL_L2, ulp_floor=0.0):
    """rel L2 and max error in bf16 ulp against the CPU reference (rounded once to bf16 when the output
    is bf16). `ulp_floor`: for composite steps whose outputs cancel (a weighted sum of expert outputs),
    the ulp is taken at max(|ref|, ulp_floor * rms(ref)): two ulp of an output that cancelled to ~0 is
    below the f32 accumulation error of its terms."""
    if bf16_out:
        ref_f32 = synth.bf16_to_f32(synth.bf16_bits(ref_f32))
    got, ref = got_f32.astype(np.float64), ref_f32.astype(np.float64)
    rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
    assert rel <= rel_l2, f"{what}: rel L2 {rel:.3e}"
    if bf16_out:
        at = np.maximum(np.abs(ref_f32), ulp_floor * np.sqrt(np.mean(ref * ref))).astype(np.float32)
        worst = np.max(np.abs(got - ref) / bf16_ulp(at))
        assert worst <= BF16_ULPS, f"{what}: {worst:.2f} bf16 ulp"


def to_dev_bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)


def from_dev_bf16(t):
    return synth.bf16_to_f32(t.view(torch.int16).cpu().numpy().view(np.uint16))


def make(rows, cols, seed, gs=1.0, sigma=0.05):
    rng = np.random.default_rng(seed)
    w = synth.nvfp4_matrix(rows, cols, rng, sigma)
    return rng, w, ops.Fp4.from_host(w, rows, cols, gs)


def test_dequantised_weights_are_bit_exact():
    rng = np.random.default_rng(5)
    rows, cols = 64, 256
    blocks = rows * cols // 64
    raw = rng.integers(0, 256, size=(blocks, 36), dtype=np.uint8)
    raw[:, :4] = (np.arange(blocks * 4) % 256).astype(np.uint8).reshape(blocks, 4)  # every scale byte
    for rule in (False, True):
        m = ops.Fp4.from_host(raw.reshape(-1), rows, cols, 2.3e-4)
        got = ops.dequant(m, rule=rule).cpu().numpy()
        want = oracle.nvfp4_dequant(raw.reshape(-1), rows, cols, np.float32(2.3e-4), rule=rule)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (512, 2048), (2048, 512), (100, 1536), (37, 256), (1000, 5120), (260, 17408)])
@pytest.mark.parametrize("m", [1, 4])
def test_gemv_bf16_matches_the_cpu_reference(rows, cols, m):
    rng, w, dev = make(rows, cols, seed=0)
    xb, xf = synth.activations(m, cols, rng)
    ref = oracle.nvfp4_gemv(w, rows, cols, np.float32(1.0), xf, threads=8, path=1)
    y = ops.launch_gemv(dev, to_dev_bf16(xb))
    torch.cuda.synchronize()
    assert device_status() == 0
    check_close(from_dev_bf16(y), ref, f"[{rows},{cols}] m={m}")


@pytest.mark.parametrize("rows,cols", [(300, 1024), (64, 4096), (129, 768)])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8])
def test_gemv_f32_matches_the_cpu_reference(rows, cols, m):
    rng, w, dev = make(rows, cols, seed=1, gs=1.7e-3, sigma=30.0)  # scale bytes up to 0x7E
    x = rng.uniform(-2, 2, size=(m, cols)).astype(np.float32)
    ref = oracle.nvfp4_gemv(w, rows, cols, np.float32(1.7e-3), x, threads=8, path=1)
    y = ops.launch_gemv(dev, torch.from_numpy(x).cuda())
    check_close(y.cpu().numpy(), ref, f"f32 [{rows},{cols}] m={m}", bf16_out=False)
    # the reference's own bound: |y - y_exact| <= gamma(K/16 + 10) * sum|w x| (cpu_nvfp4.rs:516-536), x4 slack
    # for the different (lane-split) summation order
    y64, ab = oracle.nvfp4_gemv_f64(w, rows, cols, np.float32(1.7e-3), x, rule=True)
    nu = (cols / 16 + 10) * 2.0 ** -24
    assert np.max(np.abs(y.cpu().numpy() - y64) / (nu / (1 - nu) * ab + 1e-30)) <= 4.0


def test_scale_byte_0x7f_reads_as_448_and_bit7_is_ignored():
    rng = np.random.default_rng(0x7F)
    rows, cols = 48, 512
    w = synth.nvfp4_matrix(rows, cols, rng).reshape(-1, 36)
    w[:, :4] = np.where(rng.integers(0, 2, size=(w.shape[0], 4)) == 0, 0x7F, 0xF0 + rng.integers(0, 8, size=(w.shape[0], 4))).astype(np.uint8)
    w[:, 4:] &= 0x77
    x = (np.abs(rng.uniform(-1, 1, size=(2, cols))) + 0.01).astype(np.float32)
    gs = np.float32(9.5e-4)
    ref = oracle.nvfp4_gemv(w.reshape(-1), rows, cols, gs, x)
    y = ops.launch_gemv(ops.Fp4.from_host(w.reshape(-1), rows, cols, gs), torch.from_numpy(x).cuda()).cpu().numpy()
    check_close(y, ref, "0x7F rule", bf16_out=False)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_small_m_rows_are_bit_identical_to_one_row_calls(dtype):
    rows, cols = 777, 5120
    rng, w, dev = make(rows, cols, seed=3)
    xb, xf = synth.activations(8, cols, rng)
    xd = to_dev_bf16(xb) if dtype == "bf16" else torch.from_numpy(xf).cuda()
    ones = [ops.launch_gemv(dev, xd[i:i + 1]).view(torch.int16 if dtype == "bf16" else torch.int32).cpu().numpy()[0] for i in range(8)]
    for m in (2, 3, 4, 5, 8):
        y = ops.launch_gemv(dev, xd[:m]).view(torch.int16 if dtype == "bf16" else torch.int32).cpu().numpy()
        for i in range(m):
            assert np.array_equal(y[i], ones[i]), f"m={m} row {i}"
    # run to run
    again = ops.launch_gemv(dev, xd[:4]).view(torch.int16 if dtype == "bf16" else torch.int32).cpu().numpy()
    assert np.array_equal(again[0], ones[0])


@pytest.mark.parametrize("limit", [0.0, 10.0])
@pytest.mark.parametrize("m", [1, 4])
def test_fused_gate_up_matches_the_cpu_ffn_stage(limit, m):
    inter, cols = 1111, 2048
    rng = np.random.default_rng(11)
    wg, wu = synth.nvfp4_matrix(inter, cols, rng), synth.nvfp4_matrix(inter, cols, rng)
    gsg, gsu = np.float32(0.8), np.float32(1.3)
    xb, xf = synth.activations(m, cols, rng)
    g = oracle.nvfp4_gemv(wg, inter, cols, gsg, xf, 8, 1)
    u = oracle.nvfp4_gemv(wu, inter, cols, gsu, xf, 8, 1)
    L = oracle.lib()
    act = np.vectorize(lambda a, b: L.cn_o_swiglu_clamp(a, b, limit) if limit > 0 else L.cn_o_silu_mul(a, b))
    ref = act(g, u).astype(np.float32)
    h = ops.launch_gemv_gu(ops.Fp4.from_host(wg, inter, cols, gsg), ops.Fp4.from_host(wu, inter, cols, gsu), to_dev_bf16(xb), limit=limit)
    # the reference rounded once to bf16, like every other case; the ulp is taken no lower than rms / 64 because
    # h = silu(g) * u cancels towards zero where g does
    check_close(from_dev_bf16(h), ref, f"gate/up m={m} limit={limit}", ulp_floor=1.0 / 64)


def test_full_ffn_against_cpu_expert_ffn():
    h, i = 2048, 512
    rng = np.random.default_rng(21)
    g, u, d = (synth.nvfp4_matrix(i, h, rng), synth.nvfp4_matrix(i, h, rng), synth.nvfp4_matrix(h, i, rng))
    gs = [np.float32(0.02), np.float32(0.03), np.float32(0.05)]
    x = rng.standard_normal((3, h)).astype(np.float32)
    ref = oracle.nvfp4_ffn(g, u, d, h, i, gs, x, threads=8, path=1)
    y = ops.dense_ffn_w(ops.Fp4.from_host(g, i, h, gs[0]), ops.Fp4.from_host(u, i, h, gs[1]), ops.Fp4.from_host(d, h, i, gs[2]),
                        torch.from_numpy(x).cuda())
    check_close(y.cpu().numpy(), ref, "ffn f32", bf16_out=False)


def test_errors_are_named_not_fatal():
    _, _, dev = make(64, 256, seed=9)
    with pytest.raises(CrownestError, match="multiple of 256"):
        bad = ops.Fp4.from_host(np.zeros(64 * 3 * 36, np.uint8), 64, 192, 1.0)
        ops.launch_gemv(bad, torch.zeros((1, 192), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(CrownestError, match="1..8"):
        ops.launch_gemv(dev, torch.zeros((9, 256), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(CrownestError, match="needs"):
        ops.Fp4.from_host(np.zeros(10, np.uint8), 64, 256, 1.0)


@pytest.mark.parametrize("rows,cols,gu", [(5120, 17408, False), (6000, 17408, False), (2560, 17408, True), (640, 17408, False), (1280, 17408, False),
                                          (896, 5120, False)])
def test_k_shared_by_a_cta_pair_matches_the_cpu_reference(rows, cols, gu):
    """Shapes for which the library launches clusters of two or four CTAs (tiles that do not fill the last wave and a long
    K, the down projection of the dense stack among them, and the few long rows of a tensor-parallel rank's share of it):
    each CTA of a cluster sums its part of K and the parts meet through distributed shared memory in a fixed order."""
    rng, w, fw = make(rows, cols, rows + cols)
    xb, xf = synth.activations(1, cols, rng)
    if gu:
        w2 = synth.nvfp4_matrix(rows, cols, rng)
        fw2 = ops.Fp4.from_host(w2, rows, cols, 1.0)
        y = ops.launch_gemv_gu(fw, fw2, to_dev_bf16(xb))
        g = oracle.nvfp4_gemv(w, rows, cols, np.float32(1.0), xf, threads=8, path=1)
        u = oracle.nvfp4_gemv(w2, rows, cols, np.float32(1.0), xf, threads=8, path=1)
        ref = np.vectorize(oracle.lib().cn_o_silu_mul)(g, u).astype(np.float32)
    else:
        y = ops.launch_gemv(fw, to_dev_bf16(xb))
        ref = oracle.nvfp4_gemv(w, rows, cols, np.float32(1.0), xf, threads=8, path=1)
    y2 = ops.launch_gemv_gu(fw, fw2, to_dev_bf16(xb)) if gu else ops.launch_gemv(fw, to_dev_bf16(xb))
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))  # run to run: the same bits
    # 5120 .. 6000 outputs over k = 17408: a few cancel to 1e-4 of the row's scale, where the f32 accumulation error of
    # either side is already several bf16 ulp of the value; the ulp is taken no lower than rms / 256
    check_close(from_dev_bf16(y), ref, f"cluster pair {rows}x{cols} gu={gu}", ulp_floor=1.0 / 64 if gu else 1.0 / 256)
    assert device_status() == 0
