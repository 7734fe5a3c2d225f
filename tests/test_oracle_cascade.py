"""The CPU restatement of the reference's activation cascade (oracle/cascade.c) against the assertions the reference
makes on its own host twin (engine/src/kernels.rs:5525-5700), and the measurement that decides how many levels the
block-scaled FP4 GEMM needs: relative L2 and bf16-ulp error of the GEMV output as a function of the level count."""
import math

import numpy as np

import oracle
from crownest_b200 import synth


def test_scale_encoder_never_emits_the_nan_byte_and_rounds_up():
    L = oracle.lib()
    # geometric sweep 1e-4 .. 2000 (engine/src/kernels.rs:5543-5553)
    s = np.exp(np.linspace(math.log(1e-4), math.log(2000.0), 20000)).astype(np.float32)
    for v in s:
        b = L.cn_o_enc_ue4m3_up(float(v))
        assert b != 0x7F
        if v <= 448.0:
            assert L.cn_o_ue4m3(b) >= v  # smallest value >= s
            assert b == 0 or L.cn_o_ue4m3(b - 1) < v or (b & 7) == 0 and L.cn_o_ue4m3(b - 1) < v
    # engine/src/kernels.rs:5561-5568
    for v, want in ((460.0, 0x7E), (480.0, 0x7E), (448.0, 0x7E), (2000.0, 0x7E), (420.0, (15 << 3) | 6), (1.0, 7 << 3), (0.0, 0)):
        assert L.cn_o_enc_ue4m3_up(v) == want
    # every f32 in (448, 480]: the band that once produced 0x7F
    v = np.float32(448.0)
    while v <= 480.0:
        v = np.nextafter(v, np.float32(1e9), dtype=np.float32)
        assert L.cn_o_enc_ue4m3_up(float(v)) != 0x7F


def test_row_prescale_k_matches_its_definition():
    L = oracle.lib()
    # engine/src/kernels.rs:5650-5668
    assert L.cn_o_row_prescale_k(0.0) == 0
    assert L.cn_o_row_prescale_k(float("nan")) == 0
    assert L.cn_o_row_prescale_k(float("inf")) == 0
    assert L.cn_o_row_prescale_k(1.0) == 10
    assert L.cn_o_row_prescale_k(2047.0) == 0
    assert L.cn_o_row_prescale_k(2048.0) == -1
    a = float(np.float32(1e-45))
    while a < 1e30:
        af = float(np.float32(a))
        k = L.cn_o_row_prescale_k(af)
        e = math.floor(math.log2(af)) + 1
        assert k == max(-64, min(64, 11 - e)), af
        if -64 <= 11 - e <= 64:
            assert 1024.0 <= af * 2.0 ** k < 2048.0
        a *= 1.37


def test_rounding_is_nearest_with_ties_to_the_even_mantissa():
    L = oracle.lib()
    # tie points .25 .75 1.25 1.75 2.5 3.5 5 -> 0 1 1 2 2 4 4 (engine/src/kernels.rs:236-249)
    for v, code in ((0.25, 0), (0.75, 2), (1.25, 2), (1.75, 4), (2.5, 4), (3.5, 6), (5.0, 6), (5.01, 7), (0.26, 1), (-0.75, 10), (-6.0, 15)):
        assert L.cn_o_q_e2m1(v) == code, v


def _mean_rel(sigma, prescale, levels=3, n=64, seed=0):
    rng = np.random.default_rng(seed)
    acc = 0.0
    for _ in range(n):
        x = (rng.standard_normal(640) * sigma).astype(np.float32)
        d = oracle.act_cascade_dequant(oracle.act_cascade(x, levels, prescale), 640, levels)
        acc += np.linalg.norm(d.astype(np.float64) - x) / np.linalg.norm(x.astype(np.float64))
    return acc / n


def test_the_prescale_removes_the_absolute_floor():
    # engine/src/kernels.rs:5608-5633: three levels, rows of 640 N(0, sigma) values
    table = [(sg, _mean_rel(sg, False), _mean_rel(sg, True)) for sg in (3.0, 0.4, 0.04, 0.004, 0.0012, 1e-4)]
    reference = table[1][2]
    for sg, off, on in table:
        assert on < 2e-3, (sg, on)
        assert reference / 1.5 < on < 1.5 * reference
        assert on <= off * 1.25
    assert table[3][1] > 3e-2 and table[4][1] > 1e-1


def test_zero_rows_k_zero_rows_and_exact_rescale():
    rng = np.random.default_rng(1)
    z = np.zeros(640, np.float32)
    q = oracle.act_cascade(z)
    assert np.all(oracle.act_cascade_dequant(q, 640) == 0) and q[-4:].view(np.float32)[0] == 1.0
    x = (rng.standard_normal(640) * 300).astype(np.float32)
    x[17] = 1500.0
    assert np.array_equal(oracle.act_cascade(x, 3, True), oracle.act_cascade(x, 3, False))
    # scaling the row by 2^j leaves the level bytes unchanged and scales the dequantised row exactly
    x = (rng.standard_normal(640) * 0.01).astype(np.float32)
    q0 = oracle.act_cascade(x)
    d0 = oracle.act_cascade_dequant(q0, 640)
    for j in (-20, -3, 5, 17):
        q = oracle.act_cascade((x * np.float32(2.0 ** j)).astype(np.float32))
        assert np.array_equal(q[:-4], q0[:-4])
        assert np.array_equal(oracle.act_cascade_dequant(q, 640), d0 * np.float32(2.0 ** j))


def test_levels_needed_for_the_gemv_contract():
    """What the block-scaled FP4 tensor-core path costs in accuracy: the output of a GEMV whose bf16 N(0,1)
    activations went through an L-level cascade, against the f32 CPU reference of the exact activations.
    Three levels (the reference's choice) sit at 8e-4 relative L2 - inside 1e-3, but tens of bf16 ulp on outputs
    that are small against the row's scale; each level buys a factor of about 16."""
    rng = np.random.default_rng(0)
    rows, k = 256, 5120
    w = synth.nvfp4_matrix(rows, k, rng)
    wd = oracle.nvfp4_dequant(w, rows, k, np.float32(1.0), rule=True).astype(np.float64)
    _, xf = synth.activations(4, k, rng)
    ref = oracle.nvfp4_gemv(w, rows, k, np.float32(1.0), xf, threads=4, path=1).astype(np.float64)
    rel = {}
    for levels in (3, 4, 5, 6):
        xr = np.stack([oracle.act_cascade_dequant(oracle.act_cascade(xf[i], levels), k, levels) for i in range(4)])
        rel[levels] = np.linalg.norm(xr.astype(np.float64) @ wd.T - ref) / np.linalg.norm(ref)
    assert 3e-4 < rel[3] < 1e-3
    assert rel[4] < 1e-4 and rel[5] < 1e-5 and rel[6] < 1e-6
    assert all(rel[a] > 8 * rel[a + 1] for a in (3, 4))
