"""The NVFP4 checker against the reference's golden vectors and its own unit-test properties
(engine/src/cpu_nvfp4.rs:538-727)."""
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN


def synth(rows, cols, rng, scale_bytes=None, code_mask=0xFF):
    blocks = rows * cols // 64
    b = rng.integers(0, 256, size=(blocks, 36), dtype=np.uint8)
    b[:, 4:] &= code_mask
    if scale_bytes is not None:
        b[:, :4] = scale_bytes(rng, (blocks, 4))
    return b.reshape(-1)


def scale_mix(rng, shape):
    # realistic scale bytes 0x30..0x7F, about one in 16 the 0x7F code (cpu_nvfp4.rs:467-475)
    b = rng.integers(0, 256, size=shape, dtype=np.uint8)
    return np.where(b & 15 == 0, 0x7F, 0x30 + (b >> 4) * 3).astype(np.uint8)


def gamma(cols):
    nu = (cols / 16 + 10) * 2.0 ** -24
    return nu / (1 - nu)


def test_dequant_matches_the_reference_python_decoder_on_its_container_fixture():
    g = np.load(os.path.join(GOLDEN, "nvfp4_dequant.npz"))
    n = int(g["cnq_count"])
    assert n == 6
    for i in range(n):
        rows, cols = (int(v) for v in g[f"cnq{i}_shape"])
        got = oracle.nvfp4_dequant(g[f"cnq{i}_raw"], rows, cols, np.float32(g[f"cnq{i}_gs"]))
        want = g[f"cnq{i}_deq"].reshape(rows, cols)
        assert got.view(np.uint32).tolist() == want.view(np.uint32).tolist(), str(g[f"cnq{i}_name"])


def test_dequant_every_scale_byte_with_and_without_the_slab_rule():
    g = np.load(os.path.join(GOLDEN, "nvfp4_dequant.npz"))
    raw, gs = g["all_raw"], np.float32(g["all_gs"])
    for rule, key in ((False, "all_deq_raw"), (True, "all_deq_rule")):
        got = oracle.nvfp4_dequant(raw, 64, 256, gs, rule=rule)
        assert np.array_equal(got.view(np.uint32), g[key].view(np.uint32)), key
    # the two readings differ exactly where the scale byte is 0x7F (480 vs 448); 0xFF stays 480
    diff = g["all_deq_raw"] != g["all_deq_rule"]
    sb = raw.reshape(-1, 36)[:, :4].reshape(64, 256 // 16).repeat(16, axis=1)
    assert np.all(sb[diff] == 0x7F)


def test_tables_are_the_engine_decoders():
    L = oracle.lib()
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for nib in range(16):
        v = L.cn_o_e2m1(nib)
        assert v == (-mags[nib & 7] if nib & 8 else mags[nib & 7])
        assert np.signbit(np.float32(v)) == bool(nib & 8)
    for b in range(256):
        e, m = (b >> 3) & 0xF, b & 7
        want = m * 2.0 ** -9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)
        assert L.cn_o_ue4m3(b) == np.float32(want)
        assert L.cn_o_scale_rule(b) == (0x7E if b == 0x7F else b)
    assert L.cn_o_ue4m3(0x7F) == 480.0 and L.cn_o_ue4m3(0x7E) == 448.0


def test_shapes_are_checked():
    b = np.zeros(3 * 2 * 36, np.uint8)
    x = np.zeros(128, np.float32)
    oracle.nvfp4_gemv(b, 3, 128, 1.0, x)
    with pytest.raises(ValueError):
        oracle.nvfp4_gemv(b, 3, 96, 1.0, np.zeros(96, np.float32))
    with pytest.raises(ValueError):
        oracle.nvfp4_gemv(b[1:], 3, 128, 1.0, x)


@pytest.mark.parametrize("rows,cols", [(37, 256), (16, 2048), (9, 4096)])
def test_gemv_holds_the_fp32_bound(rows, cols):
    rng = np.random.default_rng(173)
    w = synth(rows, cols, rng, scale_mix)
    gs = np.float32(1.7e-3)
    for t in (1, 2, 3, 5, 8):
        x = rng.uniform(-2, 2, size=(t, cols)).astype(np.float32)
        yr, ab = oracle.nvfp4_gemv_f64(w, rows, cols, gs, x, rule=True)
        for path in (0, 1):
            y = oracle.nvfp4_gemv(w, rows, cols, gs, x, threads=3, path=path)
            worst = np.max(np.abs(y - yr) / np.maximum(gamma(cols) * ab, np.finfo(np.float64).tiny))
            assert worst <= 1.0, (t, path, worst)


def test_avx2_equals_scalar_bits_for_every_thread_count():
    if not oracle.lib().cn_o_have_avx2():
        pytest.skip("no AVX2 on this CPU")
    rng = np.random.default_rng(0xC0FFEE)
    rows, cols = 41, 1024
    w = synth(rows, cols, rng)  # every scale byte, bit 7 too
    for t in (1, 2, 3, 5, 8):
        x = rng.uniform(-2, 2, size=(t, cols)).astype(np.float32)
        s1 = oracle.nvfp4_gemv(w, rows, cols, 2.3e-4, x, 1, 0).view(np.uint32)
        for th in (1, 3, 8):
            assert np.array_equal(oracle.nvfp4_gemv(w, rows, cols, 2.3e-4, x, th, 0).view(np.uint32), s1)
            assert np.array_equal(oracle.nvfp4_gemv(w, rows, cols, 2.3e-4, x, th, 1).view(np.uint32), s1)


def test_scale_rule_is_the_slab_rule():
    # positive codes and activations: 448 vs 480 on half the sub-blocks moves every output far
    # beyond the fp32 bound (cpu_nvfp4.rs:609-635)
    rng = np.random.default_rng(0x7F)
    rows, cols = 12, 512
    w = synth(rows, cols, rng, lambda r, s: np.where(r.integers(0, 2, size=s) == 0, 0x7F, 0x70 + r.integers(0, 8, size=s)).astype(np.uint8), 0x77)
    gs = np.float32(9.5e-4)
    x = (np.abs(rng.uniform(-1, 1, size=(2, cols))) + 0.01).astype(np.float32)
    y448, ab448 = oracle.nvfp4_gemv_f64(w, rows, cols, gs, x, rule=True)
    y480, ab480 = oracle.nvfp4_gemv_f64(w, rows, cols, gs, x, rule=False)
    for path in (0, 1):
        y = oracle.nvfp4_gemv(w, rows, cols, gs, x, 2, path)
        assert np.max(np.abs(y - y448) / (gamma(cols) * ab448)) <= 1.0
        assert np.all(np.abs(y - y480) > gamma(cols) * ab480)
    clean = w.copy().reshape(-1, 36)
    clean[:, :4][clean[:, :4] == 0x7F] = 0x7E
    assert np.array_equal(oracle.nvfp4_gemv(clean.reshape(-1), rows, cols, gs, x).view(np.uint32),
                          oracle.nvfp4_gemv(w, rows, cols, gs, x).view(np.uint32))


def test_ffn_is_gemv_activation_gemv():
    rng = np.random.default_rng(0xF00D)
    h, i = 192, 128
    g, u, d = synth(i, h, rng, scale_mix), synth(i, h, rng, scale_mix), synth(h, i, rng, scale_mix)
    gs = [np.float32(v) for v in (2.1e-3, 1.9e-3, 2.6e-3)]
    for t in (1, 2, 5):
        x = rng.uniform(-2, 2, size=(t, h)).astype(np.float32)
        y = oracle.nvfp4_ffn(g, u, d, h, i, gs, x)
        gg, uu = oracle.nvfp4_gemv(g, i, h, gs[0], x), oracle.nvfp4_gemv(u, i, h, gs[1], x)
        L = oracle.lib()
        hk = np.array([L.cn_o_silu_mul(a, b) for a, b in zip(gg.ravel(), uu.ravel())], np.float32).reshape(t, i)
        assert np.array_equal(oracle.nvfp4_gemv(d, h, i, gs[2], hk).view(np.uint32), y.view(np.uint32))
        for th in (1, 3, 8):
            for path in (0, 1):
                assert np.array_equal(oracle.nvfp4_ffn(g, u, d, h, i, gs, x, threads=th, path=path).view(np.uint32), y.view(np.uint32))


def test_swiglu_clamp_is_the_hf_rule():
    L = oracle.lib()
    silu = lambda v: np.float32(v) / (np.float32(1) + np.exp(np.float32(-v), dtype=np.float32))
    cases = [(25.0, 3.0, silu(10.0) * np.float32(3.0)), (-25.0, 3.0, silu(-25.0) * np.float32(3.0)),
             (2.0, 40.0, silu(2.0) * np.float32(10.0)), (2.0, -40.0, silu(2.0) * np.float32(-10.0)),
             (10.0, -10.0, silu(10.0) * np.float32(-10.0)), (0.5, 0.25, silu(0.5) * np.float32(0.25))]
    for g, u, want in cases:
        assert abs(L.cn_o_swiglu_clamp(g, u, 10.0) - want) <= 1e-6 * abs(want)
    assert np.isnan(L.cn_o_swiglu_clamp(float("nan"), 1.0, 10.0))
    assert np.isnan(L.cn_o_swiglu_clamp(1.0, float("nan"), 10.0))
