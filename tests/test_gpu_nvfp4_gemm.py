"""Parity of the tcgen05 NVFP4 GEMM (through the C ABI) with the CPU checker: rel L2 <= 1e-3 and 2 bf16 ulp of
the f32-accumulated CPU reference, ragged row and token counts included.

The ulp is taken at max(|ref|, rms / 64): over thousands of outputs a few cancel to 1e-5 of the row's scale,
where the f32 accumulation error of either side (1e-6 of the scale; measured against f64, the tensor-memory
accumulator is 5e-7 .. 5e-6 off, the CPU reference 5e-7 .. 1e-6) is already several bf16 ulp of the value.
A second assert bounds the absolute error against the scale directly."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import ops, synth
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16


def cpu_rows(w, rows, k, gs, xf):
    out = np.empty((xf.shape[0], rows), np.float32)
    for t0 in range(0, xf.shape[0], 8):
        out[t0:t0 + 8] = oracle.nvfp4_gemv(w, rows, k, gs, xf[t0:t0 + 8], threads=8, path=1)
    return out


@pytest.mark.parametrize("rows,k,m", [(128, 256, 16), (256, 512, 64), (200, 1024, 130), (384, 2048, 257), (5120, 1024, 96)])
def test_gemm_matches_the_cpu_reference_bf16(rows, k, m):
    rng = np.random.default_rng(rows + k + m)
    w = synth.nvfp4_matrix(rows, k, rng)
    gs = np.float32(0.37)
    xb, xf = synth.activations(m, k, rng)
    xf[m // 2] *= np.float32(2.0 ** -20)  # a row far below the others: its own power-of-two scale
    xb = synth.bf16_bits(xf)
    xf = synth.bf16_to_f32(xb)
    fw = ops.Fp4.from_host(w, rows, k, gs)
    y = ops.launch_gemm(fw, to_dev_bf16(xb))
    ref = cpu_rows(w, rows, k, gs, xf)
    got = from_dev_bf16(y)
    for t in (0, m // 2, m - 1):
        check_close(got[t:t + 1], ref[t:t + 1], f"gemm {rows}x{k} m={m} row {t}", ulp_floor=1.0 / 64)
    check_close(got, ref, f"gemm {rows}x{k} m={m}", ulp_floor=1.0 / 64)
    # f32 rows out: the accumulator itself, against the CPU reference, relative to each row's scale
    yf = ops.launch_gemm(fw, torch.from_numpy(xf).cuda()).cpu().numpy()
    scale = np.sqrt(np.mean(ref.astype(np.float64) ** 2, axis=1, keepdims=True))
    assert np.max(np.abs(yf - ref) / scale) <= 1e-4


def test_gemm_f32_rows_and_all_scale_bytes():
    rows, k, m = 256, 256, 40
    rng = np.random.default_rng(9)
    w = synth.nvfp4_matrix(rows, k, rng).copy()
    w.reshape(-1, 36)[:, :4] = np.arange(rows * (k // 64) * 4, dtype=np.uint32).astype(np.uint8).reshape(-1, 4)  # every scale byte, 0x7F and bit 7 included
    x = rng.standard_normal((m, k)).astype(np.float32)
    fw = ops.Fp4.from_host(w, rows, k, np.float32(1.0))
    y = ops.launch_gemm(fw, torch.from_numpy(x).cuda()).cpu().numpy()
    ref = cpu_rows(w, rows, k, np.float32(1.0), x)
    check_close(y, ref, "gemm f32, all scale bytes", bf16_out=False)


def test_gemm_agrees_with_the_gemv_on_the_same_rows():
    rows, k, m = 512, 512, 8
    rng = np.random.default_rng(3)
    w = synth.nvfp4_matrix(rows, k, rng)
    xb, _ = synth.activations(m, k, rng)
    fw = ops.Fp4.from_host(w, rows, k, np.float32(0.5))
    a = from_dev_bf16(ops.launch_gemm(fw, to_dev_bf16(xb)))
    b = from_dev_bf16(ops.launch_gemv(fw, to_dev_bf16(xb)))
    assert np.max(np.abs(a - b)) <= 2 * np.max(np.abs(b)) * 2.0 ** -8


@pytest.mark.parametrize("rows,k", [(17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("m,nrows,ntok", [(64, 256, 64), (512, 256, 512), (4096, 96, 192)])
def test_gemm_on_the_batched_benchmark_matrices(rows, k, m, nrows, ntok):
    """The two matrices of the batched configuration at M = 64 / 512 / 4096, checked on a sample: `nrows` output rows
    spread over every row tile region (first and last rows included) for `ntok` of the tokens (all of them up to
    M = 512). The CPU reference only needs the sampled weight rows and tokens."""
    rng = np.random.default_rng(rows + m)
    w = synth.nvfp4_matrix(rows, k, rng)
    gs = np.float32(0.21)
    xb, xf = synth.activations(m, k, rng)
    fw = ops.Fp4.from_host(w, rows, k, gs)
    y = ops.launch_gemm(fw, to_dev_bf16(xb))
    pick = np.unique(np.concatenate([[0, 1, 127, 128, rows - 129, rows - 1], rng.integers(0, rows, size=nrows)]))
    toks = np.arange(m) if ntok >= m else np.unique(np.concatenate([[0, 127, 128, 255, 256, m - 1], rng.integers(0, m, size=ntok)]))
    rb = k // 64 * 36
    sub = np.ascontiguousarray(w.reshape(rows, rb)[pick]).reshape(-1)
    ref = cpu_rows(sub, len(pick), k, gs, np.ascontiguousarray(xf[toks]))
    got = from_dev_bf16(y)[np.ix_(toks, pick)]
    check_close(got, ref, f"gemm {rows}x{k} m={m} (sample)", ulp_floor=1.0 / 64)
