"""The block-scaled FP4 tensor-core GEMM (tcgen05 kind::mxf4nvf4, through the C ABI) and its activation cascade against the
CPU checker: cascade bytes bit-exact with the restatement of the reference's host twin; GEMM outputs within rel L2 <= 1e-3
and 2 bf16 ulp (taken no lower than rms / 64) of the f32-accumulated CPU reference of the exact activations."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import device_status, ops, synth
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16
from test_gpu_nvfp4_gemm import cpu_rows


@pytest.mark.parametrize("levels", [1, 3, 5])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_cascade_bytes_are_bit_exact(levels, dtype):
    rng = np.random.default_rng(levels)
    k = 640
    x = (rng.standard_normal((9, k)) * np.array([3.0, 0.4, 0.04, 0.004, 1e-4, 300.0, 0.0, 1.0, 1e-30])[:, None]).astype(np.float32)
    x[7, 5] = 1500.0
    if dtype == "bf16":
        xb = synth.bf16_bits(x)
        x = synth.bf16_to_f32(xb)
        got = ops.act_cascade(to_dev_bf16(xb), levels).cpu().numpy()
    else:
        got = ops.act_cascade(torch.from_numpy(x).cuda(), levels).cpu().numpy()
    for r in range(x.shape[0]):
        assert np.array_equal(got[r], oracle.act_cascade(x[r], levels)), f"row {r}"


@pytest.mark.parametrize("rows,k,m", [(128, 256, 32), (256, 512, 64), (200, 1024, 70), (384, 2048, 33), (640, 5120, 96), (1000, 768, 17)])
def test_fp4_gemm_matches_the_cpu_reference(rows, k, m):
    rng = np.random.default_rng(rows + k + m)
    w = synth.nvfp4_matrix(rows, k, rng)
    w.reshape(-1, 36)[::7, 1] = 0x7F  # the NaN code of the tensor core's scale format: must read as 448
    w.reshape(-1, 36)[::5, 2] |= 0x80  # bit 7 is ignored
    gs = np.float32(0.37)
    xb, xf = synth.activations(m, k, rng)
    xf[m // 2] *= np.float32(2.0 ** -20)
    xb = synth.bf16_bits(xf)
    xf = synth.bf16_to_f32(xb)
    fw = ops.Fp4Packed(ops.Fp4.from_host(w, rows, k, gs))
    y = ops.launch_gemm_fp4(fw, to_dev_bf16(xb))
    torch.cuda.synchronize()
    assert device_status() == 0
    ref = cpu_rows(w, rows, k, gs, xf)
    got = from_dev_bf16(y)
    for t in (0, m // 2, m - 1):
        check_close(got[t:t + 1], ref[t:t + 1], f"fp4 gemm {rows}x{k} m={m} row {t}", ulp_floor=1.0 / 64)
    check_close(got, ref, f"fp4 gemm {rows}x{k} m={m}", ulp_floor=1.0 / 64)
    yf = ops.launch_gemm_fp4(fw, torch.from_numpy(xf).cuda()).cpu().numpy()
    scale = np.sqrt(np.mean(ref.astype(np.float64) ** 2, axis=1, keepdims=True))
    assert np.max(np.abs(yf - ref) / scale) <= 1e-4
    y2 = ops.launch_gemm_fp4(fw, to_dev_bf16(xb))
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))


@pytest.mark.parametrize("rows,k", [(17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("m", [64, 512])
def test_fp4_gemm_on_the_batched_benchmark_matrices(rows, k, m):
    rng = np.random.default_rng(rows + m + 1)
    w = synth.nvfp4_matrix(rows, k, rng)
    gs = np.float32(0.21)
    xb, xf = synth.activations(m, k, rng)
    fw = ops.Fp4Packed(ops.Fp4.from_host(w, rows, k, gs))
    y = ops.launch_gemm_fp4(fw, to_dev_bf16(xb))
    pick = np.unique(np.concatenate([[0, 1, 127, 128, rows - 129, rows - 1], rng.integers(0, rows, size=256)]))
    rb = k // 64 * 36
    sub = np.ascontiguousarray(w.reshape(rows, rb)[pick]).reshape(-1)
    ref = cpu_rows(sub, len(pick), k, gs, xf)
    check_close(from_dev_bf16(y)[:, pick], ref, f"fp4 gemm {rows}x{k} m={m} (sample)", ulp_floor=1.0 / 64)
    assert device_status() == 0
