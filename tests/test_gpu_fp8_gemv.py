"""Parity of the CUDA FP8 GEMV with the CPU checker built on the reference's E4M3 codec."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import CrownestError, ops, synth
from test_gpu_nvfp4_gemv import check_close, from_dev_bf16, to_dev_bf16


def make(rows, cols, seed):
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 256, size=rows * cols, dtype=np.uint8)
    q = np.where(q & 0x7F == 0x7F, q ^ 1, q).astype(np.uint8)  # no NaN codes
    s = (rng.uniform(0.5, 2.0, size=(-(-rows // 128)) * (-(-cols // 128))) * 1e-2).astype(np.float32)
    return rng, q, s


@pytest.mark.parametrize("rows,cols", [(4096, 4096), (300, 208), (1000, 5120), (129, 17408), (256, 256)])
@pytest.mark.parametrize("m", [1, 4, 7])
def test_fp8_gemv_bf16_matches_the_cpu_reference(rows, cols, m):
    rng, q, s = make(rows, cols, rows + m)
    xb, xf = synth.activations(m, cols, rng)
    ref = oracle.fp8_gemv(q, rows, cols, s, xf)
    y = ops.fp8_gemv(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), to_dev_bf16(xb), rows, cols)
    # up to 28,000 outputs: a few cancel to 1e-4 of the row's scale, where the f32 accumulation error of either side is
    # already several bf16 ulp of the value; the ulp is taken no lower than rms / 256
    check_close(from_dev_bf16(y), ref, f"fp8 [{rows},{cols}] m={m}", ulp_floor=1.0 / 256)


def test_fp8_gemv_f32_and_row_invariance():
    rows, cols = 700, 1024
    rng, q, s = make(rows, cols, 3)
    x = rng.standard_normal((8, cols)).astype(np.float32)
    dq, ds, dx = torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), torch.from_numpy(x).cuda()
    y = ops.fp8_gemv(dq, ds, dx, rows, cols)
    check_close(y.cpu().numpy(), oracle.fp8_gemv(q, rows, cols, s, x), "fp8 f32", bf16_out=False)
    for i in range(8):
        assert torch.equal(ops.fp8_gemv(dq, ds, dx[i:i + 1], rows, cols).view(torch.int32)[0], y.view(torch.int32)[i])


def test_fp8_errors_are_named():
    with pytest.raises(CrownestError, match="scales"):
        ops.fp8_gemv(torch.zeros(256 * 256, dtype=torch.uint8, device="cuda"), torch.zeros(3, device="cuda"),
                     torch.zeros((1, 256), device="cuda"), 256, 256)
    with pytest.raises(CrownestError, match="multiple of 16"):
        ops.fp8_gemv(torch.zeros(4 * 24, dtype=torch.uint8, device="cuda"), torch.zeros(1, device="cuda"), torch.zeros((1, 24), device="cuda"), 4, 24)
