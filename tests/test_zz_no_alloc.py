"""The allocation-free MUL1 GEMV entry point against the plan-based one, through the C ABI.

Some callers of this library cannot allocate device memory where they call it: a decode loop that
must not trigger the device-wide synchronisation an allocation brings, a host process that handed out
all of its device memory at start-up, a plugin sandbox that forbids it. cn_mul1_gemv_noalloc keeps its
scratch in a fixed array inside the library instead of a plan. It runs the same kernels, so its
output has to equal cn_mul1_gemv's bit for bit; the array keeps the previous call's contents, so the
check is made on two calls in a row with different inputs and different matrices.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import oracle
from crownest_b200 import mul1
from crownest_b200._lib import CN_F32, CN_BF16, check, lib
from oracle import testkit as tk


def noalloc(which, hidden, inter, K, ptrs, x, slots, t, x_div=1):
    bits, half = mul1.bitrate(K)
    n = inter if which != 2 else hidden
    y = torch.full((slots, t, n), float("nan"), dtype=x.dtype, device="cuda")
    dt = CN_BF16 if x.dtype == torch.bfloat16 else CN_F32
    rc = lib().cn_mul1_gemv_noalloc(which, hidden, inter, bits, half, ptrs.data_ptr(), x.data_ptr(), y.data_ptr(), slots, t, x_div, dt,
                                    torch.cuda.current_stream().cuda_stream)
    return rc, y


def test_noalloc_gemv_equals_the_plan_gemv_on_two_calls_in_a_row():
    hidden, inter, K = 1024, 512, 3.0
    recs = [torch.from_numpy(tk.mul1_record(70 + i, hidden, inter, K)).cuda() for i in range(2)]
    ptrs = torch.tensor([r.data_ptr() for r in recs], dtype=torch.int64, device="cuda")
    plan = mul1.Mul1Plan(hidden, inter, K, slots=2, tokens=4)
    gen = torch.Generator(device="cuda").manual_seed(5)
    # first call: gate matrix, 2 slots x 4 rows, f32; second call: down matrix, other inputs, bf16
    for which, dtype in ((0, torch.float32), (2, torch.bfloat16), (1, torch.float32)):
        k = hidden if which != 2 else inter
        x = torch.randn((2, 4, k), device="cuda", generator=gen).to(dtype)
        want = plan.run_slots(which, ptrs, x)
        rc, got = noalloc(which, hidden, inter, K, ptrs, x, slots=2, t=4)
        check(rc)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # the tolerance of the parity tests is rel L2 <= 1e-3; the same kernels give the same bits
        rel = (got.float() - want.float()).norm() / want.float().norm()
        assert rel <= 1e-3
        assert torch.equal(got.view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                           want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    plan.free()


def test_noalloc_gemv_at_its_size_limits_against_the_cpu_reference():
    """hidden = inter = 4096 and 8 activation rows fill the fixed array to its last byte; two calls in a row (gate, then
    down with other inputs) are held to the plan-based entry point bit for bit, and the first to the CPU reference."""
    hidden = inter = 4096
    K = 3.0
    rec = tk.mul1_record(91, hidden, inter, K)
    d_rec = torch.from_numpy(rec).cuda()
    ptrs = torch.tensor([d_rec.data_ptr()], dtype=torch.int64, device="cuda")
    plan = mul1.Mul1Plan(hidden, inter, K, slots=1, tokens=8)
    rng = np.random.default_rng(6)
    tb = oracle.mul1_trellis_bytes(hidden, inter, K)
    scales, at = [], 3 * tb
    for _ in range(6):
        scales.append(rec[at:at + 2 * hidden].view(np.uint16))
        at += 2 * hidden
    for which in (0, 2):
        xh = rng.uniform(-2, 2, size=(1, 8, hidden)).astype(np.float32)
        x = torch.from_numpy(xh).cuda()
        want = plan.run_slots(which, ptrs, x)
        rc, got = noalloc(which, hidden, inter, K, ptrs, x, slots=1, t=8)
        check(rc)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
        if which == 0:
            ref = oracle.mul1_gemv(rec[:tb], scales[0], scales[1], hidden, inter, K, xh[0], threads=8)
            rel = np.linalg.norm(got.cpu().numpy()[0] - ref) / np.linalg.norm(ref)
            assert rel <= 1e-3, rel
    rc, _ = noalloc(0, hidden, inter, K, ptrs, torch.zeros((1, 8, hidden), device="cuda"), slots=1, t=8)
    check(rc)
    # a dtype the kernels do not take is refused before anything is enqueued
    rc = lib().cn_mul1_gemv_noalloc(0, hidden, inter, 3, 0, ptrs.data_ptr(), x.data_ptr(), want.data_ptr(), 1, 8, 1, 2,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 1 and b"dtype 2" in lib().cn_last_error_string()
    plan.free()


def test_noalloc_refuses_sizes_beyond_its_fixed_scratch():
    hidden, inter, K = 1024, 512, 3.0
    ptrs = torch.zeros(16, dtype=torch.int64, device="cuda")
    x = torch.zeros((16, 1, hidden), device="cuda")
    rc, _ = noalloc(0, hidden, inter, K, ptrs, x, slots=16, t=1)
    assert rc == 3 and b"fixed scratch holds 8 rows" in lib().cn_last_error_string()
    big = torch.zeros((1, 1, 8192), device="cuda")
    rc, _ = noalloc(0, 8192, 512, K, ptrs[:1], big, slots=1, t=1)
    assert rc == 3 and b"beyond the fixed scratch" in lib().cn_last_error_string()
