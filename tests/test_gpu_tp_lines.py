"""The tensor-parallel line output of the one-row GEMV on one GPU: the "peer" is a buffer of the same GPU, so the
lines the epilogue stores can be read back and compared with the host twin of the packing (crownest_b200.dense)."""
import ctypes as C

import numpy as np
import pytest
import torch

from crownest_b200 import dense, device_status, ops, synth

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1)


@pytest.mark.parametrize("rows,cols,gu", [(1024, 2048, False), (896, 5120, False), (640, 17408, False), (1280, 17408, False), (544, 5120, True)])
def test_lines_carry_the_rows_the_number_and_land_in_the_chosen_buffer(rows, cols, gu):
    rng = np.random.default_rng(rows + cols)
    fw = ops.Fp4.from_host(synth.nvfp4_matrix(rows, cols, rng), rows, cols, 1.0)
    fu = ops.Fp4.from_host(synth.nvfp4_matrix(rows, cols, rng), rows, cols, 1.0) if gu else None
    xb, _ = synth.activations(1, cols, rng)
    x = torch.from_numpy(xb.view(np.int16).copy()).cuda().view(torch.bfloat16)
    ref = ops.launch_gemv_gu(fw, fu, x) if gu else ops.launch_gemv(fw, x)
    world, me = 2, 1                      # this call plays rank 1 of two: its rows are the second half of the vector
    slice_lines = rows // 4               # lines of one rank's slice
    stride = world * slice_lines * 16     # bytes between a rank's two line buffers
    peer = torch.zeros(2 * stride // 4, dtype=torch.int32, device="cuda")  # rank 0's two line buffers
    epoch = torch.full((16,), 5, dtype=torch.int32, device="cuda")
    bases = (C.c_ulonglong * world)(peer.data_ptr(), 0)
    for tag, buf, flip in ((7, 1, 1), (8, 0, 0), (4095, 1, 0)):
        peer.zero_()
        y = torch.empty((1, rows), dtype=torch.bfloat16, device="cuda")
        ops.launch_gemv_lines(fw, x, y, (bases, world, me * rows, stride, epoch.data_ptr(), tag, buf, flip), gu=fu)
        torch.cuda.synchronize()
        assert torch.equal(y.view(torch.int16), ref.view(torch.int16))  # the rows themselves are those of the plain call
        number = dense.line_number(5, tag)
        which = buf ^ (flip & 5 & 1)
        assert which == dense.line_buffer(5, buf, flip)  # an odd count per step flips with the step counter
        got = peer.cpu().numpy().view(np.uint32).reshape(2, world * slice_lines, 4)
        want = dense.pack_lines(_bits(ref), number)
        assert np.array_equal(got[which, me * slice_lines:(me + 1) * slice_lines], want), (rows, cols, tag)
        assert not got[1 - which].any() and not got[which, :me * slice_lines].any()  # nothing anywhere else
        assert np.array_equal(dense.unpack_lines(got[which, me * slice_lines:(me + 1) * slice_lines], number), _bits(ref))
    assert device_status() == 0


def test_line_output_refuses_what_it_cannot_pack():
    from crownest_b200 import CrownestError
    rng = np.random.default_rng(0)
    fw = ops.Fp4.from_host(synth.nvfp4_matrix(66, 2048, rng), 66, 2048, 1.0)  # 66 rows: not whole lines of four
    x = torch.zeros((1, 2048), dtype=torch.bfloat16, device="cuda")
    y = torch.empty((1, 66), dtype=torch.bfloat16, device="cuda")
    buf = torch.zeros(4096, dtype=torch.int32, device="cuda")
    epoch = torch.ones(16, dtype=torch.int32, device="cuda")
    bases = (C.c_ulonglong * 2)(buf.data_ptr(), 0)
    with pytest.raises(CrownestError, match="multiples of 4"):
        ops.launch_gemv_lines(fw, x, y, (bases, 2, 0, 4096, epoch.data_ptr(), 1, 0, 0))
    fw = ops.Fp4.from_host(synth.nvfp4_matrix(64, 2048, rng), 64, 2048, 1.0)
    y = torch.empty((1, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(CrownestError, match="multiples of 4"):
        ops.launch_gemv_lines(fw, x, y, (bases, 2, 0, 4096, epoch.data_ptr(), 0, 0, 0))  # tag 0 is not a tag
