"""Host-side rules of the tensor-parallel line exchange (cn_nvfp4_gemv_lines / cn_tp_recv_lines): the numbering and the
choice of line buffer that the kernels compute on the device, restated in crownest_b200.dense."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


@pytest.mark.parametrize("per_step", [1, 2, 3, 4, 63, 64])
def test_consecutive_exchanges_of_a_vector_alternate_between_its_two_buffers(per_step):
    from crownest_b200.dense import line_buffer
    seq = [line_buffer(epoch, i, per_step) for epoch in range(1, 9) for i in range(per_step)]
    assert set(seq) <= {0, 1}
    assert all(a != b for a, b in zip(seq, seq[1:])), seq[:16]


def test_numbers_are_unique_over_steps_and_never_zero():
    from crownest_b200.dense import line_number
    seen = set()
    for epoch in range(1, 50):
        for tag in (1, 2, 255, 256, 4095):
            n = line_number(epoch, tag)
            assert n != 0 and n not in seen  # a zeroed line buffer never looks like a line of a live exchange
            seen.add(n)
