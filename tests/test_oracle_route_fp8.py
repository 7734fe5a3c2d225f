"""Routing / combine / FP8 codec of the CPU checker against the reference's unit cases
(engine/src/glm5_moe.rs:2308-2353) and golden vectors (converter/tests/fixtures/fp8-*.tsv)."""
import hashlib
import os
import struct

import numpy as np

import oracle
from conftest import GOLDEN


def sig(x):
    return np.float32(1) / (np.float32(1) + np.exp(np.float32(-x), dtype=np.float32))


def test_router_weights_come_from_the_unbiased_scores():
    logits = np.array([[2.0, 1.0, 0.5, 0.0, -3.0]], np.float32)
    bias = np.array([0, 0, 0, 0, 2.0], np.float32)
    ids, w = oracle.route_sigmoid_topk(logits, bias, 2, 2.5)
    assert ids.tolist() == [[4, 0]]
    s4, s0 = sig(-3.0), sig(2.0)
    den = (s4 + s0) + np.float32(1e-20)
    assert np.allclose(w[0], [(s4 / den) * np.float32(2.5), (s0 / den) * np.float32(2.5)], rtol=2e-7)
    assert abs(w.sum() - 2.5) < 1e-6


def test_router_ties_go_to_the_lowest_expert_and_nan_never_wins():
    logits = np.array([[0.0, 1.0, 1.0, np.nan, 1.0, -1.0, 1.0]], np.float32)
    ids, _ = oracle.route_sigmoid_topk(logits, None, 3, 1.0)
    assert ids.tolist() == [[1, 2, 4]]
    ids, _ = oracle.route_sigmoid_topk(np.full((1, 7), np.nan, np.float32), None, 3, 1.0)
    assert ids.tolist() == [[0, 1, 2]]
    l = np.full((1, 288), -1.0, np.float32)
    for j, e in enumerate([287, 256, 3, 100, 200, 270, 1, 0]):
        l[0, e] = 5.0 - j * 0.25
    ids, _ = oracle.route_sigmoid_topk(l, None, 8, 2.5)
    assert ids.tolist() == [[287, 256, 3, 100, 200, 270, 1, 0]]


def test_softmax_topk_picks_by_probability_ties_lowest_and_renormalises():
    rng = np.random.default_rng(2)
    logits = rng.standard_normal((16, 512)).astype(np.float32)
    logits[3, 100] = logits[3, 7] = 4.5  # a tie at the top
    ids, w = oracle.route_softmax_topk(logits, 10)
    for t in range(16):
        order = np.lexsort((np.arange(512), -logits[t].astype(np.float64)))[:10]
        assert ids[t].tolist() == order.tolist()
        p = np.exp(logits[t].astype(np.float64) - logits[t].max())
        p /= p.sum()
        assert np.allclose(w[t], p[order] / p[order].sum(), rtol=1e-5)
        assert abs(w[t].sum() - 1) < 1e-6
    assert ids[3, 0] == 7 and ids[3, 1] == 100


def test_combine_sums_in_pick_order_then_adds_shared():
    ye = np.array([1, 2, 10, 20, 100, 200, 1000, 2000], np.float32).reshape(4, 2)
    w = np.array([[0.5, 0.25], [2.0, 4.0]], np.float32)
    ys = np.array([[7, 8], [9, 10]], np.float32)
    y = oracle.moe_combine(ye, w, ys)
    assert y.tolist() == [[0.5 + 2.5 + 7.0, 1.0 + 5.0 + 8.0], [200.0 + 4000.0 + 9.0, 400.0 + 8000.0 + 10.0]]
    y2 = oracle.moe_acc_combo(ye, w, ys)
    assert y2.tolist() == y.tolist()
    y3 = oracle.moe_acc_combo(ye, w, ys, sgate=np.array([0.0, 100.0], np.float32))
    assert np.allclose(y3, [[3.0 + 3.5, 6.0 + 4.0], [4200.0 + 9.0, 8400.0 + 10.0]])


def test_e4m3_table_equals_torch_float8_e4m3fn():
    n = 0
    L = oracle.lib()
    for line in open(os.path.join(GOLDEN, "fp8-e4m3fn-lut.tsv")):
        if line.startswith("#"):
            continue
        code, bits = line.split("\t")
        v = np.float32(L.cn_o_e4m3_to_f32(int(code)))
        if bits.strip() == "nan":
            assert np.isnan(v)
        else:
            assert v.view(np.uint32) == int(bits, 16), code
            n += 1
    assert n == 254
    assert L.cn_o_e4m3_to_f32(0x7E) == 448.0 and L.cn_o_e4m3_to_f32(0x01) == 2.0 ** -9


def test_e4m3_encode_round_trips_and_saturates():
    L = oracle.lib()
    for b in range(256):
        if b & 0x7F == 0x7F:
            continue
        assert L.cn_o_f32_to_e4m3(L.cn_o_e4m3_to_f32(b)) == (b if b != 0x80 else 0x80)
    assert L.cn_o_f32_to_e4m3(1e9) == 0x7E and L.cn_o_f32_to_e4m3(-1e9) == 0xFE
    assert L.cn_o_f32_to_e4m3(463.9) == 0x7E and L.cn_o_f32_to_e4m3(float("nan")) == 0x7F
    assert L.cn_o_f32_to_e4m3(2.0 ** -10) == 0  # half the smallest subnormal ties to even (zero)
    assert L.cn_o_f32_to_e4m3(3 * 2.0 ** -10) == 2


def fp8_synth(rows, cols):
    i = np.arange(rows * cols, dtype=np.uint64)
    b = (((i * np.uint64(2654435761)) >> np.uint64(7)) & np.uint64(0xFF)).astype(np.uint8)
    b = np.where(b & 0x7F == 0x7F, b ^ 1, b).astype(np.uint8)
    sr, sc = -(-rows // 128), -(-cols // 128)
    j = np.arange(sr * sc, dtype=np.uint64)
    bits = (np.uint64(0x3A000000) + ((j * np.uint64(7919)) % np.uint64(0x00800000)) * np.uint64(3)).astype(np.uint32)
    return b, bits.view(np.float32)


def test_fp8_block_dequant_matches_deepseek_and_transformers_digests():
    seen = 0
    for line in open(os.path.join(GOLDEN, "fp8-dequant.tsv")):
        if line.startswith("#"):
            continue
        who, rows, cols, want, last = line.rstrip("\n").split("\t")
        rows, cols = int(rows), int(cols)
        q, s = fp8_synth(rows, cols)
        got = oracle.fp8_dequant(q, rows, cols, s)
        assert "%08x" % struct.unpack("<I", struct.pack("<f", got.reshape(-1)[-1]))[0] == last
        assert hashlib.sha256(got.astype("<f4").tobytes()).hexdigest() == want, who
        seen += 1
    assert seen == 2


def test_fp8_gemv_is_the_dequantised_product():
    rng = np.random.default_rng(8)
    rows, cols = 200, 384
    q = rng.integers(0, 256, size=rows * cols, dtype=np.uint8)
    q = np.where(q & 0x7F == 0x7F, q ^ 1, q).astype(np.uint8)
    s = rng.uniform(0.5, 2.0, size=2 * 3).astype(np.float32) * np.float32(1e-2)
    x = rng.standard_normal((3, cols)).astype(np.float32)
    y = oracle.fp8_gemv(q, rows, cols, s, x)
    ref = x.astype(np.float64) @ oracle.fp8_dequant(q, rows, cols, s).astype(np.float64).T
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) < 1e-6
