"""The MUL1 trellis checker against the reference's golden vectors (exllamav3's own reconstruct
digests, converter/src/mul1.rs:395-414) and the reference's unit-test properties
(engine/src/cpu_mul1.rs:2695-2975)."""
import hashlib
import os

import numpy as np
import pytest

import oracle
from conftest import GOLDEN
from oracle import testkit as tk


def cases():
    out = []
    for line in open(os.path.join(GOLDEN, "exl3-mul1-decode.tsv")):
        if line.startswith("#") or not line.strip():
            continue
        f = line.rstrip("\n").split("\t")
        assert len(f) == 8
        out.append(dict(name=f[0], source=f[1], K=float(f[2]), hidden=int(f[3]), inter=int(f[4]), want=f[5:8]))
    return out


def expert(c):
    """trellis words of gate, up, down"""
    shapes = [(c["hidden"], c["inter"]), (c["hidden"], c["inter"]), (c["inter"], c["hidden"])]
    tb = oracle.mul1_trellis_bytes(c["hidden"], c["inter"], c["K"])
    if c["source"].startswith("synth:"):
        seed = int(c["source"][6:])
        return [(oracle.mul1_synth_words(tb // 2, seed + 3 * i), k, n) for i, (k, n) in enumerate(shapes)]
    raw = np.fromfile(os.path.join(GOLDEN, c["source"]), np.uint8)
    assert raw.size == oracle.mul1_record_payload(c["hidden"], c["inter"], c["K"])
    return [(raw[i * tb:(i + 1) * tb].view(np.uint16), k, n) for i, (k, n) in enumerate(shapes)]


@pytest.mark.parametrize("c", cases(), ids=lambda c: c["name"])
def test_decode_is_byte_identical_to_exllamav3(c):
    for (tr, k, n), want in zip(expert(c), c["want"]):
        got = hashlib.sha256(oracle.mul1_reconstruct(tr, k, n, c["K"]).tobytes()).hexdigest()
        assert got == want, (c["name"], k, n)


def test_case_set_has_glm_shapes_and_quantizer_outputs():
    cs = cases()
    assert len(cs) == 7
    assert any(c["hidden"] == 4096 and c["inter"] == 2048 for c in cs)
    assert any(not c["source"].startswith("synth:") for c in cs)


def test_glm_record_size_at_3_bit():
    assert oracle.mul1_trellis_bytes(4096, 2048, 3.0) == 3_145_728
    assert oracle.mul1_record_payload(4096, 2048, 3.0) == 9_474_048
    assert oracle.mul1_record_bytes(4096, 2048, 3.0) == 9_474_048
    total = 0
    for line in open(os.path.join(GOLDEN, "exl3-mul1-glm-sizes.tsv")):
        if line.startswith("#"):
            continue
        f = line.split("\t")
        assert int(f[2]) == 3_145_728
        total += int(f[2]) + int(f[3]) + int(f[4])
    assert total == 9_474_048
    # the benchmark's expert shape: hidden 4096, inter 1536
    assert oracle.mul1_trellis_bytes(4096, 1536, 3.0) == 2_359_296
    assert oracle.mul1_record_payload(4096, 1536, 3.0) == 7_111_680
    assert oracle.mul1_record_bytes(4096, 1536, 3.0) == 7_114_752
    for h, i, K in [(256, 128, 3.0), (384, 256, 2.0), (128, 128, 4.0), (256, 128, 3.5)]:
        assert oracle.mul1_record_bytes(h, i, K) % 4096 == 0


def test_bitrate_set_is_exllamav3s():
    L = oracle.lib()
    for K in (1.0, 1.5, 2.0, 2.5, 3.0, 3.5, 4.0, 8.0):
        oracle.bitrate(K)
    for K in (0.0, 0.5, 4.5, 9.0, 3.05, 3.25):
        with pytest.raises(ValueError):
            oracle.bitrate(K)
    assert L.cn_o_mul1_words_per_tile(3, 0) == 48 and L.cn_o_mul1_words_per_tile(3, 1) == 56


def test_scalar_weight_equals_the_codec_for_every_state():
    # engine/src/cpu_mul1.rs:2918-2921: the 1021-entry table path gives the codec's fp16 value
    L = oracle.lib()
    table = oracle.mul1_decode_table()
    as_f32 = table.view(np.float16).astype(np.float32)
    got = np.array([L.cn_o_mul1_weight(s) for s in range(65536)], np.float32)
    assert np.array_equal(got.view(np.uint32), as_f32.view(np.uint32))
    assert np.all(np.isfinite(got)) and got.min() == -3.453125 and 3.3 < got.max() < 3.5


def test_fwht_is_the_sylvester_matrix():
    H = np.array([[1.0]])
    while H.shape[0] < 128:
        H = np.block([[H, H], [H, -H]])
    rng = np.random.default_rng(7)
    v = rng.integers(-8, 9, size=128).astype(np.float32)  # small integers: exact in f32
    assert np.array_equal(oracle.fwht128(v), (H @ v.astype(np.float64)).astype(np.float32))


def _reference_f64(tr, suh, svh, k, n, K, x):
    """W = diag(suh) H W_hat H diag(svh) / 128 in f64 (engine/src/cpu_mul1.rs:26-29)"""
    what = oracle.mul1_reconstruct(tr, k, n, K).view(np.float16).astype(np.float64)
    H = np.array([[1.0]])
    while H.shape[0] < 128:
        H = np.block([[H, H], [H, -H]])
    su, sv = suh.view(np.float16).astype(np.float64), svh.view(np.float16).astype(np.float64)
    xs = x.astype(np.float64) * su
    xh = (xs.reshape(x.shape[0], k // 128, 128) @ H).reshape(x.shape[0], k)
    yp = xh @ what
    absyp = np.abs(xh) @ np.abs(what)
    y = (yp.reshape(x.shape[0], n // 128, 128) @ H).reshape(x.shape[0], n) / 128 * sv
    bound = (absyp.reshape(x.shape[0], n // 128, 128) @ np.abs(H)).reshape(x.shape[0], n) / 128 * np.abs(sv)
    return y, bound


@pytest.mark.parametrize("K,k,n", [(3.0, 256, 128), (2.0, 384, 256), (3.5, 256, 128), (4.0, 128, 128), (3.0, 512, 384)])
def test_gemv_holds_the_fp32_bound_and_thread_independence(K, k, n):
    rng = np.random.default_rng(180)
    tr = rng.integers(0, 65536, size=oracle.mul1_trellis_bytes(k, n, K) // 2, dtype=np.uint16)
    sgn = lambda m: (rng.choice([-1.0, 1.0], size=m) * rng.uniform(0.5, 1.5, size=m)).astype(np.float16).view(np.uint16)
    suh, svh = sgn(k), sgn(n)
    for t in (1, 3, 5):
        x = rng.uniform(-2, 2, size=(t, k)).astype(np.float32)
        y = oracle.mul1_gemv(tr.view(np.uint8), suh, svh, k, n, K, x, threads=1)
        yr, bound = _reference_f64(tr, suh, svh, k, n, K, x)
        steps = k // 4 + 18  # engine/src/cpu_mul1.rs:93-96 `rounding_steps`
        nu = steps * 2.0 ** -24
        assert np.max(np.abs(y - yr) / (nu / (1 - nu) * bound + 1e-30)) <= 1.0
        for th in (2, 8):
            assert np.array_equal(oracle.mul1_gemv(tr.view(np.uint8), suh, svh, k, n, K, x, threads=th).view(np.uint32), y.view(np.uint32))


def test_rounding_step_constants():
    # engine/src/cpu_mul1.rs:2965-2966: n = k/4 + 18 -> 1042 at k 4096, 530 at k 2048
    assert 4096 // 4 + 18 == 1042 and 2048 // 4 + 18 == 530


def test_expert_ffn_is_gemv_activation_gemv_and_checks_the_record():
    hidden, inter, K = 256, 128, 3.0
    rec = tk.mul1_record(11, hidden, inter, K)
    assert rec.size == oracle.mul1_record_bytes(hidden, inter, K)
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, size=(2, hidden)).astype(np.float32)
    y = oracle.mul1_expert_ffn(rec, hidden, inter, K, x, threads=3)
    tb = oracle.mul1_trellis_bytes(hidden, inter, K)
    at = 3 * tb
    take = lambda nbytes, at=[at]: (rec[at[0]:at[0] + nbytes].view(np.uint16), at.__setitem__(0, at[0] + nbytes))[0]
    gs, gv, us, uv, ds, dv = take(2 * hidden), take(2 * inter), take(2 * hidden), take(2 * inter), take(2 * inter), take(2 * hidden)
    g = oracle.mul1_gemv(rec[:tb], gs, gv, hidden, inter, K, x)
    u = oracle.mul1_gemv(rec[tb:2 * tb], us, uv, hidden, inter, K, x)
    L = oracle.lib()
    h = np.array([L.cn_o_silu_mul(a, b) for a, b in zip(g.ravel(), u.ravel())], np.float32).reshape(2, inter)
    assert np.array_equal(oracle.mul1_gemv(rec[2 * tb:3 * tb], ds, dv, inter, hidden, K, h).view(np.uint32), y.view(np.uint32))
    with pytest.raises(ValueError):
        oracle.mul1_expert_ffn(rec[:-4096], hidden, inter, K, x)
    with pytest.raises(ValueError):
        oracle.mul1_gemv(rec[:tb], gs, gv, 200, 128, K, np.zeros((1, 200), np.float32))
