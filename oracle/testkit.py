"""The reference's own test generators, restated in numpy (TEST INFRASTRUCTURE, not product code).

The reference's golden MoE fixtures store outputs only; their inputs are regenerated from a seed
and checked against the sha256 digests in the fixture's manifest. This module reproduces those
generators bit for bit:
- `SplitMix`: the splitmix64 stream and its `f(a)` uniform (engine/src/cpu_mul1.rs:2476-2490);
- `glm5_synth`: the router / shared / dense weights and activations of
  engine/src/glm5_moe.rs:2355-2409;
- `mul1_record`: the synthetic MUL1 expert record of engine/src/cpu_mul1.rs:2656-2684.
"""
import hashlib

import numpy as np

from . import mul1_record_bytes, mul1_synth_words, mul1_trellis_bytes

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


class SplitMix:
    """splitmix64, vectorised: `next_n(n)` returns the next n outputs of the stream."""

    def __init__(self, seed):
        self.state = np.uint64(seed)

    def next_n(self, n):
        with np.errstate(over="ignore"):
            s = self.state + _GOLDEN * np.arange(1, n + 1, dtype=np.uint64)
            self.state = np.uint64(s[-1]) if n else self.state
            z = s
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            return z ^ (z >> np.uint64(31))

    @staticmethod
    def to_f(u, a):
        """uniform in [-a, a): ((u >> 40) as f32 / 2^24 * 2 - 1) * a, every step in f32"""
        v = (u >> np.uint64(40)).astype(np.float32) / np.float32(16777216.0)
        return (v * np.float32(2.0) - np.float32(1.0)) * np.float32(a)

    def f_n(self, n, a):
        return self.to_f(self.next_n(n), a)


def f32_to_bf16_bits(v):
    """engine/src/glm5_moe.rs:2370-2373: round to nearest even on the bit pattern"""
    b = np.ascontiguousarray(v, np.float32).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def _nvfp4(rows, cols, rng):
    """engine/src/glm5_moe.rs:2385-2395: scale bytes 0x30..0x3F, random code bytes"""
    blocks = rows * cols // 64
    u = rng.next_n(blocks * 36).reshape(blocks, 36)
    b = (u & np.uint64(0xFF)).astype(np.uint8)
    b[:, :4] = (np.uint64(0x30) + (u[:, :4] % np.uint64(16))).astype(np.uint8)
    return b.reshape(-1)


GLM5 = dict(hidden=4096, experts=288, topk=8, expert_inter=2048, shared_inter=2048, dense_inter=12288,
            routed_scaling=2.5, swiglu_limit=10.0, K=3.0)
TR, TM, TD = 64, 4, 2
SEED = 0x01646105
X_AMP, ROUTER_AMP, BIAS_AMP, NVFP4_GS = 0.17, 0.55, 0.09, np.float32(0.3)
RECORD_SEED = 0x1640


def glm5_synth(with_dense=True):
    """The inputs of the glm5 MoE golden, in the reference's draw order."""
    h, e = GLM5["hidden"], GLM5["experts"]
    rng = SplitMix(SEED)
    s = {}
    s["router_w"] = f32_to_bf16_bits(rng.f_n(e * h, ROUTER_AMP))
    s["bias"] = rng.f_n(e, BIAS_AMP)

    def mats(inter):
        return [(_nvfp4(inter, h, rng), inter, h), (_nvfp4(inter, h, rng), inter, h), (_nvfp4(h, inter, rng), h, inter)]

    s["shared"] = mats(GLM5["shared_inter"])
    s["dense"] = mats(GLM5["dense_inter"])
    s["x_route"] = rng.f_n(TR * h, X_AMP).reshape(TR, h)
    s["x_moe"] = rng.f_n(TM * h, X_AMP).reshape(TM, h)
    s["x_dense"] = rng.f_n(TD * h, X_AMP).reshape(TD, h)
    return s


def input_shas(s):
    """sha256 of every encoded input, keyed as the golden's manifest keys them"""
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    m = {"router.bf16": sha(s["router_w"]), "bias.f32": sha(s["bias"])}
    for name in ("shared", "dense"):
        for p, mat in zip(("gate", "up", "down"), s[name]):
            m[f"{name}_{p}.nvfp4"] = sha(mat[0])
    for k in ("x_route", "x_moe", "x_dense"):
        m[k + ".f32"] = sha(s[k])
    return m


def _synth_scales(n, rng):
    """fp16 values of random sign and magnitude 0.5 .. 1.5 (two draws per value)"""
    u = rng.next_n(2 * n).reshape(n, 2)
    mag = 1.0 + SplitMix.to_f(u[:, 0], 0.5).astype(np.float64)
    sign = np.where((u[:, 1] & np.uint64(1)) == 0, 1.0, -1.0)
    return (mag * sign).astype(np.float16).view(np.uint16)


def mul1_record(seed, hidden, inter, K):
    """The padded record of a "synth:<seed>" case: trellis streams seed + 3 i, then synthetic scales."""
    size = mul1_record_bytes(hidden, inter, K)
    words = mul1_trellis_bytes(hidden, inter, K) // 2
    rng = SplitMix(seed ^ 0x180)
    parts = [mul1_synth_words(words, seed + 3 * i) for i in range(3)]
    for k, n in ((hidden, inter), (hidden, inter), (inter, hidden)):
        parts.append(_synth_scales(k, rng))
        parts.append(_synth_scales(n, rng))
    rec = np.concatenate(parts).view(np.uint8)
    out = np.zeros(size, np.uint8)
    out[: rec.size] = rec
    return out


def glm5_expert_record(e):
    return mul1_record(RECORD_SEED + 9 * e, GLM5["hidden"], GLM5["expert_inter"], GLM5["K"])
