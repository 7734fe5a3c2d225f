"""Seeded synthetic tensors in the shapes and value distributions of the benchmark configurations.

One generator for every test and benchmark: ``numpy.random.default_rng(seed)`` (PCG64).
NVFP4 matrices come out in the container layout the kernels consume (36-byte blocks: 4 UE4M3
scale bytes then 32 code bytes, engine/src/cpu_nvfp4.rs:8-11).
"""
import numpy as np


def f32_to_e4m3_bytes(v):
    """Round-to-nearest-even, saturating E4M3FN encode of non-negative f32 (the rule of
    engine/src/cnq.rs:1312-1361), vectorised; never produces the NaN code 0x7F."""
    v = np.asarray(v, np.float32)
    out = np.zeros(v.shape, np.uint8)
    f = np.abs(v).astype(np.float64)
    sub = f < 2.0 ** -6
    m = np.rint(f / 2.0 ** -9)
    out[sub] = np.where(m[sub] >= 8, 1 << 3, m[sub].astype(np.uint8) & 7)
    nz = ~sub
    e = np.floor(np.log2(np.where(nz, f, 1.0))).astype(np.int64)
    q = np.rint(f / 2.0 ** (e - 3))
    bump = q >= 16
    e = np.where(bump, e + 1, e)
    q = np.where(bump, 8, q)
    code = ((e + 7) << 3) | (q.astype(np.int64) & 7)
    code = np.where((e + 7 > 15) | (f >= 464.0), 0x7E, code)
    out[nz] = code[nz].astype(np.uint8)
    return out


def nvfp4_matrix(rows, cols, rng, scale_sigma=0.05):
    """[rows][cols/64] blocks: codes uniform over all 16 values, one scale byte per 16 values =
    E4M3(|N(0,1)| * scale_sigma). Returns a flat uint8 array of rows * cols / 64 * 36 bytes."""
    assert cols % 64 == 0
    blocks = rows * cols // 64
    b = np.empty((blocks, 36), np.uint8)
    b[:, 4:] = rng.integers(0, 256, size=(blocks, 32), dtype=np.uint8)
    b[:, :4] = f32_to_e4m3_bytes(np.abs(rng.standard_normal((blocks, 4), dtype=np.float32)) * np.float32(scale_sigma))
    return b.reshape(-1)


def bf16_bits(v):
    """f32 -> bf16 bit patterns, round to nearest even."""
    b = np.ascontiguousarray(v, np.float32).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def activations(m, k, rng):
    """bf16 N(0,1) activation rows as (bits [m][k] uint16, the exact f32 values)."""
    bits = bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    return bits, bf16_to_f32(bits)


# the dense decode stack of the 27B-shaped configuration: (name, rows, k) per layer
DENSE_27B = dict(hidden=5120, qkv=(40 + 8 + 8) * 128, inter=17408, layers=64)


def dense_layer_shapes(cfg=DENSE_27B):
    h, i = cfg["hidden"], cfg["inter"]
    return [("qkv", cfg["qkv"], h), ("o", h, h), ("gate", i, h), ("up", i, h), ("down", h, i)]


def dense_layer_bytes(cfg=DENSE_27B):
    return sum(r * k // 64 * 36 for _, r, k in dense_layer_shapes(cfg))
