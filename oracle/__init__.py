"""CPU checker for the CUDA kernels: ctypes bindings over ``oracle/libcn_oracle.so``.

TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the tests, the smoke check and the benchmark's CPU
baseline leg may import this package; the shipped library never does. The C sources beside this
file restate the reference engine's CPU path (each function cites the reference lines it
follows); ``make -C oracle`` builds them.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcn_oracle.so")


def build(force=False):
    """Compile the C restatement with gcc (a few seconds)."""
    srcs = [os.path.join(_HERE, f) for f in ("nvfp4.c", "fp8.c", "route.c", "mul1.c", "cascade.c", "pool.c", "Makefile")]
    stale = not os.path.exists(_SO) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libcn_oracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


_u8p, _f32p, _f64p, _i32p, _u16p = (C.POINTER(t) for t in (C.c_uint8, C.c_float, C.c_double, C.c_int32, C.c_uint16))
_i64 = C.c_int64


def _declare(L):
    L.cn_o_e2m1.restype = C.c_float
    L.cn_o_e2m1.argtypes = [C.c_uint32]
    L.cn_o_ue4m3.restype = C.c_float
    L.cn_o_ue4m3.argtypes = [C.c_uint32]
    L.cn_o_scale_rule.restype = C.c_uint8
    L.cn_o_scale_rule.argtypes = [C.c_uint8]
    L.cn_o_nvfp4_dequant.argtypes = [_u8p, _i64, _i64, C.c_float, C.c_int, _f32p]
    L.cn_o_nvfp4_gemv.argtypes = [_u8p, _i64, _i64, C.c_float, _f32p, _i64, _f32p, C.c_int, C.c_int]
    L.cn_o_nvfp4_ffn.argtypes = [_u8p, _u8p, _u8p, _i64, _i64, C.c_float, C.c_float, C.c_float, C.c_float, _f32p, _i64,
                                 _f32p, C.c_int, C.c_int]
    L.cn_o_nvfp4_gemv_f64.argtypes = [_u8p, _i64, _i64, C.c_float, C.c_int, _f32p, _i64, _f64p, _f64p]
    L.cn_o_silu_mul.restype = C.c_float
    L.cn_o_silu_mul.argtypes = [C.c_float, C.c_float]
    L.cn_o_swiglu_clamp.restype = C.c_float
    L.cn_o_swiglu_clamp.argtypes = [C.c_float, C.c_float, C.c_float]
    L.cn_o_have_avx2.restype = C.c_int
    L.cn_o_e4m3_to_f32.restype = C.c_float
    L.cn_o_e4m3_to_f32.argtypes = [C.c_uint8]
    L.cn_o_f32_to_e4m3.restype = C.c_uint8
    L.cn_o_f32_to_e4m3.argtypes = [C.c_float]
    L.cn_o_fp8_dequant.argtypes = [_u8p, _i64, _i64, _f32p, _f32p]
    L.cn_o_fp8_gemv.argtypes = [_u8p, _i64, _i64, _f32p, _f32p, _i64, _f32p]
    L.cn_o_route_sigmoid_topk.argtypes = [_f32p, _f32p, _i64, C.c_int, C.c_int, C.c_float, _i32p, _f32p]
    L.cn_o_route_softmax_topk.argtypes = [_f32p, _i64, C.c_int, C.c_int, _i32p, _f32p]
    L.cn_o_moe_combine.argtypes = [C.c_int, _i64, _i64, _f32p, _f32p, _f32p, _f32p]
    L.cn_o_moe_acc_combo.argtypes = [C.c_int, _i64, _i64, _f32p, _f32p, _f32p, _f32p, _f32p]
    L.cn_o_mul1_words_per_tile.argtypes = [C.c_int, C.c_int]
    L.cn_o_mul1_end_bit.argtypes = [C.c_int, C.c_int, C.c_int]
    L.cn_o_mul1_decode.restype = C.c_uint16
    L.cn_o_mul1_decode.argtypes = [C.c_uint16]
    L.cn_o_mul1_weight.restype = C.c_float
    L.cn_o_mul1_weight.argtypes = [C.c_uint16]
    L.cn_o_f16_to_f32.restype = C.c_float
    L.cn_o_f16_to_f32.argtypes = [C.c_uint16]
    L.cn_o_f32_to_f16.restype = C.c_uint16
    L.cn_o_f32_to_f16.argtypes = [C.c_float]
    L.cn_o_mul1_reconstruct.argtypes = [_u16p, _i64, _i64, C.c_int, C.c_int, _u16p]
    L.cn_o_argmax.restype = C.c_int32
    L.cn_o_argmax.argtypes = [_f32p, _i64]
    L.cn_o_add_rmsnorm.argtypes = [_f32p, _f32p, _f32p, _f32p, _i64, _i64, C.c_float]
    L.cn_o_add_rmsnorm.restype = None
    L.cn_o_q_e2m1.restype = C.c_uint32
    L.cn_o_q_e2m1.argtypes = [C.c_float]
    L.cn_o_enc_ue4m3_up.restype = C.c_uint8
    L.cn_o_enc_ue4m3_up.argtypes = [C.c_float]
    L.cn_o_row_prescale_k.argtypes = [C.c_float]
    L.cn_o_act_cascade.argtypes = [_f32p, _i64, C.c_int, C.c_int, C.c_int, _u8p]
    L.cn_o_act_cascade.restype = None
    L.cn_o_act_cascade_dequant.argtypes = [_u8p, _i64, C.c_int, C.c_int, _f32p]
    L.cn_o_act_cascade_dequant.restype = None
    L.cn_o_mul1_synth_words.argtypes = [_u16p, _i64, C.c_uint32]
    L.cn_o_fwht128.argtypes = [_f32p]
    L.cn_o_mul1_gemv.argtypes = [_u8p, _u8p, _u8p, _i64, _i64, C.c_int, C.c_int, _f32p, _i64, _f32p, C.c_int]
    for f in (L.cn_o_mul1_trellis_bytes, L.cn_o_mul1_record_payload, L.cn_o_mul1_record_bytes):
        f.restype = _i64
        f.argtypes = [_i64, _i64, C.c_int, C.c_int]
    L.cn_o_mul1_expert_ffn.argtypes = [_u8p, _i64, _i64, C.c_int, C.c_int, C.c_float, _f32p, _i64, _f32p, C.c_int]


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def bitrate(k):
    """K (3, 3.5, ...) -> (bits, half), the set the reference accepts (converter/src/mul1.rs:57-67)."""
    bits = int(k)
    f = k - bits
    if not (1 <= bits <= 8 and (f == 0 or (f == 0.5 and bits <= 3))):
        raise ValueError(f"MUL1 trellis: unsupported bitrate {k} (integer 1..8, or 1.5 / 2.5 / 3.5)")
    return bits, int(f == 0.5)


# ---------------------------------------------------------------- NVFP4

def nvfp4_dequant(w, rows, cols, gs, rule=False):
    w = _c(w, np.uint8)
    assert w.size == rows * (cols // 64) * 36
    out = np.empty((rows, cols), np.float32)
    lib().cn_o_nvfp4_dequant(_p(w, _u8p), rows, cols, gs, int(rule), _p(out, _f32p))
    return out


def nvfp4_gemv(w, rows, cols, gs, x, threads=1, path=0):
    """x [T][cols] f32 -> y [T][rows] f32 in the reference's operation order."""
    w, x = _c(w, np.uint8), _c(x, np.float32).reshape(-1, cols)
    if w.size != rows * (cols // 64) * 36:
        raise ValueError(f"cpu_nvfp4: [{rows}, {cols}] needs {rows * (cols // 64) * 36} B, got {w.size}")
    y = np.empty((x.shape[0], rows), np.float32)
    rc = lib().cn_o_nvfp4_gemv(_p(w, _u8p), rows, cols, gs, _p(x, _f32p), x.shape[0], _p(y, _f32p), threads, path)
    if rc:
        raise ValueError(f"cpu_nvfp4: {cols} columns are not whole 64-value NVFP4 blocks")
    return y


def nvfp4_ffn(gate, up, down, hidden, inter, gs, x, limit=0.0, threads=1, path=0):
    gate, up, down = (_c(a, np.uint8) for a in (gate, up, down))
    x = _c(x, np.float32).reshape(-1, hidden)
    y = np.empty_like(x)
    rc = lib().cn_o_nvfp4_ffn(_p(gate, _u8p), _p(up, _u8p), _p(down, _u8p), hidden, inter, gs[0], gs[1], gs[2], limit,
                              _p(x, _f32p), x.shape[0], _p(y, _f32p), threads, path)
    if rc:
        raise ValueError("cpu_nvfp4: shapes are not whole NVFP4 blocks")
    return y


def nvfp4_gemv_f64(w, rows, cols, gs, x, rule=True):
    w, x = _c(w, np.uint8), _c(x, np.float32).reshape(-1, cols)
    y = np.empty((x.shape[0], rows), np.float64)
    ya = np.empty_like(y)
    lib().cn_o_nvfp4_gemv_f64(_p(w, _u8p), rows, cols, gs, int(rule), _p(x, _f32p), x.shape[0], _p(y, _f64p), _p(ya, _f64p))
    return y, ya


# ---------------------------------------------------------------- FP8

def act_cascade(x, levels=3, prescale=True, level_shift=0):
    """One f32 row -> `levels` NVFP4 levels of residuals + the row factor 2^-k (engine/src/kernels.rs:5418-5437,
    three levels there): uint8 [levels * k/64 * 36 + 4]."""
    x = _c(x, np.float32).reshape(-1)
    out = np.zeros(levels * (x.size // 64) * 36 + 4, np.uint8)
    lib().cn_o_act_cascade(_p(x, _f32p), x.size, levels, int(prescale), level_shift, _p(out, _u8p))
    return out


def act_cascade_dequant(q, k, levels=3, level_shift=0):
    """The row the MMA consumers see: (sum of the levels) * 2^-k (engine/src/kernels.rs:5462-5474)."""
    q = _c(q, np.uint8)
    out = np.empty(k, np.float32)
    lib().cn_o_act_cascade_dequant(_p(q, _u8p), k, levels, level_shift, _p(out, _f32p))
    return out


def argmax(logits):
    """argmax_k's token per row (engine/src/kernels.rs:4238-4261), ties as the kernel breaks them."""
    x = _c(logits, np.float32)
    x = x.reshape(-1, x.shape[-1])
    return np.array([lib().cn_o_argmax(_p(np.ascontiguousarray(r), _f32p), r.size) for r in x], np.int32)


def add_rmsnorm(h, y, w, eps=1e-6):
    """add_rms_1k (engine/src/kernels_p2.rs:609-633): returns (h + y, normalised output)."""
    h = _c(h, np.float32).copy()
    rows, hidden = h.shape
    out = np.empty_like(h)
    yy = None if y is None else _c(y, np.float32)
    lib().cn_o_add_rmsnorm(_p(h, _f32p), None if yy is None else _p(yy, _f32p), _p(_c(w, np.float32), _f32p), _p(out, _f32p), rows, hidden, eps)
    return h, out


def e4m3_table():
    return np.array([lib().cn_o_e4m3_to_f32(b) for b in range(256)], np.float32)


def fp8_dequant(q, rows, cols, scale):
    q, scale = _c(q, np.uint8), _c(scale, np.float32)
    out = np.empty((rows, cols), np.float32)
    if lib().cn_o_fp8_dequant(_p(q, _u8p), rows, cols, _p(scale, _f32p), _p(out, _f32p)):
        raise ValueError("FP8 NaN code - refusing to dequantize a NaN")
    return out


def fp8_gemv(q, rows, cols, scale, x):
    q, scale, x = _c(q, np.uint8), _c(scale, np.float32), _c(x, np.float32).reshape(-1, cols)
    y = np.empty((x.shape[0], rows), np.float32)
    lib().cn_o_fp8_gemv(_p(q, _u8p), rows, cols, _p(scale, _f32p), _p(x, _f32p), x.shape[0], _p(y, _f32p))
    return y


# ---------------------------------------------------------------- routing / combine

def route_sigmoid_topk(logits, bias, topk, scale):
    logits = _c(logits, np.float32)
    tokens, experts = logits.shape
    bias = _c(bias if bias is not None else np.zeros(experts), np.float32)
    ids, wts = np.empty((tokens, topk), np.int32), np.empty((tokens, topk), np.float32)
    lib().cn_o_route_sigmoid_topk(_p(logits, _f32p), _p(bias, _f32p), tokens, experts, topk, scale, _p(ids, _i32p), _p(wts, _f32p))
    return ids, wts


def route_softmax_topk(logits, topk):
    logits = _c(logits, np.float32)
    tokens, experts = logits.shape
    ids, wts = np.empty((tokens, topk), np.int32), np.empty((tokens, topk), np.float32)
    lib().cn_o_route_softmax_topk(_p(logits, _f32p), tokens, experts, topk, _p(ids, _i32p), _p(wts, _f32p))
    return ids, wts


def moe_combine(ye, weights, ys):
    """ye [T*K][H], weights [T][K], ys [T][H] or None -> y [T][H] (GLM order: experts then shared)."""
    weights = _c(weights, np.float32)
    tokens, topk = weights.shape
    ye = _c(ye, np.float32).reshape(tokens * topk, -1)
    hidden = ye.shape[1]
    y = np.empty((tokens, hidden), np.float32)
    ysp = _p(_c(ys, np.float32), _f32p) if ys is not None else None
    lib().cn_o_moe_combine(topk, tokens, hidden, _p(ye, _f32p), _p(weights, _f32p), ysp, _p(y, _f32p))
    return y


def moe_acc_combo(eo, weights, shared, sgate=None):
    """Flash-Next order: y = [sigmoid(sgate) *] shared, then y += sum_k w_k eo_k."""
    weights = _c(weights, np.float32)
    tokens, topk = weights.shape
    eo = _c(eo, np.float32).reshape(tokens * topk, -1)
    hidden = eo.shape[1]
    y = np.empty((tokens, hidden), np.float32)
    sh = _p(_c(shared, np.float32), _f32p) if shared is not None else None
    sg = _p(_c(sgate, np.float32), _f32p) if sgate is not None else None
    lib().cn_o_moe_acc_combo(topk, tokens, hidden, _p(eo, _f32p), _p(weights, _f32p), sh, sg, _p(y, _f32p))
    return y


# ---------------------------------------------------------------- MUL1

def mul1_decode_table():
    """fp16 bits of every 16-bit trellis state."""
    L = lib()
    return np.array([L.cn_o_mul1_decode(s) for s in range(65536)], np.uint16)


def mul1_reconstruct(trellis, k, n, K):
    bits, half = bitrate(K)
    trellis = _c(trellis, np.uint16)
    assert trellis.size == k // 16 * (n // 16) * lib().cn_o_mul1_words_per_tile(bits, half)
    w = np.empty((k, n), np.uint16)
    lib().cn_o_mul1_reconstruct(_p(trellis, _u16p), k, n, bits, half, _p(w, _u16p))
    return w


def mul1_synth_words(count, seed):
    out = np.empty(count, np.uint16)
    lib().cn_o_mul1_synth_words(_p(out, _u16p), count, seed & 0xFFFFFFFF)
    return out


def fwht128(v):
    v = _c(v, np.float32).copy()
    assert v.size == 128
    lib().cn_o_fwht128(_p(v, _f32p))
    return v


def mul1_gemv(trellis, suh, svh, k, n, K, x, threads=1):
    """trellis bytes, suh [k] / svh [n] fp16 bits; x [T][k] f32 -> y [T][n] f32."""
    bits, half = bitrate(K)
    tr = _c(np.frombuffer(bytes(trellis), np.uint8) if isinstance(trellis, (bytes, bytearray)) else trellis, np.uint8).reshape(-1)
    tr = tr.view(np.uint8)
    su, sv = _c(suh, np.uint16).view(np.uint8), _c(svh, np.uint16).view(np.uint8)
    x = _c(x, np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], n), np.float32)
    rc = lib().cn_o_mul1_gemv(_p(tr, _u8p), _p(su, _u8p), _p(sv, _u8p), k, n, bits, half, _p(x, _f32p), x.shape[0], _p(y, _f32p), threads)
    if rc:
        raise ValueError(f"cpu_mul1: [{k}, {n}] is not a positive multiple of 128 on both sides")
    return y


def mul1_record_bytes(hidden, inter, K):
    bits, half = bitrate(K)
    return lib().cn_o_mul1_record_bytes(hidden, inter, bits, half)


def mul1_record_payload(hidden, inter, K):
    bits, half = bitrate(K)
    return lib().cn_o_mul1_record_payload(hidden, inter, bits, half)


def mul1_trellis_bytes(k, n, K):
    bits, half = bitrate(K)
    return lib().cn_o_mul1_trellis_bytes(k, n, bits, half)


def mul1_expert_ffn(rec, hidden, inter, K, x, limit=0.0, threads=1):
    bits, half = bitrate(K)
    rec = _c(rec, np.uint8)
    if rec.size != mul1_record_bytes(hidden, inter, K):
        raise ValueError(f"cpu_mul1: record H {hidden} I {inter} K = {K} is {mul1_record_bytes(hidden, inter, K)} B, got {rec.size}")
    x = _c(x, np.float32).reshape(-1, hidden)
    y = np.empty_like(x)
    rc = lib().cn_o_mul1_expert_ffn(_p(rec, _u8p), hidden, inter, bits, half, limit, _p(x, _f32p), x.shape[0], _p(y, _f32p), threads)
    if rc:
        raise ValueError("cpu_mul1: shapes are not multiples of 128")
    return y
