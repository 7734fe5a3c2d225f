"""Host-side mirror of the reference engine's NVFP4 operator interface over the C ABI.

The reference's Rust host code holds ``Fp4 { w, gs }`` device buffers (engine/src/weights.rs:9-12)
and calls ``PW::launch_gemv`` / ``Engine::dense_proj`` / ``Engine::dense_ffn_w``
(engine/src/gen.rs:234-266, :3915, :3974), which enqueue kernels on the current stream and
return. The classes below keep those names and argument meanings; torch is used only to own
device memory and to name the current stream.
"""
import numpy as np
import torch

from . import _lib
from ._lib import CN_BF16, CN_F32, CrownestError, check, lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t):
    if t.dtype == torch.bfloat16:
        return CN_BF16
    if t.dtype == torch.float32:
        return CN_F32
    raise CrownestError(f"activations must be bf16 or f32, got {t.dtype}")


class Fp4:
    """One NVFP4 matrix on the device: ``w`` the container bytes [rows][k/64][36], ``gs`` a one-float
    device buffer with the tensor scale (engine/src/weights.rs:9-12, GpuNvfp4 engine/src/glm5_moe.rs:353)."""

    def __init__(self, w, gs, rows, cols):
        if cols <= 0 or cols % 64 != 0:
            raise CrownestError(f"cpu_nvfp4: {cols} columns are not whole 64-value NVFP4 blocks")
        want = rows * (cols // 64) * 36
        if w.numel() != want or w.dtype != torch.uint8:
            raise CrownestError(f"cpu_nvfp4: [{rows}, {cols}] needs {want} B, got {w.numel()}")
        self.w, self.gs, self.rows, self.cols = w, gs, rows, cols

    @classmethod
    def from_host(cls, bytes_, rows, cols, global_scale, device="cuda"):
        w = torch.from_numpy(np.ascontiguousarray(bytes_, np.uint8)).to(device)
        gs = torch.tensor([global_scale], dtype=torch.float32, device=device)
        return cls(w, gs, rows, cols)

    def rows_slice(self, r0, r1):
        """Rows r0..r1 as a view (the tensor-parallel shard of an [out][in] matrix)."""
        rb = self.cols // 64 * 36
        return Fp4(self.w[r0 * rb:r1 * rb], self.gs, r1 - r0, self.cols)


def launch_gemv(w: Fp4, x, y=None, ldy=None):
    """y[m][r] = sum_k W[r][k] x[m][k] for x [M][k] (M <= 8) - PW::launch_gemv / launch_gemv1,
    Engine::proj_m (engine/src/gen.rs:234-266, :5455). Enqueues and returns ``y``."""
    x2 = x.reshape(-1, w.cols)
    m = x2.shape[0]
    if y is None:
        y = torch.empty((m, w.rows), dtype=x.dtype, device=x.device)
    ld = ldy if ldy is not None else (y.stride(0) if y.dim() == 2 else w.rows)
    check(lib().cn_nvfp4_gemv(w.w.data_ptr(), w.gs.data_ptr(), x2.data_ptr(), y.data_ptr(), w.rows, w.cols, m, ld,
                              _dtype_code(x), _stream()))
    return y


def launch_gemm(w: Fp4, x, y=None, workspace=None):
    """Y[t][n] = gs * sum_k X[t][k] W[n][k] for any number of rows t - the prompt GEMM (launch_mma_d,
    engine/src/gen.rs:2491; glm5_gemm_fp4_tc, engine/src/kernels_glm5_moe.cu:349) on tcgen05 tensor cores.
    ``workspace``: a uint8 device tensor of at least ``gemm_workspace_bytes(w.cols, t)`` bytes (allocated when absent)."""
    x2 = x.reshape(-1, w.cols)
    m = x2.shape[0]
    if y is None:
        y = torch.empty((m, w.rows), dtype=x.dtype, device=x.device)
    need = gemm_workspace_bytes(w.cols, m)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib().cn_nvfp4_gemm(w.w.data_ptr(), w.gs.data_ptr(), x2.data_ptr(), y.data_ptr(), w.rows, w.cols, m, y.stride(0), _dtype_code(x),
                              workspace.data_ptr(), workspace.numel(), _stream()))
    return y


def gemm_workspace_bytes(k, m):
    return int(lib().cn_nvfp4_gemm_workspace_bytes(k, m))


class Fp4Packed:
    """An NVFP4 matrix re-laid once at load for the block-scaled FP4 tensor-core GEMM (cn_nvfp4_bs_repack): stage images
    of 128 rows x 256 columns with their scale bytes (0x7F read as 0x7E, bit 7 cleared - the reference rewrites its slabs
    the same way at load, engine/src/residency.rs:119-137)."""

    def __init__(self, w: Fp4):
        n = int(lib().cn_nvfp4_bs_packed_bytes(w.rows, w.cols))
        if n == 0:
            raise CrownestError(f"block-scaled GEMM: k = {w.cols} must be a multiple of 256")
        self.packed = torch.empty(n, dtype=torch.uint8, device=w.w.device)
        check(lib().cn_nvfp4_bs_repack(w.w.data_ptr(), self.packed.data_ptr(), w.rows, w.cols, _stream()))
        self.gs, self.rows, self.cols = w.gs, w.rows, w.cols


def launch_gemm_fp4(w: Fp4Packed, x, y=None, workspace=None):
    """Y[t][n] = gs * sum_k X[t][k] W[n][k] on the block-scaled FP4 MMA (tcgen05 kind::mxf4nvf4): gemm_fp4_dense
    (engine/src/kernels.rs:533) with the activations as a five-level NVFP4 cascade (the reference's act_cascade,
    engine/src/kernels.rs:5354-5475, has three)."""
    x2 = x.reshape(-1, w.cols)
    m = x2.shape[0]
    if y is None:
        y = torch.empty((m, w.rows), dtype=x.dtype, device=x.device)
    need = int(lib().cn_nvfp4_bs_workspace_bytes(w.rows, w.cols, m))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib().cn_nvfp4_bs_gemm(w.packed.data_ptr(), w.gs.data_ptr(), x2.data_ptr(), y.data_ptr(), w.rows, w.cols, m, y.stride(0), _dtype_code(x),
                                 workspace.data_ptr(), workspace.numel(), _stream()))
    return y


def act_cascade(x, levels=3):
    """The activation cascade in the reference's byte layout (quant_x_fp4, engine/src/kernels.rs:351): uint8
    [rows][levels * k/64 * 36 + 4]."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, k = x2.shape
    out = torch.empty((rows, levels * (k // 64) * 36 + 4), dtype=torch.uint8, device=x.device)
    check(lib().cn_nvfp4_act_cascade(x2.data_ptr(), out.data_ptr(), rows, k, levels, _dtype_code(x), _stream()))
    return out


dense_proj = launch_gemv  # Engine::dense_proj (engine/src/gen.rs:3915): same operator at t == 1 and t <= 4


def launch_gemv_lines(w: Fp4, x, y, lines, gu: Fp4 = None, limit=0.0):
    """The one-row bf16 GEMV (or fused gate/up) of a tensor-parallel rank whose output rows also go out as 16-byte lines to
    the other ranks' line buffers (cn_nvfp4_gemv_lines / _gu_lines); `lines` = (bases, world, row0, stride, step counter
    address, tag, buffer, flip) as `PeerExchange.line_args` gives them. The receiving side is cn_tp_recv_lines."""
    bases, world, row0, stride, epoch, tag, buf, flip = lines
    if x.dtype != torch.bfloat16 or x.numel() != w.cols:
        raise CrownestError("line output takes one bf16 activation row")
    if gu is None:
        check(lib().cn_nvfp4_gemv_lines(w.w.data_ptr(), w.gs.data_ptr(), x.data_ptr(), y.data_ptr(), w.rows, w.cols, bases, world, row0, stride, epoch,
                                        tag, buf, flip, _stream()))
    else:
        check(lib().cn_nvfp4_gemv_gu_lines(w.w.data_ptr(), gu.w.data_ptr(), w.gs.data_ptr(), gu.gs.data_ptr(), x.data_ptr(), y.data_ptr(), w.rows,
                                           w.cols, float(limit), bases, world, row0, stride, epoch, tag, buf, flip, _stream()))
    return y


def launch_gemv_gu(gate: Fp4, up: Fp4, x, h=None, limit=0.0):
    """h = act(gate x, up x): gemv_nvfp4_gu / _gum, the first half of Engine::dense_ffn_w
    (engine/src/gen.rs:3974-3981). limit > 0 selects the clamped SwiGLU."""
    if (gate.rows, gate.cols) != (up.rows, up.cols):
        raise CrownestError(f"cpu_nvfp4: expert shapes gate [{gate.rows}, {gate.cols}], up [{up.rows}, {up.cols}] do not fit together")
    x2 = x.reshape(-1, gate.cols)
    m = x2.shape[0]
    if h is None:
        h = torch.empty((m, gate.rows), dtype=x.dtype, device=x.device)
    check(lib().cn_nvfp4_gemv_gu(gate.w.data_ptr(), up.w.data_ptr(), gate.gs.data_ptr(), up.gs.data_ptr(), x2.data_ptr(),
                                 h.data_ptr(), gate.rows, gate.cols, m, h.stride(0) if h.dim() == 2 else gate.rows,
                                 float(limit), _dtype_code(x), _stream()))
    return h


def dense_ffn_w(gate: Fp4, up: Fp4, down: Fp4, x, limit=0.0):
    """y = down(act(gate x, up x)) - Engine::dense_ffn_w (engine/src/gen.rs:3974), GpuFfnPlan::run
    (engine/src/glm5_moe.rs:461) with limit > 0."""
    return launch_gemv(down, launch_gemv_gu(gate, up, x, limit=limit))


class GemvSeq:
    """A chain of one-row GEMV steps run by one persistent launch (cn_nvfp4_seq_*): the fused form of
    Engine::dense_ffn_w (engine/src/gen.rs:3974-3990) and of a stack of projections. Steps are added with
    ``gemv`` / ``gemv_gu`` (which return the step's index, to be named as a later step's ``after``), then ``build()``
    once and ``run()`` per token. The tensors named by the steps are borrowed: keep them alive."""

    def __init__(self):
        self.steps, self.keep, self.handle = [], [], None

    def _add(self, w, up, x, y, limit, after):
        if x.dtype != torch.bfloat16 or x.numel() != w.cols:
            raise CrownestError(f"gemv chain: x must be one bf16 row of {w.cols} values")
        if y.numel() != w.rows or y.dtype not in (torch.bfloat16, torch.float32):
            raise CrownestError(f"gemv chain: y must be one bf16 or f32 row of {w.rows} values")
        st = _lib.GemvStep(w.w.data_ptr(), None if up is None else up.w.data_ptr(), w.gs.data_ptr(), None if up is None else up.gs.data_ptr(),
                           x.data_ptr(), y.data_ptr(), w.rows, w.cols, float(limit), -1 if after is None else int(after),
                           int(y.dtype == torch.float32))
        self.steps.append(st)
        self.keep += [w, up, x, y]
        return len(self.steps) - 1

    def gemv(self, w: Fp4, x, y, after=None):
        return self._add(w, None, x, y, 0.0, after)

    def gemv_gu(self, gate: Fp4, up: Fp4, x, h, limit=0.0, after=None):
        if (gate.rows, gate.cols) != (up.rows, up.cols):
            raise CrownestError("gemv chain: gate and up shapes differ")
        return self._add(gate, up, x, h, limit, after)

    def build(self):
        import ctypes as C
        arr = (_lib.GemvStep * len(self.steps))(*self.steps)
        h = C.c_void_p()
        check(lib().cn_nvfp4_seq_create(C.byref(h), arr, len(self.steps)))
        self.handle = h
        return self

    def run(self):
        check(lib().cn_nvfp4_seq_run(self.handle, _stream()))

    def free(self):
        if self.handle:
            check(lib().cn_nvfp4_seq_destroy(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def add_norm(h, y, w, out=None, eps=1e-6):
    """h += y (y may be None), out = h * rsqrt(mean(h^2) + eps) * (1 + w): Engine::add_norm / add_rms_1k
    (engine/src/kernels_p2.rs:609). h, y, out f32 [rows][hidden], w f32 [hidden]; h is updated in place."""
    rows, hidden = h.shape
    if out is None:
        out = torch.empty_like(h)
    check(lib().cn_add_rmsnorm(h.data_ptr(), None if y is None else y.data_ptr(), w.data_ptr(), out.data_ptr(), rows, hidden, float(eps), _stream()))
    return out


def argmax(logits):
    """Token id per row with the tie rule of argmax_k (engine/src/kernels.rs:4238)."""
    rows, n = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    check(lib().cn_argmax(logits.data_ptr(), out.data_ptr(), rows, n, logits.stride(0), _dtype_code(logits), _stream()))
    return out


def lm_head_argmax(w: Fp4, x, logits=None):
    """logits = lm_head x and their argmax per row (engine/src/gen.rs:5638-5641): returns (tokens int32 [m], logits [m][vocab])."""
    x2 = x.reshape(-1, w.cols)
    m = x2.shape[0]
    if logits is None:
        logits = torch.empty((m, w.rows), dtype=x.dtype, device=x.device)
    tokens = torch.empty(m, dtype=torch.int32, device=x.device)
    check(lib().cn_lm_head_argmax(w.w.data_ptr(), w.gs.data_ptr(), x2.data_ptr(), logits.data_ptr(), tokens.data_ptr(), w.rows, w.cols, m,
                                  _dtype_code(x), _stream()))
    return tokens, logits


def dequant(w: Fp4, rule=False):
    """f32 [rows][cols] = e2m1(code) * (ue4m3(byte) * gs): dequant_fp4_flat (engine/src/kernels.rs:1460)."""
    out = torch.empty((w.rows, w.cols), dtype=torch.float32, device=w.w.device)
    check(lib().cn_nvfp4_dequant(w.w.data_ptr(), w.gs.data_ptr(), out.data_ptr(), w.rows, w.cols, int(rule), _stream()))
    return out


def fp8_gemv(w, scale, x, rows, cols, y=None):
    """y[m][r] for E4M3FN weights [rows][cols] (uint8) with f32 scales per 128x128 tile
    (the codec of converter/src/fp8.rs:44-82); x [M][cols], M <= 8."""
    x2 = x.reshape(-1, cols)
    m = x2.shape[0]
    if w.numel() != rows * cols:
        raise CrownestError(f"fp8: {w.numel()} FP8 bytes for shape [{rows}, {cols}]")
    sr, sc = -(-rows // 128), -(-cols // 128)
    if scale.numel() != sr * sc:
        raise CrownestError(f"fp8: {scale.numel()} scales, the 128x128 grid of [{rows}, {cols}] needs [{sr}, {sc}] = {sr * sc}")
    if y is None:
        y = torch.empty((m, rows), dtype=x.dtype, device=x.device)
    check(lib().cn_fp8_gemv(w.data_ptr(), scale.data_ptr(), x2.data_ptr(), y.data_ptr(), rows, cols, m, y.stride(0), _dtype_code(x), _stream()))
    return y
