"""Host-side mirror of the reference's MUL1 (EXL3 trellis) operator: ``GemvPlan`` / ``FfnPlan``
(engine/src/kernels.rs:6644-6850) and the GLM MoE step over MUL1 experts (``GpuMoePlan::experts``,
engine/src/glm5_moe.rs:741-793)."""
import ctypes as C

import torch

from ._lib import CN_BF16, CN_F32, CrownestError, check, lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def bitrate(k):
    bits = int(k)
    f = k - bits
    if not (1 <= bits <= 8 and (f == 0 or (f == 0.5 and bits <= 3))):
        raise CrownestError(f"cpu_mul1: unsupported bitrate {k} (integer 1..8, or 1.5 / 2.5 / 3.5)")
    return bits, int(f == 0.5)


def record_bytes(hidden, inter, K):
    bits, half = bitrate(K)
    wpt = 16 * bits + (8 if half else 0)
    payload = 3 * (hidden // 16) * (inter // 16) * wpt * 2 + 6 * (hidden + inter)
    return (payload + 4095) // 4096 * 4096


def _dt(x):
    return CN_BF16 if x.dtype == torch.bfloat16 else CN_F32


class Mul1Plan:
    """Scratch for up to `slots` records x `tokens` rows (GemvPlan::new(spec, slots, tokens))."""

    GATE, UP, DOWN = 0, 1, 2

    def __init__(self, hidden, inter, K, slots, tokens=1):
        if hidden <= 0 or inter <= 0 or hidden % 128 or inter % 128:
            raise CrownestError(f"cpu_mul1: [{hidden}, {inter}] is not a positive multiple of 128 on both sides")
        self.hidden, self.inter, self.K, self.slots, self.tokens = hidden, inter, K, slots, tokens
        bits, half = bitrate(K)
        h = C.c_void_p()
        check(lib().cn_mul1_plan_create(C.byref(h), hidden, inter, bits, half, slots, tokens))
        self.handle = h

    def _shape(self, which):
        return (self.hidden, self.inter) if which != self.DOWN else (self.inter, self.hidden)

    def run_slots(self, which, ptrs, x, y=None, x_div=1):
        """y[slot][t] = x[slot // x_div][t] W(which); ptrs int64 device tensor of record addresses (0 = skip)."""
        slots = ptrs.numel()
        k, n = self._shape(which)
        t = x.numel() // ((slots // x_div) * k)
        if y is None:
            y = torch.zeros((slots, t, n), dtype=x.dtype, device=x.device)
        check(lib().cn_mul1_gemv(self.handle, which, ptrs.data_ptr(), x.data_ptr(), y.data_ptr(), slots, t, x_div, _dt(x), _stream()))
        return y

    def ffn(self, ptrs, x, y=None, x_div=1, limit=0.0):
        slots = ptrs.numel()
        t = x.numel() // ((slots // x_div) * self.hidden)
        if y is None:
            y = torch.zeros((slots, t, self.hidden), dtype=x.dtype, device=x.device)
        check(lib().cn_mul1_ffn(self.handle, ptrs.data_ptr(), x.data_ptr(), y.data_ptr(), slots, t, x_div, float(limit), _dt(x), _stream()))
        return y

    def moe(self, table, ids, wts, x, shared=None, y=None, limit=0.0):
        """table int64 [E] device record addresses; ids/wts [T][topk]; shared optional f32 [T][hidden]."""
        tokens, topk = ids.shape
        if y is None:
            y = torch.empty_like(x)
        check(lib().cn_moe_mul1_run(self.handle, table.data_ptr(), ids.data_ptr(), wts.data_ptr(), None if shared is None else shared.data_ptr(),
                                    x.data_ptr(), y.data_ptr(), tokens, topk, int(table.numel()), float(limit), _dt(x), _stream()))
        return y

    def experts_only(self, table, ids, x, eo, x_div=1, limit=0.0):
        """eo[c] (f32 [combos][hidden]) = FFN of expert ids[c] on row c // x_div of x (cn_moe_mul1_experts)."""
        check(lib().cn_moe_mul1_experts(self.handle, table.data_ptr(), ids.data_ptr(), x.data_ptr(), eo.data_ptr(), ids.numel(), x_div,
                                        int(table.numel()), float(limit), _dt(x), _stream()))
        return eo

    def free(self):
        if self.handle:
            check(lib().cn_mul1_plan_destroy(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def reconstruct(trellis_u16, k, n, K):
    """fp16 bits of W_hat [k][n] on the device (codec self-check)."""
    bits, half = bitrate(K)
    out = torch.empty((k, n), dtype=torch.int16, device=trellis_u16.device)
    check(lib().cn_mul1_reconstruct(trellis_u16.data_ptr(), out.data_ptr(), k, n, bits, half, _stream()))
    return out
