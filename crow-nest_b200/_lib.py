"""ctypes binding of ``libcrownest_b200.so`` (the C ABI declared in ``include/crownest_ops.h``).

There is no fallback: when the shared library is missing or a call returns a non-zero status the
caller gets an exception. ``build()`` compiles the library in tree with nvcc for sm_100a.
"""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libcrownest_b200.so")
CSRC = os.path.join(_HERE, "csrc")

CN_F32, CN_BF16, CN_BF16_IN_F32_OUT = 0, 1, 2
CN_MAX_M = 8


class CrownestError(RuntimeError):
    pass


def build(force=False, jobs=8):
    """nvcc -gencode arch=compute_100a,code=sm_100a over csrc/*.cu (cross-compiles without a GPU)."""
    cmd = ["make", "-C", CSRC, f"-j{jobs}"]
    if force:
        cmd.append("-B")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise CrownestError("building libcrownest_b200.so failed:\n" + r.stdout[-4000:] + r.stderr[-4000:])
    return SO_PATH


_lib = None

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float

# name -> argtypes; every entry point returns int status unless listed in _RESTYPES
_SIGS = {
    "cn_nvfp4_gemv": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "cn_nvfp4_gemv_gu": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp],
    "cn_nvfp4_dequant": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "cn_add_rmsnorm": [_vp, _vp, _vp, _vp, _i, _i, _f, _vp],
    "cn_argmax": [_vp, _vp, _i, _i, _i, _i, _vp],
    "cn_lm_head_argmax": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "cn_nvfp4_seq_create": [C.POINTER(C.c_void_p), _vp, _i],
    "cn_nvfp4_seq_run": [_vp, _vp],
    "cn_nvfp4_seq_destroy": [_vp],
    "cn_route_softmax_topk": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "cn_route_sigmoid_topk": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "cn_moe_sort": [_vp, _vp, _i, _i, _vp],
    "cn_moe_combine": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "cn_moe_nvfp4_plan_create": [C.POINTER(C.c_void_p), _i, _i, _i, _i, _i, _i],
    "cn_moe_nvfp4_plan_destroy": [_vp],
    "cn_moe_nvfp4_run": [_vp] * 16 + [_i, _f, _i, _vp],
    "cn_moe_nvfp4_experts": [_vp] * 11 + [_i, _i, _f, _i, _vp],
    "cn_moe_nvfp4_finish": [_vp] * 12 + [_i, _f, _i, _vp],
    "cn_moe_nvfp4_shared_begin": [_vp] * 6 + [_i, _f, _i, _vp],
    "cn_moe_mul1_experts": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "cn_ep_flag_bytes": [],
    "cn_ep_dispatch": [C.POINTER(C.c_void_p), _i, _i, _i, _i, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp],
    "cn_ep_return": [C.POINTER(C.c_void_p), _i, _i, _i, _i, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _vp, _vp, _vp, _vp],
    "cn_nvfp4_gemm": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, C.c_size_t, _vp],
    "cn_nvfp4_gemm_workspace_bytes": [_i, _i],
    "cn_nvfp4_bs_packed_bytes": [_i, _i],
    "cn_nvfp4_bs_repack": [_vp, _vp, _i, _i, _vp],
    "cn_nvfp4_bs_workspace_bytes": [_i, _i, _i],
    "cn_nvfp4_bs_gemm": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, C.c_size_t, _vp],
    "cn_nvfp4_act_cascade": [_vp, _vp, _i, _i, _i, _i, _vp],
    "cn_peer_export": [_vp, _vp, C.POINTER(C.c_size_t)],
    "cn_peer_open": [_vp, C.c_size_t, C.POINTER(C.c_void_p)],
    "cn_peer_close": [_vp, C.c_size_t],
    "cn_tp_allgather": [C.POINTER(C.c_void_p), _i, _i, C.c_size_t, C.c_size_t, C.c_size_t, _vp],
    "cn_tp_allgather_ll": [C.POINTER(C.c_void_p), _i, _i, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, _vp],
    "cn_smem_book": [_vp, _i, _i, _i],
    "cn_tp_epoch_advance": [_vp, _vp],
    "cn_tp_recv_lines": [_vp, _i, _i, C.c_size_t, C.c_size_t, C.c_size_t, _vp, _i, _i, _i, _vp],
    "cn_nvfp4_gemv_lines": [_vp, _vp, _vp, _vp, _i, _i, C.POINTER(C.c_ulonglong), _i, _i, C.c_size_t, _vp, _i, _i, _i, _vp],
    "cn_nvfp4_gemv_gu_lines": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, C.POINTER(C.c_ulonglong), _i, _i, C.c_size_t, _vp, _i, _i, _i, _vp],
    "cn_mul1_plan_create": [C.POINTER(C.c_void_p), _i, _i, _i, _i, _i, _i],
    "cn_mul1_plan_destroy": [_vp],
    "cn_mul1_gemv": [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "cn_mul1_ffn": [_vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "cn_moe_mul1_run": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp],
    "cn_mul1_gemv_noalloc": [_i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "cn_mul1_reconstruct": [_vp, _vp, _i, _i, _i, _i, _vp],
    "cn_fp8_gemv": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "cn_device_status": [C.POINTER(C.c_int)],
    "cn_last_error_string": [],
    "cn_version": [],
}
_RESTYPES = {"cn_last_error_string": C.c_char_p, "cn_version": C.c_char_p}


class GemvStep(C.Structure):
    """cn_gemv_step of include/crownest_ops.h"""
    _fields_ = [("w", _vp), ("w_up", _vp), ("gs", _vp), ("gs_up", _vp), ("x", _vp), ("y", _vp), ("rows", _i), ("k", _i), ("limit", _f),
                ("after", _i), ("out_f32", _i)]


def exported_symbols():
    """Names the header declares; the CPU test checks the library exports each of them."""
    return sorted(_SIGS)


_RESTYPES_INIT = {"cn_nvfp4_gemm_workspace_bytes": C.c_size_t, "cn_ep_flag_bytes": C.c_size_t, "cn_nvfp4_bs_packed_bytes": C.c_size_t,
                  "cn_nvfp4_bs_workspace_bytes": C.c_size_t}


def register(name, argtypes, restype=C.c_int):
    """Other modules of the package add their entry points here before the first load."""
    _SIGS[name] = argtypes
    if restype is not C.c_int:
        _RESTYPES[name] = restype


def use_trace_library():
    """Load the diagnostic build instead (``make -C crow-nest_b200/csrc trace``): the same entry points plus
    ``cn_m1_trace(buf, launches)``, after which the next `launches` one-row GEMV launches write eight %globaltimer stamps
    per CTA into buf [launches][512][8] (u64). Must be called before the first call into the library."""
    global SO_PATH
    if _lib is not None:
        raise CrownestError("the library is already loaded")
    SO_PATH = os.path.join(_HERE, "libcrownest_b200_trace.so")
    if not os.path.exists(SO_PATH):
        raise CrownestError(f"{SO_PATH} is missing: run `make -C {CSRC} trace`")
    register("cn_m1_trace", [C.c_void_p, C.c_int], None)
    register("cn_tp_trace", [C.c_void_p, C.c_int], None)  # the same for the tensor-parallel exchange kernel: buf [launches][8]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise CrownestError(f"{SO_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                                "(there is no CPU or PyTorch fallback for these kernels)")
        L = C.CDLL(SO_PATH)
        for name, args in _SIGS.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, _RESTYPES_INIT.get(name, C.c_int))
        _lib = L
    return _lib


def check(status):
    if status != 0:
        raise CrownestError(lib().cn_last_error_string().decode() or f"status {status}")


def device_status():
    code = C.c_int(0)
    check(lib().cn_device_status(C.byref(code)))
    return code.value
