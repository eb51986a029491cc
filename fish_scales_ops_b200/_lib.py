"""ctypes binding of the C ABI in ``include/fso_b200.h``.

There is no other implementation behind these calls: when ``libfso_b200.so`` is missing or a call fails, the
caller gets an exception, never a slower path.
"""
import ctypes
import os

import torch

from . import _build

_c_i64 = ctypes.c_int64
_c_p = ctypes.c_void_p

# Every entry point of include/fso_b200.h with its argument types (the return type is int unless stated).
SIGNATURES = {
    "fso_b200_version": [],
    "fso_b200_last_error": [],
    "fso_b200_device_status": [ctypes.POINTER(ctypes.c_int)],
    "fso_b200_selftest_wait_expires": [_c_i64, _c_p],
    "fso_quantize_1x32": [_c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_requant_bs128_to_mx": [_c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_pack_ue8m0": [_c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_gemm_mxfp8_ws_bytes": [_c_i64, _c_i64, _c_i64, ctypes.POINTER(_c_i64)],
    "fso_gemm_mxfp8_describe": [_c_i64, _c_i64, _c_i64, _c_i64, ctypes.POINTER(ctypes.c_int32)],
    "fso_gemm_mxfp8": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p, _c_i64, _c_p],
    "fso_moe_plan_make": [_c_i64, _c_i64, _c_i64, _c_p],
    "fso_moe_route": [_c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_p],
    "fso_moe_route_noalloc": [_c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p, _c_p, _c_p],
    "fso_moe_gather_quant": [_c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p],
    "fso_moe_fc1_swiglu": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p,
                           _c_p],
    "fso_moe_fc2": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p],
    "fso_moe_grouped_gemm_decode": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64,
                                    _c_p, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_moe_silu_mul_quantize_rows": [_c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p],
    "fso_moe_combine": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_gemm_mxfp8_epilogue": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_i64, _c_p, _c_i64,
                                _c_p],
    "fso_quantize_activation_1x32": [_c_p, _c_p, _c_p, _c_i64, _c_i64, _c_p],
    "fso_gemm_mxfp8_fuses_quantized_output": [_c_i64, _c_i64, _c_i64, ctypes.POINTER(ctypes.c_int)],
    "fso_gemm_mxfp8_quantized": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p, _c_i64, _c_p],
    "fso_gemm_mxfp8_swiglu": [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_stream_fence": [_c_p],
    "fso_silu_mul_quantize_1x32": [_c_p, _c_p, _c_p, _c_i64, _c_i64, _c_p],
    "fso_moe_topk_from_logits": [_c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p, _c_p, _c_p,
                                 _c_p],
    "fso_ep_plan_count": [_c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p],
    "fso_ep_plan_place": [_c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p],
    "fso_ep_dispatch_push": [_c_p] * 12 + [_c_i64, _c_i64, _c_i64, _c_i64, _c_p],
    "fso_moe_gather_rows": [_c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p],
    "fso_moe_combine_scatter": [_c_p, _c_p, _c_p, _c_i64, _c_i64, _c_i64, _c_p, _c_p, _c_p, _c_i64, _c_p],
}


class MoePlan(ctypes.Structure):
    _fields_ = [("pairs", _c_i64), ("num_blocks", _c_i64), ("rows", _c_i64), ("route_scratch_bytes", _c_i64)]


_LIB = None


def lib_path() -> str:
    return _build.LIB_PATH


def lib():
    """The loaded library; raises when it has not been built (``__graft_entry__.build()`` or
    ``fish_scales_ops_b200.build()`` builds it)."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"fish_scales_ops_b200: the CUDA library {path} is missing; build it with "
                f"fish_scales_ops_b200.build() (nvcc, sm_100a). There is no fallback implementation.")
        handle = ctypes.CDLL(path)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_char_p if name == "fso_b200_last_error" else ctypes.c_int
        _LIB = handle
    return _LIB


def last_error() -> str:
    msg = lib().fso_b200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, op: str) -> None:
    """Turn a C-ABI return code into the exception the reference raises for the same condition."""
    if rc == 0:
        return
    msg = f"{op}: {last_error()}"
    if rc == -1:
        raise ValueError(msg)
    if rc == -2:
        raise NotImplementedError(msg)
    raise RuntimeError(f"{msg} (code {rc})")


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def on_device(device):
    """Context in which ``device`` is the current CUDA device: nothing at all when it already is (the usual case, and
    this sits on the path of every call), ``torch.cuda.device`` otherwise."""
    idx = device.index if isinstance(device, torch.device) else device
    if idx is None or idx == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(idx)


def stream_ptr():
    """The current stream of the current device as a raw handle (no Stream object is built: this sits on the path of
    every call)."""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def eager_or_op(body, op, *args):
    """An eager call runs the op's body directly (the dispatcher round trip of a Python custom op costs more host time
    than a decode-sized kernel runs); while torch.compile traces, the registered custom op is called instead, so the
    compiled graph records it as one node."""
    if torch.compiler.is_compiling():
        return op(*args)
    return body(*args)


def device_status() -> int:
    """The device-side status word of the current device (0 = no kernel wait ever ran out); synchronizes."""
    v = ctypes.c_int(0)
    check(lib().fso_b200_device_status(ctypes.byref(v)), "fso_b200_device_status")
    return v.value
