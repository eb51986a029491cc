"""``fso.dense`` on a B200: one dense linear behind the reference's own surface.

    weight = fso.dense.prepare_weight(w, format="mxfp8")      # load time (also "bsfp8" with scale=...)
    y = fso.dense.linear(x, weight)                             # per call: 1x32 quantize + tcgen05 MXFP8 GEMM
    xq, sx = fso.dense.quantize_activation(x)
    y = fso.dense.linear(xq, weight, x_scale=sx)               # pre-quantized activation

This module mirrors python/fish_scales_ops/dense/__init__.py of the reference for the sm_100 family: the same
names, argument meaning, handle fields, custom-op schemas (``fish_scales_ops::dense_linear``,
``::dense_linear_quantized``, ``::dense_quantize_activation``), fake implementations and error classes
(ValueError for a malformed argument, NotImplementedError for what is not served, TypeError for a wrong handle),
every refusal raised before anything is launched. Underneath there is one route per op: the hand-written
sm_100a kernels of ``libfso_b200.so``; no other architecture and no fallback.
"""
import dataclasses
import math
import os

import torch

from .. import _ops
from .._lib import eager_or_op
from .._arch import SERVED_MAJOR, arch_label, arch_major, device_arch, sm_major

__all__ = ["FORMATS", "ACTIVATIONS", "DenseWeight", "prepare_weight", "linear", "linear_quantized",
           "quantize_activation", "activation_contract", "include_dir", "supported", "describe"]

FORMATS = ("bsfp8", "mxfp8")
ACTIVATIONS = ("gelu_erf",)
_UNSERVED_ACTIVATIONS = ("gelu", "gelu_tanh", "quick_gelu", "silu", "swish", "relu", "relu2", "swiglu", "geglu")
_UNSERVED = ("bf16", "bfloat16", "fp16", "float16", "fp32", "float32", "fp8", "int8", "w8a8",
             "int4", "w4a16", "w4a8", "mxfp4", "nvfp4")
_CONTRACT_VERSION = 1
FP8 = torch.float8_e4m3fn


def supported(format, arch=None) -> bool:
    """Whether ``format`` is served on ``arch`` (this device when None). This build serves both formats on the
    sm_100 family only and answers False for anything else, including unknown formats; an ``arch`` that names no
    compute capability raises ValueError (python/fish_scales_ops/dense/__init__.py:121-140)."""
    if not isinstance(format, str) or format.strip().lower() not in FORMATS:
        return False
    major = sm_major() if arch is None else arch_major(arch)
    return major == SERVED_MAJOR


def describe() -> str:
    """The route table of this build as text, for logs; never raises."""
    arch = device_arch()
    name = ""
    if arch > 0:
        try:
            name = f" ({torch.cuda.get_device_name(0)})"
        except Exception:  # noqa: BLE001
            name = ""
    lines = [
        f"fish_scales_ops_b200.dense: MXFP8 dense linear for sm_100a; this device is {arch_label(arch)}{name}.",
        "format 'mxfp8': a bf16 weight is quantized to MXFP8 1x32 at load time; a float8_e4m3fn weight keeps its "
        "bytes and its uint8 UE8M0 scales [N, K/32] are packed into the atom layout (or its int32 atom-layout scale "
        "is kept).",
        "format 'bsfp8': a float8_e4m3fn weight with fp32 128x128 block scales is requantized to MXFP8 1x32 by one "
        "fused kernel (value = bf16(fp8 * scale), then the 1x32 rule); a bf16 weight is quantized to MXFP8 directly.",
        "linear(): the 1x32 activation quantizer, then one tcgen05 block-scaled GEMM kernel family (activation rows "
        "on MMA-M for large M, weight rows on MMA-M for M <= 64 and for M <= 128 on weights of at most one 128-row "
        "panel per SM, split-K with an ordered reduce where the tile count leaves SMs idle). bias / residual / activation 'gelu_erf' are applied to the fp32 accumulator before the one "
        "rounding; linear_quantized runs linear (bias, activation) followed by the activation quantizer.",
    ]
    if arch // 10 != SERVED_MAJOR:
        lines.append(f"This device ({arch_label(arch)}) serves no format.")
    return "\n".join(lines)


@dataclasses.dataclass(frozen=True, eq=False, repr=False)
class DenseWeight:
    """One prepared dense weight (python/fish_scales_ops/dense/__init__.py:226-263). ``weight`` is float8_e4m3fn
    [N, K]; ``scale`` is a 1-D int32 tensor of N * K/128 words in the atom layout; ``kind`` is always "mxfp8"."""

    kind: str
    format: str
    arch: int
    in_features: int
    out_features: int
    weight: torch.Tensor
    scale: torch.Tensor

    def __repr__(self) -> str:
        return (f"DenseWeight(kind={self.kind!r}, format={self.format!r}, arch=sm_{self.arch}, "
                f"in_features={self.in_features}, out_features={self.out_features}, "
                f"weight={tuple(self.weight.shape)} {self.weight.dtype}, "
                f"scale={tuple(self.scale.shape)} {self.scale.dtype} stride={tuple(self.scale.stride())})")


def _aligned_storage(t: torch.Tensor, align: int = 16) -> torch.Tensor:
    """``t`` itself when its first byte sits on an ``align``-byte boundary, else a copy with the same strides (the
    allocator's blocks start on 512-byte boundaries). TMA reads the handle's tensors in place."""
    misaligned = t.numel() > 0 and t.data_ptr() % align != 0
    return torch.empty_strided(t.size(), t.stride(), dtype=t.dtype, device=t.device).copy_(t) if misaligned else t


def _format_error(format, where: str) -> Exception:
    if isinstance(format, str) and format.strip().lower() in _UNSERVED:
        return NotImplementedError(
            f"fso.dense.prepare_weight: format {format!r} is not served on any architecture ({where}); the formats "
            f"are 'bsfp8' and 'mxfp8'")
    return ValueError(f"fso.dense.prepare_weight: unknown format {format!r} on {where}; the formats are 'bsfp8' (a "
                      f"float8_e4m3fn weight with fp32 128x128 block scales, or a bf16 weight) and 'mxfp8' (a bf16 "
                      f"weight, or a float8_e4m3fn weight with its MXFP8 scales)")


def _complete(handle: DenseWeight) -> DenseWeight:
    """One empty plain launch after the kernels that wrote the handle's tensors
    (python/fish_scales_ops/dense/__init__.py:605-620): a decode linear issued right after starts loading its weights
    before its predecessor on the stream has finished, which is only safe when that predecessor did not write them."""
    _ops.stream_fence(handle.weight.device)
    return handle


def prepare_weight(w, *, format, scale=None) -> DenseWeight:
    """Prepare one dense weight ``[N, K]`` for this device, once, at load time
    (python/fish_scales_ops/dense/__init__.py:465-602).

    ``format="mxfp8"``: a bf16 weight (quantized here), or a float8_e4m3fn weight with ``scale`` either the
    checkpoint's uint8 UE8M0 bytes ``[N, K/32]`` or the 1-D int32 atom-layout words. ``format="bsfp8"``: a
    float8_e4m3fn weight with fp32 ``[N/128, K/128]`` block scales (requantized to MXFP8), or a bf16 weight.
    ``K % 128 == 0`` and ``N % 128 == 0``. Returns a :class:`DenseWeight` whose tensors start on 16-byte
    boundaries."""
    arch = device_arch()
    where = arch_label(arch)
    if not isinstance(format, str) or format.strip().lower() not in FORMATS:
        raise _format_error(format, where)
    fmt = format.strip().lower()
    if not supported(fmt):
        raise NotImplementedError(f"fso.dense.prepare_weight: this build serves sm_100-family devices only and this "
                                  f"device is {where}")
    ctx = f"fso.dense.prepare_weight (format {fmt!r}, {where})"
    if not isinstance(w, torch.Tensor):
        raise ValueError(f"{ctx}: w must be a tensor, got {type(w).__name__}")
    if w.dim() != 2:
        raise ValueError(f"{ctx}: w must be 2-D [N, K], got shape {tuple(w.shape)}")
    if not w.is_cuda:
        raise ValueError(f"{ctx}: w must be on the CUDA device that will serve it, got {w.device}")
    if torch.cuda.get_device_capability(w.device)[0] != SERVED_MAJOR:
        raise ValueError(f"{ctx}: the weight is on {w.device}, which is not an sm_100-family device")
    n, k = int(w.shape[0]), int(w.shape[1])
    if n < 1 or k < 1:
        raise ValueError(f"{ctx}: w is empty, shape {tuple(w.shape)}")
    if k % 128 != 0:
        raise ValueError(f"{ctx}: in_features K = {k} is not a multiple of 128")
    if n % 128 != 0:
        raise ValueError(f"{ctx}: out_features N = {n} is not a multiple of 128")
    if w.dtype not in (FP8, torch.bfloat16):
        raise ValueError(f"{ctx}: w must be float8_e4m3fn (with its scale) or bf16 (quantized here), got {w.dtype}")
    is_fp8 = w.dtype == FP8
    if is_fp8 and scale is None:
        raise ValueError(f"{ctx}: a float8_e4m3fn weight needs its scale")
    if not is_fp8 and scale is not None:
        raise ValueError(f"{ctx}: a bf16 weight is quantized here and takes no scale")
    wd = w.detach()
    kb = k // 128

    if not is_fp8:
        q, sq = _ops.quantize_1x32_fp8(wd)
        return _complete(DenseWeight("mxfp8", fmt, arch, k, n, q, sq))

    if fmt == "bsfp8":
        want = (n // 128, kb)
        if not isinstance(scale, torch.Tensor) or scale.dtype != torch.float32 or tuple(scale.shape) != want:
            got = f"{scale.dtype} {list(scale.shape)}" if isinstance(scale, torch.Tensor) else type(scale).__name__
            raise ValueError(f"{ctx}: scale must be fp32 {list(want)}, one scale per 128x128 block, got {got}")
        if scale.device != w.device:
            raise ValueError(f"{ctx}: scale is on {scale.device} and the weight on {w.device}")
        q, sq = _ops.requant_block_fp8(wd.contiguous(), scale.detach().contiguous())
        return _complete(DenseWeight("mxfp8", fmt, arch, k, n, q, sq))

    # fmt == "mxfp8" with a float8_e4m3fn checkpoint
    if not isinstance(scale, torch.Tensor):
        raise ValueError(f"{ctx}: scale must be the checkpoint's uint8 UE8M0 scale [N, K/32] = [{n}, {k // 32}] or "
                         f"the 1-D int32 atom-layout scale, got {type(scale).__name__}")
    if scale.device != w.device:
        raise ValueError(f"{ctx}: scale is on {scale.device} and the weight on {w.device}")
    if scale.dtype == torch.uint8:
        if tuple(scale.shape) != (n, k // 32):
            raise ValueError(f"{ctx}: the uint8 UE8M0 scale of an [N, K] = [{n}, {k}] weight is [N, K/32] = "
                             f"{[n, k // 32]}, got {list(scale.shape)}")
        sq = _ops.pack_ue8m0(scale.detach().unsqueeze(0))[0]
    elif scale.dtype == torch.int32:
        if scale.dim() != 1 or scale.numel() != n * kb:
            raise ValueError(f"{ctx}: the int32 MXFP8 scale of an [N, K] = [{n}, {k}] weight is a 1-D tensor of "
                             f"N * K/128 = {n * kb} words in the atom layout, got shape {list(scale.shape)}")
        if scale.stride() != (1,):
            raise ValueError(f"{ctx}: the MXFP8 scale has stride {tuple(scale.stride())}; it must be contiguous")
        sq = scale.detach()
    else:
        e8m0 = getattr(torch, "float8_e8m0fnu", None)
        hint = "; a float8_e8m0fnu tensor holds the same bytes, pass scale.view(torch.uint8)" \
            if e8m0 is not None and scale.dtype == e8m0 else ""
        raise ValueError(f"{ctx}: the MXFP8 scale must be uint8 [N, K/32] or int32 atom-layout words, got "
                         f"{scale.dtype}{hint}")
    return _complete(DenseWeight("mxfp8", fmt, arch, k, n, _aligned_storage(wd.contiguous()), _aligned_storage(sq, 32)))


# ------------------------------------------------------------------------------------------------ activation contract

def _align(v, a: int):
    return (v + a - 1) // a * a


def _act_scale_words(m, k: int):
    return _align(m, 128) * (k // 128)


def _empty_act_scale(m, k: int, device) -> torch.Tensor:
    return torch.empty((_act_scale_words(m, k),), dtype=torch.int32, device=device)


def include_dir() -> str:
    """The directory that holds ``fso_b200_activation_contract.h`` (the activation contract as compilable C / C++ /
    CUDA: scale-byte rule, E4M3 conversion, word packing and the index formula, for producers of pre-quantized
    activations) and ``fso_b200.h`` (the C ABI)."""
    return os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "include")


def activation_contract() -> dict:
    """The activation contract of this device as data (python/fish_scales_ops/dense/__init__.py:715-742): what
    :func:`quantize_activation` returns and ``linear(xq, weight, x_scale=sx)`` accepts."""
    arch = device_arch()
    if arch // 10 != SERVED_MAJOR:
        raise NotImplementedError(f"fso.dense.activation_contract: this device ({arch_label(arch)}) has no dense "
                                  f"route; this build serves the sm_100 family")
    return {
        "version": _CONTRACT_VERSION,
        "arch": arch_label(arch),
        "format": "mxfp8_1x32",
        "xq": {"dtype": "float8_e4m3fn", "shape": "[M, K]", "layout": "row-major, contiguous, 16-byte aligned"},
        "k_multiple": 128,
        "x_scale_dtype": "int32",
        "x_scale_shape": "[align(M, 128) * K/128] (1-D)",
        "x_scale_strides": "(1,)",
        "x_scale_index": "word(m, kp) at ((m / 128) * (K/128) + kp) * 128 + (m % 32) * 4 + (m % 128) / 32",
        "padded_rows": "zero words",
        "rule": "per 32-element block of a row: amax = max |x| in fp32, floored at 1e-10f; q = 448.f / amax; "
                "d = 1.f / q; b = exp_field(d) + (mantissa(d) != 0), capped at 254; code = "
                "cvt.rn.satfinite.e4m3(x * 2^(127 - b)); word(m, kp) = b0 | b1 << 8 | b2 << 16 | b3 << 24",
        "header": "fso_b200_activation_contract.h",
        "include_dir": include_dir(),
    }


# ------------------------------------------------------------------------------------------------ checks

def _check_activation(activation, ctx: str):
    if activation is None:
        return None
    if isinstance(activation, str) and activation in ACTIVATIONS:
        return activation
    if isinstance(activation, str) and activation.strip().lower() in _UNSERVED_ACTIVATIONS:
        raise NotImplementedError(f"{ctx}: activation {activation!r} is not served; the known activations are "
                                  f"{ACTIVATIONS}")
    raise ValueError(f"{ctx}: activation must be None or one of {ACTIVATIONS}, got {activation!r}")


def _check_epilogue(ctx: str, m: int, n: int, device, bias, residual, activation) -> bool:
    """Validates the epilogue arguments (metadata only); True when any of them is set."""
    act = _check_activation(activation, ctx)
    if bias is not None:
        if not isinstance(bias, torch.Tensor) or bias.dtype != torch.bfloat16 or bias.dim() != 1 \
                or int(bias.shape[0]) != n:
            got = f"{bias.dtype} {list(bias.shape)}" if isinstance(bias, torch.Tensor) else type(bias).__name__
            raise ValueError(f"{ctx}: bias must be bf16 [N] = [{n}], got {got}")
        if bias.device != device:
            raise ValueError(f"{ctx}: bias is on {bias.device} and the weight on {device}")
        if not bias.is_contiguous():
            raise ValueError(f"{ctx}: bias must be contiguous, got strides {tuple(bias.stride())}")
    if residual is not None:
        if not isinstance(residual, torch.Tensor) or residual.dtype != torch.bfloat16 \
                or tuple(residual.shape) != (m, n):
            got = f"{residual.dtype} {list(residual.shape)}" if isinstance(residual, torch.Tensor) \
                else type(residual).__name__
            raise ValueError(f"{ctx}: residual must be bf16 with the output's shape [M, N] = [{m}, {n}], got {got}")
        if residual.device != device:
            raise ValueError(f"{ctx}: residual is on {residual.device} and the weight on {device}")
        if not residual.is_contiguous():
            raise ValueError(f"{ctx}: residual must be contiguous, got strides {tuple(residual.stride())}")
    return bias is not None or residual is not None or act is not None


def _check_operands(op: str, x, weight, x_scale) -> None:
    """Shapes and dtypes of the op's three main tensors (metadata only)."""
    shapes_fit = x.dim() == 2 and weight.dim() == 2 and x.shape[1] == weight.shape[1]
    if not shapes_fit:
        raise ValueError(f"{op}: expected x [M, K] and weight [N, K] sharing K; x is {tuple(x.shape)}, weight is "
                         f"{tuple(weight.shape)}")
    if weight.dtype != FP8:
        raise ValueError(f"{op}: the weight is {weight.dtype}; a prepared weight is float8_e4m3fn")
    quantized_x = x.dtype == FP8
    if x_scale is None and quantized_x:
        raise ValueError(f"{op}: a float8_e4m3fn x is a pre-quantized activation and needs the x_scale that "
                         f"fso.dense.quantize_activation returned with it")
    if x_scale is None and x.dtype != torch.bfloat16:
        raise ValueError(f"{op}: x is {x.dtype}; the op takes bf16 (or float8_e4m3fn together with x_scale)")
    if x_scale is not None and x.dtype == torch.bfloat16:
        raise ValueError(f"{op}: x_scale goes with the float8_e4m3fn activation of fso.dense.quantize_activation, "
                         f"but x is bf16")


def _check_weight_scale(op: str, kind: str, scale, n: int, k: int) -> None:
    if kind == "bsfp8":
        raise NotImplementedError(f"{op}: kind 'bsfp8' is the sm_90 block-FP8 GEMM; prepare the weight on this device "
                                  f"with fso.dense.prepare_weight, which serves block-FP8 checkpoints as MXFP8")
    if kind != "mxfp8":
        raise ValueError(f"{op}: unknown kind {kind!r}; fso.dense.prepare_weight produces 'mxfp8' handles here")
    if sm_major() != SERVED_MAJOR:
        raise NotImplementedError(f"{op}: kind 'mxfp8' needs an sm_100-family device in this build")
    if scale.dtype != torch.int32 or scale.dim() != 1 or scale.numel() != n * (k // 128) or scale.stride() != (1,):
        raise ValueError(f"{op}: scale must be a contiguous 1-D int32 tensor of {n * (k // 128)} words (the atom "
                         f"layout), got {scale.dtype} {list(scale.shape)} strides {tuple(scale.stride())}")


def _check_weight_aligned(op: str, weight, scale) -> None:
    for name, t in (("weight", weight), ("scale", scale)):
        if t.numel() > 0 and t.data_ptr() % 16 != 0:
            raise ValueError(f"{op}: the {name}'s data pointer is {t.data_ptr() % 16} bytes past a 16-byte boundary; "
                             f"the GEMM reads it in place with TMA. fso.dense.prepare_weight returns aligned tensors")
    if not weight.is_contiguous():
        raise ValueError(f"{op}: the weight must be contiguous, got strides {tuple(weight.stride())}")


def _check_xq(op: str, x, device) -> None:
    """The pre-quantized activation: e4m3, on the weight's device, dense rows, first byte on a 16-byte boundary."""
    problems = []
    if x.dtype != FP8:
        problems.append(f"its dtype is {x.dtype}, not float8_e4m3fn")
    if x.device != device:
        problems.append(f"it lives on {x.device} while the weight lives on {device}")
    if not x.is_contiguous():
        problems.append(f"it is not contiguous (strides {tuple(x.stride())})")
    elif x.numel() > 0 and x.data_ptr() % 16 != 0:
        problems.append("its data pointer is not a multiple of 16 bytes")
    if problems:
        raise ValueError(f"{op}: x passed with x_scale must be the [M, K] activation fso.dense.quantize_activation "
                         f"returned; " + "; ".join(problems))


def _check_x_scale(op: str, x_scale, m: int, k: int, device) -> None:
    """The scale tensor of a pre-quantized [m, k] activation, against activation contract v1."""
    words = _act_scale_words(m, k)
    if not isinstance(x_scale, torch.Tensor):
        found = f"a {type(x_scale).__name__}"
    elif x_scale.dtype != torch.int32:
        found = f"dtype {x_scale.dtype}"
    elif x_scale.device != device:
        found = f"a tensor on {x_scale.device} (the weight is on {device})"
    elif x_scale.dim() != 1 or int(x_scale.shape[0]) != words:
        found = f"shape {list(x_scale.shape)}"
    elif x_scale.numel() > 0 and not x_scale.is_contiguous():
        found = f"strides {tuple(x_scale.stride())}"
    elif x_scale.numel() > 0 and x_scale.data_ptr() % 16 != 0:
        found = "a data pointer that is not a multiple of 16 bytes"
    else:
        return
    raise ValueError(f"{op}: x_scale must be what activation contract v1 prescribes for an [M, K] = [{m}, {k}] "
                     f"activation on this device, a contiguous 16-byte aligned int32 [{words}] tensor in the atom "
                     f"layout; got {found}")


def _x_bf16_storage(x):
    """A contiguous bf16 x whose data pointer is not 16-byte aligned is copied once (the quantizer reads 16-byte
    vectors); python/fish_scales_ops/dense/__init__.py:800-811."""
    if x.numel() > 0 and x.is_contiguous() and x.data_ptr() % 16 != 0:
        return x.clone()
    return x


def _epilogue_storage(op: str, bias, residual):
    """The epilogue kernels read bias and residual with 16-byte loads: a bias off a 16-byte boundary is cloned (it is
    N elements); a residual off one is refused, as in the reference (a copy of [M, N] is the caller's call)."""
    if bias is not None and bias.numel() > 0 and bias.data_ptr() % 16 != 0:
        bias = bias.clone()
    if residual is not None and residual.numel() > 0 and residual.data_ptr() % 16 != 0:
        raise NotImplementedError(f"{op}: the residual's data pointer is {residual.data_ptr() % 16} bytes past a "
                                  f"16-byte boundary; the epilogue reads its rows with 16-byte loads")
    return bias, residual


# ------------------------------------------------------------------------------------------------ custom ops

def _dense_linear_body(x, weight, scale, kind, bias=None, x_scale=None, residual=None, activation=None):
    """Body of ``torch.ops.fish_scales_ops.dense_linear``: metadata checks only (no sync, no dependence on tensor
    values), then the quantizer and the GEMM (python/fish_scales_ops/dense/__init__.py:962-993)."""
    op = f"fish_scales_ops::dense_linear ({arch_label(device_arch())}, kind {kind!r})"
    _check_operands(op, x, weight, x_scale)
    m, n, k = int(x.shape[0]), int(weight.shape[0]), int(x.shape[1])
    _check_weight_scale(op, kind, scale, n, k)
    has_epi = _check_epilogue(op, m, n, weight.device, bias, residual, activation)
    if m > 0:
        _check_weight_aligned(op, weight, scale)
    if x_scale is not None:
        _check_xq(op, x, weight.device)
        _check_x_scale(op, x_scale, m, k, weight.device)
    else:
        x = _x_bf16_storage(x)
    if m == 0:
        return x.new_empty((0, n), dtype=torch.bfloat16)
    bias, residual = _epilogue_storage(op, bias, residual)
    if x_scale is None:
        x, x_scale = _ops.quantize_1x32_fp8(x, activation=True)
    return _ops.linear_mxfp8(x, weight, x_scale, scale, bias, residual, 1 if activation == "gelu_erf" else 0)


_dense_linear_op = torch.library.custom_op(
    "fish_scales_ops::dense_linear",
    mutates_args=(),
    schema="(Tensor x, Tensor weight, Tensor scale, str kind, Tensor? bias=None, Tensor? x_scale=None, "
           "Tensor? residual=None, str? activation=None) -> Tensor",
)(_dense_linear_body)


@_dense_linear_op.register_fake
def _dense_linear_fake(x, weight, scale, kind, bias=None, x_scale=None, residual=None, activation=None):
    if x.dim() != 2 or weight.dim() != 2:
        raise ValueError(f"fish_scales_ops::dense_linear: x must be [M, K] and weight [N, K], got {x.dim()}-D and "
                         f"{weight.dim()}-D tensors")
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


def _dense_linear_quantized_body(x, weight, scale, kind, bias=None, x_scale=None, activation=None):
    """Body of ``torch.ops.fish_scales_ops.dense_linear_quantized``: the result of ``dense_linear`` in the
    activation contract (python/fish_scales_ops/dense/__init__.py:1212-1241). For the shapes the GEMM serves in its
    normal orientation without split-K the quantization happens in the GEMM's epilogue (one launch, no bf16 round
    trip); for the others it is the GEMM followed by the activation quantizer. Both give the same bytes."""
    op = f"fish_scales_ops::dense_linear_quantized ({arch_label(device_arch())}, kind {kind!r})"
    _check_operands(op, x, weight, x_scale)
    m, n, k = int(x.shape[0]), int(weight.shape[0]), int(x.shape[1])
    _check_weight_scale(op, kind, scale, n, k)
    has_epi = _check_epilogue(op, m, n, weight.device, bias, None, activation)
    if m > 0:
        _check_weight_aligned(op, weight, scale)
    if x_scale is not None:
        _check_xq(op, x, weight.device)
        _check_x_scale(op, x_scale, m, k, weight.device)
    else:
        x = _x_bf16_storage(x)
    if m == 0:
        return (x.new_empty((0, n), dtype=FP8), _empty_act_scale(0, n, x.device))
    bias, _ = _epilogue_storage(op, bias, None)
    if x_scale is None:
        x, x_scale = _ops.quantize_1x32_fp8(x, activation=True)
    return _ops.linear_mxfp8_quantized(x, weight, x_scale, scale, bias, 1 if activation == "gelu_erf" else 0)


_dense_linear_quantized_op = torch.library.custom_op(
    "fish_scales_ops::dense_linear_quantized",
    mutates_args=(),
    schema="(Tensor x, Tensor weight, Tensor scale, str kind, Tensor? bias=None, Tensor? x_scale=None, "
           "str? activation=None) -> (Tensor, Tensor)",
)(_dense_linear_quantized_body)


@_dense_linear_quantized_op.register_fake
def _dense_linear_quantized_fake(x, weight, scale, kind, bias=None, x_scale=None, activation=None):
    if x.dim() != 2 or weight.dim() != 2:
        raise ValueError(f"fish_scales_ops::dense_linear_quantized: x must be [M, K] and weight [N, K], got "
                         f"{x.dim()}-D and {weight.dim()}-D tensors")
    m, n = x.shape[0], weight.shape[0]
    return (x.new_empty((m, n), dtype=FP8), _empty_act_scale(m, int(n), x.device))


def _quantize_activation_checks(x, op: str) -> None:
    arch = device_arch()
    if arch // 10 != SERVED_MAJOR:
        raise NotImplementedError(f"{op}: no dense route exists for this device ({arch_label(arch)}) in this build")
    is_bf16 = isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and x.dim() >= 1
    if not is_bf16:
        what = f"{x.dtype} {tuple(x.shape)}" if isinstance(x, torch.Tensor) else type(x).__name__
        raise ValueError(f"{op}: takes a bf16 [..., K] tensor, not {what}")
    if not x.is_cuda:
        raise ValueError(f"{op}: x is on {x.device}; it must be on the CUDA device")
    k = int(x.shape[-1])
    if k % 128 != 0:
        raise ValueError(f"{op}: activation contract v1 needs K to be a multiple of 128 and K is {k}")


def _dense_quantize_activation_body(x):
    op = f"fish_scales_ops::dense_quantize_activation ({arch_label(device_arch())})"
    _quantize_activation_checks(x, op)
    k = int(x.shape[-1])
    x2 = _x_bf16_storage(x.reshape(-1, k))
    m = int(x2.shape[0])
    if m == 0:
        return (x.new_empty((0, k), dtype=FP8), _empty_act_scale(0, k, x.device))
    return _ops.quantize_1x32_fp8(x2, activation=True)


_dense_quantize_activation_op = torch.library.custom_op(
    "fish_scales_ops::dense_quantize_activation",
    mutates_args=(),
    schema="(Tensor x) -> (Tensor, Tensor)",
)(_dense_quantize_activation_body)


@_dense_quantize_activation_op.register_fake
def _dense_quantize_activation_fake(x):
    k = x.shape[-1]
    m = math.prod(x.shape[:-1]) if x.dim() > 1 else 1
    return (x.new_empty((m, k), dtype=FP8), _empty_act_scale(m, int(k), x.device))


# ------------------------------------------------------------------------------------------------ public functions

def _trim_none(*args) -> tuple:
    """The arguments without their trailing Nones (the ops' optional arguments default to None, so a call that
    sets none of them records the short form in a traced graph)."""
    keep = len(args)
    while keep > 0 and args[keep - 1] is None:
        keep -= 1
    return tuple(args[:keep])


def _check_handle(weight, where: str, ctx: str) -> None:
    if not isinstance(weight, DenseWeight):
        raise TypeError(f"{ctx} ({where}): the weight argument is a {type(weight).__name__}; pass the DenseWeight that "
                        f"fso.dense.prepare_weight returned")
    if weight.arch // 10 != device_arch() // 10:
        raise ValueError(f"{ctx}: this weight was prepared for sm_{weight.arch}, the current device is {where}")


def _flatten_x(x, weight, x_scale, where: str, ctx: str):
    """(x as [M, K], the leading dimensions of the result). A bf16 x may have any leading dimensions; a
    pre-quantized one is already the 2-D contiguous tensor of the activation contract."""
    tag = f"{ctx} ({where}, kind {weight.kind!r})"
    k = weight.in_features
    is_tensor = isinstance(x, torch.Tensor)
    shown = (f"{x.dtype} {tuple(x.shape)} strides {tuple(x.stride())}" if is_tensor else type(x).__name__)
    if x_scale is None:
        if is_tensor and x.dtype == FP8:
            raise ValueError(f"{tag}: a float8_e4m3fn x needs its x_scale")
        if not (is_tensor and x.dtype == torch.bfloat16 and x.dim() >= 1 and x.shape[-1] == k):
            raise ValueError(f"{tag}: x must be bf16 [..., {k}] (K = in_features); got {shown}")
    elif not (is_tensor and x.dtype == FP8 and x.dim() == 2 and x.shape[1] == k and x.is_contiguous()):
        raise ValueError(f"{tag}: together with x_scale, x must be the contiguous float8_e4m3fn [M, {k}] tensor of "
                         f"fso.dense.quantize_activation; got {shown}")
    if x.device != weight.weight.device:
        raise ValueError(f"{tag}: x lives on {x.device}, the weight on {weight.weight.device}")
    lead = x.shape[:-1]
    return (x if x_scale is not None else x.reshape(-1, k)), lead


def linear(x, weight, *, bias=None, x_scale=None, residual=None, activation=None) -> torch.Tensor:
    """``y = x @ W^T`` for a prepared weight: bf16 ``[..., N]`` (python/fish_scales_ops/dense/__init__.py:1153-1209).

    ``x`` is bf16 ``[..., K]`` (quantized inside the op) or, with ``x_scale``, the float8_e4m3fn ``[M, K]`` of
    :func:`quantize_activation`. ``bias`` (bf16 ``[N]``), ``activation`` (``"gelu_erf"``) and ``residual`` (bf16, the
    result's shape) are applied in the GEMM's epilogue to the fp32 accumulator, in that order, before the one
    rounding to bf16. Nothing in the call synchronizes the device, and it can be captured into a CUDA graph after
    one eager call of the same shape."""
    where = arch_label(device_arch())
    _check_handle(weight, where, "fso.dense.linear")
    x2, lead = _flatten_x(x, weight, x_scale, where, "fso.dense.linear")
    n = weight.out_features
    out_shape = tuple(lead) + (n,)
    res2 = None
    if residual is not None:
        ok = isinstance(residual, torch.Tensor) and tuple(residual.shape) == out_shape
        if not ok:
            got = list(residual.shape) if isinstance(residual, torch.Tensor) else type(residual).__name__
            raise ValueError(f"fso.dense.linear ({where}, kind {weight.kind!r}): the residual is added to the result "
                             f"and must have its shape {list(out_shape)}; got {got}")
        if not residual.is_contiguous():
            raise ValueError(f"fso.dense.linear ({where}, kind {weight.kind!r}): the residual must be contiguous")
        res2 = residual.view(-1, n)
    extra = _trim_none(bias, x_scale, res2, activation)
    y = eager_or_op(_dense_linear_body, torch.ops.fish_scales_ops.dense_linear, x2, weight.weight, weight.scale,
                    weight.kind, *extra)
    return y.reshape(out_shape)


def linear_quantized(x, weight, *, bias=None, x_scale=None, activation=None):
    """``(xq_next, scale_next)``: :func:`linear`'s result in the activation contract, bit for bit
    ``quantize_activation(linear(...))``."""
    where = arch_label(device_arch())
    _check_handle(weight, where, "fso.dense.linear_quantized")
    x2, _ = _flatten_x(x, weight, x_scale, where, "fso.dense.linear_quantized")
    return eager_or_op(_dense_linear_quantized_body, torch.ops.fish_scales_ops.dense_linear_quantized,
        
        x2, weight.weight, weight.scale, weight.kind, *_trim_none(bias, x_scale, activation))


def quantize_activation(x):
    """``(xq, x_scale)`` of a bf16 ``[..., K]`` activation: float8_e4m3fn ``[M, K]`` and the int32 atom-layout
    scale words, the exact bytes ``linear(x, weight)`` computes inside the op."""
    return eager_or_op(_dense_quantize_activation_body, torch.ops.fish_scales_ops.dense_quantize_activation, x)
