"""The router in front of the MoE layer, under the names the reference exports them
(python/fish_scales_ops/gemm/mxfp8.py:1355-1436, reached there as ``fso.compat.moe_topk_from_logits`` and
``fso.compat.moe_router_topk``): softmax over the experts, top-k selection, renormalization, the padded-row
sentinel of a CUDA-graph bucket, the expert-parallel id map and the shared expert's gate in one kernel."""
from typing import Optional, Tuple

import torch

from . import _ops
from ._lib import eager_or_op
from ._arch import SERVED_MAJOR, arch_label, device_arch

__all__ = ["moe_topk_from_logits", "moe_router_topk", "silu_chunk_mul_quantize_1x32_fp8", "prepare_gate_up",
           "shared_expert", "moe_layer_shared",
           "linear_swiglu"]

_MAX_EXPERTS = 1024
_MAX_TOPK = 8


def _topk_from_logits_body(logits, topk, renormalize=True, with_shared_gate=False, num_token_non_padded=None,
                         expert_map=None):
    """Body of ``torch.ops.fish_scales_ops.moe_topk_from_logits`` (csrc/gemm/ops/moe_glue.cu:3074-3152): the same
    refusals, before anything is launched."""
    op = f"fish_scales_ops::moe_topk_from_logits ({arch_label(device_arch())})"
    if not logits.is_cuda or logits.dim() != 2:
        raise ValueError(f"{op}: logits must be a CUDA [M, E] tensor")
    if logits.stride(1) != 1:
        raise ValueError(f"{op}: logits must have a contiguous expert dimension")
    if logits.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError(f"{op}: logits must be bf16, fp16 or fp32, got {logits.dtype}")
    if device_arch() // 10 != SERVED_MAJOR:
        raise NotImplementedError(f"{op}: this build serves sm_100-family devices")
    e = int(logits.shape[1]) - (1 if with_shared_gate else 0)
    if not 1 <= e <= _MAX_EXPERTS:
        raise ValueError(f"{op}: num_experts must be in [1, {_MAX_EXPERTS}], got {e}")
    if not (1 <= topk <= _MAX_TOPK and topk <= e):
        raise ValueError(f"{op}: topk must be in [1, min({_MAX_TOPK}, num_experts)], got {topk}")
    n_valid = None
    if num_token_non_padded is not None and num_token_non_padded.numel() > 0:
        n_valid = num_token_non_padded
        if not n_valid.is_cuda or n_valid.dtype != torch.int32 or n_valid.numel() != 1:
            raise ValueError(f"{op}: num_token_non_padded must be a CUDA int32 tensor with one element")
    emap = None
    if expert_map is not None and expert_map.numel() > 0:
        emap = expert_map
        if not emap.is_cuda or emap.dtype != torch.int32 or not emap.is_contiguous():
            raise ValueError(f"{op}: expert_map must be a contiguous CUDA int32 tensor")
        if emap.numel() < e + 1:
            raise ValueError(f"{op}: expert_map must have num_experts + 1 entries (the last one maps the padded-row "
                             f"sentinel)")
    return _ops.moe_topk_from_logits(logits, int(topk), bool(renormalize), bool(with_shared_gate), n_valid, emap)


_topk_from_logits_op = torch.library.custom_op(
    "fish_scales_ops::moe_topk_from_logits",
    mutates_args=(),
    schema="(Tensor logits, int topk, bool renormalize=True, bool with_shared_gate=False, "
           "Tensor? num_token_non_padded=None, Tensor? expert_map=None) -> (Tensor, Tensor, Tensor)",
)(_topk_from_logits_body)


@_topk_from_logits_op.register_fake
def _topk_from_logits_fake(logits, topk, renormalize=True, with_shared_gate=False, num_token_non_padded=None,
                           expert_map=None):
    m = logits.shape[0]
    return (logits.new_empty((m, topk), dtype=torch.int32), logits.new_empty((m, topk), dtype=torch.float32),
            logits.new_empty((m if with_shared_gate else 0,), dtype=torch.float32))


def moe_topk_from_logits(logits: torch.Tensor, topk: int, *, renormalize: bool = True, with_shared_gate: bool = False,
                         num_token_non_padded: Optional[torch.Tensor] = None,
                         expert_map: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Router logits ``[M, num_experts]`` (``num_experts + 1`` columns with ``with_shared_gate``; bf16, fp16 or fp32)
    -> ``(topk_ids int32 [M, topk], topk_w fp32 [M, topk], shared_gate fp32 [M] or empty)``, one launch. Ids come
    out in descending weight order, ties broken toward the lower expert id; ``renormalize`` divides the selected
    probabilities by their own sum, otherwise the weights are the plain softmax over all experts; rows at or past
    ``num_token_non_padded`` get the sentinel id ``num_experts`` (through ``expert_map`` when given) and weight
    zero; ``expert_map`` int32 ``[num_experts + 1]`` maps global ids to an expert-parallel rank's local ids."""
    return eager_or_op(_topk_from_logits_body, torch.ops.fish_scales_ops.moe_topk_from_logits, logits, int(topk),
                       bool(renormalize), bool(with_shared_gate), num_token_non_padded, expert_map)


def moe_router_topk(hidden: torch.Tensor, router_weight: torch.Tensor, topk: int, *, renormalize: bool = True,
                    with_shared_gate: bool = False, num_token_non_padded: Optional[torch.Tensor] = None,
                    expert_map: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The whole router in two launches: the logit GEMM (a plain library GEMM, as in the reference: the gate matrix
    is a megabyte) and :func:`moe_topk_from_logits`. ``router_weight`` bf16 ``[num_experts (+1), HIDDEN]``."""
    logits = torch.nn.functional.linear(hidden, router_weight)
    return moe_topk_from_logits(logits, topk, renormalize=renormalize, with_shared_gate=with_shared_gate,
                                num_token_non_padded=num_token_non_padded, expert_map=expert_map)


def _silu_chunk_mul_quantize_body(gu, use_ue8m0=True):
    op = f"fish_scales_ops::silu_chunk_mul_quantize_1x32 ({arch_label(device_arch())})"
    if not gu.is_cuda or gu.dtype != torch.bfloat16 or gu.dim() != 2:
        raise ValueError(f"{op}: gu must be a CUDA bf16 [M, 2*INTER] tensor, got {gu.dtype} {tuple(gu.shape)}")
    if int(gu.shape[1]) % 256 != 0:
        raise ValueError(f"{op}: INTER = {int(gu.shape[1]) / 2:g} must be a multiple of 128")
    if not use_ue8m0:
        raise NotImplementedError(f"{op}: only the UE8M0 (MXFP8) scale form is served")
    if device_arch() // 10 != SERVED_MAJOR:
        raise NotImplementedError(f"{op}: this build serves sm_100-family devices")
    if not gu.is_contiguous() or gu.data_ptr() % 32 != 0:
        gu = gu.contiguous() if not gu.is_contiguous() else gu.clone()
    return _ops.silu_mul_quantize_1x32_fp8(gu)


_silu_chunk_mul_quantize_op = torch.library.custom_op(
    "fish_scales_ops::silu_chunk_mul_quantize_1x32",
    mutates_args=(),
    schema="(Tensor gu, bool use_ue8m0=True) -> (Tensor, Tensor)",
)(_silu_chunk_mul_quantize_body)


@_silu_chunk_mul_quantize_op.register_fake
def _silu_chunk_mul_quantize_fake(gu, use_ue8m0=True):
    m, inter = gu.shape[0], gu.shape[1] // 2
    return (gu.new_empty((m, inter), dtype=torch.float8_e4m3fn),
            gu.new_empty(((m + 127) // 128 * 128 * (inter // 128),), dtype=torch.int32))


def silu_chunk_mul_quantize_1x32_fp8(gu: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The step between the gate_up and the down projection of a SwiGLU MLP
    (python/fish_scales_ops/gemm/mxfp8.py:216-236): ``gu`` bf16 ``[..., 2*INTER]`` with the gate in the first INTER
    columns and up in the second; returns ``silu(gate) * up`` as ``(float8_e4m3fn [M, INTER], int32 scale words)`` in
    the activation contract, ready for ``fso.dense.linear(xq, weight, x_scale=sx)``, without the product ever
    reaching memory."""
    two_i = int(gu.shape[-1])
    return eager_or_op(_silu_chunk_mul_quantize_body, torch.ops.fish_scales_ops.silu_chunk_mul_quantize_1x32,
                       gu.reshape(-1, two_i), True)


# ------------------------------------------------------------------------------------------ dense SwiGLU, fused

def prepare_gate_up(w: torch.Tensor, *, format: str = "mxfp8", scale: Optional[torch.Tensor] = None):
    """Prepare the stacked gate_up weight ``[2*INTER, K]`` (gate rows first, as checkpoints store it) of a dense SwiGLU
    MLP for :func:`linear_swiglu`: MXFP8 with the rows interleaved (gate_j, up_j adjacent), the order the fused
    epilogue reads, which is the order ``fso.moe.prepare_experts`` gives the experts' FC1 weights
    (python/fish_scales_ops/gemm/mxfp8.py:621-633). ``format="mxfp8"`` takes a bf16 weight, ``format="bsfp8"`` a
    float8_e4m3fn weight with its fp32 ``[2*INTER/128, K/128]`` block scales. Returns a ``DenseWeight``; hand it to
    :func:`linear_swiglu` only (``fso.dense.linear`` on it would give the columns in interleaved order)."""
    from . import dense

    arch = device_arch()
    ctx = f"fso.compat.prepare_gate_up (format {format!r}, {arch_label(arch)})"
    if arch // 10 != SERVED_MAJOR:
        raise NotImplementedError(f"{ctx}: this build serves sm_100-family devices")
    if not isinstance(w, torch.Tensor) or w.dim() != 2 or not w.is_cuda:
        raise ValueError(f"{ctx}: w must be a CUDA [2*INTER, K] tensor")
    two_i, k = int(w.shape[0]), int(w.shape[1])
    if two_i % 256 != 0 or k % 128 != 0:
        raise ValueError(f"{ctx}: 2*INTER = {two_i} must be a multiple of 256 and K = {k} a multiple of 128")
    if format == "mxfp8":
        if w.dtype != torch.bfloat16 or scale is not None:
            raise ValueError(f"{ctx}: takes a bf16 weight and no scale")
        q, sq = _ops.quantize_1x32_fp8(w.detach(), interleave_i=two_i // 2)
    elif format == "bsfp8":
        if w.dtype != torch.float8_e4m3fn or not isinstance(scale, torch.Tensor) or scale.dtype != torch.float32 \
                or tuple(scale.shape) != (two_i // 128, k // 128) or (two_i // 2) % 128 != 0:
            raise ValueError(f"{ctx}: takes a float8_e4m3fn weight with fp32 [{two_i // 128}, {k // 128}] block scales "
                             f"and INTER a multiple of 128")
        q, sq = _ops.requant_block_fp8(w.detach().contiguous(), scale.detach().contiguous(), interleave_i=two_i // 2)
    else:
        raise ValueError(f"{ctx}: the formats are 'mxfp8' and 'bsfp8'")
    _ops.stream_fence(w.device)
    return dense.DenseWeight("mxfp8", format, arch, k, two_i, q, sq)


def _dense_linear_swiglu_body(x, weight, scale, x_scale=None):
    op = f"fish_scales_ops::dense_linear_swiglu ({arch_label(device_arch())})"
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise ValueError(f"{op}: x must be [M, K] and weight [2*INTER, K] with the same K, got {tuple(x.shape)} and "
                         f"{tuple(weight.shape)}")
    two_i, k = int(weight.shape[0]), int(weight.shape[1])
    if weight.dtype != torch.float8_e4m3fn or two_i % 256 != 0 or k % 128 != 0 or not weight.is_contiguous():
        raise ValueError(f"{op}: weight must be a contiguous float8_e4m3fn [2*INTER, K] with 2*INTER % 256 == 0")
    if scale.dtype != torch.int32 or scale.dim() != 1 or scale.numel() != two_i * (k // 128):
        raise ValueError(f"{op}: scale must be the 1-D int32 atom-layout scale of the weight")
    m = int(x.shape[0])
    if x_scale is None:
        if x.dtype != torch.bfloat16:
            raise ValueError(f"{op}: x must be bf16 (or float8_e4m3fn with x_scale), got {x.dtype}")
        if m > 0 and (not x.is_contiguous() or x.data_ptr() % 16 != 0):
            x = x.contiguous() if not x.is_contiguous() else x.clone()
        x, x_scale = _ops.quantize_1x32_fp8(x, activation=True)
    else:
        if x.dtype != torch.float8_e4m3fn or not x.is_contiguous() or (m > 0 and x.data_ptr() % 16 != 0):
            raise ValueError(f"{op}: with x_scale, x must be the contiguous, 16-byte aligned float8_e4m3fn activation")
        if x_scale.dtype != torch.int32 or x_scale.dim() != 1 or x_scale.numel() != _ops.sf_words(m, k):
            raise ValueError(f"{op}: x_scale must be the int32 [{_ops.sf_words(m, k)}] scale of an [M, K] activation")
    return _ops.linear_mxfp8_swiglu(x, weight, x_scale, scale)


_dense_linear_swiglu_op = torch.library.custom_op(
    "fish_scales_ops::dense_linear_swiglu",
    mutates_args=(),
    schema="(Tensor x, Tensor weight, Tensor scale, Tensor? x_scale=None) -> (Tensor, Tensor)",
)(_dense_linear_swiglu_body)


@_dense_linear_swiglu_op.register_fake
def _dense_linear_swiglu_fake(x, weight, scale, x_scale=None):
    m, inter = x.shape[0], weight.shape[0] // 2
    return (x.new_empty((m, inter), dtype=torch.float8_e4m3fn),
            x.new_empty(((m + 127) // 128 * 128 * (inter // 128),), dtype=torch.int32))


def linear_swiglu(x: torch.Tensor, gate_up, *, x_scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``silu(x W_gate^T) * (x W_up^T)`` of a dense SwiGLU MLP in ONE launch, returned in the activation contract
    ``(float8_e4m3fn [M, INTER], int32 scale words)`` ready for ``fso.dense.linear(hq, down, x_scale=hs)``: the gate_up
    GEMM with the activation and the 1x32 quantization in its epilogue (fp32 accumulators, hardware tanh), so the bf16
    ``[M, 2*INTER]`` product never reaches memory. ``gate_up`` is the handle of :func:`prepare_gate_up`. The two-kernel
    form it replaces is ``silu_chunk_mul_quantize_1x32_fp8(fso.dense.linear(x, gate_up_plain))``
    (python/fish_scales_ops/gemm/mxfp8.py:216-236)."""
    from . import dense

    if not isinstance(gate_up, dense.DenseWeight):
        raise TypeError(f"fso.compat.linear_swiglu: gate_up must be the handle of fso.compat.prepare_gate_up, got "
                        f"{type(gate_up).__name__}")
    k = gate_up.in_features
    x2 = x if x_scale is not None else x.reshape(-1, k)
    return eager_or_op(_dense_linear_swiglu_body, torch.ops.fish_scales_ops.dense_linear_swiglu, x2, gate_up.weight,
                       gate_up.scale, x_scale)


# ------------------------------------------------------------------------------------------- shared expert overlap

# One side stream per process for the shared expert, created on first use: creating a stream inside a CUDA-graph
# capture would put host-side set-up in the middle of the capture (python/fish_scales_ops/gemm/mxfp8.py:2389-2408).
_SIDE_STREAM = None


def _side_stream():
    global _SIDE_STREAM
    if _SIDE_STREAM is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("fso.compat.moe_layer_shared: the first overlapped call of a process creates the side "
                               "stream of the shared expert, which cannot happen inside a CUDA-graph capture; call it "
                               "once eagerly before capturing, or pass overlap=False (FSO_MOE_BLOCK_OVERLAP=0 turns "
                               "the overlap off process-wide)")
        _SIDE_STREAM = torch.cuda.Stream()
    return _SIDE_STREAM


def _overlap_default() -> bool:
    import os

    return os.environ.get("FSO_MOE_BLOCK_OVERLAP", "1").strip().lower() not in ("0", "false", "off", "no")


def shared_expert(hidden: torch.Tensor, gate_up, down) -> torch.Tensor:
    """The always-on dense expert of a MoE block: ``(silu(x W_gate^T) * (x W_up^T)) W_down^T`` as two GEMM launches
    and the activation quantizer (gate_up with the fused SiLU(gate)*up requantizing epilogue, then down); bf16
    ``[M, H]``. ``gate_up`` from :func:`prepare_gate_up`, ``down`` from ``fso.dense.prepare_weight``
    (python/fish_scales_ops/gemm/mxfp8.py:2421-2428 runs the same chain in four kernels)."""
    from . import dense

    hq, hs = linear_swiglu(hidden, gate_up)
    return dense.linear(hq, down, x_scale=hs)


def moe_layer_shared(hidden: torch.Tensor, experts, topk_ids: torch.Tensor, topk_w: torch.Tensor, *, gate_up, down,
                     shared_gate: Optional[torch.Tensor] = None, overlap: Optional[bool] = None) -> torch.Tensor:
    """The routed experts of ``fso.moe.layer`` plus a shared expert, added inside the combine kernel:
    ``out[t] = sum_j topk_w[t, j] * expert_{ids[t, j]}(hidden[t]) + shared_gate[t] * shared(hidden[t])``.

    With ``overlap`` (default on; ``FSO_MOE_BLOCK_OVERLAP=0`` turns it off process-wide) the shared expert depends
    only on the layer's input, so it is issued on a side stream and waited for at the latest point that needs it:
    right before the combine. The two branches run concurrently, eagerly and inside a captured graph alike; the
    output is bit-identical either way, the join being a stream dependency and not a change of arithmetic
    (python/fish_scales_ops/gemm/mxfp8.py:2578-2611)."""
    from . import moe

    use_overlap = _overlap_default() if overlap is None else bool(overlap)
    if not use_overlap or hidden.shape[0] == 0:
        bias = shared_expert(hidden, gate_up, down)
        return moe.layer(hidden, experts, topk_ids, topk_w, bias=bias, bias_scale=shared_gate)
    current = torch.cuda.current_stream()
    side = _side_stream()
    side.wait_stream(current)
    with torch.cuda.stream(side):
        bias = shared_expert(hidden, gate_up, down)
    # the combine reads it on the current stream: the allocator must not hand the block out again before that read
    bias.record_stream(current)
    moe._BEFORE_COMBINE.fn = lambda: current.wait_stream(side)
    try:
        return moe.layer(hidden, experts, topk_ids, topk_w, bias=bias, bias_scale=shared_gate)
    finally:
        moe._BEFORE_COMBINE.fn = None
