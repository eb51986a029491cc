"""``fso.moe`` on a B200: the routed experts of one MoE layer behind the reference's own surface.

    experts = fso.moe.prepare_experts(w13, w2, format="mxfp8")       # load time
    out = fso.moe.layer(hidden, experts, topk_ids, topk_w)             # per call
    fso.moe.transient_bytes(experts, tokens, topk)                     # memory one call allocates

Mirrors python/fish_scales_ops/moe/__init__.py of the reference for the sm_100 family (names, argument meaning,
handle fields, the ``fish_scales_ops::moe_layer`` schema and fake, error classes). One route: compact routing ->
token gather + 1x32 quantize -> grouped tcgen05 GEMM with the fused SiLU(gate)*up requantize -> grouped GEMM ->
weighted un-permute. Ids outside ``[0, E_local)`` are skipped, so an expert-parallel caller maps non-local experts
to -1 and reduces the partial sums itself.
"""
import dataclasses

import threading

import torch

from .. import _ops
from .._lib import eager_or_op, on_device
from .._arch import SERVED_MAJOR, arch_label, arch_major, device_arch, sm_major

__all__ = ["FORMATS", "MoeExperts", "prepare_experts", "layer", "transient_bytes", "supported", "describe"]

FORMATS = ("bsfp8", "mxfp8")
_UNSERVED = ("bf16", "bfloat16", "fp16", "float16", "fp32", "float32", "fp8", "int8", "w8a8",
             "int4", "w4a16", "w4a8", "mxfp4", "nvfp4")
FP8 = torch.float8_e4m3fn
_REGION_ALIGN = 1024
# The decode band (the reference's slot route, python/fish_scales_ops/gemm/mxfp8.py:540-551: "expected rows per expert
# <= 64"): calls of at most 64 tokens whose routed pairs are at most twice the experts they can reach, so that an
# expert in use holds a row or two, or at most 32 pairs, so that a block has one 32-row token sub-tile. There the
# swapped grouped GEMM (weights on MMA-M, only the experts in use) beats the 128-row tiles of the prefill kernels:
# measured under CUDA-graph replay, Mixtral 1 token 108 -> 81 us, 4 tokens 132 -> 114 us, 16 tokens 261 -> 242 us,
# DeepSeek-V3 16 tokens 841 -> 772 us, 64 tokens 1674 -> 1575 us (0.98 of the live weights' stream); with more rows
# per expert (Mixtral 24 to 64 tokens) the prefill kernels stream the weights faster and keep the call.
# FC2 takes the band whenever the call is in it; FC1 only when its live tiles fill the half-SM CTA slots one and a
# half times over (otherwise the fused prefill FC1, with its 256-row weight tiles, is ahead: DeepSeek-V3 1 token).
# Both choices are functions of (tokens, top-k, E, I, SM count) alone, so a captured graph replays for any routing.
# FSO_B200_MOE_DECODE=0 sends every call through the prefill kernels, =force every call of at most 64 tokens through
# the band (tests).
_DECODE_TOKENS = 64


def _sm_count() -> int:
    return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)


def _decode_band(tokens: int, topk: int, num_experts: int, inter: int):
    """(FC1 takes the decode band, FC2 takes the decode band)."""
    import os

    mode = os.environ.get("FSO_B200_MOE_DECODE", "1")
    if not 0 < tokens <= _DECODE_TOKENS or mode == "0":
        return False, False
    if mode == "force":
        return True, True
    pairs = tokens * topk
    live = min(pairs, num_experts)
    # at most two rows per expert in use, or so few pairs that every block has a single 32-row token sub-tile
    if pairs > 2 * live and pairs > 32:
        return False, False
    return live * (2 * inter // 128) >= 3 * _sm_count(), True


def supported(format, arch=None) -> bool:
    """Whether ``format`` is served on ``arch`` (this device when None); never raises for an unknown format
    (python/fish_scales_ops/moe/__init__.py:159-177)."""
    if not isinstance(format, str) or format.strip().lower() not in FORMATS:
        return False
    major = sm_major() if arch is None else arch_major(arch)
    return major == SERVED_MAJOR


def describe() -> str:
    """The routes of this build as text; never raises."""
    arch = device_arch()
    name = ""
    if arch > 0:
        try:
            name = f" ({torch.cuda.get_device_name(0)})"
        except Exception:  # noqa: BLE001
            name = ""
    lines = [
        f"fish_scales_ops_b200.moe: MXFP8 MoE layer for sm_100a; this device is {arch_label(arch)}{name}.",
        "format 'mxfp8': bf16 experts are quantized to MXFP8 1x32 at load time (FC1 rows interleaved gate/up); "
        "float8_e4m3fn experts with uint8 UE8M0 scales keep their bytes and get their scales packed.",
        "format 'bsfp8': float8_e4m3fn experts with fp32 128x128 block scales are requantized to MXFP8 1x32.",
        "layer(): compact routing (deterministic order), token gather + quantize, grouped tcgen05 GEMM with the "
        "fused SiLU(gate)*up requantize, grouped GEMM, top-k weighted un-permute; calls of at most 64 tokens with a "
        "row or two per expert take the decode band instead (weights of the experts in use on MMA-M, SiLU(gate)*up as "
        "a row-wise kernel between the two GEMMs). Top-k ids outside [0, E_local) are "
        "skipped at no expert cost, and the result is this rank's partial sum, which the caller reduces across ranks.",
    ]
    if arch // 10 != SERVED_MAJOR:
        lines.append(f"This device ({arch_label(arch)}) serves no format.")
    return "\n".join(lines)


@dataclasses.dataclass(frozen=True, eq=False, repr=False)
class MoeExperts:
    """The prepared experts of one layer (python/fish_scales_ops/moe/__init__.py:244-282): ``w13`` float8_e4m3fn
    ``[E, 2I, H]`` with its rows interleaved gate/up, ``sw13`` int32 ``[E, 2I*H/128]`` (one atom slab per expert),
    ``w2`` ``[E, H, I]``, ``sw2`` int32 ``[E, H*I/128]``."""

    kind: str
    arch: int
    num_experts: int
    hidden: int
    inter: int
    w13: torch.Tensor
    sw13: torch.Tensor
    w2: torch.Tensor
    sw2: torch.Tensor
    w13_interleaved: bool

    def __repr__(self) -> str:
        return (f"MoeExperts(kind={self.kind!r}, arch=sm_{self.arch}, num_experts={self.num_experts}, "
                f"hidden={self.hidden}, inter={self.inter}, w13_interleaved={self.w13_interleaved}, "
                f"w13={tuple(self.w13.shape)} {self.w13.dtype}, sw13={tuple(self.sw13.shape)} {self.sw13.dtype}, "
                f"w2={tuple(self.w2.shape)} {self.w2.dtype}, sw2={tuple(self.sw2.shape)} {self.sw2.dtype})")


def _check_expert_tensors(w13, w2, fmt: str, where: str):
    """(E, H, I) of a stacked expert pair after checking that the two tensors describe the same experts."""
    ctx = f"fso.moe.prepare_experts (format {fmt!r}, {where})"
    both = {"w13": w13, "w2": w2}
    for name, t in both.items():
        if not isinstance(t, torch.Tensor):
            raise ValueError(f"{ctx}: {name} is a {type(t).__name__}, not a tensor")
    for name, t in both.items():
        if t.dim() != 3:
            raise ValueError(f"{ctx}: {name} has shape {tuple(t.shape)}; experts are stacked along a leading "
                             f"dimension ([E, 2*I, H] and [E, H, I])")
        if not t.is_cuda:
            raise ValueError(f"{ctx}: {name} is on {t.device}; the experts must be on the CUDA device that runs the "
                             f"layer")
    if w13.device != w2.device:
        raise ValueError(f"{ctx}: the two tensors are on different devices ({w13.device} and {w2.device})")
    e, two_i, h = map(int, w13.shape)
    e2, h2, i = map(int, w2.shape)
    if e != e2:
        raise ValueError(f"{ctx}: {e} experts in w13 but {e2} in w2")
    if e < 1 or e > 1024:
        raise ValueError(f"{ctx}: the routing kernels serve 1 to 1024 local experts, got {e}")
    if h != h2:
        raise ValueError(f"{ctx}: the hidden size differs between w13 [E, 2*I, {h}] and w2 [E, {h2}, I]")
    if two_i != 2 * i:
        raise ValueError(f"{ctx}: w13 must stack the gate and the up projection, 2*I = {2 * i} rows per expert for "
                         f"w2's I = {i}; it has {two_i}")
    for label, v in (("hidden size H", h), ("intermediate size I (per rank)", i)):
        if v % 128 != 0:
            raise ValueError(f"{ctx}: the {label} = {v} must be a multiple of 128")
    return e, h, i


def _aligned_storage(t: torch.Tensor) -> torch.Tensor:
    return t.clone() if t.numel() > 0 and t.data_ptr() % 16 != 0 else t


def _interleave_perm(two_i: int, device) -> torch.Tensor:
    """perm[r] = source row of output row r: [gate; up] -> [g0, u0, g1, u1, ...]
    (python/fish_scales_ops/gemm/mxfp8.py:621-633)."""
    inter = two_i // 2
    idx = torch.arange(inter, dtype=torch.long, device=device)
    perm = torch.empty(two_i, dtype=torch.long, device=device)
    perm[0::2] = idx
    perm[1::2] = inter + idx
    return perm


def prepare_experts(w13, w2, *, format, sw13=None, sw2=None) -> MoeExperts:
    """Prepare one layer's local experts, once, at load time (python/fish_scales_ops/moe/__init__.py:481-601).

    ``w13`` is ``[E, 2*I, H]`` with the gate rows first, ``w2`` is ``[E, H, I]``. ``format="mxfp8"``: bf16 weights
    and no scales, or float8_e4m3fn weights with uint8 UE8M0 scales ``sw13 [E, 2I, H/32]``, ``sw2 [E, H, I/32]``.
    ``format="bsfp8"``: float8_e4m3fn weights with fp32 block scales ``sw13 [E, 2I/128, H/128]``,
    ``sw2 [E, H/128, I/128]``. The FC1 rows of the handle are always interleaved (gate_j, up_j adjacent), which the
    fused FC1 epilogue needs. ``H % 128 == 0``, ``I % 128 == 0``, ``1 <= E <= 1024``."""
    arch = device_arch()
    where = arch_label(arch)
    if not isinstance(format, str) or format.strip().lower() not in FORMATS:
        if isinstance(format, str) and format.strip().lower() in _UNSERVED:
            raise NotImplementedError(f"fso.moe.prepare_experts: format {format!r} is not served on any architecture "
                                      f"({where}); the formats are 'bsfp8' and 'mxfp8'")
        raise ValueError(f"fso.moe.prepare_experts: unknown format {format!r} on {where}; the formats are 'bsfp8' and "
                         f"'mxfp8'")
    fmt = format.strip().lower()
    if not supported(fmt):
        raise NotImplementedError(f"fso.moe.prepare_experts: this build serves sm_100-family devices only and this "
                                  f"device is {where}")
    e, h, i = _check_expert_tensors(w13, w2, fmt, where)
    ctx = f"fso.moe.prepare_experts (format {fmt!r}, {where})"
    if torch.cuda.get_device_capability(w13.device)[0] != SERVED_MAJOR:
        raise ValueError(f"{ctx}: the experts are on {w13.device}, which is not an sm_100-family device")

    if fmt == "bsfp8":
        for name, t in (("w13", w13), ("w2", w2)):
            if t.dtype != FP8:
                raise ValueError(f"{ctx}: {name} must be float8_e4m3fn, got {t.dtype}; bf16 experts are format='mxfp8'")
        want = {"sw13": (e, 2 * i // 128, h // 128), "sw2": (e, h // 128, i // 128)}
        for name, t in (("sw13", sw13), ("sw2", sw2)):
            if not isinstance(t, torch.Tensor):
                raise ValueError(f"{ctx}: {name} is required, fp32 {list(want[name])} (one scale per 128x128 block)")
            if t.dtype != torch.float32 or tuple(t.shape) != want[name]:
                raise ValueError(f"{ctx}: {name} must be fp32 {list(want[name])}, got {t.dtype} {list(t.shape)}")
            if t.device != w13.device:
                raise ValueError(f"{ctx}: {name} is on {t.device}, the weights on {w13.device}")
        q13, s13 = _ops.requant_block_fp8(w13.detach().contiguous().view(e * 2 * i, h),
                                          sw13.detach().contiguous().view(e * 2 * i // 128, h // 128), interleave_i=i)
        q2, s2 = _ops.requant_block_fp8(w2.detach().contiguous().view(e * h, i),
                                        sw2.detach().contiguous().view(e * h // 128, i // 128))
        return MoeExperts("mxfp8", arch, e, h, i, q13.view(e, 2 * i, h), s13.view(e, -1), q2.view(e, h, i),
                          s2.view(e, -1), True)

    for name, t in (("w13", w13), ("w2", w2)):
        if t.dtype not in (torch.bfloat16, FP8):
            raise ValueError(f"{ctx}: {name} is {t.dtype}; format 'mxfp8' takes bf16 experts, or float8_e4m3fn experts "
                             f"with uint8 UE8M0 scales")
    if w13.dtype != w2.dtype:
        raise ValueError(f"{ctx}: w13 is {w13.dtype} and w2 {w2.dtype}; both must have the same dtype")
    if w13.dtype == torch.bfloat16:
        if sw13 is not None or sw2 is not None:
            raise ValueError(f"{ctx}: bf16 experts are quantized here and take no scales")
        q13, s13 = _ops.quantize_experts_1x32_fp8(w13.detach().contiguous(), interleave=True)
        q2, s2 = _ops.quantize_experts_1x32_fp8(w2.detach().contiguous(), interleave=False)
        return MoeExperts("mxfp8", arch, e, h, i, q13, s13, q2, s2, True)

    want = {"sw13": (e, 2 * i, h // 32), "sw2": (e, h, i // 32)}
    for name, t in (("sw13", sw13), ("sw2", sw2)):
        if t is None or not isinstance(t, torch.Tensor):
            raise ValueError(f"{ctx}: float8_e4m3fn experts need their scales; {name} must be uint8 "
                             f"{list(want[name])}")
        if t.dtype != torch.uint8 or tuple(t.shape) != want[name]:
            raise ValueError(f"{ctx}: {name} must be uint8 {list(want[name])}, one UE8M0 byte per 32 elements along "
                             f"K, got {t.dtype} {list(t.shape)}")
        if t.device != w13.device:
            raise ValueError(f"{ctx}: {name} is on {t.device} and the weights on {w13.device}")
    perm = _interleave_perm(2 * i, w13.device)
    w13_q = w13.detach().view(torch.uint8).index_select(1, perm).view(FP8)
    s13_q = _ops.pack_ue8m0(sw13.detach(), interleave=True)
    w2_q = _aligned_storage(w2.detach().contiguous())
    s2_q = _ops.pack_ue8m0(sw2.detach())
    return MoeExperts("mxfp8", arch, e, h, i, w13_q, s13_q, w2_q, s2_q, True)


# ------------------------------------------------------------------------------------------------ the layer plan

def _alloc_bytes(nbytes: int) -> int:
    """Upper bound on what the caching allocator charges for one tensor: 512-byte blocks, and up to 1 MiB more for
    a tensor above 1 MiB served unsplit from a cached block (python/fish_scales_ops/gemm/mxfp8.py:1731-1741)."""
    n = int(nbytes)
    if n <= 0:
        return 0
    r = (n + 511) // 512 * 512
    return r + (1 << 20) if r > (1 << 20) else r


def _align_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


@dataclasses.dataclass(frozen=True)
class _LayerPlan:
    """Host-static sizes of one call: functions of (tokens, topk, E, H, I) only, so a CUDA graph captured for a token
    bucket replays for any routing. ``rows`` rows in every compact intermediate; one region holds the gathered
    activation and its scale words and is reused for the down-projection output once FC1 has consumed them."""

    pairs: int
    num_blocks: int
    rows: int
    route_scratch: int
    sh_off: int
    region: int
    gate_up: int       # bytes of the fp32 [rows, 2I] FC1 output of the decode band (0 when FC1 stays fused)
    fc2_decode: bool   # FC2 takes the decode band


def _layer_plan(tokens: int, topk: int, num_experts: int, hidden: int, inter: int) -> _LayerPlan:
    p = _ops.moe_plan(tokens, topk, num_experts)
    rows = int(p.rows)
    sh_off = _align_up(rows * hidden, _REGION_ALIGN)
    front = sh_off + 4 * rows * (hidden // 128)
    fc1_decode, fc2_decode = _decode_band(tokens, topk, num_experts, inter)
    return _LayerPlan(int(p.pairs), int(p.num_blocks), rows, int(p.route_scratch_bytes), sh_off,
                      max(front, 2 * rows * hidden), 8 * rows * inter if fc1_decode else 0, fc2_decode)


def _plan_bytes(plan: _LayerPlan, tokens: int, num_experts: int, hidden: int, inter: int) -> int:
    a = _alloc_bytes
    total = a(4 * num_experts) + a(4 * (num_experts + 1)) + a(4 * plan.pairs) + a(4 * plan.num_blocks)
    total += a(plan.route_scratch)
    total += a(plan.region)
    total += a(plan.rows * inter) + a(4 * plan.rows * (inter // 128))
    total += a(plan.gate_up)
    total += a(2 * tokens * hidden)
    return total


def _bf16_storage(t):
    if t.numel() > 0 and (not t.is_contiguous() or t.data_ptr() % 16 != 0):
        return t.contiguous() if not t.is_contiguous() else t.clone()
    return t


def _require_experts_aligned(w13, sw13, w2, sw2, where: str) -> None:
    for name, t in (("w13", w13), ("sw13", sw13), ("w2", w2), ("sw2", sw2)):
        if t.numel() > 0 and t.data_ptr() % 16 != 0:
            raise ValueError(f"fish_scales_ops::moe_layer ({where}, kind 'mxfp8'): {name}'s data pointer is "
                             f"{t.data_ptr() % 16} bytes past a 16-byte boundary; the grouped GEMMs read it in place "
                             f"with TMA. fso.moe.prepare_experts returns aligned tensors")
        if not t.is_contiguous():
            raise ValueError(f"fish_scales_ops::moe_layer ({where}, kind 'mxfp8'): {name} must be contiguous")


# A stream dependency to establish right before the combine kernel of the next layer call of this thread (set by
# fso.compat.moe_layer_shared, whose shared expert runs on a side stream and is only read by the combine).
_BEFORE_COMBINE = threading.local()


def _run_layer(hidden, w13, sw13, w2, sw2, topk_ids, topk_w, bias, bias_scale):
    t, h = int(hidden.shape[0]), int(hidden.shape[1])
    e, two_i, _ = (int(v) for v in w13.shape)
    inter = two_i // 2
    topk = int(topk_ids.shape[1])
    dev = hidden.device
    plan = _layer_plan(t, topk, e, h, inter)
    with on_device(dev):
        mplan = _ops.moe_plan(t, topk, e)
        masked_m, blk0, slot, blk_expert = _ops.moe_route(topk_ids, e, mplan)
        region = torch.empty((plan.region,), dtype=torch.uint8, device=dev)
        hq = region[:plan.rows * h].view(FP8).view(plan.rows, h)
        sh = region[plan.sh_off:plan.sh_off + 4 * plan.rows * (h // 128)].view(torch.int32)
        dq = torch.empty((plan.rows, inter), dtype=FP8, device=dev)
        sd = torch.empty((plan.rows * (inter // 128),), dtype=torch.int32, device=dev)
        out = torch.empty((t, h), dtype=torch.bfloat16, device=dev)
        _ops.moe_gather_quant(hidden, slot, topk, hq, sh)
        if plan.gate_up > 0:
            # decode band: only the experts in use are touched, their weights on MMA-M; FC1's fp32 gate / up
            # accumulators go through the row-wise silu(gate) * up requantizer
            gu = torch.empty((plan.rows, 2 * inter), dtype=torch.float32, device=dev)
            _ops.moe_grouped_gemm_decode(hq, sh, w13, sw13, masked_m, blk0, blk_expert, gu, t, topk)
            _ops.moe_silu_mul_quantize_rows(gu, masked_m, blk0, blk_expert, e, dq, sd)
        else:
            _ops.moe_fc1_swiglu(hq, sh, w13, sw13, blk0, blk_expert, dq, sd)
        dn = region[:2 * plan.rows * h].view(torch.bfloat16).view(plan.rows, h)
        if plan.fc2_decode:
            _ops.moe_grouped_gemm_decode(dq, sd, w2, sw2, masked_m, blk0, blk_expert, dn, t, topk)
        else:
            _ops.moe_fc2(dq, sd, w2, sw2, blk0, blk_expert, dn)
        join = getattr(_BEFORE_COMBINE, "fn", None)
        if join is not None:
            join()
        _ops.moe_combine(dn, slot, topk_w, bias, bias_scale, out)
    return out


def _run_layer_rows(rx_q, rx_w, experts, topk_ids, topk_w, recv_off, back_base, peer_back, world):
    """The layer over rows that arrive already quantized and whose result rows leave for other buffers: the
    expert-parallel form. ``rx_q`` e4m3 codes ``[R, H]`` and ``rx_w`` int32 scale words ``[R, H/128]`` (row-major, as
    the sending rank's dispatch kernel stored them), ``topk_ids`` int32 ``[R, k]`` local expert ids (-1 = another
    rank's expert), ``topk_w`` fp32 ``[R, k]``. Result row t is written by the combine kernel to row
    ``back_base[s] + (t - recv_off[s])`` of the bf16 buffer at address ``peer_back[s]`` (``s`` = the rank the row
    came from). Same kernels as :func:`layer` except that the gather copies instead of quantizing."""
    w13, sw13, w2, sw2 = experts.w13, experts.sw13, experts.w2, experts.sw2
    r, h = int(rx_q.shape[0]), int(rx_q.shape[1])
    if r == 0:
        return
    e, two_i, _ = (int(v) for v in w13.shape)
    inter = two_i // 2
    topk = int(topk_ids.shape[1])
    dev = rx_q.device
    _require_experts_aligned(w13, sw13, w2, sw2, "expert-parallel")
    plan = _layer_plan(r, topk, e, h, inter)
    with on_device(dev):
        mplan = _ops.moe_plan(r, topk, e)
        masked_m, blk0, slot, blk_expert = _ops.moe_route(topk_ids, e, mplan)
        region = torch.empty((plan.region,), dtype=torch.uint8, device=dev)
        hq = region[:plan.rows * h].view(FP8).view(plan.rows, h)
        sh = region[plan.sh_off:plan.sh_off + 4 * plan.rows * (h // 128)].view(torch.int32)
        dq = torch.empty((plan.rows, inter), dtype=FP8, device=dev)
        sd = torch.empty((plan.rows * (inter // 128),), dtype=torch.int32, device=dev)
        _ops.moe_gather_rows(rx_q, rx_w, slot, topk, hq, sh)
        _ops.moe_fc1_swiglu(hq, sh, w13, sw13, blk0, blk_expert, dq, sd)
        dn = region[:2 * plan.rows * h].view(torch.bfloat16).view(plan.rows, h)
        _ops.moe_fc2(dq, sd, w2, sw2, blk0, blk_expert, dn)
        _ops.moe_combine_scatter(dn, slot, topk_w, recv_off, back_base, peer_back, world)


def _moe_layer_body(hidden, w13, sw13, w2, sw2, topk_ids, topk_w, bias, bias_scale, kind, w13_interleaved):
    """Body of ``torch.ops.fish_scales_ops.moe_layer`` (python/fish_scales_ops/moe/__init__.py:651-719)."""
    arch = device_arch()
    where = arch_label(arch)
    if kind == "bsfp8":
        raise NotImplementedError(f"fish_scales_ops::moe_layer: kind 'bsfp8' is the sm_90 block-FP8 layer and this "
                                  f"device is {where}; fso.moe.prepare_experts requantizes block-FP8 experts to MXFP8")
    if kind != "mxfp8":
        raise ValueError(f"fish_scales_ops::moe_layer: unknown kind {kind!r} on {where}; the kinds are 'bsfp8' and "
                         f"'mxfp8', produced by fso.moe.prepare_experts")
    if arch // 10 != SERVED_MAJOR:
        raise NotImplementedError(f"fish_scales_ops::moe_layer: kind 'mxfp8' needs an sm_100-family device in this "
                                  f"build and this device is {where}")
    if not w13_interleaved:
        raise NotImplementedError(f"fish_scales_ops::moe_layer ({where}): this build runs the fused FC1 only, which "
                                  f"needs the interleaved gate/up rows fso.moe.prepare_experts produces")
    if int(hidden.shape[0]) > 0:
        _require_experts_aligned(w13, sw13, w2, sw2, where)
    if topk_ids.dtype != torch.int32 or not topk_ids.is_contiguous():
        topk_ids = topk_ids.to(torch.int32).contiguous()
    if topk_w.dtype != torch.float32 or not topk_w.is_contiguous():
        topk_w = topk_w.to(torch.float32).contiguous()
    hidden = _bf16_storage(hidden)
    if bias_scale is not None:
        if bias is None:
            raise ValueError(f"fish_scales_ops::moe_layer ({where}): bias_scale scales bias and needs it")
        bias_scale = bias_scale.reshape(-1).to(torch.float32).contiguous()
    if bias is not None:
        bias = _bf16_storage(bias.contiguous())
    if int(hidden.shape[0]) == 0:
        return hidden.new_empty(hidden.shape)
    return _run_layer(hidden, w13, sw13, w2, sw2, topk_ids, topk_w, bias, bias_scale)


_moe_layer_op = torch.library.custom_op(
    "fish_scales_ops::moe_layer",
    mutates_args=(),
    schema="(Tensor hidden, Tensor w13, Tensor sw13, Tensor w2, Tensor sw2, Tensor topk_ids, "
           "Tensor topk_w, Tensor? bias, Tensor? bias_scale, str kind, bool w13_interleaved) -> Tensor",
)(_moe_layer_body)


@_moe_layer_op.register_fake
def _moe_layer_fake(hidden, w13, sw13, w2, sw2, topk_ids, topk_w, bias, bias_scale, kind, w13_interleaved):
    return hidden.new_empty(hidden.shape)


def layer(hidden, experts, topk_ids, topk_w, *, bias=None, bias_scale=None) -> torch.Tensor:
    """``out[t] = sum_j topk_w[t, j] * expert_{topk_ids[t, j]}(hidden[t])`` (+ ``bias_scale[t] * bias[t]``), with
    ``expert_e(x) = (silu(x W_gate^T) * (x W_up^T)) W_down^T`` over the local experts; ids outside
    ``[0, E_local)`` are skipped; bf16 ``[M, H]`` (python/fish_scales_ops/moe/__init__.py:727-813)."""
    arch = device_arch()
    where = arch_label(arch)
    if not isinstance(experts, MoeExperts):
        raise TypeError(f"fso.moe.layer ({where}): experts is a {type(experts).__name__}; pass the MoeExperts that "
                        f"fso.moe.prepare_experts returned")
    if experts.arch // 10 != arch // 10:
        raise ValueError(f"fso.moe.layer: these experts were prepared for sm_{experts.arch}, the current device is "
                         f"{where}")
    tag = f"fso.moe.layer ({where}, kind {experts.kind!r})"
    h = experts.hidden
    if not (isinstance(hidden, torch.Tensor) and hidden.dim() == 2 and hidden.dtype == torch.bfloat16):
        raise ValueError(f"{tag}: hidden must be a bf16 [M, H] tensor")
    m = int(hidden.shape[0])
    if int(hidden.shape[1]) != h:
        raise ValueError(f"{tag}: hidden has {int(hidden.shape[1])} columns, the experts were prepared for H = {h}")
    routing_ok = (isinstance(topk_ids, torch.Tensor) and isinstance(topk_w, torch.Tensor) and topk_ids.dim() == 2
                  and topk_ids.shape == topk_w.shape and int(topk_ids.shape[0]) == m)
    if not routing_ok:
        raise ValueError(f"{tag}: topk_ids and topk_w must be two [M, topk] tensors of one shape, M = {m}")
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"{tag}: topk_ids is {topk_ids.dtype}; expert ids are int32 or int64")
    if not topk_w.is_floating_point():
        raise ValueError(f"{tag}: topk_w is {topk_w.dtype}; routing weights are floating point")
    if bias is not None and not (bias.dim() == 2 and tuple(bias.shape) == (m, h) and bias.dtype == torch.bfloat16):
        raise ValueError(f"{tag}: bias must be bf16 [{m}, {h}]; got {bias.dtype} {tuple(bias.shape)}")
    if bias_scale is not None:
        if bias is None:
            raise ValueError(f"{tag}: bias_scale multiplies bias and cannot be given without it")
        if bias_scale.numel() != m or not bias_scale.is_floating_point():
            raise ValueError(f"{tag}: bias_scale must be one floating-point factor per token ({m} of them)")
        bias_scale = bias_scale.reshape(m).to(torch.float32).contiguous()
    ids = topk_ids.to(torch.int32).contiguous()
    wts = topk_w.to(torch.float32).contiguous()
    return eager_or_op(_moe_layer_body, torch.ops.fish_scales_ops.moe_layer, hidden.contiguous(), experts.w13,
                       experts.sw13, experts.w2, experts.sw2, ids, wts, None if bias is None else bias.contiguous(),
                       bias_scale, experts.kind, experts.w13_interleaved)


def transient_bytes(experts, tokens, topk) -> int:
    """Device memory, in bytes, one :func:`layer` call with ``tokens`` rows allocates: the routing tensors, the
    shared gather / down-projection region, the FC1 output and its scales (in the decode band also its fp32 gate / up
    accumulators) and the result, each charged as the caching allocator can charge it. The layer and this function
    read the same plan (python/fish_scales_ops/moe/__init__.py:816-870)."""
    arch = device_arch()
    where = arch_label(arch)
    if not isinstance(experts, MoeExperts):
        raise TypeError(f"fso.moe.transient_bytes ({where}): experts is a {type(experts).__name__}; pass the "
                        f"MoeExperts that fso.moe.prepare_experts returned")
    if experts.arch // 10 != arch // 10:
        raise ValueError(f"fso.moe.transient_bytes: these experts were prepared for sm_{experts.arch}, the current "
                         f"device is {where}")
    counts = {"tokens": tokens, "topk": topk}
    for name, v in counts.items():
        if isinstance(v, bool) or not isinstance(v, int) or v < 0:
            raise ValueError(f"fso.moe.transient_bytes ({where}): {name} = {v!r} is not a non-negative int")
    if tokens == 0:
        return 0
    if topk == 0:
        raise ValueError(f"fso.moe.transient_bytes ({where}): a call with tokens routes each of them to at least one "
                         f"expert (topk >= 1)")
    plan = _layer_plan(tokens, topk, experts.num_experts, experts.hidden, experts.inter)
    return _plan_bytes(plan, tokens, experts.num_experts, experts.hidden, experts.inter)
