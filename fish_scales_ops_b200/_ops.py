"""Tensor-level wrappers of the C ABI: they allocate the outputs with the torch caching allocator on the current
stream and call the library with raw pointers. No wrapper synchronizes or reads a tensor's values, so every call is
capturable into a CUDA graph after one eager call of the same shape.

These are the counterparts of the reference's raw ops (csrc/gemm/bindings.cpp:189-360) for the sm_100 path:
``quantize_1x32_packed``, ``linear_mxfp8_raw``, ``moe_build_routing_compact``,
``quantize_1x32_grouped_gather_out``, ``linear_mxfp8_grouped_compact[_swiglu]`` and ``moe_combine``.
"""
import ctypes

import torch

from . import _lib
from ._lib import MoePlan, check, lib, on_device, ptr, stream_ptr

FP8 = torch.float8_e4m3fn


def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def sf_words(rows: int, k: int) -> int:
    """int32 words of the scale tensor of a [rows, k] MXFP8 tensor (padded rows included)."""
    return _align(rows, 128) * (k // 128)


def quantize_1x32_fp8(x: torch.Tensor, interleave_i: int = 0, activation: bool = False):
    """bf16 [M, K] -> (float8_e4m3fn [M, K], int32 [align(M,128) * K/128]); python/fish_scales_ops/gemm/mxfp8.py:191-213.
    ``activation``: the form whose kernel lets a decode GEMM behind it start loading weights early (same bytes)."""
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_cuda:
        raise ValueError(f"quantize_1x32_fp8: x must be a CUDA bf16 [M, K] tensor, got {x.dtype} {tuple(x.shape)}")
    x = x.contiguous()
    m, k = int(x.shape[0]), int(x.shape[1])
    if k % 128 != 0:
        raise ValueError(f"quantize_1x32_fp8: K = {k} is not a multiple of 128")
    with on_device(x.device):
        xq = torch.empty((m, k), dtype=FP8, device=x.device)
        sf = torch.empty((sf_words(m, k),), dtype=torch.int32, device=x.device)
        if m > 0 and activation and interleave_i == 0:
            check(lib().fso_quantize_activation_1x32(ptr(x), ptr(xq), ptr(sf), m, k, stream_ptr()),
                  "fso_quantize_activation_1x32")
        elif m > 0:
            check(lib().fso_quantize_1x32(ptr(x), ptr(xq), ptr(sf), m, k, int(interleave_i), stream_ptr()),
                  "fso_quantize_1x32")
    return xq, sf


def silu_mul_quantize_1x32_fp8(gu: torch.Tensor):
    """bf16 [M, 2I] (gate | up) -> (float8_e4m3fn [M, I], int32 scale words): silu(gate) * up, quantized."""
    m, two_i = int(gu.shape[0]), int(gu.shape[1])
    inter = two_i // 2
    with on_device(gu.device):
        xq = torch.empty((m, inter), dtype=FP8, device=gu.device)
        sf = torch.empty((sf_words(m, inter),), dtype=torch.int32, device=gu.device)
        if m > 0:
            check(lib().fso_silu_mul_quantize_1x32(ptr(gu), ptr(xq), ptr(sf), m, inter, stream_ptr()),
                  "fso_silu_mul_quantize_1x32")
    return xq, sf


def stream_fence(device) -> None:
    """One empty plain launch on the current stream of ``device`` (orders programmatic dependent launches)."""
    with on_device(device):
        check(lib().fso_stream_fence(stream_ptr()), "fso_stream_fence")


def quantize_experts_1x32_fp8(w: torch.Tensor, interleave: bool):
    """bf16 [E, N, K] -> (float8_e4m3fn [E, N, K], int32 [E, N * K/128]), one atom slab per expert
    (python/fish_scales_ops/gemm/mxfp8.py:1511-1582). With ``interleave`` the rows of every expert are re-ordered
    [gate; up] -> [g0, u0, g1, u1, ...] on the way."""
    e, n, k = (int(v) for v in w.shape)
    if n % 128 != 0 or k % 128 != 0:
        raise ValueError(f"quantize_experts_1x32_fp8: N = {n} and K = {k} must be multiples of 128")
    q, s = quantize_1x32_fp8(w.reshape(e * n, k), interleave_i=n // 2 if interleave else 0)
    return q.view(e, n, k), s.view(e, n * (k // 128))


def requant_block_fp8(wq: torch.Tensor, scale: torch.Tensor, interleave_i: int = 0):
    """Block-FP8 [N, K] + fp32 [N/128, K/128] -> MXFP8 (python/fish_scales_ops/dense/__init__.py:422-462).
    ``interleave_i``: the rows are stacked [2*I, K] experts re-ordered [gate; up] -> [g0, u0, ...] on the way."""
    n, k = int(wq.shape[0]), int(wq.shape[1])
    wq = wq.contiguous()
    scale = scale.contiguous()
    with on_device(wq.device):
        q = torch.empty((n, k), dtype=FP8, device=wq.device)
        sf = torch.empty((sf_words(n, k),), dtype=torch.int32, device=wq.device)
        check(lib().fso_requant_bs128_to_mx(ptr(wq), ptr(scale), ptr(q), ptr(sf), n, k, int(interleave_i), stream_ptr()),
              "fso_requant_bs128_to_mx")
    return q, sf


def pack_ue8m0(sf_u8: torch.Tensor, interleave: bool = False) -> torch.Tensor:
    """uint8 [G, N, K/32] -> int32 [G, align(N,128) * K/128] (python/fish_scales_ops/gemm/mxfp8.py:718-768)."""
    if sf_u8.dtype != torch.uint8 or sf_u8.dim() != 3 or int(sf_u8.shape[2]) % 4 != 0:
        raise ValueError(f"pack_ue8m0: sf must be uint8 [G, N, K/32] with K % 128 == 0, got {sf_u8.dtype} "
                         f"{list(sf_u8.shape)}")
    s = sf_u8.contiguous()
    g, n, k = int(s.shape[0]), int(s.shape[1]), int(s.shape[2]) * 32
    with on_device(s.device):
        out = torch.empty((g, sf_words(n, k)), dtype=torch.int32, device=s.device)
        check(lib().fso_pack_ue8m0(ptr(s), ptr(out), g, n, k, n // 2 if interleave else 0, stream_ptr()),
              "fso_pack_ue8m0")
    return out


def gemm_ws_bytes(m: int, n: int, k: int) -> int:
    v = ctypes.c_int64(0)
    check(lib().fso_gemm_mxfp8_ws_bytes(m, n, k, ctypes.byref(v)), "fso_gemm_mxfp8_ws_bytes")
    return int(v.value)


def gemm_describe(m: int, n: int, k: int, sm_count: int = 0) -> dict:
    """The route the dense GEMM takes for one shape (host arithmetic only; ``sm_count`` 0 = the current device's)."""
    out = (ctypes.c_int32 * 6)()
    check(lib().fso_gemm_mxfp8_describe(m, n, k, sm_count, out), "fso_gemm_mxfp8_describe")
    return {"swapped": bool(out[0]), "tile_n": int(out[1]), "k_slices": int(out[2]), "k_blocks_per_slice": int(out[3]),
            "pair_kernel": bool(out[4]), "tiles": int(out[5])}


def linear_mxfp8(xq: torch.Tensor, w: torch.Tensor, sx: torch.Tensor, sw: torch.Tensor, bias=None, residual=None,
                 activation: int = 0) -> torch.Tensor:
    """bf16 [M, N] = xq [M, K] @ w [N, K]^T over MXFP8 operands (python/fish_scales_ops/gemm/mxfp8.py:90-188), with
    the dense epilogue bf16(act(acc + bias) + residual) when any of its fields is given."""
    m, k = int(xq.shape[0]), int(xq.shape[1])
    n = int(w.shape[0])
    with on_device(xq.device):
        out = torch.empty((m, n), dtype=torch.bfloat16, device=xq.device)
        if m == 0:
            return out
        ws_bytes = gemm_ws_bytes(m, n, k)
        ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=xq.device) if ws_bytes > 0 else None
        if bias is None and residual is None and activation == 0:
            check(lib().fso_gemm_mxfp8(ptr(xq), ptr(sx), ptr(w), ptr(sw), ptr(out), m, n, k, ptr(ws), ws_bytes,
                                       stream_ptr()), "fso_gemm_mxfp8")
        else:
            check(lib().fso_gemm_mxfp8_epilogue(ptr(xq), ptr(sx), ptr(w), ptr(sw), ptr(out), m, n, k, ptr(bias),
                                                ptr(residual), int(activation), ptr(ws), ws_bytes, stream_ptr()),
                  "fso_gemm_mxfp8_epilogue")
    return out


_FUSES_QUANT = {}


def gemm_fuses_quantized_output(m: int, n: int, k: int) -> bool:
    """Whether this shape's GEMM can emit the activation contract itself (a pure function of the shape and the
    device's SM count; cached)."""
    key = (m, n, k, torch.cuda.current_device())
    if key not in _FUSES_QUANT:
        v = ctypes.c_int(0)
        check(lib().fso_gemm_mxfp8_fuses_quantized_output(m, n, k, ctypes.byref(v)), "fso_gemm_mxfp8_fuses_quantized_output")
        _FUSES_QUANT[key] = bool(v.value)
    return _FUSES_QUANT[key]


def linear_mxfp8_quantized(xq, w, sx, sw, bias=None, activation: int = 0):
    """(float8_e4m3fn [M, N], int32 scale words) = quantize_activation(linear_mxfp8(...)), bit for bit; one launch
    where the shape allows, otherwise the GEMM followed by the activation quantizer."""
    m, k = int(xq.shape[0]), int(xq.shape[1])
    n = int(w.shape[0])
    with on_device(xq.device):
        if m > 0 and gemm_fuses_quantized_output(m, n, k):
            out = torch.empty((m, n), dtype=FP8, device=xq.device)
            sf = torch.empty((sf_words(m, n),), dtype=torch.int32, device=xq.device)
            check(lib().fso_gemm_mxfp8_quantized(ptr(xq), ptr(sx), ptr(w), ptr(sw), ptr(out), ptr(sf), m, n, k, ptr(bias),
                                                 int(activation), stream_ptr()), "fso_gemm_mxfp8_quantized")
            return out, sf
    y = linear_mxfp8(xq, w, sx, sw, bias, None, activation)
    return quantize_1x32_fp8(y, activation=True)


def linear_mxfp8_swiglu(xq, w_interleaved, sx, sw):
    """silu(gate) * up of the gate_up projection as (float8_e4m3fn [M, I], int32 scale words), one launch;
    ``w_interleaved`` e4m3 [2I, K] with gate_j / up_j in rows 2j / 2j+1."""
    m, k = int(xq.shape[0]), int(xq.shape[1])
    two_i = int(w_interleaved.shape[0])
    inter = two_i // 2
    with on_device(xq.device):
        dq = torch.empty((m, inter), dtype=FP8, device=xq.device)
        sd = torch.empty((sf_words(m, inter),), dtype=torch.int32, device=xq.device)
        if m > 0:
            check(lib().fso_gemm_mxfp8_swiglu(ptr(xq), ptr(sx), ptr(w_interleaved), ptr(sw), ptr(dq), ptr(sd), m, two_i,
                                              k, stream_ptr()), "fso_gemm_mxfp8_swiglu")
    return dq, sd


def moe_plan(tokens: int, topk: int, num_experts: int) -> MoePlan:
    p = MoePlan()
    check(lib().fso_moe_plan_make(tokens, topk, num_experts, ctypes.byref(p)), "fso_moe_plan_make")
    return p


def moe_route(ids: torch.Tensor, num_experts: int, plan: MoePlan):
    """ids int32 [T, topk] -> (masked_m [E], blk0 [E+1], slot_of_flat [T*topk], blk_expert [num_blocks])."""
    t, topk = int(ids.shape[0]), int(ids.shape[1])
    dev = ids.device
    with on_device(dev):
        masked_m = torch.empty((num_experts,), dtype=torch.int32, device=dev)
        blk0 = torch.empty((num_experts + 1,), dtype=torch.int32, device=dev)
        slot = torch.empty((t * topk,), dtype=torch.int32, device=dev)
        blk_expert = torch.empty((int(plan.num_blocks),), dtype=torch.int32, device=dev)
        sb = int(plan.route_scratch_bytes)
        scratch = torch.empty((sb,), dtype=torch.uint8, device=dev) if sb > 0 else None
        check(lib().fso_moe_route(ptr(ids), t, topk, num_experts, int(plan.num_blocks), ptr(masked_m), ptr(blk0),
                                  ptr(slot), ptr(blk_expert), ptr(scratch), sb, stream_ptr()), "fso_moe_route")
    return masked_m, blk0, slot, blk_expert


def moe_gather_quant(hidden: torch.Tensor, slot: torch.Tensor, topk: int, hq: torch.Tensor, sh: torch.Tensor):
    t, h = int(hidden.shape[0]), int(hidden.shape[1])
    with on_device(hidden.device):
        check(lib().fso_moe_gather_quant(ptr(hidden), ptr(slot), t, topk, h, int(hq.shape[0]), ptr(hq), ptr(sh),
                                         stream_ptr()), "fso_moe_gather_quant")


def moe_fc1_swiglu(hq, sh, w13, sw13, blk0, blk_expert, dq, sd):
    e, two_i, h = (int(v) for v in w13.shape)
    with on_device(hq.device):
        check(lib().fso_moe_fc1_swiglu(ptr(hq), ptr(sh), ptr(w13), ptr(sw13), ptr(blk0), ptr(blk_expert), e, h,
                                       two_i // 2, int(blk_expert.shape[0]), int(hq.shape[0]), ptr(dq), ptr(sd),
                                       stream_ptr()), "fso_moe_fc1_swiglu")


def moe_fc2(dq, sd, w2, sw2, blk0, blk_expert, dn):
    e, h, inter = (int(v) for v in w2.shape)
    with on_device(dq.device):
        check(lib().fso_moe_fc2(ptr(dq), ptr(sd), ptr(w2), ptr(sw2), ptr(blk0), ptr(blk_expert), e, h, inter,
                                int(blk_expert.shape[0]), int(dq.shape[0]), ptr(dn), stream_ptr()), "fso_moe_fc2")


def moe_grouped_gemm_decode(act_q, act_sf, weight, sfw, masked_m, blk0, blk_expert, out, tokens: int, topk: int):
    """out [rows, n_w] (fp32 or bf16, by its dtype) = the routed rows of act_q [rows, K] times weight [E, n_w, K]^T
    per expert, decode band."""
    e, n_w, k = (int(v) for v in weight.shape)
    with on_device(act_q.device):
        check(lib().fso_moe_grouped_gemm_decode(ptr(act_q), ptr(act_sf), ptr(weight), ptr(sfw), ptr(masked_m), ptr(blk0),
                                                ptr(blk_expert), e, n_w, k, int(blk_expert.shape[0]),
                                                int(act_q.shape[0]), ptr(out), 1 if out.dtype == torch.float32 else 0,
                                                int(tokens), int(topk), stream_ptr()),
              "fso_moe_grouped_gemm_decode")


def moe_silu_mul_quantize_rows(gu, masked_m, blk0, blk_expert, num_experts: int, dq, sd):
    rows, inter = int(dq.shape[0]), int(dq.shape[1])
    with on_device(gu.device):
        check(lib().fso_moe_silu_mul_quantize_rows(ptr(gu), ptr(masked_m), ptr(blk0), ptr(blk_expert), int(num_experts),
                                                   rows, inter, ptr(dq), ptr(sd), stream_ptr()),
              "fso_moe_silu_mul_quantize_rows")


def moe_combine(dn, slot, topk_w, bias, bias_scale, out):
    t, h = int(out.shape[0]), int(out.shape[1])
    topk = int(topk_w.shape[1])
    with on_device(dn.device):
        check(lib().fso_moe_combine(ptr(dn), ptr(slot), ptr(topk_w), ptr(bias), ptr(bias_scale), ptr(out), t, topk, h,
                                    stream_ptr()), "fso_moe_combine")


_LOGIT_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def moe_topk_from_logits(logits, topk: int, renormalize: bool, with_shared_gate: bool, n_valid, expert_map):
    """logits [M, E (+1)] -> (ids int32 [M, topk], weights fp32 [M, topk], shared_gate fp32 [M] or [0])."""
    m, width = int(logits.shape[0]), int(logits.shape[1])
    e = width - (1 if with_shared_gate else 0)
    dev = logits.device
    with on_device(dev):
        ids = torch.empty((m, topk), dtype=torch.int32, device=dev)
        w = torch.empty((m, topk), dtype=torch.float32, device=dev)
        gate = torch.empty((m if with_shared_gate else 0,), dtype=torch.float32, device=dev)
        check(lib().fso_moe_topk_from_logits(ptr(logits), _LOGIT_DTYPES[logits.dtype], m, e, int(logits.stride(0)),
                                             int(topk), 1 if renormalize else 0, ptr(n_valid), ptr(expert_map),
                                             ptr(ids), ptr(w), ptr(gate) if with_shared_gate else None,
                                             stream_ptr()), "fso_moe_topk_from_logits")
    return ids, w, gate


def ep_plan_count(topk_ids: torch.Tensor, experts_per_rank: int, world: int):
    """int32 [T, k] global ids -> (rank_mask int64 [T], row int64 [world + 1] = rows per destination rank, T)."""
    t, k = int(topk_ids.shape[0]), int(topk_ids.shape[1])
    dev = topk_ids.device
    with on_device(dev):
        mask = torch.empty((t,), dtype=torch.int64, device=dev)
        row = torch.empty((world + 1,), dtype=torch.int64, device=dev)
        check(lib().fso_ep_plan_count(ptr(topk_ids), t, k, int(experts_per_rank), int(world), ptr(mask), ptr(row),
                                      stream_ptr()), "fso_ep_plan_count")
    return mask, row


def ep_plan_place(mask: torch.Tensor, table: torch.Tensor, world: int, rank: int, send_total: int):
    """-> (send_token [S], send_rank [S], send_off [G], dst_base [G], recv_off [G + 1], back_base [G], slot [T, G])."""
    t, dev = int(mask.shape[0]), mask.device
    with on_device(dev):
        lists = torch.empty((2, max(send_total, 1)), dtype=torch.int64, device=dev)
        offs = torch.empty((4 * world + 1,), dtype=torch.int64, device=dev)
        slot = torch.empty((t, world), dtype=torch.int32, device=dev)
        send_off, dst_base = offs[:world], offs[world:2 * world]
        back_base, recv_off = offs[2 * world:3 * world], offs[3 * world:]
        check(lib().fso_ep_plan_place(ptr(mask), ptr(table), t, int(world), int(rank), ptr(lists[0]), ptr(lists[1]),
                                      ptr(send_off), ptr(dst_base), ptr(recv_off), ptr(back_base), ptr(slot),
                                      stream_ptr()), "fso_ep_plan_place")
    return lists[0, :send_total], lists[1, :send_total], send_off, dst_base, recv_off, back_base, slot


def ep_dispatch_push(xq, xs, topk_ids, topk_w, send_token, send_rank, send_off, dst_base, peer_q, peer_w, peer_ids,
                     peer_wt, experts_per_rank: int):
    """Store this rank's sent rows into the destination ranks' receive buffers (peer-mapped addresses)."""
    rows, topk, h = int(send_token.shape[0]), int(topk_ids.shape[1]), int(xq.shape[1])
    with on_device(xq.device):
        check(lib().fso_ep_dispatch_push(ptr(xq), ptr(xs), ptr(topk_ids), ptr(topk_w), ptr(send_token), ptr(send_rank),
                                         ptr(send_off), ptr(dst_base), ptr(peer_q), ptr(peer_w), ptr(peer_ids),
                                         ptr(peer_wt), rows, topk, h, int(experts_per_rank), stream_ptr()),
              "fso_ep_dispatch_push")


def moe_gather_rows(rx_q, rx_w, slot, topk: int, hq, sh):
    rows_in, h = int(rx_q.shape[0]), int(rx_q.shape[1])
    with on_device(rx_q.device):
        check(lib().fso_moe_gather_rows(ptr(rx_q), ptr(rx_w), ptr(slot), rows_in, topk, h, int(hq.shape[0]), ptr(hq),
                                        ptr(sh), stream_ptr()), "fso_moe_gather_rows")


def moe_combine_scatter(dn, slot, topk_w, recv_off, back_base, peer_back, world: int):
    tokens, topk, h = int(topk_w.shape[0]), int(topk_w.shape[1]), int(dn.shape[1])
    with on_device(dn.device):
        check(lib().fso_moe_combine_scatter(ptr(dn), ptr(slot), ptr(topk_w), tokens, topk, h, ptr(recv_off),
                                            ptr(back_base), ptr(peer_back), int(world), stream_ptr()),
              "fso_moe_combine_scatter")


def device_status() -> int:
    return _lib.device_status()
