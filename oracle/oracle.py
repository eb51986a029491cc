"""TEST INFRASTRUCTURE ONLY: Python face of the CPU parity checker.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs import this module; the product
package never does (it fails loudly when its CUDA library is missing instead of falling back to anything here).

``libmxfp8_oracle.so`` (built from ``mxfp8_oracle.c`` by the Makefile beside this file) holds the byte-producing
restatements; ``_ref/libfso_ref_contract.so`` is the reference's own quantizer header compiled on the host and is
used to pin them. The dense and MoE *output* oracles are fp32 dequantize-then-matmul forms (the reference's own
test references: tests/gemm/unit/test_prequant_mxfp8.py:178-183, tests/gemm/unit/test_mxfp8_grouped.py:313-345,
tests/gemm/unit/test_moe_unified.py:170-189) and are tolerance oracles: the reference holds no golden output
vectors for them, so that part of the parity is unpinned.
"""
import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_i64 = ctypes.c_int64
_p = ctypes.c_void_p


def build():
    """Compile the checker (and, where the reference tree is present, the reference-header shim). The reference tree
    is the one FSO_REFERENCE_ROOT names, else a directory called ``reference`` beside this repository."""
    env = dict(os.environ)
    if not env.get("FSO_REFERENCE_ROOT"):
        beside = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
        if os.path.isdir(beside):
            env["FSO_REFERENCE_ROOT"] = beside
    subprocess.run(["make", "-C", _HERE, "-s"], check=True, stdout=subprocess.DEVNULL, env=env)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libmxfp8_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_e4m3_to_float.restype = ctypes.c_float
        _LIB.orc_e4m3_to_float.argtypes = [ctypes.c_uint8]
        _LIB.orc_e4m3_from_float.restype = ctypes.c_uint8
        _LIB.orc_e4m3_from_float.argtypes = [ctypes.c_float]
        _LIB.orc_bf16_from_float.restype = ctypes.c_uint16
        _LIB.orc_bf16_from_float.argtypes = [ctypes.c_float]
        for name in ("orc_e8m0_from_amax", "orc_e8m0_from_amax_int"):
            f = getattr(_LIB, name)
            f.restype = ctypes.c_uint8
            f.argtypes = [ctypes.c_float, ctypes.POINTER(ctypes.c_float)]
        _LIB.orc_sf_word_index.restype = _i64
        _LIB.orc_sf_word_index.argtypes = [_i64, _i64, _i64]
    return _LIB


def ref_lib():
    """The reference-header shim, or None where it was never built (its absence only skips the pin tests)."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libfso_ref_contract.so")
        if not os.path.exists(path):
            return None
        _REF = ctypes.CDLL(path)
        _REF.ref_e8m0_from_amax.restype = ctypes.c_uint32
        _REF.ref_e8m0_from_amax.argtypes = [ctypes.c_float, ctypes.POINTER(ctypes.c_uint32)]
        _REF.ref_e4m3_from_float.restype = ctypes.c_uint32
        _REF.ref_e4m3_from_float.argtypes = [ctypes.c_float]
        _REF.ref_sf_word_index_sm100.restype = _i64
        _REF.ref_sf_word_index_sm100.argtypes = [_i64, _i64, _i64]
    return _REF


# ------------------------------------------------------------------------------------------------ array helpers

def bf16_bits(t) -> np.ndarray:
    """uint16 bit patterns of a bf16 torch tensor (or pass-through for a uint16 array)."""
    if isinstance(t, np.ndarray):
        assert t.dtype == np.uint16
        return np.ascontiguousarray(t)
    assert t.dtype == torch.bfloat16
    return np.ascontiguousarray(t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def fp8_bytes(t) -> np.ndarray:
    if isinstance(t, np.ndarray):
        assert t.dtype == np.uint8
        return np.ascontiguousarray(t)
    return np.ascontiguousarray(t.detach().cpu().contiguous().view(torch.uint8).numpy())


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_p)


def sf_words(m: int, k: int) -> int:
    return (m + 127) // 128 * 128 * (k // 128)


def sf_word_index(rows: np.ndarray, kp: np.ndarray, k: int) -> np.ndarray:
    """Vectorised atom-layout index of word (row, kp) of an [*, k] tensor."""
    r = rows % 128
    return ((rows // 128) * (k // 128) + kp) * 128 + (r % 32) * 4 + r // 32


# ------------------------------------------------------------------------------------------------ byte producers

def quantize_1x32(x, interleave_i: int = 0):
    """bf16 [M, K] -> (uint8 e4m3 [M, K], uint32 words [align(M,128)*K/128])."""
    xb = bf16_bits(x)
    m, k = xb.shape
    q = np.empty((m, k), np.uint8)
    sf = np.empty(sf_words(m, k), np.uint32)
    lib().orc_quantize_1x32(_ptr(xb), _i64(m), _i64(k), _i64(interleave_i), _ptr(q), _ptr(sf))
    return q, sf


def ref_quantize_1x32(x):
    """The same through the reference's header (None when the shim is not built)."""
    r = ref_lib()
    if r is None:
        return None
    xb = bf16_bits(x)
    m, k = xb.shape
    q = np.empty((m, k), np.uint8)
    sf = np.empty(sf_words(m, k), np.uint32)
    r.ref_quantize_1x32_sm100(_ptr(xb), _i64(m), _i64(k), _ptr(q), _ptr(sf))
    return q, sf


def requant_bs128(wq, scale, interleave_i: int = 0):
    """Block-FP8 checkpoint (e4m3 [N, K], fp32 [N/128, K/128]) -> MXFP8 bytes and words."""
    wb = fp8_bytes(wq)
    s = np.ascontiguousarray(scale.detach().cpu().numpy() if isinstance(scale, torch.Tensor) else scale, np.float32)
    n, k = wb.shape
    q = np.empty((n, k), np.uint8)
    sf = np.empty(sf_words(n, k), np.uint32)
    lib().orc_requant_bs128(_ptr(wb), _ptr(s), _i64(n), _i64(k), _i64(interleave_i), _ptr(q), _ptr(sf))
    return q, sf


def pack_ue8m0(s_u8, interleave_i: int = 0):
    """uint8 [G, N, K/32] -> uint32 [G, align(N,128)*K/128] atom slabs."""
    s = np.ascontiguousarray(s_u8.detach().cpu().numpy() if isinstance(s_u8, torch.Tensor) else s_u8, np.uint8)
    g, n, k32 = s.shape
    k = k32 * 32
    out = np.empty((g, sf_words(n, k)), np.uint32)
    lib().orc_pack_ue8m0(_ptr(s), _i64(g), _i64(n), _i64(k), _i64(interleave_i), _ptr(out))
    return out


def dequant(q, sf) -> np.ndarray:
    """(e4m3 bytes [M, K], atom words) -> fp32 [M, K]."""
    qb = fp8_bytes(q)
    s = np.ascontiguousarray(sf.detach().cpu().numpy().view(np.uint32) if isinstance(sf, torch.Tensor) else sf,
                             np.uint32)
    m, k = qb.shape
    out = np.empty((m, k), np.float32)
    lib().orc_dequant(_ptr(qb), _ptr(s), _i64(m), _i64(k), _ptr(out))
    return out


def route(ids, num_experts: int, num_blocks: int):
    """ids int32 [T, topk] -> (masked_m [E], blk0 [E+1], slot_of_flat [T*topk], blk_expert [num_blocks])."""
    a = np.ascontiguousarray(ids.detach().cpu().numpy() if isinstance(ids, torch.Tensor) else ids, np.int32).reshape(-1)
    mm = np.empty(num_experts, np.int32)
    b0 = np.empty(num_experts + 1, np.int32)
    sl = np.empty(a.size, np.int32)
    be = np.empty(num_blocks, np.int32)
    lib().orc_route(_ptr(a), _i64(a.size), _i64(num_experts), _i64(num_blocks), _ptr(mm), _ptr(b0), _ptr(sl), _ptr(be))
    return mm, b0, sl, be


def gather_quant(hidden, topk: int, slot_of_flat: np.ndarray, rows: int):
    hb = bf16_bits(hidden)
    t, h = hb.shape
    hq = np.zeros((rows, h), np.uint8)
    sh = np.zeros(sf_words(rows, h), np.uint32)
    sl = np.ascontiguousarray(slot_of_flat, np.int32)
    lib().orc_gather_quant(_ptr(hb), _i64(t), _i64(topk), _i64(h), _ptr(sl), _ptr(hq), _ptr(sh))
    return hq, sh


def swiglu_quant(acc: np.ndarray, live: np.ndarray):
    """fp32 [rows, 2I] interleaved gate/up accumulators -> (e4m3 [rows, I], words); exact silu."""
    acc = np.ascontiguousarray(acc, np.float32)
    rows, two_i = acc.shape
    inter = two_i // 2
    dq = np.zeros((rows, inter), np.uint8)
    sd = np.zeros(sf_words(rows, inter), np.uint32)
    lv = np.ascontiguousarray(live, np.uint8)
    lib().orc_swiglu_quant(_ptr(acc), _i64(rows), _i64(inter), _ptr(lv), _ptr(dq), _ptr(sd))
    return dq, sd


def combine(dn, slot_of_flat, w, topk: int, bias=None, bias_scale=None) -> torch.Tensor:
    db = bf16_bits(dn)
    h = db.shape[1]
    sl = np.ascontiguousarray(slot_of_flat, np.int32)
    wf = np.ascontiguousarray(w.detach().cpu().numpy() if isinstance(w, torch.Tensor) else w, np.float32).reshape(-1)
    t = sl.size // topk
    out = np.empty((t, h), np.uint16)
    bb = bf16_bits(bias) if bias is not None else None
    bs = None
    if bias_scale is not None:
        bs = np.ascontiguousarray(bias_scale.detach().cpu().numpy() if isinstance(bias_scale, torch.Tensor)
                                  else bias_scale, np.float32)
    lib().orc_combine(_ptr(db), _ptr(sl), _ptr(wf), _ptr(bb) if bb is not None else None,
                      _ptr(bs) if bs is not None else None, _i64(t), _i64(topk), _i64(h), _ptr(out))
    return bf16_from_bits(out)


# ------------------------------------------------------------------------------------------------ output oracles

def dense_linear(x, w_q, w_sf) -> torch.Tensor:
    """fp32 result of the dense path on the quantized operands: dequant(quantize(x)) @ dequant(w)^T.
    x bf16 [M, K]; w_q / w_sf the prepared weight bytes and words. Returns fp32 [M, N] (not rounded)."""
    xq, xs = quantize_1x32(x)
    xd = torch.from_numpy(dequant(xq, xs))
    wd = torch.from_numpy(dequant(w_q, w_sf))
    return xd @ wd.t()


def dense_epilogue(acc: torch.Tensor, bias=None, residual=None, activation=None) -> torch.Tensor:
    """The dense epilogue on an fp32 accumulator (csrc/gemm/include/blockscale_gemm/common/epilogue.cuh:1-30 of the
    reference): v = acc + bias[n] (a +0.0 bias counts as -0.0); v = erf-GELU(v) = 0.5 v (1 + erf(v * fp32(1/sqrt 2)))
    when asked; v += residual[m, n]. fp32 throughout, not rounded (the caller compares within the output tolerance)."""
    v = acc.to(torch.float32).clone()
    if bias is not None:
        b = bias.detach().cpu().to(torch.float32)
        b = torch.where(b == 0, torch.full_like(b, -0.0), b)
        v = v + b
    if activation == "gelu_erf":
        v = 0.5 * v * (1.0 + torch.erf(v * np.float32(0.70710678118654752440)))
    elif activation is not None:
        raise ValueError(activation)
    if residual is not None:
        v = v + residual.detach().cpu().to(torch.float32)
    return v


def moe_layer(hidden, w13_q, w13_sf, w2_q, w2_sf, topk_ids, topk_w, interleaved: bool = True) -> torch.Tensor:
    """fp32 MoE layer on quantized operands, modelling both quantization points (the gathered activation and the
    fp32 silu(gate)*up intermediate requantized with the 1x32 rule before FC2); ids outside [0, E) are skipped.
    w13_q uint8 [E, 2I, H] (rows interleaved gate/up when ``interleaved``), w13_sf uint32 [E, 2I*H/128], etc."""
    hb = hidden.detach().cpu()
    t, h = hb.shape
    e, two_i, _ = w13_q.shape
    inter = two_i // 2
    ids = np.asarray(topk_ids.detach().cpu().numpy() if isinstance(topk_ids, torch.Tensor) else topk_ids)
    wts = np.asarray(topk_w.detach().cpu().numpy() if isinstance(topk_w, torch.Tensor) else topk_w, np.float32)
    xq, xs = quantize_1x32(hb)
    xd = torch.from_numpy(dequant(xq, xs))
    out = torch.zeros(t, h, dtype=torch.float32)
    for g in range(e):
        tok, slot = np.nonzero(ids == g)
        if tok.size == 0:
            continue
        w13d = torch.from_numpy(dequant(w13_q[g], w13_sf[g]))
        w2d = torch.from_numpy(dequant(w2_q[g], w2_sf[g]))
        acc = xd[tok] @ w13d.t()
        if not interleaved:
            acc = torch.stack([acc[:, :inter], acc[:, inter:]], dim=2).reshape(tok.size, two_i)
        dq, sd = swiglu_quant(acc.numpy(), np.ones(tok.size, np.uint8))
        dd = torch.from_numpy(dequant(dq, sd))
        dn = (dd @ w2d.t()).to(torch.bfloat16).to(torch.float32)
        out.index_add_(0, torch.from_numpy(tok), dn * torch.from_numpy(wts[tok, slot])[:, None])
    return out


# ------------------------------------------------------------------------------------------------------- router

def router_topk(logits, topk: int, renormalize: bool = True, with_shared_gate: bool = False, n_valid=None,
                expert_map=None):
    """CPU statement of the router (csrc/gemm/ops/moe_glue.cu:1253-1465 of the reference): per token, k picks of the
    largest remaining logit (ties to the lower expert id), weights exp(l - max) over the selected experts, summed in
    pick order in fp32, divided by that sum (``renormalize``) or by the fp32 sum of exp(l - max) over all experts;
    rows at or past ``n_valid`` get the sentinel id E and weight 0; ``expert_map`` [E + 1] is applied to every id;
    the shared gate is sigmoid of logit column E. ``logits``: torch tensor [M, E (+1)] of bf16 / fp16 / fp32.
    Returns (ids int32 [M, k], weights fp32 [M, k], gate fp32 [M] or [0]). Ids are exact; the weights depend on the
    exp implementation and are a tolerance oracle (1e-5 relative in the reference's own test,
    tests/gemm/unit/test_moe_router_topk.py:20-25)."""
    lg = logits.detach().cpu().to(torch.float32).numpy()
    m, width = lg.shape
    e = width - (1 if with_shared_gate else 0)
    ids = np.zeros((m, topk), np.int32)
    w = np.zeros((m, topk), np.float32)
    gate = np.zeros((m if with_shared_gate else 0,), np.float32)
    emap = None if expert_map is None else np.asarray(
        expert_map.detach().cpu().numpy() if isinstance(expert_map, torch.Tensor) else expert_map, np.int32)
    for t in range(m):
        if with_shared_gate:
            gate[t] = np.float32(1.0) / (np.float32(1.0) + np.exp(-lg[t, e], dtype=np.float32))
        if n_valid is not None and t >= int(n_valid):
            ids[t, :] = e if emap is None else emap[e]
            continue
        row = lg[t, :e]
        # stable sort of -logit: descending value, ascending id among equals
        order = np.argsort(-row, kind="stable")[:topk]
        sel = row[order]
        ex = np.exp(sel - sel[0], dtype=np.float32)
        denom = np.float32(0.0)
        for j in range(topk):
            denom = np.float32(denom + ex[j])
        if not renormalize:
            denom = np.exp(row - sel[0], dtype=np.float32).sum(dtype=np.float32)
        w[t] = ex * (np.float32(1.0) / denom)
        ids[t] = order if emap is None else emap[order]
    return ids, w, gate
