"""Parity of the MoE path through the C ABI: routing offsets and the canonical permutation bit-exact, gathered /
quantized rows bit-exact, grouped GEMMs and the whole layer within tolerance of the fp32 oracle that models both
quantization points."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def _route_both(oracle, ops, ids, e):
    t, k = ids.shape
    plan = ops.moe_plan(t, k, e)
    mm, b0, sl, be = ops.moe_route(ids.cuda(), e, plan)
    omm, ob0, osl, obe = oracle.route(ids, e, int(plan.num_blocks))
    return plan, (mm, b0, sl, be), (omm, ob0, osl, obe)


# (tokens, experts, topk, draw): small single-CTA calls, multi-segment calls, many experts, hot and dead experts
ROUTE_CASES = [(1, 8, 2, "random"), (64, 8, 2, "random"), (512, 8, 2, "skew"), (513, 8, 2, "random"),
               (1024, 64, 4, "random"), (4096, 256, 8, "random"), (3000, 256, 8, "skew"), (2048, 1024, 8, "random"),
               (700, 16, 4, "hot"), (700, 16, 4, "dead"), (100, 8, 2, "ep")]


def _draw(t, e, k, kind, seed):
    if kind == "skew":
        return inputs.routing(t, e, k, seed, skew=1.2)[0]
    ids = inputs.routing(t, e, k, seed)[0]
    if kind == "hot":      # one expert in every token: far more than 128 rows in one expert
        ids[:, 0] = 3
        ids[:, 1:] = torch.where(ids[:, 1:] == 3, torch.full_like(ids[:, 1:], 4), ids[:, 1:])
    elif kind == "dead":   # half of the experts unreachable
        ids = ids // 2
    elif kind == "ep":     # expert-parallel call: non-local ids are -1 / E (skipped)
        ids = torch.where(ids >= e // 2, torch.full_like(ids, -1), ids)
        ids[0, 0] = e
    return ids.contiguous()


@pytest.mark.parametrize("t,e,k,kind", ROUTE_CASES)
def test_routing_bit_exact(fso, oracle, device_ok, t, e, k, kind):
    from fish_scales_ops_b200 import _ops

    ids = _draw(t, e, k, kind, 1000 + t + e)
    _, got, want = _route_both(oracle, _ops, ids, e)
    for g, w, name in zip(got, want, ("masked_m", "blk0", "slot_of_flat", "blk_expert")):
        assert np.array_equal(g.cpu().numpy(), w), name


def test_gather_quant_bit_exact(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    t, e, k, h = 300, 8, 2, 512
    ids = _draw(t, e, k, "ep", 5)
    hidden = inputs.activation(t, h, 6)
    plan, (mm, b0, sl, be), (_, _, osl, _) = _route_both(oracle, _ops, ids, e)
    rows = int(plan.rows)
    hq = torch.zeros((rows, h), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    sh = torch.zeros((rows * h // 128,), dtype=torch.int32, device="cuda")
    _ops.moe_gather_quant(hidden.cuda(), sl, k, hq, sh)
    ohq, osh = oracle.gather_quant(hidden, k, osl, rows)
    assert np.array_equal(inputs.to_np_u8(hq), ohq)
    assert np.array_equal(inputs.to_np_u32(sh), osh)


def test_combine_matches_oracle(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    t, e, k, h = 257, 8, 2, 384
    ids = _draw(t, e, k, "ep", 9)
    w = inputs.routing(t, e, k, 9)[1]
    plan, (_, _, sl, _), (_, _, osl, _) = _route_both(oracle, _ops, ids, e)
    dn = inputs.activation(int(plan.rows), h, 10)
    bias = inputs.activation(t, h, 11)
    bs = torch.rand(t, generator=inputs.gen(12))
    for b, s in ((None, None), (bias, None), (bias, bs)):
        out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
        _ops.moe_combine(dn.cuda(), sl, w.cuda(), None if b is None else b.cuda(), None if s is None else s.cuda(), out)
        want = oracle.combine(dn, osl, w, k, bias=b, bias_scale=s)
        assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def _prepare(fso, e, h, i, seed):
    w13 = inputs.weight(e * 2 * i, h, seed).view(e, 2 * i, h)
    w2 = inputs.weight(e * h, i, seed + 1).view(e, h, i)
    return w13, w2, fso.moe.prepare_experts(w13.cuda(), w2.cuda(), format="mxfp8")


def test_prepare_experts_bytes(fso, oracle, device_ok):
    e, h, i = 3, 256, 128
    w13, w2, ex = _prepare(fso, e, h, i, 40)
    q13, s13 = oracle.quantize_1x32(w13.reshape(e * 2 * i, h), interleave_i=i)
    q2, s2 = oracle.quantize_1x32(w2.reshape(e * h, i))
    assert ex.w13_interleaved and ex.kind == "mxfp8" and (ex.num_experts, ex.hidden, ex.inter) == (e, h, i)
    assert np.array_equal(inputs.to_np_u8(ex.w13).reshape(-1, h), q13)
    assert np.array_equal(inputs.to_np_u32(ex.sw13).reshape(-1), s13)
    assert np.array_equal(inputs.to_np_u8(ex.w2).reshape(-1, i), q2)
    assert np.array_equal(inputs.to_np_u32(ex.sw2).reshape(-1), s2)
    # an MXFP8 checkpoint of the same experts (stored [gate; up], uint8 scales) gives the same handle bytes
    qs, ss = oracle.quantize_1x32(w13.reshape(e * 2 * i, h))
    rows = np.repeat(np.arange(e * 2 * i), h // 128)
    kps = np.tile(np.arange(h // 128), e * 2 * i)
    u13 = ss[oracle.sf_word_index(rows, kps, h)].reshape(e, 2 * i, h // 128).view(np.uint8).reshape(e, 2 * i, h // 32)
    rows2 = np.repeat(np.arange(e * h), i // 128)
    kps2 = np.tile(np.arange(i // 128), e * h)
    u2 = s2[oracle.sf_word_index(rows2, kps2, i)].reshape(e, h, i // 128).view(np.uint8).reshape(e, h, i // 32)
    ck = fso.moe.prepare_experts(torch.from_numpy(qs.reshape(e, 2 * i, h)).cuda().view(torch.float8_e4m3fn),
                                 torch.from_numpy(q2.reshape(e, h, i)).cuda().view(torch.float8_e4m3fn), format="mxfp8",
                                 sw13=torch.from_numpy(u13.copy()).cuda(), sw2=torch.from_numpy(u2.copy()).cuda())
    assert torch.equal(ck.w13.view(torch.uint8), ex.w13.view(torch.uint8)) and torch.equal(ck.sw13, ex.sw13)
    assert torch.equal(ck.w2.view(torch.uint8), ex.w2.view(torch.uint8)) and torch.equal(ck.sw2, ex.sw2)


# (tokens, experts, topk, H, I, draw)
LAYER_CASES = [(1, 8, 2, 256, 128, "random"), (64, 8, 2, 512, 256, "random"), (300, 8, 2, 512, 384, "skew"),
               (257, 16, 4, 256, 256, "hot"), (200, 16, 4, 384, 128, "dead"), (128, 8, 2, 256, 256, "ep"),
               (1500, 32, 8, 256, 128, "random")]


@pytest.mark.parametrize("t,e,k,h,i,kind", LAYER_CASES)
def test_layer_matches_oracle(fso, oracle, device_ok, t, e, k, h, i, kind):
    w13, w2, ex = _prepare(fso, e, h, i, 50 + t)
    ids = _draw(t, e, k, kind, 60 + t)
    wts = inputs.routing(t, e, k, 60 + t)[1]
    hidden = inputs.activation(t, h, 70 + t)
    out = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (t, h)
    ref = oracle.moe_layer(hidden, inputs.to_np_u8(ex.w13), inputs.to_np_u32(ex.sw13), inputs.to_np_u8(ex.w2),
                           inputs.to_np_u32(ex.sw2), ids, wts, interleaved=True)
    inputs.assert_close_to_oracle(out, ref, f"layer T={t} E={e} k={k} {kind}")
    # against the bf16 masters (exact silu): the reference's own layer gate is cos >= 0.997
    full = torch.zeros(t, h)
    for g in range(e):
        tok, slot = np.nonzero(ids.numpy() == g)
        if tok.size == 0:
            continue
        a = hidden[tok].float() @ w13[g].float().t()
        hh = torch.nn.functional.silu(a[:, :i]) * a[:, i:]
        full.index_add_(0, torch.from_numpy(tok), (hh @ w2[g].float().t()) * wts[tok, slot][:, None])
    if full.abs().max() > 0:
        cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), full.flatten(), dim=0)
        assert cos > 0.997


def test_layer_intermediate_and_bias(fso, oracle, device_ok):
    """The fused FC1 output against the oracle's quantized intermediate, then bias / bias_scale."""
    from fish_scales_ops_b200 import _ops

    t, e, k, h, i = 200, 8, 2, 256, 256
    w13, w2, ex = _prepare(fso, e, h, i, 90)
    ids = _draw(t, e, k, "random", 91)
    wts = inputs.routing(t, e, k, 91)[1]
    hidden = inputs.activation(t, h, 92)
    plan = _ops.moe_plan(t, k, e)
    mm, b0, sl, be = _ops.moe_route(ids.cuda(), e, plan)
    rows = int(plan.rows)
    hq = torch.zeros((rows, h), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    sh = torch.zeros((rows * h // 128,), dtype=torch.int32, device="cuda")
    dq = torch.zeros((rows, i), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    sd = torch.zeros((rows * i // 128,), dtype=torch.int32, device="cuda")
    _ops.moe_gather_quant(hidden.cuda(), sl, k, hq, sh)
    _ops.moe_fc1_swiglu(hq, sh, ex.w13, ex.sw13, b0, be, dq, sd)
    live = np.zeros(rows, np.uint8)
    slots = sl.cpu().numpy()
    live[slots[slots >= 0]] = 1
    hd = torch.from_numpy(oracle.dequant(inputs.to_np_u8(hq), inputs.to_np_u32(sh)))
    acc = torch.zeros(rows, 2 * i)
    blk_e = be.cpu().numpy()
    for b in range(int(b0[-1].item())):
        wd = torch.from_numpy(oracle.dequant(inputs.to_np_u8(ex.w13[blk_e[b]]), inputs.to_np_u32(ex.sw13[blk_e[b]])))
        acc[128 * b:128 * b + 128] = hd[128 * b:128 * b + 128] @ wd.t()
    odq, osd = oracle.swiglu_quant(acc.numpy(), live)
    got = torch.from_numpy(oracle.dequant(inputs.to_np_u8(dq), inputs.to_np_u32(sd)))[live.astype(bool)]
    want = torch.from_numpy(oracle.dequant(odq, osd))[live.astype(bool)]
    assert inputs.rel_frobenius(got, want) <= 2e-2
    same = (inputs.to_np_u8(dq)[live.astype(bool)] == odq[live.astype(bool)]).mean()
    assert same > 0.97, same
    bias = inputs.activation(t, h, 93)
    bs = torch.rand(t, generator=inputs.gen(94))
    base = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    with_b = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda(), bias=bias.cuda(), bias_scale=bs.cuda())
    delta = (with_b.float() - base.float()).cpu() - bs[:, None] * bias.float()
    assert delta.abs().max() <= 0.05 * (bs[:, None] * bias.float()).abs().max()


def test_layer_all_skipped_and_empty(fso, device_ok):
    e, h, i = 8, 256, 128
    _, _, ex = _prepare(fso, e, h, i, 3)
    hidden = inputs.activation(10, h, 4).cuda()
    ids = torch.full((10, 2), -1, dtype=torch.int64, device="cuda")
    wts = torch.full((10, 2), 0.5, device="cuda", dtype=torch.bfloat16)
    assert not fso.moe.layer(hidden, ex, ids, wts).any()
    assert tuple(fso.moe.layer(hidden[:0], ex, ids[:0], wts[:0]).shape) == (0, h)
    with pytest.raises(TypeError):
        fso.moe.layer(hidden, ex.w13, ids, wts)
    with pytest.raises(ValueError):
        fso.moe.layer(hidden[:, :128], ex, ids, wts)
    with pytest.raises(ValueError):
        fso.moe.layer(hidden, ex, ids[:5], wts)
    with pytest.raises(ValueError):
        fso.moe.layer(hidden, ex, ids, wts, bias_scale=torch.ones(10, device="cuda"))


def test_transient_bytes_bounds_the_allocation(fso, device_ok):
    """measured <= reserved <= measured + 12 MiB + 1 % (tests/gemm/unit/test_moe_transient_bytes.py:8-12)."""
    e, h, i, k = 8, 512, 256, 2
    _, _, ex = _prepare(fso, e, h, i, 7)
    for t in (1, 64, 1024):
        hidden = inputs.activation(t, h, 8).cuda()
        ids, wts = inputs.routing(t, e, k, 9)
        ids, wts = ids.cuda(), wts.cuda()
        fso.moe.layer(hidden, ex, ids, wts)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        before = torch.cuda.memory_allocated()
        out = fso.moe.layer(hidden, ex, ids, wts)
        torch.cuda.synchronize()
        measured = torch.cuda.max_memory_allocated() - before
        reserved = fso.moe.transient_bytes(ex, t, k)
        assert measured <= reserved <= measured + 12 * 2 ** 20 + measured // 100, (t, measured, reserved)
        del out


def test_layer_graph_replay_with_rewritten_routing(fso, device_ok):
    e, h, i, k, t = 8, 256, 256, 2, 96
    _, _, ex = _prepare(fso, e, h, i, 17)
    hidden = inputs.activation(t, h, 18).cuda()
    ids, wts = inputs.routing(t, e, k, 19)
    ids, wts = ids.cuda(), wts.cuda()
    eager = fso.moe.layer(hidden, ex, ids, wts)
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        fso.moe.layer(hidden, ex, ids, wts)
        with torch.cuda.graph(graph, stream=stream):
            out = fso.moe.layer(hidden, ex, ids, wts)
    torch.cuda.current_stream().wait_stream(stream)
    out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    ids2, wts2 = inputs.routing(t, e, k, 20, skew=1.2)
    ids.copy_(ids2.cuda())
    wts.copy_(wts2.cuda())
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, fso.moe.layer(hidden, ex, ids, wts))


# ------------------------------------------------------------------------------------------------ the decode band

# (tokens, experts, topk, H, I, draw): at most 64 tokens -> the swapped grouped GEMMs. "dup" names one expert twice in
# a token, so an expert holds more rows than there are tokens (a second token sub-tile of its block, and with 64
# tokens a second 128-row block of the expert); "hot" fills one expert's block to the token count.
DECODE_CASES = [(1, 8, 2, 512, 256, "random"), (7, 8, 2, 256, 384, "random"), (16, 16, 4, 512, 256, "skew"),
                (33, 8, 2, 256, 256, "hot"), (64, 8, 2, 512, 512, "random"), (64, 16, 4, 256, 128, "hot"),
                (40, 8, 2, 256, 256, "dup"), (64, 8, 4, 256, 128, "dup"), (48, 8, 2, 256, 256, "ep"),
                (64, 256, 8, 256, 128, "random"), (2, 8, 2, 1024, 3584, "random")]


@pytest.mark.parametrize("t,e,k,h,i,kind", DECODE_CASES)
def test_decode_band_matches_oracle_and_prefill_route(fso, oracle, device_ok, t, e, k, h, i, kind, monkeypatch):
    w13, w2, ex = _prepare(fso, e, h, i, 150 + t)
    ids = _draw(t, e, k, "random" if kind == "dup" else kind, 160 + t)
    if kind == "dup":
        ids[:, 1] = ids[:, 0]                  # the same expert twice: 2 rows of that expert per token
        if k > 2:
            ids[:, 3] = ids[:, 0]
    wts = inputs.routing(t, e, k, 160 + t)[1]
    hidden = inputs.activation(t, h, 170 + t)
    monkeypatch.setenv("FSO_B200_MOE_DECODE", "force")
    out = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    ref = oracle.moe_layer(hidden, inputs.to_np_u8(ex.w13), inputs.to_np_u32(ex.sw13), inputs.to_np_u8(ex.w2),
                           inputs.to_np_u32(ex.sw2), ids, wts, interleaved=True)
    inputs.assert_close_to_oracle(out, ref, f"decode band T={t} E={e} k={k} {kind}")
    # the prefill kernels on the same call: same result up to the output tolerance
    monkeypatch.setenv("FSO_B200_MOE_DECODE", "0")
    pre = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    inputs.assert_close_to_oracle(pre, ref, f"prefill route T={t}")
    assert inputs.rel_frobenius(out.float().cpu(), pre.float().cpu()) <= 1e-2
    # the route the layer picks by itself (either GEMM may take the band) agrees as well
    monkeypatch.delenv("FSO_B200_MOE_DECODE")
    auto = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    inputs.assert_close_to_oracle(auto, ref, f"default route T={t}")
    # bias and bias_scale ride the same combine
    monkeypatch.setenv("FSO_B200_MOE_DECODE", "force")
    bias = inputs.activation(t, h, 180 + t)
    bs = torch.rand(t, generator=inputs.gen(181))
    with_b = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda(), bias=bias.cuda(), bias_scale=bs.cuda())
    ref_b = ref + bs[:, None] * bias.float()
    inputs.assert_close_to_oracle(with_b, ref_b, f"decode band with bias T={t}")
    # run to run identical
    again = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    assert torch.equal(again, out)


def test_decode_band_graph_replay_with_rewritten_routing(fso, device_ok, monkeypatch):
    monkeypatch.setenv("FSO_B200_MOE_DECODE", "force")
    e, h, i, k, t = 16, 512, 256, 4, 24
    _, _, ex = _prepare(fso, e, h, i, 27)
    hidden = inputs.activation(t, h, 28).cuda()
    ids, wts = inputs.routing(t, e, k, 29)
    ids, wts = ids.cuda(), wts.cuda()
    eager = fso.moe.layer(hidden, ex, ids, wts)
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        fso.moe.layer(hidden, ex, ids, wts)
        with torch.cuda.graph(graph, stream=stream):
            out = fso.moe.layer(hidden, ex, ids, wts)
    torch.cuda.current_stream().wait_stream(stream)
    out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    for seed, skew in ((30, 1.2), (31, 0.0)):
        ids2, wts2 = inputs.routing(t, e, k, seed, skew=skew)
        ids.copy_(ids2.cuda())
        wts.copy_(wts2.cuda())
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, fso.moe.layer(hidden, ex, ids, wts))


# ------------------------------------------------------------------------------------------ shared expert overlap

def _shared_weights(fso, h, inter, seed):
    from fish_scales_ops_b200 import compat

    g = torch.Generator().manual_seed(seed)
    w_gu = (0.02 * torch.randn(2 * inter, h, generator=g)).to(torch.bfloat16)
    w_dn = (0.02 * torch.randn(h, inter, generator=g)).to(torch.bfloat16)
    return compat.prepare_gate_up(w_gu.cuda()), fso.dense.prepare_weight(w_dn.cuda(), format="mxfp8")


@pytest.mark.parametrize("t", [5, 200])
def test_shared_expert_joined_before_the_combine(fso, device_ok, t):
    """The shared expert on a side stream, joined right before the combine that adds it: the bytes of the sequential
    form and of fso.moe.layer fed the same bias (python/fish_scales_ops/gemm/mxfp8.py:2578-2611: the join is a stream
    dependency, not a change of arithmetic). Covers the decode band (5 tokens) and the prefill route."""
    from fish_scales_ops_b200 import compat

    e, h, i, k = 8, 256, 256, 2
    _, _, ex = _prepare(fso, e, h, i, 31)
    gate_up, down = _shared_weights(fso, h, 384, 32)
    hidden = inputs.activation(t, h, 33).cuda()
    ids, wts = inputs.routing(t, e, k, 34)
    ids, wts = ids.cuda(), wts.cuda()
    gate = torch.sigmoid(torch.randn(t, generator=torch.Generator().manual_seed(35))).cuda()
    bias = compat.shared_expert(hidden, gate_up, down)
    want = fso.moe.layer(hidden, ex, ids, wts, bias=bias, bias_scale=gate)
    seq = compat.moe_layer_shared(hidden, ex, ids, wts, gate_up=gate_up, down=down, shared_gate=gate, overlap=False)
    ovl = compat.moe_layer_shared(hidden, ex, ids, wts, gate_up=gate_up, down=down, shared_gate=gate, overlap=True)
    torch.cuda.synchronize()
    assert torch.equal(seq, want) and torch.equal(ovl, want)
    # and inside a captured graph (the side stream exists by now): two branches, joined before the combine
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            out = compat.moe_layer_shared(hidden, ex, ids, wts, gate_up=gate_up, down=down, shared_gate=gate)
    torch.cuda.current_stream().wait_stream(stream)
    out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
