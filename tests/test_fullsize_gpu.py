"""Parity at the benchmarked sizes: the Mixtral and DeepSeek-V3 MoE layers and the DeepSeek-V3 block-FP8 checkpoints
(BASELINE.json configs 3-5) at their real H / I / E, checked against the CPU oracle on a sample that the oracle
finishes in seconds: a few tokens of the layer's output (rows of a layer are independent), sampled 128-row blocks of
a requantized checkpoint (blocks are independent), sampled output columns of a linear."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu

FP8 = torch.float8_e4m3fn


def _experts_on_device(e: int, h: int, i: int, seed: int):
    """bf16 ~ N(0, 0.02) experts generated on the device, expert by expert (seeded per expert)."""
    w13 = torch.empty((e, 2 * i, h), dtype=torch.bfloat16, device="cuda")
    w2 = torch.empty((e, h, i), dtype=torch.bfloat16, device="cuda")
    for j in range(e):
        g = torch.Generator(device="cuda").manual_seed(seed + j)
        w13[j] = (0.02 * torch.randn(2 * i, h, generator=g, device="cuda")).to(torch.bfloat16)
        w2[j] = (0.02 * torch.randn(h, i, generator=g, device="cuda")).to(torch.bfloat16)
    return w13, w2


def _oracle_rows(oracle, ex, hidden, ids, wts, rows):
    """The oracle's layer output for the token rows ``rows``, from the handle's own bytes of the experts those
    tokens touch (the handle's bytes are pinned against the oracle's quantizer separately)."""
    ids_s = ids[rows]
    used = sorted({int(v) for v in ids_s.reshape(-1).tolist() if 0 <= int(v) < ex.num_experts})
    remap = {g: j for j, g in enumerate(used)}
    ids_l = torch.tensor([[remap.get(int(v), -1) for v in row] for row in ids_s.tolist()], dtype=torch.int32)
    sel = torch.tensor(used, device="cuda")
    q13 = inputs.to_np_u8(ex.w13.index_select(0, sel))
    s13 = inputs.to_np_u32(ex.sw13.index_select(0, sel))
    q2 = inputs.to_np_u8(ex.w2.index_select(0, sel))
    s2 = inputs.to_np_u32(ex.sw2.index_select(0, sel))
    return oracle.moe_layer(hidden[rows], q13, s13, q2, s2, ids_l, wts[rows], interleaved=True)


# (name, E, k, H, I, tokens, skew, renormalise, sampled tokens)
FULL_LAYERS = [("mixtral-uniform", 8, 2, 4096, 14336, 64, 0.0, True, 6),
               ("mixtral-zipf", 8, 2, 4096, 14336, 64, 1.2, True, 6),
               ("dsv3", 256, 8, 7168, 2048, 64, 0.0, False, 4)]

_EXPERTS = {}


def _prepared(fso, e, h, i):
    key = (e, h, i)
    if key not in _EXPERTS:
        _EXPERTS.clear()                      # one configuration's weights on the device at a time
        torch.cuda.empty_cache()
        w13, w2 = _experts_on_device(e, h, i, 7000)
        slab = (w13[e - 1, :256].cpu(), w2[0, 128:256].cpu())
        ex = fso.moe.prepare_experts(w13, w2, format="mxfp8")
        del w13, w2
        torch.cuda.empty_cache()
        _EXPERTS[key] = (ex, slab)
    return _EXPERTS[key]


@pytest.mark.parametrize("name,e,k,h,i,t,skew,renorm,sample", FULL_LAYERS, ids=[c[0] for c in FULL_LAYERS])
def test_full_size_layer_matches_oracle(fso, oracle, device_ok, name, e, k, h, i, t, skew, renorm, sample):
    ex, (slab13, slab2) = _prepared(fso, e, h, i)
    # the handle's bytes at this shape: rows [0, 256) of the last expert's gate rows (interleaved into rows 0, 2, 4..
    # of the handle) and one 128-row block of the first expert's down projection
    q, s = oracle.quantize_1x32(slab13)
    got13 = inputs.to_np_u8(ex.w13[e - 1, 0:512:2])
    assert np.array_equal(got13, q), "w13 codes of the sampled gate rows"
    q2, s2 = oracle.quantize_1x32(slab2)
    assert np.array_equal(inputs.to_np_u8(ex.w2[0, 128:256]), q2), "w2 codes of the sampled block"
    kb2 = i // 128
    assert np.array_equal(inputs.to_np_u32(ex.sw2[0])[kb2 * 128:2 * kb2 * 128], s2), "w2 scale words of the sampled block"

    ids, wts = inputs.routing(t, e, k, 8100 + len(name), skew=skew, renorm=renorm)
    hidden = inputs.activation(t, h, 8200 + len(name))
    out = fso.moe.layer(hidden.cuda(), ex, ids.cuda(), wts.cuda())
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (t, h)
    rows = torch.arange(0, t, max(1, t // sample))[:sample]
    ref = _oracle_rows(oracle, ex, hidden, ids, wts, rows)
    inputs.assert_close_to_oracle(out[rows.cuda()], ref, f"{name} layer, tokens {rows.tolist()} of {t}")


# BASELINE.json configs[2]: DeepSeek-V3 dense shapes stored as block-FP8 (one fp32 scale per 128 x 128 tile)
BSFP8_SHAPES = [(7168, 2048), (2048, 7168), (24576, 7168)]


@pytest.mark.parametrize("n,k", BSFP8_SHAPES)
def test_block_fp8_checkpoint_requant_and_linear(fso, oracle, device_ok, n, k):
    wq, s = inputs.block_fp8_checkpoint(n, k, 300 + n // 128)
    weight = fso.dense.prepare_weight(wq.cuda(), format="bsfp8", scale=s.cuda())
    assert weight.kind == "mxfp8" and weight.weight.dtype == FP8 and tuple(weight.weight.shape) == (n, k)
    kb = k // 128
    blocks = sorted({0, 1, n // 256, n // 128 - 1})
    got_q = inputs.to_np_u8(weight.weight)
    got_s = inputs.to_np_u32(weight.scale)
    for b in blocks:                       # 128-row blocks are independent: bit-exact against the oracle, block by block
        oq, osf = oracle.requant_bs128(wq[b * 128:(b + 1) * 128], s[b:b + 1])
        assert np.array_equal(got_q[b * 128:(b + 1) * 128], oq), f"codes of block {b}"
        assert np.array_equal(got_s[b * kb * 128:(b + 1) * kb * 128], osf), f"scale words of block {b}"
    # the linear on this weight, on the output columns of the sampled blocks
    cols = np.concatenate([np.arange(b * 128, (b + 1) * 128) for b in blocks])
    wq_s = got_q[cols]
    ws_s = np.concatenate([got_s[b * kb * 128:(b + 1) * kb * 128] for b in blocks])
    for m in (16, 512):
        x = inputs.activation(m, k, 400 + m)
        y = fso.dense.linear(x.cuda(), weight)
        assert tuple(y.shape) == (m, n)
        ref = oracle.dense_linear(x, wq_s, ws_s)
        inputs.assert_close_to_oracle(y[:, torch.from_numpy(cols).cuda()], ref, f"linear M={m} on [{n}, {k}] bsfp8")


def test_quantizer_follows_the_reference_on_non_finite_values(fso, oracle, device_ok):
    """A NaN never becomes a block's amax (the reference reduces with fmaxf, which passes over NaNs) and an Inf makes
    the scale byte 254: the corner-case activation holds both; codes and words equal the reference header's."""
    g = np.load(inputs.GOLDEN)
    x = inputs.edge_activation()
    assert np.array_equal(oracle.bf16_bits(x), g["edge_x_bits"])
    assert torch.isnan(x.float()).any() and torch.isinf(x.float()).any()
    xq, sx = fso.dense.quantize_activation(x.cuda())
    assert np.array_equal(inputs.to_np_u8(xq), g["edge_q"])
    assert np.array_equal(inputs.to_np_u32(sx), g["edge_sf"])
