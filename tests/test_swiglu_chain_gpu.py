"""The step between the gate_up and the down projection of a dense SwiGLU MLP (silu(gate) * up, quantized in one
kernel) against the oracle's exact-silu statement, and the whole MLP chain against its fp32 oracle. The kernel uses
the hardware tanh approximation, so codes may differ from the exact form at rounding boundaries: dequantized values
within 2e-2 relative Frobenius, at least 97 % of the codes and 99 % of the scale bytes equal (the bars the fused MoE
FC1 is held to); padded rows' scale words are zero."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,inter", [(1, 128), (16, 14336), (130, 256), (200, 1024), (1024, 2048)])
def test_silu_mul_quantize_matches_oracle(fso, oracle, device_ok, m, inter):
    gu = inputs.activation(m, 2 * inter, 5 * m + inter)
    xq, sx = fso.compat.silu_chunk_mul_quantize_1x32_fp8(gu.cuda())
    assert xq.dtype == torch.float8_e4m3fn and tuple(xq.shape) == (m, inter)
    assert sx.dtype == torch.int32 and sx.numel() == (m + 127) // 128 * 128 * (inter // 128)
    g, u = gu[:, :inter].float().numpy(), gu[:, inter:].float().numpy()
    inter_leaved = np.empty((m, 2 * inter), np.float32)
    inter_leaved[:, 0::2], inter_leaved[:, 1::2] = g, u
    oq, os_ = oracle.swiglu_quant(inter_leaved, np.ones(m, np.uint8))
    got_q, got_s = inputs.to_np_u8(xq), inputs.to_np_u32(sx)
    got = torch.from_numpy(oracle.dequant(got_q, got_s))
    want = torch.from_numpy(oracle.dequant(oq, os_))
    assert inputs.rel_frobenius(got, want) <= 2e-2
    assert (got_q == oq).mean() > 0.97
    gb, ob = got_s.view(np.uint8), np.asarray(os_).view(np.uint8)
    assert (gb == ob).mean() > 0.99
    # words of the rows past M are zero (the GEMM reads whole 128-row atoms)
    kb = inter // 128
    rows = np.arange(m, (m + 127) // 128 * 128)
    if rows.size:
        idx = oracle.sf_word_index(np.repeat(rows, kb), np.tile(np.arange(kb), rows.size), inter)
        assert not got_s[idx].any()
    # run to run identical, and leading dimensions are flattened
    xq2, sx2 = fso.compat.silu_chunk_mul_quantize_1x32_fp8(gu.cuda().view(1, m, 2 * inter))
    assert torch.equal(xq2.view(torch.uint8), xq.view(torch.uint8)) and torch.equal(sx2, sx)


@pytest.mark.parametrize("m", [16, 300])
def test_swiglu_mlp_chain(fso, oracle, device_ok, m):
    """down(silu(gate) * up) with gate_up and down as MXFP8 linears: the fused middle step gives, within the output
    tolerance, what the oracle's fp32 chain gives (activation and intermediate quantized as the kernels quantize
    them)."""
    h, inter = 512, 1024
    x = inputs.activation(m, h, 3)
    w_gu = fso.dense.prepare_weight(inputs.weight(2 * inter, h, 4).cuda(), format="mxfp8")
    w_dn = fso.dense.prepare_weight(inputs.weight(h, inter, 5).cuda(), format="mxfp8")
    gu = fso.dense.linear(x.cuda(), w_gu)
    hq, hs = fso.compat.silu_chunk_mul_quantize_1x32_fp8(gu)
    y = fso.dense.linear(hq, w_dn, x_scale=hs)
    # oracle: exact silu on the GPU's bf16 gate_up output, 1x32 rule, fp32 down projection
    g, u = gu[:, :inter].float().cpu(), gu[:, inter:].float().cpu()
    hh = (torch.nn.functional.silu(g) * u).numpy()
    inter_leaved = np.empty((m, 2 * inter), np.float32)
    inter_leaved[:, 0::2], inter_leaved[:, 1::2] = g.numpy(), u.numpy()
    oq, os_ = oracle.swiglu_quant(inter_leaved, np.ones(m, np.uint8))
    hd = torch.from_numpy(oracle.dequant(oq, os_))
    assert inputs.rel_frobenius(hd, torch.from_numpy(hh)) < 0.05          # the quantization error of e4m3 itself
    wd = torch.from_numpy(oracle.dequant(inputs.to_np_u8(w_dn.weight), inputs.to_np_u32(w_dn.scale)))
    inputs.assert_close_to_oracle(y, hd @ wd.t(), f"SwiGLU MLP chain M={m}")


@pytest.mark.parametrize("m,h,inter", [(16, 512, 1024), (300, 512, 1024), (1000, 1024, 2048)])
def test_fused_swiglu_mlp_chain(fso, oracle, device_ok, m, h, inter):
    """The same chain with the middle step inside the gate_up GEMM (fso.compat.linear_swiglu): two launches for the
    MLP's two projections, no bf16 [M, 2I] tensor. Against the oracle's fp32 chain from the quantized operands (exact
    silu on the fp32 accumulators, 1x32 rule, fp32 down projection); the intermediate against the oracle's by value,
    and against the two-kernel form, which differs only by the bf16 rounding of gate_up it inserts."""
    x = inputs.activation(m, h, 3)
    w_gu_master = inputs.weight(2 * inter, h, 4)
    w_gu = fso.compat.prepare_gate_up(w_gu_master.cuda(), format="mxfp8")
    w_dn = fso.dense.prepare_weight(inputs.weight(h, inter, 5).cuda(), format="mxfp8")
    # the handle holds the bytes of the interleaved weight
    oq, osf = oracle.quantize_1x32(w_gu_master, interleave_i=inter)
    assert np.array_equal(inputs.to_np_u8(w_gu.weight), oq) and np.array_equal(inputs.to_np_u32(w_gu.scale), osf)
    hq, hs = fso.compat.linear_swiglu(x.cuda(), w_gu)
    assert hq.dtype == torch.float8_e4m3fn and tuple(hq.shape) == (m, inter)
    assert hs.numel() == (m + 127) // 128 * 128 * (inter // 128)
    y = fso.dense.linear(hq, w_dn, x_scale=hs)
    acc = oracle.dense_linear(x, oq, osf).numpy()                       # fp32 [M, 2I], columns gate_j, up_j adjacent
    dq, sd = oracle.swiglu_quant(acc, np.ones(m, np.uint8))
    hd = torch.from_numpy(oracle.dequant(dq, sd))
    got = torch.from_numpy(oracle.dequant(inputs.to_np_u8(hq), inputs.to_np_u32(hs)))
    assert inputs.rel_frobenius(got, hd) <= 2e-2
    assert (inputs.to_np_u8(hq) == dq).mean() > 0.97
    wd = torch.from_numpy(oracle.dequant(inputs.to_np_u8(w_dn.weight), inputs.to_np_u32(w_dn.scale)))
    inputs.assert_close_to_oracle(y, hd @ wd.t(), f"fused SwiGLU MLP chain M={m}")
    # scale words of the rows past M are zero
    got_s = inputs.to_np_u32(hs)
    kb = inter // 128
    rows = np.arange(m, (m + 127) // 128 * 128)
    if rows.size:
        idx = oracle.sf_word_index(np.repeat(rows, kb), np.tile(np.arange(kb), rows.size), inter)
        assert not got_s[idx].any()
    # the two-kernel form on a plain (not interleaved) weight agrees by value
    plain = fso.dense.prepare_weight(w_gu_master.cuda(), format="mxfp8")
    q2, s2 = fso.compat.silu_chunk_mul_quantize_1x32_fp8(fso.dense.linear(x.cuda(), plain))
    two = torch.from_numpy(oracle.dequant(inputs.to_np_u8(q2), inputs.to_np_u32(s2)))
    assert inputs.rel_frobenius(got, two) <= 2e-2
    # the pre-quantized entry gives the same bytes
    xq, sx = fso.dense.quantize_activation(x.cuda())
    hq3, hs3 = fso.compat.linear_swiglu(xq, w_gu, x_scale=sx)
    assert torch.equal(hq3.view(torch.uint8), hq.view(torch.uint8)) and torch.equal(hs3, hs)


def test_silu_mul_quantize_refusals(fso, device_ok):
    with pytest.raises(ValueError):
        fso.compat.silu_chunk_mul_quantize_1x32_fp8(torch.zeros(4, 200, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        fso.compat.silu_chunk_mul_quantize_1x32_fp8(torch.zeros(4, 256, dtype=torch.float32, device="cuda"))
    q, s = fso.compat.silu_chunk_mul_quantize_1x32_fp8(torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda"))
    assert tuple(q.shape) == (0, 128)
