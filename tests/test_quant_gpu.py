"""Bit-exact parity of the quantizer family (through the C ABI) with the CPU checker and the golden vectors."""
import os

import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantize_1x32.npz")


def _check_quant(oracle, ops, x_cpu, interleave_i=0):
    q, s = ops.quantize_1x32_fp8(x_cpu.cuda(), interleave_i=interleave_i)
    oq, os_ = oracle.quantize_1x32(x_cpu, interleave_i=interleave_i)
    assert np.array_equal(inputs.to_np_u8(q), oq)
    assert np.array_equal(inputs.to_np_u32(s), os_)


def test_quantizer_golden_edge(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    g = np.load(GOLDEN)
    q, s = _ops.quantize_1x32_fp8(inputs.edge_activation().cuda())
    assert np.array_equal(inputs.to_np_u8(q), g["edge_q"])
    assert np.array_equal(inputs.to_np_u32(s), g["edge_sf"])


@pytest.mark.parametrize("m,k", [(1, 128), (3, 256), (16, 4096), (127, 512), (128, 512), (129, 384), (1000, 1024),
                                 (4096, 4096)])
def test_quantizer_matches_oracle(fso, oracle, device_ok, m, k):
    from fish_scales_ops_b200 import _ops

    _check_quant(oracle, _ops, inputs.activation(m, k, 100 + m + k))


def test_quantizer_scales_of_magnitudes(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    x = inputs.activation(256, 512, 5).float()
    scale = torch.exp2(torch.randint(-40, 40, (256, 1), generator=inputs.gen(6)).float())
    _check_quant(oracle, _ops, (x * scale).to(torch.bfloat16))


def test_expert_weight_quantizer_with_interleave(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    e, i, h = 3, 128, 256
    w = inputs.weight(e * 2 * i, h, 8)
    _check_quant(oracle, _ops, w, interleave_i=i)
    q, s = _ops.quantize_experts_1x32_fp8(w.view(e, 2 * i, h).cuda(), interleave=True)
    assert tuple(q.shape) == (e, 2 * i, h) and tuple(s.shape) == (e, 2 * i * h // 128)


@pytest.mark.parametrize("n,k", [(128, 128), (256, 512), (1024, 2048)])
def test_requant_matches_oracle(fso, oracle, device_ok, n, k):
    from fish_scales_ops_b200 import _ops

    wq, s = inputs.block_fp8_checkpoint(n, k, 31 + n)
    q, sf = _ops.requant_block_fp8(wq.cuda(), s.cuda())
    oq, osf = oracle.requant_bs128(wq, s)
    assert np.array_equal(inputs.to_np_u8(q), oq)
    assert np.array_equal(inputs.to_np_u32(sf), osf)


def test_requant_interleaved_experts(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    e, i, h = 2, 128, 256
    wq, s = inputs.block_fp8_checkpoint(e * 2 * i, h, 77)
    q, sf = _ops.requant_block_fp8(wq.cuda(), s.cuda(), interleave_i=i)
    oq, osf = oracle.requant_bs128(wq, s, interleave_i=i)
    assert np.array_equal(inputs.to_np_u8(q), oq)
    assert np.array_equal(inputs.to_np_u32(sf), osf)


def test_pack_ue8m0_matches_oracle(fso, oracle, device_ok):
    from fish_scales_ops_b200 import _ops

    g, n, k = 3, 256, 512
    s = torch.randint(118, 137, (g, n, k // 32), generator=inputs.gen(4), dtype=torch.uint8)
    out = _ops.pack_ue8m0(s.cuda())
    assert np.array_equal(inputs.to_np_u32(out), oracle.pack_ue8m0(s))
    out_i = _ops.pack_ue8m0(s.cuda(), interleave=True)
    assert np.array_equal(inputs.to_np_u32(out_i), oracle.pack_ue8m0(s, interleave_i=n // 2))


def test_quantizer_is_run_to_run_identical(fso, device_ok):
    from fish_scales_ops_b200 import _ops

    x = inputs.activation(777, 1024, 2).cuda()
    a = _ops.quantize_1x32_fp8(x)
    b = _ops.quantize_1x32_fp8(x)
    assert torch.equal(a[0].view(torch.uint8), b[0].view(torch.uint8)) and torch.equal(a[1], b[1])


def test_quantizer_narrow_and_wide_kernels_agree(fso, oracle, device_ok):
    """A 32-byte aligned input takes the 256-bit-load kernel, a 16-byte aligned one the 128-bit-load kernel; both
    give the oracle's bytes."""
    from fish_scales_ops_b200 import _ops

    m, k = 300, 640
    x = inputs.activation(m, k, 41)
    buf = torch.zeros(m * k + 8, dtype=torch.bfloat16, device="cuda")
    buf[8:] = x.reshape(-1).cuda()
    narrow = buf[8:].view(m, k)
    assert narrow.data_ptr() % 32 == 16 and narrow.is_contiguous()
    wide = x.cuda()
    assert wide.data_ptr() % 32 == 0
    oq, os_ = oracle.quantize_1x32(x)
    for t in (narrow, wide):
        q, s = _ops.quantize_1x32_fp8(t)
        assert np.array_equal(inputs.to_np_u8(q), oq) and np.array_equal(inputs.to_np_u32(s), os_)


def test_requant_narrow_and_wide_kernels_agree(fso, oracle, device_ok):
    """A checkpoint on a 32-byte boundary takes the 256-bit kernel, one 16 bytes past it the 128-bit kernel: same
    bytes, and both equal the oracle."""
    from fish_scales_ops_b200 import _ops

    n, k = 384, 512
    wq, s = inputs.block_fp8_checkpoint(n, k, 21)
    raw = torch.empty(n * k + 16, dtype=torch.uint8, device="cuda")
    shifted = raw[16:].view(torch.float8_e4m3fn).view(n, k)
    shifted.copy_(wq.cuda())
    assert shifted.data_ptr() % 32 == 16
    q_wide, sf_wide = _ops.requant_block_fp8(wq.cuda(), s.cuda())
    q_narrow, sf_narrow = _ops.requant_block_fp8(shifted, s.cuda())
    assert torch.equal(q_wide.view(torch.uint8), q_narrow.view(torch.uint8)) and torch.equal(sf_wide, sf_narrow)
    oq, osf = oracle.requant_bs128(wq, s)
    assert np.array_equal(inputs.to_np_u8(q_wide), oq) and np.array_equal(inputs.to_np_u32(sf_wide), osf)
