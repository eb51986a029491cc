"""The CPU checker against the reference: its own header compiled on the host (oracle/_ref, where present) and the
golden vectors generated from it (tests/golden/quantize_1x32.npz)."""
import ctypes
import hashlib
import os

import numpy as np
import pytest
import torch

import inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantize_1x32.npz")


def _sha(q, sf):
    return hashlib.sha256(q.tobytes() + sf.tobytes()).hexdigest()


def test_golden_edge_vector(oracle):
    g = np.load(GOLDEN)
    edge = inputs.edge_activation()
    assert np.array_equal(oracle.bf16_bits(edge), g["edge_x_bits"]), "the edge input generator drifted"
    q, sf = oracle.quantize_1x32(edge)
    assert np.array_equal(q, g["edge_q"])
    assert np.array_equal(sf, g["edge_sf"])
    # padded rows 130..255 of the second 128-row block: zero words
    rows = np.arange(130, 256)
    for kp in range(2):
        assert not sf[oracle.sf_word_index(rows, np.full_like(rows, kp), 256)].any()


def test_golden_config1(oracle):
    g = np.load(GOLDEN)
    xq, xs = oracle.quantize_1x32(inputs.activation(128, 512, 0))
    wq, ws = oracle.quantize_1x32(inputs.weight(256, 512, 1))
    assert _sha(xq, xs) == str(g["cfg1_x_sha"])
    assert _sha(wq, ws) == str(g["cfg1_w_sha"])
    assert np.array_equal(xq[:8], g["cfg1_x_q_head"])
    assert np.array_equal(xs, g["cfg1_x_sf"])


def test_known_bytes_of_the_rule(oracle):
    # amax -> scale byte examples: 0.5 -> 118, 448 -> 127, 896 -> 128, 1e-10 (the floor) -> 85
    L = oracle.lib()
    for amax, want in ((0.5, 118), (448.0, 127), (896.0, 128), (1e-10, 85)):
        qs = ctypes.c_float()
        assert L.orc_e8m0_from_amax(ctypes.c_float(amax), ctypes.byref(qs)) == want
        assert L.orc_e8m0_from_amax_int(ctypes.c_float(amax), ctypes.byref(qs)) == want


def test_integer_rule_equals_divide_rule_for_every_bf16_amax(oracle):
    L = oracle.lib()
    floor = np.float32(1e-10)
    # every bf16 magnitude from the floor up to and including +Inf (0x7F80)
    vals = [floor] + [v for v in (np.arange(1, 0x7F81, dtype=np.uint32) << 16).view(np.float32) if v >= floor]
    for v in vals:
        a, b = ctypes.c_float(), ctypes.c_float()
        x = L.orc_e8m0_from_amax(ctypes.c_float(v), ctypes.byref(a))
        y = L.orc_e8m0_from_amax_int(ctypes.c_float(v), ctypes.byref(b))
        assert x == y and np.float32(a.value).tobytes() == np.float32(b.value).tobytes(), float(v)


def test_restatement_matches_reference_header(oracle):
    R = oracle.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref is not built here (no reference tree); the golden vectors pin the same bytes")
    L = oracle.lib()
    assert R.ref_contract_version() == 1
    rng = np.random.default_rng(7)
    xs = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1, 30, 500, 1e-2, 1e-4)])
    for v in xs[::3]:
        assert L.orc_e4m3_from_float(ctypes.c_float(v)) == R.ref_e4m3_from_float(ctypes.c_float(v)), float(v)
    for m, kp, k in ((0, 0, 128), (37, 1, 512), (129, 3, 512), (1000, 7, 1024)):
        assert L.orc_sf_word_index(m, kp, k) == R.ref_sf_word_index_sm100(m, kp, k)
    x = torch.randn(257, 384, generator=inputs.gen(3)).to(torch.bfloat16)
    q, s = oracle.quantize_1x32(x)
    q2, s2 = oracle.ref_quantize_1x32(x)
    assert np.array_equal(q, q2) and np.array_equal(s, s2)


def test_interleave_is_a_row_permutation(oracle):
    e, i, k = 2, 128, 256
    w = inputs.weight(e * 2 * i, k, 5)
    q, s = oracle.quantize_1x32(w)
    qi, si = oracle.quantize_1x32(w, interleave_i=i)
    for g in range(e):
        for r in range(2 * i):
            src = g * 2 * i + (i + r // 2 if r & 1 else r // 2)
            dst = g * 2 * i + r
            assert np.array_equal(qi[dst], q[src])
            for kp in range(k // 128):
                assert si[oracle.sf_word_index(np.array(dst), np.array(kp), k)] == \
                    s[oracle.sf_word_index(np.array(src), np.array(kp), k)]


def test_pack_ue8m0_matches_quantizer_words(oracle):
    # bytes [N, K/32] taken from the quantizer's own words must pack back to the same words
    w = inputs.weight(256, 512, 11)
    _, s = oracle.quantize_1x32(w)
    n, k = 256, 512
    rows = np.repeat(np.arange(n), k // 128)
    kps = np.tile(np.arange(k // 128), n)
    words = s[oracle.sf_word_index(rows, kps, k)].reshape(n, k // 128)
    bytes_ = words.view(np.uint8).reshape(1, n, k // 32)
    assert np.array_equal(oracle.pack_ue8m0(bytes_)[0], s)


def test_requant_is_dequant_then_quantize(oracle):
    wq, s = inputs.block_fp8_checkpoint(256, 256, 21)
    q, sf = oracle.requant_bs128(wq, s)
    deq = (wq.to(torch.float32).view(2, 128, 2, 128) * s.view(2, 1, 2, 1)).view(256, 256).to(torch.bfloat16)
    q2, sf2 = oracle.quantize_1x32(deq)
    assert np.array_equal(q, q2) and np.array_equal(sf, sf2)


def test_route_contract(oracle):
    # the contract of tests/gemm/unit/test_moe_routing_compact.py:98-195 of the reference, on the canonical order
    ids, _ = inputs.routing(300, 16, 4, 9)
    ids = ids.clone()
    ids[5, 1] = -1
    ids[6, 0] = 16
    nb = max(1, (1200 + 127 * 16) // 128)
    mm, b0, sl, be = oracle.route(ids, 16, nb)
    flat = ids.reshape(-1).numpy()
    valid = (flat >= 0) & (flat < 16)
    assert np.array_equal(mm, np.bincount(flat[valid], minlength=16))
    assert np.array_equal(b0, np.concatenate([[0], np.cumsum((mm + 127) // 128)]))
    assert (sl[~valid] == -1).all()
    live = sl[valid]
    assert len(set(live.tolist())) == live.size
    for e in range(16):
        mine = np.nonzero(flat == e)[0]
        assert np.array_equal(sl[mine], b0[e] * 128 + np.arange(mine.size))
        assert (be[b0[e]:b0[e + 1]] == e).all()
    assert (be[b0[16]:] == -1).all()


def test_dense_oracle_tracks_bf16_masters(oracle):
    x = inputs.activation(32, 512, 0)
    w = inputs.weight(64, 512, 1)
    wq, ws = oracle.quantize_1x32(w)
    y = oracle.dense_linear(x, wq, ws)
    ref = x.float() @ w.float().t()
    cos = torch.nn.functional.cosine_similarity(y.flatten(), ref.flatten(), dim=0)
    assert cos > 0.999


def test_router_oracle_matches_torch_softmax_topk(oracle):
    """The router oracle against torch's softmax / topk on random fp32 logits (no ties): same ids in the same order,
    weights to fp32 rounding, with and without renormalization; padded rows, map and gate by their definitions."""
    import inputs

    for m, e, k in ((64, 128, 8), (33, 1024, 8), (17, 256, 1), (9, 40, 5)):
        lg = torch.randn(m, e + 1, generator=inputs.gen(3 * m + e), dtype=torch.float32) * 3.0
        for renorm in (True, False):
            ids, w, gate = oracle.router_topk(lg, k, renorm, True)
            p = torch.softmax(lg[:, :e], dim=-1)
            tw, ti = torch.topk(p, k, dim=-1)
            if renorm:
                tw = tw / tw.sum(dim=-1, keepdim=True)
            assert np.array_equal(ids, ti.numpy().astype(np.int32))
            assert float(np.abs(w - tw.numpy()).max()) <= 1e-5 * float(tw.max())
            assert float(np.abs(gate - torch.sigmoid(lg[:, e]).numpy()).max()) <= 1e-6
        emap = np.arange(e + 1, dtype=np.int32)[::-1].copy()
        ids_m, w_m, _ = oracle.router_topk(lg[:, :e], k, True, False, m // 2, emap)
        ids_p, _, _ = oracle.router_topk(lg[:, :e], k, True)
        assert np.array_equal(ids_m[:m // 2], emap[ids_p[:m // 2]])
        assert (ids_m[m // 2:] == emap[e]).all() and (w_m[m // 2:] == 0).all()


def test_dense_epilogue_oracle_known_answers(oracle):
    """The epilogue oracle on values whose results are known: a zero bias of either sign changes nothing (not even
    the sign of a zero accumulator), erf-GELU equals torch's, and the order is act(acc + bias) + residual."""
    acc = torch.tensor([[0.0, -0.0, 1.5, -2.0], [3.0, -0.25, 0.0, 8.0]], dtype=torch.float32)
    for zero in (0.0, -0.0):
        out = oracle.dense_epilogue(acc, torch.full((4,), zero, dtype=torch.bfloat16))
        assert torch.equal(out.view(torch.int32), acc.view(torch.int32))
    bias = torch.tensor([0.5, -1.0, 0.0, 2.0], dtype=torch.bfloat16)
    res = torch.tensor([[1.0, 1.0, 1.0, 1.0], [-2.0, 0.5, 0.25, 0.0]], dtype=torch.bfloat16)
    out = oracle.dense_epilogue(acc, bias, res, "gelu_erf")
    want = torch.nn.functional.gelu(acc + bias.float()) + res.float()
    assert float((out - want).abs().max()) <= 1e-6
    assert torch.equal(oracle.dense_epilogue(acc, None, res, None), acc + res.float())
    with pytest.raises(ValueError):
        oracle.dense_epilogue(acc, None, None, "gelu_tanh")


_CONTRACT_SHIM = r"""
#include "fso_b200_activation_contract.h"
void shim_quantize(const uint16_t* x, int64_t m, int64_t k, uint8_t* q, uint32_t* sf)
{
    int64_t const words = fso_b200_sf_words(m, k);
    for (int64_t i = 0; i < words; ++i) sf[i] = 0;
    for (int64_t r = 0; r < m; ++r)
        for (int64_t kp = 0; kp < k / FSO_B200_CHUNK; ++kp) {
            uint8_t b[4];
            for (int j = 0; j < 4; ++j) {
                float v[FSO_B200_BLOCK];
                for (int i = 0; i < FSO_B200_BLOCK; ++i)
                    v[i] = fso_b200_float_of((uint32_t)x[r * k + kp * FSO_B200_CHUNK + j * FSO_B200_BLOCK + i] << 16);
                b[j] = fso_b200_quantize_block(v, q + r * k + kp * FSO_B200_CHUNK + j * FSO_B200_BLOCK);
            }
            sf[fso_b200_sf_word_index(r, kp, k)] = fso_b200_pack_word(b[0], b[1], b[2], b[3]);
        }
}
"""


def test_shipped_contract_header_gives_the_golden_bytes(oracle, tmp_path):
    """include/fso_b200_activation_contract.h (what include_dir() hands a producer of pre-quantized activations),
    compiled as plain C on the host, reproduces the reference header's bytes on the corner-case activation (NaN and
    Inf rows included) and the oracle's on a random one."""
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "shim.c"
    src.write_text(_CONTRACT_SHIM)
    so = tmp_path / "shim.so"
    subprocess.run(["gcc", "-std=c99", "-O2", "-ffp-contract=off", "-shared", "-fPIC", "-Wall", "-Werror",
                    "-I", os.path.join(root, "include"), str(src), "-o", str(so)], check=True)
    L = ctypes.CDLL(str(so))

    def run(x):
        xb = oracle.bf16_bits(x)
        m, k = xb.shape
        q = np.empty((m, k), np.uint8)
        sf = np.empty(oracle.sf_words(m, k), np.uint32)
        L.shim_quantize(xb.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(m), ctypes.c_int64(k),
                        q.ctypes.data_as(ctypes.c_void_p), sf.ctypes.data_as(ctypes.c_void_p))
        return q, sf

    g = np.load(GOLDEN)
    q, sf = run(inputs.edge_activation())
    assert np.array_equal(q, g["edge_q"]) and np.array_equal(sf, g["edge_sf"])
    x = (inputs.activation(300, 384, 77).float() * torch.exp2(torch.randint(-30, 30, (300, 1), generator=inputs.gen(78))
                                                              .float())).to(torch.bfloat16)
    q, sf = run(x)
    oq, osf = oracle.quantize_1x32(x)
    assert np.array_equal(q, oq) and np.array_equal(sf, osf)
