"""Parity of the dense path: quantized bytes bit-exact, bf16 output within tolerance of the fp32
dequantize-then-matmul oracle (rel. Frobenius <= 1e-2, |err| <= 2e-2 * max|ref|)."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def _oracle_out(oracle, x, wq_np, ws_np):
    return oracle.dense_linear(x, wq_np, ws_np)


def test_config1_single_dense_linear(fso, oracle, device_ok):
    """x bf16 [128, 512] ~ N(0,1), w bf16 [256, 512] ~ N(0,0.02), seeds 0 / 1."""
    x, w = inputs.activation(128, 512, 0), inputs.weight(256, 512, 1)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    owq, ows = oracle.quantize_1x32(w)
    assert np.array_equal(inputs.to_np_u8(weight.weight), owq)
    assert np.array_equal(inputs.to_np_u32(weight.scale), ows)
    xq, sx = fso.dense.quantize_activation(x.cuda())
    oxq, oxs = oracle.quantize_1x32(x)
    assert np.array_equal(inputs.to_np_u8(xq), oxq) and np.array_equal(inputs.to_np_u32(sx), oxs)
    y = fso.dense.linear(x.cuda(), weight)
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (128, 256)
    inputs.assert_close_to_oracle(y, _oracle_out(oracle, x, owq, ows), "config 1")
    y2 = fso.dense.linear(xq, weight, x_scale=sx)
    assert torch.equal(y, y2)
    ref = x.float() @ w.float().t()
    cos = torch.nn.functional.cosine_similarity(y.float().cpu().flatten(), ref.flatten(), dim=0)
    assert cos > 0.999


# (M, N, K): every route of the picker: swapped orientation with 16/32/64-wide token tiles, with and without
# split-K, and with two 64-row token tiles per weight panel (65..128 rows, full and ragged second tile); normal
# orientation with 128- and 256-wide tiles, ragged M, split-K, many tiles per CTA.
SHAPES = [(1, 128, 128), (1, 256, 512), (7, 384, 1024), (16, 512, 4096), (17, 256, 512), (32, 1024, 1024),
          (33, 256, 2048), (64, 640, 512), (65, 256, 512), (128, 128, 128), (128, 256, 8192), (200, 384, 640),
          (256, 512, 256), (300, 1024, 1024), (1024, 4096, 512), (2048, 2560, 384), (100, 512, 1024),
          (96, 1024, 2048), (128, 6144, 4096), (127, 4096, 1792), (128, 19200, 256)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_dense_shapes(fso, oracle, device_ok, m, n, k):
    x, w = inputs.activation(m, k, m * 7 + k), inputs.weight(n, k, n * 3 + k)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    y = fso.dense.linear(x.cuda(), weight)
    ref = _oracle_out(oracle, x, inputs.to_np_u8(weight.weight), inputs.to_np_u32(weight.scale))
    inputs.assert_close_to_oracle(y, ref, f"M={m} N={n} K={k}")


def test_dense_nonuniform_scales(fso, oracle, device_ok):
    """Rows and K blocks with very different magnitudes: a wrong scale-factor placement cannot hide."""
    m, n, k = 192, 384, 1024
    g = inputs.gen(99)
    x = inputs.activation(m, k, 1).float() * torch.exp2(torch.randint(-6, 7, (m, k // 32), generator=g).float()
                                                        ).repeat_interleave(32, dim=1)
    w = inputs.weight(n, k, 2).float() * torch.exp2(torch.randint(-6, 7, (n, k // 32), generator=g).float()
                                                    ).repeat_interleave(32, dim=1)
    x, w = x.to(torch.bfloat16), w.to(torch.bfloat16)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    for rows in (m, 40):
        y = fso.dense.linear(x[:rows].cuda(), weight)
        ref = _oracle_out(oracle, x[:rows], inputs.to_np_u8(weight.weight), inputs.to_np_u32(weight.scale))
        inputs.assert_close_to_oracle(y, ref, f"nonuniform rows={rows}")


def test_block_fp8_checkpoint_path(fso, oracle, device_ok):
    n, k, m = 512, 1024, 48
    wq, s = inputs.block_fp8_checkpoint(n, k, 5)
    weight = fso.dense.prepare_weight(wq.cuda(), format="bsfp8", scale=s.cuda())
    oq, osf = oracle.requant_bs128(wq, s)
    assert np.array_equal(inputs.to_np_u8(weight.weight), oq) and np.array_equal(inputs.to_np_u32(weight.scale), osf)
    x = inputs.activation(m, k, 6)
    inputs.assert_close_to_oracle(fso.dense.linear(x.cuda(), weight), _oracle_out(oracle, x, oq, osf), "bsfp8")


def test_mxfp8_checkpoint_forms(fso, oracle, device_ok):
    n, k = 256, 512
    w = inputs.weight(n, k, 12)
    base = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    words = inputs.to_np_u32(base.scale)
    rows = np.repeat(np.arange(n), k // 128)
    kps = np.tile(np.arange(k // 128), n)
    u8 = torch.from_numpy(words[oracle.sf_word_index(rows, kps, k)].reshape(n, k // 128).view(np.uint8).copy())
    from_bytes = fso.dense.prepare_weight(base.weight, format="mxfp8", scale=u8.view(n, k // 32).cuda())
    assert torch.equal(from_bytes.scale, base.scale) and from_bytes.weight.data_ptr() == base.weight.data_ptr()
    from_words = fso.dense.prepare_weight(base.weight, format="mxfp8", scale=base.scale)
    assert torch.equal(from_words.scale, base.scale)


def test_leading_dims_empty_and_quantized(fso, oracle, device_ok):
    w = inputs.weight(256, 256, 3)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    x = inputs.activation(6 * 5, 256, 4).view(6, 5, 256).cuda()
    y = fso.dense.linear(x, weight)
    assert tuple(y.shape) == (6, 5, 256)
    assert torch.equal(y.view(30, 256), fso.dense.linear(x.view(30, 256), weight))
    assert tuple(fso.dense.linear(x[:0], weight).shape) == (0, 5, 256)
    q, s = fso.dense.linear_quantized(x.view(30, 256), weight)
    q2, s2 = fso.dense.quantize_activation(y.view(30, 256))
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    # a bf16 x at a 2-byte offset is copied inside the op and gives the same bytes
    buf = torch.zeros(30 * 256 + 1, dtype=torch.bfloat16, device="cuda")
    buf[1:] = x.reshape(-1)
    assert torch.equal(fso.dense.linear(buf[1:].view(30, 256), weight), y.view(30, 256))


def test_refusals_before_launch(fso, device_ok):
    w = inputs.weight(256, 256, 3).cuda()
    weight = fso.dense.prepare_weight(w, format="mxfp8")
    x = inputs.activation(8, 256, 4).cuda()
    with pytest.raises(ValueError):
        fso.dense.prepare_weight(w[:, :100], format="mxfp8")
    with pytest.raises(ValueError):
        fso.dense.prepare_weight(w[:100], format="mxfp8")
    with pytest.raises(ValueError):
        fso.dense.prepare_weight(w, format="mxfp9")
    with pytest.raises(NotImplementedError):
        fso.dense.prepare_weight(w, format="nvfp4")
    with pytest.raises(ValueError):
        fso.dense.prepare_weight(w, format="mxfp8", scale=torch.ones(2, 2, device="cuda"))
    with pytest.raises(TypeError):
        fso.dense.linear(x, w)
    with pytest.raises(ValueError):
        fso.dense.linear(x[:, :128], weight)
    with pytest.raises(ValueError):
        fso.dense.linear(x.float(), weight)
    xq, sx = fso.dense.quantize_activation(x)
    with pytest.raises(ValueError):
        fso.dense.linear(xq, weight)
    with pytest.raises(ValueError):
        fso.dense.linear(x, weight, x_scale=sx)
    with pytest.raises(ValueError):
        fso.dense.linear(xq, weight, x_scale=sx[:-1])
    with pytest.raises(ValueError):
        fso.dense.linear(x, weight, bias=torch.zeros(255, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        fso.dense.linear(x, weight, bias=torch.zeros(256, dtype=torch.float32, device="cuda"))
    with pytest.raises(ValueError):
        fso.dense.linear(x, weight, residual=torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        fso.dense.linear(x, weight, activation="nope")
    with pytest.raises(NotImplementedError):
        fso.dense.linear(x, weight, activation="silu")
    assert fso.dense.supported("mxfp8") and fso.dense.supported("bsfp8") and not fso.dense.supported("nvfp4")
    assert fso.dense.activation_contract()["format"] == "mxfp8_1x32"
    torch.cuda.synchronize()   # the context is intact after every refusal
    fso.dense.linear(x, weight)


def test_cuda_graph_capture_and_no_sync(fso, oracle, device_ok):
    """Capture after one eager call, NaN-filled replay buffers, replay == eager after rewriting x in place; the call
    never synchronizes (python side of tests/gemm/unit/test_cuda_graph.py:33-80 of the reference)."""
    # a decode-sized call, a single-CTA-kernel call and one the CTA-pair kernel takes (128 tiles of 256 x 256)
    for m, n, k in ((16, 512, 1024), (384, 512, 1024), (2048, 4096, 512)):
        w = inputs.weight(n, k, 21)
        weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
        x = inputs.activation(m, k, 22).cuda()
        eager = fso.dense.linear(x, weight)
        torch.cuda.synchronize()
        torch.cuda.set_sync_debug_mode("error")
        try:
            fso.dense.linear(x, weight)
        finally:
            torch.cuda.set_sync_debug_mode("default")
        static_x = x.clone()
        graph = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            fso.dense.linear(static_x, weight)
            with torch.cuda.graph(graph, stream=stream):
                out = fso.dense.linear(static_x, weight)
        torch.cuda.current_stream().wait_stream(stream)
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
        x2 = inputs.activation(m, k, 23).cuda()
        static_x.copy_(x2)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, fso.dense.linear(x2, weight))


def test_run_to_run_identical_including_split_k(fso, device_ok):
    w = inputs.weight(256, 8192, 1)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    for m in (4, 128):
        x = inputs.activation(m, 8192, 2).cuda()
        assert torch.equal(fso.dense.linear(x, weight), fso.dense.linear(x, weight))


@pytest.mark.parametrize("m,n,k", [(16, 28672, 4096), (128, 6144, 512), (200, 4096, 1024), (1024, 4096, 512),
                                   (2000, 4096, 1024), (4096, 6144, 4096)])
def test_bit_equal_to_cublas_block_scaled_gemm(fso, device_ok, m, n, k):
    """cuBLAS's MXFP8 GEMM (`torch._scaled_mm` with E8M0 scales in the 32x4x4 swizzle, which is this library's atom
    layout) is the kernel the reference itself sends every wide-N dense call to
    (python/fish_scales_ops/gemm/_sm100_smm.py:273-306). Both accumulate K in order in fp32 inside the tensor core
    and round once to bf16, so without split-K the outputs are equal bit for bit, whatever the tile shape (single
    CTA, CTA pair, swapped orientation)."""
    from fish_scales_ops_b200 import _ops

    e8 = getattr(torch, "float8_e8m0fnu", None)
    if e8 is None:
        pytest.skip("this torch has no float8_e8m0fnu")
    assert _ops.gemm_ws_bytes(m, n, k) == 0, "pick shapes that do not take the split-K route"
    x = inputs.activation(m, k, 11 * m + k).cuda()
    weight = fso.dense.prepare_weight(inputs.weight(n, k, 13 * n + k).cuda(), format="mxfp8")
    xq, sx = fso.dense.quantize_activation(x)
    y = fso.dense.linear(xq, weight, x_scale=sx)
    try:
        ref = torch._scaled_mm(xq, weight.weight.t(), scale_a=sx.view(torch.uint8).view(e8),
                               scale_b=weight.scale.view(torch.uint8).view(e8), out_dtype=torch.bfloat16)
    except Exception as exc:  # noqa: BLE001 - a torch / cuBLAS build without the MXFP8 recipe
        pytest.skip(f"torch._scaled_mm does not serve MXFP8 here: {str(exc)[:120]}")
    assert torch.equal(y, ref)


_CHILD = r"""
import sys, torch
sys.path.insert(0, %r); sys.path.insert(0, %r)
import inputs
import fish_scales_ops_b200 as fso
from fish_scales_ops_b200 import _ops
for m, n, k in %r:
    x = inputs.activation(m, k, m + k).cuda()
    w = fso.dense.prepare_weight(inputs.weight(n, k, n + k).cuda(), format="mxfp8")
    torch.save(fso.dense.linear(x, w).cpu(), sys.argv[1] + f".{m}.{n}.{k}.pt")
assert _ops.device_status() == 0
print("ok")
"""


def _outputs_in_child_process(shapes, env_extra, tag):
    """fso.dense.linear over `shapes` in a child process with extra environment (the switches are read once per
    process)."""
    import os
    import subprocess
    import sys

    import tempfile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tmp = tempfile.mkdtemp(prefix="fso_child_")
    base = os.path.join(tmp, tag)
    res = subprocess.run([sys.executable, "-c", _CHILD % (root, os.path.join(root, "tests"), tuple(shapes)), base],
                         env=dict(os.environ, **env_extra), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
    outs = {}
    for m, n, k in shapes:
        path = f"{base}.{m}.{n}.{k}.pt"
        outs[(m, n, k)] = torch.load(path)
        os.remove(path)
    return outs


def test_cta_pair_kernel_in_child_process(fso, device_ok):
    """The CTA-pair kernel (large calls take it unless FSO_B200_PAIR=0) gives the bytes of the single-CTA kernel,
    including a ragged M whose second CTA of the last pair has no rows."""
    shapes = ((2048, 4096, 512), (1920, 5120, 256), (2100, 4096, 1024))
    pair = _outputs_in_child_process(shapes, {"FSO_B200_PAIR": "1"}, "pair1")
    single = _outputs_in_child_process(shapes, {"FSO_B200_PAIR": "0"}, "pair0")
    for shape in shapes:
        assert torch.equal(pair[shape], single[shape]), shape


def test_cluster_split_k_equals_workspace_split_k(fso, oracle, device_ok):
    """Decode-sized problems sum their K slices inside thread-block clusters (one launch); FSO_B200_SPLITK=workspace
    keeps fp32 partials in a workspace and a second kernel. Same slices, same order of additions: same bytes. The
    shapes cover 16/32/64-wide token tiles, clusters of 2 to 8 CTAs and ragged token counts."""
    from fish_scales_ops_b200 import _ops

    shapes = ((16, 4096, 4096), (16, 6144, 4096), (5, 4096, 14336), (16, 512, 4096), (7, 384, 1024),
              (32, 1024, 1024), (29, 2560, 2048), (64, 512, 1536), (50, 1024, 1536),
              (128, 4096, 4096), (100, 1024, 2048), (65, 512, 1536))       # two token tiles per weight panel
    for m, n, k in shapes:
        assert _ops.gemm_ws_bytes(m, n, k) > 0, "pick shapes that take the split-K route"
    cluster = _outputs_in_child_process(shapes, {"FSO_B200_SPLITK": "cluster"}, "splitk_cluster")
    workspace = _outputs_in_child_process(shapes, {"FSO_B200_SPLITK": "workspace"}, "splitk_ws")
    for shape in shapes:
        assert torch.equal(cluster[shape], workspace[shape]), shape
    m, n, k = shapes[0]
    x, w = inputs.activation(m, k, m + k), inputs.weight(n, k, n + k)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    ref = _oracle_out(oracle, x, inputs.to_np_u8(weight.weight), inputs.to_np_u32(weight.scale))
    inputs.assert_close_to_oracle(cluster[shapes[0]], ref, "cluster split-K vs oracle")


_CHAIN_CHILD = r"""
import sys, torch
sys.path.insert(0, %r); sys.path.insert(0, %r)
import inputs
import fish_scales_ops_b200 as fso
from fish_scales_ops_b200 import _ops
dims = [1024, 2048, 1024, 4096, 512, 2048]
ws = [fso.dense.prepare_weight(inputs.weight(dims[i + 1], dims[i], 90 + i).cuda(), format="mxfp8")
      for i in range(len(dims) - 1)]
outs = {}
for m in (1, 16, 40):
    x = inputs.activation(m, dims[0], 80 + m).cuda()
    def chain():
        h, keep = x, []
        for w in ws:
            h = fso.dense.linear(h, w)          # quantizer + decode GEMM, each GEMM reads what the last one wrote
            keep.append(h)
        xq, sx = fso.dense.quantize_activation(x)
        for _ in range(3):                       # pre-quantized form: GEMM directly behind GEMM
            keep.append(fso.dense.linear(xq, ws[0], x_scale=sx))
        return keep
    eager = chain()
    side = torch.cuda.Stream(); side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            graphed = chain()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, graphed):
        assert torch.equal(a, b), "graph replay differs from eager"
    outs[m] = [t.cpu() for t in eager]
assert _ops.device_status() == 0
torch.save(outs, sys.argv[1] + ".pt")
print("ok")
"""


def test_dependent_launch_chain_equals_plain_launches(fso, device_ok):
    """Decode-sized GEMMs are launched with programmatic dependent launch: a GEMM starts its set-up and weight loads
    while its predecessor (the activation quantizer or the previous GEMM) still runs, and waits for it before reading
    activations or writing. A chain in which every linear consumes the previous one's output, eager and under CUDA-graph
    replay, must give the bytes of the same chain with plain launches (FSO_B200_PDL=0)."""
    import os
    import subprocess
    import sys

    import tempfile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    tmp = tempfile.mkdtemp(prefix="fso_child_")
    got = {}
    for pdl in ("1", "0"):
        base = os.path.join(tmp, f"chain_pdl{pdl}")
        res = subprocess.run([sys.executable, "-c", _CHAIN_CHILD % (root, os.path.join(root, "tests")), base],
                             env=dict(os.environ, FSO_B200_PDL=pdl), capture_output=True, text=True, timeout=600)
        assert res.returncode == 0 and "ok" in res.stdout, res.stderr[-2000:]
        got[pdl] = torch.load(base + ".pt")
        os.remove(base + ".pt")
    for m in got["1"]:
        for a, b in zip(got["1"][m], got["0"][m]):
            assert torch.equal(a, b), m


# (M, N, K): the normal kernel with 128- and 256-wide tiles and a ragged M, its split-K (epilogue in the reduce
# kernel), the swapped kernel without split, with the cluster split-K and with the workspace split-K of a long K
EPI_SHAPES = [(200, 384, 640), (300, 1024, 1024), (1024, 4096, 512), (128, 256, 8192), (16, 28672, 256),
              (16, 4096, 4096), (40, 512, 1536), (4, 256, 16384)]


@pytest.mark.parametrize("m,n,k", EPI_SHAPES)
def test_dense_epilogue_bias_gelu_residual(fso, oracle, device_ok, m, n, k):
    """out = bf16(act(acc + bias[n]) + residual[m, n]) with one rounding
    (csrc/gemm/include/blockscale_gemm/common/epilogue.cuh:1-30 of the reference), every combination of the three
    fields, against the oracle's fp32 statement within the output tolerance."""
    x, w = inputs.activation(m, k, m + k), inputs.weight(n, k, n + k)
    weight = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    g = inputs.gen(m * n)
    bias = torch.randn(n, generator=g, dtype=torch.float32).to(torch.bfloat16)
    res = torch.randn(m, n, generator=g, dtype=torch.float32).to(torch.bfloat16)
    acc = _oracle_out(oracle, x, inputs.to_np_u8(weight.weight), inputs.to_np_u32(weight.scale))
    plain = fso.dense.linear(x.cuda(), weight)
    for use_bias, use_res, act in ((1, 0, None), (0, 1, None), (0, 0, "gelu_erf"), (1, 1, "gelu_erf"), (1, 1, None)):
        y = fso.dense.linear(x.cuda(), weight, bias=bias.cuda() if use_bias else None,
                             residual=res.cuda() if use_res else None, activation=act)
        ref = oracle.dense_epilogue(acc, bias if use_bias else None, res if use_res else None, act)
        inputs.assert_close_to_oracle(y, ref, f"M={m} N={n} K={k} bias={use_bias} res={use_res} act={act}")
    # a zero bias (of either sign) and a zero residual leave the bytes of the plain call
    zb = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    assert torch.equal(fso.dense.linear(x.cuda(), weight, bias=zb), plain)
    assert torch.equal(fso.dense.linear(x.cuda(), weight, bias=-zb), plain)
    # linear_quantized = quantize(linear(bias, activation))
    yq, ys = fso.dense.linear_quantized(x.cuda(), weight, bias=bias.cuda(), activation="gelu_erf")
    want_q, want_s = fso.dense.quantize_activation(fso.dense.linear(x.cuda(), weight, bias=bias.cuda(),
                                                                    activation="gelu_erf"))
    assert torch.equal(yq.view(torch.uint8), want_q.view(torch.uint8)) and torch.equal(ys, want_s)


def test_dense_epilogue_against_torch_on_device(fso, device_ok):
    """The same epilogue written with torch ops on the fp32 result of the plain call's operands: erf-GELU and the
    additions in fp32, one rounding."""
    m, n, k = 256, 512, 1024
    x, w = inputs.activation(m, k, 1).cuda(), inputs.weight(n, k, 2).cuda()
    weight = fso.dense.prepare_weight(w, format="mxfp8")
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    res = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    y = fso.dense.linear(x, weight, bias=bias, residual=res, activation="gelu_erf")
    base = fso.dense.linear(x, weight).float()               # bf16-rounded accumulator: close enough for a bound
    want = torch.nn.functional.gelu(base + bias.float()) + res.float()
    err = (y.float() - want).abs().max() / want.abs().max()
    assert float(err) < 2e-2


@pytest.mark.parametrize("m,n,k", [(300, 1024, 512), (1024, 4096, 1024), (4096, 2048 + 128, 512), (129, 8192, 256)])
def test_linear_quantized_fused_epilogue_equals_two_launches(fso, device_ok, m, n, k):
    """For shapes the GEMM runs in its normal orientation without split-K, linear_quantized is one launch (the 1x32
    quantization happens in the GEMM's epilogue, after the rounding to bf16) and gives exactly the bytes of
    quantize_activation(linear(...)), with and without bias / activation; scale words of rows past M are zero."""
    from fish_scales_ops_b200 import _ops

    assert _ops.gemm_fuses_quantized_output(m, n, k)
    x = inputs.activation(m, k, 11).cuda()
    weight = fso.dense.prepare_weight(inputs.weight(n, k, 12).cuda(), format="mxfp8")
    bias = (0.5 * torch.randn(n, generator=inputs.gen(13))).to(torch.bfloat16).cuda()
    for kw in ({}, {"bias": bias}, {"activation": "gelu_erf"}, {"bias": bias, "activation": "gelu_erf"}):
        yq, ys = fso.dense.linear_quantized(x, weight, **kw)
        want_q, want_s = fso.dense.quantize_activation(fso.dense.linear(x, weight, **kw))
        assert yq.dtype == torch.float8_e4m3fn and tuple(yq.shape) == (m, n)
        assert torch.equal(yq.view(torch.uint8), want_q.view(torch.uint8)), kw
        assert torch.equal(ys, want_s), kw
    # small M takes the swapped orientation: two launches, same contract
    assert not _ops.gemm_fuses_quantized_output(16, n, k)
    q16, s16 = fso.dense.linear_quantized(x[:16], weight)
    w16q, w16s = fso.dense.quantize_activation(fso.dense.linear(x[:16], weight))
    assert torch.equal(q16.view(torch.uint8), w16q.view(torch.uint8)) and torch.equal(s16, w16s)
