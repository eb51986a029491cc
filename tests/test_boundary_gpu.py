"""Behaviour of the drop-in boundary on the device, after the reference's own boundary tests: one custom-op node per
``linear`` under ``torch.compile(fullgraph=True)`` (tests/gemm/unit/test_dense.py:352-393), the routing builders
under two host threads on two streams (tests/gemm/unit/test_moe_routing_threads.py), refusals that launch nothing
(tests/gemm/unit/test_misaligned_x.py, checked with torch.profiler) and the bounded device-side waits."""
import threading

import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def test_compile_records_one_custom_op_node(fso, device_ok):
    n, k = 2560, 4096
    weight = fso.dense.prepare_weight(inputs.weight(n, k, 21).cuda(), format="mxfp8")

    def f(x):
        return fso.dense.linear(x, weight)

    xs = {m: inputs.activation(m, k, 22 + m).cuda() for m in (64, 1000, 7)}
    want = {m: f(x) for m, x in xs.items()}
    graphs = []

    def record(gm, example_inputs):
        graphs.append(gm)
        return gm.forward

    torch._dynamo.reset()
    rec = torch.compile(f, backend=record, fullgraph=True)
    for m, x in xs.items():
        assert torch.equal(rec(x), want[m]), m
    assert 1 <= len(graphs) <= 3
    for g in graphs:
        ours = [str(nd.target) for nd in g.graph.nodes if nd.op == "call_function" and "fish_scales_ops" in str(nd.target)]
        assert len(ours) == 1 and "dense_linear" in ours[0], ours
    torch._dynamo.reset()
    eager = torch.compile(f, backend="aot_eager", fullgraph=True)
    for m, x in xs.items():
        assert torch.equal(eager(x), want[m]), m
    torch._dynamo.reset()


def _check_routing(oracle, ids_cpu, e, got):
    t, k = ids_cpu.shape
    from fish_scales_ops_b200 import _ops

    plan = _ops.moe_plan(t, k, e)
    want = oracle.route(ids_cpu, e, int(plan.num_blocks))
    for g, w, name in zip(got, want, ("masked_m", "blk0", "slot_of_flat", "blk_expert")):
        assert np.array_equal(g.cpu().numpy(), w), name


def test_routing_two_threads_two_streams(fso, oracle, device_ok):
    """Bursts of routing calls from two host threads, each on its own stream, with no host synchronisation inside a
    burst (so the two streams' kernels really overlap); every result is compared with the oracle afterwards. Covers
    the single-CTA and the multi-segment builder (whose scratch is allocated per call)."""
    from fish_scales_ops_b200 import _ops

    e, k = 128, 8
    draws = {"small": [inputs.routing(96, e, k, 900 + i)[0] for i in range(6)],
             "multi": [inputs.routing(2048, e, k, 950 + i, skew=1.2 if i % 2 else 0.0)[0] for i in range(6)]}
    errors = []
    start = threading.Barrier(2)

    def worker(idx):
        try:
            stream = torch.cuda.Stream()
            for name, ids_list in draws.items():
                dev = [ids.cuda() for ids in ids_list]
                torch.cuda.synchronize()
                for burst in range(3):
                    start.wait()
                    outs = []
                    with torch.cuda.stream(stream):
                        for rep in range(4):
                            for j, ids in enumerate(dev):
                                if (j + idx) % 2 == 0:
                                    plan = _ops.moe_plan(int(ids.shape[0]), k, e)
                                    outs.append((j, _ops.moe_route(ids, e, plan)))
                    stream.synchronize()
                    for j, got in outs:
                        _check_routing(oracle, ids_list[j], e, got)
        except Exception as ex:  # noqa: BLE001 - reported by the main thread
            errors.append(ex)
            try:
                start.abort()
            except Exception:  # noqa: BLE001
                pass

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors


@pytest.mark.parametrize("t,e,k", [(16, 1024, 8), (64, 720, 8), (2048, 720, 8), (3000, 1000, 8)])
def test_routing_with_many_experts(fso, oracle, device_ok, t, e, k):
    """Expert counts whose [32][E] shared-memory table passes 48 KB together with the kernels' static arrays, for the
    single-CTA and the multi-segment builder, through both entry points."""
    import ctypes

    from fish_scales_ops_b200 import _lib, _ops

    ids = inputs.routing(t, e, k, 500 + t + e)[0]
    plan = _ops.moe_plan(t, k, e)
    got = _ops.moe_route(ids.cuda(), e, plan)
    _check_routing(oracle, ids, e, got)
    if t * k <= 65536:
        dev = ids.cuda()
        outs = (torch.empty(e, dtype=torch.int32, device="cuda"), torch.empty(e + 1, dtype=torch.int32, device="cuda"),
                torch.empty(t * k, dtype=torch.int32, device="cuda"),
                torch.empty(int(plan.num_blocks), dtype=torch.int32, device="cuda"))
        rc = _lib.lib().fso_moe_route_noalloc(_lib.ptr(dev), t, k, e, int(plan.num_blocks), *[_lib.ptr(o) for o in outs],
                                              _lib.stream_ptr())
        _lib.check(rc, "fso_moe_route_noalloc")
        _check_routing(oracle, ids, e, outs)
    del ctypes


def _device_events(prof):
    names = []
    for ev in prof.events():
        dt = getattr(ev, "device_type", None)
        if dt is not None and "CUDA" in str(dt):
            names.append(ev.name)
    return names


def test_refusals_launch_nothing(fso, device_ok):
    """Malformed calls raise before anything reaches the device: no kernel, memcpy or memset is recorded while they
    run, and the context is intact afterwards. A valid call inside the same kind of profile does record kernels
    (otherwise the profiler sees no device activity on this machine and the test is skipped)."""
    from torch.profiler import ProfilerActivity, profile

    n, k = 256, 512
    w = inputs.weight(n, k, 3).cuda()
    weight = fso.dense.prepare_weight(w, format="mxfp8")
    x = inputs.activation(32, k, 4).cuda()
    xq, sx = fso.dense.quantize_activation(x)
    ex = fso.moe.prepare_experts(inputs.weight(4 * 256, 256, 5).view(4, 256, 256).cuda(),
                                 inputs.weight(4 * 256, 128, 6).view(4, 256, 128).cuda(), format="mxfp8")
    ids, wts = inputs.routing(32, 4, 2, 7)
    hidden = inputs.activation(32, 256, 8).cuda()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as control:
        fso.dense.linear(x, weight)
        torch.cuda.synchronize()
    if not _device_events(control):
        pytest.skip("torch.profiler records no device activity here")

    misaligned_sx = torch.empty(sx.numel() + 1, dtype=torch.int32, device="cuda")[1:]
    # every operand of the calls below exists before the profile starts: what the profile records is the library's
    w_fp8 = w.to(torch.float8_e4m3fn)
    long_bias = torch.zeros(n + 1, dtype=torch.bfloat16, device="cuda")
    ids_d, wts_d, ids_short = ids.cuda(), wts.cuda(), ids[:5].cuda()
    torch.cuda.synchronize()
    bad_calls = [
        (ValueError, lambda: fso.dense.prepare_weight(w[:, :100], format="mxfp8")),
        (ValueError, lambda: fso.dense.prepare_weight(w, format="no-such-format")),
        (NotImplementedError, lambda: fso.dense.prepare_weight(w, format="nvfp4")),
        (ValueError, lambda: fso.dense.prepare_weight(w_fp8, format="mxfp8")),
        (TypeError, lambda: fso.dense.linear(x, w)),
        (ValueError, lambda: fso.dense.linear(x[:, :256], weight)),
        (ValueError, lambda: fso.dense.linear(xq, weight)),
        (ValueError, lambda: fso.dense.linear(x, weight, x_scale=sx)),
        (ValueError, lambda: fso.dense.linear(xq, weight, x_scale=sx[:-1])),
        (ValueError, lambda: fso.dense.linear(xq, weight, x_scale=misaligned_sx)),
        (ValueError, lambda: fso.dense.linear(x, weight, bias=long_bias)),
        (NotImplementedError, lambda: fso.dense.linear(x, weight, activation="silu")),
        (ValueError, lambda: fso.dense.linear(x, weight, activation="no-such-activation")),
        (ValueError, lambda: fso.dense.quantize_activation(x[:, :100])),
        (TypeError, lambda: fso.moe.layer(hidden, weight, ids_d, wts_d)),
        (ValueError, lambda: fso.moe.layer(hidden[:, :128], ex, ids_d, wts_d)),
        (ValueError, lambda: fso.moe.layer(hidden, ex, ids_short, wts_d)),
        (ValueError, lambda: fso.moe.transient_bytes(ex, -1, 2)),
    ]
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for exc, call in bad_calls:
            with pytest.raises(exc):
                call()
        torch.cuda.synchronize()
    assert _device_events(prof) == [], _device_events(prof)
    # the context is intact: the same valid call gives its bytes again
    assert torch.equal(fso.dense.linear(x, weight), fso.dense.linear(xq, weight, x_scale=sx))


def test_bounded_wait_sets_the_status_word(fso):
    """A device-side wait that cannot be satisfied ends by itself and reports through the status word; the context
    stays usable (the next GEMM runs and the word reads zero again)."""
    from fish_scales_ops_b200 import _lib, _ops

    assert _ops.device_status() == 0
    _lib.check(_lib.lib().fso_b200_selftest_wait_expires(2_000_000, _lib.stream_ptr()), "selftest")   # about 1 ms
    assert _ops.device_status() == 0x700
    assert _ops.device_status() == 0                     # reading clears it
    with pytest.raises(ValueError):
        _lib.check(_lib.lib().fso_b200_selftest_wait_expires(0, _lib.stream_ptr()), "selftest")
    weight = fso.dense.prepare_weight(inputs.weight(256, 512, 1).cuda(), format="mxfp8")
    y = fso.dense.linear(inputs.activation(16, 512, 2).cuda(), weight)
    assert torch.isfinite(y.float()).all() and _ops.device_status() == 0


def test_outputs_stay_inside_their_buffers(fso, device_ok):
    """Guard bands: every output of the C-ABI calls below sits inside a larger buffer filled with a canary byte; after
    the call the bytes before and after the output still hold the canary. Shapes with ragged last tiles (rows past M
    in the last 128-row tile, the second CTA of a CTA pair without rows, a decode-sized call, the quantizing and the
    SwiGLU epilogue)."""
    from fish_scales_ops_b200 import _ops
    from fish_scales_ops_b200._ops import check, lib, ptr, sf_words, stream_ptr

    guard = 4096
    canary = 0xA5

    def banded(nbytes):
        buf = torch.full((guard + nbytes + guard,), canary, dtype=torch.uint8, device="cuda")
        return buf, buf[guard:guard + nbytes]

    def intact(buf, nbytes, what):
        torch.cuda.synchronize()
        assert bool((buf[:guard] == canary).all()) and bool((buf[guard + nbytes:] == canary).all()), what

    g = torch.Generator(device="cuda").manual_seed(77)
    for m, n, k in ((200, 512, 256), (1920, 5120, 256), (2100, 4096, 512), (5, 4096, 1024), (16, 512, 4096)):
        x = torch.randn(m, k, generator=g, device="cuda", dtype=torch.bfloat16)
        w = (0.02 * torch.randn(n, k, generator=g, device="cuda")).to(torch.bfloat16)
        weight = fso.dense.prepare_weight(w, format="mxfp8")
        # activation quantizer: codes and scale words
        qbuf, q = banded(m * k)
        sbuf, s = banded(4 * sf_words(m, k))
        check(lib().fso_quantize_activation_1x32(ptr(x), ptr(q), ptr(s), m, k, stream_ptr()), "quantize")
        intact(qbuf, m * k, f"quantizer codes {m}x{k}")
        intact(sbuf, 4 * sf_words(m, k), f"quantizer scale words {m}x{k}")
        xq, sx = q.view(torch.float8_e4m3fn).view(m, k), s.view(torch.int32)
        # GEMM, bf16 output
        ws_bytes = _ops.gemm_ws_bytes(m, n, k)
        ws = torch.empty((max(ws_bytes, 1),), dtype=torch.uint8, device="cuda")
        ybuf, y = banded(2 * m * n)
        check(lib().fso_gemm_mxfp8(ptr(xq), ptr(sx), ptr(weight.weight), ptr(weight.scale), ptr(y), m, n, k, ptr(ws),
                                   ws_bytes, stream_ptr()), "gemm")
        intact(ybuf, 2 * m * n, f"bf16 output {m}x{n}x{k}")
        assert torch.equal(y.view(torch.bfloat16).view(m, n), fso.dense.linear(x, weight))
        # GEMM with the quantizing epilogue, where the shape takes it
        if _ops.gemm_fuses_quantized_output(m, n, k):
            obuf, o = banded(m * n)
            fbuf, f = banded(4 * sf_words(m, n))
            check(lib().fso_gemm_mxfp8_quantized(ptr(xq), ptr(sx), ptr(weight.weight), ptr(weight.scale), ptr(o), ptr(f),
                                                 m, n, k, None, 0, stream_ptr()), "gemm quantized")
            intact(obuf, m * n, f"quantized output {m}x{n}x{k}")
            intact(fbuf, 4 * sf_words(m, n), f"quantized output scale words {m}x{n}x{k}")
        # gate_up with the SwiGLU epilogue (normal orientation at every M)
        if n % 256 == 0:
            obuf, o = banded(m * (n // 2))
            fbuf, f = banded(4 * sf_words(m, n // 2))
            check(lib().fso_gemm_mxfp8_swiglu(ptr(xq), ptr(sx), ptr(weight.weight), ptr(weight.scale), ptr(o), ptr(f), m,
                                              n, k, stream_ptr()), "gemm swiglu")
            intact(obuf, m * (n // 2), f"SwiGLU output {m}x{n}x{k}")
            intact(fbuf, 4 * sf_words(m, n // 2), f"SwiGLU output scale words {m}x{n}x{k}")
    assert _ops.device_status() == 0


def test_print_tile_info_switch(device_ok):
    """FSO_PRINT_TILE_INFO=1 prints, once per kernel instantiation that is launched, the tile and the resources it
    asks for; nothing is printed without the variable (read once per process: child processes)."""
    import os
    import subprocess
    import sys

    code = ("import torch, fish_scales_ops_b200 as fso\n"
            "w = fso.dense.prepare_weight(torch.randn(512, 256, device='cuda').to(torch.bfloat16), format='mxfp8')\n"
            "x = torch.randn(256, 256, device='cuda').to(torch.bfloat16)\n"
            "for _ in range(3): fso.dense.linear(x, w)\n"
            "fso.dense.linear(x[:8], w)\n"
            "torch.cuda.synchronize()\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for flag, expect in (("1", True), (None, False)):
        env = {k: v for k, v in os.environ.items() if k != "FSO_PRINT_TILE_INFO"}
        if flag is not None:
            env["FSO_PRINT_TILE_INFO"] = flag
        res = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        lines = [ln for ln in res.stderr.splitlines() if ln.startswith("[fso_b200] gemm_mxf8")]
        if expect:
            assert len(lines) == 2 and len(set(lines)) == 2, lines     # one per instantiation, not one per call
            assert "normal orientation" in lines[0] and "swapped orientation" in lines[1], lines
        else:
            assert not lines, lines
