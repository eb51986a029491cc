"""The allocation-free routing entry point against the ordinary one, through the C ABI.

`fso_moe_route_noalloc` exists for callers that cannot give the library scratch memory and must not allocate while
they run (an engine that owns all device memory, code on a path where cudaMalloc would stall the stream). Its scratch
is an array inside the library image that every call shares and that keeps the previous call's contents, so the test
makes two different calls in a row and checks each against `fso_moe_route` bit for bit. This file sorts last on
purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def _route(L, fn_name, ids, e, nb, scratch_bytes):
    t, k = ids.shape
    dev = ids.device
    mm = torch.full((e,), -7, dtype=torch.int32, device=dev)
    b0 = torch.full((e + 1,), -7, dtype=torch.int32, device=dev)
    sl = torch.full((t * k,), -7, dtype=torch.int32, device=dev)
    be = torch.full((nb,), -7, dtype=torch.int32, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda x: ctypes.c_void_p(x.data_ptr())  # noqa: E731
    if fn_name == "fso_moe_route":
        scratch = torch.empty((max(scratch_bytes, 4),), dtype=torch.uint8, device=dev)
        rc = L.fso_moe_route(p(ids), t, k, e, nb, p(mm), p(b0), p(sl), p(be), p(scratch), scratch_bytes, st)
    else:
        rc = L.fso_moe_route_noalloc(p(ids), t, k, e, nb, p(mm), p(b0), p(sl), p(be), st)
    torch.cuda.synchronize()
    return rc, (mm, b0, sl, be)


def test_noalloc_routing_matches_ordinary_routing_twice(fso, device_ok):
    from fish_scales_ops_b200 import _lib, _ops

    L = _lib.lib()
    # two calls in a row with different sizes and expert counts: the second one finds the first one's leftovers
    for t, e, k, seed, skew in ((4096, 256, 8, 1, 0.0), (3000, 64, 4, 2, 1.2), (40, 8, 2, 3, 0.0)):
        ids = inputs.routing(t, e, k, seed, skew=skew)[0]
        ids[1, 0] = -1
        ids = ids.cuda()
        plan = _ops.moe_plan(t, k, e)
        nb = int(plan.num_blocks)
        rc_a, a = _route(L, "fso_moe_route", ids, e, nb, int(plan.route_scratch_bytes))
        rc_b, b = _route(L, "fso_moe_route_noalloc", ids, e, nb, 0)
        assert rc_a == 0 and rc_b == 0, _lib.last_error()
        for x, y, name in zip(a, b, ("masked_m", "blk0", "slot_of_flat", "blk_expert")):
            assert torch.equal(x, y), (name, t, e, k)


def test_noalloc_routing_refuses_what_it_cannot_hold(fso, device_ok):
    from fish_scales_ops_b200 import _lib, _ops

    L = _lib.lib()
    t, e, k = 16384, 8, 8      # 131072 pairs: beyond the built-in scratch
    ids = torch.zeros((t, k), dtype=torch.int32, device="cuda")
    plan = _ops.moe_plan(t, k, e)
    rc, _ = _route(L, "fso_moe_route_noalloc", ids, e, int(plan.num_blocks), 0)
    assert rc == -1 and "65536" in _lib.last_error()
