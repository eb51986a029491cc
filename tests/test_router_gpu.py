"""The fused router top-k against the CPU oracle and against torch's own softmax / topk on the GPU, in the cases
the reference's test covers (tests/gemm/unit/test_moe_router_topk.py: shapes up to 1024 experts, bf16 / fp32
logits, renormalize on and off, descending order, padded rows, expert map, shared gate, GEMM + top-k, graph
replay), plus exact ties, which the reference leaves unchecked. Ids must match exactly; weights within 1e-5
relative to the row's largest weight; the gate within 1e-6."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu

CASES = [(1, 256, 8), (7, 256, 8), (64, 128, 8), (512, 256, 8), (2048, 64, 8), (33, 1024, 8), (17, 256, 1),
         (129, 512, 4), (5, 8, 2), (40, 100, 6), (3, 1, 1)]
W_TOL = 1e-5


def _logits(m, e, seed, dtype):
    g = inputs.gen(seed)
    return (torch.randn(m, e, generator=g, dtype=torch.float32) * 3.0).to(dtype)


def _close(w, want):
    err = np.abs(w - want).max() / max(1e-12, float(np.abs(want).max()))
    assert err <= W_TOL, err


@pytest.mark.parametrize("m,e,k", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_topk_matches_oracle(fso, oracle, device_ok, m, e, k, dtype):
    logits = _logits(m, e, 1000 + 31 * m + e, dtype)
    for renorm in (True, False):
        ids, w, gate = fso.compat.moe_topk_from_logits(logits.cuda(), k, renormalize=renorm)
        assert ids.dtype == torch.int32 and w.dtype == torch.float32 and gate.numel() == 0
        want_ids, want_w, _ = oracle.router_topk(logits, k, renorm)
        assert np.array_equal(ids.cpu().numpy(), want_ids)
        _close(w.cpu().numpy(), want_w)
        if k > 1:
            assert bool((w[:, :-1] >= w[:, 1:]).all())
        # torch's own statement of the same thing, on the device
        probs = torch.softmax(logits.cuda().float(), dim=-1)
        tw, tids = torch.topk(probs, k, dim=-1)
        if renorm:
            tw = tw / tw.sum(dim=-1, keepdim=True)
        same = ids.to(torch.int64).sort(dim=-1).values == tids.sort(dim=-1).values
        if bool(same.all()):                       # bf16 / fp16 logits can tie at the boundary, where torch may differ
            order, torder = ids.to(torch.int64).argsort(dim=-1), tids.argsort(dim=-1)
            _close(torch.gather(w, 1, order).cpu().numpy(), torch.gather(tw, 1, torder).cpu().numpy())
        else:
            assert dtype != torch.float32


def test_exact_ties_go_to_the_lower_id(fso, oracle, device_ok):
    logits = torch.zeros(6, 96, dtype=torch.float32)
    logits[1, [70, 5, 40, 41]] = 2.0                      # four equal maxima across and inside lanes
    logits[2] = torch.arange(96, dtype=torch.float32).flip(0) // 4     # runs of four equal values
    logits[3, 95] = 1.0
    logits[4, :] = -float("inf")
    logits[4, [9, 50]] = -1.0
    logits[5, 64:] = 1.5
    ids, w, _ = fso.compat.moe_topk_from_logits(logits.cuda(), 8)
    want_ids, want_w, _ = oracle.router_topk(logits, 8)
    assert np.array_equal(ids.cpu().numpy()[[0, 1, 2, 3, 5]], want_ids[[0, 1, 2, 3, 5]])
    assert ids[0].tolist() == list(range(8))
    assert ids[1].tolist()[:4] == [5, 40, 41, 70]
    assert ids[4].tolist()[:2] == [9, 50]
    _close(w.cpu().numpy()[[0, 1, 2, 3, 5]], want_w[[0, 1, 2, 3, 5]])


@pytest.mark.parametrize("m,e,k", [(7, 256, 8), (64, 128, 8), (33, 1024, 8), (129, 512, 4)])
def test_padded_rows_expert_map_and_shared_gate(fso, oracle, device_ok, m, e, k):
    logits = _logits(m, e, 77 + m, torch.bfloat16)
    ids, w, _ = fso.compat.moe_topk_from_logits(logits.cuda(), k)
    n_real = max(1, m // 2)
    n_valid = torch.tensor([n_real], dtype=torch.int32, device="cuda")
    ids_p, w_p, _ = fso.compat.moe_topk_from_logits(logits.cuda(), k, num_token_non_padded=n_valid)
    assert torch.equal(ids_p[:n_real], ids[:n_real]) and torch.equal(w_p[:n_real], w[:n_real])
    assert bool((ids_p[n_real:] == e).all()) and bool((w_p[n_real:] == 0).all())
    e_local = e // 2
    emap = torch.full((e + 1,), -1, dtype=torch.int32)
    emap[:e_local] = torch.arange(e_local, dtype=torch.int32)
    emap[e] = e_local
    ids_m, w_m, _ = fso.compat.moe_topk_from_logits(logits.cuda(), k, num_token_non_padded=n_valid,
                                                    expert_map=emap.cuda())
    assert torch.equal(ids_m[:n_real].cpu(), emap[ids_p[:n_real].cpu().to(torch.int64)])
    assert bool((ids_m[n_real:] == e_local).all()) and torch.equal(w_m, w_p)
    want = oracle.router_topk(logits, k, True, False, n_real, emap)
    assert np.array_equal(ids_m.cpu().numpy(), want[0])
    extra = (torch.randn(m, 1, generator=inputs.gen(5), dtype=torch.float32) * 2.0).to(torch.bfloat16)
    wide = torch.cat([logits, extra], dim=1)
    ids_s, w_s, gate = fso.compat.moe_topk_from_logits(wide.cuda(), k, with_shared_gate=True)
    assert torch.equal(ids_s, ids) and torch.equal(w_s, w)
    assert float((gate.cpu() - torch.sigmoid(extra.float().squeeze(1))).abs().max()) <= 1e-6
    # a row-major slice with a longer row stride is accepted as it is
    ids_v, w_v, _ = fso.compat.moe_topk_from_logits(wide.cuda()[:, :e], k)
    assert torch.equal(ids_v, ids) and torch.equal(w_v, w)


def test_router_gemm_plus_topk_and_graph_replay(fso, oracle, device_ok):
    m, e, h, k = 64, 256, 2048, 8
    g = inputs.gen(7)
    hidden = torch.randn(m, h, generator=g, dtype=torch.float32).to(torch.bfloat16).cuda()
    rw = (torch.randn(e + 1, h, generator=g, dtype=torch.float32) * 0.05).to(torch.bfloat16).cuda()
    ids, w, gate = fso.compat.moe_router_topk(hidden, rw, k, with_shared_gate=True)
    logits = torch.nn.functional.linear(hidden, rw)
    want_ids, want_w, want_gate = oracle.router_topk(logits, k, True, True)
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    _close(w.cpu().numpy(), want_w)
    assert float(np.abs(gate.cpu().numpy() - want_gate).max()) <= 1e-6
    # the router feeds the layer: ids / weights are what fso.moe.layer takes
    buf = _logits(64, 256, 9, torch.bfloat16).cuda()
    n_valid = torch.tensor([64], dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fso.compat.moe_topk_from_logits(buf, 8, num_token_non_padded=n_valid)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ids_g, w_g, _ = fso.compat.moe_topk_from_logits(buf, 8, num_token_non_padded=n_valid)
    torch.cuda.current_stream().wait_stream(side)
    new = _logits(64, 256, 10, torch.bfloat16)
    buf.copy_(new.cuda())
    n_valid.fill_(40)
    graph.replay()
    torch.cuda.synchronize()
    want_ids, want_w, _ = oracle.router_topk(new, 8, True, False, 40)
    assert np.array_equal(ids_g.cpu().numpy(), want_ids)
    _close(w_g.cpu().numpy(), want_w)


def test_router_refusals(fso, device_ok):
    lg = _logits(4, 16, 1, torch.bfloat16).cuda()
    with pytest.raises(ValueError):
        fso.compat.moe_topk_from_logits(lg, 9)
    with pytest.raises(ValueError):
        fso.compat.moe_topk_from_logits(lg[:, :4], 8)
    with pytest.raises(ValueError):
        fso.compat.moe_topk_from_logits(lg.t(), 2)
    with pytest.raises(ValueError):
        fso.compat.moe_topk_from_logits(lg.to(torch.float64), 2)
    with pytest.raises(ValueError):
        fso.compat.moe_topk_from_logits(lg, 2, expert_map=torch.zeros(16, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        fso.compat.moe_topk_from_logits(lg, 2, num_token_non_padded=torch.zeros(1, dtype=torch.int64, device="cuda"))
    ids, w, gate = fso.compat.moe_topk_from_logits(lg[:0], 2)
    assert ids.shape == (0, 2) and w.shape == (0, 2)
