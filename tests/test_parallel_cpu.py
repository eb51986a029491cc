"""Host-side logic of the multi-GPU path, run as two gloo ranks on the CPU: the expert-parallel dispatch / combine
around a stand-in local layer reproduces the single-process layer, and the shard helpers refuse bad splits."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import inputs

E, K, H, I, T = 8, 2, 64, 32, 37


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _weights():
    g = inputs.gen(5)
    w13 = 0.1 * torch.randn(E, 2 * I, H, generator=g)
    w2 = 0.1 * torch.randn(E, H, I, generator=g)
    return w13, w2


def _layer_cpu(hidden, experts, ids, wts):
    """Stand-in for fso.moe.layer on the CPU: local experts (w13 [gate; up], w2), ids outside [0, E_local) skipped."""
    w13, w2 = experts
    out = torch.zeros(hidden.shape[0], hidden.shape[1])
    for e in range(w13.shape[0]):
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        a = hidden[tok].float() @ w13[e].t()
        hh = torch.nn.functional.silu(a[:, :I]) * a[:, I:]
        out.index_add_(0, tok, (hh @ w2[e].t()) * wts[tok, slot][:, None])
    return out.to(torch.bfloat16)


def _combine_cpu(back, slot, ones):
    """Stand-in for the combine kernel: fp32 sum of the partial rows in rank order, one rounding to bf16."""
    out = torch.zeros(slot.shape[0], back.shape[1])
    for r in range(slot.shape[1]):
        sel = slot[:, r] >= 0
        out[sel] += back[slot[sel, r].long()].float()
    return out.to(torch.bfloat16)


def _batch(rank):
    hidden = inputs.activation(T + rank, H, 100 + rank)
    ids, wts = inputs.routing(T + rank, E, K, 200 + rank)
    ids = ids.clone()
    ids[0, 0] = -1          # a padded entry: belongs to no rank
    if rank == 1:
        ids[3] = torch.tensor([6, 7], dtype=torch.int32)   # a token whose experts all live on rank 1
    return hidden, ids, wts


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fish_scales_ops_b200 import parallel

        w13, w2 = _weights()
        e0, e1 = parallel.expert_shard(E, world, rank)
        hidden, ids, wts = _batch(rank)
        plan = parallel.build_dispatch(ids, E // world, world)
        out = parallel.expert_parallel_layer(hidden, (w13[e0:e1], w2[e0:e1]), ids, wts, num_experts_global=E,
                                             layer_fn=_layer_cpu, combine_fn=_combine_cpu)
        out3 = parallel.expert_parallel_layer(hidden, (w13[e0:e1], w2[e0:e1]), ids, wts, num_experts_global=E,
                                              layer_fn=_layer_cpu, combine_fn=_combine_cpu, micro_batches=3)
        assert torch.equal(out, out3), "slicing the tokens into micro-batches must not change a single byte"
        ret[rank] = (out, plan.send_counts, plan.recv_counts, parallel.dispatch_bytes(plan, rank, H, K))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_two_ranks():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    w13, w2 = _weights()
    for rank in range(world):
        hidden, ids, wts = _batch(rank)
        want = _layer_cpu(hidden, (w13, w2), ids, wts).float()
        out, send, recv, nbytes = ret[rank]
        assert out.dtype == torch.bfloat16 and tuple(out.shape) == tuple(hidden.shape)
        assert torch.allclose(out.float(), want, rtol=3e-2, atol=3e-2 * float(want.abs().max()))
        # every token is sent to each rank owning one of its experts, once
        owner = torch.where((ids >= 0) & (ids < E), ids // (E // world), torch.full_like(ids, -1))
        for r in range(world):
            assert send[r] == int((owner == r).any(dim=1).sum())
        assert nbytes == send[1 - rank] * (H * 2 + K * 8) + send[1 - rank] * H * 2
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0, and vice versa
    assert ret[0][1][1] == ret[1][2][0] and ret[1][1][0] == ret[0][2][1]


def test_shard_helpers():
    from fish_scales_ops_b200 import parallel

    for n in (6144, 28672, 4096):
        for g in (1, 2, 4, 8):
            spans = [parallel.column_shard(n, g, r) for r in range(g)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all((b - a) % 128 == 0 for a, b in spans)
    with pytest.raises(ValueError):
        parallel.column_shard(4096, 3, 0)
    with pytest.raises(ValueError):
        parallel.column_shard(384, 2, 0)      # 192 rows per rank: not a multiple of 128
    with pytest.raises(ValueError):
        parallel.column_shard(4096, 2, 2)
    assert parallel.expert_shard(256, 8, 3) == (96, 128)
    with pytest.raises(ValueError):
        parallel.expert_shard(10, 4, 0)


def test_transport_argument_is_checked_before_any_collective():
    """An unknown transport, and the peer transport asked for together with what only the collective one takes,
    are refused without touching the process group (none exists here)."""
    from fish_scales_ops_b200 import parallel

    h = torch.zeros(4, 128, dtype=torch.bfloat16)
    ids = torch.zeros(4, 2, dtype=torch.int32)
    w = torch.ones(4, 2)
    with pytest.raises(ValueError):
        parallel.expert_parallel_layer(h, None, ids, w, num_experts_global=8, transport="carrier pigeon")
    with pytest.raises(ValueError):
        parallel.expert_parallel_layer(h, None, ids, w, num_experts_global=8, transport="peer",
                                       layer_fn=lambda *a: None)
    with pytest.raises(ValueError):
        parallel.expert_parallel_layer(h, None, ids, w, num_experts_global=8, transport="peer", micro_batches=2)


def test_peer_buffer_layout_is_aligned_and_disjoint():
    from fish_scales_ops_b200 import parallel

    for world, cap, h, k in ((2, 1024, 512, 4), (8, 4096, 7168, 8), (4, 1024, 4096, 2)):
        offs, total = parallel._PeerBuffers.layout(world, cap, h, k)
        rows, back = world * cap, cap * min(k, world)
        sizes = {"q": rows * h, "w": rows * (h // 128) * 4, "ids": rows * k * 4, "wt": rows * k * 4,
                 "back": back * h * 2}
        spans = sorted((offs[n], offs[n] + sizes[n]) for n in sizes)
        assert all(o % 256 == 0 for o, _ in spans)
        assert all(spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1))
        assert spans[-1][1] <= total
