"""The two ways the path shards, on two GPUs of one box (skipped with fewer): the column-parallel N-split of a dense
linear (no collective) and the expert-parallel MoE layer, once with the rows stored into the peer GPU's memory by the
library's kernels and once with NCCL all-to-all-v dispatch and combine. Each rank is a child process; NVLS is
switched off for NCCL in them and no multicast object is created for the symmetric buffers."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import inputs

pytestmark = pytest.mark.gpu

E, K, H, I, T = 16, 4, 512, 256, 300
N_DENSE, K_DENSE, M_DENSE = 1024, 512, 200


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _moe_weights():
    return inputs.weight(E * 2 * I, H, 31).view(E, 2 * I, H), inputs.weight(E * H, I, 32).view(E, H, I)


def _moe_batch(rank):
    hidden = inputs.activation(T + 8 * rank, H, 40 + rank)
    ids, wts = inputs.routing(T + 8 * rank, E, K, 50 + rank)
    return hidden, ids, wts


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import fish_scales_ops_b200 as fso
        from fish_scales_ops_b200 import _ops, parallel

        # dense N-split: this rank's rows of the weight, the same activation, no exchange
        w = inputs.weight(N_DENSE, K_DENSE, 7)
        x = inputs.activation(M_DENSE, K_DENSE, 8).cuda()
        r0, r1 = parallel.column_shard(N_DENSE, world, rank)
        y_part = fso.dense.linear(x, fso.dense.prepare_weight(w[r0:r1].cuda(), format="mxfp8"))
        # expert-parallel MoE
        w13, w2 = _moe_weights()
        e0, e1 = parallel.expert_shard(E, world, rank)
        experts = fso.moe.prepare_experts(w13[e0:e1].cuda(), w2[e0:e1].cuda(), format="mxfp8")
        hidden, ids, wts = _moe_batch(rank)
        hidden, ids, wts = hidden.cuda(), ids.cuda(), wts.cuda()
        out = parallel.expert_parallel_layer(hidden, experts, ids, wts, num_experts_global=E, transport="peer")
        # the receive buffers are reused: another batch in between, then the first one again
        other = parallel.expert_parallel_layer(hidden.flip(0).contiguous(), experts, ids, wts, num_experts_global=E,
                                               transport="peer")
        again = parallel.expert_parallel_layer(hidden, experts, ids, wts, num_experts_global=E)
        coll = parallel.expert_parallel_layer(hidden, experts, ids, wts, num_experts_global=E, transport="collective")
        # several layers back to back with different routings and token counts (the receive buffers and the fences are
        # reused from call to call): the peer transport must give the collective transport's bytes every time
        rounds = []
        for r in range(4):
            t_r = 64 + 57 * r + 16 * rank
            h_r = inputs.activation(t_r, H, 300 + 10 * r + rank).cuda()
            ids_r, w_r = inputs.routing(t_r, E, K, 400 + 10 * r + rank, skew=1.2 if r % 2 else 0.0)
            ids_r, w_r = ids_r.cuda(), w_r.cuda()
            a = parallel.expert_parallel_layer(h_r, experts, ids_r, w_r, num_experts_global=E, transport="peer")
            b = parallel.expert_parallel_layer(h_r, experts, ids_r, w_r, num_experts_global=E, transport="collective")
            rounds.append(bool(torch.equal(a, b)))
        torch.cuda.synchronize()
        ret[rank] = (y_part.cpu(), out.cpu(), _ops.device_status(), again.cpu(), coll.cpu(), other.cpu(), rounds)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_n_split_and_expert_parallel_on_two_gpus(fso, oracle):
    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    # dense: the concatenated column slices equal the single-GPU result within the output tolerance
    w = inputs.weight(N_DENSE, K_DENSE, 7)
    x = inputs.activation(M_DENSE, K_DENSE, 8)
    full = fso.dense.prepare_weight(w.cuda(), format="mxfp8")
    ref = oracle.dense_linear(x, inputs.to_np_u8(full.weight), inputs.to_np_u32(full.scale))
    y = torch.cat([ret[0][0], ret[1][0]], dim=1)
    inputs.assert_close_to_oracle(y, ref, "N-split")
    # MoE: every rank's tokens get the full layer over all experts
    w13, w2 = _moe_weights()
    ex = fso.moe.prepare_experts(w13.cuda(), w2.cuda(), format="mxfp8")
    for rank in range(world):
        hidden, ids, wts = _moe_batch(rank)
        want = oracle.moe_layer(hidden, inputs.to_np_u8(ex.w13), inputs.to_np_u32(ex.sw13), inputs.to_np_u8(ex.w2),
                                inputs.to_np_u32(ex.sw2), ids, wts)
        inputs.assert_close_to_oracle(ret[rank][1], want, f"expert parallel rank {rank}")
        assert ret[rank][2] == 0
        # same bytes on a second use of the buffers and through the collective transport
        assert torch.equal(ret[rank][1].view(torch.int16), ret[rank][3].view(torch.int16))
        assert torch.equal(ret[rank][1].view(torch.int16), ret[rank][4].view(torch.int16))
        assert not torch.equal(ret[rank][1].view(torch.int16), ret[rank][5].view(torch.int16))
        assert ret[rank][6] == [True] * 4, ret[rank][6]
