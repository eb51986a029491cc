"""The expert-parallel exchange kernels on ONE GPU: the "ranks" are separate buffer sets in the same device memory
and their steps run one after the other on one stream, so no kernel ever waits for another. The plan kernels are
checked against the same logic written with numpy, the whole exchange against the library's single-GPU layer run
once per (source rank, expert rank) and added in rank order."""
import numpy as np
import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu

E, K, H, I = 16, 4, 512, 256
WORLD = 4
PER = E // WORLD
TOKENS = [200, 131, 0, 260]


def _ids(rank):
    ids, wts = inputs.routing(max(TOKENS[rank], 1), E, K, 70 + rank)
    ids, wts = ids[:TOKENS[rank]].clone(), wts[:TOKENS[rank]].clone()
    if TOKENS[rank] > 8:
        ids[3, 1] = -1            # nobody's expert
        ids[5, 0] = E + 2         # out of range: nobody's either
        ids[7] = -1               # a token no rank needs
    return ids, wts


def _needs(ids):
    owner = np.where((ids >= 0) & (ids < E), ids // PER, -1)
    return np.stack([(owner == r).any(axis=1) for r in range(WORLD)], axis=0)        # [G, T]


def _plan_all(device_ok):
    from fish_scales_ops_b200 import _ops

    masks, rows = [], []
    for r in range(WORLD):
        ids, _ = _ids(r)
        m, row = _ops.ep_plan_count(ids.cuda(), PER, WORLD)
        masks.append(m)
        rows.append(row)
    return masks, torch.stack(rows)


def test_plan_kernels_match_host_logic(fso, device_ok):
    from fish_scales_ops_b200 import _ops

    masks, table = _plan_all(device_ok)
    needs = [_needs(_ids(r)[0].numpy()) for r in range(WORLD)]
    want_table = np.array([[int(n[d].sum()) for d in range(WORLD)] + [TOKENS[r]] for r, n in enumerate(needs)])
    assert np.array_equal(table.cpu().numpy(), want_table)
    for r in range(WORLD):
        want_mask = sum((needs[r][d].astype(np.int64) << d) for d in range(WORLD))
        assert np.array_equal(masks[r].cpu().numpy(), want_mask)
    cm = want_table[:, :WORLD]
    for r in range(WORLD):
        send_total = int(cm[r].sum())
        send_token, send_rank, send_off, dst_base, recv_off, back_base, slot = _ops.ep_plan_place(
            masks[r], table, WORLD, r, send_total)
        dst, tok = np.nonzero(needs[r])                      # rank-major, tokens ascending
        assert np.array_equal(send_rank.cpu().numpy(), dst)
        assert np.array_equal(send_token.cpu().numpy(), tok)
        assert np.array_equal(send_off.cpu().numpy(), np.cumsum(cm[r]) - cm[r])
        assert np.array_equal(dst_base.cpu().numpy(), cm[:r].sum(axis=0))
        assert np.array_equal(recv_off.cpu().numpy(), np.concatenate([[0], np.cumsum(cm[:, r])]))
        assert np.array_equal(back_base.cpu().numpy(), (np.cumsum(cm, axis=1) - cm)[:, r])
        pos = (np.cumsum(needs[r].reshape(-1)) - 1).reshape(WORLD, -1)
        assert np.array_equal(slot.cpu().numpy(), np.where(needs[r], pos, -1).T)


def test_exchange_on_one_gpu_equals_per_rank_layers_added_in_rank_order(fso, device_ok):
    from fish_scales_ops_b200 import _ops, parallel

    dev = torch.device("cuda")
    w13 = inputs.weight(E * 2 * I, H, 31).view(E, 2 * I, H)
    w2 = inputs.weight(E * H, I, 32).view(E, H, I)
    experts = [fso.moe.prepare_experts(w13[r * PER:(r + 1) * PER].cuda(), w2[r * PER:(r + 1) * PER].cuda(),
                                       format="mxfp8") for r in range(WORLD)]
    hidden = [inputs.activation(TOKENS[r], H, 60 + r).cuda() for r in range(WORLD)]
    routing = [tuple(t.cuda() for t in _ids(r)) for r in range(WORLD)]

    cap = 512
    _, total = parallel._PeerBuffers.layout(WORLD, cap, H, K)
    raw = [torch.zeros((total,), dtype=torch.uint8, device=dev) for _ in range(WORLD)]
    bases = [b.data_ptr() for b in raw]
    bufs = [parallel._PeerBuffers(WORLD, cap, H, K, dev, emulated_bases=bases, buf=raw[r]) for r in range(WORLD)]

    for _ in range(2):                                         # the second pass reuses the buffers
        masks, table = _plan_all(device_ok)
        host = table.tolist()
        states = [parallel._peer_dispatch(hidden[r], routing[r][0], routing[r][1], masks[r], table, host, r, WORLD,
                                          PER, bufs[r]) for r in range(WORLD)]
        for r in range(WORLD):
            parallel._peer_local(states[r], experts[r], bufs[r])
        outs = [parallel._peer_reduce(states[r], bufs[r]) for r in range(WORLD)]
        torch.cuda.synchronize()
        assert _ops.device_status() == 0

        for r in range(WORLD):
            ids, wts = routing[r]
            acc = torch.zeros((TOKENS[r], H), dtype=torch.float32, device=dev)
            for s in range(WORLD):
                local = torch.where((ids >= s * PER) & (ids < (s + 1) * PER), ids - s * PER, torch.full_like(ids, -1))
                if TOKENS[r] > 0:
                    acc += fso.moe.layer(hidden[r], experts[s], local, wts).float()
            assert outs[r].shape == (TOKENS[r], H)
            assert torch.equal(outs[r].view(torch.int16), acc.to(torch.bfloat16).view(torch.int16)), f"rank {r}"
