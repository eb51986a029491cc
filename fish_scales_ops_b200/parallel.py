"""Multi-GPU use of the path, one process per GPU over ``torch.distributed``.

The reference has no communication code: tensor- and expert-parallel callers shard the weights themselves and
reduce the partial results (docs/guide.md:139-141, python/fish_scales_ops/moe/__init__.py:733-739). Two helpers
cover the two ways the path shards:

* dense linears split along N (column parallel): every rank prepares its own rows of the weight and computes its
  own output columns from the same activation; there is no exchange step, so nothing here calls a collective;
* MoE layers split by expert (expert parallel): rank r owns experts ``[r*E/G, (r+1)*E/G)``. Each token row is
  sent once to every rank that owns at least one of its top-k experts (all-to-all-v dispatch), the local layer runs
  with the ids of other ranks' experts rewritten to -1 (the layer skips them at no cost and returns a partial sum),
  the partial rows travel back (all-to-all-v combine) and the source rank adds them in rank order in fp32.

Kernels only ever READ this GPU's memory. With the default transport the rows are stored into the destination GPU's
receive buffers by this library's own kernels (plain peer stores, ordered by two stream-ordered collectives); with
``transport="collective"`` they travel through NCCL all-to-all-v. Either way a kernel touches a row only once it
lies in its own GPU's memory.
"""
import dataclasses
import os
from typing import Callable, Optional

import torch
import torch.distributed as dist


def column_shard(n: int, world: int, rank: int):
    """Rows ``[r0, r1)`` of an ``[N, K]`` weight that rank ``rank`` of ``world`` serves (N-split). Every shard must
    keep ``N / world`` a multiple of 128, which the MXFP8 GEMM requires."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"column_shard: rank {rank} of world {world}")
    if n % world != 0 or (n // world) % 128 != 0:
        raise ValueError(f"column_shard: N = {n} split {world} ways leaves {n / world:g} rows per rank, which is not "
                         f"a multiple of 128")
    per = n // world
    return rank * per, (rank + 1) * per


def expert_shard(num_experts: int, world: int, rank: int):
    """Experts ``[e0, e1)`` owned by ``rank`` under expert parallelism."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"expert_shard: rank {rank} of world {world}")
    if num_experts % world != 0:
        raise ValueError(f"expert_shard: {num_experts} experts do not split evenly over {world} ranks")
    per = num_experts // world
    return rank * per, (rank + 1) * per


@dataclasses.dataclass
class DispatchPlan:
    """What one rank sends where, for one batch. Row i of the send buffer is token ``send_token[i]`` bound for rank
    ``send_rank[i]``; the rows for destination rank r are the contiguous range given by ``send_counts``."""

    send_token: torch.Tensor          # int64 [S]: source token of each sent row, grouped by destination rank
    send_rank: torch.Tensor           # int64 [S]: destination rank of each sent row (non-decreasing)
    send_counts: list                 # python ints [G]
    recv_counts: list                 # python ints [G]


def build_dispatch(topk_ids: torch.Tensor, experts_per_rank: int, world: int, group=None) -> DispatchPlan:
    """Which token goes to which rank: a token is sent to rank r when at least one of its top-k ids lies in r's
    expert range (ids outside ``[0, E_global)`` belong to nobody). Rows are grouped by destination rank with the
    tokens ascending inside a group (deterministic). One small count exchange tells every rank how many rows it will
    receive; its result is the only host read of the exchange."""
    t = int(topk_ids.shape[0])
    ids = topk_ids.to(torch.int64)
    valid = (ids >= 0) & (ids < experts_per_rank * world)
    owner = torch.where(valid, ids // experts_per_rank, torch.full_like(ids, -1))
    ranks = torch.arange(world, device=ids.device, dtype=torch.int64)
    needs = (owner.unsqueeze(-1) == ranks).any(dim=1)                      # [T, G]
    flat = needs.t().reshape(-1)                                            # rank-major
    # stable sort puts the needed (rank, token) pairs first, in rank-major / token-ascending order; no host read
    order = torch.sort((~flat).to(torch.int8), stable=True).indices
    counts = needs.sum(dim=0).to(torch.int64)
    recv = torch.empty_like(counts)
    dist.all_to_all_single(recv, counts, group=group)
    both = torch.cat([counts, recv]).tolist()                               # the one host read
    send_counts, recv_counts = [int(v) for v in both[:world]], [int(v) for v in both[world:]]
    order = order[:sum(send_counts)]
    return DispatchPlan(order % t, order // t, send_counts, recv_counts)


def _a2a_rows(rows: torch.Tensor, in_counts, out_counts, group) -> torch.Tensor:
    out = rows.new_empty((sum(out_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(out_counts),
                           input_split_sizes=list(in_counts), group=group)
    return out


def _combine_partials(back: torch.Tensor, slot: torch.Tensor, ones: torch.Tensor) -> torch.Tensor:
    """out[t] = bf16(sum over ranks r, ascending, of back[slot[t, r]]) with the library's combine kernel (fp32
    accumulation in rank order, one rounding; slot -1 = no partial from that rank)."""
    from . import _ops

    out = torch.empty((slot.shape[0], back.shape[1]), dtype=torch.bfloat16, device=back.device)
    if back.shape[0] == 0:
        return out.zero_()
    _ops.moe_combine(back, slot.reshape(-1), ones, None, None, out)
    return out


def _a2a_rows_async(rows: torch.Tensor, in_counts, out_counts, group):
    out = rows.new_empty((sum(out_counts),) + tuple(rows.shape[1:]))
    work = dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(out_counts),
                                  input_split_sizes=list(in_counts), group=group, async_op=True)
    return out, work


# ------------------------------------------------------------------------------- the exchange over peer memory

def _align_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class _PeerBuffers:
    """Receive buffers of one rank, allocated as symmetric memory so that every rank of the group holds the
    addresses of every other rank's copy: dispatch rows (e4m3 codes, scale words, ids, weights) for up to
    ``world * cap_tokens`` rows and combine rows (bf16) for up to ``cap_tokens * min(k, world)`` rows. Only plain
    peer stores touch them (no multicast object is created)."""

    def __init__(self, world: int, cap_tokens: int, h: int, k: int, device, group=None, emulated_bases=None,
                 buf=None):
        """With ``group``: a collective symmetric allocation. With ``buf`` / ``emulated_bases`` (tests): this
        "rank"'s buffer is the given plain tensor and the ranks' base addresses are given, all on one device."""
        self.cap_tokens, self.h, self.k, self.world = cap_tokens, h, k, world
        cap_rows = world * cap_tokens
        cap_back = cap_tokens * min(k, world)
        kb = h // 128
        offs, total = self.layout(world, cap_tokens, h, k)
        if buf is None:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm

            self.buf = symm.empty(total, dtype=torch.uint8, device=device)
            handle = symm.rendezvous(self.buf, dist.group.WORLD if group is None else group)
            bases = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
        else:
            self.buf, bases = buf, [int(b) for b in emulated_bases]

        def table(name):
            return torch.tensor([b + offs[name] for b in bases], dtype=torch.int64, device=device)

        def view(name, n):
            return self.buf[offs[name]:offs[name] + n]

        self.peer_q, self.peer_w, self.peer_ids = table("q"), table("w"), table("ids")
        self.peer_wt, self.peer_back = table("wt"), table("back")
        self.rx_q = view("q", cap_rows * h).view(torch.float8_e4m3fn).view(cap_rows, h)
        self.rx_w = view("w", cap_rows * kb * 4).view(torch.int32).view(cap_rows, kb)
        self.rx_ids = view("ids", cap_rows * k * 4).view(torch.int32).view(cap_rows, k)
        self.rx_wt = view("wt", cap_rows * k * 4).view(torch.float32).view(cap_rows, k)
        self.rx_back = view("back", cap_back * h * 2).view(torch.bfloat16).view(cap_back, h)
        self.fence_word = torch.zeros((1,), dtype=torch.float32, device=device)
        self.ones = torch.ones((cap_tokens, world), dtype=torch.float32, device=device)

    @staticmethod
    def layout(world: int, cap_tokens: int, h: int, k: int):
        """Byte offsets of the five regions inside one rank's buffer, and the buffer's size."""
        cap_rows = world * cap_tokens
        cap_back = cap_tokens * min(k, world)
        sizes = [("q", cap_rows * h), ("w", cap_rows * (h // 128) * 4), ("ids", cap_rows * k * 4),
                 ("wt", cap_rows * k * 4), ("back", cap_back * h * 2)]
        offs, total = {}, 0
        for name, n in sizes:
            offs[name] = total
            total = _align_up(total + n, 256)
        return offs, total


_PEER_BUFFERS = {}
_RETIRED_BUFFERS = []     # outgrown buffers stay mapped: a peer may still have stores to them in flight


def _peer_buffers(group, world: int, tokens_max: int, h: int, k: int, device) -> _PeerBuffers:
    """The buffers for this (group, H, k), grown (by at least 2x) when a batch needs more rows than they hold.
    ``tokens_max`` is the largest token count over the ranks, which every rank knows, so that every rank takes the
    same decision and the collective allocation matches."""
    # keyed on the group's member ranks, not on id(group): Python may hand a destroyed group's id to a new one
    members = tuple(dist.get_process_group_ranks(group)) if group is not None else ("world", world)
    key = (members, h, k, str(device))
    have = _PEER_BUFFERS.get(key)
    if have is not None and have.cap_tokens >= tokens_max:
        return have
    cap = _align_up(max(tokens_max, 1), 1024)
    if have is not None:
        cap = max(cap, 2 * have.cap_tokens)
        _RETIRED_BUFFERS.append(have)
    _PEER_BUFFERS[key] = _PeerBuffers(world, cap, h, k, device, group=group)
    return _PEER_BUFFERS[key]


def _fence(bufs: _PeerBuffers, group) -> None:
    """Orders the ranks on their streams: the collective completes on a rank only after every rank's stream has
    reached it, that is after every rank's earlier kernels (and their peer stores) have completed."""
    dist.all_reduce(bufs.fence_word, group=group)


# Phase trace of the peer transport (measurement only): when this is a list, every phase boundary of
# _expert_parallel_peer appends (name, CUDA event recorded on the current stream).
PHASE_TRACE = None


def _mark(name: str) -> None:
    if PHASE_TRACE is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        PHASE_TRACE.append((name, ev))


def _expert_parallel_peer(hidden, experts, topk_ids, topk_w, per: int, world: int, group) -> torch.Tensor:
    """Expert parallelism with the rows stored straight into the destination GPU's memory.

    1. every rank quantizes its tokens once (codes + scale words; half the bytes of the bf16 rows on the wire) and
       counts its rows per destination (one kernel); one all-gather of the counts gives every rank the full
       world x world table (the only host read), from which a second kernel derives every offset, the send list and
       the slot table of step 4;
    2. the dispatch kernel stores each sent row (codes, scale words, local ids, weights) into the destination's
       receive buffers;
    3. after a fence the local layer runs over the received rows (its gather copies the codes instead of quantizing)
       and its combine kernel stores each partial row into the source rank's receive buffer, at the position the row
       had in the source's send order;
    4. after a second fence the source adds a token's partial rows in rank order (fp32, one rounding)."""
    from . import _ops

    rank = dist.get_rank(group)
    t, h, k = int(hidden.shape[0]), int(hidden.shape[1]), int(topk_ids.shape[1])
    _mark("start")
    ids32 = topk_ids.to(torch.int32).contiguous()
    w32 = topk_w.to(torch.float32).contiguous()
    mask, row = _ops.ep_plan_count(ids32, per, world)
    table = torch.empty((world, world + 1), dtype=torch.int64, device=hidden.device)
    dist.all_gather_into_tensor(table, row, group=group)
    _mark("plan count + all-gather")
    quantized = _ops.quantize_1x32_fp8(hidden) if t > 0 else None            # runs while the host waits below
    _mark("quantize")
    host = table.tolist()                                                     # the one host read
    bufs = _peer_buffers(group, world, max(r[world] for r in host), h, k, hidden.device)
    _mark("host read")
    st = _peer_dispatch(hidden, ids32, w32, mask, table, host, rank, world, per, bufs, quantized)
    _mark("plan place + dispatch")
    _fence(bufs, group)
    _mark("fence")
    _peer_local(st, experts, bufs)
    _mark("local layer incl. scatter combine")
    _fence(bufs, group)
    _mark("fence 2")
    out = _peer_reduce(st, bufs)
    _mark("final reduce")
    return out


def _peer_dispatch(hidden, ids32, w32, mask, table, host, rank: int, world: int, per: int, bufs: _PeerBuffers,
                   quantized=None) -> dict:
    """Steps 1-2 of :func:`_expert_parallel_peer` after the count exchange: the plan's second kernel, the quantizer
    and the dispatch kernel. ``host`` is the table as nested python lists. Returns what the later steps need."""
    from . import _ops

    t = int(hidden.shape[0])
    send_total = sum(host[rank][:world])
    recv_total = sum(host[s][rank] for s in range(world))
    send_token, send_rank, send_off, dst_base, recv_off, back_base, slot = _ops.ep_plan_place(
        mask, table, world, rank, send_total)
    if t > 0:
        xq, xs = quantized if quantized is not None else _ops.quantize_1x32_fp8(hidden)
        _ops.ep_dispatch_push(xq, xs, ids32, w32, send_token, send_rank, send_off, dst_base, bufs.peer_q, bufs.peer_w,
                              bufs.peer_ids, bufs.peer_wt, per)
    return dict(tokens=t, world=world, send_total=send_total, recv_total=recv_total, recv_off=recv_off,
                back_base=back_base, slot=slot)


def _peer_local(st: dict, experts, bufs: _PeerBuffers) -> None:
    """Step 3: the local experts over the received rows; partial rows go to their source ranks' buffers."""
    from . import moe

    n = st["recv_total"]
    moe._run_layer_rows(bufs.rx_q[:n], bufs.rx_w[:n], experts, bufs.rx_ids[:n], bufs.rx_wt[:n], st["recv_off"],
                        st["back_base"], bufs.peer_back, st["world"])


def _peer_reduce(st: dict, bufs: _PeerBuffers) -> torch.Tensor:
    """Step 4: out[t] = bf16(sum over ranks, ascending, of the partial rows that came back for token t)."""
    return _combine_partials(bufs.rx_back[:st["send_total"]], st["slot"], bufs.ones[:st["tokens"]])


def expert_parallel_layer(hidden: torch.Tensor, experts, topk_ids: torch.Tensor, topk_w: torch.Tensor, *,
                          num_experts_global: int, group=None, layer_fn: Optional[Callable] = None,
                          combine_fn: Optional[Callable] = None, micro_batches: Optional[int] = None,
                          transport: Optional[str] = None) -> torch.Tensor:
    """One MoE layer under expert parallelism: ``hidden`` bf16 ``[T, H]`` are this rank's tokens, ``topk_ids``
    ``[T, k]`` are GLOBAL expert ids, ``experts`` holds this rank's local experts. Returns the full result
    ``[T, H]`` for this rank's tokens (bf16), equal to the single-GPU layer over all experts up to the rounding of
    the per-rank partial sums.

    The tokens are processed in ``micro_batches`` slices (default 1; the environment variable
    ``FSO_B200_EP_MICRO_BATCHES`` overrides the default) whose exchanges are
    issued asynchronously: while the grouped GEMMs of one slice run, the next slice's dispatch and the previous
    slice's combine are on the wire.

    ``transport``: ``"peer"`` stores the rows straight into the destination GPU's memory with this library's
    kernels (:func:`_expert_parallel_peer`); ``"collective"`` moves them with ``all_to_all_single``. The default is
    ``"peer"`` for CUDA tensors when neither stand-in function nor micro-batching is asked for (the environment
    variable ``FSO_B200_EP_TRANSPORT`` overrides the default); both give the same bytes.

    ``layer_fn(hidden, experts, local_ids, weights)`` defaults to :func:`fish_scales_ops_b200.moe.layer` and
    ``combine_fn(back, slot, ones)`` to the library's combine kernel; the CPU tests of the exchange logic pass
    stand-ins for both."""
    if transport is None:
        transport = os.environ.get("FSO_B200_EP_TRANSPORT", "")
        if transport == "":
            sliced = micro_batches not in (None, 1) or os.environ.get("FSO_B200_EP_MICRO_BATCHES", "") not in ("", "1")
            transport = ("peer" if hidden.is_cuda and layer_fn is None and combine_fn is None and not sliced
                         else "collective")
    if transport not in ("peer", "collective"):
        raise ValueError(f"expert_parallel_layer: transport {transport!r}; the transports are 'peer' and 'collective'")
    if transport == "peer":
        if layer_fn is not None or combine_fn is not None or micro_batches not in (None, 1):
            raise ValueError("expert_parallel_layer: transport 'peer' runs the library's own layer in one slice; "
                             "stand-in functions and micro-batching need transport 'collective'")
        world = dist.get_world_size(group)
        if num_experts_global % world != 0:
            raise ValueError(f"expert_parallel_layer: {num_experts_global} experts over {world} ranks")
        return _expert_parallel_peer(hidden, experts, topk_ids, topk_w, num_experts_global // world, world, group)
    if layer_fn is None:
        from . import moe

        layer_fn = moe.layer
    if combine_fn is None:
        combine_fn = _combine_partials
    world = dist.get_world_size(group)
    if num_experts_global % world != 0:
        raise ValueError(f"expert_parallel_layer: {num_experts_global} experts over {world} ranks")
    per = num_experts_global // world
    t, k = int(hidden.shape[0]), int(topk_ids.shape[1])
    if micro_batches is None:
        env = os.environ.get("FSO_B200_EP_MICRO_BATCHES", "")
        # slicing streams the local experts' weights once per slice and shrinks every kernel; measured slower than
        # one slice on 2 GPUs (2.90 -> 4.10 ms) and on 4 GPUs (3.15 -> 3.86 ms), so one slice is the default
        micro_batches = int(env) if env.isdigit() and int(env) > 0 else 1
    micro_batches = max(1, min(int(micro_batches), max(1, t)))
    bounds = [t * i // micro_batches for i in range(micro_batches + 1)]
    out = torch.empty((t, int(hidden.shape[1])), dtype=torch.bfloat16, device=hidden.device)

    # stage 1: plan every slice and put its dispatch on the wire (token rows; ids localized for the destination rank
    # and weights packed into one int32 tensor)
    slices = []
    for i in range(micro_batches):
        t0, t1 = bounds[i], bounds[i + 1]
        ids_i, w_i = topk_ids[t0:t1], topk_w[t0:t1]
        plan = build_dispatch(ids_i, per, world, group)
        send_rows = hidden[t0:t1].index_select(0, plan.send_token)
        ids_sel = ids_i.to(torch.int64).index_select(0, plan.send_token)
        lo = (plan.send_rank * per).unsqueeze(1)
        local_ids = torch.where((ids_sel >= lo) & (ids_sel < lo + per), ids_sel - lo, torch.full_like(ids_sel, -1))
        meta = torch.cat([local_ids.to(torch.int32),
                          w_i.to(torch.float32).index_select(0, plan.send_token).view(torch.int32)], dim=1)
        recv_rows, w_rows = _a2a_rows_async(send_rows, plan.send_counts, plan.recv_counts, group)
        recv_meta, w_meta = _a2a_rows_async(meta, plan.send_counts, plan.recv_counts, group)
        slices.append(dict(t0=t0, t1=t1, plan=plan, recv_rows=recv_rows, recv_meta=recv_meta, works=(w_rows, w_meta),
                           keep=(send_rows, meta)))

    # stage 2: local experts of each slice, its partial rows go back asynchronously
    for sl in slices:
        for w in sl["works"]:
            w.wait()
        meta = sl["recv_meta"]
        partial = layer_fn(sl["recv_rows"], experts, meta[:, :k].contiguous(),
                           meta[:, k:].contiguous().view(torch.float32))
        sl["back"], sl["work_back"] = _a2a_rows_async(partial, sl["plan"].recv_counts, sl["plan"].send_counts, group)
        sl["keep"] = (partial,)

    # stage 3: the source rank adds a token's partial rows in rank order (fp32, one rounding)
    for sl in slices:
        sl["work_back"].wait()
        plan, n = sl["plan"], sl["t1"] - sl["t0"]
        slot = torch.full((n, world), -1, dtype=torch.int32, device=hidden.device)
        slot[plan.send_token, plan.send_rank] = torch.arange(sl["back"].shape[0], dtype=torch.int32,
                                                            device=hidden.device)
        ones = torch.ones((n, world), dtype=torch.float32, device=hidden.device)
        out[sl["t0"]:sl["t1"]] = combine_fn(sl["back"], slot, ones)
    return out


def dispatch_bytes(plan: DispatchPlan, rank: int, hidden_size: int, topk: int) -> int:
    """Bytes this rank puts on the wire for one layer (dispatch rows + ids + weights, and the combine rows it will
    get back are the same count): rows to other ranks only."""
    remote = sum(c for r, c in enumerate(plan.send_counts) if r != rank)
    return remote * (hidden_size * 2 + topk * 8) + remote * hidden_size * 2
