"""The two places where the path shards across the GPUs of one node (one process per GPU,
torch.distributed over NCCL / NVLink; gloo on CPU for the tests of the host logic).

* Expert-parallel MoE: rank r owns experts [r*E/G, (r+1)*E/G); every rank routes its own
  tokens, sends each (token, slot) row to the rank that owns its expert (all-to-all with
  a preceding all-to-all of the per-expert counts), runs the grouped GEMMs on what it
  received, and the results travel back the same way.
* Column-split prefill: rank r owns output columns [r*N/G, (r+1)*N/G) of a weight (a
  contiguous slab of packed rows); activations are replicated; one all-gather assembles
  the output.

The reference has no multi-GPU code; these functions define that layer.  Two forms of each:
through torch.distributed collectives (rows land in local memory before any kernel reads
them), and through peer memory (EpPeerExchange, ColumnSplitPeer: the kernels store straight
into the other GPUs' buffers, separated by the library's own time-limited flag barrier).
Decode mat-vec and the quantizers do not shard ("replicas only").
"""
import os

import torch
import torch.distributed as dist


class FlagBarrier:
    """Stream-ordered barrier over the ranks of a group on peer memory (lsg_ep_barrier): each
    rank stores a growing count into every peer's flag array and polls its own, for at most
    the library's wait limit; a peer that never arrives costs the limit and leaves code 6 in
    the device status word instead of a spinning kernel."""

    def __init__(self, group=None):
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.flags = symm.empty((self.world + 1,), dtype=torch.int32, device=dev)
        self._h = symm.rendezvous(self.flags, group)
        self.flags.zero_()
        torch.cuda.synchronize()
        dist.barrier(group)            # every array is zero before anybody arrives
        self.ptrs = torch.tensor([int(p) for p in self._h.buffer_ptrs], dtype=torch.int64, device=dev)

    def __call__(self):
        from . import capi
        capi.check(capi.lib.lsg_ep_barrier(self.ptrs.data_ptr(), self.rank, self.world, 3,
                                           torch.cuda.current_stream().cuda_stream))


def expert_range(rank, world, num_experts):
    """Experts owned by `rank`: a contiguous block, E divisible by world."""
    if num_experts % world != 0:
        raise ValueError(f"num_experts={num_experts} must be divisible by world size {world}")
    per = num_experts // world
    return rank * per, (rank + 1) * per


class EpPlan:
    """Everything both directions of the exchange need, derived from the per-expert row
    counts of every rank.  The index arithmetic stays on the device of the counts; the host
    only learns the split sizes of the all-to-all (one small device-to-host copy)."""

    def __init__(self, send_counts, recv_counts, experts_per_rank):
        # send_counts [world, per]: rows this rank sends, by destination rank and local expert
        # recv_counts [world, per]: rows this rank receives, by source rank and local expert
        self.per = experts_per_rank
        world = recv_counts.shape[0]
        both = torch.stack((send_counts.sum(1), recv_counts.sum(1))).cpu()   # the one host copy
        self.send_splits = both[0].tolist()
        self.recv_splits = both[1].tolist()
        self.recv_rows = int(sum(self.recv_splits))
        dev = recv_counts.device
        self.inv_order = None
        if recv_counts.is_cuda:
            # device kernels: block starts in both orders, then one thread per row
            from . import ops
            self.local_offsets, order, inv = ops.ep_expert_order(recv_counts, world, self.per, self.recv_rows)
            self.to_expert_order = order
            self.inv_order = inv
            return
        # CPU (tests of the host logic): the same arrays with torch operations.
        # received order is (source, expert, row); the grouped GEMM wants (expert, source, row)
        blocks = recv_counts.reshape(-1)                       # [(s, e)] sizes
        starts = torch.cumsum(blocks, 0) - blocks              # start of block (s, e) in recv order
        order = torch.arange(world * self.per, device=dev).reshape(world, self.per).t().reshape(-1)  # (e, s)
        sizes = blocks[order]
        src = torch.repeat_interleave(starts[order], sizes, output_size=self.recv_rows)
        first = torch.repeat_interleave(torch.cumsum(sizes, 0) - sizes, sizes, output_size=self.recv_rows)
        within = torch.arange(self.recv_rows, device=dev) - first
        self.to_expert_order = (src + within).to(torch.int64)  # gather index: expert-order row -> recv row
        self.local_offsets = torch.zeros(self.per + 1, dtype=torch.int32, device=dev)
        self.local_offsets[1:] = torch.cumsum(recv_counts.sum(0), 0).to(torch.int32)


class EpExchangeError(RuntimeError):
    """The expert-parallel exchange cannot proceed: a rank's routing metadata is inconsistent
    (raised on EVERY rank, before any row moves), or a peer did not take part in a collective."""


def make_ep_plan(expert_offsets, num_experts, group=None, rows=None):
    """expert_offsets: int32 [E+1] of THIS rank's permuted rows (device or CPU tensor).

    `rows` (this rank's number of permuted rows) lets the plan be checked: offsets that do not
    start at 0, decrease, or do not end at `rows` would make the row exchange send the wrong
    amounts.  The verdict travels with the counts (one extra column of the same all-to-all), so
    every rank learns of a bad rank and all of them raise EpExchangeError together instead of
    some waiting in a collective the others never enter."""
    world = dist.get_world_size(group)
    per = num_experts // world
    offs = expert_offsets.to(torch.int64)
    diffs = offs[1:] - offs[:-1]
    bad = (offs[0] != 0) | (diffs < 0).any()
    if rows is not None:
        bad = bad | (offs[-1] != rows)
    send = torch.empty((world, per + 1), dtype=torch.int64, device=offs.device)
    send[:, :per] = diffs.reshape(world, per)
    send[:, per] = bad.to(torch.int64)
    recv = torch.empty_like(send)
    try:
        dist.all_to_all_single(recv, send, group=group)
    except RuntimeError as exc:   # a peer that left, a timed-out process group
        raise EpExchangeError(f"expert-parallel count exchange failed: {exc}") from exc
    flags = recv[:, per].cpu()
    if bool(bad) or bool(flags.any()):
        who = [r for r in range(world) if int(flags[r]) != 0]
        raise EpExchangeError(f"inconsistent expert_offsets on rank(s) {who}: they must start at 0, not decrease, "
                              "and end at the rank's row count")
    return EpPlan(send[:, :per].contiguous(), recv[:, :per].contiguous(), per)


def ep_dispatch(rows, plan, group=None):
    """rows [P, H] permuted by global expert id -> rows of this rank's experts, grouped by
    local expert: ([R, H], local expert_offsets int32 [per+1] on rows.device)."""
    out = rows.new_empty((plan.recv_rows, rows.shape[1]))
    dist.all_to_all_single(out, rows.contiguous(), plan.recv_splits, plan.send_splits, group=group)
    if plan.inv_order is not None and rows.dtype == torch.bfloat16 and rows.shape[1] % 8 == 0:
        from . import ops
        return ops.moe_permute(out, plan.to_expert_order, 1), plan.local_offsets
    idx = plan.to_expert_order.to(rows.device).to(torch.int64)
    return out.index_select(0, idx), plan.local_offsets.to(rows.device)


def ep_combine(expert_rows, plan, group=None):
    """Inverse of ep_dispatch for the experts' outputs: [R, H'] -> [P, H'] in the sender's order."""
    if plan.inv_order is not None and expert_rows.dtype == torch.bfloat16 and expert_rows.shape[1] % 8 == 0:
        from . import ops
        recv_order = ops.moe_permute(expert_rows.contiguous(), plan.inv_order, 1)
    else:
        idx = plan.to_expert_order.to(expert_rows.device).to(torch.int64)
        recv_order = torch.empty_like(expert_rows)
        recv_order.index_copy_(0, idx, expert_rows)
    out = expert_rows.new_empty((int(sum(plan.send_splits)), expert_rows.shape[1]))
    dist.all_to_all_single(out, recv_order, plan.send_splits, plan.recv_splits, group=group)
    return out


def ep_moe_layer(hidden, logits, top_k, num_experts, expert_ffn, route, permutation, permute, unpermute,
                 group=None):
    """One expert-parallel MoE layer on this rank's tokens.

    expert_ffn(rows [R,H], local_offsets int32 [per+1]) -> [R,H] applies this rank's experts
    (gate / up grouped GEMMs, SwiGLU, down grouped GEMM).  route / permutation / permute /
    unpermute are the routing operators (the CUDA ones on a GPU; torch stand-ins in CPU
    tests of this host logic)."""
    idx, w = route(logits, top_k)
    offs, perm, inv = permutation(idx, num_experts)
    plan = make_ep_plan(offs, num_experts, group, rows=hidden.shape[0] * top_k)
    x = permute(hidden, perm, top_k)
    try:
        rows, local_offs = ep_dispatch(x, plan, group)
    except RuntimeError as exc:
        raise EpExchangeError(f"expert-parallel row dispatch failed: {exc}") from exc
    y = expert_ffn(rows, local_offs)
    try:
        back = ep_combine(y, plan, group)
    except RuntimeError as exc:
        raise EpExchangeError(f"expert-parallel row return failed: {exc}") from exc
    return unpermute(back, inv, w)


class EpPeerExchange:
    """Expert-parallel MoE layer with the row exchange over peer memory: the routed rows are
    stored straight into the destination GPU's receive buffer, the expert outputs straight
    back (lsg_ep_* kernels), with stream-ordered barriers in between.  No all-to-all, no
    device-to-host copy, no regrouping pass: rows arrive already grouped by (local expert,
    source rank).

    buffers: dict with, per name in ("counts", "recv", "back"), the LOCAL tensor and a CUDA
    int64 tensor of the `world` peer addresses (entry = rank p's tensor).  `barrier()` must
    order all ranks on the current stream (a symmetric-memory barrier, or a tiny all-reduce).
    `make()` builds everything from torch symmetric memory."""

    def __init__(self, rank, world, num_experts, top_k, H, num_pairs, capacity, buffers, barrier):
        self.rank, self.world, self.E, self.k, self.H = rank, world, num_experts, top_k, H
        self.per = num_experts // world
        self.P, self.cap = num_pairs, capacity
        self.b = buffers
        self.barrier = barrier
        dev = buffers["recv"][0].device
        self.send_base = torch.empty((num_experts,), dtype=torch.int32, device=dev)
        self.local_offsets = torch.empty((self.per + 1,), dtype=torch.int32, device=dev)
        self.dst_start = torch.empty((num_experts,), dtype=torch.int32, device=dev)
        self.ret_base = torch.empty((num_experts,), dtype=torch.int32, device=dev)
        self.info = torch.zeros((2,), dtype=torch.int32, device=dev)

    @staticmethod
    def make(num_experts, top_k, H, tokens_per_rank, capacity_factor=1.5, group=None):
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        P = tokens_per_rank * top_k
        cap = int(P * capacity_factor + 255) // 256 * 256
        local = {"counts": symm.empty((world, num_experts), dtype=torch.int32, device=dev),
                 "recv": symm.empty((cap, H), dtype=torch.bfloat16, device=dev),
                 "back": symm.empty((P, H), dtype=torch.bfloat16, device=dev)}
        handles = {n: symm.rendezvous(t, group) for n, t in local.items()}
        bufs = {n: (local[n], torch.tensor([int(p) for p in handles[n].buffer_ptrs], dtype=torch.int64, device=dev))
                for n in local}
        ex = EpPeerExchange(rank, world, num_experts, top_k, H, P, cap, bufs, FlagBarrier(group))
        ex._handles = handles   # keep the mappings alive
        return ex

    def check_inputs(self, hidden, logits):
        """Everything rank-local that could fail is checked here, before the first barrier of
        a layer: a rank that raised between two barriers would leave its peers waiting for
        the limit of theirs."""
        if not (hidden.is_cuda and hidden.dtype == torch.bfloat16 and hidden.dim() == 2 and hidden.is_contiguous()
                and hidden.shape[1] == self.H and hidden.data_ptr() % 16 == 0):
            raise ValueError(f"EpPeerExchange: hidden must be a contiguous, 16-byte aligned bf16 [T, {self.H}] CUDA tensor")
        if hidden.shape[0] * self.k != self.P:
            raise ValueError(f"EpPeerExchange: built for {self.P // self.k} tokens per rank, got {hidden.shape[0]}")
        if not (logits.is_cuda and logits.dim() == 2 and tuple(logits.shape) == (hidden.shape[0], self.E)):
            raise ValueError(f"EpPeerExchange: logits must be a CUDA tensor [{hidden.shape[0]}, {self.E}]")

    # A layer in three phases, so that a caller can interleave two exchanges (EpPeerPipeline):
    # dispatch (route, sort, publish, barrier, plan, send, barrier), experts, finish (return
    # rows, barrier, combine).  layer() runs them back to back on the current stream.
    def dispatch(self, hidden, logits, route, permutation):
        from . import capi
        lib = capi.lib
        st = torch.cuda.current_stream().cuda_stream
        p = lambda t: t.data_ptr()
        self.check_inputs(hidden, logits)
        idx, w = route(logits, self.k)
        offs, perm, inv = permutation(idx, self.E)
        counts, counts_ptrs = self.b["counts"]
        recv, recv_ptrs = self.b["recv"]
        back, _ = self.b["back"]
        capi.check(lib.lsg_ep_publish_counts(p(offs), self.E, self.rank, self.world, p(counts_ptrs), st))
        self.barrier()
        capi.check(lib.lsg_ep_plan(p(counts), self.rank, self.world, self.E, self.cap, p(self.send_base),
                                   p(self.local_offsets), p(self.dst_start), p(self.ret_base), p(self.info), st))
        capi.check(lib.lsg_ep_send_rows(p(hidden), p(perm), p(offs), p(self.send_base), self.P, self.k, self.H,
                                        self.E, self.world, p(recv_ptrs), self.cap, p(back), st))
        self.barrier()
        return (offs, perm, inv, w)      # offs and perm stay referenced until the layer is done

    def experts(self, expert_ffn):
        return expert_ffn(self.b["recv"][0], self.local_offsets)

    def finish(self, y, state, unpermute):
        from . import capi
        st = torch.cuda.current_stream().cuda_stream
        p = lambda t: t.data_ptr()
        back, back_ptrs = self.b["back"]
        capi.check(capi.lib.lsg_ep_return_rows(p(y), p(self.dst_start), p(self.ret_base), p(self.info), self.world,
                                               self.per, y.shape[1], self.cap, p(back_ptrs), st))
        self.barrier()
        return unpermute(back, state[2], state[3])

    def layer(self, hidden, logits, expert_ffn, route, permutation, unpermute):
        state = self.dispatch(hidden, logits, route, permutation)
        y = self.experts(expert_ffn)
        return self.finish(y, state, unpermute)

    def overflowed(self):
        """True if some rank's receive buffer was too small in the last layer (synchronizes).
        The same condition leaves code 7 in the device status word (capi.device_status()), so
        a caller that checks the status after a run needs no extra call; rows that did not fit
        contributed zeros."""
        return bool(self.info[1].item())


class EpPeerPipeline:
    """An expert-parallel layer as `chunks` EpPeerExchange halves on side streams, staggered so
    that the row exchange of one half runs under the expert GEMMs of the other:

        stream 0:  dispatch 0 | experts 0             | finish 0
        stream 1:             | dispatch 1 | experts 1            | finish 1

    (dispatch 1 starts when dispatch 0 is done, experts 1 when experts 0 is done.)  Every half has
    its own symmetric buffers and barrier flags, so the halves never wait for each other across
    GPUs; the copy kernels are small enough to be resident next to the GEMM's CTAs.  Results are
    those of one EpPeerExchange per half: each token's output depends on its own row only.
    The whole layer can be captured into one CUDA graph (the side streams fork from and join the
    capturing stream)."""

    def __init__(self, exchanges):
        self.ex = exchanges
        self.chunks = len(exchanges)
        self.streams = [torch.cuda.Stream() for _ in exchanges]
        self.tokens = sum(e.P // e.k for e in exchanges)

    @staticmethod
    def make(num_experts, top_k, H, tokens_per_rank, chunks=2, capacity_factor=1.5, group=None):
        if tokens_per_rank % chunks != 0:
            raise ValueError(f"EpPeerPipeline: {tokens_per_rank} tokens per rank do not split into {chunks} chunks")
        return EpPeerPipeline([EpPeerExchange.make(num_experts, top_k, H, tokens_per_rank // chunks,
                                                   capacity_factor, group) for _ in range(chunks)])

    def layer(self, hidden, logits, expert_ffn, route, permutation, unpermute):
        n = self.chunks
        if hidden.shape[0] != self.tokens:
            raise ValueError(f"EpPeerPipeline: built for {self.tokens} tokens per rank, got {hidden.shape[0]}")
        per = self.tokens // n
        hs = [hidden[c * per:(c + 1) * per] for c in range(n)]
        ls = [logits[c * per:(c + 1) * per].contiguous() for c in range(n)]
        for c in range(n):     # every rank-local check before anything waits for a peer
            self.ex[c].check_inputs(hs[c], ls[c])
        cur = torch.cuda.current_stream()
        states, ys, outs = [None] * n, [None] * n, [None] * n
        ev_a = [torch.cuda.Event() for _ in range(n)]
        ev_b = [torch.cuda.Event() for _ in range(n)]
        for c in range(n):
            st = self.streams[c]
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                if c > 0:
                    st.wait_event(ev_a[c - 1])
                states[c] = self.ex[c].dispatch(hs[c], ls[c], route, permutation)
                ev_a[c].record(st)
        for c in range(n):
            st = self.streams[c]
            with torch.cuda.stream(st):
                if c > 0:
                    st.wait_event(ev_b[c - 1])
                ys[c] = self.ex[c].experts(expert_ffn)
                ev_b[c].record(st)
        for c in range(n):
            with torch.cuda.stream(self.streams[c]):
                outs[c] = self.ex[c].finish(ys[c], states[c], unpermute)
        for c in range(n):
            cur.wait_stream(self.streams[c])
            outs[c].record_stream(cur)
        return torch.cat(outs, 0)

    def overflowed(self):
        return any(e.overflowed() for e in self.ex)


class EpPeerGroups:
    """The peer-memory exchange with each rank's local experts in `groups` groups, staggered on
    side streams so that one group's rows travel while another group's expert GEMMs run:

        main:      route, sort, publish counts | barrier | plan
        stream 0:  send group 0 | barrier | experts 0                 | return 0 | barrier
        stream 1:               send group 1 | barrier | experts 1               | return 1 | barrier
        main:      combine

    (send g starts when send g-1 is done, experts g when experts g-1 are done.)  Unlike a split by
    tokens (EpPeerPipeline) every expert's weights are still decoded once per layer: the receive
    layout is grouped by local expert, so a group's rows are one contiguous range.  Every group
    has its own barrier flags.  `expert_ffn(rows, offsets, lo, hi)` runs local experts [lo, hi):
    `offsets` is the slice local_offsets[lo : hi + 1] (absolute rows of `rows`)."""

    def __init__(self, exchange, groups, group=None):
        self.ex = exchange
        per = exchange.per
        self.groups = max(1, min(groups, per))
        self.bounds = [per * g // self.groups for g in range(self.groups + 1)]
        self.bars = [FlagBarrier(group) for _ in range(self.groups)]
        self.streams = [torch.cuda.Stream() for _ in range(self.groups)]
        self.chunks = self.groups        # for callers that report how the layer is pipelined

    @staticmethod
    def make(num_experts, top_k, H, tokens_per_rank, groups=2, capacity_factor=1.5, group=None):
        return EpPeerGroups(EpPeerExchange.make(num_experts, top_k, H, tokens_per_rank, capacity_factor, group),
                            groups, group)

    def layer(self, hidden, logits, expert_ffn, route, permutation, unpermute):
        from . import capi
        lib, ex = capi.lib, self.ex
        p = lambda t: t.data_ptr()
        ex.check_inputs(hidden, logits)
        cur = torch.cuda.current_stream()
        st = cur.cuda_stream
        idx, w = route(logits, ex.k)
        offs, perm, inv = permutation(idx, ex.E)
        counts, counts_ptrs = ex.b["counts"]
        recv, recv_ptrs = ex.b["recv"]
        back, back_ptrs = ex.b["back"]
        capi.check(lib.lsg_ep_publish_counts(p(offs), ex.E, ex.rank, ex.world, p(counts_ptrs), st))
        ex.barrier()
        capi.check(lib.lsg_ep_plan(p(counts), ex.rank, ex.world, ex.E, ex.cap, p(ex.send_base), p(ex.local_offsets),
                                   p(ex.dst_start), p(ex.ret_base), p(ex.info), st))
        n = self.groups
        ev_a = [torch.cuda.Event() for _ in range(n)]
        ev_b = [torch.cuda.Event() for _ in range(n)]
        ys = [None] * n
        for g in range(n):
            s = self.streams[g]
            s.wait_stream(cur)
            lo, hi = self.bounds[g], self.bounds[g + 1]
            with torch.cuda.stream(s):
                if g > 0:
                    s.wait_event(ev_a[g - 1])
                capi.check(lib.lsg_ep_send_rows_group(p(hidden), p(perm), p(offs), p(ex.send_base), ex.P, ex.k, ex.H,
                                                      ex.E, ex.world, p(recv_ptrs), ex.cap, p(back), lo, hi,
                                                      s.cuda_stream))
                self.bars[g]()
                ev_a[g].record(s)
        for g in range(n):
            s = self.streams[g]
            lo, hi = self.bounds[g], self.bounds[g + 1]
            with torch.cuda.stream(s):
                if g > 0:
                    s.wait_event(ev_b[g - 1])
                ys[g] = expert_ffn(recv, ex.local_offsets[lo:hi + 1], lo, hi)
                ev_b[g].record(s)
        for g in range(n):
            s = self.streams[g]
            lo, hi = self.bounds[g], self.bounds[g + 1]
            with torch.cuda.stream(s):
                y = ys[g]
                capi.check(lib.lsg_ep_return_rows_group(p(y), p(ex.dst_start), p(ex.ret_base), p(ex.info), ex.world,
                                                        ex.per, y.shape[1], ex.cap, p(back_ptrs), p(ex.local_offsets),
                                                        lo, hi, s.cuda_stream))
                self.bars[g]()
        for g in range(n):
            cur.wait_stream(self.streams[g])
            ys[g].record_stream(cur)
        return unpermute(back, inv, w)

    def overflowed(self):
        return self.ex.overflowed()


def column_slab(rank, world, N, align=128):
    """Output columns [n0, n1) owned by `rank`: contiguous, multiples of `align`."""
    if N % (world * align) != 0:
        raise ValueError(f"N={N} must be divisible by world*{align}")
    per = N // world
    return rank * per, (rank + 1) * per


class ColumnSplitPeer:
    """Column-split prefill GEMM with the all-gather fused into the GEMM's epilogue: every rank
    computes its slab of output columns and stores each tile into the full [M, N] output of
    every rank (peer-memory stores over NVLink, overlapped with the tensor-core work on the
    following tiles); one barrier afterwards and every rank holds the whole product.  The
    outputs are torch symmetric-memory allocations."""

    def __init__(self, M, N, dtype=torch.bfloat16, group=None, multicast=True):
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.M, self.N = M, N
        self.out = symm.empty((M, N), dtype=dtype, device=dev)
        self._h = symm.rendezvous(self.out, group)
        self.ptrs = torch.tensor([int(p) for p in self._h.buffer_ptrs], dtype=torch.int64, device=dev)
        # NVLink multicast address of the output, where the fabric offers one: a rank then sends its
        # slab once (multimem.st) and the switch replicates it, instead of one store per peer.
        # Measured equal to plain peer stores at 4 and 8 GPUs (0.245 / 0.237 ms against 0.247 /
        # 0.236 ms at M = 4096: every rank still receives (G-1)/G of the product), so it is off
        # unless asked for.
        self.multicast_ptr = 0
        mode = os.environ.get("LSG_GATHER_MULTICAST", "0")     # 0: never, 1: with three or more ranks, 2: always
        if multicast and mode != "0" and (self.world > 2 or mode == "2"):
            try:
                self.multicast_ptr = int(getattr(self._h, "multicast_ptr", 0) or 0)
            except Exception:   # noqa: BLE001 - older handles have no such attribute
                self.multicast_ptr = 0
        self.barrier = FlagBarrier(group)

    def gemm(self, A, slab, type, K):
        """A [M, K] bf16 (replicated), slab = this rank's packed rows [N / world, ...] -> the
        full [M, N] product on every rank (the returned tensor is reused by the next call)."""
        from . import ops
        n0, n1 = column_slab(self.rank, self.world, self.N)
        self.barrier()   # every rank is done reading the previous product
        ops.gguf_mmq_gather(A, slab, type, n1 - n0, K, self.ptrs, self.N, n0, out_dtype=self.out.dtype,
                            multicast_ptr=self.multicast_ptr)
        self.barrier()   # every slab has landed everywhere
        return self.out


def column_split_gather(local_out, group=None):
    """local_out [M, N/G] of every rank -> [M, N] on every rank (one all-gather)."""
    world = dist.get_world_size(group)
    M, n = local_out.shape
    buf = local_out.new_empty((world * M, n))
    dist.all_gather_into_tensor(buf, local_out.contiguous(), group=group)
    return buf.view(world, M, n).permute(1, 0, 2).reshape(M, world * n)
