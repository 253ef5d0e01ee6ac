"""Expert parallelism for prefill-sized batches: experts sharded over the GPUs of one box, tokens
data-parallel, one all-to-all each way per layer.

The reference has no multi-device path (one Metal device, no collective library); this is the
B200 addition.  Rank r of g holds experts [r*E/g, (r+1)*E/g) of every layer in its own HBM; the
router and the shared FFN are replicated; every rank owns T/g token rows.  Per layer:

  1. local router -> (token, rank) routes with global expert ids;
  2. routes are ordered by destination rank (stable, so (token, rank) order is kept inside a
     destination) and the per-destination counts are exchanged;
  3. dispatch: all-to-all of the routed token rows (bf16) and their local expert ids;
  4. the receiving rank runs its experts on the rows it got — the grouped INT4 GEMM path with one
     route per row — reading only its own memory;
  5. combine: all-to-all of the bf16 partial rows back to the tokens' home ranks;
  6. the home rank puts them back in (token, rank) order and does the weighted reduce, adding its
     shared-FFN rows.

The collective is torch.distributed's all_to_all_single: NCCL over NVLink/NVSwitch on GPUs, gloo
in the CPU tests.  Decode and verify do not use this: they run as independent replicas.
The planning functions are plain tensor arithmetic so they run (and are tested) on CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    order: torch.Tensor         # int64 [routes]: route index (token*K + rank) in send order
    send_counts: torch.Tensor   # int64 [world]: routes going to each rank
    local_expert: torch.Tensor  # int32 [routes]: expert id on the destination rank, in send order
    token: torch.Tensor         # int64 [routes]: source token row, in send order


@dataclass
class Placement:
    """Which rank holds each expert and under which local id.  The blob layout of a layer file is
    not touched: a rank simply loads the blobs of its experts in `experts_of(rank)` order."""
    rank_of: torch.Tensor   # int64 [experts]
    local_of: torch.Tensor  # int64 [experts]
    world: int

    def experts_of(self, rank: int):
        mine = torch.nonzero(self.rank_of == rank).reshape(-1)
        return mine[torch.argsort(self.local_of[mine])].tolist()

    def tables_on(self, device):
        """rank_of and local_of on `device`, copied there once (a copy per layer would make every
        plan wait for the host)."""
        cache = self.__dict__.setdefault("_device_tables", {})
        key = str(device)
        if key not in cache:
            cache[key] = (self.rank_of.to(device), self.local_of.to(device))
        return cache[key]


def contiguous_placement(experts: int, world: int) -> Placement:
    """Expert e on rank e // (experts/world): contiguous blocks."""
    per = experts // world
    e = torch.arange(experts, dtype=torch.int64)
    return Placement(torch.div(e, per, rounding_mode="floor"), e % per, world)


def balanced_placement(load, world: int) -> Placement:
    """Equal expert counts per rank, expected load balanced: experts in decreasing load go to the
    least-loaded rank that still has room (longest-processing-time greedy).  `load` is the expected
    share of routes per expert (e.g. the router's prior); ties keep expert order."""
    load = [float(v) for v in load]
    experts = len(load)
    per = experts // world
    order = sorted(range(experts), key=lambda e: (-load[e], e))
    totals, counts = [0.0] * world, [0] * world
    rank_of, local_of = [0] * experts, [0] * experts
    for e in order:
        r = min((r for r in range(world) if counts[r] < per), key=lambda r: (totals[r], r))
        rank_of[e], local_of[e] = r, counts[r]
        counts[r] += 1
        totals[r] += load[e]
    return Placement(torch.tensor(rank_of, dtype=torch.int64), torch.tensor(local_of, dtype=torch.int64), world)


def dispatch_plan(ids: torch.Tensor, experts_per_rank: int, world: int,
                  placement: Optional[Placement] = None, route_sorter: Optional[Callable] = None) -> DispatchPlan:
    """Routes ordered by destination rank, (token, rank) order kept inside a destination.  Expert
    ids past the group's experts raise on the CPU; on a GPU, where looking at them would stall the
    stream, they are clamped into range instead (the library's own router never produces one)."""
    tokens, k = ids.shape
    flat = ids.reshape(-1).to(torch.int64)
    total = experts_per_rank * world
    if flat.is_cuda:
        flat = flat.clamp(0, total - 1)
    elif tokens and (int(flat.max()) >= total or int(flat.min()) < 0):
        raise ValueError("route expert out of range for this expert-parallel group")
    if placement is None:
        dest = torch.div(flat, experts_per_rank, rounding_mode="floor")
        local_all = flat - dest * experts_per_rank
    else:
        rank_of, local_of = placement.tables_on(flat.device)
        dest = rank_of[flat]
        local_all = local_of[flat]
    if route_sorter is not None and flat.is_cuda:
        # the library's counting sort (three launches) in place of a general sort and a histogram
        pairs, offsets = route_sorter(dest.to(torch.int32).reshape(tokens, k), world)
        token = pairs[:, 0].to(torch.int64)
        order = token * k + pairs[:, 2].to(torch.int64)
        send_counts = (offsets[1:] - offsets[:-1]).to(torch.int64)
        return DispatchPlan(order, send_counts, local_all[order].to(torch.int32), token)
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world).to(torch.int64)
    local = local_all[order].to(torch.int32)
    return DispatchPlan(order, send_counts, local, torch.div(order, k, rounding_mode="floor"))


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts, group=group)
    return recv


def all_to_all_rows(rows: torch.Tensor, send_counts, recv_counts, group=None, async_op: bool = False,
                    out: Optional[torch.Tensor] = None):
    """Variable-split all-to-all along dim 0; counts are python lists of row counts.  Returns the
    received rows (in `out` when given), and with async_op the work handle to wait on before using
    them."""
    if out is None:
        out = torch.empty((int(sum(recv_counts)),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    work = dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                                  input_split_sizes=list(send_counts), group=group, async_op=async_op)
    return (out, work) if async_op else out


class PeerBuffers:
    """Two buffers in symmetric memory (every rank's copy is mapped into every other rank of the
    box) through which dispatch and combine move rows with plain peer stores over NVLink instead of
    a collective: a rank writes the rows for rank p straight into p's buffer at the offset that the
    exchanged counts give it, and a barrier across the ranks (signals in symmetric memory, on the
    stream) says when everybody's rows have landed.  One instance serves every layer of a stack.
    `available()` is false where symmetric memory cannot be set up (CPU tests, gloo)."""

    def __init__(self, capacity_rows: int, row_elems: int, dtype, device, group=None, ids_width: int = 1):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only
        import torch.distributed._symmetric_memory as symm
        self.capacity = int(capacity_rows)
        name = (group if group is not None else dist.group.WORLD).group_name
        self.recv = symm.empty((self.capacity, row_elems), dtype=dtype, device=device)    # rows for my experts
        self.back = symm.empty((self.capacity, row_elems), dtype=dtype, device=device)    # partial rows of my tokens
        self.ids_width = int(ids_width)  # local expert ids per received row (top-K wide for one row per token)
        self.ids = symm.empty((self.capacity, self.ids_width), dtype=torch.int32, device=device)
        self.ids_handle = symm.rendezvous(self.ids, name)
        self.recv_handle = symm.rendezvous(self.recv, name)
        self.back_handle = symm.rendezvous(self.back, name)
        self.shape = (self.capacity, row_elems)
        self.dtype = dtype

    def peer_recv(self, rank: int) -> torch.Tensor:
        return self.recv_handle.get_buffer(rank, self.shape, self.dtype)

    def peer_back(self, rank: int) -> torch.Tensor:
        return self.back_handle.get_buffer(rank, self.shape, self.dtype)

    def peer_ids(self, rank: int) -> torch.Tensor:
        return self.ids_handle.get_buffer(rank, (self.capacity, self.ids_width), torch.int32)

    def barrier(self):
        self.recv_handle.barrier()


class PhaseTimer:
    """Per-phase device times of ExpertParallelMoE.forward, by CUDA events on the current stream
    (CPU tensors: no-op).  `totals()` waits for the device and returns {phase: milliseconds}."""

    def __init__(self):
        self.records = []

    def phase(self, name, tensor):
        timer = self

        class _Scope:
            def __enter__(self_inner):
                self_inner.events = None
                if tensor.is_cuda:
                    self_inner.events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    self_inner.events[0].record()

            def __exit__(self_inner, *exc):
                if self_inner.events:
                    self_inner.events[1].record()
                    timer.records.append((name, *self_inner.events))
                return False

        return _Scope()

    def totals(self):
        out = {}
        if self.records:
            torch.cuda.synchronize()
        for name, begin, end in self.records:
            out[name] = out.get(name, 0.0) + begin.elapsed_time(end)
        self.records = []
        return out


class _NoTimer:
    def phase(self, name, tensor):
        import contextlib
        return contextlib.nullcontext()


class ExpertParallelMoE:
    """One MoE layer under expert parallelism.

    `router_fn(x) -> (ids int32 [T,K], weights [T,K])`, `shared_fn(x) -> [T,D] or None`,
    `experts_fn(rows [R,D], local_ids int32 [R]) -> partial rows [R,D]`,
    `reduce_fn(partials [T*K,D], weights, residual) -> y [T,D]` are supplied by the caller: the CUDA
    library on GPUs (see `cuda_layer_fns`), plain torch functions in the CPU tests.

    `chunks` > 1 cuts the local tokens into that many runs: the dispatch of run i+1 and the combine
    of run i-1 are in flight (on the collective library's stream) while the experts of run i
    compute.  `peer` (a PeerBuffers) moves the rows by peer stores into symmetric memory instead
    of the collective.  The result depends on neither.  A `reduce_fn` with the attribute
    `indexed = True` takes a fourth argument, the int32 row index of every route's partial row, and
    spares the pass that would put the rows back into (token, rank) order."""

    def __init__(self, experts: int, top_k: int, router_fn: Callable, shared_fn: Callable,
                 experts_fn: Callable, reduce_fn: Callable, group=None,
                 placement: Optional[Placement] = None, chunks: int = 1, peer: "Optional[PeerBuffers]" = None,
                 one_row_per_token: bool = False, route_sorter: Optional[Callable] = None):
        self.group = group
        self.placement = placement
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts % self.world:
            raise ValueError("experts must divide evenly over the ranks")
        self.experts, self.top_k = experts, top_k
        self.experts_per_rank = experts // self.world
        self.router_fn, self.shared_fn = router_fn, shared_fn
        self.experts_fn, self.reduce_fn = experts_fn, reduce_fn
        self.chunks = max(1, int(chunks))
        self.peer = peer  # PeerBuffers: exchange rows by peer stores instead of the collective
        self._side = None  # second stream of the peer path (shared FFN beside the dispatch)
        # peer path: a token's row crosses to a destination rank once, with all of the token's local
        # expert ids there (needs an expert context created with topK = K and peer buffers with
        # ids_width = K); otherwise once per route
        self.one_row_per_token = bool(one_row_per_token)
        # (group ids int32 [T][K], groups) -> (pairs int32 [T*K][4], offsets int32 [groups+1]) on the device
        self.route_sorter = route_sorter
        self.last_recv_rows = 0
        self.last_expert_counts = None  # routes per (global) expert of the last forward, on request
        self.count_experts = False
        self.timer = _NoTimer()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.peer is not None and self.one_row_per_token:
            return self._forward_peer_tokens(x)
        if self.peer is not None:
            return self._forward_peer(x)
        T, K, W = x.shape[0], self.top_k, self.world
        tm = self.timer
        with tm.phase("router", x):
            ids, weights = self.router_fn(x)
        if self.count_experts:
            self.last_expert_counts = torch.bincount(ids.reshape(-1).to(torch.int64), minlength=self.experts)
        with tm.phase("plan", x):
            bounds = [T * c // self.chunks for c in range(self.chunks + 1)]
            plans = [dispatch_plan(ids[bounds[c]:bounds[c + 1]], self.experts_per_rank, W, self.placement, self.route_sorter)
                     for c in range(self.chunks)]
            send = torch.stack([p.send_counts for p in plans]).to(x.device)        # [chunks, world]
            # counts of every run to every rank in one exchange: rank r receives column r of every
            # rank's table; the one host read below is the step's only wait on the device
            recv = exchange_counts(send.t().contiguous(), self.group).t()            # [chunks, world]
            both = torch.stack([send, recv]).tolist()
        send_lists, recv_lists = both
        self.last_recv_rows = int(sum(sum(r) for r in recv_lists))
        on_gpu = x.is_cuda
        indexed = bool(getattr(self.reduce_fn, "indexed", False))

        def dispatch(c):
            p = plans[c]
            rows = x[bounds[c]:bounds[c + 1]].index_select(0, p.token.to(x.device))
            r = all_to_all_rows(rows, send_lists[c], recv_lists[c], self.group, async_op=on_gpu)
            l = all_to_all_rows(p.local_expert.to(x.device), send_lists[c], recv_lists[c], self.group,
                                async_op=on_gpu)
            return r, l

        def ready(pending):
            if on_gpu:
                (rows, w0), (local, w1) = pending
                w0.wait()
                w1.wait()
                return rows, local
            return pending

        # the partial rows come back grouped by chunk and, inside a chunk, in the order they were sent
        # (by destination); `partials` receives them as they lie and `row_index` says where the row of
        # route (t, k) is — or, for a reduce that wants (token, rank) order, they are put back first
        partials = torch.empty((T * K,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        with tm.phase("dispatch", x):
            pending = dispatch(0)
        residual = None
        backs = []
        for c in range(self.chunks):
            if c == 0:
                # the shared FFN needs no exchange: it is queued while the first dispatch is in flight
                with tm.phase("shared", x):
                    residual = self.shared_fn(x)
            with tm.phase("dispatch", x):
                rows, local = ready(pending)
                if c + 1 < self.chunks:
                    pending = dispatch(c + 1)
            with tm.phase("experts", x):
                partial_rows = self.experts_fn(rows, local)
            with tm.phase("combine", x):
                out = partials[bounds[c] * K:bounds[c + 1] * K] if indexed else None
                backs.append(all_to_all_rows(partial_rows, recv_lists[c], send_lists[c], self.group,
                                             async_op=on_gpu, out=out))
        with tm.phase("combine", x):
            row_index = torch.empty(T * K, dtype=torch.int32, device=x.device) if indexed else None
            for c, back in enumerate(backs):
                if on_gpu:
                    back, work = back
                    work.wait()
                order = plans[c].order.to(x.device)
                if indexed:
                    n = order.numel()
                    row_index[bounds[c] * K + order] = torch.arange(bounds[c] * K, bounds[c] * K + n, dtype=torch.int32,
                                                                    device=x.device)
                else:
                    partials[bounds[c] * K + order] = back
        with tm.phase("reduce", x):
            if indexed:
                return self.reduce_fn(partials, weights, residual, row_index)
            return self.reduce_fn(partials, weights, residual)

    def _forward_peer(self, x: torch.Tensor) -> torch.Tensor:
        """Dispatch and combine as peer stores into symmetric memory (see PeerBuffers): the routed
        rows are gathered straight into the destination ranks' buffers, the partial rows are copied
        straight into their home ranks' buffers, and the reduce reads them where they lie."""
        T, K, W = x.shape[0], self.top_k, self.world
        tm, pb = self.timer, self.peer
        with tm.phase("router", x):
            ids, weights = self.router_fn(x)
        if self.count_experts:
            self.last_expert_counts = torch.bincount(ids.reshape(-1).to(torch.int64), minlength=self.experts)
        with tm.phase("plan", x):
            plan = dispatch_plan(ids, self.experts_per_rank, W, self.placement, self.route_sorter)
            table = torch.empty((W, W), dtype=torch.int64, device=x.device)    # [source][destination]
            dist.all_gather_into_tensor(table, plan.send_counts.to(x.device), group=self.group)
            counts = table.tolist()                                             # the step's only host read
            order = plan.order.to(x.device)
            row_index = torch.empty(T * K, dtype=torch.int32, device=x.device)
            row_index[order] = torch.arange(T * K, dtype=torch.int32, device=x.device)
        me = self.rank
        recv_total = sum(counts[s][me] for s in range(W))
        if max(recv_total, T * K) > pb.capacity:
            raise ValueError(f"{recv_total} rows exceed the peer buffers' capacity {pb.capacity}")
        self.last_recv_rows = recv_total
        token = plan.token.to(x.device)
        local_expert = plan.local_expert.to(x.device)
        # the shared FFN needs no exchange: it runs on a second stream beside the dispatch
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=x.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            with tm.phase("shared", x):
                residual = self.shared_fn(x)
        x.record_stream(self._side)
        if residual is not None:
            residual.record_stream(main)
        with tm.phase("dispatch", x):
            pb.barrier()  # every rank is done with the previous contents of the buffers
            start = 0
            for p in range(W):
                n = counts[me][p]
                offset = sum(counts[s][p] for s in range(me))
                if n:
                    torch.index_select(x, 0, token[start:start + n], out=pb.peer_recv(p)[offset:offset + n])
                    pb.peer_ids(p)[offset:offset + n, 0].copy_(local_expert[start:start + n])
                start += n
            pb.barrier()  # everybody's rows and their local expert ids have landed
        with tm.phase("experts", x):
            partial_rows = self.experts_fn(pb.recv[:recv_total], pb.ids[:recv_total, 0])
        with tm.phase("combine", x):
            start = 0
            for s in range(W):
                n = counts[s][me]
                offset = sum(counts[s][p] for p in range(me))  # where my block starts in s's send order
                if n:
                    pb.peer_back(s)[offset:offset + n].copy_(partial_rows[start:start + n])
                start += n
            pb.barrier()  # my tokens' partial rows have landed
        main.wait_stream(self._side)
        with tm.phase("reduce", x):
            return self.reduce_fn(pb.back[:T * K], weights, residual, row_index)


    def _forward_peer_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """The peer-store exchange with one row per (token, destination rank) on dispatch: a token
        whose routes name several experts of one rank crosses NVLink once, together with the K-wide
        list of its local expert ids there (ids of other ranks' routes are replaced by an id past
        the rank's experts, which the receiver's sort drops).  The partial rows come back one per
        route, in the order the per-route plan gives, so the reduce is the same as everywhere."""
        T, K, W = x.shape[0], self.top_k, self.world
        tm, pb = self.timer, self.peer
        epr = self.experts_per_rank
        with tm.phase("router", x):
            ids, weights = self.router_fn(x)
        if self.count_experts:
            self.last_expert_counts = torch.bincount(ids.reshape(-1).to(torch.int64), minlength=self.experts)
        with tm.phase("plan", x):
            plan = dispatch_plan(ids, epr, W, self.placement, self.route_sorter)
            flat = ids.reshape(-1).to(torch.int64).clamp(0, self.experts - 1)
            if self.placement is None:
                dest = torch.div(flat, epr, rounding_mode="floor")
                local = flat - dest * epr
            else:
                rank_of, local_of = self.placement.tables_on(x.device)
                dest, local = rank_of[flat], local_of[flat]
            dest, local = dest.reshape(T, K), local.reshape(T, K).to(torch.int32)
            hit = torch.zeros((T, W), dtype=torch.bool, device=x.device)
            hit.scatter_(1, dest, True)                                   # token t has a route to rank p
            both = torch.cat([plan.send_counts.to(x.device), hit.sum(0)])  # routes, then tokens, per destination
            table = torch.empty((W, 2 * W), dtype=torch.int64, device=x.device)
            dist.all_gather_into_tensor(table, both, group=self.group)
            counts = table.tolist()                                       # the step's only host read
            order = plan.order.to(x.device)
            row_index = torch.empty(T * K, dtype=torch.int32, device=x.device)
            row_index[order] = torch.arange(T * K, dtype=torch.int32, device=x.device)
        me = self.rank
        routes = [[counts[s][p] for p in range(W)] for s in range(W)]        # [source][destination]
        tokens = [[counts[s][W + p] for p in range(W)] for s in range(W)]
        recv_tokens = sum(tokens[s][me] for s in range(W))
        recv_routes = sum(routes[s][me] for s in range(W))
        if max(recv_tokens, T * K) > pb.capacity or pb.ids_width != K:
            raise ValueError("peer buffers too small (or not K ids wide) for one row per token")
        self.last_recv_rows = recv_routes
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=x.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            with tm.phase("shared", x):
                residual = self.shared_fn(x)
        x.record_stream(self._side)
        if residual is not None:
            residual.record_stream(main)
        with tm.phase("dispatch", x):
            pb.barrier()  # every rank is done with the previous contents of the buffers
            for p in range(W):
                n = tokens[me][p]
                if not n:
                    continue
                offset = sum(tokens[s][p] for s in range(me))
                # the tokens with a route to p, in token order (no host read: their number is known)
                mine = torch.argsort(~hit[:, p], stable=True)[:n]
                torch.index_select(x, 0, mine, out=pb.peer_recv(p)[offset:offset + n])
                pb.peer_ids(p)[offset:offset + n].copy_(
                    torch.where(dest[mine] == p, local[mine], torch.full_like(local[mine], epr)))
            pb.barrier()  # everybody's rows and id lists have landed
        with tm.phase("experts", x):
            got_ids = pb.ids[:recv_tokens]
            partial_rows = self.experts_fn(pb.recv[:recv_tokens], got_ids)       # [recv_tokens * K, D]
            # rows of the routes that are this rank's, in (source, token, rank) order
            live = torch.argsort(~(got_ids.reshape(-1) < epr), stable=True)[:recv_routes]
        with tm.phase("combine", x):
            start = 0
            for s in range(W):
                n = routes[s][me]
                offset = sum(routes[s][p] for p in range(me))  # where my block starts in s's per-route order
                if n:
                    torch.index_select(partial_rows, 0, live[start:start + n], out=pb.peer_back(s)[offset:offset + n])
                start += n
            pb.barrier()  # my tokens' partial rows have landed
        main.wait_stream(self._side)
        with tm.phase("reduce", x):
            return self.reduce_fn(pb.back[:T * K], weights, residual, row_index)


def cuda_route_sorter(home_ctx):
    """`route_sorter` for ExpertParallelMoE backed by the library's device permute (ff_sort_routes);
    `home_ctx` needs topK = K, at least as many experts as there are ranks and maxTokens > 16."""
    from . import hotpath
    grouping = hotpath.PrefillGroupedRoutedMoE(home_ctx)
    return lambda group_ids, groups: grouping.sortRoutesOnDevice(None, group_ids.contiguous(), groups)


def cuda_layer_fns(home_ctx, expert_ctx, layer: int, expert_layer: Optional[int] = None):
    """The four callables for `ExpertParallelMoE` backed by libfieldfare_cuda.so.

    `home_ctx`: a HotpathContext holding the replicated router and shared FFN of `layer`
    (topK = K); `expert_ctx`: a HotpathContext with experts = E/g holding this rank's experts (in
    slot `expert_layer`, default `layer`), created with topK = 1 — a received row with one local
    expert id is a one-route token — or, for one row per token and destination, with topK = K."""
    from . import hotpath

    router = hotpath.PrefillRouter(home_ctx)
    shared = hotpath.PrefillSharedExpert(home_ctx)
    reduce = hotpath.PrefillMoE(home_ctx)
    routed = hotpath.PrefillGroupedRoutedMoE(expert_ctx)
    d, k = home_ctx.d, home_ctx.topK
    slot = layer if expert_layer is None else expert_layer

    def router_fn(x):
        t = x.shape[0]
        ids = torch.empty((t, k), dtype=torch.int32, device=x.device)
        w = torch.empty((t, k), dtype=torch.bfloat16, device=x.device)
        router.encodeGemma4Block(None, layer, x, ids, w, t)
        return ids, w

    def shared_fn(x):
        if not home_ctx.sharedF:
            return None
        y = torch.empty((x.shape[0], d), dtype=torch.bfloat16, device=x.device)
        shared.encodeBlock(None, layer, x, y, x.shape[0])
        return y

    def experts_fn(rows, local_ids):
        # one partial row per (received row, route slot of the expert context)
        wide = expert_ctx.topK
        out = torch.empty((rows.shape[0] * wide, rows.shape[1]), dtype=rows.dtype, device=rows.device)
        if rows.shape[0]:
            routed.encodeStreamedBatched(None, slot, rows, local_ids.reshape(-1, wide).contiguous(), out,
                                         rows.shape[0])
        return out

    def reduce_fn(partials, weights, residual, row_index=None):
        t = weights.shape[0]
        y = torch.empty((t, d), dtype=torch.bfloat16, device=partials.device)
        reduce.encodeReduceTokenMajor(None, partials, weights, y, t, residual=residual, rowIndex=row_index)
        return y

    reduce_fn.indexed = True

    return router_fn, shared_fn, experts_fn, reduce_fn
