"""Expert-parallel routed-MoE layer: one process per GPU, experts sharded by id, tokens data-parallel.

The reference runs on one GPU and has no counterpart of this file; the arithmetic per token is still the MoE branch
of its layer body (src/kimi_exec.cu:836-877).  Expert e lives on rank e // (experts / world).  Per step:

  1. every rank routes its own tokens (router replicated),
  2. dispatch: each (token, slot) assignment travels to the owner of its expert   -- all-to-all #1 (+ counts)
  3. the owner runs its local experts on what it received (grouped W4A16 GEMM),
  4. combine: the per-assignment outputs travel back                              -- all-to-all #2
  5. the token's rank applies the routing weights in slot order and adds its shared expert (replicated).

torch.distributed (NCCL over NVLink/NVSwitch on GPUs, gloo in the CPU tests) is the plumbing; the compute steps are
callables so that the same dispatch/combine logic is exercised on the CPU with stand-in experts.  Receive buffers are
ordinary local tensors: no kernel ever reads a peer's memory.
"""
import torch
import torch.distributed as dist


class RoutingError(RuntimeError):
    pass


def plan_dispatch(ids, experts, world):
    """ids int [T, topk] (global expert ids).  Returns (order, send_counts, local_expert):
    order        [T*topk] assignment indices sorted by destination rank (stable, so ascending assignment id per rank)
    send_counts  [world]  assignments per destination rank
    local_expert [T*topk] expert id on its owner (id % experts_per_rank), in send order."""
    if experts % world:
        raise RoutingError("experts (%d) must divide evenly over %d ranks" % (experts, world))
    per = experts // world
    flat = ids.reshape(-1).to(torch.int64)
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= experts):
        raise RoutingError("expert id outside [0, %d)" % experts)
    dest = flat // per
    order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=world)
    return order, send_counts, (flat[order] % per).to(torch.int32)


class ExpertParallelMoe:
    """router_fn(x) -> (ids [T, topk] int, wts [T, topk] f32)
    experts_fn(rows [N, H], local_expert int32 [N]) -> [N, H]   (this rank's experts, unweighted)
    combine_fn(y_assign [T*topk, H], wts, shared or None) -> [T, H]
    shared_fn(x) -> [T, H] or None"""

    def __init__(self, router_fn, experts_fn, combine_fn, shared_fn, experts, topk, group=None):
        self.router_fn, self.experts_fn, self.combine_fn, self.shared_fn = router_fn, experts_fn, combine_fn, shared_fn
        self.experts, self.topk, self.group = experts, topk, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.last_stats = {}

    def _all_to_all(self, send, send_counts, recv_counts):
        recv = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
        if self.world == 1:
            recv.copy_(send)
            return recv
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=self.group)
        return recv

    def _side_stream(self, device):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=device)
        return self._side

    def forward(self, x):
        T, H = x.shape
        # The shared expert needs nothing from the exchange: on a GPU it runs on a side stream while the tokens travel.
        shared, side = None, None
        if self.shared_fn is not None and x.is_cuda:
            side = self._side_stream(x.device)
            side.wait_stream(torch.cuda.current_stream(x.device))
            with torch.cuda.stream(side):
                shared = self.shared_fn(x)
        ids, wts = self.router_fn(x)
        ids64 = ids.to(torch.int64) & 0xFFFF if ids.dtype == torch.int16 else ids.to(torch.int64)
        # Plan and counts with ONE wait for the device: the per-destination counts and the number of ids outside the
        # expert range travel together, every rank gathers every rank's row, and a bad id is reported on all ranks
        # (none is left waiting in a collective for a peer that raised).
        per = self.experts // self.world
        flat = ids64.reshape(-1)
        bad = (flat < 0) | (flat >= self.experts)
        dest = torch.where(bad, torch.zeros_like(flat), flat) // per
        order = torch.sort(dest, stable=True).indices
        local_e = (flat[order] % per).to(torch.int32)
        meta = torch.cat([torch.bincount(dest, minlength=self.world), bad.sum().view(1)])
        if self.world > 1:
            table = [torch.empty_like(meta) for _ in range(self.world)]
            dist.all_gather(table, meta, group=self.group)
            table = torch.stack(table).tolist()
        else:
            table = [meta.tolist()]
        culprits = [r for r in range(self.world) if table[r][self.world]]
        if culprits:
            raise RoutingError("expert id outside [0, %d) on rank(s) %s" % (self.experts, culprits))
        send_counts = [int(v) for v in table[self.rank][:self.world]]
        recv_counts = [int(table[r][self.rank]) for r in range(self.world)]
        rows = x.index_select(0, (order // self.topk).to(x.device))
        recv_rows = self._all_to_all(rows, send_counts, recv_counts)
        recv_e = self._all_to_all(local_e.to(x.device), send_counts, recv_counts)
        y_recv = self.experts_fn(recv_rows, recv_e.contiguous())
        if y_recv.shape[0] != recv_rows.shape[0]:
            raise RoutingError("experts_fn returned %d rows for %d assignments" % (y_recv.shape[0], recv_rows.shape[0]))
        y_back = self._all_to_all(y_recv.contiguous(), recv_counts, send_counts)
        y_assign = torch.empty_like(y_back)
        y_assign.index_copy_(0, order.to(x.device), y_back)        # back to assignment order t*topk + k
        if side is not None:
            torch.cuda.current_stream(x.device).wait_stream(side)
            shared.record_stream(torch.cuda.current_stream(x.device))
        elif self.shared_fn is not None:
            shared = self.shared_fn(x)
        remote = sum(c for r, c in enumerate(send_counts) if r != self.rank)
        self.last_stats = dict(assignments=T * self.topk, remote=remote, bytes_each_way=remote * H * x.element_size(),
                               received=int(sum(recv_counts)))
        return self.combine_fn(y_assign, wts, shared)


def gpu_layer(layer_weights, experts, topk=8, routed_scale=2.827, max_tokens=2048, group=None):
    """The GPU product path: this rank's shard of the experts in a blok_b200 MoeLayer, router and shared expert replicated."""
    from . import lib
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    per = experts // world
    layer = lib.MoeLayer(layer_weights, topk=topk, routed_scale=routed_scale, expert_base=rank * per,
                         max_tokens=max(max_tokens, 2) * (world if world > 1 else 1))
    w = layer.weights
    ep = ExpertParallelMoe(
        router_fn=lambda x: lib.router(w["router_w"], w["router_bias"], x, topk=topk, routed_scale=routed_scale),
        experts_fn=lambda rows, e: layer.experts_grouped(rows, e),
        combine_fn=lambda y, wts, sh: lib.moe_combine(y, wts, sh),
        shared_fn=(lambda x: layer.shared(x)) if w.get("shared_gate") is not None else None,
        experts=experts, topk=topk, group=group)
    ep.layer = layer
    return ep
