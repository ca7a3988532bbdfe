"""Expert parallelism for large-expert-count layers: experts sharded over the ranks of a process
group, tokens data-parallel, one all-to-all each way.

The reference is single-device; this extends its tiled operator (router -> route plan -> expert
tiles -> weighted sum, `src/weights/compute/feed_forward.rs:165-274`) by putting an exchange
between the stages:

    1. route        every rank routes its own tokens (router weights replicated)
    2. dispatch     routes sorted by destination rank (stable, so rows arrive ordered by source
                    rank and route index); counts exchanged; rows and local expert ids sent with
                    all_to_all_single
    3. experts      each rank runs its expert shard on the rows it received
    4. combine      outputs travel back with the reverse all-to-all, are put back in route order
                    and summed with the routing weights onto the residual

Rank g of N owns experts [g * E/N, (g+1) * E/N). The index arithmetic (`dispatch_layout`) is plain
integer code shared by the CPU test (gloo ranks, the oracle standing in for the kernels) and the
GPU path (NCCL over NVLink, the C-ABI stage calls).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch
import torch.distributed as dist


def dispatch_layout(ids: torch.Tensor, n_ranks: int, experts_per_rank: int):
    """ids: integer tensor [T, K] of global expert ids. Returns (order, send_counts, local_ids):
    `order` lists the route indices (t * K + r) grouped by destination rank, ascending within a
    rank; send_counts[g] routes go to rank g; local_ids are the expert ids within the owner's
    shard, in `order`."""
    routes = ids.reshape(-1).to(torch.int64)
    dest = routes // experts_per_rank
    order = torch.sort(dest, stable=True).indices
    send_counts = torch.bincount(dest, minlength=n_ranks)
    local_ids = (routes - dest * experts_per_rank)[order]
    return order, send_counts, local_ids


@dataclass
class Backend:
    """The three compute stages. route(x) -> (ids [T,K], probs [T,K]); experts(rows [R,H], local
    ids [R]) -> y [R,H]; combine(y_routes [T*K,H], probs [T,K], residual [T,H]) updates residual in
    place. Rows are bf16 bit patterns held in int16 tensors."""
    route: Callable
    experts: Callable
    combine: Callable


def forward(x: torch.Tensor, residual: torch.Tensor, backend: Backend, experts_total: int,
            group: Optional[dist.ProcessGroup] = None, timings: Optional[dict] = None,
            exchange: Optional[Callable] = None, uniform: bool = False) -> None:
    """One expert-parallel MoE layer over this rank's tokens. x, residual: int16 [T, H].
    `exchange` has the signature of `dist.all_to_all_single` and replaces it when given (a
    benchmark passes a local stand-in to find how much of the step the exchange costs).
    `uniform`: every rank holds the same number of tokens; the ranks then gather each other's
    expert ids once (a few KB) instead of exchanging counts and ids per destination."""
    a2a = exchange or dist.all_to_all_single
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    epr = experts_total // world
    T, H = x.shape
    ids, probs = backend.route(x)         # a rank without tokens still takes part in every exchange
    K = ids.shape[1]
    order, send_counts, local_ids = dispatch_layout(ids, world, epr)
    send_rows = x.index_select(0, order // K)
    if uniform and exchange is None:
        ids_flat = torch.empty(world * T * K, dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(ids_flat, ids.reshape(-1).to(torch.int32).contiguous(), group=group)
        ids_all = ids_flat.view(world, T * K)
        mine = (ids_all // epr) == rank                      # [world, T*K]: routes each rank sends here
        recv_counts = mine.sum(dim=1)
        recv_ids = (ids_all[mine] - rank * epr).to(torch.int32)   # row-major: by source rank, then route order
        send_split = send_counts.tolist()
        recv_split = recv_counts.tolist()
        R = int(sum(recv_split))
    else:
        # counts first, then the rows and their expert ids
        recv_counts = torch.empty_like(send_counts)
        a2a(recv_counts, send_counts, group=group)
        send_split = send_counts.tolist()
        recv_split = recv_counts.tolist()
        R = int(sum(recv_split))
        recv_ids = torch.empty(R, dtype=torch.int32, device=x.device)
        a2a(recv_ids, local_ids.to(torch.int32), recv_split, send_split, group=group)
    ev = None
    if timings is not None and x.is_cuda:
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        ev[0].record()
    recv_rows = torch.empty((R, H), dtype=x.dtype, device=x.device)
    # rows travel as bytes: every backend moves uint8, not every one moves 16-bit integers
    a2a(recv_rows.view(torch.uint8), send_rows.contiguous().view(torch.uint8), recv_split, send_split, group=group)
    if ev:
        ev[1].record()
    y_recv = backend.experts(recv_rows, recv_ids)
    if ev:
        ev[2].record()
    y_back = torch.empty((T * K, H), dtype=x.dtype, device=x.device)
    a2a(y_back.view(torch.uint8), y_recv.contiguous().view(torch.uint8), send_split, recv_split, group=group)
    if ev:
        ev[3].record()
    y_routes = torch.empty_like(y_back)
    y_routes.index_copy_(0, order, y_back)           # back to route order
    if T:
        backend.combine(y_routes, probs, residual)
    if ev:
        torch.cuda.synchronize()
        timings["dispatch_ms"] = ev[0].elapsed_time(ev[1])
        timings["experts_ms"] = ev[1].elapsed_time(ev[2])
        timings["combine_a2a_ms"] = ev[2].elapsed_time(ev[3])
        timings["routes_received"] = R


class CudaBackend:
    """The stages through liboco_moe.so: a router-only plan over all experts and an expert plan
    over this rank's shard."""

    def __init__(self, layer, rank: int, world: int, max_rows: int, device="cuda"):
        from . import _lib, moe, synth
        self._lib, self._moe = _lib, moe
        E = layer.experts
        assert E % world == 0, "experts must divide evenly over the ranks"
        if layer.shared_ffn:
            # the always-on expert belongs to the token-owning rank, beside the routed sum; this protocol moves
            # routed rows only, so a layer with a shared expert is refused rather than silently losing that term
            raise moe.OcoError(_lib.UNSUPPORTED_SHAPE, "expert parallelism does not run layers with a shared expert")
        self.epr = E // world
        lo, hi = rank * self.epr, (rank + 1) * self.epr
        self.layer = layer
        self.K = layer.top_k
        # router plan: all experts, router weights only
        self.router_plan = moe._Plan(layer.arch, layer.hidden, layer.ffn, E, layer.top_k, layer.fmt,
                                     normalize=layer.normalize, scale=layer.scale)
        self.router_w = moe._Weights(router_w=moe._dev_bytes(layer.router_w, device),
                                     router_b=moe._dev_bytes(layer.router_b, device))
        self.router_plan.reserve(max_rows, device)
        self.router_plan.bind(self.router_w)
        # expert plan: this rank's shard (the packed spans of experts lo..hi, unchanged)
        shard = synth.Layer(**{**layer.__dict__})
        shard.experts = self.epr
        for name in ("gate_w", "up_w", "down_w", "gate_b", "up_b", "down_b"):
            a = getattr(layer, name)
            setattr(shard, name, None if a is None else a[lo:hi])
        shard.router_w = shard.router_b = None
        self.expert_plan = moe._Plan(layer.arch, layer.hidden, layer.ffn, self.epr, layer.top_k, layer.fmt,
                                     normalize=layer.normalize, scale=layer.scale)
        self.expert_w = moe._Weights.from_layer(shard, device)
        # every route of the whole job may land here in the worst case; size for the expected load with slack
        self.expert_rows = max_rows * world
        self.expert_plan.reserve(self.expert_rows, device)
        self.expert_plan.bind(self.expert_w)

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def route(self, x):
        T = x.shape[0]
        if T == 0:
            return (torch.empty((0, self.K), dtype=torch.int32, device=x.device),
                    torch.empty((0, self.K), dtype=torch.float32, device=x.device))
        p = self.router_plan
        p._check(self._lib.lib().oco_moe_route(p.handle, C.c_void_p(x.data_ptr()), T, self._stream()))
        v = self._lib.RoutingView()
        self._lib.lib().oco_moe_routing(p.handle, C.byref(v))
        # views into the plan's workspace (valid until the next call on it)
        base = p.workspace.data_ptr()
        n = T * self.K
        ids = p.workspace[v.ids - base: v.ids - base + 4 * n].view(torch.int32).reshape(T, self.K)
        probs = p.workspace[v.probs - base: v.probs - base + 4 * n].view(torch.float32).reshape(T, self.K)
        return ids, probs

    def experts(self, rows, local_ids):
        R = rows.shape[0]
        y = torch.empty_like(rows)
        if R:
            if R > self.expert_rows * self.K:
                raise self._moe.OcoError(self._lib.UNSUPPORTED_SHAPE, f"{R} routes exceed this rank's workspace")
            p = self.expert_plan
            p._check(self._lib.lib().oco_moe_experts(p.handle, C.c_void_p(rows.data_ptr()),
                                                    C.c_void_p(local_ids.data_ptr()), R, C.c_void_p(y.data_ptr()),
                                                    self._stream()))
        return y

    def combine(self, y_routes, probs, residual):
        p = self.router_plan
        p._check(self._lib.lib().oco_moe_combine(p.handle, C.c_void_p(y_routes.data_ptr()),
                                                C.c_void_p(probs.contiguous().data_ptr()),
                                                C.c_void_p(residual.data_ptr()), residual.shape[0], self._stream()))

    def launches(self) -> int:
        """Kernels launched by the last route, experts and combine calls together."""
        # combine runs on the router plan after route, so the router plan's count is combine's; the
        # route call before it launched one kernel (two on the first call of a weight set)
        return self.router_plan.launch_count() + 1 + self.expert_plan.launch_count()

    def backend(self) -> Backend:
        return Backend(self.route, self.experts, self.combine)
