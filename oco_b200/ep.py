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

`forward_window` is the same layer without a collective on the rows' way (`forward` above is the
portable form and the one that runs on CPU ranks). Token rows and route outputs live in two windows
(`Windows`: one address range whose slot g is GPU g's memory, so a row has the same global number
on every rank):

    1. route        as above, on the rank's own rows, which sit in its slot of the token window
    2. ids          one all-gather of the expert ids (a few KB per rank); it also orders every
                    rank's rows before any peer's reads of them
    3. experts      oco_moe_experts_window over ALL ranks' routes: ids of other shards are skipped by
                    the route plan, the gather reads the owned routes' token rows from the peers'
                    slots (plain loads over NVLink), the down tiles store each output row into its
                    token owner's slot of the output window (plain stores)
    4. arrive       one all-reduce of a word: every rank's stores are complete
    5. combine      on the rank's own slot of the output window

No step waits on the host: nothing data-dependent is read back, all five are enqueued on the stream.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import socket
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
    ids [R]) -> y [R,H]; combine(y_routes [T*K,H], probs [T,K], residual [T,H], shared) updates
    residual in place. `shared` (optional): x [T,H] -> the always-on expert's output [T,H], computed
    by the rank that owns the tokens while the routed rows travel; combine receives it (else None).
    Rows are bf16 bit patterns held in int16 tensors."""
    route: Callable
    experts: Callable
    combine: Callable
    shared: Optional[Callable] = None


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
    shared_out = backend.shared(x) if backend.shared is not None and T else None
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
        backend.combine(y_routes, probs, residual, shared_out)
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
        self.shared = None
        if layer.shared_ffn:
            # the always-on expert belongs to the rank that owns the tokens: a dense feed-forward beside the routed
            # rows' journey, joined in the combine. At least two rows are reserved so that a rank with one token
            # still takes the tiles' arithmetic, as every other rank does.
            from . import dense
            self._shared_plan = dense.DensePlan(dense.FFN_RELU2, layer.fmt, layer.hidden, layer.shared_ffn)
            self._shared_plan.reserve(max(max_rows, 2), device)
            self._shared_plan.bind(layer.shared_up_w, None, layer.shared_down_w, device)
            self._shared_x = torch.zeros((2, layer.hidden), dtype=torch.int16, device=device)
            self._shared_y = torch.empty((max(max_rows, 2), layer.hidden), dtype=torch.int16, device=device)
            self.shared = self._shared_expert
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
        shard.shared_ffn, shard.shared_up_w, shard.shared_down_w = 0, None, None
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

    def experts_window(self, win: "Windows"):
        """Stage 3 of forward_window: every rank's routes, this shard's experts, rows through the windows."""
        p = self.expert_plan
        routes = win.world * win.cap_routes
        if routes > self.expert_rows * self.K:
            raise self._moe.OcoError(self._lib.UNSUPPORTED_SHAPE, f"{routes} routes exceed this rank's workspace")
        p._check(self._lib.lib().oco_moe_experts_window(
            p.handle, C.c_void_p(win.x_base), C.c_void_p(win.ids_local.data_ptr()), routes, self.K, win.cap_routes,
            win.slot_routes, win.cap_routes, C.c_void_p(win.y_base), self._stream()))

    def _shared_expert(self, x):
        T = x.shape[0]
        if T == 1:
            self._shared_x[0].copy_(x[0])
            x, T = self._shared_x, 2
        self._shared_plan.forward(x, self._shared_y, T)
        return self._shared_y

    def combine(self, y_routes, probs, residual, shared=None):
        p = self.router_plan
        if shared is not None:
            p._check(self._lib.lib().oco_moe_combine_shared(p.handle, C.c_void_p(y_routes.data_ptr()),
                                                           C.c_void_p(probs.contiguous().data_ptr()), C.c_void_p(shared.data_ptr()),
                                                           C.c_void_p(residual.data_ptr()), residual.shape[0], self._stream()))
            return
        p._check(self._lib.lib().oco_moe_combine(p.handle, C.c_void_p(y_routes.data_ptr()),
                                                C.c_void_p(probs.contiguous().data_ptr()),
                                                C.c_void_p(residual.data_ptr()), residual.shape[0], self._stream()))

    def launches(self) -> int:
        """Kernels launched by the last route, experts and combine calls together."""
        # combine runs on the router plan after route, so the router plan's count is combine's; the
        # route call before it launched one kernel (two on the first call of a weight set)
        return self.router_plan.launch_count() + 1 + self.expert_plan.launch_count()

    def backend(self) -> Backend:
        return Backend(self.route, self.experts, self.combine, self.shared)


# ---------------------------------------------------------------------------------------------
# Windows


def window_geometry(hidden: int, top_k: int, max_tokens: int, granularity: int):
    """(slot_tokens, slot_routes): token rows and route rows per window slot. A slot must start on a
    multiple of the allocation granularity in BOTH windows and hold whole rows, so slot_tokens is the
    smallest multiple of granularity / gcd(granularity, row bytes) that holds max_tokens; the output
    window's slot holds top_k rows per token."""
    row = hidden * 2
    unit = granularity // math.gcd(granularity, row)
    slot_tokens = (max_tokens + unit - 1) // unit * unit
    return slot_tokens, slot_tokens * top_k


def window_labels(world: int, cap_routes: int, slot_routes: int) -> np.ndarray:
    """Label of each entry of the gathered id list (source rank major, cap_routes per rank): the route's
    row in the output window, top_k times its token's row in the token window. The kernels compute the
    same from (seg_routes, seg_stride) = (cap_routes, slot_routes)."""
    i = np.arange(world * cap_routes, dtype=np.int64)
    return (i // cap_routes) * slot_routes + i % cap_routes


def exchange_descriptors(fd: int, group=None) -> list:
    """Every rank's file descriptor, received by every rank: passed as SCM_RIGHTS over abstract Unix
    sockets (the ranks are processes of one machine). Returns descriptors indexed by rank (own: fd)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    tag = [os.urandom(8).hex() if rank == 0 else None]
    dist.broadcast_object_list(tag, src=0, group=group)
    name = lambda r: f"\0oco_ep_{tag[0]}_{r}"
    listener = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    listener.bind(name(rank))
    listener.listen(world)
    _barrier(group)
    # connect to every peer first (a pending connection needs no accept yet), then serve, then receive
    conns = {}
    for r in range(world):
        if r != rank:
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.connect(name(r))
            conns[r] = c
    for _ in range(world - 1):
        served, _addr = listener.accept()
        socket.send_fds(served, [b"f"], [fd])
        served.close()
    fds = [fd] * world
    for r, c in conns.items():
        _msg, got, _flags, _addr = socket.recv_fds(c, 1, 1)
        fds[r] = got[0]
        c.close()
    listener.close()
    return fds


def _barrier(group):
    # an object all-gather: works on every backend without touching a device stream
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, 0, group=group)


class _DevicePointer:
    """Lets torch wrap device memory it did not allocate (zero copy)."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


class Windows:
    """The token window and the output window of one expert-parallel group, plus the small buffers of
    the id exchange. `max_tokens` is the most tokens a rank brings to one step (all ranks agree)."""

    def __init__(self, hidden: int, top_k: int, max_tokens: int, group=None, device=None):
        from . import _lib, moe
        self._lib = _lib
        lib = _lib.lib()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.hidden, self.top_k, self.max_tokens = hidden, top_k, max_tokens
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        gran = C.c_size_t()
        self._check(lib.oco_ep_window_granularity(C.byref(gran)))
        self.slot_tokens, self.slot_routes = window_geometry(hidden, top_k, max_tokens, gran.value)
        self.cap_routes = max_tokens * top_k
        row = hidden * 2
        self._handles = []
        self.x_base = self._make(self.slot_tokens * row, max_tokens * row)
        self.y_base = self._make(self.slot_routes * row, self.cap_routes * row)
        self.x_local = torch.as_tensor(_DevicePointer(self.x_base + self.rank * self.slot_tokens * row, (max_tokens, hidden), "<i2"),
                                       device=self.device)
        self.y_local = torch.as_tensor(_DevicePointer(self.y_base + self.rank * self.slot_routes * row, (self.cap_routes, hidden), "<i2"),
                                       device=self.device)
        self.ids_send = torch.full((self.cap_routes,), -1, dtype=torch.int32, device=self.device)
        self.ids_all = torch.empty((self.world * self.cap_routes,), dtype=torch.int32, device=self.device)
        self.ids_local = torch.empty_like(self.ids_all)
        self.arrived = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._filled = 0

    def _check(self, rc):
        if rc:
            from . import moe
            raise moe.OcoError(rc, self._lib.lib().oco_ep_window_error().decode())

    def _make(self, stride: int, backed: int) -> int:
        lib = self._lib.lib()
        h = C.c_void_p()
        self._check(lib.oco_ep_window_create(self.rank, self.world, stride, backed, C.byref(h)))
        self._handles.append(h)
        fds = exchange_descriptors(lib.oco_ep_window_fd(h), self.group)
        for r, fd in enumerate(fds):
            if r != self.rank:
                rc = lib.oco_ep_window_attach(h, r, fd)
                os.close(fd)
                self._check(rc)
        _barrier(self.group)
        return lib.oco_ep_window_base(h)

    def close(self):
        torch.cuda.synchronize()
        _barrier(self.group)      # no peer still reads or writes this rank's slots
        self.x_local = self.y_local = None
        for h in self._handles:
            self._lib.lib().oco_ep_window_destroy(h)
        self._handles = []


def forward_window(x: torch.Tensor, residual: torch.Tensor, backend: "CudaBackend", win: Windows,
                   timings: Optional[dict] = None) -> None:
    """One expert-parallel MoE layer over this rank's tokens through the windows. x (int16 [T, H]) is
    copied into the rank's slot unless it already is `win.x_local[:T]`; residual int16 [T, H] is
    updated in place. T may differ between ranks and steps, up to win.max_tokens."""
    T, K = x.shape[0], win.top_k
    if T > win.max_tokens:
        raise ValueError(f"{T} tokens exceed the windows' capacity of {win.max_tokens}")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if timings is not None else None
    if ev:
        ev[0].record()
    xs = win.x_local[:T]
    if T and x.data_ptr() != xs.data_ptr():
        xs.copy_(x)
    ids, probs = backend.route(xs)
    if win._filled > T * K:
        win.ids_send[T * K: win._filled].fill_(-1)     # ids of a fuller earlier step
    if T:
        win.ids_send[: T * K].copy_(ids.reshape(-1))
    win._filled = T * K
    dist.all_gather_into_tensor(win.ids_all, win.ids_send, group=win.group)
    if ev:
        ev[1].record()
    shared = getattr(backend, "shared", None)
    shared_out = shared(xs) if shared is not None and T else None
    # shard numbering: an id of another shard (or the padding) leaves 0 .. experts_per_rank - 1 and is skipped
    torch.sub(win.ids_all, win.rank * backend.epr, out=win.ids_local)
    backend.experts_window(win)
    if ev:
        ev[2].record()
    dist.all_reduce(win.arrived, group=win.group)
    if ev:
        ev[3].record()
    if T:
        backend.combine(win.y_local[: T * K], probs, residual, shared_out)
    if ev:
        ev[4].record()
        torch.cuda.synchronize()
        timings["route_ids_ms"] = ev[0].elapsed_time(ev[1])
        timings["experts_ms"] = ev[1].elapsed_time(ev[2])
        timings["arrive_ms"] = ev[2].elapsed_time(ev[3])
        timings["combine_ms"] = ev[3].elapsed_time(ev[4])
