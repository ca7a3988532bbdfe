"""Worker of the expert-parallel CPU test: one process per rank over gloo, the CPU oracle standing
in for the CUDA stages. Launched by tests/test_ep_gloo.py through torch.distributed.run."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oco_b200 import ep, synth  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # 11 tokens: ranks hold uneven shares; 12: equal shares; 2: with four ranks some hold no token at all
    for T, uniform in ((11, False), (12, True), (2, False)):
        run_case(rank, world, T, uniform and T % world == 0)     # equal shares only when the tokens divide evenly
    run_shared_case(rank, world, 9)
    descriptors_reach_every_rank(rank, world)
    for T in (11, 12, 2):
        run_window_case(rank, world, T)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


def run_case(rank, world, T, uniform):
    E, K, H, F = 8, 2, 64, 96
    layer = synth.make_layer(synth.ARCH_GPT_OSS, H, F, E, K, synth.FMT_MXFP4, seed=77)
    x_all, res_all = synth.make_tokens(H, T, 5, "normal")
    bounds = np.linspace(0, T, world + 1).astype(int)
    lo, hi = bounds[rank], bounds[rank + 1]
    epr = E // world
    e_lo = rank * epr

    def route(x):
        if x.shape[0] == 0:
            return torch.empty((0, K), dtype=torch.int32), torch.empty((0, K), dtype=torch.float32)
        _, ids, probs = oracle.router_gptoss(x.numpy().view(np.uint16), layer.router_w, layer.router_b, K)
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(probs)

    def experts(rows, local_ids):
        xr = rows.numpy().view(np.uint16)
        gids = local_ids.numpy().astype(np.uint32) + e_lo
        if len(gids) == 0:
            return torch.empty_like(rows)
        up = oracle.expert_up_tile(layer.up_w, xr, layer.up_b, 1.0, gids, 1, H, F)
        gate = oracle.expert_up_tile(layer.gate_w, xr, layer.gate_b, 0.0, gids, 1, H, F)
        act = oracle.moe_activate(gate, up)
        y = oracle.expert_down_tile(layer.down_w, act, layer.down_b, gids, F, H)
        return torch.from_numpy(y.view(np.int16))

    def combine(y_routes, probs, residual, shared_out=None):
        out = oracle.moe_sum(y_routes.numpy().view(np.uint16), probs.numpy(), residual.numpy().view(np.uint16), K)
        residual.copy_(torch.from_numpy(out.view(np.int16)))

    x = torch.from_numpy(x_all[lo:hi].view(np.int16).copy())
    res = torch.from_numpy(res_all[lo:hi].view(np.int16).copy())
    ep.forward(x, res, ep.Backend(route, experts, combine), E, uniform=uniform)
    ref = oracle.moe_forward(layer, x_all, res_all, mode=2)
    got = res.numpy().view(np.uint16)
    assert np.array_equal(got, ref.out[lo:hi]), f"rank {rank}: expert-parallel result differs from the single-process oracle"
    # the layout itself: routes leave grouped by destination rank, in ascending route order
    ids = torch.from_numpy(ref.ids[lo:hi].astype(np.int64))
    order, counts, local = ep.dispatch_layout(ids, world, epr)
    dest = (ids.reshape(-1) // epr)[order]
    assert torch.all(dest[1:] >= dest[:-1])
    for g in range(world):
        sel = order[dest == g]
        assert torch.all(sel[1:] > sel[:-1])
    assert counts.sum().item() == ids.numel() and torch.all(local < epr)


def run_shared_case(rank, world, T):
    """A layer with an always-on expert (Nemotron): the token owner computes it beside the exchange and the
    combine joins it as the tiled path does (bf16 add ahead of the routed sum)."""
    E, K, H, F, S = 8, 2, 64, 96, 128
    layer = synth.make_layer(synth.ARCH_NEMOTRON, H, F, E, K, synth.FMT_Q4_0, seed=79, shared_ffn=S, normalize=True, scale=2.5)
    x_all, res_all = synth.make_tokens(H, T, 7, "normal")
    bounds = np.linspace(0, T, world + 1).astype(int)
    lo, hi = bounds[rank], bounds[rank + 1]
    e_lo = rank * (E // world)

    def route(x):
        if x.shape[0] == 0:
            return torch.empty((0, K), dtype=torch.int32), torch.empty((0, K), dtype=torch.float32)
        _, ids, probs = oracle.router_sigmoid(x.numpy().view(np.uint16), layer.router_w, layer.router_b, K, True, 2.5)
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(probs)

    def experts(rows, local_ids):
        if rows.shape[0] == 0:
            return torch.empty_like(rows)
        gids = local_ids.numpy().astype(np.uint32) + e_lo
        up = oracle.expert_up_tile(layer.up_w, rows.numpy().view(np.uint16), None, 0.0, gids, 1, H, F, fmt=synth.FMT_Q4_0)
        v = np.maximum(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(up)), 0.0)
        act = (v * v).astype(np.float32).astype(np.float16).view(np.uint16)
        y = oracle.expert_down_tile(layer.down_w, act, None, gids, F, H, fmt=synth.FMT_Q4_0)
        return torch.from_numpy(y.view(np.int16))

    def shared(x):
        out = oracle.dense_forward(1, synth.FMT_Q4_0, H, S, layer.shared_up_w, None, layer.shared_down_w,
                                   x.numpy().view(np.uint16), tile=True)
        return torch.from_numpy(out.view(np.int16))

    def combine(y_routes, probs, residual, shared_out=None):
        res = residual.numpy().view(np.uint16)
        res = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(res) + synth.bf16_bits_to_f32(shared_out.numpy().view(np.uint16)[: len(res)]))
        out = oracle.moe_add(y_routes.numpy().view(np.uint16), probs.numpy(), res, None, K)
        residual.copy_(torch.from_numpy(out.view(np.int16)))

    x = torch.from_numpy(x_all[lo:hi].view(np.int16).copy())
    res = torch.from_numpy(res_all[lo:hi].view(np.int16).copy())
    ep.forward(x, res, ep.Backend(route, experts, combine, shared), E)
    ref = oracle.moe_forward(layer, x_all, res_all, mode=2)
    assert np.array_equal(res.numpy().view(np.uint16), ref.out[lo:hi]), f"rank {rank}: shared-expert layer differs from the single-process oracle"


def descriptors_reach_every_rank(rank, world):
    """ep.exchange_descriptors with plain files standing in for the memory handles."""
    import tempfile
    with tempfile.TemporaryFile() as f:
        f.write(f"slot of rank {rank}".encode())
        f.flush()
        fds = ep.exchange_descriptors(f.fileno())
        assert fds[rank] == f.fileno() and len(fds) == world
        for r, fd in enumerate(fds):
            if r == rank:
                continue
            assert os.pread(fd, 64, 0) == f"slot of rank {r}".encode()
            os.close(fd)
        dist.barrier()       # every peer has read before the file goes away


class SharedWindows:
    """ep.Windows on CPU ranks: the two windows are POSIX shared memory that every rank maps, laid out as
    the device windows are (slot strides from ep.window_geometry for a 4096-byte granularity)."""

    def __init__(self, hidden, top_k, max_tokens):
        from multiprocessing import shared_memory
        self.group = None
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.hidden, self.top_k, self.max_tokens = hidden, top_k, max_tokens
        self.slot_tokens, self.slot_routes = ep.window_geometry(hidden, top_k, max_tokens, 4096)
        self.cap_routes = max_tokens * top_k
        tag = [os.urandom(6).hex() if self.rank == 0 else None]
        dist.broadcast_object_list(tag, src=0)
        self._shm = []
        views = []
        for which, rows in (("x", self.slot_tokens), ("y", self.slot_routes)):
            name, size = f"oco_ep_test_{tag[0]}_{which}", self.world * rows * hidden * 2
            if self.rank == 0:
                shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            dist.barrier()
            if self.rank != 0:
                shm = shared_memory.SharedMemory(name=name)
                try:      # rank 0 owns the segment: the other ranks' resource trackers must not unlink it again
                    from multiprocessing import resource_tracker
                    resource_tracker.unregister(shm._name, "shared_memory")
                except Exception:
                    pass
            self._shm.append(shm)
            views.append(np.ndarray((self.world * rows, hidden), dtype=np.int16, buffer=shm.buf))
        self.x_all, self.y_all = views
        self.x_local = torch.from_numpy(self.x_all[self.rank * self.slot_tokens:][:max_tokens])
        self.y_local = torch.from_numpy(self.y_all[self.rank * self.slot_routes:][:self.cap_routes])
        self.ids_send = torch.full((self.cap_routes,), -1, dtype=torch.int32)
        self.ids_all = torch.empty((self.world * self.cap_routes,), dtype=torch.int32)
        self.ids_local = torch.empty_like(self.ids_all)
        self.arrived = torch.zeros(1)
        self._filled = 0

    def close(self):
        dist.barrier()
        self.x_local = self.y_local = self.x_all = self.y_all = None
        for shm in self._shm:
            shm.close()
        dist.barrier()
        if self.rank == 0:
            for shm in self._shm:
                shm.unlink()


def run_window_case(rank, world, T):
    """ep.forward_window over shared-memory windows, the oracle reading and writing rows by their labels as
    oco_moe_experts_window does; two steps in a row, the second with fewer tokens per rank."""
    E, K, H, F = 8, 2, 64, 96
    layer = synth.make_layer(synth.ARCH_GPT_OSS, H, F, E, K, synth.FMT_MXFP4, seed=78)
    x_all, res_all = synth.make_tokens(H, T, 6, "normal")
    bounds = np.linspace(0, T, world + 1).astype(int)
    cap = max(1, int(np.max(np.diff(bounds))))
    epr = E // world
    win = SharedWindows(H, K, cap)
    labels = ep.window_labels(world, win.cap_routes, win.slot_routes)

    class OracleBackend:
        pass

    be = OracleBackend()
    be.epr = epr

    def route(x):
        if x.shape[0] == 0:
            return torch.empty((0, K), dtype=torch.int32), torch.empty((0, K), dtype=torch.float32)
        _, ids, probs = oracle.router_gptoss(x.numpy().view(np.uint16), layer.router_w, layer.router_b, K)
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(probs)

    def experts_window(w):
        local = w.ids_local.numpy()
        mine = np.nonzero((local >= 0) & (local < epr))[0]
        if len(mine) == 0:
            return
        lab = labels[mine]
        xr = w.x_all[lab // K].view(np.uint16)
        gids = local[mine].astype(np.uint32) + rank * epr
        up = oracle.expert_up_tile(layer.up_w, xr, layer.up_b, 1.0, gids, 1, H, F)
        gate = oracle.expert_up_tile(layer.gate_w, xr, layer.gate_b, 0.0, gids, 1, H, F)
        y = oracle.expert_down_tile(layer.down_w, oracle.moe_activate(gate, up), layer.down_b, gids, F, H)
        w.y_all[lab] = y.view(np.int16)

    def combine(y_routes, probs, residual, shared_out=None):
        out = oracle.moe_sum(y_routes.numpy().view(np.uint16), probs.numpy(), residual.numpy().view(np.uint16), K)
        residual.copy_(torch.from_numpy(out.view(np.int16)))

    be.route, be.experts_window, be.combine = route, experts_window, combine
    for shrink in (1, 2):
        counts = [(bounds[g + 1] - bounds[g]) // shrink for g in range(world)]
        tok = np.concatenate([np.arange(bounds[g], bounds[g] + counts[g]) for g in range(world)]).astype(int)
        if len(tok) == 0:
            continue
        at, n = int(sum(counts[:rank])), counts[rank]
        x = torch.from_numpy(x_all[tok][at:at + n].view(np.int16).copy())
        res = torch.from_numpy(res_all[tok][at:at + n].view(np.int16).copy())
        ep.forward_window(x, res, be, win)
        ref = oracle.moe_forward(layer, x_all[tok], res_all[tok], mode=2)
        assert np.array_equal(res.numpy().view(np.uint16), ref.out[at:at + n]), \
            f"rank {rank}: window protocol differs from the single-process oracle (T {T}, shrink {shrink})"
    win.close()


if __name__ == "__main__":
    main()
