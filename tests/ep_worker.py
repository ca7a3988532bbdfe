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
        run_case(rank, world, T, uniform)
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

    def combine(y_routes, probs, residual):
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


if __name__ == "__main__":
    main()
