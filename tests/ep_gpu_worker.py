"""Worker of the expert-parallel GPU test: one process per GPU over NCCL, the C-ABI stage calls
(route, experts, combine) doing the arithmetic, first around the all-to-all exchange, then through
the windows over peer memory. Launched by tests/test_gpu_ep.py through
torch.distributed.run; the oracle checks each rank's rows."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oco_b200 import ep, synth  # noqa: E402

REL_L2 = 1e-3


def rel_l2(got_bits, ref_bits):
    g = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    r = synth.bf16_bits_to_f32(ref_bits).astype(np.float64)
    return np.linalg.norm(g - r) / max(np.linalg.norm(r), 1e-30)


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    # tokens divisible by the world size also run the protocol for equal shares (ids gathered once)
    cases = [(synth.ARCH_GPT_OSS, 16, 4, 320, 288, 203, synth.FMT_MXFP4),
             (synth.ARCH_GPT_OSS, 16, 4, 320, 288, 200, synth.FMT_MXFP4),
             (synth.ARCH_GPT_OSS, 8, 2, 64, 96, 11, synth.FMT_MXFP4),
             (synth.ARCH_GPT_OSS, 32, 4, 320, 288, 16, synth.FMT_MXFP4),
             (synth.ARCH_NEMOTRON, 16, 6, 256, 192, 150, synth.FMT_Q4_0),
             (synth.ARCH_NEMOTRON, 16, 6, 256, 192, 3, synth.FMT_Q4_0)]
    for n, (arch, E, K, H, F, T, fmt) in enumerate(cases):
        # the Nemotron cases carry the always-on expert, computed by the rank that owns the tokens
        layer = synth.make_layer(arch, H, F, E, K, fmt, seed=31 + n, shared_ffn=320 if arch == synth.ARCH_NEMOTRON else 0,
                                 normalize=arch == synth.ARCH_NEMOTRON, scale=2.5 if arch == synth.ARCH_NEMOTRON else 1.0)
        x_all, res_all = synth.make_tokens(H, T, 9 + n, "normal")
        bounds = np.linspace(0, T, world + 1).astype(int)
        lo, hi = bounds[rank], bounds[rank + 1]
        be = ep.CudaBackend(layer, rank, world, max_rows=T)
        x = torch.from_numpy(x_all[lo:hi].view(np.int16).copy()).cuda()
        res = torch.from_numpy(res_all[lo:hi].view(np.int16).copy()).cuda()
        ep.forward(x, res, be.backend(), E, uniform=T % world == 0)
        torch.cuda.synchronize()
        be.router_plan.poll(); be.expert_plan.poll()
        ref = oracle.moe_forward(layer, x_all, res_all, mode=2)
        got = res.cpu().numpy().view(np.uint16)
        err = rel_l2(got, ref.out[lo:hi])
        assert err <= REL_L2, f"rank {rank} case {n}: rel-L2 {err}"
        ids, _ = be.route(x)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref.ids[lo:hi].astype(np.uint32)), "expert ids differ"
        # the same layer through the windows (rows read from and written to the peers' memory by the expert
        # stage itself), with the route plan made by one CTA and by many; then a step with fewer tokens on
        # every rank, whose id list is shorter than the one before it
        cap = int(np.max(np.diff(bounds)))
        for single_max in ("2048", "0"):
            os.environ["OCO_MOE_ROUTE_PLAN_SINGLE_MAX"] = single_max
            bw = ep.CudaBackend(layer, rank, world, max_rows=max(cap, 1))
            del os.environ["OCO_MOE_ROUTE_PLAN_SINGLE_MAX"]
            win = ep.Windows(H, K, max(cap, 1))
            res_w = torch.from_numpy(res_all[lo:hi].view(np.int16).copy()).cuda()
            ep.forward_window(x, res_w, bw, win)
            torch.cuda.synchronize()
            bw.router_plan.poll(); bw.expert_plan.poll()
            err = rel_l2(res_w.cpu().numpy().view(np.uint16), ref.out[lo:hi])
            assert err <= REL_L2, f"rank {rank} case {n} (windows, single_max {single_max}): rel-L2 {err}"
            keep = (hi - lo) // 2
            tok = np.concatenate([np.arange(bounds[g], bounds[g] + (bounds[g + 1] - bounds[g]) // 2) for g in range(world)])
            ref2 = oracle.moe_forward(layer, x_all[tok], res_all[tok], mode=2)
            at = int(sum((bounds[g + 1] - bounds[g]) // 2 for g in range(rank)))
            res_2 = torch.from_numpy(res_all[lo:lo + keep].view(np.int16).copy()).cuda()
            ep.forward_window(x[:keep], res_2, bw, win)
            torch.cuda.synchronize()
            bw.router_plan.poll(); bw.expert_plan.poll()
            if keep:
                err = rel_l2(res_2.cpu().numpy().view(np.uint16), ref2.out[at:at + keep])
                assert err <= REL_L2, f"rank {rank} case {n} (windows, shorter step): rel-L2 {err}"
            win.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
