"""Multi-rank check + timing of the expert-parallel MoE (launch with torch.distributed.run, one rank per GPU):
fused peer-memory path and NCCL all-to-all baseline against a single-device PyTorch oracle on the same
routes.  Prints one JSON line on rank 0."""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def oracle(x, idx, wts, w13, w2, residual, extra):
    """fp32 math with the kernels' rounding points (bf16 after SwiGLU and after the weighted expert output)."""
    T, H = x.shape
    I = w13.shape[1] // 2
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for t in range(T):
        for s in range(idx.shape[1]):
            e = int(idx[t, s])
            y = x[t].float() @ w13[e].float().T
            h = (torch.nn.functional.silu(y[:I]) * y[I:]).bfloat16().float()
            out[t] += ((h @ w2[e].float().T) * wts[t, s]).bfloat16().float()
    if extra is not None:
        out += extra.float()
    if residual is not None:
        out += residual.float()
    return out


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from ferrule_b200.ops import _lib
    from ferrule_b200.parallel.ep import ExpertParallelMoE
    H, I, k, E, T = 1024, 512, 4, 8 * world, 24
    g = torch.Generator().manual_seed(7)
    w13_all = (torch.randn(E, 2 * I, H, generator=g) * 0.03).bfloat16()
    w2_all = (torch.randn(E, H, I, generator=g) * 0.03).bfloat16()
    el = E // world
    w13, w2 = w13_all[rank * el:(rank + 1) * el].to(dev).contiguous(), w2_all[rank * el:(rank + 1) * el].to(dev).contiguous()
    res = {"world": world, "checks": {}}
    ok = True
    for fused in (True, False):
        ep = ExpertParallelMoE(rank, world, dev, H, I, k, E, max_local_tokens=32, fused=fused, allgather=True)
        for step in range(3):
            gs = torch.Generator().manual_seed(100 * step + rank)
            Tl = T - 3 * rank if step == 1 else T                       # ragged token counts per rank
            x = (torch.randn(Tl, H, generator=gs) * 0.5).bfloat16().to(dev)
            idx = torch.stack([torch.randperm(E, generator=gs)[:k] for _ in range(Tl)]).int().to(dev)
            if step == 2:
                idx[:, 0] = 0                                             # skew: everything also hits rank 0
            wts = torch.rand(Tl, k, generator=gs).to(dev)
            resid = (torch.randn(Tl, H, generator=gs) * 0.5).bfloat16().to(dev)
            extra = (torch.randn(Tl, H, generator=gs) * 0.1).bfloat16().to(dev)
            got = ep.forward(x, idx, wts, w13, w2, residual=resid, extra=extra, allgather=fused)
            gathered = None
            if isinstance(got, tuple):
                got, gathered = got
            torch.cuda.synchronize()
            want = oracle(x, idx, wts, w13_all.to(dev), w2_all.to(dev), resid, extra)
            err = float((got.float() - want).abs().max())
            scale = float(want.abs().max())
            name = f"{'fused' if fused else 'nccl'}_step{step}_err"
            res["checks"][name] = err
            ok &= err <= 0.02 * scale + 1e-2
            if gathered is not None:
                # every rank must see every rank's rows
                mine = torch.zeros(32, H, dtype=torch.bfloat16, device=dev)
                mine[:Tl] = got
                allv = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(allv, mine)
                lens = torch.tensor([Tl], device=dev)
                all_l = [torch.empty_like(lens) for _ in range(world)]
                dist.all_gather(all_l, lens)
                for r in range(world):
                    n = int(all_l[r])
                    ok &= bool(torch.equal(gathered[r, :n], allv[r][:n]))
                res["checks"][f"allgather_step{step}"] = bool(ok)
        # timing: decode-sized call, device events, max over ranks
        x = (torch.randn(T, H) * 0.5).bfloat16().to(dev)
        idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).int().to(dev)
        wts = torch.rand(T, k).to(dev)
        for _ in range(5):
            ep.forward(x, idx, wts, w13, w2)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(50):
            ep.forward(x, idx, wts, w13, w2)
        e1.record()
        torch.cuda.synchronize()
        tms = torch.tensor([e0.elapsed_time(e1) / 50], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        res[f"{'fused' if fused else 'nccl'}_us_per_call"] = round(float(tms) * 1e3, 1)
        dist.barrier()
    st = _lib.read_status()
    res["device_status"] = st
    ok &= st[0] == 0
    flags = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    res["ok"] = bool(int(flags))
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
