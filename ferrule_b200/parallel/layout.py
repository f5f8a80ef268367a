"""Rank layout of one model replica: `pp` pipeline stages of `tp` tensor-parallel ranks each.

Global rank = stage * tp + tensor rank.  Tensor-parallel groups hold the ranks of one stage (they share the
fused collectives' peer memory), pipeline groups the ranks with the same tensor rank (they hand activations to
each other).  `build_parallel` creates the process groups and the `TensorParallel` / `PipelineParallel` objects
a `DeepSeekRunner` takes.

The reference keeps six inert degrees in its ParallelismPlan (crates/ferrule-model/src/support/policies.rs:56-77);
this is the part of that plan this build executes inside one replica.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch.distributed as dist


@dataclass
class ParallelLayout:
    pp_rank: int
    tp_rank: int
    pp_size: int
    tp_size: int
    tp: Optional[object]          # parallel.tp.TensorParallel (None when tp_size == 1)
    pp: Optional[object]          # parallel.pp.PipelineParallel (None when pp_size == 1)
    tp_ranks: List[int]
    pp_ranks: List[int]


def build_parallel(rank: int, world: int, device, pp: int = 1, tp: Optional[int] = None, microbatches: int = 1,
                   payload: str = "bf16", fused: bool = True, collective: str = "ll",
                   multicast_push: bool = False) -> ParallelLayout:
    tp = world // pp if tp is None else tp
    if pp * tp != world:
        raise ValueError(f"{pp} stages x {tp} tensor ranks != {world} ranks")
    pp_rank, tp_rank = divmod(rank, tp)
    tp_groups = [list(range(s * tp, (s + 1) * tp)) for s in range(pp)]
    pp_groups = [[s * tp + t for s in range(pp)] for t in range(tp)]
    # every rank creates every group (collective call), in the same order
    tp_pg = [dist.new_group(g) for g in tp_groups] if (pp > 1 and tp > 1) else None
    pp_pg = [dist.new_group(g) for g in pp_groups] if (pp > 1 and tp > 1) else None
    tpo = ppo = None
    if tp > 1:
        from .tp import TensorParallel
        tpo = TensorParallel(tp_rank, tp, device, fused=fused, payload=payload, collective=collective,
                             multicast_push=multicast_push, group=tp_pg[pp_rank] if tp_pg else None)
    if pp > 1:
        from .pp import PipelineParallel
        ppo = PipelineParallel(pp_rank, pp, group=pp_pg[tp_rank] if pp_pg else None, microbatches=microbatches,
                               ranks=pp_groups[tp_rank])
    return ParallelLayout(pp_rank, tp_rank, pp, tp, tpo, ppo, tp_groups[pp_rank], pp_groups[tp_rank])
