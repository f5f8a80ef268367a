"""Pipeline parallelism: consecutive layer ranges on consecutive ranks, activations handed over with
point-to-point sends (NCCL on GPUs, gloo on CPU).

A stage owns `layers[lo:hi]`, its own KV pool for those layers (same page geometry on every stage, so
block tables and write slots are valid everywhere), the embedding on the first stage and the final norm +
LM head on the last.  One step: first stage embeds, every stage runs its layers, the hidden rows travel to
the next stage, the last stage produces the greedy tokens and broadcasts them.  With `microbatches > 1` a
decode batch is cut into row ranges that flow through the stages back to back: stage s works on range j
while its send of range j - 1 and the receive of range j + 1 are in flight (the transfers run on the
communication library's own streams).

The reference is single-GPU (its ParallelismPlan is inert:
crates/ferrule-model/src/support/policies.rs:56-77); this file is the pipeline-boundary row of the
parallelism inventory.
"""
from __future__ import annotations

import copy
from dataclasses import replace
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.deepseek import DeviceBatch
from ..models.weights import ModelWeights


def stage_range(n_layers: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous split; earlier stages take the remainder (they also hold the embedding)."""
    base, rem = divmod(n_layers, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def stage_weights(w: ModelWeights, rank: int, world: int) -> ModelWeights:
    """Weight image of one stage: its layers only; cfg.n_layers is the stage's count (the KV pool is sized from it)."""
    lo, hi = stage_range(len(w.layers), rank, world)
    out = copy.copy(w)
    out.layers = list(w.layers[lo:hi])
    out.cfg = replace(w.cfg, n_layers=hi - lo, n_mtp_layers=0)
    out.mtp = []
    return out


class PipelineParallel:
    def __init__(self, rank: int, world: int, group=None, microbatches: int = 1):
        self.rank, self.world, self.group, self.microbatches = rank, world, group, max(1, microbatches)
        self.first, self.last = rank == 0, rank == world - 1
        self.sends = 0

    def _slice(self, b: DeviceBatch, r0: int, r1: int) -> DeviceBatch:
        n = r1 - r0
        lr = torch.arange(n, dtype=torch.int32, device=b.token_ids.device)
        return DeviceBatch(b.token_ids[r0:r1], b.positions[r0:r1], b.write_slot[r0:r1], b.row_seq[r0:r1],
                           b.row_pos[r0:r1], b.block_table, lr, n, n)

    def step(self, fwd, b: DeviceBatch, hidden: int, dtype, cuda: bool):
        """Runs the packed batch through all stages.  Returns (ids, vals) of the greedy tokens on every rank
        (float logit values as a second tensor)."""
        T = b.n_rows
        m = self.microbatches if (b.n_logit == T and T >= self.microbatches) else 1
        bounds = [(j * T // m, (j + 1) * T // m) for j in range(m)]
        dev = b.token_ids.device
        outs: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
        pending = []
        for (r0, r1) in bounds:
            mb = b if m == 1 else self._slice(b, r0, r1)
            n = r1 - r0
            if self.first:
                h = fwd.embed_rows(mb, n) if cuda else fwd.embed_rows(mb)
            else:
                h = torch.empty(n, hidden, dtype=dtype, device=dev)
                dist.recv(h, src=self.rank - 1, group=self.group)
            h = fwd.run_layers(h, mb, n) if cuda else fwd.run_layers(h, mb)
            if not self.last:
                hs = h.contiguous().clone()             # the stage's buffer is reused by the next range
                pending.append((dist.isend(hs, dst=self.rank + 1, group=self.group), hs))
                self.sends += 1
                outs.append(None)
            else:
                if cuda:
                    ids, vals, _ = fwd.head(h, mb, fwd.w.final_norm)
                    outs.append((ids.clone(), vals.clone()))
                else:
                    logits = fwd.logits_from_hidden(h, mb)
                    vals, ids = logits.max(-1)
                    outs.append((ids.to(torch.int32), vals.float()))
        for work, _ in pending:
            work.wait()
        L = b.n_logit
        ids = torch.empty(L, dtype=torch.int32, device=dev)
        vals = torch.empty(L, dtype=torch.float32, device=dev)
        if self.last:
            ids.copy_(torch.cat([o[0] for o in outs]))
            vals.copy_(torch.cat([o[1] for o in outs]))
        dist.broadcast(ids, src=self.world - 1, group=self.group)
        dist.broadcast(vals, src=self.world - 1, group=self.group)
        return ids, vals
