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
    """`rank` / `world`: this stage and the number of stages.  `group`: the process group of the stages that hold
    the same tensor-parallel shard (None: all ranks); `ranks`: its members' global ranks in stage order.

    On GPUs the transfers run on a side stream and are tied to the compute stream by events only: the receive of
    row range j + 1 and the send of range j - 1 are in flight while range j is being computed, every range has
    its own receive and send buffer, nothing on the compute stream waits for a transfer it does not consume."""

    def __init__(self, rank: int, world: int, group=None, microbatches: int = 1, ranks: Optional[List[int]] = None):
        self.rank, self.world, self.group, self.microbatches = rank, world, group, max(1, microbatches)
        self.first, self.last = rank == 0, rank == world - 1
        self.ranks = list(ranks) if ranks is not None else list(range(world))
        self.sends = 0
        self.comm_stream = None
        self._bufs = {}

    def _g(self, stage: int) -> int:
        return self.ranks[stage]

    def _slice(self, b: DeviceBatch, r0: int, r1: int) -> DeviceBatch:
        n = r1 - r0
        lr = torch.arange(n, dtype=torch.int32, device=b.token_ids.device)
        return DeviceBatch(b.token_ids[r0:r1], b.positions[r0:r1], b.write_slot[r0:r1], b.row_seq[r0:r1],
                           b.row_pos[r0:r1], b.block_table, lr, n, n)

    def _buf(self, kind: str, j: int, rows: int, hidden: int, dtype, dev) -> torch.Tensor:
        key = (kind, j)
        t = self._bufs.get(key)
        if t is None or t.shape[0] < rows or t.dtype != dtype:
            t = self._bufs[key] = torch.empty(max(rows, 1), hidden, dtype=dtype, device=dev)
        return t[:rows]

    def step(self, fwd, b: DeviceBatch, hidden: int, dtype, cuda: bool, allreduce=None, gather_vocab=None):
        """Runs the packed batch through all stages.  Returns (ids, vals) of the greedy tokens on every rank
        (float logit values as a second tensor).  `allreduce` / `gather_vocab`: the tensor-parallel reference
        collectives of a stage whose layers are sharded (host path; the GPU forward carries its own)."""
        T = b.n_rows
        m = self.microbatches if (b.n_logit == T and T >= self.microbatches) else 1
        bounds = [(j * T // m, (j + 1) * T // m) for j in range(m)]
        dev = b.token_ids.device
        if cuda:
            return self._step_cuda(fwd, b, bounds, hidden, dtype, dev)
        outs: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
        pending = []
        for (r0, r1) in bounds:
            mb = b if m == 1 else self._slice(b, r0, r1)
            n = r1 - r0
            if self.first:
                h = fwd.embed_rows(mb)
            else:
                h = torch.empty(n, hidden, dtype=dtype, device=dev)
                dist.recv(h, src=self._g(self.rank - 1), group=self.group)
            h = fwd.run_layers(h, mb, allreduce)
            if not self.last:
                hs = h.contiguous().clone()             # the stage's buffer is reused by the next range
                pending.append((dist.isend(hs, dst=self._g(self.rank + 1), group=self.group), hs))
                self.sends += 1
                outs.append(None)
            else:
                logits = fwd.logits_from_hidden(h, mb)
                if gather_vocab is not None:
                    logits = gather_vocab(logits)
                vals, ids = logits.max(-1)
                outs.append((ids.to(torch.int32), vals.float()))
        for work, _ in pending:
            work.wait()
        return self._broadcast(b, outs, dev)

    def _broadcast(self, b: DeviceBatch, outs, dev):
        L = b.n_logit
        ids = torch.empty(L, dtype=torch.int32, device=dev)
        vals = torch.empty(L, dtype=torch.float32, device=dev)
        if L == 0:
            return ids, vals
        if self.last:
            ids.copy_(torch.cat([o[0] for o in outs]))
            vals.copy_(torch.cat([o[1] for o in outs]))
        dist.broadcast(ids, src=self._g(self.world - 1), group=self.group)
        dist.broadcast(vals, src=self._g(self.world - 1), group=self.group)
        return ids, vals

    def _step_cuda(self, fwd, b: DeviceBatch, bounds, hidden: int, dtype, dev):
        main = torch.cuda.current_stream(dev)
        if self.comm_stream is None:
            self.comm_stream = torch.cuda.Stream(device=dev)
        comm = self.comm_stream
        m = len(bounds)
        outs: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
        # A stage whose layers are tensor-parallel runs kernels that wait for their peers from inside the kernel
        # (fused collectives) and, for large batches, collectives of a second communicator.  A transfer kernel that
        # sits on the GPU waiting for the neighbouring stage at the same time would share the machine with them for
        # an unbounded time, so such a stage keeps its transfers out of its compute: a receive is posted when its
        # range is due, and the next range starts after the send has left.
        overlap = getattr(fwd, "tp", None) is None

        def post_recv(j: int):
            r0, r1 = bounds[j]
            with torch.cuda.stream(comm):
                hin = self._buf("recv", j, r1 - r0, hidden, dtype, dev)
                dist.recv(hin, src=self._g(self.rank - 1), group=self.group)
                ev = torch.cuda.Event()
                ev.record(comm)
            return ev

        recv_ev = []
        if not self.first:
            comm.wait_stream(main)                       # the buffers' previous readers (the last step) are done
            if overlap:
                # all receives are posted up front on the side stream: range j + 1 arrives while range j computes
                recv_ev = [post_recv(j) for j in range(m)]
        send_done = []
        for j, (r0, r1) in enumerate(bounds):
            mb = b if m == 1 else self._slice(b, r0, r1)
            n = r1 - r0
            if self.first:
                h = fwd.embed_rows(mb, n)
            else:
                if not overlap:
                    comm.wait_stream(main)
                    recv_ev.append(post_recv(j))
                main.wait_event(recv_ev[j])
                h = self._buf("recv", j, n, hidden, dtype, dev)
            h = fwd.run_layers(h, mb, n)
            if not self.last:
                hs = self._buf("send", j, n, hidden, dtype, dev)
                hs.copy_(h)                              # the stage's activation buffer is reused by the next range
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    dist.send(hs, dst=self._g(self.rank + 1), group=self.group)
                    ev = torch.cuda.Event()
                    ev.record(comm)
                    send_done.append(ev)
                if not overlap:
                    main.wait_event(ev)
                self.sends += 1
                outs.append(None)
            else:
                ids, vals, _ = fwd.head(h, mb, fwd.w.final_norm)
                outs.append((ids.clone(), vals.clone()))
        for ev in send_done:
            main.wait_event(ev)                          # the send buffers are free for the next step
        return self._broadcast(b, outs, dev)
