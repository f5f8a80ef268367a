"""Model runner: binds the DeepSeek forward pass to the runtime's transaction contract.

Per transaction: physical copy-on-write page copies, one host->device copy of the packed
batch metadata from pinned memory, the forward pass (a captured CUDA graph for pure decode
batches, eager kernels otherwise), one device->host copy of the greedy result.  The CPU
path runs the PyTorch reference forward through exactly the same interface.

Counterpart of crates/ferrule-model/src/models/deepseek_v4/runner.rs:577-617 (runner),
:4322-4517 (prepare / end_transaction), :4842-4956 (execute) and the async top-k download of
cuda_cache.rs:3539-3700.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..runtime.execution import (ExecutionBatch, ExecutionCapabilities, ExecutionOutput, Intent, KvLayoutSchema,
                                 KvPlaneDescriptor, LogitsKind, RowOutput)
from ..runtime.runner import Complete, EndIntent, EndStatus, ModelRunner, Proposal
from .config import ModelConfig
from .deepseek import CudaForward, DecodeGraph, DeviceBatch, KvPool, ReferenceForward
from .weights import ModelWeights


class BatchStaging:
    """Pinned host mirror + device buffer of one packed batch; tensors of `DeviceBatch` are views.

    Layout (int32 words): write_slot (int64, 2R) | token_ids R | positions R | row_seq R | row_pos R |
    logit_rows R | block_table S*MB.
    """

    def __init__(self, rows: int, seqs: int, max_blocks: int, device):
        self.rows, self.seqs, self.max_blocks = rows, seqs, max_blocks
        R = rows
        self.words = 7 * R + seqs * max_blocks
        cuda = torch.device(device).type == "cuda"
        self.host = torch.zeros(self.words, dtype=torch.int32)
        if cuda:
            self.host = self.host.pin_memory()
        self.dev = torch.zeros(self.words, dtype=torch.int32, device=device) if cuda else self.host
        self.np = self.host.numpy()
        self.np_slot = self.np[:2 * R].view(np.int64)
        o = 2 * R
        self.np_ids, self.np_pos, self.np_seq, self.np_rpos, self.np_lrows = (
            self.np[o + i * R:o + (i + 1) * R] for i in range(5))
        self.np_bt = self.np[o + 5 * R:].reshape(seqs, max_blocks)
        d = self.dev
        self.d_slot = d[:2 * R].view(torch.int64)
        self.d_ids, self.d_pos, self.d_seq, self.d_rpos, self.d_lrows = (d[o + i * R:o + (i + 1) * R] for i in range(5))
        self.d_bt = d[o + 5 * R:].view(seqs, max_blocks)
        self.cuda = cuda

    def fill(self, b: ExecutionBatch, pad_rows: int = 0):
        T = b.rows
        R = max(T, pad_rows)
        if R > self.rows or len(b.sequences) > self.seqs:
            raise ValueError("batch exceeds staging capacity")
        self.np_ids[:T] = b.token_ids
        self.np_pos[:T] = b.positions
        self.np_rpos[:T] = b.positions
        self.np_slot[:T] = b.write_slots
        if R > T:
            self.np_ids[T:R] = 0
            self.np_pos[T:R] = 0
            self.np_rpos[T:R] = -1
            self.np_slot[T:R] = -1
            self.np_seq[T:R] = 0
        for i, s in enumerate(b.sequences):
            self.np_seq[s.query_start:s.query_start + s.query_len] = i
            if s.block_len > self.max_blocks:
                raise ValueError("sequence has more pages than the block table holds")
            self.np_bt[i, :s.block_len] = b.block_ids[s.block_start:s.block_start + s.block_len]
        lrows = b.logit_rows()
        self.np_lrows[:len(lrows)] = lrows
        return T, R, lrows

    def upload(self) -> int:
        if self.cuda:
            self.dev.copy_(self.host, non_blocking=True)
        return self.words * 4

    def device_batch(self, R: int, n_logit: int) -> DeviceBatch:
        return DeviceBatch(self.d_ids[:R], self.d_pos[:R], self.d_slot[:R], self.d_seq[:R], self.d_rpos[:R],
                           self.d_bt, self.d_lrows, R, n_logit)


@dataclass
class RunnerStats:
    transactions: int = 0
    graph_steps: int = 0
    eager_steps: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    kernel_launches: int = 0
    graph_captures: int = 0
    cow_copies: int = 0
    forward_ns: int = 0


class DeepSeekRunner(ModelRunner):
    def __init__(self, weights: ModelWeights, n_pages: int, page_size: int, max_rows: int = 2048,
                 max_seqs: int = 64, max_seq_len: int = 4096, device=None, tp=None, use_graphs: bool = True,
                 emulate_bf16: bool = False, attn_splits: int = 8):
        self.w, self.cfg = weights, weights.cfg
        self.device = torch.device(device if device is not None else weights.embed.device)
        self.is_cuda = self.device.type == "cuda"
        self.vocab_size, self.eos_token_id = self.cfg.vocab_size, self.cfg.eos_token_id
        self.page_size, self.max_rows, self.max_seqs, self.max_seq_len = page_size, max_rows, max_seqs, max_seq_len
        self.max_blocks = (max_seq_len + page_size - 1) // page_size
        self.pool = KvPool(self.cfg, n_pages, page_size, self.device,
                           dtype=torch.bfloat16 if self.is_cuda else weights.embed.dtype)
        self.tp = tp
        self.use_graphs = use_graphs and self.is_cuda
        self.stats = RunnerStats()
        self.staging = BatchStaging(max_rows, max_seqs, self.max_blocks, self.device)
        if self.is_cuda:
            self.fwd = CudaForward(weights, self.pool, max_rows=max_rows, max_logit_rows=max(max_seqs, 1),
                                   decode_rows=max_seqs, max_seq_len=max_seq_len, attn_splits=attn_splits, tp=tp)
            L = self.fwd.ws.max_logit_rows
            self.out_host = torch.zeros(2 * L, dtype=torch.int32).pin_memory()
        else:
            self.fwd = ReferenceForward(weights, self.pool, emulate_bf16=emulate_bf16)
        self.graphs: Dict[int, tuple] = {}
        self.txns: Dict[int, ExecutionBatch] = {}
        self._hidden_rows: Dict[int, torch.Tensor] = {}     # state slot -> last hidden state (MTP input)

    # ------------------------------------------------------------------ contract
    def capabilities(self) -> ExecutionCapabilities:
        return ExecutionCapabilities(max_batch_rows=self.max_rows, max_sequences=self.max_seqs, max_topk=40,
                                     supports_provisional=True, supports_full_logits=False)

    def kv_schema(self) -> KvLayoutSchema:
        return KvLayoutSchema((KvPlaneDescriptor("latent_kv", self.cfg.kv_row_dim, self.pool.n_layers),),
                              self.page_size, self.max_seq_len)

    def prepare_batch(self, txn_id: int, batch: ExecutionBatch) -> None:
        batch.validate(self.capabilities())
        pairs = [(c.source, c.replacement) for s in batch.sequences for c in s.cow]
        if pairs:
            self.pool.copy_pages(pairs)
            self.stats.cow_copies += len(pairs)
        self.txns[txn_id] = batch
        self.stats.transactions += 1

    def _graph_for(self, rows: int):
        g = self.graphs.get(rows)
        if g is None:
            st = BatchStaging(rows, rows, self.max_blocks, self.device)
            st.np_rpos[:] = -1
            st.np_slot[:] = -1
            st.np_lrows[:] = np.arange(rows)
            st.upload()
            graph = DecodeGraph(self.fwd, rows, rows, self.max_blocks, batch=st.device_batch(rows, rows))
            graph.capture()
            self.stats.graph_captures += 1
            g = (st, graph)
            self.graphs[rows] = g
        return g

    def execute(self, txn_id: int):
        b = self.txns[txn_id]
        t0 = time.perf_counter_ns()
        if not self.is_cuda:
            out = self._execute_reference(b)
        else:
            out = self._execute_cuda(b)
        self.stats.forward_ns += time.perf_counter_ns() - t0
        return Complete(out)

    def resume(self, txn_id: int):
        return self.execute(txn_id)

    def end_transaction(self, txn_id: int, intent: EndIntent) -> EndStatus:
        self.txns.pop(txn_id, None)
        return EndStatus.COMPLETE

    def release_pages(self, pages: Sequence[int]) -> None:
        pass        # every launch that could touch them has been synchronised by execute()

    def snapshot_pages(self, pages):
        return self.pool.snapshot_pages(pages)

    def restore_pages(self, pages, snapshot) -> None:
        self.pool.restore_pages(pages, snapshot)

    def release_slot(self, state_slot: int) -> None:
        self._hidden_rows.pop(state_slot, None)

    # ------------------------------------------------------------------ execution paths
    def _is_pure_decode(self, b: ExecutionBatch) -> bool:
        return (b.intent == Intent.COMMITTED and len(b.sequences) == b.rows
                and all(lr.kind == LogitsKind.TOPK and lr.k == 1 for lr in b.logits))

    def _execute_cuda(self, b: ExecutionBatch) -> ExecutionOutput:
        fwd = self.fwd
        if self.use_graphs and self._is_pure_decode(b) and b.rows <= self.max_seqs:
            st, graph = self._graph_for(b.rows)
            T, R, lrows = st.fill(b)
            self.stats.h2d_bytes += st.upload()
            graph.replay()
            self.stats.graph_steps += 1
            self.stats.kernel_launches += graph.launches
            L = len(lrows)
            want_topk = False
        else:
            st = self.staging
            T, R, lrows = st.fill(b)
            self.stats.h2d_bytes += st.upload()
            L = len(lrows)
            if L > fwd.ws.max_logit_rows:
                raise ValueError("more logit rows than the runner was sized for")
            want_topk = any(b.logits[r].k > 1 for r in lrows)
            fwd.forward(st.device_batch(T, L), want_logits=want_topk)
            self.stats.eager_steps += 1
            self.stats.kernel_launches += fwd.launches
        rows: List[RowOutput] = []
        if L:
            Lcap = fwd.ws.max_logit_rows
            self.out_host.copy_(fwd.ws.out_buf, non_blocking=True)
            topk = None
            if want_topk:
                kmax = max(b.logits[r].k for r in lrows)
                ids, vals = fwd.K.topk_logits(fwd.ws.logits[:L], kmax)
                topk = (ids.cpu(), vals.cpu())
            torch.cuda.current_stream().synchronize()
            self.stats.d2h_bytes += 2 * Lcap * 4
            ids_h = self.out_host[:L].tolist()
            vals_h = self.out_host[Lcap:Lcap + L].view(torch.float32).tolist()
            for i, r in enumerate(lrows):
                k = b.logits[r].k
                if topk is not None and k > 1:
                    ti, tv = topk[0][i, :k].tolist(), topk[1][i, :k].tolist()
                    keep = [(a, v) for a, v in zip(ti, tv) if a >= 0 and v == v and abs(v) != float("inf")]
                    rows.append(RowOutput(r, [a for a, _ in keep], [v for _, v in keep]))
                elif ids_h[i] < 0 or vals_h[i] != vals_h[i] or abs(vals_h[i]) == float("inf"):
                    rows.append(RowOutput(r, [], []))
                else:
                    rows.append(RowOutput(r, [ids_h[i]], [vals_h[i]]))
        else:
            torch.cuda.current_stream().synchronize()
        from ..ops import _lib
        return ExecutionOutput(rows)

    def _execute_reference(self, b: ExecutionBatch) -> ExecutionOutput:
        st = self.staging
        T, R, lrows = st.fill(b)
        L = len(lrows)
        db = st.device_batch(T, L)
        rows: List[RowOutput] = []
        allreduce = self.tp.allreduce_reference if self.tp is not None else None
        gather = self.tp.gather_vocab_reference if self.tp is not None else None
        with torch.no_grad():
            h = self.fwd.hidden_states(db, allreduce)
            if L == 0:
                return ExecutionOutput(rows)
            logits = self.fwd.logits_from_hidden(h, db)
            if gather is not None:
                logits = gather(logits)
        from ..ops import reference as ref
        for i, r in enumerate(lrows):
            k = max(b.logits[r].k, 1)
            ids, vals = ref.topk_logits(logits[i:i + 1], k)
            keep = [(int(a), float(v)) for a, v in zip(ids[0], vals[0]) if torch.isfinite(v)]
            rows.append(RowOutput(r, [a for a, _ in keep], [v for _, v in keep]))
        self.stats.eager_steps += 1
        return ExecutionOutput(rows)

    def observability(self) -> Dict[str, object]:
        d = dict(vars(self.stats))
        d["graphs"] = sorted(self.graphs)
        d["weights_bytes"] = self.w.nbytes()
        d["kv_pool_bytes"] = self.pool.data.numel() * self.pool.data.element_size()
        return d
