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

import logging
import os
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..runtime.execution import (ExecutionBatch, ExecutionCapabilities, ExecutionOutput, Intent, KvLayoutSchema,
                                 KvPlaneDescriptor, LogitsKind, RowOutput)
from ..runtime.runner import (Complete, EndIntent, EndStatus, ModelRunner, Proposal, Waiting,
                              predict_next_decode_batch, same_decode_batch)
from .deepseek import CudaForward, DecodeGraph, DeviceBatch, KvPool, ReferenceForward
from .weights import ModelWeights

_PREFILL_LOG = logging.getLogger("ferrule_prefill")


class BatchStaging:
    """Pinned host mirror + device buffer of one packed batch; tensors of `DeviceBatch` are views.

    Layout (int32 words): write_slot (int64, 2R) | token_ids R | positions R | row_seq R | row_pos R |
    logit_rows R | block_table S*MB | prefill attention tiles 4*TC (only with tc_heads).

    tc_heads > 0: sequences that bring at least `tc_min_rows` query rows are cut into the 128-row tiles of the
    tensor-core prefill attention kernel (128 / tc_heads positions x all heads); the other rows - decode rows,
    verification rows, short chunk tails - stay with the row-tile kernel, whose split boundaries make a
    verification row bit-equal to the decode row of the same position.
    """

    def __init__(self, rows: int, seqs: int, max_blocks: int, device, tc_heads: int = 0, tc_min_rows: int = 16):
        self.rows, self.seqs, self.max_blocks = rows, seqs, max_blocks
        R = rows
        self.tc_heads, self.tc_min_rows = tc_heads, tc_min_rows
        self.tile_cap = (R // (128 // tc_heads) + seqs + 1) if tc_heads else 0
        self.tile_off = (7 * R + seqs * max_blocks + 3) // 4 * 4          # 16-byte aligned
        self.words = self.tile_off + 4 * self.tile_cap
        self.n_tiles, self.rest_ranges = 0, None
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
        self.np_bt = self.np[o + 5 * R:o + 5 * R + seqs * max_blocks].reshape(seqs, max_blocks)
        self.np_tiles = self.np[self.tile_off:self.tile_off + 4 * self.tile_cap].reshape(self.tile_cap, 4)
        d = self.dev
        self.d_slot = d[:2 * R].view(torch.int64)
        self.d_ids, self.d_pos, self.d_seq, self.d_rpos, self.d_lrows = (d[o + i * R:o + (i + 1) * R] for i in range(5))
        self.d_bt = d[o + 5 * R:o + 5 * R + seqs * max_blocks].view(seqs, max_blocks)
        self.d_tiles = d[self.tile_off:self.tile_off + 4 * self.tile_cap].view(self.tile_cap, 4)
        self.cuda = cuda
        self._arange = np.arange(R, dtype=np.int32)

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
        seqs = b.sequences
        n = len(seqs)
        L = seqs[0].block_len
        if (n == T and L <= self.max_blocks and len(b.block_ids) == n * L
                and all(s.block_len == L and s.block_start == i * L for i, s in enumerate(seqs))):
            # decode step with one row per sequence and equally long page lists laid out back to back (the
            # common steady state): two array assignments instead of a loop over the sequences
            self.np_seq[:T] = self._arange[:T]
            self.np_bt[:n, :L] = np.asarray(b.block_ids, dtype=np.int32).reshape(n, L)
        else:
            for i, s in enumerate(seqs):
                self.np_seq[s.query_start:s.query_start + s.query_len] = i
                if s.block_len > self.max_blocks:
                    raise ValueError("sequence has more pages than the block table holds")
                self.np_bt[i, :s.block_len] = b.block_ids[s.block_start:s.block_start + s.block_len]
        lrows = b.logit_rows()
        self.np_lrows[:len(lrows)] = lrows
        self.n_tiles, self.rest_ranges = 0, None
        if self.tc_heads and n != T and any(s.query_len >= self.tc_min_rows for s in seqs):
            from ..ops.kernels import prefill_tiles
            tiles, rest = prefill_tiles([(i, s.query_start, s.query_len, int(b.positions[s.query_start]))
                                         for i, s in enumerate(seqs)], self.tc_heads, self.tc_min_rows)
            if len(tiles) <= self.tile_cap:
                self.np_tiles[:len(tiles)] = tiles
                self.n_tiles, self.rest_ranges = len(tiles), rest
        return T, R, lrows

    def upload(self) -> int:
        if self.cuda:
            self.dev.copy_(self.host, non_blocking=True)
        return self.words * 4

    def device_batch(self, R: int, n_logit: int) -> DeviceBatch:
        db = DeviceBatch(self.d_ids[:R], self.d_pos[:R], self.d_slot[:R], self.d_seq[:R], self.d_rpos[:R],
                         self.d_bt, self.d_lrows, R, n_logit)
        if self.n_tiles:
            db.tc_tiles, db.n_tc_tiles, db.rest_ranges = self.d_tiles, self.n_tiles, self.rest_ranges
        return db


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
    mtp_proposals: int = 0
    waits: int = 0
    lookahead_launched: int = 0     # decode steps launched before the host had published their predecessor
    lookahead_hits: int = 0         # ... that the engine then asked for unchanged


class _MtpTrack:
    """Published rows of one sequence that still lack their MTP row: `hidden[j]` / `tokens[j]` belong
    to position `next_pos + j`."""
    __slots__ = ("next_pos", "hidden", "tokens", "blocks")

    def __init__(self, next_pos: int):
        self.next_pos, self.hidden, self.tokens, self.blocks = next_pos, [], [], []


class DeepSeekRunner(ModelRunner):
    def __init__(self, weights: ModelWeights, n_pages: int, page_size: int, max_rows: int = 2048,
                 max_seqs: int = 64, max_seq_len: int = 4096, device=None, tp=None, use_graphs: bool = True,
                 emulate_bf16: bool = False, attn_splits: int = 8, enable_mtp: bool = True, max_draft: int = 1,
                 expert_residency: Optional[float] = None, async_streaming: bool = False,
                 lookahead: bool = True, pp=None, sequence_parallel: bool = False):
        self.w, self.cfg = weights, weights.cfg
        self.device = torch.device(device if device is not None else weights.embed.device)
        self.is_cuda = self.device.type == "cuda"
        self.vocab_size, self.eos_token_id = self.cfg.vocab_size, self.cfg.eos_token_id
        self.page_size, self.max_rows, self.max_seqs, self.max_seq_len = page_size, max_rows, max_seqs, max_seq_len
        self.max_blocks = (max_seq_len + page_size - 1) // page_size
        self.pool = KvPool(self.cfg, n_pages, page_size, self.device,
                           dtype=torch.bfloat16 if self.is_cuda else weights.embed.dtype)
        self.tp = tp
        # pipeline parallelism (parallel.pp.PipelineParallel): `weights` is this stage's share; every step runs
        # through all stages, the last one's greedy tokens are broadcast, so all ranks' engines stay in step
        self.pp = pp
        if pp is not None:
            use_graphs, enable_mtp = False, False
        # streamed routed experts: a fraction of every layer's experts is resident, the rest comes from pinned host
        # memory on demand; the step then synchronises with the host per MoE layer, so it cannot be one graph
        # `async_streaming`: a batch that routes to a non-resident expert returns `Waiting`; the engine's load
        # registry drives `self.provider` and resumes the transaction at the layer it stopped at.  (On the CPU the
        # oracle keeps reading the full weights; the residency protocol runs beside it.)
        self.arena = None
        self.provider = None
        self.telemetry = None                  # route counts per layer and local expert (streamed experts only)
        self.async_streaming = bool(async_streaming and expert_residency is not None)
        if expert_residency is not None and (self.is_cuda or self.async_streaming):
            from .expert_arena import ExpertArena
            self.arena = ExpertArena(weights, expert_residency, replace_weights=self.is_cuda)
            use_graphs = False
            if self.async_streaming:
                from .expert_async import ArenaProvider
                self.provider = ArenaProvider(self.arena, self.cfg.name)
        # profiling switches are read once, here: a stage table or a debug tap needs host callbacks between the
        # kernels of a step, so such a runner steps eagerly
        from ..utils.stage_profile import DebugTap, StageProfiler, prefill_progress_enabled
        self.profiler = StageProfiler.from_env(self.device)
        self.debug_tap = DebugTap.from_env()
        self.prefill_progress = prefill_progress_enabled()
        if self.profiler is not None or self.debug_tap is not None:
            use_graphs = False
        self.use_graphs = use_graphs and self.is_cuda
        self.stats = RunnerStats()
        tc_heads = 0
        if self.is_cuda and pp is None and os.environ.get("FERRULE_PREFILL_TC", "1") != "0":
            from ..ops.kernels import prefill_tc_supported
            if prefill_tc_supported(weights.heads_local, self.cfg.kv_lora_rank, self.cfg.qk_rope_dim, page_size):
                tc_heads = weights.heads_local
        self.staging = BatchStaging(max_rows, max_seqs, self.max_blocks, self.device, tc_heads=tc_heads)
        if self.is_cuda:
            # a verification batch asks for logits on the anchor and on every draft row of each sequence
            logit_rows = max(max_seqs, 1) * (1 + (max_draft if weights.mtp and enable_mtp else 0))
            self.fwd = CudaForward(weights, self.pool, max_rows=max_rows, max_logit_rows=logit_rows,
                                   decode_rows=max_seqs, max_seq_len=max_seq_len, attn_splits=attn_splits, tp=tp)
            self.fwd.arena = self.arena
            if self.arena is not None:
                from ..utils.telemetry import ExpertTelemetry
                self.fwd.telemetry = ExpertTelemetry(self.cfg.n_layers + len(weights.mtp),
                                                     max(weights.e_hi - weights.e_lo, 1))
                self.telemetry = self.fwd.telemetry
            L = self.fwd.ws.max_logit_rows
            self.out_host = torch.zeros(2 * L, dtype=torch.int32).pin_memory()
        else:
            self.fwd = ReferenceForward(weights, self.pool, emulate_bf16=emulate_bf16)
        self.graphs: Dict[int, tuple] = {}
        # captured decode graphs and their staging, one per row count (exact-key reuse, build on first use)
        from ..runtime.arena import PersistentArenaPool
        self.graph_pool: PersistentArenaPool = PersistentArenaPool()
        self.txns: Dict[int, ExecutionBatch] = {}
        # decode look-ahead: while the host publishes step n, step n + 1 already runs on the device, fed by the
        # greedy tokens that are still there.  The step is launched for the batch the engine is predicted to
        # lower next; if the engine then asks for exactly that batch, only its result is read, otherwise the
        # launched step is ignored (it wrote KV rows past every committed length, which nothing reads) and
        # the requested batch runs as usual behind it on the same stream.
        self.lookahead = bool(lookahead and self.use_graphs and not (enable_mtp and weights.mtp))
        self._ahead = None                     # (predicted batch, rows, done event)
        self._predict_next_decode = None
        # multi-token prediction: per state slot, the hidden rows whose MTP row is not written yet
        self.mtp_enabled = bool(enable_mtp and weights.mtp)
        self._mtp: Dict[int, _MtpTrack] = {}
        self._txn_hidden: Dict[int, torch.Tensor] = {}
        self._txn_keep: Dict[int, Dict[int, int]] = {}
        self._mtp_staging: Optional[BatchStaging] = None
        self._mtp_hidden: Optional[torch.Tensor] = None
        # asynchronous expert streaming: leases and the stop point of every parked transaction
        self._txn_leases: Dict[int, Dict[int, Dict[int, tuple]]] = {}
        self._txn_waves: Dict[int, Dict[int, dict]] = {}       # txn -> layer -> finished waves of a parked layer
        self._wave_state: Dict[int, dict] = {}
        self._txn_resume: Dict[int, tuple] = {}
        if self.async_streaming:
            if self.is_cuda:
                self.fwd.async_stream = True
            else:
                self.fwd.expert_gate = self._expert_gate
        self.fwd.prof, self.fwd.tap = self.profiler, self.debug_tap
        # sequence parallelism over the tensor-parallel ranks: the residual stream stays sharded by rows between the
        # reduce-scatter behind a sublayer and the all-gather in front of the next (not with parked transactions:
        # a layer that stops half-way hands its input rows back whole)
        self.sequence_parallel = bool(sequence_parallel and tp is not None and tp.world > 1 and not self.async_streaming
                                      and pp is None)
        if self.sequence_parallel:
            if self.is_cuda:
                self.fwd.sequence_parallel = True       # batches above the fused all-reduce's row limit
            else:
                self.fwd.sp = tp
        if self.arena is not None and self.telemetry is None:
            from ..utils.telemetry import ExpertTelemetry
            self.telemetry = ExpertTelemetry(self.cfg.n_layers + len(weights.mtp), max(weights.e_hi - weights.e_lo, 1))
        # hot-set predictor (frequency, recency, step-to-step transitions per layer): ranks the prefetch candidates
        # of parked transactions.  Built by the first call of `prefetch_candidates` - a runner nobody asks for
        # candidates does not pay for the observations (tens of microseconds per streamed layer pass)
        self.predictor = None

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
            def build():
                st = BatchStaging(rows, rows, self.max_blocks, self.device)
                st.np_rpos[:] = -1
                st.np_slot[:] = -1
                st.np_lrows[:] = np.arange(rows)
                st.upload()
                graph = DecodeGraph(self.fwd, rows, rows, self.max_blocks, batch=st.device_batch(rows, rows))
                graph.capture()
                self.stats.graph_captures += 1
                return (st, graph)
            # stays checked out while the runner lives: a decode step of this row count is always in reach
            g = self.graph_pool.checkout((rows, self.max_blocks), build).arena
            self.graphs[rows] = g
        return g

    def make_registry(self, **kw):
        """The load registry that drives this runner's expert provider (pass it to the engine)."""
        from ..runtime.registry import LoadRegistry
        if self.provider is None:
            raise RuntimeError("the runner was not built with async_streaming")
        reg = LoadRegistry(self.provider, **kw)
        self.provider.attach(reg)
        return reg

    def prefetch_candidates(self, layer: int, n: int):
        """Payloads a transaction parked at `layer` will probably want next: for the streamed layers after it,
        nearest first, the non-resident experts the hot-set predictor ranks highest (at most as many per layer as
        the layer has frames) - at most `n` materialization keys.  The engine requests them without a waiter
        while the transaction waits."""
        if not self.async_streaming or n <= 0:
            return []
        if self.predictor is None:
            from ..runtime.expert_prediction import ExpertPredictor
            self.predictor = ExpertPredictor(max(self.w.e_hi - self.w.e_lo, 1))
            if self.is_cuda:
                self.fwd.predictor = self.predictor
            return []                       # nothing observed yet
        out = []
        for l in sorted(k for k in self.arena.layers if k > layer):
            la = self.arena.layers[l]
            resident = set(la.coord.resident())
            for e in self.predictor.predict(l, min(n - len(out), la.frames), exclude=resident):
                out.append(self.provider.key(l, e))
            if len(out) >= n:
                break
        return out

    def _expert_gate(self, layer: int, experts) -> None:
        """Residency protocol of the host path (the oracle multiplies with the full weights): the batch's experts
        are taken in waves of at most `frames`; a wave with a missing expert parks the transaction, finished waves
        are remembered per transaction and give their frames back."""
        from .expert_async import NeedExperts
        if layer not in self.arena.layers:
            return                      # a layer whose experts are all resident (the proposal stage)
        if not self._wave_state.get(layer, {}).get("done"):
            self.telemetry.record(layer, experts)           # once per layer pass, not per resumed wave
            if self.predictor is not None:
                self.predictor.observe(layer, experts)
        frames = self.arena.frames(layer)
        held = self._lease_sink.setdefault(layer, {})
        if len(experts) <= frames:
            held.update(self.arena.lease_resident(layer, [e for e in experts if e not in held]))
            missing = self.arena.missing(layer, experts)
            if missing:
                raise NeedExperts(layer, missing)
            return
        done = self._wave_state.setdefault(layer, {"done": set(), "rows": None})["done"]
        pending = [e for e in experts if e not in done]
        while pending:
            wave = pending[:frames]
            held.update(self.arena.lease_resident(layer, [e for e in wave if e not in held]))
            missing = self.arena.missing(layer, wave)
            if missing:
                raise NeedExperts(layer, missing)
            done.update(wave)
            self.arena.release_leases(layer, [held.pop(e) for e in wave if e in held])
            pending = pending[len(wave):]
        done.clear()

    def execute(self, txn_id: int):
        b = self.txns[txn_id]
        t0 = time.perf_counter_ns()
        start_layer, h0 = self._txn_resume.pop(txn_id, (0, None))
        if self.debug_tap is not None:
            self.debug_tap.next_step()
        if self.prefill_progress:
            for s in b.sequences:
                if s.query_len > 1:
                    _PREFILL_LOG.info("prefill slot=%d rows=%d done=%d", s.state_slot, s.query_len, s.sequence_len)
        if self.async_streaming:
            self._lease_sink = self._txn_leases.setdefault(txn_id, {})
            self._wave_state = self._txn_waves.setdefault(txn_id, {})
            if self.is_cuda:
                self.fwd.lease_sink = self._lease_sink
                self.fwd.wave_state = self._wave_state
        try:
            if not self.is_cuda:
                out = self._execute_reference(b, start_layer, h0)
            else:
                out = self._execute_cuda(b, start_layer, h0)
        except Exception as exc:  # noqa: BLE001
            if not (self.async_streaming and hasattr(exc, "missing")):
                raise
            # parked: the resident experts stay leased, the missing ones become the continuation's dependencies
            self._txn_resume[txn_id] = (exc.layer, exc.hidden)
            self.stats.forward_ns += time.perf_counter_ns() - t0
            self.stats.waits += 1
            return Waiting([self.provider.key(exc.layer, e) for e in exc.missing], exc.layer)
        self.stats.forward_ns += time.perf_counter_ns() - t0
        if self.mtp_enabled:
            self._txn_hidden[txn_id] = self._last_hidden[:b.rows].clone()
        return Complete(out)

    def resume(self, txn_id: int):
        return self.execute(txn_id)

    def retain_provisional_prefixes(self, txn_id: int, rows_by_slot: Dict[int, int]) -> None:
        # rejected rows stay in the pool as dead rows past the committed length; only the MTP
        # bookkeeping needs to know how many rows of each sequence survive
        self._txn_keep[txn_id] = dict(rows_by_slot)

    def end_transaction(self, txn_id: int, intent: EndIntent) -> EndStatus:
        b = self.txns.pop(txn_id, None)
        self._txn_resume.pop(txn_id, None)
        for layer, held in self._txn_leases.pop(txn_id, {}).items():
            self.arena.release_leases(layer, list(held.values()))
        self._txn_waves.pop(txn_id, None)
        h = self._txn_hidden.pop(txn_id, None)
        keep = self._txn_keep.pop(txn_id, None)
        if b is not None and h is not None and intent == EndIntent.PUBLISH:
            self._mtp_track(b, h, keep)
        return EndStatus.COMPLETE

    def release_pages(self, pages: Sequence[int]) -> None:
        pass        # every launch that could touch them has been synchronised by execute()

    def snapshot_pages(self, pages):
        return self.pool.snapshot_pages(pages)

    def restore_pages(self, pages, snapshot) -> None:
        self.pool.restore_pages(pages, snapshot)

    def release_slot(self, state_slot: int) -> None:
        self._mtp.pop(state_slot, None)

    # ------------------------------------------------------------------ multi-token prediction
    def _mtp_track(self, b: ExecutionBatch, h: torch.Tensor, keep: Optional[Dict[int, int]]) -> None:
        """Queue the published rows: MTP row i pairs hidden state i with token i + 1, so a row can
        only be written once its successor token is known (at the next `propose`)."""
        for s in b.sequences:
            n = s.query_len if keep is None else min(s.query_len, keep.get(s.state_slot, 0))
            if n <= 0:
                continue
            q0 = s.query_start
            first = b.positions[q0]
            tr = self._mtp.get(s.state_slot)
            if tr is None or tr.next_pos + len(tr.tokens) != first:
                # no history for this slot (or a gap, e.g. after a fork): start from here; earlier
                # MTP rows keep whatever the shared pages hold, which only affects draft quality
                tr = self._mtp[s.state_slot] = _MtpTrack(first)
            tr.hidden.append(h[q0:q0 + n])
            tr.tokens.extend(b.token_ids[q0:q0 + n])
            tr.blocks = list(b.block_ids[s.block_start:s.block_start + s.block_len])

    def proposals_enabled(self) -> bool:
        return self.mtp_enabled

    def propose(self, slots, anchors, positions, views, max_draft):
        """One draft token per sequence from the first MTP stage.  Writes the MTP layer's KV rows for
        every published position that has none yet, then reads the stage's greedy token at the last one.
        Mirrors the reference's hidden-tap driven proposal (crates/ferrule-model/src/models/deepseek_v4/runner.rs:3906 and proposal_attachment.rs:57-181)."""
        out = [Proposal([], []) for _ in slots]
        if not self.mtp_enabled or max_draft < 1:
            return out
        if self.async_streaming and any(l >= self.cfg.n_layers for l in self.arena.layers):
            # the arena also streams the proposal stage (`mtp_resident=False`): drafting runs outside a transaction
            # and cannot park, so its experts are uploaded inline
            saved = (getattr(self.fwd, "async_stream", False), getattr(self.fwd, "expert_gate", None))
            if self.is_cuda:
                self.fwd.async_stream = False
            else:
                self.fwd.expert_gate = None
            try:
                self.async_streaming = False
                return self.propose(slots, anchors, positions, views, max_draft)
            finally:
                self.async_streaming = True
                if self.is_cuda:
                    self.fwd.async_stream = saved[0]
                else:
                    self.fwd.expert_gate = saved[1]
        todo = []
        for i, (slot, pos) in enumerate(zip(slots, positions)):
            tr = self._mtp.get(slot)
            if tr is not None and tr.tokens and tr.next_pos + len(tr.tokens) == pos:
                todo.append((i, slot, tr))
        ps = self.page_size
        while todo:
            group, rows = [], 0
            while todo and len(group) < self.max_seqs and rows + len(todo[0][2].tokens) <= self.max_rows:
                rows += len(todo[0][2].tokens)
                group.append(todo.pop(0))
            if not group:
                todo.pop(0)       # a single backlog larger than the row budget: skip drafting for it
                continue
            if self._mtp_staging is None:
                self._mtp_staging = BatchStaging(self.max_rows, self.max_seqs, self.max_blocks, self.device)
            st = self._mtp_staging
            r = 0
            hs = []
            for j, (i, slot, tr) in enumerate(group):
                k = len(tr.tokens)
                pos0 = tr.next_pos
                st.np_ids[r:r + k] = tr.tokens[1:] + [anchors[i]]
                pp = np.arange(pos0, pos0 + k)
                st.np_pos[r:r + k] = pp
                st.np_rpos[r:r + k] = pp
                st.np_seq[r:r + k] = j
                blocks = np.asarray(tr.blocks, dtype=np.int64)
                st.np_slot[r:r + k] = blocks[pp // ps] * ps + pp % ps
                st.np_bt[j, :len(tr.blocks)] = tr.blocks
                st.np_lrows[j] = r + k - 1
                hs.extend(tr.hidden)
                r += k
            self.stats.h2d_bytes += st.upload()
            db = st.device_batch(r, len(group))
            if self.is_cuda and len(hs) > 1:
                # rows of several published steps, packed by the row-copy kernel (no library launch on the path)
                from ..ops import movers as M
                if self._mtp_hidden is None:
                    self._mtp_hidden = torch.zeros(self.max_rows, self.cfg.hidden, dtype=hs[0].dtype, device=self.device)
                r0 = 0
                for hpart in hs:
                    M.copy_rows(self._mtp_hidden, r0, hpart.contiguous())
                    r0 += hpart.shape[0]
                h_prev = self._mtp_hidden[:r0]
            else:
                h_prev = torch.cat(hs, 0) if len(hs) > 1 else hs[0]
            if self.is_cuda:
                ids, vals, _ = self.fwd.mtp_forward(0, h_prev, db)
                ids_h, vals_h = ids.tolist(), vals.tolist()
            else:
                allreduce = self.tp.allreduce_reference if self.tp is not None else None
                with torch.no_grad():
                    logits, _ = self.fwd.mtp_forward(0, h_prev.float(), db, allreduce)
                    if self.tp is not None:
                        logits = self.tp.gather_vocab_reference(logits)
                vals_t, ids_t = logits.max(-1)
                ids_h, vals_h = ids_t.tolist(), vals_t.tolist()
            for j, (i, slot, tr) in enumerate(group):
                # every queued row now has its MTP row; the anchor's own row follows once it is published
                tr.next_pos += len(tr.tokens)
                tr.tokens, tr.hidden = [], []
                if ids_h[j] >= 0 and vals_h[j] == vals_h[j]:
                    out[i] = Proposal([int(ids_h[j])], [float(vals_h[j])])
            self.stats.mtp_proposals += len(group)
        return out

    # ------------------------------------------------------------------ execution paths
    def _is_pure_decode(self, b: ExecutionBatch) -> bool:
        return (b.intent == Intent.COMMITTED and len(b.sequences) == b.rows
                and all(lr.kind == LogitsKind.TOPK and lr.k == 1 for lr in b.logits))

    def _execute_cuda(self, b: ExecutionBatch, start_layer: int = 0, h0=None) -> ExecutionOutput:
        fwd = self.fwd
        ahead, self._ahead = self._ahead, None
        graph_step = self.use_graphs and self._is_pure_decode(b) and b.rows <= self.max_seqs
        if graph_step and ahead is not None and same_decode_batch(ahead[0], b):
            # this very step was launched while the host was still publishing its predecessor
            st, graph = self._graph_for(b.rows)
            lrows = b.logit_rows()
            L = len(lrows)
            ahead[2].synchronize()
            self.stats.lookahead_hits += 1
            self._last_hidden = graph.hidden
            return self._read_greedy(b, lrows, L, None, b, launched=True)
        if ahead is not None:
            ahead[2].synchronize()      # mispredicted step: its input staging and result buffer are reused below
        if graph_step:
            st, graph = self._graph_for(b.rows)
            T, R, lrows = st.fill(b)
            self.stats.h2d_bytes += st.upload()
            graph.replay()
            self._last_hidden = graph.hidden
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
            if self.pp is not None:
                if want_topk:
                    raise ValueError("pipeline-parallel runs return the greedy token only")
                from ..ops import _lib as _l
                l0 = _l.LAUNCHES[0]
                ids_t, vals_t = self.pp.step(fwd, st.device_batch(T, L), self.cfg.hidden, torch.bfloat16, True)
                if L:
                    fwd.ws.next_id[:L].copy_(ids_t)
                    fwd.ws.next_val[:L].copy_(vals_t)
                self._last_hidden = None
                self.stats.kernel_launches += _l.LAUNCHES[0] - l0
            else:
                fwd.forward(st.device_batch(T, L), want_logits=want_topk, start_layer=start_layer, h0=h0)
                self._last_hidden = fwd.last_hidden
                self.stats.kernel_launches += fwd.launches
            self.stats.eager_steps += 1
        topk = None
        if L:
            self.out_host.copy_(fwd.ws.out_buf, non_blocking=True)
            if want_topk:
                kmax = max(b.logits[r].k for r in lrows)
                ids, vals = fwd.K.topk_logits(fwd.ws.logits[:L], kmax)
                topk = (ids.cpu(), vals.cpu())
        torch.cuda.current_stream().synchronize()
        return self._read_greedy(b, lrows, L, topk, b if graph_step else None)

    def _read_greedy(self, b: ExecutionBatch, lrows, L: int, topk, decode_batch, launched: bool = False
                     ) -> ExecutionOutput:
        """Parse the greedy result that the step left in pinned host memory (its device->host copy has been
        waited for).  `decode_batch`: the step was a graph decode step, so its successor may be launched now."""
        fwd = self.fwd
        rows: List[RowOutput] = []
        if L:
            Lcap = fwd.ws.max_logit_rows
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
            if decode_batch is not None and self.lookahead and L == b.rows:
                self._launch_ahead(decode_batch, ids_h)
        return ExecutionOutput(rows)

    def _launch_ahead(self, b: ExecutionBatch, ids_h: List[int]) -> None:
        """Launch the decode step that follows `b` if the engine's next batch can be told now."""
        predict = self._predict_next_decode
        if predict is None:
            return
        nxt = predict({s.state_slot: ids_h[i] for i, s in enumerate(b.sequences)})
        if not nxt:
            return
        pred = predict_next_decode_batch(b, ids_h, nxt)
        if pred is None:
            return
        fwd = self.fwd
        st, graph = self._graph_for(pred.rows)
        st.fill(pred)
        self.stats.h2d_bytes += st.upload()
        # the ids just uploaded equal the ones on the device; taking them from there keeps the step independent
        # of the host copy and is what lets it start before the host has looked at them
        fwd.K.decode_advance(fwd.ws.next_id[:pred.rows], graph.batch, self.cfg.vocab_size, self.page_size, False)
        graph.replay()
        self.out_host.copy_(fwd.ws.out_buf, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._ahead = (pred, pred.rows, ev)
        self.stats.lookahead_launched += 1
        self.stats.graph_steps += 1
        self.stats.kernel_launches += graph.launches + 1

    def _execute_reference(self, b: ExecutionBatch, start_layer: int = 0, h0=None) -> ExecutionOutput:
        st = self.staging
        T, R, lrows = st.fill(b)
        L = len(lrows)
        db = st.device_batch(T, L)
        rows: List[RowOutput] = []
        allreduce = self.tp.allreduce_reference if self.tp is not None else None
        gather = self.tp.gather_vocab_reference if self.tp is not None else None
        if self.pp is not None:
            with torch.no_grad():
                ids_t, vals_t = self.pp.step(self.fwd, db, self.cfg.hidden, self.w.embed.dtype, False,
                                             allreduce=allreduce, gather_vocab=gather)
            self._last_hidden = None
            for i, r in enumerate(lrows):
                if int(ids_t[i]) >= 0 and torch.isfinite(vals_t[i]):
                    rows.append(RowOutput(r, [int(ids_t[i])], [float(vals_t[i])]))
                else:
                    rows.append(RowOutput(r, [], []))
            self.stats.eager_steps += 1
            return ExecutionOutput(rows)
        with torch.no_grad():
            h = self.fwd.hidden_states(db, allreduce, start_layer, h0)
            self._last_hidden = h
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
        if self.arena is not None:
            d["expert_arena"] = dict(vars(self.arena.stats))
            d["expert_telemetry"] = self.telemetry.snapshot()
        if self.predictor is not None:
            d["expert_predictor"] = dict(vars(self.predictor.stats), precision=round(self.predictor.stats.precision, 4))
        if self.profiler is not None:
            d["stage_table"] = self.profiler.by_stage()
            d["stage_table_layers"] = self.profiler.table()
        if self.debug_tap is not None:
            d["debug_tap_files"] = len(self.debug_tap.written)
        return d
