"""Engine runner for the DeepSeek-V4 family: hyper-connections, compressed + indexed sparse attention and hash /
learned routing behind the same transaction contract as the MLA runner.

The V4 attention state of a sequence is not a pool of uniform KV pages: per layer it is a raw sliding window, a
plane of compressed rows (one per `ratio` tokens), the compressor's projected inputs and, on indexed layers, the
indexer's own compressed plane.  `V4Cuda` keeps those as position-indexed tables per state slot, so this runner
binds state by slot (`KvBindingMode` stays paged for the engine's page accounting: pages are the admission
budget, the tables are what the kernels read).  Every table row is addressed by (slot, position): re-executing a
position after an abort or a rejected draft simply overwrites it, which is what makes transactions abortable
without a snapshot.

Prefill on the kernels is batched: all rows of a transaction - prompt chunks of several sequences, verification
rows, decode rows - go through the layers as one batch (`V4Cuda.step_rows`: every GEMM sees all rows, each row's
selection list is cut at its own position).  The oracle path runs token by token.  Swapping a sequence out needs no copy (a
suspended sequence keeps its slot and with it its tables; the pages it returns are admission budget), so
`auto_preempt` works; sharing a prefix between sequences (copy-on-write pages, exact forks, the prompt-prefix
cache) is refused, because two slots cannot share table rows.

Counterpart of the V4 runtime of the reference (crates/ferrule-model/src/deepseek_v4/: model assembly, state
pools for window / compressed / indexer planes, one-token decode schedule).
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Sequence

import torch

from ..runtime.execution import (ExecutionBatch, ExecutionCapabilities, ExecutionOutput, KvLayoutSchema,
                                 KvPlaneDescriptor, LogitsKind, RowOutput)
from ..runtime.runner import Complete, EndIntent, EndStatus, ModelRunner, Proposal
from .v4_model import V4Cuda, V4Reference, V4SeqCache, V4Weights


def _truncate(c: V4SeqCache, cfg, pos: int) -> None:
    """Oracle cache back to `pos` committed tokens (rows past it came from an aborted or rejected step)."""
    for i in range(cfg.n_layers):
        del c.kv[i][pos:]
        r = cfg.ratio(i)
        if r:
            del c.comp[i][pos // r:]
            del c.icomp[i][pos // r:]
        del c.cstate[i].kv[pos:]
        del c.cstate[i].gate[pos:]
        del c.istate[i].kv[pos:]
        del c.istate[i].gate[pos:]
    for rows in c.pctx:
        del rows[pos:]
    c.position = pos


from ..runtime.arena import SequenceStateCore


class V4Runner(ModelRunner):
    # the attention state lives in slot-bound tables, not in the pages the engine accounts: two sequences cannot
    # share a prefix by sharing pages (the engine's prompt-prefix cache and exact forks stay off for this runner)
    supports_prefix_sharing = False
    # no captured step: the output head runs for the rows that ask for logits only
    skip_unread_logits = True

    def __init__(self, weights: V4Weights, n_pages: int, page_size: int = 64, max_seqs: int = 8,
                 max_seq_len: int = 1024, max_rows: int = 2048, eos_token_id: int = -1,
                 batched_prefill: Optional[bool] = None):
        self.w, self.cfg = weights, weights.cfg
        self.device = weights.embed.device
        self.is_cuda = self.device.type == "cuda"
        self.vocab_size, self.eos_token_id = self.cfg.vocab_size, eos_token_id
        self.page_size, self.n_pages = page_size, n_pages
        self.max_seqs, self.max_seq_len, self.max_rows = max_seqs, max_seq_len, max_rows
        # prompt chunks (and verification rows) go through the layers as one batch of rows; off = one row per
        # sequence per pass, the decode schedule
        self.batched_prefill = (os.environ.get("FERRULE_V4_BATCHED_PREFILL", "1") != "0") if batched_prefill is None \
            else batched_prefill
        if self.is_cuda:
            self.fwd = V4Cuda(weights, max_seqs, max_seq_len, max_rows=max_rows if self.batched_prefill else 0)
        else:
            self.fwd = V4Reference(weights)
            self.caches: Dict[int, V4SeqCache] = {}
        from ..utils.stage_profile import StageProfiler
        self.profiler = self.fwd.prof = StageProfiler.from_env(self.device)      # read once, here
        self.txns: Dict[int, ExecutionBatch] = {}
        self.steps = 0
        self.forward_ns = 0
        self.proposal_blocks = 0
        self.proposal_ns = 0
        # committed cursor of every slot-bound sequence state: a step binds to (generation, position) when it
        # starts and commits only if both still hold; a step that fails half-way poisons the slot until release
        self.seq_state: Dict[int, SequenceStateCore] = {}
        self._bindings: Dict[int, Dict[int, tuple]] = {}

    # ------------------------------------------------------------------ contract
    def capabilities(self) -> ExecutionCapabilities:
        return ExecutionCapabilities(max_batch_rows=self.max_rows, max_sequences=self.max_seqs, max_topk=40,
                                     supports_provisional=True, supports_full_logits=False)

    def kv_schema(self) -> KvLayoutSchema:
        cfg = self.cfg
        planes = [KvPlaneDescriptor("window_kv", cfg.head_dim, cfg.n_layers)]
        n_comp = sum(1 for i in range(cfg.n_layers) if cfg.ratio(i))
        n_idx = sum(1 for i in range(cfg.n_layers) if cfg.has_indexer(i))
        if n_comp:
            planes.append(KvPlaneDescriptor("compressed_kv", cfg.head_dim, n_comp))
        if n_idx:
            planes.append(KvPlaneDescriptor("indexer_plane", cfg.index_head_dim, n_idx))
        return KvLayoutSchema(tuple(planes), self.page_size, self.max_seq_len)

    def prepare_batch(self, txn_id: int, batch: ExecutionBatch) -> None:
        batch.validate(self.capabilities())
        for s in batch.sequences:
            if s.cow:
                raise RuntimeError("V4 state is bound by slot: shared (copy-on-write) pages are not supported")
            if s.state_slot >= self.max_seqs or s.sequence_len > self.max_seq_len:
                raise RuntimeError(f"sequence in slot {s.state_slot} exceeds the runner's tables")
        self.txns[txn_id] = batch

    def execute(self, txn_id: int):
        b = self.txns[txn_id]
        t0 = time.perf_counter_ns()
        binds = self._bindings[txn_id] = {}
        for s in b.sequences:
            core = self.seq_state.setdefault(s.state_slot, SequenceStateCore())
            if core.position != s.context_len and not core.poisoned:
                if s.context_len > core.position:
                    raise RuntimeError(f"slot {s.state_slot}: state holds {core.position} tokens, batch expects "
                                       f"{s.context_len}")
                core.rewind(s.context_len)            # rejected / aborted rows will be overwritten
            binds[s.state_slot] = (core.begin_step(), s.query_len)
        try:
            with torch.no_grad():
                out = self._execute_cuda(b) if self.is_cuda else self._execute_reference(b)
        except Exception:
            for slot, (binding, _) in binds.items():
                self.seq_state[slot].poison_step(binding)
            raise
        self.forward_ns += time.perf_counter_ns() - t0
        return Complete(out)

    def resume(self, txn_id: int):
        return self.execute(txn_id)

    def retain_provisional_prefixes(self, txn_id: int, rows_by_slot: Dict[int, int]) -> None:
        binds = self._bindings.get(txn_id, {})
        for slot, rows in rows_by_slot.items():
            if slot in binds:
                binds[slot] = (binds[slot][0], min(rows, binds[slot][1]))

    def end_transaction(self, txn_id: int, intent: EndIntent) -> EndStatus:
        self.txns.pop(txn_id, None)        # aborted rows are overwritten when their positions run again
        for slot, (binding, rows) in self._bindings.pop(txn_id, {}).items():
            core = self.seq_state.get(slot)
            if core is not None and intent == EndIntent.PUBLISH and not core.poisoned:
                core.commit_step(binding, rows)
        return EndStatus.COMPLETE

    def release_pages(self, pages: Sequence[int]) -> None:
        pass

    # ------------------------------------------------------------------ drafting
    def proposals_enabled(self) -> bool:
        return self.w.proposal is not None

    def propose(self, slots, anchors, positions, views, max_draft) -> List[Proposal]:
        """One proposal block per sequence: the checkpoint's block drafter reads the context rows that the
        target's committed positions left in the proposal stages' planes (rows past `position` - from a
        rejected draft or an aborted step - are not read) and returns up to `gamma` drafts after the anchor."""
        if self.w.proposal is None:
            return [Proposal([], []) for _ in slots]
        out: List[Proposal] = []
        t0 = time.perf_counter_ns()
        for slot, anchor, pos in zip(slots, anchors, positions):
            core = self.seq_state.get(slot)
            if core is None or core.poisoned or core.position < pos:
                out.append(Proposal([], []))            # no committed context for this slot: draft nothing
                continue
            if self.is_cuda:
                toks, conf = self.fwd.propose(slot, pos, anchor)
            else:
                toks, conf = self.fwd.propose(self.caches[slot], pos, anchor)
            out.append(Proposal(toks[:max_draft], conf[:max_draft]))
            self.proposal_blocks += 1
        self.proposal_ns += time.perf_counter_ns() - t0
        return out

    def snapshot_pages(self, pages):
        """Swap-out of a V4 sequence: its state sits in the tables of its slot, and a suspended sequence keeps
        its slot, so nothing has to be copied - the pages the engine takes back are its admission budget, not
        memory the tables use.  The token returned is what `restore_pages` expects back."""
        return ("v4-slot-state", len(pages))

    def restore_pages(self, pages, snapshot) -> None:
        if not (isinstance(snapshot, tuple) and snapshot and snapshot[0] == "v4-slot-state"):
            raise RuntimeError("not a snapshot of this runner")

    def release_slot(self, state_slot: int) -> None:
        self.seq_state.pop(state_slot, None)
        if self.is_cuda:
            self.fwd.positions[state_slot] = 0
        else:
            self.caches.pop(state_slot, None)

    def observability(self) -> Dict[str, object]:
        d = {"model": "deepseek-v4", "decode_steps": self.steps, "forward_ms": self.forward_ns / 1e6,
             "proposal_blocks": self.proposal_blocks, "proposal_ms": self.proposal_ns / 1e6}
        if self.profiler is not None:
            d["stage_table"] = self.profiler.by_stage()
            d["stage_table_layers"] = self.profiler.table()
        return d

    # ------------------------------------------------------------------ execution
    @staticmethod
    def _rows_out(b: ExecutionBatch, logits_by_row: Dict[int, torch.Tensor]) -> ExecutionOutput:
        from ..ops import reference as ref
        rows: List[RowOutput] = []
        for r in sorted(logits_by_row):
            k = max(b.logits[r].k, 1)
            ids, vals = ref.topk_logits(logits_by_row[r][None].float().cpu(), k)
            keep = [(int(a), float(v)) for a, v in zip(ids[0], vals[0]) if torch.isfinite(v)]
            rows.append(RowOutput(r, [a for a, _ in keep], [v for _, v in keep]))
        return ExecutionOutput(rows)

    def _execute_cuda(self, b: ExecutionBatch) -> ExecutionOutput:
        """All rows of the batch in one pass through the layers (`V4Cuda.step_rows`): prompt chunks, verification
        rows and decode rows alike; pieces of at most `max_rows` rows when the batch is larger.  With
        `batched_prefill` off, wave j feeds the j-th row of every sequence that still has one."""
        fwd = self.fwd
        for s in b.sequences:
            fwd.positions[s.state_slot] = s.context_len
        want: Dict[int, torch.Tensor] = {}
        if self.batched_prefill:
            rows = [(s.state_slot, s.query_start + j, s.context_len + j) for s in b.sequences for j in range(s.query_len)]
            for _, r, p in rows:
                assert b.positions[r] == p, "rows of a sequence must be consecutive positions"
            for i0 in range(0, len(rows), fwd.max_rows):
                piece = rows[i0:i0 + fwd.max_rows]
                wanted = [i for i, (_, r, _) in enumerate(piece) if b.logits[r].kind != LogitsKind.NONE]
                _, logits = fwd.step_rows([sl for sl, _, _ in piece], [b.token_ids[r] for _, r, _ in piece],
                                          [p for _, _, p in piece], want_rows=wanted)
                self.steps += 1
                for k, i in enumerate(wanted):
                    want[piece[i][1]] = logits[k]
            return self._rows_out(b, want)
        waves = max(s.query_len for s in b.sequences)
        for j in range(waves):
            live = [s for s in b.sequences if s.query_len > j]
            slots = [s.state_slot for s in live]
            rows = [s.query_start + j for s in live]
            for s, r in zip(live, rows):
                assert b.positions[r] == s.context_len + j, "rows of a sequence must be consecutive positions"
            _, logits = fwd.step(slots, [b.token_ids[r] for r in rows])
            self.steps += 1
            for i, r in enumerate(rows):
                if b.logits[r].kind != LogitsKind.NONE:
                    want[r] = logits[i]
        return self._rows_out(b, want)

    def _execute_reference(self, b: ExecutionBatch) -> ExecutionOutput:
        want: Dict[int, torch.Tensor] = {}
        for s in b.sequences:
            c = self.caches.get(s.state_slot)
            if c is None or s.context_len == 0:
                c = self.caches[s.state_slot] = V4SeqCache(self.cfg)
            if c.position != s.context_len:
                assert c.position > s.context_len, "sequence state is behind the committed length"
                _truncate(c, self.cfg, s.context_len)
            for j in range(s.query_len):
                r = s.query_start + j
                logits = self.fwd.step(c, b.token_ids[r])
                self.steps += 1
                if b.logits[r].kind != LogitsKind.NONE:
                    want[r] = logits
        return self._rows_out(b, want)
