"""Speculative decoding with exact packed verification.

One cycle for a pure-decode cohort:
  1. ask the runner's proposal head for draft tokens after each sequence's staged token and cut the
     draft where the head's confidence (sigmoid of its logit) falls below the threshold,
  2. reserve KV rows for [staged token, drafts...] and run ONE provisional batch over all of them
     (prefill-phase rows, top-1 logits on every row),
  3. accept drafts while the target's top-1 equals the draft (`verify_causal_slice`); the target's
     top-1 after the last accepted row is the correction (or bonus) token,
  4. keep only the accepted prefix in the backend (`retain_provisional_prefixes`), commit
     `accepted + 1` KV rows, retire the rejected suffix pages, publish the tokens and stage the
     correction/bonus token as the next decode input.
The emitted token stream is exactly what greedy decoding without speculation produces.

Counterpart of crates/ferrule-runtime/src/speculation.rs:223-262 (cohort), :293-440 (provisional
batch), :614-770 (result), :1038-1061 (verify_causal_slice), metrics :129-215, and the driver's
confidence cut / publish (engine/driver.rs:56-81, :5039-5352).
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .execution import ExecutionBatch, Intent, LogitsRequest, Phase, SequenceSlice
from .resources import ResourceKind
from .session import FinishReason, SequenceState


def verify_causal_slice(drafts: Sequence[int], target_top1: Sequence[Optional[int]]) -> Tuple[int, Optional[int]]:
    """drafts d_0..d_{n-1}; target_top1[i] is the target's greedy token after row i, where row 0 is
    the anchor and row i+1 carries d_i.  Returns (accepted, target_next): accept while
    target_top1[i] == d_i; target_next is the top-1 at the first mismatch row, or the bonus row."""
    accepted = 0
    for i, d in enumerate(drafts):
        t = target_top1[i]
        if t is None or t != d:
            break
        accepted += 1
    return accepted, target_top1[accepted]


@dataclass
class SpeculativeMetrics:
    cycles: int = 0
    sequences: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0
    zero_draft_cycles: int = 0
    rollbacks: int = 0
    pruned_by_confidence: int = 0
    accepted_prefix_hist: Dict[int, int] = field(default_factory=dict)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    def to_dict(self) -> dict:
        d = dict(vars(self))
        d["acceptance_rate"] = self.acceptance_rate
        return d


@dataclass
class SpecMember:
    seq: SequenceState
    res_id: int
    drafts: List[int]
    query_start: int = 0


@dataclass
class SpecCohort:
    members: List[SpecMember]


class SpeculativeDecoder:
    def __init__(self, engine):
        self.engine = engine
        self.metrics = SpeculativeMetrics()

    # ------------------------------------------------------------------ cycle start
    def try_execute(self, decodes: List[SequenceState]) -> bool:
        eng = self.engine
        cfg = eng.cfg
        if not decodes:
            return False
        ctx = cfg.scheduler.ctx_size
        views = [None] * len(decodes)
        props = eng.runner.propose([s.slot for s in decodes], [s.staged_token for s in decodes],
                                   [s.position for s in decodes], views, cfg.max_draft)
        plans: List[Tuple[SequenceState, List[int]]] = []
        any_draft = False
        for seq, p in zip(decodes, props):
            drafts: List[int] = []
            room = min(cfg.max_draft, seq.request.max_new_tokens - seq.generated - 1, ctx - seq.position - 1)
            for tok, conf in zip(p.tokens, p.confidence):
                if len(drafts) >= max(room, 0):
                    break
                if 1.0 / (1.0 + math.exp(-conf)) < cfg.confidence_threshold:
                    self.metrics.pruned_by_confidence += 1
                    break
                drafts.append(tok)
            any_draft |= bool(drafts)
            plans.append((seq, drafts))
        if not any_draft:
            self.metrics.zero_draft_cycles += 1
            return False
        from .engine import Transaction, TxnSeq
        eng._drive_retirements()
        members: List[SpecMember] = []
        tx_members: List[TxnSeq] = []
        claimed = {ResourceKind.KV_PAGES: 0}
        stalled: List[SequenceState] = []
        for seq, drafts in plans:
            rows = 1 + len(drafts)
            need = eng.kv.required_physical_pages(seq.kv_seq, rows)
            if need > eng.kv.free_pages:
                rows, drafts = 1, []
                need = eng.kv.required_physical_pages(seq.kv_seq, 1)
                if need > eng.kv.free_pages:
                    stalled.append(seq)
                    continue
            r = eng.kv.reserve(seq.kv_seq, rows)
            claimed[ResourceKind.KV_PAGES] += need
            members.append(SpecMember(seq, r.res_id, drafts))
            tx_members.append(TxnSeq(seq, r.res_id, rows, True))
        for seq in stalled:
            eng.stats.kv_stalls += 1
            eng.scheduler.requeue_unchanged(seq)
        if not members:
            if stalled:
                eng._break_page_deadlock(stalled)        # nobody could reserve: same way out as for plain steps
            return True
        grant = eng.broker.try_claim(claimed, required=True)
        txn = Transaction(eng._next_txn, tx_members, grant=grant, t_start_ns=time.perf_counter_ns())
        txn.speculative = SpecCohort(members)
        eng._next_txn += 1
        eng.stats.transactions += 1
        self.metrics.cycles += 1
        try:
            txn.batch = self._lower(txn)
            eng.runner.prepare_batch(txn.txn_id, txn.batch)
            if grant is not None:
                eng.broker.mark_submitted(grant)
            t0 = time.perf_counter_ns()
            progress = eng.runner.execute(txn.txn_id)
            eng.stats.runner_ns += time.perf_counter_ns() - t0
        except Exception as exc:  # noqa: BLE001
            self.metrics.rollbacks += 1
            eng._abort(txn, exc)
            return True
        eng._on_progress(txn, progress)
        return True

    def _lower(self, txn) -> ExecutionBatch:
        eng = self.engine
        ps = eng.cfg.page_size
        token_ids: List[int] = []
        positions: List[int] = []
        write_slots: List[int] = []
        seqs: List[SequenceSlice] = []
        block_ids: List[int] = []
        for m, tm in zip(txn.speculative.members, txn.members):
            seq = m.seq
            r = eng.kv.reservation(m.res_id)
            eng.kv.bind_reservation_execution(m.res_id, txn.txn_id)
            blocks, slots = eng.kv.reservation_bindings(m.res_id)
            m.query_start = tm.query_start = len(token_ids)
            rows = 1 + len(m.drafts)
            token_ids.append(seq.staged_token)
            token_ids.extend(m.drafts)
            positions.extend(range(seq.position, seq.position + rows))
            write_slots.extend(slots)
            seqs.append(SequenceSlice(seq.slot, Phase.PREFILL, m.query_start, rows, seq.position, seq.position + rows,
                                      len(block_ids), len(blocks), (r.cow,) if r.cow is not None else ()))
            block_ids.extend(blocks)
        logits = [LogitsRequest.topk(1)] * len(token_ids)
        return ExecutionBatch(token_ids, positions, write_slots, logits, seqs, block_ids,
                              Intent.PROVISIONAL_VERIFICATION, ps)

    # ------------------------------------------------------------------ verification result
    def on_verified(self, txn) -> None:
        """Called by the engine when the provisional batch completed and its output validated."""
        eng = self.engine
        out = txn.output.by_row()
        eos = eng.runner.eos_token_id
        commits: List[Tuple[int, int]] = []
        keep: Dict[int, int] = {}
        decisions = []
        for m in txn.speculative.members:
            seq = m.seq
            n = len(m.drafts)
            top1 = [out[m.query_start + i].top1 if (m.query_start + i) in out else None for i in range(n + 1)]
            accepted, target_next = verify_causal_slice(m.drafts, top1)
            # tokens that become committed: the anchor and the accepted drafts, cut where greedy decoding
            # would have stopped (token budget, EOS chosen by the target)
            remaining = seq.request.max_new_tokens - seq.generated
            commit_tokens = [seq.staged_token] + m.drafts[:accepted]
            finish: Optional[FinishReason] = None
            for i in range(accepted):
                if m.drafts[i] == eos and not seq.request.ignore_eos:
                    commit_tokens = commit_tokens[:i + 1]
                    finish = FinishReason.EOS
                    break
            if len(commit_tokens) >= remaining:
                commit_tokens = commit_tokens[:max(remaining, 0)]
                finish = FinishReason.MAX_TOKENS
            rows = len(commit_tokens)
            commits.append((m.res_id, rows))
            keep[seq.slot] = rows
            decisions.append((m, commit_tokens, finish, target_next if finish is None else None, accepted))
        try:
            eng.runner.retain_provisional_prefixes(txn.txn_id, keep)
            txn.commit_id = eng.kv.prepare_commit(commits)
        except Exception as exc:  # noqa: BLE001
            self.metrics.rollbacks += 1
            eng._abort(txn, exc)
            return
        txn.spec_decisions = decisions
        from .engine import TxnState
        txn.state = TxnState.PUBLISHING
        eng._end(txn)

    def publish(self, txn) -> None:
        """Backend completed the publish: commit KV rows, publish tokens, stage the next token."""
        eng = self.engine
        ret = eng.kv.publish_commit(txn.commit_id)
        txn.commit_id = None
        eng._retire(ret)
        if txn.grant is not None:
            eng.broker.complete(txn.grant)
        from .engine import TxnState
        txn.state = TxnState.DONE
        now = time.perf_counter_ns()
        eng.stats.decode_steps += 1
        for m, commit_tokens, finish, target_next, accepted in txn.spec_decisions:
            seq = m.seq
            self.metrics.sequences += 1
            self.metrics.drafted += len(m.drafts)
            self.metrics.accepted += accepted
            self.metrics.emitted += len(commit_tokens)
            h = self.metrics.accepted_prefix_hist
            h[accepted] = h.get(accepted, 0) + 1
            eng.stats.decode_rows += len(commit_tokens)
            cancelled = seq.finish == FinishReason.CANCELLED
            stopped = False
            # publish token by token so stop strings cut at the right place
            seq.staged_token = None
            for tok in commit_tokens:
                seq.tokens.append(tok)
                seq.position += 1
                seq.generated += 1
                eng._emit_token(seq, tok, now)
                if not cancelled and seq.request.stop and seq.text and any(
                        s and seq.text.endswith(s) for s in seq.request.stop):
                    stopped = True
                    break
            from .session import SeqStatus
            seq.status = SeqStatus.DECODE
            eng.scheduler.decode_ready.append(seq)
            if cancelled:
                eng._finish(seq, FinishReason.CANCELLED)
            elif stopped:
                # the cycle committed KV rows beyond the stop string: roll the sequence's KV back to the
                # published position, so that a retained session continues from rows that match its tokens
                kvs = eng.kv.sequence(seq.kv_seq)
                if kvs.committed_tokens > seq.position:
                    eng._retire(eng.kv.truncate_sequence(seq.kv_seq, seq.position))
                eng._finish(seq, FinishReason.STOP_STRING)
            elif finish is not None:
                eng._finish(seq, finish)
            elif eng._post_commit_finish(seq):
                pass
            else:
                eng._apply_output(seq, target_next)
