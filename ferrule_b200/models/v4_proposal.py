"""DeepSeek-V4 proposal attachment: the checkpoint's `mtp.*` stages as a block drafter.

This is not an autoregressive MTP stack.  Two halves:

  context (runs with every target row): the hidden states tapped after the target layers named by the
      checkpoint (mean over the hyper-connection copies, concatenated) are projected and normalised once
      (`main_proj`, `main_norm`); every proposal stage turns that row into one KV row of its own
      (stage `wkv` -> RMSNorm -> RoPE at the row's position) and appends it to its context plane.
  proposal (one pass per drafting cycle): a block of `gamma` rows - the carried anchor token followed by
      `gamma - 1` noise tokens - is embedded into hyper-connection state and flows through the stages, each a
      full V4 layer (hc_pre -> norm -> attention -> hc_post -> hc_pre -> norm -> MoE -> hc_post) whose
      attention lets EVERY block row see the last `window` context rows of its stage plus ALL block rows (not
      causal); block KV is ephemeral.  The last stage's heads reduce the copies (`hc_head`), normalise, take
      LM-head logits and run the low-rank Markov chain: draft_j = argmax(logits_j + w2 . w1[prev]) with
      prev = anchor, then draft_{j-1}; the confidence logit of draft_j is conf . [hidden_j ; w1[prev_j]].

The target then verifies `1 + gamma` rows (the anchor and the drafts) in one provisional batch.

The block is `gamma` rows of one sequence, far below the size where the tensor-core GEMMs of the decode step
pay: linears, norms, RoPE and the hyper-connection mixes are PyTorch tensor operations that run on either
device; on the GPU the block attention is the decode step's selection-mode attention kernel and the Markov chain
is the device kernel.

Counterpart of crates/ferrule-model/src/models/deepseek_v4/proposal_attachment.rs:57-181 (stages, heads,
row protocol), cuda_cache.rs:2002-2125 (taps, main projection, head), :2178-2400 (block attention over
context window + block rows; per-stage context KV) and
crates/ferrule-backend/native/cuda/implementations/cutlass/capabilities/proposal_head.cuh:245-331
(Markov chain + confidence).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from ..ops import reference as ref
from . import v4
from .config import SCORE_SQRT_SOFTPLUS


def _lin(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """bf16(x @ w^T) as fp32: fp32 accumulation of bf16-valued operands, rounded once."""
    if x.is_cuda:
        return torch.nn.functional.linear(x.to(torch.bfloat16), w.to(torch.bfloat16)).float()
    return ref.bf16_round(x.float() @ w.float().T)


def _rope_rows(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, rdim: int,
               inverse: bool = False) -> torch.Tensor:
    """x [rows, ..., dim]: rotate the last `rdim` entries of row r at positions[r]."""
    out = x.clone()
    c, s = cos[positions.long()], sin[positions.long()]
    while c.dim() < x.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    out[..., -rdim:] = ref.apply_rope(x[..., -rdim:], c, s, inverse=inverse)
    return out


class V4Proposal:
    def __init__(self, weights, rope: Tuple[torch.Tensor, torch.Tensor]):
        self.w, self.cfg, self.p = weights, weights.cfg, weights.proposal
        assert self.p is not None, "the weights carry no proposal attachment"
        self.rope = rope
        cfg = self.cfg
        if len(self.p.stages) != cfg.n_proposal_stages or not cfg.proposal_target_layers:
            raise ValueError("proposal attachment does not match the configuration")
        if list(cfg.proposal_target_layers) != sorted(set(cfg.proposal_target_layers)) or \
                cfg.proposal_target_layers[-1] >= cfg.n_layers:
            raise ValueError("proposal target layers must be strictly increasing layer indices of the target")
        if self.p.main_proj.shape != (cfg.hidden, len(cfg.proposal_target_layers) * cfg.hidden):
            raise ValueError(f"main_proj is {tuple(self.p.main_proj.shape)}")
        rank = self.p.markov_w1.shape[1]
        if self.p.markov_w2.shape != self.p.markov_w1.shape or self.p.confidence_proj.shape != (1, cfg.hidden + rank):
            raise ValueError("proposal head shapes do not match")

    # ------------------------------------------------------------------ row protocol
    @property
    def gamma(self) -> int:
        return self.cfg.proposal_block_size

    def draft_input_ids(self, anchor: int) -> List[int]:
        return [int(anchor)] + [self.cfg.proposal_noise_token] * (self.gamma - 1)

    def target_rows_for_drafts(self, drafts: int) -> int:
        if drafts > self.gamma:
            raise ValueError(f"{drafts} drafts above the checkpoint's block of {self.gamma}")
        return drafts + 1

    # ------------------------------------------------------------------ context half
    def tap(self, state: torch.Tensor) -> torch.Tensor:
        """state [T, hc, H] after a tapped target layer -> [T, H] (mean over the copies, bf16 values)."""
        return ref.bf16_round(state.float().sum(1) / self.cfg.hc_mult)

    def _aq(self, x: torch.Tensor) -> torch.Tensor:
        """Input of a linear the checkpoint stores quantised (QAT checkpoints only)."""
        return v4.qat_linear_input(x) if self.cfg.qat else x

    def main_rows(self, taps) -> torch.Tensor:
        """taps: one [T, H] per target layer, in layer order, or the concatenated [T, taps * H] rows (the kernel
        path's tap kernel writes them side by side) -> projected + normalised rows [T, H]."""
        cat = taps if isinstance(taps, torch.Tensor) else torch.cat(list(taps), dim=-1)
        x = _lin(self._aq(cat), self.p.main_proj)
        return ref.bf16_round(ref.rmsnorm(x, self.p.main_norm, self.cfg.norm_eps))

    def context_kv(self, stage: int, main_x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One context KV row per target row for `stage`: [T, head_dim] fp32 holding bf16 values."""
        cfg, lw = self.cfg, self.p.stages[stage]
        kv = ref.bf16_round(ref.rmsnorm(_lin(self._aq(main_x), lw.wkv), lw.kv_norm, cfg.norm_eps))
        kv = ref.bf16_round(_rope_rows(kv, self.rope[0], self.rope[1], positions, cfg.rope_dim))
        return v4.qat_kv_rows(kv, cfg.rope_dim) if cfg.qat else kv

    # ------------------------------------------------------------------ proposal half
    def _attention(self, lw, xn: torch.Tensor, ctx: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg, rnd = self.cfg, ref.bf16_round
        G = xn.shape[0]
        hd, rd, nh = cfg.head_dim, cfg.rope_dim, cfg.n_heads
        xa = self._aq(xn)
        qn = rnd(ref.rmsnorm(_lin(xa, lw.wq_a), lw.q_norm, cfg.norm_eps))
        q = _lin(self._aq(qn), lw.wq_b).view(G, nh, hd)
        q = rnd(ref.rmsnorm(q, None, cfg.norm_eps))
        q = rnd(_rope_rows(q, self.rope[0], self.rope[1], positions, rd))
        kv = rnd(ref.rmsnorm(_lin(xa, lw.wkv), lw.kv_norm, cfg.norm_eps))
        kv = rnd(_rope_rows(kv, self.rope[0], self.rope[1], positions, rd))
        if cfg.qat:
            kv = v4.qat_kv_rows(kv, rd)
        table = torch.cat([ctx.float(), kv], dim=0)             # context window rows, then the whole block
        sel = torch.arange(table.shape[0], dtype=torch.int32, device=xn.device)[None].expand(G, -1)
        if xn.is_cuda:
            # the selection-mode attention kernel of the decode step: every block row selects the whole table
            from ..ops import v4 as K4
            o = K4.sparse_sink_attention(q.to(torch.bfloat16).contiguous(), table.to(torch.bfloat16).contiguous(),
                                         sel.contiguous(), hd, 0, cfg.softmax_scale, sink=lw.sink).float()
        else:
            o = rnd(v4.sparse_sink_attention(q, table, sel, hd, cfg.softmax_scale, sink=lw.sink))
        o = rnd(_rope_rows(o, self.rope[0], self.rope[1], positions, rd, inverse=True))
        og = o.reshape(G, cfg.o_groups, cfg.group_in)
        lat = rnd(torch.einsum("tgk,gnk->tgn", og, lw.wo_a.float())).reshape(G, -1)
        return _lin(self._aq(lat), lw.wo_b)

    def _moe(self, lw, xn: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        cfg, rnd = self.cfg, ref.bf16_round
        logits = xn.float() @ lw.router_w.float().T
        idx, wts = ref.route(logits, cfg.topk, SCORE_SQRT_SOFTPLUS, bias=lw.router_bias, normalize=True,
                             route_scale=cfg.route_scale, hash_table=lw.hash_table, token_ids=tokens)
        I = cfg.moe_inter
        out = torch.zeros_like(xn, dtype=torch.float32)
        idx_h, wts_h = idx.tolist(), wts.tolist()
        for r in range(xn.shape[0]):
            acc = torch.zeros_like(out[r])
            for e, wt in zip(idx_h[r], wts_h[r]):
                y = xn[r].float() @ lw.e_w13[e].float().T
                h = rnd(ref.swiglu(y[:I], y[I:], cfg.swiglu_limit))
                acc = acc + rnd((h @ lw.e_w2[e].float().T) * wt)
            out[r] = acc
        y = self._aq(xn).float() @ lw.w13[0].float().T
        sI = y.shape[1] // 2
        h = rnd(ref.swiglu(y[:, :sI], y[:, sI:], cfg.swiglu_limit))
        return rnd(out + _lin(self._aq(h), lw.w2[0]))

    def block_hidden(self, context: Sequence[torch.Tensor], n_committed: int, token_ids: Sequence[int]) -> torch.Tensor:
        """Run the block rows `token_ids` (positions n_committed ...) through the stages -> [rows, H] after the
        head reduction and final norm.  context[s]: stage s's context rows of positions [0, n_committed) (only
        the last `window` of them are read)."""
        cfg, rnd, w = self.cfg, ref.bf16_round, self.w
        dev = w.embed.device
        G = len(token_ids)
        tok = torch.tensor(list(token_ids), dtype=torch.int64, device=dev)
        pos = torch.arange(n_committed, n_committed + G, device=dev)
        if n_committed + G > cfg.max_position:
            raise ValueError("proposal block runs past the position tables")
        state = w.embed[tok].float()[:, None, :].repeat(1, cfg.hc_mult, 1)
        for s, lw in enumerate(self.p.stages):
            ctx = context[s][max(0, n_committed - cfg.window):n_committed]
            x, (_, post, comb) = v4.hc_pre(state, lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, cfg.hc)
            xn = rnd(ref.rmsnorm(rnd(x), lw.attn_norm, cfg.norm_eps))
            a = self._attention(lw, xn, ctx, pos)
            state = rnd(v4.hc_post(a, state, post, comb))
            x, (_, post, comb) = v4.hc_pre(state, lw.hc_ffn_fn, lw.hc_ffn_scale, lw.hc_ffn_base, cfg.hc)
            xn = rnd(ref.rmsnorm(rnd(x), lw.ffn_norm, cfg.norm_eps))
            f = self._moe(lw, xn, tok)
            state = rnd(v4.hc_post(f, state, post, comb))
        h = rnd(v4.hc_head(state, self.p.hc_head_fn, self.p.hc_head_scale, self.p.hc_head_base, cfg.hc))
        return rnd(ref.rmsnorm(h, self.p.norm, cfg.norm_eps))

    def heads(self, hn: torch.Tensor, anchor: int) -> Tuple[List[int], List[float]]:
        """Markov chain over the block's LM-head logits + confidence logits -> (drafts, confidence)."""
        p = self.p
        if hn.is_cuda:
            # the chain runs on the device (one launch per draft, each reads its predecessor from device memory)
            from ..ops import v4 as K4
            logits = torch.nn.functional.linear(hn.to(torch.bfloat16), self.w.lm_head).float().contiguous()
            ids, _ = K4.markov_head(logits, p.markov_w1, p.markov_w2,
                                    torch.tensor([int(anchor)], dtype=torch.int32, device=hn.device))
            drafts = [int(t) for t in ids.tolist()]
        else:
            logits = hn.float() @ self.w.lm_head.float().T
            drafts, _ = v4.markov_head(logits, p.markov_w1, p.markov_w2, anchor)
        H = self.cfg.hidden
        cw = p.confidence_proj.float()[0]
        conf: List[float] = []
        prev = int(anchor)
        for j, d in enumerate(drafts):
            conf.append(float(hn[j].float() @ cw[:H] + p.markov_w1[prev].float() @ cw[H:]))
            prev = d
        return drafts, conf

    def propose(self, context: Sequence[torch.Tensor], n_committed: int, anchor: int) -> Tuple[List[int], List[float]]:
        """Drafts for the `gamma` positions after the anchor (which will sit at position `n_committed`)."""
        with torch.no_grad():
            hn = self.block_hidden(context, n_committed, self.draft_input_ids(anchor))
            return self.heads(hn, anchor)
