"""DeepSeek-V4-only operators: hyper-connections, KV compressor pooling, learned indexer,
explicit-selection sink attention.  PyTorch reference math (fp32 with the bf16 write-backs of the
checkpoint's computation contract) plus dispatch to the CUDA kernels of `csrc/v4_ops.cu`.

* Hyper-connections keep `hc` copies of the residual stream.  `hc_pre` reduces them to one hidden
  vector: mixes = (W_fn . state) * rms(state); pre = sigmoid(mix*s0 + b) + eps; post = 2*sigmoid(.);
  comb = Sinkhorn(softmax rows + eps); hidden = sum_j pre_j * state_j.  `hc_post` writes the copies
  back: out_j = post_j * hidden + sum_i comb[i, j] * residual_i.  `hc_head` is the final reduction.
* The compressor emits one pooled KV row per `ratio` tokens: a per-dimension softmax over the
  window (the group, plus the previous group when `overlap`), scores = gate + position embedding,
  entries before the start of the sequence count as score -inf / value 0; result rounded to bf16.
* The indexer scores compressed rows for a query: per head bf16(q_h . row) -> bf16(relu * w_h) ->
  fp32 sum over heads -> bf16, then a stable top-k (ties -> lower row, non-finite excluded, unused
  slots = -1).
* Selection = sliding window rows U chosen compressed rows; attention runs over that explicit row
  list with a per-head sink logit in the softmax denominator.

Counterpart of crates/ferrule-model/src/hyper_connection.rs:175-420, attention_backend.rs:47-185,
models/deepseek_v4/attention.rs:1194-1364, :2831-3395 and the device kernels hc_kernel /
compressor_kernel / indexer_kernel (portable/entrypoints.cu:912-1266, :1614-1840).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import reference as ref


@dataclass(frozen=True)
class HcConfig:
    hc: int = 4
    hidden: int = 4096
    eps: float = 1e-6
    norm_eps: float = 1e-6
    sinkhorn_iters: int = 20

    @property
    def mix(self) -> int:
        return 2 * self.hc + self.hc * self.hc


def hc_split_sinkhorn(mixes: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, cfg: HcConfig):
    """mixes [T, 2hc + hc*hc] -> (pre [T,hc], post [T,hc], comb [T,hc,hc])."""
    hc, eps = cfg.hc, cfg.eps
    m = mixes.float()
    pre = torch.sigmoid(m[:, :hc] * scale[0] + base[:hc]) + eps
    post = 2.0 * torch.sigmoid(m[:, hc:2 * hc] * scale[1] + base[hc:2 * hc])
    c = (m[:, 2 * hc:] * scale[2] + base[2 * hc:]).view(-1, hc, hc)
    c = torch.softmax(c, dim=-1) + eps
    c = c / (c.sum(1, keepdim=True) + eps)                     # columns
    for _ in range(1, cfg.sinkhorn_iters):
        c = c / (c.sum(2, keepdim=True) + eps)                 # rows
        c = c / (c.sum(1, keepdim=True) + eps)                 # columns
    return pre, post, c


def hc_pre(state: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, cfg: HcConfig):
    """state [T, hc, hidden], fn [mix, hc*hidden] -> (hidden [T, hidden] fp32, (pre, post, comb))."""
    T = state.shape[0]
    x = state.float().reshape(T, -1)
    rms = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
    mixes = (x @ fn.float().T) * rms
    pre, post, comb = hc_split_sinkhorn(mixes, scale.float(), base.float(), cfg)
    hidden = (pre.unsqueeze(-1) * state.float()).sum(1)
    return hidden, (pre, post, comb)


def hc_post(hidden: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """hidden [T, hidden], residual [T, hc, hidden] -> [T, hc, hidden]: out_j = post_j*hidden + sum_i comb[i,j]*res_i."""
    mix = torch.einsum("tij,tid->tjd", comb.float(), residual.float())
    return post.float().unsqueeze(-1) * hidden.float().unsqueeze(1) + mix


def hc_head(state: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, cfg: HcConfig) -> torch.Tensor:
    T = state.shape[0]
    x = state.float().reshape(T, -1)
    rms = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
    pre = torch.sigmoid((x @ fn.float().T) * rms * scale[0] + base[:cfg.hc].float()) + cfg.eps
    return (pre.unsqueeze(-1) * state.float()).sum(1)


def compressor_pool(kv: torch.Tensor, gate: torch.Tensor, ape: torch.Tensor, ratio: int, overlap: bool,
                    dim: Optional[int] = None) -> torch.Tensor:
    """kv, gate [tokens, out_dim] projected rows of one sequence (position 0 first); ape [ratio, out_dim].
    out_dim = dim without overlap, 2 * dim with it: rows of the previous group are read from columns [0, dim),
    rows of the current group from [dim, 2 dim), each with the embedding of its position inside its group.
    Returns pooled [tokens // ratio, dim], rounded to bf16."""
    tokens, out_dim = kv.shape
    dim = (out_dim // 2 if overlap else out_dim) if dim is None else dim
    groups = tokens // ratio
    out = torch.zeros(groups, dim, dtype=torch.float32, device=kv.device)
    kvf, gf, af = kv.float(), gate.float(), ape.float()
    cur = dim if overlap else 0
    for g in range(groups):
        lo = g * ratio
        rows = [kvf[lo:lo + ratio, cur:cur + dim]]
        score = [gf[lo:lo + ratio, cur:cur + dim] + af[:, cur:cur + dim]]
        if overlap and g > 0:
            rows.insert(0, kvf[lo - ratio:lo, :dim])
            score.insert(0, gf[lo - ratio:lo, :dim] + af[:, :dim])
        rows, score = torch.cat(rows), torch.cat(score)
        out[g] = (torch.softmax(score, dim=0) * rows).sum(0)
    return ref.bf16_round(out)


def indexer_topk(q: torch.Tensor, rows: torch.Tensor, head_w: torch.Tensor, k: int, n_visible: int):
    """q [heads, d], rows [n, d] (compressed indexer plane), head_w [heads] -> (indices [k] int32 (-1 = unused),
    scores [n] fp32 holding bf16 values).  Only the first `n_visible` rows may be chosen."""
    b = ref.bf16_round
    dots = b(q.float() @ rows.float().T)                                   # [heads, n]
    contrib = b(torch.relu(dots) * b(head_w.float())[:, None])
    score = b(contrib.sum(0))
    cand = score[:n_visible].clone()
    cand = torch.where(torch.isfinite(cand), cand, torch.full_like(cand, float("-inf")))
    take = min(k, n_visible)
    idx = torch.full((k,), -1, dtype=torch.int32, device=q.device)
    if take > 0:
        order = torch.sort(cand, descending=True, stable=True).indices[:take]
        good = torch.isfinite(cand[order])
        idx[:take] = torch.where(good, order.to(torch.int32), torch.full_like(order, -1).to(torch.int32))
    return idx, score


def sliding_window_indices(position: int, window: int) -> torch.Tensor:
    """Rows visible through the window at `position` (inclusive): [window] int32, -1 where none."""
    lo = position - window + 1
    idx = torch.arange(lo, position + 1, dtype=torch.int32)
    return torch.where(idx >= 0, idx, torch.full_like(idx, -1))


def sparse_sink_attention(q: torch.Tensor, table: torch.Tensor, selection: torch.Tensor, kv_lora: int, scale: float,
                          sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [rows, heads, D]; table [n, D]; selection [rows, W] int32 row ids (-1 = masked) -> [rows, heads, kv_lora].
    probabilities are rounded to bf16 before the value product, like the device contract."""
    rows, heads, _ = q.shape
    out = torch.zeros(rows, heads, kv_lora, dtype=torch.float32, device=q.device)
    for r in range(rows):
        sel = selection[r]
        ok = sel >= 0
        if not bool(ok.any()):
            continue
        kv = table.float()[sel[ok].long()]
        logits = q[r].float() @ kv.T * scale
        if sink is not None:
            m = torch.maximum(logits.max(-1).values, sink.float())
            p = torch.exp(logits - m[:, None])
            p = p / (p.sum(-1) + torch.exp(sink.float() - m))[:, None]
        else:
            p = torch.softmax(logits, -1)
        out[r] = p @ kv[:, :kv_lora]
    return out


def markov_head(logits: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, anchor: int):
    """Sequential Markov proposal head over a block of draft rows.  logits [gamma, vocab] fp32 (LM head of the
    block's backbone rows), w1 / w2 [vocab, rank]: draft_j = argmax_t(logits[j, t] + w2[t] . w1[prev]) with
    prev = anchor for j = 0 and draft_{j-1} after; ties go to the lower id.  Returns (drafts, biased logits)."""
    prev = int(anchor)
    ids, vals = [], []
    for j in range(logits.shape[0]):
        biased = logits[j].float() + w2.float() @ w1[prev].float()
        best = torch.max(biased)
        tok = int(torch.nonzero(biased == best)[0])
        ids.append(tok)
        vals.append(float(best))
        prev = tok
    return ids, vals


def hc_mean_taps(states, hc: int) -> torch.Tensor:
    """Proposal target taps: for every tapped layer the mean over the hc copies, concatenated along the feature
    dimension and rounded to bf16.  states: list of [T, hc, hidden]."""
    return torch.cat([ref.bf16_round(s.float().sum(1) / hc) for s in states], dim=-1)


# ------------------------------------------------------------------------------------------ QAT steps
# The checkpoint was trained with these quantisations inside the forward pass; a runtime that leaves them out
# computes a (slightly) different function.  All three quantise and come straight back to bf16 values, on
# whichever device the rows live (crates/ferrule-model/src/models/deepseek_v4/helpers.rs:138-201,
# crates/ferrule-model/src/checkpoint/encoding.rs:199-300).
def qat_kv_rows(rows: torch.Tensor, rope_dim: int, block: int = 64) -> torch.Tensor:
    """KV rows [..., head_dim] after RoPE: the non-rotary part goes through FP8 e4m3 with one power-of-two scale
    per `block` features (per row when the width is not a multiple of it); the rotary tail is left alone."""
    from ..io import encoding as enc
    hd = rows.shape[-1]
    n = hd - rope_dim
    if n <= 0:
        return rows
    out = rows.float().clone()
    out[..., :n] = enc.fp8_qat(out[..., :n], block if n % block == 0 else n)
    return out.to(rows.dtype)


def qat_indexer_rows(rows: torch.Tensor) -> torch.Tensor:
    """Indexer queries / compressed indexer rows [..., d] (d a power of two, multiple of 32): bf16 -> orthonormal
    Hadamard transform -> bf16 -> FP4 e2m1 with one power-of-two scale per 32 features."""
    from ..io import encoding as enc
    x = enc.bf16_round(enc.hadamard(enc.bf16_round(rows.float())))
    return enc.fp4_qat(x, 32).to(rows.dtype)


def qat_linear_input(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Activation rows in front of a linear whose checkpoint weight is quantised: FP8 e4m3, one power-of-two
    scale per 1 x `block` (amax floored at 1e-4)."""
    from ..io import encoding as enc
    n = x.shape[-1]
    return enc.fp8_qat(x.float(), block if n % block == 0 else n).to(x.dtype)


# ------------------------------------------------------------------------------------------ CUDA dispatch
def hc_pre_cuda(state, fn, scale, base, cfg: HcConfig):
    from ..ops import v4 as K4
    return K4.hc_pre(state, fn, scale, base, cfg)


def hc_post_cuda(hidden, residual, post, comb):
    from ..ops import v4 as K4
    return K4.hc_post(hidden, residual, post, comb)
