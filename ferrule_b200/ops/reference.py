"""Plain PyTorch reference math (fp32 unless told otherwise).

This is both the CPU execution path of the framework and the oracle every CUDA
kernel is tested against.  The functions mirror the reference's CPU layer math:
RMSNorm / RoPE (crates/ferrule-model/src/models/common), routing
(crates/ferrule-model/src/moe/routing.rs:89-193), clamped SwiGLU experts
(crates/ferrule-model/src/moe/executor.rs:26-160) and sink-denominator attention over an
explicit row selection (crates/ferrule-model/src/attention_backend.rs:47-160).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even to bf16 and back (the storage boundary of the runtime)."""
    return x.to(torch.bfloat16).to(x.dtype)


def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = xf * inv
    if weight is not None:
        y = y * weight.float()
    return y


# ---------------------------------------------------------------------------
# rotary embedding (interleaved pairs), with YaRN frequency scaling
# ---------------------------------------------------------------------------
def yarn_inv_freq(dim: int, theta: float, factor: float = 1.0, original_max_pos: int = 4096,
                  beta_fast: float = 32.0, beta_slow: float = 1.0) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    if factor <= 1.0:
        return inv.float()

    def correction_dim(num_rot: float) -> float:
        return dim * math.log(original_max_pos / (num_rot * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    smooth = 1.0 - ramp
    inv = inv / factor * (1 - smooth) + inv * smooth
    return inv.float()


def yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    return 1.0 if factor <= 1.0 else 0.1 * mscale * math.log(factor) + 1.0


def rope_tables(max_pos: int, dim: int, theta: float, factor: float = 1.0,
                original_max_pos: int = 4096, beta_fast: float = 32.0,
                beta_slow: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [max_pos, dim/2] in fp32."""
    inv = yarn_inv_freq(dim, theta, factor, original_max_pos, beta_fast, beta_slow).double()
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float(), ang.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """x[..., dim] with interleaved pairs; cos/sin broadcastable to x[..., dim/2]."""
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    if inverse:
        sin = -sin
    ra = a * cos - b * sin
    rb = a * sin + b * cos
    return torch.stack((ra, rb), dim=-1).flatten(-2)


# ---------------------------------------------------------------------------
# routing
# ---------------------------------------------------------------------------
SCORE_SOFTMAX, SCORE_SIGMOID, SCORE_SQRT_SOFTPLUS = 0, 1, 2


def stable_topk(values: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k with ties broken toward the lower index (deterministic on every device)."""
    order = torch.sort(values, dim=-1, descending=True, stable=True)
    return order.values[..., :k], order.indices[..., :k]


def route(logits: torch.Tensor, topk: int, score_fn: int = SCORE_SOFTMAX,
          bias: Optional[torch.Tensor] = None, n_groups: int = 1, topk_groups: int = 1,
          normalize: bool = False, route_scale: float = 1.0,
          hash_table: Optional[torch.Tensor] = None,
          token_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (expert ids [T,k] int32, weights [T,k] fp32)."""
    lf = logits.float()
    if score_fn == SCORE_SOFTMAX:
        score = torch.softmax(lf, dim=-1)
    elif score_fn == SCORE_SIGMOID:
        score = torch.sigmoid(lf)
    else:
        score = torch.sqrt(torch.nn.functional.softplus(lf))
    if hash_table is not None:
        idx = hash_table[token_ids.long()][:, :topk].long()
        w = torch.gather(score, 1, idx)
    else:
        sel = score if bias is None else score + bias.float()
        if n_groups > 1 and topk_groups < n_groups:
            T, E = sel.shape
            grp = sel.view(T, n_groups, E // n_groups)
            gscore = stable_topk(grp, 2)[0].sum(-1)
            _, gidx = stable_topk(gscore, topk_groups)
            mask = torch.zeros(T, n_groups, dtype=torch.bool, device=sel.device)
            mask.scatter_(1, gidx, True)
            sel = grp.masked_fill(~mask[:, :, None], float("-inf")).reshape(T, E)
        _, idx = stable_topk(sel, topk)
        w = torch.gather(score, 1, idx)
    if normalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx.to(torch.int32), (w * route_scale).float()


def swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    g, u = gate.float(), up.float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return torch.nn.functional.silu(g) * u


# ---------------------------------------------------------------------------
# absorbed MLA attention over a paged latent-KV pool
# ---------------------------------------------------------------------------
def mla_paged_attention(q: torch.Tensor, kv_pool: torch.Tensor, block_table: torch.Tensor,
                        row_seq: torch.Tensor, row_pos: torch.Tensor, page_size: int,
                        kv_lora: int, scale: float,
                        sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [rows, heads, kv_lora+rope]; kv_pool [pool_rows, kv_lora+rope] -> [rows, heads, kv_lora] fp32.

    Row r attends to kv positions 0..row_pos[r] of sequence row_seq[r]; with `sink`, a per-head
    logit joins the softmax denominator only.
    """
    rows, heads, _ = q.shape
    out = torch.zeros(rows, heads, kv_lora, dtype=torch.float32, device=q.device)
    qf = q.float()
    poolf = kv_pool.float()
    for r in range(rows):
        n = int(row_pos[r]) + 1
        if n <= 0:
            continue
        s = int(row_seq[r])
        tok = torch.arange(n, device=q.device)
        slots = block_table[s, tok // page_size].long() * page_size + tok % page_size
        kv = poolf[slots]                                   # [n, D]
        logits = qf[r] @ kv.T * scale                       # [heads, n]
        if sink is not None:
            m = torch.maximum(logits.max(-1).values, sink.float())
            p = torch.exp(logits - m[:, None])
            den = p.sum(-1) + torch.exp(sink.float() - m)
            p = p / den[:, None]
        else:
            p = torch.softmax(logits, dim=-1)
        out[r] = p @ kv[:, :kv_lora]
    return out


def greedy_argmax(logits: torch.Tensor) -> torch.Tensor:
    """Top-1 with ties toward the lower token id; -1 where no finite candidate exists."""
    lf = logits.float()
    lf = torch.where(torch.isnan(lf), torch.full_like(lf, float("-inf")), lf)
    mx = lf.max(-1, keepdim=True).values
    V = lf.shape[-1]
    ids = torch.arange(V, device=lf.device).expand_as(lf)
    cand = torch.where(lf == mx, ids, torch.full_like(ids, V))
    best = cand.min(-1).values
    none = torch.isinf(mx.squeeze(-1)) & (mx.squeeze(-1) < 0)
    return torch.where(none, torch.full_like(best, -1), best).to(torch.int32)


def topk_logits(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sorted logit-descending, token-ascending on ties."""
    v, i = stable_topk(logits.float(), k)
    return i.to(torch.int32), v
