"""PyTorch stand-ins for the kernel wrappers `V4Cuda` calls, so that its host-side logic (row / position
bookkeeping, table addressing, selection lists, batched rows, QAT and proposal hooks) runs in CPU tests.  Each
function has the wrapper's signature and contract; the math is the oracle's (`models/v4.py`, `ops/reference.py`)."""
from types import SimpleNamespace

import torch

from ferrule_b200.models import v4
from ferrule_b200.models.config import SCORE_SQRT_SOFTPLUS
from ferrule_b200.ops import reference as ref

EPI_SWIGLU, EPI_SCATTER = "swiglu", "scatter"
BF = torch.bfloat16


def _gemm(x, w, out=None, *, out_dtype=BF, x_group_koff=0, out_group_coff=0, **_):
    xf = x.float()
    if w.dim() == 3 and x_group_koff:
        parts = [xf[:, g * x_group_koff:(g + 1) * x_group_koff] @ w[g].float().T for g in range(w.shape[0])]
        y = torch.cat(parts, dim=1)
        assert parts[0].shape[1] == out_group_coff
    else:
        y = xf @ (w[0] if w.dim() == 3 else w).float().T
    y = y.to(out_dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def _add_rmsnorm(x, weight, eps, norm_out=None):
    norm_out.copy_(ref.rmsnorm(x, weight, eps).to(norm_out.dtype))


def _argmax(logits):
    return logits.argmax(-1).to(torch.int32)


class _Plan:
    @staticmethod
    def allocate(*_a, **_k):
        return None


def _hc_pre(state, fn, scale, base, cfg, out_fp32=False, head_only=False):
    if head_only:
        return v4.hc_head(state, fn, scale, base, cfg).to(torch.float32 if out_fp32 else BF), None
    hidden, (pre, post, comb) = v4.hc_pre(state, fn, scale, base, cfg)
    coeff = torch.cat([pre, post, comb.reshape(state.shape[0], -1)], dim=1)
    return hidden.to(torch.float32 if out_fp32 else BF), coeff


def _hc_post(hidden, residual, coeff):
    hc = residual.shape[1]
    post, comb = coeff[:, hc:2 * hc], coeff[:, 2 * hc:].reshape(-1, hc, hc)
    return v4.hc_post(hidden, residual, post, comb).to(BF)


def _compressor_pool(kv, gate, ape, ratio, overlap, groups=None, row0=None, out=None):
    assert groups == 1
    W = ratio * (2 if overlap else 1)
    end = row0 + W
    dim = kv.shape[1] // 2 if overlap else kv.shape[1]
    return v4.compressor_pool(kv[:end], gate[:end], ape, ratio, overlap, dim)[-1:].to(BF)


def _hc_mean_scatter(state, taps, tap_index):
    H = state.shape[2]
    taps[:, tap_index * H:(tap_index + 1) * H] = v4.hc_mean_taps([state], state.shape[1]).to(taps.dtype)
    return taps


def _rope_rows(x, positions, cos, sin, off, rdim, inverse=False):
    p = positions.long()
    c, s = cos[p][:, None, :], sin[p][:, None, :]
    x[..., off:off + rdim] = ref.apply_rope(x[..., off:off + rdim], c, s, inverse=inverse).to(x.dtype)
    return x


def _indexer_scores(q, plane, head_w, out=None, **_):
    res = torch.stack([v4.indexer_topk(q[i], plane, head_w[i], 1, plane.shape[0])[1] for i in range(q.shape[0])])
    out.copy_(res)
    return out


def _indexer_topk(scores, k, n_visible=None):
    Q, n = scores.shape
    out = torch.full((Q, k), -1, dtype=torch.int32)
    for i in range(Q):
        vis = n if n_visible is None else int(n_visible[i])
        cand = scores[i, :vis]
        take = min(k, vis)
        if take:
            order = torch.sort(cand, descending=True, stable=True).indices[:take]
            good = torch.isfinite(cand[order])
            out[i, :take] = torch.where(good, order.to(torch.int32), torch.full_like(order, -1).to(torch.int32))
    return out


def _sparse_sink_attention(q, table, selection, kv_lora, rope_dim, scale, sink=None, **_):
    return v4.sparse_sink_attention(q, table, selection, kv_lora + rope_dim, scale, sink=sink).to(BF)


def _window_index_fill(sel, col0, window, positions, base):
    for r in range(sel.shape[0]):
        for j in range(window):
            p = int(positions[r]) - (window - 1 - j)
            sel[r, col0 + j] = int(base[r]) + p if p >= 0 else -1


def _offset_index_fill(sel, col0, idx, base):
    for r in range(sel.shape[0]):
        for j in range(idx.shape[1]):
            sel[r, col0 + j] = int(base[r]) + int(idx[r, j]) if int(idx[r, j]) >= 0 else -1


def _count_index_fill(sel, col0, width, counts, base):
    for r in range(sel.shape[0]):
        for j in range(width):
            sel[r, col0 + j] = int(base[r]) + j if j < int(counts[r]) else -1


def _moe(self, lw, xn, tok_t, B):
    """Routed + shared experts of `V4Cuda._moe` (router, top-k, SwiGLU experts, weighted sum) in plain tensors."""
    cfg = self.cfg
    rnd = ref.bf16_round
    x = xn.float()
    idx, wts = ref.route(x @ lw.router_w.float().T, cfg.topk, SCORE_SQRT_SOFTPLUS, bias=lw.router_bias, normalize=True,
                         route_scale=cfg.route_scale, hash_table=lw.hash_table, token_ids=tok_t)
    I = cfg.moe_inter
    out = torch.zeros_like(x)
    for r in range(B):
        for s_ in range(cfg.topk):
            e = int(idx[r, s_])
            y = x[r] @ lw.e_w13[e].float().T
            h = rnd(ref.swiglu(y[:I], y[I:], cfg.swiglu_limit))
            out[r] += rnd((h @ lw.e_w2[e].float().T) * wts[r, s_])
    aq = v4.qat_linear_input if cfg.qat else (lambda t: t)
    y = aq(x) @ lw.w13[0].float().T
    sI = y.shape[1] // 2
    h = rnd(ref.swiglu(y[:, :sI], y[:, sI:], cfg.swiglu_limit))
    return rnd(out + rnd(aq(h) @ lw.w2[0].float().T)).to(BF)


def install(model):
    """Point a `V4Cuda` built on CPU tensors at the stand-ins."""
    model.K = SimpleNamespace(gemm=_gemm, add_rmsnorm=_add_rmsnorm, argmax=_argmax, MoePlan=_Plan,
                              embedding=lambda tok, table: table[tok.long()], EPI_SWIGLU=EPI_SWIGLU, EPI_SCATTER=EPI_SCATTER)
    model.K4 = SimpleNamespace(hc_pre=_hc_pre, hc_post=_hc_post, compressor_pool=_compressor_pool, rope_rows=_rope_rows,
                               indexer_scores=_indexer_scores, indexer_topk=_indexer_topk, hc_mean_scatter=_hc_mean_scatter,
                               sparse_sink_attention=_sparse_sink_attention)
    model.M = SimpleNamespace(window_index_fill=_window_index_fill, offset_index_fill=_offset_index_fill,
                              count_index_fill=_count_index_fill)
    model._moe = _moe.__get__(model)
    return model
