"""DeepSeek-V4 family model: hyper-connected residual streams, hybrid sparse attention over a sliding
window plus compressed KV (ratio-4 layers pick compressed rows with a learned indexer, ratio-128 layers
see all of them), grouped low-rank output projection, hash / sqrt-softplus routed MoE.

    layer:  hc_pre -> RMSNorm -> attention -> hc_post -> hc_pre -> RMSNorm -> MoE (+ shared) -> hc_post
    attention (one shared K = V head of `head_dim`, RoPE on its tail):
        q = per-head-RMS(wq_b . RMS(wq_a . x)), RoPE tail        kv = RoPE tail(RMS(wkv . x)) -> window
        compressor: softmax-pool every `ratio` projected rows (overlapping for ratio 4) -> RMS -> RoPE
        selection = last `window` rows U (indexer top-k | all) compressed rows, sink in the denominator
        out = wo_b . grouped(wo_a)(inverse-RoPE tail(attn))

`V4Reference` is the fp32 PyTorch oracle (token by token, explicit caches); `V4Cuda` runs decode steps for
a batch of sequences on the sm_100a kernels (`ops/v4.py`, the tcgen05 GEMMs and the MoE kernels) with
device-resident tables.  Weights bind to checkpoint names through `TENSOR_NAMES`.

Counterpart of crates/ferrule-model/src/models/deepseek_v4/{config.rs:118-272, attention.rs:1194-1364,
layer.rs:391-470, helpers.rs:395-505, checkpoint_binding.rs:31-700}; family constants from
crates/ferrule-model/src/families/deepseek_v4.rs:9-38.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import reference as ref
from . import v4
from .config import SCORE_SQRT_SOFTPLUS


@dataclass(frozen=True)
class V4Config:
    hidden: int = 4096
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    norm_eps: float = 1e-6
    n_layers: int = 43
    n_hash_layers: int = 3
    n_heads: int = 64
    head_dim: int = 512
    q_lora_rank: int = 1024
    rope_dim: int = 64
    o_groups: int = 8
    o_lora_rank: int = 1024
    window: int = 128
    vocab_size: int = 129_280
    n_routed_experts: int = 256
    topk: int = 6
    moe_inter: int = 2048
    n_shared_experts: int = 1
    swiglu_limit: float = 10.0
    route_scale: float = 1.5
    rope_theta: float = 10_000.0
    compress_rope_theta: float = 160_000.0
    rope_factor: float = 16.0
    rope_orig_max_pos: int = 65_536
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 512
    compress_ratios: Tuple[int, ...] = ()          # per layer: 0 (window only), 4 (indexer) or 128 (all rows)
    indexer_ratio: int = 4                          # the ratio whose layers overlap windows and use the indexer
    proposal_block_size: int = 5
    max_position: int = 4096
    # proposal attachment (the checkpoint's `mtp.*` stages): 0 stages = none.  Stages are window-only V4 layers
    # with a learned router; `proposal_target_layers` names the target layers whose output is tapped
    n_proposal_stages: int = 0
    proposal_target_layers: Tuple[int, ...] = ()
    proposal_noise_token: int = 0
    proposal_markov_rank: int = 256
    # quantisation-aware-training steps inside the forward pass (FP8 on KV rows and on the inputs of the linears
    # the checkpoint stores quantised, Hadamard + FP4 on the indexer's rows): on for checkpoints trained that way
    qat: bool = False

    def ratio(self, layer: int) -> int:
        return self.compress_ratios[layer] if layer < len(self.compress_ratios) else 0

    def has_indexer(self, layer: int) -> bool:
        return self.ratio(layer) == self.indexer_ratio and self.indexer_ratio > 0

    @property
    def group_in(self) -> int:
        return self.n_heads // self.o_groups * self.head_dim

    @property
    def hc(self) -> v4.HcConfig:
        return v4.HcConfig(self.hc_mult, self.hidden, self.hc_eps, self.norm_eps, self.hc_sinkhorn_iters)

    @property
    def softmax_scale(self) -> float:
        return self.head_dim ** -0.5

    def with_(self, **kw) -> "V4Config":
        return replace(self, **kw)


def deepseek_v4_flash() -> V4Config:
    """Family defaults; the per-layer compression schedule alternates ratio 4 and ratio 128 after a window-only
    first layer (the checkpoint's config.json overrides it)."""
    ratios = tuple(0 if i == 0 else (4 if i % 2 else 128) for i in range(43))
    return V4Config(compress_ratios=ratios)


def tiny_v4() -> V4Config:
    """Small shape that exercises every branch: window-only, ratio-4 + indexer, direct ratio-8 layers, one
    hash-routed layer."""
    return V4Config(hidden=256, hc_mult=4, n_layers=3, n_hash_layers=1, n_heads=4, head_dim=64, q_lora_rank=128,
                    rope_dim=16, o_groups=2, o_lora_rank=64, window=8, vocab_size=512, n_routed_experts=8, topk=2,
                    moe_inter=128, index_n_heads=4, index_head_dim=32, index_topk=4, compress_ratios=(0, 4, 8),
                    rope_factor=1.0, max_position=512)


# checkpoint tensor names (HuggingFace DeepSeek-V4 layout) -> attribute of V4LayerWeights / V4Weights
TENSOR_NAMES: Dict[str, str] = {
    "embed.weight": "embed", "norm.weight": "final_norm", "head.weight": "lm_head",
    "hc_head_fn": "hc_head_fn", "hc_head_scale": "hc_head_scale", "hc_head_base": "hc_head_base",
    "layers.{i}.attn_norm.weight": "attn_norm", "layers.{i}.attn.wq_a.weight": "wq_a",
    "layers.{i}.attn.q_norm.weight": "q_norm", "layers.{i}.attn.wq_b.weight": "wq_b",
    "layers.{i}.attn.wkv.weight": "wkv", "layers.{i}.attn.kv_norm.weight": "kv_norm",
    "layers.{i}.attn.attn_sink": "sink", "layers.{i}.attn.wo_a.weight": "wo_a", "layers.{i}.attn.wo_b.weight": "wo_b",
    "layers.{i}.attn.compressor.wkv.weight": "c_wkv", "layers.{i}.attn.compressor.wgate.weight": "c_wgate",
    "layers.{i}.attn.compressor.ape": "c_ape", "layers.{i}.attn.compressor.norm.weight": "c_norm",
    "layers.{i}.attn.indexer.wq_b.weight": "i_wq_b", "layers.{i}.attn.indexer.weights_proj.weight": "i_weights",
    "layers.{i}.attn.indexer.compressor.wkv.weight": "ic_wkv", "layers.{i}.attn.indexer.compressor.wgate.weight": "ic_wgate",
    "layers.{i}.attn.indexer.compressor.ape": "ic_ape", "layers.{i}.attn.indexer.compressor.norm.weight": "ic_norm",
    "layers.{i}.ffn_norm.weight": "ffn_norm", "layers.{i}.ffn.gate.weight": "router_w", "layers.{i}.ffn.gate.bias": "router_bias",
    "layers.{i}.ffn.gate.tid2eid": "hash_table", "layers.{i}.hc_attn_fn": "hc_attn_fn", "layers.{i}.hc_attn_scale": "hc_attn_scale",
    "layers.{i}.hc_attn_base": "hc_attn_base", "layers.{i}.hc_ffn_fn": "hc_ffn_fn", "layers.{i}.hc_ffn_scale": "hc_ffn_scale",
    "layers.{i}.hc_ffn_base": "hc_ffn_base",
}


@dataclass
class V4LayerWeights:
    hc_attn_fn: torch.Tensor
    hc_attn_scale: torch.Tensor
    hc_attn_base: torch.Tensor
    hc_ffn_fn: torch.Tensor
    hc_ffn_scale: torch.Tensor
    hc_ffn_base: torch.Tensor
    attn_norm: torch.Tensor
    wq_a: torch.Tensor
    q_norm: torch.Tensor
    wq_b: torch.Tensor
    wkv: torch.Tensor
    kv_norm: torch.Tensor
    sink: torch.Tensor
    wo_a: torch.Tensor            # [o_groups, o_lora, group_in]
    wo_b: torch.Tensor
    ffn_norm: torch.Tensor
    router_w: torch.Tensor
    e_w13: torch.Tensor
    e_w2: torch.Tensor
    w13: torch.Tensor
    w2: torch.Tensor
    router_bias: Optional[torch.Tensor] = None
    hash_table: Optional[torch.Tensor] = None
    c_wkv: Optional[torch.Tensor] = None
    c_wgate: Optional[torch.Tensor] = None
    c_ape: Optional[torch.Tensor] = None
    c_norm: Optional[torch.Tensor] = None
    i_wq_b: Optional[torch.Tensor] = None
    i_weights: Optional[torch.Tensor] = None
    ic_wkv: Optional[torch.Tensor] = None
    ic_wgate: Optional[torch.Tensor] = None
    ic_ape: Optional[torch.Tensor] = None
    ic_norm: Optional[torch.Tensor] = None


@dataclass
class V4ProposalWeights:
    """The `mtp.*` namespace: stages (stage 0 also owns the projection of the target taps), prediction heads of
    the last stage (crates/ferrule-model/src/models/deepseek_v4/proposal_attachment.rs:57-91)."""
    stages: List[V4LayerWeights]
    main_proj: torch.Tensor          # [hidden, taps * hidden]
    main_norm: torch.Tensor
    hc_head_fn: torch.Tensor
    hc_head_scale: torch.Tensor
    hc_head_base: torch.Tensor
    norm: torch.Tensor
    markov_w1: torch.Tensor          # [vocab, rank]
    markov_w2: torch.Tensor          # [vocab, rank]
    confidence_proj: torch.Tensor    # [1, hidden + rank]


@dataclass
class V4Weights:
    cfg: V4Config
    embed: torch.Tensor
    layers: List[V4LayerWeights]
    hc_head_fn: torch.Tensor
    hc_head_scale: torch.Tensor
    hc_head_base: torch.Tensor
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    proposal: Optional[V4ProposalWeights] = None


def random_v4_weights(cfg: V4Config, device="cpu", seed: int = 0, std: float = 0.05) -> V4Weights:
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16

    def n(*shape, dtype=bf, s=std):
        return (torch.randn(*shape, generator=g) * s).to(dtype).to(device)

    def ones(*shape):
        return torch.ones(*shape, dtype=bf, device=device)

    H, hc, hd = cfg.hidden, cfg.hc_mult, cfg.head_dim
    mix = 2 * hc + hc * hc

    def layer(hashed: bool, r: int, indexer: bool) -> V4LayerWeights:
        E, I = cfg.n_routed_experts, cfg.moe_inter
        sI = cfg.n_shared_experts * I
        lw = V4LayerWeights(
            hc_attn_fn=n(mix, hc * H, dtype=torch.float32, s=0.02), hc_attn_scale=torch.tensor([0.7, 1.1, 0.9], device=device),
            hc_attn_base=n(mix, dtype=torch.float32, s=0.3),
            hc_ffn_fn=n(mix, hc * H, dtype=torch.float32, s=0.02), hc_ffn_scale=torch.tensor([0.9, 0.8, 1.2], device=device),
            hc_ffn_base=n(mix, dtype=torch.float32, s=0.3),
            attn_norm=ones(H), wq_a=n(cfg.q_lora_rank, H), q_norm=ones(cfg.q_lora_rank), wq_b=n(cfg.n_heads * hd, cfg.q_lora_rank),
            wkv=n(hd, H), kv_norm=ones(hd), sink=n(cfg.n_heads, dtype=torch.float32, s=0.5),
            wo_a=n(cfg.o_groups, cfg.o_lora_rank, cfg.group_in), wo_b=n(H, cfg.o_groups * cfg.o_lora_rank),
            ffn_norm=ones(H), router_w=n(E, H),
            e_w13=n(E, 2 * I, H), e_w2=n(E, H, I), w13=n(1, 2 * sI, H), w2=n(1, H, sI))
        if hashed:
            lw.hash_table = torch.randint(0, E, (cfg.vocab_size, cfg.topk), generator=g).to(device)
        else:
            lw.router_bias = n(E, dtype=torch.float32, s=0.1)
        if r:
            od = hd * (2 if indexer else 1)
            lw.c_wkv, lw.c_wgate = n(od, H), n(od, H)
            lw.c_ape, lw.c_norm = n(r, od, dtype=torch.float32, s=0.5), ones(hd)
        if indexer:
            idim = cfg.index_head_dim
            lw.i_wq_b, lw.i_weights = n(cfg.index_n_heads * idim, cfg.q_lora_rank), n(cfg.index_n_heads, H)
            lw.ic_wkv, lw.ic_wgate = n(2 * idim, H), n(2 * idim, H)
            lw.ic_ape, lw.ic_norm = n(r, 2 * idim, dtype=torch.float32, s=0.5), ones(idim)
        return lw

    layers = [layer(i < cfg.n_hash_layers, cfg.ratio(i), cfg.has_indexer(i)) for i in range(cfg.n_layers)]
    w = V4Weights(cfg, n(cfg.vocab_size, H, s=0.5), layers, n(hc, hc * H, dtype=torch.float32, s=0.02),
                  torch.tensor([1.0], device=device), n(hc, dtype=torch.float32, s=0.3), ones(H), n(cfg.vocab_size, H))
    if cfg.n_proposal_stages:
        rank = cfg.proposal_markov_rank
        w.proposal = V4ProposalWeights(
            stages=[layer(False, 0, False) for _ in range(cfg.n_proposal_stages)],
            main_proj=n(H, len(cfg.proposal_target_layers) * H), main_norm=ones(H),
            hc_head_fn=n(hc, hc * H, dtype=torch.float32, s=0.02), hc_head_scale=torch.tensor([1.0], device=device),
            hc_head_base=n(hc, dtype=torch.float32, s=0.3), norm=ones(H),
            markov_w1=n(cfg.vocab_size, rank, s=0.3), markov_w2=n(cfg.vocab_size, rank, s=0.3),
            confidence_proj=n(1, H + rank, s=0.3))
    return w


def _rope_tables(cfg: V4Config, theta: float, dim: int, device):
    cos, sin = ref.rope_tables(cfg.max_position, dim, theta, cfg.rope_factor, cfg.rope_orig_max_pos)
    return cos.to(device), sin.to(device)


def _rope_tail(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: int, rdim: int, inverse: bool = False):
    """x [..., head_dim]: rotate the last `rdim` entries at position `pos`."""
    out = x.clone()
    out[..., -rdim:] = ref.apply_rope(x[..., -rdim:], cos[pos], sin[pos], inverse=inverse)
    return out


class _CompressorState:
    """Projected rows of one sequence for one compressor (the oracle keeps all of them)."""

    def __init__(self):
        self.kv: List[torch.Tensor] = []
        self.gate: List[torch.Tensor] = []


class V4SeqCache:
    """Per-sequence oracle state: per layer raw KV rows, compressed rows, indexer rows, compressor inputs."""

    def __init__(self, cfg: V4Config):
        L = cfg.n_layers
        self.kv = [[] for _ in range(L)]
        self.comp = [[] for _ in range(L)]
        self.icomp = [[] for _ in range(L)]
        self.cstate = [_CompressorState() for _ in range(L)]
        self.istate = [_CompressorState() for _ in range(L)]
        self.pctx = [[] for _ in range(cfg.n_proposal_stages)]     # proposal stages' context KV rows by position
        self.position = 0


class V4Reference:
    def __init__(self, w: V4Weights):
        self.w, self.cfg = w, w.cfg
        dev = w.embed.device
        cfg = self.cfg
        self.rope = _rope_tables(cfg, cfg.rope_theta, cfg.rope_dim, dev)
        self.crope = _rope_tables(cfg, cfg.compress_rope_theta, cfg.rope_dim, dev)
        self.irope = _rope_tables(cfg, cfg.compress_rope_theta, min(cfg.rope_dim, cfg.index_head_dim), dev)
        self.rnd = ref.bf16_round
        self.proposal = None
        if w.proposal is not None:
            from .v4_proposal import V4Proposal
            self.proposal = V4Proposal(w, self.rope)
        self.prof = None               # utils.stage_profile.StageProfiler

    def propose(self, c: V4SeqCache, n_committed: int, anchor: int):
        """Drafts after `anchor` for a sequence with `n_committed` committed tokens -> (token ids, confidence logits)."""
        hd = self.cfg.head_dim
        ctx = [torch.stack(rows[:n_committed]) if n_committed else torch.zeros(0, hd, device=self.w.embed.device)
               for rows in c.pctx]
        return self.proposal.propose(ctx, n_committed, anchor)

    def _compress(self, st: _CompressorState, wkv, wgate, ape, norm, xn, pos: int, ratio: int, overlap: bool, dim: int,
                  rope, rdim: int, indexer_plane: bool = False) -> Optional[torch.Tensor]:
        st.kv.append(xn @ wkv.float().T)
        st.gate.append(xn @ wgate.float().T)
        if (pos + 1) % ratio:
            return None
        pooled = v4.compressor_pool(torch.stack(st.kv), torch.stack(st.gate), ape, ratio, overlap, dim)[-1]
        row = self.rnd(ref.rmsnorm(pooled[None], norm, self.cfg.norm_eps))[0]
        row = self.rnd(_rope_tail(row, rope[0], rope[1], pos + 1 - ratio, rdim))
        if self.cfg.qat:
            row = v4.qat_indexer_rows(row) if indexer_plane else v4.qat_kv_rows(row, rdim)
        return row

    def _attention(self, lw: V4LayerWeights, layer: int, x: torch.Tensor, c: V4SeqCache, pos: int) -> torch.Tensor:
        cfg, rnd = self.cfg, self.rnd
        hd, rd, nh = cfg.head_dim, cfg.rope_dim, cfg.n_heads
        aq = v4.qat_linear_input if cfg.qat else (lambda t: t)       # inputs of the linears stored quantised
        xa = aq(x)
        q_lat = rnd(xa @ lw.wq_a.float().T)
        qn = rnd(ref.rmsnorm(q_lat[None], lw.q_norm, cfg.norm_eps))[0]
        q = rnd(aq(qn) @ lw.wq_b.float().T).view(nh, hd)
        q = rnd(ref.rmsnorm(q, None, cfg.norm_eps))
        q = rnd(_rope_tail(q, self.rope[0], self.rope[1], pos, rd))
        kv = rnd(xa @ lw.wkv.float().T)
        kv = rnd(ref.rmsnorm(kv[None], lw.kv_norm, cfg.norm_eps))[0]
        kv = rnd(_rope_tail(kv, self.rope[0], self.rope[1], pos, rd))
        if cfg.qat:
            kv = v4.qat_kv_rows(kv, rd)
        c.kv[layer].append(kv)
        ratio = cfg.ratio(layer)
        sel_comp: List[int] = []
        if ratio:
            if cfg.has_indexer(layer):
                idim = cfg.index_head_dim
                new_i = self._compress(c.istate[layer], lw.ic_wkv, lw.ic_wgate, lw.ic_ape, lw.ic_norm, x, pos, ratio, True,
                                       idim, self.irope, min(rd, idim), indexer_plane=True)
                if new_i is not None:
                    c.icomp[layer].append(new_i)
            new_c = self._compress(c.cstate[layer], lw.c_wkv, lw.c_wgate, lw.c_ape, lw.c_norm, x, pos, ratio,
                                   cfg.has_indexer(layer), hd, self.crope, rd)
            if new_c is not None:
                c.comp[layer].append(new_c)
            n_c = len(c.comp[layer])
            if cfg.has_indexer(layer) and n_c:
                idim, ih = cfg.index_head_dim, cfg.index_n_heads
                iq = rnd(aq(qn) @ lw.i_wq_b.float().T).view(ih, idim)
                iq = rnd(_rope_tail(iq, self.irope[0], self.irope[1], pos, min(rd, idim)))
                if cfg.qat:
                    iq = v4.qat_indexer_rows(iq)
                wts = rnd(x @ lw.i_weights.float().T)
                wts = rnd(wts * (idim ** -0.5 * ih ** -0.5))
                idx, _ = v4.indexer_topk(iq, torch.stack(c.icomp[layer]), wts, cfg.index_topk, n_c)
                sel_comp = [int(i) for i in idx.tolist() if i >= 0]
            else:
                sel_comp = list(range(n_c))
        win = [p for p in range(pos - cfg.window + 1, pos + 1) if p >= 0]
        rows = [c.kv[layer][p] for p in win] + [c.comp[layer][j] for j in sel_comp]
        table = torch.stack(rows)
        sel = torch.arange(len(rows), dtype=torch.int32, device=table.device)[None]
        o = v4.sparse_sink_attention(q[None], table, sel, hd, cfg.softmax_scale, sink=lw.sink)[0]      # [heads, hd]
        o = rnd(o)
        o = rnd(_rope_tail(o, self.rope[0], self.rope[1], pos, rd, inverse=True))
        og = o.reshape(cfg.o_groups, cfg.group_in)
        # the grouped first stage multiplies dequantised weights without quantising its input; the second is a linear
        lat = rnd(torch.einsum("gk,gnk->gn", og, lw.wo_a.float())).reshape(-1)
        return rnd(aq(lat) @ lw.wo_b.float().T)

    def _moe(self, lw: V4LayerWeights, x: torch.Tensor, token: int) -> torch.Tensor:
        cfg, rnd = self.cfg, self.rnd
        logits = (x @ lw.router_w.float().T)[None]
        tok = torch.tensor([token], device=x.device)
        idx, wts = ref.route(logits, cfg.topk, SCORE_SQRT_SOFTPLUS, bias=lw.router_bias, normalize=True,
                             route_scale=cfg.route_scale, hash_table=lw.hash_table, token_ids=tok)
        I = cfg.moe_inter
        out = torch.zeros_like(x)
        for s in range(cfg.topk):
            e = int(idx[0, s])
            y = x @ lw.e_w13[e].float().T
            h = rnd(ref.swiglu(y[:I], y[I:], cfg.swiglu_limit))
            out = out + rnd((h @ lw.e_w2[e].float().T) * wts[0, s])
        aq = v4.qat_linear_input if cfg.qat else (lambda t: t)       # the shared experts are stored in FP8
        y = aq(x) @ lw.w13[0].float().T
        sI = y.shape[0] // 2
        h = rnd(ref.swiglu(y[:sI], y[sI:], cfg.swiglu_limit))
        return rnd(out + rnd(aq(h) @ lw.w2[0].float().T))

    def step(self, c: V4SeqCache, token: int) -> torch.Tensor:
        """Feed one token of one sequence; returns fp32 logits [vocab]."""
        cfg, rnd, w = self.cfg, self.rnd, self.w
        pos = c.position
        state = w.embed[token].float()[None, None].repeat(1, cfg.hc_mult, 1)            # [1, hc, H]
        taps = []
        prof = self.prof
        for i, lw in enumerate(w.layers):
            if prof is not None:
                prof.mark(i, "attn")
            x, (_, post, comb) = v4.hc_pre(state, lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, cfg.hc)
            x = rnd(x)
            xn = rnd(ref.rmsnorm(x, lw.attn_norm, cfg.norm_eps))[0]
            a = self._attention(lw, i, xn, c, pos)
            state = rnd(v4.hc_post(a[None], state, post, comb))
            if prof is not None:
                prof.mark(i, "moe")
            x, (_, post, comb) = v4.hc_pre(state, lw.hc_ffn_fn, lw.hc_ffn_scale, lw.hc_ffn_base, cfg.hc)
            x = rnd(x)
            xn = rnd(ref.rmsnorm(x, lw.ffn_norm, cfg.norm_eps))[0]
            f = self._moe(lw, xn, token)
            state = rnd(v4.hc_post(f[None], state, post, comb))
            if self.proposal is not None and i in cfg.proposal_target_layers:
                taps.append(self.proposal.tap(state))
        if prof is not None:
            prof.mark(cfg.n_layers, "head")
        if self.proposal is not None:
            # every target row leaves one context KV row per proposal stage at its position
            main_x = self.proposal.main_rows(taps)
            pos_t = torch.tensor([pos], device=main_x.device)
            for s_, rows in enumerate(c.pctx):
                del rows[pos:]
                rows.append(self.proposal.context_kv(s_, main_x, pos_t)[0])
        h = rnd(v4.hc_head(state, w.hc_head_fn, w.hc_head_scale, w.hc_head_base, cfg.hc))
        hn = rnd(ref.rmsnorm(h, w.final_norm, cfg.norm_eps))[0]
        c.position += 1
        logits = hn @ w.lm_head.float().T
        if prof is not None:
            prof.mark(cfg.n_layers, None)
        return logits


class _OffsetRows:
    """Rows [lo, hi) of a position-indexed plane, sliced with absolute positions (`x[a:b]` with lo <= a)."""

    def __init__(self, plane: torch.Tensor, lo: int, hi: int):
        self.plane, self.lo, self.hi = plane, lo, hi

    def __getitem__(self, sl: slice) -> torch.Tensor:
        a, b = max(sl.start or 0, self.lo), min(self.hi if sl.stop is None else sl.stop, self.hi)
        return self.plane[a:max(a, b)]


class V4Cuda:
    """Decode steps for a batch of sequences on the sm_100a kernels.

    Device-resident per layer: one combined KV table per sequence (`[max_len raw rows | max_len / ratio
    compressed rows]`, bf16), the compressors' projected rows (fp32, pooled at every group boundary) and the
    indexer's compressed plane.  Every step runs one token per active sequence; sequence slots are fixed.
    """

    def __init__(self, w: V4Weights, max_seqs: int, max_len: int, max_rows: int = 0):
        from ..ops import kernels as K
        from ..ops import movers as M
        from ..ops import v4 as K4
        self.K, self.K4, self.M = K, K4, M
        self.w, self.cfg = w, w.cfg
        cfg = self.cfg
        dev = w.embed.device
        self.device, self.max_seqs, self.max_len = dev, max_seqs, max_len
        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.rope = _rope_tables(cfg, cfg.rope_theta, cfg.rope_dim, dev)
        self.crope = _rope_tables(cfg, cfg.compress_rope_theta, cfg.rope_dim, dev)
        self.irope = _rope_tables(cfg, cfg.compress_rope_theta, min(cfg.rope_dim, cfg.index_head_dim), dev)
        hd = cfg.head_dim
        self.tables, self.proj, self.iproj, self.iplane, self.stride = [], [], [], [], []
        for i in range(cfg.n_layers):
            r = cfg.ratio(i)
            n_c = max_len // r if r else 0
            self.stride.append(max_len + n_c)
            self.tables.append(torch.zeros(max_seqs, max_len + n_c, hd, **bf))
            od = hd * (2 if cfg.has_indexer(i) else 1)
            self.proj.append((torch.zeros(max_seqs, max_len, od, **f32), torch.zeros(max_seqs, max_len, od, **f32)) if r else None)
            if cfg.has_indexer(i):
                idim = cfg.index_head_dim
                self.iproj.append((torch.zeros(max_seqs, max_len, 2 * idim, **f32), torch.zeros(max_seqs, max_len, 2 * idim, **f32)))
                self.iplane.append(torch.zeros(max_seqs, n_c, idim, **bf))
            else:
                self.iproj.append(None)
                self.iplane.append(None)
        E, k = cfg.n_routed_experts, cfg.topk
        R = self.max_rows = max(max_rows, max_seqs)          # rows of one call: decode rows or a prefill chunk
        self.plan = K.MoePlan.allocate(R * k, E, 16, dev)
        self.ones_hd = torch.ones(hd, **bf)
        self.ones_id = torch.ones(cfg.index_head_dim, **bf)
        self.positions = [0] * max_seqs
        self.launch_note = "decode: one token per sequence per step"
        # proposal attachment: one context KV plane per stage, addressed by (slot, position) like the other tables
        self.prof = None               # utils.stage_profile.StageProfiler (marks are CUDA events)
        self.proposal = None
        self.pctx = []
        if w.proposal is not None:
            from .v4_proposal import V4Proposal
            self.proposal = V4Proposal(w, self.rope)
            self.pctx = [torch.zeros(max_seqs, max_len, hd, **bf) for _ in range(cfg.n_proposal_stages)]

    def propose(self, slot: int, n_committed: int, anchor: int):
        lo = max(0, n_committed - self.cfg.window)
        # the proposal reads rows [lo, n_committed): hand it a view whose row index is the position
        ctx = [_OffsetRows(t[slot], lo, n_committed) for t in self.pctx]
        return self.proposal.propose(ctx, n_committed, anchor)

    # -- helpers ---------------------------------------------------------------------------
    def _norm(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        self.K.add_rmsnorm(x, weight, self.cfg.norm_eps, norm_out=out)
        return out

    def _compress(self, layer: int, proj, wkv, wgate, ape, norm_w, xn, seqs, pos, ratio, overlap, dim, rope, rdim,
                  indexer_plane: bool = False):
        """Append the projected rows of this step; return [(sequence, group, bf16 row)] for finished groups."""
        K, K4, cfg = self.K, self.K4, self.cfg
        pk = K.gemm(xn, wkv, out_dtype=torch.float32)
        pg = K.gemm(xn, wgate, out_dtype=torch.float32)
        sl = torch.tensor(seqs, device=self.device)
        pl = torch.tensor(pos, device=self.device)
        proj[0][sl, pl] = pk
        proj[1][sl, pl] = pg
        done = []
        W = ratio * (2 if overlap else 1)
        for s, p in zip(seqs, pos):
            if (p + 1) % ratio:
                continue
            g = (p + 1) // ratio - 1
            pooled = K4.compressor_pool(proj[0][s], proj[1][s], ape, ratio, overlap, groups=1,
                                        row0=(g + 1) * ratio - W)
            row = self._norm(pooled, norm_w)
            cp = torch.tensor([p + 1 - ratio], dtype=torch.int32, device=self.device)
            K4.rope_rows(row.view(1, 1, dim), cp, rope[0], rope[1], off=dim - rdim, rdim=rdim)
            if cfg.qat:
                row = v4.qat_indexer_rows(row) if indexer_plane else v4.qat_kv_rows(row, rdim)
            done.append((s, g, row[0]))
        return done

    def step(self, seqs: List[int], tokens: List[int]):
        """One decode step for the sequences in slots `seqs` -> (next token ids [B] int32, fp32 logits [B, vocab])."""
        return self.step_rows(seqs, tokens)

    def step_rows(self, seqs: List[int], tokens: List[int], positions: Optional[List[int]] = None,
                  want_rows: Optional[List[int]] = None):
        """Rows of any mix of sequences in one pass: row r feeds `tokens[r]` to the sequence in slot `seqs[r]` at
        `positions[r]` (default: one row per sequence at its current position - a decode step).  The rows of a
        sequence must be consecutive positions in increasing order: a prompt chunk goes through the layers as ONE
        batch - every GEMM sees all rows, the tables take all rows of a layer before its attention reads them,
        and each row's selection list (window, visible compressed rows) is cut at its own position, which is what
        keeps the chunk causal.  `want_rows`: rows whose logits are wanted (default all).
        -> (next token ids, fp32 logits) for the wanted rows."""
        K, K4, M, cfg, w = self.K, self.K4, self.M, self.cfg, self.w
        dev = self.device
        B = len(seqs)
        assert 0 < B <= self.max_rows, f"{B} rows, the workspace holds {self.max_rows}"
        hd, rd, nh, H, hc = cfg.head_dim, cfg.rope_dim, cfg.n_heads, cfg.hidden, cfg.hc_mult
        pos = [self.positions[s] for s in seqs] if positions is None else list(positions)
        last = {}
        for s, p in zip(seqs, pos):
            assert p == last.get(s, p - 1) + 1, "rows of a sequence must be consecutive positions"
            last[s] = p
        assert max(pos) < self.max_len
        pos_t = torch.tensor(pos, dtype=torch.int32, device=dev)
        seq_t = torch.tensor(seqs, dtype=torch.int64, device=dev)
        tok_t = torch.tensor(tokens, dtype=torch.int32, device=dev)
        emb = K.embedding(tok_t, w.embed)
        state = emb[:, None, :].expand(B, hc, H).contiguous()
        taps = None
        if self.proposal is not None:
            taps = torch.empty(B, len(cfg.proposal_target_layers) * H, dtype=torch.bfloat16, device=dev)
        prof = self.prof
        for i, lw in enumerate(w.layers):
            if prof is not None:
                prof.mark(i, "attn.proj")
            x, coeff = K4.hc_pre(state, lw.hc_attn_fn, lw.hc_attn_scale, lw.hc_attn_base, cfg.hc)
            xn = self._norm(x, lw.attn_norm)
            # ---- attention ----
            # QAT checkpoints: FP8 quantise-dequantise of the rows in front of the linears stored quantised, of
            # the KV rows, Hadamard + FP4 of the indexer's rows (elementwise tensor operations on a few rows)
            aq = v4.qat_linear_input if cfg.qat else (lambda t: t)
            xa = aq(xn)
            qn = self._norm(K.gemm(xa, lw.wq_a), lw.q_norm)
            qa = aq(qn)
            q = K.gemm(qa, lw.wq_b)
            q = self._norm(q.view(B * nh, hd), self.ones_hd).view(B, nh, hd)
            K4.rope_rows(q, pos_t, self.rope[0], self.rope[1], off=hd - rd, rdim=rd)
            kv = self._norm(K.gemm(xa, lw.wkv), lw.kv_norm)
            K4.rope_rows(kv.view(B, 1, hd), pos_t, self.rope[0], self.rope[1], off=hd - rd, rdim=rd)
            if cfg.qat:
                kv = v4.qat_kv_rows(kv, rd)
            if prof is not None:
                prof.mark(i, "attn.select")
            table = self.tables[i]
            table[seq_t, pos_t.long()] = kv
            ratio = cfg.ratio(i)
            stride = self.stride[i]
            base = seq_t * stride
            # selection list [window | compressed rows], filled in place by the index-fill kernels
            n_c = [(p + 1) // ratio for p in pos] if ratio else []
            n_max = max(n_c) if n_c else 0
            sel_w = cfg.window + ((min(cfg.index_topk, 512) if n_max else 0) if (ratio and cfg.has_indexer(i)) else n_max)
            selection = torch.empty(B, sel_w, dtype=torch.int32, device=dev)
            M.window_index_fill(selection, 0, cfg.window, pos_t, base)
            if ratio:
                if cfg.has_indexer(i):
                    idim = cfg.index_head_dim
                    for s, g, row in self._compress(i, self.iproj[i], lw.ic_wkv, lw.ic_wgate, lw.ic_ape, lw.ic_norm, xn,
                                                    seqs, pos, ratio, True, idim, self.irope, min(rd, idim),
                                                    indexer_plane=True):
                        self.iplane[i][s, g] = row
                for s, g, row in self._compress(i, self.proj[i], lw.c_wkv, lw.c_wgate, lw.c_ape, lw.c_norm, xn, seqs,
                                                pos, ratio, cfg.has_indexer(i), hd, self.crope, rd):
                    table[s, self.max_len + g] = row
                if n_max:
                    if cfg.has_indexer(i):
                        idim, ih = cfg.index_head_dim, cfg.index_n_heads
                        iq = K.gemm(qa, lw.i_wq_b).view(B, ih, idim)
                        K4.rope_rows(iq, pos_t, self.irope[0], self.irope[1], off=idim - min(rd, idim), rdim=min(rd, idim))
                        if cfg.qat:
                            iq = v4.qat_indexer_rows(iq).contiguous()
                        wts = K.gemm(xn, lw.i_weights, out_dtype=torch.float32)
                        wts = (wts.bfloat16().float() * (idim ** -0.5 * ih ** -0.5)).bfloat16().float().contiguous()
                        scores = torch.full((B, n_max), float("-inf"), dtype=torch.float32, device=dev)
                        b0 = 0
                        while b0 < B:                          # every sequence scores its own plane: one call for
                            b1 = b0 + 1                        # the run of rows it has in this batch
                            while b1 < B and seqs[b1] == seqs[b0]:
                                b1 += 1
                            n_run = n_c[b1 - 1]                # positions increase along a run
                            if n_run:
                                K4.indexer_scores(iq[b0:b1], self.iplane[i][seqs[b0], :n_run], wts[b0:b1],
                                                  out=scores[b0:b1, :n_run])
                            b0 = b1
                        vis = torch.tensor(n_c, dtype=torch.int32, device=dev)
                        idx = K4.indexer_topk(scores, min(cfg.index_topk, 512), vis)
                        assert idx.shape[1] == sel_w - cfg.window
                        M.offset_index_fill(selection, cfg.window, idx.int().contiguous(), base + self.max_len)
                    else:
                        vis = torch.tensor(n_c, dtype=torch.int32, device=dev)
                        M.count_index_fill(selection, cfg.window, n_max, vis, base + self.max_len)
            if prof is not None:
                prof.mark(i, "attn.core")
            o = K4.sparse_sink_attention(q, table.view(-1, hd), selection, hd, 0, cfg.softmax_scale, sink=lw.sink)
            if prof is not None:
                prof.mark(i, "attn.out")
            K4.rope_rows(o, pos_t, self.rope[0], self.rope[1], off=hd - rd, rdim=rd, inverse=True)
            lat = K.gemm(o.view(B, nh * hd), lw.wo_a, x_group_koff=cfg.group_in, out_group_coff=cfg.o_lora_rank)
            a = K.gemm(aq(lat), lw.wo_b)
            state = K4.hc_post(a, state, coeff)
            # ---- MoE ----
            if prof is not None:
                prof.mark(i, "moe")
            x, coeff = K4.hc_pre(state, lw.hc_ffn_fn, lw.hc_ffn_scale, lw.hc_ffn_base, cfg.hc)
            xn = self._norm(x, lw.ffn_norm)
            f = self._moe(lw, xn, tok_t, B)
            state = K4.hc_post(f, state, coeff)
            if self.proposal is not None and i in cfg.proposal_target_layers:
                K4.hc_mean_scatter(state, taps, cfg.proposal_target_layers.index(i))      # mean over the copies
        if self.proposal is not None:
            main_x = self.proposal.main_rows(taps)
            for s_, plane in enumerate(self.pctx):
                plane[seq_t, pos_t.long()] = self.proposal.context_kv(s_, main_x, pos_t).to(plane.dtype)
        if prof is not None:
            prof.mark(cfg.n_layers, "head")
        for s, p in last.items():
            self.positions[s] = p + 1
        if want_rows is not None:
            if not want_rows:
                return None, None
            if len(want_rows) != B:
                state = state[torch.tensor(want_rows, dtype=torch.int64, device=dev)].contiguous()
        h, _ = K4.hc_pre(state, w.hc_head_fn, w.hc_head_scale, w.hc_head_base, cfg.hc, head_only=True)
        hn = self._norm(h, w.final_norm)
        logits = K.gemm(hn, w.lm_head, out_dtype=torch.float32)
        nxt = K.argmax(logits)
        if prof is not None:
            prof.mark(cfg.n_layers, None)
        return nxt, logits

    def _moe(self, lw: V4LayerWeights, xn: torch.Tensor, tok_t: torch.Tensor, B: int) -> torch.Tensor:
        K, cfg = self.K, self.cfg
        k, H, E = cfg.topk, cfg.hidden, cfg.n_routed_experts
        logits = K.gemm(xn, lw.router_w, out_dtype=torch.float32)
        idx = torch.empty(B, k, dtype=torch.int32, device=self.device)
        wts = torch.empty(B, k, dtype=torch.float32, device=self.device)
        K.router_topk(logits, k, SCORE_SQRT_SOFTPLUS, bias=lw.router_bias, normalize=True, route_scale=cfg.route_scale,
                      hash_table=lw.hash_table, token_ids=tok_t, out_idx=idx, out_w=wts)
        slots = k + 1
        plan = self.plan
        K.moe_plan(idx, wts, plan, 0, E, dst_slots=slots)
        xg = torch.empty(B * k, H, dtype=torch.bfloat16, device=self.device)
        K.gather_rows(xn, plan, xg, cap_rows=B * k)
        hmid = K.gemm(xg, lw.e_w13, epilogue=K.EPI_SWIGLU, plan=plan, act_limit=cfg.swiglu_limit)
        route_out = torch.zeros(B, slots, H, dtype=torch.bfloat16, device=self.device)
        K.gemm(hmid, lw.e_w2, out=route_out.view(B * slots, H), epilogue=K.EPI_SCATTER, plan=plan, scatter_rows=B * slots)
        aq = v4.qat_linear_input if cfg.qat else (lambda t: t)
        mid = K.gemm(aq(xn), lw.w13, epilogue=K.EPI_SWIGLU, act_limit=cfg.swiglu_limit)
        K.gemm(aq(mid), lw.w2, out=route_out[:, k])
        return K.moe_reduce(route_out.view(B * slots, H), slots, k, idx, 0, E, B, H)
