"""Device-resident weight image of a DeepSeek-family model, laid out for the kernels.

Weights are re-packed once at load time into the shapes the tcgen05 GEMM consumes
(K-major bf16 `[groups, out, in]`):

  w_qkv_a   [q_or_qlora + kv_lora + rope, hidden]   q (or q_a) and kv_a fused: one GEMM per token
  w_q_b     [heads_local * q_head_dim, q_lora]      only with a q low-rank projection
  w_uk_t    [heads_local, kv_lora, nope]            absorbed key up-projection (transposed)
  w_uv      [heads_local, v_head, kv_lora]          absorbed value up-projection
  w_o       [hidden, heads_local * v_head]
  w13/w2    dense or shared FFN: [1, 2*inter_local, hidden] / [1, hidden, inter_local]
  e_w13/e_w2 routed experts of this rank: [E_local, 2*I, hidden] / [E_local, hidden, I]

Tensor parallelism shards heads, FFN inner dims and the vocabulary; routed experts are
sharded by expert id (activations are replicated between the collectives, so expert
parallelism needs no token dispatch).  The static-weight "execution image" role matches
crates/ferrule-model/src/models/deepseek_v4/cuda_cache.rs:2905-3160; tensor naming for
checkpoints follows the HuggingFace DeepSeek layout (see `families.py`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
import os
from typing import List, Optional, Sequence, Tuple

import torch

from .config import ModelConfig


class QuantWeight:
    """A quantised linear weight `[groups, out, in]`.

    group32 = False: FP8 e4m3 codes `q` with one UE8M0 scale per 128 x 128 block,
    `scale [groups, ceil(out/128), ceil(in/128)]` (the DeepSeek-V3 checkpoint format).
    group32 = True: MXFP4, one UE8M0 scale per row per 32 inputs, `scale [groups, out, in/32]`, in one of two
    forms.  Native (`packed` set): two e2m1 values per byte, `packed [groups, out, in/2]` (the checkpoint's own
    layout, half a byte per weight) plus `sf`, the scales re-arranged for the block-scaled tensor-core GEMM.
    Container (`q` set): the e2m1 values expanded to e4m3 codes (every e2m1 value is exactly representable) for
    the group-scaled FP8 GEMM; this is the form used where the native library is absent (CPU).
    """
    __slots__ = ("q", "scale", "group32", "packed", "sf")

    def __init__(self, q: Optional[torch.Tensor], scale: torch.Tensor, group32: bool = False,
                 packed: Optional[torch.Tensor] = None, sf: Optional[torch.Tensor] = None):
        self.q, self.scale, self.group32, self.packed, self.sf = q, scale, group32, packed, sf

    @property
    def native_mxfp4(self) -> bool:
        return self.packed is not None

    @property
    def native_mx(self) -> bool:
        """Held in a form the block-scaled tensor-core GEMM takes: packed MXFP4, or e4m3 codes whose 128 x 128
        block scales have been replicated into the per-32 scale layout (`sf`)."""
        return self.sf is not None

    def attach_block_sf_(self) -> "QuantWeight":
        """FP8 128 x 128 weights on a GPU: add `sf` so that the GEMM runs on the block-scaled MMA (scales applied by
        the tensor core) instead of rescaling every k-block in the epilogue.  No-op where it does not apply."""
        if (self.sf is None and self.packed is None and not self.group32 and self.q is not None and self.q.is_cuda
                and self.q.shape[-1] % 128 == 0 and os.environ.get("FERRULE_FP8_NATIVE_MX", "1") != "0"):
            from ..ops import quant as Q
            self.sf = Q.fp8_block_sf(self.scale, self.q.shape[-2], self.q.shape[-1])
            if self.q.dim() == 2:
                self.sf = self.sf[0]
        return self

    @property
    def shape(self):
        if self.packed is not None:
            return torch.Size(list(self.packed.shape[:-1]) + [self.packed.shape[-1] * 2])
        return self.q.shape

    def nbytes(self) -> int:
        n = self.scale.numel()
        for t in (self.q, self.packed, self.sf):
            if t is not None:
                n += t.numel()
        return n

    def dequant(self) -> torch.Tensor:
        """bf16 tensor with exactly the values the quantised GEMM multiplies by."""
        from ..io import encoding as enc
        codes = self.packed if self.packed is not None else self.q
        two_d = codes.dim() == 2
        codes, scale = (codes.unsqueeze(0), self.scale.unsqueeze(0)) if two_d else (codes, self.scale)
        v = enc.fp4_unpack(codes).float() if self.packed is not None else enc.e4m3_decode(codes)
        G, O, I = v.shape
        sc = enc.e8m0_decode(scale)
        if self.group32:
            out = (v.view(G, O, I // 32, 32) * sc.unsqueeze(-1)).view(G, O, I)
        else:
            out = v * sc.repeat_interleave(128, 1)[:, :O].repeat_interleave(128, 2)[:, :, :I]
        out = out.to(torch.bfloat16)
        return out[0] if two_d else out

    @staticmethod
    def from_bf16(w: torch.Tensor, fmt: str) -> "QuantWeight":
        """fmt 'fp8_block' or 'mxfp4'; w [groups, out, in] (or [out, in])."""
        from ..io import encoding as enc
        two_d = w.dim() == 2
        if two_d:
            w = w.unsqueeze(0)
        if fmt == "mxfp4" and w.is_cuda and w.shape[-1] % 128 == 0:
            # native form, quantised and laid out on the device
            from ..ops import quant as Q
            G, O, I = w.shape
            packed, sb = Q.quant_mxfp4_rows(w.reshape(G * O, I).contiguous().to(torch.bfloat16))
            packed, sb = packed.view(G, O, I // 2), sb.view(G, O, I // 32)
            sf = Q.mxfp4_prepare_sf(sb)
            if two_d:
                return QuantWeight(None, sb[0], True, packed[0], sf[0])
            return QuantWeight(None, sb, True, packed, sf)
        qs, ss = [], []
        for g in range(w.shape[0]):
            if fmt == "fp8_block":
                q, sb = enc.weight_quant_fp8_block(w[g])
            elif fmt == "mxfp4":
                # quantise in row chunks: the nearest-code search expands every element eightfold
                parts = [enc.weight_quant_mxfp4(w[g][r:r + 1024]) for r in range(0, w.shape[1], 1024)]
                packed, sb = torch.cat([a for a, _ in parts]), torch.cat([b for _, b in parts])
                q = enc.e4m3_encode(enc.fp4_unpack(packed))
            else:
                raise ValueError(f"unknown weight format {fmt}")
            qs.append(q)
            ss.append(sb)
        q, sc = torch.stack(qs).contiguous(), torch.stack(ss).contiguous()
        out = QuantWeight(q[0] if two_d else q, sc[0] if two_d else sc, fmt == "mxfp4")
        return out.attach_block_sf_() if fmt == "fp8_block" else out


WEIGHT_FORMATS = ("bf16", "fp8_block", "fp8_mxfp4")
_DENSE_FIELDS = ("w_qkv_a", "w_q_b", "w_o", "w13", "w2")
_EXPERT_FIELDS = ("e_w13", "e_w2")


def quantize_layer_(lw: "LayerWeights", fmt: str) -> "LayerWeights":
    """In place: dense / attention projections -> FP8 128 x 128 blocks; routed experts -> FP8 blocks
    ('fp8_block') or MXFP4 ('fp8_mxfp4').  Norms, router, absorbed W_UK / W_UV stay bf16."""
    if fmt == "bf16":
        return lw
    assert fmt in WEIGHT_FORMATS
    def fits(name: str, t: torch.Tensor) -> bool:
        # 1 x 128 activation blocks need in % 128 == 0; the SwiGLU pair splits at a 128-row boundary
        out_dim, in_dim = t.shape[-2], t.shape[-1]
        return in_dim % 128 == 0 and (name not in ("w13", "e_w13") or (out_dim // 2) % 128 == 0)

    ffn_ok = all(fits(n, getattr(lw, n)) for n in ("w13", "w2") if isinstance(getattr(lw, n), torch.Tensor))
    for name in _DENSE_FIELDS:
        t = getattr(lw, name)
        if isinstance(t, torch.Tensor) and fits(name, t) and (ffn_ok or name not in ("w13", "w2")):
            setattr(lw, name, QuantWeight.from_bf16(t, "fp8_block"))
    experts_ok = all(fits(n, getattr(lw, n)) for n in _EXPERT_FIELDS if isinstance(getattr(lw, n), torch.Tensor))
    for name in _EXPERT_FIELDS:
        t = getattr(lw, name)
        if isinstance(t, torch.Tensor) and experts_ok:
            setattr(lw, name, QuantWeight.from_bf16(t, "mxfp4" if fmt == "fp8_mxfp4" else "fp8_block"))
    return lw


def dequantized_copy(w: "ModelWeights") -> "ModelWeights":
    """bf16 model holding the values a quantised model computes with (oracle for parity tests)."""
    import copy

    def layer(lw):
        c = copy.copy(lw)
        for name in _DENSE_FIELDS + _EXPERT_FIELDS:
            t = getattr(c, name)
            if isinstance(t, QuantWeight):
                d = t.dequant()
                setattr(c, name, d)
        return c

    out = copy.copy(w)
    out.layers = [layer(l) for l in w.layers]
    out.mtp = []
    for m in w.mtp:
        mc = copy.copy(m)
        mc.layer = layer(m.layer)
        out.mtp.append(mc)
    out.weight_format = "bf16"
    out.act_quant = w.weight_format != "bf16"
    # weights that run on the block-scaled tensor-core GEMM multiply MXFP8 activations (1 x 32 scale blocks)
    def native(names):
        return any(isinstance(getattr(l, n), QuantWeight) and getattr(l, n).native_mx for l in w.layers for n in names)
    out.expert_act_block = 32 if native(_EXPERT_FIELDS) else 128
    out.dense_act_block = 32 if native(_DENSE_FIELDS) else 128
    return out


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    w_qkv_a: torch.Tensor
    q_norm: Optional[torch.Tensor]
    w_q_b: Optional[torch.Tensor]
    kv_norm: torch.Tensor
    w_uk_t: torch.Tensor
    w_uv: torch.Tensor
    w_o: torch.Tensor
    ffn_norm: torch.Tensor
    # dense FFN or shared experts (None if absent)
    w13: Optional[torch.Tensor] = None
    w2: Optional[torch.Tensor] = None
    # routed MoE
    router_w: Optional[torch.Tensor] = None
    router_bias: Optional[torch.Tensor] = None
    hash_table: Optional[torch.Tensor] = None
    e_w13: Optional[torch.Tensor] = None
    e_w2: Optional[torch.Tensor] = None
    attn_sink: Optional[torch.Tensor] = None
    is_moe: bool = False


@dataclass
class MtpWeights:
    """One multi-token-prediction stage: norms + projection over [embedding ; hidden] + a layer body.

    `eh_proj` columns follow published DeepSeek-V3 checkpoints (and vLLM / SGLang, which compute
    `eh_proj(cat([enorm(embed), hnorm(hidden)]))`): the first `hidden` columns multiply the normalised
    embedding of the next token, the last `hidden` columns the normalised hidden state.  `embed` / `lm_head`
    are the stage's own `embed_tokens` / `shared_head.head` when a checkpoint stores ones that differ from
    the main model's (None: shared with the main model, as in the published checkpoints)."""
    enorm: torch.Tensor
    hnorm: torch.Tensor
    eh_proj: torch.Tensor         # [hidden, 2*hidden], columns [embedding | hidden]
    layer: LayerWeights
    final_norm: torch.Tensor
    embed: Optional[torch.Tensor] = None
    lm_head: Optional[torch.Tensor] = None


@dataclass
class ModelWeights:
    cfg: ModelConfig
    embed: torch.Tensor           # [vocab, hidden] (replicated)
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor         # [vocab_local, hidden]
    mtp: List[MtpWeights] = field(default_factory=list)
    tp_rank: int = 0
    tp_world: int = 1
    e_lo: int = 0
    e_hi: int = 0
    vocab_lo: int = 0
    weight_format: str = "bf16"
    act_quant: bool = False       # oracle only: emulate the 1 x 128 FP8 activation quantisation of the FP8 path
    expert_act_block: int = 128   # oracle only: scale-block width of the routed experts' activation quantisation
    shared_replicated: bool = False   # shared experts hold their full inner dimension on every rank (token-dispatch EP)

    @property
    def heads_local(self) -> int:
        return self.cfg.n_heads // self.tp_world

    def nbytes(self) -> int:
        total = 0
        seen = set()

        def add(t):
            nonlocal total
            if isinstance(t, QuantWeight):
                for part in (t.q, t.scale, t.packed, t.sf):
                    add(part)
            elif isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()

        for t in (self.embed, self.final_norm, self.lm_head):
            add(t)
        for lw in list(self.layers) + [m.layer for m in self.mtp]:
            for v in vars(lw).values():
                add(v)
        for m in self.mtp:
            for t in (m.enorm, m.hnorm, m.eh_proj, m.final_norm):
                add(t)
        return total


def _shard_range(n: int, rank: int, world: int):
    assert n % world == 0, f"{n} not divisible by {world}"
    per = n // world
    return rank * per, (rank + 1) * per


class _Init:
    """Deterministic N(0, std) initialiser that produces identical full tensors on every rank
    (generated on CPU from a per-tensor seed) so sharded replicas agree with a single-GPU run."""

    def __init__(self, seed: int, std: float, device, dtype, on_device: bool):
        self.seed, self.std, self.device, self.dtype, self.on_device = seed, std, device, dtype, on_device
        self.counter = 0

    def normal(self, *shape) -> torch.Tensor:
        self.counter += 1
        if self.on_device and torch.device(self.device).type == "cuda":
            g = torch.Generator(device=self.device).manual_seed(self.seed * 100003 + self.counter)
            t = torch.empty(*shape, device=self.device, dtype=torch.float32)
            t.normal_(0.0, self.std, generator=g)
            return t.to(self.dtype)
        g = torch.Generator().manual_seed(self.seed * 100003 + self.counter)
        return (torch.randn(*shape, generator=g) * self.std).to(self.dtype).to(self.device)

    def ones(self, *shape) -> torch.Tensor:
        return torch.ones(*shape, dtype=self.dtype, device=self.device)


def _layer_random(cfg: ModelConfig, layer: int, init: _Init, tp_rank: int, tp_world: int,
                  force_moe: Optional[bool] = None, replicate_shared: bool = False,
                  expert_order: Optional[Sequence[int]] = None) -> LayerWeights:
    H = cfg.hidden
    h_lo, h_hi = _shard_range(cfg.n_heads, tp_rank, tp_world)
    hl = h_hi - h_lo
    qhd, lora, rope, nope, vd = cfg.q_head_dim, cfg.kv_lora_rank, cfg.qk_rope_dim, cfg.qk_nope_dim, cfg.v_head_dim
    # full tensors are drawn first and sliced, so every TP layout sees the same model
    if cfg.q_lora_rank:
        w_q_a = init.normal(cfg.q_lora_rank, H)
        w_q_b_full = init.normal(cfg.n_heads * qhd, cfg.q_lora_rank)
        q_norm = init.ones(cfg.q_lora_rank)
        w_q_b = w_q_b_full[h_lo * qhd:h_hi * qhd].contiguous()
        q_part = w_q_a
    else:
        w_q_full = init.normal(cfg.n_heads * qhd, H)
        q_part = w_q_full[h_lo * qhd:h_hi * qhd]
        q_norm, w_q_b = None, None
    w_kv_a = init.normal(lora + rope, H)
    w_qkv_a = torch.cat([q_part, w_kv_a], dim=0).contiguous()
    w_kv_b = init.normal(cfg.n_heads, nope + vd, lora)[h_lo:h_hi]
    w_uk_t = w_kv_b[:, :nope, :].transpose(1, 2).contiguous()      # [hl, lora, nope]
    w_uv = w_kv_b[:, nope:, :].contiguous()                         # [hl, vd, lora]
    w_o = init.normal(H, cfg.n_heads * vd)[:, h_lo * vd:h_hi * vd].contiguous()
    lw = LayerWeights(attn_norm=init.ones(H), w_qkv_a=w_qkv_a, q_norm=q_norm, w_q_b=w_q_b,
                      kv_norm=init.ones(lora), w_uk_t=w_uk_t, w_uv=w_uv, w_o=w_o, ffn_norm=init.ones(H))
    if cfg.attn_sink:
        lw.attn_sink = init.normal(cfg.n_heads).float()[h_lo:h_hi].contiguous()
    is_moe = cfg.is_moe_layer(layer) if force_moe is None else force_moe
    lw.is_moe = is_moe

    def ffn(inter: int, replicated: bool = False):
        i_lo, i_hi = (0, inter) if replicated else _shard_range(inter, tp_rank, tp_world)
        gate, up, down = init.normal(inter, H), init.normal(inter, H), init.normal(H, inter)
        w13 = torch.cat([gate[i_lo:i_hi], up[i_lo:i_hi]], dim=0).unsqueeze(0).contiguous()
        w2 = down[:, i_lo:i_hi].unsqueeze(0).contiguous()
        return w13, w2

    if not is_moe:
        lw.w13, lw.w2 = ffn(cfg.dense_inter)
        return lw
    E, I = cfg.n_routed_experts, cfg.moe_inter
    lw.router_w = init.normal(E, H)
    if cfg.router_bias:
        lw.router_bias = init.normal(E).float()
    if layer < cfg.n_dense_layers + cfg.n_hash_layers and cfg.n_hash_layers:
        g = torch.Generator().manual_seed(init.seed + 7919 * (layer + 1))
        lw.hash_table = torch.randint(0, E, (cfg.vocab_size, cfg.topk), generator=g).to(init.device)
    e_lo, e_hi = _shard_range(E, tp_rank, tp_world)
    # experts are drawn one by one so only the local ones are ever materialised.  `expert_order` (a placement plan,
    # parallel/placement.py): physical id j holds original expert order[j] - the router rows, the bias and the
    # hash table are renumbered, and each expert keeps the draws of its original id
    order = list(range(E)) if expert_order is None else list(expert_order)
    if expert_order is not None:
        if sorted(order) != list(range(E)):
            raise ValueError("expert_order is not a permutation of the layer's experts")
        idx = torch.tensor(order, dtype=torch.int64, device=lw.router_w.device)
        lw.router_w = lw.router_w[idx].contiguous()
        if lw.router_bias is not None:
            lw.router_bias = lw.router_bias[idx].contiguous()
        if lw.hash_table is not None:
            inv = torch.empty(E, dtype=torch.int64, device=lw.hash_table.device)
            inv[idx.to(lw.hash_table.device)] = torch.arange(E, device=lw.hash_table.device)
            lw.hash_table = inv[lw.hash_table.long()]
    w13s, w2s = [], []
    base = init.counter
    for j in range(e_lo, e_hi):
        init.counter = base + 3 * order[j]
        gate, up, down = init.normal(I, H), init.normal(I, H), init.normal(H, I)
        w13s.append(torch.cat([gate, up], dim=0))
        w2s.append(down)
    init.counter = base + 3 * E
    lw.e_w13 = torch.stack(w13s).contiguous()
    lw.e_w2 = torch.stack(w2s).contiguous()
    if cfg.n_shared_experts:
        # token-dispatch expert parallelism runs the shared experts on each rank's own token slice: full weights
        lw.w13, lw.w2 = ffn(cfg.n_shared_experts * I, replicated=replicate_shared)
    return lw


def random_weights(cfg: ModelConfig, device="cpu", dtype=torch.bfloat16, seed: int = 0, std: float = 0.02,
                   tp_rank: int = 0, tp_world: int = 1, fast_device_init: bool = False,
                   weight_format: str = "bf16", replicate_shared: bool = False,
                   layer_range: Optional[Tuple[int, int]] = None, router_zipf: float = 0.0,
                   expert_orders: Optional[dict] = None) -> ModelWeights:
    """Random-init weights N(0, std), norms = 1.

    fast_device_init draws on the GPU (much faster for multi-GB models; values then differ
    between TP layouts, which is fine for throughput runs but not for parity tests).
    router_zipf s > 0: skewed expert popularity for residency / streaming runs - router rows are scaled so that
    logits over normalised activations are N(0, 1), and every MoE layer gets a selection bias that follows a
    Zipf(s) popularity over a fixed random order of its experts (see `zipf_router_bias`).
    layer_range (lo, hi): build only these layers (a pipeline stage of a model whose whole image does not fit one
    GPU); the other entries of `layers` are None and the draws differ from the full image's, so it needs
    fast_device_init.
    expert_orders {layer: order}: a placement plan (`parallel.placement.plan_expert_placement`): the layer's experts
    are renumbered so that physical id j is original expert order[j] - the same function, other owners.
    """
    orders = expert_orders or {}
    if layer_range is not None and not fast_device_init:
        raise ValueError("layer_range skips draws: use it with fast_device_init only")
    init = _Init(seed, std, device, dtype, fast_device_init)
    embed = init.normal(cfg.vocab_size, cfg.hidden)
    lo_l, hi_l = layer_range if layer_range is not None else (0, cfg.n_layers)
    # quantise layer by layer so that at most one layer exists in bf16 at a time
    layers = [quantize_layer_(_layer_random(cfg, i, init, tp_rank, tp_world, replicate_shared=replicate_shared,
                                            expert_order=orders.get(i)),
                              weight_format) if lo_l <= i < hi_l else None for i in range(cfg.n_layers)]
    v_lo, v_hi = _shard_range(cfg.vocab_size, tp_rank, tp_world)
    lm_head = init.normal(cfg.vocab_size, cfg.hidden)[v_lo:v_hi].contiguous()
    mtp = []
    for m in range(cfg.n_mtp_layers if layer_range is None else 0):
        mtp.append(MtpWeights(enorm=init.ones(cfg.hidden), hnorm=init.ones(cfg.hidden),
                              eh_proj=init.normal(cfg.hidden, 2 * cfg.hidden),
                              layer=quantize_layer_(_layer_random(cfg, cfg.n_layers + m, init, tp_rank, tp_world,
                                                                  force_moe=cfg.n_routed_experts > 0,
                                                                  replicate_shared=replicate_shared),
                                                    weight_format),
                              final_norm=init.ones(cfg.hidden)))
    e_lo, e_hi = _shard_range(cfg.n_routed_experts, tp_rank, tp_world) if cfg.n_routed_experts else (0, 0)
    w = ModelWeights(cfg, embed, layers, init.ones(cfg.hidden), lm_head, mtp, tp_rank, tp_world,
                     e_lo, e_hi, v_lo, weight_format=weight_format)
    w.shared_replicated = bool(replicate_shared and tp_world > 1)
    if router_zipf > 0:
        for i, lw in enumerate(w.layers):
            if lw is not None and lw.is_moe and lw.router_w is not None:
                lw.router_w = (lw.router_w.float() * (1.0 / (std * cfg.hidden ** 0.5))).to(lw.router_w.dtype)
                bias = zipf_router_bias(cfg.n_routed_experts, router_zipf, seed * 7919 + i, sigmoid=cfg.score_fn != 0)
                if i in orders:
                    bias = bias[torch.tensor(list(orders[i]), dtype=torch.int64)]     # popularity follows the expert
                lw.router_bias = bias.to(lw.router_w.device)
    return w


def zipf_router_bias(n_experts: int, s: float, seed: int, sigmoid: bool = True) -> torch.Tensor:
    """Selection bias that makes expert popularity follow Zipf(s): popularity p_r ~ r^-s over a fixed random order of
    the experts, bias = log p (centred).  Routers that pick on sigmoid scores in (0, 1) get the bias scaled into
    [-0.5, 0.5], so that the skew shapes the choice without fixing it; softmax-style routers add it to the logits'
    scale directly."""
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_experts, generator=g)
    logp = -s * torch.log(torch.arange(1, n_experts + 1, dtype=torch.float32))
    logp = logp - logp.mean()
    if sigmoid:
        logp = 0.5 * logp / logp.abs().max()
    bias = torch.empty(n_experts, dtype=torch.float32)
    bias[order] = logp
    return bias
