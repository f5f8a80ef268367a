"""DeepSeek-V4 checkpoint directories: load into `V4Weights`, and write one from a weight image.

Layout (HuggingFace DeepSeek-V4): `config.json` + safetensors shards.  Attention and shared-expert linears are
`<base>.weight` F8_E4M3 with `<base>.scale` F8_E8M0 (one scale per 128 x 128 block); routed experts are one
`w1` / `w3` / `w2` triple per expert, `.weight` I8 holding two e2m1 values per byte with `.scale` F8_E8M0 per 32
inputs; norms are BF16, hyper-connection parameters, router bias and attention sinks F32, the hash-routing table
`tid2eid` I64.  Compressor and indexer tensors (plain BF16 / F32) exist on the layers whose compression ratio is
non-zero.  The loader decodes every linear to the dense bf16 tensor the model multiplies with
(`io/checkpoint.py:read_linear` picks the decoder from the stored dtypes, so plain BF16 checkpoints load too);
the writer quantises the same way a published checkpoint is quantised, so `load(write(w))` returns exactly the
values of the format's round trip.

Counterpart of crates/ferrule-model/src/models/deepseek_v4/checkpoint.rs:48 (open + bind),
checkpoint_binding.rs:31-700 (names and shapes); the tensor catalogue of the synthetic fixture is
scripts/dsv4_synthetic_fixture.py:109-269.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Optional

import torch

from ..models.v4_model import V4Config, V4LayerWeights, V4ProposalWeights, V4Weights
from .checkpoint import _put_linear, read_linear
from .safetensors import CheckpointError, ShardedCheckpoint, fails_closed, write_sharded


def v4_config_from_hf(hf: dict) -> V4Config:
    """config.json of a DeepSeek-V4 checkpoint -> V4Config (absent keys keep the family defaults)."""
    d = V4Config()
    n_layers = int(hf.get("num_hidden_layers", d.n_layers))
    ratios = hf.get("compress_ratios")
    if ratios is None:
        ratios = [0 if i == 0 else (4 if i % 2 else 128) for i in range(n_layers)]
    rope = hf.get("rope_scaling") or {}
    return V4Config(
        hidden=int(hf.get("hidden_size", d.hidden)), hc_mult=int(hf.get("hc_mult", d.hc_mult)),
        hc_sinkhorn_iters=int(hf.get("hc_sinkhorn_iters", d.hc_sinkhorn_iters)), hc_eps=float(hf.get("hc_eps", d.hc_eps)),
        norm_eps=float(hf.get("rms_norm_eps", d.norm_eps)), n_layers=n_layers,
        n_hash_layers=int(hf.get("num_hash_layers", d.n_hash_layers)), n_heads=int(hf.get("num_attention_heads", d.n_heads)),
        head_dim=int(hf.get("head_dim", d.head_dim)), q_lora_rank=int(hf.get("q_lora_rank", d.q_lora_rank)),
        rope_dim=int(hf.get("qk_rope_head_dim", d.rope_dim)), o_groups=int(hf.get("o_groups", d.o_groups)),
        o_lora_rank=int(hf.get("o_lora_rank", d.o_lora_rank)), window=int(hf.get("sliding_window", d.window)),
        vocab_size=int(hf.get("vocab_size", d.vocab_size)), n_routed_experts=int(hf.get("n_routed_experts", d.n_routed_experts)),
        topk=int(hf.get("num_experts_per_tok", d.topk)), moe_inter=int(hf.get("moe_intermediate_size", d.moe_inter)),
        n_shared_experts=int(hf.get("n_shared_experts", d.n_shared_experts)),
        swiglu_limit=float(hf.get("swiglu_limit", d.swiglu_limit)), route_scale=float(hf.get("routed_scaling_factor", d.route_scale)),
        rope_theta=float(hf.get("rope_theta", d.rope_theta)),
        compress_rope_theta=float(hf.get("compress_rope_theta", d.compress_rope_theta)),
        rope_factor=float(rope.get("factor", hf.get("rope_factor", d.rope_factor))),
        rope_orig_max_pos=int(rope.get("original_max_position_embeddings", hf.get("rope_orig_max_pos", d.rope_orig_max_pos))),
        index_n_heads=int(hf.get("index_n_heads", d.index_n_heads)), index_head_dim=int(hf.get("index_head_dim", d.index_head_dim)),
        index_topk=int(hf.get("index_topk", d.index_topk)), compress_ratios=tuple(int(r) for r in ratios),
        indexer_ratio=int(hf.get("indexer_ratio", d.indexer_ratio)),
        proposal_block_size=int(hf.get("proposal_block_size", d.proposal_block_size)),
        max_position=int(hf.get("max_position_embeddings", d.max_position)),
        n_proposal_stages=int(hf.get("num_nextn_predict_layers", 0)),
        proposal_target_layers=tuple(int(i) for i in hf.get("proposal_target_layer_ids", ())),
        proposal_noise_token=int(hf.get("proposal_noise_token_id", d.proposal_noise_token)),
        proposal_markov_rank=int(hf.get("proposal_markov_rank", d.proposal_markov_rank)),
        # published checkpoints were trained with the quantisation steps in the forward pass and say so through
        # their quantization_config; directories written here carry the flag itself
        qat=bool(hf["qat"]) if "qat" in hf else hf.get("quantization_config") is not None)


def v4_config_to_hf(cfg: V4Config) -> dict:
    return {
        "model_type": "deepseek_v4", "architectures": ["DeepseekV4ForCausalLM"],
        "hidden_size": cfg.hidden, "hc_mult": cfg.hc_mult, "hc_sinkhorn_iters": cfg.hc_sinkhorn_iters, "hc_eps": cfg.hc_eps,
        "rms_norm_eps": cfg.norm_eps, "num_hidden_layers": cfg.n_layers, "num_hash_layers": cfg.n_hash_layers,
        "num_attention_heads": cfg.n_heads, "head_dim": cfg.head_dim, "q_lora_rank": cfg.q_lora_rank,
        "qk_rope_head_dim": cfg.rope_dim, "o_groups": cfg.o_groups, "o_lora_rank": cfg.o_lora_rank,
        "sliding_window": cfg.window, "vocab_size": cfg.vocab_size, "n_routed_experts": cfg.n_routed_experts,
        "num_experts_per_tok": cfg.topk, "moe_intermediate_size": cfg.moe_inter, "n_shared_experts": cfg.n_shared_experts,
        "swiglu_limit": cfg.swiglu_limit, "routed_scaling_factor": cfg.route_scale, "rope_theta": cfg.rope_theta,
        "compress_rope_theta": cfg.compress_rope_theta,
        "rope_scaling": {"factor": cfg.rope_factor, "original_max_position_embeddings": cfg.rope_orig_max_pos},
        "index_n_heads": cfg.index_n_heads, "index_head_dim": cfg.index_head_dim, "index_topk": cfg.index_topk,
        "compress_ratios": list(cfg.compress_ratios), "indexer_ratio": cfg.indexer_ratio,
        "proposal_block_size": cfg.proposal_block_size, "max_position_embeddings": cfg.max_position,
        "num_nextn_predict_layers": cfg.n_proposal_stages, "proposal_target_layer_ids": list(cfg.proposal_target_layers),
        "proposal_noise_token_id": cfg.proposal_noise_token, "proposal_markov_rank": cfg.proposal_markov_rank,
        "scoring_func": "sqrtsoftplus", "qat": cfg.qat,
    }


def _lin(ck: ShardedCheckpoint, base: str, dev, rows: Optional[int] = None, cols: Optional[int] = None) -> torch.Tensor:
    w = read_linear(ck, base, torch.bfloat16)
    if (rows is not None and w.shape[0] != rows) or (cols is not None and w.shape[1] != cols):
        raise CheckpointError(f"{base}: shape {tuple(w.shape)} where [{rows}, {cols}] is bound")
    return w.to(dev)


def _raw(ck: ShardedCheckpoint, name: str, dev, dtype=None) -> torch.Tensor:
    t = ck.read(name)
    return (t.to(dtype) if dtype is not None else t).to(dev)


@fails_closed
def load_v4_hf(directory, device="cpu", max_layers: int = 0) -> V4Weights:
    """Bind a DeepSeek-V4 checkpoint directory: every linear decoded to bf16, experts stacked per layer
    ([E, 2 * inter, hidden] gate over up, [E, hidden, inter]), the output projection's first stage regrouped to
    [o_groups, o_lora, group_in]."""
    d = Path(directory)
    cfg = v4_config_from_hf(json.loads((d / "config.json").read_text()))
    if 0 < max_layers < cfg.n_layers:
        # a smoke run over the first layers of a large checkpoint: the proposal attachment taps layers that may
        # not be bound then, so it is left out
        cfg = cfg.with_(n_layers=max_layers, compress_ratios=tuple(cfg.compress_ratios[:max_layers]),
                        n_hash_layers=min(cfg.n_hash_layers, max_layers), n_proposal_stages=0, proposal_target_layers=())
    ck = ShardedCheckpoint(d)
    H, hd, E, I = cfg.hidden, cfg.head_dim, cfg.n_routed_experts, cfg.moe_inter
    bf, f32 = torch.bfloat16, torch.float32
    def layer(p: str, i: int, r: int, indexer: bool, hashed: bool) -> V4LayerWeights:
        """One transformer body under prefix `p` (`layers.{i}.` of the target, `mtp.{i}.` of the proposal)."""
        a = p + "attn."
        wo_a = _lin(ck, a + "wo_a", device, cfg.o_groups * cfg.o_lora_rank, cfg.group_in)
        sh = p + "ffn.shared_experts."
        sI = cfg.n_shared_experts * I
        w13 = torch.cat([_lin(ck, sh + "w1", device, sI, H), _lin(ck, sh + "w3", device, sI, H)], 0).unsqueeze(0)
        e13, e2 = [], []
        for e in range(E):
            ep = f"{p}ffn.experts.{e}."
            e13.append(torch.cat([_lin(ck, ep + "w1", device, I, H), _lin(ck, ep + "w3", device, I, H)], 0))
            e2.append(_lin(ck, ep + "w2", device, H, I))
        lw = V4LayerWeights(
            hc_attn_fn=_raw(ck, p + "hc_attn_fn", device, f32), hc_attn_scale=_raw(ck, p + "hc_attn_scale", device, f32),
            hc_attn_base=_raw(ck, p + "hc_attn_base", device, f32),
            hc_ffn_fn=_raw(ck, p + "hc_ffn_fn", device, f32), hc_ffn_scale=_raw(ck, p + "hc_ffn_scale", device, f32),
            hc_ffn_base=_raw(ck, p + "hc_ffn_base", device, f32),
            attn_norm=_raw(ck, p + "attn_norm.weight", device, bf),
            wq_a=_lin(ck, a + "wq_a", device, cfg.q_lora_rank, H), q_norm=_raw(ck, a + "q_norm.weight", device, bf),
            wq_b=_lin(ck, a + "wq_b", device, cfg.n_heads * hd, cfg.q_lora_rank),
            wkv=_lin(ck, a + "wkv", device, hd, H), kv_norm=_raw(ck, a + "kv_norm.weight", device, bf),
            sink=_raw(ck, a + "attn_sink", device, f32),
            wo_a=wo_a.view(cfg.o_groups, cfg.o_lora_rank, cfg.group_in).contiguous(),
            wo_b=_lin(ck, a + "wo_b", device, H, cfg.o_groups * cfg.o_lora_rank),
            ffn_norm=_raw(ck, p + "ffn_norm.weight", device, bf), router_w=_raw(ck, p + "ffn.gate.weight", device, bf),
            e_w13=torch.stack(e13), e_w2=torch.stack(e2), w13=w13, w2=_lin(ck, sh + "w2", device, H, sI).unsqueeze(0))
        if ck.has(p + "ffn.gate.tid2eid"):
            lw.hash_table = _raw(ck, p + "ffn.gate.tid2eid", device, torch.int64)
        if ck.has(p + "ffn.gate.bias"):
            lw.router_bias = _raw(ck, p + "ffn.gate.bias", device, f32)
        if (lw.hash_table is None) == hashed:
            raise CheckpointError(f"{p}: hash-routing table {'missing' if lw.hash_table is None else 'unexpected'}")
        c = a + "compressor."
        if r:
            od = hd * (2 if indexer else 1)
            lw.c_wkv, lw.c_wgate = _lin(ck, c + "wkv", device, od, H), _lin(ck, c + "wgate", device, od, H)
            lw.c_ape, lw.c_norm = _raw(ck, c + "ape", device, f32), _raw(ck, c + "norm.weight", device, bf)
        elif ck.has(c + "wkv.weight"):
            raise CheckpointError(f"{p}: compressor tensors on a window-only layer")
        if indexer:
            x = a + "indexer."
            idim = cfg.index_head_dim
            lw.i_wq_b = _lin(ck, x + "wq_b", device, cfg.index_n_heads * idim, cfg.q_lora_rank)
            lw.i_weights = _lin(ck, x + "weights_proj", device, cfg.index_n_heads, H)
            lw.ic_wkv = _lin(ck, x + "compressor.wkv", device, 2 * idim, H)
            lw.ic_wgate = _lin(ck, x + "compressor.wgate", device, 2 * idim, H)
            lw.ic_ape = _raw(ck, x + "compressor.ape", device, f32)
            lw.ic_norm = _raw(ck, x + "compressor.norm.weight", device, bf)
        return lw

    try:
        layers = [layer(f"layers.{i}.", i, cfg.ratio(i), cfg.has_indexer(i), i < cfg.n_hash_layers)
                  for i in range(cfg.n_layers)]
        proposal = None
        if cfg.n_proposal_stages:
            # the `mtp.*` namespace: window-only stages with a learned router; stage 0 owns the projection of the
            # target taps, the last stage the prediction heads
            last = f"mtp.{cfg.n_proposal_stages - 1}."
            taps = len(cfg.proposal_target_layers)
            if not taps:
                raise CheckpointError("proposal stages without proposal_target_layer_ids")
            rank = cfg.proposal_markov_rank
            proposal = V4ProposalWeights(
                stages=[layer(f"mtp.{m}.", m, 0, False, False) for m in range(cfg.n_proposal_stages)],
                main_proj=_lin(ck, "mtp.0.main_proj", device, H, taps * H), main_norm=_raw(ck, "mtp.0.main_norm.weight", device, bf),
                hc_head_fn=_raw(ck, last + "hc_head_fn", device, f32), hc_head_scale=_raw(ck, last + "hc_head_scale", device, f32),
                hc_head_base=_raw(ck, last + "hc_head_base", device, f32), norm=_raw(ck, last + "norm.weight", device, bf),
                markov_w1=_lin(ck, last + "markov_head.markov_w1", device, cfg.vocab_size, rank),
                markov_w2=_lin(ck, last + "markov_head.markov_w2", device, cfg.vocab_size, rank),
                confidence_proj=_lin(ck, last + "confidence_head.proj", device, 1, H + rank))
        return V4Weights(cfg, _raw(ck, "embed.weight", device, bf), layers, _raw(ck, "hc_head_fn", device, f32),
                         _raw(ck, "hc_head_scale", device, f32), _raw(ck, "hc_head_base", device, f32),
                         _raw(ck, "norm.weight", device, bf), _raw(ck, "head.weight", device, bf), proposal)
    finally:
        ck.close()


def export_v4_hf(w: V4Weights, directory, dense_format: str = "fp8_block", expert_format: str = "mxfp4",
                 shard_bytes: int = 1 << 30) -> None:
    """Write `w` as a DeepSeek-V4 checkpoint directory.  dense_format 'fp8_block' | 'plain' for attention and
    shared-expert linears, expert_format 'mxfp4' | 'fp8_block' | 'plain' for the routed experts; a linear whose
    input width does not divide the format's block (128 / 32) is written plain."""
    cfg = w.cfg
    out: Dict[str, torch.Tensor] = {}
    names: Dict[str, str] = {}

    def put(base: str, t: torch.Tensor, fmt: str) -> None:
        blk = {"fp8_block": 128, "mxfp4": 32}.get(fmt, 1)
        _put_linear(out, names, base, t, fmt if t.shape[-1] % blk == 0 else "plain")

    out["embed.weight"], out["norm.weight"], out["head.weight"] = w.embed.cpu(), w.final_norm.cpu(), w.lm_head.cpu()
    out["hc_head_fn"], out["hc_head_scale"], out["hc_head_base"] = (w.hc_head_fn.float().cpu(), w.hc_head_scale.float().cpu(),
                                                                  w.hc_head_base.float().cpu())
    I = cfg.moe_inter

    def layer(p: str, lw: V4LayerWeights) -> None:
        a = p + "attn."
        for k in ("hc_attn_fn", "hc_attn_scale", "hc_attn_base", "hc_ffn_fn", "hc_ffn_scale", "hc_ffn_base"):
            out[p + k] = getattr(lw, k).float().cpu()
        out[p + "attn_norm.weight"], out[p + "ffn_norm.weight"] = lw.attn_norm.cpu(), lw.ffn_norm.cpu()
        out[a + "q_norm.weight"], out[a + "kv_norm.weight"] = lw.q_norm.cpu(), lw.kv_norm.cpu()
        out[a + "attn_sink"] = lw.sink.float().cpu()
        put(a + "wq_a", lw.wq_a, dense_format)
        put(a + "wq_b", lw.wq_b, dense_format)
        put(a + "wkv", lw.wkv, dense_format)
        put(a + "wo_a", lw.wo_a.reshape(cfg.o_groups * cfg.o_lora_rank, cfg.group_in), dense_format)
        put(a + "wo_b", lw.wo_b, dense_format)
        out[p + "ffn.gate.weight"] = lw.router_w.cpu()
        if lw.hash_table is not None:
            out[p + "ffn.gate.tid2eid"] = lw.hash_table.to(torch.int64).cpu()
        if lw.router_bias is not None:
            out[p + "ffn.gate.bias"] = lw.router_bias.float().cpu()
        sI = cfg.n_shared_experts * I
        sh = p + "ffn.shared_experts."
        put(sh + "w1", lw.w13[0][:sI], dense_format)
        put(sh + "w3", lw.w13[0][sI:], dense_format)
        put(sh + "w2", lw.w2[0], dense_format)
        for e in range(cfg.n_routed_experts):
            ep = f"{p}ffn.experts.{e}."
            put(ep + "w1", lw.e_w13[e][:I], expert_format)
            put(ep + "w3", lw.e_w13[e][I:], expert_format)
            put(ep + "w2", lw.e_w2[e], expert_format)
        if lw.c_wkv is not None:
            c = a + "compressor."
            out[c + "wkv.weight"], out[c + "wgate.weight"] = lw.c_wkv.cpu(), lw.c_wgate.cpu()
            out[c + "ape"], out[c + "norm.weight"] = lw.c_ape.float().cpu(), lw.c_norm.cpu()
        if lw.i_wq_b is not None:
            x = a + "indexer."
            out[x + "wq_b.weight"], out[x + "weights_proj.weight"] = lw.i_wq_b.cpu(), lw.i_weights.cpu()
            out[x + "compressor.wkv.weight"], out[x + "compressor.wgate.weight"] = lw.ic_wkv.cpu(), lw.ic_wgate.cpu()
            out[x + "compressor.ape"], out[x + "compressor.norm.weight"] = lw.ic_ape.float().cpu(), lw.ic_norm.cpu()

    for i, lw in enumerate(w.layers):
        layer(f"layers.{i}.", lw)
    if w.proposal is not None:
        pw = w.proposal
        for m, lw in enumerate(pw.stages):
            layer(f"mtp.{m}.", lw)
        last = f"mtp.{len(pw.stages) - 1}."
        out["mtp.0.main_proj.weight"], out["mtp.0.main_norm.weight"] = pw.main_proj.cpu(), pw.main_norm.cpu()
        out[last + "hc_head_fn"], out[last + "hc_head_scale"] = pw.hc_head_fn.float().cpu(), pw.hc_head_scale.float().cpu()
        out[last + "hc_head_base"], out[last + "norm.weight"] = pw.hc_head_base.float().cpu(), pw.norm.cpu()
        out[last + "markov_head.markov_w1.weight"] = pw.markov_w1.cpu()
        out[last + "markov_head.markov_w2.weight"] = pw.markov_w2.cpu()
        out[last + "confidence_head.proj.weight"] = pw.confidence_proj.cpu()
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    write_sharded(out, d, shard_bytes, names)
    (d / "config.json").write_text(json.dumps(v4_config_to_hf(cfg), indent=1))
