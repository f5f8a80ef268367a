"""Binding a HuggingFace DeepSeek checkpoint directory to the kernel-ready weight image, and back.

Format inference per linear layer `<base>`:
  * `<base>.weight` BF16/F16/F32                                   -> plain
  * `<base>.weight` F8_E4M3 + 2-D scale (`<base>.weight_scale_inv` F32, or `<base>.scale` F8_E8M0)
                                                                    -> FP8, one scale per 128x128 block
  * `<base>.weight` I8 (two E2M1 values per byte) + E8M0 `<base>.scale` [out, in/g]
                                                                    -> MXFP4 with group g = in / scale_cols (32)
Quantised weights are decoded to bf16 here for the bf16 tcgen05 path; the raw payloads stay
available to the quantised kernels and to expert streaming through `ExpertSourceCatalog`.

Counterpart of crates/ferrule-model/src/checkpoint/weight.rs:229-330 (format inference),
models/deepseek_v4/checkpoint.rs:34-360 and checkpoint_binding.rs:31-700 (tensor binding), and the
tensor catalogue of scripts/dsv4_synthetic_fixture.py:134-269.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch

from ..models.config import ModelConfig, from_hf_config
from ..models.weights import LayerWeights, ModelWeights, MtpWeights, _shard_range
from . import encoding as enc
from .safetensors import CheckpointError, ShardedCheckpoint, write_sharded, fails_closed


def infer_weight_format(ck: ShardedCheckpoint, base: str) -> Tuple[str, Optional[str], int]:
    """-> (format, scale tensor name, block/group size)."""
    w = ck.info(base + ".weight")
    if w.dtype in ("BF16", "F16", "F32"):
        return "plain", None, 0
    scale_name = next((n for n in (base + ".weight_scale_inv", base + ".scale", base + ".weight_scale")
                       if ck.has(n)), None)
    if scale_name is None:
        raise CheckpointError(f"{base}: quantised weight without a scale tensor")
    s = ck.info(scale_name)
    if w.dtype == "F8_E4M3":
        if len(s.shape) != 2:
            raise CheckpointError(f"{base}: FP8 weight needs a 2-D block scale")
        return "fp8_block", scale_name, 128
    if w.dtype in ("I8", "U8"):
        cols = w.shape[1] * 2
        if len(s.shape) != 2 or s.shape[0] != w.shape[0] or cols % s.shape[1]:
            raise CheckpointError(f"{base}: FP4 scale shape {s.shape} does not divide {cols} columns")
        return "mxfp4", scale_name, cols // s.shape[1]
    raise CheckpointError(f"{base}: unsupported weight dtype {w.dtype}")


def read_linear(ck: ShardedCheckpoint, base: str, dtype=torch.bfloat16) -> torch.Tensor:
    """Decode `<base>` to a dense [out, in] tensor."""
    fmt, scale_name, block = infer_weight_format(ck, base)
    w = ck.read(base + ".weight")
    if fmt == "plain":
        return w.to(dtype)
    s = ck.read(scale_name)
    if fmt == "fp8_block":
        sb = s if s.dtype == torch.uint8 else None
        if sb is not None:
            return enc.weight_dequant_fp8_block(w.view(torch.uint8), sb, block).to(dtype)
        scale = s.float().repeat_interleave(block, 0)[:w.shape[0]].repeat_interleave(block, 1)[:, :w.shape[1]]
        return (enc.e4m3_decode(w.view(torch.uint8)) * scale).to(dtype)
    return enc.weight_dequant_mxfp4(w.view(torch.uint8), s.view(torch.uint8), block).to(dtype)


def _attn(ck, p: str, cfg: ModelConfig, rank: int, world: int, dev, dt) -> dict:
    h_lo, h_hi = _shard_range(cfg.n_heads, rank, world)
    qhd, nope, vd, lora = cfg.q_head_dim, cfg.qk_nope_dim, cfg.v_head_dim, cfg.kv_lora_rank
    kv_a = read_linear(ck, p + "kv_a_proj_with_mqa", dt)
    if cfg.q_lora_rank:
        q_part = read_linear(ck, p + "q_a_proj", dt)
        q_norm = ck.read(p + "q_a_layernorm.weight").to(dt)
        w_q_b = read_linear(ck, p + "q_b_proj", dt)[h_lo * qhd:h_hi * qhd].contiguous()
    else:
        q_part = read_linear(ck, p + "q_proj", dt)[h_lo * qhd:h_hi * qhd]
        q_norm, w_q_b = None, None
    kv_b = read_linear(ck, p + "kv_b_proj", dt).view(cfg.n_heads, nope + vd, lora)[h_lo:h_hi]
    w_o = read_linear(ck, p + "o_proj", dt)[:, h_lo * vd:h_hi * vd]
    mv = lambda t: None if t is None else t.contiguous().to(dev)
    return dict(w_qkv_a=mv(torch.cat([q_part, kv_a], 0)), q_norm=mv(q_norm), w_q_b=mv(w_q_b),
                kv_norm=mv(ck.read(p + "kv_a_layernorm.weight").to(dt)),
                w_uk_t=mv(kv_b[:, :nope].transpose(1, 2)), w_uv=mv(kv_b[:, nope:]), w_o=mv(w_o))


def _ffn(ck, p: str, rank: int, world: int, dev, dt):
    gate, up, down = (read_linear(ck, p + n, dt) for n in ("gate_proj", "up_proj", "down_proj"))
    i_lo, i_hi = _shard_range(gate.shape[0], rank, world)
    w13 = torch.cat([gate[i_lo:i_hi], up[i_lo:i_hi]], 0).unsqueeze(0).contiguous().to(dev)
    return w13, down[:, i_lo:i_hi].unsqueeze(0).contiguous().to(dev)


def _layer(ck, prefix: str, layer: int, cfg: ModelConfig, rank: int, world: int, dev, dt, is_moe: bool) -> LayerWeights:
    a = _attn(ck, prefix + "self_attn.", cfg, rank, world, dev, dt)
    lw = LayerWeights(attn_norm=ck.read(prefix + "input_layernorm.weight").to(dt).to(dev),
                      ffn_norm=ck.read(prefix + "post_attention_layernorm.weight").to(dt).to(dev), **a)
    lw.is_moe = is_moe
    if not is_moe:
        lw.w13, lw.w2 = _ffn(ck, prefix + "mlp.", rank, world, dev, dt)
        return lw
    lw.router_w = ck.read(prefix + "mlp.gate.weight").to(dt).to(dev)
    if ck.has(prefix + "mlp.gate.e_score_correction_bias"):
        lw.router_bias = ck.read(prefix + "mlp.gate.e_score_correction_bias").float().to(dev)
    if ck.has(prefix + "mlp.gate.tid2eid"):
        lw.hash_table = ck.read(prefix + "mlp.gate.tid2eid").long().to(dev)
    e_lo, e_hi = _shard_range(cfg.n_routed_experts, rank, world)
    w13s, w2s = [], []
    for e in range(e_lo, e_hi):
        ep = f"{prefix}mlp.experts.{e}."
        w13s.append(torch.cat([read_linear(ck, ep + "gate_proj", dt), read_linear(ck, ep + "up_proj", dt)], 0))
        w2s.append(read_linear(ck, ep + "down_proj", dt))
    lw.e_w13 = torch.stack(w13s).contiguous().to(dev)
    lw.e_w2 = torch.stack(w2s).contiguous().to(dev)
    if cfg.n_shared_experts:
        lw.w13, lw.w2 = _ffn(ck, prefix + "mlp.shared_experts.", rank, world, dev, dt)
    return lw


@fails_closed
def load_deepseek_hf(directory, device="cpu", dtype=torch.bfloat16, tp_rank: int = 0, tp_world: int = 1,
                     cfg: Optional[ModelConfig] = None, max_layers: int = 0) -> ModelWeights:
    """`max_layers` > 0: bind only the first layers of the checkpoint (a smoke run of a large model; the proposal
    stage, which continues from the last layer's hidden state, is then left out)."""
    ck = ShardedCheckpoint(directory)
    cfg = cfg or from_hf_config(directory)
    if 0 < max_layers < cfg.n_layers:
        cfg = cfg.with_(n_layers=max_layers, n_mtp_layers=0)
    dev, dt = torch.device(device), dtype
    embed = ck.read("model.embed_tokens.weight").to(dt).to(dev)
    layers = [_layer(ck, f"model.layers.{i}.", i, cfg, tp_rank, tp_world, dev, dt, cfg.is_moe_layer(i))
              for i in range(cfg.n_layers)]
    v_lo, v_hi = _shard_range(cfg.vocab_size, tp_rank, tp_world)
    head_name = "lm_head.weight" if ck.has("lm_head.weight") else "model.embed_tokens.weight"
    lm_head = ck.read(head_name).to(dt)[v_lo:v_hi].contiguous().to(dev)
    mtp = []
    for m in range(cfg.n_mtp_layers):
        p = f"model.layers.{cfg.n_layers + m}."
        if not ck.has(p + "eh_proj.weight"):
            break
        own_embed = own_head = None
        if ck.has(p + "embed_tokens.weight"):
            t = ck.read(p + "embed_tokens.weight").to(dt)
            if not torch.equal(t, embed.cpu()):
                own_embed = t.to(dev)
        if ck.has(p + "shared_head.head.weight"):
            t = ck.read(p + "shared_head.head.weight").to(dt)[v_lo:v_hi].contiguous()
            if not torch.equal(t, lm_head.cpu()):
                own_head = t.to(dev)
        mtp.append(MtpWeights(embed=own_embed, lm_head=own_head,
                              enorm=ck.read(p + "enorm.weight").to(dt).to(dev),
                              hnorm=ck.read(p + "hnorm.weight").to(dt).to(dev),
                              eh_proj=read_linear(ck, p + "eh_proj", dt).to(dev),
                              layer=_layer(ck, p, cfg.n_layers + m, cfg, tp_rank, tp_world, dev, dt,
                                           cfg.n_routed_experts > 0),
                              final_norm=ck.read(p + "shared_head.norm.weight").to(dt).to(dev)))
    e_lo, e_hi = _shard_range(cfg.n_routed_experts, tp_rank, tp_world) if cfg.n_routed_experts else (0, 0)
    w = ModelWeights(cfg, embed, layers, ck.read("model.norm.weight").to(dt).to(dev), lm_head, mtp, tp_rank, tp_world,
                     e_lo, e_hi, v_lo)
    ck.close()
    return w


# ---------------------------------------------------------------------------------------- export
def _put_linear(out: Dict[str, torch.Tensor], names: Dict[str, str], base: str, w: torch.Tensor, fmt: str) -> None:
    w = w.detach().cpu()
    if fmt == "fp8_block":
        q, sb = enc.weight_quant_fp8_block(w.float())
        out[base + ".weight"], out[base + ".scale"] = q, sb
        names[base + ".weight"], names[base + ".scale"] = "F8_E4M3", "F8_E8M0"
    elif fmt == "mxfp4":
        p, sb = enc.weight_quant_mxfp4(w.float())
        out[base + ".weight"], out[base + ".scale"] = p.view(torch.int8), sb
        names[base + ".scale"] = "F8_E8M0"
    else:
        out[base + ".weight"] = w


def export_hf(w: ModelWeights, directory, dense_format: str = "plain", expert_format: str = "plain",
              shard_bytes: int = 1 << 30) -> None:
    """Write a single-rank weight image as an HF DeepSeek directory (config.json + index + shards)."""
    if w.tp_world != 1:
        raise ValueError("export needs the unsharded weight image")
    cfg = w.cfg
    out: Dict[str, torch.Tensor] = {}
    names: Dict[str, str] = {}
    out["model.embed_tokens.weight"] = w.embed.cpu()
    out["model.norm.weight"] = w.final_norm.cpu()
    out["lm_head.weight"] = w.lm_head.cpu()
    qhd, nope = cfg.q_head_dim, cfg.qk_nope_dim

    def put_layer(p: str, lw: LayerWeights) -> None:
        a = p + "self_attn."
        out[p + "input_layernorm.weight"] = lw.attn_norm.cpu()
        out[p + "post_attention_layernorm.weight"] = lw.ffn_norm.cpu()
        q_rows = cfg.q_lora_rank if cfg.q_lora_rank else cfg.n_heads * qhd
        if cfg.q_lora_rank:
            _put_linear(out, names, a + "q_a_proj", lw.w_qkv_a[:q_rows], dense_format)
            out[a + "q_a_layernorm.weight"] = lw.q_norm.cpu()
            _put_linear(out, names, a + "q_b_proj", lw.w_q_b, dense_format)
        else:
            _put_linear(out, names, a + "q_proj", lw.w_qkv_a[:q_rows], dense_format)
        _put_linear(out, names, a + "kv_a_proj_with_mqa", lw.w_qkv_a[q_rows:], dense_format)
        out[a + "kv_a_layernorm.weight"] = lw.kv_norm.cpu()
        kv_b = torch.cat([lw.w_uk_t.transpose(1, 2), lw.w_uv], dim=1).reshape(-1, cfg.kv_lora_rank)
        _put_linear(out, names, a + "kv_b_proj", kv_b, dense_format)
        _put_linear(out, names, a + "o_proj", lw.w_o, dense_format)

        def put_ffn(fp: str, w13, w2, fmt):
            inter = w13.shape[-2] // 2
            _put_linear(out, names, fp + "gate_proj", w13[:inter], fmt)
            _put_linear(out, names, fp + "up_proj", w13[inter:], fmt)
            _put_linear(out, names, fp + "down_proj", w2, fmt)

        if not lw.is_moe:
            put_ffn(p + "mlp.", lw.w13[0], lw.w2[0], dense_format)
            return
        out[p + "mlp.gate.weight"] = lw.router_w.cpu()
        if lw.router_bias is not None:
            out[p + "mlp.gate.e_score_correction_bias"] = lw.router_bias.cpu()
        if lw.hash_table is not None:
            out[p + "mlp.gate.tid2eid"] = lw.hash_table.cpu()
        for e in range(lw.e_w13.shape[0]):
            put_ffn(f"{p}mlp.experts.{e}.", lw.e_w13[e], lw.e_w2[e], expert_format)
        if lw.w13 is not None:
            put_ffn(p + "mlp.shared_experts.", lw.w13[0], lw.w2[0], dense_format)

    for i, lw in enumerate(w.layers):
        put_layer(f"model.layers.{i}.", lw)
    for m, mt in enumerate(w.mtp):
        p = f"model.layers.{cfg.n_layers + m}."
        out[p + "enorm.weight"], out[p + "hnorm.weight"] = mt.enorm.cpu(), mt.hnorm.cpu()
        out[p + "eh_proj.weight"] = mt.eh_proj.cpu()
        out[p + "shared_head.norm.weight"] = mt.final_norm.cpu()
        if mt.embed is not None:
            out[p + "embed_tokens.weight"] = mt.embed.cpu()
        if mt.lm_head is not None:
            out[p + "shared_head.head.weight"] = mt.lm_head.cpu()
        put_layer(p, mt.layer)
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    write_sharded(out, d, shard_bytes, names)
    score = {0: "softmax", 1: "sigmoid", 2: "sqrtsoftplus"}[cfg.score_fn]
    (d / "config.json").write_text(json.dumps({
        "model_type": cfg.name, "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden,
        "num_hidden_layers": cfg.n_layers, "num_attention_heads": cfg.n_heads, "q_lora_rank": cfg.q_lora_rank or None,
        "kv_lora_rank": cfg.kv_lora_rank, "qk_nope_head_dim": cfg.qk_nope_dim, "qk_rope_head_dim": cfg.qk_rope_dim,
        "v_head_dim": cfg.v_head_dim, "rope_theta": cfg.rope_theta,
        "rope_scaling": ({"type": "yarn", "factor": cfg.rope_factor,
                          "original_max_position_embeddings": cfg.rope_orig_max_pos, "beta_fast": cfg.rope_beta_fast,
                          "beta_slow": cfg.rope_beta_slow, "mscale": cfg.rope_mscale,
                          "mscale_all_dim": cfg.rope_mscale_all_dim} if cfg.rope_factor > 1 else None),
        "max_position_embeddings": cfg.max_position, "rms_norm_eps": cfg.rms_eps,
        "first_k_dense_replace": cfg.n_dense_layers, "intermediate_size": cfg.dense_inter,
        "n_routed_experts": cfg.n_routed_experts, "n_shared_experts": cfg.n_shared_experts,
        "num_experts_per_tok": cfg.topk, "moe_intermediate_size": cfg.moe_inter, "scoring_func": score,
        "n_group": cfg.n_groups, "topk_group": cfg.topk_groups, "norm_topk_prob": cfg.norm_topk_prob,
        "routed_scaling_factor": cfg.route_scale, "topk_method": "noaux_tc" if cfg.router_bias else "greedy",
        "num_nextn_predict_layers": cfg.n_mtp_layers, "eos_token_id": cfg.eos_token_id,
        "bos_token_id": cfg.bos_token_id}, indent=1))
