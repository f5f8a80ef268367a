"""Family registry: tensor name -> semantic role, for every checkpoint naming this runtime meets.

Roles tell the loader what a tensor is (attention projection, norm, router, routed / shared expert
weight, scale, MTP part ...) independent of the naming scheme.  Families: DeepSeek (HuggingFace
V2/V3 names: `model.layers.N.self_attn.q_a_proj.weight`), DeepSeek-V4 (the reference's flat names:
`layers.N.attn.wq_a.weight`, `ffn.experts.E.w1.weight`, `mtp.M.*`), Qwen3 and generic
Llama-style.  Only the DeepSeek family executes; the others are classified for inspection.

Counterpart of crates/ferrule-model/src/families/mod.rs:20-115, families/deepseek_v4.rs:9-300 and
support/*.rs (TensorRole / ModelLayout).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from enum import Enum
from typing import Dict, Iterable, Optional


class TensorRole(Enum):
    EMBEDDING = "embedding"
    FINAL_NORM = "final_norm"
    OUTPUT_HEAD = "output_head"
    ATTN_NORM = "attn_norm"
    FFN_NORM = "ffn_norm"
    ATTN_Q = "attn_q"
    ATTN_Q_A = "attn_q_a"
    ATTN_Q_B = "attn_q_b"
    ATTN_Q_NORM = "attn_q_norm"
    ATTN_K = "attn_k"
    ATTN_V = "attn_v"
    ATTN_KV_A = "attn_kv_a"
    ATTN_KV_B = "attn_kv_b"
    ATTN_KV_NORM = "attn_kv_norm"
    ATTN_OUT = "attn_out"
    ATTN_OUT_A = "attn_out_a"
    ATTN_OUT_B = "attn_out_b"
    ATTN_SINK = "attn_sink"
    COMPRESSOR = "compressor"
    INDEXER = "indexer"
    HYPER_CONNECTION = "hyper_connection"
    ROUTER = "router"
    ROUTER_BIAS = "router_bias"
    ROUTER_HASH = "router_hash"
    EXPERT_GATE = "expert_gate"
    EXPERT_UP = "expert_up"
    EXPERT_DOWN = "expert_down"
    SHARED_GATE = "shared_gate"
    SHARED_UP = "shared_up"
    SHARED_DOWN = "shared_down"
    DENSE_GATE = "dense_gate"
    DENSE_UP = "dense_up"
    DENSE_DOWN = "dense_down"
    MTP = "mtp"
    SCALE = "scale"
    UNKNOWN = "unknown"


@dataclass(frozen=True)
class TensorClass:
    role: TensorRole
    layer: Optional[int] = None
    expert: Optional[int] = None
    is_scale: bool = False
    mtp_stage: Optional[int] = None


class Family(Enum):
    DEEPSEEK_HF = "deepseek_hf"
    DEEPSEEK_V4 = "deepseek_v4"
    QWEN3 = "qwen3"
    LLAMA = "llama"


_SCALE_SUFFIX = (".weight_scale_inv", ".scale", ".weight_scale")

_HF_ATTN = {"q_proj": TensorRole.ATTN_Q, "q_a_proj": TensorRole.ATTN_Q_A, "q_b_proj": TensorRole.ATTN_Q_B,
            "q_a_layernorm": TensorRole.ATTN_Q_NORM, "kv_a_proj_with_mqa": TensorRole.ATTN_KV_A,
            "kv_b_proj": TensorRole.ATTN_KV_B, "kv_a_layernorm": TensorRole.ATTN_KV_NORM, "o_proj": TensorRole.ATTN_OUT,
            "k_proj": TensorRole.ATTN_K, "v_proj": TensorRole.ATTN_V, "q_norm": TensorRole.ATTN_Q_NORM,
            "k_norm": TensorRole.ATTN_KV_NORM}
_HF_FFN = {"gate_proj": 0, "up_proj": 1, "down_proj": 2}
_V4_ATTN = {"wq_a": TensorRole.ATTN_Q_A, "wq_b": TensorRole.ATTN_Q_B, "wkv": TensorRole.ATTN_KV_A,
            "wo_a": TensorRole.ATTN_OUT_A, "wo_b": TensorRole.ATTN_OUT_B, "q_norm": TensorRole.ATTN_Q_NORM,
            "kv_norm": TensorRole.ATTN_KV_NORM, "attn_sink": TensorRole.ATTN_SINK}
_V4_FFN = {"w1": 0, "w3": 1, "w2": 2}


def _ffn_role(kind: str, idx: int) -> TensorRole:
    table = {"expert": (TensorRole.EXPERT_GATE, TensorRole.EXPERT_UP, TensorRole.EXPERT_DOWN),
             "shared": (TensorRole.SHARED_GATE, TensorRole.SHARED_UP, TensorRole.SHARED_DOWN),
             "dense": (TensorRole.DENSE_GATE, TensorRole.DENSE_UP, TensorRole.DENSE_DOWN)}
    return table[kind][idx]


def classify(name: str, family: Family, n_layers: Optional[int] = None) -> TensorClass:
    is_scale = name.endswith(_SCALE_SUFFIX)
    base = name
    for s in _SCALE_SUFFIX + (".weight", ".bias"):
        if base.endswith(s):
            base = base[: -len(s)]
            break
    if family in (Family.DEEPSEEK_HF, Family.QWEN3, Family.LLAMA):
        if base in ("model.embed_tokens",):
            return TensorClass(TensorRole.EMBEDDING)
        if base == "model.norm":
            return TensorClass(TensorRole.FINAL_NORM)
        if base == "lm_head":
            return TensorClass(TensorRole.OUTPUT_HEAD)
        m = re.match(r"model\.layers\.(\d+)\.(.*)", base)
        if not m:
            return TensorClass(TensorRole.UNKNOWN)
        layer, rest = int(m.group(1)), m.group(2)
        mtp = layer - n_layers if (n_layers is not None and layer >= n_layers) else None
        if rest == "input_layernorm":
            return TensorClass(TensorRole.ATTN_NORM, layer, mtp_stage=mtp)
        if rest == "post_attention_layernorm":
            return TensorClass(TensorRole.FFN_NORM, layer, mtp_stage=mtp)
        if rest in ("enorm", "hnorm", "eh_proj", "shared_head.norm", "shared_head.head", "embed_tokens"):
            return TensorClass(TensorRole.MTP, layer, mtp_stage=mtp)
        if rest.startswith("self_attn."):
            role = _HF_ATTN.get(rest.split(".", 1)[1])
            return TensorClass(role or TensorRole.UNKNOWN, layer, is_scale=is_scale, mtp_stage=mtp)
        if rest == "mlp.gate":
            return TensorClass(TensorRole.ROUTER if name.endswith(".weight") else TensorRole.ROUTER_BIAS, layer, mtp_stage=mtp)
        if rest == "mlp.gate.e_score_correction_bias" or name.endswith("e_score_correction_bias"):
            return TensorClass(TensorRole.ROUTER_BIAS, layer, mtp_stage=mtp)
        if name.endswith("gate.tid2eid"):
            return TensorClass(TensorRole.ROUTER_HASH, layer, mtp_stage=mtp)
        m2 = re.match(r"mlp\.experts\.(\d+)\.(\w+)", rest)
        if m2 and m2.group(2) in _HF_FFN:
            return TensorClass(_ffn_role("expert", _HF_FFN[m2.group(2)]), layer, int(m2.group(1)), is_scale, mtp)
        m3 = re.match(r"mlp\.shared_experts?\.(\w+)", rest)
        if m3 and m3.group(1) in _HF_FFN:
            return TensorClass(_ffn_role("shared", _HF_FFN[m3.group(1)]), layer, None, is_scale, mtp)
        m4 = re.match(r"mlp\.(\w+)", rest)
        if m4 and m4.group(1) in _HF_FFN:
            return TensorClass(_ffn_role("dense", _HF_FFN[m4.group(1)]), layer, None, is_scale, mtp)
        return TensorClass(TensorRole.UNKNOWN, layer)
    # ---- DeepSeek-V4 flat names ----
    if base == "embed":
        return TensorClass(TensorRole.EMBEDDING)
    if base == "norm":
        return TensorClass(TensorRole.FINAL_NORM)
    if base == "head":
        return TensorClass(TensorRole.OUTPUT_HEAD)
    if base.startswith("hc_head_"):
        return TensorClass(TensorRole.HYPER_CONNECTION)
    mtp = None
    m = re.match(r"mtp\.(\d+)\.(.*)", base)
    if m:
        mtp, rest = int(m.group(1)), m.group(2)
        if not re.match(r"(attn|ffn|hc_|attn_norm|ffn_norm)", rest):
            return TensorClass(TensorRole.MTP, None, mtp_stage=mtp)
        layer = None
    else:
        m = re.match(r"layers\.(\d+)\.(.*)", base)
        if not m:
            return TensorClass(TensorRole.UNKNOWN)
        layer, rest = int(m.group(1)), m.group(2)
    if rest == "attn_norm":
        return TensorClass(TensorRole.ATTN_NORM, layer, mtp_stage=mtp)
    if rest == "ffn_norm":
        return TensorClass(TensorRole.FFN_NORM, layer, mtp_stage=mtp)
    if rest.startswith("hc_"):
        return TensorClass(TensorRole.HYPER_CONNECTION, layer, mtp_stage=mtp)
    if rest.startswith("attn.compressor"):
        return TensorClass(TensorRole.COMPRESSOR, layer, mtp_stage=mtp)
    if rest.startswith("attn.indexer"):
        return TensorClass(TensorRole.INDEXER, layer, mtp_stage=mtp)
    if rest.startswith("attn."):
        role = _V4_ATTN.get(rest.split(".")[1])
        return TensorClass(role or TensorRole.UNKNOWN, layer, is_scale=is_scale, mtp_stage=mtp)
    if rest == "ffn.gate":
        if name.endswith("tid2eid"):
            return TensorClass(TensorRole.ROUTER_HASH, layer, mtp_stage=mtp)
        return TensorClass(TensorRole.ROUTER_BIAS if name.endswith(".bias") else TensorRole.ROUTER, layer, mtp_stage=mtp)
    if rest == "ffn.gate.tid2eid" or name.endswith("ffn.gate.tid2eid"):
        return TensorClass(TensorRole.ROUTER_HASH, layer, mtp_stage=mtp)
    m2 = re.match(r"ffn\.experts\.(\d+)\.(w[123])", rest)
    if m2:
        return TensorClass(_ffn_role("expert", _V4_FFN[m2.group(2)]), layer, int(m2.group(1)), is_scale, mtp)
    m3 = re.match(r"ffn\.shared_experts\.(w[123])", rest)
    if m3:
        return TensorClass(_ffn_role("shared", _V4_FFN[m3.group(1)]), layer, None, is_scale, mtp)
    return TensorClass(TensorRole.UNKNOWN, layer, mtp_stage=mtp)


def detect_family(names: Iterable[str], model_type: str = "") -> Family:
    names = list(names)
    if any(n.startswith("layers.") and ".attn.wq_a" in n for n in names) or any(n.startswith("mtp.") for n in names):
        return Family.DEEPSEEK_V4
    mt = model_type.lower()
    if "qwen" in mt:
        return Family.QWEN3
    if any("kv_a_proj_with_mqa" in n for n in names) or "deepseek" in mt:
        return Family.DEEPSEEK_HF
    return Family.LLAMA


def layout_summary(names: Iterable[str], family: Family, n_layers: Optional[int] = None) -> Dict[str, int]:
    """Role histogram of a checkpoint (used by `ferrule info` / `inspect-weightpack`)."""
    out: Dict[str, int] = {}
    for n in names:
        r = classify(n, family, n_layers).role.value
        out[r] = out.get(r, 0) + 1
    return out
