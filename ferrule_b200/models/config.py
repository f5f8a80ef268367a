"""Model hyper-parameters for the DeepSeek family (MLA attention + routed MoE + MTP).

One parameterised description covers the V2-Lite and V3 shapes that are measured here,
the CPU fixture, and the V4-only switches (sqrt-softplus / hash routing, clamp, sink,
hyper-connections).  `from_hf_config` reads a HuggingFace `config.json`.

Counterpart of the reference's config and family constants
(crates/ferrule-model/src/models/deepseek_v4/config.rs:78-272,
 crates/ferrule-model/src/families/deepseek_v4.rs:9-39) and its policy set
(crates/ferrule-model/src/support/policies.rs:56-77 for the parallelism plan).
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, replace
from pathlib import Path

SCORE_SOFTMAX, SCORE_SIGMOID, SCORE_SQRT_SOFTPLUS = 0, 1, 2
_SCORE_NAMES = {"softmax": 0, "sigmoid": 1, "sqrtsoftplus": 2, "sqrt_softplus": 2}


@dataclass(frozen=True)
class ModelConfig:
    name: str = "deepseek"
    vocab_size: int = 1024
    hidden: int = 256
    n_layers: int = 2
    n_heads: int = 4
    q_lora_rank: int = 0            # 0: direct q projection
    kv_lora_rank: int = 64
    qk_nope_dim: int = 32
    qk_rope_dim: int = 16
    v_head_dim: int = 32
    rope_theta: float = 10000.0
    rope_factor: float = 1.0        # YaRN factor (1 = plain RoPE)
    rope_orig_max_pos: int = 4096
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rope_mscale: float = 1.0
    rope_mscale_all_dim: float = 0.0
    max_position: int = 4096
    rms_eps: float = 1e-6
    n_dense_layers: int = 1         # leading layers with a dense FFN
    dense_inter: int = 512
    n_routed_experts: int = 8
    n_shared_experts: int = 1
    topk: int = 2
    moe_inter: int = 128
    score_fn: int = SCORE_SIGMOID
    n_groups: int = 1
    topk_groups: int = 1
    norm_topk_prob: bool = True
    route_scale: float = 1.0
    router_bias: bool = False
    n_hash_layers: int = 0          # V4: leading MoE layers routed by token-id hash table
    swiglu_limit: float = 0.0       # V4: clamp
    attn_sink: bool = False         # V4: per-head sink logit in the softmax denominator
    n_mtp_layers: int = 0
    eos_token_id: int = 1
    bos_token_id: int = 0
    weight_format: str = "bf16"     # bf16 | fp8_block | fp8_block+mxfp4_experts

    # ---- derived ----
    @property
    def q_head_dim(self) -> int:
        return self.qk_nope_dim + self.qk_rope_dim

    @property
    def kv_row_dim(self) -> int:
        return self.kv_lora_rank + self.qk_rope_dim

    @property
    def softmax_scale(self) -> float:
        s = 1.0 / math.sqrt(self.q_head_dim)
        if self.rope_factor > 1.0 and self.rope_mscale_all_dim:
            m = 0.1 * self.rope_mscale_all_dim * math.log(self.rope_factor) + 1.0
            s *= m * m
        return s

    def is_moe_layer(self, layer: int) -> bool:
        return self.n_routed_experts > 0 and layer >= self.n_dense_layers

    def param_count(self) -> int:
        h = self.hidden
        attn = (self.q_lora_rank * (h + self.n_heads * self.q_head_dim) if self.q_lora_rank
                else h * self.n_heads * self.q_head_dim)
        attn += h * self.kv_row_dim + self.kv_lora_rank * self.n_heads * (self.qk_nope_dim + self.v_head_dim)
        attn += self.n_heads * self.v_head_dim * h
        dense = 3 * h * self.dense_inter
        moe = (self.n_routed_experts + self.n_shared_experts) * 3 * h * self.moe_inter + h * self.n_routed_experts
        n_moe = max(self.n_layers - self.n_dense_layers, 0) if self.n_routed_experts else 0
        n_dense = self.n_layers - n_moe
        return 2 * self.vocab_size * h + self.n_layers * attn + n_dense * dense + n_moe * moe

    def to_dict(self) -> dict:
        return asdict(self)

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)


def tiny_fixture() -> ModelConfig:
    """The CPU correctness fixture: 2 layers, MLA + dense + MoE(8, top-2 sigmoid, 1 shared) + 1 MTP."""
    return ModelConfig(name="tiny-fixture", vocab_size=1024, hidden=256, n_layers=2, n_heads=4,
                       q_lora_rank=128, kv_lora_rank=64, qk_nope_dim=32, qk_rope_dim=16, v_head_dim=32,
                       rope_theta=10000.0, n_dense_layers=1, dense_inter=512, n_routed_experts=8,
                       n_shared_experts=1, topk=2, moe_inter=128, score_fn=SCORE_SIGMOID,
                       norm_topk_prob=True, n_mtp_layers=1, max_position=2048)


def smoke_gpu() -> ModelConfig:
    """Small model with the production head geometry (kv_lora 512 / rope 64) for GPU smoke tests."""
    return ModelConfig(name="smoke-gpu", vocab_size=4096, hidden=512, n_layers=3, n_heads=8,
                       q_lora_rank=0, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128,
                       n_dense_layers=1, dense_inter=1024, n_routed_experts=16, n_shared_experts=2,
                       topk=4, moe_inter=256, score_fn=SCORE_SOFTMAX, norm_topk_prob=False,
                       max_position=4096)


def deepseek_v2_lite() -> ModelConfig:
    return ModelConfig(name="deepseek-v2-lite", vocab_size=102400, hidden=2048, n_layers=27, n_heads=16,
                       q_lora_rank=0, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128,
                       rope_theta=10000.0, rope_factor=40.0, rope_orig_max_pos=4096, rope_beta_fast=32.0,
                       rope_beta_slow=1.0, rope_mscale=0.707, rope_mscale_all_dim=0.707,
                       max_position=163840, n_dense_layers=1, dense_inter=10944, n_routed_experts=64,
                       n_shared_experts=2, topk=6, moe_inter=1408, score_fn=SCORE_SOFTMAX,
                       n_groups=1, topk_groups=1, norm_topk_prob=False, route_scale=1.0,
                       eos_token_id=100001, bos_token_id=100000)


def deepseek_v3() -> ModelConfig:
    return ModelConfig(name="deepseek-v3", vocab_size=129280, hidden=7168, n_layers=61, n_heads=128,
                       q_lora_rank=1536, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128,
                       rope_theta=10000.0, rope_factor=40.0, rope_orig_max_pos=4096, rope_mscale=1.0,
                       rope_mscale_all_dim=1.0, max_position=163840, n_dense_layers=3, dense_inter=18432,
                       n_routed_experts=256, n_shared_experts=1, topk=8, moe_inter=2048,
                       score_fn=SCORE_SIGMOID, n_groups=8, topk_groups=4, norm_topk_prob=True,
                       route_scale=2.5, router_bias=True, n_mtp_layers=1, eos_token_id=1,
                       weight_format="fp8_block")


PRESETS = {"tiny-fixture": tiny_fixture, "smoke-gpu": smoke_gpu, "deepseek-v2-lite": deepseek_v2_lite,
           "deepseek-v3": deepseek_v3}


def from_hf_config(path) -> ModelConfig:
    """Read a HuggingFace DeepSeek-V2/V3 style config.json."""
    p = Path(path)
    if p.is_dir():
        p = p / "config.json"
    c = json.loads(p.read_text())
    rs = c.get("rope_scaling") or {}
    score = _SCORE_NAMES.get(str(c.get("scoring_func", "softmax")).lower(), 0)
    return ModelConfig(
        name=c.get("model_type", "deepseek"), vocab_size=c["vocab_size"], hidden=c["hidden_size"],
        n_layers=c["num_hidden_layers"], n_heads=c["num_attention_heads"],
        q_lora_rank=c.get("q_lora_rank") or 0, kv_lora_rank=c["kv_lora_rank"],
        qk_nope_dim=c["qk_nope_head_dim"], qk_rope_dim=c["qk_rope_head_dim"], v_head_dim=c["v_head_dim"],
        rope_theta=float(c.get("rope_theta", 10000.0)), rope_factor=float(rs.get("factor", 1.0)),
        rope_orig_max_pos=int(rs.get("original_max_position_embeddings", 4096)),
        rope_beta_fast=float(rs.get("beta_fast", 32.0)), rope_beta_slow=float(rs.get("beta_slow", 1.0)),
        rope_mscale=float(rs.get("mscale", 1.0)), rope_mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)),
        max_position=int(c.get("max_position_embeddings", 4096)), rms_eps=float(c.get("rms_norm_eps", 1e-6)),
        n_dense_layers=int(c.get("first_k_dense_replace", 0)), dense_inter=int(c.get("intermediate_size", 0)),
        n_routed_experts=int(c.get("n_routed_experts") or 0), n_shared_experts=int(c.get("n_shared_experts") or 0),
        topk=int(c.get("num_experts_per_tok") or 1), moe_inter=int(c.get("moe_intermediate_size") or 0),
        score_fn=score, n_groups=int(c.get("n_group") or 1), topk_groups=int(c.get("topk_group") or 1),
        norm_topk_prob=bool(c.get("norm_topk_prob", False)), route_scale=float(c.get("routed_scaling_factor", 1.0)),
        router_bias=c.get("topk_method") == "noaux_tc", n_mtp_layers=int(c.get("num_nextn_predict_layers") or 0),
        eos_token_id=int(c.get("eos_token_id", 1) if not isinstance(c.get("eos_token_id"), list) else c["eos_token_id"][0]),
        bos_token_id=int(c.get("bos_token_id", 0)),
        weight_format="fp8_block" if (c.get("quantization_config") or {}).get("quant_method") == "fp8" else "bf16")


@dataclass(frozen=True)
class ParallelConfig:
    """How one model replica is laid over GPUs.  All sizes default to 1 (single GPU)."""
    tp: int = 1        # tensor parallel (attention heads, dense/shared FFN inter dim, vocab)
    ep: int = 1        # expert parallel (routed experts); ep == tp shares the same group
    pp: int = 1        # pipeline stages
    dp: int = 1        # replicas
    rank: int = 0
    fused_collectives: bool = True   # False: NCCL baseline path

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.dp
