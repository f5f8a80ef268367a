"""Support contract: which policies a model needs and whether this build can execute it.

`PolicySet` derives, from a model configuration and a deployment request, the eleven policy areas
(attention, router, expert, quantisation, KV cache, residency, parallelism, speculation, tokenizer,
validation, semantics).  `EnginePlan.from_policies` compares them with what the build implements and
answers Executable / MetadataOnly / Unsupported with the list of missing areas - nothing runs on
a guess.  Unlike the reference, whose `ParallelismPlan` is six inert fields, every degree here maps
to an implemented layout: tensor (heads, FFN inner dims, vocabulary), expert (token dispatch),
pipeline (layer ranges), data (engine replicas) and sequence (token-sharded activations between the
reduce-scatter / all-gather pairs); context parallelism stays at 1.

Counterpart of crates/ferrule-model/src/support/policies.rs:10-160 and support/plan.rs:84-115.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional, Tuple

from .config import SCORE_SIGMOID, SCORE_SOFTMAX, ModelConfig


class AttentionKind(Enum):
    MLA = "mla"                       # latent KV, weight-absorbed (DeepSeek-V2 / V3)
    HYBRID_SPARSE_MLA = "hybrid_mla"  # single latent head + window + compressed selection (DeepSeek-V4)


class RouterKind(Enum):
    NONE = "none"
    SOFTMAX_TOPK = "softmax_topk"
    SIGMOID_GROUP_TOPK = "sigmoid_group_topk"
    SQRT_SOFTPLUS_TOPK = "sqrt_softplus_topk"
    HASH = "hash"


class SpeculationMode(Enum):
    NONE = "none"
    MULTI_TOKEN_PREDICTION = "mtp"
    MARKOV_BLOCK = "markov_block"


@dataclass(frozen=True)
class AttentionPolicy:
    kind: AttentionKind
    kv_row_dim: int
    heads: int
    sink: bool


@dataclass(frozen=True)
class RouterPolicy:
    kind: RouterKind
    topk: int
    groups: Tuple[int, int]           # (n_groups, topk_groups)


@dataclass(frozen=True)
class ExpertPolicy:
    routed: int
    shared: int
    dense_layers: int


@dataclass(frozen=True)
class QuantPolicy:
    weight_format: str                # bf16 | fp8_block | fp8_mxfp4
    activation_blocks: Tuple[int, ...]


@dataclass(frozen=True)
class KvPolicy:
    paged: bool
    page_size: int
    planes: Tuple[str, ...]
    quantized: bool = False


@dataclass(frozen=True)
class ResidencyPolicy:
    streaming_allowed: bool
    resident_fraction: float


@dataclass(frozen=True)
class ParallelismPlan:
    data_parallel: int = 1
    tensor_parallel: int = 1
    expert_parallel: int = 1
    sequence_parallel: int = 1
    context_parallel: int = 1
    pipeline_parallel: int = 1

    @property
    def gpus(self) -> int:
        return self.data_parallel * self.tensor_parallel * self.pipeline_parallel


@dataclass(frozen=True)
class SpeculationPolicy:
    mode: SpeculationMode
    max_draft: int


@dataclass(frozen=True)
class TokenizerPolicy:
    requires_external_encoding: bool
    has_chat_template: bool


@dataclass(frozen=True)
class ValidationPolicy:
    supports_cpu_reference: bool
    requires_reference_engine: bool = False


@dataclass(frozen=True)
class PolicySet:
    attention: AttentionPolicy
    router: RouterPolicy
    expert: ExpertPolicy
    quant: QuantPolicy
    kv: KvPolicy
    residency: ResidencyPolicy
    parallelism: ParallelismPlan
    speculation: SpeculationPolicy
    tokenizer: TokenizerPolicy
    validation: ValidationPolicy
    semantics: str                    # "deepseek-v2" | "deepseek-v3" | "deepseek-v4"

    @staticmethod
    def from_config(cfg, weight_format: str = "bf16", parallelism: Optional[ParallelismPlan] = None,
                    page_size: int = 64, resident_fraction: float = 1.0, chat_template: bool = True,
                    tokenizer_files: bool = False) -> "PolicySet":
        par = parallelism or ParallelismPlan()
        v4 = not isinstance(cfg, ModelConfig)          # models.v4_model.V4Config
        if v4:
            att = AttentionPolicy(AttentionKind.HYBRID_SPARSE_MLA, cfg.head_dim, cfg.n_heads, True)
            router = RouterPolicy(RouterKind.HASH if cfg.n_hash_layers >= cfg.n_layers else RouterKind.SQRT_SOFTPLUS_TOPK,
                                  cfg.topk, (1, 1))
            expert = ExpertPolicy(cfg.n_routed_experts, cfg.n_shared_experts, 0)
            planes = ("window_kv", "compressed_kv", "indexer_plane")
            spec = SpeculationPolicy(SpeculationMode.MARKOV_BLOCK if getattr(cfg, "mtp_block", 0) else SpeculationMode.NONE,
                                     getattr(cfg, "mtp_block", 0))
            sem = "deepseek-v4"
        else:
            att = AttentionPolicy(AttentionKind.MLA, cfg.kv_row_dim, cfg.n_heads, bool(cfg.attn_sink))
            if not cfg.n_routed_experts:
                rk = RouterKind.NONE
            elif cfg.n_hash_layers:
                rk = RouterKind.HASH
            elif cfg.score_fn == SCORE_SOFTMAX:
                rk = RouterKind.SOFTMAX_TOPK
            elif cfg.score_fn == SCORE_SIGMOID:
                rk = RouterKind.SIGMOID_GROUP_TOPK
            else:
                rk = RouterKind.SQRT_SOFTPLUS_TOPK
            router = RouterPolicy(rk, cfg.topk, (cfg.n_groups, cfg.topk_groups))
            expert = ExpertPolicy(cfg.n_routed_experts, cfg.n_shared_experts, cfg.n_dense_layers)
            planes = ("latent_kv",)
            spec = SpeculationPolicy(SpeculationMode.MULTI_TOKEN_PREDICTION if cfg.n_mtp_layers else SpeculationMode.NONE,
                                     1 if cfg.n_mtp_layers else 0)
            sem = "deepseek-v3" if cfg.q_lora_rank else "deepseek-v2"
        blocks = {"bf16": (), "fp8_block": (128,), "fp8_mxfp4": (128, 32)}[weight_format]
        return PolicySet(att, router, expert, QuantPolicy(weight_format, blocks),
                         KvPolicy(True, page_size, planes),
                         ResidencyPolicy(expert.routed > 0, resident_fraction), par, spec,
                         TokenizerPolicy(not tokenizer_files, chat_template), ValidationPolicy(True), sem)


class EnginePlanStatus(Enum):
    EXECUTABLE = "executable"
    METADATA_ONLY = "metadata_only"
    UNSUPPORTED = "unsupported"


@dataclass(frozen=True)
class MissingPolicy:
    area: str
    reason: str


@dataclass
class EnginePlan:
    family: str
    status: EnginePlanStatus
    policies: PolicySet
    missing: List[MissingPolicy] = field(default_factory=list)

    @property
    def is_executable(self) -> bool:
        return self.status == EnginePlanStatus.EXECUTABLE

    @staticmethod
    def from_policies(p: PolicySet, n_heads: int, n_experts: int, n_layers: int, vocab: int) -> "EnginePlan":
        """Check every area against what this build implements; anything else is reported, not guessed."""
        missing: List[MissingPolicy] = []
        par = p.parallelism
        if par.context_parallel != 1:
            missing.append(MissingPolicy("parallelism", "context parallelism is not implemented (long context is "
                                         "handled by KV compression + sparse selection on one GPU)"))
        if par.tensor_parallel > 1 and (n_heads % par.tensor_parallel or vocab % par.tensor_parallel):
            missing.append(MissingPolicy("parallelism", "heads and vocabulary must divide by the tensor-parallel degree"))
        if par.expert_parallel > 1 and (n_experts % par.expert_parallel or par.expert_parallel != par.tensor_parallel):
            missing.append(MissingPolicy("parallelism", "expert parallelism runs over the tensor-parallel group and "
                                         "must divide the expert count"))
        if par.sequence_parallel not in (1, par.tensor_parallel):
            missing.append(MissingPolicy("parallelism", "sequence parallelism is the token-sharded form of the "
                                         "tensor-parallel group (degree 1 or the tensor-parallel degree)"))
        if par.pipeline_parallel > 1 and n_layers < par.pipeline_parallel:
            missing.append(MissingPolicy("parallelism", "fewer layers than pipeline stages"))
        if p.semantics == "deepseek-v4":
            if p.quant.weight_format != "bf16":
                missing.append(MissingPolicy("quantization", "the V4 step runs bf16 weights (quantised checkpoints are "
                                             "dequantised at load time)"))
            if par.tensor_parallel > 1 or par.pipeline_parallel > 1:
                missing.append(MissingPolicy("parallelism", "the V4 runner is single-GPU"))
        if p.residency.resident_fraction < 1.0 and p.quant.weight_format != "bf16" and p.semantics != "deepseek-v4":
            pass        # quantised experts stream through the same arena (frames hold the packed form)
        status = EnginePlanStatus.EXECUTABLE if not missing else EnginePlanStatus.METADATA_ONLY
        return EnginePlan(p.semantics, status, p, missing)
