"""Execution plan: which native operators a model needs, checked against what the loaded library
provides, before anything runs.  Compilation fails closed: a missing operator is an error that names
it, never a silent fallback to another path.

* `ProviderRegistry` - catalog of operator groups, built by probing the native library's entry points
  (the library's manifest) or from an explicit set (tests).
* `ExecutableStage` / `ResolvedStage` - per-layer stages with their operator requirements, dependencies,
  resource accesses and workspace bytes; `ResourceRetention` says how long a stage's resources are held
  (Stage, Transaction, Persistent).
* `compile_model_plan(cfg, ...)` - lowers a model configuration (+ weight format, parallel layout,
  speculation) to the ordered stage list and resolves it against the registry.
* Materialization boundary types (`MaterializationRequest`, `Placement`, `Preparation`) - what a stage
  hands to the materialization provider when one of its resources is not resident.

Counterpart of crates/ferrule-backend/src/cuda/provider.rs:21-270 (registry, fail-closed compile) and
crates/ferrule-backend/src/plan.rs:41-495 (operations, launch descriptors, model plan),
crates/ferrule-model/src/execution/stage.rs:20-470 (stage types) and
crates/ferrule-model/src/materialization.rs:16-320 (boundary types).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, FrozenSet, Iterable, List, Optional, Sequence, Tuple

from .io_protocol import MaterializationKey


class PlanError(RuntimeError):
    """The model cannot run on this build: an operator or bundle it needs is absent."""


# operator group -> entry points of the native library that implement it
OPERATOR_GROUPS: Dict[str, Tuple[str, ...]] = {
    "gemm_bf16": ("fb_gemm_bf16",),
    "gemm_fp8_block": ("fb_gemm_fp8", "fb_quant_fp8_rows"),
    "gemm_mxfp4_experts": ("fb_gemm_fp8", "fb_quant_fp8_rows"),
    "attention_mla_paged": ("fb_mla_attention", "fb_mla_prep"),
    "attention_sparse_selection": ("fb_mla_attention", "fb_indexer_scores", "fb_indexer_topk", "fb_rope_rows"),
    "kv_compressor": ("fb_compressor_pool",),
    "hyper_connection": ("fb_hc_pre", "fb_hc_post"),
    "norm_embedding": ("fb_add_rmsnorm", "fb_embedding"),
    "router_plan": ("fb_router_topk", "fb_moe_plan", "fb_gather_rows", "fb_moe_reduce"),
    "router_plan_fused": ("fb_router_plan_fused",),
    "router_static_slots": ("fb_router_append", "fb_moe_reduce_norm"),
    "sampling_greedy": ("fb_argmax", "fb_topk_logits"),
    "kv_pages": ("fb_copy_pages",),
    "collective_allreduce": ("fb_moe_reduce_allreduce", "fb_ipc_alloc", "fb_ipc_open"),
    "collective_vocab_argmax": ("fb_argmax_allgather",),
    "expert_dispatch": ("fb_ep_dispatch", "fb_ep_collect", "fb_ep_combine_reduce"),
    "expert_slot_table": ("fb_expert_table_apply", "fb_expert_table_resolve"),
    "direct_reader": ("fb_reader_create", "fb_reader_submit", "fb_reader_poll"),
}


class ProviderRegistry:
    def __init__(self, available: Iterable[str]):
        self.available: FrozenSet[str] = frozenset(available)

    @classmethod
    def from_library(cls, lib=None) -> "ProviderRegistry":
        """Probe the native library: a group is available when every one of its entry points resolves."""
        if lib is None:
            from ..ops._lib import get_lib
            lib = get_lib(required=False)
        have = set()
        if lib is not None:
            for group, symbols in OPERATOR_GROUPS.items():
                if all(_has_symbol(lib, s) for s in symbols):
                    have.add(group)
        return cls(have)

    def require(self, groups: Iterable[str], what: str) -> None:
        missing = sorted(set(groups) - self.available)
        if missing:
            raise PlanError(f"{what}: operator group(s) not provided by this build: {', '.join(missing)}")

    def manifest(self) -> Dict[str, bool]:
        return {g: g in self.available for g in sorted(OPERATOR_GROUPS)}


def _has_symbol(lib, name: str) -> bool:
    try:
        getattr(lib, name)
        return True
    except AttributeError:
        return False


class ResourceRetention(Enum):
    STAGE = "stage"                # scratch: free once the stage's kernels have been issued
    TRANSACTION = "transaction"    # held until the transaction publishes or aborts (KV rows, leases)
    PERSISTENT = "persistent"      # weights and tables


class AccessMode(Enum):
    READ = "read"
    WRITE = "write"
    READ_WRITE = "read_write"


@dataclass(frozen=True)
class ResourceAccess:
    resource: str
    mode: AccessMode
    retention: ResourceRetention
    streamed: bool = False         # may be absent at execution time -> materialization request


@dataclass(frozen=True)
class ExecutableStage:
    name: str
    layer: int                     # -1: not tied to a layer (embedding, head)
    operators: Tuple[str, ...]
    accesses: Tuple[ResourceAccess, ...] = ()
    workspace_bytes: int = 0


@dataclass(frozen=True)
class ResolvedStage:
    index: int
    stage: ExecutableStage
    dependencies: Tuple[int, ...]  # indices of the stages whose outputs this one reads


@dataclass
class ModelPlan:
    model: str
    stages: List[ResolvedStage]
    operators: FrozenSet[str]
    workspace_bytes: int
    suspends_at: Tuple[int, ...]   # stage indices that can return Waiting (streamed resources)

    def summary(self) -> Dict[str, object]:
        return {"model": self.model, "stages": len(self.stages), "operators": sorted(self.operators),
                "workspace_bytes": self.workspace_bytes, "suspendable_stages": len(self.suspends_at)}


def _weights(name: str, streamed: bool = False) -> ResourceAccess:
    return ResourceAccess(name, AccessMode.READ, ResourceRetention.PERSISTENT, streamed)


def compile_model_plan(cfg, registry: Optional[ProviderRegistry] = None, *, weight_format: str = "bf16",
                       tp_world: int = 1, expert_dispatch: bool = False, streamed_experts: bool = False,
                       speculative: bool = False, max_rows: int = 2048) -> ModelPlan:
    """Lower a `ModelConfig` (DeepSeek-V2/V3 family) or `V4Config` to stages and resolve them.  Raises
    `PlanError` naming every missing operator group."""
    registry = registry or ProviderRegistry.from_library()
    v4 = hasattr(cfg, "hc_mult")
    gemm = {"bf16": "gemm_bf16", "fp8_block": "gemm_fp8_block", "fp8_mxfp4": "gemm_fp8_block"}.get(weight_format)
    if gemm is None:
        raise PlanError(f"unknown weight format {weight_format!r}")
    expert_gemm = "gemm_mxfp4_experts" if weight_format == "fp8_mxfp4" else gemm
    H = cfg.hidden
    stages: List[ExecutableStage] = [ExecutableStage("embedding", -1, ("norm_embedding",), (_weights("embed"),))]
    n_layers = cfg.n_layers
    for i in range(n_layers):
        if v4:
            ops = ["hyper_connection", "norm_embedding", "gemm_bf16", "attention_sparse_selection"]
            if cfg.ratio(i):
                ops.append("kv_compressor")
            acc = (_weights(f"layers.{i}.attn"), ResourceAccess(f"kv.{i}", AccessMode.READ_WRITE, ResourceRetention.TRANSACTION))
            stages.append(ExecutableStage(f"layers.{i}.attention", i, tuple(ops), acc, max_rows * H * 2 * 8))
            moe = True
        else:
            ops = ["norm_embedding", gemm, "gemm_bf16", "attention_mla_paged", "kv_pages"]
            if tp_world > 1:
                ops.append("collective_allreduce")
            acc = (_weights(f"layers.{i}.attn"), ResourceAccess(f"kv.{i}", AccessMode.READ_WRITE, ResourceRetention.TRANSACTION))
            stages.append(ExecutableStage(f"layers.{i}.attention", i, tuple(ops), acc, max_rows * H * 2 * 6))
            moe = cfg.is_moe_layer(i)
        if moe:
            ops = ["norm_embedding", "router_plan", expert_gemm, gemm]
            if not v4 and weight_format == "bf16" and not streamed_experts:
                ops.append("router_static_slots")      # decode-sized batches: fixed per-expert row slots
            if v4:
                ops.append("hyper_connection")
            if expert_dispatch:
                ops.append("expert_dispatch")
            elif tp_world > 1:
                ops.append("collective_allreduce")
            if streamed_experts:
                ops.append("expert_slot_table")
            acc = (_weights(f"layers.{i}.router"), _weights(f"layers.{i}.shared_experts"),
                   _weights(f"layers.{i}.experts", streamed=streamed_experts))
            stages.append(ExecutableStage(f"layers.{i}.moe", i, tuple(ops), acc, max_rows * cfg.topk * H * 2 * 2))
        else:
            ops = ["norm_embedding", gemm] + (["collective_allreduce"] if tp_world > 1 else [])
            stages.append(ExecutableStage(f"layers.{i}.ffn", i, tuple(ops), (_weights(f"layers.{i}.ffn"),),
                                          max_rows * cfg.dense_inter * 2))
    head_ops = ["norm_embedding", "gemm_bf16", "sampling_greedy"]
    if v4:
        head_ops.append("hyper_connection")
    if tp_world > 1:
        head_ops.append("collective_vocab_argmax")
    stages.append(ExecutableStage("head", -1, tuple(head_ops), (_weights("final_norm"), _weights("lm_head"))))
    if speculative:
        if not v4 and not getattr(cfg, "n_mtp_layers", 0):
            raise PlanError("speculative decoding needs a proposal (MTP) stage, the model has none")
        stages.append(ExecutableStage("proposal", n_layers, tuple(head_ops) + (gemm,), (_weights("mtp.0"),)))
    needed = set()
    for s in stages:
        needed.update(s.operators)
    registry.require(needed, getattr(cfg, "name", "deepseek-v4"))
    resolved = [ResolvedStage(j, s, (j - 1,) if j else ()) for j, s in enumerate(stages)]
    suspends = tuple(j for j, s in enumerate(stages) if any(a.streamed for a in s.accesses))
    return ModelPlan(getattr(cfg, "name", "deepseek-v4"), resolved, frozenset(needed),
                     max((s.workspace_bytes for s in stages), default=0), suspends)


# ---------------------------------------------------------------------------------------- materialization boundary
class Placement(Enum):
    DEVICE_ARENA = "device_arena"      # a stable slot of a routed-expert arena
    HOST_PINNED = "host_pinned"        # staged in pinned host memory only (prefetch)


class PreparationKind(Enum):
    RESIDENT = "resident"              # already usable: nothing to wait for
    TRANSFER = "transfer"              # a read and/or an upload is required first


@dataclass(frozen=True)
class MaterializationRequest:
    key: MaterializationKey
    placement: Placement
    bytes: int
    required: bool = True              # False: prefetch, may be dropped under pressure


@dataclass(frozen=True)
class Preparation:
    request: MaterializationRequest
    kind: PreparationKind
    slot: Optional[int] = None         # resident: the slot that holds it
    generation: int = 0


def requests_for_stage(stage: ExecutableStage, keys: Sequence[MaterializationKey], bytes_each: int,
                       required: bool = True) -> List[MaterializationRequest]:
    """The materialization requests a suspended stage raises for its streamed resources."""
    if not any(a.streamed for a in stage.accesses):
        raise PlanError(f"stage {stage.name} has no streamed resource")
    return [MaterializationRequest(k, Placement.DEVICE_ARENA, bytes_each, required) for k in keys]
