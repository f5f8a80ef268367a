"""Fail-closed plan compilation, stage types, the validating executor and the owner-thread guard."""
import threading

import pytest

from ferrule_b200.models import config as C
from ferrule_b200.models import v4_model as M4
from ferrule_b200.runtime import plan as P
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.execution import ExecutionOutput, RowOutput
from ferrule_b200.runtime.facade import AffinityError, InferenceCompletionOwner, NativeExecutor
from ferrule_b200.runtime.runner import Complete, MockRunner
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest

ALL = P.ProviderRegistry(P.OPERATOR_GROUPS)


def test_plan_lists_stages_and_operators_for_v2_lite():
    cfg = C.deepseek_v2_lite()
    plan = P.compile_model_plan(cfg, ALL, tp_world=8)
    names = [s.stage.name for s in plan.stages]
    assert names[0] == "embedding" and names[-1] == "head"
    assert names.count("layers.0.ffn") == 1 and "layers.1.moe" in names and len(plan.stages) == 2 + 2 * 27
    assert {"gemm_bf16", "attention_mla_paged", "router_plan", "collective_allreduce", "collective_vocab_argmax"} <= plan.operators
    assert all(s.dependencies == ((s.index - 1,) if s.index else ()) for s in plan.stages)
    assert plan.suspends_at == ()


def test_plan_fails_closed_and_names_the_missing_group():
    cfg = C.deepseek_v3()
    reg = P.ProviderRegistry(set(P.OPERATOR_GROUPS) - {"gemm_fp8_block", "expert_slot_table"})
    with pytest.raises(P.PlanError) as e:
        P.compile_model_plan(cfg, reg, weight_format="fp8_block", streamed_experts=True)
    assert "gemm_fp8_block" in str(e.value) and "expert_slot_table" in str(e.value)
    ok = P.compile_model_plan(cfg, ALL, weight_format="fp8_mxfp4", streamed_experts=True, speculative=True)
    assert "gemm_mxfp4_experts" in ok.operators and len(ok.suspends_at) == 58 and ok.stages[-1].stage.name == "proposal"
    with pytest.raises(P.PlanError):
        P.compile_model_plan(C.deepseek_v2_lite(), ALL, speculative=True)       # no MTP stage in that model
    with pytest.raises(P.PlanError):
        P.compile_model_plan(cfg, ALL, weight_format="int3")


def test_v4_plan_needs_hyper_connections_and_sparse_attention():
    cfg = M4.tiny_v4()
    plan = P.compile_model_plan(cfg, ALL)
    assert {"hyper_connection", "attention_sparse_selection", "kv_compressor"} <= plan.operators
    with pytest.raises(P.PlanError) as e:
        P.compile_model_plan(cfg, P.ProviderRegistry(set(P.OPERATOR_GROUPS) - {"hyper_connection"}))
    assert "hyper_connection" in str(e.value)
    st = [s.stage for s in plan.stages if s.stage.name == "layers.1.moe"][0]
    with pytest.raises(P.PlanError):
        P.requests_for_stage(st, [], 10)                                         # nothing streamed in this plan


def test_registry_probe_reports_a_manifest():
    reg = P.ProviderRegistry.from_library()
    man = reg.manifest()
    assert set(man) == set(P.OPERATOR_GROUPS)
    if man["gemm_bf16"]:                       # the library is built in this tree
        assert man["attention_mla_paged"] and man["hyper_connection"] and man["expert_dispatch"]


def _engine(runner):
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=16, ctx_size=256)
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=64, page_size=16))


def test_native_executor_validates_and_passes_through():
    ex = NativeExecutor(MockRunner())
    eng = _engine(ex)
    eng.submit(GenerateRequest("a", list(range(1, 20)), max_new_tokens=5))
    ev = []
    eng.run_until_idle(ev.append)
    assert len([e for e in ev if isinstance(e, TokenEvent)]) == 5
    assert ex.validated_batches > 0 and ex.validated_outputs == ex.validated_batches


def test_native_executor_rejects_malformed_backend_output():
    class Bad(MockRunner):
        def execute(self, txn_id):
            out = super().execute(txn_id)
            rows = list(out.output.rows)
            return Complete(ExecutionOutput(rows + [RowOutput(rows[-1].row, [1], [0.0])]))   # duplicate row

    eng = _engine(NativeExecutor(Bad()))
    eng.submit(GenerateRequest("a", [1, 2, 3], max_new_tokens=2))
    eng.run_until_idle(lambda e: None)
    assert eng.last_error is not None and eng.stats.aborted_transactions >= 1


def test_owner_guard_refuses_other_threads():
    owner = InferenceCompletionOwner(_engine(MockRunner()))
    owner.submit(GenerateRequest("a", [1, 2, 3], max_new_tokens=3))
    seen = []
    t = threading.Thread(target=lambda: seen.append(_try(owner)))
    t.start()
    t.join()
    assert seen == ["refused"]
    toks = []
    owner.run_until_idle(lambda e: toks.append(e) if isinstance(e, TokenEvent) else None)
    assert len(toks) == 3 and owner.steps > 0


def _try(owner):
    try:
        owner.run_once(lambda e: None)
        return "ran"
    except AffinityError:
        return "refused"
