"""Stage tables and debug taps of the forward pass (environment switches read when the runner is built)."""
import json
import logging

import pytest
import torch

from ferrule_b200.models import config as C
from ferrule_b200.models import weights as W
from ferrule_b200.models.runner import DeepSeekRunner
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest
from ferrule_b200.utils.stage_profile import DebugTap, StageProfiler


def test_marks_build_a_table():
    p = StageProfiler("cpu")
    for layer in range(2):
        p.mark(layer, "attn")
        p.mark(layer, "moe")
    p.mark(2, None)
    p.mark(0, "attn")
    p.mark(0, None)
    rows = {(r["layer"], r["stage"]): r for r in p.table()}
    assert set(rows) == {(0, "attn"), (0, "moe"), (1, "attn"), (1, "moe")}
    assert rows[(0, "attn")]["calls"] == 2 and rows[(1, "moe")]["calls"] == 1
    assert abs(sum(r["share"] for r in rows.values()) - 1.0) < 1e-2
    by = p.by_stage()
    assert {r["stage"] for r in by} == {"attn", "moe"} and by[0]["total_us"] >= by[1]["total_us"]
    p.reset()
    assert p.table() == []


def _serve(device, monkeypatch, tmp_path, dtype):
    monkeypatch.setenv("FERRULE_PROFILE", "1")
    monkeypatch.setenv("FERRULE_PREFILL_PROGRESS", "1")
    monkeypatch.setenv("FERRULE_DEBUG_STAGE_DUMP_DIR", str(tmp_path / "taps"))
    monkeypatch.setenv("FERRULE_DEBUG_LAYER", "1")
    cfg = C.tiny_fixture() if device == "cpu" else C.smoke_gpu()
    w = W.random_weights(cfg, device=device, dtype=dtype, seed=2, std=0.05)
    runner = DeepSeekRunner(w, n_pages=32, page_size=16, max_rows=64, max_seqs=4, max_seq_len=128, device=device,
                            enable_mtp=False)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=8,
                            ctx_size=128)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
    g = torch.Generator().manual_seed(3)
    for i, n in enumerate((9, 14)):
        eng.submit(GenerateRequest(f"r{i}", torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(),
                                   max_new_tokens=4, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=2000)
    return cfg, runner, [e for e in ev if isinstance(e, TokenEvent)]


def test_runner_collects_stage_table_taps_and_prefill_progress_on_cpu(monkeypatch, tmp_path, caplog):
    with caplog.at_level(logging.INFO, logger="ferrule_prefill"):
        cfg, runner, toks = _serve("cpu", monkeypatch, tmp_path, torch.float32)
    assert len(toks) == 8 and not runner.use_graphs
    obs = runner.observability()
    stages = {r["stage"] for r in obs["stage_table"]}
    assert {"attn", "attn.reduce", "moe", "ffn", "ffn.reduce"} <= stages
    layers = {r["layer"] for r in obs["stage_table_layers"]}
    assert layers == set(range(cfg.n_layers))
    assert all(r["calls"] > 0 and r["total_us"] > 0 for r in obs["stage_table_layers"])
    json.dumps(obs["stage_table"])
    files = sorted((tmp_path / "taps").glob("*.pt"))
    assert files and all("_layer1_" in f.name for f in files)
    assert {f.name.split("_layer1_")[1] for f in files} == {"attn_out.pt", "layer_out.pt"}
    t = torch.load(files[0])
    assert t.dim() == 2 and t.shape[1] == cfg.hidden and torch.isfinite(t).all()
    assert any("prefill slot=" in r.getMessage() for r in caplog.records)
    # without the switches a runner has neither
    for k in ("FERRULE_PROFILE", "FERRULE_PREFILL_PROGRESS", "FERRULE_DEBUG_STAGE_DUMP_DIR", "FERRULE_DEBUG_LAYER"):
        monkeypatch.delenv(k)
    plain = DeepSeekRunner(W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2), n_pages=8, page_size=16,
                           max_rows=32, max_seqs=2, max_seq_len=64, device="cpu", enable_mtp=False)
    assert plain.profiler is None and plain.debug_tap is None and "stage_table" not in plain.observability()


def test_debug_tap_filters():
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        tap = DebugTap(d, layer=2, stage="attn_out")
        tap.write(1, "attn_out", torch.ones(2, 4))
        tap.write(2, "layer_out", torch.ones(2, 4))
        tap.next_step()
        tap.write(2, "attn_out", torch.ones(2, 4, dtype=torch.bfloat16))
        assert len(tap.written) == 1 and tap.written[0].endswith("step00001_layer2_attn_out.pt")
        assert torch.load(tap.written[0]).dtype == torch.float32


@pytest.mark.gpu
def test_runner_collects_stage_table_on_the_kernels(monkeypatch, tmp_path):
    cfg, runner, toks = _serve("cuda", monkeypatch, tmp_path, torch.bfloat16)
    assert len(toks) == 8 and not runner.use_graphs
    obs = runner.observability()
    stages = {r["stage"] for r in obs["stage_table"]}
    assert {"attn.norm", "attn.qkv", "attn.prep+absorb", "attn.core", "attn.uv", "attn.o_proj+norm", "moe", "moe.reduce",
            "ffn"} <= stages
    assert all(r["total_us"] > 0 for r in obs["stage_table"])
    assert sorted((tmp_path / "taps").glob("*_layer1_layer_out.pt"))
    from ferrule_b200.ops import _lib
    assert _lib.read_status()[0] == 0


def test_v4_runner_stage_table_on_cpu_and_on_the_kernel_path_logic(monkeypatch):
    import v4_cpu_shim as shim
    from ferrule_b200.models import v4_model as M
    from ferrule_b200.models.v4_runner import V4Runner
    monkeypatch.setenv("FERRULE_PROFILE", "1")
    cfg = M.tiny_v4()
    w = M.random_v4_weights(cfg, seed=3)
    for kernel_path in (False, True):
        runner = V4Runner(w, n_pages=32, page_size=16, max_seqs=4, max_seq_len=128, max_rows=64)
        if kernel_path:
            runner.is_cuda = True
            runner.fwd = shim.install(M.V4Cuda(w, 4, 128, max_rows=64))
            runner.fwd.prof = runner.profiler
        sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=12,
                                ctx_size=128)
        eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
        eng.submit(GenerateRequest("r", list(range(3, 14)), max_new_tokens=3, ignore_eos=True))
        eng.run_until_idle(lambda e: None, max_steps=500)
        stages = {r["stage"] for r in runner.observability()["stage_table"]}
        want = {"attn.proj", "attn.select", "attn.core", "attn.out", "moe", "head"} if kernel_path else {"attn", "moe", "head"}
        assert stages == want
        assert {r["layer"] for r in runner.observability()["stage_table_layers"]} == set(range(cfg.n_layers + 1))
