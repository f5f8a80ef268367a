"""Command-line entry points on the CPU."""
import json
import subprocess
import sys


def run(*args):
    p = subprocess.run([sys.executable, "-m", "ferrule_b200", *args], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout


def test_cli_fixture_inspect_generate_bench(tmp_path):
    d = str(tmp_path / "fx")
    out = json.loads(run("make-fixture", "--out", d, "--expert-format", "mxfp4", "--dense-format", "fp8_block"))
    assert out["params"] > 0
    ins = json.loads(run("inspect-weightpack", d, "--json", "--limit", "500"))
    fmts = {t["name"]: t["format"] for t in ins["tensors"]}
    assert fmts["model.layers.1.mlp.experts.0.gate_proj.weight"] == "mxfp4"
    assert fmts["model.layers.0.self_attn.o_proj.weight"] == "fp8_block" and ins["family"] == "deepseek_hf"
    info = json.loads(run("info", "--model-dir", d))
    assert info["checkpoint"]["roles"]["expert_gate"] == 32 and info["native_library_built"]
    common = ["--device", "cpu", "--ctx-size", "256", "--max-seqs", "2", "--page-size", "16"]
    g1 = json.loads(run("generate", "--model-dir", d, "--tokens", "5,6,7", "--max-tokens", "4", *common))
    g2 = json.loads(run("generate", "--model-dir", d, "--tokens", "5,6,7", "--max-tokens", "4", *common))
    assert g1["tokens"] == g2["tokens"] and len(g1["tokens"]) == 4 and g1["finish_reason"] == "length"
    rep = json.loads(run("bench-interactive", "--preset", "tiny-fixture", "--turns", "2", "--prompt-len", "6",
                         "--max-tokens", "3", *common))
    assert rep["report_version"] == 2 and len(rep["turns"]) == 2
    assert rep["turns"][1]["prompt_tokens"] > rep["turns"][0]["prompt_tokens"]        # the session was continued
    assert rep["shutdown_residual"] == {"kv_used_pages": 0, "grants": 0}
    sm = json.loads(run("expert-stream-smoke", d, "--device", "cpu", "--device-mb", "8"))
    assert sm["ok"] and sm["registry"]["published"] == sm["experts"]


def test_cli_golden_trace_parity_and_chunk_sweep(tmp_path):
    common = ["--preset", "tiny-fixture", "--device", "cpu", "--ctx-size", "256", "--max-seqs", "4", "--page-size", "16"]
    gold = str(tmp_path / "golden.json")
    rep = json.loads(run("bench-interactive", "--turns", "2", "--prompt-len", "6", "--max-tokens", "5",
                         "--write-golden", gold, *common))
    assert rep["golden_written"] == gold
    again = json.loads(run("bench-interactive", "--turns", "2", "--prompt-len", "6", "--max-tokens", "5",
                           "--golden", gold, *common))
    assert again["golden_match"] and again["golden"]["turns_compared"] == 2
    # a golden trace that differs is reported with the first diverging position, exit code 2
    g = json.load(open(gold))
    g["turns"][1]["tokens"][2] = (g["turns"][1]["tokens"][2] + 1) % 1000
    json.dump(g, open(gold, "w"))
    p = subprocess.run([sys.executable, "-m", "ferrule_b200", "bench-interactive", "--turns", "2", "--prompt-len", "6",
                        "--max-tokens", "5", "--golden", gold, *common], capture_output=True, text=True, timeout=300)
    assert p.returncode == 2
    bad = json.loads(p.stdout)
    assert bad["golden"]["first_divergence"]["turn"] == 1 and bad["golden"]["first_divergence"]["index"] == 2
    # prompt / token parity file
    cases = str(tmp_path / "cases.json")
    toks = rep["turns"][0]["tokens"]
    first_prompt_run = json.loads(run("generate", "--tokens", "9,8,7", "--max-tokens", "4", *common))
    json.dump({"cases": [{"prompt_tokens": [9, 8, 7], "expected_tokens": first_prompt_run["tokens"]}]}, open(cases, "w"))
    par = json.loads(run("generation-parity", "--cases", cases, *common))
    assert par["all_match"] and par["cases"][0]["generated"] == first_prompt_run["tokens"] and len(toks) == 5
    sw = json.loads(run("chunk-sweep", "--chunks", "8", "32", "--requests", "2", "--prompt-len", "40", "--max-tokens", "3",
                        *common))
    assert [r["prefill_chunk"] for r in sw["sweep"]] == [8, 32]
    assert sw["sweep"][0]["prefill_chunks"] > sw["sweep"][1]["prefill_chunks"]


import pytest


@pytest.mark.parametrize("preset", ["tiny-fixture", "tiny-v4"])
def test_chat_continues_one_retained_session_and_answers_the_slash_commands(preset):
    script = "\n".join(["hello there", "/stats", "/ctx", "and again", "/stats", "/experts", "/reset", "/stats", "fresh start",
                        "/exit"]) + "\n"
    p = subprocess.run([sys.executable, "-m", "ferrule_b200", "chat", "--preset", preset, "--device", "cpu",
                        "--ctx-size", "256", "--max-seqs", "2", "--page-size", "16", "--max-tokens", "4"],
                       input=script, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    out = p.stdout
    stats = [l for l in out.splitlines() if "position=" in l]
    assert len(stats) == 3
    pos = [int(l.split("position=")[1].split()[0]) for l in stats]
    turns = [int(l.split("turns=")[1].split()[0]) for l in stats]
    assert turns == [1, 2, 0] and 0 < pos[0] < pos[1] and pos[2] == 0, "the second turn extended the first; /reset emptied it"
    assert "session reset." in out and "expert report not available." in out
    ctx_line = next(l for l in out.splitlines() if l.startswith("> context") or "context " in l)
    assert "/ 256 tokens" in ctx_line


def test_reference_style_invocations(tmp_path):
    """Positional model directory, -p / -n, the deepseek-v4-generate command (drafter of the checkpoint unless
    --no-speculative) and the reference's serve flag names."""
    d = str(tmp_path / "v4")
    json.loads(run("make-fixture", "--family", "v4", "--out", d, "--layers", "2", "--proposal-stages", "1", "--plain"))
    common = ["--device", "cpu", "--ctx-size", "64", "--max-active-sequences", "2", "--page-size", "16",
              "--prefill-chunk-size", "8"]
    a = json.loads(run("deepseek-v4-generate", d, "--tokens", "5,9,11", "-n", "5", "--no-stop-eos", "--json", *common))
    b = json.loads(run("deepseek-v4-generate", d, "--tokens", "5,9,11", "-n", "5", "--no-stop-eos", "--no-speculative",
                       "--json", *common))
    assert a["tokens"] == b["tokens"] and len(a["tokens"]) == 5
    assert a["report_version"] == 2 and a["speculative"]["drafted"] > 0 and "speculative" not in b
    assert a["runner"]["proposal_blocks"] > 0 and b["runner"]["proposal_blocks"] == 0
    info = json.loads(run("info", d))
    assert info["checkpoint"]["family"] == "deepseek_v4"
    p = subprocess.run([sys.executable, "-m", "ferrule_b200", "generate", d, "-p", "hi", "-n", "2", "--chat", "--verbose-tokens",
                        "--warmup-tokens", "2", *common], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and p.stderr.count("[token ") == 2, p.stderr[-500:]
    helptext = run("serve", "--help")
    for flag in ("--served-model-name", "--request-queue-capacity", "--event-queue-capacity", "--admission-timeout-secs",
                 "--decode-cohort-target", "--decode-cohort-max-deferrals", "--chat-template", "--kv-cache-mb"):
        assert flag in helptext, flag


def test_max_layers_binds_a_prefix_of_the_checkpoint(tmp_path):
    from ferrule_b200.io.checkpoint import load_deepseek_hf
    from ferrule_b200.io.v4_checkpoint import load_v4_hf
    d4, ds = str(tmp_path / "v4"), str(tmp_path / "ds")
    run("make-fixture", "--family", "v4", "--out", d4, "--plain", "--proposal-stages", "1")
    run("make-fixture", "--out", ds)
    w = load_v4_hf(d4, max_layers=2)
    assert len(w.layers) == 2 and w.cfg.n_layers == 2 and w.cfg.compress_ratios == (0, 4) and w.proposal is None
    assert load_v4_hf(d4).proposal is not None and len(load_v4_hf(d4, max_layers=9).layers) == 3
    full = load_deepseek_hf(ds)
    part = load_deepseek_hf(ds, max_layers=1)
    assert len(part.layers) == 1 and part.cfg.n_layers == 1 and not part.mtp and len(full.layers) == 2
    out = json.loads(run("generate", ds, "--device", "cpu", "--tokens", "5,9", "-n", "3", "--ignore-eos", "--ctx-size", "64",
                         "--page-size", "16", "--max-seqs", "2", "--max-layers", "1"))
    assert len(out["tokens"]) == 3
