"""Tensor-parallel path on 2 GPUs: fused collectives vs NCCL and TP model vs single GPU."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_selftest_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(ROOT, "tests", "dist", "tp_selftest.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert lines, p.stdout[-2000:] + p.stderr[-4000:]
    res = json.loads(lines[-1])
    assert res["ok"], res
    assert p.returncode == 0
    assert res["fused_calls"] > 0


def test_expert_parallel_dispatch_combine_two_ranks():
    """Token-sharded expert parallelism: fused peer-memory dispatch/combine and the NCCL all-to-all baseline
    against a single-device oracle (ragged token counts, skewed routing, all-gather of the outputs)."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29519", os.path.join(ROOT, "tests", "dist", "ep_selftest.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert lines, p.stdout[-2000:] + p.stderr[-4000:]
    res = json.loads(lines[-1])
    assert res["ok"], res
    assert p.returncode == 0
    assert res["device_status"][0] == 0


def test_selftest_two_ranks_in_switch_collectives():
    """The same checks with the all-reduces, reduce-scatter and all-gather running through the NVLink switch
    (multimem); skipped when the node offers no multicast."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29521", os.path.join(ROOT, "tests", "dist", "tp_selftest.py"),
           "--collective", "multimem", "--payload", "bf16"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    if "offers no NVLink multicast" in p.stderr + p.stdout:
        pytest.skip("no NVLS on this node")
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert lines, p.stdout[-2000:] + p.stderr[-4000:]
    res = json.loads(lines[-1])
    assert res["ok"], res
    assert res["checks"]["allreduce_bits_equal_across_ranks"] and res["checks"]["ep_model_tokens_match"]


def test_pipeline_parallel_engine_two_stages_on_gpus():
    """Two pipeline stages on two GPUs (NCCL send / recv on a side stream, two row ranges in flight): the engine's
    token streams equal those of one GPU holding the whole model."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29523", os.path.join(ROOT, "tests", "dist", "pp_selftest.py"),
           "--pp", "2"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert lines, p.stdout[-2000:] + p.stderr[-4000:]
    res = json.loads(lines[-1])
    assert res["ok"] and res["requests_equal"] == 5 and res["sends"] > 0, res

