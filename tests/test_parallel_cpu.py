"""Multi-process host-side parallel paths on the gloo backend (no GPU): pipeline stages over send/recv,
tensor-parallel reference collectives, rank-failure detection through a short process-group timeout."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script: str, world: int, port: int, timeout: int = 180):
    path = os.path.join(ROOT, "tests", f"_tmp_pp_{port}.py")
    with open(path, "w") as f:
        f.write(textwrap.dedent(script))
    try:
        env = dict(os.environ, PYTHONPATH=ROOT, FERRULE_NO_CUDA="1")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
               "--master-addr", "127.0.0.1", "--master-port", str(port), path]
        return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT, env=env)
    finally:
        os.remove(path)


def test_pipeline_two_stages_equal_single_process():
    p = _run('''
        import os, torch, torch.distributed as dist
        from ferrule_b200.models import config as C, weights as W, deepseek as D
        from ferrule_b200.parallel.pp import PipelineParallel, stage_weights
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        cfg = C.tiny_fixture()
        w = W.random_weights(cfg, device="cpu", seed=0)
        page = 16
        def batch(lens, new, seed):
            g = torch.Generator().manual_seed(seed)
            ids, pos, slot, rseq, lrows = [], [], [], [], []
            bt = torch.zeros(len(lens), 8, dtype=torch.int32)
            pc = 1
            for s, (n0, nn) in enumerate(zip(lens, new)):
                for j in range((n0 + nn + page - 1) // page):
                    bt[s, j] = pc; pc += 1
                for j in range(nn):
                    p_ = n0 + j
                    ids.append(int(torch.randint(0, cfg.vocab_size, (1,), generator=g))); pos.append(p_)
                    slot.append(int(bt[s, p_ // page]) * page + p_ % page); rseq.append(s)
                lrows.append(len(ids) - 1)
            t = lambda v, dt: torch.tensor(v, dtype=dt)
            return D.DeviceBatch(t(ids, torch.int32), t(pos, torch.int32), t(slot, torch.int64), t(rseq, torch.int32),
                                 t(pos, torch.int32), bt, t(lrows, torch.int32), len(ids), len(lrows))
        full = D.ReferenceForward(w, D.KvPool(cfg, 32, page, "cpu", dtype=torch.float32))
        ws = stage_weights(w, rank, world)
        stage = D.ReferenceForward(ws, D.KvPool(ws.cfg, 32, page, "cpu", dtype=torch.float32))
        pp = PipelineParallel(rank, world)
        ok = True
        lens, new = [0, 0], [19, 7]
        for step in range(3):
            b = batch(lens, new, step)
            want = full.forward(b)
            ids, vals = pp.step(stage, b, cfg.hidden, torch.float32, cuda=False)
            ok &= bool(torch.equal(ids.long(), want.argmax(-1))) and bool(torch.allclose(vals, want.max(-1).values, atol=1e-4))
            lens = [l + n for l, n in zip(lens, new)]; new = [1, 1]
        # micro-batched decode: two row ranges in flight
        pp2 = PipelineParallel(rank, world, microbatches=2)
        b = batch(lens, [1, 1], 9)
        want = full.forward(b)
        ids, vals = pp2.step(stage, b, cfg.hidden, torch.float32, cuda=False)
        ok &= bool(torch.equal(ids.long(), want.argmax(-1)))
        print("PP_OK" if ok else "PP_BAD", rank, flush=True)
        dist.destroy_process_group()
    ''', 2, 29611)
    assert p.stdout.count("PP_OK") == 2, p.stdout[-2000:] + p.stderr[-3000:]


def test_rank_that_never_joins_is_detected_by_timeout():
    """Failure made on the host: rank 1 exits between steps; rank 0's next collective ends with an error after the
    short process-group timeout instead of hanging."""
    p = _run('''
        import datetime, os, sys, torch, torch.distributed as dist
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
        rank = dist.get_rank()
        t = torch.ones(4)
        dist.all_reduce(t)                       # step 0: everyone is here
        if rank == 1:
            print("RANK1_LEAVES", flush=True)
            os._exit(0)                          # leaves between steps, nothing in flight
        try:
            dist.all_reduce(t)                   # step 1: the peer is gone
            print("NO_ERROR", flush=True)
        except Exception as exc:
            print("DETECTED", type(exc).__name__, flush=True)
        os._exit(0)
    ''', 2, 29612, timeout=120)
    assert "DETECTED" in p.stdout and "NO_ERROR" not in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]


def test_tensor_parallel_reference_on_gloo_equals_single_process():
    """Heads, FFN inner dims, experts and the vocabulary sharded over two CPU ranks: the engine's greedy stream
    equals the single-process one (reference forward + gloo all-reduce / all-gather)."""
    p = _run('''
        import torch, torch.distributed as dist
        from ferrule_b200.models import config as C, weights as W
        from ferrule_b200.models.runner import DeepSeekRunner
        from ferrule_b200.parallel.tp import TensorParallel
        from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
        from ferrule_b200.runtime.scheduler import SchedulerConfig
        from ferrule_b200.runtime.session import GenerateRequest
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        cfg = C.tiny_fixture()
        def run(w, tp):
            runner = DeepSeekRunner(w, n_pages=32, page_size=16, max_rows=128, max_seqs=4, max_seq_len=256, device="cpu",
                                    tp=tp, enable_mtp=False)
            sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=32,
                                    ctx_size=256)
            eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
            g = torch.Generator().manual_seed(5)
            for i, n in enumerate((21, 40)):
                eng.submit(GenerateRequest(f"r{i}", torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(),
                                           max_new_tokens=6, ignore_eos=True))
            ev = []
            eng.run_until_idle(ev.append, max_steps=2000)
            assert eng.last_error is None, eng.last_error
            return [(e.request_id, e.token) for e in ev if isinstance(e, TokenEvent)]
        want = run(W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32), None)
        got = run(W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32, tp_rank=rank, tp_world=world),
                  TensorParallel(rank, world, "cpu", fused=False))
        print("TP_OK" if got == want and len(want) == 12 else "TP_BAD", rank, flush=True)
        dist.destroy_process_group()
    ''', 2, 29613)
    assert p.stdout.count("TP_OK") == 2, p.stdout[-2000:] + p.stderr[-3000:]


def test_engine_over_two_pipeline_stages_streams_the_single_process_tokens():
    """The whole engine (scheduler, KV transactions, chunked prefill, decode) on two pipeline stages: every rank
    runs the same owner loop, the last stage's greedy tokens reach all of them, and the token streams equal
    those of one process holding all layers."""
    p = _run('''
        import torch, torch.distributed as dist
        from ferrule_b200.models import config as C, weights as W
        from ferrule_b200.models.runner import DeepSeekRunner
        from ferrule_b200.parallel.pp import PipelineParallel, stage_weights
        from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
        from ferrule_b200.runtime.scheduler import SchedulerConfig
        from ferrule_b200.runtime.session import GenerateRequest
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        cfg = C.tiny_fixture().with_(n_mtp_layers=0)
        w = W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32)
        def run(runner):
            sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=48,
                                    prefill_chunk_size=16, ctx_size=128)
            eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
            g = torch.Generator().manual_seed(3)
            for i in range(3):
                eng.submit(GenerateRequest(f"r{i}", torch.randint(0, cfg.vocab_size, (9 + 11 * i,), generator=g).tolist(),
                                           max_new_tokens=6, ignore_eos=True))
            ev = []
            eng.run_until_idle(ev.append)
            return {r: [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == r] for r in ("r0", "r1", "r2")}
        want = run(DeepSeekRunner(w, n_pages=32, page_size=16, max_rows=64, max_seqs=4, max_seq_len=128, device="cpu"))
        pp = PipelineParallel(rank, world, microbatches=2)
        got = run(DeepSeekRunner(stage_weights(w, rank, world), n_pages=32, page_size=16, max_rows=64, max_seqs=4,
                                 max_seq_len=128, device="cpu", pp=pp))
        print("PPE_OK" if got == want and all(len(v) == 6 for v in got.values()) else f"PPE_BAD {got} {want}", rank, flush=True)
        dist.destroy_process_group()
    ''', 2, 29613)
    assert p.stdout.count("PPE_OK") == 2, p.stdout[-2000:] + p.stderr[-3000:]


def test_serving_replica_over_two_tensor_parallel_ranks_mirrors_the_command_stream():
    """The serving worker on rank 0 and a follower on rank 1, each with its shard of a tensor-parallel model
    (reference forward, gloo): submissions and a cancellation reach both engines in the same order, both take
    the same steps, and the follower's token streams equal what the leader streamed to its clients."""
    p = _run('''
        import argparse, asyncio, json, torch, torch.distributed as dist
        from ferrule_b200.cli.main import _add_model_args, build_engine, replica_layout
        from ferrule_b200.parallel.mirror import follower_loop
        from ferrule_b200.runtime.engine import TokenEvent, FinishEvent
        from ferrule_b200.server.worker import ModelWorker, WorkerConfig
        from ferrule_b200.utils.tokenizer import load_tokenizer
        ap = argparse.ArgumentParser(); _add_model_args(ap)
        args = ap.parse_args(["--preset", "tiny-fixture", "--device", "cpu", "--max-seqs", "4", "--ctx-size", "256",
                              "--page-size", "16", "--max-batch-tokens", "64", "--prefill-chunk", "32"])
        layout, mirror = replica_layout(args)
        assert layout.tp_size == 2 and layout.pp is None
        if not mirror.is_leader:
            eng, _, _ = build_engine(args, layout)
            seen = {}
            def sink(ev):
                if isinstance(ev, TokenEvent):
                    seen.setdefault(ev.request_id, []).append(ev.token)
            steps = follower_loop(eng, mirror, sink)
            out = [None, None]
            dist.all_gather_object(out, {"steps": steps, "tokens": seen})
        else:
            tok = load_tokenizer(None)
            worker = ModelWorker(lambda: build_engine(args, layout)[0], tok, WorkerConfig(), mirror=mirror).start()
            async def one(i, n_out, cancel_after=None):
                g = torch.Generator().manual_seed(i)
                ids = torch.randint(0, 200, (17 + 9 * i,), generator=g).tolist()
                st = await worker.submit(text=None, token_ids=ids, max_tokens=n_out, stop=[], ignore_eos=True)
                toks = []
                while True:
                    ev = await st.next()
                    if ev.kind == "token" and ev.token is not None:
                        toks.append(ev.token)
                        if cancel_after is not None and len(toks) == cancel_after:
                            worker.cancel(st.request_id)
                    elif ev.kind in ("finish", "error"):
                        return st.request_id, toks, ev.kind
            async def all_():
                return await asyncio.gather(one(0, 6), one(1, 9), one(2, 40, cancel_after=3))
            res = asyncio.run(all_())
            worker.stop()
            steps = worker.steps
            out = [None, None]
            dist.all_gather_object(out, {"steps": steps, "tokens": {r: t for r, t, _ in res}})
            lead, foll = out[0], out[1]
            ok = lead["steps"] == foll["steps"] and len(lead["tokens"]) == 3
            for rid, toks in lead["tokens"].items():
                # the follower may see a few more tokens of the cancelled request than the client read
                ok = ok and foll["tokens"].get(rid, [])[:len(toks)] == toks and len(toks) >= 3
            ok = ok and [len(t) for t in lead["tokens"].values()][:2] == [6, 9]
            print("MIRROR_OK" if ok else "MIRROR_BAD", json.dumps(out), flush=True)
        dist.destroy_process_group()
    ''', 2, 29617)
    assert "MIRROR_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]


def test_engine_over_two_stages_of_two_tensor_ranks_each():
    """pp 2 x tp 2 on four CPU ranks through `build_parallel` (stage-major rank layout, one process group per
    stage and per tensor rank): the engine's greedy streams equal the single-process ones on every rank."""
    p = _run('''
        import torch, torch.distributed as dist
        from ferrule_b200.models import config as C, weights as W
        from ferrule_b200.models.runner import DeepSeekRunner
        from ferrule_b200.parallel.layout import build_parallel
        from ferrule_b200.parallel.pp import stage_weights
        from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
        from ferrule_b200.runtime.scheduler import SchedulerConfig
        from ferrule_b200.runtime.session import GenerateRequest
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        lay = build_parallel(rank, world, "cpu", pp=2, tp=2, microbatches=2, fused=False)
        assert (lay.pp_rank, lay.tp_rank) == divmod(rank, 2) and lay.tp_ranks == [2 * lay.pp_rank, 2 * lay.pp_rank + 1]
        cfg = C.tiny_fixture().with_(n_mtp_layers=0)
        def run(runner):
            sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=48,
                                    prefill_chunk_size=16, ctx_size=128)
            eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
            g = torch.Generator().manual_seed(3)
            for i in range(3):
                eng.submit(GenerateRequest(f"r{i}", torch.randint(0, cfg.vocab_size, (9 + 11 * i,), generator=g).tolist(),
                                           max_new_tokens=6, ignore_eos=True))
            ev = []
            eng.run_until_idle(ev.append, max_steps=2000)
            assert eng.last_error is None, eng.last_error
            return {r: [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == r] for r in ("r0", "r1", "r2")}
        want = run(DeepSeekRunner(W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32), n_pages=32,
                                  page_size=16, max_rows=64, max_seqs=4, max_seq_len=128, device="cpu"))
        w = W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32, tp_rank=lay.tp_rank, tp_world=2)
        got = run(DeepSeekRunner(stage_weights(w, lay.pp_rank, 2), n_pages=32, page_size=16, max_rows=64, max_seqs=4,
                                 max_seq_len=128, device="cpu", tp=lay.tp, pp=lay.pp))
        print("PPTP_OK" if got == want and all(len(v) == 6 for v in got.values()) else f"PPTP_BAD {got} {want}", rank, flush=True)
        dist.destroy_process_group()
    ''', 4, 29619, timeout=240)
    assert p.stdout.count("PPTP_OK") == 4, p.stdout[-2000:] + p.stderr[-3000:]


def test_sequence_parallel_reference_on_gloo_equals_single_process():
    """Tensor-parallel ranks that keep the residual stream sharded by rows between reduce-scatter and all-gather
    (row counts that do not divide by the world size included): the engine's greedy stream equals the
    single-process one, and equals the all-reduce form's."""
    p = _run('''
        import torch, torch.distributed as dist
        from ferrule_b200.models import config as C, weights as W
        from ferrule_b200.models.runner import DeepSeekRunner
        from ferrule_b200.parallel.tp import TensorParallel
        from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
        from ferrule_b200.runtime.scheduler import SchedulerConfig
        from ferrule_b200.runtime.session import GenerateRequest
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        cfg = C.tiny_fixture()
        def run(w, tp, sp):
            runner = DeepSeekRunner(w, n_pages=32, page_size=16, max_rows=128, max_seqs=4, max_seq_len=256, device="cpu",
                                    tp=tp, enable_mtp=False, sequence_parallel=sp)
            assert runner.sequence_parallel == (sp and tp is not None)
            sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=32,
                                    ctx_size=256)
            eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16))
            g = torch.Generator().manual_seed(5)
            for i, n in enumerate((21, 40, 7)):
                eng.submit(GenerateRequest(f"r{i}", torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(),
                                           max_new_tokens=6, ignore_eos=True))
            ev = []
            eng.run_until_idle(ev.append, max_steps=2000)
            assert eng.last_error is None, eng.last_error
            return [(e.request_id, e.token) for e in ev if isinstance(e, TokenEvent)]
        want = run(W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32), None, False)
        shard = lambda: W.random_weights(cfg, device="cpu", seed=0, dtype=torch.float32, tp_rank=rank, tp_world=world)
        tp = TensorParallel(rank, world, "cpu", fused=False)
        assert tp.row_range(7) == ((0, 4) if rank == 0 else (4, 7)) and tp.row_range(1) == ((0, 1) if rank == 0 else (1, 1))
        got_sp = run(shard(), tp, True)
        got_ar = run(shard(), tp, False)
        ok = got_sp == want and got_ar == want and len(want) == 18
        print("SP_OK" if ok else "SP_BAD", rank, flush=True)
        dist.destroy_process_group()
    ''', 2, 29641)
    assert p.stdout.count("SP_OK") == 2, p.stdout[-2000:] + p.stderr[-3000:]
