#!/usr/bin/env python
"""Headline benchmark: greedy decode throughput of the DeepSeek-V2-Lite-shape MoE model.

  python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)
  python bench.py --impl reference ...                   (the reference arm)

Config: 27 layers, hidden 2048, 16 heads, MLA (kv_lora 512, nope 128, rope 64, v 128), layer 0
dense (inter 10944), 26 MoE layers (64 routed + 2 shared experts, top-6, inter 1408), vocab
102400, bf16, random-init N(0, 0.02), batch 32, 512-token uniform-random prompts, paged KV with
64-token pages.  One "step" is one decode step of the whole batch (32 new tokens).  N > 1 runs
tensor parallel over N ranks on the same batch (strong scaling).

Two numbers over the same K decode steps (the same sequences, the same context window, which grows by
one token per step):
  e2e   : the K steps driven through the public engine API (`Engine.step`): scheduler, KV
          reservation/commit, one pinned host->device copy of every step's inputs, the captured graph,
          one device->host read of the greedy tokens, token publication.
  value : the K steps again, from the same starting state, without the host: after every graph replay
          one small kernel feeds the greedy tokens back and moves positions and KV write slots on
          (device time of the kernels only, CUDA events).
Every step streams the full weight set (31 GB, far larger than the 126 MB L2), so no L2 flush is
needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

BASELINE_TOK_S = 16.0        # the reference's only stated throughput figure (a target, not a measurement)


def reference_arm() -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a Rust workspace (no setup.py/pyproject.toml; pip install fails with "
                       "'not installable'), needs cargo nightly-2026-08-01 and a network CUTLASS checkout, and "
                       "its plan compiler fails closed on sm_100",
    }))


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None
        self.gpu_index = gpu_index

    def start(self) -> None:
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:  # noqa: BLE001 - sampling is best effort
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:  # noqa: BLE001
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--model", default="deepseek-v2-lite")
    ap.add_argument("--weight-format", default="bf16", choices=["bf16", "fp8_block", "fp8_mxfp4"],
                    help="bf16 is the headline configuration; the FP8 formats are reported with their own dtype")
    ap.add_argument("--shard-as", type=int, default=0,
                    help="debug only: on one GPU, hold rank 0's shard of a TP-N layout and skip the collectives "
                         "(compute-only time of one rank; the result is marked invalid)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override layer count (result is marked invalid)")
    ap.add_argument("--ar-payload", default="bf16", choices=["fp32", "bf16"],
                    help="what the fused all-reduces push over NVLink: bf16 partials (default, as bf16 all-reduces do) or fp32")
    ap.add_argument("--no-fused", action="store_true", help="use the NCCL baseline collectives instead of fused kernels")
    ap.add_argument("--mc-push", action="store_true",
                    help="ll collectives: push partials through the NVLink multicast address (one store reaches all ranks)")
    ap.add_argument("--collective", default="ll", choices=["ll", "multimem"],
                    help="fused all-reduces: tagged peer pushes (ll) or reduce + broadcast inside the NVLink switch")
    ap.add_argument("--moe", default="replicated", choices=["replicated", "dispatch"],
                    help="N > 1: experts by id over replicated activations, or token-dispatch expert parallelism "
                         "(every rank routes its slice of the tokens; dispatch / combine all-to-alls over peer memory)")
    ap.add_argument("--router-zipf", type=float, default=0.0,
                    help="expert popularity skew: N(0, 1) router logits plus a Zipf(s) selection bias per layer")
    ap.add_argument("--pp", type=int, default=1,
                    help="pipeline stages (N must be a multiple): each stage holds a contiguous range of layers over "
                         "N/pp tensor-parallel ranks; steps run eagerly (no graphs), so the device-timed number is the "
                         "engine loop")
    ap.add_argument("--microbatches", type=int, default=2, help="pipeline microbatches per step (--pp > 1)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import torch
    import torch.distributed as dist

    from ferrule_b200.models import config as C
    from ferrule_b200.models import weights as W
    from ferrule_b200.models.runner import DeepSeekRunner
    from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
    from ferrule_b200.runtime.scheduler import SchedulerConfig
    from ferrule_b200.runtime.session import GenerateRequest

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py ...")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp = pp = lay = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from ferrule_b200.parallel.layout import build_parallel
        lay = build_parallel(rank, world, dev, pp=args.pp, microbatches=args.microbatches, payload=args.ar_payload,
                             fused=not args.no_fused, collective=args.collective, multicast_push=args.mc_push)
        tp, pp = lay.tp, lay.pp

    cfg = C.PRESETS[args.model]()
    if cfg.n_mtp_layers:
        # plain greedy decoding: the multi-token-prediction module only serves speculative decoding and is not
        # instantiated (its weights are not part of the decode step's traffic either way)
        cfg = cfg.with_(n_mtp_layers=0)
    if args.layers:
        cfg = cfg.with_(n_layers=args.layers)
    B, P, K, Wm = args.batch, args.prompt_len, args.steps, args.warmup
    page = 64
    margin = 64                      # sequences that finish prefill early decode ahead of the others
    k_total = K * (2 if args.pp > 1 else 1)       # pipeline runs time two windows of engine steps
    max_seq = P + k_total + Wm + margin + 2 * page
    pages_per_seq = (max_seq + page - 1) // page
    tp_world = lay.tp_size if lay else 1
    from ferrule_b200.parallel.pp import stage_range, stage_weights
    weights = W.random_weights(cfg, device=dev, seed=0, tp_rank=lay.tp_rank if lay else 0, tp_world=args.shard_as or tp_world,
                               fast_device_init=True, weight_format=args.weight_format,
                               replicate_shared=(tp_world > 1 and args.moe == "dispatch"), router_zipf=args.router_zipf,
                               layer_range=stage_range(cfg.n_layers, lay.pp_rank, lay.pp_size) if pp is not None else None)
    if pp is not None:
        weights = stage_weights(weights, lay.pp_rank, lay.pp_size)
    runner = DeepSeekRunner(weights, n_pages=B * pages_per_seq + 8, page_size=page, max_rows=2048, max_seqs=B,
                            max_seq_len=pages_per_seq * page, device=dev, tp=tp, pp=pp,
                            enable_mtp=False)
    if tp is not None:
        tp.attach(runner.fwd)
        if args.moe == "dispatch":
            if pp is not None:
                raise SystemExit("--moe dispatch runs inside one tensor-parallel group; use it without --pp")
            from ferrule_b200.parallel.ep import ExpertParallelMoE
            ep = ExpertParallelMoE(rank, world, dev, cfg.hidden, cfg.moe_inter, cfg.topk, cfg.n_routed_experts,
                                   max_local_tokens=(B + world - 1) // world, allgather=True)
            runner.fwd.attach_ep(ep)
    sched = SchedulerConfig(max_active_sequences=B, max_decode_batch=B, max_batch_tokens=2048, prefill_chunk_size=512,
                            mixed_batches=True, ctx_size=pages_per_seq * page)
    engine = Engine(runner, EngineConfig(scheduler=sched, kv_pages=B * pages_per_seq + 8, page_size=page))

    # synthetic prompts: token ids uniform over the vocabulary, identical on every rank
    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    # warm-up wave: the same number of prompts of the same length (other tokens), two output tokens each, so that
    # the first-token latency below is not the cost of loading every kernel for the first time
    warm = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    for i in range(B):
        engine.submit(GenerateRequest(f"warm{i}", warm[i].tolist(), max_new_tokens=2, ignore_eos=True))
    engine.run_until_idle(lambda ev: None)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_submit = time.perf_counter()
    for i in range(B):
        engine.submit(GenerateRequest(f"req{i}", prompts[i].tolist(), max_new_tokens=k_total + Wm + margin, ignore_eos=True))
    first_token_t, token_times = {}, {}

    def emit(ev) -> None:
        if isinstance(ev, TokenEvent):
            now = time.perf_counter()
            first_token_t.setdefault(ev.request_id, now)
            token_times.setdefault(ev.request_id, []).append(now)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- prefill (untimed for the decode metric; TTFT and prefill tokens/s are reported from it) ----
    barrier()
    t_pf0 = time.perf_counter()
    while any(s.prefill_remaining > 0 for s in engine.scheduler.active.values()) or engine.scheduler.waiting:
        engine.step(emit)
    barrier()
    prefill_s = time.perf_counter() - t_pf0
    # one decode step so that every sequence has emitted its first token
    engine.step(emit)
    ttft = sorted(first_token_t[r] - t_submit for r in first_token_t)
    for _ in range(Wm):
        engine.step(emit)
    torch.cuda.synchronize()
    # the state the timed window starts from (row order of the decode batch = admission order)
    seqs0 = list(engine.scheduler.active.values())
    start_ids = [s.staged_token for s in seqs0]
    start_pos = [s.position for s in seqs0]

    # ---- e2e: K engine steps, device-timed around the whole loop ----
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    h2d0, d2h0, l0 = runner.stats.h2d_bytes, runner.stats.d2h_bytes, runner.stats.kernel_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps_before = engine.stats.decode_steps
    e0.record()
    for _ in range(K):
        engine.step(emit)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    assert engine.stats.decode_steps - steps_before == K, \
        "a timed engine step was not a decode step (last engine error: %r)" % (engine.last_error,)
    h2d = (runner.stats.h2d_bytes - h2d0) // K
    d2h = (runner.stats.d2h_bytes - d2h0) // K
    e2e_launches = runner.stats.kernel_launches - l0

    if pp is not None:
        # pipeline stages step eagerly through the engine on every rank: the device-timed number is a second
        # window of K engine steps (the stage hand-offs are NCCL transfers on a side stream)
        class _G:
            launches = 0
        graph = _G()
        barrier()
        _lib_l0 = runner.stats.kernel_launches
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(K):
            engine.step(emit)
        d1.record()
        barrier()
        graph.launches = (runner.stats.kernel_launches - _lib_l0) // K - 1
        from ferrule_b200.ops import _lib
    else:
        # ---- device-only: the same K steps from the same starting state, fed back on the device ----
        import numpy as np
        from ferrule_b200.ops import _lib
        from ferrule_b200.ops import kernels as KK
        st, graph = runner.graphs[B]
        runner._ahead = None                    # a step launched ahead by the last engine step is not consumed
        torch.cuda.synchronize()
        pages = [engine.kv.sequence(s.kv_seq).pages for s in seqs0]     # by now they cover the whole window

        def rewind() -> None:
            st.np_ids[:B] = start_ids
            st.np_pos[:B] = start_pos
            st.np_rpos[:B] = start_pos
            st.np_seq[:B] = np.arange(B)
            st.np_bt[:] = 0
            for i, pg in enumerate(pages):
                st.np_bt[i, :len(pg)] = pg
                st.np_slot[i] = pg[start_pos[i] // page] * page + start_pos[i] % page
            st.upload()

        def device_steps(n: int) -> None:
            for _ in range(n):
                graph.replay()
                KK.decode_advance(runner.fwd.ws.next_id[:B], graph.batch, cfg.vocab_size, page, True)

        rewind()
        device_steps(3)
        rewind()
        barrier()
        _lib.read_peer_wait()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        device_steps(K)
        d1.record()
        barrier()
    clocks = sampler.stop()
    dev_ms = d0.elapsed_time(d1)
    wait_ns, wait_n = _lib.read_peer_wait()

    status = _lib.read_status()
    times = torch.tensor([dev_ms, e2e_ms, prefill_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, prefill_s = times.tolist()
    tpots = []
    for r, ts in token_times.items():
        if len(ts) > 2:
            tpots.append((ts[-1] - ts[1]) / (len(ts) - 2))
    # what a decode step reads: every weight except the embedding table (a step gathers B of its rows)
    streamed_bytes = weights.nbytes()
    if weights.embed.data_ptr() != weights.lm_head.data_ptr():
        streamed_bytes -= weights.embed.numel() * weights.embed.element_size()
    if rank == 0:
        value = B * K / (dev_ms / 1e3)
        e2e_value = B * K / (e2e_ms / 1e3)
        par = ("pp%d x tp%d (%d microbatches)" % (lay.pp_size, lay.tp_size, args.microbatches)) if pp is not None else "single-gpu" if world == 1 else ("tp%d" % world if args.moe == "replicated" else "tp%d-attention + ep%d-dispatch" % (world, world))
        line = {
            "metric": "decode tokens/s (whole job, max over ranks)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / BASELINE_TOK_S, 1), "dtype": {"bf16": "bf16", "fp8_block": "fp8 e4m3 weights (128x128 scales) + fp8 activations (1x128), bf16 elsewhere", "fp8_mxfp4": "mxfp4 experts + fp8 dense, bf16 elsewhere"}[args.weight_format],
            "data": "synthetic (uniform-random token ids, random-init N(0,0.02) weights)",
            "config": {"model": cfg.name, "global_batch": B, "seq_len": P,
                       "decode_context": "%d..%d (grows one token per step, in both numbers)"
                                         % (min(start_pos), max(start_pos) + K),
                       "parallelism": par, "kv_page_size": page, "layers": cfg.n_layers,
                       "l2_policy": "inputs larger than L2: each step streams %.1f GB of weights per GPU"
                                    % (streamed_bytes / 1e9),
                       "collectives": "none" if world == 1 else ("nccl" if args.no_fused else (
                           "fused-p2p%s, %s partials" % (" (multicast push)" if args.mc_push else "", args.ar_payload) if args.collective == "ll"
                           else "in-switch multimem reduce + broadcast (bf16)"))},
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / K, 4),
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "path": "Engine.step (scheduler + KV transactions + pinned H2D + graph + D2H)"},
            "peer_wait": {"waits_per_step": wait_n // max(K, 1),
                          "avg_wait_us": round(wait_ns / 1e3 / max(wait_n, 1), 2),
                          "note": "rank 0: spins of a CTA on a peer's arrival word, and their mean length"},
            "gpu_launches": int((graph.launches + 1) * K),
            "gpu_launches_e2e": int(e2e_launches),
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"]},
            "prefill": {"tokens_per_s": round(B * P / prefill_s, 1), "seconds": round(prefill_s, 4),
                        "tokens": B * P, "chunk": sched.prefill_chunk_size, "timing": "host clock around the engine "
                        "steps of the prefill phase, device synchronised on both sides"},
            "lookahead": {"launched": runner.stats.lookahead_launched, "hits": runner.stats.lookahead_hits},
            "ttft_p50_s": round(ttft[len(ttft) // 2], 4) if ttft else None,
            "tpot_p50_s": round(statistics.median(tpots), 6) if tpots else None,
            "device_status": list(status),
            "impl": "ours",
        }
        if args.layers:
            line["invalid"] = "debug run with a reduced layer count"
        if args.shard_as:
            line["invalid"] = "debug run: one rank's shard of a TP-%d layout without collectives" % args.shard_as
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
