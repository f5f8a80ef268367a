"""Command line: `python -m ferrule_b200 <command>`.

  info                 package, device and library status; model presets or a checkpoint's layout
  cuda                 smoke benchmark of the native kernels (GEMV-sized GEMM, RMSNorm, launch overhead)
  make-fixture         write a random-init (or zero) checkpoint directory in the HF DeepSeek layout
  inspect-weightpack   tensor names / dtypes / shapes / inferred quant formats / role histogram
  generate             load a checkpoint (or a random-init preset) and greedily generate from token ids or text
  chat                 interactive REPL on top of the same engine
  serve                OpenAI-compatible HTTP server
  bench-interactive    multi-turn timing report (JSON) with engine, KV and speculative statistics
  bench-serve          synthetic serving sweep against a running server (Poisson arrivals, shared prefixes)
  expert-stream-smoke  stream routed experts of a checkpoint through the materialization stack

Counterpart of crates/ferrule-cli/src/args.rs:34-230, commands/serve.rs:20-168,
commands/bench_interactive.rs:57-235 and scripts/bench_vllm_serve.sh, dsv4_synthetic_fixture.py.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Any, Dict, List, Optional


def _add_model_args(p: argparse.ArgumentParser) -> None:
    p.add_argument("model", nargs="?", help="HF checkpoint directory (same as --model-dir)")
    p.add_argument("--model-dir", help="HF checkpoint directory (config.json + safetensors)")
    p.add_argument("--preset", default="tiny-fixture", help="random-init preset when no --model-dir is given")
    p.add_argument("--device", default=None, help="cuda[:N] or cpu (default: cuda when available)")
    p.add_argument("--kv-cache-mb", type=int, default=0, help="KV pool size; 0 = from --max-seqs x --ctx-size")
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--ctx-size", type=int, default=4096)
    p.add_argument("--max-seqs", "--max-active-sequences", dest="max_seqs", type=int, default=32)
    p.add_argument("--max-batch-tokens", type=int, default=2048)
    p.add_argument("--prefill-chunk", "--prefill-chunk-size", dest="prefill_chunk", type=int, default=512)
    p.add_argument("--speculative", action="store_true")
    p.add_argument("--decode-cohort-target", type=int, default=1,
                   help="ready decode requests wanted before a decode cohort is dispatched")
    p.add_argument("--decode-cohort-max-deferrals", type=int, default=0,
                   help="prefill decisions a decode cohort below its target may wait for")
    p.add_argument("--chat-template", choices=["chatml", "llama3", "qwen", "deepseek", "plain"],
                   help="override the chat template chosen from the model name")
    p.add_argument("--expert-residency", type=float, default=None,
                   help="fraction of every layer's routed experts kept on the device; the rest streams from pinned host memory")
    p.add_argument("--moe-hotset-experts", type=int, default=0,
                   help="routed-expert slots per layer on the device (another way to say --expert-residency; 0 = unset)")
    p.add_argument("--async-streaming", action="store_true",
                   help="with --expert-residency: a batch that needs a non-resident expert parks and resumes instead of "
                        "uploading inline")
    p.add_argument("--transaction-prefetch", type=int, default=0,
                   help="with --async-streaming: payloads a parked transaction may prefetch for later layers")
    p.add_argument("--materialization-timeout-secs", type=float, default=0.0,
                   help="with --async-streaming: roll a parked transaction back with an error after this long (0 = no limit)")
    p.add_argument("--expert-plan", help="JSON written by plan-placement: renumber the routed experts (random-init "
                                         "presets; every rank of a multi-rank launch must get the same file)")
    p.add_argument("--router-zipf", type=float, default=0.0,
                   help="random-init presets: skewed expert popularity (Zipf exponent) instead of a uniform router")
    p.add_argument("--prefix-cache-tokens", type=int, default=0,
                   help="keep the KV pages of finished prompts (whole 512-token blocks, this many tokens in total) "
                        "and fork them for later prompts that start with the same tokens; 0 = off")
    p.add_argument("--max-draft", type=int, default=1)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--weight-format", default="bf16", choices=["bf16", "fp8_block", "fp8_mxfp4"],
                   help="random-init presets: quantise the weights to this format")
    p.add_argument("--layers", "--max-layers", dest="layers", type=int, default=0, help="random-init presets: override the layer count")
    p.add_argument("--pp", type=int, default=1,
                   help="pipeline stages; under torch.distributed.run the ranks form pp stages x (world / pp) "
                        "tensor-parallel ranks, rank 0 serves and the others mirror its command stream")
    p.add_argument("--microbatches", type=int, default=2)
    p.add_argument("--collective", default="ll", choices=["ll", "multimem"])
    p.add_argument("--sequence-parallel", action="store_true",
                   help="tensor-parallel replicas: keep the residual stream sharded by rows between reduce-scatter and "
                        "all-gather (prefill-sized batches)")
    p.add_argument("--mc-push", action="store_true")


def replica_layout(args):
    """Process groups of a multi-rank launch (torch.distributed.run sets RANK / WORLD_SIZE): -> (layout, mirror),
    (None, None) in a single process."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        return None, None
    import torch
    import torch.distributed as dist

    from ..parallel.layout import build_parallel
    from ..parallel.mirror import CommandMirror
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    cuda = torch.cuda.is_available() and (args.device or "cuda").startswith("cuda")
    if cuda:
        torch.cuda.set_device(local)
        args.device = f"cuda:{local}"
    if not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo",
                                **({"device_id": torch.device("cuda", local)} if cuda else {}))
    dev = torch.device(args.device) if cuda else torch.device("cpu")
    lay = build_parallel(rank, world, dev, pp=args.pp, microbatches=args.microbatches,
                         collective=args.collective, multicast_push=args.mc_push, fused=cuda)
    host_group = dist.new_group(list(range(world)), backend="gloo") if cuda else None
    return lay, CommandMirror(rank, world, host_group)


def build_engine(args, layout=None):
    """-> (engine, tokenizer, model name).  Shared by generate / chat / serve / bench-interactive.  `layout`
    (parallel.layout.ParallelLayout): build this rank's shard of a tensor / pipeline parallel replica."""
    import torch

    from ..models import config as C
    from ..models import weights as W
    from ..models.runner import DeepSeekRunner
    from ..runtime.engine import Engine, EngineConfig
    from ..runtime.scheduler import SchedulerConfig
    from ..utils.tokenizer import load_tokenizer
    dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if getattr(args, "model", None) and not args.model_dir:
        args.model_dir = args.model
    if args.model_dir and _is_v4_dir(args.model_dir):
        return _build_v4_engine(args, dev, args.model_dir)
    if args.model_dir:
        from ..io.checkpoint import load_deepseek_hf
        weights = load_deepseek_hf(args.model_dir, device=dev, dtype=torch.bfloat16 if dev != "cpu" else torch.float32,
                                   max_layers=getattr(args, "layers", 0))
        name = os.path.basename(os.path.normpath(args.model_dir))
    elif args.preset == "tiny-v4":
        return _build_v4_engine(args, dev)
    else:
        cfg = C.PRESETS[args.preset]()
        if cfg.n_mtp_layers and not args.speculative:
            cfg = cfg.with_(n_mtp_layers=0)         # the MTP module only serves speculative decoding
        if getattr(args, "layers", 0):
            cfg = cfg.with_(n_layers=args.layers)
        tp_rank, tp_world = (layout.tp_rank, layout.tp_size) if layout is not None else (0, 1)
        staged = layout is not None and layout.pp is not None
        from ..parallel.pp import stage_range, stage_weights
        weights = W.random_weights(cfg, device=dev, dtype=torch.bfloat16 if dev != "cpu" else torch.float32,
                                   seed=args.seed, fast_device_init=dev != "cpu", tp_rank=tp_rank, tp_world=tp_world,
                                   weight_format=getattr(args, "weight_format", "bf16"),
                                   layer_range=stage_range(cfg.n_layers, layout.pp_rank, layout.pp_size)
                                   if (staged and dev != "cpu") else None,
                                   router_zipf=getattr(args, "router_zipf", 0.0), expert_orders=_expert_plan(args))
        if staged:
            weights = stage_weights(weights, layout.pp_rank, layout.pp_size)
        name = cfg.name
    if layout is not None and args.model_dir:
        raise SystemExit("checkpoint directories load on one rank; multi-rank launches take --preset")
    if args.speculative == "auto":                   # use the checkpoint's proposal stage when it has one
        args.speculative = bool(weights.mtp)
    cfg = weights.cfg
    ctx = min(args.ctx_size, cfg.max_position)
    pages_per_seq = (ctx + args.page_size - 1) // args.page_size
    if args.kv_cache_mb:
        per_page = (cfg.n_layers + cfg.n_mtp_layers) * args.page_size * cfg.kv_row_dim * 2
        n_pages = max(args.kv_cache_mb * (1 << 20) // per_page, pages_per_seq + 1)
    else:
        n_pages = args.max_seqs * pages_per_seq + 8
    residency = getattr(args, "expert_residency", None)
    if residency is None and getattr(args, "moe_hotset_experts", 0) and cfg.n_routed_experts:
        residency = min(args.moe_hotset_experts / cfg.n_routed_experts, 1.0)
    streaming = bool(getattr(args, "async_streaming", False) and residency is not None)
    if streaming and layout is not None:
        # the ranks of a replica replay one command stream and must take every scheduling decision alike; when an
        # upload completes differs from rank to rank, so transactions would resume in different steps
        raise SystemExit("--async-streaming runs on one rank; multi-rank replicas stream experts inline (--expert-residency)")
    runner = DeepSeekRunner(weights, n_pages=n_pages, page_size=args.page_size, max_rows=args.max_batch_tokens,
                            max_seqs=args.max_seqs, max_seq_len=pages_per_seq * args.page_size, device=dev,
                            tp=layout.tp if layout is not None else None, pp=layout.pp if layout is not None else None,
                            sequence_parallel=getattr(args, "sequence_parallel", False),
                            expert_residency=residency, async_streaming=streaming, enable_mtp=args.speculative,
                            max_draft=max(args.max_draft, 1))
    if layout is not None and layout.tp is not None and str(dev) != "cpu":
        layout.tp.attach(runner.fwd)
    sched = SchedulerConfig(max_active_sequences=args.max_seqs, max_decode_batch=args.max_seqs,
                            max_batch_tokens=args.max_batch_tokens, prefill_chunk_size=args.prefill_chunk,
                            decode_cohort_target=getattr(args, "decode_cohort_target", 1),
                            decode_cohort_max_deferrals=getattr(args, "decode_cohort_max_deferrals", 0),
                            ctx_size=pages_per_seq * args.page_size)
    block = max(512 // args.page_size, 1) * args.page_size
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=n_pages, page_size=args.page_size,
                                      speculative=args.speculative, max_draft=args.max_draft,
                                      prefix_cache_tokens=getattr(args, "prefix_cache_tokens", 0), prefix_block=block,
                                      transaction_prefetch=getattr(args, "transaction_prefetch", 0) if streaming else 0,
                                      materialization_timeout_s=getattr(args, "materialization_timeout_secs", 0.0)),
                 registry=runner.make_registry() if streaming else None)
    return eng, load_tokenizer(args.model_dir), name


def _is_v4_dir(model_dir: str) -> bool:
    try:
        with open(os.path.join(model_dir, "config.json")) as f:
            return json.load(f).get("model_type") == "deepseek_v4"
    except OSError:
        return False


def _chat_template(args):
    """The `--chat-template` override as a `ChatTemplate`, or None (the model name decides)."""
    from ..utils.tokenizer import ChatTemplate
    name = getattr(args, "chat_template", None)
    return ChatTemplate(name) if name else None


def _expert_plan(args):
    """{layer: order} from the file `--expert-plan` names (the `plan` of a plan-placement report)."""
    path = getattr(args, "expert_plan", None)
    if not path:
        return None
    with open(path) as f:
        doc = json.load(f)
    return {int(l): [int(e) for e in o] for l, o in doc.get("plan", doc).items()}


def _build_v4_engine(args, dev, model_dir: Optional[str] = None):
    """DeepSeek-V4 family model behind the engine (slot-bound state): a checkpoint directory, or the random-init
    tiny shape."""
    import torch

    from ..models.v4_model import random_v4_weights, tiny_v4
    from ..models.v4_runner import V4Runner
    from ..runtime.engine import Engine, EngineConfig
    from ..runtime.scheduler import SchedulerConfig
    from ..utils.tokenizer import load_tokenizer
    if model_dir:
        from ..io.v4_checkpoint import load_v4_hf
        weights = load_v4_hf(model_dir, device=dev, max_layers=getattr(args, "layers", 0))
        cfg = weights.cfg
    else:
        cfg = tiny_v4()
        if args.speculative:
            cfg = cfg.with_(n_proposal_stages=2, proposal_target_layers=(0, cfg.n_layers - 1), proposal_noise_token=1,
                            proposal_markov_rank=32)
        weights = random_v4_weights(cfg, device=dev, seed=args.seed)
    if args.speculative == "auto":                   # use the checkpoint's drafter when it has one
        args.speculative = weights.proposal is not None
    if args.speculative and weights.proposal is None:
        raise SystemExit("--speculative: this DeepSeek-V4 checkpoint has no `mtp.*` proposal stages")
    ctx = min(args.ctx_size, cfg.max_position)
    pages_per_seq = (ctx + args.page_size - 1) // args.page_size
    n_pages = args.max_seqs * pages_per_seq + 8
    runner = V4Runner(weights, n_pages=n_pages, page_size=args.page_size, max_seqs=args.max_seqs,
                      max_seq_len=pages_per_seq * args.page_size, max_rows=args.max_batch_tokens)
    sched = SchedulerConfig(max_active_sequences=args.max_seqs, max_decode_batch=args.max_seqs,
                            max_batch_tokens=args.max_batch_tokens, prefill_chunk_size=args.prefill_chunk,
                            decode_cohort_target=getattr(args, "decode_cohort_target", 1),
                            decode_cohort_max_deferrals=getattr(args, "decode_cohort_max_deferrals", 0),
                            ctx_size=pages_per_seq * args.page_size)
    # the block drafter proposes `proposal_block_size` tokens at once: --max-draft above 1 caps it, the default
    # takes the whole block
    draft = cfg.proposal_block_size if args.max_draft <= 1 else min(args.max_draft, cfg.proposal_block_size)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=n_pages, page_size=args.page_size,
                                      speculative=args.speculative, max_draft=draft))
    name = os.path.basename(os.path.normpath(model_dir)) if model_dir else "deepseek-v4-tiny"
    return eng, load_tokenizer(model_dir), name


# ------------------------------------------------------------------------------------------ commands
def cmd_info(args) -> int:
    import torch

    if getattr(args, "model", None) and not args.model_dir:
        args.model_dir = args.model

    from .. import __version__, _build
    from ..models import config as C
    out = {"version": __version__, "torch": torch.__version__, "cuda_available": torch.cuda.is_available(),
           "native_library": str(_build.LIB_PATH), "native_library_built": _build.LIB_PATH.exists(),
           "native_library_current": _build.is_current()}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        out["device"] = {"name": p.name, "sm": f"{p.major}{p.minor}", "sms": p.multi_processor_count,
                         "memory_gb": round(p.total_memory / 2 ** 30, 1)}
    def plan_of(cfg, weight_format="bf16", tp=1, pp=1):
        """The support contract's verdict on a configuration: which policies apply and whether this build runs it."""
        from dataclasses import asdict
        from ..models.support import EnginePlan, ParallelismPlan, PolicySet
        ps = PolicySet.from_config(cfg, weight_format, ParallelismPlan(tensor_parallel=tp, pipeline_parallel=pp))
        plan = EnginePlan.from_policies(ps, cfg.n_heads, cfg.n_routed_experts, cfg.n_layers, cfg.vocab_size)
        def enc(o):
            return {k: (v.value if hasattr(v, "value") else (list(v) if isinstance(v, tuple) else v))
                    for k, v in asdict(o).items()}
        return {"family": plan.family, "status": plan.status.value,
                "missing": [{"area": m.area, "reason": m.reason} for m in plan.missing],
                "policies": {k: enc(getattr(ps, k)) for k in ("attention", "router", "expert", "quant", "kv", "residency",
                                                             "parallelism", "speculation")}}
    if args.model_dir and _is_v4_dir(args.model_dir):
        from dataclasses import asdict
        from ..io.safetensors import ShardedCheckpoint
        from ..io.v4_checkpoint import v4_config_from_hf
        with open(os.path.join(args.model_dir, "config.json")) as f:
            vcfg = v4_config_from_hf(json.load(f))
        ck = ShardedCheckpoint(args.model_dir)
        out["checkpoint"] = {"family": "deepseek_v4", "tensors": len(ck.names()),
                             "shards": len(set(ck.weight_map.values())), "config": asdict(vcfg)}
        out["engine_plan"] = plan_of(vcfg)
    elif args.model_dir:
        from ..io.safetensors import ShardedCheckpoint
        from ..models.families import detect_family, layout_summary
        ck = ShardedCheckpoint(args.model_dir)
        cfg = C.from_hf_config(args.model_dir) if os.path.exists(os.path.join(args.model_dir, "config.json")) else None
        fam = detect_family(ck.names(), cfg.name if cfg else "")
        out["checkpoint"] = {"family": fam.value, "tensors": len(ck.names()), "shards": len(set(ck.weight_map.values())),
                             "roles": layout_summary(ck.names(), fam, cfg.n_layers if cfg else None),
                             "config": cfg.to_dict() if cfg else None}
        if cfg is not None:
            out["engine_plan"] = plan_of(cfg)
    else:
        out["presets"] = {k: {"params_b": round(f().param_count() / 1e9, 3), "layers": f().n_layers,
                              "hidden": f().hidden, "engine_plan": plan_of(f())["status"]} for k, f in C.PRESETS.items()}
    print(json.dumps(out, indent=1))
    return 0


def cmd_cuda(args) -> int:
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    from ..ops import kernels as K
    dev = "cuda"

    def timed(fn, n=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3
    res = {}
    for rows, n, k in ((1, 4096, 4096), (32, 4096, 4096), (32, 16384, 4096)):
        ws = [torch.randn(n, k, device=dev).bfloat16() for _ in range(8)]
        x = torch.randn(rows, k, device=dev).bfloat16()
        out = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        i = [0]

        def f():
            K.gemm(x, ws[i[0] % 8], out=out)
            i[0] += 1
        us = timed(f)
        res[f"gemm_{rows}x{n}x{k}_us"] = round(us, 2)
        res[f"gemm_{rows}x{n}x{k}_gbs"] = round(n * k * 2 / us / 1e3, 1)
    x = torch.randn(32, 4096, device=dev).bfloat16()
    w = torch.ones(4096, device=dev).bfloat16()
    o = torch.empty_like(x)
    res["rmsnorm_32x4096_us"] = round(timed(lambda: K.add_rmsnorm(x, w, 1e-6, norm_out=o)), 2)
    ids = torch.zeros(1, dtype=torch.int32, device=dev)
    tab = torch.zeros(8, 64, device=dev).bfloat16()
    eo = torch.empty(1, 64, device=dev, dtype=torch.bfloat16)
    res["launch_overhead_us"] = round(timed(lambda: K.embedding(ids, tab, out=eo), 200), 2)
    print(json.dumps(res, indent=1))
    return 0


def cmd_make_fixture(args) -> int:
    import torch

    from ..io.checkpoint import export_hf
    from ..models import config as C
    from ..models import weights as W
    if args.family == "v4":
        # DeepSeek-V4 layout: FP8 attention / shared experts, packed FP4 routed experts unless told otherwise
        from ..io.v4_checkpoint import export_v4_hf
        from ..models.v4_model import random_v4_weights, tiny_v4
        cfg = tiny_v4()
        if args.layers:
            ratios = tuple(cfg.compress_ratios[i % len(cfg.compress_ratios)] for i in range(args.layers))
            cfg = cfg.with_(n_layers=args.layers, compress_ratios=ratios)
        if args.proposal_stages:
            # the `mtp.*` block drafter: taps after the first and the last target layer
            taps = tuple(sorted({0, cfg.n_layers - 1}))
            cfg = cfg.with_(n_proposal_stages=args.proposal_stages, proposal_target_layers=taps,
                            proposal_noise_token=1, proposal_markov_rank=32)
        w = random_v4_weights(cfg, seed=args.seed, std=0.0 if args.zeros else 0.05)
        dense = "fp8_block" if args.dense_format == "plain" and not args.plain else args.dense_format
        expert = "mxfp4" if args.expert_format == "plain" and not args.plain else args.expert_format
        export_v4_hf(w, args.out, dense_format=dense, expert_format=expert, shard_bytes=args.shard_mb << 20)
        print(json.dumps({"written": args.out, "family": "deepseek_v4", "layers": cfg.n_layers,
                          "proposal_stages": cfg.n_proposal_stages, "dense_format": dense, "expert_format": expert}))
        return 0
    cfg = C.PRESETS[args.preset]()
    if args.layers:
        cfg = cfg.with_(n_layers=args.layers)
    w = W.random_weights(cfg, dtype=torch.bfloat16, seed=args.seed, std=0.0 if args.zeros else 0.02)
    export_hf(w, args.out, dense_format=args.dense_format, expert_format=args.expert_format,
              shard_bytes=args.shard_mb << 20)
    print(json.dumps({"written": args.out, "params": cfg.param_count(), "dense_format": args.dense_format,
                      "expert_format": args.expert_format}))
    return 0


def cmd_inspect(args) -> int:
    from ..io.checkpoint import infer_weight_format
    from ..io.safetensors import ShardedCheckpoint
    from ..models.families import detect_family, layout_summary
    ck = ShardedCheckpoint(args.model_dir)
    fam = detect_family(ck.names())
    rows, total = [], 0
    for n in sorted(ck.names()):
        i = ck.info(n)
        total += i.nbytes
        fmt = ""
        if n.endswith(".weight"):
            try:
                fmt = infer_weight_format(ck, n[:-7])[0]
            except Exception:  # noqa: BLE001
                fmt = "?"
        rows.append((n, i.dtype, list(i.shape), i.nbytes, fmt))
    if args.json:
        print(json.dumps({"family": fam.value, "bytes": total, "roles": layout_summary(ck.names(), fam),
                          "tensors": [dict(name=r[0], dtype=r[1], shape=r[2], bytes=r[3], format=r[4]) for r in rows[:args.limit]]}))
    else:
        print(f"family {fam.value}, {len(rows)} tensors, {total / 2 ** 20:.1f} MiB")
        for r in rows[:args.limit]:
            print(f"{r[0]:70s} {r[1]:8s} {str(r[2]):20s} {r[4]}")
    return 0


def _collect(eng, emit_text=None):
    from ..runtime.engine import FinishEvent, TokenEvent
    toks, fin = {}, {}

    def emit(ev):
        if isinstance(ev, TokenEvent):
            toks.setdefault(ev.request_id, []).append(ev.token)
            if emit_text and ev.text:
                emit_text(ev.text)
        elif isinstance(ev, FinishEvent):
            fin[ev.request_id] = ev
            if emit_text and ev.tail:
                emit_text(ev.tail)
    eng.run_until_idle(emit)
    return toks, fin


def _add_generate_args(p) -> None:
    p.add_argument("-p", "--prompt", default="hello"); p.add_argument("--tokens")
    p.add_argument("-n", "--max-tokens", type=int, default=16)
    p.add_argument("--ignore-eos", "--no-stop-eos", dest="ignore_eos", action="store_true")
    p.add_argument("--chat", action="store_true", help="wrap --prompt in the model's chat template")
    p.add_argument("--verbose-tokens", action="store_true", help="print every generated token id to stderr")
    p.add_argument("--warmup-tokens", type=int, default=0, help="decode this many tokens of a throw-away request first")
    p.add_argument("--json", action="store_true", help="add the engine / runner / registry report to the output")


def cmd_generate(args) -> int:
    from ..runtime.session import GenerateRequest
    if getattr(args, "v4_generate", False):
        args.speculative = "auto" if not args.no_speculative else False
    eng, tok, name = build_engine(args)
    eng.detokenize = tok.decode
    text = args.prompt
    if args.chat and not args.tokens:
        from ..utils.tokenizer import ChatMessage, render_chat, template_for_model
        text = render_chat([ChatMessage("user", args.prompt)], _chat_template(args) or template_for_model(name))
    prompt = [int(t) for t in args.tokens.split(",")] if args.tokens else tok.encode(text)
    prompt = [t % eng.runner.vocab_size for t in prompt]
    if args.warmup_tokens > 0:
        eng.submit(GenerateRequest("warmup", prompt[:8] or [1], max_new_tokens=args.warmup_tokens, ignore_eos=True))
        _collect(eng)
    t0 = time.perf_counter()
    eng.submit(GenerateRequest("gen", prompt, max_new_tokens=args.max_tokens, ignore_eos=args.ignore_eos))
    toks, fin = _collect(eng)
    dt = time.perf_counter() - t0
    f = fin["gen"]
    if args.verbose_tokens:
        for i, t in enumerate(toks.get("gen", [])):
            print(f"[token {i}] id={t} text={tok.decode([t])!r}", file=sys.stderr)
    out = {"model": name, "prompt_tokens": len(prompt), "tokens": toks.get("gen", []), "text": f.text,
           "finish_reason": f.reason.openai(), "seconds": round(dt, 4), "ttft_s": round(f.ttft_s, 4),
           "tpot_s": round(f.tpot_s, 6)}
    if args.json:
        out["report_version"] = 2
        out["engine"] = eng.snapshot_stats()
        out["runner"] = eng.runner.observability()
        if eng.spec is not None:
            out["speculative"] = eng.spec.metrics.to_dict()
        if eng.registry is not None and hasattr(eng.registry, "stats"):
            out["registry"] = dict(vars(eng.registry.stats))
    print(json.dumps(out))
    return 0


def cmd_plan_placement(args) -> int:
    """Count the routes of a calibration workload and print the expert placement that evens the ranks' loads
    (`parallel/placement.py`); `--expert-plan FILE` of the model commands applies it."""
    import torch

    from ..parallel.placement import RouteCounter, imbalance
    from ..runtime.session import GenerateRequest
    eng, _, name = build_engine(args)
    runner = eng.runner
    cfg = getattr(runner, "cfg", None)
    if cfg is None or not getattr(cfg, "n_routed_experts", 0) or not hasattr(runner.fwd, "route_observer"):
        raise SystemExit("plan-placement: this model has no routed experts to place")
    # the observer reads every layer's expert ids on the host: calibration steps run eagerly
    runner.use_graphs = False
    runner.lookahead = False
    counter = RouteCounter(cfg.n_layers, cfg.n_routed_experts).attach(runner.fwd)
    g = torch.Generator().manual_seed(args.seed)
    for i in range(args.requests):
        ids = torch.randint(0, runner.vocab_size, (args.prompt_tokens,), generator=g).tolist()
        eng.submit(GenerateRequest(f"cal{i}", ids, max_new_tokens=args.max_tokens, ignore_eos=True))
    _collect(eng)
    RouteCounter.detach(runner.fwd)
    counts = counter.telemetry.counts
    plan = counter.plan(args.ranks, n_groups=cfg.n_groups if cfg.topk_groups < cfg.n_groups else 1, min_gain=args.min_gain)
    ident = list(range(cfg.n_routed_experts))
    report = {"model": name, "ranks": args.ranks, "routes": int(sum(sum(r) for r in counts)),
              "layers": {str(l): {"imbalance_by_id": round(imbalance(counts[l], ident, args.ranks), 4),
                                  "imbalance_planned": round(imbalance(counts[l], plan.get(l, ident), args.ranks), 4)}
                         for l in range(cfg.n_layers) if sum(counts[l])},
              "plan": {str(l): o for l, o in plan.items()}}
    if args.out:
        with open(args.out, "w") as f:
            json.dump(report, f)
        report = {k: v for k, v in report.items() if k != "plan"}
        report["written"] = args.out
    print(json.dumps(report))
    return 0


def cmd_chat(args) -> int:
    """Interactive chat.  The conversation is one retained session: every turn feeds only its new text to the
    model and continues from the cached history.  /reset clears the session, /stats, /ctx and /experts report, /exit or an empty line ends.
    Mirrors the reference's chat command (crates/ferrule-cli/src/commands/chat.rs:205-275)."""
    from ..runtime.session import GenerateRequest
    from ..utils.tokenizer import ChatMessage, render_chat, template_for_model
    eng, tok, name = build_engine(args)
    eng.detokenize = tok.decode
    history: List[ChatMessage] = []
    tmpl = _chat_template(args) or template_for_model(name)
    retained = True
    session = "chat"
    cached_text = ""                 # the rendered text whose tokens the session's cache holds
    ctx = eng.cfg.scheduler.ctx_size
    print(f"{name}: /reset /stats /ctx /experts /exit; empty line or Ctrl-D to quit")
    turn = generated = 0

    def position() -> int:
        s = eng._sessions.get(session)
        return s.position if s is not None else 0

    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        cmd = line.strip()
        if not cmd or cmd in ("/exit", "/quit"):
            break
        if cmd in ("/reset", "/clear"):
            eng.reset_session(session)
            history, cached_text, turn, generated = [], "", 0, 0
            print("session reset.")
            continue
        if cmd == "/stats":
            print(f"position={position()} generated={generated} turns={turn}")
            continue
        if cmd == "/ctx":
            print(f"context {position()} / {ctx} tokens ({100.0 * position() / max(ctx, 1):.1f} %)")
            continue
        if cmd == "/experts":
            obs = eng.runner.observability()
            rep = {k: obs[k] for k in ("expert_arena", "expert_telemetry") if k in obs}
            print(json.dumps(rep) if rep else "expert report not available.")
            continue
        history.append(ChatMessage("user", line))
        full = render_chat(history, tmpl)
        if retained and cached_text and full.startswith(cached_text):
            new_text = full[len(cached_text):]
        else:
            if retained and cached_text:
                eng.reset_session(session)       # the rendering no longer extends the cached text: start over
            new_text = full
        ids = [t % eng.runner.vocab_size for t in tok.encode(new_text)]
        try:
            eng.submit(GenerateRequest(f"turn{turn}", ids, max_new_tokens=args.max_tokens,
                                       session_id=session if retained else None, retain_session=retained))
        except ValueError as exc:
            history.pop()
            print(f"[{exc}] use /reset to start a new conversation")
            continue
        _, fin = _collect(eng, lambda s: (sys.stdout.write(s), sys.stdout.flush()))
        print()
        f = fin[f"turn{turn}"]
        history.append(ChatMessage("assistant", f.text))
        cached_text = full + f.text
        generated += f.generated_tokens
        turn += 1
    return 0


def cmd_serve(args) -> int:
    from ..server.http import serve
    from ..server.worker import ModelWorker, WorkerConfig
    from ..utils.observability import init_tracing, start_periodic_dump
    init_tracing()
    start_periodic_dump()
    holder = {}
    layout, mirror = replica_layout(args)
    if mirror is not None and not mirror.is_leader:
        # a follower rank of the replica: same engine, driven by the leader's command stream
        from ..parallel.mirror import follower_loop
        eng, _, _ = build_engine(args, layout)
        steps = follower_loop(eng, mirror)
        print(json.dumps({"follower": mirror.rank, "steps": steps}), flush=True)
        return 0

    def factory():
        if layout is not None and str(args.device).startswith("cuda"):
            import torch
            torch.cuda.set_device(torch.device(args.device))     # the worker thread needs the rank's device current
        eng, tok, name = build_engine(args, layout)
        holder["tok"], holder["name"] = tok, name
        return eng
    # the engine is built on the worker thread (it owns the CUDA context and every graph)
    from ..utils.tokenizer import load_tokenizer
    tok = load_tokenizer(args.model_dir)
    worker = ModelWorker(factory, tok, WorkerConfig(command_queue=args.command_queue, event_queue=args.event_queue,
                                                    admission_timeout_s=args.admission_timeout),
                         model_name=args.served_name or args.preset, mirror=mirror).start()
    print(json.dumps({"serving": holder.get("name"), "host": args.host, "port": args.port}), flush=True)
    serve(worker, args.host, args.port, args.served_name or holder.get("name"), template=_chat_template(args))
    return 0


def _compare_traces(got: List[List[int]], want: List[List[int]]) -> Dict[str, Any]:
    """Turn-by-turn comparison of token traces: the first diverging turn / index and both tokens there."""
    out: Dict[str, Any] = {"match": got == want, "turns_compared": min(len(got), len(want))}
    if len(got) != len(want):
        out["turn_count"] = {"got": len(got), "want": len(want)}
    for t, (g, w) in enumerate(zip(got, want)):
        if g != w:
            i = next((j for j, (a, b) in enumerate(zip(g, w)) if a != b), min(len(g), len(w)))
            out["first_divergence"] = {"turn": t, "index": i, "got": g[i] if i < len(g) else None,
                                       "want": w[i] if i < len(w) else None, "got_len": len(g), "want_len": len(w)}
            break
    return out


def cmd_bench_interactive(args) -> int:
    """Multi-turn session benchmark: one retained session, `--turns` turns of a synthetic (or `--trace` given)
    prompt; JSON report (version 2) with per-turn timing, engine / runner / registry / speculative /
    hard-resource statistics and, with `--golden`, a token-exact comparison against a recorded trace."""
    import random

    from ..runtime.session import GenerateRequest
    eng, tok, name = build_engine(args)
    rng = random.Random(args.seed)
    V = eng.runner.vocab_size
    report = {"report_version": 2, "model": name, "turns": []}
    sid = "bench-session"
    trace = json.load(open(args.trace)) if args.trace else None
    n_turns = len(trace["turns"]) if trace else args.turns
    full: List[List[int]] = []
    for turn in range(n_turns):
        if trace:
            t = trace["turns"][turn]
            prompt = t["prompt_tokens"] if "prompt_tokens" in t else tok.encode(t.get("prompt", ""))
            max_new = int(t.get("max_tokens", args.max_tokens))
        else:
            prompt, max_new = [rng.randrange(V) for _ in range(args.prompt_len)], args.max_tokens
        t0 = time.perf_counter()
        eng.submit(GenerateRequest(f"t{turn}", prompt, max_new_tokens=max_new, ignore_eos=True,
                                   session_id=sid, retain_session=True))
        toks, fin = _collect(eng)
        f = fin[f"t{turn}"]
        full.append(list(toks.get(f"t{turn}", [])))
        report["turns"].append({"turn": turn, "prompt_tokens": f.prompt_tokens, "generated": f.generated_tokens,
                                "seconds": round(time.perf_counter() - t0, 4), "ttft_s": round(f.ttft_s, 4),
                                "tpot_s": round(f.tpot_s, 6), "finish": f.reason.value, "tokens": full[-1]})
    report["engine"] = eng.snapshot_stats()
    report["runner"] = eng.runner.observability()
    if eng.registry is not None:
        report["registry"] = dict(vars(eng.registry.stats)) if hasattr(eng.registry, "stats") else {}
        if hasattr(eng.registry, "ledger"):
            report["critical_path"] = eng.registry.ledger.snapshot() if hasattr(eng.registry.ledger, "snapshot") else {}
    if args.write_golden:
        with open(args.write_golden, "w") as fh:
            json.dump({"model": name, "turns": [{"tokens": t} for t in full]}, fh)
        report["golden_written"] = args.write_golden
    if args.golden:
        golden = json.load(open(args.golden))
        want = [list(t["tokens"]) for t in golden.get("turns", [])]
        # a golden trace may hold a prefix of every turn's tokens (older reports kept eight)
        got = [g[:len(w)] if len(w) < len(g) else g for g, w in zip(full, want)] + full[len(want):]
        report["golden"] = _compare_traces(got, want)
        report["golden_match"] = report["golden"]["match"]
    eng.shutdown()
    report["shutdown_residual"] = {"kv_used_pages": eng.kv.stats().used_pages, "grants": eng.broker.outstanding()}
    print(json.dumps(report))
    return 0 if report.get("golden_match", True) else 2


def cmd_generation_parity(args) -> int:
    """Prompt / token parity against a recorded file: `{"cases": [{"prompt_tokens": [...] | "prompt": "...",
    "expected_tokens": [...]}]}`.  Every case runs greedily for len(expected) tokens; exit code 2 on a mismatch.
    Plays the role of the reference's scripts/dsv4_generation_parity.py."""
    from ..runtime.session import GenerateRequest
    eng, tok, name = build_engine(args)
    spec = json.load(open(args.cases))
    results, ok = [], True
    for i, c in enumerate(spec["cases"]):
        prompt = c["prompt_tokens"] if "prompt_tokens" in c else tok.encode(c["prompt"])
        want = list(c.get("expected_tokens", []))
        n = len(want) or int(c.get("max_tokens", args.max_tokens))
        eng.submit(GenerateRequest(f"case{i}", prompt, max_new_tokens=n, ignore_eos=True))
        toks, _ = _collect(eng)
        got = list(toks.get(f"case{i}", []))
        cmp_ = _compare_traces([got], [want]) if want else {"match": True}
        ok &= cmp_["match"]
        results.append({"case": i, "prompt_tokens": len(prompt), "generated": got, **cmp_})
    eng.shutdown()
    print(json.dumps({"model": name, "cases": results, "all_match": ok}))
    return 0 if ok else 2


def cmd_chunk_sweep(args) -> int:
    """Sweep the prefill chunk size of the resident driver on one synthetic prompt set and report TTFT,
    prefill tokens/s and decode tokens/s per setting (the reference's scripts/dsv4_runtime_driver_chunk_sweep.py)."""
    import random

    from ..runtime.session import GenerateRequest
    rows = []
    for chunk in args.chunks:
        args.prefill_chunk = chunk
        args.max_batch_tokens = max(args.max_batch_tokens, chunk)
        eng, tok, name = build_engine(args)
        rng = random.Random(args.seed)
        V = eng.runner.vocab_size
        t0 = time.perf_counter()
        for i in range(args.requests):
            eng.submit(GenerateRequest(f"r{i}", [rng.randrange(V) for _ in range(args.prompt_len)],
                                       max_new_tokens=args.max_tokens, ignore_eos=True))
        toks, fin = _collect(eng)
        wall = time.perf_counter() - t0
        ttft = sorted(f.ttft_s for f in fin.values())
        gen = sum(f.generated_tokens for f in fin.values())
        st = eng.snapshot_stats()
        rows.append({"prefill_chunk": chunk, "seconds": round(wall, 4), "ttft_p50_s": round(ttft[len(ttft) // 2], 4),
                     "ttft_max_s": round(ttft[-1], 4), "generated_tokens": gen,
                     "tokens_per_s": round((gen + args.requests * args.prompt_len) / wall, 1),
                     "prefill_chunks": st["prefill_chunks"], "decode_steps": st["decode_steps"]})
        eng.shutdown()
    print(json.dumps({"model": name, "prompt_len": args.prompt_len, "requests": args.requests, "sweep": rows}))
    return 0


def cmd_bench_serve(args) -> int:
    from ..server.bench_serve import run_sweep
    print(json.dumps(run_sweep(args.url, args.model, args.concurrency, args.requests, args.seed, args.vocab,
                               args.min_in, args.max_in, args.min_out, args.max_out, args.shared_prefix,
                               args.shared_fraction)))
    return 0


def cmd_expert_stream_smoke(args) -> int:
    import torch

    from ..io.safetensors import ShardedCheckpoint
    from ..models import config as C
    from ..runtime.expert_residency import ExpertResidencyController, plan_residency
    from ..runtime.expert_streaming import (ExpertArena, ExpertMaterializationProvider, ExpertSourceCatalog,
                                            HostStagedExpertCache, PinnedSlabPool)
    from ..runtime.registry import LoadRegistry
    cfg = C.from_hf_config(args.model_dir)
    ck = ShardedCheckpoint(args.model_dir)
    layers = [l for l in range(cfg.n_layers) if cfg.is_moe_layer(l)]
    dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    cat = ExpertSourceCatalog(cfg.name, ck, layers, cfg.n_routed_experts, backend=dev)
    caps = plan_residency(args.device_mb << 20, cat.max_payload_bytes(), layers, cfg.n_routed_experts, cfg.topk,
                          args.residency)
    res = ExpertResidencyController(layers, caps, cfg.n_routed_experts)
    arena = ExpertArena(layers, caps, cat.max_payload_bytes(), dev)
    try:
        from ..io.direct_reader import NativeDirectReader
        reader = NativeDirectReader(args.threads)
    except Exception:  # noqa: BLE001
        reader = None
    prov = ExpertMaterializationProvider(cat, res, arena, PinnedSlabPool(cat.max_payload_bytes(), args.slabs),
                                         HostStagedExpertCache(args.host_cache_mb << 20, args.host_cache_mb << 20), reader)
    reg = LoadRegistry(prov)
    t0 = time.perf_counter()
    want = [(l, e) for l in layers for e in range(min(caps[l], cfg.n_routed_experts))]
    reg.register_continuation(0, [cat.key(l, e) for l, e in want])
    while not reg._ready and not reg._failed and time.perf_counter() - t0 < args.timeout:
        reg.drive()
        time.sleep(0.0005)
    dt = time.perf_counter() - t0
    print(json.dumps({"experts": len(want), "ok": bool(reg._ready), "seconds": round(dt, 3),
                      "gib_per_s": round(prov.bytes_uploaded / dt / 2 ** 30, 3), "bytes": prov.bytes_uploaded,
                      "registry": vars(reg.stats), "slab_high_water": prov.slabs.high_water,
                      "arena_mb": arena.nbytes() >> 20}))
    prov.close()
    return 0 if reg._ready else 1


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="ferrule_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("info"); p.add_argument("model", nargs="?"); p.add_argument("--model-dir"); p.set_defaults(fn=cmd_info)
    p = sub.add_parser("cuda"); p.set_defaults(fn=cmd_cuda)
    p = sub.add_parser("make-fixture")
    p.add_argument("--preset", default="tiny-fixture"); p.add_argument("--out", required=True)
    p.add_argument("--layers", type=int, default=0); p.add_argument("--seed", type=int, default=0)
    p.add_argument("--zeros", action="store_true"); p.add_argument("--shard-mb", type=int, default=1024)
    p.add_argument("--dense-format", default="plain", choices=["plain", "fp8_block"])
    p.add_argument("--expert-format", default="plain", choices=["plain", "fp8_block", "mxfp4"])
    p.add_argument("--family", default="deepseek", choices=["deepseek", "v4"],
                   help="v4: a DeepSeek-V4 directory (tiny shape; FP8 dense + packed FP4 experts unless --plain)")
    p.add_argument("--plain", action="store_true", help="--family v4: keep every linear in BF16")
    p.add_argument("--proposal-stages", type=int, default=0,
                   help="--family v4: also write this many `mtp.*` proposal stages with their prediction heads")
    p.set_defaults(fn=cmd_make_fixture)
    p = sub.add_parser("inspect-weightpack"); p.add_argument("model_dir"); p.add_argument("--json", action="store_true")
    p.add_argument("--limit", type=int, default=40); p.set_defaults(fn=cmd_inspect)
    p = sub.add_parser("generate"); _add_model_args(p)
    _add_generate_args(p); p.set_defaults(fn=cmd_generate)
    # the reference's name for greedy generation from a DeepSeek-V4 directory: speculative decoding with the
    # checkpoint's own drafter unless --no-speculative
    p = sub.add_parser("deepseek-v4-generate"); _add_model_args(p); _add_generate_args(p)
    p.add_argument("--no-speculative", action="store_true"); p.set_defaults(fn=cmd_generate, v4_generate=True)
    p = sub.add_parser("plan-placement"); _add_model_args(p)
    p.add_argument("--ranks", type=int, required=True, help="ranks the experts will be sharded over")
    p.add_argument("--requests", type=int, default=8); p.add_argument("--prompt-tokens", type=int, default=64)
    p.add_argument("--max-tokens", type=int, default=16); p.add_argument("--min-gain", type=float, default=0.02)
    p.add_argument("--out", help="write the report (with the plan) to this JSON file")
    p.set_defaults(fn=cmd_plan_placement)
    p = sub.add_parser("chat"); _add_model_args(p); p.add_argument("--max-tokens", type=int, default=128)
    p.set_defaults(fn=cmd_chat)
    p = sub.add_parser("serve"); _add_model_args(p)
    p.add_argument("--host", default="127.0.0.1"); p.add_argument("--port", type=int, default=8000)
    p.add_argument("--served-name", "--served-model-name", dest="served_name")
    p.add_argument("--command-queue", "--request-queue-capacity", dest="command_queue", type=int, default=256)
    p.add_argument("--event-queue", "--event-queue-capacity", dest="event_queue", type=int, default=32)
    p.add_argument("--admission-timeout", "--admission-timeout-secs", dest="admission_timeout", type=float, default=30.0)
    p.set_defaults(fn=cmd_serve)
    p = sub.add_parser("bench-interactive"); _add_model_args(p)
    p.add_argument("--turns", type=int, default=2); p.add_argument("--prompt-len", type=int, default=32)
    p.add_argument("--max-tokens", type=int, default=16); p.add_argument("--golden"); p.add_argument("--write-golden")
    p.add_argument("--trace", help="JSON {turns: [{prompt_tokens | prompt, max_tokens}]} instead of synthetic turns")
    p.set_defaults(fn=cmd_bench_interactive)
    p = sub.add_parser("generation-parity"); _add_model_args(p)
    p.add_argument("--cases", required=True); p.add_argument("--max-tokens", type=int, default=16)
    p.set_defaults(fn=cmd_generation_parity)
    p = sub.add_parser("chunk-sweep"); _add_model_args(p)
    p.add_argument("--chunks", type=int, nargs="+", default=[64, 128, 256, 512]); p.add_argument("--requests", type=int, default=4)
    p.add_argument("--prompt-len", type=int, default=256); p.add_argument("--max-tokens", type=int, default=8)
    p.set_defaults(fn=cmd_chunk_sweep)
    p = sub.add_parser("bench-serve")
    p.add_argument("--url", default="http://127.0.0.1:8000"); p.add_argument("--model", default="")
    p.add_argument("--concurrency", type=int, nargs="+", default=[1, 8, 32]); p.add_argument("--requests", type=int, default=64)
    p.add_argument("--seed", type=int, default=0); p.add_argument("--vocab", type=int, default=1024)
    p.add_argument("--min-in", type=int, default=128); p.add_argument("--max-in", type=int, default=8192)
    p.add_argument("--min-out", type=int, default=64); p.add_argument("--max-out", type=int, default=1024)
    p.add_argument("--shared-prefix", type=int, default=2048); p.add_argument("--shared-fraction", type=float, default=0.3)
    p.set_defaults(fn=cmd_bench_serve)
    p = sub.add_parser("expert-stream-smoke"); p.add_argument("model_dir"); p.add_argument("--device")
    p.add_argument("--device-mb", type=int, default=1024); p.add_argument("--residency", type=float, default=0.5)
    p.add_argument("--slabs", type=int, default=8); p.add_argument("--threads", type=int, default=4)
    p.add_argument("--host-cache-mb", type=int, default=256); p.add_argument("--timeout", type=float, default=120.0)
    p.set_defaults(fn=cmd_expert_stream_smoke)
    args = ap.parse_args(argv)
    from ..io.safetensors import CheckpointError
    try:
        return args.fn(args)
    except CheckpointError as exc:
        print(f"error: {exc}", file=sys.stderr)          # a checkpoint that cannot be bound: say why, no traceback
        return 2


if __name__ == "__main__":
    sys.exit(main())
