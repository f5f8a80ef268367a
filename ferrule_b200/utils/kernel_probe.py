"""Small, self-ending workloads of one kernel family each, for profiler captures and quick timings.

    python -m ferrule_b200.utils.kernel_probe <case> [reps]
    python -m ferrule_b200.utils.kernel_probe decode_step <layers> [eager|graph] [bf16|fp8_block|fp8_mxfp4]

Cases use decode-step shapes of the DeepSeek-V2-Lite configuration (batch 32, context about 640) unless
noted; weight sets are rotated through more buffers than fit in L2 where the kernel is bandwidth-bound, and
no case holds more than about 2 GB on the device.  Each case prints one JSON line with the CUDA-event time
per call.
"""
from __future__ import annotations

import json
import sys

import torch

from ferrule_b200.ops import kernels as K

DEV = "cuda"


def rnd(*s, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*s, device=DEV) * scale).to(dtype)


def timed(fn, reps):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(3 + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def case_attention(reps):
    """Paged MLA decode attention: 32 sequences x 16 heads, context 640, 8 KV splits merged in a cluster."""
    B, H, DL, DR, page, ctx = 32, 16, 512, 64, 64, 640
    D = DL + DR
    blocks = (ctx + page - 1) // page
    pool = rnd(B * blocks + 1, page, D, scale=0.3)
    bt = (torch.arange(B * blocks, device=DEV, dtype=torch.int32) + 1).view(B, blocks)
    q = rnd(B, H, D, scale=0.3)
    out = torch.zeros(B, H, DL, dtype=torch.bfloat16, device=DEV)
    rseq = torch.arange(B, device=DEV, dtype=torch.int32)
    rpos = torch.full((B,), ctx - 1, device=DEV, dtype=torch.int32)
    fn = lambda i: K.mla_attention(q, pool, bt, rseq, rpos, page, DL, DR, 0.07, out, splits=8, split_tokens=128)
    return timed(fn, reps), {"kv_bytes": B * ctx * D * 2}


def case_gemm_dense(reps):
    """q|kv_a projection: [32 x 2048] x [3648 x 2048]^T, weights rotated over 24 copies (360 MB)."""
    ws = [rnd(3648, 2048, scale=0.02) for _ in range(24)]
    x = rnd(32, 2048)
    out = torch.zeros(32, 3648, dtype=torch.bfloat16, device=DEV)
    return timed(lambda i: K.gemm(x, ws[i % 24], out=out), reps), {"weight_bytes": 3648 * 2048 * 2}


def _plan(T, k, E, ntok):
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).int()
    w = torch.rand(T, k, device=DEV)
    plan = K.MoePlan.allocate(T * k, E, ntok, DEV)
    K.moe_plan(idx, w, plan, 0, E, dst_slots=k + 1)
    return idx, w, plan


def case_gemm_grouped(reps):
    """Routed experts of one layer: 192 routes over 64 experts, gate|up + SwiGLU then down + scatter (1.1 GB of weights)."""
    T, k, E, H, I = 32, 6, 64, 2048, 1408
    idx, w, plan = _plan(T, k, E, 16)
    w13 = [rnd(E, 2 * I, H, scale=0.02) for _ in range(2)]
    w2 = [rnd(E, H, I, scale=0.02) for _ in range(2)]
    xg = rnd(T * k, H)
    hmid = torch.zeros(T * k, I, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(T * (k + 1), H, dtype=torch.bfloat16, device=DEV)

    def fn(i):
        K.gemm(xg, w13[i % 2], out=hmid, epilogue=K.EPI_SWIGLU, plan=plan)
        K.gemm(hmid, w2[i % 2], out=out, epilogue=K.EPI_SCATTER, plan=plan, scatter_rows=T * (k + 1))
    return timed(fn, reps), {"weight_bytes": E * 3 * H * I * 2}


def case_gemm_fp8(reps):
    """Block-scaled FP8 grouped gate|up + SwiGLU on the same expert shape (weights 0.37 GB per copy)."""
    from ferrule_b200.models.weights import QuantWeight
    from ferrule_b200.ops import quant as Q
    T, k, E, H, I = 32, 6, 64, 2048, 1408
    idx, w, plan = _plan(T, k, E, 16)
    qw = [QuantWeight.from_bf16(rnd(E, 2 * I, H, scale=0.02), "fp8_block") for _ in range(3)]
    xg = rnd(T * k, H)
    xq = Q.quant_fp8_rows(xg)
    hmid = torch.zeros(T * k, I, dtype=torch.bfloat16, device=DEV)
    fn = lambda i: Q.gemm_fp8(xq[0], xq[1], qw[i % 3].q, qw[i % 3].scale, out=hmid, epilogue=1, plan=plan)
    return timed(fn, reps), {"weight_bytes": E * 2 * I * H}


def case_small(reps):
    """The latency-bound kernels of one layer back to back: add+RMSNorm, fused router + plan, gather, MoE reduce,
    chunked arg-max, then the decode forms (static-slot router, reduce + norm)."""
    T, H, E, k = 32, 2048, 64, 6
    x, d = rnd(T, H), rnd(T, H)
    nw = torch.ones(H, dtype=torch.bfloat16, device=DEV)
    res, xn = torch.zeros_like(x), torch.zeros_like(x)
    rw = rnd(E, H, scale=0.05)
    plan = K.MoePlan.allocate(T * k, E, 16, DEV)
    idx = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, k, dtype=torch.float32, device=DEV)
    ctr = torch.zeros(4, dtype=torch.int32, device=DEV)
    xg = torch.zeros(T * k, H, dtype=torch.bfloat16, device=DEV)
    route_out = rnd(T * (k + 1), H)
    logits = torch.randn(T, 102400, device=DEV)
    scratch = K.ArgmaxScratch.allocate(T, DEV)
    nid = torch.zeros(T, dtype=torch.int32, device=DEV)
    nval = torch.zeros(T, dtype=torch.float32, device=DEV)

    cnt = torch.zeros(E, dtype=torch.int32, device=DEV)
    splan = K.static_plan(32, E, cnt)
    xgs = torch.zeros(E * 32, H, dtype=torch.bfloat16, device=DEV)
    x2, xn2 = torch.zeros_like(x), torch.zeros_like(x)

    def fn(i):
        K.add_rmsnorm(x, nw, 1e-6, delta=d, res_out=res, norm_out=xn)
        K.router_plan_fused(xn, rw, k, 0, plan, 0, E, idx, wts, ctr, dst_slots=k + 1)
        K.gather_rows(xn, plan, xg, cap_rows=T * k)
        K.moe_reduce(route_out, k + 1, k, idx, 0, E, T, H, residual=res, out=x)
        K.argmax_chunked(logits, scratch, nid, nval)
        # decode path: static per-expert row slots (router + reservation + gather) and reduce + next-layer norm
        cnt.zero_()
        K.router_append(xn, rw, k, 0, splan, 0, E, idx, wts, xgs, dst_slots=k + 1)
        K.moe_reduce_norm(route_out, k + 1, k, idx, 0, E, T, H, res, x2, nw, xn2, 1e-6)
    return timed(fn, reps), {}


def case_v4(reps):
    """DeepSeek-V4 operators at family size: hc_pre (4 x 4096), compressor pooling (ratio 4, overlap), indexer
    scores over 16384 compressed rows + top-512, selection attention over 128 + 512 rows."""
    from ferrule_b200.models import v4
    from ferrule_b200.ops import v4 as K4
    cfg = v4.HcConfig(4, 4096)
    T = 32
    state = rnd(T, 4, 4096)
    fn_w = torch.randn(cfg.mix, 4 * 4096, device=DEV) * 0.02
    scale = torch.tensor([0.7, 1.1, 0.9], device=DEV)
    base = torch.randn(cfg.mix, device=DEV) * 0.3
    kvp, gp = torch.randn(64, 1024, device=DEV), torch.randn(64, 1024, device=DEV)
    ape = torch.randn(4, 1024, device=DEV)
    n = 16384
    iq = rnd(T, 64, 128, scale=0.3)
    plane = rnd(n, 128, scale=0.3)
    hw = torch.randn(T, 64, device=DEV)
    table = rnd(n + 4096, 512, scale=0.3)
    q = rnd(T, 64, 512, scale=0.1)
    scores = torch.zeros(T, n, device=DEV)

    def fn(i):
        hid, coeff = K4.hc_pre(state, fn_w, scale, base, cfg)
        K4.hc_post(hid, state, coeff)
        K4.compressor_pool(kvp, gp, ape, 4, True)
        K4.indexer_scores(iq, plane, hw, out=scores)
        idx = K4.indexer_topk(scores, 512)
        win = torch.arange(n, n + 128, device=DEV, dtype=torch.int32)[None].expand(T, 128)
        sel = torch.cat([win, idx], dim=1).contiguous()
        K4.sparse_sink_attention(q, table, sel, 512, 0, 0.044, splits=4)
    return timed(fn, reps), {}


def case_prefill(reps):
    """One 2048-token prefill chunk (4 sequences x 512 new tokens, empty cache) through 2 layers (one dense, one
    MoE) of the DeepSeek-V2-Lite shape: the per-kernel launch list of this case is the prefill profile."""
    from ferrule_b200.models import config as C, deepseek as D, weights as W
    cfg = C.deepseek_v2_lite().with_(n_layers=2)
    w = W.random_weights(cfg, device=DEV, seed=0, fast_device_init=True)
    page, S, P = 64, 4, 512
    pool = D.KvPool(cfg, S * (P // page) + 2, page, DEV)
    fwd = D.CudaForward(w, pool, max_rows=2048, max_logit_rows=8, decode_rows=32, max_seq_len=1024, attn_splits=8)
    T = S * P
    i32 = dict(dtype=torch.int32, device=DEV)
    pos = torch.arange(P, **i32).repeat(S)
    seq = torch.arange(S, **i32).repeat_interleave(P)
    bt = (torch.arange(S * (P // page), **i32) + 1).view(S, P // page)
    slot = (bt[seq.long(), (pos // page).long()].long() * page + (pos % page).long())
    b = D.DeviceBatch(torch.randint(0, cfg.vocab_size, (T,), **i32), pos, slot, seq, pos.clone(), bt,
                      torch.arange(S, **i32) * P + P - 1, T, S)
    import os
    tc = os.environ.get("FERRULE_PREFILL_TC", "1") != "0"
    if tc:      # what the runner's batch staging adds for sequences with many query rows
        from ferrule_b200.ops import kernels as K
        tiles, rest = K.prefill_tiles([(i, i * P, P, 0) for i in range(S)], w.heads_local)
        b.tc_tiles, b.n_tc_tiles, b.rest_ranges = torch.from_numpy(tiles).to(DEV), len(tiles), rest
    return timed(lambda i: fwd.forward(b), reps), {"tokens": T, "attention": "tcgen05 tiles" if tc else "row tiles"}


def case_v3_fp8_decode(reps):
    """Decode step of one rank's TP8 / EP8 shard of the DeepSeek-V3 shape in FP8 (hidden 7168, 16 local heads,
    32 local experts), 4 layers (3 dense + 1 MoE), 64 sequences at context 256: launch list of the FP8 path."""
    import os
    from ferrule_b200.models import config as C, deepseek as D, weights as W
    fmt = os.environ.get("FERRULE_PROBE_FORMAT", "fp8_block")
    cfg = C.deepseek_v3().with_(n_layers=4, n_mtp_layers=0)
    w = W.random_weights(cfg, device=DEV, seed=0, tp_rank=0, tp_world=8, fast_device_init=True, weight_format=fmt)
    page, S, ctx = 64, 64, 256
    pool = D.KvPool(cfg, S * (ctx // page + 1) + 2, page, DEV)
    fwd = D.CudaForward(w, pool, max_rows=256, max_logit_rows=64, decode_rows=64, max_seq_len=512, attn_splits=4)
    i32 = dict(dtype=torch.int32, device=DEV)
    blocks = ctx // page + 1
    bt = (torch.arange(S * blocks, **i32) + 1).view(S, blocks)
    pos = torch.full((S,), ctx, **i32)
    seq = torch.arange(S, **i32)
    slot = bt[:, ctx // page].long() * page + ctx % page
    b = D.DeviceBatch(torch.randint(0, cfg.vocab_size, (S,), **i32), pos, slot, seq, pos.clone(), bt,
                      torch.arange(S, **i32), S, S)
    return timed(lambda i: fwd.forward(b), reps), {"format": fmt}


def case_decode_step(layers: int, eager: bool, weight_format: str = "bf16"):
    """One decode step of the DeepSeek-V2-Lite shape (bf16, batch 32, context 640) with `layers` layers.
    `eager`: three eager steps and nothing else - the form used for a launch list, where every kernel of the
    step is one launch.  Otherwise the step is captured in a CUDA graph and 20 replays are timed."""
    from ferrule_b200.models import config as C, deepseek as D, weights as W
    cfg = C.deepseek_v2_lite()
    cfg = cfg.with_(n_layers=layers or cfg.n_layers)
    w = W.random_weights(cfg, device=DEV, fast_device_init=True, weight_format=weight_format)
    B, ctx, page, max_blocks = 32, 640, 64, 16
    pool = D.KvPool(cfg, B * max_blocks + 1, page, DEV)
    pool.data.normal_(0, 0.3)
    fwd = D.CudaForward(w, pool, max_rows=64, max_logit_rows=64, decode_rows=64, max_seq_len=1024, attn_splits=8)
    g = D.DecodeGraph(fwd, B, B, max_blocks)
    bt = torch.arange(1, B * max_blocks + 1, dtype=torch.int32, device=DEV).view(B, max_blocks)
    g.batch.block_table.copy_(bt)
    g.batch.token_ids.random_(0, cfg.vocab_size)
    g.batch.positions.fill_(ctx)
    g.batch.row_pos.fill_(ctx)
    g.batch.row_seq.copy_(torch.arange(B, device=DEV))
    g.batch.write_slot.copy_((bt[:, ctx // page].long() * page + ctx % page))
    extra = {"layers": cfg.n_layers, "weight_bytes": w.nbytes(), "weight_format": weight_format}
    if eager:
        for _ in range(3):
            fwd.forward(g.batch)
        torch.cuda.synchronize()
        extra["launches_per_step"] = fwd.launches
        return 0.0, extra
    g.capture()
    extra["launches_per_step"] = g.launches
    us = timed(lambda i: g.replay(), 20)
    extra["tokens_per_s"] = round(B / us * 1e6, 1)
    return us, extra


CASES = {"v3_fp8_decode": case_v3_fp8_decode, "prefill": case_prefill, "attention": case_attention, "gemm_dense": case_gemm_dense, "gemm_grouped": case_gemm_grouped,
         "gemm_fp8": case_gemm_fp8, "small": case_small, "v4": case_v4}


def main() -> int:
    name = sys.argv[1] if len(sys.argv) > 1 else "attention"
    reps = int(sys.argv[2]) if len(sys.argv) > 2 else 20
    torch.manual_seed(0)
    if name == "decode_step":           # second argument: number of layers (0 = all), third: "eager"
        us, extra = case_decode_step(reps if len(sys.argv) > 2 else 0, len(sys.argv) > 3 and sys.argv[3] == "eager",
                                     sys.argv[4] if len(sys.argv) > 4 else "bf16")
        reps = 20
    else:
        us, extra = CASES[name](reps)
    out = {"case": name, "reps": reps, "us_per_call": round(us, 2)}
    out.update(extra)
    for key in ("weight_bytes", "kv_bytes"):
        if key in extra and us > 0:
            out["gb_per_s"] = round(extra[key] / us / 1e3, 1)
    from ferrule_b200.ops import _lib
    out["device_status"] = _lib.read_status()[0]
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
