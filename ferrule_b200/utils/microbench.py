"""Warm per-kernel latencies: every kernel of the decode step, timed inside a CUDA graph (50 calls per
graph, weights rotated through more buffers than fit in L2).

  python -m ferrule_b200.utils.microbench
"""
import torch
from ferrule_b200.ops import kernels as K
dev = "cuda"
def rnd(*s, scale=1.0):
    return (torch.randn(*s, device=dev) * scale).to(torch.bfloat16)
def timeit(fn, n=200):
    for _ in range(10): fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n): fn(i)
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1000
def graph_time(fn, n=50, reps=20):
    """n calls captured in one graph -> per-call us without host launch overhead."""
    s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(3): fn(i)
    torch.cuda.current_stream().wait_stream(s); torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n): fn(i)
    g.replay(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps): g.replay()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (n * reps) * 1000


def main() -> None:
    T = 32
    x2048 = rnd(T, 2048)
    NB = 24
    for name, n, k in [("o_proj 2048x2048", 2048, 2048), ("qkv 3648x2048", 3648, 2048), ("shared_down 2048x2816", 2048, 2816), ("router 64x2048", 64, 2048)]:
        ws = [rnd(n, k, scale=0.02) for _ in range(NB)]
        x = rnd(T, k)
        out = torch.zeros(T, n, dtype=torch.bfloat16, device=dev)
        for split in (1, 2, 4, 8):
            try:
                t = graph_time(lambda i: K.gemm(x, ws[i % NB], out=out, split_k=split))
                print(f"{name:28s} split {split}: {t:7.2f} us  ({n*k*2/t/1e6:.2f} TB/s)")
            except Exception as e:
                print(f"{name:28s} split {split}: n/a")
        del ws
    ws = [rnd(2 * 2816, 2048, scale=0.02) for _ in range(NB)]
    out = torch.zeros(T, 2816, dtype=torch.bfloat16, device=dev)
    for split in (1, 2, 4):
        t = graph_time(lambda i: K.gemm(x2048, ws[i % NB], out=out, epilogue=K.EPI_SWIGLU, split_k=split))
        print(f"shared gate/up swiglu          split {split}: {t:7.2f} us")
    del ws
    # small elementwise
    w = rnd(2048)
    o = torch.zeros(T, 2048, dtype=torch.bfloat16, device=dev)
    print("add_rmsnorm", graph_time(lambda i: K.add_rmsnorm(x2048, w, 1e-6, norm_out=o)))
    # empty-ish kernel floor: embedding of 32 rows
    tab = rnd(1000, 2048); ids = torch.randint(0, 1000, (T,), device=dev, dtype=torch.int32)
    print("embedding", graph_time(lambda i: K.embedding(ids, tab, out=o)))
    # attention decode
    heads, dl, dr, page = 16, 512, 64, 64
    ctx = 640
    S = 32; mb = 16
    pool = rnd(S * mb * page + page, dl + dr, scale=0.3)
    bt = torch.arange(S * mb, dtype=torch.int32, device=dev).view(S, mb)
    rs = torch.arange(S, dtype=torch.int32, device=dev); rp = torch.full((S,), ctx, dtype=torch.int32, device=dev)
    q = rnd(S, heads, dl + dr, scale=0.3)
    ao = torch.zeros(S, heads, dl, dtype=torch.bfloat16, device=dev)
    for splits, st in [(1, 1 << 20), (4, 256), (8, 128), (16, 64)]:
        for mik in (True, False):
            if splits == 1 and not mik: continue
            wsa = K.AttnWorkspace(torch.zeros(S, splits, heads, dl, device=dev), torch.zeros(S, splits, heads, 2, device=dev), S, splits,
                                  torch.zeros(S, dtype=torch.int32, device=dev) if mik else None) if splits > 1 else None
            t = graph_time(lambda i: K.mla_attention(q, pool, bt, rs, rp, page, dl, dr, 0.1, ao, splits=splits, split_tokens=st, ws=wsa))
            print(f"attention ctx {ctx} splits {splits} merge_in_kernel {mik}: {t:7.2f} us")
        if splits in (2, 4, 8):
            t = graph_time(lambda i: K.mla_attention(q, pool, bt, rs, rp, page, dl, dr, 0.1, ao, splits=splits, split_tokens=st, ws=None))
            print(f"attention ctx {ctx} splits {splits} cluster merge: {t:7.2f} us")
    # router fused vs separate
    wr = rnd(64, 2048, scale=0.02)
    plan = K.MoePlan.allocate(T * 6, 64, 16, dev)
    idx = torch.zeros(T, 6, dtype=torch.int32, device=dev); wts = torch.zeros(T, 6, device=dev); ctr = torch.zeros(4, dtype=torch.int32, device=dev)
    print("router_plan_fused", graph_time(lambda i: K.router_plan_fused(x2048, wr, 6, 0, plan, 0, 64, idx, wts, ctr, dst_slots=7)))
    lg = torch.zeros(T, 64, device=dev)
    def sep(i):
        K.gemm(x2048, wr, out=lg); K.router_topk(lg, 6, 0, out_idx=idx, out_w=wts); K.moe_plan(idx, wts, plan, 0, 64, dst_slots=7)
    print("router separate (3 kernels)", graph_time(sep))
    print("moe_plan alone", graph_time(lambda i: K.moe_plan(idx, wts, plan, 0, 64, dst_slots=7)))


if __name__ == "__main__":
    main()
