"""Decode-step probe for profiling: DeepSeek-V2-Lite shape, batch 32, one decode step.

  python -m ferrule_b200.utils.decode_probe [layers] [eager]

Builds random-init weights with `layers` layers (default: all 27), fills a KV pool for a context of
640 tokens, then either captures the step in a CUDA graph and times 20 replays with CUDA events, or
(with `eager`) runs three eager steps and exits - the form used under `ncu`, where every kernel of
the step is one launch.
"""
import sys, time, torch
from ferrule_b200.models import config as C, deepseek as D, weights as W
cfg = C.deepseek_v2_lite()
layers = int(sys.argv[1]) if len(sys.argv) > 1 else cfg.n_layers
cfg = cfg.with_(n_layers=layers)
dev = "cuda"
t0 = time.time()
w = W.random_weights(cfg, device=dev, fast_device_init=True)
torch.cuda.synchronize(); print("weights", w.nbytes()/1e9, "GB", time.time()-t0, "s", flush=True)
B, ctx, page = 32, 640, 64
max_blocks = 16
pool = D.KvPool(cfg, B*max_blocks+1, page, dev)
pool.data.normal_(0, 0.3)
fwd = D.CudaForward(w, pool, max_rows=64, max_logit_rows=64, decode_rows=64, max_seq_len=1024, attn_splits=8)
g = D.DecodeGraph(fwd, B, B, max_blocks)
bt = torch.arange(1, B*max_blocks+1, dtype=torch.int32, device=dev).view(B, max_blocks)
g.batch.block_table.copy_(bt)
g.batch.token_ids.random_(0, cfg.vocab_size)
g.batch.positions.fill_(ctx); g.batch.row_pos.fill_(ctx)
g.batch.row_seq.copy_(torch.arange(B, device=dev))
g.batch.write_slot.copy_((bt[:, ctx//page].long()*page + ctx % page))
if len(sys.argv) > 2 and sys.argv[2] == "eager":
    for _ in range(3): fwd.forward(g.batch)
    torch.cuda.synchronize(); print("eager done", fwd.launches); sys.exit(0)
g.capture(); print("launches/step", g.launches, flush=True)
from ferrule_b200.ops import _lib
print("status", _lib.read_status())
for _ in range(3): g.replay()
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
N = 20
e0.record()
for _ in range(N): g.replay()
e1.record(); torch.cuda.synchronize()
ms = e0.elapsed_time(e1)/N
print(f"decode step {ms:.3f} ms -> {B/ms*1000:.0f} tok/s; weight bytes/step floor {w.nbytes()/6.55e12*1e3:.3f} ms")
# eager per-kernel breakdown via events
fwd.forward(g.batch); torch.cuda.synchronize()
e0.record(); fwd.forward(g.batch); e1.record(); torch.cuda.synchronize()
print("eager step", e0.elapsed_time(e1), "ms")
