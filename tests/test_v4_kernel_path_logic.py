"""Host-side logic of the DeepSeek-V4 kernel path (`V4Cuda`, the runner's batched execution) on CPU: the kernel
wrappers are replaced by PyTorch stand-ins with the same contracts (`tests/v4_cpu_shim.py`), everything else -
positions, table addressing, selection lists, compressor group boundaries, batched rows, QAT hooks, the proposal
planes - is the code that runs on the GPU."""
import pytest
import torch

import v4_cpu_shim as shim
from ferrule_b200.models import v4_model as M
from ferrule_b200.models.v4_runner import V4Runner
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest


def _cfg(**kw):
    return M.tiny_v4().with_(n_proposal_stages=2, proposal_target_layers=(0, 2), proposal_noise_token=3,
                             proposal_markov_rank=16, **kw)


def _same(a, b, qat):
    """Equal up to matmul summation order; with QAT a value on a rounding boundary may land on the neighbouring
    FP8 / FP4 code in one of the two runs, so a small share of entries may differ by one quantisation step."""
    a, b = a.float(), b.float()
    off = (a - b).abs() > 2e-2
    if not qat:
        return not bool(off.any())
    return float(off.float().mean()) < 0.02 and float((a - b).abs().max()) <= 0.3 * float(b.abs().max())


def _tokens(cfg, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()


@pytest.mark.parametrize("qat", [False, True])
def test_kernel_path_decodes_what_the_oracle_decodes(qat):
    cfg = _cfg(qat=qat)
    w = M.random_v4_weights(cfg, seed=0)
    oracle, cache = M.V4Reference(w), M.V4SeqCache(cfg)
    model = shim.install(M.V4Cuda(w, max_seqs=2, max_len=64))
    for t in _tokens(cfg, 26):
        want = oracle.step(cache, t)
        nxt, logits = model.step([1], [t])
        assert torch.allclose(logits[0], want, atol=1e-3 * float(want.abs().max()))
        assert int(nxt[0]) == int(want.argmax())
    # the proposal planes hold the oracle's context rows, and the drafts agree
    for s in range(cfg.n_proposal_stages):
        assert torch.allclose(model.pctx[s][1, :26].float(), torch.stack(cache.pctx[s]), atol=1e-2)
    assert model.propose(1, 26, 5)[0] == oracle.propose(cache, 26, 5)[0]
    assert model.propose(1, 10, 5)[0] == oracle.propose(cache, 10, 5)[0]


@pytest.mark.parametrize("qat", [False, True])
def test_a_batch_of_rows_equals_the_same_rows_one_at_a_time(qat):
    """Two prompt chunks and a decode row in one pass: chunk rows cross compressor group boundaries (ratio 4 and
    8), the indexed layer picks among rows that the same pass wrote, the window slides inside the chunk."""
    cfg = _cfg(qat=qat)
    w = M.random_v4_weights(cfg, seed=1)
    a, b, c = _tokens(cfg, 21, 1), _tokens(cfg, 13, 2), _tokens(cfg, 9, 3)
    one = shim.install(M.V4Cuda(w, max_seqs=3, max_len=64))
    many = shim.install(M.V4Cuda(w, max_seqs=3, max_len=64, max_rows=64))
    # sequence 2 is 8 tokens in on both; sequence 0 has its first 6 tokens
    for m in (one, many):
        for t in c[:8]:
            m.step([2], [t])
        for t in a[:6]:
            m.step([0], [t])
    last = {}
    for t in a[6:]:
        last[0] = one.step([0], [t])[1][0]
    for t in b:
        last[1] = one.step([1], [t])[1][0]
    last[2] = one.step([2], [c[8]])[1][0]
    seqs = [0] * 15 + [1] * 13 + [2]
    pos = list(range(6, 21)) + list(range(13)) + [8]
    nxt, logits = many.step_rows(seqs, a[6:] + b + [c[8]], pos, want_rows=[14, 27, 28])
    assert logits.shape[0] == 3
    for k, s in enumerate((0, 1, 2)):
        assert torch.allclose(logits[k], last[s], atol=(0.15 if qat else 2e-2) * float(last[s].abs().max()))
        top2 = last[s].topk(2).values
        if float(top2[0] - top2[1]) > 0.3 * float(last[s].abs().max()) or not qat:
            assert int(nxt[k]) == int(last[s].argmax())
    assert many.positions == one.positions == [21, 13, 9]
    for layer in range(cfg.n_layers):
        assert _same(many.tables[layer], one.tables[layer], qat)
    assert _same(many.iplane[1], one.iplane[1], qat)
    for s in range(cfg.n_proposal_stages):
        assert _same(many.pctx[s], one.pctx[s], qat)
    # rows out of order within a sequence are refused
    with pytest.raises(AssertionError):
        many.step_rows([0, 0], [1, 2], [22, 21])
    assert many.step_rows([0], [1], [21], want_rows=[]) == (None, None)


def _engine_on_kernel_path(w, speculative, batched):
    runner = V4Runner(w, n_pages=48, page_size=16, max_seqs=4, max_seq_len=128, max_rows=64, batched_prefill=batched)
    # the runner was built on CPU tensors: give it the kernel path with stand-in kernels
    runner.is_cuda = True
    runner.fwd = shim.install(M.V4Cuda(w, 4, 128, max_rows=64 if batched else 0))
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=12,
                            ctx_size=128)
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=48, page_size=16, speculative=speculative, max_draft=5,
                                       confidence_threshold=0.0)), runner


def _greedy(w, prompt, n_new):
    r, c = M.V4Reference(w), M.V4SeqCache(w.cfg)
    for t in prompt:
        logits = r.step(c, t)
    out = []
    for _ in range(n_new):
        out.append(int(torch.argmax(logits)))
        logits = r.step(c, out[-1])
    return out


@pytest.mark.parametrize("speculative,batched", [(False, True), (True, True), (True, False)])
def test_engine_on_the_kernel_path_streams_the_oracle_tokens(speculative, batched):
    w = M.random_v4_weights(_cfg(), seed=3)
    prompts = [_tokens(w.cfg, n, 10 + n) for n in (9, 20, 14)]
    eng, runner = _engine_on_kernel_path(w, speculative, batched)
    for i, p in enumerate(prompts):
        eng.submit(GenerateRequest(f"r{i}", p, max_new_tokens=8, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=5000)
    for i, p in enumerate(prompts):
        got = [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == f"r{i}"]
        assert got == _greedy(w, p, 8)
    if speculative:
        assert eng.spec.metrics.drafted > 0 and runner.proposal_blocks > 0
    if batched:
        # prompts of 9 + 20 + 14 tokens in chunks of 12 under a 32-row budget: far fewer passes than tokens
        assert runner.steps < 43
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0
