"""utils: tokenizer streaming, chat templates, LRU, completion hub, failpoints, metrics, families."""
import asyncio
import threading

import pytest

from ferrule_b200.models.families import Family, TensorRole, classify, detect_family, layout_summary
from ferrule_b200.utils.async_wake import CompletionHub
from ferrule_b200.utils.errors import ErrorKind, FerruleError, quant_type
from ferrule_b200.utils.failpoints import FAILPOINTS, FailpointTriggered, OpCounters
from ferrule_b200.utils.memory import MemoryPoolLimits, OwnerMemoryLru
from ferrule_b200.utils.observability import Metrics
from ferrule_b200.utils.tokenizer import (ByteTokenizer, ChatMessage, ChatTemplate, IncrementalDecodeState,
                                          render_chat, template_for_model)


def test_incremental_decode_never_splits_utf8():
    tok = ByteTokenizer()
    text = "héllo 世界 🙂!"
    st = IncrementalDecodeState(tok)
    out = []
    for t in tok.encode(text):
        d = st.push(t)
        assert "�" not in d
        out.append(d)
    assert "".join(out) + st.finish() == text
    assert sum(1 for d in out if d == "") >= 6          # continuation bytes were held back


def test_chat_templates():
    msgs = [ChatMessage("system", "S"), ChatMessage("user", "hi")]
    assert render_chat(msgs, ChatTemplate.CHATML).endswith("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n")
    assert "<|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|>" in render_chat(msgs, ChatTemplate.LLAMA3)
    assert render_chat(msgs, ChatTemplate.DEEPSEEK) == "<｜begin▁of▁sentence｜>S<｜User｜>hi<｜Assistant｜>"
    assert render_chat(msgs[1:], ChatTemplate.QWEN).startswith("<|im_start|>system\nYou are a helpful assistant.")
    assert render_chat(msgs, ChatTemplate.PLAIN, add_generation_prompt=False) == "system: S\nuser: hi\n"
    assert template_for_model("DeepSeek-V3") == ChatTemplate.DEEPSEEK and template_for_model("x") == ChatTemplate.CHATML


def test_owner_lru_bytes_entries_and_pins():
    evicted = []
    lru = OwnerMemoryLru(MemoryPoolLimits(max_bytes=100, max_entries=3, reserve_bytes=10), lambda k, v: evicted.append(k))
    assert lru.put("a", 1, 40) and lru.put("b", 2, 40)
    assert lru.get("a") == 1                       # a becomes most recent
    assert lru.put("c", 3, 40) and evicted == ["b"] and lru.bytes == 80
    lru.pin("a")
    assert lru.put("d", 4, 50) and evicted == ["b", "c"]
    assert not lru.put("e", 5, 60) and "a" in lru   # only the pinned entry is left to evict
    assert not lru.put("big", 0, 95)
    lru.unpin("a")
    assert lru.put("e", 5, 60) and "a" not in lru


def test_completion_hub_no_lost_wakeup():
    hub = CompletionHub()
    t = hub.listen()
    hub.notify()                                     # notified between listen and wait
    assert hub.wait(t, timeout=0.0)
    t2 = hub.listen()
    assert not hub.wait(t2, timeout=0.01)
    threading.Timer(0.02, hub.notify).start()
    assert hub.wait(t2, timeout=2.0)

    async def main():
        tk = hub.listen()
        threading.Timer(0.02, hub.notify).start()
        assert await hub.wait_async(tk, timeout=2.0)
        assert not await hub.wait_async(hub.listen(), timeout=0.01)
    asyncio.run(main())


def test_failpoints_counters_errors_metrics():
    FAILPOINTS.disarm_all()
    FAILPOINTS.check("expert_upload")
    FAILPOINTS.arm("expert_upload", 2)
    for _ in range(2):
        with pytest.raises(FailpointTriggered):
            FAILPOINTS.check("expert_upload")
    FAILPOINTS.check("expert_upload")
    with pytest.raises(KeyError):
        FAILPOINTS.arm("nope")
    c = OpCounters()
    c.add("gemm", 3); c.add("gemm")
    assert c.snapshot() == {"gemm": 4}
    e = FerruleError(ErrorKind.IO, "short read", cleanup=[RuntimeError("x")]).context("expert 3").context("layer 1")
    assert str(e) == "[io] layer 1: expert 3: short read (+1 clean-up failure(s))"
    assert quant_type(12).bytes_for(512) == 288
    m = Metrics()
    m.add(requests_finished=2, ttft_sum_s=1.0)
    assert m.snapshot()["ttft_mean_s"] == 0.5


def test_family_classification():
    hf = ["model.embed_tokens.weight", "model.layers.3.self_attn.kv_a_proj_with_mqa.weight",
          "model.layers.3.mlp.experts.17.down_proj.weight_scale_inv", "model.layers.3.mlp.gate.weight",
          "model.layers.3.mlp.gate.e_score_correction_bias", "model.layers.0.mlp.up_proj.weight",
          "model.layers.61.eh_proj.weight", "lm_head.weight"]
    assert detect_family(hf) == Family.DEEPSEEK_HF
    c = classify(hf[2], Family.DEEPSEEK_HF, 61)
    assert (c.role, c.layer, c.expert, c.is_scale) == (TensorRole.EXPERT_DOWN, 3, 17, True)
    assert classify(hf[4], Family.DEEPSEEK_HF).role == TensorRole.ROUTER_BIAS
    assert classify(hf[5], Family.DEEPSEEK_HF).role == TensorRole.DENSE_UP
    assert classify(hf[6], Family.DEEPSEEK_HF, 61).mtp_stage == 0
    v4 = ["embed.weight", "layers.2.attn.wq_a.weight", "layers.2.attn.wq_a.scale", "layers.2.ffn.experts.5.w2.weight",
          "layers.0.ffn.gate.tid2eid", "layers.2.hc_attn_fn", "layers.2.attn.compressor.wkv.weight",
          "mtp.0.main_proj.weight", "mtp.0.ffn.experts.1.w1.scale", "layers.2.attn.attn_sink"]
    assert detect_family(v4) == Family.DEEPSEEK_V4
    roles = [classify(n, Family.DEEPSEEK_V4).role for n in v4]
    assert roles == [TensorRole.EMBEDDING, TensorRole.ATTN_Q_A, TensorRole.ATTN_Q_A, TensorRole.EXPERT_DOWN,
                     TensorRole.ROUTER_HASH, TensorRole.HYPER_CONNECTION, TensorRole.COMPRESSOR, TensorRole.MTP,
                     TensorRole.EXPERT_GATE, TensorRole.ATTN_SINK]
    assert classify(v4[8], Family.DEEPSEEK_V4).mtp_stage == 0
    assert layout_summary(hf, Family.DEEPSEEK_HF, 61)["expert_down"] == 1


def test_incremental_detokenisation_is_exact_and_linear():
    """Pushing token by token yields exactly the text of one decode of everything (multi-byte characters are held
    back until complete), and the cost per token does not grow with the length of the output."""
    import time
    from ferrule_b200.utils.tokenizer import ByteTokenizer, IncrementalDecodeState
    tok = ByteTokenizer()
    text = "héllo ✓ wörld — 日本語のテキスト 🙂 end"
    ids = tok.encode(text)
    st = IncrementalDecodeState(tok)
    out, partial = "", []
    for t in ids:
        d = st.push(t)
        assert "\\ufffd" not in d
        out += d
        partial.append(out)
    out += st.finish()
    assert out == tok.decode(ids) == text and st.emitted == text
    assert all(text.startswith(p) for p in partial)

    # a tokenizer whose pieces merge with their neighbours (a space is only known once the next piece arrives)
    class Merging:
        def decode(self, ids):
            return " ".join(f"w{t}" for t in ids).replace("w7 w8", "w78")
    m = Merging()
    seq = [1, 7, 8, 2, 7, 7, 8, 3]
    st = IncrementalDecodeState(m)
    got = "".join(st.push(t) for t in seq) + st.finish()
    assert got.replace(" ", "") == m.decode(seq).replace(" ", "")

    # an incomplete character at the very end is dropped, not emitted as a replacement character
    st = IncrementalDecodeState(tok)
    cut = tok.encode("ab✓")[:-1]
    assert "".join(st.push(t) for t in cut) + st.finish() == "ab"

    calls = {"tokens": 0}

    class Counting(ByteTokenizer):
        def decode(self, ids):
            calls["tokens"] += len(ids)
            return super().decode(ids)
    st = IncrementalDecodeState(Counting())
    t0 = time.perf_counter()
    for i in range(5000):
        st.push(97 + i % 26)
    assert calls["tokens"] < 5000 * 8, "a few token decodes per token, not the whole history"
    assert time.perf_counter() - t0 < 2.0


def test_owner_lru_failed_replacement_keeps_the_old_value():
    lru = OwnerMemoryLru(MemoryPoolLimits(max_bytes=100))
    assert lru.put("a", "A", 40) and lru.put("b", "B", 40)
    lru.pin("b")
    # replacing "a" by something that only fits if the pinned "b" went: refused, and "a" is still what it was
    assert not lru.put("a", "A2", 70)
    assert lru.get("a") == "A" and lru.bytes == 80 and len(lru) == 2
    lru.unpin("b")
    assert lru.put("a", "A2", 70) and lru.get("a") == "A2" and "b" not in lru and lru.bytes == 70


def test_owner_lru_random_operations_keep_the_byte_count():
    import random
    for seed in range(40):
        r = random.Random(seed)
        gone = []
        lru = OwnerMemoryLru(MemoryPoolLimits(max_bytes=r.randint(50, 200), max_entries=r.randint(1, 8),
                                              reserve_bytes=r.randint(0, 30)), lambda k, v: gone.append(k))
        model, pins = {}, {}
        for _ in range(300):
            k = r.randrange(12)
            op = r.random()
            if op < 0.5:
                n = r.randint(1, 90)
                before = dict(model)
                ok = lru.put(k, (k, n), n)
                for g in gone:
                    assert g not in pins and g != k
                    before.pop(g, None)
                gone.clear()
                model = before
                if ok:
                    model[k] = n
            elif op < 0.65:
                assert (lru.get(k) is not None) == (k in model)
            elif op < 0.8:
                assert (lru.pop(k) is not None) == (k in model)
                model.pop(k, None)
            elif op < 0.9:
                lru.pin(k)
                pins[k] = pins.get(k, 0) + 1
            else:
                lru.unpin(k)
                if pins.get(k, 0) <= 1:
                    pins.pop(k, None)
                else:
                    pins[k] -= 1
            assert set(lru.keys_lru_first()) == set(model) and lru.bytes == sum(model.values())
            assert lru.bytes <= lru.limits.usable() and len(lru) <= lru.limits.max_entries
