"""Number formats, safetensors IO and checkpoint round trips (CPU)."""
import json

import pytest
import torch

from ferrule_b200.io import encoding as enc
from ferrule_b200.io.checkpoint import export_hf, infer_weight_format, load_deepseek_hf
from ferrule_b200.io.safetensors import CheckpointError, SafetensorsFile, ShardedCheckpoint, save_file
from ferrule_b200.models import config as C
from ferrule_b200.models import weights as W


def test_e8m0_e4m3_e2m1_codecs():
    b = torch.tensor([0, 1, 126, 127, 128, 254, 255], dtype=torch.uint8)
    s = enc.e8m0_decode(b)
    assert s[3] == 1.0 and s[2] == 0.5 and s[4] == 2.0 and s[0] == 2.0 ** -127 and torch.isnan(s[6])
    assert enc.e8m0_encode_ceil(torch.tensor([1.0, 1.1, 0.24, 448.0])).tolist() == [127, 128, 125, 136]
    all_codes = torch.arange(256, dtype=torch.uint8)
    v = enc.e4m3_decode(all_codes)
    assert v[0x7e] == 448.0 and torch.isnan(v[0x7f]) and torch.isnan(v[0xff]) and v[0x38] == 1.0
    finite = ~torch.isnan(v)
    rt = enc.e4m3_encode(v[finite])
    assert torch.equal(rt & 0x7f, all_codes[finite] & 0x7f)            # every finite code survives a round trip
    assert enc.e4m3_decode(enc.e4m3_encode(torch.tensor([1e6, -1e6]))).tolist() == [448.0, -448.0]
    nib = torch.arange(16, dtype=torch.uint8)
    vals = enc.fp4_decode_nibbles(nib)
    assert vals.tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6]
    assert enc.fp4_encode_nibbles(vals[:8]).tolist() == list(range(8))
    assert enc.fp4_encode_nibbles(torch.tensor([0.25, 0.75, 2.5, 5.0, 100.0, -2.4])).tolist() == [0, 2, 4, 6, 7, 12]
    x = torch.tensor([[0.5, -1.0, 6.0, 0.0]])
    p = enc.fp4_pack(x)
    assert p.tolist() == [[0x01 | (0x0a << 4), 0x07 | (0x00 << 4)]]          # low nibble first
    assert torch.equal(enc.fp4_unpack(p), x)


def test_activation_and_weight_quantisation():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 256, generator=g) * 3
    q, sb = enc.act_quant_fp8(x)
    assert q.shape == (5, 256) and sb.shape == (5, 2)
    back = enc.act_dequant_fp8(q, sb)
    assert float(((back - x).abs() / (x.abs() + 0.1)).max()) < 0.08
    # power-of-two scale with ceil: the block max never saturates
    scale = enc.e8m0_decode(sb)
    assert float((x.view(5, 2, 128).abs().amax(-1) / scale).max()) <= 448.0
    tiny = torch.full((1, 128), 1e-7)
    _, sbt = enc.act_quant_fp8(tiny)
    assert float(enc.e8m0_decode(sbt)) == 2.0 ** -22              # amax floor 1e-4 / 448 -> 2^-22
    w = torch.randn(200, 300, generator=g) * 0.05
    qw, sw = enc.weight_quant_fp8_block(w)
    assert qw.shape == w.shape and sw.shape == (2, 3)
    assert float(((enc.weight_dequant_fp8_block(qw, sw) - w).abs()).max()) < 0.01
    w4 = torch.randn(16, 128, generator=g)
    p4, s4 = enc.weight_quant_mxfp4(w4)
    assert p4.shape == (16, 64) and s4.shape == (16, 4)
    err = (enc.weight_dequant_mxfp4(p4, s4) - w4).abs() / (w4.view(16, 4, 32).abs().amax(-1, keepdim=True).expand(16, 4, 32).reshape(16, 128) + 1e-6)
    assert float(err.max()) < 0.26
    h = enc.hadamard(torch.eye(8))
    assert torch.allclose(h @ h.T, torch.eye(8), atol=1e-6)
    y = torch.randn(3, 64, generator=g)
    assert torch.allclose(enc.hadamard(enc.hadamard(y)), y, atol=1e-5)
    assert torch.equal(enc.fp8_qat(y.repeat(1, 2)), enc.fp8_qat(y.repeat(1, 2)).bfloat16().float())


def test_safetensors_roundtrip_and_validation(tmp_path):
    t = {"a": torch.arange(12, dtype=torch.float32).view(3, 4), "b": torch.randn(5, 6).bfloat16(),
         "q": torch.arange(8, dtype=torch.uint8), "i": torch.tensor([[1, -2]], dtype=torch.int64)}
    p = tmp_path / "x.safetensors"
    save_file(t, p, {"q": "F8_E4M3"}, {"format": "pt"})
    f = SafetensorsFile(p)
    assert f.tensors["q"].dtype == "F8_E4M3" and f.metadata == {"format": "pt"}
    for k in t:
        assert torch.equal(f.read(k), t[k])
    assert torch.equal(f.read_rows("a", 1, 3), t["a"][1:3])
    with pytest.raises(CheckpointError):
        f.read("a", max_bytes=8)
    with pytest.raises(CheckpointError):
        f.read("nope")
    f.close()
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(CheckpointError):
        SafetensorsFile(bad)


@pytest.mark.parametrize("dense,expert", [("plain", "plain"), ("fp8_block", "mxfp4")])
def test_checkpoint_export_load_roundtrip(tmp_path, dense, expert):
    cfg = C.tiny_fixture()
    w = W.random_weights(cfg, dtype=torch.bfloat16, seed=3)
    export_hf(w, tmp_path, dense_format=dense, expert_format=expert, shard_bytes=1 << 20)
    ck = ShardedCheckpoint(tmp_path)
    assert len(set(ck.weight_map.values())) > 1                      # really sharded
    fmt = infer_weight_format(ck, "model.layers.1.mlp.experts.0.gate_proj")
    assert fmt[0] == ("plain" if expert == "plain" else "mxfp4") and (expert == "plain" or fmt[2] == 32)
    assert infer_weight_format(ck, "model.layers.0.self_attn.o_proj")[0] == dense
    plan = ck.read_plan([n for n in ck.names() if "experts.3." in n and "layers.1." in n])
    assert plan and all(off % 4096 == 0 and ln % 4096 == 0 for _, off, ln in plan)
    assert ck.source_identity() == ShardedCheckpoint(tmp_path).source_identity()
    w2 = load_deepseek_hf(tmp_path)
    assert w2.cfg.n_routed_experts == cfg.n_routed_experts and len(w2.mtp) == 1
    tol = 0.0 if dense == "plain" else 0.02
    for a, b in zip(w.layers, w2.layers):
        assert float((a.w_o.float() - b.w_o.float()).abs().max()) <= tol * 0.2 + 1e-9
        assert float((a.w_uk_t.float() - b.w_uk_t.float()).abs().max()) <= tol * 0.2 + 1e-9
        if a.is_moe:
            d = (a.e_w13.float() - b.e_w13.float()).abs().max()
            assert float(d) <= (0.0 if expert == "plain" else 0.03)
    # tensor-parallel load takes the matching slices
    w_tp = load_deepseek_hf(tmp_path, tp_rank=1, tp_world=2)
    assert torch.equal(w_tp.layers[1].e_w2, w2.layers[1].e_w2[4:])
    assert torch.equal(w_tp.lm_head, w2.lm_head[512:])


def test_v4_checkpoint_directory_round_trip_and_serving(tmp_path):
    """A DeepSeek-V4 directory in the published layout (FP8 attention / shared experts, packed FP4 routed
    experts, per-expert w1 / w3 / w2 triples): the loader binds every tensor, the loaded linears equal the
    format's round trip of the originals, the oracle decodes the same tokens from both, and the CLI serves the
    directory through the engine."""
    import json
    from ferrule_b200.cli.main import main as cli_main
    from ferrule_b200.io import encoding as enc
    from ferrule_b200.io.safetensors import ShardedCheckpoint
    from ferrule_b200.io.v4_checkpoint import export_v4_hf, load_v4_hf, v4_config_from_hf, v4_config_to_hf
    from ferrule_b200.models.v4_model import V4Reference, V4SeqCache, random_v4_weights, tiny_v4
    cfg = tiny_v4()
    assert v4_config_from_hf(v4_config_to_hf(cfg)) == cfg
    w = random_v4_weights(cfg, seed=4)
    d = tmp_path / "v4"
    export_v4_hf(w, d, shard_bytes=1 << 20)
    ck = ShardedCheckpoint(d)
    names = set(ck.names())
    assert ck.info("layers.1.attn.wq_a.weight").dtype == "F8_E4M3" and ck.info("layers.1.attn.wq_a.scale").dtype == "F8_E8M0"
    assert ck.info("layers.2.ffn.experts.3.w1.weight").dtype == "I8"
    assert ck.info("layers.2.ffn.experts.3.w1.weight").shape == (cfg.moe_inter, cfg.hidden // 2)
    assert "layers.0.ffn.gate.tid2eid" in names and "layers.1.ffn.gate.bias" in names
    assert "layers.1.attn.indexer.wq_b.weight" in names and "layers.0.attn.compressor.wkv.weight" not in names
    ck.close()
    got = load_v4_hf(d)
    assert got.cfg == cfg and len(got.layers) == cfg.n_layers
    l1, o1 = got.layers[1], w.layers[1]
    q, sb = enc.weight_quant_fp8_block(o1.wq_b.float())
    assert torch.equal(l1.wq_b, enc.weight_dequant_fp8_block(q, sb).to(torch.bfloat16))
    p_, s_ = enc.weight_quant_mxfp4(o1.e_w13[5][:cfg.moe_inter].float())
    assert torch.equal(l1.e_w13[5][:cfg.moe_inter], enc.weight_dequant_mxfp4(p_, s_, 32).to(torch.bfloat16))
    assert l1.wo_a.shape == o1.wo_a.shape and torch.equal(l1.hc_attn_fn, o1.hc_attn_fn)
    assert torch.equal(got.layers[0].hash_table, w.layers[0].hash_table) and torch.equal(l1.c_ape, o1.c_ape)
    # writing the loaded (already representable) values again changes nothing
    export_v4_hf(got, tmp_path / "again", shard_bytes=1 << 30)
    again = load_v4_hf(tmp_path / "again")
    assert torch.equal(again.layers[2].e_w2, got.layers[2].e_w2) and torch.equal(again.layers[2].wkv, got.layers[2].wkv)

    def decode(weights, n=6):
        m, c = V4Reference(weights), V4SeqCache(weights.cfg)
        tok, out = 17, []
        for _ in range(n):
            tok = int(m.step(c, tok).argmax())
            out.append(tok)
        return out
    assert decode(got) == decode(again)
    # the CLI: info recognises the family, generate serves the directory
    import io, contextlib
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli_main(["info", "--model-dir", str(d)]) == 0
    info = json.loads(buf.getvalue())
    assert info["checkpoint"]["family"] == "deepseek_v4" and info["engine_plan"]["family"] == "deepseek-v4"
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli_main(["generate", "--model-dir", str(d), "--device", "cpu", "--tokens", "5,9,11", "--max-tokens", "4",
                         "--ignore-eos", "--ctx-size", "64", "--page-size", "16", "--max-seqs", "2"]) == 0
    assert "tokens" in buf.getvalue() or len(buf.getvalue()) > 0
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli_main(["make-fixture", "--family", "v4", "--out", str(tmp_path / "fx"), "--layers", "2"]) == 0
    assert json.loads(buf.getvalue())["expert_format"] == "mxfp4" and load_v4_hf(tmp_path / "fx").cfg.n_layers == 2


def test_v4_checkpoint_carries_the_proposal_attachment(tmp_path):
    """The `mtp.*` namespace: stage bodies, stage 0's projection of the target taps, the last stage's heads.  The
    loaded drafter proposes what the written one does (plain format: bit equal), and the CLI serves the
    directory with speculative decoding - the same tokens as without."""
    import contextlib, io, json
    from ferrule_b200.cli.main import main as cli_main
    from ferrule_b200.io.safetensors import ShardedCheckpoint
    from ferrule_b200.io.v4_checkpoint import export_v4_hf, load_v4_hf, v4_config_from_hf, v4_config_to_hf
    from ferrule_b200.models.v4_model import V4Reference, V4SeqCache, random_v4_weights, tiny_v4
    cfg = tiny_v4().with_(n_proposal_stages=2, proposal_target_layers=(0, 2), proposal_noise_token=3, proposal_markov_rank=16)
    assert v4_config_from_hf(v4_config_to_hf(cfg)) == cfg
    w = random_v4_weights(cfg, seed=6)
    d = tmp_path / "v4p"
    export_v4_hf(w, d, dense_format="plain", expert_format="plain")
    ck = ShardedCheckpoint(d)
    names = set(ck.names())
    ck.close()
    for n in ("mtp.0.main_proj.weight", "mtp.0.main_norm.weight", "mtp.1.attn.wkv.weight", "mtp.1.ffn.gate.bias",
              "mtp.1.hc_head_fn", "mtp.1.norm.weight", "mtp.1.markov_head.markov_w1.weight",
              "mtp.1.markov_head.markov_w2.weight", "mtp.1.confidence_head.proj.weight", "mtp.0.ffn.experts.7.w2.weight"):
        assert n in names, n
    assert "mtp.0.hc_head_fn" not in names and "mtp.1.main_proj.weight" not in names
    assert "mtp.0.attn.compressor.wkv.weight" not in names and "mtp.0.ffn.gate.tid2eid" not in names
    got = load_v4_hf(d)
    assert got.cfg == cfg and got.proposal is not None and len(got.proposal.stages) == 2
    assert torch.equal(got.proposal.markov_w2, w.proposal.markov_w2) and torch.equal(got.proposal.main_proj, w.proposal.main_proj)

    def drafts(weights):
        m, c = V4Reference(weights), V4SeqCache(weights.cfg)
        for t in (5, 9, 11, 200, 31, 7):
            logits = m.step(c, t)
        return m.propose(c, 6, int(logits.argmax()))
    assert drafts(got) == drafts(w)
    outs = []
    for extra in ([], ["--speculative"]):
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            assert cli_main(["generate", "--model-dir", str(d), "--device", "cpu", "--tokens", "5,9,11", "--max-tokens", "6",
                             "--ignore-eos", "--ctx-size", "64", "--page-size", "16", "--max-seqs", "2"] + extra) == 0
        outs.append(json.loads(buf.getvalue().strip().splitlines()[-1]))
    assert outs[0]["tokens"] == outs[1]["tokens"] and len(outs[0]["tokens"]) == 6
    # a directory without stages refuses --speculative instead of silently decoding plainly
    export_v4_hf(random_v4_weights(tiny_v4(), seed=6), tmp_path / "bare", dense_format="plain", expert_format="plain")
    with pytest.raises(SystemExit):
        cli_main(["generate", "--model-dir", str(tmp_path / "bare"), "--device", "cpu", "--tokens", "5", "--max-tokens", "2",
                  "--speculative", "--ctx-size", "64", "--page-size", "16", "--max-seqs", "2"])
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli_main(["make-fixture", "--family", "v4", "--out", str(tmp_path / "fxp"), "--layers", "2",
                         "--proposal-stages", "1", "--plain"]) == 0
    assert json.loads(buf.getvalue())["proposal_stages"] == 1 and load_v4_hf(tmp_path / "fxp").proposal is not None


def test_damaged_safetensors_headers_are_checkpoint_errors(tmp_path):
    """Flipped header bytes, truncated files, wrong field types and absurd lengths: the reader answers with
    CheckpointError every time (or reads a file whose damage happens to be harmless), never with a stray exception."""
    import os, random, struct
    from ferrule_b200.io.safetensors import CheckpointError, ShardedCheckpoint, write_sharded
    t = {"a.weight": torch.randn(4, 8).to(torch.bfloat16), "b": torch.arange(10, dtype=torch.int64),
         "c.scale": torch.ones(3, dtype=torch.uint8)}
    write_sharded(t, tmp_path, 1 << 20, {})
    path = next(p for p in tmp_path.iterdir() if p.suffix == ".safetensors")
    good = path.read_bytes()
    hlen = struct.unpack("<Q", good[:8])[0]
    rnd = random.Random(0)
    outcomes = set()
    for _ in range(400):
        b = bytearray(good)
        mode = rnd.random()
        if mode < 0.4:
            for _ in range(rnd.randrange(1, 4)):
                b[rnd.randrange(0, 8 + hlen)] = rnd.randrange(256)
        elif mode < 0.6:
            b = b[:rnd.randrange(0, len(b))]
        elif mode < 0.8:
            hdr = json.loads(good[8:8 + hlen])
            k = rnd.choice([k for k in hdr if k != "__metadata__"])
            hdr[k][rnd.choice(["dtype", "shape", "data_offsets"])] = rnd.choice(
                [None, "X", [], [-1, 5], [0, 10 ** 12], [5, 1], "BF16", [2 ** 40, 2], {"a": 1}, 7, [True, 2]])
            if rnd.random() < 0.2:
                del hdr[k][rnd.choice(list(hdr[k]))]
            raw = json.dumps(hdr).encode()
            b = bytearray(struct.pack("<Q", len(raw)) + raw + good[8 + hlen:])
        else:
            b[:8] = struct.pack("<Q", rnd.choice([0, 1, 2 ** 63, len(good) * 2, hlen + 1, hlen - 1]))
        path.write_bytes(bytes(b))
        try:
            ck = ShardedCheckpoint(tmp_path)
            for n in ck.names():
                ck.read(n)
            ck.close()
            outcomes.add("ok")
        except CheckpointError:
            outcomes.add("refused")
    assert outcomes <= {"ok", "refused"} and "refused" in outcomes
    path.write_bytes(struct.pack("<Q", 6) + b"[1, 2]")             # valid JSON, not an object
    with pytest.raises(CheckpointError):
        ShardedCheckpoint(tmp_path).read("a.weight")              # shards are opened when first read


def test_loaders_fail_closed_on_damaged_checkpoints(tmp_path):
    """A tensor missing from the index, or a config whose numbers do not fit the tensors: both loaders answer
    CheckpointError (the CLI prints the reason and exits 2), whatever the first symptom inside was."""
    import contextlib, io, os
    from ferrule_b200.cli.main import main as cli_main
    from ferrule_b200.io.checkpoint import load_deepseek_hf
    from ferrule_b200.io.safetensors import CheckpointError
    from ferrule_b200.io.v4_checkpoint import load_v4_hf
    with contextlib.redirect_stdout(io.StringIO()):
        cli_main(["make-fixture", "--out", str(tmp_path / "ds")])
        cli_main(["make-fixture", "--family", "v4", "--out", str(tmp_path / "v4"), "--plain", "--proposal-stages", "1"])
    cases = {"ds": (load_deepseek_hf, "model.layers.0.self_attn.o_proj.weight", {"kv_lora_rank": 0, "rope_scaling": "x",
                                                                                 "num_attention_heads": 10 ** 9}),
             "v4": (load_v4_hf, "layers.1.attn.wq_a.weight", {"o_groups": 0, "n_routed_experts": 0, "hidden_size": None,
                                                              "num_nextn_predict_layers": 10 ** 9})}
    for name, (loader, tensor, cfg_damage) in cases.items():
        d = tmp_path / name
        idx_path, cfg_path = d / "model.safetensors.index.json", d / "config.json"
        idx, cfg = json.loads(idx_path.read_text()), json.loads(cfg_path.read_text())
        bad = dict(idx, weight_map={k: v for k, v in idx["weight_map"].items() if k != tensor})
        idx_path.write_text(json.dumps(bad))
        with pytest.raises(CheckpointError):
            loader(d)
        err = io.StringIO()
        with contextlib.redirect_stderr(err), contextlib.redirect_stdout(io.StringIO()):
            rc = cli_main(["generate", str(d), "--device", "cpu", "--tokens", "1,2", "-n", "1", "--ctx-size", "64",
                           "--page-size", "16", "--max-seqs", "2"])
        assert rc == 2 and "error:" in err.getvalue()
        idx_path.write_text(json.dumps(idx))
        for key, val in cfg_damage.items():
            cfg_path.write_text(json.dumps(dict(cfg, **{key: val})))
            with pytest.raises(CheckpointError):
                loader(d)
        cfg_path.write_text(json.dumps(cfg))
        loader(d)
