"""GGUF inspection reader, Q4_K decode, sparse-attention address resolvers, ring helpers, expert telemetry."""
import struct

import numpy as np
import pytest

from ferrule_b200.io import gguf
from ferrule_b200.models import sparse_layout as SL
from ferrule_b200.utils.telemetry import ExpertTelemetry


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def test_gguf_header_metadata_and_tensor_directory(tmp_path):
    kv = _s("general.architecture") + struct.pack("<I", 8) + _s("llama")
    kv += _s("llama.block_count") + struct.pack("<I", 4) + struct.pack("<I", 2)
    kv += _s("tokenizer.ggml.tokens") + struct.pack("<I", 9) + struct.pack("<I", 8) + struct.pack("<Q", 2) + _s("a") + _s("b")
    ti = _s("blk.0.attn_q.weight") + struct.pack("<I", 2) + struct.pack("<QQ", 256, 4) + struct.pack("<I", 12) + struct.pack("<Q", 0)
    ti += _s("output_norm.weight") + struct.pack("<I", 1) + struct.pack("<Q", 256) + struct.pack("<I", 0) + struct.pack("<Q", 576)
    body = b"GGUF" + struct.pack("<I", 3) + struct.pack("<QQ", 2, 3) + kv + ti
    p = tmp_path / "m.gguf"
    p.write_bytes(body + b"\0" * 64)
    g = gguf.read_gguf(str(p))
    assert g.version == 3 and g.metadata["general.architecture"] == "llama" and g.metadata["llama.block_count"] == 2
    assert g.metadata["tokenizer.ggml.tokens"] == ["a", "b"]
    assert [t.name for t in g.tensors] == ["blk.0.attn_q.weight", "output_norm.weight"]
    assert g.tensors[0].shape == (256, 4) and g.tensors[0].type_name == "Q4_K" and g.tensors[1].type_name == "F32"
    assert g.data_offset % 32 == 0 and g.data_offset >= len(body)
    assert g.summary()["tensor_types"] == {"Q4_K": 1, "F32": 1}
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + body[4:])
    with pytest.raises(gguf.GgufError):
        gguf.read_gguf(str(bad))


def test_q4_k_decode_matches_hand_computation():
    d, dmin = np.float16(0.5), np.float16(0.25)
    sc = np.zeros(12, dtype=np.uint8)
    sc[0], sc[4] = 3, 2              # sub-block 0: scale 3, min 2
    sc[1], sc[5] = 1, 0              # sub-block 1: scale 1, min 0
    qs = np.zeros(128, dtype=np.uint8)
    qs[0] = 0x21                     # element 0 -> code 1, element 32 -> code 2
    blk = d.tobytes() + dmin.tobytes() + sc.tobytes() + qs.tobytes()
    out = gguf.decode_q4_k(blk, 256)
    assert out[0] == pytest.approx(0.5 * 3 * 1 - 0.25 * 2) and out[1] == pytest.approx(-0.5)
    assert out[32] == pytest.approx(0.5 * 1 * 2) and out[64] == 0.0
    with pytest.raises(gguf.GgufError):
        gguf.decode_q4_k(blk, 100)


def test_layout_resolvers_and_ring():
    assert SL.ContiguousLayout(64).resolve(2, 5) == 133
    bt = [7, 3, -1]
    paged = SL.PagedLayout(16)
    assert paged.resolve(bt, 0) == 112 and paged.resolve(bt, 17) == 49
    with pytest.raises(SL.LayoutError):
        paged.resolve(bt, 40)
    dual = SL.DualPlanePagedLayout(page_tokens=16, ratio=4)
    assert dual.resolve_raw(bt, 17) == (0, 49) and dual.resolve_compressed(bt, 5) == (1, 3 * 4 + 1)
    ring = SL.CombinedRing(8)
    assert ring.ring_slot(19) == 3 and ring.logical_of_slot(3, 19) == 19 and ring.logical_of_slot(4, 19) == 12
    assert ring.logical_of_slot(5, 2) is None
    assert ring.selection(9, [0, 2]) == [2, 3, 4, 5, 6, 7, 0, 1, 8, 10]
    st = SL.CompressorStateShape(ratio=4, head_dim=64, overlap=True)
    assert (st.out_dim, st.rows, st.state_elems) == (128, 8, 1024) and st.row_of(6) == 6 and st.is_boundary(7)
    assert SL.CompressorStateShape(128, 512, False).row_of(130) == 2


def test_expert_telemetry_counts_and_coverage():
    t = ExpertTelemetry(2, 8)
    t.record(0, [1, 1, 5])
    t.record_counts(0, [0, 3, 0, 0, 0, 1, 0, 0], tokens=2)
    assert t.hottest(0, 2) == [1, 5] and t.tokens == [3, 0]
    assert t.coverage(0, [1]) == pytest.approx(5 / 7) and t.coverage(1, []) == 1.0
    assert t.snapshot()["top"][0][0] == 1


@pytest.mark.parametrize("value", [struct.pack("<I", 4) + struct.pack("<I", 0),            # u32 0
                                   struct.pack("<I", 4) + struct.pack("<I", 48),           # not a power of two
                                   struct.pack("<I", 8) + _s("32"),                        # a string
                                   struct.pack("<I", 6) + struct.pack("<f", 32.0)])        # a float
def test_gguf_refuses_an_alignment_that_is_not_a_power_of_two(tmp_path, value):
    body = b"GGUF" + struct.pack("<I", 3) + struct.pack("<QQ", 0, 1) + _s("general.alignment") + value
    p = tmp_path / "a.gguf"
    p.write_bytes(body)
    with pytest.raises(gguf.GgufError, match="alignment"):
        gguf.read_gguf(str(p))


def test_gguf_mutated_headers_fail_closed(tmp_path):
    """Random byte, length-field and truncation damage to a valid header only ever raises GgufError."""
    import random
    kv = _s("general.architecture") + struct.pack("<I", 8) + _s("llama")
    kv += _s("general.alignment") + struct.pack("<I", 4) + struct.pack("<I", 32)
    kv += _s("t") + struct.pack("<I", 9) + struct.pack("<I", 8) + struct.pack("<Q", 2) + _s("a") + _s("b")
    ti = _s("w") + struct.pack("<I", 2) + struct.pack("<QQ", 256, 4) + struct.pack("<I", 12) + struct.pack("<Q", 0)
    body = b"GGUF" + struct.pack("<I", 3) + struct.pack("<QQ", 1, 3) + kv + ti + b"\\0" * 32
    p = tmp_path / "f.gguf"
    for seed in range(400):
        r = random.Random(seed)
        b = bytearray(body)
        for _ in range(r.randint(1, 3)):
            k = r.random()
            if k < 0.5:
                b[r.randrange(len(b))] = r.randrange(256)
            elif k < 0.7 and len(b) > 24:
                del b[r.randrange(8, len(b)):]
            elif len(b) > 24:
                i = r.randrange(len(b) - 8)
                b[i:i + 8] = struct.pack("<Q", r.choice([0, 2 ** 63, 2 ** 64 - 1, 1 << 27, 2 ** 32]))
        p.write_bytes(bytes(b))
        try:
            gguf.read_gguf(str(p))
        except gguf.GgufError:
            pass
