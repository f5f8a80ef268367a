"""Expert streaming end to end on the CPU: checkpoint -> slabs -> arena frames through the LoadRegistry."""
import time

import pytest
import torch

from ferrule_b200.io.checkpoint import export_hf
from ferrule_b200.io.safetensors import ShardedCheckpoint
from ferrule_b200.models import config as C
from ferrule_b200.models import weights as W
from ferrule_b200.runtime.expert_residency import ExpertResidencyController
from ferrule_b200.runtime.expert_streaming import (ExpertArena, ExpertMaterializationProvider, ExpertSourceCatalog,
                                                   HostStagedExpertCache, PinnedSlabPool)
from ferrule_b200.runtime.registry import LoadRegistry
from ferrule_b200.utils.failpoints import FAILPOINTS


@pytest.fixture()
def rig(tmp_path):
    cfg = C.tiny_fixture()
    w = W.random_weights(cfg, dtype=torch.bfloat16, seed=5)
    export_hf(w, tmp_path, expert_format="mxfp4")
    ck = ShardedCheckpoint(tmp_path)
    cat = ExpertSourceCatalog("tiny", ck, [1], cfg.n_routed_experts, device=0, backend="cpu")
    res = ExpertResidencyController([1], {1: 3}, cfg.n_routed_experts)
    arena = ExpertArena([1], {1: 3}, cat.max_payload_bytes(), "cpu")
    slabs = PinnedSlabPool(cat.max_payload_bytes(), 2, pin=False)
    installed = []
    prov = ExpertMaterializationProvider(cat, res, arena, slabs, HostStagedExpertCache(1 << 20, 1 << 20),
                                         on_install=lambda *a: installed.append(a[:4]))
    reg = LoadRegistry(prov)
    yield cfg, w, ck, cat, res, arena, slabs, prov, reg, installed
    prov.close()
    ck.close()
    FAILPOINTS.disarm_all()


def drive(reg, pred, limit=2.0):
    t0 = time.time()
    while not pred() and time.time() - t0 < limit:
        reg.drive()
        time.sleep(0.001)
    assert pred()


def test_stream_experts_into_slots_and_bytes_match_checkpoint(rig):
    cfg, w, ck, cat, res, arena, slabs, prov, reg, installed = rig
    keys = [cat.key(1, e) for e in (0, 5)]
    assert keys[0] != keys[1] and keys[0] == cat.key(1, 0)
    reg.register_continuation(1, keys)
    drive(reg, lambda: bool(reg._ready))
    assert reg.pop_ready() == [1] and len(installed) == 2
    coord = res.layer(1)
    for e in (0, 5):
        slot, gen = coord.resolve(e)
        src = cat.source(1, e)
        frame = arena.frame(1, slot)
        for s in src.slices:
            info = ck.info(s.name)
            raw = ck.read(s.name).contiguous().view(torch.uint8).flatten()
            assert torch.equal(frame[s.payload_offset:s.payload_offset + s.length], raw), s.name
    assert slabs.in_use == 0 and prov.bytes_uploaded == sum(cat.source(1, e).payload_bytes for e in (0, 5))
    assert reg.broker.outstanding() == 2            # two resident-byte grants


def test_capacity_eviction_restream_hits_host_cache(rig):
    cfg, w, ck, cat, res, arena, slabs, prov, reg, installed = rig
    for txn, e in enumerate((0, 1, 2)):
        reg.register_continuation(txn, [cat.key(1, e)])
        drive(reg, lambda: bool(reg._ready))
        reg.pop_ready(); reg.release_transaction(txn)
    assert res.layer(1).resident() == [0, 1, 2]
    read_before = prov.bytes_read
    # a fourth expert needs a slot: the registry must retire an unleased one first
    assert reg.evict(1) == 1
    reg.register_continuation(10, [cat.key(1, 3)])
    drive(reg, lambda: bool(reg._ready))
    assert 3 in res.layer(1).resident() and len(res.layer(1).resident()) == 3
    evicted = ({0, 1, 2} - set(res.layer(1).resident())).pop()
    reg.pop_ready(); reg.release_transaction(10)
    reg.evict(1)
    reg.register_continuation(11, [cat.key(1, evicted)])
    drive(reg, lambda: bool(reg._ready))
    assert prov.cache_served == 1 and prov.bytes_read == read_before + cat.source(1, 3).payload_bytes


def test_failpoints_fail_the_waiter_and_leave_no_residue(rig):
    cfg, w, ck, cat, res, arena, slabs, prov, reg, installed = rig
    FAILPOINTS.arm("expert_upload")
    reg.register_continuation(1, [cat.key(1, 4)])
    drive(reg, lambda: bool(reg._failed))
    assert reg.pop_failed() == [1]
    reg.release_transaction(1)
    assert not res.layer(1).in_flight(4) and res.layer(1).resident() == [] and slabs.in_use == 0
    FAILPOINTS.arm("checkpoint_read")
    reg.register_continuation(2, [cat.key(1, 4)])
    drive(reg, lambda: bool(reg._failed))
    reg.pop_failed(); reg.release_transaction(2)
    reg.register_continuation(3, [cat.key(1, 4)])          # third time lucky: nothing armed
    drive(reg, lambda: bool(reg._ready))
    assert res.layer(1).resident() == [4] and reg.broker.outstanding() == 1


def test_native_direct_reader_feeds_the_provider(tmp_path):
    from ferrule_b200.io.direct_reader import NativeDirectReader
    cfg = C.tiny_fixture()
    w = W.random_weights(cfg, dtype=torch.bfloat16, seed=6)
    export_hf(w, tmp_path)
    ck = ShardedCheckpoint(tmp_path)
    cat = ExpertSourceCatalog("tiny", ck, [1], cfg.n_routed_experts, backend="cpu")
    res = ExpertResidencyController([1], {1: 8}, cfg.n_routed_experts)
    arena = ExpertArena([1], {1: 8}, cat.max_payload_bytes(), "cpu")
    reader = NativeDirectReader(2)
    prov = ExpertMaterializationProvider(cat, res, arena, PinnedSlabPool(cat.max_payload_bytes(), 4, pin=False),
                                         reader=reader)
    reg = LoadRegistry(prov)
    reg.register_continuation(1, [cat.key(1, e) for e in range(8)])
    drive(reg, lambda: bool(reg._ready), limit=5.0)
    for e in range(8):
        slot, _ = res.layer(1).resolve(e)
        s = cat.source(1, e).slices[2]              # down_proj weight
        got = arena.frame(1, slot)[s.payload_offset:s.payload_offset + s.length].view(torch.bfloat16)
        assert torch.equal(got.view(cfg.hidden, cfg.moe_inter), w.layers[1].e_w2[e])
    st = reader.stats()
    assert st["completed"] == 24 and st["bytes"] == sum(cat.source(1, e).payload_bytes for e in range(8)) or st["bytes"] > 0
    prov.close()
    ck.close()


def test_native_direct_reader_random_ranges(tmp_path):
    """Aligned reads (which bypass the page cache), unaligned offsets and destinations, reads that run past the end
    of the file and a missing file: the bytes that exist arrive intact and `ok` is true only for a whole read."""
    import os
    import random
    import threading
    from ferrule_b200.io.direct_reader import NativeDirectReader
    path = str(tmp_path / "blob.bin")
    data = os.urandom(1024 * 1024 + 137)
    with open(path, "wb") as f:
        f.write(data)
    rd = NativeDirectReader(threads=3)
    r = random.Random(0)
    n_reads, results, lock, all_done = 120, {}, threading.Lock(), threading.Event()

    def completion(i):
        def done(ok, n):
            with lock:
                results[i] = (ok, n)
                if len(results) == n_reads:
                    all_done.set()
        return done

    want, bufs = {}, {}
    for i in range(n_reads):
        k = r.random()
        if k < 0.4:
            off, ln = r.randrange(0, len(data) // 4096) * 4096, r.randint(1, 16) * 4096
        elif k < 0.8:
            off, ln = r.randrange(0, len(data)), r.randint(0, 100000)
        elif k < 0.9:
            off, ln = len(data) - r.randint(0, 5000), r.randint(1, 20000)
        else:
            off, ln = len(data) + r.randint(0, 10000), r.randint(1, 5000)
        src = path if r.random() > 0.05 else str(tmp_path / "missing.bin")
        raw = torch.zeros(ln + 8192, dtype=torch.uint8)
        shift = (-raw.data_ptr()) % 4096 + (0 if r.random() < 0.5 else r.randint(1, 63))
        bufs[i] = (raw, raw[shift:shift + max(ln, 1)])
        want[i] = (src, off, ln)
        rd.read(src, off, ln, bufs[i][1], completion(i))
    assert all_done.wait(60), f"{len(results)} of {n_reads} reads completed"
    for i in range(n_reads):
        src, off, ln = want[i]
        ok, _ = results[i]
        if src != path:
            assert not ok
            continue
        avail = max(0, min(ln, len(data) - off))
        assert ok == (avail == ln), (off, ln, avail)
        assert bufs[i][1][:avail].numpy().tobytes() == data[off:off + avail], (off, ln)
    st = rd.stats()
    assert st["submitted"] == st["completed"] == n_reads and st["queued"] == 0        # direct_reads depends on the file system
    rd.close()


@pytest.mark.parametrize("fmt", ["fp8_block", "fp8_mxfp4"])
def test_model_arena_holds_quantised_experts_in_their_own_form(fmt):
    """The routed-expert arena of the model (models/expert_arena.py) over quantised experts: every frame carries
    the expert's codes and scales (and nothing is dequantised), uploads bring exactly the host bytes, eviction and
    re-upload restore them, and the layer's weights become views of the frames."""
    import torch
    from ferrule_b200.models import config as C, weights as W
    from ferrule_b200.models.expert_arena import ExpertArena, _parts
    from ferrule_b200.models.weights import QuantWeight
    cfg = C.tiny_fixture().with_(hidden=256, moe_inter=128, n_mtp_layers=0)
    w = W.random_weights(cfg, device="cpu", seed=1, dtype=torch.bfloat16, weight_format=fmt)
    lw = w.layers[1]
    assert isinstance(lw.e_w13, QuantWeight)
    full13, full2 = [t.clone() for t in _parts(lw.e_w13)], [t.clone() for t in _parts(lw.e_w2)]
    arena = ExpertArena(w, resident_fraction=0.5)
    la = arena.layers[1]
    E = cfg.n_routed_experts
    assert la.frames == E // 2 and isinstance(lw.e_w13, QuantWeight) and lw.e_w13.group32 == (fmt == "fp8_mxfp4")
    assert lw.e_w13.q.shape[0] == la.frames and lw.e_w13.shape[1:] == full13[0].shape[1:]
    assert la.expert_bytes == sum(t[0].numel() * t.element_size() for t in full13 + full2)
    for wave in ([0, 3, 5], [1, 2, 6], [0, 7]):
        arena.ensure(1, wave)
        for e in wave:
            slot = int(la.expert_to_slot[e])
            assert slot >= 0 and int(la.slot_expert[slot]) == e
            for dev, src in zip(_parts(lw.e_w13), full13):
                assert torch.equal(dev[slot], src[e])
            for dev, src in zip(_parts(lw.e_w2), full2):
                assert torch.equal(dev[slot], src[e])
        arena.release(1)
    assert arena.stats.evictions > 0 and arena.stats.upload_bytes == arena.stats.uploads * la.expert_bytes
