"""The logical VRAM tier driving the physical HBM slots (mer_expert_demand_admit / _hot_promote / _touch), and
admission racing layers in flight.  Outputs are checked against the CPU oracle."""
import numpy as np
import pytest

import mer_b200
import oracle
from mer_b200 import GpuExpertDispatchErrorKind as Kind
from mer_b200 import GpuHotPromotionOutcome as Hot

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("mer_b200.synth")


def rel_rms_err(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


def make_backend(dtype, D, F, slots, **kw):
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    return mer_b200.Backend(dtype, D, F, stride * slots, kw.pop("max_experts", 64), **kw)


def test_demand_admission_evicts_through_to_the_slots_and_anchor_survives():
    dtype, D, F = oracle.Q8_0, 256, 256
    eb = mer_b200.expert_bytes(dtype, D, F)
    blobs = {e: synth.make_expert_blob(dtype, D, F, 61, 0, e) for e in range(6)}
    x = synth.make_activations(3, D, 61)
    cache = mer_b200.GpuExpertCache(4 * eb, 0.25, 2)  # one anchor slot's worth, three LRU
    with make_backend(dtype, D, F, slots=4, max_tokens=4) as b:
        gens = {}
        for e in (0, 1, 2):
            gens[e] = b.demand_admit(cache, e, blobs[e])
        assert gens[0] < gens[1] < gens[2] and cache.lru_len() == 3 and cache.anchor_len() == 0
        assert b.demand_admit(cache, 1, None) == gens[1]  # already admitted and uploaded: nothing to do, no payload needed
        # expert 1 becomes threshold-hot: the existing admission graduates intact and its slot is pinned
        assert cache.claim_promotion(1, 2)
        assert b.hot_promote(cache, 1) == Hot.MovedLruToAnchor
        assert cache.current_generation(1) == gens[1] and b.contains_generation(1, gens[1])
        # routing feedback: 0 is touched, so 2 is now the LRU victim
        b.touch(cache, [0, 0xFFFFFFFF])
        assert (cache.hits(), cache.misses()) == (1, 0)
        b.touch(cache, [5])
        assert cache.misses() == 1
        for e in (3, 4):  # LRU budget is three: admitting 3 fits, admitting 4 evicts 2
            gens[e] = b.demand_admit(cache, e, blobs[e])
        assert not cache.contains(2) and not b.contains_generation(2, gens[2])
        assert b.snapshot()["evictions"] == 1
        gens[5] = b.demand_admit(cache, 5, blobs[5])  # evicts 0 (touched before 3 and 4 came in)
        assert not cache.contains(0) and cache.contains(1) and b.contains_generation(1, gens[1])
        for e in (1, 3, 4, 5):
            got = b.expert_forward_f32(0, e, x)
            for t in range(3):
                assert rel_rms_err(got[t], oracle.expert_forward(dtype, blobs[e], x[t], D, F)) <= 1e-3
        with pytest.raises(mer_b200.GpuExpertDispatchError) as err:
            b.expert_forward_f32(0, 2, x)
        assert err.value.kind == Kind.ResidencyMiss
        # readmission gets a newer generation and the weights of the new payload
        g2 = b.demand_admit(cache, 2, blobs[0])
        assert g2 > gens[5] and b.contains_generation(2, g2)
        got = b.expert_forward_f32(0, 2, x)
        assert rel_rms_err(got[0], oracle.expert_forward(dtype, blobs[0], x[0], D, F)) <= 1e-3
        # a payload larger than the LRU budget is refused with the typed capacity error, nothing changes
        tiny = mer_b200.GpuExpertCache(eb - 1, 0.0, 0)
        with pytest.raises(mer_b200.GpuExpertDispatchError) as err:
            b.demand_admit(tiny, 9, blobs[0])
        assert err.value.kind == Kind.PhysicalCapacity and tiny.used_bytes() == 0


def test_hot_promotion_of_an_absent_expert_installs_anchor_and_is_never_evicted():
    dtype, D, F = oracle.Q4_0, 256, 256
    eb = mer_b200.expert_bytes(dtype, D, F)
    blobs = [synth.make_expert_blob(dtype, D, F, 62, 0, e) for e in range(5)]
    cache = mer_b200.GpuExpertCache(4 * eb, 0.3, 1)  # Anchor Core: one expert's worth; LRU Edge: two
    x = synth.make_activations(1, D, 62)
    with make_backend(dtype, D, F, slots=3, max_tokens=4) as b:
        assert cache.claim_promotion(0, 1)
        assert b.hot_promote(cache, 0) == Hot.PayloadRequired  # no payload passed: the claim stays pending
        assert b.hot_promote(cache, 0, blobs[0]) == Hot.InstalledAnchor
        g0 = cache.current_generation(0)
        for e in (1, 2, 3, 4):  # two LRU slots churn; the anchor stays
            b.demand_admit(cache, e, blobs[e])
        assert b.contains_generation(0, g0) and cache.anchor_len() == 1 and cache.lru_len() == 2
        got = b.expert_forward_f32(0, 0, x)
        assert rel_rms_err(got[0], oracle.expert_forward(dtype, blobs[0], x[0], D, F)) <= 1e-3


def test_async_admission_that_evicts_an_expert_of_a_layer_in_flight():
    # Full arena; layers in flight on the pipelined entry use every resident expert; asynchronous admissions evict
    # experts those layers read.  Every result must equal the oracle's: the eviction's table update and the slot
    # overwrite are ordered after the layers already enqueued.
    torch = pytest.importorskip("torch")
    dtype, E, D, F, k, B = oracle.Q8_0, 8, 512, 256, 4, 16
    blobs = [synth.make_expert_blob(dtype, D, F, 63, 0, e) for e in range(E)]
    spare = [synth.make_expert_blob(dtype, D, F, 63, 1, e) for e in range(4)]
    W = synth.make_router(E, D, 63)
    xs = [synth.make_activations(B, D, 63, i) for i in range(4)]
    gate = oracle.LinearGate(W, E, D, k)
    refs = [oracle.moe_layer_forward(dtype, gate, blobs, x, F, n_threads=8)[0] for x in xs]
    with make_backend(dtype, D, F, slots=E, max_experts=64, max_tokens=B, max_top_k=k) as b:
        for e in range(E):
            b.admit(e, 1, blobs[e])
        mer_b200.LinearGate(W, E, D, k).bind(b, 0)
        pin_x = [torch.from_numpy(x.copy()).pin_memory() for x in xs]
        pin_o = [torch.zeros(B, D).pin_memory() for _ in xs]
        for rep in range(3):
            for i in range(4):
                b.moe_layer_forward_submit(0, pin_x[i].numpy(), pin_o[i].numpy(), i)
            for j in range(4):  # ids 32.. are not routed to: each admission evicts a resident expert of layer 0
                b.admit(32 + j, rep + 1, spare[j], wait=False)
            for i in range(4):
                b.moe_layer_forward_wait(i)
                assert rel_rms_err(pin_o[i].numpy(), refs[i]) <= 1e-3, (rep, i)
            b.synchronize()
            for e in range(E):  # restore the layer's experts for the next round (evicting the spares again)
                if not b.contains_generation(e, 1):
                    b.admit(e, 1, blobs[e])


def test_admission_waits_for_a_layer_on_a_caller_stream():
    # device entry on a caller-owned stream, then an admission that replaces a slot the layer reads
    torch = pytest.importorskip("torch")
    dtype, E, D, F, k, B = oracle.Q8_0, 4, 512, 512, 2, 8
    blobs = [synth.make_expert_blob(dtype, D, F, 64, 0, e) for e in range(E)]
    other = synth.make_expert_blob(dtype, D, F, 64, 1, 0)
    W = synth.make_router(E, D, 64)
    x = synth.make_activations(B, D, 64)
    ref = oracle.moe_layer_forward(dtype, oracle.LinearGate(W, E, D, k), blobs, x, F)[0]
    with make_backend(dtype, D, F, slots=E, max_tokens=B, max_top_k=k) as b:
        for e in range(E):
            b.admit(e, 1, blobs[e])
        mer_b200.LinearGate(W, E, D, k).bind(b, 0)
        dev = torch.device("cuda", 0)
        xd = torch.from_numpy(x).to(dev)
        outs = [torch.empty(B, D, device=dev) for _ in range(6)]
        side = torch.cuda.Stream()
        torch.cuda.synchronize()
        for o in outs:
            b.moe_layer_forward_device(0, xd.data_ptr(), B, o.data_ptr(), side.cuda_stream)
        for e in range(E):  # newer generations replace every slot in place while the layers are queued
            b.admit(e, 2, other, wait=False)
        side.synchronize()
        b.synchronize()
        for o in outs:
            assert rel_rms_err(o.cpu().numpy(), ref) <= 1e-3
