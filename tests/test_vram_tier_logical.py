"""The logical VRAM tier (mer_gpu_cache_*) against the reference's own GpuExpertCache tests
(expert_cache.rs:1644-2208), case by case, through the C ABI.  Host-only: no GPU needed.

Payloads are identified by an integer tag here where the reference compares Arc pointers."""
import pytest

import mer_b200
from mer_b200 import GpuDemandAdmissionError as DemandError
from mer_b200 import GpuDemandAdmissionPreflight as Preflight
from mer_b200 import GpuExpertCache
from mer_b200 import GpuHotPromotionOutcome as Hot
from mer_b200 import GpuLookup

U64_MAX = 2 ** 64 - 1


def test_budget_split_follows_anchor_ratio():
    # GpuExpertCache::new (expert_cache.rs:798-828): ratio clamped to [0, 1], anchor share truncated, rest is LRU
    for cap, ratio, anchor in [(100, 0.5, 50), (100, 0.0, 0), (100, 1.0, 100), (100, 7.0, 100), (100, -1.0, 0), (101, 0.5, 50),
                               (20, 0.25, 5)]:
        s = GpuExpertCache(cap, ratio, 0).stats()
        assert (s["anchor_capacity_bytes"], s["lru_capacity_bytes"]) == (anchor, cap - anchor)
    assert GpuExpertCache(96, 0.0, 0).capacity_bytes() == 96
    assert GpuExpertCache(8, 0.5, 0).next_generation() == 1  # generations start at 1


def test_try_promote_lru_no_evict_skips_when_lru_full():
    cache = GpuExpertCache(100, 0.0, 0)
    assert cache.try_promote_lru_no_evict(1, 60)
    assert cache.try_promote_lru_no_evict(2, 40)
    assert cache.lru_len() == 2
    assert not cache.try_promote_lru_no_evict(3, 1)  # no room, and it must not evict
    assert cache.contains(1) and cache.contains(2) and not cache.contains(3)
    assert cache.promotions() == 2


def test_try_promote_lru_no_evict_never_uses_anchor_core():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.try_promote_lru_no_evict(7, 40)
    assert cache.anchor_len() == 0 and cache.lru_len() == 1


def test_try_promote_lru_no_evict_is_idempotent():
    cache = GpuExpertCache(100, 0.0, 0)
    assert cache.try_promote_lru_no_evict(9, 32)
    assert not cache.try_promote_lru_no_evict(9, 32)
    assert cache.promotions() == 1 and cache.used_bytes() == 32
    assert not cache.try_promote_lru_no_evict(10, 0)  # an empty payload is never admitted


def test_failed_no_evict_promotion_preserves_eviction_rearm():
    cache = GpuExpertCache(20, 0.0, 3)
    assert cache.promote_sync(1, 8)
    assert cache.promote_sync(2, 20)
    assert cache.last_evicted == [1]
    assert not cache.contains(1), "id 1 must be rearmed by logical eviction"
    assert not cache.try_promote_lru_no_evict(1, 8)
    assert cache.claim_promotion(1, 99), "failed opportunistic admission must leave one rearm claim"
    assert not cache.claim_promotion(1, 100), "rearm remains one-shot"


def test_failed_no_evict_promotion_preserves_pending_claim():
    cache = GpuExpertCache(20, 0.0, 3)
    assert cache.promote_sync(1, 8)
    assert cache.promote_sync(2, 20)
    assert not cache.contains(1)
    assert cache.claim_promotion(1, 3)
    assert not cache.try_promote_lru_no_evict(1, 8)
    assert not cache.claim_promotion(1, 3), "failed opportunistic admission must keep the existing claim pending"


@pytest.mark.parametrize("ratio,region", [(1.0, "anchor"), (0.0, "lru")])
def test_current_admission_does_not_change_counters(ratio, region):
    cache = GpuExpertCache(100, ratio, 0)
    assert cache.promote_sync(1, 32, tag=0xABC)
    assert (cache.anchor_len(), cache.lru_len()) == ((1, 0) if region == "anchor" else (0, 1))
    adm = cache.current_admission(1)
    assert adm.payload_tag == 0xABC
    assert adm.generation() == cache.current_generation(1)
    assert cache.hits() == 0 and cache.misses() == 0


def test_current_admission_lru_does_not_update_recency():
    cache = GpuExpertCache(20, 0.0, 0)
    assert cache.promote_sync(1, 10) and cache.promote_sync(2, 10)
    assert cache.current_admission(1) is not None
    assert cache.promote_sync(3, 10)
    assert not cache.contains(1), "non-mutating lookup must leave id 1 LRU"
    assert cache.contains(2) and cache.contains(3)


def test_current_admission_miss_does_not_increment_misses():
    cache = GpuExpertCache(20, 0.0, 0)
    assert cache.current_admission(99) is None
    assert cache.hits() == 0 and cache.misses() == 0


def test_demand_preflight_detects_anchor_without_state_changes():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.promote_sync(99, 40)
    generation = cache.current_generation(99)
    before = cache.stats()
    assert cache.demand_admission_preflight(99, 40) == Preflight.AlreadyAdmitted
    assert cache.contains_generation(99, generation)
    assert cache.stats() == before
    assert cache.anchor_len() == 1 and cache.lru_len() == 0


def test_demand_preflight_detects_lru_without_touching_recency():
    cache = GpuExpertCache(20, 0.0, 0)
    assert cache.demand_admit_lru(1, 10) is True
    assert cache.demand_admit_lru(2, 10) is True
    hits, misses = cache.hits(), cache.misses()
    assert cache.demand_admission_preflight(1, 10) == Preflight.AlreadyAdmitted
    assert (cache.hits(), cache.misses()) == (hits, misses)
    assert cache.demand_admit_lru(3, 10) is True
    assert not cache.contains(1), "preflight must leave id 1 as LRU"
    assert cache.contains(2) and cache.contains(3)


def test_demand_preflight_absent_fit_needs_payload_and_zero_is_typed():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.demand_admission_preflight(7, 50) == Preflight.NeedsPayload
    with pytest.raises(DemandError) as e:
        cache.demand_admission_preflight(7, 0)
    assert e.value.kind == "EmptyPayload"


def test_oversized_demand_preflight_preserves_all_logical_state():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.promote_sync(99, 40)
    assert cache.demand_admit_lru(1, 25) is True
    ag, lg = cache.current_generation(99), cache.current_generation(1)
    before = cache.stats()
    with pytest.raises(DemandError) as e:
        cache.demand_admission_preflight(2, 51)
    assert e.value == DemandError(-2, 51, 50)
    assert cache.contains_generation(99, ag) and cache.contains_generation(1, lg) and not cache.contains(2)
    assert cache.stats() == before


def test_demand_install_rechecks_existing_admission_after_preflight():
    cache = GpuExpertCache(100, 0.0, 0)
    assert cache.demand_admission_preflight(7, 32) == Preflight.NeedsPayload
    assert cache.demand_admit_lru(7, 32) is True
    generation = cache.current_generation(7)
    before = cache.stats()
    assert cache.demand_admit_lru(7, 64) is False
    assert cache.contains_generation(7, generation)
    assert cache.stats() == before
    assert cache.lru_len() == 1


def test_cold_demand_admits_to_lru_without_consuming_anchor():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.demand_admit_lru(1, 40) is True
    assert cache.current_admission(1) is not None
    assert (cache.anchor_len(), cache.lru_len(), cache.used_bytes(), cache.hits(), cache.misses()) == (0, 1, 40, 0, 0)


def test_demand_admission_evicts_lru_and_preserves_anchor():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.promote_sync(99, 40)
    ag = cache.current_generation(99)
    assert cache.demand_admit_lru(1, 25) is True
    assert cache.demand_admit_lru(2, 25) is True
    assert cache.demand_admit_lru(3, 25) is True
    assert cache.last_evicted == [1]
    assert not cache.contains(1), "oldest dynamic entry must be evicted"
    assert cache.contains(2) and cache.contains(3)
    assert cache.contains_generation(99, ag)
    assert (cache.anchor_len(), cache.lru_len()) == (1, 2)


def test_existing_demand_preserves_generation_bytes_and_counters():
    cache = GpuExpertCache(96, 0.0, 0)
    assert cache.demand_admit_lru(7, 32) is True
    assert cache.demand_admit_lru(8, 32) is True
    generation = cache.current_generation(7)
    before = cache.stats()
    assert cache.demand_admit_lru(7, 48) is False
    assert cache.contains_generation(7, generation)
    assert cache.stats() == before
    assert cache.demand_admit_lru(9, 40) is True
    assert not cache.contains(7), "existing demand lookup must not touch LRU"
    assert cache.contains(8) and cache.contains(9)


def test_demand_admitted_threshold_hot_lru_moves_to_anchor_with_exact_identity():
    cache = GpuExpertCache(100, 0.5, 3)
    assert cache.demand_admit_lru(7, 40, tag=0x77) is True
    before = cache.current_admission(7)
    used, next_gen = cache.used_bytes(), cache.next_generation()
    assert not cache.claim_promotion(7, 2)
    assert cache.claim_promotion(7, 3)
    assert not cache.claim_promotion(7, 3), "threshold-hot LRU admission must have one pending request"
    assert cache.promote_hot_existing(7) == Hot.MovedLruToAnchor
    after = cache.current_admission(7)
    assert after.generation() == before.generation() and after.payload_tag == 0x77
    assert after.region == 1
    s = cache.stats()
    assert (s["anchor_len"], s["lru_len"], s["used_bytes"]) == (1, 0, used)
    assert s["promotions"] == 2, "demand install + tier graduation"
    assert (s["anchor_used_bytes"], s["lru_used_bytes"], s["next_generation"]) == (40, 0, next_gen)
    assert cache.markers(7) == (False, False)


def test_hot_lru_move_preserves_unrelated_lru_recency():
    cache = GpuExpertCache(120, 0.5, 3)
    for i in (1, 2, 3):
        assert cache.demand_admit_lru(i, 20) is True
    assert cache.claim_promotion(2, 3)
    assert cache.promote_hot_existing(2) == Hot.MovedLruToAnchor
    assert cache.demand_admit_lru(4, 40) is True
    assert not cache.contains(1), "oldest unrelated LRU entry must remain victim"
    assert cache.contains(2) and cache.contains(3) and cache.contains(4)
    assert (cache.anchor_len(), cache.lru_len()) == (1, 2)


def test_anchor_full_hot_lru_is_unchanged_and_does_not_requeue():
    cache = GpuExpertCache(100, 0.5, 3)
    assert cache.promote_hot_sync(99, 50) == Hot.InstalledAnchor
    assert cache.demand_admit_lru(7, 25, tag=7) is True
    assert cache.demand_admit_lru(8, 25) is True
    generation = cache.current_generation(7)
    before = cache.stats()
    assert cache.claim_promotion(7, 3)
    assert cache.promote_hot_existing(7) == Hot.AlreadyLruAnchorFull
    assert cache.current_generation(7) == generation and cache.current_admission(7).payload_tag == 7
    after = cache.stats()
    for key in ("used_bytes", "promotions", "next_generation", "anchor_len", "lru_len"):
        assert after[key] == before[key]
    assert not cache.claim_promotion(7, 4)
    assert not cache.claim_promotion(7, 99)
    assert cache.demand_admit_lru(9, 25) is True
    assert not cache.contains(7), "Anchor-full attempt must not touch LRU recency"
    assert cache.contains(8) and cache.contains(9)


def test_already_anchor_hot_promotion_is_uncounted_noop():
    cache = GpuExpertCache(100, 0.5, 3)
    assert cache.promote_hot_sync(7, 40, tag=5) == Hot.InstalledAnchor
    generation, used, promotions = cache.current_generation(7), cache.used_bytes(), cache.promotions()
    assert not cache.claim_promotion(7, 3)
    assert cache.promote_hot_existing(7) == Hot.AlreadyAnchor
    assert cache.current_generation(7) == generation and cache.current_admission(7).payload_tag == 5
    assert (cache.used_bytes(), cache.promotions()) == (used, promotions)


def test_demand_wins_threshold_race_then_existing_admission_moves_intact():
    cache = GpuExpertCache(100, 0.5, 3)
    assert cache.claim_promotion(7, 3)
    assert cache.promote_hot_existing(7) == Hot.PayloadRequired
    assert cache.demand_admit_lru(7, 40, tag=111) is True
    generation = cache.current_generation(7)
    assert cache.promote_hot_sync(7, 40, tag=222) == Hot.MovedLruToAnchor
    cur = cache.current_admission(7)
    assert cur.generation() == generation and cur.payload_tag == 111  # the demand admission moved, the redundant payload was dropped
    assert (cache.anchor_len(), cache.lru_len(), cache.promotions()) == (1, 0, 2)


def test_background_wins_threshold_race_then_demand_recheck_is_noop():
    cache = GpuExpertCache(100, 0.5, 3)
    assert cache.demand_admission_preflight(7, 40) == Preflight.NeedsPayload
    assert cache.claim_promotion(7, 3)
    assert cache.promote_hot_existing(7) == Hot.PayloadRequired
    assert cache.promote_hot_sync(7, 40, tag=333) == Hot.InstalledAnchor
    generation, next_gen = cache.current_generation(7), cache.next_generation()
    assert cache.demand_admit_lru(7, 40, tag=444) is False
    cur = cache.current_admission(7)
    assert cur.generation() == generation and cur.payload_tag == 333
    assert cache.next_generation() == next_gen
    assert (cache.promotions(), cache.anchor_len(), cache.lru_len()) == (1, 1, 0)


def test_demand_readmission_allocates_a_newer_generation():
    cache = GpuExpertCache(20, 0.0, 0)
    assert cache.demand_admit_lru(7, 10) is True
    first = cache.current_generation(7)
    assert cache.demand_admit_lru(8, 20) is True
    assert not cache.contains(7)
    assert cache.demand_admit_lru(7, 10) is True
    assert cache.current_generation(7) > first


def test_oversized_demand_fails_without_mutating_existing_state():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.demand_admit_lru(1, 25) is True
    generation, used, promotions = cache.current_generation(1), cache.used_bytes(), cache.promotions()
    with pytest.raises(DemandError) as e:
        cache.demand_admit_lru(2, 51)
    assert e.value == DemandError(-2, 51, 50)
    assert cache.contains_generation(1, generation) and not cache.contains(2)
    assert (cache.used_bytes(), cache.promotions()) == (used, promotions)


def test_generation_exhaustion_does_not_evict_existing_demand():
    cache = GpuExpertCache(20, 0.0, 0)
    assert cache.demand_admit_lru(1, 10) is True
    generation = cache.current_generation(1)
    cache.set_next_generation(U64_MAX)
    with pytest.raises(DemandError) as e:
        cache.demand_admit_lru(2, 20)
    assert e.value.kind == "GenerationExhausted"
    assert cache.contains_generation(1, generation) and not cache.contains(2)
    assert cache.used_bytes() == 10
    assert cache.promote_hot_sync(3, 5) == Hot.GenerationExhausted
    assert not cache.promote_sync(3, 5) and not cache.try_promote_lru_no_evict(3, 5)


def test_get_retains_counter_and_lru_recency_behavior():
    cache = GpuExpertCache(20, 0.0, 0)
    assert cache.promote_sync(1, 10) and cache.promote_sync(2, 10)
    assert cache.get(1)[0] == GpuLookup.LruHit
    assert cache.get(99)[0] == GpuLookup.Miss
    assert (cache.hits(), cache.misses()) == (1, 1)
    assert cache.promote_sync(3, 10)
    assert cache.contains(1), "mutating get must make id 1 MRU"
    assert not cache.contains(2), "id 2 must remain the LRU victim"
    assert cache.contains(3)
    anchored = GpuExpertCache(20, 1.0, 0)
    assert anchored.promote_sync(5, 10)
    assert anchored.get(5)[0] == GpuLookup.AnchorHit and anchored.hits() == 1


def test_logical_admission_generation_changes_only_after_eviction_and_readmission():
    cache = GpuExpertCache(16, 0.0, 0)
    assert cache.promote_sync(7, 8)
    g1 = cache.current_generation(7)
    kind, adm = cache.get(7)
    assert kind == GpuLookup.LruHit and adm.generation() == g1, "ordinary hits preserve generation"
    assert cache.promote_sync(8, 16)
    assert not cache.contains(7), "larger admission evicts old generation"
    assert cache.promote_sync(7, 8)
    assert cache.current_generation(7) != g1, "readmission must never reuse physical identity"


def test_promotion_claim_rearms_after_logical_eviction_above_hit_threshold():
    cache = GpuExpertCache(16, 0.0, 3)
    assert cache.promote_sync(7, 8)
    assert not cache.claim_promotion(7, 99), "admitted id needs no request"
    assert cache.promote_sync(8, 16)
    assert not cache.contains(7)
    assert cache.claim_promotion(7, 99), "evicted id can claim again without a fresh RAM-hit edge"
    assert not cache.claim_promotion(7, 100), "only one request may be pending"
    assert cache.promote_sync(7, 8)
    assert cache.contains(7)


def test_cancelled_claim_can_be_claimed_once_more_and_threshold_zero_disables():
    # cancel_promotion (expert_cache.rs:947-952): the released claim re-arms exactly one new request
    cache = GpuExpertCache(100, 0.5, 3)
    assert cache.claim_promotion(4, 3)
    cache.cancel_promotion(4)
    assert cache.markers(4) == (False, True)
    assert cache.claim_promotion(4, 50) and not cache.claim_promotion(4, 51)
    off = GpuExpertCache(100, 0.5, 0)  # promote_after_hits = 0: promotion disabled (expert_cache.rs:918-920)
    assert not off.should_promote(10 ** 9) and not off.claim_promotion(1, 0)


def test_remove_releases_the_bytes_of_the_current_generation_only():
    cache = GpuExpertCache(100, 0.5, 0)
    assert cache.promote_sync(1, 40) and cache.demand_admit_lru(2, 30) is True
    g1, g2 = cache.current_generation(1), cache.current_generation(2)
    assert not cache.remove(2, g2 + 5)
    assert cache.remove(2, g2) and cache.remove(1, g1)
    s = cache.stats()
    assert (s["used_bytes"], s["anchor_len"], s["lru_len"]) == (0, 0, 0)
    assert cache.demand_admit_lru(2, 30) is True and cache.current_generation(2) > g2


def test_python_mirror_exports():
    assert mer_b200.GpuHotPromotionOutcome.InstalledLru.is_transition()
    assert not mer_b200.GpuHotPromotionOutcome.NoCapacity.is_transition()
