"""Mirror of the reference's logical GPU admission cache, GpuExpertCache (expert_cache.rs:734-1350), over the
C ABI (mer_gpu_cache_*).  Host-only bookkeeping: works without a CUDA device.  Names and return conventions
follow the reference so that its tests port line by line; payloads stay with the caller and are identified by
an opaque integer tag."""
import ctypes as C
import enum

import numpy as np

from . import capi


class GpuLookup(enum.IntEnum):
    """expert_cache.rs:629-637"""
    Miss = 0
    AnchorHit = 1
    LruHit = 2


class GpuHotPromotionOutcome(enum.IntEnum):
    """expert_cache.rs:667-692"""
    MovedLruToAnchor = 0
    InstalledAnchor = 1
    InstalledLru = 2
    AlreadyAnchor = 3
    AlreadyLruAnchorFull = 4
    PayloadRequired = 5
    NoCapacity = 6
    GenerationExhausted = 7

    def is_transition(self):
        return self in (self.MovedLruToAnchor, self.InstalledAnchor, self.InstalledLru)


class GpuDemandAdmissionPreflight(enum.IntEnum):
    AlreadyAdmitted = 0
    NeedsPayload = 1


class GpuDemandAdmissionError(Exception):
    """expert_cache.rs:649-661: EmptyPayload, PayloadExceedsLruCapacity{bytes, capacity}, GenerationExhausted."""
    KINDS = {-1: "EmptyPayload", -2: "PayloadExceedsLruCapacity", -3: "GenerationExhausted"}

    def __init__(self, code, bytes=None, capacity=None):
        self.kind, self.bytes, self.capacity = self.KINDS[code], bytes, capacity
        super().__init__(self.kind if bytes is None else f"{self.kind}: {bytes} bytes > {capacity}")

    def __eq__(self, other):
        return isinstance(other, GpuDemandAdmissionError) and (self.kind, self.bytes, self.capacity) == (
            other.kind, other.bytes, other.capacity)

    __hash__ = Exception.__hash__


class GpuAdmission:
    """expert_cache.rs:604-623: one installed logical admission."""

    def __init__(self, raw):
        self.expert_id, self.region = int(raw.expert_id), int(raw.region)
        self._generation, self._bytes, self.payload_tag = int(raw.generation), int(raw.bytes), int(raw.payload_tag)

    def generation(self):
        return self._generation

    def byte_len(self):
        return self._bytes


class GpuExpertCache:
    def __init__(self, capacity_bytes, anchor_ratio, promote_after_hits):
        self.lib = capi.load_library()
        h = C.c_void_p()
        rc = self.lib.mer_gpu_cache_create(int(capacity_bytes), float(anchor_ratio), int(promote_after_hits), C.byref(h))
        if rc != 0:
            raise MemoryError("mer_gpu_cache_create failed")
        self.h = h
        self.last_evicted = []

    def close(self):
        if getattr(self, "h", None):
            self.lib.mer_gpu_cache_destroy(self.h)
            self.h = None

    __del__ = close

    # -- statistics ---------------------------------------------------------------------------
    def stats(self):
        s = capi.MerGpuCacheStats()
        self.lib.mer_gpu_cache_stats_read(self.h, C.byref(s))
        return s.as_dict()

    def capacity_bytes(self):
        s = self.stats()
        return s["anchor_capacity_bytes"] + s["lru_capacity_bytes"]

    used_bytes = lambda self: self.stats()["used_bytes"]
    promotions = lambda self: self.stats()["promotions"]
    hits = lambda self: self.stats()["hits"]
    misses = lambda self: self.stats()["misses"]
    anchor_len = lambda self: self.stats()["anchor_len"]
    lru_len = lambda self: self.stats()["lru_len"]
    next_generation = lambda self: self.stats()["next_generation"]

    def set_next_generation(self, v):
        assert self.lib.mer_gpu_cache_set_next_generation(self.h, v) == 0

    def markers(self, expert_id):
        """(promotion pending, re-armed after eviction)"""
        m = self.lib.mer_gpu_cache_marker_state(self.h, expert_id)
        return bool(m & 1), bool(m & 2)

    # -- lookups --------------------------------------------------------------------------------
    def get(self, expert_id):
        a = capi.MerGpuAdmission()
        kind = GpuLookup(self.lib.mer_gpu_cache_get(self.h, expert_id, C.byref(a)))
        return kind, (GpuAdmission(a) if kind != GpuLookup.Miss else None)

    def current_admission(self, expert_id):
        a = capi.MerGpuAdmission()
        return GpuAdmission(a) if self.lib.mer_gpu_cache_current_admission(self.h, expert_id, C.byref(a)) else None

    def current_generation(self, expert_id):
        a = self.current_admission(expert_id)
        return a.generation() if a else None

    def contains(self, expert_id):
        return bool(self.lib.mer_gpu_cache_contains(self.h, expert_id))

    def contains_generation(self, expert_id, generation):
        return bool(self.lib.mer_gpu_cache_contains_generation(self.h, expert_id, generation))

    # -- promotion claims -------------------------------------------------------------------
    def should_promote(self, ram_hits):
        return bool(self.lib.mer_gpu_cache_should_promote(self.h, ram_hits))

    def claim_promotion(self, expert_id, ram_hits):
        return bool(self.lib.mer_gpu_cache_claim_promotion(self.h, expert_id, ram_hits))

    def cancel_promotion(self, expert_id):
        self.lib.mer_gpu_cache_cancel_promotion(self.h, expert_id)

    # -- admissions ---------------------------------------------------------------------------
    def _evicting(self, fn, expert_id, nbytes, tag):
        ev = np.zeros(64, np.uint32)
        n, gen = C.c_size_t(0), C.c_uint64(0)
        rc = fn(self.h, expert_id, nbytes, tag, ev.ctypes.data_as(C.c_void_p), 64, C.byref(n), C.byref(gen))
        self.last_evicted = ev[:min(n.value, 64)].tolist()
        return rc, gen.value

    def promote_hot_existing(self, expert_id):
        return GpuHotPromotionOutcome(self.lib.mer_gpu_cache_promote_hot_existing(self.h, expert_id))

    def promote_hot_sync(self, expert_id, nbytes, tag=0):
        rc, _ = self._evicting(self.lib.mer_gpu_cache_promote_hot_sync, expert_id, nbytes, tag)
        return GpuHotPromotionOutcome(rc)

    def promote_sync(self, expert_id, nbytes, tag=0):
        rc, _ = self._evicting(self.lib.mer_gpu_cache_promote_sync, expert_id, nbytes, tag)
        return bool(rc)

    def try_promote_lru_no_evict(self, expert_id, nbytes, tag=0):
        gen = C.c_uint64(0)
        return bool(self.lib.mer_gpu_cache_try_promote_lru_no_evict(self.h, expert_id, nbytes, tag, C.byref(gen)))

    def _demand_error(self, rc, nbytes):
        if rc == -2:
            return GpuDemandAdmissionError(rc, nbytes, self.stats()["lru_capacity_bytes"])
        return GpuDemandAdmissionError(rc)

    def demand_admission_preflight(self, expert_id, payload_bytes):
        rc = self.lib.mer_gpu_cache_demand_admission_preflight(self.h, expert_id, payload_bytes)
        if rc < 0:
            raise self._demand_error(rc, payload_bytes)
        return GpuDemandAdmissionPreflight(rc)

    def demand_admit_lru(self, expert_id, nbytes, tag=0):
        """True for a new admission, False when the id was admitted already (nothing changes)."""
        rc, _ = self._evicting(self.lib.mer_gpu_cache_demand_admit_lru, expert_id, nbytes, tag)
        if rc < 0:
            raise self._demand_error(rc, nbytes)
        return rc == 2

    def remove(self, expert_id, generation):
        return bool(self.lib.mer_gpu_cache_remove(self.h, expert_id, generation))
