"""Mirror of the reference's routed-expert backend boundary (backend/mod.rs) over the C ABI."""
import ctypes as C
import enum
import os

import numpy as np

from . import capi


class GpuExpertDispatchErrorKind(enum.IntEnum):
    """GpuExpertDispatchErrorKind (backend/mod.rs:349-361) plus the C-boundary extensions."""
    ResidencyMiss = 1
    PhysicalCapacity = 2
    Upload = 3
    ValidationDispatch = 4
    Submission = 5
    ReadbackChannel = 6
    ReadbackMap = 7
    DeviceLost = 8
    RuntimeInvariant = 9
    Ineligible = 10
    Timeout = 11
    InvalidArgument = 12
    Numerical = 13

    def __str__(self):
        return capi.load_library().mer_error_kind_name(int(self)).decode()


class GpuExpertDispatchError(Exception):
    """GpuExpertDispatchError{layer, expert_id, kind, detail} (backend/mod.rs:423-447)."""

    def __init__(self, layer, expert_id, kind, detail, device_status=0):
        self.layer, self.expert_id, self.kind, self.detail = layer, expert_id, GpuExpertDispatchErrorKind(kind), detail
        self.device_status = device_status
        super().__init__(f"GPU routed expert {expert_id} (layer {layer}) failed at {self.kind}: {detail}")


class GpuExpertBatchDispatchOutcome(enum.Enum):
    """GpuExpertBatchDispatchOutcome (backend/mod.rs:454-458); Failed carries the error."""
    Ineligible = 0
    Completed = 1
    Failed = 2


def expert_bytes(dtype, d_model, d_ff):
    return int(capi.load_library().mer_expert_bytes(dtype, d_model, d_ff))


def routed_expert_gpu_compatibility(dtype, d_model, d_ff):
    """routed_expert_gpu_compatibility (backend/mod.rs:4691-4720): True when the shape can run on the GPU."""
    return capi.load_library().mer_routed_expert_compatibility(dtype, d_model, d_ff) == 0


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Backend:
    """One CUDA routed-expert backend: HBM slot arena + router table + dispatch."""

    def __init__(self, dtype, d_model, d_ff, vram_capacity_bytes, max_experts, max_tokens=64, max_top_k=8, device=0,
                 swiglu_limit=0.0):
        self.lib = capi.load_library()
        self.dtype, self.d_model, self.d_ff = dtype, d_model, d_ff
        self.max_tokens, self.max_top_k = max_tokens, max_top_k
        cfg = capi.MerBackendCfg(device, dtype, d_model, d_ff, vram_capacity_bytes, max_experts, max_tokens, max_top_k,
                                 swiglu_limit, 0, 0)
        handle = C.c_void_p()
        rc = self.lib.mer_backend_create(C.byref(cfg), C.byref(handle))
        if rc != 0:
            raise GpuExpertDispatchError(0, capi.EXPERT_NONE, rc, "mer_backend_create failed "
                                         "(no CUDA device, bad shape or not enough HBM); there is no CPU fallback")
        self.h = handle
        self._routers = {}

    def close(self):
        if getattr(self, "h", None):
            self.lib.mer_backend_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- errors ---------------------------------------------------------------------------
    def last_error(self):
        info = capi.MerErrorInfo()
        self.lib.mer_last_error(self.h, C.byref(info))
        return info

    def _check(self, rc):
        if rc != 0:
            e = self.last_error()
            raise GpuExpertDispatchError(e.layer, e.expert_id, rc, e.detail.decode(errors="replace"), e.device_status)

    def snapshot(self):
        c = capi.MerCounters()
        self.lib.mer_snapshot(self.h, C.byref(c))
        return c.as_dict()

    def synchronize(self):
        self._check(self.lib.mer_backend_synchronize(self.h))

    def stage_timing_enable(self, on=True):
        self._check(self.lib.mer_stage_timing_enable(self.h, int(on)))

    def stage_timings(self):
        """Accumulated per-stage device times (ms) since stage_timing_enable(True): stage_timing.rs names."""
        t = capi.MerStageTimings()
        self._check(self.lib.mer_stage_timings_read(self.h, C.byref(t)))
        return t.as_dict()

    def set_kernel_path(self, path):
        self._check(self.lib.mer_set_kernel_path(self.h, path))

    # -- residency (VRAM tier) ------------------------------------------------------------
    def admit(self, expert_id, generation, blob, anchor=False, wait=True):
        blob = np.ascontiguousarray(blob, dtype=np.uint8)
        flags = (capi.ADMIT_ANCHOR if anchor else 0) | (0 if wait else capi.ADMIT_ASYNC)
        self._check(self.lib.mer_expert_admit(self.h, expert_id, generation, _ptr(blob), blob.size, flags))

    def admit_device(self, expert_id, generation, device_ptr, nbytes, anchor=False, wait=True):
        flags = (capi.ADMIT_ANCHOR if anchor else 0) | (0 if wait else capi.ADMIT_ASYNC)
        self._check(self.lib.mer_expert_admit_device(self.h, expert_id, generation, C.c_void_p(device_ptr), nbytes, flags))

    def admit_file(self, expert_id, generation, path, block_align=4096, anchor=False, wait=True):
        """expert_<id>.bin -> HBM slot: strips a UTH1 / UTH2 header, checks dtype and shape, streams the payload through
        the pinned staging buffers."""
        flags = (capi.ADMIT_ANCHOR if anchor else 0) | (0 if wait else capi.ADMIT_ASYNC)
        self._check(self.lib.mer_expert_admit_file(self.h, expert_id, generation, os.fsencode(path), block_align, flags))

    def retire(self, expert_id, generation):
        self._check(self.lib.mer_expert_retire(self.h, expert_id, generation))

    def contains_generation(self, expert_id, generation):
        return bool(self.lib.mer_expert_contains_generation(self.h, expert_id, generation))

    def demand_admit(self, cache, expert_id, blob, wait=True, reader_wait=True):
        """Foreground demand (engine.rs:2382-2429): logical admission into the LRU Edge of `cache`, victims retired,
        payload uploaded under the new generation.  Returns the expert's current generation."""
        blob = None if blob is None else np.ascontiguousarray(blob, dtype=np.uint8)
        gen = C.c_uint64(0)
        flags = (0 if wait else capi.ADMIT_ASYNC) | (0 if reader_wait else capi.ADMIT_NO_READER_WAIT)
        self._check(self.lib.mer_expert_demand_admit(self.h, cache.h, expert_id, _ptr(blob), 0 if blob is None else blob.size, flags,
                                                     C.byref(gen)))
        return gen.value

    def hot_promote(self, cache, expert_id, blob=None, wait=True, reader_wait=True):
        """Threshold-driven promotion into the Anchor Core; returns the GpuHotPromotionOutcome."""
        from .expert_cache import GpuHotPromotionOutcome
        blob = None if blob is None else np.ascontiguousarray(blob, dtype=np.uint8)
        out = C.c_int(0)
        flags = (0 if wait else capi.ADMIT_ASYNC) | (0 if reader_wait else capi.ADMIT_NO_READER_WAIT)
        self._check(self.lib.mer_expert_hot_promote(self.h, cache.h, expert_id, _ptr(blob), 0 if blob is None else blob.size, flags,
                                                    C.byref(out)))
        return GpuHotPromotionOutcome(out.value)

    def touch(self, cache, expert_ids):
        """Routing feedback: one cache.get per id (hits / misses / recency) and physical slot recency."""
        ids = np.ascontiguousarray(expert_ids, dtype=np.uint32).reshape(-1)
        self._check(self.lib.mer_expert_touch(self.h, cache.h if cache is not None else None, _ptr(ids), ids.size))

    # -- router -----------------------------------------------------------------------------
    def install_router(self, layer, gate, shared_expert_id=capi.EXPERT_NONE):
        """Installs a LinearGate (gating.py) as the router of `layer`."""
        w = np.ascontiguousarray(gate.weights, dtype=np.float32)
        cb = None if gate.correction_bias is None else np.ascontiguousarray(gate.correction_bias, dtype=np.float32)
        lb = None if gate.logit_bias is None else np.ascontiguousarray(gate.logit_bias, dtype=np.float32)
        cfg = capi.MerRouterCfg(gate.num_experts, gate.top_k, int(gate.scoring_func), int(gate.normalise_topk),
                                gate.n_group, gate.topk_group, gate.routed_scaling_factor, shared_expert_id,
                                cb.ctypes.data if cb is not None else None, lb.ctypes.data if lb is not None else None)
        self._check(self.lib.mer_router_install(self.h, layer, _ptr(w), C.byref(cfg)))
        self._routers[layer] = gate

    def install_layer(self, layer, rms_weight=None, rms_eps=1e-6, shared_gate=None, residual=False):
        """The steps either side of the MoE block of `layer` (after install_router): pre-MoE RMSNorm
        (transformer.rs:52-95), the shared expert's sigmoid gate vector (transformer.rs:2224-2237), residual add."""
        rw = None if rms_weight is None else np.ascontiguousarray(rms_weight, dtype=np.float32)
        sg = None if shared_gate is None else np.ascontiguousarray(shared_gate, dtype=np.float32)
        assert rw is None or rw.size == self.d_model
        assert sg is None or sg.size == self.d_model
        cfg = capi.MerLayerCfg(rw.ctypes.data if rw is not None else None, sg.ctypes.data if sg is not None else None,
                               float(rms_eps), capi.LAYER_RESIDUAL if residual else 0)
        self._check(self.lib.mer_layer_install(self.h, layer, C.byref(cfg)))

    def route(self, layer, x):
        gate = self._routers[layer]
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.d_model)
        ids = np.empty((x.shape[0], gate.top_k), np.uint32)
        w = np.empty((x.shape[0], gate.top_k), np.float32)
        self._check(self.lib.mer_router_route(self.h, layer, _ptr(x), x.shape[0], _ptr(ids), _ptr(w)))
        return ids, w

    # -- compute ----------------------------------------------------------------------------
    def routed_expert_matmul(self, layer, expert_id, x_f16, d_model, d_ff):
        """BackendBox::routed_expert_matmul (backend/mod.rs:4421-4441): f16 in, f16 out."""
        x = np.ascontiguousarray(x_f16, dtype=np.float16)
        out = np.empty(d_model, np.float16)
        self._check(self.lib.mer_routed_expert_matmul(self.h, layer, expert_id, _ptr(x), d_model, d_ff, _ptr(out)))
        return out

    def routed_expert_matmul_batch_q4(self, layer, expert_ids, x_f16, d_model, d_ff):
        """BackendBox::routed_expert_matmul_batch_q4 (backend/mod.rs:4401-4418).

        Returns (outcome, out[n, d_model] f16 or None, error or None)."""
        ids = np.ascontiguousarray(expert_ids, dtype=np.uint32)
        x = np.ascontiguousarray(x_f16, dtype=np.float16)
        out = np.empty((ids.size, d_model), np.float16)
        rc = self.lib.mer_routed_expert_matmul_batch(self.h, layer, _ptr(ids), ids.size, _ptr(x), d_model, d_ff, _ptr(out))
        if rc == 0:
            return GpuExpertBatchDispatchOutcome.Completed, out, None
        e = self.last_error()
        err = GpuExpertDispatchError(e.layer, e.expert_id, rc, e.detail.decode(errors="replace"), e.device_status)
        if rc == int(GpuExpertDispatchErrorKind.Ineligible):
            return GpuExpertBatchDispatchOutcome.Ineligible, None, err
        return GpuExpertBatchDispatchOutcome.Failed, None, err

    def expert_forward_f32(self, layer, expert_id, x):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.d_model)
        out = np.empty_like(x)
        self._check(self.lib.mer_routed_expert_forward_f32(self.h, layer, expert_id, _ptr(x), x.shape[0], _ptr(out)))
        return out

    def moe_step_weighted_into(self, layer, x, expert_ids, weights):
        """Engine::moe_step_weighted_into (engine.rs:5174): routing given, one token."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        ids = np.ascontiguousarray(expert_ids, dtype=np.uint32)
        w = np.ascontiguousarray(weights, dtype=np.float32)
        assert ids.size == w.size and x.size == self.d_model
        out = np.empty(self.d_model, np.float32)
        self._check(self.lib.mer_moe_step_weighted_into(self.h, layer, _ptr(x), _ptr(ids), _ptr(w), ids.size, _ptr(out)))
        return out

    def moe_layer_forward(self, layer, x, return_routing=True, out=None):
        """The whole path for a batch of host rows; `out` may be a caller-owned (e.g. pinned) array."""
        gate = self._routers[layer]
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.d_model)
        if out is None:
            out = np.empty_like(x)
        assert out.dtype == np.float32 and out.size == x.size and out.flags.c_contiguous
        ids = np.empty((x.shape[0], gate.top_k), np.uint32) if return_routing else None
        w = np.empty((x.shape[0], gate.top_k), np.float32) if return_routing else None
        self._check(self.lib.mer_moe_layer_forward(self.h, layer, _ptr(x), x.shape[0], _ptr(out), _ptr(ids), _ptr(w)))
        return (out, ids, w) if return_routing else out

    def moe_layer_forward_submit(self, layer, x_pinned, out_pinned, slot):
        """Pipelined host entry: enqueue upload, layer and read-back for pinned numpy views; returns at once."""
        assert x_pinned.dtype == np.float32 and out_pinned.dtype == np.float32 and x_pinned.flags.c_contiguous
        n = x_pinned.size // self.d_model
        self._check(self.lib.mer_moe_layer_forward_submit(self.h, layer, _ptr(x_pinned), n, _ptr(out_pinned), slot))

    def moe_layer_forward_wait(self, slot):
        self._check(self.lib.mer_moe_layer_forward_wait(self.h, slot))

    def moe_layer_forward_device(self, layer, d_x, n_tokens, d_out, stream=0, d_ids=0, d_weights=0):
        """Device pointers (ints) in, asynchronous on `stream` (a cudaStream_t as int)."""
        self._check(self.lib.mer_moe_layer_forward_device(self.h, layer, C.c_void_p(d_x), n_tokens, C.c_void_p(d_out),
                                                          C.c_void_p(d_ids), C.c_void_p(d_weights), C.c_void_p(stream)))

    def stream_check(self, layer, stream=0):
        """Synchronises `stream` and raises the typed error the device status word holds, if any (for _device calls)."""
        self._check(self.lib.mer_stream_check(self.h, layer, C.c_void_p(stream)))

    def qualification_matvec(self, weights, x, rows, columns, w_block_off=0, dtype=None):
        """GpuBackend::qualification_q4_0_matvec (backend/mod.rs:3532): raw block-stream matvec."""
        w = np.ascontiguousarray(weights, dtype=np.uint8)
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(rows, np.float32)
        self._check(self.lib.mer_qualification_matvec(self.h, self.dtype if dtype is None else dtype, _ptr(w), w.size,
                                                      _ptr(x), rows, columns, w_block_off, _ptr(out)))
        return out

    def dequant_projection(self, expert_id, projection):
        out = np.empty(self.d_model * self.d_ff, np.float32)
        self._check(self.lib.mer_dequant_projection_f32(self.h, expert_id, projection, _ptr(out)))
        return out


NOALLOC_MAX_TOKENS, NOALLOC_MAX_DIM = 8, 16384


def expert_forward_noalloc(dtype, d_model, d_ff, d_expert_blob, d_x, n_tokens, d_out, swiglu_limit=0.0, stream=0):
    """mer_expert_forward_noalloc: device pointers (ints) in and out, nothing allocated, asynchronous on
    `stream` of the current device.  All calls on a GPU share one fixed scratch array inside the library,
    so the caller must not let two of them overlap."""
    msg = C.create_string_buffer(256)
    rc = capi.load_library().mer_expert_forward_noalloc(dtype, d_model, d_ff, C.c_void_p(d_expert_blob), C.c_void_p(d_x),
                                                        n_tokens, C.c_void_p(d_out), swiglu_limit, C.c_void_p(stream), msg, 256)
    if rc != 0:
        raise GpuExpertDispatchError(0, capi.EXPERT_NONE, rc, msg.value.decode(errors="replace"))
