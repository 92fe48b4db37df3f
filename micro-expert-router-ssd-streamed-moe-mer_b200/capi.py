"""ctypes declarations for every symbol of include/mer_b200.h."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MER_B200_LIB") or os.path.join(HERE, "libmer_b200.so")  # MER_B200_LIB: another build of the library

DTYPE_Q4_0, DTYPE_Q8_0 = 0, 1
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
EXPERT_NONE = 0xFFFFFFFF
ADMIT_ANCHOR, ADMIT_ASYNC, ADMIT_NO_READER_WAIT = 1, 2, 4
LAYER_RESIDUAL = 1


class MerBackendCfg(C.Structure):
    _fields_ = [("device", C.c_int32), ("dtype", C.c_int32), ("d_model", C.c_uint64), ("d_ff", C.c_uint64),
                ("vram_capacity_bytes", C.c_uint64), ("max_experts", C.c_uint32), ("max_tokens", C.c_uint32),
                ("max_top_k", C.c_uint32), ("swiglu_limit", C.c_float), ("flags", C.c_uint32), ("reserved", C.c_uint32)]


class MerRouterCfg(C.Structure):
    _fields_ = [("num_experts", C.c_uint32), ("top_k", C.c_uint32), ("scoring_func", C.c_int32),
                ("normalise_topk", C.c_int32), ("n_group", C.c_uint32), ("topk_group", C.c_uint32),
                ("routed_scaling_factor", C.c_float), ("shared_expert_id", C.c_uint32),
                ("correction_bias", C.c_void_p), ("logit_bias", C.c_void_p)]


class MerLayerCfg(C.Structure):
    _fields_ = [("rms_weight", C.c_void_p), ("shared_gate", C.c_void_p), ("rms_eps", C.c_float), ("flags", C.c_uint32)]


class MerUthProjection(C.Structure):
    _fields_ = [("uth_dtype_id", C.c_uint32), ("weights", C.c_uint32), ("offset", C.c_uint64), ("len", C.c_uint64)]


class MerUthInfo(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("version", C.c_uint32), ("uth_dtype_id", C.c_uint32), ("dtype", C.c_int32),
                ("shape_rank", C.c_uint32), ("flags", C.c_uint32), ("shape", C.c_uint32 * 4), ("d_model", C.c_uint64),
                ("d_ff", C.c_uint64), ("payload_offset", C.c_uint64), ("payload_bytes", C.c_uint64), ("proj", MerUthProjection * 3)]


class MerDatasetInfo(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("format_version", "num_experts", "d_model", "d_ff", "expert_size", "maximum_payload_bytes",
                                          "block_align", "experts_written", "num_layers", "experts_per_layer", "top_k")] + [
        ("dtype", C.c_int32), ("dtype_name", C.c_char * 16), ("q4_0_layout", C.c_char * 32), ("conversion_mode", C.c_char * 32)]


class MerErrorInfo(C.Structure):
    _fields_ = [("layer", C.c_uint32), ("expert_id", C.c_uint32), ("kind", C.c_int32), ("device_status", C.c_uint32),
                ("detail", C.c_char * 256)]


class MerCounters(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "selected_routed_experts", "gpu_dispatch_attempts", "gpu_dispatch_successes", "gpu_dispatch_failures",
        "batch_calls", "kernel_launches", "expert_uploads", "expert_upload_bytes", "hidden_upload_bytes",
        "readback_bytes", "evictions", "resident_experts", "resident_bytes", "arena_bytes", "slot_stride_bytes",
        "slot_count")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class MerGpuAdmission(C.Structure):
    _fields_ = [("expert_id", C.c_uint32), ("region", C.c_uint32), ("generation", C.c_uint64), ("bytes", C.c_uint64),
                ("payload_tag", C.c_uint64)]


class MerGpuCacheStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "anchor_capacity_bytes", "lru_capacity_bytes", "anchor_used_bytes", "lru_used_bytes", "used_bytes", "anchor_len",
        "lru_len", "promotions", "hits", "misses", "next_generation", "promote_after_hits", "pending_promotions",
        "rearmed_promotions")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class MerEpCfg(C.Structure):
    _fields_ = [("rank", C.c_uint32), ("world", C.c_uint32), ("experts_per_layer", C.c_uint32),
                ("max_tokens_per_rank", C.c_uint32), ("wait_ms", C.c_uint32), ("reserved", C.c_uint32)]


class MerStageTimings(C.Structure):
    _fields_ = [("samples", C.c_uint64), ("router_gate_ms", C.c_double), ("expert_gate_up_kernel_ms", C.c_double),
                ("expert_down_kernel_ms", C.c_double), ("moe_weighted_combination_ms", C.c_double),
                ("expert_compute_ms", C.c_double)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


_vp, _sz, _u32, _u64, _i32 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint64, C.c_int

# name -> (restype, argtypes); the list every header declaration must appear in
ABI_SYMBOLS = {
    "mer_abi_version": (C.c_int, []),
    "mer_error_kind_name": (C.c_char_p, [_i32]),
    "mer_expert_bytes": (_u64, [C.c_int32, _u64, _u64]),
    "mer_routed_expert_compatibility": (C.c_int, [C.c_int32, _u64, _u64]),
    "mer_backend_create": (C.c_int, [C.POINTER(MerBackendCfg), C.POINTER(_vp)]),
    "mer_backend_destroy": (None, [_vp]),
    "mer_backend_synchronize": (C.c_int, [_vp]),
    "mer_expert_admit": (C.c_int, [_vp, _u32, _u64, _vp, _sz, _u32]),
    "mer_expert_admit_device": (C.c_int, [_vp, _u32, _u64, _vp, _sz, _u32]),
    "mer_expert_retire": (C.c_int, [_vp, _u32, _u64]),
    "mer_expert_contains_generation": (C.c_int, [_vp, _u32, _u64]),
    "mer_gpu_cache_create": (C.c_int, [_u64, C.c_float, _u64, C.POINTER(_vp)]),
    "mer_gpu_cache_destroy": (None, [_vp]),
    "mer_gpu_cache_get": (C.c_int, [_vp, _u32, C.POINTER(MerGpuAdmission)]),
    "mer_gpu_cache_current_admission": (C.c_int, [_vp, _u32, C.POINTER(MerGpuAdmission)]),
    "mer_gpu_cache_contains": (C.c_int, [_vp, _u32]),
    "mer_gpu_cache_contains_generation": (C.c_int, [_vp, _u32, _u64]),
    "mer_gpu_cache_should_promote": (C.c_int, [_vp, _u64]),
    "mer_gpu_cache_claim_promotion": (C.c_int, [_vp, _u32, _u64]),
    "mer_gpu_cache_cancel_promotion": (None, [_vp, _u32]),
    "mer_gpu_cache_promote_hot_existing": (C.c_int, [_vp, _u32]),
    "mer_gpu_cache_promote_hot_sync": (C.c_int, [_vp, _u32, _u64, _u64, _vp, _sz, C.POINTER(_sz), C.POINTER(_u64)]),
    "mer_gpu_cache_promote_sync": (C.c_int, [_vp, _u32, _u64, _u64, _vp, _sz, C.POINTER(_sz), C.POINTER(_u64)]),
    "mer_gpu_cache_try_promote_lru_no_evict": (C.c_int, [_vp, _u32, _u64, _u64, C.POINTER(_u64)]),
    "mer_gpu_cache_demand_admission_preflight": (C.c_int, [_vp, _u32, _u64]),
    "mer_gpu_cache_demand_admit_lru": (C.c_int, [_vp, _u32, _u64, _u64, _vp, _sz, C.POINTER(_sz), C.POINTER(_u64)]),
    "mer_gpu_cache_remove": (C.c_int, [_vp, _u32, _u64]),
    "mer_gpu_cache_stats_read": (C.c_int, [_vp, C.POINTER(MerGpuCacheStats)]),
    "mer_gpu_cache_set_next_generation": (C.c_int, [_vp, _u64]),
    "mer_gpu_cache_marker_state": (C.c_int, [_vp, _u32]),
    "mer_expert_demand_admit": (C.c_int, [_vp, _vp, _u32, _vp, _sz, _u32, C.POINTER(_u64)]),
    "mer_expert_hot_promote": (C.c_int, [_vp, _vp, _u32, _vp, _sz, _u32, C.POINTER(C.c_int)]),
    "mer_expert_touch": (C.c_int, [_vp, _vp, _vp, _sz]),
    "mer_uth_probe": (C.c_int, [_vp, _sz, _sz, C.POINTER(MerUthInfo)]),
    "mer_uth_probe_prefix": (C.c_int, [_vp, _sz, _u64, _sz, C.POINTER(MerUthInfo)]),
    "mer_uth1_write": (C.c_int, [C.c_int32, _u64, _u64, _sz, _vp, _sz, C.POINTER(_sz)]),
    "mer_uth2_write": (C.c_int, [_u64, _u64, C.POINTER(MerUthProjection), _sz, _vp, _sz, C.POINTER(_sz)]),
    "mer_dataset_metadata_parse": (C.c_int, [C.c_char_p, _sz, C.POINTER(MerDatasetInfo)]),
    "mer_expert_admit_file": (C.c_int, [_vp, _u32, _u64, C.c_char_p, _sz, _u32]),
    "mer_router_install": (C.c_int, [_vp, _u32, _vp, C.POINTER(MerRouterCfg)]),
    "mer_layer_install": (C.c_int, [_vp, _u32, C.POINTER(MerLayerCfg)]),
    "mer_router_route": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _vp]),
    "mer_routed_expert_matmul": (C.c_int, [_vp, _u32, _u32, _vp, _sz, _sz, _vp]),
    "mer_routed_expert_matmul_batch": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _sz, _sz, _vp]),
    "mer_routed_expert_forward_f32": (C.c_int, [_vp, _u32, _u32, _vp, _sz, _vp]),
    "mer_moe_step_weighted_into": (C.c_int, [_vp, _u32, _vp, _vp, _vp, _sz, _vp]),
    "mer_moe_layer_forward": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _vp, _vp]),
    "mer_moe_layer_forward_device": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _vp, _vp, _vp]),
    "mer_dequant_projection_f32": (C.c_int, [_vp, _u32, _i32, _vp]),
    "mer_qualification_matvec": (C.c_int, [_vp, C.c_int32, _vp, _sz, _vp, _sz, _sz, _sz, _vp]),
    "mer_stage_timing_enable": (C.c_int, [_vp, _i32]),
    "mer_stage_timings_read": (C.c_int, [_vp, C.POINTER(MerStageTimings)]),
    "mer_expert_forward_noalloc": (C.c_int, [C.c_int32, _u64, _u64, _vp, _vp, _sz, _vp, C.c_float, _vp, C.c_char_p, _sz]),
    "mer_last_error": (C.c_int, [_vp, C.POINTER(MerErrorInfo)]),
    "mer_snapshot": (C.c_int, [_vp, C.POINTER(MerCounters)]),
    "mer_set_kernel_path": (C.c_int, [_vp, _i32]),
    "mer_ep_init": (C.c_int, [_vp, C.POINTER(MerEpCfg)]),
    "mer_ep_exchange_bytes": (_sz, [_vp]),
    "mer_ep_set_placement": (C.c_int, [_vp, _vp, _sz]),
    "mer_ep_export_handle": (C.c_int, [_vp, _vp]),
    "mer_ep_attach_handles": (C.c_int, [_vp, _vp, _sz]),
    "mer_ep_exchange_buffer": (_vp, [_vp]),
    "mer_ep_attach_pointers": (C.c_int, [_vp, C.POINTER(_vp), _sz]),
    "mer_router_route_device": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _vp, _vp]),
    "mer_ep_local_experts_forward_device": (C.c_int, [_vp, _u32, _vp, _vp, _vp, _sz, _sz, _vp, _vp]),
    "mer_ep_layer_forward_device": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _vp]),
    "mer_ep_nccl_unique_id": (C.c_int, [_vp]),
    "mer_ep_nccl_init": (C.c_int, [_vp, _vp]),
    "mer_ep_layer_forward_a2a_device": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _vp]),
    "mer_stream_check": (C.c_int, [_vp, _u32, _vp]),
    "mer_moe_layer_forward_submit": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _u32]),
    "mer_moe_layer_forward_wait": (C.c_int, [_vp, _u32]),
    "mer_ep_layer_forward_submit": (C.c_int, [_vp, _u32, _vp, _sz, _vp, _u32]),
}

_lib = None


def load_library():
    """Loads libmer_b200.so; raises (no fallback) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py build` "
                               "(there is no CPU fallback for this path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in ABI_SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError if the library does not export it
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
