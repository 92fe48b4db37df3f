"""Host-side mirror of the reference's routed-expert GPU boundary over the C-ABI library.

The product is libmer_b200.so (hand-written sm_100a CUDA behind `extern "C"` entry points,
declared in include/mer_b200.h).  This package only binds it with ctypes and mirrors the
reference's operator names (`routed_expert_matmul`, `routed_expert_matmul_batch_q4`,
`LinearGate.route`, `moe_step_weighted_into`, typed `GpuExpertDispatchError`) so that tests
read like the reference's own.  There is no CPU fallback: if the library is missing or no
CUDA device is present, calls raise.
"""
from .capi import (ABI_SYMBOLS, DTYPE_Q4_0, DTYPE_Q8_0, EXPERT_NONE, LIB_PATH, SCORE_SIGMOID, SCORE_SOFTMAX,
                   MerCounters, MerErrorInfo, load_library)
from .backend import (Backend, GpuExpertBatchDispatchOutcome, GpuExpertDispatchError, GpuExpertDispatchErrorKind,
                      expert_bytes, expert_forward_noalloc, routed_expert_gpu_compatibility)
from .expert_cache import (GpuAdmission, GpuDemandAdmissionError, GpuDemandAdmissionPreflight, GpuExpertCache,
                           GpuHotPromotionOutcome, GpuLookup)
from .gating import LinearGate, RoutingDecision, ScoringFunc

__all__ = [
    "ABI_SYMBOLS", "Backend", "DTYPE_Q4_0", "DTYPE_Q8_0", "EXPERT_NONE", "GpuExpertBatchDispatchOutcome",
    "GpuAdmission", "GpuDemandAdmissionError", "GpuDemandAdmissionPreflight", "GpuExpertCache",
    "GpuExpertDispatchError", "GpuExpertDispatchErrorKind", "GpuHotPromotionOutcome", "GpuLookup", "LIB_PATH", "LinearGate", "MerCounters", "MerErrorInfo",
    "RoutingDecision", "SCORE_SIGMOID", "SCORE_SOFTMAX", "ScoringFunc", "expert_bytes", "expert_forward_noalloc",
    "load_library",
    "routed_expert_gpu_compatibility",
]
