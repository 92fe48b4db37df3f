"""ctypes/numpy front end of the CPU oracle (oracle/mer_oracle.c).

TEST INFRASTRUCTURE ONLY.  The oracle restates the reference's CPU arithmetic for
the routed quantized SwiGLU expert-FFN path and is the parity checker and the
timed CPU baseline.  Only the test-suite, the smoke check and the benchmark's
CPU-baseline legs may import it; the product package never does.

Parity pinning: the reference (Rust) cannot be built in this environment, so the
oracle is pinned against the literal fixtures of the reference's own unit tests
(tests/golden/), not against a reference binary.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libmer_oracle.so")

Q4_0, Q8_0 = 0, 1
BLOCK_ELEMS = 32
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34}
FWD_AUTHORITATIVE, FWD_Q8_SCALAR, FWD_BLOCK_PARTIAL, FWD_F64, FWD_SIMD8X4 = range(5)
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
OK, ERR_INVALID_LAYOUT, ERR_BUFFER_TOO_SMALL, ERR_TRUNCATED = range(4)


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (oracle/Makefile) if the library is missing or stale."""
    src = os.path.join(_HERE, "mer_oracle.c")
    hdr = os.path.join(_HERE, "mer_oracle.h")
    stale = not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in (src, hdr))
    if force or stale:
        subprocess.check_call(["make", "-s", "-C", _HERE] + (["-B"] if force else []))
    return _LIB_PATH


class _Gate(C.Structure):
    _fields_ = [("weights", C.c_void_p), ("num_experts", C.c_size_t), ("d_model", C.c_size_t),
                ("top_k", C.c_size_t), ("normalise_topk", C.c_int), ("scoring_func", C.c_int),
                ("correction_bias", C.c_void_p), ("n_group", C.c_size_t), ("topk_group", C.c_size_t),
                ("routed_scaling_factor", C.c_float), ("logit_bias", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        vp, sz, f32, i32, u64 = C.c_void_p, C.c_size_t, C.c_float, C.c_int, C.c_uint64
        L.mer_oracle_f16_to_f32.restype = f32
        L.mer_oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.mer_oracle_f32_to_f16.restype = C.c_uint16
        L.mer_oracle_f32_to_f16.argtypes = [f32]
        for n in ("dequant_q4_0_block", "dequant_q8_0_block"):
            getattr(L, "mer_oracle_" + n).argtypes = [vp, vp]
        for n in ("quant_q4_0_block", "quant_q8_0_block"):
            getattr(L, "mer_oracle_" + n).argtypes = [vp, sz, vp]
        L.mer_oracle_dequant_stream.argtypes = [i32, vp, sz, sz, vp]
        L.mer_oracle_projection_bytes.restype = sz
        L.mer_oracle_projection_bytes.argtypes = [i32, sz, sz]
        L.mer_oracle_expert_bytes.restype = sz
        L.mer_oracle_expert_bytes.argtypes = [i32, sz, sz]
        L.mer_oracle_silu.restype = f32
        L.mer_oracle_silu.argtypes = [f32]
        L.mer_oracle_expert_forward.argtypes = [i32, i32, vp, sz, vp, sz, sz, f32, vp, vp]
        L.mer_oracle_expert_forward_mt.argtypes = [i32, vp, sz, vp, sz, sz, f32, vp, i32]
        L.mer_oracle_q4_matvec.argtypes = [vp, sz, vp, sz, sz, sz, vp]
        L.mer_oracle_q8_row_dot_scalar.restype = f32
        L.mer_oracle_q8_row_dot_scalar.argtypes = [vp, vp, sz]
        L.mer_oracle_q8_row_dot_simd8x4.restype = f32
        L.mer_oracle_q8_row_dot_simd8x4.argtypes = [vp, vp, sz]
        L.mer_oracle_softmax_inplace.argtypes = [vp, sz]
        L.mer_oracle_route.argtypes = [C.POINTER(_Gate), vp, vp, vp, C.POINTER(sz), vp, C.POINTER(f32)]
        L.mer_oracle_route_stable.argtypes = [C.POINTER(_Gate), vp, vp, vp, C.POINTER(sz)]
        L.mer_oracle_combine.argtypes = [vp, vp, sz, sz, vp, i32]
        L.mer_oracle_accumulate_ordered_f16.argtypes = [vp, sz, vp, sz, sz, vp]
        L.mer_oracle_rmsnorm.argtypes = [vp, vp, sz, f32, vp]
        L.mer_oracle_rmsnorm.restype = None
        L.mer_oracle_shared_gate_scale.argtypes = [vp, vp, sz]
        L.mer_oracle_shared_gate_scale.restype = f32
        L.mer_oracle_add_residual.argtypes = [vp, vp, sz, vp]
        L.mer_oracle_add_residual.restype = None
        L.mer_oracle_synth_hidden_state.argtypes = [u64, sz, u64, vp]
        L.mer_oracle_randomized_q8_expert.argtypes = [sz, sz, u64, vp]
        L.mer_oracle_moe_layer_forward.argtypes = [i32, i32, C.POINTER(_Gate), vp, sz, vp, vp, sz, sz,
                                                   f32, vp, vp, vp, vp, i32]
        L.mer_oracle_moe_layer_forward_production.argtypes = [i32, C.POINTER(_Gate), vp, sz, vp, vp, sz, sz, f32, vp, i32]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _u8(a):
    a = np.ascontiguousarray(np.frombuffer(a, dtype=np.uint8) if isinstance(a, (bytes, bytearray)) else a,
                             dtype=np.uint8)
    return a


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class OracleError(Exception):
    def __init__(self, code):
        self.code = code
        super().__init__({1: "InvalidLayout", 2: "BufferTooSmall", 3: "TruncatedPayload"}.get(code, str(code)))


def f16_to_f32(bits: int) -> float:
    return float(lib().mer_oracle_f16_to_f32(int(bits) & 0xFFFF))


def f32_to_f16(v: float) -> int:
    return int(lib().mer_oracle_f32_to_f16(float(v)))


def dequant_block(dtype, block) -> np.ndarray:
    block = _u8(block)
    assert block.size == BLOCK_BYTES[dtype]
    out = np.empty(BLOCK_ELEMS, np.float32)
    (lib().mer_oracle_dequant_q4_0_block if dtype == Q4_0 else lib().mer_oracle_dequant_q8_0_block)(_p(block), _p(out))
    return out


def quant_block(dtype, values) -> np.ndarray:
    values = _f32(values)
    assert values.size <= BLOCK_ELEMS
    out = np.empty(BLOCK_BYTES[dtype], np.uint8)
    (lib().mer_oracle_quant_q4_0_block if dtype == Q4_0 else lib().mer_oracle_quant_q8_0_block)(
        _p(values), values.size, _p(out))
    return out


def dequant_stream(dtype, src, n_weights) -> np.ndarray:
    src = _u8(src)
    out = np.empty(n_weights, np.float32)
    rc = lib().mer_oracle_dequant_stream(dtype, _p(src), src.size, n_weights, _p(out))
    if rc:
        raise OracleError(rc)
    return out


def projection_bytes(dtype, d_model, d_ff) -> int:
    return lib().mer_oracle_projection_bytes(dtype, d_model, d_ff)


def expert_bytes(dtype, d_model, d_ff) -> int:
    return lib().mer_oracle_expert_bytes(dtype, d_model, d_ff)


def silu(x: float) -> float:
    return float(lib().mer_oracle_silu(float(x)))


def expert_forward(dtype, blob, x, d_model, d_ff, variant=FWD_AUTHORITATIVE, swiglu_limit=0.0,
                   return_gated=False):
    blob, x = _u8(blob), _f32(x)
    assert x.size == d_model
    y = np.empty(d_model, np.float32)
    gated = np.empty(d_ff, np.float32) if return_gated else None
    rc = lib().mer_oracle_expert_forward(dtype, variant, _p(blob), blob.size, _p(x), d_model, d_ff,
                                         swiglu_limit, _p(y), _p(gated))
    if rc:
        raise OracleError(rc)
    return (y, gated) if return_gated else y


def expert_forward_mt(dtype, blob, x, d_model, d_ff, n_threads, swiglu_limit=0.0) -> np.ndarray:
    blob, x = _u8(blob), _f32(x)
    y = np.empty(d_model, np.float32)
    rc = lib().mer_oracle_expert_forward_mt(dtype, _p(blob), blob.size, _p(x), d_model, d_ff, swiglu_limit,
                                            _p(y), n_threads)
    if rc < 0:
        raise OracleError(-rc)
    return y


def has_avx2_fma() -> bool:
    return bool(lib().mer_oracle_has_avx2_fma())


def q4_matvec(weights, x, rows, columns, w_block_off=0) -> np.ndarray:
    weights, x = _u8(weights), _f32(x)
    out = np.empty(rows, np.float32)
    rc = lib().mer_oracle_q4_matvec(_p(weights), weights.size, _p(x), rows, columns, w_block_off, _p(out))
    if rc:
        raise OracleError(rc)
    return out


def q8_row_dot(row, x, simd=False) -> float:
    row, x = _u8(row), _f32(x)
    f = lib().mer_oracle_q8_row_dot_simd8x4 if simd else lib().mer_oracle_q8_row_dot_scalar
    return float(f(_p(row), _p(x), x.size))


def softmax(v) -> np.ndarray:
    v = _f32(v).copy()
    lib().mer_oracle_softmax_inplace(_p(v), v.size)
    return v


class LinearGate:
    """Mirror of the reference's LinearGate (gating.rs:118-238) evaluated by the C oracle."""

    def __init__(self, weights, num_experts, d_model, top_k, scoring_func=SCORE_SOFTMAX, normalise_topk=True,
                 correction_bias=None, n_group=1, topk_group=1, routed_scaling_factor=1.0, logit_bias=None):
        assert 0 < top_k <= num_experts, "top_k must be in 1..=num_experts"
        self.weights = _f32(weights).reshape(num_experts, d_model)
        self.bias = None if correction_bias is None else _f32(correction_bias)
        self.logit_bias = None if logit_bias is None else _f32(logit_bias)
        if self.bias is not None:
            assert self.bias.size == num_experts
        self.num_experts, self.d_model, self.top_k = num_experts, d_model, top_k
        self.c = _Gate(self.weights.ctypes.data, num_experts, d_model, top_k, int(normalise_topk), scoring_func,
                       self.bias.ctypes.data if self.bias is not None else None, max(n_group, 1), topk_group,
                       routed_scaling_factor, self.logit_bias.ctypes.data if self.logit_bias is not None else None)

    def route(self, x, stable=False, detail=False):
        x = _f32(x)
        assert x.size == self.d_model
        ids = np.zeros(self.top_k, np.uint32)
        w = np.zeros(self.top_k, np.float32)
        n = C.c_size_t(0)
        if stable:
            rc = lib().mer_oracle_route_stable(C.byref(self.c), _p(x), _p(ids), _p(w), C.byref(n))
            if rc:
                raise OracleError(rc)
            return ids[:n.value], w[:n.value]
        scores = np.empty(self.num_experts, np.float32)
        gap = C.c_float(0)
        rc = lib().mer_oracle_route(C.byref(self.c), _p(x), _p(ids), _p(w), C.byref(n), _p(scores), C.byref(gap))
        if rc:
            raise OracleError(rc)
        if detail:
            return ids[:n.value], w[:n.value], scores, gap.value
        return ids[:n.value], w[:n.value]


def combine(outputs, scores, skip_zero=False) -> np.ndarray:
    outputs, scores = _f32(outputs), _f32(scores)
    k = scores.size
    if k == 0:
        return np.empty(0, np.float32)
    d = outputs.size // k
    out = np.empty(d, np.float32)
    lib().mer_oracle_combine(_p(outputs), _p(scores), k, d, _p(out), int(skip_zero))
    return out


def rmsnorm(x, weight, eps=1e-6) -> np.ndarray:
    """RmsNorm::forward (transformer.rs:62-80)."""
    x, weight = _f32(x), _f32(weight)
    assert x.size == weight.size
    y = np.empty_like(x)
    lib().mer_oracle_rmsnorm(_p(x), _p(weight), x.size, C.c_float(eps), _p(y))
    return y


def shared_gate_scale(gate_inp, x) -> float:
    """sigmoid(gate_inp . x): the shared expert's gate scalar (transformer.rs:2224-2231)."""
    g, x = _f32(gate_inp), _f32(x)
    assert g.size == x.size
    return float(lib().mer_oracle_shared_gate_scale(_p(g), _p(x), x.size))


def add_residual(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().mer_oracle_add_residual(_p(a), _p(b), a.size, _p(out))
    return out


def moe_block_forward(dtype, gate, expert_blobs, hidden, d_ff, rms_weight=None, eps=1e-6, shared_blob=None, shared_gate=None,
                      residual=True, variant=FWD_AUTHORITATIVE, n_threads=1):
    """The MoE block of a decoder layer, token by token (transformer.rs:2493-2574, model.rs:2742-2763):
    normed = RMSNorm(hidden); routing and routed experts on normed; x = hidden + sum_slots w * y (slot order); then
    x = x + scale * shared(normed) with scale = sigmoid(shared_gate . normed) when a gate vector is given.
    Returns (out[B, D], ids[B, k], weights[B, k])."""
    hidden = _f32(hidden).reshape(-1, gate.d_model)
    normed = np.stack([rmsnorm(h, rms_weight, eps) for h in hidden]) if rms_weight is not None else hidden
    moe, ids, w, _ = moe_layer_forward(dtype, gate, expert_blobs, normed, d_ff, variant=variant, n_threads=n_threads)
    out = np.stack([add_residual(h, m) for h, m in zip(hidden, moe)]) if residual else moe
    if shared_blob is not None:
        rows = []
        for t in range(hidden.shape[0]):
            y = expert_forward(dtype, shared_blob, normed[t], gate.d_model, d_ff, variant=variant)
            if shared_gate is not None:
                y = (y * np.float32(shared_gate_scale(shared_gate, normed[t]))).astype(np.float32)
            rows.append(add_residual(out[t], y))
        out = np.stack(rows)
    return out, ids, w


def accumulate_ordered_f16(outputs_f16_bits, weights, d_model):
    o = np.ascontiguousarray(outputs_f16_bits, dtype=np.uint16)
    w = _f32(weights)
    out = np.empty(d_model, np.float32)
    ok = lib().mer_oracle_accumulate_ordered_f16(_p(o), o.size, _p(w), w.size, d_model, _p(out))
    return out if ok else None


def synth_hidden_state(token_idx, d_model, seed) -> np.ndarray:
    out = np.empty(d_model, np.float32)
    lib().mer_oracle_synth_hidden_state(token_idx, d_model, seed, _p(out))
    return out


def randomized_q8_expert(d_model, d_ff, state) -> np.ndarray:
    out = np.empty(expert_bytes(Q8_0, d_model, d_ff), np.uint8)
    lib().mer_oracle_randomized_q8_expert(d_model, d_ff, state & (2**64 - 1), _p(out))
    return out


def moe_layer_forward(dtype, gate: LinearGate, expert_blobs, x, d_ff, variant=FWD_AUTHORITATIVE,
                      shared_blob=None, swiglu_limit=0.0, n_threads=1):
    """Token-by-token MoE layer: route -> experts -> slot-order weighted sum.

    Returns (out[B,D], ids[B,k] (0xFFFFFFFF where unselected), weights[B,k], gaps[B])."""
    x = _f32(x).reshape(-1, gate.d_model)
    blobs = [_u8(b) for b in expert_blobs]
    blob_len = blobs[0].size
    assert all(b.size == blob_len for b in blobs)
    ptrs = (C.c_void_p * len(blobs))(*[b.ctypes.data for b in blobs])
    shared = _u8(shared_blob) if shared_blob is not None else None
    B = x.shape[0]
    out = np.empty((B, gate.d_model), np.float32)
    ids = np.empty((B, gate.top_k), np.uint32)
    w = np.empty((B, gate.top_k), np.float32)
    gaps = np.empty(B, np.float32)
    rc = lib().mer_oracle_moe_layer_forward(dtype, variant, C.byref(gate.c), ptrs, blob_len, _p(shared), _p(x), B,
                                            d_ff, swiglu_limit, _p(out), _p(ids), _p(w), _p(gaps), n_threads)
    if rc:
        raise OracleError(rc)
    return out, ids, w, gaps


def moe_layer_forward_production(dtype, gate: LinearGate, expert_blobs, x, d_ff, n_threads, shared_blob=None,
                                 swiglu_limit=0.0, _ptr_cache={}):
    """Production-shaped (fused zero-copy AVX2 rows, threaded) layer forward: the timed CPU baseline."""
    x = _f32(x).reshape(-1, gate.d_model)
    blobs = [_u8(b) for b in expert_blobs]
    ptrs = (C.c_void_p * len(blobs))(*[b.ctypes.data for b in blobs])
    shared = _u8(shared_blob) if shared_blob is not None else None
    out = np.empty_like(x)
    rc = lib().mer_oracle_moe_layer_forward_production(dtype, C.byref(gate.c), ptrs, blobs[0].size, _p(shared), _p(x),
                                                       x.shape[0], d_ff, swiglu_limit, _p(out), n_threads)
    if rc:
        raise OracleError(rc)
    return out
