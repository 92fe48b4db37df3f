"""The tcgen05 / TMEM grouped-GEMM family of the expert FFN (groups of a dozen tokens and more)
against the CPU oracle, through the same C-ABI entry points as the decode kernels."""
import numpy as np
import pytest

import mer_b200
import oracle
from mer_b200 import GpuExpertDispatchErrorKind as Kind

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("mer_b200.synth")

FFN_TOL = 1e-3  # max-abs error relative to the RMS of the reference output


def rel_rms_err(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


def backend(dtype, D, F, n_experts, **kw):
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    return mer_b200.Backend(dtype, D, F, stride * n_experts, kw.pop("max_experts", max(n_experts, 16)), **kw)


@pytest.mark.parametrize("dtype", [oracle.Q8_0, oracle.Q4_0])
@pytest.mark.parametrize("D,F,n_tokens", [(256, 256, 16), (256, 512, 13), (512, 256, 40), (1024, 768, 130), (2048, 768, 64)])
def test_one_expert_many_tokens_matches_oracle(dtype, D, F, n_tokens):
    blob = synth.make_expert_blob(dtype, D, F, 81, 0, 0)
    x = synth.make_activations(n_tokens, D, 81)
    with backend(dtype, D, F, 2, max_tokens=n_tokens) as b:
        b.admit(1, 1, blob)
        b.set_kernel_path(3)
        got = b.expert_forward_f32(0, 1, x)
        b.set_kernel_path(2)
        streamed = b.expert_forward_f32(0, 1, x)
    worst = 0.0
    for t in range(n_tokens):
        ref = oracle.expert_forward(dtype, blob, x[t], D, F, oracle.FWD_AUTHORITATIVE)
        worst = max(worst, rel_rms_err(got[t], ref))
    assert worst <= FFN_TOL, worst
    assert rel_rms_err(got, streamed) <= 1e-4  # both kernel families carry ~22-bit operands


def test_automatic_selection_takes_the_gemm_path_for_large_groups():
    dtype, E, D, F, k, B = oracle.Q8_0, 8, 512, 256, 2, 160  # 320 pairs over 8 experts: 40 tokens per expert
    blobs = [synth.make_expert_blob(dtype, D, F, 82, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 82)
    x = synth.make_activations(B, D, 82)
    with backend(dtype, D, F, E, max_tokens=B, max_top_k=k) as b:
        for e in range(E):
            b.admit(e, 1, blobs[e])
        mer_b200.LinearGate(W, E, D, k).bind(b, 0)
        out, ids, w = b.moe_layer_forward(0, x)
        b.set_kernel_path(2)
        out_stream, ids2, _ = b.moe_layer_forward(0, x)
        b.set_kernel_path(1)
        out_generic, _, _ = b.moe_layer_forward(0, x)
    ref, rids, rw, _ = oracle.moe_layer_forward(dtype, oracle.LinearGate(W, E, D, k), blobs, x, F, n_threads=8)
    assert (ids == rids).all() and (ids2 == rids).all()
    assert rel_rms_err(out, ref) <= FFN_TOL
    assert rel_rms_err(out, out_stream) <= 1e-4 and rel_rms_err(out, out_generic) <= 1e-4
    # automatic selection really differs from the streaming family here (different summation order)
    assert not np.array_equal(out, out_stream)


def test_ragged_groups_shared_expert_and_empty_experts():
    # Zipf-like skew: a few experts take most tokens, several get none; shared expert sees every token
    dtype, E, D, F, k, B = oracle.Q4_0, 16, 256, 256, 2, 70
    blobs = [synth.make_expert_blob(dtype, D, F, 83, 0, e) for e in range(E + 1)]
    W = synth.make_router(E, D, 83)
    bias = synth.zipf_logit_bias(E, 1.2, 83) if hasattr(synth, "zipf_logit_bias") else None
    x = synth.make_activations(B, D, 83)
    gate = mer_b200.LinearGate(W, E, D, k)
    with backend(dtype, D, F, E + 1, max_experts=64, max_tokens=B, max_top_k=k + 1) as b:
        for e in range(E + 1):
            b.admit(e, 1, blobs[e])
        gate.bind(b, 0, shared_expert_id=E)
        b.set_kernel_path(3)
        out, ids, w = b.moe_layer_forward(0, x)
    ref, rids, rw, _ = oracle.moe_layer_forward(dtype, oracle.LinearGate(W, E, D, k), blobs[:E], x, F, shared_blob=blobs[E], n_threads=8)
    assert (ids == rids).all()
    assert rel_rms_err(out, ref) <= FFN_TOL


def test_gemm_path_fails_closed_on_a_missing_expert():
    dtype, E, D, F, k, B = oracle.Q8_0, 4, 256, 256, 4, 20  # top-4 of 4: every expert is hit
    blobs = [synth.make_expert_blob(dtype, D, F, 84, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 84)
    x = synth.make_activations(B, D, 84)
    with backend(dtype, D, F, E, max_tokens=B, max_top_k=k) as b:
        for e in range(E):
            if e != 2:
                b.admit(e, 1, blobs[e])
        mer_b200.LinearGate(W, E, D, k).bind(b, 0)
        b.set_kernel_path(3)
        with pytest.raises(mer_b200.GpuExpertDispatchError) as err:
            b.moe_layer_forward(0, x)
        assert err.value.kind == Kind.ResidencyMiss


def test_swiglu_limit_and_nonfinite_rows_on_the_gemm_path():
    dtype, D, F, n = oracle.Q8_0, 256, 256, 24
    blob = synth.make_expert_blob(dtype, D, F, 85, 0, 0)
    x = synth.make_activations(n, D, 85) * 8.0
    x[5, 17] = np.nan
    with backend(dtype, D, F, 2, max_tokens=n, swiglu_limit=0.5) as b:
        b.admit(0, 1, blob)
        b.set_kernel_path(3)
        got = b.expert_forward_f32(0, 0, x)
    assert np.isnan(got[5]).all()  # a NaN activation poisons its own row only
    for t in (0, 6, 23):
        ref = oracle.expert_forward(dtype, blob, x[t], D, F, oracle.FWD_AUTHORITATIVE, swiglu_limit=0.5)
        assert rel_rms_err(got[t], ref) <= FFN_TOL


def test_full_size_prefill_properties_and_spot_check():
    # benchmark configuration 3 at full size: 2048 tokens, D=2048, F=768, E=128, k=8, Q8_0, Zipf-skewed routing.  Size-independent
    # properties: token-order invariance (bit-exact per token), agreement of the two kernel families, linearity in
    # the routing weights; plus an oracle spot check on a few tokens.
    cfg = synth.CONFIGS["cfg3-qwen3-prefill-q8_0"]
    E, D, F, k, B = cfg.num_experts, cfg.d_model, cfg.d_ff, cfg.top_k, 2048
    blobs = [synth.make_expert_blob(cfg.dtype, D, F, cfg.seed, 0, e) for e in range(E)]
    W = synth.make_router(E, D, cfg.seed)
    bias = synth.zipf_logit_bias(E, 1.0, cfg.seed, 0, strength=0.25)
    x = synth.make_activations(B, D, cfg.seed)
    gate = mer_b200.LinearGate(W, E, D, k)
    gate.logit_bias = bias
    perm = np.random.default_rng(3).permutation(B)
    with backend(cfg.dtype, D, F, E, max_experts=E, max_tokens=B, max_top_k=k) as b:
        for e in range(E):
            b.admit(e, 1, blobs[e])
        gate.bind(b, 0)
        out, ids, w = b.moe_layer_forward(0, x)          # automatic selection: the GEMM kernels at 128 tokens per expert
        again, _, _ = b.moe_layer_forward(0, x)
        shuffled, sids, _ = b.moe_layer_forward(0, x[perm])
        b.set_kernel_path(2)
        streamed, ids2, _ = b.moe_layer_forward(0, x)
    assert np.isfinite(out).all()
    # 16384 pairs are grouped with atomics, so the passes are cut differently from run to run; the bits must not change
    assert (again.view(np.uint32) == out.view(np.uint32)).all()
    counts = np.bincount(ids.ravel(), minlength=E)
    assert counts.max() > 2 * counts.mean() > 0 and counts.sum() == B * k  # skewed, every pair accounted for
    assert (sids == ids[perm]).all()
    # passes are cut differently, but the order of a token's additions depends only on its expert's token count
    assert rel_rms_err(shuffled, out[perm]) <= 1e-5
    assert (ids2 == ids).all()
    worst = max(rel_rms_err(out[t], streamed[t]) for t in range(B))
    assert worst <= 1e-4, worst
    og = oracle.LinearGate(W, E, D, k, logit_bias=bias)
    ref, rids, rw, _ = oracle.moe_layer_forward(cfg.dtype, og, blobs, x[:4], F, n_threads=4)
    assert (ids[:4] == rids).all()
    assert rel_rms_err(out[:4], ref) <= FFN_TOL
