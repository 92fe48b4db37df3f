"""Whole MoE layers at the full sizes of the benchmark configurations, through the C ABI, spot-checked against the
CPU oracle: the DeepSeek-V3-shaped layer (D=7168, F=2048, Q4_0, 256 routed experts + shared, sigmoid gating with
8 groups / top-4 groups, top-8, x2.5) and the Mixtral-shaped layer (D=4096, F=14336, Q4_0, 8 experts, top-2), each
at a decode batch (streaming kernels) and at a batch large enough for the tcgen05 GEMM kernels.

The resident experts are generated in device memory (the torch form of the generator); the oracle reads the numpy
form of the same generator for the few experts the checked tokens are routed to."""
import numpy as np
import pytest

import mer_b200
import oracle

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("mer_b200.synth")
FFN_TOL = 1e-3


def fill_layer(b, cfg, torch, shared_id=None):
    dev = torch.device("cuda", 0)
    eb = mer_b200.expert_bytes(cfg.dtype, cfg.d_model, cfg.d_ff)
    experts = list(range(cfg.num_experts)) + ([cfg.num_experts] if shared_id is not None else [])
    chunk = max(1, int((1 << 30) // (eb * 10)))
    for i in range(0, len(experts), chunk):
        part = experts[i:i + chunk]
        blobs = synth.make_expert_blobs_torch(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, 0, part, dev)
        torch.cuda.synchronize()
        for j, e in enumerate(part):
            b.admit_device(shared_id if e == cfg.num_experts else e, 1, blobs[j].data_ptr(), eb, wait=False)
        b.synchronize()
        del blobs


def check_tokens(cfg, og, x, out, ids, w, tokens):
    """Oracle recomputation of the given token rows: routing identical (tie-ambiguous tokens skipped), mixing weights
    equal, outputs within the bar."""
    routed = {t: og.route(x[t], detail=True) for t in tokens}
    need = sorted({int(e) for r in routed.values() for e in r[0]})
    eb = mer_b200.expert_bytes(cfg.dtype, cfg.d_model, cfg.d_ff)
    filler = np.zeros(eb, np.uint8)
    have = {e: synth.make_expert_blob(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, 0, e) for e in need}
    shared = synth.make_expert_blob(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, 0, cfg.num_experts) if cfg.shared else None
    blob_list = [have.get(e, filler) for e in range(cfg.num_experts)]
    ref, rids, rw, _ = oracle.moe_layer_forward(cfg.dtype, og, blob_list, x[list(tokens)], cfg.d_ff, shared_blob=shared, n_threads=8)
    checked = 0
    for i, t in enumerate(tokens):
        rid, _, scores, gap = routed[t]
        sel = np.sort(scores[rid] + (og.bias[rid] if og.bias is not None else 0))
        if gap < 1e-6 * abs(sel[0]) or (np.diff(sel) < 1e-6 * np.abs(sel[1:])).any():
            continue
        checked += 1
        assert ids[t].tolist() == rids[i].tolist(), f"token {t}: top-k expert indices differ"
        assert np.abs(w[t] - rw[i]).max() <= 4e-6 * max(1.0, float(np.abs(rw[i]).max()))
        rms = float(np.sqrt(np.mean(ref[i].astype(np.float64) ** 2)))
        err = float(np.abs(out[t].astype(np.float64) - ref[i]).max()) / rms
        assert err <= FFN_TOL, f"token {t}: max-abs / RMS = {err}"
    assert checked >= 1


def test_deepseek_v3_shaped_layer_at_full_size():
    torch = pytest.importorskip("torch")
    cfg = synth.CONFIGS["cfg4-deepseek-v3-q4_0"]
    E, D, F, k = cfg.num_experts, cfg.d_model, cfg.d_ff, cfg.top_k
    assert (E, D, F, k, cfg.n_group, cfg.topk_group, cfg.scaling) == (256, 7168, 2048, 8, 8, 4, 2.5)
    rng = np.random.default_rng(4)
    bias = rng.normal(0, 0.02, E).astype(np.float32)  # e_score_correction_bias: steers selection only (gating.rs:406-416)
    W = synth.make_router(E, D, cfg.seed, 0)
    og = oracle.LinearGate(W, E, D, k, scoring_func=oracle.SCORE_SIGMOID, correction_bias=bias, n_group=8, topk_group=4,
                           routed_scaling_factor=2.5)
    eb = mer_b200.expert_bytes(cfg.dtype, D, F)
    stride = (256 + eb + 4095) // 4096 * 4096
    B_big = 1024  # 9 x 1024 pairs over 257 experts: a mean of 36 tokens per expert, the tcgen05 GEMM kernels run
    shared_id = E
    with mer_b200.Backend(cfg.dtype, D, F, stride * (E + 1), 2 * E, max_tokens=B_big, max_top_k=k + 1) as b:
        fill_layer(b, cfg, torch, shared_id=shared_id)
        gate = mer_b200.LinearGate.with_routing(W, E, D, k, mer_b200.ScoringFunc.Sigmoid, True, bias, 8, 4, 2.5)
        gate.bind(b, 0, shared_id)
        for B, tokens in ((1, [0]), (16, [0, 9, 15]), (B_big, [0, 511, 1023])):
            x = synth.make_activations(B, D, cfg.seed, B)
            before = b.snapshot()["kernel_launches"]
            out, ids, w = b.moe_layer_forward(0, x)
            assert b.snapshot()["kernel_launches"] > before
            check_tokens(cfg, og, x, out, ids, w, tokens)


def test_mixtral_shaped_layer_at_full_size():
    torch = pytest.importorskip("torch")
    cfg = synth.CONFIGS["cfg0-mixtral-q4_0"]
    E, D, F, k = cfg.num_experts, cfg.d_model, cfg.d_ff, cfg.top_k
    assert (E, D, F, k) == (8, 4096, 14336, 2)
    W = synth.make_router(E, D, cfg.seed, 0)
    og = oracle.LinearGate(W, E, D, k)
    eb = mer_b200.expert_bytes(cfg.dtype, D, F)
    assert eb == 99090432
    stride = (256 + eb + 4095) // 4096 * 4096
    with mer_b200.Backend(cfg.dtype, D, F, stride * E, E, max_tokens=256, max_top_k=k) as b:
        fill_layer(b, cfg, torch)
        mer_b200.LinearGate(W, E, D, k).bind(b, 0)
        # batch 16: more than eight tokens on the popular experts, the streaming kernels make two passes per expert;
        # batch 256: 64 tokens per expert on average, the GEMM kernels run with K = 14336 in the down projection
        for B, tokens in ((1, [0]), (16, [3, 12]), (256, [0, 255])):
            x = synth.make_activations(B, D, cfg.seed, 100 + B)
            out, ids, w = b.moe_layer_forward(0, x)
            check_tokens(cfg, og, x, out, ids, w, tokens)
        # the kernel families agree with each other at this size too
        x = synth.make_activations(24, D, cfg.seed, 7)
        b.set_kernel_path(2)
        stream_out, _, _ = b.moe_layer_forward(0, x)
        b.set_kernel_path(3)
        gemm_out, _, _ = b.moe_layer_forward(0, x)
        rms = np.sqrt(np.mean(stream_out.astype(np.float64) ** 2, axis=1, keepdims=True))
        assert float((np.abs(stream_out - gemm_out) / rms).max()) <= 5e-4
