"""Pins the CPU oracle against the literal fixtures of the reference's own unit tests.

Each test names the reference test it mirrors (paths relative to rust-engine/src/)."""
import math

import numpy as np
import pytest

import oracle

DT = {"q4_0": oracle.Q4_0, "q8_0": oracle.Q8_0}


def test_q4_0_non_symmetric_block_matches_literal(golden):
    # inference.rs:5613-5626
    g = golden["q4_0_non_symmetric_block"]
    got = oracle.dequant_block(oracle.Q4_0, np.array(g["block"], np.uint8))
    assert got.tolist() == g["expected"]


def test_q4_0_writer_emits_exact_ggml_nibble_bytes(golden):
    # inference.rs:5640-5661
    g = golden["q4_0_writer"]
    assert oracle.quant_block(oracle.Q4_0, g["src"]).tolist() == g["expected_block"]


@pytest.mark.parametrize("dtype", [oracle.Q4_0, oracle.Q8_0])
def test_zero_block_round_trips_to_zero(dtype):
    # inference.rs:5735-5745, 5789-5797
    blk = oracle.quant_block(dtype, np.zeros(32, np.float32))
    assert blk[0] == 0 and blk[1] == 0
    if dtype == oracle.Q4_0:
        assert (blk[2:] == 0x88).all()
    assert (oracle.dequant_block(dtype, blk) == 0.0).all()


@pytest.mark.parametrize("dtype,scale,div", [(oracle.Q4_0, 1.5, 7.0), (oracle.Q8_0, 1.5, 127.0)])
def test_quantize_dequantize_round_trip_bound(dtype, scale, div):
    # inference.rs:5664-5732, 5761-5786: |err| <= d * 1.01 with d = max_abs / 7 (resp. 127)
    state = 0xCAFEBABE if dtype == oracle.Q4_0 else 0xC0FFEE
    vals = []
    for _ in range(32):
        state ^= (state << 13) & (2**64 - 1)
        state ^= state >> 7
        state ^= (state << 17) & (2**64 - 1)
        vals.append((np.float32(state >> 40) / np.float32(1 << 23) - np.float32(1.0)) * np.float32(scale))
    vals = np.array(vals, np.float32)
    dec = oracle.dequant_block(dtype, oracle.quant_block(dtype, vals))
    d = np.abs(vals).max() / div
    assert np.abs(dec - vals).max() <= d * 1.01


def test_expert_bytes(golden):
    # inference.rs:5748-5758, 5800-5805 and the benchmark shapes
    for c in golden["expert_bytes"]:
        assert oracle.expert_bytes(DT[c["dtype"]], c["d_model"], c["d_ff"]) == c["bytes"]


def test_canonical_raw_q4_cases(golden):
    # q4_parity.rs:470-572 with cpu_q4_matvec 591-619; expectation from the independent restatement
    g = golden["q4_raw_cases"]
    assert len(g["cases"]) == 8
    for c in g["cases"]:
        got = oracle.q4_matvec(np.array(c["weights"], np.uint8), c["input"], c["rows"], c["columns"], c["w_block_off"])
        assert got.tolist() == c["expected"], c["name"]  # same fp32 order => bit-equal
    zero = g["cases"][0]
    assert zero["expected"] == [0.0]


def test_q4_complete_expert_variants(golden):
    # q4_parity.rs:574-589 inputs over the expert of inference.rs:6552-6566
    g = golden["q4_complete_expert"]
    blob = np.array(g["blob"], np.uint8)
    assert blob.size == oracle.expert_bytes(oracle.Q4_0, g["d_model"], g["d_ff"])
    for x, exp in zip(g["inputs"], g["expected_f64"]):
        exp = np.array(exp)
        for variant in range(5):
            y = oracle.expert_forward(oracle.Q4_0, blob, x, g["d_model"], g["d_ff"], variant)
            tol = 1e-5 + 1e-4 * np.abs(exp)  # RAW tolerance, q4_parity.rs:26-27
            assert (np.abs(y - exp) <= tol).all(), variant
        # f16 boundary emulation (engine.rs:4943-4989): f16(x) -> forward -> f16(y), tol 2e-3 + 5e-3*|ref|
        xh = np.array(x, np.float32).astype(np.float16).astype(np.float32)
        yh = oracle.expert_forward(oracle.Q4_0, blob, xh, g["d_model"], g["d_ff"]).astype(np.float16).astype(np.float32)
        assert (np.abs(yh - exp) <= g["abs_tol_f16_boundary"] + g["rel_tol_f16_boundary"] * np.abs(exp)).all()


def test_q8_row_cases(golden):
    # kernels/avx2.rs:262-288: SIMD-order row dot vs scalar order, 5 widths x 7 cases x 3 seeds x {gate, up}
    g = golden["q8_row_cases"]
    assert len(g["rows"]) == 5 * 7 * 3 * 2
    mask = 2**64 - 1
    for rc in g["rows"]:
        width, case, state = rc["width"], rc["case"], rc["seed"]
        row = np.zeros(width // 32 * 34, np.uint8)
        for block in range(width // 32):
            bits = {0: 0, 1: 1, 2: 0x7BFF, 6: 0x0400}.get(case)
            if bits is None:
                bits = int(np.float16(np.float32(0.003) + np.float32(block) * np.float32(0.00001)).view(np.uint16))
            row[block * 34] = bits & 0xFF
            row[block * 34 + 1] = bits >> 8
            for i in range(32):
                if case == 3:
                    q = 0
                elif case == 4:
                    q = -128 if (i + block) % 2 == 0 else 127
                elif case == 5:
                    q = -1 if (i + block) % 2 == 0 else 1
                else:
                    state ^= (state << 13) & mask
                    state ^= state >> 7
                    state ^= (state << 17) & mask
                    q = state & 0xFF
                row[block * 34 + 2 + i] = q & 0xFF
        x = (np.sin(np.arange(width, dtype=np.float32) * np.float32(0.013)).astype(np.float32) * np.float32(0.01))
        ref = rc["expected_scalar"]
        scalar = oracle.q8_row_dot(row, x, simd=False)
        simd = oracle.q8_row_dot(row, x, simd=True)
        tol = g["abs_tol"] + abs(ref) * g["rel_tol"]
        assert abs(scalar - ref) <= tol and abs(simd - ref) <= tol, rc


def test_randomized_q8_expert_and_direct_forward(golden):
    # inference.rs:5905-5926 generator; 5983-6110 direct vs dequant forward at tol 3e-3*max(|a|,1)+3e-5
    g = golden["randomized_q8_expert"]
    for c in g["cases"]:
        blob = oracle.randomized_q8_expert(c["d_model"], c["d_ff"], c["state"])
        assert blob.size == c["blob_len"] and blob[:68].tolist() == c["blob_head"] and int(blob.sum()) == c["blob_sum"]
        x = oracle.synth_hidden_state(c["token"], c["d_model"], c["seed"])
        exp = np.array(c["expected_f64"])
        for variant in range(5):
            y = oracle.expert_forward(oracle.Q8_0, blob, x, c["d_model"], c["d_ff"], variant)
            assert (np.abs(y - exp) <= g["rel_tol"] * np.maximum(np.abs(exp), 1.0) + g["abs_tol"]).all()
        ymt = oracle.expert_forward_mt(oracle.Q8_0, blob, x, c["d_model"], c["d_ff"], 3)
        simd = oracle.expert_forward(oracle.Q8_0, blob, x, c["d_model"], c["d_ff"], oracle.FWD_SIMD8X4)
        assert (np.abs(ymt - simd) <= 2e-5 * np.maximum(np.abs(simd), 1.0) + 3e-5).all()
    # rows that straddle blocks (37x45, 64x45, 37x64): flat fallbacks agree with the dequantised forward
    for dm, df in g["unaligned_shapes"]:
        blob = oracle.randomized_q8_expert(dm, df, 0x51A1A11E)
        x = oracle.synth_hidden_state(9, dm, 3)
        a = oracle.expert_forward(oracle.Q8_0, blob, x, dm, df, oracle.FWD_AUTHORITATIVE)
        b = oracle.expert_forward(oracle.Q8_0, blob, x, dm, df, oracle.FWD_Q8_SCALAR)
        t = oracle.expert_forward(oracle.Q8_0, blob, x, dm, df, oracle.FWD_F64)
        assert (np.abs(a - t) <= 3e-3 * np.maximum(np.abs(t), 1.0) + 3e-5).all()
        assert (np.abs(b - t) <= 3e-3 * np.maximum(np.abs(t), 1.0) + 3e-5).all()


def test_truncated_and_short_payloads():
    # inference.rs:6180-6245: a shortfall within one page is Truncated, a larger one BufferTooSmall
    dm, df = 128, 96
    blob = oracle.randomized_q8_expert(dm, df, 7)
    x = oracle.synth_hidden_state(0, dm, 0)
    with pytest.raises(oracle.OracleError) as e:
        oracle.expert_forward(oracle.Q8_0, blob[:-1], x, dm, df)
    assert e.value.code == oracle.ERR_TRUNCATED
    with pytest.raises(oracle.OracleError) as e:
        oracle.expert_forward(oracle.Q8_0, blob[:blob.size // 2], x, dm, df)
    assert e.value.code == oracle.ERR_BUFFER_TOO_SMALL
    padded = np.concatenate([blob, np.full(4096, 0xAB, np.uint8)])  # page padding after the payload is ignored
    assert (oracle.expert_forward(oracle.Q8_0, padded, x, dm, df) == oracle.expert_forward(oracle.Q8_0, blob, x, dm, df)).all()


def test_nan_and_inf_propagate():
    # inference.rs:6215-6245: non-finite activations reach the output instead of being masked
    dm, df = 32, 32
    blob = oracle.randomized_q8_expert(dm, df, 11)
    x = oracle.synth_hidden_state(1, dm, 1)
    x[3] = np.nan
    assert np.isnan(oracle.expert_forward(oracle.Q8_0, blob, x, dm, df)).all()


def test_synth_hidden_state_bit_exact(golden):
    # inference.rs:3064-3082
    for c in golden["synth_hidden_state"]:
        got = oracle.synth_hidden_state(c["token"], c["d_model"], c["seed"])
        assert got.tolist() == c["values"]
        assert (got >= -1.0).all() and (got < 1.0).all()


def test_synth_q4_0_blob_forward(golden):
    # inference.rs:6610-6623: scale 0.05, all nibbles 9 => every weight = 0.05
    c = golden["synth_q4_0_blob"]
    dm, df = c["d_model"], c["d_ff"]
    blk = np.array([0, 0] + [c["nibble"] | (c["nibble"] << 4)] * 16, np.uint8)
    bits = oracle.f32_to_f16(c["scale"])
    blk[0], blk[1] = bits & 0xFF, bits >> 8
    blob = np.tile(blk, 3 * dm * df // 32)
    w = oracle.dequant_stream(oracle.Q4_0, blob, dm * df)
    assert (w == np.float32(oracle.f16_to_f32(bits))).all()
    x = np.ones(dm, np.float32)
    y = oracle.expert_forward(oracle.Q4_0, blob, x, dm, df)
    s = oracle.f16_to_f32(bits)
    g = dm * s
    exp = df * s * (g / (1 + math.exp(-g)) * g)
    assert np.allclose(y, exp, rtol=1e-5)


def _gate(c):
    return oracle.LinearGate(
        c["weights"], c["num_experts"], c["d_model"], c["top_k"],
        scoring_func=oracle.SCORE_SIGMOID if c.get("scoring") == "sigmoid" else oracle.SCORE_SOFTMAX,
        normalise_topk=c.get("normalise_topk", True), correction_bias=c.get("correction_bias"),
        n_group=c.get("n_group", 1), topk_group=c.get("topk_group", 1),
        routed_scaling_factor=c.get("routed_scaling_factor", 1.0))


def test_router_cases(golden):
    # gating.rs:527-911
    for c in golden["router_cases"]:
        gate = _gate(c)
        ids, w = gate.route(c["x"])
        assert ids.tolist() == c["experts"], c["name"]
        if "weights_expected" in c:
            assert np.abs(w - np.array(c["weights_expected"])).max() < c["tol"], c["name"]
        if "weight_sum" in c:
            assert abs(float(w.sum()) - c["weight_sum"]) < c.get("tol", 1e-5), c["name"]
        if c.get("descending"):
            assert w[0] > w[1]
        sid, sw = gate.route(c["x"], stable=True)  # reference_route_stable, gating.rs:684-764
        assert sid.tolist() == ids.tolist() and np.abs(sw - w).max() < 1e-6, c["name"]


def test_router_non_finite_scores_are_skipped_and_softmax_falls_back_to_uniform():
    # gating.rs:315-318 (non-finite skipped), transformer.rs:2807-2819 (non-finite row -> uniform)
    gate = oracle.LinearGate(np.eye(4, dtype=np.float32), 4, 4, 2, scoring_func=oracle.SCORE_SIGMOID,
                             normalise_topk=False, correction_bias=[0, float("nan"), 0, 0])
    ids, w = gate.route([1.0, 9.0, 0.5, 0.0])
    assert ids.tolist() == [0, 2]
    sm = oracle.softmax([1.0, float("nan"), 2.0, 3.0])
    assert sm.tolist() == [0.25] * 4
    assert oracle.softmax([float("inf"), 0.0]).tolist() == [0.5, 0.5]


def test_combine_cases(golden):
    # inference.rs:4628-4705
    for c in golden["combine_cases"]:
        out = oracle.combine(np.array(c["outputs"], np.float32).reshape(-1), c["scores"])
        assert out.size == len(c["expected"])
        if out.size:
            assert np.abs(out - np.array(c["expected"])).max() <= c["tol"]


def test_ordered_f16_batch_combine(golden):
    # engine.rs:6579-6588
    c = golden["ordered_f16_batch"]
    out = oracle.accumulate_ordered_f16(c["outputs_f16_bits"], c["weights"], c["d_model"])
    assert out.tolist() == c["expected"]
    assert oracle.accumulate_ordered_f16(c["outputs_f16_bits"][:15], c["weights"], c["d_model"]) is None


def test_layer_forward_equals_per_token_loop():
    # model.rs:2716-2750 + engine.rs:5575-5581: layer = per-token route, experts, slot-order weighted sum
    rng = np.random.default_rng(3)
    E, D, F, k, B = 8, 64, 96, 2, 5
    gate = oracle.LinearGate(rng.normal(0, 0.02, (E, D)).astype(np.float32), E, D, k)
    blobs = [oracle.randomized_q8_expert(D, F, 100 + e) for e in range(E)]
    x = rng.standard_normal((B, D)).astype(np.float32)
    out, ids, w, gaps = oracle.moe_layer_forward(oracle.Q8_0, gate, blobs, x, F, n_threads=2)
    for t in range(B):
        i2, w2 = gate.route(x[t])
        assert ids[t].tolist() == i2.tolist() and (w[t] == w2).all()
        ys = np.stack([oracle.expert_forward(oracle.Q8_0, blobs[e], x[t], D, F) for e in i2])
        assert (oracle.combine(ys.reshape(-1), w2, skip_zero=True) == out[t]).all()
    assert (gaps > 0).all()
