#!/usr/bin/env python3
"""Writes tests/golden/reference_fixtures.json.

The reference is Rust and cannot be built or imported in this environment, so the
fixtures are the literal inputs and the stated (closed-form) expectations of the
reference's own unit tests, transcribed here.  Where the reference test compares
against its own scalar code instead of a literal, the expectation is recomputed by
the small pure-Python/numpy restatement in THIS file, which shares no code with the
C oracle: agreement of the two is the pin.

Sources (paths relative to rust-engine/src/ of the reference):
  inference.rs:5613-5626   q4_0_non_symmetric_block_matches_ggml_and_candle
  inference.rs:5640-5661   q4_0_writer_emits_exact_ggml_nibble_bytes
  inference.rs:5735-5758, 5789-5805  zero blocks and byte sizes
  q4_parity.rs:451-572     canonical raw Q4_0 cases (+ oracle 591-619, tolerance 26-27)
  q4_parity.rs:574-589     complete-expert input vectors
  kernels/avx2.rs:193-288  Q8_0 row cases
  inference.rs:5905-5926   randomized_q8_expert
  inference.rs:6552-6566   closed-form Q4_0 32x64 expert
  inference.rs:3064-3082   synth_hidden_state
  gating.rs:527-911        router cases
  inference.rs:4628-4705   combine cases;  engine.rs:6579-6588 ordered f16 batch combine

Run:  python tests/golden/make_golden.py
"""
import json
import math
import os

import numpy as np

M64 = (1 << 64) - 1
f32 = np.float32


def f16_bits(v):
    return int(np.float16(v).view(np.uint16))


def f16_val(bits):
    return float(np.uint16(bits).view(np.float16).astype(np.float32))


def q4_block(scale, nibbles):
    b = f16_bits(scale)
    return [b & 0xFF, b >> 8] + [int(n) for n in nibbles]


def q4_dequant(block):
    d = f32(f16_val(block[0] | (block[1] << 8)))
    out = [f32(0)] * 32
    for j in range(16):
        byte = block[2 + j]
        out[j] = d * f32((byte & 15) - 8)
        out[j + 16] = d * f32((byte >> 4) - 8)
    return out


def q8_dequant(block):
    d = f32(f16_val(block[0] | (block[1] << 8)))
    return [d * f32(b - 256 if b > 127 else b) for b in block[2:34]]


def seq_dot(w, x):
    acc = f32(0)
    for a, b in zip(w, x):
        acc = f32(acc + f32(f32(a) * f32(b)))
    return acc


def deterministic_input(n, seed):
    # q4_parity.rs:458-467: multiples of 1/32, exact in f16 and f32
    return [float(((i * (seed * 2 + 3) + seed) % 31) - 15) / 32.0 for i in range(n)]


def xorshift(state):
    state ^= (state << 13) & M64
    state ^= state >> 7
    state ^= (state << 17) & M64
    return state


def synth_hidden_state(token_idx, d_model, seed):
    s = (token_idx * 0x9E3779B97F4A7C15 + seed * 0xBF58476D1CE4E5B9) & M64
    out = []
    for _ in range(d_model):
        s = (s + 0x9E3779B97F4A7C15) & M64
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
        z ^= z >> 31
        u = z >> 40
        out.append(float(f32(f32(u) / f32(1 << 23)) - f32(1.0)))
    return out


def quant_q4(values):
    # inference.rs:797-841
    v = [f32(x) for x in values] + [f32(0)] * (32 - len(values))
    max_abs = f32(max(abs(x) for x in v[:len(values)])) if values else f32(0)
    d = f32(max_abs / f32(7.0))
    blk = q4_block(float(d), [0x88] * 16)
    if d == 0:
        return blk
    inv = f32(f32(1.0) / d)

    def q(x):
        r = float(f32(x * inv))
        r = math.floor(abs(r) + 0.5) * (1 if r >= 0 else -1)  # round half away from zero
        return int(min(15, max(0, r + 8)))
    for j in range(16):
        blk[2 + j] = q(v[j]) | (q(v[j + 16]) << 4)
    return blk


def quant_q8(values):
    # inference.rs:920-957
    n = len(values)
    v = [f32(x) for x in values] + [f32(0)] * (32 - n)
    max_abs = f32(max(abs(x) for x in v[:n])) if n else f32(0)
    d = f32(max_abs / f32(127.0))
    b = f16_bits(float(d))
    blk = [b & 0xFF, b >> 8] + [0] * 32
    if d == 0:
        return blk
    inv = f32(f32(1.0) / d)
    for i in range(32):
        r = float(f32(v[i] * inv))
        r = math.floor(abs(r) + 0.5) * (1 if r >= 0 else -1)
        blk[2 + i] = int(min(127, max(-128, r))) & 0xFF
    return blk


def silu(x):
    x = f32(x)
    return f32(x / f32(f32(1.0) + f32(math.exp(-float(x)))))


def expert_forward_f64(dequant, blob, bb, x, d_model, d_ff):
    """Exact-arithmetic (float64) SwiGLU FFN over a block stream; the reference
    compares fp32 kernels to each other within tolerances, so the fixture keeps the
    high-precision value and the reference's own tolerance."""
    proj = d_model * d_ff // 32 * bb

    def matvec(off, rows, cols, v):
        out = []
        for r in range(rows):
            acc = 0.0
            for b in range(cols // 32):
                s = off + (r * (cols // 32) + b) * bb
                w = dequant(blob[s:s + bb])
                for i in range(32):
                    acc += float(w[i]) * float(v[b * 32 + i])
            out.append(acc)
        return out
    g = matvec(0, d_ff, d_model, x)
    u = matvec(proj, d_ff, d_model, x)
    h = [gi / (1.0 + math.exp(-gi)) * ui for gi, ui in zip(g, u)]
    return matvec(2 * proj, d_model, d_ff, h)


def main():
    fx = {}

    # --- Q4_0 non-symmetric block (inference.rs:5613-5626)
    blk = q4_block(0.5, [j | ((15 - j) << 4) for j in range(16)])
    fx["q4_0_non_symmetric_block"] = {
        "block": blk,
        "expected": [0.5 * (j - 8.0) for j in range(16)] + [0.5 * (7.0 - j) for j in range(16)],
    }

    # --- Q4_0 writer bytes (inference.rs:5640-5661)
    low_q = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 8]
    high_q = [9, 10, 11, 12, 13, 14, 15, 8, 1, 2, 3, 4, 5, 6, 7, 8]
    fx["q4_0_writer"] = {
        "src": [q - 8.0 for q in low_q + high_q],
        "expected_block": [f16_bits(1.0) & 0xFF, f16_bits(1.0) >> 8] + [l | (h << 4) for l, h in zip(low_q, high_q)],
    }

    # --- byte sizes (inference.rs:5748-5758, 5800-5805) and the config shapes
    fx["expert_bytes"] = [
        {"dtype": "q4_0", "d_model": 8, "d_ff": 8, "bytes": 3 * 2 * 18},
        {"dtype": "q4_0", "d_model": 10, "d_ff": 10, "bytes": 3 * 4 * 18},
        {"dtype": "q8_0", "d_model": 8, "d_ff": 8, "bytes": 3 * 2 * 34},
        {"dtype": "q4_0", "d_model": 4096, "d_ff": 14336, "bytes": 99090432},
        {"dtype": "q8_0", "d_model": 2048, "d_ff": 768, "bytes": 5013504},
        {"dtype": "q4_0", "d_model": 7168, "d_ff": 2048, "bytes": 24772608},
    ]

    # --- canonical raw Q4_0 cases (q4_parity.rs:470-572)
    alternating = [0xF0 if i % 2 == 0 else 0x0F for i in range(16)]
    ramp = [i | ((15 - i) << 4) for i in range(16)]
    inverse_ramp = [(15 - i) | (i << 4) for i in range(16)]
    projection_stream = q4_block(0.25, ramp) + q4_block(-0.5, inverse_ramp) + q4_block(0.0, alternating)
    multiple_blocks = q4_block(0.125, alternating) + q4_block(-0.25, ramp)
    multi_row_stream = q4_block(0.0, alternating) + q4_block(0.125, ramp) + q4_block(-0.25, inverse_ramp)
    raw = [
        ("zero-scale-extrema", q4_block(0.0, alternating), 32, 1, 1, 0),
        ("positive-scale-extrema", q4_block(0.25, alternating), 32, 2, 1, 0),
        ("negative-scale-sign", q4_block(-0.5, ramp), 32, 3, 1, 0),
        ("multiple-blocks-nontrivial-hidden", multiple_blocks, 64, 4, 1, 0),
        ("gate-projection-offset-zero", projection_stream, 32, 5, 1, 0),
        ("up-projection-offset-one-unaligned", projection_stream, 32, 6, 1, 1),
        ("down-projection-offset-two", projection_stream, 32, 7, 1, 2),
        ("multi-row-offset-row-stride", multi_row_stream, 32, 8, 2, 1),
    ]
    cases = []
    for name, weights, cols, seed, rows, off in raw:
        x = deterministic_input(cols, seed)
        exp = []
        for r in range(rows):
            acc = f32(0)
            for b in range(cols // 32):
                s = (off + r * (cols // 32) + b) * 18
                w = q4_dequant(weights[s:s + 18])
                for c in range(32):
                    acc = f32(acc + f32(w[c] * f32(x[b * 32 + c])))
            exp.append(float(acc))
        cases.append({"name": name, "weights": weights, "input": x, "rows": rows, "columns": cols,
                      "w_block_off": off, "expected": exp})
    fx["q4_raw_cases"] = {"abs_tol": 1.0e-5, "rel_tol": 1.0e-4, "cases": cases}

    # --- complete-expert inputs (q4_parity.rs:574-589) over the closed-form 32x64 expert (inference.rs:6552-6566)
    d_model, d_ff = 32, 64
    blob = []
    for projection in range(3):
        for block_idx in range(d_model * d_ff // 32):
            w = [(1.0 if (i + block_idx + projection) & 1 == 0 else -1.0)
                 * float(f32(f32((i * 11 + block_idx * 7 + projection * 5) % 17) / f32(20.0))) for i in range(32)]
            blob += quant_q4(w)
    third = []
    for i in range(d_model):
        m = i % 7
        num = 0 if m == 0 else ((i % 13 + 1) if m in (1, 2) else -(i % 11 + 1))
        third.append(num / 64.0)
    inputs = [deterministic_input(d_model, 11), deterministic_input(d_model, 19), third,
              synth_hidden_state(0, d_model, 1)]
    fx["q4_complete_expert"] = {
        "d_model": d_model, "d_ff": d_ff, "blob": blob, "inputs": inputs,
        "expected_f64": [expert_forward_f64(q4_dequant, blob, 18, x, d_model, d_ff) for x in inputs],
        "abs_tol_f16_boundary": 2.0e-3, "rel_tol_f16_boundary": 5.0e-3,
    }
    fx["synth_q4_0_blob"] = {"d_model": 32, "d_ff": 32, "scale": 0.05, "nibble": 9}

    # --- Q8_0 row cases (kernels/avx2.rs:193-288)
    def q8_row(width, case, seed):
        out = []
        state = seed
        for block in range(width // 32):
            if case == 0:
                bits = 0
            elif case == 1:
                bits = 1
            elif case == 2:
                bits = 0x7BFF
            elif case == 6:
                bits = 0x0400
            else:
                bits = f16_bits(float(f32(f32(0.003) + f32(f32(block) * f32(0.00001)))))
            blk = [bits & 0xFF, bits >> 8]
            for i in range(32):
                if case == 3:
                    q = 0
                elif case == 4:
                    q = -128 if (i + block) % 2 == 0 else 127
                elif case == 5:
                    q = -1 if (i + block) % 2 == 0 else 1
                else:
                    state = xorshift(state)
                    q = state & 0xFF
                blk.append(q & 0xFF)
            out += blk
        return out
    rows = []
    for width in (32, 64, 96, 768, 2048):
        x = [float(f32(f32(math.sin(float(f32(f32(i) * f32(0.013))))) * f32(0.01))) for i in range(width)]
        for case in range(7):
            for seed in (1, 0x12345678, 0xFEEDBEEF):
                for s in (seed, seed ^ 0xA5A55A5A):
                    row = q8_row(width, case, s)
                    acc = f32(0)  # q8_scalar order: scale*q*x, left to right (avx2.rs:232-246)
                    for b in range(width // 32):
                        blkb = row[b * 34:(b + 1) * 34]
                        sc = f32(f16_val(blkb[0] | (blkb[1] << 8)))
                        for i in range(32):
                            q = blkb[2 + i]
                            q = q - 256 if q > 127 else q
                            with np.errstate(over="ignore", invalid="ignore"):
                                acc = f32(acc + f32(f32(sc * f32(q)) * f32(x[b * 32 + i])))
                    rows.append({"width": width, "case": case, "seed": s, "expected_scalar": float(acc)})
    fx["q8_row_cases"] = {"abs_tol": 2e-4, "rel_tol": 2e-5, "x_formula": "sin(0.013*i)*0.01 in f32", "rows": rows}

    # --- randomized_q8_expert (inference.rs:5905-5926) at the tiny shapes; f64 expectation
    def randomized_q8_expert(dm, df, state):
        weights = dm * df
        blocks = -(-weights // 32)
        out = []
        for projection in range(3):
            for block in range(blocks):
                count = min(32, weights - block * 32)
                vals = []
                for _ in range(count):
                    state = xorshift(state)
                    unit = f32(f32(f32(state >> 40) / f32((1 << 24) - 1)) - f32(0.5))
                    vals.append(float(f32(unit * f32(f32(0.08) + f32(f32(projection) * f32(0.01))))))
                out += quant_q8(vals)
        return out
    q8_cases = []
    for dm, df, st, tok, seed in ((32, 32, 0x51A1A11E, 9, 3), (128, 96, 128 ^ 96, 19, 7)):
        blob8 = randomized_q8_expert(dm, df, st)
        x = synth_hidden_state(tok, dm, seed)
        q8_cases.append({"d_model": dm, "d_ff": df, "state": st, "token": tok, "seed": seed,
                         "blob_head": blob8[:68], "blob_len": len(blob8), "blob_sum": int(sum(blob8)),
                         "expected_f64": expert_forward_f64(q8_dequant, blob8, 34, x, dm, df)})
    fx["randomized_q8_expert"] = {"rel_tol": 3e-3, "abs_tol": 3e-5, "cases": q8_cases,
                                  "unaligned_shapes": [[37, 45], [64, 45], [37, 64]]}

    # --- synth_hidden_state (inference.rs:3064-3082)
    fx["synth_hidden_state"] = [{"token": t, "d_model": d, "seed": s, "values": synth_hidden_state(t, d, s)}
                                for t, d, s in ((0, 8, 1), (9, 37, 3), (19, 64, 7), (123456789, 16, 0xDEADBEEF))]

    # --- router (gating.rs:527-911); identity gate => logit[i] = x[i]
    def ident(n):
        return [1.0 if i == j else 0.0 for i in range(n) for j in range(n)]

    def sig(v):
        return 1.0 / (1.0 + math.exp(-v))
    r = []
    r.append({"name": "picks_largest_logit_first", "weights": [float(i + 1) for i in range(4) for _ in range(3)],
              "num_experts": 4, "d_model": 3, "top_k": 2, "x": [1.0, 1.0, 1.0],
              "experts": [3, 2], "weight_sum": 1.0, "descending": True})
    r.append({"name": "top_k_equals_num_experts", "weights": [0.0] * 8, "num_experts": 4, "d_model": 2, "top_k": 4,
              "x": [0.0, 0.0], "experts": [0, 1, 2, 3], "weights_expected": [0.25] * 4, "tol": 1e-5})
    r.append({"name": "sigmoid_unnormalised", "weights": ident(4), "num_experts": 4, "d_model": 4, "top_k": 2,
              "scoring": "sigmoid", "normalise_topk": False, "x": [2.0, 1.0, -5.0, -5.0],
              "experts": [0, 1], "weights_expected": [0.880797, 0.731058], "tol": 1e-4})
    r.append({"name": "correction_bias_selection_only", "weights": ident(4), "num_experts": 4, "d_model": 4, "top_k": 1,
              "scoring": "sigmoid", "normalise_topk": False, "correction_bias": [0.0, 0.0, 0.0, 10.0],
              "x": [3.0, 0.0, 0.0, 1.0], "experts": [3], "weights_expected": [0.731058], "tol": 1e-4})
    r.append({"name": "grouped_topk", "weights": ident(8), "num_experts": 8, "d_model": 8, "top_k": 2,
              "scoring": "sigmoid", "normalise_topk": False, "n_group": 2, "topk_group": 1,
              "x": [3.0, -9.0, -9.0, -9.0, 4.0, 5.0, -9.0, -9.0], "experts": [5, 4],
              "weights_expected": [sig(5.0), sig(4.0)], "tol": 1e-5})
    r.append({"name": "routed_scaling", "weights": ident(4), "num_experts": 4, "d_model": 4, "top_k": 2,
              "scoring": "sigmoid", "normalise_topk": True, "routed_scaling_factor": 2.5,
              "x": [2.0, 1.0, -5.0, -5.0], "experts": [0, 1], "weight_sum": 2.5, "tol": 1e-4})
    r.append({"name": "ties_lower_id", "weights": [0.0] * 12, "num_experts": 6, "d_model": 2, "top_k": 4,
              "x": [1.0, -1.0], "experts": [0, 1, 2, 3], "weights_expected": [0.25] * 4, "tol": 1e-6})
    r.append({"name": "softmax_default", "weights": ident(4), "num_experts": 4, "d_model": 4, "top_k": 2,
              "x": [5.0, 4.0, 0.0, 0.0], "experts": [0, 1], "weight_sum": 1.0, "tol": 1e-5})
    # scratch_route_matches_stable_reference_across_routing_modes (gating.rs:788-836): expectation = stable sort
    sm = [0.5, 2.0, 2.0, -1.0, 3.0, 0.0, 3.0, -2.0]
    e = [math.exp(v - 3.0) for v in sm]
    tot = e[4] + e[6] + e[1]
    r.append({"name": "modes_softmax", "weights": ident(8), "num_experts": 8, "d_model": 8, "top_k": 3, "x": sm,
              "experts": [4, 6, 1], "weights_expected": [e[4] / tot, e[6] / tot, e[1] / tot], "tol": 1e-6,
              "compare_stable": True})
    xb = [3.0, -1.0, 1.0, 2.0, 4.0, 5.0, 0.5, -9.0]
    bias = [0.0, 0.0, 0.0, 0.0, 0.1, 0.0, 1.25, 0.0]
    # groups {0..3},{4..7}; group scores (top-2 of score+bias): g0 = s(3)+s(2); g1 = (s(.5)+1.25)+(s(4)+.1) -> g1 wins
    sel = {i: sig(xb[i]) + bias[i] for i in range(4, 8)}
    order = sorted(sel, key=lambda i: (-sel[i], i))[:3]
    ws = [sig(xb[i]) for i in order]
    r.append({"name": "modes_biased_group", "weights": ident(8), "num_experts": 8, "d_model": 8, "top_k": 3,
              "scoring": "sigmoid", "normalise_topk": True, "correction_bias": bias, "n_group": 2, "topk_group": 1,
              "routed_scaling_factor": 1.5, "x": xb, "experts": order,
              "weights_expected": [w / sum(ws) * 1.5 for w in ws], "tol": 1e-6, "compare_stable": True})
    xs = [-2.0, 4.0, 1.0, 4.0, 0.5, -3.0, 0.0, 2.0]
    r.append({"name": "modes_sigmoid", "weights": ident(8), "num_experts": 8, "d_model": 8, "top_k": 4,
              "scoring": "sigmoid", "normalise_topk": False, "x": xs, "experts": [1, 3, 7, 2],
              "weights_expected": [sig(4.0), sig(4.0), sig(2.0), sig(1.0)], "tol": 1e-6, "compare_stable": True})
    fx["router_cases"] = r

    # --- combine (inference.rs:4628-4705) and the ordered f16 batch KAT (engine.rs:6579-6588)
    fx["combine_cases"] = [
        {"outputs": [[1.0, 2.0, 3.0], [3.0, 2.0, 1.0]], "scores": [0.5, 0.5], "expected": [2.0, 2.0, 2.0], "tol": 0.0},
        {"outputs": [[1.0] * 4, [2.0] * 4, [4.0] * 4], "scores": [0.5, 0.25, 0.25], "expected": [2.0] * 4, "tol": 1e-6},
        {"outputs": [], "scores": [], "expected": [], "tol": 0.0},
    ]
    fx["ordered_f16_batch"] = {"outputs_f16_bits": [f16_bits(v / 4.0) for v in range(16)], "d_model": 2,
                               "weights": [0.5, 0.0, -0.25, 1.0, 0.125, -0.5, 0.25, 0.75],
                               "expected": [3.625, 4.09375]}

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixtures.json")
    with open(path, "w") as f:
        json.dump(fx, f, separators=(",", ":"))
        f.write("\n")
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
