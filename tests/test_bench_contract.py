"""The benchmark's reference arm runs on CPU: one JSON line on stdout with the agreed keys."""
import json
import os
import subprocess
import sys


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1",
                        "--cpu-seconds", "0.5"], cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout[-2000:]
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert "workload" in d["config"] and "model" not in d["config"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_calibration_counts_follow_the_oracles_selection():
    """The benchmark places experts by a numpy restatement of the routing's selection step; on a small group-limited
    sigmoid configuration and on a softmax one its per-expert token counts must equal the oracle's."""
    import importlib
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import bench
    import oracle
    oracle.build()
    synth = importlib.import_module("mer_b200.synth")
    for scoring, n_group, topk_group in ((1, 4, 2), (0, 1, 1)):
        cfg = synth.MoeShape("calib-test", oracle.Q8_0, 256, 256, 32, 4, seed=3, scoring=scoring, n_group=n_group,
                             topk_group=topk_group, scaling=1.0, shared=False, layers=1)
        n = 96
        counts = bench.calibration_counts(synth, cfg, 0, 1.0, 1.0, n_tokens=n)
        gate = bench.oracle_gate(oracle, synth, cfg, 0, 1.0, 1.0)
        x = synth.make_activations(n, cfg.d_model, cfg.seed, 7000)
        ref = np.zeros(cfg.num_experts, np.int64)
        for t in range(n):
            for e in gate.route(x[t])[0]:
                ref[int(e)] += 1
        assert counts.sum() == n * cfg.top_k
        assert np.abs(counts - ref).sum() <= 2, (counts, ref)  # a tie within fp32 noise may move one pair
