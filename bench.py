#!/usr/bin/env python3
"""Benchmark of the routed quantized SwiGLU expert-FFN path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload cfgN] [--batch B] [--layers L]

The default workload is the largest configuration that fits one GPU and the only one defined at 1 / 2 / 4 / 8
GPUs: the Qwen3-30B-A3B-shaped Q8_0 prefill (48 MoE layers x 128 experts resident, 30.8 GB; a 2048-token batch,
top-8, Zipf(s=1.0) logit bias).  A STEP is the token batch through every resident layer once (router top-k ->
permute -> gate/up + SiLU*mul -> down -> weighted combine, L times); `value` counts tokens x layers per second,
i.e. tokens/s through one MoE layer.  At N > 1 the global batch stays 2048 tokens and every rank holds 128/N
experts of each layer (strong scaling).  Prints ONE JSON line (rank 0).

  value      inputs already in HBM (device pointers), CUDA events around exactly K steps, max over ranks
  e2e        the same steps through the host-buffer entry points: pinned host rows uploaded and results read back
             inside the timed region (pipelined: three calls in flight); e2e_sync = the synchronous host call
  roofline   dominant kernel (the gate/up launch): algorithmic FLOPs or bytes / its CUDA-event time against the
             measured peak (MEASURED_PEAKS.json)
  parity     rank 0 recomputes a few of its tokens with the CPU oracle outside the timed region; the run fails
             when routing or outputs differ beyond the stated bar or a device status bit is latched
  sweep      (N = 1) the other configurations at their stated decode batches, measured the same way
  cpu_baseline  the CPU restatement of the reference's path on this host's cores (rank 0, N = 1)

`--impl reference` times the CPU path only (the reference itself is Rust and cannot be built here; the oracle
port stands in for it).
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {  # name -> (config, default batch, default resident layers, Zipf s or None)
    "cfg0": ("cfg0-mixtral-q4_0", 1, 8, None),
    "cfg1": ("cfg1-qwen3-q8_0", 64, 8, None),
    "cfg2": ("cfg2-mixtral-stack-q4_0", 16, 32, 1.1),
    "cfg3": ("cfg3-qwen3-prefill-q8_0", 2048, 48, 1.0),
    "cfg4": ("cfg4-deepseek-v3-q4_0", 16, 1, None),
}
SWEEP = [  # (workload, batches) measured after the headline at N = 1; cfg1 / cfg0 reuse the resident cfg3 / cfg2 stacks
    ("cfg1", (1, 8, 64)),
    ("cfg2", (1, 4, 16, 64, 256)),
    ("cfg0", (1, 16)),
    ("cfg4", (16,)),
]
DTYPE_NAME = {0: "q4_0", 1: "q8_0"}
GEMM_MEAN_TOKENS = 12  # mean tokens per expert from which the library's automatic selection runs the tcgen05 GEMM kernels
PARITY_TOKENS = 4
PARITY_BAR = 1e-3      # max-abs error of a token's output relative to the RMS of the oracle's output
PARALLELISM_NOTE = {
    "replicas": "{n} replicas, tokens data-parallel, no data-path collective",
    "ep-peer": "expert-parallel over {n} GPUs ({e} experts per GPU and layer, {placement}; tokens data-parallel), dispatch and combine by the "
               "library's kernels through peer memory over NVLink",
    "ep-collective": "expert-parallel over {n} GPUs ({e} experts per GPU and layer, {placement}; tokens data-parallel), NCCL all-gather of "
                     "tokens+routing and reduce-scatter of partial outputs",
    "ep-nccl": "expert-parallel over {n} GPUs ({e} experts per GPU and layer, {placement}; tokens data-parallel), NCCL all-to-all dispatch and "
               "combine issued by the library (grouped ncclSend / ncclRecv of the rows that hit a peer's experts)",
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="tokens per step over all GPUs (cfg3) or per GPU (other workloads)")
    ap.add_argument("--layers", type=int, default=0, help="resident layers a step runs through (default: the whole stack)")
    ap.add_argument("--kernel-path", type=int, default=0, help="0 auto, 1 generic, 2 streaming, 3 GEMM")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="bound on the CPU baseline leg")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--zipf-strength", type=float, default=1.0)
    ap.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                    help="expert-parallel modes: experts placed by the token counts of a calibration batch (greedy, the same "
                         "number of experts on every GPU), or rank j holds experts [j*E/N, (j+1)*E/N)")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "replicas", "ep-peer", "ep-collective", "ep-nccl"],
                    help="N > 1: expert-parallel with the exchange through peer memory (default) or through NCCL "
                         "collectives, or independent token-parallel replicas")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the GPU is busy."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        pw = [float(r[2]) for r in self.rows if len(r) >= 7 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        busy = [s for s, p in zip(sm, pw) if p >= 0.5 * max(pw)] if pw else sm  # samples taken under load
        return {"sm_mhz": statistics.median(busy or sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "power_w_max": max(pw) if pw else None, "reasons": reasons}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return 6650.0, 1590.0, 1400.0, "fallback"


def ncu_traffic(key):
    """Per-launch DRAM traffic of the dominant kernel from the committed ncu summary, if one covers this workload."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return json.load(f).get(key)
    except Exception:
        return None


def zipf_bias(synth, cfg, zipf_s, layer, strength):
    return None if zipf_s is None else synth.zipf_logit_bias(cfg.num_experts, zipf_s, cfg.seed, layer, strength=strength)


def calibration_counts(synth, cfg, layer, zipf_s, strength, n_tokens=2048):
    """Tokens per routed expert of a calibration batch (its own seed, not a batch the benchmark times), by a numpy
    restatement of the selection: enough to rank the experts by popularity, no parity claim."""
    E, k = cfg.num_experts, cfg.top_k
    x = synth.make_activations(n_tokens, cfg.d_model, cfg.seed, 7000 + layer)
    logits = x @ synth.make_router(E, cfg.d_model, cfg.seed, layer).T
    bias = zipf_bias(synth, cfg, zipf_s, layer, strength)
    if bias is not None:
        logits = logits + bias
    sel = 1.0 / (1.0 + np.exp(-logits)) if cfg.scoring == 1 else logits  # softmax keeps the order of the logits
    if cfg.n_group > 1 and 0 < cfg.topk_group < cfg.n_group:
        g = sel.reshape(n_tokens, cfg.n_group, E // cfg.n_group)
        gscore = np.sort(g, axis=2)[:, :, -2:].sum(axis=2)
        keep = np.argsort(-gscore, axis=1)[:, :cfg.topk_group]
        mask = np.zeros((n_tokens, cfg.n_group), bool)
        np.put_along_axis(mask, keep, True, axis=1)
        sel = np.where(np.repeat(mask, E // cfg.n_group, axis=1), sel, -np.inf)
    top = np.argpartition(-sel, k - 1, axis=1)[:, :k]
    return np.bincount(top.ravel(), minlength=E)


def ep_placement(epm, synth, cfg, n_layers, zipf_s, strength, rank, world, policy):
    """(owner table by global expert id or None, this rank's local expert indices per layer)."""
    E = cfg.num_experts
    if policy == "contiguous":
        mine = list(epm.local_expert_range(rank, world, E))
        return None, [mine] * n_layers
    owner = np.zeros(n_layers * E, np.uint16)
    mine = []
    for l in range(n_layers):
        o = epm.balanced_placement(calibration_counts(synth, cfg, l, zipf_s, strength), world)
        owner[l * E:(l + 1) * E] = o
        mine.append([e for e in range(E) if o[e] == rank])
    return owner, mine


def host_blobs(synth, cfg, layer, experts, threads):
    """Expert blobs of one layer on the host (numpy generator), generated by a pool of threads."""
    with ThreadPoolExecutor(max_workers=max(1, threads)) as pool:
        return dict(zip(experts, pool.map(lambda e: synth.make_expert_blob(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, layer, e),
                                          experts)))


def oracle_gate(oracle, synth, cfg, layer, zipf_s, strength):
    W = synth.make_router(cfg.num_experts, cfg.d_model, cfg.seed, layer)
    return oracle.LinearGate(W, cfg.num_experts, cfg.d_model, cfg.top_k, scoring_func=cfg.scoring, n_group=cfg.n_group,
                             topk_group=cfg.topk_group, routed_scaling_factor=cfg.scaling,
                             logit_bias=zipf_bias(synth, cfg, zipf_s, layer, strength))


def parity_check(oracle, synth, cfg, layer, zipf_s, strength, x_rows, got_rows, got_ids, threads):
    """Recomputes the given token rows of `layer` with the CPU oracle.  Returns the `parity` object; raises SystemExit
    when routing differs on a token that is not tie-ambiguous or an output exceeds the bar."""
    gate = oracle_gate(oracle, synth, cfg, layer, zipf_s, strength)
    routed = [gate.route(x, detail=True) for x in x_rows]
    need = sorted({int(e) for ids, _, _, _ in routed for e in ids})
    blobs = host_blobs(synth, cfg, layer, need + ([cfg.num_experts] if cfg.shared else []), threads)
    filler = np.zeros(synth.expert_bytes(cfg.dtype, cfg.d_model, cfg.d_ff), np.uint8)  # experts no checked token is routed to
    blob_list = [blobs.get(e, filler) for e in range(cfg.num_experts)]
    ref, rids, _, gaps = oracle.moe_layer_forward(cfg.dtype, gate, blob_list, np.stack(x_rows), cfg.d_ff,
                                                  shared_blob=blobs.get(cfg.num_experts) if cfg.shared else None, n_threads=threads)
    worst, identical, checked = 0.0, True, 0
    for t in range(len(x_rows)):
        ids, _, scores, gap = routed[t]
        sel = np.sort(scores[ids])
        if gap < 1e-6 * float(np.abs(sel).max()) or (np.diff(sel) < 1e-6 * np.abs(sel[1:])).any():
            continue  # scores tie within the logit summation noise: the choice or its order is ambiguous, not wrong
        checked += 1
        if got_ids is not None and [int(v) for v in got_ids[t]] != [int(v) for v in rids[t]]:
            identical = False
        rms = float(np.sqrt(np.mean(ref[t].astype(np.float64) ** 2))) + 1e-30
        worst = max(worst, float(np.abs(got_rows[t].astype(np.float64) - ref[t]).max()) / rms)
    par = {"tokens": checked, "max_rel_rms": worst, "topk_identical": identical, "bar": PARITY_BAR, "layer": layer}
    if checked == 0 or not identical or not (worst <= PARITY_BAR):
        raise SystemExit(f"bench.py: parity check against the CPU oracle failed: {par}")
    return par


def cpu_rate(oracle, synth, cfg, layer, zipf_s, strength, x, threads, seconds, steps=None, warmup=1):
    """tokens/s of the CPU path on (a bounded sample of) one layer pass of the step."""
    experts = list(range(cfg.num_experts + (1 if cfg.shared else 0)))
    blobs = host_blobs(synth, cfg, layer, experts, threads)
    gate = oracle_gate(oracle, synth, cfg, layer, zipf_s, strength)
    blob_list = [blobs[e] for e in range(cfg.num_experts)]
    shared = blobs.get(cfg.num_experts) if cfg.shared else None
    run = lambda rows: oracle.moe_layer_forward_production(cfg.dtype, gate, blob_list, rows, cfg.d_ff, threads, shared_blob=shared)
    t0 = time.perf_counter()
    run(x[:1])
    per_token = time.perf_counter() - t0
    n_tok = int(max(1, min(x.shape[0], seconds / 4 / max(per_token, 1e-6))))
    sample = x[:n_tok]
    for _ in range(warmup):
        run(sample)
    reps, t0 = 0, time.perf_counter()
    while True:
        run(sample)
        reps += 1
        el = time.perf_counter() - t0
        if (steps is not None and reps >= steps) or (steps is None and (el > seconds / 2 or reps >= 50)):
            break
    return n_tok * reps / el, el / reps * 1e3, f"{n_tok} of {x.shape[0]} tokens of one layer pass, {reps} repetitions, {threads} threads"


class Stack:
    """A resident stack of MoE layers of one configuration on one backend."""

    def __init__(self, mer_b200, synth, cfg, n_layers, max_tokens, device_index, mine=None, rank_tokens=None):
        import torch
        self.mer, self.synth, self.cfg, self.L = mer_b200, synth, cfg, n_layers
        self.torch, self.dev = torch, torch.device("cuda", device_index)
        # the routed experts this backend holds: all, one list for every layer, or one list per layer
        if mine is None:
            mine = list(range(cfg.num_experts))
        self.mine = [list(m) for m in mine] if len(mine) and isinstance(mine[0], (list, tuple, range)) else [list(mine)] * n_layers
        self.slots = cfg.top_k + (1 if cfg.shared else 0)
        self.exp_bytes = mer_b200.expert_bytes(cfg.dtype, cfg.d_model, cfg.d_ff)
        stride = (256 + self.exp_bytes + 4095) // 4096 * 4096
        n_slots = sum(len(m) for m in self.mine) + (n_layers if cfg.shared else 0)
        self.be = mer_b200.Backend(cfg.dtype, cfg.d_model, cfg.d_ff, stride * n_slots,
                                   (n_layers + 1) * cfg.num_experts + n_layers, max_tokens=max_tokens, max_top_k=self.slots,
                                   device=device_index)
        self.resident_bytes = self.exp_bytes * n_slots
        # fill the slots: every layer's experts are generated in device memory (seed = the configuration's, layer = its index)
        chunk = max(1, int((1 << 30) // (self.exp_bytes * 10)))  # the generator's 64-bit temporaries are ~10x the blob
        for l in range(n_layers):
            todo = [(e, l * cfg.num_experts + e) for e in self.mine[l]]
            if cfg.shared:
                todo.append((cfg.num_experts, n_layers * cfg.num_experts + l))
            for i in range(0, len(todo), chunk):
                part = todo[i:i + chunk]
                blobs = synth.make_expert_blobs_torch(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, l, [e for e, _ in part], self.dev)
                torch.cuda.synchronize()  # the admission runs on the library's copy stream: the bytes must be there first
                for j, (_, gid) in enumerate(part):
                    self.be.admit_device(gid, 1, blobs[j].data_ptr(), self.exp_bytes, wait=False)
                self.be.synchronize()  # the admission reads the generator's tensor: keep it alive until the copy stream is done
                del blobs

    def install_routers(self, zipf_s, strength):
        m = self.mer
        for l in range(self.L):
            cfg = self.cfg
            gate = m.LinearGate.with_routing(self.synth.make_router(cfg.num_experts, cfg.d_model, cfg.seed, l), cfg.num_experts,
                                             cfg.d_model, cfg.top_k, cfg.scoring, True, None, cfg.n_group, cfg.topk_group, cfg.scaling)
            gate.logit_bias = zipf_bias(self.synth, cfg, zipf_s, l, strength)
            self.be.install_router(l, gate, self.L * cfg.num_experts + l if cfg.shared else 0xFFFFFFFF)

    def close(self):
        self.be.close()


def cuda_time_ms(torch, fn):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def measure_point(stack, name, zipf_s, B, layers, passes, warm, peaks, x_seed_base=0):
    """One single-GPU measurement: `passes` layer passes of a B-token batch rotating over `layers` resident layers.
    Returns (entry dict, per-layer hit-expert bytes)."""
    torch, be, cfg, synth = stack.torch, stack.be, stack.cfg, stack.synth
    hbm_peak, tf_burst, tf_sustained, kind = peaks
    xs_host = [synth.make_activations(B, cfg.d_model, cfg.seed, x_seed_base + i) for i in range(min(len(layers), 8))]
    xs = [torch.from_numpy(x).to(stack.dev) for x in xs_host]
    out = torch.empty(B, cfg.d_model, device=stack.dev)
    stream = torch.cuda.current_stream().cuda_stream
    hit = []
    for i, l in enumerate(layers):
        _, ids, _ = be.moe_layer_forward(l, xs_host[i % len(xs)])
        hit.append((len(np.unique(ids[ids != 0xFFFFFFFF])) + (1 if cfg.shared else 0)) * stack.exp_bytes)

    def run(n):
        for i in range(n):
            be.moe_layer_forward_device(layers[i % len(layers)], xs[(i % len(layers)) % len(xs)].data_ptr(), B, out.data_ptr(), stream)

    run(max(warm, 3))
    ms = cuda_time_ms(torch, lambda: run(passes))
    be.stream_check(layers[0], stream)
    n_t = min(passes, 2048)
    be.stage_timing_enable(True)
    run(n_t)
    torch.cuda.synchronize()
    st = be.stage_timings()
    be.stage_timing_enable(False)
    n = max(st["samples"], 1)
    gu_ms, dn_ms = st["expert_gate_up_kernel_ms"] / n, st["expert_down_kernel_ms"] / n
    mean_hit = sum(hit[i % len(layers)] for i in range(passes)) / passes
    layer_bytes = mean_hit + cfg.num_experts * cfg.d_model * 4 + 2 * B * cfg.d_model * 4 + B * cfg.top_k * 8
    per_layer_ms = ms / passes
    gemm = B * stack.slots >= GEMM_MEAN_TOKENS * (cfg.num_experts + (1 if cfg.shared else 0))
    if gemm:
        flops = 2.0 * B * stack.slots * 2 * cfg.d_model * cfg.d_ff
        tf = flops / (gu_ms * 1e-3) / 1e12 if gu_ms > 0 else None
        roof = {"bound": "tensor", "kernel": "expert_gate_up (grouped dequant GEMM, tcgen05, + SiLU*mul)", "achieved": tf, "peak": tf_burst,
                "unit": "TFLOP/s", "frac": tf / tf_burst if tf else None, "peak_source": f"of {kind} (burst)",
                "frac_of_sustained_peak": tf / tf_sustained if tf else None, "algorithmic_flops_per_launch": flops, "avg_launch_ms": gu_ms}
    else:
        fused = dn_ms == 0.0
        kb = (mean_hit if fused else mean_hit * 2 / 3) + B * cfg.d_model * 4
        ach = kb / (gu_ms * 1e-3) / 1e9 if gu_ms > 0 else None
        roof = {"bound": "hbm", "kernel": "expert_gate_up (gate/up dequant-matvec + SiLU*mul)", "achieved": ach, "peak": hbm_peak,
                "unit": "GB/s", "frac": ach / hbm_peak if ach else None, "peak_source": f"of {kind}",
                "frac_of_8tbs": ach / 8000.0 if ach else None, "algorithmic_bytes_per_launch": kb, "avg_launch_ms": gu_ms}
    layer_gbs = layer_bytes / (per_layer_ms * 1e-3) / 1e9
    entry = {"workload": name, "batch": B, "layers_rotated": len(layers), "passes": passes, "tokens_per_s": B / (per_layer_ms * 1e-3),
             "ms_per_layer": per_layer_ms, "roofline": roof,
             "hbm": {"layer_algorithmic_bytes": layer_bytes, "achieved_gbs": layer_gbs, "frac_of_measured": layer_gbs / hbm_peak,
                     "frac_of_8tbs": layer_gbs / 8000.0},
             "stage_ms": {k: v / n for k, v in st.items() if k != "samples"}}
    return entry, xs_host, xs, out


def run_vram_tier(mer_b200, synth, oracle, args, local_rank, threads, n_layers=8, slots_fraction=0.5, B=16, steps=160):
    """The VRAM tier under miss traffic: a Mixtral-shaped stack whose experts do not all fit the slot arena.  The
    expert payloads sit in pinned host memory; a step is one layer pass of B tokens whose routing (Zipf-skewed) was
    computed beforehand, like the expert-id trace the reference's `run` replays (workload.rs:60-140).  Before layer
    i is enqueued, the experts layer i + 1 needs are looked up in the logical tier (GpuExpertCache semantics: LRU
    Edge demand admission, threshold promotion into the Anchor Core) and the missing ones are admitted on the copy
    stream, so their H2D copies overlap layer i's kernels.  Reported: steps/s against the all-resident rate, the miss
    rate, the H2D rate, and parity of a sampled step."""
    import torch
    cfg = synth.CONFIGS[WORKLOADS["cfg2"][0]]
    E, D, F = cfg.num_experts, cfg.d_model, cfg.d_ff
    eb = mer_b200.expert_bytes(cfg.dtype, D, F)
    stride = (256 + eb + 4095) // 4096 * 4096
    n_exp = n_layers * E
    n_slots = max(4, int(n_exp * slots_fraction))
    dev = torch.device("cuda", local_rank)
    host = torch.empty((n_exp, eb), dtype=torch.uint8).pin_memory()  # the RAM tier: every expert's payload, pinned
    for l in range(n_layers):
        host[l * E:(l + 1) * E].copy_(synth.make_expert_blobs_torch(cfg.dtype, D, F, cfg.seed, l, list(range(E)), dev))
    torch.cuda.synchronize()
    host_np = host.numpy()
    be = mer_b200.Backend(cfg.dtype, D, F, stride * n_slots, n_exp, max_tokens=B, max_top_k=cfg.top_k, device=local_rank)
    cache = mer_b200.GpuExpertCache(n_slots * eb, 0.5, 16)  # anchor_ratio and promote_after_hits of `run --gpu` (main.rs:2190-2194)
    for l in range(n_layers):
        gate = mer_b200.LinearGate(synth.make_router(E, D, cfg.seed, l), E, D, cfg.top_k)
        gate.logit_bias = zipf_bias(synth, cfg, WORKLOADS["cfg2"][3], l, args.zipf_strength)
        be.install_router(l, gate)
    xs_host = [synth.make_activations(B, D, cfg.seed, 500 + i) for i in range(16)]
    xs = [torch.from_numpy(x).to(dev) for x in xs_host]
    out = torch.empty(B, D, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    # the trace: which experts every step needs (routing needs no resident expert)
    order = [(i * 5) % n_layers for i in range(steps)]  # layers in a scattered order: consecutive steps share no expert
    need = []
    for i, l in enumerate(order):
        ids, _ = be.route(l, xs_host[i % len(xs)])
        need.append(sorted({int(v) + l * E for v in ids.reshape(-1) if v != 0xFFFFFFFF}))
    ram_hits = {}
    stats = {"admissions": 0, "lookups": 0}

    def ensure(i):
        """Foreground demand for step i (engine.rs:2382-2429): lookup, admit what is missing, promote what got hot."""
        for gid in need[i]:
            stats["lookups"] += 1
            kind, _ = cache.get(gid)
            ram_hits[gid] = ram_hits.get(gid, 0) + 1
            if kind == mer_b200.GpuLookup.Miss:
                be.demand_admit(cache, gid, host_np[gid], wait=False, reader_wait=False)
                stats["admissions"] += 1
            elif not be.contains_generation(gid, cache.current_generation(gid)):
                be.demand_admit(cache, gid, host_np[gid], wait=False, reader_wait=False)  # admitted logically, evicted physically
                stats["admissions"] += 1
            if cache.claim_promotion(gid, ram_hits[gid]):
                be.hot_promote(cache, gid, host_np[gid], wait=False, reader_wait=False)

    def run(n, check_step=None):
        ensure(0)
        got = None
        for i in range(n):
            be.moe_layer_forward_device(order[i], xs[i % len(xs)].data_ptr(), B, out.data_ptr(), stream)
            if i + 1 < n:
                # the next step's admissions ride the copy stream while this step's kernels run: the victims they evict are
                # the least recently looked-up experts, this step's experts the most recent, so no slot this step reads is
                # rewritten and the copies need not wait for it (MER_ADMIT_NO_READER_WAIT)
                ensure(i + 1)
            if check_step == i:
                be.stream_check(order[i], stream)
                got = out.cpu().numpy().copy()
        be.stream_check(order[0], stream)
        return got

    run(min(steps, 2 * n_layers))  # warm: fills the arena, builds the graphs
    m0, a0, l0 = cache.misses(), stats["admissions"], stats["lookups"]
    up0 = be.snapshot()["expert_upload_bytes"]
    t0 = time.perf_counter()
    ms = cuda_time_ms(torch, lambda: run(steps))
    wall = time.perf_counter() - t0
    snap = be.snapshot()
    misses, lookups = cache.misses() - m0, stats["lookups"] - l0
    uploaded = snap["expert_upload_bytes"] - up0
    # parity of one step that ran with admissions in flight
    probe = steps // 2
    got = run(probe + 1, check_step=probe)
    lp = order[probe]
    gate = oracle_gate(oracle, synth, cfg, lp, WORKLOADS["cfg2"][3], args.zipf_strength)
    xr = xs_host[probe % len(xs)][:2]
    ref, _, _, _ = oracle.moe_layer_forward(cfg.dtype, gate, [host_np[lp * E + e] for e in range(E)], xr, F, n_threads=threads)
    worst = max(float(np.abs(got[t].astype(np.float64) - ref[t]).max() / (np.sqrt(np.mean(ref[t].astype(np.float64) ** 2)) + 1e-30))
                for t in range(2))
    par = {"tokens": 2, "max_rel_rms": worst, "bar": PARITY_BAR, "layer": lp}
    if not worst <= PARITY_BAR:
        raise SystemExit(f"bench.py: VRAM-tier step differs from the CPU oracle: {par}")
    cs = cache.stats()
    entry = {"workload": f"{cfg.name} VRAM tier under miss traffic: {n_layers} layers x {E} experts in pinned RAM, {n_slots} HBM slots "
                         f"({slots_fraction:.0%} of the stack), decode batch {B}, admissions overlap the previous step's kernels",
             "batch": B, "steps": steps, "steps_per_s": steps / (ms * 1e-3), "tokens_per_s": B * steps / (ms * 1e-3), "ms_per_step": ms / steps,
             "wall_ms_per_step": wall * 1e3 / steps, "miss_rate": misses / max(lookups, 1), "expert_admissions": stats["admissions"] - a0,
             "h2d_gbs": uploaded / (ms * 1e-3) / 1e9, "h2d_bytes": uploaded, "evictions": snap["evictions"],
             "logical_tier": {k: cs[k] for k in ("anchor_len", "lru_len", "promotions", "hits", "misses")}, "parity": par}
    be.close()
    del host
    return entry


def run_sweep(mer_b200, synth, oracle, args, qwen_stack, local_rank, peaks, threads):
    """The other configurations at their stated decode batches.  cfg1 runs on the resident Qwen3 stack (same shapes
    and seed as cfg3), cfg0 on the Mixtral stack of cfg2."""
    import torch
    entries = []

    def point(stack, wl, zipf_s, B, n_rot):
        cfg_name = WORKLOADS[wl][0]
        layers = list(range(min(stack.L, n_rot)))
        target_s = 0.15
        probe, *_ = measure_point(stack, cfg_name, zipf_s, B, layers, 16, 3, peaks)
        passes = int(min(4000, max(32, target_s / (probe["ms_per_layer"] * 1e-3))))
        entry, xs_host, xs, out = measure_point(stack, cfg_name, zipf_s, B, layers, passes, 3, peaks)
        # parity of this point: a few tokens of the first rotated layer against the oracle
        stream = torch.cuda.current_stream().cuda_stream
        ids_dev = torch.empty(B, stack.slots, dtype=torch.int32, device=stack.dev)
        stack.be.moe_layer_forward_device(layers[0], xs[0].data_ptr(), B, out.data_ptr(), stream, d_ids=ids_dev.data_ptr())
        stack.be.stream_check(layers[0], stream)
        n = min(PARITY_TOKENS, B)
        got = out[:n].cpu().numpy()
        gids = ids_dev[:n, :stack.cfg.top_k].cpu().numpy().astype(np.int64) - layers[0] * stack.cfg.num_experts
        entry["parity"] = parity_check(oracle, synth, stack.cfg, layers[0], zipf_s, args.zipf_strength, list(xs_host[0][:n]), got, gids,
                                       threads)
        entries.append(entry)

    if qwen_stack is not None:
        qwen_stack.install_routers(None, 0.0)
        for B in dict(SWEEP)["cfg1"]:
            point(qwen_stack, "cfg1", None, B, 8)
        qwen_stack.close()
    torch.cuda.empty_cache()
    cfg2 = synth.CONFIGS[WORKLOADS["cfg2"][0]]
    st = Stack(mer_b200, synth, cfg2, WORKLOADS["cfg2"][2], 256, local_rank)
    st.install_routers(WORKLOADS["cfg2"][3], args.zipf_strength)
    for B in dict(SWEEP)["cfg2"]:
        point(st, "cfg2", WORKLOADS["cfg2"][3], B, 32)
    st.install_routers(None, 0.0)
    for B in dict(SWEEP)["cfg0"]:
        point(st, "cfg0", None, B, 8)
    st.close()
    torch.cuda.empty_cache()
    cfg4 = synth.CONFIGS[WORKLOADS["cfg4"][0]]
    st = Stack(mer_b200, synth, cfg4, 1, 64, local_rank)
    st.install_routers(None, 0.0)
    for B in dict(SWEEP)["cfg4"]:
        point(st, "cfg4", None, B, 1)
    st.close()
    torch.cuda.empty_cache()
    entries.append(run_vram_tier(mer_b200, synth, oracle, args, local_rank, threads))
    return entries


def run_ep_point(mer_b200, synth, oracle, epm, args, wl, n_layers, B_rank, mode, rank, world, local_rank, passes, threads, peaks):
    """One expert-parallel measurement of another configuration (all ranks call this together): B_rank tokens per rank
    through `passes` layer passes rotating over n_layers resident layers, max over ranks of the CUDA-event time, and
    rank 0's first tokens against the oracle."""
    import torch
    import torch.distributed as dist
    cfg_name, _, _, zipf_s = WORKLOADS[wl]
    cfg = synth.CONFIGS[cfg_name]
    owner, mine = ep_placement(epm, synth, cfg, n_layers, zipf_s, args.zipf_strength, rank, world, args.placement)
    stack = Stack(mer_b200, synth, cfg, n_layers, B_rank * world, local_rank, mine=mine)
    stack.install_routers(zipf_s, args.zipf_strength)
    ep = epm.ExpertParallel(stack.be, rank, world, cfg.num_experts, B_rank)
    if owner is not None:
        ep.set_placement(owner)
    if mode == "ep-nccl":
        ep.nccl_init()
    else:
        ep.attach()
    dist.barrier()
    x_host = synth.make_activations(B_rank, cfg.d_model, cfg.seed, 900 + rank)
    x = torch.from_numpy(x_host).to(stack.dev)
    out = torch.empty(B_rank, cfg.d_model, device=stack.dev)
    stream = torch.cuda.current_stream().cuda_stream
    fwd = ep.layer_forward_a2a if mode == "ep-nccl" else ep.layer_forward_peer

    def run(n):
        for i in range(n):
            fwd(i % n_layers, x.data_ptr(), B_rank, out.data_ptr(), stream)

    fwd(0, x.data_ptr(), B_rank, out.data_ptr(), stream)
    ep.check(0, stream)
    par = None
    if rank == 0:
        n = min(2, B_rank)
        rid, _ = stack.be.route(0, x_host[:n])
        par = parity_check(oracle, synth, cfg, 0, zipf_s, args.zipf_strength, list(x_host[:n]), out[:n].cpu().numpy(), rid.astype(np.int64),
                           threads)
    run(3)
    torch.cuda.synchronize()
    dist.barrier()
    ms = cuda_time_ms(torch, lambda: run(passes))
    ep.check(0, stream)
    t = torch.tensor([ms], device=stack.dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    dist.barrier()
    stack.close()
    torch.cuda.empty_cache()
    slots = cfg.top_k + (1 if cfg.shared else 0)
    per_layer = ms / passes
    entry = {"workload": cfg_name, "parallelism": mode, "n_gpus": world, "batch_per_gpu": B_rank, "resident_layers": n_layers,
             "experts_per_gpu_per_layer": len(mine[0]) + (1 if cfg.shared else 0), "placement": args.placement,
             "resident_expert_gb_per_gpu": round(stack.resident_bytes / 1e9, 2), "passes": passes, "ms_per_layer": per_layer,
             "tokens_per_s": B_rank * world / (per_layer * 1e-3), "parity": par}
    if B_rank * world * slots >= GEMM_MEAN_TOKENS * cfg.num_experts:
        flops = 2.0 * B_rank * world * slots * 3 * cfg.d_model * cfg.d_ff
        entry["algorithmic_tflops_all_gpus"] = flops / (per_layer * 1e-3) / 1e12
    return entry


def main():
    args = parse_args()
    # Libraries (NCCL's version banner, for one) write to stdout; the JSON line must be the only thing there.
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg_name, def_batch, def_layers, zipf_s = WORKLOADS[args.workload]
    strong = args.workload == "cfg3"  # a fixed global batch split over the ranks; the other workloads keep B per GPU
    B_global = args.batch or def_batch
    if strong and world > 1:
        assert B_global % world == 0, "the global batch must divide by the number of GPUs"
    B = B_global // world if strong else B_global  # tokens this rank brings to a step
    L = args.layers or def_layers
    mode = args.parallelism
    if mode == "auto":
        mode = "ep-peer" if world > 1 else "replicas"
    if world == 1:
        mode = "replicas"
    ep_mode = mode.startswith("ep-")
    import mer_b200  # noqa: F401  (registers the package alias)
    synth = importlib.import_module("mer_b200.synth")
    cfg = synth.CONFIGS[cfg_name]
    threads = os.cpu_count() or 1
    kind = "prefill" if B_global * cfg.top_k >= GEMM_MEAN_TOKENS * cfg.num_experts else "decode"
    skew = f", Zipf(s={zipf_s}) logit bias x{args.zipf_strength:g}" if zipf_s is not None else ""
    workload = (f"{cfg_name} {kind}: a {B_global}-token batch through {L} resident MoE layers per step "
                f"({cfg.num_experts} experts top-{cfg.top_k}, D={cfg.d_model} F={cfg.d_ff}{skew}; weights and routers seeded per layer)")
    base = {"metric": "moe_layer_tokens_per_s", "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic"}
    exp_bytes = synth.expert_bytes(cfg.dtype, cfg.d_model, cfg.d_ff)
    config = {"workload": workload, "weights": DTYPE_NAME[cfg.dtype], "global_batch": B_global if strong else B * world,
              "batch_per_gpu": B, "resident_layers": L, "layer_passes_per_step": L,
              "resident_expert_gb": round(exp_bytes * (cfg.num_experts + (1 if cfg.shared else 0)) * L / 1e9, 2),
              "value_counts": "tokens x layers per second = tokens/s through one MoE layer",
              "l2": f"a step streams {L} distinct resident layers; every layer pass reads more expert bytes than L2 holds",
              "parallelism": "single GPU" if args.gpus == 1 else PARALLELISM_NOTE[mode].format(
                  n=args.gpus, e=-(-cfg.num_experts // world),
                  placement="placed by the token counts of a calibration batch, largest first onto the least loaded GPU" if args.placement == "balanced"
                  else "rank j holds experts [j*E/N, (j+1)*E/N)")}

    if args.impl == "reference":
        if rank != 0:
            return
        import oracle
        oracle.build()
        x = synth.make_activations(B_global, cfg.d_model, cfg.seed, 0)
        rate, ms, sample = cpu_rate(oracle, synth, cfg, 0, zipf_s, args.zipf_strength, x, threads, args.cpu_seconds * 4,
                                    steps=args.steps, warmup=max(1, min(args.warmup, 2)))
        line = dict(base, impl="reference", value=rate, ms_per_step=ms, config=config,
                    cpu_baseline={"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
                    e2e={"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    note="the reference is Rust and cannot be built here; this is the C restatement of its CPU kernels (oracle/); "
                         "each timed step is a bounded sample of one layer pass, ms_per_step is that sample's time")
        json_out.write(json.dumps(line) + "\n")
        json_out.flush()
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import oracle
    oracle.build()
    peaks = measured_peaks()
    hbm_peak, tf_burst, tf_sustained, peak_kind = peaks

    epm = importlib.import_module("mer_b200.expert_parallel")
    owner = None
    if ep_mode:
        owner, mine = ep_placement(epm, synth, cfg, L, zipf_s, args.zipf_strength, rank, world, args.placement)
    else:
        mine = [list(range(cfg.num_experts))] * L
    stack = Stack(mer_b200, synth, cfg, L, B * world if ep_mode else B, local_rank, mine=mine)
    be, slots = stack.be, stack.slots
    if args.kernel_path:
        be.set_kernel_path(args.kernel_path)
    stack.install_routers(zipf_s, args.zipf_strength)
    be.synchronize()

    dev = stack.dev
    n_x = min(L, 8)  # distinct activation batches, rotated over the layers
    xs_host = [synth.make_activations(B, cfg.d_model, cfg.seed, rank * 64 + i) for i in range(n_x)]
    xs = [torch.from_numpy(x).to(dev) for x in xs_host]
    out = torch.empty(B, cfg.d_model, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    ep = None
    if ep_mode:
        ep = epm.ExpertParallel(be, rank, world, cfg.num_experts, B)
        if owner is not None:
            ep.set_placement(owner)
        if mode == "ep-peer":
            ep.attach()
            dist.barrier()
        elif mode == "ep-nccl":
            ep.nccl_init()

    def layer_pass(l, x, o):
        if mode == "ep-peer":
            ep.layer_forward_peer(l, x.data_ptr(), B, o.data_ptr(), stream)
        elif mode == "ep-nccl":
            ep.layer_forward_a2a(l, x.data_ptr(), B, o.data_ptr(), stream)
        elif mode == "ep-collective":
            ep.layer_forward_collective(l, x, o, slots)
        else:
            be.moe_layer_forward_device(l, x.data_ptr(), B, o.data_ptr(), stream)

    def step():
        for l in range(L):
            layer_pass(l, xs[l % n_x], out)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- parity (outside the timed region): rank 0 recomputes a few of its own tokens of layer 0 with the oracle
    parity = None
    ids_dev = torch.empty(B, slots, dtype=torch.int32, device=dev)
    if ep_mode:
        layer_pass(0, xs[0], out)
        ep.check(0, stream)
        gids = None
        if rank == 0:
            rid, _ = be.route(0, xs_host[0][:PARITY_TOKENS])
            gids = rid.astype(np.int64)
    else:
        be.moe_layer_forward_device(0, xs[0].data_ptr(), B, out.data_ptr(), stream, d_ids=ids_dev.data_ptr())
        be.stream_check(0, stream)
        gids = ids_dev[:PARITY_TOKENS, :cfg.top_k].cpu().numpy().astype(np.int64)  # layer 0: global id = local id
    if rank == 0:
        n = min(PARITY_TOKENS, B)
        parity = parity_check(oracle, synth, cfg, 0, zipf_s, args.zipf_strength, list(xs_host[0][:n]), out[:n].cpu().numpy(),
                              gids[:n], threads)
    barrier()

    # ---- the timed region: exactly K steps, CUDA events on the launching stream, max over ranks
    sampler = ClockSampler(local_rank)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = be.snapshot()["kernel_launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = be.snapshot()["kernel_launches"] - launches0
    # a latched device status (bounded wait expired, missing expert, non-finite router) fails the run here
    if ep_mode:
        ep.check(0, stream)
    else:
        be.stream_check(0, stream)

    # ---- stage timers (same steps, events around each stage) for the roofline of the dominant kernel
    st = None
    hit_bytes = []
    if not ep_mode:
        for l in range(L):
            _, ids, _ = be.moe_layer_forward(l, xs_host[l % n_x])
            hit_bytes.append((len(np.unique(ids[ids != 0xFFFFFFFF])) + (1 if cfg.shared else 0)) * exp_bytes)
        be.stage_timing_enable(True)
        for _ in range(max(1, min(args.steps, 4000 // L))):
            step()
        torch.cuda.synchronize()
        st = be.stage_timings()
        be.stage_timing_enable(False)
    else:
        for l in range(L):
            x_all = np.concatenate([synth.make_activations(B, cfg.d_model, cfg.seed, r * 64 + (l % n_x)) for r in range(world)])
            ids, _ = be.route(l, x_all)
            local = {l * cfg.num_experts + e for e in mine[l]}
            hit = [e for e in np.unique(ids[ids != 0xFFFFFFFF]) if int(e) in local]
            hit_bytes.append((len(hit) + (1 if cfg.shared else 0)) * exp_bytes)
    ep_stages = None
    if mode == "ep-peer":
        # where a rank's layer time goes (plain launches with events between the stages; every rank runs the same steps):
        # router_gate = router + publish + signal + gather (with its wait for the peers) + grouping, combine = signal +
        # wait for the peers + pull
        barrier()
        be.stage_timing_enable(True)
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        t = be.stage_timings()
        be.stage_timing_enable(False)
        mine_ms = {k: round(v / max(t["samples"], 1), 4) for k, v in t.items() if k != "samples"}
        ep_stages = [None] * world
        dist.all_gather_object(ep_stages, mine_ms)

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region
    e2e_ms = e2e_sync_ms = None
    if not args.no_e2e:
        pinned_in = [torch.from_numpy(x).pin_memory() for x in xs_host]
        depth = 3
        outs = [torch.empty(B, cfg.d_model).pin_memory() for _ in range(depth)]
        if mode in ("ep-collective", "ep-nccl"):
            x_dev = torch.empty(B, cfg.d_model, device=dev)

            def e2e_steps(k):
                for _ in range(k):
                    for l in range(L):
                        x_dev.copy_(pinned_in[l % n_x], non_blocking=True)
                        layer_pass(l, x_dev, out)
                        outs[0].copy_(out, non_blocking=True)
                        torch.cuda.current_stream().synchronize()
        else:
            submit = ep.layer_forward_peer_submit if mode == "ep-peer" else be.moe_layer_forward_submit

            def e2e_steps(k):
                # independent layer calls through the pipelined host entry: every call uploads its pinned rows and reads
                # its result back to pinned memory; upload, layer and read-back of neighbouring calls overlap
                n_calls = k * L
                for i in range(n_calls + depth):
                    if i >= depth:
                        be.moe_layer_forward_wait(i % depth)
                    if i < n_calls:
                        l = i % L
                        submit(l, pinned_in[l % n_x].numpy(), outs[i % depth].numpy(), i % depth)
        e2e_steps(1)
        barrier()
        t0 = time.perf_counter()
        e2e_steps(args.steps)
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        if not ep_mode:
            pin_out = outs[0]
            for l in range(L):  # first call per (layer, buffers) captures its graph
                be.moe_layer_forward(l, pinned_in[l % n_x].numpy(), return_routing=False, out=pin_out.numpy())
            n_sync = max(1, min(args.steps, 5))
            t0 = time.perf_counter()
            for _ in range(n_sync):
                for l in range(L):
                    be.moe_layer_forward(l, pinned_in[l % n_x].numpy(), return_routing=False, out=pin_out.numpy())
            e2e_sync_ms = (time.perf_counter() - t0) * 1e3 * args.steps / n_sync
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms_total, e2e_ms or 0.0, e2e_sync_ms or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, e2e_sync_ms = float(times[0]), float(times[1]) or None, float(times[2]) or None
    ep_extra = None
    if ep_mode and strong and not args.no_sweep:
        # the other expert-parallel configuration: the DeepSeek-V3-shaped stack (256 routed experts split over the ranks, the
        # shared expert replicated), a subset of its 58 layers resident, at a decode batch and at a 4096-token prefill
        stack.close()
        stack = None
        torch.cuda.empty_cache()
        ep_extra = []
        for B_all, n_pass in ((16 * world, 60), (4096, 12)):
            ep_extra.append(run_ep_point(mer_b200, synth, oracle, epm, args, "cfg4", 4, B_all // world, mode, rank, world, local_rank,
                                         n_pass, threads, peaks))
    if rank != 0:
        # every rank tears down in the same order (the library's communicator, then torch's): destroying a NCCL
        # communicator waits for its peers, so two communicators destroyed in different orders wait for each other
        if stack is not None:
            stack.close()
        if world > 1:
            dist.destroy_process_group()
        return

    steps = args.steps
    tokens_global = (B_global if strong else B * world)
    layer_tokens = tokens_global * L * steps  # tokens x layers over the timed region, all ranks
    value = layer_tokens / (ms_total * 1e-3)
    mean_hit = sum(hit_bytes) / len(hit_bytes)
    router_bytes = cfg.num_experts * cfg.d_model * 4
    io_bytes = 2 * B * cfg.d_model * 4 + B * cfg.top_k * 8
    layer_bytes = mean_hit + router_bytes + io_bytes
    per_layer_ms = ms_total / (steps * L)
    hbm_gbs = layer_bytes / (per_layer_ms * 1e-3) / 1e9
    gemm = tokens_global * slots >= GEMM_MEAN_TOKENS * (cfg.num_experts + (1 if cfg.shared else 0))
    traffic = ncu_traffic(f"{args.workload}-b{B_global}")
    stages = None
    if st is not None:
        n = max(st["samples"], 1)
        gu_ms, dn_ms = st["expert_gate_up_kernel_ms"] / n, st["expert_down_kernel_ms"] / n
        stages = {k: v / n for k, v in st.items() if k != "samples"}
        if gemm and gu_ms > 0:
            # Algorithmic FLOPs of the gate/up launch: every (token, slot) pair through two [F x D] projections.
            flops = 2.0 * B * slots * 2 * cfg.d_model * cfg.d_ff
            tf = flops / (gu_ms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": "expert_gate_up (grouped dequant GEMM, tcgen05, + SiLU*mul)", "achieved": tf,
                        "peak": tf_burst, "unit": "TFLOP/s", "frac": tf / tf_burst, "peak_source": f"of {peak_kind} (burst figure)",
                        "frac_of_sustained_peak": tf / tf_sustained, "traffic": traffic, "algorithmic_flops_per_launch": flops,
                        "avg_launch_ms": gu_ms,
                        "note": "each algorithmic product is issued as three f16 MMAs (hi*hi, hi*lo, lo*hi) to hold the fp32 "
                                "parity bar, so the tensor pipe does 3x these FLOPs"}
        else:
            fused = dn_ms == 0.0
            kernel_bytes = (mean_hit if fused else mean_hit * 2 / 3) + B * cfg.d_model * 4
            achieved = kernel_bytes / (gu_ms * 1e-3) / 1e9 if gu_ms > 0 else None
            roofline = {"bound": "hbm", "kernel": "expert_gate_up (gate/up dequant-matvec + SiLU*mul)", "achieved": achieved, "peak": hbm_peak,
                        "unit": "GB/s", "frac": achieved / hbm_peak if achieved else None, "peak_source": f"of {peak_kind}",
                        "traffic": traffic, "algorithmic_bytes_per_launch": kernel_bytes, "avg_launch_ms": gu_ms,
                        "frac_of_8tbs": achieved / 8000.0 if achieved else None}
    elif gemm:
        # expert-parallel step: no per-stage timers; rank 0's share of the layer's algorithmic FLOPs over its whole layer pass
        flops = 2.0 * tokens_global * slots * 3 * cfg.d_model * cfg.d_ff / world
        tf = flops / (per_layer_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "whole expert-parallel layer pass of one rank (router, exchange, local experts, combine)",
                    "achieved": tf, "peak": tf_burst, "unit": "TFLOP/s", "frac": tf / tf_burst, "peak_source": f"of {peak_kind} (burst figure)",
                    "traffic": None, "algorithmic_flops_per_launch": flops, "avg_launch_ms": per_layer_ms}
    else:
        roofline = {"bound": "hbm", "kernel": "whole expert-parallel layer pass of one rank (router, exchange, local experts, combine)",
                    "achieved": hbm_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": hbm_gbs / hbm_peak, "peak_source": f"of {peak_kind}",
                    "traffic": None, "algorithmic_bytes_per_launch": layer_bytes, "avg_launch_ms": per_layer_ms}
    step_bytes = B * cfg.d_model * 4 * L
    line = dict(base, value=value, ms_per_step=ms_total / steps, ms_per_layer_pass=per_layer_ms, config=config, clocks=clocks,
                gpu_launches=int(launches), roofline=roofline, parity=parity,
                hbm={"layer_algorithmic_bytes": layer_bytes, "achieved_gbs_per_gpu": hbm_gbs,
                     "frac_of_8tbs": hbm_gbs / 8000.0, "frac_of_measured": hbm_gbs / hbm_peak},
                stage_ms=stages, timed_region_s=ms_total * 1e-3)
    if e2e_ms:
        line["e2e"] = {"value": layer_tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": step_bytes,
                       "d2h_bytes_per_step": step_bytes, "mode": "pipelined host entry, three layer calls in flight"}
    if e2e_sync_ms:
        line["e2e_sync"] = {"value": layer_tokens / (e2e_sync_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": step_bytes,
                            "d2h_bytes_per_step": step_bytes, "mode": "synchronous host entry (mer_moe_layer_forward), one call at a time"}
    if ep_mode and stack is not None:
        stack.close()  # before anything slow on this rank: the other ranks are waiting in the same teardown
        stack = None
    if rank == 0 and args.gpus == 1 and not args.no_cpu:
        rate, ms, sample = cpu_rate(oracle, synth, cfg, 0, zipf_s, args.zipf_strength, xs_host[0], threads, args.cpu_seconds)
        line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
    if rank == 0 and args.gpus == 1 and not args.no_sweep and args.workload == "cfg3":
        line["sweep"] = run_sweep(mer_b200, synth, oracle, args, stack, local_rank, peaks, threads)
    elif stack is not None:
        stack.close()
    if ep_stages is not None:
        line["stage_ms_per_rank"] = ep_stages
    if ep_extra is not None:
        line["sweep"] = ep_extra
    json_out.write(json.dumps(line) + "\n")
    json_out.flush()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
