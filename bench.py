#!/usr/bin/env python3
"""Benchmark of the routed quantized SwiGLU expert-FFN path (one MoE layer per step).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1] [--batch B] [--impl reference]

A step is one pass of the whole hot path (router top-k -> permute -> gate/up + SiLU*mul -> down ->
weighted combine) over one batch of synthetic tokens.  Steps rotate over `--layers` distinct resident
layers so that no step finds its weights in L2.  Prints ONE JSON line (rank 0).

  value     tokens/s with inputs already in HBM (device pointers, mer_moe_layer_forward_device)
  e2e       tokens/s through the host-buffer entry points (mer_moe_layer_forward_submit / _wait): every step
            uploads its pinned host rows and reads its result back to pinned host memory inside the timed
            region; three independent steps are in flight so that copies and compute overlap
  roofline  dominant kernel: algorithmic bytes / its CUDA-event time, against the measured HBM peak
  cpu_baseline  the CPU restatement of the reference's path timed on this host's cores (rank 0, N=1)

`--impl reference` times the CPU path only (the reference itself is Rust and cannot be built here;
the oracle port stands in for it).
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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {  # name -> (config, default batch, default layers)
    "cfg0": ("cfg0-mixtral-q4_0", 1, 4),
    "cfg1": ("cfg1-qwen3-q8_0", 64, 4),
    "cfg2": ("cfg2-mixtral-stack-q4_0", 16, 32),   # 32 layers x 8 experts resident (25 GB of HBM slots), Zipf(1.1) skew
    "cfg3": ("cfg3-qwen3-prefill-q8_0", 2048, 2),  # prefill: ~128 tokens per expert, Zipf(1.0) skew -> tcgen05 GEMM path
    "cfg4": ("cfg4-deepseek-v3-q4_0", 16, 1),
}
ZIPF = {"cfg2": 1.1, "cfg3": 1.0}  # routing-locality skew added to the router logits of a workload
DTYPE_NAME = {0: "q4_0", 1: "q8_0"}
PARALLELISM_NOTE = {
    "replicas": "{n} replicas, tokens data-parallel, no data-path collective",
    "ep-peer": "expert-parallel over {n} GPUs (experts split contiguously, tokens data-parallel), dispatch and combine by the "
               "library's kernels through peer memory over NVLink",
    "ep-collective": "expert-parallel over {n} GPUs (experts split contiguously, tokens data-parallel), NCCL all-gather of "
                     "tokens+routing and reduce-scatter of partial outputs",
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))  # cfg2: weights of 2 layers repeat over the 32
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--kernel-path", type=int, default=0, help="0 auto, 1 generic, 2 streaming")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="bound on the CPU baseline leg")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "replicas", "ep-peer", "ep-collective"],
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
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": reasons}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def ncu_traffic(key):
    """Per-launch DRAM traffic of the dominant kernel from the committed ncu summary, if one covers this workload."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return json.load(f).get(key)
    except Exception:
        return None


def build_layers(synth, cfg, n_layers, distinct_weight_layers=None):
    """Per layer: expert blobs, shared-expert blob, router.  With distinct_weight_layers = m the expert weights of
    layer l are those of layer l % m (a deep resident stack without minutes of host-side generation); routers and
    activations stay distinct per layer."""
    layers = []
    m = distinct_weight_layers or n_layers
    for l in range(n_layers):
        if l < m:
            blobs = [synth.make_expert_blob(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, l, e) for e in range(cfg.num_experts)]
            shared = synth.make_expert_blob(cfg.dtype, cfg.d_model, cfg.d_ff, cfg.seed, l, cfg.num_experts) if cfg.shared else None
        else:
            blobs, shared = layers[l % m][0], layers[l % m][1]
        layers.append((blobs, shared, synth.make_router(cfg.num_experts, cfg.d_model, cfg.seed, l)))
    return layers


def cpu_layer_rate(oracle, cfg, layer, x, threads, seconds, steps=None, warmup=1):
    """tokens/s of the CPU path on (a bounded sample of) the same step."""
    blobs, shared, W = layer
    gate = oracle.LinearGate(W, cfg.num_experts, cfg.d_model, cfg.top_k, scoring_func=cfg.scoring, n_group=cfg.n_group,
                             topk_group=cfg.topk_group, routed_scaling_factor=cfg.scaling)
    t0 = time.perf_counter()
    oracle.moe_layer_forward_production(cfg.dtype, gate, blobs, x[:1], cfg.d_ff, threads, shared_blob=shared)
    per_token = time.perf_counter() - t0
    n_tok = int(max(1, min(x.shape[0], seconds / 4 / max(per_token, 1e-6))))
    sample = x[:n_tok]
    for _ in range(warmup):
        oracle.moe_layer_forward_production(cfg.dtype, gate, blobs, sample, cfg.d_ff, threads, shared_blob=shared)
    reps, t0 = 0, time.perf_counter()
    while True:
        oracle.moe_layer_forward_production(cfg.dtype, gate, blobs, sample, cfg.d_ff, threads, shared_blob=shared)
        reps += 1
        el = time.perf_counter() - t0
        if (steps is not None and reps >= steps) or (steps is None and (el > seconds / 2 or reps >= 50)):
            break
    return n_tok * reps / el, el / reps * 1e3, f"{n_tok} of {x.shape[0]} tokens of one step, {reps} repetitions, {threads} threads"


def main():
    args = parse_args()
    # Libraries (NCCL's version banner, for one) write to stdout; the JSON line must be the only thing there.
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg_name, def_batch, def_layers = WORKLOADS[args.workload]
    B = args.batch or def_batch
    R = args.layers or def_layers
    mode = args.parallelism
    if mode == "auto":
        mode = "ep-peer" if world > 1 else "replicas"
    if world == 1:
        mode = "replicas"
    ep_mode = mode.startswith("ep-")
    import mer_b200  # noqa: F401  (registers the package alias)
    synth = importlib.import_module("mer_b200.synth")
    cfg = synth.CONFIGS[cfg_name]
    workload = f"{cfg_name} decode batch {B}: 1 MoE layer/step, {cfg.num_experts} experts top-{cfg.top_k}, D={cfg.d_model} F={cfg.d_ff}"
    base = {"metric": "moe_layer_tokens_per_s", "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic"}
    config = {"workload": workload, "weights": DTYPE_NAME[cfg.dtype], "batch_per_gpu": B, "resident_layers": R,
              "l2": f"steps rotate over {R} distinct resident layers; one step streams more expert bytes than L2 holds" if R > 1
              else "single layer", "parallelism": "single GPU" if args.gpus == 1 else PARALLELISM_NOTE[mode].format(n=args.gpus)}

    if args.impl == "reference":
        if rank != 0:
            return
        import oracle
        oracle.build()
        threads = os.cpu_count() or 1
        layer = build_layers(synth, cfg, 1)[0]
        x = synth.make_activations(B, cfg.d_model, cfg.seed, 0)
        rate, ms, sample = cpu_layer_rate(oracle, cfg, layer, x, threads, args.cpu_seconds * 4, steps=args.steps, warmup=args.warmup)
        line = dict(base, impl="reference", value=rate, ms_per_step=ms, config=config,
                    cpu_baseline={"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
                    e2e={"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                    note="the reference is Rust and cannot be built here; this is the C restatement of its CPU kernels (oracle/)")
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

    slots = cfg.top_k + (1 if cfg.shared else 0)
    n_exp = cfg.num_experts + (1 if cfg.shared else 0)
    exp_bytes = mer_b200.expert_bytes(cfg.dtype, cfg.d_model, cfg.d_ff)
    stride = (256 + exp_bytes + 4095) // 4096 * 4096
    epm = importlib.import_module("mer_b200.expert_parallel")
    mine = set(epm.local_expert_range(rank, world, cfg.num_experts)) if ep_mode else set(range(cfg.num_experts))
    n_local = len(mine) + (1 if cfg.shared else 0)
    be = mer_b200.Backend(cfg.dtype, cfg.d_model, cfg.d_ff, stride * n_local * R, (R + 1) * cfg.num_experts + R,
                          max_tokens=B * world if ep_mode else B, max_top_k=slots, device=local_rank)
    if args.kernel_path:
        be.set_kernel_path(args.kernel_path)
    layers = build_layers(synth, cfg, R, distinct_weight_layers=2 if args.workload == "cfg2" else None)
    hit_bytes = []
    xs_host = []
    for l, (blobs, shared, W) in enumerate(layers):
        for e, blob in enumerate(blobs):
            if e in mine:
                be.admit(l * cfg.num_experts + e, 1, blob, wait=False)
        shared_id = 0xFFFFFFFF
        if shared is not None:
            shared_id = R * cfg.num_experts + l
            be.admit(shared_id, 1, shared, wait=False)
        gate = mer_b200.LinearGate.with_routing(W, cfg.num_experts, cfg.d_model, cfg.top_k, cfg.scoring, True, None, cfg.n_group,
                                                cfg.topk_group, cfg.scaling)
        if args.workload in ZIPF:
            gate.logit_bias = synth.zipf_logit_bias(cfg.num_experts, ZIPF[args.workload], cfg.seed, l, strength=0.25)
        be.install_router(l, gate, shared_id)
        xs_host.append(synth.make_activations(B, cfg.d_model, cfg.seed, rank * R + l))
    be.synchronize()
    keep_for_cpu = layers[0] if (rank == 0 and args.gpus == 1 and not args.no_cpu) else None
    x_cpu = xs_host[0]
    del layers

    dev = torch.device("cuda", local_rank)
    xs = [torch.from_numpy(x).to(dev) for x in xs_host]
    out = torch.empty(B, cfg.d_model, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for l in range(R):  # routing per layer -> distinct (local) experts hit -> algorithmic bytes of this rank
        if ep_mode:
            x_all = np.concatenate([synth.make_activations(B, cfg.d_model, cfg.seed, r * R + l) for r in range(world)])
            ids, _ = be.route(l, x_all)
            hit = [e for e in np.unique(ids[ids != 0xFFFFFFFF]) if int(e) in mine]
            distinct = len(hit) + (1 if cfg.shared else 0)
        else:
            _, ids, _ = be.moe_layer_forward(l, xs_host[l])
            distinct = len(np.unique(ids[ids != 0xFFFFFFFF])) + (1 if cfg.shared else 0)
        hit_bytes.append(distinct * exp_bytes)
    router_bytes = cfg.num_experts * cfg.d_model * 4
    io_bytes = 2 * B * cfg.d_model * 4 + B * cfg.top_k * 8

    ep = None
    if ep_mode:
        ep = epm.ExpertParallel(be, rank, world, cfg.num_experts, B)
        if mode == "ep-peer":
            ep.attach()
            dist.barrier()

    def step(i, x=None, o=None):
        l = i % R
        x = xs[l] if x is None else x
        o = out if o is None else o
        if mode == "ep-peer":
            ep.layer_forward_peer(l, x.data_ptr(), B, o.data_ptr(), stream)
        elif mode == "ep-collective":
            ep.layer_forward_collective(l, x, o, slots)
        else:
            be.moe_layer_forward_device(l, x.data_ptr(), B, o.data_ptr(), stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = be.snapshot()["kernel_launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = be.snapshot()["kernel_launches"] - launches0
    if ep_mode:
        ep.check(0, stream)  # surfaces a latched device status (a peer that never answered, a missing expert)
    else:
        be.synchronize()

    # stage timing pass (same steps, events around each stage) for the roofline of the dominant kernel
    st = None
    if not ep_mode:
        be.stage_timing_enable(True)
        for i in range(args.steps):
            step(i)
        torch.cuda.synchronize()
        st = be.stage_timings()
        be.stage_timing_enable(False)

    # end to end: host buffers in, host buffers out, copies inside the timed region
    pinned_in = [torch.from_numpy(x).pin_memory() for x in xs_host]
    pinned_out = torch.empty(B, cfg.d_model).pin_memory()
    x_dev = torch.empty(B, cfg.d_model, device=dev)

    def e2e_step(i):
        if ep_mode:  # pinned host rows -> device, the expert-parallel layer, result back to pinned host memory
            x_dev.copy_(pinned_in[i % R], non_blocking=True)
            step(i, x_dev, out)
            pinned_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        else:  # the library's host entry point does the same copies itself
            be.moe_layer_forward(i % R, pinned_in[i % R].numpy(), return_routing=False, out=pinned_out.numpy())

    for i in range(3):
        e2e_step(i)
    barrier()
    if mode == "ep-collective":
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    else:
        # independent token batches through the pipelined host entry: every step uploads its pinned rows and reads its
        # result back to pinned memory; upload, layer and read-back of neighbouring steps overlap (three in flight)
        depth = 3
        outs = [torch.empty(B, cfg.d_model).pin_memory() for _ in range(depth)]
        submit = ep.layer_forward_peer_submit if mode == "ep-peer" else be.moe_layer_forward_submit
        for i in range(depth):  # warm the slots (allocations, graph capture)
            submit(i % R, pinned_in[i % R].numpy(), outs[i].numpy(), i)
        for i in range(depth):
            be.moe_layer_forward_wait(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps + depth):
            if i >= depth:
                be.moe_layer_forward_wait(i % depth)
            if i < args.steps:
                submit(i % R, pinned_in[i % R].numpy(), outs[i % depth].numpy(), i % depth)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([ms_total, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(times[0]), float(times[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    steps = args.steps
    tokens = B * steps * world
    value = tokens / (ms_total * 1e-3)
    mean_hit = sum(hit_bytes[i % R] for i in range(steps)) / steps
    layer_bytes = mean_hit + router_bytes + io_bytes
    hbm_gbs = layer_bytes * steps / (ms_total * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    if st is not None:
        n = max(st["samples"], 1)
        gu_ms, dn_ms = st["expert_gate_up_kernel_ms"] / n, st["expert_down_kernel_ms"] / n
        fused = dn_ms == 0.0
        kernel_bytes = (mean_hit if fused else mean_hit * 2 / 3) + B * cfg.d_model * 4
        achieved = kernel_bytes / (gu_ms * 1e-3) / 1e9 if gu_ms > 0 else None
        kname = "expert_ffn (gate/up + SiLU*mul + down)" if fused else "expert_gate_up (gate/up dequant-matvec + SiLU*mul)"
        roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak if achieved else None, "peak_source": f"of {peak_kind}",
                    "traffic": ncu_traffic(f"{args.workload}-b{B}"), "algorithmic_bytes_per_launch": kernel_bytes,
                    "avg_launch_ms": gu_ms, "frac_of_8tbs": achieved / 8000.0 if achieved else None}
        stages = {k: v / n for k, v in st.items() if k != "samples"}
        if B * slots >= 32 * n_exp and not fused and gu_ms > 0:
            # a mean of 32 tokens per expert and more: the tcgen05 GEMM kernels run, bounded by the tensor pipe.
            # Algorithmic FLOPs of the gate/up launch: every (token, slot) pair through two [F x D] projections.
            tpeak, tkind = measured_tensor_peak()
            flops = 2.0 * B * slots * 2 * cfg.d_model * cfg.d_ff
            tf = flops / (gu_ms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": "expert_gate_up (grouped dequant GEMM, tcgen05, + SiLU*mul)", "achieved": tf,
                        "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak, "peak_source": f"of {tkind}",
                        "traffic": ncu_traffic(f"{args.workload}-b{B}"), "algorithmic_flops_per_launch": flops,
                        "avg_launch_ms": gu_ms,
                        "note": "each algorithmic product is issued as three f16 MMAs (hi*hi, hi*lo, lo*hi) to hold the fp32 "
                                "parity bar, so the tensor pipe does 3x these FLOPs"}
    else:
        # expert-parallel step: no per-stage timers; the whole step of rank 0 against the bytes its experts stream
        roofline = {"bound": "hbm", "kernel": "whole expert-parallel step of one rank (router, exchange, local experts, combine)",
                    "achieved": hbm_gbs, "peak": peak, "unit": "GB/s", "frac": hbm_gbs / peak, "peak_source": f"of {peak_kind}",
                    "traffic": None, "algorithmic_bytes_per_launch": layer_bytes, "avg_launch_ms": ms_total / steps}
        stages = None
    line = dict(base, value=value, ms_per_step=ms_total / steps, config=config, clocks=clocks,
                e2e={"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": B * cfg.d_model * 4,
                     "d2h_bytes_per_step": B * cfg.d_model * 4},
                gpu_launches=int(launches), roofline=roofline,
                hbm={"layer_algorithmic_bytes": layer_bytes, "achieved_gbs_per_gpu": hbm_gbs,
                     "frac_of_8tbs": hbm_gbs / 8000.0, "frac_of_measured": hbm_gbs / peak},
                stage_ms=stages)
    if keep_for_cpu is not None:
        import oracle
        oracle.build()
        threads = os.cpu_count() or 1
        rate, ms, sample = cpu_layer_rate(oracle, cfg, keep_for_cpu, x_cpu, threads, args.cpu_seconds)
        line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
    json_out.write(json.dumps(line) + "\n")
    json_out.flush()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
