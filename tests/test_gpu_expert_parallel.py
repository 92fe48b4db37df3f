"""Expert-parallel path on the GPU.  One GPU is enough for most of it: the ranks of the
collective mode are run one after the other (their kernels never wait on each other) with the
gathers and the reduction done by torch on the same device; the peer mode is run as a world of
one.  The real multi-process run (2+ GPUs, NCCL and CUDA IPC) is `tests/ep_worker.py`, started
here as child processes when the machine has at least two GPUs."""
import os
import subprocess
import sys

import numpy as np
import pytest

import mer_b200
import oracle
from mer_b200 import GpuExpertDispatchErrorKind as Kind
from mer_b200.expert_parallel import ExpertParallel, local_expert_range

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("mer_b200.synth")
torch = pytest.importorskip("torch")

FFN_TOL = 1e-3


def rel_rms_err(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


def scattered_owner(E, world, layer):
    """A placement table that is neither contiguous nor round-robin, with uneven shares: owner by global expert id."""
    owner = np.zeros((layer + 1) * E, np.uint16)
    owner[layer * E:] = [(e * 7 + e // 3) % world for e in range(E)]
    return owner


def make_rank(dtype, E, D, F, k, world, rank, blobs, W, B, layer, shared_blob=None, gate_kw=None, skip=(), owner=None):
    """A backend that holds only rank's experts of `layer` (+ the shared expert)."""
    mine = [e for e in local_expert_range(rank, world, E) if e not in skip]
    if owner is not None:
        mine = [e for e in range(E) if owner[layer * E + e] == rank and e not in skip]
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    slots = k + (1 if shared_blob is not None else 0)
    b = mer_b200.Backend(dtype, D, F, stride * (len(mine) + 2), (layer + 1) * E + 1, max_tokens=B * world, max_top_k=slots)
    for e in mine:
        b.admit(layer * E + e, 1, blobs[e])
    shared_id = mer_b200.EXPERT_NONE
    if shared_blob is not None:
        shared_id = (layer + 1) * E
        b.admit(shared_id, 1, shared_blob)
    gate = mer_b200.LinearGate.with_routing(W, E, D, k, *gate_kw) if gate_kw else mer_b200.LinearGate(W, E, D, k)
    gate.bind(b, layer, shared_expert_id=shared_id)
    ep = ExpertParallel(b, rank, world, E, B)
    if owner is not None:
        ep.set_placement(owner)
    return b, ep


@pytest.mark.parametrize("placement", ["contiguous", "table"])
@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("case", ["q8-16x4", "q4-32x4-shared"])
def test_collective_mode_ranks_in_turn_match_the_oracle(world, case, placement):
    if case == "q8-16x4":
        dtype, E, D, F, k, B, layer, shared, gate_kw, ogate_kw = oracle.Q8_0, 16, 256, 256, 4, 6, 1, False, None, {}
    else:
        dtype, E, D, F, k, B, layer, shared = oracle.Q4_0, 32, 256, 256, 4, 5, 0, True
        bias = np.random.default_rng(5).normal(0, 0.05, E).astype(np.float32)
        gate_kw = (1, True, bias, 4, 2, 2.5)
        ogate_kw = dict(scoring_func=oracle.SCORE_SIGMOID, correction_bias=bias, n_group=4, topk_group=2, routed_scaling_factor=2.5)
    blobs = [synth.make_expert_blob(dtype, D, F, 61, 0, e) for e in range(E + 1)]
    W = synth.make_router(E, D, 61)
    T = B * world
    x_all = synth.make_activations(T, D, 61)
    slots = k + int(shared)
    dev = torch.device("cuda:0")
    owner = scattered_owner(E, world, layer) if placement == "table" else None
    ranks = [make_rank(dtype, E, D, F, k, world, r, blobs, W, B, layer, blobs[E] if shared else None, gate_kw, owner=owner)
             for r in range(world)]
    try:
        # every rank routes its own tokens; "all-gather" = concatenation in rank order
        ids_parts, w_parts = [], []
        for r, (b, ep) in enumerate(ranks):
            x = torch.from_numpy(x_all[r * B:(r + 1) * B]).to(dev)
            ids = torch.empty(B, slots, dtype=torch.int32, device=dev)
            w = torch.empty(B, slots, dtype=torch.float32, device=dev)
            import ctypes as C
            b._check(b.lib.mer_router_route_device(b.h, layer, C.c_void_p(x.data_ptr()), B, C.c_void_p(ids.data_ptr()),
                                                   C.c_void_p(w.data_ptr()), C.c_void_p(0)))
            ep.check(layer)
            ids_parts.append(ids), w_parts.append(w)
        ids_all, w_all = torch.cat(ids_parts).contiguous(), torch.cat(w_parts).contiguous()
        xg = torch.from_numpy(x_all).to(dev)
        total = torch.zeros(T, D, dtype=torch.float32, device=dev)
        for b, ep in ranks:
            partial = torch.empty(T, D, dtype=torch.float32, device=dev)
            b._check(b.lib.mer_ep_local_experts_forward_device(
                b.h, layer, C.c_void_p(xg.data_ptr()), C.c_void_p(ids_all.data_ptr()), C.c_void_p(w_all.data_ptr()), T, B,
                C.c_void_p(partial.data_ptr()), C.c_void_p(0)))
            ep.check(layer)
            total += partial  # "reduce-scatter" = sum over ranks
        got = total.cpu().numpy()
    finally:
        for b, _ in ranks:
            b.close()
    og = oracle.LinearGate(W, E, D, k, **ogate_kw)
    ref, rids, rw, _ = oracle.moe_layer_forward(dtype, og, blobs[:E], x_all, F, shared_blob=blobs[E] if shared else None, n_threads=4)
    got_ids = ids_all.cpu().numpy().astype(np.int64)[:, :k] - layer * E
    assert (got_ids == rids).all()
    assert rel_rms_err(got, ref) <= FFN_TOL


def test_peer_mode_world_of_one_equals_the_single_gpu_entry_point():
    dtype, E, D, F, k, B, layer = oracle.Q8_0, 16, 256, 512, 4, 7, 0
    blobs = [synth.make_expert_blob(dtype, D, F, 62, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 62)
    x = synth.make_activations(B, D, 62)
    b, ep = make_rank(dtype, E, D, F, k, 1, 0, blobs, W, B, layer)
    try:
        ep.attach()
        dev = torch.device("cuda:0")
        xd = torch.from_numpy(x).to(dev)
        out = torch.empty(B, D, dtype=torch.float32, device=dev)
        for _ in range(3):  # epochs advance; buffers are reused
            ep.layer_forward_peer(layer, xd.data_ptr(), B, out.data_ptr())
            ep.check(layer)
        got = out.cpu().numpy()
        single, _, _ = b.moe_layer_forward(layer, x)
    finally:
        b.close()
    ref, _, _, _ = oracle.moe_layer_forward(dtype, oracle.LinearGate(W, E, D, k), blobs, x, F, n_threads=4)
    assert rel_rms_err(got, ref) <= FFN_TOL
    assert rel_rms_err(got, single) <= 1e-5


@pytest.mark.parametrize("shared", [False, True])
def test_nccl_all_to_all_mode_world_of_one_equals_the_single_gpu_entry_point(shared):
    # the library's own NCCL communicator with one rank: pack, count exchange, self send / recv, local experts over the
    # dispatched rows (one row per pair), return, combine in slot order
    dtype, E, D, F, k, B, layer = oracle.Q8_0, 16, 256, 512, 4, 16, 1
    blobs = [synth.make_expert_blob(dtype, D, F, 63, 0, e) for e in range(E + 1)]
    W = synth.make_router(E, D, 63)
    x = synth.make_activations(B, D, 63)
    b, ep = make_rank(dtype, E, D, F, k, 1, 0, blobs[:E], W, B, layer, shared_blob=blobs[E] if shared else None)
    try:
        ep.nccl_init()
        dev = torch.device("cuda:0")
        xd = torch.from_numpy(x).to(dev)
        out = torch.empty(B, D, dtype=torch.float32, device=dev)
        for _ in range(3):
            ep.layer_forward_a2a(layer, xd.data_ptr(), B, out.data_ptr())
            ep.check(layer)
        got = out.cpu().numpy()
        single, _, _ = b.moe_layer_forward(layer, x)
        # a larger group: GEMM-sized dispatch of the received rows
        b.set_kernel_path(3)
        ep.layer_forward_a2a(layer, xd.data_ptr(), B, out.data_ptr())
        ep.check(layer)
        gemm = out.cpu().numpy()
    finally:
        b.close()
    ref, _, _, _ = oracle.moe_layer_forward(dtype, oracle.LinearGate(W, E, D, k), blobs[:E], x, F, shared_blob=blobs[E] if shared else None,
                                            n_threads=4)
    assert rel_rms_err(got, ref) <= FFN_TOL
    assert rel_rms_err(got, single) <= 1e-5
    assert rel_rms_err(gemm, ref) <= FFN_TOL


def test_a_missing_local_expert_is_a_typed_residency_miss():
    dtype, E, D, F, k, B, layer = oracle.Q8_0, 8, 256, 256, 8, 3, 0  # top-8 of 8: every expert is hit
    blobs = [synth.make_expert_blob(dtype, D, F, 63, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 63)
    x = synth.make_activations(B, D, 63)
    b, ep = make_rank(dtype, E, D, F, k, 1, 0, blobs, W, B, layer, skip=(5,))
    try:
        dev = torch.device("cuda:0")
        xd = torch.from_numpy(x).to(dev)
        out = torch.empty(B, D, dtype=torch.float32, device=dev)
        ep.layer_forward_peer(layer, xd.data_ptr(), B, out.data_ptr())
        with pytest.raises(mer_b200.GpuExpertDispatchError) as e:
            ep.check(layer)
        assert e.value.kind == Kind.ResidencyMiss
    finally:
        b.close()


def test_a_peer_that_never_answers_runs_the_bounded_wait_out():
    # failure detection without a fault: rank 0 of a world of two whose "peer" is never driven.  Both exchange-buffer
    # slots point at rank 0's own buffer, so nothing ever raises rank 1's flag: the gather and combine kernels give
    # up after wait_ms, latch the timeout bit and return; the call fails typed and the backend stays usable.
    import ctypes as C
    dtype, E, D, F, k, B, layer = oracle.Q8_0, 8, 256, 256, 2, 3, 0
    blobs = [synth.make_expert_blob(dtype, D, F, 65, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 65)
    x = synth.make_activations(B, D, 65)
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    b = mer_b200.Backend(dtype, D, F, stride * (E + 1), E, max_tokens=2 * B, max_top_k=k)
    try:
        for e in range(E):
            b.admit(e, 1, blobs[e])
        mer_b200.LinearGate(W, E, D, k).bind(b, layer)
        ep = ExpertParallel(b, 0, 2, E, B, wait_ms=200)
        own = b.lib.mer_ep_exchange_buffer(b.h)
        bufs = (C.c_void_p * 2)(own, own)
        b._check(b.lib.mer_ep_attach_pointers(b.h, bufs, 2))
        dev = torch.device("cuda:0")
        xd = torch.from_numpy(x).to(dev)
        out = torch.empty(B, D, dtype=torch.float32, device=dev)
        ep.layer_forward_peer(layer, xd.data_ptr(), B, out.data_ptr())
        with pytest.raises(mer_b200.GpuExpertDispatchError) as e:
            ep.check(layer)
        assert e.value.kind == Kind.Timeout
        # the context is intact: the plain single-GPU entry point still answers, and correctly
        got, _, _ = b.moe_layer_forward(layer, x)
        ref, _, _, _ = oracle.moe_layer_forward(dtype, oracle.LinearGate(W, E, D, k), blobs, x, F, n_threads=2)
        assert rel_rms_err(got, ref) <= FFN_TOL
    finally:
        b.close()


def test_ep_argument_validation():
    dtype, E, D, F, k, B = oracle.Q8_0, 8, 256, 256, 2, 4
    blobs = [synth.make_expert_blob(dtype, D, F, 64, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 64)
    b, ep = make_rank(dtype, E, D, F, k, 1, 0, blobs, W, B, 0)
    try:
        with pytest.raises(mer_b200.GpuExpertDispatchError):  # second init
            ExpertParallel(b, 0, 1, E, B)
        with pytest.raises(mer_b200.GpuExpertDispatchError) as e:  # more tokens than the group was sized for
            ep.layer_forward_peer(0, 1, B + 1, 1)
        assert e.value.kind == Kind.ValidationDispatch
        with pytest.raises(mer_b200.GpuExpertDispatchError):  # an owner outside the group
            ep.set_placement(np.ones(E, np.uint16))
        with pytest.raises(mer_b200.GpuExpertDispatchError):  # more ids than the backend's id space
            ep.set_placement(np.zeros(10_000, np.uint16))
        ep.set_placement(np.zeros(E, np.uint16))  # everything on rank 0 of a group of one
        ep.set_placement(None)                    # back to the contiguous rule
    finally:
        b.close()
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    with mer_b200.Backend(dtype, D, F, stride * 2, 16, max_tokens=4, max_top_k=2) as small:
        with pytest.raises(mer_b200.GpuExpertDispatchError):  # max_tokens does not cover 2 ranks x 4 tokens
            ExpertParallel(small, 0, 2, E, 4)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("placement", ["contiguous", "table"])
@pytest.mark.parametrize("mode", ["collective", "peer", "a2a"])
def test_two_processes_two_gpus(mode, placement):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(root, "tests", "ep_worker.py"), "--mode", mode, "--placement", placement]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "EP-WORKER-OK" in r.stdout
