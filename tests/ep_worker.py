"""One rank of the multi-process expert-parallel check (started by torch.distributed.run).

Backend nccl on GPUs (one GPU per rank), gloo on CPU where only the host logic runs: the
partition, the handle exchange and the sharded arithmetic (each rank computes the partial sums of
its experts with the CPU oracle; the reduction must reproduce the unsharded oracle).  On GPUs the
library computes and the oracle checks."""
import argparse
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import oracle  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["collective", "peer", "a2a", "cpu"], default="collective")
    ap.add_argument("--placement", choices=["contiguous", "table"], default="contiguous")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cpu = args.mode == "cpu"
    dist.init_process_group("gloo" if cpu else "nccl", rank=rank, world_size=world,
                            device_id=None if cpu else torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))))
    from mer_b200 import expert_parallel as epm
    synth = __import__("importlib").import_module("mer_b200.synth")
    dtype, E, D, F, k, B, layer = oracle.Q8_0, 16, 256, 512, 4, 6, 1
    T = B * world
    blobs = [synth.make_expert_blob(dtype, D, F, 71, 0, e) for e in range(E)]
    W = synth.make_router(E, D, 71)
    x_all = synth.make_activations(T, D, 71)
    og = oracle.LinearGate(W, E, D, k)
    ref, rids, rw, _ = oracle.moe_layer_forward(dtype, og, blobs, x_all, F, n_threads=2)
    mine = epm.local_expert_range(rank, world, E)
    owner = None
    if args.placement == "table":  # neither contiguous nor round-robin, uneven shares; by global expert id
        owner = np.zeros((layer + 1) * E, np.uint16)
        owner[layer * E:] = [(e * 7 + e // 3) % world for e in range(E)]
        mine = [e for e in range(E) if owner[layer * E + e] == rank]

    # the handle exchange must return every rank's bytes in rank order, whatever the backend
    fake = bytes([rank]) * 64
    if cpu:
        got = epm.exchange_handles(fake)
        assert got == b"".join(bytes([r]) * 64 for r in range(world))
        # sharded arithmetic with the oracle: partial sums of the local experts, then a reduction
        partial = np.zeros((T, D), np.float32)
        for t in range(T):
            for s in range(k):
                e = int(rids[t, s])
                if epm.expert_owner(e, world, E) == rank:
                    assert e in mine
                    y = oracle.expert_forward(dtype, blobs[e], x_all[t], D, F)
                    partial[t] += rw[t, s] * y
        tot = torch.from_numpy(partial)
        dist.all_reduce(tot)
        err = np.abs(tot.numpy() - ref).max() / np.sqrt(np.mean(ref.astype(np.float64) ** 2))
        assert err <= 1e-5, err
        owners = sorted(e for r in range(world) for e in epm.local_expert_range(r, world, E))
        assert owners == list(range(E))
    else:
        import mer_b200
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
        b = mer_b200.Backend(dtype, D, F, stride * (len(mine) + 1), (layer + 1) * E, max_tokens=T, max_top_k=k, device=local)
        for e in mine:
            b.admit(layer * E + e, 1, blobs[e])
        mer_b200.LinearGate(W, E, D, k).bind(b, layer)
        ep = epm.ExpertParallel(b, rank, world, E, B)
        if owner is not None:
            ep.set_placement(owner)
        x = torch.from_numpy(x_all[rank * B:(rank + 1) * B]).to(dev)
        out = torch.empty(B, D, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        if args.mode == "peer":
            ep.attach()
            dist.barrier()
            for _ in range(4):
                ep.layer_forward_peer(layer, x.data_ptr(), B, out.data_ptr(), stream)
                ep.check(layer, stream)
            first = out.cpu().numpy().copy()
            # the pipelined host form: pinned rows in, pinned rows out, three calls in flight
            xp = torch.from_numpy(x_all[rank * B:(rank + 1) * B].copy()).pin_memory()
            ops = [torch.zeros(B, D).pin_memory() for _ in range(3)]
            for i in range(3):
                ep.layer_forward_peer_submit(layer, xp.numpy(), ops[i].numpy(), i)
            for i in range(3):
                ep.wait(i)
                assert (ops[i].numpy().view(np.uint32) == first.view(np.uint32)).all(), f"rank {rank}: pipelined call {i} differs"
        elif args.mode == "a2a":
            ep.nccl_init()  # the library's own NCCL communicator: all-to-all dispatch and combine inside the library
            for _ in range(3):
                ep.layer_forward_a2a(layer, x.data_ptr(), B, out.data_ptr(), stream)
                ep.check(layer, stream)
        else:
            for _ in range(2):
                ep.layer_forward_collective(layer, x, out, k)
                ep.check(layer, stream)
        got = out.cpu().numpy()
        mref = ref[rank * B:(rank + 1) * B]
        err = np.abs(got - mref).max() / np.sqrt(np.mean(mref.astype(np.float64) ** 2))
        assert err <= 1e-3, f"rank {rank}: {err}"
        dist.barrier()
        b.close()
    dist.barrier()
    if rank == 0:
        print("EP-WORKER-OK", args.mode, world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
