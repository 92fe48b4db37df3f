"""Expert-parallel execution of a MoE layer: one process per GPU, experts split contiguously by id or by a placement table.

Stands in for the reference's expert sharding (`ShardRouter`, distributed.rs; docs/distributed.md:16-50:
the router node computes the full top-k, fans out to the shards that own the experts, sums the
weighted outputs, a shard that times out contributes zero and is counted).  Here the shards are the
GPUs of one NVSwitch box.  Two exchange modes over the same partition:

* ``peer``       -- the library's kernels exchange through peer memory (exchange buffers mapped with
                    CUDA IPC): publish, flag, pull.  Summation stays in slot order.
* ``a2a``        -- the library calls NCCL itself: all-to-all dispatch of only the rows that hit a peer's experts
                    (grouped ncclSend / ncclRecv), local experts, all-to-all return, combine in slot order.
* ``collective`` -- torch.distributed (NCCL) moves the data: all-gather of tokens and routing,
                    reduce-scatter of the partial outputs.

torch.distributed is plumbing only (handle exchange, the collectives of the second mode).
"""
import ctypes as C

from . import capi


def experts_per_rank(experts_per_layer, world):
    return (experts_per_layer + world - 1) // world


def local_expert_range(rank, world, experts_per_layer):
    """Local (within-layer) expert indices owned by `rank`: contiguous blocks of ceil(E / world)."""
    epr = experts_per_rank(experts_per_layer, world)
    return range(min(rank * epr, experts_per_layer), min((rank + 1) * epr, experts_per_layer))


def expert_owner(local_index, world, experts_per_layer):
    return local_index // experts_per_rank(experts_per_layer, world)


def balanced_placement(counts, world):
    """Placement of one layer's experts by measured popularity: `counts[e]` = tokens expert e received in a
    calibration batch.  Greedy (largest first, onto the least loaded rank that still has room), every rank gets
    the same number of experts (ceil(E / world) at most).  Returns owner[e] as a list; deterministic, so every rank
    that computes it from the same counts gets the same table."""
    E = len(counts)
    cap = experts_per_rank(E, world)
    load, held, owner = [0] * world, [0] * world, [0] * E
    for e in sorted(range(E), key=lambda i: (-int(counts[i]), i)):
        r = min((j for j in range(world) if held[j] < cap), key=lambda j: (load[j], j))
        owner[e] = r
        load[r] += int(counts[e])
        held[r] += 1
    return owner


def exchange_handles(handle_bytes, group=None):
    """All ranks' 64-byte handles in rank order (any torch.distributed backend)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(handle_bytes), group=group)
    return b"".join(gathered)


class ExpertParallel:
    """The expert-parallel view of one `Backend` (which must have been created with
    max_tokens >= world * max_tokens_per_rank and holds only this rank's experts)."""

    def __init__(self, backend, rank, world, experts_per_layer, max_tokens_per_rank, wait_ms=2000):
        self.b, self.rank, self.world = backend, rank, world
        self.experts_per_layer, self.max_tokens_per_rank = experts_per_layer, max_tokens_per_rank
        cfg = capi.MerEpCfg(rank, world, experts_per_layer, max_tokens_per_rank, wait_ms, 0)
        backend._check(backend.lib.mer_ep_init(backend.h, C.byref(cfg)))
        self._bufs = {}

    def local_experts(self):
        return local_expert_range(self.rank, self.world, self.experts_per_layer)

    def owns(self, local_index):
        return expert_owner(local_index, self.world, self.experts_per_layer) == self.rank

    def set_placement(self, owner_by_global_id):
        """Installs owner[global expert id] = rank (the same table on every rank) in place of the contiguous rule;
        None restores it.  The host admits the experts the table gives this rank."""
        import numpy as np
        if owner_by_global_id is None:
            self.b._check(self.b.lib.mer_ep_set_placement(self.b.h, None, 0))
            return
        t = np.ascontiguousarray(owner_by_global_id, dtype=np.uint16)
        self.b._check(self.b.lib.mer_ep_set_placement(self.b.h, t.ctypes.data_as(C.c_void_p), t.size))

    # -- peer mode ------------------------------------------------------------------------
    def export_handle(self):
        buf = C.create_string_buffer(64)
        self.b._check(self.b.lib.mer_ep_export_handle(self.b.h, buf))
        return buf.raw

    def attach(self, group=None):
        """Exchange the IPC handles of all ranks and map the peers' exchange buffers."""
        if self.world == 1:
            return
        handles = exchange_handles(self.export_handle(), group)
        assert len(handles) == 64 * self.world
        self.b._check(self.b.lib.mer_ep_attach_handles(self.b.h, handles, self.world))

    def layer_forward_peer(self, layer, d_x, n_tokens, d_out, stream=0):
        self.b._check(self.b.lib.mer_ep_layer_forward_device(self.b.h, layer, C.c_void_p(d_x), n_tokens, C.c_void_p(d_out),
                                                             C.c_void_p(stream)))

    def layer_forward_peer_submit(self, layer, x_pinned, out_pinned, slot):
        """Pipelined host form of layer_forward_peer: pinned numpy views in and out, returns at once."""
        n = x_pinned.size // self.b.d_model
        self.b._check(self.b.lib.mer_ep_layer_forward_submit(
            self.b.h, layer, x_pinned.ctypes.data_as(C.c_void_p), n, out_pinned.ctypes.data_as(C.c_void_p), slot))

    def wait(self, slot):
        self.b._check(self.b.lib.mer_moe_layer_forward_wait(self.b.h, slot))

    # -- NCCL all-to-all mode ---------------------------------------------------------------
    def nccl_init(self, group=None):
        """Rank 0 creates the ncclUniqueId, torch.distributed hands it round, every rank joins the library's own
        NCCL communicator (collective)."""
        import torch.distributed as dist
        ident = [None]
        if self.rank == 0:
            buf = C.create_string_buffer(128)
            self.b._check(self.b.lib.mer_ep_nccl_unique_id(buf))
            ident[0] = buf.raw
        if self.world > 1:
            dist.broadcast_object_list(ident, src=0, group=group)
        self.b._check(self.b.lib.mer_ep_nccl_init(self.b.h, ident[0]))

    def layer_forward_a2a(self, layer, d_x, n_tokens, d_out, stream=0):
        self.b._check(self.b.lib.mer_ep_layer_forward_a2a_device(self.b.h, layer, C.c_void_p(d_x), n_tokens, C.c_void_p(d_out),
                                                                 C.c_void_p(stream)))

    # -- collective mode --------------------------------------------------------------------
    def _buffers(self, n_tokens, slots, device):
        import torch
        key = (n_tokens, slots)
        if key not in self._bufs:
            T, D = n_tokens * self.world, self.b.d_model
            f32, i32 = torch.float32, torch.int32
            self._bufs[key] = dict(
                ids=torch.empty(n_tokens, slots, dtype=i32, device=device), w=torch.empty(n_tokens, slots, dtype=f32, device=device),
                x_all=torch.empty(T, D, dtype=f32, device=device), ids_all=torch.empty(T, slots, dtype=i32, device=device),
                w_all=torch.empty(T, slots, dtype=f32, device=device), partial=torch.empty(T, D, dtype=f32, device=device))
        return self._bufs[key]

    def layer_forward_collective(self, layer, x, out, slots, group=None):
        """x, out: [n_tokens, d_model] f32 CUDA tensors of this rank; runs on torch's current stream."""
        import torch
        import torch.distributed as dist
        n = x.shape[0]
        s = torch.cuda.current_stream().cuda_stream
        B = self._buffers(n, slots, x.device)
        lib, h = self.b.lib, self.b.h
        self.b._check(lib.mer_router_route_device(h, layer, C.c_void_p(x.data_ptr()), n, C.c_void_p(B["ids"].data_ptr()),
                                                  C.c_void_p(B["w"].data_ptr()), C.c_void_p(s)))
        if self.world > 1:
            dist.all_gather_into_tensor(B["x_all"], x, group=group)
            dist.all_gather_into_tensor(B["ids_all"], B["ids"], group=group)
            dist.all_gather_into_tensor(B["w_all"], B["w"], group=group)
            x_all, ids_all, w_all = B["x_all"], B["ids_all"], B["w_all"]
        else:
            x_all, ids_all, w_all = x, B["ids"], B["w"]
        partial = B["partial"] if self.world > 1 else out
        self.b._check(lib.mer_ep_local_experts_forward_device(
            h, layer, C.c_void_p(x_all.data_ptr()), C.c_void_p(ids_all.data_ptr()), C.c_void_p(w_all.data_ptr()),
            n * self.world, n, C.c_void_p(partial.data_ptr()), C.c_void_p(s)))
        if self.world > 1:
            dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=group)

    def check(self, layer, stream=0):
        """Synchronise the stream and raise the typed error the device status word holds, if any."""
        self.b._check(self.b.lib.mer_stream_check(self.b.h, layer, C.c_void_p(stream)))
