"""World-size-2 CPU run (gloo) of the expert-parallel host logic: partition, handle exchange in
rank order, and the sharded arithmetic checked against the unsharded oracle."""
import os
import subprocess
import sys

import pytest

from mer_b200.expert_parallel import balanced_placement, expert_owner, experts_per_rank, local_expert_range


def test_partition_is_contiguous_and_complete():
    for E, world in [(128, 8), (128, 2), (256, 8), (8, 1), (10, 4), (3, 8)]:
        epr = experts_per_rank(E, world)
        seen = []
        for r in range(world):
            rng = local_expert_range(r, world, E)
            assert all(expert_owner(e, world, E) == r for e in rng)
            assert len(rng) <= epr
            seen += list(rng)
        assert seen == list(range(E))


def test_balanced_placement_gives_every_rank_the_same_number_of_experts_and_levels_the_load():
    import numpy as np
    rng = np.random.default_rng(0)
    for E, world in [(128, 2), (128, 4), (128, 8), (256, 8), (10, 4)]:
        counts = (16384 / (rng.permutation(E) + 1.0)).astype(np.int64)  # Zipf(1.0) popularity, shuffled
        owner = balanced_placement(counts, world)
        assert len(owner) == E and set(owner) <= set(range(world))
        held = np.bincount(owner, minlength=world)
        assert held.max() <= experts_per_rank(E, world) and held.sum() == E
        load = np.bincount(owner, weights=counts, minlength=world)
        contiguous = np.array([counts[list(local_expert_range(r, world, E))].sum() for r in range(world)])
        assert load.max() <= contiguous.max()
        # never worse than 1.05 x the mean, or the busiest expert together with the least busy ones that fill its rank
        cap = experts_per_rank(E, world)
        assert load.max() <= max(counts.max() + np.sort(counts)[:cap - 1].sum(), 1.05 * counts.sum() / world)
        assert balanced_placement(counts, world) == owner  # deterministic


@pytest.mark.timeout(300)
def test_two_gloo_ranks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(root, "tests", "ep_worker.py"), "--mode", "cpu"]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "EP-WORKER-OK" in r.stdout
