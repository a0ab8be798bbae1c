"""Host-side logic of the document-sharded retrieve on CPU ranks (gloo, world size 2 and 3):
shard bounds, padding of short shards, the all-gather layout and the final merge.  The per-shard
scoring and the merge kernel are replaced by the CPU oracle here; their CUDA versions are covered by
the GPU tests."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from late_interaction_kernels_b200 import sharded
from oracle import maxsim_oracle as O


def test_shard_bounds_cover_the_corpus():
    for n, w in [(0, 2), (1, 4), (7, 2), (8, 8), (1000003, 8), (5, 8)]:
        spans = [sharded.shard_bounds(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all(lo <= hi for lo, hi in spans)
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 2, 2)


def test_pad_candidates():
    s = torch.tensor([[3.0, 1.0]])
    i = torch.tensor([[5, 9]])
    ps, pi = sharded.pad_candidates(s, i, 4)
    assert ps.tolist() == [[3.0, 1.0, float("-inf"), float("-inf")]] and pi.tolist() == [[5, 9, -1, -1]]
    ps, pi = sharded.pad_candidates(s, i, 3, largest=False)
    assert ps[0, 2] == float("inf") and pi[0, 2] == -1
    with pytest.raises(ValueError):
        sharded.pad_candidates(s, i, 1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, top_k, out_dir, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        Q, D, dm = cases.retrieve_case(10)
        lo, hi = sharded.shard_bounds(D.shape[0], world, rank)
        if rank == fail_rank:
            raise RuntimeError("injected failure before the gather")
        k = min(top_k, D.shape[0])
        if hi > lo:
            s, i = O.retrieve(Q, D[lo:hi], min(k, hi - lo), d_mask=dm[lo:hi])
            i = i + lo
        else:
            s, i = np.zeros((Q.shape[0], 0), np.float32), np.zeros((Q.shape[0], 0), np.int64)
        s, i = sharded.pad_candidates(torch.from_numpy(s), torch.from_numpy(i), k)
        gs, gi = sharded.gather_candidates(s, i)
        assert gs.shape == (world, Q.shape[0], k)
        ms, mi = O.merge_topk(np.moveaxis(gs.numpy(), 0, 1).reshape(Q.shape[0], -1),
                              np.moveaxis(gi.numpy(), 0, 1).reshape(Q.shape[0], -1), k)
        np.savez(os.path.join(out_dir, f"r{rank}.npz"), s=ms, i=mi)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,top_k", [(2, 5), (3, 30), (2, 100)])
def test_sharded_retrieve_equals_single_rank(tmp_path, world, top_k):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, top_k, str(tmp_path), -1), nprocs=world, join=True)
    Q, D, dm = cases.retrieve_case(10)
    ws, wi = O.retrieve(Q, D, top_k, d_mask=dm)
    for r in range(world):
        got = np.load(tmp_path / f"r{r}.npz")
        assert np.array_equal(got["i"], wi), f"rank {r}"
        np.testing.assert_allclose(got["s"], ws, rtol=1e-6)


def test_a_rank_that_raises_fails_the_job(tmp_path):
    """Failure detection on the host: a rank that raises before the collective makes the launcher
    report the failure instead of hanging (the surviving rank's gather errors out or is torn down)."""
    port = _free_port()
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(2, port, 5, str(tmp_path), 1), nprocs=2, join=True)
