"""One rank of the multi-GPU sharded-retrieve check (launched by test_gpu_sharded_nccl.py through
torch.distributed.run, NCCL backend, one process per GPU).  Every rank builds the same seeded
corpus, keeps its own document slice, runs the sharded calls and compares the result with the
single-GPU call on the whole corpus (and rank 0 with the CPU oracle)."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    from golden import cases
    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import plaid, sharded
    from oracle import maxsim_oracle as O

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda")
    dist.init_process_group("nccl")

    rng = np.random.default_rng(11)
    Nq, Lq, Nd, Ld, d, k = 9, 12, 257, 37, 64, 20
    Q = cases.unit(rng.standard_normal((Nq, Lq, d))).astype(np.float32)
    D = cases.unit(rng.standard_normal((Nd, Ld, d))).astype(np.float32)
    lens = rng.integers(1, Ld + 1, size=Nd)
    dm = np.arange(Ld)[None, :] < lens[:, None]
    tq = torch.from_numpy(Q).to(dev, torch.bfloat16)
    tD = torch.from_numpy(D).to(dev, torch.bfloat16)
    tm = torch.from_numpy(dm).to(dev)

    lo, hi = sharded.shard_bounds(Nd, world, rank)
    s, i = sharded.retrieve_sharded(tq, tD[lo:hi], k, d_mask=tm[lo:hi], doc_offset=lo, n_docs_total=Nd, normalize=False, chunk=50)
    ws, wi = lik.retrieve(tq, tD, k, d_mask=tm, normalize=False, chunk=50)
    assert torch.equal(s, ws), "sharded scores differ from the single-GPU retrieve"
    assert torch.equal(i, wi), "sharded indices differ from the single-GPU retrieve"
    if rank == 0:
        os_, oi = O.retrieve(tq.float().cpu().numpy(), tD.float().cpu().numpy(), k, d_mask=dm, normalize=False)
        assert O.rel_err(s.cpu().numpy(), os_) < 2e-2
        got = np.take_along_axis(O.maxsim(tq.float().cpu().numpy(), tD.float().cpu().numpy(), None, dm), i.cpu().numpy(), axis=1)
        assert O.rel_err(got, os_) < 2e-2, "indices do not point at the top scores"

    # PLAID index sharded by document: codes / residuals / offsets sliced and re-based per rank
    nbits, ncent = 2, 64
    plens = rng.integers(0, 30, size=Nd)
    T = int(plens.sum())
    codes = rng.integers(0, ncent, size=T).astype(np.int32)
    res = rng.integers(0, 256, size=(T, d * nbits // 8)).astype(np.uint8)
    cu = np.concatenate([[0], np.cumsum(plens)]).astype(np.int64)
    cent = torch.from_numpy(cases.unit(rng.standard_normal((ncent, d))).astype(np.float16)).to(dev)
    bw = torch.from_numpy(np.linspace(-0.1, 0.1, 4).astype(np.float32)).to(dev)
    t0, t1 = int(cu[lo]), int(cu[hi])
    s, i = sharded.retrieve_plaid_sharded(
        tq, torch.from_numpy(codes[t0:t1]).to(dev), torch.from_numpy(res[t0:t1]).to(dev),
        torch.from_numpy((cu[lo:hi + 1] - cu[lo]).astype(np.int32)).to(dev), cent, bw, nbits, k, doc_offset=lo, n_docs_total=Nd, chunk=64)
    ws, wi = plaid.retrieve_residual_varlen(tq, torch.from_numpy(codes).to(dev), torch.from_numpy(res).to(dev),
                                            torch.from_numpy(cu.astype(np.int32)).to(dev), cent, bw, nbits, k, chunk=64)
    assert torch.equal(s, ws) and torch.equal(i, wi), "sharded PLAID retrieve differs from the single-GPU call"

    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("sharded worker ok", flush=True)


if __name__ == "__main__":
    main()
