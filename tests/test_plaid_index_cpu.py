"""CPU checks of the PLAID front stage's host logic: the fast-plaid file reader and the inverted file."""

import json
import os

import numpy as np
import torch

import cases
from oracle import maxsim_oracle as O


def write_fastplaid_files(path, codes, residuals, lens, centroids, buckets, nbits, *, merged, pad_rows=0, chunks=2):
    """Files in the layout the reference's benchmark reads (benchmarks/plaid/bench_fastplaid_e2e.py:76-140)."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "metadata.json"), "w") as f:
        json.dump({"nbits": nbits, "num_chunks": chunks}, f)
    np.save(os.path.join(path, "centroids.npy"), centroids)
    np.save(os.path.join(path, "bucket_weights.npy"), buckets)
    bounds = np.linspace(0, len(lens), chunks + 1).astype(int)
    cu = np.concatenate([[0], np.cumsum(lens)])
    for c in range(chunks):
        with open(os.path.join(path, f"doclens.{c}.json"), "w") as f:
            json.dump([int(x) for x in lens[bounds[c]:bounds[c + 1]]], f)
        if not merged:
            a, b = cu[bounds[c]], cu[bounds[c + 1]]
            np.save(os.path.join(path, f"codes.{c}.npy"), codes[a:b].astype(np.int64))
            np.save(os.path.join(path, f"residuals.{c}.npy"), residuals[a:b])
    if merged:
        pad_c = np.concatenate([codes, np.zeros(pad_rows, codes.dtype)]).astype(np.int64)
        pad_r = np.concatenate([residuals, np.zeros((pad_rows, residuals.shape[1]), np.uint8)])
        np.save(os.path.join(path, "merged_codes.npy"), pad_c)
        np.save(os.path.join(path, "merged_residuals.npy"), pad_r.reshape(-1))  # stored flat, as fast-plaid may


def small_index(seed=3, nd=40, d=32, nbits=2, ncent=16, max_len=12):
    rng = np.random.default_rng(seed)
    lens = rng.integers(0, max_len + 1, size=nd)
    T = int(lens.sum())
    codes = rng.integers(0, ncent, size=T).astype(np.int32)
    res = rng.integers(0, 256, size=(T, d * nbits // 8)).astype(np.uint8)
    cent = cases.unit(rng.standard_normal((ncent, d))).astype(np.float16)
    bw = np.linspace(-0.1, 0.1, 2**nbits).astype(np.float32)
    return codes, res, lens, cent, bw, nbits


def test_reader_round_trip_merged_and_chunked(tmp_path):
    from late_interaction_kernels_b200.plaid_index import read_fastplaid_index

    codes, res, lens, cent, bw, nbits = small_index()
    for merged in (True, False):
        p = str(tmp_path / f"idx_{int(merged)}")
        write_fastplaid_files(p, codes, res, lens, cent, bw, nbits, merged=merged, pad_rows=5)
        ix = read_fastplaid_index(p, device="cpu")
        assert ix.nbits == nbits and ix.n_docs == len(lens) and ix.dim == 32
        assert ix.codes_flat.dtype == torch.int32 and np.array_equal(ix.codes_flat.numpy(), codes)
        assert ix.residuals_flat.dtype == torch.uint8 and np.array_equal(ix.residuals_flat.numpy(), res)
        assert np.array_equal(ix.doc_lengths.numpy(), lens)
        assert np.array_equal(ix.cu_seqlens_d.numpy(), np.concatenate([[0], np.cumsum(lens)]))
        assert np.array_equal(ix.centroids.numpy(), cent) and np.array_equal(ix.bucket_weights.numpy(), bw)


def test_inverted_file_matches_the_oracle():
    from late_interaction_kernels_b200.plaid_index import PlaidIndexData, build_ivf

    codes, res, lens, cent, bw, nbits = small_index(seed=5, nd=60, ncent=23)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ix = PlaidIndexData(nbits, torch.from_numpy(cent), torch.from_numpy(bw), torch.from_numpy(codes), torch.from_numpy(res),
                        torch.from_numpy(lens.astype(np.int64)), torch.from_numpy(cu))
    build_ivf(ix)
    docs, off = O.plaid_ivf(codes, cu, 23)
    assert np.array_equal(ix.ivf_docs.numpy(), docs) and np.array_equal(ix.ivf_offsets.numpy(), off)
    # brute force: document j is on the list of centroid c exactly when one of its tokens has code c
    for c in range(23):
        want = [j for j in range(60) if (codes[cu[j]:cu[j + 1]] == c).any()]
        assert docs[off[c]:off[c + 1]].tolist() == want
