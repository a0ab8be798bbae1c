"""GPU tests of the top-k selection over score rows (``lik_topk_rows``): exact agreement - scores and indices - with
a stable sort (better score first, ties to the lower document index), over rows of one and of many register slabs,
rows full of ties, masked (-inf) columns, every k up to the maximum, smallest-first, and a running list merged
chunk by chunk in and out of order."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _want(scores, k, largest=True, index=None):
    """Stable reference: ties to the lower index (``index`` gives every column's document index)."""
    n = scores.shape[1]
    idx = torch.arange(n, device=scores.device).expand_as(scores) if index is None else index
    key = scores if largest else -scores
    # order by (key desc, idx asc): sort by idx first (stable), then by key (stable)
    o1 = torch.sort(idx, dim=1, stable=True).indices
    k1 = torch.gather(key, 1, o1)
    o2 = torch.sort(k1, dim=1, descending=True, stable=True).indices
    order = torch.gather(o1, 1, o2)[:, :k]
    return torch.gather(scores, 1, order), torch.gather(idx, 1, order)


@pytest.mark.parametrize("rows,cols,k", [(7, 50, 10), (3, 4096, 100), (5, 4097, 128), (2, 20000, 1024), (4, 9000, 1), (33, 300, 300),
                                          (1, 70000, 32), (6, 12, 100)])
@pytest.mark.parametrize("largest", [True, False])
def test_rows_match_a_stable_sort(rows, cols, k, largest):
    from late_interaction_kernels_b200 import _ops

    g = torch.Generator(device="cuda").manual_seed(rows * 1000 + cols)
    sc = torch.randn((rows, cols), generator=g, device="cuda")
    s, i = _ops.topk_rows(sc, k, largest=largest, index_offset=5)
    kk = min(k, cols)
    ws, wi = _want(sc, kk, largest)
    assert torch.equal(s[:, :kk], ws) and torch.equal(i[:, :kk], wi + 5)
    if k > cols:  # the list is padded
        fill = float("-inf") if largest else float("inf")
        assert (s[:, cols:] == fill).all() and (i[:, cols:] == -1).all()


@pytest.mark.parametrize("levels", [1, 3, 40])
def test_ties_go_to_the_lower_index(levels):
    from late_interaction_kernels_b200 import _ops

    g = torch.Generator(device="cuda").manual_seed(levels)
    sc = torch.randint(0, levels, (9, 13000), generator=g, device="cuda").float()
    sc[:, ::7] = float("-inf")  # masked documents
    sc[2] = 0.0                 # a row of nothing but one value
    sc[3, 5:] = -0.0            # the two zeros are one value
    for k in (1, 100, 1000):
        s, i = _ops.topk_rows(sc, k)
        ws, wi = _want(sc, k)
        assert torch.equal(s, ws) and torch.equal(i, wi), (levels, k)
        s, i = _ops.topk_rows(sc, k, largest=False)
        ws, wi = _want(sc, k, largest=False)
        assert torch.equal(s, ws) and torch.equal(i, wi), (levels, k, "smallest")


@pytest.mark.parametrize("order", ["ascending", "shuffled"])
def test_running_list_over_chunks(order):
    from late_interaction_kernels_b200 import _ops

    g = torch.Generator(device="cuda").manual_seed(11)
    sc = torch.randint(0, 50, (6, 30000), generator=g, device="cuda").float()  # ties across chunks
    k, chunk = 100, 4096
    starts = list(range(0, sc.shape[1], chunk))
    if order == "shuffled":
        starts = [starts[j] for j in torch.randperm(len(starts), generator=torch.Generator().manual_seed(1)).tolist()]
    out = None
    for s0 in starts:
        out = _ops.topk_rows(sc[:, s0:s0 + chunk].contiguous(), k, index_offset=s0, out=out)
    ws, wi = _want(sc, k)
    assert torch.equal(out[0], ws) and torch.equal(out[1], wi)


@pytest.mark.parametrize("rows,cols,k", [(3, 20000, 1025), (2, 30000, 4096), (2, 9000, 8192), (1, 5000, 8192), (2, 20000, 9000)])
def test_large_k(rows, cols, k):
    """k above 1024 takes the 1024-thread shape of the selection kernel (up to 8192); beyond that the library-sort path.
    Same contract: exact agreement with the stable sort, chunked or not, ties included."""
    from late_interaction_kernels_b200 import _ops

    g = torch.Generator(device="cuda").manual_seed(cols + k)
    sc = torch.randint(0, 2000, (rows, cols), generator=g, device="cuda").float()  # many ties
    kk = min(k, cols)
    ws, wi = _want(sc, kk)
    s, i = _ops.topk_rows(sc, k)
    assert torch.equal(s[:, :kk], ws) and torch.equal(i[:, :kk], wi)
    if k > cols:
        assert (i[:, cols:] == -1).all()
    out = None
    for s0 in range(0, cols, 4096):
        out = _ops.topk_rows(sc[:, s0:s0 + 4096].contiguous(), k, index_offset=s0, out=out)
    assert torch.equal(out[0][:, :kk], ws) and torch.equal(out[1][:, :kk], wi)
    s, i = _ops.topk_rows(sc, k, largest=False)
    ws, wi = _want(sc, kk, largest=False)
    assert torch.equal(s[:, :kk], ws) and torch.equal(i[:, :kk], wi)


def test_merge_of_lists_with_large_k():
    from late_interaction_kernels_b200 import _ops

    g = torch.Generator(device="cuda").manual_seed(5)
    k, n_lists, rows = 3000, 3, 2
    sc = torch.randint(0, 500, (rows, n_lists * 5000), generator=g, device="cuda").float()
    parts = [_ops.topk_rows(sc[:, j * 5000:(j + 1) * 5000].contiguous(), k, index_offset=j * 5000) for j in range(n_lists)]
    cs = torch.stack([p[0] for p in parts])
    ci = torch.stack([p[1] for p in parts])
    s, i = _ops.topk_merge(cs, ci, k)
    ws, wi = _want(sc, k)
    assert torch.equal(s, ws) and torch.equal(i, wi)


def test_maxsim_topk_with_k_above_1024():
    import late_interaction_kernels_b200 as lik

    g = torch.Generator(device="cuda").manual_seed(3)
    Q = torch.nn.functional.normalize(torch.randn((2, 8, 64), generator=g, device="cuda"), dim=-1).bfloat16()
    D = torch.nn.functional.normalize(torch.randn((3000, 12, 64), generator=g, device="cuda"), dim=-1).bfloat16()
    from late_interaction_kernels_b200.topk import maxsim_topk

    s, i = maxsim_topk(Q, D, 2000, chunk_size=1024)
    full = lik.maxsim(Q, D)
    ws, wi = _want(full, 2000)
    assert torch.equal(s, ws) and torch.equal(i, wi)
