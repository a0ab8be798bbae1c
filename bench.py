"""Benchmark of the MaxSim hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference ...                       # the reference algorithm on host cores

Headline workload ("ColBERTv2-shaped in-batch training"): bf16 Q[512,32,128] and D[512,300,128] ~N(0,1)
L2-normalised, document lengths U[64,300] as a boolean d_mask, full q_mask, one step = forward + backward
(gradients w.r.t. Q and D) through the autograd path.  Inputs are seeded synthetic data.  With N > 1 every
rank runs its own replica of the step (MaxSim training does not shard; data parallelism is the caller's),
so the whole-job figure is N times the per-rank work over the slowest rank's time ("weak" scaling).

Metric: TFLOP/s counting only algorithmic work on valid tokens:
    forward  2 * d * sum_{(i,j)} lq_i * ld_j        backward  4 * d * sum_{(i,j)} lq_i
Before anything is timed a sampled block of scores and gradients is compared with the CPU oracle; the run
stops if it is off.  One JSON line is printed by rank 0; `extra` carries the retrieve / PLAID / other-shape
legs, each with the roofline that bounds it.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

_JSON_OUT = None  # the process's original stdout once main() has redirected descriptor 1 (see there)


def emit(obj):
    out = _JSON_OUT if _JSON_OUT is not None else sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


METRIC = "MaxSim fwd+bwd TFLOP/s (bf16)"
WORKLOAD = "colbert_inbatch_train_bf16: Q[512,32,128] x D[512,300,128], d_len U[64,300], fwd+bwd"
NQ, ND, LQ, LD, DIM = 512, 512, 32, 300, 128
CHUNK = 4096  # documents per seeded chunk of the synthetic corpora


def make_inputs(seed=0):
    rng = np.random.default_rng(seed)
    Q = rng.standard_normal((NQ, LQ, DIM), dtype=np.float32)
    D = rng.standard_normal((ND, LD, DIM), dtype=np.float32)
    Q /= np.linalg.norm(Q, axis=-1, keepdims=True)
    D /= np.linalg.norm(D, axis=-1, keepdims=True)
    lens = rng.integers(64, LD + 1, size=ND)
    dm = np.arange(LD)[None, :] < lens[:, None]
    g = rng.standard_normal((NQ, ND), dtype=np.float32)
    return Q, D, dm, lens, g


def flops_of(lens, n_q=NQ, lq=LQ):
    fwd = 2.0 * DIM * n_q * lq * float(lens.sum())
    bwd = 4.0 * DIM * n_q * lq * len(lens)
    return fwd, bwd


def measured_peaks(sustained=False):
    """(bf16 TFLOP/s, HBM GB/s, source).  `sustained`: the cuBLAS figure of a seconds-long loop under the power cap,
    the denominator for a leg that itself runs for seconds; otherwise the burst figure, for a kernel timed alone."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        tf = float(d.get("bf16_tflops_sustained", d["bf16_tflops"])) if sustained else float(d["bf16_tflops"])
        return tf, float(d["hbm_gbs"]), "measured (sustained)" if sustained else "measured"
    return (1400.0 if sustained else 1590.0), 6650.0, "fallback"


def profiled_traffic(kernel_key):
    """DRAM bytes per launch of a kernel from the committed ncu capture (profiles/dram_traffic.json); None when
    that capture is absent."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(p) as f:
            return json.load(f).get(kernel_key)
    except (OSError, ValueError):
        return None


def scaled_traffic(kernel_key, units):
    """DRAM bytes of a launch from a capture of a smaller case of the same kernel: the committed figure is per unit
    (document, token) and traffic grows in proportion to the units."""
    per = profiled_traffic(kernel_key)
    return None if per is None else per * float(units)


def roofline(bound, work, seconds, *, kernel, note=None, traffic=None, sustained=False):
    """One roofline entry: achieved = algorithmic FLOPs (bound "tensor") or bytes (bound "hbm") / time."""
    peak_tf, peak_gb, which = measured_peaks(sustained)
    if bound == "tensor":
        achieved, peak, unit = work / seconds / 1e12, peak_tf, "TFLOP/s"
    else:
        achieved, peak, unit = work / seconds / 1e9, peak_gb, "GB/s"
    r = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": traffic,
         "kernel": kernel, "kernel_ms": seconds * 1e3, "peak_source": which, "algorithmic_work": work}
    if note:
        r["note"] = note
    return r


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self._proc = None
        self._t = None

    def _run(self):
        try:
            for line in self._proc.stdout:
                if line.strip():
                    self.rows.append([c.strip() for c in line.split(",")])
        except Exception:  # noqa: BLE001
            pass

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
            time.sleep(0.3)  # let the first sample arrive
        except Exception:  # noqa: BLE001
            self._proc = None
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:  # noqa: BLE001
                self._proc.kill()
            if self._t is not None:
                self._t.join(timeout=5)

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:  # noqa: BLE001
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------------------
# CPU legs (the oracle = the reference algorithm restated in numpy; the only place bench.py runs it)
# --------------------------------------------------------------------------------------------------------
def cpu_reference_step(sample_q, Q, D, dm, g):
    """One forward + backward of the reference algorithm on the first `sample_q` queries against all documents."""
    from oracle import maxsim_oracle as O

    s = O.maxsim(Q[:sample_q], D, None, dm)
    gq, gd = O.maxsim_grads(g[:sample_q], Q[:sample_q], D, None, dm)
    return float(s.sum()) + float(gq.sum()) + float(gd.sum())


def _best_of(fn, reps, budget_s):
    fn()
    best, n, t_all = float("inf"), 0, time.perf_counter()
    while n < reps and (n == 0 or time.perf_counter() - t_all < budget_s):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
        n += 1
    return best, n


def cpu_other_workloads():
    """The other workload shapes on host cores, each bounded to a few seconds (oracle port, all host threads)."""
    from oracle import maxsim_oracle as O

    out = {}
    rng = np.random.default_rng(0)
    # fp32 in-batch forward with both masks and fused normalisation, in full
    Q = rng.standard_normal((32, 32, 128)).astype(np.float32)
    D = rng.standard_normal((32, 180, 128)).astype(np.float32)
    qm = np.arange(32)[None] < rng.integers(8, 33, size=32)[:, None]
    dmk = np.arange(180)[None] < rng.integers(32, 181, size=32)[:, None]
    t, n = _best_of(lambda: O.maxsim(Q, D, qm, dmk, normalize=True), 5, 5.0)
    fl = 2.0 * 128 * float(qm.sum()) * float(dmk.sum())
    out["inbatch_fp32_fwd_32x32"] = {"ms": t * 1e3, "tflops_valid": fl / t / 1e12, "sample": f"whole workload, best of {n}"}
    # KD layout forward, in full
    Qk = rng.standard_normal((64, 32, 128)).astype(np.float32)
    Dk = rng.standard_normal((64, 32, 300, 128)).astype(np.float32)
    lk = rng.integers(64, 301, size=(64, 32))
    dk = np.arange(300)[None, None] < lk[..., None]
    t, n = _best_of(lambda: O.maxsim_kd(Qk, Dk, None, dk), 2, 8.0)
    out["kd_fwd_64x32"] = {"ms": t * 1e3, "tflops_valid": 2.0 * 128 * 32 * float(lk.sum()) / t / 1e12, "sample": f"whole workload, best of {n}"}
    # packed ColPali shape: 16 x 16 of the 128 x 128 pairs, forward + backward
    ql = rng.integers(16, 33, size=16)
    dl = rng.integers(900, 1031, size=16)
    Qp = rng.standard_normal((int(ql.sum()), 128)).astype(np.float32)
    Dp = rng.standard_normal((int(dl.sum()), 128)).astype(np.float32)
    cq, cd = np.concatenate([[0], np.cumsum(ql)]), np.concatenate([[0], np.cumsum(dl)])
    gg = rng.standard_normal((16, 16)).astype(np.float32)

    def packed():
        O.maxsim_varlen(Qp, Dp, cq, cd)
        O.varlen_grads(gg, Qp, Dp, cq, cd)

    t, n = _best_of(packed, 2, 8.0)
    fl = 2.0 * 128 * float(ql.sum()) * float(dl.sum()) + 4.0 * 128 * float(ql.sum()) * 16
    out["packed_colpali_fwd_bwd"] = {"ms": t * 1e3, "tflops_valid": fl / t / 1e12, "sample": f"16 x 16 of 128 x 128 pairs, best of {n}"}
    # retrieve: 8 queries against one 4096-document chunk of the corpus, top-100
    Qr = rng.standard_normal((8, 32, 128)).astype(np.float32)
    Dr = rng.standard_normal((CHUNK, 300, 128)).astype(np.float32)
    lr = rng.integers(32, 301, size=CHUNK)
    dr = np.arange(300)[None] < lr[:, None]
    t, n = _best_of(lambda: O.retrieve(Qr, Dr, 100, d_mask=dr, normalize=False, chunk=1024), 1, 10.0)
    out["retrieve_chunk"] = {"ms": t * 1e3, "queries_per_s_on_4096_docs": 8 / t,
                             "queries_per_s_extrapolated_to_1M_docs": 8 / t * CHUNK / 1e6,
                             "sample": "8 queries x one 4096-document chunk, top-100 (the 1M figure is an extrapolation)"}
    return out


def run_reference(args, rank):
    if rank != 0:
        return
    Q, D, dm, lens, g = make_inputs()
    sample_q = 16
    fwd, bwd = flops_of(lens, n_q=sample_q)
    for _ in range(max(args.warmup, 0) and 1):
        cpu_reference_step(sample_q, Q, D, dm, g)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(sample_q, Q, D, dm, g)
    dt = time.perf_counter() - t0
    val = (fwd + bwd) * args.steps / dt / 1e12
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"first {sample_q} of {NQ} queries against all {ND} documents per step"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"{sample_q} queries x {ND} docs fwd+bwd per step, numpy (OpenBLAS, all host threads)"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------------
# Parity before timing
# --------------------------------------------------------------------------------------------------------
def assert_step_parity(lik, dQ, dD, dM, dG, Q, D, dm, g):
    """Sampled scores and gradients of the timed step against the oracle (bf16 tolerance 2e-2).  Raises SystemExit."""
    import torch

    from oracle import maxsim_oracle as O

    f32 = lambda t: t.detach().float().cpu().numpy()  # noqa: E731
    Qt, Dt = dQ.clone().requires_grad_(), dD.clone().requires_grad_()
    s = lik.maxsim(Qt, Dt, d_mask=dM)
    qi = [0, 1, 255, 511]
    gm = torch.zeros_like(dG)
    gm[qi] = dG[qi]
    s.backward(gm)
    Qr, Dr = f32(dQ), f32(dD)
    errs = {"scores": O.rel_err(f32(s)[:8, :16], O.maxsim(Qr[:8], Dr[:16], None, dm[:16]))}
    wq, wd = O.maxsim_grads(g[qi], Qr[qi], Dr, None, dm)
    errs["grad_q"] = O.rel_err(f32(Qt.grad)[qi], wq)
    errs["grad_d"] = O.rel_err(f32(Dt.grad), wd)
    bad = {k: v for k, v in errs.items() if not v < 2e-2}
    if bad:
        raise SystemExit(f"bench.py: parity check failed before timing: {bad}")
    return errs


def verify_topk(Q, score_docs, n_docs, result, *, n_queries=4, n_random=2000, tol=2e-2, seed=0):
    """Re-score, on the CPU oracle, the returned top-k of a few queries plus random documents: the returned
    scores must match, and no sampled document outside the list may beat its k-th score by more than the
    tolerance.  `score_docs(q_rows, doc_ids)` -> oracle scores [len(q_rows), len(doc_ids)]."""
    s, i = result
    rng = np.random.default_rng(seed)
    qs = sorted(rng.choice(s.shape[0], size=min(n_queries, s.shape[0]), replace=False).tolist())
    worst = {"score_rel_err": 0.0, "outsider_margin": -float("inf")}
    for q in qs:
        top = i[q].cpu().numpy()
        rand = rng.choice(n_docs, size=min(n_random, n_docs), replace=False)
        ids = np.unique(np.concatenate([top, rand]))
        sc = score_docs([q], ids)[0]
        pos = {int(d): n for n, d in enumerate(ids)}
        got = s[q].cpu().numpy()
        want = np.array([sc[pos[int(d)]] for d in top])
        scale = max(1e-6, float(np.abs(want).max()))
        worst["score_rel_err"] = max(worst["score_rel_err"], float(np.abs(got - want).max() / scale))
        kth = float(want.min())
        outsiders = np.setdiff1d(ids, top)
        if outsiders.size:
            best_out = max(float(sc[pos[int(d)]]) for d in outsiders)
            worst["outsider_margin"] = max(worst["outsider_margin"], (best_out - kth) / scale)
    if not worst["score_rel_err"] < tol or not worst["outsider_margin"] < tol:
        raise SystemExit(f"bench.py: retrieve verification failed: {worst}")
    worst["queries_checked"] = len(qs)
    worst["random_docs_per_query"] = int(min(n_random, n_docs))
    return worst


# --------------------------------------------------------------------------------------------------------
# Seeded synthetic corpora (chunk-addressable: any rank can build any chunk; the tests use the same ones)
# --------------------------------------------------------------------------------------------------------
def dense_corpus(lo, hi, dev, Ld=300, d=DIM):
    """Documents [lo, hi) of the dense corpus: bf16 [n, Ld, d] L2-normalised rows and lengths U[32, Ld]."""
    import torch

    nd = hi - lo
    D = torch.empty((nd, Ld, d), dtype=torch.bfloat16, device=dev)
    lens = torch.empty(nd, dtype=torch.int64, device=dev)
    g = torch.Generator(device=dev)
    c = lo // CHUNK
    while c * CHUNK < hi:
        a, b = c * CHUNK, (c + 1) * CHUNK
        g.manual_seed(1234 + c)
        x = torch.randn((CHUNK, Ld, d), generator=g, device=dev, dtype=torch.float32)
        ln = torch.randint(32, Ld + 1, (CHUNK,), generator=g, device=dev)
        s0, s1 = max(a, lo), min(b, hi)
        D[s0 - lo:s1 - lo] = torch.nn.functional.normalize(x[s0 - a:s1 - a], dim=-1).to(torch.bfloat16)
        lens[s0 - lo:s1 - lo] = ln[s0 - a:s1 - a]
        c += 1
    return D, lens


def plaid_corpus(lo, hi, dev, d=DIM):
    """Documents [lo, hi) of the PLAID corpus: lengths U[32,300], uniform codes over 65536 centroids, uniform 2-bit
    residual bytes; returns (codes int32 [T], residuals uint8 [T, d/4], lens int64 [n])."""
    import torch

    g = torch.Generator(device=dev)
    codes, res, lens = [], [], []
    c = lo // CHUNK
    while c * CHUNK < hi:
        a, b = c * CHUNK, (c + 1) * CHUNK
        g.manual_seed(4321 + c)
        ln = torch.randint(32, 301, (CHUNK,), generator=g, device=dev)
        T = int(ln.sum())
        cc = torch.randint(0, 65536, (T,), generator=g, device=dev, dtype=torch.int32)
        rr = torch.randint(0, 256, (T, d // 4), generator=g, device=dev, dtype=torch.uint8)
        s0, s1 = max(a, lo), min(b, hi)
        cu = torch.nn.functional.pad(ln.cumsum(0), (1, 0))
        t0, t1 = int(cu[s0 - a]), int(cu[s1 - a])
        codes.append(cc[t0:t1])
        res.append(rr[t0:t1])
        lens.append(ln[s0 - a:s1 - a])
        c += 1
    return torch.cat(codes), torch.cat(res), torch.cat(lens)


def plaid_tables(dev, d=DIM):
    import torch

    g = torch.Generator(device=dev).manual_seed(5)
    cent = torch.nn.functional.normalize(torch.randn((65536, d), generator=g, device=dev), dim=-1).half()
    bw = torch.linspace(-0.1, 0.1, 4, device=dev)
    return cent, bw


def retrieve_queries(n, dev, d=DIM):
    import torch

    g = torch.Generator(device=dev).manual_seed(99)
    return torch.nn.functional.normalize(torch.randn((n, 32, d), generator=g, device=dev), dim=-1).to(torch.bfloat16)


def _timed(run, dev, reps, world):
    """Device time of run() per repetition: every repetition between its own event pair, max over ranks per repetition."""
    import torch
    import torch.distributed as dist

    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    last = None
    for a, b in ev:
        a.record()
        last = run()
        b.record()
    torch.cuda.synchronize(dev)
    t = torch.tensor([a.elapsed_time(b) for a, b in ev], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.cpu().numpy()
    return float(ms.min()), float(np.median(ms)), last


def retrieve_bench(n_docs, world, rank, dev, verify):
    """Sharded top-k retrieve: `n_docs` documents of U[32,300] tokens, d=128, bf16 normalised, split by document over
    the ranks; 1024 queries x 32 tokens, top_k=100.  Strong scaling: the corpus is fixed, every rank scores its slice
    in one pass of the fused scoring + top-k kernel, then one all-gather + merge."""
    import torch
    import torch.distributed as dist

    from late_interaction_kernels_b200 import _lib, sharded

    lo, hi = sharded.shard_bounds(n_docs, world, rank)
    D, lens = dense_corpus(lo, hi, dev)
    dm = torch.arange(300, device=dev)[None, :] < lens[:, None]
    Q = retrieve_queries(1024, dev)
    valid_tokens = torch.tensor([float(lens.sum())], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(valid_tokens)
    n_tok = float(valid_tokens.item())

    def run(q=Q, normalize=False):
        return sharded.retrieve_sharded(q, D, 100, d_mask=dm, doc_offset=lo, n_docs_total=n_docs, normalize=normalize, chunk=CHUNK)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    lib = _lib.load()
    n0 = lib.lik_launch_count()
    res = run()
    launches = lib.lik_launch_count() - n0
    barrier()
    with ClockSampler(dev.index or 0) as clk:
        ms_min, ms_med, res = _timed(run, dev, 3, world)
    flops = 2.0 * DIM * 1024 * 32 * n_tok
    out = {"metric": "retrieve queries/s", "value": 1024 / (ms_med * 1e-3), "unit": "queries/s", "ms_per_batch": ms_med,
           "ms_per_batch_min": ms_min, "repetitions": 3, "n_docs": n_docs, "queries": 1024, "top_k": 100, "scaling": "strong",
           "tflops_valid": flops / (ms_med * 1e-3) / 1e12, "launches_per_batch_per_rank": int(launches),
           "clocks": clk.summary(),
           "roofline": roofline("tensor", flops / world, ms_med * 1e-3, kernel="fwd_tc_kernel (bf16, fused top-k)", sustained=True,
                                traffic=scaled_traffic("fwd_tc_kernel_topk_per_document", n_docs / world),
                                note="per GPU: valid FLOPs of the shard over the batch time; one kernel runs for the whole "
                                     "batch, so the power cap sets the clock and the sustained cuBLAS figure is the peak")}
    # the default of retrieve(): fused L2 normalisation of both sides
    barrier()
    run(normalize=True)
    ms_min, ms_med, _ = _timed(lambda: run(normalize=True), dev, 2, world)
    out["normalize_true"] = {"ms_per_batch": ms_med, "queries_per_s": 1024 / (ms_med * 1e-3), "tflops_valid": flops / (ms_med * 1e-3) / 1e12}
    # end to end: queries from pinned host memory, [Nq, k] scores and indices back to the host
    hQ = Q.cpu().pin_memory()
    hS = torch.empty((1024, 100), dtype=torch.float32).pin_memory()
    hI = torch.empty((1024, 100), dtype=torch.int64).pin_memory()
    dQ = torch.empty_like(Q)

    def e2e():
        dQ.copy_(hQ, non_blocking=True)
        s, i = run(q=dQ)
        hS.copy_(s, non_blocking=True)
        hI.copy_(i, non_blocking=True)
        return s, i

    e2e()
    barrier()
    ms_min, ms_med, _ = _timed(e2e, dev, 2, world)
    out["e2e"] = {"value": 1024 / (ms_med * 1e-3), "unit": "queries/s", "h2d_bytes_per_batch": hQ.numel() * 2,
                  "d2h_bytes_per_batch": hS.numel() * 4 + hI.numel() * 8}
    # few queries: the documents are read once, so the bound is HBM
    if world == 1:
        Q8 = retrieve_queries(8, dev)
        run(q=Q8)
        ms_min, ms_med, _ = _timed(lambda: run(q=Q8), dev, 3, world)
        out["eight_queries"] = {"ms_per_batch": ms_med, "queries_per_s": 8 / (ms_med * 1e-3),
                                "roofline": roofline("hbm", n_tok * DIM * 2, ms_med * 1e-3, kernel="fwd_tc_kernel (bf16, fused top-k)",
                                                     note="valid document bytes read once; 256 rows of queries make it tensor work "
                                                          "at the same time (256 FLOP per byte)")}
    if verify and world == 1:
        from oracle import maxsim_oracle as O

        Qh = Q.float().cpu().numpy()

        def score_docs(q_rows, ids):
            sub = D[torch.as_tensor(ids, device=dev)].float().cpu().numpy()
            sm = dm[torch.as_tensor(ids, device=dev)].cpu().numpy()
            return O.maxsim(Qh[q_rows], sub, None, sm)

        out["verified"] = verify_topk(Q, score_docs, n_docs, res)
    out["best_index_q0"] = int(res[1][0, 0])
    return out


def plaid_retrieve_bench(n_docs, world, rank, dev, verify):
    """Sharded top-k over a PLAID index (2-bit residuals, d=128, 65536 fp16 centroids): 1024 queries, top-100.  With
    this many queries every token is decoded once per call, in pieces, and the scoring kernel carries its candidate
    lists from piece to piece."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from late_interaction_kernels_b200 import sharded

    lo, hi = sharded.shard_bounds(n_docs, world, rank)
    codes, res, lens = plaid_corpus(lo, hi, dev)
    T = int(codes.numel())
    cu = F.pad(lens.cumsum(0), (1, 0)).int()
    cent, bw = plaid_tables(dev)
    Q = retrieve_queries(1024, dev)
    lens_host = lens.cpu()
    tok = torch.tensor([float(T)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tok)
    n_tok = float(tok.item())

    def run():
        return sharded.retrieve_plaid_sharded(Q, codes, res, cu, cent, bw, 2, 100, doc_offset=lo, n_docs_total=n_docs, chunk=16 * CHUNK,
                                              doc_lengths_host=lens_host)

    out_res = run()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms_min, ms_med, out_res = _timed(run, dev, 3, world)
    flops = 2.0 * DIM * 1024 * 32 * n_tok
    out = {"metric": "PLAID retrieve queries/s", "value": 1024 / (ms_med * 1e-3), "unit": "queries/s", "ms_per_batch": ms_med,
           "ms_per_batch_min": ms_min, "repetitions": 3, "n_docs": n_docs, "queries": 1024, "top_k": 100, "nbits": 2, "scaling": "strong",
           "tflops_valid": flops / (ms_med * 1e-3) / 1e12,
           "roofline": roofline("tensor", flops / world, ms_med * 1e-3, kernel="plaid_decompress16_kernel + fwd_tc_kernel (fused top-k)",
                                sustained=True,
                                note="per GPU; 128 query-tile groups share every decoded token, so the tensor pipe bounds it")}
    if verify and world == 1:
        from oracle import maxsim_oracle as O

        Qh = Q.float().cpu().numpy()
        cu_h = F.pad(lens_host.cumsum(0), (1, 0)).numpy()
        cent_h, bw_h = cent.float().cpu().numpy(), bw.cpu().numpy()

        def score_docs(q_rows, ids):
            cs, rs, ls = [], [], []
            for j in ids:
                a, b = int(cu_h[j]), int(cu_h[j + 1])
                cs.append(codes[a:b])
                rs.append(res[a:b])
                ls.append(b - a)
            cc, rr = torch.cat(cs).cpu().numpy(), torch.cat(rs).cpu().numpy()
            c2 = np.concatenate([[0], np.cumsum(ls)])
            emb = torch.from_numpy(O.plaid_decompress(cc, rr, cent_h, bw_h, 2)).to(torch.bfloat16).float().numpy()
            outp = np.zeros((len(q_rows), len(ids)), np.float32)
            for n in range(len(ids)):
                dj = emb[c2[n]:c2[n + 1]]
                outp[:, n] = np.einsum("isd,td->ist", Qh[q_rows], dj).max(-1).sum(-1)
            return outp

        out["verified"] = verify_topk(Q, score_docs, n_docs, out_res, n_random=1000)
    return out


def _time_us(fn, dev, iters=10, warm=3, graph=False):
    """Mean device time of fn() in microseconds.  With graph=True the call is captured once into a CUDA
    graph and replayed, so that host launch overhead does not hide the device time of a small problem."""
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize(dev)
    run = fn
    if graph:
        try:
            st = torch.cuda.Stream(dev)
            with torch.cuda.stream(st):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    fn()
            run = gr.replay
            run()
            torch.cuda.synchronize(dev)
        except Exception:  # noqa: BLE001  (not capturable: time it eagerly)
            torch.cuda.synchronize(dev)
            run = fn
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1) / iters * 1e3


def hidden_inputs(n_q, n_d, ld, dev, d_model=768, d_out=128):
    """Inputs of maxsim_from_hidden at the reference's ModernBERT-base head shape (benchmarks/kernels/
    bench_fused_head_train.py:53-66): hidden states [n_d, ld, 768] -> 128, 32-token queries, bf16."""
    import torch
    import torch.nn.functional as F

    g = torch.Generator(device=dev).manual_seed(11)
    H = torch.randn((n_d, ld, d_model), generator=g, device=dev).bfloat16()
    W = (torch.randn((d_out, d_model), generator=g, device=dev) / d_model ** 0.5).bfloat16()
    b = (0.1 * torch.randn((d_out,), generator=g, device=dev)).bfloat16()
    Q = F.normalize(torch.randn((n_q, 32, d_out), generator=g, device=dev), dim=-1).bfloat16()
    return Q, H, W, b


def other_configs(dev):
    """Kernel timings of the other workload shapes (rank 0, one GPU), each with the roofline that bounds it: the KD
    layout in bf16 and e4m3 (HBM: document bytes read once), the packed ColPali-shaped batch forward and forward +
    backward (tensor: valid FLOPs), the PLAID candidate score, decode kernel and few-query rerank (HBM: compressed
    bytes), and the per-row top-k kernel (HBM: score bytes)."""
    import torch
    import torch.nn.functional as F

    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import _ops, fp8, plaid

    out = {}
    g = torch.Generator(device=dev).manual_seed(7)
    # the small fp32 case (the one the CPU oracle runs in full): Q[32,32,128] x D[32,180,128], fused normalisation, ragged both sides
    Qf = torch.randn((32, 32, 128), generator=g, device=dev)
    Df = torch.randn((32, 180, 128), generator=g, device=dev)
    qlf = torch.randint(8, 33, (32,), generator=g, device=dev)
    dlf = torch.randint(32, 181, (32,), generator=g, device=dev)
    qmf = torch.arange(32, device=dev)[None, :] < qlf[:, None]
    dmf = torch.arange(180, device=dev)[None, :] < dlf[:, None]
    t = _time_us(lambda: lik.maxsim(Qf, Df, q_mask=qmf, d_mask=dmf, normalize=True), dev, graph=True)
    flf = 2.0 * 128 * float(qlf.sum()) * float(dlf.sum())
    out["inbatch_fp32_fwd_32x32"] = {"us": t, "shape": "fp32 Q[32,32,128] x D[32,180,128], normalize, q U[8,32], d U[32,180]",
                                     "tflops_valid": flf / (t * 1e-6) / 1e12,
                                     "note": "exact fp32-FMA kernel (fwd_generic_kernel); a launch-latency-sized problem"}
    # KD: Q[64,32,128] x D[64,32,300,128], lengths U[64,300] per candidate
    Q = F.normalize(torch.randn((64, 32, 128), generator=g, device=dev), dim=-1)
    D = F.normalize(torch.randn((64, 32, 300, 128), generator=g, device=dev), dim=-1)
    lens = torch.randint(64, 301, (64, 32), generator=g, device=dev)
    dm = torch.arange(300, device=dev)[None, None, :] < lens[..., None]
    valid = float(lens.sum())
    qb, db = Q.bfloat16(), D.bfloat16()
    t = _time_us(lambda: lik.maxsim(qb, db, d_mask=dm), dev, graph=True)
    out["kd_bf16_fwd"] = {"us": t, "shape": "Q[64,32,128] x D[64,32,300,128]",
                          "roofline": roofline("hbm", valid * 256 + qb.numel() * 2, t * 1e-6, kernel="fwd_tc_kernel (grouped)",
                                               note="valid document rows + queries, read once")}
    q8, sq = fp8.quantize_fp8_per_token(Q)
    d8, sd = fp8.quantize_fp8_per_token(D)
    t = _time_us(lambda: fp8.maxsim_inference_fp8(q8, d8, scale_Q=sq, scale_D=sd, d_mask=dm), dev, graph=True)
    out["kd_e4m3_fwd"] = {"us": t, "roofline": roofline("hbm", valid * (128 + 4) + q8.numel(), t * 1e-6, kernel="fwd_tc_kernel (e4m3, grouped)",
                                                        note="valid e4m3 rows + their fp32 scales, read once")}
    del D, db, d8
    # packed: 128 queries of U[16,32] tokens x 128 documents of U[900,1030] tokens
    ql = torch.randint(16, 33, (128,), generator=g, device=dev)
    dl = torch.randint(900, 1031, (128,), generator=g, device=dev)
    cq = F.pad(ql.cumsum(0), (1, 0)).int()
    cd = F.pad(dl.cumsum(0), (1, 0)).int()
    Qp = F.normalize(torch.randn((int(ql.sum()), 128), generator=g, device=dev), dim=-1).bfloat16()
    Dp = F.normalize(torch.randn((int(dl.sum()), 128), generator=g, device=dev), dim=-1).bfloat16()
    fl = 2.0 * 128 * float(ql.sum()) * float(dl.sum())
    t = _time_us(lambda: lik.maxsim_varlen(Qp, Dp, cq, cd, 32, 1030), dev, graph=True)
    out["varlen_fwd"] = {"us": t, "shape": "128 q U[16,32] x 128 docs U[900,1030]",
                         "roofline": roofline("tensor", fl, t * 1e-6, kernel="fwd_tc_kernel (packed)")}
    Qr, Dr = Qp.clone().requires_grad_(), Dp.clone().requires_grad_()
    go = torch.randn((128, 128), generator=g, device=dev)

    def fb():
        Qr.grad = None
        Dr.grad = None
        lik.maxsim_varlen(Qr, Dr, cq, cd, 32, 1030).backward(go)

    t = _time_us(fb, dev, graph=True)
    flb = fl + 4.0 * 128 * float(ql.sum()) * 128
    out["varlen_fwd_bwd"] = {"us": t, "timed": "CUDA-graph replay of forward + backward",
                             "roofline": roofline("tensor", flb, t * 1e-6, kernel="fwd_tc_kernel + bwd_dq16 + bwd_dd_sort4 + bwd_dd_reduce16",
                                                  note="the 60 % target is quoted on this shape")}
    # PLAID candidate score: 65536 centroids, 8192 candidate documents of up to 300 codes
    qcs = torch.randn((65536, 32), generator=g, device=dev)
    codes = torch.randint(0, 65536, (8192, 300), generator=g, device=dev, dtype=torch.int32)
    cl = torch.randint(32, 301, (8192,), generator=g, device=dev)
    t = _time_us(lambda: plaid.plaid_approx_score(qcs, codes, cl), dev, graph=True)
    out["plaid_approx"] = {"us": t, "shape": "8192 docs x <=300 codes, 32 query tokens",
                           "roofline": roofline("hbm", float(cl.sum()) * 4, t * 1e-6, kernel="plaid_approx_kernel",
                                                note="code bytes only: the 8.4 MB score table stays in L2, its rows are not HBM traffic")}
    # PLAID: decode kernel alone, and the few-query rerank (the reference's published PLAID shape: one query x 10k / 25k docs)
    cent, bw = plaid_tables(dev)
    for nd in (10_000, 25_000):
        pc, pr, pl_ = plaid_corpus(0, nd, dev)
        pcu = F.pad(pl_.cumsum(0), (1, 0)).int()
        T = int(pc.numel())
        if nd == 25_000:
            ix, keep = _ops.plaid_index(pc, pr, cent, bw, 2, 128)
            t = _time_us(lambda: _ops.plaid_decompress(ix, 0, T, True, torch.bfloat16, dev), dev)
            out["plaid_decompress"] = {"us": t, "tokens": T,
                                       "roofline": roofline("hbm", T * (36.0 + 256.0), t * 1e-6, kernel="plaid_decompress16_kernel",
                                                            traffic=scaled_traffic("plaid_decompress16_kernel_per_token", T),
                                                            note="4 B code + 32 B residual in, 256 B bf16 row out per token")}
        for nq in (1, 8, 32):
            Qq = retrieve_queries(nq, dev)
            t = _time_us(lambda: plaid.retrieve_residual_varlen(Qq, pc, pr, pcu, cent, bw, 2, 10), dev, iters=5)
            out[f"plaid_top10_{nq}q_{nd // 1000}k_docs"] = {
                "us": t, "tokens": T,
                "roofline": roofline("hbm", T * 36.0, t * 1e-6, kernel="plaid_decompress16_kernel + fwd_tc_kernel (fused top-k) + topk_slots_kernel",
                                     note="compressed bytes (36 B per token) read once; the decoded rows (256 B per token) are written and "
                                          "read back, and with 256 query rows the scoring is tensor work: HBM on compressed bytes is a loose bound")}
    # document head: 1 query x 1024 documents of 2048 hidden states (768 -> 128), the largest shape of the reference's
    # fused-head benchmark; forward alone, and the training step against projecting with F.linear first
    from late_interaction_kernels_b200.fused_head import maxsim_from_hidden
    hq, hh, hw, hb = hidden_inputs(1, 1024, 2048, dev)
    # parity before timing: the first documents against a projection in fp32 followed by the scorer
    got_h = maxsim_from_hidden(hq, hh, hw, hb)[:, :16].float()
    want_h = lik.maxsim(hq.float(), F.normalize(F.linear(hh[:16].float(), hw.float(), hb.float()), dim=-1))
    err_h = float((got_h - want_h).abs().max() / want_h.abs().max())
    if not err_h < 2e-2:
        raise SystemExit(f"maxsim_from_hidden differs from the fp32 projection + scorer: relative error {err_h:.3e}")
    t = _time_us(lambda: maxsim_from_hidden(hq, hh, hw, hb), dev)
    h_bytes = hh.numel() * 2.0
    out["hidden_head_fwd"] = {"us": t, "shape": "Q[1,32,128] x H[1024,2048,768] -> 128, bf16",
                              "roofline": roofline("hbm", h_bytes + hw.numel() * 2.0 + hq.numel() * 2.0 + 4.0 * 1024, t * 1e-6, kernel="head_tc_kernel",
                                                   traffic=scaled_traffic("head_tc_kernel_per_token", 1024 * 2048),
                                                   note="hidden states read once; the projected tokens stay on chip")}
    t_unf = _time_us(lambda: lik.maxsim(hq, F.normalize(F.linear(hh, hw, hb), dim=-1)), dev, iters=5)
    out["hidden_head_fwd"]["unfused_us"] = t_unf

    def head_step(fused):
        Hg, Wg, Qg = hh.detach().requires_grad_(True), hw.detach().requires_grad_(True), hq.detach().requires_grad_(True)
        sc_ = maxsim_from_hidden(Qg, Hg, Wg, hb) if fused else lik.maxsim(Qg, F.normalize(F.linear(Hg, Wg, hb), dim=-1))
        sc_.sum().backward()

    out["hidden_head_step"] = {"us": _time_us(lambda: head_step(True), dev, iters=5), "unfused_us": _time_us(lambda: head_step(False), dev, iters=3),
                               "note": "forward + backward into Q, H and W; the backward touches the winning rows and writes grad_H once"}
    del hh
    torch.cuda.empty_cache()
    # rerank shapes of the reference's FP8 table (benchmarks/kernels/bench_fp8.py:32-41): one or four queries against
    # thousands of short documents, bf16 and e4m3 with per-token scales; bound by the document bytes
    for label, nq_r, nd_r, ld_r in (("colbert_rerank_8k", 1, 8192, 256), ("batched_rerank_16k", 4, 4096, 256), ("long_docs_2k", 1, 2048, 512)):
        Qr_ = F.normalize(torch.randn((nq_r, 32, 128), generator=g, device=dev), dim=-1).bfloat16()
        Dr_ = F.normalize(torch.randn((nd_r, ld_r, 128), generator=g, device=dev), dim=-1).bfloat16()
        q8_, sq_ = fp8.quantize_fp8_per_token(Qr_)
        d8_, sd_ = fp8.quantize_fp8_per_token(Dr_)
        tb = _time_us(lambda: lik.maxsim(Qr_, Dr_), dev, graph=True)
        t8 = _time_us(lambda: fp8.maxsim_inference_fp8(q8_, d8_, scale_Q=sq_, scale_D=sd_), dev, graph=True)
        out[f"rerank_{label}"] = {
            "shape": f"Q[{nq_r},32,128] x D[{nd_r},{ld_r},128]", "bf16_us": tb, "e4m3_us": t8,
            "roofline": roofline("hbm", Dr_.numel() * 2.0, tb * 1e-6, kernel="fwd_tc_kernel (bf16, few queries)", note="document bytes read once"),
            "roofline_e4m3": roofline("hbm", d8_.numel() * 1.0 + sd_.numel() * 4.0, t8 * 1e-6, kernel="fwd_tc_kernel (e4m3, per-token scales)",
                                      note="e4m3 document bytes + fp32 scales read once")}
        del Dr_, d8_
    # long documents (the reference's benchmarks/kernels/bench_longdoc.py shapes, fp16): forward, forward with winners, backward
    for label, nq_l, nd_l, ld_l in (("train_8k", 8, 16, 8192), ("rerank_8k", 1, 256, 8192), ("huge_doc", 1, 32, 16384)):
        Ql = F.normalize(torch.randn((nq_l, 32, 128), generator=g, device=dev), dim=-1).half()
        Dl = F.normalize(torch.randn((nd_l, ld_l, 128), generator=g, device=dev), dim=-1).half()
        qsl, dsl = _ops.padded_spec(Ql), _ops.padded_spec(Dl)
        gl = torch.randn((nq_l, nd_l), generator=g, device=dev)
        _, aml = _ops.forward(qsl, dsl, save_argmax=True)
        tf = _time_us(lambda: _ops.forward(qsl, dsl), dev, graph=True)
        out[f"longdoc_{label}"] = {
            "shape": f"Q[{nq_l},32,128] x D[{nd_l},{ld_l},128] fp16", "fwd_us": tf,
            "fwd_winners_us": _time_us(lambda: _ops.forward(qsl, dsl, save_argmax=True), dev, graph=True),
            "bwd_us": _time_us(lambda: _ops.backward(qsl, dsl, gl, aml), dev, graph=True),
            "roofline": roofline("hbm", Dl.numel() * 2.0, tf * 1e-6, kernel="fwd_tc_kernel (fp16, few queries)",
                                 note=f"document bytes read once; a document is never split across CTAs, so {nd_l} documents keep "
                                      f"{min(nd_l, 148)} of the 148 SMs busy")}
        del Dl
    # cached-contrastive tile grid (the reference's docs/benchmarks.md:396-426: bs = 256, Lq = 128, mini = 32 -> 64 tiles,
    # forward + backward): the whole grid in one call against one call per tile
    from late_interaction_kernels_b200.loss_heads import maxsim_tiles
    for ld_cc in (2048, 8192):
        qc = [F.normalize(torch.randn((32, 128, 128), generator=g, device=dev), dim=-1).bfloat16().requires_grad_() for _ in range(8)]
        dc = [F.normalize(torch.randn((32, ld_cc, 128), generator=g, device=dev), dim=-1).bfloat16().requires_grad_() for _ in range(8)]
        gg = torch.randn((256, 256), generator=g, device=dev)

        def clear():
            for x in qc + dc:
                x.grad = None

        def grid_step():
            clear()
            maxsim_tiles(qc, dc).backward(gg)

        def tile_step():
            clear()
            for i_ in range(8):
                for j_ in range(8):
                    lik.maxsim(qc[i_], dc[j_]).backward(gg[32 * i_:32 * i_ + 32, 32 * j_:32 * j_ + 32])

        fl_cc = 2.0 * 128 * (256 * 128) * (256 * ld_cc)
        t = _time_us(grid_step, dev, iters=3, warm=2)
        out[f"cached_contrastive_bs256_ld{ld_cc}"] = {
            "us": t, "per_tile_calls_us": _time_us(tile_step, dev, iters=2, warm=1), "shape": f"bs 256, Lq 128, Ld {ld_cc}, d 128, 64 tiles of 32 x 32",
            "roofline": roofline("tensor", fl_cc + 4.0 * 128 * (256 * 128) * 256, t * 1e-6, sustained=ld_cc >= 8192,
                                 kernel="fwd_tc_kernel + bwd_dq16 + bwd_dd_sort4 + bwd_dd_reduce16 (+ the cat of the chunks and its backward)",
                                 note="forward + backward of the whole grid in one call (loss_heads.maxsim_tiles)")}
        del qc, dc
        torch.cuda.empty_cache()
    # per-row top-k kernel on a score matrix
    sc = torch.randn((1024, 4096), generator=g, device=dev)
    t = _time_us(lambda: _ops.topk_rows(sc, 100), dev, graph=True)
    out["topk_rows"] = {"us": t, "shape": "[1024, 4096] fp32 -> top-100",
                        "roofline": roofline("hbm", sc.numel() * 4.0, t * 1e-6, kernel="topk_select_kernel",
                                             traffic=profiled_traffic("topk_select_kernel_1024x4096"),
                                             note="one read of the scores; the kernel is bound by its radix-select passes "
                                                  "(shared-memory counters) and the sort of the k winners")}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--retrieve-docs", type=int, default=1_000_000,
                    help="corpus size of the sharded top-k retrieve reported under extra.retrieve (0 = skip)")
    ap.add_argument("--only", default=None, choices=["fwd", "fwd_infer", "bwd", "step", "retrieve", "plaid", "topk_rows", "decompress", "hidden"],
                    help="profiling aid: launch only this part, --steps times, and print its mean time")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    # stdout carries exactly one JSON line: libraries that write to file descriptor 1 on their own (NCCL's version
    # banner does) are sent to stderr for the whole run, and the line is written to the saved descriptor at the end
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import _lib, _ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # keep stdout for the one JSON line: NCCL's own log lines (version banner, warnings) go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    Q, D, dm, lens, g = make_inputs()
    fwd_flops, bwd_flops = flops_of(lens)
    hQ = torch.from_numpy(Q).to(torch.bfloat16).pin_memory()
    hD = torch.from_numpy(D).to(torch.bfloat16).pin_memory()
    hM = torch.from_numpy(dm).pin_memory()
    hG = torch.from_numpy(g).pin_memory()
    dQ, dD, dM, dG = hQ.to(dev), hD.to(dev), hM.to(dev), hG.to(dev)
    Qr, Dr = dQ.clone().requires_grad_(), dD.clone().requires_grad_()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2

    def step():
        Qr.grad = None
        Dr.grad = None
        s = lik.maxsim(Qr, Dr, d_mask=dM)
        s.backward(dG)
        return s

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.only:
        from late_interaction_kernels_b200 import plaid as plaid_mod
        from late_interaction_kernels_b200.backward import maxsim_backward_lowmem

        qs, ds = _ops.padded_spec(dQ), _ops.padded_spec(dD, dM)
        if args.only in ("fwd", "fwd_infer", "bwd", "step"):
            _, am = _ops.forward(qs, ds, save_argmax=True)
            part = {
                "fwd": lambda: _ops.forward(qs, ds, save_argmax=True),
                "fwd_infer": lambda: _ops.forward(qs, ds),
                "bwd": lambda: maxsim_backward_lowmem(dG, dQ, dD, am),
                "step": step,
            }[args.only]
        elif args.only == "retrieve":  # 1024 queries, fused top-k, over one 4096-document chunk (or the first --retrieve-docs documents)
            n_only = CHUNK if args.retrieve_docs >= 1_000_000 else max(args.retrieve_docs, 1)
            Dc, lc = dense_corpus(0, n_only, dev)
            mc = torch.arange(300, device=dev)[None, :] < lc[:, None]
            Qc = retrieve_queries(1024, dev)
            part = lambda: lik.retrieve(Qc, Dc, 100, d_mask=mc, normalize=False)  # noqa: E731
        elif args.only == "plaid":  # 8 queries x 25k compressed documents: decode inside the scoring kernel, fused top-k
            pc, pr, pl_ = plaid_corpus(0, 25_000, dev)
            pcu = torch.nn.functional.pad(pl_.cumsum(0), (1, 0)).int()
            cent, bw = plaid_tables(dev)
            Qc = retrieve_queries(8, dev)
            part = lambda: plaid_mod.retrieve_residual_varlen(Qc, pc, pr, pcu, cent, bw, 2, 10)  # noqa: E731
        elif args.only == "hidden":  # document head chained into MaxSim: 1 query x 128 documents of 2048 hidden states (0.4 GB)
            from late_interaction_kernels_b200.fused_head import maxsim_from_hidden
            hq, hh, hw, hb = hidden_inputs(1, 128, 2048, dev)
            part = lambda: maxsim_from_hidden(hq, hh, hw, hb)  # noqa: E731
        elif args.only == "decompress":
            pc, pr, pl_ = plaid_corpus(0, 25_000, dev)
            cent, bw = plaid_tables(dev)
            ix, keep = _ops.plaid_index(pc, pr, cent, bw, 2, 128)
            part = lambda: _ops.plaid_decompress(ix, 0, int(pc.numel()), True, torch.bfloat16, dev)  # noqa: E731
        else:
            sc = torch.randn((1024, 4096), device=dev)
            part = lambda: _ops.topk_rows(sc, 100)  # noqa: E731
        for _ in range(args.warmup):
            part()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            part()
        b.record()
        torch.cuda.synchronize()
        emit({"only": args.only, "ms": a.elapsed_time(b) / args.steps, "steps": args.steps})
        return

    parity = assert_step_parity(lik, dQ, dD, dM, dG, Q, D, dm, g) if rank == 0 else None

    for _ in range(args.warmup):
        step()
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        n_launch0 = lib.lik_launch_count()
        for a, b in ev:
            flush.zero_()
            a.record()
            step()
            b.record()
        n_launch = lib.lik_launch_count() - n_launch0
        barrier()
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    lik.check_device_status(dev)
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    value = world * (fwd_flops + bwd_flops) * args.steps / (total_ms * 1e-3) / 1e12

    # ---- end to end: host buffers in, results out, every step ----
    # Every step copies its own inputs from pinned host memory and its scores and gradients back.  The
    # copies of neighbouring steps overlap the compute of the current one (two device input sets, one
    # copy-in and one copy-out stream), as a training loop with a prefetching loader would run it.
    hS = torch.empty((NQ, ND), dtype=torch.float32).pin_memory()
    hGQ, hGD = torch.empty_like(hQ).pin_memory(), torch.empty_like(hD).pin_memory()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    cur = torch.cuda.current_stream(dev)
    sets = [[torch.empty_like(dQ), torch.empty_like(dD), torch.empty_like(dM), torch.empty_like(dG)] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = torch.cuda.Event()

    def stage_in(k):
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[k])  # the step that last used this input set has finished
            for dst, src in zip(sets[k], (hQ, hD, hM, hG)):
                dst.copy_(src, non_blocking=True)
            ev_in[k].record(s_in)

    def e2e_run(n):
        for k in range(2):
            ev_done[k].record(cur)
        ev_out.record(s_out)
        stage_in(0)
        for it in range(n):
            k = it & 1
            cur.wait_event(ev_in[k])
            if it + 1 < n:
                stage_in(k ^ 1)
            q = sets[k][0].detach().requires_grad_()
            d = sets[k][1].detach().requires_grad_()
            s = lik.maxsim(q, d, d_mask=sets[k][2])
            s.backward(sets[k][3])
            ev_done[k].record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                for t in (s, q.grad, d.grad):
                    t.record_stream(s_out)
                hS.copy_(s.detach(), non_blocking=True)
                hGQ.copy_(q.grad, non_blocking=True)
                hGD.copy_(d.grad, non_blocking=True)
                ev_out.record(s_out)
        cur.wait_event(ev_out)  # the timed region ends when the last results are on the host

    e2e_run(2)
    barrier()
    n_e2e = max(4, min(args.steps, 40))  # enough steps for the first copy-in and the last copy-out to be a small share
    # three repetitions, the fastest counts: the copies cross a host that other tenants of the machine share, and one
    # repetition in a few runs at a fraction of the usual rate (every repetition is the max over ranks)
    e2e_ms = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(n_e2e)
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms.append(float(te.item()))
    e2e_val = world * (fwd_flops + bwd_flops) * n_e2e / (min(e2e_ms) * 1e-3) / 1e12
    h2d = hQ.numel() * 2 + hD.numel() * 2 + hM.numel() + hG.numel() * 4
    d2h = hS.numel() * 4 + hGQ.numel() * 2 + hGD.numel() * 2

    # ---- roofline of the dominant kernel (the tcgen05 forward with argmax), timed alone; and of the backward ----
    qs, ds = _ops.padded_spec(dQ), _ops.padded_spec(dD, dM)

    def alone(fn, n=10):
        for _ in range(3):
            fn()
        fev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in fev:
            flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return float(np.mean([a.elapsed_time(b) for a, b in fev]))

    fwd_ms = alone(lambda: _ops.forward(qs, ds, save_argmax=True))
    infer_ms = alone(lambda: _ops.forward(qs, ds))
    _, am = _ops.forward(qs, ds, save_argmax=True)
    bwd_ms = alone(lambda: _ops.backward(qs, ds, dG, am))
    rows_valid = float(lens.sum())
    fwd_bytes = dQ.numel() * 2 + rows_valid * DIM * 2 + dM.numel() + NQ * ND * 4 + NQ * ND * LQ * 4
    bwd_bytes = dQ.numel() * 2 + rows_valid * DIM * 2 + NQ * ND * LQ * 4 + NQ * ND * 4 + dQ.numel() * 2 + dD.numel() * 2
    main_roof = roofline("tensor", fwd_flops, fwd_ms * 1e-3, kernel="fwd_tc_kernel (bf16, argmax, masked)",
                         traffic=profiled_traffic("fwd_tc_kernel_argmax_inbatch"))
    main_roof["traffic_unit"] = "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum; null when no capture is committed)"
    main_roof["algorithmic_bytes"] = fwd_bytes

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"replicas x{world}", "l2": "flushed between steps (256 MB write)",
                   "fwd_flops_per_step": fwd_flops, "bwd_flops_per_step": bwd_flops},
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": n_e2e, "repetitions_ms": e2e_ms, "note": "fastest of three repetitions of `steps` steps"},
        # kernels of this library launched inside the timed region (counted by the library, lik_launch_count)
        "gpu_launches": int(n_launch),
        "roofline": main_roof,
        "parity_before_timing": parity,
        "clocks": clocks.summary(),
        "extra": {
            "step_kernels": {
                "forward_no_argmax": roofline("tensor", fwd_flops, infer_ms * 1e-3, kernel="fwd_tc_kernel (bf16, masked)"),
                "backward": roofline("hbm", bwd_bytes, bwd_ms * 1e-3, kernel="bwd_dq16 + bwd_dd_sort4 + bwd_dd_reduce16",
                                     traffic=profiled_traffic("bwd_three_kernels_inbatch"),
                                     note="algorithmic bytes: Q, valid D rows, winners, upstream gradient in; both gradients out.  "
                                          "The kernels gather one 256-byte row per (pair, query token) out of L2, 34x these bytes"),
            },
        },
    }
    if args.retrieve_docs > 0:
        del Qr, Dr, flush, sets
        torch.cuda.empty_cache()
        line["extra"]["retrieve"] = retrieve_bench(args.retrieve_docs, world, rank, dev, verify=rank == 0)
        torch.cuda.empty_cache()
        line["extra"]["plaid_retrieve"] = plaid_retrieve_bench(args.retrieve_docs, world, rank, dev, verify=rank == 0)
        torch.cuda.empty_cache()
        if world == 1:
            line["extra"]["other_configs"] = other_configs(dev)
    lik.check_device_status(dev)
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            sample_q = 16
            cf, cb = flops_of(lens, n_q=sample_q)
            t0 = time.perf_counter()
            reps = 0
            while reps < 2 or (time.perf_counter() - t0 < 10 and reps < 50):
                cpu_reference_step(sample_q, Q, D, dm, g)
                reps += 1
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": (cf + cb) * reps / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count() or 1,
                                    "kind": "port", "sample": f"{reps} x ({sample_q} queries x {ND} docs fwd+bwd), numpy oracle, all host threads",
                                    "other_workloads": cpu_other_workloads()}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
