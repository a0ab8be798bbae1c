"""Benchmark of the MaxSim hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference ...                       # the reference algorithm on host cores

Workload (BASELINE config 2, "ColBERTv2-shaped in-batch training"): bf16 Q[512,32,128] and
D[512,300,128] ~N(0,1) L2-normalised, document lengths U[64,300] as a boolean d_mask, full q_mask,
one step = forward + backward (gradients w.r.t. Q and D) through the autograd path.  Inputs are
seeded synthetic data.  With N > 1 every rank runs its own replica of the step (MaxSim training does
not shard; data parallelism is the caller's), so the whole-job figure is N times the per-rank work
over the slowest rank's time ("weak" scaling).

Metric: TFLOP/s counting only algorithmic work on valid tokens:
    forward  2 * d * sum_{(i,j)} lq_i * ld_j        backward  4 * d * sum_{(i,j)} lq_i
One JSON line is printed by rank 0.
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


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


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


def cpu_reference_step(sample_q, Q, D, dm, g):
    """One forward + backward of the reference algorithm (the CPU oracle, a port of the reference's
    reference.py) on the first `sample_q` queries against all documents."""
    from oracle import maxsim_oracle as O

    s = O.maxsim(Q[:sample_q], D, None, dm)
    gq, gd = O.maxsim_grads(g[:sample_q], Q[:sample_q], D, None, dm)
    return float(s.sum()) + float(gq.sum()) + float(gd.sum())


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


def retrieve_bench(n_docs, world, rank, dev):
    """Sharded top-k retrieve (BASELINE config 5 shape): `n_docs` documents of U[32,300] tokens, d=128, bf16
    normalised, split by document over the ranks; 1024 queries x 32 tokens, top_k=100, chunk=4096.
    Strong scaling: the corpus is fixed, every rank scores its slice, one all-gather + merge."""
    import torch
    import torch.distributed as dist

    from late_interaction_kernels_b200 import sharded

    lo, hi = sharded.shard_bounds(n_docs, world, rank)
    nd, Ld, d, chunk = hi - lo, 300, 128, 4096
    D = torch.empty((nd, Ld, d), dtype=torch.bfloat16, device=dev)
    lens = torch.empty(nd, dtype=torch.int64, device=dev)
    g = torch.Generator(device=dev)
    for c0 in range(0, nd, chunk):  # chunk-addressable seeds: any rank can regenerate any chunk
        c1 = min(nd, c0 + chunk)
        g.manual_seed(1234 + (lo + c0) // chunk)
        x = torch.randn((c1 - c0, Ld, d), generator=g, device=dev, dtype=torch.float32)
        D[c0:c1] = torch.nn.functional.normalize(x, dim=-1).to(torch.bfloat16)
        lens[c0:c1] = torch.randint(32, Ld + 1, (c1 - c0,), generator=g, device=dev)
    dm = torch.arange(Ld, device=dev)[None, :] < lens[:, None]
    g.manual_seed(99)
    Q = torch.nn.functional.normalize(torch.randn((1024, 32, d), generator=g, device=dev), dim=-1).to(torch.bfloat16)
    valid_tokens = torch.tensor([float(lens.sum())], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(valid_tokens)

    def run():
        return sharded.retrieve_sharded(Q, D, 100, d_mask=dm, doc_offset=lo, n_docs_total=n_docs, normalize=False, chunk=chunk)

    run()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    reps = 2
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        s, i = run()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops = 2.0 * d * 1024 * 32 * float(valid_tokens.item())
    return {"metric": "retrieve queries/s", "value": 1024 / (ms * 1e-3), "unit": "queries/s", "ms_per_batch": ms,
            "n_docs": n_docs, "queries": 1024, "top_k": 100, "chunk": chunk, "scaling": "strong",
            "tflops_valid": flops / (ms * 1e-3) / 1e12, "best_index_q0": int(i[0, 0])}


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
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
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


def other_configs(dev):
    """Kernel timings of the other BASELINE shapes (rank 0, one GPU): the KD layout in bf16 and e4m3
    (HBM-bound: GB/s over the document bytes read once), the packed ColPali-shaped batch forward and
    forward + backward (TFLOP/s on valid tokens), and the PLAID candidate score (GB/s over codes + table rows)."""
    import torch
    import torch.nn.functional as F

    import late_interaction_kernels_b200 as lik
    from late_interaction_kernels_b200 import fp8, plaid

    out = {}
    g = torch.Generator(device=dev).manual_seed(7)
    # KD: Q[64,32,128] x D[64,32,300,128], lengths U[64,300] per candidate
    Q = F.normalize(torch.randn((64, 32, 128), generator=g, device=dev), dim=-1)
    D = F.normalize(torch.randn((64, 32, 300, 128), generator=g, device=dev), dim=-1)
    lens = torch.randint(64, 301, (64, 32), generator=g, device=dev)
    dm = torch.arange(300, device=dev)[None, None, :] < lens[..., None]
    qb, db = Q.bfloat16(), D.bfloat16()
    t = _time_us(lambda: lik.maxsim(qb, db, d_mask=dm), dev, graph=True)
    out["kd_bf16_fwd"] = {"us": t, "GBps_document_bytes": db.numel() * 2 / t / 1e3, "shape": "Q[64,32,128] x D[64,32,300,128]"}
    q8, sq = fp8.quantize_fp8_per_token(Q)
    d8, sd = fp8.quantize_fp8_per_token(D)
    t = _time_us(lambda: fp8.maxsim_inference_fp8(q8, d8, scale_Q=sq, scale_D=sd, d_mask=dm), dev, graph=True)
    out["kd_e4m3_fwd"] = {"us": t, "GBps_document_bytes": (d8.numel() + sd.numel() * 4) / t / 1e3}
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
    out["varlen_fwd"] = {"us": t, "tflops_valid": fl / t / 1e6, "shape": "128 q U[16,32] x 128 docs U[900,1030]"}
    Qr, Dr = Qp.clone().requires_grad_(), Dp.clone().requires_grad_()
    go = torch.randn((128, 128), generator=g, device=dev)

    def fb():
        Qr.grad = None
        Dr.grad = None
        lik.maxsim_varlen(Qr, Dr, cq, cd, 32, 1030).backward(go)

    t = _time_us(fb, dev)
    out["varlen_fwd_bwd"] = {"us": t, "tflops_valid": (fl + 4.0 * 128 * float(ql.sum()) * 128) / t / 1e6}
    # PLAID candidate score: 65536 centroids, 8192 candidate documents of up to 300 codes
    qcs = torch.randn((65536, 32), generator=g, device=dev)
    codes = torch.randint(0, 65536, (8192, 300), generator=g, device=dev, dtype=torch.int32)
    cl = torch.randint(32, 301, (8192,), generator=g, device=dev)
    t = _time_us(lambda: plaid.plaid_approx_score(qcs, codes, cl), dev, graph=True)
    out["plaid_approx"] = {"us": t, "GBps_codes_and_rows": float(cl.sum()) * (4 + 32 * 4) / t / 1e3, "shape": "8192 docs x <=300 codes, 32 query tokens"}
    return out


def plaid_retrieve_bench(n_docs, world, rank, dev):
    """Sharded top-k over a PLAID index (2-bit residuals, d=128, 65536 fp16 centroids): the shard's
    codes and residual bytes are decompressed chunk by chunk, scored and merged; 1024 queries, top-100."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from late_interaction_kernels_b200 import sharded

    lo, hi = sharded.shard_bounds(n_docs, world, rank)
    g = torch.Generator(device=dev).manual_seed(4321 + rank)
    lens = torch.randint(32, 301, (hi - lo,), generator=g, device=dev)
    T = int(lens.sum())
    codes = torch.randint(0, 65536, (T,), generator=g, device=dev, dtype=torch.int32)
    res = torch.randint(0, 256, (T, 32), generator=g, device=dev, dtype=torch.uint8)
    cu = F.pad(lens.cumsum(0), (1, 0)).int()
    g.manual_seed(5)
    cent = F.normalize(torch.randn((65536, 128), generator=g, device=dev), dim=-1).half()
    bw = torch.linspace(-0.1, 0.1, 4, device=dev)
    Q = F.normalize(torch.randn((1024, 32, 128), generator=g, device=dev), dim=-1).bfloat16()
    tok = torch.tensor([float(T)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tok)

    def run():
        return sharded.retrieve_plaid_sharded(Q, codes, res, cu, cent, bw, 2, 100, doc_offset=lo, n_docs_total=n_docs, chunk=4096)

    run()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    s, i = run()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    n_tok = float(tok.item())
    return {"metric": "PLAID retrieve queries/s", "value": 1024 / (ms * 1e-3), "unit": "queries/s", "ms_per_batch": ms, "n_docs": n_docs,
            "queries": 1024, "top_k": 100, "nbits": 2, "scaling": "strong", "tflops_valid": 2.0 * 128 * 1024 * 32 * n_tok / (ms * 1e-3) / 1e12,
            "compressed_GBps": n_tok * 36 / (ms * 1e-3) / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--retrieve-docs", type=int, default=1_000_000,
                    help="corpus size of the sharded top-k retrieve reported under extra.retrieve (0 = skip)")
    ap.add_argument("--only", default=None, choices=["fwd", "fwd_infer", "bwd", "step"],
                    help="profiling aid: launch only this part of the step, --steps times, and print its mean time")
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
    _lib.load()

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
        from late_interaction_kernels_b200.backward import maxsim_backward_lowmem

        qs, ds = _ops.padded_spec(dQ), _ops.padded_spec(dD, dM)
        _, am = _ops.forward(qs, ds, save_argmax=True)
        part = {
            "fwd": lambda: _ops.forward(qs, ds, save_argmax=True),
            "fwd_infer": lambda: _ops.forward(qs, ds),
            "bwd": lambda: maxsim_backward_lowmem(dG, dQ, dD, am),
            "step": step,
        }[args.only]
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

    for _ in range(args.warmup):
        step()
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        for a, b in ev:
            flush.zero_()
            a.record()
            step()
            b.record()
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
    n_e2e = max(4, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_run(n_e2e)
    e1.record()
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_val = world * (fwd_flops + bwd_flops) * n_e2e / (float(te.item()) * 1e-3) / 1e12
    h2d = hQ.numel() * 2 + hD.numel() * 2 + hM.numel() + hG.numel() * 4
    d2h = hS.numel() * 4 + hGQ.numel() * 2 + hGD.numel() * 2

    # ---- roofline of the dominant kernel (the tcgen05 forward with argmax), timed alone ----
    qs, ds = _ops.padded_spec(dQ), _ops.padded_spec(dD, dM)
    for _ in range(3):
        _ops.forward(qs, ds, save_argmax=True)
    fev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
    for a, b in fev:
        flush.zero_()
        a.record()
        _ops.forward(qs, ds, save_argmax=True)
        b.record()
    torch.cuda.synchronize()
    fwd_ms = float(np.mean([a.elapsed_time(b) for a, b in fev]))
    peak_tf, _, which = measured_peaks()
    achieved = fwd_flops / (fwd_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the
                # ncu capture summarised in profiles/fwd_tc_kernel_argmax_c2.txt (31.55 MB + 4.02 MB)
                "traffic": 35.57e6, "traffic_unit": "bytes per launch",
                "kernel": "fwd_tc_kernel (bf16, argmax, masked)", "kernel_ms": fwd_ms, "peak_source": which}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"replicas x{world}", "l2": "flushed between steps (256 MB write)",
                   "fwd_flops_per_step": fwd_flops, "bwd_flops_per_step": bwd_flops},
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        # per step: mask_lens + fwd_tc (forward), bwd_dq_fast + bwd_dd_sort + bwd_dd_reduce (backward)
        "gpu_launches": 5 * args.steps,
        "roofline": roofline,
        "clocks": clocks.summary(),
    }
    if args.retrieve_docs > 0:
        del Qr, Dr, flush
        torch.cuda.empty_cache()
        line["extra"] = {"retrieve": retrieve_bench(args.retrieve_docs, world, rank, dev)}
        torch.cuda.empty_cache()
        line["extra"]["plaid_retrieve"] = plaid_retrieve_bench(args.retrieve_docs, world, rank, dev)
        torch.cuda.empty_cache()
        if world == 1:
            line["extra"]["other_configs"] = other_configs(dev)
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
                                    "kind": "port", "sample": f"{reps} x ({sample_q} queries x {ND} docs fwd+bwd), numpy oracle, all host threads"}
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
