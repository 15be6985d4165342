#!/usr/bin/env python
"""Benchmark of the block-sparse attention hot path.

Workload (benchmark configuration "long-sequence strided pattern"): fp16, batch 4 x heads 16
(Z = 64 slices per GPU), seq 4096, head_dim 64, block 64, layout = every 8th block diagonal
plus a band of half-width 2 (762 of 4096 blocks, 18.6 %), non-causal, softmax scale 1/8.
One step = forward SDD(Q.K^T) -> softmax -> DSD(P.V) and the backward the autograd layer
issues: SDD(dO.V^T), DSD(P^T.dO), softmax backward, DSD(dS.K), DSD(dS^T.Q): six block-sparse
matmuls and two softmax kernels.  Metric: nonzero-block TFLOP/s = 6 * 2*B*B*D*blocks / step time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 runs under torchrun, one rank per GPU; every rank owns its own Z = 64 slices (weak
scaling, no collective on the data path) and the reported value is the whole-job aggregate
over the slowest rank's device time.  The timed region of K steps is repeated (``--repeats``,
default 7) and the median is reported.  After the timing every rank checks one of its own slices
against the CPU oracle and the per-rank errors are gathered over NCCL (``verify``); a failed check
makes the run exit non-zero.  ``--impl reference`` times the masked dense torch computation on the
host CPU (the reference ships no CPU implementation and its CUDA kernels are wrong for 5 of 12
variants, so the masked-dense definition is its CPU arm); that arm loads no native code of this
repository.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(REPO, "experiments-pytorch-cuda-extension-for-sparse-matmul_b200")

import torch  # noqa: E402

WORKLOAD = dict(name="cfg3_strided_local_seq4096", batch=4, heads=16, seq=4096, head_dim=64, block=64,
                stride=8, window=2, scale=0.125, dtype="f16")
METRIC = "nonzero-block TFLOP/s, block-sparse attention step fwd+bwd (6 SDD/DSD matmuls + softmax fwd/bwd), seq 4096 block 64 fp16"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
VERIFY_TOL = 1e-2           # fp16 contract: max |got - ref| / max |ref| against the masked dense fp32 computation


def load_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS if k in p} | {"source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


def use_oracle():
    """The CPU oracle: the checker of `verify` and the timed CPU baseline.  Never on the measured GPU path."""
    if REPO not in sys.path:
        sys.path.insert(0, REPO)
    from oracle import oracle
    return oracle


def use_package():
    if PKG not in sys.path:
        sys.path.insert(0, PKG)


def workload_config(world, z):
    """The `config` object of the JSON line; both arms print the same one."""
    w = WORKLOAD
    nnz = int(use_oracle().strided_local_pattern(w["seq"] // w["block"], w["stride"], w["window"]).sum())
    return {"workload": w["name"] + ("" if z == w["batch"] * w["heads"] else "_REDUCED_%d_slices" % z),
            "batch_per_gpu": w["batch"], "heads": w["heads"], "slices_per_gpu": z, "seq": w["seq"],
            "head_dim": w["head_dim"], "block": w["block"], "nnz_blocks_per_head": nnz,
            "layout": "strided(8)+local(2), non-causal", "parallelism": "head-sharded x%d" % world,
            "l2": "no flush: the four sparse tensors of a step are 400 MB each, above the 126 MB L2"}


def seeded_heads(first_head, count, seq, dim, salt):
    """fp16 inputs drawn on the CPU in fp32, one generator per GLOBAL head index."""
    out = torch.empty(count, seq, dim, dtype=torch.float16)
    for i in range(count):
        gen = torch.Generator().manual_seed(3000 + 10 * (first_head + i) + salt)
        out[i] = torch.randn(seq, dim, generator=gen).half()
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.proc, self.index = None, device_index
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-i", str(device_index), "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- reference / CPU arm
def cpu_attention_sample(heads, threads=None):
    """Time the masked dense torch attention step (fwd + bwd) on `heads` slices of the workload.
    Returns (seconds, nonzero-block FLOP of the sample, dense FLOP the CPU actually executed)."""
    oracle = use_oracle()
    w = WORKLOAD
    torch.set_num_threads(threads or os.cpu_count())
    pattern = oracle.strided_local_pattern(w["seq"] // w["block"], w["stride"], w["window"])
    q, k, v, do = (seeded_heads(0, heads, w["seq"], w["head_dim"], s).float() for s in range(4))
    t0 = time.perf_counter()
    oracle.attention_step_dense(q, k, v, do, pattern, w["block"], w["scale"], False)
    dt = time.perf_counter() - t0
    nnz = int(pattern.sum())
    flops = 6 * 2.0 * w["block"] ** 2 * w["head_dim"] * nnz * heads
    dense_flops = 6 * 2.0 * w["seq"] ** 2 * w["head_dim"] * heads
    return dt, flops, dense_flops


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOAD
    heads = 1
    for _ in range(args.warmup):
        cpu_attention_sample(heads)
    times, flops, dense = [], 0.0, 0.0
    for _ in range(args.steps):
        dt, flops, dense = cpu_attention_sample(heads)
        times.append(dt)
    total = sum(times)
    value = flops * len(times) / total / 1e12
    z = w["batch"] * w["heads"]
    sample = ("%d of %d (batch*head) slices per step; a dense port: masked dense torch fp32 attention fwd+bwd on the "
              "host cores, credited with the nonzero-block FLOP only (it executes %.1fx as many)"
              % (heads, z, dense / flops))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(max(1, args.gpus), z),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample, "dense_TFLOP/s": dense * len(times) / total / 1e12,
                             "note": "one host at every N: the ratio to the N-GPU arm is not a scaling curve"},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


# --------------------------------------------------------------------------- our arm
OPS = ["sdd_qk", "softmax_fwd", "dsd_pv", "sdd_dp", "dsd_dv", "softmax_bwd", "dsd_dq", "dsd_dk"]


def device_step(ops, lay, q, k, v, do, scale, block, events=None, causal=False):
    """The eight native calls of one forward + backward attention step (what the autograd ops issue)."""
    rl, cl = lay.row_layout, lay.col_layout
    calls = [
        lambda st: ops.sparse_matmul(q, k, "sdd", rl, cl, False, True, block),
        lambda st: ops.sparse_softmax_forward(st["s"], rl[0], rl[1], scale, causal, None, lay.max_row_blocks),
        lambda st: ops.sparse_matmul(st["p"], v, "dsd", rl, cl, False, False, block),
        lambda st: ops.sparse_matmul(do, v, "sdd", rl, cl, False, True, block),
        lambda st: ops.sparse_matmul(st["p"], do, "dsd", rl, cl, True, False, block),
        lambda st: ops.sparse_softmax_backward(st["p"], st["dp"], rl[0], rl[1], scale, lay.max_row_blocks),
        lambda st: ops.sparse_matmul(st["ds"], k, "dsd", rl, cl, False, False, block),
        lambda st: ops.sparse_matmul(st["ds"], q, "dsd", rl, cl, True, False, block),
    ]
    keys = ["s", "p", "o", "dp", "dv", "ds", "dq", "dk"]
    st = {}
    for i, (call, key) in enumerate(zip(calls, keys)):
        if events is not None:
            events[i][0].record()
        st[key] = call(st)
        if events is not None:
            events[i][1].record()
    return st


def fused_step(lay, q, k, v, do, scale, causal=False):
    """The same step through the public fused op (one forward kernel, two backward kernels)."""
    from sparse import attention
    q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    o = attention(q, k, v, lay, scale, causal)
    o.backward(do)
    return o.detach(), q.grad, k.grad, v.grad


def timed(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def graph_replayed(fn, iters=20):
    """Capture `fn` into a CUDA graph (after a side-stream warm-up, as torch requires) and time replays."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return timed(graph.replay, iters)


def rel_err(got, ref):
    ref = ref.float()
    return float((got.detach().float().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def side_cfg2(sparse_ops, dev):
    """Benchmark configuration 2 (the reference's block size): fp16, batch 8 x heads 12, seq 1024, head_dim 64,
    block 32, causal local window 4 + 1 global block row / column, scale 1/8 with the element-level causal mask."""
    from sparse import SparseLayout
    from sparse.patterns import local_global_causal
    z, seq, dim, block, scale = 96, 1024, 64, 32, 0.125
    lay = SparseLayout(local_global_causal(seq // block, 4, 1), block=block, device=dev)
    gen = torch.Generator(device=dev).manual_seed(2000)
    q, k, v, do = (torch.randn(z, seq, dim, device=dev, generator=gen).half() for _ in range(4))
    unfused = lambda: device_step(sparse_ops, lay, q, k, v, do, scale, block, None, True)   # noqa: E731
    fused = lambda: fused_step(lay, q, k, v, do, scale, True)                                # noqa: E731
    out = {"unfused_step_us": round(1e3 * timed(unfused, 20), 1), "fused_step_us": round(1e3 * timed(fused, 20), 1)}
    out["unfused_step_graph_us"] = round(1e3 * graph_replayed(unfused), 1)
    out["fused_step_graph_us"] = round(1e3 * graph_replayed(fused), 1)
    # block-32 engine at seq 4096 (fp16, the benchmark pattern at block 32): how far from the HBM roofline
    from sparse.patterns import strided_local
    lay4 = SparseLayout(strided_local(128, 16, 4), block=block, device=dev)
    z4, seq4 = 32, 4096
    a, b = (torch.randn(z4, seq4, dim, device=dev, generator=gen).half() for _ in range(2))
    rl, cl = lay4.row_layout, lay4.col_layout
    s4 = sparse_ops.sparse_matmul(a, b, "sdd", rl, cl, False, True, block)
    byts = s4.numel() * 2 + 2 * a.numel() * 2
    peaks = load_peaks()
    for name, fn in (("sdd", lambda: sparse_ops.sparse_matmul(a, b, "sdd", rl, cl, False, True, block)),
                     ("dsd", lambda: sparse_ops.sparse_matmul(s4, b, "dsd", rl, cl, False, False, block))):
        ms = timed(fn, 10)
        out["seq4096_block32_%s" % name] = {"us": round(1e3 * ms, 1), "hbm_frac": round(byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
    out["note"] = ("whole step forward + backward, 96 slices, 150 blocks of 32 per head; about 10 us of HBM-bound work, "
                   "so launch and per-item costs dominate")
    return out


def side_cfg4(sparse_ops, dev):
    """Benchmark configuration 4: fp32 through the 3xTF32 split, batch 2 x heads 8, seq 2048, head_dim 128, block 32,
    Bernoulli(0.1) + diagonal (one head's pattern for all slices), inputs U(-1, 1); error against the fp64 oracle."""
    from sparse import SparseLayout
    from sparse.patterns import random_with_diagonal
    oracle = use_oracle()
    z, seq, dim, block = 16, 2048, 128, 32
    pattern = random_with_diagonal(seq // block, seq // block, 0.1, 4000)
    lay = SparseLayout(pattern, block=block, device=dev)
    gen = torch.Generator().manual_seed(4000)
    a = (torch.rand(z, seq, dim, generator=gen) * 2 - 1)
    b = (torch.rand(z, seq, dim, generator=gen) * 2 - 1)
    sp = (torch.rand(z, lay.num_blocks, block, block, generator=gen) * 2 - 1)
    ad, bd, spd = a.to(dev), b.to(dev), sp.to(dev)
    rl, cl = lay.row_layout, lay.col_layout
    cases = {"sdd_NT": (ad, bd, "sdd", False, True, a, b), "dsd_NN": (spd, bd, "dsd", False, False, sp, b),
             "dsd_TN": (spd, bd, "dsd", True, False, sp, b), "dds_TN": (ad, spd, "dds", True, False, a, sp)}
    out = {}
    for name, (x, y, mode, ta, tb, xc, yc) in cases.items():
        fn = lambda: sparse_ops.sparse_matmul(x, y, mode, rl, cl, ta, tb, block)       # noqa: E731
        us = 1e3 * timed(fn, 10)
        ref = oracle.sparse_matmul(xc[:1], yc[:1], mode, pattern.numpy(), block, ta, tb, dtype=torch.float64)
        out[name] = {"us": round(us, 1), "rel_err_vs_fp64": float("%.2e" % rel_err(fn()[:1], ref))}
    out["tol"] = 1e-4
    return out


def side_cfg5_strong(sparse_ops, dev, world, dist):
    """Benchmark configuration 5 as it is defined: batch 16 x heads 32 = 512 slices split over the ranks (strong
    scaling), fp16, seq 8192, head_dim 128, block 64, BigBird layout (1 262 blocks)."""
    from sparse import SparseLayout
    from sparse.patterns import bigbird
    total, seq, dim, block, scale = 512, 8192, 128, 64, 128 ** -0.5
    z = total // world
    lay = SparseLayout(bigbird(seq // block, 1, 2, 3, 5000), block=block, device=dev)
    gen = torch.Generator(device=dev).manual_seed(5000 + int(os.environ.get("RANK", "0")))
    q, k, v, do = (torch.randn(z, seq, dim, device=dev, generator=gen).half() for _ in range(4))
    for _ in range(2):
        device_step(sparse_ops, lay, q, k, v, do, scale, block)
    steps = 3
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in OPS] for _ in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        device_step(sparse_ops, lay, q, k, v, do, scale, block, ev[i])
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms[0])
    nnz = lay.num_blocks
    flops = 6 * 2.0 * block * block * dim * nnz * total
    sparse_bytes, dense_bytes = z * nnz * block * block * 2, z * seq * dim * 2
    peaks = load_peaks()
    ops = {}
    for j, name in enumerate(OPS):
        t = sum(ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(steps)) / steps
        byts = {"softmax_fwd": 2 * sparse_bytes, "softmax_bwd": 3 * sparse_bytes}.get(name, sparse_bytes + 2 * dense_bytes)
        ops[name] = {"ms": round(t, 3), "hbm_frac": round(byts / (t * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
    # the same step through the fused public op (head dim 128: single-group forward kernel, general backward kernels)
    for _ in range(2):
        fused_step(lay, q, k, v, do, scale)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for i in range(steps):
        fused_step(lay, q, k, v, do, scale)
    e1.record()
    torch.cuda.synchronize()
    fms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(fms, op=dist.ReduceOp.MAX)
    fms = float(fms[0])
    del q, k, v, do
    torch.cuda.empty_cache()
    return {"slices_total": total, "slices_per_gpu": z, "step_ms": round(ms, 3), "TFLOP/s": round(flops / (ms * 1e-3) / 1e12, 1),
            "fused_step_ms": round(fms, 3), "fused_TFLOP/s": round(flops / (fms * 1e-3) / 1e12, 1),
            "scaling": "strong", "ops_rank0": ops}


def verify(sparse_ops, lay, q, k, v, do, scale, block, pattern, world, rank, dev):
    """Every rank checks its own last slice -- output and dQ, dK, dV of the unfused step and of the fused step --
    against the masked dense CPU computation; the per-rank errors are gathered over the process group."""
    from sparse.distributed import gather_slices
    oracle = use_oracle()
    i = q.shape[0] - 1
    sl = slice(i, i + 1)
    st = device_step(sparse_ops, lay, q[sl], k[sl], v[sl], do[sl], scale, block)
    fo, fq, fk, fv = fused_step(lay, q[sl], k[sl], v[sl], do[sl], scale)
    torch.cuda.synchronize()
    ref = oracle.attention_step_dense(q[sl].float().cpu(), k[sl].float().cpu(), v[sl].float().cpu(), do[sl].float().cpu(),
                                      pattern, block, scale, False)
    errs = [rel_err(g, r) for g, r in zip((st["o"], st["dq"], st["dk"], st["dv"], fo, fq, fk, fv), ref + ref)]
    mine = torch.tensor([[max(errs[:4]), max(errs[4:])]], device=dev, dtype=torch.float64)     # one row per rank
    everyone = gather_slices(mine, world) if world > 1 else mine
    worst = float(everyone.max())
    return {"ranks": int(everyone.shape[0]), "what": "last slice of every rank: o, dq, dk, dv of the unfused and of the fused step "
            "against masked dense torch on the CPU", "max_rel_err_unfused": float("%.3e" % float(everyone[:, 0].max())),
            "max_rel_err_fused": float("%.3e" % float(everyone[:, 1].max())), "max_rel_err": float("%.3e" % worst),
            "tol": VERIFY_TOL, "ok": bool(worst <= VERIFY_TOL)}


def run_ours(args):
    import torch.distributed as dist
    use_package()
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    from sparse.patterns import strided_local
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the block-sparse kernels have no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit("bench.py: --gpus %d needs torchrun with %d ranks (WORLD_SIZE=%d)" % (args.gpus, args.gpus, world))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # host side of the end-to-end step: this rank's threads and pinned buffers on the GPU's own NUMA node
    from sparse.distributed import bind_host_to_device
    props = torch.cuda.get_device_properties(local_rank)
    numa_node = bind_host_to_device(getattr(props, "pci_domain_id", 0), getattr(props, "pci_bus_id", -1),
                                    getattr(props, "pci_device_id", 0)) if hasattr(props, "pci_bus_id") else None
    print("bench.py: rank %d, GPU %d at PCI %04x:%02x, host NUMA node %s" % (
        rank, local_rank, getattr(props, "pci_domain_id", 0), getattr(props, "pci_bus_id", 0), numa_node), file=sys.stderr)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOAD
    z = args.slices or w["batch"] * w["heads"]
    block, seq, dim, scale = w["block"], w["seq"], w["head_dim"], w["scale"]
    pattern = strided_local(seq // block, w["stride"], w["window"])
    lay = SparseLayout(pattern, block=block, device=dev)
    nnz = lay.num_blocks
    first_head = rank * z           # weak scaling: every rank owns z slices, seeded by global index
    # one pinned allocation per direction: a step uploads / downloads with a single copy
    host_in = torch.empty(4, z, seq, dim, dtype=torch.float16).pin_memory()
    for s in range(4):
        host_in[s] = seeded_heads(first_head, z, seq, dim, s)
    q, k, v, do = (t.contiguous() for t in host_in.to(dev, non_blocking=True).unbind(0))
    torch.cuda.synchronize()

    es = 2
    sparse_bytes = z * nnz * block * block * es
    dense_bytes = z * seq * dim * es
    flops_matmul = 2.0 * block * block * dim * nnz * z
    alg_bytes = {"sdd_qk": sparse_bytes + 2 * dense_bytes, "dsd_pv": sparse_bytes + 2 * dense_bytes,
                 "sdd_dp": sparse_bytes + 2 * dense_bytes, "dsd_dv": sparse_bytes + 2 * dense_bytes,
                 "dsd_dq": sparse_bytes + 2 * dense_bytes, "dsd_dk": sparse_bytes + 2 * dense_bytes,
                 "softmax_fwd": 2 * sparse_bytes, "softmax_bwd": 3 * sparse_bytes}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from before the warm-up until after the end-to-end loop, so all timed
    # regions are covered (a timed region of a few tens of ms is shorter than one sampling period)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # ---- device-resident timing (value): `repeats` timed regions of `steps` steps each, two events per region.
    # (Events between the launches cost 50-65 us per step: the per-op times come from a pass of their own.)
    for _ in range(args.warmup):
        device_step(sparse_ops, lay, q, k, v, do, scale, block)
    barrier()
    region_ms = []
    for _ in range(args.repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(args.steps):
            device_step(sparse_ops, lay, q, k, v, do, scale, block)
        stop.record()
        barrier()
        region_ms.append(start.elapsed_time(stop))
    # ---- per-op times: the same loop once more with a pair of events around every launch
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in OPS] for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        device_step(sparse_ops, lay, q, k, v, do, scale, block, ev[i])
    stop.record()
    barrier()
    op_ms = {name: sum(ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(args.steps)) / args.steps
             for j, name in enumerate(OPS)}
    instrumented_ms = start.elapsed_time(stop) / args.steps
    # ---- the step replayed from a CUDA graph (no launch gaps): reported beside the eager value
    graph_ms = graph_replayed(lambda: device_step(sparse_ops, lay, q, k, v, do, scale, block), args.steps)
    sparse_ops.check_device_status(local_rank)

    # ---- end-to-end timing through the public API with host buffers.  Every step copies its four
    # inputs from pinned host memory (one copy), runs forward + backward through the public fused op
    # `sparse.attention` and copies the four results back to pinned host memory (one copy).  Copies run
    # on their own streams so that step i + 1's upload and step i - 1's download overlap step i's
    # kernels (double-buffered device inputs and host outputs); the timed region covers all of it.
    e2e_steps = max(1, min(args.steps, 50))
    outs_host = [torch.empty(4, z, seq, dim, dtype=torch.float16).pin_memory() for _ in range(2)]
    dev_in = [torch.empty(4, z, seq, dim, dtype=torch.float16, device=dev) for _ in range(2)]
    dev_out = [torch.empty(4, z, seq, dim, dtype=torch.float16, device=dev) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)

    def e2e_run(steps, kernels=True):
        computed = [None, None]          # event: kernels that read dev_in[b] / wrote dev_out[b] are done
        downloaded = [None, None]        # event: outs_host[b] has been filled from dev_out[b]
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if computed[b] is not None:
                    s_in.wait_event(computed[b])
                dev_in[b].copy_(host_in, non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(s_in)
            main.wait_event(uploaded)
            if downloaded[b] is not None:
                main.wait_event(downloaded[b])
            if kernels:
                res = fused_step(lay, *dev_in[b].unbind(0), scale)
                for slot, r in enumerate(res):
                    dev_out[b][slot].copy_(r)
            computed[b] = torch.cuda.Event()
            computed[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[b])
                outs_host[b].copy_(dev_out[b], non_blocking=True)
                downloaded[b] = torch.cuda.Event()
                downloaded[b].record(s_out)
        for ev_ in downloaded:
            if ev_ is not None:
                main.wait_event(ev_)

    def e2e_timed(kernels):
        e2e_run(min(args.warmup, 3), kernels)
        barrier()
        e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e_start.record()
        e2e_run(e2e_steps, kernels)
        e_stop.record()
        barrier()
        return e_start.elapsed_time(e_stop)

    e2e_ms = e2e_timed(True)
    copy_floor_ms = e2e_timed(False)        # the same copies on the same streams with all ranks active, no kernels
    clocks = sampler.stop() if sampler else None
    del dev_in, dev_out, outs_host

    # ---- every op of the step alone: 20 launches of the same op back to back between two events (the pair of
    # events around a launch inside the step adds about 5 us of launch latency to every op of `ops`)
    st_ = device_step(sparse_ops, lay, q, k, v, do, scale, block)
    rl_, cl_ = lay.row_layout, lay.col_layout
    alone_calls = {
        "sdd_qk": lambda: sparse_ops.sparse_matmul(q, k, "sdd", rl_, cl_, False, True, block),
        "softmax_fwd": lambda: sparse_ops.sparse_softmax_forward(st_["s"], rl_[0], rl_[1], scale, False, None, lay.max_row_blocks),
        "dsd_pv": lambda: sparse_ops.sparse_matmul(st_["p"], v, "dsd", rl_, cl_, False, False, block),
        "sdd_dp": lambda: sparse_ops.sparse_matmul(do, v, "sdd", rl_, cl_, False, True, block),
        "dsd_dv": lambda: sparse_ops.sparse_matmul(st_["p"], do, "dsd", rl_, cl_, True, False, block),
        "softmax_bwd": lambda: sparse_ops.sparse_softmax_backward(st_["p"], st_["dp"], rl_[0], rl_[1], scale, lay.max_row_blocks),
        "dsd_dq": lambda: sparse_ops.sparse_matmul(st_["ds"], k, "dsd", rl_, cl_, False, False, block),
        "dsd_dk": lambda: sparse_ops.sparse_matmul(st_["ds"], q, "dsd", rl_, cl_, True, False, block),
    }
    alone_ms = {name: timed(fn, 20) for name, fn in alone_calls.items()}
    # ---- DDS side measurement (not part of the step): dV^T = dO^T . P as dds(T,N)
    p_blocks = st_["p"]
    dds_ms = timed(lambda: sparse_ops.sparse_matmul(do, p_blocks, "dds", lay.row_layout, lay.col_layout, True, False, block), 5)
    del p_blocks, st_, alone_calls
    # the fused forward (one kernel for sdd -> softmax -> dsd) and the fused backward (dQ by block
    # rows, dK / dV by block columns), reported beside the unfused operators
    from sparse.attention import attention_lse
    fused_ms = timed(lambda: attention_lse(q, k, v, lay, scale), 20)
    o_f, lse_f = attention_lse(q, k, v, lay, scale)
    rl_f, cl_f = lay.row_layout, lay.col_layout
    fused_bwd_ms = timed(lambda: sparse_ops.sparse_attention_backward(q, k, v, o_f, do, lse_f, rl_f[0], rl_f[1], cl_f[0], cl_f[1],
                                                                     block, scale, False, None), 20)
    sparse_ops.check_device_status(local_rank)

    # ---- parity inside the benchmark, on every rank
    check = verify(sparse_ops, lay, q, k, v, do, scale, block, pattern.numpy(), world, rank, dev)
    sparse_ops.check_device_status(local_rank)

    # ---- side reports on the other benchmark configurations (outside every timed region)
    side = {}
    if not args.no_side:
        if rank == 0:
            side["cfg2"] = side_cfg2(sparse_ops, dev)
            sparse_ops.check_device_status(local_rank)
            side["cfg4"] = side_cfg4(sparse_ops, dev)
            sparse_ops.check_device_status(local_rank)
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
        del q, k, v, do, o_f, lse_f
        torch.cuda.empty_cache()
        side["cfg5_strong"] = side_cfg5_strong(sparse_ops, dev, world, dist)
        sparse_ops.check_device_status(local_rank)

    # ---- max over ranks
    t = torch.tensor(region_ms + [e2e_ms, copy_floor_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    region_ms, e2e_ms, copy_floor_ms = [float(x) for x in t[:-2]], float(t[-2]), float(t[-1])

    if rank == 0:
        peaks = load_peaks()
        per_step = sorted(r / args.steps for r in region_ms)
        ms_per_step = statistics.median(per_step)
        value = 6 * flops_matmul * world / (ms_per_step * 1e-3) / 1e12
        e2e_value = 6 * flops_matmul * world / (e2e_ms / e2e_steps * 1e-3) / 1e12
        ops_report = {}
        for name in OPS:
            gbs = alg_bytes[name] / (op_ms[name] * 1e-3) / 1e9
            entry = {"ms": round(op_ms[name], 4), "GB/s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4),
                     "alone_ms": round(alone_ms[name], 4),
                     "alone_hbm_frac": round(alg_bytes[name] / (alone_ms[name] * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
            if not name.startswith("softmax"):
                tf = flops_matmul / (op_ms[name] * 1e-3) / 1e12
                entry["TFLOP/s"] = round(tf, 1)
                entry["tensor_frac"] = round(tf / peaks["bf16_tflops"], 4)
            ops_report[name] = entry
        dds_gbs = alg_bytes["dsd_dv"] / (dds_ms * 1e-3) / 1e9
        ops_report["dds_dvT"] = {"ms": round(dds_ms, 4), "GB/s": round(dds_gbs, 1),
                                 "hbm_frac": round(dds_gbs / peaks["hbm_gbs"], 4),
                                 "TFLOP/s": round(flops_matmul / (dds_ms * 1e-3) / 1e12, 1),
                                 "tensor_frac": round(flops_matmul / (dds_ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4)}
        unfused_fwd_ms = op_ms["sdd_qk"] + op_ms["softmax_fwd"] + op_ms["dsd_pv"]
        fused_tf = 2 * flops_matmul / (fused_ms * 1e-3) / 1e12
        fused_report = {"kernel": "attention_forward_pipes_kernel", "ms": round(fused_ms, 4),
                        "TFLOP/s": round(fused_tf, 1), "tensor_frac": round(fused_tf / peaks["bf16_tflops"], 4),
                        "unfused_forward_ms": round(unfused_fwd_ms, 4), "speedup": round(unfused_fwd_ms / fused_ms, 2),
                        "hbm_bytes": 4 * dense_bytes,
                        "note": "forward only, outside the timed step; Q, K, V read and O written once, "
                                "scores and probabilities never leave the SM"}
        fused_step_ms = fused_ms + fused_bwd_ms
        fused_step_report = {"kernels": "attention_forward_pipes_kernel + attention_backward_rows_pipes_kernel + attention_backward_cols_pipes_kernel",
                             "forward_ms": round(fused_ms, 4), "backward_ms": round(fused_bwd_ms, 4),
                             "ms": round(fused_step_ms, 4),
                             "TFLOP/s": round(6 * flops_matmul / (fused_step_ms * 1e-3) / 1e12, 1),
                             "executed_TFLOP/s": round(9 * flops_matmul / (fused_step_ms * 1e-3) / 1e12, 1),
                             "tensor_frac_executed": round(9 * flops_matmul / (fused_step_ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4),
                             "unfused_step_ms": round(ms_per_step, 4), "speedup": round(ms_per_step / fused_step_ms, 2),
                             "note": "same gradients as the timed step, outside it; TFLOP/s counts the step's 6 block "
                                     "products, executed counts the 9 the fused kernels run (S and dP are recomputed)"}
        # dominant kernel = the kernel with the largest total time inside a step
        kernels = {
            "tc_matmul_kernel<dsd> (4 launches/step)": ["dsd_pv", "dsd_dv", "dsd_dq", "dsd_dk"],
            "tc_matmul_kernel<sdd> (2 launches/step)": ["sdd_qk", "sdd_dp"],
            "softmax_rows_kernel<fwd>": ["softmax_fwd"],
            "softmax_rows_kernel<bwd>": ["softmax_bwd"],
        }
        dom = max(kernels, key=lambda name: sum(op_ms[n] for n in kernels[name]))
        dom_ops = kernels[dom]
        dom_bytes = alg_bytes[dom_ops[0]]
        dom_ms = sum(op_ms[n] for n in dom_ops) / len(dom_ops)
        # measured DRAM bytes per launch and slice of each kernel family (one profiler capture of a reduced case;
        # every byte of the sparse operand is read or written once, so the traffic grows with the slices)
        traffic = None
        try:
            with open(os.path.join(REPO, "profiles", "dram_traffic.json")) as f:
                per_slice = json.load(f)["bytes_per_launch_and_slice"].get(dom.split(" ")[0])
            traffic = None if per_slice is None else round(per_slice * z)
        except (OSError, KeyError, ValueError):
            traffic = None
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        cpu_dt = cpu_flops = cpu_heads = cpu_dense = None
        if world == 1 and not args.no_cpu:
            probe_dt, _, _ = cpu_attention_sample(1)                 # size the sample: about 10 s of CPU work
            cpu_heads = int(max(2, min(z, 10.0 / max(probe_dt, 1e-3))))
            cpu_dt, cpu_flops, cpu_dense = cpu_attention_sample(cpu_heads)
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "repeats": args.repeats,
            "ms_per_step_min": round(per_step[0], 4), "ms_per_step_max": round(per_step[-1], 4),
            "ms_per_step_graph": round(graph_ms, 4), "ms_per_step_with_op_events": round(instrumented_ms, 4),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(world, z),
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": traffic,
                         "peak_source": peaks["source"]},
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "steps": e2e_steps,
                    "ms_per_step": round(e2e_ms / e2e_steps, 4), "copy_floor_ms": round(copy_floor_ms / e2e_steps, 4),
                    "api": "sparse.attention (fused forward and backward), one pinned buffer per direction",
                    "host_numa_node_rank0": numa_node,
                    "h2d_bytes_per_step": 4 * dense_bytes, "d2h_bytes_per_step": 4 * dense_bytes},
            "gpu_launches": len(OPS) * args.steps * args.repeats,
            "clocks": clocks, "verify": check, "ops": ops_report, "fused_forward": fused_report,
            "fused_step": fused_step_report,
            "engine": os.environ.get("BSA_MATMUL_ENGINE", "auto"),
        }
        line.update(side)
        if cpu_dt is not None:
            line["cpu_baseline"] = {"value": round(cpu_flops / cpu_dt / 1e12, 5), "unit": "TFLOP/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "dense_TFLOP/s": round(cpu_dense / cpu_dt / 1e12, 5),
                                    "sample": "%d of %d (batch*head) slices, masked dense torch fp32 fwd+bwd (a dense port: it "
                                              "executes %.1fx the nonzero-block FLOP it is credited with), %.1f s"
                                              % (cpu_heads, z, cpu_dense / cpu_flops, cpu_dt)}
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not check["ok"]:
        raise SystemExit("bench.py: verification against the CPU oracle failed: %r" % (check,))


_RESULT_FD = None


def emit(line):
    """The one JSON line of the run, on the stdout this process was started with."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # stdout carries the JSON line and nothing else: whatever libraries print there while the run lasts (NCCL's
    # version banner at the first collective) goes to stderr instead
    global _RESULT_FD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-side", action="store_true", help="skip the side reports on the other configurations")
    ap.add_argument("--slices", type=int, default=0,
                    help="(batch*head) slices per GPU; default is the workload's 64. A smaller value is a reduced "
                         "case for profiler captures, not a benchmark result")
    args = ap.parse_args()
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        args.repeats = max(args.repeats, 1)
        run_ours(args)


if __name__ == "__main__":
    main()
