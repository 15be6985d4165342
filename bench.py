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
over the slowest rank's device time.  ``--impl reference`` times the masked dense torch
computation on the host CPU (the reference ships no CPU implementation and its CUDA kernels
are wrong for 5 of 12 variants, so the masked-dense definition is its CPU arm).
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
for _p in (PKG, REPO):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

WORKLOAD = dict(name="cfg3_strided_local_seq4096", batch=4, heads=16, seq=4096, head_dim=64, block=64,
                stride=8, window=2, scale=0.125, dtype="f16")
METRIC = "nonzero-block TFLOP/s, block-sparse attention step fwd+bwd (6 SDD/DSD matmuls + softmax fwd/bwd), seq 4096 block 64 fp16"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS if k in p} | {"source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


def workload_pattern():
    from sparse.patterns import strided_local
    w = WORKLOAD
    return strided_local(w["seq"] // w["block"], w["stride"], w["window"])


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
    """Time the masked dense torch attention step (fwd + bwd) on `heads` slices of the workload."""
    from oracle import oracle
    w = WORKLOAD
    torch.set_num_threads(threads or os.cpu_count())
    pattern = workload_pattern()
    q, k, v, do = (seeded_heads(0, heads, w["seq"], w["head_dim"], s).float() for s in range(4))
    t0 = time.perf_counter()
    oracle.attention_step_dense(q, k, v, do, pattern.numpy(), w["block"], w["scale"], False)
    dt = time.perf_counter() - t0
    nnz = int(pattern.sum())
    flops = 6 * 2.0 * w["block"] ** 2 * w["head_dim"] * nnz * heads
    return dt, flops


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOAD
    heads = 1
    for _ in range(args.warmup):
        cpu_attention_sample(heads)
    times, flops = [], 0.0
    for _ in range(args.steps):
        dt, flops = cpu_attention_sample(heads)
        times.append(dt)
    total = sum(times)
    value = flops * len(times) / total / 1e12
    sample = "%d of %d (batch*head) slices per step, masked dense torch fp32 fwd+bwd" % (heads, w["batch"] * w["heads"])
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], **{k: w[k] for k in ("batch", "heads", "seq", "head_dim", "block")},
                       "sample": sample},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
OPS = ["sdd_qk", "softmax_fwd", "dsd_pv", "sdd_dp", "dsd_dv", "softmax_bwd", "dsd_dq", "dsd_dk"]


def device_step(ops, lay, q, k, v, do, scale, block, events=None):
    """The eight native calls of one forward + backward attention step (what the autograd ops issue)."""
    rl, cl = lay.row_layout, lay.col_layout
    calls = [
        lambda st: ops.sparse_matmul(q, k, "sdd", rl, cl, False, True, block),
        lambda st: ops.sparse_softmax_forward(st["s"], rl[0], rl[1], scale, False, None, lay.max_row_blocks),
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


def api_step(lay, q, k, v, do, scale):
    """The same step through the public autograd API."""
    from sparse import matmul, softmax
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))
    s = matmul(q, k, "sdd", lay, False, True)
    p = softmax(s, lay, scale)
    o = matmul(p, v, "dsd", lay, False, False)
    o.backward(do)
    return o.detach(), q.grad, k.grad, v.grad


def run_ours(args):
    import torch.distributed as dist
    from sparse import SparseLayout
    from sparse.kernel import sparse_ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the block-sparse kernels have no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit("bench.py: --gpus %d needs torchrun with %d ranks (WORLD_SIZE=%d)" % (args.gpus, args.gpus, world))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOAD
    z = args.slices or w["batch"] * w["heads"]
    block, seq, dim, scale = w["block"], w["seq"], w["head_dim"], w["scale"]
    pattern = workload_pattern()
    lay = SparseLayout(pattern, block=block, device=dev)
    nnz = lay.num_blocks
    first_head = rank * z           # weak scaling: every rank owns z slices, seeded by global index
    host = [seeded_heads(first_head, z, seq, dim, s).pin_memory() for s in range(4)]
    q, k, v, do = (t.to(dev, non_blocking=True) for t in host)
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

    # clocks are sampled from before the warm-up until after the end-to-end loop, so both timed
    # regions are covered (a timed region of a few tens of ms is shorter than one sampling period)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # ---- device-resident timing (value) with per-op events
    for _ in range(args.warmup):
        device_step(sparse_ops, lay, q, k, v, do, scale, block)
    barrier()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in OPS]
          for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        device_step(sparse_ops, lay, q, k, v, do, scale, block, ev[i])
    stop.record()
    barrier()
    sparse_ops.check_device_status(local_rank)
    elapsed_ms = start.elapsed_time(stop)
    op_ms = {name: sum(ev[i][j][0].elapsed_time(ev[i][j][1]) for i in range(args.steps)) / args.steps
             for j, name in enumerate(OPS)}

    # ---- end-to-end timing through the public API with host buffers.  Every step copies its four
    # inputs from pinned host memory, runs forward + backward through the autograd ops and copies the
    # four results back to pinned host memory.  Copies run on their own streams so that step i + 1's
    # upload and step i - 1's download overlap step i's kernels (double-buffered device inputs and
    # host outputs); the timed region covers all of it.
    e2e_steps = max(1, min(args.steps, 50))
    outs_host = [[torch.empty(z, seq, dim, dtype=torch.float16).pin_memory() for _ in range(4)] for _ in range(2)]
    dev_in = [[torch.empty(z, seq, dim, dtype=torch.float16, device=dev) for _ in range(4)] for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)

    def e2e_run(steps):
        computed = [None, None]          # event: kernels that read dev_in[b] are done
        downloaded = [None, None]        # event: outs_host[b] has been filled
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if computed[b] is not None:
                    s_in.wait_event(computed[b])
                for dst, src in zip(dev_in[b], host):
                    dst.copy_(src, non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(s_in)
            main.wait_event(uploaded)
            res = api_step(lay, *(t.detach() for t in dev_in[b]), scale)
            computed[b] = torch.cuda.Event()
            computed[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[b])
                for dst, src in zip(outs_host[b], res):
                    dst.copy_(src, non_blocking=True)
                    src.record_stream(s_out)
                downloaded[b] = torch.cuda.Event()
                downloaded[b].record(s_out)
        for ev in downloaded:
            if ev is not None:
                main.wait_event(ev)

    e2e_run(min(args.warmup, 3))
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    e2e_run(e2e_steps)
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)
    clocks = sampler.stop() if sampler else None

    # ---- DDS side measurement (not part of the step): dV^T = dO^T . P as dds(T,N)
    p_blocks = device_step(sparse_ops, lay, q, k, v, do, scale, block)["p"]
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        sparse_ops.sparse_matmul(do, p_blocks, "dds", lay.row_layout, lay.col_layout, True, False, block)
    d0.record()
    for _ in range(5):
        sparse_ops.sparse_matmul(do, p_blocks, "dds", lay.row_layout, lay.col_layout, True, False, block)
    d1.record()
    torch.cuda.synchronize()
    dds_ms = d0.elapsed_time(d1) / 5
    # the fused forward (one kernel for sdd -> softmax -> dsd), reported beside the unfused operators
    from sparse.attention import attention_lse
    for _ in range(3):
        attention_lse(q, k, v, lay, scale)
    d0.record()
    for _ in range(10):
        attention_lse(q, k, v, lay, scale)
    d1.record()
    torch.cuda.synchronize()
    fused_ms = d0.elapsed_time(d1) / 10
    # the fused backward (statistics, dQ by block rows, dK / dV by block columns) from the fused forward's output
    o_f, lse_f = attention_lse(q, k, v, lay, scale)
    rl_f, cl_f = lay.row_layout, lay.col_layout
    for _ in range(3):
        sparse_ops.sparse_attention_backward(q, k, v, o_f, do, lse_f, rl_f[0], rl_f[1], cl_f[0], cl_f[1], block, scale, False, None)
    d0.record()
    for _ in range(10):
        sparse_ops.sparse_attention_backward(q, k, v, o_f, do, lse_f, rl_f[0], rl_f[1], cl_f[0], cl_f[1], block, scale, False, None)
    d1.record()
    torch.cuda.synchronize()
    sparse_ops.check_device_status(local_rank)
    fused_bwd_ms = d0.elapsed_time(d1) / 10

    # ---- max over ranks
    t = torch.tensor([elapsed_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peaks = load_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = 6 * flops_matmul * world / (ms_per_step * 1e-3) / 1e12
        e2e_value = 6 * flops_matmul * world / (e2e_ms / e2e_steps * 1e-3) / 1e12
        ops_report = {}
        for name in OPS:
            gbs = alg_bytes[name] / (op_ms[name] * 1e-3) / 1e9
            entry = {"ms": round(op_ms[name], 4), "GB/s": round(gbs, 1), "hbm_frac": round(gbs / peaks["hbm_gbs"], 4)}
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
        fused_report = {"kernel": "attention_forward_kernel", "ms": round(fused_ms, 4),
                        "TFLOP/s": round(fused_tf, 1), "tensor_frac": round(fused_tf / peaks["bf16_tflops"], 4),
                        "unfused_forward_ms": round(unfused_fwd_ms, 4), "speedup": round(unfused_fwd_ms / fused_ms, 2),
                        "hbm_bytes": 4 * dense_bytes,
                        "note": "forward only, outside the timed step; Q, K, V read and O written once, "
                                "scores and probabilities never leave the SM"}
        fused_step_ms = fused_ms + fused_bwd_ms
        fused_step_report = {"kernels": "attention_forward_kernel + attention_backward_kernel<rows> + <columns> (+ statistics)",
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
        # DRAM bytes per launch from the ncu capture under profiles/ (taken at 32 slices, where every
        # byte of the sparse operand is read once; traffic grows in proportion to the slices)
        ncu_traffic_per_slice = {"tc_matmul_kernel<dsd> (4 launches/step)": 231.0e6 / 32}
        traffic = ncu_traffic_per_slice.get(dom)
        traffic = None if traffic is None else round(traffic * z)
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        cpu_dt = cpu_flops = cpu_heads = None
        if world == 1 and not args.no_cpu:
            probe_dt, _ = cpu_attention_sample(1)                    # size the sample: about 10 s of CPU work
            cpu_heads = int(max(2, min(z, 10.0 / max(probe_dt, 1e-3))))
            cpu_dt, cpu_flops = cpu_attention_sample(cpu_heads)
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": w["name"] + ("" if z == w["batch"] * w["heads"] else "_REDUCED_%d_slices" % z),
                       "batch_per_gpu": w["batch"], "heads": w["heads"], "slices_per_gpu": z, "seq": seq,
                       "head_dim": dim, "block": block, "nnz_blocks_per_head": nnz,
                       "layout": "strided(8)+local(2), non-causal", "parallelism": "head-sharded x%d" % world,
                       "l2": "no flush: the four sparse tensors of a step are 400 MB each, above the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": traffic,
                         "peak_source": peaks["source"]},
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "steps": e2e_steps,
                    "ms_per_step": round(e2e_ms / e2e_steps, 4),
                    "h2d_bytes_per_step": 4 * dense_bytes, "d2h_bytes_per_step": 4 * dense_bytes},
            "gpu_launches": len(OPS) * args.steps,
            "clocks": clocks, "ops": ops_report, "fused_forward": fused_report, "fused_step": fused_step_report,
            "engine": os.environ.get("BSA_MATMUL_ENGINE", "auto"),
        }
        if cpu_dt is not None:
            line["cpu_baseline"] = {"value": round(cpu_flops / cpu_dt / 1e12, 5), "unit": "TFLOP/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": "%d of %d (batch*head) slices, masked dense torch fp32 fwd+bwd, %.1f s" % (cpu_heads, z, cpu_dt)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--slices", type=int, default=0,
                    help="(batch*head) slices per GPU; default is the workload's 64. A smaller value is a reduced "
                         "case for profiler captures, not a benchmark result")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()
