"""Benchmark of the block-scaled FP8 GEMM path on B200 (one JSON line on stdout, rank 0).

    python bench.py --gpus N --steps K --warmup W [--workload dense_fp8] [--impl reference]

Workloads (all synthetic: seeded N(0,1) bf16 matrices quantised to e4m3 with per-128 UE8M0 scales):
  dense_fp8   (default at N = 1) one step = one pass over the ten dense DeepSeek-V3 projection GEMMs
              M in {128, 4096} x (N, K) in {(2112,7168), (24576,1536), (7168,16384), (4096,7168), (7168,2048)}.
              The dense GEMM does not shard; with --workload dense_fp8 at N > 1 every rank runs a replica.
  moe_ep      (default at N > 1) the contiguous m-grouped FP8 GEMM pair of a DeepSeek-V3 MoE layer, experts
              sharded 256/N per GPU: 8192 tokens per rank, top-8 of 256 experts from softmax of seeded N(0,1)
              router logits; one step = plan + all-to-all dispatch of e4m3 rows and scales + gate/up grouped
              GEMM (N=4096, K=7168) + down grouped GEMM (N=7168, K=2048, on an independent resident operand:
              the benchmark defines the two GEMMs as independent) + all-to-all combine and weighted
              reduction.  Flops count the routed (unpadded) rows of both GEMMs.
The metric is whole-job TFLOP/s: 2*M*N*K summed over the GEMMs of a step, times ranks, over the
step time (CUDA events, max over ranks).  `e2e` is the same pass driven from pinned host buffers
(operands copied host->device and the result device->host inside the timed region).
`--impl reference` times the CPU restatement of the reference crate's own CPU GEMM
(deepgemm/src/reference.rs:85-114) on all host threads, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DENSE_NK = [(2112, 7168), (24576, 1536), (7168, 16384), (4096, 7168), (7168, 2048)]
DENSE_SHAPES = [(m, n, k) for m in (128, 4096) for (n, k) in DENSE_NK]
DOMINANT = (4096, 7168, 16384)            # the launch the roofline entry describes
CPU_SAMPLE_ROWS, CPU_SAMPLE_COLS = 32, 256  # per GEMM, for the CPU legs


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dense_flops():
    return sum(2 * m * n * k for (m, n, k) in DENSE_SHAPES)


def cpu_sample_inputs(seed=7):
    """Quantised operands of the bounded CPU sample: the first rows / columns of every dense GEMM."""
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    cases = []
    for (m, n, k) in DENSE_SHAPES:
        rows, cols = min(CPU_SAMPLE_ROWS, m), min(CPU_SAMPLE_COLS, n)
        a = O.bf16_bits(rng.standard_normal((rows, k)).astype(np.float32))
        b = O.bf16_bits(rng.standard_normal((cols, k)).astype(np.float32))
        aq, ae = O.quantize_fp8_ue8m0_blocks(a, k, 1)
        bq, be = O.quantize_fp8_ue8m0_blocks(b, k, 128)
        cases.append((aq, O.exps_to_f32(ae), bq, O.exps_to_f32(be), rows, cols, k))
    return cases


def cpu_step(cases, threads):
    from oracle import oracle as O
    t0 = time.perf_counter()
    for (aq, sfa, bq, sfb, rows, cols, k) in cases:
        O.ref_fp8_gemm_nt(aq, sfa, bq, sfb, threads=threads)
    return time.perf_counter() - t0


def cpu_sample_flops(cases):
    return sum(2 * rows * cols * k for (_, _, _, _, rows, cols, k) in cases)


def run_reference(args):
    """The reference's CPU implementation of the path, all host threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    threads = O.max_threads()
    cases = cpu_sample_inputs()
    for _ in range(max(args.warmup, 0)):
        cpu_step(cases, threads)
    times = [cpu_step(cases, threads) for _ in range(max(args.steps, 1))]
    sec = sum(times) / len(times)
    value = cpu_sample_flops(cases) / sec / 1e12
    sample = f"first {CPU_SAMPLE_ROWS} rows x {CPU_SAMPLE_COLS} columns of each of the {len(DENSE_SHAPES)} dense GEMMs, full K"
    line = {"impl": "reference", "metric": "fp8_block_scaled_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": "dense_fp8_dsv3", "shapes": DENSE_SHAPES, "gran_k": 128, "out": "f32 (CPU)"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


MOE = {"experts": 256, "topk": 8, "tokens_per_rank": 8192, "hidden": 7168, "gate_up_n": 4096, "down_k": 2048, "down_n": 7168}


def run_moe(args, torch, dist, dg, rank, world, local_rank):
    """Expert-parallel contiguous grouped GEMM workload (see the module docstring)."""
    from deepgemm_rust_b200.moe_ep import DeviceRowOps, ExpertParallel
    c = MOE
    dev = torch.device("cuda", local_rank)
    ctx = dg.DgContext(local_rank)
    peaks = measured_peaks()
    local_e = c["experts"] // world
    gen = torch.Generator(device=dev).manual_seed(3000 + rank)

    def quant_weights(n, k):
        q = torch.empty((local_e * n, k), dtype=torch.uint8, device=dev)
        sf = dg.alloc_sf(ctx, local_e * n, k, 128, local_e)
        cols, stride, chunk = dg.sf_packed_cols(k, 128), dg.sf_aligned_rows(n), 8
        for g0 in range(0, local_e, chunk):
            gn = min(chunk, local_e - g0)
            w = torch.randn((gn * n, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            wq, wsf = dg.cast_bf16_to_fp8_sf_dev(ctx, w, k, gn * n, k, 128, gn)
            q[g0 * n:(g0 + gn) * n] = wq
            sf.view(local_e, cols, stride)[g0:g0 + gn] = wsf.view(gn, cols, stride)
        return q, sf

    w1q, w1sf = quant_weights(c["gate_up_n"], c["hidden"])
    w2q, w2sf = quant_weights(c["down_n"], c["down_k"])
    tokens = c["tokens_per_rank"]
    x = torch.randn((tokens, c["hidden"]), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn((tokens, c["experts"]), generator=gen, device=dev, dtype=torch.float32)
    topw, topi = torch.softmax(logits, -1).topk(c["topk"], dim=-1)
    topw = topw.contiguous()
    xq, xsf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, c["hidden"], tokens, c["hidden"], 128)
    ep = ExpertParallel(c["experts"], c["topk"], DeviceRowOps(ctx))
    cap = 2 * tokens * c["topk"] + 128 * local_e            # arena capacity for the resident down-GEMM operand
    act = torch.randn((cap, c["down_k"]), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    actq, actsf_full = dg.cast_bf16_to_fp8_sf_dev(ctx, act, c["down_k"], cap, c["down_k"], 128)
    del act
    w1 = dg.LpOperand(w1q, w1sf, local_e * c["gate_up_n"], c["hidden"], c["hidden"])
    w2 = dg.LpOperand(w2q, w2sf, local_e * c["down_n"], c["down_k"], c["down_k"])
    ctx.sync()
    stats = {}

    def step(xq_, xsf_, topi_, topw_):
        plan = ep.plan(topi_)
        if plan.m_pad > cap:
            raise RuntimeError(f"arena of {plan.m_pad} rows exceeds the benchmark capacity {cap}")
        a, a_sf = ep.dispatch(plan, xq_, xsf_, c["hidden"])
        h = torch.empty((plan.m_pad, c["gate_up_n"]), dtype=torch.bfloat16, device=dev)
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(a, a_sf, plan.m_pad, c["hidden"], c["hidden"]), plan.m_indices, w1,
                                                 dg.Sm100Out.Bf16(h, c["gate_up_n"]), local_e)
        # the resident operand's scale words use stride align4(cap); the GEMM wants stride align4(m_pad): rows are a prefix,
        # so pass the full-capacity view (rows = cap) and let the group table bound the work
        y = torch.empty((cap, c["down_n"]), dtype=torch.bfloat16, device=dev)
        m_idx_cap = torch.full((cap,), -1, dtype=torch.int32, device=dev)
        m_idx_cap[:plan.m_pad] = plan.m_indices
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(actq, actsf_full, cap, c["down_k"], c["down_k"]), m_idx_cap, w2,
                                                 dg.Sm100Out.Bf16(y, c["down_n"]), local_e)
        out = ep.combine(plan, y, topw_)
        stats["rows"] = plan.n_recv
        stats["m_pad"] = plan.m_pad
        return out

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step(xq, xsf, topi, topw)
    fence()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step(xq, xsf, topi, topw)
    end.record()
    fence()
    t = torch.tensor([start.elapsed_time(end)], device=dev, dtype=torch.float64)
    rows = torch.tensor([float(stats["rows"])], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows, op=dist.ReduceOp.SUM)
    ms_per_step = float(t.item()) / args.steps
    flops_per_row = 2.0 * (c["gate_up_n"] * c["hidden"] + c["down_n"] * c["down_k"])
    value = float(rows.item()) * flops_per_row / (ms_per_step * 1e-3) / 1e12

    # the gate/up grouped GEMM alone (dominant kernel of this workload), CUDA events on its stream
    plan = ep.plan(topi)
    a, a_sf = ep.dispatch(plan, xq, xsf, c["hidden"])
    h = torch.empty((plan.m_pad, c["gate_up_n"]), dtype=torch.bfloat16, device=dev)
    a_op = dg.LpOperand(a, a_sf, plan.m_pad, c["hidden"], c["hidden"])
    times = []
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a_op, plan.m_indices, w1, dg.Sm100Out.Bf16(h, c["gate_up_n"]), local_e)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    gemm_ms = statistics.median(times[1:])
    fence()

    # end to end from pinned host buffers: this rank's quantised tokens, scales, routing in; reduced rows out
    e2e = None
    if not args.no_e2e:
        hx, hsf, hi, hw = xq.cpu().pin_memory(), xsf.cpu().pin_memory(), topi.cpu().pin_memory(), topw.cpu().pin_memory()
        hout = torch.empty((tokens, c["down_n"]), dtype=torch.bfloat16).pin_memory()
        dx, dsf, di, dw = torch.empty_like(xq), torch.empty_like(xsf), torch.empty_like(topi), torch.empty_like(topw)

        def e2e_step():
            dx.copy_(hx, non_blocking=True)
            dsf.copy_(hsf, non_blocking=True)
            di.copy_(hi, non_blocking=True)
            dw.copy_(hw, non_blocking=True)
            hout.copy_(step(dx, dsf, di, dw), non_blocking=True)

        e2e_steps = max(3, min(args.steps, 10))
        e2e_step()
        fence()
        start.record()
        for _ in range(e2e_steps):
            e2e_step()
        end.record()
        fence()
        t = torch.tensor([start.elapsed_time(end)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / e2e_steps
        h2d = sum(z.numel() * z.element_size() for z in (hx, hsf, hi, hw))
        e2e = {"value": float(rows.item()) * flops_per_row / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": hout.numel() * hout.element_size(), "ms_per_step": e2e_ms, "steps": e2e_steps}
    clocks = sampler.stop() if rank == 0 else None
    ctx.sync()
    if rank == 0:
        n_valid = plan.n_recv
        gemm_flops = 2.0 * n_valid * c["gate_up_n"] * c["hidden"]
        gemm_bytes = n_valid * c["hidden"] + local_e * c["gate_up_n"] * c["hidden"] + n_valid * c["gate_up_n"] * 2
        t_tensor = gemm_flops / (2 * peaks["bf16_tflops_sustained"] * 1e12)
        t_hbm = gemm_bytes / (peaks["hbm_gbs"] * 1e9)
        if t_hbm > t_tensor:
            roofline = {"bound": "hbm", "achieved": gemm_bytes / (gemm_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s"}
        else:
            roofline = {"bound": "tensor", "achieved": gemm_flops / (gemm_ms * 1e-3) / 1e12, "peak": 2 * peaks["bf16_tflops_sustained"],
                        "unit": "TFLOP/s"}
        roofline.update({"frac": roofline["achieved"] / roofline["peak"], "traffic": None,
                         "kernel": "dg_gemm_kernel<fp8, bf16 out> contiguous grouped, gate/up",
                         "launch": f"rank 0: {n_valid} routed rows over {local_e} local experts, N={c['gate_up_n']} K={c['hidden']}",
                         "peak_source": f"{peaks['source']} peaks (tensor: 2 x bf16 sustained)", "us": gemm_ms * 1e3})
        line = {"metric": "fp8_block_scaled_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp8_e4m3", "data": "synthetic",
                "config": {"workload": "moe_contiguous_ep", **c, "experts_per_gpu": local_e, "mk_alignment": 128,
                           "parallelism": f"ep{world}", "collective": "nccl all_to_all_single" if world > 1 else "none",
                           "l2": "weights of one rank (0.9-7.5 GB) and the arena exceed the 126 MB L2"},
                "clocks": clocks, "gpu_launches": args.steps * 10, "roofline": roofline}
        if e2e is not None:
            line["e2e"] = e2e
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="dgb200")
    ap.add_argument("--workload", default=None, help="dense_fp8 (default at 1 GPU) or moe_ep (default at more)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--moe-experts", type=int, default=None, help="moe_ep: total experts (default 256); 32 gives one rank of an 8-GPU job")
    ap.add_argument("--only", default=None, help="M,N,K: restrict the dense pass to one GEMM (profiling captures)")
    args = ap.parse_args()
    if args.only:
        global DENSE_SHAPES, DOMINANT
        DOMINANT = tuple(int(x) for x in args.only.split(","))
        DENSE_SHAPES = [DOMINANT]
    if args.moe_experts:
        MOE["experts"] = args.moe_experts
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    import deepgemm_rust_b200 as dg

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    workload = args.workload or ("dense_fp8" if world == 1 else "moe_ep")
    if workload == "moe_ep":
        run_moe(args, torch, dist, dg, rank, world, local_rank)
        return
    dev = torch.device("cuda", local_rank)
    ctx = dg.DgContext(local_rank)
    peaks = measured_peaks()

    # ---- build the workload (untimed): operands resident in HBM, quantised by the library's own kernels
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    problems = []
    for (m, n, k) in DENSE_SHAPES:
        a = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        b = torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, a, k, m, k, 128)
        bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, b, k, n, k, 128)
        d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        problems.append({"shape": (m, n, k), "a": dg.LpOperand(aq, asf, m, k, k), "b": dg.LpOperand(bq, bsf, n, k, k),
                         "out": dg.Sm100Out.Bf16(d, n), "d": d})
        del a, b
    ctx.sync()

    def step(record=None):
        for p in problems:
            mark = record is not None and p["shape"] == DOMINANT
            if mark:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
            dg.fp8_fp4_gemm_dev(ctx, p["a"], p["b"], p["out"])
            if mark:
                e1.record()
                record.append((e0, e1))

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    fence()
    dominant_events = []
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    n_before = len(sampler.samples)
    start.record()
    for _ in range(args.steps):
        step(dominant_events)
    end.record()
    fence()
    n_timed = len(sampler.samples) - n_before
    ms = start.elapsed_time(end)
    # the timed region lasts milliseconds; keep the same step loop running for about a second so the
    # clock record also shows what the GPU settles at under this load
    if rank == 0:
        t_soak = time.perf_counter()
        while time.perf_counter() - t_soak < 1.2:
            for _ in range(20):
                step()
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "warm-up + timed region + 1.2 s of the same step loop"
        clocks["samples_in_timed_region"] = n_timed
    if world > 1:
        dist.barrier()
    ctx.sync()
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = dense_flops() * world / (ms_per_step * 1e-3) / 1e12
    dom_ms = sum(a.elapsed_time(b) for a, b in dominant_events) / max(len(dominant_events), 1)

    # per-GEMM timings (each launch alone, L2 flushed by a 256 MB write in between), for the report
    per_shape = []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for p in problems:
        m, n, k = p["shape"]
        times = []
        for _ in range(5):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dg.fp8_fp4_gemm_dev(ctx, p["a"], p["b"], p["out"])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        t_ms = statistics.median(times[1:])
        alg_bytes = m * k + n * k + 2 * m * n + 4 * ((k + 511) // 512) * (m + n)
        per_shape.append({"m": m, "n": n, "k": k, "us": round(t_ms * 1e3, 2), "tflops": round(2 * m * n * k / t_ms / 1e9, 1),
                          "gbs": round(alg_bytes / t_ms / 1e6, 1)})
    del flush

    # ---- end to end from pinned host buffers through the same public call
    e2e = None
    if not args.no_e2e:
        host = []
        for p in problems:
            h = {}
            for name, ten in (("a", p["a"].data), ("asf", p["a"].sf), ("b", p["b"].data), ("bsf", p["b"].sf)):
                h[name] = ten.cpu().pin_memory()
            h["d"] = torch.empty(p["d"].shape, dtype=p["d"].dtype).pin_memory()
            host.append(h)
        h2d = sum(h[n].numel() * h[n].element_size() for h in host for n in ("a", "asf", "b", "bsf"))
        d2h = sum(h["d"].numel() * h["d"].element_size() for h in host)

        def e2e_step():
            for p, h in zip(problems, host):
                p["a"].data.copy_(h["a"], non_blocking=True)
                p["a"].sf.copy_(h["asf"], non_blocking=True)
                p["b"].data.copy_(h["b"], non_blocking=True)
                p["b"].sf.copy_(h["bsf"], non_blocking=True)
                dg.fp8_fp4_gemm_dev(ctx, p["a"], p["b"], p["out"])
                h["d"].copy_(p["d"], non_blocking=True)

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        fence()
        start.record()
        for _ in range(e2e_steps):
            e2e_step()
        end.record()
        fence()
        t = torch.tensor([start.elapsed_time(end)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / e2e_steps
        e2e = {"value": dense_flops() * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps}
        ctx.sync()

    if rank == 0:
        m, n, k = DOMINANT
        achieved = 2 * m * n * k / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else None
        peak = 2 * peaks["bf16_tflops_sustained"]
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak if achieved else None,
                    # dram__bytes_read.sum + dram__bytes_write.sum of this launch, one ncu capture
                    # (profiles/dg_gemm_kernel_fp8_M4096_N7168_K16384.md); algorithmic bytes are 2.447e8
                    "traffic": 6.48e8 if DOMINANT == (4096, 7168, 16384) else None,
                    "kernel": "dg_gemm_kernel<fp8, bf16 out>", "launch": f"M={m} N={n} K={k}",
                    "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} peaks (e4m3 issues at twice the bf16 rate)",
                    "frac_of_nominal_fp8_4500": achieved / 4500.0 if achieved else None}
        line = {"metric": "fp8_block_scaled_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp8_e4m3", "data": "synthetic",
                "config": {"workload": "dense_fp8_dsv3", "shapes": DENSE_SHAPES, "gran_k": 128, "out": "bf16",
                           "parallelism": "replicas only" if world > 1 else "single GPU",
                           "l2": "ten GEMMs per step touch 1.1 GB of operands, far more than the 126 MB L2"},
                "clocks": clocks, "gpu_launches": args.steps * len(problems), "roofline": roofline, "per_gemm": per_shape}
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as O
            threads = O.max_threads()
            cases = cpu_sample_inputs()
            sec = cpu_step(cases, threads)
            line["cpu_baseline"] = {"value": cpu_sample_flops(cases) / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"first {CPU_SAMPLE_ROWS} rows x {CPU_SAMPLE_COLS} columns of each dense GEMM, full K, one pass "
                                              f"({sec:.1f} s)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
