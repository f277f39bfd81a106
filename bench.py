"""Benchmark of the block-scaled FP8 GEMM path on B200 (one JSON line on stdout, rank 0).

    python bench.py --gpus N --steps K --warmup W [--workload dense_fp8] [--impl reference]

Workloads (all synthetic: seeded N(0,1) bf16 matrices quantised to e4m3 with per-128 UE8M0 scales):
  dsv3        (default at every N) one step = the dense_fp8 pass followed by the moe_ep step below, i.e. every FP8
              GEMM configuration the benchmark contract names, the same work per GPU at every N (weak scaling).
              The dense GEMMs do not shard (every rank runs its own replica); the grouped GEMMs shard by expert.
              `parts` in the JSON line gives each half on its own.
  dense_fp8   one step = one pass over the ten dense DeepSeek-V3 projection GEMMs
              M in {128, 4096} x (N, K) in {(2112,7168), (24576,1536), (7168,16384), (4096,7168), (7168,2048)}.
              The dense GEMM does not shard; at N > 1 every rank runs a replica.
  moe_ep      the contiguous m-grouped FP8 GEMM pair of a DeepSeek-V3 MoE layer, experts
              sharded 256/N per GPU: 8192 tokens per rank, top-8 of 256 experts from softmax of seeded N(0,1)
              router logits; one step = plan + all-to-all dispatch of e4m3 rows and scales + gate/up grouped
              GEMM (N=4096, K=7168) + silu(gate)*up quantised to e4m3 + down grouped GEMM (N=7168, K=2048)
              on that activation + all-to-all combine and weighted reduction.  Flops count the routed
              (unpadded) rows of both GEMMs only.
  configs     (report, one GPU) every benchmark configuration launched alone against its roofline: the ten dense
              shapes, MXFP4 and FP8xFP4 4096x7168x7168, the quantisers, the masked decode GEMM with FP8 output, and the
              grouped GEMM pair with its row movers for one rank of a 1-GPU and of an 8-GPU job.
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
    """Quantised operands of the bounded CPU sample: the first rows / columns of every dense GEMM, and a 4-expert slice
    (32 rows each, 256 columns) of the two grouped GEMMs."""
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    cases = []
    for (m, n, k) in DENSE_SHAPES:
        rows, cols = min(CPU_SAMPLE_ROWS, m), min(CPU_SAMPLE_COLS, n)
        a = O.bf16_bits(rng.standard_normal((rows, k)).astype(np.float32))
        b = O.bf16_bits(rng.standard_normal((cols, k)).astype(np.float32))
        aq, ae = O.quantize_fp8_ue8m0_blocks(a, k, 1)
        bq, be = O.quantize_fp8_ue8m0_blocks(b, k, 128)
        cases.append(("dense", aq, O.exps_to_f32(ae), bq, O.exps_to_f32(be), rows, cols, k, None))
    experts, rows_per = 4, CPU_SAMPLE_ROWS
    m_idx = np.repeat(np.arange(experts, dtype=np.int32), rows_per)
    for (n, k) in ((MOE["gate_up_n"], MOE["hidden"]), (MOE["down_n"], MOE["down_k"])):
        cols = min(CPU_SAMPLE_COLS, n)
        a = O.bf16_bits(rng.standard_normal((experts * rows_per, k)).astype(np.float32))
        b = O.bf16_bits(rng.standard_normal((experts * cols, k)).astype(np.float32))
        aq, ae = O.quantize_fp8_ue8m0_blocks(a, k, 1)
        bq, be = O.quantize_fp8_ue8m0_blocks(b, k, 128)
        cases.append(("grouped", aq, O.exps_to_f32(ae), bq, O.exps_to_f32(be), experts * rows_per, cols, k, m_idx))
    return cases


def cpu_step(cases, threads):
    from oracle import oracle as O
    t0 = time.perf_counter()
    for (kind, aq, sfa, bq, sfb, rows, cols, k, m_idx) in cases:
        if kind == "dense":
            O.ref_fp8_gemm_nt(aq, sfa, bq, sfb, threads=threads)
        else:
            O.ref_m_grouped_contiguous(aq, sfa, m_idx, bq, sfb.reshape(-1), cols, per_group_sfb=True, threads=threads)
    return time.perf_counter() - t0


def cpu_sample_flops(cases):
    return sum(2 * c[5] * c[6] * c[7] for c in cases)


CPU_SAMPLE_TEXT = (f"first {CPU_SAMPLE_ROWS} rows x {CPU_SAMPLE_COLS} columns of each of the ten dense GEMMs, and 4 experts x "
                   f"{CPU_SAMPLE_ROWS} rows x {CPU_SAMPLE_COLS} columns of the two grouped GEMMs, full K")


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
    sample = CPU_SAMPLE_TEXT
    line = {"impl": "reference", "metric": "fp8_block_scaled_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": "dsv3_fp8_gemms (dense pass + expert-parallel MoE pair)", "gran_k": 128, "out": "f32 (CPU)",
                       "dense_shapes": DENSE_SHAPES, "moe": MOE},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


MOE = {"experts": 256, "topk": 8, "tokens_per_rank": 8192, "hidden": 7168, "gate_up_n": 4096, "down_k": 2048, "down_n": 7168}


class DenseWork:
    """The ten dense FP8 GEMMs; operands quantised once by the library's own kernels and kept resident."""

    def __init__(self, torch, dg, ctx, dev, seed):
        self.torch, self.dg, self.ctx = torch, dg, ctx
        gen = torch.Generator(device=dev).manual_seed(seed)
        self.problems = []
        for (m, n, k) in DENSE_SHAPES:
            a = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            b = torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, a, k, m, k, 128)
            bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, b, k, n, k, 128)
            d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            self.problems.append({"shape": (m, n, k), "a": dg.LpOperand(aq, asf, m, k, k), "b": dg.LpOperand(bq, bsf, n, k, k),
                                  "out": dg.Sm100Out.Bf16(d, n), "d": d})
            del a, b
        self.flops = float(dense_flops())           # per rank per step
        # GEMM launches plus the reduce launch of every GEMM whose K is cut into ranges
        self.launches = len(self.problems) + sum(1 for (m, n, k) in DENSE_SHAPES if dg.best_config(dg.Sm100Desc(0, m, n, k)).num_splits > 1)
        self.host = None

    def step(self, record=None):
        torch, dg = self.torch, self.dg
        for p in self.problems:
            mark = record is not None and p["shape"] == DOMINANT
            if mark:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            dg.fp8_fp4_gemm_dev(self.ctx, p["a"], p["b"], p["out"])
            if mark:
                e1.record()
                record.append((e0, e1))

    def e2e_setup(self):
        torch = self.torch
        self.host = []
        for p in self.problems:
            h = {name: ten.cpu().pin_memory() for name, ten in (("a", p["a"].data), ("asf", p["a"].sf), ("b", p["b"].data), ("bsf", p["b"].sf))}
            h["d"] = torch.empty(p["d"].shape, dtype=p["d"].dtype).pin_memory()
            self.host.append(h)
        h2d = sum(h[n].numel() * h[n].element_size() for h in self.host for n in ("a", "asf", "b", "bsf"))
        d2h = sum(h["d"].numel() * h["d"].element_size() for h in self.host)
        return h2d, d2h

    def e2e_step(self, pipes):
        """Operands in on the upload stream, GEMM on the compute stream, D out on the download stream: the copies of one
        GEMM overlap the others' compute and each other (PCIe is full duplex).  Events order each buffer's writers and readers,
        across steps too (an operand is not overwritten before the previous step's GEMM has read it, D not before it has left)."""
        torch = self.torch
        main = torch.cuda.current_stream()
        for p, h in zip(self.problems, self.host):
            with torch.cuda.stream(pipes.up):
                if "done" in h:
                    pipes.up.wait_event(h["done"])
                p["a"].data.copy_(h["a"], non_blocking=True)
                p["a"].sf.copy_(h["asf"], non_blocking=True)
                p["b"].data.copy_(h["b"], non_blocking=True)
                p["b"].sf.copy_(h["bsf"], non_blocking=True)
                landed = h.setdefault("landed", torch.cuda.Event())
                landed.record(pipes.up)
            main.wait_event(landed)
            if "left" in h:
                main.wait_event(h["left"])
            self.dg.fp8_fp4_gemm_dev(self.ctx, p["a"], p["b"], p["out"])
            done = h.setdefault("done", torch.cuda.Event())
            done.record(main)
            with torch.cuda.stream(pipes.down):
                pipes.down.wait_event(done)
                h["d"].copy_(p["d"], non_blocking=True)
                left = h.setdefault("left", torch.cuda.Event())
                left.record(pipes.down)

    def per_gemm(self):
        """Each launch alone with the L2 flushed by a 256 MB write before it (for the report)."""
        torch, dg = self.torch, self.dg
        out = []
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.problems[0]["d"].device)
        for p in self.problems:
            m, n, k = p["shape"]
            times = []
            for _ in range(5):
                flush.fill_(1)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                dg.fp8_fp4_gemm_dev(self.ctx, p["a"], p["b"], p["out"])
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            t_ms = statistics.median(times[1:])
            alg_bytes = m * k + n * k + 2 * m * n + 4 * ((k + 511) // 512) * (m + n)
            out.append({"m": m, "n": n, "k": k, "us": round(t_ms * 1e3, 2), "tflops": round(2 * m * n * k / t_ms / 1e9, 1),
                        "gbs": round(alg_bytes / t_ms / 1e6, 1)})
        return out


class MoeWork:
    """Expert-parallel contiguous grouped GEMM pair (see the module docstring)."""

    def __init__(self, torch, dist, dg, ctx, dev, rank, world, exchange="peer", chunks=1, blocks_per_sm=2, fused_act=False):
        from deepgemm_rust_b200.moe_ep import DeviceRowOps, ExpertParallel, PeerExpertParallel, PipelinedPeerMoe
        self.torch, self.dg, self.ctx, self.dev, self.world = torch, dg, ctx, dev, world
        c = self.c = dict(MOE)
        self.local_e = local_e = c["experts"] // world
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
        self.tokens = tokens = c["tokens_per_rank"]
        x = torch.randn((tokens, c["hidden"]), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        logits = torch.randn((tokens, c["experts"]), generator=gen, device=dev, dtype=torch.float32)
        topw, self.topi = torch.softmax(logits, -1).topk(c["topk"], dim=-1)
        self.topw = topw.contiguous()
        self.xq, self.xsf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, c["hidden"], tokens, c["hidden"], 128)
        del x
        # rows travel through peer memory (kernels of the library) unless the peers cannot be mapped; every rank must agree
        self.peer, self.pipe, self.chunks, self.exchange_note = None, None, max(1, chunks), "nccl all_to_all_single"
        self.fused_act = False
        if exchange == "peer":
            try:
                if self.chunks > 1:
                    self.pipe = PipelinedPeerMoe(ctx, c["experts"], c["topk"], tokens, c["hidden"], c["down_n"], self.chunks,
                                                 blocks_per_sm=blocks_per_sm)
                    self.peer = self.pipe.exchanges[0]
                else:
                    self.peer = PeerExpertParallel(ctx, c["experts"], c["topk"], tokens, c["hidden"], c["down_n"])
                ok = 1
            except dg.DgError as e:
                ok, self.exchange_note = 0, f"nccl all_to_all_single (peer mapping failed: {e})"
            if world > 1:
                agreed = torch.tensor([ok], device=dev, dtype=torch.int32)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                ok = int(agreed.item())
            if not ok and self.peer is not None:
                (self.pipe or self.peer).close()
                self.peer, self.pipe, self.exchange_note = None, None, "nccl all_to_all_single (a peer could not be mapped)"
        if self.peer is not None:
            cap = self.peer.capacity
            self.exchange_note = "peer-memory stores/loads (library kernels) + count all-gather" if world > 1 else "none (local arena)"
            if self.pipe is not None:
                self.exchange_note += f"; {self.chunks} token micro-batches, exchange of one overlapping the GEMMs of another"
            # per micro-batch: gate/up output (only when the activation is a kernel of its own) and the quantised activation
            # (capacity rows each); the fused epilogue writes one scale per 32 columns, the separate kernel one per 128
            self.fused_act = fused_act
            self.act_gran = 32 if fused_act else 128
            self.bufs = {id(pe): (None if fused_act else torch.empty((cap, c["gate_up_n"]), dtype=torch.bfloat16, device=dev),
                                  (torch.empty((cap, c["down_k"]), dtype=torch.uint8, device=dev), dg.alloc_sf(ctx, cap, c["down_k"], self.act_gran)))
                         for pe in (self.pipe.exchanges if self.pipe is not None else [self.peer])}
            self.h, self.act = self.bufs[id(self.peer)]
        else:
            self.ep = ExpertParallel(c["experts"], c["topk"], DeviceRowOps(ctx))
        self.w1 = dg.LpOperand(w1q, w1sf, local_e * c["gate_up_n"], c["hidden"], c["hidden"])
        self.w2 = dg.LpOperand(w2q, w2sf, local_e * c["down_n"], c["down_k"], c["down_k"])
        self.flops_per_row = 2.0 * (c["gate_up_n"] * c["hidden"] + c["down_n"] * c["down_k"])
        self.rows = 0
        if self.peer is not None:
            # per micro-batch: pair ranking, chunk scan, layout, dispatch, 2 GEMMs, combine (+ the SiLU-mul quantiser when not fused)
            self.launches = (7 if self.fused_act else 8) * self.chunks
        else:
            # pack, unpack, 2 x (group-end kernel, scan kernel, GEMM), SiLU-mul quantiser, combine, plus the result gather when rows travel
            self.launches = 10 + (1 if world > 1 else 0)
        self.host = None

    def step(self, xq=None, xsf=None, topi=None, topw=None):
        torch, dg, c, ctx = self.torch, self.dg, self.c, self.ctx
        xq = self.xq if xq is None else xq
        xsf = self.xsf if xsf is None else xsf
        topi = self.topi if topi is None else topi
        topw = self.topw if topw is None else topw
        if self.pipe is not None:
            return self.pipe.run(topi, xq, xsf, topw, self.experts_compute)
        if self.peer is not None:
            pe = self.peer
            a_op, ends = pe.dispatch(topi, xq, xsf)
            self.experts_compute(pe, a_op, ends)
            return pe.combine(topw)
        plan = self.ep.plan(topi)
        a, a_sf = self.ep.dispatch(plan, xq, xsf, c["hidden"])
        h = torch.empty((plan.m_pad, c["gate_up_n"]), dtype=torch.bfloat16, device=self.dev)
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(a, a_sf, plan.m_pad, c["hidden"], c["hidden"]), plan.m_indices, self.w1,
                                                 dg.Sm100Out.Bf16(h, c["gate_up_n"]), self.local_e)
        # silu(gate) * up, quantised for the down projection without the bf16 activation touching memory
        actq, actsf = dg.silu_mul_cast_fp8_sf_dev(ctx, h, c["gate_up_n"], plan.m_pad, c["down_k"], 128)
        y = torch.empty((plan.m_pad, c["down_n"]), dtype=torch.bfloat16, device=self.dev)
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(actq, actsf, plan.m_pad, c["down_k"], c["down_k"]), plan.m_indices,
                                                 self.w2, dg.Sm100Out.Bf16(y, c["down_n"]), self.local_e)
        out = self.ep.combine(plan, y, topw)
        self.rows, self.plan = plan.n_recv, plan
        return out

    def experts_compute(self, pe, a_op, ends):
        """gate/up grouped GEMM, silu(gate) * up quantised for the down projection (the bf16 activation never touches memory),
        down grouped GEMM into the buffer the combine reads."""
        dg, c, ctx = self.dg, self.c, self.ctx
        h, act = self.bufs[id(pe)]
        if self.fused_act:
            # the weights are [gate rows; up rows] per expert: the epilogue writes e4m3(silu(gate) * up) and its scales
            dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, self.w1, dg.Sm100Out.SwiGluFp8(act[0], c["down_k"], act[1]), self.local_e)
        else:
            dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, self.w1, dg.Sm100Out.Bf16(h, c["gate_up_n"]), self.local_e)
            dg.silu_mul_cast_fp8_sf_dev(ctx, h, c["gate_up_n"], pe.capacity, c["down_k"], 128, live_rows=pe.totals, out=act)
        dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, dg.LpOperand(act[0], act[1], pe.capacity, c["down_k"], c["down_k"], 8, self.act_gran),
                                                      ends, self.w2, dg.Sm100Out.Bf16(pe.result, c["down_n"]), self.local_e)

    def routed_rows(self):
        """Valid arena rows of this rank in the last step (a host read, outside any timed region)."""
        if self.pipe is not None:
            return self.pipe.routed_rows()
        return int(self.peer.totals[1].item()) if self.peer is not None else self.rows

    def e2e_setup(self):
        torch = self.torch
        self.host = [t.cpu().pin_memory() for t in (self.xq, self.xsf, self.topi, self.topw)]
        self.hout = torch.empty((self.tokens, self.c["down_n"]), dtype=torch.bfloat16).pin_memory()
        self.staged = [torch.empty_like(t) for t in (self.xq, self.xsf, self.topi, self.topw)]
        return sum(z.numel() * z.element_size() for z in self.host), self.hout.numel() * self.hout.element_size()

    def e2e_step(self, pipes):
        torch = self.torch
        main = torch.cuda.current_stream()
        ev = self.e2e_events = getattr(self, "e2e_events", None) or {k: torch.cuda.Event() for k in ("landed", "done", "left")}
        with torch.cuda.stream(pipes.up):
            if getattr(self, "e2e_ran", False):
                pipes.up.wait_event(ev["done"])          # the previous step has read the staged inputs
            for d, h in zip(self.staged, self.host):
                d.copy_(h, non_blocking=True)
            ev["landed"].record(pipes.up)
        main.wait_event(ev["landed"])
        out = self.step(*self.staged)
        ev["done"].record(main)
        with torch.cuda.stream(pipes.down):
            pipes.down.wait_event(ev["done"])
            self.hout.copy_(out, non_blocking=True)
            out.record_stream(pipes.down)
            ev["left"].record(pipes.down)
        self.e2e_ran = True

    def gate_up_alone(self):
        """The gate/up grouped GEMM on this rank's arena, CUDA events around the launch; returns (ms, rows)."""
        torch, dg, c = self.torch, self.dg, self.c
        if self.peer is not None:
            pe = self.peer
            if self.pipe is not None:
                # one micro-batch on its own (all ranks take this branch together); rows reported are that micro-batch's
                torch.cuda.synchronize()
                t1 = self.pipe.chunk_tokens
                with torch.cuda.stream(self.pipe.side):
                    a_op, ends = pe.dispatch(self.topi[:t1], self.xq[:t1], self.xsf, dg.sf_aligned_rows(self.tokens))
                self.pipe.side.synchronize()
            else:
                a_op, ends = pe.dispatch(self.topi, self.xq, self.xsf)
            times = []
            for _ in range(6):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = dg.Sm100Out.SwiGluFp8(self.act[0], c["down_k"], self.act[1]) if self.fused_act else dg.Sm100Out.Bf16(self.h, c["gate_up_n"])
                dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(self.ctx, a_op, ends, self.w1, out, self.local_e)
                e1.record()
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            if self.pipe is not None:
                with torch.cuda.stream(self.pipe.side):
                    pe.combine(self.topw[:self.pipe.chunk_tokens])
                self.pipe.side.synchronize()
                return statistics.median(times[1:]), int(pe.totals[1].item())
            pe.combine(self.topw)        # keeps the ranks' dispatch / combine fences paired
            return statistics.median(times[1:]), self.routed_rows()
        plan = self.ep.plan(self.topi)
        a, a_sf = self.ep.dispatch(plan, self.xq, self.xsf, c["hidden"])
        h = torch.empty((plan.m_pad, c["gate_up_n"]), dtype=torch.bfloat16, device=self.dev)
        a_op = dg.LpOperand(a, a_sf, plan.m_pad, c["hidden"], c["hidden"])
        times = []
        for _ in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dg.m_grouped_fp8_fp4_gemm_contiguous_dev(self.ctx, a_op, plan.m_indices, self.w1, dg.Sm100Out.Bf16(h, c["gate_up_n"]), self.local_e)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        return statistics.median(times[1:]), plan.n_recv



def run_config_table(args, torch, dg, ctx, dev, peaks):
    """`--workload configs`: every benchmark configuration on one GPU, each launch alone behind an L2 flush, against the
    bound its algorithmic bytes and flops give (slower of tensor peak and HBM).  A report, not the bench line: prints one
    JSON object {"rows": [...]}.  Tensor peaks: 2 x (FP8) or 4 x (FP4) the measured bf16 figure (burst: launches timed alone)."""
    hbm, tc8, tc4 = peaks["hbm_gbs"] * 1e9, 2e12 * peaks["bf16_tflops"], 4e12 * peaks["bf16_tflops"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    gen = torch.Generator(device=dev).manual_seed(1234)
    rows = []

    def timeit(fn, reps=6):
        times = []
        for _ in range(reps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1e-3)
        return statistics.median(times[1:])

    def add(name, t, flops, nbytes, tc):
        t_tc, t_hbm = (flops / tc if flops else 0.0), nbytes / hbm
        bound = "tensor" if t_tc >= t_hbm else "hbm"
        row = {"config": name, "us": round(t * 1e6, 1), "bound": bound, "roofline_us": round(max(t_tc, t_hbm) * 1e6, 1),
               "frac": round(max(t_tc, t_hbm) / t, 3), "gbs": round(nbytes / t / 1e9, 1)}
        if flops:
            row["tflops"] = round(flops / t / 1e12, 1)
        rows.append(row)
        print(json.dumps(row), file=sys.stderr, flush=True)

    def randn(r, c):
        return torch.randn((r, c), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)

    def sf_bytes(k, gran, r):
        return 4 * ((k + 4 * gran - 1) // (4 * gran)) * r

    # config 2: dense FP8
    for (m, n, k) in DENSE_SHAPES:
        aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn(m, k), k, m, k, 128)
        bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn(n, k), k, n, k, 128)
        d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        a, b, out = dg.LpOperand(aq, asf, m, k, k), dg.LpOperand(bq, bsf, n, k, k), dg.Sm100Out.Bf16(d, n)
        t = timeit(lambda: dg.fp8_fp4_gemm_dev(ctx, a, b, out))
        add(f"dense fp8 {m}x{n}x{k}", t, 2.0 * m * n * k, m * k + n * k + 2 * m * n + sf_bytes(k, 128, m + n), tc8)
    # config 3: MXFP4 and FP8 x FP4
    m, n, k = 4096, 7168, 7168
    x, w = randn(m, k), randn(n, k)
    a4q, a4sf = dg.cast_bf16_to_fp4_packed_sf_dev(ctx, x, k, m, k, 1, dg.SF_RULE_RANGE_FIT)
    b4q, b4sf = dg.cast_bf16_to_fp4_packed_sf_dev(ctx, w, k, n, k, 1, dg.SF_RULE_RANGE_FIT)
    a8q, a8sf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, k, m, k, 32)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    out = dg.Sm100Out.Bf16(d, n)
    a4, b4 = dg.LpOperand(a4q, a4sf, m, k, k, 4, 32), dg.LpOperand(b4q, b4sf, n, k, k, 4, 32)
    a8 = dg.LpOperand(a8q, a8sf, m, k, k, 8, 32)
    t = timeit(lambda: dg.fp8_fp4_gemm_dev(ctx, a4, b4, out))
    add(f"mxfp4 {m}x{n}x{k}", t, 2.0 * m * n * k, (m + n) * k // 2 + 2 * m * n + sf_bytes(k, 32, m + n), tc4)
    t = timeit(lambda: dg.fp8_fp4_gemm_dev(ctx, a8, b4, out))
    add(f"fp8 x fp4 {m}x{n}x{k}", t, 2.0 * m * n * k, m * k + n * k // 2 + 2 * m * n + sf_bytes(k, 32, m + n), tc8)
    t = timeit(lambda: dg.bf16_gemm_dev(ctx, x, k, m, w, k, n, k, out))
    add(f"bf16 {m}x{n}x{k}", t, 2.0 * m * n * k, 2 * (m + n) * k + 2 * m * n, 1e12 * peaks["bf16_tflops"])
    del x, w, a4q, b4q, a8q, d
    # quantisers
    for (r, c) in [(4096, 7168), (7168, 16384)]:
        src = randn(r, c)
        t = timeit(lambda: dg.cast_bf16_to_fp8_sf_dev(ctx, src, c, r, c, 128))
        add(f"quantise bf16->e4m3 {r}x{c} gran 128", t, 0.0, 3 * r * c + sf_bytes(c, 128, r), tc8)
        t = timeit(lambda: dg.cast_bf16_to_fp4_packed_sf_dev(ctx, src, c, r, c, 1, dg.SF_RULE_RANGE_FIT))
        add(f"quantise bf16->e2m1 {r}x{c}", t, 0.0, 2.5 * r * c + sf_bytes(c, 32, r), tc8)
    del src
    # config 5: masked decode GEMM, FP8 output
    g, m_max, n, k = 32, 256, 4096, 7168
    masked = torch.randint(0, m_max + 1, (g,), generator=torch.Generator().manual_seed(4000), dtype=torch.int32)
    valid = int(masked.sum())
    aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn(g * m_max, k), k, g * m_max, k, 128, g)
    bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn(g * n, k), k, g * n, k, 128, g)
    d8 = torch.empty((g * m_max, n), dtype=torch.uint8, device=dev)
    sfd = torch.zeros(g * (n // 128) * m_max, dtype=torch.int32, device=dev)
    a, b, mm = dg.LpOperand(aq, asf, m_max, k, k), dg.LpOperand(bq, bsf, g * n, k, k), masked.to(dev)
    t = timeit(lambda: dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a, mm, b, dg.Sm100Out.Fp8(d8, n, sfd), g, valid // g))
    add(f"masked fp8-out {g} experts x <= {m_max} rows ({valid} valid), N={n} K={k}", t, 2.0 * valid * n * k,
        valid * k + g * n * k + valid * n * (1 + 1 / 32) + sf_bytes(k, 128, valid + g * n), tc8)
    del aq, bq, d8
    # config 4: the two contiguous grouped GEMMs and the row movers around them, one rank of a 1-GPU and of an 8-GPU job
    for experts in (MOE["experts"], MOE["experts"] // 8):
        saved = dict(MOE)
        MOE["experts"] = experts
        moe = MoeWork(torch, None, dg, ctx, dev, 0, 1, "peer")
        MOE.update(saved)
        pe, c = moe.peer, moe.c
        a_op, ends = pe.dispatch(moe.topi, moe.xq, moe.xsf)
        rows_valid = moe.routed_rows()
        h_out, y_out = dg.Sm100Out.Bf16(moe.h, c["gate_up_n"]), dg.Sm100Out.Bf16(pe.result, c["down_n"])
        act_op = dg.LpOperand(moe.act[0], moe.act[1], pe.capacity, c["down_k"], c["down_k"])
        tag = f"{experts} local experts, {rows_valid} rows"
        t = timeit(lambda: dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, moe.w1, h_out, experts))
        n, k = c["gate_up_n"], c["hidden"]
        add(f"grouped gate/up ({tag})", t, 2.0 * rows_valid * n * k, rows_valid * k + experts * n * k + 2 * rows_valid * n + sf_bytes(k, 128, rows_valid + experts * n), tc8)
        t = timeit(lambda: dg.silu_mul_cast_fp8_sf_dev(ctx, moe.h, c["gate_up_n"], pe.capacity, c["down_k"], 128, live_rows=pe.totals, out=moe.act))
        add(f"silu*up + quantise ({tag})", t, 0.0, rows_valid * c["down_k"] * 5, tc8)
        act32 = (moe.act[0], dg.alloc_sf(ctx, pe.capacity, c["down_k"], 32))
        t = timeit(lambda: dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, moe.w1, dg.Sm100Out.SwiGluFp8(act32[0], c["down_k"], act32[1]), experts))
        add(f"grouped gate/up with silu*up + quantise in its epilogue ({tag})", t, 2.0 * rows_valid * n * k,
            rows_valid * k + experts * n * k + rows_valid * c["down_k"] * (1 + 1 / 32) + sf_bytes(k, 128, rows_valid + experts * n), tc8)
        n, k = c["down_n"], c["down_k"]
        t = timeit(lambda: dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, act_op, ends, moe.w2, y_out, experts))
        add(f"grouped down ({tag})", t, 2.0 * rows_valid * n * k, rows_valid * k + experts * n * k + 2 * rows_valid * n + sf_bytes(k, 128, rows_valid + experts * n), tc8)
        t = timeit(lambda: pe.dispatch(moe.topi, moe.xq, moe.xsf))
        add(f"route + dispatch, local ({tag})", t, 0.0, moe.tokens * c["hidden"] + rows_valid * c["hidden"], tc8)
        t = timeit(lambda: pe.combine(moe.topw))
        add(f"combine, local ({tag})", t, 0.0, 2 * rows_valid * c["down_n"] + 2 * moe.tokens * c["down_n"], tc8)
        pe.close()
        del moe, pe, a_op, act_op, h_out, y_out
        torch.cuda.empty_cache()
    print(json.dumps({"rows": rows, "peaks": peaks, "note": "each launch alone, L2 flushed before it; frac = roofline time / measured time"}))

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="dgb200")
    ap.add_argument("--workload", default="dsv3", choices=["dsv3", "dense_fp8", "moe_ep", "configs"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--moe-experts", type=int, default=None, help="moe_ep: total experts (default 256); 32 gives one rank of an 8-GPU job")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="how MoE rows travel between ranks: peer-memory kernels of the library (default) or NCCL all-to-all")
    ap.add_argument("--moe-chunks", type=int, default=1,
                    help="token micro-batches of the MoE step whose exchange overlaps the other micro-batches' GEMMs (measured slower "
                         "than 1 on 2 and 4 GPUs: the GEMMs lose more to the exchange kernels sharing their SMs than the overlap returns)")
    ap.add_argument("--ep-blocks-per-sm", type=int, default=2, help="grid bound of the exchange kernels when they run beside the GEMMs")
    ap.add_argument("--fused-act", action="store_true",
                    help="MoE step: silu(gate)*up and its quantiser run in the gate/up GEMM's epilogue (output kind DG_OUT_SWIGLU_FP8) instead of "
                         "a kernel of their own; measured slower: the 192-wide tile it needs costs the GEMM more than the kernel it saves")
    ap.add_argument("--moe-tokens", type=int, default=None, help="moe_ep: tokens per rank (default 8192); smaller values for profiling captures")
    ap.add_argument("--only", default=None, help="M,N,K: run just this dense GEMM (profiling captures); implies --workload dense_fp8")
    args = ap.parse_args()
    if args.only:
        global DENSE_SHAPES, DOMINANT
        DOMINANT = tuple(int(x) for x in args.only.split(","))
        DENSE_SHAPES = [DOMINANT]
        args.workload = "dense_fp8"
    if args.moe_experts:
        MOE["experts"] = args.moe_experts
    if args.moe_tokens:
        MOE["tokens_per_rank"] = args.moe_tokens
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
    dev = torch.device("cuda", local_rank)
    ctx = dg.DgContext(local_rank)
    peaks = measured_peaks()

    if args.workload == "configs":
        if world > 1:
            raise SystemExit("--workload configs is a single-GPU report")
        run_config_table(args, torch, dg, ctx, dev, peaks)
        return

    # ---- build the workload (untimed): operands resident in HBM, quantised by the library's own kernels
    dense = DenseWork(torch, dg, ctx, dev, 1000 + rank) if args.workload in ("dsv3", "dense_fp8") else None
    chunks = max(1, args.moe_chunks)
    moe = MoeWork(torch, dist, dg, ctx, dev, rank, world, args.ep, chunks, args.ep_blocks_per_sm, args.fused_act) if args.workload in ("dsv3", "moe_ep") else None
    ctx.sync()

    def step(record=None):
        if dense is not None:
            dense.step(record)
        if moe is not None:
            moe.step()

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, finish=None):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fence()
        start.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        end.record()
        fence()
        return max_over_ranks(start.elapsed_time(end)) / steps

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    dominant_events = []
    n_before = len(sampler.samples)
    ms_per_step = timed(lambda: step(dominant_events), args.steps)
    n_timed = len(sampler.samples) - n_before
    # whole-job flops of one step: dense replicas + routed rows of all ranks
    moe_rows = 0.0
    if moe is not None:
        r = torch.tensor([float(moe.routed_rows())], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(r, op=dist.ReduceOp.SUM)
        moe_rows = float(r.item())
    flops = (dense.flops * world if dense is not None else 0.0) + (moe_rows * moe.flops_per_row if moe is not None else 0.0)
    value = flops / (ms_per_step * 1e-3) / 1e12

    # the timed region lasts milliseconds; keep the same step loop running for about a second so the clock record also
    # shows what the GPU settles at under this load (all ranks take part: the step contains collectives)
    soak_steps = max(1, int(1200.0 / max(ms_per_step, 0.05)))
    for _ in range(min(soak_steps, 2000)):
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "warm-up + timed region + about 1.2 s of the same step loop"
        clocks["samples_in_timed_region"] = n_timed

    # ---- each half on its own (same K steps), the dominant launches, per-GEMM times
    parts = {}
    if dense is not None:
        d_ms = timed(dense.step, args.steps) if moe is not None else ms_per_step
        parts["dense_fp8"] = {"tflops": dense.flops * world / (d_ms * 1e-3) / 1e12, "ms_per_step": d_ms, "parallelism": "replica per GPU"}
    if moe is not None:
        m_ms = timed(moe.step, args.steps) if dense is not None else ms_per_step
        gemm_ms, gemm_rows = moe.gate_up_alone()
        parts["moe_ep"] = {"tflops": moe_rows * moe.flops_per_row / (m_ms * 1e-3) / 1e12, "ms_per_step": m_ms, "routed_rows_all_ranks": moe_rows,
                           "gate_up_gemm_us_rank0": gemm_ms * 1e3,
                           "gate_up_gemm_tflops_rank0": 2.0 * gemm_rows * MOE["gate_up_n"] * MOE["hidden"] / (gemm_ms * 1e-3) / 1e12,
                           "parallelism": f"ep{world}: {moe.local_e} experts per GPU"}
    per_shape = dense.per_gemm() if (dense is not None and rank == 0 and world == 1) else None
    fence()

    # ---- end to end from pinned host buffers through the same public calls
    e2e = None
    if not args.no_e2e:
        h2d = d2h = 0
        for w in (dense, moe):
            if w is not None:
                a, b = w.e2e_setup()
                h2d, d2h = h2d + a, d2h + b

        class Pipes:
            up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def e2e_step():
            if dense is not None:
                dense.e2e_step(Pipes)
            if moe is not None:
                moe.e2e_step(Pipes)

        def e2e_drain():
            # the timed region ends when the last result has reached the host
            main = torch.cuda.current_stream()
            main.wait_stream(Pipes.down)
            main.wait_stream(Pipes.up)

        e2e_steps = max(3, min(args.steps, 10))
        e2e_step()
        e2e_ms = timed(e2e_step, e2e_steps, e2e_drain)
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_ms, "steps": e2e_steps,
               "what": "dense: A, B and scale words in, D out; MoE: this rank's e4m3 tokens, scales, routing in, reduced rows out; "
                       "uploads, compute and downloads on three streams, ordered per buffer by events"}
    ctx.sync()

    if rank == 0:
        if dense is not None:
            m, n, k = DOMINANT
            dom_ms = sum(a.elapsed_time(b) for a, b in dominant_events) / max(len(dominant_events), 1)
            achieved = 2 * m * n * k / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else None
            peak = 2 * peaks["bf16_tflops_sustained"]
            roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                        "frac": achieved / peak if achieved else None,
                        # dram__bytes_read.sum + dram__bytes_write.sum of this launch, one ncu capture
                        # (profiles/dg_gemm_kernel_fp8_M4096_N7168_K16384.md); algorithmic bytes are 2.447e8
                        "traffic": 5.37e8 if DOMINANT == (4096, 7168, 16384) else None,
                        "kernel": "dg_gemm_kernel<fp8, bf16 out, CTA pair>", "launch": f"dense M={m} N={n} K={k}",
                        "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} peaks (e4m3 issues at twice the bf16 rate)",
                        "frac_of_nominal_fp8_4500": achieved / 4500.0 if achieved else None}
        else:
            gemm_ms = parts["moe_ep"]["gate_up_gemm_us_rank0"] * 1e-3
            achieved = parts["moe_ep"]["gate_up_gemm_tflops_rank0"]
            peak = 2 * peaks["bf16_tflops_sustained"]
            roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                        "kernel": "dg_gemm_kernel<fp8, bf16 out> contiguous grouped, gate/up",
                        "launch": f"rank 0: routed rows over {moe.local_e} local experts, N={MOE['gate_up_n']} K={MOE['hidden']}, {gemm_ms * 1e3:.0f} us",
                        "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} peaks"}
        config = {"workload": {"dsv3": "dsv3_fp8_gemms (dense pass + expert-parallel MoE pair)", "dense_fp8": "dense_fp8_dsv3",
                               "moe_ep": "moe_contiguous_ep"}[args.workload],
                  "gran_k": 128, "out": "bf16", "parallelism": ("single GPU" if world == 1 else f"dense: replica per GPU; MoE: ep{world}"),
                  "l2": "a step touches 1.1 GB of dense operands and 1.4-11 GB of expert weights per GPU, far more than the 126 MB L2"}
        if dense is not None:
            config["dense_shapes"] = DENSE_SHAPES
        if moe is not None:
            config["moe"] = dict(MOE, experts_per_gpu=moe.local_e, mk_alignment=128,
                                 collective=moe.exchange_note)
        launches = (dense.launches if dense is not None else 0) + (moe.launches if moe is not None else 0)
        line = {"metric": "fp8_block_scaled_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp8_e4m3", "data": "synthetic", "config": config, "clocks": clocks, "gpu_launches": args.steps * launches,
                "roofline": roofline, "parts": parts}
        if per_shape is not None:
            line["per_gemm"] = per_shape
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as O
            threads = O.max_threads()
            cases = cpu_sample_inputs()
            sec = cpu_step(cases, threads)
            line["cpu_baseline"] = {"value": cpu_sample_flops(cases) / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{CPU_SAMPLE_TEXT}, one pass ({sec:.1f} s)"}
        print(json.dumps(line), flush=True)
    if moe is not None and moe.peer is not None:
        # unmap the peers' buffers and free this rank's, in step with the other ranks, before the process group goes away
        (moe.pipe or moe.peer).close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
