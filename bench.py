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


def host_threads():
    """Threads of the CPU legs: the cores this process may run on, whatever OMP_NUM_THREADS says (launchers set it to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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
    threads = host_threads()
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


def weights_by_expert_id(torch, dg, ctx, dev, seed_base, experts, n, k, gran):
    """e4m3 weights (len(experts) * n, k) and their packed per-`gran` scale words, one (n, k) block per listed expert.  An expert's
    matrix depends only on its id (seeded N(0,1) bf16), so any rank can rebuild any expert's weights; the parity checks do."""
    experts = list(experts)
    q = torch.empty((len(experts) * n, k), dtype=torch.uint8, device=dev)
    sf = dg.alloc_sf(ctx, len(experts) * n, k, gran, len(experts))
    cols, stride, chunk = dg.sf_packed_cols(k, gran), dg.sf_aligned_rows(n), 8
    gen = torch.Generator(device=dev)
    for g0 in range(0, len(experts), chunk):
        ids = experts[g0:g0 + chunk]
        w = torch.empty((len(ids) * n, k), dtype=torch.bfloat16, device=dev)
        for i, e in enumerate(ids):
            gen.manual_seed(seed_base + int(e))
            w[i * n:(i + 1) * n] = torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        wq, wsf = dg.cast_bf16_to_fp8_sf_dev(ctx, w, k, len(ids) * n, k, gran, len(ids))
        q[g0 * n:(g0 + len(ids)) * n] = wq
        sf.view(len(experts), cols, stride)[g0:g0 + len(ids)] = wsf.view(len(ids), cols, stride)
    return q, sf


class _Phase:
    def __init__(self, torch, record, name):
        self.torch, self.record, self.name = torch, record, name

    def __enter__(self):
        if self.record is not None:
            self.e0 = self.torch.cuda.Event(enable_timing=True)
            self.e0.record()

    def __exit__(self, *exc):
        if self.record is not None:
            e1 = self.torch.cuda.Event(enable_timing=True)
            e1.record()
            self.record.setdefault(self.name, []).append((self.e0, e1))
        return False


def phase_us(record):
    """Mean duration of every recorded phase in microseconds (events must have completed)."""
    return {k: 1e3 * sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in record.items() if v}


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

    def step(self, record=None, ctx=None, first=0, last=None):
        """Launch problems [first, last) of the pass on `ctx` (default: the context the operands were made on)."""
        for p in self.problems[first:last]:
            with _Phase(self.torch, record, "dense %dx%dx%d" % p["shape"]):
                self.dg.fp8_fp4_gemm_dev(ctx or self.ctx, p["a"], p["b"], p["out"])

    def e2e_setup(self):
        """Weights (B and its scale words) are parameters: they stay resident in HBM, as in any caller of a GEMM library.  A step
        uploads the activations (A and its scale words) of every GEMM and downloads every D."""
        torch = self.torch
        self.host = []
        for p in self.problems:
            h = {name: ten.cpu().pin_memory() for name, ten in (("a", p["a"].data), ("asf", p["a"].sf))}
            h["d"] = torch.empty(p["d"].shape, dtype=p["d"].dtype).pin_memory()
            self.host.append(h)
        h2d = sum(h[n].numel() * h[n].element_size() for h in self.host for n in ("a", "asf"))
        d2h = sum(h["d"].numel() * h["d"].element_size() for h in self.host)
        return h2d, d2h

    def e2e_step(self, pipes):
        """Activations in on the upload stream, GEMM on the compute stream, D out on the download stream: the copies of one
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

    def per_gemm(self, peaks):
        """Each launch alone with the L2 flushed by a 256 MB write before it (for the report), against its roofline."""
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
            out.append(dict({"m": m, "n": n, "k": k}, **launch_bound(2.0 * m * n * k, dense_bytes(m, n, k), t_ms * 1e-3, peaks, 2)))
        return out


class MoeWork:
    """Expert-parallel contiguous grouped GEMM pair (see the module docstring)."""

    def __init__(self, torch, dist, dg, ctx, dev, rank, world, exchange="peer", chunks=1, blocks_per_sm=2, fused_act=False):
        from deepgemm_rust_b200.moe_ep import DeviceRowOps, ExpertParallel, PeerExpertParallel, PipelinedPeerMoe
        self.torch, self.dg, self.ctx, self.dev, self.world = torch, dg, ctx, dev, world
        c = self.c = dict(MOE)
        self.local_e = local_e = c["experts"] // world
        gen = torch.Generator(device=dev).manual_seed(3000 + rank)
        self.rank, self.first_expert = rank, rank * local_e
        w1q, w1sf = self.expert_weights(range(self.first_expert, self.first_expert + local_e), 1)
        w2q, w2sf = self.expert_weights(range(self.first_expert, self.first_expert + local_e), 2)
        self.tokens = tokens = c["tokens_per_rank"]
        x = torch.randn((tokens, c["hidden"]), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        logits = torch.randn((tokens, c["experts"]), generator=gen, device=dev, dtype=torch.float32)
        topw, self.topi = torch.softmax(logits, -1).topk(c["topk"], dim=-1)
        self.topw = topw.contiguous()
        self.xq, self.xsf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, c["hidden"], tokens, c["hidden"], 128)
        del x
        # rows travel through peer memory (kernels of the library) unless the peers cannot be mapped; every rank must agree
        self.peer, self.pipe, self.chunks, self.exchange_note = None, None, max(1, chunks), "nccl all_to_all_single"
        self.before_combine = None
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

    def expert_weights(self, experts, layer):
        """Quantised weights of the given (global) experts for layer 1 (gate/up) or 2 (down), stacked in that order."""
        c = self.c
        n, k = (c["gate_up_n"], c["hidden"]) if layer == 1 else (c["down_n"], c["down_k"])
        return weights_by_expert_id(self.torch, self.dg, self.ctx, self.dev, 500000 * layer, experts, n, k, 128)

    def parity_check(self, out, sample_tokens=6):
        """Outside any timed region: recomputes the layer output of a few of this rank's tokens without any exchange -- their rows
        laid out locally, one group per (token, expert) pair, the weights of exactly those experts rebuilt here, the same grouped
        GEMMs, activation kernel and reduction -- and compares with what the expert-parallel step returned for those tokens,
        bit for bit.  A row that travelled to the wrong arena row, expert or rank, or came back to the wrong token, shows up."""
        torch, dg, c, ctx, dev = self.torch, self.dg, self.c, self.ctx, self.dev
        tok = torch.linspace(0, self.tokens - 1, sample_tokens, device=dev).long()
        topi, topw = self.topi[tok], self.topw[tok].contiguous()
        experts = topi.reshape(-1).tolist()                               # one group per pair, in (token, j) order
        groups, align = len(experts), dg.get_mk_alignment_for_contiguous_layout()
        rows = groups * align
        xq = torch.zeros((rows, c["hidden"]), dtype=torch.uint8, device=dev)
        xq[::align] = self.xq[tok].repeat_interleave(c["topk"], 0)
        cols = dg.sf_packed_cols(c["hidden"], 128)
        xsf = torch.zeros((cols, dg.sf_aligned_rows(rows)), dtype=torch.int32, device=dev)
        xsf[:, :rows:align] = self.xsf.view(cols, -1)[:, tok].repeat_interleave(c["topk"], 1)
        m_idx = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        m_idx[::align] = torch.arange(groups, dtype=torch.int32, device=dev)
        w1q, w1sf = self.expert_weights(experts, 1)
        w2q, w2sf = self.expert_weights(experts, 2)
        a_op, w1 = dg.LpOperand(xq, xsf, rows, c["hidden"], c["hidden"]), dg.LpOperand(w1q, w1sf, groups * c["gate_up_n"], c["hidden"], c["hidden"])
        if self.fused_act:
            actq = torch.empty((rows, c["down_k"]), dtype=torch.uint8, device=dev)
            actsf = dg.alloc_sf(ctx, rows, c["down_k"], 32)
            dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a_op, m_idx, w1, dg.Sm100Out.SwiGluFp8(actq, c["down_k"], actsf), groups)
        else:
            h = torch.empty((rows, c["gate_up_n"]), dtype=torch.bfloat16, device=dev)
            dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a_op, m_idx, w1, dg.Sm100Out.Bf16(h, c["gate_up_n"]), groups)
            actq, actsf = dg.silu_mul_cast_fp8_sf_dev(ctx, h, c["gate_up_n"], rows, c["down_k"], 128)
        y = torch.empty((rows, c["down_n"]), dtype=torch.bfloat16, device=dev)
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(actq, actsf, rows, c["down_k"], c["down_k"], 8, self.act_gran), m_idx,
                                                 dg.LpOperand(w2q, w2sf, groups * c["down_n"], c["down_k"], c["down_k"]),
                                                 dg.Sm100Out.Bf16(y, c["down_n"]), groups)
        pos = (torch.arange(groups, dtype=torch.int32, device=dev) * align).view(sample_tokens, c["topk"]).contiguous()
        want = dg.moe_combine_dev(ctx, y, pos, topw)
        ctx.sync()
        return bool(torch.equal(want.view(torch.int16), out[tok].view(torch.int16))), sample_tokens

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
            with self.phase("dispatch"):
                a_op, ends = pe.dispatch(topi, xq, xsf)
            self.experts_compute(pe, a_op, ends)
            if self.before_combine is not None:
                self.before_combine()          # the dense GEMMs that run beside the combine are released here
            with self.phase("combine"):
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
            with self.phase("gate_up"):
                dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, self.w1, dg.Sm100Out.SwiGluFp8(act[0], c["down_k"], act[1]), self.local_e)
        else:
            with self.phase("gate_up"):
                dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, self.w1, dg.Sm100Out.Bf16(h, c["gate_up_n"]), self.local_e)
            with self.phase("silu_mul_quant"):
                dg.silu_mul_cast_fp8_sf_dev(ctx, h, c["gate_up_n"], pe.capacity, c["down_k"], 128, live_rows=pe.totals, out=act)
        with self.phase("down"):
            dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, dg.LpOperand(act[0], act[1], pe.capacity, c["down_k"], c["down_k"], 8, self.act_gran),
                                                          ends, self.w2, dg.Sm100Out.Bf16(pe.result, c["down_n"]), self.local_e)

    def phase(self, name):
        """Context manager: CUDA events around a phase of the step while `self.record` is a dict (timed steps), nothing otherwise."""
        return _Phase(self.torch, getattr(self, "record", None), name)

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
    # the older f32-scale API on the same shape: exact per-K-block scaling (scales with mantissas) and the exponent-only route
    a8u, b8u = (torch.randint(0, 120, (r, k), dtype=torch.uint8, device=dev) for r in (m, n))
    sfa32 = torch.rand((m, k // 128), device=dev) + 0.5
    sfb32 = torch.rand((n // 128, k // 128), device=dev) + 0.5
    a_sf_t = dg.transform_sf_dev(ctx, sfa32, m, k // 128, 1)
    nt = lambda: dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(a8u, m, k, k), a_sf_t, dg.Fp8Tensor(b8u, n, k, k), sfb32, d, n)
    saved = os.environ.pop("DG_F32_SCALES", None)
    t = timeit(nt)
    add(f"fp8 {m}x{n}x{k}, f32 scales applied exactly per K block", t, 2.0 * m * n * k, (m + n) * k + 2 * m * n + 4 * (m + n // 128) * (k // 128), tc8)
    os.environ["DG_F32_SCALES"] = "exponent"
    t = timeit(nt)
    add(f"fp8 {m}x{n}x{k}, f32 scales reduced to their exponents", t, 2.0 * m * n * k, (m + n) * k + 2 * m * n + 4 * (m + n // 128) * (k // 128), tc8)
    if saved is None:
        os.environ.pop("DG_F32_SCALES", None)
    else:
        os.environ["DG_F32_SCALES"] = saved
    del x, w, a4q, b4q, a8q, d, a8u, b8u
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

MASKED = {"local_experts": 32, "slot_rows": 256, "topk": 8, "hidden": 7168, "n": 4096, "next_n": 7168}


def launch_bound(flops, nbytes, seconds, peaks, tensor_mult):
    """Roofline of one launch: the slower of tensor time (tensor_mult x the measured bf16 rate: 2 for e4m3, 4 for e2m1) and HBM time
    for its algorithmic flops and bytes.  Fractions against the burst and the sustained tensor figure, and the nominal part figures."""
    hbm = peaks["hbm_gbs"] * 1e9
    t_hbm = nbytes / hbm
    t_tc = flops / (tensor_mult * 1e12 * peaks["bf16_tflops"]) if flops else 0.0
    row = {"us": round(seconds * 1e6, 2), "gbs": round(nbytes / seconds / 1e9, 1)}
    if flops:
        row["tflops"] = round(flops / seconds / 1e12, 1)
    if t_tc >= t_hbm:
        row.update(bound="tensor", frac_burst=round(t_tc / seconds, 3),
                   frac_sustained=round(flops / (tensor_mult * 1e12 * peaks["bf16_tflops_sustained"]) / seconds, 3),
                   frac_nominal=round(flops / (tensor_mult * 2.25e15) / seconds, 3))
    else:
        row.update(bound="hbm", frac=round(t_hbm / seconds, 3), frac_nominal=round(nbytes / 8e12 / seconds, 3))
    return row


def dense_bytes(m, n, k):
    return m * k + n * k + 2 * m * n + 4 * ((k + 511) // 512) * (m + n)


def time_alone(torch, fn, flush, reps=6):
    """One launch at a time behind an L2 flush (a 256 MB write); median of the runs after the first, in seconds."""
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


def dequant_rows(torch, q, sf, idx, k, gran, total_rows):
    """Plain torch f64 values of rows `idx` of an e4m3 operand with packed UE8M0 scale words (cols, align4(total_rows))."""
    vals = q[idx].view(torch.float8_e4m3fn).to(torch.float64)
    stride = (total_rows + 3) // 4 * 4
    words = sf.view(-1, stride)[:, idx].to(torch.int64) & 0xFFFFFFFF            # (cols, rows)
    kb = torch.arange(k // gran, device=q.device)
    exps = (words[kb // 4] >> (8 * (kb % 4)).unsqueeze(1)) & 0xFF                # (k / gran, rows)
    scale = torch.pow(2.0, (exps - 127).to(torch.float64)).t()
    return vals * scale.repeat_interleave(gran, dim=1)


def dense_parity(torch, problem, samples=48):
    """calc_diff of sampled rows x columns of a dense GEMM's bf16 output against a plain torch f64 product of the dequantised operands."""
    m, n, k = problem["shape"]
    dev = problem["d"].device
    g = torch.Generator(device=dev).manual_seed(11)
    rows = torch.unique(torch.cat([torch.randint(0, m, (samples,), generator=g, device=dev), torch.tensor([0, m - 1], device=dev)]))
    cols = torch.unique(torch.cat([torch.randint(0, n, (2 * samples,), generator=g, device=dev), torch.tensor([0, n - 1], device=dev)]))
    want = dequant_rows(torch, problem["a"].data, problem["a"].sf, rows, k, 128, m) @ dequant_rows(torch, problem["b"].data, problem["b"].sf, cols, k, 128, n).t()
    got = problem["d"][rows][:, cols].to(torch.float64)
    return float(1.0 - 2.0 * (got * want).sum() / ((got * got).sum() + (want * want).sum()))


class SingleLaunches:
    """The configurations that are one launch each and do not shard: MXFP4 and FP8 x FP4 4096x7168x7168, and the masked decode
    GEMM (32 experts, up to 256 rows each drawn uniformly, N=4096, K=7168, e4m3 output with per-32 scales), each timed alone."""

    def __init__(self, torch, dg, ctx, dev, peaks):
        self.torch, self.dg, self.ctx, self.dev, self.peaks = torch, dg, ctx, dev, peaks

    def run(self):
        torch, dg, ctx, dev, peaks = self.torch, self.dg, self.ctx, self.dev, self.peaks
        gen = torch.Generator(device=dev).manual_seed(1234)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        out = {}

        def randn(r, c):
            return torch.randn((r, c), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)

        def sf_bytes(k, gran, r):
            return 4 * ((k + 4 * gran - 1) // (4 * gran)) * r

        m, n, k = 4096, 7168, 7168
        x, w = randn(m, k), randn(n, k)
        a4q, a4sf = dg.cast_bf16_to_fp4_packed_sf_dev(ctx, x, k, m, k, 1, dg.SF_RULE_RANGE_FIT)
        b4q, b4sf = dg.cast_bf16_to_fp4_packed_sf_dev(ctx, w, k, n, k, 1, dg.SF_RULE_RANGE_FIT)
        a8q, a8sf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, k, m, k, 32)
        d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        o = dg.Sm100Out.Bf16(d, n)
        a4, b4 = dg.LpOperand(a4q, a4sf, m, k, k, 4, 32), dg.LpOperand(b4q, b4sf, n, k, k, 4, 32)
        a8 = dg.LpOperand(a8q, a8sf, m, k, k, 8, 32)
        t = time_alone(torch, lambda: dg.fp8_fp4_gemm_dev(ctx, a4, b4, o), flush)
        out["mxfp4 4096x7168x7168"] = launch_bound(2.0 * m * n * k, (m + n) * k // 2 + 2 * m * n + sf_bytes(k, 32, m + n), t, peaks, 4)
        t = time_alone(torch, lambda: dg.fp8_fp4_gemm_dev(ctx, a8, b4, o), flush)
        out["fp8 x fp4 4096x7168x7168"] = launch_bound(2.0 * m * n * k, m * k + n * k // 2 + 2 * m * n + sf_bytes(k, 32, m + n), t, peaks, 2)
        del x, w, a4q, b4q, a8q, d
        g, m_max, n, k = MASKED["local_experts"], MASKED["slot_rows"], MASKED["n"], MASKED["hidden"]
        masked = torch.randint(0, m_max + 1, (g,), generator=torch.Generator().manual_seed(4000), dtype=torch.int32)
        valid = int(masked.sum())
        aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn(g * m_max, k), k, g * m_max, k, 128, g)
        bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn(g * n, k), k, g * n, k, 128, g)
        d8 = torch.empty((g * m_max, n), dtype=torch.uint8, device=dev)
        sfd = torch.zeros(g * (n // 128) * m_max, dtype=torch.int32, device=dev)
        a, b, mm = dg.LpOperand(aq, asf, m_max, k, k), dg.LpOperand(bq, bsf, g * n, k, k), masked.to(dev)
        t = time_alone(torch, lambda: dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a, mm, b, dg.Sm100Out.Fp8(d8, n, sfd), g, max(1, valid // g)), flush)
        row = launch_bound(2.0 * valid * n * k, valid * k + g * n * k + valid * n * (1 + 1 / 32) + sf_bytes(k, 128, valid + g * n), t, peaks, 2)
        row["valid_rows"] = valid
        out["masked fp8-out 32 experts x <=256 rows, N=4096 K=7168"] = row
        self.launches = 6 * 3
        return out


class MaskedEpWork:
    """The masked decode configuration sharded by expert: 32 experts per GPU (32 x N in all), every expert receiving a row count
    drawn uniformly from [0, 256] (seed 4000) split evenly over the source ranks.  One step = route + dispatch into the
    (32, 256, K) slots of the owners (peer memory), the masked grouped GEMM N=4096, K=7168 with e4m3 output and per-32 scales,
    a second masked GEMM (N=7168, K=4096) that consumes that output and its scales as its operand and leaves bf16 rows, and the
    weighted combine back on the token ranks.  Flops count the valid rows of both GEMMs."""

    def __init__(self, torch, dist, dg, ctx, dev, rank, world):
        from deepgemm_rust_b200.moe_ep import PeerExpertParallel
        self.torch, self.dg, self.ctx, self.dev, self.world, self.rank = torch, dg, ctx, dev, world, rank
        c = self.c = dict(MASKED)
        local, slot, topk = c["local_experts"], c["slot_rows"], c["topk"]
        experts = local * world
        per_expert = torch.randint(0, slot + 1, (experts,), generator=torch.Generator().manual_seed(4000), dtype=torch.int64)
        mine = per_expert // world + (rank < per_expert % world).to(torch.int64)          # this rank's rows for every expert
        pairs = torch.repeat_interleave(torch.arange(experts), mine)
        self.tokens = tokens = max((pairs.numel() + topk - 1) // topk, slot + 1)
        # pair i goes to token i % tokens: an expert's pairs are consecutive and at most `slot` < tokens, so no token gets an expert twice
        topi = torch.full((topk, tokens), -1, dtype=torch.int64)
        topi.view(-1)[:pairs.numel()] = pairs
        self.topi = topi.t().contiguous().to(dev)
        gen = torch.Generator(device=dev).manual_seed(4100 + rank)
        self.topw = torch.softmax(torch.randn((tokens, topk), generator=gen, device=dev), -1).contiguous()
        x = torch.randn((tokens, c["hidden"]), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.xq, self.xsf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, c["hidden"], tokens, c["hidden"], 128)
        del x
        mine_ids = range(rank * local, (rank + 1) * local)
        w1q, w1sf = weights_by_expert_id(torch, dg, ctx, dev, 1500000, mine_ids, c["n"], c["hidden"], 128)
        w2q, w2sf = weights_by_expert_id(torch, dg, ctx, dev, 2500000, mine_ids, c["next_n"], c["n"], 32)
        self.w1 = dg.LpOperand(w1q, w1sf, local * c["n"], c["hidden"], c["hidden"])
        self.w2 = dg.LpOperand(w2q, w2sf, local * c["next_n"], c["n"], c["n"], 8, 32)
        self.pe = PeerExpertParallel(ctx, experts, topk, tokens, c["hidden"], c["next_n"], slot_rows=slot)
        self.d8 = torch.empty((local * slot, c["n"]), dtype=torch.uint8, device=dev)
        self.sfd = torch.zeros(local * (c["n"] // 128) * slot, dtype=torch.int32, device=dev)
        self.valid_local = int(per_expert[rank * local:(rank + 1) * local].sum())
        self.valid_all = int(per_expert.sum())
        self.expected_m = max(1, self.valid_local // local)
        self.flops_per_row = 2.0 * (c["n"] * c["hidden"] + c["next_n"] * c["n"])
        self.launches = 7            # pair ranking, chunk scan, layout, dispatch, 2 GEMMs, combine
        self.record = None

    def phase(self, name):
        return _Phase(self.torch, self.record, name)

    def step(self):
        dg, c, ctx, pe = self.dg, self.c, self.ctx, self.pe
        local, slot = c["local_experts"], c["slot_rows"]
        with self.phase("dispatch"):
            a_op, masked_m = pe.dispatch(self.topi, self.xq, self.xsf)
        with self.phase("masked_gemm_fp8_out"):
            dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a_op, masked_m, self.w1, dg.Sm100Out.Fp8(self.d8, c["n"], self.sfd), local, self.expected_m)
        with self.phase("masked_gemm_next"):
            dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, dg.LpOperand(self.d8, self.sfd, slot, c["n"], c["n"], 8, 32), masked_m, self.w2,
                                                 dg.Sm100Out.Bf16(pe.result, c["next_n"]), local, self.expected_m)
        with self.phase("combine"):
            return pe.combine(self.topw)

    def parity_check(self, out, sample_tokens=6):
        """Outside any timed region: a few of this rank's tokens recomputed without the exchange -- one local slot per (token,
        expert) pair holding that token's row, the weights of exactly those experts rebuilt from their ids, the same two masked
        GEMMs and the same reduction -- compared bit for bit with what the expert-parallel step returned for those tokens."""
        torch, dg, c, ctx, dev = self.torch, self.dg, self.c, self.ctx, self.dev
        tok = torch.linspace(0, self.tokens - 1, sample_tokens, device=dev).long()
        topi, topw = self.topi[tok], self.topw[tok].contiguous()
        flat = topi.reshape(-1)
        live = (flat >= 0).nonzero().flatten()
        experts = flat[live].tolist()
        groups, slot = len(experts), 16
        xq = torch.zeros((groups * slot, c["hidden"]), dtype=torch.uint8, device=dev)
        xq[::slot] = self.xq[tok].repeat_interleave(c["topk"], 0)[live]
        cols = dg.sf_packed_cols(c["hidden"], 128)
        xsf = torch.zeros((groups, cols, dg.sf_aligned_rows(slot)), dtype=torch.int32, device=dev)
        xsf[:, :, 0] = self.xsf.view(cols, -1)[:, tok].repeat_interleave(c["topk"], 1)[:, live].t()
        masked_m = torch.ones(groups, dtype=torch.int32, device=dev)
        w1q, w1sf = weights_by_expert_id(torch, dg, ctx, dev, 1500000, experts, c["n"], c["hidden"], 128)
        w2q, w2sf = weights_by_expert_id(torch, dg, ctx, dev, 2500000, experts, c["next_n"], c["n"], 32)
        d8 = torch.empty((groups * slot, c["n"]), dtype=torch.uint8, device=dev)
        sfd = torch.zeros(groups * (c["n"] // 128) * dg.sf_aligned_rows(slot), dtype=torch.int32, device=dev)
        dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, dg.LpOperand(xq, xsf, slot, c["hidden"], c["hidden"]), masked_m,
                                             dg.LpOperand(w1q, w1sf, groups * c["n"], c["hidden"], c["hidden"]),
                                             dg.Sm100Out.Fp8(d8, c["n"], sfd), groups, 1)
        y = torch.empty((groups * slot, c["next_n"]), dtype=torch.bfloat16, device=dev)
        dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, dg.LpOperand(d8, sfd, slot, c["n"], c["n"], 8, 32), masked_m,
                                             dg.LpOperand(w2q, w2sf, groups * c["next_n"], c["n"], c["n"], 8, 32),
                                             dg.Sm100Out.Bf16(y, c["next_n"]), groups, 1)
        pos = torch.full((sample_tokens * c["topk"],), -1, dtype=torch.int32, device=dev)
        pos[live] = torch.arange(groups, dtype=torch.int32, device=dev) * slot
        want = dg.moe_combine_dev(ctx, y, pos.view(sample_tokens, c["topk"]).contiguous(), topw)
        ctx.sync()
        return bool(torch.equal(want.view(torch.int16), out[tok].view(torch.int16))) and not self.pe.overflowed(), sample_tokens

    def close(self):
        self.pe.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="dgb200")
    ap.add_argument("--workload", default="dsv3", choices=["dsv3", "dense_fp8", "moe_ep", "moe_masked_ep", "configs"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the parts timed outside the step (single launches, masked decode step, parity)")
    ap.add_argument("--moe-experts", type=int, default=None, help="moe_ep: total experts (default 256); 32 gives one rank of an 8-GPU job")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="how MoE rows travel between ranks: peer-memory kernels of the library (default) or NCCL all-to-all")
    ap.add_argument("--moe-chunks", type=int, default=1,
                    help="token micro-batches of the MoE step whose exchange overlaps the other micro-batches' GEMMs (measured slower "
                         "than 1 on 2 and 4 GPUs: the GEMMs lose more to the exchange kernels sharing their SMs than the overlap returns)")
    ap.add_argument("--overlap-dense", type=int, default=1,
                    help="default step: 1 (default) runs the dense GEMMs on a second stream beside the MoE layer's exchange kernels "
                         "(measured +3 % at 1 and 2 GPUs), 0 runs the dense pass first and the MoE layer after it")
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
    masked = MaskedEpWork(torch, dist, dg, ctx, dev, rank, world) if args.workload == "moe_masked_ep" else None
    ctx.sync()
    record = {}

    # --overlap-dense: the dense pass has no data in common with the MoE layer, so its GEMMs run on a second stream beside
    # the layer's exchange kernels, which leave the tensor cores idle: the M = 128 GEMMs and the largest M = 4096 one beside
    # route + dispatch, the other four beside the combine.  GEMM kernels of the two streams never share an SM (each needs
    # most of its shared memory), so they simply take turns; the exchange kernels (two 256-thread blocks per SM) do.
    overlap = bool(args.overlap_dense and dense is not None and moe is not None and moe.peer is not None and moe.pipe is None)
    side = side_ctx = None
    if overlap:
        side = torch.cuda.Stream(device=dev)
        side_ctx = dg.DgContext(local_rank, stream=side.cuda_stream)
        order = sorted(range(len(dense.problems)), key=lambda i: (dense.problems[i]["shape"][0] != 128, dense.problems[i]["shape"] != (4096, 7168, 16384)))
        dense.problems = [dense.problems[i] for i in order]      # M = 128 shapes, the largest GEMM, then the rest
        n_first = 6

    def step(rec=None):
        if overlap:
            main = torch.cuda.current_stream(dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                dense.step(rec, side_ctx, 0, n_first)

            def rest_of_dense():
                side.wait_stream(main)                      # after the down GEMM has been queued
                with torch.cuda.stream(side):
                    dense.step(rec, side_ctx, n_first, None)
            moe.record, moe.before_combine = rec, rest_of_dense
            moe.step()
            moe.record, moe.before_combine = None, None
            main.wait_stream(side)
            return
        if dense is not None:
            dense.step(rec)
        if moe is not None:
            moe.record = rec
            moe.step()
            moe.record = None
        if masked is not None:
            masked.record = rec
            masked.step()
            masked.record = None

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

    def sum_over_ranks(x):
        t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
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
    n_before = len(sampler.samples)
    ms_per_step = timed(lambda: step(record), args.steps)
    n_timed = len(sampler.samples) - n_before
    launch_us = phase_us(record)                 # this rank's launches, CUDA events inside the timed region
    # whole-job flops of one step: dense replicas + routed rows of all ranks
    moe_rows = sum_over_ranks(moe.routed_rows()) if moe is not None else 0.0
    flops = (dense.flops * world if dense is not None else 0.0) + (moe_rows * moe.flops_per_row if moe is not None else 0.0)
    if masked is not None:
        flops += masked.valid_all * masked.flops_per_row
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

    # ---- each half on its own (same K steps), per-GEMM times
    parts = {}
    extra_launches = 0
    if dense is not None:
        dense_rec = {}
        d_ms = timed(lambda: dense.step(dense_rec), args.steps) if moe is not None else ms_per_step
        parts["dense_fp8"] = {"tflops": dense.flops * world / (d_ms * 1e-3) / 1e12, "ms_per_step": d_ms, "parallelism": "replica per GPU",
                              "launch_us_in_step_rank0": {k[6:]: round(v, 1) for k, v in launch_us.items() if k.startswith("dense ")}}
        if overlap:
            # on its own stream a dense launch queues behind the other stream's GEMMs: the events around it in the step measure
            # that wait too, so the launch times used for the roofline come from the dense pass run on its own
            parts["dense_fp8"]["launch_us_in_step_rank0_note"] = "includes time queued behind the MoE GEMMs of the other stream"
            alone = phase_us(dense_rec)
            parts["dense_fp8"]["launch_us_dense_pass_alone_rank0"] = {k[6:]: round(v, 1) for k, v in alone.items()}
            launch_us.update(alone)
    if moe is not None:
        m_ms = timed(moe.step, args.steps) if dense is not None else ms_per_step
        gemm_ms, gemm_rows = moe.gate_up_alone()
        parts["moe_ep"] = {"tflops": moe_rows * moe.flops_per_row / (m_ms * 1e-3) / 1e12, "ms_per_step": m_ms, "routed_rows_all_ranks": moe_rows,
                           "gate_up_gemm_us_rank0": gemm_ms * 1e3,
                           "gate_up_gemm_tflops_rank0": 2.0 * gemm_rows * MOE["gate_up_n"] * MOE["hidden"] / (gemm_ms * 1e-3) / 1e12,
                           "phases_us_rank0": {k: round(v, 1) for k, v in launch_us.items() if not k.startswith("dense")},
                           "parallelism": f"ep{world}: {moe.local_e} experts per GPU"}
    per_shape = dense.per_gemm(peaks) if (dense is not None and rank == 0 and world == 1) else None
    fence()

    # ---- parity, outside every timed region, on every rank
    parity = None
    if not args.no_extras:
        parity = {}
        ok = 1
        if moe is not None and moe.peer is not None and moe.pipe is None:
            good, n_tok = moe.parity_check(moe.step())
            ok = int(good)
            parity["moe_tokens_checked"] = int(sum_over_ranks(n_tok))
            parity["moe_check"] = ("sampled tokens of every rank recomputed without the exchange (local one-pair groups, the experts' weights "
                                   "rebuilt from their ids, same grouped GEMMs, activation kernel and reduction), compared bit for bit")
        if masked is not None:
            good, n_tok = masked.parity_check(masked.step())
            ok = int(good)
            parity["masked_tokens_checked"] = int(sum_over_ranks(n_tok))
            parity["masked_check"] = "sampled tokens of every rank recomputed without the exchange (one local slot per pair), compared bit for bit"
        flag = torch.tensor([ok], device=dev, dtype=torch.int32)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity["bit_exact"] = bool(flag.item())
        if dense is not None:
            big = max(dense.problems, key=lambda p: p["shape"][0] * p["shape"][1] * p["shape"][2])
            small = min(dense.problems, key=lambda p: p["shape"][0] * p["shape"][1] * p["shape"][2])
            diffs = torch.tensor([dense_parity(torch, big), dense_parity(torch, small)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(diffs, op=dist.ReduceOp.MAX)
            parity["dense_calc_diff"] = float(diffs[0].item())
            parity["dense_calc_diff_launch"] = "dense %dx%dx%d, sampled rows x columns against a torch f64 product of the dequantised operands (max over ranks)" % big["shape"]
            parity["skinny_calc_diff"] = float(diffs[1].item())
            parity["skinny_calc_diff_launch"] = "dense %dx%dx%d" % small["shape"]
            parity["tolerance"] = 1e-3
    fence()

    # ---- configurations outside the step: single launches on rank 0, the masked decode step on every rank
    if not args.no_extras and args.workload == "dsv3":
        if rank == 0:
            singles = SingleLaunches(torch, dg, ctx, dev, peaks)
            parts["single_launches_rank0"] = singles.run()
            extra_launches += singles.launches
            del singles
            torch.cuda.empty_cache()
        fence()
        mk = MaskedEpWork(torch, dist, dg, ctx, dev, rank, world)
        for _ in range(3):
            mk.step()
        rec = {}
        mk.record = rec
        mk_ms = timed(mk.step, args.steps)
        mk.record = None
        good, n_tok = mk.parity_check(mk.step())
        flag = torch.tensor([int(good)], device=dev, dtype=torch.int32)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ph = phase_us(rec)
        c5 = MASKED
        c5_bytes = mk.valid_local * c5["hidden"] + c5["local_experts"] * c5["n"] * c5["hidden"] + mk.valid_local * c5["n"] * (1 + 1 / 32) \
            + 4 * ((c5["hidden"] + 511) // 512) * (mk.valid_local + c5["local_experts"] * c5["n"])
        parts["moe_masked_ep"] = {"tflops": mk.valid_all * mk.flops_per_row / (mk_ms * 1e-3) / 1e12, "ms_per_step": mk_ms,
                                  "valid_rows_all_ranks": mk.valid_all, "tokens_per_rank": mk.tokens,
                                  "phases_us_rank0": {k: round(v, 1) for k, v in ph.items()},
                                  "masked_gemm_fp8_out_rank0": launch_bound(2.0 * mk.valid_local * c5["n"] * c5["hidden"], c5_bytes,
                                                                            ph["masked_gemm_fp8_out"] * 1e-6, peaks, 2),
                                  "bit_exact": bool(flag.item()), "tokens_checked": int(sum_over_ranks(n_tok)),
                                  "parallelism": f"ep{world}: {c5['local_experts']} experts per GPU, {c5['local_experts'] * world} in all",
                                  "what": "route + dispatch into the owners' (32, 256, K) slots over peer memory, masked GEMM N=4096 K=7168 with e4m3 "
                                          "output and per-32 scales, a masked GEMM N=7168 K=4096 consuming that output, weighted combine"}
        extra_launches += mk.launches * (args.steps + 3)
        mk.close()
        del mk
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
        if h2d:
            e2e_step()
            e2e_ms = timed(e2e_step, e2e_steps, e2e_drain)
            e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "ms_per_step": e2e_ms, "steps": e2e_steps,
                   "h2d_gbs_per_rank": round(h2d / e2e_ms / 1e6, 1), "d2h_gbs_per_rank": round(d2h / e2e_ms / 1e6, 1),
                   "what": "per rank and step: the activations (A and its scale words) of every dense GEMM in, every D out; MoE: this rank's "
                           "e4m3 tokens, scales and routing in, reduced rows out.  Weights are parameters and stay resident in HBM.  Uploads, "
                           "compute and downloads on three streams, ordered per buffer by events; the host side of the copies is shared by "
                           "all ranks of the node"}
    ctx.sync()
    if side_ctx is not None:
        side_ctx.sync()          # a device-side wait that ran out on the second stream is reported like one on the first

    if rank == 0:
        # ---- the launch with the largest share of this rank's step is the one the roofline entry describes
        sm_mhz = clocks.get("sm_mhz") if clocks else None
        sustained = bool(sm_mhz and clocks.get("sm_max_mhz") and sm_mhz < 0.85 * clocks["sm_max_mhz"])
        candidates = []
        if dense is not None:
            for (m, n, k) in DENSE_SHAPES:
                us = launch_us.get("dense %dx%dx%d" % (m, n, k))
                if us:
                    candidates.append((us, "dense fp8 %dx%dx%d" % (m, n, k), 2.0 * m * n * k, dense_bytes(m, n, k),
                                       "dg_gemm_kernel<e4m3, bf16 out>"))
        if moe is not None and "gate_up" in launch_us:
            rows0 = moe.routed_rows()
            for name, n, k in (("gate_up", MOE["gate_up_n"], MOE["hidden"]), ("down", MOE["down_n"], MOE["down_k"])):
                nbytes = rows0 * k + moe.local_e * n * k + 2 * rows0 * n + 4 * ((k + 511) // 512) * (rows0 + moe.local_e * n)
                candidates.append((launch_us[name], f"grouped {name} ({moe.local_e} local experts, {rows0} routed rows, N={n} K={k})",
                                   2.0 * rows0 * n * k, nbytes, "dg_gemm_kernel<e4m3, bf16 out>, contiguous grouped layout"))
        if masked is not None:
            c5 = MASKED
            nbytes = masked.valid_local * c5["hidden"] + c5["local_experts"] * c5["n"] * c5["hidden"] + masked.valid_local * c5["n"] * (1 + 1 / 32)
            candidates.append((launch_us["masked_gemm_fp8_out"], f"masked fp8-out ({masked.valid_local} valid rows)",
                               2.0 * masked.valid_local * c5["n"] * c5["hidden"], nbytes, "dg_gemm_kernel<e4m3, e4m3 out>, masked layout"))
        traffic_table = {}
        try:
            with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
                traffic_table = json.load(f)
        except (OSError, ValueError):
            pass

        def roofline_entry(cand):
            us, name, fl, nbytes, kernel = cand
            row = launch_bound(fl, nbytes, us * 1e-6, peaks, 2)

            def rows_match(entry):
                # an entry measured (or scaled) for a given number of routed rows only describes launches within 5 % of it
                want = entry.get("routed_rows")
                if not want or "routed rows" not in name:
                    return True
                have = int(name.split(" routed rows")[0].split(", ")[-1])
                return abs(have - want) <= 0.05 * want
            keys = [key for key in traffic_table if name.startswith(key) and rows_match(traffic_table[key])]
            tr = traffic_table[max(keys, key=len)] if keys else None
            entry = {"bound": row["bound"], "kernel": kernel, "launch": name, "us_in_step": round(us, 1),
                     "share_of_step": round(us * 1e-3 / ms_per_step, 3), "sm_mhz_median": sm_mhz,
                     "traffic": tr["dram_bytes_per_launch"] if tr else None, "traffic_source": tr["source"] if tr else None,
                     "algorithmic_bytes": nbytes, "algorithmic_flops": fl}
            if row["bound"] == "tensor":
                peak = 2 * (peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"])
                entry.update(achieved=fl / (us * 1e-6) / 1e12, peak=peak, unit="TFLOP/s", frac=fl / (us * 1e-6) / 1e12 / peak,
                             frac_burst=row["frac_burst"], frac_sustained=row["frac_sustained"], frac_of_nominal_fp8_4500=row["frac_nominal"],
                             peak_source=f"2 x bf16_tflops{'_sustained' if sustained else ''} of {peaks['source']} peaks (e4m3 issues at twice the "
                                         f"bf16 rate); {'sustained' if sustained else 'burst'} figure because the SM clock sampled under this load "
                                         f"is {sm_mhz} MHz")
            else:
                entry.update(achieved=nbytes / (us * 1e-6) / 1e9, peak=peaks["hbm_gbs"], unit="GB/s", frac=row["frac"],
                             frac_of_nominal_8000=row["frac_nominal"], peak_source=f"hbm_gbs of {peaks['source']} peaks (copy bandwidth)")
            return entry

        candidates.sort(key=lambda c: -c[0])
        roofline = roofline_entry(candidates[0]) if candidates else None
        others = [roofline_entry(c) for c in candidates[1:4]]
        config = {"workload": {"dsv3": "dsv3_fp8_gemms (dense pass + expert-parallel MoE pair)", "dense_fp8": "dense_fp8_dsv3",
                               "moe_ep": "moe_contiguous_ep", "moe_masked_ep": "moe_masked_decode_ep"}[args.workload],
                  "gran_k": 128, "out": "bf16", "parallelism": ("single GPU" if world == 1 else f"dense: replica per GPU; MoE: ep{world}"),
                  "l2": "a step touches 1.1 GB of dense operands and 1.4-11 GB of expert weights per GPU, far more than the 126 MB L2"}
        if dense is not None:
            config["dense_shapes"] = DENSE_SHAPES
        if overlap:
            config["streams"] = ("the dense GEMMs run on a second stream beside the MoE layer's dispatch and combine kernels; both streams start "
                                 "inside the step and are joined before it ends")
        if moe is not None:
            config["moe"] = dict(MOE, experts_per_gpu=moe.local_e, mk_alignment=128,
                                 collective=moe.exchange_note)
        if masked is not None:
            config["masked"] = dict(MASKED, tokens_per_rank=masked.tokens)
        launches = (dense.launches if dense is not None else 0) + (moe.launches if moe is not None else 0) + (masked.launches if masked is not None else 0)
        line = {"metric": "fp8_block_scaled_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp8_e4m3", "data": "synthetic", "config": config, "clocks": clocks, "gpu_launches": args.steps * launches,
                "roofline": roofline, "roofline_next": others, "parts": parts}
        if parity is not None:
            line["parity"] = parity
        if per_shape is not None:
            line["per_gemm"] = per_shape
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            threads = host_threads()
            cases = cpu_sample_inputs()
            cpu_step(cases, threads)                      # warm pass: thread pool up, operands in cache
            secs = [cpu_step(cases, threads) for _ in range(2)]
            sec = min(secs)
            line["cpu_baseline"] = {"value": cpu_sample_flops(cases) / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{CPU_SAMPLE_TEXT}; best of 2 passes after a warm one ({sec:.1f} s each)"}
        print(json.dumps(line), flush=True)
    if moe is not None and moe.peer is not None:
        # unmap the peers' buffers and free this rank's, in step with the other ranks, before the process group goes away
        (moe.pipe or moe.peer).close()
    if masked is not None:
        masked.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
