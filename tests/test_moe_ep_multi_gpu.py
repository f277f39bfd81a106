"""Expert-parallel dispatch -> grouped GEMM -> combine on 2 GPUs, over NCCL all-to-all and over peer memory, checked on every rank against
a local recomputation: each rank also holds all experts' weights (same seed), so for its own tokens
out[t] = sum_j w[t,j] * (x_t . W[e_j]^T) can be computed with the dense GEMM path one expert at a time.
Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import deepgemm_rust_b200 as dg
        from deepgemm_rust_b200.moe_ep import DeviceRowOps, ExpertParallel, PeerExpertParallel, PipelinedPeerMoe
        from oracle import oracle as O
        dev = torch.device("cuda", rank)
        ctx = dg.DgContext(rank)
        experts, topk, tokens, k, n = 8, 2, 300, 512, 256
        local = experts // world
        g = torch.Generator(device=dev).manual_seed(7)                      # same weights everywhere
        w = torch.randn((experts * n, k), generator=g, device=dev).to(torch.bfloat16)
        wq, wsf = dg.cast_bf16_to_fp8_sf_dev(ctx, w, k, experts * n, k, 128, experts)
        cols, stride = dg.sf_packed_cols(k, 128), dg.sf_aligned_rows(n)
        wq_local = wq[rank * local * n:(rank + 1) * local * n].contiguous()
        wsf_local = wsf.view(experts, cols, stride)[rank * local:(rank + 1) * local].contiguous().view(-1)
        g2 = torch.Generator(device=dev).manual_seed(100 + rank)            # different tokens per rank
        x = torch.randn((tokens, k), generator=g2, device=dev).to(torch.bfloat16)
        topw, topi = torch.softmax(torch.randn((tokens, experts), generator=g2, device=dev), -1).topk(topk, dim=-1)
        topw = topw.contiguous()
        xq, xsf = dg.cast_bf16_to_fp8_sf_dev(ctx, x, k, tokens, k, 128)
        ep = ExpertParallel(experts, topk, DeviceRowOps(ctx))
        plan = ep.plan(topi)
        a, a_sf = ep.dispatch(plan, xq, xsf, k)
        h = torch.zeros((plan.m_pad, n), dtype=torch.bfloat16, device=dev)
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(a, a_sf, plan.m_pad, k, k), plan.m_indices,
                                                 dg.LpOperand(wq_local, wsf_local, local * n, k, k), dg.Sm100Out.Bf16(h, n), local)
        out = ep.combine(plan, h, topw)
        ctx.sync()
        # local recomputation: y_all[e] = x . W[e]^T for every expert through the dense GEMM, then the oracle reduction
        y_all = torch.zeros((experts * tokens, n), dtype=torch.bfloat16, device=dev)
        for e in range(experts):
            b_op = dg.LpOperand(wq[e * n:(e + 1) * n].contiguous(), wsf.view(experts, cols, stride)[e].contiguous().view(-1), n, k, k)
            dg.fp8_fp4_gemm_dev(ctx, dg.LpOperand(xq, xsf, tokens, k, k), b_op, dg.Sm100Out.Bf16(y_all[e * tokens:(e + 1) * tokens], n))
        ctx.sync()
        pos = (topi * tokens + torch.arange(tokens, device=dev).unsqueeze(1)).to(torch.int32).cpu().numpy()
        want = O.moe_combine(y_all.view(torch.int16).cpu().numpy().view(np.uint16), pos, topw.cpu().numpy())
        got = out.view(torch.int16).cpu().numpy().view(np.uint16)
        ok = bool(np.array_equal(got, want))
        # the same step over peer memory: rows written into / read from the owner's buffers directly
        pe = PeerExpertParallel(ctx, experts, topk, tokens, k, n)
        for _ in range(2):
            a_op, ends = pe.dispatch(topi, xq, xsf)
            dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, dg.LpOperand(wq_local, wsf_local, local * n, k, k),
                                                          dg.Sm100Out.Bf16(pe.result, n), local)
            out2 = pe.combine(topw)
            ctx.sync()
            ok = ok and bool(np.array_equal(out2.view(torch.int16).cpu().numpy().view(np.uint16), want)) and not pe.overflowed()
            totals = pe.totals.cpu().numpy()
            ok = ok and int(totals[1]) == plan.n_recv and int(totals[0]) == plan.m_pad
        pe.close()
        # and in token micro-batches whose exchange overlaps the other micro-batch's GEMM
        w_local = dg.LpOperand(wq_local, wsf_local, local * n, k, k)

        def compute(ex, a_op, ends):
            dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, w_local, dg.Sm100Out.Bf16(ex.result, n), local)

        pipe = PipelinedPeerMoe(ctx, experts, topk, tokens, k, n, chunks=2)
        for _ in range(2):
            out3 = pipe.run(topi, xq, xsf, topw, compute)
            torch.cuda.synchronize()
            ok = ok and bool(np.array_equal(out3.view(torch.int16).cpu().numpy().view(np.uint16), want))
        pipe.close()
        # masked layout (decode-style): fixed slots per local expert, the masked grouped GEMM on the exchange's own buffers
        pm = PeerExpertParallel(ctx, experts, topk, tokens, k, n, slot_rows=256)
        a_op, masked_m = pm.dispatch(topi, xq, xsf)
        dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a_op, masked_m, w_local, dg.Sm100Out.Bf16(pm.result, n), local, 150)
        out4 = pm.combine(topw)
        ctx.sync()
        ok = ok and bool(np.array_equal(out4.view(torch.int16).cpu().numpy().view(np.uint16), want)) and not pm.overflowed()
        pm.close()
        results[rank] = ok
        ctx.close()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        assert dict(results) == {0: True, 1: True}
