"""Parity at the benchmark contract's full sizes for the configurations beyond dense FP8: MXFP4 and FP8 x FP4
4096x7168x7168, the contiguous m-grouped pair with 256 experts and 65 536 routed rows, and the masked decode GEMM
(32 experts x up to 256 rows, N=4096, K=7168) with the FP8-requantising epilogue.

Operands are quantised on the GPU (the quantisers are bit-exact with the oracle: tests/test_quant_gpu.py); outputs are
compared with the CPU oracle on sampled rows and columns that include every kind of tile and group edge.  Tolerance:
calc_diff <= 1e-3 is the contract; identical quantised inputs must agree to 2e-5 with a bf16 output and 1e-6 with f32,
and the FP8 output bytes and scale words must be bit-exact against the oracle epilogue applied to the GPU's own f32
accumulators.
"""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from oracle import oracle as O
from tests.helpers import dev, sample_indices, to_f32

pytestmark = pytest.mark.gpu
TOL, TIGHT_BF16, TIGHT_F32 = 1e-3, 2e-5, 1e-6


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


def randn_bf16(gen, rows, k):
    return torch.randn((rows, k), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)


def idx_dev(idx):
    return torch.from_numpy(np.asarray(idx, dtype=np.int64)).cuda()


def compact_rows(data, sf, idx, k, gran, stride):
    """Rows `idx` of a flat operand and their scale words (sf[c * stride + row]) as a small operand the oracle can take whole."""
    cols = dg.sf_packed_cols(k, gran)
    words = sf.view(-1, stride)[:, idx_dev(idx)].cpu().numpy().view(np.uint32)
    packed = np.zeros((cols, dg.sf_aligned_rows(len(idx))), np.uint32)
    packed[:, :len(idx)] = words
    return data[idx_dev(idx)].cpu().numpy(), packed.reshape(-1)


@pytest.mark.parametrize("kind", ["mxfp4_reference_rule", "mxfp4_range_fit", "fp8_x_fp4", "fp4_x_fp8"])
def test_c3_mxfp4_and_mixed_full_size(ctx, kind):
    # reference entry: ops_sm100.rs:719 with 4-bit operands; checker: mxfp4_gemm_reference (reference.rs:293-329) for the
    # pure FP4 case, the dequantise + f64 product for the mixed one (no CPU function in the reference covers it)
    m, n, k = 4096, 7168, 7168
    gen = torch.Generator(device="cuda").manual_seed(1003)
    x, w = randn_bf16(gen, m, k), randn_bf16(gen, n, k)
    rule = dg.SF_RULE_REFERENCE_CPU if kind == "mxfp4_reference_rule" else dg.SF_RULE_RANGE_FIT

    def quant(src, rows, bits):
        if bits == 4:
            q, sf = dg.cast_bf16_to_fp4_packed_sf_dev(ctx, src, k, rows, k, 1, rule)
        else:
            q, sf = dg.cast_bf16_to_fp8_sf_dev(ctx, src, k, rows, k, 32)
        return q, sf

    a_bits = 8 if kind == "fp8_x_fp4" else 4
    b_bits = 8 if kind == "fp4_x_fp8" else 4
    aq, asf = quant(x, m, a_bits)
    bq, bsf = quant(w, n, b_bits)
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, dg.LpOperand(aq, asf, m, k, k, a_bits, 32), dg.LpOperand(bq, bsf, n, k, k, b_bits, 32), dg.Sm100Out.Bf16(d, n))
    ctx.sync()
    assert not torch.isnan(d).any()
    rows, cols = sample_indices(m, 24, 5), sample_indices(n, 40, 6, edges=(0, 1, 127, 128, 223, 224, 255, 256, 447, 448, 511, 512))
    an, asfn = compact_rows(aq, asf, rows, k, 32, dg.sf_aligned_rows(m))
    bn, bsfn = compact_rows(bq, bsf, cols, k, 32, dg.sf_aligned_rows(n))
    got = to_f32(d[idx_dev(rows)][:, idx_dev(cols)])
    if a_bits == 4 and b_bits == 4:
        want = O.mxfp4_gemm_reference(an, asfn, len(rows), bn, bsfn, len(cols), k, threads=8)
    else:
        want = O.lp_gemm_rows(an, asfn, a_bits, 32, 1, len(rows), np.arange(len(rows), dtype=np.uint32),
                              bn, bsfn, b_bits, 32, 1, len(cols), np.arange(len(cols), dtype=np.uint32), k)
    diff = O.calc_diff(got, want)
    assert diff <= TOL and diff <= TIGHT_BF16, diff


def routed_group_sizes(tokens=8192, experts=256, topk=8, seed=3000):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn((tokens, experts), generator=g, device="cuda", dtype=torch.float32)
    topi = torch.softmax(logits, -1).topk(topk, dim=-1).indices
    return torch.bincount(topi.reshape(-1), minlength=experts).cpu().numpy()


@pytest.mark.parametrize("n,k", [(4096, 7168), (7168, 2048)])
def test_c4_contiguous_256_experts_full_size(ctx, n, k):
    # reference entry: ops_sm100.rs:759; checker: the per-row expert product of reference.rs:133-168 on sampled rows of every
    # expert (first, second, last valid row, a row either side of every 128-row tile edge inside the group) and sampled
    # columns; alignment padding rows past the group's last 32-row store box must keep the caller's contents
    experts = 256
    sizes = routed_group_sizes()
    assert sizes.sum() == 65536
    starts = np.concatenate([[0], np.cumsum((sizes + 127) // 128 * 128)])
    m_total = int(starts[-1])
    m_idx = np.full(m_total, -1, np.int32)
    for e in range(experts):
        m_idx[starts[e]:starts[e] + sizes[e]] = e
    gen = torch.Generator(device="cuda").manual_seed(1004 + n)
    aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn_bf16(gen, m_total, k), k, m_total, k, 128)
    bq = torch.empty((experts * n, k), dtype=torch.uint8, device="cuda")
    bsf = dg.alloc_sf(ctx, experts * n, k, 128, experts)
    cols_sf, stride_b = dg.sf_packed_cols(k, 128), dg.sf_aligned_rows(n)
    for e0 in range(0, experts, 16):
        wq, wsf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn_bf16(gen, 16 * n, k), k, 16 * n, k, 128, 16)
        bq[e0 * n:(e0 + 16) * n] = wq
        bsf.view(experts, cols_sf, stride_b)[e0:e0 + 16] = wsf.view(16, cols_sf, stride_b)
    d = torch.full((m_total, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(aq, asf, m_total, k, k), torch.from_numpy(m_idx).cuda(),
                                             dg.LpOperand(bq, bsf, experts * n, k, k), dg.Sm100Out.Bf16(d, n), experts)
    ctx.sync()
    valid = m_idx >= 0
    nan_rows = torch.isnan(d.float()).any(dim=1).cpu().numpy()
    assert not nan_rows[valid].any()              # every routed row was written
    for e in range(experts):                      # stores go out in 32-row boxes: padding rows past a group's last box are never written
        first_untouched = int(starts[e]) + (int(sizes[e]) + 31) // 32 * 32
        assert nan_rows[first_untouched:int(starts[e + 1])].all(), e
    cols = sample_indices(n, 20, 9, edges=(0, 127, 128, 255, 256))
    worst = 0.0
    for e in range(experts):
        s, cnt = int(starts[e]), int(sizes[e])
        if cnt == 0:
            continue
        local = sorted({r for r in (0, 1, 127, 128, 129, 255, 256, 257, cnt - 2, cnt - 1) if 0 <= r < cnt})
        rows = np.array([s + r for r in local], dtype=np.int64)
        an, asfn = compact_rows(aq, asf, rows, k, 128, dg.sf_aligned_rows(m_total))
        bn = bq[idx_dev(e * n + cols.astype(np.int64))].cpu().numpy()
        bsfn = bsf.view(experts, cols_sf, stride_b)[e][:, idx_dev(cols)].cpu().numpy().view(np.uint32)
        packed = np.zeros((cols_sf, dg.sf_aligned_rows(len(cols))), np.uint32)
        packed[:, :len(cols)] = bsfn
        want = O.lp_gemm_rows(an, asfn, 8, 128, 1, len(rows), np.arange(len(rows), dtype=np.uint32),
                              bn, packed.reshape(-1), 8, 128, 1, len(cols), np.arange(len(cols), dtype=np.uint32), k)
        got = to_f32(d[idx_dev(rows)][:, idx_dev(cols)])
        worst = max(worst, O.calc_diff(got, want))
    assert worst <= TOL and worst <= TIGHT_BF16, worst


def test_c5_masked_decode_fp8_out_full_size(ctx):
    # reference entry: ops_sm100.rs:815 (the FP8 output on this layout is new here); masked_m ~ randint(0, 257), seed 4000
    # (the benchmark contract's draw); checker: reference.rs:172-208 on sampled rows through the f32 output, then the oracle's
    # requantising epilogue applied to the GPU's own f32 accumulators must reproduce the e4m3 bytes and scale words bit for bit
    g, m_max, n, k = 32, 256, 4096, 7168
    masked = torch.randint(0, m_max + 1, (g,), generator=torch.Generator().manual_seed(4000), dtype=torch.int32)
    mm = masked.numpy()
    gen = torch.Generator(device="cuda").manual_seed(1005)
    aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn_bf16(gen, g * m_max, k), k, g * m_max, k, 128, g)
    bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, randn_bf16(gen, g * n, k), k, g * n, k, 128, g)
    a, b = dg.LpOperand(aq, asf, m_max, k, k), dg.LpOperand(bq, bsf, g * n, k, k)
    d32 = torch.full((g * m_max, n), float("nan"), dtype=torch.float32, device="cuda")
    d8 = torch.full((g * m_max, n), 0xAA, dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(g * (n // 128) * m_max, dtype=torch.int32, device="cuda")
    expected = max(1, int(mm.sum()) // g)
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a, masked.cuda(), b, dg.Sm100Out.F32(d32, n), g, expected)
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a, masked.cuda(), b, dg.Sm100Out.Fp8(d8, n, sfd), g, expected)
    ctx.sync()
    cols_sf = dg.sf_packed_cols(k, 128)
    cols = sample_indices(n, 24, 3, edges=(0, 127, 128, 255, 256))
    got8 = d8.cpu().numpy()
    got_sfd = sfd.cpu().numpy().view(np.uint32).reshape(g, n // 128, m_max)
    worst = 0.0
    for e in range(g):
        v = int(mm[e])
        if v == 0:
            continue
        local = sorted({r for r in (0, 1, 31, 32, 127, 128, 129, v - 2, v - 1) if 0 <= r < v})
        rows = np.array([e * m_max + r for r in local], dtype=np.int64)
        an = aq[idx_dev(rows)].cpu().numpy()
        aw = asf.view(g, cols_sf, m_max)[e][:, idx_dev(local)].cpu().numpy().view(np.uint32)
        ap = np.zeros((cols_sf, dg.sf_aligned_rows(len(local))), np.uint32)
        ap[:, :len(local)] = aw
        bn = bq[idx_dev(e * n + cols.astype(np.int64))].cpu().numpy()
        bw = bsf.view(g, cols_sf, dg.sf_aligned_rows(n))[e][:, idx_dev(cols)].cpu().numpy().view(np.uint32)
        bp = np.zeros((cols_sf, dg.sf_aligned_rows(len(cols))), np.uint32)
        bp[:, :len(cols)] = bw
        want = O.lp_gemm_rows(an, ap.reshape(-1), 8, 128, 1, len(local), np.arange(len(local), dtype=np.uint32),
                              bn, bp.reshape(-1), 8, 128, 1, len(cols), np.arange(len(cols), dtype=np.uint32), k)
        worst = max(worst, O.calc_diff(to_f32(d32[idx_dev(rows)][:, idx_dev(cols)]), want))
        # FP8 output of every valid row of the group against the oracle epilogue on the GPU's f32 accumulators
        acc = d32[e * m_max:e * m_max + v].cpu().numpy()
        want8 = np.zeros((v, n), np.uint8)
        want_sfd = np.zeros(g * (n // 128) * m_max, np.uint32)
        O.requant_fp8(acc, e, m_max, want8, want_sfd)
        assert np.array_equal(got8[e * m_max:e * m_max + v], want8), e
        assert np.array_equal(got_sfd[e, :, :v], want_sfd.reshape(g, n // 128, m_max)[e, :, :v]), e
    assert worst <= TOL and worst <= TIGHT_F32, worst
    # rows of tiles that were never scheduled keep the caller's contents
    for e in range(g):
        first_untouched = e * m_max + (int(mm[e]) + 255) // 256 * 256
        if first_untouched < (e + 1) * m_max:
            assert (got8[first_untouched:(e + 1) * m_max] == 0xAA).all()


def test_dense_mn_major_full_size_equals_k_major(ctx):
    # MN-major e4m3 operands at a benchmark shape: bit-identical to the K-major call on the same bytes, which the tests above
    # hold to the oracle (every tile and k-block boundary of the 4096 x 7168 x 7168 problem is crossed)
    m, n, k = 4096, 7168, 7168
    gen = torch.Generator(device="cuda").manual_seed(77)
    aq = torch.randint(0, 0x7E, (m, k), dtype=torch.uint8, device="cuda", generator=gen)
    bq = torch.randint(0, 0x7E, (n, k), dtype=torch.uint8, device="cuda", generator=gen)
    words = lambda rows: dg.sf_packed_cols(k, 128) * dg.sf_aligned_rows(rows)
    asf = torch.randint(118, 130, (words(m) * 4,), dtype=torch.uint8, device="cuda", generator=gen).view(torch.int32)
    bsf = torch.randint(118, 130, (words(n) * 4,), dtype=torch.uint8, device="cuda", generator=gen).view(torch.int32)
    want = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, dg.LpOperand(aq, asf, m, k, k), dg.LpOperand(bq, bsf, n, k, k), dg.Sm100Out.Bf16(want, n))
    a_t = aq.t().contiguous()          # (k, m): rows contiguous
    b_t = bq.t().contiguous()
    for a_op, b_op in ((dg.LpOperand(a_t, asf, m, k, m, 8, 128, True), dg.LpOperand(bq, bsf, n, k, k)),
                       (dg.LpOperand(aq, asf, m, k, k), dg.LpOperand(b_t, bsf, n, k, n, 8, 128, True)),
                       (dg.LpOperand(a_t, asf, m, k, m, 8, 128, True), dg.LpOperand(b_t, bsf, n, k, n, 8, 128, True))):
        d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.fp8_fp4_gemm_dev(ctx, a_op, b_op, dg.Sm100Out.Bf16(d, n))
        ctx.sync()
        assert torch.equal(d, want)


def test_f32_scale_gemm_full_size_sampled(ctx):
    # the exact f32-scale route (ref_fp8_gemm_nt, reference.rs:85-114) at 4096 x 7168 x 7168 with scales that have mantissas:
    # sampled rows x two 128-column blocks against the literal reference
    m, n, k = 4096, 7168, 7168
    rng = np.random.default_rng(5)
    a = rng.integers(0, 0x7E, (m, k), dtype=np.uint8)
    b = rng.integers(0, 0x7E, (n, k), dtype=np.uint8)
    a[rng.random((m, k)) < 0.5] |= 0x80                       # both signs
    sfa = (rng.random((m, k // 128), dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    sfb = (rng.random((n // 128, k // 128), dtype=np.float32) * 0.02 + 0.001).astype(np.float32)
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), m, k // 128, 1)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(dev(a), m, k, k), a_sf_t, dg.Fp8Tensor(dev(b), n, k, k), dev(sfb), out, n)
    ctx.sync()
    rows = np.array(sorted(set(rng.integers(0, m, 40).tolist() + [0, 127, 128, 4095])), dtype=np.int64)
    got = to_f32(out)
    for blk in (0, 31, 55):
        cols = np.arange(blk * 128, (blk + 1) * 128)
        want = O.ref_fp8_gemm_nt(a[rows], sfa[rows], b[cols], sfb[blk:blk + 1], threads=8)
        g = got[rows][:, cols]
        assert np.max(np.abs(g - want) / np.maximum(np.abs(want), 1.0)) < 0.05          # tests/e2e.rs tolerance
        assert O.calc_diff(g, want) <= 2e-5
