"""MN-major e4m3 operands (LpOperand.major_mn, ops_sm100.rs:44,336-362): the same bytes stored (k, ld) with the rows of a
group contiguous.  The products are the K-major ones, so every case is held to the CPU oracle and, bit for bit, to the K-major
call on the same data (each output element adds its K products in the same order whatever the tile shape)."""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from oracle import oracle as O
from tests.helpers import dev, fp4_operand, fp8_operand_1d, sample_indices, to_f32

pytestmark = pytest.mark.gpu
TIGHT_BF16 = 2e-5
TIGHT_F32 = 1e-6


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


def k_major(q, sf, rows, k, gran=128):
    return dg.LpOperand(dev(q), dev(sf), rows, k, k, 8, gran)


def mn_major(q, sf, rows_per_group, k, groups=1, pad=0, gran=128, op_rows=None):
    """q: (groups * rows_per_group, k) bytes -> (groups, k, ld) with ld = rows rounded up to 16 bytes (+ pad), padding poisoned."""
    ld = (rows_per_group + 15) // 16 * 16 + pad
    t = torch.full((groups, k, ld), 0x7E, dtype=torch.uint8, device="cuda")      # 0x7E = 448: a stray read would show
    t[:, :, :rows_per_group] = dev(q).view(groups, rows_per_group, k).transpose(1, 2)
    return dg.LpOperand(t, dev(sf), rows_per_group if op_rows is None else op_rows, k, ld, 8, gran, True)


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("m,n,k,out_kind", [
    (128, 256, 512, 0),
    (300, 456, 1152, 1),      # ragged rows on both sides, nine k-blocks
    (77, 128, 128, 0),
    (520, 1000, 640, 0),
])
def test_dense_mn_major_equals_k_major(ctx, m, n, k, out_kind, ctas, a_mn, b_mn, monkeypatch):
    monkeypatch.setenv("DG_CTAS", str(ctas))
    _, aq, asf = fp8_operand_1d(m, k, 501)
    _, bq, bsf = fp8_operand_1d(n, k, 502)
    dtype = torch.bfloat16 if out_kind == 0 else torch.float32
    want_d = torch.zeros((m, n), dtype=dtype, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, k_major(aq, asf, m, k), k_major(bq, bsf, n, k), dg.Sm100Out(out_kind, want_d, n))
    a = mn_major(aq, asf, m, k, pad=16) if a_mn else k_major(aq, asf, m, k)
    b = mn_major(bq, bsf, n, k) if b_mn else k_major(bq, bsf, n, k)
    cfg = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, m, n, k, cd_dtype=out_kind, major_a_mn=a_mn, major_b_mn=b_mn))
    if b_mn:
        assert (cfg.block_n // cfg.cluster_m) % 128 == 0          # whole 128-row boxes per CTA
    d = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out(out_kind, d, n))
    ctx.sync()
    assert torch.equal(d, want_d)
    rows, cols = sample_indices(m, 40, 7), sample_indices(n, 48, 8)
    want = O.lp_gemm_rows(aq, asf, 8, 128, 1, m, rows, bq, bsf, 8, 128, 1, n, cols, k)
    got = to_f32(d)[np.asarray(rows, np.int64)][:, np.asarray(cols, np.int64)]
    assert O.calc_diff(got, want) <= (TIGHT_BF16 if out_kind == 0 else TIGHT_F32)


def test_dense_mn_major_with_k_ranges_and_accumulate(ctx, monkeypatch):
    # skinny problem: the heuristic cuts K into ranges (f32 partial planes + reduce kernel); then D += A.B^T
    m, n, k = 128, 1024, 4096
    _, aq, asf = fp8_operand_1d(m, k, 511)
    _, bq, bsf = fp8_operand_1d(n, k, 512)
    want_d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, k_major(aq, asf, m, k), k_major(bq, bsf, n, k), dg.Sm100Out.Bf16(want_d, n))
    d = torch.zeros_like(want_d)
    a, b = mn_major(aq, asf, m, k), mn_major(bq, bsf, n, k, pad=32)
    dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.Bf16(d, n))
    ctx.sync()
    assert torch.equal(d, want_d)
    acc = torch.ones((m, n), dtype=torch.float32, device="cuda")
    acc_k = acc.clone()
    dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.F32(acc, n), dg.Sm100Epilogue(accumulate=True))
    dg.fp8_fp4_gemm_dev(ctx, k_major(aq, asf, m, k), k_major(bq, bsf, n, k), dg.Sm100Out.F32(acc_k, n), dg.Sm100Epilogue(accumulate=True))
    ctx.sync()
    assert torch.equal(acc, acc_k)


def test_dense_mn_major_per_32_scales_and_fp4_partner(ctx):
    m, n, k = 200, 384, 1024
    _, aq, asf = fp8_operand_1d(m, k, 521, 32)
    _, bq4, bsf4 = fp4_operand(n, k, 522)
    b4 = dg.LpOperand(dev(bq4), dev(bsf4), n, k, k, 4, 32)
    want_d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, k_major(aq, asf, m, k, 32), b4, dg.Sm100Out.Bf16(want_d, n))
    d = torch.zeros_like(want_d)
    dg.fp8_fp4_gemm_dev(ctx, mn_major(aq, asf, m, k, gran=32), b4, dg.Sm100Out.Bf16(d, n))
    ctx.sync()
    assert torch.equal(d, want_d)
    rows, cols = sample_indices(m, 32, 9), sample_indices(n, 32, 10)
    want = O.lp_gemm_rows(aq, asf, 8, 32, 1, m, rows, bq4, bsf4, 4, 32, 1, n, cols, k)
    got = to_f32(d)[np.asarray(rows, np.int64)][:, np.asarray(cols, np.int64)]
    assert O.calc_diff(got, want) <= TIGHT_BF16


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
def test_bmm_and_masked_mn_major(ctx, a_mn, b_mn):
    groups, m, n, k = 3, 160, 256, 512
    _, aq, asf = fp8_operand_1d(groups * m, k, 531, 128, groups)
    _, bq, bsf = fp8_operand_1d(groups * n, k, 532, 128, groups)
    want_d = torch.zeros((groups * m, n), dtype=torch.float32, device="cuda")
    dg.fp8_fp4_bmm_dev(ctx, k_major(aq, asf, m, k), k_major(bq, bsf, n, k), dg.Sm100Out.F32(want_d, n), groups)
    a = mn_major(aq, asf, m, k, groups) if a_mn else k_major(aq, asf, m, k)
    b = mn_major(bq, bsf, n, k, groups, pad=16) if b_mn else k_major(bq, bsf, n, k)
    d = torch.zeros_like(want_d)
    dg.fp8_fp4_bmm_dev(ctx, a, b, dg.Sm100Out.F32(d, n), groups)
    ctx.sync()
    assert torch.equal(d, want_d)
    for g in range(groups):
        rows = np.arange(g * m, (g + 1) * m, dtype=np.uint32)
        colsb = np.arange(g * n, (g + 1) * n, dtype=np.uint32)
        want = O.lp_gemm_rows(aq, asf, 8, 128, groups, m, rows, bq, bsf, 8, 128, groups, n, colsb, k)
        assert O.calc_diff(to_f32(d)[g * m:(g + 1) * m], want) <= TIGHT_F32
    # masked layout over the same buffers: only the first masked_m[g] rows of every group are computed
    masked = np.array([160, 7, 0], np.int32)
    want_m = torch.full((groups * m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, k_major(aq, asf, m, k), dev(masked), k_major(bq, bsf, groups * n, k),
                                         dg.Sm100Out.Bf16(want_m, n), groups, 56)
    dm = torch.full_like(want_m, float("nan"))
    bm = mn_major(bq, bsf, n, k, groups, pad=16, op_rows=groups * n) if b_mn else k_major(bq, bsf, groups * n, k)
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a, dev(masked), bm, dg.Sm100Out.Bf16(dm, n), groups, 56)
    ctx.sync()
    for g in range(groups):
        sl = slice(g * m, g * m + int(masked[g]))
        assert torch.equal(dm[sl], want_m[sl]) and not torch.isnan(dm[sl]).any()


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("alignment", [128, 32])
def test_contiguous_mn_major(ctx, a_mn, b_mn, alignment):
    sizes, n, k = [37, 128, 1, 0, 200, 64], 384, 768
    groups = len(sizes)
    m_idx = []
    for g, s in enumerate(sizes):
        m_idx += [g] * s + [-1] * ((-s) % alignment)
    m_idx = np.array(m_idx, np.int32)
    m_total = len(m_idx)
    _, aq, asf = fp8_operand_1d(m_total, k, 541)
    _, bq, bsf = fp8_operand_1d(groups * n, k, 542, 128, groups)
    valid = torch.from_numpy(np.nonzero(m_idx >= 0)[0]).cuda()
    dg.set_mk_alignment_for_contiguous_layout(alignment)
    try:
        want_d = torch.zeros((m_total, n), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, k_major(aq, asf, m_total, k), dev(m_idx), k_major(bq, bsf, groups * n, k),
                                                 dg.Sm100Out.Bf16(want_d, n), groups)
        a = mn_major(aq, asf, m_total, k) if a_mn else k_major(aq, asf, m_total, k)
        b = mn_major(bq, bsf, n, k, groups, op_rows=groups * n) if b_mn else k_major(bq, bsf, groups * n, k)
        d = torch.zeros_like(want_d)
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a, dev(m_idx), b, dg.Sm100Out.Bf16(d, n), groups)
        ctx.sync()
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)
    assert torch.equal(d[valid], want_d[valid])
    g = 4
    rows = np.nonzero(m_idx == g)[0].astype(np.uint32)
    want = O.lp_gemm_rows(aq, asf, 8, 128, 1, m_total, rows, bq, bsf, 8, 128, groups, n, np.arange(g * n, (g + 1) * n, dtype=np.uint32), k)
    assert O.calc_diff(to_f32(d)[rows.astype(np.int64)], want) <= TIGHT_BF16


def test_mn_major_argument_errors(ctx):
    m, n, k = 128, 128, 256
    _, aq, asf = fp8_operand_1d(m, k, 551)
    _, bq4, bsf4 = fp4_operand(n, k, 552)
    d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    b4 = dg.LpOperand(dev(bq4), dev(bsf4), n, k, k, 4, 32, True)
    with pytest.raises(dg.DgError) as e:       # ops_sm100.rs:55,304
        dg.fp8_fp4_gemm_dev(ctx, k_major(aq, asf, m, k), b4, dg.Sm100Out.Bf16(d, n))
    assert e.value.kind == "Shape" and "K-major" in str(e.value)
    a = mn_major(aq, asf, m, k)
    a.ld = 96                                   # pitch shorter than the rows
    with pytest.raises(dg.DgError):
        dg.fp8_fp4_gemm_dev(ctx, a, k_major(aq, asf, m, k), dg.Sm100Out.Bf16(d, n))
    a.ld = 136                                  # not a multiple of 16 bytes
    with pytest.raises(dg.DgError):
        dg.fp8_fp4_gemm_dev(ctx, a, k_major(aq, asf, m, k), dg.Sm100Out.Bf16(d, n))
