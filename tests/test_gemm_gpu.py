"""Parity of the tcgen05 GEMM family with the CPU oracle, through the C ABI.

Tolerance: calc_diff = 1 - 2*sum(xy)/sum(x^2+y^2) <= 1e-3 is the contract; both sides compute
the same quantised products, so the tests also hold the kernel to a much tighter internal bound
(bf16 rounding of the output is the only expected difference).
"""
import os

import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from oracle import oracle as O
from tests.helpers import dev, fp4_operand, fp8_operand_1d, fp8_operand_2d, randn_bf16, sample_indices, to_f32

pytestmark = pytest.mark.gpu
TOL = 1e-3          # contract
TIGHT_BF16 = 2e-5   # what identical quantised inputs should give with a bf16 output
TIGHT_F32 = 1e-6


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


# DG_SWAP pins the tile family: "0" activation rows on the UMMA M dimension (128 / 256-row tiles), "1" weight rows on UMMA M and
# activation rows on a UMMA N that follows the rows a tile has; None leaves the choice to the heuristic
both_families = pytest.mark.parametrize("family", ["0", "1"])


def pin_family(monkeypatch, family):
    if family is not None:
        monkeypatch.setenv("DG_SWAP", family)


def lp(q, sf, rows, k, bits=8, gran=128):
    return dg.LpOperand(dev(q), dev(sf), rows, k, k, bits, gran)


def check_sampled(d, a, a_meta, b, b_meta, k, rows, cols, tight, d_rows=None):
    """d: numpy f32 (all rows, n); compare d[d_rows][:, cols] with the oracle on operand rows `rows`."""
    aq, asf, abits, agran, agroups, agr = a_meta
    bq, bsf, bbits, bgran, bgroups, bgr = b_meta
    want = O.lp_gemm_rows(aq, asf, abits, agran, agroups, agr, rows, bq, bsf, bbits, bgran, bgroups, bgr, cols, k)
    got = d[np.asarray(rows if d_rows is None else d_rows, dtype=np.int64)][:, np.asarray(cols, dtype=np.int64) % d.shape[1]]
    diff = O.calc_diff(got, want)
    assert diff <= TOL, diff
    assert diff <= tight, diff
    return diff


def run_dense(ctx, m, n, k, gran=128, out_kind=0, alpha=None, seed=0, b_tile_scales=True):
    _, aq, asf = fp8_operand_1d(m, k, 1000 + seed, gran)
    if b_tile_scales and gran == 128 and n % 128 == 0:
        _, bq, bsf, _ = fp8_operand_2d(n, k, 2000 + seed)
    else:
        _, bq, bsf = fp8_operand_1d(n, k, 2000 + seed, gran)
    dtype = torch.bfloat16 if out_kind == 0 else torch.float32
    d = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    out = dg.Sm100Out(out_kind, d, n)
    dg.fp8_fp4_gemm_dev(ctx, lp(aq, asf, m, k, 8, gran), lp(bq, bsf, n, k, 8, gran), out, dg.Sm100Epilogue(alpha=alpha))
    ctx.sync()
    dn = to_f32(d)
    assert not np.isnan(dn).any()
    rows, cols = sample_indices(m, 48, seed), sample_indices(n, 64, seed + 1)
    if alpha is not None:
        dn = dn / np.float32(alpha)
    return check_sampled(dn, aq, (aq, asf, 8, gran, 1, m), bq, (bq, bsf, 8, gran, 1, n), k, rows, cols,
                         TIGHT_BF16 if out_kind == 0 else TIGHT_F32)


@pytest.mark.parametrize("m,n,k", [
    (128, 256, 512),      # the CPU-runnable case's shape
    (256, 512, 768),      # reference e2e shape (tests/e2e.rs:47)
    (128, 128, 128),      # one tile, one k-block
    (100, 192, 640),      # ragged M, 5 k-blocks (scale word with a 1-byte tail)
    (384, 2112, 1024),    # N not a multiple of the tile width
    (1, 64, 256), (129, 72, 384),
])
@both_families
def test_dense_fp8_small(ctx, m, n, k, family, monkeypatch):
    pin_family(monkeypatch, family)
    run_dense(ctx, m, n, k)


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("block_n", [32, 64, 96, 128, 160, 192, 224, 256])
@pytest.mark.parametrize("slabs", [1, 2])
def test_dense_fp8_every_tile_shape(ctx, ctas, block_n, slabs, monkeypatch):
    # DG_BLOCK_N / DG_CTAS pin the tile the heuristic would otherwise choose: every width the epilogue can
    # store, single CTA and CTA pair (256-row tiles, B split between the two CTAs), single- and
    # double-buffered accumulators, with ragged M and N so edge tiles are partly out of bounds
    if block_n % (16 * ctas) != 0:
        pytest.skip("tile width not issuable")
    monkeypatch.setenv("DG_BLOCK_N", str(block_n))
    monkeypatch.setenv("DG_CTAS", str(ctas))
    monkeypatch.setenv("DG_K_SLABS", str(slabs))     # 128 or 256 bytes of K per pipeline stage (K = 1152 leaves a half-empty last stage)
    try:
        cfg = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 600, 1000, 1152))
    except dg.DgError:
        pytest.skip("this tile does not fit three stages of two slabs")
    assert cfg.block_n == block_n and cfg.cluster_m == ctas and cfg.block_m == 128 * ctas and cfg.block_k == 128 * slabs
    run_dense(ctx, 600, 1000, 1152, seed=block_n + ctas)
    try:
        dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 600, 1000, 1152, cd_dtype=1))
    except dg.DgError:
        return                                       # the wider f32 staging buffers leave too few stages for this tile
    run_dense(ctx, 600, 1000, 1152, out_kind=1, seed=block_n + ctas)


@pytest.mark.parametrize("splits", [2, 3, 5])
def test_dense_fp8_split_k(ctx, splits, monkeypatch):
    # first tile family: K ranges computed by different CTAs, f32 partials summed by a second kernel; ranges are multiples of
    # 4 k-blocks, the last one may be shorter (K = 36 k-blocks here)
    monkeypatch.setenv("DG_SPLITS", str(splits))
    monkeypatch.setenv("DG_SWAP", "0")
    cfg = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 128, 1000, 4608))
    assert cfg.num_splits == splits and not cfg.swap_ab
    run_dense(ctx, 128, 1000, 4608, seed=splits)
    run_dense(ctx, 100, 512, 4608, out_kind=1, seed=splits, alpha=0.5)
    run_dense(ctx, 300, 256, 9216, out_kind=0, seed=splits, alpha=2.0)


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("splits", [1, 2, 3, 4, 5, 7, 8])
def test_swapped_dense_k_ranges_in_a_cluster(ctx, splits, ctas, monkeypatch):
    # swapped family (what the reference runs for few rows: heuristics_sm100.rs:341-452): weight rows on UMMA M, the rows of A on
    # UMMA N; K is cut into `splits` ranges, one per CTA (or pair) of a cluster, whose partial tiles are summed through shared
    # memory in range order.  Ranges may start inside a scale word (37 k-blocks here), N is ragged, M takes the values a
    # decode batch has.  The sum does not depend on how the launch went: two runs give the same bits.
    if splits * ctas > 8:
        pytest.skip("a cluster holds at most 8 CTAs")
    monkeypatch.setenv("DG_SWAP", "1")
    monkeypatch.setenv("DG_SPLITS", str(splits))
    monkeypatch.setenv("DG_CTAS", str(ctas))
    cfg = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 128, 1000, 4736))
    assert cfg.swap_ab and cfg.num_splits == splits and cfg.cluster_n == ctas
    for m in (1, 16, 17, 100, 128, 250):
        run_dense(ctx, m, 1000, 4736, seed=splits + m)
    run_dense(ctx, 100, 520, 4736, out_kind=1, seed=splits, alpha=0.5)
    run_dense(ctx, 128, 328, 2176, gran=32, seed=splits)
    _, aq, asf = fp8_operand_1d(77, 4736, 5)
    _, bq, bsf = fp8_operand_1d(1000, 4736, 6)
    outs = []
    for _ in range(2):
        d = torch.zeros((77, 1000), dtype=torch.float32, device="cuda")
        dg.fp8_fp4_gemm_dev(ctx, lp(aq, asf, 77, 4736), lp(bq, bsf, 1000, 4736), dg.Sm100Out.F32(d, 1000))
        ctx.sync()
        outs.append(d)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("block_n", [16, 32, 48, 96, 112, 128, 160, 208, 256])
@pytest.mark.parametrize("slabs", [1, 2])
def test_swapped_dense_every_width(ctx, ctas, block_n, slabs, monkeypatch):
    # every UMMA N the swapped family can issue (multiples of 16, of 32 for a CTA pair), one and two K slabs per stage,
    # with a problem that has fewer rows than the tile, exactly as many, and several tiles of rows
    if block_n % (16 * ctas) != 0:
        pytest.skip("tile width not issuable")
    monkeypatch.setenv("DG_SWAP", "1")
    monkeypatch.setenv("DG_BLOCK_N", str(block_n))
    monkeypatch.setenv("DG_CTAS", str(ctas))
    monkeypatch.setenv("DG_K_SLABS", str(slabs))
    try:
        cfg = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, block_n, 1000, 1152))
    except dg.DgError:
        pytest.skip("this tile does not fit three stages of two slabs")
    assert cfg.swap_ab and cfg.block_m == block_n and cfg.block_n == 128 * ctas and cfg.block_k == 128 * slabs
    for m in (max(1, block_n - 9), block_n, 2 * block_n + 5):
        run_dense(ctx, m, 1000, 1152, seed=block_n + m)
    run_dense(ctx, block_n, 712, 1152, out_kind=1, seed=block_n)


def test_dense_fp8_matches_scalar_reference_and_golden(ctx):
    # the committed fixture holds quantised inputs of the 128x256x512 case and the output of the scalar
    # restatement of ref_fp8_gemm_nt (f32); the GPU f32 output must agree with it
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "fp8_gemm_128x256x512.npz"))
    aq, bq, asf, bsf, want = z["a"], z["b"], z["a_sf_packed"], z["b_sf_packed"], z["out"]
    d = torch.zeros((128, 256), dtype=torch.float32, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, lp(aq, asf, 128, 512), lp(bq, bsf, 256, 512), dg.Sm100Out.F32(d, 256))
    ctx.sync()
    diff = O.calc_diff(to_f32(d), want)
    assert diff <= TIGHT_F32, diff


@pytest.mark.parametrize("gran", [32])
@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (200, 320, 1152)])
@both_families
def test_dense_fp8_gran32(ctx, m, n, k, gran, family, monkeypatch):
    pin_family(monkeypatch, family)
    run_dense(ctx, m, n, k, gran=gran)


@both_families
def test_dense_f32_and_alpha(ctx, family, monkeypatch):
    pin_family(monkeypatch, family)
    run_dense(ctx, 256, 384, 1024, out_kind=1)
    run_dense(ctx, 256, 384, 1024, out_kind=0, alpha=0.125)
    run_dense(ctx, 128, 96, 512, out_kind=1, alpha=3.0)


@pytest.mark.parametrize("ctas", [1, 2])
def test_tensor_core_duty_cycle_pauses_without_changing_results(ctx, ctas, monkeypatch):
    # Sm100Epilogue::tc_util (ops_sm100.rs:114-131; device side cuda/bf16_gemm_sm100.rs:358-371): below 100 the UMMA warp idles after
    # every k-block.  The product is bit-identical, and a 20 % duty cycle takes visibly longer than an unthrottled run.
    monkeypatch.setenv("DG_CTAS", str(ctas))
    m, n, k = 2048, 2048, 8192
    _, aq, asf = fp8_operand_1d(m, k, 91)
    _, bq, bsf = fp8_operand_1d(n, k, 92)
    a, b = lp(aq, asf, m, k), lp(bq, bsf, n, k)
    outs, times = [], []
    for util in (100, 20, 0):
        d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        for _ in range(2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.Bf16(d, n), dg.Sm100Epilogue(tc_util=util))
            e1.record()
            ctx.sync()
        outs.append(d)
        times.append(e0.elapsed_time(e1))
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert times[1] > 1.3 * times[0] and times[2] < 1.3 * times[0]     # 0 means "unset" = unthrottled


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("out_kind", [0, 1])
@both_families
def test_dense_accumulate_adds_into_the_output(ctx, out_kind, ctas, family, monkeypatch):
    pin_family(monkeypatch, family)
    # D += A.B^T (with_accumulation, ops_sm100.rs:150): tiles are added to what the output holds. f32 outputs add
    # in f32; bf16 outputs add the bf16-rounded tile to the bf16 addend and round once more, so the bound is
    # two bf16 roundings. Ragged M and N: rows and columns outside the problem must stay untouched.
    monkeypatch.setenv("DG_CTAS", str(ctas))
    m, n, k, ld = 300, 456, 1152, 512
    _, aq, asf = fp8_operand_1d(m, k, 77)
    _, bq, bsf = fp8_operand_1d(n, k, 78)
    want = O.lp_gemm_rows(aq, asf, 8, 128, 1, m, np.arange(m), bq, bsf, 8, 128, 1, n, np.arange(n), k)
    dtype = torch.bfloat16 if out_kind == 0 else torch.float32
    base = (torch.randn((m + 4, ld), device="cuda") * float(np.abs(want).mean())).to(dtype)
    d = base.clone()
    a, b = lp(aq, asf, m, k), lp(bq, bsf, n, k)
    out = dg.Sm100Out(out_kind, d, ld)
    dg.fp8_fp4_gemm_dev(ctx, a, b, out, dg.Sm100Epilogue(accumulate=True))
    ctx.sync()
    got, base_n = to_f32(d), to_f32(base)
    assert np.array_equal(got[m:], base_n[m:]) and np.array_equal(got[:, n:], base_n[:, n:])
    diff = O.calc_diff(got[:m, :n], want + base_n[:m, :n])
    assert diff <= (2 * TIGHT_BF16 if out_kind == 0 else TIGHT_F32), diff
    # a second call adds the product once more
    dg.fp8_fp4_gemm_dev(ctx, a, b, out, dg.Sm100Epilogue(accumulate=True))
    ctx.sync()
    diff = O.calc_diff(to_f32(d)[:m, :n], 2 * want + base_n[:m, :n])
    assert diff <= (3 * TIGHT_BF16 if out_kind == 0 else TIGHT_F32), diff


@pytest.mark.parametrize("m,family", [(128, None), (4096, None), (128, "1"), (77, "1")])
@pytest.mark.parametrize("n,k", [(2112, 7168), (24576, 1536), (7168, 16384), (4096, 7168), (7168, 2048)])
def test_dense_fp8_full_size_sampled(ctx, m, n, k, family, monkeypatch):
    # full benchmark shapes: operands quantised on the GPU (bit-exactness of that kernel is its own test),
    # outputs compared with the oracle on sampled rows / columns including every kind of tile edge; the skinny shapes also
    # through the swapped tile family with its K ranges summed inside a cluster (and with a row count off the 16-row grid)
    pin_family(monkeypatch, family)
    g = torch.Generator(device="cuda").manual_seed(1000 + n + k)
    a = torch.randn((m, k), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    b = torch.randn((n, k), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    aq, asf = dg.cast_bf16_to_fp8_sf_dev(ctx, a, k, m, k, 128)
    bq, bsf = dg.cast_bf16_to_fp8_sf_dev(ctx, b, k, n, k, 128)
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, dg.LpOperand(aq, asf, m, k, k), dg.LpOperand(bq, bsf, n, k, k), dg.Sm100Out.Bf16(d, n))
    ctx.sync()
    assert not torch.isnan(d).any()
    rows, cols = sample_indices(m, 24, n), sample_indices(n, 48, k)
    aqn, asfn = aq[torch.from_numpy(rows.astype(np.int64)).cuda()].cpu().numpy(), asf.cpu().numpy().view(np.uint32)
    bqn, bsfn = bq[torch.from_numpy(cols.astype(np.int64)).cuda()].cpu().numpy(), bsf.cpu().numpy().view(np.uint32)
    # dequantise only the sampled rows: gather their scale words into a compact layout first
    def compact(sf_words, total_rows, idx):
        cols_n = dg.sf_packed_cols(k, 128)
        w = sf_words.reshape(cols_n, dg.sf_aligned_rows(total_rows))[:, idx]
        out = np.zeros((cols_n, dg.sf_aligned_rows(len(idx))), np.uint32)
        out[:, :len(idx)] = w
        return out.reshape(-1)
    ar = np.arange(len(rows), dtype=np.uint32)
    br = np.arange(len(cols), dtype=np.uint32)
    want = O.lp_gemm_rows(aqn, compact(asfn, m, rows), 8, 128, 1, len(rows), ar, bqn, compact(bsfn, n, cols), 8, 128, 1, len(cols), br, k)
    got = to_f32(d[torch.from_numpy(rows.astype(np.int64)).cuda()][:, torch.from_numpy(cols.astype(np.int64)).cuda()])
    diff = O.calc_diff(got, want)
    assert diff <= TIGHT_BF16, diff


def contiguous_layout(group_sizes, alignment=128):
    starts, m_idx = [], []
    pos = 0
    for g, s in enumerate(group_sizes):
        starts.append(pos)
        m_idx += [g] * s
        pad = (-s) % alignment
        m_idx += [-1] * pad
        pos += s + pad
    return np.array(m_idx, np.int32), starts


@pytest.mark.parametrize("sizes,n,k", [
    ([128, 128, 128, 128], 256, 512),           # reference e2e shape (tests/e2e.rs:439-500)
    ([37, 128, 1, 64, 15, 100, 128, 3], 384, 1024),
    ([200, 0, 300, 0, 0, 129], 512, 768),       # empty experts, multi-tile experts
])
@pytest.mark.parametrize("ctas", [1, 2])
@both_families
def test_m_grouped_contiguous(ctx, sizes, n, k, ctas, family, monkeypatch):
    pin_family(monkeypatch, family)
    # with a CTA pair the 256-row tile of a group's tail reaches into the next group's rows: those rows are
    # computed but must never be stored
    monkeypatch.setenv("DG_CTAS", str(ctas))
    groups = len(sizes)
    m_idx, starts = contiguous_layout(sizes)
    m_total = len(m_idx)
    _, aq, asf = fp8_operand_1d(m_total, k, 11)
    _, bq, bsf, sfb_tiles = fp8_operand_2d(groups * n, k, 12, groups)
    d = torch.full((m_total, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    a_op = lp(aq, asf, m_total, k)
    b_op = lp(bq, bsf, groups * n, k)
    dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a_op, dev(m_idx), b_op, dg.Sm100Out.Bf16(d, n), groups)
    ctx.sync()
    dn = to_f32(d)
    valid = np.nonzero(m_idx >= 0)[0]
    assert not np.isnan(dn[valid]).any()
    # rows of empty 128-row slots (whole slots of padding) are never touched
    for slot in range(m_total // 128):
        if np.all(m_idx[slot * 128:(slot + 1) * 128] < 0):
            assert np.isnan(dn[slot * 128:(slot + 1) * 128]).all()
    # the scalar restatement of ref_m_grouped_fp8_gemm_nt_contiguous on every valid row (per-expert tile scales)
    kb = k // 128
    sfa = np.stack([O.exps_to_f32(((asf.reshape(-1, dg.sf_aligned_rows(m_total))[c // 4] >> ((c % 4) * 8)) & 0xFF).astype(np.uint8))
                    for c in range(kb)], axis=1)[:m_total]
    want = O.ref_m_grouped_contiguous(aq, sfa, m_idx, bq, sfb_tiles.reshape(-1), n, per_group_sfb=True, threads=8)
    diff = O.calc_diff(dn[valid], want[valid])
    assert diff <= TIGHT_BF16, diff
    # the prebuilt-table entry point gives the same bytes
    d2 = torch.zeros_like(d)
    ends = dg.psum_from_m_indices_dev(ctx, dev(m_idx), groups)
    dg.m_grouped_fp8_fp4_gemm_contiguous_ends_dev(ctx, a_op, ends, b_op, dg.Sm100Out.Bf16(d2, n), groups)
    ctx.sync()
    assert torch.equal(d[torch.from_numpy(valid).cuda()], d2[torch.from_numpy(valid).cuda()])


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("out_kind", [0, 1])
@pytest.mark.parametrize("alignment", [64, 32, 16, 256])
@both_families
def test_m_grouped_contiguous_other_alignments(ctx, alignment, out_kind, ctas, family, monkeypatch):
    pin_family(monkeypatch, family)
    # set_mk_alignment_for_contiguous_layout (types.rs:195): groups start at multiples of 16..256 rows.  Tiles stay 128 / 256
    # rows tall, so a group's last tile runs into the following groups' rows: those must come out as their own group computes
    # them, never as this tile computes them (several rounds: a wrong store would race with the right one)
    monkeypatch.setenv("DG_CTAS", str(ctas))
    sizes, n, k = [37, 5, 0, 130, 64, 1, 17, 200, 16, 3], 328, 640
    groups = len(sizes)
    m_idx, starts = contiguous_layout(sizes, alignment)
    m_total = len(m_idx)
    _, aq, asf = fp8_operand_1d(m_total, k, 61)
    _, bq, bsf = fp8_operand_1d(groups * n, k, 62, 128, groups)       # per-row scales: n need not be a multiple of 128
    valid = np.nonzero(m_idx >= 0)[0]
    want = np.zeros((m_total, n), np.float32)
    for g in range(groups):
        rows = valid[m_idx[valid] == g].astype(np.uint32)
        if rows.size:
            want[rows.astype(np.int64)] = O.lp_gemm_rows(aq, asf, 8, 128, 1, m_total, rows, bq, bsf, 8, 128, groups, n,
                                                         np.arange(g * n, (g + 1) * n, dtype=np.uint32), k)
    ld = 336
    dg.set_mk_alignment_for_contiguous_layout(alignment)
    try:
        assert dg.get_mk_alignment_for_contiguous_layout() == alignment
        for _ in range(4):
            d = torch.full((m_total, ld), float("nan"), dtype=torch.bfloat16 if out_kind == 0 else torch.float32, device="cuda")
            dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, lp(aq, asf, m_total, k), dev(m_idx), lp(bq, bsf, groups * n, k),
                                                     dg.Sm100Out(out_kind, d, ld), groups)
            ctx.sync()
            dn = to_f32(d)
            assert not np.isnan(dn[valid][:, :n]).any()
            assert np.isnan(dn[:, n:]).all()                      # columns past n are never written
            diff = O.calc_diff(dn[valid][:, :n], want[valid])
            assert diff <= (TIGHT_BF16 if out_kind == 0 else TIGHT_F32), diff
            # row-wise: a row taken from the wrong group would show up as a large per-row error
            err = np.abs(dn[valid][:, :n] - want[valid]).max(axis=1)
            assert (err <= 0.02 * np.abs(want[valid]).max()).all()
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("masked,m_max,n,k", [
    ([37, 128, 1, 64, 15, 100, 128, 3], 128, 256, 512),   # reference fixture (tests/e2e.rs:131,566)
    ([0, 256, 17, 129, 255, 16, 0, 1], 256, 384, 1024),
    ([100, 7], 100, 128, 256),                               # m_max not a multiple of the tile
])
@both_families
def test_m_grouped_masked(ctx, masked, m_max, n, k, ctas, family, monkeypatch):
    pin_family(monkeypatch, family)
    monkeypatch.setenv("DG_CTAS", str(ctas))
    groups = len(masked)
    masked_m = np.array(masked, np.int32)
    _, aq, asf = fp8_operand_1d(groups * m_max, k, 21, 128, groups)
    _, bq, bsf, sfb_tiles = fp8_operand_2d(groups * n, k, 22, groups)
    d = torch.full((groups * m_max, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, lp(aq, asf, m_max, k), dev(masked_m), lp(bq, bsf, groups * n, k),
                                         dg.Sm100Out.Bf16(d, n), groups, max(1, int(masked_m.mean())))
    ctx.sync()
    dn = to_f32(d)
    kb = k // 128
    stride = dg.sf_aligned_rows(m_max)
    cols = dg.sf_packed_cols(k, 128)
    sfa = np.zeros((groups * m_max, kb), np.float32)
    w = asf.reshape(groups, cols, stride)
    for c in range(kb):
        sfa[:, c] = O.exps_to_f32(((w[:, c // 4, :m_max] >> ((c % 4) * 8)) & 0xFF).astype(np.uint8)).reshape(-1)
    want = O.ref_m_grouped_masked(aq, sfa, masked_m, m_max, bq, sfb_tiles.reshape(-1), n, per_group_sfb=True, threads=8)
    valid = np.concatenate([np.arange(g * m_max, g * m_max + masked[g]) for g in range(groups)]).astype(np.int64)
    assert not np.isnan(dn[valid]).any()
    diff = O.calc_diff(dn[valid], want[valid])
    assert diff <= TIGHT_BF16, diff
    # rows of a group whose tiles were never scheduled keep the caller's contents (no stray writes)
    for g in range(groups):
        # first family: whole 128- or 256-row tiles; swapped family: exactly the valid rows
        first_untouched = g * m_max + (masked[g] if family == "1" else ((masked[g] + 128 * ctas - 1) // (128 * ctas)) * 128 * ctas)
        if first_untouched < (g + 1) * m_max:
            assert np.isnan(dn[first_untouched:(g + 1) * m_max]).all()


def test_bmm_and_fp8_requant_epilogue(ctx):
    groups, m, n, k = 3, 160, 256, 512
    _, aq, asf = fp8_operand_1d(groups * m, k, 31, 128, groups)
    _, bq, bsf = fp8_operand_1d(groups * n, k, 32, 128, groups)
    a_op, b_op = lp(aq, asf, m, k), lp(bq, bsf, n, k)
    d32 = torch.zeros((groups * m, n), dtype=torch.float32, device="cuda")
    dg.fp8_fp4_bmm_dev(ctx, a_op, b_op, dg.Sm100Out.F32(d32, n), groups)
    ctx.sync()
    dn = to_f32(d32)
    for g in range(groups):
        rows = np.arange(g * m, (g + 1) * m, dtype=np.uint32)
        colsb = np.arange(g * n, (g + 1) * n, dtype=np.uint32)
        want = O.lp_gemm_rows(aq, asf, 8, 128, groups, m, rows, bq, bsf, 8, 128, groups, n, colsb, k)
        assert O.calc_diff(dn[g * m:(g + 1) * m], want) <= TIGHT_F32
    # FP8 output: the same accumulators, rounded to bf16, scaled per 32 columns, cast to e4m3.  The CPU
    # epilogue applied to the GPU's own f32 output must give the identical bytes and scale words.
    d8 = torch.zeros((groups * m, n), dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(groups * (n // 128) * dg.sf_aligned_rows(m), dtype=torch.int32, device="cuda")
    dg.fp8_fp4_bmm_dev(ctx, a_op, b_op, dg.Sm100Out.Fp8(d8, n, sfd), groups)
    ctx.sync()
    want8 = np.zeros((groups * m, n), np.uint8)
    want_sfd = np.zeros(sfd.numel(), np.uint32)
    for g in range(groups):
        O.requant_fp8(dn[g * m:(g + 1) * m], g, dg.sf_aligned_rows(m), want8[g * m:(g + 1) * m], want_sfd)
    assert np.array_equal(d8.cpu().numpy(), want8)
    assert np.array_equal(sfd.cpu().numpy().view(np.uint32), want_sfd)


def test_masked_fp8_requant_feeds_next_gemm(ctx):
    # decode-style: masked GEMM with FP8 output whose D/SFD are directly the next masked GEMM's operand (gran 32)
    groups, m_max, n, k = 4, 128, 512, 1024
    masked_m = np.array([128, 5, 0, 77], np.int32)
    _, aq, asf = fp8_operand_1d(groups * m_max, k, 41, 128, groups)
    _, bq, bsf, _ = fp8_operand_2d(groups * n, k, 42, groups)
    a_op, b_op = lp(aq, asf, m_max, k), lp(bq, bsf, groups * n, k)
    d32 = torch.zeros((groups * m_max, n), dtype=torch.float32, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a_op, dev(masked_m), b_op, dg.Sm100Out.F32(d32, n), groups, 64)
    d8 = torch.zeros((groups * m_max, n), dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(groups * (n // 128) * m_max, dtype=torch.int32, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a_op, dev(masked_m), b_op, dg.Sm100Out.Fp8(d8, n, sfd), groups, 64)
    ctx.sync()
    dn = to_f32(d32)
    got8, got_sfd = d8.cpu().numpy(), sfd.cpu().numpy().view(np.uint32).reshape(groups, n // 128, m_max)
    for g in range(groups):
        v = int(masked_m[g])
        if v == 0:
            continue
        want8 = np.zeros((v, n), np.uint8)
        want_sfd = np.zeros(groups * (n // 128) * m_max, np.uint32)
        O.requant_fp8(dn[g * m_max:g * m_max + v], g, m_max, want8, want_sfd)
        assert np.array_equal(got8[g * m_max:g * m_max + v], want8)
        assert np.array_equal(got_sfd[g, :, :v], want_sfd.reshape(groups, n // 128, m_max)[g, :, :v])
    # second GEMM consumes (d8, sfd) as an e4m3 operand with per-32 scales
    n2 = 256
    _, wq, wsf = fp8_operand_1d(groups * n2, n, 43, 32, groups)
    d2 = torch.zeros((groups * m_max, n2), dtype=torch.bfloat16, device="cuda")
    a2 = dg.LpOperand(d8, sfd, m_max, n, n, 8, 32)
    dg.m_grouped_fp8_fp4_gemm_masked_dev(ctx, a2, dev(masked_m), lp(wq, wsf, groups * n2, n, 8, 32), dg.Sm100Out.Bf16(d2, n2), groups, 64)
    ctx.sync()
    d2n = to_f32(d2)
    for g in range(groups):
        v = int(masked_m[g])
        if v == 0:
            continue
        rows = np.arange(g * m_max, g * m_max + v, dtype=np.uint32)
        colsb = np.arange(g * n2, (g + 1) * n2, dtype=np.uint32)
        want = O.lp_gemm_rows(got8, sfd.cpu().numpy().view(np.uint32), 8, 32, groups, m_max, rows, wq, wsf, 8, 32, groups, n2, colsb, n)
        assert O.calc_diff(d2n[g * m_max:g * m_max + v], want) <= TIGHT_BF16


@pytest.mark.parametrize("m,n,k,rule", [(128, 256, 512, 0), (256, 512, 768, 1), (8, 8, 128, 0), (200, 192, 1280, 1)])
@both_families
def test_dense_mxfp4(ctx, m, n, k, rule, family, monkeypatch):
    pin_family(monkeypatch, family)
    # reference e2e MXFP4 shapes (tests/e2e.rs:266-350) against mxfp4_gemm_reference (reference.rs:293-329)
    _, aq, asf = fp4_operand(m, k, 51, 1, rule)
    _, bq, bsf = fp4_operand(n, k, 52, 1, rule)
    d = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, dg.LpOperand(dev(aq), dev(asf), m, k, k, 4, 32), dg.LpOperand(dev(bq), dev(bsf), n, k, k, 4, 32),
                        dg.Sm100Out.F32(d, n))
    ctx.sync()
    want = O.mxfp4_gemm_reference(aq, asf, m, bq, bsf, n, k, threads=8)
    assert O.calc_diff(to_f32(d), want) <= TIGHT_F32


@pytest.mark.parametrize("a_bits,b_bits,gran8", [(8, 4, 128), (8, 4, 32), (4, 8, 128)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (300, 448, 1408)])
@both_families
def test_dense_mixed_fp8_fp4(ctx, m, n, k, a_bits, b_bits, gran8, family, monkeypatch):
    pin_family(monkeypatch, family)
    # e4m3 (per-128 or per-32 scales) against packed e2m1 (per-32 scales) on the byte-operand tensor-core kind
    def operand(rows, bits, seed):
        if bits == 8:
            _, q, sf = fp8_operand_1d(rows, k, seed, gran8)
            return q, sf, gran8
        _, q, sf = fp4_operand(rows, k, seed, 1, 1)
        return q, sf, 32
    aq, asf, ga = operand(m, a_bits, 71)
    bq, bsf, gb = operand(n, b_bits, 72)
    d = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, dg.LpOperand(dev(aq), dev(asf), m, k, k, a_bits, ga), dg.LpOperand(dev(bq), dev(bsf), n, k, k, b_bits, gb),
                        dg.Sm100Out.F32(d, n))
    ctx.sync()
    rows, cols = np.arange(m, dtype=np.uint32), np.arange(n, dtype=np.uint32)
    want = O.lp_gemm_rows(aq, asf, a_bits, ga, 1, m, rows, bq, bsf, b_bits, gb, 1, n, cols, k)
    assert O.calc_diff(to_f32(d), want) <= TIGHT_F32


def fused_activation_reference(h):
    """bf16 gate|up GEMM output (torch, (rows, 2n)) -> what the fused epilogue must write: the oracle's silu * up on those
    bf16 bits, then its e4m3 quantiser with one scale per 32 columns."""
    h_bits = h.view(torch.int16).cpu().numpy().view(np.uint16)
    n = h_bits.shape[1] // 2
    return O.cast_bf16_to_fp8_sf(O.silu_mul_bf16(h_bits), n, 32)


@pytest.mark.parametrize("block_n", [0, 64, 128, 192, 256])
def test_fused_gate_up_activation_dense(ctx, block_n, monkeypatch):
    # out kind 3: B = [gate rows; up rows]; the GEMM writes e4m3(silu(gate) * up) + per-32 scales.  Must equal, bit for bit,
    # the unfused sequence on the same operands: bf16 GEMM output -> silu * up -> quantise (the oracle's two steps)
    m, n, k = 300, 384, 1152
    _, aq, asf = fp8_operand_1d(m, k, 71)
    _, bq, bsf = fp8_operand_1d(2 * n, k, 72)
    a, b = lp(aq, asf, m, k), lp(bq, bsf, 2 * n, k)
    h = torch.zeros((m, 2 * n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.Bf16(h, 2 * n))
    ctx.sync()
    want_q, want_sf = fused_activation_reference(h)
    if block_n:
        monkeypatch.setenv("DG_BLOCK_N", str(block_n))
    q = torch.full((m, n), 0xAB, dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(dg.sf_packed_cols(n, 32) * dg.sf_aligned_rows(m), dtype=torch.int32, device="cuda")
    dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.SwiGluFp8(q, n, sfd))
    ctx.sync()
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(sfd.cpu().numpy().view(np.uint32), want_sf)


@pytest.mark.parametrize("alignment", [128, 32])
def test_fused_gate_up_activation_grouped_feeds_the_down_gemm(ctx, alignment):
    sizes, n, k, n2 = [200, 0, 300, 129, 31], 256, 640, 320
    groups = len(sizes)
    m_idx, _ = contiguous_layout(sizes, alignment)
    m_total = len(m_idx)
    _, aq, asf = fp8_operand_1d(m_total, k, 73)
    _, bq, bsf = fp8_operand_1d(groups * 2 * n, k, 74, 128, groups)
    _, wq, wsf = fp8_operand_1d(groups * n2, n, 75, 128, groups)
    a, b = lp(aq, asf, m_total, k), lp(bq, bsf, groups * 2 * n, k)
    valid = np.nonzero(m_idx >= 0)[0]
    dg.set_mk_alignment_for_contiguous_layout(alignment)
    try:
        h = torch.zeros((m_total, 2 * n), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a, dev(m_idx), b, dg.Sm100Out.Bf16(h, 2 * n), groups)
        ctx.sync()
        want_q, want_sf = fused_activation_reference(h)
        q = torch.zeros((m_total, n), dtype=torch.uint8, device="cuda")
        sfd = torch.zeros(dg.sf_packed_cols(n, 32) * dg.sf_aligned_rows(m_total), dtype=torch.int32, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a, dev(m_idx), b, dg.Sm100Out.SwiGluFp8(q, n, sfd), groups)
        ctx.sync()
        assert np.array_equal(q.cpu().numpy()[valid], want_q[valid])
        got_sf = sfd.cpu().numpy().view(np.uint32).reshape(-1, dg.sf_aligned_rows(m_total))
        assert np.array_equal(got_sf[:, valid], want_sf.reshape(got_sf.shape)[:, valid])
        # the activation is the down projection's operand as it is (per-32 scales)
        y = torch.zeros((m_total, n2), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(q, sfd, m_total, n, n, 8, 32), dev(m_idx), lp(wq, wsf, groups * n2, n),
                                                 dg.Sm100Out.Bf16(y, n2), groups)
        ctx.sync()
        yn = to_f32(y)
        q_np, sf_np = q.cpu().numpy(), sfd.cpu().numpy().view(np.uint32)
        for g in range(groups):
            rows = valid[m_idx[valid] == g].astype(np.uint32)
            if rows.size:
                want = O.lp_gemm_rows(q_np, sf_np, 8, 32, 1, m_total, rows, wq, wsf, 8, 128, groups, n2, np.arange(g * n2, (g + 1) * n2, dtype=np.uint32), n)
                assert O.calc_diff(yn[rows.astype(np.int64)], want) <= TIGHT_BF16
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)


def test_fp4_convenience_entry_points(ctx):
    # ops_sm100.rs:1646 / :1693: bf16 host tensors -> quantise -> MXF4 GEMM -> bf16 host result; equals the oracle's
    # quantiser followed by its f64 MXFP4 reference, to bf16 rounding
    m, n, k = 96, 160, 640
    a, b = randn_bf16(m, k, 91), randn_bf16(n, k, 92)
    out = dg.fp4_gemm_nt_native(ctx, torch.from_numpy(a.view(np.int16)).view(torch.bfloat16), torch.from_numpy(b.view(np.int16)).view(torch.bfloat16), m, n, k)
    aq, asf = O.cast_bf16_to_fp4_packed_sf(a, k, 1, 0)
    bq, bsf = O.cast_bf16_to_fp4_packed_sf(b, k, 1, 0)
    want = O.mxfp4_gemm_reference(aq, asf, m, bq, bsf, n, k, threads=O.max_threads())
    assert O.calc_diff(to_f32(out), want) <= TIGHT_BF16


@both_families
def test_m_grouped_mxfp4(ctx, family, monkeypatch):
    pin_family(monkeypatch, family)
    groups, gm, n, k = 4, 128, 256, 512     # tests/e2e.rs:439-500
    _, aq, asf = fp4_operand(groups * gm, k, 61, 1, 1)
    _, bq, bsf = fp4_operand(groups * n, k, 62, groups, 1)
    m_idx = np.repeat(np.arange(groups, dtype=np.int32), gm)
    d = torch.zeros((groups * gm, n), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, dg.LpOperand(dev(aq), dev(asf), groups * gm, k, k, 4, 32), dev(m_idx),
                                             dg.LpOperand(dev(bq), dev(bsf), groups * n, k, k, 4, 32), dg.Sm100Out.Bf16(d, n), groups)
    ctx.sync()
    dn = to_f32(d)
    for g in range(groups):
        rows = np.arange(g * gm, (g + 1) * gm, dtype=np.uint32)
        colsb = np.arange(g * n, (g + 1) * n, dtype=np.uint32)
        want = O.lp_gemm_rows(aq, asf, 4, 32, 1, groups * gm, rows, bq, bsf, 4, 32, groups, n, colsb, k)
        assert O.calc_diff(dn[g * gm:(g + 1) * gm], want) <= TIGHT_BF16


def test_argument_errors(ctx):
    _, aq, asf = fp8_operand_1d(128, 512, 1)
    _, bq, bsf = fp8_operand_1d(128, 512, 2)
    a, b = lp(aq, asf, 128, 512), lp(bq, bsf, 128, 512)
    d = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    out = dg.Sm100Out.Bf16(d, 128)

    def kind(fn):
        with pytest.raises(dg.DgError) as e:
            fn()
        return e.value.kind

    d8 = torch.zeros((128, 128), dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(128, dtype=torch.int32, device="cuda")
    assert kind(lambda: dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.Fp8(d8, 128, sfd))) == "Shape"      # ops_sm100.rs:727
    assert kind(lambda: dg.fp8_fp4_gemm_dev(ctx, a, b, out, dg.Sm100Epilogue(alpha=2.0, accumulate=True))) == "Shape"  # :150
    bad = dg.LpOperand(a.data, a.sf, 128, 512, 512, 8, 64)
    assert kind(lambda: dg.fp8_fp4_gemm_dev(ctx, bad, b, out)) == "Shape"                               # :52
    bad = dg.LpOperand(a.data, a.sf, 256, 512, 512)
    assert kind(lambda: dg.fp8_fp4_gemm_dev(ctx, bad, b, dg.Sm100Out.Bf16(torch.zeros((256, 128), dtype=torch.bfloat16, device="cuda"), 128))) == "Shape"  # :71
    bad = dg.LpOperand(a.data, a.sf, 128, 384, 512)
    assert kind(lambda: dg.fp8_fp4_gemm_dev(ctx, bad, b, out)) == "Shape"                               # k mismatch
    assert kind(lambda: dg.fp8_fp4_gemm_dev(ctx, a, b, dg.Sm100Out.Bf16(d, 64))) == "Shape"             # ld < n
    assert kind(lambda: dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a, dev(np.zeros(128, np.int32)), b, out, 3)) == "Shape"
    with pytest.raises(dg.DgError):
        dg.set_mk_alignment_for_contiguous_layout(48)          # not a power of two (types.rs:196)
    ctx.sync()


def test_bounded_wait_reports_timeout_and_context_survives():
    # a wait nothing satisfies must end by itself, surface as a Timeout error on the host and leave the context usable
    c = dg.DgContext(0)
    dg.debug_expire_wait(c, 1000)
    with pytest.raises(dg.DgError) as e:
        c.sync()
    assert e.value.kind == "Timeout" and "0x700" in str(e.value)
    c.sync()                                  # the record is cleared by the report
    run_dense(c, 128, 256, 512)               # and the same context still computes correctly
    c.close()
