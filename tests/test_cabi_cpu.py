"""CPU-side checks of the C-ABI library: it loads, exports everything include/dgb200.h declares,
and its pure-host entry points (size helpers, mk alignment knob, tile heuristics, argument
errors) behave like the reference's (deepgemm/tests/unit.rs:5-70,160-195; types.rs:195-223)."""
import ctypes
import os
import re

import pytest

import deepgemm_rust_b200 as dg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "dgb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dg_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(os.path.join(ROOT, "deepgemm_rust_b200", "libdgb200.so"))
    names = declared_functions()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), name


def test_size_helpers_match_reference_formulas():
    # ops_sm100.rs:1091-1098, types.rs:223
    assert dg.sf_packed_cols(7168, 128) == 14 and dg.sf_packed_cols(512, 32) == 4 and dg.sf_packed_cols(640, 128) == 2
    assert dg.sf_aligned_rows(37) == 40 and dg.sf_aligned_rows(4096) == 4096
    assert dg._sf_words(4096, 7168, 128, 1) == 14 * 4096
    assert dg._sf_words(4 * 6, 256, 32, 4) == 2 * 4 * 8


def test_mk_alignment_knob():
    # types.rs:195-219
    assert dg.get_mk_alignment_for_contiguous_layout() == 128
    dg.set_mk_alignment_for_contiguous_layout(256)
    assert dg.get_mk_alignment_for_contiguous_layout() == 256
    assert dg.get_theoretical_mk_alignment_for_contiguous_layout(10) == 256
    assert dg.get_theoretical_mk_alignment_for_contiguous_layout(9) == 128
    for bad in (0, 8, 96, 512):
        with pytest.raises(dg.DgError) as e:
            dg.set_mk_alignment_for_contiguous_layout(bad)
        assert e.value.kind == "Shape"
    dg.set_mk_alignment_for_contiguous_layout(128)


def test_heuristics_block_k_and_budgets():
    # tests/unit.rs:5-41: MXF4 -> block K 256, FP8 -> 128, a deep pipeline, shared memory within capacity
    d4 = dg.Sm100Desc(dg.GemmType.Normal, 4096, 7168, 7168, a_bits=4, b_bits=4, gran_a=32, gran_b=32)
    c4 = dg.best_config(d4)
    # block_k counts the K elements of one pipeline stage: one or two 128-byte slabs (256 e2m1 / 128 e4m3 each)
    assert c4.block_k in (256, 512) and c4.num_stages >= 2 and c4.smem_size <= dg.SM100_SMEM_CAPACITY
    d8 = dg.Sm100Desc(dg.GemmType.Normal, 4096, 7168, 7168)
    c8 = dg.best_config(d8)
    assert c8.block_k in (128, 256) and c8.num_stages >= 2 and c8.smem_size <= dg.SM100_SMEM_CAPACITY
    assert c8.block_m == 128 * c8.cluster_m and c8.cluster_m in (1, 2) and c8.block_n % 16 == 0 and c8.block_n <= 256
    # TMEM budget: accumulators (x stages) plus scale columns within 512 columns
    for c, sf_cols in ((c8, 4 + 4 * ((c8.block_n + 127) // 128)), (c4, 8 + 8 * ((c4.block_n + 127) // 128))):
        assert c.num_accum_stages * c.block_n + sf_cols <= 512


def test_heuristics_grouped_and_output_kinds():
    # tests/unit.rs:43-70: the m-grouped layouts tile M by the 128-row alignment
    d = dg.Sm100Desc(dg.GemmType.MGroupedContiguous, 8192, 7168, 7168, num_groups=256)
    c = dg.best_config(d)
    assert c.block_m == 128 and c.cluster_m == 1 and c.smem_size <= dg.SM100_SMEM_CAPACITY
    # tests/unit.rs:160-195: with the 256-row alignment the tile may follow the knob (a CTA pair per 256 rows)
    dg.set_mk_alignment_for_contiguous_layout(256)
    try:
        c = dg.best_config(d)
        assert c.block_m in (128, 256) and c.block_m == 128 * c.cluster_m and c.smem_size <= dg.SM100_SMEM_CAPACITY
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)
    # FP8 output stores 128-column rows, so BLOCK_N is a multiple of 128
    c = dg.best_config(dg.Sm100Desc(dg.GemmType.MGroupedMasked, 256, 4096, 7168, num_groups=32, expected_m=128, cd_dtype=2))
    assert c.block_n % 128 == 0
    # skinny problems get narrow tiles so more SMs have work
    c = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 128, 2112, 7168))
    assert c.block_n <= 128
    # ... and a long K with few tiles is cut into K ranges; grouped and FP8-output GEMMs never are
    c = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 128, 7168, 16384))
    assert c.num_splits > 1 and c.num_tiles * c.num_splits >= 100
    assert dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 4096, 7168, 16384)).num_splits == 1
    assert dg.best_config(dg.Sm100Desc(dg.GemmType.MGroupedMasked, 128, 4096, 16384, num_groups=2, expected_m=64)).num_splits == 1
    assert dg.best_config(dg.Sm100Desc(dg.GemmType.Batched, 128, 1024, 16384, num_groups=2, cd_dtype=2)).num_splits == 1
    # e4m3 x e2m1 runs on the byte-operand kind: 128 K elements per 128-byte slab like e4m3 x e4m3
    c = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 4096, 7168, 7168, a_bits=8, b_bits=4, gran_a=128, gran_b=32))
    assert c.block_k in (128, 256)
    with pytest.raises(dg.DgError):
        dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 128, 128, 128, a_bits=6, b_bits=4))
    # MN-major operands (heuristics_sm100.rs:72-73): an MN-major B tile is whole 128-row boxes per CTA; FP4 must be K-major
    for m, n, k in ((4096, 7168, 7168), (128, 2112, 7168), (300, 456, 1152)):
        c = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, m, n, k, major_b_mn=True))
        assert (c.block_n // c.cluster_m) % 128 == 0 and not c.swap_ab
        c = dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, m, n, k, major_a_mn=True))
        assert c.block_m == 128 * c.cluster_m and not c.swap_ab
    with pytest.raises(dg.DgError):
        dg.best_config(dg.Sm100Desc(dg.GemmType.Normal, 128, 128, 256, a_bits=8, b_bits=4, gran_b=32, major_b_mn=True))


def test_no_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(dg.DgError) as e:
        dg.DgContext(0, own_stream=True)
    assert e.value.kind == "Driver" and "no CPU path" in str(e.value)
    with pytest.raises(dg.DgError):
        dg.DgContext(0)
