"""numpy front end of the CPU oracle (oracle/dg_oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by __graft_entry__.smoke() and
by bench.py's CPU-baseline legs; the product package never imports it.

Each wrapper names the reference function it restates (paths are relative to
the reference crate).  Where the reference has no CPU definition the docstring
says "parity unpinned".
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = C.CDLL(_build.build())

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def _sig(name, res, *args):
    f = getattr(_lib, name)
    f.restype = res
    f.argtypes = list(args)
    return f


_e4m3_to_f32 = _sig("dgo_e4m3_to_f32", C.c_float, C.c_uint8)
_f32_to_e4m3 = _sig("dgo_f32_to_e4m3", C.c_uint8, C.c_float)
_f32_to_e4m3_fast = _sig("dgo_f32_to_e4m3_fast", C.c_uint8, C.c_float)
_f32_to_bf16 = _sig("dgo_f32_to_bf16", C.c_uint16, C.c_float)
_bf16_to_f32 = _sig("dgo_bf16_to_f32", C.c_float, C.c_uint16)
_e2m1_to_f32 = _sig("dgo_e2m1_to_f32", C.c_float, C.c_uint8)
_encode_e2m1 = _sig("dgo_encode_e2m1", C.c_uint8, C.c_float)
_f32_to_ue8m0 = _sig("dgo_f32_to_ue8m0", C.c_uint8, C.c_float)
_ue8m0_to_f32 = _sig("dgo_ue8m0_to_f32", C.c_float, C.c_uint8)
_sf_exp_e2m1 = _sig("dgo_sf_exp_e2m1", C.c_uint32, C.c_float, C.c_int)
_sf_exp_e4m3 = _sig("dgo_sf_exp_e4m3", C.c_uint32, C.c_float)
_sf_exp_e4m3_bf16 = _sig("dgo_sf_exp_e4m3_bf16", C.c_uint32, C.c_uint16)
_sf_words = _sig("dgo_sf_words", C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32)
_cast_fp4 = _sig("dgo_cast_bf16_to_fp4_packed_sf", None, _u16p, C.c_uint32, C.c_uint32, C.c_uint32,
                 C.c_uint32, C.c_int, _u8p, _u32p)
_cast_fp8 = _sig("dgo_cast_bf16_to_fp8_sf", None, _u16p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                 C.c_uint32, _u8p, _u32p)
_quant_blocks = _sig("dgo_quantize_fp8_ue8m0_blocks", None, _u16p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _u8p, _u8p)
_quant_f32scale = _sig("dgo_quantize_fp8_f32scale", None, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _u8p, _f32p)
_tsf1d = _sig("dgo_transform_sf1d_packed", None, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
              C.c_uint32, _u32p)
_tsf2d = _sig("dgo_transform_sf2d_packed", None, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _u32p)
_tsf_f32 = _sig("dgo_transform_sf_f32", None, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _f32p)
_tsf_t = _sig("dgo_transform_sf_t_packed", None, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _u32p)
_psum = _sig("dgo_psum_from_m_indices", None, _i32p, C.c_uint32, C.c_uint32, _u32p)
_ref_gemm = _sig("dgo_ref_fp8_gemm_nt", None, _u8p, _f32p, C.c_uint32, _u8p, _f32p, C.c_uint32, C.c_uint32,
                 _f32p, C.c_int)
_ref_contig = _sig("dgo_ref_m_grouped_contiguous", None, _u8p, _f32p, _i32p, C.c_uint32, _u8p, _f32p,
                   C.c_size_t, C.c_uint32, C.c_uint32, _f32p, C.c_int)
_ref_masked = _sig("dgo_ref_m_grouped_masked", None, _u8p, _f32p, _i32p, C.c_uint32, C.c_uint32, _u8p, _f32p,
                   C.c_size_t, C.c_uint32, C.c_uint32, _f32p, C.c_int)
_mxfp4_ref = _sig("dgo_mxfp4_gemm_reference", None, _u8p, _u32p, C.c_uint32, _u8p, _u32p, C.c_uint32,
                  C.c_uint32, _f32p, C.c_int)
_dequant = _sig("dgo_dequant_rows", None, _u8p, _u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                C.c_uint32, _u32p, C.c_uint32, _f32p)
_requant = _sig("dgo_requant_fp8", None, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _u8p, _u32p)
_moe_combine = _sig("dgo_moe_combine", None, _u16p, C.c_size_t, _i32p, _f32p, C.c_uint32, C.c_uint32, C.c_uint32, _u16p)
_calc_diff = _sig("dgo_calc_diff", C.c_double, _f32p, _f32p, C.c_size_t)
_max_threads = _sig("dgo_max_threads", C.c_int)

SF_RULE_REFERENCE_CPU = 0
SF_RULE_RANGE_FIT = 1


# ---- scalar codecs (reference.rs:5-80, 215-262) -------------------------------
def e4m3_to_f32(code):
    return float(_e4m3_to_f32(int(code) & 0xFF))


def f32_to_e4m3(v):
    return int(_f32_to_e4m3(float(np.float32(v))))


def f32_to_e4m3_fast(v):
    return int(_f32_to_e4m3_fast(float(np.float32(v))))


def f32_to_bf16(v):
    return int(_f32_to_bf16(float(np.float32(v))))


def bf16_to_f32(b):
    return float(_bf16_to_f32(int(b) & 0xFFFF))


def e2m1_to_f32(code):
    return float(_e2m1_to_f32(int(code) & 0xF))


def encode_e2m1(v):
    return int(_encode_e2m1(float(np.float32(v))))


def f32_to_ue8m0(v):
    return int(_f32_to_ue8m0(float(np.float32(v))))


def ue8m0_to_f32(e):
    return float(_ue8m0_to_f32(int(e) & 0xFF))


def sf_exp_e2m1(amax, rule):
    return int(_sf_exp_e2m1(float(np.float32(amax)), int(rule)))


def sf_exp_e4m3(amax):
    return int(_sf_exp_e4m3(float(np.float32(amax))))


def sf_exp_e4m3_bf16(bits):
    return int(_sf_exp_e4m3_bf16(int(bits) & 0xFFFF))


def max_threads():
    return int(_max_threads())


# ---- array helpers -------------------------------------------------------------
def bf16_bits(x):
    """f32 array -> bf16 bit patterns with reference.rs:67-76 rounding."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    lsb = (bits & 0xFFFF).astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)
    return ((bits >> 16) + (lsb > 0xFFFF)).astype(np.uint16)


def bf16_to_f32_array(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def sf_words(rows, k, gran, groups=1):
    return int(_sf_words(rows, k, gran, max(groups, 1)))


def sf_packed_cols(k, gran):
    return (k + 4 * gran - 1) // (4 * gran)


def sf_aligned_rows(rows):
    return (rows + 3) // 4 * 4


# ---- quantizers ------------------------------------------------------------------
def cast_bf16_to_fp4_packed_sf(src_bits, k, groups=1, rule=SF_RULE_REFERENCE_CPU):
    """reference.rs:266-285 over a (rows, k) bf16-bit matrix; packed layout of tests/e2e.rs:413-430."""
    src_bits = np.ascontiguousarray(src_bits, dtype=np.uint16)
    rows, ld = src_bits.shape
    dst = np.zeros((rows, k // 2), np.uint8)
    sf = np.zeros(sf_words(rows, k, 32, groups), np.uint32)
    _cast_fp4(src_bits, ld, rows, k, groups, rule, dst, sf)
    return dst, sf


def cast_bf16_to_fp8_sf(src_bits, k, gran, groups=1):
    """bf16 -> e4m3 + packed UE8M0 (parity unpinned; rule stated in dg_oracle.c)."""
    src_bits = np.ascontiguousarray(src_bits, dtype=np.uint16)
    rows, ld = src_bits.shape
    dst = np.zeros((rows, k), np.uint8)
    sf = np.zeros(sf_words(rows, k, gran, groups), np.uint32)
    _cast_fp8(src_bits, ld, rows, k, gran, groups, dst, sf)
    return dst, sf


def quantize_fp8_ue8m0_blocks(src_bits, k, block_rows):
    """bf16 -> e4m3 with one UE8M0 exponent per (block_rows x 128) block; returns (bytes, exponents)."""
    src_bits = np.ascontiguousarray(src_bits, dtype=np.uint16)
    rows, ld = src_bits.shape
    dst = np.zeros((rows, k), np.uint8)
    exps = np.zeros(((rows + block_rows - 1) // block_rows, k // 128), np.uint8)
    _quant_blocks(src_bits, ld, rows, k, block_rows, dst, exps)
    return dst, exps


def exps_to_f32(exps):
    """UE8M0 bytes -> f32 powers of two (reference.rs:260-262)."""
    return (np.ascontiguousarray(exps, np.uint8).astype(np.uint32) << 23).view(np.float32)


def quantize_fp8_f32scale(x, block_rows):
    """amax/448 f32-scale recipe (parity unpinned), scales indexed as reference.rs:104-105."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    q = np.zeros((rows, k), np.uint8)
    sf = np.zeros(((rows + block_rows - 1) // block_rows, (k + 127) // 128), np.float32)
    _quant_f32scale(x, rows, k, block_rows, q, sf)
    return q, sf


# ---- SF transforms ---------------------------------------------------------------
def transform_sf1d_packed(src, k, gran, groups=1):
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows, ld = src.shape
    dst = np.zeros(sf_words(rows, k, gran, groups), np.uint32)
    _tsf1d(src, ld, rows, k, gran, groups, dst)
    return dst


def transform_sf2d_packed(src, rows, k, groups=1):
    src = np.ascontiguousarray(src, dtype=np.float32)
    dst = np.zeros(sf_words(rows, k, 128, groups), np.uint32)
    _tsf2d(src, src.shape[1], rows, k, groups, dst)
    return dst


def transform_sf_f32(src, mn, sf_k, batches=1):
    src = np.ascontiguousarray(src, dtype=np.float32).reshape(batches, mn, sf_k)
    dst = np.zeros((batches * sf_k, sf_aligned_rows(mn)), np.float32)
    _tsf_f32(src, mn, sf_k, batches, dst)
    return dst


def transform_sf_t_packed(src_t, rows, k, gran, groups=1):
    src_t = np.ascontiguousarray(src_t, dtype=np.float32)
    dst = np.zeros(sf_words(rows, k, gran, groups), np.uint32)
    _tsf_t(src_t, rows, k, gran, groups, dst)
    return dst


def psum_from_m_indices(m_indices, groups):
    m_indices = np.ascontiguousarray(m_indices, dtype=np.int32)
    out = np.zeros(groups, np.uint32)
    _psum(m_indices, m_indices.size, groups, out)
    return out


# ---- reference GEMMs ---------------------------------------------------------------
def ref_fp8_gemm_nt(a, sfa, b, sfb, threads=1):
    """reference.rs:85-114."""
    a = np.ascontiguousarray(a, np.uint8)
    b = np.ascontiguousarray(b, np.uint8)
    m, k = a.shape
    n = b.shape[0]
    out = np.zeros((m, n), np.float32)
    _ref_gemm(a, np.ascontiguousarray(sfa, np.float32), m, b, np.ascontiguousarray(sfb, np.float32), n, k, out,
              threads)
    return out


def ref_m_grouped_contiguous(a, sfa, m_indices, b, sfb, n, per_group_sfb=False, threads=1):
    """reference.rs:133-168; per_group_sfb=True gives every group its own (n/128, k/128) scale block."""
    a = np.ascontiguousarray(a, np.uint8)
    b = np.ascontiguousarray(b, np.uint8)
    m, k = a.shape
    kb = (k + 127) // 128
    stride = ((n + 127) // 128) * kb if per_group_sfb else 0
    out = np.zeros((m, n), np.float32)
    _ref_contig(a, np.ascontiguousarray(sfa, np.float32), np.ascontiguousarray(m_indices, np.int32), m, b,
                np.ascontiguousarray(sfb, np.float32), stride, n, k, out, threads)
    return out


def ref_m_grouped_masked(a, sfa, masked_m, m_per_group, b, sfb, n, per_group_sfb=False, threads=1):
    """reference.rs:172-208."""
    a = np.ascontiguousarray(a, np.uint8)
    b = np.ascontiguousarray(b, np.uint8)
    masked_m = np.ascontiguousarray(masked_m, np.int32)
    groups = masked_m.size
    k = a.shape[1]
    kb = (k + 127) // 128
    stride = ((n + 127) // 128) * kb if per_group_sfb else 0
    out = np.zeros((groups * m_per_group, n), np.float32)
    _ref_masked(a, np.ascontiguousarray(sfa, np.float32), masked_m, groups, m_per_group, b,
                np.ascontiguousarray(sfb, np.float32), stride, n, k, out, threads)
    return out


def mxfp4_gemm_reference(a, a_sf, m, b, b_sf, n, k, threads=1):
    """reference.rs:293-329."""
    out = np.zeros((m, n), np.float32)
    _mxfp4_ref(np.ascontiguousarray(a, np.uint8), np.ascontiguousarray(a_sf, np.uint32), m,
               np.ascontiguousarray(b, np.uint8), np.ascontiguousarray(b_sf, np.uint32), n, k, out, threads)
    return out


def dequant_rows(data, sf, bits, gran, k, groups, group_rows, row_ids):
    """Rows of a packed operand as f32 with their UE8M0 scales applied."""
    row_ids = np.ascontiguousarray(row_ids, np.uint32)
    out = np.zeros((row_ids.size, k), np.float32)
    _dequant(np.ascontiguousarray(data, np.uint8).reshape(-1), np.ascontiguousarray(sf, np.uint32), bits, gran, k,
             groups, group_rows, row_ids, row_ids.size, out)
    return out


def lp_gemm_rows(a, a_sf, a_bits, a_gran, a_groups, a_group_rows, a_rows,
                 b, b_sf, b_bits, b_gran, b_groups, b_group_rows, b_rows, k):
    """D[a_rows, b_rows] of a packed-operand GEMM in f64 (dequantise, then one BLAS call).

    Validated against ref_fp8_gemm_nt / mxfp4_gemm_reference on small shapes by
    the oracle tests; used for sub-sampled parity at sizes the scalar loops
    cannot finish.
    """
    af = dequant_rows(a, a_sf, a_bits, a_gran, k, a_groups, a_group_rows, a_rows).astype(np.float64)
    bf = dequant_rows(b, b_sf, b_bits, b_gran, k, b_groups, b_group_rows, b_rows).astype(np.float64)
    return (af @ bf.T).astype(np.float32)


def requant_fp8(d, batch, n_total_rows_stride, out, sfd):
    """FP8-requantize epilogue of one batch/group (order of operations: cuda/sm100_common.rs:1046-1074)."""
    d = np.ascontiguousarray(d, np.float32)
    rows, n = d.shape
    _requant(d, rows, n, batch, n_total_rows_stride, out, sfd)


def moe_combine(rows_bits, pos, w):
    """out[t] = bf16(sum_j w[t,j] * rows[pos[t,j]]) (cuda/layout.rs:192-216 as a gather-reduce); bf16 bit patterns in and out."""
    rows_bits = np.ascontiguousarray(rows_bits, np.uint16)
    pos = np.ascontiguousarray(pos, np.int32)
    w = np.ascontiguousarray(w, np.float32)
    tokens, topk = pos.shape
    n = rows_bits.shape[1]
    out = np.zeros((tokens, n), np.uint16)
    _moe_combine(rows_bits, n, pos, w, tokens, topk, n, out)
    return out


_ref_bf16 = _sig("dgo_ref_bf16_gemm_nt", None, _u16p, C.c_uint32, _u16p, C.c_uint32, C.c_uint32, _f32p, C.c_int)


def ref_bf16_gemm_nt(a_bits, b_bits, threads=1):
    """reference.rs:117: (m, k) x (n, k)^T over bf16 bit patterns, f64 accumulation -> f32."""
    a_bits = np.ascontiguousarray(a_bits, np.uint16)
    b_bits = np.ascontiguousarray(b_bits, np.uint16)
    m, k = a_bits.shape
    n = b_bits.shape[0]
    out = np.zeros((m, n), np.float32)
    _ref_bf16(a_bits, m, b_bits, n, k, out, threads)
    return out


_silu_mul = _sig("dgo_silu_mul_bf16", None, _u16p, C.c_uint32, C.c_uint32, C.c_uint32, _u16p)


def silu_mul_bf16(gate_up_bits):
    """(rows, 2n) bf16 bits [gate | up] -> (rows, n) bf16 bits of silu(gate) * up (cuda/layout.rs:218-233)."""
    gate_up_bits = np.ascontiguousarray(gate_up_bits, np.uint16)
    rows, ld = gate_up_bits.shape
    out = np.zeros((rows, ld // 2), np.uint16)
    _silu_mul(gate_up_bits, ld, rows, ld // 2, out)
    return out


def calc_diff(x, y):
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    y = np.ascontiguousarray(y, np.float32).reshape(-1)
    return float(_calc_diff(x, y, x.size))


def lcg_values(seed, count, scale):
    """The reference tests' input generator (tests/e2e.rs:11-30): 64-bit LCG, top 31 bits / u32::MAX - 0.5."""
    out = np.empty(count, np.float32)
    s = seed & 0xFFFFFFFFFFFFFFFF
    umax = np.float32(0xFFFFFFFF)
    for i in range(count):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = (np.float32(s >> 33) / umax - np.float32(0.5)) * np.float32(scale)
    return out
