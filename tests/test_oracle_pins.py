"""Pins the CPU oracle to the reference crate's own known-answer vectors.

Sources (paths inside the reference crate):
  deepgemm/src/reference.rs:336-376  e4m3 decode table, quantize / bf16 round trips
  deepgemm/tests/unit.rs:72-88       e2m1 codes and ties, UE8M0
  deepgemm/tests/unit.rs:90-158      MXFP4 GEMM self-consistency on modular inputs
  deepgemm/tests/e2e.rs:413-430      grouped packed scale-factor layout
"""
import numpy as np
import pytest

from oracle import oracle as O


def test_e4m3_decode_known_answers():
    # reference.rs:336-346
    assert O.e4m3_to_f32(0x00) == 0.0
    assert O.e4m3_to_f32(0x40) == 2.0
    assert O.e4m3_to_f32(0x38) == 1.0
    assert O.e4m3_to_f32(0x30) == 0.5
    assert O.e4m3_to_f32(0x28) == 0.25
    assert O.e4m3_to_f32(0x01) == 2.0 ** -9
    assert O.e4m3_to_f32(0x7E) == 448.0
    assert np.isnan(O.e4m3_to_f32(0x7F))
    assert O.e4m3_to_f32(0xC0) == -2.0


def test_e4m3_quantize_round_trip():
    # reference.rs:349-367
    for x in [0.0, 0.5, 1.0, -1.0, 2.0, 0.25, -0.125, 448.0, -448.0, 2.0 ** -9]:
        d = O.e4m3_to_f32(O.f32_to_e4m3(x))
        assert abs(d - x) / max(abs(x), 1e-6) < 0.2
    # every finite code is a fixed point of encode(decode(.)) except -0 (sign comes from v < 0)
    for c in range(256):
        if c & 0x7F == 0x7F:
            continue
        want = 0 if c == 0x80 else c
        assert O.f32_to_e4m3(O.e4m3_to_f32(c)) == want
    assert O.f32_to_e4m3(float("nan")) == 0x7F
    assert O.f32_to_e4m3(1e9) == 0x7E and O.f32_to_e4m3(-1e9) == 0xFE
    assert O.f32_to_e4m3(-0.0) == 0x00
    assert O.f32_to_e4m3(-1e-9) == 0x80


def test_bf16_round_trip():
    # reference.rs:370-376
    for x in [0.0, 1.0, -2.5, 0.25, 100.0]:
        d = O.bf16_to_f32(O.f32_to_bf16(x))
        assert abs(d - x) / max(abs(x), 1e-6) < 0.01
    # ties to even: 1 + 2^-8 is halfway between two bf16 values
    assert O.f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    assert O.f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    assert np.array_equal(O.bf16_bits(x), np.array([O.f32_to_bf16(v) for v in x], np.uint16))


def test_fast_e4m3_encoder_equals_search_encoder():
    # all 65536 bf16 bit patterns (the quantizer's inputs are bf16 times a power of two) ...
    bits = np.arange(65536, dtype=np.uint32)
    vals = (bits << 16).view(np.float32)
    for scale in (1.0, 2.0 ** -5, 2.0 ** 7, 2.0 ** -13):
        for v in vals[::7]:
            x = np.float32(v) * np.float32(scale)
            assert O.f32_to_e4m3(x) == O.f32_to_e4m3_fast(x), (v, scale)
    # ... and arbitrary f32, including exact halfway points of the grid
    rng = np.random.default_rng(1)
    for x in np.concatenate([rng.standard_normal(4000) * 100, rng.uniform(-2 ** -6, 2 ** -6, 2000)]):
        assert O.f32_to_e4m3(x) == O.f32_to_e4m3_fast(x), x
    for c in range(0x7E):
        mid = (O.e4m3_to_f32(c) + O.e4m3_to_f32(c + 1)) / 2
        assert O.f32_to_e4m3(mid) == O.f32_to_e4m3_fast(mid) == (c if c % 2 == 0 else c + 1)


def test_e2m1_and_ue8m0_known_answers():
    # tests/unit.rs:72-88
    values = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
    for code, v in enumerate(values):
        assert O.encode_e2m1(v) == code
        assert O.e2m1_to_f32(code) == v
    assert O.encode_e2m1(0.25) == 0
    assert O.encode_e2m1(0.75) == 2
    assert O.encode_e2m1(5.0) == 6
    assert O.encode_e2m1(100.0) == 7
    assert O.f32_to_ue8m0(1.0) == 127
    assert O.ue8m0_to_f32(127) == 1.0
    assert O.ue8m0_to_f32(130) == 8.0
    assert O.f32_to_ue8m0(0.0) == 1  # floored at 1 (reference.rs:256)


def _modular_rows():
    # tests/unit.rs:93-109
    m, n, k = 8, 8, 128
    a = np.array([[(((i * 13 + j * 7) % 17) - 8.0) / 8.0 for j in range(k)] for i in range(m)], np.float32)
    b = np.array([[(((i * 11 + j * 5) % 19) - 9.0) / 9.0 for j in range(k)] for i in range(n)], np.float32)
    return m, n, k, a, b


def test_mxfp4_reference_gemm_matches_float():
    # tests/unit.rs:90-158.  The reference feeds f32 rows straight into the row quantizer; the values
    # here are not all bf16-exact, so quantize from f32 with the same rule via the scalar entry points.
    m, n, k, a, b = _modular_rows()

    def quant_row(row):
        packed, sfs = [], []
        for g in range(0, k, 32):
            blk = row[g:g + 32]
            e = O.sf_exp_e2m1(np.max(np.abs(blk)), O.SF_RULE_REFERENCE_CPU)
            inv = np.float32(1.0) / np.float32(O.ue8m0_to_f32(e))
            sfs.append(e)
            for i in range(0, 32, 2):
                packed.append(O.encode_e2m1(blk[i] * inv) | (O.encode_e2m1(blk[i + 1] * inv) << 4))
        return packed, sfs

    def pack_sf(sfs, rows):
        aligned = (rows + 3) // 4 * 4
        out = np.zeros(((k + 127) // 128) * aligned, np.uint32)
        for r, s in enumerate(sfs):
            for j, e in enumerate(s):
                out[(j // 4) * aligned + r] |= np.uint32(e << ((j % 4) * 8))
        return out

    ap, asf = zip(*[quant_row(r) for r in a])
    bp, bsf = zip(*[quant_row(r) for r in b])
    ap, bp = np.array(ap, np.uint8), np.array(bp, np.uint8)
    got = O.mxfp4_gemm_reference(ap, pack_sf(asf, m), m, bp, pack_sf(bsf, n), n, k)

    def dequant(p, sfs):
        out = np.zeros((p.shape[0], k), np.float32)
        for r in range(p.shape[0]):
            for kk in range(k):
                byte = int(p[r, kk // 2])
                code = (byte >> 4) if kk % 2 else (byte & 0xF)
                out[r, kk] = np.float32(O.e2m1_to_f32(code)) * np.float32(O.ue8m0_to_f32(sfs[r][kk // 32]))
        return out

    want = np.zeros((m, n), np.float32)
    aq, bq = dequant(ap, asf), dequant(bp, bsf)
    for i in range(m):
        for j in range(n):
            acc = np.float32(0)
            for kk in range(k):
                acc = np.float32(acc + aq[i, kk] * bq[j, kk])
            want[i, j] = acc
    assert np.max(np.abs(got - want)) < 1e-3
    # the reference-CPU rule keeps every scale at 2^1 or above (reference.rs:273)
    assert min(min(s) for s in asf) >= 128
    # and the generic dequantise+matmul checker agrees with the scalar restatement
    rows = np.arange(m, dtype=np.uint32)
    d2 = O.lp_gemm_rows(ap, pack_sf(asf, m), 4, 32, 1, m, rows, bp, pack_sf(bsf, n), 4, 32, 1, n, rows, k)
    assert np.max(np.abs(d2 - got)) < 1e-4


def test_array_fp4_quantizer_matches_row_rule_and_grouped_layout():
    # tests/e2e.rs:413-430: word of (group g, local row, col) at (g*cols + col)*align4(group_rows) + local
    rng = np.random.default_rng(5)
    groups, group_rows, k = 3, 6, 256
    x = O.bf16_bits(rng.standard_normal((groups * group_rows, k)).astype(np.float32))
    for rule in (O.SF_RULE_REFERENCE_CPU, O.SF_RULE_RANGE_FIT):
        q, sf = O.cast_bf16_to_fp4_packed_sf(x, k, groups, rule)
        xf = O.bf16_to_f32_array(x)
        aligned, cols = 8, 2
        assert sf.size == groups * cols * aligned
        for r in range(groups * group_rows):
            g, local = divmod(r, group_rows)
            for j in range(k // 32):
                blk = xf[r, j * 32:(j + 1) * 32]
                e = O.sf_exp_e2m1(np.max(np.abs(blk)), rule)
                w = int(sf[(g * cols + j // 4) * aligned + local])
                assert (w >> ((j % 4) * 8)) & 0xFF == e
                inv = np.float32(1.0) / np.float32(O.ue8m0_to_f32(e))
                for i in range(0, 32, 2):
                    want = O.encode_e2m1(blk[i] * inv) | (O.encode_e2m1(blk[i + 1] * inv) << 4)
                    assert q[r, (j * 32 + i) // 2] == want
        # padding rows of the aligned stride stay zero
        assert np.all(sf.reshape(groups * cols, aligned)[:, group_rows:] == 0)


def test_sf_exponent_rules():
    # rule 1 for e2m1: smallest power of two with amax/sf <= 6; e4m3: <= 448, floor 2^-22
    for amax in [1e-30, 1e-4, 0.3, 1.0, 2.0, 4.5, 6.0, 6.01, 448.0, 448.5, 1000.0, 3e38]:
        e = O.sf_exp_e4m3(amax)
        sf = O.ue8m0_to_f32(e)
        assert e >= 105
        if e > 105:
            assert amax / sf <= 448.0 and amax / (sf / 2) > 448.0
        e = O.sf_exp_e2m1(amax, O.SF_RULE_RANGE_FIT)
        sf = O.ue8m0_to_f32(e)
        if e > 1:
            assert amax / sf <= 6.0 and amax / (sf / 2) > 6.0
        # reference CPU rule: max(rounded, 128)
        assert O.sf_exp_e2m1(amax, O.SF_RULE_REFERENCE_CPU) >= 128
    assert O.sf_exp_e4m3(448.0) == 127 and O.sf_exp_e4m3(1.0) == 119 and O.sf_exp_e4m3(0.0) == 105
    assert O.sf_exp_e2m1(6.0, 1) == 127 and O.sf_exp_e2m1(3.0, 0) == 128
    # bf16 flavour agrees with the f32 flavour on bf16 inputs
    for bits in range(0, 0x7F80, 37):
        assert O.sf_exp_e4m3_bf16(bits) == O.sf_exp_e4m3(O.bf16_to_f32(bits))


def test_fp8_reference_gemm_against_dequant_matmul():
    # The scalar restatement (reference.rs:85-114) and the dequantise+matmul checker agree when scales are
    # powers of two; this is what lets sub-sampled parity run at full problem sizes.
    rng = np.random.default_rng(7)
    m, n, k = 16, 256, 512
    a = O.bf16_bits(rng.standard_normal((m, k)).astype(np.float32))
    b = O.bf16_bits(rng.standard_normal((n, k)).astype(np.float32))
    aq, asf = O.cast_bf16_to_fp8_sf(a, k, 128)
    bq, bsf = O.cast_bf16_to_fp8_sf(b, k, 128)
    kb = k // 128
    sfa = np.array([[O.ue8m0_to_f32((int(asf[(c // 4) * 16 + r]) >> ((c % 4) * 8)) & 0xFF) for c in range(kb)]
                    for r in range(m)], np.float32)
    # reference indexes weight scales per 128-row tile: give every row of a tile the same scale
    bsf_rows = np.array([[(int(bsf[(c // 4) * 256 + r]) >> ((c % 4) * 8)) & 0xFF for c in range(kb)]
                         for r in range(n)])
    tile_e = bsf_rows.reshape(n // 128, 128, kb).max(axis=1)
    sfb = np.vectorize(O.ue8m0_to_f32)(tile_e).astype(np.float32)
    bsf_tile = O.transform_sf2d_packed(sfb, n, k)
    # requantise b under the tile scale so the bytes match the scales
    bf = O.bf16_to_f32_array(b)
    bq2 = np.zeros_like(bq)
    for r in range(n):
        for c in range(kb):
            inv = np.float32(1.0) / sfb[r // 128, c]
            for i in range(128):
                bq2[r, c * 128 + i] = O.f32_to_e4m3_fast(bf[r, c * 128 + i] * inv)
    want = O.ref_fp8_gemm_nt(aq, sfa, bq2, sfb)
    rows_a, rows_b = np.arange(m, dtype=np.uint32), np.arange(n, dtype=np.uint32)
    got = O.lp_gemm_rows(aq, asf, 8, 128, 1, m, rows_a, bq2, bsf_tile, 8, 128, 1, n, rows_b, k)
    assert O.calc_diff(got, want) < 1e-6
    # threads do not change the scalar restatement's result
    assert np.array_equal(want, O.ref_fp8_gemm_nt(aq, sfa, bq2, sfb, threads=4))


def test_grouped_reference_gemms():
    rng = np.random.default_rng(9)
    groups, n, k, mpg = 4, 128, 256, 8
    masked = np.array([3, 8, 0, 1], np.int32)  # shape of the reference fixture masked_m = [37,128,1,64,...]
    a = rng.integers(0, 0x7E, (groups * mpg, k), dtype=np.uint8)
    b = rng.integers(0, 0x7E, (groups * n, k), dtype=np.uint8)
    sfa = np.full((groups * mpg, k // 128), 0.01, np.float32)  # constant scales like tests/e2e.rs
    sfb = np.full((n // 128, k // 128), 0.02, np.float32)
    out = O.ref_m_grouped_masked(a, sfa, masked, mpg, b, sfb, n)
    for g in range(groups):
        blk = out[g * mpg:(g + 1) * mpg]
        assert np.all(blk[masked[g]:] == 0)
        if masked[g]:
            want = O.ref_fp8_gemm_nt(a[g * mpg:g * mpg + masked[g]], sfa[:masked[g]], b[g * n:(g + 1) * n], sfb)
            assert np.array_equal(blk[:masked[g]], want)
    m_idx = np.repeat(np.arange(groups, dtype=np.int32), mpg)
    m_idx[5] = -1
    out = O.ref_m_grouped_contiguous(a, sfa, m_idx, b, sfb, n)
    assert np.all(out[5] == 0)
    want = O.ref_fp8_gemm_nt(a[8:16], sfa[8:16], b[n:2 * n], sfb)
    assert np.array_equal(out[8:16], want)
    # psum: one-past-last row per group, empty groups inherit the running end
    assert list(O.psum_from_m_indices(np.array([0, 0, -1, -1, 2, 2, 2, -1], np.int32), 4)) == [2, 2, 7, 7]


def test_sf_transforms():
    rng = np.random.default_rng(11)
    rows, k = 10, 1024 + 128  # 9 k-blocks: last word has 3 tail bytes that read as 127
    e = rng.integers(100, 140, (rows, 9))
    sf = np.vectorize(O.ue8m0_to_f32)(e).astype(np.float32)
    w = O.transform_sf1d_packed(sf, k, 128)
    assert w.size == 3 * 12
    for r in range(rows):
        for c in range(9):
            assert (int(w[(c // 4) * 12 + r]) >> ((c % 4) * 8)) & 0xFF == e[r, c]
        assert int(w[2 * 12 + r]) >> 8 == 0x7F7F7F
    t = O.transform_sf_f32(sf, rows, 9)
    assert t.shape == (9, 12) and np.array_equal(t[:, :rows], sf.T) and np.all(t[:, rows:] == 0)
    assert np.array_equal(O.transform_sf_t_packed(t, rows, k, 128), w)
    # mantissa bits are dropped, not rounded (cuda/sm100_cast.rs:214)
    w2 = O.transform_sf1d_packed(sf * np.float32(1.9), k, 128)
    assert np.array_equal(w2, w)
    sf2 = np.vectorize(O.ue8m0_to_f32)(rng.integers(110, 130, (2, 9))).astype(np.float32)
    w2d = O.transform_sf2d_packed(sf2, 256, k)
    assert np.array_equal(w2d, O.transform_sf1d_packed(np.repeat(sf2, 128, axis=0), k, 128))


def test_bf16_reference_gemm_on_the_reference_test_pattern():
    # tests/e2e.rs:188-217 inputs; reference.rs:117-129 accumulates in f64 and rounds once, so it must agree with a
    # float64 matmul of the same bf16 values to f32 rounding
    m, n, k = 128, 256, 512
    a = O.bf16_bits(((np.arange(m * k) % 13).astype(np.float32) / np.float32(13.0) - np.float32(0.5)).reshape(m, k))
    b = O.bf16_bits(((np.arange(n * k) % 11).astype(np.float32) / np.float32(11.0) - np.float32(0.5)).reshape(n, k))
    got = O.ref_bf16_gemm_nt(a, b, threads=2)
    want = O.bf16_to_f32_array(a).astype(np.float64) @ O.bf16_to_f32_array(b).astype(np.float64).T
    assert np.allclose(got, want.astype(np.float32), rtol=2e-7, atol=1e-9)
    assert np.array_equal(got, O.ref_bf16_gemm_nt(a, b, threads=1))


def test_silu_mul_restatement_tracks_the_formula():
    # cuda/layout.rs:231 computes g / (1 + exp(-g)) * u in f32 with the device's fast exponential and rounds to bf16;
    # the restatement's explicit exponential must land on the bf16 nearest the f64 value, or its neighbour
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((64, 1024)) * 6).astype(np.float32)
    bits = O.bf16_bits(x)
    got_bits = O.silu_mul_bf16(bits)
    xb = O.bf16_to_f32_array(bits).astype(np.float64)
    g, u = xb[:, :512], xb[:, 512:]
    want = g / (1.0 + np.exp(-g)) * u
    want_bits = O.bf16_bits(want.astype(np.float32))
    delta = np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32))
    assert delta.max() <= 1
    assert (delta != 0).mean() < 2e-3
    edge = O.bf16_bits(np.array([[0.0, 20.0, -20.0, -100.0, 2.0, 3.0, 4.0, 5.0]], np.float32))
    out = O.bf16_to_f32_array(O.silu_mul_bf16(edge))[0]
    assert out[0] == 0.0 and out[1] == 60.0 and abs(out[2] + 20 * np.exp(-20.0) * 4.0) < 1e-9 and out[3] == 0.0


def test_lcg_generator_matches_reference_recurrence():
    # tests/e2e.rs:11-30: s = s*6364136223846793005 + 1442695040888963407; ((s >> 33) / u32::MAX - 0.5) * scale
    v = O.lcg_values(999, 4, 2.0)
    s = 999
    for i in range(4):
        s = (s * 6364136223846793005 + 1442695040888963407) % 2 ** 64
        assert v[i] == (np.float32(s >> 33) / np.float32(4294967295.0) - np.float32(0.5)) * np.float32(2.0)
    assert np.all(np.abs(v) <= 1.0)


def test_golden_fixtures_reproduce():
    # the committed vectors (tests/golden/make_golden.py) are what the oracle computes today
    import os
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    z = np.load(os.path.join(here, "fp8_gemm_128x256x512.npz"))
    assert np.array_equal(O.ref_fp8_gemm_nt(z["a"], z["sfa"], z["b"], z["sfb"]), z["out"])
    assert np.array_equal(O.transform_sf1d_packed(z["sfa"], 512, 128), z["a_sf_packed"])
    assert np.array_equal(O.transform_sf2d_packed(z["sfb"], 256, 512), z["b_sf_packed"])
    a_bits = O.bf16_bits(np.random.default_rng(1001).standard_normal((128, 512)).astype(np.float32))
    aq, a_exp = O.quantize_fp8_ue8m0_blocks(a_bits, 512, 1)
    assert np.array_equal(aq, z["a"]) and np.array_equal(O.exps_to_f32(a_exp), z["sfa"])
    z = np.load(os.path.join(here, "mxfp4_8x8x128.npz"))
    assert np.array_equal(O.mxfp4_gemm_reference(z["a"], z["a_sf"], 8, z["b"], z["b_sf"], 8, 128), z["out"])
