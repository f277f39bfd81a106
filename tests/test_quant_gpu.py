"""Bit-exact parity of the quantise / scale-factor kernels with the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from oracle import oracle as O
from tests.helpers import dev, randn_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


def words(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("rows,k,gran,groups,ld_pad", [
    (128, 512, 128, 1, 0), (37, 1024, 128, 1, 0), (64, 1536, 128, 4, 64), (4096, 7168, 128, 1, 0),
    (128, 128, 32, 1, 0), (39, 640, 32, 3, 8), (256, 7168, 32, 1, 0), (1, 512, 128, 1, 0),
])
def test_cast_fp8_bit_exact(ctx, rows, k, gran, groups, ld_pad):
    ld = k + ld_pad
    src = np.zeros((rows, ld), np.uint16)
    src[:, :k] = randn_bf16(rows, k, seed=rows * 7 + k + gran)
    # exercise the scale floor, large magnitudes and exact zeros
    src[0, :min(k, 128)] = 0
    src[-1, :8] = O.bf16_bits(np.array([1e-30, -1e-30, 3e38, -448.0, 448.0, 0.0, -0.0, 1e-6], np.float32))
    want_q, want_sf = O.cast_bf16_to_fp8_sf(src[:, :k].copy(), k, gran, groups)
    q, sf = dg.cast_bf16_to_fp8_sf_dev(ctx, dev(src, torch.bfloat16), ld, rows, k, gran, groups)
    ctx.sync()
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(words(sf), want_sf)


@pytest.mark.parametrize("rows,k,groups,rule", [
    (128, 512, 1, 0), (128, 512, 1, 1), (37, 128, 1, 0), (24, 640, 4, 1), (512, 7168, 1, 0), (512, 7168, 2, 1),
])
def test_cast_fp4_bit_exact(ctx, rows, k, groups, rule):
    src = randn_bf16(rows, k, seed=rows + k + rule)
    src[0, :32] = 0
    src[-1, :4] = O.bf16_bits(np.array([100.0, -100.0, 1e-20, -0.0], np.float32))
    want_q, want_sf = O.cast_bf16_to_fp4_packed_sf(src, k, groups, rule)
    q, sf = dg.cast_bf16_to_fp4_packed_sf_dev(ctx, dev(src, torch.bfloat16), k, rows, k, groups, rule)
    ctx.sync()
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(words(sf), want_sf)


@pytest.mark.parametrize("rows,n,gran,groups,ld_pad", [
    (128, 512, 128, 1, 0), (37, 2048, 128, 1, 0), (64, 1536, 128, 4, 64), (2048, 2048, 128, 1, 0),
    (39, 640, 32, 3, 8), (256, 2048, 32, 1, 0),
])
def test_silu_mul_cast_fp8_bit_exact(ctx, rows, n, gran, groups, ld_pad):
    # the fused kernel must give what the two reference steps give one after the other: bf16(silu(gate) * up)
    # (moe.rs:273-296), then the FP8 quantiser on that bf16 matrix
    ld = 2 * n + ld_pad
    src = np.zeros((rows, ld), np.uint16)
    src[:, :2 * n] = O.bf16_bits(O.bf16_to_f32_array(randn_bf16(rows, 2 * n, seed=rows * 3 + n + gran)) * np.float32(3.0))
    src[0, :8] = O.bf16_bits(np.array([0.0, -0.0, 100.0, -100.0, 1e-30, -1e30, 30.0, -30.0], np.float32))
    src[-1, n:n + 8] = O.bf16_bits(np.array([0.0, -0.0, 1e20, -1e-20, 448.0, 1.0, -1.0, 7.0], np.float32))
    act = O.silu_mul_bf16(src[:, :2 * n].copy())
    want_q, want_sf = O.cast_bf16_to_fp8_sf(act, n, gran, groups)
    q, sf = dg.silu_mul_cast_fp8_sf_dev(ctx, dev(src, torch.bfloat16), ld, rows, n, gran, groups)
    ctx.sync()
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.array_equal(words(sf), want_sf)


def test_cast_argument_errors(ctx):
    with pytest.raises(dg.DgError) as e:
        dg.silu_mul_cast_fp8_sf_dev(ctx, torch.zeros((8, 1024), dtype=torch.bfloat16, device="cuda"), 512, 8, 512)   # ld < 2n
    assert e.value.kind == "Shape"
    src = torch.zeros((8, 512), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(dg.DgError) as e:
        dg.cast_bf16_to_fp8_sf_dev(ctx, src, 512, 8, 512, 64)
    assert e.value.kind == "Shape"
    with pytest.raises(dg.DgError):
        dg.cast_bf16_to_fp8_sf_dev(ctx, src, 512, 8, 384, 128)     # k % 512 != 0 (ops_sm100.rs:1198)
    with pytest.raises(dg.DgError):
        dg.cast_bf16_to_fp4_packed_sf_dev(ctx, src, 512, 8, 96)    # k % 128 != 0 (ops_sm100.rs:1143)


def test_transform_sf_family(ctx):
    rng = np.random.default_rng(3)
    for rows, k, gran, groups in [(100, 7168, 128, 1), (64, 1152, 128, 2), (96, 640, 32, 3), (4096, 7168, 128, 1)]:
        kb = (k + gran - 1) // gran
        exps = rng.integers(90, 150, (rows, kb)).astype(np.uint8)
        sf = O.exps_to_f32(exps) * np.float32(1.5)    # mantissa bits must be dropped, not rounded
        got = dg.transform_sf1d_packed_ue8m0_dev(ctx, dev(sf), kb, rows, k, gran, groups)
        assert np.array_equal(words(got), O.transform_sf1d_packed(sf, k, gran, groups))
        gr = rows // groups
        t_want = O.transform_sf_f32(sf, gr, kb, groups)
        t_got = dg.transform_sf_dev(ctx, dev(sf), gr, kb, groups)
        assert np.array_equal(t_got.cpu().numpy(), t_want)
        got_t = dg.transform_sf_t_packed_ue8m0_dev(ctx, t_got, rows, k, gran, groups)
        assert np.array_equal(words(got_t), O.transform_sf_t_packed(t_want, rows, k, gran, groups))
    for rows, k, groups in [(256, 1152, 1), (512, 7168, 2), (4096, 2048, 1)]:
        kb = k // 128
        sf2 = O.exps_to_f32(rng.integers(100, 140, (rows // 128, kb)).astype(np.uint8))
        got = dg.transform_sf2d_packed_ue8m0_dev(ctx, dev(sf2), kb, rows, k, groups)
        assert np.array_equal(words(got), O.transform_sf2d_packed(sf2, rows, k, groups))
    with pytest.raises(dg.DgError):
        dg.transform_sf2d_packed_ue8m0_dev(ctx, dev(np.ones((3, 4), np.float32)), 4, 384, 512, 2)  # 192-row groups
    ctx.sync()


def test_group_ends_and_unpack(ctx):
    rng = np.random.default_rng(4)
    for groups, m in [(4, 512), (256, 98304), (1500, 4096), (3, 7)]:
        # contiguous layout: sorted groups, some empty, padding rows (-1) after each group
        sizes = rng.integers(0, max(2, 2 * m // groups), groups)
        idx = np.full(m, -1, np.int32)
        pos = 0
        for g, s in enumerate(sizes):
            s = int(min(s, m - pos))
            idx[pos:pos + s] = g
            pos = min(m, pos + s + int(rng.integers(0, 3)))
        got = dg.psum_from_m_indices_dev(ctx, dev(idx), groups)
        assert np.array_equal(words(got), O.psum_from_m_indices(idx, groups))
    for n in (16, 4096, 1000, 7168 * 64 // 2):
        src = rng.integers(0, 256, n, dtype=np.uint8)
        got = dg.unpack_fp4_raw_dev(ctx, dev(src), n).cpu().numpy()
        assert np.array_equal(got[0::2], src & 0xF) and np.array_equal(got[1::2], src >> 4)
    ctx.sync()
