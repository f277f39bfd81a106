"""The older f32-scale API (deepgemm/src/ops.rs:328,422,535,635), checked against the literal CPU references
(reference.rs:85-208) in the style of the reference's own end-to-end tests (deepgemm/tests/e2e.rs:47-249): LCG inputs
quantised with f32_to_e4m3, constant scales, the same shapes and the same masked_m fixture.

Two routes serve these calls.  The default applies every f32 scale exactly, K block by K block (dg_gemm_f32scale_kernel): it
is run with the reference's own scale values 0.01 / 0.02, with per-block amax / 448 scales (the CPU-runnable benchmark case as
the contract words it, against a committed fixture), and with powers of two.  DG_F32_SCALES=exponent is what the reference
itself does on Blackwell -- only the exponent of each scale reaches the block-scaled kernel (cuda/sm100_cast.rs:214) -- and
is exact for powers of two only, so it is run with 2^-6 / 2^-5."""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from oracle import oracle as O
from tests.helpers import dev, to_f32

pytestmark = pytest.mark.gpu
import os

# (route, activation scale, weight scale)
ROUTES = [("exact", 0.01, 0.02), ("exact", 2.0 ** -6, 2.0 ** -5), ("exponent", 2.0 ** -6, 2.0 ** -5)]
routes = pytest.mark.parametrize("route,SFA,SFB", ROUTES)


def pin_route(monkeypatch, route):
    if route == "exponent":
        monkeypatch.setenv("DG_F32_SCALES", "exponent")
    else:
        monkeypatch.delenv("DG_F32_SCALES", raising=False)


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


def lcg_e4m3(seed, rows, k):
    v = O.lcg_values(seed, rows * k, 2.0).reshape(rows, k)
    return np.vectorize(O.f32_to_e4m3_fast, otypes=[np.uint8])(v)


def reference_tolerance(got, want):
    # e2e.rs: |g - w| / max(|w|, 1) < 0.05
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1.0)) < 0.05
    assert O.calc_diff(got, want) <= 2e-5


@routes
def test_fp8_gemm_nt(ctx, route, SFA, SFB, monkeypatch):
    pin_route(monkeypatch, route)
    m, n, k = 256, 512, 768                                  # e2e.rs:47
    a, b = lcg_e4m3(1, m, k), lcg_e4m3(2, n, k)
    sfa = np.full((m, k // 128), SFA, np.float32)
    sfb = np.full((n // 128, k // 128), SFB, np.float32)
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), m, k // 128, 1)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(dev(a), m, k, k), a_sf_t, dg.Fp8Tensor(dev(b), n, k, k), dev(sfb), out, n)
    ctx.sync()
    reference_tolerance(to_f32(out), O.ref_fp8_gemm_nt(a, sfa, b, sfb, threads=8))


@routes
def test_m_grouped_contiguous(ctx, route, SFA, SFB, monkeypatch):
    pin_route(monkeypatch, route)
    groups, gm, n, k = 4, 128, 256, 512                      # e2e.rs:88
    m = groups * gm
    a, b = lcg_e4m3(3, m, k), lcg_e4m3(4, groups * n, k)
    sfa = np.full((m, k // 128), SFA, np.float32)
    sfb = np.full((groups * n // 128, k // 128), SFB, np.float32)
    m_idx = np.repeat(np.arange(groups, dtype=np.int32), gm)
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), m, k // 128, 1)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_gemm_nt_contiguous_dev(ctx, dg.Fp8Tensor(dev(a), m, k, k), a_sf_t, dg.Fp8Tensor(dev(b), groups * n, k, k), dev(sfb), out, n,
                                            dev(m_idx), groups)
    ctx.sync()
    want = O.ref_m_grouped_contiguous(a, sfa, m_idx, b, sfb[:n // 128].reshape(-1), n, threads=8)   # the reference indexes one shared scale block
    reference_tolerance(to_f32(out), want)


@routes
def test_m_grouped_masked_and_bmm(ctx, route, SFA, SFB, monkeypatch):
    pin_route(monkeypatch, route)
    masked = np.array([37, 128, 1, 64, 15, 100, 128, 3], np.int32)   # e2e.rs:131
    groups, m_max, n, k = len(masked), 128, 256, 512
    a, b = lcg_e4m3(5, groups * m_max, k), lcg_e4m3(6, groups * n, k)
    sfa = np.full((groups * m_max, k // 128), SFA, np.float32)
    sfb = np.full((groups * n // 128, k // 128), SFB, np.float32)
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), m_max, k // 128, groups)
    out = torch.zeros((groups * m_max, n), dtype=torch.bfloat16, device="cuda")
    A, B = dg.Fp8Tensor(dev(a), groups * m_max, k, k), dg.Fp8Tensor(dev(b), groups * n, k, k)
    dg.m_grouped_fp8_gemm_nt_masked_dev(ctx, A, a_sf_t, B, dev(sfb), out, n, dev(masked), groups, m_max, 64)
    ctx.sync()
    want = O.ref_m_grouped_masked(a, sfa, masked, m_max, b, sfb[:n // 128].reshape(-1), n, threads=8)
    got = to_f32(out)
    valid = np.concatenate([np.arange(g * m_max, g * m_max + masked[g]) for g in range(groups)])
    reference_tolerance(got[valid], want[valid])
    # batched: every row of every group
    out2 = torch.zeros((groups * m_max, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_bmm_nt_dev(ctx, A, a_sf_t, B, dev(sfb), out2, n, groups, m_max, n)
    ctx.sync()
    want2 = O.ref_m_grouped_masked(a, sfa, np.full(groups, m_max, np.int32), m_max, b, sfb[:n // 128].reshape(-1), n, threads=8)
    reference_tolerance(to_f32(out2), want2)


def test_shape_errors(ctx):
    a = torch.zeros((128, 256), dtype=torch.uint8, device="cuda")
    sf = torch.ones((2, 128), dtype=torch.float32, device="cuda")
    out = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(dg.DgError) as e:                      # ops.rs:308 k % 128
        dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(a, 128, 192, 256), sf, dg.Fp8Tensor(a, 128, 192, 256), sf, out, 128)
    assert e.value.kind == "Shape"
    with pytest.raises(dg.DgError):                           # ops.rs:313 n % 8
        dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(a, 128, 256, 256), sf, dg.Fp8Tensor(a, 100, 256, 256), sf, out, 128)


def test_cpu_runnable_case_with_amax_over_448_scales(ctx):
    # the benchmark contract's first configuration as it is worded: M=128, N=256, K=512, e4m3 with f32 scales amax / 448 (A per
    # 1x128, B per 128x128), f32 accumulation, bf16 output -- committed fixture: inputs, scales and ref_fp8_gemm_nt's output
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "fp8_gemm_f32scale_128x256x512.npz"))
    a, b, sfa, sfb, want = z["a"], z["b"], z["sfa"], z["sfb"], z["out"]
    m, n, k = 128, 256, 512
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), m, k // 128, 1)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(dev(a), m, k, k), a_sf_t, dg.Fp8Tensor(dev(b), n, k, k), dev(sfb), out, n)
    ctx.sync()
    assert O.calc_diff(to_f32(out), want) <= 2e-5             # contract: 1e-3; only the bf16 rounding of the output separates the two


def test_exact_route_ragged_shapes_and_varying_scales(ctx):
    # scales that differ per row, per tile and per K block (mantissas included), M and N off the tile grid, several tiles and
    # k-blocks per CTA; contiguous groups of uneven size with alignment padding
    rng = np.random.default_rng(5)
    m, n, k = 333, 392, 1664
    a, b = lcg_e4m3(11, m, k), lcg_e4m3(12, n, k)
    sfa = rng.uniform(0.004, 0.03, (m, k // 128)).astype(np.float32)
    sfb = rng.uniform(0.004, 0.03, ((n + 127) // 128, k // 128)).astype(np.float32)
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), m, k // 128, 1)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt_dev(ctx, dg.Fp8Tensor(dev(a), m, k, k), a_sf_t, dg.Fp8Tensor(dev(b), n, k, k), dev(sfb), out, n)
    ctx.sync()
    reference_tolerance(to_f32(out), O.ref_fp8_gemm_nt(a, sfa, b, sfb, threads=8))
    sizes, gn = [200, 0, 37, 129], 256
    m_idx = np.concatenate([np.concatenate([np.full(s, g, np.int32), np.full((-s) % 128, -1, np.int32)]) for g, s in enumerate(sizes)])
    mt, groups = len(m_idx), len(sizes)
    a, b = lcg_e4m3(13, mt, k), lcg_e4m3(14, groups * gn, k)
    sfa = rng.uniform(0.004, 0.03, (mt, k // 128)).astype(np.float32)
    sfb = rng.uniform(0.004, 0.03, (groups * gn // 128, k // 128)).astype(np.float32)
    a_sf_t = dg.transform_sf_dev(ctx, dev(sfa), mt, k // 128, 1)
    out = torch.full((mt, gn), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_gemm_nt_contiguous_dev(ctx, dg.Fp8Tensor(dev(a), mt, k, k), a_sf_t, dg.Fp8Tensor(dev(b), groups * gn, k, k), dev(sfb), out, gn,
                                            dev(m_idx), groups)
    ctx.sync()
    want = O.ref_m_grouped_contiguous(a, sfa, m_idx, b, sfb.reshape(-1), gn, per_group_sfb=True, threads=8)
    valid = np.nonzero(m_idx >= 0)[0]
    got = to_f32(out)
    assert not np.isnan(got[valid]).any()
    reference_tolerance(got[valid], want[valid])
