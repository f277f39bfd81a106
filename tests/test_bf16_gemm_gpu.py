"""BF16 GEMM (ops_sm100.rs:893 bf16_gemm_dev, ops.rs:769 bf16_gemm_nt_dev) against the CPU restatement of
ref_bf16_gemm_nt (reference.rs:117), through the C ABI."""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from oracle import oracle as O
from tests.helpers import dev, randn_bf16, sample_indices, to_f32

pytestmark = pytest.mark.gpu

TIGHT_BF16 = 2e-5
TIGHT_F32 = 1e-6


@pytest.fixture(scope="module")
def ctx():
    c = dg.DgContext(0)
    yield c
    c.sync()
    c.close()


def run(ctx, m, n, k, out_kind=0, alpha=None, ld_pad=0, seed=0):
    a, b = randn_bf16(m, k, seed=500 + seed), randn_bf16(n, k, seed=600 + seed)
    a_ld, b_ld = k + ld_pad, k + 2 * ld_pad
    a_full, b_full = np.zeros((m, a_ld), np.uint16), np.zeros((n, b_ld), np.uint16)
    a_full[:, :k], b_full[:, :k] = a, b
    a_full[:, k:], b_full[:, k:] = 0x7FC0, 0x7FC0           # NaN beyond k: must never be read into the product
    dtype = torch.bfloat16 if out_kind == 0 else torch.float32
    d = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    dg.bf16_gemm_dev(ctx, dev(a_full, torch.bfloat16), a_ld, m, dev(b_full, torch.bfloat16), b_ld, n, k, dg.Sm100Out(out_kind, d, n),
                     dg.Sm100Epilogue(alpha=alpha))
    ctx.sync()
    got = to_f32(d)
    assert not np.isnan(got).any()
    rows, cols = sample_indices(m, 40, seed), sample_indices(n, 64, seed + 1)
    want = O.ref_bf16_gemm_nt(a[rows], b[cols], threads=O.max_threads())
    if alpha is not None:
        got = got / np.float32(alpha)
    diff = O.calc_diff(got[np.ix_(rows, cols)], want)
    assert diff <= (TIGHT_BF16 if out_kind == 0 else TIGHT_F32), diff


def test_reference_e2e_case(ctx):
    # tests/e2e.rs:188-217: (128, 256, 512), a = (i % 13) / 13 - 0.5, b = (i % 11) / 11 - 0.5, max relative error < 0.02
    m, n, k = 128, 256, 512
    a = O.bf16_bits(((np.arange(m * k) % 13).astype(np.float32) / np.float32(13.0) - np.float32(0.5)).reshape(m, k))
    b = O.bf16_bits(((np.arange(n * k) % 11).astype(np.float32) / np.float32(11.0) - np.float32(0.5)).reshape(n, k))
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    dg.bf16_gemm_nt_dev(ctx, dg.Bf16Tensor(dev(a, torch.bfloat16), m, k), dg.Bf16Tensor(dev(b, torch.bfloat16), n, k), out, n)
    ctx.sync()
    got, want = to_f32(out), O.ref_bf16_gemm_nt(a, b)
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1.0)
    assert rel.max() < 0.02
    assert O.calc_diff(got, want) <= TIGHT_BF16


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (1, 64, 256), (300, 456, 1032), (129, 72, 392), (512, 2112, 2048)])
def test_bf16_gemm_shapes(ctx, m, n, k):
    run(ctx, m, n, k, seed=m + n)


@pytest.mark.parametrize("ctas", [1, 2])
@pytest.mark.parametrize("block_n", [64, 128, 224, 256])
def test_bf16_gemm_tiles(ctx, ctas, block_n, monkeypatch):
    monkeypatch.setenv("DG_BLOCK_N", str(block_n))
    monkeypatch.setenv("DG_CTAS", str(ctas))
    run(ctx, 600, 1000, 1160, seed=block_n + ctas)
    run(ctx, 600, 1000, 1160, out_kind=1, seed=block_n + ctas)


def test_bf16_gemm_epilogues_and_pitches(ctx, monkeypatch):
    run(ctx, 256, 384, 1024, out_kind=1, alpha=0.25)
    run(ctx, 256, 384, 1024, out_kind=0, alpha=3.0, ld_pad=8)
    monkeypatch.setenv("DG_SPLITS", "3")                    # K ranges + reduce pass
    run(ctx, 128, 512, 4608, seed=3)
    monkeypatch.delenv("DG_SPLITS")
    # D += A.B^T
    m, n, k = 200, 320, 768
    a, b = randn_bf16(m, k, seed=71), randn_bf16(n, k, seed=72)
    base = torch.randn((m, n), device="cuda") * 20
    d = base.clone()
    dg.bf16_gemm_dev(ctx, dev(a, torch.bfloat16), k, m, dev(b, torch.bfloat16), k, n, k, dg.Sm100Out.F32(d, n), dg.Sm100Epilogue(accumulate=True))
    ctx.sync()
    assert O.calc_diff(to_f32(d), O.ref_bf16_gemm_nt(a, b, threads=O.max_threads()) + to_f32(base)) <= TIGHT_F32


def test_bf16_gemm_full_size_sampled(ctx):
    run(ctx, 4096, 7168, 4096, seed=9)


def test_bf16_gemm_argument_errors(ctx):
    a = torch.zeros((128, 512), dtype=torch.bfloat16, device="cuda")
    d = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(dg.DgError) as e:
        dg.bf16_gemm_dev(ctx, a, 512, 128, a, 512, 128, 100, dg.Sm100Out.Bf16(d, 128))       # k % 8
    assert e.value.kind == "Shape"
    with pytest.raises(dg.DgError) as e:
        dg.bf16_gemm_dev(ctx, a, 256, 128, a, 512, 128, 512, dg.Sm100Out.Bf16(d, 128))       # ld < k
    assert e.value.kind == "Shape"
    d8 = torch.zeros((128, 128), dtype=torch.uint8, device="cuda")
    sfd = torch.zeros(128, dtype=torch.int32, device="cuda")
    with pytest.raises(dg.DgError) as e:
        dg.bf16_gemm_dev(ctx, a, 512, 128, a, 512, 128, 512, dg.Sm100Out.Fp8(d8, 128, sfd))
    assert e.value.kind == "Unsupported"
