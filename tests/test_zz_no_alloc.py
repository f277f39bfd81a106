"""The allocation-free contiguous grouped GEMM (dg_m_grouped_fp8_fp4_gemm_contiguous_static).

Collected last on purpose: it exercises an extra entry point for hosts that must not allocate device
memory while running, and a failure here should not hide results of the main parity tests.  The
entry point is called through the C ABI twice in a row on one stream; both results must equal, bit
for bit, what the context-based entry point produces for the same inputs.  The second call uses
fewer groups than the first, so entries of the first call's group-end table are still sitting in the
library's built-in scratch when it starts.
"""
import numpy as np
import pytest
import torch

import deepgemm_rust_b200 as dg
from tests.helpers import dev, fp8_operand_1d, fp8_operand_2d

pytestmark = pytest.mark.gpu


def _layout(sizes, alignment=128):
    idx = []
    for g, s in enumerate(sizes):
        idx += [g] * s + [-1] * ((-s) % alignment)
    return np.array(idx, np.int32)


def _case(sizes, n, k, seed):
    m_idx = _layout(sizes)
    m_total, groups = len(m_idx), len(sizes)
    _, aq, asf = fp8_operand_1d(m_total, k, seed)
    _, bq, bsf, _ = fp8_operand_2d(groups * n, k, seed + 1, groups)
    a = dg.LpOperand(dev(aq), dev(asf), m_total, k, k)
    b = dg.LpOperand(dev(bq), dev(bsf), groups * n, k, k)
    return a, b, dev(m_idx), m_idx, groups, m_total


def test_static_entry_point_matches_context_entry_point_twice():
    ctx = dg.DgContext(0)
    stream = torch.cuda.current_stream().cuda_stream
    n, k = 384, 1024
    for sizes, seed in (([130, 0, 64, 257, 1, 128], 71), ([200, 56], 73)):
        a, b, m_idx_dev, m_idx, groups, m_total = _case(sizes, n, k, seed)
        want = torch.full((m_total, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_contiguous_dev(ctx, a, m_idx_dev, b, dg.Sm100Out.Bf16(want, n), groups)
        got = torch.full((m_total, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_contiguous_static_dev(0, stream, a, m_idx_dev, b, dg.Sm100Out.Bf16(got, n), groups)
        ctx.sync()
        valid = torch.from_numpy(np.nonzero(m_idx >= 0)[0]).cuda()
        assert not torch.isnan(got[valid].float()).any()
        assert torch.equal(got[valid].view(torch.int16), want[valid].view(torch.int16))
        # no wait ran out in the kernels of the context-less call (its record lives in the built-in array)
        dg.static_check_status(0, stream)
    ctx.close()


def test_static_entry_point_rejects_too_many_groups():
    a, b, m_idx_dev, _, _, m_total = _case([128], 128, 256, 75)
    out = dg.Sm100Out.Bf16(torch.zeros((m_total, 128), dtype=torch.bfloat16, device="cuda"), 128)
    with pytest.raises(dg.DgError) as e:
        dg.m_grouped_fp8_fp4_gemm_contiguous_static_dev(0, torch.cuda.current_stream().cuda_stream, a, m_idx_dev, b, out,
                                                        dg.STATIC_MAX_GROUPS + 1)
    assert e.value.kind == "Shape" and "4096" in str(e.value)
