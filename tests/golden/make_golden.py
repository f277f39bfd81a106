"""Generates the golden fixtures of this directory from the CPU oracle (run from the repo root:
`python tests/golden/make_golden.py`).  The reference crate is Rust and cannot be run in this
environment, so the vectors come from the C restatement of its reference.rs, which is itself
pinned to the reference's known-answer tests.

fp8_gemm_128x256x512.npz -- the CPU-runnable benchmark case: bf16 N(0,1) inputs (seeds 1001 / 2001)
quantised to e4m3 with UE8M0 scales (A per 1x128, B per 128x128 tile), and the f32 output of the
scalar restatement of ref_fp8_gemm_nt (reference.rs:85-114) on those bytes.
fp8_gemm_f32scale_128x256x512.npz -- the same case as the benchmark contract words it: e4m3 with f32 scales amax / 448, A per
1x128, B per 128x128 tile (scales with mantissas), and the f32 output of ref_fp8_gemm_nt on those bytes and scales.
mxfp4_8x8x128.npz -- the modular-pattern case of tests/unit.rs:90-158 through the reference-CPU
MXFP4 rule and mxfp4_gemm_reference (reference.rs:293-329).
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    m, n, k = 128, 256, 512
    a_bits = O.bf16_bits(np.random.default_rng(1001).standard_normal((m, k)).astype(np.float32))
    b_bits = O.bf16_bits(np.random.default_rng(2001).standard_normal((n, k)).astype(np.float32))
    aq, a_exp = O.quantize_fp8_ue8m0_blocks(a_bits, k, 1)
    bq, b_exp = O.quantize_fp8_ue8m0_blocks(b_bits, k, 128)
    sfa, sfb = O.exps_to_f32(a_exp), O.exps_to_f32(b_exp)
    out = O.ref_fp8_gemm_nt(aq, sfa, bq, sfb)
    np.savez_compressed(os.path.join(HERE, "fp8_gemm_128x256x512.npz"), a=aq, b=bq, sfa=sfa, sfb=sfb,
                        a_sf_packed=O.transform_sf1d_packed(sfa, k, 128), b_sf_packed=O.transform_sf2d_packed(sfb, n, k),
                        out=out)
    m, n, k = 128, 256, 512
    aq, sfa = O.quantize_fp8_f32scale(O.bf16_to_f32_array(a_bits), 1)
    bq, sfb = O.quantize_fp8_f32scale(O.bf16_to_f32_array(b_bits), 128)
    np.savez_compressed(os.path.join(HERE, "fp8_gemm_f32scale_128x256x512.npz"), a=aq, b=bq, sfa=sfa, sfb=sfb,
                        out=O.ref_fp8_gemm_nt(aq, sfa, bq, sfb))
    m, n, k = 8, 8, 128
    a = np.array([[(((i * 13 + j * 7) % 17) - 8.0) / 8.0 for j in range(k)] for i in range(m)], np.float32)
    b = np.array([[(((i * 11 + j * 5) % 19) - 9.0) / 9.0 for j in range(k)] for i in range(n)], np.float32)
    aq, asf = O.cast_bf16_to_fp4_packed_sf(O.bf16_bits(a), k, 1, O.SF_RULE_REFERENCE_CPU)
    bq, bsf = O.cast_bf16_to_fp4_packed_sf(O.bf16_bits(b), k, 1, O.SF_RULE_REFERENCE_CPU)
    np.savez_compressed(os.path.join(HERE, "mxfp4_8x8x128.npz"), a=aq, b=bq, a_sf=asf, b_sf=bsf,
                        out=O.mxfp4_gemm_reference(aq, asf, m, bq, bsf, n, k))


if __name__ == "__main__":
    main()
