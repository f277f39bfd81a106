// silu(gate) * up in reproducible f32 steps, shared by the activation quantiser and the fused gate/up GEMM epilogue.
#pragma once
#include "dg_ptx.cuh"

namespace dg {

// bf16(silu(g) * u) as f32, silu(g) = g / (1 + exp(-g)).  exp is spelled out in correctly rounded f32 operations so
// that a host restatement with fmaf gives the same bits (within 3e-6 of exp, far inside a bf16 rounding step):
//   gate clamped to [-87, 30] (beyond 30, 1 + exp(-g) rounds to 1);
//   n = rint(-g log2 e) read from the low mantissa bits of fma(g, -log2 e, 1.5 * 2^23);
//   r = -g - n ln 2 (ln 2 in two parts), exp(r) - 1 as a degree-5 Taylor polynomial on |r| <= ln2/2;
//   exp(-g) = (exp(r)) * 2^n by adding n to the exponent field;
//   1 / (1 + exp(-g)) by three Newton steps x <- x (2 - d x) from the exponent-flip estimate 0x7EF311C7 - bits(d)
//   (relative error 0.12 -> 4e-8; no special-function unit, no branches); silu = g * that; gates below -87 give 0.
// Two elements at a time: the f32 arithmetic goes through the packed f32x2 instructions of sm_100 (two IEEE
// operations per instruction, same results as the scalar forms), halving the arithmetic instruction count.
DG_DEVICE float2 silu_mul_bf16x2(float2 g, float2 u) {
    const float2 gc = make_float2(fminf(fmaxf(g.x, -87.0f), 30.0f), fminf(fmaxf(g.y, -87.0f), 30.0f));
    const float2 magic = make_float2(12582912.0f, 12582912.0f);
    const float2 t = __ffma2_rn(gc, make_float2(-1.44269504f, -1.44269504f), magic);
    const float2 n = __fadd2_rn(t, make_float2(-12582912.0f, -12582912.0f));
    const float2 ngc = make_float2(-gc.x, -gc.y);
    float2 r = __ffma2_rn(n, make_float2(-0.693145752f, -0.693145752f), ngc);
    r = __ffma2_rn(n, make_float2(-1.42860677e-6f, -1.42860677e-6f), r);
    float2 q = __ffma2_rn(make_float2(1.0f / 120.0f, 1.0f / 120.0f), r, make_float2(1.0f / 24.0f, 1.0f / 24.0f));
    q = __ffma2_rn(q, r, make_float2(1.0f / 6.0f, 1.0f / 6.0f));
    q = __ffma2_rn(q, r, make_float2(0.5f, 0.5f));
    q = __ffma2_rn(q, __fmul2_rn(r, r), r);
    const float2 one = make_float2(1.0f, 1.0f), two = make_float2(2.0f, 2.0f);
    const float2 s = __fadd2_rn(q, one);
    const float2 e = make_float2(__uint_as_float(__float_as_uint(s.x) + (__float_as_uint(t.x) << 23)),
                                 __uint_as_float(__float_as_uint(s.y) + (__float_as_uint(t.y) << 23)));
    const float2 d = __fadd2_rn(one, e);
    const float2 nd = make_float2(-d.x, -d.y);
    float2 x = make_float2(__uint_as_float(0x7EF311C7u - __float_as_uint(d.x)), __uint_as_float(0x7EF311C7u - __float_as_uint(d.y)));
    x = __fmul2_rn(x, __ffma2_rn(nd, x, two));
    x = __fmul2_rn(x, __ffma2_rn(nd, x, two));
    x = __fmul2_rn(x, __ffma2_rn(nd, x, two));
    float2 silu = __fmul2_rn(g, x);
    silu.x = g.x < -87.0f ? 0.0f : silu.x;   // |g exp(g)| < 2e-36 below -87
    silu.y = g.y < -87.0f ? 0.0f : silu.y;
    const float2 act = __fmul2_rn(silu, u);
    const uint32_t packed = pack_bf16x2(act.x, act.y);
    return make_float2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xFFFF0000u));
}

}  // namespace dg
