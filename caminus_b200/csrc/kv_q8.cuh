// The Q8_0 KV cache row of the reference (Q8_0 block encode kernels/own_kv_codec.h:31-75; 128-point Hadamard transform
// kernels/own_kv_rot128.h:21-33; CPU reference python/caminus/ref_kv.py), as device functions of the q/k norm + RoPE kernel.
//
// Every head's rotated result is rounded to fp16 and back (the value the F16 cache would hold) and transformed by the orthonormal
// Walsh-Hadamard matrix (butterflies h = 1, 2, .. 64 in that order, then times fp32(1 / sqrt(128))). q heads store fp16 of the
// transform into q16. kv heads store the transformed K as four Q8_0 blocks (fp16 d = amax / 127, q = roundf(x * (1 / d))) and the
// fp16-rounded V, untransformed, as four more, into the cache row pos: [K blocks of all heads | V blocks of all heads], 34 bytes
// per block. A block with a non-finite value or a scale outside fp32 / fp16 range is refused: its bytes are left alone and 2 is
// ORed into *err.
//
// A half-warp holds a head: lane l has dims 4l .. 4l + 3 and 64 + 4l .. 64 + 4l + 3, so butterflies 1, 2 and 64 are inside the lane
// and 4, 8, 16, 32 are lane exchanges; a Q8_0 block of 32 dims is 8 lanes' low or high values.
#pragma once
#include "cam_common.cuh"

CAM_DEV float f16r(float x) { return __half2float(__float2half_rn(x)); }
CAM_DEV bool finite_f(float x) { return fabsf(x) <= 3.402823466e38f; }      // false for inf and NaN

// one Q8_0 block held as 4 values in each of 8 adjacent lanes (l8 = the lane's place among them). Every lane of the warp calls this
// (the reductions are full-warp shuffles); only lanes with store set write.
CAM_DEV void q8_0_store(const float (&v)[4], uint8_t * blk, int l8, int * err, bool store) {
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; c++) amax = fmaxf(amax, finite_f(v[c]) ? fabsf(v[c]) : __int_as_float(0x7f800000));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, o));
    const float d = fdiv(amax, 127.0f);
    const float inv = d != 0.0f ? frcp(d) : 0.0f;                    // (1.0f / d: the IEEE reciprocal is that quotient)
    const __half stored = __float2half_rn(d);
    const bool refuse = !finite_f(amax) || (amax != 0.0f && (d == 0.0f || !finite_f(d) || !finite_f(inv) || !finite_f(__half2float(stored))));
    if (!store) return;
    if (refuse) { if (l8 == 0) atomicOr(err, 2); return; }
    // roundf(t), t = v inv, without the special-function unit's rounding and conversion: t + 1.5 2^23 is t rounded to the nearest integer,
    // ties to even, its two's complement in the sum's low byte (|t| <= 127 (1 + 2^-22) here: every value is a number). roundf differs on
    // exact ties only, and t - rint(t) is exact: a lane that sees |t - rint(t)| = 0.5 takes roundf.
    const f32x2 inv2 = pk2(inv, inv), big2 = pk2(12582912.0f, 12582912.0f);
    const f32x2 ta = prod2(pk2(v[0], v[1]), inv2), tb = prod2(pk2(v[2], v[3]), inv2);      // (prod2: the sums below must see the rounded t)
    const f32x2 sa = add2(ta, big2), sb = add2(tb, big2);
    const f32x2 ea = sub2(ta, sub2(sa, big2)), eb = sub2(tb, sub2(sb, big2));
    uint32_t q[4] = {__float_as_uint(lo2(sa)), __float_as_uint(hi2(sa)), __float_as_uint(lo2(sb)), __float_as_uint(hi2(sb))};
    if (fmaxf(fmaxf(fabsf(lo2(ea)), fabsf(hi2(ea))), fmaxf(fabsf(lo2(eb)), fabsf(hi2(eb)))) >= 0.5f) {
#pragma unroll
        for (int c = 0; c < 4; c++) q[c] = (uint32_t)__float2int_rn(roundf(fmul(v[c], inv)));
    }
    uint16_t * o = reinterpret_cast<uint16_t *>(blk + 2 + 4 * l8);              // (34-byte blocks: 2-byte alignment)
    o[0] = (uint16_t)__byte_perm(q[0], q[1], 0x0040); o[1] = (uint16_t)__byte_perm(q[2], q[3], 0x0040);
    if (l8 == 0) *reinterpret_cast<uint16_t *>(blk) = __half_as_ushort(stored);
}

// x[0..3] = dims 4l .. 4l + 3, x[4..7] = dims 64 + 4l ..: the orthonormal Walsh-Hadamard transform of the half-warp's 128 values
CAM_DEV void hadamard128(float (&x)[8], int l16) {
#pragma unroll
    for (int b = 0; b < 8; b += 4) {                 // h = 1, then h = 2, inside each group of four
        float a0 = fadd(x[b], x[b + 1]), a1 = fsub(x[b], x[b + 1]), a2 = fadd(x[b + 2], x[b + 3]), a3 = fsub(x[b + 2], x[b + 3]);
        x[b] = fadd(a0, a2); x[b + 2] = fsub(a0, a2); x[b + 1] = fadd(a1, a3); x[b + 3] = fsub(a1, a3);
    }
    f32x2 p2[4] = {pk2(x[0], x[1]), pk2(x[2], x[3]), pk2(x[4], x[5]), pk2(x[6], x[7])};      // (two values per instruction below: the same roundings)
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) {               // h = 4, 8, 16, 32: lanes l ^ 1, 2, 4, 8
        const float sg = (l16 & m) ? -1.0f : 1.0f;      // the upper lane of a pair holds partner - own: fma(own, -1, partner), one rounding
        const f32x2 sg2 = pk2(sg, sg);
#pragma unroll
        for (int c = 0; c < 4; c++)
            p2[c] = fma2(p2[c], sg2, pk2(__shfl_xor_sync(CAM_FULL, lo2(p2[c]), m), __shfl_xor_sync(CAM_FULL, hi2(p2[c]), m)));
    }
    const f32x2 r2 = pk2(0x1.6a09e6p-4f, 0x1.6a09e6p-4f);
#pragma unroll
    for (int c = 0; c < 2; c++) {                    // h = 64, then the scale
        const f32x2 a = p2[c], b = p2[2 + c];
        const f32x2 lo = mul2(add2(a, b), r2), hi = mul2(sub2(a, b), r2);
        x[2 * c] = lo2(lo); x[2 * c + 1] = hi2(lo); x[4 + 2 * c] = lo2(hi); x[4 + 2 * c + 1] = hi2(hi);
    }
}
