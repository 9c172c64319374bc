// Shared device helpers of the glue kernels (sm_100a).
//
// Arithmetic rule of this library: every value a kernel stores is produced by IEEE-754 operations with round-to-nearest
// (the __f*_rn intrinsics are never contracted or reassociated by the compiler; the translation units are also built
// with -fmad=false), so a result does not depend on the approximate special-function unit and can be restated
// operation by operation on a CPU. The reference leaves expf, rsqrtf, powf and cosf / sinf to its device library;
// here they are the explicit sequences cam_expf, cam_rsqrt, cam_powi and cam_sincos below.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CAM_DEV __device__ __forceinline__
#define CAM_FULL 0xffffffffu

// ---- argument refusals of the C entry points (negative; CUDA errors are returned as their positive cudaError_t) --------
#define CAM_OK 0
#define CAM_ERR_ARG (-1)        // a count, size or null pointer the entry does not take
#define CAM_ERR_ALIGN (-2)      // a pointer or stride that is not 16-byte aligned
#define CAM_ERR_SHAPE (-3)      // a row length or head layout outside what the kernels are built for
#define CAM_ERR_CAPACITY (-4)   // more than a fixed-size buffer of the library holds

CAM_DEV float fmul(float a, float b) { return __fmul_rn(a, b); }
CAM_DEV float fadd(float a, float b) { return __fadd_rn(a, b); }
CAM_DEV float fsub(float a, float b) { return __fsub_rn(a, b); }
CAM_DEV float ffma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
CAM_DEV float fdiv(float a, float b) { return __fdiv_rn(a, b); }
// 1 / b correctly rounded: the same bits as fdiv(1.0f, b) (both are the IEEE quotient) in fewer instructions
CAM_DEV float frcp(float b) { return __frcp_rn(b); }

// exp(a), a clamped to [-87, 88]: n = rint(a log2 e) through the 1.5 * 2^23 constant, r = a - n ln 2 in two fma steps,
// a degree-6 polynomial, n added to the exponent field.
CAM_DEV float cam_expf(float a) {
    a = fminf(fmaxf(a, -87.0f), 88.0f);
    const float t = ffma(a, 0x1.715476p+0f, 12582912.0f);
    const float n = fsub(t, 12582912.0f);
    float r = ffma(n, -0x1.62e430p-1f, a);
    r = ffma(n, 0x1.05c610p-29f, r);
    float p = 0x1.687b46p-10f;
    p = ffma(p, r, 0x1.123bdcp-7f);
    p = ffma(p, r, 0x1.555b5cp-5f);
    p = ffma(p, r, 0x1.55548ep-3f);
    p = ffma(p, r, 0x1.fffff8p-2f);
    p = ffma(p, r, 1.0f);
    p = ffma(p, r, 1.0f);
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}
// the reference's gg_silu, x / (1 + expf(-x)) (kernels/k3_gguf_ops.h:53), with an IEEE division
CAM_DEV float cam_silu(float x) { return fdiv(x, fadd(1.0f, cam_expf(-x))); }
// 1 / sqrt(v): IEEE square root then IEEE division
CAM_DEV float cam_rsqrt(float v) { return frcp(__fsqrt_rn(v)); }
// base^e (integer e >= 0) by binary exponentiation in binary64, rounded once to binary32
CAM_DEV float cam_powi(float base, int e) {
    double b = (double)base, p = 1.0;
    while (e) { if (e & 1) p = __dmul_rn(p, b); b = __dmul_rn(b, b); e >>= 1; }
    return __double2float_rn(p);
}
// sin, cos of theta (|theta| < 2^22): n = rint(theta 2/pi), r = theta - n pi/2 in three fma steps, polynomials on
// [-pi/4, pi/4], quadrant from n's two low bits
CAM_DEV void cam_sincos(float theta, float & sn, float & cs) {
    const float t = ffma(theta, 0x1.45f306p-1f, 12582912.0f);
    const float n = fsub(t, 12582912.0f);
    const uint32_t q = __float_as_uint(t) & 3u;
    float r = ffma(n, -0x1.921fb6p+0f, theta);
    r = ffma(n, 0x1.777a5cp-25f, r);
    r = ffma(n, 0x1.ee59dap-50f, r);
    const float z = fmul(r, r);
    float ps = -0x1.99518cp-13f;
    ps = ffma(ps, z, 0x1.11076ep-7f);
    ps = ffma(ps, z, -0x1.555546p-3f);
    const float s = ffma(fmul(r, z), ps, r);
    float pc = 0x1.994222p-16f;
    pc = ffma(pc, z, -0x1.6c08c4p-10f);
    pc = ffma(pc, z, 0x1.55553ep-5f);
    pc = ffma(pc, z, -0.5f);
    const float c = ffma(z, pc, 1.0f);
    const float s0 = (q & 1u) ? c : s, c0 = (q & 1u) ? s : c;
    sn = (q & 2u) ? -s0 : s0;
    cs = ((q + 1u) & 2u) ? -c0 : c0;
}

// ---- two fp32 operations in one instruction (sm_100: fma / mul / add .f32x2 on a 64-bit register pair) ---------------------------------
// Each half is the IEEE round-to-nearest operation of the scalar instruction (no flush to zero), so a packed statement stores the
// bits of the two scalar statements it stands for; what changes is the instruction count of a kernel that the issue rate bounds.
typedef unsigned long long f32x2;
CAM_DEV f32x2 pk2(float lo, float hi) { f32x2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
CAM_DEV float lo2(f32x2 v) { float a; asm("mov.b64 {%0, _}, %1;" : "=f"(a) : "l"(v)); return a; }
CAM_DEV float hi2(f32x2 v) { float b; asm("mov.b64 {_, %0}, %1;" : "=f"(b) : "l"(v)); return b; }
CAM_DEV f32x2 mul2(f32x2 a, f32x2 b) { f32x2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
CAM_DEV f32x2 sub2(f32x2 a, f32x2 b) { f32x2 r; asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
CAM_DEV f32x2 add2(f32x2 a, f32x2 b) { f32x2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
CAM_DEV f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { f32x2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
// The rounded product where a packed addition or subtraction consumes it: the assembler contracts mul.rn.f32x2 followed by
// add / sub.rn.f32x2 into one packed fma (seen on this toolchain: t = v inv = 63.5 exactly, t - 63 came out as 0.49999997, the
// unrounded product's; a b + (-0) as an fma is simplified to the product and contracted all the same). The scalar mul.rn is never
// contracted, so the two products are scalar and packed afterwards.
CAM_DEV f32x2 prod2(f32x2 a, f32x2 b) { return pk2(fmul(lo2(a), lo2(b)), fmul(hi2(a), hi2(b))); }

// ---- fp16 <-> fp32 (the widening is exact; the narrowing rounds to nearest even) --------------------------------------------
CAM_DEV float2 h2_to_f2(uint32_t v) { return __half22float2(*reinterpret_cast<const __half2 *>(&v)); }
CAM_DEV uint32_t f2_to_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
CAM_DEV uint16_t f_to_h(float a) { return __half_as_ushort(__float2half_rn(a)); }

// ---- fp32 -> bf16, round to nearest even, two at a time (lo in the low half) ---------------------------------------------------
// The reference's integer statements, u + 0x7fff + ((u >> 16) & 1), are IEEE round-to-nearest-even for every number, which is what
// the conversion instruction does. For a NaN operand the integer statements decide the bits: NANQ true: 0x7fc0 (the training
// line's f2bf, kernels/actq.hip:23-28, kernels/core.hip); false: the carry may turn a NaN into an infinity (prefill_glue's to_bf16).
// The false form is for bits a caller stored (a plain conversion of an input). A NaN this device COMPUTED is 0x7fffffff, which the
// integer statements would carry into 0x8000, a zero, where the reference's hardware returns the operand's quieted payload (0x7fc0 for
// the usual NaN) that they keep a NaN: computed values under prefill_glue's rule therefore use the true form, so a NaN stays a NaN.
template <bool NANQ> CAM_DEV uint32_t bf16_soft(float f) {
    uint32_t u = __float_as_uint(f);
    if (NANQ && (u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0u;
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}
template <bool NANQ> CAM_DEV uint32_t bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    if (NANQ) {      // (two predicated selects, no branch: a branch per pair kept the compiler from batching a row's loads and stores)
        if (lo != lo) r = (r & 0xffff0000u) | 0x7fc0u;
        if (hi != hi) r = (r & 0x0000ffffu) | 0x7fc00000u;
    } else if (lo != lo || hi != hi) r = bf16_soft<NANQ>(lo) | (bf16_soft<NANQ>(hi) << 16);
    return r;
}

// cam_expf of two values: the same statements, the fma chain two values per instruction (clamp and exponent insertion stay per value)
CAM_DEV f32x2 cam_expf2(float a0, float a1) {
    a0 = fminf(fmaxf(a0, -87.0f), 88.0f); a1 = fminf(fmaxf(a1, -87.0f), 88.0f);
    const f32x2 a = pk2(a0, a1), magic = pk2(12582912.0f, 12582912.0f);
    const f32x2 t = fma2(a, pk2(0x1.715476p+0f, 0x1.715476p+0f), magic);
    const f32x2 n = sub2(t, magic);
    f32x2 r = fma2(n, pk2(-0x1.62e430p-1f, -0x1.62e430p-1f), a);
    r = fma2(n, pk2(0x1.05c610p-29f, 0x1.05c610p-29f), r);
    f32x2 p = pk2(0x1.687b46p-10f, 0x1.687b46p-10f);
    p = fma2(p, r, pk2(0x1.123bdcp-7f, 0x1.123bdcp-7f));
    p = fma2(p, r, pk2(0x1.555b5cp-5f, 0x1.555b5cp-5f));
    p = fma2(p, r, pk2(0x1.55548ep-3f, 0x1.55548ep-3f));
    p = fma2(p, r, pk2(0x1.fffff8p-2f, 0x1.fffff8p-2f));
    const f32x2 one = pk2(1.0f, 1.0f);
    p = fma2(p, r, one);
    p = fma2(p, r, one);
    return pk2(__uint_as_float(__float_as_uint(lo2(p)) + (__float_as_uint(lo2(t)) << 23)), __uint_as_float(__float_as_uint(hi2(p)) + (__float_as_uint(hi2(t)) << 23)));
}

// ---- 128-bit global accesses ------------------------------------------------------------------------------------------
CAM_DEV uint4 ldg128(const void * p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }          // read-only data
CAM_DEV uint4 ld128(const void * p) { return *reinterpret_cast<const uint4 *>(p); }                 // data this kernel also writes
CAM_DEV void st128(void * p, uint4 v) { *reinterpret_cast<uint4 *>(p) = v; }
CAM_DEV void st64(void * p, uint2 v) { *reinterpret_cast<uint2 *>(p) = v; }
// 256-bit accesses (sm_100: one request per lane covers a whole 32-byte sector; two 16-byte stores at a 32-byte lane stride write every
// sector of the warp's span twice, half at a time, and the second level sees twice the write requests). p 32-byte aligned.
CAM_DEV void st256_cs(float * p, float4 a, float4 b) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w), "f"(b.x), "f"(b.y), "f"(b.z),
                 "f"(b.w) : "memory");
}
CAM_DEV void st256_cs(void * p, uint4 a, uint4 b) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z),
                 "r"(b.w) : "memory");
}
CAM_DEV void st256(void * p, uint4 a, uint4 b) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z),
                 "r"(b.w) : "memory");
}
CAM_DEV void ldg256(const void * p, uint4 & a, uint4 & b) {          // read-only data, 32-byte aligned
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p));
}
// eight floats at p: one 256-bit store when `wide` (p 32-byte aligned), else two 128-bit ones
CAM_DEV void st8f_cs(float * p, float4 a, float4 b, bool wide) {
    if (wide) st256_cs(p, a, b);
    else { __stcs(reinterpret_cast<float4 *>(p), a); __stcs(reinterpret_cast<float4 *>(p) + 1, b); }
}
static inline bool cam_aligned32(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }
CAM_DEV void st128_stream(void * p, uint4 v) { __stcs(reinterpret_cast<uint4 *>(p), v); }           // written once, not re-read here
CAM_DEV void st64_stream(void * p, uint2 v) { __stcs(reinterpret_cast<uint2 *>(p), v); }

// ---- 8 consecutive values of a row as fp32 (fp32 or fp16 storage), and one value -----------------------------------------
template <typename T> struct Load8;
template <> struct Load8<float> {
    static CAM_DEV void get(const float * p, float (&f)[8]) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static CAM_DEV float one(const float * p) { return __ldg(p); }
};
template <> struct Load8<uint16_t> {
    static CAM_DEV void get(const uint16_t * p, float (&f)[8]) {
        const uint4 v = ldg128(p);
        const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), c = h2_to_f2(v.z), e = h2_to_f2(v.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = e.x; f[7] = e.y;
    }
    static CAM_DEV float one(const uint16_t * p) { return __half2float(__ushort_as_half(__ldg(p))); }
};

// ---- the special-function unit's approximations, used only where a kernel proves the stored bytes do not depend on them ---
// (.ftz: a denormal exponent argument counts as 0 and a denormal 2^a as 0; both are below 1e-38 beside the 1 they are added to)
CAM_DEV float ex2_approx(float a) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }
CAM_DEV float rcp_approx(float a) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a)); return r; }


// bf16(silu(g)) for N values without the exact statements' two divisions and polynomial where that provably gives the same bits: the
// special-function evaluation s^ = g rcp(1 + ex2(-g log2 e)) is within 1.35e-6 |s| of cam_silu(g) for g >= -8 and 3e-38 <= |g| < 3e38
// (the analysis at the fused SwiGLU + Q8_1 kernel, csrc/swiglu_q8.cu, without its last product). If s^ (1 - 1.55e-6) and s^ (1 + 1.55e-6) round to the same
// bf16, no rounding boundary and no tie lies in the interval that holds cam_silu(g), and that bf16 is its rounding. The conditions are
// ranges are gathered over the N values (minimum, largest and smallest magnitude) and tested once: an item with a value outside the
// range, a zero or an infinity evaluates the exact statements for all N, a pair with an interval that holds a boundary (1 value in
// about 1400) for its two. A NaN gate passes the gathered tests (minimum and maximum skip it) and gives the conversion's NaN, 0x7fff:
// the callers' NaN test of the result sends such an item to the exact statements too. out[k] = values 2 k (low half), 2 k + 1.
// Returns the pairs to redo with the exact statements, bit k for out[k] (0: none): a pair whose two roundings differ, every pair
// when a range test fails. (A warp runs the redo when one of its lanes asks: per pair that is 1 step in 22, per item it was 1 in 6.)
template <int N> CAM_DEV uint32_t silu_bf16_fast(const float (&g)[N], uint32_t (&out)[N / 2]) {
    float gmin = g[0], amax = fabsf(g[0]), amin = fabsf(g[0]);
    uint32_t redo = 0;
    const f32x2 nl2 = pk2(-0x1.715476p+0f, -0x1.715476p+0f), one2 = pk2(1.0f, 1.0f), up2 = pk2(0x1.00001ap+0f, 0x1.00001ap+0f), dn2 = pk2(0x1.ffffccp-1f, 0x1.ffffccp-1f);
#pragma unroll
    for (int k = 0; k < N; k += 2) {                   // (two values per instruction: the same roundings as one by one)
        const f32x2 g2 = pk2(g[k], g[k + 1]);
        const f32x2 a2 = mul2(g2, nl2);
        const f32x2 den = add2(one2, pk2(ex2_approx(lo2(a2)), ex2_approx(hi2(a2))));
        const f32x2 s2 = mul2(g2, pk2(rcp_approx(lo2(den)), rcp_approx(hi2(den))));
        const f32x2 hi_ = mul2(s2, up2), lo_ = mul2(s2, dn2);
        uint32_t lo;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out[k >> 1]) : "f"(hi2(hi_)), "f"(lo2(hi_)));
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(hi2(lo_)), "f"(lo2(lo_)));
        if (out[k >> 1] != lo) redo |= 1u << (k >> 1);
        if (k) { gmin = fminf(gmin, g[k]); amax = fmaxf(amax, fabsf(g[k])); amin = fminf(amin, fabsf(g[k])); }
        gmin = fminf(gmin, g[k + 1]); amax = fmaxf(amax, fabsf(g[k + 1])); amin = fminf(amin, fabsf(g[k + 1]));
    }
    return (gmin >= -8.0f && amax < 3.0e38f && amin >= 3.0e-38f) ? redo : (1u << (N / 2)) - 1u;
}
CAM_DEV bool bf16_pair_has_nan(uint32_t w) { return (w & 0x7fffu) > 0x7f80u || (w & 0x7fff0000u) > 0x7f800000u; }

// ---- the reference's 256-thread sum on a warp: thread tid owns elements tid + 256 j (an fma chain over j), the 32 lanes of a wave
// add by the xor butterfly 16, 8, 4, 2, 1, the 8 wave sums are added in order. Here lane l holds elements 128 m + 4 l + c, i.e.
// thread 128 (m & 1) + 4 l + c with j = m >> 1: accumulator a[c + 4 (m & 1)]; partners 16, 8, 4 are lanes l ^ 4, 2, 1, partners 2, 1
// are inside the lane; wave w is lanes 8 (w & 3) .. with b = w >> 2.
// a[c + 4 b] (c < 4, b < 2). Returns the workgroup total (every lane).
CAM_DEV float ref_total_f32(float (&a)[8], int lane) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < 8; k++) a[k] = fadd(a[k], __shfl_xor_sync(CAM_FULL, a[k], o));
    float P[2];
#pragma unroll
    for (int b = 0; b < 2; b++) {
        const float t0 = fadd(a[4 * b + 0], a[4 * b + 2]), t1 = fadd(a[4 * b + 1], a[4 * b + 3]);   // partner 2
        P[b] = fadd(t0, t1);                                                                        // partner 1
    }
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot = fadd(tot, __shfl_sync(CAM_FULL, P[w >> 2], 8 * (w & 3)));    // wave w: lanes 8 (w & 3) .., b = w >> 2
    return tot;
}

// ref_total_f32 on accumulator pairs (a2[c] = accumulators 2 c, 2 c + 1 of a[8]): the butterfly's additions two per instruction
CAM_DEV float ref_total_f32_pairs(f32x2 (&a2)[4], int lane) {            // a2[c] = accumulators 2 c, 2 c + 1 of ref_total_f32's a[8]
#pragma unroll
    for (int o = 4; o > 0; o >>= 1)
#pragma unroll
        for (int c = 0; c < 4; c++) a2[c] = add2(a2[c], pk2(__shfl_xor_sync(CAM_FULL, lo2(a2[c]), o), __shfl_xor_sync(CAM_FULL, hi2(a2[c]), o)));
    const f32x2 t0 = add2(a2[0], a2[1]), t1 = add2(a2[2], a2[3]);        // partner 2: (a0 + a2, a1 + a3), (a4 + a6, a5 + a7)
    const float P0 = fadd(lo2(t0), hi2(t0)), P1 = fadd(lo2(t1), hi2(t1));   // partner 1
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot = fadd(tot, __shfl_sync(CAM_FULL, w < 4 ? P0 : P1, 8 * (w & 3)));
    return tot;
}
// two such sums at once, a[] and b[]: in the first butterfly stage a lane keeps one of the two (lanes with bit 2 clear a's, the others b's) and
// sends the other, so each stage costs one set of shuffles for both; the additions and their order are ref_total_f32's. Returns the
// total of the lane's own sum (a's where lane & 4 is clear).
CAM_DEV float ref_total_f32_two(const f32x2 (&a)[4], const f32x2 (&b)[4], int lane) {
    const bool up = (lane & 4) != 0;
    f32x2 v[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const f32x2 keep = up ? b[c] : a[c], send = up ? a[c] : b[c];
        v[c] = add2(keep, pk2(__shfl_xor_sync(CAM_FULL, lo2(send), 4), __shfl_xor_sync(CAM_FULL, hi2(send), 4)));
    }
#pragma unroll
    for (int o = 2; o > 0; o >>= 1)
#pragma unroll
        for (int c = 0; c < 4; c++) v[c] = add2(v[c], pk2(__shfl_xor_sync(CAM_FULL, lo2(v[c]), o), __shfl_xor_sync(CAM_FULL, hi2(v[c]), o)));
    const f32x2 t0 = add2(v[0], v[1]), t1 = add2(v[2], v[3]);
    const float P0 = fadd(lo2(t0), hi2(t0)), P1 = fadd(lo2(t1), hi2(t1));
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot = fadd(tot, __shfl_sync(CAM_FULL, w < 4 ? P0 : P1, 8 * (w & 3) + (lane & 4)));
    return tot;
}
// the same sum for fp16 rows, where lane l holds the 8 halves at 8 l + 256 m: accumulator c is thread 8 l + c with j = m; wave l >> 2,
// wave lane 8 (l & 3) + c: partners 16, 8 are lanes l ^ 2, l ^ 1; partners 4, 2, 1 are inside the lane
CAM_DEV float ref_total_f16(float (&a)[8], int lane) {
#pragma unroll
    for (int o = 2; o > 0; o >>= 1)
#pragma unroll
        for (int k = 0; k < 8; k++) a[k] = fadd(a[k], __shfl_xor_sync(CAM_FULL, a[k], o));
    const float u0 = fadd(a[0], a[4]), u1 = fadd(a[1], a[5]), u2 = fadd(a[2], a[6]), u3 = fadd(a[3], a[7]);   // partner 4
    const float P = fadd(fadd(u0, u2), fadd(u1, u3));                                                           // partners 2, 1
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot = fadd(tot, __shfl_sync(CAM_FULL, P, 4 * w));
    return tot;
}

// ---- cp.async (16 bytes per thread, L2 only) with commit / wait groups --------------------------------------------------------
CAM_DEV void cp_async16(void * smem, const void * gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
CAM_DEV void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> CAM_DEV void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

static inline bool cam_aligned16(const void * p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// multiprocessors of the current device (cached per device)
int cam_sm_count();

// A grid of looping blocks: `over` times as many as the device holds at once, capped by the work. `want` = blocks that would each get one
// unit of work. over = 1: exactly the resident blocks (what a kernel whose blocks wait for one another needs). Streaming kernels mostly
// run faster with over = 8: resident blocks that loop stay in step (all load, then all compute, then all store), while a finished
// block's successor starts with its loads at once and the phases drift apart (measured per kernel; the launchers say which).
// resident blocks per multiprocessor of a kernel at a block size and dynamic shared-memory size (cached per device)
int cam_blocks_per_sm(const void * kernel, int threads, size_t smem);

template <typename K>
static inline int cam_resident_grid(K kernel, int threads, size_t smem, long want, int over = 1) {
    const int per_sm = cam_blocks_per_sm(reinterpret_cast<const void *>(kernel), threads, smem);
    const long cap = (long)cam_sm_count() * per_sm * over;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

// A grid of looping blocks sized by the work per block: each block gets about `iters` units (at least the resident blocks, at most
// one block per unit). The SwiGLU + Q8_1 kernels run fastest at 7 to 8 units per block whatever the batch (65536 x 25600 values:
// 1229 us, against 1268 us with 8 x the resident blocks, 1289 us with a block per unit and 1309 us with the resident blocks alone).
template <typename K>
static inline int cam_iter_grid(K kernel, int threads, size_t smem, long want, int iters) {
    const long resident = cam_resident_grid(kernel, threads, smem, want);
    const long by_iters = (want + iters - 1) / iters;
    const long g = by_iters > resident ? by_iters : resident;
    return (int)(g > 0x7fffffffL ? 0x7fffffffL : g);
}

// One-time, per device: a kernel's opt-in to more dynamic shared memory than the default limit. `done` is the caller's static word,
// one bit per device ordinal: after the first launch on a device the attribute call (a driver call) is skipped.
template <typename Kn> static inline cudaError_t cam_allow_smem(Kn kernel, size_t bytes, unsigned long long & done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && ((__atomic_load_n(&done, __ATOMIC_ACQUIRE) >> dev) & 1ull)) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && dev >= 0 && dev < 64) __atomic_fetch_or(&done, 1ull << dev, __ATOMIC_RELEASE);
    return e;
}

// csrc/add_rms.cu: the warp-per-row path of the hyper-connection norms (CAM_ERR_SHAPE: does not apply to this call)
int cam_rms_rows_vec(float * x, const float * w, float * y, void * ybf, float * scl, int R, int wr, float eps, int K, const float * b,
                     const float * inj, int HC, float rs, void * stream, void * yq = nullptr);
