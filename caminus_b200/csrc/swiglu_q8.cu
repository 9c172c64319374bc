// SwiGLU and the Q8_1 activation quantiser, fused and unfused.
//
// Reference statements: gg_silu(x) = x / (1 + expf(-x)) (kernels/k3_gguf_ops.h:53); the tape op gg_op_q8_1 with work = 2,
// xi = gg_silu(x) * mul then quantize_q8_1_lane (kernels/k3_gguf_ops.h:55-77), restated in-tree as q8_lane
// (kernels/k3_gguf_ops.h:145-153): amax = max |xi| and sum over the block of 32, d = amax / 127.0f, q = amax == 0 ? 0 :
// roundf(xi / d) with a true division, block = { half d, half sum, int8 qs[32] } = 36 bytes. Unfused forms: q3p_swiglu
// (kernels/q3m_prefill.hip:515-518), gg_silu_mul (kernels/k3_gguf.hip:74-77), gg_quantize_q8_1 (kernels/k3_gguf.hip:29-36).
//
// Mapping of the exact kernel: a thread owns 8 consecutive values (one 16-byte load of fp16 gate and up, or two of fp32), 4 adjacent
// lanes own a block (the fused fast pass further down takes 16 values per thread, 2 lanes per block). amax is order-free; the block sum follows the order of the reference's 8-lane quantiser aq_fill
// (kernels/k3_gguf_ops.h:83-120): (e0 + e1) + (e2 + e3) per group of four, then partners 4, 2, 1 over the 8 groups. A lane
// holds groups 2q and 2q + 1 (q its place in the quad): partner 4 is lane q ^ 2, partner 2 is lane q ^ 1, partner 1 is the
// lane's other group. d and the codes are quantize_q8_1_lane's bits whatever the order.
// A block's 36 bytes are written as 4-byte words: the quad's lanes write 8 codes each, lane 0 also (d, sum).
#include "cam_common.cuh"

namespace {

constexpr int Q8_THREADS = 256;

CAM_DEV int q8_code(float x, float d, float amax) {
    const float v = fdiv(x, d);
    return (amax != 0.0f && fabsf(v) < 127.5f) ? __float2int_rn(roundf(v)) : 0;   // (false for a NaN: code 0)
}

// SWIGLU: xi = silu(g) u; else xi = g. Full blocks [0, nb).
template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(Q8_THREADS) q8_1_kernel(const T * __restrict__ g, const T * __restrict__ u, uint8_t * __restrict__ y,
                                                          long nb) {
    const int lane = threadIdx.x & 31, q = lane & 3;
    const long ngroups = nb * 4;
    const long stride = (long)gridDim.x * Q8_THREADS;
    for (long base = (long)blockIdx.x * Q8_THREADS + (threadIdx.x & ~31); base < ngroups; base += stride) {
        const long gi = base + lane;
        const bool on = gi < ngroups;
        float h[8];
        if (on) {
            Load8<T>::get(g + gi * 8, h);
            if (SWIGLU) {
                float uv[8];
                Load8<T>::get(u + gi * 8, uv);
#pragma unroll
                for (int k = 0; k < 8; k++) h[k] = fmul(cam_silu(h[k]), uv[k]);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; k++) h[k] = 0.0f;
        }
        float amax = fabsf(h[0]);
#pragma unroll
        for (int k = 1; k < 8; k++) amax = fmaxf(amax, fabsf(h[k]));
        amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, 2));
        float sa = fadd(fadd(h[0], h[1]), fadd(h[2], h[3])), sb = fadd(fadd(h[4], h[5]), fadd(h[6], h[7]));
        sa = fadd(sa, __shfl_xor_sync(CAM_FULL, sa, 2)); sb = fadd(sb, __shfl_xor_sync(CAM_FULL, sb, 2));   // partner 4
        sa = fadd(sa, __shfl_xor_sync(CAM_FULL, sa, 1)); sb = fadd(sb, __shfl_xor_sync(CAM_FULL, sb, 1));   // partner 2
        const float sum = fadd(sa, sb);                                                                     // partner 1
        const float d = fdiv(amax, 127.0f);
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            w0 |= (uint32_t)(q8_code(h[k], d, amax) & 0xff) << (8 * k);
            w1 |= (uint32_t)(q8_code(h[4 + k], d, amax) & 0xff) << (8 * k);
        }
        if (on) {
            uint32_t * o = reinterpret_cast<uint32_t *>(y + (gi >> 2) * 36);
            if (q == 0) __stcs(o, f2_to_h2(d, sum));
            __stcs(o + 1 + 2 * q, w0);
            __stcs(o + 2 + 2 * q, w1);
        }
    }
}

// ---- the fused SwiGLU + Q8_1 kernel: a fast pass with proof margins, exact recomputation where a margin is not met --------
//
// The exact statements (cam_silu: a 12-operation exp, two IEEE divisions per value) cost about twice the instructions the
// memory system leaves time for. The fast pass therefore evaluates h^ = g * rcp(1 + ex2(-g log2 e)) * u on the
// special-function unit and quantises with a reciprocal, which is NOT bit-reproducible by itself. It is used only where it
// provably gives the exact statements' bytes. With h the exact value of an element, |h^ - h| <= EPS |h|, EPS = 1.35e-6,
// whenever g >= -8 (and |g| >= 3e-38, which only an fp32 gate can miss): against the true value the fast pass is within 1.02e-6 (the rounding of ex2's argument, 6e-8 |g|, and
// ex2.approx's 2^-22, both scaled by e / (1 + e) <= 1; the rounding of 1 + e; rcp.approx's 2^-23; two products) and the exact
// sequence within 3.2e-7 (2.2 ulp measured over the whole range, and its product). From that:
//   d:     d^ = amax^ / 127 is within 1.53e-6 (< 26 fp32 ulps) of the exact fp32 d. If d^'s low 13 bits are more than 40 away
//          from the fp16 rounding tie (0x1000) and d^ is in fp16's normal range, fp16(d^) = fp16(d): the stored scale is exact.
//   codes: t^ = h^ / d^ is within 3.06e-6 |t| of the exact fp32 quotient t. If t^ (1 - 3.2e-6) and t^ (1 + 3.2e-6) round to the
//          same integer, no rounding boundary and no tie lies in the interval that holds t, and that integer is roundf(t).
//   sum (SUMS): the fast pass adds the h^ in the exact statements' order. Its sum S^ is within 1.95e-6 A of theirs, A = sum |h^| (1.35e-6 A
//          from the values, 3e-7 A from the five levels of fp32 additions of either tree). If S^ - 2.2e-6 A and S^ + 2.2e-6 A round
//          to the same fp16, no fp16 rounding boundary lies in the interval that holds the exact sum: the stored sum is exact.
// A block (32 values) where any of this fails: some g < -8, an interval that holds a rounding boundary, d^ near an fp16
// tie or outside [6.2e-5, 6e4), a sum that is not finite (NaN or infinite input): is recomputed by the whole warp with
// the exact statements, one lane per value. About 2 % of the blocks of Gaussian inputs take that path (4 % with the sum test).
// The stored scale d and the 32 codes are therefore always the exact statements' bytes. With SUMS so is the block sum: all 36 bytes.
// Without it the sum of a block on the fast pass is the fp16 rounding of S^: it can differ from the exact statements' sum by one fp16
// ulp (or by 2e-6 A when the values cancel). The reference reports that field and does not gate it (tests/engine/golden_util.py:145-146).
// The sum test costs a quarter of the throughput (the recomputation of twice as many blocks no longer hides behind the memory system),
// so it is a separate entry.
// One warp-wide step over 16 blocks (512 values) starting at pair `base` (a multiple of 32): 16 values per lane, two lanes per block.
// (With 8 values per lane and four lanes per block the same pass ran at 88 % of the copy bandwidth: the work that does not depend on
// the number of values (loop, indices, margins, ballots, store addresses) was a third of its instructions; spent once per 16 values
// the kernel is memory-bound.) FULL: all 32 lanes have a pair.
// Block sum in aq_fill's order: a lane holds groups 4 q .. 4 q + 3 (q its place in the pair): partner 4 is the other lane, partners 2
// and 1 are the lane's own groups.
// SUMS: also prove the block sum (else it is the fp16 rounding of the fast pass's own sum, within one fp16 ulp of the exact one)
// The margins of the three proofs. fp32 gates: the analytic bound EPS = 1.35e-6 (above). fp16 gates: there are 65 536 of them, so the
// special-function value s^ = g rcp(1 + ex2(-g log2 e)) was compared with the exact statements' silu(g) for EVERY gate >= -8 on this
// architecture: max |s^ - s| / |s| = 5.43e-7 (tests/test_gpu_enumerated.py re-measures it on the device it runs on and fails above
// 5.6e-7); with the two roundings of the product by u, |h^ - h| <= 7.0e-7 |h|. From that, as above with 7.0e-7 for 1.35e-6:
// d^ within 8.8e-7 (15 fp32 ulps) of d: the tie test keeps 24 ulps clear; t^ within 1.76e-6 |t| of t: the two-ended test with
// 1 -+ 2.0e-6; S^ within 1.3e-6 A of the exact sum: the interval test with 1.5e-6 A. Half the margins, half the blocks sent to the
// exact statements.
template <typename T> struct Q8Margins {            // fp32 gates
    static constexpr int TIE = 40;
    static CAM_DEV float hi() { return 0x1.000036p+0f; }      // 1 + 3.2e-6
    static CAM_DEV float lo() { return 0x1.ffff94p-1f; }      // 1 - 3.2e-6
    static CAM_DEV float sum() { return 2.2e-6f; }
};
template <> struct Q8Margins<uint16_t> {            // fp16 gates: the enumerated bound
    static constexpr int TIE = 24;
    static CAM_DEV float hi() { return 0x1.000022p+0f; }      // 1 + 2.03e-6
    static CAM_DEV float lo() { return 0x1.ffffbcp-1f; }      // 1 - 2.03e-6
    static CAM_DEV float sum() { return 1.5e-6f; }
};

// SCALED: the values are silu(g rs), with no second operand (u is not read): the tape op's work = 1, ggml_scale then ggml_silu
template <typename T, bool FULL, bool SUMS, bool SCALED = false>
CAM_DEV void swiglu_q8_step(const T * __restrict__ g, const T * __restrict__ u, uint8_t * __restrict__ y, int base, int npairs, int lane, float rs = 1.0f) {
    const int pi = base + lane, q = lane & 1;
    const bool on = FULL || pi < npairs;
    float gv[16], uv[16], h[16];
    if (on) {
        float t[8];
        Load8<T>::get(g + (size_t)pi * 16, t);
#pragma unroll
        for (int k = 0; k < 8; k++) gv[k] = t[k];
        Load8<T>::get(g + (size_t)pi * 16 + 8, t);
#pragma unroll
        for (int k = 0; k < 8; k++) gv[8 + k] = t[k];
        if (SCALED) {
#pragma unroll
            for (int k = 0; k < 16; k++) { gv[k] = fmul(gv[k], rs); uv[k] = 1.0f; }      // (the product with 1 is exact: h = silu(g rs))
        } else {
            Load8<T>::get(u + (size_t)pi * 16, t);
#pragma unroll
            for (int k = 0; k < 8; k++) uv[k] = t[k];
            Load8<T>::get(u + (size_t)pi * 16 + 8, t);
#pragma unroll
            for (int k = 0; k < 8; k++) uv[8 + k] = t[k];
        }
    } else {
#pragma unroll
        for (int k = 0; k < 16; k++) { gv[k] = 0.0f; uv[k] = 0.0f; }
    }
    float gmin = gv[0], amax = 0.0f, gsm = fabsf(gv[0]), sabs0 = 0.0f, sabs1 = 0.0f;
#pragma unroll
    for (int k = 1; k < 16; k++) { gmin = fminf(gmin, gv[k]); if (sizeof(T) == 4) gsm = fminf(gsm, fabsf(gv[k])); }
    // two values per instruction where the statements allow it (the same fp32 roundings): the exponent's argument, 1 + e, the two products
    const f32x2 nlog2e = pk2(-0x1.715476p+0f, -0x1.715476p+0f), one2 = pk2(1.0f, 1.0f);
    f32x2 h2[8];
#pragma unroll
    for (int k = 0; k < 16; k += 2) {
        const f32x2 g2 = pk2(gv[k], gv[k + 1]);
        const f32x2 a2 = mul2(g2, nlog2e);
        const f32x2 den = add2(one2, pk2(ex2_approx(lo2(a2)), ex2_approx(hi2(a2))));
        h2[k >> 1] = mul2(mul2(g2, pk2(rcp_approx(lo2(den)), rcp_approx(hi2(den)))), pk2(uv[k], uv[k + 1]));
        h[k] = lo2(h2[k >> 1]); h[k + 1] = hi2(h2[k >> 1]);
        amax = fmaxf(amax, fmaxf(fabsf(h[k]), fabsf(h[k + 1])));
        if (SUMS) { sabs0 = fadd(sabs0, fabsf(h[k])); sabs1 = fadd(sabs1, fabsf(h[k + 1])); }
    }
    amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, 1));
    float sabs = fadd(sabs0, sabs1);
    if (SUMS) sabs = fadd(sabs, __shfl_xor_sync(CAM_FULL, sabs, 1));                                      // sum |h^| of the block
    float sg[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        sg[j] = fadd(fadd(h[4 * j], h[4 * j + 1]), fadd(h[4 * j + 2], h[4 * j + 3]));
        sg[j] = fadd(sg[j], __shfl_xor_sync(CAM_FULL, sg[j], 1));                                         // partner 4
    }
    const float sum = fadd(fadd(sg[0], sg[2]), fadd(sg[1], sg[3]));                                        // partners 2, 1
    const float d = fmul(amax, 0x1.020408p-7f);
    const float inv = rcp_approx(d);
    // the margins of the proofs above; for fp16 gates the ones that follow from the enumerated 7.0e-7 (Q8Margins)
    const float inv_hi = fmul(inv, Q8Margins<T>::hi()), inv_lo = fmul(inv, Q8Margins<T>::lo());
    const f32x2 ih2 = pk2(inv_hi, inv_hi), il2 = pk2(inv_lo, inv_lo), magic2 = pk2(12582912.0f, 12582912.0f);
    uint32_t v[16], differ = 0;
#pragma unroll
    for (int k = 0; k < 16; k += 2) {
        const f32x2 a = fma2(h2[k >> 1], ih2, magic2), b = fma2(h2[k >> 1], il2, magic2);
        v[k] = __float_as_uint(lo2(a)); v[k + 1] = __float_as_uint(hi2(a));
        differ |= (v[k] ^ __float_as_uint(lo2(b))) | (v[k + 1] ^ __float_as_uint(hi2(b)));
    }
    const int low = (int)(__float_as_uint(d) & 0x1fffu) - 0x1000;
    const float smargin = fmul(sabs, Q8Margins<T>::sum());
    const bool sum_open = SUMS && __half_as_ushort(__float2half_rn(fsub(sum, smargin))) != __half_as_ushort(__float2half_rn(fadd(sum, smargin)));
    const bool redo = differ != 0 || !(gmin >= -8.0f) || !(d >= 6.2e-5f && d < 6.0e4f) || (low >= -Q8Margins<T>::TIE && low <= Q8Margins<T>::TIE) || !(fabsf(sum) < 3.0e38f) ||
                      (sizeof(T) == 4 && on && !(gsm >= 3.0e-38f));
    const uint32_t mask = __ballot_sync(CAM_FULL, redo && on);
    const uint32_t pairs = (mask | (mask >> 1)) & 0x55555555u;              // bit 2 j: block j of this warp
    uint32_t resum = 0;                                                     // SUMS: blocks whose scale and codes are proven and whose sum is not
    if (SUMS) { const uint32_t ms = __ballot_sync(CAM_FULL, sum_open && on); resum = (ms | (ms >> 1)) & 0x55555555u & ~pairs; }
    if (on && !((pairs >> (lane & ~1)) & 1u)) {
        uint32_t * o = reinterpret_cast<uint32_t *>(y + (size_t)(pi >> 1) * 36);
        if (q == 0 && !((resum >> (lane & ~1)) & 1u)) __stcs(o, f2_to_h2(d, sum));
#pragma unroll
        for (int j = 0; j < 4; j++)
            __stcs(o + 1 + 4 * q + j, __byte_perm(__byte_perm(v[4 * j], v[4 * j + 1], 0x0040), __byte_perm(v[4 * j + 2], v[4 * j + 3], 0x0040), 0x5410));
    }
    // SUMS: the exact values' sum alone for the blocks in resum (the proven scale comes from the block's even lane)
    for (uint32_t m = resum; m; m &= m - 1) {
        const int j2 = __ffs(m) - 1;
        const size_t blk = (size_t)(base >> 1) + (j2 >> 1);
        const float x = SCALED ? cam_silu(fmul(Load8<T>::one(g + blk * 32 + lane), rs)) : fmul(cam_silu(Load8<T>::one(g + blk * 32 + lane)), Load8<T>::one(u + blk * 32 + lane));
        float sx = fadd(x, __shfl_xor_sync(CAM_FULL, x, 1));
        sx = fadd(sx, __shfl_xor_sync(CAM_FULL, sx, 2));
        sx = fadd(sx, __shfl_xor_sync(CAM_FULL, sx, 16));
        sx = fadd(sx, __shfl_xor_sync(CAM_FULL, sx, 8));
        sx = fadd(sx, __shfl_xor_sync(CAM_FULL, sx, 4));
        const float dj = __shfl_sync(CAM_FULL, d, j2);
        if (lane == 0) *reinterpret_cast<uint32_t *>(y + blk * 36) = f2_to_h2(dj, sx);
    }
    // exact recomputation of the flagged blocks: the whole warp, one lane per value (uniform: pairs is the same in every lane)
    for (uint32_t m = pairs; m; m &= m - 1) {
        const size_t blk = (size_t)(base >> 1) + ((__ffs(m) - 1) >> 1);
        const float x = SCALED ? cam_silu(fmul(Load8<T>::one(g + blk * 32 + lane), rs)) : fmul(cam_silu(Load8<T>::one(g + blk * 32 + lane)), Load8<T>::one(u + blk * 32 + lane));
        float am = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(CAM_FULL, am, o));
        float s = fadd(x, __shfl_xor_sync(CAM_FULL, x, 1));
        s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 2));
        s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 16));
        s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 8));
        s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 4));
        const float de = fdiv(am, 127.0f);
        uint8_t * o = y + blk * 36;
        o[4 + lane] = (uint8_t)q8_code(x, de, am);
        if (lane == 0) *reinterpret_cast<uint32_t *>(o) = f2_to_h2(de, s);
    }
}

template <typename T, bool SUMS, bool SCALED = false>
__global__ void __launch_bounds__(Q8_THREADS) swiglu_q8_fast_kernel(const T * __restrict__ g, const T * __restrict__ u,
                                                                      uint8_t * __restrict__ y, int nb, float rs = 1.0f) {
    const int lane = threadIdx.x & 31;
    const int npairs = nb * 2;
    const int stride = gridDim.x * Q8_THREADS;
    int base = blockIdx.x * Q8_THREADS + (threadIdx.x & ~31);
    for (; base + 32 <= npairs; base += stride) swiglu_q8_step<T, true, SUMS, SCALED>(g, u, y, base, npairs, lane, rs);
    if (base < npairs) swiglu_q8_step<T, false, SUMS, SCALED>(g, u, y, base, npairs, lane, rs);
}

// the last, partial block (n % 32 values, the rest 0): one warp, one lane per value
template <typename T, bool SWIGLU, bool SCALED = false>
__global__ void __launch_bounds__(32) q8_1_tail_kernel(const T * __restrict__ g, const T * __restrict__ u, uint8_t * __restrict__ y,
                                                       long first, int rem, float rs = 1.0f) {
    const int lane = threadIdx.x;
    float x = 0.0f;
    if (lane < rem) {
        x = Load8<T>::one(g + first + lane);
        if (SWIGLU) x = fmul(cam_silu(x), Load8<T>::one(u + first + lane));
        if (SCALED) x = cam_silu(fmul(x, rs));
    }
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, o));
    float s = fadd(x, __shfl_xor_sync(CAM_FULL, x, 1));      // e0 + e1 | e2 + e3
    s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 2));            // (e0 + e1) + (e2 + e3): the group's sum
    s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 16));           // partners 4, 2, 1 of the 8 groups
    s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 8));
    s = fadd(s, __shfl_xor_sync(CAM_FULL, s, 4));
    const float d = fdiv(amax, 127.0f);
    uint8_t * o = y + (first >> 5) * 36;
    o[4 + lane] = (uint8_t)q8_code(x, d, amax);
    if (lane == 0) *reinterpret_cast<uint32_t *>(o) = f2_to_h2(d, s);
}

// The plain quantiser (gg_quantize_q8_1) at memory speed, every byte the exact statements': the values are given, so amax, d and
// the block sum are exact as they stand; only the 32 divisions x / d are replaced, where that provably changes nothing: x * rcp(d)
// is within 1.8e-7 |t| of the IEEE quotient t; if its two ends t (1 -+ 4.8e-7) round to one integer, no rounding boundary lies
// between them and that integer is roundf(t). A lane whose test fails (or whose block has a zero, tiny, huge or NaN scale or sum)
// divides its 16 values. Mapping as swiglu_q8_step: 16 values per lane, two lanes per block.
template <typename T, bool FULL>
CAM_DEV void q8_plain_step(const T * __restrict__ x, uint8_t * __restrict__ y, int base, int npairs, int lane) {
    const int pi = base + lane, q = lane & 1;
    const bool on = FULL || pi < npairs;
    float h[16];
    if (on) {
        float t[8];
        Load8<T>::get(x + (size_t)pi * 16, t);
#pragma unroll
        for (int k = 0; k < 8; k++) h[k] = t[k];
        Load8<T>::get(x + (size_t)pi * 16 + 8, t);
#pragma unroll
        for (int k = 0; k < 8; k++) h[8 + k] = t[k];
    } else {
#pragma unroll
        for (int k = 0; k < 16; k++) h[k] = 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; k++) amax = fmaxf(amax, fabsf(h[k]));
    amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, 1));
    float sg[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        sg[j] = fadd(fadd(h[4 * j], h[4 * j + 1]), fadd(h[4 * j + 2], h[4 * j + 3]));
        sg[j] = fadd(sg[j], __shfl_xor_sync(CAM_FULL, sg[j], 1));                                         // partner 4
    }
    const float sum = fadd(fadd(sg[0], sg[2]), fadd(sg[1], sg[3]));                                        // partners 2, 1
    const float d = fdiv(amax, 127.0f);
    const float inv = rcp_approx(d);
    const float inv_hi = fmul(inv, 0x1.000008p+0f), inv_lo = fmul(inv, 0x1.fffff0p-1f);
    uint32_t v[16], differ = 0;
#pragma unroll
    for (int k = 0; k < 16; k++) {
        v[k] = __float_as_uint(ffma(h[k], inv_hi, 12582912.0f));
        differ |= v[k] ^ __float_as_uint(ffma(h[k], inv_lo, 12582912.0f));
    }
    if (differ != 0 || !(d >= 1.0e-30f && d < 3.0e38f) || !(fabsf(sum) < 3.0e38f)) {
#pragma unroll
        for (int k = 0; k < 16; k++) v[k] = (uint32_t)q8_code(h[k], d, amax);
    }
    if (on) {
        uint32_t * o = reinterpret_cast<uint32_t *>(y + (size_t)(pi >> 1) * 36);
        if (q == 0) __stcs(o, f2_to_h2(d, sum));
#pragma unroll
        for (int j = 0; j < 4; j++)
            __stcs(o + 1 + 4 * q + j, __byte_perm(__byte_perm(v[4 * j], v[4 * j + 1], 0x0040), __byte_perm(v[4 * j + 2], v[4 * j + 3], 0x0040), 0x5410));
    }
}

template <typename T>
__global__ void __launch_bounds__(Q8_THREADS) q8_plain_kernel(const T * __restrict__ x, uint8_t * __restrict__ y, int nb) {
    const int lane = threadIdx.x & 31;
    const int npairs = nb * 2;
    const int stride = gridDim.x * Q8_THREADS;
    int base = blockIdx.x * Q8_THREADS + (threadIdx.x & ~31);
    for (; base + 32 <= npairs; base += stride) q8_plain_step<T, true>(x, y, base, npairs, lane);
    if (base < npairs) q8_plain_step<T, false>(x, y, base, npairs, lane);
}

// FAST 1: the two-pass fused kernel (SwiGLU only); 2: the same with the block sums proven too. Plain quantisation: q8_plain_kernel.
// Strict SwiGLU (FAST 0): the exact statements for every value
template <typename T, bool SWIGLU, int FAST = 0>
int launch_q8(const T * g, const T * u, void * y, long n, cudaStream_t stream) {
    if (n < 0 || !g || !y || (SWIGLU && !u)) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (!cam_aligned16(g) || (SWIGLU && !cam_aligned16(u)) || (reinterpret_cast<uintptr_t>(y) & 3u)) return CAM_ERR_ALIGN;
    const long nb = n >> 5;
    if (nb > 0) {
        const long want = (nb * 4 + Q8_THREADS - 1) / Q8_THREADS;
        if (FAST) {
            const long piece = 1L << 28;                                   // blocks per launch
            // (about 8 units of 4096 values per thread block: 1309 -> 1229 us for 65536 x 25600 values, the all-bytes form 0.83 -> 0.88)
            for (long b0 = 0; b0 < nb; b0 += piece) {
                const long m = nb - b0 < piece ? nb - b0 : piece;
                const long w = (m * 2 + Q8_THREADS - 1) / Q8_THREADS;
                swiglu_q8_fast_kernel<T, FAST == 2><<<cam_iter_grid(swiglu_q8_fast_kernel<T, FAST == 2>, Q8_THREADS, 0, w, 8), Q8_THREADS, 0, stream>>>(
                    g + b0 * 32, u + b0 * 32, (uint8_t *)y + b0 * 36, (int)m);
            }
        } else if (!SWIGLU) {
            const long piece = 1L << 28;
            for (long b0 = 0; b0 < nb; b0 += piece) {
                const long m = nb - b0 < piece ? nb - b0 : piece;
                const long w = (m * 2 + Q8_THREADS - 1) / Q8_THREADS;
                q8_plain_kernel<T><<<cam_resident_grid(q8_plain_kernel<T>, Q8_THREADS, 0, w), Q8_THREADS, 0, stream>>>(g + b0 * 32, (uint8_t *)y + b0 * 36, (int)m);
            }
        } else q8_1_kernel<T, SWIGLU><<<cam_resident_grid(q8_1_kernel<T, SWIGLU>, Q8_THREADS, 0, want, 8), Q8_THREADS, 0, stream>>>(g, u, (uint8_t *)y, nb);
    }
    if (n & 31) q8_1_tail_kernel<T, SWIGLU><<<1, 32, 0, stream>>>(g, u, (uint8_t *)y, nb << 5, (int)(n & 31));
    return (int)cudaGetLastError();
}

// the tape op's work = 1: Q8_1 blocks of silu(x rs) (SUMS: all 36 bytes the exact statements'; else the scale and the codes)
template <bool SUMS>
int launch_q8_scaled(const float * x, float rs, void * y, long n, cudaStream_t stream) {
    if (n < 0 || !x || !y) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (!cam_aligned16(x) || (reinterpret_cast<uintptr_t>(y) & 3u)) return CAM_ERR_ALIGN;
    const long nb = n >> 5, piece = 1L << 28;
    for (long b0 = 0; b0 < nb; b0 += piece) {
        const long m = nb - b0 < piece ? nb - b0 : piece;
        const long w = (m * 2 + Q8_THREADS - 1) / Q8_THREADS;
        swiglu_q8_fast_kernel<float, SUMS, true><<<cam_iter_grid(swiglu_q8_fast_kernel<float, SUMS, true>, Q8_THREADS, 0, w, 8), Q8_THREADS, 0, stream>>>(
            x + b0 * 32, nullptr, (uint8_t *)y + b0 * 36, (int)m, rs);
    }
    if (n & 31) q8_1_tail_kernel<float, false, true><<<1, 32, 0, stream>>>(x, nullptr, (uint8_t *)y, nb << 5, (int)(n & 31), rs);
    return (int)cudaGetLastError();
}

// y = silu(g) u elementwise: fp16 (q3p_swiglu) or fp32 (gg_silu_mul) out
template <bool HALF_OUT>
__global__ void __launch_bounds__(256) silu_mul_kernel(const float * __restrict__ g, const float * __restrict__ u, void * __restrict__ y,
                                                       long n, int vec) {
    const long stride = (long)gridDim.x * 256;
    const long n4 = vec ? n >> 2 : 0;
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(g) + i), b = __ldg(reinterpret_cast<const float4 *>(u) + i);
        const float4 v = make_float4(fmul(cam_silu(a.x), b.x), fmul(cam_silu(a.y), b.y), fmul(cam_silu(a.z), b.z), fmul(cam_silu(a.w), b.w));
        if (HALF_OUT) st64_stream(reinterpret_cast<uint16_t *>(y) + 4 * i, make_uint2(f2_to_h2(v.x, v.y), f2_to_h2(v.z, v.w)));
        else __stcs(reinterpret_cast<float4 *>(y) + i, v);
    }
    for (long i = 4 * n4 + (long)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
        const float v = fmul(cam_silu(__ldg(g + i)), __ldg(u + i));
        if (HALF_OUT) reinterpret_cast<uint16_t *>(y)[i] = f_to_h(v);
        else reinterpret_cast<float *>(y)[i] = v;
    }
}

// the two evaluations of silu side by side, for the test that enumerates the fp16 gates
__global__ void __launch_bounds__(256) silu_probe_kernel(const uint16_t * __restrict__ g, float * __restrict__ fast, float * __restrict__ exact, int n) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const float x = __half2float(__ushort_as_half(g[i]));
    exact[i] = cam_silu(x);
    fast[i] = fmul(x, rcp_approx(fadd(1.0f, ex2_approx(fmul(x, -0x1.715476p+0f)))));
}

template <bool HALF_OUT>
int launch_silu_mul(const float * g, const float * u, void * y, long n, cudaStream_t stream) {
    if (n < 0 || !g || !u || !y) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    const int vec = cam_aligned16(g) && cam_aligned16(u) && cam_aligned16(y);
    const long want = ((vec ? (n + 3) / 4 : n) + 255) / 256;
    silu_mul_kernel<HALF_OUT><<<cam_resident_grid(silu_mul_kernel<HALF_OUT>, 256, 0, want), 256, 0, stream>>>(g, u, y, n, vec);
    return (int)cudaGetLastError();
}

}   // namespace

// q3p_swiglu: y16[i] = fp16(silu(g[i]) u[i]), i < n. Reference: kernels/q3m_prefill.hip:516-518; python/caminus/prefill/q3m_ops.py:106-107.
extern "C" int q3p_swiglu(const float * g, const float * u, void * y16, int n, void * stream) {
    return launch_silu_mul<true>(g, u, y16, n, (cudaStream_t)stream);
}
// gg_silu_mul: h[i] = silu(g[i]) u[i] in fp32. Reference: kernels/k3_gguf.hip:74-77; python/caminus/engine/gguf.py:57-61.
extern "C" int gg_silu_mul(const float * g, const float * u, float * h, int n, void * stream) {
    return launch_silu_mul<false>(g, u, h, n, (cudaStream_t)stream);
}
// gg_quantize_q8_1: n fp32 values -> ceil(n / 32) blocks of 36 bytes; values past n quantise as 0. (The reference's launch
// also writes whole blocks of zeros up to the next multiple of 8 blocks; this entry writes exactly ceil(n / 32).)
// Reference: kernels/k3_gguf.hip:29-36; python/caminus/engine/gguf.py:39-46.
extern "C" int gg_quantize_q8_1(const float * x, void * y, int n, void * stream) {
    return launch_q8<float, false>(x, nullptr, y, n, (cudaStream_t)stream);
}
// gg_swiglu_q8_1: Q8_1 blocks of silu(x[i]) mul[i]: the tape op OP_GG_Q8_1 with work = 2 as one launch.
// Reference: kernels/k3_gguf_ops.h:55-77 (semantics); python/caminus/engine/k3.py:649-659 (Engine.gg_q8_1(x, yq, mul=u)).
extern "C" int gg_swiglu_q8_1(const float * x, const float * mul, void * y, long n, void * stream) {
    return launch_q8<float, true, 1>(x, mul, y, n, (cudaStream_t)stream);
}
// the same with fp16 gate and up (widened exactly to fp32 before the same statements)
extern "C" int gg_swiglu_q8_1_f16(const void * g, const void * u, void * y, long n, void * stream) {
    return launch_q8<uint16_t, true, 1>((const uint16_t *)g, (const uint16_t *)u, y, n, (cudaStream_t)stream);
}
// The _sums forms: the fast pass with the block sum proven as well: all 36 bytes are the exact statements' bytes, at about three quarters
// of the copy bandwidth (one block in 15 visits the exact statements instead of one in 50, most of them for the sum alone).
extern "C" int gg_swiglu_q8_1_sums(const float * x, const float * mul, void * y, long n, void * stream) {
    return launch_q8<float, true, 2>(x, mul, y, n, (cudaStream_t)stream);
}
extern "C" int gg_swiglu_q8_1_f16_sums(const void * g, const void * u, void * y, long n, void * stream) {
    return launch_q8<uint16_t, true, 2>((const uint16_t *)g, (const uint16_t *)u, y, n, (cudaStream_t)stream);
}
// gg_silu_scale_q8_1: Q8_1 blocks of silu(x[i] * rs): the tape op OP_GG_Q8_1 with work = 1 (ggml_scale, then ggml_silu, then the
// quantiser: the hyper-connection down output) as one launch. Reference: kernels/k3_gguf_ops.h:70 (semantics);
// python/caminus/engine/k3.py:649-659 (Engine.gg_q8_1(x, yq, silu_scale=rs)). d and the codes are the exact statements' bytes, the sum
// as for gg_swiglu_q8_1; the _sums form proves the sum too.
extern "C" int gg_silu_scale_q8_1(const float * x, float rs, void * y, long n, void * stream) {
    return launch_q8_scaled<false>(x, rs, y, n, (cudaStream_t)stream);
}
extern "C" int gg_silu_scale_q8_1_sums(const float * x, float rs, void * y, long n, void * stream) {
    return launch_q8_scaled<true>(x, rs, y, n, (cudaStream_t)stream);
}
// cam_probe_silu_f16: for n fp16 gates, exact[i] = the exact statements' silu(g[i]) and fast[i] = the special-function evaluation the fast
// passes use, g rcp(1 + ex2(-g log2 e)). No counterpart in the reference: it lets a test measure, on the device it runs on, the bound the
// fp16 entries' proofs rest on (max |fast - exact| / |exact| over all gates >= -8).
extern "C" int cam_probe_silu_f16(const void * g, float * fast, float * exact, int n, void * stream) {
    if (n < 0 || !g || !fast || !exact) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    silu_probe_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const uint16_t *)g, fast, exact, n);
    return (int)cudaGetLastError();
}
// The strict forms: every value through the exact statements, so the block sums are the exact statements' bytes as well as
// d and the codes (which the entries above already guarantee). About half the throughput.
extern "C" int gg_swiglu_q8_1_strict(const float * x, const float * mul, void * y, long n, void * stream) {
    return launch_q8<float, true>(x, mul, y, n, (cudaStream_t)stream);
}
extern "C" int gg_swiglu_q8_1_f16_strict(const void * g, const void * u, void * y, long n, void * stream) {
    return launch_q8<uint16_t, true>((const uint16_t *)g, (const uint16_t *)u, y, n, (cudaStream_t)stream);
}
