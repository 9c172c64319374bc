// The training line's fused activation quantiser, forward (the reference's kernels/actq.hip: actq_fwd_*, silu_mul_actq_fwd,
// block_entry_fwd; wrappers python/caminus/train/actq.py:22-169).
//
// Per row of K values (a multiple of 128, <= 8192): the source value is rounded to bf16, each chunk of 128 goes through the
// unnormalised Walsh-Hadamard butterflies (1, 2 inside a lane's four values, 4 .. 64 across the lanes of a warp), times the bf16
// value of 1 / sqrt(128), rounded to bf16; the row's amax gives s = max(amax clip / qmax, 1e-8); the codes are
// clamp(rint(u / s), -qmax - 1, qmax); outputs: the dequantised bf16 values (optional), the row scale, the int4 codes packed four
// to 16 bits (optional). Sources: a bf16 or fp32 tensor; the MLP activation bf16(bf16(silu(g)) u) computed from [g | u] rows; the
// RMSNorm (x rstd) w never materialised (block entry), which also emits up to 16 thin bf16 gate projections.
// Rows of up to 2048 values: a warp per row (the row's chunks in the warp's registers between the amax and the codes; no barrier):
// the butterflies of a chunk are the reference's lane for lane, the row's amax is order-free, and the block entry's two ordered sums
// (sum of squares, thin projections: thread tid owns tid + 256 j, wave butterflies, 8 wave sums in order) are reproduced on the warp
// by ref_total_f32. Longer rows: the reference's mapping (one block of 8 warps per row, warp w takes chunks w, w + 8, ..).
#include "cam_common.cuh"

namespace {

constexpr int AQ_WAVES = 8, AQ_MAXC = 8, AQ_NAB = 16;

CAM_DEV float bf2f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
CAM_DEV uint16_t f2bf(float f) {
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
CAM_DEV float rbf(float f) { return bf2f(f2bf(f)); }
// four values rounded to bf16 (the conversion instruction, two values at a time), and packed bf16 pairs widened again
CAM_DEV uint2 pack4(const float (&v)[4]) { return make_uint2(bf16x2<true>(v[0], v[1]), bf16x2<true>(v[2], v[3])); }
CAM_DEV void unpack4(uint2 p, float (&v)[4]) {
    v[0] = __uint_as_float(p.x << 16); v[1] = __uint_as_float(p.x & 0xffff0000u); v[2] = __uint_as_float(p.y << 16); v[3] = __uint_as_float(p.y & 0xffff0000u);
}
CAM_DEV void rbf4(float (&v)[4]) { unpack4(pack4(v), v); }

CAM_DEV void fwht128(float (&v)[4], int lane) {
    float a = v[0], b = v[1]; v[0] = fadd(a, b); v[1] = fsub(a, b);
    a = v[2]; b = v[3]; v[2] = fadd(a, b); v[3] = fsub(a, b);
    a = v[0]; b = v[2]; v[0] = fadd(a, b); v[2] = fsub(a, b);
    a = v[1]; b = v[3]; v[1] = fadd(a, b); v[3] = fsub(a, b);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float sg = (lane & m) ? -1.0f : 1.0f;      // the upper lane of a pair holds partner - own: fma(own, -1, partner), one rounding
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = ffma(v[e], sg, __shfl_xor_sync(CAM_FULL, v[e], m));
    }
}
CAM_DEV float wave_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(CAM_FULL, v, m));
    return v;
}
CAM_DEV float wave_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fadd(v, __shfl_xor_sync(CAM_FULL, v, m));
    return v;
}
CAM_DEV float block_reduce(float v, float * lds, int wave, int lane, bool is_max) {
    __syncthreads();
    if (lane == 0) lds[wave] = v;
    __syncthreads();
    float r = lds[0];
    for (int w = 1; w < AQ_WAVES; w++) r = is_max ? fmaxf(r, lds[w]) : fadd(r, lds[w]);
    return r;
}

CAM_DEV void bf4(uint2 w, float (&v)[4]) { v[0] = __uint_as_float(w.x << 16); v[1] = __uint_as_float(w.x & 0xffff0000u); v[2] = __uint_as_float(w.y << 16); v[3] = __uint_as_float(w.y & 0xffff0000u); }
// get4: four consecutive values at k (a multiple of 4; rows 8-byte / 16-byte aligned: checked by the launcher)
struct PlainBf16 {
    const uint16_t * x; int K;
    CAM_DEV float operator()(int row, int k) const { return bf2f(__ldg(x + (size_t)row * K + k)); }
    CAM_DEV void get4(int row, int k, float (&v)[4]) const { bf4(__ldg(reinterpret_cast<const uint2 *>(x + (size_t)row * K + k)), v); }
    static constexpr bool kBf16 = true;            // get4's values are bf16 numbers already
    static constexpr bool kHeavy = false;          // (a source whose loads carry arithmetic of their own keeps the transformed row in shared memory sooner)
    static constexpr bool kPrologue = false;       // (no work per row before the steps)
    // sixteen consecutive values at k (a multiple of 16; rows 16-byte aligned) as pairs; zeros when off
    CAM_DEV void get16(bool on, int row, int k, f32x2 (&p)[8]) const {
        uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
        if (on) { const uint4 * r = reinterpret_cast<const uint4 *>(x + (size_t)row * K + k); a = __ldg(r); b = __ldg(r + 1); }
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++) p[i] = pk2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
};
struct PlainF32 {
    const float * x; int K;
    CAM_DEV float operator()(int row, int k) const { return __ldg(x + (size_t)row * K + k); }
    CAM_DEV void get4(int row, int k, float (&v)[4]) const {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(x + (size_t)row * K + k)); v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static constexpr bool kBf16 = false;
    static constexpr bool kHeavy = false, kPrologue = false;
    CAM_DEV void get16(bool on, int row, int k, f32x2 (&p)[8]) const {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on) a = __ldg(reinterpret_cast<const float4 *>(x + (size_t)row * K + k) + q);
            const uint32_t w0 = bf16x2<true>(a.x, a.y), w1 = bf16x2<true>(a.z, a.w);
            p[2 * q] = pk2(__uint_as_float(w0 << 16), __uint_as_float(w0 & 0xffff0000u));
            p[2 * q + 1] = pk2(__uint_as_float(w1 << 16), __uint_as_float(w1 & 0xffff0000u));
        }
    }
};
// the exact statements' bf16(silu(g)) of two gates (out of line: the fast passes call it for one pair in some hundreds)
__device__ __noinline__ uint32_t silu_pair_bf16_exact(float g0, float g1) { return bf16_soft<true>(cam_silu(g0)) | (bf16_soft<true>(cam_silu(g1)) << 16); }
struct SiluMulSrc {
    const uint16_t * gu; int ld, F;
    CAM_DEV float operator()(int row, int k) const {
        const uint16_t * r = gu + (size_t)row * ld;
        return rbf(fmul(rbf(cam_silu(bf2f(__ldg(r + k)))), bf2f(__ldg(r + F + k))));
    }
    CAM_DEV void get4(int row, int k, float (&v)[4]) const {
        const uint16_t * r = gu + (size_t)row * ld;
        float g[4], u[4];
        bf4(__ldg(reinterpret_cast<const uint2 *>(r + k)), g); bf4(__ldg(reinterpret_cast<const uint2 *>(r + F + k)), u);
        uint32_t w2[2];                       // bf16(silu(g)): the special-function value where its bits are proven, else the exact statements (silu_bf16_fast)
        const uint32_t redo = silu_bf16_fast<4>(g, w2);
#pragma unroll
        for (int p = 0; p < 2; p++)
            if (((redo >> p) & 1u) || bf16_pair_has_nan(w2[p])) w2[p] = bf16_soft<true>(cam_silu(g[2 * p])) | (bf16_soft<true>(cam_silu(g[2 * p + 1])) << 16);
        unpack4(make_uint2(w2[0], w2[1]), v);
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = fmul(v[e], u[e]);
        rbf4(v);
    }
    static constexpr bool kBf16 = true;
    static constexpr bool kHeavy = true, kPrologue = false;
    // sixteen consecutive activations at k as pairs (rows and F 16-byte aligned: ld and F multiples of 8, checked by the launcher)
    CAM_DEV void get16(bool on, int row, int k, f32x2 (&p)[8]) const {
        if (!on) {                               // (no gates: zeros, and no visit to the exact statements that a zero gate asks for)
#pragma unroll
            for (int i = 0; i < 8; i++) p[i] = pk2(0.f, 0.f);
            return;
        }
        const uint4 * r = reinterpret_cast<const uint4 *>(gu + (size_t)row * ld + k);
        const uint4 * q = reinterpret_cast<const uint4 *>(gu + (size_t)row * ld + F + k);
        const uint4 ga = __ldg(r), gb = __ldg(r + 1), ua = __ldg(q), ub = __ldg(q + 1);
        const uint32_t gw[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w}, uw[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
        float g[16];
        const f32x2 zero2 = pk2(0.f, 0.f);
        f32x2 zg = zero2;                        // 0 g summed: a NaN iff a gate is a NaN or an infinity
#pragma unroll
        for (int i = 0; i < 8; i++) {
            g[2 * i] = __uint_as_float(gw[i] << 16); g[2 * i + 1] = __uint_as_float(gw[i] & 0xffff0000u);
            zg = fma2(pk2(g[2 * i], g[2 * i + 1]), zero2, zg);
        }
        uint32_t sw[8];                          // bf16(silu(g)): the special-function value where its bits are proven, else the exact statements
        uint32_t redo = silu_bf16_fast<16>(g, sw);
        const float zs = fadd(lo2(zg), hi2(zg));
        if (zs != zs) redo = 0xffu;
        if (redo) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                if ((redo >> i) & 1u) sw[i] = silu_pair_bf16_exact(g[2 * i], g[2 * i + 1]);
        }
        f32x2 zp = zero2;
        uint32_t hw[8];                          // bf16(bf16(silu(g)) u)
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const f32x2 h = mul2(pk2(__uint_as_float(sw[i] << 16), __uint_as_float(sw[i] & 0xffff0000u)),
                                 pk2(__uint_as_float(uw[i] << 16), __uint_as_float(uw[i] & 0xffff0000u)));
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hw[i]) : "f"(hi2(h)), "f"(lo2(h)));
            zp = fma2(h, zero2, zp);
        }
        const float zq = fadd(lo2(zp), hi2(zp));
        if (zq != zq) {                          // a product that is a NaN is stored as 0x7fc0 (the conversion gives 0x7fff)
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if ((hw[i] & 0x7fffu) > 0x7f80u) hw[i] = (hw[i] & 0xffff0000u) | 0x7fc0u;
                if ((hw[i] & 0x7fff0000u) > 0x7f800000u) hw[i] = (hw[i] & 0x0000ffffu) | 0x7fc00000u;
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++) p[i] = pk2(__uint_as_float(hw[i] << 16), __uint_as_float(hw[i] & 0xffff0000u));
    }
};
struct RmsSrc {
    const float * x; const float * w; float rstd; int d;
    CAM_DEV float operator()(int row, int k) const { return fmul(fmul(__ldg(x + (size_t)row * d + k), rstd), __ldg(w + k)); }
};

// VEC: the source is read four values at a time (get4; rows aligned for it)
template <typename Src, bool VEC = false>
CAM_DEV void actq_fwd_src(Src src, uint16_t * __restrict__ y, float * __restrict__ s_out, int K, float clip, int qmax, uint16_t * __restrict__ codes,
                          float * lds) {
    const int row = blockIdx.x, wave = threadIdx.x >> 5, lane = threadIdx.x & 31, nch = K / 128;
    float u[AQ_MAXC][4];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < AQ_MAXC; c++) {
        const int ch = wave + c * AQ_WAVES;
        if (ch < nch) {                                            // (uniform per warp)
            if constexpr (VEC) {
                src.get4(row, ch * 128 + lane * 4, u[c]);
                if (!Src::kBf16) rbf4(u[c]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) u[c][e] = src(row, ch * 128 + lane * 4 + e);
                rbf4(u[c]);
            }
            fwht128(u[c], lane);
#pragma unroll
            for (int e = 0; e < 4; e++) u[c][e] = fmul(u[c][e], 0.08837890625f);
            rbf4(u[c]);
#pragma unroll
            for (int e = 0; e < 4; e++) amax = fmaxf(amax, fabsf(u[c][e]));
        }
    }
    amax = block_reduce(wave_max(amax), lds, wave, lane, true);
    const float s = fmaxf(fdiv(fmul(amax, clip), (float)qmax), 1e-8f);
    if (threadIdx.x == 0 && s_out) s_out[row] = s;
    const float inv = rcp_approx(s);
    const float inv_hi = fmul(inv, 0x1.000008p+0f), inv_lo = fmul(inv, 0x1.fffff0p-1f);
    const bool fast = s < 3.0e38f && fmul(amax, inv) < 4.0e6f;
    uint16_t * yr = y ? y + (size_t)row * K : nullptr;
#pragma unroll
    for (int c = 0; c < AQ_MAXC; c++) {
        const int ch = wave + c * AQ_WAVES;
        if (ch < nch) {
            float q[4];
            bool slow = !fast;
#pragma unroll
            for (int e = 0; e < 4; e++) {       // (the division-free rint of actq_emit below)
                const float vh = ffma(u[c][e], inv_hi, 12582912.0f), vl = ffma(u[c][e], inv_lo, 12582912.0f);
                q[e] = __uint_as_float(__float_as_uint(fsub(vh, 12582912.0f)) | (__float_as_uint(u[c][e]) & 0x80000000u));
                slow |= vh != vl;
            }
            if (slow) {
#pragma unroll
                for (int e = 0; e < 4; e++) q[e] = rintf(fdiv(u[c][e], s));
            }
#pragma unroll
            for (int e = 0; e < 4; e++) q[e] = fminf(fmaxf(q[e], (float)(-qmax - 1)), (float)qmax);
            const uint32_t pk = ((uint32_t)(int)q[0] & 0xFu) | (((uint32_t)(int)q[1] & 0xFu) << 4) | (((uint32_t)(int)q[2] & 0xFu) << 8) | (((uint32_t)(int)q[3] & 0xFu) << 12);
            if (y) st64(yr + ch * 128 + lane * 4, make_uint2(bf16x2<true>(fmul(q[0], s), fmul(q[1], s)), bf16x2<true>(fmul(q[2], s), fmul(q[3], s))));
            if (codes) codes[(size_t)row * (K / 4) + ch * 32 + lane] = (uint16_t)pk;
        }
    }
}

template <typename Src, bool VEC = false>
__global__ void __launch_bounds__(256) actq_kernel(Src src, uint16_t * y, float * s, int K, float clip, int qmax, uint16_t * codes) {
    __shared__ float lds[AQ_WAVES];
    actq_fwd_src<Src, VEC>(src, y, s, K, clip, qmax, codes, lds);
}

__global__ void __launch_bounds__(256) block_entry_kernel(const float * __restrict__ x, const float * __restrict__ nw, const uint16_t * __restrict__ wab, int nab,
                                                          float eps, uint16_t * y, float * s, uint16_t * codes, uint16_t * ab, float * rstd_out, int d,
                                                          float clip, int qmax) {
    __shared__ float lds[AQ_WAVES];
    __shared__ float part[AQ_WAVES][AQ_NAB];
    const int row = blockIdx.x, wave = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float * xr = x + (size_t)row * d;
    float ss = 0.f;
    for (int k = threadIdx.x; k < d; k += 256) { const float v = __ldg(xr + k); ss = ffma(v, v, ss); }
    ss = block_reduce(wave_sum(ss), lds, wave, lane, false);
    const float rstd = cam_rsqrt(fadd(fdiv(ss, (float)d), eps));
    if (threadIdx.x == 0) rstd_out[row] = rstd;
    actq_fwd_src(RmsSrc{x, nw, rstd, d}, y, s, d, clip, qmax, codes, lds);
    if (nab) {
        float acc[AQ_NAB];
#pragma unroll
        for (int j = 0; j < AQ_NAB; j++) acc[j] = 0.f;
        for (int k = threadIdx.x; k < d; k += 256) {
            const float hb = rbf(fmul(fmul(__ldg(xr + k), rstd), __ldg(nw + k)));
#pragma unroll
            for (int j = 0; j < AQ_NAB; j++)
                if (j < nab) acc[j] = ffma(hb, bf2f(__ldg(wab + (size_t)j * d + k)), acc[j]);
        }
#pragma unroll
        for (int j = 0; j < AQ_NAB; j++)
            if (j < nab) { const float v = wave_sum(acc[j]); if (lane == 0) part[wave][j] = v; }
        __syncthreads();
        if (threadIdx.x < nab) {
            float v = 0.f;
            for (int w = 0; w < AQ_WAVES; w++) v = fadd(v, part[w][threadIdx.x]);
            ab[(size_t)row * nab + threadIdx.x] = f2bf(v);
        }
    }
}

// ---- a warp per row (K <= 128 MAXC) ---------------------------------------------------------------------------------------------
// one lane's four quantised values of chunk ch: clamped, packed to a 16-bit code word, dequantised to bf16
CAM_DEV void actq_store(float (&q)[4], float s, float lo, float hi, int row, int ch, int lane, uint16_t * __restrict__ y, int K, uint16_t * __restrict__ codes) {
#pragma unroll
    for (int e = 0; e < 4; e++) q[e] = fminf(fmaxf(q[e], lo), hi);
    const uint32_t pk = ((uint32_t)(int)q[0] & 0xFu) | (((uint32_t)(int)q[1] & 0xFu) << 4) | (((uint32_t)(int)q[2] & 0xFu) << 8) | (((uint32_t)(int)q[3] & 0xFu) << 12);
    if (y) st64(y + (size_t)row * K + ch * 128 + lane * 4, make_uint2(bf16x2<true>(fmul(q[0], s), fmul(q[1], s)), bf16x2<true>(fmul(q[2], s), fmul(q[3], s))));
    if (codes) codes[(size_t)row * (K / 4) + ch * 32 + lane] = (uint16_t)pk;
}

// the codes, values and scale of a row whose transformed chunks u[c] (c < nch) are in the warp's registers
template <int MAXC>
CAM_DEV void actq_emit(const uint2 (&up)[MAXC], float amax, int nch, int row, int lane, uint16_t * __restrict__ y, float * __restrict__ s_out, int K,
                       float clip, int qmax, uint16_t * __restrict__ codes) {
    amax = wave_max(amax);
    const float s = fmaxf(fdiv(fmul(amax, clip), (float)qmax), 1e-8f);
    if (lane == 0 && s_out) s_out[row] = s;
    const float lo = (float)(-qmax - 1), hi = (float)qmax;
    // rint(u / s) without the division where that is provably the same integer: u * rcp(s) is within 1.8e-7 |t| of the IEEE quotient
    // t; if u * rcp(s) (1 - 4.8e-7) and u * rcp(s) (1 + 4.8e-7) round to one integer, no rounding boundary and no tie lies between
    // them, and that integer is rint(t). Otherwise (and for a row whose scale is not an ordinary number) the value is divided.
    const float inv = rcp_approx(s);
    const float inv_hi = fmul(inv, 0x1.000008p+0f), inv_lo = fmul(inv, 0x1.fffff0p-1f);
    const bool fast = s < 3.0e38f && fmul(amax, inv) < 4.0e6f;                 // (s >= 1e-8; false for a NaN)
    uint32_t redo = 0;                                   // bit c: this lane's four values of chunk c take the division (settled after the loop:
#pragma unroll                                           //  a branch per chunk kept the compiler from batching the row's stores)
    for (int c = 0; c < MAXC; c++)
        if (c < nch) {
            float q[4], u[4];
            unpack4(up[c], u);
            bool slow = !fast;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float vh = ffma(u[e], inv_hi, 12582912.0f), vl = ffma(u[e], inv_lo, 12582912.0f);
                q[e] = __uint_as_float(__float_as_uint(fsub(vh, 12582912.0f)) | (__float_as_uint(u[e]) & 0x80000000u));     // (rint keeps the sign of a zero)
                slow |= vh != vl;
            }
            if (slow) redo |= 1u << c;
            actq_store(q, s, lo, hi, row, c, lane, y, K, codes);
        }
    while (redo) {                                       // (rare: the lane's four values divided, stored over the fast ones)
        const int c = __ffs(redo) - 1;
        redo &= redo - 1;
        uint2 pk = up[0];
#pragma unroll
        for (int k = 1; k < MAXC; k++) if (k == c) pk = up[k];
        float q[4], u[4];
        unpack4(pk, u);
#pragma unroll
        for (int e = 0; e < 4; e++) q[e] = rintf(fdiv(u[e], s));
        actq_store(q, s, lo, hi, row, c, lane, y, K, codes);
    }
}

template <typename Src, int MAXC>
__global__ void __launch_bounds__(256) actq_rows_kernel(Src src, uint16_t * __restrict__ y, float * __restrict__ s_out, int K, float clip, int qmax,
                                                        uint16_t * __restrict__ codes, int M) {
    const int lane = threadIdx.x & 31, nch = K >> 7;
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < M; row += gridDim.x * 8) {
        uint2 up[MAXC];                                                   // the row's transformed values, bf16 pairs
        float amax = 0.f;
#pragma unroll
        for (int c0 = 0; c0 < MAXC; c0 += 8) {                           // eight chunks' loads in flight at a time
            float u[8][4];
#pragma unroll
            for (int c = 0; c < 8; c++)
                if (c0 + c < nch) src.get4(row, (c0 + c) * 128 + lane * 4, u[c]);
#pragma unroll
            for (int c = 0; c < 8; c++)
                if (c0 + c < nch) {
                    if (!Src::kBf16) rbf4(u[c]);
                    fwht128(u[c], lane);
#pragma unroll
                    for (int e = 0; e < 4; e++) u[c][e] = fmul(u[c][e], 0.08837890625f);
                    up[c0 + c] = pack4(u[c]);
                    unpack4(up[c0 + c], u[c]);
#pragma unroll
                    for (int e = 0; e < 4; e++) amax = fmaxf(amax, fabsf(u[c][e]));
                }
        }
        actq_emit<MAXC>(up, amax, nch, row, lane, y, s_out, K, clip, qmax, codes);
    }
}

template <int MAXC>
__global__ void __launch_bounds__(256) block_entry_rows_kernel(const float * __restrict__ x, const float * __restrict__ nw, const uint16_t * __restrict__ wab,
                                                               int nab, float eps, uint16_t * __restrict__ y, float * __restrict__ s_out,
                                                               uint16_t * __restrict__ codes, uint16_t * __restrict__ ab, float * __restrict__ rstd_out,
                                                               int d, float clip, int qmax, int M) {
    const int lane = threadIdx.x & 31, nch = d >> 7;
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < M; row += gridDim.x * 8) {
        float u[MAXC][4];
        const float * xr = x + (size_t)row * d + lane * 4;
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nch) { const float4 a = __ldg(reinterpret_cast<const float4 *>(xr + c * 128)); u[c][0] = a.x; u[c][1] = a.y; u[c][2] = a.z; u[c][3] = a.w; }
        float a8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nch) {
#pragma unroll
                for (int e = 0; e < 4; e++) a8[4 * (c & 1) + e] = ffma(u[c][e], u[c][e], a8[4 * (c & 1) + e]);
            }
        const float rstd = cam_rsqrt(fadd(fdiv(ref_total_f32(a8, lane), (float)d), eps));
        if (lane == 0) rstd_out[row] = rstd;
        // hb = bf16((x rstd) w): the quantiser's source and the projections' operand
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nch) {
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(nw + c * 128 + lane * 4));
                u[c][0] = fmul(fmul(u[c][0], rstd), w4.x); u[c][1] = fmul(fmul(u[c][1], rstd), w4.y);
                u[c][2] = fmul(fmul(u[c][2], rstd), w4.z); u[c][3] = fmul(fmul(u[c][3], rstd), w4.w);
                rbf4(u[c]);
            }
        for (int j = 0; j < nab; j++) {
            const uint16_t * wr = wab + (size_t)j * d + lane * 4;
            float p8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < MAXC; c++)
                if (c < nch) {
                    float wv[4];
                    bf4(__ldg(reinterpret_cast<const uint2 *>(wr + c * 128)), wv);
#pragma unroll
                    for (int e = 0; e < 4; e++) p8[4 * (c & 1) + e] = ffma(u[c][e], wv[e], p8[4 * (c & 1) + e]);
                }
            const float tot = ref_total_f32(p8, lane);
            if (lane == 0) ab[(size_t)row * nab + j] = f2bf(tot);
        }
        float amax = 0.f;
        uint2 up[MAXC];
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nch) {
                fwht128(u[c], lane);
#pragma unroll
                for (int e = 0; e < 4; e++) u[c][e] = fmul(u[c][e], 0.08837890625f);
                up[c] = pack4(u[c]);
                unpack4(up[c], u[c]);
#pragma unroll
                for (int e = 0; e < 4; e++) amax = fmaxf(amax, fabsf(u[c][e]));
            }
        actq_emit<MAXC>(up, amax, nch, row, lane, y, s_out, d, clip, qmax, codes);
    }
}

// ---- sixteen values per lane --------------------------------------------------------------------------------------------------------
// The kernels above give a lane 4 values of a chunk of 128, so five of the seven butterfly stages cross lanes: a shuffle and an fma per
// value and stage. Here a lane holds 16 consecutive values (8 lanes a chunk, four chunks per warp step): stages 1 .. 8 stay inside the
// lane, stages 16, 32, 64 exchange with lanes l ^ 1, l ^ 2, l ^ 4, and the arithmetic of neighbouring values runs two at a time (packed
// fp32 add, sub, fma, mul: the same roundings). A stage's statements are the reference's whatever lane holds a value: the element
// whose index has the stage's bit clear becomes own + partner, the other partner - own. Per 32 values 24 warp instructions instead of
// 44. A row's transformed values stay in registers as bf16 pairs between the amax and the codes; rows longer than 2048 take two or four
// warps (at most 2048 values each: 80 registers) that exchange their maxima through shared memory.
CAM_DEV void fwht_wide(f32x2 (&p)[8], int l8) {
    // stage 1: the two values of a pair
#pragma unroll
    for (int i = 0; i < 8; i++) { const float a = lo2(p[i]), b = hi2(p[i]); p[i] = pk2(fadd(a, b), fsub(a, b)); }
    // stages 2, 4, 8: pairs of register pairs
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (!(i & h)) { const f32x2 a = p[i], b = p[i + h]; p[i] = add2(a, b); p[i + h] = sub2(a, b); }
    // stages 16, 32, 64: lanes l ^ 1, l ^ 2, l ^ 4 of the chunk's eight
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
        const float sg = (l8 & m) ? -1.0f : 1.0f;        // the upper lane of a pair holds partner - own: fma(own, -1, partner), one rounding
        const f32x2 sg2 = pk2(sg, sg);
#pragma unroll
        for (int i = 0; i < 8; i++)
            p[i] = fma2(p[i], sg2, pk2(__shfl_xor_sync(CAM_FULL, lo2(p[i]), m), __shfl_xor_sync(CAM_FULL, hi2(p[i]), m)));
    }
}
CAM_DEV bool bf16_word_has_nan(uint32_t w) { return (((w & 0x7fff7fffu) + 0x007f007fu) & 0x80008000u) != 0; }

// The block entry as a source of the sixteen-values-per-lane kernel: a prologue per row on the warp (lane l holds the four values 4 l ..
// of every chunk of 128, the layout in which the reference's ordered sums are in-lane fma chains) forms rstd, stores
// hb = bf16((x rstd) w) into the warp's shared-memory slice and the thin projections ab = bf16(hb . wab[j]); the quantiser's steps then
// read hb back sixteen values per lane. Sums: thread tid owns tid + 256 j, wave butterflies, 8 wave sums in order (ref_total_f32's
// statements, the butterfly's additions two accumulators per instruction).
// NCH: the row's chunks of 128 when known at compile time (0: counted from d, up to 8)
template <int NCH>
struct BlockEntrySrc {
    static constexpr int MAXC = NCH ? NCH : 8;
    const float * x; const float * nw; const uint16_t * wab; int nab; float eps; uint16_t * ab; float * rstd_out; int d;
    uint16_t * stage;                              // this warp's slice of shared memory (set by the kernel): d bf16 values
    static constexpr bool kBf16 = true, kHeavy = false, kPrologue = true;
    CAM_DEV void begin_row(bool on, int row, int lane) const {
        const int nch = NCH ? NCH : d >> 7;
        f32x2 u[MAXC][2];                          // chunk c: (v0, v1), (v2, v3) of this lane's four
        const float * xr = x + (size_t)(on ? row : 0) * d + lane * 4;
#pragma unroll
        for (int c = 0; c < MAXC; c++) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            if (on && c < nch) a = __ldg(reinterpret_cast<const float4 *>(xr + c * 128));
            u[c][0] = pk2(a.x, a.y); u[c][1] = pk2(a.z, a.w);
        }
        f32x2 a2[4] = {pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f)};
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nch) { a2[2 * (c & 1)] = fma2(u[c][0], u[c][0], a2[2 * (c & 1)]); a2[2 * (c & 1) + 1] = fma2(u[c][1], u[c][1], a2[2 * (c & 1) + 1]); }
        const float rstd = cam_rsqrt(fadd(fdiv(ref_total_f32_pairs(a2, lane), (float)d), eps));
        if (lane == 0 && on) rstd_out[row] = rstd;
        const f32x2 r2 = pk2(rstd, rstd);
#pragma unroll
        for (int c = 0; c < MAXC; c++)
            if (c < nch) {                         // hb = bf16((x rstd) w): the quantiser's source and the projections' operand
                const float4 w4 = __ldg(reinterpret_cast<const float4 *>(nw + c * 128 + lane * 4));
                const f32x2 h0 = mul2(mul2(u[c][0], r2), pk2(w4.x, w4.y)), h1 = mul2(mul2(u[c][1], r2), pk2(w4.z, w4.w));
                const uint32_t b0 = bf16x2<true>(lo2(h0), hi2(h0)), b1 = bf16x2<true>(lo2(h1), hi2(h1));
                *reinterpret_cast<uint2 *>(stage + c * 128 + lane * 4) = make_uint2(b0, b1);
                u[c][0] = pk2(__uint_as_float(b0 << 16), __uint_as_float(b0 & 0xffff0000u));
                u[c][1] = pk2(__uint_as_float(b1 << 16), __uint_as_float(b1 & 0xffff0000u));
            }
        for (int j = 0; j < nab; j += 2) {         // two projections at a time (an odd count's last one beside a row of zeros)
            const bool two = j + 1 < nab;
            const uint16_t * wr = wab + (size_t)j * d + lane * 4, * wr1 = wr + (two ? d : 0);
            f32x2 pa[4] = {pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f)}, pb[4] = {pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < MAXC; c++)
                if (c < nch) {
                    const uint2 wv = __ldg(reinterpret_cast<const uint2 *>(wr + c * 128)), wz = __ldg(reinterpret_cast<const uint2 *>(wr1 + c * 128));
                    pa[2 * (c & 1)] = fma2(u[c][0], pk2(__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xffff0000u)), pa[2 * (c & 1)]);
                    pa[2 * (c & 1) + 1] = fma2(u[c][1], pk2(__uint_as_float(wv.y << 16), __uint_as_float(wv.y & 0xffff0000u)), pa[2 * (c & 1) + 1]);
                    pb[2 * (c & 1)] = fma2(u[c][0], pk2(__uint_as_float(wz.x << 16), __uint_as_float(wz.x & 0xffff0000u)), pb[2 * (c & 1)]);
                    pb[2 * (c & 1) + 1] = fma2(u[c][1], pk2(__uint_as_float(wz.y << 16), __uint_as_float(wz.y & 0xffff0000u)), pb[2 * (c & 1) + 1]);
                }
            const float tot = ref_total_f32_two(pa, pb, lane);
            if (on && (lane == 0 || (lane == 4 && two))) ab[(size_t)row * nab + j + (lane >> 2)] = f2bf(tot);
        }
        __syncwarp();                              // (hb is read back by other lanes)
    }
    CAM_DEV void get16(bool on, int row, int k, f32x2 (&p)[8]) const {
        uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
        if (on) { const uint4 * r = reinterpret_cast<const uint4 *>(stage + k); a = r[0]; b = r[1]; }
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++) p[i] = pk2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
};

// the codes, dequantised values and stores of one warp step in general: every value clamped (a clip below 1 lets quotients pass qmax; a
// NaN or an infinity among the values needs fminf / fmaxf's treatment of a NaN)
__device__ __noinline__ void actq_wide_emit_clamped(uint4 ua, uint4 ub, float s, float inv, bool fast, float lo, float hi, size_t at, uint16_t * __restrict__ y,
                                                    uint16_t * __restrict__ codes) {
    const uint32_t up[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
    const f32x2 ih2 = pk2(fmul(inv, 0x1.000008p+0f), fmul(inv, 0x1.000008p+0f)), il2 = pk2(fmul(inv, 0x1.fffff0p-1f), fmul(inv, 0x1.fffff0p-1f));
    const f32x2 magic2 = pk2(12582912.0f, 12582912.0f), s2 = pk2(s, s);
    uint32_t yw[8], cw[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t w = up[i];
        const float u0 = __uint_as_float(w << 16), u1 = __uint_as_float(w & 0xffff0000u);
        const f32x2 u = pk2(u0, u1);
        const f32x2 vh = fma2(u, ih2, magic2), vl = fma2(u, il2, magic2);
        const f32x2 r = sub2(vh, magic2);
        f32x2 q2 = pk2(copysignf(lo2(r), u0), copysignf(hi2(r), u1));                                   // (rint keeps the sign of a zero)
        if ((((__float_as_uint(lo2(vh)) ^ __float_as_uint(lo2(vl))) | (__float_as_uint(hi2(vh)) ^ __float_as_uint(hi2(vl)))) != 0) || !fast)
            q2 = pk2(rintf(fdiv(u0, s)), rintf(fdiv(u1, s)));
        const float a = fminf(fmaxf(lo2(q2), lo), hi), b = fminf(fmaxf(hi2(q2), lo), hi);
        const uint32_t na = __float_as_uint(fadd(a, 12582912.0f)) & 0xFu, nb = __float_as_uint(fadd(b, 12582912.0f)) & 0xFu;
        cw[i >> 2] |= (na | (nb << 4)) << (8 * (i & 3));
        const f32x2 d2 = mul2(pk2(a, b), s2);
        yw[i] = bf16x2<true>(lo2(d2), hi2(d2));
    }
    if (y) { st128(y + at, make_uint4(yw[0], yw[1], yw[2], yw[3])); st128(y + at + 8, make_uint4(yw[4], yw[5], yw[6], yw[7])); }
    if (codes) st64(codes + (at >> 2), make_uint2(cw[0], cw[1]));
}

// one pair by the division (no clamp: the caller's row needs none): its two bf16 values and its code byte
__device__ __noinline__ void actq_wide_divided_pair(uint32_t w, float s, uint16_t * __restrict__ y2, uint8_t * __restrict__ code) {
    const float u0 = __uint_as_float(w << 16), u1 = __uint_as_float(w & 0xffff0000u);
    const float q0 = rintf(fdiv(u0, s)), q1 = rintf(fdiv(u1, s));
    if (y2) *reinterpret_cast<uint32_t *>(y2) = bf16x2<true>(fmul(q0, s), fmul(q1, s));
    if (code) *code = (uint8_t)(((uint32_t)(int)q0 & 0xFu) | (((uint32_t)(int)q1 & 0xFu) << 4));
}

// STEPS: warp steps of 512 values per row and warp; WPR: warps per row (1, 2 or 4)
template <typename Src, int STEPS, int WPR, bool SM>
__global__ void __launch_bounds__(256) actq_wide_kernel(Src src, uint16_t * __restrict__ y, float * __restrict__ s_out, int K, float clip, int qmax,
                                                        uint16_t * __restrict__ codes, int M) {
    __shared__ float wmax[8];
    extern __shared__ uint4 aq_sm[];                                     // SM: [warp][step][2][lane], a lane reads back its own words only (no barrier)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g8 = lane >> 3, l8 = lane & 7;
    const int nch = K >> 7;
    const bool y32 = (reinterpret_cast<uintptr_t>(y) & 31u) == 0;
    uint4 * const mine = aq_sm + (SM ? warp * (STEPS * 64) + lane : 0);
    if constexpr (Src::kPrologue) src.stage = reinterpret_cast<uint16_t *>(aq_sm + (SM ? 8 * STEPS * 64 : 0)) + warp * (STEPS * 512);      // (K bf16 values per warp)
    constexpr int RPB = 8 / WPR;                                         // rows per block and pass
    const int part = WPR == 1 ? 0 : (warp & (WPR - 1));                  // this warp's part of the row: chunks part STEPS 4 ..
    for (int r0 = blockIdx.x * RPB; r0 < M; r0 += gridDim.x * RPB) {     // (block-uniform: every warp takes part in the barrier below)
        const int row = r0 + warp / WPR;
        const bool row_on = row < M;
        uint32_t upr[SM ? 1 : STEPS][8];                                 // the transformed values, bf16 pairs (SM: in shared memory instead)
        float amax = 0.f;                                                // over the values before their rounding to bf16 (rounded below: rounding is monotone)
        if constexpr (Src::kPrologue) src.begin_row(row_on, row, lane);
        bool odd = false;                                                // a NaN or an infinity among this lane's transformed values
#pragma unroll (SM ? 1 : STEPS)
        for (int st = 0; st < STEPS; st++) {
            const int ch = (part * STEPS + st) * 4 + g8;
            const bool on = row_on && ch < nch;
            uint32_t w8[8];
            f32x2 p[8];
            src.get16(on, row, ch * 128 + l8 * 16, p);
            fwht_wide(p, l8);
            const f32x2 c2 = pk2(0.08837890625f, 0.08837890625f), zero2 = pk2(0.f, 0.f);
            f32x2 z2 = zero2;                                            // 0 t summed: a NaN iff some t is a NaN or an infinity (one packed fma per pair)
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const f32x2 t = mul2(p[i], c2);
                uint32_t w;
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(hi2(t)), "f"(lo2(t)));
                w8[i] = w;
                z2 = fma2(t, zero2, z2);
                amax = fmaxf(amax, fmaxf(fabsf(lo2(t)), fabsf(hi2(t))));
            }
            const float zs = fadd(lo2(z2), hi2(z2));
            if (zs != zs) {                                              // (a NaN is stored as 0x7fc0, the reference's f2bf; the conversion gives 0x7fff)
                odd = true;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    uint32_t w = w8[i];
                    if ((w & 0x7fffu) > 0x7f80u) w = (w & 0xffff0000u) | 0x7fc0u;
                    if ((w & 0x7fff0000u) > 0x7f800000u) w = (w & 0x0000ffffu) | 0x7fc00000u;
                    w8[i] = w;
                }
            }
            if constexpr (SM) { mine[st * 64] = make_uint4(w8[0], w8[1], w8[2], w8[3]); mine[st * 64 + 32] = make_uint4(w8[4], w8[5], w8[6], w8[7]); }
            else {
#pragma unroll
                for (int i = 0; i < 8; i++) upr[st][i] = w8[i];
            }
        }
        amax = wave_max(amax);
        if (WPR > 1) {
            if (lane == 0) wmax[warp] = amax;
            __syncthreads();
#pragma unroll
            for (int i = 0; i < WPR; i++) amax = fmaxf(amax, wmax[(warp & ~(WPR - 1)) + i]);
            __syncthreads();
        }
        amax = __uint_as_float(bf16x2<false>(amax, 0.f) << 16);          // the largest rounded magnitude = the largest magnitude, rounded (never a NaN)
        const float s = fmaxf(fdiv(fmul(amax, clip), (float)qmax), 1e-8f);
        if (lane == 0 && part == 0 && row_on && s_out) s_out[row] = s;
        const float lo = (float)(-qmax - 1), hi = (float)qmax;
        // rint(u / s) without the division where that is provably the same integer (actq_emit above): two-ended rounding test per value
        const float inv = rcp_approx(s);
        const bool fast = s < 3.0e38f && fmul(amax, inv) < 4.0e6f;       // (s >= 1e-8; false for a NaN)
        // No value passes the clamp when clip >= 1 and every value is a number: |u| <= amax and s >= fl(amax / qmax) put the quotient
        // below qmax + 0.5. The warp then skips the clamp, takes the code from the rounded sum's own low bits (1.5 2^23 + 8 + q holds
        // q + 8 in its last four bits) and the zero's sign from the source word.
        const bool plain = clip >= 1.0f && amax < 3.0e38f && s < 3.0e38f && !__any_sync(CAM_FULL, odd);
        const f32x2 ih2 = pk2(fmul(inv, 0x1.000008p+0f), fmul(inv, 0x1.000008p+0f)), il2 = pk2(fmul(inv, 0x1.fffff0p-1f), fmul(inv, 0x1.fffff0p-1f));
        const f32x2 magic2 = pk2(12582920.0f, 12582920.0f), s2 = pk2(s, s);
#pragma unroll (SM ? 1 : STEPS)
        for (int st = 0; st < STEPS; st++) {
            const int ch = (part * STEPS + st) * 4 + g8;
            if (!(row_on && ch < nch)) continue;
            const size_t at = (size_t)row * K + ch * 128 + l8 * 16;
            uint32_t w8[8];
            if constexpr (SM) {
                const uint4 a = mine[st * 64], b = mine[st * 64 + 32];
                w8[0] = a.x; w8[1] = a.y; w8[2] = a.z; w8[3] = a.w; w8[4] = b.x; w8[5] = b.y; w8[6] = b.z; w8[7] = b.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) w8[i] = upr[st][i];
            }
            if (!plain) {                                                // (out of line: rare, and the straight-line code below stays short)
                actq_wide_emit_clamped(make_uint4(w8[0], w8[1], w8[2], w8[3]), make_uint4(w8[4], w8[5], w8[6], w8[7]), s, inv, fast, lo, hi, at, y, codes);
                continue;
            }
            uint32_t yw[8], nb[8];
            uint32_t bad = fast ? 0u : 0xffu;                            // pairs to divide
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t w = w8[i];
                const f32x2 u = pk2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
                const f32x2 vh = fma2(u, ih2, magic2), vl = fma2(u, il2, magic2);
                // a pair whose two ends differ (a quotient on or next to a .5 boundary: bf16 operands make exact ties common) is divided below
                if (((__float_as_uint(lo2(vh)) ^ __float_as_uint(lo2(vl))) | (__float_as_uint(hi2(vh)) ^ __float_as_uint(hi2(vl)))) != 0) bad |= 1u << i;
                const f32x2 d2 = mul2(sub2(vh, magic2), s2);
                uint32_t yv;
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(yv) : "f"(hi2(d2)), "f"(lo2(d2)));
                yw[i] = yv | (w & 0x80008000u);                          // (rint keeps the sign of a zero; elsewhere the signs agree already)
                nb[i] = __float_as_uint(hi2(vh)) * 16u + __float_as_uint(lo2(vh));        // low byte: (q1 + 8) << 4 | (q0 + 8)
            }
            if (y) {                                                     // (a lane's 32 bytes as one store where they are a whole sector: two 16-byte stores write each sector twice)
                if (y32) st256(y + at, make_uint4(yw[0], yw[1], yw[2], yw[3]), make_uint4(yw[4], yw[5], yw[6], yw[7]));
                else { st128(y + at, make_uint4(yw[0], yw[1], yw[2], yw[3])); st128(y + at + 8, make_uint4(yw[4], yw[5], yw[6], yw[7])); }
            }
            if (codes) {
                const uint32_t c0 = __byte_perm(__byte_perm(nb[0], nb[1], 0x0040), __byte_perm(nb[2], nb[3], 0x0040), 0x5410);
                const uint32_t c1 = __byte_perm(__byte_perm(nb[4], nb[5], 0x0040), __byte_perm(nb[6], nb[7], 0x0040), 0x5410);
                st64(codes + (at >> 2), make_uint2(c0 ^ 0x88888888u, c1 ^ 0x88888888u));
            }
            while (bad) {                                                // a divided pair's word and code byte, stored over the ones above (one pair in 250)
                const int i = __ffs(bad) - 1;
                bad &= bad - 1;
                uint32_t w = w8[0];
#pragma unroll
                for (int k = 1; k < 8; k++) if (k == i) w = w8[k];
                actq_wide_divided_pair(w, s, y ? y + at + 2 * i : nullptr, codes ? reinterpret_cast<uint8_t *>(codes) + (at >> 1) + i : nullptr);
            }
        }
    }
}

// the sixteen-values-per-lane launch: rows of up to 8192 values whose loads and stores are 16-byte aligned; false: the caller's other kernels
template <typename Src>
bool launch_actq_wide(Src src, bool aligned, int M, uint16_t * y, float * s, int K, float clip, int qmax, uint16_t * codes, cudaStream_t stream) {
    if (!aligned || (y && !cam_aligned16(y)) || (codes && (reinterpret_cast<uintptr_t>(codes) & 7u))) return false;
    const long want8 = ((long)M + 7) / 8, want4 = ((long)M + 3) / 4, want2 = ((long)M + 1) / 2;
    // SMV: the row's transformed values wait in shared memory (1 KB per warp and step) and the step loops are loops: a third of the
    // registers and a quarter of the code of the unrolled form, which long rows pay for in resident warps and instruction fetches
    static const char * force = getenv("CAMINUS_B200_ACTQ_SM");            // (tuning: "0" / "1" overrides the choice)
#define CAM_AQ_WIDE(STV, WPRV, WANT, SMV) do { \
        const bool sm = force ? force[0] == '1' : (SMV || (Src::kHeavy && STV > 1)); \
        const size_t pro = Src::kPrologue ? (size_t)8 * STV * 1024 : 0;      /* (a prologue's staged row: STV * 512 bf16 per warp) */ \
        if (sm) actq_wide_kernel<Src, STV, WPRV, true><<<cam_resident_grid(actq_wide_kernel<Src, STV, WPRV, true>, 256, 8 * STV * 1024 + pro, WANT, Src::kPrologue ? 8 : 1), 256, 8 * STV * 1024 + pro, stream>>>(src, y, s, K, clip, qmax, codes, M); \
        else actq_wide_kernel<Src, STV, WPRV, false><<<cam_resident_grid(actq_wide_kernel<Src, STV, WPRV, false>, 256, pro, WANT, Src::kPrologue ? 8 : 1), 256, pro, stream>>>(src, y, s, K, clip, qmax, codes, M); } while (0)
    if (K <= 512) CAM_AQ_WIDE(1, 1, want8, false);
    else if (K <= 1024) CAM_AQ_WIDE(2, 1, want8, false);
    else if (K <= 2048) CAM_AQ_WIDE(4, 1, want8, true);
    else if (K <= 4096) CAM_AQ_WIDE(4, 2, want4, true);
    else CAM_AQ_WIDE(4, 4, want2, true);
#undef CAM_AQ_WIDE
    return true;
}

// the warp-per-row launch when the row fits (K <= 2048) and its loads are aligned; false: the caller uses the block-per-row kernel
template <typename Src>
bool launch_actq_rows(Src src, bool aligned, int M, uint16_t * y, float * s, int K, float clip, int qmax, uint16_t * codes, cudaStream_t stream) {
    if (!aligned || K > 2048) return false;
    const long want = ((long)M + 7) / 8;
    if (K <= 1024) actq_rows_kernel<Src, 8><<<cam_resident_grid(actq_rows_kernel<Src, 8>, 256, 0, want), 256, 0, stream>>>(src, y, s, K, clip, qmax, codes, M);
    else actq_rows_kernel<Src, 16><<<cam_resident_grid(actq_rows_kernel<Src, 16>, 256, 0, want), 256, 0, stream>>>(src, y, s, K, clip, qmax, codes, M);
    return true;
}

int check_actq(int M, int K, int qmax, const void * x, const void * s) {
    if (M < 0 || K < 128 || (K & 127) || K > AQ_WAVES * AQ_MAXC * 128 || qmax < 1 || qmax > 7 || !x || !s) return CAM_ERR_ARG;
    return CAM_OK;
}
bool misaligned8(const void * p) { return p && (reinterpret_cast<uintptr_t>(p) & 7u);
}

}   // namespace

#define CAM_ST (cudaStream_t) stream
// actq_fwd_{bf16,f32} / actq_fwd_codes_{bf16,f32}: kernels/actq.hip:315-326 (M = grid.x); wrapper python/caminus/train/actq.py:22-95.
// y nullable when codes are written; codes nullable.
extern "C" int actq_fwd_codes_bf16(int M, const void * x, void * y, float * s, void * codes, int K, float clip, int qmax, void * stream) {
    const int r = check_actq(M, K, qmax, x, s); if (r || M == 0) return r;
    if (misaligned8(y)) return CAM_ERR_ALIGN;
    if (!launch_actq_wide(PlainBf16{(const uint16_t *)x, K}, cam_aligned16(x), M, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes, CAM_ST) &&
        !launch_actq_rows(PlainBf16{(const uint16_t *)x, K}, !misaligned8(x), M, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes, CAM_ST)) {
        if (!misaligned8(x)) actq_kernel<PlainBf16, true><<<M, 256, 0, CAM_ST>>>(PlainBf16{(const uint16_t *)x, K}, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes);
        else actq_kernel<<<M, 256, 0, CAM_ST>>>(PlainBf16{(const uint16_t *)x, K}, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes);
    }
    return (int)cudaGetLastError();
}
extern "C" int actq_fwd_codes_f32(int M, const float * x, void * y, float * s, void * codes, int K, float clip, int qmax, void * stream) {
    const int r = check_actq(M, K, qmax, x, s); if (r || M == 0) return r;
    if (misaligned8(y)) return CAM_ERR_ALIGN;
    if (!launch_actq_wide(PlainF32{x, K}, cam_aligned16(x), M, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes, CAM_ST) &&
        !launch_actq_rows(PlainF32{x, K}, cam_aligned16(x), M, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes, CAM_ST)) {
        if (cam_aligned16(x)) actq_kernel<PlainF32, true><<<M, 256, 0, CAM_ST>>>(PlainF32{x, K}, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes);
        else actq_kernel<<<M, 256, 0, CAM_ST>>>(PlainF32{x, K}, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes);
    }
    return (int)cudaGetLastError();
}
extern "C" int actq_fwd_bf16(int M, const void * x, void * y, float * s, int K, float clip, int qmax, void * stream) {
    return actq_fwd_codes_bf16(M, x, y, s, nullptr, K, clip, qmax, stream);
}
extern "C" int actq_fwd_f32(int M, const float * x, void * y, float * s, int K, float clip, int qmax, void * stream) {
    return actq_fwd_codes_f32(M, x, y, s, nullptr, K, clip, qmax, stream);
}
// silu_mul_actq_fwd: kernels/actq.hip:307-310 (M = grid.x); wrapper python/caminus/train/actq.py:98-113
extern "C" int silu_mul_actq_fwd(int M, const void * gu, int ld, int F, void * y, float * s, void * codes, float clip, int qmax, void * stream) {
    const int r = check_actq(M, F, qmax, gu, s); if (r) return r;
    if (ld < 2 * F) return CAM_ERR_ARG;
    if (misaligned8(y)) return CAM_ERR_ALIGN;
    if (M == 0) return CAM_OK;
    const bool vec = !misaligned8(gu) && !(ld & 3);
    if (!launch_actq_wide(SiluMulSrc{(const uint16_t *)gu, ld, F}, cam_aligned16(gu) && !(ld & 7), M, (uint16_t *)y, s, F, clip, qmax, (uint16_t *)codes, CAM_ST) &&
        !launch_actq_rows(SiluMulSrc{(const uint16_t *)gu, ld, F}, vec, M, (uint16_t *)y, s, F, clip, qmax, (uint16_t *)codes, CAM_ST)) {
        if (vec) actq_kernel<SiluMulSrc, true><<<M, 256, 0, CAM_ST>>>(SiluMulSrc{(const uint16_t *)gu, ld, F}, (uint16_t *)y, s, F, clip, qmax, (uint16_t *)codes);
        else actq_kernel<<<M, 256, 0, CAM_ST>>>(SiluMulSrc{(const uint16_t *)gu, ld, F}, (uint16_t *)y, s, F, clip, qmax, (uint16_t *)codes);
    }
    return (int)cudaGetLastError();
}
// block_entry_fwd: kernels/actq.hip:247-249 (M = grid.x); wrapper python/caminus/train/actq.py:131-151. d <= 1024 in the reference's
// wrapper (its backward's buffer); the forward here takes d <= 8192.
extern "C" int block_entry_fwd(int M, const float * x, const float * nw, const void * wab, int nab, float eps, void * y, float * s, void * codes,
                               void * ab, float * rstd_out, int d, float clip, int qmax, void * stream) {
    const int r = check_actq(M, d, qmax, x, s); if (r) return r;
    if (!nw || !rstd_out || nab < 0 || nab > AQ_NAB || (nab && (!wab || !ab))) return CAM_ERR_ARG;
    if (misaligned8(y)) return CAM_ERR_ALIGN;
    if (M == 0) return CAM_OK;
    if (d <= 1024 && cam_aligned16(x) && cam_aligned16(nw) && !misaligned8(wab)) {
#define CAM_BE_WIDE(NCHV) launch_actq_wide(BlockEntrySrc<NCHV>{x, nw, (const uint16_t *)wab, nab, eps, (uint16_t *)ab, rstd_out, d, nullptr}, true, M, (uint16_t *)y, s, d, \
                                           clip, qmax, (uint16_t *)codes, CAM_ST)
        const bool done = d == 896 ? CAM_BE_WIDE(7) : d == 1024 ? CAM_BE_WIDE(8) : d == 512 ? CAM_BE_WIDE(4) : CAM_BE_WIDE(0);
#undef CAM_BE_WIDE
        if (done) return (int)cudaGetLastError();
    }
    if (d <= 1024 && cam_aligned16(x) && cam_aligned16(nw) && !misaligned8(wab)) {
        const long want = ((long)M + 7) / 8;
        block_entry_rows_kernel<8><<<cam_resident_grid(block_entry_rows_kernel<8>, 256, 0, want), 256, 0, CAM_ST>>>(
            x, nw, (const uint16_t *)wab, nab, eps, (uint16_t *)y, s, (uint16_t *)codes, (uint16_t *)ab, rstd_out, d, clip, qmax, M);
    } else
        block_entry_kernel<<<M, 256, 0, CAM_ST>>>(x, nw, (const uint16_t *)wab, nab, eps, (uint16_t *)y, s, (uint16_t *)codes, (uint16_t *)ab, rstd_out, d, clip, qmax);
    return (int)cudaGetLastError();
}
