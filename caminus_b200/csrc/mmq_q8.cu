// Q8_1 activations in the MMQ layout the quantised GEMMs read (the reference's block_q8_1_mmq, kernels/ggml_mmq/mmq.cuh:63-82):
// a row of K values is cut into blocks of 128; block (kb, row) is stored at index kb * rows + row (column-major by K-block)
// as 144 bytes: 16 bytes of per-32 scales, then 128 int8. Algebra of the reference's quantiser (kernels/ggml_mmq/quantize_mmq.cuh:41-140)
// and of its fused gate / up epilogue (kernels/prefill_moe.hip:364-396): per 32 values amax, d_inv = 127.0f / amax,
// q = roundf(x * d_inv), d = 1.0f / d_inv; D4 stores four fp32 d, DS4 four (fp16 d, fp16 sum) with sum = ((x0 + x1) + x2) + x3
// per four values then partners 4, 2, 1. An all-zero group stores d = 0 and codes 0 explicitly.
//
// Mapping: a lane holds 16 consecutive values (four 16-byte loads of fp32, 8-byte of fp16), two lanes a group of 32, eight lanes a
// block of 128, a warp four consecutive K-blocks of a row; a lane writes its 16 codes as one 16-byte store, the even lanes the
// groups' scales. Consecutive blocks of the grid take consecutive rows, so their 144-byte blocks are adjacent in memory.
#include "cam_common.cuh"

namespace {

// MODE 0: values = x (fp32). MODE 1: silu(x) * u (fp32). MODE 2: silu(g) * u (fp16 in).
// A lane takes 16 consecutive values (two lanes a group of 32, eight lanes a block of 128, a warp four K-blocks), so the group's
// two IEEE divisions and its reductions are spent once per 16 values of a lane. What a lane loads is held raw, so that two rows'
// loads fly together. kvalid and ld are multiples of 4: each of the lane's four quads is all inside the row or all outside.
template <int MODE> struct MmqRaw { float4 a[4], b[4]; };
template <> struct MmqRaw<0> { float4 a[4]; };
template <> struct MmqRaw<2> { uint2 a[4], b[4]; };

template <int MODE>
CAM_DEV void mmq_load(MmqRaw<MODE> & raw, const void * __restrict__ xv, const void * __restrict__ uv, int k, size_t row_at, int kvalid, bool wide = false) {
    if constexpr (MODE == 0) {
        if (wide && k + 16 <= kvalid) {                                   // (rows 32-byte aligned: a lane's 64 bytes as two whole sectors)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint4 a, b;
                ldg256((const float *)xv + row_at + k + 8 * h, a, b);
                raw.a[2 * h] = make_float4(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w));
                raw.a[2 * h + 1] = make_float4(__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w));
            }
            return;
        }
    }
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const bool in = k + 4 * s < kvalid;
        if constexpr (MODE == 2) {
            raw.a[s] = in ? __ldg(reinterpret_cast<const uint2 *>((const uint16_t *)xv + row_at + k + 4 * s)) : make_uint2(0u, 0u);
            raw.b[s] = in ? __ldg(reinterpret_cast<const uint2 *>((const uint16_t *)uv + row_at + k + 4 * s)) : make_uint2(0u, 0u);
        } else {
            raw.a[s] = in ? __ldg(reinterpret_cast<const float4 *>((const float *)xv + row_at + k + 4 * s)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if constexpr (MODE == 1) raw.b[s] = in ? __ldg(reinterpret_cast<const float4 *>((const float *)uv + row_at + k + 4 * s)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
}
// (a quad outside the row loads zeros: silu(0) * 0 = 0 exactly)
CAM_DEV void mmq_values(const MmqRaw<0> & raw, float (&v)[16]) {
#pragma unroll
    for (int s = 0; s < 4; s++) { v[4 * s] = raw.a[s].x; v[4 * s + 1] = raw.a[s].y; v[4 * s + 2] = raw.a[s].z; v[4 * s + 3] = raw.a[s].w; }
}
CAM_DEV void mmq_values(const MmqRaw<1> & raw, float (&v)[16]) {
#pragma unroll
    for (int s = 0; s < 4; s++) {
        v[4 * s] = fmul(cam_silu(raw.a[s].x), raw.b[s].x); v[4 * s + 1] = fmul(cam_silu(raw.a[s].y), raw.b[s].y);
        v[4 * s + 2] = fmul(cam_silu(raw.a[s].z), raw.b[s].z); v[4 * s + 3] = fmul(cam_silu(raw.a[s].w), raw.b[s].w);
    }
}
CAM_DEV void mmq_values(const MmqRaw<2> & raw, float (&v)[16]) {
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const float2 g0 = h2_to_f2(raw.a[s].x), g1 = h2_to_f2(raw.a[s].y), u0 = h2_to_f2(raw.b[s].x), u1 = h2_to_f2(raw.b[s].y);
        v[4 * s] = fmul(cam_silu(g0.x), u0.x); v[4 * s + 1] = fmul(cam_silu(g0.y), u0.y);
        v[4 * s + 2] = fmul(cam_silu(g1.x), u1.x); v[4 * s + 3] = fmul(cam_silu(g1.y), u1.y);
    }
}

// the lane's 16 codes and the group's scale word. The DS4 sum in the reference's order: ((x0 + x1) + x2) + x3 per quad (its
// thread), then the quads' partners 4 (the other lane), 2 and 1 (inside the lane).
template <int LAYOUT>
CAM_DEV void mmq_quant(const float (&v)[16], uint4 & w, uint32_t & hdr) {
    float amax = fabsf(v[0]), ts[4];       // (the reference's thread starts from its first value: 32 NaNs give a NaN maximum and scale; fmaxf skips a NaN among numbers)
#pragma unroll
    for (int s = 0; s < 4; s++) {
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[4 * s]), fabsf(v[4 * s + 1])), fmaxf(fabsf(v[4 * s + 2]), fabsf(v[4 * s + 3]))));
        ts[s] = fadd(fadd(fadd(v[4 * s], v[4 * s + 1]), v[4 * s + 2]), v[4 * s + 3]);
    }
    amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, 1));
    float sum = 0.0f;
    if (LAYOUT == 1) {
#pragma unroll
        for (int s = 0; s < 4; s++) ts[s] = fadd(ts[s], __shfl_xor_sync(CAM_FULL, ts[s], 1));
        sum = fadd(fadd(ts[0], ts[2]), fadd(ts[1], ts[3]));
    }
    float d = 0.0f;
    uint32_t ww[4] = {0u, 0u, 0u, 0u};
    if (amax != 0.0f) {
        const float d_inv = fdiv(127.0f, amax);
        // roundf(t) without the rounding and conversion instructions (the special-function unit's, a quarter of the fp32 rate):
        // t + 1.5 2^23 is t rounded to the nearest integer, ties to even, with that integer's two's complement in the sum's low
        // bits (|t| <= 127 (1 + 2^-23) whenever it is a number). roundf differs on exact ties only, and t - rint(t) is exact, so
        // a lane whose largest |t - rint(t)| stays below 0.5 has its codes; a tie, a NaN or an infinity among the t (0 t summed
        // is then a NaN) sends the lane to the reference's statements below.
        const f32x2 di2 = pk2(d_inv, d_inv), big2 = pk2(12582912.0f, 12582912.0f), zero2 = pk2(0.0f, 0.0f);
        f32x2 z2 = zero2;
        float em = 0.0f;
        uint32_t sb[16];
#pragma unroll
        for (int c = 0; c < 16; c += 2) {
            const f32x2 t2 = prod2(pk2(v[c], v[c + 1]), di2), s2 = add2(t2, big2), e2 = sub2(t2, sub2(s2, big2));      // (prod2: the sums must see the rounded t)
            em = fmaxf(fmaxf(em, fabsf(lo2(e2))), fabsf(hi2(e2)));
            z2 = fma2(t2, zero2, z2);
            sb[c] = __float_as_uint(lo2(s2)); sb[c + 1] = __float_as_uint(hi2(s2));
        }
        const float zs = fadd(lo2(z2), hi2(z2));
        if (em < 0.5f && zs == zs) {
#pragma unroll
            for (int k = 0; k < 4; k++)
                ww[k] = __byte_perm(__byte_perm(sb[4 * k], sb[4 * k + 1], 0x0040), __byte_perm(sb[4 * k + 2], sb[4 * k + 3], 0x0040), 0x5410);
        } else {
#pragma unroll
            for (int c = 0; c < 16; c++) {
                const float t = fmul(v[c], d_inv);
                const int q = fabsf(t) < 127.5f ? __float2int_rn(roundf(t)) : 0;
                ww[c >> 2] |= (uint32_t)(q & 0xff) << (8 * (c & 3));
            }
        }
        d = frcp(d_inv);                                            // (1.0f / d_inv, as the reference writes it: the same bits)
    }
    w = make_uint4(ww[0], ww[1], ww[2], ww[3]);
    hdr = LAYOUT == 0 ? __float_as_uint(d) : f2_to_h2(d, sum);
}
// blk: the lane's K-block (lanes 8 b .. 8 b + 7 of the warp hold K-block b of the warp's four)
CAM_DEV void mmq_write(uint8_t * __restrict__ blk, int lane, uint4 w, uint32_t hdr) {
    st128_stream(blk + 16 + (lane & 7) * 16, w);
    if ((lane & 1) == 0) reinterpret_cast<uint32_t *>(blk)[(lane >> 1) & 3] = hdr;
}

// The indexed forms of the reference's quantiser (kernels/ggml_mmq/quantize_mmq.cuh:41-140; wrappers
// python/caminus/prefill/mmq.py:245-281). Gather (SCATTER false): column c of y = row ids[c] of x (ids null: row c).
// Scatter: row t of x is quantised once and written to the k columns ids[t k + slot] of y (ncols columns in all).
// An index outside its range is clamped (the reference's host code builds them in range).
template <int LAYOUT, bool SCATTER>
__global__ void __launch_bounds__(256) mmq_q8_1_rows_kernel(const float * __restrict__ x, const int * __restrict__ ids, uint8_t * __restrict__ y,
                                                            int kvalid, int nkb, long ld, int nrows, int k, int ncols) {
    const int lane = threadIdx.x & 31;
    for (int kb0 = (blockIdx.y * 8 + (threadIdx.x >> 5)) * 4; kb0 < nkb; kb0 += gridDim.y * 32) {
        const int kb = kb0 + (lane >> 3), kk = kb * 128 + (lane & 7) * 16;
        const bool kon = kb < nkb;
        for (int r = blockIdx.x; r < nrows; r += gridDim.x) {
            int src = r;
            if (!SCATTER && ids) src = min(max(__ldg(ids + r), 0), nrows - 1);
            MmqRaw<0> raw;
            mmq_load<0>(raw, x, nullptr, kk, (size_t)src * ld, kon ? kvalid : 0);
            float v[16];
            mmq_values(raw, v);
            uint4 w; uint32_t hdr;
            mmq_quant<LAYOUT>(v, w, hdr);
            if (!kon) continue;                                   // (after the exchanges: every lane takes part in them)
            if (!SCATTER) mmq_write(y + ((size_t)kb * nrows + r) * 144, lane, w, hdr);
            else
                for (int slot = 0; slot < k; slot++) {
                    const int c = min(max(__ldg(ids + (size_t)r * k + slot), 0), ncols - 1);
                    mmq_write(y + ((size_t)kb * ncols + c) * 144, lane, w, hdr);
                }
        }
    }
}

// A warp's task is a group of four K-blocks of one row (2 KB of fp32 input); the tasks, row-major, go to the warps of the grid in turn,
// so a block reads 16 KB of consecutive input whatever the row length (K-blocks per row a multiple of 32 or not: rows of 40 K-blocks
// left three warps in four idle every second pass when a block owned 32 K-blocks of a row). A warp steps by the grid's warps as
// (rows, groups) with a carry, so no index is divided in the loop; two tasks per pass, both loads issued before either is used.
// ids (nullable): column r of y holds row ids[r] of the inputs, clamped to the rows there are
template <int MODE, int LAYOUT>
__global__ void __launch_bounds__(256) mmq_q8_1_kernel(const void * __restrict__ xv, const void * __restrict__ uv, uint8_t * __restrict__ y,
                                                       int kvalid, int nkb, long ld, int rows, const int * __restrict__ ids) {
    const int lane = threadIdx.x & 31;
    const int ng = (nkb + 3) >> 2;                                        // groups of four K-blocks per row
    const bool wide = MODE == 0 && !(ld & 7) && (reinterpret_cast<uintptr_t>(xv) & 31u) == 0;
    const unsigned first = blockIdx.x * 8u + (threadIdx.x >> 5), nw = gridDim.x * 8u;       // (the launch keeps the grid's warps within the tasks: 32-bit)
    if (first >= (unsigned long)rows * ng) return;                        // (whole warps; no block-wide barrier below)
    int r = (int)(first / (unsigned)ng), g = (int)(first - (unsigned)r * ng);
    const int dr = (int)(nw / (unsigned)ng), dg = (int)(nw - (unsigned)dr * ng);
    while (r < rows) {
        int r2 = r + dr, g2 = g + dg;
        if (g2 >= ng) { g2 -= ng; r2++; }
        const bool two = r2 < rows;
        const int kb = g * 4 + (lane >> 3), kb2 = g2 * 4 + (lane >> 3);
        const bool kon = kb < nkb, kon2 = two && kb2 < nkb;
        MmqRaw<MODE> a0, a1;
        const int s0 = ids ? min(max(__ldg(ids + r), 0), rows - 1) : r, s1 = ids && two ? min(max(__ldg(ids + r2), 0), rows - 1) : r2;
        mmq_load<MODE>(a0, xv, uv, kb * 128 + (lane & 7) * 16, (size_t)s0 * ld, kon ? kvalid : 0, wide);
        if (two) mmq_load<MODE>(a1, xv, uv, kb2 * 128 + (lane & 7) * 16, (size_t)s1 * ld, kon2 ? kvalid : 0, wide);
        float v[16];
        uint4 w; uint32_t hdr;
        mmq_values(a0, v);
        mmq_quant<LAYOUT>(v, w, hdr);
        if (kon) mmq_write(y + ((size_t)kb * rows + r) * 144, lane, w, hdr);
        if (two) {
            mmq_values(a1, v);
            mmq_quant<LAYOUT>(v, w, hdr);
            if (kon2) mmq_write(y + ((size_t)kb2 * rows + r2) * 144, lane, w, hdr);
        }
        r = r2 + dr; g = g2 + dg;
        if (g >= ng) { g -= ng; r++; }
    }
}

// the 2-D persistent grid of the kernels here: x over `nx` units, y over `ny`, together at most the resident blocks
template <typename K>
static dim3 mmq_grid(K kernel, long nx, long ny) {
    const long cap = cam_resident_grid(kernel, 256, 0, 1L << 40, 8);      // (8 x the resident blocks: the fused D4 / DS4 forms 0.69 / 0.57 -> 0.80 / 0.65, the plain quantiser 0.74 -> 0.76)
    const long gx = nx < cap ? (nx < 1 ? 1 : nx) : cap;
    long gy = cap / gx; if (gy < 1) gy = 1; if (gy > ny) gy = ny;
    return dim3((unsigned)gx, (unsigned)gy);
}

// ---- SwiGLU into D4 / DS4 blocks: a fast pass with proof margins, exact recomputation where a margin is not met ---
//
// The scale of this layout is a full fp32 number, d = 1.0f / (127.0f / amax), so it needs the exact statements' amax bit for bit.
// The fast pass evaluates h^ = g * rcp(1 + ex2(-g log2 e)) * u on the special-function unit; with h the exact statements' value
// of an element, |h^ - h| <= EPS |h|, EPS = 1.35e-6, whenever g >= -8 and g is not so small that g / (1 + e) is denormal
// (the derivation is in the header of swiglu_q8_fast_kernel, csrc/swiglu_q8.cu). From that, per group of 32 values:
//   amax:  the element with the largest exact |h| is among those with |h^| >= amax^ (1 - 3e-6) (amax^ = max |h^|). Where
//          exactly one element of the group passes that threshold, it IS the exact argmax, and the exact statements are
//          evaluated for that one element only: amax, d_inv = 127 / amax and d = 1 / d_inv are then the exact statements' bits.
//   codes: t^ = h^ d_inv is within 1.41e-6 |t| of the exact fp32 product t = h d_inv. If t^ (1 - 1.7e-6) and t^ (1 + 1.7e-6) round
//          to the same integer, no rounding boundary and no tie lies in the interval that holds t, and that integer is roundf(t).
// A group where this fails (two candidates, an interval that holds a boundary, some g < -8, a NaN or infinity, amax^ outside
// [1e-30, 3e38)) is recomputed by the whole warp with the exact statements, one lane per value. Every stored byte is
// therefore the exact statements' byte.
//
// Mapping: a lane holds 16 consecutive values (two 16-byte loads of fp16 gate and up), 2 lanes a group of 32, 8 lanes a block
// of 128; a warp takes four K-blocks of two consecutive rows (2 "chunks" of 512 values). The two candidates of a lane pair
// (one per chunk) are moved one to each of its lanes, so that the exact evaluation and the two IEEE divisions run once per
// two chunks; that lane also stores the group's scale. (16 values per lane: the per-step work that does not depend on the
// number of values is spent half as often as with 8.)
// The margins of the proofs above: fp32 gates the analytic EPS = 1.35e-6; fp16 gates the bound enumerated over all 65 536 of them,
// |h^ - h| <= 7.0e-7 |h| (csrc/swiglu_q8.cu, Q8Margins). D4: candidates for the maximum are the elements within 2 EPS (+ slack) of
// amax^; codes t^ = h^ d_inv (exact d_inv) within EPS + 6e-8. DS4: d^ within EPS + 1.3e-7 of d (27 / 14 fp32 ulps: the tie test keeps
// 44 / 24 clear); codes within 2 EPS + 3.0e-7; the sum within EPS + 7.2e-7 of the exact one, in units of A = sum |h^|.
template <typename T> struct MmqMargins {
    static constexpr int TIE = 44;
    static CAM_DEV float candidates() { return 0.999997f; }
    static CAM_DEV float d4_hi() { return 0x1.00001cp+0f; }      // 1 +- 1.67e-6
    static CAM_DEV float d4_lo() { return 0x1.ffffc8p-1f; }
    static CAM_DEV float ds4_hi() { return 0x1.000036p+0f; }     // 1 +- 3.2e-6
    static CAM_DEV float ds4_lo() { return 0x1.ffff94p-1f; }
    static CAM_DEV float sum() { return 2.3e-6f; }
};
template <> struct MmqMargins<uint16_t> {
    static constexpr int TIE = 24;
    static CAM_DEV float candidates() { return 0.9999984f; }     // 1 - 1.6e-6
    static CAM_DEV float d4_hi() { return 0x1.000010p+0f; }      // 1 +- 9.5e-7
    static CAM_DEV float d4_lo() { return 0x1.ffffe0p-1f; }
    static CAM_DEV float ds4_hi() { return 0x1.000020p+0f; }     // 1 +- 1.91e-6
    static CAM_DEV float ds4_lo() { return 0x1.ffffc0p-1f; }
    static CAM_DEV float sum() { return 1.6e-6f; }
};
CAM_DEV float max_nan(float a, float b) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
// bits |= bit where |h| >= thr (a compare and a predicated OR)
CAM_DEV void or_if_ge(uint32_t & bits, float h, float thr, uint32_t bit) {
    asm("{\n .reg .pred p;\n setp.ge.f32 p, %1, %2;\n @p or.b32 %0, %0, %3;\n}" : "+r"(bits) : "f"(fabsf(h)), "f"(thr), "r"(bit));
}

// 8 consecutive values as they were loaded: widened on use, so that the next task's loads can fly during this task's arithmetic
template <typename T> struct Raw8;
template <> struct Raw8<uint16_t> {
    uint4 v;
    CAM_DEV void load(const uint16_t * p) { v = ldg128(p); }
    CAM_DEV void fill(float x) { const uint32_t w = f2_to_h2(x, x); v = make_uint4(w, w, w, w); }
    CAM_DEV void get(float (&f)[8]) const {
        const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), c = h2_to_f2(v.z), e = h2_to_f2(v.w);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = e.x; f[7] = e.y;
    }
    CAM_DEV float pick(int i) const {
        const uint32_t w = i < 4 ? (i < 2 ? v.x : v.y) : (i < 6 ? v.z : v.w);
        return __half2float(__ushort_as_half((uint16_t)((i & 1) ? w >> 16 : w)));
    }
};
template <> struct Raw8<float> {
    float4 a, b;
    CAM_DEV void load(const float * p) { a = __ldg(reinterpret_cast<const float4 *>(p)); b = __ldg(reinterpret_cast<const float4 *>(p) + 1); }
    CAM_DEV void fill(float x) { a = make_float4(x, x, x, x); b = a; }
    CAM_DEV void get(float (&f)[8]) const { f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w; }
    CAM_DEV float pick(int i) const {
        const float4 h = i < 4 ? a : b;
        return (i & 2) ? ((i & 1) ? h.w : h.z) : ((i & 1) ? h.y : h.x);
    }
};

// a warp's task: K-blocks 4 kq .. 4 kq + 3 (8 lanes each, 16 values per lane) of rows r0, r0 + 1
template <bool IDS> struct MmqTask {
    int r0, kb, k, s0, s1;                       // s0, s1: the input rows of output columns r0, r0 + 1 (IDS false: the columns themselves)
    bool kon, kin;
    CAM_DEV MmqTask(int kq, int rp, int lane, int nkb, int kvalid, const int * __restrict__ ids, int rows) {
        r0 = rp * 2;
        kb = kq * 4 + (lane >> 3); k = kb * 128 + (lane & 7) * 16;
        kon = kb < nkb; kin = kon && k < kvalid;
        s0 = r0; s1 = r0 + 1;
        if (IDS) {
            if (r0 < rows) s0 = min(max(__ldg(ids + r0), 0), rows - 1);
            if (r0 + 1 < rows) s1 = min(max(__ldg(ids + r0 + 1), 0), rows - 1);
        }
    }
};

// chunk c (row r0 + c) of a task: a lane's 16 values as two loads of 8
// (256-bit loads of a lane's 32 or 64 bytes, which help the plain quantiser above, cost this kernel a fifth of its speed)
template <typename T, bool IDS>
CAM_DEV void mmq_fetch(const T * __restrict__ g, const T * __restrict__ u, const MmqTask<IDS> & t, long ld, int rows, Raw8<T> (&rg)[2][2], Raw8<T> (&ru)[2][2]) {
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const size_t at = (size_t)(c ? t.s1 : t.s0) * ld + t.k;
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
            if (t.kin && t.r0 + c < rows) { rg[c][hf].load(g + at + 8 * hf); ru[c][hf].load(u + at + 8 * hf); }
            else { rg[c][hf].fill(1.0f); ru[c][hf].fill(0.0f); }      // h = 0 on both passes
        }
    }
}

// PF: the next task's values are loaded before this task's arithmetic (fp16: 32 more registers)
// LAYOUT 1 (DS4: the header word of a group is (fp16 d, fp16 sum)) needs no exact amax: d^ = amax^ / 127 is within 27 fp32 ulps of the
// exact statements' d; where its low 13 bits are more than 44 from the fp16 rounding tie and d^ is in fp16's normal range, fp16(d^) is
// the stored scale. Codes: t^ = h^ (127 rcp(amax^)) is within 3.06e-6 |t| of the exact product; the two-ended test with 1 -+ 3.2e-6.
// Sum: the fast pass adds the h^ in the reference's order (((x0 + x1) + x2) + x3 per four, then partners 4, 2, 1: six levels); its sum is
// within 2.07e-6 A of the exact statements', A = sum |h^|; where S^ - 2.3e-6 A and S^ + 2.3e-6 A round to one fp16, that is the stored sum.
// Groups that fail any of it (about 7 % of Gaussian groups, most of them by the sum) are recomputed exactly as for D4.
template <typename T, bool PF, int LAYOUT, bool IDS>
__global__ void __launch_bounds__(256, 2) mmq_swiglu_fast_kernel(const T * __restrict__ g, const T * __restrict__ u, uint8_t * __restrict__ y,
                                                                 int kvalid, int nkb, long ld, int rows, const int * __restrict__ ids) {
    const int lane = threadIdx.x & 31, pb = lane & 30, pi = lane & 1;      // a group of 32 values = the lane pair pb, pb + 1
    // grid.x walks pairs of rows (8 per block, one per warp), grid.y the quads of K-blocks; no index is divided
    const int nrp = (rows + 1) >> 1, nkq = (nkb + 3) >> 2;
    const int rp0 = blockIdx.x * 8 + (threadIdx.x >> 5), rstride = gridDim.x * 8;
    if (rp0 >= nrp) return;
    int kq = blockIdx.y, rp = rp0;
    Raw8<T> rg[2][2], ru[2][2], ng[2][2], nu[2][2];
    if (PF && kq < nkq) mmq_fetch(g, u, MmqTask<IDS>(kq, rp, lane, nkb, kvalid, ids, rows), ld, rows, rg, ru);
    while (kq < nkq) {
        const MmqTask<IDS> t(kq, rp, lane, nkb, kvalid, ids, rows);
        const int kq_now = kq;
        rp += rstride;                                                // the next task
        if (rp >= nrp) { rp = rp0; kq += gridDim.y; }
        if (!PF) mmq_fetch(g, u, t, ld, rows, rg, ru);
        else if (kq < nkq) mmq_fetch(g, u, MmqTask<IDS>(kq, rp, lane, nkb, kvalid, ids, rows), ld, rows, ng, nu);
        float h[2][16], eg = 1.0f, eu = 0.0f;
        float am2[2] = {0.0f, 0.0f}, sum2[2] = {0.0f, 0.0f}, sab2[2] = {0.0f, 0.0f};      // DS4: the chunks' amax^, S^, A
        uint32_t bad = 0;                                             // bit c: chunk c of this lane fails a margin
#pragma unroll
        for (int c = 0; c < 2; c++) {
            float gv[16], uv[16];
            {
                float t8[8];
                rg[c][0].get(t8);
#pragma unroll
                for (int e = 0; e < 8; e++) gv[e] = t8[e];
                rg[c][1].get(t8);
#pragma unroll
                for (int e = 0; e < 8; e++) gv[8 + e] = t8[e];
                ru[c][0].get(t8);
#pragma unroll
                for (int e = 0; e < 8; e++) uv[e] = t8[e];
                ru[c][1].get(t8);
#pragma unroll
                for (int e = 0; e < 8; e++) uv[8 + e] = t8[e];
            }
            float amax = 0.0f, gmin = gv[0], gsm = fabsf(gv[0]);
            const f32x2 nlog2e = pk2(-0x1.715476p+0f, -0x1.715476p+0f), one2 = pk2(1.0f, 1.0f);      // two values per instruction: the same roundings
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
                const f32x2 g2 = pk2(gv[e], gv[e + 1]);
                const f32x2 a2 = mul2(g2, nlog2e);
                const f32x2 den = add2(one2, pk2(ex2_approx(lo2(a2)), ex2_approx(hi2(a2))));
                const f32x2 hh = mul2(mul2(g2, pk2(rcp_approx(lo2(den)), rcp_approx(hi2(den)))), pk2(uv[e], uv[e + 1]));
                h[c][e] = lo2(hh); h[c][e + 1] = hi2(hh);
                amax = max_nan(amax, max_nan(fabsf(h[c][e]), fabsf(h[c][e + 1])));
                gmin = fminf(gmin, fminf(gv[e], gv[e + 1]));
                if (sizeof(T) == 4) gsm = fminf(gsm, fminf(fabsf(gv[e]), fabsf(gv[e + 1])));
            }
            amax = max_nan(amax, __shfl_xor_sync(CAM_FULL, amax, 1));
            if constexpr (LAYOUT == 0) {
                const float thr = fmul(amax, MmqMargins<T>::candidates());
                uint32_t bits = 0;
#pragma unroll
                for (int e = 0; e < 16; e++) or_if_ge(bits, h[c][e], thr, 1u << e);
                const uint32_t ball = (__ballot_sync(CAM_FULL, bits != 0) >> pb) & 0x3u;
                if ((bits & (bits - 1)) != 0 || ball == 3u || ball == 0 || !(gmin >= -8.0f) || !(amax >= 1.0e-30f && amax < 3.0e38f) ||
                    (sizeof(T) == 4 && !(gsm >= 3.0e-38f))) bad |= 1u << c;
                const int idx = (__ffs(bits) - 1) & 15, src = pb + ((ball >> 1) & 1u);
                const float cg = idx < 8 ? rg[c][0].pick(idx) : rg[c][1].pick(idx - 8), cu = idx < 8 ? ru[c][0].pick(idx) : ru[c][1].pick(idx - 8);
                const float tg = __shfl_sync(CAM_FULL, cg, src), tu = __shfl_sync(CAM_FULL, cu, src);
                if (pi == c) { eg = tg; eu = tu; }
            } else {
                float ts[4], sab = 0.0f;
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {
                    ts[q4] = fadd(fadd(fadd(h[c][4 * q4], h[c][4 * q4 + 1]), h[c][4 * q4 + 2]), h[c][4 * q4 + 3]);
                    sab = fadd(sab, fadd(fadd(fabsf(h[c][4 * q4]), fabsf(h[c][4 * q4 + 1])), fadd(fabsf(h[c][4 * q4 + 2]), fabsf(h[c][4 * q4 + 3]))));
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) ts[q4] = fadd(ts[q4], __shfl_xor_sync(CAM_FULL, ts[q4], 1));      // partner 4
                sum2[c] = fadd(fadd(ts[0], ts[2]), fadd(ts[1], ts[3]));                                          // partners 2, 1
                sab2[c] = fadd(sab, __shfl_xor_sync(CAM_FULL, sab, 1));
                am2[c] = amax;
                if (!(gmin >= -8.0f) || (sizeof(T) == 4 && !(gsm >= 3.0e-38f))) bad |= 1u << c;
            }
        }
        // D4: the exact statements for the pair's two candidates, one per lane
        float d_inv = 0.0f, d = 0.0f;
        if constexpr (LAYOUT == 0) {
            const float am = fabsf(fmul(cam_silu(eg), eu));
            d_inv = fdiv(127.0f, am); d = frcp(d_inv);
        }
        uint32_t hdr2[2] = {0u, 0u};
        uint8_t * const yb = y + ((size_t)t.kb * rows + t.r0) * 144;           // row r0's block of this lane's K-block
        uint32_t redo = 0, resum = 0;                                 // bit 2 j + c: group j (of the warp's 16) of chunk c is recomputed / only its sum is
#pragma unroll
        for (int c = 0; c < 2; c++) {
            float inv_hi, inv_lo;
            bool open = (bad >> c) & 1u, sum_open = false;       // (sum_open alone: scale and codes are proven, only the sum is recomputed)
            if constexpr (LAYOUT == 0) {
                const float di = __shfl_sync(CAM_FULL, d_inv, pb + c);
                inv_hi = fmul(di, MmqMargins<T>::d4_hi()); inv_lo = fmul(di, MmqMargins<T>::d4_lo());
            } else {
                const float dh = fmul(am2[c], 0x1.020408p-7f), di = fmul(127.0f, rcp_approx(am2[c]));
                inv_hi = fmul(di, MmqMargins<T>::ds4_hi()); inv_lo = fmul(di, MmqMargins<T>::ds4_lo());
                const int low = (int)(__float_as_uint(dh) & 0x1fffu) - 0x1000;
                const float margin = fmul(sab2[c], MmqMargins<T>::sum());
                open = open || !(dh >= 6.2e-5f && dh < 6.0e4f) || (low >= -MmqMargins<T>::TIE && low <= MmqMargins<T>::TIE) || !(fabsf(sum2[c]) < 3.0e38f);
                sum_open = __half_as_ushort(__float2half_rn(fsub(sum2[c], margin))) != __half_as_ushort(__float2half_rn(fadd(sum2[c], margin)));
                hdr2[c] = f2_to_h2(dh, sum2[c]);
            }
            uint32_t v[16], differ = 0;
            const f32x2 ih2 = pk2(inv_hi, inv_hi), il2 = pk2(inv_lo, inv_lo), magic2 = pk2(12582912.0f, 12582912.0f);
#pragma unroll
            for (int e = 0; e < 16; e += 2) {
                const f32x2 hh = pk2(h[c][e], h[c][e + 1]), a = fma2(hh, ih2, magic2), b = fma2(hh, il2, magic2);
                v[e] = __float_as_uint(lo2(a)); v[e + 1] = __float_as_uint(hi2(a));
                differ |= (v[e] ^ __float_as_uint(lo2(b))) | (v[e + 1] ^ __float_as_uint(hi2(b)));
            }
            const bool on = t.kon && t.r0 + c < rows;
            const uint32_t mask = __ballot_sync(CAM_FULL, (differ != 0 || open) && on);
            const uint32_t pair = (mask | (mask >> 1)) & 0x55555555u;
            redo |= pair << c;
            if constexpr (LAYOUT == 1) {
                const uint32_t ms = __ballot_sync(CAM_FULL, sum_open && on);
                resum |= ((ms | (ms >> 1)) & 0x55555555u & ~pair) << c;
            }
            if (on && !((pair >> pb) & 1u)) {
                uint4 w;
                w.x = __byte_perm(__byte_perm(v[0], v[1], 0x0040), __byte_perm(v[2], v[3], 0x0040), 0x5410);
                w.y = __byte_perm(__byte_perm(v[4], v[5], 0x0040), __byte_perm(v[6], v[7], 0x0040), 0x5410);
                w.z = __byte_perm(__byte_perm(v[8], v[9], 0x0040), __byte_perm(v[10], v[11], 0x0040), 0x5410);
                w.w = __byte_perm(__byte_perm(v[12], v[13], 0x0040), __byte_perm(v[14], v[15], 0x0040), 0x5410);
                st128_stream(yb + c * 144 + 16 + (lane & 7) * 16, w);
            }
        }
        // the scale of chunk pi, group (lane / 2) % 4 of this lane's K-block (this lane evaluated it)
        if (t.kon && t.r0 + pi < rows && !(((redo | resum) >> (pb + pi)) & 1u))
            reinterpret_cast<uint32_t *>(yb + pi * 144)[(lane >> 1) & 3] = LAYOUT == 0 ? __float_as_uint(d) : (pi ? hdr2[1] : hdr2[0]);
        // DS4 groups whose scale and codes are proven and whose sum is not: the exact values' sum in the reference's order, one lane per value
        for (uint32_t m = resum; m; m &= m - 1) {
            const int bit = __ffs(m) - 1, j = bit >> 1, c = bit & 1;
            const int kbj = kq_now * 4 + (j >> 2), kj = kbj * 128 + (j & 3) * 32 + lane;
            float x = 0.0f;
            if (kj < kvalid) {
                const size_t at = (size_t)(c ? t.s1 : t.s0) * ld + kj;
                x = fmul(cam_silu(Load8<T>::one(g + at)), Load8<T>::one(u + at));
            }
            float sq = fadd(x, __shfl_down_sync(CAM_FULL, x, 1));
            sq = fadd(sq, __shfl_down_sync(CAM_FULL, x, 2));
            sq = fadd(sq, __shfl_down_sync(CAM_FULL, x, 3));
            sq = fadd(sq, __shfl_xor_sync(CAM_FULL, sq, 16));
            sq = fadd(sq, __shfl_xor_sync(CAM_FULL, sq, 8));
            sq = fadd(sq, __shfl_xor_sync(CAM_FULL, sq, 4));
            const uint32_t hd = __shfl_sync(CAM_FULL, c ? hdr2[1] : hdr2[0], 2 * j);      // the group's proven fp16 scale (its pair's even lane)
            if (lane == 0) reinterpret_cast<uint32_t *>(y + ((size_t)kbj * rows + t.r0 + c) * 144)[j & 3] = (hd & 0xffffu) | ((uint32_t)__half_as_ushort(__float2half_rn(sq)) << 16);
        }
        // exact recomputation of the flagged groups: the whole warp, one lane per value (uniform: redo is the same in every lane)
        for (uint32_t m = redo; m; m &= m - 1) {
            const int bit = __ffs(m) - 1, j = bit >> 1, c = bit & 1;     // group j of the warp's 16: K-block j / 4, group j % 4
            const int kbj = kq_now * 4 + (j >> 2), kj = kbj * 128 + (j & 3) * 32 + lane;
            float x = 0.0f;
            if (kj < kvalid) {
                const size_t at = (size_t)(c ? t.s1 : t.s0) * ld + kj;
                x = fmul(cam_silu(Load8<T>::one(g + at)), Load8<T>::one(u + at));
            }
            float a = fabsf(x);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(CAM_FULL, a, o));
            uint8_t * blk = y + ((size_t)kbj * rows + t.r0 + c) * 144;
            float de = 0.0f;
            int code = 0;
            if (a != 0.0f) {
                const float di = fdiv(127.0f, a), tq = fmul(x, di);
                code = fabsf(tq) < 127.5f ? __float2int_rn(roundf(tq)) : 0;
                de = frcp(di);
            }
            blk[16 + (j & 3) * 32 + lane] = (uint8_t)code;
            if constexpr (LAYOUT == 0) { if (lane == 0) reinterpret_cast<float *>(blk)[j & 3] = de; }
            else {      // the sum in the reference's order: ((x0 + x1) + x2) + x3 in the first lane of four, then the eight quads' partners 4, 2, 1
                float sq = fadd(x, __shfl_down_sync(CAM_FULL, x, 1));
                sq = fadd(sq, __shfl_down_sync(CAM_FULL, x, 2));
                sq = fadd(sq, __shfl_down_sync(CAM_FULL, x, 3));
                sq = fadd(sq, __shfl_xor_sync(CAM_FULL, sq, 16));
                sq = fadd(sq, __shfl_xor_sync(CAM_FULL, sq, 8));
                sq = fadd(sq, __shfl_xor_sync(CAM_FULL, sq, 4));
                if (lane == 0) reinterpret_cast<uint32_t *>(blk)[j & 3] = f2_to_h2(de, sq);
            }
        }
        if (PF) {
#pragma unroll
            for (int c = 0; c < 2; c++)
#pragma unroll
                for (int hf = 0; hf < 2; hf++) { rg[c][hf] = ng[c][hf]; ru[c][hf] = nu[c][hf]; }
        }
    }
}

template <int MODE>
int launch_mmq(const void * x, const void * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, cudaStream_t stream, const int * ids = nullptr) {
    if (rows < 0 || Kpad < 128 || (Kpad & 127) || kvalid < 0 || kvalid > Kpad || (kvalid & 3) || ld < kvalid || (ld & 3) || !x || !y ||
        (MODE != 0 && !u) || (layout != 0 && layout != 1)) return CAM_ERR_ARG;
    const int elt = MODE == 2 ? 8 : 16;
    if ((reinterpret_cast<uintptr_t>(x) & (elt - 1)) || (u && (reinterpret_cast<uintptr_t>(u) & (elt - 1))) || !cam_aligned16(y) ||
        (ids && (reinterpret_cast<uintptr_t>(ids) & 3u))) return CAM_ERR_ALIGN;
    if (rows == 0) return CAM_OK;
    if (MODE != 0 && !(kvalid & 15) && !(ld & 7) && cam_aligned16(x) && cam_aligned16(u)) {
        const long nx = ((rows + 1) / 2 + 7) / 8, ny = (Kpad / 128 + 3) / 4;
#define CAM_MMQ_FAST1(TT, PF, LAY, IDSV) mmq_swiglu_fast_kernel<TT, PF, LAY, IDSV><<<mmq_grid(mmq_swiglu_fast_kernel<TT, PF, LAY, IDSV>, nx, ny), 256, 0, stream>>>( \
                (const TT *)x, (const TT *)u, (uint8_t *)y, kvalid, Kpad / 128, ld, rows, ids)
#define CAM_MMQ_FAST(TT, PF, LAY) do { if (ids) CAM_MMQ_FAST1(TT, PF, LAY, true); else CAM_MMQ_FAST1(TT, PF, LAY, false); } while (0)
        if (MODE == 2) { if (layout == 0) CAM_MMQ_FAST(uint16_t, true, 0); else CAM_MMQ_FAST(uint16_t, true, 1); }
        else { if (layout == 0) CAM_MMQ_FAST(float, false, 0); else CAM_MMQ_FAST(float, false, 1); }
#undef CAM_MMQ_FAST1
#undef CAM_MMQ_FAST
        return (int)cudaGetLastError();
    }
    const long want = ((long)rows * ((Kpad / 128 + 3) / 4) + 7) / 8;     // (warp tasks / 8)
    if (layout == 0) mmq_q8_1_kernel<MODE, 0><<<cam_resident_grid(mmq_q8_1_kernel<MODE, 0>, 256, 0, want, 8), 256, 0, stream>>>(x, u, (uint8_t *)y, kvalid, Kpad / 128, ld, rows, ids);
    else mmq_q8_1_kernel<MODE, 1><<<cam_resident_grid(mmq_q8_1_kernel<MODE, 1>, 256, 0, want, 8), 256, 0, stream>>>(x, u, (uint8_t *)y, kvalid, Kpad / 128, ld, rows, ids);
    return (int)cudaGetLastError();
}

}   // namespace

// cam_quantize_mmq_q8_1: rows of x (fp32, row stride ld floats, kvalid values each, zero-padded to Kpad = a multiple of 128) ->
// blocks [Kpad / 128][rows] of 144 bytes; layout 0 = D4, 1 = DS4. The dense case (no ids, one channel) of the reference's
// quantize_mmq_q8_1, kernels/ggml_mmq/quantize_mmq.cuh:41-45.
extern "C" int cam_quantize_mmq_q8_1(const float * x, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream) {
    return launch_mmq<0>(x, nullptr, y, kvalid, Kpad, ld, rows, layout, (cudaStream_t)stream);
}
// cam_swiglu_mmq_q8_1[_f16]: the same blocks of silu(g) * u: what the reference's fused gate / up kernel writes for the down
// projection (kernels/prefill_moe.hip:339-396), as a standalone producer for fp32 or fp16 gate and up.
extern "C" int cam_swiglu_mmq_q8_1(const float * g, const float * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream) {
    return launch_mmq<1>(g, u, y, kvalid, Kpad, ld, rows, layout, (cudaStream_t)stream);
}
extern "C" int cam_swiglu_mmq_q8_1_f16(const void * g, const void * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream) {
    return launch_mmq<2>(g, u, y, kvalid, Kpad, ld, rows, layout, (cudaStream_t)stream);
}

// cam_swiglu_mmq_q8_1[_f16]_ids: column c of y (ncols columns) = the blocks of silu(g) * u of row ids[c] of gate and up (ids null: row c;
// an index outside [0, ncols) is clamped): the fused producer for expert-grouped columns, where the reference's gate / up kernel writes
// column c0 + j of its work item (kernels/prefill_moe.hip:389-394) and its unfused path gathers rows through quantize_mmq_q8_1's index
// (python/caminus/prefill/mmq.py:245-262). gate and up hold ncols rows of stride s01.
extern "C" int cam_swiglu_mmq_q8_1_ids(const float * g, const float * u, const int * ids, void * y, int K, int Kpad, long s01, int ncols, int layout, void * stream) {
    return launch_mmq<1>(g, u, y, K, Kpad, s01, ncols, layout, (cudaStream_t)stream, ids);
}
extern "C" int cam_swiglu_mmq_q8_1_f16_ids(const void * g, const void * u, const int * ids, void * y, int K, int Kpad, long s01, int ncols, int layout, void * stream) {
    return launch_mmq<2>(g, u, y, K, Kpad, s01, ncols, layout, (cudaStream_t)stream, ids);
}

// cam_quantize_mmq_q8_1_ids: column c of y (ncols columns) = row ids[c] of x (ids null: row c); x fp32 with row stride s01 floats,
// K values per row (a multiple of 4), zero-padded to Kpad. The reference's quantize_mmq_q8_1<layout, false>,
// kernels/ggml_mmq/quantize_mmq.cuh:41-45 (instances kernels/prefill_mmq.hip:101-107); wrapper Mmq.quantize,
// python/caminus/prefill/mmq.py:245-262.
extern "C" int cam_quantize_mmq_q8_1_ids(const float * x, const int * ids, void * y, int K, int Kpad, long s01, int ncols, int layout, void * stream) {
    if (ncols < 0 || Kpad < 128 || (Kpad & 127) || K < 0 || K > Kpad || (K & 3) || s01 < K || (s01 & 3) || !x || !y || (layout != 0 && layout != 1)) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || !cam_aligned16(y) || (ids && (reinterpret_cast<uintptr_t>(ids) & 3u))) return CAM_ERR_ALIGN;
    if (ncols == 0) return CAM_OK;
    const long ny = (Kpad / 128 + 31) / 32;
    if (layout == 0) mmq_q8_1_rows_kernel<0, false><<<mmq_grid(mmq_q8_1_rows_kernel<0, false>, ncols, ny), 256, 0, (cudaStream_t)stream>>>(x, ids, (uint8_t *)y, K, Kpad / 128, s01, ncols, 1, ncols);
    else mmq_q8_1_rows_kernel<1, false><<<mmq_grid(mmq_q8_1_rows_kernel<1, false>, ncols, ny), 256, 0, (cudaStream_t)stream>>>(x, ids, (uint8_t *)y, K, Kpad / 128, s01, ncols, 1, ncols);
    return (int)cudaGetLastError();
}
// cam_quantize_mmq_q8_1_scatter: row t of x (ntok rows, stride s_tok floats) quantised once and written to the k columns
// ids_inv[t k + slot] of y (ntok k columns). The reference's quantize_mmq_q8_1<layout, true>; wrapper Mmq.quantize_scatter,
// python/caminus/prefill/mmq.py:264-281.
extern "C" int cam_quantize_mmq_q8_1_scatter(const float * x, const int * ids_inv, void * y, int K, int Kpad, long s_tok, int ntok, int k, int layout,
                                             void * stream) {
    if (ntok < 0 || k < 1 || Kpad < 128 || (Kpad & 127) || K < 0 || K > Kpad || (K & 3) || s_tok < K || (s_tok & 3) || !x || !y || !ids_inv ||
        (layout != 0 && layout != 1) || (long)ntok * k > 0x7fffffffL) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || !cam_aligned16(y) || (reinterpret_cast<uintptr_t>(ids_inv) & 3u)) return CAM_ERR_ALIGN;
    if (ntok == 0) return CAM_OK;
    const long ny = (Kpad / 128 + 31) / 32;
    if (layout == 0) mmq_q8_1_rows_kernel<0, true><<<mmq_grid(mmq_q8_1_rows_kernel<0, true>, ntok, ny), 256, 0, (cudaStream_t)stream>>>(x, ids_inv, (uint8_t *)y, K, Kpad / 128, s_tok, ntok, k, ntok * k);
    else mmq_q8_1_rows_kernel<1, true><<<mmq_grid(mmq_q8_1_rows_kernel<1, true>, ntok, ny), 256, 0, (cudaStream_t)stream>>>(x, ids_inv, (uint8_t *)y, K, Kpad / 128, s_tok, ntok, k, ntok * k);
    return (int)cudaGetLastError();
}
