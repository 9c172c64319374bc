// The Coder / hyper-connection line's glue (the reference's kernels/prefill_glue.hip: pf_rms_mul, pf_hc_post_rms, pf_hc_post,
// pf_hc_mean, pf_add_sum, pf_silu_bf16, pf_to_bf16; kernels/prefill_tp.hip: pf_swiglu; kernels/prefill_attn.hip: pf_qk_nr) and
// the training line's forwards (kernels/core.hip: embedding_f32, rmsnorm_f32, silu_mul_bf16, residual3, cast_bf16;
// kernels/fuse.hip: residual_slices_fwd).
//
// The row kernels keep the reference's own mapping: one block of 256 threads per row, thread tid owns elements
// tid + 256 j, an fma chain over j, the 32-lane butterfly (16, 8, 4, 2, 1) and the eight wave sums added in order, so the sum
// of squares has the reference's bits by construction. Elementwise kernels are grid-stride loops over coalesced elements.
#include "cam_common.cuh"

namespace {

constexpr int ROW_MAX_NI = 32;       // row lengths up to 8192

CAM_DEV uint16_t bf16_rne(float v) {       // prefill_glue.hip's to_bf16: round to nearest even, no NaN case (for stored inputs; computed values: bf16_nan)
    const uint32_t u = __float_as_uint(v);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
CAM_DEV uint16_t bf16_nan(float f) {       // core.hip's f2bf: the same, NaN -> 0x7fc0
    uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
CAM_DEV float bf16_f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
CAM_DEV float cam_sigmoid(float v) { return frcp(fadd(1.0f, cam_expf(-v))); }      // (1 / d: the IEEE reciprocal is that quotient)
// four sigmoids with the exponentials' fma chains packed: sum += x * sigmoid(g), element by element
CAM_DEV float4 fma_sigmoid4(float4 x, float4 g, float4 sum) {
    const f32x2 one = pk2(1.0f, 1.0f);
    const f32x2 d0 = add2(one, cam_expf2(-g.x, -g.y)), d1 = add2(one, cam_expf2(-g.z, -g.w));
    return make_float4(ffma(x.x, frcp(lo2(d0)), sum.x), ffma(x.y, frcp(hi2(d0)), sum.y), ffma(x.z, frcp(lo2(d1)), sum.z), ffma(x.w, frcp(hi2(d1)), sum.w));
}

// the block's sum over the threads' partial sums: wave butterfly, eight partials in order (every thread gets the total)
CAM_DEV float block_total(float ss, float * part) {
    const int lane = threadIdx.x & 31, wave = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = fadd(ss, __shfl_xor_sync(CAM_FULL, ss, o));
    if (lane == 0) part[wave] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; q++) tot = fadd(tot, part[q]);
    return tot;
}

// MODE 0: pf_rms_mul. MODE 1: pf_hc_post_rms (x = res updated in place from b and inj). MODE 2: rmsnorm_f32 (out = y).
template <int MODE>
__global__ void __launch_bounds__(256) rms_rows_kernel(const float * x, const float * __restrict__ w, float * y,
                                                       uint16_t * __restrict__ ybf, float * __restrict__ scl, int R, int wr, float eps, int K,
                                                       const float * __restrict__ b, const float * __restrict__ inj, int HC, float rs,
                                                       uint8_t * __restrict__ yq) {
    __shared__ float part[8];
    const int tid = threadIdx.x;
    for (int t = blockIdx.x; t < R; t += gridDim.x) {
        const float * xr = x + (size_t)t * K;
        const float * wv = w + (size_t)(MODE == 1 ? t % HC : MODE == 2 ? 0 : t % wr) * K;
        float xv[ROW_MAX_NI];
#pragma unroll
        for (int j = 0; j < ROW_MAX_NI; j++)
            if (tid + 256 * j < K) xv[j] = xr[tid + 256 * j];
        float ss = 0.0f;
        if (MODE == 1) {
            const float p = fmul(cam_sigmoid(fmul(__ldg(inj + t), rs)), 2.0f);
            const float * br = b + (size_t)(t / HC) * K;
#pragma unroll
            for (int j = 0; j < ROW_MAX_NI; j++)
                if (tid + 256 * j < K) {
                    xv[j] = ffma(__ldg(br + tid + 256 * j), p, xv[j]);
                    const_cast<float *>(xr)[tid + 256 * j] = xv[j];
                }
        }
#pragma unroll
        for (int j = 0; j < ROW_MAX_NI; j++)
            if (tid + 256 * j < K) ss = ffma(xv[j], xv[j], ss);
        const float tot = block_total(ss, part);
        const float scale = cam_rsqrt(fadd(fdiv(tot, (float)K), eps));
        if (scl && tid == 0) scl[t] = scale;
#pragma unroll
        for (int j = 0; j < ROW_MAX_NI; j++)
            if (tid + 256 * j < K) {
                const float v = fmul(fmul(xv[j], scale), __ldg(wv + tid + 256 * j));
                if (y) y[(size_t)t * K + tid + 256 * j] = v;
                if (ybf) ybf[(size_t)t * K + tid + 256 * j] = bf16_nan(v);
                if (yq) {      // the Q8_1 copy (q8_emit: the warp's 32 consecutive values are one block; K a multiple of 32 keeps a warp whole)
                    float amax = fabsf(v), sum = v;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) { amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, o)); sum = fadd(sum, __shfl_xor_sync(CAM_FULL, sum, o)); }
                    const float d = fdiv(amax, 127.0f);
                    const float qv = fdiv(v, d);
                    uint8_t * blk = yq + ((size_t)t * K + tid + 256 * j) / 32 * 36;
                    blk[4 + (tid & 31)] = (uint8_t)((amax != 0.0f && fabsf(qv) < 127.5f) ? __float2int_rn(roundf(qv)) : 0);
                    if ((tid & 31) == 0) *reinterpret_cast<uint32_t *>(blk) = f2_to_h2(d, sum);
                }
            }
        __syncthreads();      // part[] is reused by the next row
    }
}

__global__ void __launch_bounds__(256) hc_post_kernel(const float * __restrict__ b, const float * __restrict__ inj, float * res, int T, int HC, int D, float rs) {
    const long n = (long)T * D;
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long)gridDim.x * 256) {
        const int tt = (int)(i / D), ii = (int)(i - (long)tt * D);
        const float bv = __ldg(b + i);
        for (int h = 0; h < HC; h++) {
            const float ph = fmul(cam_sigmoid(fmul(__ldg(inj + tt * HC + h), rs)), 2.0f);
            const size_t o = (size_t)(tt * HC + h) * D + ii;
            res[o] = ffma(bv, ph, res[o]);
        }
    }
}

__global__ void __launch_bounds__(256) hc_mean_kernel(const float * __restrict__ x, const float * __restrict__ scl, const float * __restrict__ w,
                                                      const float * __restrict__ g, float * __restrict__ out, int T, int HC, int D, float rs) {
    const long n = (long)T * D;
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long)gridDim.x * 256) {
        const int tt = (int)(i / D), ii = (int)(i - (long)tt * D);
        float sum = 0.0f;
        for (int h = 0; h < HC; h++) {
            const size_t o = (size_t)(tt * HC + h) * D + ii;
            const float xv = scl ? fmul(fmul(__ldg(x + o), __ldg(scl + tt * HC + h)), __ldg(w + (size_t)h * D + ii)) : __ldg(x + o);
            sum = ffma(xv, cam_sigmoid(__ldg(g + o)), sum);
        }
        out[i] = fmul(rs, sum);
    }
}

// the two stream kernels, four consecutive elements per thread (D a multiple of 4, 16-byte aligned buffers)
// (a block per token, looping over tokens: no index is divided, and a token's HC gate factors are computed once, not once per thread)
__global__ void __launch_bounds__(256) hc_post_vec_kernel(const float * __restrict__ b, const float * __restrict__ inj, float * res, int T, int HC, int D, float rs) {
    __shared__ float ph_s[32];
    const int D4 = D >> 2;
    for (int tt = blockIdx.x; tt < T; tt += gridDim.x) {
        __syncthreads();                                     // (the previous token's readers are done with ph_s)
        if (threadIdx.x < HC && threadIdx.x < 32) ph_s[threadIdx.x] = fmul(cam_sigmoid(fmul(__ldg(inj + tt * HC + threadIdx.x), rs)), 2.0f);
        __syncthreads();
        for (int i4 = threadIdx.x; i4 < D4; i4 += 256) {
            const float4 bv = __ldg(reinterpret_cast<const float4 *>(b) + (size_t)tt * D4 + i4);
            for (int h = 0; h < HC; h++) {
                const float ph = h < 32 ? ph_s[h] : fmul(cam_sigmoid(fmul(__ldg(inj + tt * HC + h), rs)), 2.0f);
                float4 * o = reinterpret_cast<float4 *>(res + (size_t)(tt * HC + h) * D) + i4;
                const float4 r = *o;
                *o = make_float4(ffma(bv.x, ph, r.x), ffma(bv.y, ph, r.y), ffma(bv.z, ph, r.z), ffma(bv.w, ph, r.w));
            }
        }
    }
}
// (a block per token, looping over tokens: no index is divided; HCT > 0: the stream count at compile time, all streams' loads
// issued before the first sigmoid)
template <int HCT>
__global__ void __launch_bounds__(256) hc_mean_vec_kernel(const float * __restrict__ x, const float * __restrict__ scl, const float * __restrict__ w,
                                                          const float * __restrict__ g, float * __restrict__ out, int T, int HC, int D, float rs) {
    const int D4 = D >> 2, nh = HCT ? HCT : HC;
    constexpr int HM = HCT ? HCT : 1;
    for (int tt = blockIdx.x; tt < T; tt += gridDim.x) {
        for (int i4 = threadIdx.x; i4 < D4; i4 += 256) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (HCT) {
                float4 xv[HM], gv[HM];
#pragma unroll
                for (int h = 0; h < HM; h++) {
                    const size_t o = (size_t)(tt * HM + h) * D4 + i4;
                    xv[h] = __ldg(reinterpret_cast<const float4 *>(x) + o); gv[h] = __ldg(reinterpret_cast<const float4 *>(g) + o);
                }
#pragma unroll
                for (int h = 0; h < HM; h++) {
                    if (scl) {
                        const float sc = __ldg(scl + tt * HM + h);
                        const float4 wv = __ldg(reinterpret_cast<const float4 *>(w) + (size_t)h * D4 + i4);
                        xv[h] = make_float4(fmul(fmul(xv[h].x, sc), wv.x), fmul(fmul(xv[h].y, sc), wv.y), fmul(fmul(xv[h].z, sc), wv.z), fmul(fmul(xv[h].w, sc), wv.w));
                    }
                    sum = fma_sigmoid4(xv[h], gv[h], sum);
                }
            } else {
                for (int h = 0; h < nh; h++) {
                    const size_t o = (size_t)(tt * nh + h) * D4 + i4;
                    float4 xv = __ldg(reinterpret_cast<const float4 *>(x) + o);
                    const float4 gv = __ldg(reinterpret_cast<const float4 *>(g) + o);
                    if (scl) {
                        const float sc = __ldg(scl + tt * nh + h);
                        const float4 wv = __ldg(reinterpret_cast<const float4 *>(w) + (size_t)h * D4 + i4);
                        xv = make_float4(fmul(fmul(xv.x, sc), wv.x), fmul(fmul(xv.y, sc), wv.y), fmul(fmul(xv.z, sc), wv.z), fmul(fmul(xv.w, sc), wv.w));
                    }
                    sum = fma_sigmoid4(xv, gv, sum);
                }
            }
            __stcs(reinterpret_cast<float4 *>(out) + (size_t)tt * D4 + i4, make_float4(fmul(rs, sum.x), fmul(rs, sum.y), fmul(rs, sum.z), fmul(rs, sum.w)));
        }
    }
}

// elementwise ops selected at compile time
enum { EW_ADD_SUM, EW_SWIGLU, EW_RESIDUAL3, EW_CAST_BF16 };
template <int OP>
__global__ void __launch_bounds__(256) ew_kernel(const void * __restrict__ a, const void * __restrict__ b, const void * __restrict__ c, void * y, long n) {
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long)gridDim.x * 256) {
        if (OP == EW_ADD_SUM) { float * yy = (float *)y; yy[i] = fadd(yy[i], fadd(__ldg((const float *)a + i), __ldg((const float *)b + i))); }
        if (OP == EW_SWIGLU) ((float *)y)[i] = fmul(cam_silu(__ldg((const float *)a + i)), __ldg((const float *)b + i));
        if (OP == EW_RESIDUAL3)
            ((float *)y)[i] = fadd(fadd(__ldg((const float *)a + i), bf16_f(__ldg((const uint16_t *)b + i))), bf16_f(__ldg((const uint16_t *)c + i)));
        if (OP == EW_CAST_BF16) ((uint16_t *)y)[i] = bf16_nan(__ldg((const float *)a + i));
    }
}

// the same ops, four consecutive elements per item and two items in flight per thread (16-byte aligned fp32 buffers, 8-byte
// aligned bf16 buffers); the n % 4 last elements go to the first threads of block 0
CAM_DEV float2 bf16x2_f(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u)); }
template <int OP>
CAM_DEV void ew_item(const void * a, const void * b, const void * c, void * y, long i, float4 av, uint2 bw, uint2 cw, float4 bv, float4 yv) {
    if (OP == EW_ADD_SUM)
        *(reinterpret_cast<float4 *>(y) + i) = make_float4(fadd(yv.x, fadd(av.x, bv.x)), fadd(yv.y, fadd(av.y, bv.y)), fadd(yv.z, fadd(av.z, bv.z)), fadd(yv.w, fadd(av.w, bv.w)));
    if (OP == EW_SWIGLU)
        __stcs(reinterpret_cast<float4 *>(y) + i, make_float4(fmul(cam_silu(av.x), bv.x), fmul(cam_silu(av.y), bv.y), fmul(cam_silu(av.z), bv.z), fmul(cam_silu(av.w), bv.w)));
    if (OP == EW_RESIDUAL3) {
        const float2 m0 = bf16x2_f(bw.x), m1 = bf16x2_f(bw.y), l0 = bf16x2_f(cw.x), l1 = bf16x2_f(cw.y);
        __stcs(reinterpret_cast<float4 *>(y) + i, make_float4(fadd(fadd(av.x, m0.x), l0.x), fadd(fadd(av.y, m0.y), l0.y), fadd(fadd(av.z, m1.x), l1.x), fadd(fadd(av.w, m1.y), l1.y)));
    }
    if (OP == EW_CAST_BF16) __stcs(reinterpret_cast<uint2 *>(y) + i, make_uint2(bf16x2<true>(av.x, av.y), bf16x2<true>(av.z, av.w)));
}
template <int OP>
__global__ void __launch_bounds__(256) ew_vec_kernel(const void * __restrict__ a, const void * __restrict__ b, const void * __restrict__ c, void * y, long n) {
    const long n4 = n >> 2, stride = (long)gridDim.x * 256;
    for (long i0 = (long)blockIdx.x * 256 + threadIdx.x; i0 < n4; i0 += 2 * stride) {
        float4 av[2], bv[2], yv[2]; uint2 bw[2], cw[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const long i = i0 + k * stride;
            if (i >= n4) continue;
            av[k] = __ldg(reinterpret_cast<const float4 *>(a) + i);
            if (OP == EW_ADD_SUM || OP == EW_SWIGLU) bv[k] = __ldg(reinterpret_cast<const float4 *>(b) + i);
            if (OP == EW_ADD_SUM) yv[k] = *(reinterpret_cast<const float4 *>(y) + i);
            if (OP == EW_RESIDUAL3) { bw[k] = __ldg(reinterpret_cast<const uint2 *>(b) + i); cw[k] = __ldg(reinterpret_cast<const uint2 *>(c) + i); }
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const long i = i0 + k * stride;
            if (i < n4) ew_item<OP>(a, b, c, y, i, av[k], bw[k], cw[k], bv[k], yv[k]);
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < (int)(n & 3)) {
        const long i = (n4 << 2) + threadIdx.x;
        if (OP == EW_ADD_SUM) { float * yy = (float *)y; yy[i] = fadd(yy[i], fadd(__ldg((const float *)a + i), __ldg((const float *)b + i))); }
        if (OP == EW_SWIGLU) ((float *)y)[i] = fmul(cam_silu(__ldg((const float *)a + i)), __ldg((const float *)b + i));
        if (OP == EW_RESIDUAL3)
            ((float *)y)[i] = fadd(fadd(__ldg((const float *)a + i), bf16_f(__ldg((const uint16_t *)b + i))), bf16_f(__ldg((const uint16_t *)c + i)));
        if (OP == EW_CAST_BF16) ((uint16_t *)y)[i] = bf16_nan(__ldg((const float *)a + i));
    }
}
// pf_silu_bf16 / pf_to_bf16 over items of four elements: item i is row i / K4, columns 4 (i % K4) .. (K4 = K / 4; the division only when
// the rows are strided); items of the padding rows store zeros
template <bool SILU>
__global__ void __launch_bounds__(256) to_bf16_vec_kernel(const float * __restrict__ x, int ldx, uint16_t * __restrict__ y, unsigned live, unsigned all, unsigned K4, float rs) {
    const unsigned stride = gridDim.x * 256u;
    const bool dense = (unsigned)ldx == 4u * K4;
    for (unsigned i0 = blockIdx.x * 256u + threadIdx.x; i0 < all; i0 += 2 * stride) {
        float4 v[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const unsigned i = i0 + k * stride;
            if (i >= live) continue;
            size_t src = (size_t)i * 4;
            if (!dense) { const unsigned r = i / K4; src = (size_t)r * ldx + (size_t)(i - r * K4) * 4; }
            v[k] = __ldg(reinterpret_cast<const float4 *>(x + src));
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const unsigned i = i0 + k * stride;
            if (i >= all) continue;
            uint2 o = make_uint2(0u, 0u);
            if (i < live) {
                if (SILU) {
                    const float gv[4] = {ffma(rs, v[k].x, 0.0f), ffma(rs, v[k].y, 0.0f), ffma(rs, v[k].z, 0.0f), ffma(rs, v[k].w, 0.0f)};
                    uint32_t w2[2];
                    if (silu_bf16_fast<4>(gv, w2) || bf16_pair_has_nan(w2[0]) || bf16_pair_has_nan(w2[1])) {      // (one redo for the item's four: measured faster than one per pair here)
                        w2[0] = bf16_soft<true>(cam_silu(gv[0])) | (bf16_soft<true>(cam_silu(gv[1])) << 16);
                        w2[1] = bf16_soft<true>(cam_silu(gv[2])) | (bf16_soft<true>(cam_silu(gv[3])) << 16);
                    }
                    o = make_uint2(w2[0], w2[1]);
                }
                else o = make_uint2(bf16x2<false>(v[k].x, v[k].y), bf16x2<false>(v[k].z, v[k].w));
            }
            __stcs(reinterpret_cast<uint2 *>(y) + i, o);
        }
    }
}

// silu_mul_bf16 over items of eight elements: item i is row i / H8, columns 8 (i % H8) .. of the rows [g | u] (H8 = H / 8)
__global__ void __launch_bounds__(256) silu_mul_bf16_vec_kernel(const uint16_t * __restrict__ gu, uint16_t * __restrict__ act, unsigned H8, unsigned items) {
    const unsigned stride = gridDim.x * 256u, sdiv = stride / H8, smod = stride - sdiv * H8;
    unsigned i = blockIdx.x * 256u + threadIdx.x;
    if (i >= items) return;
    unsigned r = i / H8, c8 = i - r * H8;                              // (divided once: the next item's row and column follow by addition)
    uint4 gw = ldg128(gu + ((size_t)r * 2 * H8 + c8) * 8), uw = ldg128(gu + ((size_t)r * 2 * H8 + H8 + c8) * 8);
    for (; i < items; i += stride) {
        const uint32_t gs[4] = {gw.x, gw.y, gw.z, gw.w}, us[4] = {uw.x, uw.y, uw.z, uw.w};
        r += sdiv; c8 += smod;
        if (c8 >= H8) { c8 -= H8; r++; }
        if (i + stride < items) {                                      // the next item's loads fly during this item's arithmetic
            gw = ldg128(gu + ((size_t)r * 2 * H8 + c8) * 8); uw = ldg128(gu + ((size_t)r * 2 * H8 + H8 + c8) * 8);
        }
        float gv[8];
#pragma unroll
        for (int k = 0; k < 4; k++) { const float2 g = bf16x2_f(gs[k]); gv[2 * k] = g.x; gv[2 * k + 1] = g.y; }
        uint32_t sw[4], o[4];
        const uint32_t redo = silu_bf16_fast<8>(gv, sw);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 sv = bf16x2_f(sw[k]), u = bf16x2_f(us[k]);
            const float p0 = fmul(sv.x, u.x), p1 = fmul(sv.y, u.y);
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[k]) : "f"(p1), "f"(p0));
            if (((redo >> k) & 1u) || p0 != p0 || p1 != p1) {            // the exact statements for the pair (a NaN: f2bf's 0x7fc0)
                const float s0 = __uint_as_float(bf16_soft<true>(cam_silu(gv[2 * k])) << 16), s1 = __uint_as_float(bf16_soft<true>(cam_silu(gv[2 * k + 1])) << 16);
                o[k] = bf16_soft<true>(fmul(s0, u.x)) | (bf16_soft<true>(fmul(s1, u.y)) << 16);
            }
        }
        st128_stream(act + (size_t)i * 8, make_uint4(o[0], o[1], o[2], o[3]));
    }
}

template <bool SILU>
__global__ void __launch_bounds__(256) to_bf16_kernel(const float * __restrict__ x, int ldx, uint16_t * __restrict__ y, int T, int Tpad, int K, float rs) {
    for (int t = blockIdx.x; t < Tpad; t += gridDim.x)                 // (a block per row: no index is divided)
        for (int j = threadIdx.x; j < K; j += 256) {
            uint16_t v = 0;
            if (t < T) {
                const float xv = __ldg(x + (size_t)t * ldx + j);
                v = SILU ? bf16_nan(cam_silu(ffma(rs, xv, 0.0f))) : bf16_rne(xv);
            }
            y[(size_t)t * K + j] = v;
        }
}

__global__ void __launch_bounds__(256) silu_mul_bf16_kernel(const uint16_t * __restrict__ gu, uint16_t * __restrict__ act, int H, long n) {
    const long rows = n / H;                                           // (whole rows; a block per row: no index is divided per element)
    for (long r = blockIdx.x; r < rows; r += gridDim.x)
        for (int c = threadIdx.x; c < H; c += 256) {
            const float g = bf16_f(__ldg(gu + r * 2 * H + c)), u = bf16_f(__ldg(gu + r * 2 * H + H + c));
            const float s = bf16_f(bf16_nan(cam_silu(g)));
            act[r * H + c] = bf16_nan(fmul(s, u));
        }
    for (long i = rows * H + (long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long)gridDim.x * 256) {      // a last, partial row
        const float g = bf16_f(__ldg(gu + rows * 2 * H + (i - rows * H))), u = bf16_f(__ldg(gu + rows * 2 * H + H + (i - rows * H)));
        act[i] = bf16_nan(fmul(bf16_f(bf16_nan(cam_silu(g))), u));
    }
}

__global__ void __launch_bounds__(256) residual_slices_kernel(const float * __restrict__ x, const uint16_t * __restrict__ m, const uint16_t * __restrict__ mlp,
                                                              const uint16_t * __restrict__ ys, const int * __restrict__ pos, float * __restrict__ out, int d, long n4) {
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < n4; i += (long)gridDim.x * 256) {
        const long e = i * 4; const int r = (int)(e / d), c = (int)(e % d);
        const float4 xv = __ldg(reinterpret_cast<const float4 *>(x + e));
        const uint2 mv = __ldg(reinterpret_cast<const uint2 *>(m + e)), lv = __ldg(reinterpret_cast<const uint2 *>(mlp + e));
        const int p = pos ? __ldg(pos + r) : -1;
        uint2 sv = make_uint2(0, 0);
        if (p >= 0) sv = __ldg(reinterpret_cast<const uint2 *>(ys + (size_t)p * d + c));
        const float xs[4] = {xv.x, xv.y, xv.z, xv.w};
        const uint32_t mw[2] = {mv.x, mv.y}, lw[2] = {lv.x, lv.y}, sw[2] = {sv.x, sv.y};
        float o[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float mk = __uint_as_float((k & 1) ? (mw[k >> 1] & 0xffff0000u) : (mw[k >> 1] << 16));
            const float lk = __uint_as_float((k & 1) ? (lw[k >> 1] & 0xffff0000u) : (lw[k >> 1] << 16));
            const float sk = __uint_as_float((k & 1) ? (sw[k >> 1] & 0xffff0000u) : (sw[k >> 1] << 16));
            o[k] = fadd(fadd(fadd(xs[k], mk), lk), p >= 0 ? sk : 0.0f);
        }
        *reinterpret_cast<float4 *>(out + e) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(256) embedding_f32_kernel(const int * __restrict__ tok, const float * __restrict__ emb, float * __restrict__ out, int D) {
    const int t = blockIdx.x;
    const float * src = emb + (size_t)__ldg(tok + t) * D;
    for (int j = threadIdx.x; j < D; j += 256) out[(size_t)t * D + j] = __ldg(src + j);
}

// a warp per token row, 16 bytes per lane and load (D a multiple of 4, 16-byte aligned table and output)
__global__ void __launch_bounds__(256) embedding_f32_vec_kernel(const int * __restrict__ tok, const float * __restrict__ emb, float * __restrict__ out, int D4, int T) {
    const int lane = threadIdx.x & 31;
    for (int t = blockIdx.x * 8 + (threadIdx.x >> 5); t < T; t += gridDim.x * 8) {
        const float4 * src = reinterpret_cast<const float4 *>(emb) + (size_t)__ldg(tok + t) * D4;
        float4 * dst = reinterpret_cast<float4 *>(out) + (size_t)t * D4;
#pragma unroll 8
        for (int j = lane; j < D4; j += 32) __stcs(dst + j, __ldg(src + j));
    }
}

// pf_qk_nr, a warp per token row looping over the row's heads (D and head_stride multiples of 4, 16-byte aligned buffers, whole token
// rows; NCH = chunks of 128 values per head). The powers theta_scale^j are computed once per block and a token's sines and cosines
// once per token, by the warp that owns it, instead of once per head (the same statements on the same operands give the same bits);
// the sum of squares is the 256-thread order above (ref_total_f32), lane l holding elements 128 m + 4 l .. + 3. The normed head is
// staged in the warp's slice of shared memory, where the rotation reads its partners; the next head's values are loaded before the
// current head is reduced. No barrier after the table of powers.
constexpr int NR_WARPS = 8;
template <int NCH>
__global__ void __launch_bounds__(NR_WARPS * 32) qk_nr_vec_kernel(const float * __restrict__ xin, int head_stride, int heads, const float * __restrict__ w, int D, int nrot,
                                                                  float theta_scale, float eps, int pos0, float * __restrict__ out, int rows) {
    __shared__ float pw[64 * NCH];
    __shared__ __align__(16) float sn_s[NR_WARPS][64 * NCH], cs_s[NR_WARPS][64 * NCH];
    __shared__ __align__(16) float nrm_s[NR_WARPS][128 * NCH];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, half = nrot >> 1;
    for (int j = tid; j < half; j += NR_WARPS * 32) pw[j] = cam_powi(theta_scale, j);
    __syncthreads();
    float * nrm = nrm_s[warp]; float * sns = sn_s[warp]; float * css = cs_s[warp];
    const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 wv[NCH];
#pragma unroll
    for (int m = 0; m < NCH; m++) wv[m] = 128 * m + 4 * lane < D ? __ldg(reinterpret_cast<const float4 *>(w + 128 * m + 4 * lane)) : zero4;
    for (int row = blockIdx.x * NR_WARPS + warp; row < rows; row += gridDim.x * NR_WARPS) {
        const float * x = xin + (size_t)row * heads * head_stride + 4 * lane;
        float4 nx[NCH];
#pragma unroll
        for (int m = 0; m < NCH; m++) nx[m] = 128 * m + 4 * lane < D ? __ldg(reinterpret_cast<const float4 *>(x + 128 * m)) : zero4;
        const float pos = (float)(pos0 + row);
        for (int j = lane; j < half; j += 32) cam_sincos(fmul(pos, pw[j]), sns[j], css[j]);
        __syncwarp();
        for (int h = 0; h < heads; h++) {
            float4 xv[NCH];
#pragma unroll
            for (int m = 0; m < NCH; m++) xv[m] = nx[m];
            if (h + 1 < heads) {
                const float * xn = x + (size_t)(h + 1) * head_stride;
#pragma unroll
                for (int m = 0; m < NCH; m++) nx[m] = 128 * m + 4 * lane < D ? __ldg(reinterpret_cast<const float4 *>(xn + 128 * m)) : zero4;
            }
            float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int m = 0; m < NCH; m++) {
                const int q = 4 * (m & 1);
                a[q + 0] = ffma(xv[m].x, xv[m].x, a[q + 0]); a[q + 1] = ffma(xv[m].y, xv[m].y, a[q + 1]);
                a[q + 2] = ffma(xv[m].z, xv[m].z, a[q + 2]); a[q + 3] = ffma(xv[m].w, xv[m].w, a[q + 3]);
            }
            const float tot = ref_total_f32(a, lane);
            const float scale = cam_rsqrt(fadd(fdiv(tot, (float)D), eps));
#pragma unroll
            for (int m = 0; m < NCH; m++) {
                xv[m] = make_float4(fmul(fmul(scale, xv[m].x), wv[m].x), fmul(fmul(scale, xv[m].y), wv[m].y), fmul(fmul(scale, xv[m].z), wv[m].z),
                                    fmul(fmul(scale, xv[m].w), wv[m].w));
                if (128 * m < nrot) *reinterpret_cast<float4 *>(nrm + 128 * m + 4 * lane) = xv[m];
            }
            __syncwarp();
            float * y = out + ((size_t)row * heads + h) * D + 4 * lane;
#pragma unroll
            for (int m = 0; m < NCH; m++) {
                const int e = 128 * m + 4 * lane;
                if (e >= D) continue;
                float o[4] = {xv[m].x, xv[m].y, xv[m].z, xv[m].w};
                if (e + 3 < nrot && !(half & 3)) {       // the four elements rotate and lie on one side of the half: partners and tables by 16-byte reads
                    const bool low = e < half;
                    const int j = low ? e : e - half;
                    const float4 x0 = *reinterpret_cast<const float4 *>(nrm + j), x1 = *reinterpret_cast<const float4 *>(nrm + j + half);
                    const float4 sn = *reinterpret_cast<const float4 *>(sns + j), cs = *reinterpret_cast<const float4 *>(css + j);
                    o[0] = low ? ffma(x0.x, cs.x, -fmul(x1.x, sn.x)) : ffma(x0.x, sn.x, fmul(x1.x, cs.x));
                    o[1] = low ? ffma(x0.y, cs.y, -fmul(x1.y, sn.y)) : ffma(x0.y, sn.y, fmul(x1.y, cs.y));
                    o[2] = low ? ffma(x0.z, cs.z, -fmul(x1.z, sn.z)) : ffma(x0.z, sn.z, fmul(x1.z, cs.z));
                    o[3] = low ? ffma(x0.w, cs.w, -fmul(x1.w, sn.w)) : ffma(x0.w, sn.w, fmul(x1.w, cs.w));
                } else if (e < nrot) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const int i = e + c;
                        if (i >= nrot) continue;
                        const int j = i < half ? i : i - half;
                        const float x0 = nrm[j], x1 = nrm[j + half], sn = sns[j], cs = css[j];
                        o[c] = i < half ? ffma(x0, cs, -fmul(x1, sn)) : ffma(x0, sn, fmul(x1, cs));
                    }
                }
                __stcs(reinterpret_cast<float4 *>(y + 128 * m), make_float4(o[0], o[1], o[2], o[3]));
            }
            __syncwarp();     // the next head overwrites the slice, the next token the table
        }
    }
}
// Two heads per pass (heads even, D = 128 NCH, the rotated range a multiple of 8 values): the two ordered sums share their shuffles
// (ref_total_f32_two: a lane ends with one head's total and computes that head's scale, a shuffle hands each scale to the other half),
// squares, scale and weight products are packed, the rotation reads partners and tables by 16-byte shared-memory loads with no
// per-element cases: 95 warp instructions per head against 294.
template <int NCH>
__global__ void __launch_bounds__(NR_WARPS * 32) qk_nr_pair_kernel(const float * __restrict__ xin, int head_stride, int heads, const float * __restrict__ w, int nrot,
                                                                   float theta_scale, float eps, int pos0, float * __restrict__ out, int rows) {
    constexpr int D = 128 * NCH;
    __shared__ float pw[64 * NCH];
    __shared__ __align__(16) float sn_s[NR_WARPS][64 * NCH], cs_s[NR_WARPS][64 * NCH];
    __shared__ __align__(16) float nrm_s[NR_WARPS][2][128 * NCH];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, half = nrot >> 1;
    for (int j = tid; j < half; j += NR_WARPS * 32) pw[j] = cam_powi(theta_scale, j);
    __syncthreads();
    float * sns = sn_s[warp]; float * css = cs_s[warp];
    f32x2 wv[NCH][2];
#pragma unroll
    for (int m = 0; m < NCH; m++) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(w + 128 * m + 4 * lane));
        wv[m][0] = pk2(t.x, t.y); wv[m][1] = pk2(t.z, t.w);
    }
    for (int row = blockIdx.x * NR_WARPS + warp; row < rows; row += gridDim.x * NR_WARPS) {
        const float * x = xin + (size_t)row * heads * head_stride + 4 * lane;
        float4 nx[2][NCH];
#pragma unroll
        for (int g = 0; g < 2; g++)
#pragma unroll
            for (int m = 0; m < NCH; m++) nx[g][m] = __ldg(reinterpret_cast<const float4 *>(x + (size_t)g * head_stride + 128 * m));
        const float pos = (float)(pos0 + row);
        for (int j = lane; j < half; j += 32) cam_sincos(fmul(pos, pw[j]), sns[j], css[j]);
        __syncwarp();
        for (int h = 0; h < heads; h += 2) {
            f32x2 xv[2][NCH][2];
#pragma unroll
            for (int g = 0; g < 2; g++)
#pragma unroll
                for (int m = 0; m < NCH; m++) { xv[g][m][0] = pk2(nx[g][m].x, nx[g][m].y); xv[g][m][1] = pk2(nx[g][m].z, nx[g][m].w); }
            if (h + 2 < heads) {
#pragma unroll
                for (int g = 0; g < 2; g++)
#pragma unroll
                    for (int m = 0; m < NCH; m++) nx[g][m] = __ldg(reinterpret_cast<const float4 *>(x + (size_t)(h + 2 + g) * head_stride + 128 * m));
            }
            f32x2 aa[4] = {pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f)}, ab[4] = {pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f), pk2(0.f, 0.f)};
#pragma unroll
            for (int m = 0; m < NCH; m++) {
                const int q = 2 * (m & 1);
                aa[q] = fma2(xv[0][m][0], xv[0][m][0], aa[q]); aa[q + 1] = fma2(xv[0][m][1], xv[0][m][1], aa[q + 1]);
                ab[q] = fma2(xv[1][m][0], xv[1][m][0], ab[q]); ab[q + 1] = fma2(xv[1][m][1], xv[1][m][1], ab[q + 1]);
            }
            const float tot = ref_total_f32_two(aa, ab, lane);            // head h where lane & 4 is clear, head h + 1 elsewhere
            const float own = cam_rsqrt(fadd(fdiv(tot, (float)D), eps));
            const float sc[2] = {__shfl_sync(CAM_FULL, own, lane & ~4), __shfl_sync(CAM_FULL, own, lane | 4)};
#pragma unroll
            for (int g = 0; g < 2; g++) {
                const f32x2 s2 = pk2(sc[g], sc[g]);
#pragma unroll
                for (int m = 0; m < NCH; m++) {
                    xv[g][m][0] = mul2(mul2(s2, xv[g][m][0]), wv[m][0]); xv[g][m][1] = mul2(mul2(s2, xv[g][m][1]), wv[m][1]);
                    if (128 * m < nrot) *reinterpret_cast<float4 *>(nrm_s[warp][g] + 128 * m + 4 * lane) = make_float4(lo2(xv[g][m][0]), hi2(xv[g][m][0]), lo2(xv[g][m][1]), hi2(xv[g][m][1]));
                }
            }
            __syncwarp();
#pragma unroll
            for (int g = 0; g < 2; g++) {
                float * y = out + ((size_t)row * heads + h + g) * D + 4 * lane;
                const float * nrm = nrm_s[warp][g];
#pragma unroll
                for (int m = 0; m < NCH; m++) {
                    const int e = 128 * m + 4 * lane;
                    float4 o = make_float4(lo2(xv[g][m][0]), hi2(xv[g][m][0]), lo2(xv[g][m][1]), hi2(xv[g][m][1]));
                    if (e < nrot) {                  // (nrot a multiple of 8: the four values rotate together and lie on one side of the half)
                        const bool low = e < half;
                        const int j = low ? e : e - half;
                        const float4 x0 = *reinterpret_cast<const float4 *>(nrm + j), x1 = *reinterpret_cast<const float4 *>(nrm + j + half);
                        const float4 sn = *reinterpret_cast<const float4 *>(sns + j), cs = *reinterpret_cast<const float4 *>(css + j);
                        o.x = low ? ffma(x0.x, cs.x, -fmul(x1.x, sn.x)) : ffma(x0.x, sn.x, fmul(x1.x, cs.x));
                        o.y = low ? ffma(x0.y, cs.y, -fmul(x1.y, sn.y)) : ffma(x0.y, sn.y, fmul(x1.y, cs.y));
                        o.z = low ? ffma(x0.z, cs.z, -fmul(x1.z, sn.z)) : ffma(x0.z, sn.z, fmul(x1.z, cs.z));
                        o.w = low ? ffma(x0.w, cs.w, -fmul(x1.w, sn.w)) : ffma(x0.w, sn.w, fmul(x1.w, cs.w));
                    }
                    __stcs(reinterpret_cast<float4 *>(y + 128 * m), o);
                }
            }
            __syncwarp();     // the next pair overwrites the slices, the next token the table
        }
    }
}

template <int NCH>
void launch_qk_nr_vec(const float * xin, int head_stride, int heads, const float * w, int D, int nrot, float theta_scale, float eps, int pos0, float * out, int rows,
                      cudaStream_t stream) {
    const int grid = cam_resident_grid(qk_nr_vec_kernel<NCH>, NR_WARPS * 32, 0, (rows + NR_WARPS - 1) / NR_WARPS);
    qk_nr_vec_kernel<NCH><<<grid, NR_WARPS * 32, 0, stream>>>(xin, head_stride, heads, w, D, nrot, theta_scale, eps, pos0, out, rows);
}

// pf_qk_nr: block t = row * heads + head; D <= 512
__global__ void __launch_bounds__(256) qk_nr_kernel(const float * __restrict__ xin, int head_stride, int heads, const float * __restrict__ w, int D, int nrot,
                                                    float theta_scale, float eps, int pos0, float * __restrict__ out) {
    __shared__ float part[8];
    __shared__ float nrm[512];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float * x = xin + (size_t)t * head_stride;
    float * y = out + (size_t)t * D;
    float ss = 0.0f;
    for (int i = tid; i < D; i += 256) { const float v = __ldg(x + i); ss = ffma(v, v, ss); }
    const float tot = block_total(ss, part);
    const float scale = cam_rsqrt(fadd(fdiv(tot, (float)D), eps));
    for (int i = tid; i < D; i += 256) nrm[i] = fmul(fmul(scale, __ldg(x + i)), __ldg(w + i));
    __syncthreads();
    const float pos = (float)(pos0 + t / heads);
    for (int i = tid; i < D; i += 256) {
        if (i >= nrot) { y[i] = nrm[i]; continue; }
        const int j = i < nrot / 2 ? i : i - nrot / 2;
        float sn, c;
        cam_sincos(fmul(pos, cam_powi(theta_scale, j)), sn, c);
        const float x0 = nrm[j], x1 = nrm[j + nrot / 2];
        y[i] = i < nrot / 2 ? ffma(x0, c, -fmul(x1, sn)) : ffma(x0, sn, fmul(x1, c));
    }
}

int grid_for(long n) {
    const long want = (n + 255) / 256, cap = (long)cam_sm_count() * 8;
    return (int)(want < 1 ? 1 : want < cap ? want : cap);
}

}   // namespace

#define CAM_STREAM (cudaStream_t) stream

// pf_rms_mul: kernels/prefill_glue.hip:94-95; wrapper python/caminus/prefill/glue.py:143-153. K (the reference bakes it into the
// code object: 2560 / 2048 / 5120) is the entry's last argument before the stream; R is also the reference's grid.x.
extern "C" int pf_rms_mul(const float * x, const float * w, float * y, void * ybf, float * scl, int R, int wr, float eps, int K, void * stream) {
    if (R < 0 || wr < 1 || K < 1 || K > 256 * ROW_MAX_NI || !x || !w) return CAM_ERR_ARG;
    if (R == 0) return CAM_OK;
    {   // in place (y == x) is safe on the vector path too: a lane reads all of its row's values before it stores any
        const int r = cam_rms_rows_vec(const_cast<float *>(x), w, y, ybf, scl, R, wr, eps, K, nullptr, nullptr, 1, 0.0f, stream);
        if (r != CAM_ERR_SHAPE) return r;
    }
    rms_rows_kernel<0><<<R < cam_sm_count() * 8 ? R : cam_sm_count() * 8, 256, 0, CAM_STREAM>>>(x, w, y, (uint16_t *)ybf, scl, R, wr, eps, K, nullptr, nullptr, 1, 0.0f, nullptr);
    return (int)cudaGetLastError();
}
// cam_rms_mul_q8_1: pf_rms_mul's norm with the Q8_1 copy of the normed rows the decode op emits for the quantised matvec that follows
// (op_rms_mul with Seg.asum: q8_emit_n, kernels/k3_gguf_ops.h:178-196, 1253): yq = R * K / 32 blocks of 36 bytes, the bytes
// gg_quantize_q8_1 gives for y (quantize_q8_1_lane: lane butterfly sums); y fp32 optional. K a multiple of 32.
extern "C" int cam_rms_mul_q8_1(const float * x, const float * w, float * y, void * yq, int R, int wr, float eps, int K, void * stream) {
    if (R < 0 || wr < 1 || K < 32 || (K & 31) || K > 256 * ROW_MAX_NI || !x || !w || !yq) return CAM_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(yq) & 3u) return CAM_ERR_ALIGN;
    if (R == 0) return CAM_OK;
    {
        const int r = cam_rms_rows_vec(const_cast<float *>(x), w, y, nullptr, nullptr, R, wr, eps, K, nullptr, nullptr, 1, 0.0f, stream, yq);
        if (r != CAM_ERR_SHAPE) return r;
    }
    rms_rows_kernel<0><<<R < cam_sm_count() * 8 ? R : cam_sm_count() * 8, 256, 0, CAM_STREAM>>>(x, w, y, nullptr, nullptr, R, wr, eps, K, nullptr, nullptr, 1, 0.0f, (uint8_t *)yq);
    return (int)cudaGetLastError();
}
// pf_hc_post_rms: kernels/prefill_glue.hip:130-131; wrapper python/caminus/prefill/glue.py:155-164. N = the row length (as K above).
extern "C" int pf_hc_post_rms(const float * b, const float * inj, float * res, const float * w, float * xn, void * xnbf, float * scl, int T, int HC,
                              float rs, float eps, int N, void * stream) {
    if (T < 0 || HC < 1 || N < 1 || N > 256 * ROW_MAX_NI || !b || !inj || !res || !w) return CAM_ERR_ARG;
    const long R = (long)T * HC;
    if (R == 0) return CAM_OK;
    if (R > 0x7fffffffL) return CAM_ERR_SHAPE;
    {
        const int r = cam_rms_rows_vec(res, w, xn, xnbf, scl, (int)R, 1, eps, N, b, inj, HC, rs, stream);
        if (r != CAM_ERR_SHAPE) return r;
    }
    const int grid = (int)(R < (long)cam_sm_count() * 8 ? R : (long)cam_sm_count() * 8);
    rms_rows_kernel<1><<<grid, 256, 0, CAM_STREAM>>>(res, w, xn, (uint16_t *)xnbf, scl, (int)R, 1, eps, N, b, inj, HC, rs, nullptr);
    return (int)cudaGetLastError();
}
// pf_hc_post / pf_hc_mean / pf_add_sum: kernels/prefill_glue.hip:175-176, 194-195, 417
extern "C" int pf_hc_post(const float * b, const float * inj, float * res, int T, int HC, int D, float rs, void * stream) {
    if (T < 0 || HC < 1 || D < 1 || !b || !inj || !res) return CAM_ERR_ARG;
    if (T == 0) return CAM_OK;
    if (!(D & 3) && cam_aligned16(b) && cam_aligned16(res)) hc_post_vec_kernel<<<cam_resident_grid(hc_post_vec_kernel, 256, 0, T, 8), 256, 0, CAM_STREAM>>>(b, inj, res, T, HC, D, rs);
    else hc_post_kernel<<<grid_for((long)T * D), 256, 0, CAM_STREAM>>>(b, inj, res, T, HC, D, rs);
    return (int)cudaGetLastError();
}
extern "C" int pf_hc_mean(const float * x, const float * scl, const float * w, const float * g, float * out, int T, int HC, int D, float rs, void * stream) {
    if (T < 0 || HC < 1 || D < 1 || !x || !g || !out || (scl && !w)) return CAM_ERR_ARG;
    if (T == 0) return CAM_OK;
    if (!(D & 3) && cam_aligned16(x) && cam_aligned16(g) && cam_aligned16(out) && (!w || cam_aligned16(w)))
    {
        if (HC == 4) hc_mean_vec_kernel<4><<<cam_resident_grid(hc_mean_vec_kernel<4>, 256, 0, T), 256, 0, CAM_STREAM>>>(x, scl, w, g, out, T, HC, D, rs);
        else if (HC == 2) hc_mean_vec_kernel<2><<<cam_resident_grid(hc_mean_vec_kernel<2>, 256, 0, T), 256, 0, CAM_STREAM>>>(x, scl, w, g, out, T, HC, D, rs);
        else hc_mean_vec_kernel<0><<<cam_resident_grid(hc_mean_vec_kernel<0>, 256, 0, T), 256, 0, CAM_STREAM>>>(x, scl, w, g, out, T, HC, D, rs);
    }
    else hc_mean_kernel<<<grid_for((long)T * D), 256, 0, CAM_STREAM>>>(x, scl, w, g, out, T, HC, D, rs);
    return (int)cudaGetLastError();
}
extern "C" int pf_add_sum(const float * a, const float * b, float * y, long n, void * stream) {
    if (n < 0 || !a || !b || !y) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (n >= 4 && cam_aligned16(a) && cam_aligned16(b) && cam_aligned16(y))
        ew_vec_kernel<EW_ADD_SUM><<<cam_resident_grid(ew_vec_kernel<EW_ADD_SUM>, 256, 0, ((n >> 2) + 511) / 512, 8), 256, 0, CAM_STREAM>>>(a, b, nullptr, y, n);
    else ew_kernel<EW_ADD_SUM><<<grid_for(n), 256, 0, CAM_STREAM>>>(a, b, nullptr, y, n);
    return (int)cudaGetLastError();
}
// pf_swiglu: kernels/prefill_tp.hip:37-43
extern "C" int pf_swiglu(const float * g, const float * u, float * y, long n, void * stream) {
    if (n < 0 || !g || !u || !y) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (n >= 4 && cam_aligned16(g) && cam_aligned16(u) && cam_aligned16(y))
        ew_vec_kernel<EW_SWIGLU><<<cam_resident_grid(ew_vec_kernel<EW_SWIGLU>, 256, 0, ((n >> 2) + 511) / 512, 8), 256, 0, CAM_STREAM>>>(g, u, nullptr, y, n);
    else ew_kernel<EW_SWIGLU><<<grid_for(n), 256, 0, CAM_STREAM>>>(g, u, nullptr, y, n);
    return (int)cudaGetLastError();
}
// pf_silu_bf16 / pf_to_bf16: kernels/prefill_glue.hip:554, 561
extern "C" int pf_silu_bf16(const float * x, int ldx, void * y, int T, int Tpad, int K, float rs, void * stream) {
    if (T < 0 || Tpad < T || K < 1 || ldx < K || !x || !y) return CAM_ERR_ARG;
    if (Tpad == 0) return CAM_OK;
    if (!(K & 3) && !(ldx & 3) && (long)Tpad * (K >> 2) < 0x7fffffffL && cam_aligned16(x) && !(reinterpret_cast<uintptr_t>(y) & 7u)) {
        const unsigned K4 = (unsigned)(K >> 2), live = (unsigned)T * K4, all = (unsigned)Tpad * K4;
        to_bf16_vec_kernel<true><<<cam_resident_grid(to_bf16_vec_kernel<true>, 256, 0, ((long)all + 511) / 512, 8), 256, 0, CAM_STREAM>>>(x, ldx, (uint16_t *)y, live, all, K4, rs);
    } else to_bf16_kernel<true><<<cam_resident_grid(to_bf16_kernel<true>, 256, 0, Tpad), 256, 0, CAM_STREAM>>>(x, ldx, (uint16_t *)y, T, Tpad, K, rs);
    return (int)cudaGetLastError();
}
extern "C" int pf_to_bf16(const float * x, int ldx, void * y, int T, int Tpad, int K, void * stream) {
    if (T < 0 || Tpad < T || K < 1 || ldx < K || !x || !y) return CAM_ERR_ARG;
    if (Tpad == 0) return CAM_OK;
    if (!(K & 3) && !(ldx & 3) && (long)Tpad * (K >> 2) < 0x7fffffffL && cam_aligned16(x) && !(reinterpret_cast<uintptr_t>(y) & 7u)) {
        const unsigned K4 = (unsigned)(K >> 2), live = (unsigned)T * K4, all = (unsigned)Tpad * K4;
        to_bf16_vec_kernel<false><<<cam_resident_grid(to_bf16_vec_kernel<false>, 256, 0, ((long)all + 511) / 512, 8), 256, 0, CAM_STREAM>>>(x, ldx, (uint16_t *)y, live, all, K4, 0.0f);
    } else to_bf16_kernel<false><<<cam_resident_grid(to_bf16_kernel<false>, 256, 0, Tpad), 256, 0, CAM_STREAM>>>(x, ldx, (uint16_t *)y, T, Tpad, K, 0.0f);
    return (int)cudaGetLastError();
}
// pf_qk_nr: kernels/prefill_attn.hip:105-106 (= op_qk_nr, kernels/k3_gguf_ops.h:1490-1518); nblocks = rows * heads is the reference's grid.x
extern "C" int pf_qk_nr(int nblocks, const float * xin, int head_stride, int heads, const float * w, int D, int nrot, float theta_scale, float eps,
                        int pos0, float * out, void * stream) {
    if (nblocks < 0 || heads < 1 || D < 1 || D > 512 || nrot < 0 || nrot > D || (nrot & 1) || head_stride < D || pos0 < 0 || !xin || !w || !out) return CAM_ERR_ARG;
    if ((long)pos0 + nblocks / heads > (1L << 22)) return CAM_ERR_SHAPE;
    if (nblocks == 0) return CAM_OK;
    if (!(D & 3) && !(head_stride & 3) && nblocks % heads == 0 && cam_aligned16(xin) && cam_aligned16(w) && cam_aligned16(out)) {
        const int rows = nblocks / heads;
        if (!(heads & 1) && !(nrot & 7) && (D == 128 || D == 256)) {       // the usual shapes: two heads per pass; up to 8 x the resident blocks (a block per 8 tokens: 50.3 us against 52.8 us)
            if (D == 128) qk_nr_pair_kernel<1><<<cam_resident_grid(qk_nr_pair_kernel<1>, NR_WARPS * 32, 0, (rows + NR_WARPS - 1) / NR_WARPS, 8), NR_WARPS * 32, 0, CAM_STREAM>>>(
                    xin, head_stride, heads, w, nrot, theta_scale, eps, pos0, out, rows);
            else qk_nr_pair_kernel<2><<<cam_resident_grid(qk_nr_pair_kernel<2>, NR_WARPS * 32, 0, (rows + NR_WARPS - 1) / NR_WARPS, 8), NR_WARPS * 32, 0, CAM_STREAM>>>(
                    xin, head_stride, heads, w, nrot, theta_scale, eps, pos0, out, rows);
            return (int)cudaGetLastError();
        }
        if (D <= 128) launch_qk_nr_vec<1>(xin, head_stride, heads, w, D, nrot, theta_scale, eps, pos0, out, rows, CAM_STREAM);
        else if (D <= 256) launch_qk_nr_vec<2>(xin, head_stride, heads, w, D, nrot, theta_scale, eps, pos0, out, rows, CAM_STREAM);
        else launch_qk_nr_vec<4>(xin, head_stride, heads, w, D, nrot, theta_scale, eps, pos0, out, rows, CAM_STREAM);
    } else qk_nr_kernel<<<nblocks, 256, 0, CAM_STREAM>>>(xin, head_stride, heads, w, D, nrot, theta_scale, eps, pos0, out);
    return (int)cudaGetLastError();
}
// embedding_f32 / rmsnorm_f32 / silu_mul_bf16 / residual3 / cast_bf16: kernels/core.hip:23-66 (T, rows = the reference's grid.x);
// launched from runtime/s1.cpp:14-18, 31, 106
extern "C" int embedding_f32(int T, const int * tok, const float * emb, float * out, int D, void * stream) {
    if (T < 0 || D < 1 || !tok || !emb || !out) return CAM_ERR_ARG;
    if (T == 0) return CAM_OK;
    if (!(D & 3) && cam_aligned16(emb) && cam_aligned16(out))
        embedding_f32_vec_kernel<<<cam_resident_grid(embedding_f32_vec_kernel, 256, 0, (T + 7) / 8), 256, 0, CAM_STREAM>>>(tok, emb, out, D >> 2, T);
    else embedding_f32_kernel<<<T, 256, 0, CAM_STREAM>>>(tok, emb, out, D);
    return (int)cudaGetLastError();
}
extern "C" int rmsnorm_f32(int rows, const float * x, const float * w, float * out, int D, float eps, void * stream) {
    if (rows < 0 || D < 1 || D > 256 * ROW_MAX_NI || !x || !w || !out) return CAM_ERR_ARG;
    if (rows == 0) return CAM_OK;
    {
        const int r = cam_rms_rows_vec(const_cast<float *>(x), w, out, nullptr, nullptr, rows, 1, eps, D, nullptr, nullptr, 1, 0.0f, stream);
        if (r != CAM_ERR_SHAPE) return r;
    }
    rms_rows_kernel<2><<<rows < cam_sm_count() * 8 ? rows : cam_sm_count() * 8, 256, 0, CAM_STREAM>>>(x, w, out, nullptr, nullptr, rows, 1, eps, D, nullptr, nullptr, 1, 0.0f, nullptr);
    return (int)cudaGetLastError();
}
extern "C" int silu_mul_bf16(const void * gu, void * act, int H, long n, void * stream) {
    if (n < 0 || H < 1 || !gu || !act) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    const long rows = n / H;
    if (!(H & 7) && rows > 0 && rows * (H >> 3) < 0x7fffffffL && cam_aligned16(gu) && cam_aligned16(act)) {     // whole rows by vectors, a last partial row by elements
        const unsigned items = (unsigned)(rows * (H >> 3));
        silu_mul_bf16_vec_kernel<<<cam_resident_grid(silu_mul_bf16_vec_kernel, 256, 0, (items + 255) / 256, 8), 256, 0, CAM_STREAM>>>((const uint16_t *)gu, (uint16_t *)act,
                                                                                                                        (unsigned)(H >> 3), items);
        const long rest = n - rows * H;
        if (rest) silu_mul_bf16_kernel<<<grid_for(rest), 256, 0, CAM_STREAM>>>((const uint16_t *)gu + rows * 2 * H, (uint16_t *)act + rows * H, H, rest);
    } else silu_mul_bf16_kernel<<<grid_for(n), 256, 0, CAM_STREAM>>>((const uint16_t *)gu, (uint16_t *)act, H, n);
    return (int)cudaGetLastError();
}
extern "C" int residual3(const float * x, const void * m, const void * y, float * out, long n, void * stream) {
    if (n < 0 || !x || !m || !y || !out) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (n >= 4 && cam_aligned16(x) && cam_aligned16(out) && !(reinterpret_cast<uintptr_t>(m) & 7u) && !(reinterpret_cast<uintptr_t>(y) & 7u))
        ew_vec_kernel<EW_RESIDUAL3><<<cam_resident_grid(ew_vec_kernel<EW_RESIDUAL3>, 256, 0, ((n >> 2) + 511) / 512, 8), 256, 0, CAM_STREAM>>>(x, m, y, out, n);
    else ew_kernel<EW_RESIDUAL3><<<grid_for(n), 256, 0, CAM_STREAM>>>(x, m, y, out, n);
    return (int)cudaGetLastError();
}
extern "C" int cast_bf16(const float * x, void * out, long n, void * stream) {
    if (n < 0 || !x || !out) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (n >= 4 && cam_aligned16(x) && !(reinterpret_cast<uintptr_t>(out) & 7u))
        ew_vec_kernel<EW_CAST_BF16><<<cam_resident_grid(ew_vec_kernel<EW_CAST_BF16>, 256, 0, ((n >> 2) + 511) / 512, 8), 256, 0, CAM_STREAM>>>(x, nullptr, nullptr, out, n);
    else ew_kernel<EW_CAST_BF16><<<grid_for(n), 256, 0, CAM_STREAM>>>(x, nullptr, nullptr, out, n);
    return (int)cudaGetLastError();
}
// residual_slices_fwd: kernels/fuse.hip:19-20; wrapper python/caminus/train/fuse.py:19-30. d a multiple of 4.
extern "C" int residual_slices_fwd(const float * x, const void * m, const void * mlp, const void * ys, const int * pos, float * out, int d, long n4,
                                   void * stream) {
    if (n4 < 0 || d < 4 || (d & 3) || !x || !m || !mlp || !out || (pos && !ys)) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || !cam_aligned16(out) || (reinterpret_cast<uintptr_t>(m) & 7u) || (reinterpret_cast<uintptr_t>(mlp) & 7u) ||
        (ys && (reinterpret_cast<uintptr_t>(ys) & 7u))) return CAM_ERR_ALIGN;
    if (n4 == 0) return CAM_OK;
    residual_slices_kernel<<<grid_for(n4), 256, 0, CAM_STREAM>>>(x, (const uint16_t *)m, (const uint16_t *)mlp, (const uint16_t *)ys, pos, out, d, n4);
    return (int)cudaGetLastError();
}
