// Residual add + RMSNorm (the reference's q3p_add_rms16, kernels/q3m_prefill.hip:382-415, = own_op_add_rms16,
// kernels/k3_own_ops.h:305-383; q35p_add_rms16, kernels/q35_prefill.hip:628-660, = q35_op_add_rms16,
// kernels/k3_q35_ops.h:88-130), an fp16-storage form of the same statements, and a tensor-parallel pair.
//
// The reference runs one workgroup of 256 threads per row: thread tid owns elements tid + 256 j, sums their squares in an
// fma chain over j, the 8 waves reduce by the xor butterfly (partners 16, 8, 4, 2, 1) and the 8 wave sums are added in
// order. Here ONE WARP owns a row and every lane stands for 8 of the reference's threads, with 128-bit accesses:
//   fp32 rows: lane l reads float4 chunks at 4l + 128 m; accumulator (c, m & 1) is reference thread v = 4l + c + 128 (m & 1),
//              whose chain runs over j = m >> 1 in order. v's wave is (l >> 3) + 4 (m & 1), its wave lane 4 (l & 7) + c:
//              butterfly partners 16, 8, 4 are lanes l ^ 4, l ^ 2, l ^ 1; partners 2 and 1 are inside the lane.
//   fp16 rows: lane l reads 8 halves at 8l + 256 m; accumulator c is thread v = 8l + c, chain over j = m; wave l >> 2, wave
//              lane 8 (l & 3) + c: partners 16, 8 are lanes l ^ 2, l ^ 1; partners 4, 2, 1 are inside the lane.
// Adding in that order reproduces the reference's sum of squares bit for bit (addition is commutative, so both partners of
// a butterfly step hold the same bits), without a block-wide barrier.
#include "cam_common.cuh"

#include <cstdlib>

#include <mutex>

namespace {

// ---- the reference's reduction on this file's two layouts ------------------------------------------------------------------
// (ref_total_f32, the fp32 layout's reduction, is in cam_common.cuh: the training line's block entry uses it too)
// (ref_total_f16, the fp16 layout's reduction, is in cam_common.cuh as well: the one-kernel tensor-parallel norm uses it)

// ---- fp32 rows ----------------------------------------------------------------------------------------------------------
// CH > 0: N = 128 CH, the row stays in registers. CH = 0: any N (a multiple of 256), the row is read again from memory.
// Q35: x = x + d (one addend). Otherwise the weighted slots of q3p_add_rms16: acc from 0 in slot order.
constexpr int RMS_WARPS = 4;

CAM_DEV float4 add4(float4 a, float4 b) { return make_float4(fadd(a.x, b.x), fadd(a.y, b.y), fadd(a.z, b.z), fadd(a.w, b.w)); }
CAM_DEV float4 fma4(float w, float4 d, float4 acc) { return make_float4(ffma(w, d.x, acc.x), ffma(w, d.y, acc.y), ffma(w, d.z, acc.z), ffma(w, d.w, acc.w)); }

// the generic-N path's per-chunk addend (one chunk at a time)
CAM_DEV float4 slot_add(float4 xv, const float * __restrict__ dr, const float * __restrict__ wr, int S, int N, int i, bool q35) {
    if (q35) return add4(xv, __ldg(reinterpret_cast<const float4 *>(dr + i)));
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int sl = 0; sl < S; sl++) {
        const float4 dv = __ldg(reinterpret_cast<const float4 *>(dr + (size_t)sl * N + i));
        acc = wr ? fma4(__ldg(wr + sl), dv, acc) : add4(acc, dv);
    }
    return add4(xv, acc);
}

CAM_DEV void norm_store(float4 xv, float scale, float4 wv, float * hr, uint16_t * h16r, int i) {
    const float4 v = make_float4(fmul(fmul(xv.x, scale), wv.x), fmul(fmul(xv.y, scale), wv.y), fmul(fmul(xv.z, scale), wv.z),
                                 fmul(fmul(xv.w, scale), wv.w));
    if (hr) __stcs(reinterpret_cast<float4 *>(hr + i), v);
    st64_stream(h16r + i, make_uint2(f2_to_h2(v.x, v.y), f2_to_h2(v.z, v.w)));
}

template <int CH>
__global__ void __launch_bounds__(RMS_WARPS * 32) add_rms_f32_kernel(float * __restrict__ x, const float * __restrict__ d,
                                                                     const float * __restrict__ w, int S, const float * __restrict__ nw,
                                                                     float eps, float * __restrict__ h, uint16_t * __restrict__ h16,
                                                                     int N, int n, int q35) {
    __shared__ __align__(16) float snw[CH > 0 ? 128 * CH : 4];          // the norm weights, staged once per block (CH > 0)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nch = CH > 0 ? CH : N >> 7;
    const bool add = q35 ? d != nullptr : S > 0;
    if (CH > 0) {
        for (int i = threadIdx.x * 4; i < 128 * CH; i += RMS_WARPS * 128) *reinterpret_cast<float4 *>(snw + i) = __ldg(reinterpret_cast<const float4 *>(nw + i));
        __syncthreads();
    }
    for (int t = blockIdx.x * RMS_WARPS + warp; t < n; t += gridDim.x * RMS_WARPS) {
        float * xr = x + (size_t)t * N;
        const float * dr = d ? d + (size_t)t * (q35 ? 1 : S) * N : nullptr;
        const float * wr = w ? w + (size_t)t * S : nullptr;
        float * hr = h ? h + (size_t)t * N : nullptr;
        uint16_t * h16r = h16 + (size_t)t * N;
        float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (CH > 0) {
            // every load of a phase is issued before any of its values is used: a warp keeps the whole row in flight
            float4 xv[CH > 0 ? CH : 1];
#pragma unroll
            for (int m = 0; m < CH; m++) xv[m] = *reinterpret_cast<const float4 *>(xr + 4 * lane + 128 * m);
            if (add) {
                if (q35 || (S == 1 && !wr)) {        // one addend: x + d (q35p), x + (0 + d) (q3p's accumulator from 0)
                    float4 dv[CH > 0 ? CH : 1];
#pragma unroll
                    for (int m = 0; m < CH; m++) dv[m] = __ldg(reinterpret_cast<const float4 *>(dr + 4 * lane + 128 * m));
#pragma unroll
                    for (int m = 0; m < CH; m++) xv[m] = add4(xv[m], q35 ? dv[m] : add4(make_float4(0.0f, 0.0f, 0.0f, 0.0f), dv[m]));
                } else {                             // the slots in order, each slot's row loaded whole
                    float4 acc[CH > 0 ? CH : 1];
#pragma unroll
                    for (int m = 0; m < CH; m++) acc[m] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    for (int sl = 0; sl < S; sl++) {
                        float4 dv[CH > 0 ? CH : 1];
#pragma unroll
                        for (int m = 0; m < CH; m++) dv[m] = __ldg(reinterpret_cast<const float4 *>(dr + (size_t)sl * N + 4 * lane + 128 * m));
                        if (wr) {
                            const float ws = __ldg(wr + sl);
#pragma unroll
                            for (int m = 0; m < CH; m++) acc[m] = fma4(ws, dv[m], acc[m]);
                        } else {
#pragma unroll
                            for (int m = 0; m < CH; m++) acc[m] = add4(acc[m], dv[m]);
                        }
                    }
#pragma unroll
                    for (int m = 0; m < CH; m++) xv[m] = add4(xv[m], acc[m]);
                }
#pragma unroll
                for (int m = 0; m < CH; m++) *reinterpret_cast<float4 *>(xr + 4 * lane + 128 * m) = xv[m];
            }
#pragma unroll
            for (int m = 0; m < CH; m++) {
                const int b = 4 * (m & 1);
                a[b + 0] = ffma(xv[m].x, xv[m].x, a[b + 0]); a[b + 1] = ffma(xv[m].y, xv[m].y, a[b + 1]);
                a[b + 2] = ffma(xv[m].z, xv[m].z, a[b + 2]); a[b + 3] = ffma(xv[m].w, xv[m].w, a[b + 3]);
            }
            const float tot = ref_total_f32(a, lane);
            const float scale = cam_rsqrt(fadd(fdiv(tot, (float)N), eps));
#pragma unroll
            for (int m = 0; m < CH; m++)
                norm_store(xv[m], scale, *reinterpret_cast<const float4 *>(snw + 4 * lane + 128 * m), hr, h16r, 4 * lane + 128 * m);
        } else {
            for (int m = 0; m < nch; m += 2) {                 // (N is a multiple of 256: chunks come in pairs b = 0, 1)
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    const int i = 4 * lane + 128 * (m + b);
                    float4 xv = *reinterpret_cast<const float4 *>(xr + i);
                    if (add) { xv = slot_add(xv, dr, wr, S, N, i, q35); *reinterpret_cast<float4 *>(xr + i) = xv; }
                    a[4 * b + 0] = ffma(xv.x, xv.x, a[4 * b + 0]); a[4 * b + 1] = ffma(xv.y, xv.y, a[4 * b + 1]);
                    a[4 * b + 2] = ffma(xv.z, xv.z, a[4 * b + 2]); a[4 * b + 3] = ffma(xv.w, xv.w, a[4 * b + 3]);
                }
            }
            const float tot = ref_total_f32(a, lane);
            const float scale = cam_rsqrt(fadd(fdiv(tot, (float)N), eps));
            for (int m = 0; m < nch; m++) {      // (each lane reads back what it wrote itself)
                const int i = 4 * lane + 128 * m;
                norm_store(*reinterpret_cast<const float4 *>(xr + i), scale, __ldg(reinterpret_cast<const float4 *>(nw + i)), hr, h16r, i);
            }
        }
    }
}

// A few rows (decode: T = 1): one block of 256 threads per row with the reference's own mapping (thread tid owns
// tid + 256 j), so that a row's loads are spread over 8 warps and its latency is one trip to memory, not sixteen
// loads deep in one warp. N <= 2048.
__global__ void __launch_bounds__(256) add_rms_f32_row_kernel(float * __restrict__ x, const float * __restrict__ d, const float * __restrict__ w,
                                                              int S, const float * __restrict__ nw, float eps, float * __restrict__ h,
                                                              uint16_t * __restrict__ h16, int N, int q35) {
    __shared__ float part[8];
    const int tid = threadIdx.x, lane = tid & 31, wave = tid >> 5, NI = N >> 8, t = blockIdx.x;
    float * xr = x + (size_t)t * N;
    const float * dr = d ? d + (size_t)t * (q35 ? 1 : S) * N : nullptr;
    const float * wr = w ? w + (size_t)t * S : nullptr;
    const bool add = q35 ? d != nullptr : S > 0;
    float xv[8], wv[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
        if (j < NI) { xv[j] = xr[tid + 256 * j]; wv[j] = __ldg(nw + tid + 256 * j); }
    if (add) {
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (j < NI) {
                if (q35) xv[j] = fadd(xv[j], __ldg(dr + tid + 256 * j));
                else {
                    float acc = 0.0f;
                    for (int sl = 0; sl < S; sl++) {
                        const float dv = __ldg(dr + (size_t)sl * N + tid + 256 * j);
                        acc = wr ? ffma(__ldg(wr + sl), dv, acc) : fadd(acc, dv);
                    }
                    xv[j] = fadd(xv[j], acc);
                }
                xr[tid + 256 * j] = xv[j];
            }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++)
        if (j < NI) ss = ffma(xv[j], xv[j], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = fadd(ss, __shfl_xor_sync(CAM_FULL, ss, o));
    if (lane == 0) part[wave] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; q++) tot = fadd(tot, part[q]);
    const float scale = cam_rsqrt(fadd(fdiv(tot, (float)N), eps));
#pragma unroll
    for (int j = 0; j < 8; j++)
        if (j < NI) {
            const float v = fmul(fmul(xv[j], scale), wv[j]);
            if (h) h[(size_t)t * N + tid + 256 * j] = v;
            h16[(size_t)t * N + tid + 256 * j] = f_to_h(v);
        }
}

// ---- the hyper-connection line's row norms on the warp-per-row mapping (pf_rms_mul, pf_hc_post_rms; K = 128 CH) -----------------
// The same reference-order reduction as above. POST: the row is res[t, h], first updated in place to fma(b[t], p, res) with
// p = 2 sigmoid(inj[t, h] rs). Outputs optional: y fp32, ybf bf16 (round to nearest even as prefill_glue.hip's to_bf16; a NaN result stays a NaN, 0x7fc0: see bf16_soft), scl.
// Q8: also the Q8_1 copy of the normed row (yq: 36-byte blocks, the bytes of gg_quantize_q8_1 on y). 8 adjacent lanes hold a block
// of 32. The block sum follows the quantiser's 32-lane butterfly (partners 16, 8, 4 are lanes l ^ 4, 2, 1 here, partners 2, 1
// are inside the lane). The codes roundf(v / d) come from v * rcp(d) where that provably rounds the same way: the product is
// within 1.8e-7 |t| of the IEEE quotient; if t (1 - 4.8e-7) and t (1 + 4.8e-7) round to one integer, no rounding boundary lies
// between them and that integer is the quotient's. A lane where they differ (or with a zero, tiny or non-finite block) divides.
template <int CH, bool POST, bool Q8>
__global__ void __launch_bounds__(RMS_WARPS * 32) rms_rows_vec_kernel(float * x, const float * __restrict__ w, float * y, uint16_t * __restrict__ ybf,
                                                                      float * __restrict__ scl, int R, int wr, float eps, const float * __restrict__ b,
                                                                      const float * __restrict__ inj, int HC, float rs, uint8_t * __restrict__ yq) {
    constexpr int K = 128 * CH;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int t = blockIdx.x * RMS_WARPS + warp; t < R; t += gridDim.x * RMS_WARPS) {
        float * xr = x + (size_t)t * K + 4 * lane;
        float4 xv[CH];
#pragma unroll
        for (int m = 0; m < CH; m++) xv[m] = *reinterpret_cast<const float4 *>(xr + 128 * m);
        if (POST) {
            const float * br = b + (size_t)(t / HC) * K + 4 * lane;
            const float p = fmul(frcp(fadd(1.0f, cam_expf(-fmul(__ldg(inj + t), rs)))), 2.0f);
#pragma unroll
            for (int m = 0; m < CH; m++) {
                const float4 bv = __ldg(reinterpret_cast<const float4 *>(br + 128 * m));
                xv[m] = make_float4(ffma(bv.x, p, xv[m].x), ffma(bv.y, p, xv[m].y), ffma(bv.z, p, xv[m].z), ffma(bv.w, p, xv[m].w));
                *reinterpret_cast<float4 *>(xr + 128 * m) = xv[m];
            }
        }
        unsigned long long redo = 0;                           // Q8: bit m: this lane's four values of chunk m take the exact statements
        float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int m = 0; m < CH; m++) {
            const int q = 4 * (m & 1);
            a[q + 0] = ffma(xv[m].x, xv[m].x, a[q + 0]); a[q + 1] = ffma(xv[m].y, xv[m].y, a[q + 1]);
            a[q + 2] = ffma(xv[m].z, xv[m].z, a[q + 2]); a[q + 3] = ffma(xv[m].w, xv[m].w, a[q + 3]);
        }
        const float tot = ref_total_f32(a, lane);
        const float scale = cam_rsqrt(fadd(fdiv(tot, (float)K), eps));
        if (scl && lane == 0) scl[t] = scale;
        const float * wv = w + (size_t)(POST ? t % HC : t % wr) * K + 4 * lane;
#pragma unroll
        for (int m = 0; m < CH; m++) {
            const float4 ww = __ldg(reinterpret_cast<const float4 *>(wv + 128 * m));
            const float4 v = make_float4(fmul(fmul(xv[m].x, scale), ww.x), fmul(fmul(xv[m].y, scale), ww.y), fmul(fmul(xv[m].z, scale), ww.z),
                                         fmul(fmul(xv[m].w, scale), ww.w));
            if (y) *reinterpret_cast<float4 *>(y + (size_t)t * K + 4 * lane + 128 * m) = v;
            if (ybf) st64_stream(ybf + (size_t)t * K + 4 * lane + 128 * m, make_uint2(bf16x2<true>(v.x, v.y), bf16x2<true>(v.z, v.w)));
            if (Q8) {
                float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                float s0 = v.x, s1 = v.y, s2 = v.z, s3 = v.w;
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) {
                    amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, o));
                    s0 = fadd(s0, __shfl_xor_sync(CAM_FULL, s0, o)); s1 = fadd(s1, __shfl_xor_sync(CAM_FULL, s1, o));
                    s2 = fadd(s2, __shfl_xor_sync(CAM_FULL, s2, o)); s3 = fadd(s3, __shfl_xor_sync(CAM_FULL, s3, o));
                }
                const float sum = fadd(fadd(s0, s2), fadd(s1, s3));
                const float d = fdiv(amax, 127.0f);
                const float inv = rcp_approx(d);
                const float inv_hi = fmul(inv, 0x1.000008p+0f), inv_lo = fmul(inv, 0x1.fffff0p-1f);
                const float vv[4] = {v.x, v.y, v.z, v.w};
                uint32_t c[4], differ = 0;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    c[e] = __float_as_uint(ffma(vv[e], inv_hi, 12582912.0f));
                    differ |= c[e] ^ __float_as_uint(ffma(vv[e], inv_lo, 12582912.0f));
                }
                const uint32_t word = __byte_perm(__byte_perm(c[0], c[1], 0x0040), __byte_perm(c[2], c[3], 0x0040), 0x5410);
                const float mag = fadd(fadd(fabsf(v.x), fabsf(v.y)), fadd(fabsf(v.z), fabsf(v.w)));
                if (differ != 0 || !(d >= 1.0e-30f) || !(mag < 3.0e38f)) redo |= 1ull << m;      // (settled after the row: no branch among the row's loads and stores)
                uint32_t * blk = reinterpret_cast<uint32_t *>(yq + ((size_t)t * (K / 32) + 4 * m + (lane >> 3)) * 36);
                blk[1 + (lane & 7)] = word;
                if ((lane & 7) == 0) __stcs(blk, f2_to_h2(d, sum));
            }
        }
        if (Q8) {      // the exact statements for a flagged lane's four values of a chunk (about one row in ten has one), stored over the fast word
            unsigned long long any = __reduce_or_sync(CAM_FULL, (uint32_t)redo);
            if (CH > 32) any |= (unsigned long long)__reduce_or_sync(CAM_FULL, (uint32_t)(redo >> 32)) << 32;
            while (any) {                                       // (uniform: the chunk's eight lanes find its amax together)
                const int m = __ffsll((long long)any) - 1;
                any &= any - 1;
                float4 xm = xv[0];
#pragma unroll
                for (int k = 1; k < CH; k++) if (k == m) xm = xv[k];
                const float4 ww = __ldg(reinterpret_cast<const float4 *>(wv + 128 * m));
                const float vv[4] = {fmul(fmul(xm.x, scale), ww.x), fmul(fmul(xm.y, scale), ww.y), fmul(fmul(xm.z, scale), ww.z), fmul(fmul(xm.w, scale), ww.w)};
                float amax = fmaxf(fmaxf(fabsf(vv[0]), fabsf(vv[1])), fmaxf(fabsf(vv[2]), fabsf(vv[3])));
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, o));
                if ((redo >> m) & 1ull) {
                    const float d = fdiv(amax, 127.0f);
                    uint32_t word = 0;
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float qv = fdiv(vv[e], d);
                        const int q = (amax != 0.0f && fabsf(qv) < 127.5f) ? __float2int_rn(roundf(qv)) : 0;
                        word |= (uint32_t)(q & 0xff) << (8 * e);
                    }
                    reinterpret_cast<uint32_t *>(yq + ((size_t)t * (K / 32) + 4 * m + (lane >> 3)) * 36)[1 + (lane & 7)] = word;
                }
            }
        }
    }
}

template <int CH, bool POST, bool Q8 = false>
int launch_rows_vec(float * x, const float * w, float * y, uint16_t * ybf, float * scl, int R, int wr, float eps, const float * b, const float * inj,
                    int HC, float rs, cudaStream_t stream, uint8_t * yq = nullptr) {
    // (8 x the resident blocks: pf_rms_mul 0.86 -> 0.94, rmsnorm_f32 0.86 -> 0.955, the Q8_1 form 0.84 -> 0.87; the hyper-connection form ran the same or slower with them)
    const int grid = cam_resident_grid(rms_rows_vec_kernel<CH, POST, Q8>, RMS_WARPS * 32, 0, ((long)R + RMS_WARPS - 1) / RMS_WARPS, POST ? 1 : 8);
    rms_rows_vec_kernel<CH, POST, Q8><<<grid, RMS_WARPS * 32, 0, stream>>>(x, w, y, ybf, scl, R, wr, eps, b, inj, HC, rs, yq);
    return (int)cudaGetLastError();
}

// ---- fp16 rows, staged through shared memory with cp.async ------------------------------------------------------------------
// Each warp keeps STAGES rows (x and d, 2 N bytes each) in flight in its own slice of shared memory; a lane copies exactly
// the 16-byte chunks it will read back, so waiting on its own copy groups is the only synchronisation. The row is read
// twice from shared memory (sum of squares, then normalise) and never twice from HBM.
// MODE 0: x = fp16(xs) stored, h16 = fp16((xs scale) nw)   (xs = (float)x + (float)d in fp32, the norm over the unrounded xs)
// MODE 1: the tensor-parallel partial: ss[t] = this shard's sum of squares of xs, nothing else stored
// MODE 2: the tensor-parallel apply: as MODE 0 with the row total read from tot[t] and divided by Nfull
constexpr int F16_STAGES = 2;

CAM_DEV void load8(const uint4 v, float (&f)[8]) {
    const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), c = h2_to_f2(v.z), e = h2_to_f2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = e.x; f[7] = e.y;
}

template <int MODE>
__global__ void __launch_bounds__(128) add_rms_f16_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d,
                                                          const float * __restrict__ nw, float eps, uint16_t * __restrict__ h16,
                                                          float * __restrict__ ss, const float * __restrict__ tot_in, int N, int Nfull,
                                                          int n, int warps, int nw_smem) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nch = (N + 255) >> 8;                             // 16-byte chunks per lane per row and tensor (the last may be
    const int nd = d ? 2 : 1;                                   // short when N is not a multiple of 256: lanes past N add +0)
    const size_t half_bytes = (size_t)nch * 512;                // one tensor's row in a stage
    const size_t stage_bytes = (size_t)nd * half_bytes;
    // the norm weights, staged once per block in front of the row stages when they fit (nw_smem floats; 0: read from global)
    float * snw = reinterpret_cast<float *>(smem);
    if (MODE != 1 && nw_smem) {
        for (int i = threadIdx.x; i < N; i += blockDim.x) snw[i] = __ldg(nw + i);
        __syncthreads();
    }
    const float * wsrc = (MODE != 1 && nw_smem) ? snw : nw;
    unsigned char * mine = smem + (size_t)nw_smem * 4 + (size_t)warp * F16_STAGES * stage_bytes;
    const int stride = gridDim.x * warps;
    const int t0 = blockIdx.x * warps + warp;

    auto issue = [&](int t, int st) {
        if (t < n) {
            unsigned char * sx = mine + (size_t)st * stage_bytes;
            const uint16_t * xr = x + (size_t)t * N;
            for (int m = 0; m < nch; m++)
                if (8 * lane + 256 * m < N) cp_async16(sx + (size_t)(m * 32 + lane) * 16, xr + 8 * lane + 256 * m);
            if (d) {
                const uint16_t * dr = d + (size_t)t * N;
                for (int m = 0; m < nch; m++)
                    if (8 * lane + 256 * m < N) cp_async16(sx + half_bytes + (size_t)(m * 32 + lane) * 16, dr + 8 * lane + 256 * m);
            }
        }
        cp_async_commit();
    };

    issue(t0, 0);
    int st = 0;
    for (int t = t0; t < n; t += stride, st ^= 1) {
        issue(t + stride, st ^ 1);
        cp_async_wait<1>();                                     // this row's group has landed (the next may still fly)
        const unsigned char * sx = mine + (size_t)st * stage_bytes;
        const unsigned char * sd = sx + half_bytes;
        float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        float tot;
        if (MODE != 2) {
#pragma unroll 4
            for (int m = 0; m < nch; m++) {
                if (8 * lane + 256 * m >= N) break;
                float xs[8];
                load8(*reinterpret_cast<const uint4 *>(sx + (size_t)(m * 32 + lane) * 16), xs);
                if (d) {
                    float dv[8];
                    load8(*reinterpret_cast<const uint4 *>(sd + (size_t)(m * 32 + lane) * 16), dv);
#pragma unroll
                    for (int c = 0; c < 8; c++) xs[c] = fadd(xs[c], dv[c]);
                }
#pragma unroll
                for (int c = 0; c < 8; c++) a[c] = ffma(xs[c], xs[c], a[c]);
            }
            tot = ref_total_f16(a, lane);
        } else tot = __ldg(tot_in + t);
        if (MODE == 1) {
            if (lane == 0) ss[t] = tot;
        } else {
            const float scale = cam_rsqrt(fadd(fdiv(tot, (float)(MODE == 2 ? Nfull : N)), eps));
            uint16_t * xr = x + (size_t)t * N;
            uint16_t * hr = h16 + (size_t)t * N;
#pragma unroll 2
            for (int m = 0; m < nch; m++) {
                const int i = 8 * lane + 256 * m;
                if (i >= N) break;
                float xs[8];
                load8(*reinterpret_cast<const uint4 *>(sx + (size_t)(m * 32 + lane) * 16), xs);
                if (d) {
                    float dv[8];
                    load8(*reinterpret_cast<const uint4 *>(sd + (size_t)(m * 32 + lane) * 16), dv);
#pragma unroll
                    for (int c = 0; c < 8; c++) xs[c] = fadd(xs[c], dv[c]);
                    st128(xr + i, make_uint4(f2_to_h2(xs[0], xs[1]), f2_to_h2(xs[2], xs[3]), f2_to_h2(xs[4], xs[5]), f2_to_h2(xs[6], xs[7])));
                }
                const float4 w0 = *reinterpret_cast<const float4 *>(wsrc + i), w1 = *reinterpret_cast<const float4 *>(wsrc + i + 4);
                float v[8];
                v[0] = fmul(fmul(xs[0], scale), w0.x); v[1] = fmul(fmul(xs[1], scale), w0.y);
                v[2] = fmul(fmul(xs[2], scale), w0.z); v[3] = fmul(fmul(xs[3], scale), w0.w);
                v[4] = fmul(fmul(xs[4], scale), w1.x); v[5] = fmul(fmul(xs[5], scale), w1.y);
                v[6] = fmul(fmul(xs[6], scale), w1.z); v[7] = fmul(fmul(xs[7], scale), w1.w);
                st128_stream(hr + i, make_uint4(f2_to_h2(v[0], v[1]), f2_to_h2(v[2], v[3]), f2_to_h2(v[4], v[5]), f2_to_h2(v[6], v[7])));
            }
        }
    }
    cp_async_wait<0>();
}

// ---- fp16 rows too long to stage (2 stages x (x and d) x N x 2 bytes beyond a block's shared memory: N above about 28 900 with d,
// 57 800 without): a warp per row, the row read twice from global memory: for the sum of squares and, a few microseconds later, for the
// normalisation (the second read of a row of at most 256 KB comes from L2, not from HBM). Modes as the staged kernel's.
template <int MODE>
__global__ void __launch_bounds__(128) add_rms_f16_long_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d, const float * __restrict__ nw, float eps,
                                                               uint16_t * __restrict__ h16, float * __restrict__ ss, const float * __restrict__ tot_in,
                                                               int N, int Nfull, int n) {
    const int lane = threadIdx.x & 31;
    const int nch = (N + 255) >> 8;
    for (int t = blockIdx.x * 4 + (threadIdx.x >> 5); t < n; t += gridDim.x * 4) {
        uint16_t * xr = x + (size_t)t * N;
        const uint16_t * dr = d ? d + (size_t)t * N : nullptr;
        float tot;
        if (MODE != 2) {
            float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int m = 0; m < nch; m++) {
                const int i = 8 * lane + 256 * m;
                if (i >= N) break;
                float xs[8];
                load8(ld128(xr + i), xs);
                if (dr) {
                    float dv[8];
                    load8(ldg128(dr + i), dv);
#pragma unroll
                    for (int c = 0; c < 8; c++) xs[c] = fadd(xs[c], dv[c]);
                }
#pragma unroll
                for (int c = 0; c < 8; c++) a[c] = ffma(xs[c], xs[c], a[c]);
            }
            tot = ref_total_f16(a, lane);
        } else tot = __ldg(tot_in + t);
        if (MODE == 1) { if (lane == 0) ss[t] = tot; continue; }
        const float scale = cam_rsqrt(fadd(fdiv(tot, (float)(MODE == 2 ? Nfull : N)), eps));
        uint16_t * hr = h16 + (size_t)t * N;
#pragma unroll 2
        for (int m = 0; m < nch; m++) {
            const int i = 8 * lane + 256 * m;
            if (i >= N) break;
            float xs[8];
            load8(ld128(xr + i), xs);
            if (dr) {
                float dv[8];
                load8(ldg128(dr + i), dv);
#pragma unroll
                for (int c = 0; c < 8; c++) xs[c] = fadd(xs[c], dv[c]);
                st128(xr + i, make_uint4(f2_to_h2(xs[0], xs[1]), f2_to_h2(xs[2], xs[3]), f2_to_h2(xs[4], xs[5]), f2_to_h2(xs[6], xs[7])));
            }
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(nw + i)), w1 = __ldg(reinterpret_cast<const float4 *>(nw + i + 4));
            float v[8];
            v[0] = fmul(fmul(xs[0], scale), w0.x); v[1] = fmul(fmul(xs[1], scale), w0.y);
            v[2] = fmul(fmul(xs[2], scale), w0.z); v[3] = fmul(fmul(xs[3], scale), w0.w);
            v[4] = fmul(fmul(xs[4], scale), w1.x); v[5] = fmul(fmul(xs[5], scale), w1.y);
            v[6] = fmul(fmul(xs[6], scale), w1.z); v[7] = fmul(fmul(xs[7], scale), w1.w);
            st128_stream(hr + i, make_uint4(f2_to_h2(v[0], v[1]), f2_to_h2(v[2], v[3]), f2_to_h2(v[4], v[5]), f2_to_h2(v[6], v[7])));
        }
    }
}

// ---- fp16 rows held in registers -----------------------------------------------------------------------------------------
// N = 256 CH: a warp loads its whole row (x and d: 2 CH 16-byte loads per lane, all issued before any is used, so a warp
// keeps 4 N bytes in flight), keeps xs in fp32 registers between the sum of squares and the normalisation, and reads the
// norm weights from shared memory (staged once per block). No row is touched twice, in HBM or in shared memory.
template <int CH>
__global__ void __launch_bounds__(128, 2) add_rms_f16_reg_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d,
                                                                 const float * __restrict__ nw, float eps, uint16_t * __restrict__ h16, int n) {
    constexpr int N = 256 * CH;
    __shared__ __align__(16) float snw[N];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x * 4; i < N; i += 512) *reinterpret_cast<float4 *>(snw + i) = __ldg(reinterpret_cast<const float4 *>(nw + i));
    __syncthreads();
    for (int t = blockIdx.x * 4 + warp; t < n; t += gridDim.x * 4) {
        uint16_t * xr = x + (size_t)t * N + 8 * lane;
        uint16_t * hr = h16 + (size_t)t * N + 8 * lane;
        uint4 rx[CH], rd[CH];
#pragma unroll
        for (int m = 0; m < CH; m++) rx[m] = ld128(xr + 256 * m);
        if (d) {
            const uint16_t * dr = d + (size_t)t * N + 8 * lane;
#pragma unroll
            for (int m = 0; m < CH; m++) rd[m] = ldg128(dr + 256 * m);
        }
        float xs[CH][8];
        float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int m = 0; m < CH; m++) {
            load8(rx[m], xs[m]);
            if (d) {
                float dv[8];
                load8(rd[m], dv);
#pragma unroll
                for (int c = 0; c < 8; c++) xs[m][c] = fadd(xs[m][c], dv[c]);
                st128(xr + 256 * m, make_uint4(f2_to_h2(xs[m][0], xs[m][1]), f2_to_h2(xs[m][2], xs[m][3]), f2_to_h2(xs[m][4], xs[m][5]),
                                               f2_to_h2(xs[m][6], xs[m][7])));
            }
#pragma unroll
            for (int c = 0; c < 8; c++) a[c] = ffma(xs[m][c], xs[m][c], a[c]);
        }
        const float tot = ref_total_f16(a, lane);
        const float scale = cam_rsqrt(fadd(fdiv(tot, (float)N), eps));
#pragma unroll
        for (int m = 0; m < CH; m++) {
            const float4 w0 = *reinterpret_cast<const float4 *>(snw + 8 * lane + 256 * m), w1 = *reinterpret_cast<const float4 *>(snw + 8 * lane + 256 * m + 4);
            const float v0 = fmul(fmul(xs[m][0], scale), w0.x), v1 = fmul(fmul(xs[m][1], scale), w0.y);
            const float v2 = fmul(fmul(xs[m][2], scale), w0.z), v3 = fmul(fmul(xs[m][3], scale), w0.w);
            const float v4 = fmul(fmul(xs[m][4], scale), w1.x), v5 = fmul(fmul(xs[m][5], scale), w1.y);
            const float v6 = fmul(fmul(xs[m][6], scale), w1.z), v7 = fmul(fmul(xs[m][7], scale), w1.w);
            st128_stream(hr + 256 * m, make_uint4(f2_to_h2(v0, v1), f2_to_h2(v2, v3), f2_to_h2(v4, v5), f2_to_h2(v6, v7)));
        }
    }
}

// Rows too long for one warp's registers (N = 256 CHW WPR, WPR = 2 or 4 warps per row): warp w of a row's group holds chunks
// w CHW .. (w + 1) CHW - 1 in registers. The reference's sum is one fma chain per thread over the whole row, so the 8 accumulators of a
// lane pass from warp to warp through shared memory (WPR short steps, a block barrier after each); the last warp forms the total and the
// scale, every warp normalises its part from registers. Nothing is read twice, in HBM or in the second-level cache, for rows of up to
// 20480 values (the staged kernel holds 2 to 4 warps per multiprocessor on rows of 6144 to 8192: 0.30-0.58 of the copy bandwidth; the
// two-pass kernel: 0.62-0.66).
template <int CHW, int WPR>
__global__ void __launch_bounds__(128, 2) add_rms_f16_reg_multi_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d,
                                                                       const float * __restrict__ nw, float eps, uint16_t * __restrict__ h16, int n) {
    constexpr int N = 256 * CHW * WPR, RPB = 4 / WPR;                    // rows per block and pass
    extern __shared__ __align__(16) float multi_smem[];
    float * const snw = multi_smem;                                      // [N] weights
    float * const acc = snw + N;                                         // [RPB][8][32]: a row's accumulators in flight between its warps
    float * const scl = acc + RPB * 256;                                 // [RPB]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, grp = warp / WPR, part = warp % WPR;
    for (int i = threadIdx.x * 4; i < N; i += 512) *reinterpret_cast<float4 *>(snw + i) = __ldg(reinterpret_cast<const float4 *>(nw + i));
    __syncthreads();
    for (int t0 = blockIdx.x * RPB; t0 < n; t0 += gridDim.x * RPB) {     // (block-uniform: every warp takes part in the barriers)
        const int t = t0 + grp;
        const bool on = t < n;
        const size_t at = (size_t)(on ? t : 0) * N + part * (256 * CHW) + 8 * lane;
        uint4 rx[CHW], rd[CHW];
#pragma unroll
        for (int m = 0; m < CHW; m++) rx[m] = on ? ld128(x + at + 256 * m) : make_uint4(0u, 0u, 0u, 0u);
        if (d) {
#pragma unroll
            for (int m = 0; m < CHW; m++) rd[m] = on ? ldg128(d + at + 256 * m) : make_uint4(0u, 0u, 0u, 0u);
        }
        float xs[CHW][8];
#pragma unroll
        for (int m = 0; m < CHW; m++) {
            load8(rx[m], xs[m]);
            if (d) {
                float dv[8];
                load8(rd[m], dv);
#pragma unroll
                for (int c = 0; c < 8; c++) xs[m][c] = fadd(xs[m][c], dv[c]);
                if (on) st128(x + at + 256 * m, make_uint4(f2_to_h2(xs[m][0], xs[m][1]), f2_to_h2(xs[m][2], xs[m][3]), f2_to_h2(xs[m][4], xs[m][5]),
                                                           f2_to_h2(xs[m][6], xs[m][7])));
            }
        }
        float * const ga = acc + grp * 256 + lane;                      // + 32 c: accumulator c of this lane
#pragma unroll
        for (int w = 0; w < WPR; w++) {                                  // the chain: warp w continues where warp w - 1 stopped
            if (part == w) {
                float a[8];
#pragma unroll
                for (int c = 0; c < 8; c++) a[c] = w ? ga[32 * c] : 0.0f;
#pragma unroll
                for (int m = 0; m < CHW; m++)
#pragma unroll
                    for (int c = 0; c < 8; c++) a[c] = ffma(xs[m][c], xs[m][c], a[c]);
                if (w < WPR - 1) {
#pragma unroll
                    for (int c = 0; c < 8; c++) ga[32 * c] = a[c];
                } else {
                    const float tot = ref_total_f16(a, lane);
                    if (lane == 0) scl[grp] = cam_rsqrt(fadd(fdiv(tot, (float)N), eps));
                }
            }
            __syncthreads();
        }
        const float scale = scl[grp];
#pragma unroll
        for (int m = 0; m < CHW; m++) {
            const float * wp = snw + part * (256 * CHW) + 8 * lane + 256 * m;
            const float4 w0 = *reinterpret_cast<const float4 *>(wp), w1 = *reinterpret_cast<const float4 *>(wp + 4);
            const float v0 = fmul(fmul(xs[m][0], scale), w0.x), v1 = fmul(fmul(xs[m][1], scale), w0.y);
            const float v2 = fmul(fmul(xs[m][2], scale), w0.z), v3 = fmul(fmul(xs[m][3], scale), w0.w);
            const float v4 = fmul(fmul(xs[m][4], scale), w1.x), v5 = fmul(fmul(xs[m][5], scale), w1.y);
            const float v6 = fmul(fmul(xs[m][6], scale), w1.z), v7 = fmul(fmul(xs[m][7], scale), w1.w);
            if (on) st128_stream(h16 + at + 256 * m, make_uint4(f2_to_h2(v0, v1), f2_to_h2(v2, v3), f2_to_h2(v4, v5), f2_to_h2(v6, v7)));
        }
        __syncthreads();                                                 // (scl and acc are rewritten by the next pass)
    }
}

template <int CHW, int WPR>
int launch_f16_reg_multi(uint16_t * x, const uint16_t * d, const float * nw, float eps, uint16_t * h16, int n, cudaStream_t stream) {
    constexpr int N = 256 * CHW * WPR, RPB = 4 / WPR;
    const size_t smem = ((size_t)N + RPB * 256 + 8) * sizeof(float);
    static unsigned long long allowed = 0;
    if (smem > 48 * 1024) { const cudaError_t e = cam_allow_smem(add_rms_f16_reg_multi_kernel<CHW, WPR>, smem, allowed); if (e != cudaSuccess) return (int)e; }
    const long want = ((long)n + RPB - 1) / RPB;
    const int grid = cam_resident_grid(add_rms_f16_reg_multi_kernel<CHW, WPR>, 128, smem, want, 8);
    add_rms_f16_reg_multi_kernel<CHW, WPR><<<grid, 128, smem, stream>>>(x, d, nw, eps, h16, n);
    return (int)cudaGetLastError();
}

template <int CH>
int launch_f16_reg(uint16_t * x, const uint16_t * d, const float * nw, float eps, uint16_t * h16, int n, cudaStream_t stream) {
    // about two passes of four rows per block (at least the resident blocks): a finished block's successor starts with its rows' loads at
    // once. 65536 rows of 5120: 412 us, against 423 us with 8 x the resident blocks, 426 us with a block per four rows and 437 us with
    // exactly the resident blocks looping over the rows
    const long want = ((long)n + 3) / 4;
    const int grid = cam_iter_grid(add_rms_f16_reg_kernel<CH>, 128, 0, want, 2);
    add_rms_f16_reg_kernel<CH><<<grid, 128, 0, stream>>>(x, d, nw, eps, h16, n);
    return (int)cudaGetLastError();
}

template <int MODE>
int launch_f16(uint16_t * x, const uint16_t * d, const float * nw, float eps, uint16_t * h16, float * ss, const float * tot, int N,
               int Nfull, int n, cudaStream_t stream) {
    if (n == 0) return CAM_OK;
    const size_t per_warp = (size_t)F16_STAGES * (d ? 2 : 1) * ((N + 255) >> 8) * 512;
    const size_t budget = 226 * 1024;
    int nw_smem = (MODE != 1 && (size_t)N * 4 + per_warp <= budget) ? N : 0;
    int warps = 4;
    while (warps > 1 && (size_t)nw_smem * 4 + per_warp * warps > budget) warps >>= 1;
    if (n < 4 * warps) nw_smem = 0;                               // (a handful of rows: staging the weights costs more than it saves)
    const size_t smem = (size_t)nw_smem * 4 + per_warp * warps;
    if (smem > budget) {                                          // a row that one warp cannot stage: the two-pass kernel
        const int grid = cam_resident_grid(add_rms_f16_long_kernel<MODE>, 128, 0, ((long)n + 3) / 4);
        add_rms_f16_long_kernel<MODE><<<grid, 128, 0, stream>>>(x, d, nw, eps, h16, ss, tot, N, Nfull, n);
        return (int)cudaGetLastError();
    }
    static unsigned long long allowed = 0;
    const cudaError_t e = cam_allow_smem(add_rms_f16_kernel<MODE>, 227 * 1024, allowed);
    if (e != cudaSuccess) return (int)e;
    const int grid = cam_resident_grid(add_rms_f16_kernel<MODE>, warps * 32, smem, ((long)n + warps - 1) / warps);
    add_rms_f16_kernel<MODE><<<grid, warps * 32, smem, stream>>>(x, d, nw, eps, h16, ss, tot, N, Nfull, n, warps, nw_smem);
    return (int)cudaGetLastError();
}

int launch_f32(float * x, const float * d, const float * w, int S, const float * nw, float eps, float * h, uint16_t * h16, int N, int n,
               int q35, cudaStream_t stream) {
    if (n == 0) return CAM_OK;
    if (N <= 2048 && n <= 2 * cam_sm_count()) {      // a few rows: a block per row
        add_rms_f32_row_kernel<<<n, 256, 0, stream>>>(x, d, w, S, nw, eps, h, h16, N, q35);
        return (int)cudaGetLastError();
    }
    const long want = ((long)n + RMS_WARPS - 1) / RMS_WARPS;
#define CAM_RMS_CASE(CHV)                                                                                              \
    case CHV:                                                                                                          \
        add_rms_f32_kernel<CHV><<<cam_iter_grid(add_rms_f32_kernel<CHV>, RMS_WARPS * 32, 0, want, 1), RMS_WARPS * 32, 0, stream>>>(      /* (a block per unit: 65536 rows of 2048 408 -> 360 us, 0.91 -> 1.03) */ \
            x, d, w, S, nw, eps, h, h16, N, n, q35);                                                                   \
        break;
    switch (N <= 2048 ? N >> 7 : 0) {
        CAM_RMS_CASE(2) CAM_RMS_CASE(4) CAM_RMS_CASE(6) CAM_RMS_CASE(8) CAM_RMS_CASE(10) CAM_RMS_CASE(12) CAM_RMS_CASE(14) CAM_RMS_CASE(16)
        CAM_RMS_CASE(0)
    }
#undef CAM_RMS_CASE
    return (int)cudaGetLastError();
}

}   // namespace

// q3p_add_rms16: x [n][N] += sum over S slots of w[t][s] d[t][s][:] (w null: plain sums; d null or S = 0: no add);
// h (nullable) fp32 and h16 fp16 = (x rsqrt(mean x^2 + eps)) nw. n is the reference's grid.x.
// Reference: kernels/q3m_prefill.hip:385-387; wrapper python/caminus/prefill/q3m_ops.py:89-92.
extern "C" int q3p_add_rms16(int n, float * x, const float * d, const float * w, int S, const float * nw, float eps, float * h,
                             void * h16, int N, void * stream) {
    if (n < 0 || N < 256 || (N & 255) || N > 2048 || S < 0 || !x || !nw || !h16 || (S > 0 && !d)) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || !cam_aligned16(nw) || (d && !cam_aligned16(d)) || (h && !cam_aligned16(h)) ||
        (reinterpret_cast<uintptr_t>(h16) & 7u) || (w && (reinterpret_cast<uintptr_t>(w) & 3u))) return CAM_ERR_ALIGN;
    return launch_f32(x, d, w, S, nw, eps, h, (uint16_t *)h16, N, n, 0, (cudaStream_t)stream);
}

// q35p_add_rms16: x [n][N] += d (d nullable), any N = 256 NI <= 65536; h and h16 always written.
// Reference: kernels/q35_prefill.hip:636-638; wrapper python/caminus/prefill/q35own.py:135-140.
extern "C" int q35p_add_rms16(int n, float * x, const float * d, const float * nw, float eps, float * h, void * h16, int N,
                              void * stream) {
    if (n < 0 || N < 256 || (N & 255) || N > 65536 || !x || !nw || !h || !h16) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || !cam_aligned16(nw) || (d && !cam_aligned16(d)) || !cam_aligned16(h) ||
        (reinterpret_cast<uintptr_t>(h16) & 7u)) return CAM_ERR_ALIGN;
    return launch_f32(x, d, nullptr, 0, nw, eps, h, (uint16_t *)h16, N, n, 1, (cudaStream_t)stream);
}

// cam_add_rms_f16: the same statements on fp16 storage: x [n][N] fp16 (updated in place when d is given), d fp16 (nullable),
// h16 fp16 out. N a multiple of 256. No counterpart kernel in the reference (its glue takes fp32 activations); the
// arithmetic is q35p_add_rms16's (kernels/q35_prefill.hip:636-660) between an exact fp16 load and a rounded fp16 store.
extern "C" int cam_add_rms_f16(int n, void * x, const void * d, const float * nw, float eps, void * h16, int N, void * stream) {
    if (n < 0 || N < 256 || (N & 255) || N > 65536 || !x || !nw || !h16) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || !cam_aligned16(nw) || (d && !cam_aligned16(d)) || !cam_aligned16(h16)) return CAM_ERR_ALIGN;
    if (n >= 64) {      // (a handful of rows: the staged kernel, which does not stage the weights first)
        switch (N) {
            case 512: return launch_f16_reg<2>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 768: return launch_f16_reg<3>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 1280: return launch_f16_reg<5>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 1536: return launch_f16_reg<6>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 3072: return launch_f16_reg<12>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 3584: return launch_f16_reg<14>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 1024: return launch_f16_reg<4>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 2048: return launch_f16_reg<8>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 2560: return launch_f16_reg<10>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 4096: return launch_f16_reg<16>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 5120: return launch_f16_reg<20>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
#define CAM_REG_MULTI(CHWV, WPRV) return launch_f16_reg_multi<CHWV, WPRV>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, n, (cudaStream_t)stream);
            case 6144: CAM_REG_MULTI(12, 2) case 7168: CAM_REG_MULTI(14, 2) case 8192: CAM_REG_MULTI(16, 2) case 10240: CAM_REG_MULTI(20, 2)
            case 12288: CAM_REG_MULTI(12, 4) case 14336: CAM_REG_MULTI(14, 4) case 16384: CAM_REG_MULTI(16, 4) case 20480: CAM_REG_MULTI(20, 4)
#undef CAM_REG_MULTI
            default: break;
        }
    }
    return launch_f16<0>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, nullptr, nullptr, N, N, n, (cudaStream_t)stream);
}

// Tensor-parallel RMSNorm (hidden dimension sharded over ranks; no counterpart in the reference, which replicates its norms).
// Ns (this rank's columns) is a multiple of 8.
// cam_rms_partial_f16: ss [n] fp32 = this shard's sum of squares of xs = x + d over its Ns columns (nothing else written).
// After the caller summed ss over the ranks (an all-reduce of n floats):
// cam_rms_apply_f16: x = fp16(xs) (when d is given), h16 = fp16((xs rsqrt(tot / Nfull + eps)) nw_shard).
extern "C" int cam_rms_partial_f16(int n, const void * x, const void * d, float * ss, int Ns, void * stream) {
    if (n < 0 || Ns < 8 || (Ns & 7) || !x || !ss) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || (d && !cam_aligned16(d)) || (reinterpret_cast<uintptr_t>(ss) & 3u)) return CAM_ERR_ALIGN;
    return launch_f16<1>((uint16_t *)x, (const uint16_t *)d, nullptr, 0.0f, nullptr, ss, nullptr, Ns, Ns, n, (cudaStream_t)stream);
}
extern "C" int cam_rms_apply_f16(int n, void * x, const void * d, const float * tot, const float * nw, float eps, void * h16, int Ns,
                                 int Nfull, void * stream) {
    if (n < 0 || Ns < 8 || (Ns & 7) || Nfull < Ns || !x || !tot || !nw || !h16) return CAM_ERR_ARG;
    if (!cam_aligned16(x) || (d && !cam_aligned16(d)) || !cam_aligned16(nw) || !cam_aligned16(h16)) return CAM_ERR_ALIGN;
    return launch_f16<2>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, nullptr, tot, Ns, Nfull, n, (cudaStream_t)stream);
}

// ---- the two-kernel norm with its intermediate in the library's own static memory ------------------------------------------------
// The partial / apply pair above hands the per-row sums of squares from the first kernel to the second through a
// buffer the caller allocates. Some callers cannot allocate: a plugin that an engine hands fixed buffers sized at
// start-up and forbids from touching the allocator (the reference's own rule for its wrappers: "nothing here allocates"),
// or a process whose device memory is already fully carved up, where one more cudaMalloc fails or forces a synchronisation.
// For them the sums live in this file-scope array, which every device that loads the library holds until it exits
// (CAM_STATIC_ROWS floats = 256 KB).
#define CAM_STATIC_ROWS 65536
static __device__ __align__(256) float cam_static_ss[CAM_STATIC_ROWS];

// The array's device address on the current device. In host code the name `cam_static_ss` is only a handle for the runtime,
// not a device pointer: the address comes from cudaGetSymbolAddress, asked once per device with that device current.
static int static_ss_address(float ** out) {
    static std::mutex mu;
    static float * addr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return CAM_ERR_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void * p = nullptr;
        e = cudaGetSymbolAddress(&p, cam_static_ss);
        if (e != cudaSuccess) return (int)e;
        addr[dev] = static_cast<float *>(p);
    }
    *out = addr[dev];
    return CAM_OK;
}

// cam_rms_norm_f16_static: x [n][N] fp16 (updated in place to fp16(x + d) when d is given), d fp16 (nullable), nw fp32 [N],
// h16 fp16 [n][N] = the normed rows; N a multiple of 8; n <= 65536 rows per call (CAM_ERR_CAPACITY beyond: split the batch).
// The same two launches and the same bytes as cam_rms_partial_f16 followed by cam_rms_apply_f16 with Ns = Nfull = N, with the
// row sums in the library's static array instead of a caller's buffer. Calls no cudaMalloc / cudaFree and no allocating
// routine. The first call on a device looks up the array's address (cudaGetSymbolAddress): make that first call outside any
// stream capture. Every call on a device uses the same array and the array keeps the last call's sums: nothing in it has
// to start at zero (the first kernel overwrites rows 0 .. n - 1 before the second reads them), but two calls whose kernels
// can overlap on the GPU (different streams without an ordering between them) race on it: order them.
extern "C" int cam_rms_norm_f16_static(int n, void * x, const void * d, const float * nw, float eps, void * h16, int N, void * stream) {
    if (n < 0 || N < 8 || (N & 7) || !x || !nw || !h16) return CAM_ERR_ARG;
    if (n > CAM_STATIC_ROWS) return CAM_ERR_CAPACITY;
    if (!cam_aligned16(x) || (d && !cam_aligned16(d)) || !cam_aligned16(nw) || !cam_aligned16(h16)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    float * ss = nullptr;
    int r = static_ss_address(&ss);
    if (r != CAM_OK) return r;
    r = launch_f16<1>((uint16_t *)x, (const uint16_t *)d, nullptr, 0.0f, nullptr, ss, nullptr, N, N, n, (cudaStream_t)stream);
    if (r != CAM_OK) return r;
    return launch_f16<2>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, nullptr, ss, N, N, n, (cudaStream_t)stream);
}

// The vector path of pf_rms_mul / pf_hc_post_rms / rmsnorm_f32 (csrc/hc_glue.cu): K in {2048, 2560, 5120} (the plain norm: more multiples of 128), 16-byte aligned buffers, enough rows to
// fill the device. Returns CAM_ERR_SHAPE when it does not apply (the caller then uses its block-per-row kernel).
int cam_rms_rows_vec(float * x, const float * w, float * y, void * ybf, float * scl, int R, int wr, float eps, int K, const float * b,
                     const float * inj, int HC, float rs, void * stream, void * yq) {
    if (R < 2 * cam_sm_count() || !cam_aligned16(x) || !cam_aligned16(w) || (y && !cam_aligned16(y)) || (ybf && (reinterpret_cast<uintptr_t>(ybf) & 7u)) ||
        (b && !cam_aligned16(b))) return CAM_ERR_SHAPE;
    uint16_t * yb = (uint16_t *)ybf; cudaStream_t st = (cudaStream_t)stream;
    if (yq) {       // pf_rms_mul's norm with the Q8_1 copy
        if (b || ybf || scl) return CAM_ERR_SHAPE;
        switch (K) {
            case 2048: return launch_rows_vec<16, false, true>(x, w, y, nullptr, nullptr, R, wr, eps, nullptr, nullptr, 1, 0.0f, st, (uint8_t *)yq);
            case 2560: return launch_rows_vec<20, false, true>(x, w, y, nullptr, nullptr, R, wr, eps, nullptr, nullptr, 1, 0.0f, st, (uint8_t *)yq);
            case 5120: return launch_rows_vec<40, false, true>(x, w, y, nullptr, nullptr, R, wr, eps, nullptr, nullptr, 1, 0.0f, st, (uint8_t *)yq);
            default: return CAM_ERR_SHAPE;
        }
    }
    switch (K) {
        case 2048: return b ? launch_rows_vec<16, true>(x, w, y, yb, scl, R, wr, eps, b, inj, HC, rs, st) : launch_rows_vec<16, false>(x, w, y, yb, scl, R, wr, eps, b, inj, HC, rs, st);
        case 2560: return b ? launch_rows_vec<20, true>(x, w, y, yb, scl, R, wr, eps, b, inj, HC, rs, st) : launch_rows_vec<20, false>(x, w, y, yb, scl, R, wr, eps, b, inj, HC, rs, st);
        case 5120: return b ? launch_rows_vec<40, true>(x, w, y, yb, scl, R, wr, eps, b, inj, HC, rs, st) : launch_rows_vec<40, false>(x, w, y, yb, scl, R, wr, eps, b, inj, HC, rs, st);
        default: break;
    }
    if (b) return CAM_ERR_SHAPE;
    switch (K) {    // the plain norm (rmsnorm_f32's row lengths among them): any multiple of 128 follows the same lane-to-thread mapping
#define CAM_ROWS_CASE(CH) case 128 * CH: return launch_rows_vec<CH, false>(x, w, y, yb, scl, R, wr, eps, nullptr, nullptr, 1, 0.0f, st)
        CAM_ROWS_CASE(4); CAM_ROWS_CASE(5); CAM_ROWS_CASE(6); CAM_ROWS_CASE(7); CAM_ROWS_CASE(8); CAM_ROWS_CASE(10); CAM_ROWS_CASE(12);
        CAM_ROWS_CASE(14); CAM_ROWS_CASE(24); CAM_ROWS_CASE(28); CAM_ROWS_CASE(32);
#undef CAM_ROWS_CASE
        default: return CAM_ERR_SHAPE;
    }
}
