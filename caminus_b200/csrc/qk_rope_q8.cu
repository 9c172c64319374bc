// The Q8_0 KV cache form of the q/k RMSNorm + NeoX RoPE kernel (the reference's q3p_qk_rope_q8, kernels/q3m_prefill.hip:526-535,
// 541-546, 572-583; Q8_0 block encode kernels/own_kv_codec.h:31-75; 128-point Hadamard transform kernels/own_kv_rot128.h:21-33;
// CPU reference python/caminus/ref_kv.py).
//
// Same norm and rotation statements as csrc/qk_rope.cu. Then every head's result is rounded to fp16 and back (the value the F16
// cache would hold) and transformed by the orthonormal Walsh-Hadamard matrix (butterflies h = 1, 2, .. 64 in that order, then
// times fp32(1 / sqrt(128))). q heads store fp16 of the transform into q16. kv heads store the transformed K as four Q8_0 blocks
// (fp16 d = amax / 127, q = roundf(x * (1 / d))) and the fp16-rounded V, untransformed, as four more, into the cache row
// pos: [K blocks of all heads | V blocks of all heads], 34 bytes per block. A block with a non-finite value or a scale outside
// fp32 / fp16 range is refused: its bytes are left alone and 2 is ORed into *err.
//
// Mapping: a block per token, a half-warp per head; lane l holds dims 4l .. 4l + 3 and 64 + 4l .. 64 + 4l + 3, so butterflies 1, 2
// and 64 are inside the lane and 4, 8, 16, 32 are lane exchanges; a Q8_0 block of 32 dims is 8 lanes' low or high values.
#include "cam_common.cuh"

namespace {

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
    const float inv = d != 0.0f ? fdiv(1.0f, d) : 0.0f;
    const __half stored = __float2half_rn(d);
    const bool refuse = !finite_f(amax) || (amax != 0.0f && (d == 0.0f || !finite_f(d) || !finite_f(inv) || !finite_f(__half2float(stored))));
    if (!store) return;
    if (refuse) { if (l8 == 0) atomicOr(err, 2); return; }
    int q[4];
#pragma unroll
    for (int c = 0; c < 4; c++) q[c] = __float2int_rn(roundf(fmul(v[c], inv))) & 0xff;
    uint16_t * o = reinterpret_cast<uint16_t *>(blk + 2 + 4 * l8);              // (34-byte blocks: 2-byte alignment)
    o[0] = (uint16_t)(q[0] | (q[1] << 8)); o[1] = (uint16_t)(q[2] | (q[3] << 8));
    if (l8 == 0) *reinterpret_cast<uint16_t *>(blk) = __half_as_ushort(stored);
}

// x[0..3] = dims 4l .. 4l + 3, x[4..7] = dims 64 + 4l ..: the orthonormal Walsh-Hadamard transform of the half-warp's 128 values
CAM_DEV void hadamard128(float (&x)[8], int l16) {
#pragma unroll
    for (int b = 0; b < 8; b += 4) {                 // h = 1, then h = 2, inside each group of four
        float a0 = fadd(x[b], x[b + 1]), a1 = fsub(x[b], x[b + 1]), a2 = fadd(x[b + 2], x[b + 3]), a3 = fsub(x[b + 2], x[b + 3]);
        x[b] = fadd(a0, a2); x[b + 2] = fsub(a0, a2); x[b + 1] = fadd(a1, a3); x[b + 3] = fsub(a1, a3);
    }
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) {               // h = 4, 8, 16, 32: lanes l ^ 1, 2, 4, 8
        const bool hi = (l16 & m) != 0;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const float p = __shfl_xor_sync(CAM_FULL, x[c], m);
            x[c] = hi ? fsub(p, x[c]) : fadd(x[c], p);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; c++) {                    // h = 64, then the scale
        const float a = x[c], b = x[4 + c];
        x[c] = fmul(fadd(a, b), 0x1.6a09e6p-4f); x[4 + c] = fmul(fsub(a, b), 0x1.6a09e6p-4f);
    }
}

__global__ void __launch_bounds__(256) qk_rope_q8_kernel(const float * __restrict__ qkv, int ldq, int nh, int nkv, const float * __restrict__ par,
                                                         int pos0, uint16_t * __restrict__ q16, uint8_t * __restrict__ cache, int * err, int n, int yarn) {
    __shared__ __align__(16) float wq[128], wk[128], freq[64], rc[64], rs[64];
    const int tid = threadIdx.x, lane = tid & 31, l16 = lane & 15, hwarp = tid >> 4;       // 16 half-warps
    const int H = nh + nkv;
    const size_t M = (size_t)nkv * 128, rowb = 2 * (M / 32) * 34;
    const float eps = __ldg(par + 257), mscale = yarn ? __ldg(par + 322) : 1.0f;
    if (tid < 128) { wq[tid] = __ldg(par + tid); wk[tid] = __ldg(par + 128 + tid); }
    if (tid < 64) freq[tid] = yarn ? __ldg(par + 258 + tid) : cam_powi(__ldg(par + 256), tid);
    for (int t = blockIdx.x; t < n; t += gridDim.x) {
        const int pos = pos0 + t;
        __syncthreads();                              // (the previous token's readers are done with rc / rs; the first pass: wq, wk, freq are written)
        if (tid < 64) {
            float sn, cs;
            cam_sincos(fmul((float)pos, freq[tid]), sn, cs);
            rc[tid] = yarn ? fmul(cs, mscale) : cs; rs[tid] = yarn ? fmul(sn, mscale) : sn;
        }
        __syncthreads();
        const float * row = qkv + (size_t)t * ldq;
        uint8_t * cw = cache + (size_t)pos * rowb;
        const float4 c4 = *reinterpret_cast<const float4 *>(rc + 4 * l16), s4 = *reinterpret_cast<const float4 *>(rs + 4 * l16);
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
        for (int h0 = 0; h0 < H; h0 += 16) {          // 16 heads per round; both half-warps of a warp run every shuffle
            const int hy = h0 + hwarp;
            const bool on = hy < H, isq = hy < nh;
            const int g = hy - nh;
            float x[8];
            if (on) {
                const float * hp = row + (size_t)hy * 128 + 4 * l16;               // q heads, then k heads
                const float4 lo = __ldg(reinterpret_cast<const float4 *>(hp)), hi = __ldg(reinterpret_cast<const float4 *>(hp + 64));
                x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) x[c] = 0.0f;
            }
            float sl = 0.0f, sh = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) { sl = ffma(x[c], x[c], sl); sh = ffma(x[4 + c], x[4 + c], sh); }
            float ss = fadd(sl, sh);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss = fadd(ss, __shfl_xor_sync(CAM_FULL, ss, o));
            const float scale = cam_rsqrt(fadd(fmul(ss, 0.0078125f), eps));
            const float * wn = (isq ? wq : wk) + 4 * l16;
            const float4 wlo = *reinterpret_cast<const float4 *>(wn), whi = *reinterpret_cast<const float4 *>(wn + 64);
            const float wl[4] = {wlo.x, wlo.y, wlo.z, wlo.w}, wh[4] = {whi.x, whi.y, whi.z, whi.w};
            float y[8];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float x0 = fmul(fmul(scale, x[c]), wl[c]), x1 = fmul(fmul(scale, x[4 + c]), wh[c]);
                y[c] = f16r(ffma(x0, cc[c], -fmul(x1, sn[c])));
                y[4 + c] = f16r(ffma(x1, cc[c], fmul(x0, sn[c])));
            }
            hadamard128(y, l16);
            float v[8];
            if (on && !isq) {
                const float * vp = row + (size_t)nh * 128 + M + (size_t)g * 128 + 4 * l16;
                const float4 lo = __ldg(reinterpret_cast<const float4 *>(vp)), hi = __ldg(reinterpret_cast<const float4 *>(vp + 64));
                v[0] = f16r(lo.x); v[1] = f16r(lo.y); v[2] = f16r(lo.z); v[3] = f16r(lo.w);
                v[4] = f16r(hi.x); v[5] = f16r(hi.y); v[6] = f16r(hi.z); v[7] = f16r(hi.w);
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) v[c] = 0.0f;
            }
            if (on && isq) {
                uint16_t * o = q16 + ((size_t)t * nh + hy) * 128 + 4 * l16;
                st64(o, make_uint2(f2_to_h2(y[0], y[1]), f2_to_h2(y[2], y[3])));
                st64(o + 64, make_uint2(f2_to_h2(y[4], y[5]), f2_to_h2(y[6], y[7])));
            }
            // the kv heads' eight blocks: every lane runs the group reductions, only a kv head's lanes store
            const bool kv = on && !isq;
            if (__any_sync(CAM_FULL, kv)) {
                const int w = l16 >> 3, l8 = l16 & 7;
                const float klo[4] = {y[0], y[1], y[2], y[3]}, khi[4] = {y[4], y[5], y[6], y[7]};
                const float vlo[4] = {v[0], v[1], v[2], v[3]}, vhi[4] = {v[4], v[5], v[6], v[7]};
                uint8_t * kb = cw + (size_t)(kv ? g : 0) * 4 * 34;
                uint8_t * vb = kb + (M / 32) * 34;
                q8_0_store(klo, kb + (size_t)w * 34, l8, err, kv);
                q8_0_store(khi, kb + (size_t)(2 + w) * 34, l8, err, kv);
                q8_0_store(vlo, vb + (size_t)w * 34, l8, err, kv);
                q8_0_store(vhi, vb + (size_t)(2 + w) * 34, l8, err, kv);
            }
        }
    }
}

}   // namespace

// q3p_qk_rope_q8 / its YaRN object: as q3p_qk_rope with the cache a uint8 buffer of Q8_0 rows (2 * (nkv * 128 / 32) * 34 bytes per
// position) and err an int32 word a refused block ORs 2 into. Replaces q3p_qk_rope_q8, kernels/q3m_prefill.hip:534-535 (objects
// q3m_prefill_kvq8 and q3m_prefill_kvq8_yarn); wrapper python/caminus/prefill/q3m_ops.py:122-137.
static int rope_q8_entry(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache, int * err,
                         int yarn, void * stream) {
    if (n < 0 || nh < 1 || nkv < 1 || !qkv || !par || !q16 || !cache || !err || pos0 < 0 || ldq < (nh + 2 * nkv) * 128) return CAM_ERR_ARG;
    if ((long)pos0 + n > (1L << 22)) return CAM_ERR_SHAPE;
    if (!cam_aligned16(qkv) || (ldq & 3) || (reinterpret_cast<uintptr_t>(q16) & 7u) || (reinterpret_cast<uintptr_t>(cache) & 3u) ||
        (reinterpret_cast<uintptr_t>(err) & 3u)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    const int grid = cam_resident_grid(qk_rope_q8_kernel, 256, 0, n);
    qk_rope_q8_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(qkv, ldq, nh, nkv, par, pos0, (uint16_t *)q16, (uint8_t *)cache, err, n, yarn);
    return (int)cudaGetLastError();
}
extern "C" int q3p_qk_rope_q8(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache, int * err,
                              void * stream) {
    return rope_q8_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, err, 0, stream);
}
extern "C" int q3p_qk_rope_q8_yarn(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                                   int * err, void * stream) {
    return rope_q8_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, err, 1, stream);
}
