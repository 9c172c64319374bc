// The training line's fused activation quantiser, forward (the reference's kernels/actq.hip: actq_fwd_*, silu_mul_actq_fwd,
// block_entry_fwd; wrappers python/caminus/train/actq.py:22-169).
//
// Per row of K values (a multiple of 128, <= 8192): the source value is rounded to bf16, each chunk of 128 goes through the
// unnormalised Walsh-Hadamard butterflies (1, 2 inside a lane's four values, 4 .. 64 across the lanes of a warp), times the bf16
// value of 1 / sqrt(128), rounded to bf16; the row's amax gives s = max(amax clip / qmax, 1e-8); the codes are
// clamp(rint(u / s), -qmax - 1, qmax); outputs: the dequantised bf16 values (optional), the row scale, the int4 codes packed four
// to 16 bits (optional). Sources: a bf16 or fp32 tensor; the MLP activation bf16(bf16(silu(g)) u) computed from [g | u] rows; the
// RMSNorm (x rstd) w never materialised (block entry), which also emits up to 16 thin bf16 gate projections.
// The mapping is the reference's (one block of 8 warps per row, warp w takes chunks w, w + 8, ..), so every reduction has its order.
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

struct PlainBf16 { const uint16_t * x; int K; CAM_DEV float operator()(int row, int k) const { return bf2f(__ldg(x + (size_t)row * K + k)); } };
struct PlainF32 { const float * x; int K; CAM_DEV float operator()(int row, int k) const { return __ldg(x + (size_t)row * K + k); } };
struct SiluMulSrc {
    const uint16_t * gu; int ld, F;
    CAM_DEV float operator()(int row, int k) const {
        const uint16_t * r = gu + (size_t)row * ld;
        return rbf(fmul(rbf(cam_silu(bf2f(__ldg(r + k)))), bf2f(__ldg(r + F + k))));
    }
};
struct RmsSrc {
    const float * x; const float * w; float rstd; int d;
    CAM_DEV float operator()(int row, int k) const { return fmul(fmul(__ldg(x + (size_t)row * d + k), rstd), __ldg(w + k)); }
};

template <typename Src>
CAM_DEV void actq_fwd_src(Src src, uint16_t * __restrict__ y, float * __restrict__ s_out, int K, float clip, int qmax, uint16_t * __restrict__ codes,
                          float * lds) {
    const int row = blockIdx.x, wave = threadIdx.x >> 5, lane = threadIdx.x & 31, nch = K / 128;
    float u[AQ_MAXC][4];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < AQ_MAXC; c++) {
        const int ch = wave + c * AQ_WAVES;
        if (ch < nch) {                                            // (uniform per warp)
#pragma unroll
            for (int e = 0; e < 4; e++) u[c][e] = rbf(src(row, ch * 128 + lane * 4 + e));
            fwht128(u[c], lane);
#pragma unroll
            for (int e = 0; e < 4; e++) { u[c][e] = rbf(fmul(u[c][e], 0.08837890625f)); amax = fmaxf(amax, fabsf(u[c][e])); }
        }
    }
    amax = block_reduce(wave_max(amax), lds, wave, lane, true);
    const float s = fmaxf(fdiv(fmul(amax, clip), (float)qmax), 1e-8f);
    if (threadIdx.x == 0 && s_out) s_out[row] = s;
    uint16_t * yr = y ? y + (size_t)row * K : nullptr;
#pragma unroll
    for (int c = 0; c < AQ_MAXC; c++) {
        const int ch = wave + c * AQ_WAVES;
        if (ch < nch) {
            uint32_t pk = 0;
            uint16_t o[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float q = fminf(fmaxf(rintf(fdiv(u[c][e], s)), (float)(-qmax - 1)), (float)qmax);
                o[e] = f2bf(fmul(q, s));
                pk |= ((uint32_t)(int)q & 0xFu) << (4 * e);
            }
            if (y) st64(yr + ch * 128 + lane * 4, make_uint2(o[0] | ((uint32_t)o[1] << 16), o[2] | ((uint32_t)o[3] << 16)));
            if (codes) codes[(size_t)row * (K / 4) + ch * 32 + lane] = (uint16_t)pk;
        }
    }
}

template <typename Src>
__global__ void __launch_bounds__(256) actq_kernel(Src src, uint16_t * y, float * s, int K, float clip, int qmax, uint16_t * codes) {
    __shared__ float lds[AQ_WAVES];
    actq_fwd_src(src, y, s, K, clip, qmax, codes, lds);
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
    actq_kernel<<<M, 256, 0, CAM_ST>>>(PlainBf16{(const uint16_t *)x, K}, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes);
    return (int)cudaGetLastError();
}
extern "C" int actq_fwd_codes_f32(int M, const float * x, void * y, float * s, void * codes, int K, float clip, int qmax, void * stream) {
    const int r = check_actq(M, K, qmax, x, s); if (r || M == 0) return r;
    if (misaligned8(y)) return CAM_ERR_ALIGN;
    actq_kernel<<<M, 256, 0, CAM_ST>>>(PlainF32{x, K}, (uint16_t *)y, s, K, clip, qmax, (uint16_t *)codes);
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
    actq_kernel<<<M, 256, 0, CAM_ST>>>(SiluMulSrc{(const uint16_t *)gu, ld, F}, (uint16_t *)y, s, F, clip, qmax, (uint16_t *)codes);
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
    block_entry_kernel<<<M, 256, 0, CAM_ST>>>(x, nw, (const uint16_t *)wab, nab, eps, (uint16_t *)y, s, (uint16_t *)codes, (uint16_t *)ab, rstd_out, d, clip, qmax);
    return (int)cudaGetLastError();
}
