// Qwen3 per-head q/k RMSNorm fused with NeoX rotary embedding (the reference's q3p_qk_rope, kernels/q3m_prefill.hip:520-591;
// its T = 1 form is the norm + RoPE part of own_op_attn / OP_OWN_ATTS, kernels/k3_own_ops.h:515-542).
//
// Reference statements per head of 128 (one thread per dim, 4 waves): ss = x x; wave sums by the xor butterfly (16, 8, 4, 2, 1),
// the 4 wave sums added in order; scale = rsqrtf(tot / 128 + eps); y1 = (scale x) w; pair (j, j + 64):
// theta = (float)pos powf(theta_scale, (float)j) [YaRN objects: (float)pos freq[j], cos and sin times mscale];
// out[j] = fma(y1[j], c, -(y1[j + 64] s)), out[j + 64] = fma(y1[j + 64], c, y1[j] s); stored as fp16.
//
// Mapping: one thread block per token, looping over tokens. The token's heads are brought into shared memory with cp.async
// (16 bytes per thread, two stages: the next token's copy flies while this one is computed). The 64 cos / sin of a
// position are computed once per token (64 threads) and shared by all of its heads; the reference recomputes them in every
// (token, head) workgroup. A half-warp owns a head: lane l holds dims 4l .. 4l + 3 and 64 + 4l .. 64 + 4l + 3, i.e. complete
// rotation pairs, so the rotation needs no exchange. The reference's sum order is kept: a lane's 8 squares are 8 of its
// threads; butterfly partners 16, 8, 4 are lanes l ^ 4, l ^ 2, l ^ 1, partners 2 and 1 are inside the lane, and the four wave
// sums sit in lanes 0 and 8 of the half-warp (low dims) and again there for the high dims.
#include "cam_common.cuh"

namespace {

struct RopeArgs {
    const void * in0;      // CACHE: qkv fp32 [n][ldq]. Otherwise q fp16 [n][nh][128]
    const void * in1;      // otherwise k fp16 [n][nkv][128]
    const float * par;     // q_norm[128] | k_norm[128] | theta_scale | eps (| freq[64] | mscale)
    uint16_t * out0;       // q16 [n][nh][128]
    uint16_t * out1;       // CACHE: the KV cache (rows of 2 nkv 128 halves). Otherwise k out [n][nkv][128]
    int ldq, nh, nkv, pos0, n, yarn;
};

template <typename T> struct In;
template <> struct In<float> {
    static CAM_DEV void get4(const unsigned char * p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4 *>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <> struct In<uint16_t> {
    static CAM_DEV void get4(const unsigned char * p, float (&f)[4]) {
        const uint2 v = *reinterpret_cast<const uint2 *>(p);
        const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    }
};

// T: the input type. CACHE: the reference's signature (fp32 qkv rows in, q16 and the cache row's K | V halves out).
template <typename T, bool CACHE>
__global__ void __launch_bounds__(384) qk_rope_kernel(const RopeArgs A) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int nh = A.nh, nkv = A.nkv, H = nh + nkv;
    const int in_heads = CACHE ? nh + 2 * nkv : H;                       // heads staged per token
    const size_t stage_bytes = (size_t)in_heads * 128 * sizeof(T);
    float * wq = reinterpret_cast<float *>(smem);                        // [128] | wk [128] | freq [64] | rc [2][64] | rs [2][64]
    float * wk = wq + 128, * freq = wk + 128, * rc = freq + 64, * rs = rc + 128;
    unsigned char * stage = smem + (128 + 128 + 64 + 128 + 128) * 4;
    const float eps = __ldg(A.par + 257);

    if (tid < 128) { wq[tid] = __ldg(A.par + tid); wk[tid] = __ldg(A.par + 128 + tid); }
    if (tid < 64) freq[tid] = A.yarn ? __ldg(A.par + 258 + tid) : cam_powi(__ldg(A.par + 256), tid);
    const float mscale = A.yarn ? __ldg(A.par + 322) : 1.0f;

    auto issue = [&](int t, int st) {
        if (t < A.n) {
            unsigned char * s = stage + (size_t)st * stage_bytes;
            if (CACHE) {
                const unsigned char * src = reinterpret_cast<const unsigned char *>(reinterpret_cast<const float *>(A.in0) + (size_t)t * A.ldq);
                for (int c = tid; c < in_heads * 32; c += blockDim.x) cp_async16(s + (size_t)c * 16, src + (size_t)c * 16);
            } else {
                const unsigned char * sq = reinterpret_cast<const unsigned char *>(reinterpret_cast<const uint16_t *>(A.in0) + (size_t)t * nh * 128);
                const unsigned char * sk = reinterpret_cast<const unsigned char *>(reinterpret_cast<const uint16_t *>(A.in1) + (size_t)t * nkv * 128);
                for (int c = tid; c < nh * 16; c += blockDim.x) cp_async16(s + (size_t)c * 16, sq + (size_t)c * 16);
                for (int c = tid; c < nkv * 16; c += blockDim.x) cp_async16(s + (size_t)(nh * 16 + c) * 16, sk + (size_t)c * 16);
            }
        }
        cp_async_commit();
    };
    auto tables = [&](int t, int buf) {      // threads 0 .. 63 (freq is theirs: thread j wrote freq[j])
        float sn, cs;
        cam_sincos(fmul((float)(A.pos0 + t), freq[tid]), sn, cs);
        rc[buf * 64 + tid] = A.yarn ? fmul(cs, mscale) : cs;
        rs[buf * 64 + tid] = A.yarn ? fmul(sn, mscale) : sn;
    };

    const int t0 = blockIdx.x;
    issue(t0, 0);
    if (tid < 64 && t0 < A.n) tables(t0, 0);
    int st = 0;
    const int hw = lane >> 4, l16 = lane & 15, base = lane & 16;
    for (int t = t0; t < A.n; t += gridDim.x, st ^= 1) {
        const int tn = t + gridDim.x;
        issue(tn, st ^ 1);
        if (tid < 64 && tn < A.n) tables(tn, st ^ 1);
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char * s = stage + (size_t)st * stage_bytes;
        const float * crc = rc + st * 64, * crs = rs + st * 64;
        const int pos = A.pos0 + t;
        for (int h0 = 0; h0 < H; h0 += 2 * nwarps) {
            const int hy = h0 + 2 * warp + hw;
            const bool on = hy < H;
            const bool isq = hy < nh;
            float x[8];
            if (on) {
                const unsigned char * hp = s + (size_t)hy * 128 * sizeof(T);       // q heads then k heads, in both input forms
                float lo[4], hi[4];
                In<T>::get4(hp + (size_t)(4 * l16) * sizeof(T), lo);
                In<T>::get4(hp + (size_t)(64 + 4 * l16) * sizeof(T), hi);
#pragma unroll
                for (int c = 0; c < 4; c++) { x[c] = lo[c]; x[4 + c] = hi[c]; }
            } else {
#pragma unroll
                for (int c = 0; c < 8; c++) x[c] = 0.0f;
            }
            float a[8];
#pragma unroll
            for (int c = 0; c < 8; c++) a[c] = fmul(x[c], x[c]);
#pragma unroll
            for (int o = 4; o > 0; o >>= 1)
#pragma unroll
                for (int c = 0; c < 8; c++) a[c] = fadd(a[c], __shfl_xor_sync(CAM_FULL, a[c], o));          // partners 16, 8, 4
            const float P0 = fadd(fadd(a[0], a[2]), fadd(a[1], a[3])), P1 = fadd(fadd(a[4], a[6]), fadd(a[5], a[7]));   // 2, 1
            float tot = 0.0f;
            tot = fadd(tot, __shfl_sync(CAM_FULL, P0, base));
            tot = fadd(tot, __shfl_sync(CAM_FULL, P0, base + 8));
            tot = fadd(tot, __shfl_sync(CAM_FULL, P1, base));
            tot = fadd(tot, __shfl_sync(CAM_FULL, P1, base + 8));
            if (!on) continue;                                              // (uniform per half-warp; no shuffle follows)
            const float scale = cam_rsqrt(fadd(fdiv(tot, 128.0f), eps));
            const float * wn = isq ? wq : wk;
            const float4 wlo = *reinterpret_cast<const float4 *>(wn + 4 * l16), whi = *reinterpret_cast<const float4 *>(wn + 64 + 4 * l16);
            const float4 c4 = *reinterpret_cast<const float4 *>(crc + 4 * l16), s4 = *reinterpret_cast<const float4 *>(crs + 4 * l16);
            const float wl[4] = {wlo.x, wlo.y, wlo.z, wlo.w}, wh[4] = {whi.x, whi.y, whi.z, whi.w};
            const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
            float ylo[4], yhi[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float x0 = fmul(fmul(scale, x[c]), wl[c]), x1 = fmul(fmul(scale, x[4 + c]), wh[c]);
                ylo[c] = ffma(x0, cc[c], -fmul(x1, sn[c]));
                yhi[c] = ffma(x1, cc[c], fmul(x0, sn[c]));
            }
            uint16_t * o;
            if (isq) o = A.out0 + ((size_t)t * nh + hy) * 128;
            else if (CACHE) o = A.out1 + (size_t)pos * 2 * nkv * 128 + (size_t)(hy - nh) * 128;
            else o = A.out1 + ((size_t)t * nkv + (hy - nh)) * 128;
            st64_stream(o + 4 * l16, make_uint2(f2_to_h2(ylo[0], ylo[1]), f2_to_h2(ylo[2], ylo[3])));
            st64_stream(o + 64 + 4 * l16, make_uint2(f2_to_h2(yhi[0], yhi[1]), f2_to_h2(yhi[2], yhi[3])));
        }
        if (CACHE) {      // v: copied as fp16 into the row's V half
            const float * vs = reinterpret_cast<const float *>(s) + (size_t)H * 128;
            uint16_t * vo = A.out1 + (size_t)pos * 2 * nkv * 128 + (size_t)nkv * 128;
            for (int c = tid; c < nkv * 32; c += blockDim.x) {
                const float4 v = *reinterpret_cast<const float4 *>(vs + 4 * c);
                st64_stream(vo + 4 * c, make_uint2(f2_to_h2(v.x, v.y), f2_to_h2(v.z, v.w)));
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
}

// the block size whose half-warps divide the token's heads with the least idle half-warps (more warps on a tie)
int pick_warps(int H) {
    int best = 8, waste = 1 << 30;
    for (int w = 12; w >= 4; w--) {
        const int passes = (H + 2 * w - 1) / (2 * w);
        const int idle = passes * 2 * w - H;
        if (idle < waste) { waste = idle; best = w; }
    }
    return best;
}

template <typename T, bool CACHE>
int launch_rope(const RopeArgs & A, cudaStream_t stream) {
    const int H = A.nh + A.nkv;
    const int in_heads = CACHE ? A.nh + 2 * A.nkv : H;
    const size_t smem = (128 + 128 + 64 + 128 + 128) * 4 + 2 * (size_t)in_heads * 128 * sizeof(T);
    if (smem > 227 * 1024) return CAM_ERR_SHAPE;
    const cudaError_t e = cudaFuncSetAttribute(qk_rope_kernel<T, CACHE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    const int warps = pick_warps(H);
    const int grid = cam_resident_grid(qk_rope_kernel<T, CACHE>, warps * 32, smem, A.n);
    qk_rope_kernel<T, CACHE><<<grid, warps * 32, smem, stream>>>(A);
    return (int)cudaGetLastError();
}

int check_common(int n, int nh, int nkv, const void * par, int pos0) {
    if (n < 0 || nh < 1 || nkv < 0 || !par || pos0 < 0) return CAM_ERR_ARG;
    if ((long)pos0 + n > (1L << 22)) return CAM_ERR_SHAPE;      // the angle's range reduction holds below 2^22 radians
    if (reinterpret_cast<uintptr_t>(par) & 3u) return CAM_ERR_ALIGN;
    return CAM_OK;
}

}   // namespace

// q3p_qk_rope: qkv fp32 [n][ldq] = q (nh heads) | k (nkv) | v (nkv); q16 fp16 [n][nh][128]; cache fp16, row pos0 + t =
// K [nkv][128] | V [nkv][128]. n and nh + nkv are the reference's grid.x and grid.y. yarn = 0: the plain object
// (q3m_prefill); yarn = 1: the YaRN objects (q3m_prefill_yarn), par carries freq[64] | mscale after eps.
// Reference: kernels/q3m_prefill.hip:537-538; wrapper python/caminus/prefill/q3m_ops.py:122-139 (which checks the span).
static int qk_rope_entry(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                         int yarn, void * stream) {
    const int r = check_common(n, nh, nkv, par, pos0);
    if (r != CAM_OK) return r;
    if (nkv < 1 || !qkv || !q16 || !cache || ldq < (nh + 2 * nkv) * 128) return CAM_ERR_ARG;
    if (!cam_aligned16(qkv) || (ldq & 3) || (reinterpret_cast<uintptr_t>(q16) & 7u) || (reinterpret_cast<uintptr_t>(cache) & 7u))
        return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    const RopeArgs A = {qkv, nullptr, par, (uint16_t *)q16, (uint16_t *)cache, ldq, nh, nkv, pos0, n, yarn};
    return launch_rope<float, true>(A, (cudaStream_t)stream);
}
extern "C" int q3p_qk_rope(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                           void * stream) {
    return qk_rope_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, 0, stream);
}
extern "C" int q3p_qk_rope_yarn(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16,
                                void * cache, void * stream) {
    return qk_rope_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, 1, stream);
}

// cam_qk_rope_f16: the same statements on fp16 q [n][nh][128] and k [n][nkv][128] (widened exactly), fp16 out (qo / ko may be
// q / k: a token's heads are staged before any of them is written). No counterpart entry in the reference, whose kernel
// takes fp32 GEMM outputs; arithmetic as q3p_qk_rope (kernels/q3m_prefill.hip:552-590).
extern "C" int cam_qk_rope_f16(int n, const void * q, const void * k, int nh, int nkv, const float * par, int pos0, void * qo,
                               void * ko, int yarn, void * stream) {
    const int r = check_common(n, nh, nkv, par, pos0);
    if (r != CAM_OK) return r;
    if (!q || !qo || (nkv > 0 && (!k || !ko))) return CAM_ERR_ARG;
    if (!cam_aligned16(q) || !cam_aligned16(qo) || (nkv > 0 && (!cam_aligned16(k) || !cam_aligned16(ko)))) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    const RopeArgs A = {q, k, par, (uint16_t *)qo, (uint16_t *)ko, 0, nh, nkv, pos0, n, yarn};
    return launch_rope<uint16_t, false>(A, (cudaStream_t)stream);
}
