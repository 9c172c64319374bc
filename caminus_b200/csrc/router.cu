// The router glue of the Qwen3-MoE prefill (the reference's q3p_router, q3p_topk, q3p_group, kernels/q3m_prefill.hip:417-513;
// wrappers python/caminus/prefill/q3m_ops.py:94-104): fp32 router logits, softmax + rank-based top-k with lower-index-first
// ties, and the grouping of (token, slot) pairs by expert into work items of at most 64 pairs. The mappings are the
// reference's (a warp per logit row; a warp per token; one block of 1024 threads for the grouping), so every sum has its order.
#include "cam_common.cuh"

namespace {

struct MMItem { int e, off, cnt, pad; };
constexpr int MM_M = 64;

CAM_DEV float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fadd(v, __shfl_xor_sync(CAM_FULL, v, o));
    return v;
}
CAM_DEV float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(CAM_FULL, v, o));
    return v;
}
CAM_DEV bool finite_f(float x) { return fabsf(x) <= 3.402823466e38f; }

__global__ void __launch_bounds__(256) router_kernel(const float * __restrict__ h, const float * __restrict__ Wr, int E, int K, float * __restrict__ logits) {
    const int lane = threadIdx.x & 31, wave = threadIdx.x >> 5, t = blockIdx.x;
    const float * x = h + (size_t)t * K;
    for (int e = wave; e < E; e += 8) {
        const float * wr = Wr + (size_t)e * K;
        float acc = 0.0f;
        for (int k0 = lane * 4; k0 < K; k0 += 128) {
            const float4 wv = __ldg(reinterpret_cast<const float4 *>(wr + k0)), xv = __ldg(reinterpret_cast<const float4 *>(x + k0));
            float d = fmul(wv.x, xv.x); d = ffma(wv.y, xv.y, d); d = ffma(wv.z, xv.z, d); d = ffma(wv.w, xv.w, d);
            acc = fadd(acc, d);
        }
        acc = wsum(acc);
        if (lane == 0) logits[(size_t)t * E + e] = acc;
    }
}

// The same sums for many tokens: a warp holds TT tokens x EE experts (one accumulator per pair in every lane, the lanes
// splitting K as above), so a step over 128 values of K costs TT + EE 16-byte loads for TT EE pairs instead of two per pair; the
// 16 warps of a block take 16 EE experts of the same TT tokens, whose rows they share through L1. Per pair the statements and
// their order are router_kernel's.
template <int TT, int EE>
__global__ void __launch_bounds__(512) router_tile_kernel(const float * __restrict__ h, const float * __restrict__ Wr, int E, int K,
                                                          float * __restrict__ logits, int n) {
    const int lane = threadIdx.x & 31, wave = threadIdx.x >> 5;
    const int t0 = blockIdx.x * TT, e0 = (blockIdx.y * 16 + wave) * EE;
    if (e0 >= E) return;
    const float * xp[TT], * wp[EE];
#pragma unroll
    for (int i = 0; i < TT; i++) xp[i] = h + (size_t)min(t0 + i, n - 1) * K + lane * 4;       // (a tile's overhang recomputes the last row / expert)
#pragma unroll
    for (int j = 0; j < EE; j++) wp[j] = Wr + (size_t)min(e0 + j, E - 1) * K + lane * 4;
    float acc[TT][EE];
#pragma unroll
    for (int i = 0; i < TT; i++)
#pragma unroll
        for (int j = 0; j < EE; j++) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 128) {
        float4 xv[TT], wv[EE];
#pragma unroll
        for (int i = 0; i < TT; i++) xv[i] = __ldg(reinterpret_cast<const float4 *>(xp[i] + k0));
#pragma unroll
        for (int j = 0; j < EE; j++) wv[j] = __ldg(reinterpret_cast<const float4 *>(wp[j] + k0));
#pragma unroll
        for (int i = 0; i < TT; i++)
#pragma unroll
            for (int j = 0; j < EE; j++) {
                float d = fmul(wv[j].x, xv[i].x); d = ffma(wv[j].y, xv[i].y, d); d = ffma(wv[j].z, xv[i].z, d); d = ffma(wv[j].w, xv[i].w, d);
                acc[i][j] = fadd(acc[i][j], d);
            }
    }
    float mine = 0.0f;
#pragma unroll
    for (int i = 0; i < TT; i++)
#pragma unroll
        for (int j = 0; j < EE; j++) { const float v = wsum(acc[i][j]); if (lane == i * EE + j) mine = v; }      // (every lane holds the same total)
    const int ti = t0 + lane / EE, ej = e0 + lane % EE;
    if (lane < TT * EE && ti < n && ej < E) logits[(size_t)ti * E + ej] = mine;
}

// (a warp per token as in the reference, eight tokens to a block)
__global__ void __launch_bounds__(256) topk_kernel(const float * __restrict__ logits, int E, int k, float floor_, int * __restrict__ ids,
                                                   float * __restrict__ wts, int * __restrict__ err, int n) {
    __shared__ int sel_[8][64];
    const int lane = threadIdx.x & 31, t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= n) return;                                  // (whole warps; no block-wide barrier below)
    int * sel = sel_[threadIdx.x >> 5];
    const float * lg = logits + (size_t)t * E;
    float v[4]; bool bad = false;
#pragma unroll
    for (int j = 0; j < 4; j++) { const int e = lane + 32 * j; v[j] = e < E ? __ldg(lg + e) : -__int_as_float(0x7f800000); if (e < E && !finite_f(v[j])) bad = true; }
    const float m = wmax(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (lane + 32 * j < E) { v[j] = cam_expf(fsub(v[j], m)); sum = fadd(sum, v[j]); } else v[j] = 0.0f;
    }
    sum = wsum(sum);
    const float inv = fdiv(1.0f, sum);
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = fmul(v[j], inv);
    int rk[4] = {0, 0, 0, 0};
    for (int src = 0; src < 32; src++) {
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float pj = __shfl_sync(CAM_FULL, v[jj], src); const int ej = src + 32 * jj;
#pragma unroll
            for (int j = 0; j < 4; j++) { const int ei = lane + 32 * j; if (ej < E && ei < E) rk[j] += (pj > v[j]) || (pj == v[j] && ej < ei); }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) if (lane + 32 * j < E && rk[j] < k) sel[rk[j]] = lane + 32 * j;
    __syncwarp();
    const int i = lane < k ? sel[lane] : 0;
    float pv[4];
#pragma unroll
    for (int j = 0; j < 4; j++) pv[j] = __shfl_sync(CAM_FULL, v[j], i & 31);
    const float p_i = pv[(i >> 5) & 3];
    float ws = 0.0f;
    for (int j = 0; j < k; j++) ws = fadd(ws, __shfl_sync(CAM_FULL, p_i, j));
    ws = fmaxf(ws, floor_);
    if (lane < k) { ids[(size_t)t * k + lane] = i; wts[(size_t)t * k + lane] = fdiv(p_i, ws); }
    if (bad) atomicOr(err, 1);
}

__global__ void __launch_bounds__(1024) group_kernel(const int * __restrict__ ids, int npairs, int k, int E, int * __restrict__ xs, int * __restrict__ yd,
                                                     MMItem * __restrict__ items, int * __restrict__ nitems, int * __restrict__ err) {
    __shared__ int cnt[1024], off[1024], cur[1024], ioff[1024];
    const int tid = threadIdx.x;
    if (tid < E) { cnt[tid] = 0; cur[tid] = 0; }
    __syncthreads();
    for (int p = tid; p < npairs; p += 1024) {
        int e = ids[p];
        if (e < 0 || e >= E) { atomicOr(err, 2); e = 0; }
        atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (tid == 0) {
        int o = 0, io = 0;
        for (int e = 0; e < E; e++) { off[e] = o; ioff[e] = io; o += cnt[e]; io += (cnt[e] + MM_M - 1) / MM_M; }
        *nitems = io;
    }
    __syncthreads();
    for (int p = tid; p < npairs; p += 1024) {
        int e = ids[p]; if (e < 0 || e >= E) e = 0;
        const int sl = off[e] + atomicAdd(&cur[e], 1);
        xs[sl] = p / k; yd[sl] = p;
    }
    if (tid < E) {
        const int c = cnt[tid];
        for (int j = 0; j * MM_M < c; j++) { MMItem it; it.e = tid; it.off = off[tid] + j * MM_M; it.cnt = min(MM_M, c - j * MM_M); it.pad = 0; items[ioff[tid] + j] = it; }
    }
}

}   // namespace

// q3p_router: kernels/q3m_prefill.hip:419-420 (n = grid.x); K a multiple of 128, 16-byte aligned rows
extern "C" int q3p_router(int n, const float * h, const float * Wr, int E, int K, float * logits, void * stream) {
    if (n < 0 || E < 1 || K < 128 || (K & 127) || !h || !Wr || !logits) return CAM_ERR_ARG;
    if (!cam_aligned16(h) || !cam_aligned16(Wr)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    if (n >= 64) router_tile_kernel<8, 4><<<dim3((n + 7) / 8, (E + 63) / 64), 512, 0, (cudaStream_t)stream>>>(h, Wr, E, K, logits, n);
    else router_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(h, Wr, E, K, logits);
    return (int)cudaGetLastError();
}
// q3p_topk: kernels/q3m_prefill.hip:440-441 (n = grid.x); E <= 128, k <= 32
extern "C" int q3p_topk(int n, const float * logits, int E, int k, float floor_, int * ids, float * wts, int * err, void * stream) {
    if (n < 0 || E < 1 || E > 128 || k < 1 || k > 32 || k > E || !logits || !ids || !wts || !err) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    topk_kernel<<<(n + 7) / 8, 256, 0, (cudaStream_t)stream>>>(logits, E, k, floor_, ids, wts, err, n);
    return (int)cudaGetLastError();
}
// q3p_group: kernels/q3m_prefill.hip:490-492; items are { int e, off, cnt, pad }; E <= 1024
extern "C" int q3p_group(const int * ids, int npairs, int k, int E, int * xs, int * yd, void * items, int * nitems, int * err, void * stream) {
    if (npairs < 0 || k < 1 || E < 1 || E > 1024 || !ids || !xs || !yd || !items || !nitems || !err) return CAM_ERR_ARG;
    group_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, npairs, k, E, xs, yd, (MMItem *)items, nitems, err);
    return (int)cudaGetLastError();
}
