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

// The same sums for many tokens: a block takes a tile of 32 tokens x 16 experts, a warp 8 tokens x 8 experts of it (one
// accumulator per pair in every lane, the lanes splitting K as above). Steps of 128 values of K are brought into shared memory
// with cp.async, three stages deep (32 rows of h and 16 of Wr, 512 bytes each), so a step costs a warp 16 16-byte shared-memory
// loads for 64 pairs instead of two global loads per pair, and no load waits on DRAM. Per pair the statements and their order
// are router_kernel's.
constexpr int RT_TOK = 32, RT_EXP = 16, RT_STAGES = 3, RT_STAGE_FLOATS = (RT_TOK + RT_EXP) * 128;

__global__ void __launch_bounds__(256) router_tile_kernel(const float * __restrict__ h, const float * __restrict__ Wr, int E, int K,
                                                          float * __restrict__ logits, int n) {
    extern __shared__ __align__(16) float rt_smem[];
    const int tid = threadIdx.x, lane = tid & 31, wave = tid >> 5;
    const int t0 = blockIdx.x * RT_TOK, e0 = blockIdx.y * RT_EXP;
    const int wt = (wave >> 1) * 8, we = (wave & 1) * 8;                   // this warp's tokens wt .. wt + 7, experts we .. we + 7 of the tile
    // a thread copies chunks tid, tid + 256, .. of a stage's 1536 (row = chunk / 32: 32 token rows, then 16 expert rows)
    const float * src[6];
#pragma unroll
    for (int c = 0; c < 6; c++) {
        const int row = (tid + 256 * c) >> 5;
        src[c] = (row < RT_TOK ? h + (size_t)min(t0 + row, n - 1) * K : Wr + (size_t)min(e0 + row - RT_TOK, E - 1) * K) + 4 * lane;
    }                                                                      // (a tile's overhang recomputes the last row / expert)
    const int nks = K >> 7;
    auto issue = [&](int ks) {
        if (ks < nks) {
            float * st = rt_smem + (ks % RT_STAGES) * RT_STAGE_FLOATS;
#pragma unroll
            for (int c = 0; c < 6; c++) cp_async16(st + (tid + 256 * c) * 4, src[c] + ks * 128);
        }
        cp_async_commit();
    };
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;
    issue(0); issue(1);
    for (int ks = 0; ks < nks; ks++) {
        cp_async_wait<1>();
        __syncthreads();                                                   // stage ks has landed for everyone; everyone is done with stage ks - 1
        issue(ks + 2);
        const float * st = rt_smem + (ks % RT_STAGES) * RT_STAGE_FLOATS + 4 * lane;
        float4 xv[8], wv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) xv[i] = *reinterpret_cast<const float4 *>(st + (wt + i) * 128);
#pragma unroll
        for (int j = 0; j < 8; j++) wv[j] = *reinterpret_cast<const float4 *>(st + (RT_TOK + we + j) * 128);
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float d = fmul(wv[j].x, xv[i].x); d = ffma(wv[j].y, xv[i].y, d); d = ffma(wv[j].z, xv[i].z, d); d = ffma(wv[j].w, xv[i].w, d);
                acc[i][j] = fadd(acc[i][j], d);
            }
    }
    cp_async_wait<0>();
    float mine[2] = {0.0f, 0.0f};                                          // lane l stores pairs (token l / 8 and 4 + l / 8, expert l % 8)
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) { const float v = wsum(acc[i][j]); if (lane == (i & 3) * 8 + j) mine[i >> 2] = v; }      // (every lane holds the same total)
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int ti = t0 + wt + 4 * hh + (lane >> 3), ej = e0 + we + (lane & 7);
        if (ti < n && ej < E) logits[(size_t)ti * E + ej] = mine[hh];
    }
}

// (a warp per token as in the reference, eight tokens to a block)
__global__ void __launch_bounds__(256) topk_kernel(const float * __restrict__ logits, int E, int k, float floor_, int * __restrict__ ids,
                                                   float * __restrict__ wts, int * __restrict__ err, int n) {
    const int lane = threadIdx.x & 31, t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= n) return;                                  // (whole warps; no block-wide barrier below)
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
    // rank-based top-k (rank = how many probabilities are larger, or equal with a lower index): the element of rank r is the r-th
    // maximum under that order, so k rounds of a warp-wide argmax over the key (probability bits, then lower index first) give
    // sel[0 .. k - 1]. Probabilities are >= 0, so their bit patterns order like the numbers.
    long long key[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int e = lane + 32 * j;
        key[j] = e < E ? (long long)(((unsigned long long)__float_as_uint(v[j]) << 32) | (unsigned)(0x7fffffff - e)) : -1;
    }
    int i = 0;
    for (int r = 0; r < k; r++) {
        long long best = key[0] > key[1] ? key[0] : key[1];
        const long long b2 = key[2] > key[3] ? key[2] : key[3];
        best = best > b2 ? best : b2;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { const long long q = __shfl_xor_sync(CAM_FULL, best, o); best = q > best ? q : best; }
        const int e = 0x7fffffff - (int)(unsigned)(best & 0xffffffffll);
        if (lane == r) i = e;
        if (lane == (e & 31)) {
#pragma unroll
            for (int j = 0; j < 4; j++) if ((e >> 5) == j) key[j] = -1;
        }
    }
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
    if (n >= 64) {
        const size_t smem = (size_t)RT_STAGES * RT_STAGE_FLOATS * 4;
        const cudaError_t e = cudaFuncSetAttribute(router_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     // (72 KB: above the default limit)
        if (e != cudaSuccess) return (int)e;
        router_tile_kernel<<<dim3((n + RT_TOK - 1) / RT_TOK, (E + RT_EXP - 1) / RT_EXP), 256, smem, (cudaStream_t)stream>>>(h, Wr, E, K, logits, n);
    } else router_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(h, Wr, E, K, logits);
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
