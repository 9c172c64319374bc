// The router glue of the Qwen3-MoE prefill (the reference's q3p_router, q3p_topk, q3p_group, kernels/q3m_prefill.hip:417-513;
// wrappers python/caminus/prefill/q3m_ops.py:94-104) and the hyper-connection line's pf_router (kernels/prefill_glue.hip:208-308):
// fp32 router logits, softmax + rank-based top-k with lower-index-first ties, and the grouping of (token, slot) pairs by expert into
// work items of at most 64 pairs. What the reference fixes is the order of every floating-point sum (stated at each kernel); the
// mappings onto the device are this library's: logits by shared-memory tiles (many tokens) or one warp per expert (few tokens), the
// softmax and top-k by one warp per token, the grouping by a thread-block cluster that counts, scans through distributed shared
// memory and scatters in pair order.
#include "cam_common.cuh"

#include <cooperative_groups.h>
#include <cstdlib>

namespace cg = cooperative_groups;

namespace {

struct WorkItem { int expert, first, count, zero; };       // the reference's 16-byte work item { e, off, cnt, pad } (q3m_prefill.hip MMItem)
constexpr int ITEM_PAIRS = 64;                             // pairs per work item (python/caminus/prefill/q3m_ops.py:21 MM_M)

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
CAM_DEV float dot4(const float4 w, const float4 x) {        // the reference's per-step expression w.x x.x + w.y x.y + .. as it contracts: one product, three fma
    float d = fmul(w.x, x.x); d = ffma(w.y, x.y, d); d = ffma(w.z, x.z, d); return ffma(w.w, x.w, d);
}

// Few tokens (n < 64): the weights are what is read (E K floats), the tokens fit in cache. A warp owns one expert and walks the tokens
// two at a time, so an expert's row comes from DRAM once and the grid is E warps wide whatever n is (a block per token would leave
// most of the device idle at n = 1). Per (token, expert) the statements are the reference's: lane l adds the float4 products of
// k = 4 l + 128 i in the order of i, then the xor butterfly 16, 8, 4, 2, 1.
__global__ void __launch_bounds__(256) router_few_kernel(const float * __restrict__ h, const float * __restrict__ Wr, int E, int K,
                                                         float * __restrict__ logits, int n) {
    const int lane = threadIdx.x & 31, e = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (e >= E) return;                                                    // (whole warps; no block-wide barrier below)
    const float4 * wr = reinterpret_cast<const float4 *>(Wr + (size_t)e * K) + lane;
    const int steps = K >> 7;
    for (int t = 0; t < n; t += 2) {
        const int t1 = min(t + 1, n - 1);
        const float4 * x0 = reinterpret_cast<const float4 *>(h + (size_t)t * K) + lane, * x1 = reinterpret_cast<const float4 *>(h + (size_t)t1 * K) + lane;
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 4
        for (int i = 0; i < steps; i++) {
            const float4 wv = __ldg(wr + 32 * i);
            a0 = fadd(a0, dot4(wv, __ldg(x0 + 32 * i))); a1 = fadd(a1, dot4(wv, __ldg(x1 + 32 * i)));
        }
        a0 = wsum(a0); a1 = wsum(a1);
        if (lane == 0) { logits[(size_t)t * E + e] = a0; if (t1 != t) logits[(size_t)t1 * E + e] = a1; }
    }
}

// The same sums for many tokens: a block takes a tile of 32 tokens x 16 experts, a warp 8 tokens x 8 experts of it (one
// accumulator per pair in every lane, the lanes splitting K as above). Steps of 128 values of K are brought into shared memory
// with cp.async, three stages deep (32 rows of h and 16 of Wr, 512 bytes each), so a step costs a warp 16 16-byte shared-memory
// loads for 64 pairs instead of two global loads per pair, and no load waits on DRAM. Per pair the statements and their order
// are the ones stated above router_few_kernel.
constexpr int RT_TOK = 32, RT_EXP = 16, RT_STAGES = 3, RT_STAGE_FLOATS = (RT_TOK + RT_EXP) * 128;
constexpr int RT_SUMS_PITCH = RT_TOK * RT_EXP + 1;                        // a lane's 512 partial sums (+ 1: the lanes of a warp on different banks)
static_assert(32 * RT_SUMS_PITCH <= RT_STAGES * RT_STAGE_FLOATS, "the partial sums reuse the stages");

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
            for (int j = 0; j < 8; j++) acc[i][j] = fadd(acc[i][j], dot4(wv[j], xv[i]));
    }
    cp_async_wait<0>();
    __syncthreads();                                                       // (the stages become the partial sums [lane][token][expert])
    // The 32 lanes' partial sums of a pair meet in shared memory and one thread adds them as the xor butterfly 16, 8, 4, 2, 1 does
    // (lane 0's tree; the additions commute, so every lane's total is that one): 31 additions per pair instead of 160 and no shuffles.
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) rt_smem[lane * RT_SUMS_PITCH + (wt + i) * RT_EXP + we + j] = acc[i][j];
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int pair = tid + 256 * hh;
        float p[32];
#pragma unroll
        for (int c = 0; c < 32; c++) p[c] = rt_smem[c * RT_SUMS_PITCH + pair];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int c = 0; c < o; c++) p[c] = fadd(p[c], p[c + o]);
        const int ti = t0 + (pair >> 4), ej = e0 + (pair & 15);
        if (ti < n && ej < E) logits[(size_t)ti * E + ej] = p[0];
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

// ---- pf_router: softmax over E <= 1024 logits and the k <= 64 most probable experts of a token ----------------------------------------
// The reference runs a workgroup of 256 per token: thread tid owns logits tid + 256 j (j < 4), its sum is the chain over j from 0.0f, a
// wave adds by the butterfly 16, 8, 4, 2, 1 and the eight wave sums are added in wave order (kernels/prefill_glue.hip:251-268). Here a
// warp owns the token: lane l holds, for every wave w of the reference, the values of that wave's lane l (logits 32 w + l + 256 j), so
// a wave's butterfly is a warp butterfly and the eight totals are added in a register. The k experts come from k rounds of a warp-wide
// argmax over (probability bits as a signed integer, lower index first): the r-th round's winner is the element of rank r under the
// reference's order (rank = how many are larger, or equal with a lower index), so ids and weights are slot for slot the reference's.
// Each pick is masked out before the next round: the k ids are distinct and below E by construction, also for a token whose logits are
// not finite (err |= 1; the reference's further flags 2 and 4, an id out of range or repeated, cannot arise).
template <int NJ>
__global__ void __launch_bounds__(256) softmax_topk_rows_kernel(const float * __restrict__ logits, int E, int k, float clamp, int * __restrict__ ids,
                                                                float * __restrict__ wts, int * __restrict__ err, int n) {
    const int lane = threadIdx.x & 31, t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= n) return;                                                    // (whole warps; no block-wide barrier below)
    const float * lg = logits + (size_t)t * E;
    const float ninf = -__int_as_float(0x7f800000);
    float v[8][NJ]; bool bad = false; float m = ninf;
#pragma unroll
    for (int j = 0; j < NJ; j++)
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const int e = 32 * w + lane + 256 * j;
            v[w][j] = e < E ? __ldg(lg + e) : ninf;
            if (e < E) { bad |= !finite_f(v[w][j]); m = fmaxf(m, v[w][j]); }
        }
    m = wmax(m);
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < NJ; j++)
            if (32 * w + lane + 256 * j < E) { v[w][j] = cam_expf(fsub(v[w][j], m)); s = fadd(s, v[w][j]); }
        s = wsum(s);
        total = w == 0 ? s : fadd(total, s);
    }
    const float inv = fdiv(1.0f, total);
    const long long none = (long long)0x8000000000000000ull;               // below every key of a real element (a probability's bits are never 0x80000000)
    long long key[8][NJ];
#pragma unroll
    for (int w = 0; w < 8; w++)
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const int e = 32 * w + lane + 256 * j;
            const unsigned pb = __float_as_uint(fmul(v[w][j], inv));
            key[w][j] = e < E ? (long long)(((unsigned long long)pb << 32) | (unsigned)(0x7fffffff - e)) : none;
        }
    int sel_e[2] = {0, 0}; float sel_p[2] = {0.0f, 0.0f};                  // lane l keeps slots l and l + 32
    for (int r = 0; r < k; r++) {
        long long best = none;
#pragma unroll
        for (int w = 0; w < 8; w++)
#pragma unroll
            for (int j = 0; j < NJ; j++) best = key[w][j] > best ? key[w][j] : best;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { const long long q = __shfl_xor_sync(CAM_FULL, best, o); best = q > best ? q : best; }
        const int e = 0x7fffffff - (int)(unsigned)(best & 0xffffffffll);
        if (lane == (r & 31)) { sel_e[r >> 5] = e; sel_p[r >> 5] = __uint_as_float((unsigned)((unsigned long long)best >> 32)); }
        if (lane == (e & 31)) {
#pragma unroll
            for (int w = 0; w < 8; w++)
#pragma unroll
                for (int j = 0; j < NJ; j++) if (((e >> 5) & 7) == w && (e >> 8) == j) key[w][j] = none;
        }
    }
    float ws = 0.0f;
    for (int j = 0; j < k; j++) ws = fadd(ws, __shfl_sync(CAM_FULL, j < 32 ? sel_p[0] : sel_p[1], j & 31));
    ws = fmaxf(ws, clamp);
#pragma unroll
    for (int q = 0; q < 2; q++) {
        const int slot = lane + 32 * q;
        if (slot < k) { ids[(size_t)t * k + slot] = sel_e[q]; wts[(size_t)t * k + slot] = fdiv(sel_p[q], ws); }
    }
    if (bad) atomicOr(err, 1);
}

// ---- q3p_group: the (token, slot) pairs of a chunk listed by expert, and the experts' lists cut into work items of at most 64 pairs ------
// One thread-block cluster of up to 8 blocks x 32 warps; no global scratch. A warp takes a contiguous run of pairs, 32 at a time:
//   count    lanes holding the same expert find each other (a ballot per bit of the expert's number); the first of them adds their number to the warp's own
//            counter of that expert in shared memory (a cell per warp and expert: no atomics);
//   scan     a block adds its warps' cells (a warp per expert, by shuffles), the blocks read one another's totals through distributed
//            shared memory, and every block derives the same expert offsets (an exclusive scan over the experts) and its own start
//            inside every expert's list; the warps' cells become their write cursors (a warp scan per expert);
//   scatter  the second pass over the same pairs (kept in registers when a warp has at most 8 steps) writes pair p at cursor + its
//            rank among the step's equal lanes.
// A warp's pairs are ascending and the cursors follow (block, warp) order, so every expert's list is in ascending pair order: the
// result does not depend on timing (the reference's order follows its atomics; it states that the order inside a list changes no bit
// downstream), and the rows a GEMM gathers through xs ascend. An id outside [0, E) counts as expert 0 and sets err |= 2.
constexpr int GR_WARPS = 32, GR_KEEP = 8, GR_PITCH = GR_WARPS + 1;

// the lanes whose v equals this lane's (v < 2^nbits): one ballot per bit. (match.any gives the same mask, but takes a step per distinct
// value in the warp: 28 of them for 32 pairs spread over 128 experts, against 7 ballots.)
CAM_DEV unsigned same_lanes(unsigned v, int nbits) {
    unsigned same = CAM_FULL;
    for (int b = 0; b < nbits; b++) {
        const unsigned set = __ballot_sync(CAM_FULL, (v >> b) & 1u);
        same &= ((v >> b) & 1u) ? set : ~set;
    }
    return same;
}

CAM_DEV int wscan_excl(int v, int lane) {            // exclusive prefix sum over the warp's lanes
    int s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int t = __shfl_up_sync(CAM_FULL, s, o); if (lane >= o) s += t; }
    return s - v;
}

// kmul, kshift: p / k = (p * kmul) >> kshift for every 0 <= p < 2^31 (the host's round-up reciprocal of k)
__global__ void __launch_bounds__(1024) group_cluster_kernel(const int * __restrict__ ids, int npairs, int k, int E, int * __restrict__ xs,
                                                             int * __restrict__ yd, WorkItem * __restrict__ items, int * __restrict__ nitems,
                                                             int * __restrict__ err, unsigned long long kmul, int kshift) {
    extern __shared__ int gr_smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int nblk = (int)cluster.num_blocks(), blk = (int)cluster.block_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int * cells = gr_smem;                       // [E][GR_PITCH]: cell (e, w) = warp w's count of expert e, later its cursor (a scan walks a row conflict-free)
    int * mine = cells + E * GR_PITCH;           // [E]: this block's count per expert (read by the other blocks)
    int * first = mine + E;                      // [E]: where an expert's list starts
    int * ifirst = first + E;                    // [E]: where an expert's work items start
    int * total = ifirst + E;                    // [E]: pairs of an expert over all blocks
    int * before = total + E;                    // [E]: pairs of an expert in the blocks before this one
    int * wsum_ = before + E;                    // [3][32]: the expert scan's per-warp sums, then their prefixes; [96]: the number of items
    // this warp's run of pairs: `per` (a multiple of 32) consecutive pairs per warp, warps in (block, warp) order
    const int nw = nblk * GR_WARPS;
    const int per = ((npairs + nw - 1) / nw + 31) & ~31;
    const long lo = (long)(blk * GR_WARPS + warp) * per;
    const int steps = lo >= npairs ? 0 : (int)((min((long)npairs, lo + per) - lo + 31) >> 5);
    // the first GR_KEEP steps' ids are requested at once and stay in registers for the second pass
    int kept[GR_KEEP];
    bool bad = false;
#pragma unroll
    for (int q = 0; q < GR_KEEP; q++) {
        const long p = lo + 32 * q + lane;
        kept[q] = q < steps && p < npairs ? __ldg(ids + p) : -1;
    }
#pragma unroll
    for (int q = 0; q < GR_KEEP; q++)
        if (q < steps && lo + 32 * q + lane < npairs && (kept[q] < 0 || kept[q] >= E)) { bad = true; kept[q] = 0; }
    for (int i = tid; i < E * GR_PITCH; i += 1024) cells[i] = 0;
    __syncthreads();
    const unsigned below = (1u << lane) - 1u;
    int nbits = 1; while ((1 << nbits) <= E) nbits++;             // an expert + 1 (0: no pair) in nbits bits
    int * const col = cells + warp;              // + e GR_PITCH: this warp's cell of expert e
    auto later = [&](int s) {                    // the expert of this lane's pair in a step past the kept ones (-1: past the end), range-checked
        const long p = lo + 32 * s + lane;
        if (p >= npairs) return -1;
        int e = __ldg(ids + p);
        if (e < 0 || e >= E) { bad = true; e = 0; }
        return e;
    };
    unsigned keptsame[GR_KEEP];                  // (the kept steps' equal-lane masks serve both passes)
#pragma unroll
    for (int q = 0; q < GR_KEEP; q++)
        if (q < steps) {
            const int e = kept[q];
            const unsigned same = keptsame[q] = same_lanes((unsigned)(e + 1), nbits);
            if (e >= 0 && (same & below) == 0) col[e * GR_PITCH] += __popc(same);
            __syncwarp();
        }
    for (int s = GR_KEEP; s < steps; s++) {
        const int e = later(s);
        const unsigned same = same_lanes((unsigned)(e + 1), nbits);
        if (e >= 0 && (same & below) == 0) col[e * GR_PITCH] += __popc(same);
        __syncwarp();
    }
    if (__any_sync(CAM_FULL, bad) && lane == 0) atomicOr(err, 2);
    __syncthreads();
    for (int e = warp; e < E; e += GR_WARPS) {   // a warp adds an expert's 32 cells
        int c = cells[e * GR_PITCH + lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(CAM_FULL, c, o);
        if (lane == 0) mine[e] = c;
    }
    cluster.sync();
    // E <= 1024: thread e owns expert e for the scan over the experts
    int bef = 0, tot = 0;
    if (tid < E) {
        for (int b = 0; b < nblk; b++) {
            const int c = cluster.map_shared_rank(mine, b)[tid];
            tot += c; if (b < blk) bef += c;
        }
        total[tid] = tot; before[tid] = bef;
    }
    const int nit = (tot + ITEM_PAIRS - 1) / ITEM_PAIRS;
    const int ex_c = wscan_excl(tot, lane), ex_i = wscan_excl(nit, lane);
    if (lane == 31) { wsum_[warp] = ex_c + tot; wsum_[32 + warp] = ex_i + nit; }
    __syncthreads();
    if (warp == 0) {                             // the 32 warp sums' prefixes
        const int a = wsum_[lane], b = wsum_[32 + lane];
        const int pa = wscan_excl(a, lane), pb = wscan_excl(b, lane);
        wsum_[lane] = pa; wsum_[32 + lane] = pb;
        if (lane == 31) wsum_[96] = pb + b;
    }
    __syncthreads();
    if (tid < E) { first[tid] = wsum_[warp] + ex_c; ifirst[tid] = wsum_[32 + warp] + ex_i; }
    const int all_items = wsum_[96];
    if (blk == 0 && tid == 0) *nitems = all_items;
    __syncthreads();
    for (int e = warp; e < E; e += GR_WARPS) {   // an expert's cells become its warps' cursors: the list's start, the earlier blocks, the earlier warps
        const int c = cells[e * GR_PITCH + lane];
        cells[e * GR_PITCH + lane] = first[e] + before[e] + wscan_excl(c, lane);
    }
    __syncthreads();
    auto place = [&](int e, int s, unsigned same) {
        if (e >= 0) {
            const int p = (int)(lo + 32 * s + lane), at = col[e * GR_PITCH] + __popc(same & below);
            xs[at] = (int)(((unsigned long long)(unsigned)p * kmul) >> kshift); yd[at] = p;
        }
        __syncwarp();
        if (e >= 0 && (same & below) == 0) col[e * GR_PITCH] += __popc(same);
        __syncwarp();
    };
#pragma unroll
    for (int q = 0; q < GR_KEEP; q++)
        if (q < steps) place(kept[q], q, keptsame[q]);
    for (int s = GR_KEEP; s < steps; s++) {
        const long p = lo + 32 * s + lane;
        int e = -1;
        if (p < npairs) { e = __ldg(ids + p); if (e < 0 || e >= E) e = 0; }
        place(e, s, same_lanes((unsigned)(e + 1), nbits));
    }
    // the work items, spread over all threads of the cluster: item i belongs to the last expert whose items start at or before i
    for (int i = blk * 1024 + tid; i < all_items; i += nblk * 1024) {
        int a = 0, b = E - 1;
        while (a < b) { const int mid = (a + b + 1) >> 1; if (ifirst[mid] <= i) a = mid; else b = mid - 1; }
        const int j = i - ifirst[a];
        WorkItem it; it.expert = a; it.first = first[a] + j * ITEM_PAIRS; it.count = min(ITEM_PAIRS, total[a] - j * ITEM_PAIRS); it.zero = 0;
        items[i] = it;
    }
    cluster.sync();                              // (no block leaves while another may still read its counts)
}

}   // namespace

// q3p_router: kernels/q3m_prefill.hip:419-420 (n = grid.x); K a multiple of 128, 16-byte aligned rows
extern "C" int q3p_router(int n, const float * h, const float * Wr, int E, int K, float * logits, void * stream) {
    if (n < 0 || E < 1 || K < 128 || (K & 127) || !h || !Wr || !logits) return CAM_ERR_ARG;
    if (!cam_aligned16(h) || !cam_aligned16(Wr)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    if (n >= 64) {
        static unsigned long long allowed = 0;
        const size_t smem = (size_t)RT_STAGES * RT_STAGE_FLOATS * 4;                 // (72 KB: above the default limit)
        const cudaError_t e = cam_allow_smem(router_tile_kernel, smem, allowed);
        if (e != cudaSuccess) return (int)e;
        router_tile_kernel<<<dim3((n + RT_TOK - 1) / RT_TOK, (E + RT_EXP - 1) / RT_EXP), 256, smem, (cudaStream_t)stream>>>(h, Wr, E, K, logits, n);
    } else router_few_kernel<<<(E + 7) / 8, 256, 0, (cudaStream_t)stream>>>(h, Wr, E, K, logits, n);
    return (int)cudaGetLastError();
}
// q3p_topk: kernels/q3m_prefill.hip:440-441 (n = grid.x); E <= 128, k <= 32
extern "C" int q3p_topk(int n, const float * logits, int E, int k, float floor_, int * ids, float * wts, int * err, void * stream) {
    if (n < 0 || E < 1 || E > 128 || k < 1 || k > 32 || k > E || !logits || !ids || !wts || !err) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    topk_kernel<<<(n + 7) / 8, 256, 0, (cudaStream_t)stream>>>(logits, E, k, floor_, ids, wts, err, n);
    return (int)cudaGetLastError();
}
// pf_router: kernels/prefill_glue.hip:242-243 (T = grid.x); E <= 1024, k <= min(64, E)
extern "C" int pf_router(int T, const float * logits, int E, int k, float clamp, int * ids, float * wts, int * err, void * stream) {
    if (T < 0 || E < 1 || E > 1024 || k < 1 || k > 64 || k > E || !logits || !ids || !wts || !err) return CAM_ERR_ARG;
    if (T == 0) return CAM_OK;
    const dim3 grid((T + 7) / 8);
    cudaStream_t st = (cudaStream_t)stream;
    switch ((E + 255) / 256) {
        case 1: softmax_topk_rows_kernel<1><<<grid, 256, 0, st>>>(logits, E, k, clamp, ids, wts, err, T); break;
        case 2: softmax_topk_rows_kernel<2><<<grid, 256, 0, st>>>(logits, E, k, clamp, ids, wts, err, T); break;
        case 3: softmax_topk_rows_kernel<3><<<grid, 256, 0, st>>>(logits, E, k, clamp, ids, wts, err, T); break;
        default: softmax_topk_rows_kernel<4><<<grid, 256, 0, st>>>(logits, E, k, clamp, ids, wts, err, T); break;
    }
    return (int)cudaGetLastError();
}
// q3p_group: kernels/q3m_prefill.hip:490-492; items are { int e, off, cnt, pad }; E <= 1024
extern "C" int q3p_group(const int * ids, int npairs, int k, int E, int * xs, int * yd, void * items, int * nitems, int * err, void * stream) {
    if (npairs < 0 || k < 1 || E < 1 || E > 1024 || !ids || !xs || !yd || !items || !nitems || !err) return CAM_ERR_ARG;
    static unsigned long long allowed = 0;
    const size_t smem = ((size_t)(GR_PITCH + 5) * E + 128) * sizeof(int);             // (E = 1024: 152 KB)
    if (smem > 48 * 1024) { const cudaError_t e = cam_allow_smem(group_cluster_kernel, smem, allowed); if (e != cudaSuccess) return (int)e; }
    // p / k as a multiplication: kshift = 32 + ceil(log2 k), kmul = ceil(2^kshift / k): exact for every p below 2^32
    int l = 0; while ((1LL << l) < k) l++;
    const int kshift = 32 + l;
    const unsigned long long kmul = (unsigned long long)((((unsigned __int128)1 << kshift) + (unsigned)k - 1) / (unsigned)k);
    // A cluster of 16 (beyond the portable 8) where the device schedules one: asked once per device
    static int max16[64] = {};                                                         // 0: not asked, 1: no, 2: yes
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && max16[dev] == 0) {
        int ok = 1;
        if (cudaFuncSetAttribute(group_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t q = {};
            q.gridDim = dim3(16); q.blockDim = dim3(1024); q.dynamicSmemBytes = smem;
            cudaLaunchAttribute qa[1];
            qa[0].id = cudaLaunchAttributeClusterDimension; qa[0].val.clusterDim.x = 16; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
            q.attrs = qa; q.numAttrs = 1;
            int nclusters = 0;
            if (cudaOccupancyMaxActiveClusters(&nclusters, group_cluster_kernel, &q) == cudaSuccess && nclusters >= 1) ok = 2;
        }
        (void)cudaGetLastError();
        max16[dev] = ok;
    }
    const int cap = dev >= 0 && dev < 64 && max16[dev] == 2 && smem <= 48 * 1024 ? 16 : 8;
    int nblk = 1;
    while (nblk < cap && (long)nblk * 4096 < npairs) nblk *= 2;                       // 4 steps of 32 pairs per warp before the cluster grows
    if (const char * e = getenv("CAMINUS_B200_GROUP_BLOCKS")) { const int v = atoi(e); if (v == 1 || v == 2 || v == 4 || v == 8 || (v == 16 && cap == 16)) nblk = v; }      // (tuning)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nblk); cfg.blockDim = dim3(1024); cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = nblk; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, group_cluster_kernel, ids, npairs, k, E, xs, yd, (WorkItem *)items, nitems, err, kmul, kshift);
}
