// Tensor-parallel RMSNorm as ONE kernel: the hidden dimension is sharded over the ranks (one GPU each); a rank reduces its
// columns of a row to one fp32 sum of squares, writes it straight into every rank's exchange buffer over NVLink (plain peer
// stores), and normalises its columns once all ranks' partials of that row have arrived in its own buffer. The two-kernel form
// (cam_rms_partial_f16 -> all-reduce of [T] floats -> cam_rms_apply_f16, csrc/add_rms.cu) reads every row twice from HBM and pays a
// collective's launch between the kernels; here a warp keeps its rows in registers (the usual shard widths) or in shared memory from
// the sum of squares to the normalisation (rows too long for that are read a second time, a few rows later), and the exchange
// overlaps the arithmetic row by row. The reference has no counterpart (it replicates its norms,
// python/caminus/engine/q3moe_tp.py:18-20).
//
// Exchange buffer of a rank (the caller allocates it and maps every rank's into every process): 64-bit words
// [2 parities][world sources][cap rows], word = (tag << 32) | bits of the fp32 partial. The tag is the call's sequence number
// (never 0; the buffer starts zeroed), the same on every rank, so a word is valid exactly when its tag matches: no flags to
// reset, no fence between value and flag (one 8-byte store), and a call cannot mistake the previous call's words (parity = tag & 1
// alternates; a rank can be at most one call ahead of another, because it needs the other's partials of this call to finish).
// Row total = the partials added in rank order from 0.0f: the same bits on every rank.
//
// Every wait is bounded: a lane polls its source's word for at most CAM_TP_WAIT_NS of the global timer; on expiry the warp ORs 1
// into *status and stops taking rows (its peers' waits for this rank's later rows expire the same way). Nothing is left in flight:
// the kernel uses plain loads and stores only. Ranks run on different GPUs; this kernel must never be launched for two ranks on
// one GPU (the second would wait for a kernel that cannot start).
#include "cam_common.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace {

constexpr unsigned long long CAM_TP_WAIT_NS = 2000000000ull;      // 2 s: the default limit of a wait (CAMINUS_B200_TP_WAIT_MS overrides it)

CAM_DEV void st_sys_u64(unsigned long long * p, unsigned long long v) { asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }
CAM_DEV unsigned long long ld_sys_u64(const unsigned long long * p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
CAM_DEV unsigned long long global_ns() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }

CAM_DEV void widen8(const uint4 v, float (&f)[8]) {
    const float2 a = h2_to_f2(v.x), b = h2_to_f2(v.y), c = h2_to_f2(v.z), e = h2_to_f2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = e.x; f[7] = e.y;
}
// DEPTH: rows between a warp's partial of a row and its normalisation of that row (the exchange's round trip hides behind them)
template <int DEPTH>
__global__ void __launch_bounds__(128) tp_rms_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d, const float * __restrict__ nw, float eps,
                                                     uint16_t * __restrict__ h16, int Ns, int Nfull, int n, unsigned long long * const * __restrict__ peers,
                                                     int rank, int world, int cap, unsigned tag, int * status, unsigned long long wait_ns) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nch = (Ns + 255) >> 8;                                     // 16-byte chunks per lane and row (the last may be short)
    const int t0 = blockIdx.x * 4 + warp, stride = gridDim.x * 4;
    const size_t slot0 = (size_t)(tag & 1u) * world * cap;               // this call's half of every buffer
    unsigned long long * const mine = lane < world ? peers[lane] + slot0 + (size_t)rank * cap : nullptr;   // where lane r writes: rank r's buffer, source = this rank
    const unsigned long long * const from = lane < world ? peers[rank] + slot0 + (size_t)lane * cap : nullptr;   // where lane r polls: own buffer, source r
    const int rows = t0 < n ? (n - t0 + stride - 1) / stride : 0;       // this warp's rows t0, t0 + stride, ..
    bool dead = false;
    for (int k = 0; k < rows + DEPTH; k++) {
        if (k < rows && !dead) {                                         // ---- this shard's sum of squares of row t, sent to every rank
            const int t = t0 + k * stride;
            const uint16_t * xr = x + (size_t)t * Ns, * dr = d ? d + (size_t)t * Ns : nullptr;
            float a[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int m = 0; m < nch; m++) {
                const int i = 8 * lane + 256 * m;
                if (i >= Ns) break;
                float xs[8];
                widen8(ld128(xr + i), xs);
                if (dr) {
                    float dv[8];
                    widen8(ldg128(dr + i), dv);
#pragma unroll
                    for (int c = 0; c < 8; c++) xs[c] = fadd(xs[c], dv[c]);
                }
#pragma unroll
                for (int c = 0; c < 8; c++) a[c] = ffma(xs[c], xs[c], a[c]);
            }
            const float part = ref_total_f16(a, lane);      // (the bits of cam_rms_partial_f16)
            if (mine) st_sys_u64(mine + t, ((unsigned long long)tag << 32) | __float_as_uint(part));
        }
        const int kd = k - DEPTH;
        if (kd >= 0 && kd < rows && !dead) {                             // ---- row t of DEPTH rows ago: gather the partials, normalise
            const int t = t0 + kd * stride;
            float part = 0.0f;
            bool late = false;
            if (from) {
                unsigned long long w = ld_sys_u64(from + t);
                if ((unsigned)(w >> 32) != tag) {
                    const unsigned long long start = global_ns();
                    do {
                        __nanosleep(64);
                        w = ld_sys_u64(from + t);
                        late = (unsigned)(w >> 32) != tag;
                    } while (late && global_ns() - start < wait_ns);
                }
                part = __uint_as_float((unsigned)w);
            }
            if (__any_sync(CAM_FULL, late)) {                            // a source never arrived: report, take no more rows
                if (lane == 0) atomicOr(status, 1);
                dead = true;
                continue;
            }
            float tot = 0.0f;
            for (int r = 0; r < world; r++) tot = fadd(tot, __shfl_sync(CAM_FULL, part, r));
            const float scale = cam_rsqrt(fadd(fdiv(tot, (float)Nfull), eps));
            uint16_t * xr = x + (size_t)t * Ns, * hr = h16 + (size_t)t * Ns;
            const uint16_t * dr = d ? d + (size_t)t * Ns : nullptr;
#pragma unroll 2
            for (int m = 0; m < nch; m++) {
                const int i = 8 * lane + 256 * m;
                if (i >= Ns) break;
                float xs[8];
                widen8(ld128(xr + i), xs);
                if (dr) {
                    float dv[8];
                    widen8(ldg128(dr + i), dv);
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
}

// The staged form: a warp keeps LA + DEPTH + 1 rows of its shard (x and d as stored) in its own slice of shared memory, brought in with
// cp.async (a lane copies exactly the 16-byte chunks it reads back, so its own copy groups are the only synchronisation). Per step
// k of a warp: row k + LA is requested; row k has landed: its sum of squares is formed and sent to every rank; row k - DEPTH, whose
// partials have had DEPTH rows of time to cross NVLink, is gathered, normalised from shared memory and stored. No row is read from
// HBM twice. A warp's wait (for its row, for the partials) is covered by the other warps of the multiprocessor: the launcher
// trades slots per warp for resident warps.
// NCHT: the 16-byte chunks per lane and row fixed at compile time (0: computed from Ns): the chunk loops unroll, nothing is counted
template <int LA, int DEPTH, int NCHT = 0>
__global__ void __launch_bounds__(256) tp_rms_staged_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d, const float * __restrict__ nw, float eps,
                                                            uint16_t * __restrict__ h16, int Ns, int Nfull, int n, unsigned long long * const * __restrict__ peers,
                                                            int rank, int world, int cap, unsigned tag, int * status, int warps, unsigned long long wait_ns) {
    constexpr int S = LA + DEPTH + 1;
    extern __shared__ __align__(16) unsigned char tp_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nch = NCHT ? NCHT : (Ns + 255) >> 8;
    const size_t half_bytes = (size_t)nch * 512, row_bytes = (d ? 2 : 1) * half_bytes;
    unsigned char * const slots = tp_smem + (size_t)warp * S * row_bytes;
    const int t0 = blockIdx.x * warps + warp, stride = gridDim.x * warps;
    const size_t slot0 = (size_t)(tag & 1u) * world * cap;
    unsigned long long * const mine = lane < world ? peers[lane] + slot0 + (size_t)rank * cap : nullptr;
    const unsigned long long * const from = lane < world ? peers[rank] + slot0 + (size_t)lane * cap : nullptr;
    const int rows = t0 < n ? (n - t0 + stride - 1) / stride : 0;

    auto request = [&](int k) {                                          // row k of this warp into slot k % S (one copy group per call)
        if (k < rows) {
            unsigned char * sx = slots + (size_t)(k % S) * row_bytes;
            const size_t at = (size_t)(t0 + k * stride) * Ns + 8 * lane;
#pragma unroll
            for (int m = 0; m < (NCHT ? NCHT : nch); m++)
                if (8 * lane + 256 * m < Ns) {
                    cp_async16(sx + (size_t)(m * 32 + lane) * 16, x + at + 256 * m);
                    if (d) cp_async16(sx + half_bytes + (size_t)(m * 32 + lane) * 16, d + at + 256 * m);
                }
        }
        cp_async_commit();
    };
    auto row_values = [&](const unsigned char * sx, int m, f32x2 (&xs)[4]) {   // xs = x + d of this lane's chunk m, two values per register pair
        float xv[8];
        widen8(*reinterpret_cast<const uint4 *>(sx + (size_t)(m * 32 + lane) * 16), xv);
#pragma unroll
        for (int c = 0; c < 4; c++) xs[c] = pk2(xv[2 * c], xv[2 * c + 1]);
        if (d) {
            float dv[8];
            widen8(*reinterpret_cast<const uint4 *>(sx + half_bytes + (size_t)(m * 32 + lane) * 16), dv);
#pragma unroll
            for (int c = 0; c < 4; c++) xs[c] = add2(xs[c], pk2(dv[2 * c], dv[2 * c + 1]));
        }
    };

#pragma unroll
    for (int k = 0; k < LA; k++) request(k);
    bool dead = false;
    for (int k = 0; k < rows + DEPTH; k++) {
        request(k + LA);                                                 // (its slot held row k - DEPTH - 1, stored a step ago)
        cp_async_wait<LA>();                                             // row k has landed (later rows may still fly)
        if (k < rows && !dead) {                                         // ---- row k: this shard's sum of squares, sent to every rank
            const unsigned char * sx = slots + (size_t)(k % S) * row_bytes;
            f32x2 a2[4] = {pk2(0.0f, 0.0f), pk2(0.0f, 0.0f), pk2(0.0f, 0.0f), pk2(0.0f, 0.0f)};
#pragma unroll
            for (int m = 0; m < (NCHT ? NCHT : nch); m++) {
                if (8 * lane + 256 * m < Ns) {
                    f32x2 xs[4];
                    row_values(sx, m, xs);
#pragma unroll
                    for (int c = 0; c < 4; c++) a2[c] = fma2(xs[c], xs[c], a2[c]);
                }
            }
            float a[8];
#pragma unroll
            for (int c = 0; c < 4; c++) { a[2 * c] = lo2(a2[c]); a[2 * c + 1] = hi2(a2[c]); }
            const float part = ref_total_f16(a, lane);                   // (the bits of cam_rms_partial_f16)
            if (mine) st_sys_u64(mine + (t0 + k * stride), ((unsigned long long)tag << 32) | __float_as_uint(part));
        }
        const int kd = k - DEPTH;
        if (kd >= 0 && kd < rows && !dead) {                             // ---- row kd: gather the partials, normalise, store
            const int t = t0 + kd * stride;
            float part = 0.0f;
            bool late = false;
            if (from) {
                unsigned long long w = ld_sys_u64(from + t);
                if ((unsigned)(w >> 32) != tag) {
                    const unsigned long long start = global_ns();
                    do {
                        __nanosleep(64);
                        w = ld_sys_u64(from + t);
                        late = (unsigned)(w >> 32) != tag;
                    } while (late && global_ns() - start < wait_ns);
                }
                part = __uint_as_float((unsigned)w);
            }
            if (__any_sync(CAM_FULL, late)) {                            // a source never arrived: report, take no more rows
                if (lane == 0) atomicOr(status, 1);
                dead = true;
                continue;
            }
            float tot = 0.0f;
            for (int r = 0; r < world; r++) tot = fadd(tot, __shfl_sync(CAM_FULL, part, r));
            const float scale = cam_rsqrt(fadd(fdiv(tot, (float)Nfull), eps));
            const unsigned char * sx = slots + (size_t)(kd % S) * row_bytes;
            const size_t at = (size_t)t * Ns + 8 * lane;
            const f32x2 s2 = pk2(scale, scale);
#pragma unroll
            for (int m = 0; m < (NCHT ? NCHT : nch); m++) {
                const int i = 8 * lane + 256 * m;
                if (i < Ns) {
                    f32x2 xs[4];
                    row_values(sx, m, xs);
                    if (d) st128(x + at + 256 * m, make_uint4(f2_to_h2(lo2(xs[0]), hi2(xs[0])), f2_to_h2(lo2(xs[1]), hi2(xs[1])), f2_to_h2(lo2(xs[2]), hi2(xs[2])),
                                                              f2_to_h2(lo2(xs[3]), hi2(xs[3]))));
                    const float4 w0 = __ldg(reinterpret_cast<const float4 *>(nw + i)), w1 = __ldg(reinterpret_cast<const float4 *>(nw + i + 4));
                    const f32x2 v0 = mul2(mul2(xs[0], s2), pk2(w0.x, w0.y)), v1 = mul2(mul2(xs[1], s2), pk2(w0.z, w0.w));
                    const f32x2 v2 = mul2(mul2(xs[2], s2), pk2(w1.x, w1.y)), v3 = mul2(mul2(xs[3], s2), pk2(w1.z, w1.w));
                    st128_stream(h16 + at + 256 * m, make_uint4(f2_to_h2(lo2(v0), hi2(v0)), f2_to_h2(lo2(v1), hi2(v1)), f2_to_h2(lo2(v2), hi2(v2)), f2_to_h2(lo2(v3), hi2(v3))));
                }
            }
        }
    }
    cp_async_wait<0>();
}

// The form for the usual shards (Ns = G x 8 x CH with G = 16 or 32 lanes per row: 512 / 640 columns on a half-warp, two rows per warp;
// 1024 / 1280 / 2048 / 2560 on a warp): every lane of every instruction is busy, nothing is counted or tested per chunk, and the row is
// converted once. Element of lane l, chunk q, value c: G = 32: 256 q + 8 l + c (thread 8 l + c of the reference's 256, its j = q);
// G = 16, lane h of the half-warp: 128 q + 8 h + c (thread 128 (q & 1) + 8 h + c, j = q >> 1).
template <int G> CAM_DEV float tp_row_total(float (&a)[2][8], int lane) {
    // a[g][c]: thread 128 g + 8 h + c (G = 16; g = 0 only for G = 32, thread 8 l + c). Wave butterfly 16, 8 = lanes ^ 2, ^ 1; 4, 2, 1 inside
    // the lane; then the 8 wave sums in order: wave w = thread >> 5 sits in lane 4 (w & 3) of the row's lanes (G = 16: its g = w >> 2)
    constexpr int NG = G == 16 ? 2 : 1;
    float P[NG];
#pragma unroll
    for (int g = 0; g < NG; g++) {
#pragma unroll
        for (int o = 2; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < 8; k++) a[g][k] = fadd(a[g][k], __shfl_xor_sync(CAM_FULL, a[g][k], o));
        const float u0 = fadd(a[g][0], a[g][4]), u1 = fadd(a[g][1], a[g][5]), u2 = fadd(a[g][2], a[g][6]), u3 = fadd(a[g][3], a[g][7]);
        P[g] = fadd(fadd(u0, u2), fadd(u1, u3));
    }
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) tot = fadd(tot, G == 16 ? __shfl_sync(CAM_FULL, P[(w >> 2) % NG], 4 * (w & 3), 16) : __shfl_sync(CAM_FULL, P[0], 4 * w));
    return tot;
}

// The next block number of this call, in the order blocks actually start: word = (tag << 32) | blocks started. The first block of a call
// finds another tag there and replaces it. With numbers handed out this way the lowest unfinished number on every rank belongs to a
// running block, so the rank that is behind always holds the block whose partials the others wait for, whatever order the hardware
// starts blocks in (each block sends its partials before it waits).
CAM_DEV unsigned tp_take_number(unsigned long long * counter, unsigned tag) {
    for (;;) {
        const unsigned long long w = *reinterpret_cast<volatile unsigned long long *>(counter);
        if ((unsigned)(w >> 32) == tag) return (unsigned)atomicAdd(counter, 1ull);
        if (atomicCAS(counter, w, ((unsigned long long)tag << 32) | 1ull) == w) return 0u;
    }
}

// Nothing is parked: a warp loads its row(s) straight into registers, stores fp16(x + d), sends the partial, waits for the others' and
// normalises from the fp32 sums it still holds. Blocks of four warps, a block per 4 or 8 rows, so more blocks than are resident (a finished
// block's successor starts with its loads at once, and the blocks' load, arithmetic and store phases drift apart instead of running in
// step): the shape of add_rms_f16_reg_kernel. 65536 rows of 640 columns on one rank: 57 us (0.89); the pipelined kernels that parked rows
// in shared memory on resident, looping blocks: 63-68 us, and this kernel itself on resident blocks that loop: 63.8 us.
template <int G, int CH>
__global__ void __launch_bounds__(128) tp_rms_direct_kernel(uint16_t * __restrict__ x, const uint16_t * __restrict__ d, const float * __restrict__ nw, float eps,
                                                            uint16_t * __restrict__ h16, int Nfull, int n, unsigned long long * const * __restrict__ peers,
                                                            int rank, int world, int cap, unsigned tag, int * status, unsigned long long wait_ns) {
    constexpr int RPW = 32 / G, Ns = G * 8 * CH;
    __shared__ unsigned number;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, h = lane & (G - 1), sub = lane / G;
    if (threadIdx.x == 0) number = tp_take_number(peers[rank] + (size_t)2 * world * cap, tag);      // (the word after this rank's exchange words)
    __syncthreads();
    const size_t slot0 = (size_t)(tag & 1u) * world * cap;
    unsigned long long * const mine = h < world ? peers[h] + slot0 + (size_t)rank * cap : nullptr;
    const unsigned long long * const from = h < world ? peers[rank] + slot0 + (size_t)h * cap : nullptr;
    {                                                                    // one block = 4 RPW rows (the grid covers n)
        const int first = ((int)number * 4 + warp) * RPW;                // (warp-uniform)
        if (first >= n) return;
        const int t = first + sub;
        const bool on = t < n;
        const size_t at = (size_t)(on ? t : 0) * Ns + 8 * h;
        uint4 xv[CH], dv[CH];
#pragma unroll
        for (int q = 0; q < CH; q++) {
            xv[q] = on ? ld128(x + at + G * 8 * q) : make_uint4(0u, 0u, 0u, 0u);
            dv[q] = on && d ? ldg128(d + at + G * 8 * q) : make_uint4(0u, 0u, 0u, 0u);
        }
        f32x2 xs[CH][4];
        float a[2][8];
#pragma unroll
        for (int c = 0; c < 8; c++) a[0][c] = a[1][c] = 0.0f;
#pragma unroll
        for (int q = 0; q < CH; q++) {
            const uint32_t xw[4] = {xv[q].x, xv[q].y, xv[q].z, xv[q].w}, dw[4] = {dv[q].x, dv[q].y, dv[q].z, dv[q].w};
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float2 xf = h2_to_f2(xw[c]);
                xs[q][c] = pk2(xf.x, xf.y);
                if (d) { const float2 df = h2_to_f2(dw[c]); xs[q][c] = add2(xs[q][c], pk2(df.x, df.y)); }
            }
            if (d && on) st128(x + at + G * 8 * q, make_uint4(f2_to_h2(lo2(xs[q][0]), hi2(xs[q][0])), f2_to_h2(lo2(xs[q][1]), hi2(xs[q][1])),
                                                              f2_to_h2(lo2(xs[q][2]), hi2(xs[q][2])), f2_to_h2(lo2(xs[q][3]), hi2(xs[q][3]))));
            constexpr int NGq = G == 16 ? 2 : 1;
            float (&ag)[8] = a[q % NGq];
#pragma unroll
            for (int c = 0; c < 4; c++) { ag[2 * c] = ffma(lo2(xs[q][c]), lo2(xs[q][c]), ag[2 * c]); ag[2 * c + 1] = ffma(hi2(xs[q][c]), hi2(xs[q][c]), ag[2 * c + 1]); }
        }
        const float own = tp_row_total<G>(a, lane);                      // (the bits of cam_rms_partial_f16)
        if (mine && on) st_sys_u64(mine + t, ((unsigned long long)tag << 32) | __float_as_uint(own));
        float part = 0.0f;
        bool late = false;
        if (from && on) {
            if (h == rank) part = own;                                   // (this rank's own partial needs no trip through memory)
            else {
                unsigned long long w = ld_sys_u64(from + t);
                if ((unsigned)(w >> 32) != tag && (*reinterpret_cast<volatile int *>(status) & 1)) late = true;      // (a wait ran out already: no block waits again)
                else if ((unsigned)(w >> 32) != tag) {
                    const unsigned long long start = global_ns();
                    do {
                        __nanosleep(64);
                        w = ld_sys_u64(from + t);
                        late = (unsigned)(w >> 32) != tag;
                    } while (late && global_ns() - start < wait_ns);
                }
                part = __uint_as_float((unsigned)w);
            }
        }
        if (__any_sync(CAM_FULL, late)) {                                // a source never arrived: report, take no more rows
            if (lane == 0) atomicOr(status, 1);
            return;
        }
        float tot = 0.0f;
        for (int r = 0; r < world; r++) tot = fadd(tot, __shfl_sync(CAM_FULL, part, r, G));
        const float scale = cam_rsqrt(fadd(fdiv(tot, (float)Nfull), eps));
        const f32x2 s2 = pk2(scale, scale);
#pragma unroll
        for (int q = 0; q < CH; q++) {
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(nw + 8 * h + G * 8 * q)), w1 = __ldg(reinterpret_cast<const float4 *>(nw + 8 * h + G * 8 * q + 4));
            const f32x2 v0 = mul2(mul2(xs[q][0], s2), pk2(w0.x, w0.y)), v1 = mul2(mul2(xs[q][1], s2), pk2(w0.z, w0.w));
            const f32x2 v2 = mul2(mul2(xs[q][2], s2), pk2(w1.x, w1.y)), v3 = mul2(mul2(xs[q][3], s2), pk2(w1.z, w1.w));
            if (on) st128_stream(h16 + at + G * 8 * q, make_uint4(f2_to_h2(lo2(v0), hi2(v0)), f2_to_h2(lo2(v1), hi2(v1)), f2_to_h2(lo2(v2), hi2(v2)), f2_to_h2(lo2(v3), hi2(v3))));
        }
    }
}

template <int G, int CH>
int launch_tp_direct(int n, void * x, const void * d, const float * nw, float eps, void * h16, int Nfull, const void * peers, int rank, int world, int cap,
                     unsigned tag, int * status, unsigned long long wait_ns, cudaStream_t stream) {
    const int rpb = 4 * (32 / G);
    // (Measured on two GPUs and not kept: the rows in chunks that fit the second-level cache, a first pass over a chunk sending the partials and a
    // second one, from the cache, normalising, so that no block waits with a row in its registers: 79 us against 64 us at shards of 640.)
    // (Measured on eight GPUs and not kept either: a block's partial sums gathered in shared memory and sent by its first threads, 64 contiguous
    // bytes per peer instead of a 16-byte piece per warp and peer: 71.9-72.2 us against 71.3 us at shards of 640; on two GPUs 65.0 against 62.9.)
    // a block per 4 or 8 rows, so more blocks than are resident: 56.0 us against 63.8 us for resident blocks that loop (65536 rows of 640, one rank)
    const int grid = (n + rpb - 1) / rpb;
    tp_rms_direct_kernel<G, CH><<<grid, 128, 0, stream>>>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, Nfull, n,
                                                          (unsigned long long * const *)peers, rank, world, cap, tag, status, wait_ns);
    return (int)cudaGetLastError();
}

template <int LA, int DEPTH, int NCHT = 0>
int launch_tp_staged(int warps, size_t smem, int n, void * x, const void * d, const float * nw, float eps, void * h16, int Ns, int Nfull, const void * peers,
                     int rank, int world, int cap, unsigned tag, int * status, unsigned long long wait_ns, cudaStream_t stream) {
    static unsigned long long allowed = 0;
    const cudaError_t e = cam_allow_smem(tp_rms_staged_kernel<LA, DEPTH, NCHT>, 227 * 1024, allowed);
    if (e != cudaSuccess) return (int)e;
    const int grid = cam_resident_grid(tp_rms_staged_kernel<LA, DEPTH, NCHT>, warps * 32, smem, ((long)n + warps - 1) / warps);
    tp_rms_staged_kernel<LA, DEPTH, NCHT><<<grid, warps * 32, smem, stream>>>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, Ns, Nfull, n,
                                                                        (unsigned long long * const *)peers, rank, world, cap, tag, status, warps, wait_ns);
    return (int)cudaGetLastError();
}

}   // namespace

// cam_tp_rms_words: 64-bit words of one rank's exchange buffer for up to cap rows per call (the caller allocates them zeroed):
// [2 parities][world sources][cap rows] and 8 words of the library's own
extern "C" int cam_tp_rms_words(int cap, int world) {
    const long w = 2L * world * cap + 8;             // (+ 8: the word after the exchange words counts a call's started blocks)
    return cap < 1 || world < 1 || world > 32 || w > 0x7fffffffL ? CAM_ERR_ARG : (int)w;
}

// cam_tp_rms_norm_f16: x [n][Ns] fp16 = this rank's columns (updated in place to fp16(x + d) when d is given), d fp16 (nullable),
// nw fp32 [Ns] = this rank's weights, h16 fp16 [n][Ns] out; Nfull = the row length over all ranks. peers: device array of `world`
// pointers, entry r = rank r's exchange buffer as mapped in this process (entry `rank` = this rank's own), each
// cam_tp_rms_words(cap, world) words; n <= cap (CAM_ERR_CAPACITY beyond). tag: the call's sequence number, not 0, the same on
// every rank, consecutive LAUNCHES differing in parity (1, 2, 3, ..: a call with n = 0 launches nothing and must not use one up).
// status: an int32 word in this rank's memory; bit 0 is set when a wait ran out (some rank did not take part, or not with the same n
// and tag; the limit is 2 s, or CAMINUS_B200_TP_WAIT_MS milliseconds). The call's rows are then partly updated: a row whose partial was
// sent may hold x = fp16(x + d) already, the rows normalised before the wait ran out hold their h16 too, the others are untouched, so a
// retry needs x restored from a copy.
// Every rank must make the matching call; no rank's call may share a GPU with another's. Ns a multiple of 8, world <= 32.
extern "C" int cam_tp_rms_norm_f16(int n, void * x, const void * d, const float * nw, float eps, void * h16, int Ns, int Nfull,
                                   const void * peers, int rank, int world, int cap, unsigned tag, int * status, void * stream) {
    if (n < 0 || Ns < 8 || (Ns & 7) || Nfull < Ns || world < 1 || world > 32 || rank < 0 || rank >= world || cap < 1 || tag == 0 || !x || !nw || !h16 ||
        !peers || !status) return CAM_ERR_ARG;
    if (n > cap) return CAM_ERR_CAPACITY;
    if (!cam_aligned16(x) || (d && !cam_aligned16(d)) || !cam_aligned16(nw) || !cam_aligned16(h16) || (reinterpret_cast<uintptr_t>(peers) & 7u) ||
        (reinterpret_cast<uintptr_t>(status) & 3u)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;                      // (the caller must not advance its tag for such a call: nothing was stamped with it)
    cudaStream_t st = (cudaStream_t)stream;
    unsigned long long wait_ns = CAM_TP_WAIT_NS;    // CAMINUS_B200_TP_WAIT_MS: the limit of a wait in milliseconds (1 .. 600000)
    if (const char * e = getenv("CAMINUS_B200_TP_WAIT_MS")) { const long ms = atol(e); if (ms >= 1 && ms <= 600000) wait_ns = (unsigned long long)ms * 1000000ull; }
    if (world <= 16 && !getenv("CAMINUS_B200_TP_CFG")) {                // the usual shards: rows in registers (a row on 16 or 32 lanes, chunks counted at compile time)
#define CAM_TP_DIRECT(GV, CHV) return launch_tp_direct<GV, CHV>(n, x, d, nw, eps, h16, Nfull, peers, rank, world, cap, tag, status, wait_ns, st);
        switch (Ns) {
            case 512: CAM_TP_DIRECT(16, 4) case 640: CAM_TP_DIRECT(16, 5) case 1024: CAM_TP_DIRECT(32, 4) case 1280: CAM_TP_DIRECT(32, 5)
            case 2048: CAM_TP_DIRECT(32, 8) case 2560: CAM_TP_DIRECT(32, 10)
            default: break;
        }
#undef CAM_TP_DIRECT
    }
    // Other shard widths: rows staged in shared memory on resident blocks that loop. Measured on B200 (T = 65536, shards of 640 / 1280 / 2560
    // columns, before the kernel above took those): resident warps matter more than rows in flight per warp: two slots per warp (one row
    // waiting for its partials while the next is loaded and reduced) where that still leaves 20 warps per multiprocessor, else one slot.
    // CAMINUS_B200_TP_CFG="slots,warps" overrides (tuning, and it keeps the usual shards on this kernel too).
    {
        const size_t row_bytes = (size_t)(d ? 2 : 1) * ((Ns + 255) >> 8) * 512, budget = 224 * 1024;
        int slots = 2 * 20 * row_bytes <= budget ? 2 : 1, warps = 8;
        if (const char * e = getenv("CAMINUS_B200_TP_CFG")) {
            int sl = 0, wp = 0;
            if (sscanf(e, "%d,%d", &sl, &wp) == 2 && sl >= 1 && sl <= 4 && wp >= 1 && wp <= 8) { slots = sl; warps = wp; }
        }
        while (warps > 1 && (size_t)slots * warps * row_bytes > budget) warps--;
        const size_t smem = (size_t)slots * warps * row_bytes;
        if (smem <= budget) {
#define CAM_TP_STAGED(LAV, DV) return launch_tp_staged<LAV, DV>(warps, smem, n, x, d, nw, eps, h16, Ns, Nfull, peers, rank, world, cap, tag, status, wait_ns, st);
#define CAM_TP_FIXED(LAV, DV, NCHV) return launch_tp_staged<LAV, DV, NCHV>(warps, smem, n, x, d, nw, eps, h16, Ns, Nfull, peers, rank, world, cap, tag, status, wait_ns, st);
            // the usual shards (5120 or 4096 columns over 2, 4 or 8 ranks): the chunk count is a compile-time constant
            const int nch_ = (Ns + 255) >> 8;
            if (slots == 2) { switch (nch_) { case 2: CAM_TP_FIXED(0, 1, 2) case 3: CAM_TP_FIXED(0, 1, 3) case 4: CAM_TP_FIXED(0, 1, 4) case 5: CAM_TP_FIXED(0, 1, 5) default: break; } }
            if (slots == 1) { switch (nch_) { case 8: CAM_TP_FIXED(0, 0, 8) case 10: CAM_TP_FIXED(0, 0, 10) default: break; } }
            switch (slots) {
                case 1: CAM_TP_STAGED(0, 0)
                case 2: CAM_TP_STAGED(0, 1)
                case 3: CAM_TP_STAGED(1, 1)
                default: CAM_TP_STAGED(1, 2)
            }
#undef CAM_TP_STAGED
#undef CAM_TP_FIXED
        }
    }
    // longer rows: two passes over the row, four rows apart
    const int grid = cam_resident_grid(tp_rms_kernel<4>, 128, 0, ((long)n + 3) / 4);
    tp_rms_kernel<4><<<grid, 128, 0, st>>>((uint16_t *)x, (const uint16_t *)d, nw, eps, (uint16_t *)h16, Ns, Nfull, n,
                                           (unsigned long long * const *)peers, rank, world, cap, tag, status, wait_ns);
    return (int)cudaGetLastError();
}

// cam_ipc_open: maps an allocation another process exported (the 64 bytes of its cudaIpcMemHandle_t) into the current device's
// address space, enabling peer access to the exporting device when it is another one (kernels of the current device can then
// load and store there over NVLink). *base = the start of that allocation. cam_ipc_close unmaps it. Nothing is allocated.
extern "C" int cam_ipc_open(const void * handle64, void ** base) {
    if (!handle64 || !base) return CAM_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return (int)cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int cam_ipc_close(void * base) { return base ? (int)cudaIpcCloseMemHandle(base) : CAM_ERR_ARG; }
