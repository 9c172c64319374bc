// The IQ4 row gathers of the prefill's host feed (the reference's embd_rows_iq4xs and ple_rows_iq4nl, kernels/prefill_feed.hip:24-54;
// siblings of the Q4_K embedding gather): bitwise the host decoders (python/caminus/own_dequant.py iq4_xs; gguf-py).
// y = (d * (ls - 32)) * kvalue (IQ4_XS) / d * kvalue (IQ4_NL): lone products, rounded one by one. The 16 kvalues are ggml's IQ4_NL
// codebook, part of the format's definition. An index outside its table is clamped before the read and reported in *err.
// Mapping: a block per row, looping over rows; a thread takes four consecutive bytes of a 32-value sub-block (one 32-bit load) and
// writes the eight outputs they hold: values j .. j + 3 from the low nibbles, 16 + j .. 16 + j + 3 from the high ones (two 16-byte
// stores). The codebook sits in shared memory (16 words in 16 banks: any mix of indices is served in one pass; from constant
// memory, lanes with different indices are served one after another). Tables that are not 8-byte (IQ4_XS) / 2-byte (IQ4_NL)
// aligned take the byte-wise kernels.
#include "cam_common.cuh"

#include <cstdlib>

namespace {

__constant__ float kIQ4NL[16] = {-127.f, -104.f, -83.f, -65.f, -49.f, -35.f, -22.f, -10.f, 1.f, 13.f, 25.f, 38.f, 53.f, 69.f, 89.f, 113.f};

CAM_DEV float f16_at(const uint8_t * p) { return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8)))); }

__global__ void __launch_bounds__(256) embd_rows_iq4xs_bytes_kernel(const uint8_t * __restrict__ table, const int * __restrict__ tok, int nvocab, int n, int nblk,
                                                              float * __restrict__ out, int * err) {
    const int D4 = nblk * 64; const long total = (long)n * D4;
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long)gridDim.x * 256) {
        const int p = (int)(i / D4), k = (int)(i - (long)p * D4) * 4, bl = k >> 8, w = k & 255, ib = w >> 5, j = w & 31;
        int t = __ldg(tok + p);
        if (t < 0 || t >= nvocab) { atomicOr(err, 2); t = t < 0 ? 0 : nvocab - 1; }
        const uint8_t * b = table + (size_t)t * (size_t)(nblk * 136) + (size_t)bl * 136;
        const int sh = b[2] | (b[3] << 8), sl = b[4 + (ib >> 1)];
        const int ls = ((sl >> ((ib & 1) * 4)) & 15) | (((sh >> (2 * ib)) & 3) << 4);
        const float dl = fmul(f16_at(b), (float)(ls - 32));
        const uint8_t * qp = b + 8 + 16 * ib + (j & 15);
        const int hi = j < 16 ? 0 : 4;
        float4 y;
        y.x = fmul(dl, kIQ4NL[(qp[0] >> hi) & 15]); y.y = fmul(dl, kIQ4NL[(qp[1] >> hi) & 15]);
        y.z = fmul(dl, kIQ4NL[(qp[2] >> hi) & 15]); y.w = fmul(dl, kIQ4NL[(qp[3] >> hi) & 15]);
        __stcs(reinterpret_cast<float4 *>(out) + i, y);
    }
}

__global__ void __launch_bounds__(256) ple_rows_iq4nl_bytes_kernel(const uint8_t * __restrict__ raw, const int * __restrict__ inv, int nuniq, int nrows, int bpr,
                                                             float * __restrict__ out, int * err) {
    const int hd4 = bpr * 8; const long total = (long)nrows * hd4;
    for (long i = (long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long)gridDim.x * 256) {
        const int r = (int)(i / hd4), k = (int)(i - (long)r * hd4) * 4, b = k >> 5, j = k & 31;
        int u = __ldg(inv + r);
        if (u < 0 || u >= nuniq) { atomicOr(err, 1); u = u < 0 ? 0 : nuniq - 1; }
        const uint8_t * blk = raw + (size_t)u * (size_t)(bpr * 18) + (size_t)b * 18;
        const float d = f16_at(blk);
        const uint8_t * qp = blk + 2 + (j & 15);
        const int hi = j < 16 ? 0 : 4;
        float4 y;
        y.x = fmul(d, kIQ4NL[(qp[0] >> hi) & 15]); y.y = fmul(d, kIQ4NL[(qp[1] >> hi) & 15]);
        y.z = fmul(d, kIQ4NL[(qp[2] >> hi) & 15]); y.w = fmul(d, kIQ4NL[(qp[3] >> hi) & 15]);
        __stcs(reinterpret_cast<float4 *>(out) + i, y);
    }
}

CAM_DEV void iq4_store8(float * o, const float * kv, uint32_t w, float dl) {
    float4 lo, hi;
    lo.x = fmul(dl, kv[w & 15]); lo.y = fmul(dl, kv[(w >> 8) & 15]); lo.z = fmul(dl, kv[(w >> 16) & 15]); lo.w = fmul(dl, kv[(w >> 24) & 15]);
    hi.x = fmul(dl, kv[(w >> 4) & 15]); hi.y = fmul(dl, kv[(w >> 12) & 15]); hi.z = fmul(dl, kv[(w >> 20) & 15]); hi.w = fmul(dl, kv[w >> 28]);
    __stcs(reinterpret_cast<float4 *>(o), lo);
    __stcs(reinterpret_cast<float4 *>(o + 16), hi);
}

__global__ void __launch_bounds__(256) embd_rows_iq4xs_kernel(const uint8_t * __restrict__ table, const int * __restrict__ tok, int nvocab, int n, int nblk,
                                                              float * __restrict__ out, int * err) {
    __shared__ float kv[16];
    if (threadIdx.x < 16) kv[threadIdx.x] = kIQ4NL[threadIdx.x];
    __syncthreads();
    const int units = nblk * 32;
    for (int p = blockIdx.x; p < n; p += gridDim.x) {
        int t = __ldg(tok + p);
        if (t < 0 || t >= nvocab) { if (threadIdx.x == 0) atomicOr(err, 2); t = t < 0 ? 0 : nvocab - 1; }
        const uint8_t * row = table + (size_t)t * (size_t)(nblk * 136);
        float * orow = out + (size_t)p * (size_t)(nblk * 256);
        for (int q = threadIdx.x; q < units; q += 256) {
            const int bl = q >> 5, ib = (q >> 2) & 7, jq = q & 3;
            const uint8_t * b = row + (size_t)bl * 136;
            const uint2 hd = __ldg(reinterpret_cast<const uint2 *>(b));                         // d | scales_h | scales_l[4]
            const int sh = hd.x >> 16, sl = (hd.y >> (8 * (ib >> 1))) & 0xff;
            const int ls = ((sl >> ((ib & 1) * 4)) & 15) | (((sh >> (2 * ib)) & 3) << 4);
            const float dl = fmul(__half2float(__ushort_as_half((unsigned short)(hd.x & 0xffffu))), (float)(ls - 32));
            iq4_store8(orow + bl * 256 + ib * 32 + 4 * jq, kv, __ldg(reinterpret_cast<const uint32_t *>(b + 8 + 16 * ib + 4 * jq)), dl);
        }
    }
}

__global__ void __launch_bounds__(256) ple_rows_iq4nl_kernel(const uint8_t * __restrict__ raw, const int * __restrict__ inv, int nuniq, int nrows, int bpr,
                                                             float * __restrict__ out, int * err) {
    __shared__ float kv[16];
    if (threadIdx.x < 16) kv[threadIdx.x] = kIQ4NL[threadIdx.x];
    __syncthreads();
    const int units = bpr * 4;
    for (int r = blockIdx.x; r < nrows; r += gridDim.x) {
        int u = __ldg(inv + r);
        if (u < 0 || u >= nuniq) { if (threadIdx.x == 0) atomicOr(err, 1); u = u < 0 ? 0 : nuniq - 1; }
        const uint8_t * row = raw + (size_t)u * (size_t)(bpr * 18);
        float * orow = out + (size_t)r * (size_t)(bpr * 32);
        for (int q = threadIdx.x; q < units; q += 256) {
            const int b = q >> 2, jq = q & 3;
            const uint16_t * blk = reinterpret_cast<const uint16_t *>(row + (size_t)b * 18);    // d, then 16 bytes of nibbles
            const uint32_t w = (uint32_t)__ldg(blk + 1 + 2 * jq) | ((uint32_t)__ldg(blk + 2 + 2 * jq) << 16);
            iq4_store8(orow + b * 32 + 4 * jq, kv, w, __half2float(__ushort_as_half(__ldg(blk))));
        }
    }
}

// ---- Q6_K rows (no kernel of the reference gathers them; its host decoder python/caminus/own_dequant.py:40-53 is the definition) -----
// 210-byte blocks of 256 values: ql[128] | qh[64] | int8 sc[16] | fp16 d. Per half n of 128 and group qd of 32, lane l:
// q = nibble of ql[n][(qd & 1) 32 + l] (high for qd >= 2) | ((qh[n][l] >> 2 qd) & 3) << 4; y = (d * sc[8 n + 2 qd + (l >= 16)]) * (q - 32).
// A thread takes four consecutive l of a half and writes their values of all four groups (16 outputs, four 16-byte stores) from
// 12 bytes of the block (2-byte aligned: six 16-bit loads).
__global__ void __launch_bounds__(256) emb_rows_q6k_kernel(const uint8_t * __restrict__ W, int rb, int vocab, const int * __restrict__ toks,
                                                           float * __restrict__ x, int n, int N) {
    const int units = (N >> 8) * 16;
    for (int p = blockIdx.x; p < n; p += gridDim.x) {
        const int t = min(max(__ldg(toks + p), 0), vocab - 1);
        const uint8_t * row = W + (size_t)t * rb;
        float * orow = x + (size_t)p * N;
        for (int q = threadIdx.x; q < units; q += 256) {
            const int bl = q >> 4, nn = (q >> 3) & 1, l = (q & 7) * 4;
            const uint8_t * b = row + (size_t)bl * 210;
            const uint16_t * b16 = reinterpret_cast<const uint16_t *>(b);
            const int lo_at = (nn * 64 + l) >> 1, hi_at = (128 + nn * 32 + l) >> 1;
            const uint32_t qa = (uint32_t)__ldg(b16 + lo_at) | ((uint32_t)__ldg(b16 + lo_at + 1) << 16);             // ql[n][l .. l + 3]
            const uint32_t qb = (uint32_t)__ldg(b16 + lo_at + 16) | ((uint32_t)__ldg(b16 + lo_at + 17) << 16);       // ql[n][32 + l ..]
            const uint32_t qh = (uint32_t)__ldg(b16 + hi_at) | ((uint32_t)__ldg(b16 + hi_at + 1) << 16);             // qh[n][l ..]
            const float d = __half2float(__ushort_as_half(__ldg(b16 + 104)));
            const int8_t * sc = reinterpret_cast<const int8_t *>(b + 192 + nn * 8 + (l >= 16));
#pragma unroll
            for (int qd = 0; qd < 4; qd++) {
                const float ds = fmul(d, (float)(int)sc[2 * qd]);
                const uint32_t src = (qd & 1) ? qb : qa;
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t byte = (src >> (8 * e)) & 0xffu, hb = (qh >> (8 * e)) & 0xffu;
                    const int qv = (int)((qd >= 2 ? byte >> 4 : byte & 15u) | (((hb >> (2 * qd)) & 3u) << 4)) - 32;
                    v[e] = fmul(ds, (float)qv);
                }
                __stcs(reinterpret_cast<float4 *>(orow + bl * 256 + nn * 128 + qd * 32 + l), make_float4(v[0], v[1], v[2], v[3]));
            }
        }
    }
}

// ---- IQ2_S rows: q35t_emb_iq2s (kernels/q35_prefill_tcap.hip:94-113) = q35t_op_emb (kernels/k3_q35t_ops.h:147-175) --------------------
// 82-byte blocks of 256 values: fp16 d | qs[32] | signs[32] | qh[8] | scales[8]. A thread decodes one group of 8 values (one 10-bit grid
// index, one byte of signs): five 16-bit loads in, two 16-byte stores out. The grid (1024 entries of eight 2-bit magnitude codes, packed
// two to a word as the reference's kernels hold it) is GGUF's format constant; the caller supplies it and each block stages it once.
constexpr int IQ2S_ROWS = 4;      // token rows a block decodes together: a thread's loads of the four rows are issued before the first decode
__global__ void __launch_bounds__(256) emb_rows_iq2s_kernel(const uint8_t * __restrict__ W, int rb, int vocab, const int * __restrict__ toks, float * __restrict__ x,
                                                            int n, int N, const uint32_t * __restrict__ grid) {
    __shared__ uint32_t gs[512];
    // two neighbouring values at once: entry (c0 | c1 << 2 | s0 << 4 | s1 << 5) = (+-mag(c0), +-mag(c1)), mag = 8, 25, 43; sixteen copies, one per
    // lane of a 64-bit shared-memory pass (copy j in bank pair j): a warp's lookup is two conflict-free passes whatever the codes are
    __shared__ __align__(8) float2 mag2[64 * 16];
    for (int i = threadIdx.x; i < 512; i += 256) gs[i] = __ldg(grid + i);
    for (int t = threadIdx.x; t < 64 * 16; t += 256) {
        const int i = t >> 4, c0 = i & 3, c1 = (i >> 2) & 3;
        const float m0 = c0 == 0 ? 8.0f : c0 == 1 ? 25.0f : 43.0f, m1 = c1 == 0 ? 8.0f : c1 == 1 ? 25.0f : 43.0f;
        mag2[t] = make_float2((i & 16) ? -m0 : m0, (i & 32) ? -m1 : m1);
    }
    __syncthreads();
    const int units = N >> 3;
    for (int p0 = blockIdx.x * IQ2S_ROWS; p0 < n; p0 += gridDim.x * IQ2S_ROWS) {
        const uint8_t * row[IQ2S_ROWS];
#pragma unroll
        for (int r = 0; r < IQ2S_ROWS; r++) {
            int t = __ldg(toks + (p0 + r < n ? p0 + r : n - 1)); t = t < 0 ? 0 : t >= vocab ? vocab - 1 : t;
            row[r] = W + (size_t)t * rb;
        }
        for (int q = threadIdx.x; q < units; q += 256) {
            const int j8 = q & 31, ib = j8 >> 2, g = j8 & 3;
            uint32_t raw[IQ2S_ROWS][5];
#pragma unroll
            for (int r = 0; r < IQ2S_ROWS; r++) {
                const uint16_t * b16 = reinterpret_cast<const uint16_t *>(row[r] + (size_t)(q >> 5) * 82);
                raw[r][0] = __ldg(b16); raw[r][1] = __ldg(b16 + 1 + (j8 >> 1)); raw[r][2] = __ldg(b16 + 33 + (ib >> 1));
                raw[r][3] = __ldg(b16 + 37 + (ib >> 1)); raw[r][4] = __ldg(b16 + 17 + (j8 >> 1));
            }
#pragma unroll
            for (int r = 0; r < IQ2S_ROWS; r++) {
                if (p0 + r >= n) break;
                const float d = __half2float(__ushort_as_half((unsigned short)raw[r][0]));
                const uint32_t lo = (raw[r][1] >> (8 * (j8 & 1))) & 0xffu;                 // qs[j8]
                const uint32_t qh = (raw[r][2] >> (8 * (ib & 1))) & 0xffu;                 // qh[ib]
                const uint32_t sb = (raw[r][3] >> (8 * (ib & 1))) & 0xffu;                 // scales[ib]
                const uint32_t sg = (raw[r][4] >> (8 * (j8 & 1))) & 0xffu;                 // signs[j8]
                const uint32_t idx = lo | (((qh >> (2 * g)) & 3u) << 8);
                const uint32_t codes = (gs[idx >> 1] >> (16 * (idx & 1u))) & 0xffffu;
                const float db = fmul(fmul(d, fadd(0.5f, (float)((sb >> (4 * ((j8 >> 1) & 1))) & 15u))), 0.25f);
                // db times the signed magnitude: the product's bits are those of -(db mag) or db mag (the sign of an IEEE product is exact)
                const f32x2 db2 = pk2(db, db);
                f32x2 v[4];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 m = mag2[((((codes >> (4 * k)) & 15u) | (((sg >> (2 * k)) & 3u) << 4)) << 4) | (threadIdx.x & 15u)];
                    v[k] = mul2(db2, pk2(m.x, m.y));
                }
                float * o = x + (size_t)(p0 + r) * N + 8 * q;
                __stcs(reinterpret_cast<float4 *>(o), make_float4(lo2(v[0]), hi2(v[0]), lo2(v[1]), hi2(v[1])));      // (one 256-bit store here measured slower: 40.8 us against 32.6 us)
                __stcs(reinterpret_cast<float4 *>(o + 4), make_float4(lo2(v[2]), hi2(v[2]), lo2(v[3]), hi2(v[3])));
            }
        }
    }
}

// The same rows with the table's bytes staged: a warp per token row copies the row's blocks into its own shared-memory slice by 16-byte
// cp.async (the next row's copy in flight while this one is decoded: the id, the row and its bytes are three dependent loads otherwise;
// the first copy is issued before the block builds its tables) and decodes from there: block bl's group `lane` per step, byte reads
// that cost no global request. Rows 16-byte aligned (table and rb).
// The magnitudes come from byte permutes: the grid entry is held as eight 4-bit selectors (the 2-bit code, bit 2 = the value's sign bit,
// spread from the signs byte by a 256-entry table); one permute over the pools 128 + {8, 25, 43, 43} and 128 - {8, 25, 43, 43} yields
// four biased signed bytes, a second one per value puts the byte under the bits of 1.5 2^23, and a packed subtraction leaves the signed
// magnitude as a float, exactly. The group's eight floats leave as ONE 256-bit store: two 16-byte stores at a 32-byte lane stride write
// every 32-byte sector twice, half at a time (the second level saw 7.8 M sector writes for 4.2 M sectors, and the kernel 45 us
// whatever its arithmetic cost: 30 us with the one store).
CAM_DEV void iq2s_copy_row(uint8_t * dst, const uint8_t * src, int chunks, int lane) {
    for (int c = lane; c < chunks; c += 32) cp_async16(dst + 16 * c, src + 16 * c);
}
CAM_DEV uint32_t spread2to4(uint32_t e) {         // sixteen bits as eight 2-bit fields -> eight nibbles
    e = (e | (e << 8)) & 0x00ff00ffu; e = (e | (e << 4)) & 0x0f0f0f0fu; e = (e | (e << 2)) & 0x33333333u;
    return e;
}
template <int NBLK, int WPB>
__global__ void __launch_bounds__(32 * WPB) emb_rows_iq2s_staged_kernel(const uint8_t * __restrict__ W, int rb, int vocab, const int * __restrict__ toks,
                                                                   float * __restrict__ x, int n, int N, const uint32_t * __restrict__ grid) {
    __shared__ uint32_t sel[1024];                                        // grid entry -> selectors (code per nibble)
    __shared__ uint32_t sgn[256];                                         // signs byte -> bit 2 of nibble j = bit j
    extern __shared__ __align__(16) uint8_t iq2s_stage[];                 // [warp][2][chunks * 16]
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31u) == 0;       // (rows are multiples of 1 KB: every group's eight floats are 32-byte aligned then)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nblk = NBLK ? NBLK : N >> 8, chunks = (nblk * 82 + 15) >> 4, stride = gridDim.x * WPB;
    uint8_t * const mine = iq2s_stage + (size_t)warp * 2 * chunks * 16;
    auto clamp_id = [&](int t) { return t < 0 ? 0 : t >= vocab ? vocab - 1 : t; };
    // a warp per row; the ids of this warp's first three rows are loaded before anything waits for one
    int p = blockIdx.x * WPB + warp;
    const int id0 = p < n ? __ldg(toks + p) : 0, id1 = p + stride < n ? __ldg(toks + p + stride) : 0;
    int id2 = p + 2 * stride < n ? __ldg(toks + p + 2 * stride) : 0;
    if (p < n) iq2s_copy_row(mine, W + (size_t)clamp_id(id0) * rb, chunks, lane);
    cp_async_commit();
    for (int i = threadIdx.x; i < 512; i += 32 * WPB) {
        const uint32_t w = __ldg(grid + i);
        sel[2 * i] = spread2to4(w & 0xffffu); sel[2 * i + 1] = spread2to4(w >> 16);
    }
    for (uint32_t v = threadIdx.x; v < 256; v += 32 * WPB) {
        uint32_t t = (v | (v << 12)) & 0x000f000fu; t = (t | (t << 6)) & 0x03030303u; t = (t | (t << 3)) & 0x11111111u;
        sgn[v] = t << 2;
    }
    __syncthreads();
    if (p >= n) return;
    const int qsh = 2 * (lane & 3), ssh = 4 * ((lane >> 1) & 1);
    int idn = id1;                                                        // the next row's id (loaded a pass ago)
    for (int buf = 0;; buf ^= 1) {
        const int pn = p + stride;
        if (pn < n) iq2s_copy_row(mine + (buf ^ 1) * chunks * 16, W + (size_t)clamp_id(idn) * rb, chunks, lane);
        cp_async_commit();
        idn = id2;
        if (pn + 2 * stride < n) id2 = __ldg(toks + pn + 2 * stride);   // (used two passes from now)
        cp_async_wait<1>();
        __syncwarp();
        const uint8_t * bq = mine + buf * chunks * 16 + lane, * bh = mine + buf * chunks * 16 + (lane >> 2);
        float * orow = x + (size_t)p * N + 8 * lane;
#pragma unroll
        for (int bl = 0; bl < nblk; bl++) {
            const int off = 82 * bl;
            const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(mine + buf * chunks * 16 + off)));
            const uint32_t lo = bq[off + 2], sg = bq[off + 34], qh = bh[off + 66], sb = bh[off + 74];
            const uint32_t s8 = sel[lo + (((qh >> qsh) & 3u) << 8)] | sgn[sg];
            const float db = fmul(fmul(d, fadd(0.5f, (float)((sb >> ssh) & 15u))), 0.25f);
            const f32x2 db2 = pk2(db, db);
            // four signed magnitudes each, as bytes biased by 128: 128 + {8, 25, 43, 43} and 128 - {8, 25, 43, 43}
            const uint32_t m0 = __byte_perm(0xabab9988u, 0x55556778u, s8), m1 = __byte_perm(0xabab9988u, 0x55556778u, s8 >> 16);
            // a byte under the bits of 1.5 2^23 is the float 12582912 + byte: minus 12583040 it is the signed magnitude, exactly (a
            // permute and half a packed subtraction per value, against a shift, a sign extension and a conversion)
            const f32x2 bias = pk2(-12583040.0f, -12583040.0f);
            const f32x2 f0 = add2(pk2(__uint_as_float(__byte_perm(m0, 0x4b400000u, 0x7650)), __uint_as_float(__byte_perm(m0, 0x4b400000u, 0x7651))), bias);
            const f32x2 f1 = add2(pk2(__uint_as_float(__byte_perm(m0, 0x4b400000u, 0x7652)), __uint_as_float(__byte_perm(m0, 0x4b400000u, 0x7653))), bias);
            const f32x2 f2 = add2(pk2(__uint_as_float(__byte_perm(m1, 0x4b400000u, 0x7650)), __uint_as_float(__byte_perm(m1, 0x4b400000u, 0x7651))), bias);
            const f32x2 f3 = add2(pk2(__uint_as_float(__byte_perm(m1, 0x4b400000u, 0x7652)), __uint_as_float(__byte_perm(m1, 0x4b400000u, 0x7653))), bias);
            // db times the signed magnitude: the product's bits are those of -(db mag) or db mag (the sign of an IEEE product is exact)
            const f32x2 v0 = mul2(db2, f0), v1 = mul2(db2, f1), v2 = mul2(db2, f2), v3 = mul2(db2, f3);
            st8f_cs(orow + bl * 256, make_float4(lo2(v0), hi2(v0), lo2(v1), hi2(v1)), make_float4(lo2(v2), hi2(v2), lo2(v3), hi2(v3)), wide);
        }
        __syncwarp();                                                    // (the slice read here is the one the copy after next writes)
        if (pn >= n) break;
        p = pn;
    }
    cp_async_wait<0>();
}

}   // namespace

// embd_rows_iq4xs / ple_rows_iq4nl: kernels/prefill_feed.hip:40-41, 24-25 (one thread per output float there)
extern "C" int embd_rows_iq4xs(const void * table, const int * tok, int nvocab, int n, int nblk, float * out, int * err, void * stream) {
    if (n < 0 || nvocab < 1 || nblk < 1 || !table || !tok || !out || !err) return CAM_ERR_ARG;
    if (!cam_aligned16(out)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    const long want = ((long)n * nblk * 64 + 255) / 256;
    if (reinterpret_cast<uintptr_t>(table) & 7u)
        embd_rows_iq4xs_bytes_kernel<<<cam_resident_grid(embd_rows_iq4xs_bytes_kernel, 256, 0, want), 256, 0, (cudaStream_t)stream>>>((const uint8_t *)table, tok, nvocab, n, nblk, out, err);
    else embd_rows_iq4xs_kernel<<<cam_resident_grid(embd_rows_iq4xs_kernel, 256, 0, n), 256, 0, (cudaStream_t)stream>>>((const uint8_t *)table, tok, nvocab, n, nblk, out, err);
    return (int)cudaGetLastError();
}
extern "C" int ple_rows_iq4nl(const void * raw, const int * inv, int nuniq, int nrows, int bpr, float * out, int * err, void * stream) {
    if (nrows < 0 || nuniq < 1 || bpr < 1 || !raw || !inv || !out || !err) return CAM_ERR_ARG;
    if (!cam_aligned16(out)) return CAM_ERR_ALIGN;
    if (nrows == 0) return CAM_OK;
    const long want = ((long)nrows * bpr * 8 + 255) / 256;
    if (reinterpret_cast<uintptr_t>(raw) & 1u)
        ple_rows_iq4nl_bytes_kernel<<<cam_resident_grid(ple_rows_iq4nl_bytes_kernel, 256, 0, want), 256, 0, (cudaStream_t)stream>>>((const uint8_t *)raw, inv, nuniq, nrows, bpr, out, err);
    else ple_rows_iq4nl_kernel<<<cam_resident_grid(ple_rows_iq4nl_kernel, 256, 0, nrows), 256, 0, (cudaStream_t)stream>>>((const uint8_t *)raw, inv, nuniq, nrows, bpr, out, err);
    return (int)cudaGetLastError();
}

// cam_emb_rows_q6k: x [n][N] fp32 = the Q6_K rows toks[i] of a table (vocab rows of rb = N / 256 * 210 bytes), ids clamped to the
// vocabulary; the floats of the reference's host decoder (python/caminus/own_dequant.py:40-53, bitwise gguf-py). N a multiple of 256,
// W 2-byte aligned, x 16-byte aligned.
extern "C" int cam_emb_rows_q6k(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, void * stream) {
    if (n < 0 || vocab < 1 || N < 256 || (N & 255) || rb < N / 256 * 210 || !W || !toks || !x) return CAM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(W) & 1u) || (rb & 1) || !cam_aligned16(x)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    emb_rows_q6k_kernel<<<cam_resident_grid(emb_rows_q6k_kernel, 256, 0, n, 8), 256, 0, (cudaStream_t)stream>>>((const uint8_t *)W, rb, vocab, toks, x, n, N);
    return (int)cudaGetLastError();
}

// q35t_emb_iq2s: x [n][N] fp32 = the IQ2_S rows toks[i] of a table (vocab rows of rb >= N / 256 * 82 bytes), ids clamped to the vocabulary:
// kernels/q35_prefill_tcap.hip:94-113 (n = the reference's grid.x). grid: 512 words on the device, the packed IQ2_S grid of the reference's
// kernels/iq2s_grid.h (a constant of its code object; here the caller's). N a multiple of 256, W and rb 2-byte aligned, x 16-byte aligned.
extern "C" int q35t_emb_iq2s(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, const unsigned int * grid, void * stream) {
    if (n < 0 || vocab < 1 || N < 256 || (N & 255) || rb < N / 256 * 82 || !W || !toks || !x || !grid) return CAM_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(W) & 1u) || (rb & 1) || !cam_aligned16(x) || (reinterpret_cast<uintptr_t>(grid) & 3u)) return CAM_ERR_ALIGN;
    if (n == 0) return CAM_OK;
    const size_t stage = (size_t)8 * 2 * ((N / 256 * 82 + 15) / 16) * 16;
    if (cam_aligned16(W) && !(rb & 15) && stage <= 36 * 1024) {         // (rows of up to 15616 values; longer ones take the kernel below)
        // a warp per row, a block per eight rows; more blocks than are resident (measured: 29.1 us against 30.7 us for resident blocks that
        // loop; blocks of four or two warps 30.6-33.9 us), up to a grid the loop in the kernel then covers
        long g8 = ((long)n + 7) / 8;
        if (g8 > (1L << 20)) g8 = 1L << 20;
        if (N == 2048) emb_rows_iq2s_staged_kernel<8, 8><<<(int)g8, 256, stage, (cudaStream_t)stream>>>((const uint8_t *)W, rb, vocab, toks, x, n, N, grid);
        else emb_rows_iq2s_staged_kernel<0, 8><<<(int)g8, 256, stage, (cudaStream_t)stream>>>((const uint8_t *)W, rb, vocab, toks, x, n, N, grid);
        return (int)cudaGetLastError();
    }
    const long want = ((long)n + IQ2S_ROWS - 1) / IQ2S_ROWS;
    long g = cam_resident_grid(emb_rows_iq2s_kernel, 256, 0, want);
    emb_rows_iq2s_kernel<<<(int)g, 256, 0, (cudaStream_t)stream>>>((const uint8_t *)W, rb, vocab, toks, x, n, N, grid);
    return (int)cudaGetLastError();
}
