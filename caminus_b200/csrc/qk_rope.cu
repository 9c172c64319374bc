// Qwen3 per-head q/k RMSNorm fused with NeoX rotary embedding (the reference's q3p_qk_rope, kernels/q3m_prefill.hip:520-591;
// its T = 1 form is the norm + RoPE part of own_op_attn / OP_OWN_ATTS, kernels/k3_own_ops.h:515-542).
//
// Reference statements per head of 128 (one thread per dim, 4 waves): ss = x x; wave sums by the xor butterfly (16, 8, 4, 2, 1),
// the 4 wave sums added in order; scale = rsqrtf(tot / 128 + eps); y1 = (scale x) w; pair (j, j + 64):
// theta = (float)pos powf(theta_scale, (float)j) [YaRN objects: (float)pos freq[j], cos and sin times mscale];
// out[j] = fma(y1[j], c, -(y1[j + 64] s)), out[j + 64] = fma(y1[j + 64], c, y1[j] s); stored as fp16.
//
// Mapping: one thread block per token, looping over tokens. The token's heads are brought into shared memory with cp.async
// (16 bytes per thread, three stages: the next two tokens' copies fly while this one is computed). The 64 cos / sin of a
// position are computed once per token (64 threads) and shared by all of its heads; the reference recomputes them in every
// (token, head) workgroup. A half-warp owns a head: lane l holds dims 4l .. 4l + 3 and 64 + 4l .. 64 + 4l + 3, i.e. complete
// rotation pairs, so the rotation needs no exchange.
// Sum of squares: the order of THIS mapping, not the reference's: per lane an fma chain over its 4 low dims and one over
// its 4 high dims, added, then the half-warp butterfly with partners 8, 4, 2, 1. (The reference's order, squares rounded one
// by one and a 32-lane butterfly per 32 consecutive dims, costs 13 shuffles and 20 additions per head here against 4 and 5,
// on a kernel that is instruction-bound; the sum is one input of a tolerance-gated fp16 result.) Every other statement is
// the reference's.
#include "cam_common.cuh"
#include "kv_q8.cuh"

#include <cstdio>
#include <cstdlib>

namespace {

struct RopeArgs {
    const void * in0;      // CACHE: qkv fp32 [n][ldq]. Otherwise q fp16 [n][nh][128]
    const void * in1;      // otherwise k fp16 [n][nkv][128]
    const float * par;     // q_norm[128] | k_norm[128] | theta_scale | eps (| freq[64] | mscale)
    uint16_t * out0;       // q16 [n][nh][128]
    uint16_t * out1;       // CACHE: the KV cache (rows of 2 nkv 128 halves). Otherwise k out [n][nkv][128]
    int ldq, nh, nkv, pos0, n, yarn;
    int * err;             // Q8: the word a refused Q8_0 block ORs 2 into
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
// P: heads per half-warp and round: a warp takes 2 P heads of a token at a time, reduces them all, then ONE pass of the
// scale's square root and divisions serves all of them (lane j computes head j's), instead of one per head.
// Q8 (with CACHE): the Q8_0 KV cache form (q3p_qk_rope_q8, kernels/q3m_prefill.hip:526-535, 572-583; csrc/kv_q8.cuh): out1 is the
// byte cache, q16 and K are Hadamard-transformed, K and V are stored as Q8_0 blocks.
// ONE: the block's warps cover the token's heads in exactly one round (H = 2 P warps): no head loop and no bounds tests, and
// everything that depends only on the head (offsets in the stage and in the output, the weight row) is computed before
// the token loop.
constexpr int ROPE_STAGES = 3;        // tokens in flight per block: two copies fly while one token is computed

template <typename T, bool CACHE, int P, bool ONE, bool Q8 = false>
__global__ void __launch_bounds__(384) qk_rope_kernel(const RopeArgs A) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int nh = A.nh, nkv = A.nkv, H = nh + nkv;
    const int in_heads = CACHE ? nh + 2 * nkv : H;                       // heads staged per token
    const int stage_bytes = in_heads * 128 * (int)sizeof(T);
    float * wq = reinterpret_cast<float *>(smem);                        // [128] | wk [128] | freq [64] | rc [S][64] | rs [S][64]
    float * wk = wq + 128, * freq = wk + 128, * rc = freq + 64, * rs = rc + 64 * ROPE_STAGES;
    unsigned char * stage = smem + (128 + 128 + 64 + 2 * 64 * ROPE_STAGES) * 4;
    const float eps = __ldg(A.par + 257);

    const float mscale = A.yarn ? __ldg(A.par + 322) : 1.0f;

    auto issue = [&](int t, int st) {
        if (t < A.n) {
            unsigned char * s = stage + st * stage_bytes;
            if (CACHE) {
                const unsigned char * src = reinterpret_cast<const unsigned char *>(reinterpret_cast<const float *>(A.in0) + (size_t)t * A.ldq);
                for (int c = tid; c < in_heads * 32; c += blockDim.x) cp_async16(s + c * 16, src + c * 16);
            } else {
                const unsigned char * sq = reinterpret_cast<const unsigned char *>(reinterpret_cast<const uint16_t *>(A.in0) + (size_t)t * nh * 128);
                const unsigned char * sk = reinterpret_cast<const unsigned char *>(reinterpret_cast<const uint16_t *>(A.in1) + (size_t)t * nkv * 128);
                for (int c = tid; c < nh * 16; c += blockDim.x) cp_async16(s + c * 16, sq + c * 16);
                for (int c = tid; c < nkv * 16; c += blockDim.x) cp_async16(s + (nh * 16 + c) * 16, sk + c * 16);
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

    const int hw = lane >> 4, l16 = lane & 15;
    const int xoff = 4 * l16 * (int)sizeof(T);
    // head-only quantities of the ONE form (head hy_p = 2 (warp P + p) + hw)
    int soff[P], ooff[P];
    const float * wrow[P];
    bool isq_[P];
#pragma unroll
    for (int p = 0; p < P; p++) {
        const int hy = 2 * (warp * P + p) + hw;
        isq_[p] = hy < nh;
        soff[p] = hy * 128 * (int)sizeof(T) + xoff;
        ooff[p] = (isq_[p] ? hy : hy - nh) * 128 + 4 * l16;
        wrow[p] = (isq_[p] ? wq : wk) + 4 * l16;
    }

    const int t0 = blockIdx.x, g = gridDim.x;
#pragma unroll
    for (int k = 0; k < ROPE_STAGES - 1; k++) issue(t0 + k * g, k);        // (the first tokens' copies fly while the parameters are read)
    if (tid < 128) { wq[tid] = __ldg(A.par + tid); wk[tid] = __ldg(A.par + 128 + tid); }
    if (tid < 64) {
        freq[tid] = A.yarn ? __ldg(A.par + 258 + tid) : cam_powi(__ldg(A.par + 256), tid);
#pragma unroll
        for (int k = 0; k < ROPE_STAGES - 1; k++)
            if (t0 + k * g < A.n) tables(t0 + k * g, k);
    }
    int st = 0;
    for (int t = t0; t < A.n; t += g, st = st + 1 == ROPE_STAGES ? 0 : st + 1) {
        const int tn = t + (ROPE_STAGES - 1) * g, sn_ = st == 0 ? ROPE_STAGES - 1 : st - 1;      // the stage freed by the previous token
        issue(tn, sn_);
        if (tid < 64 && tn < A.n) tables(tn, sn_);
        cp_async_wait<ROPE_STAGES - 1>();
        __syncthreads();
        const unsigned char * s = stage + st * stage_bytes;
        const float4 c4 = *reinterpret_cast<const float4 *>(rc + st * 64 + 4 * l16), s4 = *reinterpret_cast<const float4 *>(rs + st * 64 + 4 * l16);
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
        const int pos = A.pos0 + t;
        uint16_t * const qbase = A.out0 + (size_t)t * nh * 128;
        uint16_t * const kbase = CACHE ? A.out1 + (size_t)pos * 2 * nkv * 128 : A.out1 + (size_t)t * nkv * 128;
        uint8_t * const cw = reinterpret_cast<uint8_t *>(A.out1) + (size_t)pos * (2 * nkv * 4 * 34);       // Q8: the row's K blocks | V blocks
        for (int h0 = 2 * warp * P; h0 < H; h0 += 2 * nwarps * P) {        // this warp's heads h0 .. h0 + 2 P - 1 (ONE: a single round)
            float x[P][8], tot[P];
#pragma unroll
            for (int p = 0; p < P; p++) {
                const int hy = h0 + 2 * p + hw;
                if (ONE || hy < H) {
                    const unsigned char * hp = ONE ? s + soff[p] : s + hy * 128 * (int)sizeof(T) + xoff;   // q heads then k heads
                    float lo[4], hi[4];
                    In<T>::get4(hp, lo);
                    In<T>::get4(hp + 64 * sizeof(T), hi);
#pragma unroll
                    for (int c = 0; c < 4; c++) { x[p][c] = lo[c]; x[p][4 + c] = hi[c]; }
                } else {
#pragma unroll
                    for (int c = 0; c < 8; c++) x[p][c] = 0.0f;
                }
                // the head's sum of squares: per lane an fma chain over its 4 low and its 4 high dims, then the half-warp butterfly
                float sl = 0.0f, sh = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; c++) { sl = ffma(x[p][c], x[p][c], sl); sh = ffma(x[p][4 + c], x[p][4 + c], sh); }
                float ss = fadd(sl, sh);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) ss = fadd(ss, __shfl_xor_sync(CAM_FULL, ss, o));
                tot[p] = ss;
            }
            // lane j < 2 P computes the scale of head h0 + j (pass j >> 1, half-warp j & 1); then every lane fetches its heads' scales
            float mine = 1.0f;
#pragma unroll
            for (int p = 0; p < P; p++) {
                const float v = __shfl_sync(CAM_FULL, tot[p], 16 * (lane & 1));
                if ((lane >> 1) == p) mine = v;
            }
            const float scale_mine = cam_rsqrt(fadd(fmul(mine, 0.0078125f), eps));      // tot / 128: the same bits as the division
#pragma unroll
            for (int p = 0; p < P; p++) {
                const float scale = __shfl_sync(CAM_FULL, scale_mine, 2 * p + hw);
                const int hy = h0 + 2 * p + hw;
                const bool on = ONE || hy < H;
                if (Q8 || on) {                 // (Q8: every lane takes part in the exchanges below; an idle half-warp holds zeros)
                    const bool isq = ONE ? isq_[p] : hy < nh;
                    const float * wn = ONE ? wrow[p] : (isq ? wq : wk) + 4 * l16;
                    const float4 wlo = *reinterpret_cast<const float4 *>(wn), whi = *reinterpret_cast<const float4 *>(wn + 64);
                    const float wl[4] = {wlo.x, wlo.y, wlo.z, wlo.w}, wh[4] = {whi.x, whi.y, whi.z, whi.w};
                    float ylo[4], yhi[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const float x0 = fmul(fmul(scale, x[p][c]), wl[c]), x1 = fmul(fmul(scale, x[p][4 + c]), wh[c]);
                        ylo[c] = ffma(x0, cc[c], -fmul(x1, sn[c]));
                        yhi[c] = ffma(x1, cc[c], fmul(x0, sn[c]));
                    }
                    if (!Q8) {
                        uint16_t * o = (isq ? qbase : kbase) + (ONE ? ooff[p] : (isq ? hy : hy - nh) * 128 + 4 * l16);
                        st64_stream(o, make_uint2(f2_to_h2(ylo[0], ylo[1]), f2_to_h2(ylo[2], ylo[3])));
                        st64_stream(o + 64, make_uint2(f2_to_h2(yhi[0], yhi[1]), f2_to_h2(yhi[2], yhi[3])));
                    } else {
                        float y[8];
#pragma unroll
                        for (int c = 0; c < 4; c++) { y[c] = f16r(ylo[c]); y[4 + c] = f16r(yhi[c]); }
                        hadamard128(y, l16);
                        if (on && isq) {
                            uint16_t * o = qbase + (ONE ? ooff[p] : hy * 128 + 4 * l16);
                            st64_stream(o, make_uint2(f2_to_h2(y[0], y[1]), f2_to_h2(y[2], y[3])));
                            st64_stream(o + 64, make_uint2(f2_to_h2(y[4], y[5]), f2_to_h2(y[6], y[7])));
                        }
                        // a warp's second head is the later one: it is a k head whenever either is (warp-uniform test)
                        if (ONE ? 2 * (warp * P + p) + 1 >= nh : __any_sync(CAM_FULL, on && !isq)) {
                            const bool kv = on && !isq;
                            uint8_t * kb = cw + (size_t)(kv ? hy - nh : 0) * 4 * 34 + (size_t)(l16 >> 3) * 34;
                            const float klo[4] = {y[0], y[1], y[2], y[3]}, khi[4] = {y[4], y[5], y[6], y[7]};
                            q8_0_store(klo, kb, l16 & 7, A.err, kv);
                            q8_0_store(khi, kb + 2 * 34, l16 & 7, A.err, kv);
                        }
                    }
                }
            }
        }
        if (CACHE && Q8) {      // v: rounded to fp16, then Q8_0 blocks of 32: 8 lanes a block (whole warps: nkv 32 is a multiple of 32)
            const float * vs = reinterpret_cast<const float *>(s) + (size_t)H * 128;
            uint8_t * vb = cw + (size_t)nkv * 4 * 34;
            for (int c = tid; c < nkv * 32; c += blockDim.x) {
                const float4 v = *reinterpret_cast<const float4 *>(vs + 4 * c);
                const float vv[4] = {f16r(v.x), f16r(v.y), f16r(v.z), f16r(v.w)};
                q8_0_store(vv, vb + (size_t)(c >> 3) * 34, c & 7, A.err, true);
            }
        } else if (CACHE) {      // v: copied as fp16 into the row's V half
            const float * vs = reinterpret_cast<const float *>(s) + (size_t)H * 128;
            uint16_t * vo = kbase + (size_t)nkv * 128;
            for (int c = tid; c < nkv * 32; c += blockDim.x) {
                const float4 v = *reinterpret_cast<const float4 *>(vs + 4 * c);
                st64_stream(vo + 4 * c, make_uint2(f2_to_h2(v.x, v.y), f2_to_h2(v.z, v.w)));
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
}

// ---- the fp16-storage form (cam_qk_rope_f16) without a block-wide step per token -----------------------------------------------------
// A warp owns a token and walks first its q heads, then its k heads, 2 P at a time (a half-warp per head, as above; nh and nkv even,
// so a round is all q or all k and a pair of heads is whole). Every lane copies exactly the two 8-byte pieces of a head that it will
// read (dims 4 l .. 4 l + 3 and 64 + 4 l ..) into the warp's own ring in shared memory with cp.async, RING - 1 rounds ahead, so its own
// copy groups are the only synchronisation: nothing in the token loop waits on another warp (the staged kernel above holds a block at
// two barriers per token, which a batch of a few thousand tokens, four or five per block, never amortises), and a warp keeps RING - 1
// rounds of loads in flight without holding them in registers. A round's addresses are one base (q or k of the token) plus constants.
// The 64 frequencies are formed once per block (the only barrier; the first rounds' copies are already flying); a token's cosines and
// sines are formed by its warp: each half-warp computes two of a lane's four angles and the halves swap. The arithmetic is written
// with the packed fp32 instructions where two statements run on neighbouring dims (the norm's two products, the rotation): the same
// IEEE operations, half the instructions. Sums and statement order are the staged kernel's. In place (qo = q, ko = k) is safe: a lane
// stores exactly the addresses it copied, after its copy has landed.
constexpr int ROPE_RING = 4;

CAM_DEV void cp_async8_s(uint32_t smem_addr, const void * gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_addr), "l"(gmem) : "memory");
}
CAM_DEV void cp_async16_s(uint32_t smem_addr, const void * gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem) : "memory");
}
CAM_DEV uint2 lds64(uint32_t smem_addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(smem_addr));
    return v;
}

template <int P>
__global__ void __launch_bounds__(128) qk_rope_f16_warp_kernel(const RopeArgs A) {
    __shared__ __align__(16) float wq[128], wk[128], freq[64];
    __shared__ __align__(16) unsigned char ring_all[4 * ROPE_RING * P * 512];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nh = A.nh, nkv = A.nkv;
    const int rq_n = (nh + 2 * P - 1) / (2 * P), rounds = rq_n + (nkv + 2 * P - 1) / (2 * P);      // q rounds, then k rounds
    const int hw = lane >> 4, l16 = lane & 15;
    const int lane_off = hw * 256 + l16 * 8;                             // bytes: this lane's low piece inside a pair of heads (the high piece: + 128)
    const unsigned char * const qin = reinterpret_cast<const unsigned char *>(A.in0), * const kin = reinterpret_cast<const unsigned char *>(A.in1);
    unsigned char * const qout = reinterpret_cast<unsigned char *>(A.out0), * const kout = reinterpret_cast<unsigned char *>(A.out1);
    const int tw = blockIdx.x * 4 + warp, stride = gridDim.x * 4;
    const int ntok = tw < A.n ? (A.n - tw + stride - 1) / stride : 0;
    const size_t qrow = (size_t)nh * 256, krow = (size_t)nkv * 256;      // bytes per token
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_all) + warp * (ROPE_RING * P * 512) + lane_off;
    // the round to request next: token kq (its q and k rows), round rq, ring slot sq
    int rq = 0, kq = 0, sq = 0;
    const unsigned char * rq_q = qin + (size_t)tw * qrow + lane_off, * rq_k = kin + (size_t)tw * krow + lane_off;
    auto request = [&]() {                                               // one copy group per call (empty past the warp's last token)
        if (kq < ntok) {
            const bool isq = rq < rq_n;
            const int h0 = isq ? rq * 2 * P : (rq - rq_n) * 2 * P, np = min(P, ((isq ? nh : nkv) - h0) >> 1);
            const unsigned char * src = (isq ? rq_q : rq_k) + h0 * 256;
            const uint32_t dst = ring + sq * (P * 512);
#pragma unroll
            for (int p = 0; p < P; p++)
                if (p < np) { cp_async8_s(dst + p * 512, src + p * 512); cp_async8_s(dst + p * 512 + 128, src + p * 512 + 128); }
        }
        cp_async_commit();
        if (++rq == rounds) { rq = 0; kq++; rq_q += (size_t)stride * qrow; rq_k += (size_t)stride * krow; }
        sq = sq + 1 == ROPE_RING ? 0 : sq + 1;
    };
#pragma unroll
    for (int i = 0; i < ROPE_RING - 1; i++) request();
    wq[tid] = __ldg(A.par + tid); wk[tid] = __ldg(A.par + 128 + tid);
    if (tid < 64) freq[tid] = A.yarn ? __ldg(A.par + 258 + tid) : cam_powi(__ldg(A.par + 256), tid);
    const float eps = __ldg(A.par + 257), mscale = A.yarn ? __ldg(A.par + 322) : 1.0f;
    __syncthreads();
    const float f0 = freq[4 * l16 + 2 * hw], f1 = freq[4 * l16 + 2 * hw + 1];      // this half-warp's two of the lane's four angles
    f32x2 cc[2], sn[2], nsn[2];                                          // cos, sin, -sin of dims (4 l16, + 1) and (+ 2, + 3)
    int r = 0, sc = 0, t = tw;
    unsigned char * out_q = qout + (size_t)tw * qrow + lane_off, * out_k = kout + (size_t)tw * krow + lane_off;
    for (int k = 0; k < ntok;) {
        request();
        if (r == 0) {
            const float pos = (float)(A.pos0 + t);
            float s0, c0, s1, c1;
            cam_sincos(fmul(pos, f0), s0, c0); cam_sincos(fmul(pos, f1), s1, c1);
            if (A.yarn) { c0 = fmul(c0, mscale); s0 = fmul(s0, mscale); c1 = fmul(c1, mscale); s1 = fmul(s1, mscale); }
            const float oc0 = __shfl_xor_sync(CAM_FULL, c0, 16), os0 = __shfl_xor_sync(CAM_FULL, s0, 16);
            const float oc1 = __shfl_xor_sync(CAM_FULL, c1, 16), os1 = __shfl_xor_sync(CAM_FULL, s1, 16);
            const float ca = hw ? oc0 : c0, cb = hw ? oc1 : c1, cc_ = hw ? c0 : oc0, cd = hw ? c1 : oc1;      // dims 0, 1 come from the lower half-warp
            const float sa = hw ? os0 : s0, sb = hw ? os1 : s1, sc_ = hw ? s0 : os0, sd = hw ? s1 : os1;
            cc[0] = pk2(ca, cb); cc[1] = pk2(cc_, cd); sn[0] = pk2(sa, sb); sn[1] = pk2(sc_, sd); nsn[0] = pk2(-sa, -sb); nsn[1] = pk2(-sc_, -sd);
        }
        cp_async_wait<ROPE_RING - 1>();                                  // this round's pieces have landed (the later ones may still fly)
        const bool isq = r < rq_n;
        const int h0 = isq ? r * 2 * P : (r - rq_n) * 2 * P, np = min(P, ((isq ? nh : nkv) - h0) >> 1);
        const uint32_t src = ring + sc * (P * 512);
        f32x2 xl[P][2], xh[P][2]; float tot[P];
#pragma unroll
        for (int p = 0; p < P; p++) {
            uint2 vlo = make_uint2(0u, 0u), vhi = make_uint2(0u, 0u);
            if (p < np) { vlo = lds64(src + p * 512); vhi = lds64(src + p * 512 + 128); }
            const float2 a = h2_to_f2(vlo.x), b = h2_to_f2(vlo.y), c = h2_to_f2(vhi.x), e = h2_to_f2(vhi.y);
            // the head's sum of squares: per lane an fma chain over its 4 low and its 4 high dims, then the half-warp butterfly
            float sl = ffma(a.x, a.x, 0.0f), sh = ffma(c.x, c.x, 0.0f);
            sl = ffma(a.y, a.y, sl); sh = ffma(c.y, c.y, sh); sl = ffma(b.x, b.x, sl); sh = ffma(e.x, e.x, sh); sl = ffma(b.y, b.y, sl); sh = ffma(e.y, e.y, sh);
            float ss = fadd(sl, sh);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss = fadd(ss, __shfl_xor_sync(CAM_FULL, ss, o));
            tot[p] = ss;
            xl[p][0] = pk2(a.x, a.y); xl[p][1] = pk2(b.x, b.y); xh[p][0] = pk2(c.x, c.y); xh[p][1] = pk2(e.x, e.y);
        }
        // lane j < 2 P computes the scale of head h0 + j (pass j >> 1, half-warp j & 1); then every lane fetches its heads' scales
        float own = 1.0f;
#pragma unroll
        for (int p = 0; p < P; p++) {
            const float v = __shfl_sync(CAM_FULL, tot[p], 16 * (lane & 1));
            if ((lane >> 1) == p) own = v;
        }
        const float scale_own = cam_rsqrt(fadd(fmul(own, 0.0078125f), eps));      // tot / 128: the same bits as the division
        const float * wn = (isq ? wq : wk) + 4 * l16;
        const float4 wlo = *reinterpret_cast<const float4 *>(wn), whi = *reinterpret_cast<const float4 *>(wn + 64);
        const f32x2 wl2[2] = {pk2(wlo.x, wlo.y), pk2(wlo.z, wlo.w)}, wh2[2] = {pk2(whi.x, whi.y), pk2(whi.z, whi.w)};
        unsigned char * const o = (isq ? out_q : out_k) + h0 * 256;
#pragma unroll
        for (int p = 0; p < P; p++) {
            const float scale = __shfl_sync(CAM_FULL, scale_own, 2 * p + hw);
            if (p < np) {
                const f32x2 s2 = pk2(scale, scale);
                uint32_t olo[2], ohi[2];
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const f32x2 x0 = mul2(mul2(s2, xl[p][c]), wl2[c]), x1 = mul2(mul2(s2, xh[p][c]), wh2[c]);
                    const f32x2 ylo = fma2(x0, cc[c], mul2(x1, nsn[c])), yhi = fma2(x1, cc[c], mul2(x0, sn[c]));
                    olo[c] = f2_to_h2(lo2(ylo), hi2(ylo)); ohi[c] = f2_to_h2(lo2(yhi), hi2(yhi));
                }
                st64_stream(o + p * 512, make_uint2(olo[0], olo[1]));
                st64_stream(o + p * 512 + 128, make_uint2(ohi[0], ohi[1]));
            }
        }
        sc = sc + 1 == ROPE_RING ? 0 : sc + 1;
        if (++r == rounds) { r = 0; k++; t += stride; out_q += (size_t)stride * qrow; out_k += (size_t)stride * krow; }
    }
    cp_async_wait<0>();
}

// ---- the same mapping with the token's shape fixed at compile time ----------------------------------------------------------------------
// NQ2 pairs of q heads and NK2 pairs of k heads per token (NQ2 a multiple of 4, NK2 <= 4 or a multiple of 4): the token's rounds of four
// pairs are unrolled, so every address is a token base plus a constant and nothing is counted or selected at run time. A pair of heads
// is 512 contiguous bytes, copied by the warp as one 16-byte cp.async per lane (a warp barrier then stands between the copies and the
// lanes' reads of their own 8-byte pieces; 8-byte copies, which need none, were measured slower: four times the requests). The ring
// has one slot per round: as soon as a round of this token has been read, the same round of the warp's next token is requested into
// its slot, so almost a whole token of copies is in flight per warp. The four heads' sums of squares of a half-warp are reduced
// together: after the exchange with partner 8 a lane keeps two of the four sums, after partner 4 one (the sums a butterfly forms at
// those lanes, addition being commutative), and partners 2 and 1 finish it: 5 exchanges for four heads instead of 16. Instruction
// count is what bounds this op on a batch of a few thousand tokens (the output of such a batch stays in L2).
template <int NQ2, int NK2>
__global__ void __launch_bounds__(128) qk_rope_f16_tok_kernel(const RopeArgs A) {
    constexpr int RQ = NQ2 / 4, RK = (NK2 + 3) / 4, R = RQ + RK;
    static_assert(NQ2 % 4 == 0 && (NK2 <= 4 || NK2 % 4 == 0), "rounds of four pairs of heads");
    __shared__ __align__(16) float wsm[256], freq[64];
    extern __shared__ __align__(16) unsigned char ring_all[];            // [4 warps][R rounds][2048]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hw = lane >> 4, l16 = lane & 15;
    const int lane_off = hw * 256 + l16 * 8;                             // bytes: this lane's low piece inside a pair of heads (the high piece: + 128)
    constexpr size_t qrow = (size_t)NQ2 * 512, krow = (size_t)NK2 * 512;  // bytes per token
    const int tw = blockIdx.x * 4 + warp, stride = gridDim.x * 4;
    const int ntok = tw < A.n ? (A.n - tw + stride - 1) / stride : 0;
    const uint32_t slots = (uint32_t)__cvta_generic_to_shared(ring_all) + warp * (R * 2048) + lane * 16;      // where this lane copies to
    const uint32_t ring = slots - lane * 16 + lane_off;                                                          // where it reads its pieces
    const unsigned char * in_q = reinterpret_cast<const unsigned char *>(A.in0) + (size_t)tw * qrow + lane * 16;
    const unsigned char * in_k = reinterpret_cast<const unsigned char *>(A.in1) + (size_t)tw * krow + lane * 16;
    unsigned char * out_q = reinterpret_cast<unsigned char *>(A.out0) + (size_t)tw * qrow + lane_off;
    unsigned char * out_k = reinterpret_cast<unsigned char *>(A.out1) + (size_t)tw * krow + lane_off;
    const size_t qstep = (size_t)stride * qrow, kstep = (size_t)stride * krow;
    auto request = [&](int i, const unsigned char * bq, const unsigned char * bk, bool on) {      // round i (a constant after unrolling) of the token at bq / bk
        if (on) {
            const bool isq = i < RQ;
            const int np = isq ? 4 : (NK2 - 4 * (i - RQ) < 4 ? NK2 - 4 * (i - RQ) : 4);
            const unsigned char * src = isq ? bq + i * 2048 : bk + (i - RQ) * 2048;
#pragma unroll
            for (int p = 0; p < 4; p++)                                  // a pair of heads is 512 contiguous bytes: 16 per lane
                if (p < np) cp_async16_s(slots + i * 2048 + p * 512, src + p * 512);
        }
        cp_async_commit();
    };
#pragma unroll
    for (int i = 0; i < R; i++) request(i, in_q, in_k, ntok > 0);
    wsm[tid] = __ldg(A.par + tid); wsm[128 + tid] = __ldg(A.par + 128 + tid);
    if (tid < 64) freq[tid] = A.yarn ? __ldg(A.par + 258 + tid) : cam_powi(__ldg(A.par + 256), tid);
    const float eps = __ldg(A.par + 257), mscale = A.yarn ? __ldg(A.par + 322) : 1.0f;
    __syncthreads();
    const float f0 = freq[4 * l16 + 2 * hw], f1 = freq[4 * l16 + 2 * hw + 1];      // this half-warp's two of the lane's four angles
    f32x2 wq2[4], wk2[4];                                                // the lane's weights: dims (0, 1), (2, 3), (64, 65), (66, 67) + 4 l16
    {
        const float4 a = *reinterpret_cast<const float4 *>(wsm + 4 * l16), b = *reinterpret_cast<const float4 *>(wsm + 64 + 4 * l16);
        const float4 c = *reinterpret_cast<const float4 *>(wsm + 128 + 4 * l16), e = *reinterpret_cast<const float4 *>(wsm + 192 + 4 * l16);
        wq2[0] = pk2(a.x, a.y); wq2[1] = pk2(a.z, a.w); wq2[2] = pk2(b.x, b.y); wq2[3] = pk2(b.z, b.w);
        wk2[0] = pk2(c.x, c.y); wk2[1] = pk2(c.z, c.w); wk2[2] = pk2(e.x, e.y); wk2[3] = pk2(e.z, e.w);
    }
    const bool up8 = l16 & 8, up4 = l16 & 4;
    int t = tw;
    for (int k = 0; k < ntok; k++, t += stride) {
        f32x2 cc[2], sn[2], nsn[2];                                      // cos, sin, -sin of dims (4 l16, + 1) and (+ 2, + 3)
        {
            const float pos = (float)(A.pos0 + t);
            float s0, c0, s1, c1;
            cam_sincos(fmul(pos, f0), s0, c0); cam_sincos(fmul(pos, f1), s1, c1);
            if (A.yarn) { c0 = fmul(c0, mscale); s0 = fmul(s0, mscale); c1 = fmul(c1, mscale); s1 = fmul(s1, mscale); }
            const float oc0 = __shfl_xor_sync(CAM_FULL, c0, 16), os0 = __shfl_xor_sync(CAM_FULL, s0, 16);
            const float oc1 = __shfl_xor_sync(CAM_FULL, c1, 16), os1 = __shfl_xor_sync(CAM_FULL, s1, 16);
            const float ca = hw ? oc0 : c0, cb = hw ? oc1 : c1, cc_ = hw ? c0 : oc0, cd = hw ? c1 : oc1;      // dims 0, 1 come from the lower half-warp
            const float sa = hw ? os0 : s0, sb = hw ? os1 : s1, sc_ = hw ? s0 : os0, sd = hw ? s1 : os1;
            cc[0] = pk2(ca, cb); cc[1] = pk2(cc_, cd); sn[0] = pk2(sa, sb); sn[1] = pk2(sc_, sd); nsn[0] = pk2(-sa, -sb); nsn[1] = pk2(-sc_, -sd);
        }
        const bool more = k + 1 < ntok;
        const unsigned char * nq = in_q + qstep, * nk = in_k + kstep;      // the warp's next token
#pragma unroll
        for (int i = 0; i < R; i++) {
            cp_async_wait<R - 1>();                                      // this lane's copies of round i have landed (R groups are always outstanding)
            __syncwarp();                                                // .. and every other lane's
            const bool isq = i < RQ;
            const int np = isq ? 4 : (NK2 - 4 * (i - RQ) < 4 ? NK2 - 4 * (i - RQ) : 4);
            f32x2 xl[4][2], xh[4][2]; float ss[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                if (p < np) {
                    const uint2 vlo = lds64(ring + i * 2048 + p * 512), vhi = lds64(ring + i * 2048 + p * 512 + 128);
                    const float2 a = h2_to_f2(vlo.x), b = h2_to_f2(vlo.y), c = h2_to_f2(vhi.x), e = h2_to_f2(vhi.y);
                    // the head's sum of squares: per lane an fma chain over its 4 low and its 4 high dims, added
                    float sl = ffma(a.x, a.x, 0.0f), sh = ffma(c.x, c.x, 0.0f);
                    sl = ffma(a.y, a.y, sl); sh = ffma(c.y, c.y, sh); sl = ffma(b.x, b.x, sl); sh = ffma(e.x, e.x, sh); sl = ffma(b.y, b.y, sl); sh = ffma(e.y, e.y, sh);
                    ss[p] = fadd(sl, sh);
                    xl[p][0] = pk2(a.x, a.y); xl[p][1] = pk2(b.x, b.y); xh[p][0] = pk2(c.x, c.y); xh[p][1] = pk2(e.x, e.y);
                } else ss[p] = 0.0f;
            }
            __syncwarp();                                                // every lane has read its pieces of the slot
            request(i, nq, nk, more);                                    // this round of the next token into it
            // the half-warp sums of the four heads: partner 8 (a lane keeps heads 0, 1 or 2, 3), partner 4 (one head), partners 2, 1
            float scale[4];
            if (np > 2) {
                const float g0 = __shfl_xor_sync(CAM_FULL, up8 ? ss[0] : ss[2], 8), g1 = __shfl_xor_sync(CAM_FULL, up8 ? ss[1] : ss[3], 8);
                const float k0 = fadd(up8 ? ss[2] : ss[0], g0), k1 = fadd(up8 ? ss[3] : ss[1], g1);      // heads (0, 1) or (2, 3)
                const float g2 = __shfl_xor_sync(CAM_FULL, up4 ? k0 : k1, 4);
                float tot = fadd(up4 ? k1 : k0, g2);                         // head 2 up8 + up4 of the four
                tot = fadd(tot, __shfl_xor_sync(CAM_FULL, tot, 2));
                tot = fadd(tot, __shfl_xor_sync(CAM_FULL, tot, 1));
                const float sc = cam_rsqrt(fadd(fmul(tot, 0.0078125f), eps));      // tot / 128: the same bits as the division
#pragma unroll
                for (int p = 0; p < 4; p++) scale[p] = __shfl_sync(CAM_FULL, sc, 16 * hw + 4 * p);      // head p's lanes: l16 = 4 p ..
            } else {
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if (p < np) {
                        float tot = ss[p];
#pragma unroll
                        for (int o = 8; o > 0; o >>= 1) tot = fadd(tot, __shfl_xor_sync(CAM_FULL, tot, o));
                        scale[p] = cam_rsqrt(fadd(fmul(tot, 0.0078125f), eps));
                    }
                }
            }
            unsigned char * const o = isq ? out_q + i * 2048 : out_k + (i - RQ) * 2048;
#pragma unroll
            for (int p = 0; p < 4; p++) {
                if (p < np) {
                    const f32x2 s2 = pk2(scale[p], scale[p]);
                    uint32_t olo[2], ohi[2];
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        const f32x2 x0 = mul2(mul2(s2, xl[p][c]), isq ? wq2[c] : wk2[c]), x1 = mul2(mul2(s2, xh[p][c]), isq ? wq2[2 + c] : wk2[2 + c]);
                        const f32x2 ylo = fma2(x0, cc[c], mul2(x1, nsn[c])), yhi = fma2(x1, cc[c], mul2(x0, sn[c]));
                        olo[c] = f2_to_h2(lo2(ylo), hi2(ylo)); ohi[c] = f2_to_h2(lo2(yhi), hi2(yhi));
                    }
                    st64_stream(o + p * 512, make_uint2(olo[0], olo[1]));
                    st64_stream(o + p * 512 + 128, make_uint2(ohi[0], ohi[1]));
                }
            }
        }
        in_q = nq; in_k = nk; out_q += qstep; out_k += kstep;
    }
    cp_async_wait<0>();
}

// ---- the reference's signature (fp32 qkv rows in; q16 and the KV cache row out) with the token-shaped mapping --------------------------
// As qk_rope_f16_tok_kernel: a warp owns a token and walks its q rounds, its k rounds and then its v rounds of four pairs of heads,
// unrolled. A pair of fp32 heads is 1024 bytes (two 16-byte cp.async per lane); the ring has two slots of a round each, the next round
// requested while this one is computed. q heads go to q16, k heads into the K half of cache row pos0 + t, v heads are rounded to fp16
// into its V half. Q8: the Q8_0 cache form (csrc/kv_q8.cuh): every q and k head is rounded to fp16, transformed (Hadamard-128) and
// stored as fp16 (q16) or as four Q8_0 blocks (K); V as four Q8_0 blocks of its fp16-rounded values.
CAM_DEV float4 lds128f(uint32_t smem_addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(smem_addr));
    return v;
}

template <int NQ2, int NK2, bool Q8>
__global__ void __launch_bounds__(128) qk_rope_cache_tok_kernel(const RopeArgs A) {
    constexpr int RQ = NQ2 / 4, RK = (NK2 + 3) / 4, R = RQ + 2 * RK;
    static_assert(NQ2 % 4 == 0 && (NK2 <= 4 || NK2 % 4 == 0), "rounds of four pairs of heads");
    __shared__ __align__(16) float wsm[256], freq[64];
    __shared__ __align__(16) unsigned char ring_all[4 * 2 * 4096];       // [4 warps][2 slots][a round: 4 pairs x 1024 bytes]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hw = lane >> 4, l16 = lane & 15;
    const int tw = blockIdx.x * 4 + warp, stride = gridDim.x * 4;
    const int ntok = tw < A.n ? (A.n - tw + stride - 1) / stride : 0;
    const uint32_t slots = (uint32_t)__cvta_generic_to_shared(ring_all) + warp * 8192 + lane * 16;      // where this lane copies to
    const uint32_t mine = slots - lane * 16 + hw * 512 + l16 * 16;                                      // where it reads its low piece (the high piece: + 256)
    const size_t tstep = (size_t)stride * A.ldq * 4;                                                    // bytes between this warp's tokens
    const unsigned char * in = reinterpret_cast<const unsigned char *>(A.in0) + (size_t)tw * A.ldq * 4 + lane * 16;
    auto np_of = [&](int i) { return i < RQ ? 4 : ((i - RQ) % RK == RK - 1 && (NK2 & 3) ? (NK2 & 3) : 4); };      // pairs in round i
    auto src_of = [&](int i) { return i < RQ ? i * 4096 : (i < RQ + RK ? NQ2 * 1024 + (i - RQ) * 4096 : (NQ2 + NK2) * 1024 + (i - RQ - RK) * 4096); };
    auto request = [&](int i, const unsigned char * tok, uint32_t slot, bool on) {      // round i (a constant after unrolling) of the token at `tok`
        if (on) {
            const int np = np_of(i);
            const unsigned char * src = tok + src_of(i);
#pragma unroll
            for (int p = 0; p < 4; p++)
                if (p < np) { cp_async16_s(slots + slot + p * 1024, src + p * 1024); cp_async16_s(slots + slot + p * 1024 + 512, src + p * 1024 + 512); }
        }
        cp_async_commit();
    };
    request(0, in, 0, ntok > 0);
    wsm[tid] = __ldg(A.par + tid); wsm[128 + tid] = __ldg(A.par + 128 + tid);
    if (tid < 64) freq[tid] = A.yarn ? __ldg(A.par + 258 + tid) : cam_powi(__ldg(A.par + 256), tid);
    const float eps = __ldg(A.par + 257), mscale = A.yarn ? __ldg(A.par + 322) : 1.0f;
    __syncthreads();
    const float f0 = freq[4 * l16 + 2 * hw], f1 = freq[4 * l16 + 2 * hw + 1];
    f32x2 wq2[4], wk2[4];
    {
        const float4 a = *reinterpret_cast<const float4 *>(wsm + 4 * l16), b = *reinterpret_cast<const float4 *>(wsm + 64 + 4 * l16);
        const float4 c = *reinterpret_cast<const float4 *>(wsm + 128 + 4 * l16), e = *reinterpret_cast<const float4 *>(wsm + 192 + 4 * l16);
        wq2[0] = pk2(a.x, a.y); wq2[1] = pk2(a.z, a.w); wq2[2] = pk2(b.x, b.y); wq2[3] = pk2(b.z, b.w);
        wk2[0] = pk2(c.x, c.y); wk2[1] = pk2(c.z, c.w); wk2[2] = pk2(e.x, e.y); wk2[3] = pk2(e.z, e.w);
    }
    const bool up8 = l16 & 8, up4 = l16 & 4;
    uint32_t cur = 0;                                                    // the ring slot (byte offset 0 / 4096) that holds the round being computed
    int t = tw;
    for (int k = 0; k < ntok; k++, t += stride) {
        f32x2 cc[2], sn[2], nsn[2];
        {
            const float pos = (float)(A.pos0 + t);
            float s0, c0, s1, c1;
            cam_sincos(fmul(pos, f0), s0, c0); cam_sincos(fmul(pos, f1), s1, c1);
            if (A.yarn) { c0 = fmul(c0, mscale); s0 = fmul(s0, mscale); c1 = fmul(c1, mscale); s1 = fmul(s1, mscale); }
            const float oc0 = __shfl_xor_sync(CAM_FULL, c0, 16), os0 = __shfl_xor_sync(CAM_FULL, s0, 16);
            const float oc1 = __shfl_xor_sync(CAM_FULL, c1, 16), os1 = __shfl_xor_sync(CAM_FULL, s1, 16);
            const float ca = hw ? oc0 : c0, cb = hw ? oc1 : c1, cc_ = hw ? c0 : oc0, cd = hw ? c1 : oc1;
            const float sa = hw ? os0 : s0, sb = hw ? os1 : s1, sc_ = hw ? s0 : os0, sd = hw ? s1 : os1;
            cc[0] = pk2(ca, cb); cc[1] = pk2(cc_, cd); sn[0] = pk2(sa, sb); sn[1] = pk2(sc_, sd); nsn[0] = pk2(-sa, -sb); nsn[1] = pk2(-sc_, -sd);
        }
        const bool more = k + 1 < ntok;
        const unsigned char * nxt = in + tstep;
        const int pos = A.pos0 + t;
        uint16_t * const qrow = A.out0 + (size_t)t * NQ2 * 256 + hw * 128 + 4 * l16;
        uint16_t * const krow = A.out1 + (size_t)pos * NK2 * 512 + hw * 128 + 4 * l16;                      // F16 cache: K [nkv][128] | V [nkv][128]
        uint8_t * const cw = reinterpret_cast<uint8_t *>(A.out1) + (size_t)pos * (NK2 * 4 * 4 * 34) + (size_t)hw * 4 * 34 + (size_t)(l16 >> 3) * 34;   // Q8: K blocks | V blocks
#pragma unroll
        for (int i = 0; i < R; i++) {
            // the next round (of this token, or the first of the next) into the other slot, then wait for this round's copies
            if (i + 1 < R) request(i + 1, in, cur ^ 4096u, true); else request(0, nxt, cur ^ 4096u, more);
            cp_async_wait<1>();
            __syncwarp();
            const int np = np_of(i);
            const bool isq = i < RQ, isk = !isq && i < RQ + RK;
            const int h0 = isq ? 8 * i : (isk ? 8 * (i - RQ) : 8 * (i - RQ - RK));      // the round's first head within its kind
            if (isq || isk) {
                f32x2 xl[4][2], xh[4][2]; float ss[4];
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if (p < np) {
                        const float4 a = lds128f(mine + cur + p * 1024), c = lds128f(mine + cur + p * 1024 + 256);
                        float sl = ffma(a.x, a.x, 0.0f), sh = ffma(c.x, c.x, 0.0f);
                        sl = ffma(a.y, a.y, sl); sh = ffma(c.y, c.y, sh); sl = ffma(a.z, a.z, sl); sh = ffma(c.z, c.z, sh); sl = ffma(a.w, a.w, sl); sh = ffma(c.w, c.w, sh);
                        ss[p] = fadd(sl, sh);
                        xl[p][0] = pk2(a.x, a.y); xl[p][1] = pk2(a.z, a.w); xh[p][0] = pk2(c.x, c.y); xh[p][1] = pk2(c.z, c.w);
                    } else ss[p] = 0.0f;
                }
                float scale[4];
                if (np > 2) {
                    const float g0 = __shfl_xor_sync(CAM_FULL, up8 ? ss[0] : ss[2], 8), g1 = __shfl_xor_sync(CAM_FULL, up8 ? ss[1] : ss[3], 8);
                    const float k0 = fadd(up8 ? ss[2] : ss[0], g0), k1 = fadd(up8 ? ss[3] : ss[1], g1);
                    const float g2 = __shfl_xor_sync(CAM_FULL, up4 ? k0 : k1, 4);
                    float tot = fadd(up4 ? k1 : k0, g2);
                    tot = fadd(tot, __shfl_xor_sync(CAM_FULL, tot, 2));
                    tot = fadd(tot, __shfl_xor_sync(CAM_FULL, tot, 1));
                    const float sc = cam_rsqrt(fadd(fmul(tot, 0.0078125f), eps));
#pragma unroll
                    for (int p = 0; p < 4; p++) scale[p] = __shfl_sync(CAM_FULL, sc, 16 * hw + 4 * p);
                } else {
#pragma unroll
                    for (int p = 0; p < 4; p++)
                        if (p < np) {
                            float tot = ss[p];
#pragma unroll
                            for (int o = 8; o > 0; o >>= 1) tot = fadd(tot, __shfl_xor_sync(CAM_FULL, tot, o));
                            scale[p] = cam_rsqrt(fadd(fmul(tot, 0.0078125f), eps));
                        }
                }
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if (p < np) {
                        const f32x2 s2 = pk2(scale[p], scale[p]);
                        f32x2 ylo[2], yhi[2];
#pragma unroll
                        for (int c = 0; c < 2; c++) {
                            const f32x2 x0 = mul2(mul2(s2, xl[p][c]), isq ? wq2[c] : wk2[c]), x1 = mul2(mul2(s2, xh[p][c]), isq ? wq2[2 + c] : wk2[2 + c]);
                            ylo[c] = fma2(x0, cc[c], mul2(x1, nsn[c])); yhi[c] = fma2(x1, cc[c], mul2(x0, sn[c]));
                        }
                        const int head = h0 + 2 * p;                     // (+ hw: inside the row pointers)
                        if (!Q8) {
                            uint16_t * o = (isq ? qrow : krow) + head * 128;
                            st64_stream(o, make_uint2(f2_to_h2(lo2(ylo[0]), hi2(ylo[0])), f2_to_h2(lo2(ylo[1]), hi2(ylo[1]))));
                            st64_stream(o + 64, make_uint2(f2_to_h2(lo2(yhi[0]), hi2(yhi[0])), f2_to_h2(lo2(yhi[1]), hi2(yhi[1]))));
                        } else {
                            float y[8] = {f16r(lo2(ylo[0])), f16r(hi2(ylo[0])), f16r(lo2(ylo[1])), f16r(hi2(ylo[1])),
                                          f16r(lo2(yhi[0])), f16r(hi2(yhi[0])), f16r(lo2(yhi[1])), f16r(hi2(yhi[1]))};
                            hadamard128(y, l16);
                            if (isq) {
                                uint16_t * o = qrow + head * 128;
                                st64_stream(o, make_uint2(f2_to_h2(y[0], y[1]), f2_to_h2(y[2], y[3])));
                                st64_stream(o + 64, make_uint2(f2_to_h2(y[4], y[5]), f2_to_h2(y[6], y[7])));
                            } else {
                                uint8_t * kb = cw + (size_t)head * 4 * 34;
                                const float klo[4] = {y[0], y[1], y[2], y[3]}, khi[4] = {y[4], y[5], y[6], y[7]};
                                q8_0_store(klo, kb, l16 & 7, A.err, true);
                                q8_0_store(khi, kb + 2 * 34, l16 & 7, A.err, true);
                            }
                        }
                    }
                }
            } else {                                                     // v heads: rounded to fp16 (Q8: then Q8_0 blocks)
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if (p < np) {
                        const float4 a = lds128f(mine + cur + p * 1024), c = lds128f(mine + cur + p * 1024 + 256);
                        const int head = h0 + 2 * p;
                        if (!Q8) {
                            uint16_t * o = krow + NK2 * 256 + head * 128;
                            st64_stream(o, make_uint2(f2_to_h2(a.x, a.y), f2_to_h2(a.z, a.w)));
                            st64_stream(o + 64, make_uint2(f2_to_h2(c.x, c.y), f2_to_h2(c.z, c.w)));
                        } else {
                            uint8_t * vb = cw + (size_t)NK2 * 2 * 4 * 34 + (size_t)head * 4 * 34;
                            const float vlo[4] = {f16r(a.x), f16r(a.y), f16r(a.z), f16r(a.w)}, vhi[4] = {f16r(c.x), f16r(c.y), f16r(c.z), f16r(c.w)};
                            q8_0_store(vlo, vb, l16 & 7, A.err, true);
                            q8_0_store(vhi, vb + 2 * 34, l16 & 7, A.err, true);
                        }
                    }
                }
            }
            __syncwarp();                                                // every lane has read the slot before the next request overwrites it
            cur ^= 4096u;
        }
        in = nxt;
    }
    cp_async_wait<0>();
}

// warps per block (4 .. 12) and heads per half-warp and round (1 .. 4): the pair with the fewest idle half-warp slots over a
// token's H heads; among equals the most heads per round (one scale computation serves 2 P heads), then the most warps
void pick_shape(int H, int & warps, int & P) {
    if (const char * e = getenv("CAMINUS_B200_ROPE_SHAPE")) {      // "warps,P": overrides the choice (tuning)
        int w = 0, p = 0;
        if (sscanf(e, "%d,%d", &w, &p) == 2 && w >= 4 && w <= 12 && p >= 1 && p <= 4) { warps = w; P = p; return; }
    }
    int waste = 1 << 30;
    warps = 8; P = 1;
    for (int p = 4; p >= 1; p--)
        for (int w = 12; w >= 4; w--) {
            const int per_round = 2 * w * p;
            const int idle = (H + per_round - 1) / per_round * per_round - H;
            if (idle < waste) { waste = idle; warps = w; P = p; }
        }
}

template <typename T, bool CACHE, int P, bool ONE, bool Q8>
int launch_rope_p(const RopeArgs & A, int warps, size_t smem, cudaStream_t stream) {
    static unsigned long long allowed = 0;
    const cudaError_t e = cam_allow_smem(qk_rope_kernel<T, CACHE, P, ONE, Q8>, 227 * 1024, allowed);
    if (e != cudaSuccess) return (int)e;
    const int grid = cam_resident_grid(qk_rope_kernel<T, CACHE, P, ONE, Q8>, warps * 32, smem, A.n);
    qk_rope_kernel<T, CACHE, P, ONE, Q8><<<grid, warps * 32, smem, stream>>>(A);
    return (int)cudaGetLastError();
}

template <typename T, bool CACHE, bool Q8 = false>
int launch_rope(const RopeArgs & A, cudaStream_t stream) {
    const int H = A.nh + A.nkv;
    const int in_heads = CACHE ? A.nh + 2 * A.nkv : H;
    const size_t smem = (128 + 128 + 64 + 2 * 64 * ROPE_STAGES) * 4 + ROPE_STAGES * (size_t)in_heads * 128 * sizeof(T);
    if (smem > 227 * 1024) return CAM_ERR_SHAPE;
    int warps, P;
    pick_shape(H, warps, P);
    const bool one = H == 2 * warps * P;
#define CAM_ROPE_CASE(PV) \
    case PV: return one ? launch_rope_p<T, CACHE, PV, true, Q8>(A, warps, smem, stream) : launch_rope_p<T, CACHE, PV, false, Q8>(A, warps, smem, stream);
    switch (P) {
        CAM_ROPE_CASE(1) CAM_ROPE_CASE(2) CAM_ROPE_CASE(3)
        default: return one ? launch_rope_p<T, CACHE, 4, true, Q8>(A, warps, smem, stream) : launch_rope_p<T, CACHE, 4, false, Q8>(A, warps, smem, stream);
    }
#undef CAM_ROPE_CASE
}

// the token-shaped kernel of the reference's signature for the head counts it is built for; CAM_ERR_SHAPE: the caller's staged kernel
template <bool Q8>
int launch_cache_tok(const RopeArgs & A, cudaStream_t stream) {
    if (const char * e = getenv("CAMINUS_B200_ROPE_STAGED")) { if (e[0] == '1') return CAM_ERR_SHAPE; }      // (tuning: the staged kernel)
    const long blocks = ((long)A.n + 3) / 4;
    const char * grid_mode = getenv("CAMINUS_B200_ROPE_GRID");       // (tuning: "full" / "resident")
#define CAM_ROPE_CTOK(NQ2V, NK2V)                                                                                                  \
    if (A.nh == 2 * NQ2V && A.nkv == 2 * NK2V) {                                                                                   \
        const int cap = cam_resident_grid(qk_rope_cache_tok_kernel<NQ2V, NK2V, Q8>, 128, 0, blocks);                               \
        const bool full = grid_mode ? grid_mode[0] == 'f' : blocks > 2L * cap;                                                     \
        qk_rope_cache_tok_kernel<NQ2V, NK2V, Q8><<<full ? (int)blocks : cap, 128, 0, stream>>>(A);                                 \
        return (int)cudaGetLastError();                                                                                            \
    }
    CAM_ROPE_CTOK(16, 2) CAM_ROPE_CTOK(32, 4) CAM_ROPE_CTOK(20, 4) CAM_ROPE_CTOK(16, 4)
#undef CAM_ROPE_CTOK
    return CAM_ERR_SHAPE;
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
    const RopeArgs A = {qkv, nullptr, par, (uint16_t *)q16, (uint16_t *)cache, ldq, nh, nkv, pos0, n, yarn, nullptr};
    const int r2 = launch_cache_tok<false>(A, (cudaStream_t)stream);
    return r2 != CAM_ERR_SHAPE ? r2 : launch_rope<float, true>(A, (cudaStream_t)stream);
}
extern "C" int q3p_qk_rope(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                           void * stream) {
    return qk_rope_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, 0, stream);
}
extern "C" int q3p_qk_rope_yarn(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16,
                                void * cache, void * stream) {
    return qk_rope_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, 1, stream);
}

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
    const RopeArgs A = {qkv, nullptr, par, (uint16_t *)q16, (uint16_t *)cache, ldq, nh, nkv, pos0, n, yarn, err};
    const int r2 = launch_cache_tok<true>(A, (cudaStream_t)stream);
    return r2 != CAM_ERR_SHAPE ? r2 : launch_rope<float, true, true>(A, (cudaStream_t)stream);
}
extern "C" int q3p_qk_rope_q8(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache, int * err,
                              void * stream) {
    return rope_q8_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, err, 0, stream);
}
extern "C" int q3p_qk_rope_q8_yarn(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                                   int * err, void * stream) {
    return rope_q8_entry(n, qkv, ldq, nh, nkv, par, pos0, q16, cache, err, 1, stream);
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
    const RopeArgs A = {q, k, par, (uint16_t *)qo, (uint16_t *)ko, 0, nh, nkv, pos0, n, yarn, nullptr};
    if (const char * e = getenv("CAMINUS_B200_ROPE_STAGED")) { if (e[0] == '1') return launch_rope<uint16_t, false>(A, (cudaStream_t)stream); }      // (tuning: the staged kernel)
    // a warp per token, heads 8 at a time; as many blocks of four warps as the device holds at once, or as the tokens need
    if ((nh & 1) || (nkv & 1)) return launch_rope<uint16_t, false>(A, (cudaStream_t)stream);       // (a pair of heads must be whole: odd counts take the staged kernel)
    const long blocks = ((long)n + 3) / 4;
    cudaStream_t st = (cudaStream_t)stream;
    const char * pick = getenv("CAMINUS_B200_ROPE_P");               // (tuning: 2 / 4 = the generic warp kernel with that many pairs per round)
    // the shapes with a compile-time token layout (Qwen3: 32 + 4, 64 + 8, 40 + 8 and 32 + 8 heads)
    // Grid: a block per four tokens when that is more than twice what the device holds at once (measured at 65536 tokens: 358 us against
    // 409 us for a resident grid whose warps loop over tokens; a finished block's successor starts with a whole token of copies in
    // flight), else exactly the resident blocks, the warps taking a second token where there are more tokens than warps (measured at
    // 4096 tokens of 36 heads: 16.5 us against 18.8 us).
#define CAM_ROPE_TOK(NQ2V, NK2V)                                                                                                   \
    if (!pick && nh == 2 * NQ2V && nkv == 2 * NK2V) {                                                                              \
        static unsigned long long allowed = 0;                                                                                     \
        constexpr size_t smem = 4 * (NQ2V / 4 + (NK2V + 3) / 4) * 2048;                                                            \
        const cudaError_t e = cam_allow_smem(qk_rope_f16_tok_kernel<NQ2V, NK2V>, smem, allowed);                                   \
        if (e != cudaSuccess) return (int)e;                                                                                       \
        const int cap = cam_resident_grid(qk_rope_f16_tok_kernel<NQ2V, NK2V>, 128, smem, blocks);                                  \
        const bool full = grid_mode ? grid_mode[0] == 'f' : blocks > 2L * cap;                                                     \
        qk_rope_f16_tok_kernel<NQ2V, NK2V><<<full ? (int)blocks : cap, 128, smem, st>>>(A);                                        \
        return (int)cudaGetLastError();                                                                                            \
    }
    const char * grid_mode = getenv("CAMINUS_B200_ROPE_GRID");       // (tuning: "full" / "resident")
    CAM_ROPE_TOK(16, 2) CAM_ROPE_TOK(32, 4) CAM_ROPE_TOK(20, 4) CAM_ROPE_TOK(16, 4)
#undef CAM_ROPE_TOK
    // other shapes: heads per round 8 (one scale computation per four pairs of heads, 20 resident warps per multiprocessor) when every
    // warp gets many tokens, else 4 (32 resident warps: a batch of a few thousand tokens is one token per warp in a single wave)
    const int g4 = cam_resident_grid(qk_rope_f16_warp_kernel<4>, 128, 0, blocks);
    int P = blocks >= 8L * g4 ? 4 : 2;
    if (pick && (pick[0] == '2' || pick[0] == '4')) P = pick[0] - '0';
    if (P == 4) qk_rope_f16_warp_kernel<4><<<g4, 128, 0, st>>>(A);
    else qk_rope_f16_warp_kernel<2><<<cam_resident_grid(qk_rope_f16_warp_kernel<2>, 128, 0, blocks), 128, 0, st>>>(A);
    return (int)cudaGetLastError();
}
