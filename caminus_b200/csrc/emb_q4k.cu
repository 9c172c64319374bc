// Q4_K embedding rows: gather + dequantise (the reference's q3p_emb, kernels/q3m_prefill.hip:362-380; its T = 1 form
// own_op_emb, kernels/k3_own_ops.h:273-304; the host decoder own_dequant.q4_k, python/caminus/own_dequant.py:19-37).
//
// A Q4_K super-block is 144 bytes for 256 values: fp16 d, fp16 dmin, 12 bytes of packed 6-bit scales / mins, 128 bytes of
// nibbles (sub-blocks 2k and 2k + 1 are the low and high nibbles of bytes 32k .. 32k + 31). Value j of a block:
//   y = fl(fl(fl(d * sc) * q) - fl(dmin * m))        three roundings, no fma: the host decoder's bits.
//
// Mapping: a warp takes one row's super-blocks, EMB_NB at a time (a row of 2048 values is one such group): the token id is read once,
// the 3 EMB_NB loads of the group (a 16-byte header and two 32-bit nibble words per super-block and lane) are all issued before the first
// value is decoded, and the grid is rows x groups, so no index is divided. Within a super-block lane l writes values 4l .. 4l + 3 and
// 128 + 4l .. 128 + 4l + 3 (two 16-byte stores, the warp's stores cover 512 contiguous bytes each). Both groups of four lie in one
// sub-block each (l >> 3 and 4 + (l >> 3)), so a lane needs one scale / min pair per group, and its nibbles are one aligned 32-bit word
// per group. The two products and the subtraction of neighbouring values run as packed fp32 instructions (the same roundings).
// HBM traffic per row of N values: 4 (id) + 144 N / 256 (blocks) + 4 N (output): the kernel is store-bound.
#include "cam_common.cuh"

namespace {

constexpr int EMB_WARPS = 8, EMB_NB = 8;

__global__ void __launch_bounds__(EMB_WARPS * 32) emb_q4k_kernel(const uint8_t * __restrict__ W, int rb, int vocab,
                                                                 const int * __restrict__ toks, float * __restrict__ x, int N, int n) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = N >> 8, b0 = blockIdx.y * EMB_NB;
    const int sb0 = lane >> 3;                       // sub-block of the first group (the second is sb0 + 4)
    const int sh = 8 * sb0;                          // its byte in a scale word
    const int nib = 4 * (sb0 & 1);                   // low or high nibble
    const int qoff = 16 + (lane >> 4) * 32 + 4 * (lane & 7);
    const f32x2 bias = pk2(-8388608.0f, -8388608.0f);
    for (int t = blockIdx.x * EMB_WARPS + warp; t < n; t += gridDim.x * EMB_WARPS) {
        const int tok = min(max(__ldg(toks + t), 0), vocab - 1);
        const uint8_t * row = W + (size_t)tok * rb + (size_t)b0 * 144;
        uint4 hdr[EMB_NB]; uint32_t w0[EMB_NB], w1[EMB_NB];
#pragma unroll
        for (int j = 0; j < EMB_NB; j++)
            if (b0 + j < nblk) {
                const uint8_t * blk = row + j * 144;
                hdr[j] = ldg128(blk);
                w0[j] = __ldg(reinterpret_cast<const uint32_t *>(blk + qoff));
                w1[j] = __ldg(reinterpret_cast<const uint32_t *>(blk + qoff + 64));
            }
        float * o = x + (size_t)t * N + (size_t)b0 * 256 + 4 * lane;
#pragma unroll
        for (int j = 0; j < EMB_NB; j++)
            if (b0 + j < nblk) {
                const float2 dd = h2_to_f2(hdr[j].x);                            // (d, dmin)
                const uint32_t s_lo = (hdr[j].y >> sh) & 0xffu, s_mid = (hdr[j].z >> sh) & 0xffu, s_hi = (hdr[j].w >> sh) & 0xffu;   // s[sb0], s[sb0 + 4], s[sb0 + 8]
                const uint32_t sc0 = s_lo & 63u, m0 = s_mid & 63u;
                const uint32_t sc1 = (s_hi & 0xfu) | ((s_lo >> 6) << 4), m1 = (s_hi >> 4) | ((s_mid >> 6) << 4);
                const float dl0 = fmul(dd.x, (float)sc0), ml0 = -fmul(dd.y, (float)m0);
                const float dl1 = fmul(dd.x, (float)sc1), ml1 = -fmul(dd.y, (float)m1);
                // nibble c of a word as a float: its byte is placed under the exponent of 2^23 (one byte permute), then 2^23 is
                // subtracted: exact for 0 .. 15, and two operations instead of shift, mask and convert
                const uint32_t n0 = (w0[j] >> nib) & 0x0f0f0f0fu, n1 = (w1[j] >> nib) & 0x0f0f0f0fu;
                const f32x2 d0 = pk2(dl0, dl0), d1 = pk2(dl1, dl1), c0 = pk2(ml0, ml0), c1 = pk2(ml1, ml1);
                // y = fl(fl(dl q) - ml): the subtraction as the addition of -ml (the same rounding). dl q is exact (dl = an fp16 times an integer
                // below 64: 17 bits; q below 16), so a product contracted into the addition by the assembler gives the same bits
                const f32x2 a0 = add2(mul2(d0, add2(pk2(__uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7440)), __uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7441))), bias)), c0);
                const f32x2 a1 = add2(mul2(d0, add2(pk2(__uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7442)), __uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7443))), bias)), c0);
                const f32x2 e0 = add2(mul2(d1, add2(pk2(__uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7440)), __uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7441))), bias)), c1);
                const f32x2 e1 = add2(mul2(d1, add2(pk2(__uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7442)), __uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7443))), bias)), c1);
                __stcs(reinterpret_cast<float4 *>(o + j * 256), make_float4(lo2(a0), hi2(a0), lo2(a1), hi2(a1)));
                __stcs(reinterpret_cast<float4 *>(o + j * 256 + 128), make_float4(lo2(e0), hi2(e0), lo2(e1), hi2(e1)));
            }
    }
}

}   // namespace

// q3p_emb: x [n][N] fp32 = rows toks[i] (clamped to [0, vocab)) of the Q4_K table W (rb bytes per row). n is the reference's
// grid.x. Reference: kernels/q3m_prefill.hip:364-365; wrapper python/caminus/prefill/q3m_ops.py:86-87.
extern "C" int q3p_emb(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, void * stream) {
    if (n < 0 || vocab < 1 || N < 256 || (N & 255) || rb < (N >> 8) * 144 || !W || !toks || !x) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (!cam_aligned16(W) || (rb & 15) || !cam_aligned16(x) || (reinterpret_cast<uintptr_t>(toks) & 3u)) return CAM_ERR_ALIGN;
    const int groups = ((N >> 8) + EMB_NB - 1) / EMB_NB;                             // grid.y: a row's super-blocks, EMB_NB per warp
    if (groups > 65535) return CAM_ERR_SHAPE;
    const long want = ((long)n + EMB_WARPS - 1) / EMB_WARPS;
    const int cap = cam_resident_grid(emb_q4k_kernel, EMB_WARPS * 32, 0, want * groups);
    const int gx = (int)(want < (cap + groups - 1) / groups ? want : (cap + groups - 1) / groups);
    emb_q4k_kernel<<<dim3(gx < 1 ? 1 : gx, groups), EMB_WARPS * 32, 0, (cudaStream_t)stream>>>((const uint8_t *)W, rb, vocab, toks, x, N, n);
    return (int)cudaGetLastError();
}
