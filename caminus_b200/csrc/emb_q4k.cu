// Q4_K embedding rows: gather + dequantise (the reference's q3p_emb, kernels/q3m_prefill.hip:362-380; its T = 1 form
// own_op_emb, kernels/k3_own_ops.h:273-304; the host decoder own_dequant.q4_k, python/caminus/own_dequant.py:19-37).
//
// A Q4_K super-block is 144 bytes for 256 values: fp16 d, fp16 dmin, 12 bytes of packed 6-bit scales / mins, 128 bytes of
// nibbles (sub-blocks 2k and 2k + 1 are the low and high nibbles of bytes 32k .. 32k + 31). Value j of a block:
//   y = fl(fl(fl(d * sc) * q) - fl(dmin * m))        three roundings, no fma: the host decoder's bits.
//
// Mapping: one warp per super-block. Lane l writes values 4l .. 4l + 3 and 128 + 4l .. 128 + 4l + 3 (two 16-byte stores, the
// warp's stores cover 512 contiguous bytes each). Both groups lie in one sub-block each (l >> 3 and 4 + (l >> 3)), so a lane
// needs one scale / min pair per group, and its nibbles are one aligned 32-bit word per group. The header is one 16-byte
// load. HBM traffic per row of N values: 4 (id) + 144 N / 256 (blocks) + 4 N (output): the kernel is store-bound.
#include "cam_common.cuh"

namespace {

constexpr int EMB_WARPS = 8;

__global__ void __launch_bounds__(EMB_WARPS * 32) emb_q4k_kernel(const uint8_t * __restrict__ W, int rb, int vocab,
                                                                 const int * __restrict__ toks, float * __restrict__ x, int N, int n) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = N >> 8;
    const long total = (long)n * nblk;
    const int sb0 = lane >> 3;                       // sub-block of the first group (the second is sb0 + 4)
    const int sh = 8 * sb0;                          // its byte in a scale word
    const int nib = 4 * (sb0 & 1);                   // low or high nibble
    const int qoff = 16 + (lane >> 4) * 32 + 4 * (lane & 7);
    for (long task = (long)blockIdx.x * EMB_WARPS + warp; task < total; task += (long)gridDim.x * EMB_WARPS) {
        const int t = (int)(task / nblk), b = (int)(task - (long)t * nblk);
        const int tok = min(max(__ldg(toks + t), 0), vocab - 1);
        const uint8_t * blk = W + (size_t)tok * rb + (size_t)b * 144;
        const uint4 hdr = ldg128(blk);
        const uint32_t w0 = __ldg(reinterpret_cast<const uint32_t *>(blk + qoff));
        const uint32_t w1 = __ldg(reinterpret_cast<const uint32_t *>(blk + qoff + 64));
        const float2 dd = h2_to_f2(hdr.x);                                   // (d, dmin)
        const uint32_t s_lo = (hdr.y >> sh) & 0xffu, s_mid = (hdr.z >> sh) & 0xffu, s_hi = (hdr.w >> sh) & 0xffu;   // s[sb0], s[sb0 + 4], s[sb0 + 8]
        const uint32_t sc0 = s_lo & 63u, m0 = s_mid & 63u;
        const uint32_t sc1 = (s_hi & 0xfu) | ((s_lo >> 6) << 4), m1 = (s_hi >> 4) | ((s_mid >> 6) << 4);
        const float dl0 = fmul(dd.x, (float)sc0), ml0 = fmul(dd.y, (float)m0);
        const float dl1 = fmul(dd.x, (float)sc1), ml1 = fmul(dd.y, (float)m1);
        // nibble c of a word as a float: its byte is placed under the exponent of 2^23 (one byte permute), then 2^23 is
        // subtracted: exact for 0 .. 15, and two operations instead of shift, mask and convert
        const uint32_t n0 = (w0 >> nib) & 0x0f0f0f0fu, n1 = (w1 >> nib) & 0x0f0f0f0fu;
        float4 y0, y1;
        y0.x = fsub(fmul(dl0, fsub(__uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7440)), 8388608.0f)), ml0);
        y0.y = fsub(fmul(dl0, fsub(__uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7441)), 8388608.0f)), ml0);
        y0.z = fsub(fmul(dl0, fsub(__uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7442)), 8388608.0f)), ml0);
        y0.w = fsub(fmul(dl0, fsub(__uint_as_float(__byte_perm(n0, 0x4b000000u, 0x7443)), 8388608.0f)), ml0);
        y1.x = fsub(fmul(dl1, fsub(__uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7440)), 8388608.0f)), ml1);
        y1.y = fsub(fmul(dl1, fsub(__uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7441)), 8388608.0f)), ml1);
        y1.z = fsub(fmul(dl1, fsub(__uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7442)), 8388608.0f)), ml1);
        y1.w = fsub(fmul(dl1, fsub(__uint_as_float(__byte_perm(n1, 0x4b000000u, 0x7443)), 8388608.0f)), ml1);
        float * o = x + (size_t)t * N + (size_t)b * 256 + 4 * lane;
        __stcs(reinterpret_cast<float4 *>(o), y0);
        __stcs(reinterpret_cast<float4 *>(o + 128), y1);
    }
}

}   // namespace

// q3p_emb: x [n][N] fp32 = rows toks[i] (clamped to [0, vocab)) of the Q4_K table W (rb bytes per row). n is the reference's
// grid.x. Reference: kernels/q3m_prefill.hip:364-365; wrapper python/caminus/prefill/q3m_ops.py:86-87.
extern "C" int q3p_emb(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, void * stream) {
    if (n < 0 || vocab < 1 || N < 256 || (N & 255) || rb < (N >> 8) * 144 || !W || !toks || !x) return CAM_ERR_ARG;
    if (n == 0) return CAM_OK;
    if (!cam_aligned16(W) || (rb & 15) || !cam_aligned16(x) || (reinterpret_cast<uintptr_t>(toks) & 3u)) return CAM_ERR_ALIGN;
    const long total = (long)n * (N >> 8);
    const long want = (total + EMB_WARPS - 1) / EMB_WARPS;
    const int grid = cam_resident_grid(emb_q4k_kernel, EMB_WARPS * 32, 0, want);
    emb_q4k_kernel<<<grid, EMB_WARPS * 32, 0, (cudaStream_t)stream>>>((const uint8_t *)W, rb, vocab, toks, x, N, n);
    return (int)cudaGetLastError();
}
