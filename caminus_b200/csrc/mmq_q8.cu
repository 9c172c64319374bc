// Q8_1 activations in the MMQ layout the quantised GEMMs read (the reference's block_q8_1_mmq, kernels/ggml_mmq/mmq.cuh:63-82):
// a row of K values is cut into blocks of 128; block (kb, row) is stored at index kb * rows + row (column-major by K-block)
// as 144 bytes: 16 bytes of per-32 scales, then 128 int8. Algebra of the reference's quantiser (kernels/ggml_mmq/quantize_mmq.cuh:41-140)
// and of its fused gate / up epilogue (kernels/prefill_moe.hip:364-396): per 32 values amax, d_inv = 127.0f / amax,
// q = roundf(x * d_inv), d = 1.0f / d_inv; D4 stores four fp32 d, DS4 four (fp16 d, fp16 sum) with sum = ((x0 + x1) + x2) + x3
// per four values then partners 4, 2, 1. An all-zero group stores d = 0 and codes 0 explicitly.
//
// Mapping: a warp per block of 128 values: a lane holds 4 consecutive values (one 16-byte load of fp32, 8-byte of fp16), the 8
// lanes of a group reduce by shuffles, the warp writes the block's 128 codes as one 4-byte word per lane and the four scales
// from lanes 0, 8, 16, 24: 144 contiguous bytes. Consecutive warps take consecutive rows of the same K-block, so their blocks
// are adjacent in memory.
#include "cam_common.cuh"

namespace {

// MODE 0: values = x (fp32). MODE 1: silu(x) * u (fp32). MODE 2: silu(g) * u (fp16 in).
template <int MODE, int LAYOUT>
__global__ void __launch_bounds__(256) mmq_q8_1_kernel(const void * __restrict__ xv, const void * __restrict__ uv, uint8_t * __restrict__ y,
                                                       int kvalid, int nkb, long ld, int rows) {
    const int lane = threadIdx.x & 31;
    const long total = (long)nkb * rows;
    for (long task = (long)blockIdx.x * 8 + (threadIdx.x >> 5); task < total; task += (long)gridDim.x * 8) {
        const int kb = (int)(task / rows), r = (int)(task - (long)kb * rows);
        const int k = kb * 128 + 4 * lane;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (k < kvalid) {       // (kvalid and ld are multiples of 4: a lane's four values are all inside or all outside)
            if (MODE == 2) {
                const uint2 g = __ldg(reinterpret_cast<const uint2 *>((const uint16_t *)xv + (size_t)r * ld + k));
                const uint2 u = __ldg(reinterpret_cast<const uint2 *>((const uint16_t *)uv + (size_t)r * ld + k));
                const float2 g0 = h2_to_f2(g.x), g1 = h2_to_f2(g.y), u0 = h2_to_f2(u.x), u1 = h2_to_f2(u.y);
                v[0] = fmul(cam_silu(g0.x), u0.x); v[1] = fmul(cam_silu(g0.y), u0.y);
                v[2] = fmul(cam_silu(g1.x), u1.x); v[3] = fmul(cam_silu(g1.y), u1.y);
            } else {
                const float4 a = __ldg(reinterpret_cast<const float4 *>((const float *)xv + (size_t)r * ld + k));
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                if (MODE == 1) {
                    const float4 b = __ldg(reinterpret_cast<const float4 *>((const float *)uv + (size_t)r * ld + k));
                    v[0] = fmul(cam_silu(v[0]), b.x); v[1] = fmul(cam_silu(v[1]), b.y);
                    v[2] = fmul(cam_silu(v[2]), b.z); v[3] = fmul(cam_silu(v[3]), b.w);
                }
            }
        }
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        float sum = fadd(fadd(fadd(v[0], v[1]), v[2]), v[3]);
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(CAM_FULL, amax, o));
            sum = fadd(sum, __shfl_xor_sync(CAM_FULL, sum, o));
        }
        float d = 0.0f;
        uint32_t w = 0;
        if (amax != 0.0f) {
            const float d_inv = fdiv(127.0f, amax);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float t = fmul(v[c], d_inv);
                const int q = fabsf(t) < 127.5f ? __float2int_rn(roundf(t)) : 0;
                w |= (uint32_t)(q & 0xff) << (8 * c);
            }
            d = fdiv(1.0f, d_inv);
        }
        uint8_t * blk = y + (size_t)task * 144;
        reinterpret_cast<uint32_t *>(blk + 16)[lane] = w;
        if ((lane & 7) == 0) reinterpret_cast<uint32_t *>(blk)[lane >> 3] = LAYOUT == 0 ? __float_as_uint(d) : f2_to_h2(d, sum);
    }
}

template <int MODE>
int launch_mmq(const void * x, const void * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, cudaStream_t stream) {
    if (rows < 0 || Kpad < 128 || (Kpad & 127) || kvalid < 0 || kvalid > Kpad || (kvalid & 3) || ld < kvalid || (ld & 3) || !x || !y ||
        (MODE != 0 && !u) || (layout != 0 && layout != 1)) return CAM_ERR_ARG;
    const int elt = MODE == 2 ? 8 : 16;
    if ((reinterpret_cast<uintptr_t>(x) & (elt - 1)) || (u && (reinterpret_cast<uintptr_t>(u) & (elt - 1))) || !cam_aligned16(y)) return CAM_ERR_ALIGN;
    if (rows == 0) return CAM_OK;
    const long total = (long)(Kpad / 128) * rows, want = (total + 7) / 8;
    if (layout == 0) mmq_q8_1_kernel<MODE, 0><<<cam_resident_grid(mmq_q8_1_kernel<MODE, 0>, 256, 0, want), 256, 0, stream>>>(x, u, (uint8_t *)y, kvalid, Kpad / 128, ld, rows);
    else mmq_q8_1_kernel<MODE, 1><<<cam_resident_grid(mmq_q8_1_kernel<MODE, 1>, 256, 0, want), 256, 0, stream>>>(x, u, (uint8_t *)y, kvalid, Kpad / 128, ld, rows);
    return (int)cudaGetLastError();
}

}   // namespace

// cam_quantize_mmq_q8_1: rows of x (fp32, row stride ld floats, kvalid values each, zero-padded to Kpad = a multiple of 128) ->
// blocks [Kpad / 128][rows] of 144 bytes; layout 0 = D4, 1 = DS4. The dense case (no ids, one channel) of the reference's
// quantize_mmq_q8_1, kernels/ggml_mmq/quantize_mmq.cuh:41-45.
extern "C" int cam_quantize_mmq_q8_1(const float * x, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream) {
    return launch_mmq<0>(x, nullptr, y, kvalid, Kpad, ld, rows, layout, (cudaStream_t)stream);
}
// cam_swiglu_mmq_q8_1[_f16]: the same blocks of silu(g) * u: what the reference's fused gate / up kernel writes for the down
// projection (kernels/prefill_moe.hip:339-396), as a standalone producer for fp32 or fp16 gate and up.
extern "C" int cam_swiglu_mmq_q8_1(const float * g, const float * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream) {
    return launch_mmq<1>(g, u, y, kvalid, Kpad, ld, rows, layout, (cudaStream_t)stream);
}
extern "C" int cam_swiglu_mmq_q8_1_f16(const void * g, const void * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream) {
    return launch_mmq<2>(g, u, y, kvalid, Kpad, ld, rows, layout, (cudaStream_t)stream);
}
