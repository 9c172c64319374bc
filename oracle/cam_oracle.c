/* CPU oracle for the fused glue ops: TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement, statement by statement and in the same order of floating-point operations, of the reference's
 * (jdominick05/caminus) HIP glue kernels. Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
 * call it; the shipped library never links or loads it.
 *
 * Every operation below is an IEEE-754 binary32/binary64 operation with round-to-nearest-even (compile with
 * -ffp-contract=off, no fast-math): products and sums are rounded one by one, fused multiply-adds appear exactly where the
 * reference writes fma. The four library calls the reference leaves to AMD's device library (expf, rsqrtf, powf,
 * cosf/sinf) have no portable bit pattern, so they are replaced by explicit sequences of IEEE operations, defined once here
 * (orc_expf, orc_rsqrt, orc_powi, orc_sincos) and restated with the same operations in the CUDA kernels: the CUDA path
 * is held bit-for-bit to this file, and this file is held to the reference's own CPU code (own_dequant.q4_k, q8_host,
 * the float64 norm / RoPE references of its tests) by tests/test_oracle_pins.py and the fixtures in tests/golden/.
 *
 * Thread mapping restated from the reference: a workgroup of 256 threads = 8 waves of 32; a wave sum is the xor butterfly
 * with partners 16, 8, 4, 2, 1 (kernels/q3m_prefill.hip:351-355); the workgroup total is the wave partials added in wave
 * order from 0.0f (kernels/q3m_prefill.hip:405-406).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stddef.h>

typedef _Float16 f16;

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline float h2f(uint16_t h) { f16 v; memcpy(&v, &h, 2); return (float)v; }           /* exact */
static inline uint16_t f2h(float f) { f16 v = (f16)f; uint16_t h; memcpy(&h, &v, 2); return h; } /* RNE */

/* ---- the four explicit sequences ------------------------------------------------------------------------------------ */

/* exp(a), a clamped to [-87, 88]: n = rint(a log2 e) by the 1.5 * 2^23 constant, r = a - n ln2 in two fma steps,
 * a degree-6 polynomial in fma form, then n added to the exponent field. Relative error below 1 ulp on the clamped range. */
float orc_expf(float a) {
    a = fminf(fmaxf(a, -87.0f), 88.0f);
    const float t = fmaf(a, 0x1.715476p+0f, 12582912.0f);
    const float n = t - 12582912.0f;
    float r = fmaf(n, -0x1.62e430p-1f, a);
    r = fmaf(n, 0x1.05c610p-29f, r);
    float p = 0x1.687b46p-10f;
    p = fmaf(p, r, 0x1.123bdcp-7f);
    p = fmaf(p, r, 0x1.555b5cp-5f);
    p = fmaf(p, r, 0x1.55548ep-3f);
    p = fmaf(p, r, 0x1.fffff8p-2f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    return u2f(f2u(p) + (f2u(t) << 23));
}

/* the reference's gg_silu, x / (1 + expf(-x)) (kernels/k3_gguf_ops.h:53), on orc_expf; the division is IEEE */
float orc_silu(float x) { return x / (1.0f + orc_expf(-x)); }

/* 1 / sqrt(v): IEEE square root, then IEEE division (stands for rsqrtf) */
float orc_rsqrt(float v) { return 1.0f / sqrtf(v); }

/* base^e for an integer e >= 0: binary exponentiation in binary64, rounded once to binary32 (stands for powf(base, (float)e)) */
float orc_powi(float base, int e) {
    double b = (double)base, p = 1.0;
    while (e) { if (e & 1) p = p * b; b = b * b; e >>= 1; }
    return (float)p;
}

/* sin and cos of theta (|theta| < 2^22): n = rint(theta 2/pi), r = theta - n pi/2 in three fma steps, polynomials on
 * [-pi/4, pi/4], quadrant from n's two low bits. Absolute error below 2 ulp of 1. */
void orc_sincos(float theta, float * sn, float * cs) {
    const float t = fmaf(theta, 0x1.45f306p-1f, 12582912.0f);
    const float n = t - 12582912.0f;
    const uint32_t q = f2u(t) & 3u;
    float r = fmaf(n, -0x1.921fb6p+0f, theta);
    r = fmaf(n, 0x1.777a5cp-25f, r);
    r = fmaf(n, 0x1.ee59dap-50f, r);
    const float z = r * r;
    float ps = -0x1.99518cp-13f;
    ps = fmaf(ps, z, 0x1.11076ep-7f);
    ps = fmaf(ps, z, -0x1.555546p-3f);
    const float s = fmaf(r * z, ps, r);
    float pc = 0x1.994222p-16f;
    pc = fmaf(pc, z, -0x1.6c08c4p-10f);
    pc = fmaf(pc, z, 0x1.55553ep-5f);
    pc = fmaf(pc, z, -0.5f);
    const float c = fmaf(z, pc, 1.0f);
    const float s0 = (q & 1u) ? c : s, c0 = (q & 1u) ? s : c;
    *sn = (q & 2u) ? -s0 : s0;
    *cs = ((q + 1u) & 2u) ? -c0 : c0;
}

/* ---- wave / workgroup sums ------------------------------------------------------------------------------------------ */

/* v[32] -> every lane's butterfly total (partners 16, 8, 4, 2, 1); returns lane 0's (all lanes hold the same bits) */
static float wave_sum(const float * v) {
    float a[32], b[32];
    memcpy(a, v, sizeof a);
    for (int o = 16; o > 0; o >>= 1) {
        for (int l = 0; l < 32; l++) b[l] = a[l] + a[l ^ o];
        memcpy(a, b, sizeof a);
    }
    return a[0];
}
static float wave_max(const float * v) {
    float m = v[0];
    for (int l = 1; l < 32; l++) m = fmaxf(m, v[l]);   /* max is exact: any order gives the butterfly's bits */
    return m;
}

/* ---- Q4_K embedding rows (kernels/q3m_prefill.hip:362-380; host form python/caminus/own_dequant.py:19-37) ---------------- */
void orc_q4k_get_rows(const uint8_t * W, int rb, int vocab, const int32_t * toks, float * x, int n, int N) {
    for (int t = 0; t < n; t++) {
        int tok = toks[t]; tok = tok < 0 ? 0 : tok; tok = tok > vocab - 1 ? vocab - 1 : tok;
        const uint8_t * row = W + (size_t)tok * rb;
        float * xr = x + (size_t)t * N;
        for (int i = 0; i < N; i++) {
            const uint8_t * blk = row + (size_t)(i >> 8) * 144;
            const int j = i & 255, sb = j >> 5, l = j & 31, is = sb >> 1, hi = sb & 1;
            const uint8_t * s = blk + 4;
            const uint32_t sc = sb < 4 ? (s[sb] & 63u) : ((s[sb + 4] & 0xfu) | ((uint32_t)(s[sb - 4] >> 6) << 4));
            const uint32_t m = sb < 4 ? (s[sb + 4] & 63u) : ((uint32_t)(s[sb + 4] >> 4) | ((uint32_t)(s[sb] >> 6) << 4));
            const float d = h2f((uint16_t)(blk[0] | (blk[1] << 8)));
            const float dm = h2f((uint16_t)(blk[2] | (blk[3] << 8)));
            const float q = (float)((blk[16 + is * 32 + l] >> (4 * hi)) & 15);
            const float a = d * (float)sc, b = a * q, c = dm * (float)m;
            xr[i] = b - c;
        }
    }
}

/* ---- residual add + RMSNorm ----------------------------------------------------------------------------------------- */

/* one row of N = 256 NI values already added (xs): thread tid's chain over tid + 256 j, the 8 wave sums in order */
static float row_ss(const float * xs, int N) {
    float part[8];
    for (int wv = 0; wv < 8; wv++) {
        float v[32];
        for (int l = 0; l < 32; l++) {
            const int tid = wv * 32 + l;
            float ss = 0.0f;
            for (int i = tid; i < N; i += 256) ss = fmaf(xs[i], xs[i], ss);
            v[l] = ss;
        }
        part[wv] = wave_sum(v);
    }
    float tot = 0.0f;
    for (int q = 0; q < 8; q++) tot += part[q];
    return tot;
}

/* q3p_add_rms16 (kernels/q3m_prefill.hip:382-415): x [n][N] += sum over slots (d [n][S][N], w [n][S] or null);
 * h (nullable) and h16 = the normed row. */
void orc_add_rms16(float * x, const float * d, const float * w, int S, const float * nw, float eps, float * h, uint16_t * h16,
                   int n, int N) {
    for (int t = 0; t < n; t++) {
        float * xr = x + (size_t)t * N;
        const float * dr = d ? d + (size_t)t * S * N : NULL;
        const float * wr = w ? w + (size_t)t * S : NULL;
        for (int i = 0; i < N; i++) {
            float acc = 0.0f;
            for (int sl = 0; sl < S; sl++) acc = wr ? fmaf(wr[sl], dr[(size_t)sl * N + i], acc) : acc + dr[(size_t)sl * N + i];
            if (S > 0) xr[i] = xr[i] + acc;
        }
        const float tot = row_ss(xr, N);
        const float scale = orc_rsqrt(tot / (float)N + eps);
        for (int i = 0; i < N; i++) {
            const float v = (xr[i] * scale) * nw[i];
            if (h) h[(size_t)t * N + i] = v;
            h16[(size_t)t * N + i] = f2h(v);
        }
    }
}

/* q35p_add_rms16 (kernels/q35_prefill.hip:628-660): x += d (d nullable), any N = 256 NI; h always written */
void orc_add_rms16_q35(float * x, const float * d, const float * nw, float eps, float * h, uint16_t * h16, int n, int N) {
    for (int t = 0; t < n; t++) {
        float * xr = x + (size_t)t * N;
        if (d) for (int i = 0; i < N; i++) xr[i] = xr[i] + d[(size_t)t * N + i];
        const float tot = row_ss(xr, N);
        const float scale = orc_rsqrt(tot / (float)N + eps);
        for (int i = 0; i < N; i++) {
            const float v = (xr[i] * scale) * nw[i];
            h[(size_t)t * N + i] = v;
            h16[(size_t)t * N + i] = f2h(v);
        }
    }
}

/* the fp16-storage form of the same statements (the benchmark's per-layer config): xs = (float)x + (float)d in fp32,
 * x = fp16(xs) stored, the norm taken over the unrounded xs, h16 = fp16((xs scale) nw) */
void orc_add_rms_f16(uint16_t * x, const uint16_t * d, const float * nw, float eps, uint16_t * h16, int n, int N) {
    for (int t = 0; t < n; t++) {
        float xs[N];
        uint16_t * xr = x + (size_t)t * N;
        for (int i = 0; i < N; i++) {
            xs[i] = h2f(xr[i]);
            if (d) { xs[i] = xs[i] + h2f(d[(size_t)t * N + i]); xr[i] = f2h(xs[i]); }
        }
        const float tot = row_ss(xs, N);
        const float scale = orc_rsqrt(tot / (float)N + eps);
        for (int i = 0; i < N; i++) h16[(size_t)t * N + i] = f2h((xs[i] * scale) * nw[i]);
    }
}

/* tensor-parallel form (no reference counterpart: the reference replicates its norms): this rank holds a column shard
 * x [n][Ns] of rows of Nfull. Kernel 1: the shard's partial sum of squares of xs = x + d with the same thread mapping on
 * its Ns columns, nothing stored. Kernel 2, after the partials were summed over ranks: x = fp16(xs), h16 = the normed shard. */
void orc_rms_partial_f16(const uint16_t * x, const uint16_t * d, float * ss, int n, int Ns) {
    for (int t = 0; t < n; t++) {
        float xs[Ns];
        for (int i = 0; i < Ns; i++) {
            xs[i] = h2f(x[(size_t)t * Ns + i]);
            if (d) xs[i] = xs[i] + h2f(d[(size_t)t * Ns + i]);
        }
        ss[t] = row_ss(xs, Ns);
    }
}
void orc_rms_apply_f16(uint16_t * x, const uint16_t * d, const float * tot, const float * nw, float eps, uint16_t * h16,
                       int n, int Ns, int Nfull) {
    for (int t = 0; t < n; t++) {
        const float scale = orc_rsqrt(tot[t] / (float)Nfull + eps);
        for (int i = 0; i < Ns; i++) {
            float xs = h2f(x[(size_t)t * Ns + i]);
            if (d) { xs = xs + h2f(d[(size_t)t * Ns + i]); x[(size_t)t * Ns + i] = f2h(xs); }
            h16[(size_t)t * Ns + i] = f2h((xs * scale) * nw[i]);
        }
    }
}

/* ---- SwiGLU and Q8_1 ------------------------------------------------------------------------------------------------ */

/* q3p_swiglu (kernels/q3m_prefill.hip:515-518): y = fp16(silu(g) u) */
void orc_swiglu16(const float * g, const float * u, uint16_t * y, long n) {
    for (long i = 0; i < n; i++) y[i] = f2h(orc_silu(g[i]) * u[i]);
}
/* gg_silu_mul (kernels/k3_gguf.hip:74-77): h = silu(g) u in fp32 */
void orc_silu_mul(const float * g, const float * u, float * h, long n) {
    for (long i = 0; i < n; i++) h[i] = orc_silu(g[i]) * u[i];
}

/* one block of 32 values -> 36 bytes: fp16 d, fp16 sum, int8 qs[32].
 * quantize_q8_1_lane as the reference restates it in q8_lane (kernels/k3_gguf_ops.h:145-153): amax and sum by the wave
 * butterfly, d = amax / 127.0f, q = amax == 0 ? 0 : roundf(x / d) (true division; halves away from zero).
 * sum_order 0: the lane butterfly (gg_op_q8_1, kernels/k3_gguf_ops.h:55-77). sum_order 1: aq_fill's order, 8 lanes of a
 * float4 each: (e0 + e1) + (e2 + e3) per lane, then partners 4, 2, 1 (kernels/k3_gguf_ops.h:83-120); d and the codes are
 * the same in both ("d = amax / 127 and q = roundf(x / d) per element exactly as quantize_q8_1_lane").
 * A value that is not finite gives code 0 (the reference leaves that conversion undefined). */
static void q8_1_block(const float * xi, uint8_t * out, int sum_order) {
    float a[32];
    for (int l = 0; l < 32; l++) a[l] = fabsf(xi[l]);
    const float amax = wave_max(a);
    float sum;
    if (sum_order == 0) sum = wave_sum(xi);
    else {
        float p[8], q[8];
        for (int l = 0; l < 8; l++) p[l] = (xi[4 * l] + xi[4 * l + 1]) + (xi[4 * l + 2] + xi[4 * l + 3]);
        for (int m = 4; m >= 1; m >>= 1) {
            for (int l = 0; l < 8; l++) q[l] = p[l] + p[l ^ m];
            memcpy(p, q, sizeof p);
        }
        sum = p[0];
    }
    const float d = amax / 127.0f;
    const uint16_t hd = f2h(d), hs = f2h(sum);
    memcpy(out, &hd, 2); memcpy(out + 2, &hs, 2);
    for (int l = 0; l < 32; l++) {
        int8_t q = 0;
        if (amax != 0.0f) {
            const float v = xi[l] / d;
            if (fabsf(v) < 127.5f) q = (int8_t)roundf(v);   /* (false for NaN; a finite block never exceeds 127.00002) */
        }
        out[4 + l] = (uint8_t)q;
    }
}

/* gg_quantize_q8_1 (kernels/k3_gguf.hip:29-36): n values, blocks of 32, values past n are 0 */
void orc_q8_1(const float * x, uint8_t * y, long n, int sum_order) {
    const long nb = (n + 31) / 32;
    for (long b = 0; b < nb; b++) {
        float xi[32];
        for (int l = 0; l < 32; l++) { const long i = b * 32 + l; xi[l] = i < n ? x[i] : 0.0f; }
        q8_1_block(xi, y + b * 36, sum_order);
    }
}
/* gg_op_q8_1 work = 2 (kernels/k3_gguf_ops.h:70-72): xi = silu(x) * mul, then the block quantiser */
void orc_swiglu_q8_1(const float * g, const float * u, uint8_t * y, long n, int sum_order) {
    const long nb = (n + 31) / 32;
    for (long b = 0; b < nb; b++) {
        float xi[32];
        for (int l = 0; l < 32; l++) { const long i = b * 32 + l; xi[l] = i < n ? orc_silu(g[i]) * u[i] : 0.0f; }
        q8_1_block(xi, y + b * 36, sum_order);
    }
}
/* the same with fp16 gate / up (converted exactly to fp32 first) */
/* the tape op's work = 1 (kernels/k3_gguf_ops.h:70): xi = gg_silu(x * rs), ggml_scale then ggml_silu, then the quantiser */
void orc_silu_scale_q8_1(const float * x, float rs, uint8_t * y, long n, int sum_order) {
    for (long b = 0; b * 32 < n; b++) {
        float xi[32];
        for (int i = 0; i < 32; i++) { const long k = b * 32 + i; xi[i] = k < n ? orc_silu(x[k] * rs) : 0.0f; }
        q8_1_block(xi, y + b * 36, sum_order);
    }
}
void orc_swiglu_q8_1_f16(const uint16_t * g, const uint16_t * u, uint8_t * y, long n, int sum_order) {
    const long nb = (n + 31) / 32;
    for (long b = 0; b < nb; b++) {
        float xi[32];
        for (int l = 0; l < 32; l++) { const long i = b * 32 + l; xi[l] = i < n ? orc_silu(h2f(g[i])) * h2f(u[i]) : 0.0f; }
        q8_1_block(xi, y + b * 36, sum_order);
    }
}
/* the fp32 products the quantiser saw (for the reference's flip rule, tests/engine/golden_util.py:132-173) */
void orc_swiglu_f32_from_f16(const uint16_t * g, const uint16_t * u, float * h, long n) {
    for (long i = 0; i < n; i++) h[i] = orc_silu(h2f(g[i])) * h2f(u[i]);
}

/* ---- q/k RMSNorm + NeoX RoPE ---------------------------------------------------------------------------------------- */

/* one head of 128 (kernels/q3m_prefill.hip:552-590): ss = x x per dim, four wave sums in order, scale = rsqrt(tot / 128 +
 * eps), y1 = (scale x) w, pairs (j, j + 64): fma(x0, c, -(x1 s)) and fma(x1, c, x0 s) */
/* sum_order 0: the reference's (above). sum_order 1: the CUDA kernel's mapping, 16 lanes per head: lane l sums its dims
 * 4l .. 4l + 3 and 64 + 4l .. 64 + 4l + 3 in two fma chains, adds them, then a butterfly with partners 8, 4, 2, 1. */
static void head_norm_rope(const float * x, const float * wn, float eps, const float * rc, const float * rs, float * y, int sum_order) {
    float part[4], sq[128], y1[128];
    float tot = 0.0f;
    if (sum_order == 0) {
        for (int i = 0; i < 128; i++) sq[i] = x[i] * x[i];
        for (int wv = 0; wv < 4; wv++) part[wv] = wave_sum(sq + 32 * wv);
        for (int q = 0; q < 4; q++) tot += part[q];
    } else {
        float p[16], q[16];
        for (int l = 0; l < 16; l++) {
            float sl = 0.0f, sh = 0.0f;
            for (int c = 0; c < 4; c++) { sl = fmaf(x[4 * l + c], x[4 * l + c], sl); sh = fmaf(x[64 + 4 * l + c], x[64 + 4 * l + c], sh); }
            p[l] = sl + sh;
        }
        for (int o = 8; o > 0; o >>= 1) {
            for (int l = 0; l < 16; l++) q[l] = p[l] + p[l ^ o];
            memcpy(p, q, sizeof p);
        }
        tot = p[0];
    }
    const float scale = orc_rsqrt(tot / 128.0f + eps);
    for (int i = 0; i < 128; i++) y1[i] = (scale * x[i]) * wn[i];
    for (int j = 0; j < 64; j++) {
        const float c = rc[j], sn = rs[j], x0 = y1[j], x1 = y1[j + 64];
        y[j] = fmaf(x0, c, -(x1 * sn));
        y[j + 64] = fmaf(x1, c, x0 * sn);
    }
}
/* cos / sin of a position: plain (theta = (float)pos powf(theta_scale, j), kernels/q3m_prefill.hip:565) or the YaRN table
 * (theta = (float)pos freq[j], both times mscale, kernels/q3m_prefill.hip:560-563) */
static void pos_table(const float * par, int pos, int yarn, float * rc, float * rs) {
    for (int j = 0; j < 64; j++) {
        float s, c;
        if (yarn) { orc_sincos((float)pos * par[258 + j], &s, &c); rc[j] = c * par[322]; rs[j] = s * par[322]; }
        else { orc_sincos((float)pos * orc_powi(par[256], j), &s, &c); rc[j] = c; rs[j] = s; }
    }
}

/* q3p_qk_rope (kernels/q3m_prefill.hip:520-591, the F16 cache form): qkv fp32 [n][ldq] = q | k | v; q16 [n][nh][128];
 * cache row pos = K [nkv][128] | V [nkv][128] fp16. par = q_norm[128] | k_norm[128] | theta_scale | eps (| freq[64] | mscale) */
void orc_qk_rope(const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, uint16_t * q16, uint16_t * cache,
                 int n, int yarn, int sum_order) {
    const size_t M = (size_t)nkv * 128;
    for (int t = 0; t < n; t++) {
        const int pos = pos0 + t;
        float rc[64], rs[64], y[128];
        pos_table(par, pos, yarn, rc, rs);
        const float * row = qkv + (size_t)t * ldq;
        uint16_t * cw = cache + (size_t)pos * 2 * M;
        for (int hy = 0; hy < nh + nkv; hy++) {
            const int isq = hy < nh, g = hy - nh;
            const float * x = isq ? row + (size_t)hy * 128 : row + (size_t)nh * 128 + (size_t)g * 128;
            head_norm_rope(x, isq ? par : par + 128, par[257], rc, rs, y, sum_order);
            uint16_t * o = isq ? q16 + ((size_t)t * nh + hy) * 128 : cw + (size_t)g * 128;
            for (int i = 0; i < 128; i++) o[i] = f2h(y[i]);
            if (!isq) for (int i = 0; i < 128; i++) cw[M + (size_t)g * 128 + i] = f2h(row[(size_t)nh * 128 + M + (size_t)g * 128 + i]);
        }
    }
}
/* the same statements on fp16 q [n][nh][128] and k [n][nkv][128] (converted exactly to fp32), fp16 out (may alias in) */
void orc_qk_rope_f16(const uint16_t * q, const uint16_t * k, int nh, int nkv, const float * par, int pos0, uint16_t * qo,
                     uint16_t * ko, int n, int yarn, int sum_order) {
    for (int t = 0; t < n; t++) {
        float rc[64], rs[64], x[128], y[128];
        pos_table(par, pos0 + t, yarn, rc, rs);
        for (int hy = 0; hy < nh + nkv; hy++) {
            const int isq = hy < nh;
            const size_t off = isq ? ((size_t)t * nh + hy) * 128 : ((size_t)t * nkv + (hy - nh)) * 128;
            const uint16_t * in = isq ? q + off : k + off;
            uint16_t * o = isq ? qo + off : ko + off;
            for (int i = 0; i < 128; i++) x[i] = h2f(in[i]);
            head_norm_rope(x, isq ? par : par + 128, par[257], rc, rs, y, sum_order);
            for (int i = 0; i < 128; i++) o[i] = f2h(y[i]);
        }
    }
}

int orc_version(void) { return 1; }

/* ==== the Coder / hyper-connection line and the training line's forwards (kernels/prefill_glue.hip, core.hip, fuse.hip) ==== */

static inline uint16_t f2bf_rne(float v) {          /* prefill_glue.hip:75-78 to_bf16: round to nearest even, no NaN case */
    const uint32_t u = f2u(v);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
static inline uint16_t f2bf_nan(float f) {          /* core.hip:17-22 f2bf: the same with NaN -> 0x7fc0 */
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float bf2f(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline float orc_sigmoid(float v) { return 1.0f / (1.0f + orc_expf(-v)); }

/* pf_rms_mul (kernels/prefill_glue.hip:90-124): y[r] = (x[r] rsqrt(sum x^2 / K + eps)) w[r % wr]; outputs optional:
 * y fp32 (may be x), ybf bf16, scl the row scale. K = 256 NI. */
void orc_pf_rms_mul(const float * x, const float * w, float * y, uint16_t * ybf, float * scl, int R, int wr, float eps, int K) {
    for (int t = 0; t < R; t++) {
        const float * xr = x + (size_t)t * K, * wv = w + (size_t)(t % wr) * K;
        const float scale = orc_rsqrt(row_ss(xr, K) / (float)K + eps);
        if (scl) scl[t] = scale;
        for (int i = 0; i < K; i++) {
            const float v = (xr[i] * scale) * wv[i];
            if (ybf) ybf[(size_t)t * K + i] = f2bf_rne(v);
            if (y) y[(size_t)t * K + i] = v;
        }
    }
}

/* pf_hc_post_rms (kernels/prefill_glue.hip:126-171): row q = (token tt, stream h): res = fma(b[tt], 2 sigmoid(inj[q] rs), res)
 * in place, then the norm of res with w[h]: xn, xnbf, scl optional */
void orc_pf_hc_post_rms(const float * b, const float * inj, float * res, const float * w, float * xn, uint16_t * xnbf, float * scl,
                        int T, int HC, float rs, float eps, int N) {
    for (int q = 0; q < T * HC; q++) {
        const int h = q % HC, tt = q / HC;
        float * rr = res + (size_t)q * N;
        const float v = inj[q] * rs, p = orc_sigmoid(v) * 2.0f;
        for (int i = 0; i < N; i++) rr[i] = fmaf(b[(size_t)tt * N + i], p, rr[i]);
        const float scale = orc_rsqrt(row_ss(rr, N) / (float)N + eps);
        if (scl) scl[q] = scale;
        for (int i = 0; i < N; i++) {
            const float o = (rr[i] * scale) * w[(size_t)h * N + i];
            if (xn) xn[(size_t)q * N + i] = o;
            if (xnbf) xnbf[(size_t)q * N + i] = f2bf_rne(o);
        }
    }
}

/* pf_hc_post (kernels/prefill_glue.hip:173-191): the residual update alone, every stream */
void orc_pf_hc_post(const float * b, const float * inj, float * res, int T, int HC, int D, float rs) {
    for (long i = 0; i < (long)T * D; i++) {
        const int tt = (int)(i / D), ii = (int)(i - (long)tt * D);
        for (int h = 0; h < HC; h++) {
            const float ph = orc_sigmoid(inj[tt * HC + h] * rs) * 2.0f;
            const size_t o = (size_t)(tt * HC + h) * D + ii;
            res[o] = fmaf(b[i], ph, res[o]);
        }
    }
}

/* pf_hc_mean (kernels/prefill_glue.hip:193-206): out = rs sum_h xn sigmoid(g) (fma chain over h from 0); xn given, or
 * recomputed as (x scl) w when scl is not null */
void orc_pf_hc_mean(const float * x, const float * scl, const float * w, const float * g, float * out, int T, int HC, int D, float rs) {
    for (long i = 0; i < (long)T * D; i++) {
        const int tt = (int)(i / D), ii = (int)(i - (long)tt * D);
        float sum = 0.0f;
        for (int h = 0; h < HC; h++) {
            const size_t o = (size_t)(tt * HC + h) * D + ii;
            const float xv = scl ? (x[o] * scl[tt * HC + h]) * w[(size_t)h * D + ii] : x[o];
            sum = fmaf(xv, orc_sigmoid(g[o]), sum);
        }
        out[i] = rs * sum;
    }
}

/* pf_add_sum (kernels/prefill_glue.hip:417-423): y = y + (a + b) */
void orc_pf_add_sum(const float * a, const float * b, float * y, long n) {
    for (long i = 0; i < n; i++) { const float ab = a[i] + b[i]; y[i] = y[i] + ab; }
}
/* pf_swiglu (kernels/prefill_tp.hip:37-43): y = silu(g) u in fp32 */
void orc_pf_swiglu(const float * g, const float * u, float * y, long n) {
    for (long i = 0; i < n; i++) y[i] = orc_silu(g[i]) * u[i];
}
/* pf_silu_bf16 / pf_to_bf16 (kernels/prefill_glue.hip:552-566): bf16(silu(fma(rs, x, 0))) / bf16(x), rows T .. Tpad - 1 zero */
void orc_pf_silu_bf16(const float * x, int ldx, uint16_t * y, int T, int Tpad, int K, float rs) {
    for (long i = 0; i < (long)Tpad * K; i++) {
        const int t = (int)(i / K), j = (int)(i - (long)t * K);
        y[i] = t < T ? f2bf_rne(orc_silu(fmaf(rs, x[(size_t)t * ldx + j], 0.0f))) : 0;
    }
}
void orc_pf_to_bf16(const float * x, int ldx, uint16_t * y, int T, int Tpad, int K) {
    for (long i = 0; i < (long)Tpad * K; i++) {
        const int t = (int)(i / K), j = (int)(i - (long)t * K);
        y[i] = t < T ? f2bf_rne(x[(size_t)t * ldx + j]) : 0;
    }
}

/* core.hip:23-66 */
void orc_embedding_f32(const int32_t * tok, const float * emb, float * out, int D, int T) {
    for (int t = 0; t < T; t++) memcpy(out + (size_t)t * D, emb + (size_t)tok[t] * D, (size_t)D * 4);
}
/* rmsnorm_f32 (core.hip:30-46): thread t sums x[j]^2 over j = t, t + 256, ... (contracted: s = fma(x, x, s)), the butterfly,
 * the eight partials in order; out = (x inv) w */
void orc_rmsnorm_f32(const float * x, const float * w, float * out, int D, float eps, int R) {
    for (int r = 0; r < R; r++) {
        const float * xr = x + (size_t)r * D;
        const float inv = orc_rsqrt(row_ss(xr, D) / (float)D + eps);
        for (int j = 0; j < D; j++) out[(size_t)r * D + j] = (xr[j] * inv) * w[j];
    }
}
/* silu_mul_bf16 (core.hip:48-55): act = bf16(bf16(silu(g)) u) over rows gu = [g | u] of 2 H bf16 */
void orc_silu_mul_bf16(const uint16_t * gu, uint16_t * act, int H, long n) {
    for (long i = 0; i < n; i++) {
        const long r = i / H, c = i % H;
        const float g = bf2f(gu[r * 2 * H + c]), u = bf2f(gu[r * 2 * H + H + c]);
        const float s = bf2f(f2bf_nan(orc_silu(g)));
        act[i] = f2bf_nan(s * u);
    }
}
/* residual3 (core.hip:57-61): out = (x + m) + y, m and y bf16 */
void orc_residual3(const float * x, const uint16_t * m, const uint16_t * y, float * out, long n) {
    for (long i = 0; i < n; i++) out[i] = (x[i] + bf2f(m[i])) + bf2f(y[i]);
}
void orc_cast_bf16(const float * x, uint16_t * out, long n) { for (long i = 0; i < n; i++) out[i] = f2bf_nan(x[i]); }
/* residual_slices_fwd (kernels/fuse.hip:19-33): out = ((x + m) + mlp) + (pos[r] >= 0 ? ys[pos[r]] : 0) */
void orc_residual_slices_fwd(const float * x, const uint16_t * m, const uint16_t * mlp, const uint16_t * ys, const int32_t * pos,
                             float * out, int d, long n4) {
    for (long e = 0; e < n4 * 4; e++) {
        const int r = (int)(e / d), c = (int)(e % d);
        const int p = pos ? pos[r] : -1;
        out[e] = ((x[e] + bf2f(m[e])) + bf2f(mlp[e])) + (p >= 0 ? bf2f(ys[(size_t)p * d + c]) : 0.0f);
    }
}

/* pf_qk_nr (kernels/prefill_attn.hip:103-129) = op_qk_nr (kernels/k3_gguf_ops.h:1490-1518): block t = row heads + head; head
 * dim D <= 512, rotation over the first nrot dims (pairs j, j + nrot / 2), fp32 out; default contraction: ss = fma(x, x, ss)
 * per thread over i = tid + 256 k, y = fma(x0, c, -(x1 sn)) and fma(x0, sn, x1 c) */
void orc_pf_qk_nr(const float * xin, int head_stride, int heads, const float * w, int D, int nrot, float theta_scale, float eps,
                  int pos0, float * out, int nblocks) {
    for (int t = 0; t < nblocks; t++) {
        const float * x = xin + (size_t)t * head_stride;
        float * y = out + (size_t)t * D;
        float nrm[512];
        const float scale = orc_rsqrt(row_ss(x, D) / (float)D + eps);
        for (int i = 0; i < D; i++) nrm[i] = (scale * x[i]) * w[i];
        const float pos = (float)(pos0 + t / heads);
        for (int i = 0; i < D; i++) {
            if (i >= nrot) { y[i] = nrm[i]; continue; }
            const int j = i < nrot / 2 ? i : i - nrot / 2;
            float sn, c;
            orc_sincos(pos * orc_powi(theta_scale, j), &sn, &c);
            const float x0 = nrm[j], x1 = nrm[j + nrot / 2];
            y[i] = i < nrot / 2 ? fmaf(x0, c, -(x1 * sn)) : fmaf(x0, sn, x1 * c);
        }
    }
}

/* ==== Q8_1 in the MMQ layout (kernels/ggml_mmq/mmq.cuh:63-82 block_q8_1_mmq; algebra of kernels/ggml_mmq/quantize_mmq.cuh:41-140 and
 * of the fused gate / up epilogue, kernels/prefill_moe.hip:364-396) ==================================================================
 * Rows of K values are cut into blocks of 128; block (kb, row) sits at index kb * rows + row and is 144 bytes: 16 bytes of scales
 * then 128 int8. Per group of 32: amax; d_inv = 127.0f / amax; q = roundf(x * d_inv) (a product, not the division of the 36-byte
 * form); d = 1.0f / d_inv. layout 0 (D4): four fp32 d. layout 1 (DS4): four (fp16 d, fp16 sum), sum = ((x0 + x1) + x2) + x3 per
 * four values, then partners 4, 2, 1 over the group's eight fours. An all-zero group stores d = 0 and codes 0 (the reference's
 * arithmetic yields 0 * inf = NaN there, whose int8 conversion is 0 on its GPUs). Values at k >= kvalid are 0 (row padding). */
static void mmq_group(const float * x, int8_t * q, float * d_out, float * sum_out) {
    float amax = fabsf(x[0]);                     /* (as the reference's thread starts from its first value: a group of 32 NaNs has a NaN for a maximum and a scale; */
    for (int i = 1; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));      /*  a NaN among numbers is skipped by fmaxf) */
    float p[8], t[8];
    for (int l = 0; l < 8; l++) p[l] = ((x[4 * l] + x[4 * l + 1]) + x[4 * l + 2]) + x[4 * l + 3];
    for (int m = 4; m >= 1; m >>= 1) { for (int l = 0; l < 8; l++) t[l] = p[l] + p[l ^ m]; memcpy(p, t, sizeof p); }
    *sum_out = p[0];
    if (amax == 0.0f) { *d_out = 0.0f; memset(q, 0, 32); return; }
    const float d_inv = 127.0f / amax;
    for (int i = 0; i < 32; i++) {
        const float v = x[i] * d_inv;
        q[i] = fabsf(v) < 127.5f ? (int8_t)roundf(v) : 0;
    }
    *d_out = 1.0f / d_inv;
}
static void mmq_store(uint8_t * blk, int grp, int layout, float d, float sum, const int8_t * q) {
    if (layout == 0) memcpy(blk + 4 * grp, &d, 4);
    else { const uint16_t hd = f2h(d), hs = f2h(sum); memcpy(blk + 4 * grp, &hd, 2); memcpy(blk + 4 * grp + 2, &hs, 2); }
    memcpy(blk + 16 + 32 * grp, q, 32);
}
/* x: rows of stride ld floats; K padded to Kpad (a multiple of 128) with zeros past kvalid; mode 0: values = x; 1: silu(x) * u */
void orc_mmq_q8_1(const float * x, const float * u, uint8_t * y, int kvalid, int Kpad, long ld, int rows, int layout, int mode) {
    for (int r = 0; r < rows; r++)
        for (int kb = 0; kb < Kpad / 128; kb++) {
            uint8_t * blk = y + ((size_t)kb * rows + r) * 144;
            for (int grp = 0; grp < 4; grp++) {
                float v[32]; int8_t q[32]; float d, s;
                for (int i = 0; i < 32; i++) {
                    const int k = kb * 128 + grp * 32 + i;
                    v[i] = k < kvalid ? (mode ? orc_silu(x[(size_t)r * ld + k]) * u[(size_t)r * ld + k] : x[(size_t)r * ld + k]) : 0.0f;
                }
                mmq_group(v, q, &d, &s);
                mmq_store(blk, grp, layout, d, s, q);
            }
        }
}
void orc_mmq_q8_1_f16(const uint16_t * g, const uint16_t * u, uint8_t * y, int kvalid, int Kpad, long ld, int rows, int layout) {
    for (int r = 0; r < rows; r++)
        for (int kb = 0; kb < Kpad / 128; kb++) {
            uint8_t * blk = y + ((size_t)kb * rows + r) * 144;
            for (int grp = 0; grp < 4; grp++) {
                float v[32]; int8_t q[32]; float d, s;
                for (int i = 0; i < 32; i++) {
                    const int k = kb * 128 + grp * 32 + i;
                    v[i] = k < kvalid ? orc_silu(h2f(g[(size_t)r * ld + k])) * h2f(u[(size_t)r * ld + k]) : 0.0f;
                }
                mmq_group(v, q, &d, &s);
                mmq_store(blk, grp, layout, d, s, q);
            }
        }
}

/* ==== the Q8_0 KV cache form of q3p_qk_rope (kernels/q3m_prefill.hip:526-535, 541-546, 572-583; kernels/own_kv_codec.h:31-75;
 * kernels/own_kv_rot128.h:21-33; CPU reference python/caminus/ref_kv.py hadamard128 / encode_q8_kv) =========================== */
static inline float f16r(float x) { return h2f(f2h(x)); }                 /* own_kv_f16r: rounded to fp16 and back */

/* the orthonormal Walsh-Hadamard transform of 128 values: for h = 1, 2, .. 64 the pair (i, i + h) of i with bit h clear becomes
 * (a + b, a - b), then each value times fp32(1 / sqrt(128)) */
static void hadamard128(float * y) {
    for (int h = 1; h < 128; h <<= 1)
        for (int i = 0; i < 128; i++)
            if (!(i & h)) { const float a = y[i], b = y[i + h]; y[i] = a + b; y[i + h] = a - b; }
    for (int i = 0; i < 128; i++) y[i] = y[i] * 0x1.6a09e6p-4f;
}
/* own_kv_q8_encode: one block of 32 -> 34 bytes (fp16 d, 32 int8); returns 0 when the block is refused (its bytes are left alone) */
static int q8_0_encode(const float * x, uint8_t * y) {
    float amax = 0.0f; int finite = 1;
    for (int j = 0; j < 32; j++) { finite &= isfinite(x[j]) != 0; amax = fmaxf(amax, fabsf(x[j])); }
    if (!finite) return 0;
    const float d = amax / 127.0f;
    const float inv = d != 0.0f ? 1.0f / d : 0.0f;
    const uint16_t stored = f2h(d);
    if (amax != 0.0f && (d == 0.0f || !isfinite(d) || !isfinite(inv) || !isfinite(h2f(stored)))) return 0;
    memcpy(y, &stored, 2);
    for (int j = 0; j < 32; j++) y[2 + j] = (uint8_t)(int8_t)roundf(x[j] * inv);
    return 1;
}
/* q3p_qk_rope_q8: as orc_qk_rope; q16 = fp16 of the transform of the fp16-rounded RoPE result; the cache row (2 (M / 32) 34 bytes,
 * M = nkv 128) = Q8_0 blocks of the transformed fp16-rounded K, then of the fp16-rounded V; a refused block ORs 2 into *err */
void orc_qk_rope_q8(const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, uint16_t * q16, uint8_t * cache,
                    int32_t * err, int n, int yarn, int sum_order) {
    const size_t M = (size_t)nkv * 128, rowb = 2 * (M / 32) * 34;
    for (int t = 0; t < n; t++) {
        const int pos = pos0 + t;
        float rc[64], rs[64], y[128];
        pos_table(par, pos, yarn, rc, rs);
        const float * row = qkv + (size_t)t * ldq;
        uint8_t * cw = cache + (size_t)pos * rowb;
        for (int hy = 0; hy < nh + nkv; hy++) {
            const int isq = hy < nh, g = hy - nh;
            const float * x = isq ? row + (size_t)hy * 128 : row + (size_t)nh * 128 + (size_t)g * 128;
            head_norm_rope(x, isq ? par : par + 128, par[257], rc, rs, y, sum_order);
            for (int i = 0; i < 128; i++) y[i] = f16r(y[i]);
            hadamard128(y);
            if (isq) { for (int i = 0; i < 128; i++) q16[((size_t)t * nh + hy) * 128 + i] = f2h(y[i]); continue; }
            for (int w = 0; w < 4; w++) if (!q8_0_encode(y + 32 * w, cw + ((size_t)g * 4 + w) * 34)) *err |= 2;
            float v[128];
            for (int i = 0; i < 128; i++) v[i] = f16r(row[(size_t)nh * 128 + M + (size_t)g * 128 + i]);
            for (int w = 0; w < 4; w++) if (!q8_0_encode(v + 32 * w, cw + (M / 32 + (size_t)g * 4 + w) * 34)) *err |= 2;
        }
    }
}
void orc_hadamard128(float * y, int rows) { for (int r = 0; r < rows; r++) hadamard128(y + (size_t)r * 128); }
/* rows of K [rows][nkv][128] (already rotated by the caller) and V -> Q8_0 cache rows (python/caminus/ref_kv.py encode_q8_kv); returns
 * the number of refused blocks */
int orc_q8_kv_rows(const float * k, const float * v, uint8_t * out, int rows, int nkv) {
    const size_t M = (size_t)nkv * 128, rowb = 2 * (M / 32) * 34; int bad = 0;
    for (int r = 0; r < rows; r++)
        for (size_t b = 0; b < M / 32; b++) {
            bad += !q8_0_encode(k + (size_t)r * M + b * 32, out + (size_t)r * rowb + b * 34);
            bad += !q8_0_encode(v + (size_t)r * M + b * 32, out + (size_t)r * rowb + (M / 32 + b) * 34);
        }
    return bad;
}

/* ==== the training line's activation quantiser (kernels/actq.hip:40-132, 225-274, 307-326) =========================================
 * Per row of K (a multiple of 128, <= 8192), one workgroup of 8 waves; wave w takes chunks w, w + 8, ...; lane l of a chunk holds
 * elements 4l .. 4l + 3. u = bf16(FWHT128(bf16(src)) * bf16(1 / sqrt(128))); amax by wave butterfly then lds[0], lds[1], .. in order;
 * s = max(amax * clip / qmax, 1e-8); q = clamp(rint(u / s), -qmax - 1, qmax); y = bf16(q s); codes packed four per 16 bits. */
static inline float rbf(float f) { return bf2f(f2bf_nan(f)); }
static void fwht128(float * v) {      /* v[128]: lane l = v[4l .. 4l + 3]: stages 1, 2 inside the lane, 4 .. 64 across lanes (kernels/actq.hip:40-53) */
    for (int l = 0; l < 32; l++) {
        float * p = v + 4 * l; float a = p[0], b = p[1]; p[0] = a + b; p[1] = a - b;
        a = p[2]; b = p[3]; p[2] = a + b; p[3] = a - b;
        a = p[0]; b = p[2]; p[0] = a + b; p[2] = a - b;
        a = p[1]; b = p[3]; p[1] = a + b; p[3] = a - b;
    }
    for (int m = 1; m < 32; m <<= 1) {
        float t[128];
        for (int l = 0; l < 32; l++) for (int e = 0; e < 4; e++) {
            const float own = v[4 * l + e], pr = v[4 * (l ^ m) + e];
            t[4 * l + e] = (l & m) ? (pr - own) : (own + pr);
        }
        memcpy(v, t, sizeof t);
    }
}
/* src: K values of one row already in fp32 (before the bf16 rounding of the input) */
static void actq_row(const float * src, uint16_t * y, float * s_out, int K, float clip, int qmax, uint16_t * codes) {
    const int nch = K / 128;
    float u[8192]; float wmax[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int ch = 0; ch < nch; ch++) {
        float * c = u + 128 * ch;
        for (int i = 0; i < 128; i++) c[i] = rbf(src[128 * ch + i]);
        fwht128(c);
        for (int i = 0; i < 128; i++) { c[i] = rbf(c[i] * 0.08837890625f); wmax[ch % 8] = fmaxf(wmax[ch % 8], fabsf(c[i])); }
    }
    float amax = wmax[0];
    for (int w = 1; w < 8; w++) amax = fmaxf(amax, wmax[w]);
    const float s = fmaxf(amax * clip / (float)qmax, 1e-8f);
    if (s_out) *s_out = s;
    for (int ch = 0; ch < nch; ch++) for (int l = 0; l < 32; l++) {
        uint32_t pk = 0;
        for (int e = 0; e < 4; e++) {
            const int k = ch * 128 + l * 4 + e;
            const float q = fminf(fmaxf(rintf(u[k] / s), (float)(-qmax - 1)), (float)qmax);
            if (y) y[k] = f2bf_nan(q * s);
            pk |= ((uint32_t)(int)q & 0xFu) << (4 * e);
        }
        if (codes) codes[ch * 32 + l] = (uint16_t)pk;
    }
}
/* actq_fwd[_codes]_{bf16,f32} (kernels/actq.hip:315-326): x [M][K] bf16 (is_bf16) or fp32 */
void orc_actq_fwd(const void * x, int is_bf16, uint16_t * y, float * s, uint16_t * codes, int M, int K, float clip, int qmax) {
    for (int r = 0; r < M; r++) {
        float src[8192];
        for (int k = 0; k < K; k++) src[k] = is_bf16 ? bf2f(((const uint16_t *)x)[(size_t)r * K + k]) : ((const float *)x)[(size_t)r * K + k];
        actq_row(src, y ? y + (size_t)r * K : NULL, s ? s + r : NULL, K, clip, qmax, codes ? codes + (size_t)r * (K / 4) : NULL);
    }
}
/* silu_mul_actq_fwd (kernels/actq.hip:307-310, SiluMulSrc :89-95): the source is bf16(bf16(silu(g)) u) of gu rows [g | u], stride ld */
void orc_silu_mul_actq_fwd(const uint16_t * gu, int ld, int F, uint16_t * y, float * s, uint16_t * codes, int M, float clip, int qmax) {
    for (int r = 0; r < M; r++) {
        float src[8192]; const uint16_t * row = gu + (size_t)r * ld;
        for (int k = 0; k < F; k++) src[k] = rbf(rbf(orc_silu(bf2f(row[k]))) * bf2f(row[F + k]));
        actq_row(src, y ? y + (size_t)r * F : NULL, s ? s + r : NULL, F, clip, qmax, codes ? codes + (size_t)r * (F / 4) : NULL);
    }
}
/* the workgroup sum of actq.hip (wave butterfly, then lds[0] + lds[1] + ..): thread t's partial over k = t, t + 256, .. */
static float block_sum_of(const float * part256) {
    float lds[8];
    for (int w = 0; w < 8; w++) lds[w] = wave_sum(part256 + 32 * w);
    float r = lds[0];
    for (int w = 1; w < 8; w++) r = r + lds[w];
    return r;
}
/* block_entry_fwd (kernels/actq.hip:247-274): rstd = rsqrt(mean(x^2) + eps); the quantiser's source is x rstd w; nab gate
 * projections ab[j] = bf16(sum_k bf16(h_k) wab[j][k]) */
void orc_block_entry_fwd(const float * x, const float * nw, const uint16_t * wab, int nab, float eps, uint16_t * y, float * s,
                         uint16_t * codes, uint16_t * ab, float * rstd_out, int M, int d, float clip, int qmax) {
    for (int r = 0; r < M; r++) {
        const float * xr = x + (size_t)r * d;
        float part[256];
        for (int t = 0; t < 256; t++) { float ss = 0.f; for (int k = t; k < d; k += 256) ss = fmaf(xr[k], xr[k], ss); part[t] = ss; }
        const float rstd = orc_rsqrt(block_sum_of(part) / (float)d + eps);
        rstd_out[r] = rstd;
        float src[8192];
        for (int k = 0; k < d; k++) src[k] = xr[k] * rstd * nw[k];
        actq_row(src, y ? y + (size_t)r * d : NULL, s ? s + r : NULL, d, clip, qmax, codes ? codes + (size_t)r * (d / 4) : NULL);
        for (int j = 0; j < nab; j++) {
            for (int t = 0; t < 256; t++) {
                float acc = 0.f;
                for (int k = t; k < d; k += 256) acc = fmaf(rbf(xr[k] * rstd * nw[k]), bf2f(wab[(size_t)j * d + k]), acc);
                part[t] = acc;
            }
            float lds[8]; for (int w = 0; w < 8; w++) lds[w] = wave_sum(part + 32 * w);
            float v = 0.f; for (int w = 0; w < 8; w++) v += lds[w];
            ab[(size_t)r * nab + j] = f2bf_nan(v);
        }
    }
}

/* ==== the router glue of the Qwen3-MoE prefill (kernels/q3m_prefill.hip:417-513) ===================================================== */
/* q3p_router: logits[t][e] = h[t] . Wr[e]: lane l sums float4 dots at k0 = 4 l + 128 i (i ascending), then the wave butterfly. The
 * reference leaves the contraction of its dot to the compiler; here a dot is w0 x0, then three fma, added to the lane's sum. */
void orc_router(const float * h, const float * Wr, int E, int K, float * logits, int n) {
    for (int t = 0; t < n; t++) for (int e = 0; e < E; e++) {
        const float * x = h + (size_t)t * K, * wr = Wr + (size_t)e * K; float v[32];
        for (int l = 0; l < 32; l++) {
            float acc = 0.0f;
            for (int k0 = 4 * l; k0 < K; k0 += 128) {
                float d = wr[k0] * x[k0]; d = fmaf(wr[k0 + 1], x[k0 + 1], d); d = fmaf(wr[k0 + 2], x[k0 + 2], d); d = fmaf(wr[k0 + 3], x[k0 + 3], d);
                acc = acc + d;
            }
            v[l] = acc;
        }
        logits[(size_t)t * E + e] = wave_sum(v);
    }
}
/* q3p_topk: softmax over E <= 128 logits (lane owns logits lane + 32 j: max, exp(v - m), the lane's sum over j then the butterfly,
 * p = v (1 / sum)), rank = #{p_j > p_i, or p_j == p_i and j < i}, the k lowest ranks in rank order, weights p / max(sum of the k in
 * slot order, floor); err |= 1 for a logit that is not finite */
void orc_topk(const float * logits, int E, int k, float floor_, int32_t * ids, float * wts, int32_t * err, int n) {
    for (int t = 0; t < n; t++) {
        const float * lg = logits + (size_t)t * E; float v[128], lane_sum[32]; float m = -INFINITY;
        for (int e = 0; e < E; e++) { if (!isfinite(lg[e])) *err |= 1; m = fmaxf(m, lg[e]); }
        for (int l = 0; l < 32; l++) {
            float s = 0.0f;
            for (int j = 0; j < 4; j++) { const int e = l + 32 * j; if (e < E) { v[e] = orc_expf(lg[e] - m); s += v[e]; } }
            lane_sum[l] = s;
        }
        const float inv = 1.0f / wave_sum(lane_sum);
        for (int e = 0; e < E; e++) v[e] = v[e] * inv;
        int sel[64];
        for (int i = 0; i < E; i++) {
            int rk = 0;
            for (int j = 0; j < E; j++) rk += (v[j] > v[i]) || (v[j] == v[i] && j < i);
            if (rk < k) sel[rk] = i;
        }
        float ws = 0.0f;
        for (int j = 0; j < k; j++) ws = ws + v[sel[j]];
        ws = fmaxf(ws, floor_);
        for (int j = 0; j < k; j++) { ids[(size_t)t * k + j] = sel[j]; wts[(size_t)t * k + j] = v[sel[j]] / ws; }
    }
}

/* pf_router (kernels/prefill_glue.hip:242-308): softmax over E <= 1024 logits by a workgroup of 256 (thread tid owns logits tid + 256 j:
 * the maximum; v = exp(v - m); the thread's sum over j from 0.0f, the wave butterfly, the eight wave sums in wave order; p = v (1 / sum)),
 * rank = #{bits(p_j) > bits(p_i) as signed integers, or equal and j < i}, the k <= 64 lowest ranks in rank order, weights
 * p / max(sum of the k in slot order, clamp); err |= 1 for a logit that is not finite */
void orc_pf_router(const float * logits, int E, int k, float clamp, int32_t * ids, float * wts, int32_t * err, int n) {
    for (int t = 0; t < n; t++) {
        const float * lg = logits + (size_t)t * E; float v[1024]; float m = -INFINITY;
        for (int e = 0; e < E; e++) { if (!isfinite(lg[e])) *err |= 1; m = fmaxf(m, lg[e]); }
        float sum = 0.0f;
        for (int w = 0; w < 8; w++) {
            float lane_sum[32];
            for (int l = 0; l < 32; l++) {
                float s = 0.0f;
                for (int j = 0; j < 4; j++) { const int e = 32 * w + l + 256 * j; if (e < E) { v[e] = orc_expf(lg[e] - m); s += v[e]; } }
                lane_sum[l] = s;
            }
            const float ws = wave_sum(lane_sum);
            sum = w == 0 ? ws : sum + ws;
        }
        const float inv = 1.0f / sum;
        for (int e = 0; e < E; e++) v[e] = v[e] * inv;
        int sel[64];
        for (int i = 0; i < E; i++) {
            int rk = 0; const int32_t pi = (int32_t)f2u(v[i]);
            for (int j = 0; j < E; j++) { const int32_t pj = (int32_t)f2u(v[j]); rk += (pj > pi) || (pj == pi && j < i); }
            if (rk < k) sel[rk] = i;
        }
        float ws = 0.0f;
        for (int j = 0; j < k; j++) ws = ws + v[sel[j]];
        ws = fmaxf(ws, clamp);
        for (int j = 0; j < k; j++) { ids[(size_t)t * k + j] = sel[j]; wts[(size_t)t * k + j] = v[sel[j]] / ws; }
    }
}

/* ==== the IQ4 row gathers of the host feed (kernels/prefill_feed.hip:24-54; host decoders python/caminus/own_dequant.py iq4_xs) ====
 * The 16 values of a 4-bit index are ggml's IQ4_NL codebook (part of the format's definition). IQ4_NL block: f16 d, 16 bytes of
 * nibbles (low nibble = value j, high = value j + 16), y = d * kvalue. IQ4_XS block (136 bytes, 256 values): f16 d, u16 scales_h,
 * u8 scales_l[4], qs[128]; sub-block ib's scale ls = (scales_l[ib / 2] >> 4 (ib & 1)) & 15 | ((scales_h >> 2 ib) & 3) << 4,
 * y = (d * (ls - 32)) * kvalue. An index outside its table is clamped and reported in err (bit 0 / bit 1). */
static const float kIQ4NL[16] = {-127.f, -104.f, -83.f, -65.f, -49.f, -35.f, -22.f, -10.f, 1.f, 13.f, 25.f, 38.f, 53.f, 69.f, 89.f, 113.f};
void orc_ple_rows_iq4nl(const uint8_t * raw, const int32_t * inv, int nuniq, int nrows, int bpr, float * out, int32_t * err) {
    const int hd = bpr * 32;
    for (long i = 0; i < (long)nrows * hd; i++) {
        const int r = (int)(i / hd), k = (int)(i % hd), b = k >> 5, j = k & 31;
        int u = inv[r];
        if (u < 0 || u >= nuniq) { *err |= 1; u = u < 0 ? 0 : nuniq - 1; }
        const uint8_t * blk = raw + (size_t)u * (size_t)(bpr * 18) + (size_t)b * 18;
        const uint8_t q = blk[2 + (j & 15)];
        out[i] = h2f((uint16_t)(blk[0] | (blk[1] << 8))) * kIQ4NL[j < 16 ? (q & 15) : (q >> 4)];
    }
}
void orc_embd_rows_iq4xs(const uint8_t * table, const int32_t * tok, int nvocab, int n, int nblk, float * out, int32_t * err) {
    const int D = nblk * 256;
    for (long i = 0; i < (long)n * D; i++) {
        const int p = (int)(i / D), k = (int)(i % D), bl = k >> 8, w = k & 255, ib = w >> 5, j = w & 31;
        int t = tok[p];
        if (t < 0 || t >= nvocab) { *err |= 2; t = t < 0 ? 0 : nvocab - 1; }
        const uint8_t * b = table + (size_t)t * (size_t)(nblk * 136) + (size_t)bl * 136;
        const int sh = b[2] | (b[3] << 8), sl = b[4 + (ib >> 1)];
        const int ls = ((sl >> ((ib & 1) * 4)) & 15) | (((sh >> (2 * ib)) & 3) << 4);
        const float dl = h2f((uint16_t)(b[0] | (b[1] << 8))) * (float)(ls - 32);
        const uint8_t q = b[8 + 16 * ib + (j & 15)];
        out[i] = dl * kIQ4NL[j < 16 ? (q & 15) : (q >> 4)];
    }
}

/* Q6_K row gather (no kernel of the reference does this; its host decoder python/caminus/own_dequant.py:40-53 is the definition, bitwise
 * gguf-py): 210-byte blocks of 256 = ql[128] | qh[64] | int8 sc[16] | fp16 d; per half n of 128 and group qd of 32, lane l:
 * q = nibble (ql[n][(qd & 1) 32 + l], high for qd >= 2) | ((qh[n][l] >> 2 qd) & 3) << 4; y = (d * sc[8 n + 2 qd + (l >= 16)]) * (q - 32),
 * two roundings. Token ids are clamped to the vocabulary. */
void orc_emb_rows_q6k(const uint8_t * W, int rb, int vocab, const int32_t * toks, float * x, int n, int N) {
    for (int p = 0; p < n; p++) {
        int t = toks[p]; t = t < 0 ? 0 : t >= vocab ? vocab - 1 : t;
        const uint8_t * row = W + (size_t)t * rb;
        for (int i = 0; i < N; i++) {
            const uint8_t * b = row + (size_t)(i >> 8) * 210;
            const int w = i & 255, nn = w >> 7, qd = (w >> 5) & 3, l = w & 31;
            const uint8_t qlb = b[nn * 64 + (qd & 1) * 32 + l], qhb = b[128 + nn * 32 + l];
            const int q = ((qd >= 2 ? qlb >> 4 : qlb & 15) | (((qhb >> (2 * qd)) & 3) << 4)) - 32;
            const float d = h2f((uint16_t)(b[208] | (b[209] << 8)));
            const float ds = d * (float)(int8_t)b[192 + nn * 8 + 2 * qd + (l >= 16)];
            x[(size_t)p * N + i] = ds * (float)q;
        }
    }
}

/* IQ2_S row gather: q35t_emb_iq2s (kernels/q35_prefill_tcap.hip:94-113) = q35t_op_emb (kernels/k3_q35t_ops.h:147-175), the floats of the host
 * decoder python/caminus/own_dequant.py:128-137. 82-byte blocks of 256 = fp16 d | qs[32] | signs[32] | qh[8] | scales[8]; value j of a block:
 * group j >> 3 has the 10-bit grid index qs[j >> 3] | ((qh[j >> 5] >> 2 ((j >> 3) & 3)) & 3) << 8, its magnitude k = j & 7 is the 2-bit code at
 * bits 2 k of the grid's 16-bit entry (0: 8, 1: 25, else 43); y = +-(((d (0.5 + s)) 0.25) mag) with s the nibble j >> 4 of scales and the sign
 * bit j & 7 of signs[j >> 3]. grid: the 1024 entries packed two to a 32-bit word (entry 2 w in word w's low half), GGUF's format constant,
 * which the caller supplies. Token ids are clamped to the vocabulary. */
void orc_emb_rows_iq2s(const uint8_t * W, int rb, int vocab, const int32_t * toks, float * x, int n, int N, const uint32_t * grid) {
    for (int p = 0; p < n; p++) {
        int t = toks[p]; t = t < 0 ? 0 : t >= vocab ? vocab - 1 : t;
        const uint8_t * row = W + (size_t)t * rb;
        for (int i = 0; i < N; i++) {
            const uint8_t * b = row + (size_t)(i >> 8) * 82;
            const int j = i & 255, ib = j >> 5, g = (j >> 3) & 3, k = j & 7;
            const float d = h2f((uint16_t)(b[0] | (b[1] << 8)));
            const uint32_t idx = b[2 + 4 * ib + g] | ((((uint32_t)b[66 + ib] >> (2 * g)) & 3u) << 8);
            const uint32_t code = ((grid[idx >> 1] >> (16 * (idx & 1u))) >> (2 * k)) & 3u;
            const float mag = code == 0 ? 8.0f : code == 1 ? 25.0f : 43.0f;
            const float sc = (float)((b[74 + ib] >> (4 * ((j >> 4) & 1))) & 15);
            const float db = (d * (0.5f + sc)) * 0.25f;
            const float v = db * mag;
            x[(size_t)p * N + i] = ((b[34 + (j >> 3)] >> k) & 1) ? -v : v;
        }
    }
}
