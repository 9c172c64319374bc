/* caminus_b200: C ABI of the B200 (sm_100a) glue kernels: libcaminus_b200.so.
 *
 * Each entry replaces one `extern "C" __global__` kernel of the reference (jdominick05/caminus, HIP for gfx1100) and
 * takes that kernel's parameters in the reference's order, device pointers as plain pointers. Where the reference conveys
 * a row or head count only through the launch grid, the count is the explicit leading argument here. The last argument
 * is the CUDA stream (a cudaStream_t passed as void *, 0 = the default stream). Nothing here allocates device memory;
 * every buffer is the caller's and must stay alive until the stream has run the launch.
 *
 * Return value: 0 = launched; negative = the arguments were refused and nothing was launched (CAM_ERR_*);
 * positive = a cudaError_t from the launch. cam_error_string() gives the text of any of them.
 *
 * Alignment: pointers to row data must be 16-byte aligned and row strides multiples of 16 bytes (128-bit accesses);
 * an entry returns CAM_ERR_ALIGN otherwise. fp16 buffers are IEEE binary16 passed as void *.
 *
 * Arithmetic: every stored value is produced by IEEE-754 round-to-nearest operations in the order of the reference's
 * statements (including its wave-butterfly summation order). expf, rsqrtf, powf and cosf / sinf of the reference's device
 * library are explicit sequences of IEEE operations (csrc/cam_common.cuh), so results are reproducible bit for bit on a CPU.
 */
#ifndef CAMINUS_B200_H
#define CAMINUS_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define CAM_OK 0
#define CAM_ERR_ARG (-1)
#define CAM_ERR_ALIGN (-2)
#define CAM_ERR_SHAPE (-3)
#define CAM_ERR_CAPACITY (-4)

/* Library. Replaces the loader half of runtime/rt.h:55-70 (rt::Module::load / fn / launch) and the error text of
 * python/caminus/device/hip.py:35-37. */
int cam_abi_version(void);
const char * cam_error_string(int code);

/* Q4_K embedding rows: x [n][N] fp32 = rows toks[i], clamped to [0, vocab), of the raw-block table W (rb bytes per row,
 * 144-byte super-blocks of 256 values). Bitwise the host decoder own_dequant.q4_k.
 * Replaces q3p_emb, kernels/q3m_prefill.hip:364-365 (n = grid.x); wrapper python/caminus/prefill/q3m_ops.py:86-87. */
int q3p_emb(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, void * stream);

/* Residual add + RMSNorm, Qwen3-MoE form: x [n][N] += sum over S slots of w[t][s] * d[t][s][:] (w null: plain sums; S = 0:
 * no add); h (nullable) fp32 and h16 fp16 = (x * rsqrt(mean(x^2) + eps)) * nw. N a multiple of 256, <= 2048.
 * Replaces q3p_add_rms16, kernels/q3m_prefill.hip:385-387 (n = grid.x); wrapper python/caminus/prefill/q3m_ops.py:89-92. */
int q3p_add_rms16(int n, float * x, const float * d, const float * w, int S, const float * nw, float eps, float * h, void * h16,
                  int N, void * stream);

/* Residual add + RMSNorm, dense form: x [n][N] += d (d nullable); h fp32 and h16 fp16 always written; N = 256 k <= 65536.
 * Replaces q35p_add_rms16, kernels/q35_prefill.hip:636-638 (n = grid.x); wrapper python/caminus/prefill/q35own.py:135-140. */
int q35p_add_rms16(int n, float * x, const float * d, const float * nw, float eps, float * h, void * h16, int N, void * stream);

/* The same statements on fp16 storage: x [n][N] fp16 (updated in place when d is given), d fp16 (nullable), h16 fp16.
 * xs = (float)x + (float)d; x = fp16(xs); h16 = fp16((xs * rsqrt(mean(xs^2) + eps)) * nw).
 * No kernel of this signature in the reference (its glue takes fp32 activations); arithmetic of
 * kernels/q35_prefill.hip:636-660 between an exact fp16 load and a rounded fp16 store. */
int cam_add_rms_f16(int n, void * x, const void * d, const float * nw, float eps, void * h16, int N, void * stream);

/* Tensor-parallel RMSNorm, hidden dimension sharded (Ns columns of Nfull on this rank, Ns a multiple of 8).
 * partial: ss [n] fp32 = this shard's sum of squares of xs = x + d (d nullable); nothing else is written.
 * apply (after ss was summed over the ranks into tot): x = fp16(xs) when d is given; h16 = fp16((xs * rsqrt(tot / Nfull +
 * eps)) * nw_shard). No counterpart in the reference, which replicates its norms on both cards
 * (python/caminus/engine/q3moe_tp.py:18-20). */
int cam_rms_partial_f16(int n, const void * x, const void * d, float * ss, int Ns, void * stream);
int cam_rms_apply_f16(int n, void * x, const void * d, const float * tot, const float * nw, float eps, void * h16, int Ns,
                      int Nfull, void * stream);

/* The tensor-parallel RMSNorm as one kernel per rank (no reference counterpart; one rank per GPU). Each rank's exchange buffer holds
 * cam_tp_rms_words(cap, world) 64-bit words (2 * world * cap exchange words and 8 of the library's own: a call's blocks are numbered
 * there in the order they start), zeroed once, and is mapped into every rank's process; peers is a device array of `world`
 * pointers to them (entry `rank` = the caller's own). A rank writes its per-row partial sums into every buffer by peer stores and
 * normalises a row when all ranks' partials have arrived; tag = the call's sequence number (1, 2, 3, ..: never 0, the same on every
 * rank; a call with n = 0 launches nothing and must not use a tag up). Waits are bounded (2 s, or CAMINUS_B200_TP_WAIT_MS milliseconds):
 * on expiry bit 0 of *status is set and the warp takes no more rows, so the call's rows are PARTLY updated: those normalised before
 * hold x = fp16(x + d) and their h16, a row whose partial had been sent may hold x = fp16(x + d) without its h16, the others are
 * untouched; a retry needs x restored from the caller's copy. n <= cap.
 * One exchange buffer serves every norm of a model: the buffer does not depend on the weights (caminus_b200.dist.TPExchange). */
int cam_ipc_open(const void * handle64, void ** base);      /* map another process's exported allocation (its 64-byte cudaIpcMemHandle_t) for the current device, peer access included */
int cam_ipc_close(void * base);
int cam_tp_rms_words(int cap, int world);
int cam_tp_rms_norm_f16(int n, void * x, const void * d, const float * nw, float eps, void * h16, int Ns, int Nfull, const void * peers, int rank,
                        int world, int cap, unsigned tag, int * status, void * stream);

/* The partial / apply pair above as ONE call that allocates nothing: the per-row sums of squares that pass from the first
 * kernel to the second live in a static device array inside the library (65536 floats, 256 KB per device that loads it)
 * instead of a caller's buffer. For callers that must not allocate device memory: a plugin working in buffers its engine
 * sized at start-up, or a process whose device memory is already fully handed out. x [n][N] fp16 (updated in place when d is
 * given), d fp16 (nullable), nw fp32 [N], h16 fp16 [n][N]; N a multiple of 8; same bytes as the pair with Ns = Nfull = N.
 * n > 65536 returns CAM_ERR_CAPACITY (split the batch). The first call on a device resolves the array's address: make it
 * before any stream capture. The address is kept per device ordinal for the life of the process: it does not survive a
 * cudaDeviceReset (a process that resets a device must not call this entry on it again). All calls on a device share the
 * array: calls that can overlap on the GPU race; order them. This entry has no counterpart in the reference. */
int cam_rms_norm_f16_static(int n, void * x, const void * d, const float * nw, float eps, void * h16, int N, void * stream);

/* y16[i] = fp16(silu(g[i]) * u[i]), i < n.
 * Replaces q3p_swiglu, kernels/q3m_prefill.hip:516-518; wrapper python/caminus/prefill/q3m_ops.py:106-107. */
int q3p_swiglu(const float * g, const float * u, void * y16, int n, void * stream);

/* h[i] = silu(g[i]) * u[i] in fp32.
 * Replaces gg_silu_mul, kernels/k3_gguf.hip:74-77; wrapper python/caminus/engine/gguf.py:57-61. */
int gg_silu_mul(const float * g, const float * u, float * h, int n, void * stream);

/* Q8_1 quantiser: n fp32 values -> ceil(n / 32) blocks of 36 bytes { fp16 d = amax / 127, fp16 sum, int8 qs[32] }; values
 * past n quantise as 0. Writes exactly ceil(n / 32) blocks (the reference's launch pads to a multiple of 8 blocks).
 * Replaces gg_quantize_q8_1, kernels/k3_gguf.hip:29-36; wrapper python/caminus/engine/gguf.py:39-46. */
int gg_quantize_q8_1(const float * x, void * y, int n, void * stream);

/* SwiGLU fused with the Q8_1 quantiser: blocks of silu(x[i]) * mul[i]. One launch for the reference's tape op OP_GG_Q8_1 with
 * work = 2 (kernels/k3_gguf_ops.h:55-77; built by Engine.gg_q8_1(x, yq, mul=u), python/caminus/engine/k3.py:649-659).
 * The _f16 form takes fp16 gate and up (widened exactly to fp32 first).
 * d and the 32 codes of every block are the bytes of the exact statements (a fast pass is used only where that is proven,
 * the rest is recomputed exactly: csrc/swiglu_q8.cu). The block sum may differ from the exact statements' by one fp16 ulp; the
 * reference reports that field and does not gate it (tests/engine/golden_util.py:145-146). The _strict forms run the exact
 * statements for every value (the sums are exact too) at about a third of the throughput. */
int gg_swiglu_q8_1(const float * x, const float * mul, void * y, long n, void * stream);
int gg_swiglu_q8_1_f16(const void * g, const void * u, void * y, long n, void * stream);
/* the same with the block sum proven as well: all 36 bytes of every block are the exact statements', at about four fifths of the copy bandwidth */
int gg_swiglu_q8_1_sums(const float * x, const float * mul, void * y, long n, void * stream);
int gg_swiglu_q8_1_f16_sums(const void * g, const void * u, void * y, long n, void * stream);
int gg_swiglu_q8_1_strict(const float * x, const float * mul, void * y, long n, void * stream);
int gg_swiglu_q8_1_f16_strict(const void * g, const void * u, void * y, long n, void * stream);
/* The same tape op with work = 1: blocks of silu(x[i] * rs) (ggml_scale, then ggml_silu, then the quantiser; kernels/k3_gguf_ops.h:70;
 * built by Engine.gg_q8_1(x, yq, silu_scale=rs), python/caminus/engine/k3.py:649-659). d and the codes are the exact statements' bytes;
 * the _sums form proves the block sum as well. */
int gg_silu_scale_q8_1(const float * x, float rs, void * y, long n, void * stream);
int gg_silu_scale_q8_1_sums(const float * x, float rs, void * y, long n, void * stream);
/* For tests: exact[i] = the exact statements' silu of fp16 gate g[i], fast[i] = the special-function evaluation the fused entries' fast
 * passes use. The fp16 entries' proofs rest on max |fast - exact| / |exact| <= 5.6e-7 over all gates >= -8 (measured: 5.43e-7 on sm_100a);
 * tests/test_gpu_enumerated.py checks it on the device it runs on. No counterpart in the reference. */
int cam_probe_silu_f16(const void * g, float * fast, float * exact, int n, void * stream);
/* Block sums of the Q8_1 entries above (gg_quantize_q8_1, gg_swiglu_q8_1*, gg_silu_scale_q8_1*): added in the order of the reference's
 * eight-lane quantiser aq_fill (kernels/k3_gguf_ops.h:83-120: four values per lane, then partners 4, 2, 1), which the reference itself
 * uses beside the lane butterfly of gg_op_q8_1 (kernels/k3_gguf_ops.h:55-77) and documents as bitwise-equivalent for every consumer:
 * the two orders can differ by one fp16 ulp in that field, never in d or the codes. cam_rms_mul_q8_1 uses the lane butterfly. */

/* Per-head q/k RMSNorm + NeoX RoPE. qkv fp32 [n][ldq] = q (nh heads of 128) | k (nkv) | v (nkv); q16 fp16 [n][nh][128];
 * cache fp16: row pos0 + t = K [nkv][128] | V [nkv][128] (V copied). par = q_norm[128] | k_norm[128] | theta_scale | eps
 * (the _yarn entry, the reference's q3m_prefill_yarn object: then freq[64] | mscale). The caller checks that rows
 * pos0 .. pos0 + n - 1 exist in the cache (the reference's wrapper does); pos0 + n <= 2^22.
 * Replaces q3p_qk_rope, kernels/q3m_prefill.hip:537-538 (n = grid.x, nh + nkv = grid.y); wrapper
 * python/caminus/prefill/q3m_ops.py:122-139. */
int q3p_qk_rope(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                void * stream);
int q3p_qk_rope_yarn(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                     void * stream);

/* The Q8_0 KV cache form: cache is a uint8 buffer of rows of 2 * (nkv * 128 / 32) * 34 bytes (Q8_0 blocks of K for all heads, then
 * of V); K and q16 are the 128-point Walsh-Hadamard transform of the fp16-rounded RoPE result, V the fp16-rounded values; err is
 * an int32 word a refused block (non-finite value, scale out of range) ORs 2 into, its bytes left alone.
 * Replaces q3p_qk_rope_q8, kernels/q3m_prefill.hip:534-535 (objects q3m_prefill_kvq8 / q3m_prefill_kvq8_yarn); codec
 * kernels/own_kv_codec.h:31-75, transform kernels/own_kv_rot128.h:21-33; wrapper python/caminus/prefill/q3m_ops.py:122-137. */
int q3p_qk_rope_q8(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache, int * err,
                   void * stream);
int q3p_qk_rope_q8_yarn(int n, const float * qkv, int ldq, int nh, int nkv, const float * par, int pos0, void * q16, void * cache,
                        int * err, void * stream);

/* The same statements on fp16 q [n][nh][128] and k [n][nkv][128], fp16 out (qo / ko may alias q / k); yarn as above.
 * No kernel of this signature in the reference; arithmetic of kernels/q3m_prefill.hip:552-590. */
int cam_qk_rope_f16(int n, const void * q, const void * k, int nh, int nkv, const float * par, int pos0, void * qo, void * ko,
                    int yarn, void * stream);

/* ---- the IQ4 row gathers of the host feed: kernels/prefill_feed.hip:24-54 (module prefill_feed). out fp32, bitwise the host decoders.
 * embd_rows_iq4xs: out [n][nblk * 256] = rows tok[p] of an IQ4_XS table (nblk * 136 bytes per row); a token outside [0, nvocab) is
 *   clamped and sets err |= 2. ple_rows_iq4nl: out [nrows][bpr * 32] = rows inv[r] of an IQ4_NL table (bpr * 18 bytes per row); an
 *   index outside [0, nuniq) is clamped and sets err |= 1. ---- */
int embd_rows_iq4xs(const void * table, const int * tok, int nvocab, int n, int nblk, float * out, int * err, void * stream);
int ple_rows_iq4nl(const void * raw, const int * inv, int nuniq, int nrows, int bpr, float * out, int * err, void * stream);
/* cam_emb_rows_q6k: the Q6_K row gather (210-byte blocks; the reference decodes this format on the host only:
 *   python/caminus/own_dequant.py:40-53, whose floats these are). x [n][N] = rows toks[i] (clamped to [0, vocab)) of a table of rb-byte rows. */
int cam_emb_rows_q6k(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, void * stream);
/* x [n][N] fp32 = the IQ2_S rows toks[i] of a table (82-byte blocks of 256; vocab rows of rb bytes), ids clamped to the vocabulary.
 * grid: 512 words on the device, GGUF's IQ2_S grid packed as the reference's kernels hold it (kernels/iq2s_grid.h: entry e = eight 2-bit
 * magnitude codes, entries 2 w and 2 w + 1 in word w); a constant of the reference's code object, the caller's argument here.
 * Replaces q35t_emb_iq2s, kernels/q35_prefill_tcap.hip:94-113 (= q35t_op_emb, kernels/k3_q35t_ops.h:147-175); n = grid.x. */
int q35t_emb_iq2s(int n, const void * W, int rb, int vocab, const int * toks, float * x, int N, const unsigned int * grid, void * stream);

/* ---- the router glue of the Qwen3-MoE prefill: kernels/q3m_prefill.hip:417-513; wrappers python/caminus/prefill/q3m_ops.py:94-104 ----
 * q3p_router: logits [n][E] = h [n][K] . Wr [E][K] in fp32 (n = grid.x; K a multiple of 128).
 * q3p_topk: per token softmax over E <= 128 logits, the k <= 32 most probable (ties: lower index first), ids int32 [n][k], wts =
 *   p / max(sum of the k, floor_); err |= 1 for a logit that is not finite (n = grid.x).
 * q3p_group: the n * k (token, slot) pairs grouped by expert: xs[i] = token, yd[i] = pair, work items { int e, off, cnt, pad } of at
 *   most 64 pairs, their count in *nitems; an id outside [0, E) sets err |= 2 and counts as expert 0. Every expert's list is in
 *   ascending pair order (the reference's follows its atomics). One cluster of at most 8 blocks; E <= 1024.
 * pf_router: the hyper-connection line's softmax + top-k, kernels/prefill_glue.hip:242-308 (T = grid.x); wrapper Glue.router,
 *   python/caminus/prefill/glue.py:182-192: E <= 1024 logits per token, k <= min(64, E) ids and weights p / max(sum of the k, clamp) in
 *   rank order; err |= 1 for a logit that is not finite (the ids of such a token are still k distinct experts below E). */
int q3p_router(int n, const float * h, const float * Wr, int E, int K, float * logits, void * stream);
int q3p_topk(int n, const float * logits, int E, int k, float floor_, int * ids, float * wts, int * err, void * stream);
int q3p_group(const int * ids, int npairs, int k, int E, int * xs, int * yd, void * items, int * nitems, int * err, void * stream);
int pf_router(int T, const float * logits, int E, int k, float clamp, int * ids, float * wts, int * err, void * stream);

/* ---- Q8_1 in the MMQ layout (block_q8_1_mmq, kernels/ggml_mmq/mmq.cuh:63-82): blocks [Kpad / 128][rows] of 144 bytes = 16 bytes of
 * per-32 scales + 128 int8; d_inv = 127 / amax, q = roundf(x * d_inv), d = 1 / d_inv. layout 0 = D4 (four fp32 d), 1 = DS4 (four
 * (fp16 d, fp16 sum)). x rows of stride ld, kvalid values each (a multiple of 4), zero-padded to Kpad (a multiple of 128). An
 * all-zero group stores d = 0 and codes 0.
 * cam_quantize_mmq_q8_1 replaces the dense case of quantize_mmq_q8_1, kernels/ggml_mmq/quantize_mmq.cuh:41-140.
 * cam_swiglu_mmq_q8_1[_f16] write the blocks of silu(g) * u: the epilogue of the reference's fused gate / up kernel,
 * kernels/prefill_moe.hip:339-396, as a standalone producer. ---- */
int cam_quantize_mmq_q8_1(const float * x, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream);
int cam_swiglu_mmq_q8_1(const float * g, const float * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream);
int cam_swiglu_mmq_q8_1_f16(const void * g, const void * u, void * y, int kvalid, int Kpad, long ld, int rows, int layout, void * stream);
/* The fused producer with a row index: column c of y (ncols columns) = the blocks of silu(g) * u of row ids[c] of gate and up (ids null:
 * row c; an index outside [0, ncols) is clamped): expert-grouped columns, as the reference's fused gate / up kernel writes column
 * c0 + j of its work item (kernels/prefill_moe.hip:389-394) and its unfused path gathers rows through the quantiser's index
 * (python/caminus/prefill/mmq.py:245-262). gate and up hold ncols rows of stride s01; K values per row (a multiple of 4). */
int cam_swiglu_mmq_q8_1_ids(const float * g, const float * u, const int * ids, void * y, int K, int Kpad, long s01, int ncols, int layout, void * stream);
int cam_swiglu_mmq_q8_1_f16_ids(const void * g, const void * u, const int * ids, void * y, int K, int Kpad, long s01, int ncols, int layout, void * stream);
/* The indexed forms of quantize_mmq_q8_1 (kernels/ggml_mmq/quantize_mmq.cuh:41-140; instances kernels/prefill_mmq.hip:101-107; wrappers
 * Mmq.quantize / Mmq.quantize_scatter, python/caminus/prefill/mmq.py:245-281). _ids: column c of y (ncols columns) = row ids[c] of x
 * (ids null: row c; x holds ncols rows of stride s01). _scatter: row t of x (ntok rows of stride s_tok) is quantised once and written
 * to the k columns ids_inv[t k + slot] of y (ntok k columns). An index outside its range is clamped. */
int cam_quantize_mmq_q8_1_ids(const float * x, const int * ids, void * y, int K, int Kpad, long s01, int ncols, int layout, void * stream);
int cam_quantize_mmq_q8_1_scatter(const float * x, const int * ids_inv, void * y, int K, int Kpad, long s_tok, int ntok, int k, int layout,
                                  void * stream);

/* ---- the hyper-connection ("Coder") line's glue: kernels/prefill_glue.hip; wrappers python/caminus/prefill/glue.py:143-313 ----
 * The reference bakes the row width (GLUE_NI x 256 = 2560 / 2048 / 5120) into three code objects; here it is the last argument
 * before the stream (K, N <= 8192). Optional outputs are null pointers. bf16 buffers are raw bits (void *). */

/* y[r] = (x[r] * rsqrt(mean(x[r]^2) + eps)) * w[r % wr]; outputs optional: y fp32 (may be x), ybf its bf16 copy (round to
 * nearest even), scl [R] the row scale. Replaces pf_rms_mul, kernels/prefill_glue.hip:94-95 (= op_rms_mul, k3_gguf_ops.h:1230-1268). */
int pf_rms_mul(const float * x, const float * w, float * y, void * ybf, float * scl, int R, int wr, float eps, int K, void * stream);
/* pf_rms_mul's norm that also emits the Q8_1 copy of the normed rows (36-byte blocks, the bytes gg_quantize_q8_1 gives for y) for the
 * quantised matvec that follows: the decode op's op_rms_mul with its q8_emit_n, kernels/k3_gguf_ops.h:178-196, 1253. y optional. */
int cam_rms_mul_q8_1(const float * x, const float * w, float * y, void * yq, int R, int wr, float eps, int K, void * stream);
/* res[t, h] = b[t] * 2 sigmoid(inj[t, h] * rs) + res[t, h] in place, then that row's norm with w[h]: xn fp32, xnbf bf16, scl,
 * each optional. Replaces pf_hc_post_rms, kernels/prefill_glue.hip:130-131. */
int pf_hc_post_rms(const float * b, const float * inj, float * res, const float * w, float * xn, void * xnbf, float * scl, int T, int HC,
                   float rs, float eps, int N, void * stream);
/* The residual update alone / the stream mix out = rs * sum_h xn * sigmoid(g) (xn given, or recomputed as (x * scl) * w when scl
 * is not null) / y = y + (a + b). Replace pf_hc_post, pf_hc_mean, pf_add_sum, kernels/prefill_glue.hip:175-176, 194-195, 417. */
int pf_hc_post(const float * b, const float * inj, float * res, int T, int HC, int D, float rs, void * stream);
int pf_hc_mean(const float * x, const float * scl, const float * w, const float * g, float * out, int T, int HC, int D, float rs, void * stream);
int pf_add_sum(const float * a, const float * b, float * y, long n, void * stream);
/* y [Tpad, K] bf16 = bf16(silu(fma(rs, x, 0))) / bf16(x) for the T rows of x (row stride ldx), zero rows up to Tpad.
 * Replace pf_silu_bf16, pf_to_bf16, kernels/prefill_glue.hip:554, 561. */
int pf_silu_bf16(const float * x, int ldx, void * y, int T, int Tpad, int K, float rs, void * stream);
int pf_to_bf16(const float * x, int ldx, void * y, int T, int Tpad, int K, void * stream);
/* y = silu(g) * u in fp32. Replaces pf_swiglu, kernels/prefill_tp.hip:37-43. */
int pf_swiglu(const float * g, const float * u, float * y, long n, void * stream);
/* Generic per-head RMSNorm + partial NeoX rotation, fp32 out: block t = row * heads + head reads D <= 512 floats at
 * xin + t * head_stride, rotates the first nrot dims (pairs j, j + nrot / 2) at position pos0 + t / heads.
 * Replaces pf_qk_nr, kernels/prefill_attn.hip:105-106 (= op_qk_nr, kernels/k3_gguf_ops.h:1490-1518); nblocks = grid.x. */
int pf_qk_nr(int nblocks, const float * xin, int head_stride, int heads, const float * w, int D, int nrot, float theta_scale, float eps,
             int pos0, float * out, void * stream);

/* ---- the training line's forwards: kernels/core.hip:23-66 (launched by runtime/s1.cpp:14-18, 31, 106), kernels/fuse.hip:19-33 ---- */
int embedding_f32(int T, const int * tok, const float * emb, float * out, int D, void * stream);                 /* T = grid.x */
int rmsnorm_f32(int rows, const float * x, const float * w, float * out, int D, float eps, void * stream);     /* rows = grid.x */
int silu_mul_bf16(const void * gu, void * act, int H, long n, void * stream);      /* act = bf16(bf16(silu(g)) * u), rows [g | u] */
int residual3(const float * x, const void * m, const void * y, float * out, long n, void * stream);            /* (x + m) + y */
int cast_bf16(const float * x, void * out, long n, void * stream);
/* out = ((x + m) + mlp) + (pos[r] >= 0 ? ys[pos[r]] : 0); m, mlp, ys bf16; ys, pos nullable; d a multiple of 4.
 * Replaces residual_slices_fwd, kernels/fuse.hip:19-20; wrapper python/caminus/train/fuse.py:19-30. */
int residual_slices_fwd(const float * x, const void * m, const void * mlp, const void * ys, const int * pos, float * out, int d, long n4,
                        void * stream);

/* ---- the training line's activation quantiser, forward: kernels/actq.hip:96-132, 247-274, 307-326; wrappers
 * python/caminus/train/actq.py:22-169. Per row of K (a multiple of 128, <= 8192): u = bf16(FWHT128(bf16(src)) * bf16(1 / sqrt(128)));
 * s = max(amax * clip / qmax, 1e-8); q = clamp(rint(u / s), -qmax - 1, qmax), qmax <= 7; y = bf16(q * s) (bf16 [M][K], nullable when
 * codes are written), s [M], codes = the int4 codes packed two per byte along K (nullable). M = the reference's grid.x. ---- */
int actq_fwd_bf16(int M, const void * x, void * y, float * s, int K, float clip, int qmax, void * stream);
int actq_fwd_f32(int M, const float * x, void * y, float * s, int K, float clip, int qmax, void * stream);
int actq_fwd_codes_bf16(int M, const void * x, void * y, float * s, void * codes, int K, float clip, int qmax, void * stream);
int actq_fwd_codes_f32(int M, const float * x, void * y, float * s, void * codes, int K, float clip, int qmax, void * stream);
/* the source is the MLP activation bf16(bf16(silu(g)) * u) of rows gu = [g | u] (bf16, row stride ld), never materialised */
int silu_mul_actq_fwd(int M, const void * gu, int ld, int F, void * y, float * s, void * codes, float clip, int qmax, void * stream);
/* the source is RMSNorm(x) = (x * rstd) * nw, never materialised; rstd_out [M]; nab <= 16 gate projections
 * ab[j] = bf16(sum_k bf16(h_k) * wab[j][k]) (wab bf16 [nab][d], ab bf16 [M][nab]; both null when nab = 0) */
int block_entry_fwd(int M, const float * x, const float * nw, const void * wab, int nab, float eps, void * y, float * s, void * codes,
                    void * ab, float * rstd_out, int d, float clip, int qmax, void * stream);

#ifdef __cplusplus
}
#endif
#endif
