/* The f16 activation layout the prefill matrix products read, and the conversions into it.
 *
 * Drop-in for the reference's include/osmos/gpu/mm.h: the activation side mm_x16 (:13), mm_x16_rows (:35),
 * mm_x16_heads (:37) with the layout function of kernels/mm.h:41-51, and the products mm_known, mm_fits, mm_run,
 * mm_run_silu, mm_run_gated_mean, mm_run2, mm_tokens[_scaled], mm_group (:10-38) - same names, argument meaning, limits and refusals. The products
 * compute what the reference's do - the weights' exact values rounded to f16, times the f16 activations,
 * accumulated in F32 - on the tensor cores, with the tensor core's order of additions along K instead of the
 * reference's wave partitions: results agree with the reference's within its own test bound
 * ((cols / 16 + 20) 2^-24 sum |w16 x16|, tests/gpu/test_mm_gpu.hip:328-343), not bit for bit; a token's results are
 * the same bits whatever it is batched with and wherever in the batch.
 *
 * x16 holds token t's column c, of rows xts values long, at half index
 *   (t / 16) * 16 * xts + (c / 16) * 256 + (t % 16) * 16 + c % 16
 * so every 16-token x 16-column fragment is 512 contiguous bytes. Values are rounded F32 -> f16 to nearest even; a
 * value past f16's range (or a NaN) sets *overflow (a device int32 the caller clears before the step and reads after
 * it: the step's results are then refused). Rows past the last token, up to the next multiple of 16, are zero.
 *
 * Every entry returns true when the work was queued on `stream` (a cudaStream_t, NULL = default stream; not waited
 * for) and false when it was refused - then nothing was queued.
 */
#ifndef OSMOS_B200_MM_H
#define OSMOS_B200_MM_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MM_TILE 16         /* reference: mm.h:7 */
#define MM_MAX_TOKENS 2048 /* reference: mm.h:8 */

#if defined(__CUDACC__)
#define MM_HD __host__ __device__
#else
#define MM_HD
#endif

/* where token t's column c lies in a tiled x16 of rows xts long, in halves (reference: kernels/mm.h:47-49) */
static inline MM_HD uint64_t mm_x16_at(uint32_t t, uint32_t c, uint32_t xts) {
  return (uint64_t)(t / MM_TILE) * MM_TILE * xts + (uint64_t)(c / MM_TILE) * (MM_TILE * MM_TILE) + (t % MM_TILE) * MM_TILE +
         c % MM_TILE;
}

/* n rows of cols F32 (row t at x + t * xs) into x16: n rounded up to whole tiles of rows, cols f16 each
   (reference: mm.h:13, mm.hip:467-479). false for n 0 or past MM_MAX_TOKENS, cols 0 or not a multiple of 16, or,
   with more than one row, xs shorter than a row. */
bool mm_x16(const float *x, uint32_t xs, uint32_t n, uint32_t cols, void *x16, int32_t *overflow, void *stream);
/* slot s is row idx[s] of x (-1: zeros; idx a device array of `slots` ints), slots rounded up to whole tiles
   (reference: mm.h:35, mm.hip:608-617). false for no slots, cols 0 or not a multiple of 16, xs shorter than a row or
   not a multiple of 4, or x not 16-byte aligned. */
bool mm_x16_rows(const float *x, uint32_t xs, const int32_t *idx, uint32_t slots, uint32_t cols, void *x16,
                 int32_t *overflow, void *stream);
/* every head's slice of n rows (head h's cols values at x + t * xs + h * hs) to its own tiled x16, head h's at
   x16 + h * n16 * cols halves, n16 = n in whole tiles: each as mm_x16(x + h * hs, xs, n, cols) would put it
   (reference: mm.h:37, mm.hip:593-606). false for n 0 or past MM_MAX_TOKENS, no heads, cols 0 or not a multiple of
   16, hs or xs not a multiple of 4, x or x16 not 16-byte aligned, or a last head reaching past a row. */
bool mm_x16_heads(const float *x, uint32_t xs, uint32_t n, uint32_t heads, uint32_t hs, uint32_t cols, void *x16,
                  int32_t *overflow, void *stream);

/* the attention's output to f16 on the way to its output projection (reference: mm.h:14-15, kernels/mm.hip:105-135,
   480-491): of every head (head_dim values of a row) the last rope_dim values rotated back - the pair (2i, 2i + 1) by
   the angle pos[t] * freqs[i], as (a cos + b sin, b cos - a sin) - then every 32 values rounded to E4M3 under the
   scale 2^ceil(log2(max(amax, 1e-4) / 448)) (ops_fp8_round's rule), then to f16 in mm_x16's layout and with its
   overflow flag. false for n 0 or past MM_MAX_TOKENS, cols not a multiple of head_dim, head_dim or head_dim - rope_dim
   not a multiple of 32, rope_dim odd or past head_dim, xs shorter than a row. The cosine and sine are the device
   library's: a result can differ from another library's by one E4M3 step where the rotated value lies on a
   rounding boundary. */
bool mm_x16_attn(const float *x, uint32_t xs, uint32_t n, uint32_t cols, uint32_t head_dim, uint32_t rope_dim,
                 const float *freqs, const int32_t *pos, void *x16, int32_t *overflow, void *stream);

/* whether `type` has a matrix-product kernel (every block type of qtype.h), and whether a rows x cols matrix of it
   tiles: rows a multiple of 16, cols a multiple of 128 and whole blocks (reference: mm.h:10-11) */
bool mm_known(uint32_t type);
bool mm_fits(uint32_t type, uint32_t rows, uint32_t cols);
/* the launch class of a matrix with n tokens - how many 128-token accumulators a block carries at most: 1, 2 or 4; 0
   for a type without a kernel (reference: mm.h:12, kernels/mm.hip:161-167, 455-465, where it is the column tiles a
   block takes). A caller sorts mm_group's matrices by count and makes one launch a run of equal classes
   (src/run/hip_ffn.c:110-127), so that a matrix of few tokens is not run in a kernel sized for many. */
uint32_t mm_col_tiles(uint32_t type, uint32_t n);
/* y[t * ys + r] = sum_c W[r, c] x16[t][c], t < n <= MM_MAX_TOKENS; x16 as mm_x16 lays it (rows of cols values)
   (reference: mm.h:15). false for a type without a kernel, a shape that does not tile, n 0 or past MM_MAX_TOKENS,
   with more than one token ys shorter than a row, or x16 not 16-byte aligned. */
bool mm_run(uint32_t type, const void *w, uint32_t rows, uint32_t cols, const void *x16, uint32_t n, float *y,
            uint32_t ys, void *stream);
/* mm_run with y = silu(y scale) as its epilogue - silu(v) = v / (1 + expf(-v)), every operation rounded by itself -
   written to y and, as f16, into x16_out (tiled as mm_x16 lays it, rows values wide, the overflow flag set past
   f16's range): the next product's activations in the same launch (reference: mm.h:27-29, kernels/mm.hip:493-501,
   the mixers' down). x16_out must not be x16. false - nothing queued, the caller's mm_run and its own silu pass
   then - past MM_SILU_MAX_TOKENS tokens, for a shape mm_run refuses, x16_out NULL / x16 / not 16-byte aligned, or no
   overflow word. Every type mm_run takes (the reference: Q8_0 alone). */
#define MM_SILU_MAX_TOKENS 64
bool mm_run_silu(uint32_t type, const void *w, uint32_t rows, uint32_t cols, const void *x16, uint32_t n, float *y,
                 uint32_t ys, float scale, void *x16_out, int32_t *overflow, void *stream);
/* the hyper-connection mixer's up (hc dim rows: hc streams of dim) with the gated mean as its epilogue:
   out[t][d] = (sum over s in order, from zero, of xn[t][s][d] sigmoid(up_t[s dim + d])) / hc, sigmoid(v) =
   1 / (1 + expf(-v)), every operation rounded by itself; and its f16 into out16 (dim wide, token t at row row0 + t;
   NULL: none). The up's own F32 output is never stored (reference: mm.h:30-33, kernels/mm.h:668-704). out16 must not
   be x16. false - nothing queued - for more than MM_GATED_MEAN_MAX_HC streams, dim not a multiple of MM_TILE, a
   shape mm_run refuses for hc dim rows, out16 without an overflow word. Every type mm_run takes. */
#define MM_GATED_MEAN_MAX_HC 8
bool mm_run_gated_mean(uint32_t type, const void *w, uint32_t hc, uint32_t dim, uint32_t cols, const void *x16,
                       uint32_t n, const float *xn, float *out, void *out16, uint32_t row0, int32_t *overflow,
                       void *stream);
/* two matrices of one type and cols on the same x16, each the bits mm_run gives it alone (reference: mm.h:23);
   refused as a whole when either would be */
bool mm_run2(uint32_t type, const void *w0, uint32_t rows0, float *y0, uint32_t ys0, const void *w1, uint32_t rows1,
             float *y1, uint32_t ys1, uint32_t cols, const void *x16, uint32_t n, void *stream);
/* a matrix (w1 NULL) or two over any n tokens of F32 x: MM_MAX_TOKENS at a time through the one x16 - mm_x16 of the
   chunk, then the products into its rows; `ready`: x16 already holds this x (n within one x16): the conversion is
   skipped. _scaled: each matrix's sums times its scale as they are stored (reference: mm.h:17-22) */
bool mm_tokens(uint32_t type, const void *w0, uint32_t rows0, float *y0, uint32_t ys0, const void *w1, uint32_t rows1,
               float *y1, uint32_t ys1, uint32_t cols, const float *x, uint32_t xs, uint32_t n, void *x16,
               int32_t *overflow, bool ready, void *stream);
bool mm_tokens_scaled(uint32_t type, const void *w0, uint32_t rows0, float *y0, uint32_t ys0, float s0, const void *w1,
                      uint32_t rows1, float *y1, uint32_t ys1, float s1, uint32_t cols, const float *x, uint32_t xs,
                      uint32_t n, void *x16, int32_t *overflow, bool ready, void *stream);
/* n_mat matrices of one type and shape: matrix m (w[m]) over the tiled x16 from x16 + xoff[m] halves (rows xts long),
   its first cnt[m] <= max_cnt tokens' rows into y + yoff[m] + t * ys; w, cnt, xoff, yoff device arrays
   (reference: mm.h:39-41). Each token the sums mm_run gives it. */
bool mm_group(uint32_t type, const void *const *w, const int32_t *cnt, uint32_t n_mat, uint32_t max_cnt, uint32_t rows,
              uint32_t cols, const void *x16, const uint32_t *xoff, uint32_t xts, float *y, const uint32_t *yoff,
              uint32_t ys, void *stream);
/* NVFP4 weights times NVFP4 activations, W4A4 (reference: include/osmos/gpu/mm.h:45-61, kernels/mm_fp4.hip).
   mm_fp4_ok: whether this device runs the path (the reference's answers true on sm_120a only; this one on sm_100a).
   mm_fp4_quant: x's n rows (F32, or (bf16) BF16 as 16-bit words; stride xs elements) quantized under the input scale gs
   (or *gs_dev, a device float) as ModelOpt's activations: every 16 values an E4M3 scale byte into sc (n x cols / 16),
   E2M1 codes two a byte in k order, the low nibble first, into q (n x cols / 2); sr_seed 0 rounds to nearest (ties to
   the even index), else stochastically under the seed. mm_fp4_act: F32, nearest, a host scale. Bit for bit the
   reference's bytes. false without the device, for cols not whole 64s, a scale not above 0, xs shorter than a row,
   or q not 8-byte aligned.
   mm_fp4: y[t * ys + r] = scale * sum_c W[r, c] xq[t, c] over any n tokens, W an NVFP4 (QTYPE_NVFP4) matrix, xq the
   values (q, sc) hold; the tensors' scales (the weight's and the input's) belong in `scale`. Both sides' values are
   exact in f16 and go through the f16 tensor-core product (every product exact, F32 sums): within the reference's own
   bound (1e-5 relative to float64 sums, tests/gpu/test_mm_fp4_gpu.hip:150), not its bits. Shapes as mm_fits takes
   them (rows in 16s, cols in 128s; the reference: 8s and 64s). The step's f16 activations live in a stream-ordered
   allocation made and freed by the call.
   On whole 128-row tiles and 256-value steps of K the product runs on the block-scaled FP4 tensor-core instruction
   (tcgen05.mma kind::mxf4nvf4: E2M1 x E2M1 under a UE4M3 factor every 16 values on each side, F32 sums), the counterpart
   of the reference's mma.sync kind::mxf4nvf4 kernel (kernels/mm_fp4.hip:149-259); other shapes take the f16 route.
   mm_fp4_set_tensor(0) keeps every shape on the f16 route (the tests compare the two routes). */
bool mm_fp4_ok(void);
bool mm_fp4_act(const float *x, uint32_t xs, uint32_t n, uint32_t cols, float gs, void *q, void *sc, void *stream);
bool mm_fp4_quant(const void *x, uint32_t bf16, uint32_t xs, uint32_t n, uint32_t cols, float gs, const float *gs_dev,
                  uint32_t sr_seed, void *q, void *sc, void *stream);
bool mm_fp4(const void *w, uint32_t rows, uint32_t cols, const void *q, const void *sc, uint32_t n, float scale,
            float *y, uint32_t ys, void *stream);
void mm_fp4_set_tensor(int on);
/* which route mm_fp4's last call took: 1 the block-scaled FP4 MMA, 0 the f16 product, -1 no call yet (for the tests) */
int mm_fp4_last_route(void);
/* Not in the reference (it never feeds quantized activations to an MXFP4 product: kernels/mm.hip:426 decodes the weights
   to f16): MXFP4 weights (QTYPE_MXFP4) times MXFP4 activations, W4A4, on tcgen05.mma kind::mxf4 (E2M1 x E2M1 under a UE8M0
   factor every 32 values on each side, F32 sums). `packed` is what ops_fp4_round(x, n * cols, 32, false, packed, cols)
   writes: a token's cols / 2 code bytes (the even value in the low nibble), then its cols / 32 scale bytes.
   y[t * ys + r] = scale * sum_c W[r, c] xq[t, c]. false without the device, for rows not whole 128s, cols not whole 512s,
   n 0, ys shorter than a row with more than one token, or packed / w not 16- / 4-byte aligned. */
bool mm_mxfp4(const void *w, uint32_t rows, uint32_t cols, const void *packed, uint32_t n, float scale, float *y,
              uint32_t ys, void *stream);
/* the block-scaled MMA's 32-bit instruction descriptor as the kernel builds it (M 128, N n, E2M1 operands; mx: UE8M0
   factors every 32, else UE4M3 every 16; sf_id: the first factor's byte in its word) - for the host test against
   CUTLASS's encoder */
uint32_t mm_fp4_desc(uint32_t mx, uint32_t n, uint32_t sf_id);
/* Not in the reference: the products' kernel never waits without a bound; reads and clears the current device's
   record (synchronizes): bit 0 a wait ran out, the launch's outputs are not valid */
uint32_t mm_status(void);

#ifdef __cplusplus
}
#endif

#endif
