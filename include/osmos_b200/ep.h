/* Expert-parallel pieces of the routed-expert layer: one process per GPU, experts in contiguous ranges per rank,
 * tokens by home rank. No counterpart in the reference (it is single-GPU: no collective, no peer API anywhere in
 * its tree); the arithmetic is q8.h's and the combine order is the single-GPU one, so the result has the same bits
 * on any number of GPUs.
 *
 * A step on rank r (T = its home tokens, N ranks, k picks a token, E experts):
 *   1. q4x_route and q8_round on its T tokens, written straight into its segment of the dispatch buffer
 *      (ep_segment_bytes; ids, weights, int8 rows, scales);
 *   2. all-gather of the segments (NCCL), ep_unpack -> every token's ids / weights / int8 row / scales, token-major;
 *   3. lane_ffn_rows: the rows whose expert lies in [e0, e1) through gate / up / activation / down;
 *   4. ep_scatter_rows: row of pick (t, j) -> send[home(t)][(t mod T) * k + j];
 *   5. all-to-all of send (NCCL): recv[o] = what rank o computed for this rank's tokens;
 *   6. ep_combine: each home token's k rows, taken from their owners' blocks, added in ascending expert id.
 * The two exchanges have a second form that does not go through a collective library: every rank maps its peers'
 * buffers (CUDA IPC) and the producing kernels store straight into the consumer's memory over NVLink - ep_push for
 * step 2 (the segment to every rank), ep_scatter_rows_peer for steps 4 and 5 (a row to its token's home) - each
 * followed by a release of a per-sender flag in the consumer's memory, which the consumer's ep_wait polls locally
 * (bounded). Buffers are used in two alternating halves by step parity; a rank cannot run more than one step ahead of
 * a peer because it waits on that peer's flag every step, so a half is never overwritten while it is still read.
 * Every bool entry returns true when the work was queued on `stream`, false when it was refused (nothing queued).
 */
#ifndef OSMOS_B200_EP_H
#define OSMOS_B200_EP_H

#include <stdbool.h>
#include <stdint.h>

#include "osmos_b200/lane.h"

#ifdef __cplusplus
extern "C" {
#endif

/* a rank's dispatch segment for T tokens: [ids T*k i32][weights T*k f32][q T*dim i8][d T*(dim/32) f32], each part
   16-byte aligned; these give the parts' byte offsets and the segment's size (a multiple of 16) */
typedef struct EpSegment
{
  uint64_t ids, weights, q, d, bytes;
} EpSegment;
void ep_segment(uint32_t tokens, uint32_t k, uint32_t dim, EpSegment *s);

/* the gathered segments (n_ranks of them, rank-major) -> token-major arrays over all n_ranks * tokens tokens */
bool ep_unpack(const void *gathered, uint32_t n_ranks, uint32_t tokens, uint32_t k, uint32_t dim, int32_t *ids,
               float *weights, int8_t *q, float *d, void *stream);
/* rows -> the combine's send buffer: for every pick i (token t = i / k) with a row here (row_of[i] >= 0),
   send[(t / tokens) * tokens * k + (t % tokens) * k + i % k][:] = ye[row_of[i]][:] */
bool ep_scatter_rows(const float *ye, const int32_t *row_of, uint32_t n_picks, uint32_t k, uint32_t tokens,
                     uint32_t dim, float *send, void *stream);
/* out[t][:] = sum over this rank's token t's picks, in ascending expert id, of recv[owner][t * k + j][:], owner =
   expert / experts_per_rank; ids are the home tokens' picks [tokens * k]; add (or NULL) added after the sum */
bool ep_combine(const float *recv, const int32_t *ids, uint32_t tokens, uint32_t k, uint32_t experts_per_rank,
                uint32_t dim, const float *add, float *out, void *stream);

/* ---- the peer transport ---------------------------------------------------------------------------------------- */
#define EP_MAX_RANKS 16
#define EP_HANDLE_BYTES 64 /* a CUDA IPC memory handle */
/* set-up, not the step: a zeroed device buffer other processes of this machine can map, and its handle; a peer's
   buffer mapped from its handle (peer access enabled with it); their release. false when the CUDA call failed. */
bool ep_peer_alloc(uint64_t bytes, void **ptr, uint8_t handle[EP_HANDLE_BYTES]);
bool ep_peer_open(const uint8_t handle[EP_HANDLE_BYTES], void **ptr);
bool ep_peer_close(void *ptr);
bool ep_peer_free(void *ptr);
/* `bytes` (a multiple of 16) of src, local, to dst[r] for every r < n_ranks (dst, flag: device arrays of addresses,
   dst[r] and flag[r] inside rank r's memory - this rank's own included); when all of it is written and fenced,
   *flag[r] = step for every r. counter: a zeroed local device word the kernel uses and leaves zero. */
bool ep_push(const void *src, uint64_t bytes, void *const *dst, uint32_t *const *flag, uint32_t n_ranks, uint32_t step,
             uint32_t *counter, void *stream);
/* returns (on the stream) once flags[r] has reached `step` for every r < n_ranks - flags local, written by the
   peers' ep_push / ep_scatter_rows_peer - or after the wait limit (2 s), which ep_wait_status() then reports (bit 0;
   read and cleared, it synchronizes) */
bool ep_wait(const uint32_t *flags, uint32_t n_ranks, uint32_t step, void *stream);
uint32_t ep_wait_status(void);
/* ep_scatter_rows without the send buffer: the row of pick (t, j) goes to recv[t / tokens] + ((t % tokens) * k + j) *
   dim floats, recv[r] = where this rank's block lies in rank r's memory; then the flags as ep_push */
bool ep_scatter_rows_peer(const float *ye, const int32_t *row_of, uint32_t n_picks, uint32_t k, uint32_t tokens,
                          uint32_t dim, float *const *recv, uint32_t *const *flag, uint32_t n_ranks, uint32_t step,
                          uint32_t *counter, void *stream);

/* ---- the whole step in five dependent launches and one C call ---------------------------------------------------
 * The peer transport with each exchange folded into the kernel that produces or consumes its data:
 *   1. ep_route_round_push   q4x_route + q8_round of the home tokens, every result stored straight into EVERY rank's
 *                            exchange buffer (token-major over all tokens of the step: nothing is unpacked later),
 *                            then this rank's dispatch flag released in every buffer;
 *   2. ep_lane_tables        a bounded wait on all dispatch flags at its head, then lane_tables for this rank's
 *                            experts and, for each row, the address of its place in its token's home rank;
 *   3. ep_gate_up            q8_gate_up on the gathered tokens;          4. q8_round of the activations;
 *   5. ep_down_push          q8_group_tok (down) whose epilogue stores each finished row into its home rank's
 *                            receive block, the last block releasing this rank's combine flag in every buffer;
 *   6. ep_combine_wait       a bounded wait on all combine flags, then each home token's k rows added in ascending
 *                            expert id (+ add).
 * The step number lives on the device (launch 1 advances it), and the buffers' halves are chosen from its parity
 * inside the kernels, so a step's launches never change and can be captured in a CUDA graph. A wait that runs out
 * (2 s) sets bit 0 of ep_wait_status() and lets the stream go on. With one rank the same launches run with the flags
 * always already there: the single-GPU layer is this step with n_ranks = 1. */
typedef struct EpLayout /* byte offsets inside a rank's exchange buffer; the same on every rank */
{
  uint64_t flags_dispatch, flags_combine; /* n_ranks words each: word s written by rank s */
  uint64_t ids[2], weights[2], q[2], d[2]; /* all tokens' picks, routed weights, int8 rows, scales; by step parity */
  uint64_t recv[2];                        /* this rank's home tokens' rows [tokens * k][dim] F32; by step parity */
  uint64_t bytes;
} EpLayout;
/* n_tok tokens in all (a multiple of n_ranks), k picks a token, rows of dim values. false for a shape it refuses. */
bool ep_layout(uint32_t n_ranks, uint32_t n_tok, uint32_t k, uint32_t dim, EpLayout *l);

typedef struct EpPlan /* host memory; made once, read by every step */
{
  uint32_t rank, n_ranks;
  uint32_t n_tok;            /* tokens of a step over all ranks; rank r is home to [r, r + 1) * n_tok / n_ranks */
  uint32_t expert0, expert1; /* this rank's experts */
  EpLayout lay;
  void *peer[EP_MAX_RANKS]; /* every rank's exchange buffer (lay.bytes, zeroed, 256-byte aligned) as mapped here */
  uint32_t *sync;           /* device, this rank's: 4 zeroed words ([0] the step counter, [1] [2] publish counters) */
  float **rows;             /* device scratch, 2 * n_tok * k words of 8 bytes: where each of this rank's rows goes, and
                               after those n_tok * k addresses the rows' routed weights (F32) */
  LaneLayer layer;          /* the layer (its experts' addresses as this rank holds them) */
  LaneScratch scratch;      /* lane_scratch_bind's, for n_tok tokens */
  uint32_t router;          /* EP_ROUTER_*: q4x_route's softmax, or ops_router's scores */
  const float *route_bias;  /* device [n_exp]: the scored routers' bias */
  float route_scale;        /* the scored routers' weight scale */
} EpPlan;
#define EP_ROUTER_SOFTMAX 0      /* q4x_route */
#define EP_ROUTER_SQRT_SOFTPLUS 1 /* ops_router (DeepSeek's); at most 16 picks a token */
#define EP_ROUTER_SIGMOID 2      /* ops_router_scored with sigmoid scores */

/* x, logits, add (or NULL), out: this rank's home tokens ([n_tok / n_ranks][dim], [..][n_exp], [..][dim]).
   false = refused, nothing queued (a plan, type or shape the fused kernels do not take: use the unfused entries). */
bool ep_layer_step(const EpPlan *p, const float *x, const float *logits, const float *add, float *out, void *stream);
/* true when ep_layer_step takes the plan (checked by ep_layer_step itself before its first launch) */
bool ep_plan_ok(const EpPlan *p);
/* the step's stages, queued one after another by ep_layer_step (libosmos_b200/host/ep_step.c) */
bool ep_route_round_push(const EpPlan *p, const float *x, const float *logits, void *stream);
bool ep_lane_tables(const EpPlan *p, void *stream);
bool ep_gate_up(const EpPlan *p, void *stream);
bool ep_down_push(const EpPlan *p, void *stream);
bool ep_combine_wait(const EpPlan *p, const float *add, float *out, void *stream);
/* this rank's picks of the last step copied to host arrays [n_tok / n_ranks][k] (for checks; synchronizes the device) */
bool ep_last_picks(const EpPlan *p, int32_t *ids, float *weights);

/* lane_ffn's middle for one rank: tokens already rounded (q, d, token-major), the rows of experts [e0, e1) into
   s->ye (row r = the r-th of those picks sorted by (expert, pick)); s->tab.row_of says which row a pick got */
bool lane_ffn_rows(const LaneLayer *l, const LaneScratch *s, const int8_t *q, const float *d, const int32_t *ids,
                   const float *weights, uint32_t n_tok, uint32_t e0, uint32_t e1, void *stream);

#ifdef __cplusplus
}
#endif

#endif
