/*
 * C ABI of libcuda_agent_b200.so: the kernel launchers of the B200 (sm_100a)
 * operators that sit behind the agent_workdir binding API.
 *
 * Convention (reference: agent_workdir/kernels/axpby.cu:12-20 and the extern
 * declaration a binding file repeats, agent_workdir/kernels/axpby_binding.cpp:7-15):
 *   extern "C" <op>_launcher(raw device pointers, sizes, scalars, int config,
 *                            cudaStream_t stream)
 * - every pointer is a device pointer owned by the caller; nothing is copied,
 *   nothing is allocated unless a launcher's comment says so;
 * - work is enqueued on `stream` and the call returns without synchronising;
 * - `config` selects a launch variant of the same arithmetic (tuning knob,
 *   agent_workdir/kernels/axpby.cu:22-41); every value gives identical results
 *   unless stated otherwise; unknown values fall back to the default variant.
 * The reference launcher returns void and checks nothing. These return an int
 * status (CAB_OK == 0) so that a binding can raise; a caller that ignores the
 * return value sees the reference behaviour.
 *
 * No torch type appears here. `cudaStream_t` is spelled as an opaque pointer so
 * the header is usable from plain C and from ctypes/cffi.
 */
#ifndef CUDA_AGENT_B200_H_
#define CUDA_AGENT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same type that cuda_runtime.h names cudaStream_t (driver_types.h:
 * `typedef struct CUstream_st* cudaStream_t`), spelled out so that this header
 * needs no CUDA header. */
typedef struct CUstream_st* cab_stream_t;

/* 16-bit storage types: raw IEEE bfloat16 bits / e4m3 bytes. */
typedef uint16_t cab_bf16;
typedef uint8_t cab_e4m3;

enum cab_status {
  CAB_OK = 0,
  CAB_ERR_BAD_ARGUMENT = 1,   /* null pointer, non-positive size, unsupported head size ... */
  CAB_ERR_MISALIGNED = 2,     /* a pointer that must be 16-byte aligned is not */
  CAB_ERR_LAUNCH = 3,         /* cudaGetLastError() was non-zero after the launch */
  CAB_ERR_TOO_LARGE = 4,      /* a size exceeds what the entry point supports */
  CAB_ERR_DEVICE_STATUS = 5   /* a kernel's own bounded wait or index check gave up */
};

/* Human-readable text for a status code (static storage). */
const char* cab_status_string(int status);

/* Library version as major*10000 + minor*100 + patch. */
int cab_version(void);

/* Self-test of the bounded waits inside the tensor-core kernels (no counterpart */
/* in the reference, whose one kernel never waits). One small CTA waits on a      */
/* barrier for at most limit_cycles clock cycles (1 .. 1e9); with withhold != 0    */
/* the barrier's last arrival never comes, the wait gives up, *status (device int) */
/* becomes 901 and the kernel returns through its normal teardown; with withhold   */
/* == 0 the wait completes and *status stays 0. The device stays usable either way. */
int cab_wait_selftest(int* status, long long limit_cycles, int withhold, cab_stream_t stream);

/* ------------------------------------------------------------------------- */
/* axpby: the workspace's smoke-test op.                                      */
/* Replaces agent_workdir/kernels/axpby.cu:12-42 (same argument order).       */
/* out[i] = alpha * a[i] + b[i], fp32. config: 0 -> 256, 1 -> 128, 2 -> 512    */
/* threads per block. size <= 0 is a no-op returning CAB_OK.                  */
/* ------------------------------------------------------------------------- */
int axpby_launcher(float* out, const float* a, const float* b, float alpha, int size, int config,
                   cab_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Gated DeltaNet single-step decode.                                         */
/* The reference ships no such op; this fills the slot an op occupies in       */
/* agent_workdir/kernels/ (launcher ABI as above) for the eager statement      */
/*   alpha = exp(g);  u = S k;  S' = alpha*S + beta*(v - alpha*u) k^T;          */
/*   o = S' q / sqrt(128)                                                      */
/* per (batch b, value head hv), which equals                                  */
/*   S' = alpha * S (I - beta k k^T) + beta v k^T.                             */
/*                                                                             */
/* state : fp32 [B, Hv, 128 (dv), 128 (dk)] row-major, UPDATED IN PLACE        */
/* out   : fp32 [B, Hv, 128]                                                   */
/* q, k  : bf16 [B, Hq, 128]  (value head hv reads q/k head hv / (Hv/Hq))      */
/* v     : bf16 [B, Hv, 128]                                                   */
/* g     : fp32 [B, Hv]  log-decay (<= 0);   beta : fp32 [B, Hv]               */
/* Requires Hv % Hq == 0; state and out 16-byte aligned, q/k/v 8-byte aligned. */
/* config: 0 default: 256-bit accesses, a half-warp per state row, 16 rows in    */
/* flight per warp (needs state 32-byte and q/k 16-byte aligned, else config 4   */
/* is used); 3: the same with 8 rows in flight; 1 / 4 / 2: 128-bit accesses, a    */
/* warp per row, 4 / 8 / 16 rows in flight. Configs 1, 2, 4 give identical bits;  */
/* 0 and 3 reduce the dot products in a different order and agree with them to    */
/* fp32 rounding. One launch reads and writes each state element exactly once.   */
/* The low four bits of config are that choice. Bit 4 (16), with configs 0 / 3:   */
/* walk the (b, hv) units from the last to the first. A decode loop that flips it  */
/* from step to step (0, 16, 0, ...) starts every step on the rows the previous    */
/* one wrote last, of which about 80 MB are still in L2. The result of a step does */
/* not depend on the bit.                                                          */
/* ------------------------------------------------------------------------- */
int gdn_decode_launcher(float* state, float* out, const cab_bf16* q, const cab_bf16* k,
                        const cab_bf16* v, const float* g, const float* beta, int B, int Hq,
                        int Hv, int config, cab_stream_t stream);

/* ------------------------------------------------------------------------- */
/* FP8 block-scaled MoE layer. The reference ships no such op; each launcher   */
/* below fills the slot agent_workdir/kernels/<op>.cu gives a kernel (launcher */
/* ABI of agent_workdir/kernels/axpby.cu:12-20), one per stage of               */
/*   logits -> top-k routing -> stable expert permutation -> 1x128 e4m3         */
/*   quantise + dispatch -> grouped FP8 GEMM (gate/up, SwiGLU, re-quantise) ->  */
/*   grouped FP8 GEMM (down) -> weighted combine.                               */
/* Shapes: T tokens, hidden H, expert intermediate I, E experts (<= 256),      */
/* k experts per token (<= 32).                                                */
/* ------------------------------------------------------------------------- */

/* logits[T,E] (fp32) = x[T,H] (bf16) . wr[E,H]^T (bf16), fp32 accumulation.   */
/* H % 32 == 0, E % 8 == 0; x and wr 16-byte aligned. Batches of 512 tokens or   */
/* more with E % 32 == 0, E <= 256 and H % 64 == 0 run on tcgen05 (TMA-fed, one   */
/* accumulation chain per element); config 1 keeps the mma.sync kernel for every   */
/* shape. Both sum in fp32; they agree to summation-order noise.                   */
int moe_router_logits_launcher(float* logits, const cab_bf16* x, const cab_bf16* wr, int T, int H,
                               int E, int config, cab_stream_t stream);

/* Softmax routing: topk_idx[T,k] (int32) = the k largest logits per token in   */
/* descending order, equal logits -> lower expert id first; topk_w[T,k] (fp32)  */
/* = softmax over those k logits (the full softmax renormalised to sum 1).      */
int moe_route_softmax_topk_launcher(int* topk_idx, float* topk_w, const float* logits, int T, int E,
                                    int k, int config, cab_stream_t stream);

/* Sigmoid routing with a bias and group restriction: s = sigmoid(logit)        */
/* (evaluated in fp64, rounded to fp32), c = s + bias[e]; experts form n_group   */
/* contiguous groups; a group scores the sum of its two largest c; the          */
/* topk_group best groups are kept (ties -> lower group); topk_idx = the k       */
/* largest c among kept groups (descending, ties -> lower id);                   */
/* topk_w = s[idx] / sum(s[idx]) * routed_scaling_factor. n_group <= 32.         */
int moe_route_sigmoid_group_topk_launcher(int* topk_idx, float* topk_w, const float* logits,
                                          const float* bias, int T, int E, int k, int n_group,
                                          int topk_group, float routed_scaling_factor, int config,
                                          cab_stream_t stream);

/* Bytes of scratch moe_permute_launcher needs, and the number of 128-row tiles  */
/* the padded row space can hold (T*k/128 + E). Host-only helpers.               */
size_t moe_permute_scratch_bytes(int T, int k, int E);
int moe_permute_max_tiles(int T, int k, int E);

/* Stable sort of the T*k flat entries i = t*k + slot by expert id.              */
/*   counts[E], offsets[E+1]      per-expert population and its exclusive scan   */
/*   pad_offsets[E+1]             the same with every expert rounded up to 128    */
/*   perm[T*k], inv_perm[T*k]     perm[p] = entry at sorted position p; inverse   */
/*   dst_row[T*k]                 row of entry i in the padded (128-aligned per   */
/*                                expert) row space the grouped GEMMs work in     */
/*   tile_expert[max_tiles]       expert of each 128-row tile (-1 when unused)    */
/*   num_tiles[1]                 tiles in use                                    */
/* scratch: moe_permute_scratch_bytes() bytes of device memory, contents         */
/* irrelevant on entry. Positions come from scans, never from atomics, so the     */
/* result equals a CPU stable sort on every run. An entry whose expert id lies     */
/* outside [0, E) is skipped: inv_perm and dst_row hold -1 for it, the tail of     */
/* perm past the valid entries holds -1, and the last int of scratch is set to 1   */
/* (tile overflow sets it to 2). With config bit 0 set, an id of exactly -1 is the */
/* expected marker of an empty slot and is skipped without the flag. T*k == 0 is    */
/* allowed (every table is written for zero entries).                              */
int moe_permute_launcher(const int* topk_idx, int T, int k, int E, int* counts, int* offsets,
                         int* pad_offsets, int* perm, int* inv_perm, int* dst_row, int* tile_expert,
                         int* num_tiles, int max_tiles, void* scratch, int config,
                         cab_stream_t stream);

/* 1x128 e4m3 quantisation of x[T,H] (bf16) fused with the dispatch copy.        */
/* Per token and 128-column block: amax = max|x| floored at 1e-4, scale =         */
/* amax/448, q = e4m3(x/scale) (round to nearest even, saturating; both           */
/* divisions IEEE fp32). The quantised row goes to rows dst_row[t*k+slot] of      */
/* a_q[*,H] for slot < k (dst_row == NULL: k is ignored and row t is written),    */
/* its scales to scales_t[block * ld_rows + row] (block-major, "transposed").     */
int moe_quant_dispatch_launcher(cab_e4m3* a_q, float* scales_t, const cab_bf16* x,
                                const int* dst_row, int T, int H, int k, int ld_rows, int config,
                                cab_stream_t stream);

/* Expert-parallel row movement (the reference has no counterpart; slot as above). */
/* moe_quant_rows: as moe_quant_dispatch, but the scales are written row-major,     */
/*   scales[row * (H/128) + block], the layout a row is sent in.                    */
/* moe_scatter_rows: rows[i] (e4m3 [n,H]) and scales[i] (fp32 [n,H/128]) received     */
/*   from other ranks -> a_q[dst_row[i]] and scales_t[block*ld_rows + dst_row[i]];    */
/*   dst_row[i] < 0 skips the row.                                                   */
/* moe_gather_rows: out[i,:] = y[src_row[i],:] (bf16 [*,H]); src_row[i] < 0 -> zeros. */
/* moe_tiles_from_counts: offsets, 128-padded offsets, tile_expert[] and num_tiles    */
/*   from per-expert populations counts[E] (device memory), as moe_permute derives    */
/*   them from the routing.                                                          */
int moe_quant_rows_launcher(cab_e4m3* rows_q, float* scales, const cab_bf16* x, const int* dst_row, int T,
                            int H, int k, int config, cab_stream_t stream);
int moe_scatter_rows_launcher(cab_e4m3* a_q, float* scales_t, const cab_e4m3* rows, const float* scales,
                              const int* dst_row, int n, int H, int ld_rows, int config, cab_stream_t stream);
int moe_gather_rows_launcher(cab_bf16* out, const cab_bf16* y, const int* src_row, int n, int H, int config,
                             cab_stream_t stream);
int moe_tiles_from_counts_launcher(const int* counts, int E, int* offsets, int* pad_offsets, int* tile_expert,
                                   int* num_tiles, int max_tiles, int config, cab_stream_t stream);

/* out[t,:] (bf16) = sum over slot = 0..k-1, in that order, of                   */
/* weights[t,slot] * y[dst_row[t*k+slot], :] (+ extra[t,:] when non-NULL), fp32   */
/* accumulation. y, extra, out are bf16 with row length H (H % 8 == 0). A slot    */
/* whose dst_row is negative contributes nothing.                                  */
int moe_combine_launcher(cab_bf16* out, const cab_bf16* y, const int* dst_row, const float* weights,
                         const cab_bf16* extra, int T, int H, int k, int config,
                         cab_stream_t stream);

/* Grouped FP8 GEMM with fp32 block scales on tcgen05 / TMEM / TMA.               */
/*   C[m, n] = sum over 128-wide K blocks kb of                                   */
/*             a_scales_t[kb, m] * w_scales[e, n/128, kb] * (a_q[m, kb] . w_q[e, n, kb])  */
/* where e = tile_expert[m / 128] (rows live in the padded row space of            */
/* moe_permute_launcher; tile_expert == num_tiles == NULL means one dense expert   */
/* over max_m_tiles tiles and needs E == 1).                                       */
/*   mode 0: w_q = W13 e4m3 [E, 2N, K] (rows [0,N) gate, [N,2N) up), w_scales       */
/*           [E, 2N/128, K/128]; h = silu(gate) * up is re-quantised 1x128 and      */
/*           written to out (e4m3 [rows_cap, N]) and out_scales_t ([N/128,ld_rows]).*/
/*           N % 128 == 0.                                                          */
/*   mode 1: w_q = W2 e4m3 [E, N, K], w_scales [E, N/128, K/128]; out = bf16         */
/*           [rows_cap, N]; out_scales_t unused. N % 256 == 0.                       */
/* a_q: e4m3 [rows_cap, K]; a_scales_t: fp32 [K/128, ld_rows]; K % 128 == 0;         */
/* rows_cap >= 128 * max_m_tiles; ld_rows >= rows_cap. status (device int, may be    */
/* NULL) is cleared, then set non-zero if a bounded wait inside the kernel gave up.  */
/* config > 0 overrides the number of persistent CTAs (default: one per SM).         */
int moe_grouped_gemm_fp8_launcher(int mode, void* out, float* out_scales_t, const cab_e4m3* a_q,
                                  const float* a_scales_t, const cab_e4m3* w_q, const float* w_scales,
                                  const int* tile_expert, const int* num_tiles, int max_m_tiles,
                                  int rows_cap, int ld_rows, int E, int N, int K, int* status,
                                  int config, cab_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Expert-parallel MoE layer whose dispatch and return are done by the kernels   */
/* themselves over peer memory (NVLink). The reference ships no such op; the     */
/* launchers keep the ABI of agent_workdir/kernels/axpby.cu:12-20 and add what a  */
/* multi-GPU op needs: a context object that owns this rank's exchange buffer.    */
/* Ranks: expert e lives on rank e / (E / world). One process per GPU exchanges    */
/* 64-byte handles (moe_ep_peer_export / _connect_ipc: CUDA IPC); several ranks     */
/* inside one process connect with moe_ep_peer_connect_local.                      */
/*                                                                                 */
/* moe_ep_peer_create allocates (cudaMalloc, once) the exchange buffer of           */
/* moe_ep_peer_buffer_bytes(world, t_cap, H, k) bytes plus small tables, on the     */
/* current device. t_cap bounds the tokens per rank and call; every capacity is     */
/* fixed here, so a layer call allocates nothing and never synchronises with the    */
/* host. H % 256 == 0, k <= 32, world <= 16, t_cap <= 32768, e_local = experts on     */
/* each rank <= 256.                                                               */
/* All ranks must make the same sequence of layer calls.                           */
/* ------------------------------------------------------------------------- */
size_t moe_ep_peer_buffer_bytes(int world, int t_cap, int H, int k);
int moe_ep_peer_create(void** ctx_out, int rank, int world, int t_cap, int H, int k, int e_local);
int moe_ep_peer_export(void* ctx, void* handle64);                 /* writes 64 bytes */
int moe_ep_peer_connect_ipc(void* ctx, const void* handles);       /* world x 64 bytes, in rank order */
int moe_ep_peer_connect_local(void* ctx, void* const* all_ctx);    /* world contexts of this process, in rank order */
int moe_ep_peer_destroy(void* ctx);

/* The stages of one layer call (moe_ep_peer_layer_launcher runs them in order):   */
/*  dispatch: per destination rank, every local token with an expert there gets a   */
/*    row; the token is quantised 1x128 e4m3 once and stored, with its scales and    */
/*    its k (weight, local expert | -1) slots, into that rank's receive buffer;      */
/*    then the number of rows sent is published to every rank.                       */
/*  receive: waits (bounded, about 3 s) until every rank has published, then         */
/*    derives the sort keys (local expert per slot, -1 = none) of everything received.*/
/*  gather: copies received rows to dst_row[(source*t_cap + row)*k + slot] of a_q      */
/*    (scales transposed to a_scales_t[block*ld_rows + row]); dst_row comes from       */
/*    moe_permute_launcher on the keys with config 1.                                  */
/*  return: per received row, sum over its slots of weight * y[dst_row] (fp32 -> bf16) */
/*    stored into the sending rank's return buffer; then published to every rank.      */
/*  combine: waits (bounded) for every rank's return, then out[t] = sum of the          */
/*    partial rows of token t (+ shared[t]).                                           */
int moe_ep_peer_dispatch_launcher(void* ctx, const cab_bf16* x, const int* topk_idx, const float* topk_w, int T,
                                  int config, cab_stream_t stream);
int moe_ep_peer_receive_launcher(void* ctx, int config, cab_stream_t stream);
int moe_ep_peer_gather_launcher(void* ctx, cab_e4m3* a_q, float* a_scales_t, const int* dst_row, int ld_rows,
                                int config, cab_stream_t stream);
int moe_ep_peer_return_launcher(void* ctx, const cab_bf16* y, const int* dst_row, int config, cab_stream_t stream);
int moe_ep_peer_combine_launcher(void* ctx, cab_bf16* out, const cab_bf16* shared, int T, int config,
                                 cab_stream_t stream);

/* Weights and routing rule of the layer on this rank (device pointers).           */
typedef struct cab_moe_ep_layer_args {
  const cab_bf16* router_w;        /* [E, H] */
  const float* router_bias;        /* [E] (routing 1) or NULL */
  const cab_e4m3* w13_q;           /* [e_local, 2I, H] this rank's experts */
  const float* w13_s;              /* [e_local, 2I/128, H/128] */
  const cab_e4m3* w2_q;            /* [e_local, H, I] */
  const float* w2_s;               /* [e_local, H/128, I/128] */
  const cab_e4m3* shared_w13_q;    /* [2I, H] shared expert, or all four NULL */
  const float* shared_w13_s;
  const cab_e4m3* shared_w2_q;
  const float* shared_w2_s;
  int E;                           /* experts over all ranks = e_local * world */
  int I;                           /* expert intermediate size, % 128 == 0 */
  int routing;                     /* 0 softmax top-k, 1 sigmoid + bias + groups */
  int n_group, topk_group;
  float scaling;                   /* routed scaling factor */
  int entry_cap;                   /* (token, expert) entries this rank can receive per call */
  int gemm_ctas;                   /* 0 = one persistent GEMM CTA per SM */
} cab_moe_ep_layer_args;

/* One layer call: routing, dispatch, grouped GEMMs on the local experts, return,   */
/* combine, with the shared expert on a side stream of the context. `workspace`:     */
/* moe_ep_peer_workspace_bytes() bytes of device memory, 256-byte aligned, contents   */
/* irrelevant, reusable by the next call on the same stream. out: bf16 [T, H].        */
/* Entries beyond entry_cap are dropped and flagged (status word 4 = 2).              */
/* config: 0 runs the whole call. Bits select stages (1: routing, dispatch, shared     */
/* expert; 2: receive, GEMMs, return; 4: combine) for callers that step several ranks   */
/* living on ONE GPU: there every rank must finish a stage before any rank starts the    */
/* next, because a launch must never wait for a later launch of the same GPU.            */
size_t moe_ep_peer_workspace_bytes(void* ctx, const cab_moe_ep_layer_args* args);
int moe_ep_peer_layer_launcher(void* ctx, cab_bf16* out, const cab_bf16* x, int T, const cab_moe_ep_layer_args* args,
                               void* workspace, size_t workspace_bytes, int config, cab_stream_t stream);
/* Blocking: host_out8[0..3] give-up codes of the four GEMM launches, [4] permutation */
/* flag, [5] 301 if the wait for dispatches ran out, [6] 302 if the wait for returns.  */
int moe_ep_peer_read_status(void* ctx, const cab_moe_ep_layer_args* args, void* workspace, int* host_out8);
/* Blocking copy out of the context's buffers, for tests: which = 0 received rows,     */
/* 1 side band, 2 returned rows, 3 sort keys, 4 rows received per source, 5 copy rows.  */
int moe_ep_peer_debug_read(void* ctx, int which, size_t offset, void* dst, size_t bytes);

/* ------------------------------------------------------------------------- */
/* Top-k sparse MLA decode attention (absorbed latent attention, one query      */
/* token per sequence). The reference ships no such op; these launchers fill     */
/* the kernel slot of agent_workdir/kernels/ (ABI of axpby.cu:12-20).            */
/*   q        bf16 [B, 1, Hh, 576]   (512 latent + 64 rope dims), Hh % 64 == 0   */
/*   kv       bf16 [B, S, 576]       latent KV cache                             */
/*   seq_len  int32 [B]              valid rows per sequence; a value above S   */
/*                                   is read as S, so no row outside the cache   */
/*                                   is ever touched                             */
/*   idx      int32 [B, 1, topk]     selected rows, shared by all heads; an      */
/*                                   entry counts iff 0 <= idx < seq_len[b]      */
/*   out      bf16 [B, 1, Hh, 512] = softmax(q . kv[idx]^T * softmax_scale)      */
/*                                   . kv[idx][:, :512]; zeros if nothing valid  */
/* nsplit > 1 divides the topk entries over nsplit parts per (sequence, head     */
/* group) and merges their partial results; it needs `scratch`, device memory of        */
/* mla_sparse_decode_scratch_bytes(B, Hh, nsplit) bytes (16-byte aligned,         */
/* contents irrelevant on entry). status: as for moe_grouped_gemm_fp8_launcher.   */
/* config: 0 = head groups of 128 run on pairs of CTAs when Hh % 128 == 0 (the    */
/* pairs split the 576 columns), else 64 heads per CTA; 1 = always 64 heads per CTA. */
/* ------------------------------------------------------------------------- */
size_t mla_sparse_decode_scratch_bytes(int B, int Hh, int nsplit);
int mla_sparse_decode_launcher(cab_bf16* out, const cab_bf16* q, const cab_bf16* kv, const int* seq_len,
                               const int* idx, int B, int Hh, int S, int topk, float softmax_scale,
                               int nsplit, void* scratch, int* status, int config, cab_stream_t stream);

/* Several query tokens per sequence (speculative / multi-token decode): the Sq   */
/* tokens of sequence b share its cache rows, each with its own selection and its */
/* own valid length (e.g. seq_len[b, s] = cached tokens visible to token s).       */
/*   q [B, Sq, Hh, 576], seq_len int32 [B, Sq], idx int32 [B, Sq, topk],           */
/*   out [B, Sq, Hh, 512]; scratch: mla_sparse_decode_scratch_bytes(B * Sq, ...).  */
/* B * Sq <= 65535. mla_sparse_decode_launcher is the Sq = 1 case.                 */
int mla_sparse_decode_multi_launcher(cab_bf16* out, const cab_bf16* q, const cab_bf16* kv, const int* seq_len,
                                     const int* idx, int B, int Sq, int Hh, int S, int topk, float softmax_scale,
                                     int nsplit, void* scratch, int* status, int config, cab_stream_t stream);

/* Split decode that allocates nothing. No counterpart in the reference.          */
/* Same arguments and result as mla_sparse_decode_launcher, without the scratch    */
/* pointer: the split partials go to a fixed array of                               */
/* CAB_MLA_STATIC_SCRATCH_BYTES inside the library's device image. It exists for    */
/* callers that cannot provide scratch: a process whose device memory is already    */
/* owned by its own arena and that must not call cudaMalloc while serving, or an    */
/* operator interface that passes inputs and outputs only.                          */
/*  - B * nsplit * Hh * 2056 bytes must not exceed CAB_MLA_STATIC_SCRATCH_BYTES;      */
/*    otherwise CAB_ERR_TOO_LARGE is returned and nothing is launched.               */
/*  - The array occupies that much memory on every GPU that loads the library,      */
/*    until the process exits.                                                       */
/*  - All calls on a GPU share it: calls that can overlap on the device race and     */
/*    must be serialised by the caller. Old contents never leak into a result.       */
/*  - The first call on each device looks up the array's device address (a host      */
/*    call to the CUDA runtime); make that first call before capturing any stream.   */
/*  - It calls no cudaMalloc, cudaFree or other allocating routine.                   */
#define CAB_MLA_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
int mla_sparse_decode_noalloc_launcher(cab_bf16* out, const cab_bf16* q, const cab_bf16* kv,
                                       const int* seq_len, const int* idx, int B, int Hh, int S, int topk,
                                       float softmax_scale, int nsplit, int* status, int config,
                                       cab_stream_t stream);

/* The index-validation + row-gather step on its own:                            */
/* rows[b, j, :] (bf16 [B, topk, 576]) = kv[b, idx[b, j], :] for a valid entry,   */
/* zeros otherwise.                                                              */
int mla_gather_rows_launcher(cab_bf16* rows, const cab_bf16* kv, const int* seq_len, const int* idx, int B,
                             int S, int topk, int config, cab_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* CUDA_AGENT_B200_H_ */
