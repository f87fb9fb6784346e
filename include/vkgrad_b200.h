/*
 * vkgrad_b200 -- C ABI of the B200 (sm_100a) training-step library.
 *
 * This is the whole boundary between the Python object model (kernels.Matmul,
 * autograd.Linear/AdamW/TrainStep, transformer.GPT, dataparallel.Replica) and
 * the CUDA code.  Plain pointers and sizes only; every entry returns an int
 * status (0 = OK, non-zero = failed, message in vkg_last_error()) and never
 * throws or aborts, mirroring the reference runtime's `_check` (vk.py:132-134),
 * which turns every non-zero VkResult into VkError.
 *
 * Each declaration cites the reference interface it replaces (file:line in
 * BrettKnox/vkgrad).  All compute entries enqueue on the device's stream and
 * return without synchronising unless stated otherwise, so the same calls can
 * be issued between vkg_graph_begin/vkg_graph_end to record a replayable step
 * (reference: vk.Graph.record, vk.py:842-868).
 *
 * dtypes: VKG_F32 = 0, VKG_F16 = 1, VKG_BF16 = 2.
 */
#ifndef VKGRAD_B200_H
#define VKGRAD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VKG_F32 0
#define VKG_F16 1
#define VKG_BF16 2

#define VKG_ACT_NONE 0
#define VKG_ACT_GELU 1 /* tanh form, kernels.py:624-629 */
#define VKG_ACT_RELU 2 /* extension: the reference has GELU only */

typedef struct vkg_device vkg_device;
typedef struct vkg_graph vkg_graph;
typedef struct vkg_comm vkg_comm;

/* ---- runtime: replaces vk.Device / vk.Buffer / vk.Graph ------------------ */

/* Thread-local message of the last failed call (vk.VkError text, vk.py:128). */
const char* vkg_last_error(void);
/* Library version string. */
const char* vkg_version(void);
/* Number of CUDA devices visible; 0 (not an error) when there is no GPU. */
int vkg_device_count(int* count);

/* vk.Device() (vk.py:892): binds CUDA device `ordinal`, creates its stream. */
int vkg_device_create(int ordinal, vkg_device** out);
/* vk.Device.destroy (vk.py:1342). */
int vkg_device_destroy(vkg_device* dev);
/* Device.name and the numbers callers print (vk.py:1074-1100). */
int vkg_device_info(vkg_device* dev, char* name, size_t name_cap, int* sm_count,
                    size_t* total_bytes, int* cc_major, int* cc_minor);
/* Opaque cudaStream_t of the device, for callers that interoperate. */
void* vkg_device_stream(vkg_device* dev);
/* No counterpart in the reference (Vulkan orders dispatches with pipeline barriers).
 * Programmatic dependent launch for this device's kernels: when on, a kernel may be
 * scheduled while its predecessor on the stream drains and waits, before its first global
 * access, until the predecessor has completed.  Results do not depend on the setting.  It
 * is sampled when a launch is enqueued or recorded.  Off by default (the environment
 * variable VKG_PDL=1 starts a device with it on): back-to-back eager launches of one
 * kernel gain about 2 %, but a recorded training step measured 0.1 to 0.4 ms SLOWER with
 * programmatic edges in its CUDA graph, whichever kernel families carried them. */
int vkg_set_pdl(vkg_device* dev, int on);
/* No counterpart in the reference.  Switches that change how kernels are launched, never
 * what they compute; sampled when a launch is enqueued or recorded, so two recordings of
 * the same step can be compared in one process.
 *   VKG_TUNE_PDL           0 / 1, same as vkg_set_pdl
 *   VKG_TUNE_PDL_FAMILIES  bit mask of kernel families programmatic launch applies to
 *                          (1 GEMM, 2 CTA-pair GEMM, 4 grouped GEMM, 8 attention forward,
 *                          16 attention backward, 32 layernorm, 64 layernorm backward,
 *                          128 softmax-CE, 256 AdamW, 512 the small kernels)
 *   VKG_TUNE_TMA_STORE     0: GEMM epilogues store per lane; 1 (default): epilogues
 *                          without fused reads store their tiles through tensor maps
 *   VKG_TUNE_WAIT_TIMEOUT_MS  limit of a host wait on a device that has a communicator
 *                          (default 60 000): see vkg_sync
 *   VKG_TUNE_SM_LIMIT      most CTAs a persistent kernel (GEMM, grouped GEMM, attention
 *                          backward) launches; 0 = one per SM.  May also change during a
 *                          recording: launches recorded after the call use the new value
 *   VKG_TUNE_PAIR_MIN_WAVES  tenths of a tile per CTA pair from which vkg_gemm with
 *                          cta_pair == 0 takes 256 x 256 CTA-pair tiles
 *   VKG_TUNE_ATTN_ONE_PASS 1 (default): the fused attention forward computes every score tile
 *                          once and keeps a lazily rescaled running row maximum; 0: two
 *                          passes over the keys (row maximum first)
 *   VKG_TUNE_PAIR_192      1 (default): vkg_gemm with cta_pair == 0 and tile_n == 0 takes
 *                          256 x 192 CTA-pair tiles for unbatched outputs one to four such
 *                          tiles wide (N = 192 .. 768) with K >= 1536 and at least one wave
 *                          of them; 0: never.  Same bits either way. */
enum { VKG_TUNE_PDL = 0, VKG_TUNE_PDL_FAMILIES = 1, VKG_TUNE_TMA_STORE = 2,
       VKG_TUNE_WAIT_TIMEOUT_MS = 3, VKG_TUNE_SM_LIMIT = 4, VKG_TUNE_PAIR_MIN_WAVES = 5,
       VKG_TUNE_ATTN_ONE_PASS = 6, VKG_TUNE_PAIR_192 = 7 };
int vkg_set_tuning(vkg_device* dev, int key, int64_t value);
/* Waits for the stream; reports a kernel error flag (bounded waits that gave
 * up) as a failure, like the reference's 10 s fence timeout (vk.py:884-888, 1335-1339).
 * While a communicator is attached to the device this and every other host wait
 * (vkg_timer_end, vkg_graph_launch, vkg_download, vkg_comm_max_double) polls against a
 * deadline instead of blocking: on an asynchronous NCCL error, or when the limit expires (a
 * collective whose peer never arrived), the communicator is aborted with ncclCommAbort,
 * the call fails, and later collectives on that communicator fail at once. */
int vkg_sync(vkg_device* dev);
/* No counterpart in the reference.  Runs the deadline loop of the host waits against a
 * scripted device, without a GPU: "done" after ready_after_polls queries (negative: never),
 * an asynchronous communicator error from its async_error_at-th check on (negative:
 * never).  Returns what the wait returns; *aborted = number of aborts issued. */
int vkg_selftest_wait_deadline(int64_t ready_after_polls, int64_t async_error_at,
                               double timeout_s, int* aborted);

/* dev.buffer(size, kind) (vk.py:1256, memory kinds vk.py:1161-1200).
 * kind 0 "device": HBM only.  kind 1 "shared": pinned, mapped host memory the
 * GPU reads in place (host writes are visible without flush, mnist.py:170).
 * kind 2 "cached": HBM plus a pinned host mirror; vkg_upload/vkg_download are
 * Buffer.flush / Buffer.invalidate (vk.py:598-610).
 * dptr is what kernels take; hptr is the numpy-visible address or NULL. */
int vkg_alloc(vkg_device* dev, size_t bytes, int kind, void** dptr, void** hptr);
int vkg_free(vkg_device* dev, void* dptr, void* hptr, int kind);
/* Buffer.flush: host mirror -> device (synchronous). */
int vkg_upload(vkg_device* dev, void* dptr, const void* hptr, size_t bytes);
/* Buffer.invalidate: device -> host mirror (synchronous). */
int vkg_download(vkg_device* dev, void* hptr, const void* dptr, size_t bytes);
/* dev.copy(src,dst,size) (vk.py:1267): enqueued device-side copy. */
int vkg_copy(vkg_device* dev, void* dst, const void* src, size_t bytes);
/* Enqueued copies between pinned host memory and the device, for the
 * end-to-end path (inputs up, loss down) inside a recorded step. */
int vkg_copy_h2d_async(vkg_device* dev, void* dptr, const void* hptr, size_t bytes);
int vkg_copy_d2h_async(vkg_device* dev, void* hptr, const void* dptr, size_t bytes);
/* K["zero"] / arena_zero (kernels.py:853, dataparallel.py:60). */
int vkg_memset0(vkg_device* dev, void* dptr, size_t bytes);

/* Event timing around enqueued work: Device.run returns seconds (vk.py:1295). */
int vkg_timer_begin(vkg_device* dev);
int vkg_timer_end(vkg_device* dev, double* seconds); /* synchronises */

/* vk.Graph (vk.py:807-889): capture everything enqueued between begin/end. */
int vkg_graph_begin(vkg_device* dev);
int vkg_graph_end(vkg_device* dev, vkg_graph** out);
/* Graph.submit(): launch, wait, return GPU seconds (vk.py:877-889). */
int vkg_graph_launch(vkg_device* dev, vkg_graph* g, double* seconds);
/* Launch without waiting (pipelined steps). */
int vkg_graph_launch_async(vkg_device* dev, vkg_graph* g);
int vkg_graph_destroy(vkg_graph* g);
/* Number of kernel nodes in a finished graph (Graph.n_dispatch, vk.py:868). */
int vkg_graph_kernel_count(vkg_graph* g, int* count);

/* ---- the GEMM trio: replaces kernels.Matmul (kernels.py:32-138, 232-315) -- */

/*
 * C[M x N] = op(A) * op(B), 16-bit inputs, fp32 accumulation on tcgen05.
 *   trans_a = 0: A stored M x K (lda >= K).  trans_a = 1: A stored K x M
 *                (the dW = X^T dY form, kernels.py:112-118).
 *   trans_b = 0: B stored K x N (ldb >= N).  trans_b = 1: B stored N x K
 *                (the dX = dY W^T form, kernels.py:120-126).
 * Batched form (kernels.py:58-64, 98-102): batch index z = z0 + nb0 * z1 with
 * z0 < nb0, z1 < nb1; operand X is offset by z0*sX0 + z1*sX1 elements.  Two
 * strides let attention heads be addressed inside a (rows, 3D) projection
 * without the split_qkv / merge_heads permutes (tkernels.py:195-300).
 * Epilogue, in order (each optional):  v = acc; v += bias[col];
 * pre[row,col] = v (fp32);  v = act(v);  v *= act'(dact_z[row,col]);
 * v += residual[row,col];  C = v (c_dtype);  C2 = f16(v).
 * These fuse bias_gelu / bias / bias_gelu_bwd16 / residual / to16
 * (kernels.py:709-749, tkernels.py:364-387) into the producing GEMM.
 * Overwrites C like the reference (callers rely on it, transformer.py:367).
 * Leading dimensions are in elements; A/B pointers and lda/ldb*2 bytes must be
 * 16-byte aligned, N % 8 == 0.  No tile-multiple restriction (the reference
 * raises VkError for ragged shapes, kernels.py:274-276; here edges are
 * predicated).
 */
typedef struct vkg_gemm_args {
  int32_t trans_a, trans_b;
  int32_t M, N, K;
  int32_t nb0, nb1;          /* batch extents; 1,1 when not batched */
  int32_t in_dtype;          /* VKG_F16 or VKG_BF16 */
  const void* A; int64_t lda, sA0, sA1;
  const void* B; int64_t ldb, sB0, sB1;
  void* C; int64_t ldc, sC0, sC1; int32_t c_dtype; /* VKG_F32 / VKG_F16 / VKG_BF16 */
  int32_t act;               /* VKG_ACT_* applied to v */
  void* C2;                  /* optional f16 copy of the result, same ldc/strides */
  const float* bias;         /* optional, length N */
  float* pre;                /* optional fp32 pre-activation, same ldc/strides */
  const float* dact_z;       /* optional: multiply by act'(z), z fp32 same layout */
  int32_t dact;              /* VKG_ACT_* whose derivative multiplies */
  const float* residual;     /* optional fp32, same ldc/strides */
  int32_t tile_n;            /* 0 = choose; else 64/128/192/256 */
  int32_t max_ctas;          /* 0 = one per SM */
  float alpha;               /* 0 treated as 1: scales acc before bias */
  int32_t split_k;           /* K cut into slices: each slice's partial tile goes to
                                `workspace` and a second kernel adds the slices in order
                                (deterministic).  Plain fp32 epilogue, unbatched only.
                                0 = library decides (splits only if a workspace is given),
                                1 = never, n > 1 = exactly n slices. */
  void* workspace;           /* scratch for the slices: slices * M * N floats */
  int64_t workspace_bytes;
  int32_t causal;            /* attention shortcuts for square (T x T) causal operands:
                                1: C is lower-triangular -- tiles wholly above the diagonal
                                   are skipped and left untouched (scores, dP);
                                2: A (M x K) is lower-triangular -- k-blocks right of the
                                   tile's last row are skipped (P V, dS K);
                                3: A stored K x M is lower-triangular in (k, m) -- k-blocks
                                   before the tile's first row are skipped (P^T dO, dS^T Q). */
  int32_t cta_pair;          /* 256 x 256 tiles computed by two CTAs of a cluster with one
                                tcgen05.mma.cta_group::2 (each CTA loads half of the B tile):
                                0 = the library decides, 1 = always (when the shape allows it;
                                tile_n = 192 then asks for 256 x 192 tiles), -1 = never.  Not
                                available with causal != 0. */
  float* colsum;             /* optional, N floats: column sums of the output as stored (after
                                the epilogue and the narrowing), the bias gradient of the layer
                                that produced this GEMM's dY (replaces the col_sum pass of
                                transformer.py:30-36 over it).  Deterministic.  Unbatched,
                                causal == 0, K not split. */
  float* colsum_scratch;     /* with colsum: vkg_gemm_colsum_scratch_floats(M, N) floats */
} vkg_gemm_args;

int64_t vkg_gemm_colsum_scratch_floats(int M, int N);

/* Many independent plain GEMMs (fp32 output, unbatched, no epilogue extras) in ONE launch: the
 * dW = X^T dY of every Linear of a model (autograd.py:217-219, transformer.py:97-98), which
 * have too few tiles each to fill the GPU and thousands together.  Results are those of
 * vkg_gemm on each problem with split_k = 1, bit for bit.  vkg_gemm_group_prepare builds the
 * launch table in device memory the caller owns (vkg_gemm_group_table_bytes(n) bytes, 128-byte
 * aligned; synchronous, so before any stream capture; operand pointers are baked in) and
 * returns in *total_units the value to hand to vkg_gemm_group_launch, which enqueues the
 * launch and may be captured.  cta_pair > 0 asks for 256 x 256 tiles on 2-CTA clusters (used
 * when every problem has more than 128 rows; *total_units is then negative). */
int64_t vkg_gemm_group_table_bytes(int n);
int vkg_gemm_group_prepare(vkg_device* dev, const vkg_gemm_args* args, int n, void* table,
                           int cta_pair, int* total_units);
int vkg_gemm_group_launch(vkg_device* dev, const void* table, int n, int total_units);

/* No reference counterpart.  Launches a one-thread kernel that waits, with the bounded wait
 * all tcgen05 / TMA kernels of this library use, on an mbarrier nothing arrives on, for at
 * most budget_cycles (<= 1e8) SM cycles.  The wait gives up, the kernel returns normally, and
 * the next vkg_sync reports the timeout like it would for a real kernel; the device stays
 * usable.  For tests of the failure path. */
int vkg_selftest_wait_timeout(vkg_device* dev, int64_t budget_cycles);

int vkg_gemm(vkg_device* dev, const vkg_gemm_args* args);


/* ---- MLP-step fused ops: replaces kernels.make_kernels (kernels.py:699-862) */

/* bias_gelu (kernels.py:709-718): z = acc + bias[i % ncol]; y16 = f16(act(z)). */
int vkg_bias_act(vkg_device* dev, const float* acc, const float* bias, float* z,
                 void* y16, int64_t n, int ncol, int act);
/* bias_gelu_bwd / bwd16 (kernels.py:721-739): g = dy * act'(z); dz32 optional. */
int vkg_bias_act_bwd(vkg_device* dev, const float* dy, const float* z, void* dz16,
                     float* dz32, int64_t n, int act);
/* bias (kernels.py:742-749): z = acc + bias[i % ncol]. */
int vkg_bias(vkg_device* dev, const float* acc, const float* bias, float* z,
             int64_t n, int ncol);
/* col_sum (kernels.py:753-761): sums[c] = sum_r g[r*ncol + c], fp32 input. */
int vkg_col_sum(vkg_device* dev, const float* g, float* sums, int ncol, int nrow);
/* softmax_ce / softmax_ce_w (kernels.py:766-827).  Per row: loss, and
 * dl = (softmax - onehot) * (w ? w[row] * (grad_scale ? grad_scale : 1) : grad_scale);
 * classes >= ncls are masked to exactly 0.  Without weights grad_scale is 1/rows for
 * the reference's mean, times a static loss scale when one is used; with weights
 * (which already carry the normalisation) it is the static loss scale alone, 0 or 1
 * for none.  dl16 is written in f16; dl32 optional. */
int vkg_softmax_ce(vkg_device* dev, const float* logits, const uint32_t* labels,
                   const float* w, void* dl16, float* dl32, float* loss,
                   int rows, int stride, int ncls, float grad_scale);
/* adamw (kernels.py:832-851): hp = {lr,b1,b2,bc1,bc2,eps,(gscale)} read from
 * memory at run time so a recorded step replays with new values
 * (autograd.py:313-323).  hp[6], when non-zero, multiplies the gradient first:
 * the 1/(workers * loss_scale) of grad_pull (dataparallel.py:69-73) fused in. */
int vkg_adamw(vkg_device* dev, float* w, const float* g, float* m, float* v,
              void* w16, const float* hp, int64_t n, float wd);
/* All parameter tensors in one launch (the reference issues one dispatch per
 * tensor, autograd.py:331-335).  Arrays of length ntensors live on the host;
 * the table is copied to device memory owned by `table` (opaque, reusable). */
int vkg_adamw_table_create(vkg_device* dev, int ntensors, float* const* w,
                           const float* const* g, float* const* m, float* const* v,
                           void* const* w16, const int64_t* n, const float* wd,
                           void** table);
int vkg_adamw_table_destroy(vkg_device* dev, void* table);
int vkg_adamw_multi(vkg_device* dev, void* table, const float* hp);
/* cast16 / to16 (kernels.py:857-860, tkernels.py:384-387). */
int vkg_cast16(vkg_device* dev, const float* src, void* dst16, int64_t n);

/* ---- transformer ops: replaces tkernels.make_transformer_kernels --------- */

/* layernorm (tkernels.py:32-54): eps 1e-5, biased variance; saves mu, rstd. */
int vkg_layernorm(vkg_device* dev, const float* x, const float* gamma,
                  const float* beta, void* y16, float* mu, float* rstd,
                  int rows, int D);
/* layernorm_bwd (tkernels.py:58-88).  dx = LN'(dy) [+ dres when given];
 * dx16 optional f16 copy; dyxh16/dy16 optional (the reference's inputs to its
 * column sums).  When dgamma/dbeta are given they receive the column sums of
 * dy*xhat and dy directly (deterministic two-stage reduction through
 * `scratch`, which must hold vkg_layernorm_bwd_scratch_floats(rows, D)).
 * dxsum (optional, D % 128 == 0, D <= 1024) also receives the column sums of dx:
 * the bias gradient of the Dense that consumes dx (Dense.backward's col_sum,
 * transformer.py:99), saving that pass. */
int vkg_layernorm_bwd(vkg_device* dev, const float* dy, const float* x,
                      const float* gamma, const float* mu, const float* rstd,
                      const float* dres, float* dx, void* dx16, void* dyxh16,
                      void* dy16, float* dgamma, float* dbeta, float* dxsum,
                      float* scratch, int rows, int D);
int64_t vkg_layernorm_bwd_scratch_floats(int rows, int D);
/* attn_softmax / attn_softmax_doc (tkernels.py:105-161): causal, scaled;
 * seg (optional) restricts a query to keys >= seg[b*T+q]; rows = nbh*T.
 * fill_block = 0 writes the zeros above the diagonal to the end of the row as
 * the reference does; fill_block = n > 0 stops at the end of the n-wide column
 * block holding the diagonal, for consumers that use vkg_gemm's causal modes
 * and never read further. */
int vkg_attn_softmax(vkg_device* dev, const float* s, const uint32_t* seg,
                     void* p16, int64_t rows, int T, int H, float scale,
                     int fill_block);
/* attn_softmax_bwd (tkernels.py:167-188): ds = P*(dP - sum dP*P)*scale. */
int vkg_attn_softmax_bwd(vkg_device* dev, const float* dp, const void* p16,
                         void* ds16, int64_t rows, int T, float scale,
                         int fill_block);
/* Fused causal attention, head dimension 64: one kernel for
 * QK^T matmul + attn_softmax(_doc) + PV matmul (transformer.py:141-157,
 * tkernels.py:105-161) with no T x T tensor in memory.  qkv16 is the (B*T, 3D)
 * fp16 projection with the qkv bias already added; out16 receives the
 * head-merged (B*T, D) fp16 attention output (what merge_heads produces,
 * tkernels.py:274-286); lse2 (B*H, T) receives log2(sum_j exp(scale * s_ij)),
 * which the backward kernels use to rebuild P. */
int vkg_attn_fwd(vkg_device* dev, const void* qkv16, const uint32_t* seg,
                 void* out16, float* lse2, int B, int T, int H, int hd, float scale);
/* Backward of vkg_attn_fwd: the reference's split_heads, four batched matmuls,
 * attn_softmax_bwd and merge_qkv_grad (transformer.py:160-186, tkernels.py:167-232)
 * as two persistent launches: a dQ kernel (items = query tiles), which also forms
 * delta = rowsum(dO * O) and leaves it in `delta`, and a dK/dV kernel (items = key tiles),
 * both rebuilding P from lse2.
 * dout16 is the (B*T, D) fp16 gradient of out16; dqkv16 (B*T, 3D) fp16 receives
 * [dQ | dK | dV]; delta is B*H*T floats of scratch.  Deterministic (no atomics).
 * dbias (optional, 3D floats) receives the column sums of dqkv16 as stored -- the gradient
 * of the qkv bias, which the reference takes with a col_sum pass over the merged gradient
 * (transformer.py:30-36, 183-186); dbias_scratch then holds
 * vkg_attn_bwd_dbias_scratch_floats(B, T, H, hd) floats. */
int vkg_attn_bwd(vkg_device* dev, const void* qkv16, const void* dout16,
                 const void* out16, const float* lse2, const uint32_t* seg,
                 void* dqkv16, float* delta, float* dbias, float* dbias_scratch,
                 int B, int T, int H, int hd, float scale);
int64_t vkg_attn_bwd_dbias_scratch_floats(int B, int T, int H, int hd);
/* split_qkv / merge_qkv_grad / merge_heads / split_heads (tkernels.py:195-300). */
int vkg_split_qkv(vkg_device* dev, const float* qkv, const float* bias, void* q16,
                  void* k16, void* v16, int64_t n, int D, int T, int H, int hd);
int vkg_merge_qkv_grad(vkg_device* dev, const float* dq, const float* dk,
                       const float* dv, void* dqkv16, int64_t n, int D, int T,
                       int H, int hd);
int vkg_merge_heads(vkg_device* dev, const float* src, void* y16, int64_t n, int D,
                    int T, int H, int hd);
int vkg_split_heads(vkg_device* dev, const float* src, void* dst16, int64_t n,
                    int D, int T, int H, int hd);
/* col_sum_zero + col_sum_chunk(16) (tkernels.py:238-270, transformer.py:30-36):
 * sums[c] (+)= sum_r g[r*ncol+c].  Deterministic: fixed-order partial sums in
 * `scratch` (vkg_col_sum_scratch_floats(ncol, nrow) floats), no atomics.
 * g_dtype VKG_F32 or VKG_F16; accumulate != 0 adds into sums instead of
 * overwriting (the reference's chunk kernel adds into a zeroed buffer). */
int vkg_col_sum_det(vkg_device* dev, const void* g, int g_dtype, float* sums,
                    float* scratch, int ncol, int nrow, int accumulate);
int64_t vkg_col_sum_scratch_floats(int ncol, int nrow);
/* Deferred final passes.  The reference issues one dispatch per column-sum stage
 * (col_sum_zero + col_sum_chunk per bias gradient, transformer.py:30-36; two per
 * layernorm, tkernels.py:238-270).  Here the producers (vkg_layernorm_bwd with dgamma,
 * vkg_attn_bwd with dbias, vkg_gemm with colsum) leave partial sums in their scratch and
 * finish with a short second pass; between vkg_finals_defer(dev, 1) and vkg_finals_flush
 * those second passes are collected instead of launched and flush runs them all as one
 * launch.  While deferral is on, every producer call must be given scratch of its own,
 * which has to stay untouched until the flush has run; the destinations hold their sums
 * only after the flush.  vkg_finals_defer(dev, 0) with passes pending is an error;
 * vkg_finals_defer(dev, -1) switches deferral off and drops pending passes (for a
 * recording that was abandoned half way). */
int vkg_finals_defer(vkg_device* dev, int on);
int vkg_finals_flush(vkg_device* dev);

/* No counterpart in the reference.  The same deterministic column sum as
 * vkg_col_sum_det for callers that are not allowed to allocate device memory
 * (a plugin inside a process that owns the allocator, a latency-critical loop):
 * the partial sums go to a 4 MiB array
 * built into the library instead of caller scratch, and the call performs no
 * cudaMalloc / cudaFree.  Shapes whose partial sums need more than
 * vkg_col_sum_static_max_floats() floats (see vkg_col_sum_scratch_floats) are
 * refused with an error.  The first call on each device looks the array's
 * device address up (cudaGetSymbolAddress); make that first call before any
 * stream capture begins (during a capture it returns an error instead).  All calls on a device share the one array: two calls
 * whose kernels may overlap on the GPU (different streams or devices handles on
 * the same GPU) race on it, so keep them on one stream. */
int vkg_col_sum_static(vkg_device* dev, const void* g, int g_dtype, float* sums,
                       int ncol, int nrow, int accumulate);
int64_t vkg_col_sum_static_max_floats(void);
/* embed / embed_doc (tkernels.py:303-313, 334-345). */
int vkg_embed(vkg_device* dev, const float* tok, const float* pos,
              const uint32_t* ids, const uint32_t* seg, float* x, int64_t n, int D,
              int T);
/* embed_bwd / embed_doc_bwd (tkernels.py:317-360): scatter-add into dtok, dpos. */
int vkg_embed_bwd(vkg_device* dev, const float* dx, const uint32_t* ids,
                  const uint32_t* seg, float* dtok, float* dpos, int64_t n, int D,
                  int T);
/* The same scatter-add without atomics: rows that hit one table row are added in row
 * order by one warp, so the result is bit-reproducible from run to run (the reference's
 * float atomics are not).  D a multiple of 128 up to 1024; scratch holds
 * vkg_embed_bwd_scratch_bytes(n / D) bytes. */
int64_t vkg_embed_bwd_scratch_bytes(int64_t rows);
int vkg_embed_bwd_det(vkg_device* dev, const float* dx, const uint32_t* ids,
                      const uint32_t* seg, float* dtok, float* dpos, void* scratch,
                      int64_t n, int D, int T);
/* residual (tkernels.py:364-371): out = res + acc + bias[i % D]. */
int vkg_residual(vkg_device* dev, const float* acc, const float* bias,
                 const float* res, float* out, int64_t n, int D);
/* add (tkernels.py:373-377); out16 optional f16 copy. */
int vkg_add(vkg_device* dev, const float* a, const float* b, float* out,
            void* out16, int64_t n);
/* add_bias (tkernels.py:380-382): x[i] += bias[i % ncol]. */
int vkg_add_bias(vkg_device* dev, float* x, const float* bias, int64_t n, int ncol);

/* ---- data parallel: replaces dataparallel.make_reduce_kernels ------------ */

/* grad_add (dataparallel.py:54-58): arena[off+i] += g[i]. */
int vkg_grad_add(vkg_device* dev, const float* g, float* arena, int64_t n,
                 int64_t off);
/* grad_pull (dataparallel.py:69-73): g[i] = arena[off+i] * scale. */
int vkg_grad_pull(vkg_device* dev, const float* arena, float* g, int64_t n,
                  int64_t off, float scale);
/* Bucket pack/unpack with the loss-unscale cast fused: dst16 = f16/bf16(src*scale)
 * and dst32 = float(src16)*scale. */
int vkg_bucket_pack16(vkg_device* dev, const float* src, void* dst16, int dtype,
                      int64_t n, float scale);
int vkg_bucket_unpack16(vkg_device* dev, const void* src16, int dtype, float* dst,
                        int64_t n, float scale);

/* NCCL replaces the shared host arena + atomicAdd push (dataparallel.py:40-47,
 * 119-126).  The unique id is 128 bytes, made on rank 0 and passed to the other
 * ranks by the caller (file, socket or a torch.distributed store). */
int vkg_comm_unique_id(uint8_t id[128]);
int vkg_comm_create(vkg_device* dev, int rank, int nranks, const uint8_t id[128],
                    vkg_comm** out);
/* The same with NCCL held to at most max_ctas CTAs (ncclConfig_t.maxCTAs; 0 = NCCL's own
 * choice): for collectives that run on the side stream while the compute stream keeps the
 * other SMs busy (see VKG_TUNE_SM_LIMIT). */
int vkg_comm_create_limited(vkg_device* dev, int rank, int nranks, const uint8_t id[128],
                            int max_ctas, vkg_comm** out);
int vkg_comm_destroy(vkg_comm* comm);
/* In-place sum over ranks of `count` elements of dtype, on the device stream. */
int vkg_allreduce_sum(vkg_comm* comm, void* buf, int64_t count, int dtype);
/* The same all-reduce on a second stream, so that a part of the gradient bucket whose
 * gradients are complete is summed while the compute stream goes on with the rest of the
 * backward (the reference's workers push each tensor as soon as it exists,
 * dataparallel.py:119-126), and the optimiser over parts already summed runs while the last
 * part is still in flight.  side_begin orders the
 * side stream after everything enqueued on the device's stream so far; allreduce_sum_side
 * enqueues there and marks its end with event `slot` (0..15); side_wait makes the device's
 * stream wait for that event.  Not for use inside a stream capture. */
int vkg_comm_side_begin(vkg_comm* comm);
int vkg_allreduce_sum_side(vkg_comm* comm, void* buf, int64_t count, int dtype, int slot);
int vkg_comm_side_wait(vkg_comm* comm, int slot);
/* max over ranks of one host double (timing), and a barrier. */
int vkg_comm_max_double(vkg_comm* comm, double* value);
int vkg_comm_barrier(vkg_comm* comm);

#ifdef __cplusplus
}
#endif
#endif /* VKGRAD_B200_H */
