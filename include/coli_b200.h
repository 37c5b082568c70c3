/* C ABI of libcoli_b200.so — the B200 (sm_100a) backend for the routed-expert MoE block of
 * GriffinPilz/SpeedyColibri.
 *
 * The first half keeps the names, argument meaning and return convention of the reference's
 * CUDA backend (crates/colibri-backend/cuda/backend_cuda.h; Rust declarations in
 * crates/colibri-backend/src/cuda.rs:32-395), so the engine's expert dispatch
 * (crates/colibri-engine/src/gpu.rs) links against it unchanged.  The second half
 * (coli_b200_*) is the whole-block entry the reference does not have: router, top-k, permute,
 * grouped expert FFN, weighted combine and shared expert in one device-resident call, plus
 * the per-stage calls the expert-parallel path is assembled from.
 *
 * Conventions (backend_cuda.h throughout): every int-returning call returns 1 when it ran and
 * 0 when it declined or failed.  There is no CPU fallback behind a 0 in this library; the
 * reason is available from coli_cuda_last_error().  Matrices are row-major; a weight W[O,I]
 * maps x[S,I] to y[S,O].  All pointers are plain host or device addresses as stated per call.
 */
#ifndef COLI_B200_H
#define COLI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COLI_CUDA_MAX_DEVICES 16

/* Weight formats.  0..6 are the reference's QTensor fmt codes
 * (crates/colibri-core/src/quant.rs:707-746); 8 is the 128x128 block-scaled FP8 form the
 * reference only reads in its converter (crates/colibri-engine/src/convert.rs:674-745). */
#define COLI_FMT_F32 0
#define COLI_FMT_E4M3_ROW 4
#define COLI_FMT_NVFP4 5
#define COLI_FMT_MXFP4 6
#define COLI_FMT_FP8_B128 8

/* Opaque, persistent HBM copy of one quantised matrix (backend_cuda.h:24). */
typedef struct ColiCudaTensor ColiCudaTensor;

/* ---- lifecycle ------------------------------------------------------------------------- */
/* backend_cuda.h:27 / backend_cuda.cu:2611-2655.  `devices` are CUDA ordinals.  Idempotent for
 * the same set; refuses a different set while live.  Refuses a device that is not sm_100. */
int coli_cuda_init(const int *devices, int count);
/* backend_cuda.h:28. */
void coli_cuda_shutdown(void);
/* backend_cuda.h:32-33. */
int coli_cuda_device_count(void);
int coli_cuda_device_at(int index);
/* backend_cuda.h:34. */
int coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes);
/* backend_cuda.h:46. */
int coli_cuda_device_sync(int device);
/* backend_cuda.h:31; same three forms as backend_cuda.cu:380-392: oai != 0 clamped OpenAI-SwiGLU
 * (math.rs:143-148), oai == 0 with limit > 0 SwiGLU under the asymmetric clamp (dsv4.rs:738-742),
 * otherwise plain SiLU SwiGLU.  Process-wide; a ColiMoe handle keeps the setting it was created
 * under, the host-pointer expert calls read it per call. */
void coli_cuda_set_activation(int oai, float alpha, float limit);
/* backend_cuda.h:48.  Resident tensors on `device` (< 0: all devices). */
void coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes);
/* backend_cuda.h:51: live scratch of the host-pointer calls on `device` (< 0: all devices), not
 * counting the resident weights. */
size_t coli_cuda_scratch_bytes(int device);
/* backend_cuda.h:52-53: totals over the grouped expert calls since load (calls, experts, rows) and
 * their device-timed upload / kernel / download milliseconds. */
void coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows, double *h2d_ms, double *kernel_ms,
                           double *d2h_ms);
/* backend_cuda.h:86: 1 if the device reads pageable host memory in place.  Always 0 here: weights
 * live in HBM and a "wrap" copies (the engine then skips its zero-copy branches, gpu.rs:207). */
int coli_cuda_pageable_access(int device);
/* backend_cuda.h:66 and 69: residency switches of the reference's unified-memory box; accepted
 * and without effect (weights and expert staging are always device copies here). */
void coli_cuda_set_weight_zerocopy(int on);
void coli_cuda_set_ffn_devcopy(int on);
/* backend_cuda.h:87-91: page-lock / release host memory the caller owns.  register returns 0 on
 * failure with the error cleared; the caller carries on with pageable memory. */
int coli_cuda_host_register(void *p, size_t bytes);
void coli_cuda_host_unregister(void *p);
/* Added: text of the most recent failure on the calling thread ("" if none).  The reference
 * logs "[CUDA] what: msg" to stderr (backend_cuda.cu:102-106); this library does both. */
const char *coli_cuda_last_error(void);

/* ---- resident weights -------------------------------------------------------------------- */
/* backend_cuda.h:57-59 / backend_cuda.cu:2880-2920.  Copies a host matrix into HBM.  fmt 4:
 * `weights` = e4m3 codes [O,I], `scales` = f32 [O].  fmt 8: `weights` = e4m3 codes [O,I],
 * `scales` = f32 [ceil(O/128), ceil(I/128)].  fmt 5 must use coli_cuda_tensor_wrap_nvfp4.
 * If *tensor is already set, only checks fmt/I/O/device and returns (backend_cuda.cu:2892-2895). */
int coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt,
                            int I, int O, int device);
/* backend_cuda.h:80-82.  Same as upload here: B200 has no pageable zero-copy at speed, so a
 * "wrap" copies into HBM and the handle owns that copy. */
int coli_cuda_tensor_wrap(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt, int I,
                          int O, int device);
/* crates/colibri-backend/src/cuda.rs:69-77 / backend_cuda.cu:5311-5330.  `weights` = packed
 * e2m1 nibbles [O, ceil(I/2)] (low nibble = even column), `bscale` = ue4m3 per-16 block scales
 * [O, ceil(I/16)], `gscale` = per-tensor f32.  Host pointers; copied into HBM. */
int coli_cuda_tensor_wrap_nvfp4(ColiCudaTensor **tensor, const void *weights, const void *bscale, float gscale,
                                int I, int O, int device);
/* backend_cuda.h:71-72 (Rust declaration cuda.rs:83-91).  MXFP4: the same packed e2m1 nibbles,
 * `bscale` = one OCP E8M0 byte (2^(b-127)) per 32 inputs, [O, ceil(I/32)]; `gscale` is 1.0 in real
 * containers (linear.rs:134-175).  Host pointers; copied into HBM, where the matrix is held in the
 * NVFP4 form: every block scale becomes the ue4m3 code of the same power of two relative to the
 * tensor's largest block scale (one shift per tensor, folded into gscale), so the decoded weights
 * are bit-identical as long as a block lies within 17 binades of the largest one; a block further
 * below decodes as zero (its weights are under 2^-17 of the largest block's), and a scale byte
 * of 0xFF (NaN) stays NaN.  Blocks whose nibbles are all zero are ignored when the shift is chosen. */
int coli_cuda_tensor_wrap_mxfp4(ColiCudaTensor **tensor, const void *weights, const void *bscale, float gscale,
                                int I, int O, int device);
/* Added: the host half of the call above, on HOST pointers and without touching a GPU: the ue4m3
 * per-16 scale bytes [O, ceil(I/16)] and the tensor scale under which an MXFP4 matrix is held. */
int coli_b200_mxfp4_resident_scales(const void *weights, const void *bscale, float gscale, int I, int O,
                                    void *bscale16_out, float *gscale_out);
/* backend_cuda.h:270-272. */
void coli_cuda_tensor_free(ColiCudaTensor *tensor);
size_t coli_cuda_tensor_bytes(const ColiCudaTensor *tensor);
int coli_cuda_tensor_device(const ColiCudaTensor *tensor);

/* Added: build a handle from matrices that already sit in device memory, in the same layouts
 * as the host-pointer calls above (q = nibbles or codes, s = ue4m3 bytes or f32 scales). */
int coli_b200_tensor_from_device(ColiCudaTensor **tensor, int fmt, const void *d_q, const void *d_s,
                                 float gscale, int I, int O, int device);
/* Added: copy a handle's contents back to HOST memory in the layouts of the upload calls
 * (inverse of the HBM repack).  `gscale` may be NULL. */
int coli_b200_tensor_export(const ColiCudaTensor *tensor, void *q_host, void *s_host, float *gscale);
/* Added: device-side quantisers, bit-identical to the reference's
 * (crates/colibri-engine/src/convert.rs:1107-1135 for NVFP4; the 128x128 FP8 encoder is the
 * per-row rule of convert.rs:1042-1054 applied per block).  All pointers are device pointers,
 * `d_w` is f32 [O,I]; nvfp4 returns the per-tensor scale through the host pointer `gscale`. */
int coli_b200_quantize_nvfp4(int device, const float *d_w, int O, int I, void *d_nibbles, void *d_bscale,
                             float *gscale);
int coli_b200_quantize_fp8_b128(int device, const float *d_w, int O, int I, void *d_codes, float *d_scales);

/* ---- expert FFN, reference signatures ------------------------------------------------------
 * x is rounded from f32 to f16 on the device (nearest even, saturating at +-65504), as the
 * reference's GPU path does before its fp16 MMA; y is f32.  A group that averages at least 8 rows
 * per expert runs on the tcgen05 kernels, whose result passes through bf16 (2^-9 relative) before
 * it is widened to f32; smaller groups write f32 directly.  The choice depends on the row counts
 * alone. */
/* backend_cuda.h:97-99 semantics for NVFP4 (backend_cuda.cu:3668-3806): y = down(silu(gate x) * up x),
 * x and y are HOST f32 [S, D] with D = gate->I; synchronous. */
int coli_cuda_expert_mlp_nvfp4(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                               const float *x, int S);
/* backend_cuda.h:104-105 (fmt 4 per-row scaled e4m3; this library also accepts fmt 8). */
int coli_cuda_expert_mlp_fp8(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                             const float *x, int S);
/* backend_cuda.h:75-76 and cuda.rs:212-220 (backend_cuda.cu:5707): the MXFP4 forms of the two
 * calls above; fmt must be 6 on every tensor.  Same host-f32, synchronous contract. */
int coli_cuda_expert_mlp_mxfp4(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y, const float *x,
                               int S);
int coli_cuda_expert_group_mxfp4(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups, ColiCudaTensor *const *downs,
                                 const int *rows, int count, float *y, const float *x);
/* backend_cuda.h:77-79: the same expert under Kimi-K3's "situ" activation.  That activation is not
 * part of this library: the call always declines with 0 and an error text, as the reference's
 * does when it cannot run (gpu.rs try_expert_ffn_mxfp4_situ falls back on a 0). */
int coli_cuda_expert_mlp_mxfp4_situ(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                    const float *x, int S, float beta, float linear_beta);
/* backend_cuda.h:107-109 and 136-140: the format-agnostic forms of the calls above.  Accepted
 * formats are the ones this library keeps resident (4, 5, 8); the reference's f32 / int8 / int2
 * expert tensors are declined with 0. */
int coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y, const float *x, int S);
int coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups, ColiCudaTensor *const *downs,
                           const int *rows, int count, float *y, const float *x);
/* backend_cuda.h:127-129: y[S,O] = x[S,I] @ W[O,I]^T for an NVFP4 matrix (host f32 in and out,
 * synchronous).  The first call copies the container into HBM through *tensor, later calls reuse
 * the handle; x is rounded to f16 on the device as in the expert calls. */
int coli_cuda_matmul_nvfp4(ColiCudaTensor **tensor, float *y, const float *x, const void *weights, const void *bscale,
                           float gscale, int S, int I, int O, int device);
/* backend_cuda.h:131-132, 152-160: gateless ReLU^2 NVFP4 experts, y = down(relu(up x)^2)
 * (moe.rs:1189-1199).  x, y: host f32, sum(rows) consecutive rows of up->I values in call order.
 * The three forms differ only in how the reference batches its launches; here all run the whole
 * group in two launches.  `exact` is accepted and has no effect: a row's result never depends on
 * the other rows of a call. */
int coli_cuda_expert_mlp_nvfp4_relu2(ColiCudaTensor *up, ColiCudaTensor *down, float *y, const float *x, int S, int exact);
int coli_cuda_expert_group_nvfp4_relu2(ColiCudaTensor *const *ups, ColiCudaTensor *const *downs, const int *rows, int count,
                                       float *y, const float *x);
int coli_cuda_expert_seg_nvfp4_relu2(ColiCudaTensor *const *ups, ColiCudaTensor *const *downs, const int *rows, int count,
                                     float *y, const float *x);
/* backend_cuda.h:134-140 / backend_cuda.cu:4410-4792: packed group of same-shaped experts; x and
 * y hold sum(rows) consecutive [D] HOST f32 rows in call order. */
int coli_cuda_expert_group_nvfp4(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                 ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                                 const float *x);
/* backend_cuda.h:89-92 restricted to fmt 0, the router GEMM the engine issues through it
 * (crates/colibri-engine/src/gpu.rs:2219-2249): y[S,O] = x[S,I] @ W[O,I]^T with a k-ascending
 * f32 sum per output.  HOST pointers; `tensor` caches the device copy of W as in the reference. */
int coli_cuda_matmul(ColiCudaTensor **tensor, float *y, const float *x, const void *weights,
                     const float *scales, int fmt, int S, int I, int O, int device);

/* ---- whole block (no counterpart in the reference: its router, top-k, gather, combine and
 * shared-expert add run on the CPU in crates/colibri-engine/src/moe.rs:1799-1895) ----------- */
#define COLI_SCORE_SOFTMAX 0
#define COLI_SCORE_SIGMOID 1

typedef struct ColiMoeLayer {
  int32_t H, E, k, I;      /* hidden, routed experts, top-k, expert intermediate */
  int32_t score;           /* COLI_SCORE_* (colibri_core::RouterScore) */
  int32_t norm_topk;       /* cfg.norm_topk */
  float routed_scale;      /* cfg.routed_scale */
  int32_t n_group;         /* 1 = ungrouped (the reference's only mode) */
  int32_t topk_group;
  int32_t fmt;             /* COLI_FMT_NVFP4, _MXFP4, _FP8_B128 or _E4M3_ROW, all experts alike */
  int32_t device;
  const void *router_w;    /* HOST bf16 [E,H]; copied at create */
  const float *select_bias;/* HOST f32 [E] or NULL; sigmoid arm, selection only (moe.rs:1104) */
  const float *logit_bias; /* HOST f32 [E] or NULL; extension: added to the logits */
  ColiCudaTensor *const *gate; /* E entries; NULL entry = expert not resident on this rank */
  ColiCudaTensor *const *up;
  ColiCudaTensor *const *down;
  ColiCudaTensor *sh_gate; /* shared expert or NULL (all three) */
  ColiCudaTensor *sh_up;
  ColiCudaTensor *sh_down;
  int32_t ep_rank, ep_world;   /* expert-parallel placement; 0/1 = single GPU */
  const int32_t *expert_owner; /* HOST [E] or NULL = contiguous e*world/E (sharding.rs:197-203) */
  void *nccl_comm;             /* ncclComm_t over the ep_world ranks (this rank = ep_rank), or NULL; needed by
                                  coli_b200_moe_block_ep_dev only.  Stays the caller's: the handle never destroys it. */
} ColiMoeLayer;

typedef struct ColiMoe ColiMoe; /* layer tables + workspace for up to max_tokens tokens */

int coli_b200_moe_create(ColiMoe **moe, const ColiMoeLayer *layer, int max_tokens);
void coli_b200_moe_destroy(ColiMoe *moe);
/* Bytes of HBM workspace the handle owns (excludes the weights). */
size_t coli_b200_moe_workspace_bytes(const ColiMoe *moe);

/* One block call, synchronous, HOST bf16 x[T,H] -> HOST bf16 out[T,H] (host<->device copies
 * inside).  topk_idx [T,k] int32 and topk_w [T,k] f32 are optional HOST outputs.  All experts
 * must be resident (single GPU). */
int coli_b200_moe_block(ColiMoe *moe, const void *x, void *out, int T, int32_t *topk_idx, float *topk_w);
/* Same with DEVICE pointers, asynchronous on `stream` (a cudaStream_t; NULL is CUDA's default
 * stream, coli_b200_moe_stream() gives the handle's own).  One handle's workspace serves one
 * call at a time: calls on different streams must not overlap. */
int coli_b200_moe_block_dev(ColiMoe *moe, const void *x_dev, void *out_dev, int T, void *stream);
/* The layer step around the block (forward.rs:376-393), all on device pointers and asynchronous
 * on `stream`: x = bf16(rmsnorm(resid, post_ln_w, eps)) (math.rs:8-20, mean square in f64), then
 * resid += moe_block(x), the add fused into the combine so the block output is not rounded first.
 * resid_dev: f32 [T,H], updated in place; post_ln_w_dev: f32 [H].  H must be a multiple of 8.
 * No reference C symbol corresponds to it: the reference runs these steps on the host. */
int coli_b200_moe_layer_step_dev(ColiMoe *moe, float *resid_dev, const float *post_ln_w_dev, float eps, int T, void *stream);
/* Synchronise the device and return 1 if every kernel launched through this handle since the
 * last check ran to completion, 0 (with an error text) if one abandoned a bounded device-side
 * wait.  The host-pointer call above performs this check itself. */
int coli_b200_moe_check(ColiMoe *moe);
/* Copy the last call's routing to HOST (after synchronising the stream). */
int coli_b200_moe_last_routing(ColiMoe *moe, int T, int32_t *topk_idx, float *topk_w);

/* ---- stages, DEVICE pointers, asynchronous (what the expert-parallel path is built from; they
 * replace crates/colibri-engine/src/moe.rs:1620-1734 `sharded_experts_partial`).  The sequence on
 * every rank is: topk (own tokens) -> all-gather of tokens and routing -> gather_local -> experts
 * -> combine_partial -> reduce-scatter of the partials -> finish (+ shared expert of the own
 * tokens).  All sizes exchanged between ranks follow from (T, H, k) alone, so no host
 * synchronisation is needed anywhere.  A handle used this way is created with max_tokens = the
 * token count of ALL ranks. ------------------------------------------------------------------ */
/* Number of routed experts resident on this rank (= segments of gather_local / experts). */
int coli_b200_moe_local_experts(const ColiMoe *moe);
/* Router GEMM + score + top-k for x_dev[T,H] -> topk_idx_dev [T,k] int32, topk_w_dev [T,k] f32. */
int coli_b200_moe_topk_dev(ColiMoe *moe, const void *x_dev, int T, int32_t *topk_idx_dev, float *topk_w_dev,
                           void *stream);
/* For routing topk_idx_dev[T,k] over x_dev[T,H]: copy the rows of the (token, kk) pairs whose
 * expert is resident here into rows_dev (2 bytes per element, capacity T*k rows; the encoding is
 * the library's own -- the bf16 values held as f16 -- and only experts_dev reads it), expert-contiguous in ascending
 * expert id, tokens ascending inside an expert (moe.rs:1373-1387).  seg_count_dev[n_local]
 * receives the rows per resident expert, slot_dev[T*k] the row of each pair or -1. */
int coli_b200_moe_gather_local_dev(ColiMoe *moe, const void *x_dev, const int32_t *topk_idx_dev, int T, void *rows_dev,
                                   int32_t *seg_count_dev, int32_t *slot_dev, void *stream);
/* Grouped SwiGLU FFN of the resident experts over those rows -> y_dev (bf16 [rows, H]); the
 * device-pointer form of coli_cuda_expert_group_nvfp4.  rows_cap = rows the two buffers hold;
 * rows_expected (e.g. T*k/world) only selects the kernel family.  rows_dev and y_dev must be
 * 16-byte aligned (TMA reads the rows; the tcgen05 kernels write result rows 8 bytes at a time). */
int coli_b200_moe_experts_dev(ColiMoe *moe, const void *rows_dev, const int32_t *seg_count_dev, int rows_cap,
                              int rows_expected, void *y_dev, void *stream);
/* Shared expert over x_dev[T,H] -> y_dev[T,H] (bf16). */
int coli_b200_moe_shared_dev(ColiMoe *moe, const void *x_dev, int T, void *y_dev, void *stream);
/* partial[t] = sum over kk with slot >= 0 of w[t,kk] * y_rows[slot[t,kk]], kk ascending, f32 [T,H]
 * (moe.rs:1549-1553 restricted to this rank's experts; ranks are summed by the reduce-scatter as
 * moe.rs:1725-1733 folds peer partials). */
int coli_b200_moe_combine_partial_dev(ColiMoe *moe, const void *y_rows_dev, const int32_t *slot_dev,
                                      const float *topk_w_dev, float *partial_dev, int T, void *stream);
/* out[t] = bf16(partial[t] + shared_y[t]) (shared_y_dev may be NULL) — moe.rs:1875-1885. */
int coli_b200_moe_finish_dev(ColiMoe *moe, const float *partial_dev, const void *shared_y_dev, void *out_dev, int T,
                             void *stream);

/* ---- expert-parallel block: one call per rank (replaces crates/colibri-engine/src/moe.rs:1737-1794
 * `moe_sharded` and :1620-1734 `sharded_experts_partial`; the TCP request/response of
 * crates/colibri-cluster/src/transport.rs:33-58 becomes an all-to-all over NCCL send/recv) -----------
 * The handle is created with ep_rank / ep_world / expert_owner, the experts this rank owns, the
 * shared expert (replicated) and nccl_comm; max_tokens bounds the tokens of ALL ranks in one call.
 * Every rank calls with its own x_dev[T_local,H] (bf16; T_local may differ between ranks and may be
 * 0) and receives out_dev[T_local,H].  Sequence: router + top-k of the own tokens; each token row is
 * sent ONCE to every rank that owns at least one of its k experts (with the k expert ids); the
 * owners run the grouped expert FFN over the rows they received and send the result row of every
 * (token, kk) pair back unweighted; the home rank applies the routing weights in the token's own kk
 * order and adds its shared expert, so the arithmetic is that of the single-GPU block.  The shared
 * expert runs on a second stream beside the exchange.
 * Transport.  By default ("direct") every rank keeps its receive buffers in one slab that the other
 * ranks map at create time (cudaIpc handles, all-gathered over nccl_comm); the pack kernels store
 * rows, expert ids and the per-rank counts straight into the destination's slab over NVLink, and a
 * barrier after the stores tells a rank that its senders are done: every rank publishes a growing
 * count in a flag row of each peer's slab and waits, for about two seconds at most, until all peers'
 * counts in its own row have caught up (a wait that runs out fails the call: coli_b200_moe_check).
 * COLI_EP_BARRIER=nccl at create replaces it with a one-word NCCL all-gather.
 * Nothing needs the host: the call only queues work on `stream`.  With COLI_EP_TRANSPORT=nccl in
 * the environment when the handle is created, rows are packed into send buffers and exchanged with
 * grouped ncclSend / ncclRecv instead; the host then waits once per call for the counts those need.
 * The call must be made by every rank of the communicator, in the same order.  Limits: at most 8
 * ranks, k <= 16; all ranks together may bring at most max_tokens tokens to a call (a call that
 * brings more computes nothing for the overflowing rank and coli_b200_moe_check reports it). */
int coli_b200_moe_block_ep_dev(ColiMoe *moe, const void *x_dev, void *out_dev, int T_local, void *stream);
/* The same sequence for `world` handles of ONE process on ONE device (ranks[r] has ep_rank = r, no
 * communicator): phases run rank after rank on `stream`, the exchanges are device-to-device copies.
 * For checking the expert-parallel path on a single GPU; x_dev / out_dev / T_local have one entry
 * per rank. */
int coli_b200_moe_block_ep_emulate(ColiMoe *const *ranks, int world, const void *const *x_dev, void *const *out_dev,
                                   const int *T_local, void *stream);
/* Test aid for the bounded wait of the direct transport's barrier: one barrier on this handle alone,
 * with a wait of about 13 ms.  peers_arrive != 0 writes the peers' counts into the own flag row
 * first (the wait succeeds); with 0 nothing sets them, the wait runs out and coli_b200_moe_check
 * reports the abandoned barrier (and clears the report).  The handle must have made an
 * expert-parallel or emulated call before. */
int coli_b200_ep_barrier_probe(ColiMoe *moe, int peers_arrive, void *stream);
/* For callers without a communicator of their own: rank 0 obtains a 128-byte id, passes it to the
 * other ranks by any means, and every rank creates its end (ncclGetUniqueId / ncclCommInitRank of
 * the NCCL library already in the process, else libnccl.so.2).  `device` must be initialised. */
int coli_b200_nccl_unique_id(void *id128);
int coli_b200_nccl_comm_create(void **comm, const void *id128, int rank, int world, int device);
void coli_b200_nccl_comm_destroy(void *comm);
/* Host-only (no GPU is touched): the layout rank `rank` derives from a count table [world][2*world]
 * as returned by coli_b200_ep_last_counts.  out is int32 [8][world]: tokens sent to d, pairs owned by
 * d, tokens received from s, pairs received from s, then the first row of each peer's segment in the
 * send buffer, the receive buffer, the return-send buffer and the return-receive buffer.  Segments
 * are laid out own first, then the peers in ascending rank, on both sides of both exchanges. */
int coli_b200_ep_layout(const int32_t *table, int world, int rank, int32_t *out);
/* Stage timing of the expert-parallel call (measurement mode: synchronises at the end of every
 * call while on).  ms[COLI_EP_STAGES]: router+top-k, plan+pack, count exchange (includes the host
 * wait), dispatch, permute, expert FFN, return pack, return exchange, combine. */
#define COLI_EP_STAGES 9
int coli_b200_ep_profile(ColiMoe *moe, int enable);
int coli_b200_ep_stage_ms(ColiMoe *moe, float *ms /* [COLI_EP_STAGES] */, int *calls);
/* The count table of the last expert-parallel call, HOST int32 [world][2*world]: row s = rank s's
 * tokens sent to each rank, then its (token, kk) pairs owned by each rank. */
int coli_b200_ep_last_counts(ColiMoe *moe, int32_t *table);

/* ---- tracing (the role of the reference's COLI_PROFILE phase counters ROUTER_US, MOE_PREP_US,
 * GPUFFN_US, SCATTER_US, crates/colibri-engine/src/forward.rs:86-160) ------------------------ */
#define COLI_PHASE_ROUTER 0  /* router GEMM + score + top-k */
#define COLI_PHASE_PERMUTE 1 /* segment counts, offsets, row permutation, work list */
#define COLI_PHASE_GATE_UP 2 /* grouped gate/up GEMM with SiLU*mul */
#define COLI_PHASE_DOWN 3    /* grouped down GEMM */
#define COLI_PHASE_COMBINE 4 /* weighted combine + shared add */
#define COLI_PHASES 5
/* With profiling on, coli_b200_moe_block_dev brackets each phase with CUDA events on the
 * launching stream and synchronises at the end of the call to accumulate them (so it is a
 * measurement mode, not a fast path).  Turning it on clears the accumulators. */
int coli_b200_moe_profile(ColiMoe *moe, int enable);
/* Accumulated milliseconds per phase and the number of block calls they cover. */
int coli_b200_moe_phase_ms(ColiMoe *moe, float *ms /* [COLI_PHASES] */, int *calls);
/* The handle's own stream (a cudaStream_t), on which the host-pointer block call runs. */
void *coli_b200_moe_stream(ColiMoe *moe);
/* Kernels this library has launched in the calling process since it was loaded. */
uint64_t coli_b200_launch_count(void);

/* ---- routing with no allocation (no counterpart in the reference: there the router runs on the
 * CPU, crates/colibri-engine/src/moe.rs:1047-1132, and allocates freely) ------------------------
 * For callers that cannot allocate device memory at all — a server whose HBM is fully handed to
 * its weight and KV pools (cudaMalloc would fail or upset its memory ledger), or a decode loop
 * that cannot take the device-wide stall of cudaMalloc/cudaFree.  Router GEMM + score + top-k
 * for x_dev[T,H] (bf16) against router_w_dev[E,H] (bf16); results go to topk_idx_dev [T,k] and
 * topk_w_dev [T,k], bit-identical to what a ColiMoe handle computes.  Everything is a DEVICE
 * pointer supplied by the caller; the only scratch, the [T,E] f32 logits, sits in a fixed
 * 512 KiB device array built into the library (resident on every GPU that loads it, until
 * exit), so the call makes no cudaMalloc/cudaFree and needs T*E <= COLI_ROUTE_NOALLOC_MAX_LOGITS
 * (larger batches are refused with an error).
 * The first call on a device looks up that array's device address (once per device, with the
 * device current) — make that first call before starting any stream capture.
 * All calls on one GPU share the one array: it keeps the previous call's logits (harmless, each
 * call overwrites its own [T,E] before reading) and two calls that overlap on the GPU — on
 * different streams, or from different threads — race on it; serialise them.
 * x_dev and router_w_dev must be 16-byte aligned (128-bit loads); a misaligned pointer is refused. */
#define COLI_ROUTE_NOALLOC_MAX_LOGITS 131072
int coli_b200_route_noalloc(const void *x_dev, const void *router_w_dev, const float *select_bias_dev,
                            const float *logit_bias_dev, int T, int H, int E, int k, int score, int norm_topk,
                            float routed_scale, int n_group, int topk_group, int32_t *topk_idx_dev,
                            float *topk_w_dev, void *stream);

/* FNV-1a fingerprint of an expert->rank map (crates/colibri-cluster/src/sharding.rs:251-265);
 * `owner` NULL = contiguous.  Ranks compare it before the first exchange. */
uint64_t coli_b200_sharding_fingerprint(uint32_t num_nodes, uint32_t n_experts, const uint32_t *owner);

#ifdef __cplusplus
}
#endif
#endif /* COLI_B200_H */
