// Internal declarations shared by the translation units of libcoli_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/coli_b200.h"
#include "coli_math.h"

// ---- resident weight handle -----------------------------------------------------------------
// HBM layout ("k-tile major"): the K (input) axis is cut into tiles of 128; for each k-tile
// all O rows are stored back to back, so the slab a CTA streams for (rows r0..r0+n, k-tile kt)
// is one contiguous run of bytes.
//   NVFP4     q: [KT][Op][64 B]   16 B chunk c of a row covers k = kt*128 + 32c .. +31; every
//                                 byte holds two consecutive k, low nibble first (the operand
//                                 form of cvt.rn.f16x2.e2m1x2).
//             s: [KT][Op][8 B]    the ue4m3 code of each 16-wide block, k ascending
//   FP8_B128  q: [KT][Op][128 B]  e4m3 codes, k ascending
//             s: f32 [ceil(O/128)][KT]   (the reference's own grid, convert.rs:731-741)
//   E4M3_ROW  q as FP8_B128; s: f32 [O] row scales (linear.rs:93-109)
//   MXFP4     held in the NVFP4 form above: at upload each E8M0 scale 2^e of a 32-wide block is
//             re-expressed as the ue4m3 code of 2^(e + shift) for both of its 16-wide halves, with
//             one shift per tensor folded into the tensor scale (gscale x 2^-shift), so every
//             expert kernel reads it unchanged; `s_src` keeps the container's own scale bytes for
//             the export call.  The handle's fmt stays 6; kernels are given coli_kernel_fmt(fmt).
// Op = O rounded up to 16, Kp = I rounded up to 128; padding bytes are zero (decode to 0.0).
//
// Arithmetic type of the expert GEMMs: f16 x f16 -> f32.  FP4/FP8 codes convert to f16 with one
// hardware cvt per pair, a decoded weight (code x block scale, at most 6 significant bits, between
// 2^-10 and 2688) is exact in f16, and a bf16 activation is exact in f16 whenever its magnitude
// lies in [2^-14, 65504]; smaller ones lose at most 2^-25 absolute, larger ones saturate.  The
// intermediate h keeps the value rounded to bf16 (what the reference stores) held in f16.
struct ColiCudaTensor {
  int fmt, I, O, device;
  int Kp, Op, KT;
  uint8_t *q;
  uint8_t *s;
  float gscale;
  size_t q_bytes, s_bytes;
  uint8_t *s_src;       // MXFP4 only: the E8M0 block scales as uploaded, [O, ceil(I/32)]
  size_t s_src_bytes;
  float gscale_src;     // MXFP4 only: the tensor scale as uploaded (gscale above carries the shift)
};
// the format the expert kernels decode for a handle of format `fmt`
static inline int coli_kernel_fmt(int fmt) { return fmt == COLI_FMT_MXFP4 ? COLI_FMT_NVFP4 : fmt; }

// What a kernel needs to read one matrix.
struct WeightRef {
  const uint8_t *q;
  const uint8_t *s;
  float g;
  int pad;
};

static inline int round_up(int a, int b) { return (a + b - 1) / b * b; }
// Upper bound of the work items `rows` rows in at most `nseg` segments cut into: a segment of n
// rows gives ceil(n / rpi) <= n / rpi + 1 items and at most min(nseg, rows) segments hold a row.
// Kernel grids are sized from this bound, so a loose one costs idle CTAs on every decode step.
static inline int max_work_items(int rows, int nseg, int rpi) { return rows / rpi + (rows < nseg ? rows : nseg); }

// ---- error reporting -------------------------------------------------------------------------
void coli_set_error(const char *fmt, ...);
bool coli_cuda_check(cudaError_t e, const char *what);
#define CK(call, what)                          \
  do {                                          \
    if (!coli_cuda_check((call), (what))) return 0; \
  } while (0)

// every kernel launch of the library bumps this (read through coli_b200_launch_count)
void coli_count_launch(int n);

// A "done once" flag per CUDA device.  Function attributes (cudaFuncSetAttribute) and occupancy
// figures belong to one device's copy of a kernel, and one process may drive several devices
// (coli_cuda_init takes a list), so a launcher that has to raise a kernel's shared-memory limit
// keeps one of these per kernel instead of a process-wide bool.  The guarded action must be
// idempotent: two host threads may both see "not done" for the same device.
struct ColiPerDeviceOnce {
  unsigned done_mask = 0;  // bit d = done on device ordinal d (ordinals >= 32 are never cached)
  // the current device's ordinal, or -1; `done` tells whether the action already ran there
  int current(bool *done) const {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    *done = dev >= 0 && dev < 32 && ((__atomic_load_n(&done_mask, __ATOMIC_ACQUIRE) >> dev) & 1u);
    return dev;
  }
  void mark(int dev) {
    if (dev >= 0 && dev < 32) __atomic_fetch_or(&done_mask, 1u << dev, __ATOMIC_RELEASE);
  }
};
// Raise a kernel's dynamic shared-memory limit on the current device, once per device.
template <class K>
static inline bool coli_set_smem_limit(ColiPerDeviceOnce &once, K kernel, size_t bytes, const char *what) {
  bool done = false;
  const int dev = once.current(&done);
  if (done) return true;
  if (!coli_cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes), what)) return false;
  once.mark(dev);
  return true;
}

// ---- launchers (defined in the kernel translation units) ------------------------------------
namespace colib {

// layout.cu
int pack_nvfp4(const uint8_t *d_nib, const uint8_t *d_bs, int O, int I, ColiCudaTensor *t, cudaStream_t st);
int pack_fp8(const uint8_t *d_codes, int O, int I, ColiCudaTensor *t, cudaStream_t st);
int unpack_nvfp4(const ColiCudaTensor *t, uint8_t *d_nib, uint8_t *d_bs, cudaStream_t st);
int unpack_fp8(const ColiCudaTensor *t, uint8_t *d_codes, cudaStream_t st);
int quantize_nvfp4(const float *d_w, int O, int I, uint8_t *d_nib, uint8_t *d_bs, float *d_amax_scratch,
                   float *gscale_out, cudaStream_t st);
int quantize_fp8_b128(const float *d_w, int O, int I, uint8_t *d_codes, float *d_scales, cudaStream_t st);

// routing.cu
struct RouteParams {
  int T, H, E, k;
  int score, norm_topk;
  float routed_scale;
  int n_group, topk_group;
  const __nv_bfloat16 *x;         // [T,H]
  const __nv_bfloat16 *router_w;  // [E,H]
  const float *select_bias;       // [E] or null
  const float *logit_bias;        // [E] or null
  float *logits;                  // [T,E] scratch
  int32_t *topk_idx;              // [T,k]
  float *topk_w;                  // [T,k]
};
int launch_router(const RouteParams &p, cudaStream_t st);

struct PermuteParams {
  int T, H, E, k;
  int nseg_routed;             // routed segments: E, or the number of experts resident on this rank
  int has_shared;              // append T identity rows for the shared expert (segment index nseg_routed)
  int rows_per_item;           // token rows per work item
  const int32_t *topk_idx;     // [T,k]
  const int32_t *expert_slot;  // [E] segment position of each expert (null = identity, < 0 = not resident)
  int32_t *local_rank;         // [T*k] scratch
  int32_t *chunk_cnt;          // [nchunk][E] scratch
  int32_t *seg_count;          // [E] out: rows per segment (segment order)
  int32_t *seg_off;            // [E+2] out: exclusive offsets (+shared)
  int32_t *slot;               // [T*k] out: row position of (t,kk)
  int32_t *row_token;          // [T*k (+T)] out: token of each row
  int32_t *item_seg;           // work list out: segment (expert position) of each item
  int32_t *item_row0;          //                first row
  int32_t *item_nrows;         //                rows (<= rows_per_item)
  int32_t *n_items;            // [1]
  const __nv_bfloat16 *x;      // [T,H]  (null = do not materialise rows)
  __half *xg;                  // [T*k (+T),H] gathered rows as f16 (null = skip)
  int gather_shared;           // also copy the shared expert's T identity rows into xg
  __half *x16;                 // [T,H] f16 copy of x in token order (null = skip)
  // Virtual batch (expert parallelism): the tokens are the concatenation of up to 8 segments that
  // sit at fixed places of a larger buffer, with their lengths known on the device only.  When
  // `virt` is set, T above is an upper bound used for grid sizes, the token count is virt->total, and
  // token j lives in row virt->phys[s] * virt->stride + (j - virt->off[s]) of x / topk_idx, s being its segment.
  const struct VirtualBatch *virt;
  int rows_cap;                // rows xg / row_token hold; a pair beyond it gets no row and raises *overflow
  int *overflow;               // device word (may be null)
};
struct VirtualBatch {
  int32_t nseg, stride, total, pad;
  int32_t off[9];   // first token of each segment (off[nseg] = total)
  int32_t phys[8];  // buffer slot of each segment
};
__device__ __forceinline__ int coli_virt_row(const VirtualBatch *v, int j) {
  int s = 0;
  while (s + 1 < v->nseg && j >= v->off[s + 1]) ++s;
  return v->phys[s] * v->stride + (j - v->off[s]);
}
int launch_permute(const PermuteParams &p, cudaStream_t st);
// Router + top-k + permutation of a decode-sized batch (T <= 8) in one launch.  Returns 1 on
// success, 0 on error, -1 when the shapes do not qualify (run launch_router + launch_permute).
// `ticket` is a device word that is zero between launches.
int launch_decode_front(const RouteParams &rp, const PermuteParams &pp, unsigned int *ticket, cudaStream_t st);
// Work list for rows that are already expert-contiguous (counts on the device).
int launch_items_from_counts(const int32_t *seg_count, int nseg, int rows_per_item, int32_t *seg_off,
                             int32_t *item_seg, int32_t *item_row0, int32_t *item_nrows, int32_t *n_items,
                             cudaStream_t st);

// Gate/up combine of the expert FFN (coli_math.h: coli_act_combine states the three forms).
struct ActParams {
  int oai;
  float alpha, limit;
};

// expert_small.cu
struct FfnParams {
  int fmt, H, I;
  const WeightRef *gate, *up, *down;  // indexed by segment->expert table
  const int32_t *seg_expert;          // [nseg] weight-table index of each segment (null = identity)
  const int32_t *item_seg, *item_row0, *item_nrows, *n_items;
  int max_items;
  int rows_per_item;         // rows per work item the list was cut with (<= 32)
  int items_expected;        // host estimate of the work items (selects split-K vs tile-per-warp)
  const __half *x;           // source rows (f16)
  const int32_t *row_token;  // row -> source row index (null = identity)
  __half *h;                 // [rows, I] scratch
  __nv_bfloat16 *y;          // [rows, H] out (bf16), or
  float *y32;                // [rows, H] out (f32) when not null
  __half *relu2_out;         // down form only, when not null: write relu(v)^2 (rounded to bf16, held in
                             // f16) here instead of y -- the first half of a gateless ReLU^2 expert
  ActParams act;
};
int launch_gate_up_small(const FfnParams &p, cudaStream_t st);  // h = silu(gate x) * (up x)
int launch_down_small(const FfnParams &p, cudaStream_t st);     // y = down h
int launch_ffn_small(const FfnParams &p, cudaStream_t st);      // both

// expert_tc.cu — tcgen05 path for prefill-sized segments
constexpr int TC_MAX_TOKENS = 256;  // token rows per tile = rows per work item on this path
struct TcParams {
  int fmt;  // COLI_FMT_NVFP4 (both kernels); COLI_FMT_FP8_B128 / COLI_FMT_E4M3_ROW (tensor-memory kernel only)
  int H, I;
  const WeightRef *gate, *up, *down;
  const int32_t *seg_expert;
  const int32_t *item_seg, *item_row0, *item_nrows, *n_items;
  int max_items;
  int tile_tokens;   // rows per item the work list was cut with: TC_MAX_TOKENS, TCT_MAX_TOKENS or TCT_SHORT_TOKENS
  __half *h;         // [rows, I]
  __nv_bfloat16 *y;  // [rows, H]
  int *status;       // device word: 0, or the code of the first bounded wait that gave up
  ActParams act;
};
// x_rows: f16 [rows_cap, H] expert-contiguous rows (row index = position in the work list)
int launch_gate_up_tc(const TcParams &p, const void *x_rows, int rows_cap, int sm_count, cudaStream_t st);
int launch_down_tc(const TcParams &p, int rows_cap, int sm_count, cudaStream_t st);
// expert_tc_tmem.cu — the same two stages with the weight operand in tensor memory; tiles of at
// most TCT_MAX_TOKENS rows (the work list must be cut with that many rows per item)
constexpr int TCT_MAX_TOKENS = 160;
// ... or with TCT_SHORT_TOKENS rows per item, for layers whose segments are short: narrower
// accumulators leave tensor memory for a weight ring twice as deep (TcParams::tile_tokens says which)
constexpr int TCT_SHORT_TOKENS = 64;
int launch_gate_up_tct(const TcParams &p, const void *x_rows, int rows_cap, int sm_count, cudaStream_t st);
int launch_down_tct(const TcParams &p, int rows_cap, int sm_count, cudaStream_t st);

// combine.cu
struct CombineParams {
  int T, H, k;
  int has_shared;
  const __nv_bfloat16 *y;         // routed rows [T*k, H]
  const __nv_bfloat16 *shared_y;  // [T,H] shared-expert rows (used when has_shared)
  const int32_t *slot;            // [T*k]
  const float *topk_w;            // [T*k]
  __nv_bfloat16 *out;             // [T,H] bf16 result, or
  float *out32;                   // [T,H] f32 result when not null: the partial sum of this rank's experts
                                  // (has_shared = 0), or with `resid` the layer's new residual stream
  const float *resid;             // [T,H] f32 residual stream added to the block output (forward.rs:391-393);
                                  // may alias out32 (every element is read and written by one thread)
};
int launch_combine(const CombineParams &p, cudaStream_t st);
int launch_finish(const float *partial, const __nv_bfloat16 *shared_y, __nv_bfloat16 *out, int T, int H, cudaStream_t st);
int launch_f32_to_bf16(const float *src, __nv_bfloat16 *dst, size_t n, cudaStream_t st);
// out[t] = bf16(x[t] * r_t * w), r_t = 1 / sqrt(mean(x[t]^2) + eps) with the mean square accumulated
// in f64 (math.rs:8-20); H must be a multiple of 4
int launch_rmsnorm_bf16(const float *x, const float *w, float eps, __nv_bfloat16 *out, int T, int H, cudaStream_t st);
// activations for the expert GEMMs: the block's bf16 values held in f16; the host-f32 calls of the
// reference's API round f32 to f16 directly (nearest even, saturating), as the reference's GPU path does
int launch_bf16_to_f16(const __nv_bfloat16 *src, __half *dst, size_t n, cudaStream_t st);
int launch_f32_to_f16(const float *src, __half *dst, size_t n, cudaStream_t st);
int launch_bf16_to_f32(const __nv_bfloat16 *src, float *dst, size_t n, cudaStream_t st);
// y[S,O] = x[S,I] @ W[O,I]^T, all f32, one thread per output, multiply then add per k in order
// (crates/colibri-engine/src/linear.rs:199-220).
int launch_matmul_f32_seq(const float *x, const float *w, float *y, int S, int I, int O, cudaStream_t st);

// Programmatic dependent launch.  The kernels of the decode step are a few microseconds each, so
// the launch latency between them is a visible share of the step: launched with this helper, a
// kernel may be scheduled while its predecessor in the stream is still running; it must then
// execute coli_grid_dependency_sync() before its first global-memory access, which returns once
// the predecessor has completed and its writes are visible.  Launched the ordinary way (as the
// profiled path does, with an event between kernels) the two device calls are no-ops.
__device__ __forceinline__ void coli_grid_dependency_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // let the successor be scheduled early too
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// bf16 pair (one 32-bit word) -> f16 pair, saturating at the largest finite f16
__device__ __forceinline__ uint32_t coli_bf16x2_to_f16x2(uint32_t w) {
  const float lo = fminf(fmaxf(__uint_as_float(w << 16), -65504.0f), 65504.0f);
  const float hi = fminf(fmaxf(__uint_as_float(w & 0xffff0000u), -65504.0f), 65504.0f);
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ uint4 coli_bf16x8_to_f16x8(uint4 v) {
  return make_uint4(coli_bf16x2_to_f16x2(v.x), coli_bf16x2_to_f16x2(v.y), coli_bf16x2_to_f16x2(v.z),
                    coli_bf16x2_to_f16x2(v.w));
}
// coli_act_combine with the fast exponential: silu(g) * u, or its clamped / OpenAI forms.
// Written with selects on the (uniform) mode instead of branches: inlined sixteen times in an
// unrolled epilogue, a branch per call turns the sixteen independent chains (exp, reciprocal, two
// roundings: ~150 cycles each) into sixteen basic blocks that run one after the other.
__device__ __forceinline__ float coli_act_fast(float g, float u, const ActParams &a) {
  const bool oai = a.oai != 0;
  const bool clamp = oai || a.limit > 0.0f;
  const float gl = fminf(g, a.limit), ul = fminf(fmaxf(u, -a.limit), a.limit);
  g = clamp ? gl : g;
  u = clamp ? ul : u;
  const float al = oai ? a.alpha : 1.0f;
  const float add = oai ? 1.0f : 0.0f;
  return __fdividef(g, 1.0f + __expf(-al * g)) * (u + add);
}
// f32 -> (rounded to bf16) -> f16 bits, saturating
__device__ __forceinline__ __half coli_f32_to_f16_via_bf16(float v) {
  const float r = __bfloat162float(__float2bfloat16_rn(v));
  return __float2half_rn(fminf(fmaxf(r, -65504.0f), 65504.0f));
}

}  // namespace colib
