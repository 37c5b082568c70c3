// Expert FFN for segments of up to 160 rows per tile on the 5th-generation tensor cores, with the
// weight operand in TENSOR MEMORY.
//
// Same formulation as expert_tc.cu (features on the MMA's M = 128, the ragged token count on its
// N), but the decoded weights never pass through shared memory:
// * A operand: 16 producer warps stream the packed NVFP4 or FP8 bytes from HBM with 256-bit loads
//   (one thread = one weight row = one TMEM lane), convert them to f16 in registers and write 64 k
//   per stage straight into a ring of 32-column TMEM slots with tcgen05.st.  A stage holds two
//   weight tiles (gate + up of the same 128 features, or two adjacent 128-feature tiles of down);
//   the ring is three stages deep beside 160-column accumulators, six beside 64-column ones.
// * B operand: up to 160 token rows x 64 k of f16 activations per stage, copied by TMA as ONE box
//   (cp.async.bulk.tensor, 128-byte swizzle, no multicast; one tensor map per box height) into a
//   6-deep shared-memory ring and shared by both weight tiles of the stage.
// * tcgen05.mma kind::f16 with A from tensor memory and B through a shared-memory descriptor,
//   two accumulators of 160 columns, each fed by its own issuing thread (the instruction stream
//   of a single issuing thread, not the tensor core, bounded the first version of this kernel);
//   the epilogue forms act(g, u) or writes the two down tiles.
// Why: with both operands in shared memory an MMA of 128 x 128 x 16 fetches 8 KB per 64 cycles,
// the whole shared-memory bandwidth of an SM, before a single decoded weight is stored there
// (expert_tc.cu tops out near half of the tensor peak at 128 tokens per expert).  Here shared
// memory carries only the token tiles: 16-20 KB written + twice that read per stage.
// TMEM budget: 2 x 160 accumulator columns + 6 x 32 weight columns = 512, which is why this
// kernel takes tiles of at most 160 tokens (a layer with 128 rows per expert on average has
// nearly all of its segments under that); wider segments are cut into several work items.
// Layers with short segments run a second instantiation with 2 x 64 + 12 x 32 columns.
//
// Roles are warp-specialised and synchronise through mbarriers only; the kernel is persistent.
// Every barrier wait is bounded: on a time-out the CTA raises a status word, stops issuing work,
// waits for its own copies and frees its TMEM before returning.
#include "tc_common.cuh"

#ifdef COLI_TT_TRACE
// Measurement aid (never compiled into the library as shipped): clock stamps of CTA 0's first stages.
__device__ long long g_tt_trace[256 * 8];
extern "C" int coli_debug_tt_trace(long long *host) {
  return cudaMemcpyFromSymbol(host, g_tt_trace, sizeof(g_tt_trace)) == cudaSuccess ? 1 : 0;
}
#define TT_TRACE(it, k)                                                                 \
  do {                                                                                  \
    if (GATED && blockIdx.x == 0 && (it) < 256u) g_tt_trace[(it) * 8 + (k)] = clock64(); \
  } while (0)
#else
#define TT_TRACE(it, k) \
  do {                  \
  } while (0)
#endif

namespace colib {

// TMEM budget (512 columns): two accumulators of ACC columns (= the most token rows of a tile) and a
// weight ring of 64 columns per stage (gate + up, or two down tiles, of 64 k).  ACC = 160 leaves 3
// stages; ACC = 64, for layers whose segments are short, leaves 6: the hand-over of a weight
// stage (fill -> store wait -> barrier -> MMA -> commit -> barrier) is a latency chain of a few
// thousand cycles, so the stage rate of a tile with few tokens grows with the depth of this ring.
template <int ACC>
struct TtBudget {
  static constexpr int A_STAGES = (512 - 2 * ACC) / 64;
  static constexpr int A_COL0 = 2 * ACC;
  static_assert(ACC % 32 == 0 && A_STAGES >= 3 && A_COL0 + A_STAGES * 64 <= 512, "TMEM budget");
  // shared-memory ring of token tiles (ACC rows x 64 k of f16 per stage); its depth is also the
  // number of stage barriers (a ring twice as deep was measured and changed nothing)
  static constexpr int B_BYTES = ACC * TC_BK * 2;
  static constexpr int B_STAGES = 6;
  static constexpr int NBARS = 2 * B_STAGES + 2;
  static_assert(B_STAGES % A_STAGES == 0 && B_BYTES % 1024 == 0, "a stage barrier serves both rings");
};
// The token tile of a stage arrives as ONE box of N rows: the copy engine of an SM takes about 64
// cycles per box plus 4 per 128-byte row (measured: 21 B/clk with 32-row boxes, 31 B/clk with
// 160-row ones, on 8 SMs as on 148), and at 21 B/clk the 20 KB tile of a 160-token stage takes
// longer than the stage's MMAs.  One tensor map per box height (32, 64, ... rows).
struct TtMaps {
  CUtensorMap m[TCT_MAX_TOKENS / TC_BOXN];
};
constexpr int TT_PROD_WARPS = 16;
constexpr int TT_MMA2_WARP = 2 + TC_EPI_WARPS + TT_PROD_WARPS;       // the second MMA-issuing warp
constexpr int TT_THREADS = 32 * (TT_MMA2_WARP + 1);                  // 736

// The MMAs of one 64-k stage into ONE accumulator and the commit that releases the stage's
// operands, as one instruction sequence: four k steps of 16 (8 TMEM columns of f16 weights, 32
// bytes = 2 descriptor units of tokens per step).
__device__ __forceinline__ void tt_issue_stage(uint32_t acc, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate_first,
                                               uint32_t bar) {
  asm volatile(
      "{\n"
      ".reg .pred pf, pt;\n"
      ".reg .b64 bd;\n"
      ".reg .b32 a;\n"
      "setp.ne.b32 pf, %4, 0;\n"
      "setp.eq.b32 pt, %4, %4;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, pf;\n"
      "add.s64 bd, %2, 2;\n"
      "add.u32 a, %1, 8;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %3, pt;\n"
      "add.s64 bd, %2, 4;\n"
      "add.u32 a, %1, 16;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %3, pt;\n"
      "add.s64 bd, %2, 6;\n"
      "add.u32 a, %1, 24;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %3, pt;\n"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n"
      "}\n"
      ::"r"(acc), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate_first), "r"(bar)
      : "memory");
}
// 32 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
      "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The 64 weights (32 packed bytes) and 4 block-scale bytes of one row for one 64-k stage.
struct TtPacked {
  uint4 q0, q1;
  uint32_t sc;
};
__device__ __forceinline__ TtPacked tt_load_packed(const WeightRef &w, int Op, int row, int kb) {
  TtPacked r;
  r.q0 = make_uint4(0, 0, 0, 0);
  r.q1 = r.q0;
  r.sc = 0;
  if (row < Op) {
    const size_t base = (size_t)(kb >> 1) * Op + row;
    const uint8_t *qp = w.q + base * 64 + (kb & 1) * 32;
    // one 256-bit load: the 32-byte sector of this row and stage is requested from L2 once
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.q0.x), "=r"(r.q0.y), "=r"(r.q0.z), "=r"(r.q0.w), "=r"(r.q1.x), "=r"(r.q1.y), "=r"(r.q1.z), "=r"(r.q1.w)
                 : "l"(qp));
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r.sc) : "l"(w.s + base * 8 + (kb & 1) * 4));
  }
  return r;
}
// Convert one stage of one row and hand it to the tensor core through 32 TMEM columns.
__device__ __forceinline__ void tt_convert(const TtPacked &pk, uint32_t (&r)[32]) {
  uint32_t m0, m1, m2, m3;
  tc_scales(pk.sc, m0, m1);
  tc_scales(pk.sc >> 16, m2, m3);
  const uint32_t w[8] = {pk.q0.x, pk.q0.y, pk.q0.z, pk.q0.w, pk.q1.x, pk.q1.y, pk.q1.z, pk.q1.w};
  const uint32_t m[4] = {m0, m1, m2, m3};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint4 o = tc_dequant_word(w[j], m[j >> 1]);
    r[4 * j] = o.x;
    r[4 * j + 1] = o.y;
    r[4 * j + 2] = o.z;
    r[4 * j + 3] = o.w;
  }
}

// FP8 (e4m3 codes, one byte per weight): the 64 codes of one row for one 64-k stage and the
// multiplier of the stage.  A weight is code x scale[row block][k-tile] (convert.rs:731-741, f32);
// the accumulator runs over all of K inside tensor memory, so the scale cannot be applied per
// k-tile to partial sums as the register-level kernel does.  Instead each 128-row tile is
// normalised by the largest scale of its row block: the stage's codes are multiplied by
// TT_FP8_HEADROOM x scale / max scale (an f16 in (0, 16], one rounding of 2^-11 relative per weight)
// and the epilogue multiplies the finished sum by max scale / TT_FP8_HEADROOM in f32.  The
// headroom keeps products of small codes with small relative scales out of the f16 subnormals.
// Per-row scales (linear.rs:93-109) need no multiplier: the epilogue thread owns one row.
constexpr float TT_FP8_HEADROOM = 16.0f;
struct TtPacked8 {
  uint4 q[4];
  uint32_t mult;  // f16 multiplier in both halves
};
__device__ __forceinline__ uint32_t tt_f16x2_both(float v) {
  const __half2 h = __float2half2_rn(v);
  return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ TtPacked8 tt_zero_packed8() {
  TtPacked8 r;
#pragma unroll
  for (int j = 0; j < 4; ++j) r.q[j] = make_uint4(0, 0, 0, 0);
  r.mult = 0;
  return r;
}
// `norm` = TT_FP8_HEADROOM / max scale of the row block (block-scaled form), `srow` = that block's
// row of the scale grid; both unused for per-row scales.
template <int FMT>
__device__ __forceinline__ TtPacked8 tt_load_packed8(const WeightRef &w, int Op, int row, int kb, const float *srow, float norm) {
  TtPacked8 r = tt_zero_packed8();
  if (row < Op) {
    const uint8_t *qp = w.q + ((size_t)(kb >> 1) * Op + row) * 128 + (kb & 1) * 64;
    // 256-bit loads: each 32-byte sector of this row and stage is requested from L2 once
#pragma unroll
    for (int j = 0; j < 2; ++j)
      asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(r.q[2 * j].x), "=r"(r.q[2 * j].y), "=r"(r.q[2 * j].z), "=r"(r.q[2 * j].w), "=r"(r.q[2 * j + 1].x),
                     "=r"(r.q[2 * j + 1].y), "=r"(r.q[2 * j + 1].z), "=r"(r.q[2 * j + 1].w)
                   : "l"(qp + 32 * j));
    r.mult = FMT == COLI_FMT_FP8_B128 ? tt_f16x2_both(__ldg(srow + (kb >> 1)) * norm) : 0x3c003c00u /* 1.0 */;
  }
  return r;
}
__device__ __forceinline__ void tt_cvt_e4m3x4(uint32_t w, uint32_t &p0, uint32_t &p1) {
  asm("{ .reg .b16 h0, h1;\n"
      "  mov.b32 {h0, h1}, %2;\n"
      "  cvt.rn.f16x2.e4m3x2 %0, h0;\n"
      "  cvt.rn.f16x2.e4m3x2 %1, h1; }\n"
      : "=r"(p0), "=r"(p1)
      : "r"(w));
}
template <int FMT>
__device__ __forceinline__ void tt_convert8(const TtPacked8 &pk, uint32_t (&r)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 v = pk.q[j];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      tt_cvt_e4m3x4(w[i], r[8 * j + 2 * i], r[8 * j + 2 * i + 1]);
      if (FMT == COLI_FMT_FP8_B128) {
        r[8 * j + 2 * i] = tc_hmul2(r[8 * j + 2 * i], pk.mult);
        r[8 * j + 2 * i + 1] = tc_hmul2(r[8 * j + 2 * i + 1], pk.mult);
      }
    }
  }
}
// Largest scale of one row block over all k-tiles (every thread of a tile computes the same value).
__device__ __forceinline__ float tt_block_scale_max(const float *srow, int KT) {
  float m = 0.0f;
  for (int kt = 0; kt < KT; ++kt) m = fmaxf(m, __ldg(srow + kt));
  return m;
}

// GATED: the two weight tiles of a stage are gate and up of the same 128 features, result
// h = act(g, u).  Otherwise: two adjacent 128-feature tiles of the down projection, result y.
template <bool GATED, int FMT, int ACC>
__global__ void __launch_bounds__(TT_THREADS, 1) k_ffn_tct(const __grid_constant__ TtMaps maps, TcParams p) {
  constexpr int TT_A_STAGES = TtBudget<ACC>::A_STAGES, TT_A_COL0 = TtBudget<ACC>::A_COL0, TT_ACC_COLS = ACC;
  constexpr int TT_B_STAGES = TtBudget<ACC>::B_STAGES, TT_B_BYTES = TtBudget<ACC>::B_BYTES, TT_NBARS = TtBudget<ACC>::NBARS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TT_B_STAGES * TT_B_BYTES);
  // One "filled" and one "drained" barrier per stage of the token ring serve both operands: the
  // issuing threads then pay one wait and one commit per stage.  filled[s]: 8 producer warps + the
  // TMA thread's expect_tx arrival.  drained[s]: the commits of the two issuing threads.  The
  // weight ring is half as deep, so a producer about to fill stage `it` waits for drained of
  // stage it - TT_A_STAGES.
  const uint32_t full_s = smem_u32(bars), empty_s = smem_u32(bars + TT_B_STAGES);
  const uint32_t acc_full = smem_u32(bars + TT_NBARS - 2), acc_empty = smem_u32(bars + TT_NBARS - 1);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + TT_NBARS);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = GATED ? p.H : p.I, Oout = GATED ? p.I : p.H;
  const int Op = (Oout + 15) & ~15;
  const int KB = ((K + 127) >> 7) * 2;      // 64-wide k blocks, covering the zero-padded k tiles
  const int FT = GATED ? TC_BM : 2 * TC_BM;  // output features per tile
  const int n_ftiles = (Oout + FT - 1) / FT;
  const int n_work = *p.n_items * n_ftiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TT_B_STAGES; ++s) {
      mbar_init(full_s + 8 * s, 9);
      mbar_init(empty_s + 8 * s, 2);
    }
    mbar_init(acc_full, 2);
    mbar_init(acc_empty, TC_EPI_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA: token tiles ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < n_work && alive; w += gridDim.x) {
        const int item = w / n_ftiles;
        const int row0 = p.item_row0[item], nrows = p.item_nrows[item];
        const int N = (nrows + TC_BOXN - 1) / TC_BOXN * TC_BOXN;
        const CUtensorMap *tmap = &maps.m[N / TC_BOXN - 1];  // the map whose box is N rows
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % TT_B_STAGES, ph = (it / TT_B_STAGES) & 1u;
          if (!mbar_wait(empty_s + 8 * s, ph ^ 1u, abort_flag, p.status, TC_ERR_TMA_WAIT, 32)) {
            alive = false;
            break;
          }
          TT_TRACE(it, 6);
          const uint32_t dst = smem_u32(smem + s * TT_B_BYTES);
          mbar_expect_tx(full_s + 8 * s, (uint32_t)N * TC_BK * 2);
          tma_load_2d(dst, tmap, kb * TC_BK, row0, full_s + 8 * s);
        }
      }
      if (!alive) {
        // copies already issued still land in this CTA's shared memory: give them time before exit
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1 || warp == TT_MMA2_WARP) {
    // ---------------- MMA issue: warp 1 feeds accumulator 0, the extra warp accumulator 1 ----------------
    // One thread per accumulator keeps the order of its additions fixed, so results repeat bit for
    // bit from run to run.  (Two threads per accumulator taking alternate stages were measured: the
    // additions then interleave differently each run and the time per stage does not change.)
    if (lane == 0) {
      const uint32_t which = warp == 1 ? 0u : 1u;
      uint32_t tix = 0;
      bool alive = true;
      const uint64_t bdesc_ring = umma_smem_desc(smem_u32(smem));  // token-tile stage 0; stages are TT_B_BYTES apart
      const uint32_t acc = tmem_base + which * TT_ACC_COLS;
      const uint32_t a_ring = tmem_base + TT_A_COL0 + which * 32;
      // ring positions as counters: this thread's instruction stream is on the critical path of the
      // kernel, so no division or modulo per stage
      uint32_t sa = 0, sb = 0, phb = 0;
      for (int w = blockIdx.x; w < n_work && alive; w += gridDim.x, ++tix) {
        const int item = w / n_ftiles;
        const int nrows = p.item_nrows[item];
        const int N = (nrows + TC_BOXN - 1) / TC_BOXN * TC_BOXN;
        const uint32_t idesc = umma_idesc(N);
        if (!mbar_wait(acc_empty, (tix & 1u) ^ 1u, abort_flag, p.status, TC_ERR_MMA_WAIT, 1)) break;
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb) {
          if (which == 0) TT_TRACE(tix * KB + kb, 0);
          if (!mbar_wait(full_s + 8 * sb, phb, abort_flag, p.status, TC_ERR_MMA_WAIT, 1)) {
            alive = false;
            break;
          }
          if (which == 0) TT_TRACE(tix * KB + kb, 1);
          tc_fence_after();
          // both issuers commit: the rings are refilled once both accumulators have read them
          tt_issue_stage(acc, a_ring + sa * 64, bdesc_ring + (uint64_t)(sb * (TT_B_BYTES >> 4)), idesc, kb ? 1u : 0u, empty_s + 8 * sb);
          if (which == 0) TT_TRACE(tix * KB + kb, 2);
          if (++sa == TT_A_STAGES) sa = 0;
          if (++sb == TT_B_STAGES) {
            sb = 0;
            phb ^= 1u;
          }
        }
        if (alive) umma_commit(acc_full);
      }
    }
  } else if (warp < 2 + TC_EPI_WARPS) {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int lg = warp & 3;  // TMEM lane group this warp may read
    uint32_t tix = 0;
    for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++tix) {
      const int item = w / n_ftiles, ft = w % n_ftiles;
      const int seg = p.item_seg[item], row0 = p.item_row0[item], nrows = p.item_nrows[item];
      const int ex = p.seg_expert ? p.seg_expert[seg] : seg;
      const int N = (nrows + TC_BOXN - 1) / TC_BOXN * TC_BOXN;
      const int f = ft * FT + lg * 32 + lane;  // accumulator 0; accumulator 1 is feature f + 128 of down
      const WeightRef w0 = GATED ? p.gate[ex] : p.down[ex], w1 = GATED ? p.up[ex] : p.down[ex];
      float s0 = w0.g, s1 = w1.g;
      if (FMT == COLI_FMT_FP8_B128) {
        // undo the per-tile normalisation of the producers (both tiles of a stage are 128-row aligned)
        const int KT = KB >> 1;
        const int rb0 = (ft * FT) >> 7, rb1 = GATED ? rb0 : rb0 + 1, nrb = (Oout + 127) >> 7;
        s0 = tt_block_scale_max(reinterpret_cast<const float *>(w0.s) + (size_t)rb0 * KT, KT) * (1.0f / TT_FP8_HEADROOM);
        s1 = rb1 < nrb ? tt_block_scale_max(reinterpret_cast<const float *>(w1.s) + (size_t)rb1 * KT, KT) * (1.0f / TT_FP8_HEADROOM) : 0.0f;
      } else if (FMT == COLI_FMT_E4M3_ROW) {
        const int f1 = GATED ? f : f + TC_BM;
        s0 = f < Oout ? __ldg(reinterpret_cast<const float *>(w0.s) + f) : 0.0f;
        s1 = f1 < Oout ? __ldg(reinterpret_cast<const float *>(w1.s) + f1) : 0.0f;
      }
      bool ok = true;
      if (lg == 0 && lane == 0) TT_TRACE(240 + tix, 0);
      if (lane == 0) ok = mbar_wait(acc_full, tix & 1u, abort_flag, p.status, TC_ERR_EPI_WAIT, 256);
      if (lg == 0 && lane == 0) TT_TRACE(240 + tix, 1);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(lg * 32) << 16);
      for (int c0 = 0; c0 < N; c0 += 16) {
        uint32_t g[16], u[16];
#ifdef COLI_TT_TRACE
        if (GATED && blockIdx.x == 0 && lg == 0 && lane == 0 && tix == 2) g_tt_trace[(200 + c0 / 16) * 8 + 0] = clock64();
#endif
        tmem_ld16(tbase + c0, g);
        tmem_ld16(tbase + TT_ACC_COLS + c0, u);
        tmem_ld_wait();
#ifdef COLI_TT_TRACE
        if (GATED && blockIdx.x == 0 && lg == 0 && lane == 0 && tix == 2) g_tt_trace[(200 + c0 / 16) * 8 + 1] = clock64();
        if (GATED && blockIdx.x == 0 && lg == 0 && lane == 0 && tix == 2)
          g_tt_trace[(200 + c0 / 16) * 8 + 3] = clock64() + (long long)(g[0] == 0x12345u) + (long long)(u[15] == 0x12345u) + (long long)(g[7] == 0x12345u);
#endif
        // all 16 columns are computed first, branch-free, so that their dependent chains (scale,
        // exponential, reciprocal, two roundings) overlap; a branch per column would run them one
        // after the other.  Columns beyond the item's rows hold other rows' sums and are not stored.
        const int fq = f & ~3;  // first feature of this lane's quad
        const int cols_valid = nrows - c0;
        if (GATED) {
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            pk[j] = tc_pack_f16x2_via_bf16(coli_act_fast(__uint_as_float(g[2 * j]) * s0, __uint_as_float(u[2 * j]) * s1, p.act),
                                           coli_act_fast(__uint_as_float(g[2 * j + 1]) * s0, __uint_as_float(u[2 * j + 1]) * s1, p.act));
          tc_store_cols16(pk, p.h + (size_t)(row0 + c0) * Oout + fq, (size_t)Oout, cols_valid, fq < Oout, lane);
        } else {
          uint32_t pk0[8], pk1[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            pk0[j] = tc_pack_bf16x2(__uint_as_float(g[2 * j]) * s0, __uint_as_float(g[2 * j + 1]) * s0);
            pk1[j] = tc_pack_bf16x2(__uint_as_float(u[2 * j]) * s1, __uint_as_float(u[2 * j + 1]) * s1);
          }
          __nv_bfloat16 *yq = p.y + (size_t)(row0 + c0) * Oout + fq;
          tc_store_cols16(pk0, yq, (size_t)Oout, cols_valid, fq < Oout, lane);
          tc_store_cols16(pk1, yq + TC_BM, (size_t)Oout, cols_valid, fq + TC_BM < Oout, lane);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lg == 0 && lane == 0) TT_TRACE(240 + tix, 2);
      if (lane == 0) mbar_arrive(acc_empty);
    }
  } else {
    // ---------------- weight producers: HBM -> registers -> f16 -> tensor memory ----------------
    // four groups of four warps (128 lanes = 128 weight rows each): group g fills weight tile
    // (g & 1) of the stages whose index has parity (g >> 1)
    const int grp = (warp - 2 - TC_EPI_WARPS) >> 2;
    const int mtx = grp & 1, par = grp >> 1;
    const int quarter = warp & 3;  // TMEM lane quarter this warp may write
    const int row = quarter * 32 + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + TT_A_COL0 + mtx * 32;
    uint32_t it0 = 0;
    bool alive = true;
    // The conversion runs BEFORE the wait for the slot, so that only the store stands between the
    // slot's release and the barrier that hands it to the issuing threads.
    auto stage = [&](const auto &pk, uint32_t it) -> bool {
      uint32_t r[32];
      if constexpr (FMT == COLI_FMT_NVFP4)
        tt_convert(pk, r);
      else
        tt_convert8<FMT>(pk, r);
      const uint32_t sa = it % TT_A_STAGES;
      bool ok = true;
      if (mtx == 0 && quarter == 0 && lane == 0) TT_TRACE(it, 3);
      if (it >= (uint32_t)TT_A_STAGES) {  // the weight slot was last read by stage it - TT_A_STAGES
        const uint32_t u = it - TT_A_STAGES;
        if (lane == 0) ok = mbar_wait(empty_s + 8 * (u % TT_B_STAGES), (u / TT_B_STAGES) & 1u, abort_flag, p.status, TC_ERR_PROD_WAIT, 1);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) return false;
        tc_fence_after();
      }
      if (mtx == 0 && quarter == 0 && lane == 0) TT_TRACE(it, 4);
      tmem_st32(taddr + sa * 64, r);
      tmem_st_wait();
      if (mtx == 0 && quarter == 0 && lane == 0) TT_TRACE(it, 5);
      tc_fence_before();
      __syncwarp();
#ifdef COLI_TT_TRACE
      if (GATED && blockIdx.x == 0 && lane == 0 && it < 256u) atomicMax((unsigned long long *)&g_tt_trace[it * 8 + 7], (unsigned long long)clock64());
#endif
      if (lane == 0) mbar_arrive(full_s + 8 * (it % TT_B_STAGES));
      return true;
    };
    for (int w = blockIdx.x; w < n_work && alive; w += gridDim.x, it0 += KB) {
      const int item = w / n_ftiles, ft = w % n_ftiles;
      const int seg = p.item_seg[item];
      const int ex = p.seg_expert ? p.seg_expert[seg] : seg;
      const WeightRef wr = GATED ? (mtx ? p.up[ex] : p.gate[ex]) : p.down[ex];
      const int grow = GATED ? ft * TC_BM + row : ft * FT + mtx * TC_BM + row;
      // this group's k blocks of the tile: those whose global stage index it0 + kb has parity `par`
      const int kb0 = (int)((par - it0) & 1u);
      // two register sets alternate (kb, kb+2 | kb+4, kb+6 | ...): the bytes of the next two stages
      // of this group are in flight while one is converted, and no set is refilled before it is used
      if constexpr (FMT == COLI_FMT_NVFP4) {
        TtPacked pa, pb;
        pa.q0 = make_uint4(0, 0, 0, 0);
        pa.q1 = pa.q0;
        pa.sc = 0;
        pb = pa;
        if (kb0 < KB) pa = tt_load_packed(wr, Op, grow, kb0);
        if (kb0 + 2 < KB) pb = tt_load_packed(wr, Op, grow, kb0 + 2);
        for (int kb = kb0; kb < KB && alive; kb += 4) {
          alive = stage(pa, it0 + kb);
          if (kb + 4 < KB) pa = tt_load_packed(wr, Op, grow, kb + 4);
          if (alive && kb + 2 < KB) alive = stage(pb, it0 + kb + 2);
          if (kb + 6 < KB) pb = tt_load_packed(wr, Op, grow, kb + 6);
        }
      } else {
        const float *srow = nullptr;
        float norm = 0.0f;
        if (FMT == COLI_FMT_FP8_B128 && grow < Op) {
          const int KT = KB >> 1;
          srow = reinterpret_cast<const float *>(wr.s) + (size_t)(grow >> 7) * KT;
          // a row block whose scales are all zero (an all-zero or padded weight block: the encoder
          // writes scale = amax / 448 = 0) decodes to zeros, as code x 0 does in convert.rs:731-741
          const float mx = tt_block_scale_max(srow, KT);
          norm = mx > 0.0f ? TT_FP8_HEADROOM / mx : 0.0f;
        }
        TtPacked8 pa = tt_zero_packed8(), pb = pa;
        if (kb0 < KB) pa = tt_load_packed8<FMT>(wr, Op, grow, kb0, srow, norm);
        if (kb0 + 2 < KB) pb = tt_load_packed8<FMT>(wr, Op, grow, kb0 + 2, srow, norm);
        for (int kb = kb0; kb < KB && alive; kb += 4) {
          alive = stage(pa, it0 + kb);
          if (kb + 4 < KB) pa = tt_load_packed8<FMT>(wr, Op, grow, kb + 4, srow, norm);
          if (alive && kb + 2 < KB) alive = stage(pb, it0 + kb + 2);
          if (kb + 6 < KB) pb = tt_load_packed8<FMT>(wr, Op, grow, kb + 6, srow, norm);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

template <bool GATED, int FMT, int ACC>
static int launch_tct(const TcParams &p, const void *rows_base, int rows_cap, int sm_count, cudaStream_t st) {
  const size_t smem = (size_t)TtBudget<ACC>::B_STAGES * TtBudget<ACC>::B_BYTES + 1024 /*align*/ + 8 * TtBudget<ACC>::NBARS + 16 + 64;
  static ColiPerDeviceOnce attr_once;
  if (!coli_set_smem_limit(attr_once, k_ffn_tct<GATED, FMT, ACC>, smem, "tcgen05 kernel shared-memory attribute")) return 0;
  TtMaps maps;
  for (int j = 0; j < TCT_MAX_TOKENS / TC_BOXN; ++j)
    if (!make_rows_map(&maps.m[j], rows_base, rows_cap, GATED ? p.H : p.I, (j + 1) * TC_BOXN)) return 0;
  const int FT = GATED ? TC_BM : 2 * TC_BM;
  const int n_ftiles = ((GATED ? p.I : p.H) + FT - 1) / FT;
  const long max_work = (long)p.max_items * n_ftiles;
  const int grid = (int)(max_work < sm_count ? max_work : sm_count);
  if (grid <= 0) return 1;
  k_ffn_tct<GATED, FMT, ACC><<<grid, TT_THREADS, smem, st>>>(maps, p);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "tcgen05 expert ffn launch") ? 1 : 0;
}
template <bool GATED, int FMT>
static int launch_tct_acc(const TcParams &p, const void *rows_base, int rows_cap, int sm_count, cudaStream_t st) {
  if (p.tile_tokens == TCT_SHORT_TOKENS) return launch_tct<GATED, FMT, TCT_SHORT_TOKENS>(p, rows_base, rows_cap, sm_count, st);
  if (p.tile_tokens == TCT_MAX_TOKENS) return launch_tct<GATED, FMT, TCT_MAX_TOKENS>(p, rows_base, rows_cap, sm_count, st);
  coli_set_error("tcgen05 expert ffn: the work list must be cut with %d or %d rows per item, not %d", TCT_SHORT_TOKENS, TCT_MAX_TOKENS,
                 p.tile_tokens);
  return 0;
}
template <bool GATED>
static int launch_tct_fmt(const TcParams &p, const void *rows_base, int rows_cap, int sm_count, cudaStream_t st) {
  switch (p.fmt) {
    case COLI_FMT_NVFP4:
      return launch_tct_acc<GATED, COLI_FMT_NVFP4>(p, rows_base, rows_cap, sm_count, st);
    case COLI_FMT_FP8_B128:
      return launch_tct_acc<GATED, COLI_FMT_FP8_B128>(p, rows_base, rows_cap, sm_count, st);
    case COLI_FMT_E4M3_ROW:
      return launch_tct_acc<GATED, COLI_FMT_E4M3_ROW>(p, rows_base, rows_cap, sm_count, st);
  }
  coli_set_error("tcgen05 expert ffn: unsupported weight format %d", p.fmt);
  return 0;
}

int launch_gate_up_tct(const TcParams &p, const void *x_rows, int rows_cap, int sm_count, cudaStream_t st) {
  return launch_tct_fmt<true>(p, x_rows, rows_cap, sm_count, st);
}
int launch_down_tct(const TcParams &p, int rows_cap, int sm_count, cudaStream_t st) {
  return launch_tct_fmt<false>(p, p.h, rows_cap, sm_count, st);
}

}  // namespace colib
