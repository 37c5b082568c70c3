// Expert FFN for prefill-sized segments on the 5th-generation tensor cores.
//
// Formulation (operands swapped so that the ragged token count lands on the MMA's N, which
// has a granularity of 16, and the always-full feature axis on its M = 128):
//     D[feature, token] = W[feature, :] . X[token, :]^T          per expert segment
// * A operand (M side): a 128-feature x 64-k tile of the expert matrix.  The packed NVFP4
//   bytes are streamed from HBM with 128-bit loads by the producer warps, converted to f16 in
//   registers (cvt.rn.f16x2.e2m1x2 per byte, one half2 multiply by the block scale; exact:
//   E2M1 x ue4m3 has <= 6 significant bits) and stored to shared memory in the K-major
//   128-byte-swizzled layout the MMA reads.
// * B operand (N side): up to 256 token rows x 64 k of f16 activations, copied by TMA
//   (cp.async.bulk.tensor, 128-byte swizzle, no multicast) straight into the same layout.
// * tcgen05.mma kind::f16 (f16 x f16 -> f32), issued by one thread, accumulates in TMEM; the
//   gate and the up projection of the same 128 features use two accumulators fed from the same
//   token tile, so SiLU(g)*u is formed in the epilogue registers and only h is written.  The 512
//   TMEM columns hold two such accumulator pairs when a tile has at most 128 tokens, so the
//   epilogue of one tile drains while the MMAs of the next one run; a tile of up to 256 tokens
//   takes all 512 columns.
// * 4 epilogue warps read TMEM with tcgen05.ld (one lane = one feature), apply the per-tensor
//   scale, the activation, and store h (f16 holding the bf16-rounded value) or y (bf16).
// Roles are warp-specialised and synchronise through mbarriers only; the kernel is persistent
// (one CTA per SM walks the device-built work list).  Every barrier wait is bounded: on a
// time-out the CTA raises a status word, stops issuing work, waits for its own copies and frees
// its TMEM before returning, so a logic error can end as an error code but not as a hung GPU.
//
// This replaces the reference's dequant-to-half + wmma kernels nvfp4_matmul / nvfp4_gate_up
// (crates/colibri-backend/cuda/backend_cuda.cu:1355-1430) and its separate silu_mul launch
// (backend_cuda.cu:3785-3787).
#include "tc_common.cuh"

namespace colib {

// weight-producer warps: every thread decodes one 16-byte chunk (32 weights) of one matrix per
// stage; 256 threads cover a 128-row tile, so the gated kernel runs 16 producer warps, the down kernel 8
template <bool GATED>
struct TcCfg {
  static constexpr int PROD_WARPS = 16;
  static constexpr int THREADS = 32 * (2 + TC_EPI_WARPS + PROD_WARPS);
};
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;                        // 16 KiB
constexpr int TC_B_BYTES = TC_MAX_TOKENS * TC_BK * 2;                // 32 KiB
struct TcPacked {
  uint4 q;      // 32 weights of one row
  uint32_t sc;  // their two block-scale bytes
};
// What one producer thread needs of one k-tile (128 k) of one row: its 16-byte chunk of each
// 64-k half and the row's eight block-scale bytes.
struct TcPackedKT {
  uint4 q0, q1;
  uint2 sc;
};
__device__ __forceinline__ TcPackedKT tc_load_kt(const WeightRef &w, int Op, int row, int kt, int c) {
  TcPackedKT r;
  r.q0 = make_uint4(0, 0, 0, 0);
  r.q1 = make_uint4(0, 0, 0, 0);
  r.sc = make_uint2(0, 0);
  if (row < Op) {
    const size_t base = (size_t)kt * Op + row;
    const uint8_t *qp = w.q + base * 64 + c * 16;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.q0.x), "=r"(r.q0.y), "=r"(r.q0.z), "=r"(r.q0.w)
                 : "l"(qp));
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.q1.x), "=r"(r.q1.y), "=r"(r.q1.z), "=r"(r.q1.w)
                 : "l"(qp + 32));
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.sc.x), "=r"(r.sc.y) : "l"(w.s + base * 8));
  }
  return r;
}
__device__ __forceinline__ TcPacked tc_half(const TcPackedKT &t, int half, int c) {
  TcPacked r;
  r.q = half ? t.q1 : t.q0;
  r.sc = ((half ? t.sc.y : t.sc.x) >> (16 * c)) & 0xffffu;
  return r;
}
// Decode 32 weights and store them as chunks 4c..4c+3 of row `row` of a swizzled 128x64 tile.
__device__ __forceinline__ void tc_store_tile(uint8_t *tile, int row, int c, const TcPacked &pk) {
  uint32_t m0, m1;
  tc_scales(pk.sc, m0, m1);
  uint8_t *rbase = tile + (row >> 3) * 1024 + (row & 7) * 128;
  const int sw = row & 7;
  *reinterpret_cast<uint4 *>(rbase + (((c * 4 + 0) ^ sw) << 4)) = tc_dequant_word(pk.q.x, m0);
  *reinterpret_cast<uint4 *>(rbase + (((c * 4 + 1) ^ sw) << 4)) = tc_dequant_word(pk.q.y, m0);
  *reinterpret_cast<uint4 *>(rbase + (((c * 4 + 2) ^ sw) << 4)) = tc_dequant_word(pk.q.z, m1);
  *reinterpret_cast<uint4 *>(rbase + (((c * 4 + 3) ^ sw) << 4)) = tc_dequant_word(pk.q.w, m1);
}

// The token tile of a stage arrives as ONE box of N rows (the copy engine of an SM takes about 64
// cycles per box plus 4 per 128-byte row, so eight 32-row boxes per 256-token stage cost a third
// more than one): one tensor map per box height.
struct TcMaps {
  CUtensorMap m[TC_MAX_TOKENS / TC_BOXN];
};
template <bool GATED>
__global__ void __launch_bounds__(TcCfg<GATED>::THREADS, 1) k_ffn_tc(const __grid_constant__ TcMaps maps, TcParams p) {
  constexpr int MATS = 2;    // gate + up of the same 128 features, or two adjacent 128-feature tiles of down
  constexpr int STAGES = 3;
  constexpr int STAGE_BYTES = MATS * TC_A_BYTES + TC_B_BYTES;
  constexpr int TC_PROD_WARPS = TcCfg<GATED>::PROD_WARPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
  const uint32_t full_a = smem_u32(bars), full_b = smem_u32(bars + STAGES), empty = smem_u32(bars + 2 * STAGES);
  // two accumulator buffers (each: two accumulators of <= 128 token columns); a tile of more than
  // 128 tokens takes both
  const uint32_t acc_full = smem_u32(bars + 3 * STAGES), acc_empty = smem_u32(bars + 3 * STAGES + 2);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *prod_ok = reinterpret_cast<volatile int *>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = GATED ? p.H : p.I, Oout = GATED ? p.I : p.H;
  const int Op = (Oout + 15) & ~15;
  const int KB = ((K + 127) >> 7) * 2;  // 64-wide k blocks, covering the zero-padded k tiles
  const int FT = GATED ? TC_BM : 2 * TC_BM;  // output features per tile
  const int n_ftiles = (Oout + FT - 1) / FT;
  const int n_work = *p.n_items * n_ftiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_a + 8 * s, TC_PROD_WARPS);
      mbar_init(full_b + 8 * s, 1);
      mbar_init(empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + 8 * b, 1);
      mbar_init(acc_empty + 8 * b, TC_EPI_WARPS);
    }
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
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag, p.status, TC_ERR_TMA_WAIT, 64)) {
            alive = false;
            break;
          }
          const uint32_t dst = smem_u32(smem + s * STAGE_BYTES + MATS * TC_A_BYTES);
          mbar_expect_tx(full_b + 8 * s, (uint32_t)N * TC_BK * 2);
          tma_load_2d(dst, tmap, kb * TC_BK, row0, full_b + 8 * s);
        }
      }
      if (!alive) {
        // copies already issued still land in this CTA's shared memory: give them time before exit
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issue ----------------
    // (one issuing thread: with both operands in shared memory this kernel is bound by that
    // memory's bandwidth, and a second issuing thread, which helps expert_tc_tmem.cu, measured
    // no faster here)
    if (lane == 0) {
      uint32_t it = 0, small_units = 0;
      uint32_t waits[2] = {0u, 0u};  // completed waits on each buffer's "drained" barrier
      bool alive = true;
      for (int w = blockIdx.x; w < n_work && alive; w += gridDim.x) {
        const int item = w / n_ftiles;
        const int nrows = p.item_nrows[item];
        const int N = (nrows + TC_BOXN - 1) / TC_BOXN * TC_BOXN;
        const uint32_t idesc = umma_idesc(N);
        // Tiles of <= 128 tokens alternate between the two accumulator buffers, so the epilogue
        // of one tile drains while the next tile's MMAs run; a wider tile needs both buffers.
        const bool big = N > TC_MAX_TOKENS / 2;
        const uint32_t buf = big ? 0u : (small_units++ & 1u);
        bool ok = true;
        for (uint32_t b = big ? 0u : buf; ok && b <= (big ? 1u : buf); ++b) {
          ok = mbar_wait(acc_empty + 8 * b, (waits[b] & 1u) ^ 1u, abort_flag, p.status, TC_ERR_MMA_WAIT, 1);
          waits[b]++;
        }
        if (!ok) break;
        const uint32_t acc0 = tmem_base + buf * TC_MAX_TOKENS;
        const uint32_t acc1 = acc0 + (big ? TC_MAX_TOKENS : TC_MAX_TOKENS / 2);
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
          if (!mbar_wait(full_a + 8 * s, ph, abort_flag, p.status, TC_ERR_MMA_WAIT, 1) ||
              !mbar_wait(full_b + 8 * s, ph, abort_flag, p.status, TC_ERR_MMA_WAIT, 1)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint32_t a0 = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b0 = a0 + MATS * TC_A_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
            const uint64_t bd = umma_smem_desc(b0 + k4 * 32);
            const uint32_t acc = (kb | k4) ? 1u : 0u;
            umma_f16(acc0, umma_smem_desc(a0 + k4 * 32), bd, idesc, acc);
            umma_f16(acc1, umma_smem_desc(a0 + TC_A_BYTES + k4 * 32), bd, idesc, acc);
          }
          umma_commit(empty + 8 * s);  // the stage may be refilled once these MMAs have read it
        }
        if (alive) umma_commit(acc_full + 8 * buf);
      }
    }
  } else if (warp < 2 + TC_EPI_WARPS) {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int lg = warp & 3;  // TMEM lane group this warp may read
    uint32_t small_units = 0;
    uint32_t fills[2] = {0u, 0u};  // completed waits on each buffer's "filled" barrier
    for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
      const int item = w / n_ftiles, ft = w % n_ftiles;
      const int seg = p.item_seg[item], row0 = p.item_row0[item], nrows = p.item_nrows[item];
      const int ex = p.seg_expert ? p.seg_expert[seg] : seg;
      const int N = (nrows + TC_BOXN - 1) / TC_BOXN * TC_BOXN;
      const float s0 = GATED ? p.gate[ex].g : p.down[ex].g;
      const float s1 = GATED ? p.up[ex].g : p.down[ex].g;
      const bool big = N > TC_MAX_TOKENS / 2;  // same buffer walk as the MMA warp
      const uint32_t buf = big ? 0u : (small_units++ & 1u);
      bool ok = true;
      if (lane == 0) ok = mbar_wait(acc_full + 8 * buf, fills[buf] & 1u, abort_flag, p.status, TC_ERR_EPI_WAIT, 256);
      fills[buf]++;
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const int f = ft * FT + lg * 32 + lane;  // accumulator 0; accumulator 1 is feature f + 128 of down
      const uint32_t tbase = tmem_base + buf * TC_MAX_TOKENS + ((uint32_t)(lg * 32) << 16);
      const uint32_t acc1_off = big ? TC_MAX_TOKENS : TC_MAX_TOKENS / 2;
      for (int c0 = 0; c0 < N; c0 += 16) {
        uint32_t g[16], u[16];
        tmem_ld16(tbase + c0, g);
        tmem_ld16(tbase + acc1_off + c0, u);
        tmem_ld_wait();
        // all 16 columns are computed first, branch-free, so that their dependent chains (scale,
        // exponential, reciprocal, two roundings) overlap; a branch per column would run them one
        // after the other.  Columns beyond the item's rows hold zeros and are simply not stored.
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
      if (lane == 0) {
        mbar_arrive(acc_empty + 8 * buf);
        if (big) mbar_arrive(acc_empty + 8);
      }
    }
  } else {
    // ---------------- weight producers: HBM -> registers -> f16 -> swizzled shared memory ----------------
    // thread -> (matrix, row, 16-byte chunk): 256 threads cover one 128-row tile of one matrix
    const int pt = threadIdx.x - 32 * (2 + TC_EPI_WARPS);
    const int mtx = pt >> 8, row = (pt & 255) >> 1, c = pt & 1;
    uint32_t it = 0;
    bool alive = true;
    for (int w = blockIdx.x; w < n_work && alive; w += gridDim.x) {
      const int item = w / n_ftiles, ft = w % n_ftiles;
      const int seg = p.item_seg[item];
      const int ex = p.seg_expert ? p.seg_expert[seg] : seg;
      const WeightRef wr = GATED ? (mtx ? p.up[ex] : p.gate[ex]) : p.down[ex];
      const int grow = GATED ? ft * TC_BM + row : ft * FT + mtx * TC_BM + row;
      const int KT = KB >> 1;
      // Register ring of depth 4: while k-tile kt is decoded, the packed bytes of kt+1..kt+3 are
      // in flight.  The loop is unrolled by the ring depth so that every slot is a fixed set of
      // registers; rotating slots with moves would stall on the youngest load at every step.
      TcPackedKT ring[4];
#pragma unroll
      for (int j = 0; j < 3; ++j) {
        ring[j].q0 = make_uint4(0, 0, 0, 0);
        ring[j].q1 = ring[j].q0;
        ring[j].sc = make_uint2(0, 0);
        if (j < KT) ring[j] = tc_load_kt(wr, Op, grow, j, c);
      }
      for (int kt0 = 0; kt0 < KT && alive; kt0 += 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int kt = kt0 + j;
          if (kt >= KT || !alive) break;
          if (kt + 3 < KT) ring[(j + 3) & 3] = tc_load_kt(wr, Op, grow, kt + 3, c);
#pragma unroll
          for (int half = 0; half < 2; ++half, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
            bool ok = true;
            // One thread polls the mbarrier for all producer warps and releases them through a
            // hardware named barrier: many warps polling one mbarrier word serialise in the
            // shared-memory pipe and each poll then costs hundreds of cycles.
            if (pt == 0) *prod_ok = mbar_wait(empty + 8 * s, ph ^ 1u, abort_flag, p.status, TC_ERR_PROD_WAIT, 1) ? 1 : 0;
            asm volatile("bar.sync 1, %0;" ::"r"(TC_PROD_WARPS * 32) : "memory");
            ok = *prod_ok != 0;
            if (!ok) {
              alive = false;
              break;
            }
            tc_store_tile(smem + s * STAGE_BYTES + mtx * TC_A_BYTES, row, c, tc_half(ring[j], half, c));
            fence_proxy_async_smem();  // make these generic-proxy stores visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(full_a + 8 * s);
          }
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

template <bool GATED>
static int launch_tc(const TcParams &p, const void *rows_base, int rows_cap, int sm_count, cudaStream_t st) {
  constexpr int MATS = 2;
  constexpr int STAGES = 3;
  const size_t smem = (size_t)STAGES * (MATS * TC_A_BYTES + TC_B_BYTES) + 1024 /*align*/ + 8 * (3 * STAGES + 4) + 16 + 64;
  static ColiPerDeviceOnce attr_once;
  if (!coli_set_smem_limit(attr_once, k_ffn_tc<GATED>, smem, "tcgen05 kernel shared-memory attribute")) return 0;
  TcMaps maps;
  for (int j = 0; j < TC_MAX_TOKENS / TC_BOXN; ++j)
    if (!make_rows_map(&maps.m[j], rows_base, rows_cap, GATED ? p.H : p.I, (j + 1) * TC_BOXN)) return 0;
  const int FT = GATED ? TC_BM : 2 * TC_BM;
  const int n_ftiles = ((GATED ? p.I : p.H) + FT - 1) / FT;
  const long max_work = (long)p.max_items * n_ftiles;
  const int grid = (int)(max_work < sm_count ? max_work : sm_count);
  if (grid <= 0) return 1;
  k_ffn_tc<GATED><<<grid, TcCfg<GATED>::THREADS, smem, st>>>(maps, p);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "tcgen05 expert ffn launch") ? 1 : 0;
}

int launch_gate_up_tc(const TcParams &p, const void *x_rows, int rows_cap, int sm_count, cudaStream_t st) {
  return launch_tc<true>(p, x_rows, rows_cap, sm_count, st);
}
int launch_down_tc(const TcParams &p, int rows_cap, int sm_count, cudaStream_t st) {
  return launch_tc<false>(p, p.h, rows_cap, sm_count, st);
}

}  // namespace colib
