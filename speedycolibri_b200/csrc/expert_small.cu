// Expert FFN for decode-sized segments: a weight-streaming dequant-GEMV/GEMM in which every
// weight byte is read from HBM exactly once per work item with 128-bit loads, converted to
// f16 in registers (one hardware cvt per pair of FP4 or FP8 codes, one half2 multiply by the
// block scale for NVFP4), and contracted against up to 32 token rows with warp-level f16 MMA
// (m16n8k16, f32 accumulate).  The path is HBM-bound: the MMA only takes the multiply-adds
// off the CUDA cores so that the decode arithmetic (about one operation per FP4 weight) is
// all the SM has to issue per byte streamed.
//
// It replaces the reference's per-expert launch trios nvfp4_gemv / nvfp4_wsmm / fp8a16_gemv
// (crates/colibri-backend/cuda/backend_cuda.cu:707-1110,1436-1510,468-496, dispatched from
// 4738-4783) with two launches for ALL experts of a layer: gate+up with SiLU*mul fused
// (the reference runs `silu_mul` as a separate launch, backend_cuda.cu:3785-3787), then down.
//
// Numerics (W4A16 as in crates/colibri-engine/src/linear.rs:110-133): activations are the bf16
// values held in f16 (exact in [2^-14, 65504]), a decoded weight E2M1*ue4m3 has at most 6
// significant bits and is exact in f16, so
// each product is exact and only the f32 summation order differs from the CPU sum.  The
// per-tensor scale is applied once per output, as the reference does.  The intermediate
// h = silu(g)*u is rounded to bf16 (then held in f16) before the down projection.
//
// Work decomposition: grid = (row tiles of 16 outputs, work items); an item is at most 8*NB
// consecutive rows of one expert segment.  The W warps of a CTA split the K axis (k-tile kt
// goes to warp kt % W) so that even a single-token decode exposes thousands of warps, and
// reduce through shared memory.
#include "internal.cuh"

namespace colib {

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hmul2_f16(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Two bytes of a NVFP4 word (each byte = two consecutive k, low nibble first) -> two f16x2.
// HI selects bytes 2,3 of the word, otherwise bytes 0,1.
template <bool HI>
__device__ __forceinline__ void cvt_e2m1x4(uint32_t w, uint32_t &p0, uint32_t &p1) {
  if (HI)
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        "  mov.b32 {b0, b1, b2, b3}, %2;\n"
        "  cvt.rn.f16x2.e2m1x2 %0, b2;\n"
        "  cvt.rn.f16x2.e2m1x2 %1, b3; }\n"
        : "=r"(p0), "=r"(p1)
        : "r"(w));
  else
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        "  mov.b32 {b0, b1, b2, b3}, %2;\n"
        "  cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "  cvt.rn.f16x2.e2m1x2 %1, b1; }\n"
        : "=r"(p0), "=r"(p1)
        : "r"(w));
}
// One FP8 word (four consecutive k) -> two f16x2; also used for a pair of ue4m3 block scales.
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t &p0, uint32_t &p1) {
  asm("{ .reg .b16 h0, h1;\n"
      "  mov.b32 {h0, h1}, %2;\n"
      "  cvt.rn.f16x2.e4m3x2 %0, h0;\n"
      "  cvt.rn.f16x2.e4m3x2 %1, h1; }\n"
      : "=r"(p0), "=r"(p1)
      : "r"(w));
}

template <int FMT>
struct AFrag {
  // raw bytes of rows g and g+8 of one 16-row tile for one k-tile, as loaded by this lane
  uint4 lo[FMT == COLI_FMT_NVFP4 ? 1 : 2], hi[FMT == COLI_FMT_NVFP4 ? 1 : 2];
  uint32_t sc;  // NVFP4: two scale bytes of row g (low 16 bits) and of row g+8 (high 16 bits)
};

template <int FMT>
__device__ __forceinline__ void load_a(AFrag<FMT> &f, const WeightRef &w, int Op, int r0, int kt, int lane) {
  if (FMT == COLI_FMT_NVFP4) {
    const uint8_t *slab = w.q + ((size_t)kt * Op + r0) * 64;
    f.lo[0] = ldg_nc_v4(slab + lane * 16);
    f.hi[0] = ldg_nc_v4(slab + 512 + lane * 16);
    const uint8_t *ss = w.s + ((size_t)kt * Op + r0) * 8;
    const uint32_t s0 = *reinterpret_cast<const uint16_t *>(ss + lane * 2);
    const uint32_t s1 = *reinterpret_cast<const uint16_t *>(ss + 64 + lane * 2);
    f.sc = s0 | (s1 << 16);
  } else {
    const uint8_t *slab = w.q + ((size_t)kt * Op + r0) * 128;
    f.lo[0] = ldg_nc_v4(slab + lane * 32);
    f.lo[1] = ldg_nc_v4(slab + lane * 32 + 16);
    f.hi[0] = ldg_nc_v4(slab + 1024 + lane * 32);
    f.hi[1] = ldg_nc_v4(slab + 1024 + lane * 32 + 16);
    f.sc = 0;
  }
}

// Per k-tile: the lane's four block scales (rows g and g+8, two 16-k blocks each) as f16x2
// with the scale in both halves.
struct AScale {
  uint32_t lo[2], hi[2];
};
template <int FMT>
__device__ __forceinline__ AScale decode_scales(const AFrag<FMT> &f) {
  AScale r;
  if (FMT == COLI_FMT_NVFP4) {
    uint32_t sl, sh;
    cvt_e4m3x4(f.sc, sl, sh);  // (s_blk0, s_blk1) of row g; of row g+8
    r.lo[0] = __byte_perm(sl, sl, 0x1010);
    r.lo[1] = __byte_perm(sl, sl, 0x3232);
    r.hi[0] = __byte_perm(sh, sh, 0x1010);
    r.hi[1] = __byte_perm(sh, sh, 0x3232);
  } else {
    r.lo[0] = r.lo[1] = r.hi[0] = r.hi[1] = 0;
  }
  return r;
}

// Decode the fragment of MMA step m (0..7) of a k-tile: a[0],a[2] = row g pairs, a[1],a[3] = row g+8.
template <int FMT>
__device__ __forceinline__ void decode_a(const AFrag<FMT> &f, const AScale &sc, int m, uint32_t (&a)[4]) {
  if (FMT == COLI_FMT_NVFP4) {
    const uint32_t wl = (&f.lo[0].x)[m >> 1], wh = (&f.hi[0].x)[m >> 1];
    uint32_t l0, l1, h0, h1;
    if (m & 1) {
      cvt_e2m1x4<true>(wl, l0, l1);
      cvt_e2m1x4<true>(wh, h0, h1);
    } else {
      cvt_e2m1x4<false>(wl, l0, l1);
      cvt_e2m1x4<false>(wh, h0, h1);
    }
    const uint32_t ml = sc.lo[m >> 2], mh = sc.hi[m >> 2];
    a[0] = hmul2_f16(l0, ml);
    a[2] = hmul2_f16(l1, ml);
    a[1] = hmul2_f16(h0, mh);
    a[3] = hmul2_f16(h1, mh);
  } else {
    const uint32_t wl = (&f.lo[m >> 2].x)[m & 3], wh = (&f.hi[m >> 2].x)[m & 3];
    cvt_e4m3x4(wl, a[0], a[2]);
    cvt_e4m3x4(wh, a[1], a[3]);
  }
}

// GATED: two matrices (gate, up) -> h = silu(g)*u;  otherwise one matrix (down) -> y.
// SPLITK: grid = (row tiles, work items); the W warps of a CTA share one 16-row tile and split
// the k-tiles (few work items: a single-token decode).  Otherwise the grid is one-dimensional
// and sized to what is resident at once; every warp walks (item, row tile) tasks with a stride,
// owns its tile over all of K and needs no cross-warp reduction.
template <int FMT, int NB, bool GATED, bool SPLITK>
__global__ void __launch_bounds__(SPLITK ? 256 : 64, SPLITK                  ? 1
                                                      : FMT == COLI_FMT_NVFP4 ? (NB == 1 ? 10 : NB == 2 ? 8 : 4)
                                                                              : (NB == 1 ? 7 : NB == 2 ? 5 : 4))
    k_ffn_mm(FfnParams p) {
  constexpr int MATS = GATED ? 2 : 1;
  // weight ring depth (k-tiles) and token-fragment ring depth (quarter k-tiles)
  constexpr int D = 2;
  constexpr int R = NB <= 2 ? 4 : 2;
  constexpr int PF = R - 1;
  extern __shared__ __align__(16) float red[];  // [W][MATS*NB*4][32]
  coli_grid_dependency_sync();
  const int n_items = *p.n_items;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = GATED ? p.H : p.I;     // contraction length
  const int Oout = GATED ? p.I : p.H;  // output features
  const int Kp = (K + 127) & ~127, KT = Kp >> 7, Op = (Oout + 15) & ~15;
  const int row_tiles = Op >> 4;
  const __half *src = GATED ? p.x : p.h;

  int task = SPLITK ? (int)blockIdx.y * row_tiles + (int)blockIdx.x : (int)blockIdx.x * W + warp;
  const int task_stride = SPLITK ? 0x40000000 : (int)gridDim.x * W;
  const int n_tasks = n_items * row_tiles;
  for (; task < n_tasks; task += task_stride) {
    const int item = task / row_tiles, r0 = (task - item * row_tiles) * 16;
    const int seg = p.item_seg[item], row0 = p.item_row0[item], nrows = p.item_nrows[item];
    const int ex = p.seg_expert ? p.seg_expert[seg] : seg;
    const WeightRef w0 = GATED ? p.gate[ex] : p.down[ex];
    const WeightRef w1 = GATED ? p.up[ex] : w0;

    // source row of token column g of each 8-token block (nullptr = column beyond the item)
    const __half *xrow[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int r = 8 * j + g;
      if (r < nrows) {
        const int row = row0 + r;
        const size_t sidx = (GATED && p.row_token) ? (size_t)p.row_token[row] : (size_t)row;
        xrow[j] = src + sidx * K;
      } else {
        xrow[j] = nullptr;
      }
    }

    float acc[MATS][NB][4];
#pragma unroll
    for (int mtx = 0; mtx < MATS; ++mtx)
#pragma unroll
      for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mtx][j][c] = 0.0f;

    const int kstep = SPLITK ? W : 1;
    const int kt_first = SPLITK ? warp : 0;

    // token fragments: lane (g,t) reads x[token g][kt*128 + 32t + 8c .. +7] (16 bytes, two MMA
    // steps) for quarter c of k-tile kt
    auto load_x = [&](uint4 (&dst)[NB], int kt, int c) {
      const int k0 = kt * 128 + t * 32 + c * 8;
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        dst[j] = make_uint4(0, 0, 0, 0);
        if (xrow[j] != nullptr && kt < KT && k0 + 8 <= K) dst[j] = *reinterpret_cast<const uint4 *>(xrow[j] + k0);
      }
    };

    // Register rings, both unrolled so that every slot is a fixed set of registers (rotating
    // slots with copies would make each iteration wait for the youngest load): packed weight
    // fragments D k-tiles deep, token fragments R quarter-k-tiles deep.
    AFrag<FMT> ring[D][MATS];
    uint4 xq[R][NB];
#pragma unroll
    for (int j = 0; j < D - 1; ++j) {
      const int ktl = kt_first + j * kstep;
      if (ktl < KT) {
        load_a<FMT>(ring[j][0], w0, Op, r0, ktl, lane);
        if (GATED) load_a<FMT>(ring[j][MATS - 1], w1, Op, r0, ktl, lane);
      }
    }
#pragma unroll
    for (int f = 0; f < PF; ++f) load_x(xq[f % R], kt_first + (f / 4) * kstep, f % 4);

    for (int kt0 = kt_first; kt0 < KT; kt0 += D * kstep) {
#pragma unroll
      for (int slot = 0; slot < D; ++slot) {
        const int kt = kt0 + slot * kstep;
        if (kt >= KT) break;
        const int ktn = kt + (D - 1) * kstep;
        if (ktn < KT) {
          load_a<FMT>(ring[(slot + D - 1) % D][0], w0, Op, r0, ktn, lane);
          if (GATED) load_a<FMT>(ring[(slot + D - 1) % D][MATS - 1], w1, Op, r0, ktn, lane);
        }
        AScale asc[MATS];
#pragma unroll
        for (int mtx = 0; mtx < MATS; ++mtx) asc[mtx] = decode_scales<FMT>(ring[slot][mtx]);
        float part[MATS][NB][4];
        if (FMT == COLI_FMT_FP8_B128) {
#pragma unroll
          for (int mtx = 0; mtx < MATS; ++mtx)
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
              for (int c = 0; c < 4; ++c) part[mtx][j][c] = 0.0f;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int f = slot * 4 + c;  // position in the unrolled body; 4*D is a multiple of R
          load_x(xq[(f + PF) % R], kt + ((c + PF) / 4) * kstep, (c + PF) % 4);
          const uint4(&xb)[NB] = xq[f % R];
#pragma unroll
          for (int mm = 0; mm < 2; ++mm) {
            const int m = 2 * c + mm;
#pragma unroll
            for (int mtx = 0; mtx < MATS; ++mtx) {
              uint32_t a[4];
              decode_a<FMT>(ring[slot][mtx], asc[mtx], m, a);
#pragma unroll
              for (int j = 0; j < NB; ++j) {
                const uint32_t b0 = mm ? xb[j].z : xb[j].x, b1 = mm ? xb[j].w : xb[j].y;
                if (FMT == COLI_FMT_FP8_B128)
                  mma_f16_16816(part[mtx][j], a, b0, b1);
                else
                  mma_f16_16816(acc[mtx][j], a, b0, b1);
              }
            }
          }
        }
        if (FMT == COLI_FMT_FP8_B128) {
          // one f32 scale per (128-row block, k-tile): convert.rs:731-741
#pragma unroll
          for (int mtx = 0; mtx < MATS; ++mtx) {
            const float *sc = reinterpret_cast<const float *>(mtx == 0 ? w0.s : w1.s);
            const float s = sc[(size_t)(r0 >> 7) * KT + kt];
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
              for (int c = 0; c < 4; ++c) acc[mtx][j][c] = fmaf(s, part[mtx][j][c], acc[mtx][j][c]);
          }
        }
      }
    }

    // epilogue of one 8-token block given its reduced accumulators
    auto emit = [&](int j, const float(&v)[MATS][4]) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int orow = r0 + g + ((c & 2) ? 8 : 0);  // output feature
        const int col = 8 * j + 2 * t + (c & 1);      // token within the item
        if (orow >= Oout || col >= nrows) continue;
        float s0 = 1.0f, s1 = 1.0f;
        if (FMT == COLI_FMT_NVFP4) {
          s0 = w0.g;
          s1 = w1.g;
        } else if (FMT == COLI_FMT_E4M3_ROW) {
          s0 = reinterpret_cast<const float *>(w0.s)[orow];
          s1 = reinterpret_cast<const float *>(w1.s)[orow];
        }
        const size_t row = (size_t)(row0 + col);
        if (GATED) {
          const float gv = v[0][c] * s0, uv = v[MATS - 1][c] * s1;
          const float hv = coli_act_fast(gv, uv, p.act);
          p.h[row * p.I + orow] = coli_f32_to_f16_via_bf16(hv);
        } else {
          if (p.relu2_out) {
            const float r = fmaxf(v[0][c] * s0, 0.0f);
            p.relu2_out[row * p.H + orow] = coli_f32_to_f16_via_bf16(r * r);
          } else if (p.y32) {
            p.y32[row * p.H + orow] = v[0][c] * s0;
          } else {
            p.y[row * p.H + orow] = __float2bfloat16_rn(v[0][c] * s0);
          }
        }
      }
    };

    if (!SPLITK) {
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        float v[MATS][4];
#pragma unroll
        for (int mtx = 0; mtx < MATS; ++mtx)
#pragma unroll
          for (int c = 0; c < 4; ++c) v[mtx][c] = acc[mtx][j][c];
        emit(j, v);
      }
      continue;
    }

    // cross-warp (split-K) reduction; every warp of the CTA is on the same task
    constexpr int NV = MATS * NB * 4;
#pragma unroll
    for (int mtx = 0; mtx < MATS; ++mtx)
#pragma unroll
      for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[((size_t)warp * NV + (mtx * NB + j) * 4 + c) * 32 + lane] = acc[mtx][j][c];
    __syncthreads();

    for (int j = warp; j < NB; j += W) {
      float v[MATS][4];
#pragma unroll
      for (int mtx = 0; mtx < MATS; ++mtx)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float s = 0.0f;
          for (int w = 0; w < W; ++w) s += red[((size_t)w * NV + (mtx * NB + j) * 4 + c) * 32 + lane];
          v[mtx][c] = s;
        }
      emit(j, v);
    }
  }
}


static int pick_w(int KT) { return KT >= 8 ? 8 : KT >= 4 ? 4 : KT >= 2 ? 2 : 1; }

// Split K across the warps of a CTA only when there are too few (item, row tile) tasks to fill
// the SMs with one warp each; `p.items_expected` is a host-side estimate from shapes alone.
template <int FMT, int NB>
static int launch_one(const FfnParams &p, bool gated, cudaStream_t st) {
  const int K = gated ? p.H : p.I, O = gated ? p.I : p.H;
  const int KT = (K + 127) / 128, row_tiles = (O + 15) / 16;
  const long tasks = (long)row_tiles * (p.items_expected > 0 ? p.items_expected : 1);
  const bool splitk = tasks < 148L * 12;
  if (splitk) {
    const int W = pick_w(KT);
    dim3 grid(row_tiles, p.max_items);
    const size_t sm = (size_t)W * (gated ? 2 : 1) * NB * 4 * 32 * sizeof(float);
    const cudaError_t e = gated ? launch_dependent(k_ffn_mm<FMT, NB, true, true>, grid, dim3(W * 32), sm, st, p)
                                : launch_dependent(k_ffn_mm<FMT, NB, false, true>, grid, dim3(W * 32), sm, st, p);
    coli_count_launch(1);
    return coli_cuda_check(e, "expert ffn launch") ? 1 : 0;
  } else {
    // two warps per CTA keep the per-SM share of tasks even; the grid covers what fits at once
    constexpr int W = 2;
    // resident CTAs per kernel variant and device ordinal (an occupancy figure belongs to one device)
    static int resident_tab[2][32];
    int dev = 0;
    if (!coli_cuda_check(cudaGetDevice(&dev), "device query")) return 0;
    int uncached = 0;
    int &resident_slot = (dev >= 0 && dev < 32) ? resident_tab[gated ? 1 : 0][dev] : uncached;
    if (resident_slot == 0) {
      int sms = 0, per_sm = 0;
      if (!coli_cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "device query")) return 0;
      const cudaError_t e = gated ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_ffn_mm<FMT, NB, true, false>, W * 32, 0)
                                  : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_ffn_mm<FMT, NB, false, false>, W * 32, 0);
      if (!coli_cuda_check(e, "occupancy query")) return 0;
      resident_slot = sms * (per_sm > 0 ? per_sm : 1);
    }
    const int resident_ctas = resident_slot;
    const long max_ctas = ((long)row_tiles * p.max_items + W - 1) / W;
    const int grid = (int)(max_ctas < resident_ctas ? max_ctas : resident_ctas);
    const cudaError_t e = gated ? launch_dependent(k_ffn_mm<FMT, NB, true, false>, dim3(grid), dim3(W * 32), 0, st, p)
                                : launch_dependent(k_ffn_mm<FMT, NB, false, false>, dim3(grid), dim3(W * 32), 0, st, p);
    coli_count_launch(1);
    return coli_cuda_check(e, "expert ffn launch") ? 1 : 0;
  }
}

// rows_per_item the caller cut the work list with selects NB (8 * NB >= rows per item).
static int launch_ffn_stage(const FfnParams &p, bool gated, cudaStream_t st) {
  if (p.max_items <= 0) return 1;
  if (p.H % 8 || p.I % 8) {
    coli_set_error("expert ffn: H=%d and I=%d must be multiples of 8", p.H, p.I);
    return 0;
  }
  if (p.rows_per_item > 32) {
    coli_set_error("expert ffn: rows_per_item=%d exceeds 32", p.rows_per_item);
    return 0;
  }
  const int nb = p.rows_per_item <= 8 ? 1 : p.rows_per_item <= 16 ? 2 : 4;
#define COLI_DISPATCH(F) \
  (nb == 1 ? launch_one<F, 1>(p, gated, st) : nb == 2 ? launch_one<F, 2>(p, gated, st) : launch_one<F, 4>(p, gated, st))
  switch (p.fmt) {
    case COLI_FMT_NVFP4:
      return COLI_DISPATCH(COLI_FMT_NVFP4);
    case COLI_FMT_FP8_B128:
      return COLI_DISPATCH(COLI_FMT_FP8_B128);
    case COLI_FMT_E4M3_ROW:
      return COLI_DISPATCH(COLI_FMT_E4M3_ROW);
    default:
      coli_set_error("expert ffn: unsupported weight format %d", p.fmt);
      return 0;
  }
#undef COLI_DISPATCH
}

int launch_gate_up_small(const FfnParams &p, cudaStream_t st) { return launch_ffn_stage(p, true, st); }
int launch_down_small(const FfnParams &p, cudaStream_t st) { return launch_ffn_stage(p, false, st); }
int launch_ffn_small(const FfnParams &p, cudaStream_t st) {
  return launch_gate_up_small(p, st) && launch_down_small(p, st);
}

}  // namespace colib
