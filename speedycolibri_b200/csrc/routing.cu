// Routing: router GEMM with a strictly k-ascending f32 sum per logit, score + top-k
// (softmax / sigmoid+bias / group-limited), and the permutation of (token, kk) pairs into
// expert-contiguous row segments.
//
// Bit-exactness contract.  The CPU restatement of crates/colibri-engine/src/moe.rs:1047-1132
// sums each logit sequentially over k in f32 (linear.rs:199-220), scores with exp, sums the
// softmax denominator sequentially over e, and picks k experts by a strict `>` scan from e = 0.
// Every one of those steps is reproduced here operation for operation:
//   * x and the router weights are bf16, so each product is exact in f32 and one fused
//     multiply-add per k equals the reference's multiply-then-add; each logit is owned by ONE
//     thread that walks k = 0..H-1 in order (no split-K, no tensor cores);
//   * exp / sigmoid come from coli_math.h, compiled identically for host and device;
//   * adds, subs, divides that the compiler could contract or reorder are spelled with the
//     CF_* round-to-nearest intrinsics;
//   * the arg-max of each round is the largest value with the lowest index, which is what the
//     ascending strict-`>` scan returns; a round with no candidate above -inf returns 0.
#include <cstdlib>

#include "internal.cuh"

namespace colib {

// ---------------------------------------------------------------------------------------------
// Router GEMM, general shape.  Block = 16x16 threads, thread tile TM x TN, k-chunk 32 staged in
// shared memory as f32 (transposed so the inner loop reads broadcast / consecutive words).
// ---------------------------------------------------------------------------------------------
template <int TM, int TN>
__global__ void __launch_bounds__(256) k_router_gemm(RouteParams p) {
  constexpr int BM = 16 * TM, BN = 16 * TN, BK = 32;
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < p.H; k0 += BK) {
    // stage x[m0..m0+BM, k0..k0+32) and w[n0..n0+BN, k0..k0+32), zero beyond the edges
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      const int r = idx / BK, c = idx % BK;
      const int m = m0 + r, k = k0 + c;
      float v = 0.0f;
      if (m < p.T && k < p.H) v = __bfloat162float(p.x[(size_t)m * p.H + k]);
      xs[c][r] = v;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
      const int r = idx / BK, c = idx % BK;
      const int n = n0 + r, k = k0 + c;
      float v = 0.0f;
      if (n < p.E && k < p.H) v = __bfloat162float(p.router_w[(size_t)n * p.H + k]);
      ws[c][r] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int m = m0 + ty * TM + i, n = n0 + tx * TN + j;
      if (m < p.T && n < p.E) {
        float v = acc[i][j];
        if (p.logit_bias) v = __fadd_rn(v, p.logit_bias[n]);
        p.logits[(size_t)m * p.E + n] = v;
      }
    }
}

// Router GEMM, batched shapes: BM tokens x 64 experts per CTA of NT threads, (BM*16/NT) x 4
// outputs per thread, k-chunks of 32 staged with 16-byte loads and stored transposed as f32, so
// the inner loop is a few 128-bit shared loads per block of FMAs.  Same arithmetic as above: each
// output is one thread's k-ascending fmaf chain.  Needs H % 8 == 0.  The chain makes the kernel
// issue-bound with a fixed time per CTA, so the variants trade work per thread against the number
// of CTAs: the launcher takes the largest tile that still covers the SMs.
// Two independent f32 FMAs in one instruction (sm_100): c.x = fma(a.x, b, c.x), c.y = fma(a.y, b, c.y),
// each rounded as a scalar fmaf, so an output's k-ascending chain is unchanged.  It halves the FMA
// instructions of k_router_gemm_big (0.51 -> 0.475 ms at 4096 tokens x 256 experts x 7168); the 8 x 8
// register-tiled kernel below measured the same with and without it and keeps scalar FMAs.
__device__ __forceinline__ void coli_ffma2(float2 &c, const float2 a, const float b) {
  unsigned long long cc, aa, bb;
  asm("mov.b64 %0, {%1, %2};" : "=l"(cc) : "f"(c.x), "f"(c.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(aa) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %1};" : "=l"(bb) : "f"(b));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(cc) : "l"(aa), "l"(bb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(c.x), "=f"(c.y) : "l"(cc));
}

template <int BM, int NT>
__global__ void __launch_bounds__(NT) k_router_gemm_big(RouteParams p) {
  constexpr int TMR = BM * 16 / NT;  // token rows per thread
  constexpr int BN = 64, BK = 32, LDX = BM + 4, LDW = BN + 4;
  constexpr int SR = NT / 4;                  // rows staged per pass (4 chunks of 8 k each)
  constexpr int XP = (BM + SR - 1) / SR, WP = BN / SR;
  static_assert(TMR >= 1 && BN % SR == 0, "tile / thread-count mismatch");
  // two buffers of each staged tile: chunk i+1 is written while chunk i is multiplied, so one
  // barrier per chunk suffices
  extern __shared__ __align__(16) float rsm[];
  float(*xs)[BK][LDX] = reinterpret_cast<float(*)[BK][LDX]>(rsm);                  // [2][BK][LDX]
  float(*ws)[BK][LDW] = reinterpret_cast<float(*)[BK][LDW]>(rsm + 2 * BK * LDX);   // [2][BK][LDW]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // tx -> 4 experts, ty -> TMR tokens
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  static_assert(TMR % 2 == 0, "token rows are accumulated in pairs");
  float2 acc[TMR / 2][4];  // .x = token row 2i, .y = row 2i + 1
#pragma unroll
  for (int i = 0; i < TMR / 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = make_float2(0.0f, 0.0f);
  // staging assignment: the threads of a warp take consecutive rows of one 8-k chunk, so their
  // transposed stores fall into consecutive banks
  const int sr = threadIdx.x % SR, sc = threadIdx.x / SR;
  uint4 xv[XP], wv[WP];
  auto fetch = [&](int k0) {  // global -> registers; issued one chunk ahead of its use
    const int k = k0 + sc * 8;
#pragma unroll
    for (int h = 0; h < XP; ++h) {
      const int m = m0 + sr + SR * h;
      xv[h] = make_uint4(0, 0, 0, 0);
      if (sr + SR * h < BM && m < p.T && k < p.H) xv[h] = *reinterpret_cast<const uint4 *>(p.x + (size_t)m * p.H + k);
    }
#pragma unroll
    for (int h = 0; h < WP; ++h) {
      const int n = n0 + sr + SR * h;
      wv[h] = make_uint4(0, 0, 0, 0);
      if (n < p.E && k < p.H) wv[h] = *reinterpret_cast<const uint4 *>(p.router_w + (size_t)n * p.H + k);
    }
  };
  auto stage = [&](int buf) {  // registers -> shared memory, bf16 -> f32, transposed
#pragma unroll
    for (int h = 0; h < XP; ++h) {
      if (sr + SR * h >= BM) break;
      const uint32_t u[4] = {xv[h].x, xv[h].y, xv[h].z, xv[h].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xs[buf][sc * 8 + 2 * j][sr + SR * h] = __uint_as_float(u[j] << 16);
        xs[buf][sc * 8 + 2 * j + 1][sr + SR * h] = __uint_as_float(u[j] & 0xffff0000u);
      }
    }
#pragma unroll
    for (int h = 0; h < WP; ++h) {
      const uint32_t u[4] = {wv[h].x, wv[h].y, wv[h].z, wv[h].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        ws[buf][sc * 8 + 2 * j][sr + SR * h] = __uint_as_float(u[j] << 16);
        ws[buf][sc * 8 + 2 * j + 1][sr + SR * h] = __uint_as_float(u[j] & 0xffff0000u);
      }
    }
  };
  fetch(0);
  stage(0);
  __syncthreads();
  if (BK < p.H) fetch(BK);
  int buf = 0;
  for (int k0 = 0; k0 < p.H; k0 += BK, buf ^= 1) {
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      float a[TMR];
      if (TMR >= 4) {
#pragma unroll
        for (int q = 0; q < TMR / 4; ++q) {
          const float4 v = *reinterpret_cast<const float4 *>(&xs[buf][kk][ty * TMR + 4 * q]);
          a[4 * q] = v.x;
          a[4 * q + 1] = v.y;
          a[4 * q + 2] = v.z;
          a[4 * q + 3] = v.w;
        }
      } else if (TMR == 2) {
        const float2 v = *reinterpret_cast<const float2 *>(&xs[buf][kk][ty * 2]);
        a[0] = v.x;
        a[TMR - 1] = v.y;
      } else {
#pragma unroll
        for (int i = 0; i < TMR; ++i) a[i] = xs[buf][kk][ty * TMR + i];
      }
      const float4 b = *reinterpret_cast<const float4 *>(&ws[buf][kk][tx * 4]);
      const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < TMR / 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) coli_ffma2(acc[i][j], make_float2(a[2 * i], a[2 * i + 1]), bb[j]);
    }
    if (k0 + BK < p.H) {
      stage(buf ^ 1);  // chunk k0 + BK, fetched while this one was multiplied; that buffer was last read one barrier ago
      if (k0 + 2 * BK < p.H) fetch(k0 + 2 * BK);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TMR; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * TMR + i, n = n0 + tx * 4 + j;
      if (m < p.T && n < p.E) {
        float v = (i & 1) ? acc[i >> 1][j].y : acc[i >> 1][j].x;
        if (p.logit_bias) v = __fadd_rn(v, p.logit_bias[n]);
        p.logits[(size_t)m * p.E + n] = v;
      }
    }
}

// Router GEMM, register-tiled: every thread owns TM tokens x TN experts (TM*TN independent
// k-ascending fmaf chains), a CTA of NT threads covers (NT/16)*TM tokens x 16*TN experts.  The
// kernel is bound by the shared-memory operand traffic per FMA, (TM + TN) / (TM * TN) words: an
// 8 x 8 tile needs a quarter of what a 2 x 4 tile does, so large batches take the largest tile and
// small ones the largest tile that still gives every SM a CTA.  Operands are staged as f32,
// transposed (k-major), two buffers, 16-byte loads one chunk ahead; a thread's experts are
// {tx*4 + j} in each 64-wide group, so the 16 lanes of a row read consecutive 16-byte words.
// Same arithmetic as the other router kernels: the tile shape never changes an output's k order.
// Needs H % 8 == 0.
template <int TM, int TN, int NT>
__global__ void __launch_bounds__(NT) k_router_rt(RouteParams p) {
  static_assert(TN % 4 == 0 && (TM % 4 == 0 || TM == 2), "tile shape");
  constexpr int BM = (NT / 16) * TM, BN = 16 * TN, BK = 32, LDX = BM + 4, LDW = BN + 4;
  constexpr int SR = NT / 4;  // rows staged per pass (4 chunks of 8 k each)
  constexpr int XP = (BM + SR - 1) / SR, WP = (BN + SR - 1) / SR;
  extern __shared__ __align__(16) float rsm[];
  float(*xs)[BK][LDX] = reinterpret_cast<float(*)[BK][LDX]>(rsm);
  float(*ws)[BK][LDW] = reinterpret_cast<float(*)[BK][LDW]>(rsm + 2 * BK * LDX);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
  const int sr = threadIdx.x % SR, sc = threadIdx.x / SR;
  uint4 xv[XP], wv[WP];
  auto fetch = [&](int k0) {
    const int k = k0 + sc * 8;
#pragma unroll
    for (int h = 0; h < XP; ++h) {
      const int r = sr + SR * h, m = m0 + r;
      xv[h] = make_uint4(0, 0, 0, 0);
      if (r < BM && m < p.T && k < p.H) xv[h] = *reinterpret_cast<const uint4 *>(p.x + (size_t)m * p.H + k);
    }
#pragma unroll
    for (int h = 0; h < WP; ++h) {
      const int r = sr + SR * h, n = n0 + r;
      wv[h] = make_uint4(0, 0, 0, 0);
      if (r < BN && n < p.E && k < p.H) wv[h] = *reinterpret_cast<const uint4 *>(p.router_w + (size_t)n * p.H + k);
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int h = 0; h < XP; ++h) {
      const int r = sr + SR * h;
      if (r < BM) {
        const uint32_t u[4] = {xv[h].x, xv[h].y, xv[h].z, xv[h].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xs[buf][sc * 8 + 2 * j][r] = __uint_as_float(u[j] << 16);
          xs[buf][sc * 8 + 2 * j + 1][r] = __uint_as_float(u[j] & 0xffff0000u);
        }
      }
    }
#pragma unroll
    for (int h = 0; h < WP; ++h) {
      const int r = sr + SR * h;
      if (r < BN) {
        const uint32_t u[4] = {wv[h].x, wv[h].y, wv[h].z, wv[h].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ws[buf][sc * 8 + 2 * j][r] = __uint_as_float(u[j] << 16);
          ws[buf][sc * 8 + 2 * j + 1][r] = __uint_as_float(u[j] & 0xffff0000u);
        }
      }
    }
  };
  fetch(0);
  stage(0);
  __syncthreads();
  if (BK < p.H) fetch(BK);
  int buf = 0;
  for (int k0 = 0; k0 < p.H; k0 += BK, buf ^= 1) {
#pragma unroll 4
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
      if (TM == 2) {
        const float2 v = *reinterpret_cast<const float2 *>(&xs[buf][kk][ty * 2]);
        a[0] = v.x;
        a[TM - 1] = v.y;
      } else {
#pragma unroll
        for (int q = 0; q < TM / 4; ++q) {
          const float4 v = *reinterpret_cast<const float4 *>(&xs[buf][kk][ty * TM + 4 * q]);
          a[4 * q] = v.x;
          a[4 * q + 1] = v.y;
          a[4 * q + 2] = v.z;
          a[4 * q + 3] = v.w;
        }
      }
#pragma unroll
      for (int q = 0; q < TN / 4; ++q) {
        const float4 v = *reinterpret_cast<const float4 *>(&ws[buf][kk][q * 64 + tx * 4]);
        b[4 * q] = v.x;
        b[4 * q + 1] = v.y;
        b[4 * q + 2] = v.z;
        b[4 * q + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
    }
    if (k0 + BK < p.H) {
      stage(buf ^ 1);
      if (k0 + 2 * BK < p.H) fetch(k0 + 2 * BK);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int m = m0 + ty * TM + i, n = n0 + (j >> 2) * 64 + tx * 4 + (j & 3);
      if (m < p.T && n < p.E) {
        float v = acc[i][j];
        if (p.logit_bias) v = __fadd_rn(v, p.logit_bias[n]);
        p.logits[(size_t)m * p.E + n] = v;
      }
    }
}

// Decode shape (T <= 8): one thread per (token, expert) walking its own k chain; the block's 8
// expert rows and all token rows are staged in shared memory as bf16 with coalesced 16-byte
// loads first.  The chain of H dependent FMAs is the latency floor of bit-exact routing.
__device__ __forceinline__ void router_decode_block(const RouteParams &p, unsigned char *smem_raw) {
  // rows of H bf16 plus 16 bytes of padding: the chain threads of a warp read 4 token rows and 8
  // expert rows at the same column, and unpadded rows (a multiple of 128 bytes apart) would all
  // start in the same shared-memory bank
  uint4 *xs = reinterpret_cast<uint4 *>(smem_raw);  // [T][vec + 1]
  const int e0 = blockIdx.x * 8;
  const int H = p.H;
  const int vec = H / 8;  // H % 8 == 0 checked by the launcher
  const int rs = vec + 1; // row stride in 16-byte units
  uint4 *ws = xs + (size_t)p.T * rs;                // [8][vec + 1]
  // staging in batches of 8 independent 16-byte loads per thread: a load-store loop would pay one
  // memory round trip per iteration
  const int nx = p.T * vec, nw = 8 * vec;
  for (int base = 0; base < nx + nw; base += 8 * (int)blockDim.x) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = base + u * (int)blockDim.x + (int)threadIdx.x;
      v[u] = make_uint4(0, 0, 0, 0);
      if (idx < nx) {
        v[u] = reinterpret_cast<const uint4 *>(p.x)[idx];
      } else if (idx < nx + nw) {
        const int r = (idx - nx) / vec, c = (idx - nx) % vec;
        if (e0 + r < p.E) v[u] = reinterpret_cast<const uint4 *>(p.router_w + (size_t)(e0 + r) * H)[c];
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = base + u * (int)blockDim.x + (int)threadIdx.x;
      if (idx < nx + nw) xs[(idx / vec) * rs + idx % vec] = v[u];  // ws follows xs directly
    }
  }
  __syncthreads();
  const int t = threadIdx.x >> 3, el = threadIdx.x & 7;
  if (t >= p.T || e0 + el >= p.E) return;
  const uint4 *xr = xs + (size_t)t * rs;
  const uint4 *wr = ws + (size_t)el * rs;
  float acc = 0.0f;
#pragma unroll 4
  for (int c = 0; c < vec; ++c) {
    const uint4 xv = xr[c], wv = wr[c];
    const uint32_t xa[4] = {xv.x, xv.y, xv.z, xv.w}, wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc = __fmaf_rn(__uint_as_float(xa[j] << 16), __uint_as_float(wa[j] << 16), acc);
      acc = __fmaf_rn(__uint_as_float(xa[j] & 0xffff0000u), __uint_as_float(wa[j] & 0xffff0000u), acc);
    }
  }
  if (p.logit_bias) acc = __fadd_rn(acc, p.logit_bias[e0 + el]);
  p.logits[(size_t)t * p.E + e0 + el] = acc;
}
__global__ void __launch_bounds__(256) k_router_decode(RouteParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  router_decode_block(p, smem_raw);
}

// ---------------------------------------------------------------------------------------------
// Score + top-k: one warp per token.  Expert e lives in lane e % 32, slot e / 32 (<= 16 slots).
// ---------------------------------------------------------------------------------------------
constexpr int kMaxSlots = 16;  // E <= 512

// Warp arg-max with the reference's tie rule: larger value wins, equal values -> lower index.
// `has` marks lanes that hold a candidate (value strictly above -inf).
__device__ __forceinline__ void warp_argmax(float &v, int &i, bool &has) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, off);
    const int oi = __shfl_xor_sync(0xffffffffu, i, off);
    const bool oh = __shfl_xor_sync(0xffffffffu, (int)has, off) != 0;
    if (oh && (!has || ov > v || (ov == v && oi < i))) {
      v = ov;
      i = oi;
      has = true;
    }
  }
}

// One warp scores token t and selects its experts; score/choice are E floats of shared memory
// each, private to the warp.
__device__ __forceinline__ void route_topk_token(const RouteParams &p, int t, float *score, float *choice, int lane) {
  const int E = p.E, k = min(p.k, p.E);
  const float *z = p.logits + (size_t)t * E;
  const float NEG_INF = __uint_as_float(0xff800000u);

  if (p.score == COLI_SCORE_SOFTMAX) {
    float mx = NEG_INF;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, __ldcg(z + e));  // max is order-independent
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    for (int e = lane; e < E; e += 32) score[e] = coli_expf(__fsub_rn(__ldcg(z + e), mx));
    __syncwarp();
    float tot = 0.0f;  // sequential over e, every lane redundantly (moe.rs:1068)
    for (int e = 0; e < E; ++e) tot = __fadd_rn(tot, score[e]);
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
      float s = score[e];
      if (tot > 0.0f) s = __fdiv_rn(s, tot);
      score[e] = s;
      choice[e] = s;
    }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float s = coli_sigmoidf(__ldcg(z + e));
      score[e] = s;
      choice[e] = __fadd_rn(s, p.select_bias ? p.select_bias[e] : 0.0f);
    }
  }
  __syncwarp();

  // group-limited selection: allowed-group bit mask (n_group <= 32)
  uint32_t gmask = 0xffffffffu;
  int gs = E;
  if (p.n_group > 1) {
    const int G = p.n_group;
    gs = E / G;
    const int kg = min(p.topk_group, G);
    float gscore = NEG_INF;
    if (lane < G) {
      float m1 = NEG_INF, m2 = NEG_INF;
      for (int e = lane * gs; e < (lane + 1) * gs; ++e) {
        const float c = choice[e];
        if (c > m1) {
          m2 = m1;
          m1 = c;
        } else if (c > m2) {
          m2 = c;
        }
      }
      gscore = __fadd_rn(m1, m2);
    }
    gmask = 0;
    bool taken = false;
    for (int j = 0; j < kg; ++j) {
      float v = gscore;
      int i = lane;
      bool has = (lane < G) && !taken && (gscore > NEG_INF);
      warp_argmax(v, i, has);
      const int best = has ? i : 0;
      if (lane == best) taken = true;
      gmask |= 1u << best;
    }
  }

  // k rounds of arg-max over the allowed, not yet chosen experts.  Every lane keeps the best of
  // its own remaining experts as an order-preserving integer key (0 = none left; a candidate
  // must be above -inf, as in the reference's scan from -inf with a strict compare); a round is
  // two warp reductions -- the largest key, then the lowest expert id among its holders -- and
  // only the winning lane rescans its experts.
  const bool grouped = p.n_group > 1;
  auto lane_best = [&](uint32_t chosen_mask, uint32_t &key, uint32_t &idx) {
    key = 0u;
    idx = 0xffffffffu;
    for (int s = 0; s < kMaxSlots; ++s) {
      const int e = lane + 32 * s;
      if (e >= E) break;
      if ((chosen_mask >> s) & 1u) continue;
      if (grouped && !((gmask >> (e / gs)) & 1u)) continue;
      const float c = choice[e];
      if (!(c > NEG_INF)) continue;
      const uint32_t bits = __float_as_uint(__fadd_rn(c, 0.0f));  // -0 and +0 tie like the float compare
      const uint32_t kk = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
      if (kk > key) {  // ascending e within the lane: strict > keeps the lowest index
        key = kk;
        idx = (uint32_t)e;
      }
    }
  };
  uint32_t chosen = 0;  // bit s = slot s of this lane already chosen
  int my_idx = 0;       // lane kk keeps idx[kk]
  float my_w = 0.0f;
  uint32_t bkey, bidx;
  lane_best(chosen, bkey, bidx);
  for (int kk = 0; kk < k; ++kk) {
    const uint32_t top = __reduce_max_sync(0xffffffffu, bkey);
    const uint32_t win = __reduce_min_sync(0xffffffffu, (top != 0u && bkey == top) ? bidx : 0xffffffffu);
    const int best = top != 0u ? (int)win : 0;
    if (top != 0u && (best & 31) == lane) {
      chosen |= 1u << (best >> 5);
      lane_best(chosen, bkey, bidx);
    }
    if (lane == kk) {
      my_idx = best;
      my_w = score[best];
    }
  }
  if (p.norm_topk) {
    float smv = 0.0f;
    for (int kk = 0; kk < k; ++kk) smv = __fadd_rn(smv, __shfl_sync(0xffffffffu, my_w, kk));
    smv = __fadd_rn(smv, 1e-20f);
    my_w = __fdiv_rn(my_w, smv);
  }
  my_w = __fmul_rn(my_w, p.routed_scale);
  if (lane < k) {
    p.topk_idx[(size_t)t * k + lane] = my_idx;
    p.topk_w[(size_t)t * k + lane] = my_w;
  }
}

__global__ void __launch_bounds__(128) k_route_topk(RouteParams p) {
  extern __shared__ float sm[];  // per warp: score[E] then choice[E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= p.T) return;
  route_topk_token(p, t, sm + (size_t)warp * 2 * p.E, sm + (size_t)warp * 2 * p.E + p.E, lane);
}

template <int BM, int NT>
static bool launch_router_big(const RouteParams &p, dim3 grid, cudaStream_t st) {
  constexpr size_t smem = (size_t)2 * 32 * ((BM + 4) + (64 + 4)) * sizeof(float);
  static ColiPerDeviceOnce attr_once;
  if (smem > 48 * 1024 && !coli_set_smem_limit(attr_once, k_router_gemm_big<BM, NT>, smem, "router shared-memory attribute")) return false;
  k_router_gemm_big<BM, NT><<<grid, NT, smem, st>>>(p);
  return true;
}

template <int TM, int TN, int NT>
static bool launch_router_rt(const RouteParams &p, cudaStream_t st) {
  constexpr int BM = (NT / 16) * TM, BN = 16 * TN;
  constexpr size_t smem = (size_t)2 * 32 * ((BM + 4) + (BN + 4)) * sizeof(float);
  static ColiPerDeviceOnce attr_once;
  if (smem > 48 * 1024 && !coli_set_smem_limit(attr_once, k_router_rt<TM, TN, NT>, smem, "router shared-memory attribute")) return false;
  dim3 grid((p.E + BN - 1) / BN, (p.T + BM - 1) / BM);
  k_router_rt<TM, TN, NT><<<grid, NT, smem, st>>>(p);
  return true;
}
// The register-tiled variants, largest tile first; `force` (1-based, from COLI_ROUTER_TILE, a
// measurement aid) picks one regardless of the batch.  Returns -1 when none applies.
static int launch_router_tiled(const RouteParams &p, cudaStream_t st) {
  if (p.H % 8 != 0 || p.E < 64) return -1;
  const char *fe = getenv("COLI_ROUTER_TILE");
  const int force = fe ? atoi(fe) : 0;
  auto ctas = [&](int bm, int bn) { return (long)((p.T + bm - 1) / bm) * ((p.E + bn - 1) / bn); };
  int pick = force;
  if (pick <= 0) {
    // Measured on B200 (H = 7168 / 6144): the 8 x 8 tile pays once a batch gives every SM well over one
    // 128 x 128 CTA (T = 16384, E = 384: 1.92 ms against 2.17); below that the narrower tiles of
    // k_router_gemm_big, which keep two warps per scheduler, are as fast or faster.
    if (p.E >= 128 && ctas(128, 128) >= 240) pick = 7;
    else return -1;
  }
  bool ok = false;
  switch (pick) {
    case 1: ok = launch_router_rt<8, 8, 128>(p, st); break;   // 64 tokens x 128 experts
    case 2: ok = launch_router_rt<4, 8, 128>(p, st); break;   // 32 x 128
    case 3: ok = launch_router_rt<4, 4, 128>(p, st); break;   // 32 x 64
    case 4: ok = launch_router_rt<4, 4, 64>(p, st); break;    // 16 x 64, two warps
    case 5: ok = launch_router_rt<2, 4, 64>(p, st); break;    // 8 x 64
    case 6: ok = launch_router_rt<8, 4, 128>(p, st); break;   // 64 x 64
    case 7: ok = launch_router_rt<8, 8, 256>(p, st); break;   // 128 x 128
    default: return -1;
  }
  return ok ? 1 : 0;
}

int launch_router(const RouteParams &p, cudaStream_t st) {
  if (p.T <= 0) return 1;
  if (p.E > 32 * kMaxSlots) {
    coli_set_error("router: E=%d exceeds the supported maximum of %d", p.E, 32 * kMaxSlots);
    return 0;
  }
  if (p.k > 32 || p.n_group > 32 || (p.n_group > 1 && p.E % p.n_group != 0)) {
    coli_set_error("router: unsupported k=%d / n_group=%d for E=%d", p.k, p.n_group, p.E);
    return 0;
  }
  if (p.n_group > 1 && p.k > min(p.topk_group, p.n_group) * (p.E / p.n_group)) {
    coli_set_error("router: k=%d exceeds the experts of the %d groups a token may use", p.k, p.topk_group);
    return 0;
  }
  const size_t dec_smem = (size_t)(p.T + 8) * (p.H + 8) * sizeof(__nv_bfloat16);
  if (p.T <= 8 && p.H % 8 == 0 && dec_smem <= 200 * 1024) {
    static ColiPerDeviceOnce attr_once;
    if (!coli_set_smem_limit(attr_once, k_router_decode, 200 * 1024, "decode router shared-memory attribute")) return 0;
    k_router_decode<<<(p.E + 7) / 8, 256, dec_smem, st>>>(p);  // 256 threads stage the rows, T*8 of them walk the chains
    coli_count_launch(1);
  } else if (const int tiled = launch_router_tiled(p, st); tiled >= 0) {
    if (tiled == 0) return 0;
    coli_count_launch(1);
  } else {
    // the largest tile that still covers the SMs; every variant has identical arithmetic
    auto blocks = [&](int bm, int bn) { return (long)((p.T + bm - 1) / bm) * ((p.E + bn - 1) / bn); };
    const long want = 120;
    if (p.H % 8 == 0 && blocks(128, 64) >= want) {
      dim3 grid((p.E + 63) / 64, (p.T + 127) / 128);
      if (!launch_router_big<128, 256>(p, grid, st)) return 0;
    } else if (p.H % 8 == 0 && blocks(64, 64) >= want) {
      dim3 grid((p.E + 63) / 64, (p.T + 63) / 64);
      if (!launch_router_big<64, 256>(p, grid, st)) return 0;
    } else if (p.H % 8 == 0 && blocks(32, 64) >= want) {
      dim3 grid((p.E + 63) / 64, (p.T + 31) / 32);
      if (!launch_router_big<32, 128>(p, grid, st)) return 0;
    } else if (p.H % 8 == 0 && p.T >= 16) {
      dim3 grid((p.E + 63) / 64, (p.T + 15) / 16);
      if (!launch_router_big<16, 128>(p, grid, st)) return 0;
    } else if (blocks(32, 32) >= 96) {
      dim3 grid((p.E + 31) / 32, (p.T + 31) / 32);
      k_router_gemm<2, 2><<<grid, 256, 0, st>>>(p);
    } else {
      dim3 grid((p.E + 15) / 16, (p.T + 15) / 16);
      k_router_gemm<1, 1><<<grid, 256, 0, st>>>(p);
    }
    coli_count_launch(1);
  }
  const size_t sm = (size_t)4 * 2 * p.E * sizeof(float);
  k_route_topk<<<(p.T + 3) / 4, 128, sm, st>>>(p);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "router launch") ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------
// Permutation into expert-contiguous segments.  Stable: rows of one expert keep ascending
// token order (moe.rs:1373-1387), positions are a pure function of the routing.
//   1. k_seg_count : one warp per chunk of 32 tokens walks its tokens in order; lane kk bumps
//                    a shared-memory counter of expert idx[t][kk] and records the rank.  A
//                    token's experts are distinct except in the degenerate case the reference's
//                    scan also has (a row of NaN logits selects expert 0 k times); lanes that
//                    hold the same expert are ranked among themselves so that every pair still
//                    gets a row of its own.  An id outside [0, E) gets no row (slot -1).
//   2. k_seg_scan  : per expert an exclusive running sum over chunks; exclusive scan over the
//                    segment order; builds the work list (segments cut into row_per_item runs).
//   3. k_permute   : row position = segment offset + chunk prefix + rank; copies the token row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k_seg_count(PermuteParams p, int nchunk) {
  extern __shared__ int cnt_sm[];  // [4][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * 4 + warp;
  int *cnt = cnt_sm + (size_t)warp * p.E;
  for (int e = lane; e < p.E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int T = p.virt ? p.virt->total : p.T;
  if (chunk >= nchunk || chunk * 32 >= T) return;
  const int t0 = chunk * 32, t1 = min(T, t0 + 32);
  // all of the chunk's expert ids are requested before the ordered walk: a load per step would put a
  // memory round trip on each of the 32 steps
  int ids[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    ids[i] = -1;
    if (lane < p.k && t0 + i < t1) ids[i] = p.topk_idx[(size_t)(p.virt ? coli_virt_row(p.virt, t0 + i) : t0 + i) * p.k + lane];
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int t = t0 + i;
    if (t >= t1) break;  // uniform across the warp
    const int e = ids[i];
    const bool valid = e >= 0 && e < p.E;
    // invalid lanes share one key: the instruction takes a pass per distinct key, and their group is never read
    const unsigned same = __match_any_sync(0xffffffffu, valid ? e : -1);
    int base = 0;
    if (valid) base = cnt[e];
    __syncwarp();
    if (valid) {
      p.local_rank[(size_t)t * p.k + lane] = base + __popc(same & ((1u << lane) - 1u));
      if ((same & ((1u << lane) - 1u)) == 0) cnt[e] = base + __popc(same);  // lowest lane of the group
    }
    __syncwarp();
  }
  for (int e = lane; e < p.E; e += 32) p.chunk_cnt[(size_t)chunk * p.E + e] = cnt[e];
}

// Segment offsets and the work list from per-segment row counts in shared memory, by the whole
// CTA: warp 0 runs a chunked shuffle scan over the counts (row offsets and item bases at once),
// then one thread per segment writes that segment's items.  off and ibase hold nseg + 1 entries.
// A serial walk by one thread costs ~60 ns per segment, more than the decode GEMV of a layer
// with a few hundred experts.
__device__ __forceinline__ void build_work_list(const PermuteParams &p, const int *cnt, int nseg, int max_items, int *off,
                                                int *ibase) {
  const int rpi = p.rows_per_item;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int run = 0, items = 0;
    for (int base = 0; base < nseg; base += 32) {
      const int s = base + lane;
      const int n = s < nseg ? cnt[s] : 0;
      const int ni = (n + rpi - 1) / rpi;
      int a = n, b = ni;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int ua = __shfl_up_sync(0xffffffffu, a, o), ub = __shfl_up_sync(0xffffffffu, b, o);
        if (lane >= o) {
          a += ua;
          b += ub;
        }
      }
      if (s < nseg) {
        off[s] = run + a - n;
        ibase[s] = items + b - ni;
      }
      run += __shfl_sync(0xffffffffu, a, 31);
      items += __shfl_sync(0xffffffffu, b, 31);
    }
    if (lane == 0) {
      off[nseg] = run;
      ibase[nseg] = items;
      *p.n_items = min(items, max_items);
    }
  }
  __syncthreads();
  for (int s = threadIdx.x; s < nseg; s += blockDim.x) {
    const int n = cnt[s], r0 = off[s];
    int it = ibase[s];
    for (int r = 0; r < n; r += rpi, ++it) {
      if (it < max_items) {
        p.item_seg[it] = s;
        p.item_row0[it] = r0 + r;
        p.item_nrows[it] = min(rpi, n - r);
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(1024) k_seg_scan(PermuteParams p, int nchunk, int max_items) {
  __shared__ int seg_cnt[1024 + 1];
  __shared__ int seg_off[1024 + 2];
  __shared__ int seg_ibase[1024 + 2];
  const int E = p.E;
  if (p.virt) nchunk = min(nchunk, (p.virt->total + 31) / 32);
  const int nrt = p.nseg_routed;  // routed segments: E, or the experts resident on this rank
  const int nseg = nrt + (p.has_shared ? 1 : 0);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int pos = p.expert_slot ? p.expert_slot[e] : e;
    if (pos < 0) continue;  // expert lives on another rank: its pairs get no row here
    int run = 0;
    for (int c0 = 0; c0 < nchunk; c0 += 8) {  // loads of a group are independent of its stores
      int v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (c0 + j < nchunk) ? p.chunk_cnt[(size_t)(c0 + j) * E + e] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c0 + j < nchunk) {
          p.chunk_cnt[(size_t)(c0 + j) * E + e] = run;
          run += v[j];
        }
    }
    seg_cnt[pos] = run;
  }
  if (threadIdx.x == 0 && p.has_shared) seg_cnt[nrt] = p.virt ? p.virt->total : p.T;
  __syncthreads();
  if (p.rows_cap != 0x7fffffff) {  // a batch that does not fit the row buffers is not run at all (and reported)
    __shared__ int too_many;
    if (threadIdx.x == 0) {
      long total = 0;
      for (int s = 0; s < nseg; ++s) total += seg_cnt[s];
      too_many = total > (long)p.rows_cap ? 1 : 0;
      if (too_many && p.overflow) atomicExch(p.overflow, 1);
    }
    __syncthreads();
    if (too_many)
      for (int s = threadIdx.x; s < nseg; s += blockDim.x) seg_cnt[s] = 0;
    __syncthreads();
  }
  build_work_list(p, seg_cnt, nseg, max_items, seg_off, seg_ibase);
  for (int s = threadIdx.x; s <= nseg; s += blockDim.x) p.seg_off[s] = seg_off[s];
  for (int s = threadIdx.x; s < nrt; s += blockDim.x) p.seg_count[s] = seg_cnt[s];
}

__global__ void __launch_bounds__(256) k_permute(PermuteParams p) {
  // one warp per (t, kk) row; rows T*k .. T*k+T-1 are the shared expert's identity rows; when a
  // token-order f16 copy of x is wanted, T more warps write it
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int T = p.virt ? p.virt->total : p.T;
  const int nrouted = T * p.k;
  const int total = nrouted + (p.has_shared ? T : 0);
  if (warp >= total) {
    const int t = warp - total;
    if (p.x16 && t < T) {
      const int vec = p.H / 8;
      const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)t * p.H);
      uint4 *dst = reinterpret_cast<uint4 *>(p.x16 + (size_t)t * p.H);
      for (int c = lane; c < vec; c += 32) dst[c] = coli_bf16x8_to_f16x8(src[c]);
    }
    return;
  }
  int t, pos;
  int trow;  // row of the token in x / topk_idx
  if (warp < nrouted) {
    t = warp / p.k;
    trow = p.virt ? coli_virt_row(p.virt, t) : t;
    const int e = p.topk_idx[(size_t)trow * p.k + (warp - t * p.k)];
    const int s = (e < 0 || e >= p.E) ? -1 : (p.expert_slot ? p.expert_slot[e] : e);
    if (s < 0) {  // not resident here (or not an expert id): no row, the combine skips negative slots
      if (lane == 0) p.slot[warp] = -1;
      return;
    }
    pos = p.seg_off[s] + p.chunk_cnt[(size_t)(t >> 5) * p.E + e] + p.local_rank[warp];
    if (pos >= p.rows_cap) {  // more rows than the buffers hold: drop the pair and report it
      if (lane == 0) {
        p.slot[warp] = -1;
        if (p.overflow) atomicExch(p.overflow, 1);
      }
      return;
    }
    if (lane == 0) p.slot[warp] = pos;
  } else {
    t = warp - nrouted;
    trow = t;
    pos = p.seg_off[p.nseg_routed] + t;
  }
  if (lane == 0) p.row_token[pos] = t;
  if (p.xg && (warp < nrouted || p.gather_shared)) {
    const int vec = p.H / 8;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)trow * p.H);
    uint4 *dst = reinterpret_cast<uint4 *>(p.xg + (size_t)pos * p.H);
    for (int c = lane; c < vec; c += 32) dst[c] = coli_bf16x8_to_f16x8(src[c]);
  }
}

// Decode-sized batches (T*k <= 1024 pairs): count, scan, work list and row positions by ONE CTA
// instead of three launches (each launch costs about as much as the whole decode GEMV).
// Same stable order as the three-kernel path: positions ascend with the token inside an expert.
struct PermuteSmallSmem {
  int cnt[1024 + 1];
  int off[1024 + 2];
  int rank[1024];
  int idx[1024];
  int ibase[1024 + 2];
};
__device__ __forceinline__ void permute_small_body(const PermuteParams &p, int max_items, PermuteSmallSmem &sm) {
  int *cnt = sm.cnt, *off = sm.off, *rank_sm = sm.rank, *idx_sm = sm.idx;
  const int E = p.E, nrt = p.nseg_routed, nseg = nrt + (p.has_shared ? 1 : 0);
  const int npairs = p.T * p.k;
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  // segment of every pair, fetched with independent loads before the ordered walk below
  for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
    const int e = p.topk_idx[i];
    idx_sm[i] = (e < 0 || e >= E) ? -1 : (p.expert_slot ? p.expert_slot[e] : e);
  }
  __syncthreads();
  if (threadIdx.x < 32) {  // one warp walks the tokens in order; lane kk owns pair (t, kk)
    const int ln = (int)threadIdx.x;
    for (int t = 0; t < p.T; ++t) {  // lanes holding the same segment (a degenerate routing) rank among themselves
      const int s = ln < p.k ? idx_sm[t * p.k + ln] : -1;
      const unsigned same = __match_any_sync(0xffffffffu, s >= 0 ? s : -1);  // one key for all lanes without a row
      int base = 0;
      if (s >= 0) base = cnt[s];
      __syncwarp();
      if (s >= 0) {
        rank_sm[t * p.k + ln] = base + __popc(same & ((1u << ln) - 1u));
        if ((same & ((1u << ln) - 1u)) == 0) cnt[s] = base + __popc(same);
      }
      __syncwarp();
    }
    if (threadIdx.x == 0 && p.has_shared) cnt[nrt] = p.T;
  }
  __syncthreads();
  build_work_list(p, cnt, nseg, max_items, off, sm.ibase);
  for (int s = threadIdx.x; s <= nseg; s += blockDim.x) p.seg_off[s] = off[s];
  for (int s = threadIdx.x; s < nrt; s += blockDim.x) p.seg_count[s] = cnt[s];
  for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
    const int s = idx_sm[i];
    if (s < 0) {
      p.slot[i] = -1;
      continue;
    }
    const int pos = off[s] + rank_sm[i];
    p.slot[i] = pos;
    p.row_token[pos] = i / p.k;
  }
  if (p.has_shared)
    for (int t = threadIdx.x; t < p.T; t += blockDim.x) p.row_token[off[nrt] + t] = t;
  if (p.xg) {  // gather rows: one warp per row
    const int total = npairs + ((p.has_shared && p.gather_shared) ? p.T : 0);
    const int vec = p.H / 8;
    for (int r = threadIdx.x >> 5; r < total; r += blockDim.x >> 5) {
      int t, pos;
      if (r < npairs) {
        const int s = idx_sm[r];
        if (s < 0) continue;
        t = r / p.k;
        pos = off[s] + rank_sm[r];
      } else {
        t = r - npairs;
        pos = off[nrt] + t;
      }
      const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)t * p.H);
      uint4 *dst = reinterpret_cast<uint4 *>(p.xg + (size_t)pos * p.H);
      for (int c = threadIdx.x & 31; c < vec; c += 32) dst[c] = coli_bf16x8_to_f16x8(src[c]);
    }
  }
}

__global__ void __launch_bounds__(1024) k_permute_small(PermuteParams p, int max_items) {
  __shared__ PermuteSmallSmem sm;
  if (blockIdx.x > 0) {  // the extra CTAs only write the token-order f16 copy of x
    const size_t n = (size_t)p.T * p.H / 8;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.x);
    uint4 *dst = reinterpret_cast<uint4 *>(p.x16);
    for (size_t i = (size_t)(blockIdx.x - 1) * blockDim.x + threadIdx.x; i < n; i += (size_t)(gridDim.x - 1) * blockDim.x)
      dst[i] = coli_bf16x8_to_f16x8(src[i]);
    return;
  }
  permute_small_body(p, max_items, sm);
}

// Decode front end (T <= 8): router logits, top-k and the permutation in ONE launch.  Every CTA
// computes the logits of 8 experts (and converts its slice of the staged tokens to f16); the CTA
// that finishes last -- found with an atomic ticket, nobody waits for anybody -- scores the
// tokens and builds the segments.  `ticket` must be zero at launch and is left zero.
__global__ void __launch_bounds__(256) k_decode_front(RouteParams rp, PermuteParams pp, int max_items, unsigned int *ticket) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ PermuteSmallSmem psm;
  __shared__ int is_last;
  coli_grid_dependency_sync();
  router_decode_block(rp, smem_raw);
  if (pp.x16) {
    const int n = rp.T * (rp.H / 8);
    const int per = (n + (int)gridDim.x - 1) / (int)gridDim.x;
    const int lo = (int)blockIdx.x * per, hi = min(n, lo + per);
    const uint4 *xs = reinterpret_cast<const uint4 *>(smem_raw);  // staged tokens, bf16, padded rows
    const int vec = rp.H / 8;
    uint4 *dst = reinterpret_cast<uint4 *>(pp.x16);
    for (int i = lo + (int)threadIdx.x; i < hi; i += (int)blockDim.x) dst[i] = coli_bf16x8_to_f16x8(xs[(i / vec) * (vec + 1) + i % vec]);
  }
  __threadfence();  // this CTA's logits are visible device-wide before its ticket is
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    float *sm = reinterpret_cast<float *>(smem_raw);  // the staging area is free now
    for (int t = warp; t < rp.T; t += nwarp) route_topk_token(rp, t, sm + (size_t)warp * 2 * rp.E, sm + (size_t)warp * 2 * rp.E + rp.E, lane);
  }
  __syncthreads();  // the routing this CTA wrote is read back below
  permute_small_body(pp, max_items, psm);
  if (threadIdx.x == 0) *ticket = 0u;
}

static bool permute_small_ok(const PermuteParams &p) { return p.T * p.k <= 1024 && p.k <= 32 && p.E <= 1024; }
static int permute_max_items(const PermuteParams &p) {
  return max_work_items(p.T * p.k + (p.has_shared ? p.T : 0), p.nseg_routed + (p.has_shared ? 1 : 0), p.rows_per_item);
}

int launch_decode_front(const RouteParams &rp, const PermuteParams &pp, unsigned int *ticket, cudaStream_t st) {
  const size_t stage = (size_t)(rp.T + 8) * (rp.H + 8) * sizeof(__nv_bfloat16);
  const size_t topk = (size_t)8 * 2 * rp.E * sizeof(float);
  const size_t smem = stage > topk ? stage : topk;
  if (!(rp.T >= 1 && rp.T <= 8 && rp.H % 8 == 0 && smem <= 180 * 1024 && rp.E <= 32 * kMaxSlots && rp.k <= 32 &&
        rp.n_group <= 32 && (rp.n_group <= 1 || rp.E % rp.n_group == 0) && permute_small_ok(pp) && ticket != nullptr))
    return -1;  // not applicable: the caller runs the separate stages
  static ColiPerDeviceOnce attr_once;
  if (!coli_set_smem_limit(attr_once, k_decode_front, 180 * 1024, "decode front shared-memory attribute")) return 0;
  coli_count_launch(1);
  return coli_cuda_check(launch_dependent(k_decode_front, dim3((rp.E + 7) / 8), dim3(256), smem, st, rp, pp, permute_max_items(pp), ticket),
                         "decode front launch")
             ? 1
             : 0;
}

int launch_permute(const PermuteParams &p, cudaStream_t st) {
  if (p.T <= 0) return 1;
  if (p.E > 1024) {
    coli_set_error("permute: E=%d exceeds 1024", p.E);
    return 0;
  }
  const int nchunk = (p.T + 31) / 32;
  const int max_items = permute_max_items(p);
  // the one-CTA form also gathers the rows: fine up to ~128 KB of them, far too slow for a megabyte
  if (!p.virt && permute_small_ok(p) && (!p.xg || (size_t)p.T * (p.k + 1) * p.H * 2 <= 128 * 1024)) {
    int conv = 0;
    if (p.x16) {
      const size_t n = (size_t)p.T * p.H / 8;
      conv = (int)((n + 1023) / 1024);
      if (conv > 64) conv = 64;
    }
    k_permute_small<<<1 + conv, 1024, 0, st>>>(p, max_items);
    coli_count_launch(1);
    return coli_cuda_check(cudaGetLastError(), "permute launch") ? 1 : 0;
  }
  k_seg_count<<<(nchunk + 3) / 4, 128, (size_t)4 * p.E * sizeof(int), st>>>(p, nchunk);
  coli_count_launch(1);
  k_seg_scan<<<1, 1024, 0, st>>>(p, nchunk, max_items);
  coli_count_launch(1);
  const int total = p.T * p.k + (p.has_shared ? p.T : 0) + (p.x16 ? p.T : 0);
  k_permute<<<(total + 7) / 8, 256, 0, st>>>(p);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "permute launch") ? 1 : 0;
}

__global__ void k_items_from_counts(const int32_t *seg_count, int nseg, int rows_per_item, int32_t *seg_off,
                                    int32_t *item_seg, int32_t *item_row0, int32_t *item_nrows,
                                    int32_t *n_items) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int run = 0, items = 0;
  for (int s = 0; s < nseg; ++s) {
    seg_off[s] = run;
    const int n = seg_count[s];
    for (int r = 0; r < n; r += rows_per_item) {
      item_seg[items] = s;
      item_row0[items] = run + r;
      item_nrows[items] = min(rows_per_item, n - r);
      ++items;
    }
    run += n;
  }
  seg_off[nseg] = run;
  *n_items = items;
}

int launch_items_from_counts(const int32_t *seg_count, int nseg, int rows_per_item, int32_t *seg_off,
                             int32_t *item_seg, int32_t *item_row0, int32_t *item_nrows, int32_t *n_items,
                             cudaStream_t st) {
  k_items_from_counts<<<1, 32, 0, st>>>(seg_count, nseg, rows_per_item, seg_off, item_seg, item_row0,
                                        item_nrows, n_items);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "work list launch") ? 1 : 0;
}

}  // namespace colib

// ---------------------------------------------------------------------------------------------
// Routing without any allocation.
//
// The router needs a [T,E] f32 logits buffer between its GEMM and its top-k kernel.  Every
// other entry point takes that buffer from a handle's cudaMalloc'ed workspace.  This one is for
// callers that must not allocate at all: a serving process that handed every free byte of HBM
// to its weight and KV pools at start-up (a later cudaMalloc there fails, or trips the host's
// memory ledger), and decode loops that cannot afford the device-wide synchronisation a
// cudaMalloc/cudaFree implies.  The logits live in a fixed array that is part of the library
// image, so each GPU that loads the library carries it (512 KiB) until the process exits.
//
// `g_route_scratch` below is a device symbol.  In host code the name is only a stand-in for
// it, not a device address, so the address handed to the kernels is looked up once per device
// with cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_route_scratch[COLI_ROUTE_NOALLOC_MAX_LOGITS];

// Device address of the array per device ordinal, null until the first call on that device has
// looked it up.  Several host threads may make that first call at once: the address is published
// with release/acquire ordering, and two threads that both look it up store the same value.
static float *g_route_scratch_addr[COLI_CUDA_MAX_DEVICES];

extern "C" int coli_b200_route_noalloc(const void *x_dev, const void *router_w_dev, const float *select_bias_dev,
                                       const float *logit_bias_dev, int T, int H, int E, int k, int score,
                                       int norm_topk, float routed_scale, int n_group, int topk_group,
                                       int32_t *topk_idx_dev, float *topk_w_dev, void *stream) {
  if (!x_dev || !router_w_dev || !topk_idx_dev || !topk_w_dev || T < 0 || H < 1 || E < 1 || k < 1 || k > E) {
    coli_set_error("route_noalloc: null pointer or bad shape (T=%d H=%d E=%d k=%d)", T, H, E, k);
    return 0;
  }
  if ((long long)T * E > (long long)COLI_ROUTE_NOALLOC_MAX_LOGITS) {
    coli_set_error("route_noalloc: T*E = %lld exceeds the built-in scratch of %d logits; use a ColiMoe handle for larger batches",
                   (long long)T * E, COLI_ROUTE_NOALLOC_MAX_LOGITS);
    return 0;
  }
  if (score != COLI_SCORE_SOFTMAX && score != COLI_SCORE_SIGMOID) {
    coli_set_error("route_noalloc: unknown score function %d", score);
    return 0;
  }
  int dev = -1;
  if (!coli_cuda_check(cudaGetDevice(&dev), "route_noalloc: cudaGetDevice")) return 0;
  if (dev < 0 || dev >= COLI_CUDA_MAX_DEVICES) {
    coli_set_error("route_noalloc: device ordinal %d out of range", dev);
    return 0;
  }
  float *scratch = __atomic_load_n(&g_route_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    // set-up, once per device, with that device current: resolve the symbol to its device address
    float *ptr = nullptr;
    if (!coli_cuda_check(cudaGetSymbolAddress((void **)&ptr, g_route_scratch), "route_noalloc: cudaGetSymbolAddress")) return 0;
    if (!ptr) {
      coli_set_error("route_noalloc: scratch symbol resolved to a null address");
      return 0;
    }
    __atomic_store_n(&g_route_scratch_addr[dev], ptr, __ATOMIC_RELEASE);
    scratch = ptr;
  }
  if (T == 0) return 1;
  if (H % 8 == 0 && ((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(router_w_dev)) & 15)) {
    coli_set_error("route_noalloc: x_dev and router_w_dev must be 16-byte aligned (the router reads them with 128-bit loads)");
    return 0;
  }
  colib::RouteParams p;
  p.T = T;
  p.H = H;
  p.E = E;
  p.k = k;
  p.score = score;
  p.norm_topk = norm_topk;
  p.routed_scale = routed_scale;
  p.n_group = n_group < 1 ? 1 : n_group;
  p.topk_group = topk_group < 1 ? 1 : topk_group;
  p.x = (const __nv_bfloat16 *)x_dev;
  p.router_w = (const __nv_bfloat16 *)router_w_dev;
  p.select_bias = select_bias_dev;
  p.logit_bias = logit_bias_dev;
  p.logits = scratch;  // every logit of [T,E] is written before it is read: nothing to clear
  p.topk_idx = topk_idx_dev;
  p.topk_w = topk_w_dev;
  return colib::launch_router(p, (cudaStream_t)stream);
}

