// TEST INFRASTRUCTURE — not part of the product.  CPU restatement of the reference's
// routed-expert MoE block (GriffinPilz/SpeedyColibri), used only by tests/, by the smoke
// check and by the CPU-baseline / reference arm of bench.py as the checker and the timed
// CPU baseline.  The library under speedycolibri_b200/ never links or calls this file.
//
// Why a restatement: the reference is a Rust workspace and no Rust toolchain exists in the
// build image, so the original cannot be compiled.  Every function below cites the
// reference file:line it follows.  Pinning: tests/test_oracle_pins.py checks this file
// against the known-answer vectors held by the reference's own unit tests
// (crates/colibri-engine/src/moe.rs:2252-2325,2543-2646; convert.rs:2512-2535,2583-2599,
// 2662-2700; crates/colibri-core/src/dtype.rs:297-310; linear.rs:449-485).
//
// Three deliberate, documented departures from the reference (none is exercised by a
// reference test, so parity for them is unpinned):
//   * exp(): the reference calls libm through Rust std; here coli_expf (f64 evaluation,
//     one rounding) is used so that device and host agree bit for bit.
//   * group-limited routing (n_group > 1) is not implemented by the reference
//     (crates/colibri-core/src/config.rs:703-707 rejects it); defined in orc_route below.
//   * logit_bias (additive bias on the logits before a softmax) does not exist in the
//     reference; its softmax arm ignores the bias vector (moe.rs:1051-1101).
//
// Build: make -C oracle   (g++ -O3 -march=native -ffp-contract=off -pthread)
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#include "../speedycolibri_b200/csrc/coli_math.h"

#include <functional>
#include <thread>

// Static-chunk parallel loop over [0,n) on g_threads std::threads (no OpenMP runtime, so the
// library can sit in one process with PyTorch's own).  Bodies write disjoint outputs.
static int g_threads = 1;
template <class F>
static void parallel_for(int n, F &&body) {
  const int nt = std::max(1, std::min(g_threads, n));
  if (nt == 1) {
    for (int i = 0; i < n; ++i) body(i);
    return;
  }
  std::vector<std::thread> th;
  th.reserve(nt);
  for (int t = 0; t < nt; ++t)
    th.emplace_back([&, t]() {
      const int lo = (int)((int64_t)n * t / nt), hi = (int)((int64_t)n * (t + 1) / nt);
      for (int i = lo; i < hi; ++i) body(i);
    });
  for (auto &x : th) x.join();
}

extern "C" {

// Weight formats: the reference's fmt codes (crates/colibri-core/src/quant.rs:707-746) plus
// one code for the 128x128 block-scaled FP8 form that the reference only reads in its
// converter (crates/colibri-engine/src/convert.rs:674-745).
enum { ORC_FMT_F32 = 0, ORC_FMT_E4M3_ROW = 4, ORC_FMT_NVFP4 = 5, ORC_FMT_MXFP4 = 6, ORC_FMT_FP8_B128 = 8 };

// OCP E8M0 block-scale byte: 2^(b - 127), 0xFF = NaN (crates/colibri-core/src/dtype.rs:136-141).
static inline float e8m0_to_f32(uint8_t b) {
  if (b == 0xFF) return std::numeric_limits<float>::quiet_NaN();
  return ldexpf(1.0f, (int)b - 127);
}

typedef struct {
  int32_t H, E, k, I;
  int32_t score;      // 0 softmax, 1 sigmoid   (colibri_core::RouterScore)
  int32_t norm_topk;  // cfg.norm_topk
  float routed_scale;
  int32_t n_group, topk_group;  // 1/1 = ungrouped (the only mode the reference has)
  int32_t fmt;                  // ORC_FMT_NVFP4 or ORC_FMT_FP8_B128
  int32_t has_shared;
  const uint16_t *router_w;  // bf16 [E,H]
  const float *select_bias;  // [E] or NULL; sigmoid arm: selection only
  const float *logit_bias;   // [E] or NULL; extension, added to the logits
  // Per-expert pointer tables with E (+1 when has_shared, the shared expert last) entries;
  // an expert that is never routed to may be NULL.
  // NVFP4: q = nibbles [O, K/2], s = ue4m3 bytes [O, K/16], g = f32 per matrix.
  // MXFP4: q = nibbles [O, K/2], s = E8M0 bytes [O, K/32], g = f32 per matrix (1.0 in real containers).
  // FP8_B128: q = codes [O, K], s = f32 [ceil(O/128), ceil(K/128)], g unused.
  const uint8_t *const *gate_q, *const *up_q, *const *down_q;
  const void *const *gate_s, *const *up_s, *const *down_s;
  const float *gate_g, *up_g, *down_g;
} OrcLayer;

// ---- codecs (thin exports of the shared header, so Python can pin them) ---------------
uint8_t orc_f32_to_e4m3(float x) { return coli_f32_to_e4m3(x); }
float orc_e4m3_to_f32(uint8_t b) { return coli_e4m3_to_f32(b); }
uint8_t orc_e2m1_code(float t) { return coli_e2m1_code(t); }
float orc_e2m1_to_f32(uint8_t n) { return coli_e2m1_to_f32(n); }
uint16_t orc_f32_to_bf16(float v) { return coli_f32_to_bf16(v); }
float orc_bf16_to_f32(uint16_t h) { return coli_bf16_to_f32(h); }
float orc_e8m0_to_f32(uint8_t b) { return e8m0_to_f32(b); }
float orc_expf(float x) { return coli_expf(x); }
float orc_sigmoidf(float x) { return coli_sigmoidf(x); }
float orc_siluf(float x) { return coli_siluf(x); }
void orc_expf_array(const float *x, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = coli_expf(x[i]);
}

// ---- quantisers ------------------------------------------------------------------------
// crates/colibri-engine/src/convert.rs:1107-1135 (quantize_nvfp4).
void orc_quantize_nvfp4(const float *w, int o, int i, uint8_t *nib, uint8_t *bsc, float *global_out) {
  float amax = 0.0f;
  for (int64_t j = 0; j < (int64_t)o * i; ++j) amax = std::max(amax, std::fabs(w[j]));
  const float global = coli_nvfp4_global(amax);
  const int nb = (i + 15) / 16, rb = (i + 1) / 2;
  memset(nib, 0, (size_t)o * rb);
  parallel_for(o, [&](int r) {
    for (int b = 0; b < nb; ++b) {
      const int c0 = b * 16, c1 = std::min((b + 1) * 16, i);
      float bmax = 0.0f;
      for (int c = c0; c < c1; ++c) bmax = std::max(bmax, std::fabs(w[(int64_t)r * i + c]));
      const uint8_t code = coli_nvfp4_block_code(bmax, global);
      bsc[(int64_t)r * nb + b] = code;
      for (int c = c0; c < c1; ++c) {
        const uint8_t cd = coli_nvfp4_nibble(w[(int64_t)r * i + c], code, global);
        nib[(int64_t)r * rb + (c >> 1)] |= (c & 1) ? (uint8_t)(cd << 4) : cd;
      }
    }
  });
  *global_out = global;
}

// Encoder for the 128x128 block-scaled FP8 form (decode rule convert.rs:731-741; the
// encoder rule is stated in coli_math.h).
void orc_quantize_fp8_b128(const float *w, int o, int i, uint8_t *codes, float *scales) {
  const int nbo = (o + 127) / 128, nbi = (i + 127) / 128;
  parallel_for(nbo * nbi, [&](int blk) {
      const int bo = blk / nbi, bi = blk % nbi;
      float amax = 0.0f;
      const int r1 = std::min((bo + 1) * 128, o), c1 = std::min((bi + 1) * 128, i);
      for (int r = bo * 128; r < r1; ++r)
        for (int c = bi * 128; c < c1; ++c) amax = std::max(amax, std::fabs(w[(int64_t)r * i + c]));
      const float s = coli_fp8_block_scale(amax);
      scales[bo * nbi + bi] = s;
      for (int r = bo * 128; r < r1; ++r)
        for (int c = bi * 128; c < c1; ++c)
          codes[(int64_t)r * i + c] = coli_fp8_block_code(w[(int64_t)r * i + c], s);
  });
}

// ---- dequant-matmul ---------------------------------------------------------------------
// Decode one weight row to the f32 values the reference multiplies by x[k]:
//   NVFP4   E2M1[nib] * e4m3(bs[k/16])            (linear.rs:110-133; the tensor scale g is
//                                                   applied once per output, after the sum)
//   E4M3_ROW e4m3(w)                               (linear.rs:93-109; row scale after the sum)
//   FP8_B128 e4m3(w) * scale[(o/128)*nbi + k/128]  (convert.rs:731-741, then an f32 matmul)
// MXFP4 encoder of the reference's benchmark (crates/colibri-engine/src/gpubench.rs:84-119): per
// block of 32 the smallest power of two 2^e with bmax / 2^e <= 6 (e = ceil(log2(bmax / 6)),
// clamped to +-127, 0 for an all-zero block), scale byte 127 + e, nibble = nearest E2M1 level of
// w / 2^e (first minimum wins, convert.rs:1078-1090).  No global scale (g = 1.0).
void orc_quantize_mxfp4(const float *w, int o, int i, uint8_t *nib, uint8_t *bsc) {
  const int nb = (i + 31) / 32, rb = (i + 1) / 2;
  memset(nib, 0, (size_t)o * rb);
  parallel_for(o, [&](int r) {
    for (int b = 0; b < nb; ++b) {
      const int c0 = b * 32, c1 = std::min((b + 1) * 32, i);
      float bmax = 0.0f;
      for (int c = c0; c < c1; ++c) bmax = std::max(bmax, std::fabs(w[(int64_t)r * i + c]));
      int e = bmax > 0.0f ? (int)ceilf(log2f(bmax / 6.0f)) : 0;
      e = std::max(-127, std::min(127, e));
      bsc[(int64_t)r * nb + b] = (uint8_t)(127 + e);
      const float sc = exp2f((float)e);
      for (int c = c0; c < c1; ++c) {
        const uint8_t code = coli_e2m1_code(w[(int64_t)r * i + c] / sc);
        nib[(int64_t)r * rb + (c >> 1)] |= (c & 1) ? (uint8_t)(code << 4) : code;
      }
    }
  });
}

static void decode_row(int fmt, const uint8_t *q, const void *s, int row, int K, float *wr) {
  if (fmt == ORC_FMT_NVFP4) {
    const int rb = (K + 1) / 2, nb = (K + 15) / 16;
    const uint8_t *qr = q + (int64_t)row * rb;
    const uint8_t *br = (const uint8_t *)s + (int64_t)row * nb;
    for (int k = 0; k < K; ++k) {
      const uint8_t byte = qr[k >> 1];
      const uint8_t n = (k & 1) ? (byte >> 4) : (byte & 0x0f);
      wr[k] = coli_e2m1_to_f32(n) * coli_e4m3_to_f32(br[k >> 4]);
    }
  } else if (fmt == ORC_FMT_MXFP4) {
    // linear.rs:134-175: W[o,k] = E2M1[nib] * 2^(bs[o*nb + k/32] - 127), block scales decoded once per row
    const int rb = (K + 1) / 2, nb = (K + 31) / 32;
    const uint8_t *qr = q + (int64_t)row * rb;
    const uint8_t *br = (const uint8_t *)s + (int64_t)row * nb;
    for (int k = 0; k < K; ++k) {
      const uint8_t byte = qr[k >> 1];
      const uint8_t n = (k & 1) ? (byte >> 4) : (byte & 0x0f);
      wr[k] = coli_e2m1_to_f32(n) * e8m0_to_f32(br[k >> 5]);
    }
  } else if (fmt == ORC_FMT_E4M3_ROW) {
    const uint8_t *qr = q + (int64_t)row * K;
    for (int k = 0; k < K; ++k) wr[k] = coli_e4m3_to_f32(qr[k]);
  } else if (fmt == ORC_FMT_FP8_B128) {
    const int nbi = (K + 127) / 128;
    const uint8_t *qr = q + (int64_t)row * K;
    const float *sr = (const float *)s + (int64_t)(row / 128) * nbi;
    for (int k = 0; k < K; ++k) wr[k] = coli_e4m3_to_f32(qr[k]) * sr[k >> 7];
  } else {  // f32
    memcpy(wr, (const float *)q + (int64_t)row * K, sizeof(float) * K);
  }
}

// y[S,O] = x[S,K] @ W[O,K]^T with a strictly k-ascending f32 sum per output
// (linear.rs:18-175,199-220).  Tokens are accumulated side by side in blocks of 8, 4, 2 or 1
// (independent accumulators, so each output is still the reference's sequential sum; a block is
// never wider than the tokens left, so a one-row call does one row's arithmetic); rows of W are
// spread over threads (disjoint outputs).
extern "C++" {
template <int W>
static inline void dot_block(const float *wr, const float *xp, int K, float *acc) {
  for (int j = 0; j < W; ++j) acc[j] = 0.0f;
  for (int k = 0; k < K; ++k) {
    const float wv = wr[k];
    for (int j = 0; j < W; ++j) acc[j] += wv * xp[(size_t)k * W + j];
  }
}
}
void orc_matmul_qt(int fmt, const uint8_t *q, const void *s, float g, const float *x, float *y, int S,
                   int K, int O) {
  // token blocks: as many of 8 as fit, then one each of 4, 2, 1 for the remainder
  struct Blk { int s0, w; size_t off; };
  std::vector<Blk> blks;
  size_t total = 0;
  for (int s0 = 0; s0 < S;) {
    const int left = S - s0, w = left >= 8 ? 8 : left >= 4 ? 4 : left >= 2 ? 2 : 1;
    blks.push_back({s0, w, total});
    total += (size_t)K * w;
    s0 += w;
  }
  std::vector<float> xb(total);  // per block [k][w]
  for (const Blk &b : blks)
    for (int j = 0; j < b.w; ++j)
      for (int k = 0; k < K; ++k) xb[b.off + (size_t)k * b.w + j] = x[(size_t)(b.s0 + j) * K + k];
  // rows in chunks of 16 so each task amortises its scratch row
  const int nchunk = (O + 15) / 16;
  parallel_for(nchunk, [&](int ch) {
    std::vector<float> wr(K);
    for (int row = ch * 16; row < std::min(O, ch * 16 + 16); ++row) {
      decode_row(fmt, q, s, row, K, wr.data());
      float rs = 1.0f;
      const bool scaled = fmt == ORC_FMT_NVFP4 || fmt == ORC_FMT_MXFP4 || fmt == ORC_FMT_E4M3_ROW;
      if (fmt == ORC_FMT_NVFP4 || fmt == ORC_FMT_MXFP4) rs = g;
      if (fmt == ORC_FMT_E4M3_ROW) rs = ((const float *)s)[row];
      for (const Blk &b : blks) {
        float acc[8];
        const float *xp = &xb[b.off];
        switch (b.w) {
          case 8: dot_block<8>(wr.data(), xp, K, acc); break;
          case 4: dot_block<4>(wr.data(), xp, K, acc); break;
          case 2: dot_block<2>(wr.data(), xp, K, acc); break;
          default: dot_block<1>(wr.data(), xp, K, acc); break;
        }
        for (int j = 0; j < b.w; ++j) y[(size_t)(b.s0 + j) * O + row] = scaled ? acc[j] * rs : acc[j];
      }
    }
  });
}

// RMSNorm of one row: mean square accumulated left to right in f64, the scale and the products in
// f32, (x * r) * w (math.rs:8-20).
void orc_rmsnorm(float *out, const float *x, const float *w, int d, float eps) {
  double ms = 0.0;
  for (int k = 0; k < d; ++k) ms += (double)x[k] * (double)x[k];
  const float r = 1.0f / sqrtf((float)(ms / (double)d) + eps);
  for (int k = 0; k < d; ++k) out[k] = x[k] * r * w[k];
}

// Process-wide activation setting, as the reference keeps it (gpu::set_activation, moe.rs:103).
static int g_orc_oai = 0;
static float g_orc_alpha = 1.702f, g_orc_limit = 0.0f;
void orc_set_activation(int oai, float alpha, float limit) {
  g_orc_oai = oai;
  g_orc_alpha = alpha;
  g_orc_limit = limit;
}
float orc_act_combine(float g, float u, int oai, float alpha, float limit) { return coli_act_combine(g, u, oai, alpha, limit); }

// Gated FFN of one expert over nr rows (moe.rs:1187-1230: SiLU, clamped and OpenAI arms).
static void ffn(const OrcLayer *L, int ei, const float *x, int nr, float *out) {
  const int H = L->H, I = L->I;
  if (!L->gate_q[ei] || !L->up_q[ei] || !L->down_q[ei]) {
    fprintf(stderr, "oracle: expert %d was routed to but has no weights\n", ei);
    abort();
  }
  const float gg = L->gate_g ? L->gate_g[ei] : 1.0f, ug = L->up_g ? L->up_g[ei] : 1.0f,
              dg = L->down_g ? L->down_g[ei] : 1.0f;
  std::vector<float> g((size_t)nr * I), u((size_t)nr * I);
  orc_matmul_qt(L->fmt, L->gate_q[ei], L->gate_s[ei], gg, x, g.data(), nr, H, I);
  orc_matmul_qt(L->fmt, L->up_q[ei], L->up_s[ei], ug, x, u.data(), nr, H, I);
  for (size_t j = 0; j < g.size(); ++j) g[j] = coli_act_combine(g[j], u[j], g_orc_oai, g_orc_alpha, g_orc_limit);
  orc_matmul_qt(L->fmt, L->down_q[ei], L->down_s[ei], dg, g.data(), out, nr, I, H);
}

void orc_expert_ffn(const OrcLayer *L, int ei, const float *x, int nr, float *out) { ffn(L, ei, x, nr, out); }

// ---- routing ----------------------------------------------------------------------------
// k rounds of a strict-`>` scan from e = 0 (lowest id wins a tie); a round in which nothing
// beats -inf picks expert 0 again, as the reference's loop does (moe.rs:1075-1088,1109-1122).
static void topk_scan(const float *choice, const uint8_t *allowed, int E, int k, int32_t *idx) {
  std::vector<uint8_t> chosen(E, 0);
  for (int kk = 0; kk < k; ++kk) {
    int best = 0;
    float bv = -std::numeric_limits<float>::infinity();
    for (int e = 0; e < E; ++e) {
      if (allowed && !allowed[e]) continue;
      if (!chosen[e] && choice[e] > bv) {
        bv = choice[e];
        best = e;
      }
    }
    chosen[best] = 1;
    idx[kk] = best;
  }
}

// One token.  `logits` already holds router·x (+ logit_bias).  moe.rs:1047-1132.
// n_group > 1 (not in the reference): experts form n_group contiguous groups; a group's
// score is the sum of its two largest selection scores; the topk_group best groups are kept
// (ties -> lowest group id); the top-k scan then runs over experts of kept groups only.
void orc_route(const OrcLayer *L, const float *logits, int32_t *idx, float *w) {
  const int E = L->E, k = std::min(L->k, L->E);
  std::vector<float> score(E), choice(E);
  if (L->score == 0) {
    float mx = -std::numeric_limits<float>::infinity();
    for (int e = 0; e < E; ++e) mx = std::max(mx, logits[e]);
    float tot = 0.0f;
    for (int e = 0; e < E; ++e) {
      score[e] = coli_expf(logits[e] - mx);
      tot += score[e];
    }
    if (tot > 0.0f)
      for (int e = 0; e < E; ++e) score[e] /= tot;
    choice = score;
  } else {
    for (int e = 0; e < E; ++e) {
      score[e] = coli_sigmoidf(logits[e]);
      choice[e] = score[e] + (L->select_bias ? L->select_bias[e] : 0.0f);
    }
  }
  std::vector<uint8_t> allowed;
  if (L->n_group > 1) {
    const int G = L->n_group, gs = E / G, kg = std::min(L->topk_group, G);
    std::vector<float> gscore(G);
    for (int g = 0; g < G; ++g) {
      float m1 = -std::numeric_limits<float>::infinity(), m2 = m1;
      for (int e = g * gs; e < (g + 1) * gs; ++e) {
        const float c = choice[e];
        if (c > m1) {
          m2 = m1;
          m1 = c;
        } else if (c > m2) {
          m2 = c;
        }
      }
      gscore[g] = m1 + m2;
    }
    std::vector<int32_t> gidx(kg);
    topk_scan(gscore.data(), nullptr, G, kg, gidx.data());
    allowed.assign(E, 0);
    for (int j = 0; j < kg; ++j)
      for (int e = gidx[j] * gs; e < (gidx[j] + 1) * gs; ++e) allowed[e] = 1;
  }
  topk_scan(choice.data(), allowed.empty() ? nullptr : allowed.data(), E, k, idx);
  for (int kk = 0; kk < k; ++kk) w[kk] = score[idx[kk]];
  if (L->norm_topk) {
    float sm = 0.0f;
    for (int kk = 0; kk < k; ++kk) sm += w[kk];
    sm += 1e-20f;
    for (int kk = 0; kk < k; ++kk) w[kk] /= sm;
  }
  for (int kk = 0; kk < k; ++kk) w[kk] *= L->routed_scale;
}

// logits[T,E] = x·W_r^T, k-ascending f32 sum (moe.rs:1589-1604; linear.rs:199-220), on the
// bf16 inputs widened to f32, plus the logit_bias extension.
void orc_router_logits(const OrcLayer *L, const uint16_t *x, int T, float *logits) {
  const int H = L->H, E = L->E;
  parallel_for(T, [&](int t) {
    std::vector<float> xf(H);
    for (int h = 0; h < H; ++h) xf[h] = coli_bf16_to_f32(x[(size_t)t * H + h]);
    for (int e = 0; e < E; ++e) {
      float acc = 0.0f;
      const uint16_t *wr = L->router_w + (size_t)e * H;
      for (int h = 0; h < H; ++h) acc += xf[h] * coli_bf16_to_f32(wr[h]);
      if (L->logit_bias) acc += L->logit_bias[e];
      logits[(size_t)t * E + e] = acc;
    }
  });
}

void orc_route_tokens(const OrcLayer *L, const uint16_t *x, int T, int32_t *idx, float *w) {
  std::vector<float> logits((size_t)T * L->E);
  orc_router_logits(L, x, T, logits.data());
  const int k = std::min(L->k, L->E);
  parallel_for(T, [&](int t) { orc_route(L, &logits[(size_t)t * L->E], idx + (size_t)t * k, w + (size_t)t * k); });
}

// ---- the block --------------------------------------------------------------------------
// moe.rs:1799-1895 with the expert loop of moe.rs:1339-1564: route every token; experts in
// first-appearance order (moe.rs:1243-1267); per expert the rows with non-zero weight in
// ascending token order (moe.rs:1373-1387); out[t] += w * ffn(x[t]) (moe.rs:1549-1553); the
// shared expert over all rows added last (moe.rs:1868-1885).  When `owner` is given
// (expert-parallel, moe.rs:1620-1734) each rank's experts accumulate into that rank's own
// partial, and partials are folded in ascending rank order before the shared expert.
// x, out: bf16 [T,H]; idx/w: [T,k] (outputs, may be NULL); out_f32 optional [T,H].
int orc_moe_block(const OrcLayer *L, const uint16_t *x, uint16_t *out, int T, int32_t *idx_out, float *w_out,
                  float *out_f32, int world, const int32_t *owner) {
  const int H = L->H, E = L->E, k = std::min(L->k, L->E);
  if (T <= 0) return 1;
  std::vector<float> xf((size_t)T * H);
  for (size_t j = 0; j < xf.size(); ++j) xf[j] = coli_bf16_to_f32(x[j]);
  std::vector<int32_t> idx((size_t)T * k);
  std::vector<float> w((size_t)T * k);
  orc_route_tokens(L, x, T, idx.data(), w.data());
  if (idx_out) memcpy(idx_out, idx.data(), sizeof(int32_t) * idx.size());
  if (w_out) memcpy(w_out, w.data(), sizeof(float) * w.size());

  // union_and_weights
  std::vector<int> seen(E, -1), uniq;
  for (size_t j = 0; j < idx.size(); ++j)
    if (seen[idx[j]] < 0) {
      seen[idx[j]] = (int)uniq.size();
      uniq.push_back(idx[j]);
    }
  const int nu = (int)uniq.size();
  std::vector<float> wmat((size_t)T * nu, 0.0f);
  for (int t = 0; t < T; ++t)
    for (int kk = 0; kk < k; ++kk) wmat[(size_t)t * nu + seen[idx[(size_t)t * k + kk]]] = w[(size_t)t * k + kk];

  if (world < 1) world = 1;
  std::vector<std::vector<float>> partial(world);
  for (int r = 0; r < world; ++r) partial[r].assign((size_t)T * H, 0.0f);
  std::vector<float> xg, hh;
  for (int ui = 0; ui < nu; ++ui) {
    const int e = uniq[ui];
    std::vector<int> rows;
    std::vector<float> rw;
    for (int t = 0; t < T; ++t) {
      const float wt = wmat[(size_t)t * nu + ui];
      if (wt != 0.0f) {
        rows.push_back(t);
        rw.push_back(wt);
      }
    }
    if (rows.empty()) continue;
    const int nr = (int)rows.size();
    xg.resize((size_t)nr * H);
    hh.resize((size_t)nr * H);
    for (int r = 0; r < nr; ++r) memcpy(&xg[(size_t)r * H], &xf[(size_t)rows[r] * H], sizeof(float) * H);
    ffn(L, e, xg.data(), nr, hh.data());
    int rk = 0;
    if (world > 1) rk = owner ? owner[e] : (int)((int64_t)e * world / E);  // sharding.rs:197-203
    float *po = partial[rk].data();
    for (int r = 0; r < nr; ++r) {
      const float wt = rw[r];
      const int t = rows[r];
      for (int d = 0; d < H; ++d) po[(size_t)t * H + d] += wt * hh[(size_t)r * H + d];
    }
  }
  std::vector<float> acc = partial[0];
  if (world > 1) {
    std::fill(acc.begin(), acc.end(), 0.0f);
    for (int r = 0; r < world; ++r)
      for (size_t j = 0; j < acc.size(); ++j) acc[j] += partial[r][j];
  }
  if (L->has_shared) {
    std::vector<float> sh((size_t)T * H);
    ffn(L, E, xf.data(), T, sh.data());
    for (size_t j = 0; j < acc.size(); ++j) acc[j] += sh[j];
  }
  if (out_f32) memcpy(out_f32, acc.data(), sizeof(float) * acc.size());
  if (out)
    for (size_t j = 0; j < acc.size(); ++j) out[j] = coli_f32_to_bf16(acc[j]);
  return 1;
}

void orc_set_threads(int n) { g_threads = n > 0 ? n : 1; }
int orc_get_threads(void) { return g_threads; }
int orc_hardware_threads(void) { return (int)std::max(1u, std::thread::hardware_concurrency()); }

// FNV-1a over (num_nodes, n_experts, owner(0..E)) — crates/colibri-cluster/src/sharding.rs:251-265.
uint64_t orc_sharding_fingerprint(uint32_t num_nodes, uint32_t n_experts, const uint32_t *owner) {
  uint64_t h = 0xcbf29ce484222325ull;
  auto mix = [&](uint32_t v) {
    for (int b = 0; b < 4; ++b) {
      h ^= (uint64_t)((v >> (8 * b)) & 0xff);
      h *= 0x00000100000001b3ull;
    }
  };
  mix(num_nodes);
  mix(n_experts);
  for (uint32_t e = 0; e < n_experts; ++e) mix(owner ? owner[e] : (uint32_t)((uint64_t)e * num_nodes / n_experts));
  return h;
}

}  // extern "C"
