// Pieces shared by the tcgen05 expert kernels: PTX wrappers (mbarrier, TMA, tcgen05), bounded waits,
// UMMA descriptors, the NVFP4 -> f16 conversion, and the host-side tensor map for token rows.
#pragma once
#include <cuda.h>

#include "internal.cuh"

namespace colib {

constexpr int TC_BM = 128;   // features per tile (UMMA M)
constexpr int TC_BK = 64;    // k per pipeline stage: one 128-byte swizzle row of f16
constexpr int TC_BOXN = 32;  // token rows per TMA box
constexpr int TC_EPI_WARPS = 4;

constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

enum { TC_OK = 0, TC_ERR_TMA_WAIT = 1, TC_ERR_MMA_WAIT = 2, TC_ERR_PROD_WAIT = 3, TC_ERR_EPI_WAIT = 4 };

// ---- PTX wrappers ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait with a suspend-time hint: the thread stays suspended in hardware (taking no issue slots)
// until the phase completes or about `ns` nanoseconds have passed
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the barrier did not flip in time or another role gave up.
// sleep_ns = 0 polls with test_wait (never suspends); otherwise every poll is a try_wait that the
// hardware suspends for up to max(sleep_ns, 1000) ns or until the phase completes.  A waiting warp
// must not spin: the trace of the tensor-memory kernel showed twenty polling warps taking four
// fifths of the issue slots from the one warp per scheduler that had work (the epilogue ran at a
// tenth of an instruction per cycle, the MMA-issuing threads lost ~500 cycles per stage).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code,
                                          uint32_t sleep_ns = 0) {
  const uint32_t hint = sleep_ns > 1000u ? sleep_ns : 1000u;
  const uint32_t limit = sleep_ns ? (TC_SPIN_LIMIT >> 4) : TC_SPIN_LIMIT;  // at most ~0.3 s of suspended polls
  for (uint32_t i = 0; i < limit; ++i) {
    if (sleep_ns ? mbar_try_wait_hint(bar, parity, hint) : mbar_test_wait(bar, parity)) return true;
    if ((i & 7u) == 7u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(status, TC_OK, code);
  return false;
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;          // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;          // descriptor version of this architecture
  d |= (uint64_t)2 << 61;          // SWIZZLE_128B
  return d;
}
// kind::f16: D = f32, A = B = f16 (format code 0), both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ uint32_t tc_hmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// One NVFP4 word (8 consecutive k, two per byte, low nibble first) -> 8 f16 (four f16x2, k
// ascending) times the block scale held in both halves of `mult`.
__device__ __forceinline__ uint4 tc_dequant_word(uint32_t w, uint32_t mult) {
  uint4 o;
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      "  mov.b32 {b0, b1, b2, b3}, %4;\n"
      "  cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "  cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "  cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "  cvt.rn.f16x2.e2m1x2 %3, b3; }\n"
      : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
      : "r"(w));
  o.x = tc_hmul2(o.x, mult);
  o.y = tc_hmul2(o.y, mult);
  o.z = tc_hmul2(o.z, mult);
  o.w = tc_hmul2(o.w, mult);
  return o;
}
// two ue4m3 block scales (low 16 bits of sc) -> each as f16 in both halves of a word
__device__ __forceinline__ void tc_scales(uint32_t sc, uint32_t &m0, uint32_t &m1) {
  uint32_t v;
  asm("{ .reg .b16 h0, h1;\n"
      "  mov.b32 {h0, h1}, %1;\n"
      "  cvt.rn.f16x2.e4m3x2 %0, h0; }\n"
      : "=r"(v)
      : "r"(sc));
  m0 = __byte_perm(v, v, 0x1010);
  m1 = __byte_perm(v, v, 0x3232);
}

// ---- epilogue stores ------------------------------------------------------------------------------------
// An epilogue lane owns ONE feature (its TMEM lane) and 16 token columns of it, while the result
// matrices are token-major: written lane by lane, every value is a 2-byte store of its own, and
// those store instructions (32 per 16-column chunk of the down kernel) were what the epilogue
// spent its time on.  Instead the four lanes of a quad (features 4q .. 4q+3) exchange their values
// with two shuffles per four columns, so that lane r of the quad holds the four features of column
// 4g + r and writes them with one 8-byte store: a quarter of the store instructions.
__device__ __forceinline__ uint32_t tc_pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// two f32 -> each rounded to bf16, then held as f16 (saturating): the pair form of coli_f32_to_f16_via_bf16
__device__ __forceinline__ uint32_t tc_pack_f16x2_via_bf16(float lo, float hi) {
  const uint32_t b = tc_pack_bf16x2(lo, hi);
  const float rl = fminf(fmaxf(__uint_as_float(b << 16), -65504.0f), 65504.0f);
  const float rh = fminf(fmaxf(__uint_as_float(b & 0xffff0000u), -65504.0f), 65504.0f);
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(rh), "f"(rl));
  return d;
}
// pk[i] = the lane's values of columns 2i (low half) and 2i + 1 (high half), 16-bit each.
// quad_base = &out[first column of the chunk][feature of the quad's first lane], ld = elements
// per token row, cols_valid = how many of the 16 columns are rows of the item, feat_ok = the quad's
// features exist (feature counts are multiples of 8, so a quad is whole or absent).  Every lane of
// the warp must call this (shuffles).
template <typename T16>
__device__ __forceinline__ void tc_store_cols16(const uint32_t (&pk)[8], T16 *quad_base, size_t ld, int cols_valid, bool feat_ok,
                                                int lane) {
  static_assert(sizeof(T16) == 2, "16-bit elements");
  const bool odd = (lane & 1) != 0, hi2 = (lane & 2) != 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint32_t p01 = pk[2 * g], p23 = pk[2 * g + 1];
    // lanes 2j and 2j+1: the even lane keeps columns 0 and 2 of the group, the odd one 1 and 3
    const uint32_t send1 = odd ? __byte_perm(p01, p23, 0x5410) : __byte_perm(p01, p23, 0x7632);
    const uint32_t r1 = __shfl_xor_sync(0xffffffffu, send1, 1);
    const uint32_t xa = odd ? __byte_perm(p01, r1, 0x3254) : __byte_perm(p01, r1, 0x5410);  // features (even, odd) of column odd / 0
    const uint32_t xb = odd ? __byte_perm(p23, r1, 0x3276) : __byte_perm(p23, r1, 0x7610);  // ... of column 2 + odd
    // lanes j and j+2: the lower pair keeps column xa and takes the upper pair's features of it
    const uint32_t r2 = __shfl_xor_sync(0xffffffffu, hi2 ? xa : xb, 2);
    const uint32_t o0 = hi2 ? r2 : xa, o1 = hi2 ? xb : r2;
    const int col = 4 * g + (odd ? 1 : 0) + (hi2 ? 2 : 0);
    if (feat_ok && col < cols_valid) *reinterpret_cast<uint2 *>(quad_base + (size_t)col * ld) = make_uint2(o0, o1);
  }
}

// ---- host side ----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !ptr) {
      coli_set_error("cuTensorMapEncodeTiled is not available from the driver");
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// f16 [rows, K] row-major; box = 64 k x box_rows rows; 128-byte swizzle; out-of-range reads give zeros
static inline bool make_rows_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows = TC_BOXN) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (K % 8)) {
    coli_set_error("tensor map: row buffer must be 16-byte aligned with K a multiple of 8 (K=%d)", K);
    return false;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    coli_set_error("cuTensorMapEncodeTiled failed with code %d (rows=%d K=%d)", (int)r, rows, K);
    return false;
  }
  return true;
}

}  // namespace colib
