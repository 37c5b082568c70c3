// Weight layout: repack between the reference's row-major container layouts
// (crates/colibri-core/src/quant.rs:707-781: NVFP4 nibbles [O, ceil(I/2)] low nibble = even
// column + ue4m3 block scales [O, ceil(I/16)]; e4m3 codes [O, I]) and the k-tile-major HBM layout
// described in internal.cuh, plus the device-side quantisers.
#include "internal.cuh"

namespace colib {

// ---- NVFP4 ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t nib_at(const uint8_t *nib, int rb, int row, int k, int O, int I) {
  if (row >= O || k >= I) return 0u;
  const uint8_t b = nib[(size_t)row * rb + (k >> 1)];
  return (k & 1) ? (uint32_t)(b >> 4) : (uint32_t)(b & 0x0f);
}

// one thread per 32-bit word of the packed array: (kt, row, word j) covers k = kt*128 + 8j .. +7,
// k ascending from the least significant nibble (the container's own order: byte = two
// consecutive k, low nibble first, which is what cvt.rn.f16x2.e2m1x2 consumes)
__global__ void k_pack_nvfp4_q(const uint8_t *nib, uint32_t *q, int O, int I, int Op, int KT) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)KT * Op * 16;
  if (idx >= total) return;
  const int j = (int)(idx % 16);
  const int row = (int)((idx / 16) % Op);
  const int kt = (int)(idx / 16 / Op);
  const int rb = (I + 1) / 2;
  const int k0 = kt * 128 + j * 8;
  uint32_t w = 0;
#pragma unroll
  for (int el = 0; el < 8; ++el) w |= nib_at(nib, rb, row, k0 + el, O, I) << (4 * el);
  q[idx] = w;
}
__global__ void k_pack_nvfp4_s(const uint8_t *bs, uint8_t *s, int O, int I, int Op, int KT) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)KT * Op * 8;
  if (idx >= total) return;
  const int b = (int)(idx % 8);
  const int row = (int)((idx / 8) % Op);
  const int kt = (int)(idx / 8 / Op);
  const int nb = (I + 15) / 16, kb = kt * 8 + b;
  s[idx] = (row < O && kb < nb) ? bs[(size_t)row * nb + kb] : (uint8_t)0;
}
// inverse: one thread per output byte of the row-major nibble array / scale array
__global__ void k_unpack_nvfp4_q(const uint32_t *q, uint8_t *nib, int O, int I, int Op) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int rb = (I + 1) / 2;
  if (idx >= (size_t)O * rb) return;
  const int row = (int)(idx / rb), byte = (int)(idx % rb);
  uint32_t out = 0;
  for (int h = 0; h < 2; ++h) {
    const int k = byte * 2 + h;
    if (k >= I) break;
    const int kt = k >> 7, j = (k & 127) >> 3, el = k & 7;
    const uint32_t w = q[((size_t)kt * Op + row) * 16 + j];
    out |= ((w >> (4 * el)) & 0xfu) << (4 * h);
  }
  nib[idx] = (uint8_t)out;
}
__global__ void k_unpack_nvfp4_s(const uint8_t *s, uint8_t *bs, int O, int I, int Op) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int nb = (I + 15) / 16;
  if (idx >= (size_t)O * nb) return;
  const int row = (int)(idx / nb), kb = (int)(idx % nb);
  bs[idx] = s[((size_t)(kb >> 3) * Op + row) * 8 + (kb & 7)];
}

// ---- FP8 ---------------------------------------------------------------------------------------
// bytes stay in k order: a 16-bit half word is one (k, k+1) pair for cvt.rn.f16x2.e4m3x2
__global__ void k_pack_fp8(const uint8_t *codes, uint8_t *q, int O, int I, int Op, int KT) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)KT * Op * 128;
  if (idx >= total) return;
  const int j = (int)(idx % 128);
  const int row = (int)((idx / 128) % Op);
  const int kt = (int)(idx / 128 / Op);
  const int k = kt * 128 + j;
  const uint8_t v = (row < O && k < I) ? codes[(size_t)row * I + k] : (uint8_t)0;
  q[idx] = v;
}
__global__ void k_unpack_fp8(const uint8_t *q, uint8_t *codes, int O, int I, int Op) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)O * I) return;
  const int row = (int)(idx / I), k = (int)(idx % I);
  const int kt = k >> 7, j = k & 127;
  codes[idx] = q[((size_t)kt * Op + row) * 128 + j];
}

static inline unsigned nblk(size_t n, int b) { return (unsigned)((n + b - 1) / b); }

int pack_nvfp4(const uint8_t *d_nib, const uint8_t *d_bs, int O, int I, ColiCudaTensor *t, cudaStream_t st) {
  k_pack_nvfp4_q<<<nblk((size_t)t->KT * t->Op * 16, 256), 256, 0, st>>>(d_nib, (uint32_t *)t->q, O, I, t->Op, t->KT);
  coli_count_launch(1);
  k_pack_nvfp4_s<<<nblk((size_t)t->KT * t->Op * 8, 256), 256, 0, st>>>(d_bs, t->s, O, I, t->Op, t->KT);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "nvfp4 repack") ? 1 : 0;
}
int pack_fp8(const uint8_t *d_codes, int O, int I, ColiCudaTensor *t, cudaStream_t st) {
  k_pack_fp8<<<nblk((size_t)t->KT * t->Op * 128, 256), 256, 0, st>>>(d_codes, t->q, O, I, t->Op, t->KT);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "fp8 repack") ? 1 : 0;
}
int unpack_nvfp4(const ColiCudaTensor *t, uint8_t *d_nib, uint8_t *d_bs, cudaStream_t st) {
  const int rb = (t->I + 1) / 2, nb = (t->I + 15) / 16;
  k_unpack_nvfp4_q<<<nblk((size_t)t->O * rb, 256), 256, 0, st>>>((const uint32_t *)t->q, d_nib, t->O, t->I, t->Op);
  coli_count_launch(1);
  k_unpack_nvfp4_s<<<nblk((size_t)t->O * nb, 256), 256, 0, st>>>(t->s, d_bs, t->O, t->I, t->Op);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "nvfp4 export") ? 1 : 0;
}
int unpack_fp8(const ColiCudaTensor *t, uint8_t *d_codes, cudaStream_t st) {
  k_unpack_fp8<<<nblk((size_t)t->O * t->I, 256), 256, 0, st>>>(t->q, d_codes, t->O, t->I, t->Op);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "fp8 export") ? 1 : 0;
}

// ---- quantisers ----------------------------------------------------------------------------------
// |w| maximum: non-negative floats order like their bit patterns, so an integer atomicMax works.
__global__ void k_amax(const float *w, size_t n, unsigned int *amax_bits) {
  float m = 0.0f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(w[i]));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));
}
// one thread per 16-wide block (convert.rs:1114-1133)
__global__ void k_quant_nvfp4(const float *w, int O, int I, uint8_t *nib, uint8_t *bsc, const float *amax) {
  const int nb = (I + 15) / 16, rb = (I + 1) / 2;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)O * nb) return;
  const int r = (int)(idx / nb), b = (int)(idx % nb);
  const float global = coli_nvfp4_global(*amax);
  const int c0 = b * 16, c1 = min(c0 + 16, I);
  const float *wr = w + (size_t)r * I;
  float bmax = 0.0f;
  for (int c = c0; c < c1; ++c) bmax = fmaxf(bmax, fabsf(wr[c]));
  const uint8_t code = coli_nvfp4_block_code(bmax, global);
  bsc[idx] = code;
  for (int c = c0; c < c1; c += 2) {
    uint8_t lo = coli_nvfp4_nibble(wr[c], code, global);
    uint8_t hi = (c + 1 < c1) ? coli_nvfp4_nibble(wr[c + 1], code, global) : (uint8_t)0;
    nib[(size_t)r * rb + (c >> 1)] = (uint8_t)(lo | (hi << 4));
  }
}
int quantize_nvfp4(const float *d_w, int O, int I, uint8_t *d_nib, uint8_t *d_bs, float *d_amax_scratch,
                   float *gscale_out, cudaStream_t st) {
  if (!coli_cuda_check(cudaMemsetAsync(d_amax_scratch, 0, sizeof(float), st), "amax clear")) return 0;
  const size_t n = (size_t)O * I;
  k_amax<<<(unsigned)((n + 256 * 8 - 1) / (256 * 8) > 1184 ? 1184 : (n + 256 * 8 - 1) / (256 * 8)), 256, 0, st>>>(
      d_w, n, (unsigned int *)d_amax_scratch);
  coli_count_launch(1);
  const size_t blocks = (size_t)O * ((I + 15) / 16);
  k_quant_nvfp4<<<nblk(blocks, 128), 128, 0, st>>>(d_w, O, I, d_nib, d_bs, d_amax_scratch);
  coli_count_launch(1);
  if (!coli_cuda_check(cudaGetLastError(), "nvfp4 quantise")) return 0;
  float amax = 0.0f;
  if (!coli_cuda_check(cudaMemcpyAsync(&amax, d_amax_scratch, sizeof(float), cudaMemcpyDeviceToHost, st), "amax read"))
    return 0;
  if (!coli_cuda_check(cudaStreamSynchronize(st), "nvfp4 quantise sync")) return 0;
  *gscale_out = coli_nvfp4_global(amax);
  return 1;
}

// one CTA per 128x128 block
__global__ void __launch_bounds__(256) k_quant_fp8_b128(const float *w, int O, int I, uint8_t *codes,
                                                        float *scales) {
  __shared__ float red[8];
  const int nbi = (I + 127) / 128;
  const int bo = blockIdx.x / nbi, bi = blockIdx.x % nbi;
  const int r0 = bo * 128, c0 = bi * 128;
  float m = 0.0f;
  for (int idx = threadIdx.x; idx < 128 * 128; idx += 256) {
    const int r = r0 + idx / 128, c = c0 + idx % 128;
    if (r < O && c < I) m = fmaxf(m, fabsf(w[(size_t)r * I + c]));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  const float s = coli_fp8_block_scale(m);
  if (threadIdx.x == 0) scales[blockIdx.x] = s;
  for (int idx = threadIdx.x; idx < 128 * 128; idx += 256) {
    const int r = r0 + idx / 128, c = c0 + idx % 128;
    if (r < O && c < I) codes[(size_t)r * I + c] = coli_fp8_block_code(w[(size_t)r * I + c], s);
  }
}
int quantize_fp8_b128(const float *d_w, int O, int I, uint8_t *d_codes, float *d_scales, cudaStream_t st) {
  const int nbo = (O + 127) / 128, nbi = (I + 127) / 128;
  k_quant_fp8_b128<<<nbo * nbi, 256, 0, st>>>(d_w, O, I, d_codes, d_scales);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "fp8 quantise") ? 1 : 0;
}

}  // namespace colib
