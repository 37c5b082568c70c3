// Weighted combine: out[t] = sum_kk w[t,kk] * y[slot[t,kk]] (kk ascending, f32) + shared[t],
// rounded once to bf16 — crates/colibri-engine/src/moe.rs:1549-1553 (routed accumulate),
// 1875-1885 (shared expert added after the routed sum).  A gather per output row instead of the
// reference's scatter-add, so the f32 order is fixed and no atomics are needed.  The order is a
// token's own kk order; the reference adds expert by expert in the batch's first-appearance order
// (moe.rs:1243-1267), so the two f32 sums agree to rounding (tolerance-level), not bit for bit.
#include "internal.cuh"

namespace colib {

__global__ void __launch_bounds__(256) k_combine(CombineParams p, const __nv_bfloat16 *shared_y) {
  coli_grid_dependency_sync();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;  // 8-element column group
  if (c * 8 >= p.H) return;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  // batches of 8 experts: all slots and weights, then all rows, are requested before the first
  // is used (a load-use loop would pay two memory round trips per expert); the sum itself runs
  // in ascending kk
  for (int k0 = 0; k0 < p.k; k0 += 8) {
    float w[8];
    int row[8];
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = k0 + j < p.k;
      w[j] = in ? p.topk_w[(size_t)t * p.k + k0 + j] : 0.0f;
      row[j] = in ? p.slot[(size_t)t * p.k + k0 + j] : -1;  // < 0: the expert lives on another rank, which adds its own partial
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = make_uint4(0, 0, 0, 0);
      if (row[j] >= 0) v[j] = *reinterpret_cast<const uint4 *>(p.y + (size_t)row[j] * p.H + c * 8);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (row[j] < 0) continue;
      const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] = fmaf(w[j], __uint_as_float(u[i] << 16), acc[2 * i]);
        acc[2 * i + 1] = fmaf(w[j], __uint_as_float(u[i] & 0xffff0000u), acc[2 * i + 1]);
      }
    }
  }
  if (shared_y) {
    const uint4 v = *reinterpret_cast<const uint4 *>(shared_y + (size_t)t * p.H + c * 8);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += __uint_as_float(u[i] << 16);
      acc[2 * i + 1] += __uint_as_float(u[i] & 0xffff0000u);
    }
  }
  if (p.resid) {  // x += moe(x): the residual add of the layer, in f32 (forward.rs:391-393)
    const float4 *r4 = reinterpret_cast<const float4 *>(p.resid + (size_t)t * p.H + c * 8);
    const float4 a = r4[0], b = r4[1];
    acc[0] = a.x + acc[0];
    acc[1] = a.y + acc[1];
    acc[2] = a.z + acc[2];
    acc[3] = a.w + acc[3];
    acc[4] = b.x + acc[4];
    acc[5] = b.y + acc[5];
    acc[6] = b.z + acc[6];
    acc[7] = b.w + acc[7];
  }
  if (p.out32) {  // f32 out: the partial sum of this rank's experts, or the new residual stream
    float4 *o32 = reinterpret_cast<float4 *>(p.out32 + (size_t)t * p.H + c * 8);
    o32[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o32[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    return;
  }
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = __bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * i]));
    const uint32_t hi = __bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * i + 1]));
    o[i] = lo | (hi << 16);
  }
  *reinterpret_cast<uint4 *>(p.out + (size_t)t * p.H + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

int launch_combine(const CombineParams &p, cudaStream_t st) {
  if (p.T <= 0) return 1;
  if (p.H % 8) {
    coli_set_error("combine: H=%d must be a multiple of 8", p.H);
    return 0;
  }
  const __nv_bfloat16 *shared_y = p.has_shared ? p.shared_y : nullptr;
  dim3 grid(p.T, (p.H / 8 + 255) / 256);
  coli_count_launch(1);
  return coli_cuda_check(launch_dependent(k_combine, grid, dim3(256), 0, st, p, shared_y), "combine launch") ? 1 : 0;
}

// out = bf16(partial + shared): the last step of the expert-parallel block
__global__ void __launch_bounds__(256) k_finish(const float *partial, const __nv_bfloat16 *shared_y, __nv_bfloat16 *out, size_t n8) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4 *>(partial)[2 * i], b = reinterpret_cast<const float4 *>(partial)[2 * i + 1];
  float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  if (shared_y) {
    const uint4 sv = reinterpret_cast<const uint4 *>(shared_y)[i];
    const uint32_t u[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] += __uint_as_float(u[j] << 16);
      v[2 * j + 1] += __uint_as_float(u[j] & 0xffff0000u);
    }
  }
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v[2 * j])) |
           ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v[2 * j + 1])) << 16);
  reinterpret_cast<uint4 *>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
}
int launch_finish(const float *partial, const __nv_bfloat16 *shared_y, __nv_bfloat16 *out, int T, int H, cudaStream_t st) {
  if (T <= 0) return 1;
  if (H % 8) {
    coli_set_error("finish: H=%d must be a multiple of 8", H);
    return 0;
  }
  const size_t n8 = (size_t)T * H / 8;
  k_finish<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(partial, shared_y, out, n8);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "finish launch") ? 1 : 0;
}

// One warp per token row.  Lane partial sums in f64, combined by a shuffle tree: not the
// reference's left-to-right order, but 53-bit partials of 24-bit squares differ from it by less
// than the f32 rounding of the mean in all but ~1e-9 of rows.
__global__ void __launch_bounds__(256) k_rmsnorm_bf16(const float *x, const float *w, float eps, __nv_bfloat16 *out, int T, int H) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= T) return;
  const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * H);
  const float4 *wr = reinterpret_cast<const float4 *>(w);
  double ms = 0.0;
  for (int i = lane; i < H / 4; i += 32) {
    const float4 v = xr[i];
    ms += (double)v.x * (double)v.x + (double)v.y * (double)v.y + (double)v.z * (double)v.z + (double)v.w * (double)v.w;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, off);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(ms / (double)H), eps)));
  uint2 *o = reinterpret_cast<uint2 *>(out + (size_t)row * H);
  for (int i = lane; i < H / 4; i += 32) {
    const float4 v = xr[i], g = wr[i];
    const uint32_t a = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(__fmul_rn(v.x, r), g.x)));
    const uint32_t b = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(__fmul_rn(v.y, r), g.y)));
    const uint32_t c = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(__fmul_rn(v.z, r), g.z)));
    const uint32_t d = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(__fmul_rn(v.w, r), g.w)));
    o[i] = make_uint2(a | (b << 16), c | (d << 16));
  }
}
int launch_rmsnorm_bf16(const float *x, const float *w, float eps, __nv_bfloat16 *out, int T, int H, cudaStream_t st) {
  if (T <= 0) return 1;
  if (H % 4) {
    coli_set_error("rmsnorm: H=%d must be a multiple of 4", H);
    return 0;
  }
  k_rmsnorm_bf16<<<(T + 7) / 8, 256, 0, st>>>(x, w, eps, out, T, H);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "rmsnorm launch") ? 1 : 0;
}

__global__ void k_f32_to_bf16(const float *src, __nv_bfloat16 *dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}
int launch_f32_to_bf16(const float *src, __nv_bfloat16 *dst, size_t n, cudaStream_t st) {
  if (n == 0) return 1;
  const size_t blocks = (n + 255) / 256;
  k_f32_to_bf16<<<(unsigned)(blocks > 4736 ? 4736 : blocks), 256, 0, st>>>(src, dst, n);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "f32->bf16 launch") ? 1 : 0;
}

__global__ void k_f32_to_f16(const float *src, __half *dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __float2half_rn(fminf(fmaxf(src[i], -65504.0f), 65504.0f));
}
int launch_f32_to_f16(const float *src, __half *dst, size_t n, cudaStream_t st) {
  if (n == 0) return 1;
  const size_t blocks = (n + 255) / 256;
  k_f32_to_f16<<<(unsigned)(blocks > 4736 ? 4736 : blocks), 256, 0, st>>>(src, dst, n);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "f32->f16 launch") ? 1 : 0;
}
__global__ void k_bf16_to_f32(const __nv_bfloat16 *src, float *dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]);
}
int launch_bf16_to_f32(const __nv_bfloat16 *src, float *dst, size_t n, cudaStream_t st) {
  if (n == 0) return 1;
  const size_t blocks = (n + 255) / 256;
  k_bf16_to_f32<<<(unsigned)(blocks > 4736 ? 4736 : blocks), 256, 0, st>>>(src, dst, n);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "bf16->f32 launch") ? 1 : 0;
}
// n must be a multiple of 8 (rows of H elements, H % 8 == 0)
__global__ void k_bf16_to_f16(const uint4 *src, uint4 *dst, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = coli_bf16x8_to_f16x8(src[i]);
}
int launch_bf16_to_f16(const __nv_bfloat16 *src, __half *dst, size_t n, cudaStream_t st) {
  if (n == 0) return 1;
  if (n % 8) {
    coli_set_error("bf16->f16: element count %zu is not a multiple of 8", n);
    return 0;
  }
  const size_t n8 = n / 8, blocks = (n8 + 255) / 256;
  k_bf16_to_f16<<<(unsigned)(blocks > 4736 ? 4736 : blocks), 256, 0, st>>>(reinterpret_cast<const uint4 *>(src),
                                                                           reinterpret_cast<uint4 *>(dst), n8);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "bf16->f16 launch") ? 1 : 0;
}

__global__ void k_matmul_f32_seq(const float *x, const float *w, float *y, int S, int I, int O) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)S * O) return;
  const int s = (int)(idx / O), o = (int)(idx % O);
  const float *xr = x + (size_t)s * I, *wr = w + (size_t)o * I;
  float acc = 0.0f;
  for (int k = 0; k < I; ++k) acc = __fadd_rn(acc, __fmul_rn(xr[k], wr[k]));
  y[idx] = acc;
}
int launch_matmul_f32_seq(const float *x, const float *w, float *y, int S, int I, int O, cudaStream_t st) {
  const size_t n = (size_t)S * O;
  if (n == 0) return 1;
  k_matmul_f32_seq<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(x, w, y, S, I, O);
  coli_count_launch(1);
  return coli_cuda_check(cudaGetLastError(), "f32 matmul launch") ? 1 : 0;
}

}  // namespace colib
