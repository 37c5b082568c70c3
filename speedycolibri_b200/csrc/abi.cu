// Host side of libcoli_b200.so: the extern "C" entry points declared in include/coli_b200.h.
// Lifecycle, resident-weight handles, the whole-block call and its stages, and the reference's
// host-pointer expert calls expressed through the same kernels.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "host_state.cuh"

// ---- errors ---------------------------------------------------------------------------------
static thread_local char g_err[512] = "";
void coli_set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  fprintf(stderr, "[CUDA] %s\n", g_err);  // the reference's log format, backend_cuda.cu:102-106
}
bool coli_cuda_check(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return true;
  coli_set_error("%s: %s", what, cudaGetErrorString(e));
  return false;
}
extern "C" const char *coli_cuda_last_error(void) { return g_err; }

#include <atomic>
static std::atomic<uint64_t> g_launches{0};
void coli_count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
extern "C" uint64_t coli_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// ---- device contexts (backend_cuda.cu:87-129, 2594-2655) --------------------------------------
namespace {
std::mutex g_init_mu;
DeviceContext *g_ctx[COLI_CUDA_MAX_DEVICES];
int g_ndev = 0;
int g_act_oai = 0;  // process-wide gate/up combine, backend_cuda.cu:339-350
float g_act_alpha = 1.702f;
float g_act_limit = 0.0f;

bool reserve(DeviceContext *c, int slot, size_t bytes) {
  if (c->cap[slot] >= bytes) return true;
  if (c->buf[slot]) cudaFree(c->buf[slot]);
  c->buf[slot] = nullptr;
  c->cap[slot] = 0;
  if (!coli_cuda_check(cudaMalloc(&c->buf[slot], bytes), "scratch allocation")) return false;
  c->cap[slot] = bytes;
  return true;
}
}  // namespace

DeviceContext *coli_find_ctx(int device) {
  for (int i = 0; i < g_ndev; ++i)
    if (g_ctx[i] && g_ctx[i]->device == device) return g_ctx[i];
  coli_set_error("device %d is not initialised (call coli_cuda_init)", device);
  return nullptr;
}
bool coli_select_ctx(DeviceContext *c) { return c && coli_cuda_check(cudaSetDevice(c->device), "cudaSetDevice"); }
static DeviceContext *find_ctx(int device) { return coli_find_ctx(device); }
static bool select_ctx(DeviceContext *c) { return coli_select_ctx(c); }

extern "C" int coli_cuda_init(const int *devices, int count) {
  std::lock_guard<std::mutex> lk(g_init_mu);
  for (int i = 0; devices && i < count && i < COLI_CUDA_MAX_DEVICES; ++i)  // a repeated ordinal is refused, backend_cuda.cu:2636-2640
    for (int j = 0; j < i; ++j)
      if (devices[i] == devices[j]) {
        coli_set_error("coli_cuda_init: device %d is listed twice", devices[i]);
        return 0;
      }
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n < 1) {
    coli_set_error("no CUDA device is visible");
    return 0;
  }
  int def = 0;
  if (!devices || count <= 0) {
    devices = &def;
    count = 1;
  }
  if (count > COLI_CUDA_MAX_DEVICES) {
    coli_set_error("too many devices (%d)", count);
    return 0;
  }
  if (g_ndev > 0) {  // idempotent for the same set only
    bool same = g_ndev == count;
    for (int i = 0; same && i < count; ++i) same = g_ctx[i]->device == devices[i];
    if (!same) coli_set_error("coli_cuda_init: already initialised with a different device set");
    return same ? 1 : 0;
  }
  for (int i = 0; i < count; ++i) {
    cudaDeviceProp prop;
    if (devices[i] < 0 || devices[i] >= n || !coli_cuda_check(cudaGetDeviceProperties(&prop, devices[i]), "device properties"))
      return 0;
    if (prop.major != 10) {
      coli_set_error("device %d is sm_%d%d; this library is built for sm_100a only", devices[i], prop.major, prop.minor);
      return 0;
    }
  }
  for (int i = 0; i < count; ++i) {
    DeviceContext *c = new DeviceContext();
    c->device = devices[i];
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, devices[i]);
    if (!coli_cuda_check(cudaSetDevice(c->device), "cudaSetDevice") ||
        !coli_cuda_check(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking), "stream creation")) {
      delete c;
      return 0;
    }
    g_ctx[g_ndev++] = c;
  }
  return 1;
}

extern "C" void coli_cuda_shutdown(void) {
  std::lock_guard<std::mutex> lk(g_init_mu);
  for (int i = 0; i < g_ndev; ++i) {
    DeviceContext *c = g_ctx[i];
    if (!c) continue;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    for (int s = 0; s < 8; ++s)
      if (c->buf[s]) cudaFree(c->buf[s]);
    for (int s = 0; s < 4; ++s)
      if (c->ev[s]) cudaEventDestroy(c->ev[s]);
    cudaStreamDestroy(c->stream);
    delete c;
    g_ctx[i] = nullptr;
  }
  g_ndev = 0;
}
extern "C" int coli_cuda_device_count(void) { return g_ndev; }
extern "C" int coli_cuda_device_at(int index) { return (index >= 0 && index < g_ndev) ? g_ctx[index]->device : -1; }
extern "C" int coli_cuda_mem_info(int device, size_t *free_bytes, size_t *total_bytes) {
  DeviceContext *c = find_ctx(device);
  if (!select_ctx(c) || !free_bytes || !total_bytes) return 0;
  return coli_cuda_check(cudaMemGetInfo(free_bytes, total_bytes), "cudaMemGetInfo") ? 1 : 0;
}
extern "C" int coli_cuda_device_sync(int device) {
  DeviceContext *c = find_ctx(device);
  if (!select_ctx(c)) return 0;
  return coli_cuda_check(cudaDeviceSynchronize(), "device sync") ? 1 : 0;
}
extern "C" void coli_cuda_set_activation(int oai, float alpha, float limit) {
  g_act_oai = oai;
  g_act_alpha = alpha;
  g_act_limit = limit;
}
static colib::ActParams current_activation() { return colib::ActParams{g_act_oai, g_act_alpha, g_act_limit}; }
extern "C" void coli_cuda_stats(int device, size_t *tensor_count, size_t *tensor_bytes) {
  size_t n = 0, b = 0;
  for (int i = 0; i < g_ndev; ++i)
    if (g_ctx[i] && (device < 0 || g_ctx[i]->device == device)) {
      n += g_ctx[i]->tensor_count;
      b += g_ctx[i]->tensor_bytes;
    }
  if (tensor_count) *tensor_count = n;
  if (tensor_bytes) *tensor_bytes = b;
}
// Live scratch of the host-pointer calls on `device` (< 0: all), excluding the weights that
// coli_cuda_stats reports (backend_cuda.h:48-51).
extern "C" size_t coli_cuda_scratch_bytes(int device) {
  size_t b = 0;
  for (int i = 0; i < g_ndev; ++i)
    if (g_ctx[i] && (device < 0 || g_ctx[i]->device == device))
      for (int s = 0; s < 8; ++s) b += g_ctx[i]->cap[s];
  return b;
}
// backend_cuda.h:86: whether the device reads pageable host memory in place.  A B200 behind PCIe
// does not (at any useful speed): every "wrap" of this library copies into HBM, so the answer is 0
// and the engine never takes its zero-copy branches (gpu.rs:207).
extern "C" int coli_cuda_pageable_access(int device) {
  (void)device;
  return 0;
}
// backend_cuda.h:66-69: residency switches of the reference's unified-memory box.  Weights are
// always copied into HBM here and expert weights are always device copies, so both are accepted
// and change nothing.
extern "C" void coli_cuda_set_weight_zerocopy(int on) { (void)on; }
extern "C" void coli_cuda_set_ffn_devcopy(int on) { (void)on; }
// backend_cuda.h:87-91: page-lock host memory the engine owns, so that the copies of the
// host-pointer calls run as DMA out of it.  0 on failure with the sticky error cleared: the caller
// carries on with pageable memory.
extern "C" int coli_cuda_host_register(void *p, size_t bytes) {
  if (!p || bytes == 0) return 0;
  if (cudaHostRegister(p, bytes, cudaHostRegisterDefault) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return 1;
}
extern "C" void coli_cuda_host_unregister(void *p) {
  if (p && cudaHostUnregister(p) != cudaSuccess) cudaGetLastError();
}
// ---- resident weights ----------------------------------------------------------------------------
static bool fmt_supported(int fmt) {
  return fmt == COLI_FMT_NVFP4 || fmt == COLI_FMT_MXFP4 || fmt == COLI_FMT_FP8_B128 || fmt == COLI_FMT_E4M3_ROW;
}

static size_t src_q_bytes(int fmt, int I, int O) {
  return (fmt == COLI_FMT_NVFP4 || fmt == COLI_FMT_MXFP4) ? (size_t)O * ((I + 1) / 2) : (size_t)O * I;
}
static size_t src_s_bytes(int fmt, int I, int O) {
  if (fmt == COLI_FMT_NVFP4) return (size_t)O * ((I + 15) / 16);
  if (fmt == COLI_FMT_MXFP4) return (size_t)O * ((I + 31) / 32);
  if (fmt == COLI_FMT_FP8_B128) return sizeof(float) * (size_t)((O + 127) / 128) * ((I + 127) / 128);
  return sizeof(float) * (size_t)O;
}

// Allocates the handle's HBM and fills it from device-resident source arrays.
static int build_tensor(ColiCudaTensor **slot, DeviceContext *ctx, int fmt, const void *d_q, const void *d_s,
                        float gscale, int I, int O) {
  ColiCudaTensor *t = static_cast<ColiCudaTensor *>(calloc(1, sizeof(ColiCudaTensor)));
  if (!t) return 0;
  t->fmt = fmt;
  t->I = I;
  t->O = O;
  t->device = ctx->device;
  t->Kp = round_up(I, 128);
  t->Op = round_up(O, 16);
  t->KT = t->Kp / 128;
  t->gscale = gscale;
  t->q_bytes = (size_t)t->KT * t->Op * (fmt == COLI_FMT_NVFP4 ? 64 : 128);
  t->s_bytes = fmt == COLI_FMT_NVFP4 ? (size_t)t->KT * t->Op * 8 : src_s_bytes(fmt, I, O);
  bool ok = coli_cuda_check(cudaMalloc((void **)&t->q, t->q_bytes), "tensor allocation") &&
            coli_cuda_check(cudaMalloc((void **)&t->s, t->s_bytes), "scale allocation");
  if (ok) {
    if (fmt == COLI_FMT_NVFP4) {
      ok = colib::pack_nvfp4((const uint8_t *)d_q, (const uint8_t *)d_s, O, I, t, ctx->stream);
    } else {
      ok = colib::pack_fp8((const uint8_t *)d_q, O, I, t, ctx->stream) &&
           coli_cuda_check(cudaMemcpyAsync(t->s, d_s, t->s_bytes, cudaMemcpyDeviceToDevice, ctx->stream), "scale copy");
    }
    ok = ok && coli_cuda_check(cudaStreamSynchronize(ctx->stream), "tensor repack");
  }
  if (!ok) {
    if (t->q) cudaFree(t->q);
    if (t->s) cudaFree(t->s);
    free(t);
    return 0;
  }
  ctx->tensor_count++;
  ctx->tensor_bytes += t->q_bytes + t->s_bytes;
  *slot = t;
  return 1;
}

static int existing_matches(ColiCudaTensor *t, int fmt, int I, int O, int device) {
  return t->fmt == fmt && t->I == I && t->O == O && t->device == device;
}

static int upload_from_host(ColiCudaTensor **tensor, const void *q, const void *s, float gscale, int fmt, int I,
                            int O, int device) {
  if (!tensor || !q || !s || I < 1 || O < 1) {
    coli_set_error("tensor upload: null pointer or empty shape");
    return 0;
  }
  if (!fmt_supported(fmt)) {
    coli_set_error("tensor upload: format %d is not part of the MoE expert path (supported: 4, 5, 8)", fmt);
    return 0;
  }
  if (fmt == COLI_FMT_MXFP4) {
    coli_set_error("tensor upload: MXFP4 carries E8M0 block scales; use coli_cuda_tensor_wrap_mxfp4");
    return 0;
  }
  if (*tensor) return existing_matches(*tensor, fmt, I, O, device);
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  const size_t qb = src_q_bytes(fmt, I, O), sb = src_s_bytes(fmt, I, O);
  void *dq = nullptr, *ds = nullptr;
  int ok = coli_cuda_check(cudaMalloc(&dq, qb), "staging allocation") &&
           coli_cuda_check(cudaMalloc(&ds, sb), "staging allocation") &&
           coli_cuda_check(cudaMemcpyAsync(dq, q, qb, cudaMemcpyHostToDevice, ctx->stream), "tensor upload") &&
           coli_cuda_check(cudaMemcpyAsync(ds, s, sb, cudaMemcpyHostToDevice, ctx->stream), "scale upload");
  ok = ok && build_tensor(tensor, ctx, fmt, dq, ds, gscale, I, O);
  if (dq) cudaFree(dq);
  if (ds) cudaFree(ds);
  return ok;
}

extern "C" int coli_cuda_tensor_upload(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt,
                                       int I, int O, int device) {
  if (fmt == COLI_FMT_NVFP4) {
    coli_set_error("tensor upload: NVFP4 carries byte block scales; use coli_cuda_tensor_wrap_nvfp4");
    return 0;
  }
  return upload_from_host(tensor, weights, scales, 1.0f, fmt, I, O, device);
}
extern "C" int coli_cuda_tensor_wrap(ColiCudaTensor **tensor, const void *weights, const float *scales, int fmt,
                                     int I, int O, int device) {
  return coli_cuda_tensor_upload(tensor, weights, scales, fmt, I, O, device);
}
extern "C" int coli_cuda_tensor_wrap_nvfp4(ColiCudaTensor **tensor, const void *weights, const void *bscale,
                                           float gscale, int I, int O, int device) {
  return upload_from_host(tensor, weights, bscale, gscale, COLI_FMT_NVFP4, I, O, device);
}
// MXFP4 -> the resident NVFP4 form.  A block scale 2^e (E8M0 byte e + 127) becomes the ue4m3 code
// of 2^(e + shift) in both 16-wide halves of its 32-wide block; shift = 8 - (largest e among blocks
// that hold a non-zero weight), so the largest block scale lands on 2^8, the top of ue4m3's powers
// of two, and blocks down to 2^-9 (17 binades lower) stay exact.  The tensor scale absorbs 2^-shift.
static bool mxfp4_to_resident_scales(const uint8_t *nib, const uint8_t *e8, int O, int I, float gscale,
                                     std::vector<uint8_t> &bs16, float *gscale_out) {
  const int nb32 = (I + 31) / 32, nb16 = (I + 15) / 16, rb = (I + 1) / 2;
  int max_e = -1000;
  for (int o = 0; o < O; ++o)
    for (int b = 0; b < nb32; ++b) {
      const uint8_t code = e8[(size_t)o * nb32 + b];
      if (code == 0xFF || (int)code - 127 <= max_e) continue;
      const uint8_t *p = nib + (size_t)o * rb + 16 * b;
      const int nbytes = (rb - 16 * b) < 16 ? (rb - 16 * b) : 16;
      bool nonzero = false;
      for (int j = 0; j < nbytes && !nonzero; ++j) nonzero = (p[j] & 0x77) != 0;  // magnitude bits of both nibbles
      if (nonzero) max_e = (int)code - 127;
    }
  const int shift = max_e == -1000 ? 0 : 8 - max_e;
  const double g2 = ldexp((double)gscale, -shift);
  const float gf = (float)g2;
  if (gscale != 0.0f && (!(fabs(g2) <= 3.0e38) || fabs(g2) < 1.2e-38)) {
    coli_set_error("tensor_wrap_mxfp4: tensor scale %g with block exponents up to %d leaves the f32 range", (double)gscale, max_e);
    return false;
  }
  bs16.assign((size_t)O * nb16, 0);
  for (int o = 0; o < O; ++o)
    for (int b = 0; b < nb16; ++b) {
      const uint8_t code = e8[(size_t)o * nb32 + (b >> 1)];
      uint8_t out;
      if (code == 0xFF) {
        out = 0x7F;  // NaN stays NaN (dtype.rs:137-139)
      } else {
        const int ec = (int)code - 127 + shift;
        out = ec > 8 ? 0x78 /* only all-zero blocks get here */ : ec >= -6 ? (uint8_t)((ec + 7) << 3) : ec >= -9 ? (uint8_t)(1u << (ec + 9)) : 0;
      }
      bs16[(size_t)o * nb16 + b] = out;
    }
  *gscale_out = gf;
  return true;
}

extern "C" int coli_b200_mxfp4_resident_scales(const void *weights, const void *bscale, float gscale, int I, int O,
                                               void *bscale16_out, float *gscale_out) {
  if (!weights || !bscale || !bscale16_out || !gscale_out || I < 1 || O < 1) {
    coli_set_error("mxfp4_resident_scales: null pointer or empty shape");
    return 0;
  }
  std::vector<uint8_t> bs16;
  if (!mxfp4_to_resident_scales((const uint8_t *)weights, (const uint8_t *)bscale, O, I, gscale, bs16, gscale_out)) return 0;
  memcpy(bscale16_out, bs16.data(), bs16.size());
  return 1;
}

extern "C" int coli_cuda_tensor_wrap_mxfp4(ColiCudaTensor **tensor, const void *weights, const void *bscale,
                                           float gscale, int I, int O, int device) {
  if (!tensor || !weights || !bscale || I < 1 || O < 1) {
    coli_set_error("tensor_wrap_mxfp4: null pointer or empty shape");
    return 0;
  }
  if (*tensor) return existing_matches(*tensor, COLI_FMT_MXFP4, I, O, device);
  std::vector<uint8_t> bs16;
  float g2 = 0.0f;
  if (!mxfp4_to_resident_scales((const uint8_t *)weights, (const uint8_t *)bscale, O, I, gscale, bs16, &g2)) return 0;
  ColiCudaTensor *t = nullptr;
  if (!upload_from_host(&t, weights, bs16.data(), g2, COLI_FMT_NVFP4, I, O, device)) return 0;
  DeviceContext *ctx = find_ctx(device);
  t->s_src_bytes = src_s_bytes(COLI_FMT_MXFP4, I, O);
  if (!select_ctx(ctx) || !coli_cuda_check(cudaMalloc((void **)&t->s_src, t->s_src_bytes), "scale allocation") ||
      !coli_cuda_check(cudaMemcpy(t->s_src, bscale, t->s_src_bytes, cudaMemcpyHostToDevice), "scale upload")) {
    coli_cuda_tensor_free(t);
    return 0;
  }
  t->fmt = COLI_FMT_MXFP4;
  t->gscale_src = gscale;
  ctx->tensor_bytes += t->s_src_bytes;
  *tensor = t;
  return 1;
}

extern "C" int coli_b200_tensor_from_device(ColiCudaTensor **tensor, int fmt, const void *d_q, const void *d_s,
                                            float gscale, int I, int O, int device) {
  if (fmt == COLI_FMT_MXFP4) {
    coli_set_error("tensor_from_device: MXFP4 is transcoded on the host; use coli_cuda_tensor_wrap_mxfp4");
    return 0;
  }
  if (!tensor || !d_q || !d_s || I < 1 || O < 1 || !fmt_supported(fmt)) {
    coli_set_error("tensor_from_device: bad argument");
    return 0;
  }
  if (*tensor) return existing_matches(*tensor, fmt, I, O, device);
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  // the source arrays may have been written on another stream
  if (!coli_cuda_check(cudaDeviceSynchronize(), "tensor_from_device sync")) return 0;
  return build_tensor(tensor, ctx, fmt, d_q, d_s, gscale, I, O);
}
extern "C" int coli_b200_tensor_export(const ColiCudaTensor *t, void *q_host, void *s_host, float *gscale) {
  if (!t || !q_host || !s_host) {
    coli_set_error("tensor_export: null pointer");
    return 0;
  }
  DeviceContext *ctx = find_ctx(t->device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  const size_t qb = src_q_bytes(t->fmt, t->I, t->O), sb = src_s_bytes(t->fmt, t->I, t->O);
  void *dq = nullptr, *ds = nullptr;
  int ok = coli_cuda_check(cudaMalloc(&dq, qb), "staging allocation") && coli_cuda_check(cudaMalloc(&ds, sb), "staging allocation");
  if (ok) {
    if (t->fmt == COLI_FMT_MXFP4) {
      // nibbles from the resident form, block scales as they were uploaded
      void *d16 = nullptr;
      ok = coli_cuda_check(cudaMalloc(&d16, src_s_bytes(COLI_FMT_NVFP4, t->I, t->O)), "staging allocation") &&
           colib::unpack_nvfp4(t, (uint8_t *)dq, (uint8_t *)d16, ctx->stream) &&
           coli_cuda_check(cudaMemcpyAsync(ds, t->s_src, sb, cudaMemcpyDeviceToDevice, ctx->stream), "scale copy") &&
           coli_cuda_check(cudaStreamSynchronize(ctx->stream), "tensor export sync");
      if (d16) cudaFree(d16);
    } else if (t->fmt == COLI_FMT_NVFP4)
      ok = colib::unpack_nvfp4(t, (uint8_t *)dq, (uint8_t *)ds, ctx->stream);
    else
      ok = colib::unpack_fp8(t, (uint8_t *)dq, ctx->stream) &&
           coli_cuda_check(cudaMemcpyAsync(ds, t->s, sb, cudaMemcpyDeviceToDevice, ctx->stream), "scale copy");
  }
  ok = ok && coli_cuda_check(cudaMemcpyAsync(q_host, dq, qb, cudaMemcpyDeviceToHost, ctx->stream), "tensor export") &&
       coli_cuda_check(cudaMemcpyAsync(s_host, ds, sb, cudaMemcpyDeviceToHost, ctx->stream), "scale export") &&
       coli_cuda_check(cudaStreamSynchronize(ctx->stream), "tensor export sync");
  if (dq) cudaFree(dq);
  if (ds) cudaFree(ds);
  if (ok && gscale) *gscale = t->fmt == COLI_FMT_MXFP4 ? t->gscale_src : t->gscale;
  return ok;
}
extern "C" void coli_cuda_tensor_free(ColiCudaTensor *t) {
  if (!t) return;
  for (int i = 0; i < g_ndev; ++i)
    if (g_ctx[i] && g_ctx[i]->device == t->device) {
      cudaSetDevice(t->device);
      g_ctx[i]->tensor_count--;
      g_ctx[i]->tensor_bytes -= t->q_bytes + t->s_bytes + t->s_src_bytes;
    }
  if (t->q) cudaFree(t->q);
  if (t->s) cudaFree(t->s);
  if (t->s_src) cudaFree(t->s_src);
  free(t);
}
extern "C" size_t coli_cuda_tensor_bytes(const ColiCudaTensor *t) { return t ? t->q_bytes + t->s_bytes + t->s_src_bytes : 0; }
extern "C" int coli_cuda_tensor_device(const ColiCudaTensor *t) { return t ? t->device : -1; }

extern "C" int coli_b200_quantize_nvfp4(int device, const float *d_w, int O, int I, void *d_nibbles, void *d_bscale,
                                        float *gscale) {
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx) || !d_w || !d_nibbles || !d_bscale || !gscale) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  if (!reserve(ctx, 7, 256)) return 0;
  if (!coli_cuda_check(cudaDeviceSynchronize(), "quantise sync")) return 0;
  return colib::quantize_nvfp4(d_w, O, I, (uint8_t *)d_nibbles, (uint8_t *)d_bscale, (float *)ctx->buf[7], gscale, ctx->stream);
}
extern "C" int coli_b200_quantize_fp8_b128(int device, const float *d_w, int O, int I, void *d_codes, float *d_scales) {
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx) || !d_w || !d_codes || !d_scales) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  if (!coli_cuda_check(cudaDeviceSynchronize(), "quantise sync")) return 0;
  return colib::quantize_fp8_b128(d_w, O, I, (uint8_t *)d_codes, d_scales, ctx->stream) &&
         coli_cuda_check(cudaStreamSynchronize(ctx->stream), "fp8 quantise sync");
}

// ---- the block ------------------------------------------------------------------------------------
extern "C" void coli_b200_moe_destroy(ColiMoe *m) {
  if (!m) return;
  if (m->ctx) {
    cudaSetDevice(m->ctx->device);
    cudaDeviceSynchronize();
  }
  coli_ep_destroy(m);
  for (void *p : m->allocs) cudaFree(p);
  for (int i = 0; i <= COLI_PHASES; ++i)
    if (m->ev[i]) cudaEventDestroy(m->ev[i]);
  delete m;
}

extern "C" int coli_b200_moe_profile(ColiMoe *m, int enable) {
  if (!m || !select_ctx(m->ctx)) return 0;
  if (enable) {
    for (int i = 0; i <= COLI_PHASES; ++i)
      if (!m->ev[i]) CK(cudaEventCreate(&m->ev[i]), "event creation");
    for (int i = 0; i < COLI_PHASES; ++i) m->phase_ms[i] = 0.0f;
    m->phase_calls = 0;
  }
  m->profiling = enable != 0;
  return 1;
}
extern "C" int coli_b200_moe_phase_ms(ColiMoe *m, float *ms, int *calls) {
  if (!m || !ms) return 0;
  for (int i = 0; i < COLI_PHASES; ++i) ms[i] = m->phase_ms[i];
  if (calls) *calls = m->phase_calls;
  return 1;
}
extern "C" void *coli_b200_moe_stream(ColiMoe *m) { return m ? (void *)m->ctx->stream : nullptr; }

// The tcgen05 path takes over from 8 rows per segment on average: below that the register-level
// kernel re-reads so few token rows per weight tile that it wins; a pure function of (rows,
// segments, format) so that kernel selection never depends on data or addresses.
// Which tcgen05 kernel: the one with the weight operand in tensor memory takes tiles of at most
// 160 tokens and wins while segments are about that long; longer NVFP4 segments amortise the
// shared-memory weight tiles of the other kernel over 256 tokens.  The FP8 formats exist in the
// tensor-memory kernel only (longer segments are cut into several of its tiles).
bool coli_use_tct(int fmt, int rows, int nseg) {
  return fmt != COLI_FMT_NVFP4 || rows <= 160 * (nseg > 0 ? nseg : 1);
}
// Tile width of the tensor-memory kernel: short tiles (and a weight ring twice as deep) while the
// average segment fits one of them with room to spare, the full width otherwise.
int coli_tct_tile_tokens(int rows, int nseg) {
  return rows <= 48 * (nseg > 0 ? nseg : 1) ? colib::TCT_SHORT_TOKENS : colib::TCT_MAX_TOKENS;
}
bool coli_use_tc_path(int fmt, int rows, int nseg) {
  return (fmt == COLI_FMT_NVFP4 || fmt == COLI_FMT_FP8_B128 || fmt == COLI_FMT_E4M3_ROW) && nseg > 0 && rows / nseg >= 8;
}

int coli_rows_per_item_for(int rows, int nseg) {
  const int avg = (rows + nseg - 1) / (nseg > 0 ? nseg : 1);
  return avg <= 8 ? 8 : avg <= 16 ? 16 : 32;
}
static bool use_tct(int fmt, int rows, int nseg) { return coli_use_tct(fmt, rows, nseg); }
static int tct_tile_tokens(int rows, int nseg) { return coli_tct_tile_tokens(rows, nseg); }
static bool use_tc_path(int fmt, int rows, int nseg) { return coli_use_tc_path(fmt, rows, nseg); }
static int rows_per_item_for(const ColiMoeLayer &, int rows, int nseg) { return coli_rows_per_item_for(rows, nseg); }

extern "C" int coli_b200_moe_create(ColiMoe **out, const ColiMoeLayer *L, int max_tokens) {
  if (!out || !L || max_tokens < 1) {
    coli_set_error("moe_create: bad argument");
    return 0;
  }
  if (L->H < 8 || L->H % 8 || L->I < 8 || L->I % 8 || L->E < 1 || L->E > 512 || L->k < 1 || L->k > 32 || L->k > L->E) {
    coli_set_error("moe_create: unsupported shape H=%d I=%d E=%d k=%d (H, I multiples of 8; E <= 512; k <= min(32,E))", L->H, L->I, L->E, L->k);
    return 0;
  }
  if (L->n_group > 1 && (L->E % L->n_group || L->n_group > 32 || L->topk_group < 1)) {
    coli_set_error("moe_create: n_group=%d must divide E=%d and be <= 32", L->n_group, L->E);
    return 0;
  }
  if (L->n_group > 1 && L->k > (L->topk_group < L->n_group ? L->topk_group : L->n_group) * (L->E / L->n_group)) {
    // the kept groups hold fewer than k experts: the scan would run out of candidates and repeat expert 0
    coli_set_error("moe_create: k=%d exceeds the %d experts of the %d groups a token may use", L->k,
                   (L->topk_group < L->n_group ? L->topk_group : L->n_group) * (L->E / L->n_group), L->topk_group);
    return 0;
  }
  if (!fmt_supported(L->fmt) || !L->router_w || !L->gate || !L->up || !L->down) {
    coli_set_error("moe_create: missing router/expert tables or unsupported format %d", L->fmt);
    return 0;
  }
  DeviceContext *ctx = find_ctx(L->device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  ColiMoe *m = new ColiMoe();
  m->L = *L;
  m->ctx = ctx;
  m->max_tokens = max_tokens;
  m->act = current_activation();
  m->ws_bytes = 0;
  m->profiling = false;
  m->phase_calls = 0;
  for (int i = 0; i <= COLI_PHASES; ++i) m->ev[i] = nullptr;
  for (int i = 0; i < COLI_PHASES; ++i) m->phase_ms[i] = 0.0f;
  m->has_shared = L->sh_gate && L->sh_up && L->sh_down;
  m->nseg = L->E + (m->has_shared ? 1 : 0);
  const int E = L->E, H = L->H, I = L->I, k = L->k;
  const int world = L->ep_world > 1 ? L->ep_world : 1;

  // segment order = experts sorted by (owner rank, expert id); sharding.rs:197-203 for the default map
  std::vector<int> owner(E);
  for (int e = 0; e < E; ++e) {
    owner[e] = world > 1 ? (L->expert_owner ? L->expert_owner[e] : (int)((int64_t)e * world / E)) : 0;
    if (owner[e] < 0 || owner[e] >= world) {
      coli_set_error("moe_create: expert %d has owner %d outside [0,%d)", e, owner[e], world);
      delete m;
      return 0;
    }
  }
  m->h_owner.assign(owner.begin(), owner.end());
  m->h_expert_slot.assign(E, 0);
  m->h_seg_expert.assign(E + 1, E);
  m->first_local_seg = 0;
  m->n_local_seg = 0;
  {
    int pos = 0;
    for (int r = 0; r < world; ++r) {
      if (r == L->ep_rank) m->first_local_seg = pos;
      for (int e = 0; e < E; ++e)
        if (owner[e] == r) {
          m->h_expert_slot[e] = pos;
          m->h_seg_expert[pos] = e;
          ++pos;
          if (r == L->ep_rank || world == 1) m->n_local_seg++;
        }
    }
  }
  // weight tables
  std::vector<WeightRef> tg(E + 1), tu(E + 1), td(E + 1);
  auto ref = [&](ColiCudaTensor *t, int wantI, int wantO, WeightRef &r, const char *name, int e) -> bool {
    r.q = nullptr;
    r.s = nullptr;
    r.g = 0.0f;
    r.pad = 0;
    if (!t) return true;
    if (t->fmt != L->fmt || t->I != wantI || t->O != wantO || t->device != L->device) {
      coli_set_error("moe_create: %s of expert %d has fmt/shape/device %d/[%d,%d]/%d, expected %d/[%d,%d]/%d", name, e, t->fmt,
                     t->O, t->I, t->device, L->fmt, wantO, wantI, L->device);
      return false;
    }
    r.q = t->q;
    r.s = t->s;
    r.g = t->gscale;
    return true;
  };
  m->all_resident = true;
  bool ok = true;
  for (int e = 0; e < E && ok; ++e) {
    ok = ref(L->gate[e], H, I, tg[e], "gate", e) && ref(L->up[e], H, I, tu[e], "up", e) && ref(L->down[e], I, H, td[e], "down", e);
    const bool have = L->gate[e] && L->up[e] && L->down[e];
    if (!have) m->all_resident = false;
    if (ok && !have && (world == 1 || owner[e] == L->ep_rank)) {
      coli_set_error("moe_create: expert %d is owned by this rank but has no resident weights", e);
      ok = false;
    }
  }
  if (ok && m->has_shared)
    ok = ref(L->sh_gate, H, I, tg[E], "shared gate", E) && ref(L->sh_up, H, I, tu[E], "shared up", E) &&
         ref(L->sh_down, I, H, td[E], "shared down", E);
  else if (ok)
    ref(nullptr, 0, 0, tg[E], "", E), ref(nullptr, 0, 0, tu[E], "", E), ref(nullptr, 0, 0, td[E], "", E);

  const size_t T = (size_t)max_tokens;
  const size_t rows = T * k + T;
  m->item_cap = (int)(rows / 8 + m->nseg + 1);
  const int nchunk = (max_tokens + 31) / 32;
  ok = ok && ws_alloc(m, &m->router_w, (size_t)E * H) && ws_alloc(m, &m->gate, E + 1) && ws_alloc(m, &m->up, E + 1) &&
       ws_alloc(m, &m->down, E + 1) && ws_alloc(m, &m->expert_slot, E) && ws_alloc(m, &m->seg_expert, E + 1) && ws_alloc(m, &m->local_slot, E) &&
       ws_alloc(m, &m->logits, T * E) && ws_alloc(m, &m->topk_w, T * k) && ws_alloc(m, &m->topk_idx, T * k) &&
       ws_alloc(m, &m->local_rank, T * k) && ws_alloc(m, &m->chunk_cnt, (size_t)nchunk * E) &&
       ws_alloc(m, &m->seg_count, E + 1) && ws_alloc(m, &m->seg_off, E + 2) && ws_alloc(m, &m->slot, T * k) &&
       ws_alloc(m, &m->row_token, rows) && ws_alloc(m, &m->item_seg, m->item_cap) &&
       ws_alloc(m, &m->item_row0, m->item_cap) && ws_alloc(m, &m->item_nrows, m->item_cap) && ws_alloc(m, &m->n_items, 1) &&
       ws_alloc(m, &m->h, rows * I) && ws_alloc(m, &m->y, rows * H) && ws_alloc(m, &m->x_stage, T * H) &&
       ws_alloc(m, &m->out_stage, T * H) && ws_alloc(m, &m->x16, T * H);
  m->h_rows_cap = rows;
  m->seg_main.h = m->h;
  m->seg_main.h_rows = rows;
  m->seg_main.item_seg = m->item_seg;
  m->seg_main.item_row0 = m->item_row0;
  m->seg_main.item_nrows = m->item_nrows;
  m->seg_main.n_items = m->n_items;
  m->seg_main.seg_off = m->seg_off;
  m->seg_main.item_cap = m->item_cap;
  m->seg_main.seg_cap = E + 1;
  m->ep = nullptr;
  m->xg = nullptr;
  m->status = nullptr;
  {
    cudaDeviceProp prop;
    ok = ok && coli_cuda_check(cudaGetDeviceProperties(&prop, L->device), "device properties");
    m->sm_count = ok ? prop.multiProcessorCount : 0;
  }
  ok = ok && ws_alloc(m, &m->status, 1) && coli_cuda_check(cudaMemset(m->status, 0, sizeof(int)), "status clear");
  m->ticket = nullptr;
  ok = ok && ws_alloc(m, &m->ticket, 1) && coli_cuda_check(cudaMemset(m->ticket, 0, sizeof(unsigned int)), "ticket clear");
  if (ok && use_tc_path(coli_kernel_fmt(L->fmt), (int)rows, m->nseg)) ok = ws_alloc(m, &m->xg, rows * H);
  m->select_bias = nullptr;
  m->logit_bias = nullptr;
  if (ok && L->select_bias) ok = ws_alloc(m, &m->select_bias, E);
  if (ok && L->logit_bias) ok = ws_alloc(m, &m->logit_bias, E);
  cudaStream_t st = ctx->stream;
  ok = ok && coli_cuda_check(cudaMemcpyAsync(m->router_w, L->router_w, (size_t)E * H * 2, cudaMemcpyHostToDevice, st), "router upload") &&
       coli_cuda_check(cudaMemcpyAsync(m->gate, tg.data(), sizeof(WeightRef) * (E + 1), cudaMemcpyHostToDevice, st), "table upload") &&
       coli_cuda_check(cudaMemcpyAsync(m->up, tu.data(), sizeof(WeightRef) * (E + 1), cudaMemcpyHostToDevice, st), "table upload") &&
       coli_cuda_check(cudaMemcpyAsync(m->down, td.data(), sizeof(WeightRef) * (E + 1), cudaMemcpyHostToDevice, st), "table upload") &&
       coli_cuda_check(cudaMemcpyAsync(m->expert_slot, m->h_expert_slot.data(), sizeof(int32_t) * E, cudaMemcpyHostToDevice, st), "table upload") &&
       coli_cuda_check(cudaMemcpyAsync(m->seg_expert, m->h_seg_expert.data(), sizeof(int32_t) * (E + 1), cudaMemcpyHostToDevice, st), "table upload");
  std::vector<int32_t> h_local_slot(E, -1);
  for (int e = 0; e < E; ++e)
    if (world == 1 || owner[e] == L->ep_rank) h_local_slot[e] = m->h_expert_slot[e] - m->first_local_seg;
  ok = ok && coli_cuda_check(cudaMemcpyAsync(m->local_slot, h_local_slot.data(), sizeof(int32_t) * E, cudaMemcpyHostToDevice, st), "table upload");
  if (ok && L->select_bias)
    ok = coli_cuda_check(cudaMemcpyAsync(m->select_bias, L->select_bias, sizeof(float) * E, cudaMemcpyHostToDevice, st), "bias upload");
  if (ok && L->logit_bias)
    ok = coli_cuda_check(cudaMemcpyAsync(m->logit_bias, L->logit_bias, sizeof(float) * E, cudaMemcpyHostToDevice, st), "bias upload");
  ok = ok && coli_cuda_check(cudaStreamSynchronize(st), "moe_create sync");
  if (ok && world > 1 && L->nccl_comm) ok = coli_ep_ensure(m, L->nccl_comm) != 0;
  // from here on the handle's format is the one its kernels decode (MXFP4 is resident in the NVFP4 form)
  m->L.fmt = coli_kernel_fmt(L->fmt);
  // the handle keeps no host pointers
  m->L.router_w = nullptr;
  m->L.select_bias = nullptr;
  m->L.logit_bias = nullptr;
  m->L.expert_owner = nullptr;
  m->L.gate = m->L.up = m->L.down = nullptr;
  m->L.nccl_comm = nullptr;
  if (!ok) {
    coli_ep_destroy(m);
    for (void *p : m->allocs) cudaFree(p);
    delete m;
    return 0;
  }
  *out = m;
  return 1;
}

extern "C" size_t coli_b200_moe_workspace_bytes(const ColiMoe *m) { return m ? m->ws_bytes : 0; }

// A null stream is CUDA's default stream, as everywhere else in the runtime.
static cudaStream_t pick_stream(ColiMoe *m, void *stream) {
  (void)m;
  return (cudaStream_t)stream;
}

static bool check_T(ColiMoe *m, int T, const char *who) { return coli_check_T(m, T, who); }
bool coli_check_T(ColiMoe *m, int T, const char *who) {
  if (!m) {
    coli_set_error("%s: null handle", who);
    return false;
  }
  if (T < 0 || T > m->max_tokens) {
    coli_set_error("%s: T=%d outside [0,%d]", who, T, m->max_tokens);
    return false;
  }
  return select_ctx(m->ctx);
}

static colib::RouteParams route_params(ColiMoe *m, const void *x_dev, int T) { return coli_route_params(m, x_dev, T); }
colib::RouteParams coli_route_params(ColiMoe *m, const void *x_dev, int T) {
  colib::RouteParams rp;
  rp.T = T;
  rp.H = m->L.H;
  rp.E = m->L.E;
  rp.k = m->L.k;
  rp.score = m->L.score;
  rp.norm_topk = m->L.norm_topk;
  rp.routed_scale = m->L.routed_scale;
  rp.n_group = m->L.n_group;
  rp.topk_group = m->L.topk_group;
  rp.x = (const __nv_bfloat16 *)x_dev;
  rp.router_w = m->router_w;
  rp.select_bias = m->select_bias;
  rp.logit_bias = m->logit_bias;
  rp.logits = m->logits;
  rp.topk_idx = m->topk_idx;
  rp.topk_w = m->topk_w;
  return rp;
}

static colib::PermuteParams permute_params(ColiMoe *m, const void *x_dev, int T, bool with_shared, int rpi, void *rows_dev,
                                           int32_t *seg_count, int32_t *slot) {
  return coli_permute_params(m, x_dev, T, with_shared, rpi, rows_dev, seg_count, slot);
}
colib::PermuteParams coli_permute_params(ColiMoe *m, const void *x_dev, int T, bool with_shared, int rpi, void *rows_dev,
                                         int32_t *seg_count, int32_t *slot) {
  colib::PermuteParams pp;
  pp.T = T;
  pp.H = m->L.H;
  pp.E = m->L.E;
  pp.k = m->L.k;
  pp.nseg_routed = m->L.E;
  pp.has_shared = with_shared ? 1 : 0;
  pp.rows_per_item = rpi;
  pp.topk_idx = m->topk_idx;
  pp.expert_slot = m->expert_slot;
  pp.local_rank = m->local_rank;
  pp.chunk_cnt = m->chunk_cnt;
  pp.seg_count = seg_count;
  pp.seg_off = m->seg_off;
  pp.slot = slot;
  pp.row_token = m->row_token;
  pp.item_seg = m->item_seg;
  pp.item_row0 = m->item_row0;
  pp.item_nrows = m->item_nrows;
  pp.n_items = m->n_items;
  pp.x = (const __nv_bfloat16 *)x_dev;
  pp.xg = (__half *)rows_dev;
  pp.gather_shared = 0;
  pp.x16 = nullptr;
  pp.virt = nullptr;
  pp.rows_cap = 0x7fffffff;
  pp.overflow = nullptr;
  return pp;
}

// The block on device pointers.  out_dev: bf16 [T,H] block output; or, when resid_io is given,
// resid_io[T,H] (f32) += block output without an intermediate rounding (out_dev unused).
static int moe_block_impl(ColiMoe *m, const void *x_dev, void *out_dev, float *resid_io, int T, void *stream) {
  if (!check_T(m, T, "moe_block_dev")) return 0;
  if (!x_dev || (!out_dev && !resid_io)) {
    coli_set_error("moe_block_dev: null pointer");
    return 0;
  }
  if (!m->all_resident) {
    coli_set_error("moe_block_dev: not every expert is resident on this rank; use the stage calls for expert parallelism");
    return 0;
  }
  if (T == 0) return 1;
  cudaStream_t st = pick_stream(m, stream);
  const int k = m->L.k;
  const int rows = T * k + (m->has_shared ? T : 0);
  const bool tc = use_tc_path(m->L.fmt, rows, m->nseg) && m->xg != nullptr;
  const bool tct = tc && use_tct(m->L.fmt, rows, m->nseg);
  const int rpi = tc ? (tct ? tct_tile_tokens(rows, m->nseg) : colib::TC_MAX_TOKENS) : rows_per_item_for(m->L, rows, m->nseg);
  const int max_items = max_work_items(rows, m->nseg, rpi);
  const bool prof = m->profiling;
#define COLI_MARK(i)                                                         \
  do {                                                                       \
    if (prof) CK(cudaEventRecord(m->ev[i], st), "phase event");              \
  } while (0)
  COLI_MARK(0);
  {
    colib::PermuteParams pp = permute_params(m, x_dev, T, m->has_shared, rpi, tc ? m->xg : nullptr, m->seg_count, m->slot);
    pp.gather_shared = tc ? 1 : 0;
    pp.x16 = tc ? nullptr : m->x16;
    // decode-sized batches: one launch for router, top-k and permutation (its time is booked
    // under the router phase)
    const int fused = T <= 8 ? colib::launch_decode_front(route_params(m, x_dev, T), pp, m->ticket, st) : -1;
    if (fused == 0) return 0;
    if (fused < 0 && !colib::launch_router(route_params(m, x_dev, T), st)) return 0;
    COLI_MARK(1);
    if (fused < 0 && !colib::launch_permute(pp, st)) return 0;
  }
  COLI_MARK(2);
  if (tc) {
    colib::TcParams tp;
    tp.fmt = m->L.fmt;
    tp.H = m->L.H;
    tp.I = m->L.I;
    tp.gate = m->gate;
    tp.up = m->up;
    tp.down = m->down;
    tp.seg_expert = m->seg_expert;
    tp.item_seg = m->item_seg;
    tp.item_row0 = m->item_row0;
    tp.item_nrows = m->item_nrows;
    tp.n_items = m->n_items;
    tp.max_items = max_items;
    tp.tile_tokens = rpi;
    tp.h = m->h;
    tp.y = m->y;
    tp.status = m->status;
    tp.act = m->act;
    if (!(tct ? colib::launch_gate_up_tct(tp, m->xg, rows, m->sm_count, st) : colib::launch_gate_up_tc(tp, m->xg, rows, m->sm_count, st)))
      return 0;
    COLI_MARK(3);
    if (!(tct ? colib::launch_down_tct(tp, rows, m->sm_count, st) : colib::launch_down_tc(tp, rows, m->sm_count, st))) return 0;
  } else {
    colib::FfnParams fp;
    fp.fmt = m->L.fmt;
    fp.H = m->L.H;
    fp.I = m->L.I;
    fp.gate = m->gate;
    fp.up = m->up;
    fp.down = m->down;
    fp.seg_expert = m->seg_expert;
    fp.item_seg = m->item_seg;
    fp.item_row0 = m->item_row0;
    fp.item_nrows = m->item_nrows;
    fp.n_items = m->n_items;
    fp.max_items = max_items;
    fp.rows_per_item = rpi;
    fp.items_expected = (rows < m->nseg ? rows : m->nseg) + rows / rpi;
    fp.x = m->x16;
    fp.row_token = m->row_token;
    fp.h = m->h;
    fp.y = m->y;
    fp.y32 = nullptr;
    fp.relu2_out = nullptr;
    fp.act = m->act;
    if (!colib::launch_gate_up_small(fp, st)) return 0;
    COLI_MARK(3);
    if (!colib::launch_down_small(fp, st)) return 0;
  }
  COLI_MARK(4);
  colib::CombineParams cp;
  cp.T = T;
  cp.H = m->L.H;
  cp.k = k;
  cp.has_shared = m->has_shared ? 1 : 0;
  cp.y = m->y;
  cp.shared_y = m->y + (size_t)T * k * m->L.H;
  cp.slot = m->slot;
  cp.topk_w = m->topk_w;
  cp.out = (__nv_bfloat16 *)out_dev;
  cp.out32 = resid_io;
  cp.resid = resid_io;
  if (!colib::launch_combine(cp, st)) return 0;
  COLI_MARK(5);
#undef COLI_MARK
  if (prof) {
    CK(cudaEventSynchronize(m->ev[COLI_PHASES]), "phase event sync");
    for (int i = 0; i < COLI_PHASES; ++i) {
      float ms = 0.0f;
      CK(cudaEventElapsedTime(&ms, m->ev[i], m->ev[i + 1]), "phase event read");
      m->phase_ms[i] += ms;
    }
    m->phase_calls++;
  }
  return 1;
}

extern "C" int coli_b200_moe_block_dev(ColiMoe *m, const void *x_dev, void *out_dev, int T, void *stream) {
  if (!out_dev) {
    coli_set_error("moe_block_dev: null pointer");
    return 0;
  }
  return moe_block_impl(m, x_dev, out_dev, nullptr, T, stream);
}

// The step around the block in the reference's layer loop (forward.rs:376-393): post-attention
// RMSNorm of the f32 residual stream (math.rs:8-20), the MoE block on the normed rows rounded to
// bf16, and the residual add, which is fused into the combine so that the block output is never
// rounded on its way into the stream.
extern "C" int coli_b200_moe_layer_step_dev(ColiMoe *m, float *resid_dev, const float *post_ln_w_dev, float eps, int T,
                                            void *stream) {
  if (!check_T(m, T, "moe_layer_step_dev")) return 0;
  if (!resid_dev || !post_ln_w_dev) {
    coli_set_error("moe_layer_step_dev: null pointer");
    return 0;
  }
  if (!m->all_resident) {
    coli_set_error("moe_layer_step_dev: not every expert is resident on this rank");
    return 0;
  }
  if (T == 0) return 1;
  cudaStream_t st = pick_stream(m, stream);
  if (!colib::launch_rmsnorm_bf16(resid_dev, post_ln_w_dev, eps, m->x_stage, T, m->L.H, st)) return 0;
  return moe_block_impl(m, m->x_stage, nullptr, resid_dev, T, stream);
}

// Synchronises the device and reports whether any kernel of this handle gave up on a bounded wait.
extern "C" int coli_b200_moe_check(ColiMoe *m) {
  if (!m || !select_ctx(m->ctx)) return 0;
  CK(cudaDeviceSynchronize(), "moe_check sync");
  int st = 0;
  CK(cudaMemcpy(&st, m->status, sizeof(int), cudaMemcpyDeviceToHost), "status read");
  if (st != 0) {
    coli_set_error("a tcgen05 expert kernel abandoned a bounded wait (code %d: 1 copy, 2 MMA, 3 weight producer, 4 epilogue); results of that call are invalid", st);
    cudaMemset(m->status, 0, sizeof(int));
    return 0;
  }
  return coli_ep_check(m);
}

extern "C" int coli_b200_moe_last_routing(ColiMoe *m, int T, int32_t *topk_idx, float *topk_w) {
  if (!check_T(m, T, "moe_last_routing")) return 0;
  if (!coli_cuda_check(cudaDeviceSynchronize(), "routing read sync")) return 0;
  const size_t n = (size_t)T * m->L.k;
  if (topk_idx && !coli_cuda_check(cudaMemcpy(topk_idx, m->topk_idx, n * sizeof(int32_t), cudaMemcpyDeviceToHost), "routing read")) return 0;
  if (topk_w && !coli_cuda_check(cudaMemcpy(topk_w, m->topk_w, n * sizeof(float), cudaMemcpyDeviceToHost), "routing read")) return 0;
  return 1;
}

extern "C" int coli_b200_moe_block(ColiMoe *m, const void *x, void *out, int T, int32_t *topk_idx, float *topk_w) {
  if (!check_T(m, T, "moe_block")) return 0;
  if (!x || !out) {
    coli_set_error("moe_block: null pointer");
    return 0;
  }
  if (T == 0) return 1;
  std::lock_guard<std::mutex> lk(m->ctx->mu);
  cudaStream_t st = m->ctx->stream;
  const size_t bytes = (size_t)T * m->L.H * sizeof(__nv_bfloat16);
  CK(cudaMemcpyAsync(m->x_stage, x, bytes, cudaMemcpyHostToDevice, st), "moe_block input upload");
  if (!coli_b200_moe_block_dev(m, m->x_stage, m->out_stage, T, st)) return 0;
  CK(cudaMemcpyAsync(out, m->out_stage, bytes, cudaMemcpyDeviceToHost, st), "moe_block output download");
  const size_t n = (size_t)T * m->L.k;
  if (topk_idx) CK(cudaMemcpyAsync(topk_idx, m->topk_idx, n * sizeof(int32_t), cudaMemcpyDeviceToHost, st), "routing download");
  if (topk_w) CK(cudaMemcpyAsync(topk_w, m->topk_w, n * sizeof(float), cudaMemcpyDeviceToHost, st), "routing download");
  CK(cudaStreamSynchronize(st), "moe_block sync");
  int kst = 0;
  CK(cudaMemcpy(&kst, m->status, sizeof(int), cudaMemcpyDeviceToHost), "status read");
  if (kst != 0) {
    coli_set_error("a tcgen05 expert kernel abandoned a bounded wait (code %d); the output is invalid", kst);
    cudaMemset(m->status, 0, sizeof(int));
    return 0;
  }
  return 1;
}

// ---- stages (expert parallelism) ---------------------------------------------------------------------
// The expert-parallel block is assembled from these by the host (speedycolibri_b200/cluster.py):
//   topk (own tokens) -> all-gather tokens + routing -> gather_local -> experts -> combine_partial
//   -> reduce-scatter of the f32 partials -> finish (+ shared expert of the own tokens).
// Every size that crosses ranks is fixed by (T, H, k), so no step needs a host synchronisation.
extern "C" int coli_b200_moe_local_experts(const ColiMoe *m) { return m ? m->n_local_seg : 0; }

extern "C" int coli_b200_moe_topk_dev(ColiMoe *m, const void *x_dev, int T, int32_t *topk_idx_dev, float *topk_w_dev,
                                      void *stream) {
  if (!check_T(m, T, "moe_topk_dev")) return 0;
  if (T == 0) return 1;
  if (!x_dev || !topk_idx_dev || !topk_w_dev) {
    coli_set_error("moe_topk_dev: null pointer");
    return 0;
  }
  colib::RouteParams rp = route_params(m, x_dev, T);
  rp.topk_idx = topk_idx_dev;
  rp.topk_w = topk_w_dev;
  return colib::launch_router(rp, pick_stream(m, stream));
}

extern "C" int coli_b200_moe_gather_local_dev(ColiMoe *m, const void *x_dev, const int32_t *topk_idx_dev, int T,
                                              void *rows_dev, int32_t *seg_count_dev, int32_t *slot_dev, void *stream) {
  if (!check_T(m, T, "moe_gather_local_dev")) return 0;
  if (!x_dev || !topk_idx_dev || !rows_dev || !seg_count_dev || !slot_dev) {
    coli_set_error("moe_gather_local_dev: null pointer");
    return 0;
  }
  cudaStream_t st = pick_stream(m, stream);
  if (T == 0) return coli_cuda_check(cudaMemsetAsync(seg_count_dev, 0, sizeof(int32_t) * m->n_local_seg, st), "count clear") ? 1 : 0;
  colib::PermuteParams pp = permute_params(m, x_dev, T, false, colib::TC_MAX_TOKENS, rows_dev, seg_count_dev, slot_dev);
  pp.topk_idx = topk_idx_dev;
  pp.expert_slot = m->local_slot;
  pp.nseg_routed = m->n_local_seg;
  return colib::launch_permute(pp, st);
}

// scratch of a grouped-FFN run grows on demand (synchronises the device when it does)
static bool ensure_h(ColiMoe *m, SegScratch &sc, size_t rows) {
  if (rows <= sc.h_rows) return true;
  if (!coli_cuda_check(cudaDeviceSynchronize(), "scratch regrow sync")) return false;
  __half *nh = nullptr;
  if (!coli_cuda_check(cudaMalloc((void **)&nh, rows * m->L.I * sizeof(__half)), "scratch regrow")) return false;
  m->allocs.push_back(nh);  // the old block is released with the handle
  m->ws_bytes += rows * m->L.I * sizeof(__half);
  sc.h = nh;
  sc.h_rows = rows;
  return true;
}
static bool ensure_items(ColiMoe *m, SegScratch &sc, int need, int n_seg) {
  if (n_seg > sc.seg_cap) {
    if (!coli_cuda_check(cudaDeviceSynchronize(), "work list regrow sync")) return false;
    if (!ws_alloc(m, &sc.seg_off, (size_t)n_seg + 2)) return false;
    sc.seg_cap = n_seg;
  }
  if (!sc.n_items && !ws_alloc(m, &sc.n_items, 1)) return false;
  if (need <= sc.item_cap) return true;
  if (!coli_cuda_check(cudaDeviceSynchronize(), "work list regrow sync")) return false;
  sc.item_cap = need;
  return ws_alloc(m, &sc.item_seg, need) && ws_alloc(m, &sc.item_row0, need) && ws_alloc(m, &sc.item_nrows, need);
}

// rows_cap bounds the rows the buffers hold (the work list is sized from it); rows_expected only
// selects the kernel family, so that the choice is a function of shapes, never of data.
int coli_run_segments(ColiMoe *m, SegScratch &sc, const WeightRef *g, const WeightRef *u, const WeightRef *d,
                      const int32_t *seg_expert_dev, const void *rows_dev, const int32_t *seg_count_dev, int n_seg,
                      int rows_cap, int rows_expected, void *y_dev, cudaStream_t st) {
  if (rows_cap == 0 || n_seg == 0) return 1;
  const bool tc = use_tc_path(m->L.fmt, rows_expected, n_seg);
  const bool tct = tc && use_tct(m->L.fmt, rows_expected, n_seg);
  const int rpi = tc ? (tct ? tct_tile_tokens(rows_expected, n_seg) : colib::TC_MAX_TOKENS) : rows_per_item_for(m->L, rows_expected, n_seg);
  const int max_items = max_work_items(rows_cap, n_seg, rpi);
  if (!ensure_h(m, sc, (size_t)rows_cap) || !ensure_items(m, sc, max_items, n_seg)) return 0;
  if (!colib::launch_items_from_counts(seg_count_dev, n_seg, rpi, sc.seg_off, sc.item_seg, sc.item_row0, sc.item_nrows,
                                       sc.n_items, st))
    return 0;
  if (tc) {
    colib::TcParams tp;
    tp.fmt = m->L.fmt;
    tp.H = m->L.H;
    tp.I = m->L.I;
    tp.gate = g;
    tp.up = u;
    tp.down = d;
    tp.seg_expert = seg_expert_dev;
    tp.item_seg = sc.item_seg;
    tp.item_row0 = sc.item_row0;
    tp.item_nrows = sc.item_nrows;
    tp.n_items = sc.n_items;
    tp.max_items = max_items;
    tp.tile_tokens = rpi;
    tp.h = sc.h;
    tp.y = (__nv_bfloat16 *)y_dev;
    tp.status = m->status;
    tp.act = m->act;
    if (tct) return colib::launch_gate_up_tct(tp, rows_dev, rows_cap, m->sm_count, st) && colib::launch_down_tct(tp, rows_cap, m->sm_count, st);
    return colib::launch_gate_up_tc(tp, rows_dev, rows_cap, m->sm_count, st) && colib::launch_down_tc(tp, rows_cap, m->sm_count, st);
  }
  colib::FfnParams fp;
  fp.fmt = m->L.fmt;
  fp.H = m->L.H;
  fp.I = m->L.I;
  fp.gate = g;
  fp.up = u;
  fp.down = d;
  fp.seg_expert = seg_expert_dev;
  fp.item_seg = sc.item_seg;
  fp.item_row0 = sc.item_row0;
  fp.item_nrows = sc.item_nrows;
  fp.n_items = sc.n_items;
  fp.max_items = max_items;
  fp.rows_per_item = rpi;
  fp.items_expected = (rows_expected < n_seg ? rows_expected : n_seg) + rows_expected / rpi;
  fp.x = (const __half *)rows_dev;
  fp.row_token = nullptr;
  fp.h = sc.h;
  fp.y = (__nv_bfloat16 *)y_dev;
  fp.y32 = nullptr;
  fp.relu2_out = nullptr;
  fp.act = m->act;
  return colib::launch_ffn_small(fp, st);
}
static int run_segments(ColiMoe *m, const WeightRef *g, const WeightRef *u, const WeightRef *d, const int32_t *seg_expert_dev,
                        const void *rows_dev, const int32_t *seg_count_dev, int n_seg, int rows_cap, int rows_expected,
                        void *y_dev, cudaStream_t st) {
  return coli_run_segments(m, m->seg_main, g, u, d, seg_expert_dev, rows_dev, seg_count_dev, n_seg, rows_cap, rows_expected, y_dev, st);
}

extern "C" int coli_b200_moe_experts_dev(ColiMoe *m, const void *rows_dev, const int32_t *seg_count_dev, int rows_cap,
                                         int rows_expected, void *y_dev, void *stream) {
  if (!m || !select_ctx(m->ctx)) return 0;
  if (rows_cap < 0 || rows_expected < 0 || (rows_cap > 0 && (!rows_dev || !y_dev || !seg_count_dev))) {
    coli_set_error("moe_experts_dev: bad row bounds or null pointer");
    return 0;
  }
  if ((reinterpret_cast<uintptr_t>(rows_dev) | reinterpret_cast<uintptr_t>(y_dev)) & 15) {
    coli_set_error("moe_experts_dev: rows_dev and y_dev must be 16-byte aligned");
    return 0;
  }
  return run_segments(m, m->gate, m->up, m->down, m->seg_expert + m->first_local_seg, rows_dev, seg_count_dev, m->n_local_seg,
                      rows_cap, rows_expected < rows_cap ? rows_expected : rows_cap, y_dev, pick_stream(m, stream));
}

extern "C" int coli_b200_moe_shared_dev(ColiMoe *m, const void *x_dev, int T, void *y_dev, void *stream) {
  if (!check_T(m, T, "moe_shared_dev")) return 0;
  if (!m->has_shared) {
    coli_set_error("moe_shared_dev: the layer has no shared expert");
    return 0;
  }
  if (T == 0) return 1;
  if (!y_dev || (reinterpret_cast<uintptr_t>(y_dev) & 15)) {
    coli_set_error("moe_shared_dev: y_dev must be a 16-byte aligned device buffer");
    return 0;
  }
  cudaStream_t st = pick_stream(m, stream);
  // one segment of T rows; its count lives in seg_count[E]
  if (!coli_cuda_check(cudaMemcpyAsync(m->seg_count + m->L.E, &T, sizeof(int32_t), cudaMemcpyHostToDevice, st), "shared count"))
    return 0;
  if (!colib::launch_bf16_to_f16((const __nv_bfloat16 *)x_dev, m->x16, (size_t)T * m->L.H, st)) return 0;
  return run_segments(m, m->gate + m->L.E, m->up + m->L.E, m->down + m->L.E, nullptr, m->x16, m->seg_count + m->L.E, 1, T, T, y_dev, st);
}

extern "C" int coli_b200_moe_combine_partial_dev(ColiMoe *m, const void *y_rows_dev, const int32_t *slot_dev,
                                                 const float *topk_w_dev, float *partial_dev, int T, void *stream) {
  if (!check_T(m, T, "moe_combine_partial_dev")) return 0;
  if (T == 0) return 1;
  if (!y_rows_dev || !slot_dev || !topk_w_dev || !partial_dev) {
    coli_set_error("moe_combine_partial_dev: null pointer");
    return 0;
  }
  colib::CombineParams cp;
  cp.T = T;
  cp.H = m->L.H;
  cp.k = m->L.k;
  cp.has_shared = 0;
  cp.y = (const __nv_bfloat16 *)y_rows_dev;
  cp.shared_y = nullptr;
  cp.slot = slot_dev;
  cp.topk_w = topk_w_dev;
  cp.out = nullptr;
  cp.out32 = partial_dev;
  cp.resid = nullptr;
  return colib::launch_combine(cp, pick_stream(m, stream));
}

extern "C" int coli_b200_moe_finish_dev(ColiMoe *m, const float *partial_dev, const void *shared_y_dev, void *out_dev, int T,
                                        void *stream) {
  if (!check_T(m, T, "moe_finish_dev")) return 0;
  if (T == 0) return 1;
  if (!partial_dev || !out_dev) {
    coli_set_error("moe_finish_dev: null pointer");
    return 0;
  }
  return colib::launch_finish(partial_dev, (const __nv_bfloat16 *)shared_y_dev, (__nv_bfloat16 *)out_dev, T, m->L.H,
                              pick_stream(m, stream));
}

// sharding.rs:251-265
extern "C" uint64_t coli_b200_sharding_fingerprint(uint32_t num_nodes, uint32_t n_experts, const uint32_t *owner) {
  uint64_t h = 0xcbf29ce484222325ull;
  auto mix = [&](uint32_t v) {
    for (int b = 0; b < 4; ++b) {
      h ^= (uint64_t)((v >> (8 * b)) & 0xffu);
      h *= 0x00000100000001b3ull;
    }
  };
  mix(num_nodes);
  mix(n_experts);
  for (uint32_t e = 0; e < n_experts; ++e) mix(owner ? owner[e] : (uint32_t)((uint64_t)e * num_nodes / n_experts));
  return h;
}

// ---- the reference's host-pointer expert calls -------------------------------------------------------
// Same contract as backend_cuda.cu:3668-3806 / 4410-4792 (host f32 in, host f32 out, synchronous,
// one mutex per device held across the call).  Activations are rounded from f32 to f16 on the device
// (the kernels are W4A16 / W8A16, as the reference's GPU path is); outputs are written as f32.
// Kernel selection follows the row counts alone, as the reference's does (backend_cuda.cu:4738-4783
// switches kernels at 32 rows): from 8 rows per expert on average the group runs on the tcgen05
// kernels, whose y is rounded to bf16 before it is widened to f32; below that on the
// register-level kernel, which writes f32 directly.
namespace {
std::mutex g_group_stats_mu;  // backend_cuda.cu:98-100
uint64_t g_group_calls = 0, g_group_experts = 0, g_group_rows = 0;
double g_group_h2d_ms = 0.0, g_group_kernel_ms = 0.0, g_group_d2h_ms = 0.0;
}  // namespace
extern "C" void coli_cuda_group_stats(uint64_t *calls, uint64_t *experts, uint64_t *rows, double *h2d_ms, double *kernel_ms,
                                      double *d2h_ms) {
  std::lock_guard<std::mutex> lk(g_group_stats_mu);
  if (calls) *calls = g_group_calls;
  if (experts) *experts = g_group_experts;
  if (rows) *rows = g_group_rows;
  if (h2d_ms) *h2d_ms = g_group_h2d_ms;
  if (kernel_ms) *kernel_ms = g_group_kernel_ms;
  if (d2h_ms) *d2h_ms = g_group_d2h_ms;
}

static int run_host_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups, ColiCudaTensor *const *downs,
                          const int *rows, int count, float *y, const float *x, int want_fmt_a, int want_fmt_b,
                          const char *who) {
  if (!gates || !ups || !downs || !rows || !x || !y || count < 1 || !gates[0]) {
    coli_set_error("%s: null pointer or empty group", who);
    return 0;
  }
  const int device = gates[0]->device, D = gates[0]->I, I = gates[0]->O, fmt = gates[0]->fmt;
  long total = 0;
  for (int c = 0; c < count; ++c) {
    ColiCudaTensor *g = gates[c], *u = ups[c], *d = downs[c];
    if (!g || !u || !d || rows[c] < 1 || g->fmt != fmt || u->fmt != fmt || d->fmt != fmt ||
        (fmt != want_fmt_a && fmt != want_fmt_b) || g->device != device || u->device != device || d->device != device ||
        g->I != D || g->O != I || u->I != D || u->O != I || d->I != I || d->O != D) {
      coli_set_error("%s: expert %d has a mismatched format, shape or device", who, c);
      return 0;
    }
    total += rows[c];
  }
  if (D % 8 || I % 8) {
    coli_set_error("%s: D=%d and I=%d must be multiples of 8", who, D, I);
    return 0;
  }
  if (total > (1L << 24)) {
    coli_set_error("%s: %ld rows in one call", who, total);
    return 0;
  }
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  cudaStream_t st = ctx->stream;
  const int kfmt = coli_kernel_fmt(fmt);
  const bool tc = use_tc_path(kfmt, (int)total, count);
  const bool tct = tc && use_tct(kfmt, (int)total, count);
  const int avg = (int)((total + count - 1) / count);
  const int rpi = tc ? (tct ? tct_tile_tokens((int)total, count) : colib::TC_MAX_TOKENS) : (avg <= 8 ? 8 : avg <= 16 ? 16 : 32);
  const int max_items = max_work_items((int)total, count, rpi);
  const size_t xb = (size_t)total * D;
  // slots: 0 x f32 / y f32, 1 x f16, 2 h f16, 3 tables + counts + work list + status word, 4 y bf16 (tcgen05 path)
  const size_t tbl_bytes = sizeof(WeightRef) * 3 * count + sizeof(int32_t) * (2 * count + 2 + 3 * (size_t)max_items + 2);
  if (!reserve(ctx, 0, xb * sizeof(float)) || !reserve(ctx, 1, xb * sizeof(__half)) ||
      !reserve(ctx, 2, (size_t)total * I * sizeof(__half)) || !reserve(ctx, 3, tbl_bytes) ||
      (tc && !reserve(ctx, 4, xb * sizeof(__nv_bfloat16))))
    return 0;
  if (!ctx->ev[0])
    for (int i = 0; i < 4; ++i) CK(cudaEventCreate(&ctx->ev[i]), "event creation");
  std::vector<WeightRef> tbl(3 * (size_t)count);
  for (int c = 0; c < count; ++c) {
    tbl[c] = WeightRef{gates[c]->q, gates[c]->s, gates[c]->gscale, 0};
    tbl[count + c] = WeightRef{ups[c]->q, ups[c]->s, ups[c]->gscale, 0};
    tbl[2 * count + c] = WeightRef{downs[c]->q, downs[c]->s, downs[c]->gscale, 0};
  }
  WeightRef *d_tbl = (WeightRef *)ctx->buf[3];
  int32_t *d_cnt = (int32_t *)(d_tbl + 3 * (size_t)count);
  int32_t *d_off = d_cnt + count;
  int32_t *d_iseg = d_off + count + 1;
  int32_t *d_irow = d_iseg + max_items;
  int32_t *d_inr = d_irow + max_items;
  int32_t *d_nit = d_inr + max_items;
  int32_t *d_status = d_nit + 1;
  CK(cudaEventRecord(ctx->ev[0], st), "phase event");
  CK(cudaMemcpyAsync(ctx->buf[0], x, xb * sizeof(float), cudaMemcpyHostToDevice, st), "expert input upload");
  CK(cudaMemcpyAsync(d_tbl, tbl.data(), sizeof(WeightRef) * tbl.size(), cudaMemcpyHostToDevice, st), "expert table upload");
  CK(cudaMemcpyAsync(d_cnt, rows, sizeof(int32_t) * count, cudaMemcpyHostToDevice, st), "row count upload");
  CK(cudaMemsetAsync(d_status, 0, sizeof(int32_t), st), "status clear");
  CK(cudaEventRecord(ctx->ev[1], st), "phase event");
  CK(cudaStreamSynchronize(st), "expert upload sync");  // tbl is a local; rows/x belong to the caller
  if (!colib::launch_f32_to_f16((const float *)ctx->buf[0], (__half *)ctx->buf[1], xb, st)) return 0;
  if (!colib::launch_items_from_counts(d_cnt, count, rpi, d_off, d_iseg, d_irow, d_inr, d_nit, st)) return 0;
  if (tc) {
    colib::TcParams tp;
    tp.fmt = kfmt;
    tp.H = D;
    tp.I = I;
    tp.gate = d_tbl;
    tp.up = d_tbl + count;
    tp.down = d_tbl + 2 * count;
    tp.seg_expert = nullptr;
    tp.item_seg = d_iseg;
    tp.item_row0 = d_irow;
    tp.item_nrows = d_inr;
    tp.n_items = d_nit;
    tp.max_items = max_items;
    tp.tile_tokens = rpi;
    tp.h = (__half *)ctx->buf[2];
    tp.y = (__nv_bfloat16 *)ctx->buf[4];
    tp.status = d_status;
    tp.act = current_activation();
    const int sms = ctx->sm_count;
    const int ok = tct ? colib::launch_gate_up_tct(tp, ctx->buf[1], (int)total, sms, st) && colib::launch_down_tct(tp, (int)total, sms, st)
                       : colib::launch_gate_up_tc(tp, ctx->buf[1], (int)total, sms, st) && colib::launch_down_tc(tp, (int)total, sms, st);
    if (!ok || !colib::launch_bf16_to_f32((const __nv_bfloat16 *)ctx->buf[4], (float *)ctx->buf[0], xb, st)) return 0;
  } else {
    colib::FfnParams fp;
    fp.fmt = kfmt;
    fp.H = D;
    fp.I = I;
    fp.gate = d_tbl;
    fp.up = d_tbl + count;
    fp.down = d_tbl + 2 * count;
    fp.seg_expert = nullptr;
    fp.item_seg = d_iseg;
    fp.item_row0 = d_irow;
    fp.item_nrows = d_inr;
    fp.n_items = d_nit;
    fp.max_items = max_items;
    fp.rows_per_item = rpi;
    fp.items_expected = max_items;
    fp.x = (const __half *)ctx->buf[1];
    fp.row_token = nullptr;
    fp.h = (__half *)ctx->buf[2];
    fp.y = nullptr;
    fp.y32 = (float *)ctx->buf[0];  // x f32 is dead once converted
    fp.relu2_out = nullptr;
    fp.act = current_activation();
    if (!colib::launch_ffn_small(fp, st)) return 0;
  }
  CK(cudaEventRecord(ctx->ev[2], st), "phase event");
  int32_t kst = 0;
  CK(cudaMemcpyAsync(y, ctx->buf[0], xb * sizeof(float), cudaMemcpyDeviceToHost, st), "expert output download");
  if (tc) CK(cudaMemcpyAsync(&kst, d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, st), "status read");
  CK(cudaEventRecord(ctx->ev[3], st), "phase event");
  CK(cudaStreamSynchronize(st), "expert call sync");
  if (kst != 0) {
    coli_set_error("%s: a tcgen05 expert kernel abandoned a bounded wait (code %d); the output is invalid", who, (int)kst);
    return 0;
  }
  float ms[3] = {0.0f, 0.0f, 0.0f};
  for (int i = 0; i < 3; ++i) cudaEventElapsedTime(&ms[i], ctx->ev[i], ctx->ev[i + 1]);
  {
    std::lock_guard<std::mutex> sl(g_group_stats_mu);
    g_group_calls++;
    g_group_experts += (uint64_t)count;
    g_group_rows += (uint64_t)total;
    g_group_h2d_ms += ms[0];
    g_group_kernel_ms += ms[1];
    g_group_d2h_ms += ms[2];
  }
  return 1;
}

extern "C" int coli_cuda_expert_group_nvfp4(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                            ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                                            const float *x) {
  return run_host_group(gates, ups, downs, rows, count, y, x, COLI_FMT_NVFP4, COLI_FMT_NVFP4, "expert_group_nvfp4");
}
extern "C" int coli_cuda_expert_mlp_nvfp4(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                          const float *x, int S) {
  return run_host_group(&gate, &up, &down, &S, 1, y, x, COLI_FMT_NVFP4, COLI_FMT_NVFP4, "expert_mlp_nvfp4");
}
extern "C" int coli_cuda_expert_mlp_fp8(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                        const float *x, int S) {
  return run_host_group(&gate, &up, &down, &S, 1, y, x, COLI_FMT_E4M3_ROW, COLI_FMT_FP8_B128, "expert_mlp_fp8");
}

// MXFP4 experts (backend_cuda.h:71-79, backend_cuda.cu:5707): the same two launches; the handles
// hold the weights in the NVFP4 resident form (see coli_cuda_tensor_wrap_mxfp4).
extern "C" int coli_cuda_expert_mlp_mxfp4(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                          const float *x, int S) {
  return run_host_group(&gate, &up, &down, &S, 1, y, x, COLI_FMT_MXFP4, COLI_FMT_MXFP4, "expert_mlp_mxfp4");
}
extern "C" int coli_cuda_expert_group_mxfp4(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups,
                                            ColiCudaTensor *const *downs, const int *rows, int count, float *y,
                                            const float *x) {
  return run_host_group(gates, ups, downs, rows, count, y, x, COLI_FMT_MXFP4, COLI_FMT_MXFP4, "expert_group_mxfp4");
}
extern "C" int coli_cuda_expert_mlp_mxfp4_situ(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y,
                                               const float *x, int S, float beta, float linear_beta) {
  (void)gate, (void)up, (void)down, (void)y, (void)x, (void)S, (void)beta, (void)linear_beta;
  coli_set_error("expert_mlp_mxfp4_situ: the situ activation is not part of this library (declined)");
  return 0;
}

// Gateless ReLU^2 experts (Nemotron-H): y = down(relu(up x)^2), moe.rs:1189-1199;
// backend_cuda.h:131-160.  Two launches for the whole group: the up projection with the
// activation in its epilogue, then the down projection.  x, y hold sum(rows) rows of up->I
// values in call order.
static int run_host_group_relu2(ColiCudaTensor *const *ups, ColiCudaTensor *const *downs, const int *rows, int count,
                                float *y, const float *x, const char *who) {
  if (!ups || !downs || !rows || !x || !y || count < 1 || !ups[0]) {
    coli_set_error("%s: null pointer or empty group", who);
    return 0;
  }
  const int device = ups[0]->device, D = ups[0]->I, I = ups[0]->O;
  long total = 0;
  for (int c = 0; c < count; ++c) {
    ColiCudaTensor *u = ups[c], *d = downs[c];
    if (!u || !d || rows[c] < 1 || u->fmt != COLI_FMT_NVFP4 || d->fmt != COLI_FMT_NVFP4 || u->device != device ||
        d->device != device || u->I != D || u->O != I || d->I != I || d->O != D) {
      coli_set_error("%s: expert %d has a mismatched format, shape or device", who, c);
      return 0;
    }
    total += rows[c];
  }
  if (D % 8 || I % 8) {
    coli_set_error("%s: D=%d and I=%d must be multiples of 8", who, D, I);
    return 0;
  }
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  cudaStream_t st = ctx->stream;
  const int avg = (int)((total + count - 1) / count);
  const int rpi = avg <= 8 ? 8 : avg <= 16 ? 16 : 32;
  const int max_items = max_work_items((int)total, count, rpi);
  const size_t xb = (size_t)total * D;
  // slots: 0 x f32 / y f32, 1 x f16, 2 h f16, 3 tables + counts + work list
  const size_t tbl_bytes = sizeof(WeightRef) * 2 * count + sizeof(int32_t) * (2 * count + 2 + 3 * (size_t)max_items + 1);
  if (!reserve(ctx, 0, xb * sizeof(float)) || !reserve(ctx, 1, xb * sizeof(__half)) ||
      !reserve(ctx, 2, (size_t)total * I * sizeof(__half)) || !reserve(ctx, 3, tbl_bytes))
    return 0;
  std::vector<WeightRef> tbl(2 * (size_t)count);
  for (int c = 0; c < count; ++c) {
    tbl[c] = WeightRef{ups[c]->q, ups[c]->s, ups[c]->gscale, 0};
    tbl[count + c] = WeightRef{downs[c]->q, downs[c]->s, downs[c]->gscale, 0};
  }
  WeightRef *d_tbl = (WeightRef *)ctx->buf[3];
  int32_t *d_cnt = (int32_t *)(d_tbl + 2 * (size_t)count);
  int32_t *d_off = d_cnt + count;
  int32_t *d_iseg = d_off + count + 1;
  int32_t *d_irow = d_iseg + max_items;
  int32_t *d_inr = d_irow + max_items;
  int32_t *d_nit = d_inr + max_items;
  CK(cudaMemcpyAsync(ctx->buf[0], x, xb * sizeof(float), cudaMemcpyHostToDevice, st), "expert input upload");
  CK(cudaMemcpyAsync(d_tbl, tbl.data(), sizeof(WeightRef) * tbl.size(), cudaMemcpyHostToDevice, st), "expert table upload");
  CK(cudaMemcpyAsync(d_cnt, rows, sizeof(int32_t) * count, cudaMemcpyHostToDevice, st), "row count upload");
  CK(cudaStreamSynchronize(st), "expert upload sync");  // tbl is a local; rows/x belong to the caller
  if (!colib::launch_f32_to_f16((const float *)ctx->buf[0], (__half *)ctx->buf[1], xb, st)) return 0;
  if (!colib::launch_items_from_counts(d_cnt, count, rpi, d_off, d_iseg, d_irow, d_inr, d_nit, st)) return 0;
  colib::FfnParams fp;
  fp.fmt = COLI_FMT_NVFP4;
  fp.seg_expert = nullptr;
  fp.item_seg = d_iseg;
  fp.item_row0 = d_irow;
  fp.item_nrows = d_inr;
  fp.n_items = d_nit;
  fp.max_items = max_items;
  fp.rows_per_item = rpi;
  fp.items_expected = max_items;
  fp.x = nullptr;
  fp.row_token = nullptr;
  fp.y = nullptr;
  fp.act = current_activation();
  // up: rows [total, D] -> relu^2 -> h [total, I]   (the kernel's "down" form: contracts its I, writes its H)
  fp.H = I;
  fp.I = D;
  fp.gate = fp.up = fp.down = d_tbl;
  fp.h = (__half *)ctx->buf[1];
  fp.y32 = nullptr;
  fp.relu2_out = (__half *)ctx->buf[2];
  if (!colib::launch_down_small(fp, st)) return 0;
  // down: h [total, I] -> y [total, D]
  fp.H = D;
  fp.I = I;
  fp.gate = fp.up = fp.down = d_tbl + count;
  fp.h = (__half *)ctx->buf[2];
  fp.y32 = (float *)ctx->buf[0];  // x f32 is dead once converted
  fp.relu2_out = nullptr;
  if (!colib::launch_down_small(fp, st)) return 0;
  CK(cudaMemcpyAsync(y, ctx->buf[0], xb * sizeof(float), cudaMemcpyDeviceToHost, st), "expert output download");
  CK(cudaStreamSynchronize(st), "expert call sync");
  return 1;
}
// `exact` asks the reference for per-row kernels so that results do not depend on S
// (gpu.rs:122-146); here a row's result never depends on the other rows of the call, so the flag
// changes nothing.
extern "C" int coli_cuda_expert_mlp_nvfp4_relu2(ColiCudaTensor *up, ColiCudaTensor *down, float *y, const float *x, int S,
                                                int exact) {
  (void)exact;
  return run_host_group_relu2(&up, &down, &S, 1, y, x, "expert_mlp_nvfp4_relu2");
}
extern "C" int coli_cuda_expert_group_nvfp4_relu2(ColiCudaTensor *const *ups, ColiCudaTensor *const *downs, const int *rows,
                                                  int count, float *y, const float *x) {
  return run_host_group_relu2(ups, downs, rows, count, y, x, "expert_group_nvfp4_relu2");
}
extern "C" int coli_cuda_expert_seg_nvfp4_relu2(ColiCudaTensor *const *ups, ColiCudaTensor *const *downs, const int *rows,
                                                int count, float *y, const float *x) {
  return run_host_group_relu2(ups, downs, rows, count, y, x, "expert_seg_nvfp4_relu2");
}

// The format-agnostic forms of the two calls above (backend_cuda.h:107-109, 136-140): any resident
// expert format this library holds (NVFP4, e4m3 per row, e4m3 128x128); the reference's int8 /
// int2 / f32 experts are not resident formats here and are declined.
extern "C" int coli_cuda_expert_mlp(ColiCudaTensor *gate, ColiCudaTensor *up, ColiCudaTensor *down, float *y, const float *x,
                                    int S) {
  const int fmt = gate ? gate->fmt : -1;
  if (!fmt_supported(fmt)) {
    coli_set_error("expert_mlp: format %d is not a resident expert format of this library", fmt);
    return 0;
  }
  return run_host_group(&gate, &up, &down, &S, 1, y, x, fmt, fmt, "expert_mlp");
}
extern "C" int coli_cuda_expert_group(ColiCudaTensor *const *gates, ColiCudaTensor *const *ups, ColiCudaTensor *const *downs,
                                      const int *rows, int count, float *y, const float *x) {
  const int fmt = (gates && count > 0 && gates[0]) ? gates[0]->fmt : -1;
  if (!fmt_supported(fmt)) {
    coli_set_error("expert_group: format %d is not a resident expert format of this library", fmt);
    return 0;
  }
  return run_host_group(gates, ups, downs, rows, count, y, x, fmt, fmt, "expert_group");
}

// y[S,O] = x[S,I] @ W[O,I]^T for one resident quantised matrix: the down-projection kernel with
// the whole input as a single segment.
static int run_host_matmul(ColiCudaTensor *w, float *y, const float *x, int S, const char *who) {
  if (!w || !x || !y || S < 1 || !fmt_supported(w->fmt)) {
    coli_set_error("%s: null pointer, empty input or a format that is not resident here", who);
    return 0;
  }
  if (w->I % 8) {
    coli_set_error("%s: I=%d must be a multiple of 8", who, w->I);
    return 0;
  }
  DeviceContext *ctx = find_ctx(w->device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  cudaStream_t st = ctx->stream;
  const int I = w->I, O = w->O;
  const int rpi = S <= 8 ? 8 : S <= 16 ? 16 : 32;
  const int max_items = max_work_items(S, 1, rpi);
  const size_t xb = (size_t)S * I, yb = (size_t)S * O;
  // slots: 0 x f32, 1 x f16, 2 y f32, 3 table + count + work list
  const size_t tbl_bytes = sizeof(WeightRef) + sizeof(int32_t) * (1 + 2 + 3 * (size_t)max_items + 1);
  if (!reserve(ctx, 0, xb * sizeof(float)) || !reserve(ctx, 1, xb * sizeof(__half)) || !reserve(ctx, 2, yb * sizeof(float)) ||
      !reserve(ctx, 3, tbl_bytes))
    return 0;
  const WeightRef ref{w->q, w->s, w->gscale, 0};
  WeightRef *d_tbl = (WeightRef *)ctx->buf[3];
  int32_t *d_cnt = (int32_t *)(d_tbl + 1);
  int32_t *d_off = d_cnt + 1;
  int32_t *d_iseg = d_off + 2;
  int32_t *d_irow = d_iseg + max_items;
  int32_t *d_inr = d_irow + max_items;
  int32_t *d_nit = d_inr + max_items;
  CK(cudaMemcpyAsync(ctx->buf[0], x, xb * sizeof(float), cudaMemcpyHostToDevice, st), "matmul input upload");
  CK(cudaMemcpyAsync(d_tbl, &ref, sizeof(WeightRef), cudaMemcpyHostToDevice, st), "matmul table upload");
  CK(cudaMemcpyAsync(d_cnt, &S, sizeof(int32_t), cudaMemcpyHostToDevice, st), "matmul row count upload");
  CK(cudaStreamSynchronize(st), "matmul upload sync");  // ref and S are locals
  if (!colib::launch_f32_to_f16((const float *)ctx->buf[0], (__half *)ctx->buf[1], xb, st)) return 0;
  if (!colib::launch_items_from_counts(d_cnt, 1, rpi, d_off, d_iseg, d_irow, d_inr, d_nit, st)) return 0;
  colib::FfnParams fp;
  fp.fmt = coli_kernel_fmt(w->fmt);
  fp.H = O;  // the kernel's "down" form contracts over its I and writes H features per row
  fp.I = I;
  fp.gate = fp.up = fp.down = d_tbl;
  fp.seg_expert = nullptr;
  fp.item_seg = d_iseg;
  fp.item_row0 = d_irow;
  fp.item_nrows = d_inr;
  fp.n_items = d_nit;
  fp.max_items = max_items;
  fp.rows_per_item = rpi;
  fp.items_expected = max_items;
  fp.x = nullptr;
  fp.row_token = nullptr;
  fp.h = (__half *)ctx->buf[1];
  fp.y = nullptr;
  fp.y32 = (float *)ctx->buf[2];
  fp.relu2_out = nullptr;
  fp.act = current_activation();
  if (!colib::launch_down_small(fp, st)) return 0;
  CK(cudaMemcpyAsync(y, ctx->buf[2], yb * sizeof(float), cudaMemcpyDeviceToHost, st), "matmul output download");
  CK(cudaStreamSynchronize(st), "matmul sync");
  return 1;
}

// backend_cuda.h:127-129 (backend_cuda.cu:3102-3128): the first call copies the weight into HBM
// through *tensor, later calls reuse it.
extern "C" int coli_cuda_matmul_nvfp4(ColiCudaTensor **tensor, float *y, const float *x, const void *weights, const void *bscale,
                                      float gscale, int S, int I, int O, int device) {
  if (!tensor) {
    coli_set_error("coli_cuda_matmul_nvfp4: null tensor slot");
    return 0;
  }
  if (!coli_cuda_tensor_wrap_nvfp4(tensor, weights, bscale, gscale, I, O, device)) return 0;
  return run_host_matmul(*tensor, y, x, S, "coli_cuda_matmul_nvfp4");
}

// Router GEMM through the generic matmul entry (fmt 0 only): gpu.rs:2219-2249 -> backend_cuda.cu:3063-3075.
extern "C" int coli_cuda_matmul(ColiCudaTensor **tensor, float *y, const float *x, const void *weights,
                                const float *scales, int fmt, int S, int I, int O, int device) {
  (void)scales;
  if (fmt != COLI_FMT_F32) {
    coli_set_error("coli_cuda_matmul: only fmt 0 (the f32 router GEMM) goes through this entry; got %d", fmt);
    return 0;
  }
  if (!tensor || !y || !x || S < 1 || I < 1 || O < 1 || (!*tensor && !weights)) {
    coli_set_error("coli_cuda_matmul: bad argument");
    return 0;
  }
  DeviceContext *ctx = find_ctx(device);
  if (!select_ctx(ctx)) return 0;
  std::lock_guard<std::mutex> lk(ctx->mu);
  cudaStream_t st = ctx->stream;
  if (*tensor) {
    if (!existing_matches(*tensor, fmt, I, O, device)) {
      coli_set_error("coli_cuda_matmul: cached tensor does not match fmt/I/O/device");
      return 0;
    }
  } else {
    ColiCudaTensor *t = static_cast<ColiCudaTensor *>(calloc(1, sizeof(ColiCudaTensor)));
    if (!t) return 0;
    t->fmt = fmt;
    t->I = I;
    t->O = O;
    t->device = device;
    t->q_bytes = sizeof(float) * (size_t)I * O;
    if (!coli_cuda_check(cudaMalloc((void **)&t->q, t->q_bytes), "tensor allocation") ||
        !coli_cuda_check(cudaMemcpyAsync(t->q, weights, t->q_bytes, cudaMemcpyHostToDevice, st), "tensor upload") ||
        !coli_cuda_check(cudaStreamSynchronize(st), "tensor upload sync")) {
      if (t->q) cudaFree(t->q);
      free(t);
      return 0;
    }
    ctx->tensor_count++;
    ctx->tensor_bytes += t->q_bytes;
    *tensor = t;
  }
  const size_t xb = sizeof(float) * (size_t)S * I, yb = sizeof(float) * (size_t)S * O;
  if (!reserve(ctx, 0, xb) || !reserve(ctx, 1, yb)) return 0;
  CK(cudaMemcpyAsync(ctx->buf[0], x, xb, cudaMemcpyHostToDevice, st), "matmul input upload");
  if (!colib::launch_matmul_f32_seq((const float *)ctx->buf[0], (const float *)(*tensor)->q, (float *)ctx->buf[1], S, I, O, st))
    return 0;
  CK(cudaMemcpyAsync(y, ctx->buf[1], yb, cudaMemcpyDeviceToHost, st), "matmul output download");
  CK(cudaStreamSynchronize(st), "matmul sync");
  return 1;
}
