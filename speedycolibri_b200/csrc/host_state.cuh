// Host-side state shared by the translation units that implement the C ABI (abi.cu: lifecycle,
// handles, the single-GPU block; ep.cu: the expert-parallel block).
#pragma once
#include <mutex>
#include <vector>

#include "internal.cuh"

struct DeviceContext {
  int device = -1;
  cudaStream_t stream = nullptr;
  std::mutex mu;  // held across a whole host-pointer call, as the reference does
  size_t tensor_count = 0, tensor_bytes = 0;
  // scratch of the host-pointer expert calls, grown on demand
  void *buf[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t cap[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};  // phase marks of the host-pointer group calls
  int sm_count = 0;
};
DeviceContext *coli_find_ctx(int device);
bool coli_select_ctx(DeviceContext *c);

// Scratch of one grouped-FFN run (work list, segment offsets, the intermediate h rows).  The block
// owns one; the expert-parallel block owns a second one so that its shared expert can run on
// another stream while the routed experts use the first.
struct SegScratch {
  __half *h = nullptr;  // [h_rows, I]
  size_t h_rows = 0;
  int32_t *item_seg = nullptr, *item_row0 = nullptr, *item_nrows = nullptr, *n_items = nullptr, *seg_off = nullptr;
  int item_cap = 0;
  int seg_cap = 0;      // seg_off holds seg_cap + 1 entries
};

struct ColiEp;  // expert-parallel state (ep.cu), null on a single-GPU handle

struct ColiMoe {
  ColiMoeLayer L;
  DeviceContext *ctx;
  int max_tokens;
  int nseg;            // E (+1 with a shared expert)
  bool has_shared;
  bool all_resident;
  std::vector<int32_t> h_expert_slot;  // expert -> segment position in (owner, id) order
  std::vector<int32_t> h_seg_expert;   // segment position -> weight-table index
  std::vector<int32_t> h_owner;        // expert -> owning rank
  int first_local_seg, n_local_seg;
  // device tables
  __nv_bfloat16 *router_w;
  float *select_bias, *logit_bias;
  WeightRef *gate, *up, *down;  // [E+1], entry E = shared expert
  int32_t *expert_slot, *seg_expert;
  int32_t *local_slot;  // expert -> position among this rank's experts, or -1
  // workspace
  float *logits, *topk_w;
  int32_t *topk_idx, *local_rank, *chunk_cnt, *seg_count, *seg_off, *slot, *row_token;
  int32_t *item_seg, *item_row0, *item_nrows, *n_items;
  int item_cap;
  SegScratch seg_main;  // views of h / the work list / seg_off above, for run_segments
  __nv_bfloat16 *y, *x_stage, *out_stage;
  __half *h;    // intermediate rows of the expert FFN
  __half *x16;  // token-order f16 copy of the activations (small-batch path, shared expert stage)
  __half *xg;   // gathered f16 rows for the tcgen05 path (null when max_tokens never reaches it)
  int *status;        // device status word of the tcgen05 kernels
  unsigned int *ticket;  // device word of the fused decode front end (zero between launches)
  colib::ActParams act;  // the process-wide activation setting when the handle was created
  int sm_count;
  size_t h_rows_cap;  // rows the h scratch holds
  size_t ws_bytes;
  std::vector<void *> allocs;
  // tracing
  bool profiling;
  cudaEvent_t ev[COLI_PHASES + 1];
  float phase_ms[COLI_PHASES];
  int phase_calls;
  ColiEp *ep;
};


template <class T>
static inline bool ws_alloc(ColiMoe *m, T **p, size_t count) {
  const size_t bytes = (count ? count : 1) * sizeof(T);
  if (!coli_cuda_check(cudaMalloc((void **)p, bytes), "workspace allocation")) return false;
  m->allocs.push_back(*p);
  m->ws_bytes += bytes;
  return true;
}


// kernel-family selection: pure functions of (format, rows, segments)
bool coli_use_tct(int fmt, int rows, int nseg);
int coli_tct_tile_tokens(int rows, int nseg);
bool coli_use_tc_path(int fmt, int rows, int nseg);
int coli_rows_per_item_for(int rows, int nseg);

bool coli_check_T(ColiMoe *m, int T, const char *who);
colib::RouteParams coli_route_params(ColiMoe *m, const void *x_dev, int T);
colib::PermuteParams coli_permute_params(ColiMoe *m, const void *x_dev, int T, bool with_shared, int rpi, void *rows_dev,
                                         int32_t *seg_count, int32_t *slot);
// Grouped FFN over expert-contiguous rows whose per-segment counts are on the device.  rows_cap
// bounds the rows the buffers hold (the work list is sized from it); rows_expected only selects
// the kernel family.
int coli_run_segments(ColiMoe *m, SegScratch &sc, const WeightRef *g, const WeightRef *u, const WeightRef *d,
                      const int32_t *seg_expert_dev, const void *rows_dev, const int32_t *seg_count_dev, int n_seg,
                      int rows_cap, int rows_expected, void *y_dev, cudaStream_t st);
// ep.cu
void coli_ep_destroy(ColiMoe *m);
// Allocate the expert-parallel state of a handle created with ep_world > 1 (idempotent); `comm` is an
// ncclComm_t or null (a handle without a communicator can only take part in the one-GPU emulation).
int coli_ep_ensure(ColiMoe *m, void *comm);
int coli_ep_check(ColiMoe *m);
