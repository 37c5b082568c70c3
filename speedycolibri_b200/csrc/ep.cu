// Expert-parallel MoE block: one call per rank, experts sharded over the GPUs of one box.
//
// It takes the place of crates/colibri-engine/src/moe.rs:1737-1794 `moe_sharded` and
// 1620-1734 `sharded_experts_partial`, whose transport (crates/colibri-cluster/src/transport.rs:33-58
// over TCP, rank 0 driving every peer with all of x) is replaced by an all-to-all over NCCL
// send/recv.  What is kept from the reference: the expert -> rank map (sharding.rs:197-203 or an
// explicit table), "activations travel, weights never do", and that a failed peer fails the call.
//
// Every rank holds T_local tokens and the experts the map gives it.  One call, on the caller's
// stream S plus one auxiliary stream A for the shared expert:
//   S  router + score + top-k of the own tokens                          (routing.cu)
//   S  plan: per destination rank the ascending list of own tokens that have at least one expert
//      there (a token is sent ONCE per rank however many of its k experts live there), the number of
//      (token, kk) pairs per rank, and for every own pair the row its result will come back in
//   S  pack: token rows + their k expert ids into one send segment per rank; the rows for this
//      rank's own experts go straight into the receive buffer
//   A  shared expert of the own tokens (replicated weights), overlapping everything below
//   S  all-gather of the 2 x world counts, copied to pinned host memory; THE HOST WAITS HERE ONCE
//      (send/recv sizes must be known to the host that posts them)
//   S  dispatch: grouped ncclSend / ncclRecv of bf16 rows and int32 ids
//   S  permute the received tokens' pairs that hit resident experts into expert-contiguous rows,
//      grouped expert FFN (the same kernels as the single-GPU block)
//   S  return pack: result rows in (source rank, token, kk) order; grouped ncclSend / ncclRecv back
//   S  weighted combine on the home rank in the token's own kk order + shared expert, one rounding
// The result rows travel unweighted and the home rank applies the routing weights, so the f32
// accumulation (moe.rs:1549-1553) is the single-GPU block's, whatever the number of ranks.
//
// That is the NCCL transport.  The default ("direct") transport keeps the same plan, layouts and
// kernels downstream but moves the rows itself: every rank's receive buffers sit in one slab that the
// peers map through CUDA IPC, the pack kernels store rows, ids and counts straight into it over
// NVLink, and a flag barrier with a bounded wait (k_ep_flag_barrier) stands where the collectives
// stood, so the host never waits.
//
// NCCL is bound at run time (dlopen of libnccl.so.2, the copy already in the process if there is
// one), so the library loads and runs single-GPU without it.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "host_state.cuh"

// ---- NCCL, bound at run time ------------------------------------------------------------------------
typedef struct ncclComm *ncclComm_t;
typedef struct {
  char internal[128];
} ncclUniqueId;
typedef int ncclResult_t;  // 0 = ncclSuccess
enum { COLI_NCCL_INT8 = 0, COLI_NCCL_INT32 = 2, COLI_NCCL_BF16 = 9 };  // ncclDataType_t values

namespace {
struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId *);
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
  ncclResult_t (*CommDestroy)(ncclComm_t);
  ncclResult_t (*CommCount)(const ncclComm_t, int *);
  ncclResult_t (*CommUserRank)(const ncclComm_t, int *);
  ncclResult_t (*GroupStart)(void);
  ncclResult_t (*GroupEnd)(void);
  ncclResult_t (*Send)(const void *, size_t, int, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*Recv)(void *, size_t, int, int, ncclComm_t, cudaStream_t);
  ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t);
  const char *(*GetErrorString)(ncclResult_t);
};
std::mutex g_nccl_mu;
NcclApi g_nccl;
int g_nccl_state = 0;  // 0 not tried, 1 loaded, -1 unavailable

NcclApi *nccl_api() {
  std::lock_guard<std::mutex> lk(g_nccl_mu);
  if (g_nccl_state == 1) return &g_nccl;
  if (g_nccl_state < 0) {
    coli_set_error("expert parallelism: libnccl.so.2 could not be loaded");
    return nullptr;
  }
  void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) {
    g_nccl_state = -1;
    coli_set_error("expert parallelism: libnccl.so.2 could not be loaded (%s)", dlerror());
    return nullptr;
  }
  bool ok = true;
  auto sym = [&](const char *name) -> void * {
    void *p = dlsym(h, name);
    if (!p) ok = false;
    return p;
  };
  g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))sym("ncclGetUniqueId");
  g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))sym("ncclCommInitRank");
  g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))sym("ncclCommDestroy");
  g_nccl.CommCount = (decltype(g_nccl.CommCount))sym("ncclCommCount");
  g_nccl.CommUserRank = (decltype(g_nccl.CommUserRank))sym("ncclCommUserRank");
  g_nccl.GroupStart = (decltype(g_nccl.GroupStart))sym("ncclGroupStart");
  g_nccl.GroupEnd = (decltype(g_nccl.GroupEnd))sym("ncclGroupEnd");
  g_nccl.Send = (decltype(g_nccl.Send))sym("ncclSend");
  g_nccl.Recv = (decltype(g_nccl.Recv))sym("ncclRecv");
  g_nccl.AllGather = (decltype(g_nccl.AllGather))sym("ncclAllGather");
  g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))sym("ncclGetErrorString");
  if (!ok) {
    g_nccl_state = -1;
    coli_set_error("expert parallelism: libnccl.so.2 lacks a required symbol");
    return nullptr;
  }
  g_nccl_state = 1;
  return &g_nccl;
}
bool nccl_ok(NcclApi *api, ncclResult_t r, const char *what) {
  if (r == 0) return true;
  coli_set_error("%s: NCCL error %d (%s)", what, (int)r, api->GetErrorString ? api->GetErrorString(r) : "?");
  return false;
}
}  // namespace

constexpr int EP_MAX_WORLD = 8;  // the GPUs of one NVSwitch box
constexpr uint32_t EP_BARRIER_POLLS = 1u << 23;  // x 200 ns of sleep between polls: about two seconds
constexpr int EP_MAX_K = 16;     // a token's destination ranks are packed 4 bits per kk

// Stages timed when profiling is on (coli_b200_ep_stage_ms).
enum { EPS_ROUTE = 0, EPS_PLAN_PACK, EPS_COUNTS, EPS_DISPATCH, EPS_GATHER, EPS_EXPERTS, EPS_RETURN_PACK, EPS_RETURN, EPS_COMBINE, EPS_N };

struct ColiEp {
  int rank = 0, world = 1;
  ncclComm_t comm = nullptr;
  cudaStream_t aux = nullptr;
  cudaEvent_t ev_x = nullptr, ev_shared = nullptr, ev_counts = nullptr;
  uint8_t *owner = nullptr;        // [E] expert -> rank
  int32_t *cnt = nullptr;          // [2*world]: tokens sent to d, (token, kk) pairs owned by d
  int32_t *send_off = nullptr;     // [world] first row of d's send segment (self: unused)
  int32_t *all_cnt = nullptr;      // [world][2*world], all-gathered
  int32_t *h_all_cnt = nullptr;    // pinned host copy
  int32_t *send_pos = nullptr;     // [T*world] position of token t in d's list, or -1
  int32_t *home_slot = nullptr;    // [T*k] row of pair (t, kk) in ret_recv
  __nv_bfloat16 *send_x = nullptr, *recv_x = nullptr;  // token rows
  int32_t *send_meta = nullptr, *recv_meta = nullptr;  // their k expert ids
  int32_t *recv_slot = nullptr;    // [R*k] row of a received pair among the resident experts' rows, or -1
  int32_t *ret_pos = nullptr;      // [R*k] row of a received pair in the return stream, or -1
  __nv_bfloat16 *ret_send = nullptr, *ret_recv = nullptr, *shared_y = nullptr;
  __half *rows = nullptr;          // expert-contiguous f16 rows of the resident experts
  int32_t *seg_count = nullptr;    // [n_local]
  int32_t *shared_cnt = nullptr;   // [1]
  SegScratch seg_shared;
  // direct transport: rows are stored straight into the peers' receive buffers over NVLink
  bool direct = false;
  uint8_t *slab = nullptr;         // table + recv_meta + recv_x + ret_recv of THIS rank; peers write into it
  uint8_t *peer_slab[EP_MAX_WORLD] = {};  // the same slab of every rank as mapped into this process (own entry = slab)
  bool peer_mapped[EP_MAX_WORLD] = {};    // opened with cudaIpcOpenMemHandle (to be closed)
  size_t table_off = 0, flag_off = 0, meta_off = 0, x_off = 0, ret_off = 0, slab_bytes = 0;
  bool flag_barrier = true;  // direct transport: barrier by flags in the peers' slabs (else a one-word NCCL all-gather)
  int32_t epoch = 0;         // barriers passed so far; every rank runs the same sequence
  int32_t *bar_status = nullptr;  // device word: set when a barrier wait gave up
  int tl_cap = 0;                  // rows per source segment of recv_x / recv_meta
  struct EpRecvInfo *info = nullptr;  // device: what this rank received, derived from the table
  int32_t *bar_src = nullptr, *bar_dst = nullptr;  // operands of the tiny collective used as a barrier
  int *overflow = nullptr;         // device word: a batch exceeded the row buffers
  bool timing = false;
  cudaEvent_t ev_t[EPS_N + 1] = {};
  float stage_ms[EPS_N] = {};
  int calls = 0;
};

// ---- kernels --------------------------------------------------------------------------------------------
namespace colib {

// Order in which rank r lays out the segments of its peers: its own first, then the others ascending.
__host__ __device__ inline int ep_rank_at(int pos, int r) { return pos == 0 ? r : (pos <= r ? pos - 1 : pos); }

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += u;
  }
  return v;
}

// The receive slab of every rank (own entry included), by value into the kernels that store to peers.
struct EpPeers {
  uint8_t *slab[EP_MAX_WORLD];
};

struct EpPlanParams {
  int T, k, E, world, rank;
  const int32_t *topk_idx;  // [T,k]
  const uint8_t *owner;     // [E]
  int32_t *cnt;             // [2*world] out
  int32_t *send_off;        // [world] out
  int32_t *send_pos;        // [T*world] out
  int32_t *home_slot;       // [T*k] out
  int publish;              // direct transport: store the counts into row `rank` of every rank's table
  EpPeers peers;
  size_t table_off;
};

// One CTA.  Warp w owns a contiguous range of 32-token chunks, so that positions ascend with the
// token; pass 1 counts per destination, a scan over the warps gives every warp its base, pass 2
// writes the positions.  A token's destination ranks are held 4 bits per kk (0xF = no valid expert).
__global__ void __launch_bounds__(1024) k_ep_plan(EpPlanParams p) {
  __shared__ int w_tok[32][EP_MAX_WORLD], w_pair[32][EP_MAX_WORLD];
  __shared__ int tot_tok[EP_MAX_WORLD], tot_pair[EP_MAX_WORLD], ret_off[EP_MAX_WORLD];
  __shared__ uint8_t own_sm[512];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) own_sm[e] = p.owner[e];
  __syncthreads();
  const int nchunk = (p.T + 31) / 32, cpw = (nchunk + 31) / 32;
  const int c0 = min(nchunk, warp * cpw), c1 = min(nchunk, c0 + cpw);
  auto dests_of = [&](int t) -> unsigned long long {
    unsigned long long dd = ~0ull;
    if (t < p.T)
      for (int kk = 0; kk < p.k; ++kk) {
        const int e = p.topk_idx[(size_t)t * p.k + kk];
        const unsigned long long d = (e >= 0 && e < p.E) ? (unsigned long long)own_sm[e] : 0xFull;
        dd = (dd & ~(0xFull << (4 * kk))) | (d << (4 * kk));
      }
    return dd;
  };
  auto count_of = [&](unsigned long long dd, int d) -> int {
    int n = 0;
    for (int kk = 0; kk < p.k; ++kk) n += (int)((dd >> (4 * kk)) & 0xFull) == d ? 1 : 0;
    return n;
  };
  int tok[EP_MAX_WORLD], pair[EP_MAX_WORLD];
#pragma unroll
  for (int d = 0; d < EP_MAX_WORLD; ++d) tok[d] = pair[d] = 0;
  for (int c = c0; c < c1; ++c) {
    const unsigned long long dd = dests_of(c * 32 + lane);
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d) {
      if (d < p.world) {  // uniform across the warp
        const int n = count_of(dd, d);
        tok[d] += __popc(__ballot_sync(0xffffffffu, n > 0));
        pair[d] += __reduce_add_sync(0xffffffffu, n);
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d) {
      w_tok[warp][d] = tok[d];
      w_pair[warp][d] = pair[d];
    }
  }
  __syncthreads();
  if (threadIdx.x < (unsigned)p.world) {
    const int d = threadIdx.x;
    int rt = 0, rp = 0;
    for (int w = 0; w < 32; ++w) {
      const int a = w_tok[w][d], b = w_pair[w][d];
      w_tok[w][d] = rt;
      w_pair[w][d] = rp;
      rt += a;
      rp += b;
    }
    tot_tok[d] = rt;
    tot_pair[d] = rp;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc_pair = 0, acc_tok = 0;
    for (int pos = 0; pos < p.world; ++pos) {
      const int d = ep_rank_at(pos, p.rank);
      ret_off[d] = acc_pair;
      acc_pair += tot_pair[d];
      p.send_off[d] = pos == 0 ? 0 : acc_tok;  // the own rows bypass the send buffer
      if (pos > 0) acc_tok += tot_tok[d];
      p.cnt[d] = tot_tok[d];
      p.cnt[p.world + d] = tot_pair[d];
    }
  }
  if (p.publish && threadIdx.x < (unsigned)p.world) {
    int32_t *row = reinterpret_cast<int32_t *>(p.peers.slab[threadIdx.x] + p.table_off) + (size_t)p.rank * 2 * p.world;
    for (int d = 0; d < p.world; ++d) {
      row[d] = tot_tok[d];
      row[p.world + d] = tot_pair[d];
    }
    __threadfence_system();
  }
  __syncthreads();
#pragma unroll
  for (int d = 0; d < EP_MAX_WORLD; ++d) {
    tok[d] = w_tok[warp][d];
    pair[d] = w_pair[warp][d];
  }
  const unsigned lt = (1u << lane) - 1u;
  for (int c = c0; c < c1; ++c) {
    const int t = c * 32 + lane;
    const unsigned long long dd = dests_of(t);
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d) {
      if (d >= p.world) continue;  // uniform across the warp
      const int n = count_of(dd, d);
      const unsigned bal = __ballot_sync(0xffffffffu, n > 0);
      const int incl = warp_incl_scan(n, lane);
      if (t < p.T) {
        p.send_pos[(size_t)t * p.world + d] = n > 0 ? tok[d] + __popc(bal & lt) : -1;
        if (n > 0) {
          int row = ret_off[d] + pair[d] + incl - n;
          for (int kk = 0; kk < p.k; ++kk)
            if ((int)((dd >> (4 * kk)) & 0xFull) == d) p.home_slot[(size_t)t * p.k + kk] = row++;
        }
      }
      tok[d] += __popc(bal);
      pair[d] += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (t < p.T)
      for (int kk = 0; kk < p.k; ++kk)
        if (((dd >> (4 * kk)) & 0xFull) == 0xFull) p.home_slot[(size_t)t * p.k + kk] = -1;  // no such expert: no row
  }
}

struct EpPackParams {
  int T, H, k, world, rank;
  const __nv_bfloat16 *x;
  const int32_t *topk_idx, *send_pos, *send_off;
  __nv_bfloat16 *send_x, *recv_x;
  int32_t *send_meta, *recv_meta;
};
// One warp per token: the row is read once and stored to the segment of every rank it visits.
__global__ void __launch_bounds__(256) k_ep_pack(EpPackParams p) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= p.T) return;
  uint4 *row[EP_MAX_WORLD];
  int32_t *meta[EP_MAX_WORLD];
#pragma unroll
  for (int d = 0; d < EP_MAX_WORLD; ++d) {
    row[d] = nullptr;
    meta[d] = nullptr;
    if (d < p.world) {
      const int pos = p.send_pos[(size_t)t * p.world + d];
      if (pos >= 0) {
        const size_t r = d == p.rank ? (size_t)pos : (size_t)p.send_off[d] + pos;
        row[d] = reinterpret_cast<uint4 *>((d == p.rank ? p.recv_x : p.send_x) + r * p.H);
        meta[d] = (d == p.rank ? p.recv_meta : p.send_meta) + r * p.k;
      }
    }
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)t * p.H);
  const int vec = p.H / 8;
  int c = lane;
  for (; c + 96 < vec; c += 128) {  // four loads in flight per lane before their stores
    const uint4 v0 = src[c], v1 = src[c + 32], v2 = src[c + 64], v3 = src[c + 96];
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d)
      if (row[d]) {
        row[d][c] = v0;
        row[d][c + 32] = v1;
        row[d][c + 64] = v2;
        row[d][c + 96] = v3;
      }
  }
  for (; c < vec; c += 32) {
    const uint4 v = src[c];
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d)
      if (row[d]) row[d][c] = v;
  }
  if (lane < p.k) {
    const int32_t e = p.topk_idx[(size_t)t * p.k + lane];
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d)
      if (meta[d]) meta[d][lane] = e;
  }
}

// Row of every received (token, kk) pair in the return stream: the running count of pairs that hit
// a resident expert (slot >= 0), in (source segment, token, kk) order.  One CTA, warps own
// contiguous ranges.
__global__ void __launch_bounds__(1024) k_ep_ret_plan(const int32_t *slot, int n, int32_t *ret_pos) {
  __shared__ int w_cnt[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nchunk = (n + 31) / 32, cpw = (nchunk + 31) / 32;
  const int c0 = min(nchunk, warp * cpw), c1 = min(nchunk, c0 + cpw);
  int cnt = 0;
  for (int c = c0; c < c1; ++c) {
    const int i = c * 32 + lane;
    cnt += __popc(__ballot_sync(0xffffffffu, i < n && slot[i] >= 0));
  }
  if (lane == 0) w_cnt[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int a = w_cnt[w];
      w_cnt[w] = run;
      run += a;
    }
  }
  __syncthreads();
  int base = w_cnt[warp];
  const unsigned lt = (1u << lane) - 1u;
  for (int c = c0; c < c1; ++c) {
    const int i = c * 32 + lane;
    const bool v = i < n && slot[i] >= 0;
    const unsigned bal = __ballot_sync(0xffffffffu, v);
    if (i < n) ret_pos[i] = v ? base + __popc(bal & lt) : -1;
    base += __popc(bal);
  }
}

// One warp per received pair: its result row goes to the return stream; the rows of this rank's
// own tokens (the first `self_pairs` of the stream) go straight into its own ret_recv.
__global__ void __launch_bounds__(256) k_ep_ret_pack(const __nv_bfloat16 *y, const int32_t *slot, const int32_t *ret_pos, int n, int H,
                                                     int self_pairs, __nv_bfloat16 *ret_send, __nv_bfloat16 *ret_recv) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (i >= n) return;
  const int pos = ret_pos[i];
  if (pos < 0) return;
  const uint4 *src = reinterpret_cast<const uint4 *>(y + (size_t)slot[i] * H);
  uint4 *dst = reinterpret_cast<uint4 *>(pos < self_pairs ? ret_recv + (size_t)pos * H : ret_send + (size_t)(pos - self_pairs) * H);
  const int vec = H / 8;
  for (int c = lane; c < vec; c += 32) dst[c] = src[c];
}

__global__ void k_set_i32(int32_t *p, int32_t v) { *p = v; }
__global__ void k_fill_i32(int32_t *p, int n, int32_t v) {
  if ((int)threadIdx.x < n) p[threadIdx.x] = v;
}

// Barrier of the direct transport.  Every thread that stored into a peer's slab has run
// __threadfence_system() behind its stores and its kernel has ended (stream order) before this one
// starts; thread d then publishes this rank's barrier count in peer d's flag row, and thread s waits
// until rank s's count in the own row has reached it.  Counts only grow, so a peer that is already
// one barrier ahead satisfies the wait as well.  The wait is bounded (about two seconds): a rank
// whose peer never arrives sets the status word and goes on, and the call is reported as failed.
// Ranks are separate processes on separate GPUs; one GPU never runs two ranks of this kernel (the
// single-GPU emulation orders the ranks' phases by the stream instead).
__global__ void k_ep_flag_barrier(EpPeers peers, size_t flag_off, int rank, int world, int32_t epoch, uint32_t max_polls, int32_t *status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  int32_t *dst = reinterpret_cast<int32_t *>(peers.slab[t] + flag_off) + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
  const int32_t *src = reinterpret_cast<const int32_t *>(peers.slab[rank] + flag_off) + t;
  bool ok = false;
  for (uint32_t i = 0; i < max_polls && !ok; ++i) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
    ok = v - epoch >= 0;
    if (!ok) __nanosleep(200);
  }
  if (!ok) atomicExch(status, 1);
  __threadfence_system();
}

// ---- direct transport -----------------------------------------------------------------------------------
// Receive buffers have one fixed segment of tl_cap rows per source rank, so a sender needs nobody
// else's counts to know where its rows go: token number `pos` of rank s's list for rank d is row
// s * tl_cap + pos of d's recv_x.
struct EpPackDirectParams {
  int T, H, k, world, rank, tl_cap;
  const __nv_bfloat16 *x;
  const int32_t *topk_idx, *send_pos;
  EpPeers peers;
  size_t x_off, meta_off;
};
__global__ void __launch_bounds__(256) k_ep_pack_direct(EpPackDirectParams p) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= p.T) return;
  uint4 *row[EP_MAX_WORLD];
  int32_t *meta[EP_MAX_WORLD];
#pragma unroll
  for (int d = 0; d < EP_MAX_WORLD; ++d) {
    row[d] = nullptr;
    meta[d] = nullptr;
    if (d < p.world) {
      const int pos = p.send_pos[(size_t)t * p.world + d];
      if (pos >= 0 && pos < p.tl_cap) {
        const size_t r = (size_t)p.rank * p.tl_cap + pos;
        row[d] = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.peers.slab[d] + p.x_off) + r * p.H);
        meta[d] = reinterpret_cast<int32_t *>(p.peers.slab[d] + p.meta_off) + r * p.k;
      }
    }
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(p.x + (size_t)t * p.H);
  const int vec = p.H / 8;
  for (int c = lane; c < vec; c += 32) {
    const uint4 v = src[c];
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d)
      if (row[d]) row[d][c] = v;
  }
  if (lane < p.k) {
    const int32_t e = p.topk_idx[(size_t)t * p.k + lane];
#pragma unroll
    for (int d = 0; d < EP_MAX_WORLD; ++d)
      if (meta[d]) meta[d][lane] = e;
  }
  __threadfence_system();
}

}  // namespace colib
// What a rank received, derived on the device from its (complete) copy of the count table.
struct EpRecvInfo {
  colib::VirtualBatch vb;   // the received tokens: segments in this rank's order (own first), slot = source rank
  int32_t pair_base[9];     // pairs that hit this rank's experts in the segments before each one
  int32_t ret_dst_off[8];   // per segment: first row of this rank's results in the source's ret_recv
  int32_t src_rank[8];
};
namespace colib {
__global__ void k_ep_recv_layout(const int32_t *table, int world, int rank, int tl_cap, EpRecvInfo *info) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int w2 = 2 * world;
  int tok = 0, pair = 0;
  info->vb.nseg = world;
  info->vb.stride = tl_cap;
  for (int pos = 0; pos < world; ++pos) {
    const int s = ep_rank_at(pos, rank);
    int n = table[s * w2 + rank];
    n = n < 0 ? 0 : (n > tl_cap ? tl_cap : n);
    info->vb.off[pos] = tok;
    info->vb.phys[pos] = s;
    info->src_rank[pos] = s;
    info->pair_base[pos] = pair;
    tok += n;
    pair += table[s * w2 + world + rank];
    // where rank s expects the results of this rank: its own first, then the others ascending
    int off = 0;
    if (rank != s) {
      off = table[s * w2 + world + s];
      for (int d = 0; d < rank; ++d)
        if (d != s) off += table[s * w2 + world + d];
    }
    info->ret_dst_off[pos] = off;
  }
  info->vb.off[world] = tok;
  info->vb.total = tok;
  info->pair_base[world] = pair;
}

// k_ep_ret_plan over a batch whose size is known on the device only
__global__ void __launch_bounds__(1024) k_ep_ret_plan_virt(const int32_t *slot, const EpRecvInfo *info, int k, int32_t *ret_pos) {
  __shared__ int w_cnt[32];
  const int n = info->vb.total * k;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nchunk = (n + 31) / 32, cpw = (nchunk + 31) / 32;
  const int c0 = min(nchunk, warp * cpw), c1 = min(nchunk, c0 + cpw);
  int cnt = 0;
  for (int c = c0; c < c1; ++c) {
    const int i = c * 32 + lane;
    cnt += __popc(__ballot_sync(0xffffffffu, i < n && slot[i] >= 0));
  }
  if (lane == 0) w_cnt[warp] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int a = w_cnt[w];
      w_cnt[w] = run;
      run += a;
    }
  }
  __syncthreads();
  int base = w_cnt[warp];
  const unsigned lt = (1u << lane) - 1u;
  for (int c = c0; c < c1; ++c) {
    const int i = c * 32 + lane;
    const bool v = i < n && slot[i] >= 0;
    const unsigned bal = __ballot_sync(0xffffffffu, v);
    if (i < n) ret_pos[i] = v ? base + __popc(bal & lt) : -1;
    base += __popc(bal);
  }
}

// One warp per received pair: its result row is stored into the ret_recv of the token's home rank.
__global__ void __launch_bounds__(256) k_ep_ret_pack_direct(const __nv_bfloat16 *y, const int32_t *slot, const int32_t *ret_pos,
                                                            const EpRecvInfo *info, int k, int H, int ret_rows_cap, EpPeers peers,
                                                            size_t ret_off, int *overflow) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (i >= info->vb.total * k) return;
  const int pos = ret_pos[i];
  if (pos < 0) return;
  const int j = i / k;
  int s = 0;
  while (s + 1 < info->vb.nseg && j >= info->vb.off[s + 1]) ++s;
  const int row = info->ret_dst_off[s] + (pos - info->pair_base[s]);
  if (row < 0 || row >= ret_rows_cap) {
    if (lane == 0 && overflow) atomicExch(overflow, 1);
    return;
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(y + (size_t)slot[i] * H);
  uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(peers.slab[info->src_rank[s]] + ret_off) + (size_t)row * H);
  const int vec = H / 8;
  // four loads in flight per lane before their stores: a row is one warp's serial copy otherwise
  int c = lane;
  for (; c + 96 < vec; c += 128) {
    const uint4 v0 = src[c], v1 = src[c + 32], v2 = src[c + 64], v3 = src[c + 96];
    dst[c] = v0;
    dst[c + 32] = v1;
    dst[c + 64] = v2;
    dst[c + 96] = v3;
  }
  for (; c < vec; c += 32) dst[c] = src[c];
  __threadfence_system();
}

}  // namespace colib

// ---- host side ------------------------------------------------------------------------------------------
namespace {

// What one rank learns from the all-gathered count table [world][2*world] (row s = rank s's counts:
// tokens sent to each rank, then pairs owned by each rank).  Segments are laid out own first, then the
// peers ascending (ep_rank_at), on both sides of both exchanges.
struct EpCounts {
  int send_tok[EP_MAX_WORLD], send_pair[EP_MAX_WORLD];  // this rank -> d
  int recv_tok[EP_MAX_WORLD], recv_pair[EP_MAX_WORLD];  // s -> this rank
  int send_off[EP_MAX_WORLD];      // first row of d's segment in send_x (peers only)
  int recv_off[EP_MAX_WORLD];      // first row of s's segment in recv_x (own segment at 0)
  int ret_send_off[EP_MAX_WORLD];  // first row of s's segment in ret_send (peers only)
  int ret_recv_off[EP_MAX_WORLD];  // first row of d's segment in ret_recv (own segment at 0)
  int R;                           // tokens received, own included
  int pairs_here;                  // pairs that hit this rank's experts
  long total_pairs;                // over all ranks
};
void ep_counts(const int32_t *tab, int world, int rank, EpCounts &c) {
  const int w2 = 2 * world;
  c.R = 0;
  c.pairs_here = 0;
  c.total_pairs = 0;
  for (int s = 0; s < world; ++s) {
    c.send_tok[s] = tab[rank * w2 + s];
    c.send_pair[s] = tab[rank * w2 + world + s];
    c.recv_tok[s] = tab[s * w2 + rank];
    c.recv_pair[s] = tab[s * w2 + world + rank];
    c.R += c.recv_tok[s];
    c.pairs_here += c.recv_pair[s];
    for (int d = 0; d < world; ++d) c.total_pairs += tab[s * w2 + world + d];
  }
  int so = 0, ro = 0, rso = 0, rro = 0;
  for (int pos = 0; pos < world; ++pos) {
    const int p = colib::ep_rank_at(pos, rank);
    c.send_off[p] = pos == 0 ? 0 : so;
    if (pos > 0) so += c.send_tok[p];
    c.recv_off[p] = ro;
    ro += c.recv_tok[p];
    c.ret_send_off[p] = pos == 0 ? 0 : rso;
    if (pos > 0) rso += c.recv_pair[p];
    c.ret_recv_off[p] = rro;
    rro += c.send_pair[p];
  }
}

#define EP_MARK(i)                                                                  \
  do {                                                                              \
    if (ep->timing) CK(cudaEventRecord(ep->ev_t[i], st), "stage event");            \
  } while (0)

// Phase A: route the own tokens, plan and pack the dispatch, start the shared expert on the auxiliary stream.
int ep_phase_a(ColiMoe *m, const void *x_dev, int T, cudaStream_t st) {
  ColiEp *ep = m->ep;
  EP_MARK(0);
  CK(cudaEventRecord(ep->ev_x, st), "event record");
  if (T > 0) {
    if (!colib::launch_router(coli_route_params(m, x_dev, T), st)) return 0;
  }
  EP_MARK(1);
  colib::EpPlanParams pl;
  pl.T = T;
  pl.k = m->L.k;
  pl.E = m->L.E;
  pl.world = ep->world;
  pl.rank = ep->rank;
  pl.topk_idx = m->topk_idx;
  pl.owner = ep->owner;
  pl.cnt = ep->cnt;
  pl.send_off = ep->send_off;
  pl.send_pos = ep->send_pos;
  pl.home_slot = ep->home_slot;
  pl.publish = ep->direct ? 1 : 0;
  for (int d = 0; d < EP_MAX_WORLD; ++d) pl.peers.slab[d] = ep->peer_slab[d];
  pl.table_off = ep->table_off;
  colib::k_ep_plan<<<1, 1024, 0, st>>>(pl);
  coli_count_launch(1);
  if (T > 0 && ep->direct) {
    colib::EpPackDirectParams pk;
    pk.T = T;
    pk.H = m->L.H;
    pk.k = m->L.k;
    pk.world = ep->world;
    pk.rank = ep->rank;
    pk.tl_cap = ep->tl_cap;
    pk.x = (const __nv_bfloat16 *)x_dev;
    pk.topk_idx = m->topk_idx;
    pk.send_pos = ep->send_pos;
    pk.peers = pl.peers;
    pk.x_off = ep->x_off;
    pk.meta_off = ep->meta_off;
    colib::k_ep_pack_direct<<<(T + 7) / 8, 256, 0, st>>>(pk);
    coli_count_launch(1);
  } else if (T > 0) {
    colib::EpPackParams pk;
    pk.T = T;
    pk.H = m->L.H;
    pk.k = m->L.k;
    pk.world = ep->world;
    pk.rank = ep->rank;
    pk.x = (const __nv_bfloat16 *)x_dev;
    pk.topk_idx = m->topk_idx;
    pk.send_pos = ep->send_pos;
    pk.send_off = ep->send_off;
    pk.send_x = ep->send_x;
    pk.recv_x = ep->recv_x;
    pk.send_meta = ep->send_meta;
    pk.recv_meta = ep->recv_meta;
    colib::k_ep_pack<<<(T + 7) / 8, 256, 0, st>>>(pk);
    coli_count_launch(1);
  }
  CK(cudaGetLastError(), "dispatch plan launch");
  EP_MARK(2);
  if (m->has_shared && T > 0) {  // independent of the exchange: runs beside it
    cudaStream_t ax = ep->aux;
    CK(cudaStreamWaitEvent(ax, ep->ev_x, 0), "stream wait");
    colib::k_set_i32<<<1, 1, 0, ax>>>(ep->shared_cnt, T);
    coli_count_launch(1);
    if (!colib::launch_bf16_to_f16((const __nv_bfloat16 *)x_dev, m->x16, (size_t)T * m->L.H, ax)) return 0;
    if (!coli_run_segments(m, ep->seg_shared, m->gate + m->L.E, m->up + m->L.E, m->down + m->L.E, nullptr, m->x16, ep->shared_cnt, 1,
                           T, T, ep->shared_y, ax))
      return 0;
    CK(cudaEventRecord(ep->ev_shared, ax), "event record");
  }
  return 1;
}

// Phase B (after the dispatch): rows of the received pairs that hit resident experts, the grouped
// FFN over them, and the result rows packed in return order.
int ep_phase_b(ColiMoe *m, const EpCounts &c, cudaStream_t st) {
  ColiEp *ep = m->ep;
  const int k = m->L.k, H = m->L.H;
  EP_MARK(4);
  if (c.R > 0) {
    colib::PermuteParams pp = coli_permute_params(m, ep->recv_x, c.R, false, colib::TC_MAX_TOKENS, ep->rows, ep->seg_count, ep->recv_slot);
    pp.topk_idx = ep->recv_meta;
    pp.expert_slot = m->local_slot;
    pp.nseg_routed = m->n_local_seg;
    if (!colib::launch_permute(pp, st)) return 0;
  }
  EP_MARK(5);
  if (c.pairs_here > 0) {
    const long expect = c.total_pairs / ep->world;
    if (!coli_run_segments(m, m->seg_main, m->gate, m->up, m->down, m->seg_expert + m->first_local_seg, ep->rows, ep->seg_count,
                           m->n_local_seg, c.pairs_here, (int)(expect > 0 ? expect : 1), m->y, st))
      return 0;
  }
  EP_MARK(6);
  if (c.R > 0) {
    const int n = c.R * k;
    colib::k_ep_ret_plan<<<1, 1024, 0, st>>>(ep->recv_slot, n, ep->ret_pos);
    coli_count_launch(1);
    if (c.pairs_here > 0) {
      colib::k_ep_ret_pack<<<(n + 7) / 8, 256, 0, st>>>(m->y, ep->recv_slot, ep->ret_pos, n, H, c.recv_pair[ep->rank], ep->ret_send, ep->ret_recv);
      coli_count_launch(1);
    }
    CK(cudaGetLastError(), "return pack launch");
  }
  EP_MARK(7);
  return 1;
}

// Phase C (after the return exchange): weighted combine of the own tokens + shared expert.
int ep_phase_c(ColiMoe *m, void *out_dev, int T, cudaStream_t st) {
  ColiEp *ep = m->ep;
  EP_MARK(8);
  if (T > 0) {
    if (m->has_shared) CK(cudaStreamWaitEvent(st, ep->ev_shared, 0), "stream wait");
    colib::CombineParams cp;
    cp.T = T;
    cp.H = m->L.H;
    cp.k = m->L.k;
    cp.has_shared = m->has_shared ? 1 : 0;
    cp.y = ep->direct ? reinterpret_cast<const __nv_bfloat16 *>(ep->slab + ep->ret_off) : ep->ret_recv;
    cp.shared_y = ep->shared_y;
    cp.slot = ep->home_slot;
    cp.topk_w = m->topk_w;
    cp.out = (__nv_bfloat16 *)out_dev;
    cp.out32 = nullptr;
    cp.resid = nullptr;
    if (!colib::launch_combine(cp, st)) return 0;
  }
  EP_MARK(9);
  return 1;
}

// Direct transport, after the barrier that follows the dispatch stores: every peer's rows and counts
// are in this rank's slab.  Nothing here needs the host to know a count: grids are sized from the
// handle's capacity and the kernels read the actual sizes from the device.
int ep_direct_phase_b(ColiMoe *m, cudaStream_t st) {
  ColiEp *ep = m->ep;
  const int k = m->L.k, H = m->L.H, cap_tok = m->max_tokens;
  const long rows_cap = (long)cap_tok * k;
  colib::k_ep_recv_layout<<<1, 32, 0, st>>>(reinterpret_cast<const int32_t *>(ep->slab + ep->table_off), ep->world, ep->rank, ep->tl_cap, ep->info);
  coli_count_launch(1);
  EP_MARK(4);
  colib::PermuteParams pp = coli_permute_params(m, ep->slab + ep->x_off, cap_tok, false, colib::TC_MAX_TOKENS, ep->rows, ep->seg_count, ep->recv_slot);
  pp.topk_idx = reinterpret_cast<const int32_t *>(ep->slab + ep->meta_off);
  pp.expert_slot = m->local_slot;
  pp.nseg_routed = m->n_local_seg;
  pp.virt = &ep->info->vb;
  pp.rows_cap = (int)rows_cap;
  pp.overflow = ep->overflow;
  if (!colib::launch_permute(pp, st)) return 0;
  EP_MARK(5);
  if (m->n_local_seg > 0) {
    const long expect = rows_cap / ep->world;
    if (!coli_run_segments(m, m->seg_main, m->gate, m->up, m->down, m->seg_expert + m->first_local_seg, ep->rows, ep->seg_count,
                           m->n_local_seg, (int)rows_cap, (int)(expect > 0 ? expect : 1), m->y, st))
      return 0;
  }
  EP_MARK(6);
  colib::k_ep_ret_plan_virt<<<1, 1024, 0, st>>>(ep->recv_slot, ep->info, k, ep->ret_pos);
  coli_count_launch(1);
  colib::EpPeers peers;
  for (int d = 0; d < EP_MAX_WORLD; ++d) peers.slab[d] = ep->peer_slab[d];
  colib::k_ep_ret_pack_direct<<<(unsigned)((rows_cap + 7) / 8), 256, 0, st>>>(m->y, ep->recv_slot, ep->ret_pos, ep->info, k, H,
                                                                             ep->tl_cap * k, peers, ep->ret_off, ep->overflow);
  coli_count_launch(1);
  CK(cudaGetLastError(), "return store launch");
  EP_MARK(7);
  return 1;
}

bool ep_check_capacity(ColiMoe *m, const int32_t *tab) {
  const int world = m->ep->world;
  for (int r = 0; r < world; ++r) {  // every rank checks every rank, so that all of them decide alike
    EpCounts c;
    ep_counts(tab, world, r, c);
    if (c.R > m->max_tokens || c.pairs_here > (long)m->max_tokens * m->L.k) {
      coli_set_error("moe_block_ep: rank %d would receive %d tokens / %d pairs, more than a handle of max_tokens=%d holds", r, c.R,
                     c.pairs_here, m->max_tokens);
      return false;
    }
  }
  return true;
}

int ep_finish_timing(ColiMoe *m) {
  ColiEp *ep = m->ep;
  if (!ep->timing) return 1;
  CK(cudaEventSynchronize(ep->ev_t[EPS_N]), "stage event sync");
  for (int i = 0; i < EPS_N; ++i) {
    float ms = 0.0f;
    CK(cudaEventElapsedTime(&ms, ep->ev_t[i], ep->ev_t[i + 1]), "stage event read");
    ep->stage_ms[i] += ms;
  }
  ep->calls++;
  return 1;
}

}  // namespace

// Direct transport: every rank publishes the IPC handle of its receive slab (all-gathered with the
// communicator) and maps the slabs of the others.
static bool ep_connect_direct(ColiMoe *m) {
  ColiEp *ep = m->ep;
  NcclApi *api = nccl_api();
  if (!api) return false;
  const int world = ep->world, rank = ep->rank;
  cudaIpcMemHandle_t mine;
  if (!coli_cuda_check(cudaIpcGetMemHandle(&mine, ep->slab), "cudaIpcGetMemHandle")) return false;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  uint8_t *dbuf = nullptr;
  std::vector<cudaIpcMemHandle_t> all(world);
  cudaStream_t st = m->ctx->stream;
  bool ok = coli_cuda_check(cudaMalloc((void **)&dbuf, (size_t)64 * world), "handle buffer") &&
            coli_cuda_check(cudaMemcpyAsync(dbuf + (size_t)64 * rank, &mine, 64, cudaMemcpyHostToDevice, st), "handle upload") &&
            nccl_ok(api, api->AllGather(dbuf + (size_t)64 * rank, dbuf, 64, COLI_NCCL_INT8, ep->comm, st), "handle all-gather") &&
            coli_cuda_check(cudaMemcpyAsync(all.data(), dbuf, (size_t)64 * world, cudaMemcpyDeviceToHost, st), "handle download") &&
            coli_cuda_check(cudaStreamSynchronize(st), "handle exchange");
  for (int p = 0; ok && p < world; ++p) {
    if (p == rank) continue;
    void *ptr = nullptr;
    ok = coli_cuda_check(cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    if (ok) {
      ep->peer_slab[p] = (uint8_t *)ptr;
      ep->peer_mapped[p] = true;
    }
  }
  if (dbuf) cudaFree(dbuf);
  return ok;
}

int coli_ep_ensure(ColiMoe *m, void *comm) {
  if (!m) return 0;
  if (m->ep) {
    if (comm && !m->ep->comm) {
      m->ep->comm = (ncclComm_t)comm;
      if (m->ep->direct && !ep_connect_direct(m)) return 0;
    }
    return 1;
  }
  const int world = m->L.ep_world, rank = m->L.ep_rank, k = m->L.k, H = m->L.H, E = m->L.E;
  if (world < 2 || world > EP_MAX_WORLD || rank < 0 || rank >= world) {
    coli_set_error("expert parallelism: ep_world=%d / ep_rank=%d outside 2..%d ranks", world, rank, EP_MAX_WORLD);
    return 0;
  }
  if (k > EP_MAX_K || E > 512) {
    coli_set_error("expert parallelism: k=%d (max %d) or E=%d (max 512) not supported", k, EP_MAX_K, E);
    return 0;
  }
  if (!coli_select_ctx(m->ctx)) return 0;
  ColiEp *ep = new ColiEp();
  m->ep = ep;
  ep->rank = rank;
  ep->world = world;
  ep->comm = (ncclComm_t)comm;
  const size_t T = (size_t)m->max_tokens;
  const size_t send_rows = T * (size_t)(k < world - 1 ? k : world - 1);
  std::vector<uint8_t> own(E);
  for (int e = 0; e < E; ++e) own[e] = (uint8_t)m->h_owner[e];
  bool ok = coli_cuda_check(cudaStreamCreateWithFlags(&ep->aux, cudaStreamNonBlocking), "stream creation") &&
            coli_cuda_check(cudaEventCreateWithFlags(&ep->ev_x, cudaEventDisableTiming), "event creation") &&
            coli_cuda_check(cudaEventCreateWithFlags(&ep->ev_shared, cudaEventDisableTiming), "event creation") &&
            coli_cuda_check(cudaEventCreateWithFlags(&ep->ev_counts, cudaEventDisableTiming), "event creation") &&
            coli_cuda_check(cudaMallocHost((void **)&ep->h_all_cnt, sizeof(int32_t) * 2 * world * world), "pinned allocation");
  ok = ok && ws_alloc(m, &ep->owner, (size_t)E) && ws_alloc(m, &ep->cnt, 2 * (size_t)world) && ws_alloc(m, &ep->send_off, (size_t)world) &&
       ws_alloc(m, &ep->send_pos, T * world) && ws_alloc(m, &ep->home_slot, T * k) && ws_alloc(m, &ep->recv_slot, T * k) &&
       ws_alloc(m, &ep->ret_pos, T * k) && ws_alloc(m, &ep->seg_count, (size_t)(m->n_local_seg > 0 ? m->n_local_seg : 1)) &&
       ws_alloc(m, &ep->shared_cnt, 1) && ws_alloc(m, &ep->overflow, 1) &&
       coli_cuda_check(cudaMemset(ep->overflow, 0, sizeof(int)), "flag clear");
  // Transport.  "direct" (default): every rank's receive buffers sit in one slab that the peers map
  // (cudaIpc) and store into over NVLink; "nccl" (COLI_EP_TRANSPORT=nccl, or when the slab cannot be
  // shared): rows are packed into send buffers and exchanged with ncclSend / ncclRecv.
  const char *tr = getenv("COLI_EP_TRANSPORT");
  ep->direct = !(tr && strcmp(tr, "nccl") == 0);
  if (ok && ep->direct) {
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    ep->tl_cap = m->max_tokens;
    ep->table_off = 0;
    ep->flag_off = up(sizeof(int32_t) * 2 * world * world);
    ep->meta_off = ep->flag_off + 256;  // one row of barrier counts, [world] int32
    ep->x_off = ep->meta_off + up(sizeof(int32_t) * (size_t)world * ep->tl_cap * k);
    ep->ret_off = ep->x_off + up(sizeof(__nv_bfloat16) * (size_t)world * ep->tl_cap * H);
    ep->slab_bytes = ep->ret_off + up(sizeof(__nv_bfloat16) * (size_t)ep->tl_cap * k * H);
    ok = coli_cuda_check(cudaMalloc((void **)&ep->slab, ep->slab_bytes), "receive slab allocation");
    if (ok) {
      m->allocs.push_back(ep->slab);
      m->ws_bytes += ep->slab_bytes;
      ep->peer_slab[rank] = ep->slab;
      ok = coli_cuda_check(cudaMemset(ep->slab, 0, ep->meta_off), "table clear") && ws_alloc(m, &ep->info, 1) &&
           ws_alloc(m, &ep->bar_src, 1) && ws_alloc(m, &ep->bar_dst, (size_t)world) && ws_alloc(m, &ep->bar_status, 1) &&
           coli_cuda_check(cudaMemset(ep->bar_status, 0, sizeof(int32_t)), "flag clear");
      const char *bk = getenv("COLI_EP_BARRIER");
      ep->flag_barrier = !(bk && strcmp(bk, "nccl") == 0);
    }
    if (ok && comm && !ep_connect_direct(m)) ok = false;
  } else if (ok) {
    ok = ws_alloc(m, &ep->all_cnt, 2 * (size_t)world * world) && ws_alloc(m, &ep->send_x, send_rows * H) &&
         ws_alloc(m, &ep->send_meta, send_rows * k) && ws_alloc(m, &ep->recv_x, T * H) && ws_alloc(m, &ep->recv_meta, T * k) &&
         ws_alloc(m, &ep->ret_send, T * k * H) && ws_alloc(m, &ep->ret_recv, T * k * H);
  }
  if (ok) {
    if (m->xg) {
      ep->rows = m->xg;  // the block's own gathered-row buffer: (T*k + T) rows
    } else {
      ok = ws_alloc(m, &ep->rows, T * k * H);
    }
  }
  if (ok && m->has_shared) {
    const int items = (int)(T / 8 + 2);
    ok = ws_alloc(m, &ep->shared_y, T * H) && ws_alloc(m, &ep->seg_shared.h, T * m->L.I) && ws_alloc(m, &ep->seg_shared.item_seg, (size_t)items) &&
         ws_alloc(m, &ep->seg_shared.item_row0, (size_t)items) && ws_alloc(m, &ep->seg_shared.item_nrows, (size_t)items) &&
         ws_alloc(m, &ep->seg_shared.n_items, 1) && ws_alloc(m, &ep->seg_shared.seg_off, 3);
    ep->seg_shared.h_rows = T;
    ep->seg_shared.item_cap = items;
    ep->seg_shared.seg_cap = 1;
  }
  ok = ok && coli_cuda_check(cudaMemcpy(ep->owner, own.data(), (size_t)E, cudaMemcpyHostToDevice), "owner table upload");
  if (!ok) {
    coli_ep_destroy(m);
    return 0;
  }
  return 1;
}

void coli_ep_destroy(ColiMoe *m) {
  if (!m || !m->ep) return;
  ColiEp *ep = m->ep;
  if (ep->aux) cudaStreamDestroy(ep->aux);
  for (cudaEvent_t e : {ep->ev_x, ep->ev_shared, ep->ev_counts})
    if (e) cudaEventDestroy(e);
  for (int i = 0; i <= EPS_N; ++i)
    if (ep->ev_t[i]) cudaEventDestroy(ep->ev_t[i]);
  if (ep->h_all_cnt) cudaFreeHost(ep->h_all_cnt);
  for (int p = 0; p < EP_MAX_WORLD; ++p)
    if (ep->peer_mapped[p] && ep->peer_slab[p]) cudaIpcCloseMemHandle(ep->peer_slab[p]);
  delete ep;  // device buffers are in the handle's allocation list; the communicator belongs to the caller
  m->ep = nullptr;
}

// 1 if no expert-parallel call of this handle ran out of row capacity since the last check.
int coli_ep_check(ColiMoe *m) {
  if (!m || !m->ep || !m->ep->overflow) return 1;
  int v = 0;
  CK(cudaMemcpy(&v, m->ep->overflow, sizeof(int), cudaMemcpyDeviceToHost), "flag read");
  if (v != 0) {
    cudaMemset(m->ep->overflow, 0, sizeof(int));
    coli_set_error("an expert-parallel call brought more tokens than the handle's max_tokens=%d holds; its results are invalid", m->max_tokens);
    return 0;
  }
  if (m->ep->bar_status) {
    CK(cudaMemcpy(&v, m->ep->bar_status, sizeof(int), cudaMemcpyDeviceToHost), "flag read");
    if (v != 0) {
      cudaMemset(m->ep->bar_status, 0, sizeof(int));
      coli_set_error("an expert-parallel call gave up waiting for a peer rank at a barrier; its results are invalid");
      return 0;
    }
  }
  return 1;
}

// ---- communicator helpers: for callers that have no ncclComm_t of their own -------------------------------
extern "C" int coli_b200_nccl_unique_id(void *id128) {
  NcclApi *api = nccl_api();
  if (!api || !id128) return 0;
  ncclUniqueId id;
  if (!nccl_ok(api, api->GetUniqueId(&id), "ncclGetUniqueId")) return 0;
  memcpy(id128, &id, sizeof(id));
  return 1;
}
extern "C" int coli_b200_nccl_comm_create(void **comm, const void *id128, int rank, int world, int device) {
  NcclApi *api = nccl_api();
  if (!api || !comm || !id128 || world < 1 || rank < 0 || rank >= world) {
    if (api) coli_set_error("nccl_comm_create: bad argument");
    return 0;
  }
  if (!coli_select_ctx(coli_find_ctx(device))) return 0;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclComm_t c = nullptr;
  if (!nccl_ok(api, api->CommInitRank(&c, world, id, rank), "ncclCommInitRank")) return 0;
  *comm = (void *)c;
  return 1;
}
extern "C" void coli_b200_nccl_comm_destroy(void *comm) {
  NcclApi *api = nccl_api();
  if (api && comm) api->CommDestroy((ncclComm_t)comm);
}

extern "C" int coli_b200_ep_profile(ColiMoe *m, int enable) {
  if (!m || !coli_ep_ensure(m, nullptr) || !coli_select_ctx(m->ctx)) return 0;
  ColiEp *ep = m->ep;
  if (enable) {
    for (int i = 0; i <= EPS_N; ++i)
      if (!ep->ev_t[i]) CK(cudaEventCreate(&ep->ev_t[i]), "event creation");
    for (int i = 0; i < EPS_N; ++i) ep->stage_ms[i] = 0.0f;
    ep->calls = 0;
  }
  ep->timing = enable != 0;
  return 1;
}
extern "C" int coli_b200_ep_stage_ms(ColiMoe *m, float *ms, int *calls) {
  if (!m || !m->ep || !ms) return 0;
  for (int i = 0; i < EPS_N; ++i) ms[i] = m->ep->stage_ms[i];
  if (calls) *calls = m->ep->calls;
  return 1;
}
extern "C" int coli_b200_ep_last_counts(ColiMoe *m, int32_t *table) {
  if (!m || !m->ep || !table || !coli_select_ctx(m->ctx)) return 0;
  const size_t bytes = sizeof(int32_t) * 2 * m->ep->world * m->ep->world;
  if (m->ep->direct) {  // the table lives in the slab; nothing on the host has seen it yet
    CK(cudaDeviceSynchronize(), "count read sync");
    CK(cudaMemcpy(table, m->ep->slab + m->ep->table_off, bytes, cudaMemcpyDeviceToHost), "count read");
    return 1;
  }
  memcpy(table, m->ep->h_all_cnt, bytes);
  return 1;
}

// Host-only: the segment layout one rank derives from the count table (what the call itself uses).
extern "C" int coli_b200_ep_layout(const int32_t *table, int world, int rank, int32_t *out) {
  if (!table || !out || world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world) {
    coli_set_error("ep_layout: bad argument");
    return 0;
  }
  EpCounts c;
  ep_counts(table, world, rank, c);
  const int *rows[8] = {c.send_tok, c.send_pair, c.recv_tok, c.recv_pair, c.send_off, c.recv_off, c.ret_send_off, c.ret_recv_off};
  for (int i = 0; i < 8; ++i)
    for (int d = 0; d < world; ++d) out[i * world + d] = rows[i][d];
  return 1;
}

// ---- the call ---------------------------------------------------------------------------------------------
extern "C" int coli_b200_moe_block_ep_dev(ColiMoe *m, const void *x_dev, void *out_dev, int T_local, void *stream) {
  if (!coli_check_T(m, T_local, "moe_block_ep_dev")) return 0;
  if ((T_local > 0 && (!x_dev || !out_dev))) {
    coli_set_error("moe_block_ep_dev: null pointer");
    return 0;
  }
  if (!m->ep || !m->ep->comm) {
    coli_set_error("moe_block_ep_dev: the handle was created without a communicator (ColiMoeLayer.nccl_comm, ep_world > 1)");
    return 0;
  }
  NcclApi *api = nccl_api();
  if (!api) return 0;
  ColiEp *ep = m->ep;
  cudaStream_t st = (cudaStream_t)stream;
  const int world = ep->world, rank = ep->rank, H = m->L.H, k = m->L.k;
  if (!ep_phase_a(m, x_dev, T_local, st)) return 0;
  if (ep->direct) {
    // the rows and counts were stored straight into the peers' slabs; a tiny collective after the stores
    // is the barrier that tells every rank that all of its senders are done (and nothing needs the host)
    auto barrier = [&](const char *what) -> bool {
      if (!ep->flag_barrier) return nccl_ok(api, api->AllGather(ep->bar_src, ep->bar_dst, 1, COLI_NCCL_INT32, ep->comm, st), what);
      colib::EpPeers peers;
      for (int d = 0; d < EP_MAX_WORLD; ++d) peers.slab[d] = d < world ? ep->peer_slab[d] : nullptr;
      ++ep->epoch;
      colib::k_ep_flag_barrier<<<1, 32, 0, st>>>(peers, ep->flag_off, rank, world, ep->epoch, EP_BARRIER_POLLS, ep->bar_status);
      coli_count_launch(1);
      return coli_cuda_check(cudaGetLastError(), what);
    };
    if (!barrier("dispatch barrier")) return 0;
    EP_MARK(3);
    if (!ep_direct_phase_b(m, st)) return 0;
    if (!barrier("return barrier")) return 0;
    if (!ep_phase_c(m, out_dev, T_local, st)) return 0;
    return ep_finish_timing(m);
  }
  // counts: every rank's 2 x world figures to every rank, then to the host
  if (!nccl_ok(api, api->AllGather(ep->cnt, ep->all_cnt, (size_t)2 * world, COLI_NCCL_INT32, ep->comm, st), "count all-gather")) return 0;
  CK(cudaMemcpyAsync(ep->h_all_cnt, ep->all_cnt, sizeof(int32_t) * 2 * world * world, cudaMemcpyDeviceToHost, st), "count download");
  CK(cudaEventRecord(ep->ev_counts, st), "event record");
  CK(cudaEventSynchronize(ep->ev_counts), "count wait");
  EP_MARK(3);
  if (!ep_check_capacity(m, ep->h_all_cnt)) return 0;
  EpCounts c;
  ep_counts(ep->h_all_cnt, world, rank, c);
  // dispatch: token rows and their expert ids
  bool ok = nccl_ok(api, api->GroupStart(), "ncclGroupStart");
  for (int pos = 1; ok && pos < world; ++pos) {
    const int p = colib::ep_rank_at(pos, rank);
    if (c.send_tok[p] > 0)
      ok = nccl_ok(api, api->Send(ep->send_x + (size_t)c.send_off[p] * H, (size_t)c.send_tok[p] * H, COLI_NCCL_BF16, p, ep->comm, st), "dispatch send") &&
           nccl_ok(api, api->Send(ep->send_meta + (size_t)c.send_off[p] * k, (size_t)c.send_tok[p] * k, COLI_NCCL_INT32, p, ep->comm, st), "dispatch send");
    if (ok && c.recv_tok[p] > 0)
      ok = nccl_ok(api, api->Recv(ep->recv_x + (size_t)c.recv_off[p] * H, (size_t)c.recv_tok[p] * H, COLI_NCCL_BF16, p, ep->comm, st), "dispatch recv") &&
           nccl_ok(api, api->Recv(ep->recv_meta + (size_t)c.recv_off[p] * k, (size_t)c.recv_tok[p] * k, COLI_NCCL_INT32, p, ep->comm, st), "dispatch recv");
  }
  ok = nccl_ok(api, api->GroupEnd(), "ncclGroupEnd") && ok;
  if (!ok) return 0;
  if (!ep_phase_b(m, c, st)) return 0;
  // return: result rows of the pairs, unweighted
  ok = nccl_ok(api, api->GroupStart(), "ncclGroupStart");
  for (int pos = 1; ok && pos < world; ++pos) {
    const int p = colib::ep_rank_at(pos, rank);
    if (c.recv_pair[p] > 0)
      ok = nccl_ok(api, api->Send(ep->ret_send + (size_t)c.ret_send_off[p] * H, (size_t)c.recv_pair[p] * H, COLI_NCCL_BF16, p, ep->comm, st), "return send");
    if (ok && c.send_pair[p] > 0)
      ok = nccl_ok(api, api->Recv(ep->ret_recv + (size_t)c.ret_recv_off[p] * H, (size_t)c.send_pair[p] * H, COLI_NCCL_BF16, p, ep->comm, st), "return recv");
  }
  ok = nccl_ok(api, api->GroupEnd(), "ncclGroupEnd") && ok;
  if (!ok) return 0;
  if (!ep_phase_c(m, out_dev, T_local, st)) return 0;
  return ep_finish_timing(m);
}

// One barrier of the direct transport on this handle alone, for the test of the bounded wait: the
// handle signals its peers and waits for them exactly as inside the expert-parallel call, with a wait
// of about 13 ms instead of two seconds.  With `peers_arrive` the peers' counts are written into the own
// flag row first (the wait succeeds); without it nothing ever sets them, the wait runs out, and
// coli_b200_moe_check reports the abandoned barrier.  Needs a handle of the direct transport whose peer
// slabs are known (any expert-parallel or emulated call made before).
extern "C" int coli_b200_ep_barrier_probe(ColiMoe *m, int peers_arrive, void *stream) {
  if (!m || !m->ep || !m->ep->direct || !m->ep->slab || !coli_select_ctx(m->ctx)) {
    coli_set_error("ep_barrier_probe: the handle has no direct-transport expert-parallel state");
    return 0;
  }
  ColiEp *ep = m->ep;
  cudaStream_t st = (cudaStream_t)stream;
  colib::EpPeers peers;
  for (int d = 0; d < EP_MAX_WORLD; ++d) {
    peers.slab[d] = d < ep->world ? ep->peer_slab[d] : nullptr;
    if (d < ep->world && !peers.slab[d]) {
      coli_set_error("ep_barrier_probe: the slab of rank %d is not known to this handle yet", d);
      return 0;
    }
  }
  ++ep->epoch;
  if (peers_arrive)
    colib::k_fill_i32<<<1, 32, 0, st>>>(reinterpret_cast<int32_t *>(ep->slab + ep->flag_off), ep->world, ep->epoch);
  colib::k_ep_flag_barrier<<<1, 32, 0, st>>>(peers, ep->flag_off, ep->rank, ep->world, ep->epoch, 1u << 16, ep->bar_status);
  return coli_cuda_check(cudaGetLastError(), "barrier probe launch") ? 1 : 0;
}

// The same call for `world` handles that live on ONE device in ONE process (ranks[r] created with
// ep_rank = r): the phases run rank after rank on `stream` and the two exchanges are device-to-device
// copies between the handles' buffers.  No rank ever waits for another on the device, so this is safe
// where separate processes sharing a GPU would not be; it exists so that every kernel and every offset
// of the expert-parallel path can be checked against the oracle on a single GPU.
extern "C" int coli_b200_moe_block_ep_emulate(ColiMoe *const *ranks, int world, const void *const *x_dev, void *const *out_dev,
                                              const int *T_local, void *stream) {
  if (!ranks || world < 2 || world > EP_MAX_WORLD || !x_dev || !out_dev || !T_local) {
    coli_set_error("moe_block_ep_emulate: bad argument");
    return 0;
  }
  cudaStream_t st = (cudaStream_t)stream;
  for (int r = 0; r < world; ++r) {
    ColiMoe *m = ranks[r];
    if (!coli_check_T(m, T_local[r], "moe_block_ep_emulate") || !coli_ep_ensure(m, nullptr)) return 0;
    if (m->ep->world != world || m->ep->rank != r || m->ctx != ranks[0]->ctx) {
      coli_set_error("moe_block_ep_emulate: handle %d must have ep_rank=%d, ep_world=%d and share rank 0's device", r, r, world);
      return 0;
    }
  }
  const int H = ranks[0]->L.H, k = ranks[0]->L.k;
  if (ranks[0]->ep->direct) {  // the slabs of the other handles are plain pointers in this process
    for (int r = 0; r < world; ++r) {
      if (!ranks[r]->ep->direct || ranks[r]->max_tokens != ranks[0]->max_tokens) {
        coli_set_error("moe_block_ep_emulate: all handles must use the same transport and max_tokens");
        return 0;
      }
      for (int j = 0; j < world; ++j) ranks[r]->ep->peer_slab[j] = ranks[j]->ep->slab;
    }
    for (int r = 0; r < world; ++r)
      if (!ep_phase_a(ranks[r], x_dev[r], T_local[r], st)) return 0;
    for (int r = 0; r < world; ++r) {  // stream order is the barrier here
      ColiEp *ep = ranks[r]->ep;
      if (ep->timing) CK(cudaEventRecord(ep->ev_t[3], st), "stage event");
      if (!ep_direct_phase_b(ranks[r], st)) return 0;
    }
    for (int r = 0; r < world; ++r) {
      if (!ep_phase_c(ranks[r], out_dev[r], T_local[r], st)) return 0;
      if (!ep_finish_timing(ranks[r])) return 0;
    }
    return 1;
  }
  for (int r = 0; r < world; ++r)
    if (!ep_phase_a(ranks[r], x_dev[r], T_local[r], st)) return 0;
  for (int r = 0; r < world; ++r)
    for (int j = 0; j < world; ++j)
      CK(cudaMemcpyAsync(ranks[j]->ep->all_cnt + (size_t)r * 2 * world, ranks[r]->ep->cnt, sizeof(int32_t) * 2 * world, cudaMemcpyDeviceToDevice, st),
         "count copy");
  for (int r = 0; r < world; ++r)
    CK(cudaMemcpyAsync(ranks[r]->ep->h_all_cnt, ranks[r]->ep->all_cnt, sizeof(int32_t) * 2 * world * world, cudaMemcpyDeviceToHost, st), "count download");
  CK(cudaStreamSynchronize(st), "count wait");
  std::vector<EpCounts> cs(world);
  for (int r = 0; r < world; ++r) {
    ColiEp *ep = ranks[r]->ep;
    if (ep->timing) CK(cudaEventRecord(ep->ev_t[3], st), "stage event");
    if (!ep_check_capacity(ranks[r], ep->h_all_cnt)) return 0;
    ep_counts(ep->h_all_cnt, world, r, cs[r]);
  }
  for (int s = 0; s < world; ++s)
    for (int d = 0; d < world; ++d) {
      if (s == d || cs[s].send_tok[d] == 0) continue;
      const size_t n = (size_t)cs[s].send_tok[d];
      CK(cudaMemcpyAsync(ranks[d]->ep->recv_x + (size_t)cs[d].recv_off[s] * H, ranks[s]->ep->send_x + (size_t)cs[s].send_off[d] * H,
                         n * H * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice, st), "dispatch copy");
      CK(cudaMemcpyAsync(ranks[d]->ep->recv_meta + (size_t)cs[d].recv_off[s] * k, ranks[s]->ep->send_meta + (size_t)cs[s].send_off[d] * k,
                         n * k * sizeof(int32_t), cudaMemcpyDeviceToDevice, st), "dispatch copy");
    }
  for (int r = 0; r < world; ++r)
    if (!ep_phase_b(ranks[r], cs[r], st)) return 0;
  for (int s = 0; s < world; ++s)  // s = expert rank, d = home rank
    for (int d = 0; d < world; ++d) {
      if (s == d || cs[s].recv_pair[d] == 0) continue;
      CK(cudaMemcpyAsync(ranks[d]->ep->ret_recv + (size_t)cs[d].ret_recv_off[s] * H, ranks[s]->ep->ret_send + (size_t)cs[s].ret_send_off[d] * H,
                         (size_t)cs[s].recv_pair[d] * H * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice, st), "return copy");
    }
  for (int r = 0; r < world; ++r) {
    if (!ep_phase_c(ranks[r], out_dev[r], T_local[r], st)) return 0;
    if (!ep_finish_timing(ranks[r])) return 0;
  }
  return 1;
}
