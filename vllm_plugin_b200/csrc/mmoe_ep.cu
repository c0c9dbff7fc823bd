// Expert-parallel exchange over NVLink peer memory: every rank's workspace is mapped into every other rank's address
// space (symmetric allocation), and three small kernels move the data with plain peer stores -- no host round trip, no
// split sizes on the host, so a whole EP call can be captured in a CUDA graph.
//
//   publish   per-(source, local expert) route counts and per-destination totals into every peer + flag 0
//   push      wait flag 0; copy each route's FP8 row, scale words and weight straight from the staged inputs into the
//             destination rank's receive buffers (receive order = source rank, expert, token, slot) + flag 1
//   return    after the experts ran: copy every BF16 output row back into its source rank's `ret_recv` at the
//             source's own send position + flag 2; when the GEMM2 epilogue stores its rows straight into the source
//             rank's `ret_recv` (fused write-back), only the flag is left to do
//
// The same exchange exists in the reference as in-kernel NVLink pushes/pulls (backend/kernel/dispatch.py:348-589,
// epilogue.py:407-413, comm.py:277-318).  Flags are per-call epochs written with release semantics at system scope and
// read with acquire loads; every wait is bounded and reports through the status words instead of trapping.  No
// multimem, no TMA from peer memory: plain 16-byte loads and stores only.
#include <stddef.h>

#include "mmoe_common.cuh"

namespace mmoe {

namespace {

constexpr int kMaxRanks = 32;
struct EpSync {                       // lives in the `ep_sync` region of every rank's workspace
  int32_t epoch;                      // epoch of the call in progress (written by publish)
  int32_t done[2];                    // blocks of push / return that have finished (reset by publish)
  int32_t pad[13];
  uint32_t flags[3][kMaxRanks];       // flags[b][s] = last epoch for which rank s passed barrier b towards this rank
  int32_t totals[kMaxRanks][kMaxRanks];   // totals[s][d] = routes rank s sends to rank d in the current call
};

struct Peers {
  char* base[kMaxRanks];
};

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// one warp copies a row of `vec` 16-byte vectors, four loads in flight per lane
__device__ __forceinline__ void copy_row(uint4* __restrict__ dst, const uint4* __restrict__ src, int vec, int lane) {
  for (int v0 = lane; v0 < vec; v0 += 128) {
    uint4 q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v0 + 32 * u < vec) q[u] = src[v0 + 32 * u];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v0 + 32 * u < vec) dst[v0 + 32 * u] = q[u];
  }
}

// thread s < R waits until rank s has passed barrier `b` of epoch `epoch`; bounded
__device__ void wait_flags(EpSync* sync, int b, int num_ranks, uint32_t epoch, int64_t timeout_ns, int32_t* status) {
  if ((int)threadIdx.x < num_ranks) {
    const uint64_t t0 = timer_ns();
    uint32_t spins = 0;
    while (ld_acquire_sys(&sync->flags[b][threadIdx.x]) < epoch) {
      if ((++spins & 255u) == 0u && timer_ns() - t0 > (uint64_t)timeout_ns) {
        if (atomicCAS(&status[kStatusTimeout], 0, 1) == 0) {
          status[kStatusKernel] = 10 + b;
          status[kStatusRole] = threadIdx.x;      // the rank that did not arrive
          status[kStatusBlock] = blockIdx.x;
        }
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(1024) ep_publish_kernel(Peers peers, MmoeLayout lay, int num_ranks, int me, int e_local) {
  char* ws = peers.base[me];
  EpSync* sync = reinterpret_cast<EpSync*>(ws + lay.ep_sync);
  const int32_t* send_count = reinterpret_cast<const int32_t*>(ws + lay.send_count);
  __shared__ int32_t tot[kMaxRanks];
  const uint32_t epoch = static_cast<uint32_t>(sync->epoch) + 1u;
  if ((int)threadIdx.x < num_ranks) {
    int t = 0;
    for (int e = 0; e < e_local; ++e) t += send_count[threadIdx.x * e_local + e];
    tot[threadIdx.x] = t;
  }
  __syncthreads();
  const int num_experts = num_ranks * e_local;
  for (int i = threadIdx.x; i < num_experts; i += blockDim.x) {      // recv_count[me][e] on the rank that owns expert i
    const int d = i / e_local, e = i - d * e_local;
    reinterpret_cast<int32_t*>(peers.base[d] + lay.recv_count)[me * e_local + e] = send_count[i];
  }
  for (int i = threadIdx.x; i < num_ranks * num_ranks; i += blockDim.x) {   // my totals row into every rank's table
    const int d = i / num_ranks, dd = i - d * num_ranks;
    reinterpret_cast<EpSync*>(peers.base[d] + lay.ep_sync)->totals[me][dd] = tot[dd];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    sync->epoch = static_cast<int32_t>(epoch);
    sync->done[0] = 0;
    sync->done[1] = 0;
    __threadfence();
  }
  if ((int)threadIdx.x < num_ranks)
    st_release_sys(&reinterpret_cast<EpSync*>(peers.base[threadIdx.x] + lay.ep_sync)->flags[0][me], epoch);
}

// one warp per route of this rank, in send order
__global__ void __launch_bounds__(256) ep_push_kernel(Peers peers, MmoeLayout lay, int num_ranks, int me, int e_local,
                                                      int h, int k, int64_t timeout_ns) {
  char* ws = peers.base[me];
  EpSync* sync = reinterpret_cast<EpSync*>(ws + lay.ep_sync);
  int32_t* status = reinterpret_cast<int32_t*>(ws + lay.status);
  const uint32_t epoch = static_cast<uint32_t>(sync->epoch);
  wait_flags(sync, 0, num_ranks, epoch, timeout_ns, status);         // every rank's counts and totals have landed here
  __shared__ int32_t send_off[kMaxRanks + 1], recv_base[kMaxRanks];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int d = 0; d < num_ranks; ++d) { send_off[d] = run; run += sync->totals[me][d]; }
    send_off[num_ranks] = run;
  }
  if ((int)threadIdx.x < num_ranks) {                                 // where my block starts in rank d's receive order
    int b = 0;
    for (int s = 0; s < me; ++s) b += sync->totals[s][threadIdx.x];
    recv_base[threadIdx.x] = b;
  }
  __syncthreads();
  const int total = send_off[num_ranks];
  const uint4* x = reinterpret_cast<const uint4*>(ws + lay.x);
  const int32_t* x_sf = reinterpret_cast<const int32_t*>(ws + lay.x_sf);
  const float* topk_w = reinterpret_cast<const float*>(ws + lay.topk_weights);
  const int32_t* sorted_route = reinterpret_cast<const int32_t*>(ws + lay.sorted_route);
  const int vec = h / 16, words = h / kTileK;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < total; p += warps) {
    int d = 0;
    while (p >= send_off[d + 1]) ++d;
    const int64_t row = recv_base[d] + (p - send_off[d]);
    const int route = sorted_route[p];
    const int t = route / k;
    char* peer = peers.base[d];
    uint4* dx = reinterpret_cast<uint4*>(peer + lay.recv_x) + row * vec;
    copy_row(dx, x + (int64_t)t * vec, vec, lane);
    int32_t* dsf = reinterpret_cast<int32_t*>(peer + lay.recv_sf) + row * words;
    for (int w = lane; w < words; w += 32) dsf[w] = x_sf[(int64_t)t * words + w];
    if (lane == 0) reinterpret_cast<float*>(peer + lay.recv_w)[row] = topk_w[route];
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = atomicAdd(&sync->done[0], 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (last && (int)threadIdx.x < num_ranks) {
    __threadfence_system();
    st_release_sys(&reinterpret_cast<EpSync*>(peers.base[threadIdx.x] + lay.ep_sync)->flags[1][me], epoch);
  }
}

__global__ void __launch_bounds__(32) ep_wait_kernel(Peers peers, MmoeLayout lay, int num_ranks, int me, int barrier,
                                                     int64_t timeout_ns) {
  char* ws = peers.base[me];
  EpSync* sync = reinterpret_cast<EpSync*>(ws + lay.ep_sync);
  wait_flags(sync, barrier, num_ranks, static_cast<uint32_t>(sync->epoch), timeout_ns,
             reinterpret_cast<int32_t*>(ws + lay.status));
}

// one warp per received route: its BF16 output row goes home to the source rank, at the source's send position
__global__ void __launch_bounds__(256) ep_return_kernel(Peers peers, MmoeLayout lay, int num_ranks, int me, int h) {
  char* ws = peers.base[me];
  EpSync* sync = reinterpret_cast<EpSync*>(ws + lay.ep_sync);
  const uint32_t epoch = static_cast<uint32_t>(sync->epoch);
  __shared__ int32_t rank_off[kMaxRanks + 1], home_base[kMaxRanks];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int s = 0; s < num_ranks; ++s) { rank_off[s] = run; run += sync->totals[s][me]; }
    rank_off[num_ranks] = run;
  }
  if ((int)threadIdx.x < num_ranks) {          // where the rows that rank s sent to me start in rank s's send order
    int b = 0;
    for (int d = 0; d < me; ++d) b += sync->totals[threadIdx.x][d];
    home_base[threadIdx.x] = b;
  }
  __syncthreads();
  const int total = rank_off[num_ranks];
  const int vec = h / 8;
  const uint4* ret = reinterpret_cast<const uint4*>(ws + lay.ret);
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < total; r += warps) {
    int s = 0;
    while (r >= rank_off[s + 1]) ++s;
    const int64_t row = home_base[s] + (r - rank_off[s]);
    uint4* dst = reinterpret_cast<uint4*>(peers.base[s] + lay.ret_recv) + row * vec;
    copy_row(dst, ret + (int64_t)r * vec, vec, lane);
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = atomicAdd(&sync->done[1], 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (last && (int)threadIdx.x < num_ranks) {
    __threadfence_system();
    st_release_sys(&reinterpret_cast<EpSync*>(peers.base[threadIdx.x] + lay.ep_sync)->flags[2][me], epoch);
  }
}

// Fused write-back: the GEMM2 epilogue has already stored every output row into its source rank's `ret_recv`; the
// kernel boundary completed those stores, so one warp only has to publish barrier 2.
__global__ void __launch_bounds__(32) ep_signal_kernel(Peers peers, MmoeLayout lay, int num_ranks, int me) {
  EpSync* sync = reinterpret_cast<EpSync*>(peers.base[me] + lay.ep_sync);
  const uint32_t epoch = static_cast<uint32_t>(sync->epoch);
  __threadfence_system();
  if ((int)threadIdx.x < num_ranks)
    st_release_sys(&reinterpret_cast<EpSync*>(peers.base[threadIdx.x] + lay.ep_sync)->flags[2][me], epoch);
}

Peers make_peers(const void* const* peer_ws, int num_ranks) {
  Peers p{};
  for (int i = 0; i < num_ranks; ++i) p.base[i] = static_cast<char*>(const_cast<void*>(peer_ws[i]));
  return p;
}

}  // namespace

int ep_sync_bytes() { return static_cast<int>(sizeof(EpSync)); }
int ep_totals_offset() { return static_cast<int>(offsetof(EpSync, totals)); }
static_assert(kMaxRanks == 32, "the GEMM2 kernel indexes the totals table as [32][32]");

cudaError_t launch_ep_dispatch(const Ctx& c, const void* const* peer_ws, int m, int64_t timeout_ns, cudaStream_t s) {
  (void)m;
  const Peers peers = make_peers(peer_ws, c.geo.num_ranks);
  ep_publish_kernel<<<1, 1024, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank, c.e_local);
  ep_push_kernel<<<148 * 2, 256, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank, c.e_local, c.geo.hidden, c.geo.num_topk,
                                         timeout_ns);
  ep_wait_kernel<<<1, 32, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank, 1, timeout_ns);
  return cudaGetLastError();
}

cudaError_t launch_ep_return(const Ctx& c, const void* const* peer_ws, int64_t timeout_ns, cudaStream_t s) {
  const Peers peers = make_peers(peer_ws, c.geo.num_ranks);
  ep_return_kernel<<<148 * 2, 256, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank, c.geo.hidden);
  ep_wait_kernel<<<1, 32, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank, 2, timeout_ns);
  return cudaGetLastError();
}

cudaError_t launch_ep_signal_return(const Ctx& c, const void* const* peer_ws, int64_t timeout_ns, cudaStream_t s) {
  const Peers peers = make_peers(peer_ws, c.geo.num_ranks);
  ep_signal_kernel<<<1, 32, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank);
  ep_wait_kernel<<<1, 32, 0, s>>>(peers, c.lay, c.geo.num_ranks, c.geo.rank, 2, timeout_ns);
  return cudaGetLastError();
}

}  // namespace mmoe
