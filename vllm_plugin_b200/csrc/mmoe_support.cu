// HBM-bound support kernels of the MegaMoE layer for sm_100a: input quantiser, route ordering, pool plan and
// placement, top-k combine.  All integer work here is deterministic (no order-dependent atomics), so the dispatch
// layout is reproducible run to run.
#include <stdlib.h>

#include <algorithm>
#include <atomic>

#include <cuda_fp4.h>

#include "mmoe_common.cuh"

namespace mmoe {

// ---------------------------------------------------------------------------------------------------------------------
// Host side of the chained (programmatic dependent) launches.  MMOE_DISABLE_CHAINED_LAUNCH=1 in the environment turns
// the attribute off for the whole process (every launch then waits for the full completion of its predecessor).
// ---------------------------------------------------------------------------------------------------------------------
namespace {
thread_local bool g_break_chain = false;
thread_local bool g_chain_scope = false;   // inside a ChainScope(true) of this thread
bool chaining_enabled() {
  static const bool on = [] {
    const char* v = getenv("MMOE_DISABLE_CHAINED_LAUNCH");
    return !(v != nullptr && v[0] != '\0' && v[0] != '0');
  }();
  return on;
}
}  // namespace

ChainScope::ChainScope(bool on) : saved_(g_chain_scope) { g_chain_scope = on && chaining_enabled(); }
ChainScope::~ChainScope() { g_chain_scope = saved_; }

void break_chain() { g_break_chain = true; }

bool take_chain_flag() {
  const bool broken = g_break_chain;
  g_break_chain = false;
  return g_chain_scope && !broken;
}

// =====================================================================================================================
// Kernel (a): BF16 -> MXFP8 E4M3 with one UE8M0 scale per 32 elements, four scale bytes per int32 word.
// Follows the reference quantiser (backend/staging.py:36-82): scale = 2^ceil(log2(max(amax, 1e-4) / 448)), exponent
// clamped to [1, 254]; values multiplied by the exact reciprocal and rounded to nearest even.
// One thread converts 8 elements (one 16-byte load, one 8-byte store); 4 threads share a scale, 16 a scale word.
// =====================================================================================================================
__device__ __forceinline__ void stage_vector(const uint4& raw, bool live, int64_t i, int vec_per_row, int h,
                                             uint2* __restrict__ x_q, int32_t* __restrict__ x_sf,
                                             int32_t* __restrict__ shared_sf, int64_t shared_rows, int shared_bm) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float v[8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, 1e-4f);
  const uint32_t bits = __float_as_uint(__fdiv_rn(amax, 448.0f));
  int e = static_cast<int>((bits >> 23) & 0xFFu) + ((bits & 0x7FFFFFu) != 0u);
  e = min(max(e, 1), 254);
  const float inv = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);   // exact reciprocal of 2^(e-127), e in [1, 253]
  const float inv_exact = e == 254 ? __fdiv_rn(1.0f, __uint_as_float(254u << 23)) : inv;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= static_cast<uint32_t>(float_to_e4m3(__fmul_rn(v[j], inv_exact))) << (8 * j);
    hi |= static_cast<uint32_t>(float_to_e4m3(__fmul_rn(v[4 + j], inv_exact))) << (8 * j);
  }
  if (live) x_q[i] = make_uint2(lo, hi);
  // scale word: lanes 0,4,8,12 of each 16-lane group hold the four exponents
  const int lane = threadIdx.x & 31;
  const int base = lane & 16;
  uint32_t word = static_cast<uint32_t>(__shfl_sync(0xffffffffu, e, base + 0));
  word |= static_cast<uint32_t>(__shfl_sync(0xffffffffu, e, base + 4)) << 8;
  word |= static_cast<uint32_t>(__shfl_sync(0xffffffffu, e, base + 8)) << 16;
  word |= static_cast<uint32_t>(__shfl_sync(0xffffffffu, e, base + 12)) << 24;
  if (live && (lane & 15) == 0) {
    const int64_t t = i / vec_per_row;
    const int w = static_cast<int>(i - t * vec_per_row) / 16;
    x_sf[t * (h / kTileK) + w] = static_cast<int32_t>(word);
    if (shared_bm > 0) {
      // row of token t in the BLOCK_M-dependent shared-expert scale layout (backend/staging.py:85-95)
      const int64_t mm = t % shared_bm;
      const int64_t bm_al = (shared_bm + 127) / 128 * 128;
      const int64_t row = (t / shared_bm) * bm_al + (mm / 128) * 128 + (mm % 32) * 4 + (mm % 128) / 32;
      shared_sf[(int64_t)w * shared_rows + row] = static_cast<int32_t>(word);
    }
  }
}

// Router in front of the quantiser (one warp per token): the k largest gate logits (ties: the lower expert id), weights =
// softmax over the selected logits, and -- when a replica table is given -- the physical copy `(token + slot) % copies`
// of every selected logical expert, which is the choice a serving engine makes before it calls the layer.
struct RouterArgs {
  const float* logits;           // [m, num_logical] or NULL: ids / weights are given and only repacked
  int num_logical;
  const int32_t* replica_count;  // [num_logical] or NULL: logical id == physical id
  const int32_t* replica_slots;  // [num_logical, max_copies]
  int max_copies;
};

__device__ void route_token(const RouterArgs& r, int64_t t, int k, bool is_pad, int64_t* __restrict__ ids_out,
                            float* __restrict__ w_out) {
  const int lane = threadIdx.x & 31;
  const float* row = r.logits + t * r.num_logical;
  uint64_t taken = 0;                               // bit j: this lane's element lane + 32 j has been selected
  float best_val = 0.f, sum = 0.f;
  float my_val = 0.f;                               // lane s < k keeps the s-th selection
  int my_idx = -1;
  for (int s = 0; s < k; ++s) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int e = lane, j = 0; e < r.num_logical; e += 32, ++j) {
      const float x = row[e];
      if (!((taken >> j) & 1ull) && (x > v || (x == v && e < idx))) { v = x; idx = e; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, d);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, d);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if ((idx & 31) == lane && idx < r.num_logical) taken |= 1ull << (idx >> 5);
    if (s == 0) best_val = v;
    const float ex = expf(v - best_val);
    sum += ex;
    if (lane == s) { my_val = ex; my_idx = idx; }
  }
  if (lane < k) {
    int64_t id = my_idx;
    if (r.replica_count != nullptr && my_idx >= 0 && my_idx < r.num_logical) {
      const int copies = max(1, r.replica_count[my_idx]);
      id = r.replica_slots[(int64_t)my_idx * r.max_copies + static_cast<int>((t + lane) % copies)];
    }
    ids_out[t * k + lane] = is_pad ? -1 : id;
    w_out[t * k + lane] = is_pad ? 0.f : __fdiv_rn(my_val, sum);
  }
}

__global__ void __launch_bounds__(256) stage_kernel(
    const uint4* __restrict__ hidden, uint2* __restrict__ x_q, int32_t* __restrict__ x_sf,
    int32_t* __restrict__ shared_sf, int64_t shared_rows, int shared_bm,
    const void* __restrict__ ids_in, int ids64, const float* __restrict__ w_in, const uint8_t* __restrict__ pad,
    int64_t* __restrict__ ids_out, float* __restrict__ w_out, int m, int h, int k, RouterArgs router) {
  chain_begin();
  const int vec_per_row = h / 8;
  const int64_t total = (int64_t)m * vec_per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total_padded = (total + 31) / 32 * 32;   // whole warps iterate together (shuffles inside)
  // four independent 16-byte loads in flight per thread before any of them is consumed
  for (int64_t i = tid; i < total_padded; i += 4 * stride) {
    uint4 raw[4];
    bool live[4], active[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t iu = i + u * stride;
      active[u] = iu < total_padded;           // warp-uniform: stride and total_padded are multiples of 32
      live[u] = iu < total;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (live[u]) raw[u] = hidden[iu];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (active[u]) stage_vector(raw[u], live[u], i + u * stride, vec_per_row, h, x_q, x_sf, shared_sf, shared_rows, shared_bm);
  }
  if (router.logits != nullptr) {
    const int64_t warp = tid >> 5, warps = stride >> 5;
    for (int64_t t = warp; t < m; t += warps) route_token(router, t, k, pad != nullptr && pad[t] != 0, ids_out, w_out);
    return;
  }
  // routing repack (backend/staging.py:244-251)
  const int64_t routes = (int64_t)m * k;
  for (int64_t r = tid; r < routes; r += stride) {
    const int64_t t = r / k;
    const bool is_pad = pad != nullptr && pad[t] != 0;
    const int64_t id = ids64 ? static_cast<const int64_t*>(ids_in)[r] : static_cast<const int32_t*>(ids_in)[r];
    ids_out[r] = is_pad ? -1 : id;
    w_out[r] = is_pad ? 0.f : w_in[r];
  }
}

cudaError_t launch_stage(const Ctx& c, const void* hidden, const void* ids, int ids64, const float* w,
                         const uint8_t* pad, int m, int shared_bm, cudaStream_t s) {
  return launch_route_stage(c, hidden, ids, ids64, w, nullptr, 0, nullptr, nullptr, 0, pad, m, shared_bm, s);
}

cudaError_t launch_route_stage(const Ctx& c, const void* hidden, const void* ids, int ids64, const float* w,
                               const float* logits, int num_logical, const int32_t* replica_count,
                               const int32_t* replica_slots, int max_copies, const uint8_t* pad, int m, int shared_bm,
                               cudaStream_t s) {
  if (m == 0) return cudaSuccess;
  const int h = c.geo.hidden;
  const int64_t total = (int64_t)m * h / 8;
  int blocks = static_cast<int>(std::min<int64_t>((total + 1023) / 1024, 148 * 8));
  if (blocks < 1) blocks = 1;
  const RouterArgs router{logits, num_logical, replica_count, replica_slots, max_copies};
  launch_chained(stage_kernel, dim3(blocks), dim3(256), 0, s, static_cast<const uint4*>(hidden), c.at<uint2>(c.lay.x), c.at<int32_t>(c.lay.x_sf),
      c.at<int32_t>(c.lay.shared_x_sf), c.lay.shared_sf_rows, c.geo.num_shared_experts > 0 ? shared_bm : 0, ids, ids64, w,
      pad, c.at<int64_t>(c.lay.topk_idx), c.at<float>(c.lay.topk_weights), m, h, c.geo.num_topk, router);
  return cudaGetLastError();
}

// =====================================================================================================================
// NVFP4 activation staging: BF16 -> packed E2M1 with one E4M3 scale per 16 elements and a per-tensor FP32 scale (the
// two-level NVFP4 recipe).  The serving engine's hook names such a staging call next to the MXFP8 one
// (patches/vllm-megamoe-plugin.patch:10, `prepare_megamoe_nvfp4_inputs`); the reference plugin itself never implements
// it.  Per block of 16:  s = e4m3_rn(amax * global_scale / 6);  q_i = e2m1_rn(x_i * global_scale / s)  (0 when s == 0);
// x is recovered as q * s / global_scale.  Low nibble = even K, as in the MXFP4 weights.  One thread owns a block (two
// 16-byte loads, one 8-byte store, one scale byte).
// =====================================================================================================================
__global__ void __launch_bounds__(256) stage_nvfp4_kernel(const uint4* __restrict__ hidden, uint2* __restrict__ q_out,
                                                          uint8_t* __restrict__ sf_out, float global_scale, int64_t blocks16) {
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks16; b += (int64_t)gridDim.x * blockDim.x) {
    const uint4 raw[2] = {hidden[2 * b], hidden[2 * b + 1]};
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        v[8 * u + 2 * j] = f.x;
        v[8 * u + 2 * j + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
    const float s = fminf(__fdiv_rn(__fmul_rn(amax, global_scale), 6.0f), 448.0f);
    const uint8_t s8 = float_to_e4m3(s);
    const float sf = e4m3_to_float(s8);
    const float inv = sf != 0.f ? __fdiv_rn(global_scale, sf) : 0.f;
    uint32_t w[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t byte = __nv_cvt_float2_to_fp4x2(make_float2(__fmul_rn(v[2 * j], inv), __fmul_rn(v[2 * j + 1], inv)), __NV_E2M1,
                                                     cudaRoundNearest);
      w[j >> 2] |= (byte & 0xFFu) << (8 * (j & 3));
    }
    q_out[b] = make_uint2(w[0], w[1]);
    sf_out[b] = s8;
  }
}

cudaError_t launch_stage_nvfp4(const void* hidden, void* q_out, void* sf_out, float global_scale, int64_t num_tokens, int hidden_size,
                               cudaStream_t s) {
  const int64_t blocks16 = num_tokens * hidden_size / 16;
  if (blocks16 == 0) return cudaSuccess;
  const int grid = static_cast<int>(std::min<int64_t>((blocks16 + 255) / 256, 148 * 16));
  stage_nvfp4_kernel<<<grid, 256, 0, s>>>(static_cast<const uint4*>(hidden), static_cast<uint2*>(q_out),
                                          static_cast<uint8_t*>(sf_out), global_scale, blocks16);
  return cudaGetLastError();
}

// =====================================================================================================================
// Route ordering: a stable counting sort of the routes (token*k + slot) by destination expert in three passes over
// chunks of 128 tokens.  Replaces the atomics-ordered slot assignment of the reference (backend/kernel/dispatch.py:
// 348-410) with a deterministic order; the per-expert counts are the same numbers.
// =====================================================================================================================
// ---------------------------------------------------------------------------------------------------------------------
// small block-level building blocks of the route ordering and the plan
// ---------------------------------------------------------------------------------------------------------------------
// Exclusive prefix sum of `in[0..n)` into `out[0..n]` (out[n] = total), n <= 1024, whole block (>= 32 threads, a
// multiple of 32) participates; `in` and `out` may not alias.  Ends with a barrier.
__device__ void block_exclusive_scan(const int32_t* in, int32_t* out, int n) {
  __shared__ int32_t warp_tot[33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  __syncthreads();
  int carry = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    int v = i < n ? in[i] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = lane < nwarps ? warp_tot[lane] : 0;
      int wi = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += t;
      }
      warp_tot[lane] = wi - w;                 // exclusive offset of each warp
      if (lane == 31) warp_tot[32] = wi;       // block total of this round
    }
    __syncthreads();
    if (i < n) out[i] = carry + warp_tot[warp] + incl - v;
    carry += warp_tot[32];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[n] = carry;
  __syncthreads();
}

// Stable rank of every route among the routes of the same expert, by ONE warp walking the routes in order, 32 at a
// time: lanes with the same expert find each other with match.any, the lowest such lane owns the running counter.
// `ids[i]` (-1 = masked) in shared memory, `count[e]` zeroed shared counters; writes rank[i] (or -1).
__device__ void warp_rank_routes(const int32_t* ids, int n, int32_t* count, int32_t* rank) {
  const int lane = threadIdx.x & 31;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    const int e = i < n ? ids[i] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    int r = -1;
    if (e >= 0) {
      const int before = __popc(peers & ((1u << lane) - 1u));
      const int start = count[e];
      r = start + before;
    }
    __syncwarp();
    if (e >= 0 && (peers & ((1u << lane) - 1u)) == 0u) count[e] += __popc(peers);   // lowest lane of each expert group
    __syncwarp();
    if (i < n) rank[i] = r;
  }
}

constexpr int kSortThreads = 256;

// pass A: per chunk, local rank of every route among the chunk's routes to the same expert + per-chunk expert counts
__global__ void __launch_bounds__(kSortThreads) sort_local_kernel(
    const int64_t* __restrict__ topk_idx, int32_t* __restrict__ route_pos, int32_t* __restrict__ chunk_count,
    int32_t* __restrict__ status, int m, int k, int num_experts) {
  chain_begin();
  extern __shared__ int32_t sm[];
  int32_t* ids = sm;                                // [chunk routes]
  int32_t* hist = sm + kSortChunkTokens * k;        // [num_experts]
  const int chunk = blockIdx.x;
  const int r0 = chunk * kSortChunkTokens * k;
  const int n = min(kSortChunkTokens * k, m * k - r0);
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int64_t id = topk_idx[r0 + i];
    if (id >= num_experts) { if (status != nullptr) report_bad_index(status); id = -1; }
    ids[i] = id < 0 ? -1 : static_cast<int32_t>(id);
  }
  __syncthreads();
  if (threadIdx.x < 32) warp_rank_routes(ids, n, hist, route_pos + r0);
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) chunk_count[(int64_t)chunk * num_experts + e] = hist[e];
}

// pass B: one block; per expert an exclusive scan over chunks, then an exclusive scan over experts
__global__ void __launch_bounds__(1024) sort_scan_kernel(
    int32_t* __restrict__ chunk_count, int32_t* __restrict__ send_count, int32_t* __restrict__ send_offset,
    int32_t* __restrict__ recv_count_if_single, int num_chunks, int num_experts) {
  chain_begin();
  __shared__ int32_t totals[2048 + 1];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < num_chunks; ++c) {
      const int v = chunk_count[(int64_t)c * num_experts + e];
      chunk_count[(int64_t)c * num_experts + e] = run;
      run += v;
    }
    totals[e] = run;
    send_count[e] = run;
    if (recv_count_if_single != nullptr) recv_count_if_single[e] = run;
  }
  __shared__ int32_t offs[2048 + 1];
  block_exclusive_scan(totals, offs, num_experts);
  for (int e = threadIdx.x; e <= num_experts; e += blockDim.x) send_offset[e] = offs[e];
}

// pass C: final position of every route, and the inverse map
__global__ void __launch_bounds__(kSortThreads) sort_place_kernel(
    const int64_t* __restrict__ topk_idx, const int32_t* __restrict__ chunk_base,
    const int32_t* __restrict__ send_offset, int32_t* __restrict__ route_pos, int32_t* __restrict__ sorted_route,
    int m, int k, int num_experts) {
  chain_begin();
  const int64_t total = (int64_t)m * k;
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < total; r += (int64_t)gridDim.x * blockDim.x) {
    const int64_t id = topk_idx[r];
    int pos = -1;
    if (id >= 0 && id < num_experts) {
      const int chunk = static_cast<int>(r / (kSortChunkTokens * k));
      pos = send_offset[id] + chunk_base[(int64_t)chunk * num_experts + id] + route_pos[r];
      sorted_route[pos] = static_cast<int32_t>(r);
    }
    route_pos[r] = pos;
  }
}

cudaError_t launch_count_sort(const Ctx& c, int m, cudaStream_t s) {
  const int k = c.geo.num_topk, e = c.geo.num_experts;
  const int chunks = max(1, (m + kSortChunkTokens - 1) / kSortChunkTokens);
  int32_t* chunk_count = c.at<int32_t>(c.lay.sort_scratch);
  const size_t smem = (size_t)(kSortChunkTokens * k + e) * sizeof(int32_t);
  launch_chained(sort_local_kernel, dim3(chunks), dim3(kSortThreads), smem, s, c.at<int64_t>(c.lay.topk_idx), c.at<int32_t>(c.lay.route_pos),
                                                       chunk_count, c.at<int32_t>(c.lay.status), m, k, e);
  launch_chained(sort_scan_kernel, dim3(1), dim3(1024), 0, s, chunk_count, c.at<int32_t>(c.lay.send_count), c.at<int32_t>(c.lay.send_offset),
                                      c.geo.num_ranks == 1 ? c.at<int32_t>(c.lay.recv_count) : nullptr, chunks, e);
  if (m > 0) {
    const int blocks = static_cast<int>(std::min<int64_t>(((int64_t)m * k + kSortThreads - 1) / kSortThreads, 148 * 8));
    launch_chained(sort_place_kernel, dim3(blocks), dim3(kSortThreads), 0, s, c.at<int64_t>(c.lay.topk_idx), chunk_count,
                                                      c.at<int32_t>(c.lay.send_offset), c.at<int32_t>(c.lay.route_pos),
                                                      c.at<int32_t>(c.lay.sorted_route), m, k, e);
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------------
// Route ordering without any allocation.  The per-chunk expert counts, the only scratch the three passes need, live in
// a file-scope device array: every GPU that loads this library holds these 64 KB until the process exits.  Host code
// may only use the array's *address*, obtained once per device with cudaGetSymbolAddress while that device is current
// (the bare symbol name is a host-side stand-in, not a device pointer).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kStaticMaxTokens = 4096;                                   // 32 chunks of 128 tokens
constexpr int kStaticMaxExperts = 512;
constexpr int kStaticScratchInts = (kStaticMaxTokens / kSortChunkTokens) * kStaticMaxExperts;
static __device__ __align__(256) int32_t g_route_order_scratch[kStaticScratchInts];

namespace {
constexpr int kMaxDevices = 64;
// Written by the first call on a device; every writer stores the same address, so the only requirement is that the
// store and the loads are not torn or reordered: relaxed atomics.
std::atomic<int32_t*> g_scratch_ptr[kMaxDevices] = {};
}

cudaError_t route_order_static(const int64_t* topk_idx, int m, int k, int num_experts, int32_t* send_count,
                               int32_t* send_offset, int32_t* route_pos, int32_t* sorted_route, cudaStream_t s) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  int32_t* chunk_count = g_scratch_ptr[dev].load(std::memory_order_relaxed);
  if (chunk_count == nullptr) {                  // set-up: first call on this device
    // Resolving the symbol may load the module, which a capturing stream forbids: refuse instead of breaking the capture.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(s, &capturing);
    if (e != cudaSuccess) return e;
    if (capturing != cudaStreamCaptureStatusNone) return cudaErrorStreamCaptureUnsupported;
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_route_order_scratch);
    if (e != cudaSuccess) return e;
    chunk_count = static_cast<int32_t*>(ptr);
    g_scratch_ptr[dev].store(chunk_count, std::memory_order_relaxed);
  }
  // nothing in the scratch has to start at zero: pass A overwrites every (chunk, expert) cell that passes B and C read
  const int chunks = std::max(1, (m + kSortChunkTokens - 1) / kSortChunkTokens);
  const size_t smem = (size_t)(kSortChunkTokens * k + num_experts) * sizeof(int32_t);
  sort_local_kernel<<<chunks, kSortThreads, smem, s>>>(topk_idx, route_pos, chunk_count, nullptr, m, k, num_experts);
  sort_scan_kernel<<<1, 1024, 0, s>>>(chunk_count, send_count, send_offset, nullptr, chunks, num_experts);
  if (m > 0) {
    const int blocks = static_cast<int>(std::min<int64_t>(((int64_t)m * k + kSortThreads - 1) / kSortThreads, 148 * 8));
    sort_place_kernel<<<blocks, kSortThreads, 0, s>>>(topk_idx, chunk_count, send_offset, route_pos, sorted_route, m, k,
                                                      num_experts);
  }
  return cudaGetLastError();
}

int route_order_static_max_tokens() { return kStaticMaxTokens; }
int route_order_static_max_experts() { return kStaticMaxExperts; }

// =====================================================================================================================
// EP > 1: gather the rows, scale words and weights of this rank's routes into send order (sorted by destination
// expert, hence by destination rank), ready for the all-to-allv.
// =====================================================================================================================
__global__ void __launch_bounds__(256) pack_kernel(
    const uint4* __restrict__ x, const int32_t* __restrict__ x_sf, const float* __restrict__ topk_w,
    const int32_t* __restrict__ sorted_route, const int32_t* __restrict__ send_offset, uint4* __restrict__ send_x,
    int32_t* __restrict__ send_sf, float* __restrict__ send_w, int h, int k, int num_experts) {
  const int total = send_offset[num_experts];
  const int vec = h / 16, words = h / kTileK;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int p = warp; p < total; p += nwarps) {
    const int route = sorted_route[p];
    const int t = route / k;
    for (int v = lane; v < vec; v += 32) send_x[(int64_t)p * vec + v] = x[(int64_t)t * vec + v];
    for (int w = lane; w < words; w += 32) send_sf[(int64_t)p * words + w] = x_sf[(int64_t)t * words + w];
    if (lane == 0) send_w[p] = topk_w[route];
  }
}

cudaError_t launch_pack(const Ctx& c, int m, cudaStream_t s) {
  if (m == 0) return cudaSuccess;
  pack_kernel<<<148 * 4, 256, 0, s>>>(c.at<uint4>(c.lay.x), c.at<int32_t>(c.lay.x_sf), c.at<float>(c.lay.topk_weights),
                                      c.at<int32_t>(c.lay.sorted_route), c.at<int32_t>(c.lay.send_offset),
                                      c.at<uint4>(c.lay.send_x), c.at<int32_t>(c.lay.send_sf), c.at<float>(c.lay.send_w),
                                      c.geo.hidden, c.geo.num_topk, c.geo.num_experts);
  return cudaGetLastError();
}

// =====================================================================================================================
// Pool plan (one block).  Pool order: local experts ascending, each expert starting on a BLOCK_M boundary
// (backend/kernel/dispatch.py:431-447); inside an expert, source ranks ascending and each source's routes in its send
// order (token, slot) -- a fixed order where the reference's is arrival order.
// =====================================================================================================================

// Shared expert: the call's own tokens in blocks of block_m rows; the scale chunks were written by the quantiser in the
// layout the engine prescribes (128-row chunks inside each block, backend/staging.py:85-95), so a tile is one chunk, or
// one of its two 64-row halves when the chunk holds more rows than a tile may.
__device__ int emit_shared_tiles(Tile* out, int n, int block_m, int cap, bool pair) {
  const int cpb = (block_m + kChunkRows - 1) / kChunkRows;
  int count = 0;
  for (int b = 0; b * block_m < n; ++b) {
    const int in_block = min(block_m, n - b * block_m);
    for (int s = 0; s < cpb; ++s) {
      const int rows = min(kChunkRows, in_block - s * kChunkRows);
      if (rows <= 0) break;
      const int row0 = b * block_m + s * kChunkRows;
      const int chunk = b * cpb + s;
      if (rows > cap) {
        out[count] = Tile{kSharedExpert, row0, 64, chunk, 0, {0, 0, 0}};
        out[count + 1] = Tile{kSharedExpert, row0 + 64, rows - 64, chunk, 2, {0, 0, 0}};
        count += 2;
      } else {
        out[count] = Tile{kSharedExpert, row0, rows, chunk, 0, {0, 0, 0}};
        count += 1;
      }
    }
  }
  if (pair && (count & 1)) out[count++] = Tile{kSharedExpert, 0, 0, 0, 0, {0, 0, 0}};   // empty second half of the last pair
  return count;
}

// Routed expert: its n rows are contiguous in the pool, starting on a block_m boundary (pool block `first_block`).
// They are cut into ceil(n / cap) equal tiles (rounded up to 16 rows) regardless of the block boundaries inside the
// expert; for CTA pairs into an even number of them (the last may be empty), so that tiles 2j and 2j + 1 of the table
// always belong to the same expert.  The scale chunks of the pool are this library's own: tile j of the expert uses chunk j of the
// chunks reserved for the expert's blocks.
__device__ __forceinline__ void tile_cut(int n, int cap, bool pair, int* parts_out, int* step_out) {
  const int parts = pair ? 2 * ((n + 2 * cap - 1) / (2 * cap)) : (n + cap - 1) / cap;
  *parts_out = parts;
  *step_out = parts == 1 ? n : ((n + parts - 1) / parts + 15) & ~15;
}

__device__ int emit_tiles(Tile* out, int expert, int row_base, int n, int block_m, int cap, bool pair, int first_block,
                          bool write) {
  if (n <= 0) return 0;
  int parts, step;
  tile_cut(n, cap, pair, &parts, &step);
  if (write) {
    const int chunk0 = first_block * chunks_per_block(block_m);
    for (int j = 0; j < parts; ++j)
      out[j] = Tile{expert, row_base + j * step, max(0, min(step, n - j * step)), chunk0 + j, 0, {0, 0, 0}};
  }
  return parts;
}

// The shared expert's tiles depend only on the token count, so they can be planned (and run) before the routed
// experts' receive counts are known: written at the tail of the tile table, counted in the header.
__global__ void shared_plan_kernel(char* __restrict__ plan_base, int e_local, int num_ranks, int m, int block_m,
                                   int cap, int pair, int64_t first_tile) {
  chain_begin();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    PlanView pv = plan_view(plan_base, e_local, num_ranks);
    pv.hdr->num_early_shared_tiles = emit_shared_tiles(pv.tiles + first_tile, m, block_m, cap, pair != 0);
  }
}

__global__ void __launch_bounds__(1024) plan_kernel(
    char* __restrict__ plan_base, const int32_t* __restrict__ recv_count, int32_t* __restrict__ stats, int e_local,
    int num_ranks, int block_m, int cap, int pair, int m, int has_shared) {
  chain_begin();
  PlanView pv = plan_view(plan_base, e_local, num_ranks);
  __shared__ int32_t s_blocks[513], s_tiles[513];
  // per-source totals -> rank offsets in receive order
  if (threadIdx.x <= num_ranks) {
    // rank_off[r] = sum over sources < r of all their routes to this rank
    int run = 0;
    for (int r = 0; r < (int)threadIdx.x; ++r)
      for (int e = 0; e < e_local; ++e) run += recv_count[r * e_local + e];
    pv.rank_off[threadIdx.x] = run;
    if ((int)threadIdx.x == num_ranks) pv.hdr->total_recv = run;
  }
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) {
    int tot = 0;
    for (int r = 0; r < num_ranks; ++r) tot += recv_count[r * e_local + e];
    pv.expert_total[e] = tot;
    s_blocks[e] = (tot + block_m - 1) / block_m;
    s_tiles[e] = emit_tiles(nullptr, e, 0, tot, block_m, cap, pair != 0, 0, false);
    if (stats != nullptr) stats[e] += tot;      // cumulative per-expert receive statistics (dispatch.py:644-650)
  }
  __shared__ int32_t s_boff[514], s_toff[514];
  block_exclusive_scan(s_blocks, s_boff, e_local);
  block_exclusive_scan(s_tiles, s_toff, e_local);
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) {
    pv.expert_block_off[e] = s_boff[e];
    pv.expert_tile_off[e] = s_toff[e];
  }
  if (threadIdx.x == 0) {
    const int rt = s_toff[e_local];
    pv.hdr->num_routed_tiles = rt;
    pv.hdr->num_pool_blocks = s_boff[e_local];
    pv.hdr->block_m = block_m;
    pv.hdr->num_tokens = m;
    // shared-expert tiles: the call's own tokens in blocks of block_m (chunk numbering of backend/staging.py:85-95)
    int ns = 0;
    if (has_shared) ns = emit_shared_tiles(pv.tiles + rt, m, block_m, cap, pair != 0);
    pv.hdr->num_shared_tiles = ns;
  }
  __syncthreads();
  // per-source cumulative offsets over experts in receive order (one thread per source rank)
  if ((int)threadIdx.x < num_ranks) {
    const int r = threadIdx.x;
    int run = pv.rank_off[r];
    for (int e = 0; e < e_local; ++e) {
      pv.seg_recv_start[e * num_ranks + r] = run;
      run += recv_count[r * e_local + e];
    }
  }
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) {
    int run = pv.expert_block_off[e] * block_m;
    for (int r = 0; r < num_ranks; ++r) {
      pv.seg_pool_start[e * num_ranks + r] = run;
      run += recv_count[r * e_local + e];
    }
    emit_tiles(pv.tiles + pv.expert_tile_off[e], e, pv.expert_block_off[e] * block_m, pv.expert_total[e], block_m, cap,
               pair != 0, pv.expert_block_off[e], true);
  }
}

// Decode path at EP1 (one chunk of at most 128 tokens): route ordering and pool plan in ONE single-block launch
// instead of four, because at a handful of tokens the layer is bound by launch latency.  Same results as
// sort_local/scan/place + plan_kernel (tested against them).
// Placement arguments of route_plan_small_kernel (pool_x == nullptr: the placement kernel follows as its own launch)
struct SmallPlace {
  const uint4* src_x;
  const int32_t* src_sf;
  const float* src_w;
  uint4* pool_x;
  int32_t* pool_sf;
  float* pool_w;
  int32_t* pool_dst;
  int64_t pool_sf_rows;
  int h;
};

__global__ void __launch_bounds__(1024) route_plan_small_kernel(
    const int64_t* __restrict__ topk_idx, int32_t* __restrict__ route_pos, int32_t* __restrict__ sorted_route,
    int32_t* __restrict__ send_count, int32_t* __restrict__ send_offset, int32_t* __restrict__ recv_count,
    char* __restrict__ plan_base, int32_t* __restrict__ stats, int32_t* __restrict__ status, int m, int k,
    int num_experts, int block_m, int cap, int pair, int has_shared, SmallPlace place) {
  chain_begin();
  extern __shared__ int32_t sm[];
  int32_t* ids = sm;                              // [m*k]
  int32_t* hist = sm + kSortChunkTokens * k;      // [E]
  int32_t* off = hist + num_experts;              // [E+1]  send offsets
  int32_t* boff = off + num_experts + 1;          // [E+1]  pool block offsets
  int32_t* toff = boff + num_experts + 1;         // [E+1]  tile offsets
  PlanView pv = plan_view(plan_base, num_experts, 1);
  const int n = m * k;
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int64_t id = topk_idx[i];
    if (id >= num_experts) { report_bad_index(status); id = -1; }
    ids[i] = id < 0 ? -1 : static_cast<int32_t>(id);
  }
  __syncthreads();
  int32_t* rank = toff + num_experts + 1;         // [m*k]
  if (threadIdx.x < 32) warp_rank_routes(ids, n, hist, rank);
  __syncthreads();
  int32_t* blocks = rank + kSortChunkTokens * k;  // [E] scratch of the scans
  int32_t* tiles_n = blocks + num_experts;        // [E]
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int tot = hist[e];
    blocks[e] = (tot + block_m - 1) / block_m;
    tiles_n[e] = emit_tiles(nullptr, e, 0, tot, block_m, cap, pair != 0, 0, false);
  }
  block_exclusive_scan(hist, off, num_experts);
  block_exclusive_scan(blocks, boff, num_experts);
  block_exclusive_scan(tiles_n, toff, num_experts);
  if (threadIdx.x == 0) {
    const int to = toff[num_experts];
    pv.hdr->num_routed_tiles = to;
    pv.hdr->num_pool_blocks = boff[num_experts];
    pv.hdr->total_recv = off[num_experts];
    pv.hdr->block_m = block_m;
    pv.hdr->num_tokens = m;
    pv.hdr->num_shared_tiles = has_shared ? emit_shared_tiles(pv.tiles + to, m, block_m, cap, pair != 0) : 0;
    pv.rank_off[0] = 0;
    pv.rank_off[1] = off[num_experts];
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = threadIdx.x + u * blockDim.x;
    if (i < n) {
      int pos = -1;
      if (rank[i] >= 0) {
        pos = off[ids[i]] + rank[i];
        sorted_route[pos] = i;
      }
      route_pos[i] = pos;
    }
  }
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int tot = hist[e];
    send_count[e] = tot;
    recv_count[e] = tot;
    send_offset[e] = off[e];
    pv.expert_total[e] = tot;
    pv.expert_block_off[e] = boff[e];
    pv.expert_tile_off[e] = toff[e];
    pv.seg_pool_start[e] = boff[e] * block_m;
    pv.seg_recv_start[e] = off[e];
    if (stats != nullptr) stats[e] += tot;
    emit_tiles(pv.tiles + toff[e], e, boff[e] * block_m, tot, block_m, cap, pair != 0, boff[e], true);
  }
  if (threadIdx.x == 0) {
    send_offset[num_experts] = off[num_experts];
    pv.expert_block_off[num_experts] = boff[num_experts];
    pv.expert_tile_off[num_experts] = toff[num_experts];
  }
  // A handful of routes: this block also places them (one warp per route), which saves the placement launch.  Route i
  // of expert e with rank r among the expert's routes is pool row boff[e] * block_m + r, row r - j * step of the
  // expert's tile j (the cut emit_tiles makes).
  if (place.pool_x != nullptr) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int vec = place.h / 16, words = place.h / kTileK;
    for (int i = warp; i < n; i += warps) {
      if (rank[i] < 0) continue;
      const int e = ids[i], r = rank[i];
      int parts, step;
      tile_cut(hist[e], cap, pair != 0, &parts, &step);
      const int j = r / step;
      const int p = boff[e] * block_m + r;
      const int64_t src_row = i / k;
      const uint4* src = place.src_x + src_row * vec;
      uint4* dst = place.pool_x + (int64_t)p * vec;
      for (int v0 = lane; v0 < vec; v0 += 128) {
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + 32 * u < vec) q[u] = src[v0 + 32 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + 32 * u < vec) dst[v0 + 32 * u] = q[u];
      }
      const int pos = (boff[e] * chunks_per_block(block_m) + j) * kChunkRows + chunk_pos(r - j * step);
      for (int wd = lane; wd < words; wd += 32)
        place.pool_sf[(int64_t)wd * place.pool_sf_rows + pos] = place.src_sf[src_row * words + wd];
      if (lane == 0) {
        place.pool_w[p] = place.src_w[i];
        place.pool_dst[p] = off[e] + r;
      }
    }
  }
}

// Place: one warp per pool row of every routed tile: copy the FP8 row, scatter its scale words into the chunk layout,
// record the top-k weight and the receive-order row that takes the expert output.  A block takes 32 rows of a tile at a
// time (a tile has at most 4 such slices), so the grid stays busy whatever the number of tiles, and every lane keeps
// four 16-byte loads in flight.
__global__ void __launch_bounds__(256) place_kernel(
    char* __restrict__ plan_base, const uint4* __restrict__ src_x, const int32_t* __restrict__ src_sf,
    const float* __restrict__ src_w, const int32_t* __restrict__ sorted_route, uint4* __restrict__ pool_x,
    int32_t* __restrict__ pool_sf, float* __restrict__ pool_w, int32_t* __restrict__ pool_dst, int64_t pool_sf_rows,
    int e_local, int num_ranks, int h, int k, int direct) {
  chain_begin();
  PlanView pv = plan_view(plan_base, e_local, num_ranks);
  const int ntiles = pv.hdr->num_routed_tiles;
  const int block_m = pv.hdr->block_m;
  const int vec = h / 16, words = h / kTileK;
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  constexpr int kSlices = (kTokenMajorTileRows + 31) / 32;
  for (int task = blockIdx.x; task < ntiles * kSlices; task += gridDim.x) {
    const int slice = task / ntiles, t = task - slice * ntiles;   // slice-major: the first slices are the populated ones
    const Tile tile = pv.tiles[t];
    const int i_end = min(tile.n_valid, 32 * slice + 32);
    if (32 * slice >= i_end) continue;
    const int e = tile.expert;
    const int expert_row0 = pv.expert_block_off[e] * block_m;
    for (int i = 32 * slice + warp_in_block; i < i_end; i += warps) {
      const int p = tile.row0 + i;
      const int j = p - expert_row0;           // index of this row among the expert's routes
      int r = 0, acc = 0;
      for (; r < num_ranks - 1; ++r) {          // source rank that owns the j-th route
        const int next = pv.seg_pool_start[e * num_ranks + r + 1] - expert_row0;
        if (j < next) break;
      }
      acc = pv.seg_pool_start[e * num_ranks + r] - expert_row0;
      const int recv_row = pv.seg_recv_start[e * num_ranks + r] + (j - acc);
      int64_t src_row = recv_row;
      float w;
      if (direct) {                              // EP1: read the staged inputs in place
        const int route = sorted_route[recv_row];
        src_row = route / k;
        w = src_w[route];
      } else {
        w = src_w[recv_row];
      }
      const uint4* src = src_x + src_row * vec;
      uint4* dst = pool_x + (int64_t)p * vec;
      for (int v0 = lane; v0 < vec; v0 += 128) {
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + 32 * u < vec) q[u] = src[v0 + 32 * u];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + 32 * u < vec) dst[v0 + 32 * u] = q[u];
      }
      const int pos = tile.sf_chunk * kChunkRows + chunk_pos(tile.sf_col * 32 + i);
      for (int wd = lane; wd < words; wd += 32) pool_sf[(int64_t)wd * pool_sf_rows + pos] = src_sf[src_row * words + wd];
      if (lane == 0) {
        pool_w[p] = w;
        pool_dst[p] = recv_row;
      }
    }
  }
}

// EP1, M <= 128: fused route ordering + plan; up to 128 routes the same block also places them, beyond that the
// placement kernel follows
cudaError_t launch_route_plan_place_small(const Ctx& c, int m, int block_m, int32_t* stats, cudaStream_t s) {
  const int k = c.geo.num_topk, e = c.geo.num_experts;
  const size_t smem = (size_t)(2 * kSortChunkTokens * k + 6 * e + 3) * sizeof(int32_t);
  const bool place_here = m * k <= 128;
  SmallPlace place = {};
  if (place_here)
    place = SmallPlace{c.at<uint4>(c.lay.x), c.at<int32_t>(c.lay.x_sf), c.at<float>(c.lay.topk_weights),
                       c.at<uint4>(c.lay.pool_x), c.at<int32_t>(c.lay.pool_sf), c.at<float>(c.lay.pool_w),
                       c.at<int32_t>(c.lay.pool_dst), c.lay.pool_sf_rows, c.geo.hidden};
  launch_chained(route_plan_small_kernel, dim3(1), dim3(1024), smem, s, c.at<int64_t>(c.lay.topk_idx),
                 c.at<int32_t>(c.lay.route_pos), c.at<int32_t>(c.lay.sorted_route), c.at<int32_t>(c.lay.send_count),
                 c.at<int32_t>(c.lay.send_offset), c.at<int32_t>(c.lay.recv_count), c.ws + c.lay.plan, stats,
                 c.at<int32_t>(c.lay.status), m, k, e, block_m, tile_cap(block_m, c.family),
                 c.family == kFamilyTokensAsAPair, c.geo.num_shared_experts > 0, place);
  if (!place_here)
    launch_chained(place_kernel, dim3(148 * 2), dim3(256), 0, s, c.ws + c.lay.plan, c.at<uint4>(c.lay.x),
                   c.at<int32_t>(c.lay.x_sf), c.at<float>(c.lay.topk_weights), c.at<int32_t>(c.lay.sorted_route),
                   c.at<uint4>(c.lay.pool_x), c.at<int32_t>(c.lay.pool_sf), c.at<float>(c.lay.pool_w),
                   c.at<int32_t>(c.lay.pool_dst), c.lay.pool_sf_rows, c.e_local, 1, c.geo.hidden, c.geo.num_topk, 1);
  return cudaGetLastError();
}

cudaError_t launch_shared_plan(const Ctx& c, int m, int block_m, cudaStream_t s) {
  launch_chained(shared_plan_kernel, dim3(1), dim3(32), 0, s, c.ws + c.lay.plan, c.e_local, c.geo.num_ranks, m, block_m,
                                      tile_cap(block_m, c.family), c.family == kFamilyTokensAsAPair, c.lay.max_tiles - shared_tile_capacity(c.geo.num_max_tokens));
  return cudaGetLastError();
}

cudaError_t launch_plan_place(const Ctx& c, int m, int block_m, int32_t* stats, cudaStream_t s) {
  const int R = c.geo.num_ranks;
  launch_chained(plan_kernel, dim3(1), dim3(1024), 0, s, c.ws + c.lay.plan, c.at<int32_t>(c.lay.recv_count), stats, c.e_local, R, block_m,
                                 tile_cap(block_m, c.family), c.family == kFamilyTokensAsAPair, m,
                                 c.geo.num_shared_experts > 0);
  const bool direct = R == 1;
  launch_chained(place_kernel, dim3(148 * 8), dim3(256), 0, s, c.ws + c.lay.plan, direct ? c.at<uint4>(c.lay.x) : c.at<uint4>(c.lay.recv_x),
      direct ? c.at<int32_t>(c.lay.x_sf) : c.at<int32_t>(c.lay.recv_sf),
      direct ? c.at<float>(c.lay.topk_weights) : c.at<float>(c.lay.recv_w), c.at<int32_t>(c.lay.sorted_route),
      c.at<uint4>(c.lay.pool_x), c.at<int32_t>(c.lay.pool_sf), c.at<float>(c.lay.pool_w), c.at<int32_t>(c.lay.pool_dst),
      c.lay.pool_sf_rows, c.e_local, R, c.geo.hidden, c.geo.num_topk, direct ? 1 : 0);
  return cudaGetLastError();
}

// =====================================================================================================================
// Combine: y[t] = bf16_rn(sum of the token's valid slots in ascending slot order, shared expert last), sequential FP32
// additions starting from zero (backend/kernel/combine.py:128-199).  One thread owns 8 consecutive output elements.
// =====================================================================================================================
__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
    acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
  }
}

__global__ void __launch_bounds__(256) combine_kernel(
    const uint4* __restrict__ rows, const int32_t* __restrict__ route_pos, const uint4* __restrict__ shared_out,
    const uint4* __restrict__ residual, uint4* __restrict__ y, int m, int h, int k) {
  chain_begin();
  const int vec = h / 8;
  const int64_t total = (int64_t)m * vec;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / vec;
    const int v = static_cast<int>(i % vec);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < k; ++s) {
      const int pos = route_pos[t * k + s];
      if (pos >= 0) add_bf16x8(acc, rows[(int64_t)pos * vec + v]);
    }
    if (shared_out != nullptr) add_bf16x8(acc, shared_out[i]);
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    if (residual != nullptr) {
      // what the serving engine's separate BF16 addition leaves: the layer output rounded to BF16 first, then the sum
      // of the two BF16 values rounded once more
      const uint4 res = residual[i];
      const __nv_bfloat162* r = reinterpret_cast<const __nv_bfloat162*>(&res);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(o[j]), b = __bfloat1622float2(r[j]);
        o[j] = __floats2bfloat162_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
      }
    }
    y[i] = out;
  }
}

cudaError_t launch_combine(const Ctx& c, void* y, const void* residual, int m, cudaStream_t s) {
  if (m == 0) return cudaSuccess;
  const int64_t total = (int64_t)m * c.geo.hidden / 8;
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  const uint4* rows = c.geo.num_ranks == 1 ? c.at<uint4>(c.lay.ret) : c.at<uint4>(c.lay.ret_recv);
  launch_chained(combine_kernel, dim3(blocks), dim3(256), 0, s, rows, c.at<int32_t>(c.lay.route_pos),
                                        c.geo.num_shared_experts > 0 ? c.at<uint4>(c.lay.shared_out) : nullptr,
                                        static_cast<const uint4*>(residual), static_cast<uint4*>(y), m, c.geo.hidden,
                                        c.geo.num_topk);
  return cudaGetLastError();
}

// =====================================================================================================================
// Scalar validation engine (tests only): the same plan, pool, epilogues and output addressing as the tensor-core
// kernels, with the two block-scaled GEMMs written as plain FP32 dot products.  One warp = one 32-channel scale group.
// =====================================================================================================================
template <bool kFp8Weights>
__device__ __forceinline__ float dot_group(const uint8_t* __restrict__ xrow, const uint8_t* __restrict__ wrow) {
  // 32 K elements: xrow -> 32 e4m3 bytes; wrow -> 16 packed bytes (FP4) or 32 e4m3 bytes
  float acc = 0.f;
  if (kFp8Weights) {
#pragma unroll 8
    for (int j = 0; j < 32; ++j) acc = fmaf(e4m3_to_float(xrow[j]), e4m3_to_float(wrow[j]), acc);
  } else {
#pragma unroll 8
    for (int j = 0; j < 16; ++j) {
      const uint32_t b = wrow[j];
      acc = fmaf(e4m3_to_float(xrow[2 * j]), e2m1_to_float(b & 15u), acc);
      acc = fmaf(e4m3_to_float(xrow[2 * j + 1]), e2m1_to_float(b >> 4), acc);
    }
  }
  return acc;
}

// scale byte of weight row `row` (within its matrix of n_rows rows), K group g, in the 4x32-transposed MN-major layout
__device__ __forceinline__ uint32_t weight_sf_byte(const int32_t* __restrict__ sf, int n_rows, int row, int g) {
  const int blk = row / 128, in = row % 128;
  const int pos = blk * 128 + chunk_pos(in);
  const uint32_t word = static_cast<uint32_t>(sf[(int64_t)(g / 4) * n_rows + pos]);
  return (word >> (8 * (g % 4))) & 0xFFu;
}

__device__ __forceinline__ uint32_t token_sf_byte(const int32_t* __restrict__ sf, int64_t sf_rows, const Tile& tile,
                                                  int i, int g) {
  const int pos = tile.sf_chunk * kChunkRows + chunk_pos(tile.sf_col * 32 + i);
  const uint32_t word = static_cast<uint32_t>(sf[(int64_t)(g / 4) * sf_rows + pos]);
  return (word >> (8 * (g % 4))) & 0xFFu;
}

// address of weight row `row` (0..rows_per_expert) of expert e, for plain and two-slice weight tensors
__device__ __forceinline__ const uint8_t* weight_row_ptr(const uint8_t* base, int e, int row, int rows_per_expert,
                                                         int64_t row_bytes, int64_t slice_stride) {
  if (slice_stride > 0) {
    const int half = rows_per_expert / 2;
    return base + (row / half) * slice_stride + ((int64_t)e * half + row % half) * row_bytes;
  }
  return base + ((int64_t)e * rows_per_expert + row) * row_bytes;
}

__global__ void __launch_bounds__(128) simt_l1_kernel(
    char* __restrict__ plan_base, int e_local, int num_ranks, int first_tile, int num_tiles_from_hdr_shared,
    const uint8_t* __restrict__ tok_x, const int32_t* __restrict__ tok_sf, int64_t tok_sf_rows,
    const float* __restrict__ tok_w, const uint8_t* __restrict__ w13, const int32_t* __restrict__ w13_sf,
    uint8_t* __restrict__ act_x, uint8_t* __restrict__ act_sf, int64_t act_sf_rows, int h, int inter, float clamp,
    int fast_math, int fp8_weights, int64_t slice_stride) {
  PlanView pv = plan_view(plan_base, e_local, num_ranks);
  const int ntiles = num_tiles_from_hdr_shared ? pv.hdr->num_shared_tiles : pv.hdr->num_routed_tiles;
  const int base = num_tiles_from_hdr_shared ? pv.hdr->num_routed_tiles : 0;
  const int groups = inter / 32;
  const int lane = threadIdx.x & 31;
  const int64_t work = (int64_t)ntiles * groups;
  const int64_t wstride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t wi = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wi < work; wi += wstride) {
    const Tile tile = pv.tiles[base + wi / groups];
    const int g_out = static_cast<int>(wi % groups);
    const int c = g_out * 32 + lane;
    const bool shared = tile.expert == kSharedExpert;
    const int e = shared ? 0 : tile.expert;
    const int64_t wrow_bytes = fp8_weights ? h : h / 2;
    // stored W13 rows: [g0..7, u0..7, g8..15, u8..15, ...]
    const int row_g = 16 * (c / 8) + (c % 8), row_u = row_g + 8;
    const uint8_t* wg = weight_row_ptr(w13, e, row_g, 2 * inter, wrow_bytes, slice_stride);
    const uint8_t* wu = weight_row_ptr(w13, e, row_u, 2 * inter, wrow_bytes, slice_stride);
    const int32_t* wsf = w13_sf + (int64_t)e * (h / 128) * 2 * inter;
    for (int i = 0; i < tile.n_valid; ++i) {
      const uint8_t* xr = tok_x + (int64_t)(tile.row0 + i) * h;
      float accg = 0.f, accu = 0.f;
      for (int g = 0; g < h / 32; ++g) {
        const float sx = ue8m0_to_float(token_sf_byte(tok_sf, tok_sf_rows, tile, i, g));
        const float sg = ue8m0_to_float(weight_sf_byte(wsf, 2 * inter, row_g, g));
        const float su = ue8m0_to_float(weight_sf_byte(wsf, 2 * inter, row_u, g));
        float dg, du;
        if (fp8_weights) {
          dg = dot_group<true>(xr + g * 32, wg + g * 32);
          du = dot_group<true>(xr + g * 32, wu + g * 32);
        } else {
          dg = dot_group<false>(xr + g * 32, wg + g * 16);
          du = dot_group<false>(xr + g * 32, wu + g * 16);
        }
        accg = fmaf(dg, sx * sg, accg);
        accu = fmaf(du, sx * su, accu);
      }
      const float wt = shared ? 1.0f : tok_w[tile.row0 + i];
      const float act = swiglu_act(accg, accu, wt, clamp, fast_math != 0);
      const float amax = warp_max_nonneg(fabsf(act));
      const int sf_exp = ue8m0_exp_of_amax(amax);
      act_x[(int64_t)(tile.row0 + i) * inter + c] = float_to_e4m3(__fmul_rn(act, ue8m0_inv(sf_exp)));
      if (lane == 0) {
        const int pos = tile.sf_chunk * kChunkRows + chunk_pos(tile.sf_col * 32 + i);
        act_sf[((int64_t)(g_out / 4) * act_sf_rows + pos) * 4 + (g_out % 4)] = static_cast<uint8_t>(sf_exp);
      }
    }
  }
}

__global__ void __launch_bounds__(128) simt_l2_kernel(
    char* __restrict__ plan_base, int e_local, int num_ranks, int use_shared_tiles,
    const uint8_t* __restrict__ act_x, const int32_t* __restrict__ act_sf, int64_t act_sf_rows,
    const uint8_t* __restrict__ w2, const int32_t* __restrict__ w2_sf, const int32_t* __restrict__ pool_dst,
    __nv_bfloat16* __restrict__ out, int h, int inter, int fp8_weights, int64_t slice_stride) {
  PlanView pv = plan_view(plan_base, e_local, num_ranks);
  const int ntiles = use_shared_tiles ? pv.hdr->num_shared_tiles : pv.hdr->num_routed_tiles;
  const int base = use_shared_tiles ? pv.hdr->num_routed_tiles : 0;
  const int groups = h / 32;
  const int lane = threadIdx.x & 31;
  const int64_t work = (int64_t)ntiles * groups;
  const int64_t wstride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t wi = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wi < work; wi += wstride) {
    const Tile tile = pv.tiles[base + wi / groups];
    const int row = static_cast<int>(wi % groups) * 32 + lane;   // output feature
    const bool shared = tile.expert == kSharedExpert;
    const int e = shared ? 0 : tile.expert;
    const int64_t wrow_bytes = fp8_weights ? inter : inter / 2;
    const uint8_t* wr = weight_row_ptr(w2, e, row, h, wrow_bytes, slice_stride);
    const int32_t* wsf = w2_sf + (int64_t)e * (inter / 128) * h;
    for (int i = 0; i < tile.n_valid; ++i) {
      const uint8_t* xr = act_x + (int64_t)(tile.row0 + i) * inter;
      float acc = 0.f;
      for (int g = 0; g < inter / 32; ++g) {
        const float sx = ue8m0_to_float(token_sf_byte(act_sf, act_sf_rows, tile, i, g));
        const float sw = ue8m0_to_float(weight_sf_byte(wsf, h, row, g));
        const float d = fp8_weights ? dot_group<true>(xr + g * 32, wr + g * 32) : dot_group<false>(xr + g * 32, wr + g * 16);
        acc = fmaf(d, sx * sw, acc);
      }
      const int64_t dst = shared ? (tile.row0 + i) : pool_dst[tile.row0 + i];
      out[dst * h + row] = __float2bfloat16_rn(acc);
    }
  }
}

cudaError_t launch_experts_simt(const Ctx& c, const MmoeWeights& w, const MmoeOptions& o, int m, int block_m,
                                cudaStream_t s) {
  const int h = c.geo.hidden, inter = c.geo.intermediate;
  const int blocks = 148 * 8;
  char* plan = c.ws + c.lay.plan;
  simt_l1_kernel<<<blocks, 128, 0, s>>>(plan, c.e_local, c.geo.num_ranks, 0, 0, c.at<uint8_t>(c.lay.pool_x),
                                        c.at<int32_t>(c.lay.pool_sf), c.lay.pool_sf_rows, c.at<float>(c.lay.pool_w),
                                        static_cast<const uint8_t*>(w.w13), static_cast<const int32_t*>(w.w13_sf),
                                        c.at<uint8_t>(c.lay.act_x), c.at<uint8_t>(c.lay.act_sf), c.lay.pool_sf_rows, h,
                                        inter, o.activation_clamp, o.fast_math, 0, w.w13_slice_stride);
  simt_l2_kernel<<<blocks, 128, 0, s>>>(plan, c.e_local, c.geo.num_ranks, 0, c.at<uint8_t>(c.lay.act_x),
                                        c.at<int32_t>(c.lay.act_sf), c.lay.pool_sf_rows,
                                        static_cast<const uint8_t*>(w.w2), static_cast<const int32_t*>(w.w2_sf),
                                        c.at<int32_t>(c.lay.pool_dst), c.at<__nv_bfloat16>(c.lay.ret), h, inter, 0,
                                        w.w2_slice_stride);
  if (c.geo.num_shared_experts > 0 && m > 0) {
    simt_l1_kernel<<<blocks, 128, 0, s>>>(plan, c.e_local, c.geo.num_ranks, 0, 1, c.at<uint8_t>(c.lay.x),
                                          c.at<int32_t>(c.lay.shared_x_sf), c.lay.shared_sf_rows, nullptr,
                                          static_cast<const uint8_t*>(w.shared_w13),
                                          static_cast<const int32_t*>(w.shared_w13_sf),
                                          c.at<uint8_t>(c.lay.shared_act_x), c.at<uint8_t>(c.lay.shared_act_sf),
                                          c.lay.shared_sf_rows, h, inter, o.activation_clamp, o.fast_math, 1, 0);
    simt_l2_kernel<<<blocks, 128, 0, s>>>(plan, c.e_local, c.geo.num_ranks, 1, c.at<uint8_t>(c.lay.shared_act_x),
                                          c.at<int32_t>(c.lay.shared_act_sf), c.lay.shared_sf_rows,
                                          static_cast<const uint8_t*>(w.shared_w2),
                                          static_cast<const int32_t*>(w.shared_w2_sf), nullptr,
                                          c.at<__nv_bfloat16>(c.lay.shared_out), h, inter, 1, 0);
  }
  return cudaGetLastError();
}

}  // namespace mmoe
