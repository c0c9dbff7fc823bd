// Shared definitions of the sm_100a MegaMoE kernels: plan tables, number-format helpers and the two epilogue
// functions (SwiGLU + requantisation, BF16 store) that both the tcgen05 kernels and the scalar validation kernels call.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/mmoe.h"

namespace mmoe {

constexpr int kGroupK = 32;        // K elements per UE8M0 scale
constexpr int kTileK = 128;        // K elements per pipeline stage = one packed scale word
constexpr int kTileRows = 128;     // weight rows per tile (UMMA M)
constexpr int kChunkRows = 128;    // token rows per scale-factor chunk (one 512-byte tcgen05.cp source per K stage)
constexpr int kMaxTileTokens = 112;  // largest UMMA N of one task
// Largest token tile of a BLOCK_M variant; an expert with more rows is cut into equal tiles.  BLOCK_M = 128 caps its
// tiles at 80 rows: the 10 KB token slot buys a fifth pipeline stage.  192 / 240 keep 112 (the tensor-bound
// expert-parallel shapes, where fewer and larger tiles matter more than pipeline depth).
__host__ __device__ inline int max_tile_rows(int block_m) { return block_m <= 64 ? block_m : (block_m == 128 ? 80 : kMaxTileTokens); }
// Kernel family of a launch, hence how its tile list is cut: weights-as-A kernels (tiles of at most max_tile_rows),
// tokens-as-A kernels (tiles of up to 128 rows whatever BLOCK_M is), tokens-as-A kernels on CTA pairs (an even number of
// tiles per expert: tiles 2j and 2j + 1 are the two halves of one pair task).
enum { kFamilyWeightsAsA = 0, kFamilyTokensAsA = 1, kFamilyTokensAsAPair = 2 };
constexpr int kTokenMajorTileRows = 128;
__host__ __device__ inline int tile_cap(int block_m, int family) { return family != kFamilyWeightsAsA ? kTokenMajorTileRows : max_tile_rows(block_m); }
// Scale-factor chunks (128 token rows each) reserved per pool block of a BLOCK_M variant: at least as many as the
// tiles an expert's rows are cut into (ceil(n / max_tile_rows) <= ceil(n / block_m) * chunks_per_block for every n).
__host__ __device__ inline int chunks_per_block(int block_m) { return block_m <= 64 ? 1 : (block_m <= 192 ? 2 : 3); }
constexpr int kSortChunkTokens = 128;
constexpr int kSharedExpert = -2;  // MmoeTile::expert of a shared-expert tile

// One unit of token rows handed to the grouped GEMMs: `n_valid` (<= 112) rows starting at `row0` of the token matrix
// (pool rows for routed experts, token indices for the shared expert), whose scales live in chunk `sf_chunk`
// starting at row `32 * sf_col` of that chunk.
struct Tile {
  int32_t expert;    // local expert index, or kSharedExpert
  int32_t row0;
  int32_t n_valid;
  int32_t sf_chunk;
  int32_t sf_col;    // 0 or 2: first 32-row group of the chunk this tile uses
  int32_t pad[3];
};
static_assert(sizeof(Tile) == 32, "tile record is 32 bytes");

struct PlanHeader {
  int32_t num_routed_tiles;
  int32_t num_shared_tiles;
  int32_t num_pool_blocks;     // sum over experts of ceil(n_e / BLOCK_M)
  int32_t total_recv;          // routes received by this rank
  int32_t block_m;
  int32_t num_tokens;
  int32_t num_early_shared_tiles;   // shared-expert tiles written ahead of the routed plan, at the tail of the tile table
  int32_t pad[9];
};
static_assert(sizeof(PlanHeader) == 64, "plan header is 64 bytes");

// Plan region: header | expert_total[E_l] | expert_block_off[E_l+1] | expert_tile_off[E_l+1] | rank_off[R+1] |
// seg_pool_start[E_l*R] | seg_recv_start[E_l*R] | tiles[max_tiles]
struct PlanView {
  PlanHeader* hdr;
  int32_t* expert_total;
  int32_t* expert_block_off;
  int32_t* expert_tile_off;
  int32_t* rank_off;
  int32_t* seg_pool_start;
  int32_t* seg_recv_start;
  Tile* tiles;
};

__host__ __device__ inline int64_t align_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// tile records reserved for the shared expert of a call with at most `max_tokens` tokens (they sit at the tail of the
// tile table when the shared expert is planned ahead of the routed experts)
__host__ __device__ inline int64_t shared_tile_capacity(int64_t max_tokens) { return (max_tokens / 16 + 2) * 2; }

__host__ __device__ inline int64_t plan_bytes(int e_local, int num_ranks, int64_t max_tiles) {
  int64_t ints = e_local + 2 * (e_local + 1) + (num_ranks + 1) + 2 * (int64_t)e_local * num_ranks;
  return 64 + align_up(ints * 4, 32) + max_tiles * (int64_t)sizeof(Tile);
}

__host__ __device__ inline PlanView plan_view(void* base, int e_local, int num_ranks) {
  PlanView v;
  char* p = static_cast<char*>(base);
  v.hdr = reinterpret_cast<PlanHeader*>(p);
  int32_t* q = reinterpret_cast<int32_t*>(p + 64);
  v.expert_total = q;            q += e_local;
  v.expert_block_off = q;        q += e_local + 1;
  v.expert_tile_off = q;         q += e_local + 1;
  v.rank_off = q;                q += num_ranks + 1;
  v.seg_pool_start = q;          q += (int64_t)e_local * num_ranks;
  v.seg_recv_start = q;          q += (int64_t)e_local * num_ranks;
  int64_t ints = q - reinterpret_cast<int32_t*>(p + 64);
  v.tiles = reinterpret_cast<Tile*>(p + 64 + align_up(ints * 4, 32));
  return v;
}

// Row of a 128-row scale chunk that holds token row i of the chunk: the layout `tcgen05.cp.32x128b.warpx4` expects
// (lane i%32 receives the four 32-row groups side by side).
__host__ __device__ inline int chunk_pos(int i) { return (i & 31) * 4 + ((i >> 5) & 3); }

// Device status words (int32[8]): [0] != 0 means a bounded wait expired; [1] kernel id, [2] role, [3] block,
// [4] bad-argument counter (e.g. an expert id out of range seen by the dispatch).
enum { kStatusTimeout = 0, kStatusKernel = 1, kStatusRole = 2, kStatusBlock = 3, kStatusBadIndex = 4 };

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------------------------
// number formats
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(__half(h));
}

__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6 with the sign in bit 3
  const uint32_t mag = nib & 7u;
  float v = mag < 4u ? 0.5f * mag : (mag == 4u ? 2.f : (mag == 5u ? 3.f : (mag == 6u ? 4.f : 6.f)));
  return (nib & 8u) ? -v : v;
}

__device__ __forceinline__ float ue8m0_to_float(uint32_t b) { return __uint_as_float(b << 23); }

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---------------------------------------------------------------------------------------------------------------
// L1 epilogue for one (token, channel): BF16 rounding of both accumulators, clamp (upper only for the gate),
// sigmoid, (gate*sig)*up*weight.  Operation order and roundings follow the reference's epilogue
// (backend/kernel/epilogue.py:190-221).
// ---------------------------------------------------------------------------------------------------------------
template <bool kFast>
__device__ __forceinline__ float swiglu_act_t(float gate_acc, float up_acc, float weight, float clamp) {
  float g = bf16_round(gate_acc);
  float u = bf16_round(up_acc);
  g = fminf(g, clamp);                       // clamp is a BF16-representable value (or +inf)
  u = fminf(fmaxf(u, -clamp), clamp);
  float gated;
  if (kFast) {
    float e, r;
    const float t = __fmul_rn(-g, 1.4426950408889634f);
    asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(t));
    const float d = __fadd_rn(1.0f, e);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    gated = __fmul_rn(g, r);
  } else {
    gated = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  }
  return __fmul_rn(__fmul_rn(gated, u), weight);
}
__device__ __forceinline__ float swiglu_act(float gate_acc, float up_acc, float weight, float clamp, bool fast_math) {
  return fast_math ? swiglu_act_t<true>(gate_acc, up_acc, weight, clamp) : swiglu_act_t<false>(gate_acc, up_acc, weight, clamp);
}

// UE8M0 exponent of a non-negative amax by the integer-carry method (backend/kernel/ptx_g.py:235-241).
__device__ __forceinline__ int ue8m0_exp_of_amax(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  const int rounded = static_cast<int>((bits + (0x7FFFFFu - (0x60u << 16))) >> 23);
  return max(rounded, 105 + 8) - 8;
}

__device__ __forceinline__ float ue8m0_inv(int sf_exp) { return __uint_as_float(static_cast<uint32_t>(254 - sf_exp) << 23); }

// max over the warp of non-negative floats (IEEE bits of non-negative floats order like unsigned integers)
__device__ __forceinline__ float warp_max_nonneg(float v) {
  return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
}

__device__ __forceinline__ void report_bad_index(int32_t* status) { atomicAdd(&status[kStatusBadIndex], 1); }
#endif  // __CUDACC__

// kernels and launchers implemented in the .cu files ------------------------------------------------------------------
struct Ctx {             // resolved pointers of one call
  MmoeGeometry geo;
  MmoeLayout lay;
  char* ws;
  int e_local;
  int kmax;              // min(k, E/R)
  const void* const* peer_ws = nullptr;   // set by the call that fuses the write-back into GEMM2 (EP > 1)
  int tile_select = 0;                    // 0: every tile of the plan, 1: routed tiles only, 2: the early shared tiles only
  int family = kFamilyWeightsAsA;         // kernel family the tiles this call plans / runs are cut for
  template <typename T> T* at(int64_t off) const { return reinterpret_cast<T*>(ws + off); }
};


// ---------------------------------------------------------------------------------------------------------------------
// Programmatic dependent launch.  The kernels of one call form a chain on a stream; each of them begins with
// chain_begin(): it lets the NEXT kernel of the stream be scheduled as soon as every block of this one has started
// (so that kernel's launch latency and set-up -- barrier initialisation, tensor-memory allocation -- overlap this
// kernel's run) and then waits until everything BEFORE this kernel in the stream has completed and its memory is
// visible.  A kernel must not touch global memory before chain_begin().  The wait is transitive: the next kernel's
// wait ends only when this grid has completed, and this grid completes only after its own wait has.  Both
// instructions do nothing in a kernel that was launched without the attribute below.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_begin() {
  chain_release();
  chain_wait();
}

// Chaining is used for calls of at most 128 tokens, where the launch gaps are a visible part of the call (measured at
// E=384: 56.7 -> 54.7 us at one token); past that the waiting blocks of the next kernel take room from the kernels
// that still run (1.574 -> 1.608 ms at 3840 tokens), so an entry point opens a ChainScope only for small calls and
// every launch outside a scope is an ordinary one.
struct ChainScope {
  explicit ChainScope(bool on);
  ~ChainScope();
  ChainScope(const ChainScope&) = delete;
  ChainScope& operator=(const ChainScope&) = delete;
 private:
  bool saved_;
};
// The next launch_chained() of this host thread launches without the attribute (used for the first kernel after a
// cross-stream event wait, where the kernel has more than one predecessor).
void break_chain();
bool take_chain_flag();   // true: launch with the attribute; resets the one-shot break

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = take_chain_flag() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

cudaError_t launch_stage(const Ctx& c, const void* hidden, const void* ids, int ids64, const float* w,
                         const uint8_t* pad, int m, int shared_bm, cudaStream_t s);
cudaError_t launch_route_stage(const Ctx& c, const void* hidden, const void* ids, int ids64, const float* w,
                               const float* logits, int num_logical, const int32_t* replica_count,
                               const int32_t* replica_slots, int max_copies, const uint8_t* pad, int m, int shared_bm,
                               cudaStream_t s);
cudaError_t launch_stage_nvfp4(const void* hidden, void* q_out, void* sf_out, float global_scale, int64_t num_tokens, int hidden_size,
                               cudaStream_t s);
cudaError_t launch_count_sort(const Ctx& c, int m, cudaStream_t s);
cudaError_t launch_pack(const Ctx& c, int m, cudaStream_t s);
cudaError_t launch_route_plan_place_small(const Ctx& c, int m, int block_m, int32_t* stats, cudaStream_t s);
cudaError_t launch_plan_place(const Ctx& c, int m, int block_m, int32_t* stats, cudaStream_t s);
cudaError_t launch_shared_plan(const Ctx& c, int m, int block_m, cudaStream_t s);
cudaError_t launch_combine(const Ctx& c, void* y, const void* residual, int m, cudaStream_t s);
cudaError_t launch_experts_simt(const Ctx& c, const MmoeWeights& w, const MmoeOptions& o, int m, int block_m, cudaStream_t s);
cudaError_t launch_experts_umma(const Ctx& c, const MmoeWeights& w, const MmoeOptions& o, int m, int block_m, cudaStream_t s);
int prepare_umma(const MmoeGeometry& geo);   // returns an MMOE_* code
bool tc_ready();                             // prepare_umma() has run on the current device
void set_tuning(int max_stages, int orientation);
int tuned_orientation();                     // 0: per call, 1: weights-as-A, 2: tokens-as-A, 3: tokens-as-A on CTA pairs
cudaError_t route_order_static(const int64_t* topk_idx, int m, int k, int num_experts, int32_t* send_count,
                               int32_t* send_offset, int32_t* route_pos, int32_t* sorted_route, cudaStream_t s);
int route_order_static_max_tokens();
int route_order_static_max_experts();
cudaError_t launch_interleave_rows(const void* src, void* dst, int groups, int rows, int row_bytes, cudaStream_t s);
cudaError_t launch_scale_layout(const int32_t* src, int32_t* dst, int groups, int rows, int row_stride, int kwords,
                                int interleave, cudaStream_t s);
int ep_sync_bytes();
int ep_totals_offset();                      // byte offset of the [32][32] route-total table inside the ep_sync region
cudaError_t launch_ep_signal_return(const Ctx& c, const void* const* peer_ws, int64_t timeout_ns, cudaStream_t s);
cudaError_t launch_ep_dispatch(const Ctx& c, const void* const* peer_ws, int m, int64_t timeout_ns, cudaStream_t s);
cudaError_t launch_ep_return(const Ctx& c, const void* const* peer_ws, int64_t timeout_ns, cudaStream_t s);

}  // namespace mmoe
