// Building blocks shared by the two tcgen05 grouped-GEMM kernel families (weights-as-A for small token counts,
// tokens-as-A for the tensor-bound shapes): inline-PTX wrappers for mbarriers, TMA / bulk copies and the tcgen05
// instructions, the bounded barrier wait, and the host-side tensor-map encoders.
#pragma once

#include <cuda.h>

#include "mmoe_common.cuh"

namespace mmoe {

constexpr int kSmemBudget = 227 * 1024 - 1024;   // the 227 KB a CTA may have, less the slack for aligning the base to 1024 bytes
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kWaitHintNs = 200000;         // upper bound of one hardware-suspended barrier wait (the loop around it re-arms)
constexpr uint32_t kOutSlotShift = 26;           // packed destination of a fused write-back row: slot << 26 | row

#ifdef __CUDACC__
// ---------------------------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint64_t global_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

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
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kWaitHintNs)     // the thread sleeps in hardware until the phase completes or the hint expires
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Tile loads: plain per-CTA TMA, never with cluster multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t tmem_addr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// 32 consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Instruction descriptor of the block-scaled MMA (M = 128): [4,6) B scale id, [7,10) A format, [10,13) B format
// (0 = E4M3, 5 = E2M1), [15]/[16] A/B major (0 = K), [17,23) N>>3, [23] scale format (1 = UE8M0), [24,29) M>>4,
// [29,31) A scale id.
__device__ __forceinline__ uint32_t make_idesc(uint32_t a_format, uint32_t b_format, uint32_t n, uint32_t sf_id) {
  return (sf_id << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) |
         (sf_id << 29);
}
// high words of the shared-memory matrix descriptors: K-major operand tile with 128-byte swizzle (8-row groups 1024
// bytes apart), and the un-swizzled scale chunk read by tcgen05.cp (8-row groups `group_bytes` apart)
__device__ __forceinline__ uint64_t desc_hi_sw128() {
  return (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_hi_sf(uint32_t group_bytes) {
  return (static_cast<uint64_t>(group_bytes >> 4) << 32) | (1ull << 46);
}

// A bounded barrier wait.  When the budget expires the CTA records {kernel, role, block} in the status words, raises
// its abort flag (every role of the CTA drains) and the kernel returns; nothing traps.
struct Waiter {
  volatile int32_t* abort_flag;
  int32_t* status;
  uint64_t deadline;
  int kernel_id, role;
  // whole-warp wait: one lane watches the barrier, the others sleep at the warp barrier (a polling warp would put 32
  // requests on the barrier unit per probe and slow the producer and MMA threads that share it)
  __device__ __forceinline__ bool wait_warp(uint32_t bar, uint32_t parity) {
    // common case: the phase has completed already -- one probe by the whole warp (one broadcast read) and a vote
    if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = wait(bar, parity);
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  }
  // true when the call is being abandoned: another role gave up, or this wait has used up the budget (recorded)
  __device__ __forceinline__ bool abandoned() {
    if (*abort_flag != 0) return true;
    if (global_timer() > deadline) {
      *abort_flag = 1;
      if (atomicCAS(&status[kStatusTimeout], 0, 1) == 0) {
        status[kStatusKernel] = kernel_id;
        status[kStatusRole] = role;
        status[kStatusBlock] = static_cast<int32_t>(blockIdx.x);
      }
      return true;
    }
    return false;
  }
  // true when the phase completed, false when the call is being abandoned
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity) {
    // one non-blocking probe first: a hardware-suspended wait wakes up late, and that latency lands on the critical
    // path of whichever role the pipeline is waiting for
    if (mbar_test_wait(bar, parity)) return true;
    for (uint32_t spin = 0;; ++spin) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((spin & 63u) == 63u && abandoned()) return false;
    }
  }
};
#endif  // __CUDACC__

// ---------------------------------------------------------------------------------------------------------------
// host side: tensor maps (implemented in mmoe_umma.cu)
// ---------------------------------------------------------------------------------------------------------------
// token rows: 2-D map [rows, K] of E4M3 bytes, box `box_rows` x 128 K
int make_token_map(CUtensorMap* map, const void* base, uint64_t k_elems, uint64_t rows, uint32_t box_rows);
// weights: 3-D map [slices, rows per slice, K] of packed E2M1 (expanded to byte containers on the way into shared
// memory) or E4M3, box `box_rows` x 128 K; a plain tensor is one slice
int make_weight_map(CUtensorMap* map, bool fp4, const void* base, uint64_t k_elems, uint64_t rows_total,
                    int64_t slice_stride, uint32_t box_rows);
int tc_num_sms();          // SM count of the device mmoe_prepare() ran on last (0 before)
bool tc_ready();

// parameters of one launch of the tokens-as-A kernels (mmoe_umma_tm.cu)
struct TmParams {
  CUtensorMap map_w_routed;        // box 192 rows x 128 K (96 rows for CTA pairs)
  CUtensorMap map_w_shared;
  CUtensorMap map_tok_routed[2];   // boxes of 64 / 128 token rows
  CUtensorMap map_tok_shared[2];
  const char* plan;
  const int32_t* wsf_routed;       // [E_l][K/128][rows_per_expert] scale words, 4x32 transposed per 128 rows
  const int32_t* wsf_shared;
  const int32_t* tsf_routed;       // token scale chunks: word w of chunk row r at w * tsf_rows + r
  const int32_t* tsf_shared;
  int64_t tsf_rows_routed, tsf_rows_shared;
  uint8_t* act_routed;             // layer-1 outputs
  uint8_t* act_shared;
  uint8_t* act_sf_routed;
  uint8_t* act_sf_shared;
  int64_t act_sf_rows_routed, act_sf_rows_shared;
  const float* pool_w;
  __nv_bfloat16* ret;              // layer-2 outputs
  __nv_bfloat16* shared_out;
  const int32_t* pool_dst;
  int tile_select;                 // 0: every tile of the plan, 1: routed tiles only, 2: the early shared tiles only
  int64_t early_shared_first;
  int early_shared_cap;
  int ep_me;                       // fused write-back (layer 2, EP > 1)
  const int32_t* ep_totals;
  __nv_bfloat16* ep_ret_recv[32];
  int32_t* status;
  int64_t timeout_ns;
  int e_local, num_ranks;
  int k_dim;                       // reduction length: H (layer 1) or I (layer 2)
  int rows_per_expert;             // 2I (layer 1) or H (layer 2)
  int routed_sliced;
  int hidden, inter;
  float clamp;
  int fast_math;
  int has_shared_weights;
};
cudaError_t tm_prepare();
cudaError_t tm_launch(int layer, bool fused, int ctas, const TmParams& p, cudaStream_t s);   // ctas: 1, or 2 for CTA pairs

}  // namespace mmoe
