// Grouped block-scaled GEMMs of the MegaMoE layer, tokens-as-A form, for the tensor-bound shapes (about a hundred
// tokens per expert and more, and the shared expert of any call past the decode sizes).
//
//   task  = (tile of <= 128 token rows, 192 consecutive STORED weight rows of the tile's expert)
//   UMMA  = tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale, M = 128 (token rows, E4M3), N = 192 (weight rows,
//           E2M1 routed / E4M3 shared), K = 32, FP32 accumulator of 128 lanes x 192 columns in TMEM, two accumulators
//
// Why this orientation.  One accumulator chain of N >= 160 runs the tensor pipe at its full rate (8192 MAC/clk/SM
// measured; N <= 128 is bounded by the 128 B/clk shared-memory read rate and by a 72-clk floor per instruction), so
// four instructions per 128-K stage keep the pipe busy for 384 clk and leave the one-thread issue loops slack.  A
// thread of the epilogue owns a TOKEN (TMEM lane) and sees all 192 weight rows of the task as consecutive columns:
//   * the stored W13 row order [g0..7, u0..7, g8..15, ...] (backend/weights.py:83-97 of the reference) puts the gate and
//     the up value of a channel 8 columns apart in the same thread -- no de-interleaving tensor map, no shuffles, and the
//     stored scale words (4x32 transposed per 128 stored rows) are already what tcgen05.cp wants: nothing is permuted;
//   * the amax of 32 output channels is a reduction inside one thread;
//   * outputs leave in rows: 32 E4M3 bytes per scale group as two 16-byte stores (layer 1); layer 2 passes a block of
//     32 rows x 64 columns through a swizzled staging area so that 8 lanes write 128 contiguous bytes of one row -- also
//     when the row goes straight into the source rank's buffer over NVLink (kFused).
//
//   warp 0     tile producer: per 128-K stage one TMA box of token rows and one of weight rows (packed FP4 expands to
//              byte containers on the way into shared memory; no cluster multicast)
//   warp 6     scale producer: per stage one 512-byte chunk of token scales and one or two of weight scales
//   warp 7     scale copier: tcgen05.cp of the stage's chunks into that stage's own TMEM columns, then a commit that
//              arrives on the stage's `full` barrier
//   warp 1     MMA issuer: per stage one barrier probe, 4 UMMAs, one commit
//   warps 2-5  epilogue
//
// Every tcgen05 instruction costs its issuing thread about 50 clk, so the one thread that feeds the tensor pipe issues
// nothing but the UMMAs and the commit (measured: with the three scale copies and a whole-warp barrier probe in the
// same loop a stage took 510 clk of issue against 384 clk of tensor work).  The scale columns are per pipeline stage
// (12 of the 128 TMEM columns the two accumulators leave free), so the copier runs ahead of the issuer like the
// producers do.
//
// CTA pairs (kCtas = 2, `tcgen05.mma.cta_group::2`, M = 256): two token tiles of the same expert share one task.  Each
// CTA stages its own token tile and HALF of the task's weight rows (96), the pair's tensor cores read both halves; the
// leader CTA's threads issue the scale copies and the UMMAs for both.  Both kernel families are bound by shared-memory
// bandwidth (about 146 B/clk for TMA fills and operand reads together, measured on both): a single CTA moves 20 KB per
// UMMA slot of 96 clk; a pair was meant to move 14 KB per CTA, but the peer's half of the weight rows is still read out
// of the peer's shared memory (about 17 KB per SM), and the pair's issuing thread pays two commits per stage.  Measured,
// pairs are no faster than single CTAs at any token density, so the automatic choice never takes them (orientation 3
// selects them).  No load uses cluster multicast: every CTA fetches its own boxes, completion crosses the pair as plain
// mbarrier arrivals.
//
// The same roles exist in the reference's kernel (backend/kernel/tma_warps.py, mma_warp.py, epilogue.py).  Persistent
// CTAs (one per SM) walk the static task list tile-major, so that the CTAs working at the same time share a token tile
// and the tiles of one expert share its weights in L2.  Every wait is bounded (see Waiter).
#include <cuda_fp8.h>

#include "mmoe_tc.cuh"

namespace mmoe {

namespace {

constexpr int kTmThreads = 256;
constexpr int kTmN = 192;                          // weight rows of a full task (UMMA N)
constexpr int kTmRows = 128;                       // token rows of a tile (UMMA M per CTA)
constexpr int kTmSfColsPerStage = 12;              // 4: scales of the 128 token rows, 8: scales of up to 256 weight rows

template <int kCtas>
struct TmShape {
  static constexpr int kBoxN = kTmN / kCtas;                // weight rows one CTA stages
  static constexpr int kABytes = kTmRows * kTileK;          // 16 KB
  static constexpr int kBBytes = kBoxN * kTileK;            // 24 KB / 12 KB of byte containers
  static constexpr int kSfBytes = 512 + 2 * 512;            // token scale chunk, two weight scale chunks
  static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;
  static constexpr int kStagesRaw = (kSmemBudget - 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kStagingBytes = 4 * 32 * 128;        // layer 2: one 32-row x 128-byte output block per epilogue warp
  static constexpr int kMainBytes = 1024 + kStages * kStageBytes;          // control block + stages
  // + staging (layer 2 only: layer 1 leaves the rest of the SM's shared memory to the small kernels that run beside the
  // shared expert's GEMM1 on the second stream) + alignment slack
  static constexpr int smem_bytes(int layer) { return kMainBytes + (layer == 2 ? kStagingBytes : 0) + 1024; }
  static constexpr int kSmemBytes = kMainBytes + kStagingBytes + 1024;
  static constexpr int kAccCols = kTmN;                     // TMEM columns of one accumulator
  static constexpr int kSfCol = 2 * kAccCols;               // scale columns of stage s: [kSfCol + 12 s, + 12)
  static_assert(kStages >= 4, "pipeline depth");
  static_assert(kSfCol + kStages * kTmSfColsPerStage <= (int)kTmemCols, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct TmControl {        // lives at the start of shared memory (same layout in both CTAs of a pair)
  uint64_t tile_full[8];  // tile producer -> scale copier / relay: this CTA's boxes of the stage have landed
  uint64_t sf_full[8];    // scale producer -> scale copier / relay: this CTA's scale chunks have landed
  uint64_t pair_ready[8]; // leader only: the peer CTA's boxes and chunks of the stage have landed
  uint64_t mma_ready[8];  // leader only: scale copier -> MMA issuer: everything of the stage is in place in both CTAs
  uint64_t empty[8];      // MMA issuer -> producers (of both CTAs): the stage may be overwritten
  uint64_t tmem_full[2];  // MMA issuer -> epilogue (of both CTAs)
  uint64_t tmem_empty[2]; // leader only: epilogue warps (of both CTAs) -> MMA issuer
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  // layer 2 with the write-back fused in: slot s < 32 is `ret_recv` of source rank s
  __nv_bfloat16* out_base[32];
  int32_t rank_off[33];   // first receive-order row of each source rank
  int32_t home_base[32];  // send position on that rank of the first row it sent here
};
static_assert(sizeof(TmControl) <= 1024, "control block");

// ---------------------------------------------------------------------------------------------------------------
// cluster / CTA-pair helpers
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <int kCtas>
__device__ __forceinline__ void tm_commit(uint32_t bar) {
  if (kCtas == 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  else asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int kCtas>
__device__ __forceinline__ void tm_cp_sf(uint32_t tmem_addr, uint64_t sdesc) {
  if (kCtas == 1) asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
  else asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
}
template <int kCtas>
__device__ __forceinline__ void tm_mma(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                       uint32_t accumulate) {
  if (kCtas == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

// A task's slice of the expert's stored weight rows.  The rows of an expert are handled as two halves (the two slices
// of the `localize()` form, or simply the two halves of a plain tensor); a half is cut into blocks of 192 rows, the last
// one possibly shorter (a multiple of 64).  A CTA stages `n_cols / kCtas` of the block's rows; when that is fewer than
// its box holds, it loads the box that ENDS at its last row, so that every box lies inside the half, and skips the
// leading rows through the operand descriptor.
struct TmBlock {
  int part, r0, n_cols;   // half, first stored row (within the expert), rows used
};
__device__ __forceinline__ TmBlock tm_block(int nb, int half, int blocks_per_half) {
  TmBlock b;
  b.part = nb / blocks_per_half;
  const int r_part = (nb - b.part * blocks_per_half) * kTmN;
  b.n_cols = min(kTmN, half - r_part);
  b.r0 = b.part * half + r_part;
  return b;
}

// Layer-1 epilogue of one scale group: 64 accumulator columns = 32 channels (columns 16b + j hold the gate, 16b + 8 + j
// the up value of channel 8b + j) -> SwiGLU, x top-k weight, amax, UE8M0 exponent, 32 E4M3 bytes.  The fast-math choice
// is a template parameter: a per-element branch would serialise the 32 independent dependency chains.
template <bool kFast>
__device__ __forceinline__ int tm_l1_group(const uint32_t (&v)[64], float wt, float clamp, uint32_t (&w)[8]) {
  float a[32];
  uint32_t amax_bits = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x = swiglu_act_t<kFast>(__uint_as_float(v[16 * b + j]), __uint_as_float(v[16 * b + 8 + j]), wt, clamp);
      a[8 * b + j] = x;
      amax_bits = max(amax_bits, __float_as_uint(fabsf(x)));
    }
  const int sf_exp = ue8m0_exp_of_amax(__uint_as_float(amax_bits));
  const float inv = ue8m0_inv(sf_exp);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[4 * c], inv), __fmul_rn(a[4 * c + 1], inv)),
                                                 __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[4 * c + 2], inv), __fmul_rn(a[4 * c + 3], inv)),
                                                 __NV_SATFINITE, __NV_E4M3);
    w[c] = lo | (hi << 16);
  }
  return sf_exp;
}

template <int kLayer, bool kFused, int kCtas>
__global__ void __launch_bounds__(kTmThreads, 1) tm_kernel(const __grid_constant__ TmParams p) {
  static_assert(!kFused || kLayer == 2, "only GEMM2 writes rows back");
  using S = TmShape<kCtas>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);   // the same offset in both CTAs of a pair
  TmControl* ctl = reinterpret_cast<TmControl*>(smem);
  uint8_t* a_base = smem + 1024;
  uint8_t* b_base = a_base + S::kStages * S::kABytes;
  uint8_t* sf_base = b_base + S::kStages * S::kBBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = kCtas == 2 ? cluster_ctarank() : 0u;      // 0 = leader
  const bool leader = cta == 0;
  const int unit = blockIdx.x / kCtas, num_units = gridDim.x / kCtas;   // a unit = one CTA or one CTA pair
  chain_release();

  if (threadIdx.x == 0) {
    for (int i = 0; i < S::kStages; ++i) {
      mbar_init(smem_u32(&ctl->tile_full[i]), 1);
      mbar_init(smem_u32(&ctl->sf_full[i]), 1);
      mbar_init(smem_u32(&ctl->pair_ready[i]), 1);
      mbar_init(smem_u32(&ctl->mma_ready[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[i]), 4 * kCtas);        // one arrival per epilogue warp of the unit
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {       // the same warp of both CTAs of a pair allocates
    if (kCtas == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  // Everything above touches only this CTA's own shared and tensor memory, so it may run while the kernel before this
  // one in the stream is still running; everything below reads what that kernel wrote.
  chain_wait();
  if (kFused) {
    const int t = threadIdx.x - 32;
    if (t >= 0 && t < p.num_ranks) {
      ctl->out_base[t] = p.ep_ret_recv[t];
      int b = 0;
      for (int d = 0; d < p.ep_me; ++d) b += p.ep_totals[t * 32 + d];
      ctl->home_base[t] = b;
    }
    if (threadIdx.x == 64) {
      int run = 0;
      for (int sr = 0; sr < p.num_ranks; ++sr) { ctl->rank_off[sr] = run; run += p.ep_totals[sr * 32 + p.ep_me]; }
      ctl->rank_off[p.num_ranks] = run;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (kCtas == 2) cluster_sync_all();       // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  PlanView pv = plan_view(const_cast<char*>(p.plan), p.e_local, p.num_ranks);
  const Tile* tiles = pv.tiles + (p.tile_select == 2 ? p.early_shared_first : 0);
  const int num_tiles = p.tile_select == 2
                            ? (p.has_shared_weights ? max(0, min(pv.hdr->num_early_shared_tiles, p.early_shared_cap)) : 0)
                            : pv.hdr->num_routed_tiles + (p.tile_select == 0 && p.has_shared_weights ? pv.hdr->num_shared_tiles : 0);
  const int half = p.rows_per_expert / 2;
  const int blocks_per_half = (half + kTmN - 1) / kTmN;
  const int n_blocks = 2 * blocks_per_half;
  // a pair plan holds an even number of tiles per expert: tiles 2j and 2j + 1 form pair j
  const int64_t num_tasks = (int64_t)(num_tiles / kCtas) * n_blocks;
  const int k_stages = p.k_dim / kTileK;
  // tile record of task `t` for this CTA
  auto tile_of = [&](int64_t t) -> Tile { return tiles[(t / n_blocks) * kCtas + cta]; };

  Waiter waiter{&ctl->abort_flag, p.status, global_timer() + static_cast<uint64_t>(p.timeout_ns), 20 + kLayer, warp};
  const uint32_t tile_full0 = smem_u32(&ctl->tile_full[0]), sf_full0 = smem_u32(&ctl->sf_full[0]);
  const uint32_t pair_ready0 = smem_u32(&ctl->pair_ready[0]), mma_ready0 = smem_u32(&ctl->mma_ready[0]);
  const uint32_t empty0 = smem_u32(&ctl->empty[0]);

  // Every role walks the same task list; a one-thread role is a loop that runs at instruction latency, so everything
  // that does not change inside a task is computed once per task.  The next task's tile record is requested at the top
  // of a task and consumed at the bottom: its latency hides behind the task instead of stalling the next one.
  if (warp == 0) {
    // --------------------------------------------------------------------------------------------- tile producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      const uint32_t a0 = smem_u32(a_base), b0 = smem_u32(b_base);
      bool ok = true;
      Tile tile = unit < num_tasks ? tile_of(unit) : Tile{};
      for (int64_t task = unit; task < num_tasks && ok; task += num_units) {
        const int nb = static_cast<int>(task % n_blocks);
        Tile next_tile = tile;
        if (task + num_units < num_tasks) next_tile = tile_of(task + num_units);
        const bool shared = tile.expert == kSharedExpert;
        const int e = shared ? 0 : tile.expert;
        const TmBlock blk = tm_block(nb, half, blocks_per_half);
        const bool sliced = !shared && p.routed_sliced != 0;
        // this CTA's rows of the block: [r0 + cta * n_cols / kCtas, + n_cols / kCtas), loaded by the box that ends there
        const int mine = blk.n_cols / kCtas;
        const int box_row = blk.r0 - blk.part * half + (int)cta * mine + mine - S::kBoxN;   // >= 0: half > 192 if short
        const int row = sliced ? e * half + box_row : e * p.rows_per_expert + blk.part * half + box_row;
        const int slice = sliced ? blk.part : 0;
        const CUtensorMap* wmap = shared ? &p.map_w_shared : &p.map_w_routed;
        const int box_sel = tile.n_valid <= 64 ? 0 : 1;
        const CUtensorMap* tmap = shared ? &p.map_tok_shared[box_sel] : &p.map_tok_routed[box_sel];
        // packed FP4 counts its global bytes
        const uint32_t tx = (box_sel ? kTmRows : 64) * kTileK + (shared ? S::kBoxN * kTileK : S::kBoxN * kTileK / 2);
        int k0 = 0;
        for (int kb = 0; kb < k_stages; ++kb, k0 += kTileK) {
          if (!waiter.wait(empty0 + 8 * stage, phase ^ 1u)) { ok = false; break; }
          const uint32_t bar = tile_full0 + 8 * stage;
          mbar_expect_tx(bar, tx);
          tma_load_3d(b0 + stage * S::kBBytes, wmap, k0, row, slice, bar);
          tma_load_2d(a0 + stage * S::kABytes, tmap, k0, tile.row0, bar);
          if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
        }
        tile = next_tile;
      }
    }
  } else if (warp == 6) {
    // --------------------------------------------------------------------------------------------- scale producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      const uint32_t sf0 = smem_u32(sf_base);
      bool ok = true;
      Tile tile = unit < num_tasks ? tile_of(unit) : Tile{};
      for (int64_t task = unit; task < num_tasks && ok; task += num_units) {
        const int nb = static_cast<int>(task % n_blocks);
        Tile next_tile = tile;
        if (task + num_units < num_tasks) next_tile = tile_of(task + num_units);
        const bool shared = tile.expert == kSharedExpert;
        const int e = shared ? 0 : tile.expert;
        const TmBlock blk = tm_block(nb, half, blocks_per_half);
        const uint32_t sfb_bytes = (blk.r0 % kChunkRows) + blk.n_cols > kChunkRows ? 1024u : 512u;
        const int32_t* wsf = (shared ? p.wsf_shared : p.wsf_routed) + (int64_t)e * k_stages * p.rows_per_expert +
                             (blk.r0 / kChunkRows) * kChunkRows;
        const int64_t tsf_rows = shared ? p.tsf_rows_shared : p.tsf_rows_routed;
        const int32_t* tsf = (shared ? p.tsf_shared : p.tsf_routed) + (int64_t)tile.sf_chunk * kChunkRows;
        for (int kb = 0; kb < k_stages; ++kb, wsf += p.rows_per_expert, tsf += tsf_rows) {
          // the stage's previous UMMAs have retired: its shared memory AND its scale columns in TMEM are free
          if (!waiter.wait(empty0 + 8 * stage, phase ^ 1u)) { ok = false; break; }
          const uint32_t bar = sf_full0 + 8 * stage;
          const uint32_t dst = sf0 + stage * S::kSfBytes;
          mbar_expect_tx(bar, 512u + sfb_bytes);
          bulk_load(dst + 512, wsf, sfb_bytes, bar);          // every CTA of a pair holds the scales of all the block's rows
          bulk_load(dst, tsf, 512, bar);
          if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
        }
        tile = next_tile;
      }
    }
  } else if (warp == 7) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      if (leader) {
        // ----------------------------------------------------------------------------------------- scale copier
        const uint64_t sf_hi = desc_hi_sf(128);
        const uint32_t sf_lo0 = (smem_u32(sf_base) & 0x3FFFFu) >> 4;
        for (int64_t task = unit; task < num_tasks && ok; task += num_units) {
          const int nb = static_cast<int>(task % n_blocks);
          const TmBlock blk = tm_block(nb, half, blocks_per_half);
          const bool two_chunks = (blk.r0 % kChunkRows) + blk.n_cols > kChunkRows;
          for (int kb = 0; kb < k_stages; ++kb) {
            if (!waiter.wait(sf_full0 + 8 * stage, phase)) { ok = false; break; }
            if (!waiter.wait(tile_full0 + 8 * stage, phase)) { ok = false; break; }
            if (kCtas == 2 && !waiter.wait(pair_ready0 + 8 * stage, phase)) { ok = false; break; }
            const uint32_t sf_lo = sf_lo0 + stage * (S::kSfBytes >> 4);
            const uint32_t col = tmem_base + S::kSfCol + stage * kTmSfColsPerStage;
            // cta_group::2: every CTA of the pair copies from its own shared memory into its own tensor memory
            tm_cp_sf<kCtas>(col, sf_hi | sf_lo);                                   // token scales
            tm_cp_sf<kCtas>(col + 4, sf_hi | (sf_lo + 32));                        // weight scales, first chunk
            if (two_chunks) tm_cp_sf<kCtas>(col + 8, sf_hi | (sf_lo + 64));
            tm_commit<kCtas>(mma_ready0 + 8 * stage);                              // arrives when the copies have completed
            if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
          }
        }
      } else {
        // ----------------------------------------------------------------------------------------- relay (peer CTA)
        // tells the leader that this CTA's boxes and scale chunks of the stage have landed
        const uint32_t remote0 = map_to_cta(pair_ready0, 0);
        for (int64_t task = unit; task < num_tasks && ok; task += num_units) {
          for (int kb = 0; kb < k_stages; ++kb) {
            if (!waiter.wait(sf_full0 + 8 * stage, phase)) { ok = false; break; }
            if (!waiter.wait(tile_full0 + 8 * stage, phase)) { ok = false; break; }
            mbar_arrive_cluster_relaxed(remote0 + 8 * stage);
            if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0 && leader) {
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      const uint64_t sw128_hi = desc_hi_sw128();
      const uint32_t a_lo0 = (smem_u32(a_base) & 0x3FFFFu) >> 4;
      const uint32_t b_lo0 = (smem_u32(b_base) & 0x3FFFFu) >> 4;
      const uint32_t peer_empty0 = kCtas == 2 ? map_to_cta(empty0, 1) : 0u;
      const uint32_t peer_tmem_full0 = kCtas == 2 ? map_to_cta(smem_u32(&ctl->tmem_full[0]), 1) : 0u;
      Tile tile = unit < num_tasks ? tile_of(unit) : Tile{};
      for (int64_t task = unit; task < num_tasks && ok; task += num_units, ++it) {
        const int nb = static_cast<int>(task % n_blocks);
        Tile next_tile = tile;
        if (task + num_units < num_tasks) next_tile = tile_of(task + num_units);
        const bool shared = tile.expert == kSharedExpert;
        const TmBlock blk = tm_block(nb, half, blocks_per_half);
        const uint32_t acc_stage = it & 1u, acc_phase = (it >> 1) & 1u;
        if (!waiter.wait(smem_u32(&ctl->tmem_empty[acc_stage]), acc_phase ^ 1u)) { ok = false; break; }
        tc_fence_after();
        // M = 128 per CTA (256 over a pair); idesc field [24,29) = M >> 4
        const uint32_t idesc0 = make_idesc(0u, shared ? 0u : 5u, static_cast<uint32_t>(blk.n_cols), 0) +
                                (kCtas == 2 ? ((128u >> 4) << 24) : 0u);
        const uint32_t d = tmem_base + acc_stage * S::kAccCols;
        const uint32_t sfa0 = tmem_base + S::kSfCol + tile.sf_col;
        const uint32_t sfb0 = tmem_base + S::kSfCol + 4 + (blk.r0 % kChunkRows) / 32;
        // rows skipped at the start of this CTA's box (whole 8-row swizzle groups); the same in both CTAs
        const uint32_t b_skip = static_cast<uint32_t>((S::kBoxN - blk.n_cols / kCtas) * kTileK) >> 4;
        for (int kb = 0; kb < k_stages; ++kb) {
          if (!waiter.wait(mma_ready0 + 8 * stage, phase)) { ok = false; break; }
          const uint32_t a_lo = a_lo0 + stage * (S::kABytes >> 4);
          const uint32_t b_lo = b_lo0 + stage * (S::kBBytes >> 4) + b_skip;
          const uint32_t sfa = sfa0 + stage * kTmSfColsPerStage, sfb = sfb0 + stage * kTmSfColsPerStage;
#pragma unroll
          for (int k = 0; k < kTileK / 32; ++k)
            tm_mma<kCtas>(d, sw128_hi | (a_lo + 2 * k), sw128_hi | (b_lo + 2 * k),
                          idesc0 + k * ((1u << 4) | (1u << 29)),            // scale byte k of both operands
                          sfa, sfb, (kb | k) != 0 ? 1u : 0u);
          // the stage is free in every CTA of the unit once these UMMAs retire
          tm_commit<kCtas>(empty0 + 8 * stage);
          if (kCtas == 2) tm_commit<kCtas>(peer_empty0 + 8 * stage);
          if (++stage == S::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          tm_commit<kCtas>(smem_u32(&ctl->tmem_full[acc_stage]));
          if (kCtas == 2) tm_commit<kCtas>(peer_tmem_full0 + 8 * acc_stage);
        }
        tile = next_tile;
      }
    }
  } else {
    // --------------------------------------------------------------------------------------------- epilogue
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    const int i = q * 32 + lane;                  // token row of the tile this thread owns
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t tmem_empty_leader0 = kCtas == 2 ? map_to_cta(smem_u32(&ctl->tmem_empty[0]), 0) : smem_u32(&ctl->tmem_empty[0]);
    uint32_t it = 0;
    bool ok = true;
    Tile tile = unit < num_tasks ? tile_of(unit) : Tile{};
    for (int64_t task = unit; task < num_tasks && ok; task += num_units, ++it) {
      const int nb = static_cast<int>(task % n_blocks);
      Tile next_tile = tile;
      if (task + num_units < num_tasks) next_tile = tile_of(task + num_units);
      const bool shared = tile.expert == kSharedExpert;
      const TmBlock blk = tm_block(nb, half, blocks_per_half);
      const uint32_t acc_stage = it & 1u, acc_phase = (it >> 1) & 1u;
      const bool live = i < tile.n_valid;
      const int64_t row = (int64_t)tile.row0 + i;
      // per-token side data, fetched before the accumulator is awaited
      float wt = 1.0f;
      __nv_bfloat16* out = nullptr;
      if (kLayer == 1) {
        if (!shared && live) wt = __ldg(p.pool_w + row);
      } else if (live) {
        if (shared) {
          out = p.shared_out + row * p.hidden;
        } else if (!kFused) {
          out = p.ret + (int64_t)__ldg(p.pool_dst + row) * p.hidden;
        } else {
          const int r = __ldg(p.pool_dst + row);          // receive-order row -> source rank and its send position
          int sr = 0;
          while (sr + 1 < p.num_ranks && r >= ctl->rank_off[sr + 1]) ++sr;
          out = ctl->out_base[sr] + (int64_t)(ctl->home_base[sr] + r - ctl->rank_off[sr]) * p.hidden;
        }
        out += blk.r0;
      }
      if (!waiter.wait_warp(smem_u32(&ctl->tmem_full[acc_stage]), acc_phase)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d0 = tmem_base + lane_sel + acc_stage * S::kAccCols;
      if (kLayer == 1) {
        uint8_t* act = (shared ? p.act_shared : p.act_routed) + row * p.inter + (blk.r0 >> 1);
        uint8_t* act_sf = shared ? p.act_sf_shared : p.act_sf_routed;
        const int64_t sf_rows = shared ? p.act_sf_rows_shared : p.act_sf_rows_routed;
        const int64_t sf_pos = (int64_t)tile.sf_chunk * kChunkRows + chunk_pos(tile.sf_col * 32 + i);
        const int grp0 = blk.r0 >> 6;
        const bool fast = p.fast_math != 0;
#pragma unroll 1
        for (int g = 0; g < (blk.n_cols >> 6); ++g) {
          uint32_t v[64], w[8];
          tc_ld32(d0 + 64 * g, v);
          tc_ld32(d0 + 64 * g + 32, v + 32);
          tc_ld_wait();
          const int sf_exp = fast ? tm_l1_group<true>(v, wt, p.clamp, w) : tm_l1_group<false>(v, wt, p.clamp, w);
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(act + 32 * g);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            const int grp = grp0 + g;                 // K group of layer 2: word grp / 4 of the chunk row, byte grp % 4
            act_sf[((int64_t)(grp >> 2) * sf_rows + sf_pos) * 4 + (grp & 3)] = static_cast<uint8_t>(sf_exp);
          }
        }
      } else {
        // Rows leave as 128-byte segments: the warp's 32 x 64 block of BF16 values goes through a swizzled staging block
        // in shared memory (16-byte chunk c of row r at chunk c ^ (r & 7): conflict-free both ways), then 8 lanes write
        // one row's 128 contiguous bytes -- four full lines per instruction instead of 32 scattered 16-byte pieces,
        // which is what matters when the destination is another rank's buffer across NVLink.
        uint8_t* stg = smem + S::kMainBytes + (warp - 2) * 4096;
        const int sub = lane >> 3, chunk = lane & 7;
        // destination of the four rows this lane helps to write in each of the eight steps (row 4j + sub)
        __nv_bfloat16* dst_row[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const unsigned long long ptr = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(out), 4 * j + sub);
          dst_row[j] = reinterpret_cast<__nv_bfloat16*>(ptr);       // null for rows past the tile's last token
        }
#pragma unroll 1
        for (int c0 = 0; c0 < blk.n_cols; c0 += 64) {
          uint32_t v[64];
          tc_ld32(d0 + c0, v);
          tc_ld32(d0 + c0 + 32, v + 32);
          tc_ld_wait();
          __syncwarp();                                   // the previous block has been read out
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(v[8 * c + 2 * t]), __uint_as_float(v[8 * c + 2 * t + 1]));
              w[t] = *reinterpret_cast<const uint32_t*>(&pr);
            }
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = 4 * j + sub;
            const uint4 val = *reinterpret_cast<const uint4*>(stg + r * 128 + ((chunk ^ (r & 7)) << 4));
            if (dst_row[j] != nullptr) *reinterpret_cast<uint4*>(dst_row[j] + c0 + chunk * 8) = val;
          }
        }
      }
      // the accumulator is drained: one arrival per warp on the leader's barrier
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kCtas == 2) mbar_arrive_cluster(tmem_empty_leader0 + 8 * acc_stage);
        else mbar_arrive(tmem_empty_leader0 + 8 * acc_stage);
      }
      tile = next_tile;
    }
  }

  // ---------------------------------------------------------------------------------------------------- teardown
  __syncwarp();
  if (ctl->abort_flag != 0) {
    // abandoned call: give copies that are still in flight time to land in this CTA's shared memory before it exits
    const uint64_t t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (kCtas == 2) cluster_sync_all();       // no CTA leaves while its peer may still arrive on its barriers
  tc_fence_after();
  if (warp == 1) {
    if (kCtas == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <int kLayer, bool kFused, int kCtas>
cudaError_t tm_launch_one(const TmParams& p, int grid, cudaStream_t s) {
  using S = TmShape<kCtas>;
  if (kCtas == 1) {
    return launch_chained(tm_kernel<kLayer, kFused, 1>, dim3(grid), dim3(kTmThreads), S::smem_bytes(kLayer), s, p);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid & ~1);
  cfg.blockDim = dim3(kTmThreads);
  cfg.dynamicSmemBytes = S::smem_bytes(kLayer);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, tm_kernel<kLayer, kFused, kCtas>, p);
}

template <int kCtas>
cudaError_t tm_prepare_ctas() {
  using S = TmShape<kCtas>;
  cudaError_t e = cudaFuncSetAttribute(tm_kernel<1, false, kCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::smem_bytes(1));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(tm_kernel<2, false, kCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::smem_bytes(2));
  if (e == cudaSuccess) e = cudaFuncSetAttribute(tm_kernel<2, true, kCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::smem_bytes(2));
  return e;
}

}  // namespace

cudaError_t tm_prepare() {
  cudaError_t e = tm_prepare_ctas<1>();
  if (e == cudaSuccess) e = tm_prepare_ctas<2>();
  return e;
}

cudaError_t tm_launch(int layer, bool fused, int ctas, const TmParams& p, cudaStream_t s) {
  const int grid = tc_num_sms();
  if (grid <= 0) return cudaErrorNotReady;
  if (ctas == 2) {
    if (layer == 1) return tm_launch_one<1, false, 2>(p, grid, s);
    return fused ? tm_launch_one<2, true, 2>(p, grid, s) : tm_launch_one<2, false, 2>(p, grid, s);
  }
  if (layer == 1) return tm_launch_one<1, false, 1>(p, grid, s);
  return fused ? tm_launch_one<2, true, 1>(p, grid, s) : tm_launch_one<2, false, 1>(p, grid, s);
}

}  // namespace mmoe
