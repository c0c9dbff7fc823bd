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
//   * outputs leave as 16-byte stores: 32 E4M3 bytes per scale group (layer 1), 384 contiguous BF16 bytes per task
//     (layer 2) -- also when the row goes straight into the source rank's buffer over NVLink (kFused).
//
//   warp 0     tile producer: per 128-K stage one TMA box of token rows and one of weight rows (packed FP4 expands to
//              byte containers on the way into shared memory; no cluster multicast)
//   warp 6     scale producer: per stage one 512-byte chunk of token scales and one or two of weight scales
//   warp 1     MMA issuer: tcgen05.cp of the scale chunks into TMEM, 4 UMMAs, commit of the stage and of the accumulator
//   warps 2-5  epilogue
//
// The same roles exist in the reference's kernel (backend/kernel/tma_warps.py, mma_warp.py, epilogue.py).  Persistent
// CTAs (one per SM) walk the static task list tile-major, so that the CTAs working at the same time share a token tile
// and the tiles of one expert share its weights in L2.  Every wait is bounded (see Waiter).
#include <cuda_fp8.h>

#include "mmoe_tc.cuh"

namespace mmoe {

namespace {

constexpr int kTmThreads = 224;
constexpr int kTmN = 192;                          // weight rows of a full task (UMMA N)
constexpr int kTmRows = 128;                       // token rows of a tile (UMMA M)
constexpr int kTmABytes = kTmRows * kTileK;        // 16 KB
constexpr int kTmBBytes = kTmN * kTileK;           // 24 KB of byte containers
constexpr int kTmSfBytes = 512 + 2 * 512;          // token scale chunk, two weight scale chunks
constexpr int kTmStageBytes = kTmABytes + kTmBBytes + kTmSfBytes;
constexpr int kTmStages = (kSmemBudget - 1024) / kTmStageBytes;
constexpr int kTmSmemBytes = 1024 + kTmStages * kTmStageBytes + 1024;   // control block + stages + alignment slack
constexpr int kTmAccCols = kTmN;                   // TMEM columns of one accumulator
constexpr int kTmSfaCol = 2 * kTmAccCols;          // 4 columns: scales of the 128 token rows
constexpr int kTmSfbCol = kTmSfaCol + 8;           // 8 columns: scales of up to 256 weight rows
static_assert(kTmStages >= 4 && kTmStages <= 8, "pipeline depth");
static_assert(kTmSfbCol + 8 <= (int)kTmemCols, "TMEM budget");
static_assert(kTmSmemBytes <= 227 * 1024, "shared memory budget");

struct TmControl {        // lives at the start of shared memory
  uint64_t full[8];       // producers -> MMA warp: the stage's copies have landed (one arrival per producer)
  uint64_t empty[8];      // MMA -> producers: the stage's shared memory may be overwritten
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  // layer 2 with the write-back fused in: slot s < 32 is `ret_recv` of source rank s
  __nv_bfloat16* out_base[32];
  int32_t rank_off[33];   // first receive-order row of each source rank
  int32_t home_base[32];  // send position on that rank of the first row it sent here
};
static_assert(sizeof(TmControl) <= 1024, "control block");

// A task's slice of the expert's stored weight rows.  The rows of an expert are handled as two halves (the two slices
// of the `localize()` form, or simply the two halves of a plain tensor); a half is cut into blocks of 192 rows, the last
// one possibly shorter (a multiple of 64).  A short block loads the 192 rows that END at its last row, so that every
// box lies inside the half, and skips the leading rows through the operand descriptor.
struct TmBlock {
  int part, r0, n_cols, shift;   // half, first stored row (within the expert), rows used, rows skipped at the box start
};
__device__ __forceinline__ TmBlock tm_block(int nb, int half, int blocks_per_half) {
  TmBlock b;
  b.part = nb / blocks_per_half;
  const int r_part = (nb - b.part * blocks_per_half) * kTmN;
  b.n_cols = min(kTmN, half - r_part);
  b.shift = kTmN - b.n_cols;
  b.r0 = b.part * half + r_part;
  return b;
}

template <int kLayer, bool kFused>
__global__ void __launch_bounds__(kTmThreads, 1) tm_kernel(const __grid_constant__ TmParams p) {
  static_assert(!kFused || kLayer == 2, "only GEMM2 writes rows back");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  TmControl* ctl = reinterpret_cast<TmControl*>(smem);
  uint8_t* a_base = smem + 1024;
  uint8_t* b_base = a_base + kTmStages * kTmABytes;
  uint8_t* sf_base = b_base + kTmStages * kTmBBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  PlanView pv = plan_view(const_cast<char*>(p.plan), p.e_local, p.num_ranks);
  const Tile* tiles = pv.tiles + (p.tile_select == 2 ? p.early_shared_first : 0);
  const int num_tiles = p.tile_select == 2
                            ? (p.has_shared_weights ? max(0, min(pv.hdr->num_early_shared_tiles, p.early_shared_cap)) : 0)
                            : pv.hdr->num_routed_tiles + (p.tile_select == 0 && p.has_shared_weights ? pv.hdr->num_shared_tiles : 0);
  const int half = p.rows_per_expert / 2;
  const int blocks_per_half = (half + kTmN - 1) / kTmN;
  const int n_blocks = 2 * blocks_per_half;
  const int64_t num_tasks = (int64_t)num_tiles * n_blocks;
  const int k_stages = p.k_dim / kTileK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kTmStages; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 2);           // the two producers
      mbar_init(smem_u32(&ctl->empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[i]), 128);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
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
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  Waiter waiter{&ctl->abort_flag, p.status, global_timer() + static_cast<uint64_t>(p.timeout_ns), 20 + kLayer, warp};
  const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);

  if (warp == 0) {
    // --------------------------------------------------------------------------------------------- tile producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      const uint32_t a0 = smem_u32(a_base), b0 = smem_u32(b_base);
      bool ok = true;
      Tile tile = blockIdx.x < num_tasks ? tiles[blockIdx.x / n_blocks] : Tile{};
      for (int64_t task = blockIdx.x; task < num_tasks && ok; task += gridDim.x) {
        const int tile_idx = static_cast<int>(task / n_blocks);
        const int nb = static_cast<int>(task - (int64_t)tile_idx * n_blocks);
        // the next task's tile record is requested now and consumed at the bottom of the loop: its latency hides behind
        // this task instead of stalling the first stage of the next one
        Tile next_tile = tile;
        if (task + gridDim.x < num_tasks) next_tile = tiles[(task + gridDim.x) / n_blocks];
        const bool shared = tile.expert == kSharedExpert;
        const int e = shared ? 0 : tile.expert;
        const TmBlock blk = tm_block(nb, half, blocks_per_half);
        const bool sliced = !shared && p.routed_sliced != 0;
        const int box_row = blk.r0 - blk.part * half - blk.shift;          // inside the half: half >= 192
        const int row = sliced ? e * half + box_row : e * p.rows_per_expert + blk.part * half + box_row;
        const int slice = sliced ? blk.part : 0;
        const CUtensorMap* wmap = shared ? &p.map_w_shared : &p.map_w_routed;
        const int box_sel = tile.n_valid <= 64 ? 0 : 1;
        const CUtensorMap* tmap = shared ? &p.map_tok_shared[box_sel] : &p.map_tok_routed[box_sel];
        // packed FP4 counts its global bytes
        const uint32_t tx = (box_sel ? kTmRows : 64) * kTileK + (shared ? kTmN * kTileK : kTmN * kTileK / 2);
        int k0 = 0;
        for (int kb = 0; kb < k_stages; ++kb, k0 += kTileK) {
          if (!waiter.wait(empty0 + 8 * stage, phase ^ 1u)) { ok = false; break; }
          const uint32_t bar = full0 + 8 * stage;
          mbar_expect_tx(bar, tx);
          tma_load_3d(b0 + stage * kTmBBytes, wmap, k0, row, slice, bar);
          tma_load_2d(a0 + stage * kTmABytes, tmap, k0, tile.row0, bar);
          if (++stage == kTmStages) { stage = 0; phase ^= 1u; }
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
      Tile tile = blockIdx.x < num_tasks ? tiles[blockIdx.x / n_blocks] : Tile{};
      for (int64_t task = blockIdx.x; task < num_tasks && ok; task += gridDim.x) {
        const int tile_idx = static_cast<int>(task / n_blocks);
        const int nb = static_cast<int>(task - (int64_t)tile_idx * n_blocks);
        // the next task's tile record is requested now and consumed at the bottom of the loop: its latency hides behind
        // this task instead of stalling the first stage of the next one
        Tile next_tile = tile;
        if (task + gridDim.x < num_tasks) next_tile = tiles[(task + gridDim.x) / n_blocks];
        const bool shared = tile.expert == kSharedExpert;
        const int e = shared ? 0 : tile.expert;
        const TmBlock blk = tm_block(nb, half, blocks_per_half);
        const uint32_t sfb_bytes = (blk.r0 % kChunkRows) + blk.n_cols > kChunkRows ? 1024u : 512u;
        const int32_t* wsf = (shared ? p.wsf_shared : p.wsf_routed) + (int64_t)e * k_stages * p.rows_per_expert +
                             (blk.r0 / kChunkRows) * kChunkRows;
        const int64_t tsf_rows = shared ? p.tsf_rows_shared : p.tsf_rows_routed;
        const int32_t* tsf = (shared ? p.tsf_shared : p.tsf_routed) + (int64_t)tile.sf_chunk * kChunkRows;
        for (int kb = 0; kb < k_stages; ++kb, wsf += p.rows_per_expert, tsf += tsf_rows) {
          if (!waiter.wait(empty0 + 8 * stage, phase ^ 1u)) { ok = false; break; }
          const uint32_t bar = full0 + 8 * stage;
          const uint32_t dst = sf0 + stage * kTmSfBytes;
          mbar_expect_tx(bar, 512u + sfb_bytes);
          bulk_load(dst + 512, wsf, sfb_bytes, bar);
          bulk_load(dst, tsf, 512, bar);
          if (++stage == kTmStages) { stage = 0; phase ^= 1u; }
        }
        tile = next_tile;
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop so that its state stays warp-uniform; one elected lane issues.
    uint32_t stage = 0, phase = 0, it = 0;
    bool ok = true;
    const uint64_t sw128_hi = desc_hi_sw128();
    const uint64_t sf_hi = desc_hi_sf(128);
    const uint32_t a_lo0 = (smem_u32(a_base) & 0x3FFFFu) >> 4;
    const uint32_t b_lo0 = (smem_u32(b_base) & 0x3FFFFu) >> 4;
    const uint32_t sf_lo0 = (smem_u32(sf_base) & 0x3FFFFu) >> 4;
    Tile tile = blockIdx.x < num_tasks ? tiles[blockIdx.x / n_blocks] : Tile{};
    for (int64_t task = blockIdx.x; task < num_tasks && ok; task += gridDim.x, ++it) {
      const int tile_idx = static_cast<int>(task / n_blocks);
      const int nb = static_cast<int>(task - (int64_t)tile_idx * n_blocks);
      Tile next_tile = tile;
      if (task + gridDim.x < num_tasks) next_tile = tiles[(task + gridDim.x) / n_blocks];
      const bool shared = tile.expert == kSharedExpert;
      const TmBlock blk = tm_block(nb, half, blocks_per_half);
      const uint32_t acc_stage = it & 1u, acc_phase = (it >> 1) & 1u;
      if (!waiter.wait_warp(smem_u32(&ctl->tmem_empty[acc_stage]), acc_phase ^ 1u)) { ok = false; break; }
      tc_fence_after();
      const uint32_t idesc0 = make_idesc(0u, shared ? 0u : 5u, static_cast<uint32_t>(blk.n_cols), 0);
      const uint32_t d = tmem_base + acc_stage * kTmAccCols;
      const uint32_t sfa = tmem_base + kTmSfaCol + tile.sf_col;
      const uint32_t sfb_tm = tmem_base + kTmSfbCol;
      const uint32_t sfb = sfb_tm + (blk.r0 % kChunkRows) / 32;
      const bool two_chunks = (blk.r0 % kChunkRows) + blk.n_cols > kChunkRows;
      const uint32_t b_skip = static_cast<uint32_t>(blk.shift * kTileK) >> 4;   // whole 8-row swizzle groups
      for (int kb = 0; kb < k_stages; ++kb) {
        if (!waiter.wait_warp(full0 + 8 * stage, phase)) { ok = false; break; }
        if (elect_one()) {
          const uint32_t a_lo = a_lo0 + stage * (kTmABytes >> 4);
          const uint32_t b_lo = b_lo0 + stage * (kTmBBytes >> 4) + b_skip;
          const uint32_t sf_lo = sf_lo0 + stage * (kTmSfBytes >> 4);
          tc_cp_sf(tmem_base + kTmSfaCol, sf_hi | sf_lo);
          tc_cp_sf(sfb_tm, sf_hi | (sf_lo + 32));
          if (two_chunks) tc_cp_sf(sfb_tm + 4, sf_hi | (sf_lo + 64));
#pragma unroll
          for (int k = 0; k < kTileK / 32; ++k)
            tc_mma(d, sw128_hi | (a_lo + 2 * k), sw128_hi | (b_lo + 2 * k),
                   idesc0 + k * ((1u << 4) | (1u << 29)),                   // scale byte k of both operands
                   sfa, sfb, (kb | k) != 0 ? 1u : 0u);
          tc_commit(empty0 + 8 * stage);              // shared memory of this stage is free once these MMAs retire
        }
        __syncwarp();
        if (++stage == kTmStages) { stage = 0; phase ^= 1u; }
      }
      if (ok && elect_one()) tc_commit(smem_u32(&ctl->tmem_full[acc_stage]));
      __syncwarp();
      tile = next_tile;
    }
  } else {
    // --------------------------------------------------------------------------------------------- epilogue
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    const int i = q * 32 + lane;                  // token row of the tile this thread owns
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    uint32_t it = 0;
    bool ok = true;
    Tile tile = blockIdx.x < num_tasks ? tiles[blockIdx.x / n_blocks] : Tile{};
    for (int64_t task = blockIdx.x; task < num_tasks && ok; task += gridDim.x, ++it) {
      const int tile_idx = static_cast<int>(task / n_blocks);
      const int nb = static_cast<int>(task - (int64_t)tile_idx * n_blocks);
      Tile next_tile = tile;
      if (task + gridDim.x < num_tasks) next_tile = tiles[(task + gridDim.x) / n_blocks];
      const bool shared = tile.expert == kSharedExpert;
      const TmBlock blk = tm_block(nb, half, blocks_per_half);
      const uint32_t acc_stage = it & 1u, acc_phase = (it >> 1) & 1u;
      const bool live = i < tile.n_valid;
      const int64_t row = (int64_t)tile.row0 + i;
      // per-token side data, fetched before the accumulator is awaited
      float wt = 1.0f;
      __nv_bfloat16* out_row = nullptr;
      if (kLayer == 1) {
        if (!shared && live) wt = __ldg(p.pool_w + row);
      } else if (live) {
        if (shared) {
          out_row = p.shared_out + row * p.hidden;
        } else if (!kFused) {
          out_row = p.ret + (int64_t)__ldg(p.pool_dst + row) * p.hidden;
        } else {
          const int r = __ldg(p.pool_dst + row);          // receive-order row -> source rank and its send position
          int sr = 0;
          while (sr + 1 < p.num_ranks && r >= ctl->rank_off[sr + 1]) ++sr;
          out_row = ctl->out_base[sr] + (int64_t)(ctl->home_base[sr] + r - ctl->rank_off[sr]) * p.hidden;
        }
      }
      if (!waiter.wait_warp(smem_u32(&ctl->tmem_full[acc_stage]), acc_phase)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d0 = tmem_base + lane_sel + acc_stage * kTmAccCols;
      if (kLayer == 1) {
        // 64 stored rows = 32 channels = one scale group: columns 16b + j hold the gate, 16b + 8 + j the up value of
        // channel 8b + j
        uint8_t* act = (shared ? p.act_shared : p.act_routed) + row * p.inter + (blk.r0 >> 1);
        uint8_t* act_sf = shared ? p.act_sf_shared : p.act_sf_routed;
        const int64_t sf_rows = shared ? p.act_sf_rows_shared : p.act_sf_rows_routed;
        const int64_t sf_pos = (int64_t)tile.sf_chunk * kChunkRows + chunk_pos(tile.sf_col * 32 + i);
        const int grp0 = blk.r0 >> 6;
#pragma unroll 1
        for (int g = 0; g < (blk.n_cols >> 6); ++g) {
          uint32_t v[64];
          tc_ld32(d0 + 64 * g, v);
          tc_ld32(d0 + 64 * g + 32, v + 32);
          tc_ld_wait();
          float a[32];
          uint32_t amax_bits = 0;
#pragma unroll
          for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float x = swiglu_act(__uint_as_float(v[16 * b + j]), __uint_as_float(v[16 * b + 8 + j]), wt, p.clamp,
                                         p.fast_math != 0);
              a[8 * b + j] = x;
              amax_bits = max(amax_bits, __float_as_uint(fabsf(x)));
            }
          const int sf_exp = ue8m0_exp_of_amax(__uint_as_float(amax_bits));
          const float inv = ue8m0_inv(sf_exp);
          uint32_t w[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[4 * c], inv), __fmul_rn(a[4 * c + 1], inv)),
                                                         __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[4 * c + 2], inv), __fmul_rn(a[4 * c + 3], inv)),
                                                         __NV_SATFINITE, __NV_E4M3);
            w[c] = lo | (hi << 16);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(act + 32 * g);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            const int grp = grp0 + g;                 // K group of layer 2: word grp / 4 of the chunk row, byte grp % 4
            act_sf[((int64_t)(grp >> 2) * sf_rows + sf_pos) * 4 + (grp & 3)] = static_cast<uint8_t>(sf_exp);
          }
        }
      } else {
        __nv_bfloat16* out = live ? out_row + blk.r0 : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < blk.n_cols; c0 += 32) {
          uint32_t v[32];
          tc_ld32(d0 + c0, v);
          tc_ld_wait();
          uint32_t w[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const __nv_bfloat162 pr = __floats2bfloat162_rn(__uint_as_float(v[2 * c]), __uint_as_float(v[2 * c + 1]));
            w[c] = *reinterpret_cast<const uint32_t*>(&pr);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(out + c0);
#pragma unroll
            for (int c = 0; c < 4; ++c) dst[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&ctl->tmem_empty[acc_stage]));
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
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

}  // namespace

cudaError_t tm_prepare() {
  cudaError_t e = cudaFuncSetAttribute(tm_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTmSmemBytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(tm_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTmSmemBytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(tm_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTmSmemBytes);
  return e;
}

cudaError_t tm_launch(int layer, bool fused, const TmParams& p, cudaStream_t s) {
  const int grid = tc_num_sms();
  if (grid <= 0) return cudaErrorNotReady;
  if (layer == 1) tm_kernel<1, false><<<grid, kTmThreads, kTmSmemBytes, s>>>(p);
  else if (fused) tm_kernel<2, true><<<grid, kTmThreads, kTmSmemBytes, s>>>(p);
  else tm_kernel<2, false><<<grid, kTmThreads, kTmSmemBytes, s>>>(p);
  return cudaGetLastError();
}

}  // namespace mmoe
