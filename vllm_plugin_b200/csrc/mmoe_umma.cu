// Grouped block-scaled GEMMs of the MegaMoE layer on the sm_100a tensor cores.
//
//   layer 1:  acc[ch, tok] = sum_k W13[e][ch, k] * x[tok, k]   (gate rows and up rows of one 128-channel tile in two
//             TMEM accumulators) -> SwiGLU, x top-k weight, per-32-channel UE8M0 requantisation to E4M3
//   layer 2:  acc[h, tok]  = sum_i W2[e][h, i] * act[tok, i]   -> BF16 rows of the return buffer
//
// Weights are the UMMA "A" operand (M = 128 rows), tokens the "B" operand (N = 16..112 tokens), so a small token
// count costs a small N instead of a padded M: `tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale`, MXFP4 (E2M1) or
// E4M3 weights x E4M3 activations with UE8M0 scales per 32 K.  The same roles exist in the reference's kernel
// (backend/kernel/tma_warps.py, mma_warp.py, epilogue.py, scheduler.py); the structure here is B200's:
//
//   warp 0     producer: one thread issues the TMA tile loads (packed FP4 expands to byte containers on the way into
//              shared memory; no cluster multicast) and 512-byte bulk copies of the scale chunks, per 128-K stage
//   warps 1,6  MMA: one warp per weight tile of the stage; an elected lane copies the scales into TMEM (tcgen05.cp) and
//              issues 4 UMMAs per stage, committing the stage's shared memory back to the producer and the finished
//              accumulator to the epilogue
//   warps 2-5  epilogue: TMEM -> registers (thread = weight row, columns = tokens), fused math, global stores
//
// Persistent CTAs (one per SM) walk a static task list (tile, 128-row weight block); TMEM accumulators are double
// buffered so the epilogue of task i overlaps the loads and MMAs of task i+1.  Every wait is bounded: when the budget
// expires the CTA records {kernel, role, block} in the status words, lets its in-flight copies land, frees its TMEM and
// returns; nothing traps.
//
// Expert parallelism: layer 2 has a second form (kFused) whose epilogue stores every BF16 row straight into the buffer
// of the rank the token came from (plain peer stores over NVLink, no TMA from or to peer memory), and `tile_select`
// restricts a launch to the routed tiles or to the shared expert's tiles planned ahead, so that the shared expert can
// run while the dispatch is still in flight on another stream.
#include <string.h>

#include <mutex>
#include <type_traits>

#include "mmoe_tc.cuh"

namespace mmoe {

namespace {

constexpr int kThreads = 224;   // producer, MMA 0, 4 epilogue warps, MMA 1

struct UmmaParams {
  CUtensorMap map_w_routed;    // FP4 weights, box 128 K x 256 rows (layer 1: the 5-D de-interleaving form)
  CUtensorMap map_w_shared;    // E4M3 weights of the shared expert
  const char* plan;
  const int32_t* wsf_routed;   // [E_l][K/128][rows_per_expert] scale words, 4x32 transposed per 128 rows
  const int32_t* wsf_shared;
  const int32_t* tsf_routed;   // token scale chunks: word w of chunk row r at w * tsf_rows + r
  const int32_t* tsf_shared;
  int64_t tsf_rows_routed, tsf_rows_shared;
  // layer-1 outputs
  uint8_t* act_routed;
  uint8_t* act_shared;
  uint8_t* act_sf_routed;      // byte view of the activation scale chunks
  uint8_t* act_sf_shared;
  int64_t act_sf_rows_routed, act_sf_rows_shared;
  const float* pool_w;
  // layer-2 outputs
  __nv_bfloat16* ret;
  __nv_bfloat16* shared_out;
  const int32_t* pool_dst;
  // layer 2 at EP > 1 with the write-back fused in: an output row goes straight into the `ret_recv` of the rank its
  // token came from (plain peer stores over NVLink), at that rank's send position
  int tile_select;             // 0: every tile of the plan, 1: routed tiles only, 2: the early shared tiles only
  int64_t early_shared_first;  // index of the first early shared tile in the tile table
  int early_shared_cap;        // tile records reserved there
  int fused_return;
  int ep_me;
  const int32_t* ep_totals;    // [32][32]: totals[s][d] = routes rank s sent to rank d in this call
  __nv_bfloat16* ep_ret_recv[32];
  int32_t* status;
  int64_t timeout_ns;
  int e_local, num_ranks;
  int k_dim;                   // reduction length: H (layer 1) or I (layer 2)
  int rows_per_expert;         // 2I (layer 1) or H (layer 2)
  int routed_sliced;           // 1: routed weights are [2, E_l, rows/2, K/2] (two slices), 0: [E_l, rows, K/2]
  int n_blocks;                // 128-row weight blocks per tile: I/128 (layer 1) or H/128 (layer 2)
  int hidden, inter;
  float clamp;
  int fast_math;
  int has_shared_weights;
  int num_stages;              // shared-memory pipeline depth in use (<= the compiled capacity)
  CUtensorMap map_tok_routed_box[5];   // token maps with boxes of 16 / 32 / 64 / 80 / 128 rows
  CUtensorMap map_tok_shared_box[5];
};

struct Control {          // lives at the start of shared memory
  uint64_t full[16];      // producer -> MMA warps: the stage's copies have landed
  uint64_t empty[16];     // MMA -> producer: the stage's shared memory may be overwritten
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile int32_t abort_flag;
  // layer 2 with the write-back fused in: where output rows go.  slot s < 32: `ret_recv` of source rank s, slot 32: the
  // shared expert's (local) output
  __nv_bfloat16* out_base[33];
  int32_t rank_off[33];   // fused write-back: first receive-order row of each source rank
  int32_t home_base[32];  // ... and the send position on that rank of the first row it sent here
};
static_assert(sizeof(Control) <= 1024, "control block");

// Every task multiplies TWO 128-row weight tiles with one token tile: layer 1 the gate rows and the up rows of 128
// channels, layer 2 two consecutive 128-row blocks of W2.  Two tiles per stage halve the per-byte cost of everything
// that is paid per stage (barrier hand-offs, token tile, token scales) and give the two MMA-issuing warps one
// accumulator each.
template <int kLayer, int kBoxRows>
struct Shape {
  static constexpr int kNCap = kBoxRows > kMaxTileTokens ? kMaxTileTokens : kBoxRows;   // accumulator columns per matrix (kBoxRows = largest tile)
  static constexpr int kABytes = 2 * kTileRows * kTileK;           // byte containers in shared memory
  static constexpr int kBBytes = kBoxRows * kTileK;
  // scale area of a stage: [weight scales of the two tiles, 2 x 512][token scales 512][layer 1: stored-order scales
  // 1024].  Layer 2 receives the two 512-byte chunks in tensor-memory order.  Layer 1 receives them in stored (gate/up
  // interleaved) order and the MMA warps rearrange them: into the first 1024 bytes from a separate landing area, or --
  // for the 32-token variant, where the saved KB is a sixth pipeline stage -- in place (measured: in place costs the
  // 4-stage 128-row variant 5 % of its GEMM1 time and buys the others nothing).
  static constexpr bool kSfInPlace = kLayer == 1 && kBoxRows == 32;
  static constexpr int kSfBytes = 3 * 512 + (kLayer == 1 && !kSfInPlace ? 1024 : 0);
  static constexpr int kStageBytes = kABytes + kBBytes + kSfBytes;
  static constexpr int kStagesRaw = (kSmemBudget - 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + 1024;   // control block + stages + alignment slack
  static constexpr int kAccCols = 2 * kNCap;                        // TMEM columns of one accumulator stage
  static constexpr int kSfCol = 2 * kAccCols;                       // scale region: A0, A1, token scales (one copy per MMA warp)
  static_assert(kSfCol + 16 <= (int)kTmemCols, "TMEM budget");
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// ---------------------------------------------------------------------------------------------------------------
// The roles, each a function of (layer, largest token box, stage layout L).
// ---------------------------------------------------------------------------------------------------------------
struct RoleState {                 // pipeline position of a role
  uint32_t stage = 0, phase = 0;   // position in the shared-memory ring
  uint32_t it = 0;                 // tasks this CTA has started: selects the accumulator buffer and its barrier phase
  bool ok = true;                  // false once the call is being abandoned
};

struct Cta {                       // where a role finds the CTA's resources
  Control* ctl;
  uint8_t* a_base;
  uint8_t* b_base;
  uint8_t* sf_base;
  uint32_t tmem_base;
  uint32_t num_stages;
};

struct TaskList {
  const Tile* tiles;
  int64_t num_tasks;
};

__device__ __forceinline__ TaskList task_list(const UmmaParams& p) {
  PlanView pv = plan_view(const_cast<char*>(p.plan), p.e_local, p.num_ranks);
  const int num_tiles = p.tile_select == 2
                            ? (p.has_shared_weights ? max(0, min(pv.hdr->num_early_shared_tiles, p.early_shared_cap)) : 0)
                            : pv.hdr->num_routed_tiles + (p.tile_select == 0 && p.has_shared_weights ? pv.hdr->num_shared_tiles : 0);
  return TaskList{pv.tiles + (p.tile_select == 2 ? p.early_shared_first : 0), (int64_t)num_tiles * p.n_blocks};
}

// ------------------------------------------------------------------------------------------------ producer
// One thread.  Everything that does not change inside a task is computed once per task; the K loop only bumps 32-bit
// coordinates and two pointers, because a one-thread loop runs at instruction latency, not throughput.
template <int kLayer, int kBoxRows, typename L>
__device__ __forceinline__ void sa_producer(const UmmaParams& p, const Cta& c, const TaskList& tl, Waiter& waiter,
                                            RoleState& st) {
  constexpr bool kInPlace = kLayer == 1 && kBoxRows == 32;
  const int k_stages = p.k_dim / kTileK;
  const uint32_t full0 = smem_u32(&c.ctl->full[0]), empty0 = smem_u32(&c.ctl->empty[0]);
  const uint32_t a0 = smem_u32(c.a_base), b0 = smem_u32(c.b_base), sf0 = smem_u32(c.sf_base);
  for (int64_t task = blockIdx.x; task < tl.num_tasks && st.ok; task += gridDim.x) {
    const int tile_idx = static_cast<int>(task / p.n_blocks);
    const int nb = static_cast<int>(task - (int64_t)tile_idx * p.n_blocks);
    const Tile tile = tl.tiles[tile_idx];
    const bool shared = tile.expert == kSharedExpert;
    // smallest token box that covers the tile (16 / 32 / 64 / 128 rows): fewer rows to move and to pad
    const int n16 = (tile.n_valid + 15) & ~15;
    const int box_sel = n16 <= 16 ? 0 : (n16 <= 32 ? 1 : (n16 <= 64 ? 2 : (n16 <= 80 ? 3 : 4)));   // never above kBoxRows
    const uint32_t box_rows = box_sel == 3 ? 80u : (box_sel == 4 ? 128u : (16u << box_sel));
    const CUtensorMap* wmap = shared ? &p.map_w_shared : &p.map_w_routed;
    const CUtensorMap* tmap = shared ? &p.map_tok_shared_box[box_sel] : &p.map_tok_routed_box[box_sel];
    const int e = shared ? 0 : tile.expert;
    // The 256 stored weight rows of the task.  Layer 1 reads W13 in its stored order [g0..7, u0..7, g8..15, ...]
    // through a 5-D map (K, row in group of 8, group of 16 rows, gate/up, slice): one box of 8 x 16 x 2 lands the
    // 128 gate rows and then the 128 up rows of 128 consecutive channels.  Layer 2 reads 256 consecutive rows.
    const bool sliced = !shared && p.routed_sliced != 0;
    const int rows_slice = sliced ? p.rows_per_expert / 2 : p.rows_per_expert;   // rows of one expert in one slice
    const int r0 = 2 * nb * kTileRows;                                           // first stored row of the task
    const int slice = sliced ? r0 / rows_slice : 0;
    const int row = e * rows_slice + r0 % rows_slice;
    const int group = row / 16;
    const int32_t* wsf = (shared ? p.wsf_shared : p.wsf_routed) + (int64_t)e * k_stages * p.rows_per_expert + r0;
    const int64_t tsf_rows = shared ? p.tsf_rows_shared : p.tsf_rows_routed;
    const int32_t* tsf = (shared ? p.tsf_shared : p.tsf_routed) + (int64_t)tile.sf_chunk * kChunkRows;
    const uint32_t a_tx = shared ? 2 * kTileRows * kTileK : kTileRows * kTileK;   // packed FP4 counts its global bytes
    const uint32_t tx = a_tx + box_rows * kTileK + 1024 + 512;
    int k0 = 0;
    for (int kb = 0; kb < k_stages; ++kb, k0 += kTileK, wsf += p.rows_per_expert, tsf += tsf_rows) {
      if (!waiter.wait(empty0 + 8 * st.stage, st.phase ^ 1u)) { st.ok = false; break; }
      const uint32_t bar = full0 + 8 * st.stage;
      mbar_expect_tx(bar, tx);
      const uint32_t a_dst = a0 + st.stage * L::kABytes;
      const uint32_t sf_dst = sf0 + st.stage * L::kSfBytes;
      if (kLayer == 1) tma_load_5d(a_dst, wmap, k0, 0, group, 0, slice, bar);
      else tma_load_3d(a_dst, wmap, k0, row, slice, bar);
      // layer 1: raw scales of the 256 stored rows, permuted by the MMA warps; layer 2: two chunks already in order
      bulk_load(sf_dst + (kLayer == 1 && !kInPlace ? 3 * 512 : 0), wsf, 1024, bar);
      tma_load_2d(b0 + st.stage * L::kBBytes, tmap, k0, tile.row0, bar);
      bulk_load(sf_dst + 2 * 512, tsf, 512, bar);
      if (++st.stage == c.num_stages) { st.stage = 0; st.phase ^= 1u; }
    }
  }
}

// ------------------------------------------------------------------------------------------------ MMA issuers
// Two warps, one per weight tile / accumulator (h = 0, 1).  The whole warp walks the loop so that loop state stays
// warp-uniform; one elected lane issues.  Each warp copies the scales it needs into its own TMEM columns, so no
// ordering between the two warps' tensor-core instructions is needed.
// Layer 1 first rearranges its tile's weight scales: the stored W13 scales follow the stored row order (gate/up
// interleaved by 8, then the 4x32 transpose inside each 128-row block), the accumulator wants the scales of 128 gate
// (h = 0) or up (h = 1) channels in tensor-memory order; each lane moves 4 of the 128 words.
template <int kLayer, int kBoxRows, typename L>
__device__ __forceinline__ void sa_mma(const UmmaParams& p, const Cta& c, const TaskList& tl, Waiter& waiter,
                                       RoleState& st, int h) {
  constexpr bool kInPlace = kLayer == 1 && kBoxRows == 32;
  const int lane = threadIdx.x & 31;
  const int k_stages = p.k_dim / kTileK;
  const uint32_t ready0 = smem_u32(&c.ctl->full[0]);
  const uint32_t empty0 = smem_u32(&c.ctl->empty[0]);
  const uint64_t sw128_hi = desc_hi_sw128();
  const uint64_t sf_hi = desc_hi_sf(128);
  // layer 1: the four 8-row groups of a weight tile's scales sit 256 bytes apart (see the rearrangement below)
  const uint64_t sfa_hi = kInPlace ? desc_hi_sf(256) : sf_hi;
  const uint32_t a_lo0 = ((smem_u32(c.a_base) & 0x3FFFFu) >> 4) + h * (kTileRows * kTileK >> 4);
  const uint32_t b_lo0 = (smem_u32(c.b_base) & 0x3FFFFu) >> 4;
  const uint32_t sf_lo0 = (smem_u32(c.sf_base) & 0x3FFFFu) >> 4;
  const uint32_t sfa_col = c.tmem_base + L::kSfCol + 4 * h;
  const uint32_t sfb_col = c.tmem_base + L::kSfCol + 8 + 4 * h;
  int src[4];                                    // layer 1: source word of the 4 destination words this lane writes
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int q = lane + 32 * t;                 // destination position inside the 128-word block
    const int m = 32 * (q & 3) + (q >> 2);       // channel of the tile that position serves
    const int r = 16 * ((m & 63) >> 3) + 8 * h + (m & 7);   // stored row inside its 128-row block
    src[t] = 128 * (m >> 6) + 4 * (r & 31) + (r >> 5);
  }
  for (int64_t task = blockIdx.x; task < tl.num_tasks && st.ok; task += gridDim.x, ++st.it) {
    const Tile tile = tl.tiles[task / p.n_blocks];
    const bool shared = tile.expert == kSharedExpert;
    const uint32_t acc_stage = st.it & 1u, acc_phase = (st.it >> 1) & 1u;
    if (!waiter.wait_warp(smem_u32(&c.ctl->tmem_empty[acc_stage]), acc_phase ^ 1u)) { st.ok = false; break; }
    tc_fence_after();
    const uint32_t n = static_cast<uint32_t>((tile.n_valid + 15) & ~15);
    const uint32_t idesc0 = make_idesc(shared ? 0u : 5u, 0u, n, 0);
    const uint32_t d = c.tmem_base + acc_stage * L::kAccCols + h * L::kNCap;
    const uint32_t sfb = sfb_col + tile.sf_col;
    for (int kb = 0; kb < k_stages; ++kb) {
      if (!waiter.wait_warp(ready0 + 8 * st.stage, st.phase)) { st.ok = false; break; }
      const uint32_t a_lo = a_lo0 + st.stage * (L::kABytes >> 4);
      const uint32_t b_lo = b_lo0 + st.stage * (L::kBBytes >> 4);
      const uint32_t sf_lo = sf_lo0 + st.stage * (L::kSfBytes >> 4);
      if (kLayer == 1 && !kInPlace) {
        uint32_t* out = reinterpret_cast<uint32_t*>(c.sf_base + st.stage * L::kSfBytes) + 128 * h;
        const uint32_t* in = reinterpret_cast<const uint32_t*>(c.sf_base + st.stage * L::kSfBytes) + 3 * 128;
        uint32_t v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = in[src[t]];
#pragma unroll
        for (int t = 0; t < 4; ++t) out[lane + 32 * t] = v[t];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to tcgen05.cp
        __syncwarp();
      }
      if (kInPlace) {
        // In stored order the scale words of the gate rows (h = 0) occupy words [64b, 64b + 32) of the 256-word
        // area (b = 0..3) and those of the up rows (h = 1) words [64b + 32, 64b + 64): the 128 words a warp reads
        // are exactly the 128 it may overwrite, so the two warps never touch each other's words.  The rearranged
        // tile is four 128-byte groups of 8 rows, 256 bytes apart, which is what the copy descriptor describes.
        uint32_t* area = reinterpret_cast<uint32_t*>(c.sf_base + st.stage * L::kSfBytes);
        uint32_t v[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) v[t] = area[src[t]];
        __syncwarp();                                                  // every lane has read before any lane writes
#pragma unroll
        for (int t = 0; t < 4; ++t) area[64 * t + 32 * h + lane] = v[t];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
      }
      if (elect_one()) {
        tc_cp_sf(sfa_col, sfa_hi | (sf_lo + (kInPlace ? 8 : 32) * h));
        tc_cp_sf(sfb_col, sf_hi | (sf_lo + 64));
#pragma unroll
        for (int k = 0; k < kTileK / 32; ++k)
          tc_mma(d, sw128_hi | (a_lo + 2 * k), sw128_hi | (b_lo + 2 * k),
                 idesc0 + k * ((1u << 4) | (1u << 29)),               // scale byte k of both operands
                 sfa_col, sfb, (kb | k) != 0 ? 1u : 0u);
        tc_commit(empty0 + 8 * st.stage);            // shared memory of this stage is free once these MMAs retire
      }
      __syncwarp();
      if (++st.stage == c.num_stages) { st.stage = 0; st.phase ^= 1u; }
    }
    if (st.ok && elect_one()) tc_commit(smem_u32(&c.ctl->tmem_full[acc_stage]));
    __syncwarp();
  }
}

// ------------------------------------------------------------------------------------------------ epilogue
// Four warps; a thread owns one weight row (accumulator lane), the columns are the tile's tokens.
// kFused (layer 2, EP > 1): every output row goes to the rank its token came from; compiled as kernels of its own so
// that the single-destination epilogue of the other cases keeps its shorter inner loop.
template <int kLayer, int kBoxRows, typename L, bool kFused>
__device__ __forceinline__ void sa_epilogue(const UmmaParams& p, const Cta& c, const TaskList& tl, Waiter& waiter,
                                            RoleState& st) {
  Control* ctl = c.ctl;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3;                     // TMEM lane quadrant this warp may read
  const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
  for (int64_t task = blockIdx.x; task < tl.num_tasks && st.ok; task += gridDim.x, ++st.it) {
    const Tile tile = tl.tiles[task / p.n_blocks];
    const int nb = static_cast<int>(task % p.n_blocks);
    const bool shared = tile.expert == kSharedExpert;
    const uint32_t acc_stage = st.it & 1u, acc_phase = (st.it >> 1) & 1u;
    // Per-token side data of the tile (top-k weight / destination row), one coalesced load per 32 tokens issued
    // before the accumulator is awaited; tokens read it by shuffle.
    float wv[4] = {1.0f, 1.0f, 1.0f, 1.0f};
    int dv[4] = {0, 0, 0, 0};
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int i = 32 * cc + lane;
      if (i < tile.n_valid) {
        if (kLayer == 1) { if (!shared) wv[cc] = __ldg(p.pool_w + tile.row0 + i); }
        else if (!kFused) dv[cc] = shared ? tile.row0 + i : __ldg(p.pool_dst + tile.row0 + i);
        else if (shared) dv[cc] = static_cast<int>((32u << kOutSlotShift) | static_cast<uint32_t>(tile.row0 + i));
        else {
          const int r = __ldg(p.pool_dst + tile.row0 + i);       // receive-order row
          int sr = 0;
          while (sr + 1 < p.num_ranks && r >= ctl->rank_off[sr + 1]) ++sr;
          dv[cc] = static_cast<int>((static_cast<uint32_t>(sr) << kOutSlotShift) |
                                    static_cast<uint32_t>(ctl->home_base[sr] + r - ctl->rank_off[sr]));
        }
      }
    }
    if (!waiter.wait_warp(smem_u32(&ctl->tmem_full[acc_stage]), acc_phase)) { st.ok = false; break; }
    tc_fence_after();
    const uint32_t d0 = c.tmem_base + lane_sel + acc_stage * L::kAccCols;
    const int n16 = (tile.n_valid + 15) & ~15;
    if (kLayer == 1) {
      const int row = nb * kTileRows + q * 32 + lane;       // channel
      uint8_t* act = shared ? p.act_shared : p.act_routed;
      uint8_t* act_sf = shared ? p.act_sf_shared : p.act_sf_routed;
      const int64_t sf_rows = shared ? p.act_sf_rows_shared : p.act_sf_rows_routed;
      // scale byte of (token i, channel group nb*4+q): word nb of the chunk row, byte q
      uint8_t* sf_out = act_sf + ((int64_t)nb * sf_rows + (int64_t)tile.sf_chunk * kChunkRows) * 4 + q;
      uint8_t* act_col = act + (int64_t)tile.row0 * p.inter + row;
      for (int i0 = 0; i0 < n16; i0 += 16) {
        uint32_t g[16], u[16];
        tc_ld16(d0 + i0, g);
        tc_ld16(d0 + L::kNCap + i0, u);
        tc_ld_wait();
        const int cc = i0 >> 5;
        const float wcur = cc == 0 ? wv[0] : (cc == 1 ? wv[1] : (cc == 2 ? wv[2] : wv[3]));
        int my_sf = 0;
        // branch-free over the 16 columns so that their dependency chains interleave (the fast-math choice is made
        // once per batch, not per element); padding columns compute garbage that is never stored
        auto batch = [&](auto fast) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float wt = __shfl_sync(0xffffffffu, wcur, (i0 & 16) + j);
            const float a = swiglu_act_t<decltype(fast)::value>(__uint_as_float(g[j]), __uint_as_float(u[j]), wt, p.clamp);
            const float amax = warp_max_nonneg(fabsf(a));
            const int sf_exp = ue8m0_exp_of_amax(amax);
            g[j] = float_to_e4m3(__fmul_rn(a, ue8m0_inv(sf_exp)));
            if (lane == j) my_sf = sf_exp;
          }
        };
        if (p.fast_math != 0) batch(std::true_type{});
        else batch(std::false_type{});
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (i0 + j < tile.n_valid) act_col[(int64_t)(i0 + j) * p.inter] = static_cast<uint8_t>(g[j]);
        if (lane < 16 && i0 + lane < tile.n_valid)
          sf_out[chunk_pos(tile.sf_col * 32 + i0 + lane) * 4] = static_cast<uint8_t>(my_sf);
      }
    } else if (!kFused) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = nb * 2 * kTileRows + h * kTileRows + q * 32 + lane;     // output feature
        __nv_bfloat16* out = (shared ? p.shared_out : p.ret) + row;
        for (int i0 = 0; i0 < n16; i0 += 16) {
          uint32_t v[16];
          tc_ld16(d0 + h * L::kNCap + i0, v);
          tc_ld_wait();
          const int cc = i0 >> 5;
          const int dcur = cc == 0 ? dv[0] : (cc == 1 ? dv[1] : (cc == 2 ? dv[2] : dv[3]));
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int dst = __shfl_sync(0xffffffffu, dcur, (i0 & 16) + j);
            if (i0 + j < tile.n_valid) out[(int64_t)dst * p.hidden] = __float2bfloat16_rn(__uint_as_float(v[j]));
          }
        }
      }
    } else {
      // one destination per token: resolve the 16 row pointers of a batch once, use them for both weight blocks
      const int row0 = nb * 2 * kTileRows + q * 32 + lane;                      // output feature of weight block 0
      for (int i0 = 0; i0 < n16; i0 += 16) {
        uint32_t v0[16], v1[16];
        tc_ld16(d0 + i0, v0);
        tc_ld16(d0 + L::kNCap + i0, v1);
        const int cc = i0 >> 5;
        const int dcur = cc == 0 ? dv[0] : (cc == 1 ? dv[1] : (cc == 2 ? dv[2] : dv[3]));
        tc_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t dst = static_cast<uint32_t>(__shfl_sync(0xffffffffu, dcur, (i0 & 16) + j));
          if (i0 + j < tile.n_valid) {
            __nv_bfloat16* out = ctl->out_base[dst >> kOutSlotShift] +
                                 (int64_t)(dst & ((1u << kOutSlotShift) - 1u)) * p.hidden + row0;
            out[0] = __float2bfloat16_rn(__uint_as_float(v0[j]));
            out[kTileRows] = __float2bfloat16_rn(__uint_as_float(v1[j]));
          }
        }
      }
    }
    tc_fence_before();
    mbar_arrive(smem_u32(&ctl->tmem_empty[acc_stage]));
  }
}

// ------------------------------------------------------------------------------------------------ set-up / teardown
template <typename L>
__device__ __forceinline__ Cta sa_carve(uint8_t* smem_raw) {
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  Cta c;
  c.ctl = reinterpret_cast<Control*>(smem);
  c.a_base = smem + 1024;
  c.b_base = c.a_base + L::kStages * L::kABytes;
  c.sf_base = c.b_base + L::kStages * L::kBBytes;
  c.tmem_base = 0;
  c.num_stages = L::kStages;
  return c;
}

// barriers and tensor memory: touches only this CTA's own shared / tensor memory
template <typename L>
__device__ __forceinline__ void sa_setup(Control* ctl) {
  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kStages; ++i) {
      mbar_init(smem_u32(&ctl->full[i]), 1);
      mbar_init(smem_u32(&ctl->empty[i]), 2);          // both MMA warps release a stage
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ctl->tmem_full[i]), 2);      // both MMA warps finish an accumulator pair
      mbar_init(smem_u32(&ctl->tmem_empty[i]), 128);
    }
    ctl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if ((threadIdx.x >> 5) == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
}

__device__ __forceinline__ void sa_teardown(Control* ctl, uint32_t tmem_base) {
  __syncwarp();
  if (ctl->abort_flag != 0) {
    // abandoned call: give copies that are still in flight time to land in this CTA's shared memory before it exits
    const uint64_t t0 = global_timer();
    while (global_timer() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if ((threadIdx.x >> 5) == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// One layer per launch.
template <int kLayer, int kBoxRows, bool kFused = false>
__global__ void __launch_bounds__(kThreads, 1) umma_kernel(const __grid_constant__ UmmaParams p) {
  static_assert(!kFused || kLayer == 2, "only GEMM2 writes rows back");
  using L = Shape<kLayer, kBoxRows>;
  extern __shared__ uint8_t smem_raw[];
  Cta c = sa_carve<L>(smem_raw);
  Control* ctl = c.ctl;
  const int warp = threadIdx.x >> 5;
  chain_release();
  sa_setup<L>(ctl);
  // Everything above touches only this CTA's own shared and tensor memory, so it may run while the kernel before this
  // one in the stream is still running; everything below reads what that kernel wrote.
  chain_wait();
  if (kFused) {
    if (threadIdx.x == 0) ctl->out_base[32] = p.shared_out;
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
  tc_fence_after();
  c.tmem_base = ctl->tmem_base;
  c.num_stages = static_cast<uint32_t>(p.num_stages);
  const TaskList tl = task_list(p);
  Waiter waiter{&ctl->abort_flag, p.status, global_timer() + static_cast<uint64_t>(p.timeout_ns), kLayer, warp};
  RoleState st;
  if (warp == 0) {
    if ((threadIdx.x & 31) == 0) sa_producer<kLayer, kBoxRows, L>(p, c, tl, waiter, st);
  } else if (warp == 1 || warp == 6) {
    sa_mma<kLayer, kBoxRows, L>(p, c, tl, waiter, st, warp == 1 ? 0 : 1);
  } else {
    sa_epilogue<kLayer, kBoxRows, L, kFused>(p, c, tl, waiter, st);
  }
  sa_teardown(ctl, c.tmem_base);
}

// ---------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
constexpr int kMaxDevices = 64;
int g_num_sms[kMaxDevices] = {};   // per device, 0 = mmoe_prepare() has not run there
int g_tune_stages = 0;             // 0: every stage that fits
int g_orientation = 0;             // 0: chosen per call, 1: weights-as-A, 2: tokens-as-A, 3: tokens-as-A on CTA pairs

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// W13 (stored rows [g0..7, u0..7, g8..15, ...]): 5-D map [slices, gate/up, groups of 16 rows, row in group of 8, K];
// a box of 8 x 16 x 2 is the 128 gate rows followed by the 128 up rows of 128 channels
int make_w13_map(CUtensorMap* map, bool fp4, const void* base, uint64_t k_elems, uint64_t rows_total, int64_t slice_stride) {
  const uint64_t row_bytes = fp4 ? k_elems / 2 : k_elems;
  const uint64_t slices = slice_stride > 0 ? 2 : 1;
  const uint64_t rows = rows_total / slices;
  const cuuint64_t dims[5] = {k_elems, 8, rows / 16, 2, slices};
  const cuuint64_t strides[4] = {row_bytes, 16 * row_bytes, 8 * row_bytes,
                                 slice_stride > 0 ? static_cast<uint64_t>(slice_stride) : rows * row_bytes};
  const cuuint32_t box[5] = {kTileK, 8, 16, 2, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = g_encode(map, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 5,
                              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

template <int kLayer, int kBoxRows>
cudaError_t prepare_one() {
  cudaError_t e = cudaFuncSetAttribute(umma_kernel<kLayer, kBoxRows, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Shape<kLayer, kBoxRows>::kSmemBytes);
  if (e == cudaSuccess && kLayer == 2)
    e = cudaFuncSetAttribute(umma_kernel<2, kBoxRows, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Shape<2, kBoxRows>::kSmemBytes);
  return e;
}

template <int kLayer, int kBoxRows>
cudaError_t launch_one(const UmmaParams& p0, cudaStream_t s) {
  using S = Shape<kLayer, kBoxRows>;
  UmmaParams p = p0;
  p.num_stages = g_tune_stages > 0 && g_tune_stages < S::kStages ? g_tune_stages : S::kStages;
  const int grid = tc_num_sms();
  if (kLayer == 2 && p.fused_return)
    launch_chained(umma_kernel<2, kBoxRows, true>, dim3(grid), dim3(kThreads), Shape<2, kBoxRows>::kSmemBytes, s, p);
  else
    launch_chained(umma_kernel<kLayer, kBoxRows, false>, dim3(grid), dim3(kThreads), S::kSmemBytes, s, p);
  return cudaGetLastError();
}

int box_rows_of(int block_m) { return block_m <= 16 ? 16 : (block_m <= 32 ? 32 : (block_m <= 64 ? 64 : (block_m == 128 ? 80 : 128))); }

template <int kLayer>
cudaError_t launch_layer(const UmmaParams& p, int box, cudaStream_t s) {
  switch (box) {
    case 16: return launch_one<kLayer, 16>(p, s);
    case 32: return launch_one<kLayer, 32>(p, s);
    case 64: return launch_one<kLayer, 64>(p, s);
    case 80: return launch_one<kLayer, 80>(p, s);
    default: return launch_one<kLayer, 128>(p, s);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Launch parameters that depend only on (workspace, weights, geometry, kernel family) -- above all the encoded tensor
// maps -- are built once and kept: a serving engine calls the layer with the same buffers thousands of times, and
// encoding two dozen tensor maps per call costs more host time than the launches themselves.  What changes per call
// (tile selection, options, peers) is patched into a copy.  The reference keeps the same kind of record per validated
// call (backend/frontend.py:650-754).
// ---------------------------------------------------------------------------------------------------------------
struct PlanKey {
  const void* ws;
  const void* w[8];
  int64_t s13, s2;
  MmoeGeometry geo;
  int family;
  int has_shared;
  int device;
  bool operator==(const PlanKey& o) const { return memcmp(this, &o, sizeof(PlanKey)) == 0; }
};
struct PlanEntry {
  PlanKey key;
  uint64_t stamp = 0;          // 0 = empty
  UmmaParams sa[2];
  TmParams tm[2];
};
constexpr int kPlanCacheSize = 16;
PlanEntry g_plans[kPlanCacheSize];
uint64_t g_plan_clock = 0;
std::mutex g_plan_mutex;

PlanKey make_key(const Ctx& c, const MmoeWeights& w, bool has_shared) {
  PlanKey k;
  memset(&k, 0, sizeof k);           // padding bytes take part in the comparison
  k.ws = c.ws;
  const void* ptrs[8] = {w.w13, w.w13_sf, w.w2, w.w2_sf, w.shared_w13, w.shared_w13_sf, w.shared_w2, w.shared_w2_sf};
  for (int i = 0; i < 8; ++i) k.w[i] = ptrs[i];
  k.s13 = w.w13_slice_stride;
  k.s2 = w.w2_slice_stride;
  k.geo = c.geo;
  k.family = c.family;
  k.has_shared = has_shared ? 1 : 0;
  k.device = current_device();
  return k;
}

// tokens-as-A form: both layers through mmoe_umma_tm.cu
bool build_tm(const Ctx& c, const MmoeWeights& w, bool has_shared, TmParams* out) {
  const int h = c.geo.hidden, inter = c.geo.intermediate, el = c.e_local;
  TmParams p1{};
  int bad = 0;
  const int ctas = c.family == kFamilyTokensAsAPair ? 2 : 1;
  const uint32_t wbox = 192 / ctas;          // a CTA of a pair stages half of a task's weight rows
  bad |= make_weight_map(&p1.map_w_routed, true, w.w13, h, (uint64_t)el * 2 * inter, w.w13_slice_stride, wbox);
  if (has_shared) bad |= make_weight_map(&p1.map_w_shared, false, w.shared_w13, h, 2 * (uint64_t)inter, 0, wbox);
  else p1.map_w_shared = p1.map_w_routed;
  const uint32_t kBoxes[2] = {64, 128};
  // a 128-row box may start up to 127 rows before the end of the token matrix; the rows past it are workspace bytes of
  // the regions that follow (never stored anywhere: they only feed accumulator lanes of rows that do not exist)
  const uint64_t x_rows = (uint64_t)c.geo.num_max_tokens + 128;
  for (int b = 0; b < 2; ++b) {
    bad |= make_token_map(&p1.map_tok_routed[b], c.ws + c.lay.pool_x, h, c.lay.pool_rows, kBoxes[b]);
    if (has_shared) bad |= make_token_map(&p1.map_tok_shared[b], c.ws + c.lay.x, h, x_rows, kBoxes[b]);
    else p1.map_tok_shared[b] = p1.map_tok_routed[b];
  }
  if (bad) return false;
  p1.plan = c.ws + c.lay.plan;
  p1.wsf_routed = static_cast<const int32_t*>(w.w13_sf);
  p1.wsf_shared = static_cast<const int32_t*>(w.shared_w13_sf);
  p1.tsf_routed = c.at<int32_t>(c.lay.pool_sf);
  p1.tsf_shared = c.at<int32_t>(c.lay.shared_x_sf);
  p1.tsf_rows_routed = c.lay.pool_sf_rows;
  p1.tsf_rows_shared = c.lay.shared_sf_rows;
  p1.act_routed = c.at<uint8_t>(c.lay.act_x);
  p1.act_shared = c.at<uint8_t>(c.lay.shared_act_x);
  p1.act_sf_routed = c.at<uint8_t>(c.lay.act_sf);
  p1.act_sf_shared = c.at<uint8_t>(c.lay.shared_act_sf);
  p1.act_sf_rows_routed = c.lay.pool_sf_rows;
  p1.act_sf_rows_shared = c.lay.shared_sf_rows;
  p1.pool_w = c.at<float>(c.lay.pool_w);
  p1.status = c.at<int32_t>(c.lay.status);
  p1.e_local = el;
  p1.num_ranks = c.geo.num_ranks;
  p1.k_dim = h;
  p1.rows_per_expert = 2 * inter;
  p1.routed_sliced = w.w13_slice_stride > 0 ? 1 : 0;
  p1.hidden = h;
  p1.inter = inter;
  p1.has_shared_weights = has_shared ? 1 : 0;
  p1.early_shared_first = c.lay.max_tiles - shared_tile_capacity(c.geo.num_max_tokens);
  p1.early_shared_cap = static_cast<int>(shared_tile_capacity(c.geo.num_max_tokens));

  TmParams p2 = p1;
  bad |= make_weight_map(&p2.map_w_routed, true, w.w2, inter, (uint64_t)el * h, w.w2_slice_stride, wbox);
  if (has_shared) bad |= make_weight_map(&p2.map_w_shared, false, w.shared_w2, inter, (uint64_t)h, 0, wbox);
  else p2.map_w_shared = p2.map_w_routed;
  for (int b = 0; b < 2; ++b) {
    bad |= make_token_map(&p2.map_tok_routed[b], c.ws + c.lay.act_x, inter, c.lay.pool_rows, kBoxes[b]);
    if (has_shared) bad |= make_token_map(&p2.map_tok_shared[b], c.ws + c.lay.shared_act_x, inter, x_rows, kBoxes[b]);
    else p2.map_tok_shared[b] = p2.map_tok_routed[b];
  }
  if (bad) return false;
  p2.wsf_routed = static_cast<const int32_t*>(w.w2_sf);
  p2.wsf_shared = static_cast<const int32_t*>(w.shared_w2_sf);
  p2.tsf_routed = c.at<int32_t>(c.lay.act_sf);
  p2.tsf_shared = c.at<int32_t>(c.lay.shared_act_sf);
  p2.ret = c.at<__nv_bfloat16>(c.lay.ret);
  p2.shared_out = c.at<__nv_bfloat16>(c.lay.shared_out);
  p2.pool_dst = c.at<int32_t>(c.lay.pool_dst);
  p2.k_dim = inter;
  p2.rows_per_expert = h;
  p2.routed_sliced = w.w2_slice_stride > 0 ? 1 : 0;
  out[0] = p1;
  out[1] = p2;
  return true;
}

bool build_sa(const Ctx& c, const MmoeWeights& w, bool has_shared, UmmaParams* out) {
  const int h = c.geo.hidden, inter = c.geo.intermediate, el = c.e_local;
  UmmaParams p1{};
  int bad = 0;
  bad |= make_w13_map(&p1.map_w_routed, true, w.w13, h, (uint64_t)el * 2 * inter, w.w13_slice_stride);
  if (has_shared) bad |= make_w13_map(&p1.map_w_shared, false, w.shared_w13, h, 2 * (uint64_t)inter, 0);
  else p1.map_w_shared = p1.map_w_routed;
  // token maps: one per box size a tile can pick (a launch never picks one above its kernel's own box)
  const uint32_t kBoxes[5] = {16, 32, 64, 80, 128};
  for (int b = 0; b < 5; ++b) {
    bad |= make_token_map(&p1.map_tok_routed_box[b], c.ws + c.lay.pool_x, h, c.lay.pool_rows, kBoxes[b]);
    if (has_shared) bad |= make_token_map(&p1.map_tok_shared_box[b], c.ws + c.lay.x, h, c.geo.num_max_tokens, kBoxes[b]);
    else p1.map_tok_shared_box[b] = p1.map_tok_routed_box[b];
  }
  if (bad) return false;
  p1.plan = c.ws + c.lay.plan;
  p1.wsf_routed = static_cast<const int32_t*>(w.w13_sf);
  p1.wsf_shared = static_cast<const int32_t*>(w.shared_w13_sf);
  p1.tsf_routed = c.at<int32_t>(c.lay.pool_sf);
  p1.tsf_shared = c.at<int32_t>(c.lay.shared_x_sf);
  p1.tsf_rows_routed = c.lay.pool_sf_rows;
  p1.tsf_rows_shared = c.lay.shared_sf_rows;
  p1.act_routed = c.at<uint8_t>(c.lay.act_x);
  p1.act_shared = c.at<uint8_t>(c.lay.shared_act_x);
  p1.act_sf_routed = c.at<uint8_t>(c.lay.act_sf);
  p1.act_sf_shared = c.at<uint8_t>(c.lay.shared_act_sf);
  p1.act_sf_rows_routed = c.lay.pool_sf_rows;
  p1.act_sf_rows_shared = c.lay.shared_sf_rows;
  p1.pool_w = c.at<float>(c.lay.pool_w);
  p1.status = c.at<int32_t>(c.lay.status);
  p1.e_local = el;
  p1.num_ranks = c.geo.num_ranks;
  p1.k_dim = h;
  p1.rows_per_expert = 2 * inter;
  p1.routed_sliced = w.w13_slice_stride > 0 ? 1 : 0;
  p1.n_blocks = inter / kTileRows;
  p1.hidden = h;
  p1.inter = inter;
  p1.has_shared_weights = has_shared ? 1 : 0;
  p1.early_shared_first = c.lay.max_tiles - shared_tile_capacity(c.geo.num_max_tokens);
  p1.early_shared_cap = static_cast<int>(shared_tile_capacity(c.geo.num_max_tokens));

  UmmaParams p2 = p1;
  bad |= make_weight_map(&p2.map_w_routed, true, w.w2, inter, (uint64_t)el * h, w.w2_slice_stride, 2 * kTileRows);
  if (has_shared) bad |= make_weight_map(&p2.map_w_shared, false, w.shared_w2, inter, (uint64_t)h, 0, 2 * kTileRows);
  else p2.map_w_shared = p2.map_w_routed;
  for (int b = 0; b < 5; ++b) {
    bad |= make_token_map(&p2.map_tok_routed_box[b], c.ws + c.lay.act_x, inter, c.lay.pool_rows, kBoxes[b]);
    if (has_shared) bad |= make_token_map(&p2.map_tok_shared_box[b], c.ws + c.lay.shared_act_x, inter, c.geo.num_max_tokens, kBoxes[b]);
    else p2.map_tok_shared_box[b] = p2.map_tok_routed_box[b];
  }
  if (bad) return false;
  p2.wsf_routed = static_cast<const int32_t*>(w.w2_sf);
  p2.wsf_shared = static_cast<const int32_t*>(w.shared_w2_sf);
  p2.tsf_routed = c.at<int32_t>(c.lay.act_sf);
  p2.tsf_shared = c.at<int32_t>(c.lay.shared_act_sf);
  p2.ret = c.at<__nv_bfloat16>(c.lay.ret);
  p2.shared_out = c.at<__nv_bfloat16>(c.lay.shared_out);
  p2.pool_dst = c.at<int32_t>(c.lay.pool_dst);
  p2.k_dim = inter;
  p2.rows_per_expert = h;
  p2.routed_sliced = w.w2_slice_stride > 0 ? 1 : 0;
  p2.n_blocks = h / (2 * kTileRows);
  out[0] = p1;
  out[1] = p2;
  return true;
}

// the kept record for (workspace, weights, geometry, family), built on first use; least recently used slot is replaced
const PlanEntry* cached_plan(const Ctx& c, const MmoeWeights& w, bool has_shared) {
  const PlanKey key = make_key(c, w, has_shared);
  std::lock_guard<std::mutex> lock(g_plan_mutex);
  PlanEntry* victim = &g_plans[0];
  for (PlanEntry& e : g_plans) {
    if (e.stamp != 0 && e.key == key) {
      e.stamp = ++g_plan_clock;
      return &e;
    }
    if (e.stamp < victim->stamp) victim = &e;
  }
  const bool ok = c.family == kFamilyWeightsAsA ? build_sa(c, w, has_shared, victim->sa) : build_tm(c, w, has_shared, victim->tm);
  if (!ok) {
    victim->stamp = 0;
    return nullptr;
  }
  victim->key = key;
  victim->stamp = ++g_plan_clock;
  return victim;
}

}  // namespace

int tc_num_sms() {
  const int dev = current_device();
  return dev < 0 ? 0 : g_num_sms[dev];
}
bool tc_ready() { return g_encode != nullptr && tc_num_sms() > 0; }

void set_tuning(int max_stages, int orientation) {
  g_tune_stages = max_stages;
  g_orientation = orientation;
}
int tuned_orientation() { return g_orientation; }

int make_token_map(CUtensorMap* map, const void* base, uint64_t k_elems, uint64_t rows, uint32_t box_rows) {
  const cuuint64_t dims[2] = {k_elems, rows};
  const cuuint64_t strides[1] = {k_elems};
  const cuuint32_t box[2] = {kTileK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int make_weight_map(CUtensorMap* map, bool fp4, const void* base, uint64_t k_elems, uint64_t rows_total,
                    int64_t slice_stride, uint32_t box_rows) {
  const uint64_t row_bytes = fp4 ? k_elems / 2 : k_elems;
  const uint64_t slices = slice_stride > 0 ? 2 : 1;
  const uint64_t rows = rows_total / slices;
  const cuuint64_t dims[3] = {k_elems, rows, slices};
  const cuuint64_t strides[2] = {row_bytes, slice_stride > 0 ? static_cast<uint64_t>(slice_stride) : rows * row_bytes};
  const cuuint32_t box[3] = {kTileK, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = g_encode(map, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                              const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// Once per device (the dynamic shared-memory limits are per device) and outside stream capture.
int prepare_umma(const MmoeGeometry& geo) {
  (void)geo;
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return MMOE_ERR_CUDA;
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const int dev = current_device();
  if (dev < 0) return MMOE_ERR_CUDA;
  if (g_num_sms[dev] > 0) return MMOE_OK;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return MMOE_ERR_CUDA;
  cudaError_t e = cudaSuccess;
  if (e == cudaSuccess) e = prepare_one<1, 16>();
  if (e == cudaSuccess) e = prepare_one<1, 32>();
  if (e == cudaSuccess) e = prepare_one<1, 64>();
  if (e == cudaSuccess) e = prepare_one<1, 80>();
  if (e == cudaSuccess) e = prepare_one<1, 128>();
  if (e == cudaSuccess) e = prepare_one<2, 16>();
  if (e == cudaSuccess) e = prepare_one<2, 32>();
  if (e == cudaSuccess) e = prepare_one<2, 64>();
  if (e == cudaSuccess) e = prepare_one<2, 80>();
  if (e == cudaSuccess) e = prepare_one<2, 128>();
  if (e == cudaSuccess) e = tm_prepare();
  if (e != cudaSuccess) return MMOE_ERR_CUDA;
  g_num_sms[dev] = sms;
  return MMOE_OK;
}

cudaError_t launch_experts_umma(const Ctx& c, const MmoeWeights& w, const MmoeOptions& o, int m, int block_m,
                                cudaStream_t s) {
  if (!tc_ready()) return cudaErrorNotReady;
  const bool has_shared = c.geo.num_shared_experts > 0 && w.shared_w13 != nullptr && m > 0;
  const int64_t timeout_ns = (o.timeout_ms > 0 ? (int64_t)o.timeout_ms : 2000) * 1000000ll;
  const PlanEntry* plan = cached_plan(c, w, has_shared);
  if (plan == nullptr) return cudaErrorInvalidValue;
  const bool fused = c.peer_ws != nullptr && c.geo.num_ranks > 1 && c.tile_select != 2;
  const int mask = o.layer_mask == 0 ? 3 : o.layer_mask;
  cudaError_t e = cudaSuccess;

  // what changes from call to call is patched into a copy of the kept parameters
  auto patch = [&](auto& p, bool layer2) {
    p.timeout_ns = timeout_ns;
    p.clamp = o.activation_clamp;
    p.fast_math = o.fast_math;
    p.tile_select = c.tile_select;
    if (layer2 && fused) {
      p.ep_me = c.geo.rank;
      p.ep_totals = reinterpret_cast<const int32_t*>(c.ws + c.lay.ep_sync + ep_totals_offset());
      for (int r = 0; r < c.geo.num_ranks; ++r)
        p.ep_ret_recv[r] = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(const_cast<void*>(c.peer_ws[r])) + c.lay.ret_recv);
    }
  };
  if (c.family != kFamilyWeightsAsA) {
    const int ctas = c.family == kFamilyTokensAsAPair ? 2 : 1;
    if (mask & 1) {
      TmParams p = plan->tm[0];
      patch(p, false);
      e = tm_launch(1, false, ctas, p, s);
    }
    if (e == cudaSuccess && (mask & 2)) {
      TmParams p = plan->tm[1];
      patch(p, true);
      e = tm_launch(2, fused, ctas, p, s);
    }
    return e;
  }
  const int box = box_rows_of(block_m);
  if (mask & 1) {
    UmmaParams p = plan->sa[0];
    patch(p, false);
    e = launch_layer<1>(p, box, s);
  }
  if (e == cudaSuccess && (mask & 2)) {
    UmmaParams p = plan->sa[1];
    patch(p, true);
    p.fused_return = fused ? 1 : 0;
    e = launch_layer<2>(p, box, s);
  }
  return e;
}

}  // namespace mmoe
