/*
 * C ABI of the B200 (sm_100a) MegaMoE expert backend: `libmmoe_b200.so`.
 *
 * Plain pointers, integers and a CUDA stream handle only; nothing throws across this boundary.  Every entry point
 * returns an MMOE_* status code; `mmoe_status_string()` names it.  Device pointers are never dereferenced on the host.
 * All kernels are enqueued on the given stream and the functions never synchronise, so a sequence of calls can be
 * captured into a CUDA graph once `mmoe_prepare()` has run for the geometry (outside capture).
 *
 * Each declaration cites the interface of the reference plugin (`vllm_sm107_megamoe`, paths relative to its project
 * root) that it stands in for.
 */
#ifndef MMOE_B200_H_
#define MMOE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MMOE_OK = 0,
  MMOE_ERR_INVALID_ARGUMENT = 1,  /* maps to AssertionError / ValueError on the Python side */
  MMOE_ERR_UNSUPPORTED = 2,       /* maps to NotImplementedError */
  MMOE_ERR_CUDA = 3,              /* a CUDA runtime / driver call failed: RuntimeError */
  MMOE_ERR_ARCH = 4,              /* the current device is not compute capability 10.0: RuntimeError */
  MMOE_ERR_NOT_PREPARED = 5,      /* a launch was requested before mmoe_prepare(): RuntimeError */
  MMOE_ERR_DEVICE_TIMEOUT = 6     /* a bounded device-side wait expired (read back with mmoe_read_status) */
};

/* Geometry of one layer instance on one rank.  Replaces the positional geometry arguments of
 * `get_symm_buffer_for_mega_moe` (api.py:39-65) and of the kernel configuration (backend/config.py:41-329). */
typedef struct MmoeGeometry {
  int32_t num_ranks;           /* expert-parallel size R (1..32) */
  int32_t rank;                /* this rank */
  int32_t num_experts;         /* physical routed experts over all ranks (E); this rank owns [rank*E/R, (rank+1)*E/R) */
  int32_t num_topk;            /* routes per token (k) */
  int32_t hidden;              /* H */
  int32_t intermediate;        /* I */
  int32_t num_shared_experts;  /* 0 or 1 */
  int32_t num_max_tokens;      /* per-rank token capacity T, a multiple of 1920 */
} MmoeGeometry;

/* Byte offsets of every region of the per-rank workspace (one allocation owned by the caller).  The first five are the
 * views the serving engine writes or reads (`SymmBuffer.x / x_sf / topk_idx / topk_weights / shared_l1_acts_sf`,
 * backend/workspace.py:72-76,147-161); the rest are private to the kernels.  Replaces `build_symm_buffer_layout`
 * (backend/heuristics.py:504-674). */
typedef struct MmoeLayout {
  int64_t total_bytes;
  int64_t x;                /* e4m3 [T, H] */
  int64_t x_sf;             /* int32 [T, H/128], byte j of word w = UE8M0 exponent of K group 4w+j */
  int64_t topk_idx;         /* int64 [T, k], -1 = masked */
  int64_t topk_weights;     /* float [T, k] */
  int64_t shared_x_sf;      /* int32 [ceil(T/8)*128, H/128], element (row, word) at word*rows + row */
  int64_t shared_sf_rows;   /* = ceil(T/8)*128 */
  int64_t send_count;       /* int32 [E]      routes of this rank per destination physical expert */
  int64_t send_offset;      /* int32 [E+1]    exclusive prefix of send_count */
  int64_t route_pos;        /* int32 [T*k]    position of a route in send order, -1 = masked */
  int64_t sorted_route;     /* int32 [T*k]    route id (token*k + slot) at each send position */
  int64_t sort_scratch;     /* int32 [ceil(T/128), E] per-chunk expert counts of the route ordering */
  int64_t recv_count;       /* int32 [R, E/R] routes received per (source rank, local expert) */
  int64_t plan;             /* MmoePlanHeader followed by per-expert and per-tile tables */
  int64_t send_x, send_sf, send_w;      /* EP>1 only: packed rows in send order */
  int64_t recv_x, recv_sf, recv_w;      /* EP>1 only: rows in receive order */
  int64_t pool_x;           /* e4m3 [pool_rows, H] */
  int64_t pool_sf;          /* int32 chunks, element (chunk row, word) at word*pool_sf_rows + row */
  int64_t pool_w;           /* float [pool_rows] top-k weight of each pool row */
  int64_t pool_dst;         /* int32 [pool_rows] row of `ret` that receives the expert output, -1 = padding */
  int64_t act_x;            /* e4m3 [pool_rows, I]   SwiGLU output of the routed experts */
  int64_t act_sf;           /* int32 chunks like pool_sf with I/128 words */
  int64_t shared_act_x;     /* e4m3 [T, I] */
  int64_t shared_act_sf;    /* int32 chunks like shared_x_sf with I/128 words */
  int64_t ret;              /* bf16 [R*T*kmax, H]  expert outputs in receive order (EP1: == send order) */
  int64_t ret_recv;         /* EP>1 only: bf16 [T*kmax, H] outputs returned to this rank, in send order */
  int64_t shared_out;       /* bf16 [T, H] */
  int64_t ep_sync;          /* EP>1 only: epoch, per-barrier arrival flags and the [R][R] route-total table of the peer exchange */
  int64_t status;           /* int32 [8] device status words, zero = healthy */
  int64_t pool_rows;        /* row capacity of pool_x / act_x */
  int64_t pool_sf_rows;     /* row capacity (multiple of 128) of the pool SF chunk matrices */
  int64_t max_routes;       /* T * min(k, E/R): rows one rank can send */
  int64_t max_tiles;        /* capacity of the tile table */
} MmoeLayout;

/* Replaces `build_symm_buffer_layout` (backend/heuristics.py:504-674) / `SymmBuffer.__init__` sizing
 * (backend/workspace.py:108-116). */
int mmoe_layout(const MmoeGeometry* geo, MmoeLayout* out);

/* Replaces `get_block_m_for_mega_moe` (api.py:103-118; backend/heuristics.py:123-197). */
int mmoe_block_m(int32_t num_ranks, int32_t num_experts, int32_t num_tokens, int32_t num_topk);

/* Load the kernels of every BLOCK_M variant, raise their dynamic shared-memory limits and resolve the driver entry
 * points used for tensor maps.  Must run once per device (with that device current) before any launch there, and
 * outside stream capture: `stream` is the stream the caller will launch on, and the call is refused with
 * MMOE_ERR_NOT_PREPARED while it is capturing.  Replaces `precompile_mega_moe_variants` (api.py:179-206;
 * backend/frontend.py:851-897) and the JIT cache (backend/jit.py:350-395).  `block_ms` receives the prepared variants
 * (capacity `cap`), `*n` their number. */
int mmoe_prepare(const MmoeGeometry* geo, int32_t* block_ms, int32_t cap, int32_t* n, void* stream);

/* Kernel (a): BF16 hidden states -> MXFP8 E4M3 + packed UE8M0 scales, routing repack (padding -> id -1 / weight 0) and
 * the shared-expert scale scatter, written into the workspace views.  Replaces `prepare_megamoe_inputs`
 * (backend/staging.py:152-251) and its Triton kernel (backend/staging_triton.py:23-226).
 * `topk_ids` may be int32 or int64 (`ids_are_int64`); `is_padding` (uint8 per token) and the shared view are optional
 * (`shared_block_m <= 0` skips the scatter). */
int mmoe_stage_inputs(const MmoeGeometry* geo, void* workspace, const void* hidden_bf16, const void* topk_ids,
                      int32_t ids_are_int64, const float* topk_weights, const uint8_t* is_padding, int32_t num_tokens,
                      int32_t shared_block_m, void* stream);

/* The step in front of kernel (a), fused into the same launch: router top-k + staging.  `router_logits` float
 * [num_tokens, num_logical_experts]; per token the `num_topk` largest logits are selected (ties: the lower expert id),
 * the weights are the softmax over the selected logits, and -- with a replica table -- every selected logical expert l
 * is mapped to its physical copy `replica_slots[l][(token + slot) % replica_count[l]]` (int32 [num_logical_experts] and
 * [num_logical_experts, max_copies]), the deterministic choice the benchmark's load-balancer configuration prescribes;
 * without a table the logical id is the physical id.  Ids and weights land in the `topk_idx` / `topk_weights` views
 * exactly as `mmoe_stage_inputs` would have repacked them; the hidden states are quantised as there.  In the reference
 * these steps belong to the serving engine in front of the hook (top-k routing and the logical -> physical mapping,
 * README.md:112-125; patches/vllm-megamoe-plugin.patch:43-69), not to the plugin. */
int mmoe_route_stage_inputs(const MmoeGeometry* geo, void* workspace, const void* hidden_bf16, const float* router_logits,
                            int32_t num_logical_experts, const int32_t* replica_count, const int32_t* replica_slots,
                            int32_t max_copies, const uint8_t* is_padding, int32_t num_tokens, int32_t shared_block_m,
                            void* stream);

/* NVFP4 activation staging: BF16 `[num_tokens, hidden]` -> packed E2M1 `[num_tokens, hidden/2]` bytes (low nibble = even
 * K) + one E4M3 scale byte per 16 elements `[num_tokens, hidden/16]`, with the per-tensor `global_scale` of the two-level
 * NVFP4 recipe: per block s = e4m3_rn(amax * global_scale / 6), q = e2m1_rn(x * global_scale / s); x ~ q * s / global_scale.
 * The serving engine's hook imports such a call beside the MXFP8 staging (`prepare_megamoe_nvfp4_inputs`,
 * patches/vllm-megamoe-plugin.patch:10); the reference plugin does not implement it.  Outputs are caller-owned buffers:
 * the layer's own GEMMs take MXFP8 activations. */
int mmoe_stage_inputs_nvfp4(const void* hidden_bf16, float global_scale, void* q_out, void* sf_out, int32_t num_tokens,
                            int32_t hidden, void* stream);

/* Weights of one rank in the layout `transform_weights_for_mega_moe` produces, which is bit-identical to the
 * reference's (backend/weights.py:120-145): W13 rows interleaved gate/up by 8 ([g0..7, u0..7, g8..15, ...]), scale words
 * in the same row order and 4x32-transposed inside every 128-row block. */
typedef struct MmoeWeights {
  const void* w13;        /* packed E2M1 [E/R, 2I, H/2], stored rows gate/up interleaved by 8 */
  const void* w13_sf;     /* int32 [E/R, H/128, 2I] (scale word w of stored row r at w*2I + r'), 4x32 transposed per 128 rows */
  const void* w2;         /* packed E2M1 [E/R, H, I/2] */
  const void* w2_sf;      /* int32 [E/R, I/128, H], 4x32 transposed per 128 rows */
  const void* shared_w13; /* E4M3 [2I, H] (same gate/up interleave) or NULL */
  const void* shared_w13_sf;
  const void* shared_w2;  /* E4M3 [H, I] or NULL */
  const void* shared_w2_sf;
  /* Routed weights may be given in the two-slice form `localize()` produces (backend/locality.py:573-587 of the
   * reference): [2, E/R, N/2, K/2] with the two slices `*_slice_stride` bytes apart, slice s holding rows
   * [s*N/2, (s+1)*N/2) of every expert.  A stride of 0 means the plain [E/R, N, K/2] tensor. */
  int64_t w13_slice_stride;
  int64_t w2_slice_stride;
} MmoeWeights;

typedef struct MmoeOptions {
  float activation_clamp;   /* SwiGLU clamp; +inf disables it */
  int32_t fast_math;        /* 1: ex2.approx / rcp.approx sigmoid, 0: IEEE expf and division */
  int32_t engine;           /* 0: tcgen05 tensor-core kernels; 1: scalar validation kernels (tests only) */
  int32_t timeout_ms;       /* bound of every device-side wait; <= 0 selects the default (2000) */
  int32_t layer_mask;       /* 0 or 3: both grouped GEMMs; 1: GEMM1 (+SwiGLU) only; 2: GEMM2 only (per-kernel timing) */
  const void* residual;     /* mmoe_forward / mmoe_forward_ep: optional bf16 [num_tokens, H] added in the combine
                             * (see mmoe_combine_residual); NULL: none */
} MmoeOptions;

/* The steps of one forward call.  At EP1 `mmoe_forward` runs all of them; at EP>1 the host interleaves the three
 * exchanges (counts, rows out, rows back) between them.  Together they replace `fp8_fp4_mega_moe`
 * (api.py:78-100; backend/frontend.py:627-848) and the device roles it launches (backend/kernel/dispatch.py,
 * scheduler.py, tma_warps.py, mma_warp.py, epilogue.py, combine.py). */

/* Count this rank's routes per destination expert and order them (send order = by expert, token, slot). */
int mmoe_dispatch_count(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, void* stream);
/* No counterpart in the reference.  Same result as the route-ordering step of `mmoe_dispatch_count`, for callers that
 * cannot let this library touch the device allocator on their behalf: a serving process that has already handed all
 * free device memory to its own pool (a late allocation fails or fragments it), or a latency-critical loop that cannot
 * afford the device-wide synchronisation cudaMalloc / cudaFree imply.  The caller passes the input (`topk_idx`, int64
 * [num_tokens, num_topk], -1 = masked route; ids >= num_experts are treated as masked) and the four outputs
 * (`send_count` int32 [num_experts], `send_offset` int32 [num_experts+1], `route_pos` and `sorted_route` int32
 * [num_tokens*num_topk]); the per-chunk counts the passes need live in a 64 KB array built into the library image,
 * which every GPU that loads the library keeps until the process exits.  Limits: num_tokens <= 4096 and
 * num_experts <= 512; larger sizes are rejected with MMOE_ERR_INVALID_ARGUMENT.  This function calls no cudaMalloc,
 * cudaFree or other allocating routine.  The first call on a device looks up the array's device address (the device
 * must be current); make that first call before any stream capture (a first call on a capturing stream is refused with
 * MMOE_ERR_CUDA and launches nothing; host threads may race on the first call).  All calls on a device share the one array: it
 * needs no clearing (every cell read is written first within the call), but two calls that overlap on the GPU (for
 * example on different streams) race on it. */
int mmoe_route_order_noalloc(const int64_t* topk_idx, int32_t num_tokens, int32_t num_topk, int32_t num_experts,
                             int32_t* send_count, int32_t* send_offset, int32_t* route_pos, int32_t* sorted_route,
                             void* stream);

/* EP>1: gather rows, scales and weights into send order. */
int mmoe_dispatch_pack(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, void* stream);
/* EP>1, device-side transport: the all-to-all of counts and rows as peer-memory stores over NVLink instead of host-issued
 * collectives.  `peer_workspaces[r]` is rank r's workspace mapped into this process (symmetric allocation; entry
 * [rank] is this rank's own).  `mmoe_ep_dispatch` runs after `mmoe_dispatch_count` and leaves `recv_count` and the
 * receive buffers filled exactly as the host-driven exchange would; `mmoe_ep_return` runs after `mmoe_experts` and
 * fills `ret_recv`.  Every rank of the group must make the same calls in the same order.  Replaces the in-kernel NVLink
 * dispatch / write-back / barriers of the reference (backend/kernel/dispatch.py:348-589, epilogue.py:407-413,
 * comm.py:277-318). */
int mmoe_ep_dispatch(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces, int32_t num_tokens,
                     const MmoeOptions* opt, void* stream);
int mmoe_ep_return(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces, const MmoeOptions* opt,
                   void* stream);

/* Build the pool plan from `recv_count`, place received rows into the BLOCK_M-aligned pool, add the per-expert totals
 * to `stats` (int32 [E/R], may be NULL).  `total_recv_rows` bounds the rows present in receive order. */
int mmoe_dispatch_place(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, int32_t block_m,
                        int32_t* stats, void* stream);
/* Grouped GEMM1 -> SwiGLU/requant -> grouped GEMM2 for routed and shared experts. */
int mmoe_experts(const MmoeGeometry* geo, void* workspace, const MmoeWeights* weights, const MmoeOptions* opt,
                 int32_t num_tokens, int32_t block_m, void* stream);
/* The two halves of `mmoe_experts` that `mmoe_forward_ep` runs on either side of the join, exported for hosts that build
 * their own overlap (and so that the split can be checked on one GPU): `mmoe_plan_shared` plans the shared expert's
 * tiles from the token count alone (before any receive count is known); `mmoe_experts_select` runs both GEMMs over
 * `tile_select` = 0 every tile of the plan (= `mmoe_experts`), 1 the routed tiles only, 2 the shared expert's tiles
 * written by `mmoe_plan_shared`.  Selections 1 and 2 together leave exactly what selection 0 leaves.  Corresponds to
 * the reference scheduling shared-expert blocks ahead of the routed ones (backend/kernel/scheduler.py:250-259). */
int mmoe_plan_shared(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, int32_t block_m, void* stream);
int mmoe_experts_select(const MmoeGeometry* geo, void* workspace, const MmoeWeights* weights, const MmoeOptions* opt,
                        int32_t num_tokens, int32_t block_m, int32_t tile_select, void* stream);
/* EP>1, device-side transport: `mmoe_experts` with the write-back fused into GEMM2 -- the epilogue stores every BF16
 * output row straight into the `ret_recv` of the rank its token came from (peer stores over NVLink while the tensor
 * cores work on the next tile), then barrier 2 is published and awaited.  Replaces `mmoe_experts` + `mmoe_ep_return`;
 * the result in `ret_recv` is bit-identical.  This is the reference's in-kernel NVLink write-back
 * (backend/kernel/epilogue.py:407-413, comm.py:277-318). */
int mmoe_experts_ep_return(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces,
                           const MmoeWeights* weights, const MmoeOptions* opt, int32_t num_tokens, int32_t block_m,
                           void* stream);
/* y[t] = bf16(sum of the token's valid slots in ascending order, shared expert last). */
int mmoe_combine(const MmoeGeometry* geo, void* workspace, void* y_bf16, int32_t num_tokens, void* stream);
/* The same with the residual stream of the decoder layer added in the same pass (the addition the serving engine makes
 * right after the layer): y[t] = bf16(float(bf16(sum)) + float(residual[t])), i.e. bit for bit what a separate BF16
 * addition of the layer output and `residual_bf16` ([num_tokens, H], 16-byte aligned, may alias y) leaves.  Saves
 * one read and one write of [num_tokens, H].  NULL residual: plain combine. */
int mmoe_combine_residual(const MmoeGeometry* geo, void* workspace, void* y_bf16, const void* residual_bf16,
                          int32_t num_tokens, void* stream);
/* EP1 convenience: count, place, experts, combine.  Past the decode sizes (num_tokens > 128, with a shared expert) the
 * routed experts' ordering, plan and placement run on the library's second stream while the shared expert's GEMMs run
 * on `stream` (fork / join with events, capturable); same result as the separate calls.  Up to 128 tokens the call is
 * one stream and five or six launches: one block orders the routes, builds the plan and (up to 128 routes) places the
 * rows; the kernels are launched as a programmatic chain, so that each one's launch and set-up overlap its
 * predecessor (MMOE_DISABLE_CHAINED_LAUNCH=1 in the environment, read once per process: ordinary launches).
 * Threading: the second stream and its two events exist once per device; call mmoe_forward / mmoe_forward_ep for one
 * device from one host thread at a time. */
int mmoe_forward(const MmoeGeometry* geo, void* workspace, const MmoeWeights* weights, const MmoeOptions* opt,
                 void* y_bf16, int32_t num_tokens, int32_t block_m, int32_t* stats, void* stream);

/* EP>1 convenience, device-side transport: count, exchange, place, experts with the fused write-back, combine.  The
 * exchange of counts and rows runs on a second stream of the library (created by `mmoe_prepare`) while the shared
 * expert, which needs only this rank's own tokens, runs both of its GEMMs on `stream`; the two streams fork and join
 * with events, so the whole call can be captured in a CUDA graph.  Same result as the separate calls.  Corresponds to
 * the reference scheduling the shared expert into the dispatch gap (backend/kernel/scheduler.py:250-259). */
int mmoe_forward_ep(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces,
                    const MmoeWeights* weights, const MmoeOptions* opt, void* y_bf16, int32_t num_tokens, int32_t block_m,
                    int32_t* stats, void* stream);

/* Load-time transform of one (weights, scale factors) pair into the layout the grouped GEMMs read; replaces the torch
 * indexing ops of `transform_weights_for_mega_moe` (backend/weights.py:83-145) with two HBM-bound kernels, bit for bit.
 * `w_in` / `w_out`: `num_groups` matrices of `rows` x `k_packed_bytes` bytes (packed FP4 or FP8), contiguous; `sf_in` /
 * `sf_out`: int32 scale words, MN-major `[num_groups][k_words][rows]` (rows % 128 == 0, dense).  `interleave` = 1 (W13):
 * rows `[gate | up]` -> `[g0..7, u0..7, g8..15, ...]` for weights and scales, then the 4x32 transpose of the scale words
 * inside every 128-row block; `interleave` = 0 (W2): only the scale transpose, `w_in` / `w_out` are not touched and may
 * be NULL.  Out of place. */
int mmoe_transform_weights(const void* w_in, void* w_out, const int32_t* sf_in, int32_t* sf_out, int32_t num_groups,
                           int32_t rows, int32_t k_packed_bytes, int32_t k_words, int32_t interleave, void* stream);

/* Copy the device status words to the host (synchronises the stream), clear them on the device and translate them:
 * MMOE_OK, MMOE_ERR_DEVICE_TIMEOUT (a bounded wait expired: the outputs of that call are not valid) or
 * MMOE_ERR_INVALID_ARGUMENT (expert ids >= num_experts were seen and treated as masked).  The words are sticky until
 * read, so one read after any number of calls reports whether any of them failed; after the read a healthy call
 * reports MMOE_OK again.  Replaces the reference's device `trap` after a 300 s spin (backend/kernel/comm.py:229-250). */
int mmoe_read_status(const MmoeGeometry* geo, void* workspace, int32_t* words8, void* stream);

/* Process-wide tuning of the tensor-core kernels (the reference keeps such knobs in `KernelOptions`,
 * backend/frontend.py:72-116).  `max_stages`: cap on the shared-memory pipeline depth of the weights-as-A kernels (0: no
 * cap).  `orientation`: 0 = chosen per call (weights-as-A kernels below about 80 expected rows per expert, tokens-as-A
 * kernels from there, and for the shared expert of a call with more than 128 tokens), 1 = weights-as-A always, 2 =
 * tokens-as-A wherever the geometry allows (intermediate >= 192, hidden >= 384), 3 = tokens-as-A on CTA pairs
 * (`tcgen05.mma.cta_group::2`) wherever the geometry and BLOCK_M (>= 128) allow; never chosen automatically: measured
 * on B200 it is slower than single CTAs at 120 to 480 rows per expert.  Every rank and every step of a call (planning, GEMM launches) must see the same
 * setting. */
int mmoe_set_tuning(int32_t max_stages, int32_t orientation);

const char* mmoe_status_string(int code);
const char* mmoe_last_error(void);   /* detail of the last failure on this thread */
int mmoe_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MMOE_B200_H_ */
