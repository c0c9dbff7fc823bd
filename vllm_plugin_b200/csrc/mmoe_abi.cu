// extern "C" entry points of libmmoe_b200.so (declared in include/mmoe.h): argument checks, workspace layout, and the
// sequencing of the kernels of one forward call.  Nothing here allocates device memory or synchronises.
#include <math.h>
#include <stdarg.h>

#include <mutex>
#include <stdio.h>
#include <string.h>

#include <string>

#include "mmoe_common.cuh"

namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(MMOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

const int kBlockMs[6] = {16, 32, 64, 128, 192, 240};

// A second stream per device on which the expert-parallel dispatch runs while the shared expert computes.
struct SideLane {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};
constexpr int kMaxDevices = 64;
SideLane g_side[kMaxDevices];

std::mutex g_side_mutex;

SideLane* side_lane(bool may_create) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideLane& l = g_side[dev];
  if (l.stream == nullptr && may_create) {
    SideLane n;
    if (cudaStreamCreateWithFlags(&n.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&n.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&n.join, cudaEventDisableTiming) != cudaSuccess)
      return nullptr;
    l = n;
  }
  return l.stream != nullptr ? &l : nullptr;
}

bool valid_block_m(int bm) {
  for (int v : kBlockMs)
    if (v == bm) return true;
  return false;
}

int check_geometry(const MmoeGeometry* g) {
  if (g == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "geometry is NULL");
  if (g->num_ranks < 1 || g->num_ranks > 32) return fail(MMOE_ERR_INVALID_ARGUMENT, "num_ranks=%d outside [1, 32]", g->num_ranks);
  if (g->rank < 0 || g->rank >= g->num_ranks) return fail(MMOE_ERR_INVALID_ARGUMENT, "rank=%d outside [0, %d)", g->rank, g->num_ranks);
  if (g->num_experts < 1 || g->num_experts % g->num_ranks != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "num_experts=%d must be a positive multiple of num_ranks=%d", g->num_experts, g->num_ranks);
  if (g->num_experts > 2048 || g->num_experts / g->num_ranks > 512)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "num_experts=%d exceeds 2048 (or 512 per rank)", g->num_experts);
  if (g->num_topk < 1 || g->num_topk > 31) return fail(MMOE_ERR_INVALID_ARGUMENT, "num_topk=%d outside [1, 31]", g->num_topk);
  if (g->hidden < 256 || g->hidden % 256 != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "hidden=%d must be a multiple of 256", g->hidden);
  if (g->intermediate < 128 || g->intermediate % 128 != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "intermediate=%d must be a multiple of 128", g->intermediate);
  if (g->num_shared_experts < 0 || g->num_shared_experts > 1)
    return fail(MMOE_ERR_UNSUPPORTED, "num_shared_experts=%d (supported: 0 or 1)", g->num_shared_experts);
  if (g->num_max_tokens < 1920 || g->num_max_tokens % 1920 != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "num_max_tokens=%d must be a positive multiple of 1920", g->num_max_tokens);
  return MMOE_OK;
}

int make_ctx(const MmoeGeometry* g, void* ws, mmoe::Ctx* c) {
  int rc = check_geometry(g);
  if (rc != MMOE_OK) return rc;
  if (ws == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "workspace is NULL");
  if ((reinterpret_cast<uintptr_t>(ws) & 1023u) != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "workspace must be 1024-byte aligned");
  c->geo = *g;
  rc = mmoe_layout(g, &c->lay);
  if (rc != MMOE_OK) return rc;
  c->ws = static_cast<char*>(ws);
  c->e_local = g->num_experts / g->num_ranks;
  c->kmax = g->num_topk < c->e_local ? g->num_topk : c->e_local;
  return MMOE_OK;
}

// Which kernel family runs a tile list, hence how the list is cut.  A pure function of the call's geometry, token
// count and BLOCK_M, so that the planning step and the GEMM launches of one call agree without talking to each other.
// `early_shared`: the shared expert's tiles planned ahead of the routed ones (tile_select 2); otherwise the routed tiles
// and the shared tiles planned with them.
int choose_family(const MmoeGeometry* g, int m, int block_m, bool early_shared) {
  // a half of each weight matrix must hold a 192-row box (more than one for the short last block of a CTA pair)
  const bool fits = g->intermediate >= 192 && g->hidden / 2 >= 192;
  const bool pair_ok = fits && block_m >= 128;        // two scale chunks per pool block: one per half of a pair
  const int forced = mmoe::tuned_orientation();
  if (!fits || forced == 1) return mmoe::kFamilyWeightsAsA;
  if (forced == 2 || (forced == 3 && !pair_ok)) return mmoe::kFamilyTokensAsA;
  if (forced == 3) return mmoe::kFamilyTokensAsAPair;
  // CTA pairs are never chosen automatically: measured on B200 at 120 / 240 / 480 rows per expert a pair step takes
  // 1.90 / 1.20 / 1.08 ms against 1.38 / 1.15 / 1.08 ms on single CTAs (the issuing thread pays two commits per stage)
  if (early_shared) return m > 128 ? mmoe::kFamilyTokensAsA : mmoe::kFamilyWeightsAsA;
  // expected rows per expert (the quantity BLOCK_M is chosen from): below ~80 the weights-as-A kernels, whose cost
  // follows the token count, win (and stream more weight bytes per stage when the call is HBM-bound)
  const double expected = (double)m * g->num_ranks * g->num_topk / g->num_experts;
  return block_m >= 64 && expected >= 80.0 ? mmoe::kFamilyTokensAsA : mmoe::kFamilyWeightsAsA;
}

int check_tokens(const MmoeGeometry* g, int m) {
  if (m < 0 || m > g->num_max_tokens) return fail(MMOE_ERR_INVALID_ARGUMENT, "num_tokens=%d outside [0, %d]", m, g->num_max_tokens);
  return MMOE_OK;
}

float bf16_round_host(float v) {
  if (isinf(v) || isnan(v)) return v;
  uint32_t b;
  memcpy(&b, &v, 4);
  b = (b + 0x7FFFu + ((b >> 16) & 1u)) & 0xFFFF0000u;
  memcpy(&v, &b, 4);
  return v;
}

}  // namespace

extern "C" {

int mmoe_abi_version(void) { return 3; }

int mmoe_set_tuning(int32_t max_stages, int32_t orientation) {
  if (max_stages < 0 || max_stages == 1) return fail(MMOE_ERR_INVALID_ARGUMENT, "max_stages=%d must be 0 or >= 2", max_stages);
  if (orientation < 0 || orientation > 3) return fail(MMOE_ERR_INVALID_ARGUMENT, "orientation=%d outside [0, 3]", orientation);
  mmoe::set_tuning(max_stages, orientation);
  return MMOE_OK;
}

const char* mmoe_last_error(void) { return g_last_error.c_str(); }

const char* mmoe_status_string(int code) {
  switch (code) {
    case MMOE_OK: return "ok";
    case MMOE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case MMOE_ERR_UNSUPPORTED: return "unsupported option";
    case MMOE_ERR_CUDA: return "CUDA call failed";
    case MMOE_ERR_ARCH: return "device is not compute capability 10.0 (B200)";
    case MMOE_ERR_NOT_PREPARED: return "mmoe_prepare() has not run";
    case MMOE_ERR_DEVICE_TIMEOUT: return "a device-side wait expired";
    default: return "unknown status";
  }
}

int mmoe_block_m(int32_t num_ranks, int32_t num_experts, int32_t num_tokens, int32_t num_topk) {
  if (num_ranks <= 0 || num_experts <= 0 || num_tokens < 0) return -1;
  // float32 arithmetic, evaluated left to right (backend/heuristics.py:140-157 of the reference)
  volatile float e = static_cast<float>(num_tokens);
  e = e * static_cast<float>(num_ranks);
  e = e * static_cast<float>(num_topk);
  e = e / static_cast<float>(num_experts);
  volatile float root = sqrtf(e);
  volatile float covered = e + root;
  if (e <= 10.f) return 16;
  if (e <= 24.f) return 32;
  volatile float q = covered / 240.f;
  int blocks = static_cast<int>(ceilf(q));
  if (blocks == 1 && covered > 192.f && num_experts / num_ranks < 14) blocks = 2;
  const int cand[4] = {64, 128, 192, 240};
  for (int c : cand)
    if (static_cast<float>(blocks * c) >= covered) return c;
  return 240;
}

int mmoe_layout(const MmoeGeometry* g, MmoeLayout* out) {
  int rc = check_geometry(g);
  if (rc != MMOE_OK) return rc;
  if (out == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "layout output is NULL");
  memset(out, 0, sizeof *out);
  const int64_t T = g->num_max_tokens, H = g->hidden, I = g->intermediate, k = g->num_topk, R = g->num_ranks;
  const int64_t E = g->num_experts, El = E / R;
  const int64_t kmax = k < El ? k : El;
  const int64_t max_routes = T * kmax;          // rows one rank can send
  const int64_t max_recv = R * max_routes;      // rows one rank can receive
  int64_t pool_rows = 0, sf_rows = 0;
  for (int bm : kBlockMs) {
    const int64_t blocks = max_recv / bm + El;
    pool_rows = blocks * bm > pool_rows ? blocks * bm : pool_rows;
    const int64_t rows = blocks * mmoe::chunks_per_block(bm) * 128;
    sf_rows = rows > sf_rows ? rows : sf_rows;
  }
  pool_rows += 128;                              // a tile box may start up to 128 rows before the end of the last block
  const int64_t shared_rows = (T + 7) / 8 * 128;
  const int64_t max_tiles = (max_recv / 16 + El) * 2 + mmoe::shared_tile_capacity(T);
  const bool ep = R > 1;
  const bool shared = g->num_shared_experts > 0;

  int64_t off = 0;
  auto take = [&off](int64_t bytes) {
    const int64_t at = off;
    off = mmoe::align_up(off + (bytes > 0 ? bytes : 0), 1024);
    return at;
  };
  out->x = take(T * H);
  out->x_sf = take(T * (H / 128) * 4);
  out->topk_idx = take(T * k * 8);
  out->topk_weights = take(T * k * 4);
  out->shared_sf_rows = shared_rows;
  out->shared_x_sf = take(shared ? shared_rows * (H / 128) * 4 : 0);
  out->send_count = take(E * 4);
  out->send_offset = take((E + 1) * 4);
  out->route_pos = take(T * k * 4);
  out->sorted_route = take(T * k * 4);
  out->sort_scratch = take(((T + 127) / 128) * E * 4);
  out->recv_count = take(R * El * 4);
  out->plan = take(mmoe::plan_bytes(static_cast<int>(El), static_cast<int>(R), max_tiles));
  out->send_x = take(ep ? max_routes * H : 0);
  out->send_sf = take(ep ? max_routes * (H / 128) * 4 : 0);
  out->send_w = take(ep ? max_routes * 4 : 0);
  out->recv_x = take(ep ? max_recv * H : 0);
  out->recv_sf = take(ep ? max_recv * (H / 128) * 4 : 0);
  out->recv_w = take(ep ? max_recv * 4 : 0);
  out->pool_x = take(pool_rows * H);
  out->pool_sf = take(sf_rows * (H / 128) * 4);
  out->pool_w = take(pool_rows * 4);
  out->pool_dst = take(pool_rows * 4);
  out->act_x = take(pool_rows * I);
  out->act_sf = take(sf_rows * (I / 128) * 4);
  out->shared_act_x = take(shared ? (T + 128) * I : 0);
  out->shared_act_sf = take(shared ? shared_rows * (I / 128) * 4 : 0);
  out->ret = take(max_recv * H * 2);
  out->ret_recv = take(ep ? max_routes * H * 2 : 0);
  out->shared_out = take(shared ? T * H * 2 : 0);
  out->ep_sync = take(ep ? mmoe::ep_sync_bytes() : 0);
  out->status = take(64);
  out->total_bytes = off;
  out->pool_rows = pool_rows;
  out->pool_sf_rows = sf_rows;
  out->max_routes = max_routes;
  out->max_tiles = max_tiles;
  return MMOE_OK;
}

int mmoe_prepare(const MmoeGeometry* geo, int32_t* block_ms, int32_t cap, int32_t* n, void* stream) {
  int rc = check_geometry(geo);
  if (rc != MMOE_OK) return rc;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  int major = 0, minor = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  if (major != 10 || minor != 0) return fail(MMOE_ERR_ARCH, "compute capability %d.%d, need 10.0", major, minor);
  cudaStreamCaptureStatus cap_status = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &cap_status) != cudaSuccess || cap_status != cudaStreamCaptureStatusNone)
    return fail(MMOE_ERR_NOT_PREPARED, "mmoe_prepare() called while the stream is capturing");
  rc = mmoe::prepare_umma(*geo);
  if (rc != MMOE_OK) return fail(rc, "loading the tensor-core kernels failed: %s", cudaGetErrorString(cudaGetLastError()));
  side_lane(true);                              // streams and events cannot be created while a stream is capturing
  // every BLOCK_M the geometry can select for M in [0, T]
  bool seen[6] = {false, false, false, false, false, false};
  for (int m = 0; m <= geo->num_max_tokens; ++m) {
    const int bm = mmoe_block_m(geo->num_ranks, geo->num_experts, m, geo->num_topk);
    for (int i = 0; i < 6; ++i)
      if (kBlockMs[i] == bm) seen[i] = true;
  }
  int count = 0;
  for (int i = 0; i < 6; ++i)
    if (seen[i]) {
      if (block_ms != nullptr && count < cap) block_ms[count] = kBlockMs[i];
      ++count;
    }
  if (n != nullptr) *n = count;
  return MMOE_OK;
}

int mmoe_stage_inputs(const MmoeGeometry* geo, void* workspace, const void* hidden_bf16, const void* topk_ids,
                      int32_t ids_are_int64, const float* topk_weights, const uint8_t* is_padding, int32_t num_tokens,
                      int32_t shared_block_m, void* stream) {
  mmoe::ChainScope chain(num_tokens <= 128);
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (num_tokens == 0) return MMOE_OK;
  if (hidden_bf16 == nullptr || topk_ids == nullptr || topk_weights == nullptr)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "staging inputs must not be NULL");
  if ((reinterpret_cast<uintptr_t>(hidden_bf16) & 15u) != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "hidden states must be 16-byte aligned");
  if (shared_block_m > 0 && !valid_block_m(shared_block_m))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "shared_block_m=%d is not a BLOCK_M value", shared_block_m);
  cudaError_t e = mmoe::launch_stage(c, hidden_bf16, topk_ids, ids_are_int64, topk_weights, is_padding, num_tokens,
                                     shared_block_m, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "stage_inputs launch");
}

int mmoe_route_stage_inputs(const MmoeGeometry* geo, void* workspace, const void* hidden_bf16, const float* router_logits,
                            int32_t num_logical_experts, const int32_t* replica_count, const int32_t* replica_slots,
                            int32_t max_copies, const uint8_t* is_padding, int32_t num_tokens, int32_t shared_block_m,
                            void* stream) {
  mmoe::ChainScope chain(num_tokens <= 128);
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (num_logical_experts < geo->num_topk || num_logical_experts > 2048)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "num_logical_experts=%d outside [num_topk, 2048]", num_logical_experts);
  if ((replica_count == nullptr) != (replica_slots == nullptr) || (replica_count != nullptr && max_copies < 1))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "the replica table needs counts, slots and max_copies >= 1 together");
  if (replica_count == nullptr && num_logical_experts > geo->num_experts)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "without a replica table logical ids are physical ids: num_logical_experts=%d > num_experts=%d",
                num_logical_experts, geo->num_experts);
  if (num_tokens == 0) return MMOE_OK;
  if (hidden_bf16 == nullptr || router_logits == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "staging inputs must not be NULL");
  if ((reinterpret_cast<uintptr_t>(hidden_bf16) & 15u) != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "hidden states must be 16-byte aligned");
  if (shared_block_m > 0 && !valid_block_m(shared_block_m))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "shared_block_m=%d is not a BLOCK_M value", shared_block_m);
  cudaError_t e = mmoe::launch_route_stage(c, hidden_bf16, nullptr, 0, nullptr, router_logits, num_logical_experts, replica_count,
                                           replica_slots, max_copies, is_padding, num_tokens, shared_block_m,
                                           static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "route_stage_inputs launch");
}

int mmoe_stage_inputs_nvfp4(const void* hidden_bf16, float global_scale, void* q_out, void* sf_out, int32_t num_tokens,
                            int32_t hidden, void* stream) {
  if (num_tokens < 0 || hidden <= 0 || hidden % 16 != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "nvfp4 staging: num_tokens=%d must be >= 0 and hidden=%d a positive multiple of 16", num_tokens, hidden);
  if (!(global_scale > 0.f) || isinf(global_scale)) return fail(MMOE_ERR_INVALID_ARGUMENT, "nvfp4 staging: global_scale must be positive and finite");
  if (num_tokens == 0) return MMOE_OK;
  if (hidden_bf16 == nullptr || q_out == nullptr || sf_out == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "nvfp4 staging: pointers must not be NULL");
  if ((reinterpret_cast<uintptr_t>(hidden_bf16) & 15u) != 0 || (reinterpret_cast<uintptr_t>(q_out) & 7u) != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "nvfp4 staging: hidden states must be 16-byte and the packed output 8-byte aligned");
  cudaError_t e = mmoe::launch_stage_nvfp4(hidden_bf16, q_out, sf_out, global_scale, num_tokens, hidden, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "nvfp4 staging launch");
}

int mmoe_dispatch_count(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  cudaError_t e = mmoe::launch_count_sort(c, num_tokens, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "dispatch_count launch");
}

int mmoe_route_order_noalloc(const int64_t* topk_idx, int32_t num_tokens, int32_t num_topk, int32_t num_experts,
                             int32_t* send_count, int32_t* send_offset, int32_t* route_pos, int32_t* sorted_route,
                             void* stream) {
  const int max_t = mmoe::route_order_static_max_tokens(), max_e = mmoe::route_order_static_max_experts();
  if (num_tokens < 0 || num_tokens > max_t)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "num_tokens=%d exceeds the built-in scratch of mmoe_route_order_noalloc (at most %d tokens)", num_tokens, max_t);
  if (num_experts < 1 || num_experts > max_e)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "num_experts=%d exceeds the built-in scratch of mmoe_route_order_noalloc (at most %d experts)", num_experts, max_e);
  if (num_topk < 1 || num_topk > 31) return fail(MMOE_ERR_INVALID_ARGUMENT, "num_topk=%d outside [1, 31]", num_topk);
  if (send_count == nullptr || send_offset == nullptr || (num_tokens > 0 && (topk_idx == nullptr || route_pos == nullptr || sorted_route == nullptr)))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "mmoe_route_order_noalloc: input and output pointers must not be NULL");
  cudaError_t e = mmoe::route_order_static(topk_idx, num_tokens, num_topk, num_experts, send_count, send_offset, route_pos,
                                           sorted_route, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "route_order_noalloc");
}

int mmoe_dispatch_pack(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (geo->num_ranks == 1) return MMOE_OK;
  cudaError_t e = mmoe::launch_pack(c, num_tokens, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "dispatch_pack launch");
}

static int check_peers(const MmoeGeometry* geo, void* workspace, const void* const* peers) {
  if (geo->num_ranks < 2) return fail(MMOE_ERR_INVALID_ARGUMENT, "the peer exchange needs num_ranks > 1");
  if (peers == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "peer_workspaces is NULL");
  for (int r = 0; r < geo->num_ranks; ++r)
    if (peers[r] == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "peer_workspaces[%d] is NULL", r);
  if (peers[geo->rank] != workspace) return fail(MMOE_ERR_INVALID_ARGUMENT, "peer_workspaces[rank] must be this rank's workspace");
  return MMOE_OK;
}

int mmoe_ep_dispatch(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces, int32_t num_tokens,
                     const MmoeOptions* opt, void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc == MMOE_OK) rc = check_tokens(geo, num_tokens);
  if (rc == MMOE_OK) rc = check_peers(geo, workspace, peer_workspaces);
  if (rc != MMOE_OK) return rc;
  const int64_t timeout_ns = (opt != nullptr && opt->timeout_ms > 0 ? (int64_t)opt->timeout_ms : 2000) * 1000000ll;
  cudaError_t e = mmoe::launch_ep_dispatch(c, peer_workspaces, num_tokens, timeout_ns, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "ep_dispatch launch");
}

int mmoe_ep_return(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces, const MmoeOptions* opt,
                   void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc == MMOE_OK) rc = check_peers(geo, workspace, peer_workspaces);
  if (rc != MMOE_OK) return rc;
  const int64_t timeout_ns = (opt != nullptr && opt->timeout_ms > 0 ? (int64_t)opt->timeout_ms : 2000) * 1000000ll;
  cudaError_t e = mmoe::launch_ep_return(c, peer_workspaces, timeout_ns, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "ep_return launch");
}

int mmoe_dispatch_place(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, int32_t block_m, int32_t* stats,
                        void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (!valid_block_m(block_m)) return fail(MMOE_ERR_INVALID_ARGUMENT, "block_m=%d is not a BLOCK_M value", block_m);
  c.family = choose_family(geo, num_tokens, block_m, false);
  cudaError_t e = mmoe::launch_plan_place(c, num_tokens, block_m, stats, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "dispatch_place launch");
}

namespace {
// `peers` != NULL: EP > 1 with the write-back fused into GEMM2, followed by barrier 2
int run_experts(const MmoeGeometry* geo, void* workspace, const void* const* peers, const MmoeWeights* weights,
                const MmoeOptions* opt, int32_t num_tokens, int32_t block_m, void* stream, int tile_select = 0);

}  // namespace

int mmoe_experts(const MmoeGeometry* geo, void* workspace, const MmoeWeights* weights, const MmoeOptions* opt,
                 int32_t num_tokens, int32_t block_m, void* stream) {
  return run_experts(geo, workspace, nullptr, weights, opt, num_tokens, block_m, stream);
}

int mmoe_plan_shared(const MmoeGeometry* geo, void* workspace, int32_t num_tokens, int32_t block_m, void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc == MMOE_OK) rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (!valid_block_m(block_m)) return fail(MMOE_ERR_INVALID_ARGUMENT, "block_m=%d is not a BLOCK_M value", block_m);
  c.family = choose_family(geo, num_tokens, block_m, true);
  cudaError_t e = mmoe::launch_shared_plan(c, num_tokens, block_m, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "shared plan launch");
}

int mmoe_experts_select(const MmoeGeometry* geo, void* workspace, const MmoeWeights* weights, const MmoeOptions* opt,
                        int32_t num_tokens, int32_t block_m, int32_t tile_select, void* stream) {
  if (tile_select < 0 || tile_select > 2) return fail(MMOE_ERR_INVALID_ARGUMENT, "tile_select=%d outside [0, 2]", tile_select);
  if (opt != nullptr && opt->engine != 0 && tile_select != 0)
    return fail(MMOE_ERR_UNSUPPORTED, "only the tensor-core engine can run a subset of the tiles");
  return run_experts(geo, workspace, nullptr, weights, opt, num_tokens, block_m, stream, tile_select);
}

int mmoe_experts_ep_return(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces,
                           const MmoeWeights* weights, const MmoeOptions* opt, int32_t num_tokens, int32_t block_m,
                           void* stream) {
  if (geo == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "geometry is NULL");
  int rc = check_peers(geo, workspace, peer_workspaces);
  if (rc != MMOE_OK) return rc;
  if (geo->num_ranks < 2) return fail(MMOE_ERR_INVALID_ARGUMENT, "the fused write-back needs num_ranks > 1");
  if (opt != nullptr && opt->layer_mask != 0 && opt->layer_mask != 3)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "the fused write-back runs both layers (layer_mask 0 or 3)");
  return run_experts(geo, workspace, peer_workspaces, weights, opt, num_tokens, block_m, stream);
}

namespace {
int run_experts(const MmoeGeometry* geo, void* workspace, const void* const* peers, const MmoeWeights* weights,
                const MmoeOptions* opt, int32_t num_tokens, int32_t block_m, void* stream, int tile_select) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (weights == nullptr || opt == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "weights / options are NULL");
  if (!valid_block_m(block_m)) return fail(MMOE_ERR_INVALID_ARGUMENT, "block_m=%d is not a BLOCK_M value", block_m);
  if (weights->w13 == nullptr || weights->w13_sf == nullptr || weights->w2 == nullptr || weights->w2_sf == nullptr)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "routed expert weights must not be NULL");
  if (geo->num_shared_experts > 0 && (weights->shared_w13 == nullptr || weights->shared_w13_sf == nullptr ||
                                      weights->shared_w2 == nullptr || weights->shared_w2_sf == nullptr))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "shared expert weights must not be NULL when num_shared_experts > 0");
  const void* aligned[] = {weights->w13, weights->w13_sf, weights->w2, weights->w2_sf, weights->shared_w13,
                           weights->shared_w13_sf, weights->shared_w2, weights->shared_w2_sf};
  for (const void* p : aligned)
    if ((reinterpret_cast<uintptr_t>(p) & 31u) != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "weight tensors must be 32-byte aligned");
  if (weights->w13_slice_stride < 0 || weights->w2_slice_stride < 0 ||
      (weights->w13_slice_stride > 0 && geo->intermediate % 256 != 0))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "two-slice W13 needs intermediate %% 256 == 0 and non-negative slice strides");
  if (!(opt->activation_clamp > 0.f)) return fail(MMOE_ERR_INVALID_ARGUMENT, "activation_clamp must be positive (use +inf for none)");
  MmoeOptions o = *opt;
  if (o.layer_mask < 0 || o.layer_mask > 3) return fail(MMOE_ERR_INVALID_ARGUMENT, "layer_mask=%d outside [0, 3]", o.layer_mask);
  o.activation_clamp = bf16_round_host(o.activation_clamp);   // the clamp is applied to BF16 values
  const int64_t timeout_ns = (o.timeout_ms > 0 ? (int64_t)o.timeout_ms : 2000) * 1000000ll;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (o.engine == 1) {
    // the scalar validation engine writes the local return buffer; the rows then go home with the copy kernel
    e = mmoe::launch_experts_simt(c, *weights, o, num_tokens, block_m, st);
    if (e == cudaSuccess && peers != nullptr) e = mmoe::launch_ep_return(c, peers, timeout_ns, st);
  } else if (o.engine == 0) {
    if (!mmoe::tc_ready()) return fail(MMOE_ERR_NOT_PREPARED, "mmoe_prepare() must run on this device before the first launch");
    c.peer_ws = peers;
    c.tile_select = tile_select;
    c.family = choose_family(geo, num_tokens, block_m, tile_select == 2);
    e = mmoe::launch_experts_umma(c, *weights, o, num_tokens, block_m, st);
    if (e == cudaSuccess && peers != nullptr) e = mmoe::launch_ep_signal_return(c, peers, timeout_ns, st);
  } else {
    return fail(MMOE_ERR_UNSUPPORTED, "engine=%d", o.engine);
  }
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "experts launch");
}
}  // namespace

int mmoe_combine_residual(const MmoeGeometry* geo, void* workspace, void* y_bf16, const void* residual_bf16,
                          int32_t num_tokens, void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  rc = check_tokens(geo, num_tokens);
  if (rc != MMOE_OK) return rc;
  if (num_tokens > 0 && (y_bf16 == nullptr || (reinterpret_cast<uintptr_t>(y_bf16) & 15u) != 0))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "y must be a 16-byte aligned device pointer");
  if ((reinterpret_cast<uintptr_t>(residual_bf16) & 15u) != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "the residual must be a 16-byte aligned device pointer");
  cudaError_t e = mmoe::launch_combine(c, y_bf16, residual_bf16, num_tokens, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "combine launch");
}

int mmoe_combine(const MmoeGeometry* geo, void* workspace, void* y_bf16, int32_t num_tokens, void* stream) {
  return mmoe_combine_residual(geo, workspace, y_bf16, nullptr, num_tokens, stream);
}

int mmoe_forward(const MmoeGeometry* geo, void* workspace, const MmoeWeights* weights, const MmoeOptions* opt,
                 void* y_bf16, int32_t num_tokens, int32_t block_m, int32_t* stats, void* stream) {
  mmoe::ChainScope chain(num_tokens <= 128);
  if (geo != nullptr && geo->num_ranks != 1)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "mmoe_forward is the single-rank sequence; call mmoe_forward_ep for num_ranks > 1");
  const bool decode = geo != nullptr && num_tokens > 0 && num_tokens <= 128 && geo->num_experts <= 512 &&
                      valid_block_m(block_m) && workspace != nullptr;
  // route ordering, plan and placement of the routed experts on stream `st`
  auto dispatch = [&](void* st) -> int {
    if (decode) {                       // one launch orders the routes and builds the plan
      mmoe::Ctx c;
      int r = make_ctx(geo, workspace, &c);
      if (r != MMOE_OK) return r;
      c.family = choose_family(geo, num_tokens, block_m, false);
      cudaError_t e = mmoe::launch_route_plan_place_small(c, num_tokens, block_m, stats, static_cast<cudaStream_t>(st));
      return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "route/plan launch");
    }
    int r = mmoe_dispatch_count(geo, workspace, num_tokens, st);
    if (r == MMOE_OK) r = mmoe_dispatch_place(geo, workspace, num_tokens, block_m, stats, st);
    return r;
  };
  cudaStream_t main_stream = static_cast<cudaStream_t>(stream);
  SideLane* lane = nullptr;
  // (only past the decode sizes: at a handful of tokens the three extra launches cost more than the overlap gains --
  // measured 61 -> 82 us at M=1, 1.742 -> 1.719 ms at M=3840)
  if (geo != nullptr && opt != nullptr && opt->engine == 0 && geo->num_shared_experts > 0 && num_tokens > 128 &&
      (opt->layer_mask == 0 || opt->layer_mask == 3)) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(main_stream, &cap);
    lane = side_lane(cap == cudaStreamCaptureStatusNone);
  }
  int rc;
  if (lane == nullptr) {
    rc = dispatch(stream);
    if (rc == MMOE_OK) rc = mmoe_experts(geo, workspace, weights, opt, num_tokens, block_m, stream);
    if (rc == MMOE_OK) rc = mmoe_combine_residual(geo, workspace, y_bf16, opt != nullptr ? opt->residual : nullptr, num_tokens, stream);
    return rc;
  }
  // The shared expert needs only the staged tokens: its two GEMMs run here while the routed experts' ordering, plan
  // and placement run on the library's second stream (fork / join with events, capturable).
  cudaError_t e = cudaEventRecord(lane->fork, main_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(lane->stream, lane->fork, 0);
  if (e != cudaSuccess) return cuda_fail(e, "forking the dispatch stream");
  mmoe::break_chain();                      // the side stream's first kernel follows an event, not a kernel
  const int rc_side = dispatch(lane->stream);
  e = cudaEventRecord(lane->join, lane->stream);
  rc = mmoe_plan_shared(geo, workspace, num_tokens, block_m, stream);
  if (rc == MMOE_OK) rc = run_experts(geo, workspace, nullptr, weights, opt, num_tokens, block_m, stream, 2);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(main_stream, lane->join, 0);
  if (e != cudaSuccess) return cuda_fail(e, "joining the dispatch stream");
  mmoe::break_chain();                      // the next kernel has two predecessors: launch it without the attribute
  if (rc_side != MMOE_OK) return rc_side;
  if (rc == MMOE_OK) rc = run_experts(geo, workspace, nullptr, weights, opt, num_tokens, block_m, stream, 1);
  if (rc == MMOE_OK) rc = mmoe_combine_residual(geo, workspace, y_bf16, opt != nullptr ? opt->residual : nullptr, num_tokens, stream);
  return rc;
}

int mmoe_forward_ep(const MmoeGeometry* geo, void* workspace, const void* const* peer_workspaces,
                    const MmoeWeights* weights, const MmoeOptions* opt, void* y_bf16, int32_t num_tokens, int32_t block_m,
                    int32_t* stats, void* stream) {
  if (geo == nullptr || opt == nullptr) return fail(MMOE_ERR_INVALID_ARGUMENT, "geometry / options are NULL");
  if (geo->num_ranks < 2) return fail(MMOE_ERR_INVALID_ARGUMENT, "mmoe_forward_ep is the num_ranks > 1 sequence");
  int rc = check_peers(geo, workspace, peer_workspaces);
  if (rc == MMOE_OK && !valid_block_m(block_m)) rc = fail(MMOE_ERR_INVALID_ARGUMENT, "block_m=%d is not a BLOCK_M value", block_m);
  if (rc == MMOE_OK) rc = mmoe_dispatch_count(geo, workspace, num_tokens, stream);
  if (rc != MMOE_OK) return rc;
  cudaStream_t main_stream = static_cast<cudaStream_t>(stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(main_stream, &cap);
  SideLane* lane = nullptr;
  if (opt->engine == 0 && geo->num_shared_experts > 0 && num_tokens > 0)
    lane = side_lane(cap == cudaStreamCaptureStatusNone);
  if (lane == nullptr) {
    // nothing to overlap (no shared expert, no tokens here, validation engine): one stream
    rc = mmoe_ep_dispatch(geo, workspace, peer_workspaces, num_tokens, opt, stream);
    if (rc == MMOE_OK) rc = mmoe_dispatch_place(geo, workspace, num_tokens, block_m, stats, stream);
    if (rc == MMOE_OK) rc = run_experts(geo, workspace, peer_workspaces, weights, opt, num_tokens, block_m, stream, 0);
    if (rc == MMOE_OK) rc = mmoe_combine_residual(geo, workspace, y_bf16, opt != nullptr ? opt->residual : nullptr, num_tokens, stream);
    return rc;
  }
  // fork: the exchange of counts and rows runs on the side stream ...
  cudaError_t e = cudaEventRecord(lane->fork, main_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(lane->stream, lane->fork, 0);
  if (e != cudaSuccess) return cuda_fail(e, "forking the dispatch stream");
  const int rc_side = mmoe_ep_dispatch(geo, workspace, peer_workspaces, num_tokens, opt, lane->stream);
  e = cudaEventRecord(lane->join, lane->stream);
  // ... while the shared expert, which needs only this rank's own tokens, runs both of its GEMMs here
  mmoe::Ctx c;
  rc = make_ctx(geo, workspace, &c);
  if (rc == MMOE_OK) c.family = choose_family(geo, num_tokens, block_m, true);
  if (rc == MMOE_OK && mmoe::launch_shared_plan(c, num_tokens, block_m, main_stream) != cudaSuccess)
    rc = cuda_fail(cudaGetLastError(), "shared plan launch");
  if (rc == MMOE_OK) rc = run_experts(geo, workspace, nullptr, weights, opt, num_tokens, block_m, stream, 2);
  // join (always, so that a capture is never left forked)
  if (e == cudaSuccess) e = cudaStreamWaitEvent(main_stream, lane->join, 0);
  if (e != cudaSuccess) return cuda_fail(e, "joining the dispatch stream");
  if (rc_side != MMOE_OK) return rc_side;
  if (rc == MMOE_OK) rc = mmoe_dispatch_place(geo, workspace, num_tokens, block_m, stats, stream);
  if (rc == MMOE_OK) rc = run_experts(geo, workspace, peer_workspaces, weights, opt, num_tokens, block_m, stream, 1);
  if (rc == MMOE_OK) rc = mmoe_combine_residual(geo, workspace, y_bf16, opt != nullptr ? opt->residual : nullptr, num_tokens, stream);
  return rc;
}


int mmoe_transform_weights(const void* w_in, void* w_out, const int32_t* sf_in, int32_t* sf_out, int32_t num_groups,
                           int32_t rows, int32_t k_packed_bytes, int32_t k_words, int32_t interleave, void* stream) {
  if (num_groups <= 0 || rows <= 0 || k_packed_bytes <= 0 || k_words <= 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: sizes must be positive");
  if (rows % 128 != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: rows=%d is not a multiple of 128", rows);
  if (interleave && rows % 16 != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: gate/up interleave needs rows %% 16 == 0");
  if (k_packed_bytes % 16 != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: a weight row must be a multiple of 16 bytes");
  if (sf_in == nullptr || sf_out == nullptr || sf_in == sf_out) return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: scale pointers must be distinct and non-NULL");
  if (interleave && (w_in == nullptr || w_out == nullptr || w_in == w_out))
    return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: weight pointers must be distinct and non-NULL when rows are interleaved");
  const void* ptrs[] = {w_in, w_out, sf_in, sf_out};
  for (const void* p : ptrs)
    if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return fail(MMOE_ERR_INVALID_ARGUMENT, "transform: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  if (interleave) e = mmoe::launch_interleave_rows(w_in, w_out, num_groups, rows, k_packed_bytes, st);
  if (e == cudaSuccess) e = mmoe::launch_scale_layout(sf_in, sf_out, num_groups, rows, rows, k_words, interleave, st);
  return e == cudaSuccess ? MMOE_OK : cuda_fail(e, "weight transform launch");
}

int mmoe_read_status(const MmoeGeometry* geo, void* workspace, int32_t* words8, void* stream) {
  mmoe::Ctx c;
  int rc = make_ctx(geo, workspace, &c);
  if (rc != MMOE_OK) return rc;
  int32_t host[8];
  cudaError_t e = cudaMemcpyAsync(host, c.ws + c.lay.status, sizeof host, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  // clear on read: the words are sticky on the device, so that a later healthy call is reported as healthy
  if (e == cudaSuccess) e = cudaMemsetAsync(c.ws + c.lay.status, 0, sizeof host, static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "reading the status words");
  if (words8 != nullptr) memcpy(words8, host, sizeof host);
  if (host[mmoe::kStatusTimeout] != 0)
    return fail(MMOE_ERR_DEVICE_TIMEOUT, "device wait expired: kernel %d role %d block %d", host[mmoe::kStatusKernel],
                host[mmoe::kStatusRole], host[mmoe::kStatusBlock]);
  if (host[mmoe::kStatusBadIndex] != 0)
    return fail(MMOE_ERR_INVALID_ARGUMENT, "%d expert ids were >= num_experts", host[mmoe::kStatusBadIndex]);
  return MMOE_OK;
}

}  // extern "C"
