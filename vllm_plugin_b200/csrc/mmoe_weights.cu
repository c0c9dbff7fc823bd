// Load-time weight transform of the MegaMoE layer as CUDA kernels for sm_100a: the byte shuffles that turn checkpoint-
// order expert weights into the layout the grouped GEMMs read (the reference does them with torch indexing ops,
// backend/weights.py:83-145).
//
//   rows     W13 [gate | up] -> [g0..7, u0..7, g8..15, u8..15, ...] per expert (W2 rows are copied unchanged)
//   scales   int32 words (four UE8M0 bytes each), MN-major [G][K/128][rows]: the same row interleave for W13, then
//            inside every 128-row block the 4x32 transpose (stored position 4c + a holds row 32a + c), which makes each
//            (128 rows, 128 K) block one contiguous 512-byte chunk in the order tcgen05.cp copies into tensor memory
//
// Pure HBM-bound byte movement: every input byte is read once and written once.
#include "mmoe_common.cuh"

namespace mmoe {

namespace {

// source row (in [gate | up] order) of output row r of a matrix with `rows` rows (rows/2 gate + rows/2 up channels)
__device__ __forceinline__ int interleave_src_row(int r, int rows) {
  const int channel = ((r >> 4) << 3) | (r & 7);
  return ((r >> 3) & 1) * (rows >> 1) + channel;
}

// One warp per output row; four 16-byte loads in flight per lane.
__global__ void __launch_bounds__(256) interleave_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                              int64_t total_rows, int rows, int vec) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < total_rows; row += warps) {
    const int64_t g = row / rows;
    const int r = static_cast<int>(row - g * rows);
    const uint4* s = src + (g * rows + interleave_src_row(r, rows)) * vec;
    uint4* d = dst + row * vec;
    for (int v0 = lane; v0 < vec; v0 += 128) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + 32 * u < vec) q[u] = s[v0 + 32 * u];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + 32 * u < vec) d[v0 + 32 * u] = q[u];
    }
  }
}

// One thread per scale word; consecutive threads write consecutive words of a K column.
// Word (g, w, p) of the output (p = stored position) comes from row  blk*128 + 32*(p%4) + (p%128)/4  of the input,
// after the optional gate/up interleave.
__global__ void __launch_bounds__(256) scale_layout_kernel(const int32_t* __restrict__ src, int32_t* __restrict__ dst,
                                                           int64_t total, int rows, int row_stride, int kwords,
                                                           int interleave) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int p = static_cast<int>(i % rows);
    const int64_t gw = i / rows;                     // g * kwords + w
    const int in_block = p & 127;
    int r = (p & ~127) + 32 * (in_block & 3) + (in_block >> 2);
    if (interleave) r = interleave_src_row(r, rows);
    dst[gw * row_stride + p] = src[gw * row_stride + r];
  }
}

}  // namespace

cudaError_t launch_interleave_rows(const void* src, void* dst, int groups, int rows, int row_bytes, cudaStream_t s) {
  const int64_t total = (int64_t)groups * rows;
  if (total == 0) return cudaSuccess;
  const int blocks = static_cast<int>(total / 8 + 1 < 148 * 16 ? total / 8 + 1 : 148 * 16);
  interleave_rows_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), total, rows,
                                               row_bytes / 16);
  return cudaGetLastError();
}

cudaError_t launch_scale_layout(const int32_t* src, int32_t* dst, int groups, int rows, int row_stride, int kwords,
                                int interleave, cudaStream_t s) {
  const int64_t total = (int64_t)groups * kwords * rows;
  if (total == 0) return cudaSuccess;
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  scale_layout_kernel<<<blocks, 256, 0, s>>>(src, dst, total, rows, row_stride, kwords, interleave);
  return cudaGetLastError();
}

}  // namespace mmoe
