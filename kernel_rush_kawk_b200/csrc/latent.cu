// Kernels of attention over one cached low-rank row per token.
//
// krk_latent_norm_write: one warp per row. The row's `rank` projected elements are divided by their root
// mean square (eps under the root), multiplied by a float32 gain and written, rounded once, to the
// position's place in a cache of one "kv head" of `rank` elements (and, if asked, to a plain row buffer as well).
//
// krk_head_linear: out[r, h, :] = scale * W_h x[r, h, :] for every head h, W [heads, N, K] contiguous;
// x and out are rows with strides. One block per (tile of output elements, head, tile of 8 rows): the
// rows' slices sit in shared memory as float32, each warp owns output elements, its lanes split K
// (coalesced reads of W's rows), sums are float32 and their order does not depend on the other rows.
#include "common.cuh"

namespace {

template <typename T>
__global__ void latent_norm_write_kernel(const T* __restrict__ proj, int stride, int c_col, int R,
                                         const float* __restrict__ gain, float eps, const int* __restrict__ row_seq,
                                         const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                                         const int* __restrict__ table, int width, int keep_pages, T* cache, int rows,
                                         T* __restrict__ rows_out) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* c = proj + (size_t)row * stride + c_col;
  float sq = 0.f;
  for (int i = lane; i < R; i += 32) {
    const float f = to_float<T>(c[i]);
    sq += f * f;
  }
  const float rstd = rsqrtf(warp_sum(sq) / (float)R + eps);
  const int pos = row_pos[row];
  const int page = page_of(table, width, seq_slot[row_seq[row]], pos, keep_pages);
  T* dst = cache + ((size_t)page * KRK_PAGE + (pos % KRK_PAGE)) * R;
  for (int i = lane; i < R; i += 32) {
    const T v = from_float<T>(to_float<T>(c[i]) * rstd * gain[i]);
    dst[i] = v;
    if (rows_out) rows_out[(size_t)row * R + i] = v;
  }
}

constexpr int HL_ROWS = 8;
constexpr int HL_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(HL_WARPS * 32)
head_linear_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale, const T* __restrict__ x,
                   int x_stride, const T* __restrict__ w, int N, int K, int rows) {
  extern __shared__ __align__(16) float xs[];  // [HL_ROWS][K4], K4 = K rounded up to a multiple of 4
  const int K4 = (K + 3) & ~3;
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.y, r0 = blockIdx.z * HL_ROWS;
  const int nr = min(HL_ROWS, rows - r0);
  for (int i = threadIdx.x; i < HL_ROWS * K; i += blockDim.x) {
    const int r = i / K, k = i - r * K;
    xs[r * K4 + k] = r < nr ? to_float<T>(x[(size_t)(r0 + r) * x_stride + (size_t)h * K + k]) : 0.f;
  }
  __syncthreads();
  for (int n = blockIdx.x * HL_WARPS + warp; n < N; n += gridDim.x * HL_WARPS) {
    const T* wr = w + ((size_t)h * N + n) * K;
    float mine = 0.f;
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) {
      if (r >= nr) break;
      const float t = warp_sum(lane_dot<T>(wr, xs + r * K4, K, lane));  // the weight row comes from L1 after the first
      if (lane == r) mine = t;
    }
    if (lane < nr) out[(size_t)(r0 + lane) * out_stride + out_col + (size_t)h * N + n] = from_float<T>(mine * out_scale);
  }
}

}  // namespace

KRK_API int krk_latent_norm_write(const void* proj, int stride, int c_col, int R, const float* gain, float eps,
                                  const int* row_seq, const int* row_pos, const int* seq_slot, const int* table, int width,
                                  int keep_pages, void* cache, int rows, void* rows_out, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  const int warps = 4;
  const unsigned blocks = (unsigned)((rows + warps - 1) / warps);
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(latent_norm_write_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, (const float*)proj,
                           stride, c_col, R, gain, eps, row_seq, row_pos, seq_slot, table, width, keep_pages,
                           (float*)cache, rows, (float*)rows_out);
  return (int)launch_pdl(latent_norm_write_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, (const bf16*)proj,
                         stride, c_col, R, gain, eps, row_seq, row_pos, seq_slot, table, width, keep_pages, (bf16*)cache,
                         rows, (bf16*)rows_out);
}

KRK_API int krk_head_linear(void* out, int out_stride, int out_col, float out_scale, const void* x, int x_stride,
                            const void* w, int heads, int N, int K, int rows, int dtype, cudaStream_t stream) {
  if (rows == 0 || heads == 0 || N == 0) return 0;
  const size_t smem = (size_t)HL_ROWS * ((K + 3) & ~3) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(head_linear_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(head_linear_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const int row_tiles = (rows + HL_ROWS - 1) / HL_ROWS;
  if (heads > 65535 || row_tiles > 65535) return -3;
  const dim3 grid((unsigned)((N + HL_WARPS - 1) / HL_WARPS), (unsigned)heads, (unsigned)row_tiles);
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(head_linear_kernel<float>, grid, dim3(HL_WARPS * 32), smem, stream, (float*)out, out_stride,
                           out_col, out_scale, (const float*)x, x_stride, (const float*)w, N, K, rows);
  return (int)launch_pdl(head_linear_kernel<bf16>, grid, dim3(HL_WARPS * 32), smem, stream, (bf16*)out, out_stride, out_col,
                         out_scale, (const bf16*)x, x_stride, (const bf16*)w, N, K, rows);
}
