// Windowed grouped-query attention with a softmax sink over the paged cache, for heads
// whose key and value sizes are run-time arguments and may differ.
//
// krk_rotate_norm_write: one warp per (row, head). A query head is rotated in place; a
// key head is rotated and written to its page; a value head is (optionally) divided by
// its root mean square and written to its page. Rotation: the first `rot` elements, element
// i with element i + rot/2, by the angle position * f_i. f_i arrives as two floats (its float32
// value and the rest of its float64 value); the product's float32 value goes through sincosf (not
// the fast forms) and the product's rounding error and the rest of f_i correct sine and cosine to
// first order, so that an angle of a thousand radians is as exact as one of a few.
//
// krk_sink_attention: one warp per (row, head). The warp takes 32 keys at a time, one key
// per lane: each lane's score is its own ordered sum over the head, the softmax runs online
// over the chunks with the sink as the starting state (maximum = sink, sum = 1, no value), and
// the weights, kept in float32, multiply the values with the lanes spread over the value
// head. A row's result depends on that row's keys only, in their order, so it is the same to
// the bit however the tokens were cut into steps or batched.
#include "common.cuh"

namespace {

constexpr int MAX_V_PER_LANE = 8;  // value heads up to 256

// sine and cosine of p * (f_hi + f_lo)
__device__ __forceinline__ void angle_sincos(float p, float f_hi, float f_lo, float* s, float* c) {
  const float a = __fmul_rn(p, f_hi);
  const float e = fmaf(p, f_hi, -a) + p * f_lo;
  float s0, c0;
  sincosf(a, &s0, &c0);
  *s = fmaf(e, c0, s0);
  *c = fmaf(-e, s0, c0);
}

template <typename T>
__global__ void rotate_norm_write_kernel(T* proj, int stride, int q_col, int k_col, int v_col, int HQ, int HKV, int D,
                                         int DV, const float* __restrict__ inv_freq, int rot, int value_norm, float eps,
                                         const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                         const int* __restrict__ seq_slot, const int* __restrict__ table, int width,
                                         T* k_cache, T* v_cache, int rows) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int per_row = HQ + 2 * HKV;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)rows * per_row) return;
  const int row = (int)(item / per_row), which = (int)(item % per_row);
  const int pos = row_pos[row];
  const float p = (float)pos;
  const int half = rot >> 1;
  T* src = proj + (size_t)row * stride;
  if (which < HQ) {
    T* q = src + q_col + (size_t)which * D;
    for (int i = lane; i < half; i += 32) {
      float s, c;
      angle_sincos(p, inv_freq[i], inv_freq[half + i], &s, &c);
      const float u = to_float<T>(q[i]), v = to_float<T>(q[i + half]);
      q[i] = from_float<T>(u * c - v * s);
      q[i + half] = from_float<T>(v * c + u * s);
    }
    return;
  }
  const int slot = seq_slot[row_seq[row]];
  const int page = page_of(table, width, slot, pos);
  if (which < HQ + HKV) {
    const int h = which - HQ;
    const T* k = src + k_col + (size_t)h * D;
    T* dst = k_cache + (((size_t)page * HKV + h) * KRK_PAGE + (pos % KRK_PAGE)) * D;
    for (int i = lane; i < half; i += 32) {
      float s, c;
      angle_sincos(p, inv_freq[i], inv_freq[half + i], &s, &c);
      const float u = to_float<T>(k[i]), v = to_float<T>(k[i + half]);
      dst[i] = from_float<T>(u * c - v * s);
      dst[i + half] = from_float<T>(v * c + u * s);
    }
    for (int i = rot + lane; i < D; i += 32) dst[i] = k[i];
    return;
  }
  const int h = which - HQ - HKV;
  const T* v = src + v_col + (size_t)h * DV;
  T* dst = v_cache + (((size_t)page * HKV + h) * KRK_PAGE + (pos % KRK_PAGE)) * DV;
  float rstd = 1.f;
  if (value_norm) {
    float sq = 0.f;
    for (int i = lane; i < DV; i += 32) {
      const float f = to_float<T>(v[i]);
      sq += f * f;
    }
    rstd = rsqrtf(warp_sum(sq) / (float)DV + eps);
  }
  for (int i = lane; i < DV; i += 32) dst[i] = from_float<T>(to_float<T>(v[i]) * rstd);
}

template <typename T> __device__ __forceinline__ float dot_row(const float* q, const T* k, int D) {
  float dot = 0.f;
  for (int d = 0; d < D; ++d) dot += q[d] * to_float<T>(k[d]);
  return dot;
}
// bfloat16 rows of a multiple of 8 elements start on 16-byte boundaries in the cache
template <> __device__ __forceinline__ float dot_row<bf16>(const float* q, const bf16* k, int D) {
  float dot = 0.f;
  if ((D & 7) == 0) {
    for (int d = 0; d < D; d += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + d);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        dot += q[d + 2 * j] * __low2float(p[j]);
        dot += q[d + 2 * j + 1] * __high2float(p[j]);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) dot += q[d] * __bfloat162float(k[d]);
  }
  return dot;
}

template <typename T>
__global__ void sink_attention_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                                      const T* __restrict__ proj, int stride, int q_col, int HQ, int HKV, int D, int DV,
                                      const float* __restrict__ sink, const int* __restrict__ row_seq,
                                      const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                                      const int* __restrict__ table, int width, const T* __restrict__ k_cache,
                                      const T* __restrict__ v_cache, int rows, float scale, int window) {
  extern __shared__ float q_s[];  // warps x D
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)rows * HQ) return;
  const int row = (int)(item / HQ), head = (int)(item % HQ);
  const int kh = head / (HQ / HKV);
  const int pos = row_pos[row];
  const int slot = seq_slot[row_seq[row]];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;

  float* qs = q_s + (size_t)warp * D;
  const T* q = proj + (size_t)row * stride + q_col + (size_t)head * D;
  for (int d = lane; d < D; d += 32) qs[d] = to_float<T>(q[d]);
  __syncwarp();

  float m = sink ? sink[head] : -INFINITY;
  float l = sink ? 1.f : 0.f;
  float acc[MAX_V_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_V_PER_LANE; ++i) acc[i] = 0.f;

  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    float s = -INFINITY;
    if (key <= pos) {
      const int page = page_of(table, width, slot, key);
      s = dot_row<T>(qs, k_cache + (((size_t)page * HKV + kh) * KRK_PAGE + (key % KRK_PAGE)) * D, D) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);  // exp(-inf) = 0 before the first key when there is no sink
    const float p = key <= pos ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_V_PER_LANE; ++i) acc[i] *= alpha;
    const int n = min(32, pos - base + 1);
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const int page = page_of(table, width, slot, kj);
      const T* vp = v_cache + (((size_t)page * HKV + kh) * KRK_PAGE + (kj % KRK_PAGE)) * DV;
#pragma unroll
      for (int i = 0; i < MAX_V_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < DV) acc[i] += pj * to_float<T>(vp[d]);
      }
    }
    m = m_new;
  }
  T* o = out + (size_t)row * out_stride + out_col + (size_t)head * DV;
  const float inv = out_scale / l;
#pragma unroll
  for (int i = 0; i < MAX_V_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < DV) o[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

KRK_API int krk_rotate_norm_write(void* proj, int stride, int q_col, int k_col, int v_col, int HQ, int HKV, int D, int DV,
                                  const float* inv_freq, int rot, int value_norm, float eps, const int* row_seq,
                                  const int* row_pos, const int* seq_slot, const int* table, int width, void* k_cache,
                                  void* v_cache, int rows, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rot < 0 || rot > D || (rot & 1)) return -2;
  const long long items = (long long)rows * (HQ + 2 * HKV);
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(rotate_norm_write_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                           (float*)proj, stride, q_col, k_col, v_col, HQ, HKV, D, DV, inv_freq, rot, value_norm, eps,
                           row_seq, row_pos, seq_slot, table, width, (float*)k_cache, (float*)v_cache, rows);
  return (int)launch_pdl(rotate_norm_write_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, (bf16*)proj,
                         stride, q_col, k_col, v_col, HQ, HKV, D, DV, inv_freq, rot, value_norm, eps, row_seq, row_pos,
                         seq_slot, table, width, (bf16*)k_cache, (bf16*)v_cache, rows);
}

KRK_API int krk_sink_attention(void* out, int out_stride, int out_col, float out_scale, const void* proj, int stride,
                               int q_col, int HQ, int HKV, int D, int DV, const float* sink, const int* row_seq,
                               const int* row_pos, const int* seq_slot, const int* table, int width, const void* k_cache,
                               const void* v_cache, int rows, float scale, int window, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (DV > 32 * MAX_V_PER_LANE || D > 2048) return -2;
  const long long items = (long long)rows * HQ;
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  const size_t smem = (size_t)warps * D * sizeof(float);
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(sink_attention_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream,
                           (float*)out, out_stride, out_col, out_scale, (const float*)proj, stride, q_col, HQ, HKV, D, DV,
                           sink, row_seq, row_pos, seq_slot, table, width, (const float*)k_cache, (const float*)v_cache,
                           rows, scale, window);
  return (int)launch_pdl(sink_attention_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream, (bf16*)out,
                         out_stride, out_col, out_scale, (const bf16*)proj, stride, q_col, HQ, HKV, D, DV, sink, row_seq,
                         row_pos, seq_slot, table, width, (const bf16*)k_cache, (const bf16*)v_cache, rows, scale, window);
}
