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
//
// krk_sink_attention_single (steps of one token per sequence): one block per (sequence, kv head).
// Its warps take the window's 32-key chunks in turn, each lane scores its key against every query head
// of the group from one read of the key (and every value row serves all of the group's heads), and the
// warps' running (maximum, sum, output) are merged in warp order at the end; the sink enters once, as
// the first warp's starting state. Where few (sequence, kv head) items would leave most SMs idle, several
// blocks share an item's chunks and a small kernel merges their results in block order.
//
// Options of all three: the cache may keep a sequence's first pages for good (`keep_pages`, see page_of); a
// windowed query may also see the first `keep_first` keys (they are walked before the window's own, in position
// order); the result may be multiplied by sigmoid(gate), one number per head (mode 1) or per element (mode 2),
// read from the columns `gate_col` of `gate`'s rows; the values that are written may be blended with another
// layer's values of the same rows, (1 - lambda) v + lambda v_first.
#include "common.cuh"

namespace {

constexpr int MAX_V_PER_LANE = 8;    // value heads up to 256
constexpr int WIDE_V_PER_LANE = 16;  // the general kernel's second form: value rows up to 512 (latent rows)

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }  // value heads up to 256

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
                                         T* k_cache, T* v_cache, int rows, int keep_pages,
                                         const T* __restrict__ mix_first, int mix_stride, float lam) {
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
  const int page = page_of(table, width, slot, pos, keep_pages);
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
  if (mix_first) {  // blended with another layer's values of this row (no design has both a blend and a value norm)
    const T* f = mix_first + (size_t)row * mix_stride + (size_t)h * DV;
    for (int i = lane; i < DV; i += 32) dst[i] = from_float<T>((1.0f - lam) * to_float<T>(v[i]) + lam * to_float<T>(f[i]));
    return;
  }
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

template <typename T, int VPL>
__global__ void sink_attention_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                                      const T* __restrict__ proj, int stride, int q_col, int HQ, int HKV, int D, int DV,
                                      const float* __restrict__ sink, const int* __restrict__ row_seq,
                                      const int* __restrict__ row_pos, const int* __restrict__ seq_slot,
                                      const int* __restrict__ table, int width, const T* __restrict__ k_cache,
                                      const T* __restrict__ v_cache, int rows, float scale, int window, int keep_first,
                                      int keep_pages, const T* __restrict__ gate, int gate_stride, int gate_col,
                                      int gate_mode) {
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
  float acc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) acc[i] = 0.f;

  // the kept first keys that the window no longer covers, then the window's own
  const int kept_hi = (window > 0 && keep_first > 0) ? min(keep_first, first) - 1 : -1;
  for (int seg = 0; seg < 2; ++seg) {
  const int lo = seg ? first : 0, hi = seg ? pos : kept_hi;
  for (int base = lo; base <= hi; base += 32) {
    const int key = base + lane;
    float s = -INFINITY;
    int my_page = 0;
    if (key <= hi) {
      my_page = page_of(table, width, slot, key, keep_pages);
      s = dot_row<T>(qs, k_cache + (((size_t)my_page * HKV + kh) * KRK_PAGE + (key % KRK_PAGE)) * D, D) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);  // exp(-inf) = 0 before the first key when there is no sink
    const float p = key <= hi ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] *= alpha;
    const int n = min(32, hi - base + 1);
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const int page = __shfl_sync(0xffffffffu, my_page, j);  // lane j looked its key's page up already
      const T* vp = v_cache + (((size_t)page * HKV + kh) * KRK_PAGE + (kj % KRK_PAGE)) * DV;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int d = lane + 32 * i;
        if (d < DV) acc[i] += pj * to_float<T>(vp[d]);
      }
    }
    m = m_new;
  }
  }
  T* o = out + (size_t)row * out_stride + out_col + (size_t)head * DV;
  float inv = out_scale / l;
  const T* gp = gate_mode ? gate + (size_t)row * gate_stride + gate_col : nullptr;
  if (gate_mode == 1) inv *= sigmoidf_(to_float<T>(gp[head]));
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int d = lane + 32 * i;
    if (d < DV) o[d] = from_float<T>(acc[i] * inv * (gate_mode == 2 ? sigmoidf_(to_float<T>(gp[(size_t)head * DV + d])) : 1.f));
  }
}

constexpr int GROUP_MAX = 8;       // query heads of one kv head that a block serves at once
constexpr int SINGLE_WARPS = 8;

template <typename T> __device__ __forceinline__ void load8(const T* p, float* f);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = p[j];
}
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* f) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __low2float(h[j]);
    f[2 * j + 1] = __high2float(h[j]);
  }
}

template <typename T> __device__ __forceinline__ void load4(const T* p, float* f, bool on);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* f, bool on) {
  const float4 v = on ? *reinterpret_cast<const float4*>(p) : make_float4(0.f, 0.f, 0.f, 0.f);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float* f, bool on) {
  const uint2 raw = on ? *reinterpret_cast<const uint2*>(p) : make_uint2(0u, 0u);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  f[0] = __low2float(h[0]); f[1] = __high2float(h[0]); f[2] = __low2float(h[1]); f[3] = __high2float(h[1]);
}

// V4: value heads of a multiple of 4 elements, lane l holding elements 4l .. 4l + 3 of every 128 of a row.
// NV: a lane's elements of a value row (4: rows up to 128; 16: up to 512, with GM = 4 query heads a block so that
// the accumulators stay in registers and the warps' shares in shared memory; four value rows in flight instead of 16)
template <typename T, bool V4, bool FUSE, int NV, int GM>
__global__ void __launch_bounds__(SINGLE_WARPS * 32)
sink_attention_single_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                             const T* __restrict__ proj, int stride, int q_col, int HQ, int HKV, int D, int DV,
                             const float* __restrict__ sink, const int* __restrict__ seq_slot,
                             const int* __restrict__ seq_start, const int* __restrict__ table, int width,
                             const T* __restrict__ k_cache, const T* __restrict__ v_cache, float scale, int window,
                             int SPL, float* __restrict__ scratch, int k_col, int v_col,
                             const float* __restrict__ inv_freq, int rot, int value_norm, float eps, T* k_cache_w,
                             T* v_cache_w, int keep_first, int keep_pages, const T* __restrict__ gate, int gate_stride,
                             int gate_col, int gate_mode) {
  extern __shared__ __align__(16) float sm1[];
  // a kv head's query heads are served GM at a time: blockIdx.y picks the group, all groups in one launch
  const int g0 = blockIdx.y * GM;
  const int GN = min(GM, HQ / HKV - g0);
  float* q_s = sm1;                       // [GN][D]
  float* part = q_s + GN * D;             // [warps][GN][DV + 2]
  // fused form: the new token's rotated key and normalised value, as the cache stores them
  T* kn = reinterpret_cast<T*>(sm1 + ((GN * D + SINGLE_WARPS * GN * (DV + 2) + 3) & ~3));
  T* vn = kn + ((D + 7) & ~7);
  __shared__ float rstd_s;
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x % SPL, item = blockIdx.x / SPL;  // the block takes every SPL-th chunk of its item
  const int seq = item / HKV, kh = item % HKV;
  const int G = HQ / HKV;
  const int head0 = kh * G + g0;          // the block's first query head
  const int pos = seq_start[seq];         // the one new token sits at the sequence's length before the step
  const int slot = seq_slot[seq];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const T* q = proj + (size_t)seq * stride + q_col + (size_t)head0 * D;
  for (int i = threadIdx.x; i < GN * D; i += blockDim.x) q_s[i] = to_float<T>(q[i]);
  __syncthreads();
  if (FUSE) {
    // what krk_rotate_norm_write does for this (sequence, kv head), here: the queries are rotated in shared memory,
    // the new key and value are made once per block and, by the item's first block, written to their page
    const float p = (float)pos;
    const int half = rot >> 1;
    for (int i = threadIdx.x; i < GN * half; i += blockDim.x) {
      const int g = i / half, j = i % half;
      float sn, cs;
      angle_sincos(p, inv_freq[j], inv_freq[half + j], &sn, &cs);
      const float u = q_s[g * D + j], v = q_s[g * D + j + half];
      q_s[g * D + j] = round_to<T>(u * cs - v * sn);
      q_s[g * D + j + half] = round_to<T>(v * cs + u * sn);
    }
    const T* kr = proj + (size_t)seq * stride + k_col + (size_t)kh * D;
    const T* vr = proj + (size_t)seq * stride + v_col + (size_t)kh * DV;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float sn, cs;
      angle_sincos(p, inv_freq[j], inv_freq[half + j], &sn, &cs);
      const float u = to_float<T>(kr[j]), v = to_float<T>(kr[j + half]);
      kn[j] = from_float<T>(u * cs - v * sn);
      kn[j + half] = from_float<T>(v * cs + u * sn);
    }
    for (int j = rot + threadIdx.x; j < D; j += blockDim.x) kn[j] = kr[j];
    if (warp == 0) {
      float rstd = 1.f;
      if (value_norm) {
        float sq = 0.f;
        for (int j = lane; j < DV; j += 32) {
          const float f = to_float<T>(vr[j]);
          sq += f * f;
        }
        rstd = rsqrtf(warp_sum(sq) / (float)DV + eps);
      }
      if (lane == 0) rstd_s = rstd;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < DV; j += blockDim.x) vn[j] = from_float<T>(to_float<T>(vr[j]) * rstd_s);
    __syncthreads();
    if (split == 0) {
      const int page = page_of(table, width, slot, pos, keep_pages);
      T* kd = k_cache_w + (((size_t)page * HKV + kh) * KRK_PAGE + (pos % KRK_PAGE)) * D;
      T* vd = v_cache_w + (((size_t)page * HKV + kh) * KRK_PAGE + (pos % KRK_PAGE)) * DV;
      for (int j = threadIdx.x; j < D; j += blockDim.x) kd[j] = kn[j];
      for (int j = threadIdx.x; j < DV; j += blockDim.x) vd[j] = vn[j];
    }
  }

  float m[GM], l[GM], acc[GM][NV];
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    const bool has = warp == 0 && split == 0 && sink != nullptr && g < GN;
    m[g] = has ? sink[head0 + g] : -INFINITY;
    l[g] = has ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[g][i] = 0.f;
  }
  const bool vec = (D & 7) == 0;  // rows of the cache then start on 16-byte boundaries (32 for float)
  // the kept first keys that the window no longer covers, then the window's own; chunks of either go round the
  // item's blocks and warps
  const int kept_hi = (window > 0 && keep_first > 0) ? min(keep_first, first) - 1 : -1;
  for (int seg = 0; seg < 2; ++seg) {
  const int lo = seg ? first : 0, hi = seg ? pos : kept_hi;
  for (int base = lo + 32 * (split + SPL * warp); base <= hi; base += 32 * SPL * SINGLE_WARPS) {
    const int key = base + lane;
    float s[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) s[g] = 0.f;
    int my_page = 0;
    if (key <= hi) {
      my_page = page_of(table, width, slot, key, keep_pages);
      const T* kp = (FUSE && key == pos) ? kn  // the new token's key is not in its page for every block yet
                                         : k_cache + (((size_t)my_page * HKV + kh) * KRK_PAGE + (key % KRK_PAGE)) * D;
      if (vec) {
        // 64 elements of the key row are requested at once (a row is a lane's own, nothing shares its
        // latency), then multiplied with every head's query
        int d = 0;
        for (; d + 64 <= D; d += 64) {
          float kf[8][8];
#pragma unroll
          for (int c = 0; c < 8; ++c) load8<T>(kp + d + 8 * c, kf[c]);
#pragma unroll
          for (int c = 0; c < 8; ++c)
#pragma unroll
            for (int g = 0; g < GM; ++g)
              if (g < GN) {
                const float4 qa = *reinterpret_cast<const float4*>(q_s + g * D + d + 8 * c);
                const float4 qb = *reinterpret_cast<const float4*>(q_s + g * D + d + 8 * c + 4);
                s[g] += qa.x * kf[c][0] + qa.y * kf[c][1] + qa.z * kf[c][2] + qa.w * kf[c][3] + qb.x * kf[c][4] +
                        qb.y * kf[c][5] + qb.z * kf[c][6] + qb.w * kf[c][7];
              }
        }
        for (; d < D; d += 8) {
          float kf[8];
          load8<T>(kp + d, kf);
#pragma unroll
          for (int g = 0; g < GM; ++g)
            if (g < GN) {
              const float4 qa = *reinterpret_cast<const float4*>(q_s + g * D + d);
              const float4 qb = *reinterpret_cast<const float4*>(q_s + g * D + d + 4);
              s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] +
                      qb.z * kf[6] + qb.w * kf[7];
            }
        }
      } else {
        for (int d = 0; d < D; ++d) {
          const float kf = to_float<T>(kp[d]);
#pragma unroll
          for (int g = 0; g < GM; ++g)
            if (g < GN) s[g] += q_s[g * D + d] * kf;
        }
      }
    }
    float p[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
      if (g >= GN) continue;
      const float sc = key <= hi ? s[g] * scale : -INFINITY;
      const float m_new = fmaxf(m[g], warp_max(sc));
      const float alpha = expf(m[g] - m_new);
      p[g] = key <= hi ? expf(sc - m_new) : 0.f;
      l[g] = l[g] * alpha + warp_sum(p[g]);
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[g][i] *= alpha;
      m[g] = m_new;
    }
    const int n = min(32, hi - base + 1);
    constexpr int VR = NV == 4 ? 16 : 4;
    for (int j0 = 0; j0 < n; j0 += VR) {  // VR value rows are requested before the first is used
      float vf[VR][NV];
#pragma unroll
      for (int jj = 0; jj < VR; ++jj) {
        const int j = j0 + jj;
        const int kj = base + j;
        const int page = __shfl_sync(0xffffffffu, my_page, j & 31);  // lane j looked its key's page up already
        const T* vp = (FUSE && kj == pos) ? vn : v_cache + (((size_t)page * HKV + kh) * KRK_PAGE + (kj % KRK_PAGE)) * DV;
        if (V4) {  // four neighbouring elements per lane, one load
#pragma unroll
          for (int cb = 0; cb < NV / 4; ++cb)
            load4<T>(vp + 128 * cb + 4 * lane, vf[jj] + 4 * cb, j < n && 128 * cb + 4 * lane < DV);
        } else {
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int d = lane + 32 * i;
            vf[jj][i] = (j < n && d < DV) ? to_float<T>(vp[d]) : 0.f;
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < VR; ++jj)
#pragma unroll
        for (int g = 0; g < GM; ++g) {
          if (g >= GN) continue;
          const float pj = __shfl_sync(0xffffffffu, p[g], (j0 + jj) & 31);  // zero beyond the last key
#pragma unroll
          for (int i = 0; i < NV; ++i) acc[g][i] += pj * vf[jj][i];
        }
    }
  }
  }
  // the warps' partial results, then one warp per head merges them in warp order
  const int PS = DV + 2;
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    if (g >= GN) continue;
    float* dst = part + ((size_t)warp * GN + g) * PS;
    if (lane == 0) { dst[DV] = m[g]; dst[DV + 1] = l[g]; }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = V4 ? (i >> 2) * 128 + 4 * lane + (i & 3) : lane + 32 * i;
      if (d < DV) dst[d] = acc[g][i];
    }
  }
  __syncthreads();
  for (int g = warp; g < GN; g += SINGLE_WARPS) {
    float mx = -INFINITY;
    for (int w = 0; w < SINGLE_WARPS; ++w) mx = fmaxf(mx, part[((size_t)w * GN + g) * PS + DV]);
    float total = 0.f, o[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i] = 0.f;
    for (int w = 0; w < SINGLE_WARPS; ++w) {
      const float* src = part + ((size_t)w * GN + g) * PS;
      const float f = src[DV] == -INFINITY ? 0.f : expf(src[DV] - mx);
      total += src[DV + 1] * f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = V4 ? (i >> 2) * 128 + 4 * lane + (i & 3) : lane + 32 * i;
        if (d < DV) o[i] += src[d] * f;
      }
    }
    if (SPL > 1) {  // this block's share of the keys: (maximum, sum, output) for the merge kernel
      float* dst = scratch + (((size_t)item * SPL + split) * G + g0 + g) * PS;
      if (lane == 0) { dst[DV] = mx; dst[DV + 1] = total; }
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = V4 ? (i >> 2) * 128 + 4 * lane + (i & 3) : lane + 32 * i;
        if (d < DV) dst[d] = o[i];
      }
      continue;
    }
    T* op = out + (size_t)seq * out_stride + out_col + (size_t)(head0 + g) * DV;
    float inv = out_scale / total;
    const T* gp = gate_mode ? gate + (size_t)seq * gate_stride + gate_col : nullptr;
    if (gate_mode == 1) inv *= sigmoidf_(to_float<T>(gp[head0 + g]));
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = V4 ? (i >> 2) * 128 + 4 * lane + (i & 3) : lane + 32 * i;
      if (d < DV)
        op[d] = from_float<T>(o[i] * inv * (gate_mode == 2 ? sigmoidf_(to_float<T>(gp[(size_t)(head0 + g) * DV + d])) : 1.f));
    }
  }
}

// The blocks' shares of one (sequence, head), merged in block order: one warp each.
template <typename T>
__global__ void sink_attention_merge_kernel(T* __restrict__ out, int out_stride, int out_col, float out_scale,
                                            const float* __restrict__ scratch, int HQ, int HKV, int DV, int SPL,
                                            int n_items, const T* __restrict__ gate, int gate_stride, int gate_col,
                                            int gate_mode) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int G = HQ / HKV, PS = DV + 2;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)n_items * G) return;
  const int item = (int)(w / G), g = (int)(w % G);
  const int seq = item / HKV, kh = item % HKV;
  // at most 8 blocks share an item: their maxima, then one factor each, then the shares added in block order
  const float* base = scratch + ((size_t)item * SPL * G + g) * PS;
  const size_t step = (size_t)G * PS;
  float ms[8], f[8];
  float mx = -INFINITY;
#pragma unroll
  for (int sp = 0; sp < 8; ++sp) {
    ms[sp] = sp < SPL ? base[sp * step + DV] : -INFINITY;
    mx = fmaxf(mx, ms[sp]);
  }
  float total = 0.f;
#pragma unroll
  for (int sp = 0; sp < 8; ++sp) {
    f[sp] = ms[sp] == -INFINITY ? 0.f : expf(ms[sp] - mx);
    if (sp < SPL) total += base[sp * step + DV + 1] * f[sp];
  }
  T* op = out + (size_t)seq * out_stride + out_col + (size_t)(kh * G + g) * DV;
  float inv = out_scale / total;
  const T* gp = gate_mode ? gate + (size_t)seq * gate_stride + gate_col : nullptr;
  if (gate_mode == 1) inv *= sigmoidf_(to_float<T>(gp[kh * G + g]));
  for (int d = lane; d < DV; d += 32) {  // value rows of any width
    float v[8];
#pragma unroll
    for (int sp = 0; sp < 8; ++sp) v[sp] = sp < SPL ? base[sp * step + d] : 0.f;
    float o = 0.f;
#pragma unroll
    for (int sp = 0; sp < 8; ++sp) o += v[sp] * f[sp];
    op[d] = from_float<T>(o * inv * (gate_mode == 2 ? sigmoidf_(to_float<T>(gp[(size_t)(kh * G + g) * DV + d])) : 1.f));
  }
}

}  // namespace

KRK_API int krk_rotate_norm_write(void* proj, int stride, int q_col, int k_col, int v_col, int HQ, int HKV, int D, int DV,
                                  const float* inv_freq, int rot, int value_norm, float eps, const int* row_seq,
                                  const int* row_pos, const int* seq_slot, const int* table, int width, void* k_cache,
                                  void* v_cache, int rows, int keep_pages, const void* mix_first, int mix_stride,
                                  float lam, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rot < 0 || rot > D || (rot & 1)) return -2;
  const long long items = (long long)rows * (HQ + 2 * HKV);
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(rotate_norm_write_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                           (float*)proj, stride, q_col, k_col, v_col, HQ, HKV, D, DV, inv_freq, rot, value_norm, eps,
                           row_seq, row_pos, seq_slot, table, width, (float*)k_cache, (float*)v_cache, rows, keep_pages,
                           (const float*)mix_first, mix_stride, lam);
  return (int)launch_pdl(rotate_norm_write_kernel<bf16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, (bf16*)proj,
                         stride, q_col, k_col, v_col, HQ, HKV, D, DV, inv_freq, rot, value_norm, eps, row_seq, row_pos,
                         seq_slot, table, width, (bf16*)k_cache, (bf16*)v_cache, rows, keep_pages, (const bf16*)mix_first,
                         mix_stride, lam);
}

KRK_API int krk_sink_attention(void* out, int out_stride, int out_col, float out_scale, const void* proj, int stride,
                               int q_col, int HQ, int HKV, int D, int DV, const float* sink, const int* row_seq,
                               const int* row_pos, const int* seq_slot, const int* table, int width, const void* k_cache,
                               const void* v_cache, int rows, float scale, int window, int keep_first, int keep_pages,
                               const void* gate, int gate_stride, int gate_col, int gate_mode, int dtype,
                               cudaStream_t stream) {
  if (rows == 0) return 0;
  if (DV > 32 * WIDE_V_PER_LANE || D > 2048) return -2;
  const long long items = (long long)rows * HQ;
  const int warps = 4;
  const long long blocks = (items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return -3;
  const size_t smem = (size_t)warps * D * sizeof(float);
  const bool wide = DV > 32 * MAX_V_PER_LANE;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(wide ? sink_attention_kernel<float, WIDE_V_PER_LANE> : sink_attention_kernel<float, MAX_V_PER_LANE>, dim3((unsigned)blocks), dim3(warps * 32), smem, stream,
                           (float*)out, out_stride, out_col, out_scale, (const float*)proj, stride, q_col, HQ, HKV, D, DV,
                           sink, row_seq, row_pos, seq_slot, table, width, (const float*)k_cache, (const float*)v_cache,
                           rows, scale, window, keep_first, keep_pages, (const float*)gate, gate_stride, gate_col, gate_mode);
  return (int)launch_pdl(wide ? sink_attention_kernel<bf16, WIDE_V_PER_LANE> : sink_attention_kernel<bf16, MAX_V_PER_LANE>,
                         dim3((unsigned)blocks), dim3(warps * 32), smem, stream, (bf16*)out,
                         out_stride, out_col, out_scale, (const bf16*)proj, stride, q_col, HQ, HKV, D, DV, sink, row_seq,
                         row_pos, seq_slot, table, width, (const bf16*)k_cache, (const bf16*)v_cache, rows, scale, window,
                         keep_first, keep_pages, (const bf16*)gate, gate_stride, gate_col, gate_mode);
}

// One token per sequence: rows are the sequences, in order. Value heads of up to 512 elements; others take
// krk_sink_attention. splits > 1: that many blocks share an item's keys and a merge kernel follows; scratch then
// holds n_seqs * HQ * splits * (DV + 2) floats. fuse: the kernel also does what krk_rotate_norm_write does for the
// step's rows (queries rotated on the way in, the new key and value made in shared memory and written to their page
// by the item's first block), so that a single-token step needs no launch of that kernel.
KRK_API int krk_sink_attention_single(void* out, int out_stride, int out_col, float out_scale, const void* proj, int stride,
                                      int q_col, int HQ, int HKV, int D, int DV, const float* sink, const int* seq_slot,
                                      const int* seq_start, const int* table, int width, const void* k_cache,
                                      const void* v_cache, int n_seqs, float scale, int window, int splits,
                                      float* scratch, int fuse, int k_col, int v_col, const float* inv_freq, int rot,
                                      int value_norm, float eps, int keep_first, int keep_pages, const void* gate,
                                      int gate_stride, int gate_col, int gate_mode, int dtype, cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  if (DV > 512 || D > 1024) return -2;
  const int G = HQ / HKV;
  const int SPL = (splits > 1 && scratch) ? splits : 1;
  if (SPL > 8) return -2;  // the merge kernel holds one factor per block of an item
  const bool wide = DV > 32 * (MAX_V_PER_LANE / 2);  // value rows beyond 128 elements: fewer heads a block
  const int gm = wide ? 4 : GROUP_MAX;
  if (fuse && (wide || G > GROUP_MAX)) return -2;  // the new key and value are made by one launch per item
  if (fuse && (rot < 0 || rot > D || (rot & 1))) return -2;
  {
    const int GN = min(gm, G);  // the most heads a block serves; blocks of the last group may serve fewer
    const int groups = (G + gm - 1) / gm;
    const size_t esz = dtype == KRK_DTYPE_F32 ? 4 : 2;
    const size_t smem = ((size_t)GN * D + (size_t)SINGLE_WARPS * GN * (DV + 2) + 4) * sizeof(float) +
                        (((size_t)D + 7) / 8 * 8 + DV + 8) * esz;
    if (smem > 96 * 1024) return -2;
    cudaError_t e;
    const bool v4 = (DV & 3) == 0;  // rows of the value cache then start on 8-byte (16 for float) boundaries
    if (dtype == KRK_DTYPE_F32) {
      auto kern = wide ? (v4 ? sink_attention_single_kernel<float, true, false, 16, 4> : sink_attention_single_kernel<float, false, false, 16, 4>)
                  : fuse ? (v4 ? sink_attention_single_kernel<float, true, true, 4, GROUP_MAX> : sink_attention_single_kernel<float, false, true, 4, GROUP_MAX>)
                         : (v4 ? sink_attention_single_kernel<float, true, false, 4, GROUP_MAX> : sink_attention_single_kernel<float, false, false, 4, GROUP_MAX>);
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
      e = launch_pdl(kern, dim3(n_seqs * HKV * SPL, groups), dim3(SINGLE_WARPS * 32), smem, stream,
                     (float*)out, out_stride, out_col, out_scale, (const float*)proj, stride, q_col, HQ, HKV, D, DV, sink,
                     seq_slot, seq_start, table, width, (const float*)k_cache, (const float*)v_cache, scale, window, SPL, scratch, k_col, v_col,
                     inv_freq, rot, value_norm, eps, (float*)k_cache, (float*)v_cache, keep_first, keep_pages,
                     (const float*)gate, gate_stride, gate_col, gate_mode);
    } else {
      auto kern = wide ? (v4 ? sink_attention_single_kernel<bf16, true, false, 16, 4> : sink_attention_single_kernel<bf16, false, false, 16, 4>)
                  : fuse ? (v4 ? sink_attention_single_kernel<bf16, true, true, 4, GROUP_MAX> : sink_attention_single_kernel<bf16, false, true, 4, GROUP_MAX>)
                         : (v4 ? sink_attention_single_kernel<bf16, true, false, 4, GROUP_MAX> : sink_attention_single_kernel<bf16, false, false, 4, GROUP_MAX>);
      if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
      e = launch_pdl(kern, dim3(n_seqs * HKV * SPL, groups), dim3(SINGLE_WARPS * 32), smem, stream,
                     (bf16*)out, out_stride, out_col, out_scale, (const bf16*)proj, stride, q_col, HQ, HKV, D, DV, sink,
                     seq_slot, seq_start, table, width, (const bf16*)k_cache, (const bf16*)v_cache, scale, window, SPL, scratch, k_col, v_col,
                     inv_freq, rot, value_norm, eps, (bf16*)k_cache, (bf16*)v_cache, keep_first, keep_pages,
                     (const bf16*)gate, gate_stride, gate_col, gate_mode);
    }
    if (e != cudaSuccess) return (int)e;
  }
  if (SPL > 1) {
    const long long warps = (long long)n_seqs * HKV * G;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    cudaError_t e;
    if (dtype == KRK_DTYPE_F32)
      e = launch_pdl(sink_attention_merge_kernel<float>, dim3(blocks), dim3(128), 0, stream, (float*)out, out_stride,
                     out_col, out_scale, (const float*)scratch, HQ, HKV, DV, SPL, n_seqs * HKV, (const float*)gate,
                     gate_stride, gate_col, gate_mode);
    else
      e = launch_pdl(sink_attention_merge_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, (bf16*)out, out_stride,
                     out_col, out_scale, (const float*)scratch, HQ, HKV, DV, SPL, n_seqs * HKV, (const bf16*)gate,
                     gate_stride, gate_col, gate_mode);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
