// Mixers with a matrix-valued recurrent state per head: the token shift of RWKV-style time
// mixing, and one scan kernel for two update rules.
//
// State S [N key channels, N value channels] per (sequence, head), float32, in global memory
// between steps. With r, k, v of a token, a decay w and (delta rule) a removal rate a:
//
//   rule 0 (WKV):    o = (S + diag(bonus) k v^T)^T r ;  S <- diag(w) S + k v^T
//   rule 1 (delta):  u = k / sqrt(sum k^2 + 1e-6) ;  S <- diag(w) S - (a * u)(u^T S) + k v^T ;  o = S^T r
//
//   z = W2 tanh(lora) + w0 ;  w = exp(-exp(z)) (rule 0)  or  exp(-decay_scale * sigmoid(z)) (rule 1)
//   a = sigmoid(rate + rate_bias)
//   out = o / sqrt(mean_head(o^2) + eps) * norm_w * gate(g) * out_scale, gate = silu (rule 0) or sigmoid (rule 1)
//
// One block per (sequence, head); thread j owns column j of S in registers for the whole pass, so
// the sums over key channels are private, ordered sums and the token loop has no barrier. Tokens
// are taken in chunks: the block first computes the chunk's decays, unit keys and rates in
// parallel into shared memory (float32), then every thread walks the chunk's tokens alone, then
// the block normalises and gates the chunk's outputs in parallel. A token's result is the same
// to the bit however the sequence was cut into steps: the chunking regroups work, not sums.
#include "common.cuh"

namespace {

// out[s, r, c] = h[r, c] + (prev[r, c] - h[r, c]) * mu[s, c]; prev is the row before, or the
// sequence's stored last row for the first row of its step.
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, const T* __restrict__ h, int h_stride, const float* last_state,
                                   const float* __restrict__ mu, int n_mix, int C, int rows,
                                   const int* __restrict__ row_seq, const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_slot) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int seq = row_seq[r];
  const bool first = cu_q[seq] == r;
  const float* last = last_state + (size_t)seq_slot[seq] * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float hv = to_float<T>(h[(size_t)r * h_stride + c]);
    const float pv = first ? last[c] : to_float<T>(h[(size_t)(r - 1) * h_stride + c]);
    const float d = pv - hv;
    for (int s = 0; s < n_mix; ++s)
      out[((size_t)s * rows + r) * C + c] = from_float<T>(hv + d * mu[(size_t)s * C + c]);
  }
}

struct ScanArgs {
  const void *r, *k, *v, *g, *rate, *lora;
  int r_stride, k_stride, v_stride, g_stride, rate_stride, lora_stride;
  const void* w2;          // [H*N, R], element type of the path
  const float* w0;         // [H*N]
  const float* rate_bias;  // [H*N] (rule 1)
  const float* bonus;      // [H*N] (rule 0)
  const float* norm_w;     // [H*N]
  float* state;            // [slots, H, N, N]
  const void* last_rows;   // rows whose last one per sequence is stored (rule 0's token shift), or null
  int last_stride, C;
  float* last_state;       // [slots, C]
  void* out;
  int out_stride, out_col;
  float out_scale, eps, decay_scale;
  int H, N, R, n_seqs;
  const int *cu_q, *seq_qlen, *seq_slot;
};

__device__ __forceinline__ float sigmoidf(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T, int RULE, int NCAP, int TC>
__global__ void __launch_bounds__(NCAP) recurrence_kernel(ScanArgs a) {
  extern __shared__ float sm[];
  const int N = a.N, R = a.R;
  float* r_s = sm;                 // [TC][N]
  float* k_s = r_s + TC * N;       // [TC][N]
  float* v_s = k_s + TC * N;       // [TC][N]
  float* w_s = v_s + TC * N;       // [TC][N] decay
  float* u_s = w_s + TC * N;       // [TC][N] unit key (rule 1) / bonus * k (rule 0)
  float* au_s = u_s + TC * N;      // [TC][N] rate * unit key (rule 1)
  float* o_s = au_s + TC * N;      // [TC][N]
  float* w2_s = o_s + TC * N;      // [R][N]
  float* th_s = w2_s + R * N;      // [TC][R] tanh of the low-rank input
  float* red_s = th_s + TC * R;    // [TC] per-token reductions

  grid_launch_dependents();
  const int seq = blockIdx.x / a.H, head = blockIdx.x % a.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  const int ch0 = head * N;
  // weights first: no kernel writes them
  for (int i = tid; i < R * N; i += blockDim.x) {
    const int m = i / N, c = i % N;
    w2_s[i] = to_float<T>(reinterpret_cast<const T*>(a.w2)[(size_t)(ch0 + c) * R + m]);
  }
  grid_dependency_wait();
  const int row0 = a.cu_q[seq], T_len = a.seq_qlen[seq], slot = a.seq_slot[seq];
  const bool on = tid < N;

  float S[NCAP];
  float* st = a.state + (((size_t)slot * a.H + head) * N) * N;
#pragma unroll
  for (int i = 0; i < NCAP; ++i) S[i] = (on && i < N) ? st[(size_t)i * N + tid] : 0.f;

  const T* rp = reinterpret_cast<const T*>(a.r);
  const T* kp = reinterpret_cast<const T*>(a.k);
  const T* vp = reinterpret_cast<const T*>(a.v);
  const T* gp = reinterpret_cast<const T*>(a.g);
  const T* ap = reinterpret_cast<const T*>(a.rate);
  const T* lp = reinterpret_cast<const T*>(a.lora);
  T* outp = reinterpret_cast<T*>(a.out);

  for (int t0 = 0; t0 < T_len; t0 += TC) {
    const int nt = min(TC, T_len - t0);
    __syncthreads();  // the chunk before is out of shared memory
    // -- stage r, k, v and the tanh of the low-rank input ------------------------------------
    for (int i = tid; i < nt * N; i += blockDim.x) {
      const int t = i / N, c = i % N;
      const size_t row = (size_t)(row0 + t0 + t);
      r_s[i] = to_float<T>(rp[row * a.r_stride + ch0 + c]);
      k_s[i] = to_float<T>(kp[row * a.k_stride + ch0 + c]);
      v_s[i] = to_float<T>(vp[row * a.v_stride + ch0 + c]);
    }
    for (int i = tid; i < nt * R; i += blockDim.x) {
      const int t = i / R, m = i % R;
      th_s[i] = round_to<T>(tanhf(to_float<T>(lp[(size_t)(row0 + t0 + t) * a.lora_stride + m])));
    }
    __syncthreads();
    // -- per token: sum of squared key channels (rule 1) ---------------------------------------
    if (RULE == 1) {
      for (int t = warp; t < nt; t += n_warps) {
        float sq = 0.f;
        for (int c = lane; c < N; c += 32) sq += k_s[t * N + c] * k_s[t * N + c];
        sq = warp_sum(sq);
        if (lane == 0) red_s[t] = rsqrtf(sq + 1e-6f);
      }
      __syncthreads();
    }
    // -- decays, unit keys, rates: thread c serves channel c of every token of the chunk --------
    if (on) {
      const float w0 = a.w0[ch0 + tid];
      const float extra = RULE == 1 ? a.rate_bias[ch0 + tid] : a.bonus[ch0 + tid];
      for (int t = 0; t < nt; ++t) {
        float z = 0.f;
        for (int m = 0; m < R; ++m) z += th_s[t * R + m] * w2_s[m * N + tid];
        z += w0;
        const int i = t * N + tid;
        if (RULE == 1) {
          w_s[i] = expf(-a.decay_scale * sigmoidf(z));
          const float u = k_s[i] * red_s[t];
          const size_t row = (size_t)(row0 + t0 + t);
          u_s[i] = u;
          au_s[i] = sigmoidf(to_float<T>(ap[row * a.rate_stride + ch0 + tid]) + extra) * u;
        } else {
          w_s[i] = expf(-expf(z));
          u_s[i] = extra * k_s[i];
        }
      }
    }
    __syncthreads();
    // -- the scan: every thread alone with its column ----------------------------------------------
    if (on) {
      for (int t = 0; t < nt; ++t) {
        const float* rr = r_s + t * N;
        const float* kk = k_s + t * N;
        const float* ww = w_s + t * N;
        const float* uu = u_s + t * N;
        const float vj = v_s[t * N + tid];
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        if (RULE == 1) {
          const float* aa = au_s + t * N;
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
          for (int i = 0; i < NCAP; i += 4) {
            if (i < N) s0 += uu[i] * S[i];
            if (i + 1 < N) s1 += uu[i + 1] * S[i + 1];
            if (i + 2 < N) s2 += uu[i + 2] * S[i + 2];
            if (i + 3 < N) s3 += uu[i + 3] * S[i + 3];
          }
          const float uS = (s0 + s1) + (s2 + s3);
#pragma unroll
          for (int i = 0; i < NCAP; i += 4) {
            if (i < N) { S[i] = ww[i] * S[i] - aa[i] * uS + kk[i] * vj; o0 += rr[i] * S[i]; }
            if (i + 1 < N) { S[i + 1] = ww[i + 1] * S[i + 1] - aa[i + 1] * uS + kk[i + 1] * vj; o1 += rr[i + 1] * S[i + 1]; }
            if (i + 2 < N) { S[i + 2] = ww[i + 2] * S[i + 2] - aa[i + 2] * uS + kk[i + 2] * vj; o2 += rr[i + 2] * S[i + 2]; }
            if (i + 3 < N) { S[i + 3] = ww[i + 3] * S[i + 3] - aa[i + 3] * uS + kk[i + 3] * vj; o3 += rr[i + 3] * S[i + 3]; }
          }
        } else {
#pragma unroll
          for (int i = 0; i < NCAP; i += 4) {
            if (i < N) { o0 += rr[i] * (S[i] + uu[i] * vj); S[i] = ww[i] * S[i] + kk[i] * vj; }
            if (i + 1 < N) { o1 += rr[i + 1] * (S[i + 1] + uu[i + 1] * vj); S[i + 1] = ww[i + 1] * S[i + 1] + kk[i + 1] * vj; }
            if (i + 2 < N) { o2 += rr[i + 2] * (S[i + 2] + uu[i + 2] * vj); S[i + 2] = ww[i + 2] * S[i + 2] + kk[i + 2] * vj; }
            if (i + 3 < N) { o3 += rr[i + 3] * (S[i + 3] + uu[i + 3] * vj); S[i + 3] = ww[i + 3] * S[i + 3] + kk[i + 3] * vj; }
          }
        }
        o_s[t * N + tid] = (o0 + o1) + (o2 + o3);
      }
    }
    __syncthreads();
    // -- per head: divide by the root mean square, weight, gate, scale --------------------------------
    for (int t = warp; t < nt; t += n_warps) {
      float sq = 0.f;
      for (int c = lane; c < N; c += 32) sq += o_s[t * N + c] * o_s[t * N + c];
      sq = warp_sum(sq);
      if (lane == 0) red_s[t] = rsqrtf(sq / (float)N + a.eps);
    }
    __syncthreads();
    for (int i = tid; i < nt * N; i += blockDim.x) {
      const int t = i / N, c = i % N;
      const size_t row = (size_t)(row0 + t0 + t);
      const float g = to_float<T>(gp[row * a.g_stride + ch0 + c]);
      const float gate = RULE == 1 ? sigmoidf(g) : g * sigmoidf(g);
      outp[row * a.out_stride + a.out_col + ch0 + c] =
          from_float<T>(o_s[i] * red_s[t] * a.norm_w[ch0 + c] * gate * a.out_scale);
    }
  }
#pragma unroll
  for (int i = 0; i < NCAP; ++i)
    if (on && i < N) st[(size_t)i * N + tid] = S[i];
  if (a.last_rows && head == 0 && T_len > 0) {
    const T* last = reinterpret_cast<const T*>(a.last_rows) + (size_t)(row0 + T_len - 1) * a.last_stride;
    float* dst = a.last_state + (size_t)slot * a.C;
    for (int c = tid; c < a.C; c += blockDim.x) dst[c] = to_float<T>(last[c]);
  }
}

template <typename T, int RULE, int NCAP>
int launch_recurrence(const ScanArgs& a, cudaStream_t stream) {
  constexpr int TC = NCAP <= 64 ? 16 : 8;
  const size_t smem = ((size_t)7 * TC * a.N + (size_t)a.R * a.N + (size_t)TC * a.R + TC) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  auto kern = recurrence_kernel<T, RULE, NCAP, TC>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return (int)launch_pdl(kern, dim3(a.n_seqs * a.H), dim3(NCAP), smem, stream, a);
}

template <typename T, int RULE>
int pick_recurrence(const ScanArgs& a, cudaStream_t stream) {
  if (a.N <= 32) return launch_recurrence<T, RULE, 32>(a, stream);
  if (a.N <= 64) return launch_recurrence<T, RULE, 64>(a, stream);
  if (a.N <= 128) return launch_recurrence<T, RULE, 128>(a, stream);
  return -2;  // a head's state column no longer fits one thread's registers
}

}  // namespace

KRK_API int krk_token_shift(void* out, const void* h, int h_stride, const float* last_state, const float* mu, int n_mix,
                            int C, int rows, const int* row_seq, const int* cu_q, const int* seq_slot, int dtype,
                            cudaStream_t stream) {
  if (rows == 0) return 0;
  const int threads = C >= 1024 ? 256 : 128;
  if (dtype == KRK_DTYPE_F32)
    return (int)launch_pdl(token_shift_kernel<float>, dim3(rows), dim3(threads), 0, stream, (float*)out, (const float*)h,
                           h_stride, last_state, mu, n_mix, C, rows, row_seq, cu_q, seq_slot);
  return (int)launch_pdl(token_shift_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, (bf16*)out, (const bf16*)h,
                         h_stride, last_state, mu, n_mix, C, rows, row_seq, cu_q, seq_slot);
}

KRK_API int krk_linear_recurrence(int rule, const void* r, int r_stride, const void* k, int k_stride, const void* v,
                                  int v_stride, const void* g, int g_stride, const void* rate, int rate_stride,
                                  const void* lora, int lora_stride, const void* w2, const float* w0,
                                  const float* rate_bias, const float* bonus, const float* norm_w, float* state,
                                  const void* last_rows, int last_stride, int C, float* last_state, void* out,
                                  int out_stride, int out_col, float out_scale, float eps, float decay_scale, int H, int N,
                                  int R, int n_seqs, const int* cu_q, const int* seq_qlen, const int* seq_slot, int dtype,
                                  cudaStream_t stream) {
  if (n_seqs == 0) return 0;
  ScanArgs a;
  a.r = r; a.k = k; a.v = v; a.g = g; a.rate = rate; a.lora = lora;
  a.r_stride = r_stride; a.k_stride = k_stride; a.v_stride = v_stride; a.g_stride = g_stride;
  a.rate_stride = rate_stride; a.lora_stride = lora_stride;
  a.w2 = w2; a.w0 = w0; a.rate_bias = rate_bias; a.bonus = bonus; a.norm_w = norm_w; a.state = state;
  a.last_rows = last_rows; a.last_stride = last_stride; a.C = C; a.last_state = last_state;
  a.out = out; a.out_stride = out_stride; a.out_col = out_col; a.out_scale = out_scale; a.eps = eps;
  a.decay_scale = decay_scale; a.H = H; a.N = N; a.R = R; a.n_seqs = n_seqs;
  a.cu_q = cu_q; a.seq_qlen = seq_qlen; a.seq_slot = seq_slot;
  if (rule != 0 && rule != 1) return -2;
  if (rule == 1 && (!rate || !rate_bias)) return -2;
  if (rule == 0 && !bonus) return -2;
  if (dtype == KRK_DTYPE_F32)
    return rule == 1 ? pick_recurrence<float, 1>(a, stream) : pick_recurrence<float, 0>(a, stream);
  return rule == 1 ? pick_recurrence<bf16, 1>(a, stream) : pick_recurrence<bf16, 0>(a, stream);
}
