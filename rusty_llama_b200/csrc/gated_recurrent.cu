// Linear attention whose decay and input strength change from token to token, through a 32-bit state per sequence:
//
//   S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T,   o_t = S_t^T (c q_t)        per head; S is [dim, vcols]
//
// a_t = exp(log_decay_t) is one number per key channel (a row of `dim`) or one per head; b_t is one number per head or 1;
// c is a constant.  With `ext` the state has one more column that is fed with v = 1: it carries n_t = a_t n_(t-1) + b_t k_t,
// and the output's last column is n_t . q_t, the normaliser of a matrix memory.  Two designs use it:
//
//   gated linear attention   a_t = sigmoid(z_t)^(1/tau) per channel (`gla_log_decay` makes log a_t), b = 1
//   matrix memory (mLSTM)    log gates i_t, f_t per head with a running maximum m_t = max(f_t + m_(t-1), i_t):
//                            a_t = exp(f_t + m_(t-1) - m_t), b_t = exp(i_t - m_t) (`mlstm_gates`), `ext` column,
//                            o_t / (max(|n_t . q_t|, exp(-m_t)) + c_den) in `head_norm_gate`
//
// The kernels:
//   gla_log_decay     log a = logsigmoid(z + bias) / tau, 32-bit, from the projection in the run's element type
//   mlstm_gates       the capped log gates, the running maximum through the sequences' records, a's logarithm, b and m per token
//   gated_attn        the recurrence token by token (decode steps, 32-bit runs, short prompts): equal bits however a sequence is cut
//   gated_attn chunked   prompts of bfloat16 runs: chunks of 64 tokens, sub-chunks of 16 (see below)
//   head_norm_gate    per head: the normaliser, the RMS norm over the head's values, weight, gate; writes the run's element type
//
// Everything between the projections and the state is 32-bit: decays and their logarithms, gates, the maximum, the state, the sums.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

__device__ __forceinline__ float gr_logistic(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float gr_log_logistic(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// ---------------------------------------------------------------- log decay of gated linear attention
template <typename T>
__global__ void gla_log_decay_kernel(const T* __restrict__ z, int z_stride, const float* __restrict__ bias, float inv_tau,
                                     float* __restrict__ out, int n, long long total) {
  pdl_trigger();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / n;
    const int i = (int)(idx - t * n);
    const float v = to_f32(z[t * z_stride + i]) + (bias ? bias[i] : 0.f);
    out[idx] = gr_log_logistic(v) * inv_tau;
  }
}

RL_API int rl_gla_log_decay(const void* z, int dtype, int z_stride, const float* bias, float tau, float* out, int n_tokens, int n,
                            cudaStream_t stream) {
  if (n_tokens <= 0 || n <= 0 || !(tau > 0.f)) RL_REFUSE(1, "gla_log_decay: T=%d n=%d tau=%g", n_tokens, n, (double)tau);
  const long long total = (long long)n_tokens * n;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch(gla_log_decay_kernel<bf16>, (int)blocks, 256, 0, stream, (const bf16*)z, z_stride, bias, 1.0f / tau, out, n, total));
  else if (dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch(gla_log_decay_kernel<float>, (int)blocks, 256, 0, stream, (const float*)z, z_stride, bias, 1.0f / tau, out, n, total));
  else
    RL_REFUSE(2, "gla_log_decay: unknown dtype %d", dtype);
  return 0;
}

// ---------------------------------------------------------------- the gates of a matrix memory
// One warp per (sequence, head).  32 tokens' gates are computed side by side; the running maximum then goes through them in
// order (one lane's values at a time, by shuffle), so its bits do not depend on where a step starts.
template <typename T>
__global__ void mlstm_gates_kernel(const T* __restrict__ gi, const T* __restrict__ gf, int in_stride, const float* __restrict__ bias_i,
                                   const float* __restrict__ bias_f, float cap, float* __restrict__ m_state, const int* __restrict__ slot_ids,
                                   const int* __restrict__ seq_start, float* __restrict__ log_a, float* __restrict__ b_out,
                                   float* __restrict__ m_out, int H) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x;
  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* mp = m_state + (size_t)slot_ids[s] * H + h;
  float m = *mp;
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  const float inv_cap = 1.0f / cap;
  for (int base = t0; base < t1; base += 32) {
    const int t = base + lane;
    float li = 0.f, lf = 0.f;
    if (t < t1) {
      li = cap * tanhf((to_f32(gi[(size_t)t * in_stride + h]) + bi) * inv_cap);
      lf = gr_log_logistic(cap * tanhf((to_f32(gf[(size_t)t * in_stride + h]) + bf) * inv_cap));
    }
    const int n = min(32, t1 - base);
    float la = 0.f, bb = 0.f, mo = 0.f;
    for (int j = 0; j < n; ++j) {
      const float lij = __shfl_sync(0xffffffffu, li, j), lfj = __shfl_sync(0xffffffffu, lf, j);
      const float m_new = fmaxf(lfj + m, lij);
      if (lane == j) {
        la = lfj + m - m_new;
        bb = expf(lij - m_new);
        mo = m_new;
      }
      m = m_new;
    }
    if (t < t1) {
      log_a[(size_t)t * H + h] = la;
      b_out[(size_t)t * H + h] = bb;
      m_out[(size_t)t * H + h] = mo;
    }
  }
  if (lane == 0) *mp = m;
}

RL_API int rl_mlstm_gates(const void* gi, const void* gf, int dtype, int in_stride, const float* bias_i, const float* bias_f, float cap,
                          float* m_state, const int* slot_ids, const int* seq_start, float* log_a, float* b_out, float* m_out,
                          int n_seqs, int H, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || !(cap > 0.f)) RL_REFUSE(1, "mlstm_gates: S=%d H=%d cap=%g", n_seqs, H, (double)cap);
  if (dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch(mlstm_gates_kernel<bf16>, n_seqs * H, 32, 0, stream, (const bf16*)gi, (const bf16*)gf, in_stride, bias_i, bias_f,
                              cap, m_state, slot_ids, seq_start, log_a, b_out, m_out, H));
  else if (dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch(mlstm_gates_kernel<float>, n_seqs * H, 32, 0, stream, (const float*)gi, (const float*)gf, in_stride, bias_i,
                              bias_f, cap, m_state, slot_ids, seq_start, log_a, b_out, m_out, H));
  else
    RL_REFUSE(2, "mlstm_gates: unknown dtype %d", dtype);
  return 0;
}

// ---------------------------------------------------------------- the recurrence, token by token
// A block owns 32 columns of one head's state for one sequence: lane = column, warp w holds rows 32 w .. 32 w + 31 of those
// columns in registers.  Tokens are taken GR_TOK at a time: their q, b k and a (whole head) and v (the block's columns) go to
// shared memory, every warp runs the tokens through its rows, and the warps' partial results are added in warp order.  The
// order of every sum is fixed by the sizes alone.
#define GR_TOK 16

template <typename T>
__global__ void gated_attn_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
                                  const float* __restrict__ log_decay, int per_channel, const float* __restrict__ in_scale, float q_scale,
                                  float* __restrict__ state, const int* __restrict__ slot_ids, const int* __restrict__ seq_start,
                                  float* __restrict__ out, int out_stride, int H, int dim, int vdim, int ext) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * 32;
  const int vcols = vdim + ext;
  const int col = col0 + lane;
  const bool col_ok = col < vcols;
  float* q_s = sm;                      // [GR_TOK][dim]
  float* k_s = q_s + GR_TOK * dim;      // [GR_TOK][dim], times b
  float* a_s = k_s + GR_TOK * dim;      // [GR_TOK][dim]
  float* v_s = a_s + GR_TOK * dim;      // [GR_TOK][32]
  float* part = v_s + GR_TOK * 32;      // [nw][GR_TOK][32]
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* st = state + (((size_t)slot_ids[s] * H + h) * dim) * vcols;
  float S[32];
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int row = w * 32 + r;
    S[r] = (row < dim && col_ok) ? st[(size_t)row * vcols + col] : 0.f;
  }
  for (int base = t0; base < t1; base += GR_TOK) {
    const int n = min(GR_TOK, t1 - base);
    for (int idx = threadIdx.x; idx < n * dim; idx += blockDim.x) {
      const int j = idx / dim, i = idx - j * dim;
      const int t = base + j;
      const size_t at = (size_t)t * in_stride + (size_t)h * dim + i;
      const float b = in_scale ? in_scale[(size_t)t * H + h] : 1.f;
      q_s[idx] = to_f32(q[at]) * q_scale;
      k_s[idx] = to_f32(k[at]) * b;
      a_s[idx] = expf(per_channel ? log_decay[((size_t)t * H + h) * dim + i] : log_decay[(size_t)t * H + h]);
    }
    for (int idx = threadIdx.x; idx < n * 32; idx += blockDim.x) {
      const int j = idx >> 5, c = col0 + (idx & 31);
      float vv = 0.f;
      if (c < vdim) vv = to_f32(v[(size_t)(base + j) * in_stride + (size_t)h * vdim + c]);
      else if (c < vcols) vv = 1.f;
      v_s[idx] = vv;
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float vj = v_s[j * 32 + lane];
      const float* kj = k_s + j * dim + w * 32;
      const float* qj = q_s + j * dim + w * 32;
      const float* aj = a_s + j * dim + w * 32;
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < 32; ++r) {
        if (w * 32 + r < dim) {
          S[r] = aj[r] * S[r] + kj[r] * vj;
          o += S[r] * qj[r];
        }
      }
      part[(w * GR_TOK + j) * 32 + lane] = o;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * 32; idx += blockDim.x) {
      const int j = idx >> 5, c = idx & 31;
      if (col0 + c < vcols) {
        float o = 0.f;
        for (int ww = 0; ww < nw; ++ww) o += part[(ww * GR_TOK + j) * 32 + c];
        out[(size_t)(base + j) * out_stride + (size_t)h * vcols + col0 + c] = o;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int row = w * 32 + r;
    if (row < dim && col_ok) st[(size_t)row * vcols + col] = S[r];
  }
}

RL_API int rl_gated_attn(const void* q, const void* k, const void* v, int dtype, int in_stride, const float* log_decay, int per_channel,
                         const float* in_scale, float q_scale, float* state, const int* slot_ids, const int* seq_start, float* out,
                         int out_stride, int n_seqs, int H, int dim, int vdim, int ext, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || (ext != 0 && ext != 1) || !log_decay)
    RL_REFUSE(1, "gated_attn: S=%d H=%d dim=%d vdim=%d ext=%d", n_seqs, H, dim, vdim, ext);
  if (dim > 1024) RL_REFUSE(2, "gated_attn: key size %d exceeds 1024", dim);
  const int tiles = (vdim + ext + 31) / 32;
  if (H > 65535 || tiles > 65535) RL_REFUSE(3, "gated_attn: %d heads or %d columns exceed the grid", H, vdim);
  const int nw = (dim + 31) / 32;
  const size_t smem = ((size_t)3 * GR_TOK * dim + GR_TOK * 32 + (size_t)nw * GR_TOK * 32) * sizeof(float);
  if (smem > 227 * 1024) RL_REFUSE(4, "gated_attn: %zu bytes of shared memory", smem);
  dim3 grid(n_seqs, H, tiles);
#define RL_GA(T)                                                                                                                   \
  do {                                                                                                                             \
    if (smem > 48 * 1024) {                                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(gated_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) RL_REFUSE(4, "gated_attn: %zu bytes of shared memory refused", smem);                                  \
    }                                                                                                                              \
    RL_LAUNCH_CHECK(rl_launch(gated_attn_kernel<T>, grid, nw * 32, smem, stream, (const T*)q, (const T*)k, (const T*)v, in_stride,  \
                              log_decay, per_channel, in_scale, q_scale, state, slot_ids, seq_start, out, out_stride, H, dim, vdim, \
                              ext));                                                                                               \
  } while (0)
  if (dtype == RL_BF16) RL_GA(bf16);
  else if (dtype == RL_F32) RL_GA(float);
  else RL_REFUSE(5, "gated_attn: unknown dtype %d", dtype);
#undef RL_GA
  return 0;
}

// ---------------------------------------------------------------- per head: normaliser, RMS norm, weight, gate
// One warp per (token, head).  x: 32-bit rows of H heads of `xh` numbers, of which the first n are the head's values; with m
// given, x[n] is the head's n . q and the values are first divided by max(|x[n]|, exp(-m)) + den_eps.  Then
//   y_i = v_i / sqrt(mean(v^2) + eps) * weight * act(gate_i)
// weight: [n] shared by the heads, or [H n]; act: 0 none, 1 the logistic function, 2 silu.
#define HN_MAX_PER_LANE 16  // head values up to 512

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ x, int x_stride, int xh, const float* __restrict__ m, float den_eps,
                                      const float* __restrict__ weight, int weight_per_head, float eps, const T* __restrict__ gate,
                                      int gate_stride, int gate_act, float out_scale, T* __restrict__ out, int out_stride, int n_rows,
                                      int H, int n) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= n_rows * H) return;
  const int t = pair / H, h = pair - t * H;
  const float* xr = x + (size_t)t * x_stride + (size_t)h * xh;
  float inv_den = 1.f;
  if (m != nullptr) inv_den = 1.0f / (fmaxf(fabsf(xr[n]), expf(-m[(size_t)t * H + h])) + den_eps);
  float vals[HN_MAX_PER_LANE];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < HN_MAX_PER_LANE; ++e) {
    const int i = lane + 32 * e;
    vals[e] = i < n ? xr[i] * inv_den : 0.f;
    ss += vals[e] * vals[e];
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
  const T* g = gate ? gate + (size_t)t * gate_stride + (size_t)h * n : nullptr;
  const float* wv = weight ? weight + (weight_per_head ? (size_t)h * n : 0) : nullptr;
  T* o = out + (size_t)t * out_stride + (size_t)h * n;
#pragma unroll
  for (int e = 0; e < HN_MAX_PER_LANE; ++e) {
    const int i = lane + 32 * e;
    if (i < n) {
      float y = vals[e] * inv;
      if (wv) y *= wv[i];
      if (g) {
        const float gv = to_f32(g[i]);
        y *= gate_act == 2 ? gv * gr_logistic(gv) : (gate_act == 1 ? gr_logistic(gv) : gv);
      }
      o[i] = from_f32<T>(y * out_scale);
    }
  }
}

RL_API int rl_head_norm_gate(const float* x, int x_stride, int xh, const float* m, float den_eps, const float* weight, int weight_per_head,
                             float eps, const void* gate, int gate_stride, int gate_act, float out_scale, void* out, int out_stride,
                             int act_dtype, int n_rows, int H, int n, cudaStream_t stream) {
  if (n_rows <= 0 || H <= 0 || n <= 0 || !x || !out) RL_REFUSE(1, "head_norm_gate: rows=%d H=%d n=%d", n_rows, H, n);
  if (n > 32 * HN_MAX_PER_LANE) RL_REFUSE(2, "head_norm_gate: a head of %d values exceeds %d", n, 32 * HN_MAX_PER_LANE);
  if (xh < n + (m != nullptr ? 1 : 0)) RL_REFUSE(3, "head_norm_gate: head stride %d too small", xh);
  const long long pairs = (long long)n_rows * H;
  const int blocks = (int)((pairs + 3) / 4);
  if (act_dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch(head_norm_gate_kernel<bf16>, blocks, 128, 0, stream, x, x_stride, xh, m, den_eps, weight, weight_per_head, eps,
                              (const bf16*)gate, gate_stride, gate_act, out_scale, (bf16*)out, out_stride, n_rows, H, n));
  else if (act_dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch(head_norm_gate_kernel<float>, blocks, 128, 0, stream, x, x_stride, xh, m, den_eps, weight, weight_per_head, eps,
                              (const float*)gate, gate_stride, gate_act, out_scale, (float*)out, out_stride, n_rows, H, n));
  else
    RL_REFUSE(4, "head_norm_gate: unknown dtype %d", act_dtype);
  return 0;
}
