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

// The same for long prompts: a block of MG_WARPS warps per (sequence, head) takes 32 MG_WARPS tokens at a time.  A token is the map
// m -> max(m + f, i); two maps in a row are again such a map, (f1, i1) then (f2, i2) = (f1 + f2, max(i1 + f2, i2)), so a warp
// composes its 32 maps by a scan of five shuffles, the warps' totals go through shared memory, and every token applies its
// composed map to the maximum that entered the round.  The sums of f are taken in another order than token by token: equal
// within rounding, not in bits, and the order depends on where the step starts.
#define MG_WARPS 8

template <typename T>
__global__ void __launch_bounds__(32 * MG_WARPS)
mlstm_gates_scan_kernel(const T* __restrict__ gi, const T* __restrict__ gf, int in_stride, const float* __restrict__ bias_i,
                        const float* __restrict__ bias_f, float cap, float* __restrict__ m_state, const int* __restrict__ slot_ids,
                        const int* __restrict__ seq_start, float* __restrict__ log_a, float* __restrict__ b_out,
                        float* __restrict__ m_out, int H) {
  __shared__ float tot_f[MG_WARPS], tot_i[MG_WARPS];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  float* mp = m_state + (size_t)slot_ids[s] * H + h;
  float m_in = *mp;
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  const float inv_cap = 1.0f / cap;
  for (int base = t0; base < t1; base += 32 * MG_WARPS) {
    const int t = base + threadIdx.x;
    float li = -INFINITY, lf = 0.f;  // past the end: the map that changes nothing
    if (t < t1) {
      li = cap * tanhf((to_f32(gi[(size_t)t * in_stride + h]) + bi) * inv_cap);
      lf = gr_log_logistic(cap * tanhf((to_f32(gf[(size_t)t * in_stride + h]) + bf) * inv_cap));
    }
    float F = lf, I = li;  // the tokens of this warp up to and with this lane's, as one map
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) {
        I = fmaxf(Ip + F, I);
        F = Fp + F;
      }
    }
    if (lane == 31) {
      tot_f[warp] = F;
      tot_i[warp] = I;
    }
    __syncthreads();
    float m_w = m_in;  // the maximum that enters this warp's tokens
    for (int w = 0; w < warp; ++w) m_w = fmaxf(m_w + tot_f[w], tot_i[w]);
    const float m_new = fmaxf(m_w + F, I);
    float m_prev = __shfl_up_sync(0xffffffffu, m_new, 1);
    if (lane == 0) m_prev = m_w;
    if (t < t1) {
      log_a[(size_t)t * H + h] = lf + m_prev - m_new;
      b_out[(size_t)t * H + h] = expf(li - m_new);
      m_out[(size_t)t * H + h] = m_new;
    }
    for (int w = warp; w < MG_WARPS; ++w) m_w = fmaxf(m_w + tot_f[w], tot_i[w]);  // the maximum after the round, in every thread
    m_in = m_w;
    __syncthreads();
  }
  if (threadIdx.x == 0) *mp = m_in;
}

RL_API int rl_mlstm_gates(const void* gi, const void* gf, int dtype, int in_stride, const float* bias_i, const float* bias_f, float cap,
                          float* m_state, const int* slot_ids, const int* seq_start, float* log_a, float* b_out, float* m_out,
                          int n_seqs, int H, int scan, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || !(cap > 0.f)) RL_REFUSE(1, "mlstm_gates: S=%d H=%d cap=%g", n_seqs, H, (double)cap);
  if (scan) {
    if (dtype == RL_BF16)
      RL_LAUNCH_CHECK(rl_launch(mlstm_gates_scan_kernel<bf16>, n_seqs * H, 32 * MG_WARPS, 0, stream, (const bf16*)gi, (const bf16*)gf, in_stride,
                                bias_i, bias_f, cap, m_state, slot_ids, seq_start, log_a, b_out, m_out, H));
    else if (dtype == RL_F32)
      RL_LAUNCH_CHECK(rl_launch(mlstm_gates_scan_kernel<float>, n_seqs * H, 32 * MG_WARPS, 0, stream, (const float*)gi, (const float*)gf,
                                in_stride, bias_i, bias_f, cap, m_state, slot_ids, seq_start, log_a, b_out, m_out, H));
    else
      RL_REFUSE(2, "mlstm_gates: unknown dtype %d", dtype);
    return 0;
  }
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

// ---------------------------------------------------------------- the same recurrence, chunk by chunk
// For prompts.  A sequence's tokens are cut into chunks of GC; with n tokens in a chunk, S the state before it,
// A_i = sum_{l <= i} log a_l (per key channel, inside the chunk) and k'_j = b_j k_j:
//   U      = sum_j diag(exp(A_(n-1) - A_j)) k'_j v_j^T                                  (1) what the chunk adds, every chunk at once
//   S_next = diag(exp(A_(n-1))) S + U                                                    (2) the states before every chunk, chunk after chunk
//   o_i    = S^T (q_i * exp(A_i)) + sum_{j<=i} (sum_r q_i[r] k'_j[r] exp(A_i[r] - A_j[r])) v_j   (3) the outputs, every chunk at once
// Only exponents <= 0 occur, whatever the decays are: the scores of (3) between tokens of the same sub-chunk of 16 take
// exp(A_i - A_j) channel by channel; between sub-chunks I > J they factor through the sub-chunks' borders,
//   exp(A_i - A_(16 I - 1)) * exp(A_(16 I - 1) - A_(16 J + 15)) * exp(A_(16 J + 15) - A_j),
// a factor of the query, one of the border pair and one of the key.  All of it is 32-bit FMA arithmetic over a scratch of one
// [dim, vcols] matrix and one row of dim decays per (sequence, head, chunk).  The order of the sums differs from the
// token-by-token kernel's and depends on where the chunks fall, so 32-bit runs keep to the other kernel.
#define GC 64       // tokens per chunk
#define GC_SUB 16   // tokens per sub-chunk
#define GC_COLS 64  // state columns per block
#define GR_LOG2E 1.4426950408889634f

__device__ __forceinline__ float gr_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A last column tile of at most four columns (a matrix memory's normaliser beside values that fill whole tiles) gets no block and
// no round of its own: the block of the tile before it adds those columns up with a thread per (row, quarter of the sum).
__host__ __device__ __forceinline__ int gc_narrow(int vcols) {
  const int tiles = (vcols + GC_COLS - 1) / GC_COLS, rem = vcols - (tiles - 1) * GC_COLS;
  return tiles > 1 && rem <= 4 ? rem : 0;
}

// (1): grid (S * H, chunks, column tiles), 256 threads: thread (ty, tx) owns rows ty + 16 a and columns 4 tx .. 4 tx + 3.
template <typename T>
__global__ void __launch_bounds__(256)
gated_chunk_state_kernel(const T* __restrict__ k, const T* __restrict__ v, int in_stride, const float* __restrict__ log_decay,
                         int per_channel, const float* __restrict__ in_scale, const int* __restrict__ seq_start,
                         float* __restrict__ scratch, float* __restrict__ chunk_decay, int max_chunks, int H, int dim, int vdim, int ext) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.y, col0 = blockIdx.z * GC_COLS;
  const int vcols = vdim + ext;
  const int t0 = seq_start[s] + c * GC;
  const int n = min(GC, seq_start[s + 1] - t0);
  if (n <= 0) return;
  float* k_s = sm;             // [GC][dim]: first the decays' logarithms, then the weighted keys
  float* v_s = sm + GC * dim;  // [GC][GC_COLS]
  float* v_x = v_s + GC * GC_COLS;  // [GC][4]: the narrow last tile's values
  const int narrow = blockIdx.z == gridDim.z - 1 ? gc_narrow(vcols) : 0;
  const int col_x0 = (int)gridDim.z * GC_COLS;
  for (int idx = threadIdx.x; idx < n * dim; idx += 256) {
    const int i = idx / dim, r = idx - i * dim;
    const size_t th = (size_t)(t0 + i) * H + h;
    k_s[idx] = GR_LOG2E * (per_channel ? log_decay[th * dim + r] : log_decay[th]);
  }
  for (int idx = threadIdx.x; idx < n * narrow; idx += 256) {
    const int i = idx / narrow, e = idx - i * narrow, cc = col_x0 + e;
    v_x[i * 4 + e] = cc < vdim ? to_f32(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + cc]) : 1.f;
  }
  for (int idx = threadIdx.x; idx < n * GC_COLS; idx += 256) {
    const int i = idx / GC_COLS, cc = col0 + (idx - i * GC_COLS);
    float vv = 0.f;
    if (cc < vdim) vv = to_f32(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + cc]);
    else if (cc < vcols) vv = 1.f;
    v_s[idx] = vv;
  }
  __syncthreads();
  // per channel: what the tokens after token i still take away, and the whole chunk's decay
  for (int r = threadIdx.x; r < dim; r += 256) {
    float after = 0.f;
    for (int i = n - 1; i >= 0; --i) {
      const float la = k_s[i * dim + r];
      k_s[i * dim + r] = after;
      after += la;
    }
    if (blockIdx.z == 0) chunk_decay[((size_t)blockIdx.x * max_chunks + c) * dim + r] = gr_exp2(after);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n * dim; idx += 256) {
    const int i = idx / dim, r = idx - i * dim;
    const float b = in_scale ? in_scale[(size_t)(t0 + i) * H + h] : 1.f;
    k_s[idx] = to_f32(k[(size_t)(t0 + i) * in_stride + (size_t)h * dim + r]) * b * gr_exp2(k_s[idx]);
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float* u = scratch + ((size_t)blockIdx.x * max_chunks + c) * dim * vcols;
  for (int r0 = 0; r0 < dim; r0 += 128) {  // 128 rows of the state at a time: eight to a thread
    float acc[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
    for (int i = 0; i < n; ++i) {
      const float4 vv = *reinterpret_cast<const float4*>(v_s + i * GC_COLS + 4 * tx);
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const int r = r0 + ty + 16 * a;
        if (r < dim) {
          const float kv = k_s[i * dim + r];
          acc[a][0] += kv * vv.x;
          acc[a][1] += kv * vv.y;
          acc[a][2] += kv * vv.z;
          acc[a][3] += kv * vv.w;
        }
      }
    }
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int r = r0 + ty + 16 * a;
      if (r < dim) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = col0 + 4 * tx + e;
          if (col < vcols) u[(size_t)r * vcols + col] = acc[a][e];
        }
      }
    }
  }
  for (int idx = threadIdx.x; idx < dim * narrow; idx += 256) {
    const int r = idx / narrow, e = idx - r * narrow;
    float acc = 0.f;
    for (int i = 0; i < n; ++i) acc += k_s[i * dim + r] * v_x[i * 4 + e];
    u[(size_t)r * vcols + col_x0 + e] = acc;
  }
}

// (2): one thread per element of a (sequence, head)'s state; leaves in every chunk's place the state BEFORE that chunk.
__global__ void gated_chunk_scan_kernel(float* __restrict__ state, const int* __restrict__ slot_ids, const int* __restrict__ seq_start,
                                        float* __restrict__ scratch, const float* __restrict__ chunk_decay, int max_chunks, int H,
                                        int dim, int vcols) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int elems = dim * vcols;
  const int e = blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= elems) return;
  const int r = e / vcols;
  const int len = seq_start[s + 1] - seq_start[s];
  float* st = state + ((size_t)slot_ids[s] * H + h) * elems + e;
  float* u = scratch + (size_t)blockIdx.x * max_chunks * elems + e;
  const float* g = chunk_decay + (size_t)blockIdx.x * max_chunks * dim + r;
  float S = *st;
  const int n_chunks = (len + GC - 1) / GC;
  for (int c0 = 0; c0 < n_chunks; c0 += 8) {  // eight chunks' additions are asked for at once, then taken in order
    float add[8], dec[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < n_chunks) {
        add[j] = __ldcg(u + (size_t)(c0 + j) * elems);
        dec[j] = __ldcg(g + (size_t)(c0 + j) * dim);
      }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < n_chunks) {
        u[(size_t)(c0 + j) * elems] = S;
        S = dec[j] * S + add[j];
      }
  }
  *st = S;
}

// (3): grid (S * H, chunks).  Thread (ty, tx): scores P[ty + 16 a][tx + 16 b] (a, b: the sub-chunks of the query and of the key),
// computed once; then, column tile after column tile, outputs for rows ty + 16 a and columns 4 tx .. 4 tx + 3.  The scores and the
// values' tile take the place of the decays' sums, and the state's tile the keys' place, once those are used up: three tiles of
// [GC][dim + 1] in all, so that two blocks share an SM at dim = 128.
template <typename T>
__global__ void __launch_bounds__(256)
gated_chunk_out_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
                       const float* __restrict__ log_decay, int per_channel, const float* __restrict__ in_scale, float q_scale,
                       const int* __restrict__ seq_start, const float* __restrict__ scratch, int max_chunks, float* __restrict__ out,
                       int out_stride, int H, int dim, int vdim, int ext) {
  extern __shared__ float sm[];
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.x / H, h = blockIdx.x % H, c = blockIdx.y;
  const int vcols = vdim + ext;
  const int t0 = seq_start[s] + c * GC;
  const int n = min(GC, seq_start[s + 1] - t0);
  if (n <= 0) return;
  const int DS = dim + 1;  // rows one apart in the banks
  float* q_s = sm;                    // [GC][DS]
  float* k_s = q_s + GC * DS;         // [GC][DS]; later the state's tile [dim][GC_COLS]
  float* a_s = k_s + GC * DS;         // [GC][DS]: A_i in units of log 2; later v_s and p_s
  float* v_s = a_s;                   // [GC][GC_COLS]
  float* p_s = v_s + GC * GC_COLS;    // [GC][GC + 1]
  float* d_s = a_s + max(GC * DS, GC * GC_COLS + GC * (GC + 1));  // [5][dim]: the decay over sub-chunk 1 and over sub-chunk 2; A at the ends of sub-chunks 0, 1, 2
  float* v_x = d_s + 5 * dim;         // [GC][4]: the narrow last tile's values
  const int narrow = gc_narrow(vcols), wide_cols = vcols - narrow;
  for (int idx = threadIdx.x; idx < n * narrow; idx += 256) {
    const int i = idx / narrow, e = idx - i * narrow, cc = wide_cols + e;
    v_x[i * 4 + e] = cc < vdim ? to_f32(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + cc]) : 1.f;
  }
  for (int idx = threadIdx.x; idx < GC * dim; idx += 256) {
    const int i = idx / dim, r = idx - i * dim;
    float qv = 0.f, kv = 0.f, la = 0.f;
    if (i < n) {
      const size_t at = (size_t)(t0 + i) * in_stride + (size_t)h * dim + r;
      const size_t th = (size_t)(t0 + i) * H + h;
      qv = to_f32(q[at]) * q_scale;
      kv = to_f32(k[at]) * (in_scale ? in_scale[th] : 1.f);
      la = GR_LOG2E * (per_channel ? log_decay[th * dim + r] : log_decay[th]);
    }
    q_s[i * DS + r] = qv;
    k_s[i * DS + r] = kv;
    a_s[i * DS + r] = la;
  }
  __syncthreads();
  for (int r = threadIdx.x; r < dim; r += 256) {  // A_i: the running sum down the chunk (rows past the last token repeat it)
    float run = 0.f;
    for (int i = 0; i < GC; ++i) {
      run += a_s[i * DS + r];
      a_s[i * DS + r] = run;
    }
  }
  __syncthreads();
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float p[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a) p[a][0] = p[a][1] = p[a][2] = p[a][3] = 0.f;
  // ---- scores inside a sub-chunk: the decay between the two tokens, channel by channel
  if (tx <= ty) {
    for (int r = 0; r < dim; ++r) {
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int i = (ty + 16 * a) * DS + r, j = (tx + 16 * a) * DS + r;
        p[a][a] += q_s[i] * k_s[j] * gr_exp2(a_s[i] - a_s[j]);
      }
    }
  }
  __syncthreads();
  // ---- queries relative to the start of their sub-chunk, keys relative to the end of theirs, and the two inner sub-chunks' decays
  for (int idx = threadIdx.x; idx < GC * dim; idx += 256) {
    const int i = idx / dim, r = idx - i * dim;
    const int sub = i / GC_SUB;
    const float mine = a_s[i * DS + r];
    const float before = sub > 0 ? a_s[(sub * GC_SUB - 1) * DS + r] : 0.f;
    const float end = a_s[(sub * GC_SUB + GC_SUB - 1) * DS + r];
    q_s[i * DS + r] *= gr_exp2(mine - before);
    k_s[i * DS + r] *= gr_exp2(end - mine);
  }
  for (int idx = threadIdx.x; idx < 2 * dim; idx += 256) {
    const int w = idx / dim, r = idx - w * dim;  // w = 0: over sub-chunk 1, w = 1: over sub-chunk 2
    d_s[idx] = gr_exp2(a_s[((w + 2) * GC_SUB - 1) * DS + r] - a_s[((w + 1) * GC_SUB - 1) * DS + r]);
  }
  for (int idx = threadIdx.x; idx < 3 * dim; idx += 256) {
    const int w = idx / dim, r = idx - w * dim;
    d_s[2 * dim + idx] = a_s[((w + 1) * GC_SUB - 1) * DS + r];
  }
  __syncthreads();  // the decays' sums are used up from here on
  // ---- scores between sub-chunks
  for (int r = 0; r < dim; ++r) {
    const float q1 = q_s[(ty + 16) * DS + r], q2 = q_s[(ty + 32) * DS + r], q3 = q_s[(ty + 48) * DS + r];
    const float k0 = k_s[tx * DS + r], k1 = k_s[(tx + 16) * DS + r], k2 = k_s[(tx + 32) * DS + r];
    const float d1 = d_s[r], d2 = d_s[dim + r];
    p[1][0] += q1 * k0;
    p[2][1] += q2 * k1;
    p[3][2] += q3 * k2;
    p[2][0] += q2 * d1 * k0;
    p[3][1] += q3 * d2 * k1;
    p[3][0] += q3 * (d1 * d2) * k0;
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) p_s[(ty + 16 * a) * (GC + 1) + tx + 16 * b] = p[a][b];  // zero above the diagonal: never added to
  __syncthreads();
  // ---- the queries against the state before the chunk take the whole decay since the chunk's start
  for (int idx = threadIdx.x; idx < GC * dim; idx += 256) {
    const int i = idx / dim, r = idx - i * dim;
    const int sub = i / GC_SUB;
    if (sub > 0) q_s[i * DS + r] *= gr_exp2(d_s[(sub + 1) * dim + r]);
  }
  const float* sp = scratch + ((size_t)blockIdx.x * max_chunks + c) * dim * vcols;
  float* s_s = k_s;  // [dim][GC_COLS]; GC * (dim + 1) >= dim * GC_COLS
  for (int col0 = 0; col0 < wide_cols; col0 += GC_COLS) {
    __syncthreads();  // scores and queries written, keys read (first tile); the tile before read
    for (int idx = threadIdx.x; idx < GC * GC_COLS; idx += 256) {
      const int i = idx / GC_COLS, cc = col0 + (idx - i * GC_COLS);
      float vv = 0.f;
      if (i < n) {
        if (cc < vdim) vv = to_f32(v[(size_t)(t0 + i) * in_stride + (size_t)h * vdim + cc]);
        else if (cc < vcols) vv = 1.f;
      }
      v_s[idx] = vv;
    }
    for (int idx = threadIdx.x; idx < dim * GC_COLS; idx += 256) {
      const int r = idx / GC_COLS, cc = col0 + (idx - r * GC_COLS);
      s_s[idx] = cc < vcols ? sp[(size_t)r * vcols + cc] : 0.f;
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
    for (int j = 0; j < n; ++j) {
      const float4 vv = *reinterpret_cast<const float4*>(v_s + j * GC_COLS + 4 * tx);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float pv = p_s[(ty + 16 * a) * (GC + 1) + j];
        acc[a][0] += pv * vv.x;
        acc[a][1] += pv * vv.y;
        acc[a][2] += pv * vv.z;
        acc[a][3] += pv * vv.w;
      }
    }
    for (int r = 0; r < dim; ++r) {
      const float4 t = *reinterpret_cast<const float4*>(s_s + r * GC_COLS + 4 * tx);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float qv = q_s[(ty + 16 * a) * DS + r];
        acc[a][0] += qv * t.x;
        acc[a][1] += qv * t.y;
        acc[a][2] += qv * t.z;
        acc[a][3] += qv * t.w;
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ty + 16 * a;
      if (i < n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = col0 + 4 * tx + e;
          if (col < vcols) out[(size_t)(t0 + i) * out_stride + (size_t)h * vcols + col] = acc[a][e];
        }
      }
    }
  }
  if (narrow > 0) {  // thread (i, part): a quarter of row i's sums over the keys and over the state's rows, added up by shuffles
    const int i = threadIdx.x >> 2, part = threadIdx.x & 3;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = part; j < n; j += 4) {
      const float pv = p_s[i * (GC + 1) + j];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < narrow) acc[e] += pv * v_x[j * 4 + e];
    }
    for (int r = part; r < dim; r += 4) {
      const float qv = q_s[i * DS + r];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < narrow) acc[e] += qv * sp[(size_t)r * vcols + wide_cols + e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
      acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
    }
    if (part == 0 && i < n) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < narrow) out[(size_t)(t0 + i) * out_stride + (size_t)h * vcols + wide_cols + e] = acc[e];
    }
  }
}

RL_API long long rl_gated_attn_chunked_scratch_floats(int n_seqs, int max_q_len, int H, int dim, int vcols) {
  return (long long)n_seqs * H * ((max_q_len + GC - 1) / GC) * dim * (vcols + 1);
}

static size_t gated_chunk_out_smem(int dim) {
  const size_t tile = (size_t)GC * (dim + 1), later = (size_t)GC * GC_COLS + GC * (GC + 1);
  return (2 * tile + (tile > later ? tile : later) + 5 * (size_t)dim + GC * 4) * sizeof(float);
}

RL_API int rl_gated_attn_chunked_takes(int dim) { return dim > 0 && gated_chunk_out_smem(dim) <= 227 * 1024; }

RL_API int rl_gated_attn_chunked(const void* q, const void* k, const void* v, int dtype, int in_stride, const float* log_decay,
                                 int per_channel, const float* in_scale, float q_scale, float* state, const int* slot_ids,
                                 const int* seq_start, float* scratch, float* out, int out_stride, int n_seqs, int max_q_len, int H,
                                 int dim, int vdim, int ext, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || H <= 0 || dim <= 0 || vdim <= 0 || (ext != 0 && ext != 1) || !log_decay || !scratch)
    RL_REFUSE(1, "gated_attn_chunked: S=%d max_q=%d H=%d dim=%d vdim=%d ext=%d", n_seqs, max_q_len, H, dim, vdim, ext);
  if (!rl_gated_attn_chunked_takes(dim)) RL_REFUSE(2, "gated_attn_chunked: key size %d needs more shared memory than an SM has", dim);
  const int vcols = vdim + ext;
  const int max_chunks = (max_q_len + GC - 1) / GC, col_tiles = (vcols + GC_COLS - 1) / GC_COLS - (gc_narrow(vcols) > 0 ? 1 : 0);
  const long long sh = (long long)n_seqs * H;
  if (sh > 0x7fffffffLL || max_chunks > 65535 || col_tiles > 65535) RL_REFUSE(3, "gated_attn_chunked: %d chunks or %d column tiles exceed the grid", max_chunks, col_tiles);
  float* chunk_decay = scratch + sh * max_chunks * dim * vcols;
  const int elems = dim * vcols;
  dim3 grid((unsigned)sh, max_chunks, col_tiles), grid2((unsigned)sh, (elems + 255) / 256), grid3((unsigned)sh, max_chunks);
  const size_t smem1 = ((size_t)GC * dim + GC * GC_COLS + GC * 4) * sizeof(float), smem3 = gated_chunk_out_smem(dim);
#define RL_GC(T)                                                                                                                     \
  do {                                                                                                                               \
    if (cudaFuncSetAttribute(gated_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1) != cudaSuccess || \
        cudaFuncSetAttribute(gated_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3) != cudaSuccess)     \
      RL_REFUSE(4, "gated_attn_chunked: %zu bytes of shared memory refused", smem3);                                                 \
    RL_LAUNCH_CHECK(rl_launch(gated_chunk_state_kernel<T>, grid, 256, smem1, stream, (const T*)k, (const T*)v, in_stride, log_decay,  \
                              per_channel, in_scale, seq_start, scratch, chunk_decay, max_chunks, H, dim, vdim, ext));               \
    RL_LAUNCH_CHECK(rl_launch(gated_chunk_scan_kernel, grid2, 256, 0, stream, state, slot_ids, seq_start, scratch,                   \
                              (const float*)chunk_decay, max_chunks, H, dim, vcols));                                                \
    RL_LAUNCH_CHECK(rl_launch(gated_chunk_out_kernel<T>, grid3, 256, smem3, stream, (const T*)q, (const T*)k, (const T*)v, in_stride,  \
                              log_decay, per_channel, in_scale, q_scale, seq_start, (const float*)scratch, max_chunks, out,          \
                              out_stride, H, dim, vdim, ext));                                                                       \
  } while (0)
  if (dtype == RL_BF16) RL_GC(bf16);
  else if (dtype == RL_F32) RL_GC(float);
  else RL_REFUSE(5, "gated_attn_chunked: unknown dtype %d", dtype);
#undef RL_GC
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
