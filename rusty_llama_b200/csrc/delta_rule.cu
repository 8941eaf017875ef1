// The gated delta rule: a linear attention whose state is corrected toward the new value instead of only added to.
// Per head, with a state S of dim x vdim numbers (32-bit, one record per sequence), unit vectors q_t and k_t, a write
// strength beta_t in (0, 1) and a decay g_t in (0, 1):
//
//     S <- g_t S;    u = beta_t (v_t - S^T k_t);    S <- S + k_t u^T;    o_t = S^T q_t
//
// in this order, so the read-out sees the token's own write.  Three kernels and a helper:
//
//   short_conv        a causal convolution over time per channel, y_t = act(sum_i w[i][c] x_(t - taps + 1 + i)), through a
//                     record of the last taps - 1 inputs per sequence (zeros before a sequence's start); a second small
//                     kernel moves the record on after the outputs are made
//   delta_prep        per token: q and k heads made unit vectors, x / sqrt(sum(x^2) + eps), q times a constant; k . q per
//                     head; beta = logistic(b); g = exp(-exp(A_log) softplus(a + dt_bias)): all 32-bit, written as float32
//   delta_rule        the recurrence, token by token: a block owns 32 columns of one head's state of one sequence, a
//                     thread 32 rows of one column in registers; a column's state evolves on its own, so the blocks never
//                     meet; the partial sums of a column's row slices (lanes of one warp) are added by shuffles in a fixed
//                     order, and u_t is folded into the read-out: o_t = (g S)^T q + u (k . q).  Prompts, parts of
//                     prompts and single tokens run the same code, so a result's bits depend neither on how a sequence
//                     was cut into steps nor on what else is in the batch.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

// ---------------------------------------------------------------- short convolution
#define CONV_MAX_TAPS 16

__device__ __forceinline__ float dr_silu(float z) { return z / (1.0f + expf(-z)); }

// One thread per (token, channel).  x: [T, >= C] rows; w: [taps][C] (tap i of every channel side by side, the last row the
// current token's); state: [slots][taps - 1][C], entry j the input at (first position of the step) - (taps - 1) + j.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ x, int x_stride, const float* __restrict__ w, const float* __restrict__ state,
                                  const int* __restrict__ slot_ids, const int* __restrict__ seq_start, const int* __restrict__ tok_seq,
                                  T* __restrict__ out, int out_stride, int n_tokens, int C, int taps, int silu) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * C) return;
  const int t = (int)(idx / C), c = (int)(idx - (long long)t * C);
  const int s = tok_seq[t];
  const int start = seq_start[s];
  const int local = t - start;
  const float* rec = state + (size_t)slot_ids[s] * (taps - 1) * C;
  float acc = 0.f;
  for (int i = 0; i < taps; ++i) {
    const int src = local - (taps - 1) + i;
    const float v = src >= 0 ? to_f32(x[(size_t)(start + src) * x_stride + c]) : rec[(size_t)(taps - 1 + src) * C + c];
    acc += w[(size_t)i * C + c] * v;
  }
  out[(size_t)t * out_stride + c] = from_f32<T>(silu ? dr_silu(acc) : acc);
}

// The same for bfloat16 rows of a multiple of 8 channels that start on 16 bytes: a thread takes 8 neighbouring channels of a token,
// sixteen bytes a load (32 from the record), the same sums in the same order.
__global__ void short_conv_rows8_kernel(const bf16* __restrict__ x, int x_stride, const float* __restrict__ w, const float* __restrict__ state,
                                        const int* __restrict__ slot_ids, const int* __restrict__ seq_start, const int* __restrict__ tok_seq,
                                        bf16* __restrict__ out, int out_stride, int n_tokens, int C, int taps, int silu) {
  const int c8s = C >> 3;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_tokens * c8s) return;
  const int t = (int)(idx / c8s), c = (int)(idx - (long long)t * c8s) * 8;
  const int s = tok_seq[t];
  const int start = seq_start[s];
  const int local = t - start;
  const float* rec = state + (size_t)slot_ids[s] * (taps - 1) * C;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = 0; i < taps; ++i) {
    const int src = local - (taps - 1) + i;
    float v[8];
    if (src >= 0) {
      bf16x8_to_f32(*reinterpret_cast<const uint4*>(x + (size_t)(start + src) * x_stride + c), v);
    } else {
      const float4 lo = *reinterpret_cast<const float4*>(rec + (size_t)(taps - 1 + src) * C + c);
      const float4 hi = *reinterpret_cast<const float4*>(rec + (size_t)(taps - 1 + src) * C + c + 4);
      v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    }
    const float4 w0 = *reinterpret_cast<const float4*>(w + (size_t)i * C + c), w1 = *reinterpret_cast<const float4*>(w + (size_t)i * C + c + 4);
    acc[0] += w0.x * v[0]; acc[1] += w0.y * v[1]; acc[2] += w0.z * v[2]; acc[3] += w0.w * v[3];
    acc[4] += w1.x * v[4]; acc[5] += w1.y * v[5]; acc[6] += w1.z * v[6]; acc[7] += w1.w * v[7];
  }
  uint4 packed;
  __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int e = 0; e < 4; ++e)
    p2[e] = __floats2bfloat162_rn(silu ? dr_silu(acc[2 * e]) : acc[2 * e], silu ? dr_silu(acc[2 * e + 1]) : acc[2 * e + 1]);
  *reinterpret_cast<uint4*>(out + (size_t)t * out_stride + c) = packed;
}

// One thread per (sequence, channel): the record after the step's tokens.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ x, int x_stride, float* __restrict__ state, const int* __restrict__ slot_ids,
                                        const int* __restrict__ seq_start, int n_seqs, int C, int taps) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n_seqs * C) return;
  const int s = (int)(idx / C), c = (int)(idx - (long long)s * C);
  const int start = seq_start[s], n = seq_start[s + 1] - start;
  float* rec = state + (size_t)slot_ids[s] * (taps - 1) * C;
  float keep[CONV_MAX_TAPS - 1];
  for (int j = 0; j < taps - 1; ++j) {
    const int src = n - (taps - 1) + j;
    keep[j] = src >= 0 ? to_f32(x[(size_t)(start + src) * x_stride + c]) : rec[(size_t)(j + n) * C + c];
  }
  for (int j = 0; j < taps - 1; ++j) rec[(size_t)j * C + c] = keep[j];
}

RL_API int rl_short_conv(const void* x, int dtype, int x_stride, const float* w, float* state, const int* slot_ids, const int* seq_start,
                         const int* tok_seq, void* out, int out_stride, int n_tokens, int n_seqs, int C, int taps, int silu,
                         cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0 || C <= 0) RL_REFUSE(1, "short_conv: T=%d S=%d C=%d", n_tokens, n_seqs, C);
  if (taps < 1 || taps > CONV_MAX_TAPS) RL_REFUSE(2, "short_conv: %d taps (1 to %d)", taps, CONV_MAX_TAPS);
  if (x_stride < C || out_stride < C) RL_REFUSE(3, "short_conv: rows shorter than %d channels", C);
  if (taps > 1 && state == nullptr) RL_REFUSE(4, "short_conv: no record of earlier inputs");
  const int threads = 256;
  const long long total = (long long)n_tokens * C, total_s = (long long)n_seqs * C;
  const int blocks = (int)((total + threads - 1) / threads), blocks_s = (int)((total_s + threads - 1) / threads);
  if (dtype == RL_BF16) {
    // (which of the two kernels runs depends on sizes and addresses only, never on the batch)
    const bool rows8 = C % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && ((((uintptr_t)x | (uintptr_t)out | (uintptr_t)state | (uintptr_t)w) & 15) == 0);
    if (rows8)
      short_conv_rows8_kernel<<<(int)((total / 8 + threads - 1) / threads), threads, 0, stream>>>((const bf16*)x, x_stride, w, state, slot_ids, seq_start,
                                                                                                   tok_seq, (bf16*)out, out_stride, n_tokens, C, taps, silu);
    else
      short_conv_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)x, x_stride, w, state, slot_ids, seq_start, tok_seq, (bf16*)out,
                                                              out_stride, n_tokens, C, taps, silu);
    if (taps > 1)
      short_conv_state_kernel<bf16><<<blocks_s, threads, 0, stream>>>((const bf16*)x, x_stride, state, slot_ids, seq_start, n_seqs, C, taps);
  } else if (dtype == RL_F32) {
    short_conv_kernel<float><<<blocks, threads, 0, stream>>>((const float*)x, x_stride, w, state, slot_ids, seq_start, tok_seq, (float*)out,
                                                             out_stride, n_tokens, C, taps, silu);
    if (taps > 1)
      short_conv_state_kernel<float><<<blocks_s, threads, 0, stream>>>((const float*)x, x_stride, state, slot_ids, seq_start, n_seqs, C, taps);
  } else {
    RL_REFUSE(5, "short_conv: unknown dtype %d", dtype);
  }
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- unit vectors, write strength, decay
// One block per token, a warp per q/k head pair.  qk: [T, >= 2 G dim] rows (G q heads, then G k heads); ba: [T, >= 2 H] rows (H
// numbers b, then H numbers a).  qn, kn: float32 [T, G dim]; kq: float32 [T, G]; beta, decay: float32 [T, H].
template <typename T>
__global__ void delta_prep_kernel(const T* __restrict__ qk, int qk_stride, const T* __restrict__ ba, int ba_stride,
                                  const float* __restrict__ a_log, const float* __restrict__ dt_bias, float unit_eps, float q_scale,
                                  float* __restrict__ qn, float* __restrict__ kn, float* __restrict__ kq, float* __restrict__ beta,
                                  float* __restrict__ decay, int G, int H, int dim) {
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const T* row = qk + (size_t)t * qk_stride;
  for (int g = warp; g < G; g += nwarps) {
    const T* qh = row + (size_t)g * dim;
    const T* kh = row + (size_t)(G + g) * dim;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float a = to_f32(qh[i]), b = to_f32(kh[i]);
      sq += a * a;
      sk += b * b;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float iq = q_scale / sqrtf(sq + unit_eps), ik = 1.0f / sqrtf(sk + unit_eps);
    float dot = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float a = to_f32(qh[i]) * iq, b = to_f32(kh[i]) * ik;
      qn[((size_t)t * G + g) * dim + i] = a;
      kn[((size_t)t * G + g) * dim + i] = b;
      dot += a * b;
    }
    dot = warp_sum(dot);
    if (lane == 0) kq[(size_t)t * G + g] = dot;
  }
  const T* bar = ba + (size_t)t * ba_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    beta[(size_t)t * H + h] = 1.0f / (1.0f + expf(-to_f32(bar[h])));
    const float z = to_f32(bar[H + h]) + dt_bias[h];
    const float sp = fmaxf(z, 0.f) + log1pf(expf(-fabsf(z)));
    decay[(size_t)t * H + h] = expf(-expf(a_log[h]) * sp);
  }
}

RL_API int rl_delta_prep(const void* qk, int dtype, int qk_stride, const void* ba, int ba_stride, const float* a_log, const float* dt_bias,
                         float unit_eps, float q_scale, float* qn, float* kn, float* kq, float* beta, float* decay, int n_tokens, int G, int H,
                         int dim, cudaStream_t stream) {
  if (n_tokens <= 0 || G <= 0 || H <= 0 || dim <= 0) RL_REFUSE(1, "delta_prep: T=%d G=%d H=%d dim=%d", n_tokens, G, H, dim);
  if (qk_stride < 2 * G * dim || ba_stride < 2 * H) RL_REFUSE(2, "delta_prep: rows too short");
  int threads = 32 * (G < 8 ? G : 8);
  if (threads < 64) threads = 64;
  if (dtype == RL_BF16)
    delta_prep_kernel<bf16><<<n_tokens, threads, 0, stream>>>((const bf16*)qk, qk_stride, (const bf16*)ba, ba_stride, a_log, dt_bias, unit_eps,
                                                              q_scale, qn, kn, kq, beta, decay, G, H, dim);
  else if (dtype == RL_F32)
    delta_prep_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)qk, qk_stride, (const float*)ba, ba_stride, a_log, dt_bias, unit_eps,
                                                               q_scale, qn, kn, kq, beta, decay, G, H, dim);
  else
    RL_REFUSE(3, "delta_prep: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the recurrence
#define DR_COLS 32    // columns of the state a block owns
#define DR_ROWS 32    // rows of a column a thread holds
#define DR_TOKENS 16  // tokens whose q, k and scalars are staged in shared memory at a time
#define DR_MAX_SLICES 8
// q and k of a staged token lie in shared memory with four floats of padding after every 32, so that the threads of a column,
// who read the same place of different row slices, read different banks, sixteen bytes a load
#define DR_SKEW(d) ((d) + (((d) >> 5) << 2))

// grid (column tiles, H, sequences); block DR_COLS * P threads, P = the row slices of 32 (a power of two): thread
// col * P + slice holds rows 32 slice .. of one column, so a column's slices are neighbouring lanes of one warp and their partial
// sums meet by shuffles, in a fixed order; the block meets only where the next tokens are staged (two stages: the copies of the
// next sixteen tokens run while these sixteen are worked).
// qn, kn: float32 [T, G dim]; kq: [T, G]; v: [T, >= H vdim] rows of T; beta, decay: float32 [T, H];
// state: float32 [slots, H, dim, vdim]; out: float32 [T, H vdim].
__device__ __forceinline__ void dr_cp_async_4(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void dr_cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void dr_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void dr_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <typename T>
__global__ void __launch_bounds__(DR_COLS * DR_MAX_SLICES)
delta_rule_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ kq, const T* __restrict__ v,
                  int v_stride, const float* __restrict__ beta, const float* __restrict__ decay, float* __restrict__ state,
                  const int* __restrict__ slot_ids, const int* __restrict__ seq_start, float* __restrict__ out, int out_stride, int H, int G,
                  int dim, int vdim, int P) {
  // two stages of DR_TOKENS tokens each: q [DR_TOKENS][skewed dim], k likewise, then per token beta, decay, k . q;
  // then v [2][DR_TOKENS][DR_COLS] as 32-bit numbers
  extern __shared__ __align__(16) float sm[];
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int col_l = tid / P, slice = tid - col_l * P;
  const int h = blockIdx.y, s = blockIdx.z, kh = h / (H / G);
  const int col = blockIdx.x * DR_COLS + col_l;
  const bool col_ok = col < vdim;
  const int row0 = slice * DR_ROWS;
  const int padded = P * DR_ROWS;
  const int sdim = DR_SKEW(padded);  // a staged row's length
  const int stage_floats = 2 * DR_TOKENS * sdim + 3 * DR_TOKENS;
  float* v_s = sm + 2 * stage_floats;
  float* S_g = state + (((size_t)slot_ids[s] * H + h) * dim) * vdim;
  float S[DR_ROWS];
#pragma unroll
  for (int r = 0; r < DR_ROWS; ++r) S[r] = (col_ok && row0 + r < dim) ? S_g[(size_t)(row0 + r) * vdim + col] : 0.f;
  // rows past the key size stay zero in both stages for good (their state is zero and stays so)
  for (int i = tid; i < 2 * stage_floats; i += nthreads) sm[i] = 0.f;
  __syncthreads();
  const int t0 = seq_start[s], t1 = seq_start[s + 1];
  auto stage_in = [&](int tb, int st) {  // the copies of up to DR_TOKENS tokens from tb on, asynchronously
    const int nt = min(DR_TOKENS, t1 - tb);
    float* base = sm + st * stage_floats;
    if ((dim & 3) == 0) {  // sixteen bytes a copy (rows of q and k start on 16 bytes, and so do their places in the stage)
      const int quads = dim >> 2;
      for (int i = tid; i < nt * quads; i += nthreads) {
        const int j = i / quads, d = (i - j * quads) << 2;
        dr_cp_async_16(base + j * sdim + DR_SKEW(d), qn + ((size_t)(tb + j) * G + kh) * dim + d);
        dr_cp_async_16(base + DR_TOKENS * sdim + j * sdim + DR_SKEW(d), kn + ((size_t)(tb + j) * G + kh) * dim + d);
      }
    } else {
      for (int i = tid; i < nt * dim; i += nthreads) {
        const int j = i / dim, d = i - j * dim;
        dr_cp_async_4(base + j * sdim + DR_SKEW(d), qn + ((size_t)(tb + j) * G + kh) * dim + d);
        dr_cp_async_4(base + DR_TOKENS * sdim + j * sdim + DR_SKEW(d), kn + ((size_t)(tb + j) * G + kh) * dim + d);
      }
    }
    if (tid < nt) {
      float* sc = base + 2 * DR_TOKENS * sdim;
      dr_cp_async_4(sc + tid, beta + (size_t)(tb + tid) * H + h);
      dr_cp_async_4(sc + DR_TOKENS + tid, decay + (size_t)(tb + tid) * H + h);
      dr_cp_async_4(sc + 2 * DR_TOKENS + tid, kq + (size_t)(tb + tid) * G + kh);
    }
  };
  // the values go through registers (they are widened on the way): asked for before a stage's tokens are worked, put into
  // the other stage afterwards, so that their way from memory is not waited for
  constexpr int V_PER_THREAD = DR_TOKENS * DR_COLS / 32;  // (a block has at least 32 threads)
  float v_reg[V_PER_THREAD];
  auto ask_v = [&](int tb) {
    const int nt = min(DR_TOKENS, t1 - tb);
#pragma unroll
    for (int n = 0; n < V_PER_THREAD; ++n) {
      const int i = tid + n * nthreads;
      const int j = i / DR_COLS, c = i - j * DR_COLS;
      const int cc = blockIdx.x * DR_COLS + c;
      v_reg[n] = (i < nt * DR_COLS && cc < vdim) ? to_f32(v[(size_t)(tb + j) * v_stride + (size_t)h * vdim + cc]) : 0.f;
    }
  };
  auto put_v = [&](int st) {
#pragma unroll
    for (int n = 0; n < V_PER_THREAD; ++n) {
      const int i = tid + n * nthreads;
      if (i < DR_TOKENS * DR_COLS) v_s[st * DR_TOKENS * DR_COLS + i] = v_reg[n];
    }
  };
  if (t0 < t1) {
    stage_in(t0, 0);
    ask_v(t0);
    put_v(0);
  }
  dr_cp_async_commit();
  int st = 0;
  for (int tb = t0; tb < t1; tb += DR_TOKENS, st ^= 1) {
    const int nt = min(DR_TOKENS, t1 - tb);
    const bool more = tb + DR_TOKENS < t1;
    if (more) {  // the stage that the tokens before last used is free: every thread has passed the barrier below since
      stage_in(tb + DR_TOKENS, st ^ 1);
      ask_v(tb + DR_TOKENS);
    }
    dr_cp_async_commit();
    dr_cp_async_wait<1>();
    __syncthreads();
    const float* base = sm + st * stage_floats;
    const float* sc = base + 2 * DR_TOKENS * sdim;
#pragma unroll 2
    for (int j = 0; j < nt; ++j) {
      const float g = sc[DR_TOKENS + j];
      const float4* qj = reinterpret_cast<const float4*>(base + j * sdim + DR_SKEW(row0));
      const float4* kj = reinterpret_cast<const float4*>(base + DR_TOKENS * sdim + j * sdim + DR_SKEW(row0));
      float kr[DR_ROWS];
      float a4[4] = {0.f, 0.f, 0.f, 0.f}, b4[4] = {0.f, 0.f, 0.f, 0.f};  // four running sums each: short chains of dependent additions
#pragma unroll
      for (int r4 = 0; r4 < DR_ROWS / 4; ++r4) {
        const float4 k4 = kj[r4], q4 = qj[r4];
        kr[4 * r4] = k4.x; kr[4 * r4 + 1] = k4.y; kr[4 * r4 + 2] = k4.z; kr[4 * r4 + 3] = k4.w;
        const float qr[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = 4 * r4 + e;
          S[r] *= g;
          a4[e] += S[r] * kr[r];
          b4[e] += S[r] * qr[e];
        }
      }
      float a = (a4[0] + a4[1]) + (a4[2] + a4[3]), b = (b4[0] + b4[1]) + (b4[2] + b4[3]);
      for (int o = 1; o < P; o <<= 1) {  // the slices of a column are neighbouring lanes; every lane ends with the same sums
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
      }
      const float u = sc[j] * (v_s[(st * DR_TOKENS + j) * DR_COLS + col_l] - a);
#pragma unroll
      for (int r = 0; r < DR_ROWS; ++r) S[r] += kr[r] * u;
      if (slice == 0 && col_ok) out[(size_t)(tb + j) * out_stride + (size_t)h * vdim + col] = b + u * sc[2 * DR_TOKENS + j];
    }
    if (more) put_v(st ^ 1);
    __syncthreads();  // this stage may be refilled from the next round on
  }
#pragma unroll
  for (int r = 0; r < DR_ROWS; ++r)
    if (col_ok && row0 + r < dim) S_g[(size_t)(row0 + r) * vdim + col] = S[r];
}

RL_API int rl_delta_rule(const float* qn, const float* kn, const float* kq, const void* v, int dtype, int v_stride, const float* beta,
                         const float* decay, float* state, const int* slot_ids, const int* seq_start, float* out, int out_stride, int n_seqs,
                         int H, int G, int dim, int vdim, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || G <= 0 || dim <= 0 || vdim <= 0) RL_REFUSE(1, "delta_rule: S=%d H=%d G=%d dim=%d vdim=%d", n_seqs, H, G, dim, vdim);
  if (H % G) RL_REFUSE(2, "delta_rule: %d heads are not a multiple of %d q/k heads", H, G);
  int P = 1;
  while (P * DR_ROWS < dim) P <<= 1;
  if (P > DR_MAX_SLICES) RL_REFUSE(3, "delta_rule: key size %d exceeds %d", dim, DR_ROWS * DR_MAX_SLICES);
  if (H > 65535 || n_seqs > 65535) RL_REFUSE(4, "delta_rule: %d heads or %d sequences exceed the grid", H, n_seqs);
  if (v_stride < H * vdim || out_stride < H * vdim) RL_REFUSE(5, "delta_rule: rows shorter than %d values", H * vdim);
  dim3 grid((vdim + DR_COLS - 1) / DR_COLS, H, n_seqs), block(DR_COLS * P);
  const size_t smem = ((size_t)2 * (2 * DR_TOKENS * DR_SKEW(P * DR_ROWS) + 3 * DR_TOKENS) + 2 * DR_TOKENS * DR_COLS) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(delta_rule_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(delta_rule_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (dtype == RL_BF16)
    delta_rule_kernel<bf16><<<grid, block, smem, stream>>>(qn, kn, kq, (const bf16*)v, v_stride, beta, decay, state, slot_ids, seq_start, out,
                                                           out_stride, H, G, dim, vdim, P);
  else if (dtype == RL_F32)
    delta_rule_kernel<float><<<grid, block, smem, stream>>>(qn, kn, kq, (const float*)v, v_stride, beta, decay, state, slot_ids, seq_start, out,
                                                            out_stride, H, G, dim, vdim, P);
  else
    RL_REFUSE(6, "delta_rule: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}
