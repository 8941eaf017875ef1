// A routed feed-forward: every token is sent to `top` of E small gated feed-forwards.
//
//   moe_router   z = W_r x in 32-bit, s = softmax(z) over all experts (or s = logistic(z), each expert on its own); the
//                `top` experts with the largest s + bias are chosen (ties to the lower index), their weights are their s
//                (optionally divided by their sum plus a small constant), times a constant factor; one more row of W_r,
//                if present, gives a per-token gate sigmoid(w_g . x)
//   moe_plan     counts the (token, choice) pairs of each expert, lays them out expert after expert (`order`,
//                with the inverse `place`), and cuts each expert's range into row tiles (`tiles`) of a given height
//   moe_gemm     one kernel for all experts: a block takes one row tile (rows of ONE expert) and one column
//                tile; rows are gathered through `order`; with ACT the block computes the gate and the up
//                product together and writes act(gate) * up
//   moe_combine  out[t] = sum_j weight[t,j] * y[place[t,j]]  (+ gate[t] * shared[t]), in the order j = 0, 1, ...
//
// Nothing here depends on the host knowing how many tokens an expert got: grids are sized by upper bounds and
// blocks without work leave, so a step with these kernels can be captured in a CUDA graph.  Each output is one
// running 32-bit sum over ascending k, whatever the tile it lies in: a token's result does not depend on what
// else is in the batch.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define MOE_TM 32  // rows of a tile: the (token, choice) pairs of one expert, 32 at a time
#define MOE_TN 64
#define MOE_TK 16

// ---------------------------------------------------------------- router
// Two kernels.  Logits: a block takes 8 tokens and 16 rows of w (four per warp), so that a row of w is read once for 8
// tokens and a token's activations once for four rows; every logit is one lane-strided sum
// followed by the warp's fixed reduction, whatever else is in the batch.  Choice: one warp per token.
// w: float32 [E (+1), d]; x in the activation type.
#define ROUTER_TOKENS 8

#define ROUTER_ROWS 4  // rows of w per warp: a token's activations are read once for four logits

template <typename T, bool VEC>
__global__ void moe_router_logits_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, int rows, int d, int n_tokens,
                                         float* __restrict__ z) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e0 = (blockIdx.y * 4 + warp) * ROUTER_ROWS, t0 = blockIdx.x * ROUTER_TOKENS;
  if (e0 >= rows) return;
  float s[ROUTER_ROWS][ROUTER_TOKENS];
#pragma unroll
  for (int r = 0; r < ROUTER_ROWS; ++r)
#pragma unroll
    for (int i = 0; i < ROUTER_TOKENS; ++i) s[r][i] = 0.f;
  if (VEC) {  // d a multiple of 8, rows 16-byte aligned: a lane takes 8 neighbouring k per round
    for (int k = lane * 8; k < d; k += 256) {
      float wv[ROUTER_ROWS][8];
#pragma unroll
      for (int r = 0; r < ROUTER_ROWS; ++r) {
        const float* wr = w + (size_t)min(e0 + r, rows - 1) * d + k;
        load4<float>(wr, wv[r]);
        load4<float>(wr + 4, wv[r] + 4);
      }
#pragma unroll
      for (int i = 0; i < ROUTER_TOKENS; ++i)
        if (t0 + i < n_tokens) {
          float xv[8];
          load4<T>(x + (size_t)(t0 + i) * ldx + k, xv);
          load4<T>(x + (size_t)(t0 + i) * ldx + k + 4, xv + 4);
#pragma unroll
          for (int r = 0; r < ROUTER_ROWS; ++r)
#pragma unroll
            for (int u = 0; u < 8; ++u) s[r][i] += xv[u] * wv[r][u];
        }
    }
  } else {
    for (int k = lane; k < d; k += 32) {
      float wv[ROUTER_ROWS];
#pragma unroll
      for (int r = 0; r < ROUTER_ROWS; ++r) wv[r] = w[(size_t)min(e0 + r, rows - 1) * d + k];
#pragma unroll
      for (int i = 0; i < ROUTER_TOKENS; ++i)
        if (t0 + i < n_tokens) {
          const float xv = to_f32(x[(size_t)(t0 + i) * ldx + k]);
#pragma unroll
          for (int r = 0; r < ROUTER_ROWS; ++r) s[r][i] += xv * wv[r];
        }
    }
  }
#pragma unroll
  for (int r = 0; r < ROUTER_ROWS; ++r)
#pragma unroll
    for (int i = 0; i < ROUTER_TOKENS; ++i) {
      const float v = warp_sum(s[r][i]);
      if (lane == 0 && t0 + i < n_tokens && e0 + r < rows) z[(size_t)(t0 + i) * rows + e0 + r] = v;
    }
}

// One warp per token (four tokens per block): softmax over the E logits (or the logistic function of each), the `top` largest of
// score + bias; weights s_e (/ (sum of the chosen s + renorm_eps) if renorm) * weight_scale.
__global__ void moe_router_choose_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int E, int rows, int top,
                                         int renorm, int n_tokens, int* __restrict__ ids, float* __restrict__ weights,
                                         float* __restrict__ gate, int logistic, float renorm_eps, float weight_scale) {
  extern __shared__ float sm[];  // per warp: E scores, E choice scores
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  float* z = sm + (size_t)warp * 2 * E;
  float* choice = z + E;
  const float* lg = logits + (size_t)t * rows;
  float mx = -INFINITY, sum = 0.f;
  if (!logistic) {
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
    mx = warp_max(mx);
    for (int e = lane; e < E; e += 32) sum += expf(lg[e] - mx);
    sum = warp_sum(sum);
  }
  for (int e = lane; e < E; e += 32) {
    const float s = logistic ? 1.0f / (1.0f + expf(-lg[e])) : expf(lg[e] - mx) / sum;
    z[e] = s;
    choice[e] = s + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  float chosen_sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (choice[e] > best) {  // ascending e within a lane: the lower index keeps a tie
        best = choice[e];
        at = e;
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    if (lane == 0) {
      ids[(size_t)t * top + j] = at;
      weights[(size_t)t * top + j] = z[at];
      choice[at] = -INFINITY;
    }
    chosen_sum += z[at];
    __syncwarp();
  }
  if (lane == 0 && (renorm || weight_scale != 1.0f))
    for (int j = 0; j < top; ++j) {
      float wj = weights[(size_t)t * top + j];
      if (renorm) wj /= (chosen_sum + renorm_eps);
      weights[(size_t)t * top + j] = wj * weight_scale;
    }
  if (rows > E && lane == 0) gate[t] = 1.0f / (1.0f + expf(-lg[E]));
}

// logits: float32 scratch of n_tokens * (E + has_gate) values.
RL_API int rl_moe_router(const void* x, int ldx, int dtype, const float* w, const float* bias, int n_tokens, int E, int d,
                         int top, int renorm, int has_gate, float* logits, int* ids, float* weights, float* gate, int logistic,
                         float renorm_eps, float weight_scale, cudaStream_t stream) {
  if (n_tokens <= 0 || E <= 0 || d <= 0 || top <= 0 || top > E) RL_REFUSE(1, "moe_router: T=%d E=%d d=%d top=%d", n_tokens, E, d, top);
  if (has_gate && gate == nullptr) RL_REFUSE(2, "moe_router: a gate row but nowhere to write the gate");
  const size_t smem = (size_t)4 * 2 * E * sizeof(float);
  if (smem > 48 * 1024) RL_REFUSE(3, "moe_router: %d experts exceed the kernel's shared memory", E);
  const int rows = E + (has_gate ? 1 : 0);
  dim3 grid((n_tokens + ROUTER_TOKENS - 1) / ROUTER_TOKENS, (rows + 4 * ROUTER_ROWS - 1) / (4 * ROUTER_ROWS));
  if (grid.y > 65535) RL_REFUSE(5, "moe_router: %d experts exceed the grid", E);
  // (which of the two loops runs depends on sizes and addresses only, never on the batch: a token's logits keep their bits)
  const bool vec = d % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0);
  if (dtype == RL_BF16 && vec)
    RL_LAUNCH_CHECK(rl_launch<false>(moe_router_logits_kernel<bf16, true>, grid, 128, 0, stream, (const bf16*)x, ldx, w, rows, d, n_tokens, logits));
  else if (dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch<false>(moe_router_logits_kernel<bf16, false>, grid, 128, 0, stream, (const bf16*)x, ldx, w, rows, d, n_tokens, logits));
  else if (dtype == RL_F32 && vec)
    RL_LAUNCH_CHECK(rl_launch<false>(moe_router_logits_kernel<float, true>, grid, 128, 0, stream, (const float*)x, ldx, w, rows, d, n_tokens, logits));
  else if (dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch<false>(moe_router_logits_kernel<float, false>, grid, 128, 0, stream, (const float*)x, ldx, w, rows, d, n_tokens, logits));
  else
    RL_REFUSE(4, "moe_router: unknown dtype %d", dtype);
  RL_LAUNCH_CHECK(rl_launch<false>(moe_router_choose_kernel, (n_tokens + 3) / 4, 128, smem, stream, (const float*)logits, bias, E, rows, top,
                                   renorm, n_tokens, ids, weights, gate, logistic, renorm_eps, weight_scale));
  return 0;
}

// ---------------------------------------------------------------- plan
// ids[n] (n = T * top pairs) -> order[n] (pairs laid out expert after expert, each expert's pairs in ascending
// pair index), place[pair] (its row in that layout), tiles[1 + 3 * max_tiles]: the number of tiles, then
// (expert, first row, rows) per tile.  One block per expert: every block counts all experts' pairs in shared memory
// (it needs the counts of the experts before its own for its first row and its first tile), then lays out its own
// expert's pairs, each thread a contiguous piece of the pairs so that their order is kept.
#define PLAN_THREADS 512

__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const int* __restrict__ ids, int n, int E, int* __restrict__ order, int* __restrict__ place,
                int* __restrict__ tiles, int tile_rows) {
  extern __shared__ int cnt[];  // E counts
  __shared__ int scan[PLAN_THREADS];
  __shared__ int first_row, first_tile;
  pdl_trigger();
  pdl_wait();
  const int e = blockIdx.x, tid = threadIdx.x;
  for (int i = tid; i < E; i += PLAN_THREADS) cnt[i] = 0;
  __syncthreads();
  const int per = (n + PLAN_THREADS - 1) / PLAN_THREADS;
  const int lo = min(n, tid * per), hi = min(n, lo + per);
  int mine = 0;
  for (int i = lo; i < hi; ++i) {
    const int id = ids[i];
    atomicAdd(&cnt[id], 1);
    mine += id == e;
  }
  scan[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    int at = 0, nt = 0;
    for (int k = 0; k < e; ++k) {
      at += cnt[k];
      nt += (cnt[k] + tile_rows - 1) / tile_rows;
    }
    first_row = at;
    first_tile = nt;
    if (e == E - 1) tiles[0] = nt + (cnt[e] + tile_rows - 1) / tile_rows;
  }
  // exclusive scan of the threads' counts (Hillis-Steele over the block)
  for (int o = 1; o < PLAN_THREADS; o <<= 1) {
    const int v = tid >= o ? scan[tid - o] : 0;
    __syncthreads();
    scan[tid] += v;
    __syncthreads();
  }
  int r = first_row + scan[tid] - mine;
  for (int i = lo; i < hi; ++i)
    if (ids[i] == e) {
      order[r] = i;
      place[i] = r;
      ++r;
    }
  const int c = cnt[e];
  for (int k = tid; k * tile_rows < c; k += PLAN_THREADS) {
    int* t = tiles + 1 + 3 * (first_tile + k);
    t[0] = e;
    t[1] = first_row + k * tile_rows;
    t[2] = min(tile_rows, c - k * tile_rows);
  }
}

// ---------------------------------------------------------------- experts chosen by a table instead of a router
// ids[t][j] = table[token[t]][j], every chosen expert with the weight 1 / top.
__global__ void moe_table_lookup_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int top, int n, int E,
                                        int* __restrict__ ids, float* __restrict__ weights) {
  pdl_trigger();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * top) return;
  const int t = idx / top, j = idx - t * top;
  const int e = table[(size_t)tokens[t] * top + j];
  ids[idx] = min(max(e, 0), E - 1);  // (the loader has checked the table; a stray id must still not index outside the weights)
  weights[idx] = 1.0f / (float)top;
}

RL_API int rl_moe_table_lookup(const int* tokens, const int* table, int top, int n_tokens, int E, int* ids, float* weights, cudaStream_t stream) {
  if (n_tokens <= 0 || top <= 0 || E <= 0) RL_REFUSE(1, "moe_table_lookup: T=%d top=%d E=%d", n_tokens, top, E);
  const int total = n_tokens * top;
  RL_LAUNCH_CHECK(rl_launch(moe_table_lookup_kernel, (total + 255) / 256, 256, 0, stream, tokens, table, top, n_tokens, E, ids, weights));
  return 0;
}

RL_API int rl_moe_tile_rows() { return MOE_TM; }

RL_API int rl_moe_plan(const int* ids, int n, int E, int* order, int* place, int* tiles, int tile_rows, cudaStream_t stream) {
  if (n <= 0 || E <= 0 || tile_rows <= 0) RL_REFUSE(1, "moe_plan: n=%d E=%d tile_rows=%d", n, E, tile_rows);
  const size_t smem = (size_t)E * sizeof(int);
  if (smem > 40 * 1024) RL_REFUSE(2, "moe_plan: %d experts exceed the kernel's shared memory", E);
  RL_LAUNCH_CHECK(rl_launch<false>(moe_plan_kernel, E, PLAN_THREADS, smem, stream, ids, n, E, order, place, tiles, tile_rows));
  return 0;
}

// ---------------------------------------------------------------- all experts' products in one launch
// Row r of the layout belongs to pair order[r]; its input row is x[order[r] / gather_div] when `order` is given
// (the token's activations), else x[r].  w: [E, N, K]; with ACT also w2: [E, N, K] and out = gated_act(x w^T, x w2^T): silu(g) * u,
// or with a limit the clamped form (common.cuh).
// blockIdx.y walks the tiles of the plan; a block beyond the plan's count leaves.
template <typename TA, typename TO, bool ACT>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* __restrict__ x, int ldx, const int* __restrict__ order, int gather_div, const TA* __restrict__ w,
                const TA* __restrict__ w2, TO* __restrict__ out, int ldo, const int* __restrict__ tiles, int N, int K, float act_alpha,
                float act_limit) {
  __shared__ float xs[MOE_TK][MOE_TM + 4];
  __shared__ float ws[MOE_TK][MOE_TN + 4];
  __shared__ float ws2[ACT ? MOE_TK : 1][MOE_TN + 4];
  __shared__ int src[MOE_TM];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.y >= tiles[0]) return;
  const int e = tiles[1 + 3 * blockIdx.y], r0 = tiles[2 + 3 * blockIdx.y], rows = tiles[3 + 3 * blockIdx.y];
  const int tid = threadIdx.x, n0 = blockIdx.x * MOE_TN;
  const int ty = tid / 16, tx = tid % 16;  // 16 x 16 threads: 2 rows x 4 columns each
  if (tid < MOE_TM) src[tid] = tid < rows ? (order ? order[r0 + tid] / gather_div : r0 + tid) : -1;
  __syncthreads();
  const TA* we = w + (size_t)e * N * K;
  const TA* we2 = ACT ? w2 + (size_t)e * N * K : nullptr;
  float acc[2][4], acc2[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = acc2[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += MOE_TK) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * 256;
      const int r = idx / MOE_TK, c = idx % MOE_TK;
      const int k = k0 + c;
      xs[c][r] = (src[r] >= 0 && k < K) ? to_f32(x[(size_t)src[r] * ldx + k]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx / MOE_TK, c = idx % MOE_TK;
      const int k = k0 + c;
      const bool in = n0 + r < N && k < K;
      ws[c][r] = in ? to_f32(we[(size_t)(n0 + r) * K + k]) : 0.f;
      if (ACT) ws2[c][r] = in ? to_f32(we2[(size_t)(n0 + r) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < MOE_TK; ++c) {
      float a[2], b[4], b2[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) a[i] = xs[c][ty * 2 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b[j] = ws[c][tx * 4 + j];
        if (ACT) b2[j] = ws2[c][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (ACT) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (ACT) v = gated_act(v, acc2[i][j], act_alpha, act_limit);
      out[(size_t)(r0 + r) * ldo + n] = from_f32<TO>(v);
    }
  }
}

// (the plan's tiles must be MOE_TM rows high: `rl_moe_tile_rows`)
RL_API int rl_moe_gemm(const void* x, int ldx, int dtype, const int* order, int gather_div, const void* w, const void* w2,
                       void* out, int out_dtype, int ldo, const int* tiles, int max_tiles, int N, int K, float act_alpha, float act_limit,
                       cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0 || K <= 0 || gather_div <= 0) RL_REFUSE(1, "moe_gemm: tiles=%d N=%d K=%d div=%d", max_tiles, N, K, gather_div);
  if (max_tiles > 65535) RL_REFUSE(2, "moe_gemm: %d row tiles exceed the grid", max_tiles);
  dim3 grid((N + MOE_TN - 1) / MOE_TN, max_tiles);
#define RL_MG(TA, TO, ACT)                                                                                                  \
  RL_LAUNCH_CHECK(rl_launch<false>(moe_gemm_kernel<TA, TO, ACT>, grid, 256, 0, stream, (const TA*)x, ldx, order, gather_div, \
                                   (const TA*)w, (const TA*)w2, (TO*)out, ldo, tiles, N, K, act_alpha, act_limit))
  if (dtype == RL_BF16 && out_dtype == RL_BF16 && w2) RL_MG(bf16, bf16, true);
  else if (dtype == RL_BF16 && out_dtype == RL_BF16) RL_MG(bf16, bf16, false);
  else if (dtype == RL_BF16 && out_dtype == RL_F32 && !w2) RL_MG(bf16, float, false);
  else if (dtype == RL_F32 && out_dtype == RL_F32 && w2) RL_MG(float, float, true);
  else if (dtype == RL_F32 && out_dtype == RL_F32) RL_MG(float, float, false);
  else RL_REFUSE(3, "moe_gemm: unsupported types in=%d out=%d act=%d", dtype, out_dtype, w2 != nullptr);
#undef RL_MG
  return 0;
}

// ---------------------------------------------------------------- weighted sum of a token's experts
// out[t, :] = sum_j weights[t, j] * y[place[t * top + j], :]  (+ gate[t] * shared[t, :]); y is float32.
template <typename TS, typename TO>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   int top, const TS* __restrict__ shared, const float* __restrict__ gate, TO* __restrict__ out, int d) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = 0.f;
    for (int j = 0; j < top; ++j) v += weights[(size_t)t * top + j] * y[(size_t)place[(size_t)t * top + j] * d + i];
    if (shared) v += (gate ? gate[t] : 1.f) * to_f32(shared[(size_t)t * d + i]);
    out[(size_t)t * d + i] = from_f32<TO>(v);
  }
}

RL_API int rl_moe_combine(const float* y, const int* place, const float* weights, int top, const void* shared, int shared_dtype,
                          const float* gate, void* out, int out_dtype, int n_tokens, int d, cudaStream_t stream) {
  if (n_tokens <= 0 || d <= 0 || top <= 0) RL_REFUSE(1, "moe_combine: T=%d d=%d top=%d", n_tokens, d, top);
#define RL_MC(TS, TO)                                                                                                          \
  RL_LAUNCH_CHECK(rl_launch<false>(moe_combine_kernel<TS, TO>, n_tokens, 256, 0, stream, y, place, weights, top, (const TS*)shared, \
                                   gate, (TO*)out, d))
  if (shared_dtype == RL_BF16 && out_dtype == RL_F32) RL_MC(bf16, float);
  else if (shared_dtype == RL_F32 && out_dtype == RL_F32) RL_MC(float, float);
  else if (shared_dtype == RL_BF16 && out_dtype == RL_BF16) RL_MC(bf16, bf16);
  else RL_REFUSE(2, "moe_combine: unsupported types shared=%d out=%d", shared_dtype, out_dtype);
#undef RL_MC
  return 0;
}
