// Many small matrix products in one launch, bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit sums):
//
//   moe_gemm_mma     the products of a routed feed-forward: a block takes one row tile of the plan that `moe_plan`
//                    left on the device (rows of ONE expert, gathered through `order`) and 64 columns of that expert's
//                    matrix; with ACT it computes the gate and the up product together and writes gated_act(gate, up) (silu(gate) * up, or the clamped form)
//   head_linear_mma  out[t, h, :] = W[h] x[t, h, :] for every head h, optionally times sigmoid(gate[t, h, :])
//
// Both are the same tile loop: BM rows x BN columns per block, k in slices of 64 through two stages of shared memory
// filled by cp.async (rows and columns past the end, and the tail of k, are filled with zeros).  128 x 64 with four
// warps (each 32 rows x 64 columns) for the many rows of a prompt step, 32 x 64 (each warp 32 rows x 16 columns) for
// the few of a decode step, where the time goes into streaming each expert's matrix once.  k must be a multiple of 8 and
// all rows 16-byte aligned; the plain kernels take everything else.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define GG_BK 64
#define GG_STRIDE (GG_BK + 8)

__device__ __forceinline__ void cp_async_16_zfill(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;  // fewer source bytes than 16: the rest of the 16 is written as zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The tile loop.  a_rows[r]: where row r of the tile starts (nullptr: a row of zeros).  w (and w2 with ACT): [N, K] with
// rows ldw apart; columns n0 .. n0 + BN - 1.  WM x WN warps; a warp holds MT x NT fragments of 16 x 8.
template <int BM, int BN, int WM, int WN, bool ACT>
struct Tile {
  static constexpr int MT = BM / WM / 16, NT = BN / WN / 8, THREADS = WM * WN * 32;
  static constexpr size_t smem_bytes = (size_t)2 * (BM + (ACT ? 2 : 1) * BN) * GG_STRIDE * sizeof(bf16);

  __device__ static void run(const bf16* const* a_rows, const bf16* __restrict__ w, const bf16* __restrict__ w2, int ldw, int N, int K,
                             int n0, bf16* smem, float (&acc)[MT][NT][4], float (&acc2)[ACT ? MT : 1][ACT ? NT : 1][4]) {
    bf16* a_s = smem;                                    // [2][BM][STRIDE]
    bf16* w_s = a_s + (size_t)2 * BM * GG_STRIDE;        // [2][BN][STRIDE]
    bf16* w2_s = w_s + (size_t)2 * BN * GG_STRIDE;    // [2][BN][STRIDE] with ACT
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WN, wn = warp % WN;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
    if (ACT) {
#pragma unroll
      for (int i = 0; i < (ACT ? MT : 1); ++i)
#pragma unroll
        for (int j = 0; j < (ACT ? NT : 1); ++j) acc2[i][j][0] = acc2[i][j][1] = acc2[i][j][2] = acc2[i][j][3] = 0.f;
    }
    auto load = [&](int stage, int k0) {
      bf16* as = a_s + (size_t)stage * BM * GG_STRIDE;
      for (int c = tid; c < BM * (GG_BK / 8); c += THREADS) {
        const int r = c / (GG_BK / 8), k = k0 + (c % (GG_BK / 8)) * 8;
        const bf16* row = a_rows[r];
        const bool ok = row != nullptr && k < K;
        cp_async_16_zfill(as + (size_t)r * GG_STRIDE + (k - k0), ok ? row + k : w, ok);
      }
      bf16* ws = w_s + (size_t)stage * BN * GG_STRIDE;
      bf16* ws2 = w2_s + (size_t)stage * BN * GG_STRIDE;
      for (int c = tid; c < BN * (GG_BK / 8); c += THREADS) {
        const int r = c / (GG_BK / 8), k = k0 + (c % (GG_BK / 8)) * 8;
        const bool ok = n0 + r < N && k < K;
        cp_async_16_zfill(ws + (size_t)r * GG_STRIDE + (k - k0), ok ? w + (size_t)(n0 + r) * ldw + k : w, ok);
        if (ACT) cp_async_16_zfill(ws2 + (size_t)r * GG_STRIDE + (k - k0), ok ? w2 + (size_t)(n0 + r) * ldw + k : w, ok);
      }
    };
    const int n_k = (K + GG_BK - 1) / GG_BK;
    load(0, 0);
    cp_async_commit();
    for (int ks = 0; ks < n_k; ++ks) {
      const int st = ks & 1;
      if (ks + 1 < n_k) {
        load(st ^ 1, (ks + 1) * GG_BK);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const bf16* as = a_s + (size_t)st * BM * GG_STRIDE;
      const bf16* ws = w_s + (size_t)st * BN * GG_STRIDE;
      const bf16* ws2 = w2_s + (size_t)st * BN * GG_STRIDE;
#pragma unroll
      for (int kk = 0; kk < GG_BK / 16; ++kk) {
        uint32_t a[MT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
          ldmatrix_x4(a[i], as + (size_t)(wm * MT * 16 + i * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * GG_STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
          uint32_t b[4];
          const size_t off = (size_t)(wn * NT * 8 + jp * 16 + (lane & 7) + 8 * (lane >> 4)) * GG_STRIDE + kk * 16 + 8 * ((lane >> 3) & 1);
          ldmatrix_x4(b, ws + off);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            mma_bf16(acc[i][2 * jp], a[i], b[0], b[1]);
            mma_bf16(acc[i][2 * jp + 1], a[i], b[2], b[3]);
          }
          if (ACT) {
            ldmatrix_x4(b, ws2 + off);
#pragma unroll
            for (int i = 0; i < (ACT ? MT : 1); ++i) {
              mma_bf16(acc2[i][ACT ? 2 * jp : 0], a[i], b[0], b[1]);
              mma_bf16(acc2[i][ACT ? 2 * jp + 1 : 0], a[i], b[2], b[3]);
            }
          }
        }
      }
      __syncthreads();
    }
  }
};

// ---------------------------------------------------------------- the experts' products
template <int BM, int BN, int WM, int WN, bool ACT, typename TO>
__global__ void __launch_bounds__(WM * WN * 32)
moe_gemm_mma_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ order, int gather_div, const bf16* __restrict__ w,
                    const bf16* __restrict__ w2, TO* __restrict__ out, int ldo, const int* __restrict__ tiles, int N, int K, float act_alpha, float act_limit) {
  using T = Tile<BM, BN, WM, WN, ACT>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ const bf16* a_rows[BM];
  pdl_trigger();
  pdl_wait();
  if ((int)blockIdx.y >= tiles[0]) return;
  const int e = tiles[1 + 3 * blockIdx.y], r0 = tiles[2 + 3 * blockIdx.y], rows = tiles[3 + 3 * blockIdx.y];
  for (int r = threadIdx.x; r < BM; r += T::THREADS)
    a_rows[r] = r < rows ? x + (size_t)(order ? order[r0 + r] / gather_div : r0 + r) * ldx : nullptr;
  __syncthreads();
  float acc[T::MT][T::NT][4], acc2[ACT ? T::MT : 1][ACT ? T::NT : 1][4];
  const int n0 = blockIdx.x * BN;
  T::run(a_rows, w + (size_t)e * N * K, ACT ? w2 + (size_t)e * N * K : nullptr, K, N, K, n0, reinterpret_cast<bf16*>(smem_raw), acc, acc2);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wm = warp / WN, wn = warp % WN, g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int i = 0; i < T::MT; ++i)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = wm * T::MT * 16 + i * 16 + g + 8 * hh;
      if (r >= rows) continue;
#pragma unroll
      for (int j = 0; j < T::NT; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn * T::NT * 8 + j * 8 + 2 * t4 + c;
          if (n >= N) continue;
          float v = acc[i][j][2 * hh + c];
          if (ACT) v = gated_act(v, acc2[ACT ? i : 0][ACT ? j : 0][2 * hh + c], act_alpha, act_limit);
          out[(size_t)(r0 + r) * ldo + n] = from_f32<TO>(v);
        }
    }
}

RL_API int rl_moe_gemm_mma(const void* x, int ldx, const int* order, int gather_div, const void* w, const void* w2, void* out,
                           int out_dtype, int ldo, const int* tiles, int max_tiles, int tile_rows, int N, int K, float act_alpha, float act_limit,
                           cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0 || K <= 0 || gather_div <= 0) RL_REFUSE(1, "moe_gemm_mma: tiles=%d N=%d K=%d div=%d", max_tiles, N, K, gather_div);
  if (max_tiles > 65535) RL_REFUSE(2, "moe_gemm_mma: %d row tiles exceed the grid", max_tiles);
  if (K % 8 || ldx % 8) RL_REFUSE(3, "moe_gemm_mma: k = %d or a row stride of %d elements breaks 16-byte alignment", K, ldx);
  if (tile_rows != 32 && tile_rows != 128) RL_REFUSE(4, "moe_gemm_mma: row tiles of %d, this kernel is built for 32 and 128", tile_rows);
#define RL_GG(BM, BN, WM, WN, ACT, TO)                                                                                              \
  do {                                                                                                                              \
    auto kern = moe_gemm_mma_kernel<BM, BN, WM, WN, ACT, TO>;                                                                       \
    const size_t smem = Tile<BM, BN, WM, WN, ACT>::smem_bytes;                                                                      \
    dim3 grid((N + BN - 1) / BN, max_tiles);                                                                                        \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)      \
      RL_REFUSE(5, "moe_gemm_mma: cannot get %zu bytes of shared memory", smem);                                                    \
    RL_LAUNCH_CHECK(rl_launch<false>(kern, grid, WM * WN * 32, smem, stream, (const bf16*)x, ldx, order, gather_div, (const bf16*)w, \
                                     (const bf16*)w2, (TO*)out, ldo, tiles, N, K, act_alpha, act_limit));                           \
    return 0;                                                                                                                       \
  } while (0)
  const bool act = w2 != nullptr;
  if (tile_rows == 128) {
    // (128 x 128 tiles for eight warps measured slower: gate/up of 64 experts of 1408 x 2048 on 2048 tokens, six each,
    // 790 us against 557: with 166 registers a thread one such block fills an SM, and four of the narrow ones hide more;
    // 256 x 64 with eight warps the same way: 743 us)
    if (act && out_dtype == RL_BF16) RL_GG(128, 64, 4, 1, true, bf16);
    if (!act && out_dtype == RL_F32) RL_GG(128, 64, 4, 1, false, float);
    if (!act && out_dtype == RL_BF16) RL_GG(128, 64, 4, 1, false, bf16);
  } else {
    if (act && out_dtype == RL_BF16) RL_GG(32, 64, 1, 4, true, bf16);
    if (!act && out_dtype == RL_F32) RL_GG(32, 64, 1, 4, false, float);
    if (!act && out_dtype == RL_BF16) RL_GG(32, 64, 1, 4, false, bf16);
  }
#undef RL_GG
  RL_REFUSE(6, "moe_gemm_mma: unsupported output type %d (activation %d)", out_dtype, (int)act);
}

// ---------------------------------------------------------------- one product per head
// x, out, gate: element (t, h, i) at base + t * ld + h * head_stride + i.  w: [H, N, K] dense.
template <int BM, int BN, int WM, int WN, bool GATE>
__global__ void __launch_bounds__(WM * WN * 32)
head_linear_mma_kernel(const bf16* __restrict__ x, int ldx, int xh, const bf16* __restrict__ w, bf16* __restrict__ out, int ldo, int oh,
                       const bf16* __restrict__ gate, int ldg, int gh, int M, int N, int K) {
  using T = Tile<BM, BN, WM, WN, false>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ const bf16* a_rows[BM];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  for (int r = threadIdx.x; r < BM; r += T::THREADS) a_rows[r] = m0 + r < M ? x + (size_t)(m0 + r) * ldx + (size_t)h * xh : nullptr;
  __syncthreads();
  float acc[T::MT][T::NT][4], none[1][1][4];
  T::run(a_rows, w + (size_t)h * N * K, nullptr, K, N, K, n0, reinterpret_cast<bf16*>(smem_raw), acc, none);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wm = warp / WN, wn = warp % WN, g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int i = 0; i < T::MT; ++i)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int m = m0 + wm * T::MT * 16 + i * 16 + g + 8 * hh;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < T::NT; ++j)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int n = n0 + wn * T::NT * 8 + j * 8 + 2 * t4 + c;
          if (n >= N) continue;
          float v = acc[i][j][2 * hh + c];
          if (GATE) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)m * ldg + (size_t)h * gh + n])));
          out[(size_t)m * ldo + (size_t)h * oh + n] = __float2bfloat16_rn(v);
        }
    }
}

// 1 if the tensor-core kernels take operands with these strides (in elements) and this k
RL_API int rl_grouped_gemm_takes(int K, int ldx, int xh) { return K % 8 == 0 && ldx % 8 == 0 && xh % 8 == 0; }

RL_API int rl_head_linear_mma(const void* x, int ldx, int xh, const void* w, void* out, int ldo, int oh, const void* gate, int ldg,
                              int gh, int M, int H, int N, int K, cudaStream_t stream) {
  if (M <= 0 || H <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "head_linear_mma: M=%d H=%d N=%d K=%d", M, H, N, K);
  if (!rl_grouped_gemm_takes(K, ldx, xh)) RL_REFUSE(2, "head_linear_mma: k = %d or strides %d / %d break 16-byte alignment", K, ldx, xh);
  const bool big = M > 32;
  const int BM = big ? 128 : 32;
  const int gy = (M + BM - 1) / BM;
  if (gy > 65535 || H > 65535) RL_REFUSE(3, "head_linear_mma: %d rows or %d heads exceed the grid", M, H);
#define RL_HL(BM, BN, WM, WN, G)                                                                                                    \
  do {                                                                                                                              \
    auto kern = head_linear_mma_kernel<BM, BN, WM, WN, G>;                                                                          \
    const size_t smem = Tile<BM, BN, WM, WN, false>::smem_bytes;                                                                    \
    dim3 grid((N + BN - 1) / BN, gy, H);                                                                                            \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)      \
      RL_REFUSE(5, "head_linear_mma: cannot get %zu bytes of shared memory", smem);                                                 \
    RL_LAUNCH_CHECK(rl_launch<false>(kern, grid, WM * WN * 32, smem, stream, (const bf16*)x, ldx, xh, (const bf16*)w, (bf16*)out,  \
                                     ldo, oh,                                                                                       \
                                     (const bf16*)gate, ldg, gh, M, N, K));                                                         \
    return 0;                                                                                                                       \
  } while (0)
  if (big && gate) RL_HL(128, 64, 4, 1, true);
  if (big) RL_HL(128, 64, 4, 1, false);
  if (gate) RL_HL(32, 64, 1, 4, true);
  RL_HL(32, 64, 1, 4, false);
#undef RL_HL
}
