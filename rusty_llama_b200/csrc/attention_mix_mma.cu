// bfloat16 flash attention on the tensor cores (mma.sync m16n8k16) for the attention with options: keys and values of unequal
// sizes, a window, a sink, a gate and a constant factor on the result, and scores that are mixed across heads before the softmax.
//
// Mixed scores.  s'_h = sum_g mix[h][g] (q_g . k_kv(g)) is linear in the queries, so it is the score of ONE longer query
// against the keys of all kv heads side by side:
//     s'_h = sum_c Q'[h][c] . k_c,    Q'[h][c] = sum_{g in group c} mix[h][g] q_g        (c = kv head)
// `fold_queries` makes Q' (32-bit sums of the rotated queries, stored as bfloat16); the attention kernel then adds the partial
// products of a head's parts c = 0 .. K-1 into one accumulator and goes on as any flash attention does.  Without a mixing
// matrix a head has one part, its own kv head's keys.
//
// A block of four warps owns 64 query rows of one head of one sequence (eight warps and 128 rows for folded queries of a
// prompt, whose many parts in shared memory leave room for one block per SM only).  A key tile is one cache page.  The loads of a tile
// are, in order, the keys of each part and then the values; they go through a ring of three buffers with cp.async, two loads
// ahead of the one in use.  The online softmax (max, sum, rescale) is 32-bit, in base-2 exponents.  Sizes are padded with
// zeros to HD in shared memory, so key and value sizes in multiples of 8 up to 256 are served.  Prompts and single tokens
// alike: a decode step is a batch of sequences with one query row each.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define BN 64   // keys per tile = page size
#define NBUF 3

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
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
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
// d += a(16x16, row) * b(16x8, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------- folded queries
// out[t][h][c][i] = sum over the heads g of kv head c of mix[h][g] * q[t][g][i], in 32-bit, stored as bfloat16.
// One block per token: the token's rotated queries (32-bit) and the mixing matrix in shared memory; a warp makes one
// (head, kv head) part at a time, its lanes the dimensions.
__global__ void __launch_bounds__(256)
fold_queries_kernel(const bf16* __restrict__ q, int q_stride, const float* __restrict__ mix, bf16* __restrict__ out, int H, int K, int kdim) {
  extern __shared__ float fq_s[];  // q [H][kdim], mix [H][H]
  float* q_s = fq_s;
  float* m_s = fq_s + H * kdim;
  const int t = blockIdx.x, rep = H / K;
  const bf16* row = q + (size_t)t * q_stride;
  if (((H * kdim) & 7) == 0 && (((uintptr_t)row) & 15) == 0) {  // sixteen bytes a load, all of a thread's loads in flight at once
#pragma unroll 4
    for (int i = threadIdx.x * 8; i < H * kdim; i += blockDim.x * 8) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + i));
      float f[8];
      bf16x8_to_f32(raw, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) q_s[i + e] = f[e];
    }
  } else {
    for (int i = threadIdx.x; i < H * kdim; i += blockDim.x) q_s[i] = __bfloat162float(row[i]);
  }
#pragma unroll 4
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) m_s[i] = __ldg(mix + i);
  __syncthreads();
  bf16* o = out + (size_t)t * H * K * kdim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  // (a step of few tokens spreads a token's parts over gridDim.y blocks)
  for (int hc = blockIdx.y * nw + warp; hc < H * K; hc += nw * gridDim.y) {
    const int h = hc / K, c = hc - h * K;
    const float* m = m_s + h * H + c * rep;
    const float* qg = q_s + (size_t)c * rep * kdim;
    for (int i = lane; i < kdim; i += 32) {
      float acc = 0.f;
      for (int g = 0; g < rep; ++g) acc += m[g] * qg[g * kdim + i];
      o[(size_t)hc * kdim + i] = __float2bfloat16_rn(acc);
    }
  }
}

RL_API int rl_fold_queries(const void* q, int q_stride, const float* mix, void* out, int n_tokens, int H, int K, int kdim,
                           cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || K <= 0 || kdim <= 0 || H % K || !q || !mix || !out) RL_REFUSE(1, "fold_queries: T=%d H=%d K=%d kdim=%d", n_tokens, H, K, kdim);
  const size_t smem = ((size_t)H * kdim + (size_t)H * H) * sizeof(float);
  if (smem > 48 * 1024) RL_REFUSE(2, "fold_queries: %d heads of %d numbers do not fit shared memory", H, kdim);
  dim3 grid(n_tokens, n_tokens >= 64 ? 1 : 8);
  fold_queries_kernel<<<grid, 256, smem, stream>>>((const bf16*)q, q_stride, mix, (bf16*)out, H, K, kdim);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the attention
// Copy rows [n_rows][width] (row stride src_stride) into rows of `stride` elements; width a multiple of 8.
template <int NTHREADS>
__device__ __forceinline__ void load_rows(bf16* dst, const bf16* src, size_t src_stride, int n_rows, int width, int stride) {
  const int chunks = width >> 3;
  for (int c = threadIdx.x; c < n_rows * chunks; c += NTHREADS) {
    const int r = c / chunks, cc = c - r * chunks;
    cp_async_16(dst + (size_t)r * stride + cc * 8, src + (size_t)r * src_stride + cc * 8);
  }
}

template <int HD, int BM>
__global__ void __launch_bounds__(BM * 2)
flash_mix_kernel(const bf16* __restrict__ q, long long q_row_stride, int q_head_stride, int parts, const bf16* __restrict__ k_pages,
                 const bf16* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                 const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, const float* __restrict__ sink,
                 const bf16* __restrict__ gate, int gate_stride, float out_scale, bf16* __restrict__ out, int out_stride, int H, int K,
                 int kdim, int vdim, int window, float scale_log2, int chunk, float softcap) {
  constexpr int STRIDE = HD + 8;  // 16 bytes of padding per row keep ldmatrix free of bank conflicts
  constexpr int KSTEPS = HD / 16;
  constexpr int NTHREADS = BM * 2;  // a warp per 16 query rows
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);  // NBUF x [BN][STRIDE]
  bf16* q_s = ring + NBUF * BN * STRIDE;           // parts x [BM][STRIDE]

  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int tok0 = seq_start[s];
  const int q_len = seq_start[s + 1] - tok0;
  const int row0 = (int)(gridDim.y - 1 - blockIdx.y) * BM;  // the row tiles with the most keys start first
  if (row0 >= q_len) return;
  const int pos0 = seq_pos0[s];
  const int kh = h / (H / K);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int rows_here = min(BM, q_len - row0);

  // ---- zero everything once (padding columns, rows past the end), then load the query parts
  {
    uint4 z = make_uint4(0, 0, 0, 0);
    uint4* p = reinterpret_cast<uint4*>(smem_raw);
    const int n16 = ((NBUF * BN + parts * BM) * STRIDE * (int)sizeof(bf16)) / 16;
    for (int i = tid; i < n16; i += NTHREADS) p[i] = z;
  }
  __syncthreads();
  for (int p = 0; p < parts; ++p)
    load_rows<NTHREADS>(q_s + (size_t)p * BM * STRIDE, q + (size_t)(tok0 + row0) * q_row_stride + (size_t)h * q_head_stride + (size_t)p * kdim,
              (size_t)q_row_stride, rows_here, kdim, STRIDE);
  const int* table = block_table + (size_t)s * table_width;
  const int last_pos = pos0 + row0 + rows_here - 1;
  const int first_pos = pos0 + row0;
  const int lowest_key = rl_first_key(first_pos, window, chunk);
  const int tile_lo = lowest_key / BN, tile_hi = last_pos / BN;
  const int per_tile = parts + 1;
  const int n_loads = (tile_hi - tile_lo + 1) * per_tile;
  auto issue = [&](int n) {
    const int tile = tile_lo + n / per_tile, part = n % per_tile;
    bf16* dst = ring + (size_t)(n % NBUF) * BN * STRIDE;
    const size_t page = (size_t)table[tile];
    if (part < parts) {
      const int kv = parts > 1 ? part : kh;
      load_rows<NTHREADS>(dst, k_pages + ((page * K + kv) * BN) * kdim, (size_t)kdim, BN, kdim, STRIDE);
    } else {
      load_rows<NTHREADS>(dst, v_pages + ((page * K + kh) * BN) * vdim, (size_t)vdim, BN, vdim, STRIDE);
    }
  };
  issue(0);
  cp_async_commit();  // (the queries travel in this group too)
  if (n_loads > 1) issue(1);
  cp_async_commit();

  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};  // per-thread partial sums, reduced over the quad at the end
  if (sink != nullptr) {        // a key without a value whose score is sink[h]
    m_run[0] = m_run[1] = sink[h] * 1.4426950408889634f;
    l_run[0] = l_run[1] = (t4 == 0) ? 1.f : 0.f;
  }
  const int qpos[2] = {first_pos + warp * 16 + g, first_pos + warp * 16 + g + 8};
  const int qlow[2] = {rl_first_key(qpos[0], window, chunk), rl_first_key(qpos[1], window, chunk)};
  float s_acc[BN / 8][4];

  for (int n = 0; n < n_loads; ++n) {
    if (n + 2 < n_loads) issue(n + 2);
    cp_async_commit();  // (an empty group where nothing was issued keeps the count of groups in step)
    cp_async_wait<2>();
    __syncthreads();
    const int tile = tile_lo + n / per_tile, part = n % per_tile;
    const bf16* buf = ring + (size_t)(n % NBUF) * BN * STRIDE;
    if (part < parts) {
      // ---- S (+)= Q_part K^T for this warp's 16 rows and the tile's 64 keys
      if (part == 0) {
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f;
      }
      const bf16* qp = q_s + (size_t)part * BM * STRIDE;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, qp + (size_t)(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, buf + (size_t)(np * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + kk * 16 + 8 * ((lane >> 3) & 1));
          mma_bf16(s_acc[2 * np], a, b[0], b[1]);
          mma_bf16(s_acc[2 * np + 1], a, b[2], b[3]);
        }
      }
    } else {
      // ---- mask, scale (to base-2 exponents) and the online softmax
      const int key0 = tile * BN;
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nn = 0; nn < BN / 8; ++nn) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          float v = rl_score_log2(s_acc[nn][e], scale_log2, softcap);
          const int key = key0 + nn * 8 + 2 * t4 + (e & 1);
          const bool seen = key <= qpos[r] && key >= qlow[r];
          if (!seen) v = -INFINITY;
          s_acc[nn][e] = v;
          tile_max[r] = fmaxf(tile_max[r], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = tile_max[r];
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;  // a row that has seen no key yet keeps exponent base 0
        alpha[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int nn = 0; nn < BN / 8; ++nn) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = e >> 1;
          const float p = exp2f(s_acc[nn][e] - m_use[r]);
          s_acc[nn][e] = p;
          l_run[r] += p;
        }
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o_acc[i][0] *= alpha[0];
        o_acc[i][1] *= alpha[0];
        o_acc[i][2] *= alpha[1];
        o_acc[i][3] *= alpha[1];
      }
      // ---- O += P V
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
        a[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
        a[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
        a[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, buf + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
          mma_bf16(o_acc[2 * dp], a, b[0], b[1]);
          mma_bf16(o_acc[2 * dp + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // all warps done with this buffer before it is refilled
  }

  // ---- normalise, gate, scale and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = (l > 0.f) ? out_scale / l : 0.f;
    const int row = warp * 16 + g + 8 * r;
    if (row < rows_here) {
      const size_t t = (size_t)(tok0 + row0 + row);
      bf16* o = out + t * out_stride + (size_t)h * vdim;
      const bf16* gr = gate ? gate + t * gate_stride + (size_t)h * vdim : nullptr;
#pragma unroll
      for (int nn = 0; nn < HD / 8; ++nn) {
        const int d = nn * 8 + 2 * t4;
        if (d < vdim) {
          float a0 = o_acc[nn][2 * r] * inv, a1 = o_acc[nn][2 * r + 1] * inv;
          if (gr) {
            a0 *= 1.0f / (1.0f + expf(-__bfloat162float(gr[d])));
            a1 *= 1.0f / (1.0f + expf(-__bfloat162float(gr[d + 1])));
          }
          *reinterpret_cast<__nv_bfloat162*>(o + d) = __floats2bfloat162_rn(a0, a1);
        }
      }
    }
  }
}

template <int HD, int BM>
static int launch_mix_rows(const bf16* q, long long q_row_stride, int q_head_stride, int parts, const bf16* k_pages, const bf16* v_pages,
                      const int* block_table, int table_width, const int* seq_start, const int* seq_pos0, const float* sink,
                      const bf16* gate, int gate_stride, float out_scale, bf16* out, int out_stride, int n_seqs, int max_q_len, int H, int K,
                      int kdim, int vdim, int window, float scale, int chunk, float softcap, cudaStream_t stream) {
  const size_t smem = (size_t)(NBUF * BN + parts * BM) * (HD + 8) * sizeof(bf16);
  auto kern = flash_mix_kernel<HD, BM>;
  if (smem > 227 * 1024) RL_REFUSE(8, "flash_mix: %zu bytes of shared memory for %d query parts exceed the SM's", smem, parts);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(8, "flash_mix: cannot get %zu bytes of shared memory", smem);
  }
  dim3 grid(H * n_seqs, (max_q_len + BM - 1) / BM);
  kern<<<grid, BM * 2, smem, stream>>>(q, q_row_stride, q_head_stride, parts, k_pages, v_pages, block_table, table_width, seq_start,
                                         seq_pos0, sink, gate, gate_stride, out_scale, out, out_stride, H, K, kdim, vdim, window,
                                         scale * 1.4426950408889634f, chunk, softcap);
  RL_LAUNCH_RESULT();
}

template <int HD>
static int launch_mix(const bf16* q, long long q_row_stride, int q_head_stride, int parts, const bf16* k_pages, const bf16* v_pages,
                      const int* block_table, int table_width, const int* seq_start, const int* seq_pos0, const float* sink,
                      const bf16* gate, int gate_stride, float out_scale, bf16* out, int out_stride, int n_seqs, int max_q_len, int H, int K,
                      int kdim, int vdim, int window, float scale, int chunk, float softcap, cudaStream_t stream) {
  // 128 rows to a block where several query parts would leave one block of 64 rows alone on its SM anyway and the step has
  // the rows to fill it
  const size_t smem128 = (size_t)(NBUF * BN + parts * 128) * (HD + 8) * sizeof(bf16);
  const size_t smem64 = (size_t)(NBUF * BN + parts * 64) * (HD + 8) * sizeof(bf16);
  if (HD <= 128 && parts > 1 && max_q_len > 64 && smem128 <= 227 * 1024 && 2 * smem64 > 227 * 1024)
    return launch_mix_rows<HD, 128>(q, q_row_stride, q_head_stride, parts, k_pages, v_pages, block_table, table_width, seq_start, seq_pos0,
                                    sink, gate, gate_stride, out_scale, out, out_stride, n_seqs, max_q_len, H, K, kdim, vdim, window, scale,
                                    chunk, softcap, stream);
  return launch_mix_rows<HD, 64>(q, q_row_stride, q_head_stride, parts, k_pages, v_pages, block_table, table_width, seq_start, seq_pos0, sink,
                                 gate, gate_stride, out_scale, out, out_stride, n_seqs, max_q_len, H, K, kdim, vdim, window, scale, chunk, softcap, stream);
}

// q: the queries [T][..], row stride q_row_stride, head h at h * q_head_stride, part p of a head at + p * kdim.
// parts: 1 (a head reads its own kv head's keys) or K (folded queries: part c goes against the keys of kv head c).
RL_API int rl_flash_mix(const void* q, long long q_row_stride, int q_head_stride, int parts, const void* k_pages, const void* v_pages,
                        const int* block_table, int table_width, const int* seq_start, const int* seq_pos0, const float* sink,
                        const void* gate, int gate_stride, float out_scale, void* out, int out_stride, int n_seqs, int max_q_len, int H,
                        int K, int kdim, int vdim, int page_size, int window, float scale, int chunk, float softcap, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || H <= 0 || K <= 0 || kdim <= 0 || vdim <= 0)
    RL_REFUSE(1, "flash_mix: S=%d max_q=%d H=%d K=%d kdim=%d vdim=%d", n_seqs, max_q_len, H, K, kdim, vdim);
  if (H % K) RL_REFUSE(2, "flash_mix: %d query heads are not a multiple of %d kv heads", H, K);
  if (page_size != BN) RL_REFUSE(3, "flash_mix: page size %d, this kernel is built for %d", page_size, BN);
  if (kdim % 8 || vdim % 8) RL_REFUSE(4, "flash_mix: key and value sizes %d / %d must be multiples of 8", kdim, vdim);
  if (q_row_stride % 8 || q_head_stride % 8 || out_stride % 2 || gate_stride % 2 || ((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages) % 16 ||
      ((uintptr_t)out | (uintptr_t)gate) % 4)
    RL_REFUSE(5, "flash_mix: strides or addresses break the alignment of 16-byte copies and paired stores");
  if ((long long)H * n_seqs > 0x7fffffffLL || max_q_len / 16 > 65535) RL_REFUSE(6, "flash_mix: the grid is too large");
  if (window < 0 || chunk < 0 || softcap < 0.f || (parts != 1 && parts != K))
    RL_REFUSE(7, "flash_mix: window %d, chunk %d, cap %g, parts %d of %d kv heads", window, chunk, (double)softcap, parts, K);
  const int hd = kdim > vdim ? kdim : vdim;
#define RL_MIX(HDV)                                                                                                                   \
  return launch_mix<HDV>((const bf16*)q, q_row_stride, q_head_stride, parts, (const bf16*)k_pages, (const bf16*)v_pages, block_table,  \
                         table_width, seq_start, seq_pos0, sink, (const bf16*)gate, gate_stride, out_scale, (bf16*)out, out_stride,      \
                         n_seqs, max_q_len, H, K, kdim, vdim, window, scale, chunk, softcap, stream)
  if (hd <= 32) RL_MIX(32);
  if (hd <= 64) RL_MIX(64);
  if (hd <= 128) RL_MIX(128);
  if (hd <= 256) RL_MIX(256);
#undef RL_MIX
  RL_REFUSE(9, "flash_mix: head size %d exceeds 256", hd);
}

// ---------------------------------------------------------------- decode steps: the rows of a block are HEADS
// One query token per sequence.  A block takes one sequence and one part of its key range, with the folded queries of ALL
// heads as the rows of its products (a warp per 16 heads): a key tile of kv head c is read once and meets part c of every
// head's query, where a block per head would read every kv head's keys again for every head.  The values differ from row
// to row (head h reads kv head h / (H / K)): for each kv head in turn the probabilities of the rows that do not read it are
// set to zero before the product, and all rows add into one accumulator.  Each block leaves its maximum (base-2 exponent),
// sum and unnormalised result per head; `flash_mix_merge_kernel` adds the parts of a key range up and applies gate and factor.
template <int HD>
__global__ void flash_mix_decode_kernel(const bf16* __restrict__ qf, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                                        const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_pos0,
                                        const float* __restrict__ sink, float* __restrict__ part_o, float* __restrict__ part_ml, int H,
                                        int K, int kdim, int vdim, int window, float scale_log2, int n_splits, int chunk, float softcap) {
  constexpr int STRIDE = HD + 8;
  constexpr int KSTEPS = HD / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ring = reinterpret_cast<bf16*>(smem_raw);  // NBUF x [BN][STRIDE]
  bf16* q_s = ring + NBUF * BN * STRIDE;           // K x [rows][STRIDE], rows = 16 * warps
  const int nthreads = blockDim.x, rows = nthreads >> 1;
  const int split = blockIdx.x, s = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int rep = H / K;
  const int pos = seq_pos0[s];  // the token's own position; its key and value are in the cache already
  const int first = rl_first_key(pos, window, chunk);
  const int tile_first = first / BN, n_tiles = pos / BN - tile_first + 1;
  const int per = (n_tiles + n_splits - 1) / n_splits;
  const int tile_lo = tile_first + split * per, tile_hi = min(tile_first + n_tiles, tile_lo + per) - 1;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;  // this thread's two rows (heads)

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  if (sink != nullptr && split == 0) {
    if (r_lo < H) {
      m_run[0] = sink[r_lo] * 1.4426950408889634f;
      l_run[0] = (t4 == 0) ? 1.f : 0.f;
    }
    if (r_hi < H) {
      m_run[1] = sink[r_hi] * 1.4426950408889634f;
      l_run[1] = (t4 == 0) ? 1.f : 0.f;
    }
  }
  if (tile_lo <= tile_hi) {
    {
      uint4 z = make_uint4(0, 0, 0, 0);
      uint4* p = reinterpret_cast<uint4*>(smem_raw);
      const int n16 = ((NBUF * BN + K * rows) * STRIDE * (int)sizeof(bf16)) / 16;
      for (int i = tid; i < n16; i += nthreads) p[i] = z;
    }
    __syncthreads();
    const int chunks = kdim >> 3;
    const bf16* qrow = qf + (size_t)s * H * K * kdim;  // [H][K][kdim]
    for (int c = tid; c < H * K * chunks; c += nthreads) {
      const int cc = c % chunks, hp = c / chunks, part = hp % K, h = hp / K;
      cp_async_16(q_s + ((size_t)part * rows + h) * STRIDE + cc * 8, qrow + (size_t)hp * kdim + cc * 8);
    }
    const int* table = block_table + (size_t)s * table_width;
    const int per_tile = 2 * K;
    const int n_loads = (tile_hi - tile_lo + 1) * per_tile;
    auto issue = [&](int n) {
      const int tile = tile_lo + n / per_tile, part = n % per_tile;
      bf16* dst = ring + (size_t)(n % NBUF) * BN * STRIDE;
      const size_t page = (size_t)table[tile];
      const bool is_k = part < K;
      const int kv = is_k ? part : part - K, width = is_k ? kdim : vdim;
      const bf16* src = (is_k ? k_pages : v_pages) + ((page * K + kv) * BN) * width;
      const int ch = width >> 3;
      for (int c = tid; c < BN * ch; c += nthreads) {
        const int r = c / ch, cc = c - r * ch;
        cp_async_16(dst + (size_t)r * STRIDE + cc * 8, src + (size_t)r * width + cc * 8);
      }
    };
    issue(0);
    cp_async_commit();
    if (n_loads > 1) issue(1);
    cp_async_commit();
    float s_acc[BN / 8][4];
    // kv heads that this warp's sixteen rows read
    const int c_first = (warp * 16) / rep, c_last = min(H - 1, warp * 16 + 15) / rep;
    const int kv_lo = r_lo / rep, kv_hi = r_hi / rep;
    for (int n = 0; n < n_loads; ++n) {
      if (n + 2 < n_loads) issue(n + 2);
      cp_async_commit();
      cp_async_wait<2>();
      __syncthreads();
      const int tile = tile_lo + n / per_tile, part = n % per_tile;
      const bf16* buf = ring + (size_t)(n % NBUF) * BN * STRIDE;
      if (part < K) {
        if (part == 0) {
#pragma unroll
          for (int i = 0; i < BN / 8; ++i) s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f;
        }
        const bf16* qp = q_s + (size_t)part * rows * STRIDE;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          uint32_t a[4];
          ldmatrix_x4(a, qp + (size_t)(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
          for (int np = 0; np < BN / 16; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, buf + (size_t)(np * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + kk * 16 + 8 * ((lane >> 3) & 1));
            mma_bf16(s_acc[2 * np], a, b[0], b[1]);
            mma_bf16(s_acc[2 * np + 1], a, b[2], b[3]);
          }
        }
      } else {
        const int c = part - K;
        if (c == 0) {
          // ---- the tile's scores are complete: mask, scale and the online softmax, once per tile
          const int key0 = tile * BN;
          float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
          for (int nn = 0; nn < BN / 8; ++nn) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = key0 + nn * 8 + 2 * t4 + (e & 1);
              float v = rl_score_log2(s_acc[nn][e], scale_log2, softcap);
              if (key > pos || key < first) v = -INFINITY;
              s_acc[nn][e] = v;
              tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
            }
          }
          float alpha[2], m_use[2];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            float mx = tile_max[r];
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[r], mx);
            m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[r] = exp2f(m_run[r] - m_use[r]);
            m_run[r] = m_new;
            l_run[r] *= alpha[r];
          }
#pragma unroll
          for (int nn = 0; nn < BN / 8; ++nn) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float p = exp2f(s_acc[nn][e] - m_use[e >> 1]);
              s_acc[nn][e] = p;
              l_run[e >> 1] += p;
            }
          }
#pragma unroll
          for (int i = 0; i < HD / 8; ++i) {
            o_acc[i][0] *= alpha[0];
            o_acc[i][1] *= alpha[0];
            o_acc[i][2] *= alpha[1];
            o_acc[i][3] *= alpha[1];
          }
        }
        // ---- O += (P of the rows that read kv head c) V_c
        if (c >= c_first && c <= c_last) {
          const bool lo = kv_lo == c, hi = kv_hi == c;
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = lo ? pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]) : 0u;
            a[1] = hi ? pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]) : 0u;
            a[2] = lo ? pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]) : 0u;
            a[3] = hi ? pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]) : 0u;
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
              uint32_t b[4];
              ldmatrix_x4_trans(b, buf + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
              mma_bf16(o_acc[2 * dp], a, b[0], b[1]);
              mma_bf16(o_acc[2 * dp + 1], a, b[2], b[3]);
            }
          }
        }
      }
      __syncthreads();
    }
  }
  // ---- this part's maximum, sum and unnormalised result per head
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int h = r ? r_hi : r_lo;
    if (h < H) {
      const size_t slot = ((size_t)s * H + h) * n_splits + split;
      if (t4 == 0) {
        part_ml[slot * 2] = m_run[r];
        part_ml[slot * 2 + 1] = l;
      }
      float* po = part_o + slot * vdim;
#pragma unroll
      for (int nn = 0; nn < HD / 8; ++nn) {
        const int d = nn * 8 + 2 * t4;
        if (d < vdim) {
          po[d] = o_acc[nn][2 * r];
          po[d + 1] = o_acc[nn][2 * r + 1];
        }
      }
    }
  }
}

// grid (H, S): out[s][h] = sum over the parts of the key range, normalised, times sigmoid(gate) and the factor.
__global__ void flash_mix_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const bf16* __restrict__ gate,
                                       int gate_stride, float out_scale, bf16* __restrict__ out, int out_stride, int H, int vdim,
                                       int n_splits) {
  const int h = blockIdx.x, s = blockIdx.y;
  const size_t base = ((size_t)s * H + h) * n_splits;
  float M = -INFINITY;
  for (int i = 0; i < n_splits; ++i) M = fmaxf(M, part_ml[(base + i) * 2]);
  float denom = 0.f;
  for (int i = 0; i < n_splits; ++i) {
    const float m = part_ml[(base + i) * 2];
    denom += ((m == -INFINITY) ? 0.f : exp2f(m - M)) * part_ml[(base + i) * 2 + 1];
  }
  const float inv = denom > 0.f ? out_scale / denom : 0.f;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < n_splits; ++i) {
      const float m = part_ml[(base + i) * 2];
      if (m != -INFINITY) acc += exp2f(m - M) * part_o[(base + i) * vdim + d];
    }
    acc *= inv;
    if (gate) acc *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)s * gate_stride + (size_t)h * vdim + d])));
    out[(size_t)s * out_stride + (size_t)h * vdim + d] = __float2bfloat16_rn(acc);
  }
}

template <int HD>
static int launch_mix_decode(const bf16* qf, const bf16* k_pages, const bf16* v_pages, const int* block_table, int table_width,
                             const int* seq_pos0, const float* sink, const bf16* gate, int gate_stride, float out_scale, float* part_o,
                             float* part_ml, bf16* out, int out_stride, int n_seqs, int H, int K, int kdim, int vdim, int window, float scale,
                             int n_splits, int chunk, float softcap, cudaStream_t stream) {
  const int warps = (H + 15) / 16;
  const size_t smem = (size_t)(NBUF * BN + K * warps * 16) * (HD + 8) * sizeof(bf16);
  auto kern = flash_mix_decode_kernel<HD>;
  if (smem > 227 * 1024) RL_REFUSE(8, "flash_mix_decode: %zu bytes of shared memory exceed the SM's", smem);
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    RL_REFUSE(8, "flash_mix_decode: cannot get %zu bytes of shared memory", smem);
  dim3 grid(n_splits, n_seqs);
  kern<<<grid, warps * 32, smem, stream>>>(qf, k_pages, v_pages, block_table, table_width, seq_pos0, sink, part_o, part_ml, H, K, kdim, vdim,
                                           window, scale * 1.4426950408889634f, n_splits, chunk, softcap);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(rl_error_buf, sizeof(rl_error_buf), "%s", cudaGetErrorString(e));
    return (int)e;
  }
  dim3 grid2(H, n_seqs);
  flash_mix_merge_kernel<<<grid2, 64, 0, stream>>>(part_o, part_ml, gate, gate_stride, out_scale, out, out_stride, H, vdim, n_splits);
  RL_LAUNCH_RESULT();
}

RL_API int rl_flash_mix_decode_smem(int H, int K, int hd_max) {
  const int HD = hd_max <= 32 ? 32 : (hd_max <= 64 ? 64 : (hd_max <= 128 ? 128 : 256));
  return (NBUF * BN + K * ((H + 15) / 16) * 16) * (HD + 8) * (int)sizeof(bf16);
}

// qf: folded queries [S][H][K][kdim] (`rl_fold_queries`; with the identity as mixing matrix for an attention without mixing).
// seq_pos0[s]: the position of sequence s's token.  part_o: S * H * n_splits * vdim floats, part_ml: S * H * n_splits * 2.
RL_API int rl_flash_mix_decode(const void* qf, const void* k_pages, const void* v_pages, const int* block_table, int table_width,
                               const int* seq_pos0, const float* sink, const void* gate, int gate_stride, float out_scale, float* part_o,
                               float* part_ml, void* out, int out_stride, int n_seqs, int H, int K, int kdim, int vdim, int page_size,
                               int window, float scale, int n_splits, int chunk, float softcap, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || K <= 0 || kdim <= 0 || vdim <= 0 || n_splits <= 0 || !part_o || !part_ml)
    RL_REFUSE(1, "flash_mix_decode: S=%d H=%d K=%d kdim=%d vdim=%d splits=%d", n_seqs, H, K, kdim, vdim, n_splits);
  if (H % K || H > 256) RL_REFUSE(2, "flash_mix_decode: %d heads on %d kv heads (at most 256 heads)", H, K);
  if (page_size != BN) RL_REFUSE(3, "flash_mix_decode: page size %d, this kernel is built for %d", page_size, BN);
  if (kdim % 8 || vdim % 8) RL_REFUSE(4, "flash_mix_decode: key and value sizes %d / %d must be multiples of 8", kdim, vdim);
  if (((uintptr_t)qf | (uintptr_t)k_pages | (uintptr_t)v_pages) % 16) RL_REFUSE(5, "flash_mix_decode: addresses break the alignment of 16-byte copies");
  if (window < 0 || chunk < 0 || softcap < 0.f || n_seqs > 65535)
    RL_REFUSE(6, "flash_mix_decode: window %d, chunk %d, cap %g, %d sequences", window, chunk, (double)softcap, n_seqs);
  const int hd = kdim > vdim ? kdim : vdim;
#define RL_MIXD(HDV)                                                                                                                    \
  return launch_mix_decode<HDV>((const bf16*)qf, (const bf16*)k_pages, (const bf16*)v_pages, block_table, table_width, seq_pos0, sink,    \
                                (const bf16*)gate, gate_stride, out_scale, part_o, part_ml, (bf16*)out, out_stride, n_seqs, H, K, kdim,    \
                                vdim, window, scale, n_splits, chunk, softcap, stream)
  if (hd <= 32) RL_MIXD(32);
  if (hd <= 64) RL_MIXD(64);
  if (hd <= 128) RL_MIXD(128);
  if (hd <= 256) RL_MIXD(256);
#undef RL_MIXD
  RL_REFUSE(9, "flash_mix_decode: head size %d exceeds 256", hd);
}
