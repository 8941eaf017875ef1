// Grouped-query attention whose weights are not a softmax: every visible key gets the weight
//
//     w_h(i, j) = logistic(cap(q_h(i) . k_j * scale) + bias_h),        cap(s) = c tanh(s / c) (or s itself without a cap),
//
// a number per key that depends on no other key (nothing is normalised over the keys), and the heads' weights are then mixed
// by a learned matrix, w'_h(i, j) = sum_g M[h][g] w_g(i, j), before head h applies them to the values of ITS kv head:
//
//     o_h(i) = sum_{j visible} w'_h(i, j) v_kv(h)(j),       out_h(i) = o_h(i) * logistic(gate_h(i)) * out_scale
//
// (the gate one number per head and token).  Visible: j <= i, optionally only the last `window` positions and only the
// query's own chunk of `chunk` positions counted from the sequence's start, as in csrc/attention_ext.cu.  q is rotated and
// k, v lie in the paged cache already (`qkv_prep` of csrc/attention_ext.cu), laid out k_pages[page][kv head][slot][kdim],
// v_pages[...][vdim], the page of position p of batch sequence s being block_table[s][p / page_size].
//
// `sigmoid_attn` takes every size, both element types, prompts and single tokens: one warp per (token, head), the keys 32 at
// a time from the first visible key, every sum in 32-bit and in a fixed order (a lane's dot product over ascending i, the
// weighted values over ascending j), so a result's bits depend neither on how its sequence was cut into steps nor on what
// else is in the batch.  With a mixing matrix the warps of a token's heads share a block and exchange the weights of a group
// of keys through shared memory.
//
// `sigmoid_attn_mma` is the bfloat16 form on the tensor cores (mma.sync m16n8k16) for key and value sizes in multiples of 8
// up to 128.  The mixing is linear in the weights, so it commutes with the sum over the keys:
//
//     o_h = sum_g M[h][g] P[g][kv(h)],       P[g][c] = sum_j w_g(i, j) v_c(j)
//
// A block takes 64 queries of one sequence, ONE query head g and ONE kv head c of values (in a decode step, where every
// sequence brings one token: the heads of one kv head as its rows, so that their keys are read once): S = Q_g
// K_kv(g)^T per key tile of one page as in any flash kernel, the weights from the 32-bit scores in registers (no running
// maximum, no rescaling: the sum over the keys is a plain sum), rounded to bfloat16 for the product with V_c, P[g][c] in
// 32-bit registers.  With a mixing matrix the grid has a block for every c, without one only for c = kv(g).  P goes to a
// float32 scratch [parts, T, H, C, vdim]; `sigmoid_attn_mix` then forms out_h = gate_h * sum_g M[h][g] P[g][kv(h)] in 32-bit,
// adding up the parts into which a decode step cuts a sequence's keys (they add plainly, since nothing is normalised).
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define SIG_MAX_V_PER_LANE 8  // value sizes up to 256

__device__ __forceinline__ float sig_weight(float dot, float scale, float softcap, float bias) {
  float s = dot * scale;
  if (softcap > 0.f) s = softcap * tanhf(s / softcap);
  return 1.0f / (1.0f + expf(-(s + bias)));
}

// blockDim = (32, HB): HB = 1 and grid (T, H) without a mixing matrix; HB = H and grid (T, 1) with one.
template <typename T>
__global__ void sigmoid_attn_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                    const int* __restrict__ block_table, int table_width, const int* __restrict__ tok_seq,
                                    const int* __restrict__ tok_pos, const float* __restrict__ head_bias, const float* __restrict__ mix,
                                    const T* __restrict__ gate, int gate_stride, float out_scale, T* __restrict__ out, int out_stride,
                                    int H, int K, int kdim, int vdim, int page_size, int window, float scale, int chunk, float softcap) {
  extern __shared__ float smem[];  // q of the block's heads [HB][kdim], then (with mix) weights [HB][32]
  const int lane = threadIdx.x;
  const int hb = threadIdx.y, HB = blockDim.y;
  const int t = blockIdx.x, h = blockIdx.y * HB + hb;
  const int kh = h / (H / K);
  const int pos = tok_pos[t];
  const int* table = block_table + (size_t)tok_seq[t] * table_width;
  float* q_s = smem + (size_t)hb * kdim;
  float* sc = smem + (size_t)HB * kdim;
  const T* qh = q + (size_t)t * q_stride + (size_t)h * kdim;
  for (int i = lane; i < kdim; i += 32) q_s[i] = to_f32(qh[i]);
  __syncwarp();
  const float bias = head_bias ? head_bias[h] : 0.f;
  const int first = rl_first_key(pos, window, chunk);
  float acc[SIG_MAX_V_PER_LANE];
#pragma unroll
  for (int i = 0; i < SIG_MAX_V_PER_LANE; ++i) acc[i] = 0.f;

  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    float p = 0.f;
    if (key <= pos) {
      const int page = table[key / page_size];
      const T* kr = k_pages + (((size_t)page * K + kh) * page_size + key % page_size) * kdim;
      float dot = 0.f;
      for (int i = 0; i < kdim; ++i) dot += q_s[i] * to_f32(kr[i]);
      p = sig_weight(dot, scale, softcap, bias);
    }
    if (mix != nullptr) {
      __syncthreads();  // the weights of the group before have been read
      sc[hb * 32 + lane] = p;
      __syncthreads();
      float mixed = 0.f;
      for (int g = 0; g < HB; ++g) mixed += mix[h * HB + g] * sc[g * 32 + lane];
      p = mixed;
    }
    const int count = min(32, pos - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const int page = table[kj / page_size];
      const T* vr = v_pages + (((size_t)page * K + kh) * page_size + kj % page_size) * vdim;
#pragma unroll
      for (int i = 0; i < SIG_MAX_V_PER_LANE; ++i) {
        const int dim = lane + 32 * i;
        if (dim < vdim) acc[i] += pj * to_f32(vr[dim]);
      }
    }
  }
  float g = out_scale;
  if (gate) g *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + h])));
  T* o = out + (size_t)t * out_stride + (size_t)h * vdim;
#pragma unroll
  for (int i = 0; i < SIG_MAX_V_PER_LANE; ++i) {
    const int dim = lane + 32 * i;
    if (dim < vdim) o[dim] = from_f32<T>(acc[i] * g);
  }
}

RL_API int rl_sigmoid_attn(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages, const int* block_table,
                           int table_width, const int* tok_seq, const int* tok_pos, const float* head_bias, const float* mix,
                           const void* gate, int gate_stride, float out_scale, void* out, int out_stride, int n_tokens, int H, int K,
                           int kdim, int vdim, int page_size, int window, float scale, int chunk, float softcap, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || K <= 0 || kdim <= 0 || vdim <= 0 || page_size <= 0)
    RL_REFUSE(1, "sigmoid_attn: T=%d H=%d K=%d kdim=%d vdim=%d page=%d", n_tokens, H, K, kdim, vdim, page_size);
  if (H % K) RL_REFUSE(2, "sigmoid_attn: %d query heads are not a multiple of %d kv heads", H, K);
  if (vdim > 32 * SIG_MAX_V_PER_LANE) RL_REFUSE(3, "sigmoid_attn: value size %d exceeds %d", vdim, 32 * SIG_MAX_V_PER_LANE);
  if (H > 65535) RL_REFUSE(4, "sigmoid_attn: %d heads exceed 65535", H);
  if (window < 0 || chunk < 0) RL_REFUSE(5, "sigmoid_attn: negative window or chunk");
  if (mix != nullptr && H > 32) RL_REFUSE(6, "sigmoid_attn: weights of %d heads cannot be mixed (at most 32)", H);
  const int HB = mix != nullptr ? H : 1;
  dim3 grid(n_tokens, H / HB), block(32, HB);
  const size_t smem = ((size_t)HB * kdim + (mix != nullptr ? (size_t)HB * 32 : 0)) * sizeof(float);
  if (smem > 48 * 1024) RL_REFUSE(7, "sigmoid_attn: %d heads of %d numbers do not fit shared memory", HB, kdim);
  if (dtype == RL_BF16)
    sigmoid_attn_kernel<bf16><<<grid, block, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)k_pages, (const bf16*)v_pages,
                                                             block_table, table_width, tok_seq, tok_pos, head_bias, mix, (const bf16*)gate,
                                                             gate_stride, out_scale, (bf16*)out, out_stride, H, K, kdim, vdim, page_size,
                                                             window, scale, chunk, softcap);
  else if (dtype == RL_F32)
    sigmoid_attn_kernel<float><<<grid, block, smem, stream>>>((const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages,
                                                              block_table, table_width, tok_seq, tok_pos, head_bias, mix, (const float*)gate,
                                                              gate_stride, out_scale, (float*)out, out_stride, H, K, kdim, vdim, page_size,
                                                              window, scale, chunk, softcap);
  else
    RL_REFUSE(8, "sigmoid_attn: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the tensor-core form
#define SG_BN 64  // keys per tile = page size
#define SG_NBUF 3

__device__ __forceinline__ void sg_cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void sg_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void sg_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void sg_ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sg_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// d += a(16x16, row) * b(16x8, col)
__device__ __forceinline__ void sg_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sg_pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Copy rows [n_rows][width] (row stride src_stride) into rows of `stride` elements; width a multiple of 8.
template <int NTHREADS>
__device__ __forceinline__ void sg_load_rows(bf16* dst, const bf16* src, size_t src_stride, int n_rows, int width, int stride) {
  const int chunks = width >> 3;
  for (int c = threadIdx.x; c < n_rows * chunks; c += NTHREADS) {
    const int r = c / chunks, cc = c - r * chunks;
    sg_cp_async_16(dst + (size_t)r * stride + cc * 8, src + (size_t)r * src_stride + cc * 8);
  }
}

// grid (H * n_seqs, row tiles, C * parts); block BM * 2 threads (a warp per 16 query rows).  C = K with `all_values`, else 1.
// part[((p * T + t) * H + h) * C + c][vdim] receives the sum over the keys of part p of w_h(t, j) v_c(j).
// GROUP (a decode step: every sequence brings one token): grid (K * n_seqs, 1, C * parts), and a block's rows are the H / K heads
// of one kv head instead of tokens, so a key tile is read once for all the heads that share it.
template <int HD, int BM, bool GROUP>
__global__ void __launch_bounds__(BM * 2)
sigmoid_attn_mma_kernel(const bf16* __restrict__ q, long long q_row_stride, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_start,
                        const int* __restrict__ seq_pos0, const float* __restrict__ head_bias, float* __restrict__ part, int n_tokens, int H,
                        int K, int kdim, int vdim, int window, float scale, int chunk, float softcap, int all_values, int parts) {
  constexpr int STRIDE = HD + 8;  // 16 bytes of padding per row keep ldmatrix free of bank conflicts
  constexpr int KSTEPS = HD / 16;
  constexpr int NTHREADS = BM * 2;
  extern __shared__ __align__(16) unsigned char sg_smem[];
  bf16* ring = reinterpret_cast<bf16*>(sg_smem);  // SG_NBUF x [SG_BN][STRIDE]
  bf16* q_s = ring + SG_NBUF * SG_BN * STRIDE;     // [BM][STRIDE]

  const int rep = H / K;
  const int s = GROUP ? blockIdx.x / K : blockIdx.x / H;
  const int h = GROUP ? (blockIdx.x % K) * rep : blockIdx.x % H;  // (GROUP: the first head of the block's rows)
  const int tok0 = seq_start[s];
  const int q_len = seq_start[s + 1] - tok0;
  const int row0 = GROUP ? 0 : (int)(gridDim.y - 1 - blockIdx.y) * BM;  // the row tiles with the most keys start first
  if (row0 >= q_len) return;
  const int C = all_values ? K : 1;
  const int c = blockIdx.z % C, p = blockIdx.z / C;
  const int pos0 = seq_pos0[s];
  const int kh = h / rep;
  const int vh = all_values ? c : kh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int rows_here = GROUP ? min(BM, rep) : min(BM, q_len - row0);
  const int last_pos = GROUP ? pos0 : pos0 + row0 + rows_here - 1;
  const int first_pos = pos0 + row0;
  const int lowest_key = rl_first_key(first_pos, window, chunk);
  // the tiles of this block's part of the key range (a part is a run of whole tiles)
  int tile_lo = lowest_key / SG_BN, tile_hi = last_pos / SG_BN;
  {
    const int n_tiles = tile_hi - tile_lo + 1, per = (n_tiles + parts - 1) / parts;
    tile_lo += p * per;
    tile_hi = min(tile_hi, tile_lo + per - 1);
  }
  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  if (tile_lo <= tile_hi) {
    // ---- zero everything once (padding columns, rows past the end), then load the queries
    {
      uint4 z = make_uint4(0, 0, 0, 0);
      uint4* zp = reinterpret_cast<uint4*>(sg_smem);
      const int n16 = ((SG_NBUF * SG_BN + BM) * STRIDE * (int)sizeof(bf16)) / 16;
      for (int i = tid; i < n16; i += NTHREADS) zp[i] = z;
    }
    __syncthreads();
    sg_load_rows<NTHREADS>(q_s, q + (size_t)(tok0 + row0) * q_row_stride + (size_t)h * kdim, GROUP ? (size_t)kdim : (size_t)q_row_stride, rows_here,
                           kdim, STRIDE);
    const int* table = block_table + (size_t)s * table_width;
    const int n_loads = (tile_hi - tile_lo + 1) * 2;
    auto issue = [&](int n) {
      const int tile = tile_lo + (n >> 1);
      bf16* dst = ring + (size_t)(n % SG_NBUF) * SG_BN * STRIDE;
      const size_t page = (size_t)table[tile];
      if ((n & 1) == 0)
        sg_load_rows<NTHREADS>(dst, k_pages + ((page * K + kh) * SG_BN) * kdim, (size_t)kdim, SG_BN, kdim, STRIDE);
      else
        sg_load_rows<NTHREADS>(dst, v_pages + ((page * K + vh) * SG_BN) * vdim, (size_t)vdim, SG_BN, vdim, STRIDE);
    };
    issue(0);
    sg_cp_async_commit();  // (the queries travel in this group too)
    issue(1);
    sg_cp_async_commit();

    float bias[2] = {0.f, 0.f};
    if (head_bias) {
#pragma unroll
      for (int r = 0; r < 2; ++r) bias[r] = GROUP ? head_bias[h + min(warp * 16 + g + 8 * r, rows_here - 1)] : head_bias[h];
    }
    const int qpos[2] = {GROUP ? pos0 : first_pos + warp * 16 + g, GROUP ? pos0 : first_pos + warp * 16 + g + 8};
    const int qlow[2] = {rl_first_key(qpos[0], window, chunk), rl_first_key(qpos[1], window, chunk)};
    const float inv_cap = softcap > 0.f ? scale / softcap : 0.f;
    float s_acc[SG_BN / 8][4];

    for (int n = 0; n < n_loads; ++n) {
      if (n + 2 < n_loads) issue(n + 2);
      sg_cp_async_commit();  // (an empty group where nothing was issued keeps the count of groups in step)
      sg_cp_async_wait<2>();
      __syncthreads();
      const int tile = tile_lo + (n >> 1);
      const bf16* buf = ring + (size_t)(n % SG_NBUF) * SG_BN * STRIDE;
      if ((n & 1) == 0) {
        // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys
#pragma unroll
        for (int i = 0; i < SG_BN / 8; ++i) s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
          uint32_t a[4];
          sg_ldmatrix_x4(a, q_s + (size_t)(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
          for (int np = 0; np < SG_BN / 16; ++np) {
            uint32_t b[4];
            sg_ldmatrix_x4(b, buf + (size_t)(np * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + kk * 16 + 8 * ((lane >> 3) & 1));
            sg_mma_bf16(s_acc[2 * np], a, b[0], b[1]);
            sg_mma_bf16(s_acc[2 * np + 1], a, b[2], b[3]);
          }
        }
      } else {
        // ---- the weights: cap, bias, logistic function; zero for keys a row does not see
        const int key0 = tile * SG_BN;
#pragma unroll
        for (int nn = 0; nn < SG_BN / 8; ++nn) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            float v = softcap > 0.f ? softcap * rl_tanh_sfu(s_acc[nn][e] * inv_cap) : s_acc[nn][e] * scale;
            const int key = key0 + nn * 8 + 2 * t4 + (e & 1);
            const bool seen = key <= qpos[r] && key >= qlow[r];
            s_acc[nn][e] = seen ? __fdividef(1.0f, 1.0f + __expf(-(v + bias[r]))) : 0.f;
          }
        }
        // ---- O += W V
#pragma unroll
        for (int kk = 0; kk < SG_BN / 16; ++kk) {
          uint32_t a[4];
          a[0] = sg_pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
          a[1] = sg_pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
          a[2] = sg_pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
          a[3] = sg_pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
          for (int dp = 0; dp < HD / 16; ++dp) {
            uint32_t b[4];
            sg_ldmatrix_x4_trans(b, buf + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
            sg_mma_bf16(o_acc[2 * dp], a, b[0], b[1]);
            sg_mma_bf16(o_acc[2 * dp + 1], a, b[2], b[3]);
          }
        }
      }
      __syncthreads();  // all warps done with this buffer before it is refilled
    }
  }
  // ---- store the 32-bit sums (zeros from a part that got no tile)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row < rows_here) {
      const size_t t = GROUP ? (size_t)tok0 : (size_t)(tok0 + row0 + row);
      float* o = part + ((((size_t)p * n_tokens + t) * H + (GROUP ? h + row : h)) * C + c) * vdim;
#pragma unroll
      for (int nn = 0; nn < HD / 8; ++nn) {
        const int d = nn * 8 + 2 * t4;
        if (d < vdim) *reinterpret_cast<float2*>(o + d) = make_float2(o_acc[nn][2 * r], o_acc[nn][2 * r + 1]);
      }
    }
  }
}

// out[t][h][:] = out_scale * logistic(gate[t][h]) * sum_p sum_g mix[h][g] part[p][t][g][kv(h)][:]   (with a mixing matrix)
//              = out_scale * logistic(gate[t][h]) * sum_p part[p][t][h][0][:]                         (without)
// A block per (token, kv head c): the sums over the parts of all heads' P[.][c] in shared memory (every load in flight at once),
// then a thread per (head of kv head c, value).  Without a mixing matrix C = 1 and the block makes all heads.
__global__ void sigmoid_attn_mix_kernel(const float* __restrict__ part, int parts, const float* __restrict__ mix, const bf16* __restrict__ gate,
                                        int gate_stride, float out_scale, bf16* __restrict__ out, int out_stride, int n_tokens, int H, int K,
                                        int vdim) {
  extern __shared__ float sums[];  // [H][vdim]
  const int t = blockIdx.x, c = blockIdx.y;
  const int rep = H / K, C = mix ? K : 1;
  for (int i = threadIdx.x; i < H * vdim; i += blockDim.x) {
    const int gh = i / vdim, d = i - gh * vdim;
    float acc = 0.f;
    for (int p = 0; p < parts; ++p) acc += part[((((size_t)p * n_tokens + t) * H + gh) * C + c) * vdim + d];
    sums[i] = acc;
  }
  __syncthreads();
  const int n_heads = mix ? rep : H;  // the heads whose values are kv head c's (all heads when nothing is mixed)
  for (int i = threadIdx.x; i < n_heads * vdim; i += blockDim.x) {
    const int hl = i / vdim, d = i - hl * vdim;
    const int h = mix ? c * rep + hl : hl;
    float acc;
    if (mix) {
      acc = 0.f;
      for (int gh = 0; gh < H; ++gh) acc += mix[h * H + gh] * sums[gh * vdim + d];
    } else {
      acc = sums[h * vdim + d];
    }
    float gv = out_scale;
    if (gate) gv *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + h])));
    out[(size_t)t * out_stride + (size_t)h * vdim + d] = __float2bfloat16_rn(acc * gv);
  }
}

template <int HD, int BM, bool GROUP>
static int sg_launch(const bf16* q, long long q_row_stride, const bf16* k_pages, const bf16* v_pages, const int* block_table, int table_width,
                     const int* seq_start, const int* seq_pos0, const float* head_bias, float* part, int n_tokens, int n_seqs, int max_q_len,
                     int H, int K, int kdim, int vdim, int window, float scale, int chunk, float softcap, int all_values, int parts,
                     cudaStream_t stream) {
  const size_t smem = (size_t)(SG_NBUF * SG_BN + BM) * (HD + 8) * sizeof(bf16);
  auto kern = sigmoid_attn_mma_kernel<HD, BM, GROUP>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(9, "sigmoid_attn_mma: cannot get %zu bytes of shared memory", smem);
  }
  dim3 grid((GROUP ? K : H) * n_seqs, GROUP ? 1 : (max_q_len + BM - 1) / BM, (all_values ? K : 1) * parts);
  kern<<<grid, BM * 2, smem, stream>>>(q, q_row_stride, k_pages, v_pages, block_table, table_width, seq_start, seq_pos0, head_bias, part,
                                       n_tokens, H, K, kdim, vdim, window, scale, chunk, softcap, all_values, parts);
  RL_LAUNCH_RESULT();
}

// part: float32 scratch of parts * n_tokens * H * (mix ? K : 1) * vdim numbers.
RL_API int rl_sigmoid_attn_mma(const void* q, long long q_row_stride, const void* k_pages, const void* v_pages, const int* block_table,
                               int table_width, const int* seq_start, const int* seq_pos0, const float* head_bias, const float* mix,
                               const void* gate, int gate_stride, float out_scale, float* part, int parts, void* out, int out_stride,
                               int n_tokens, int n_seqs, int max_q_len, int H, int K, int kdim, int vdim, int window, float scale, int chunk,
                               float softcap, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0 || max_q_len <= 0 || H <= 0 || K <= 0 || H % K || parts <= 0)
    RL_REFUSE(1, "sigmoid_attn_mma: T=%d S=%d H=%d K=%d parts=%d", n_tokens, n_seqs, H, K, parts);
  if (kdim <= 0 || vdim <= 0 || kdim % 8 || vdim % 8 || kdim > 128 || vdim > 128)
    RL_REFUSE(2, "sigmoid_attn_mma: key and value sizes %d, %d must be multiples of 8 up to 128", kdim, vdim);
  if (q_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)part & 7))
    RL_REFUSE(3, "sigmoid_attn_mma: rows must start on 16 bytes");
  if ((size_t)H * n_seqs > 2147483647u || (size_t)(mix ? K : 1) * parts > 65535u) RL_REFUSE(4, "sigmoid_attn_mma: grid too large");
  const size_t mix_smem = (size_t)H * vdim * sizeof(float);
  if (mix_smem > 48 * 1024) RL_REFUSE(5, "sigmoid_attn_mma: %d heads of %d values do not fit the second kernel's shared memory", H, vdim);
  const int hd = kdim > vdim ? kdim : vdim;
  const int all_values = mix != nullptr ? 1 : 0;
  // every sequence brings one token (and a kv head's heads fit a block's rows): the rows of a block are heads
  const bool group = max_q_len == 1 && n_tokens == n_seqs && H / K <= 64;
  const bool narrow = group && H / K <= 16;
  int rc;
#define SG_GO(HD, BM, GROUP)                                                                                                               \
  rc = sg_launch<HD, BM, GROUP>((const bf16*)q, q_row_stride, (const bf16*)k_pages, (const bf16*)v_pages, block_table, table_width,       \
                                seq_start, seq_pos0, head_bias, part, n_tokens, n_seqs, max_q_len, H, K, kdim, vdim, window, scale, chunk, \
                                softcap, all_values, parts, stream)
#define SG_PICK(HD)                          \
  if (narrow) SG_GO(HD, 16, true);           \
  else if (group) SG_GO(HD, 64, true);       \
  else SG_GO(HD, 64, false)
  if (hd <= 32) { SG_PICK(32); }
  else if (hd <= 64) { SG_PICK(64); }
  else { SG_PICK(128); }
#undef SG_PICK
#undef SG_GO
  if (rc != 0) return rc;
  int threads = H * vdim;
  threads = threads > 512 ? 512 : ((threads + 31) / 32) * 32;
  if (n_tokens > 2147483647 / 1 || (mix ? K : 1) > 65535) RL_REFUSE(10, "sigmoid_attn_mma: the second kernel's grid is too large");
  sigmoid_attn_mix_kernel<<<dim3(n_tokens, mix ? K : 1), threads, mix_smem, stream>>>(part, parts, mix, (const bf16*)gate, gate_stride, out_scale,
                                                                                      (bf16*)out, out_stride, n_tokens, H, K, vdim);
  RL_LAUNCH_RESULT();
}
