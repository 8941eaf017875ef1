// Grouped-query softmax attention with the options that a plain causal attention lacks, over the paged cache:
//
//   - keys of `kdim` and values of `vdim` numbers per head (the two may differ),
//   - biases on the projected q, k and v,
//   - an RMS norm of every q head and every k head over the head's numbers (one weight row for all q heads, one for all k
//     heads), after the biases and before the rotation,
//   - a rotation of the first `rot` dimensions of q and k in either pair layout, cosines and sines
//     multiplied by a constant `magnitude`,
//   - a score scale given by the caller,
//   - a mixing of the heads' scaled scores before the softmax, s_h <- sum_g mix[h][g] s_g,
//   - a window (query at position p sees keys j with 0 <= p - j < window),
//   - chunks (query at position p sees keys j <= p of its own chunk only, floor(j / chunk) = floor(p / chunk), positions
//     counted from the start of the sequence),
//   - a cap on the scores, s <- cap tanh(s / cap), after the scale (and the mixing),
//   - a sink per head: exp(sink_h) joins the softmax's denominator and nothing else,
//   - a gate on the result, out *= sigmoid(gate), and a constant factor `out_scale`.
//
// Two kernels.  `qkv_prep` adds the biases, rotates q in place and writes the rotated k and v to the token's
// place in its sequence's pages; with `v_src` the value that is stored is (1 - lambda) v + lambda v_src[t] (values that an
// earlier layer projected for the same token; lambda a learned number on the device), computed in 32-bit.  `attn_ext` is the attention itself, for prompts and for decoding, in both
// element types: one warp per (token, head), the keys taken 32 at a time counted from the first key the
// query may see, online softmax, every sum in 32-bit and in a fixed order, so a result's bits depend neither
// on how its sequence was cut into steps nor on what else is in the batch.  With a mixing matrix the warps
// of all heads of a token share a block and exchange their scores of a group of keys through shared memory.
//
// Cache layout of one layer: k_pages[page][kv head][slot in page][kdim], v_pages[...][vdim]; the page of
// position p of batch sequence s is block_table[s][p / page_size].
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

// ---------------------------------------------------------------- biases, rotation, cache write
// One block per token.  row = qkv[t]: H query heads of kdim, then K key heads of kdim, then K value heads of vdim.
template <typename T>
__global__ void qkv_prep_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ bias,
                                const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                const int* __restrict__ block_table, int table_width, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, const float* __restrict__ inv_freq, float magnitude,
                                const float* __restrict__ q_norm, const float* __restrict__ k_norm, float norm_eps, int H, int K,
                                int kdim, int vdim, int rot, int interleaved, int page_size, const T* __restrict__ v_src,
                                int v_src_stride, const float* __restrict__ v_lambda) {
  extern __shared__ float trig[];  // cos[rot/2], sin[rot/2], both times the magnitude; then 1 / rms of every q and k head
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const float a = (float)pos * inv_freq[j];
    float s, c;
    sincosf(a, &s, &c);
    cs[j] = c * magnitude;
    sn[j] = s * magnitude;
  }
  T* row = qkv + (size_t)t * row_stride;
  float* inv_rms = trig + rot;
  if (q_norm != nullptr || k_norm != nullptr) {  // a warp per head, the sums in lane order and then by the warp's tree
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < H + K; h += nwarps) {
      const T* head = row + (size_t)h * kdim;
      const float* b = bias ? bias + (size_t)h * kdim : nullptr;
      float ss = 0.f;
      for (int i = lane; i < kdim; i += 32) {
        const float x = to_f32(head[i]) + (b ? b[i] : 0.f);
        ss += x * x;
      }
      ss = warp_sum(ss);
      if (lane == 0) inv_rms[h] = ((h < H ? q_norm : k_norm) != nullptr) ? 1.0f / sqrtf(ss / (float)kdim + norm_eps) : 1.f;
    }
  }
  __syncthreads();
  const int page = block_table[(size_t)tok_seq[t] * table_width + pos / page_size];
  const int in_page = pos % page_size;
  // q and k heads: one thread per rotated pair or per unrotated value
  const int per_head = half + (kdim - rot);
  for (int idx = threadIdx.x; idx < (H + K) * per_head; idx += blockDim.x) {
    const int h = idx / per_head, e = idx - h * per_head;
    T* head = row + (size_t)h * kdim;
    const float* b = bias ? bias + (size_t)h * kdim : nullptr;
    const float* nw = h < H ? q_norm : k_norm;
    const float inv = nw ? inv_rms[h] : 1.f;
    T* dst = h < H ? head : k_pages + (((size_t)page * K + (h - H)) * page_size + in_page) * kdim;
    if (e < half) {
      const int i0 = interleaved ? 2 * e : e;
      const int i1 = interleaved ? 2 * e + 1 : e + half;
      float x0 = to_f32(head[i0]) + (b ? b[i0] : 0.f);
      float x1 = to_f32(head[i1]) + (b ? b[i1] : 0.f);
      if (nw) {
        x0 = x0 * inv * nw[i0];
        x1 = x1 * inv * nw[i1];
      }
      dst[i0] = from_f32<T>(x0 * cs[e] - x1 * sn[e]);
      dst[i1] = from_f32<T>(x1 * cs[e] + x0 * sn[e]);
    } else {
      const int i = rot + (e - half);
      float x = to_f32(head[i]) + (b ? b[i] : 0.f);
      if (nw) x = x * inv * nw[i];
      dst[i] = from_f32<T>(x);
    }
  }
  const T* vrow = row + (size_t)(H + K) * kdim;
  const float* vb = bias ? bias + (size_t)(H + K) * kdim : nullptr;
  const float lam = v_src ? v_lambda[0] : 0.f;
  const T* vs = v_src ? v_src + (size_t)t * v_src_stride : nullptr;
  for (int idx = threadIdx.x; idx < K * vdim; idx += blockDim.x) {
    const int h = idx / vdim, i = idx - h * vdim;
    float v = to_f32(vrow[idx]) + (vb ? vb[idx] : 0.f);
    if (vs) v = (1.0f - lam) * v + lam * to_f32(vs[idx]);
    v_pages[(((size_t)page * K + h) * page_size + in_page) * vdim + i] = from_f32<T>(v);
  }
}

// The same for bfloat16 rows whose sizes are multiples of 8 and whose pairs are neighbours (or that are not rotated at all): a
// thread takes 8 numbers of a head with one 16-byte load, the kdim / 8 threads of a head add their squares up by shuffles, and
// the four pairs a thread holds are rotated in its registers; q goes back and k, v go to their pages with 16-byte stores.
__device__ __forceinline__ void qp_unpack8(const uint4& raw, float* x) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 qp_pack8(const float* x) {
  uint4 raw;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
  return raw;
}

__device__ __forceinline__ void qp_add8(float* x, const float* b) {
  const float4 b0 = *reinterpret_cast<const float4*>(b), b1 = *reinterpret_cast<const float4*>(b + 4);
  x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w;
  x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
}

__global__ void __launch_bounds__(256)
qkv_prep_rows8_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ bias, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_seq, const int* __restrict__ block_table, int table_width,
                      bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, const float* __restrict__ inv_freq, float magnitude,
                      const float* __restrict__ q_norm, const float* __restrict__ k_norm, float norm_eps, int H, int K, int kdim,
                      int vdim, int rot, int page_size, const bf16* __restrict__ v_src, int v_src_stride,
                      const float* __restrict__ v_lambda) {
  extern __shared__ float trig[];  // cos[rot/2], sin[rot/2], both times the magnitude
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const float a = (float)pos * inv_freq[j];
    float s, c;
    sincosf(a, &s, &c);
    cs[j] = c * magnitude;
    sn[j] = s * magnitude;
  }
  __syncthreads();
  bf16* row = qkv + (size_t)t * row_stride;
  const int page = block_table[(size_t)tok_seq[t] * table_width + pos / page_size];
  const int in_page = pos % page_size;
  const int g = kdim >> 3;  // threads to a head: a power of two up to 32
  const int total = (H + K) * g;
  const bool normed = q_norm != nullptr || k_norm != nullptr;
  for (int base = 0; base < total; base += blockDim.x) {
    const int idx = base + threadIdx.x;
    const bool valid = idx < total;  // (a head's threads are all valid or all not; every lane takes part in the shuffles)
    const int h = valid ? idx / g : 0, i0 = valid ? (idx - h * g) * 8 : 0;
    float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (valid) {
      qp_unpack8(*reinterpret_cast<const uint4*>(row + (size_t)h * kdim + i0), x);
      if (bias) qp_add8(x, bias + (size_t)h * kdim + i0);
    }
    if (normed) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
      for (int o = g >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float* nw = h < H ? q_norm : k_norm;
      if (valid && nw) {
        const float inv = 1.0f / sqrtf(ss / (float)kdim + norm_eps);
        const float4 w0 = *reinterpret_cast<const float4*>(nw + i0), w1 = *reinterpret_cast<const float4*>(nw + i0 + 4);
        x[0] = x[0] * inv * w0.x; x[1] = x[1] * inv * w0.y; x[2] = x[2] * inv * w0.z; x[3] = x[3] * inv * w0.w;
        x[4] = x[4] * inv * w1.x; x[5] = x[5] * inv * w1.y; x[6] = x[6] * inv * w1.z; x[7] = x[7] * inv * w1.w;
      }
    }
    if (valid) {
      if (i0 < rot) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float c = cs[(i0 >> 1) + p], sv = sn[(i0 >> 1) + p];
          const float a = x[2 * p], b = x[2 * p + 1];
          x[2 * p] = a * c - b * sv;
          x[2 * p + 1] = b * c + a * sv;
        }
      }
      bf16* dst = h < H ? row + (size_t)h * kdim + i0 : k_pages + (((size_t)page * K + (h - H)) * page_size + in_page) * kdim + i0;
      *reinterpret_cast<uint4*>(dst) = qp_pack8(x);
    }
  }
  const bf16* vrow = row + (size_t)(H + K) * kdim;
  const float* vb = bias ? bias + (size_t)(H + K) * kdim : nullptr;
  const int gv = vdim >> 3;
  for (int idx = threadIdx.x; idx < K * gv; idx += blockDim.x) {
    const int h = idx / gv, i = (idx - h * gv) * 8;
    uint4 raw = *reinterpret_cast<const uint4*>(vrow + (size_t)h * vdim + i);
    if (vb || v_src) {
      float x[8];
      qp_unpack8(raw, x);
      if (vb) qp_add8(x, vb + (size_t)h * vdim + i);
      if (v_src) {
        const float lam = v_lambda[0];
        float y[8];
        qp_unpack8(*reinterpret_cast<const uint4*>(v_src + (size_t)t * v_src_stride + (size_t)h * vdim + i), y);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = (1.0f - lam) * x[j] + lam * y[j];
      }
      raw = qp_pack8(x);
    }
    *reinterpret_cast<uint4*>(v_pages + (((size_t)page * K + h) * page_size + in_page) * vdim + i) = raw;
  }
}

RL_API int rl_qkv_prep(void* qkv, int dtype, int row_stride, const float* bias, const int* tok_pos, const int* tok_seq,
                       const int* block_table, int table_width, void* k_pages, void* v_pages, const float* inv_freq,
                       float magnitude, const float* q_norm, const float* k_norm, float norm_eps, int n_tokens, int H, int K, int kdim,
                       int vdim, int rot, int interleaved, int page_size, const void* v_src, int v_src_stride, const float* v_lambda,
                       cudaStream_t stream) {
  if (v_src != nullptr && (v_lambda == nullptr || v_src_stride < K * vdim)) RL_REFUSE(8, "qkv_prep: values to mix in need a factor and rows of %d numbers", K * vdim);
  if (n_tokens <= 0 || H <= 0 || K <= 0 || kdim <= 0 || vdim <= 0 || page_size <= 0 || table_width <= 0)
    RL_REFUSE(1, "qkv_prep: T=%d H=%d K=%d kdim=%d vdim=%d page=%d", n_tokens, H, K, kdim, vdim, page_size);
  if (rot < 0 || rot > kdim || (rot & 1)) RL_REFUSE(2, "qkv_prep: %d rotated dimensions do not fit a head of %d", rot, kdim);
  if (row_stride < (H + K) * kdim + K * vdim) RL_REFUSE(3, "qkv_prep: row stride %d too small", row_stride);
  if (rot > 0 && inv_freq == nullptr) RL_REFUSE(4, "qkv_prep: no frequency table");
  if (!block_table || !k_pages || !v_pages || !tok_pos || !tok_seq) RL_REFUSE(5, "qkv_prep: pages, page table and positions are needed");
  const size_t smem = ((size_t)rot + H + K) * sizeof(float);
  if (smem > 48 * 1024) RL_REFUSE(6, "qkv_prep: rotary size %d or %d heads too large", rot, H + K);
  const int threads = 256;
  const int g = kdim >> 3;
  const uintptr_t bits = (uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)bias | (uintptr_t)q_norm | (uintptr_t)k_norm |
                         (uintptr_t)v_src;
  if (dtype == RL_BF16 && (interleaved || rot == 0) && kdim % 8 == 0 && vdim % 8 == 0 && rot % 8 == 0 && row_stride % 8 == 0 &&
      v_src_stride % 8 == 0 && g <= 32 && (g & (g - 1)) == 0 && (bits & 15) == 0)
    qkv_prep_rows8_kernel<<<n_tokens, threads, (size_t)rot * sizeof(float), stream>>>(
        (bf16*)qkv, row_stride, bias, tok_pos, tok_seq, block_table, table_width, (bf16*)k_pages, (bf16*)v_pages, inv_freq, magnitude,
        q_norm, k_norm, norm_eps, H, K, kdim, vdim, rot, page_size, (const bf16*)v_src, v_src_stride, v_lambda);
  else if (dtype == RL_BF16)
    qkv_prep_kernel<bf16><<<n_tokens, threads, smem, stream>>>((bf16*)qkv, row_stride, bias, tok_pos, tok_seq, block_table, table_width,
                                                               (bf16*)k_pages, (bf16*)v_pages, inv_freq, magnitude, q_norm, k_norm, norm_eps, H, K,
                                                               kdim, vdim, rot, interleaved, page_size, (const bf16*)v_src, v_src_stride, v_lambda);
  else if (dtype == RL_F32)
    qkv_prep_kernel<float><<<n_tokens, threads, smem, stream>>>((float*)qkv, row_stride, bias, tok_pos, tok_seq, block_table, table_width,
                                                                (float*)k_pages, (float*)v_pages, inv_freq, magnitude, q_norm, k_norm, norm_eps, H, K,
                                                                kdim, vdim, rot, interleaved, page_size, (const float*)v_src, v_src_stride, v_lambda);
  else
    RL_REFUSE(7, "qkv_prep: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- the attention
#define EXT_MAX_V_PER_LANE 8  // value sizes up to 256

// blockDim = (32, HB): HB = 1 and grid (T, H) without a mixing matrix; HB = H and grid (T, 1) with one.
template <typename T>
__global__ void attn_ext_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                const int* __restrict__ block_table, int table_width, const int* __restrict__ tok_seq,
                                const int* __restrict__ tok_pos, const float* __restrict__ sink, const float* __restrict__ mix,
                                const T* __restrict__ gate, int gate_stride, float out_scale, T* __restrict__ out, int out_stride,
                                int H, int K, int kdim, int vdim, int page_size, int window, float scale, int chunk, float softcap) {
  extern __shared__ float smem[];  // q of the block's heads [HB][kdim], then (with mix) scores [HB][32]
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

  int first = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
  if (chunk != 0) first = max(first, pos - pos % chunk);
  float m = -INFINITY, l = 0.f;
  if (sink != nullptr) {  // the sink is a key without a value whose score is sink[h]
    m = sink[h];
    l = 1.f;
  }
  float acc[EXT_MAX_V_PER_LANE];
#pragma unroll
  for (int i = 0; i < EXT_MAX_V_PER_LANE; ++i) acc[i] = 0.f;

  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    float s = 0.f;
    if (valid) {
      const int page = table[key / page_size];
      const T* kr = k_pages + (((size_t)page * K + kh) * page_size + key % page_size) * kdim;
      float dot = 0.f;
      for (int i = 0; i < kdim; ++i) dot += q_s[i] * to_f32(kr[i]);
      s = dot * scale;
    }
    if (mix != nullptr) {
      __syncthreads();  // the scores of the group before have been read
      sc[hb * 32 + lane] = s;
      __syncthreads();
      float mixed = 0.f;
      for (int g = 0; g < HB; ++g) mixed += mix[h * HB + g] * sc[g * 32 + lane];
      s = mixed;
    }
    if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    if (!valid) s = -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));  // finite: the group holds at least key `base`
    const float alpha = expf(m - m_new);        // 0 for the first group without a sink, where m is -inf
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < EXT_MAX_V_PER_LANE; ++i) acc[i] *= alpha;
    const int count = min(32, pos - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const int page = table[kj / page_size];
      const T* vr = v_pages + (((size_t)page * K + kh) * page_size + kj % page_size) * vdim;
#pragma unroll
      for (int i = 0; i < EXT_MAX_V_PER_LANE; ++i) {
        const int dim = lane + 32 * i;
        if (dim < vdim) acc[i] += pj * to_f32(vr[dim]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* o = out + (size_t)t * out_stride + (size_t)h * vdim;
  const T* g = gate ? gate + (size_t)t * gate_stride + (size_t)h * vdim : nullptr;
#pragma unroll
  for (int i = 0; i < EXT_MAX_V_PER_LANE; ++i) {
    const int dim = lane + 32 * i;
    if (dim < vdim) {
      float r = acc[i] * inv;
      if (g) r *= 1.0f / (1.0f + expf(-to_f32(g[dim])));
      o[dim] = from_f32<T>(r * out_scale);
    }
  }
}

RL_API int rl_attn_ext(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages, const int* block_table,
                       int table_width, const int* tok_seq, const int* tok_pos, const float* sink, const float* mix,
                       const void* gate, int gate_stride, float out_scale, void* out, int out_stride, int n_tokens, int H, int K,
                       int kdim, int vdim, int page_size, int window, float scale, int chunk, float softcap, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || K <= 0 || kdim <= 0 || vdim <= 0 || page_size <= 0)
    RL_REFUSE(1, "attn_ext: T=%d H=%d K=%d kdim=%d vdim=%d page=%d", n_tokens, H, K, kdim, vdim, page_size);
  if (H % K) RL_REFUSE(2, "attn_ext: %d query heads are not a multiple of %d kv heads", H, K);
  if (vdim > 32 * EXT_MAX_V_PER_LANE) RL_REFUSE(3, "attn_ext: value size %d exceeds %d", vdim, 32 * EXT_MAX_V_PER_LANE);
  if (H > 65535) RL_REFUSE(4, "attn_ext: %d heads exceed 65535", H);
  if (window < 0 || chunk < 0) RL_REFUSE(5, "attn_ext: negative window or chunk");
  if (mix != nullptr && H > 32) RL_REFUSE(6, "attn_ext: scores of %d heads cannot be mixed (at most 32)", H);
  const int HB = mix != nullptr ? H : 1;
  dim3 grid(n_tokens, H / HB), block(32, HB);
  const size_t smem = ((size_t)HB * kdim + (mix != nullptr ? (size_t)HB * 32 : 0)) * sizeof(float);
  if (smem > 48 * 1024) RL_REFUSE(7, "attn_ext: %d heads of %d numbers do not fit shared memory", HB, kdim);
  if (dtype == RL_BF16)
    attn_ext_kernel<bf16><<<grid, block, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)k_pages, (const bf16*)v_pages,
                                                         block_table, table_width, tok_seq, tok_pos, sink, mix, (const bf16*)gate,
                                                         gate_stride, out_scale, (bf16*)out, out_stride, H, K, kdim, vdim, page_size,
                                                         window, scale, chunk, softcap);
  else if (dtype == RL_F32)
    attn_ext_kernel<float><<<grid, block, smem, stream>>>((const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages,
                                                          block_table, table_width, tok_seq, tok_pos, sink, mix, (const float*)gate,
                                                          gate_stride, out_scale, (float*)out, out_stride, H, K, kdim, vdim, page_size,
                                                          window, scale, chunk, softcap);
  else
    RL_REFUSE(8, "attn_ext: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}
