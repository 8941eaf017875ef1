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
// `sigmoid_attn_mma` is the bfloat16 form on the tensor cores (mma.sync m16n8k16) for key and value sizes in multiples of 16
// up to 128.  The mixing is linear in the weights, so it commutes with the sum over the keys:
//
//     o_h = sum_g M[h][g] P[g][kv(h)],       P[g][c] = sum_j w_g(i, j) v_c(j)
//
// A block takes 64 queries of one sequence and ONE query head g: S = Q_g K_kv(g)^T per key tile of 64 as in any flash kernel,
// the weights from the 32-bit scores in registers (no running maximum, no rescaling: the sum over the keys is a plain sum),
// and P[g][c] for every kv head c whose values some head mixes g into (all of them with a full matrix; only kv(g) without a
// mixing matrix) accumulated in registers.  P goes to a float32 scratch [T, H, K, vdim]; `sigmoid_attn_mix` then forms
// out_h = gate_h * sum_g M[h][g] P[g][kv(h)] in 32-bit.  A single token's keys are cut into parts over several blocks whose
// partial P are added by the same second kernel.
#include "common.cuh"
#include <mma.h>

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
