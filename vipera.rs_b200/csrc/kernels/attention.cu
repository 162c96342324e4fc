// Causal grouped-query attention over the paged cache, for any mix of prompt portions and
// single decode tokens, with 32-bit scores, softmax and accumulation.
//
// Definition (crates/vipera-backend-cpu/src/model.rs:1804-1859): query head h reads KV head
// h / group; s_j = (q . k_j) * scale; a query at position p sees keys 0..p (with a window w,
// keys p-w+1..p); weights exp(s_j - max) over their sum; output = weighted sum of v_j.
// Traversal: one warp per (token, query head) folds the keys 32 at a time with a running
// (max, sum, output), the online form of the reference's chunk fold (model.rs:2752-2857) and
// of its device kernels' partials (crates/vipera-backend-gpu/src/layer.cu:307-467).
// Keys are found through the block table: position j lives in page table[j / page], slot
// j % page (model.rs:1507-1542).
//
// Three options beyond that definition, each a parameter: values of another size than keys
// (`value_dim`); with a window, the first `keep_first` keys of a request stay visible to every
// later query, at their true positions; and a sink, an extra key of score 0 without a value,
// which adds exp(0 - max) to the softmax's denominator (p_j = e^{s_j} / (1 + sum e^{s_j})).
// Instead of a window the mask may be one of chunks (`chunk`): position i sees j <= i with
// floor(i / chunk) = floor(j / chunk).  `out_scale` multiplies the output.  The sink's score may be
// learned, one per query head (`sink_values`: exp(sink_h - max) joins the denominator, unscaled), and
// the output may be gated: out[t, h, e] *= sigmoid(gate[t * gate_stride + h * value_dim + e]), the gate
// a 32-bit pre-activation.
//
// This kernel is the attention of the 32-bit path and takes every head size that is a
// up to 256 (keys and values each; sizes that are not a multiple of 8 are read value by value), any number of heads and groups, any page size.
#include "common.cuh"

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ row, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ row, int d) {
  float sum = 0.0f;
  if (d & 3) {   // rows of such a size do not start on 16 bytes
    for (int i = 0; i < d; ++i) sum = fmaf(q[i], row[i], sum);
    return sum;
  }
  const float4* r4 = reinterpret_cast<const float4*>(row);
  for (int i = 0; i < d / 4; ++i) {
    const float4 v = r4[i];
    sum = fmaf(q[4 * i + 0], v.x, sum);
    sum = fmaf(q[4 * i + 1], v.y, sum);
    sum = fmaf(q[4 * i + 2], v.z, sum);
    sum = fmaf(q[4 * i + 3], v.w, sum);
  }
  return sum;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ row, int d) {
  float sum = 0.0f;
  if (d & 7) {
    for (int i = 0; i < d; ++i) sum = fmaf(q[i], __bfloat162float(row[i]), sum);
    return sum;
  }
  const uint4* r8 = reinterpret_cast<const uint4*>(row);
  for (int i = 0; i < d / 8; ++i) {
    const uint4 raw = r8[i];
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(pairs[e]);
      sum = fmaf(q[8 * i + 2 * e], f.x, sum);
      sum = fmaf(q[8 * i + 2 * e + 1], f.y, sum);
    }
  }
  return sum;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_pool,
                 const T* __restrict__ v_pool, const int* __restrict__ token_seq,
                 const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
                 int page_size, int num_heads, int num_kv_heads, int head_dim, int value_dim, float scale,
                 int window, int keep_first, int sink, int chunk, float out_scale,
                 const float* __restrict__ sink_values, const float* __restrict__ gate, long long gate_stride) {
  __shared__ float q_shared[kWarpsPerBlock][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kWarpsPerBlock + warp;
  if (h >= num_heads) return;
  const int group = num_heads / num_kv_heads;
  const int kv_head = h / group;
  const int position = positions[t];
  const int* table = block_table + static_cast<size_t>(token_seq[t]) * table_width;
  // a mask of chunks: a query sees the keys of its own chunk of `chunk` positions, counted from 0
  const int first = chunk > 0 ? position / chunk * chunk : (window > 0 ? max(0, position - window + 1) : 0);

  const T* q_row = q + (static_cast<size_t>(t) * num_heads + h) * head_dim;
  float* qs = q_shared[warp];
  for (int i = lane; i < head_dim; i += 32) qs[i] = to_float<T>(q_row[i]);
  __syncwarp();

  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY, running_sum = 0.0f;
  const size_t row_stride = static_cast<size_t>(num_kv_heads) * head_dim;
  const size_t v_stride = static_cast<size_t>(num_kv_heads) * value_dim;
  // two runs of keys: the kept first ones that the window has left behind, then the window
  const int kept_end = window > 0 ? min(keep_first, first) : 0;

  for (int run = 0; run < 2; ++run) {
  const int run_first = run == 0 ? 0 : first;
  const int run_last = run == 0 ? kept_end - 1 : position;
  for (int base = run_first; base <= run_last; base += 32) {
    const int j = base + lane;
    const bool valid = j <= run_last;
    float score = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      const T* k_row = k_pool + (static_cast<size_t>(page) * page_size + j % page_size) * row_stride +
                       static_cast<size_t>(kv_head) * head_dim;
      score = dot_row<T>(qs, k_row, head_dim) * scale;
    }
    const float new_max = fmaxf(running_max, warp_max(score));
    const float alpha = expf(running_max - new_max);  // 0 on the first tile
    const float weight = valid ? expf(score - new_max) : 0.0f;
    running_sum = running_sum * alpha + warp_sum(weight);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= alpha;
    const int count = min(32, run_last - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float w = __shfl_sync(0xffffffffu, weight, jj);
      const int key = base + jj;
      const int page = table[key / page_size];
      const T* v_row = v_pool + (static_cast<size_t>(page) * page_size + key % page_size) * v_stride +
                       static_cast<size_t>(kv_head) * value_dim;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < value_dim) acc[i] = fmaf(w, to_float<T>(v_row[e]), acc[i]);
      }
    }
  }
  }
  if (sink || sink_values) {
    // the sink's score is 0 (or the head's learned one): fold it in like one more key whose value is zero
    const float sink_score = sink_values ? sink_values[h] : 0.0f;
    const float new_max = fmaxf(running_max, sink_score);
    const float alpha = expf(running_max - new_max);
    running_sum = running_sum * alpha + expf(sink_score - new_max);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= alpha;
  }
  const float inverse = out_scale / running_sum;
  T* out_row = out + (static_cast<size_t>(t) * num_heads + h) * value_dim;
  const float* gate_row = gate ? gate + static_cast<size_t>(t) * gate_stride + static_cast<size_t>(h) * value_dim : nullptr;
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < value_dim) {
      float value = acc[i] * inverse;
      if (gate_row) value *= 1.0f / (1.0f + expf(-gate_row[e]));
      out_row[e] = from_float<T>(value);
    }
  }
}

// q is [tokens, heads, d] and out [tokens, heads, value_dim]; the key pool is
// [pages, page_size, kv_heads, d] and the value pool the same with value_dim last.
// token_seq[t] is the row of block_table (width table_width) of token t's request and
// positions[t] its position.  The keys and values of this step's tokens must already be
// in the cache.  window = 0 means every earlier key is visible; keep_first counts only with a
// window; sink != 0 adds the sink to the denominator.
// sink_values (null: none) holds a learned sink score per query head; gate (null: none) the output
// gate's 32-bit pre-activations, row t at gate + t * gate_stride, [heads * value_dim] values.
VIPERA_API int vipera_attention_gated(const void* q, void* out, int dtype, const void* k_pool, const void* v_pool,
                                      const int* token_seq, const int* positions, const int* block_table,
                                      int table_width, int page_size, int num_tokens, int num_heads,
                                      int num_kv_heads, int head_dim, int value_dim, float scale, int window,
                                      int keep_first, int sink, int chunk, float out_scale, const float* sink_values,
                                      const float* gate, long long gate_stride, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (chunk < 0 || (chunk > 0 && window > 0)) return VIPERA_BAD_ARGUMENT;
  if (head_dim <= 0 || head_dim > kMaxHeadDim) return VIPERA_BAD_SHAPE;
  if (value_dim <= 0 || value_dim > kMaxHeadDim || keep_first < 0) return VIPERA_BAD_SHAPE;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0) return VIPERA_BAD_SHAPE;
  if (page_size <= 0 || table_width <= 0 || window < 0) return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(num_tokens, (num_heads + kWarpsPerBlock - 1) / kWarpsPerBlock);
  if (dtype == VIPERA_F32)
    attention_kernel<float><<<grid, kWarpsPerBlock * 32, 0, s>>>(
        static_cast<const float*>(q), static_cast<float*>(out), static_cast<const float*>(k_pool),
        static_cast<const float*>(v_pool), token_seq, positions, block_table, table_width, page_size,
        num_heads, num_kv_heads, head_dim, value_dim, scale, window, keep_first, sink, chunk, out_scale, sink_values,
        gate, gate_stride);
  else if (dtype == VIPERA_BF16)
    attention_kernel<__nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, s>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out),
        static_cast<const __nv_bfloat16*>(k_pool), static_cast<const __nv_bfloat16*>(v_pool), token_seq,
        positions, block_table, table_width, page_size, num_heads, num_kv_heads, head_dim, value_dim, scale, window,
        keep_first, sink, chunk, out_scale, sink_values, gate, gate_stride);
  else
    return VIPERA_BAD_DTYPE;
  return vipera_launch_status();
}

VIPERA_API int vipera_attention(const void* q, void* out, int dtype, const void* k_pool, const void* v_pool,
                                const int* token_seq, const int* positions, const int* block_table,
                                int table_width, int page_size, int num_tokens, int num_heads,
                                int num_kv_heads, int head_dim, int value_dim, float scale, int window,
                                int keep_first, int sink, int chunk, float out_scale, void* stream) {
  return vipera_attention_gated(q, out, dtype, k_pool, v_pool, token_seq, positions, block_table, table_width, page_size,
                                num_tokens, num_heads, num_kv_heads, head_dim, value_dim, scale, window, keep_first, sink,
                                chunk, out_scale, nullptr, nullptr, 0, stream);
}

VIPERA_API const char* vipera_attention_status_text(int status) { return vipera_status_text(status); }
