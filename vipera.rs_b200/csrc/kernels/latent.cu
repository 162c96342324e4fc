// Attention over a cached low-rank latent.
//
// A token leaves in the cache a latent c [rank] (RMS-normed) and one rotated key part kr [rot]
// that all heads share.  Head h's unrotated key is U_h c and its value V_h c, with U_h [d, rank]
// and V_h [dv, rank].  Since q . (U_h c) = (U_h^T q) . c and sum_j p_j V_h c_j = V_h sum_j p_j c_j, the
// heads attend to the latents themselves:
//
//   qa_h = [U_h^T q_h | rotated q_h] * scale        (latent_absorb_kernel)
//   s_j  = qa_h . [c_j | kr_j],  p = softmax over the visible j,  l_h = sum_j p_j c_j
//                                                    (latent_attention_kernel)
//   out_h = (V_h l_h) * sigmoid(gate_h)              (latent_expand_kernel)
//
// so the keys and values of earlier tokens are never expanded.  Scores, softmax, the sums over
// keys, the latent's norm and the rotation are 32-bit.  Rotation: values (2i, 2i + 1) of the
// rotated part turn by the angle whose cosine and sine the tables hold at [position, i].
#include "common.cuh"

constexpr int kMaxRank = 512;   // latent size
constexpr int kMaxRot = 128;    // rotated part
constexpr int kWarps = 4;

// ---------------------------------------------------------------------------------------
// The step's latents and rotated key parts into their pages.  `proj` [tokens, proj_width] holds
// the down projection at column kv_off: rank latent values, then rot key values.  One block per
// token.  k_pool rows are latents [rank], v_pool rows the rotated key parts [rot].
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
latent_store_kernel(const float* __restrict__ proj, long long proj_width, int kv_off, const float* __restrict__ norm_weight,
                    float eps, const int* __restrict__ positions, const float* __restrict__ cos_table,
                    const float* __restrict__ sin_table, T* __restrict__ k_pool, T* __restrict__ v_pool,
                    const int* __restrict__ token_entry, const int* __restrict__ block_table, int table_width,
                    int page_size, int rank, int rot) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = proj + static_cast<size_t>(t) * proj_width + kv_off;
  const int position = positions[t];
  const int page = block_table[static_cast<size_t>(token_entry[t]) * table_width + position / page_size];
  const size_t slot = static_cast<size_t>(page) * page_size + position % page_size;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) sum += row[i] * row[i];
  const float inverse = 1.0f / sqrtf(block_sum(sum, scratch) / static_cast<float>(rank) + eps);
  T* c_row = k_pool + slot * rank;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) c_row[i] = from_float<T>(row[i] * inverse * norm_weight[i]);
  T* r_row = v_pool + slot * rot;
  const float* cs = cos_table + static_cast<size_t>(position) * (rot / 2);
  const float* sn = sin_table + static_cast<size_t>(position) * (rot / 2);
  for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
    const float u = row[rank + 2 * i], v = row[rank + 2 * i + 1];
    r_row[2 * i] = from_float<T>(u * cs[i] - v * sn[i]);
    r_row[2 * i + 1] = from_float<T>(v * cs[i] + u * sn[i]);
  }
}

// ---------------------------------------------------------------------------------------
// qa[t, h, :rank] = scale * sum_d q[t, h, d] U[h, d, :],  qa[t, h, rank:] = scale * rotated q.
// q sits in `proj` at column q_off, head by head as [d unrotated | rot rotated].  U is stored
// [heads * d, rank].  A block serves kTile tokens of one head, so a row of U is read once per tile.
// ---------------------------------------------------------------------------------------
constexpr int kTile = 8;

template <typename TW>
__global__ void __launch_bounds__(128)
latent_absorb_kernel(const float* __restrict__ proj, long long proj_width, int q_off, const TW* __restrict__ up_k,
                     const int* __restrict__ positions, const float* __restrict__ cos_table,
                     const float* __restrict__ sin_table, float* __restrict__ qa, int num_tokens, int heads, int d,
                     int rank, int rot, float scale) {
  extern __shared__ float q_tile[];   // [kTile][d]
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * kTile, h = blockIdx.y;
  const int count = min(kTile, num_tokens - t0);
  const int head_width = d + rot;
  for (int i = threadIdx.x; i < kTile * d; i += blockDim.x) {
    const int tt = i / d, e = i % d;
    q_tile[i] = tt < count ? proj[static_cast<size_t>(t0 + tt) * proj_width + q_off + h * head_width + e] : 0.0f;
  }
  __syncthreads();
  const TW* u = up_k + static_cast<size_t>(h) * d * rank;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) {
    float acc[kTile];
#pragma unroll
    for (int tt = 0; tt < kTile; ++tt) acc[tt] = 0.0f;
    for (int e = 0; e < d; ++e) {
      const float w = to_float<TW>(u[static_cast<size_t>(e) * rank + r]);
#pragma unroll
      for (int tt = 0; tt < kTile; ++tt) acc[tt] = fmaf(q_tile[tt * d + e], w, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < kTile; ++tt)
      if (tt < count) qa[(static_cast<size_t>(t0 + tt) * heads + h) * (rank + rot) + r] = acc[tt] * scale;
  }
  for (int i = threadIdx.x; i < count * (rot / 2); i += blockDim.x) {
    const int tt = i / (rot / 2), pair = i % (rot / 2);
    const int t = t0 + tt;
    const float* q_rot = proj + static_cast<size_t>(t) * proj_width + q_off + h * head_width + d;
    const int position = positions[t];
    const float c = cos_table[static_cast<size_t>(position) * (rot / 2) + pair];
    const float s = sin_table[static_cast<size_t>(position) * (rot / 2) + pair];
    const float a = q_rot[2 * pair], b = q_rot[2 * pair + 1];
    float* dst = qa + (static_cast<size_t>(t) * heads + h) * (rank + rot) + rank;
    dst[2 * pair] = (a * c - b * s) * scale;
    dst[2 * pair + 1] = (b * c + a * s) * scale;
  }
}

// ---------------------------------------------------------------------------------------
// One warp per (token, head) folds the visible keys 32 at a time with a running (max, sum, l):
// a lane scores one key (its whole row), then the 32 latents are added with their weights, a lane
// owning every 32nd latent value.  Causal: the query at position p sees keys 0 .. p.
// ---------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float dot_span(const float* __restrict__ q, const T* __restrict__ row, int n) {
  float sum = 0.0f;
  for (int i = 0; i < n; ++i) sum = fmaf(q[i], to_float<T>(row[i]), sum);
  return sum;
}
template <>
__device__ __forceinline__ float dot_span<float>(const float* __restrict__ q, const float* __restrict__ row, int n) {
  float sum = 0.0f;
  if (n & 3) {
    for (int i = 0; i < n; ++i) sum = fmaf(q[i], row[i], sum);
    return sum;
  }
  const float4* r4 = reinterpret_cast<const float4*>(row);
  for (int i = 0; i < n / 4; ++i) {
    const float4 v = r4[i];
    sum = fmaf(q[4 * i], v.x, sum);
    sum = fmaf(q[4 * i + 1], v.y, sum);
    sum = fmaf(q[4 * i + 2], v.z, sum);
    sum = fmaf(q[4 * i + 3], v.w, sum);
  }
  return sum;
}
template <>
__device__ __forceinline__ float dot_span<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ row, int n) {
  float sum = 0.0f;
  if (n & 7) {
    for (int i = 0; i < n; ++i) sum = fmaf(q[i], __bfloat162float(row[i]), sum);
    return sum;
  }
  const uint4* r8 = reinterpret_cast<const uint4*>(row);
  for (int i = 0; i < n / 8; ++i) {
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
__global__ void __launch_bounds__(kWarps * 32)
latent_attention_kernel(const float* __restrict__ qa, float* __restrict__ mixed, const T* __restrict__ k_pool,
                        const T* __restrict__ v_pool, const int* __restrict__ token_entry,
                        const int* __restrict__ positions, const int* __restrict__ block_table, int table_width,
                        int page_size, int heads, int rank, int rot) {
  extern __shared__ float q_shared[];   // [kWarps][rank + rot]
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kWarps + warp;
  if (h >= heads) return;
  const int width = rank + rot;
  const int position = positions[t];
  const int* table = block_table + static_cast<size_t>(token_entry[t]) * table_width;
  float* qs = q_shared + warp * width;
  const float* q_row = qa + (static_cast<size_t>(t) * heads + h) * width;
  for (int i = lane; i < width; i += 32) qs[i] = q_row[i];
  __syncwarp();

  float acc[kMaxRank / 32];
#pragma unroll
  for (int i = 0; i < kMaxRank / 32; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY, running_sum = 0.0f;
  for (int base = 0; base <= position; base += 32) {
    const int j = base + lane;
    const bool valid = j <= position;
    float score = -INFINITY;
    if (valid) {
      const size_t slot = static_cast<size_t>(table[j / page_size]) * page_size + j % page_size;
      score = dot_span<T>(qs, k_pool + slot * rank, rank) + dot_span<T>(qs + rank, v_pool + slot * rot, rot);
    }
    const float new_max = fmaxf(running_max, warp_max(score));
    const float alpha = expf(running_max - new_max);   // 0 on the first tile
    const float weight = valid ? expf(score - new_max) : 0.0f;
    running_sum = running_sum * alpha + warp_sum(weight);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < kMaxRank / 32; ++i) acc[i] *= alpha;
    const int count = min(32, position - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float w = __shfl_sync(0xffffffffu, weight, jj);
      const int key = base + jj;
      const T* c_row = k_pool + (static_cast<size_t>(table[key / page_size]) * page_size + key % page_size) * rank;
#pragma unroll
      for (int i = 0; i < kMaxRank / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < rank) acc[i] = fmaf(w, to_float<T>(c_row[e]), acc[i]);
      }
    }
  }
  const float inverse = 1.0f / running_sum;
  float* out_row = mixed + (static_cast<size_t>(t) * heads + h) * rank;
#pragma unroll
  for (int i = 0; i < kMaxRank / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < rank) out_row[e] = acc[i] * inverse;
  }
}

// ---------------------------------------------------------------------------------------
// out[t, h * dv + v] = (sum_r l[t, h, r] V[h, r, v]) * sigmoid(gate[t, h * dv + v]).  V is stored
// transposed per head, [heads, rank, dv], so that neighbouring threads read neighbouring values.
// `gate` is the pre-activation in `proj` at column g_off (g_off < 0: no gate).
// ---------------------------------------------------------------------------------------
template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
latent_expand_kernel(const float* __restrict__ latent_out, const TW* __restrict__ up_v, const float* __restrict__ proj,
                     long long proj_width, int g_off, TO* __restrict__ out, int num_tokens, int heads, int dv,
                     int rank) {
  extern __shared__ float l_tile[];   // [kTile][rank]
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * kTile, h = blockIdx.y;
  const int count = min(kTile, num_tokens - t0);
  for (int i = threadIdx.x; i < kTile * rank; i += blockDim.x) {
    const int tt = i / rank, r = i % rank;
    l_tile[i] = tt < count ? latent_out[(static_cast<size_t>(t0 + tt) * heads + h) * rank + r] : 0.0f;
  }
  __syncthreads();
  const TW* w = up_v + static_cast<size_t>(h) * rank * dv;
  for (int v = threadIdx.x; v < dv; v += blockDim.x) {
    float acc[kTile];
#pragma unroll
    for (int tt = 0; tt < kTile; ++tt) acc[tt] = 0.0f;
    for (int r = 0; r < rank; ++r) {
      const float x = to_float<TW>(w[static_cast<size_t>(r) * dv + v]);
#pragma unroll
      for (int tt = 0; tt < kTile; ++tt) acc[tt] = fmaf(l_tile[tt * rank + r], x, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < kTile; ++tt) {
      if (tt >= count) continue;
      const size_t t = t0 + tt;
      float y = acc[tt];
      if (g_off >= 0) y *= 1.0f / (1.0f + expf(-proj[t * proj_width + g_off + h * dv + v]));
      out[(t * heads + h) * dv + v] = from_float<TO>(y);
    }
  }
}

struct LatentParams {
  const float* proj;       // [tokens, proj_width] 32-bit: q, the gate's pre-activation, the down projection
  long long proj_width;
  int q_off, g_off, kv_off;  // columns; g_off < 0: no gate; kv_off < 0: the layer reads a cache it does not write
  const void* up_k;        // [heads * d, rank]
  const void* up_v;        // [heads, rank, dv]
  const float* norm_weight;  // [rank]
  const int* positions;
  const int* token_entry;
  const int* block_table;
  const float* cos_table;
  const float* sin_table;
  void* k_pool;            // latents [pages, page_size, 1, rank]
  void* v_pool;            // rotated key parts [pages, page_size, 1, rot]
  float* qa;               // scratch [tokens, heads, rank + rot]
  float* latent_out;       // scratch [tokens, heads, rank]
  void* out;               // [tokens, heads * dv]
  int num_tokens, heads, d, rot, dv, rank, table_width, page_size;
  float scale, eps;
};

template <typename T>
static int launch_latent(const LatentParams& p, cudaStream_t s) {
  int status = VIPERA_OK;
  if (p.kv_off >= 0) {
    status = vipera_launch(latent_store_kernel<T>, p.num_tokens, 128, 0, s, p.proj, p.proj_width, p.kv_off, p.norm_weight,
                           p.eps, p.positions, p.cos_table, p.sin_table, static_cast<T*>(p.k_pool),
                           static_cast<T*>(p.v_pool), p.token_entry, p.block_table, p.table_width, p.page_size, p.rank,
                           p.rot);
    if (status) return status;
  }
  const dim3 tiles((p.num_tokens + kTile - 1) / kTile, p.heads);
  status = vipera_launch(latent_absorb_kernel<T>, tiles, 128, kTile * p.d * sizeof(float), s, p.proj, p.proj_width, p.q_off,
                         static_cast<const T*>(p.up_k), p.positions, p.cos_table, p.sin_table, p.qa, p.num_tokens,
                         p.heads, p.d, p.rank, p.rot, p.scale);
  if (status) return status;
  status = vipera_launch(latent_attention_kernel<T>, dim3(p.num_tokens, (p.heads + kWarps - 1) / kWarps), kWarps * 32,
                         kWarps * (p.rank + p.rot) * sizeof(float), s, p.qa, p.latent_out,
                         static_cast<const T*>(p.k_pool), static_cast<const T*>(p.v_pool), p.token_entry, p.positions,
                         p.block_table, p.table_width, p.page_size, p.heads, p.rank, p.rot);
  if (status) return status;
  const int threads = p.dv >= 128 ? 128 : (p.dv + 31) / 32 * 32;
  return vipera_launch(latent_expand_kernel<T, T>, tiles, threads, kTile * p.rank * sizeof(float), s, p.latent_out,
                       static_cast<const T*>(p.up_v), p.proj, p.proj_width, p.g_off, static_cast<T*>(p.out),
                       p.num_tokens, p.heads, p.dv, p.rank);
}

// dtype: the type of the cache pools, the two up matrices and `out`.
VIPERA_API int vipera_latent_attention(const LatentParams* params, int dtype, void* stream) {
  const LatentParams& p = *params;
  if (p.num_tokens <= 0) return VIPERA_OK;
  if (p.rank <= 0 || p.rank > kMaxRank || p.rot <= 0 || p.rot > kMaxRot || (p.rot & 1)) return VIPERA_BAD_SHAPE;
  if (p.heads <= 0 || p.d <= 0 || p.d > 1024 || p.dv <= 0 || p.page_size <= 0 || p.table_width <= 0) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == VIPERA_F32) return launch_latent<float>(p, s);
  if (dtype == VIPERA_BF16) return launch_latent<__nv_bfloat16>(p, s);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API int vipera_latent_params_size() { return static_cast<int>(sizeof(LatentParams)); }
VIPERA_API const char* vipera_latent_status_text(int status) { return vipera_status_text(status); }
