// A mixture of gated feed-forward units: router, grouping of the step's (token, expert)
// assignments by expert, and the experts' products over tiles of assignments.
//
//   z = R h (32-bit), s = sigmoid(z) or softmax(z)
//   experts in `groups` equal groups of neighbours; a group's score is the sum of its `group_top`
//   largest scores; only experts of the `keep` best groups may be chosen; the `top` largest
//   scores among those are the token's experts, with weights s (divided by their sum if asked).
//   y = sum_chosen w_e D_e (act(G_e h) * (U_e h))
//
// Assignment a = token * top + place.  moe_group_kernel sorts the assignments by expert (one
// block; the order within an expert does not matter: a row of a product depends on no other
// row) and cuts each expert's run into tiles of kTileRows rows.  The product kernels run one
// block per (tile, 64 output columns); blocks past the step's count of tiles leave at once, so
// the grid depends on the step's size class only.  Every row's sums run over the inner size in
// a fixed order.  The down product leaves w_e * (its row) in rows[a, :] (32-bit): the sum over
// a token's places is taken by whoever adds the rows into the stream, in the order of the places.
#include "common.cuh"

constexpr int kTileRows = 32;
constexpr int kTileCols = 64;
constexpr int kTileInner = 32;
constexpr int kMaxExperts = 1024;

struct MoeParams {
  const void* h;            // [tokens, hidden], the run's type
  const float* router;      // [experts, hidden]
  const void* gate;         // [experts, ff, hidden]
  const void* up;           // [experts, ff, hidden]
  const void* down;         // [experts, hidden, ff]
  int* chosen;              // [tokens * top]
  float* weight;            // [tokens * top]
  int* order;               // [tokens * top] assignments sorted by expert
  int* rank;                // [tokens * top] scratch
  int* tiles;               // [1 + 3 * max_tiles]: count, then (expert, first sorted place, rows) per tile
  void* act;                // [tokens * top, ff], the run's type, in sorted order
  float* rows;              // [tokens * top, hidden]
  int num_tokens, hidden, ff, experts, top, groups, keep, group_top, max_tiles;
  int softmax_scores, renormalize, activation;
};

// The lane holding the largest value wins; equal values go to the lower index.
__device__ __forceinline__ void warp_argmax(float& best, int& index) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, best, offset);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
    if (other > best || (other == best && other_index < index)) {
      best = other;
      index = other_index;
    }
  }
}

// A warp per token.
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(MoeParams p) {
  extern __shared__ float route_shared[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= p.num_tokens) return;
  float* score = route_shared + warp * (2 * p.experts + p.groups);
  float* open = score + p.experts;          // the score while the expert may still be chosen, else -inf
  float* group_score = open + p.experts;
  const T* h = static_cast<const T*>(p.h) + static_cast<size_t>(t) * p.hidden;
  for (int e = 0; e < p.experts; ++e) {
    const float* r = p.router + static_cast<size_t>(e) * p.hidden;
    float sum = 0.0f;
    for (int i = lane; i < p.hidden; i += 32) sum = fmaf(to_float<T>(h[i]), r[i], sum);
    sum = warp_sum(sum);
    if (lane == 0) score[e] = sum;
  }
  __syncwarp();
  if (p.softmax_scores) {
    float top_z = -INFINITY;
    for (int e = lane; e < p.experts; e += 32) top_z = fmaxf(top_z, score[e]);
    top_z = warp_max(top_z);
    float total = 0.0f;
    for (int e = lane; e < p.experts; e += 32) total += expf(score[e] - top_z);
    total = warp_sum(total);
    for (int e = lane; e < p.experts; e += 32) score[e] = expf(score[e] - top_z) / total;
  } else {
    for (int e = lane; e < p.experts; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
  }
  __syncwarp();
  // a value that is no number may not win a comparison: it counts as the lowest
  for (int e = lane; e < p.experts; e += 32) open[e] = score[e] == score[e] ? score[e] : -1.0e30f;
  __syncwarp();
  const int per_group = p.experts / p.groups;
  if (p.keep < p.groups) {
    for (int g = lane; g < p.groups; g += 32) {
      // the sum of the group's group_top largest scores, found one after the other
      float total = 0.0f;
      int taken_a = -1, taken_b = -1;   // group_top is at most 2 here; more would need a list
      for (int round = 0; round < min(p.group_top, per_group); ++round) {
        float best = -INFINITY;
        int at = -1;
        for (int i = 0; i < per_group; ++i) {
          if (i == taken_a || i == taken_b) continue;
          const float v = open[g * per_group + i];
          if (v > best) best = v, at = i;
        }
        total += best;
        if (round == 0) taken_a = at; else taken_b = at;
      }
      group_score[g] = total;
    }
    __syncwarp();
    // keep the best groups: mark them by a score of +inf, then close the experts of the others
    for (int round = 0; round < p.keep; ++round) {
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < p.groups; g += 32) {
        const float v = group_score[g];
        if (v < INFINITY && (v > best || at == 0x7fffffff)) best = v, at = g;
      }
      warp_argmax(best, at);
      if (lane == 0 && at != 0x7fffffff) group_score[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < p.experts; e += 32)
      if (group_score[e / per_group] != INFINITY) open[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.0f;
  for (int place = 0; place < p.top; ++place) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < p.experts; e += 32) {
      const float v = open[e];
      if (v > best) best = v, at = e;
    }
    warp_argmax(best, at);
    if (at == 0x7fffffff) at = 0;   // cannot happen with top <= keep * per_group; keeps the index in range
    const float w = score[at];
    total += w;
    if (lane == 0) {
      p.chosen[static_cast<size_t>(t) * p.top + place] = at;
      p.weight[static_cast<size_t>(t) * p.top + place] = w;
      open[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (p.renormalize && lane == 0)
    for (int place = 0; place < p.top; ++place) p.weight[static_cast<size_t>(t) * p.top + place] /= total;
}

// One block: assignments counted per expert, the experts' runs cut into tiles, the sorted order.
__global__ void __launch_bounds__(1024)
moe_group_kernel(MoeParams p) {
  __shared__ int count[kMaxExperts];
  __shared__ int start[kMaxExperts];
  pdl_launch_dependents();
  pdl_wait();
  const int assignments = p.num_tokens * p.top;
  for (int e = threadIdx.x; e < p.experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) p.rank[a] = atomicAdd(&count[p.chosen[a]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int place = 0, tile = 0;
    for (int e = 0; e < p.experts; ++e) {
      start[e] = place;
      for (int first = 0; first < count[e] && tile < p.max_tiles; first += kTileRows, ++tile) {
        p.tiles[1 + 3 * tile] = e;
        p.tiles[2 + 3 * tile] = place + first;
        p.tiles[3 + 3 * tile] = min(kTileRows, count[e] - first);
      }
      place += count[e];
    }
    p.tiles[0] = tile;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) p.order[start[p.chosen[a]] + p.rank[a]] = a;
}

// ---------------------------------------------------------------------------------------
// The experts' products on the CUDA cores: a block computes kTileRows x kTileCols of one tile.
// GATED: out = act(G_e x) * (U_e x) for x = h[token of the assignment], stored in sorted order.
// else:  rows[a, :] = w_a * (D_e act[sorted place of a]).
// Threads: 16 across the columns (columns c, c + 16, c + 32, c + 48) by 16 down the rows (r, r + 16).
// ---------------------------------------------------------------------------------------
template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_product_kernel(MoeParams p) {
  __shared__ float x_s[kTileRows][kTileInner + 1];
  __shared__ float w_s[GATED ? 2 : 1][kTileCols][kTileInner + 1];
  __shared__ int row_source[kTileRows];
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= p.tiles[0]) return;
  const int expert = p.tiles[1 + 3 * tile], first = p.tiles[2 + 3 * tile], rows = p.tiles[3 + 3 * tile];
  const int inner = GATED ? p.hidden : p.ff;
  const int outer = GATED ? p.ff : p.hidden;
  const int col0 = blockIdx.x * kTileCols;
  if (threadIdx.x < kTileRows) {
    int source = -1;
    if (threadIdx.x < rows) source = GATED ? p.order[first + threadIdx.x] / p.top : first + threadIdx.x;
    row_source[threadIdx.x] = source;
  }
  __syncthreads();
  const T* x = static_cast<const T*>(GATED ? p.h : p.act);
  const T* w0 = static_cast<const T*>(GATED ? p.gate : p.down) + static_cast<size_t>(expert) * outer * inner;
  const T* w1 = GATED ? static_cast<const T*>(p.up) + static_cast<size_t>(expert) * outer * inner : nullptr;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc0[2][4], acc1[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.0f;
  for (int k0 = 0; k0 < inner; k0 += kTileInner) {
    for (int i = threadIdx.x; i < kTileRows * kTileInner; i += 256) {
      const int r = i / kTileInner, k = i % kTileInner;
      const int source = row_source[r];
      x_s[r][k] = (source >= 0 && k0 + k < inner) ? to_float<T>(x[static_cast<size_t>(source) * inner + k0 + k]) : 0.0f;
    }
    for (int i = threadIdx.x; i < kTileCols * kTileInner; i += 256) {
      const int c = i / kTileInner, k = i % kTileInner;
      const bool live = col0 + c < outer && k0 + k < inner;
      const size_t at = static_cast<size_t>(col0 + c) * inner + k0 + k;
      w_s[0][c][k] = live ? to_float<T>(w0[at]) : 0.0f;
      if (GATED) w_s[1][c][k] = live ? to_float<T>(w1[at]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kTileInner; ++k) {
      const float a0 = x_s[ty][k], a1 = x_s[ty + 16][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = w_s[0][tx + 16 * j][k];
        acc0[0][j] = fmaf(a0, b, acc0[0][j]);
        acc0[1][j] = fmaf(a1, b, acc0[1][j]);
        if (GATED) {
          const float c = w_s[1][tx + 16 * j][k];
          acc1[0][j] = fmaf(a0, c, acc1[0][j]);
          acc1[1][j] = fmaf(a1, c, acc1[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty + 16 * i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx + 16 * j;
      if (c >= outer) continue;
      if (GATED) {
        static_cast<T*>(p.act)[static_cast<size_t>(first + r) * p.ff + c] =
            from_float<T>(gate_activation(acc0[i][j], p.activation) * acc1[i][j]);
      } else {
        const int a = p.order[first + r];
        p.rows[static_cast<size_t>(a) * p.hidden + c] = p.weight[a] * acc0[i][j];
      }
    }
  }
}

template <typename T>
static int launch_moe(const MoeParams& p, cudaStream_t s) {
  const size_t route_shared = 4 * static_cast<size_t>(2 * p.experts + p.groups) * sizeof(float);
  int status = vipera_launch(moe_route_kernel<T>, (p.num_tokens + 3) / 4, 128, route_shared, s, p);
  if (status) return status;
  status = vipera_launch(moe_group_kernel, 1, 1024, 0, s, p);
  if (status) return status;
  status = vipera_launch(moe_product_kernel<T, true>, dim3((p.ff + kTileCols - 1) / kTileCols, p.max_tiles), 256, 0, s, p);
  if (status) return status;
  return vipera_launch(moe_product_kernel<T, false>, dim3((p.hidden + kTileCols - 1) / kTileCols, p.max_tiles), 256, 0, s, p);
}

// dtype: the type of h, the experts' matrices and the scratch `act`.
VIPERA_API int vipera_moe(const MoeParams* params, int dtype, void* stream) {
  const MoeParams& p = *params;
  if (p.num_tokens <= 0) return VIPERA_OK;
  if (p.experts <= 0 || p.experts > kMaxExperts || p.groups <= 0 || p.experts % p.groups || p.keep <= 0 ||
      p.keep > p.groups || p.top <= 0 || p.top > p.keep * (p.experts / p.groups) || p.group_top < 1 || p.group_top > 2 ||
      p.hidden <= 0 || p.ff <= 0)
    return VIPERA_BAD_SHAPE;
  if (p.max_tiles < p.num_tokens * p.top / kTileRows + min(p.experts, p.num_tokens * p.top) || p.max_tiles > 65535)
    return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == VIPERA_F32) return launch_moe<float>(p, s);
  if (dtype == VIPERA_BF16) return launch_moe<__nv_bfloat16>(p, s);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API int vipera_moe_params_size() { return static_cast<int>(sizeof(MoeParams)); }
VIPERA_API int vipera_moe_tile_rows() { return kTileRows; }
VIPERA_API const char* vipera_moe_status_text(int status) { return vipera_status_text(status); }

// target[t, :] += sum over the places of rows[t, place, :], in the order of the places.
__global__ void __launch_bounds__(256)
moe_add_rows_kernel(const float* __restrict__ rows, int parts, float* __restrict__ target, long long count, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long t = i / hidden;
  const int c = static_cast<int>(i % hidden);
  const float* r = rows + t * parts * hidden + c;
  float sum = r[0];
  for (int p = 1; p < parts; ++p) sum += r[static_cast<size_t>(p) * hidden];
  target[i] += sum;
}

VIPERA_API int vipera_moe_add_rows(const float* rows, int parts, float* target, int num_tokens, int hidden, void* stream) {
  if (num_tokens <= 0) return VIPERA_OK;
  if (parts <= 0 || hidden <= 0) return VIPERA_BAD_SHAPE;
  const long long count = static_cast<long long>(num_tokens) * hidden;
  return vipera_launch(moe_add_rows_kernel, static_cast<unsigned>((count + 255) / 256), 256, 0,
                       static_cast<cudaStream_t>(stream), rows, parts, target, count, hidden);
}
