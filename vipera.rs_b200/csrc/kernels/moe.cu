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
// row) and cuts each expert's run into tiles of `tile_rows` rows.  Three forms of the products:
//   * few assignments (decode): tiles of 8 rows; a warp streams four weight rows once for all rows
//     of the tile (moe_skinny_kernel), so the step reads each used expert's matrices once;
//   * many assignments in bfloat16: every expert's run starts at a multiple of 128 sorted rows
//     (`padded`), the tokens' rows are gathered in that order, and the two products are grouped
//     products on the tensor cores (gemm_tc.cu: the 128 rows of a tile use the matrices of the
//     tile's expert); a last kernel weights each row and puts it at its assignment's place;
//   * otherwise (32-bit, sizes the tensor-core product refuses): tiles of 32 rows on the CUDA cores.
// Blocks past the step's count of tiles leave at once, so a grid depends on the step's size only.
// Every row's sums run over the inner size in an order that depends on the form alone.  The down
// product leaves w_e * (its row) in rows[a, :] (32-bit): the sum over a token's places is taken
// by whoever adds the rows into the stream, in the order of the places.
//
// Gate and up matrices are one tensor [experts, 2 ff, hidden]: `gate_group` gate rows, then the
// up rows of the same features, and so on (16 for the tensor-core ending; ff: all gate rows first).
//
// Options.  `gated` = 0: the units have no gate, y_e = D_e act(U_e h), and `gate_up` is [matrices,
// ff, hidden].  `correction`: a number per router output that is added to the scores for the choice
// only (the weights are the scores themselves).  `identity`: the last that many router outputs have no
// matrices; chosen, they return the token's own row times their weight (the router's block writes that
// row).  `always`: that many units beyond the router's own which every token uses with weight 1 (a
// shared unit, cut into pieces of the experts' inner size); their matrices follow the chosen experts'
// in the same tensors, and a token has `slots` = top + always assignments.  With `renormalize` the
// weights are divided by their sum + `renorm_eps`; `route_scale` multiplies them.
#include "common.cuh"

constexpr int kTileRows = 32;
constexpr int kTileCols = 64;
constexpr int kTileInner = 32;
constexpr int kMaxExperts = 1024;
constexpr int kSkinnyRows = 8;
constexpr int kRouteThreads = 256;

struct MoeParams {
  const void* h;            // [tokens, hidden], the run's type
  const float* router;      // [experts, hidden]
  const void* gate_up;      // [experts, 2 ff, hidden]
  const void* down;         // [experts, hidden, ff]
  int* chosen;              // [tokens * top]
  float* weight;            // [tokens * top]
  int* order;               // [capacity] sorted place -> assignment (-1: a place that pads a run)
  int* rank;                // [tokens * top] assignment -> sorted place
  int* tiles;               // [1 + 3 * max_tiles]: count, then (expert, first sorted place, rows) per tile
  int* tile_expert;         // [max_tiles] the tile's expert (0 past the count)
  void* act;                // [capacity, ff], the run's type, in sorted order
  float* rows;              // [tokens * top, hidden]
  void* xs;                 // padded form: [capacity, hidden] the tokens' rows in sorted order
  float* ys;                // padded form: [capacity, hidden] the down products in sorted order
  int num_tokens, hidden, ff, experts, top, groups, keep, group_top, max_tiles;
  int softmax_scores, renormalize, activation;
  int gate_group;           // gate rows and up rows alternate in groups of this many
  int tile_rows;            // 8, 32 or (padded) 128
  int padded;               // 1: every expert's run starts at a multiple of tile_rows; capacity = max_tiles * tile_rows
  const float* correction;  // [experts] added to the scores for the choice; null: nothing
  int identity;             // the last `identity` of the `experts` router outputs return their input
  int always;               // units every token uses with weight 1, after the router's own in the matrices
  int slots;                // top + always: a token's assignments
  int gated;                // 1: gated units; 0: act(U h)
  float route_scale, renorm_eps;
};

// The units that have matrices: the router's outputs without the identity ones, then the ones every token uses.
__device__ __forceinline__ int moe_matrices(const MoeParams& p) { return p.experts - p.identity + p.always; }

__device__ __forceinline__ size_t gate_row(int feature, int group) {
  return static_cast<size_t>(feature / group) * 2 * group + feature % group;
}

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

// A block per token: its warps share the experts' logits between them (a lane sums every 32nd
// product, the warp adds the lanes), then the first warp chooses.
template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(MoeParams p) {
  extern __shared__ __align__(16) float route_shared[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  float* h_s = route_shared;                // [hidden] (first: read as vectors)
  float* score = h_s + p.hidden;
  float* open = score + p.experts;          // the score while the expert may still be chosen, else -inf
  float* group_score = open + p.experts;
  const T* h = static_cast<const T*>(p.h) + static_cast<size_t>(t) * p.hidden;
  for (int i = threadIdx.x; i < p.hidden; i += kRouteThreads) h_s[i] = to_float<T>(h[i]);
  __syncthreads();
  constexpr int kWarpsHere = kRouteThreads / 32;
  if ((p.hidden & 3) == 0 && (reinterpret_cast<uintptr_t>(p.router) & 15) == 0) {
    // Four values at a time: a lane sums the products of values 4 (lane + 32 j) .. + 3, in that order.  A warp
    // walks four of its rows side by side, so that their loads are in flight together (a step of one token is
    // one block, which waits for every row it asks for).
    const float4* h4 = reinterpret_cast<const float4*>(h_s);
    for (int e0 = warp; e0 < p.experts; e0 += 4 * kWarpsHere) {
      const float4* rows[4];
      float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        rows[j] = reinterpret_cast<const float4*>(p.router + static_cast<size_t>(min(e0 + j * kWarpsHere, p.experts - 1)) * p.hidden);
#pragma unroll 4
      for (int i = lane; i < p.hidden / 4; i += 32) {
        const float4 a = h4[i];
        float4 b[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = rows[j][i];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          sums[j] = fmaf(a.x, b[j].x, sums[j]);
          sums[j] = fmaf(a.y, b[j].y, sums[j]);
          sums[j] = fmaf(a.z, b[j].z, sums[j]);
          sums[j] = fmaf(a.w, b[j].w, sums[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float sum = warp_sum(sums[j]);
        if (lane == 0 && e0 + j * kWarpsHere < p.experts) score[e0 + j * kWarpsHere] = sum;
      }
    }
  } else {
    for (int e = warp; e < p.experts; e += kWarpsHere) {
      const float* r = p.router + static_cast<size_t>(e) * p.hidden;
      float sum = 0.0f;
#pragma unroll 4
      for (int i = lane; i < p.hidden; i += 32) sum = fmaf(h_s[i], r[i], sum);
      sum = warp_sum(sum);
      if (lane == 0) score[e] = sum;
    }
  }
  __syncthreads();
  if (warp == 0) {
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
  for (int e = lane; e < p.experts; e += 32) {
    const float choice = score[e] + (p.correction ? p.correction[e] : 0.0f);
    open[e] = choice == choice ? choice : -1.0e30f;
  }
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
      // an output without matrices is marked -1 - (its index among those)
      p.chosen[static_cast<size_t>(t) * p.slots + place] = at < p.experts - p.identity ? at : -1 - (at - (p.experts - p.identity));
      p.weight[static_cast<size_t>(t) * p.slots + place] = w;
      open[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float divisor = p.renormalize ? total + p.renorm_eps : 1.0f;
    for (int place = 0; place < p.top; ++place) {
      const size_t a = static_cast<size_t>(t) * p.slots + place;
      p.weight[a] = p.weight[a] / divisor * p.route_scale;
    }
    for (int extra = 0; extra < p.always; ++extra) {
      p.chosen[static_cast<size_t>(t) * p.slots + p.top + extra] = p.experts - p.identity + extra;
      p.weight[static_cast<size_t>(t) * p.slots + p.top + extra] = 1.0f;
    }
  }
  }
  if (p.identity == 0) return;
  __syncthreads();   // the choice is written
  for (int place = 0; place < p.top; ++place) {
    const size_t a = static_cast<size_t>(t) * p.slots + place;
    if (p.chosen[a] >= 0) continue;
    const float w = p.weight[a];
    for (int i = threadIdx.x; i < p.hidden; i += kRouteThreads) p.rows[a * p.hidden + i] = w * h_s[i];
  }
}

// One block: assignments counted per expert, the experts' runs cut into tiles, the sorted order.
__global__ void __launch_bounds__(1024)
moe_group_kernel(MoeParams p) {
  __shared__ int count[kMaxExperts];
  __shared__ int start[kMaxExperts];
  pdl_launch_dependents();
  pdl_wait();
  const int assignments = p.num_tokens * p.slots;
  const int matrices = moe_matrices(p);
  for (int e = threadIdx.x; e < matrices; e += blockDim.x) count[e] = 0;
  for (int tile = threadIdx.x; tile < p.max_tiles; tile += blockDim.x) p.tile_expert[tile] = 0;
  if (p.padded)
    for (int place = threadIdx.x; place < p.max_tiles * p.tile_rows; place += blockDim.x) p.order[place] = -1;
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x)
    p.rank[a] = p.chosen[a] >= 0 ? atomicAdd(&count[p.chosen[a]], 1) : -1;   // (-1: no matrices, no place)
  __syncthreads();
  if (threadIdx.x == 0) {
    int place = 0, tile = 0;
    for (int e = 0; e < matrices; ++e) {
      start[e] = place;
      int first = 0;
      for (; first < count[e] && tile < p.max_tiles; first += p.tile_rows, ++tile) {
        p.tiles[1 + 3 * tile] = e;
        p.tiles[2 + 3 * tile] = place + first;
        p.tiles[3 + 3 * tile] = min(p.tile_rows, count[e] - first);
        p.tile_expert[tile] = e;
      }
      place += p.padded ? first : count[e];
    }
    p.tiles[0] = tile;
  }
  __syncthreads();
  for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
    if (p.chosen[a] < 0) continue;
    const int place = start[p.chosen[a]] + p.rank[a];
    p.rank[a] = place;
    p.order[place] = a;
  }
}

// Padded form: the tokens' rows in sorted order (zero where a place pads a run); a block per place.
template <typename T>
__global__ void __launch_bounds__(128)
moe_gather_kernel(MoeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int place = blockIdx.x;
  if (place / p.tile_rows >= p.tiles[0]) return;
  const int a = p.order[place];
  const int vectors = p.hidden * static_cast<int>(sizeof(T)) / 16;   // the caller sees to whole vectors
  uint4* dst = reinterpret_cast<uint4*>(static_cast<T*>(p.xs) + static_cast<size_t>(place) * p.hidden);
  if (a < 0) {
    for (int i = threadIdx.x; i < vectors; i += blockDim.x) dst[i] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(p.h) + static_cast<size_t>(a / p.slots) * p.hidden);
  for (int i = threadIdx.x; i < vectors; i += blockDim.x) dst[i] = src[i];
}

// Padded form: rows[a, :] = w_a * ys[sorted place of a, :].
__global__ void __launch_bounds__(256)
moe_scatter_kernel(MoeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int quarter = p.hidden / 4;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(p.num_tokens) * p.slots * quarter) return;
  const int a = static_cast<int>(i / quarter), c = static_cast<int>(i % quarter);
  if (p.rank[a] < 0) return;   // the router's block wrote this row
  const float w = p.weight[a];
  float4 v = reinterpret_cast<const float4*>(p.ys + static_cast<size_t>(p.rank[a]) * p.hidden)[c];
  v.x *= w, v.y *= w, v.z *= w, v.w *= w;
  reinterpret_cast<float4*>(p.rows + static_cast<size_t>(a) * p.hidden)[c] = v;
}

// ---------------------------------------------------------------------------------------
// Few assignments: a block takes one tile of up to 8 rows and 8 warps x 4 weight rows (GATED: the
// gate and up rows of 2 features per warp; else 4 output columns per warp).  The tile's rows wait
// in shared memory; a lane reads 16 bytes of each of its warp's weight rows per turn, so every
// weight byte is read once per tile, and the lanes' partial sums are added at the end.
// ---------------------------------------------------------------------------------------
template <typename T, int VEC>
__device__ __forceinline__ void load_span(const T* __restrict__ src, float (&dst)[VEC]);
template <>
__device__ __forceinline__ void load_span<float, 4>(const float* __restrict__ src, float (&dst)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
}
template <>
__device__ __forceinline__ void load_span<float, 1>(const float* __restrict__ src, float (&dst)[1]) { dst[0] = src[0]; }
template <>
__device__ __forceinline__ void load_span<__nv_bfloat16, 8>(const __nv_bfloat16* __restrict__ src, float (&dst)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(pairs[e]);
    dst[2 * e] = f.x, dst[2 * e + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load_span<__nv_bfloat16, 1>(const __nv_bfloat16* __restrict__ src, float (&dst)[1]) {
  dst[0] = __bfloat162float(src[0]);
}

// MODE 0: the down product; 1: gate and up with the gated unit as ending; 2: up alone with its activation.
template <typename T, int MODE, int VEC>
__global__ void __launch_bounds__(256)
moe_skinny_kernel(MoeParams p) {
  constexpr bool GATED = MODE == 1;
  constexpr bool FIRST = MODE != 0;
  extern __shared__ __align__(16) unsigned char skinny_shared[];
  T* x_s = reinterpret_cast<T*>(skinny_shared);   // [kSkinnyRows][inner]
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= p.tiles[0]) return;
  const int expert = p.tiles[1 + 3 * tile], first = p.tiles[2 + 3 * tile], rows = p.tiles[3 + 3 * tile];
  const int inner = FIRST ? p.hidden : p.ff;
  const int outer = FIRST ? p.ff : p.hidden;
  const T* x = static_cast<const T*>(FIRST ? p.h : p.act);
  for (int i = threadIdx.x * VEC; i < rows * inner; i += 256 * VEC) {
    const int r = i / inner, k = i % inner;   // (inner is a multiple of VEC)
    const size_t source = FIRST ? static_cast<size_t>(p.order[first + r] / p.slots) : static_cast<size_t>(first + r);
    if (VEC > 1) *reinterpret_cast<uint4*>(x_s + i) = *reinterpret_cast<const uint4*>(x + source * inner + k);
    else x_s[i] = x[source * inner + k];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this warp's four weight rows
  const int per_warp = GATED ? 2 : 4;
  const int col0 = (blockIdx.x * 8 + warp) * per_warp;
  if (col0 >= outer) return;
  const T* w_rows[4];
  const T* base = static_cast<const T*>(FIRST ? p.gate_up : p.down) +
                  static_cast<size_t>(expert) * (GATED ? 2 : 1) * outer * inner;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = min(col0 + (GATED ? j >> 1 : j), outer - 1);
    const size_t row = GATED ? gate_row(c, p.gate_group) + ((j & 1) ? p.gate_group : 0) : static_cast<size_t>(c);
    w_rows[j] = base + row * inner;
  }
  float acc[4][kSkinnyRows];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int r = 0; r < kSkinnyRows; ++r) acc[j][r] = 0.0f;
#pragma unroll 2
  for (int k = lane * VEC; k < inner; k += 32 * VEC) {
    float w[4][VEC];
#pragma unroll
    for (int j = 0; j < 4; ++j) load_span<T, VEC>(w_rows[j] + k, w[j]);
#pragma unroll
    for (int r = 0; r < kSkinnyRows; ++r) {
      if (r < rows) {
        float xv[VEC];
        load_span<T, VEC>(x_s + r * inner + k, xv);
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[j][r] = fmaf(w[j][e], xv[e], acc[j][r]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int r = 0; r < kSkinnyRows; ++r) acc[j][r] = warp_sum(acc[j][r]);
  if (lane != 0) return;
#pragma unroll
  for (int r = 0; r < kSkinnyRows; ++r) {
    if (r >= rows) continue;
    if (GATED) {
#pragma unroll
      for (int f = 0; f < 2; ++f)
        if (col0 + f < outer)
          static_cast<T*>(p.act)[static_cast<size_t>(first + r) * p.ff + col0 + f] =
              from_float<T>(gate_activation(acc[2 * f][r], p.activation) * acc[2 * f + 1][r]);
    } else if (FIRST) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (col0 + j < outer)
          static_cast<T*>(p.act)[static_cast<size_t>(first + r) * p.ff + col0 + j] = from_float<T>(gate_activation(acc[j][r], p.activation));
    } else {
      const int a = p.order[first + r];
      const float weight = p.weight[a];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (col0 + j < outer) p.rows[static_cast<size_t>(a) * p.hidden + col0 + j] = weight * acc[j][r];
    }
  }
}

// ---------------------------------------------------------------------------------------
// The experts' products on the CUDA cores: a block computes kTileRows x kTileCols of one tile.
// GATED: out = act(G_e x) * (U_e x) for x = h[token of the assignment], stored in sorted order.
// else:  rows[a, :] = w_a * (D_e act[sorted place of a]).
// Threads: 16 across the columns (columns c, c + 16, c + 32, c + 48) by 16 down the rows (r, r + 16).
// ---------------------------------------------------------------------------------------
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_product_kernel(MoeParams p) {
  constexpr bool GATED = MODE == 1;
  constexpr bool FIRST = MODE != 0;
  __shared__ float x_s[kTileRows][kTileInner + 1];
  __shared__ float w_s[GATED ? 2 : 1][kTileCols][kTileInner + 1];
  __shared__ int row_source[kTileRows];
  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y;
  if (tile >= p.tiles[0]) return;
  const int expert = p.tiles[1 + 3 * tile], first = p.tiles[2 + 3 * tile], rows = p.tiles[3 + 3 * tile];
  const int inner = FIRST ? p.hidden : p.ff;
  const int outer = FIRST ? p.ff : p.hidden;
  const int col0 = blockIdx.x * kTileCols;
  if (threadIdx.x < kTileRows) {
    int source = -1;
    if (threadIdx.x < rows) source = FIRST ? p.order[first + threadIdx.x] / p.slots : first + threadIdx.x;
    row_source[threadIdx.x] = source;
  }
  __syncthreads();
  const T* x = static_cast<const T*>(FIRST ? p.h : p.act);
  // GATED: the gate row of feature c is at gate_row(c), its up row gate_group rows further
  const T* w0 = static_cast<const T*>(FIRST ? p.gate_up : p.down) + static_cast<size_t>(expert) * (GATED ? 2 : 1) * outer * inner;
  const T* w1 = GATED ? w0 + static_cast<size_t>(p.gate_group) * inner : nullptr;
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
      const size_t at = (GATED ? gate_row(min(col0 + c, outer - 1), p.gate_group) : static_cast<size_t>(col0 + c)) * inner + k0 + k;
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
      } else if (FIRST) {
        static_cast<T*>(p.act)[static_cast<size_t>(first + r) * p.ff + c] = from_float<T>(gate_activation(acc0[i][j], p.activation));
      } else {
        const int a = p.order[first + r];
        p.rows[static_cast<size_t>(a) * p.hidden + c] = p.weight[a] * acc0[i][j];
      }
    }
  }
}

template <typename T, int MODE>
static int launch_skinny(const MoeParams& p, cudaStream_t s) {
  constexpr int kVec = 16 / static_cast<int>(sizeof(T));
  constexpr bool GATED = MODE == 1;
  constexpr bool FIRST = MODE != 0;
  const int inner = FIRST ? p.hidden : p.ff;
  const int outer = FIRST ? p.ff : p.hidden;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(FIRST ? p.h : p.act) | reinterpret_cast<uintptr_t>(FIRST ? p.gate_up : p.down);
  const bool whole = inner % kVec == 0 && (bases & 15) == 0;
  const size_t shared = static_cast<size_t>(kSkinnyRows) * inner * sizeof(T);
  const dim3 grid((outer + (GATED ? 16 : 32) - 1) / (GATED ? 16 : 32), p.max_tiles);
  if (whole) {
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(moe_skinny_kernel<T, MODE, kVec>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return VIPERA_BAD_ARGUMENT;
      configured = true;
    }
    return vipera_launch(moe_skinny_kernel<T, MODE, kVec>, grid, 256, shared, s, p);
  }
  static bool configured_single = false;
  if (!configured_single) {
    if (cudaFuncSetAttribute(moe_skinny_kernel<T, MODE, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return VIPERA_BAD_ARGUMENT;
    configured_single = true;
  }
  return vipera_launch(moe_skinny_kernel<T, MODE, 1>, grid, 256, shared, s, p);
}

// The router, the grouping and (padded form) the gathered rows.
template <typename T>
static int launch_route(const MoeParams& p, cudaStream_t s) {
  const size_t route_shared = static_cast<size_t>(2 * p.experts + p.groups + p.hidden) * sizeof(float);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(moe_route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return VIPERA_BAD_ARGUMENT;
    configured = true;
  }
  int status = vipera_launch(moe_route_kernel<T>, p.num_tokens, kRouteThreads, route_shared, s, p);
  if (status) return status;
  status = vipera_launch(moe_group_kernel, 1, 1024, 0, s, p);
  if (status || !p.padded) return status;
  return vipera_launch(moe_gather_kernel<T>, p.max_tiles * p.tile_rows, 128, 0, s, p);
}

template <typename T>
static int launch_products(const MoeParams& p, cudaStream_t s) {
  if (p.tile_rows == kSkinnyRows) {
    const int status = p.gated ? launch_skinny<T, 1>(p, s) : launch_skinny<T, 2>(p, s);
    return status ? status : launch_skinny<T, 0>(p, s);
  }
  const dim3 first_grid((p.ff + kTileCols - 1) / kTileCols, p.max_tiles);
  int status = p.gated ? vipera_launch(moe_product_kernel<T, 1>, first_grid, 256, 0, s, p)
                       : vipera_launch(moe_product_kernel<T, 2>, first_grid, 256, 0, s, p);
  if (status) return status;
  return vipera_launch(moe_product_kernel<T, 0>, dim3((p.hidden + kTileCols - 1) / kTileCols, p.max_tiles), 256, 0, s, p);
}

static int check_moe(const MoeParams& p) {
  if (p.experts <= 0 || p.experts > kMaxExperts || p.groups <= 0 || p.experts % p.groups || p.keep <= 0 ||
      p.keep > p.groups || p.top <= 0 || p.top > p.keep * (p.experts / p.groups) || p.group_top < 1 || p.group_top > 2 ||
      p.hidden <= 0 || p.ff <= 0 || (p.gated && (p.gate_group <= 0 || p.ff % p.gate_group)))
    return VIPERA_BAD_SHAPE;
  if (p.identity < 0 || p.identity > p.experts || p.always < 0 || p.slots != p.top + p.always ||
      p.experts - p.identity + p.always > kMaxExperts || (p.identity > 0 && !p.rows))
    return VIPERA_BAD_SHAPE;
  if (p.padded ? p.tile_rows != 128 : (p.tile_rows != kSkinnyRows && p.tile_rows != kTileRows)) return VIPERA_BAD_ARGUMENT;
  if (p.max_tiles < p.num_tokens * p.slots / p.tile_rows + min(p.experts - p.identity + p.always, p.num_tokens * p.slots) ||
      p.max_tiles > 65535)
    return VIPERA_BAD_ARGUMENT;
  if (static_cast<size_t>(2 * p.experts + p.groups + p.hidden) * sizeof(float) > 200 * 1024) return VIPERA_BAD_SHAPE;
  if (p.tile_rows == kSkinnyRows && static_cast<size_t>(kSkinnyRows) * max(p.hidden, p.ff) * 4 > 200 * 1024) return VIPERA_BAD_SHAPE;
  if (p.padded && (!p.xs || !p.ys || (p.hidden * 2) % 16 || (reinterpret_cast<uintptr_t>(p.xs) & 15) ||
                   (reinterpret_cast<uintptr_t>(p.h) & 15) || (reinterpret_cast<uintptr_t>(p.ys) & 15) ||
                   (reinterpret_cast<uintptr_t>(p.rows) & 15)))
    return VIPERA_BAD_ARGUMENT;
  return VIPERA_OK;
}

// Router and grouping; unless `padded`, the products too.  dtype: the type of h, the experts'
// matrices and the scratch `act`.  (Padded form: the caller runs the two grouped products on
// xs and act between this and vipera_moe_scatter.)
VIPERA_API int vipera_moe(const MoeParams* params, int dtype, void* stream) {
  const MoeParams& p = *params;
  if (p.num_tokens <= 0) return VIPERA_OK;
  int status = check_moe(p);
  if (status) return status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == VIPERA_F32) {
    if (p.padded) return VIPERA_BAD_DTYPE;
    status = launch_route<float>(p, s);
    return status ? status : launch_products<float>(p, s);
  }
  if (dtype != VIPERA_BF16) return VIPERA_BAD_DTYPE;
  status = launch_route<__nv_bfloat16>(p, s);
  return (status || p.padded) ? status : launch_products<__nv_bfloat16>(p, s);
}

VIPERA_API int vipera_moe_scatter(const MoeParams* params, void* stream) {
  const MoeParams& p = *params;
  if (p.num_tokens <= 0) return VIPERA_OK;
  if (!p.padded || p.hidden % 4) return VIPERA_BAD_ARGUMENT;
  const long long count = static_cast<long long>(p.num_tokens) * p.slots * (p.hidden / 4);
  return vipera_launch(moe_scatter_kernel, static_cast<unsigned>((count + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream), p);
}

VIPERA_API int vipera_moe_params_size() { return static_cast<int>(sizeof(MoeParams)); }
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
