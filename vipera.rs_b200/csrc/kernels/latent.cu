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
// rotated part (`pairing` 0) or values (i, i + rot/2) (`pairing` 1) turn by the angle whose cosine
// and sine the tables hold at [position, i].  With a window w > 0 the query at position p sees keys
// p - w + 1 .. p only; earlier keys' pages may have been given back and are never read.
#include "attention_mma.cuh"

constexpr int kMaxRank = 512;   // latent size
constexpr int kMaxRot = 128;    // rotated part
constexpr int kWarps = 4;

// The two values of the rotated part that turn together as pair i.
__device__ __forceinline__ void rot_pair(int pairing, int rot, int i, int& a, int& b) {
  if (pairing) { a = i; b = i + rot / 2; } else { a = 2 * i; b = 2 * i + 1; }
}

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
                    int page_size, int rank, int rot, int pairing) {
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
    int ia, ib;
    rot_pair(pairing, rot, i, ia, ib);
    const float u = row[rank + ia], v = row[rank + ib];
    r_row[ia] = from_float<T>(u * cs[i] - v * sn[i]);
    r_row[ib] = from_float<T>(v * cs[i] + u * sn[i]);
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
                     int rank, int rot, float scale, int pairing) {
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
  // (blocks along z share the rank between them)
  for (int r = blockIdx.z * blockDim.x + threadIdx.x; r < rank; r += gridDim.z * blockDim.x) {
    float acc[kTile];
#pragma unroll
    for (int tt = 0; tt < kTile; ++tt) acc[tt] = 0.0f;
#pragma unroll 8
    for (int e = 0; e < d; ++e) {
      const float w = to_float<TW>(u[static_cast<size_t>(e) * rank + r]);
#pragma unroll
      for (int tt = 0; tt < kTile; ++tt) acc[tt] = fmaf(q_tile[tt * d + e], w, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < kTile; ++tt)
      if (tt < count) qa[(static_cast<size_t>(t0 + tt) * heads + h) * (rank + rot) + r] = acc[tt] * scale;
  }
  if (blockIdx.z != 0) return;
  for (int i = threadIdx.x; i < count * (rot / 2); i += blockDim.x) {
    const int tt = i / (rot / 2), pair = i % (rot / 2);
    const int t = t0 + tt;
    const float* q_rot = proj + static_cast<size_t>(t) * proj_width + q_off + h * head_width + d;
    const int position = positions[t];
    const float c = cos_table[static_cast<size_t>(position) * (rot / 2) + pair];
    const float s = sin_table[static_cast<size_t>(position) * (rot / 2) + pair];
    int ia, ib;
    rot_pair(pairing, rot, pair, ia, ib);
    const float a = q_rot[ia], b = q_rot[ib];
    float* dst = qa + (static_cast<size_t>(t) * heads + h) * (rank + rot) + rank;
    dst[ia] = (a * c - b * s) * scale;
    dst[ib] = (b * c + a * s) * scale;
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
                        int page_size, int heads, int rank, int rot, int window) {
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
  for (int base = window > 0 ? max(0, position - window + 1) : 0; base <= position; base += 32) {
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
// The same fold on the tensor cores (bfloat16 caches; mma.sync m16n8k16, 32-bit accumulation).
// A block owns 16 query rows, a row being a (token, head): `tokens_per_tile` neighbouring tokens
// by `head_group` heads, all of one request (a tile that spans several requests is folded once per
// request, the other requests' rows masked).  Keys come 64 at a time as rows [c | kr] of shared
// memory, the next tile on its way (cp.async) while this one is used.  Per tile the eight warps
//   1. each score 8 keys against all 16 rows: S = Q K^T over rank + rot values;
//   2. each take two rows: running maximum, weights p = exp(s - m) rounded to bfloat16, their sum;
//   3. each add P C into their 1/8 of the latent's columns.
// With `num_splits` > 1 a block folds keys [split * split_keys, ...) only and leaves (m, sum,
// unnormalised columns); latent_combine_kernel joins the splits.  NR: the columns the block's
// accumulators cover (128, 256 or 512, at least the rank rounded up to 16).
// ---------------------------------------------------------------------------------------
constexpr int kFoldRows = 16;
constexpr int kFoldKeys = 64;
constexpr int kFoldThreads = 256;
constexpr int kScoreStride = kFoldKeys + 4;   // floats
constexpr int kWeightStride = kFoldKeys + 8;  // bf16

struct LatentFoldParams {
  const float* qa;                 // [tokens, heads, rank + rot]
  const __nv_bfloat16* k_pool;     // latents
  const __nv_bfloat16* v_pool;     // rotated key parts
  const int* token_entry;
  const int* positions;
  const int* block_table;
  float* out;                      // [tokens * heads, rank]
  float* part;                     // splits: [num_splits][tokens * heads][rank + 2]: columns, then m and sum
  int num_tokens, heads, rank, rot, table_width, page_size;
  int head_group, tokens_per_tile, split_keys, num_splits;
  int window;                      // > 0: a row at position p sees keys p - window + 1 .. p
  // Head-major form (the products on both sides of the fold run as grouped tensor-core products, a
  // head a group): the unrotated part of qa comes unscaled from qa_heads [heads, padded_tokens, rank]
  // and the rotated, scaled part from q_rot [tokens, heads, rot]; the folded latents leave as
  // bfloat16 rows of l_heads [heads, padded_tokens, rank].  Null: qa and out as above.
  const float* qa_heads;
  const float* q_rot;
  __nv_bfloat16* l_heads;
  int padded_tokens;
  float scale;
};

__host__ __device__ __forceinline__ int round_up(int v, int to) { return (v + to - 1) / to * to; }

template <int NR, int MT>
__global__ void __launch_bounds__(kFoldThreads)
latent_fold_kernel(LatentFoldParams p) {
  extern __shared__ __align__(16) unsigned char fold_shared[];
  const int rank_pad = round_up(p.rank, 16);
  const int width_pad = round_up(rank_pad + round_up(p.rot, 16), 32);
  const int stride = width_pad + 8;   // bf16 per row: rows 16 bytes apart modulo 128, so ldmatrix meets no bank twice
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(fold_shared);
  constexpr int kRows = kFoldRows * MT;   // MT groups of sixteen rows share every tile of keys
  __nv_bfloat16* k_s = q_s + kRows * stride;                       // two tiles of kFoldKeys rows
  float* s_s = reinterpret_cast<float*>(k_s + 2 * kFoldKeys * stride);
  __nv_bfloat16* p_s = reinterpret_cast<__nv_bfloat16*>(s_s + kRows * kScoreStride);
  float* m_s = reinterpret_cast<float*>(p_s + kRows * kWeightStride);
  float* l_s = m_s + kRows;
  float* alpha_s = l_s + kRows;
  int* limit_s = reinterpret_cast<int*>(alpha_s + kRows);
  int* row_s = limit_s + kRows;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    // everything the copies never write (the columns that pad rank and rot) must read as zero
    uint4* all = reinterpret_cast<uint4*>(fold_shared);
    const int vectors = (kRows + 2 * kFoldKeys) * stride * 2 / 16;
    for (int i = threadIdx.x; i < vectors; i += kFoldThreads) all[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = (gridDim.x - 1 - blockIdx.x) * p.tokens_per_tile;   // the longest histories of a prompt first
  const int head0 = blockIdx.y * p.head_group;
  const int split = blockIdx.z;
  const int width = p.rank + p.rot;
  const int rank_chunks = p.rank / 8, row_chunks = rank_chunks + p.rot / 8;
  const int total_rows = p.num_tokens * p.heads;
  unsigned done = 0;
  for (;;) {
    int lead = -1;
    for (int tq = 0; tq < p.tokens_per_tile; ++tq)
      if (t0 + tq < p.num_tokens && !((done >> tq) & 1u)) { lead = tq; break; }
    if (lead < 0) break;
    const int entry = p.token_entry[t0 + lead];
    int last_key = -1, first_key = 0x7fffffff;
    unsigned taken = 0;
    for (int tq = lead; tq < p.tokens_per_tile && t0 + tq < p.num_tokens; ++tq)
      if (!((done >> tq) & 1u) && p.token_entry[t0 + tq] == entry) {
        taken |= 1u << tq;
        last_key = max(last_key, p.positions[t0 + tq]);
        first_key = min(first_key, p.positions[t0 + tq]);
      }
    // the first key any of the pass's rows sees: nothing before it is read (its page may be gone)
    first_key = p.window > 0 ? max(0, first_key - p.window + 1) : 0;
    __syncthreads();   // the pass before is done with the rows' tables
    if (threadIdx.x < kRows) {
      const int r = threadIdx.x, tq = r / p.head_group, head = head0 + r % p.head_group;
      const bool valid = tq < p.tokens_per_tile && ((taken >> tq) & 1u) && head < p.heads;
      limit_s[r] = valid ? p.positions[t0 + tq] : -1;
      row_s[r] = valid ? (t0 + tq) * p.heads + head : -1;
      m_s[r] = -INFINITY;
      l_s[r] = 0.0f;
    }
    done |= taken;
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * width; i += kFoldThreads) {
      const int r = i / width, c = i % width;
      float v = 0.0f;
      if (row_s[r] >= 0) {
        if (p.qa_heads == nullptr) {
          v = p.qa[static_cast<size_t>(row_s[r]) * width + c];
        } else if (c < p.rank) {
          const int token = row_s[r] / p.heads, head = row_s[r] % p.heads;
          v = p.scale * p.qa_heads[(static_cast<size_t>(head) * p.padded_tokens + token) * p.rank + c];
        } else {
          v = p.q_rot[static_cast<size_t>(row_s[r]) * p.rot + c - p.rank];
        }
      }
      q_s[r * stride + (c < p.rank ? c : rank_pad + c - p.rank)] = __float2bfloat16(v);
    }
    // tiles are counted from the split's first key, whatever the window: the first tile that holds a
    // visible key is the first one folded
    const int split_begin = split * p.split_keys;
    const int begin = split_begin + max(0, first_key - split_begin) / kFoldKeys * kFoldKeys;
    const int end = min(last_key + 1, split_begin + p.split_keys);
    const int num_tiles = end > begin ? (end - begin + kFoldKeys - 1) / kFoldKeys : 0;
    const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;

    // A warp copies 8 keys of a tile: their page-table entries first (all lanes the same loads, in
    // flight together), then each row's 16-byte pieces, a lane taking every 32nd.
    auto copy_tile = [&](int tile) {
      __nv_bfloat16* dst_tile = k_s + (tile & 1) * kFoldKeys * stride;
      const int key0 = begin + tile * kFoldKeys + warp * 8;
      size_t slots[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int key = max(min(key0 + i, end - 1), first_key);
        slots[i] = static_cast<size_t>(table[key / p.page_size]) * p.page_size + key % p.page_size;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const bool valid = key0 + i < end && key0 + i >= first_key;
        const __nv_bfloat16* c_row = p.k_pool + slots[i] * p.rank;
        const __nv_bfloat16* r_row = p.v_pool + slots[i] * p.rot;
        __nv_bfloat16* dst = dst_tile + (warp * 8 + i) * stride;
        for (int chunk = lane; chunk < row_chunks; chunk += 32) {
          const bool latent = chunk < rank_chunks;
          cp_async_16(smem_addr(dst + (latent ? chunk * 8 : rank_pad + (chunk - rank_chunks) * 8)),
                      latent ? c_row + chunk * 8 : r_row + (chunk - rank_chunks) * 8, valid);
        }
      }
      cp_async_commit();
    };

    constexpr int kPairs = NR / 8 / 16;   // pairs of 8-column tiles a warp accumulates
    float acc[MT][2 * kPairs][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 2 * kPairs; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][j][e] = 0.0f;
    const int column0 = warp * (NR / 8);
    const int g = lane >> 2, pair = (lane & 3) * 2;
    if (num_tiles > 0) copy_tile(0);
    for (int tile = 0; tile < num_tiles; ++tile) {
      cp_async_wait<0>();
      __syncthreads();   // this tile has landed (and the queries, before the first); the tile before is read out
      if (tile + 1 < num_tiles) copy_tile(tile + 1);
      const __nv_bfloat16* keys = k_s + (tile & 1) * kFoldKeys * stride;
      const int key0 = begin + tile * kFoldKeys;
      {
        float c[MT][4], c_odd[MT][4];   // two chains of products per group of rows
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[mt][e] = c_odd[mt][e] = 0.0f;
        const uint32_t k_addr = smem_addr(keys + (warp * 8 + (lane & 7)) * stride + (lane >> 3) * 8);
        const uint32_t q_addr = smem_addr(q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * stride + (lane >> 4) * 8);
#pragma unroll 2
        for (int k0 = 0; k0 < width_pad; k0 += 32) {
          uint32_t b[4];
          ldmatrix_x4(b, k_addr + k0 * 2);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            uint32_t a[4], a_odd[4];
            ldmatrix_x4(a, q_addr + (mt * kFoldRows * stride + k0) * 2);
            ldmatrix_x4(a_odd, q_addr + (mt * kFoldRows * stride + k0 + 16) * 2);
            mma_16816(c[mt], a, b[0], b[1]);
            mma_16816(c_odd[mt], a_odd, b[2], b[3]);
          }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int row = mt * kFoldRows + g + (e >> 1) * 8, col = warp * 8 + pair + (e & 1);
            const int key = key0 + col;
            const bool seen = key <= limit_s[row] && key < end && (p.window <= 0 || key > limit_s[row] - p.window);
            s_s[row * kScoreStride + col] = seen ? c[mt][e] + c_odd[mt][e] : -INFINITY;
          }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 2 * MT; ++i) {
        const int row = warp * 2 * MT + i;
        const float v0 = s_s[row * kScoreStride + lane], v1 = s_s[row * kScoreStride + lane + 32];
        const float before = m_s[row];
        const float top = fmaxf(before, warp_max(fmaxf(v0, v1)));
        float alpha = 1.0f, w0 = 0.0f, w1 = 0.0f;
        if (top > -INFINITY) {
          alpha = expf(before - top);   // 0 while nothing was seen
          w0 = __bfloat162float(__float2bfloat16(expf(v0 - top)));
          w1 = __bfloat162float(__float2bfloat16(expf(v1 - top)));
        }
        p_s[row * kWeightStride + lane] = __float2bfloat16(w0);
        p_s[row * kWeightStride + lane + 32] = __float2bfloat16(w1);
        const float sum = warp_sum(w0 + w1);
        if (lane == 0) {
          m_s[row] = top;
          l_s[row] = l_s[row] * alpha + sum;
          alpha_s[row] = alpha;
        }
      }
      __syncthreads();
      {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const float alpha0 = alpha_s[mt * kFoldRows + g], alpha1 = alpha_s[mt * kFoldRows + g + 8];
#pragma unroll
          for (int j = 0; j < 2 * kPairs; ++j) {
            acc[mt][j][0] *= alpha0, acc[mt][j][1] *= alpha0;
            acc[mt][j][2] *= alpha1, acc[mt][j][3] *= alpha1;
          }
        }
        const uint32_t p_addr = smem_addr(p_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * kWeightStride + (lane >> 4) * 8);
        const uint32_t c_addr = smem_addr(keys + ((lane & 7) + ((lane >> 3) & 1) * 8) * stride + column0 + (lane >> 4) * 8);
#pragma unroll
        for (int kk = 0; kk < kFoldKeys / 16; ++kk) {
          uint32_t a[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(a[mt], p_addr + (mt * kFoldRows * kWeightStride + kk * 16) * 2);
#pragma unroll
          for (int j = 0; j < kPairs; ++j) {
            if (column0 + 16 * j < rank_pad) {
              uint32_t b[4];
              ldmatrix_x4_trans(b, c_addr + (kk * 16 * stride + 16 * j) * 2);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                mma_16816(acc[mt][2 * j], a[mt], b[0], b[1]);
                mma_16816(acc[mt][2 * j + 1], a[mt], b[2], b[3]);
              }
            }
          }
        }
      }
    }
    __syncthreads();   // the last sums are written
#pragma unroll
    for (int part_row = 0; part_row < 2 * MT; ++part_row) {
      const int mt = part_row >> 1, half = part_row & 1;
      const int row = mt * kFoldRows + g + half * 8;
      const int out_row = row_s[row];
      if (out_row < 0) continue;
      const float total = l_s[row];
      if (p.num_splits == 1 && p.l_heads != nullptr) {
        const float inverse = 1.0f / total;
        __nv_bfloat16* l_row = p.l_heads + (static_cast<size_t>(out_row % p.heads) * p.padded_tokens + out_row / p.heads) * p.rank;
#pragma unroll
        for (int j = 0; j < 2 * kPairs; ++j) {
          const int col = column0 + 8 * j + pair;   // (even, and the rank is a multiple of 8)
          if (col < p.rank)
            *reinterpret_cast<uint32_t*>(l_row + col) = pack_bf16(acc[mt][j][2 * half] * inverse, acc[mt][j][2 * half + 1] * inverse);
        }
      } else if (p.num_splits == 1) {
        const float inverse = 1.0f / total;
#pragma unroll
        for (int j = 0; j < 2 * kPairs; ++j) {
          const int col = column0 + 8 * j + pair;
          if (col < p.rank) p.out[static_cast<size_t>(out_row) * p.rank + col] = acc[mt][j][2 * half] * inverse;
          if (col + 1 < p.rank) p.out[static_cast<size_t>(out_row) * p.rank + col + 1] = acc[mt][j][2 * half + 1] * inverse;
        }
      } else {
        float* part = p.part + (static_cast<size_t>(split) * total_rows + out_row) * (p.rank + 2);
#pragma unroll
        for (int j = 0; j < 2 * kPairs; ++j) {
          const int col = column0 + 8 * j + pair;
          if (col < p.rank) part[col] = acc[mt][j][2 * half];
          if (col + 1 < p.rank) part[col + 1] = acc[mt][j][2 * half + 1];
        }
        if (warp == 0 && pair == 0) {
          part[p.rank] = m_s[row];
          part[p.rank + 1] = total;
        }
      }
    }
  }
}

// out[row, :] = sum_s e^(m_s - m) columns_s / sum_s e^(m_s - m) sum_s over the splits that saw a key.
// The splits' maxima and sums are read side by side (a thread a split), the weights e^(m_s - m) / total
// kept in shared memory, and a column's terms asked for four splits at a time, added in the splits' order.
constexpr int kMostSplits = 64;

__global__ void __launch_bounds__(128)
latent_combine_kernel(LatentFoldParams p) {
  __shared__ float top_s[kMostSplits], sum_s[kMostSplits], weight_s[kMostSplits];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const size_t rows = static_cast<size_t>(p.num_tokens) * p.heads, each = p.rank + 2;
  const float* first = p.part + static_cast<size_t>(row) * each;
  if (threadIdx.x < p.num_splits) {
    const float* part = first + threadIdx.x * rows * each;
    top_s[threadIdx.x] = part[p.rank];
    sum_s[threadIdx.x] = part[p.rank + 1];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float top = -INFINITY, total = 0.0f;
    for (int s = 0; s < p.num_splits; ++s)
      if (sum_s[s] > 0.0f) top = fmaxf(top, top_s[s]);
    for (int s = 0; s < p.num_splits; ++s) {
      weight_s[s] = sum_s[s] > 0.0f ? expf(top_s[s] - top) : 0.0f;
      total += sum_s[s] * weight_s[s];
    }
    const float inverse = 1.0f / total;
    for (int s = 0; s < p.num_splits; ++s) weight_s[s] *= inverse;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < p.rank; c += blockDim.x) {
    float sum = 0.0f;
    int s = 0;
    for (; s + 4 <= p.num_splits; s += 4) {
      const float v0 = first[(s * rows) * each + c], v1 = first[((s + 1) * rows) * each + c];
      const float v2 = first[((s + 2) * rows) * each + c], v3 = first[((s + 3) * rows) * each + c];
      sum = fmaf(v0, weight_s[s], sum);
      sum = fmaf(v1, weight_s[s + 1], sum);
      sum = fmaf(v2, weight_s[s + 2], sum);
      sum = fmaf(v3, weight_s[s + 3], sum);
    }
    for (; s < p.num_splits; ++s) sum = fmaf(first[(s * rows) * each + c], weight_s[s], sum);
    if (p.l_heads != nullptr)
      p.l_heads[(static_cast<size_t>(row % p.heads) * p.padded_tokens + row / p.heads) * p.rank + c] = __float2bfloat16(sum);
    else
      p.out[static_cast<size_t>(row) * p.rank + c] = sum;
  }
}

// ---------------------------------------------------------------------------------------
// Head-major form, in front of the fold: a block per token puts each head's unrotated q values
// (bfloat16) at row [head, token] of a_heads [heads, padded_tokens, d], the operand of the grouped
// product with U_h^T, and the rotated, scaled rest at q_rot [token, head, rot].  The first block
// also fills the table that gives every tile of 128 rows its head.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* __restrict__ proj, long long proj_width, int q_off, const int* __restrict__ positions,
                   const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                   __nv_bfloat16* __restrict__ a_heads, float* __restrict__ q_rot, int* __restrict__ tile_group,
                   int heads, int d, int rot, int padded_tokens, float scale, int pairing) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (t == 0)
    for (int i = threadIdx.x; i < heads * (padded_tokens / 128); i += blockDim.x) tile_group[i] = i / (padded_tokens / 128);
  const float* row = proj + static_cast<size_t>(t) * proj_width + q_off;
  for (int i = threadIdx.x; i < heads * d; i += blockDim.x) {
    const int h = i / d, e = i % d;
    a_heads[(static_cast<size_t>(h) * padded_tokens + t) * d + e] = __float2bfloat16(row[h * (d + rot) + e]);
  }
  const int position = positions[t];
  const float* cs = cos_table + static_cast<size_t>(position) * (rot / 2);
  const float* sn = sin_table + static_cast<size_t>(position) * (rot / 2);
  for (int i = threadIdx.x; i < heads * (rot / 2); i += blockDim.x) {
    const int h = i / (rot / 2), pair = i % (rot / 2);
    int ia, ib;
    rot_pair(pairing, rot, pair, ia, ib);
    const float a = row[h * (d + rot) + d + ia], b = row[h * (d + rot) + d + ib];
    float* dst = q_rot + (static_cast<size_t>(t) * heads + h) * rot;
    dst[ia] = (a * cs[pair] - b * sn[pair]) * scale;
    dst[ib] = (b * cs[pair] + a * sn[pair]) * scale;
  }
}

// Head-major form, behind the second product: out[t, h * dv + v] = o_heads[h, t, v] * sigmoid(gate).
template <typename TO>
__global__ void __launch_bounds__(256)
latent_gate_kernel(const float* __restrict__ o_heads, const float* __restrict__ proj, long long proj_width, int g_off,
                   TO* __restrict__ out, int num_tokens, int heads, int dv, int padded_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(num_tokens) * heads * dv) return;
  const long long t = i / (heads * dv);
  const int c = static_cast<int>(i % (heads * dv)), h = c / dv, v = c % dv;
  float y = o_heads[(static_cast<size_t>(h) * padded_tokens + t) * dv + v];
  if (g_off >= 0) y *= 1.0f / (1.0f + expf(-proj[t * proj_width + g_off + c]));
  out[i] = from_float<TO>(y);
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
  // A block: kTile tokens of one head, 32 values; its four warps share the rank between them and
  // add their parts in the warps' order.
  extern __shared__ float expand_shared[];
  float* l_tile = expand_shared;                 // [kTile][rank]
  float* partial = expand_shared + kTile * rank; // [4][kTile][32]
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * kTile, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int v = blockIdx.z * 32 + lane;
  const int count = min(kTile, num_tokens - t0);
  for (int i = threadIdx.x; i < kTile * rank; i += blockDim.x) {
    const int tt = i / rank, r = i % rank;
    l_tile[i] = tt < count ? latent_out[(static_cast<size_t>(t0 + tt) * heads + h) * rank + r] : 0.0f;
  }
  __syncthreads();
  const TW* w = up_v + static_cast<size_t>(h) * rank * dv;
  const int share = (rank + 3) / 4;
  const int r_end = min(rank, (warp + 1) * share);
  float acc[kTile];
#pragma unroll
  for (int tt = 0; tt < kTile; ++tt) acc[tt] = 0.0f;
  if (v < dv) {
#pragma unroll 8
    for (int r = warp * share; r < r_end; ++r) {
      const float x = to_float<TW>(w[static_cast<size_t>(r) * dv + v]);
#pragma unroll
      for (int tt = 0; tt < kTile; ++tt) acc[tt] = fmaf(l_tile[tt * rank + r], x, acc[tt]);
    }
  }
#pragma unroll
  for (int tt = 0; tt < kTile; ++tt) partial[(warp * kTile + tt) * 32 + lane] = acc[tt];
  __syncthreads();
  for (int i = threadIdx.x; i < kTile * 32; i += blockDim.x) {
    const int tt = i / 32, column = blockIdx.z * 32 + i % 32;
    if (tt >= count || column >= dv) continue;
    float y = partial[i];
#pragma unroll
    for (int part = 1; part < 4; ++part) y += partial[part * kTile * 32 + i];
    const size_t t = t0 + tt;
    if (g_off >= 0) y *= 1.0f / (1.0f + expf(-proj[t * proj_width + g_off + h * dv + column]));
    out[(t * heads + h) * dv + column] = from_float<TO>(y);
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
  float* part;             // scratch of the tensor-core fold's splits: [num_splits][tokens * heads][rank + 2], or null
  int split_keys, num_splits;   // as vipera_latent_plan gives them (1 split: the whole history in one block)
  // Head-major form (bfloat16): the caller runs the grouped products between the stages.
  //   stage 1: cache write, a_heads, q_rot, tile_group;  [qa_heads = a_heads x U_h^T]
  //   stage 2: the fold, leaving l_heads;                [o_heads = l_heads x V_h^T]
  //   stage 3: the gate and the output.    stage 0: everything in one call, without these buffers.
  int stage, padded_tokens;
  void* a_heads;           // [heads, padded_tokens, d]
  float* qa_heads;         // [heads, padded_tokens, rank]
  float* q_rot;            // [tokens, heads, rot]
  void* l_heads;           // [heads, padded_tokens, rank]
  float* o_heads;          // [heads, padded_tokens, dv]
  int* tile_group;         // [heads * padded_tokens / 128]
  int window;              // > 0: a query at position p sees keys p - window + 1 .. p
  int pairing;             // of the rotated part: 0 values (2i, 2i + 1), 1 values (i, i + rot/2)
};

// How the tensor-core fold cuts a step: {tokens per tile, heads per tile, keys per split, splits}.
// Few blocks (decode) are cut along the keys, in whole tiles of 64, until the device has some
// four blocks per SM.
// Groups of sixteen rows a block takes: two where single groups would still fill the device twice.
static int fold_groups(int tokens, int heads, int sms) {
  const int head_group = heads < kFoldRows ? heads : kFoldRows;
  const int per_tile = kFoldRows / head_group;
  const long base = static_cast<long>((tokens + per_tile - 1) / per_tile) * ((heads + head_group - 1) / head_group);
  return base >= 2L * sms && heads <= kFoldRows ? 2 : 1;
}

static void latent_plan(int tokens, int heads, int max_keys, int sms, int* plan) {
  const int head_group = heads < kFoldRows ? heads : kFoldRows;
  const int per_tile = kFoldRows * fold_groups(tokens, heads, sms) / head_group;
  const long base = static_cast<long>((tokens + per_tile - 1) / per_tile) * ((heads + head_group - 1) / head_group);
  int bound = kFoldKeys;
  while (bound < max_keys) bound *= 2;
  long want = (4L * sms) / base;
  if (want > bound / kFoldKeys) want = bound / kFoldKeys;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  int chunk = static_cast<int>((bound + want - 1) / want);
  chunk = (chunk + kFoldKeys - 1) / kFoldKeys * kFoldKeys;
  plan[0] = per_tile;
  plan[1] = head_group;
  plan[2] = chunk;
  plan[3] = (bound + chunk - 1) / chunk;
}

VIPERA_API int vipera_latent_plan(int tokens, int heads, int max_keys, int sms, int* plan) {
  if (tokens <= 0 || heads <= 0 || sms <= 0) return VIPERA_BAD_ARGUMENT;
  latent_plan(tokens, heads, max_keys < 1 ? 1 : max_keys, sms, plan);
  return VIPERA_OK;
}

template <int NR, int MT>
static int launch_fold(const LatentFoldParams& f, dim3 grid, size_t shared, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(latent_fold_kernel<NR, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024) != cudaSuccess)
      return VIPERA_BAD_ARGUMENT;
    configured = true;
  }
  return vipera_launch(latent_fold_kernel<NR, MT>, grid, kFoldThreads, shared, s, f);
}

static int launch_fold_any(const LatentParams& p, cudaStream_t s) {
  LatentFoldParams f{};
  f.qa = p.qa;
  f.k_pool = static_cast<const __nv_bfloat16*>(p.k_pool);
  f.v_pool = static_cast<const __nv_bfloat16*>(p.v_pool);
  f.token_entry = p.token_entry;
  f.positions = p.positions;
  f.block_table = p.block_table;
  f.out = p.latent_out;
  f.part = p.part;
  f.num_tokens = p.num_tokens, f.heads = p.heads, f.rank = p.rank, f.rot = p.rot;
  f.table_width = p.table_width, f.page_size = p.page_size;
  f.window = p.window;
  if (p.stage == 2) {
    f.qa_heads = p.qa_heads, f.q_rot = p.q_rot, f.l_heads = static_cast<__nv_bfloat16*>(p.l_heads);
    f.padded_tokens = p.padded_tokens, f.scale = p.scale;
  }
  int device = 0, sms = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int groups = fold_groups(p.num_tokens, p.heads, sms > 0 ? sms : 148);
  f.head_group = p.heads < kFoldRows ? p.heads : kFoldRows;
  f.tokens_per_tile = kFoldRows * groups / f.head_group;
  f.num_splits = p.num_splits > 1 && p.part ? p.num_splits : 1;
  f.split_keys = f.num_splits > 1 ? p.split_keys : 0x3fffffff;
  if (f.num_splits > kMostSplits) return VIPERA_BAD_ARGUMENT;
  const int rank_pad = round_up(p.rank, 16);
  const int stride = round_up(rank_pad + round_up(p.rot, 16), 32) + 8;
  const int rows = kFoldRows * groups;
  const size_t shared = static_cast<size_t>(rows + 2 * kFoldKeys) * stride * 2 + rows * kScoreStride * 4 +
                        rows * kWeightStride * 2 + rows * 5 * 4;
  const dim3 grid((p.num_tokens + f.tokens_per_tile - 1) / f.tokens_per_tile, (p.heads + f.head_group - 1) / f.head_group,
                  f.num_splits);
  int status;
  if (groups == 2)
    status = rank_pad <= 128 ? launch_fold<128, 2>(f, grid, shared, s)
           : rank_pad <= 256 ? launch_fold<256, 2>(f, grid, shared, s) : launch_fold<512, 2>(f, grid, shared, s);
  else
    status = rank_pad <= 128 ? launch_fold<128, 1>(f, grid, shared, s)
           : rank_pad <= 256 ? launch_fold<256, 1>(f, grid, shared, s) : launch_fold<512, 1>(f, grid, shared, s);
  if (status || f.num_splits == 1) return status;
  return vipera_launch(latent_combine_kernel, p.num_tokens * p.heads, 128, 0, s, f);
}

template <typename T>
static int launch_latent(const LatentParams& p, cudaStream_t s) {
  int status = VIPERA_OK;
  if (p.stage == 2) return launch_fold_any(p, s);
  if (p.stage == 3) {
    const long long values = static_cast<long long>(p.num_tokens) * p.heads * p.dv;
    return vipera_launch(latent_gate_kernel<T>, static_cast<unsigned>((values + 255) / 256), 256, 0, s, p.o_heads, p.proj,
                         p.proj_width, p.g_off, static_cast<T*>(p.out), p.num_tokens, p.heads, p.dv, p.padded_tokens);
  }
  if (p.kv_off >= 0) {
    status = vipera_launch(latent_store_kernel<T>, p.num_tokens, 128, 0, s, p.proj, p.proj_width, p.kv_off, p.norm_weight,
                           p.eps, p.positions, p.cos_table, p.sin_table, static_cast<T*>(p.k_pool),
                           static_cast<T*>(p.v_pool), p.token_entry, p.block_table, p.table_width, p.page_size, p.rank,
                           p.rot, p.pairing);
    if (status) return status;
  }
  if (p.stage == 1)
    return vipera_launch(latent_prep_kernel, p.num_tokens, 128, 0, s, p.proj, p.proj_width, p.q_off, p.positions, p.cos_table,
                         p.sin_table, static_cast<__nv_bfloat16*>(p.a_heads), p.q_rot, p.tile_group, p.heads, p.d, p.rot,
                         p.padded_tokens, p.scale, p.pairing);
  const dim3 tiles((p.num_tokens + kTile - 1) / kTile, p.heads);
  const dim3 absorb_grid(tiles.x, tiles.y, (p.rank + 127) / 128);
  status = vipera_launch(latent_absorb_kernel<T>, absorb_grid, 128, kTile * p.d * sizeof(float), s, p.proj, p.proj_width, p.q_off,
                         static_cast<const T*>(p.up_k), p.positions, p.cos_table, p.sin_table, p.qa, p.num_tokens,
                         p.heads, p.d, p.rank, p.rot, p.scale, p.pairing);
  if (status) return status;
  // bfloat16 caches whose rows are whole 16-byte pieces fold on the tensor cores
  if (sizeof(T) == 2 && p.rank % 8 == 0 && p.rot % 8 == 0 && p.num_tokens < (1 << 24) / p.heads &&
      (p.num_splits <= 1 || p.split_keys % kFoldKeys == 0))
    status = launch_fold_any(p, s);
  else
    status = vipera_launch(latent_attention_kernel<T>, dim3(p.num_tokens, (p.heads + kWarps - 1) / kWarps), kWarps * 32,
                           kWarps * (p.rank + p.rot) * sizeof(float), s, p.qa, p.latent_out,
                           static_cast<const T*>(p.k_pool), static_cast<const T*>(p.v_pool), p.token_entry, p.positions,
                           p.block_table, p.table_width, p.page_size, p.heads, p.rank, p.rot, p.window);
  if (status) return status;
  const dim3 expand_grid(tiles.x, tiles.y, (p.dv + 31) / 32);
  return vipera_launch(latent_expand_kernel<T, T>, expand_grid, 128, (kTile * p.rank + 4 * kTile * 32) * sizeof(float), s, p.latent_out,
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
  if (p.stage < 0 || p.stage > 3 || p.window < 0 || p.pairing < 0 || p.pairing > 1) return VIPERA_BAD_ARGUMENT;
  if (p.stage != 0) {
    if (dtype != VIPERA_BF16 || p.rank % 8 || p.rot % 8 || p.d % 8 || p.padded_tokens < p.num_tokens || p.padded_tokens % 128 ||
        !p.a_heads || !p.qa_heads || !p.q_rot || !p.l_heads || !p.o_heads || !p.tile_group ||
        p.num_tokens >= (1 << 24) / p.heads || (p.num_splits > 1 && p.split_keys % kFoldKeys))
      return VIPERA_BAD_ARGUMENT;
  }
  if (dtype == VIPERA_F32) return launch_latent<float>(p, s);
  if (dtype == VIPERA_BF16) return launch_latent<__nv_bfloat16>(p, s);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API int vipera_latent_params_size() { return static_cast<int>(sizeof(LatentParams)); }
VIPERA_API const char* vipera_latent_status_text(int status) { return vipera_status_text(status); }
