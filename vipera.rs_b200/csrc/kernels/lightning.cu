// Linear attention with one constant decay per head.
//
// Per head a matrix S [d, dv] of 32-bit floats, zero at a request's start.  With q, k, v the silu
// of their projections, for each token
//
//     S = lambda_h S + k v^T        o = S^T q
//
// and the concatenated heads' o is divided by its root mean square over the whole row, multiplied by a
// weight per value and by sigmoid(gate) (lightning_finish_kernel).
//
// A block owns 32 value columns of a head's state for one job; a lane a column, a warp a run of
// neighbouring rows (so that a thread reads its rows' k and q four at a time from shared memory),
// each thread's share of S in registers.  The operands of kStage
// tokens (silu applied) are staged in shared memory; the four warps' partial outputs are added in
// a fixed order.  Three kinds of job (own notation; a chunk is kChunk tokens of one entry, cut
// where the entry's tokens start in the step):
//   walk     a job is an entry: from the request's state (zero if fresh) over all its tokens,
//            with outputs, leaving the new state.  Steps of few tokens and of single tokens.
//   ends     a job is a chunk: from zero over the chunk, no outputs, leaving E_c = sum_s
//            lambda^(len - 1 - s) k_s v_s^T in the chunk's scratch row.
//   outputs  a job is a chunk: from the state at the chunk's start (the scratch row), with outputs.
// Between ends and outputs, lightning_carry_kernel walks each entry's chunks: start_c = S;
// S = lambda^len_c S + E_c; the request's new state is the last S.  Another cut of a prompt only
// re-associates 32-bit sums.
#include "common.cuh"

constexpr int kChunk = 64;
constexpr int kStage = 16;
constexpr int kColumns = 32;
constexpr int kRowWarps = 4;

enum LightningMode { MODE_WALK = 0, MODE_ENDS = 1, MODE_OUTPUTS = 2 };

struct LightningParams {
  const float* proj;        // [tokens, proj_width] 32-bit pre-activations of q, k, v and the gate
  long long proj_width;
  int q_off, k_off, v_off, g_off;
  const float* decay;       // [heads]
  float* state;             // [slots, heads * d * dv]
  const int* entry_starts;  // [entries + 1]
  const int* state_slots;   // [entries]
  const int* fresh;         // [entries]
  float* raw;               // [tokens, heads * dv] outputs before the norm
  const float* norm_weight; // [heads * dv]
  void* out;                // [tokens, heads * dv]
  float* chunk_state;       // [jobs, heads * d * dv] (chunked form only)
  int heads, d, dv, num_entries, num_tokens, num_jobs;
  float eps;
  int activated;            // 1: q, k and v in proj are past their silu already (the chunked form's first kernel)
};

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// The chunk a job index names: (entry, first token, one past the last), or entry -1 past the last chunk.
__device__ __forceinline__ void find_chunk(const int* __restrict__ entry_starts, int num_entries, int job, int* entry,
                                           int* begin, int* end) {
  int base = 0;
  *entry = -1;
  for (int e = 0; e < num_entries; ++e) {
    const int start = entry_starts[e], stop = entry_starts[e + 1];
    const int chunks = (stop - start + kChunk - 1) / kChunk;
    if (job < base + chunks) {
      *entry = e;
      *begin = start + (job - base) * kChunk;
      *end = min(*begin + kChunk, stop);
      return;
    }
    base += chunks;
  }
}

// The chunked form reads every token's q and k in each block of its head's columns, twice: the silu
// is applied once, in place (the gate's columns stay as they are).
__global__ void __launch_bounds__(256)
lightning_activate_kernel(LightningParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_token = p.heads * (2 * p.d + p.dv);
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(p.num_tokens) * per_token) return;
  const long long t = i / per_token;
  int c = static_cast<int>(i % per_token);
  int column;
  if (c < p.heads * p.d) column = p.q_off + c;
  else if ((c -= p.heads * p.d) < p.heads * p.d) column = p.k_off + c;
  else column = p.v_off + c - p.heads * p.d;
  float* at = const_cast<float*>(p.proj) + t * p.proj_width + column;
  *at = silu(*at);
}

template <int RPT, int MODE>
__global__ void __launch_bounds__(kRowWarps * 32)
lightning_scan_kernel(LightningParams p) {
  extern __shared__ __align__(16) float shared[];
  float* q_s = shared;                       // [kStage][d]
  float* k_s = q_s + kStage * p.d;           // [kStage][d]
  float* v_s = k_s + kStage * p.d;           // [kStage][kColumns]
  float* part = v_s + kStage * kColumns;     // [kStage][kRowWarps][kColumns]
  __shared__ int job_info[3];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, job = blockIdx.z;
  const int column = blockIdx.x * kColumns + lane;
  const bool live = column < p.dv;
  int entry, begin, end;
  if (MODE == MODE_WALK) {
    entry = job;
    begin = p.entry_starts[entry];
    end = p.entry_starts[entry + 1];
  } else {
    if (threadIdx.x == 0) find_chunk(p.entry_starts, p.num_entries, job, &job_info[0], &job_info[1], &job_info[2]);
    __syncthreads();
    entry = job_info[0], begin = job_info[1], end = job_info[2];
    if (entry < 0) return;
  }
  if (end <= begin) return;
  const float lambda = p.decay[h];
  const size_t state_size = static_cast<size_t>(p.heads) * p.d * p.dv;
  float* own = MODE == MODE_WALK ? p.state + static_cast<size_t>(p.state_slots[entry]) * state_size
                                 : p.chunk_state + static_cast<size_t>(job) * state_size;
  own += static_cast<size_t>(h) * p.d * p.dv;
  float s[RPT];
  const bool load = MODE == MODE_OUTPUTS || (MODE == MODE_WALK && !p.fresh[entry]);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int row = warp * RPT + i;
    s[i] = (load && live && row < p.d) ? own[static_cast<size_t>(row) * p.dv + column] : 0.0f;
  }
  for (int base = begin; base < end; base += kStage) {
    const int count = min(kStage, end - base);
    __syncthreads();
    for (int i = threadIdx.x; i < count * p.d; i += blockDim.x) {
      const int tt = i / p.d, e = i % p.d;
      const float* row = p.proj + static_cast<size_t>(base + tt) * p.proj_width;
      const float q_raw = MODE != MODE_ENDS ? row[p.q_off + h * p.d + e] : 0.0f, k_raw = row[p.k_off + h * p.d + e];
      if (MODE != MODE_ENDS) q_s[tt * p.d + e] = (MODE != MODE_WALK && p.activated) ? q_raw : silu(q_raw);
      k_s[tt * p.d + e] = (MODE != MODE_WALK && p.activated) ? k_raw : silu(k_raw);
    }
    for (int i = threadIdx.x; i < count * kColumns; i += blockDim.x) {
      const int tt = i / kColumns, c = blockIdx.x * kColumns + i % kColumns;
      const float v_raw = c < p.dv ? p.proj[static_cast<size_t>(base + tt) * p.proj_width + p.v_off + h * p.dv + c] : 0.0f;
      v_s[i] = (MODE != MODE_WALK && p.activated) ? v_raw : silu(v_raw);
    }
    __syncthreads();
    const bool whole_rows = (p.d & 3) == 0 && (warp + 1) * RPT <= p.d;   // this warp's rows all exist, in fours
    for (int tt = 0; tt < count; ++tt) {
      const float v = v_s[tt * kColumns + lane];
      float o = 0.0f;
      if (RPT % 4 == 0 && whole_rows) {
        const float4* k4 = reinterpret_cast<const float4*>(k_s + tt * p.d + warp * RPT);
        const float4* q4 = reinterpret_cast<const float4*>(q_s + tt * p.d + warp * RPT);
#pragma unroll
        for (int i = 0; i < RPT / 4; ++i) {
          const float4 kk = k4[i];
          s[4 * i] = fmaf(lambda, s[4 * i], kk.x * v);
          s[4 * i + 1] = fmaf(lambda, s[4 * i + 1], kk.y * v);
          s[4 * i + 2] = fmaf(lambda, s[4 * i + 2], kk.z * v);
          s[4 * i + 3] = fmaf(lambda, s[4 * i + 3], kk.w * v);
          if (MODE != MODE_ENDS) {
            const float4 qq = q4[i];
            o = fmaf(s[4 * i], qq.x, o);
            o = fmaf(s[4 * i + 1], qq.y, o);
            o = fmaf(s[4 * i + 2], qq.z, o);
            o = fmaf(s[4 * i + 3], qq.w, o);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int row = warp * RPT + i;
          if (row < p.d) {
            s[i] = fmaf(lambda, s[i], k_s[tt * p.d + row] * v);
            if (MODE != MODE_ENDS) o = fmaf(s[i], q_s[tt * p.d + row], o);
          }
        }
      }
      if (MODE != MODE_ENDS) part[(tt * kRowWarps + warp) * kColumns + lane] = o;
    }
    if (MODE != MODE_ENDS) {
      __syncthreads();
      for (int i = threadIdx.x; i < count * kColumns; i += blockDim.x) {
        const int tt = i / kColumns, l = i % kColumns, c = blockIdx.x * kColumns + l;
        if (c < p.dv) {
          const float* o = part + tt * kRowWarps * kColumns + l;
          p.raw[static_cast<size_t>(base + tt) * (p.heads * p.dv) + h * p.dv + c] =
              ((o[0] + o[kColumns]) + o[2 * kColumns]) + o[3 * kColumns];
        }
      }
    }
  }
  if (MODE != MODE_OUTPUTS && live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int row = warp * RPT + i;
      if (row < p.d) own[static_cast<size_t>(row) * p.dv + column] = s[i];
    }
  }
}

// One thread per element of a head's state and entry: the entry's chunks in a row.
__global__ void __launch_bounds__(256)
lightning_carry_kernel(LightningParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int entry = blockIdx.y;
  const size_t state_size = static_cast<size_t>(p.heads) * p.d * p.dv;
  const size_t element = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (element >= state_size) return;
  const int start = p.entry_starts[entry], stop = p.entry_starts[entry + 1];
  if (stop <= start) return;
  int job = 0;
  for (int e = 0; e < entry; ++e) job += (p.entry_starts[e + 1] - p.entry_starts[e] + kChunk - 1) / kChunk;
  const float lambda = p.decay[element / (static_cast<size_t>(p.d) * p.dv)];
  float* own = p.state + static_cast<size_t>(p.state_slots[entry]) * state_size + element;
  float s = p.fresh[entry] ? 0.0f : *own;
  float whole = 1.0f;   // lambda^kChunk by repeated multiplication, the same way the scan applies it
  for (int i = 0; i < kChunk; ++i) whole *= lambda;
  // eight chunks at a time: their endings are asked for together, then walked in order
  for (int begin = start; begin < stop; begin += 8 * kChunk, job += 8) {
    float ending[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
      ending[c] = begin + c * kChunk < stop ? p.chunk_state[static_cast<size_t>(job + c) * state_size + element] : 0.0f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int first = begin + c * kChunk;
      if (first >= stop) break;
      const int length = min(kChunk, stop - first);
      p.chunk_state[static_cast<size_t>(job + c) * state_size + element] = s;
      float power = whole;
      if (length < kChunk) {
        power = 1.0f;
        for (int i = 0; i < length; ++i) power *= lambda;
      }
      s = fmaf(power, s, ending[c]);
    }
  }
  *own = s;
}

// The norm over the concatenated heads, the norm's weight and the output gate; a block per token.
template <typename TO>
__global__ void __launch_bounds__(256)
lightning_finish_kernel(LightningParams p) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int width = p.heads * p.dv;
  const float* raw = p.raw + static_cast<size_t>(t) * width;
  const float* gate = p.proj + static_cast<size_t>(t) * p.proj_width + p.g_off;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sum += raw[i] * raw[i];
  const float inverse = 1.0f / sqrtf(block_sum(sum, scratch) / static_cast<float>(width) + p.eps);
  TO* out = static_cast<TO*>(p.out) + static_cast<size_t>(t) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[i] = from_float<TO>(raw[i] * inverse * p.norm_weight[i] * (1.0f / (1.0f + expf(-gate[i]))));
}

template <int RPT>
static int launch_scans(const LightningParams& params, bool chunked, cudaStream_t s) {
  LightningParams p = params;
  p.activated = 0;
  const size_t shared = (static_cast<size_t>(2 * kStage) * p.d + kStage * kColumns + kStage * kRowWarps * kColumns) * sizeof(float);
  const int tiles = (p.dv + kColumns - 1) / kColumns;
  if (!chunked)
    return vipera_launch(lightning_scan_kernel<RPT, MODE_WALK>, dim3(tiles, p.heads, p.num_entries), kRowWarps * 32, shared, s, p);
  p.activated = 1;
  const long long values = static_cast<long long>(p.num_tokens) * p.heads * (2 * p.d + p.dv);
  int status = vipera_launch(lightning_activate_kernel, static_cast<unsigned>((values + 255) / 256), 256, 0, s, p);
  if (status) return status;
  status = vipera_launch(lightning_scan_kernel<RPT, MODE_ENDS>, dim3(tiles, p.heads, p.num_jobs), kRowWarps * 32, shared, s, p);
  if (status) return status;
  const size_t state_size = static_cast<size_t>(p.heads) * p.d * p.dv;
  status = vipera_launch(lightning_carry_kernel, dim3(static_cast<unsigned>((state_size + 255) / 256), p.num_entries), 256, 0, s, p);
  if (status) return status;
  return vipera_launch(lightning_scan_kernel<RPT, MODE_OUTPUTS>, dim3(tiles, p.heads, p.num_jobs), kRowWarps * 32, shared, s, p);
}

// num_jobs > 0 (with chunk_state): the chunked form, num_jobs at least the step's count of chunks.
VIPERA_API int vipera_lightning(const LightningParams* params, int out_dtype, void* stream) {
  const LightningParams& p = *params;
  if (p.num_tokens <= 0 || p.num_entries <= 0) return VIPERA_OK;
  if (p.heads <= 0 || p.d <= 0 || p.d > 256 || p.dv <= 0 || p.heads > 65535 || p.num_entries > 65535) return VIPERA_BAD_SHAPE;
  const bool chunked = p.num_jobs > 0;
  if (chunked && (p.chunk_state == nullptr || p.num_jobs > 65535)) return VIPERA_BAD_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int status;
  if (p.d <= 32) status = launch_scans<8>(p, chunked, s);
  else if (p.d <= 64) status = launch_scans<16>(p, chunked, s);
  else if (p.d <= 128) status = launch_scans<32>(p, chunked, s);
  else status = launch_scans<64>(p, chunked, s);
  if (status) return status;
  if (out_dtype == VIPERA_F32) return vipera_launch(lightning_finish_kernel<float>, p.num_tokens, 256, 0, s, p);
  if (out_dtype == VIPERA_BF16) return vipera_launch(lightning_finish_kernel<__nv_bfloat16>, p.num_tokens, 256, 0, s, p);
  return VIPERA_BAD_DTYPE;
}

VIPERA_API int vipera_lightning_params_size() { return static_cast<int>(sizeof(LightningParams)); }
VIPERA_API int vipera_lightning_chunk() { return kChunk; }
VIPERA_API const char* vipera_lightning_status_text(int status) { return vipera_status_text(status); }
