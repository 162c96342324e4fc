// RMS norm over equal consecutive groups of a row, and the ending of a sublayer whose output is
// gated, normed, scaled and added into the 32-bit residual stream.
//
// group_rmsnorm:   out[r, g, :] = x[rows[r], g, :] / sqrt(mean(x[rows[r], g, :]^2) + eps) * w[g, :]
// gated_norm_add:  y = (sum_p branch[r, p, :]) * sigmoid(gate[r, :])         (gate optional)
//                  residual[r, g, :] += coef[g, :] * y[g, :] / sqrt(mean(y[g, :]^2) + eps)
// `coef` holds everything that multiplies the normed value per channel (norm weight, a scale per
// channel, the layer's multiplier).  All statistics are 32-bit; the order of every sum is fixed by
// the row's width alone, so a row's result does not depend on what else the step holds.
#include "common.cuh"

constexpr int kGroupThreads = 256;
constexpr int kKeep = 32;   // values of a group a lane keeps in registers between its two passes (groups up to 1,024 values)

// One block per output row.  A thread reads the same elements in both passes and writes them only in
// the second, so `out` may be `x` itself (32-bit, rows == nullptr).
template <typename TO>
__global__ void __launch_bounds__(kGroupThreads)
group_rmsnorm_kernel(const float* x, const float* __restrict__ weight, const int* __restrict__ rows,
                     TO* out, int hidden, int groups, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src_row = rows ? rows[r] : r;
  const float* src = x + static_cast<size_t>(src_row) * hidden;
  TO* dst = out + static_cast<size_t>(r) * hidden;
  const int part = hidden / groups;
  for (int g = 0; g < groups; ++g) {
    const float* p = src + g * part;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < part; i += kGroupThreads) sum += p[i] * p[i];
    const float total = block_sum(sum, scratch);
    const float inverse = 1.0f / sqrtf(total / static_cast<float>(part) + eps);
    for (int i = threadIdx.x; i < part; i += kGroupThreads)
      dst[g * part + i] = from_float<TO>(p[i] * inverse * weight[g * part + i]);
  }
}

// Many rows: a warp per (row, group), eight to a block; sums by shuffles.
template <typename TO>
__global__ void __launch_bounds__(kGroupThreads)
group_rmsnorm_rows_kernel(const float* x, const float* __restrict__ weight, const int* __restrict__ rows,
                          TO* out, int num_rows, int hidden, int groups, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int job = blockIdx.x * (kGroupThreads / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (job >= num_rows * groups) return;
  const int r = job / groups, g = job % groups;
  const int part = hidden / groups;
  const int src_row = rows ? rows[r] : r;
  const float* p = x + static_cast<size_t>(src_row) * hidden + g * part;
  const float* w = weight + g * part;
  TO* dst = out + static_cast<size_t>(r) * hidden + g * part;
  float sum = 0.0f;
  if (part <= 32 * kKeep) {
    // the lane's values stay in registers between the passes: no load waits behind a store
    float kept[kKeep];
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
      const int i = lane + 32 * j;
      kept[j] = i < part ? p[i] : 0.0f;
      sum += kept[j] * kept[j];
    }
    const float inverse = 1.0f / sqrtf(warp_sum(sum) / static_cast<float>(part) + eps);
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
      const int i = lane + 32 * j;
      if (i < part) dst[i] = from_float<TO>(kept[j] * inverse * w[i]);
    }
    return;
  }
#pragma unroll 4
  for (int i = lane; i < part; i += 32) sum += p[i] * p[i];
  const float inverse = 1.0f / sqrtf(warp_sum(sum) / static_cast<float>(part) + eps);
#pragma unroll 4
  for (int i = lane; i < part; i += 32) dst[i] = from_float<TO>(p[i] * inverse * w[i]);
}

VIPERA_API int vipera_group_rmsnorm(const float* x, const float* weight, const int* rows, void* out, int out_dtype,
                                    int num_rows, int hidden, int groups, float eps, void* stream) {
  if (num_rows <= 0) return VIPERA_OK;
  if (hidden <= 0 || groups <= 0 || hidden % groups) return VIPERA_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // (a warp per (row, group) for steps of every size: a row's sums then run in one order whatever the step holds)
  const bool many = hidden / groups <= 4096;
  const int warps = kGroupThreads / 32;
  if (out_dtype == VIPERA_F32) {
    if (many)
      return vipera_launch(group_rmsnorm_rows_kernel<float>, (num_rows * groups + warps - 1) / warps, kGroupThreads, 0, s,
                           x, weight, rows, static_cast<float*>(out), num_rows, hidden, groups, eps);
    return vipera_launch(group_rmsnorm_kernel<float>, num_rows, kGroupThreads, 0, s, x, weight, rows,
                         static_cast<float*>(out), hidden, groups, eps);
  }
  if (out_dtype == VIPERA_BF16) {
    if (many)
      return vipera_launch(group_rmsnorm_rows_kernel<__nv_bfloat16>, (num_rows * groups + warps - 1) / warps,
                           kGroupThreads, 0, s, x, weight, rows, static_cast<__nv_bfloat16*>(out), num_rows, hidden,
                           groups, eps);
    return vipera_launch(group_rmsnorm_kernel<__nv_bfloat16>, num_rows, kGroupThreads, 0, s, x, weight, rows,
                         static_cast<__nv_bfloat16*>(out), hidden, groups, eps);
  }
  return VIPERA_BAD_DTYPE;
}

// A warp per (row, group).  KEEP > 0: a lane keeps its KEEP values (a group of up to 32 KEEP values) in
// registers, and every pass over them is straight-line code with clamped indices, so that all its
// loads are in flight together (a lane's loads one behind the other took 60,000 cycles for 8 rows).
// KEEP == 0 (wider groups): the gated sum is parked in the first addend's place between the two
// passes (each lane reads back only what it wrote).  Either way a group's sums run in one order.
template <int KEEP>
__global__ void __launch_bounds__(kGroupThreads)
gated_norm_add_kernel(float* __restrict__ branch, int parts, const float* __restrict__ gate,
                      const float* __restrict__ coef, float* __restrict__ residual, int num_rows, int hidden,
                      int groups, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int job = blockIdx.x * (kGroupThreads / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (job >= num_rows * groups) return;
  const int r = job / groups, g = job % groups;
  const int part = hidden / groups;
  float* b = branch + static_cast<size_t>(r) * parts * hidden + g * part;
  const float* gt = gate ? gate + static_cast<size_t>(r) * hidden + g * part : nullptr;
  float* dst = residual + static_cast<size_t>(r) * hidden + g * part;
  const float* c = coef + g * part;
  float sum = 0.0f;
  if (KEEP > 0) {
    constexpr int kSlots = KEEP > 0 ? KEEP : 1;
    float y[kSlots], other[kSlots];
#pragma unroll
    for (int j = 0; j < kSlots; ++j) y[j] = b[min(lane + 32 * j, part - 1)];
    for (int p = 1; p < parts; ++p) {
      const float* more = b + static_cast<size_t>(p) * hidden;
#pragma unroll
      for (int j = 0; j < kSlots; ++j) other[j] = more[min(lane + 32 * j, part - 1)];
#pragma unroll
      for (int j = 0; j < kSlots; ++j) y[j] += other[j];
    }
    if (gt) {
#pragma unroll
      for (int j = 0; j < kSlots; ++j) other[j] = gt[min(lane + 32 * j, part - 1)];
#pragma unroll
      for (int j = 0; j < kSlots; ++j) y[j] *= 1.0f / (1.0f + expf(-other[j]));
    }
#pragma unroll
    for (int j = 0; j < kSlots; ++j) {
      if (lane + 32 * j >= part) y[j] = 0.0f;
      sum += y[j] * y[j];
    }
    const float inverse = 1.0f / sqrtf(warp_sum(sum) / static_cast<float>(part) + eps);
    float before[kSlots];
#pragma unroll
    for (int j = 0; j < kSlots; ++j) {
      other[j] = c[min(lane + 32 * j, part - 1)];
      before[j] = dst[min(lane + 32 * j, part - 1)];
    }
#pragma unroll
    for (int j = 0; j < kSlots; ++j)
      if (lane + 32 * j < part) dst[lane + 32 * j] = before[j] + other[j] * (y[j] * inverse);
  } else {
    for (int i = lane; i < part; i += 32) {
      float y = b[i];
      for (int p = 1; p < parts; ++p) y += b[static_cast<size_t>(p) * hidden + i];
      if (gt) y *= 1.0f / (1.0f + expf(-gt[i]));
      b[i] = y;
      sum += y * y;
    }
    const float inverse = 1.0f / sqrtf(warp_sum(sum) / static_cast<float>(part) + eps);
    for (int i = lane; i < part; i += 32) dst[i] += c[i] * (b[i] * inverse);
  }
}

VIPERA_API int vipera_gated_norm_add(float* branch, int parts, const float* gate, const float* coef, float* residual,
                                     int num_rows, int hidden, int groups, float eps, void* stream) {
  if (num_rows <= 0) return VIPERA_OK;
  if (hidden <= 0 || groups <= 0 || hidden % groups || parts <= 0) return VIPERA_BAD_SHAPE;
  const int warps = kGroupThreads / 32;
  const int part = hidden / groups;
  auto kernel = part <= 128 ? gated_norm_add_kernel<4> : part <= 512 ? gated_norm_add_kernel<16>
              : part <= 1024 ? gated_norm_add_kernel<32> : gated_norm_add_kernel<0>;
  return vipera_launch(kernel, (num_rows * groups + warps - 1) / warps, kGroupThreads, 0,
                       static_cast<cudaStream_t>(stream), branch, parts, gate, coef, residual, num_rows, hidden, groups,
                       eps);
}

VIPERA_API const char* vipera_groupnorm_status_text(int status) { return vipera_status_text(status); }
