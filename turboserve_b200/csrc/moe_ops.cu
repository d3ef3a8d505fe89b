// Mixture of experts: the router, and the experts' products for steps of few tokens and of many.
//
//   moe_route      per token: logits z = W_r h in fp32 (W_r is kept in fp32), s = softmax(z) over all experts,
//                  experts in `groups` equal groups of neighbours of which only the `keep` groups with the
//                  largest maximum may be chosen from, the `top` largest allowed scores, and their weights
//                  s / (sum of the chosen s + 1e-20).  Ties go to the lower index.
//   Few tokens (every request brings one): no sorting, every (token, chosen expert) pair streams its expert's rows
//     moe_pair_gate_up   hidden[pair, f] = act(gate_e[f] . h) * (up_e[f] . h), a warp per feature
//     moe_pair_down      out[t] = sum_k weight_k * (down_{e_k} hidden[t, k]) (+ addend[t]), a warp per output,
//                        the k-th expert's term added k-th, fp32, rounded once
//   Many tokens: the pairs are put in expert order so that every expert's rows are one matrix product
//     moe_count / moe_offsets / moe_place   how many pairs each expert has, where its rows start, and the
//                                           row of every pair (atomic counters: which row a pair gets within its
//                                           expert varies, what is computed for it does not)
//     moe_gather     rows of the input in that order
//     moe_combine    out[t] = sum_k weight_k * rows[place[t, k]] (+ addend[t]) in fp32, k-th term k-th
#include "common.cuh"

#define MOE_MAX_TOP 32

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ router, int width, int experts,
                 int top, int groups, int keep, int* __restrict__ chosen, float* __restrict__ weights) {
  extern __shared__ float mr_smem[];
  float* h = mr_smem;            // [width]
  float* score = h + width;      // [experts]
  float* group_best = score + experts;  // [groups]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  const T* row = x + (size_t)t * x_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) h[i] = to_float(row[i]);
  __syncthreads();
  for (int e = warp; e < experts; e += warps) {
    const float* w = router + (size_t)e * width;
    float dot = 0.0f;
    for (int i = lane; i < width; i += 32) dot = fmaf(w[i], h[i], dot);
    dot = warp_sum(dot);
    if (lane == 0) score[e] = dot;
  }
  __syncthreads();
  if (warp != 0) return;
  // softmax over all experts
  float biggest = -INFINITY;
  for (int e = lane; e < experts; e += 32) biggest = fmaxf(biggest, score[e]);
  biggest = warp_max(biggest);
  float total = 0.0f;
  for (int e = lane; e < experts; e += 32) total += expf(score[e] - biggest);
  total = warp_sum(total);
  for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - biggest) / total;
  __syncwarp();
  const int per_group = experts / groups;
  if (groups > 1 && keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per_group; e < (g + 1) * per_group; ++e) best = fmaxf(best, score[e]);
      group_best[g] = best;
    }
    __syncwarp();
    if (lane == 0) {
      // `keep` times: the best group not yet kept is marked by the value 2 (scores never exceed 1)
      for (int round = 0; round < keep; ++round) {
        int arg = -1;
        float best = -INFINITY;
        for (int g = 0; g < groups; ++g)
          if (group_best[g] <= 1.5f && group_best[g] > best) {
            best = group_best[g];
            arg = g;
          }
        if (arg < 0) break;
        group_best[arg] = 2.0f;  // scores are probabilities (<= 1): 2 marks "kept"
      }
    }
    __syncwarp();
  } else {
    for (int g = lane; g < groups; g += 32) group_best[g] = 2.0f;
    __syncwarp();
  }
  if (lane == 0) {
    int picked[MOE_MAX_TOP];
    float picked_score[MOE_MAX_TOP];
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
      int arg = -1;
      float best = -INFINITY;
      for (int e = 0; e < experts; ++e) {
        if (group_best[e / per_group] != 2.0f) continue;
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= picked[j] == e;
        if (!taken && score[e] > best) {
          best = score[e];
          arg = e;
        }
      }
      if (arg < 0) {  // fewer allowed experts than top: the remaining places carry no weight
        arg = k ? picked[0] : 0;
        best = 0.0f;
      }
      picked[k] = arg;
      picked_score[k] = best;
      sum += best;
    }
    for (int k = 0; k < top; ++k) {
      chosen[(size_t)t * top + k] = picked[k];
      weights[(size_t)t * top + k] = picked_score[k] / (sum + 1e-20f);
    }
  }
}

TS_EXPORT int ts_moe_route(int dtype, const void* x, long long x_stride, const float* router, int num_tokens,
                           int width, int experts, int top, int groups, int keep, int* chosen, float* weights,
                           cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (experts < 1 || top < 1 || top > MOE_MAX_TOP || top > experts || groups < 1 || experts % groups || keep < 1 ||
      keep > groups)
    return TS_ERR_SIZE;
  const size_t smem = ((size_t)width + experts + groups) * sizeof(float);
  if (smem > 200 * 1024) return TS_ERR_SIZE;
  if (dtype == TS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_route_kernel<float>, dim3(num_tokens), dim3(128), smem, stream, (const float*)x, x_stride, router, width,
              experts, top, groups, keep, chosen, weights);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_route_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), smem, stream, (const __nv_bfloat16*)x, x_stride,
              router, width, experts, top, groups, keep, chosen, weights);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// Steps of few tokens.
// ---------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* __restrict__ h, int n, int lane);
template <> __device__ __forceinline__ float row_dot<float>(const float* __restrict__ w, const float* __restrict__ h, int n, int lane) {
  float dot = 0.0f;
  if (n % 4 == 0 && !((uintptr_t)w & 15)) {
    for (int i = lane * 4; i < n; i += 128) {
      const float4 a = *reinterpret_cast<const float4*>(w + i);
      dot = fmaf(a.x, h[i], dot); dot = fmaf(a.y, h[i + 1], dot); dot = fmaf(a.z, h[i + 2], dot); dot = fmaf(a.w, h[i + 3], dot);
    }
  } else {
    for (int i = lane; i < n; i += 32) dot = fmaf(w[i], h[i], dot);
  }
  return warp_sum(dot);
}
template <> __device__ __forceinline__ float row_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ h, int n, int lane) {
  float dot = 0.0f;
  if (n % 8 == 0 && !((uintptr_t)w & 15)) {
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(w + i);
      const unsigned p[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        dot = fmaf(__uint_as_float(p[j] << 16), h[i + 2 * j], dot);
        dot = fmaf(__uint_as_float(p[j] & 0xffff0000u), h[i + 2 * j + 1], dot);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) dot = fmaf(__bfloat162float(w[i]), h[i], dot);
  }
  return warp_sum(dot);
}

#define MOE_FEATURES_PER_BLOCK 32

// gate_up: [experts][2 * ff][width], an expert's gate rows first, then its up rows.
template <typename T>
__global__ void __launch_bounds__(256)
moe_pair_gate_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ gate_up,
                        const int* __restrict__ chosen, T* __restrict__ hidden, int width, int ff, int top, int act) {
  extern __shared__ float mp_smem[];  // [width]
  const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  const T* row = x + (size_t)(pair / top) * x_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) mp_smem[i] = to_float(row[i]);
  __syncthreads();
  const int expert = chosen[pair];
  const T* base = gate_up + (size_t)expert * 2 * ff * width;
  const int f_end = min(ff, (int)(blockIdx.y + 1) * MOE_FEATURES_PER_BLOCK);
  for (int f = blockIdx.y * MOE_FEATURES_PER_BLOCK + warp; f < f_end; f += warps) {
    // gate and up are rounded to the activation type first, as a product that writes them would
    const float g = to_float(from_float<T>(row_dot<T>(base + (size_t)f * width, mp_smem, width, lane)));
    const float u = to_float(from_float<T>(row_dot<T>(base + (size_t)(ff + f) * width, mp_smem, width, lane)));
    if (lane == 0) hidden[(size_t)pair * ff + f] = from_float<T>(activation(g, act) * u);
  }
}

TS_EXPORT int ts_moe_pair_gate_up(int dtype, const void* x, long long x_stride, const void* gate_up, const int* chosen,
                                  void* hidden, int num_tokens, int width, int ff, int top, int act,
                                  cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024 || ff < 1 || top < 1) return TS_ERR_SIZE;
  dim3 grid(num_tokens * top, (ff + MOE_FEATURES_PER_BLOCK - 1) / MOE_FEATURES_PER_BLOCK);
  if (grid.y > 65535) return TS_ERR_SIZE;
  if (dtype == TS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_pair_gate_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_gate_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, x_stride, (const float*)gate_up,
              chosen, (float*)hidden, width, ff, top, act);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_pair_gate_up_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_gate_up_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)x, x_stride,
              (const __nv_bfloat16*)gate_up, chosen, (__nv_bfloat16*)hidden, width, ff, top, act);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// down: [experts][width][ff].
template <typename T>
__global__ void __launch_bounds__(256)
moe_pair_down_kernel(const T* __restrict__ hidden, const T* __restrict__ down, const int* __restrict__ chosen,
                     const float* __restrict__ weights, const T* __restrict__ addend, T* __restrict__ out, int width,
                     int ff, int top) {
  extern __shared__ float mp_smem[];  // [top][ff]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) mp_smem[i] = to_float(hidden[(size_t)t * top * ff + i]);
  __syncthreads();
  const int o_end = min(width, (int)(blockIdx.y + 1) * MOE_FEATURES_PER_BLOCK);
  for (int o = blockIdx.y * MOE_FEATURES_PER_BLOCK + warp; o < o_end; o += warps) {
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int expert = chosen[(size_t)t * top + k];
      const float part = row_dot<T>(down + ((size_t)expert * width + o) * ff, mp_smem + (size_t)k * ff, ff, lane);
      sum = fmaf(weights[(size_t)t * top + k], to_float(from_float<T>(part)), sum);
    }
    if (lane == 0) {
      if (addend) sum += to_float(addend[(size_t)t * width + o]);
      out[(size_t)t * width + o] = from_float<T>(sum);
    }
  }
}

TS_EXPORT int ts_moe_pair_down(int dtype, const void* hidden, const void* down, const int* chosen, const float* weights,
                               const void* addend, void* out, int num_tokens, int width, int ff, int top,
                               cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem = (size_t)top * ff * sizeof(float);
  if (smem > 200 * 1024 || ff < 1 || top < 1) return TS_ERR_SIZE;
  dim3 grid(num_tokens, (width + MOE_FEATURES_PER_BLOCK - 1) / MOE_FEATURES_PER_BLOCK);
  if (grid.y > 65535) return TS_ERR_SIZE;
  if (dtype == TS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_pair_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_down_kernel<float>, grid, dim3(256), smem, stream, (const float*)hidden, (const float*)down, chosen,
              weights, (const float*)addend, (float*)out, width, ff, top);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_pair_down_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_down_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)hidden,
              (const __nv_bfloat16*)down, chosen, weights, (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, width, ff, top);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// Steps of many tokens: pairs in expert order.
// counters: [experts] counts, then [experts + 1] offsets, then [experts] cursors (int32).
// ---------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ counters) {
  pdl_wait();
  pdl_trigger<1>();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < pairs) atomicAdd(counters + chosen[i], 1);
}

__global__ void moe_offsets_kernel(int experts, int* __restrict__ counters) {
  pdl_wait();
  pdl_trigger<1>();
  if (threadIdx.x != 0) return;
  int* offsets = counters + experts;
  int* cursors = offsets + experts + 1;
  int total = 0;
  for (int e = 0; e < experts; ++e) {
    offsets[e] = total;
    cursors[e] = 0;
    total += counters[e];
  }
  offsets[experts] = total;
}

__global__ void moe_place_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ counters,
                                 int* __restrict__ place, int* __restrict__ pair_of_row) {
  pdl_wait();
  pdl_trigger<1>();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = chosen[i];
  const int row = counters[experts + e] + atomicAdd(counters + 2 * experts + 1 + e, 1);
  place[i] = row;
  pair_of_row[row] = i;
}

TS_EXPORT int ts_moe_sort(const int* chosen, int pairs, int experts, int* counters, int* place, int* pair_of_row,
                          cudaStream_t stream) {
  if (pairs <= 0) return 0;
  cudaMemsetAsync(counters, 0, (size_t)experts * sizeof(int), stream);
  const unsigned blocks = (unsigned)((pairs + 255) / 256);
  ts_launch(moe_count_kernel, dim3(blocks), dim3(256), 0, stream, chosen, pairs, experts, counters);
  ts_launch(moe_offsets_kernel, dim3(1), dim3(32), 0, stream, experts, counters);
  ts_launch(moe_place_kernel, dim3(blocks), dim3(256), 0, stream, chosen, pairs, experts, counters, place, pair_of_row);
  return ts_launch_status();
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, long long x_stride, const int* __restrict__ pair_of_row,
                                  T* __restrict__ rows, int width, int top) {
  pdl_wait();
  pdl_trigger<1>();
  const int r = blockIdx.x;
  const T* src = x + (size_t)(pair_of_row[r] / top) * x_stride;
  T* dst = rows + (size_t)r * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

TS_EXPORT int ts_moe_gather(int dtype, const void* x, long long x_stride, const int* pair_of_row, void* rows, int pairs,
                            int width, int top, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (dtype == TS_F32)
    ts_launch(moe_gather_kernel<float>, dim3(pairs), dim3(128), 0, stream, (const float*)x, x_stride, pair_of_row,
              (float*)rows, width, top);
  else if (dtype == TS_BF16)
    ts_launch(moe_gather_kernel<__nv_bfloat16>, dim3(pairs), dim3(128), 0, stream, (const __nv_bfloat16*)x, x_stride,
              pair_of_row, (__nv_bfloat16*)rows, width, top);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place,
                                   const float* __restrict__ weights, const T* __restrict__ addend, T* __restrict__ out,
                                   int width, int top) {
  pdl_wait();
  pdl_trigger<1>();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float sum = 0.0f;
    for (int k = 0; k < top; ++k)
      sum = fmaf(weights[(size_t)t * top + k], to_float(rows[(size_t)place[(size_t)t * top + k] * width + i]), sum);
    if (addend) sum += to_float(addend[(size_t)t * width + i]);
    out[(size_t)t * width + i] = from_float<T>(sum);
  }
}

TS_EXPORT int ts_moe_combine(int dtype, const void* rows, const int* place, const float* weights, const void* addend,
                             void* out, int num_tokens, int width, int top, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dtype == TS_F32)
    ts_launch(moe_combine_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, (const float*)rows, place, weights,
              (const float*)addend, (float*)out, width, top);
  else if (dtype == TS_BF16)
    ts_launch(moe_combine_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)rows, place,
              weights, (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, width, top);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
