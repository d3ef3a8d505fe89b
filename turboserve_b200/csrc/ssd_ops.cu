// The state-space recurrence with a scalar decay per head (the "state space duality" layer), on a
// packed batch of requests with the state kept per request between steps, and the gated, grouped
// RMS norm that follows it.
//
// Per head h (value size P, state size N, group g = h / (heads / groups)) and position t:
//
//   dt_t = softplus(raw_t[h] + dt_bias[h])                   (fp32, no clamp)
//   S_t  = exp(-exp(A_log[h]) * dt_t) * S_{t-1} + dt_t * B_t[g] x_t[h]^T      (S is N x P, fp32)
//   y_t[h] = S_t^T C_t[g] + D[h] * x_t[h]
//
// ssd_scan: one block per (head, request, tile of P).  A step's positions of a request are taken in
// order, eight at a time through shared memory; a thread owns one value column p and the state
// rows n = s, s + NS, ... of it (NS lanes share a column and add their parts of y by shuffles), so
// the state stays in registers over the whole portion and is read and written once.  The state of
// a request lives in its slot of `state` ([slots, heads, P, N], fp32); a request that starts has a
// zeroed slot.  One token per request (decoding) and long portions of prompts run the same code:
// every sum has the same order however a request is cut into steps.
//
// gated_group_norm: v = y * silu(z); every one of `parts` equal parts of a row is divided by its
// own root mean square (eps inside the root) and multiplied by the weight; fp32, rounded once.
#include "common.cuh"

#define SSD_THREADS 128
#define SSD_ROWS_PER_THREAD 16
#define SSD_BATCH 8

template <typename T>
__global__ void __launch_bounds__(SSD_THREADS)
ssd_scan_kernel(const T* __restrict__ xbc, long long xbc_stride, const T* __restrict__ dt_raw, long long dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, float* __restrict__ y, const int* __restrict__ query_start,
                const int* __restrict__ slots, int heads, int groups, int P, int N, int NS) {
  extern __shared__ float smem[];
  const int head = blockIdx.x, seq = blockIdx.y;
  const int p_tile = SSD_THREADS / NS;
  const int p0 = blockIdx.z * p_tile;
  float* sB = smem;                         // [SSD_BATCH][N]
  float* sC = sB + SSD_BATCH * N;           // [SSD_BATCH][N]
  float* sx = sC + SSD_BATCH * N;           // [SSD_BATCH][p_tile]
  float* sdt = sx + SSD_BATCH * p_tile;     // [SSD_BATCH]
  float* sdecay = sdt + SSD_BATCH;          // [SSD_BATCH]
  const int tid = threadIdx.x;
  const int s = tid % NS, pl = tid / NS, p = p0 + pl;
  const int group = head / (heads / groups);
  const int inner = heads * P;
  const float rate = expf(a_log[head]);
  const float bias = dt_bias[head], skip = d_skip[head];
  pdl_wait();
  pdl_trigger();
  const int begin = query_start[seq], n = query_start[seq + 1] - begin;
  if (n <= 0) return;
  float* slot_state = state + (((size_t)slots[seq] * heads + head) * P) * N;
  float S[SSD_ROWS_PER_THREAD];
#pragma unroll
  for (int r = 0; r < SSD_ROWS_PER_THREAD; ++r) {
    const int row = s + NS * r;
    S[r] = (p < P && row < N) ? slot_state[(size_t)p * N + row] : 0.0f;
  }
  for (int base = 0; base < n; base += SSD_BATCH) {
    const int count = min(SSD_BATCH, n - base);
    __syncthreads();
    for (int i = tid; i < count * N; i += SSD_THREADS) {
      const int tt = i / N, row = i % N;
      const T* src = xbc + (size_t)(begin + base + tt) * xbc_stride + inner + group * N + row;
      sB[tt * N + row] = to_float(src[0]);
      sC[tt * N + row] = to_float(src[(size_t)groups * N]);
    }
    for (int i = tid; i < count * p_tile; i += SSD_THREADS) {
      const int tt = i / p_tile, col = p0 + i % p_tile;
      sx[i] = col < P ? to_float(xbc[(size_t)(begin + base + tt) * xbc_stride + head * P + col]) : 0.0f;
    }
    if (tid < count) {
      const float v = to_float(dt_raw[(size_t)(begin + base + tid) * dt_stride + head]) + bias;
      const float step = v > 20.0f ? v : log1pf(expf(v));
      sdt[tid] = step;
      sdecay[tid] = expf(-rate * step);
    }
    __syncthreads();
    for (int tt = 0; tt < count; ++tt) {
      const float decay = sdecay[tt];
      const float x = sx[tt * p_tile + pl];
      const float dx = sdt[tt] * x;
      const float* Bt = sB + tt * N;
      const float* Ct = sC + tt * N;
      float part = 0.0f;
#pragma unroll
      for (int r = 0; r < SSD_ROWS_PER_THREAD; ++r) {
        const int row = s + NS * r;
        if (row < N) {
          S[r] = fmaf(decay, S[r], dx * Bt[row]);
          part = fmaf(S[r], Ct[row], part);
        }
      }
      for (int offset = NS >> 1; offset > 0; offset >>= 1) part += __shfl_xor_sync(0xffffffffu, part, offset);
      if (s == 0 && p < P) y[(size_t)(begin + base + tt) * inner + head * P + p] = part + skip * x;
    }
  }
#pragma unroll
  for (int r = 0; r < SSD_ROWS_PER_THREAD; ++r) {
    const int row = s + NS * r;
    if (p < P && row < N) slot_state[(size_t)p * N + row] = S[r];
  }
}

TS_EXPORT int ts_ssd_scan(int dtype, const void* xbc, long long xbc_stride, const void* dt_raw, long long dt_stride,
                          const float* dt_bias, const float* a_log, const float* d_skip, float* state, float* y,
                          const int* query_start, const int* slots, int num_seqs, int heads, int groups, int P, int N,
                          cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || P < 1 || N < 1) return TS_ERR_SIZE;
  int NS = 1;
  while (N > SSD_ROWS_PER_THREAD * NS) NS *= 2;
  if (NS > 32) return TS_ERR_SIZE;  // state sizes above 512 are not taken
  const int p_tile = SSD_THREADS / NS;
  const int tiles = (P + p_tile - 1) / p_tile;
  if (heads > 2147483647 / 1 || num_seqs > 65535 || tiles > 65535) return TS_ERR_SIZE;
  const size_t smem = (size_t)SSD_BATCH * (2 * N + p_tile + 2) * sizeof(float);
  dim3 grid(heads, num_seqs, tiles);
  if (dtype == TS_F32)
    ts_launch(ssd_scan_kernel<float>, grid, dim3(SSD_THREADS), smem, stream, (const float*)xbc, xbc_stride,
              (const float*)dt_raw, dt_stride, dt_bias, a_log, d_skip, state, y, query_start, slots, heads, groups, P, N, NS);
  else if (dtype == TS_BF16)
    ts_launch(ssd_scan_kernel<__nv_bfloat16>, grid, dim3(SSD_THREADS), smem, stream, (const __nv_bfloat16*)xbc, xbc_stride,
              (const __nv_bfloat16*)dt_raw, dt_stride, dt_bias, a_log, d_skip, state, y, query_start, slots, heads, groups,
              P, N, NS);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride,
                                        const float* __restrict__ weight, T* __restrict__ out, int inner, int parts,
                                        float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_trigger<1>();
  const int t = blockIdx.x, part = blockIdx.y;
  const int width = inner / parts;
  const float* y_row = y + (size_t)t * inner + (size_t)part * width;
  const T* z_row = z + (size_t)t * z_stride + (size_t)part * width;
  float squares = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float gate = to_float(z_row[i]);
    const float v = y_row[i] * (gate / (1.0f + expf(-gate)));
    squares = fmaf(v, v, squares);
  }
  const float total = block_sum(squares, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  T* o_row = out + (size_t)t * inner + (size_t)part * width;
  const float* w = weight + (size_t)part * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float gate = to_float(z_row[i]);
    const float v = y_row[i] * (gate / (1.0f + expf(-gate)));
    o_row[i] = from_float<T>(v * inv * w[i]);
  }
}

TS_EXPORT int ts_gated_group_norm(int dtype, const float* y, const void* z, long long z_stride, const float* weight,
                                  void* out, int num_tokens, int inner, int parts, float eps, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (inner < 1 || parts < 1 || inner % parts || parts > 65535) return TS_ERR_SIZE;
  const int width = inner / parts;
  int threads = (width + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  dim3 grid(num_tokens, parts);
  if (dtype == TS_F32)
    ts_launch(gated_group_norm_kernel<float>, grid, dim3(threads), 0, stream, y, (const float*)z, z_stride, weight,
              (float*)out, inner, parts, eps);
  else if (dtype == TS_BF16)
    ts_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, y, (const __nv_bfloat16*)z, z_stride,
              weight, (__nv_bfloat16*)out, inner, parts, eps);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
