// Differential attention over a paged cache: two softmax maps per head over the same values,
// combined as a1 - lambda * a2, brought to unit root mean square per head and scaled.
//
// A query head has two query vectors of `dim` elements (laid out one after the other), its key
// head two key vectors; both maps attend over the value head's `vdim` elements:
//
//   s_m[j] = scale * <q_m, k_m[j]>           for the keys j = lo .. p of the query's own request,
//   a_m    = softmax(s_m) V                   lo = max(0, p - window + 1)  (window == 0: lo = 0)
//   o      = a_1 - lambda * a_2
//   out    = o / sqrt(mean(o^2) + eps) * out_scale
//
// Everything is fp32 (scores, both softmaxes with running maxima, the value sums, the norm);
// inputs and the output are in the activation type and the output is rounded once.
//
// This file holds the kernels for every type and size.  The first: one block per (query token, query head),
// keys in tiles of 32 counted from lo and dealt to DIFF_STREAMS streams (stream s takes tiles
// s, s + DIFF_STREAMS, ...); a lane scores one key for both maps, then the tile's values are
// accumulated once for both (every lane owns value elements lane, lane + 32, ...).  The streams'
// partial results are merged in stream order, so the order of every sum depends on (lo, p) only
// and the output of a token is the same bits however its request was cut into steps and
// whatever else the batch holds.  A step of few tokens runs a warp per stream, a step of many
// four warps with four streams each.
#include "common.cuh"

#define DIFF_STREAMS 16
#define DIFF_MAX_PER_LANE 8  // vdim <= 256

template <typename T>
__global__ void __launch_bounds__(DIFF_STREAMS * 32)
diff_attention_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                      const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                      const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_of_token,
                      const int* __restrict__ positions, int page_size, int num_heads, int num_kv_heads, int dim,
                      int vdim, int window, float scale, float lambda, float eps, float out_scale,
                      int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float smem[];
  float* q_s = smem;                                        // [2 * dim]
  float* part_acc = smem + 2 * dim;                         // [DIFF_STREAMS][2][vdim]
  float* part_ml = part_acc + DIFF_STREAMS * 2 * vdim;      // [DIFF_STREAMS][4]: m1, l1, m2, l2

  const int t = blockIdx.x, head = blockIdx.y;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kv_head = head / (num_heads / num_kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  const int* table = block_table + (size_t)seq * table_stride;
  const int kdim = 2 * dim;

  const T* q_row = q + (size_t)t * q_stride + (size_t)head * kdim;
  for (int i = threadIdx.x; i < kdim; i += blockDim.x) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  const int num_keys = pos - lo + 1;
  const int num_tiles = (num_keys + 31) / 32;
  for (int stream = warp; stream < DIFF_STREAMS; stream += num_warps) {
    float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
    float acc1[DIFF_MAX_PER_LANE], acc2[DIFF_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < DIFF_MAX_PER_LANE; ++i) acc1[i] = acc2[i] = 0.0f;
    for (int tile = stream; tile < num_tiles; tile += DIFF_STREAMS) {
      const int key = lo + tile * 32 + lane;
      float s1 = -INFINITY, s2 = -INFINITY;
      size_t v_row = 0;
      if (key <= pos) {
        const int page = table[key / page_size];
        if (page < 0) {
          if (status) atomicOr(status, 4);
        } else {
          const size_t slot = ((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head;
          v_row = slot * vdim;
          const T* k_row = k_pages + slot * kdim;
          float d1 = 0.0f, d2 = 0.0f;
          for (int i = 0; i < dim; ++i) d1 = fmaf(q_s[i], to_float(k_row[i]), d1);
          for (int i = 0; i < dim; ++i) d2 = fmaf(q_s[dim + i], to_float(k_row[dim + i]), d2);
          s1 = d1 * scale;
          s2 = d2 * scale;
        }
      }
      const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
      if (n1 == -INFINITY) continue;  // only unreadable keys so far (both maps see the same keys)
      const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);
      const float p1 = s1 == -INFINITY ? 0.0f : expf(s1 - n1);
      const float p2 = s2 == -INFINITY ? 0.0f : expf(s2 - n2);
      l1 = l1 * c1 + warp_sum(p1);
      l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
      for (int i = 0; i < DIFF_MAX_PER_LANE; ++i) {
        acc1[i] *= c1;
        acc2[i] *= c2;
      }
      m1 = n1;
      m2 = n2;
      const int in_tile = min(32, pos - (lo + tile * 32) + 1);
      for (int j = 0; j < in_tile; ++j) {
        const float w1 = __shfl_sync(0xffffffffu, p1, j), w2 = __shfl_sync(0xffffffffu, p2, j);
        const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)v_row, j);
        if (w1 == 0.0f && w2 == 0.0f) continue;
        const T* v = v_pages + rj;
#pragma unroll
        for (int i = 0; i < DIFF_MAX_PER_LANE; ++i) {
          const int e = lane + 32 * i;
          if (e < vdim) {
            const float x = to_float(v[e]);
            acc1[i] = fmaf(w1, x, acc1[i]);
            acc2[i] = fmaf(w2, x, acc2[i]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < DIFF_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < vdim) {
        part_acc[(stream * 2) * vdim + e] = acc1[i];
        part_acc[(stream * 2 + 1) * vdim + e] = acc2[i];
      }
    }
    if (lane == 0) {
      part_ml[stream * 4] = m1;
      part_ml[stream * 4 + 1] = l1;
      part_ml[stream * 4 + 2] = m2;
      part_ml[stream * 4 + 3] = l2;
    }
  }
  __syncthreads();
  if (warp == 0) {
    float top1 = -INFINITY, top2 = -INFINITY;
    for (int s = 0; s < DIFF_STREAMS; ++s) {
      top1 = fmaxf(top1, part_ml[s * 4]);
      top2 = fmaxf(top2, part_ml[s * 4 + 2]);
    }
    float w1[DIFF_STREAMS], w2[DIFF_STREAMS];
    float sum1 = 0.0f, sum2 = 0.0f;
    for (int s = 0; s < DIFF_STREAMS; ++s) {
      const float a = part_ml[s * 4], b = part_ml[s * 4 + 2];
      w1[s] = a == -INFINITY ? 0.0f : expf(a - top1);
      w2[s] = b == -INFINITY ? 0.0f : expf(b - top2);
      sum1 += part_ml[s * 4 + 1] * w1[s];
      sum2 += part_ml[s * 4 + 3] * w2[s];
    }
    const float inv1 = sum1 > 0.0f ? 1.0f / sum1 : 0.0f, inv2 = sum2 > 0.0f ? 1.0f / sum2 : 0.0f;
    float o[DIFF_MAX_PER_LANE];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < DIFF_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      o[i] = 0.0f;
      if (e < vdim) {
        float a1 = 0.0f, a2 = 0.0f;
        for (int s = 0; s < DIFF_STREAMS; ++s) {
          a1 += part_acc[(s * 2) * vdim + e] * w1[s];
          a2 += part_acc[(s * 2 + 1) * vdim + e] * w2[s];
        }
        o[i] = a1 * inv1 - lambda * (a2 * inv2);
        squares = fmaf(o[i], o[i], squares);
      }
    }
    squares = warp_sum(squares);
    const float unit = out_scale / sqrtf(squares / (float)vdim + eps);
    T* o_row = out + (size_t)t * out_stride + (size_t)head * vdim;
#pragma unroll
    for (int i = 0; i < DIFF_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < vdim) o_row[e] = from_float<T>(o[i] * unit);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The same, one block per (query token, key head): the QH query heads that share a key head are
// scored against every key row and accumulate every value row together, so a step that decodes
// reads its keys and values once, 16 bytes at a time (a lane reads its key's row in vectors when
// the rows are 16-byte aligned).  Sixteen warps, one per stream; a tile's weights go through a
// small buffer in shared memory from the lanes that scored the keys to all lanes for the value
// sum.  Streams are merged by one warp per head.  The order of every sum is the one of the kernel
// above, so both give the same bits.
// ---------------------------------------------------------------------------------------------
#define DIFF_GROUP_MAX_PER_LANE 4  // vdim <= 128

template <typename T> struct DiffVec;
template <> struct DiffVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct DiffVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T, int QH>
__global__ void __launch_bounds__(DIFF_STREAMS * 32)
diff_attention_group_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                            const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                            const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_of_token,
                            const int* __restrict__ positions, int page_size, int num_kv_heads, int dim, int vdim,
                            int window, float scale, float lambda, float eps, float out_scale, int vector_rows,
                            int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float smem[];
  const int kdim = 2 * dim;
  float* q_s = smem;                                                  // [QH][kdim]
  float* part_acc = q_s + QH * kdim;                                  // [DIFF_STREAMS][QH][2][vdim]
  float* part_ml = part_acc + DIFF_STREAMS * QH * 2 * vdim;           // [DIFF_STREAMS][QH][4]
  float* weights = part_ml + DIFF_STREAMS * QH * 4;                   // [DIFF_STREAMS][32][2 * QH]
  unsigned long long* rows_s = reinterpret_cast<unsigned long long*>(weights + DIFF_STREAMS * 32 * 2 * QH);  // [DIFF_STREAMS][32]

  const int t = blockIdx.x, kv_head = blockIdx.y;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* table = block_table + (size_t)seq * table_stride;
  const T* q_row = q + (size_t)t * q_stride + (size_t)kv_head * QH * kdim;
  for (int i = threadIdx.x; i < QH * kdim; i += blockDim.x) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  const int num_tiles = (pos - lo + 32) / 32;
  const int stream = warp;
  float* my_weights = weights + stream * 32 * 2 * QH;
  unsigned long long* my_rows = rows_s + stream * 32;
  float top[QH][2], sum[QH][2];
  float acc[QH][2][DIFF_GROUP_MAX_PER_LANE];
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    top[h][0] = top[h][1] = -INFINITY;
    sum[h][0] = sum[h][1] = 0.0f;
#pragma unroll
    for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) acc[h][0][i] = acc[h][1][i] = 0.0f;
  }
  for (int tile = stream; tile < num_tiles; tile += DIFF_STREAMS) {
    const int key = lo + tile * 32 + lane;
    float d[QH][2];
#pragma unroll
    for (int h = 0; h < QH; ++h) d[h][0] = d[h][1] = 0.0f;
    bool readable = false;
    size_t v_row = 0;
    if (key <= pos) {
      const int page = table[key / page_size];
      if (page < 0) {
        if (status) atomicOr(status, 4);
      } else {
        readable = true;
        const size_t slot = ((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head;
        v_row = slot * vdim;
        const T* k_row = k_pages + slot * kdim;
        if (vector_rows) {
          constexpr int W = DiffVec<T>::N;
#pragma unroll 1
          for (int m = 0; m < 2; ++m) {
#pragma unroll 4
            for (int i = 0; i < dim; i += W) {
              float kv[W];
              DiffVec<T>::load(k_row + m * dim + i, kv);
#pragma unroll
              for (int h = 0; h < QH; ++h) {
                const float* qh = q_s + h * kdim + m * dim + i;
                float total = d[h][m];
#pragma unroll
                for (int e = 0; e < W; ++e) total = fmaf(qh[e], kv[e], total);
                d[h][m] = total;
              }
            }
          }
        } else {
          for (int m = 0; m < 2; ++m) {
            for (int i = 0; i < dim; ++i) {
              const float kv = to_float(k_row[m * dim + i]);
#pragma unroll
              for (int h = 0; h < QH; ++h) d[h][m] = fmaf(q_s[h * kdim + m * dim + i], kv, d[h][m]);
            }
          }
        }
      }
    }
    bool any = false;
#pragma unroll
    for (int h = 0; h < QH; ++h) {
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const float sc = readable ? d[h][m] * scale : -INFINITY;
        const float next = fmaxf(top[h][m], warp_max(sc));
        float p = 0.0f, corr = 1.0f;
        if (next != -INFINITY) {
          any = true;
          corr = expf(top[h][m] - next);
          p = sc == -INFINITY ? 0.0f : expf(sc - next);
          sum[h][m] = sum[h][m] * corr + warp_sum(p);
          top[h][m] = next;
        }
#pragma unroll
        for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) acc[h][m][i] *= corr;
        my_weights[lane * 2 * QH + h * 2 + m] = p;
      }
    }
    my_rows[lane] = (unsigned long long)v_row;
    __syncwarp();
    if (any) {
      const int in_tile = min(32, pos - (lo + tile * 32) + 1);
#pragma unroll 4
      for (int j = 0; j < in_tile; ++j) {
        const T* v = v_pages + my_rows[j];
        float x[DIFF_GROUP_MAX_PER_LANE];
#pragma unroll
        for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) {
          const int e = lane + 32 * i;
          x[i] = e < vdim ? to_float(v[e]) : 0.0f;
        }
        const float* w = my_weights + j * 2 * QH;
#pragma unroll
        for (int h = 0; h < QH; ++h) {
          const float w1 = w[h * 2], w2 = w[h * 2 + 1];
#pragma unroll
          for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) {
            acc[h][0][i] = fmaf(w1, x[i], acc[h][0][i]);
            acc[h][1][i] = fmaf(w2, x[i], acc[h][1][i]);
          }
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int h = 0; h < QH; ++h) {
#pragma unroll
    for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < vdim) {
        part_acc[((stream * QH + h) * 2) * vdim + e] = acc[h][0][i];
        part_acc[((stream * QH + h) * 2 + 1) * vdim + e] = acc[h][1][i];
      }
    }
    if (lane == 0) {
      float* ml = part_ml + (stream * QH + h) * 4;
      ml[0] = top[h][0]; ml[1] = sum[h][0]; ml[2] = top[h][1]; ml[3] = sum[h][1];
    }
  }
  __syncthreads();
  if (warp < QH) {
    const int h = warp;
    float top1 = -INFINITY, top2 = -INFINITY;
    for (int s = 0; s < DIFF_STREAMS; ++s) {
      top1 = fmaxf(top1, part_ml[(s * QH + h) * 4]);
      top2 = fmaxf(top2, part_ml[(s * QH + h) * 4 + 2]);
    }
    float w1[DIFF_STREAMS], w2[DIFF_STREAMS];
    float sum1 = 0.0f, sum2 = 0.0f;
    for (int s = 0; s < DIFF_STREAMS; ++s) {
      const float a = part_ml[(s * QH + h) * 4], b = part_ml[(s * QH + h) * 4 + 2];
      w1[s] = a == -INFINITY ? 0.0f : expf(a - top1);
      w2[s] = b == -INFINITY ? 0.0f : expf(b - top2);
      sum1 += part_ml[(s * QH + h) * 4 + 1] * w1[s];
      sum2 += part_ml[(s * QH + h) * 4 + 3] * w2[s];
    }
    const float inv1 = sum1 > 0.0f ? 1.0f / sum1 : 0.0f, inv2 = sum2 > 0.0f ? 1.0f / sum2 : 0.0f;
    float o[DIFF_GROUP_MAX_PER_LANE];
    float squares = 0.0f;
#pragma unroll
    for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      o[i] = 0.0f;
      if (e < vdim) {
        float a1 = 0.0f, a2 = 0.0f;
        for (int s = 0; s < DIFF_STREAMS; ++s) {
          a1 += part_acc[((s * QH + h) * 2) * vdim + e] * w1[s];
          a2 += part_acc[((s * QH + h) * 2 + 1) * vdim + e] * w2[s];
        }
        o[i] = a1 * inv1 - lambda * (a2 * inv2);
        squares = fmaf(o[i], o[i], squares);
      }
    }
    squares = warp_sum(squares);
    const float unit = out_scale / sqrtf(squares / (float)vdim + eps);
    T* o_row = out + (size_t)t * out_stride + (size_t)(kv_head * QH + h) * vdim;
#pragma unroll
    for (int i = 0; i < DIFF_GROUP_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < vdim) o_row[e] = from_float<T>(o[i] * unit);
    }
  }
}

template <typename T, int QH>
static int diff_attention_group_launch(const void* q, long long q_stride, void* out, long long out_stride,
                                       const void* k_pages, const void* v_pages, const int* block_table,
                                       int table_stride, const int* seq_of_token, const int* positions, int num_tokens,
                                       int page_size, int num_kv_heads, int dim, int vdim, int window, float scale,
                                       float lambda, float eps, float out_scale, int* status, cudaStream_t stream) {
  const size_t floats = (size_t)QH * 2 * dim + (size_t)DIFF_STREAMS * QH * 2 * vdim + (size_t)DIFF_STREAMS * QH * 4 +
                        (size_t)DIFF_STREAMS * 32 * 2 * QH;
  const size_t smem = floats * sizeof(float) + (size_t)DIFF_STREAMS * 32 * sizeof(unsigned long long);
  if (smem > 200 * 1024) return TS_ERR_SIZE;
  auto kernel = diff_attention_group_kernel<T, QH>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int vector_rows = (2 * dim * sizeof(T)) % 16 == 0 && (dim * sizeof(T)) % 16 == 0 && !((uintptr_t)k_pages & 15);
  ts_launch(kernel, dim3(num_tokens, num_kv_heads), dim3(DIFF_STREAMS * 32), smem, stream, (const T*)q, q_stride, (T*)out,
            out_stride, (const T*)k_pages, (const T*)v_pages, block_table, table_stride, seq_of_token, positions, page_size,
            num_kv_heads, dim, vdim, window, scale, lambda, eps, out_scale, vector_rows, status);
  return ts_launch_status();
}

TS_EXPORT int ts_diff_attention(int dtype, const void* q, long long q_stride, void* out, long long out_stride,
                                const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                                const int* seq_of_token, const int* positions, int num_tokens, int page_size,
                                int num_heads, int num_kv_heads, int dim, int vdim, int window, float scale,
                                float lambda, float eps, float out_scale, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dim < 1 || vdim < 1 || vdim > 32 * DIFF_MAX_PER_LANE) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads) return TS_ERR_SIZE;
  if (num_heads > 65535 || page_size < 1 || window < 0) return TS_ERR_ARGUMENT;
  const int per_group = num_heads / num_kv_heads;
  if (vdim <= 32 * DIFF_GROUP_MAX_PER_LANE && num_kv_heads <= 65535 &&
      (per_group == 1 || per_group == 2 || per_group == 4 || per_group == 8) && (dtype == TS_F32 || dtype == TS_BF16)) {
#define DIFF_GROUP_CASE(TYPE, HEADS)                                                                                    \
  return diff_attention_group_launch<TYPE, HEADS>(q, q_stride, out, out_stride, k_pages, v_pages, block_table,          \
                                                  table_stride, seq_of_token, positions, num_tokens, page_size,         \
                                                  num_kv_heads, dim, vdim, window, scale, lambda, eps, out_scale, status, \
                                                  stream)
    if (dtype == TS_F32) {
      if (per_group == 1) DIFF_GROUP_CASE(float, 1);
      if (per_group == 2) DIFF_GROUP_CASE(float, 2);
      if (per_group == 4) DIFF_GROUP_CASE(float, 4);
      DIFF_GROUP_CASE(float, 8);
    }
    if (per_group == 1) DIFF_GROUP_CASE(__nv_bfloat16, 1);
    if (per_group == 2) DIFF_GROUP_CASE(__nv_bfloat16, 2);
    if (per_group == 4) DIFF_GROUP_CASE(__nv_bfloat16, 4);
    DIFF_GROUP_CASE(__nv_bfloat16, 8);
#undef DIFF_GROUP_CASE
  }
  const size_t smem = ((size_t)2 * dim + (size_t)DIFF_STREAMS * 2 * vdim + 4 * DIFF_STREAMS) * sizeof(float);
  if (smem > 48 * 1024) return TS_ERR_SIZE;
  dim3 grid(num_tokens, num_heads);
  const int threads = (long long)num_tokens * num_heads <= 2048 ? DIFF_STREAMS * 32 : 4 * 32;
  if (dtype == TS_F32)
    ts_launch(diff_attention_kernel<float>, grid, dim3(threads), smem, stream, (const float*)q, q_stride, (float*)out,
              out_stride, (const float*)k_pages, (const float*)v_pages, block_table, table_stride, seq_of_token, positions,
              page_size, num_heads, num_kv_heads, dim, vdim, window, scale, lambda, eps, out_scale, status);
  else if (dtype == TS_BF16)
    ts_launch(diff_attention_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, (const __nv_bfloat16*)q, q_stride,
              (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
              table_stride, seq_of_token, positions, page_size, num_heads, num_kv_heads, dim, vdim, window, scale, lambda,
              eps, out_scale, status);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
