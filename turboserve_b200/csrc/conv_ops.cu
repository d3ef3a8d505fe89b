// Short causal convolution over time, channel by channel, on a packed batch of requests, with
// the last inputs of every request kept as state between steps.
//
//   y[t, c] = act( bias[c] + sum_{j < J} w[c, j] * u[t - (J - 1) + j, c] )
//
// `u` are columns [first, first + C) of a row-major activation matrix (the product of a
// projection), `t` runs over the positions of one request; inputs before the request's first
// token are zero.  A step brings positions start .. start + n - 1 of a request; the J - 1 inputs
// before `start` come from the request's slot of `tail` ([slots, J - 1, C], oldest first), which
// a second kernel brings up to date after the step's outputs are computed (the first kernel
// only reads it).  A request that starts has a zeroed slot.  The sum runs over j = 0 .. J - 1 in
// that order in fp32, so an output does not depend on how the request was cut into steps.
//
// The same kernel can append a range of its output channels to a paged key cache and another to
// a paged value cache (rows of `k_width` and `v_width` elements per token: all key heads, all
// value heads), which is what an attention layer with convolved keys and values needs next.
#include "common.cuh"

#define CONV_MAX_TAPS 16
#define CONV_TOKENS 16  // tokens a thread takes in a row in a step of many tokens (1 in a small step)

struct ConvAppend {
  void* k_pages;          // [pages, page_size, k_width] or null
  void* v_pages;          // [pages, page_size, v_width]
  const int* block_table; // [seqs, table_stride]
  const int* positions;   // [tokens]
  int table_stride, page_size;
  int k_first, k_width, v_first, v_width;  // channel ranges (relative to the convolved channels)
};

// VEC adjacent channels at once (2 when the channel count, the first column and the strides are even)
template <typename T, int VEC> struct ConvIO;
template <typename T> struct ConvIO<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = to_float(p[0]); }
  static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { p[0] = from_float<T>(v[0]); }
};
template <> struct ConvIO<float, 2> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[2]) {
    const float2 x = *reinterpret_cast<const float2*>(p);
    v[0] = x.x; v[1] = x.y;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[2]) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
};
template <> struct ConvIO<__nv_bfloat16, 2> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[2]) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(p);
    v[0] = __low2float(x); v[1] = __high2float(x);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[2]) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
  }
};

// A thread takes its VEC channels through `run` tokens in a row (CONV_TOKENS in a step of many tokens, fewer
// in a small one, where every token wants a thread of its own).  The weights are fetched once;
// the J - 1 inputs before a token stay in registers from one token to the next while the tokens are
// consecutive positions of one request, and are fetched anew (from the step's rows, or from the
// request's tail where they lie before the step) at the thread's first token and at every token that
// starts another request's portion.
template <typename T, int VEC, int TMAX>  // taps <= TMAX: every loop over taps is unrolled to TMAX and predicated
__global__ void causal_conv_kernel(const T* __restrict__ in, long long in_stride, int first,
                                   const float* __restrict__ weight, const float* __restrict__ bias,
                                   const T* __restrict__ tail, T* __restrict__ out, long long out_stride,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ query_start,
                                   const int* __restrict__ slots, int num_tokens, int run, int channels, int taps, int act,
                                   ConvAppend append, int* __restrict__ status) {
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  float w[VEC][TMAX];
  float b[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    b[v] = (bias && c + v < channels) ? bias[c + v] : 0.0f;
#pragma unroll
    for (int j = 0; j < TMAX; ++j) w[v][j] = (j < taps && c + v < channels) ? weight[(size_t)(c + v) * taps + j] : 0.0f;
  }
  pdl_wait();
  pdl_trigger<1>();
  if (c >= channels) return;
  float hist[VEC][TMAX];  // hist[.][j], j < J - 1: the input j - (J - 1) positions from the current token
  int prev_seq = -1;
  const int t_end = min(num_tokens, (int)(blockIdx.x + 1) * run);
  for (int t = blockIdx.x * run; t < t_end; ++t) {
    const int seq = seq_of_token[t];
    if (seq < 0) {
      prev_seq = -1;
      continue;
    }
    const int index = t - query_start[seq];  // position within this step's portion of the request
    if (seq != prev_seq || index == 0) {
      const T* slot_tail = tail + (size_t)slots[seq] * (taps - 1) * channels;
#pragma unroll
      for (int j = 0; j < TMAX - 1; ++j) {
        if (j < taps - 1) {
          const int back = taps - 1 - j;  // how many positions before t
          float u[VEC];
          if (index - back >= 0) ConvIO<T, VEC>::load(in + (size_t)(t - back) * in_stride + first + c, u);
          else ConvIO<T, VEC>::load(slot_tail + (size_t)(taps - 1 + index - back) * channels + c, u);
#pragma unroll
          for (int v = 0; v < VEC; ++v) hist[v][j] = u[v];
        }
      }
      prev_seq = seq;
    }
    float cur[VEC], result[VEC];
    ConvIO<T, VEC>::load(in + (size_t)t * in_stride + first + c, cur);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float sum = b[v];
      float last = 0.0f;  // the weight of the current position
#pragma unroll
      for (int j = 0; j < TMAX; ++j) {
        if (j < taps - 1) sum = fmaf(w[v][j], hist[v][j], sum);
        if (j == taps - 1) last = w[v][j];
      }
      sum = fmaf(last, cur[v], sum);
      if (act == 1) sum = sum / (1.0f + expf(-sum));
      result[v] = sum;
#pragma unroll
      for (int j = 0; j < TMAX - 1; ++j) {
        if (j + 1 < taps - 1) hist[v][j] = hist[v][j + 1];
        else if (j == taps - 2) hist[v][j] = cur[v];
      }
    }
    ConvIO<T, VEC>::store(out + (size_t)t * out_stride + c, result);
    if (append.k_pages) {
      // VEC channels lie in one range: the ranges' bounds are multiples of VEC when VEC is 2
      const bool is_k = c >= append.k_first && c < append.k_first + append.k_width;
      const bool is_v = c >= append.v_first && c < append.v_first + append.v_width;
      if (is_k || is_v) {
        const int pos = append.positions[t];
        const int page = append.block_table[(size_t)seq * append.table_stride + pos / append.page_size];
        if (page < 0) {
          if (status) atomicOr(status, 2);
        } else {
          const size_t row = (size_t)page * append.page_size + pos % append.page_size;
          if (is_k) ConvIO<T, VEC>::store((T*)append.k_pages + row * append.k_width + (c - append.k_first), result);
          else ConvIO<T, VEC>::store((T*)append.v_pages + row * append.v_width + (c - append.v_first), result);
        }
      }
    }
  }
}

// tail[slot] <- the last J - 1 inputs of the request after this step: from the step's own inputs,
// and from the old tail where the step brought fewer than J - 1 positions.  A thread owns one
// (request, channel) and reads everything it needs before it writes.
template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ in, long long in_stride, int first, T* __restrict__ tail,
                                 const int* __restrict__ query_start, const int* __restrict__ slots, int channels,
                                 int taps) {
  pdl_wait();
  pdl_trigger<1>();
  const int seq = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int begin = query_start[seq], n = query_start[seq + 1] - begin;
  if (n <= 0 || c >= channels) return;
  T* slot_tail = tail + (size_t)slots[seq] * (taps - 1) * channels;
  T keep[CONV_MAX_TAPS];
  for (int k = 0; k < taps - 1; ++k) {
    const int index = n - (taps - 1) + k;
    keep[k] = index >= 0 ? in[(size_t)(begin + index) * in_stride + first + c] : slot_tail[(size_t)(k + n) * channels + c];
  }
  for (int k = 0; k < taps - 1; ++k) slot_tail[(size_t)k * channels + c] = keep[k];
}

template <typename T>
static int causal_conv_launch(const void* in, long long in_stride, int first, const float* weight, const float* bias,
                              void* tail, void* out, long long out_stride, const int* seq_of_token,
                              const int* query_start, const int* slots, int num_tokens, int num_seqs, int channels,
                              int taps, int act, ConvAppend append, int* status, cudaStream_t stream) {
  const bool pairs = channels % 2 == 0 && first % 2 == 0 && in_stride % 2 == 0 && out_stride % 2 == 0 &&
                     !((uintptr_t)in % (2 * sizeof(T))) && !((uintptr_t)out % (2 * sizeof(T))) &&
                     !((uintptr_t)tail % (2 * sizeof(T))) &&
                     (!append.k_pages || (append.k_first % 2 == 0 && append.k_width % 2 == 0 && append.v_first % 2 == 0 &&
                                          append.v_width % 2 == 0 && !((uintptr_t)append.k_pages % (2 * sizeof(T))) &&
                                          !((uintptr_t)append.v_pages % (2 * sizeof(T)))));
  const int lanes = pairs ? channels / 2 : channels;
  const int threads = lanes >= 128 ? 128 : (lanes + 31) / 32 * 32;
  const int tiles = (lanes + threads - 1) / threads;
  const int run = num_tokens >= 2048 ? CONV_TOKENS : (num_tokens >= 512 ? 4 : 1);
  const dim3 grid((num_tokens + run - 1) / run, tiles);
#define CONV_CASE(VEC, TMAX)                                                                                              \
  ts_launch(causal_conv_kernel<T, VEC, TMAX>, grid, dim3(threads), 0, stream, (const T*)in, in_stride, first, weight, bias, \
            (const T*)tail, (T*)out, out_stride, seq_of_token, query_start, slots, num_tokens, run, channels, taps, act,    \
            append, status)
  if (pairs) {
    if (taps <= 4) CONV_CASE(2, 4); else if (taps <= 8) CONV_CASE(2, 8); else CONV_CASE(2, CONV_MAX_TAPS);
  } else {
    if (taps <= 4) CONV_CASE(1, 4); else if (taps <= 8) CONV_CASE(1, 8); else CONV_CASE(1, CONV_MAX_TAPS);
  }
#undef CONV_CASE
  int code = ts_launch_status();
  if (code) return code;
  if (taps > 1) {
    const int tail_threads = channels >= 256 ? 256 : (channels + 31) / 32 * 32;
    ts_launch(conv_tail_kernel<T>, dim3(num_seqs, (channels + tail_threads - 1) / tail_threads), dim3(tail_threads), 0, stream, (const T*)in, in_stride, first,
              (T*)tail, query_start, slots, channels, taps);
    code = ts_launch_status();
  }
  return code;
}

TS_EXPORT int ts_causal_conv(int dtype, const void* in, long long in_stride, int first, const float* weight,
                             const float* bias, void* tail, void* out, long long out_stride, const int* seq_of_token,
                             const int* query_start, const int* slots, int num_tokens, int num_seqs, int channels,
                             int taps, int act, void* k_pages, void* v_pages, const int* block_table, int table_stride,
                             const int* positions, int page_size, int k_first, int k_width, int v_first, int v_width,
                             int* status, cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS || channels < 1) return TS_ERR_SIZE;
  if (act < 0 || act > 1) return TS_ERR_ARGUMENT;
  ConvAppend append;
  memset(&append, 0, sizeof(append));
  if (k_pages) {
    if (!v_pages || !block_table || !positions || page_size < 1) return TS_ERR_ARGUMENT;
    if (k_first < 0 || v_first < 0 || k_first + k_width > channels || v_first + v_width > channels) return TS_ERR_ARGUMENT;
    append.k_pages = k_pages; append.v_pages = v_pages; append.block_table = block_table; append.positions = positions;
    append.table_stride = table_stride; append.page_size = page_size;
    append.k_first = k_first; append.k_width = k_width; append.v_first = v_first; append.v_width = v_width;
  }
  if (dtype == TS_F32)
    return causal_conv_launch<float>(in, in_stride, first, weight, bias, tail, out, out_stride, seq_of_token, query_start,
                                     slots, num_tokens, num_seqs, channels, taps, act, append, status, stream);
  if (dtype == TS_BF16)
    return causal_conv_launch<__nv_bfloat16>(in, in_stride, first, weight, bias, tail, out, out_stride, seq_of_token,
                                             query_start, slots, num_tokens, num_seqs, channels, taps, act, append, status,
                                             stream);
  return TS_ERR_DTYPE;
}
