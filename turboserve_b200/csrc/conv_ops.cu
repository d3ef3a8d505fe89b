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

struct ConvAppend {
  void* k_pages;          // [pages, page_size, k_width] or null
  void* v_pages;          // [pages, page_size, v_width]
  const int* block_table; // [seqs, table_stride]
  const int* positions;   // [tokens]
  int table_stride, page_size;
  int k_first, k_width, v_first, v_width;  // channel ranges (relative to the convolved channels)
};

template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ in, long long in_stride, int first,
                                   const float* __restrict__ weight, const float* __restrict__ bias,
                                   const T* __restrict__ tail, T* __restrict__ out, long long out_stride,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ query_start,
                                   const int* __restrict__ slots, int channels, int taps, int act,
                                   ConvAppend append, int* __restrict__ status) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  float w[CONV_MAX_TAPS];
  if (c < channels) {
    for (int j = 0; j < taps; ++j) w[j] = weight[(size_t)c * taps + j];
  }
  const float b = (bias && c < channels) ? bias[c] : 0.0f;
  pdl_wait();
  pdl_trigger<1>();
  const int seq = seq_of_token[t];
  if (seq < 0 || c >= channels) return;
  const int index = t - query_start[seq];  // position within this step's portion of the request
  const T* slot_tail = tail + (size_t)slots[seq] * (taps - 1) * channels;
  float sum = b;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;  // how many positions before t
    float u;
    if (index - back >= 0) u = to_float(in[(size_t)(t - back) * in_stride + first + c]);
    else u = to_float(slot_tail[(size_t)(taps - 1 + index - back) * channels + c]);
    sum = fmaf(w[j], u, sum);
  }
  if (act == 1) sum = sum / (1.0f + expf(-sum));
  const T value = from_float<T>(sum);
  out[(size_t)t * out_stride + c] = value;
  if (append.k_pages) {
    const bool is_k = c >= append.k_first && c < append.k_first + append.k_width;
    const bool is_v = c >= append.v_first && c < append.v_first + append.v_width;
    if (is_k || is_v) {
      const int pos = append.positions[t];
      const int page = append.block_table[(size_t)seq * append.table_stride + pos / append.page_size];
      if (page < 0) {
        if (status) atomicOr(status, 2);
      } else {
        const size_t row = (size_t)page * append.page_size + pos % append.page_size;
        if (is_k) ((T*)append.k_pages)[row * append.k_width + (c - append.k_first)] = value;
        else ((T*)append.v_pages)[row * append.v_width + (c - append.v_first)] = value;
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
  const int threads = channels >= 256 ? 256 : (channels + 31) / 32 * 32;
  const int tiles = (channels + threads - 1) / threads;
  ts_launch(causal_conv_kernel<T>, dim3(num_tokens, tiles), dim3(threads), 0, stream, (const T*)in, in_stride, first,
            weight, bias, (const T*)tail, (T*)out, out_stride, seq_of_token, query_start, slots, channels, taps, act,
            append, status);
  int code = ts_launch_status();
  if (code) return code;
  if (taps > 1) {
    ts_launch(conv_tail_kernel<T>, dim3(num_seqs, tiles), dim3(threads), 0, stream, (const T*)in, in_stride, first,
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
