// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
//   retention_scan   per request and head, over the step's positions in order:
//                        q_t, k_t = rotate(q_t), rotate(k_t) * key_scale        (fp32, angles p * f_i)
//                        S_t = decay_h S_{t-1} + k_t v_t^T                       (S: dim x vdim, fp32)
//                        y_t = S_t^T q_t
//                    The state of a request lives in its slot as [heads][vdim][dim] fp32; it is read once
//                    before the step's first position and written once after its last.  q, k and v are read
//                    as projected (any type); rotation, scaling and everything after are fp32.
//   head_norm_gate   out = y / rms_head(y) * silu(g): every head's y divided by its root mean square (eps
//                    inside the root, no weight), times the gate, rounded once.
//
// A block owns one (request, head, slice of value columns).  DS lanes share a value column, each holding
// RPT rows of the state in registers (rows dl * RPT .. + RPT - 1, padded with zeros beyond dim); the
// column's output is their partial sums added by shuffles in a fixed order.  Positions are staged eight at a
// time in shared memory, rotated as they are staged.  Every sum of a position has one order whatever the
// cut of the request into steps, so a position's output is the same bits decoded alone or inside a prompt.
#include "common.cuh"

#define RS_THREADS 128
#define RS_BATCH 8

template <typename T, int RPT>
__global__ void __launch_bounds__(RS_THREADS)
retention_scan_kernel(const T* __restrict__ qkv, long long stride, int q_first, int k_first, int v_first,
                      const float* __restrict__ decay, const float* __restrict__ inv_freq, int rot,
                      float amplitude, float key_scale, const int* __restrict__ positions,
                      const int* __restrict__ query_start, const int* __restrict__ slots,
                      float* __restrict__ state, float* __restrict__ y, int heads, int dim, int vdim, int ds) {
  extern __shared__ float rs_smem[];
  const int padded = ds * RPT;
  const int cols = RS_THREADS / ds;
  float* q_s = rs_smem;                           // [RS_BATCH][padded], row r of a thread at i * ds + dl
  float* k_s = q_s + RS_BATCH * padded;           // [RS_BATCH][padded]
  float* v_s = k_s + RS_BATCH * padded;           // [RS_BATCH][cols]
  const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int tid = threadIdx.x, dl = tid % ds, col = col0 + tid / ds;
  const int half = rot / 2;
  pdl_wait();
  pdl_trigger();
  const int first = query_start[seq], last = query_start[seq + 1];
  if (last <= first) return;
  const int slot = slots[seq];
  const float gamma = decay[head];
  const bool live = col < vdim;
  float* s_ptr = state + (((size_t)slot * heads + head) * vdim + (live ? col : 0)) * dim + dl * RPT;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) s[i] = (live && dl * RPT + i < dim) ? s_ptr[i] : 0.0f;

  for (int t0 = first; t0 < last; t0 += RS_BATCH) {
    const int count = min(RS_BATCH, last - t0);
    __syncthreads();
    // stage: rotated q and k (row r goes to (r % RPT) * ds + r / RPT), and the value columns of this block
    for (int idx = tid; idx < count * padded; idx += RS_THREADS) {
      const int p = idx / padded, r = idx % padded;
      float qv = 0.0f, kv = 0.0f;
      if (r < dim) {
        const T* row = qkv + (size_t)(t0 + p) * stride + (size_t)head * dim;
        qv = to_float(row[q_first + r]);
        kv = to_float(row[k_first + r]);
        if (r < rot) {
          const int i = r < half ? r : r - half;
          const int mate = r < half ? r + half : r - half;
          float sn, cs;
          sincosf((float)positions[t0 + p] * inv_freq[i], &sn, &cs);
          sn *= amplitude;
          cs *= amplitude;
          const float qm = to_float(row[q_first + mate]), km = to_float(row[k_first + mate]);
          // the pair (u, v) becomes (u cos - v sin, v cos + u sin)
          qv = r < half ? qv * cs - qm * sn : qv * cs + qm * sn;
          kv = r < half ? kv * cs - km * sn : kv * cs + km * sn;
        }
        kv *= key_scale;
      }
      const int at = p * padded + (r % RPT) * ds + r / RPT;
      q_s[at] = qv;
      k_s[at] = kv;
    }
    for (int idx = tid; idx < count * cols; idx += RS_THREADS) {
      const int p = idx / cols, c = idx % cols;
      v_s[idx] = col0 + c < vdim ? to_float(qkv[(size_t)(t0 + p) * stride + v_first + (size_t)head * vdim + col0 + c]) : 0.0f;
    }
    __syncthreads();
    for (int p = 0; p < count; ++p) {
      const float v = v_s[p * cols + tid / ds];
      const float* kp = k_s + p * padded + dl;
      const float* qp = q_s + p * padded + dl;
      float o = 0.0f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        s[i] = fmaf(gamma, s[i], kp[i * ds] * v);
        o = fmaf(s[i], qp[i * ds], o);
      }
      for (int offset = ds >> 1; offset > 0; offset >>= 1) o += __shfl_xor_sync(0xffffffffu, o, offset);
      if (dl == 0 && live) y[(size_t)(t0 + p) * heads * vdim + (size_t)head * vdim + col] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (dl * RPT + i < dim) s_ptr[i] = s[i];
  }
}

template <typename T>
static int launch_retention_scan(const void* qkv, long long stride, int q_first, int k_first, int v_first,
                                 const float* decay, const float* inv_freq, int rot, float amplitude,
                                 float key_scale, const int* positions, const int* query_start, const int* slots,
                                 float* state, float* y, int num_seqs, int heads, int dim, int vdim,
                                 cudaStream_t stream) {
  // rows a thread: 8 up to dim 32, 16 up to 128, 32 up to 256; DS (a power of two) lanes share a column
  const int rpt = dim <= 32 ? 8 : dim <= 128 ? 16 : 32;
  int ds = 1;
  while (ds * rpt < dim) ds <<= 1;
  if (ds > 32) return TS_ERR_SIZE;
  const int cols = RS_THREADS / ds;
  dim3 grid(num_seqs, heads, (vdim + cols - 1) / cols);
  const size_t smem = ((size_t)2 * RS_BATCH * ds * rpt + (size_t)RS_BATCH * cols) * sizeof(float);
#define RS_LAUNCH(R)                                                                                              \
  ts_launch(retention_scan_kernel<T, R>, grid, dim3(RS_THREADS), smem, stream, (const T*)qkv, stride, q_first,   \
            k_first, v_first, decay, inv_freq, rot, amplitude, key_scale, positions, query_start, slots, state, y, \
            heads, dim, vdim, ds)
  if (rpt == 8) RS_LAUNCH(8);
  else if (rpt == 16) RS_LAUNCH(16);
  else RS_LAUNCH(32);
#undef RS_LAUNCH
  return ts_launch_status();
}

TS_EXPORT int ts_retention_scan(int dtype, const void* qkv, long long stride, int q_first, int k_first, int v_first,
                                const float* decay, const float* inv_freq, int rot, float amplitude,
                                float key_scale, const int* positions, const int* query_start, const int* slots,
                                float* state, float* y, int num_seqs, int heads, int dim, int vdim,
                                cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (dim < 1 || dim > 256 || vdim < 1 || heads < 1 || heads > 65535 || rot < 0 || rot % 2 || rot > dim) return TS_ERR_SIZE;
  if (dtype == TS_F32)
    return launch_retention_scan<float>(qkv, stride, q_first, k_first, v_first, decay, inv_freq, rot, amplitude,
                                        key_scale, positions, query_start, slots, state, y, num_seqs, heads, dim, vdim,
                                        stream);
  if (dtype == TS_BF16)
    return launch_retention_scan<__nv_bfloat16>(qkv, stride, q_first, k_first, v_first, decay, inv_freq, rot,
                                                amplitude, key_scale, positions, query_start, slots, state, y,
                                                num_seqs, heads, dim, vdim, stream);
  return TS_ERR_DTYPE;
}

// One warp per (token, head).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long gate_stride,
                                      T* __restrict__ out, long long pairs, int heads, int vdim, float eps) {
  pdl_wait();
  pdl_trigger<1>();
  const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = pair / heads;
  const int head = (int)(pair % heads);
  const float* row = y + (size_t)pair * vdim;
  float sum_sq = 0.0f;
  for (int i = lane; i < vdim; i += 32) sum_sq = fmaf(row[i], row[i], sum_sq);
  sum_sq = warp_sum(sum_sq);
  const float inv = 1.0f / sqrtf(sum_sq / (float)vdim + eps);
  const T* g = gate + (size_t)t * gate_stride + (size_t)head * vdim;
  T* o = out + (size_t)pair * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float z = to_float(g[i]);
    o[i] = from_float<T>(row[i] * inv * (z / (1.0f + expf(-z))));
  }
}

TS_EXPORT int ts_head_norm_gate(int dtype, const float* y, const void* gate, long long gate_stride, void* out,
                                int num_tokens, int heads, int vdim, float eps, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (heads < 1 || vdim < 1) return TS_ERR_SIZE;
  const long long pairs = (long long)num_tokens * heads;
  const int warps = 8;
  const unsigned blocks = (unsigned)((pairs + warps - 1) / warps);
  if (dtype == TS_F32)
    ts_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(32 * warps), 0, stream, y, (const float*)gate, gate_stride,
              (float*)out, pairs, heads, vdim, eps);
  else if (dtype == TS_BF16)
    ts_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(32 * warps), 0, stream, y,
              (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, pairs, heads, vdim, eps);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
