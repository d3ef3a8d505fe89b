// Differential attention for steps that bring portions of prompts: bfloat16, tensor cores.
//
// The same function as diff_attention.cu (two softmax maps per head over one set of values,
// a1 - lambda * a2, unit root mean square per head, a scale), tiled: a block takes 64 consecutive
// query positions of one request and one query head (four warps of 16 rows), and walks the keys
// its rows can see in tiles of 64, fetched from the paged cache by cp.async into a ring of two
// stages (a key row holds both maps' keys, a value row serves both maps).  Per tile and map:
// S = Q_m K_m^T by mma.sync m16n8k16 (bf16 in, fp32 out), scale and mask (causal, window) in fp32,
// running maximum and sum in fp32, P rounded to bfloat16 as the A operand of O_m += P V (the value
// fragments come transposed out of shared memory by ldmatrix).  The two accumulators are combined,
// normed and written at the end.
//
// Which rows a block takes is found on the device: tile b of the grid is the b-th tile of 64 rows
// in request order (a request of n positions has ceil(n / 64) tiles); the grid holds an upper bound
// of tiles and the blocks beyond the last one return.
//
// Sizes: dim and vdim multiples of 16, both at most 128; any page size; any grouping of heads.
#include "common.cuh"

#define DA_ROWS 64
#define DA_KEYS 64
#define DA_THREADS 128
#define DA_PAD 8  // elements between rows of a tile in shared memory: row starts fall on different banks

__device__ __forceinline__ void da_cp16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // zero bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void da_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void da_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void da_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the hardware unit (two units in the last place of fp32; -inf gives 0)
__device__ __forceinline__ float da_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ unsigned da_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <int KMAX, int VMAX>
__global__ void __launch_bounds__(DA_THREADS)
diff_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ out,
                          long long out_stride, const __nv_bfloat16* __restrict__ k_pages,
                          const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                          int table_stride, const int* __restrict__ query_start, const int* __restrict__ context_lens,
                          int num_seqs, int page_size, int num_heads, int num_kv_heads, int dim, int vdim, int window,
                          float scale, float lambda, float eps, float out_scale, int* __restrict__ status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int tile_info[3];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int head = blockIdx.y;
  const int kv_head = head / (num_heads / num_kv_heads);
  if (tid == 0) {
    int left = blockIdx.x, found = -1, first_row = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = query_start[s + 1] - query_start[s];
      const int tiles = (n + DA_ROWS - 1) / DA_ROWS;
      if (left < tiles) {
        found = s;
        first_row = left * DA_ROWS;
        break;
      }
      left -= tiles;
    }
    tile_info[0] = found;
    tile_info[1] = first_row;
  }
  __syncthreads();
  const int seq = tile_info[0];
  if (seq < 0) return;
  const int seq_begin = query_start[seq], seq_rows = query_start[seq + 1] - seq_begin;
  const int row0 = tile_info[1];
  const int rows = min(DA_ROWS, seq_rows - row0);
  const int token0 = seq_begin + row0;
  const int pos0 = context_lens[seq] - seq_rows + row0;  // position of the tile's first row
  const int pos_last = pos0 + rows - 1;
  const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int key_begin = (lo / DA_KEYS) * DA_KEYS;
  const int num_tiles = (pos_last - key_begin) / DA_KEYS + 1;
  const int* table = block_table + (size_t)seq * table_stride;

  const int kdim = 2 * dim;
  const int k_ld = kdim + DA_PAD, v_ld = vdim + DA_PAD;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [64][k_ld]
  __nv_bfloat16* k_s = q_s + DA_ROWS * k_ld;                          // [2][64][k_ld]
  __nv_bfloat16* v_s = k_s + 2 * DA_KEYS * k_ld;                      // [2][64][v_ld]

  // the queries of the tile, once
  {
    const int chunks = kdim / 8;
    for (int i = tid; i < DA_ROWS * chunks; i += DA_THREADS) {
      const int r = i / chunks, c = i % chunks;
      const bool valid = r < rows;
      const __nv_bfloat16* src = q + (size_t)(token0 + (valid ? r : 0)) * q_stride + (size_t)head * kdim + c * 8;
      da_cp16(q_s + r * k_ld + c * 8, src, valid);
    }
  }
  // two threads bring a key's row and its value row: one page lookup and one address a thread and tile
  auto fetch = [&](int tile, int stage) {
    const int key0 = key_begin + tile * DA_KEYS;
    const int k_chunks = kdim / 8, v_chunks = vdim / 8;
    const int r = tid >> 1, half = tid & 1;
    const int key = key0 + r;
    int page = -1;
    if (key <= pos_last) {
      page = table[key / page_size];
      if (page < 0 && key >= lo && status) atomicOr(status, 4);
    }
    const bool valid = page >= 0;
    const size_t slot = valid ? ((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head : 0;
    __nv_bfloat16* ks = k_s + (stage * DA_KEYS + r) * k_ld;
    __nv_bfloat16* vs = v_s + (stage * DA_KEYS + r) * v_ld;
    const __nv_bfloat16* k_src = k_pages + slot * kdim;
    const __nv_bfloat16* v_src = v_pages + slot * vdim;
    for (int c = half; c < k_chunks; c += 2) da_cp16(ks + c * 8, k_src + c * 8, valid);
    for (int c = half; c < v_chunks; c += 2) da_cp16(vs + c * 8, v_src + c * 8, valid);
  };
  fetch(0, 0);
  da_commit();

  float acc[2][VMAX][4];
  float top[2][2], sum[2][2];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
#pragma unroll
    for (int i = 0; i < VMAX; ++i) acc[m][i][0] = acc[m][i][1] = acc[m][i][2] = acc[m][i][3] = 0.0f;
    top[m][0] = top[m][1] = -INFINITY;
    sum[m][0] = sum[m][1] = 0.0f;
  }
  const int k16 = dim / 16, v16 = vdim / 16;
  const float scale_log2 = scale * 1.44269504088896340736f;
  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  const int my_pos[2] = {pos0 + my_row[0], pos0 + my_row[1]};

  for (int tile = 0; tile < num_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < num_tiles) fetch(tile + 1, stage ^ 1);
    da_commit();
    da_wait<1>();
    __syncthreads();
    const __nv_bfloat16* ks = k_s + stage * DA_KEYS * k_ld;
    const __nv_bfloat16* vs = v_s + stage * DA_KEYS * v_ld;
    const int key0 = key_begin + tile * DA_KEYS;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float s[DA_KEYS / 8][4];
#pragma unroll
      for (int n = 0; n < DA_KEYS / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < KMAX; ++kk) {
        if (kk < k16) {
          unsigned a[4];
          const __nv_bfloat16* qa = q_s + my_row[0] * k_ld + m * dim + kk * 16 + 2 * t4;
          a[0] = *reinterpret_cast<const unsigned*>(qa);
          a[1] = *reinterpret_cast<const unsigned*>(qa + 8 * k_ld);
          a[2] = *reinterpret_cast<const unsigned*>(qa + 8);
          a[3] = *reinterpret_cast<const unsigned*>(qa + 8 * k_ld + 8);
#pragma unroll
          for (int n = 0; n < DA_KEYS / 8; n += 2) {
            // four 8 x 8 pieces of the key tile: keys n * 8 .. + 15, this step's 16 elements
            const int piece = lane >> 3;
            const __nv_bfloat16* src = ks + (n * 8 + (piece >> 1) * 8 + (lane & 7)) * k_ld + m * dim + kk * 16 + (piece & 1) * 8;
            unsigned b0, b1, b2, b3;
            const unsigned addr = (unsigned)__cvta_generic_to_shared(src);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                         : "r"(addr));
            da_mma(s[n], a, b0, b1);
            da_mma(s[n + 1], a, b2, b3);
          }
        }
      }
      // scale (with log2 e folded in: the exponentials below are powers of two), mask, running maximum
      // and sum (rows g and g + 8 of the warp's 16); a tile that every row of the block sees whole
      // needs no mask
      // the running maximum is kept of the raw products (the scale is positive: the launch refuses others),
      // and scale * log2(e) goes into the exponent's one multiply-add
      float tile_top[2] = {-INFINITY, -INFINITY};
      const bool whole = key0 + DA_KEYS - 1 <= pos0 && (window <= 0 || pos0 + DA_ROWS - 1 - key0 < window);
      if (whole) {
#pragma unroll
        for (int n = 0; n < DA_KEYS / 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) tile_top[e >> 1] = fmaxf(tile_top[e >> 1], s[n][e]);
        }
      } else {
#pragma unroll
        for (int n = 0; n < DA_KEYS / 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int key = key0 + n * 8 + 2 * t4 + (e & 1);
            const bool seen = my_row[r] < rows && key <= my_pos[r] && (window <= 0 || my_pos[r] - key < window);
            if (!seen) s[n][e] = -INFINITY;
            tile_top[r] = fmaxf(tile_top[r], s[n][e]);
          }
        }
      }
      float corr[2], base[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_top[r] = fmaxf(tile_top[r], __shfl_xor_sync(0xffffffffu, tile_top[r], 1));
        tile_top[r] = fmaxf(tile_top[r], __shfl_xor_sync(0xffffffffu, tile_top[r], 2));
        const float next = fmaxf(top[m][r], tile_top[r]);
        base[r] = next == -INFINITY ? 0.0f : next * scale_log2;
        corr[r] = da_exp2(top[m][r] == -INFINITY ? -INFINITY : top[m][r] * scale_log2 - base[r]);
        top[m][r] = next;
      }
      float part[2] = {0.0f, 0.0f};
#pragma unroll
      for (int n = 0; n < DA_KEYS / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = da_exp2(fmaf(s[n][e], scale_log2, -base[e >> 1]));
          s[n][e] = p;
          part[e >> 1] += p;
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) sum[m][r] = sum[m][r] * corr[r] + part[r];
      // the maxima seldom move after a row's first tiles: nothing to rescale then
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
          acc[m][i][0] *= corr[0];
          acc[m][i][1] *= corr[0];
          acc[m][i][2] *= corr[1];
          acc[m][i][3] *= corr[1];
        }
      }
      // O_m += P V
#pragma unroll
      for (int kt = 0; kt < DA_KEYS / 16; ++kt) {
        unsigned a[4];
        a[0] = da_pack(s[2 * kt][0], s[2 * kt][1]);
        a[1] = da_pack(s[2 * kt][2], s[2 * kt][3]);
        a[2] = da_pack(s[2 * kt + 1][0], s[2 * kt + 1][1]);
        a[3] = da_pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
        for (int vt = 0; vt < VMAX / 2; ++vt) {
          if (vt < v16) {
            const int matrix = lane >> 3;
            const __nv_bfloat16* src = vs + (kt * 16 + (matrix & 1) * 8 + (lane & 7)) * v_ld + vt * 16 + (matrix >> 1) * 8;
            unsigned b0, b1, b2, b3;
            const unsigned addr = (unsigned)__cvta_generic_to_shared(src);
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                         : "r"(addr));
            da_mma(acc[m][2 * vt], a, b0, b1);
            da_mma(acc[m][2 * vt + 1], a, b2, b3);
          }
        }
      }
    }
    __syncthreads();  // the stage is free for the tile after next
  }
  da_wait<0>();

  // combine the maps, norm over the head, write
  float inv[2][2];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float total = sum[m][r];
      total += __shfl_xor_sync(0xffffffffu, total, 1);
      total += __shfl_xor_sync(0xffffffffu, total, 2);
      inv[m][r] = total > 0.0f ? 1.0f / total : 0.0f;
    }
  }
  float squares[2] = {0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < VMAX; ++i) {
    if (i < 2 * v16) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float o = acc[0][i][e] * inv[0][r] - lambda * (acc[1][i][e] * inv[1][r]);
        acc[0][i][e] = o;
        squares[r] = fmaf(o, o, squares[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    squares[r] += __shfl_xor_sync(0xffffffffu, squares[r], 1);
    squares[r] += __shfl_xor_sync(0xffffffffu, squares[r], 2);
    const float unit = out_scale / sqrtf(squares[r] / (float)vdim + eps);
    if (my_row[r] < rows) {
      __nv_bfloat16* dst = out + (size_t)(token0 + my_row[r]) * out_stride + (size_t)head * vdim + 2 * t4;
#pragma unroll
      for (int i = 0; i < VMAX; ++i) {
        if (i < 2 * v16)
          *reinterpret_cast<unsigned*>(dst + i * 8) = da_pack(acc[0][i][2 * r] * unit, acc[0][i][2 * r + 1] * unit);
      }
    }
  }
}

template <int KMAX, int VMAX>
static int diff_attention_mma_launch(const void* q, long long q_stride, void* out, long long out_stride,
                                     const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                                     const int* query_start, const int* context_lens, int num_tokens, int num_seqs,
                                     int page_size, int num_heads, int num_kv_heads, int dim, int vdim, int window,
                                     float scale, float lambda, float eps, float out_scale, int* status,
                                     cudaStream_t stream) {
  const size_t smem = ((size_t)3 * DA_ROWS * (2 * dim + DA_PAD) + (size_t)2 * DA_KEYS * (vdim + DA_PAD)) * sizeof(__nv_bfloat16);
  auto kernel = diff_attention_mma_kernel<KMAX, VMAX>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  const int tiles = (num_tokens + DA_ROWS - 1) / DA_ROWS + num_seqs;  // no request has more tiles than n / 64 + 1
  ts_launch(kernel, dim3(tiles, num_heads), dim3(DA_THREADS), smem, stream, (const __nv_bfloat16*)q, q_stride,
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
            table_stride, query_start, context_lens, num_seqs, page_size, num_heads, num_kv_heads, dim, vdim, window, scale,
            lambda, eps, out_scale, status);
  return ts_launch_status();
}

TS_EXPORT int ts_diff_attention_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                                    const int* query_start, const int* context_lens, int num_tokens, int num_seqs,
                                    int page_size, int num_heads, int num_kv_heads, int dim, int vdim, int window,
                                    float scale, float lambda, float eps, float out_scale, int* status,
                                    cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (dim < 16 || dim % 16 || vdim < 16 || vdim % 16 || dim > 128 || vdim > 128) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads || num_heads > 65535) return TS_ERR_SIZE;
  if (page_size < 1 || window < 0 || !(scale > 0.0f)) return TS_ERR_ARGUMENT;
  if (q_stride % 8 || out_stride % 2 || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
      ((uintptr_t)out & 3))
    return TS_ERR_ALIGN;
  if (dim <= 64 && vdim <= 64)
    return diff_attention_mma_launch<4, 8>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                                           query_start, context_lens, num_tokens, num_seqs, page_size, num_heads,
                                           num_kv_heads, dim, vdim, window, scale, lambda, eps, out_scale, status, stream);
  return diff_attention_mma_launch<8, 16>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                                          query_start, context_lens, num_tokens, num_seqs, page_size, num_heads,
                                          num_kv_heads, dim, vdim, window, scale, lambda, eps, out_scale, status, stream);
}
