// Attention over cache pages for layers the specialised kernels do not cover: keys and
// values of different sizes, one cached vector that is key and value at once (a latent),
// a bias on the distance between query and key, queries and outputs laid out with any
// strides.  Two kernels:
//
// qkv_prepare - one block per token and side (queries; keys and values): reads the token's projected q, k (and v), normalises
//   (per head over the head's leading elements, or over the whole projection at once, or not
//   at all), rotates a stretch of every head by the step's cosine/sine table, stores the
//   queries where the attention kernel wants them and k, v into their cache pages.
//   Everything between load and store is 32-bit.
//
// attention_general - one block per (token, kv head, group of up to 8 query heads that
//   share the kv head).  Keys [lo, pos] are cut into chunks of 32 from lo; warp w takes
//   chunks w, w + 4, ...; a lane owns one key of the chunk for the scores of all the
//   block's heads and value columns lane, lane + 32, ... for the weighted sum, so a key or
//   value row is read once for all heads of the block.  Scores, softmax and sums are 32-bit;
//   the four warps' partial results are merged in a fixed order.  A row's result does not
//   depend on what else is in the batch.
#include "attention_common.cuh"

#define GA_WARPS 4

// ---------------------------------------------------------------------------
// qkv_prepare
// ---------------------------------------------------------------------------
#define PREP_NORM_NONE 0
#define PREP_NORM_HEAD 1     // every head over its first norm_dims elements, weight [norm_dims]
#define PREP_NORM_WHOLE 2    // all heads at once, weight [heads * dim]
#define PREP_NORM_HEAD_AFTER 3   // like PREP_NORM_HEAD, but taken of the rotated head (the rotation comes first)
// A null weight in the per-head modes divides by the root mean square and multiplies by nothing.

struct PrepSide {
  const void* in;      // token t's head h starts at in + t * in_stride + h * head_stride (elements)
  int in_stride;
  int head_stride;
  int heads;
  int dim;             // elements per head
  int norm_mode;
  int norm_dims;       // PREP_NORM_HEAD: leading elements of a head that are normalised
  const float* norm_w;
  int rot_off;         // first rotated element of a head; negative: this side is not rotated
};

__device__ __forceinline__ void prep_norm_rotate(float* row, const PrepSide& s, float eps, const float2* angles,
                                                 int rot_dims, int interleaved, float* scratch) {
  const int total = s.heads * s.dim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const bool rotates = angles != nullptr && rot_dims > 0 && s.rot_off >= 0;
  auto rotate = [&]() {
    const int half = rot_dims >> 1;
    for (int p = threadIdx.x; p < s.heads * half; p += blockDim.x) {
      const int h = p / half, j = p - h * half;
      float* x = row + h * s.dim + s.rot_off;
      const int a = interleaved ? 2 * j : j, b = interleaved ? 2 * j + 1 : j + half;
      const float2 cs = angles[j];
      const float u = x[a], v = x[b];
      x[a] = u * cs.x - v * cs.y;
      x[b] = v * cs.x + u * cs.y;
    }
  };
  auto norm_heads = [&]() {
    for (int h = warp; h < s.heads; h += warps) {
      float* x = row + h * s.dim;
      float ss = 0.f;
      for (int i = lane; i < s.norm_dims; i += 32) ss = fmaf(x[i], x[i], ss);
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)s.norm_dims + eps);
      if (s.norm_w != nullptr) {
        for (int i = lane; i < s.norm_dims; i += 32) x[i] = x[i] * inv * s.norm_w[i];
      } else {
        for (int i = lane; i < s.norm_dims; i += 32) x[i] = x[i] * inv;
      }
    }
  };
  if (s.norm_mode == PREP_NORM_HEAD_AFTER) {
    if (rotates) {
      rotate();
      __syncthreads();
    }
    norm_heads();
    __syncthreads();
    return;
  }
  if (s.norm_mode == PREP_NORM_WHOLE) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < total; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)total + eps);
    for (int i = threadIdx.x; i < total; i += blockDim.x) row[i] = row[i] * inv * s.norm_w[i];
  } else if (s.norm_mode == PREP_NORM_HEAD) {
    norm_heads();
  }
  __syncthreads();
  if (rotates) rotate();
  __syncthreads();
}

template <typename TI, typename TC>
__global__ void __launch_bounds__(256)
qkv_prepare_kernel(PrepSide q, PrepSide k, const TI* __restrict__ v_in, int v_in_stride, int v_dim, float eps,
                   const float2* __restrict__ table, int rot_dims, int interleaved, TC* __restrict__ q_out,
                   long long q_out_token_stride, long long q_out_head_stride, int q_out_dim_offset,
                   TC* __restrict__ k_cache, TC* __restrict__ v_cache, const int* __restrict__ block_table,
                   int max_pages, int page_size, int num_pages, const int* __restrict__ positions,
                   const int* __restrict__ token_entry, int* status) {
  extern __shared__ float rows[];           // q row, then k row
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  // with both sides present a token has two blocks: one for the queries, one for keys and values
  const bool do_q = q.in != nullptr && (gridDim.y == 1 ? true : blockIdx.y == 0);
  const bool do_k = k.in != nullptr && (gridDim.y == 1 ? true : blockIdx.y == 1);
  const int q_total = q.in ? q.heads * q.dim : 0, k_total = k.in ? k.heads * k.dim : 0;
  float* q_row = rows;
  float* k_row = rows + (gridDim.y == 1 ? q_total : 0);
  const float2* angles = table ? table + (size_t)token * (rot_dims >> 1) : nullptr;
  if (do_q) {
    const TI* src = (const TI*)q.in + (size_t)token * q.in_stride;
    for (int i = threadIdx.x; i < q_total; i += blockDim.x) {
      const int h = i / q.dim;
      q_row[i] = to_float(src[(size_t)h * q.head_stride + (i - h * q.dim)]);
    }
  }
  if (do_k) {
    const TI* src = (const TI*)k.in + (size_t)token * k.in_stride;
    for (int i = threadIdx.x; i < k_total; i += blockDim.x) {
      const int h = i / k.dim;
      k_row[i] = to_float(src[(size_t)h * k.head_stride + (i - h * k.dim)]);
    }
  }
  __syncthreads();
  if (do_q) {
    prep_norm_rotate(q_row, q, eps, angles, rot_dims, interleaved, scratch);
    TC* dst = q_out + (size_t)token * q_out_token_stride + q_out_dim_offset;
    for (int i = threadIdx.x; i < q_total; i += blockDim.x) {
      const int h = i / q.dim, d = i - h * q.dim;
      dst[(size_t)h * q_out_head_stride + d] = from_float<TC>(q_row[i]);
    }
  }
  if (!do_k) return;
  prep_norm_rotate(k_row, k, eps, angles, rot_dims, interleaved, scratch);
  const int pos = positions[token], entry = token_entry[token];
  const int logical = pos / page_size;
  if (pos < 0 || logical >= max_pages) {
    if (threadIdx.x == 0) atomicOr(status, FE_STATUS_BAD_POSITION);
    return;
  }
  const int page = block_table[(size_t)entry * max_pages + logical];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, FE_STATUS_BAD_PAGE);
    return;
  }
  const int slot = pos - logical * page_size;
  for (int i = threadIdx.x; i < k_total; i += blockDim.x) {
    const int h = i / k.dim, d = i - h * k.dim;
    k_cache[(((size_t)page * k.heads + h) * page_size + slot) * k.dim + d] = from_float<TC>(k_row[i]);
  }
  if (v_in != nullptr && v_cache != nullptr) {
    const TI* src = v_in + (size_t)token * v_in_stride;
    for (int i = threadIdx.x; i < k.heads * v_dim; i += blockDim.x) {
      const int h = i / v_dim, d = i - h * v_dim;
      v_cache[(((size_t)page * k.heads + h) * page_size + slot) * v_dim + d] = from_float<TC>(to_float(src[i]));
    }
  }
}

FE_EXPORT int fe_qkv_prepare(const void* q_in, int q_in_stride, int q_head_stride, int q_heads, int q_dim, int q_norm_mode, int q_norm_dims,
                             const float* q_norm_w, int q_rot_off, const void* k_in, int k_in_stride, int k_heads,
                             int k_dim, int k_norm_mode, int k_norm_dims, const float* k_norm_w, int k_rot_off,
                             const void* v_in, int v_in_stride, int v_dim, int in_dtype, float eps, const float* table,
                             int rot_dims, int interleaved, void* q_out, long long q_out_token_stride,
                             long long q_out_head_stride, int q_out_dim_offset, void* k_cache, void* v_cache,
                             int cache_dtype, const int* block_table, int max_pages, int page_size, int num_pages,
                             const int* positions, const int* token_entry, int n_tokens, int* status,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (rot_dims % 2 || (q_in && q_rot_off >= 0 && q_rot_off + rot_dims > q_dim) || (k_in && k_rot_off >= 0 && k_rot_off + rot_dims > k_dim)) return FE_ERR_BAD_SHAPE;
  PrepSide q{q_in, q_in_stride, q_head_stride > 0 ? q_head_stride : q_dim, q_heads, q_dim, q_norm_mode, q_norm_dims, q_norm_w, q_rot_off};
  PrepSide k{k_in, k_in_stride, k_dim, k_heads, k_dim, k_norm_mode, k_norm_dims, k_norm_w, k_rot_off};
  const size_t q_floats = q_in ? (size_t)q_heads * q_dim : 0, k_floats = k_in ? (size_t)k_heads * k_dim : 0;
  const int sides = (q_in && k_in) ? 2 : 1;
  const size_t smem = sizeof(float) * (q_floats > k_floats ? q_floats : k_floats);
  if (smem > 200 * 1024) return FE_ERR_TOO_LARGE;
  int rc = 0;
#define LAUNCH(TI, TC)                                                                                              \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(qkv_prepare_kernel<TI, TC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    rc = fe_launch_dependent(qkv_prepare_kernel<TI, TC>, dim3(n_tokens, sides), dim3(256), smem, stream, q, k,             \
                             (const TI*)v_in, v_in_stride, v_dim, eps, (const float2*)table, rot_dims, interleaved, \
                             (TC*)q_out, q_out_token_stride, q_out_head_stride, q_out_dim_offset, (TC*)k_cache,     \
                             (TC*)v_cache, block_table, max_pages, page_size, num_pages, positions, token_entry,    \
                             status);                                                                               \
  } while (0)
  if (in_dtype == FE_DTYPE_F32 && cache_dtype == FE_DTYPE_F32) LAUNCH(float, float);
  else if (in_dtype == FE_DTYPE_F32 && cache_dtype == FE_DTYPE_BF16) LAUNCH(float, bf16);
  else if (in_dtype == FE_DTYPE_BF16 && cache_dtype == FE_DTYPE_BF16) LAUNCH(bf16, bf16);
  else return FE_ERR_BAD_DTYPE;
#undef LAUNCH
  return rc ? rc : fe_last_error();
}

// ---------------------------------------------------------------------------
// attention_general
// ---------------------------------------------------------------------------
struct GeneralAttn {
  const void* q;            // row (token, head) starts at q + token * q_token_stride + head * q_head_stride
  long long q_token_stride, q_head_stride;
  const void* k;            // [pages, kv_heads, page_size, k_row]; the first k_dim elements are the key
  int k_row, k_dim;
  const void* v;            // [pages, kv_heads, page_size, v_row]; the first v_dim elements are the value
  int v_row, v_dim;
  void* out;                // like q
  long long o_token_stride, o_head_stride;
  const int* block_table;
  int max_pages, page_size, num_pages, num_kv_heads, num_q_heads;
  const int* positions;
  const int* token_entry;
  const float* slopes;      // per query head, or null: s -= slope * (pos - key)
  const float* dist_bias;   // or null: [heads, dist_len], s += dist_bias[head, min(pos - key, dist_len - 1)]
  int dist_len;
  int window;
  float scale;
  // What the plain layer does not have (all off when zero / null):
  int keep_first;           // with a window: keys below this position stay visible to every query
  float softcap;            // s <- softcap * tanh(s / softcap), before the bias
  float temp_coef;          // scores of a query at position p are multiplied by
  int temp_every;           //   1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)
  int parts;                // score maps per head over shared values (1: the plain layer): part m of
  long long q_part_stride;  //   a head reads its query q_part_stride * m elements further on, its key
  int k_part_stride;        //   k_part_stride * m elements into the cached row, and writes
  long long o_part_stride;  //   o_part_stride * m elements further on
  const float* gate;        // or null: the row (token, head) is multiplied by sigmoid(gate[token * gate_stride + head])
  long long gate_stride;
  int out_f32;              // the output is 32-bit whatever the cache holds
  const float* sinks;       // or null: per query head a number whose exponential joins the softmax's
                            //   denominator once (unscaled, uncapped), with no key and no value
};

// 1 + coef * ln(floor((p + 1) / every) + 1): what a query's scores are multiplied by
__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
  return every > 0 ? 1.f + coef * logf((float)((pos + 1) / every + 1)) : 1.f;
}

template <typename T, int RMAX, int NV>
__global__ void __launch_bounds__(GA_WARPS * 32)
attention_general_kernel(GeneralAttn a, int* status) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int groups = a.num_q_heads / a.num_kv_heads;
  const int token = blockIdx.x, kvh = blockIdx.y / a.parts, part = blockIdx.y - kvh * a.parts;
  const int first = blockIdx.z * RMAX;                  // first of this block's heads inside the kv head's group
  const int R = min(RMAX, groups - first);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = smem;                                     // [RMAX][k_dim]
  float* part_acc = qs + RMAX * a.k_dim;                // [GA_WARPS][RMAX][v_dim]
  float* part_m = part_acc + GA_WARPS * RMAX * a.v_dim; // [GA_WARPS][RMAX]
  float* part_l = part_m + GA_WARPS * RMAX;
  const int pos = a.positions[token], entry = a.token_entry[token];
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int* table = a.block_table + (size_t)entry * a.max_pages;
  const int head0 = kvh * groups + first;

  for (int i = threadIdx.x; i < R * a.k_dim; i += blockDim.x) {
    const int r = i / a.k_dim, d = i - r * a.k_dim;
    qs[i] = to_float(((const T*)a.q)[(size_t)token * a.q_token_stride + (size_t)(head0 + r) * a.q_head_stride
                                     + (size_t)part * a.q_part_stride + d]);
  }
  __syncthreads();

  float slope[RMAX];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) slope[r] = (a.slopes && r < R) ? a.slopes[head0 + r] : 0.f;
  float acc[RMAX][NV];
  float m[RMAX], l[RMAX];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[r][i] = 0.f;
  }

  const int n_keys = pos - lo + 1;
  // keys the window has passed but that stay visible: [0, n_sink), in chunks of their own ahead of the rest
  const int n_sink = a.window > 0 ? min(a.keep_first, lo) : 0;
  const int sink_chunks = (n_sink + 31) >> 5;
  const int n_chunks = sink_chunks + ((n_keys + 31) >> 5);
  const float row_scale = a.scale * query_temperature(pos, a.temp_coef, a.temp_every);
  const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
  const bool vec = (a.k_row % 8) == 0 && (a.k_dim % 8) == 0 && (a.k_part_stride % 8) == 0 && ((uintptr_t)a.k % 32) == 0;
  for (int c = warp; c < n_chunks; c += GA_WARPS) {
    const bool sink = c < sink_chunks;
    const int key = sink ? (c << 5) + lane : lo + ((c - sink_chunks) << 5) + lane;
    bool valid = sink ? key < n_sink : key <= pos;
    long long row = -1;                                   // (page, head, slot) as a row index
    if (valid) {
      const int logical = key / a.page_size;
      int page = -1;
      if (logical < a.max_pages) page = table[logical];
      if (page < 0 || page >= a.num_pages) {
        atomicOr(status, FE_STATUS_BAD_PAGE);
        valid = false;
      } else {
        row = ((long long)page * a.num_kv_heads + kvh) * a.page_size + (key - logical * a.page_size);
      }
    }
    float s[RMAX];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) s[r] = 0.f;
    if (valid) {
      const T* kp = (const T*)a.k + row * a.k_row + part * a.k_part_stride;
      if (vec) {
        for (int d = 0; d < a.k_dim; d += 8) {
          float kk[8];
          load8(kp + d, kk);
#pragma unroll
          for (int r = 0; r < RMAX; ++r) {
            if (r < R) {
              const float* qr = qs + r * a.k_dim + d;
#pragma unroll
              for (int e = 0; e < 8; ++e) s[r] = fmaf(qr[e], kk[e], s[r]);
            }
          }
        }
      } else {
        for (int d = 0; d < a.k_dim; ++d) {
          const float kk = to_float(kp[d]);
#pragma unroll
          for (int r = 0; r < RMAX; ++r)
            if (r < R) s[r] = fmaf(qs[r * a.k_dim + d], kk, s[r]);
        }
      }
    }
    float p[RMAX];
    const float dist = (float)(pos - key);
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      float sc = s[r] * row_scale;
      if (a.softcap > 0.f) sc = a.softcap * tanhf(sc * inv_cap);
      sc = valid ? sc - slope[r] * dist : -INFINITY;
      if (a.dist_bias != nullptr && valid && r < R)
        sc += a.dist_bias[(size_t)(head0 + r) * a.dist_len + min(pos - key, a.dist_len - 1)];
      const float m_new = fmaxf(m[r], warp_max(sc));
      p[r] = valid ? expf(sc - m_new) : 0.f;
      const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
      l[r] = l[r] * corr + warp_sum(p[r]);
      m[r] = m_new;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[r][i] *= corr;
    }
    const int in_chunk = sink ? min(32, n_sink - (c << 5)) : min(32, n_keys - ((c - sink_chunks) << 5));
    for (int j = 0; j < in_chunk; ++j) {
      const long long rj = __shfl_sync(0xffffffffu, row, j);
      float pj[RMAX];
#pragma unroll
      for (int r = 0; r < RMAX; ++r) pj[r] = __shfl_sync(0xffffffffu, p[r], j);
      if (rj < 0) continue;
      const T* vp = (const T*)a.v + rj * a.v_row;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int d = lane + (i << 5);
        if (d < a.v_dim) {
          const float vv = to_float(vp[d]);
#pragma unroll
          for (int r = 0; r < RMAX; ++r) acc[r][i] = fmaf(pj[r], vv, acc[r][i]);
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    if (lane == 0) { part_m[warp * RMAX + r] = m[r]; part_l[warp * RMAX + r] = l[r]; }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = lane + (i << 5);
      if (d < a.v_dim) part_acc[((size_t)warp * RMAX + r) * a.v_dim + d] = acc[r][i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R * a.v_dim; i += blockDim.x) {
    const int r = i / a.v_dim, d = i - r * a.v_dim;
    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < GA_WARPS; ++w) big = fmaxf(big, part_m[w * RMAX + r]);
    const float sink = a.sinks ? a.sinks[head0 + r] : -INFINITY;
    big = fmaxf(big, sink);
    float num = 0.f, den = a.sinks ? expf(sink - big) : 0.f;
#pragma unroll
    for (int w = 0; w < GA_WARPS; ++w) {
      const float pm = part_m[w * RMAX + r];
      const float f = (pm == -INFINITY) ? 0.f : expf(pm - big);
      num = fmaf(part_acc[((size_t)w * RMAX + r) * a.v_dim + d], f, num);
      den = fmaf(part_l[w * RMAX + r], f, den);
    }
    float value = den > 0.f ? num / den : 0.f;
    if (a.gate) value *= 1.f / (1.f + expf(-a.gate[(size_t)token * a.gate_stride + head0 + r]));
    const size_t at = (size_t)token * a.o_token_stride + (size_t)(head0 + r) * a.o_head_stride + (size_t)part * a.o_part_stride + d;
    if (a.out_f32) ((float*)a.out)[at] = value;
    else ((T*)a.out)[at] = from_float<T>(value);
  }
}

template <typename T, int RMAX, int NV>
static int launch_general(const GeneralAttn& a, int n_tokens, int* status, cudaStream_t stream) {
  const int groups = a.num_q_heads / a.num_kv_heads;
  dim3 grid(n_tokens, a.num_kv_heads * a.parts, (groups + RMAX - 1) / RMAX);
  const size_t smem = sizeof(float) * ((size_t)RMAX * a.k_dim + (size_t)GA_WARPS * RMAX * a.v_dim + 2 * GA_WARPS * RMAX);
  if (smem > 200 * 1024) return FE_ERR_TOO_LARGE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(attention_general_kernel<T, RMAX, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int rc = fe_launch_dependent(attention_general_kernel<T, RMAX, NV>, grid, dim3(GA_WARPS * 32), smem, stream, a, status);
  return rc ? rc : fe_last_error();
}

template <typename T>
static int dispatch_general(const GeneralAttn& a, int n_tokens, int* status, cudaStream_t stream) {
  const int groups = a.num_q_heads / a.num_kv_heads;
  const int nv = (a.v_dim + 31) / 32;
  if (nv <= 1) {
    if (groups >= 8) return launch_general<T, 8, 1>(a, n_tokens, status, stream);
    if (groups >= 4) return launch_general<T, 4, 1>(a, n_tokens, status, stream);
    if (groups >= 2) return launch_general<T, 2, 1>(a, n_tokens, status, stream);
    return launch_general<T, 1, 1>(a, n_tokens, status, stream);
  }
  if (nv <= 2) {
    if (groups >= 8) return launch_general<T, 8, 2>(a, n_tokens, status, stream);
    if (groups >= 4) return launch_general<T, 4, 2>(a, n_tokens, status, stream);
    if (groups >= 2) return launch_general<T, 2, 2>(a, n_tokens, status, stream);
    return launch_general<T, 1, 2>(a, n_tokens, status, stream);
  }
  if (nv <= 4) {
    if (groups >= 8) return launch_general<T, 8, 4>(a, n_tokens, status, stream);
    if (groups >= 4) return launch_general<T, 4, 4>(a, n_tokens, status, stream);
    if (groups >= 2) return launch_general<T, 2, 4>(a, n_tokens, status, stream);
    return launch_general<T, 1, 4>(a, n_tokens, status, stream);
  }
  if (nv <= 8) {
    if (groups >= 8) return launch_general<T, 8, 8>(a, n_tokens, status, stream);
    if (groups >= 4) return launch_general<T, 4, 8>(a, n_tokens, status, stream);
    if (groups >= 2) return launch_general<T, 2, 8>(a, n_tokens, status, stream);
    return launch_general<T, 1, 8>(a, n_tokens, status, stream);
  }
  if (nv <= 16) {
    if (groups >= 4) return launch_general<T, 4, 16>(a, n_tokens, status, stream);
    if (groups >= 2) return launch_general<T, 2, 16>(a, n_tokens, status, stream);
    return launch_general<T, 1, 16>(a, n_tokens, status, stream);
  }
  if (nv <= 32) {
    if (groups >= 2) return launch_general<T, 2, 32>(a, n_tokens, status, stream);
    return launch_general<T, 1, 32>(a, n_tokens, status, stream);
  }
  return FE_ERR_BAD_SHAPE;
}

FE_EXPORT int fe_attention_general(const void* q, long long q_token_stride, long long q_head_stride, const void* k_cache,
                                   int k_row, int k_dim, const void* v_cache, int v_row, int v_dim, void* out,
                                   long long o_token_stride, long long o_head_stride, int dtype, const int* block_table,
                                   int max_pages, int page_size, int num_pages, int num_kv_heads, int num_q_heads,
                                   const int* positions, const int* token_entry, const float* slopes,
                                   const float* dist_bias, int dist_len, int window,
                                   float scale, int keep_first, float softcap, float temp_coef, int temp_every,
                                   int parts, long long q_part_stride, int k_part_stride, long long o_part_stride,
                                   const float* gate, long long gate_stride, int out_f32, const float* sinks,
                                   int n_tokens, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (parts < 1) parts = 1;
  if (num_kv_heads < 1 || num_q_heads % num_kv_heads || (long long)num_kv_heads * parts > 65535) return FE_ERR_BAD_SHAPE;
  if (k_dim < 1 || v_dim < 1 || k_part_stride * (parts - 1) + k_dim > k_row || v_dim > v_row) return FE_ERR_BAD_SHAPE;
  if (keep_first < 0 || temp_every < 0 || softcap < 0.f || (dist_bias != nullptr && dist_len < 1)) return FE_ERR_BAD_SHAPE;
  GeneralAttn a{q, q_token_stride, q_head_stride, k_cache, k_row, k_dim, v_cache, v_row, v_dim, out, o_token_stride,
                o_head_stride, block_table, max_pages, page_size, num_pages, num_kv_heads, num_q_heads, positions,
                token_entry, slopes, dist_bias, dist_len, window, scale, keep_first, softcap, temp_coef, temp_every, parts, q_part_stride,
                k_part_stride, o_part_stride, gate, gate_stride, out_f32, sinks};
  if (dtype == FE_DTYPE_F32) return dispatch_general<float>(a, n_tokens, status, stream);
  if (dtype == FE_DTYPE_BF16) return dispatch_general<bf16>(a, n_tokens, status, stream);
  return FE_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------
// differential_combine: a head's two attention maps a1, a2 (32-bit, side by side:
// [rows, 2, dv]) become o = a1 - lambda * a2, divided by its root mean square over the
// head's dv values (eps inside the root) and multiplied by `mult`.  One warp per row
// (token, head); everything 32-bit, one rounding on store.
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void __launch_bounds__(128)
differential_combine_kernel(const float* __restrict__ maps, TO* __restrict__ out, long long rows, int dv,
                            float lambda, float eps, float mult) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* a1 = maps + row * 2 * dv;
  const float* a2 = a1 + dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) {
    const float o = a1[d] - lambda * a2[d];
    ss = fmaf(o, o, ss);
  }
  const float inv = mult / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int d = lane; d < dv; d += 32) out[row * dv + d] = from_float<TO>((a1[d] - lambda * a2[d]) * inv);
}

FE_EXPORT int fe_differential_combine(const float* maps, void* out, int out_dtype, long long rows, int dv, float lambda,
                                      float eps, float mult, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dv < 1) return FE_ERR_BAD_SHAPE;
  const long long blocks = (rows + 3) / 4;
  if (blocks > 0x7fffffffLL) return FE_ERR_TOO_LARGE;
  int rc;
  if (out_dtype == FE_DTYPE_F32)
    rc = fe_launch_dependent(differential_combine_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, maps, (float*)out, rows, dv, lambda, eps, mult);
  else if (out_dtype == FE_DTYPE_BF16)
    rc = fe_launch_dependent(differential_combine_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, stream, maps, (bf16*)out, rows, dv, lambda, eps, mult);
  else return FE_ERR_BAD_DTYPE;
  return rc ? rc : fe_last_error();
}
