// Kernels of the block arrangement that normalises a sublayer's update before it joins the
// residual stream and lets every sublayer read its input through a short causal convolution.
//
//   add_normed_rmsnorm  one block per row: x = residual + update * rsqrt(mean(update^2) + eps) * w_update
//                       (written back unless told otherwise), out = x * rsqrt(mean(x^2) + eps) * w.
//                       Both norms and the sum are 32-bit; one rounding on store.  With a row map
//                       only the mapped rows are produced (the model's last norm on wanted rows).
//                       With a convolution's weights and state (a step in which every entry
//                       brings one token: row r is entry r) the row goes straight through the
//                       convolution below instead of being stored: the same arithmetic in the same
//                       order as the two kernels one after the other.
//   causal_conv_state   u_t = y_t + sum_j w[:, j] * y_(t - taps + 1 + j) per channel, over the tokens
//                       of every entry of the step.  The taps - 1 rows of y before an entry's first
//                       token come from the request's state row (zeros at a sequence's start), and
//                       the step's last taps - 1 rows are left there for the next step.  Tokens
//                       that read the state (an entry's first taps - 1) and the state's update are
//                       the work of one block per entry, so no block reads a state row that
//                       another writes; every other token has a block of its own that reads y alone.
//                       A token's result depends on the taps rows themselves only, never on how the
//                       sequence was cut into steps.
#include "common.cuh"

#define CONV_MAX_TAPS 8

// V: elements a thread takes at a time (4 where the row's length is a multiple of 4; all rows
// then start on 16 bytes).  The order of additions depends on V and the row's length alone.
template <int V> __device__ __forceinline__ void sc_load(const float* p, float* v) { if constexpr (V == 4) load4(p, v); else v[0] = p[0]; }
template <int V> __device__ __forceinline__ void sc_load(const bf16* p, float* v) { if constexpr (V == 4) load4(p, v); else v[0] = to_float(p[0]); }
template <int V> __device__ __forceinline__ void sc_store(float* p, const float* v) { if constexpr (V == 4) store4(p, v); else p[0] = v[0]; }
template <int V> __device__ __forceinline__ void sc_store(bf16* p, const float* v) { if constexpr (V == 4) store4(p, v); else p[0] = from_float<bf16>(v[0]); }

template <typename TU, typename TO, int V>
__global__ void __launch_bounds__(256)
add_normed_rmsnorm_kernel(float* __restrict__ residual, const TU* __restrict__ update, const float* __restrict__ w_update,
                          const float* __restrict__ weight, TO* __restrict__ out, const int* __restrict__ row_map, int size,
                          float eps_update, float eps, int write_residual, const float* __restrict__ conv_w,
                          float* __restrict__ conv_state, long long state_stride, const int* __restrict__ slots, int taps) {
  extern __shared__ __align__(16) float row[];       // [size]
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = row_map ? row_map[r] : r;
  float* res = residual + (size_t)src * size;
  float ss = 0.f;
  if (update != nullptr) {
    const TU* upd = update + (size_t)src * size;
    float su = 0.f;
    for (int i = threadIdx.x * V; i < size; i += blockDim.x * V) {
      float u[V];
      sc_load<V>(upd + i, u);
#pragma unroll
      for (int k = 0; k < V; ++k) su = fmaf(u[k], u[k], su);
      sc_store<V>(row + i, u);
    }
    const float inv_u = 1.f / sqrtf(block_sum(su, scratch) / (float)size + eps_update);
    for (int i = threadIdx.x * V; i < size; i += blockDim.x * V) {
      float u[V], x[V], w[V];
      sc_load<V>(row + i, u), sc_load<V>(res + i, x), sc_load<V>(w_update + i, w);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        x[k] = x[k] + u[k] * inv_u * w[k];
        ss = fmaf(x[k], x[k], ss);
      }
      sc_store<V>(row + i, x);
      if (write_residual) sc_store<V>(res + i, x);
    }
  } else {
    for (int i = threadIdx.x * V; i < size; i += blockDim.x * V) {
      float x[V];
      sc_load<V>(res + i, x);
#pragma unroll
      for (int k = 0; k < V; ++k) ss = fmaf(x[k], x[k], ss);
      sc_store<V>(row + i, x);
    }
  }
  TO* dst = out + (size_t)r * size;
  if (weight == nullptr) {
    // no norm of the stream: the sublayer reads the sum itself
    __syncthreads();
    for (int i = threadIdx.x * V; i < size; i += blockDim.x * V) {
      float x[V];
      sc_load<V>(row + i, x);
      sc_store<V>(dst + i, x);
    }
    return;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)size + eps);
  if (conv_w != nullptr) {
    // the entry's one token through the convolution: taps - 1 rows from the state, then this one
    const int back = taps - 1;
    float* st = back > 0 ? conv_state + (size_t)slots[r] * state_stride : nullptr;
    for (int i = threadIdx.x * V; i < size; i += blockDim.x * V) {
      float y[V], w[V], sum[V], hist[CONV_MAX_TAPS][V];
      sc_load<V>(row + i, y), sc_load<V>(weight + i, w);
#pragma unroll
      for (int k = 0; k < V; ++k) y[k] = y[k] * inv * w[k], sum[k] = 0.f;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j < taps) {
          if (j < back) sc_load<V>(st + (size_t)j * size + i, hist[j]);
          else {
#pragma unroll
            for (int k = 0; k < V; ++k) hist[j][k] = y[k];
          }
          sc_load<V>(conv_w + (size_t)j * size + i, w);
#pragma unroll
          for (int k = 0; k < V; ++k) sum[k] = fmaf(w[k], hist[j][k], sum[k]);
        }
      }
#pragma unroll
      for (int k = 0; k < V; ++k) sum[k] = y[k] + sum[k];
      sc_store<V>(dst + i, sum);
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
        if (j < back) sc_store<V>(st + (size_t)j * size + i, hist[j + 1]);
    }
    return;
  }
  for (int i = threadIdx.x * V; i < size; i += blockDim.x * V) {
    float x[V], w[V];
    sc_load<V>(row + i, x), sc_load<V>(weight + i, w);
#pragma unroll
    for (int k = 0; k < V; ++k) x[k] = x[k] * inv * w[k];
    sc_store<V>(dst + i, x);
  }
}

// residual 32-bit [*, size]; update [*, size] or null; w_update, weight 32-bit [size] (as they
// multiply: any offset of a stored weight is already in them); out [rows, size].
// conv_w (or null) 32-bit [taps, size], conv_state and slots as causal_conv_state takes them:
// row r is then the one token of entry r, and out gets the convolution's result.
FE_EXPORT int fe_add_normed_rmsnorm(float* residual, const void* update, int update_dtype, const float* w_update,
                                    const float* weight, void* out, int out_dtype, const int* row_map, int rows, int size,
                                    float eps_update, float eps, int write_residual, const float* conv_w,
                                    float* conv_state, long long state_stride, const int* slots, int taps,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (size < 1) return FE_ERR_BAD_SHAPE;
  if (conv_w != nullptr && (taps < 1 || taps > CONV_MAX_TAPS || row_map != nullptr || slots == nullptr ||
                            (taps > 1 && conv_state == nullptr)))
    return FE_ERR_BAD_SHAPE;
  const size_t smem = (size_t)size * sizeof(float);
  if (smem > 200 * 1024) return FE_ERR_TOO_LARGE;
  int threads = 64;
  while (threads < 256 && threads * 8 < size) threads <<= 1;
  int rc = FE_ERR_BAD_DTYPE;
  const bool wide = size % 4 == 0 && (state_stride % 4) == 0 &&
                    (((uintptr_t)residual | (uintptr_t)update | (uintptr_t)w_update | (uintptr_t)weight | (uintptr_t)out |
                      (uintptr_t)conv_w | (uintptr_t)conv_state) & 15) == 0;
#define LAUNCH_V(TU, TO, V)                                                                                            \
  do {                                                                                                                 \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(add_normed_rmsnorm_kernel<TU, TO, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           (int)smem);                                                                                 \
    rc = fe_launch_dependent(add_normed_rmsnorm_kernel<TU, TO, V>, dim3(rows), dim3(threads), smem, stream, residual,  \
                             (const TU*)update, w_update, weight, (TO*)out, row_map, size, eps_update, eps,            \
                             write_residual, conv_w, conv_state, state_stride, slots, taps);                           \
  } while (0)
#define LAUNCH(TU, TO)                                                                                                 \
  do {                                                                                                                 \
    if (wide) LAUNCH_V(TU, TO, 4);                                                                                     \
    else LAUNCH_V(TU, TO, 1);                                                                                          \
  } while (0)
  if (update == nullptr) update_dtype = FE_DTYPE_F32;
  if (update_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32) LAUNCH(float, float);
  else if (update_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16) LAUNCH(float, bf16);
  else if (update_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_F32) LAUNCH(bf16, float);
  else if (update_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16) LAUNCH(bf16, bf16);
#undef LAUNCH
#undef LAUNCH_V
  return rc ? rc : fe_last_error();
}

// y 32-bit [tokens, width]; w 32-bit [taps, width] (tap j weighs the row taps - 1 - j tokens
// back); state 32-bit, row `slot` at state + slot * state_stride holds [taps - 1, width], oldest
// row first; out [tokens, width].
template <typename TO, int V>
__global__ void __launch_bounds__(256)
causal_conv_state_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ state,
                         long long state_stride, const int* __restrict__ slots, const int* __restrict__ cu_tokens,
                         const int* __restrict__ token_entry, TO* __restrict__ out, int n_tokens, int width, int taps) {
  pdl_trigger();
  pdl_wait();
  const int back = taps - 1;
  if ((int)blockIdx.x < n_tokens) {
    // a token with all its taps inside the step
    const int t = blockIdx.x;
    const int first = cu_tokens[token_entry[t]];
    if (t - first < back) return;
    for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
      float sum[V], own[V];
#pragma unroll
      for (int k = 0; k < V; ++k) sum[k] = 0.f;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j < taps) {
          float wj[V];
          sc_load<V>(w + (size_t)j * width + c, wj), sc_load<V>(y + (size_t)(t - back + j) * width + c, own);
#pragma unroll
          for (int k = 0; k < V; ++k) sum[k] = fmaf(wj[k], own[k], sum[k]);
        }
      }
      // the last tap read the token's own row
#pragma unroll
      for (int k = 0; k < V; ++k) sum[k] = own[k] + sum[k];
      sc_store<V>(out + (size_t)t * width + c, sum);
    }
    return;
  }
  // an entry's edge: its first taps - 1 tokens, then the state for the next step
  const int entry = blockIdx.x - n_tokens;
  const int first = cu_tokens[entry], count = cu_tokens[entry + 1] - first;
  if (count <= 0 || back <= 0) return;
  float* st = state + (size_t)slots[entry] * state_stride;
  const int edge = min(count, back);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    // hist[k], k < back: the state's rows; hist[back + i]: y of the entry's token i (i < edge)
    float hist[2 * CONV_MAX_TAPS];
    float wc[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
      wc[j] = j < taps ? w[(size_t)j * width + c] : 0.f;
      hist[j] = j < back ? st[(size_t)j * width + c] : 0.f;
      hist[CONV_MAX_TAPS + j] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i)
      if (i < edge) hist[back + i] = y[(size_t)(first + i) * width + c];
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS; ++i) {
      if (i < edge) {
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
          if (j < taps) sum = fmaf(wc[j], hist[i + j], sum);
        out[(size_t)(first + i) * width + c] = from_float<TO>(hist[back + i] + sum);
      }
    }
    // the last taps - 1 rows of (state rows, the step's y rows)
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k) {
      if (k < back) {
        const int at = count + k;          // index into that sequence
        st[(size_t)k * width + c] = at < back + edge ? hist[at] : y[(size_t)(first + at - back) * width + c];
      }
    }
  }
}

FE_EXPORT int fe_causal_conv_state(const float* y, const float* w, float* state, long long state_stride, const int* slots,
                                   const int* cu_tokens, const int* token_entry, void* out, int out_dtype, int n_tokens,
                                   int n_entries, int width, int taps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS || width < 1) return FE_ERR_BAD_SHAPE;
  if (taps > 1 && state == nullptr) return FE_ERR_BAD_SHAPE;
  int threads = 64;
  while (threads < 256 && threads * 4 < width) threads <<= 1;
  const dim3 grid(n_tokens + (taps > 1 ? n_entries : 0));
  const bool wide = width % 4 == 0 && (((uintptr_t)y | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
  int rc;
#define LAUNCH(TO, V)                                                                                                  \
  rc = fe_launch_dependent(causal_conv_state_kernel<TO, V>, grid, dim3(threads), 0, stream, y, w, state, state_stride, \
                           slots, cu_tokens, token_entry, (TO*)out, n_tokens, width, taps)
  if (out_dtype == FE_DTYPE_F32) { if (wide) LAUNCH(float, 4); else LAUNCH(float, 1); }
  else if (out_dtype == FE_DTYPE_BF16) { if (wide) LAUNCH(bf16, 4); else LAUNCH(bf16, 1); }
  else return FE_ERR_BAD_DTYPE;
#undef LAUNCH
  return rc ? rc : fe_last_error();
}
