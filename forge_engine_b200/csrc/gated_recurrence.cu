// Linear attention whose forget gate also decides what is written (a gated linear recurrence).
//
// Per head a 32-bit state S [dk, dv]:
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,      o_t = S_t^T q_t,
//     q = silu(zq),  f = l + (1 - l) sigmoid(zf + b),
// zq, zf, v being columns of one 32-bit projection, l a learned lower bound and b a bias per
// head and channel.  o_t is divided by its root mean square over the head's dv values (eps
// inside the root) and multiplied by one weight vector that all heads share.
//
// gated_recurrence - one block per (head, entry) walks the entry's tokens in order, from and
//   to the request's state row.  Thread (v, s) keeps the rows d = i * DS + s of column v of
//   the state in registers; the DS threads of a column sit side by side in a warp and add
//   their shares of o_t[v] in a butterfly.  Tokens come in chunks of up to 16: all threads
//   first turn the chunk's projections into q, f and v in shared memory (the exponentials
//   run side by side there, not inside the chain), then the chain of the chunk's tokens runs
//   without a block-wide barrier, then a warp per token takes the norm and stores the row.
//   A prompt portion and a single decoded token take the same path; the state is carried in
//   32-bit, and the order of additions depends on dk and DS alone, so how a sequence is cut
//   into steps and what else is in the batch change nothing.
#include "common.cuh"

#define GR_CHUNK 16
#define GR_MAX_KPT 32

struct GatedRecurrence {
  const float* proj;      // [tokens, ld]
  long long ld;
  int q_off, f_off, v_off;
  const float* f_bias;    // [heads * dk] or null
  const float* lower;     // [heads * dk]
  const float* norm_w;    // [dv]
  float eps;
  float* state;           // [rows, heads, dk, dv]
  int state_rows;
  const int* slots;       // [entries]
  const int* cu_tokens;   // [entries + 1]
  void* out;              // [tokens, heads * dv]
  int heads, dk, dv, ds, kpt;
};

__device__ __forceinline__ float gr_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

template <typename TO, int KPT>
__global__ void __launch_bounds__(1024) gated_recurrence_kernel(GatedRecurrence p, int* status) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, entry = blockIdx.y;
  const int first = p.cu_tokens[entry], count = p.cu_tokens[entry + 1] - first;
  if (count <= 0) return;
  const int slot = p.slots[entry];
  if (slot < 0 || slot >= p.state_rows) {
    if (threadIdx.x == 0) atomicOr(status, FE_STATUS_BAD_PAGE);
    return;
  }
  const int dk = p.dk, dv = p.dv, DS = p.ds, kpt = p.kpt;
  float* fs = smem;                       // [GR_CHUNK][dk]
  float* qs = fs + GR_CHUNK * dk;         // [GR_CHUNK][dk]
  float* vs = qs + GR_CHUNK * dk;         // [GR_CHUNK][dv]
  float* os = vs + GR_CHUNK * dv;         // [GR_CHUNK][dv]
  const int tid = threadIdx.x;
  const int v = tid / DS, s = tid - v * DS;
  const bool live = v < dv;
  float* st = p.state + (((size_t)slot * p.heads + head) * dk) * dv;
  float S[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) S[i] = (live && i < kpt) ? st[(size_t)(i * DS + s) * dv + v] : 0.f;
  const float* bias = p.f_bias ? p.f_bias + head * dk : nullptr;
  const float* low = p.lower + head * dk;
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;

  for (int c0 = 0; c0 < count; c0 += GR_CHUNK) {
    const int nt = min(GR_CHUNK, count - c0);
    for (int idx = tid; idx < nt * dk; idx += blockDim.x) {
      const int t = idx / dk, d = idx - t * dk;
      const float* row = p.proj + (size_t)(first + c0 + t) * p.ld;
      const float zq = row[p.q_off + head * dk + d];
      const float zf = row[p.f_off + head * dk + d] + (bias ? bias[d] : 0.f);
      const float l = low[d];
      qs[idx] = zq * gr_sigmoid(zq);
      fs[idx] = l + (1.f - l) * gr_sigmoid(zf);
    }
    for (int idx = tid; idx < nt * dv; idx += blockDim.x) {
      const int t = idx / dv, c = idx - t * dv;
      vs[idx] = p.proj[(size_t)(first + c0 + t) * p.ld + p.v_off + head * dv + c];
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float vv = live ? vs[t * dv + v] : 0.f;
      const float* ft = fs + t * dk + s;
      const float* qt = qs + t * dk + s;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        if (i < kpt) {
          const float f = ft[i * DS];
          S[i] = fmaf(f, S[i], (1.f - f) * vv);
          acc = fmaf(S[i], qt[i * DS], acc);
        }
      }
      for (int o = DS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && s == 0) os[t * dv + v] = acc;
    }
    __syncthreads();
    for (int t = warp; t < nt; t += warps) {
      float ss = 0.f;
      for (int c = lane; c < dv; c += 32) ss = fmaf(os[t * dv + c], os[t * dv + c], ss);
      const float inv = 1.f / sqrtf(warp_sum(ss) / (float)dv + p.eps);
      TO* dst = (TO*)p.out + (size_t)(first + c0 + t) * p.heads * dv + (size_t)head * dv;
      for (int c = lane; c < dv; c += 32) dst[c] = from_float<TO>(os[t * dv + c] * inv * p.norm_w[c]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i)
    if (live && i < kpt) st[(size_t)(i * DS + s) * dv + v] = S[i];
}

// Threads of a column: the largest power of two up to 8 (4 where the block stays at 128
// threads or more: then a warp's state rows are whole 32-byte sectors) that divides dk, keeps
// the block within 1,024 threads and a thread within GR_MAX_KPT rows.  0: no such number.
static int gr_column_threads(int dk, int dv) {
  const int prefer[] = {4, 8, 2, 1, 16, 32};
  for (int pass = 0; pass < 2; ++pass) {
    for (int ds : prefer) {
      if (dk % ds || (long long)dv * ds > 1024 || dk / ds > GR_MAX_KPT) continue;
      if (pass == 0 && (dv * ds < 128 || dk / ds > 16)) continue;
      return ds;
    }
  }
  return 0;
}

FE_EXPORT int fe_gated_recurrence(const float* proj, long long ld, int q_off, int f_off, int v_off, const float* f_bias,
                                  const float* lower, const float* norm_w, float eps, float* state, int state_rows,
                                  const int* slots, const int* cu_tokens, void* out, int out_dtype, int entries, int heads,
                                  int dk, int dv, int* status, cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (heads < 1 || dk < 1 || dv < 1 || heads > 65535 || entries > 65535) return FE_ERR_BAD_SHAPE;
  const int ds = gr_column_threads(dk, dv);
  if (ds == 0) return FE_ERR_BAD_SHAPE;
  const int kpt = dk / ds;
  GatedRecurrence p{proj, ld, q_off, f_off, v_off, f_bias, lower, norm_w, eps, state, state_rows, slots, cu_tokens, out,
                    heads, dk, dv, ds, kpt};
  const int threads = (dv * ds + 31) / 32 * 32;
  const size_t smem = sizeof(float) * (size_t)GR_CHUNK * 2 * (dk + dv);
  if (smem > 200 * 1024) return FE_ERR_TOO_LARGE;
  int rc = FE_ERR_BAD_DTYPE;
#define GR_LAUNCH(TO, KPT)                                                                                            \
  do {                                                                                                                \
    if (smem > 48 * 1024)                                                                                             \
      cudaFuncSetAttribute(gated_recurrence_kernel<TO, KPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    rc = fe_launch_dependent(gated_recurrence_kernel<TO, KPT>, dim3(heads, entries), dim3(threads), smem, stream, p,  \
                             status);                                                                                 \
  } while (0)
#define GR_BY_KPT(TO)                        \
  do {                                       \
    if (kpt <= 4) GR_LAUNCH(TO, 4);          \
    else if (kpt <= 8) GR_LAUNCH(TO, 8);     \
    else if (kpt <= 16) GR_LAUNCH(TO, 16);   \
    else GR_LAUNCH(TO, 32);                  \
  } while (0)
  if (out_dtype == FE_DTYPE_F32) GR_BY_KPT(float);
  else if (out_dtype == FE_DTYPE_BF16) GR_BY_KPT(bf16);
#undef GR_BY_KPT
#undef GR_LAUNCH
  return rc ? rc : fe_last_error();
}
