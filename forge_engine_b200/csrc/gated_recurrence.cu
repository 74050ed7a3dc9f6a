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
//   into steps and what else is in the batch change nothing.  With `long_from` > 0 it leaves
//   entries of that many tokens or more to the three kernels below.
//
// Long entries (prompt portions) run chunk by chunk side by side, which is exact for a linear
// recurrence: with b_t the product of the forget gates from the chunk's first token up to t,
//     S_t = diag(b_t) S_start + S_local_t,      o_t = (q_t * b_t)^T S_start + o_local_t.
// gated_recurrence_local  - the kernel above on one chunk of GR_LONG_CHUNK tokens per block,
//   started from zero: o_local (32-bit, not yet normalised), q_t * b_t, the chunk's last local
//   state and its b.
// gated_recurrence_scan   - one thread per state element walks the entry's chunks in order:
//   S_start of every chunk, and the request's state row after the last.
// gated_recurrence_finish - per chunk (q * b)^T S_start + o_local as a small 32-bit product from
//   shared memory, then the head's norm and the store.
// There is no division by a decay anywhere (a gate may be as small as its lower bound allows),
// and everything stays 32-bit; against the token-by-token walk only the order of additions
// differs.
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
  int long_from;          // above zero: entries of this many tokens or more belong to the chunk-parallel kernels
  // scratch of the chunk-parallel kernels (32-bit)
  float* o_local;         // [tokens, heads * dv]
  float* qb;              // [tokens, heads * dk]
  float* chunk_state;     // [chunk slots, heads, dk, dv]: the chunk's local end state, then (scan) its start state
  float* chunk_start;     // [chunk slots, heads, dk, dv]
  float* chunk_decay;     // [chunk slots, heads, dk]
};

#define GR_LONG_CHUNK 64
// Chunk c of entry e has a slot of its own: the entries' first tokens are at least a chunk's
// tokens apart per chunk, so floor(first / chunk) + e + c never repeats.
__device__ __forceinline__ int gr_chunk_slot(int first, int entry, int chunk) { return first / GR_LONG_CHUNK + entry + chunk; }

__device__ __forceinline__ float gr_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }

template <typename TO, int KPT>
__global__ void __launch_bounds__(1024) gated_recurrence_kernel(GatedRecurrence p, int* status) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, entry = blockIdx.y;
  const int first = p.cu_tokens[entry], count = p.cu_tokens[entry + 1] - first;
  if (count <= 0 || (p.long_from > 0 && count >= p.long_from)) return;
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


// One chunk of a long entry from a zero state (see the head of this file).  A thread keeps the
// rows s * kpt .. s * kpt + kpt - 1 of its column, so that it reads its gates and queries of a
// token with 16-byte loads from shared memory; the rows up to KPT are padded with f = 1, q = 0
// (such a row stays zero), and a pitch of KPT + 4 keeps the eight lanes of a load in different
// banks.  The running product of the gates and q * b are the work of one thread per channel.
template <int KPT>
__global__ void __launch_bounds__(1024) gated_recurrence_local_kernel(GatedRecurrence p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, entry = blockIdx.y, chunk = blockIdx.z;
  const int entry_first = p.cu_tokens[entry], entry_count = p.cu_tokens[entry + 1] - entry_first;
  if (entry_count < p.long_from || chunk * GR_LONG_CHUNK >= entry_count) return;
  const int first = entry_first + chunk * GR_LONG_CHUNK, count = min(GR_LONG_CHUNK, entry_count - chunk * GR_LONG_CHUNK);
  const int dk = p.dk, dv = p.dv, DS = p.ds, kpt = p.kpt;
  constexpr int KP = KPT >= 8 ? KPT + 4 : KPT;
  const int pitch = DS * KP;              // floats per token
  float* fs = smem;                       // [GR_CHUNK][DS][KP]
  float* qs = fs + GR_CHUNK * pitch;      // [GR_CHUNK][DS][KP]
  float* vs = qs + GR_CHUNK * pitch;      // [GR_CHUNK][dv]
  float* bs = vs + GR_CHUNK * dv;         // [dk]: the product of the gates so far
  const int tid = threadIdx.x;
  const int v = tid / DS, s = tid - v * DS;
  const bool live = v < dv;
  float S[KPT];
#pragma unroll
  for (int i = 0; i < KPT; ++i) S[i] = 0.f;
  for (int idx = tid; idx < GR_CHUNK * pitch; idx += blockDim.x) { fs[idx] = 1.f; qs[idx] = 0.f; }
  for (int d = tid; d < dk; d += blockDim.x) bs[d] = 1.f;
  __syncthreads();
  const float* bias = p.f_bias ? p.f_bias + head * dk : nullptr;
  const float* low = p.lower + head * dk;
  for (int c0 = 0; c0 < count; c0 += GR_CHUNK) {
    const int nt = min(GR_CHUNK, count - c0);
    for (int idx = tid; idx < nt * dk; idx += blockDim.x) {
      const int t = idx / dk, d = idx - t * dk;
      const float* row = p.proj + (size_t)(first + c0 + t) * p.ld;
      const float zq = row[p.q_off + head * dk + d];
      const float zf = row[p.f_off + head * dk + d] + (bias ? bias[d] : 0.f);
      const float l = low[d];
      const int owner = d / kpt, at = t * pitch + owner * KP + (d - owner * kpt);
      qs[at] = zq * gr_sigmoid(zq);
      fs[at] = l + (1.f - l) * gr_sigmoid(zf);
    }
    for (int idx = tid; idx < nt * dv; idx += blockDim.x) {
      const int t = idx / dv, c = idx - t * dv;
      vs[idx] = p.proj[(size_t)(first + c0 + t) * p.ld + p.v_off + head * dv + c];
    }
    __syncthreads();
    for (int d = tid; d < dk; d += blockDim.x) {
      const int owner = d / kpt, at = owner * KP + (d - owner * kpt);
      float b = bs[d];
      float* dst = p.qb + (size_t)(first + c0) * p.heads * dk + (size_t)head * dk + d;
      for (int t = 0; t < nt; ++t) {
        b *= fs[t * pitch + at];
        dst[(size_t)t * p.heads * dk] = qs[t * pitch + at] * b;
      }
      bs[d] = b;
    }
    for (int t = 0; t < nt; ++t) {
      const float vv = live ? vs[t * dv + v] : 0.f;
      const float4* f4 = reinterpret_cast<const float4*>(fs + t * pitch + s * KP);
      const float4* q4 = reinterpret_cast<const float4*>(qs + t * pitch + s * KP);
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < KPT / 4; ++i) {
        const float4 f = f4[i], q = q4[i];
        S[4 * i + 0] = fmaf(f.x, S[4 * i + 0], (1.f - f.x) * vv);
        S[4 * i + 1] = fmaf(f.y, S[4 * i + 1], (1.f - f.y) * vv);
        S[4 * i + 2] = fmaf(f.z, S[4 * i + 2], (1.f - f.z) * vv);
        S[4 * i + 3] = fmaf(f.w, S[4 * i + 3], (1.f - f.w) * vv);
        acc = fmaf(S[4 * i + 0], q.x, acc);
        acc = fmaf(S[4 * i + 1], q.y, acc);
        acc = fmaf(S[4 * i + 2], q.z, acc);
        acc = fmaf(S[4 * i + 3], q.w, acc);
      }
      for (int o = DS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && s == 0) p.o_local[(size_t)(first + c0 + t) * p.heads * dv + (size_t)head * dv + v] = acc;
    }
    __syncthreads();
  }
  const size_t at = (size_t)gr_chunk_slot(entry_first, entry, chunk) * p.heads + head;
#pragma unroll
  for (int i = 0; i < KPT; ++i)
    if (live && i < kpt) p.chunk_state[(at * dk + s * kpt + i) * dv + v] = S[i];
  for (int d = tid; d < dk; d += blockDim.x) p.chunk_decay[at * dk + d] = bs[d];
}

// One thread per element (d, v) of a head's state: the start state of every chunk of a long
// entry, in order, and the request's state row after the last chunk.
__global__ void __launch_bounds__(256) gated_recurrence_scan_kernel(GatedRecurrence p, int* status) {
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, entry = blockIdx.y;
  const int first = p.cu_tokens[entry], count = p.cu_tokens[entry + 1] - first;
  if (count < p.long_from) return;
  const int slot = p.slots[entry];
  if (slot < 0 || slot >= p.state_rows) {
    if (threadIdx.x == 0 && blockIdx.z == 0) atomicOr(status, FE_STATUS_BAD_PAGE);
    return;
  }
  const int cell = blockIdx.z * blockDim.x + threadIdx.x;
  if (cell >= p.dk * p.dv) return;
  const int d = cell / p.dv;
  const int chunks = (count + GR_LONG_CHUNK - 1) / GR_LONG_CHUNK;
  float* st = p.state + ((size_t)slot * p.heads + head) * p.dk * p.dv + cell;
  float state = *st;
  const size_t stride = (size_t)p.heads * p.dk * p.dv;
  const float* __restrict__ local = p.chunk_state + ((size_t)gr_chunk_slot(first, entry, 0) * p.heads + head) * p.dk * p.dv + cell;
  float* __restrict__ start = p.chunk_start + ((size_t)gr_chunk_slot(first, entry, 0) * p.heads + head) * p.dk * p.dv + cell;
  const float* __restrict__ decay = p.chunk_decay + ((size_t)gr_chunk_slot(first, entry, 0) * p.heads + head) * p.dk + d;
#pragma unroll 4
  for (int c = 0; c < chunks; ++c) {
    start[c * stride] = state;
    state = fmaf(decay[(size_t)c * p.heads * p.dk], state, local[c * stride]);
  }
  *st = state;
}

// o_t = (q_t * b_t)^T S_start + o_local_t for the tokens of one chunk, then the head's norm.
// Thread (t, g) of 64 x 4 takes token t and, per round of 32 columns, the columns 4g .. 4g + 3
// and 16 + 4g .. 16 + 4g + 3 (dv is a multiple of 4); S_start and q * b are read from shared
// memory 16 bytes at a time.
template <typename TO>
__global__ void __launch_bounds__(256) gated_recurrence_finish_kernel(GatedRecurrence p) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int head = blockIdx.x, entry = blockIdx.y, chunk = blockIdx.z;
  const int entry_first = p.cu_tokens[entry], entry_count = p.cu_tokens[entry + 1] - entry_first;
  if (entry_count < p.long_from || chunk * GR_LONG_CHUNK >= entry_count) return;
  const int first = entry_first + chunk * GR_LONG_CHUNK, count = min(GR_LONG_CHUNK, entry_count - chunk * GR_LONG_CHUNK);
  const int dk = p.dk, dv = p.dv;
  const int dkp = (dk + 3) & ~3;            // rows in fours; the added ones are zero
  const int qld = dkp + 4;                  // 16-byte rows; a warp's eight tokens read different banks
  float* ss = smem;                         // [dkp][dv]
  float* qb = ss + dkp * dv;                // [GR_LONG_CHUNK][qld]
  float* os = qb + GR_LONG_CHUNK * qld;     // [GR_LONG_CHUNK][dv]
  const int tid = threadIdx.x;
  const float* start = p.chunk_start + ((size_t)gr_chunk_slot(entry_first, entry, chunk) * p.heads + head) * dk * dv;
  for (int i = tid; i < dkp * dv; i += blockDim.x) ss[i] = i < dk * dv ? start[i] : 0.f;
  for (int i = tid; i < count * qld; i += blockDim.x) {
    const int t = i / qld, d = i - t * qld;
    qb[i] = d < dk ? p.qb[(size_t)(first + t) * p.heads * dk + (size_t)head * dk + d] : 0.f;
  }
  __syncthreads();
  const int t = tid >> 2, g = tid & 3;
  if (t < count) {
    const float* qt = qb + t * qld;
    const float* local = p.o_local + (size_t)(first + t) * p.heads * dv + (size_t)head * dv;
    for (int v0 = 0; v0 < dv; v0 += 32) {
      const int c0 = v0 + 4 * g, c1 = c0 + 16;
      const bool has0 = c0 < dv, has1 = c1 < dv;
      float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
      for (int d = 0; d < dkp; d += 4) {
        const float4 q = *reinterpret_cast<const float4*>(qt + d);
        const float qk[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float* sr = ss + (d + k) * dv;
          if (has0) {
            const float4 x = *reinterpret_cast<const float4*>(sr + c0);
            a0.x = fmaf(qk[k], x.x, a0.x), a0.y = fmaf(qk[k], x.y, a0.y), a0.z = fmaf(qk[k], x.z, a0.z), a0.w = fmaf(qk[k], x.w, a0.w);
          }
          if (has1) {
            const float4 x = *reinterpret_cast<const float4*>(sr + c1);
            a1.x = fmaf(qk[k], x.x, a1.x), a1.y = fmaf(qk[k], x.y, a1.y), a1.z = fmaf(qk[k], x.z, a1.z), a1.w = fmaf(qk[k], x.w, a1.w);
          }
        }
      }
      if (has0) {
        const float4 l = *reinterpret_cast<const float4*>(local + c0);
        *reinterpret_cast<float4*>(os + t * dv + c0) = make_float4(a0.x + l.x, a0.y + l.y, a0.z + l.z, a0.w + l.w);
      }
      if (has1) {
        const float4 l = *reinterpret_cast<const float4*>(local + c1);
        *reinterpret_cast<float4*>(os + t * dv + c1) = make_float4(a1.x + l.x, a1.y + l.y, a1.z + l.z, a1.w + l.w);
      }
    }
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  for (int r = warp; r < count; r += warps) {
    float sq = 0.f;
    for (int c = lane; c < dv; c += 32) sq = fmaf(os[r * dv + c], os[r * dv + c], sq);
    const float inv = 1.f / sqrtf(warp_sum(sq) / (float)dv + p.eps);
    TO* dst = (TO*)p.out + (size_t)(first + r) * p.heads * dv + (size_t)head * dv;
    for (int c = lane; c < dv; c += 32) dst[c] = from_float<TO>(os[r * dv + c] * inv * p.norm_w[c]);
  }
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

// Shared memory of gated_recurrence_finish, and whether the chunk-parallel kernels take these sizes.
static size_t gr_finish_smem(int dk, int dv) {
  const size_t dkp = (size_t)(dk + 3) / 4 * 4;
  return sizeof(float) * (dkp * dv + (size_t)GR_LONG_CHUNK * (dkp + 4 + dv));
}

// 32-bit floats of scratch the chunk-parallel kernels need for a step of `tokens` tokens in
// `entries` entries (0: these sizes run token by token whatever the entries' lengths).
FE_EXPORT long long fe_gated_recurrence_scratch(int tokens, int entries, int heads, int dk, int dv) {
  if (dv % 4 != 0 || gr_finish_smem(dk, dv) > 200 * 1024 || gr_column_threads(dk, dv) == 0) return 0;
  const long long slots = tokens / GR_LONG_CHUNK + entries + 1;
  return (long long)tokens * heads * (dk + dv) + slots * heads * ((long long)2 * dk * dv + dk);
}

// Tokens from which on an entry runs chunk by chunk.
FE_EXPORT int fe_gated_recurrence_long_from() { return 2 * GR_LONG_CHUNK; }

// scratch: null, or fe_gated_recurrence_scratch floats; then entries of fe_gated_recurrence_long_from
// tokens or more (max_new is the most tokens any entry brings) run chunk by chunk
FE_EXPORT int fe_gated_recurrence(const float* proj, long long ld, int q_off, int f_off, int v_off, const float* f_bias,
                                  const float* lower, const float* norm_w, float eps, float* state, int state_rows,
                                  const int* slots, const int* cu_tokens, void* out, int out_dtype, int entries, int heads,
                                  int dk, int dv, int tokens, int max_new, float* scratch, int* status,
                                  cudaStream_t stream) {
  if (entries <= 0) return 0;
  if (heads < 1 || dk < 1 || dv < 1 || heads > 65535 || entries > 65535) return FE_ERR_BAD_SHAPE;
  const int ds = gr_column_threads(dk, dv);
  if (ds == 0) return FE_ERR_BAD_SHAPE;
  const int kpt = dk / ds;
  GatedRecurrence p{proj, ld, q_off, f_off, v_off, f_bias, lower, norm_w, eps, state, state_rows, slots, cu_tokens, out,
                    heads, dk, dv, ds, kpt, 0, nullptr, nullptr, nullptr, nullptr, nullptr};
  const bool chunked = scratch != nullptr && max_new >= fe_gated_recurrence_long_from() &&
                       fe_gated_recurrence_scratch(tokens, entries, heads, dk, dv) > 0;
  if (chunked) {
    const long long chunk_slots = tokens / GR_LONG_CHUNK + entries + 1;
    p.long_from = fe_gated_recurrence_long_from();
    p.o_local = scratch;
    p.qb = p.o_local + (size_t)tokens * heads * dv;
    p.chunk_state = p.qb + (size_t)tokens * heads * dk;
    p.chunk_start = p.chunk_state + (size_t)chunk_slots * heads * dk * dv;
    p.chunk_decay = p.chunk_start + (size_t)chunk_slots * heads * dk * dv;
  }
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
  if (rc || !chunked) return rc ? rc : fe_last_error();
  const int chunks = (max_new + GR_LONG_CHUNK - 1) / GR_LONG_CHUNK;
  if (chunks > 65535) return FE_ERR_TOO_LARGE;
  const int kpt_built = kpt <= 4 ? 4 : kpt <= 8 ? 8 : kpt <= 16 ? 16 : 32;      // the instantiation's KPT, and its pitch
  const size_t local_smem = sizeof(float) * ((size_t)GR_CHUNK * (2 * ds * (kpt_built >= 8 ? kpt_built + 4 : kpt_built) + dv) + dk);
#define GR_LOCAL(KPT)                                                                                                  \
  do {                                                                                                                 \
    if (local_smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(gated_recurrence_local_kernel<KPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                           (int)local_smem);                                                                           \
    rc = fe_launch_dependent(gated_recurrence_local_kernel<KPT>, dim3(heads, entries, chunks), dim3(threads),          \
                             local_smem, stream, p);                                                                   \
  } while (0)
  if (kpt <= 4) GR_LOCAL(4);
  else if (kpt <= 8) GR_LOCAL(8);
  else if (kpt <= 16) GR_LOCAL(16);
  else GR_LOCAL(32);
#undef GR_LOCAL
  if (rc) return rc;
  rc = fe_launch_dependent(gated_recurrence_scan_kernel, dim3(heads, entries, (dk * dv + 255) / 256), dim3(256), 0, stream,
                           p, status);
  if (rc) return rc;
  const size_t finish_smem = gr_finish_smem(dk, dv);
  if (out_dtype == FE_DTYPE_F32) {
    if (finish_smem > 48 * 1024)
      cudaFuncSetAttribute(gated_recurrence_finish_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)finish_smem);
    rc = fe_launch_dependent(gated_recurrence_finish_kernel<float>, dim3(heads, entries, chunks), dim3(256), finish_smem, stream, p);
  } else {
    if (finish_smem > 48 * 1024)
      cudaFuncSetAttribute(gated_recurrence_finish_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)finish_smem);
    rc = fe_launch_dependent(gated_recurrence_finish_kernel<bf16>, dim3(heads, entries, chunks), dim3(256), finish_smem, stream, p);
  }
  return rc ? rc : fe_last_error();
}
