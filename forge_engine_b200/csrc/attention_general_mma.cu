// Tensor-core form of the general paged attention (bfloat16), compiled once per shape:
//   -DFE_DK=<key size> -DFE_DV=<value size> -DFE_V_IN_K=<0|1>
// FE_V_IN_K = 1: the value is the first FE_DV elements of the cached key row (a latent that is
// key and value at once); then no second tile is loaded.
//
// A block of 4 warps (8 for more than 256 value columns) owns 64 rows - the (token, query head) pairs of one entry that share one
// kv head, token-major - and walks the key tiles its rows can see (causal, optional window),
// cp.async double-buffered from the cache pages.  S = Q K^T and O += P V run on mma.sync
// m16n8k16 with 32-bit accumulators; scale, distance bias, mask and the online softmax are
// 32-bit.  The weights P enter the second product as a sum of two bfloat16 numbers (the
// rounded weight and the rounded remainder), so they carry 16 bits of mantissa and not 8.
// Few rows and many keys (decoding): `splits` blocks share a row tile's key tiles and leave
// (sum, maximum, normaliser) in a workspace that a second kernel combines.
#include "attention_common.cuh"

#ifndef FE_DK
#error "compile with -DFE_DK=... -DFE_DV=... -DFE_V_IN_K=..."
#endif

#define GM_CAT2(a, b, c, d) a##b##_##c##_##d
#define GM_CAT(a, b, c, d) GM_CAT2(a, b, c, d)
#define GM_NAME(base) GM_CAT(base, FE_DK, FE_DV, FE_V_IN_K)

namespace {

constexpr int DK = FE_DK, DV = FE_DV;
constexpr bool V_IN_K = FE_V_IN_K != 0;
constexpr int BM = 64;
// more than 256 value columns: two groups of four warps share a row tile, each with half the
// columns (both take the scores; the accumulators of sixteen rows x 512 columns fit no warp)
constexpr int VSPLIT = DV > 256 ? 2 : 1;
constexpr int WARPS = 4 * VSPLIT;
constexpr int DVW = DV / VSPLIT;                // value columns of one warp
constexpr float LOG2E = 1.4426950408889634f;
// key tiles of 32 where tiles of 64 (keys and values, double-buffered) would leave room for one
// block of four warps per SM only (measured with keys of 128 and values of 256: 0.60 -> 0.48 ms
// for a 2,048-token prompt, 0.133 -> 0.090 ms for a decode step at batch 8)
constexpr int BN = (DK > 320 || (!V_IN_K && DK + DV > 320)) ? 32 : 64;
constexpr int KS = DK + 8;                     // row stride of the Q and K tiles in shared memory
constexpr int VS = DV + 8;
constexpr int QC = DK / 8, VC = DV / 8;        // 16-byte pieces per row
constexpr int K_TILE = BN * KS, V_TILE = V_IN_K ? 0 : BN * VS;
constexpr size_t SMEM_BYTES = sizeof(bf16) * (size_t)(BM * KS + 2 * K_TILE + 2 * V_TILE);

struct Params {
  const bf16* q; long long q_ts, q_hs;
  const bf16* k; int k_row;
  const bf16* v; int v_row;
  void* out; long long o_ts, o_hs;
  const int* table; int max_pages, page_size, num_pages, nkv, groups;
  const int* cu_tokens; const int* starts;
  const float* slopes; const float* dist_bias; int dist_len; int window; float scale;
  int splits; int tiles; float* part;
  // what the plain layer does not have (off when zero / null); see GeneralAttn in attention_general.cu
  int keep_first; float softcap, temp_coef; int temp_every;
  int parts; long long q_ps; int k_ps; long long o_ps;
  const float* gate; long long gate_stride; int out_f32;
  int row_hi;      // above zero: entries with more rows (new tokens x heads per kv head) are left to another kernel
  const float* sinks;   // or null: per query head a number whose exponential joins the denominator once
};

__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
  return every > 0 ? 1.f + coef * logf((float)((pos + 1) / every + 1)) : 1.f;
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + expf(-x)); }
// tanh as 1 - 2 / (1 + e^(2x)) on the fast exponential: the absolute error stays below 3e-7,
// which is what a capped score (cap * tanh, the cap a few tens) needs; it saturates to +-1
__device__ __forceinline__ float tanh_capped(float x) { return 1.f - __fdividef(2.f, 1.f + __expf(2.f * x)); }

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack2(float x, float y) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  return *reinterpret_cast<const unsigned*>(&h);
}
// the rounded pair and the rounded remainders
__device__ __forceinline__ void split2(float x, float y, unsigned& hi, unsigned& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  const float2 back = __bfloat1622float2(h);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = pack2(x - back.x, y - back.y);
}

__global__ void __launch_bounds__(WARPS * 32, 1) attention_mma_kernel(Params p, int* status) {
  extern __shared__ __align__(16) unsigned char raw[];
  bf16* Qs = reinterpret_cast<bf16*>(raw);
  bf16* Ks = Qs + BM * KS;
  bf16* Vs = Ks + 2 * K_TILE;
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
  const int entry = blockIdx.y, kvh = blockIdx.z / p.parts, part = blockIdx.z - kvh * p.parts;
  const int t_begin = p.cu_tokens[entry];
  const int count = p.cu_tokens[entry + 1] - t_begin;
  const int start = p.starts[entry];
  const int rows_total = count * p.groups;
  const int row0 = tile * BM;
  if (row0 >= rows_total || (p.row_hi > 0 && rows_total > p.row_hi)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rw = warp & 3, vcol0 = (warp >> 2) * DVW;      // the warp's sixteen rows and first value column
  const int* table = p.table + (size_t)entry * p.max_pages;

  // the row tile of Q
  for (int idx = tid; idx < BM * QC; idx += WARPS * 32) {
    const int r = idx / QC, c = idx - r * QC;
    const int rho = row0 + r;
    uint4 value = make_uint4(0, 0, 0, 0);
    if (rho < rows_total) {
      const int token = t_begin + rho / p.groups, head = kvh * p.groups + rho % p.groups;
      value = *reinterpret_cast<const uint4*>(p.q + (size_t)token * p.q_ts + (size_t)head * p.q_hs + (size_t)part * p.q_ps + c * 8);
    }
    *reinterpret_cast<uint4*>(Qs + r * KS + c * 8) = value;
  }

  const int tok_lo = row0 / p.groups, tok_hi = min(count - 1, (row0 + BM - 1) / p.groups);
  const int key_hi = start + tok_hi;                                        // last key any row sees
  const int key_lo = p.window > 0 ? max(0, start + tok_lo - p.window + 1) : 0;
  const int kt_lo = key_lo / BN, kt_hi = key_hi / BN + 1;
  // keys below keep_first stay visible after the window has passed them: their tiles (those that
  // lie before the window's first tile) are walked first; step i of the walk is key tile tile_of(i)
  const int sink_keys = p.window > 0 ? p.keep_first : 0;
  const int sink_tiles = min((sink_keys + BN - 1) / BN, kt_lo);
  const int steps = sink_tiles + kt_hi - kt_lo;
  const int per = (steps + p.splits - 1) / p.splits;
  const int my_lo = split * per, my_hi = min(steps, my_lo + per);
  auto tile_of = [&](int i) { return i < sink_tiles ? i : kt_lo + i - sink_tiles; };

  // TPR threads fetch one key row: its page is looked up once per row and tile
  constexpr int TPR = WARPS * 32 / BN;
  const int load_row = tid / TPR, load_piece = tid % TPR;
  auto load_tile = [&](int kt, int stage) {
    const int key = kt * BN + load_row;
    bool valid = (key >= key_lo || key < sink_keys) && key <= key_hi;
    size_t row = 0;
    if (valid) {
      const int logical = key / p.page_size;
      const int page = logical < p.max_pages ? table[logical] : -1;
      if (page < 0 || page >= p.num_pages) valid = false;     // a page the window has given back: its keys are masked anyway
      else row = ((size_t)page * p.nkv + kvh) * p.page_size + (key - logical * p.page_size);
    }
    const bf16* ksrc = p.k + row * p.k_row + part * p.k_ps;
    bf16* kd = Ks + stage * K_TILE + load_row * KS;
#pragma unroll
    for (int c = load_piece; c < QC; c += TPR) cp_async16(kd + c * 8, ksrc + c * 8, valid);
    if constexpr (!V_IN_K) {
      const bf16* vsrc = p.v + row * p.v_row;
      bf16* vd = Vs + stage * V_TILE + load_row * VS;
#pragma unroll
      for (int c = load_piece; c < VC; c += TPR) cp_async16(vd + c * 8, vsrc + c * 8, valid);
    }
  };

  // this thread's two rows: r_a = lane / 4 and r_a + 8 of the warp's sixteen
  const int quad = lane >> 2, pair = lane & 3;
  int row_pos[2];
  float row_slope[2], row_scale[2];
  const float* row_bias[2];    // the row's head in the table of biases by distance, or null
  bool row_live[2];
  // scores are kept in units of log 2, so that exp is one exp2; with a cap the product is first
  // brought to units of the cap, and cap * log2(e) * tanh(.) is taken
  const bool capped = p.softcap > 0.f;
  const float cap2 = p.softcap * LOG2E;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int rho = row0 + rw * 16 + quad + 8 * h;
    row_live[h] = rho < rows_total;
    row_pos[h] = row_live[h] ? start + rho / p.groups : -1;
    row_slope[h] = (row_live[h] && p.slopes) ? p.slopes[kvh * p.groups + rho % p.groups] * LOG2E : 0.f;
    row_bias[h] = (row_live[h] && p.dist_bias) ? p.dist_bias + (size_t)(kvh * p.groups + rho % p.groups) * p.dist_len : nullptr;
    const float natural = p.scale * query_temperature(max(row_pos[h], 0), p.temp_coef, p.temp_every);
    row_scale[h] = capped ? natural / p.softcap : natural * LOG2E;
  }
  // rows of this warp, first and last position (all sixteen live), for tiles that need no mask
  const bool warp_full = row0 + rw * 16 + 15 < rows_total;
  const int warp_pos_lo = start + (row0 + rw * 16) / p.groups, warp_pos_hi = start + (row0 + rw * 16 + 15) / p.groups;
  const bool warp_live = row0 + rw * 16 < rows_total;
  float o[DVW / 8][4];
#pragma unroll
  for (int n = 0; n < DVW / 8; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  if (my_lo < my_hi) {
    load_tile(tile_of(my_lo), 0);
    cp_commit();
  }
  for (int step = my_lo; step < my_hi; ++step) {
    const int kt = tile_of(step);
    const int stage = (step - my_lo) & 1;
    if (step + 1 < my_hi) {
      load_tile(tile_of(step + 1), stage ^ 1);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const bf16* kd = Ks + stage * K_TILE;
    const bf16* vd = V_IN_K ? kd : Vs + stage * V_TILE;
    constexpr int vstride = V_IN_K ? KS : VS;
    if (!warp_live) {            // a warp whose sixteen rows lie past the entry's last row only loads
      __syncthreads();
      continue;
    }

    float s[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < DK / 16; ++kk) {
      unsigned a[4];
      ldsm4(a[0], a[1], a[2], a[3], Qs + (rw * 16 + (lane & 15)) * KS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < BN / 8; j += 2) {
        unsigned b0, b1, b2, b3;
        ldsm4(b0, b1, b2, b3, kd + ((j + (lane >> 4)) * 8 + (lane & 7)) * KS + kk * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s[j], a, b0, b1);
        mma16816(s[j + 1], a, b2, b3);
      }
    }

    // scale, bias, mask; running maximum and normaliser
    float mx[2] = {-INFINITY, -INFINITY};
    // every key of the tile is visible to every row of the warp: no comparisons
    const bool inside = warp_full && kt * BN + BN - 1 <= warp_pos_lo && (p.window <= 0 || kt * BN > warp_pos_hi - p.window);
    if (inside) {
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = c >> 1;
          const int key = kt * BN + j * 8 + pair * 2 + (c & 1);
          float sc = s[j][c] * row_scale[h];
          if (capped) sc = cap2 * tanh_capped(sc);
          sc -= row_slope[h] * (float)(row_pos[h] - key);
          if (row_bias[h] != nullptr) sc = fmaf(row_bias[h][min(row_pos[h] - key, p.dist_len - 1)], LOG2E, sc);
          s[j][c] = sc;
          mx[h] = fmaxf(mx[h], sc);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int h = c >> 1;
          const int key = kt * BN + j * 8 + pair * 2 + (c & 1);
          const bool visible = row_live[h] && key <= row_pos[h] &&
                               (p.window <= 0 || key > row_pos[h] - p.window || key < sink_keys);
          float sc = s[j][c] * row_scale[h];
          if (capped) sc = cap2 * tanh_capped(sc);
          sc = visible ? sc - row_slope[h] * (float)(row_pos[h] - key) : -INFINITY;
          if (row_bias[h] != nullptr && visible) sc = fmaf(row_bias[h][min(row_pos[h] - key, p.dist_len - 1)], LOG2E, sc);
          s[j][c] = sc;
          mx[h] = fmaxf(mx[h], sc);
        }
      }
    }
    float corr[2], base[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      base[h] = m_new == -INFINITY ? 0.f : m_new;
      corr[h] = exp2f(m_run[h] - base[h]);
      m_run[h] = m_new;
      l_run[h] *= corr[h];
    }
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float w = exp2f(s[j][c] - base[c >> 1]);
        s[j][c] = w;
        l_run[c >> 1] += w;
      }
    }
#pragma unroll
    for (int n = 0; n < DVW / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }

    // O += P V, P as rounded weight + rounded remainder
#pragma unroll
    for (int ks = 0; ks < BN / 16; ++ks) {
      unsigned hi[4], lo[4];
      split2(s[2 * ks][0], s[2 * ks][1], hi[0], lo[0]);
      split2(s[2 * ks][2], s[2 * ks][3], hi[1], lo[1]);
      split2(s[2 * ks + 1][0], s[2 * ks + 1][1], hi[2], lo[2]);
      split2(s[2 * ks + 1][2], s[2 * ks + 1][3], hi[3], lo[3]);
#pragma unroll
      for (int n = 0; n < DVW / 8; n += 2) {
        unsigned b0, b1, b2, b3;
        ldsm4_trans(b0, b1, b2, b3, vd + (ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * vstride + vcol0 + (n + (lane >> 4)) * 8);
        mma16816(o[n], hi, b0, b1);             // neighbours alternate, so that no product waits
        mma16816(o[n + 1], hi, b2, b3);         // for the one just issued into its accumulator
        mma16816(o[n], lo, b0, b1);
        mma16816(o[n + 1], lo, b2, b3);
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  if (p.splits == 1) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (!row_live[h]) continue;
      const int rho = row0 + rw * 16 + quad + 8 * h;
      const int token = t_begin + rho / p.groups, head = kvh * p.groups + rho % p.groups;
      const size_t at = (size_t)token * p.o_ts + (size_t)head * p.o_hs + (size_t)part * p.o_ps;
      // a sink joins the normaliser in the units of the running maximum (log 2); one that dwarfs
      // every score makes the sum infinite and the row zero, which is its limit
      const float l_all = p.sinks ? l_run[h] + exp2f(p.sinks[head] * LOG2E - m_run[h]) : l_run[h];
      float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      if (p.gate) inv *= sigmoidf(p.gate[(size_t)token * p.gate_stride + head]);
      if (p.out_f32) {
        float* dst = reinterpret_cast<float*>(p.out) + at;
#pragma unroll
        for (int n = 0; n < DVW / 8; ++n)
          *reinterpret_cast<float2*>(dst + vcol0 + n * 8 + pair * 2) = make_float2(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
      } else {
        bf16* dst = reinterpret_cast<bf16*>(p.out) + at;
#pragma unroll
        for (int n = 0; n < DVW / 8; ++n)
          *reinterpret_cast<__nv_bfloat162*>(dst + vcol0 + n * 8 + pair * 2) =
              __floats2bfloat162_rn(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
      }
    }
    return;
  }
  // partial result of this split: [entry][tile][kvh, part][split][row][DV + 2]
  float* mine = p.part + ((((size_t)entry * p.tiles + tile) * (p.nkv * p.parts) + blockIdx.z) * p.splits + split) * (size_t)BM * (DV + 2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = rw * 16 + quad + 8 * h;
    float* dst = mine + (size_t)r * (DV + 2);
#pragma unroll
    for (int n = 0; n < DVW / 8; ++n) {
      dst[vcol0 + n * 8 + pair * 2] = o[n][2 * h];
      dst[vcol0 + n * 8 + pair * 2 + 1] = o[n][2 * h + 1];
    }
    if (pair == 0 && vcol0 == 0) {
      dst[DV] = m_run[h];
      dst[DV + 1] = l_run[h];
    }
  }
}

constexpr int MERGE_ROWS = 4, MAX_SPLITS = 32;      // a merge block has four warps, a warp has 32 lanes

// A block combines MERGE_ROWS rows of one row tile: the splits' weights once per row (in a
// fixed order), then every value column.
__global__ void __launch_bounds__(128) attention_mma_merge_kernel(Params p) {
  __shared__ float weight[MERGE_ROWS][MAX_SPLITS];
  __shared__ float inverse[MERGE_ROWS];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x / (BM / MERGE_ROWS), piece = blockIdx.x % (BM / MERGE_ROWS);
  const int entry = blockIdx.y, kvh = blockIdx.z / p.parts, part = blockIdx.z - kvh * p.parts;
  const int t_begin = p.cu_tokens[entry];
  const int rows_total = (p.cu_tokens[entry + 1] - t_begin) * p.groups;
  const int first = tile * BM + piece * MERGE_ROWS;
  if (first >= rows_total || (p.row_hi > 0 && rows_total > p.row_hi)) return;
  const float* base = p.part + (((size_t)entry * p.tiles + tile) * (p.nkv * p.parts) + blockIdx.z) * p.splits * (size_t)BM * (DV + 2);
  const int rows = min(MERGE_ROWS, rows_total - first);
  {
    // a warp per row, a lane per split: maxima and normalisers are fetched side by side
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (w < rows) {
      const int r = piece * MERGE_ROWS + w;
      const float* row = base + ((size_t)lane * BM + r) * (DV + 2);
      const float m = lane < p.splits ? row[DV] : -INFINITY;
      const float l = lane < p.splits ? row[DV + 1] : 0.f;
      float big = warp_max(m);
      float sink = -INFINITY;      // counted once per row, here where the splits meet
      if (p.sinks) {
        const int rho = tile * BM + r;
        sink = p.sinks[kvh * p.groups + rho % p.groups] * LOG2E;
        big = fmaxf(big, sink);
      }
      const float f = m == -INFINITY ? 0.f : exp2f(m - big);      // maxima are in units of log 2
      const float den = warp_sum(l * f) + (p.sinks ? exp2f(sink - big) : 0.f);
      if (lane < p.splits) weight[w][lane] = f;
      if (lane == 0) inverse[w] = den > 0.f ? 1.f / den : 0.f;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * DV; idx += blockDim.x) {
    const int lr = idx / DV, d = idx - lr * DV;
    const int r = piece * MERGE_ROWS + lr;
    float num = 0.f;
    for (int s = 0; s < p.splits; ++s) num = fmaf(base[((size_t)s * BM + r) * (DV + 2) + d], weight[lr][s], num);
    const int rho = tile * BM + r;
    const int token = t_begin + rho / p.groups, head = kvh * p.groups + rho % p.groups;
    float value = num * inverse[lr];
    if (p.gate) value *= sigmoidf(p.gate[(size_t)token * p.gate_stride + head]);
    const size_t at = (size_t)token * p.o_ts + (size_t)head * p.o_hs + (size_t)part * p.o_ps + d;
    if (p.out_f32) reinterpret_cast<float*>(p.out)[at] = value;
    else reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(value);
  }
}

}  // namespace

// Floats of workspace a launch with these sizes needs (0 for one split).
FE_EXPORT long long GM_NAME(fe_attention_gmma_workspace_)(int entries, int max_new, int groups, int nkv /* times parts */, int splits) {
  if (splits <= 1) return 0;
  const long long tiles = ((long long)max_new * groups + BM - 1) / BM;
  return (long long)entries * tiles * nkv * splits * BM * (DV + 2);
}

FE_EXPORT int GM_NAME(fe_attention_gmma_)(const void* q, long long q_ts, long long q_hs, const void* k_cache, int k_row,
                                          const void* v_cache, int v_row, void* out, long long o_ts, long long o_hs,
                                          const int* block_table, int max_pages, int page_size, int num_pages, int nkv,
                                          int num_q_heads, const int* cu_tokens, const int* starts, int entries,
                                          int max_new, const float* slopes, const float* dist_bias, int dist_len,
                                          int window, float scale, int splits,
                                          float* workspace, int keep_first, float softcap, float temp_coef,
                                          int temp_every, int parts, long long q_ps, int k_ps, long long o_ps,
                                          const float* gate, long long gate_stride, int out_f32, int row_hi,
                                          const float* sinks, int* status, cudaStream_t stream) {
  if (entries <= 0 || max_new <= 0) return 0;
  if (parts < 1) parts = 1;
  if (nkv < 1 || num_q_heads % nkv || (long long)nkv * parts > 65535 || entries > 65535) return FE_ERR_BAD_SHAPE;
  if (dist_bias != nullptr && dist_len < 1) return FE_ERR_BAD_SHAPE;
  if (keep_first < 0 || temp_every < 0 || softcap < 0.f || k_ps * (parts - 1) + DK > k_row) return FE_ERR_BAD_SHAPE;
  if (k_row % 8 || v_row % 8 || q_ts % 8 || q_hs % 8 || o_ts % 2 || o_hs % 2 || q_ps % 8 || k_ps % 8 || o_ps % 2) return FE_ERR_BAD_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 || (uintptr_t)out % 4) return FE_ERR_BAD_ALIGN;
  if (splits < 1) splits = 1;
  if (splits > MAX_SPLITS) return FE_ERR_BAD_SHAPE;
  if (splits > 1 && workspace == nullptr) return FE_ERR_BAD_SHAPE;
  const int groups = num_q_heads / nkv;
  const int tiles = (int)(((long long)max_new * groups + BM - 1) / BM);
  Params p{(const bf16*)q, q_ts, q_hs, (const bf16*)k_cache, k_row, (const bf16*)v_cache, v_row, out, o_ts, o_hs,
           block_table, max_pages, page_size, num_pages, nkv, groups, cu_tokens, starts, slopes, dist_bias, dist_len, window, scale,
           splits, tiles, workspace, keep_first, softcap, temp_coef, temp_every, parts, q_ps, k_ps, o_ps, gate,
           gate_stride, out_f32, row_hi, sinks};
  static bool configured = false;
  if (!configured) {
    const cudaError_t rc = cudaFuncSetAttribute(attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (rc != cudaSuccess) return (int)rc;
    configured = true;
  }
  dim3 grid((unsigned)tiles * splits, entries, nkv * parts);
  int rc = fe_launch_dependent(attention_mma_kernel, grid, dim3(WARPS * 32), SMEM_BYTES, stream, p, status);
  if (rc) return rc;
  if (splits > 1) {
    rc = fe_launch_dependent(attention_mma_merge_kernel, dim3(tiles * (BM / MERGE_ROWS), entries, nkv * parts), dim3(128), 0, stream, p);
    if (rc) return rc;
  }
  return fe_last_error();
}
