// A routed feed-forward: every token picks `top` of `experts` small gated units.
//
// The step's (token, choice) pairs - "slots", slot = token * top + choice - are put in the
// order of their experts, so that an expert's rows lie side by side and one tile of a matrix
// product reads the expert's weights once for all of them.  Nothing is decided on the host:
// the counts live on the device and the products are launched for the worst case
// (ceil(slots / tile) + experts row tiles), tiles beyond the real ones returning at once.  So
// the step can be captured in a CUDA graph.
//
//   moe_logits   the router's logits in plain 32-bit FMAs: a block per token and eight rows.
//   moe_route    one warp per token: scores from the 32-bit logits (sigmoid or softmax), the
//                `top` largest (ties: the lower index), weights = the chosen scores as they
//                are or divided by their sum; counts per expert by atomic adds, the value the
//                add returns being the slot's rank inside its expert.
//   moe_plan     one block: running sum of the counts (expert e's rows are [offset[e],
//                offset[e + 1])), the table of row tiles (of 16 to 128 rows, as the products
//                want them), every slot's row, and the counts zeroed again for the next call.
//   moe_gather   the rows side by side, times the slot's weight where the weight scales the
//                expert's input: the operand of the grouped tcgen05 product (gemm_tc5.cu), which
//                serves bfloat16 with sizes in sixteens.
//   moe_grouped  the products for everything else (32-bit, odd sizes).  First: rows gathered
//                from the tokens' activations, times the slot's weight, against the expert's
//                gate and up matrices at once, the gated unit applied to the two 32-bit sums.
//                Second: those rows against the expert's down matrix.  Plain FFMA tiles of 64 x
//                64 (any dtype), or mma.sync tiles for bfloat16; each output element is summed
//                over k in a fixed order, so a row's result does not depend on its neighbours.
//   moe_combine  a token's update = the sum of its slots' rows (times the weight where it
//                scales the output) + gate * the shared unit's output, in slot order.
#include "common.cuh"

#define MOE_BM 64
#define MOE_BN 64
#define MOE_BK 16
#define MOE_MAX_TOP 32

struct MoeAct { int act; float limit, slope; };

// what a product with one matrix applies to its sums: act 16 nothing, 17 the square of relu, 18 the tanh form of GELU
#define MOE_UNARY 16
__device__ __forceinline__ float moe_unary(float z, const MoeAct& a) {
  if (a.act == MOE_UNARY + 1) { const float r = fmaxf(z, 0.f); return r * r; }
  if (a.act == MOE_UNARY + 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z;
}

// the same gated units as act_mul's (0: SiLU, 1: tanh form of GELU, 2: the clamped unit)
__device__ __forceinline__ float moe_act(float z, float u, const MoeAct& a) {
  if (a.act == 0) return z / (1.f + expf(-z)) * u;
  if (a.act == 2) {
    const float g = fminf(z, a.limit);
    const float v = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.f + expf(-a.slope * g)) * (v + 1.f);
  }
  const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return 0.5f * z * (1.f + tanhf(inner)) * u;
}

// ---------------------------------------------------------------------------
// router logits: out[n, r] = sum_k x[n, k] * w[r, k] for a handful of rows r, in plain 32-bit
// FMAs.  A block takes one token (its activations in shared memory as floats) and eight rows,
// a warp one row: lanes stride over k, the 32 partial sums meet in a butterfly.  The order of
// additions depends on k alone, so a token's logits do not depend on the batch.
// ---------------------------------------------------------------------------
template <typename TX>
__global__ void __launch_bounds__(256)
moe_logits_kernel(const TX* __restrict__ x, const float* __restrict__ w, float* __restrict__ out, int rows, int k) {
  extern __shared__ float xs[];
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const TX* src = x + (size_t)token * k;
  for (int i = threadIdx.x; i < k; i += blockDim.x) xs[i] = to_float(src[i]);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* wr = w + (size_t)row * k;
  float sum = 0.f;
  if ((k & 3) == 0) {
    for (int i = lane * 4; i < k; i += 128) {
      const float4 a = *reinterpret_cast<const float4*>(wr + i);
      sum = fmaf(xs[i], a.x, sum);
      sum = fmaf(xs[i + 1], a.y, sum);
      sum = fmaf(xs[i + 2], a.z, sum);
      sum = fmaf(xs[i + 3], a.w, sum);
    }
  } else {
    for (int i = lane; i < k; i += 32) sum = fmaf(xs[i], wr[i], sum);
  }
  sum = warp_sum(sum);
  if (lane == 0) out[(size_t)token * rows + row] = sum;
}

// x [n, k] (bfloat16 or 32-bit), w [rows, k] 32-bit, out [n, rows] 32-bit
FE_EXPORT int fe_moe_logits(const void* x, int x_dtype, const float* w, float* out, int n, int rows, int k, cudaStream_t stream) {
  if (n <= 0 || rows <= 0) return 0;
  if (k <= 0 || (size_t)k * sizeof(float) > 200 * 1024 || ((uintptr_t)w & 15)) return FE_ERR_BAD_SHAPE;
  const size_t smem = (size_t)k * sizeof(float);
  dim3 grid(n, (rows + 7) / 8);
  int rc;
  if (x_dtype == FE_DTYPE_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_logits_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rc = fe_launch_dependent(moe_logits_kernel<bf16>, grid, dim3(256), smem, stream, (const bf16*)x, w, out, rows, k);
  } else if (x_dtype == FE_DTYPE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_logits_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    rc = fe_launch_dependent(moe_logits_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, w, out, rows, k);
  } else return FE_ERR_BAD_DTYPE;
  return rc ? rc : fe_last_error();
}

// ---------------------------------------------------------------------------
// route
// ---------------------------------------------------------------------------
#define MOE_MAX_GROUPS 64

// What the plain router does not have (all off when zero / null).
struct MoeRouteExtras {
  int identity;             // the router's last `identity` outputs stand for units that hand their input on;
                            //   they all count as one expert, number `experts`, that has no tiles
  const float* correction;  // [experts + identity] or null: added to the score for the choice only
  int group_count;          // 0, or: the outputs form this many equal groups of neighbours, a group's
  int group_keep;           //   mark is its largest choice score, and only the best group_keep can be chosen
  float renorm_floor;       // with renormalise: weight = score / (sum of the chosen + renorm_floor)
  float weight_scale;       // every weight is multiplied by this
  int group_top2;           // a group's mark is the sum of its two largest choice scores (of its one, in groups of one)
};

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, long long ld, int n_tokens, int experts, int top, int softmax_scores,
                 int renormalise, MoeRouteExtras x, int* __restrict__ slot_expert, float* __restrict__ slot_weight,
                 int* __restrict__ slot_rank, int* __restrict__ counts) {
  __shared__ float group_mark[4][MOE_MAX_GROUPS];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x * (blockDim.x >> 5) + warp;
  if (token >= n_tokens) return;
  const int outputs = experts + x.identity;
  const float* z = logits + (size_t)token * ld;
  float big = -INFINITY, norm = 1.f;
  if (softmax_scores) {
    for (int e = lane; e < outputs; e += 32) big = fmaxf(big, z[e]);
    big = warp_max(big);
    float sum = 0.f;
    for (int e = lane; e < outputs; e += 32) sum += expf(z[e] - big);
    norm = 1.f / warp_sum(sum);
  }
  auto score_of = [&](int e) { return softmax_scores ? expf(z[e] - big) * norm : 1.f / (1.f + expf(-z[e])); };
  auto choice_of = [&](int e) { return x.correction ? score_of(e) + x.correction[e] : score_of(e); };
  const int per_group = x.group_count > 0 ? outputs / x.group_count : outputs;
  if (x.group_count > 0) {
    for (int g = 0; g < x.group_count; ++g) {
      float mark = -INFINITY;
      int mark_e = -1;
      for (int e = g * per_group + lane; e < (g + 1) * per_group; e += 32) {
        const float c = choice_of(e);
        if (c > mark) { mark = c; mark_e = e; }
      }
      const float first = warp_max(mark);
      const bool holds_first = mark == first && mark_e >= 0;      // this lane's best is the group's largest
      mark = first;
      if (x.group_top2 && per_group > 1) {
        // the largest is left out at its lowest index (equal scores elsewhere still count), then the largest of the rest
        int first_e = holds_first ? mark_e : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) first_e = min(first_e, __shfl_xor_sync(0xffffffffu, first_e, o));
        float second = -INFINITY;
        for (int e = g * per_group + lane; e < (g + 1) * per_group; e += 32)
          if (e != first_e) second = fmaxf(second, choice_of(e));
        mark = first + warp_max(second);
      }
      if (lane == 0) group_mark[warp][g] = mark;
    }
    __syncwarp();
  }
  // whether output e may be chosen: fewer than group_keep groups rank ahead of its own (ties: the lower index)
  auto open_to_choice = [&](int e) {
    if (x.group_count <= 0) return true;
    const int g = e / per_group;
    const float mine = group_mark[warp][g];
    int ahead = 0;
    for (int o = 0; o < x.group_count; ++o) {
      const float other = group_mark[warp][o];
      ahead += (other > mine || (other == mine && o < g)) ? 1 : 0;
    }
    return ahead < x.group_keep;
  };
  int chosen[MOE_MAX_TOP];
  float weight[MOE_MAX_TOP];
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= chosen[j] == e;
      if (taken || !open_to_choice(e)) continue;
      const float score = choice_of(e);
      if (score > best || (score == best && e < best_e) || best_e == 0x7fffffff) { best = score; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other_e != 0x7fffffff && (best_e == 0x7fffffff || other > best || (other == best && other_e < best_e))) {
        best = other;
        best_e = other_e;
      }
    }
    chosen[k] = best_e;
    // the weight comes from the score without the correction
    weight[k] = x.correction ? score_of(min(best_e, outputs - 1)) : best;
    total += weight[k];
  }
  if (lane == 0) {
    for (int k = 0; k < top; ++k) {
      const int slot = token * top + k;
      const int e = min(chosen[k], experts);       // every identity unit is expert number `experts`
      slot_expert[slot] = e;
      slot_weight[slot] = (renormalise ? weight[k] / (total + x.renorm_floor) : weight[k]) * x.weight_scale;
      slot_rank[slot] = atomicAdd(&counts[e], 1);
    }
  }
}

// ---------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_plan_kernel(int* __restrict__ counts, int experts, int tiled, int slots, int max_tiles, int tile_rows, const int* __restrict__ slot_expert,
                const int* __restrict__ slot_rank, int* __restrict__ offsets, int* __restrict__ tile_expert,
                int* __restrict__ tile_row, int* __restrict__ slot_row, int* __restrict__ row_slot) {
  extern __shared__ int start[];      // [experts + 1]
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    int at = 0, tile = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      const int count = counts[e];
      // experts from `tiled` on (identity units) have rows but no products
      for (int r = 0; e < tiled && r < count && tile < max_tiles; r += tile_rows, ++tile) {
        tile_expert[tile] = e;
        tile_row[tile] = at + r;
      }
      at += count;
      counts[e] = 0;
    }
    start[experts] = at;
    for (; tile < max_tiles; ++tile) tile_expert[tile] = -1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
  for (int s = threadIdx.x; s < slots; s += blockDim.x) {
    const int row = start[slot_expert[s]] + slot_rank[s];
    slot_row[s] = row;
    row_slot[row] = s;
  }
}

// ---------------------------------------------------------------------------
// gather: sorted row r = the activations of its slot's token, times the slot's weight where
// the weight scales the expert's input (32-bit product, one rounding).  For the products that
// fetch their operands by TMA and so need the rows side by side.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ x, int width, int top, const int* __restrict__ row_slot,
                  const float* __restrict__ slot_weight, T* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int slot = row_slot[row];
  const float scale = slot_weight ? slot_weight[slot] : 1.f;
  const T* src = x + (size_t)(slot / top) * width;
  T* dst = out + (size_t)row * width;
  if ((width & 7) == 0) {
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      float v[8];
      load8(src + i, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= scale;
      store8(dst + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<T>(to_float(src[i]) * scale);
  }
}

FE_EXPORT int fe_moe_gather(const void* x, int dtype, int width, int top, int slots, const int* row_slot,
                            const float* slot_weight, void* out, cudaStream_t stream) {
  if (slots <= 0) return 0;
  int rc;
  if (dtype == FE_DTYPE_BF16)
    rc = fe_launch_dependent(moe_gather_kernel<bf16>, dim3(slots), dim3(256), 0, stream, (const bf16*)x, width, top, row_slot, slot_weight, (bf16*)out);
  else if (dtype == FE_DTYPE_F32)
    rc = fe_launch_dependent(moe_gather_kernel<float>, dim3(slots), dim3(256), 0, stream, (const float*)x, width, top, row_slot, slot_weight, (float*)out);
  else return FE_ERR_BAD_DTYPE;
  return rc ? rc : fe_last_error();
}

// ---------------------------------------------------------------------------
// grouped products, plain FFMA
// ---------------------------------------------------------------------------
struct MoeProduct {
  const void* a;            // GATHER: the tokens' activations [tokens, lda]; else the sorted rows [slots, lda]
  long long lda;
  const void* w1;           // [experts, n, k]
  const void* w2;           // DUAL: the second matrix of every expert (up), same shape
  void* out;                // sorted rows [slots, n]
  int n, k, top;
  const int* offsets;       // [experts + 1]
  const int* tile_expert;
  const int* tile_row;
  const int* row_slot;      // GATHER: slot of a sorted row (token = slot / top)
  const float* slot_weight; // GATHER: or null; the row is multiplied by its slot's weight
  MoeAct act;
};

template <typename TX, typename TW, typename TY, bool DUAL>
__global__ void __launch_bounds__(256) moe_grouped_kernel(MoeProduct p) {
  __shared__ float xs[MOE_BK][MOE_BM + 4];
  __shared__ float ws[DUAL ? 2 : 1][MOE_BK][MOE_BN + 4];
  __shared__ long long row_at[MOE_BM];     // where the tile's rows start in `a` (-1: no row)
  __shared__ float row_scale[MOE_BM];
  pdl_trigger();
  pdl_wait();
  const int expert = p.tile_expert[blockIdx.y];
  if (expert < 0) return;
  const int row0 = p.tile_row[blockIdx.y];
  const int rows = min(MOE_BM, p.offsets[expert + 1] - row0);
  const int col0 = blockIdx.x * MOE_BN;
  const int tid = threadIdx.x;
  if (tid < MOE_BM) {
    long long at = -1;
    float scale = 1.f;
    if (tid < rows) {
      if (p.row_slot != nullptr) {
        const int slot = p.row_slot[row0 + tid];
        at = (long long)(slot / p.top) * p.lda;
        if (p.slot_weight != nullptr) scale = p.slot_weight[slot];
      } else {
        at = (long long)(row0 + tid) * p.lda;
      }
    }
    row_at[tid] = at;
    row_scale[tid] = scale;
  }
  __syncthreads();
  const TX* a = (const TX*)p.a;
  const TW* w1 = (const TW*)p.w1 + (size_t)expert * p.n * p.k;
  const TW* w2 = DUAL ? (const TW*)p.w2 + (size_t)expert * p.n * p.k : nullptr;
  const int ty = tid >> 4, tx = tid & 15;
  const int lr = tid >> 2, lk = (tid & 3) << 2;
  float acc[DUAL ? 2 : 1][4][4];
#pragma unroll
  for (int m = 0; m < (DUAL ? 2 : 1); ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][i][j] = 0.f;
  const long long my_row = row_at[lr];
  const float my_scale = row_scale[lr];
  for (int k0 = 0; k0 < p.k; k0 += MOE_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + lk + e;
      const int wr = col0 + lr;
      xs[lk + e][lr] = (my_row >= 0 && kk < p.k) ? to_float(a[my_row + kk]) * my_scale : 0.f;
      ws[0][lk + e][lr] = (wr < p.n && kk < p.k) ? to_float(w1[(size_t)wr * p.k + kk]) : 0.f;
      if (DUAL) ws[1][lk + e][lr] = (wr < p.n && kk < p.k) ? to_float(w2[(size_t)wr * p.k + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MOE_BK; ++kk) {
      float av[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
        float bv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = ws[m][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][i][j] = fmaf(av[i], bv[j], acc[m][i][j]);
      }
    }
    __syncthreads();
  }
  TY* out = (TY*)p.out;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c >= p.n) continue;
      const float v = DUAL ? moe_act(acc[0][i][j], acc[DUAL ? 1 : 0][i][j], p.act) : moe_unary(acc[0][i][j], p.act);
      out[(size_t)(row0 + r) * p.n + c] = from_float<TY>(v);
    }
  }
}

// ---------------------------------------------------------------------------
// grouped products on mma.sync (bfloat16 operands, 32-bit sums): a block of four warps owns
// 64 rows x 64 columns, a warp sixteen rows; k in steps of 32 through shared memory.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned moe_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void moe_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(moe_smem(p)));
}
__device__ __forceinline__ void moe_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

#define MOE_TK 32
#define MOE_TS (MOE_TK + 8)      // row stride of the tiles in shared memory (bank spread)

template <typename TY, bool DUAL>
__global__ void __launch_bounds__(128) moe_grouped_mma_kernel(MoeProduct p) {
  __shared__ __align__(16) bf16 As[2][MOE_BM * MOE_TS];
  __shared__ __align__(16) bf16 Bs[2][DUAL ? 2 : 1][MOE_BN * MOE_TS];
  __shared__ long long row_at[MOE_BM];
  __shared__ float row_scale[MOE_BM];
  pdl_trigger();
  pdl_wait();
  const int expert = p.tile_expert[blockIdx.y];
  if (expert < 0) return;
  const int row0 = p.tile_row[blockIdx.y];
  const int rows = min(MOE_BM, p.offsets[expert + 1] - row0);
  const int col0 = blockIdx.x * MOE_BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MOE_BM) {
    long long at = -1;
    float scale = 1.f;
    if (tid < rows) {
      if (p.row_slot != nullptr) {
        const int slot = p.row_slot[row0 + tid];
        at = (long long)(slot / p.top) * p.lda;
        if (p.slot_weight != nullptr) scale = p.slot_weight[slot];
      } else {
        at = (long long)(row0 + tid) * p.lda;
      }
    }
    row_at[tid] = at;
    row_scale[tid] = scale;
  }
  __syncthreads();
  const bf16* a = (const bf16*)p.a;
  const bf16* w[2] = {(const bf16*)p.w1 + (size_t)expert * p.n * p.k,
                      DUAL ? (const bf16*)p.w2 + (size_t)expert * p.n * p.k : nullptr};
  // a thread stages 16 elements (two 16-byte pieces) of one row of every tile: row = tid / 2
  const int lr = tid >> 1, lc = (tid & 1) * 16;
  const long long my_row = row_at[lr];
  const float my_scale = row_scale[lr];
  const bool scaled = p.slot_weight != nullptr && p.row_slot != nullptr;
  auto stage = [&](int k0, int buf) {
#pragma unroll
    for (int piece = 0; piece < 2; ++piece) {
      const int kk = k0 + lc + piece * 8;
      uint4 value = make_uint4(0, 0, 0, 0);
      if (my_row >= 0 && kk < p.k) {
        value = *reinterpret_cast<const uint4*>(a + my_row + kk);
        if (scaled) {
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&value);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            h[i] = __floats2bfloat162_rn(f.x * my_scale, f.y * my_scale);
          }
        }
      }
      *reinterpret_cast<uint4*>(&As[buf][lr * MOE_TS + lc + piece * 8]) = value;
#pragma unroll
      for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
        uint4 wv = make_uint4(0, 0, 0, 0);
        if (col0 + lr < p.n && kk < p.k) wv = *reinterpret_cast<const uint4*>(w[m] + (size_t)(col0 + lr) * p.k + kk);
        *reinterpret_cast<uint4*>(&Bs[buf][m][lr * MOE_TS + lc + piece * 8]) = wv;
      }
    }
  };
  float acc[DUAL ? 2 : 1][MOE_BN / 8][4];
#pragma unroll
  for (int m = 0; m < (DUAL ? 2 : 1); ++m)
#pragma unroll
    for (int j = 0; j < MOE_BN / 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[m][j][c] = 0.f;
  const int k_steps = (p.k + MOE_TK - 1) / MOE_TK;
  stage(0, 0);
  __syncthreads();
  for (int ks = 0; ks < k_steps; ++ks) {
    const int buf = ks & 1;
    if (ks + 1 < k_steps) stage((ks + 1) * MOE_TK, buf ^ 1);
#pragma unroll
    for (int kk = 0; kk < MOE_TK / 16; ++kk) {
      unsigned af[4];
      moe_ldsm4(af[0], af[1], af[2], af[3], &As[buf][(warp * 16 + (lane & 15)) * MOE_TS + kk * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
#pragma unroll
        for (int j = 0; j < MOE_BN / 8; j += 2) {
          unsigned b0, b1, b2, b3;
          moe_ldsm4(b0, b1, b2, b3, &Bs[buf][m][((j + (lane >> 4)) * 8 + (lane & 7)) * MOE_TS + kk * 16 + ((lane >> 3) & 1) * 8]);
          moe_mma(acc[m][j], af, b0, b1);
          moe_mma(acc[m][j + 1], af, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  TY* out = (TY*)p.out;
  const int quad = lane >> 2, pair = lane & 3;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + quad + 8 * h;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < MOE_BN / 8; ++j) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = col0 + j * 8 + pair * 2 + c;
        if (col >= p.n) continue;
        const float v = DUAL ? moe_act(acc[0][j][2 * h + c], acc[DUAL ? 1 : 0][j][2 * h + c], p.act) : moe_unary(acc[0][j][2 * h + c], p.act);
        out[(size_t)(row0 + r) * p.n + col] = from_float<TY>(v);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------
template <typename TS, typename TO>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ rows, const int* __restrict__ slot_row, const float* __restrict__ slot_weight,
                   int top, int width, const TS* __restrict__ shared, const float* __restrict__ shared_logit,
                   long long shared_ld, const int* __restrict__ slot_expert, int experts, const void* __restrict__ input,
                   int input_bf16, TO* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  float gate = 0.f;
  if (shared != nullptr) gate = shared_logit ? 1.f / (1.f + expf(-shared_logit[(size_t)token * shared_ld])) : 1.f;
  if ((width & 3) == 0) {
    // four neighbouring columns per thread: 16-byte loads of the rows
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < width; c += gridDim.y * blockDim.x * 4) {
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < top; ++k) {
        const int slot = token * top + k;
        float v[4];
        if (input != nullptr && slot_expert[slot] >= experts) {
          // an identity unit: the row is the token's own input
          if (input_bf16) load4((const bf16*)input + (size_t)token * width + c, v);
          else load4((const float*)input + (size_t)token * width + c, v);
        } else {
          load4(rows + (size_t)slot_row[slot] * width + c, v);
        }
        const float w = slot_weight ? slot_weight[slot] : 1.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) sum[e] += slot_weight ? v[e] * w : v[e];
      }
      if (shared != nullptr) {
        float v[4];
        load4(shared + (size_t)token * width + c, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) sum[e] = fmaf(gate, v[e], sum[e]);
      }
      store4(out + (size_t)token * width + c, sum);
    }
    return;
  }
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int slot = token * top + k;
      float v;
      if (input != nullptr && slot_expert[slot] >= experts)
        v = input_bf16 ? to_float(((const bf16*)input)[(size_t)token * width + c]) : ((const float*)input)[(size_t)token * width + c];
      else
        v = rows[(size_t)slot_row[slot] * width + c];
      sum += slot_weight ? v * slot_weight[slot] : v;
    }
    if (shared != nullptr) sum = fmaf(gate, to_float(shared[(size_t)token * width + c]), sum);
    out[(size_t)token * width + c] = from_float<TO>(sum);
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
// Row tiles to launch for `slots` rows spread over `experts` in tiles of `tile_rows` rows
// (0: the 64 of this file's own products): every expert may end with a tile that is not full.
FE_EXPORT int fe_moe_max_tiles(int slots, int experts, int tile_rows) {
  if (tile_rows <= 0) tile_rows = MOE_BM;
  return (slots + tile_rows - 1) / tile_rows + (experts < slots ? experts : slots);
}

// logits [tokens, ld] (the first `experts` + `identity` columns); counts [experts (+ 1 with identity
// units)] must be zero and is zero again afterwards; slot_* and row_slot [tokens * top]; offsets
// [experts + 1 (+ 1)]; tile_* [max_tiles]
FE_EXPORT int fe_moe_route(const float* logits, long long ld, int n_tokens, int experts, int top, int softmax_scores,
                           int renormalise, int* counts, int* slot_expert, float* slot_weight, int* slot_rank,
                           int* slot_row, int* row_slot, int* offsets, int* tile_expert, int* tile_row, int max_tiles,
                           int tile_rows, int identity, const float* correction, int group_count, int group_keep,
                           float renorm_floor, float weight_scale, int group_top2, cudaStream_t stream) {
  if (tile_rows <= 0) tile_rows = MOE_BM;
  if (n_tokens <= 0) return 0;
  if (identity < 0) return FE_ERR_BAD_SHAPE;
  const int outputs = experts + identity;
  if (experts < 1 || top < 1 || top > outputs || top > MOE_MAX_TOP || ld < outputs) return FE_ERR_BAD_SHAPE;
  if (group_count < 0 || group_count > MOE_MAX_GROUPS) return FE_ERR_BAD_SHAPE;
  if (group_count > 0 && (outputs % group_count || group_keep < 1 || group_keep > group_count ||
                          (long long)outputs / group_count * group_keep < top)) return FE_ERR_BAD_SHAPE;
  if ((long long)n_tokens * top > 0x7fffffffLL) return FE_ERR_TOO_LARGE;
  // with identity units the tables have one more expert: the one that stands for all of them
  const int listed = experts + (identity > 0 ? 1 : 0);
  if ((size_t)(listed + 1) * sizeof(int) > 160 * 1024) return FE_ERR_TOO_LARGE;
  MoeRouteExtras extras{identity, correction, group_count, group_keep, renorm_floor, weight_scale, group_top2};
  int rc = fe_launch_dependent(moe_route_kernel, dim3((n_tokens + 3) / 4), dim3(128), 0, stream, logits, ld, n_tokens,
                               experts, top, softmax_scores, renormalise, extras, slot_expert, slot_weight, slot_rank, counts);
  if (rc) return rc;
  const size_t smem = (size_t)(listed + 1) * sizeof(int);
  if (smem > 48 * 1024) cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  rc = fe_launch_dependent(moe_plan_kernel, dim3(1), dim3(1024), smem, stream, counts, listed, experts, n_tokens * top, max_tiles, tile_rows,
                           (const int*)slot_expert, (const int*)slot_rank, offsets, tile_expert, tile_row, slot_row, row_slot);
  return rc ? rc : fe_last_error();
}

// One grouped product.  dual: out = act(a w1^T, a w2^T); gather: rows of `a` are the tokens'
// (row_slot gives the slot, slot / top the token), multiplied by slot_weight when given.
FE_EXPORT int fe_moe_grouped(const void* a, int a_dtype, long long lda, const void* w1, const void* w2, int w_dtype,
                             void* out, int out_dtype, int n, int k, int top, int max_tiles, const int* offsets,
                             const int* tile_expert, const int* tile_row, const int* row_slot, const float* slot_weight,
                             int act, float limit, float slope, int use_mma, cudaStream_t stream) {
  if (max_tiles <= 0 || n <= 0) return 0;
  if (k <= 0 || max_tiles > 65535 || lda < k) return FE_ERR_BAD_SHAPE;
  const bool dual = w2 != nullptr;
  MoeProduct p{a, lda, w1, w2, out, n, k, top, offsets, tile_expert, tile_row, row_slot, slot_weight, MoeAct{act, limit, slope}};
  dim3 grid((n + MOE_BN - 1) / MOE_BN, max_tiles);
  int rc = FE_ERR_BAD_DTYPE;
  if (use_mma && a_dtype == FE_DTYPE_BF16 && w_dtype == FE_DTYPE_BF16) {
    if (k % 8 || lda % 8 || ((uintptr_t)a | (uintptr_t)w1 | (uintptr_t)w2) % 16) return FE_ERR_BAD_ALIGN;
    if (dual && out_dtype == FE_DTYPE_BF16) rc = fe_launch_dependent(moe_grouped_mma_kernel<bf16, true>, grid, dim3(128), 0, stream, p);
    else if (dual && out_dtype == FE_DTYPE_F32) rc = fe_launch_dependent(moe_grouped_mma_kernel<float, true>, grid, dim3(128), 0, stream, p);
    else if (!dual && out_dtype == FE_DTYPE_F32) rc = fe_launch_dependent(moe_grouped_mma_kernel<float, false>, grid, dim3(128), 0, stream, p);
    else if (!dual && out_dtype == FE_DTYPE_BF16) rc = fe_launch_dependent(moe_grouped_mma_kernel<bf16, false>, grid, dim3(128), 0, stream, p);
    return rc ? rc : fe_last_error();
  }
#define MOE_LAUNCH(TX, TW, TY)                                                                                      \
  rc = dual ? fe_launch_dependent(moe_grouped_kernel<TX, TW, TY, true>, grid, dim3(256), 0, stream, p)              \
            : fe_launch_dependent(moe_grouped_kernel<TX, TW, TY, false>, grid, dim3(256), 0, stream, p)
  const int code = a_dtype * 4 + w_dtype * 2 + out_dtype;
  switch (code) {
    case 0: MOE_LAUNCH(float, float, float); break;
    case 2: MOE_LAUNCH(float, bf16, float); break;
    case 4: MOE_LAUNCH(bf16, float, float); break;
    case 6: MOE_LAUNCH(bf16, bf16, float); break;
    case 7: MOE_LAUNCH(bf16, bf16, bf16); break;
    default: return FE_ERR_BAD_DTYPE;
  }
#undef MOE_LAUNCH
  return rc ? rc : fe_last_error();
}

FE_EXPORT int fe_moe_combine(const float* rows, const int* slot_row, const float* slot_weight, int top, int width,
                             const void* shared, int shared_dtype, const float* shared_logit, long long shared_ld,
                             void* out, int out_dtype, int n_tokens, const int* slot_expert, int experts,
                             const void* input, int input_dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (input != nullptr && (slot_expert == nullptr || (input_dtype != FE_DTYPE_F32 && input_dtype != FE_DTYPE_BF16)))
    return FE_ERR_BAD_DTYPE;
  const int input_bf16 = input_dtype == FE_DTYPE_BF16 ? 1 : 0;
  int pieces = (width & 3) == 0 ? (width / 4 + 255) / 256 : (width + 255) / 256;
  if (pieces > 32) pieces = 32;
  dim3 grid(n_tokens, pieces);
  int rc = FE_ERR_BAD_DTYPE;
#define MOE_COMBINE(TS, TO)                                                                                           \
  rc = fe_launch_dependent(moe_combine_kernel<TS, TO>, grid, dim3(256), 0, stream, rows, slot_row, slot_weight, top, \
                           width, (const TS*)shared, shared_logit, shared_ld, slot_expert, experts, input, input_bf16, (TO*)out)
  if (shared == nullptr) shared_dtype = FE_DTYPE_F32;
  if (shared_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32) MOE_COMBINE(float, float);
  else if (shared_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16) MOE_COMBINE(float, bf16);
  else if (shared_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_F32) MOE_COMBINE(bf16, float);
  else if (shared_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16) MOE_COMBINE(bf16, bf16);
  else return FE_ERR_BAD_DTYPE;
#undef MOE_COMBINE
  return rc ? rc : fe_last_error();
}
