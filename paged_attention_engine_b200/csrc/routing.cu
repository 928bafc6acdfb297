// Routing of a mixture of experts, and the element-wise steps around its products.
//
//   scores   s = softmax(z) over all experts (z float32 router logits), or sigmoid(z)
//   choice   c = s + correction (a float32 vector or none); with G groups of neighbouring
//            experts, a group's score is its largest c and only the `keep` best groups can be
//            chosen (the others count as minus infinity); the `top` largest c are chosen,
//            the lower index first among equals
//   weights  w_e = s_e / (sum of the chosen s + eps) * scale for the chosen, 0 for the others;
//            or, not normalized, w_e = s_e * scale
//
// One warp per token; all arithmetic float32. The kernel leaves the chosen experts, their weights
// and, when asked, the dense row of weights [total experts].
#include "common.cuh"

#include <cfloat>

using namespace pae;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 16;      // 512 experts

struct Route {
  const float* logits;       // [splits, tokens, ld], of which the first `total` columns: the planes of a split product are added in their order
  const float* correction;   // [total] or null
  int* chosen;               // [tokens, top]
  float* weights;            // [tokens, top]
  float* dense;              // [tokens, total] or null
  int tokens, total, top, groups, keep, sigmoid;
  float eps, scale;
  int splits, ld, normalize;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// PER_LANE: experts per lane, 32 * PER_LANE >= total.
template <int PER_LANE>
__global__ void __launch_bounds__(WARPS * 32) route_kernel(const Route p) {
  dependent_launch_prologue();
  extern __shared__ float shared[];                    // per warp: choice [total], group score [groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= p.tokens) return;
  float* choice = shared + (size_t)warp * (p.total + p.groups);
  float* group_score = choice + p.total;
  const float* z = p.logits + (size_t)t * p.ld;
  float s[PER_LANE];
  float top = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    s[j] = -FLT_MAX;
    if (e < p.total) {
      float sum = z[e];
      for (int k = 1; k < p.splits; ++k) sum += z[(size_t)k * p.tokens * p.ld + e];
      s[j] = sum;
    }
    top = fmaxf(top, s[j]);
  }
  if (p.sigmoid) {
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) s[j] = lane + 32 * j < p.total ? 1.f / (1.f + expf(-s[j])) : 0.f;
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      s[j] = lane + 32 * j < p.total ? expf(s[j] - top) : 0.f;
      sum += s[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) s[j] = s[j] / sum;
  }
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    if (e < p.total) {
      choice[e] = s[j] + (p.correction != nullptr ? p.correction[e] : 0.f);
      if (p.dense != nullptr) p.dense[(size_t)t * p.total + e] = 0.f;
    }
  }
  __syncwarp();
  if (p.groups > 0) {
    const int size = p.total / p.groups;
    for (int g = lane; g < p.groups; g += 32) {
      float best = -FLT_MAX;
      for (int i = 0; i < size; ++i) best = fmaxf(best, choice[g * size + i]);
      group_score[g] = best;
    }
    __syncwarp();
    // the `keep` best groups stay (their score is marked taken); afterwards every other group's experts are closed
    for (int k = 0; k < p.keep; ++k) {
      float v = -FLT_MAX;
      int i = INT_MAX;
      for (int g = lane; g < p.groups; g += 32)
        if (group_score[g] != FLT_MAX && (group_score[g] > v || i == INT_MAX)) { v = group_score[g]; i = g; }
      warp_argmax(v, i);
      if (lane == 0 && i != INT_MAX) group_score[i] = FLT_MAX;
      __syncwarp();
    }
    for (int e = lane; e < p.total; e += 32)
      if (group_score[e / size] != FLT_MAX) choice[e] = -INFINITY;
    __syncwarp();
  }
  float chosen_sum = 0.f;
  int mine = 0;                                         // bit j: this lane's expert lane + 32 j is chosen
  for (int k = 0; k < p.top; ++k) {
    float v = -INFINITY;
    int i = INT_MAX;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < p.total && !((mine >> j) & 1) && (i == INT_MAX || choice[e] > v)) { v = choice[e]; i = e; }
    }
    warp_argmax(v, i);
    float score = 0.f;
    if (i != INT_MAX && (i & 31) == lane) {
      mine |= 1 << (i >> 5);
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j)
        if (j == (i >> 5)) score = s[j];
    }
    score = __shfl_sync(0xffffffffu, score, i == INT_MAX ? 0 : (i & 31));
    chosen_sum += score;                                // in the order of the choice, the same on every lane
    if (lane == 0) {
      p.chosen[(size_t)t * p.top + k] = i == INT_MAX ? 0 : i;
      p.weights[(size_t)t * p.top + k] = score;
    }
  }
  __syncwarp();
  const float factor = p.normalize ? p.scale / (chosen_sum + p.eps) : p.scale;
  for (int k = lane; k < p.top; k += 32) {
    const float w = p.weights[(size_t)t * p.top + k] * factor;
    p.weights[(size_t)t * p.top + k] = w;
    if (p.dense != nullptr) p.dense[(size_t)t * p.total + p.chosen[(size_t)t * p.top + k]] = w;
  }
}

// ---------------------------------------------------------------------------------------
// The experts' products over the chosen (token, expert) pairs only. The pairs are sorted by
// expert into rows of a staging matrix, every expert's rows padded to whole tiles of `tile`
// rows, so that a tile of the grouped product reads one expert's weights:
//
//   rank[i]        the pair's place among its expert's rows (any order: a row's product does not
//                  depend on where in a tile it lies), -1 for an expert without tensors
//   first[e]       the expert's first row; tiles[2 j], tiles[2 j + 1]: tile j's expert (-1: unused)
//                  and how many of its rows are pairs; the entry after the last tile: how many
//                  tiles are in use (they are the first ones)
//   rows[i]        the pair's row, -1 for an expert without tensors
// ---------------------------------------------------------------------------------------
__global__ void expert_rank_kernel(int* __restrict__ rank, int* __restrict__ counts, const int* __restrict__ chosen, int pairs,
                                   int experts) {
  dependent_launch_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = chosen[i];
  rank[i] = (e >= 0 && e < experts) ? atomicAdd(counts + e, 1) : -1;
}

__global__ void __launch_bounds__(256) expert_tiles_kernel(int* __restrict__ first, int* __restrict__ tiles,
                                                            const int* __restrict__ counts, int experts, int tile, int max_tiles) {
  dependent_launch_prologue();
  if (threadIdx.x == 0) {
    int at = 0;                                         // in tiles
    for (int e = 0; e < experts; ++e) {
      first[e] = at * tile;
      at += (counts[e] + tile - 1) / tile;
    }
    tiles[2 * max_tiles] = min(at, max_tiles);          // the tiles in use are the first ones
    tiles[2 * max_tiles + 1] = 0;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < max_tiles; j += blockDim.x) {
    tiles[2 * j] = -1;
    tiles[2 * j + 1] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = counts[e], t0 = first[e] / tile;
    for (int j = 0; j * tile < n && t0 + j < max_tiles; ++j) {
      tiles[2 * (t0 + j)] = e;
      tiles[2 * (t0 + j) + 1] = min(tile, n - j * tile);
    }
  }
}

// dst[c] = w * src[c] for c < width, a float32 product rounded once; 16 bytes a step where both rows allow it.
template <typename T>
__device__ __forceinline__ void scaled_row(T* __restrict__ dst, const T* __restrict__ src, float w, int width, int lane, int lanes) {
  constexpr int PER = 16 / (int)sizeof(T);
  if ((width % PER) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
    for (int c = lane; c < width / PER; c += lanes) {
      int4 in = ((const int4*)src)[c], out;
      const T* a = (const T*)&in;
      T* b = (T*)&out;
#pragma unroll
      for (int j = 0; j < PER; ++j) b[j] = from_float<T>(w * to_float(a[j]));
      ((int4*)dst)[c] = out;
    }
  } else {
    for (int c = lane; c < width; c += lanes) dst[c] = from_float<T>(w * to_float(src[c]));
  }
}

// One block per pair: its row is its expert's first row plus its rank; the token's input goes there.
template <typename T>
__global__ void __launch_bounds__(128) expert_gather_kernel(T* __restrict__ staged, int* __restrict__ rows, const T* __restrict__ x,
                                                            const int* __restrict__ chosen, const int* __restrict__ rank,
                                                            const int* __restrict__ first, const float* __restrict__ scale, int top,
                                                            int width, int max_rows) {
  dependent_launch_prologue();
  const int i = blockIdx.x;
  const int r = rank[i];
  int row = -1;
  if (r >= 0) {
    row = first[chosen[i]] + r;
    if (row >= max_rows) row = -1;                      // cannot happen with the bound the caller computes
  }
  if (threadIdx.x == 0) rows[i] = row;
  if (row < 0) return;
  const T* src = x + (size_t)(i / top) * width;
  T* dst = staged + (size_t)row * width;
  if (scale != nullptr) {                               // an expert that is weighted on its input
    scaled_row(dst, src, scale[i], width, (int)threadIdx.x, (int)blockDim.x);
  } else if (((sizeof(T) * width) & 15) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
    const int n = (int)(sizeof(T) * width / 16);
    for (int c = threadIdx.x; c < n; c += blockDim.x) ((int4*)dst)[c] = ((const int4*)src)[c];
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
  }
}

// The same three steps for a step of few pairs (decoding) in ONE block: counts, first rows and rows
// live in shared memory, a warp copies a pair's input row.
constexpr int SMALL_PAIRS = 2048, SMALL_THREADS = 1024;

template <typename T>
__global__ void __launch_bounds__(SMALL_THREADS) expert_plan_small_kernel(int* __restrict__ tiles, int* __restrict__ rows,
                                                                          T* __restrict__ staged, const T* __restrict__ x,
                                                                          const int* __restrict__ chosen, const float* __restrict__ scale,
                                                                          int pairs, int top, int experts, int tile, int max_tiles, int width) {
  dependent_launch_prologue();
  __shared__ int counts[32 * MAX_PER_LANE], first[32 * MAX_PER_LANE], row_of[SMALL_PAIRS];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  for (int j = threadIdx.x; j < max_tiles; j += blockDim.x) {
    tiles[2 * j] = -1;
    tiles[2 * j + 1] = 0;
  }
  __syncthreads();
  int rank[SMALL_PAIRS / SMALL_THREADS];
#pragma unroll
  for (int n = 0; n < SMALL_PAIRS / SMALL_THREADS; ++n) {
    const int i = threadIdx.x + n * SMALL_THREADS;
    rank[n] = -1;
    if (i < pairs) {
      const int e = chosen[i];
      if (e >= 0 && e < experts) rank[n] = atomicAdd(counts + e, 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = at * tile;
      at += (counts[e] + tile - 1) / tile;
    }
    tiles[2 * max_tiles] = min(at, max_tiles);
    tiles[2 * max_tiles + 1] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = counts[e], t0 = first[e] / tile;
    for (int j = 0; j * tile < n && t0 + j < max_tiles; ++j) {
      tiles[2 * (t0 + j)] = e;
      tiles[2 * (t0 + j) + 1] = min(tile, n - j * tile);
    }
  }
#pragma unroll
  for (int n = 0; n < SMALL_PAIRS / SMALL_THREADS; ++n) {
    const int i = threadIdx.x + n * SMALL_THREADS;
    if (i < pairs) {
      int row = rank[n] >= 0 ? first[chosen[i]] + rank[n] : -1;
      if (row >= max_tiles * tile) row = -1;
      row_of[i] = row;
      rows[i] = row;
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = warp; i < pairs; i += SMALL_THREADS / 32) {
    const int row = row_of[i];
    if (row < 0) continue;
    const T* src = x + (size_t)(i / top) * width;
    T* dst = staged + (size_t)row * width;
    if (scale != nullptr) {
      scaled_row(dst, src, scale[i], width, lane, 32);
    } else if (((sizeof(T) * width) & 15) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
      const int n16 = (int)(sizeof(T) * width / 16);
      for (int c = lane; c < n16; c += 32) ((int4*)dst)[c] = ((const int4*)src)[c];
    } else {
      for (int c = lane; c < width; c += 32) dst[c] = src[c];
    }
  }
}

// out[t, :] = (base[t, :], itself the sum of base_planes planes) + sum over the token's chosen experts k, in the order of the choice, of
// weights[t, k] * (y[rows[t, k], :] for an expert with tensors, x[t, :] for one that returns its input).
// weights null: every weight is 1. gate (or null): base[t, :] is first multiplied by sigmoid(gate[t, gate_col]),
// the gate itself the sum of gate_planes planes of rows of gate_ld.
template <typename T>
__global__ void expert_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const int* __restrict__ rows,
                                      const float* __restrict__ weights, const T* __restrict__ x, const float* __restrict__ base,
                                      int base_planes, const float* __restrict__ gate, int gate_planes, int gate_ld, int gate_col,
                                      long long tokens, int top, int width, long long total) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int c = (int)(i - t * width);
  float acc = 0.f;                                    // base: the planes of a split product, added in their order
  if (base != nullptr)
    for (int k = 0; k < base_planes; ++k) acc += base[(size_t)k * total + i];
  if (gate != nullptr) {
    float g = 0.f;
    for (int k = 0; k < gate_planes; ++k) g += gate[((size_t)k * tokens + t) * gate_ld + gate_col];
    acc = acc / (1.f + expf(-g));
  }
  for (int k = 0; k < top; ++k) {
    const int row = rows[t * top + k];
    const float w = weights != nullptr ? weights[t * top + k] : 1.f;
    acc += w * (row >= 0 ? y[(size_t)row * width + c] : to_float(x[i]));
  }
  out[i] = acc;
}

// The same sum, four neighbouring columns a thread (width a multiple of 4, float32 rows 16-byte aligned): a
// quarter of the row and weight look-ups and of the gate's exponentials, 16-byte loads and stores.
template <typename T>
__global__ void expert_combine4_kernel(float* __restrict__ out, const float* __restrict__ y, const int* __restrict__ rows,
                                       const float* __restrict__ weights, const T* __restrict__ x, const float* __restrict__ base,
                                       int base_planes, const float* __restrict__ gate, int gate_planes, int gate_ld, int gate_col,
                                       long long tokens, int top, int width, long long total) {
  dependent_launch_prologue();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= total) return;
  const long long t = i / width;
  const int c = (int)(i - t * width);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (base != nullptr)
    for (int k = 0; k < base_planes; ++k) {
      const float4 b = *(const float4*)(base + (size_t)k * total + i);
      acc[0] += b.x, acc[1] += b.y, acc[2] += b.z, acc[3] += b.w;
    }
  if (gate != nullptr) {
    float g = 0.f;
    for (int k = 0; k < gate_planes; ++k) g += gate[((size_t)k * tokens + t) * gate_ld + gate_col];
    const float open = 1.f + expf(-g);
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = acc[j] / open;
  }
  for (int k = 0; k < top; ++k) {
    const int row = rows[t * top + k];
    const float w = weights != nullptr ? weights[t * top + k] : 1.f;
    float v[4];
    if (row >= 0) {
      const float4 r = *(const float4*)(y + (size_t)row * width + c);
      v[0] = r.x, v[1] = r.y, v[2] = r.z, v[3] = r.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = to_float(x[i + j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] += w * v[j];
  }
  *(float4*)(out + i) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

}  // namespace

PAE_EXPORT int pae_route(int* chosen, float* weights, float* dense, const float* logits, int splits, int ld, const float* correction, int tokens,
                         int total, int top, int groups, int keep, int sigmoid, int normalize, float eps, float scale, void* stream) {
  if (tokens == 0) return 0;
  if (total < 1 || total > 32 * MAX_PER_LANE) return fail(2, "route: %d experts (1 to %d)", total, 32 * MAX_PER_LANE);
  if (top < 1 || top > total) return fail(2, "route: %d of %d experts", top, total);
  if (groups < 0 || (groups > 0 && (total % groups || keep < 1 || keep > groups || top > total / groups * keep)))
    return fail(2, "route: %d experts in %d groups of which %d are kept, %d chosen", total, groups, keep, top);
  if (splits < 1) return fail(2, "route: %d planes of logits", splits);
  if (ld < total) return fail(2, "route: %d experts in rows of %d", total, ld);
  Route p{logits, correction, chosen, weights, dense, tokens, total, top, groups, keep, sigmoid, eps, scale, splits, ld, normalize};
  const size_t smem = sizeof(float) * WARPS * (size_t)(total + groups);
  const unsigned blocks = (tokens + WARPS - 1) / WARPS;
  cudaStream_t s = (cudaStream_t)stream;
  if (total <= 32) launch_kernel(route_kernel<1>, blocks, WARPS * 32, smem, s, p);
  else if (total <= 64) launch_kernel(route_kernel<2>, blocks, WARPS * 32, smem, s, p);
  else if (total <= 128) launch_kernel(route_kernel<4>, blocks, WARPS * 32, smem, s, p);
  else if (total <= 256) launch_kernel(route_kernel<8>, blocks, WARPS * 32, smem, s, p);
  else launch_kernel(route_kernel<MAX_PER_LANE>, blocks, WARPS * 32, smem, s, p);
  return check_launch("route");
}

// How many tiles of `tile` rows the pairs of `pairs` (token, expert) choices among `experts`
// experts can need at most: every expert that has a pair may leave one tile partly filled.
PAE_EXPORT int pae_expert_max_tiles(int pairs, int experts, int tile) {
  return (pairs < experts ? pairs : experts) + pairs / tile;
}

// Sorts the pairs chosen [tokens, top] by expert (see above). scale: float32 [tokens, top] or null; with it a
// pair's staged row is scale * the token's input, rounded once. scratch: int32 [experts] counts, then
// [experts] first rows, then [tokens * top] ranks. tiles: int32 [max_tiles + 1, 2]; rows: int32
// [tokens, top]; staged [max_tiles * tile, width] receives the tokens' inputs x [tokens, width].
PAE_EXPORT int pae_expert_plan(int* scratch, int* tiles, int* rows, void* staged, const void* x, const int* chosen, const float* scale,
                               int tokens, int top, int experts, int tile, int max_tiles, int width, int dtype, void* stream) {
  const int pairs = tokens * top;
  if (pairs == 0) return 0;
  if (experts < 1 || tile < 1 || max_tiles < pae_expert_max_tiles(pairs, experts, tile))
    return fail(2, "expert_plan: %d tiles of %d rows for %d pairs over %d experts", max_tiles, tile, pairs, experts);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype != kF32 && dtype != kBF16) return fail(1, "expert_plan: unknown dtype %d", dtype);
  if (pairs <= SMALL_PAIRS && experts <= 32 * MAX_PER_LANE) {
    if (dtype == kF32)
      launch_kernel(expert_plan_small_kernel<float>, 1, SMALL_THREADS, 0, s, tiles, rows, (float*)staged, (const float*)x, chosen, scale, pairs, top, experts, tile, max_tiles, width);
    else
      launch_kernel(expert_plan_small_kernel<__nv_bfloat16>, 1, SMALL_THREADS, 0, s, tiles, rows, (__nv_bfloat16*)staged, (const __nv_bfloat16*)x, chosen, scale, pairs, top, experts, tile, max_tiles, width);
    return check_launch("expert_plan");
  }
  int *counts = scratch, *first = scratch + experts, *rank = scratch + 2 * experts;
  cudaError_t err = cudaMemsetAsync(counts, 0, sizeof(int) * experts, s);
  if (err != cudaSuccess) return fail(100, "expert_plan: %s", cudaGetErrorString(err));
  launch_kernel(expert_rank_kernel, (pairs + 255) / 256, 256, 0, s, rank, counts, chosen, pairs, experts);
  launch_kernel(expert_tiles_kernel, 1, 256, 0, s, first, tiles, (const int*)counts, experts, tile, max_tiles);
  const int max_rows = max_tiles * tile;
  if (dtype == kF32)
    launch_kernel(expert_gather_kernel<float>, pairs, 128, 0, s, (float*)staged, rows, (const float*)x, chosen, (const int*)rank, (const int*)first, scale, top, width, max_rows);
  else if (dtype == kBF16)
    launch_kernel(expert_gather_kernel<__nv_bfloat16>, pairs, 128, 0, s, (__nv_bfloat16*)staged, rows, (const __nv_bfloat16*)x, chosen, (const int*)rank, (const int*)first, scale, top, width, max_rows);
  else return fail(1, "expert_plan: unknown dtype %d", dtype);
  return check_launch("expert_plan");
}

PAE_EXPORT int pae_expert_combine(float* out, const float* y, const int* rows, const float* weights, const void* x, const float* base,
                                  int base_planes, const float* gate, int gate_planes, int gate_ld, int gate_col, int tokens, int top,
                                  int width, int dtype, void* stream) {
  const long long total = (long long)tokens * width;
  if (total == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype != kF32 && dtype != kBF16) return fail(1, "expert_combine: unknown dtype %d", dtype);
  // Four columns a thread pay from a few dozen tokens on (2,048 tokens of 1,536: 25.5 against 40.5 us); a
  // decode step's handful of rows is quicker with a column a thread (8 tokens: 7.8 against 11.9 us). Both
  // do the same operations per element.
  if (total >= 65536 && width % 4 == 0 && ((((uintptr_t)out) | ((uintptr_t)y) | ((uintptr_t)base)) & 15) == 0) {
    const unsigned blocks4 = (unsigned)((total / 4 + 255) / 256);
    if (dtype == kF32) launch_kernel(expert_combine4_kernel<float>, blocks4, 256, 0, s, out, y, rows, weights, (const float*)x, base, base_planes, gate, gate_planes, gate_ld, gate_col, (long long)tokens, top, width, total);
    else launch_kernel(expert_combine4_kernel<__nv_bfloat16>, blocks4, 256, 0, s, out, y, rows, weights, (const __nv_bfloat16*)x, base, base_planes, gate, gate_planes, gate_ld, gate_col, (long long)tokens, top, width, total);
    return check_launch("expert_combine");
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == kF32) launch_kernel(expert_combine_kernel<float>, blocks, 256, 0, s, out, y, rows, weights, (const float*)x, base, base_planes, gate, gate_planes, gate_ld, gate_col, (long long)tokens, top, width, total);
  else if (dtype == kBF16) launch_kernel(expert_combine_kernel<__nv_bfloat16>, blocks, 256, 0, s, out, y, rows, weights, (const __nv_bfloat16*)x, base, base_planes, gate, gate_planes, gate_ld, gate_col, (long long)tokens, top, width, total);
  else return fail(1, "expert_combine: unknown dtype %d", dtype);
  return check_launch("expert_combine");
}

PAE_DEFINE_LAST_ERROR()
