// Routing of a mixture of experts, and the element-wise steps around its products.
//
//   scores   s = softmax(z) over all experts (z float32 router logits), or sigmoid(z)
//   choice   c = s + correction (a float32 vector or none); with G groups of neighbouring
//            experts, a group's score is its largest c and only the `keep` best groups can be
//            chosen (the others count as minus infinity); the `top` largest c are chosen,
//            the lower index first among equals
//   weights  w_e = s_e / (sum of the chosen s + eps) * scale for the chosen, 0 for the others
//
// One warp per token; all arithmetic float32. The kernel leaves the chosen experts, their weights
// and the dense row of weights [total experts] that the products' helpers read.
#include "common.cuh"

#include <cfloat>

using namespace pae;

namespace {

constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 16;      // 512 experts

struct Route {
  const float* logits;       // [tokens, total]
  const float* correction;   // [total] or null
  int* chosen;               // [tokens, top]
  float* weights;            // [tokens, top]
  float* dense;              // [tokens, total] or null
  int tokens, total, top, groups, keep, sigmoid;
  float eps, scale;
};

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(WARPS * 32) route_kernel(const Route p) {
  dependent_launch_prologue();
  extern __shared__ float shared[];                    // per warp: choice [total], group score [groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * WARPS + warp;
  if (t >= p.tokens) return;
  float* choice = shared + (size_t)warp * (p.total + p.groups);
  float* group_score = choice + p.total;
  const float* z = p.logits + (size_t)t * p.total;
  float s[MAX_PER_LANE];
  float top = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < p.total ? z[e] : -FLT_MAX;
    top = fmaxf(top, s[j]);
  }
  if (p.sigmoid) {
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) s[j] = lane + 32 * j < p.total ? 1.f / (1.f + expf(-s[j])) : 0.f;
  } else {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      s[j] = lane + 32 * j < p.total ? expf(s[j] - top) : 0.f;
      sum += s[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int j = 0; j < MAX_PER_LANE; ++j) s[j] = s[j] / sum;
  }
#pragma unroll
  for (int j = 0; j < MAX_PER_LANE; ++j) {
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
    for (int j = 0; j < MAX_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < p.total && !((mine >> j) & 1) && (i == INT_MAX || choice[e] > v)) { v = choice[e]; i = e; }
    }
    warp_argmax(v, i);
    float score = 0.f;
    if (i != INT_MAX && (i & 31) == lane) {
      mine |= 1 << (i >> 5);
#pragma unroll
      for (int j = 0; j < MAX_PER_LANE; ++j)
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
  const float factor = p.scale / (chosen_sum + p.eps);
  for (int k = lane; k < p.top; k += 32) {
    const float w = p.weights[(size_t)t * p.top + k] * factor;
    p.weights[(size_t)t * p.top + k] = w;
    if (p.dense != nullptr) p.dense[(size_t)t * p.total + p.chosen[(size_t)t * p.top + k]] = w;
  }
}

// h[t, e * ff + j] *= dense[t, e] for the routed experts' hidden columns (e < experts); columns
// from experts * ff on (a shared expert's) stay. In place, rounded once.
template <typename T>
__global__ void weight_expert_columns_kernel(T* __restrict__ h, const float* __restrict__ dense, int ld_dense, long long total,
                                             int row, int ff, int experts) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / row;
  const int c = (int)(i - t * row), e = c / ff;
  if (e >= experts) return;
  h[i] = from_float<T>(to_float(h[i]) * dense[t * ld_dense + e]);
}

// out[t, :] = x[t, :] * sum of dense[t, first .. first + count) (+ residual[t, :]): the share of the
// experts that return their input, with what the product after it is to add anyway.
template <typename T>
__global__ void identity_share_kernel(float* __restrict__ out, const T* __restrict__ x, const float* __restrict__ dense,
                                      const float* __restrict__ residual, int ld_dense, int first, int count, long long total,
                                      int width) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float* w = dense + (i / width) * ld_dense + first;
  float sum = 0.f;
  for (int k = 0; k < count; ++k) sum += w[k];
  const float v = to_float(x[i]) * sum;
  out[i] = residual != nullptr ? v + residual[i] : v;
}

}  // namespace

PAE_EXPORT int pae_route(int* chosen, float* weights, float* dense, const float* logits, const float* correction, int tokens,
                         int total, int top, int groups, int keep, int sigmoid, float eps, float scale, void* stream) {
  if (tokens == 0) return 0;
  if (total < 1 || total > 32 * MAX_PER_LANE) return fail(2, "route: %d experts (1 to %d)", total, 32 * MAX_PER_LANE);
  if (top < 1 || top > total) return fail(2, "route: %d of %d experts", top, total);
  if (groups < 0 || (groups > 0 && (total % groups || keep < 1 || keep > groups || top > total / groups * keep)))
    return fail(2, "route: %d experts in %d groups of which %d are kept, %d chosen", total, groups, keep, top);
  Route p{logits, correction, chosen, weights, dense, tokens, total, top, groups, keep, sigmoid, eps, scale};
  const size_t smem = sizeof(float) * WARPS * (size_t)(total + groups);
  launch_kernel(route_kernel, (tokens + WARPS - 1) / WARPS, WARPS * 32, smem, (cudaStream_t)stream, p);
  return check_launch("route");
}

PAE_EXPORT int pae_weight_expert_columns(void* h, const float* dense, int ld_dense, int tokens, int row, int ff, int experts,
                                         int dtype, void* stream) {
  const long long total = (long long)tokens * row;
  if (total == 0 || experts == 0) return 0;
  if (ff < 1 || (long long)experts * ff > row || experts > ld_dense) return fail(2, "weight_expert_columns: %d experts of %d columns in rows of %d", experts, ff, row);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch_kernel(weight_expert_columns_kernel<float>, blocks, 256, 0, s, (float*)h, dense, ld_dense, total, row, ff, experts);
  else if (dtype == kBF16) launch_kernel(weight_expert_columns_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)h, dense, ld_dense, total, row, ff, experts);
  else return fail(1, "weight_expert_columns: unknown dtype %d", dtype);
  return check_launch("weight_expert_columns");
}

PAE_EXPORT int pae_identity_share(float* out, const void* x, const float* dense, const float* residual, int ld_dense, int first, int count, int tokens,
                                  int width, int dtype, void* stream) {
  const long long total = (long long)tokens * width;
  if (total == 0) return 0;
  if (first < 0 || count < 1 || first + count > ld_dense) return fail(2, "identity_share: experts %d..%d of %d", first, first + count, ld_dense);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) launch_kernel(identity_share_kernel<float>, blocks, 256, 0, s, out, (const float*)x, dense, residual, ld_dense, first, count, total, width);
  else if (dtype == kBF16) launch_kernel(identity_share_kernel<__nv_bfloat16>, blocks, 256, 0, s, out, (const __nv_bfloat16*)x, dense, residual, ld_dense, first, count, total, width);
  else return fail(1, "identity_share: unknown dtype %d", dtype);
  return check_launch("identity_share");
}

PAE_DEFINE_LAST_ERROR()
