// The element-wise steps of a decoder whose norms compute no statistics (Dynamic Tanh) and whose
// sublayers are normed on both sides:
//
//   norm      dyt(v)[c] = tanh(alpha * v[c]) * w[c] + b[c]          alpha a scalar, w and b vectors
//   write     x'[t, c] = x[t, c] + mult * post(y[t, c]) + extra[t, c]
//             post = the norm after the sublayer (none: y as it is); y may be the planes of a
//             split product, which are added in their order first; extra (or none) is a second
//             stream that joins the residual (the embedding's output before a repeated pass)
//   read      h[t, c] = next(x'[t, c]) in the engine's element type: the norm before the next sublayer
//
// Since no step needs a whole row, the write after a sublayer and the read before the next are
// ONE pass over the stream: every piece is optional, and a launch with the pieces that a caller
// has is what runs. The stream, the sums and the tanh are float32; the read is rounded once.
#include "common.cuh"

using namespace pae;

namespace {

struct DytStep {
  const float* x;          // [tokens, width] the stream
  const float* y;          // [planes, tokens, width] the sublayer's output, or null
  const float* extra;      // [tokens, width] or null
  float* x_new;            // [tokens, width] or null (nothing was added: the stream is x)
  void* normed;            // [tokens, width] or null
  const float *post_alpha, *post_w, *post_b;     // null: y is added as it is
  const float *next_alpha, *next_w, *next_b;     // null: no read
  float mult;
  int planes, width;
  long long total;
};

template <typename TO>
__global__ void __launch_bounds__(256) dyt_step_kernel(const DytStep p) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= p.total) return;
  const int c = (int)(i % p.width);
  float v = p.x[i];
  if (p.y != nullptr) {
    float s = p.y[i];
    for (int k = 1; k < p.planes; ++k) s += p.y[(size_t)k * p.total + i];
    if (p.post_w != nullptr) s = fmaf(tanhf(p.post_alpha[0] * s), p.post_w[c], p.post_b != nullptr ? p.post_b[c] : 0.f);
    v = fmaf(p.mult, s, v);
  }
  if (p.extra != nullptr) v += p.extra[i];
  if (p.x_new != nullptr) p.x_new[i] = v;
  if (p.normed != nullptr)
    ((TO*)p.normed)[i] = from_float<TO>(fmaf(tanhf(p.next_alpha[0] * v), p.next_w[c], p.next_b != nullptr ? p.next_b[c] : 0.f));
}

__device__ __forceinline__ void store4(float* to, const float* h) { *(float4*)to = make_float4(h[0], h[1], h[2], h[3]); }
__device__ __forceinline__ void store4(__nv_bfloat16* to, const float* h) {
  uint2 packed;
  *(__nv_bfloat162*)&packed.x = __floats2bfloat162_rn(h[0], h[1]);
  *(__nv_bfloat162*)&packed.y = __floats2bfloat162_rn(h[2], h[3]);
  *(uint2*)to = packed;
}

// The same, four neighbouring columns a thread (width a multiple of 4, every row 16-byte aligned).
template <typename TO>
__global__ void __launch_bounds__(256) dyt_step4_kernel(const DytStep p) {
  dependent_launch_prologue();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= p.total) return;
  const int c = (int)(i % p.width);
  const float4 x4 = *(const float4*)(p.x + i);
  float v[4] = {x4.x, x4.y, x4.z, x4.w};
  if (p.y != nullptr) {
    const float4 y4 = *(const float4*)(p.y + i);
    float s[4] = {y4.x, y4.y, y4.z, y4.w};
    for (int k = 1; k < p.planes; ++k) {
      const float4 more = *(const float4*)(p.y + (size_t)k * p.total + i);
      s[0] += more.x, s[1] += more.y, s[2] += more.z, s[3] += more.w;
    }
    const float alpha = p.post_w != nullptr ? p.post_alpha[0] : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (p.post_w != nullptr) s[j] = fmaf(tanhf(alpha * s[j]), p.post_w[c + j], p.post_b != nullptr ? p.post_b[c + j] : 0.f);
      v[j] = fmaf(p.mult, s[j], v[j]);
    }
  }
  if (p.extra != nullptr) {
    const float4 e4 = *(const float4*)(p.extra + i);
    v[0] += e4.x, v[1] += e4.y, v[2] += e4.z, v[3] += e4.w;
  }
  if (p.x_new != nullptr) *(float4*)(p.x_new + i) = make_float4(v[0], v[1], v[2], v[3]);
  if (p.normed != nullptr) {
    const float alpha = p.next_alpha[0];
    float h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = fmaf(tanhf(alpha * v[j]), p.next_w[c + j], p.next_b != nullptr ? p.next_b[c + j] : 0.f);
    store4((TO*)p.normed + i, h);
  }
}

bool aligned16(const void* ptr) { return (((uintptr_t)ptr) & 15) == 0; }

}  // namespace

// out_dtype: the element type of `normed` (0 float32, 1 bfloat16).
PAE_EXPORT int pae_dyt_step(float* x_new, void* normed, const float* x, const float* y, int planes, const float* extra,
                            const float* post_alpha, const float* post_w, const float* post_b, float mult,
                            const float* next_alpha, const float* next_w, const float* next_b, int tokens, int width,
                            int out_dtype, void* stream) {
  const long long total = (long long)tokens * width;
  if (total == 0) return 0;
  if (x == nullptr) return fail(2, "dyt_step: no stream");
  if (y != nullptr && planes < 1) return fail(2, "dyt_step: %d planes of a sublayer's output", planes);
  if ((y != nullptr || extra != nullptr) && x_new == nullptr) return fail(2, "dyt_step: a write without a place for the new stream");
  if (post_w != nullptr && post_alpha == nullptr) return fail(2, "dyt_step: a norm after the sublayer without its alpha");
  if (normed != nullptr && (next_w == nullptr || next_alpha == nullptr)) return fail(2, "dyt_step: a read without its norm");
  DytStep p{x, y, extra, x_new, normed, post_alpha, post_w, post_b, next_alpha, next_w, next_b, mult, planes, width, total};
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype != kF32 && out_dtype != kBF16) return fail(1, "dyt_step: unknown dtype %d", out_dtype);
  // The same operations per element either way: a token's numbers do not depend on which form ran.
  if (width % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(extra) && aligned16(x_new) && aligned16(normed)) {
    const unsigned blocks = (unsigned)((total / 4 + 255) / 256);
    if (out_dtype == kF32) launch_kernel(dyt_step4_kernel<float>, blocks, 256, 0, s, p);
    else launch_kernel(dyt_step4_kernel<__nv_bfloat16>, blocks, 256, 0, s, p);
    return check_launch("dyt_step");
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (out_dtype == kF32) launch_kernel(dyt_step_kernel<float>, blocks, 256, 0, s, p);
  else launch_kernel(dyt_step_kernel<__nv_bfloat16>, blocks, 256, 0, s, p);
  return check_launch("dyt_step");
}

PAE_DEFINE_LAST_ERROR()
