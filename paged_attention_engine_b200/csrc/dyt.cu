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
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == kF32) launch_kernel(dyt_step_kernel<float>, blocks, 256, 0, s, p);
  else if (out_dtype == kBF16) launch_kernel(dyt_step_kernel<__nv_bfloat16>, blocks, 256, 0, s, p);
  else return fail(1, "dyt_step: unknown dtype %d", out_dtype);
  return check_launch("dyt_step");
}

PAE_DEFINE_LAST_ERROR()
