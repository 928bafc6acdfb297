// Hyper-connections: a decoder that keeps S residual streams x_1 .. x_S per token instead of one.
//
//   read    u = sum_s a[s] x_s                       (a null: the plain sum of the streams)
//           h = u / sqrt(mean(u^2) + eps) * w        the sublayer's input, in the engine's dtype
//   write   x'_t = sum_s M[s, t] x_s + b[t] y        every stream from the old ones and from the
//                                                    sublayer's output y; M is indexed [from, to]
//
// One kernel does a write, a read, or the write of one sublayer followed by the read of the next
// (the streams then cross memory once between two sublayers). y may still be the float32 planes
// of a split product; they are added in their order here. The streams are float32 rows
// [tokens, S, width]; rows of [tokens, width] stand for S equal streams (what the embedding
// leaves). All arithmetic is float32 with fused multiply-adds in a fixed order, the sum of
// squares double; a thread keeps the columns it writes for the read, so nothing depends on how
// tokens are batched.
#include "common.cuh"

using namespace pae;

namespace {

constexpr int MAX_STREAMS = 16;       // S * S mixing weights are loaded by the block's 256 threads
constexpr int THREADS = 256;            // a block of a step of many tokens
constexpr int MAX_THREADS = 1024;       // ... of few tokens: a block per token, so the columns are spread over more threads

struct StreamsStep {
  const float* x;        // [tokens, src_streams, width]
  float* x_new;          // [tokens, streams, width]; null: nothing is written
  const float* y;        // [splits, tokens, width]; null: no write
  const float* mix;      // [streams, streams]
  const float* out_w;    // [streams]
  const float* in_w;     // [streams] or null (ones)
  const float* norm_w;   // [width]
  void* normed;          // [tokens, width]; null: no read
  long long plane;       // tokens * width
  int src_streams, streams, width, splits;
  float eps;
};

__device__ __forceinline__ double block_sum(double v, double* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < warps; ++i) total += scratch[i];     // every thread adds in the same order
  return total;
}

// The streams of one column after the write (or as they are, without one).
template <int S>
__device__ __forceinline__ void column(const StreamsStep& p, const float* mix, const float* out_w, size_t t, int c, float* now) {
  float old[S];
  const float* row = p.x + t * (size_t)p.src_streams * p.width + c;
#pragma unroll
  for (int s = 0; s < S; ++s) old[s] = p.src_streams == 1 ? row[0] : row[(size_t)s * p.width];
  if (p.y == nullptr) {
#pragma unroll
    for (int s = 0; s < S; ++s) now[s] = old[s];
    return;
  }
  // the planes of a split product, added in their order; eight loads are in flight at a time
  float y = 0.f;
  const float* plane = p.y + t * p.width + c;
  int k = 0;
  for (; k + 8 <= p.splits; k += 8) {
    float part[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) part[i] = plane[(size_t)(k + i) * p.plane];
#pragma unroll
    for (int i = 0; i < 8; ++i) y += part[i];
  }
  for (; k < p.splits; ++k) y += plane[(size_t)k * p.plane];
#pragma unroll
  for (int to = 0; to < S; ++to) {
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) v = fmaf(mix[s * S + to], old[s], v);
    now[to] = fmaf(out_w[to], y, v);
  }
}

template <int S, typename TO>
__global__ void __launch_bounds__(MAX_THREADS) streams_step_kernel(const StreamsStep p) {
  dependent_launch_prologue();
  __shared__ double scratch[MAX_THREADS / 32];
  __shared__ float mix[S * S], out_w[S], in_w[S];
  if (threadIdx.x < S * S) mix[threadIdx.x] = p.mix != nullptr ? p.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    out_w[threadIdx.x] = p.out_w != nullptr ? p.out_w[threadIdx.x] : 0.f;
    in_w[threadIdx.x] = p.in_w != nullptr ? p.in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const size_t t = blockIdx.x;
  double squares = 0.0;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    float now[S];
    column<S>(p, mix, out_w, t, c, now);
    if (p.x_new != nullptr) {
#pragma unroll
      for (int s = 0; s < S; ++s) p.x_new[(t * S + s) * p.width + c] = now[s];
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) u = fmaf(in_w[s], now[s], u);
    squares = fma((double)u, (double)u, squares);
  }
  if (p.normed == nullptr) return;
  const float inv = (float)(1.0 / sqrt(block_sum(squares, scratch) / (double)p.width + (double)p.eps));
  TO* to = (TO*)p.normed + t * p.width;
  for (int c = threadIdx.x; c < p.width; c += blockDim.x) {
    float now[S];
    column<S>(p, mix, out_w, t, c, now);       // the same instructions as above: the same bits
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s) u = fmaf(in_w[s], now[s], u);
    to[c] = from_float<TO>(u * inv * p.norm_w[c]);
  }
}

template <int S>
int launch_streams(const StreamsStep& p, int tokens, int out_dtype, cudaStream_t s) {
  // Few tokens leave most SMs idle: their blocks take a thread per column (up to 1,024), so that a
  // token's row is one or two rounds of loads instead of many. The order in which the double sum of
  // squares is added differs between the two block sizes, by less than float32 resolves.
  int threads = THREADS;
  if (tokens <= 256) threads = p.width >= MAX_THREADS ? MAX_THREADS : p.width > THREADS ? (p.width + 31) / 32 * 32 : THREADS;
  if (out_dtype == kF32) launch_kernel(streams_step_kernel<S, float>, tokens, threads, 0, s, p);
  else launch_kernel(streams_step_kernel<S, __nv_bfloat16>, tokens, threads, 0, s, p);
  return check_launch("streams_step");
}

}  // namespace

// One step over the streams of `tokens` tokens. x [tokens, src_streams, width] float32 with
// src_streams 1 or `streams`. A write when y is given (float32 [splits, tokens, width]; mix
// [streams, streams] indexed [from, to], out_w [streams]) into x_new [tokens, streams, width]; a
// read when `normed` is given (in_w [streams] or null for the plain sum, norm_w [width], the
// result in out_dtype: 0 float32, 1 bfloat16), of the written streams when both are given.
PAE_EXPORT int pae_streams_step(float* x_new, void* normed, const float* x, int src_streams, const float* y, int splits,
                                const float* mix, const float* out_w, const float* in_w, const float* norm_w, int tokens,
                                int streams, int width, float eps, int out_dtype, void* stream) {
  if (tokens == 0 || width == 0) return 0;
  if (streams < 1 || streams > MAX_STREAMS) return fail(2, "streams_step: %d streams (1 to %d)", streams, MAX_STREAMS);
  if (src_streams != 1 && src_streams != streams) return fail(2, "streams_step: rows of %d streams for %d", src_streams, streams);
  if (y != nullptr && (x_new == nullptr || mix == nullptr || out_w == nullptr || splits < 1)) return fail(2, "streams_step: a write without its operands");
  if (y == nullptr && x_new != nullptr) return fail(2, "streams_step: streams to write without a sublayer's output");
  if (normed != nullptr && norm_w == nullptr) return fail(2, "streams_step: a read without a norm weight");
  if (normed == nullptr && y == nullptr) return 0;
  if (out_dtype != kF32 && out_dtype != kBF16) return fail(1, "streams_step: unknown dtype %d", out_dtype);
  StreamsStep p{x, x_new, y, mix, out_w, in_w, norm_w, normed, (long long)tokens * width, src_streams, streams, width, splits, eps};
  cudaStream_t s = (cudaStream_t)stream;
  switch (streams) {
    case 1: return launch_streams<1>(p, tokens, out_dtype, s);
    case 2: return launch_streams<2>(p, tokens, out_dtype, s);
    case 3: return launch_streams<3>(p, tokens, out_dtype, s);
    case 4: return launch_streams<4>(p, tokens, out_dtype, s);
    case 5: return launch_streams<5>(p, tokens, out_dtype, s);
    case 6: return launch_streams<6>(p, tokens, out_dtype, s);
    case 7: return launch_streams<7>(p, tokens, out_dtype, s);
    case 8: return launch_streams<8>(p, tokens, out_dtype, s);
    case 9: return launch_streams<9>(p, tokens, out_dtype, s);
    case 10: return launch_streams<10>(p, tokens, out_dtype, s);
    case 11: return launch_streams<11>(p, tokens, out_dtype, s);
    case 12: return launch_streams<12>(p, tokens, out_dtype, s);
    case 13: return launch_streams<13>(p, tokens, out_dtype, s);
    case 14: return launch_streams<14>(p, tokens, out_dtype, s);
    case 15: return launch_streams<15>(p, tokens, out_dtype, s);
    default: return launch_streams<16>(p, tokens, out_dtype, s);
  }
}

PAE_DEFINE_LAST_ERROR()
