// Row-wise kernels of decoders that keep their residual stream in float32: the token
// embedding with a learned position table added, LayerNorm (mean and variance, weight and
// bias), and the activations of a plain two-matrix feed-forward (the exact GELU and its tanh
// form). Statistics, sums and the activation's arithmetic are float32; a result is rounded
// once, to the element type of its output.
#include "common.cuh"

using namespace pae;

namespace {

__device__ __forceinline__ double block_sum(double v, double* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
  __syncthreads();                       // scratch may still be read from the call before
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < warps; ++i) total += scratch[i];     // every thread adds in the same order
  return total;
}

// out[t, :] = token_scale * table[id, :] + position_scale * positions_table[p, :], float32 (no
// position table: the first term alone). A negative id stands for the token that the request
// sampled in the step before (last_token[state_slot[seq_index[t]]]).
template <typename T>
__global__ void embedding_positions_kernel(float* __restrict__ out, const T* __restrict__ table,
                                           const T* __restrict__ position_table, const int* __restrict__ ids,
                                           const int* __restrict__ positions, const int* __restrict__ last_token,
                                           const int* __restrict__ state_slot, const int* __restrict__ seq_index,
                                           int rows, int max_positions, int width, float position_scale,
                                           float token_scale) {
  dependent_launch_prologue();
  const int t = blockIdx.x;
  int src = ids[t];
  if (src < 0 && last_token != nullptr) src = last_token[state_slot[seq_index[t]]];
  const bool ok = src >= 0 && src < rows;
  const T* from = table + (size_t)(ok ? src : 0) * width;
  float* to = out + (size_t)t * width;
  if (position_table == nullptr) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = ok ? token_scale * to_float(from[i]) : 0.f;
    return;
  }
  const int p = positions[t];
  const bool pos_ok = p >= 0 && p < max_positions;
  const T* pos = position_table + (size_t)(pos_ok ? p : 0) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    to[i] = (ok ? token_scale * to_float(from[i]) : 0.f) + (pos_ok ? position_scale * to_float(pos[i]) : 0.f);
}

// y = x / sqrt(mean(x^2) + eps) * w, from float32 or the engine's element type into either; the
// sum of squares is double, the rest float32, one rounding at the end.
template <typename TI, typename TO>
__global__ void rms_norm_cast_kernel(TO* __restrict__ out, const TI* __restrict__ x, const float* __restrict__ weight,
                                     int width, float eps, int ld) {
  dependent_launch_prologue();
  __shared__ double scratch[32];
  const TI* row = x + (size_t)blockIdx.x * ld;       // a row of x may be a column range of a wider row
  double squares = 0.0;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const double v = (double)to_float(row[i]);
    squares = fma(v, v, squares);
  }
  const float inv = (float)(1.0 / sqrt(block_sum(squares, scratch) / (double)width + (double)eps));
  TO* to = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from_float<TO>(to_float(row[i]) * inv * weight[i]);
}

// The middle of a gated feed-forward whose gate and up projections are clamped:
//   g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1)
// for rows that hold the gate in columns [0, I) and the up projection in [I, 2I).
template <typename TI, typename TO>
__global__ void clamped_glu_kernel(TO* __restrict__ out, const TI* __restrict__ gate_up, long long total, int inter,
                                   float limit, float alpha) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / inter;
  const int c = (int)(i - t * inter);
  const float g = fminf(to_float(gate_up[t * 2 * inter + c]), limit);
  const float u = fminf(fmaxf(to_float(gate_up[t * 2 * inter + inter + c]), -limit), limit);
  out[i] = from_float<TO>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
}

// float32 rows whose half-width is a multiple of 4: four columns per thread, 16-byte loads.
template <typename TO>
__global__ void clamped_glu_f32x4_kernel(TO* __restrict__ out, const float* __restrict__ gate_up, long long quads, int inter,
                                         float limit, float alpha) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= quads) return;
  const int per_row = inter >> 2;
  const long long t = i / per_row;
  const int c = (int)(i - t * per_row) * 4;
  const float4 g4 = *(const float4*)(gate_up + t * 2 * inter + c);
  const float4 u4 = *(const float4*)(gate_up + t * 2 * inter + inter + c);
  const float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
  TO* to = out + t * inter + c;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float gate = fminf(g[e], limit), up = fminf(fmaxf(u[e], -limit), limit);
    to[e] = from_float<TO>(gate / (1.f + expf(-alpha * gate)) * (up + 1.f));
  }
}

// x <- cap * tanh(x / cap), float32 in place.
__global__ void softcap_kernel(float* __restrict__ x, long long total, float cap) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  x[i] = cap * tanhf(x[i] / cap);
}

// y = (x - mean) / sqrt(var + eps) * w + b with var the mean of the squared deviations. One block
// per row, three passes over a row that stays in L1; the sums' order depends on the width only.
template <typename TI, typename TO>
__global__ void layer_norm_kernel(TO* __restrict__ out, const TI* __restrict__ x, const float* __restrict__ weight,
                                  const float* __restrict__ bias, int width, float eps) {
  dependent_launch_prologue();
  __shared__ double scratch[32];
  const TI* row = x + (size_t)blockIdx.x * width;
  // The two sums are double: they cost nothing beside the row's traffic, and the mean and the
  // variance then carry no error of their own into every element of the row.
  double sum = 0.0;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sum += (double)to_float(row[i]);
  const float mean = (float)(block_sum(sum, scratch) / (double)width);
  double squares = 0.0;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const double dev = (double)to_float(row[i]) - (double)mean;
    squares = fma(dev, dev, squares);
  }
  const float inv = (float)(1.0 / sqrt(block_sum(squares, scratch) / (double)width + (double)eps));
  TO* to = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = (to_float(row[i]) - mean) * inv * weight[i];
    if (bias != nullptr) v += bias[i];
    to[i] = from_float<TO>(v);
  }
}

__device__ __forceinline__ float gelu_of(float z, int kind) {
  if (kind == 0) return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f));
  if (kind == 2) { z = fmaxf(z, 0.f); return z * z; }
  return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

// kind 0: 0.5 z (1 + erf(z / sqrt 2)); kind 1: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); kind 2: max(z, 0)^2.
template <typename T>
__global__ void gelu_kernel(T* __restrict__ out, const T* __restrict__ x, long long total, int kind) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  out[i] = from_float<T>(gelu_of(to_float(x[i]), kind));
}

// bfloat16, eight elements per thread, 16-byte accesses.
__global__ void gelu_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, long long chunks, int kind) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= chunks) return;
  const uint4 in = *(const uint4*)(x + i * 8);
  const __nv_bfloat162* h = (const __nv_bfloat162*)&in;
  uint4 packed;
  __nv_bfloat162* o = (__nv_bfloat162*)&packed;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    o[e] = __floats2bfloat162_rn(gelu_of(f.x, kind), gelu_of(f.y, kind));
  }
  *(uint4*)(out + i * 8) = packed;
}

// LayerNorm of float32 rows whose width is a multiple of 4: the row is read once, 16 bytes at a
// time, and stays in registers between the sums and the write. Up to 4 * PER * blockDim columns.
template <typename TO, int PER>
__global__ void layer_norm_f32x4_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ weight,
                                        const float* __restrict__ bias, int width, float eps) {
  dependent_launch_prologue();
  __shared__ double scratch[32];
  const int quads = width >> 2;
  const float4* row = (const float4*)(x + (size_t)blockIdx.x * width);
  float4 held[PER];
  double sum = 0.0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    held[j] = c < quads ? row[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) sum += ((double)held[j].x + (double)held[j].y) + ((double)held[j].z + (double)held[j].w);
  const float mean = (float)(block_sum(sum, scratch) / (double)width);
  double squares = 0.0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    if (threadIdx.x + j * blockDim.x < quads) {
      const double a = (double)held[j].x - (double)mean, b = (double)held[j].y - (double)mean;
      const double c = (double)held[j].z - (double)mean, d = (double)held[j].w - (double)mean;
      squares += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float inv = (float)(1.0 / sqrt(block_sum(squares, scratch) / (double)width + (double)eps));
  TO* to = out + (size_t)blockIdx.x * width;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < quads) {
      const float4 w = *(const float4*)(weight + 4 * c);
      const float4 b = bias != nullptr ? *(const float4*)(bias + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float v0 = (held[j].x - mean) * inv * w.x + b.x, v1 = (held[j].y - mean) * inv * w.y + b.y;
      const float v2 = (held[j].z - mean) * inv * w.z + b.z, v3 = (held[j].w - mean) * inv * w.w + b.w;
      to[4 * c] = from_float<TO>(v0);
      to[4 * c + 1] = from_float<TO>(v1);
      to[4 * c + 2] = from_float<TO>(v2);
      to[4 * c + 3] = from_float<TO>(v3);
    }
  }
}

int row_threads(int width) { return width >= 2048 ? 512 : (width >= 1024 ? 256 : (width >= 256 ? 128 : 64)); }

}  // namespace

PAE_EXPORT int pae_embedding_positions(float* out, const void* table, const void* position_table, const int* ids,
                                       const int* positions, const int* last_token, const int* state_slot,
                                       const int* seq_index, int n, int rows, int max_positions, int width,
                                       float position_scale, float token_scale, int dtype, void* stream) {
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_threads(width);
  if (dtype == kF32)
    launch_kernel(embedding_positions_kernel<float>, n, threads, 0, s, out, (const float*)table, (const float*)position_table,
                  ids, positions, last_token, state_slot, seq_index, rows, max_positions, width, position_scale, token_scale);
  else if (dtype == kBF16)
    launch_kernel(embedding_positions_kernel<__nv_bfloat16>, n, threads, 0, s, out, (const __nv_bfloat16*)table,
                  (const __nv_bfloat16*)position_table, ids, positions, last_token, state_slot, seq_index, rows,
                  max_positions, width, position_scale, token_scale);
  else
    return fail(1, "embedding_positions: unknown dtype %d", dtype);
  return check_launch("embedding_positions");
}

// x float32 or bfloat16 [rows, width] -> out float32 or bfloat16; weight, bias (may be null) float32.
PAE_EXPORT int pae_layer_norm(void* out, const void* x, const float* weight, const float* bias, int rows, int width,
                              float eps, int in_dtype, int out_dtype, void* stream) {
  if (rows == 0 || width == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_threads(width);
  using bf = __nv_bfloat16;
  const int key = in_dtype * 10 + out_dtype;
  if (in_dtype == kF32 && width % 4 == 0 && width <= 4 * 4 * 256 &&
      (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)bias) & 15) == 0 && (out_dtype == kF32 || out_dtype == kBF16)) {
    const int quads = width / 4;
    const int block = quads <= 64 ? 64 : (quads <= 128 ? 128 : 256);
    const int per = (quads + block - 1) / block;
    if (out_dtype == kF32) {
      if (per <= 1) launch_kernel(layer_norm_f32x4_kernel<float, 1>, rows, block, 0, s, (float*)out, (const float*)x, weight, bias, width, eps);
      else if (per <= 2) launch_kernel(layer_norm_f32x4_kernel<float, 2>, rows, block, 0, s, (float*)out, (const float*)x, weight, bias, width, eps);
      else launch_kernel(layer_norm_f32x4_kernel<float, 4>, rows, block, 0, s, (float*)out, (const float*)x, weight, bias, width, eps);
    } else {
      if (per <= 1) launch_kernel(layer_norm_f32x4_kernel<bf, 1>, rows, block, 0, s, (bf*)out, (const float*)x, weight, bias, width, eps);
      else if (per <= 2) launch_kernel(layer_norm_f32x4_kernel<bf, 2>, rows, block, 0, s, (bf*)out, (const float*)x, weight, bias, width, eps);
      else launch_kernel(layer_norm_f32x4_kernel<bf, 4>, rows, block, 0, s, (bf*)out, (const float*)x, weight, bias, width, eps);
    }
    return check_launch("layer_norm");
  }
  if (key == 0)
    launch_kernel(layer_norm_kernel<float, float>, rows, threads, 0, s, (float*)out, (const float*)x, weight, bias, width, eps);
  else if (key == 1)
    launch_kernel(layer_norm_kernel<float, bf>, rows, threads, 0, s, (bf*)out, (const float*)x, weight, bias, width, eps);
  else if (key == 10)
    launch_kernel(layer_norm_kernel<bf, float>, rows, threads, 0, s, (float*)out, (const bf*)x, weight, bias, width, eps);
  else if (key == 11)
    launch_kernel(layer_norm_kernel<bf, bf>, rows, threads, 0, s, (bf*)out, (const bf*)x, weight, bias, width, eps);
  else
    return fail(1, "layer_norm: element types in=%d out=%d are not supported", in_dtype, out_dtype);
  return check_launch("layer_norm");
}

// x float32 or bfloat16 [rows, width] -> out float32 or bfloat16; weight float32.
PAE_EXPORT int pae_rms_norm_cast(void* out, const void* x, const float* weight, int rows, int width, float eps,
                                 int in_dtype, int out_dtype, void* stream) {
  if (rows == 0 || width == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_threads(width);
  using bf = __nv_bfloat16;
  const int key = in_dtype * 10 + out_dtype;
  if (key == 0)
    launch_kernel(rms_norm_cast_kernel<float, float>, rows, threads, 0, s, (float*)out, (const float*)x, weight, width, eps, width);
  else if (key == 1)
    launch_kernel(rms_norm_cast_kernel<float, bf>, rows, threads, 0, s, (bf*)out, (const float*)x, weight, width, eps, width);
  else if (key == 10)
    launch_kernel(rms_norm_cast_kernel<bf, float>, rows, threads, 0, s, (float*)out, (const bf*)x, weight, width, eps, width);
  else if (key == 11)
    launch_kernel(rms_norm_cast_kernel<bf, bf>, rows, threads, 0, s, (bf*)out, (const bf*)x, weight, width, eps, width);
  else
    return fail(1, "rms_norm_cast: element types in=%d out=%d are not supported", in_dtype, out_dtype);
  return check_launch("rms_norm_cast");
}

// The same norm over columns [offset, offset + width) of float32 rows of pitch ld -> out [rows, width].
PAE_EXPORT int pae_rms_norm_columns(void* out, const float* x, int ld, int offset, const float* weight, int rows, int width,
                                    float eps, int out_dtype, void* stream) {
  if (rows == 0 || width == 0) return 0;
  if (offset < 0 || offset + width > ld) return fail(2, "rms_norm_columns: columns %d..%d of rows of %d", offset, offset + width, ld);
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = row_threads(width);
  if (out_dtype == kF32)
    launch_kernel(rms_norm_cast_kernel<float, float>, rows, threads, 0, s, (float*)out, x + offset, weight, width, eps, ld);
  else if (out_dtype == kBF16)
    launch_kernel(rms_norm_cast_kernel<float, __nv_bfloat16>, rows, threads, 0, s, (__nv_bfloat16*)out, x + offset, weight, width, eps, ld);
  else
    return fail(1, "rms_norm_columns: unknown dtype %d", out_dtype);
  return check_launch("rms_norm_columns");
}

// gate_up [tokens, 2 * inter] in in_dtype -> out [tokens, inter] in out_dtype.
PAE_EXPORT int pae_clamped_glu(void* out, const void* gate_up, int tokens, int inter, float limit, float alpha,
                               int in_dtype, int out_dtype, void* stream) {
  const long long total = (long long)tokens * inter;
  if (total == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  const int key = in_dtype * 10 + out_dtype;
  if (in_dtype == kF32 && inter % 4 == 0 && ((uintptr_t)gate_up & 15) == 0 && (out_dtype == kF32 || out_dtype == kBF16)) {
    const long long quads = total / 4;
    const unsigned quad_blocks = (unsigned)((quads + 255) / 256);
    if (out_dtype == kF32)
      launch_kernel(clamped_glu_f32x4_kernel<float>, quad_blocks, 256, 0, s, (float*)out, (const float*)gate_up, quads, inter, limit, alpha);
    else
      launch_kernel(clamped_glu_f32x4_kernel<bf>, quad_blocks, 256, 0, s, (bf*)out, (const float*)gate_up, quads, inter, limit, alpha);
    return check_launch("clamped_glu");
  }
  if (key == 0)
    launch_kernel(clamped_glu_kernel<float, float>, blocks, 256, 0, s, (float*)out, (const float*)gate_up, total, inter, limit, alpha);
  else if (key == 1)
    launch_kernel(clamped_glu_kernel<float, bf>, blocks, 256, 0, s, (bf*)out, (const float*)gate_up, total, inter, limit, alpha);
  else if (key == 11)
    launch_kernel(clamped_glu_kernel<bf, bf>, blocks, 256, 0, s, (bf*)out, (const bf*)gate_up, total, inter, limit, alpha);
  else
    return fail(1, "clamped_glu: element types in=%d out=%d are not supported", in_dtype, out_dtype);
  return check_launch("clamped_glu");
}

PAE_EXPORT int pae_softcap(float* x, long long total, float cap, void* stream) {
  if (total == 0) return 0;
  if (!(cap > 0.f)) return fail(2, "softcap: the cap %g is not positive", (double)cap);
  launch_kernel(softcap_kernel, (unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream, x, total, cap);
  return check_launch("softcap");
}

PAE_EXPORT int pae_gelu(void* out, const void* x, long long total, int kind, int dtype, void* stream) {
  if (total == 0) return 0;
  if (kind < 0 || kind > 2) return fail(2, "gelu: kind %d (0: erf, 1: tanh, 2: squared ReLU)", kind);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kBF16 && total % 8 == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
    const long long chunks = total / 8;
    launch_kernel(gelu_bf16x8_kernel, (unsigned)((chunks + 255) / 256), 256, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, chunks, kind);
    return check_launch("gelu");
  }
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == kF32)
    launch_kernel(gelu_kernel<float>, blocks, 256, 0, s, (float*)out, (const float*)x, total, kind);
  else if (dtype == kBF16)
    launch_kernel(gelu_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, total, kind);
  else
    return fail(1, "gelu: unknown dtype %d", dtype);
  return check_launch("gelu");
}

PAE_DEFINE_LAST_ERROR()
