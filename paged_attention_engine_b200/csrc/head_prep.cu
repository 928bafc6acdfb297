// What stands between a fused projection and attention, for mixers that norm and rotate their
// heads: per query and key head an optional RMS norm over the head's first channels with a
// weight shared by all heads (or one RMS norm over all query heads of the token at once, and one
// over all key heads, with a weight as long as the projection), a rotation of a span of the head
// by the step's table of cosines and sines, in either pairing, and the write of keys (and values)
// into their pages.
//
//   norm      y[i] = x[i] / sqrt(mean(x[0..span)^2) + eps) * w[i]      for i < span; the rest passes
//   or        y[h, i] = x[h, i] / sqrt(mean over all heads and channels of x^2 + eps) * w[h, i]   ("whole")
//   rotation  of channels [rot0, rot0 + dims): pair (i, i + dims/2) ("half") or (2i, 2i + 1)
//             ("interleaved"), i < dims/2:  (u, v) -> (u c_i - v s_i, v c_i + u s_i)
//   write     q -> q_out[token, head, :]; k -> keys[page, kv head, offset, :]; v likewise
//
// Query heads and key heads may differ in size, span and where their rotated channels start, so
// one launch serves grouped-query attention (all heads alike) and latent attention (query heads
// of unrotated + rotated channels; ONE key row per token that holds the normed latent and the
// shared rotated part; no values). The projection is float32 or the engine's element type; all
// arithmetic is float32 (the sum of squares double) and every result is rounded once.
//
// Also here: the table of cosines and sines with an amplitude, and the element-wise product of
// an attention's output with the sigmoid of a gate projection.
#include "common.cuh"

using namespace pae;

namespace {

struct HeadPrep {
  const void* proj;      // [tokens, ld]
  void* q_out;           // [tokens, heads, qd]
  void* keys;            // [pages, kv_heads, page_size, kd]
  void* values;          // [pages, kv_heads, page_size, dv]
  const float* q_norm;   // [q_span] or null
  const float* k_norm;   // [k_span] or null
  const float* table;    // [tokens, dims]: cosines, then sines; null: no rotation
  const int* slots;      // [tokens]: page * page_size + offset, negative: nothing is written; null: no pages
  int ld, q_off, k_off, v_off;
  int heads, kv_heads, qd, kd, dv;
  int q_span, k_span, q_rot0, k_rot0, dims, interleaved, page_size;
  float eps;
  int whole;             // the norm's mean runs over all query (key) heads of the token; weights [heads, span]
  int whole_kv_heads;    // the key heads that the mean runs over (kv_heads is 0 in a step that writes no page)
};

constexpr int WARPS = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(WARPS * 32) head_prep_kernel(const HeadPrep p) {
  dependent_launch_prologue();
  extern __shared__ float rows[];              // [WARPS][widest head]
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int widest = max(max(p.qd, p.kd), p.dv);
  float* buf = rows + warp * widest;
  const TI* in = (const TI*)p.proj + (size_t)t * p.ld;
  const bool with_values = p.values != nullptr && p.dv > 0;
  const int units = p.heads + p.kv_heads * (with_values ? 2 : 1);
  int slot = -1;
  if (p.slots != nullptr) {
    slot = p.slots[t];
    if (slot >= 0 && !slot_in_pool(slot, p.page_size)) slot = -1;
  }
  const int page = slot >= 0 ? slot / p.page_size : 0, offset = slot >= 0 ? slot - page * p.page_size : 0;
  const int half = p.dims >> 1;
  // "whole": the token's two sums of squares, by the whole block in an order that depends on
  // nothing but the sizes (so a token's result is the same in any batch)
  __shared__ double whole_sum[2][WARPS];
  float whole_inv[2] = {0.f, 0.f};
  if (p.whole) {
    for (int which = 0; which < 2; ++which) {
      const TI* src = in + (which == 0 ? p.q_off : p.k_off);
      // keys are normed whether or not the token has a page: the count is the model's, not the step's
      const int n = which == 0 ? (p.q_norm != nullptr ? p.heads * p.qd : 0) : (p.k_norm != nullptr ? p.whole_kv_heads * p.kd : 0);
      double squares = 0.0;
      for (int i = threadIdx.x; i < n; i += WARPS * 32) {
        const float v = to_float(src[i]);
        squares = fma((double)v, (double)v, squares);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, o);
      if (lane == 0) whole_sum[which][warp] = squares;
    }
    __syncthreads();
    for (int which = 0; which < 2; ++which) {
      const int n = which == 0 ? p.heads * p.qd : p.whole_kv_heads * p.kd;
      double squares = 0.0;
      for (int w = 0; w < WARPS; ++w) squares += whole_sum[which][w];
      whole_inv[which] = n > 0 ? (float)(1.0 / sqrt(squares / (double)n + (double)p.eps)) : 0.f;
    }
  }
  for (int unit = blockIdx.y * WARPS + warp; unit < units; unit += WARPS * gridDim.y) {
    const bool is_q = unit < p.heads, is_k = !is_q && unit < p.heads + p.kv_heads;
    const int index = is_q ? unit : (is_k ? unit - p.heads : unit - p.heads - p.kv_heads);
    const int d = is_q ? p.qd : (is_k ? p.kd : p.dv);
    if (!is_q && slot < 0) continue;           // a key or value without a page is not wanted
    const TI* src = in + (is_q ? p.q_off : (is_k ? p.k_off : p.v_off)) + (size_t)index * d;
    const float* weight = is_q ? p.q_norm : (is_k ? p.k_norm : nullptr);
    const int span = is_q ? p.q_span : (is_k ? p.k_span : 0);
    if (p.whole && weight != nullptr) weight += (size_t)index * span;
    double squares = 0.0;
    for (int i = lane; i < d; i += 32) {
      const float v = to_float(src[i]);
      buf[i] = v;
      if (weight != nullptr && i < span) squares = fma((double)v, (double)v, squares);
    }
    if (p.whole && weight != nullptr) {
      const float inv = whole_inv[is_q ? 0 : 1];
      __syncwarp();
      for (int i = lane; i < span; i += 32) buf[i] = buf[i] * inv * weight[i];
    } else if (weight != nullptr && span > 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, o);
      const float inv = (float)(1.0 / sqrt(squares / (double)span + (double)p.eps));
      __syncwarp();
      for (int i = lane; i < span; i += 32) buf[i] = buf[i] * inv * weight[i];
    }
    __syncwarp();
    if (p.table != nullptr && (is_q || is_k) && half > 0) {
      const int rot0 = is_q ? p.q_rot0 : p.k_rot0;
      const float* cs = p.table + (size_t)t * p.dims;
      for (int i = lane; i < half; i += 32) {
        const int a = rot0 + (p.interleaved ? 2 * i : i), b = rot0 + (p.interleaved ? 2 * i + 1 : i + half);
        float lo = buf[a], hi = buf[b];
        rotate_pair(lo, hi, cs[i], cs[half + i]);
        buf[a] = lo;
        buf[b] = hi;
      }
      __syncwarp();
    }
    TO* to;
    if (is_q)
      to = (TO*)p.q_out + ((size_t)t * p.heads + index) * d;
    else
      to = (TO*)(is_k ? p.keys : p.values) + (((size_t)page * p.kv_heads + index) * p.page_size + offset) * d;
    for (int i = lane; i < d; i += 32) to[i] = from_float<TO>(buf[i]);
    __syncwarp();
  }
}

// table[t, i] = amplitude * cos(position[t] * inv_freq[i]), table[t, half + i] = amplitude * sin(same);
// the angle is one float32 product.
__global__ void rotary_table_amplitude_kernel(float* __restrict__ table, const int* __restrict__ positions,
                                              const float* __restrict__ inv_freq, int tokens, int half, float amplitude) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)tokens * half) return;
  const int t = (int)(i / half), f = (int)(i - (long long)t * half);
  const float angle = __fmul_rn((float)positions[t], inv_freq[f]);
  float s, c;
  sincosf(angle, &s, &c);
  table[(size_t)t * 2 * half + f] = c * amplitude;
  table[(size_t)t * 2 * half + half + f] = s * amplitude;
}

// out[t, c] = x[t, c] * sigmoid(gate[t, gate_off + c / group]); the gate is a column range of a
// projection, one column for every `group` neighbouring channels (a head's size: a gate per head).
template <typename TX, typename TG>
__global__ void sigmoid_gate_kernel(TX* __restrict__ out, const TX* __restrict__ x, const TG* __restrict__ gate,
                                    long long total, int width, int gate_ld, int gate_off, int group) {
  dependent_launch_prologue();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int c = (int)(i - t * width);
  const float g = to_float(gate[t * gate_ld + gate_off + c / group]);
  out[i] = from_float<TX>(to_float(x[i]) / (1.f + expf(-g)));
}

}  // namespace

// whole: the norms' means run over all heads at once (weights [heads * span]). in_dtype: the projection's element type; out_dtype: that of q_out and of the pages (0 float32, 1 bfloat16).
PAE_EXPORT int pae_head_prep(void* q_out, void* keys, void* values, const void* proj, int ld, int q_off, int k_off,
                             int v_off, int tokens, int heads, int kv_heads, int qd, int kd, int dv,
                             const float* q_norm, int q_span, const float* k_norm, int k_span, float eps,
                             const float* table, int dims, int interleaved, int q_rot0, int k_rot0, const int* slots,
                             int page_size, int whole, int in_dtype, int out_dtype, void* stream) {
  if (tokens == 0 || heads + kv_heads == 0) return 0;
  if (heads < 0 || kv_heads < 0 || qd < 0 || kd < 0 || dv < 0) return fail(2, "head_prep: a negative size");
  if (dims % 2) return fail(2, "head_prep: %d rotated channels are not pairs", dims);
  if (table != nullptr && ((heads > 0 && q_rot0 + dims > qd) || (kv_heads > 0 && k_rot0 + dims > kd)))
    return fail(2, "head_prep: %d rotated channels from %d and %d do not fit heads of %d and %d", dims, q_rot0, k_rot0, qd, kd);
  if (q_span > qd || k_span > kd) return fail(2, "head_prep: a norm over %d or %d channels of heads of %d and %d", q_span, k_span, qd, kd);
  if (kv_heads > 0 && slots != nullptr && (keys == nullptr || page_size < 1)) return fail(2, "head_prep: slots without pages");
  if (heads > 0 && q_out == nullptr) return fail(2, "head_prep: query heads without an output");
  if (whole && ((q_norm != nullptr && q_span != qd) || (k_norm != nullptr && k_span != kd)))
    return fail(2, "head_prep: a norm over the whole projection covers every channel (%d of %d, %d of %d)", q_span, qd, k_span, kd);
  HeadPrep p{proj, q_out, keys, values, q_norm, k_norm, table, slots, ld, q_off, k_off, v_off, heads,
             slots != nullptr ? kv_heads : 0, qd, kd, dv, q_span, k_span, q_rot0, k_rot0, table != nullptr ? dims : 0,
             interleaved, page_size < 1 ? 1 : page_size, eps, whole, kv_heads};
  const int widest = qd > kd ? (qd > dv ? qd : dv) : (kd > dv ? kd : dv);
  const size_t smem = sizeof(float) * WARPS * (size_t)widest;
  if (smem > 48 * 1024) return fail(2, "head_prep: heads of %d channels are too wide", widest);
  cudaStream_t s = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  const int key = in_dtype * 10 + out_dtype;
  // few tokens: a warp per head, so that a decode step's handful of tokens still fills some SMs
  const int units = heads + p.kv_heads * (values != nullptr && dv > 0 ? 2 : 1);
  const dim3 grid(tokens, tokens < 64 ? (units + WARPS - 1) / WARPS : 1);
  if (key == 0) launch_kernel(head_prep_kernel<float, float>, grid, WARPS * 32, smem, s, p);
  else if (key == 1) launch_kernel(head_prep_kernel<float, bf>, grid, WARPS * 32, smem, s, p);
  else if (key == 11) launch_kernel(head_prep_kernel<bf, bf>, grid, WARPS * 32, smem, s, p);
  else return fail(1, "head_prep: element types in=%d out=%d are not supported", in_dtype, out_dtype);
  return check_launch("head_prep");
}

PAE_EXPORT int pae_rotary_table_amplitude(float* table, const int* positions, const float* inv_freq, int tokens, int half,
                                          float amplitude, void* stream) {
  const long long n = (long long)tokens * half;
  if (n == 0) return 0;
  launch_kernel(rotary_table_amplitude_kernel, (unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream, table, positions,
                inv_freq, tokens, half, amplitude);
  return check_launch("rotary_table_amplitude");
}

// x, out [tokens, width] in x_dtype; gate [tokens, gate_ld] in gate_dtype, columns gate_off .. gate_off + width / group.
PAE_EXPORT int pae_sigmoid_gate(void* out, const void* x, const void* gate, int tokens, int width, int gate_ld,
                                int gate_off, int group, int x_dtype, int gate_dtype, void* stream) {
  const long long total = (long long)tokens * width;
  if (total == 0) return 0;
  if (group < 1 || width % group) return fail(2, "sigmoid_gate: rows of %d channels in groups of %d", width, group);
  if (gate_off < 0 || gate_off + width / group > gate_ld) return fail(2, "sigmoid_gate: columns %d..%d of rows of %d", gate_off, gate_off + width / group, gate_ld);
  cudaStream_t s = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  const int key = x_dtype * 10 + gate_dtype;
  if (key == 0) launch_kernel(sigmoid_gate_kernel<float, float>, blocks, 256, 0, s, (float*)out, (const float*)x, (const float*)gate, total, width, gate_ld, gate_off, group);
  else if (key == 10) launch_kernel(sigmoid_gate_kernel<bf, float>, blocks, 256, 0, s, (bf*)out, (const bf*)x, (const float*)gate, total, width, gate_ld, gate_off, group);
  else if (key == 11) launch_kernel(sigmoid_gate_kernel<bf, bf>, blocks, 256, 0, s, (bf*)out, (const bf*)x, (const bf*)gate, total, width, gate_ld, gate_off, group);
  else return fail(1, "sigmoid_gate: element types x=%d gate=%d are not supported", x_dtype, gate_dtype);
  return check_launch("sigmoid_gate");
}

PAE_DEFINE_LAST_ERROR()
