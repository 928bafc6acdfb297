// Causal attention (with an optional sliding window) of many query heads over ONE key/value head whose value is the leading DV
// channels of its key row (latent attention with the expansions folded into the queries and the
// output: a key row is [latent | shared rotated part], D channels, and the latent is also the
// value), for bfloat16 on tensor cores (mma.sync m16n8k16, float32 accumulation). D may be large
// (a latent of 512 and 64 rotated channels), so neither the queries nor the output fit one warp's
// registers the way they do for head sizes up to 128:
//
//   * a block owns 32 query rows (32 consecutive tokens of one head, or, for a request that
//     brings ONE token, 32 of its heads: every key is then read once for all of them) as two
//     groups of four warps with 16 rows each, and walks the request's pages 64 keys at a time;
//     the key tile is staged once for both groups by cp.async, two stages, rows padded by 16
//     bytes so that the eight rows of an ldmatrix fall into different banks (a key tile of 576
//     channels is 73 KB: one block an SM, so the second group is also what hides the first's latencies);
//   * scores: warp w of a group computes the 16 x 16 block of the tile's keys 16w .. 16w+15 over all of D,
//     its A fragments read from the query tile in shared memory, and leaves it as MMA fragments in
//     shared memory; after a barrier every warp reads all four blocks and runs the same running
//     softmax (the same instructions on the same numbers: the warps agree bit for bit);
//   * values: warp w owns the output columns [w * cols, (w + 1) * cols) and multiplies the
//     probabilities (rounded to bfloat16) with those columns of the same key tile.
//
// A single token's keys are shared out over `splits` blocks that leave unnormalised partial
// results in scratch; `merge` adds them up in their order. Scores and the softmax are float32.
// Keys are folded in ascending order; a query's result depends on its own keys only. With a
// window w a query at position i sees the keys i - w < j <= i: a block starts at the tile of its
// first row's first key, and keys before that key are not fetched (their pages may be gone).
#include "attention_mma.cuh"

using namespace pae;
using namespace pae_attention;

namespace {

constexpr int GROUP_ROWS = 16;
constexpr int GROUPS = 2;
constexpr int ROWS = GROUP_ROWS * GROUPS;
constexpr int THREADS = GROUPS * 128;
constexpr int TILE = 64;
constexpr int MAX_COLS = 128;            // value columns per warp

struct LatentParams {
  __nv_bfloat16* out;           // [tokens, heads, DV]
  const __nv_bfloat16* q;       // [tokens, heads, D]
  const __nv_bfloat16* keys;    // [pages, 1, page_size, D]
  const int* block_table;
  const int* q_start;
  const int* q_pos0;
  const int* kv_len;
  int table_width, heads, page_size, D, DV, cols;
  float scale;
  int splits;
  int window;                   // 0: every earlier key
  float* part_out;              // [requests, heads, splits, DV]
  float* part_max;              // [requests, heads, splits]  (in units of log 2)
  float* part_sum;
};

__global__ void __launch_bounds__(THREADS) latent_kernel(const LatentParams p) {
  dependent_launch_prologue();
  extern __shared__ __align__(128) uint8_t smem[];
  const int group = threadIdx.x >> 7, warp = (threadIdx.x >> 5) & 3, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int first_token = p.q_start[b];
  const int q_count = p.q_start[b + 1] - first_token;
  const bool single = p.part_out != nullptr && q_count == 1;
  const int tile = single ? 0 : blockIdx.x, split = single ? blockIdx.x : 0;
  const int head0 = single ? blockIdx.y * ROWS : blockIdx.y;          // single: 32 of the token's heads
  if (single ? (split >= p.splits || head0 >= p.heads) : tile * ROWS >= q_count) return;
  const int rows = single ? min(ROWS, p.heads - head0) : min(ROWS, q_count - tile * ROWS);
  const int pos0 = p.q_pos0[b] + tile * ROWS;
  const int kv_end = single ? min(p.kv_len[b], pos0 + 1) : min(p.kv_len[b], pos0 + rows);
  const int kv_begin = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;      // the first key that the block's first row sees
  const int D = p.D, DV = p.DV;
  const int chunks = D >> 3;                                           // 16-byte chunks of a row
  const int row_bytes = D * 2 + 16;
  uint8_t* q_tile = smem;                                              // [ROWS][row_bytes]
  uint8_t* k_stage = q_tile + ROWS * row_bytes;                        // 2 x [TILE][row_bytes]
  float* sbuf = (float*)(k_stage + 2 * TILE * row_bytes) + group * 4 * 32 * 8;      // per group [4][32][8]
  const uint32_t q_u32 = smem_u32(q_tile), k_u32 = smem_u32(k_stage);
  const int* table = p.block_table + (size_t)b * p.table_width;

  for (int i = threadIdx.x; i < ROWS * chunks; i += THREADS) {
    const int r = i / chunks, c = i - r * chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      const size_t token = single ? first_token : first_token + tile * ROWS + r;
      const int head = single ? head0 + r : head0;
      v = *(const uint4*)(p.q + (token * p.heads + head) * D + c * 8);
    }
    *(uint4*)(q_tile + r * row_bytes + c * 16) = v;
  }

  // four threads per key row, each every fourth chunk; one page lookup per thread and tile
  const int f_row = threadIdx.x >> 2, f_chunk0 = threadIdx.x & 3;
  auto fetch = [&](int stage, int key0) {
    const int key = key0 + f_row;
    uint8_t* dst = k_stage + (size_t)stage * TILE * row_bytes + f_row * row_bytes;
    if (key < kv_end && key >= kv_begin) {
      const int index = key / p.page_size;
      const int page = checked_page(table[checked_table_index(index, p.table_width)]);
      const __nv_bfloat16* src = p.keys + ((size_t)page * p.page_size + (key - index * p.page_size)) * D;
      const uint32_t dst_u32 = smem_u32(dst);
      for (int c = f_chunk0; c < chunks; c += 4) cp_async16(dst_u32 + c * 16, src + c * 8);
    } else {
      for (int c = f_chunk0; c < chunks; c += 4) *(uint4*)(dst + c * 16) = make_uint4(0, 0, 0, 0);
    }
  };

  float o[MAX_COLS / 8][4];
#pragma unroll
  for (int n = 0; n < MAX_COLS / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float row_max[2] = {-FLT_MAX, -FLT_MAX}, row_sum[2] = {0.f, 0.f};
  const int row0 = group * GROUP_ROWS;                                 // this group's first row of the block
  const bool working = row0 < rows;                                    // a group without rows only helps to fetch
  const int my_pos[2] = {single ? pos0 : pos0 + row0 + (lane >> 2), single ? pos0 : pos0 + row0 + (lane >> 2) + 8};
  const int last_pos = single ? pos0 : pos0 + min(rows, row0 + GROUP_ROWS) - 1;
  const int c2 = (lane & 3) * 2;
  const int mid = lane >> 3, r8 = lane & 7;
  const float scale2 = p.scale * LOG2E;
  const int col0 = warp * p.cols;                                      // this warp's first value column

  const int tiles = (kv_end + TILE - 1) / TILE, tile0 = kv_begin / TILE;
  int t_begin = tile0, t_end = tiles;
  if (single) {
    const int each = (tiles - tile0 + p.splits - 1) / p.splits;
    t_begin = min(tiles, tile0 + split * each);
    t_end = min(tiles, t_begin + each);
  }
  if (t_begin < t_end) fetch(t_begin & 1, t_begin * TILE);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    if (t + 1 < t_end) fetch((t + 1) & 1, (t + 1) * TILE);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t k_tile = k_u32 + (t & 1) * TILE * row_bytes;
    if (working) {                       // scores of the keys 16 * warp .. + 15 of this tile
      // even and odd steps of D into accumulators of their own: two chains of dependent MMAs instead of one
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t a_at = q_u32 + (row0 + ((lane >> 3) & 1) * 8 + r8) * row_bytes + (lane >> 4) * 16;
      const uint32_t b_at = k_tile + (warp * 16 + (mid >> 1) * 8 + r8) * row_bytes + (mid & 1) * 16;
      const int steps = D >> 4;
#pragma unroll 2
      for (int k = 0; k + 1 < steps; k += 2) {
        uint32_t a[4], bb[4], a2[4], bb2[4];
        ldmatrix_x4(a, a_at + k * 32);
        ldmatrix_x4(bb, b_at + k * 32);
        ldmatrix_x4(a2, a_at + k * 32 + 32);
        ldmatrix_x4(bb2, b_at + k * 32 + 32);
        mma_16816(s[0], a, bb[0], bb[1]);
        mma_16816(s[1], a, bb[2], bb[3]);
        mma_16816(s2[0], a2, bb2[0], bb2[1]);
        mma_16816(s2[1], a2, bb2[2], bb2[3]);
      }
      if (steps & 1) {
        uint32_t a[4], bb[4];
        ldmatrix_x4(a, a_at + (steps - 1) * 32);
        ldmatrix_x4(bb, b_at + (steps - 1) * 32);
        mma_16816(s[0], a, bb[0], bb[1]);
        mma_16816(s[1], a, bb[2], bb[3]);
      }
      float4* to = (float4*)(sbuf + ((size_t)warp * 32 + lane) * 8);
      to[0] = make_float4(s[0][0] + s2[0][0], s[0][1] + s2[0][1], s[0][2] + s2[0][2], s[0][3] + s2[0][3]);
      to[1] = make_float4(s[1][0] + s2[1][0], s[1][1] + s2[1][1], s[1][2] + s2[1][2], s[1][3] + s2[1][3]);
    }
    __syncthreads();
#pragma unroll 1
    for (int u = 0; working && u < TILE / 16; ++u) {
      const int key0 = t * TILE + u * 16;
      if (key0 > last_pos || key0 >= kv_end) break;
      float s[2][4];
      {
        const float4* from = (const float4*)(sbuf + ((size_t)u * 32 + lane) * 8);
        const float4 lo = from[0], hi = from[1];
        s[0][0] = lo.x, s[0][1] = lo.y, s[0][2] = lo.z, s[0][3] = lo.w;
        s[1][0] = hi.x, s[1][1] = hi.y, s[1][2] = hi.z, s[1][3] = hi.w;
      }
      float block_max[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int half = j >> 1, key = key0 + i * 8 + c2 + (j & 1);
          const bool seen = key < kv_end && key <= my_pos[half] && (p.window <= 0 || key + p.window > my_pos[half]);
          s[i][j] = seen ? s[i][j] * scale2 : -FLT_MAX;
          block_max[half] = fmaxf(block_max[half], s[i][j]);
        }
      float rescale[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        block_max[half] = fmaxf(block_max[half], __shfl_xor_sync(0xffffffffu, block_max[half], 1));
        block_max[half] = fmaxf(block_max[half], __shfl_xor_sync(0xffffffffu, block_max[half], 2));
        const float new_max = fmaxf(row_max[half], block_max[half]);
        rescale[half] = row_max[half] == -FLT_MAX ? 0.f : fast_exp2(row_max[half] - new_max);
        row_max[half] = new_max;
      }
      float block_sum[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int half = j >> 1;
          const float e = s[i][j] == -FLT_MAX ? 0.f : fast_exp2(s[i][j] - row_max[half]);
          s[i][j] = e;
          block_sum[half] += e;
        }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        block_sum[half] += __shfl_xor_sync(0xffffffffu, block_sum[half], 1);
        block_sum[half] += __shfl_xor_sync(0xffffffffu, block_sum[half], 2);
        row_sum[half] = row_sum[half] * rescale[half] + block_sum[half];
      }
      if (__any_sync(0xffffffffu, rescale[0] != 1.f || rescale[1] != 1.f)) {
#pragma unroll
        for (int n = 0; n < MAX_COLS / 8; ++n) {
          o[n][0] *= rescale[0];
          o[n][1] *= rescale[0];
          o[n][2] *= rescale[1];
          o[n][3] *= rescale[1];
        }
      }
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
      const uint32_t v_at = k_tile + (u * 16 + (mid & 1) * 8 + r8) * row_bytes + ((col0 >> 3) + (mid >> 1)) * 16;
#pragma unroll
      for (int n = 0; n < MAX_COLS / 16; ++n) {
        if (n * 16 < p.cols && col0 + n * 16 < DV) {
          uint32_t bb[4];
          ldmatrix_x4_trans(bb, v_at + n * 32);
          mma_16816(o[2 * n], pa, bb[0], bb[1]);
          mma_16816(o[2 * n + 1], pa, bb[2], bb[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = row0 + (lane >> 2) + half * 8;
    if (row >= rows) continue;
    if (single) {
      const size_t at = ((size_t)b * p.heads + head0 + row) * p.splits + split;
#pragma unroll
      for (int n = 0; n < MAX_COLS / 8; ++n) {
        const int col = col0 + n * 8 + c2;
        if (n * 8 < p.cols && col < DV) {
          p.part_out[at * DV + col] = o[n][half * 2];
          p.part_out[at * DV + col + 1] = o[n][half * 2 + 1];
        }
      }
      if (warp == 0 && (lane & 3) == 0) {
        p.part_max[at] = row_max[half];
        p.part_sum[at] = row_sum[half];
      }
    } else {
      const float inv = row_sum[half] > 0.f ? 1.f / row_sum[half] : 0.f;
      __nv_bfloat16* out = p.out + ((size_t)(first_token + tile * ROWS + row) * p.heads + head0) * DV;
#pragma unroll
      for (int n = 0; n < MAX_COLS / 8; ++n) {
        const int col = col0 + n * 8 + c2;
        if (n * 8 < p.cols && col < DV) *(uint32_t*)(out + col) = pack_bf16(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
      }
    }
  }
}

// out[token of a single-token request, head, :] from the partial results of its blocks, in their order.
__global__ void latent_merge_kernel(const LatentParams p) {
  dependent_launch_prologue();
  extern __shared__ float weights[];          // [splits]
  __shared__ float inverse;
  const int h = blockIdx.x, b = blockIdx.y;
  const int first_token = p.q_start[b];
  if (p.q_start[b + 1] - first_token != 1) return;
  const size_t at = ((size_t)b * p.heads + h) * p.splits;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    float top = -FLT_MAX;
    for (int s = lane; s < p.splits; s += 32) top = fmaxf(top, p.part_max[at + s]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    for (int s = lane; s < p.splits; s += 32) {
      const float m = p.part_max[at + s];
      weights[s] = m == -FLT_MAX ? 0.f : fast_exp2(m - top);
    }
    __syncwarp();
    if (lane == 0) {
      float sum = 0.f;
      for (int s = 0; s < p.splits; ++s) sum += p.part_sum[at + s] * weights[s];
      inverse = sum > 0.f ? 1.f / sum : 0.f;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < p.DV; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.splits; ++s) acc += p.part_out[(at + s) * p.DV + c] * weights[s];
    p.out[((size_t)first_token * p.heads + h) * p.DV + c] = __float2bfloat16_rn(acc * inverse);
  }
}

size_t smem_bytes(int d) { return (size_t)(ROWS + 2 * TILE) * (d * 2 + 16) + GROUPS * 4 * 32 * 8 * sizeof(float); }

}  // namespace

// 1 when the kernel takes key rows of d channels whose first dv are the value.
PAE_EXPORT int pae_attention_latent_mma_supports(int d, int dv) {
  return d >= 16 && d % 16 == 0 && dv >= 16 && dv % 16 == 0 && dv <= d && dv <= 4 * MAX_COLS && smem_bytes(d) <= 200 * 1024 ? 1 : 0;
}

// bfloat16. out [tokens, heads, dv]; q [tokens, heads, d]; keys [pages, 1, page_size, d]. With `scratch`
// (seqs * heads * splits * (dv + 2) floats) a request that brings ONE token is taken by blocks of up to 32
// heads each, its keys shared out over `splits` blocks and merged by a second kernel. window: 0, or how many keys
// (itself included) a query sees.
PAE_EXPORT int pae_paged_attention_latent_mma(void* out, const void* q, const void* keys, const int* block_table,
                                              int table_width, const int* q_start, const int* q_pos0, const int* kv_len,
                                              int seqs, int max_q_len, int heads, int d, int dv, int page_size, float scale,
                                              int window, int splits, float* scratch, void* stream) {
  if (seqs == 0 || max_q_len == 0) return 0;
  if (!pae_attention_latent_mma_supports(d, dv)) return fail(2, "paged_attention_latent_mma: key rows of %d channels with values of %d", d, dv);
  if (splits < 1 || (scratch == nullptr && splits != 1)) return fail(2, "paged_attention_latent_mma: %d splits", splits);
  if (heads < 1 || heads > 65535 || seqs > 65535) return fail(3, "paged_attention_latent_mma: %d heads x %d requests exceed one launch", heads, seqs);
  if (page_size < 1) return fail(2, "paged_attention_latent_mma: page size %d", page_size);
  if (((uintptr_t)q | (uintptr_t)keys | (uintptr_t)out) & 15)
    return fail(2, "paged_attention_latent_mma: an operand does not start on a 16-byte boundary");
  const int cols = (((dv + 3) / 4) + 15) / 16 * 16;
  LatentParams p{(__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)keys, block_table, q_start, q_pos0, kv_len,
                 table_width, heads, page_size, d, dv, cols, scale, splits, window < 0 ? 0 : window, nullptr, nullptr, nullptr};
  if (scratch != nullptr) {
    const size_t units = (size_t)seqs * heads * splits;
    p.part_out = scratch;
    p.part_max = scratch + units * dv;
    p.part_sum = p.part_max + units;
  }
  const size_t bytes = smem_bytes(d);
  if (int err = allow_smem(latent_kernel, 200 * 1024, "paged_attention_latent_mma")) return err;
  cudaStream_t s = (cudaStream_t)stream;
  const int q_tiles = (max_q_len + ROWS - 1) / ROWS;
  dim3 grid(scratch != nullptr ? max(q_tiles, splits) : q_tiles, heads, seqs);
  launch_kernel(latent_kernel, grid, THREADS, bytes, s, p);
  if (int err = check_launch("paged_attention_latent_mma")) return err;
  if (scratch != nullptr) {
    const int threads = dv >= 512 ? 512 : (dv + 31) / 32 * 32;       // a column a thread
    launch_kernel(latent_merge_kernel, dim3(heads, seqs), threads, (size_t)splits * sizeof(float), s, p);
    return check_launch("paged_attention_latent_merge");
  }
  return 0;
}

PAE_DEFINE_LAST_ERROR()
