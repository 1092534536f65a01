// The sigmoid attention of attention_sigmoid.cu with its two large products on the tensor cores
// (mma.sync m16n8k16, bfloat16 operands, float32 sums): for every row i, query head g and cached key
// j <= i,
//   w_g(i, j) = sigmoid(q_g(i) . k_c(g)(j) * scale - r1_g ln(1 + r2_g (i - j)) + pb_g)
//   w'_h(i, j) = sum_g talk[h, g] w_g(i, j)          (talk null: w' = w)
//   out_h(i) = sum_j w'_h(i, j) v_c(h)(j)
// One CTA of eight warps takes the 16 rows of one work-list entry with ALL heads (the mixing needs every
// head's weight of a (row, key) pair in one place) and walks the keys in tiles of 32 aligned to absolute
// positions, possibly one of several CTAs that share a row's keys in chunks (their sums are added up, in
// chunk order, by a second kernel).  Per key tile: each warp forms the scores of its heads (Q K^T), turns
// them into weights in float32 and leaves them in shared memory; all threads mix the weights across
// heads in float32 and round the result to bfloat16; each warp multiplies its heads' mixed weights with
// the values (W' V) into accumulators that stay in its registers over all key tiles.  The key tile of the
// next step is fetched (cp.async) while the weights are mixed and multiplied, the value tile while the
// next scores are formed.
// Sizes: key size and value size 64 or 128, at most 16 heads (two per warp).
#include "mma_attention.cuh"

namespace mlr {

constexpr int SM_THREADS = 256;
constexpr int SM_WARPS = SM_THREADS / 32;
constexpr int SM_KEYS = 32;
constexpr int SM_ROWS = 16;
constexpr int SM_HEADS_PER_WARP = 2;
constexpr int SM_WSTRIDE = 40;      // entries between the rows of a weight matrix in shared memory (32 keys + padding)

struct SigmoidMmaArgs {
  const int *tile_seg, *tile_row0, *seg_q_start, *seg_q_len, *seg_pos0, *block_table, *seg_slot;
  const float *r1, *r2, *pb, *talk;
  int table_width, heads, kv_heads, page_size, chunk_keys, total_rows;
  float scale;
};

// grid: (work-list entries, key chunks)
// Heads of 64 and 64 leave room for two blocks per SM (128 registers a thread: 64 of them output sums),
// so that one block's barriers and dependent instructions pass under the other's work.
template <int D, int V>
__global__ void __launch_bounds__(SM_THREADS, (D <= 64 && V <= 64) ? 2 : 1)
attention_sigmoid_mma_kernel(const bf16* q, const bf16* k_pool, const bf16* v_pool, bf16* out, float* partial,
                             SigmoidMmaArgs a) {
  pdl_trigger();
  extern __shared__ __align__(128) unsigned char shared_bytes[];
  const int H = a.heads, G = a.kv_heads, per_kv = H / G;
  bf16* q_tiles = reinterpret_cast<bf16*>(shared_bytes);                  // [H][16][D], swizzled per head
  bf16* k_tiles = q_tiles + (size_t)H * SM_ROWS * D;                       // [G][32][D], swizzled per head
  bf16* v_tiles = k_tiles + (size_t)G * SM_KEYS * D;                       // [G][32][V]
  bf16* w_mix = v_tiles + (size_t)G * SM_KEYS * V;                         // [H][16][SM_WSTRIDE]
  float* w_raw = reinterpret_cast<float*>(w_mix + (size_t)H * SM_ROWS * SM_WSTRIDE);      // [H][16][SM_WSTRIDE]
  float* talk = w_raw + (size_t)H * SM_ROWS * SM_WSTRIDE;                  // [H][H]
  int* key_row = reinterpret_cast<int*>(talk + H * H);                     // [2][32]: the cached row of every key of this and the next tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (a.talk != nullptr)
    for (int i = threadIdx.x; i < H * H; i += SM_THREADS) talk[i] = a.talk[i];
  pdl_wait();
  const int seg = a.tile_seg[blockIdx.x];
  const int row0 = a.tile_row0[blockIdx.x];
  const int q_start = a.seg_q_start[seg], q_len = a.seg_q_len[seg], pos0 = a.seg_pos0[seg];
  const int rows = min(SM_ROWS, q_len - row0);
  const int* table = a.block_table + (size_t)(a.seg_slot != nullptr ? a.seg_slot[seg] : seg) * a.table_width;
  const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;
  const int chunk_first = blockIdx.y * a.chunk_keys;
  const int chunk_last = min(last_pos, chunk_first + a.chunk_keys - 1);

  // the rows' queries, every head a swizzled tile of its own; rows past the entry's end are zeros
  for (int item = threadIdx.x; item < H * SM_ROWS * (D / 8); item += SM_THREADS) {
    const int chunk = item % (D / 8), r = (item / (D / 8)) % SM_ROWS, h = item / ((D / 8) * SM_ROWS);
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) value = __ldcg(reinterpret_cast<const uint4*>(q + ((size_t)(q_start + row0 + r) * H + h) * D) + chunk);
    *reinterpret_cast<uint4*>(tile_at<D>(q_tiles + (size_t)h * SM_ROWS * D, r, chunk)) = value;
  }

  // the cached row (without the head) of every key of the tile at k0: page * G * page_size + place in the page;
  // -1 for keys past the rows' last position and pages the request does not hold
  auto find_rows = [&](int k0, int parity) {
    if (warp == 0) {
      const int key = k0 + lane;
      int row = -1;
      if (key <= last_pos) {
        const int page = table[key / a.page_size];
        if (page >= 0) row = page * G * a.page_size + key % a.page_size;
      }
      key_row[parity * SM_KEYS + lane] = row;
    }
  };
  // all key (or value) heads' rows of a tile whose keys' rows are known; missing keys become zeros
  auto fetch = [&](bool values, int parity) {
    const int W = values ? V : D;
    const bf16* pool = values ? v_pool : k_pool;
    bf16* tiles = values ? v_tiles : k_tiles;
    const int chunks = W / 8;
    for (int item = threadIdx.x; item < G * SM_KEYS * chunks; item += SM_THREADS) {
      const int chunk = item % chunks, r = (item / chunks) % SM_KEYS, c = item / (chunks * SM_KEYS);
      const int row = key_row[parity * SM_KEYS + r];
      const bool valid = row >= 0;
      const bf16* src = valid ? pool + ((size_t)row + (size_t)c * a.page_size) * W + chunk * 8 : pool;
      bf16* dst = values ? tile_at<V>(tiles + (size_t)c * SM_KEYS * V, r, chunk) : tile_at<D>(tiles + (size_t)c * SM_KEYS * D, r, chunk);
      cp_async_16(dst, src, valid);
    }
    cp_async_commit();
  };

  float o[SM_HEADS_PER_WARP][V / 8][4];
#pragma unroll
  for (int hi = 0; hi < SM_HEADS_PER_WARP; ++hi)
#pragma unroll
    for (int t = 0; t < V / 8; ++t) o[hi][t][0] = o[hi][t][1] = o[hi][t][2] = o[hi][t][3] = 0.f;

  if (chunk_first <= chunk_last) {
    find_rows(chunk_first, 0);
    __syncthreads();
    fetch(false, 0);
    fetch(true, 0);
  }
  int parity = 0;
  for (int k0 = chunk_first; k0 <= chunk_last; k0 += SM_KEYS, parity ^= 1) {
    const bool more = k0 + SM_KEYS <= chunk_last;
    if (more) find_rows(k0 + SM_KEYS, parity ^ 1);      // seen after the barriers below, before the next tile is asked for
    cp_async_wait<1>();      // this tile's keys (its values may still be on their way)
    __syncthreads();
    // ---- every head's own weights: warp w takes heads w, w + 8
#pragma unroll
    for (int hi = 0; hi < SM_HEADS_PER_WARP; ++hi) {
      const int h = warp + SM_WARPS * hi;
      if (h < H) {
        uint32_t q_frag[D / 16][4];
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
          ldmatrix_x4(q_frag[ks], tile_at<D>(q_tiles + (size_t)h * SM_ROWS * D, r, ks * 2 + (lane >> 4)));
        }
        float s[SM_KEYS / 8][4];
        warp_qk<D, SM_KEYS / 8, false, SM_KEYS>(s, q_frag, k_tiles + (size_t)(h / per_kv) * SM_KEYS * D, 0, lane);
        const float r1 = a.r1 != nullptr ? a.r1[h] : 0.f, r2 = a.r1 != nullptr ? a.r2[h] : 0.f;
        const float pb = a.pb != nullptr ? a.pb[h] : 0.f;
        float* w = w_raw + (size_t)h * SM_ROWS * SM_WSTRIDE;
#pragma unroll
        for (int j = 0; j < SM_KEYS / 8; ++j) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int row = (lane >> 2) + 8 * i;
            float pair[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int key = j * 8 + (lane & 3) * 2 + e;
              const int distance = first_pos + row - (k0 + key);
              float weight = 0.f;
              if (distance >= 0 && row < rows) {
                // the hardware's approximate logarithm, exponential and division (errors of a few units in
                // the last place of a float32, far inside the bfloat16 rounding of the weight that follows)
                float z = fmaf(s[j][2 * i + e], a.scale, pb);
                if (a.r1 != nullptr) z -= r1 * __logf(fmaf(r2, (float)distance, 1.f));
                weight = __fdividef(1.f, 1.f + __expf(fminf(-z, 80.f)));
              }
              pair[e] = weight;
            }
            *reinterpret_cast<float2*>(w + row * SM_WSTRIDE + j * 8 + (lane & 3) * 2) = make_float2(pair[0], pair[1]);
          }
        }
      }
    }
    __syncthreads();
    if (more) fetch(false, parity ^ 1); else cp_async_commit();
    // ---- the weights mixed across the heads, rounded to bfloat16 for the second product
    for (int idx = threadIdx.x; idx < H * SM_ROWS * (SM_KEYS / 2); idx += SM_THREADS) {
      const int j = (idx % (SM_KEYS / 2)) * 2, r = (idx / (SM_KEYS / 2)) % SM_ROWS, h = idx / ((SM_KEYS / 2) * SM_ROWS);
      float lo, hi;
      if (a.talk != nullptr) {
        lo = hi = 0.f;
        for (int g = 0; g < H; ++g) {
          const float2 w = *reinterpret_cast<const float2*>(w_raw + ((size_t)g * SM_ROWS + r) * SM_WSTRIDE + j);
          const float t = talk[h * H + g];
          lo = fmaf(t, w.x, lo);
          hi = fmaf(t, w.y, hi);
        }
      } else {
        const float2 w = *reinterpret_cast<const float2*>(w_raw + ((size_t)h * SM_ROWS + r) * SM_WSTRIDE + j);
        lo = w.x;
        hi = w.y;
      }
      *reinterpret_cast<uint32_t*>(w_mix + ((size_t)h * SM_ROWS + r) * SM_WSTRIDE + j) = pack_bf16(lo, hi);
    }
    cp_async_wait<1>();      // this tile's values (the next keys may still be on their way)
    __syncthreads();
    // ---- the values: out_h += W'_h V_c(h)
#pragma unroll
    for (int hi = 0; hi < SM_HEADS_PER_WARP; ++hi) {
      const int h = warp + SM_WARPS * hi;
      if (h < H) {
        const bf16* w = w_mix + (size_t)h * SM_ROWS * SM_WSTRIDE;
        bf16* v_tile = v_tiles + (size_t)(h / per_kv) * SM_KEYS * V;
#pragma unroll
        for (int kk = 0; kk < SM_KEYS / 16; ++kk) {
          uint32_t af[4];
          const int row = lane >> 2, col = kk * 16 + (lane & 3) * 2;
          af[0] = *reinterpret_cast<const uint32_t*>(w + row * SM_WSTRIDE + col);
          af[1] = *reinterpret_cast<const uint32_t*>(w + (row + 8) * SM_WSTRIDE + col);
          af[2] = *reinterpret_cast<const uint32_t*>(w + row * SM_WSTRIDE + col + 8);
          af[3] = *reinterpret_cast<const uint32_t*>(w + (row + 8) * SM_WSTRIDE + col + 8);
#pragma unroll
          for (int dp = 0; dp < V / 16; ++dp) {
            uint32_t b[4];
            const int key = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            ldmatrix_x4_trans(b, tile_at<V>(v_tile, key, dp * 2 + (lane >> 4)));
            mma_bf16(o[hi][2 * dp], af, b[0], b[1]);
            mma_bf16(o[hi][2 * dp + 1], af, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();
    if (more) fetch(true, parity ^ 1); else cp_async_commit();
  }
  cp_async_wait<0>();

  const bool split = gridDim.y > 1;
#pragma unroll
  for (int hi = 0; hi < SM_HEADS_PER_WARP; ++hi) {
    const int h = warp + SM_WARPS * hi;
    if (h >= H) continue;
#pragma unroll
    for (int t = 0; t < V / 8; ++t) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int row = (lane >> 2) + 8 * i;
        if (row >= rows) continue;
        const size_t at = ((size_t)(q_start + row0 + row) * H + h) * V + t * 8 + (lane & 3) * 2;
        if (split)
          *reinterpret_cast<float2*>(partial + (size_t)blockIdx.y * a.total_rows * H * V + at) = make_float2(o[hi][t][2 * i], o[hi][t][2 * i + 1]);
        else
          *reinterpret_cast<uint32_t*>(out + at) = pack_bf16(o[hi][t][2 * i], o[hi][t][2 * i + 1]);
      }
    }
  }
}

__global__ void __launch_bounds__(256)
add_chunks_bf16_kernel(const float* partial, bf16* __restrict__ out, long long count, int chunks) {
  pdl_trigger();
  pdl_wait();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= count) return;
  float sum = 0.f;
  for (int c = 0; c < chunks; ++c) sum += __ldcg(partial + (size_t)c * count + index);
  out[index] = __float2bfloat16_rn(sum);
}

static size_t sigmoid_mma_shared(int heads, int kv_heads, int dim, int vdim) {
  return sizeof(bf16) * ((size_t)heads * SM_ROWS * dim + (size_t)kv_heads * SM_KEYS * (dim + vdim) +
                         (size_t)heads * SM_ROWS * SM_WSTRIDE) +
         sizeof(float) * ((size_t)heads * SM_ROWS * SM_WSTRIDE + (size_t)heads * heads) + sizeof(int) * 2 * SM_KEYS;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// 1 if the tensor-core kernel takes these sizes, else 0.
MLR_EXPORT int mlr_attention_sigmoid_mma_fits(int heads, int kv_heads, int dim, int vdim) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || heads > SM_WARPS * SM_HEADS_PER_WARP) return 0;
  if ((dim != 64 && dim != 128) || (vdim != 64 && vdim != 128)) return 0;
  return sigmoid_mma_shared(heads, kv_heads, dim, vdim) <= 220 * 1024 ? 1 : 0;
}

// q: bfloat16 [rows, heads, dim]; out: bfloat16 [rows, heads, vdim]; pools bfloat16 [pages, kv_heads, page_size,
// dim | vdim]; r1, r2, pb: float32 [heads] or null (r1 and r2 together); talk: float32 [heads, heads] or null.
// tile_seg/tile_row0: entries of up to 16 rows of one segment.  chunks > 1: `partial` (float32 [chunks,
// total_rows, heads * vdim]) receives the chunks' sums, which a second kernel adds up in chunk order.
MLR_EXPORT int mlr_attention_sigmoid_mma(const void* q, const void* k_pool, const void* v_pool, void* out, float* partial,
                                         const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                         const int* seg_q_len, const int* seg_pos0, const int* block_table,
                                         const int* seg_slot, int table_width, int tiles, int total_rows, int heads,
                                         int kv_heads, int dim, int vdim, int page_size, float scale, const float* r1,
                                         const float* r2, const float* pb, const float* talk, int chunks, int chunk_keys,
                                         cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || total_rows <= 0 || page_size <= 0 || table_width <= 0 || chunks <= 0 || chunk_keys <= 0 ||
      chunk_keys % SM_KEYS != 0 || (chunks > 1 && partial == nullptr) || ((r1 == nullptr) != (r2 == nullptr)))
    return MLR_BAD_SIZE;
  if (!mlr_attention_sigmoid_mma_fits(heads, kv_heads, dim, vdim) || chunks > 65535) return MLR_TOO_LARGE;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!aligned(q) || !aligned(k_pool) || !aligned(v_pool) || !aligned(out) || !aligned(partial)) return MLR_BAD_ALIGNMENT;
  SigmoidMmaArgs a{tile_seg, tile_row0, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot, r1, r2, pb, talk,
                   table_width, heads, kv_heads, page_size, chunk_keys, total_rows, scale};
  const size_t shared = sigmoid_mma_shared(heads, kv_heads, dim, vdim);
  auto launch = [&](auto kernel) -> int {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (err != cudaSuccess) return (int)err;
    launch_kernel(kernel, dim3(tiles, chunks), dim3(SM_THREADS), shared, stream, (const bf16*)q, (const bf16*)k_pool,
                  (const bf16*)v_pool, (bf16*)out, partial, a);
    int status = launch_status();
    if (status != MLR_OK || chunks == 1) return status;
    const long long count = (long long)total_rows * heads * vdim;
    launch_kernel(add_chunks_bf16_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream,
                  (const float*)partial, (bf16*)out, count, chunks);
    return launch_status();
  };
  if (dim == 64 && vdim == 64) return launch(attention_sigmoid_mma_kernel<64, 64>);
  if (dim == 64 && vdim == 128) return launch(attention_sigmoid_mma_kernel<64, 128>);
  if (dim == 128 && vdim == 64) return launch(attention_sigmoid_mma_kernel<128, 64>);
  return launch(attention_sigmoid_mma_kernel<128, 128>);
}
