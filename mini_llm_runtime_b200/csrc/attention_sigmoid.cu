// Attention whose weights are not normalised over the keys: sigmoid instead of softmax, an optional
// bias that grows with the logarithm of the distance, and an optional mixing of the weights across
// heads before they meet the values.  Plus the kernel that prepares q, k and v of a plain-headed
// attention (per-head RMS norm with or without a weight, optional blend of the values with another
// layer's values, cache write).
//
// mlr_head_norm_kv_write   per row of the float32 projection [q heads | k heads | v heads]: every q and k
//                          head divided by its root mean square over `dim` (eps inside the root) and
//                          multiplied by a weight [dim] if one is given; v <- (1 - mix) v + mix * other
//                          if a blend is asked for; q out in the cache's dtype, k and v into their pages.
// mlr_attention_sigmoid    for every row i of the step, query head g and cached key j <= i of the row's
//                          request:
//                            w_g(i, j) = sigmoid(q_g(i) . k_c(g)(j) * scale - r1_g ln(1 + r2_g (i - j)) + pb_g)
//                            w'_h(i, j) = sum_g talk[h, g] w_g(i, j)           (talk null: w' = w)
//                            out_h(i) = sum_j w'_h(i, j) v_c(h)(j)
//                          with c(h) = h / (heads / kv_heads).  Scores, weights and sums in float32.
//                          One CTA takes a few rows of one request with ALL heads (the mixing needs every
//                          head's weight of a (row, key) pair in one place), walks the keys in tiles of 32
//                          aligned to absolute positions, and may be one of several that share a row's
//                          keys in chunks; since nothing is normalised, the chunks' results simply add up,
//                          in chunk order, in a second kernel.
#include "common.cuh"

#include <type_traits>

namespace mlr {

template <typename T>
__global__ void __launch_bounds__(128)
head_norm_kv_write_kernel(const float* qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                          const float* other_values, long long other_stride, const float* __restrict__ mix,
                          const long long* slots, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
                          int rows, int heads, int kv_heads, int dim, int vdim, int page_size, float eps, int write_kv) {
  pdl_trigger();
  pdl_wait();
  const int units = heads + 2 * kv_heads;
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= (long long)rows * units) return;
  const int row = (int)(item / units), unit = (int)(item - (long long)row * units);
  const int in_width = (heads + kv_heads) * dim + kv_heads * vdim;
  const float* in = qkv + (size_t)row * in_width;
  if (unit < heads + kv_heads) {
    const bool is_q = unit < heads;
    if (!is_q && !write_kv) return;
    const float* x = in + (size_t)unit * dim;       // q heads then k heads lie one after the other
    float sq = 0.f;
    for (int d = lane; d < dim; d += 32) {
      const float v = __ldcg(x + d);
      sq = fmaf(v, v, sq);
    }
    sq = warp_sum(sq);
    const float factor = 1.f / sqrtf(sq / (float)dim + eps);
    const float* w = is_q ? q_weight : k_weight;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)row * heads + unit) * dim;
    } else {
      const long long slot = slots[row];
      const long long page = slot / page_size, offset = slot - page * page_size;
      dst = k_pool + (((size_t)page * kv_heads + (unit - heads)) * page_size + offset) * dim;
    }
    for (int d = lane; d < dim; d += 32) {
      float v = __ldcg(x + d) * factor;
      if (w != nullptr) v *= w[d];
      dst[d] = from_float<T>(v);
    }
  } else {
    if (!write_kv) return;
    const int g = unit - heads - kv_heads;
    const float* x = in + (size_t)(heads + kv_heads) * dim + (size_t)g * vdim;
    const long long slot = slots[row];
    const long long page = slot / page_size, offset = slot - page * page_size;
    T* dst = v_pool + (((size_t)page * kv_heads + g) * page_size + offset) * vdim;
    if (other_values != nullptr) {
      const float m = mix[0];
      const float* o = other_values + (size_t)row * other_stride + (size_t)g * vdim;
      for (int d = lane; d < vdim; d += 32) dst[d] = from_float<T>(fmaf(m, __ldcg(o + d), (1.f - m) * __ldcg(x + d)));
    } else {
      for (int d = lane; d < vdim; d += 32) dst[d] = from_float<T>(__ldcg(x + d));
    }
  }
}

constexpr int KEYS = 32;          // keys per tile, one per lane
constexpr int THREADS = 256;
constexpr int PLAN_ROWS = 16;     // rows of one entry of the work list
constexpr int MAX_ACC = 32;       // output sums a thread may hold
constexpr int MAX_STAGE = 4;      // 16-byte pieces of the next tile a thread keeps in flight

struct SigmoidArgs {
  const int *tile_seg, *tile_row0, *seg_q_start, *seg_q_len, *seg_pos0, *block_table, *seg_slot;
  const float *r1, *r2, *pb, *talk;
  int table_width, heads, kv_heads, dim, vdim, page_size, rows_per_cta, chunk_keys, total_rows, tile_stride;
  float scale;
};

template <typename T> struct Piece;      // 16 bytes of a cached row as floats
template <> struct Piece<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(uint4 raw, float* dst) {
    dst[0] = __uint_as_float(raw.x); dst[1] = __uint_as_float(raw.y);
    dst[2] = __uint_as_float(raw.z); dst[3] = __uint_as_float(raw.w);
  }
};
template <> struct Piece<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 raw, float* dst) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dst[2 * i] = __uint_as_float(words[i] << 16);
      dst[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
  }
};

// grid: (work-list entries, PLAN_ROWS / rows_per_cta, key chunks).  `partial` (float32 [chunks][rows]
// [heads * vdim]) receives the sums when there are several chunks, else `out` does.
//
// A key tile passes through 2 * kv_heads phases: the keys of every key/value head (the heads' own
// weights), the mixing, then the values of every key/value head.  Each phase's tile of 32 cached rows
// goes through one shared buffer.  VECTOR (head sizes in whole 16-byte pieces): a thread asks for its
// pieces of the NEXT phase's tile before it computes on this one, so the trip to memory runs under the
// arithmetic; otherwise the tile is fetched entry by entry where it is needed.
template <typename T, bool VECTOR>
__global__ void __launch_bounds__(THREADS)
attention_sigmoid_kernel(const T* q, const T* k_pool, const T* v_pool, T* out, float* partial, SigmoidArgs a) {
  pdl_trigger();
  extern __shared__ __align__(16) float shared[];
  const int H = a.heads, G = a.kv_heads, D = a.dim, V = a.vdim, R = a.rows_per_cta, ST = a.tile_stride;
  const int per_kv = H / G;
  float* q_rows = shared;                          // [H][R][D]
  float* w_raw = q_rows + (size_t)H * R * D;       // [H][R][KEYS]: the heads' own weights
  float* w_mix = w_raw + (size_t)H * R * KEYS;     // [H][R][KEYS]: mixed over the heads
  float* tile = w_mix + (size_t)H * R * KEYS;      // [KEYS][ST]: this phase's keys or values
  float* talk = tile + KEYS * ST;                  // [H][H]
  int* key_row = reinterpret_cast<int*>(talk + H * H);      // [2][KEYS]: the cached row of every key of this and the next tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  if (a.talk != nullptr)
    for (int i = threadIdx.x; i < H * H; i += THREADS) talk[i] = a.talk[i];
  pdl_wait();
  const int seg = a.tile_seg[blockIdx.x];
  const int row0 = a.tile_row0[blockIdx.x] + blockIdx.y * R;
  const int q_start = a.seg_q_start[seg], q_len = a.seg_q_len[seg], pos0 = a.seg_pos0[seg];
  const int rows = min(R, min(PLAN_ROWS - (int)blockIdx.y * R, q_len - row0));
  if (rows <= 0) return;
  const int* table = a.block_table + (size_t)(a.seg_slot != nullptr ? a.seg_slot[seg] : seg) * a.table_width;
  const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;

  for (int idx = threadIdx.x; idx < H * R * D; idx += THREADS) {
    const int d = idx % D, r = (idx / D) % R, h = idx / (D * R);
    q_rows[idx] = r < rows ? to_float(q[((size_t)(q_start + row0 + r) * H + h) * D + d]) : 0.f;
  }

  const int outputs = H * R * V;
  float acc[MAX_ACC];
#pragma unroll
  for (int i = 0; i < MAX_ACC; ++i) acc[i] = 0.f;

  const int chunk_first = blockIdx.z * a.chunk_keys;
  const int chunk_last = min(last_pos, chunk_first + a.chunk_keys - 1);
  const int phases = 2 * G;

  // the cached row (without the head) of every key of the tile at k0: page * G * page_size + place in the page
  auto find_rows = [&](int k0, int parity) {
    if (warp == 0) {
      const int key = k0 + lane;
      int row = -1;
      if (key <= last_pos) {
        const int page = table[key / a.page_size];
        if (page >= 0) row = page * G * a.page_size + key % a.page_size;
      }
      key_row[parity * KEYS + lane] = row;
    }
  };
  // VECTOR: this thread's pieces of the tile of `phase` (keys of head phase, or values of head phase - G)
  uint4 stage[MAX_STAGE];
  auto ask = [&](int phase, int parity) {
    const bool values = phase >= G;
    const int c = values ? phase - G : phase, W = values ? V : D;
    const T* pool = values ? v_pool : k_pool;
    const int per_row = W / Piece<T>::N;
#pragma unroll
    for (int l = 0; l < MAX_STAGE; ++l) {
      const int e = threadIdx.x + THREADS * l;
      stage[l] = make_uint4(0u, 0u, 0u, 0u);
      if (e < KEYS * per_row) {
        const int j = e / per_row, piece = e - j * per_row;
        const int row = key_row[parity * KEYS + j];
        if (row >= 0)
          stage[l] = __ldcg(reinterpret_cast<const uint4*>(pool + ((size_t)row + (size_t)c * a.page_size) * W) + piece);
      }
    }
  };
  auto put = [&](int phase) {
    const int W = phase >= G ? V : D;
    const int per_row = W / Piece<T>::N;
#pragma unroll
    for (int l = 0; l < MAX_STAGE; ++l) {
      const int e = threadIdx.x + THREADS * l;
      if (e < KEYS * per_row) {
        const int j = e / per_row, piece = e - j * per_row;
        float values[Piece<T>::N];
        Piece<T>::unpack(stage[l], values);
        float* dst = tile + j * ST + piece * Piece<T>::N;
#pragma unroll
        for (int u = 0; u < Piece<T>::N; u += 4)
          *reinterpret_cast<float4*>(dst + u) = make_float4(values[u], values[u + 1], values[u + 2], values[u + 3]);
      }
    }
  };
  auto fetch = [&](int phase, int parity) {      // the same, entry by entry
    const bool values = phase >= G;
    const int c = values ? phase - G : phase, W = values ? V : D;
    const T* pool = values ? v_pool : k_pool;
    for (int idx = threadIdx.x; idx < KEYS * W; idx += THREADS) {
      const int j = idx / W, d = idx - j * W;
      const int row = key_row[parity * KEYS + j];
      tile[j * ST + d] = row >= 0 ? to_float(pool[((size_t)row + (size_t)c * a.page_size) * W + d]) : 0.f;
    }
  };

  if (chunk_first <= chunk_last) {
    find_rows(chunk_first, 0);
    __syncthreads();
    if (VECTOR) ask(0, 0);
  }
  int parity = 0;
  for (int k0 = chunk_first; k0 <= chunk_last; k0 += KEYS, parity ^= 1) {
    const bool more = k0 + KEYS <= chunk_last;
    if (more) find_rows(k0 + KEYS, parity ^ 1);      // seen after the barriers below, long before it is used
    for (int phase = 0; phase < phases; ++phase) {
      __syncthreads();      // the phase before is done with the tile, and (phase G) all weights are written
      if (phase == G && a.talk != nullptr) {
        // ---- the weights mixed across the heads
        for (int idx = threadIdx.x; idx < H * rows * KEYS; idx += THREADS) {
          const int j = idx % KEYS, r = (idx / KEYS) % rows, h = idx / (KEYS * rows);
          float sum = 0.f;
          for (int g = 0; g < H; ++g) sum = fmaf(talk[h * H + g], w_raw[((size_t)g * R + r) * KEYS + j], sum);
          w_mix[((size_t)h * R + r) * KEYS + j] = sum;
        }
      }
      if (VECTOR) {
        put(phase);
        if (phase + 1 < phases) ask(phase + 1, parity);
        else if (more) ask(0, parity ^ 1);
      } else {
        fetch(phase, parity);
      }
      __syncthreads();
      if (phase < G) {
        // ---- the own weights of the heads that read key head `phase`: (head, row) pairs, up to four per
        // warp and turn (one key entry then feeds four sums), fewer when there are too few pairs for all warps
        const int c = phase;
        const float* kr = tile + lane * ST;
        const int key = k0 + lane;
        const int pairs = per_kv * rows;
        const int per_turn = pairs >= 4 * (THREADS / 32) ? 4 : pairs >= 2 * (THREADS / 32) ? 2 : 1;
        for (int p = warp * per_turn; p < pairs; p += (THREADS / 32) * per_turn) {
          const float* qp[4];
          int hh[4], rr[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int pu = min(p + u, pairs - 1);
            hh[u] = c * per_kv + pu / rows;
            rr[u] = pu % rows;
            qp[u] = q_rows + ((size_t)hh[u] * R + rr[u]) * D;
          }
          float s[4] = {0.f, 0.f, 0.f, 0.f};
          if (VECTOR) {
            for (int d = 0; d < D; d += 4) {
              const float4 kd = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                if (u < per_turn) {
                  const float4 qd = *reinterpret_cast<const float4*>(qp[u] + d);
                  s[u] = fmaf(qd.x, kd.x, s[u]);
                  s[u] = fmaf(qd.y, kd.y, s[u]);
                  s[u] = fmaf(qd.z, kd.z, s[u]);
                  s[u] = fmaf(qd.w, kd.w, s[u]);
                }
              }
            }
          } else {
            for (int d = 0; d < D; ++d) {
              const float kd = kr[d];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (u < per_turn) s[u] = fmaf(qp[u][d], kd, s[u]);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (u >= per_turn || p + u >= pairs) break;
            const int distance = first_pos + rr[u] - key;
            float weight = 0.f;
            if (distance >= 0) {
              float z = s[u] * a.scale;
              if (a.r1 != nullptr) z -= a.r1[hh[u]] * log1pf(a.r2[hh[u]] * (float)distance);
              if (a.pb != nullptr) z += a.pb[hh[u]];
              weight = 1.f / (1.f + expf(-z));
            }
            w_raw[((size_t)hh[u] * R + rr[u]) * KEYS + lane] = weight;
          }
        }
      } else {
        // ---- the values of key/value head c; output o = (h * R + r) * V + d belongs to thread o % THREADS
        const int c = phase - G;
        const float* w_use = a.talk != nullptr ? w_mix : w_raw;
        const int o_first = c * per_kv * R * V, o_end = (c + 1) * per_kv * R * V;
        if (THREADS % V == 0) {
          // all of a thread's outputs share one value channel: its column of the tile stays in registers
          const int d = threadIdx.x % V;
          float column[KEYS];
#pragma unroll
          for (int j = 0; j < KEYS; ++j) column[j] = tile[j * ST + d];
#pragma unroll
          for (int i = 0; i < MAX_ACC; ++i) {
            const int o = threadIdx.x + THREADS * i;
            if (o >= o_first && o < o_end) {
              const int hr = o / V;
              if (hr % R < rows) {
                const float4* w4 = reinterpret_cast<const float4*>(w_use + (size_t)hr * KEYS);
                float sum = acc[i];
#pragma unroll
                for (int j4 = 0; j4 < KEYS / 4; ++j4) {
                  const float4 w = w4[j4];
                  sum = fmaf(w.x, column[4 * j4], sum);
                  sum = fmaf(w.y, column[4 * j4 + 1], sum);
                  sum = fmaf(w.z, column[4 * j4 + 2], sum);
                  sum = fmaf(w.w, column[4 * j4 + 3], sum);
                }
                acc[i] = sum;
              }
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < MAX_ACC; ++i) {
            const int o = threadIdx.x + THREADS * i;
            if (o >= o_first && o < o_end) {
              const int d = o % V, hr = o / V;
              if (hr % R < rows) {
                const float* w = w_use + (size_t)hr * KEYS;
                float sum = acc[i];
#pragma unroll 8
                for (int j = 0; j < KEYS; ++j) sum = fmaf(w[j], tile[j * ST + d], sum);
                acc[i] = sum;
              }
            }
          }
        }
      }
    }
  }

  const bool split = gridDim.z > 1;
#pragma unroll
  for (int i = 0; i < MAX_ACC; ++i) {
    const int o = threadIdx.x + THREADS * i;
    if (o >= outputs) continue;
    const int d = o % V, hr = o / V, r = hr % R, h = hr / R;
    if (r >= rows) continue;
    const size_t at = ((size_t)(q_start + row0 + r) * H + h) * V + d;
    if (split)
      partial[(size_t)blockIdx.z * a.total_rows * H * V + at] = acc[i];
    else
      out[at] = from_float<T>(acc[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
add_chunks_kernel(const float* partial, T* __restrict__ out, long long count, int chunks) {
  pdl_trigger();
  pdl_wait();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= count) return;
  float sum = 0.f;
  for (int c = 0; c < chunks; ++c) sum += __ldcg(partial + (size_t)c * count + index);
  out[index] = from_float<T>(sum);
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// qkv: float32 [rows, heads*dim + kv_heads*dim + kv_heads*vdim]; q_weight, k_weight: float32 [dim] or null;
// other_values: float32 rows of kv_heads*vdim entries spaced `other_stride` apart, or null; mix: one
// float32 on the device (read only with other_values); slots: where each row's k and v go.
MLR_EXPORT int mlr_head_norm_kv_write(const float* qkv, const float* q_weight, const float* k_weight,
                                      const float* other_values, long long other_stride, const float* mix,
                                      const long long* slots, void* q_out, void* k_pool, void* v_pool, int rows, int heads,
                                      int kv_heads, int dim, int vdim, int page_size, float eps, int write_kv, int dtype,
                                      cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || page_size <= 0) return MLR_BAD_SIZE;
  if (other_values != nullptr && mix == nullptr) return MLR_BAD_SIZE;
  const long long items = (long long)rows * (heads + 2 * kv_heads);
  const long long blocks = (items + 3) / 4;
  if (blocks > 0x7fffffffLL) return MLR_TOO_LARGE;
  if (dtype == MLR_F32)
    launch_kernel(head_norm_kv_write_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, qkv, q_weight, k_weight,
                  other_values, other_stride, mix, slots, (float*)q_out, (float*)k_pool, (float*)v_pool, rows, heads,
                  kv_heads, dim, vdim, page_size, eps, write_kv);
  else if (dtype == MLR_BF16)
    launch_kernel(head_norm_kv_write_kernel<bf16>, dim3((unsigned)blocks), dim3(128), 0, stream, qkv, q_weight, k_weight,
                  other_values, other_stride, mix, slots, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool, rows, heads, kv_heads,
                  dim, vdim, page_size, eps, write_kv);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// Floats between the rows of the shared tile: a multiple of four that is no multiple of eight (16-byte
// pieces, and a quarter warp's pieces fall into different banks), or any odd number for single entries.
static int sigmoid_tile_stride(int dim, int vdim, bool vector) {
  const int widest = dim > vdim ? dim : vdim;
  if (!vector) return widest | 1;
  return widest % 8 == 0 ? widest + 4 : widest;
}

// Shared memory of one CTA that takes `rows` rows.
static size_t sigmoid_shared_bytes(int heads, int dim, int vdim, int rows) {
  const int widest = dim > vdim ? dim : vdim;
  return sizeof(float) * ((size_t)heads * rows * dim + 2 * (size_t)heads * rows * KEYS + (size_t)KEYS * (widest + 4) +
                          (size_t)heads * heads + 2 * KEYS);
}

// Rows per CTA (a power of two, at most 16) so that a thread holds at most MAX_ACC sums and the CTA's
// shared memory fits; 0 if not even one row does.
MLR_EXPORT int mlr_attention_sigmoid_rows(int heads, int dim, int vdim) {
  for (int rows = PLAN_ROWS; rows >= 1; rows /= 2) {
    const long long outputs = (long long)heads * rows * vdim;
    if (outputs <= (long long)MAX_ACC * THREADS && sigmoid_shared_bytes(heads, dim, vdim, rows) <= 200 * 1024) return rows;
  }
  return 0;
}

// q: [rows, heads, dim]; out: [rows, heads, vdim]; pools [pages, kv_heads, page_size, dim | vdim]; r1, r2,
// pb: float32 [heads] or null (r1 and r2 together); talk: float32 [heads, heads] or null.
// tile_seg/tile_row0: entries of up to 16 rows of one segment.  chunks > 1: the keys of a row are shared
// out in chunks of chunk_keys (a multiple of 32) and `partial` (float32 [chunks, total_rows, heads * vdim])
// receives the chunks' sums, which a second kernel adds up in chunk order.
MLR_EXPORT int mlr_attention_sigmoid(const void* q, const void* k_pool, const void* v_pool, void* out, float* partial,
                                     const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                     const int* seg_q_len, const int* seg_pos0, const int* block_table,
                                     const int* seg_slot, int table_width, int tiles, int total_rows, int heads,
                                     int kv_heads, int dim, int vdim, int page_size, float scale, const float* r1,
                                     const float* r2, const float* pb, const float* talk, int chunks, int chunk_keys,
                                     int dtype, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || total_rows <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || dim <= 0 || vdim <= 0 ||
      page_size <= 0 || table_width <= 0 || chunks <= 0 || chunk_keys <= 0 || chunk_keys % KEYS != 0 ||
      (chunks > 1 && partial == nullptr) || ((r1 == nullptr) != (r2 == nullptr)))
    return MLR_BAD_SIZE;
  const int rows = mlr_attention_sigmoid_rows(heads, dim, vdim);
  if (rows == 0 || chunks > 65535) return MLR_TOO_LARGE;
  // whole 16-byte pieces: head sizes in multiples of a piece, at most MAX_STAGE pieces per thread and tile
  const int piece = dtype == MLR_BF16 ? 8 : 4;
  const int widest = dim > vdim ? dim : vdim;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vector = dim % piece == 0 && vdim % piece == 0 && KEYS * (widest / piece) <= MAX_STAGE * THREADS &&
                      aligned(k_pool) && aligned(v_pool);
  SigmoidArgs a{tile_seg, tile_row0, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot, r1, r2, pb, talk,
                table_width, heads, kv_heads, dim, vdim, page_size, rows, chunk_keys, total_rows,
                sigmoid_tile_stride(dim, vdim, vector), scale};
  const size_t shared = sigmoid_shared_bytes(heads, dim, vdim, rows);
  const dim3 grid(tiles, PLAN_ROWS / rows, chunks);
  auto launch = [&](auto kernel, auto* typed_out) -> int {
    using T = std::remove_pointer_t<decltype(typed_out)>;
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, grid, dim3(THREADS), shared, stream, (const T*)q, (const T*)k_pool, (const T*)v_pool, typed_out,
                  partial, a);
    int status = launch_status();
    if (status != MLR_OK || chunks == 1) return status;
    const long long count = (long long)total_rows * heads * vdim;
    launch_kernel(add_chunks_kernel<T>, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, (const float*)partial,
                  typed_out, count, chunks);
    return launch_status();
  };
  if (dtype == MLR_F32)
    return vector ? launch(attention_sigmoid_kernel<float, true>, (float*)out) : launch(attention_sigmoid_kernel<float, false>, (float*)out);
  if (dtype == MLR_BF16)
    return vector ? launch(attention_sigmoid_kernel<bf16, true>, (bf16*)out) : launch(attention_sigmoid_kernel<bf16, false>, (bf16*)out);
  return MLR_BAD_DTYPE;
}
