// Kernels around a softmax attention whose values are normalised and turned by their positions.
//
// mlr_rotated_prepare   one CTA per row of the step.  The row holds the float32 products
//                       [q: heads * dim | k: kv_heads * dim | v: kv_heads * vdim].  In this order:
//                         q, k   RMS norm over the WHOLE projection (all heads at once, one weight per
//                                entry; skipped without weights), then the first `rot` entries of
//                                every head turned by position * key_freq[i], sine and cosine
//                                multiplied by `magnitude`; the other entries pass;
//                         v      every head divided by its root mean square over vdim (if asked),
//                                then all vdim entries turned by position * value_freq[m] (if given);
//                         q goes out in the compute dtype, k and v into the cache pages.
//                       Pairs are (i, i + n/2) or, interleaved, (2i, 2i + 1), n being the number of
//                       turned entries.  All arithmetic is float32; sums have an order fixed by the
//                       sizes, so a row's numbers do not depend on the rest of the batch.
// mlr_turn_heads        x[row, head, :n] turned in place by sign * position * freq[i] (the way back of
//                       the values' rotation, applied to each head's attention output).
#include "common.cuh"

namespace mlr {

// the two entries of pair i among n turned entries
__device__ __forceinline__ void pair_places(int i, int n, int interleaved, int* a, int* b) {
  if (interleaved) {
    *a = 2 * i;
    *b = 2 * i + 1;
  } else {
    *a = i;
    *b = i + n / 2;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
rotated_prepare_kernel(const float* qkv, const int* positions, const float* __restrict__ q_weight,
                       const float* __restrict__ k_weight, const float* __restrict__ key_freq,
                       const float* __restrict__ value_freq, const long long* slots, T* __restrict__ q_out, T* k_pool,
                       T* v_pool, int heads, int kv_heads, int dim, int vdim, int rot, int interleaved,
                       int normalise_values, float eps, float magnitude, int page_size, int write_kv) {
  pdl_trigger();
  extern __shared__ float row[];       // [q | k | v] + 32 + kv_heads
  const int wq = heads * dim, wk = kv_heads * dim, wv = kv_heads * vdim;
  const int width = wq + wk + wv;
  float* scratch = row + width;
  float* value_scale = scratch + 32;
  const int r = blockIdx.x;
  pdl_wait();
  const float* src = qkv + (size_t)r * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) row[d] = src[d];
  __syncthreads();
  const int position = positions[r];

  // norms over whole projections
  float q_scale = 1.f, k_scale = 1.f;
  if (q_weight != nullptr) {
    float sq = 0.f;
    for (int d = threadIdx.x; d < wq; d += blockDim.x) sq = fmaf(row[d], row[d], sq);
    q_scale = 1.f / sqrtf(block_sum(sq, scratch) / (float)wq + eps);
  }
  if (k_weight != nullptr) {
    float sq = 0.f;
    for (int d = threadIdx.x; d < wk; d += blockDim.x) sq = fmaf(row[wq + d], row[wq + d], sq);
    k_scale = 1.f / sqrtf(block_sum(sq, scratch) / (float)wk + eps);
  }
  // unit root mean square per value head: a warp per head
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int g = warp; g < kv_heads; g += warps) {
      float scale = 1.f;
      if (normalise_values) {
        const float* v = row + wq + wk + g * vdim;
        float sq = 0.f;
        for (int d = lane; d < vdim; d += 32) sq = fmaf(v[d], v[d], sq);
        scale = 1.f / sqrtf(warp_sum(sq) / (float)vdim + eps);
      }
      if (lane == 0) value_scale[g] = scale;
    }
  }
  __syncthreads();

  const long long slot = slots != nullptr ? slots[r] : -1;
  const bool store = write_kv && slot >= 0;
  const long long page = store ? slot / page_size : 0;
  const int offset = store ? (int)(slot % page_size) : 0;

  // q and k: one thread per pair of the turned part, then the entries that pass
  const int half = rot / 2;
  const int q_pairs = heads * half, k_pairs = kv_heads * half;
  for (int idx = threadIdx.x; idx < q_pairs + k_pairs; idx += blockDim.x) {
    const bool is_q = idx < q_pairs;
    const int local = is_q ? idx : idx - q_pairs;
    const int head = local / half, i = local - head * half;
    int a, b;
    pair_places(i, rot, interleaved, &a, &b);
    const int base = (is_q ? 0 : wq) + head * dim;
    const float* weight = is_q ? q_weight : k_weight;
    const float scale = is_q ? q_scale : k_scale;
    float u = row[base + a] * scale, v = row[base + b] * scale;
    if (weight != nullptr) {
      u *= weight[head * dim + a];
      v *= weight[head * dim + b];
    }
    float sine, cosine;
    sincosf((float)position * key_freq[i], &sine, &cosine);
    sine *= magnitude;
    cosine *= magnitude;
    float y1, y2;
    rotate_pair(u, v, sine, cosine, &y1, &y2);
    if (is_q) {
      T* dst = q_out + (size_t)r * wq + head * dim;
      dst[a] = from_float<T>(y1);
      dst[b] = from_float<T>(y2);
    } else if (store) {
      T* dst = k_pool + (((size_t)page * kv_heads + head) * page_size + offset) * dim;
      dst[a] = from_float<T>(y1);
      dst[b] = from_float<T>(y2);
    }
  }
  const int rest = dim - rot;
  if (rest > 0) {
    for (int idx = threadIdx.x; idx < (heads + kv_heads) * rest; idx += blockDim.x) {
      const bool is_q = idx < heads * rest;
      const int local = is_q ? idx : idx - heads * rest;
      const int head = local / rest, d = rot + (local - head * rest);
      const float* weight = is_q ? q_weight : k_weight;
      float u = row[(is_q ? 0 : wq) + head * dim + d] * (is_q ? q_scale : k_scale);
      if (weight != nullptr) u *= weight[head * dim + d];
      if (is_q) q_out[(size_t)r * wq + head * dim + d] = from_float<T>(u);
      else if (store) k_pool[(((size_t)page * kv_heads + head) * page_size + offset) * dim + d] = from_float<T>(u);
    }
  }
  // v
  if (store) {
    if (value_freq != nullptr) {
      const int v_half = vdim / 2;
      for (int idx = threadIdx.x; idx < kv_heads * v_half; idx += blockDim.x) {
        const int g = idx / v_half, m = idx - g * v_half;
        int a, b;
        pair_places(m, vdim, interleaved, &a, &b);
        const float* v = row + wq + wk + g * vdim;
        const float u = v[a] * value_scale[g], w = v[b] * value_scale[g];
        float sine, cosine;
        sincosf((float)position * value_freq[m], &sine, &cosine);
        float y1, y2;
        rotate_pair(u, w, sine, cosine, &y1, &y2);
        T* dst = v_pool + (((size_t)page * kv_heads + g) * page_size + offset) * vdim;
        dst[a] = from_float<T>(y1);
        dst[b] = from_float<T>(y2);
      }
    } else {
      for (int idx = threadIdx.x; idx < wv; idx += blockDim.x) {
        const int g = idx / vdim, d = idx - g * vdim;
        v_pool[(((size_t)page * kv_heads + g) * page_size + offset) * vdim + d] =
            from_float<T>(row[wq + wk + idx] * value_scale[g]);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
turn_heads_kernel(T* x, const int* positions, const float* __restrict__ freq, int heads, int dim, int n, int interleaved,
                  float sign) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int half = n / 2;
  const float position = sign * (float)positions[r];
  T* row = x + (size_t)r * heads * dim;
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    int a, b;
    pair_places(i, n, interleaved, &a, &b);
    float sine, cosine;
    sincosf(position * freq[i], &sine, &cosine);
    T* h = row + head * dim;
    float y1, y2;
    rotate_pair(to_float(h[a]), to_float(h[b]), sine, cosine, &y1, &y2);
    h[a] = from_float<T>(y1);
    h[b] = from_float<T>(y2);
  }
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// qkv: float32 [rows, heads*dim + kv_heads*dim + kv_heads*vdim]; positions: int32 [rows]; q_weight
// [heads*dim] / k_weight [kv_heads*dim]: float32 or null (no norm); key_freq: float32 [rot/2];
// value_freq: float32 [vdim/2] or null (values are not turned); slots: int64 [rows], place of each row's
// key and value as page * page_size + offset (negative: not stored); q_out: [rows, heads*dim];
// k_pool [pages, kv_heads, page_size, dim], v_pool [pages, kv_heads, page_size, vdim] in `dtype`.
MLR_EXPORT int mlr_rotated_prepare(const float* qkv, const int* positions, const float* q_weight, const float* k_weight,
                                   const float* key_freq, const float* value_freq, const long long* slots, void* q_out,
                                   void* k_pool, void* v_pool, int rows, int heads, int kv_heads, int dim, int vdim,
                                   int rot, int interleaved, int normalise_values, float eps, float magnitude,
                                   int page_size, int write_kv, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rot < 0 || rot > dim || rot % 2 != 0 ||
      page_size <= 0 || (value_freq != nullptr && vdim % 2 != 0))
    return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * ((size_t)(heads + kv_heads) * dim + (size_t)kv_heads * vdim + 32 + kv_heads);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  // threads by the row's width alone (the sums' order follows the block's size: a row must not see the batch)
  const int row_width = (heads + kv_heads) * dim + kv_heads * vdim;
  const int threads = row_width <= 2048 ? 256 : row_width <= 4096 ? 512 : 1024;
  auto launch = [&](auto kernel, auto* q_typed, auto* k_typed, auto* v_typed) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, dim3(rows), dim3(threads), shared, stream, qkv, positions, q_weight, k_weight, key_freq, value_freq,
                  slots, q_typed, k_typed, v_typed, heads, kv_heads, dim, vdim, rot, interleaved, normalise_values, eps,
                  magnitude, page_size, write_kv);
    return launch_status();
  };
  if (dtype == MLR_F32) return launch(rotated_prepare_kernel<float>, (float*)q_out, (float*)k_pool, (float*)v_pool);
  if (dtype == MLR_BF16) return launch(rotated_prepare_kernel<bf16>, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool);
  return MLR_BAD_DTYPE;
}

// x: [rows, heads, dim] in `dtype`, the first n entries of every head turned in place by
// sign * positions[row] * freq[i] (freq: float32 [n/2]).
MLR_EXPORT int mlr_turn_heads(void* x, const int* positions, const float* freq, int rows, int heads, int dim, int n,
                              int interleaved, float sign, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || dim <= 0 || n <= 0 || n > dim || n % 2 != 0) return MLR_BAD_SIZE;
  if (dtype == MLR_F32)
    launch_kernel(turn_heads_kernel<float>, dim3(rows), dim3(256), 0, stream, (float*)x, positions, freq, heads, dim, n,
                  interleaved, sign);
  else if (dtype == MLR_BF16)
    launch_kernel(turn_heads_kernel<bf16>, dim3(rows), dim3(256), 0, stream, (bf16*)x, positions, freq, heads, dim, n,
                  interleaved, sign);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}
