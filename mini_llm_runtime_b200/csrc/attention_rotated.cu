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

#include <algorithm>
#include <type_traits>

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


// Four consecutive entries d0 .. d0 + 3 of a head after norm and rotation, from the head's float32
// entries (16-byte aligned, in shared memory): each times `scale` (times its weight), turned with its
// partner if it is among the n turned entries.  sine / cosine: the row's tables, one entry per pair.
// d0 % 4 == 0 and n % 8 == 0: the four entries turn together or not at all, interleaved partners lie
// inside the piece, the others in the piece n / 2 further on or back.  The arithmetic is rotate_pair's.
__device__ __forceinline__ float4 scaled4(const float* head, const float* __restrict__ weight, float scale, int d) {
  float4 x = *reinterpret_cast<const float4*>(head + d);
  x.x *= scale; x.y *= scale; x.z *= scale; x.w *= scale;
  if (weight != nullptr) {
    const float4 w = *reinterpret_cast<const float4*>(weight + d);
    x.x *= w.x; x.y *= w.y; x.z *= w.z; x.w *= w.w;
  }
  return x;
}

__device__ __forceinline__ float4 turned4(const float* head, const float* __restrict__ weight, float scale, int d0, int n,
                                          int interleaved, const float* sine, const float* cosine) {
  const float4 x = scaled4(head, weight, scale, d0);
  if (d0 >= n) return x;
  float4 y;
  if (interleaved) {
    const float2 s = *reinterpret_cast<const float2*>(sine + (d0 >> 1)), c = *reinterpret_cast<const float2*>(cosine + (d0 >> 1));
    rotate_pair(x.x, x.y, s.x, c.x, &y.x, &y.y);
    rotate_pair(x.z, x.w, s.y, c.y, &y.z, &y.w);
    return y;
  }
  const int half = n >> 1;
  const bool first = d0 < half;
  const int i = first ? d0 : d0 - half;
  const float4 p = scaled4(head, weight, scale, first ? d0 + half : d0 - half);
  const float4 s = *reinterpret_cast<const float4*>(sine + i), c = *reinterpret_cast<const float4*>(cosine + i);
  if (first) {
    y.x = __fsub_rn(__fmul_rn(x.x, c.x), __fmul_rn(p.x, s.x));
    y.y = __fsub_rn(__fmul_rn(x.y, c.y), __fmul_rn(p.y, s.y));
    y.z = __fsub_rn(__fmul_rn(x.z, c.z), __fmul_rn(p.z, s.z));
    y.w = __fsub_rn(__fmul_rn(x.w, c.w), __fmul_rn(p.w, s.w));
  } else {
    y.x = __fadd_rn(__fmul_rn(x.x, c.x), __fmul_rn(p.x, s.x));
    y.y = __fadd_rn(__fmul_rn(x.y, c.y), __fmul_rn(p.y, s.y));
    y.z = __fadd_rn(__fmul_rn(x.z, c.z), __fmul_rn(p.z, s.z));
    y.w = __fadd_rn(__fmul_rn(x.w, c.w), __fmul_rn(p.w, s.w));
  }
  return y;
}

// four consecutive entries to memory aligned to their size
__device__ __forceinline__ void store4_as(float* dst, float4 y) { *reinterpret_cast<float4*>(dst) = y; }
__device__ __forceinline__ void store4_as(bf16* dst, float4 y) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
  uint2 packed;
  packed.x = *reinterpret_cast<const unsigned*>(&lo);
  packed.y = *reinterpret_cast<const unsigned*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}
__device__ __forceinline__ float4 load4_as(const float* src) { return *reinterpret_cast<const float4*>(src); }
__device__ __forceinline__ float4 load4_as(const bf16* src) {
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// two sums over the block at once
__device__ __forceinline__ void block_sum_two(float* a, float* b, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float u = warp_sum(*a), v = warp_sum(*b);
  __syncthreads();
  if (lane == 0) {
    scratch[warp] = u;
    scratch[32 + warp] = v;
  }
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  *a = warp_sum(lane < warps ? scratch[lane] : 0.f);
  *b = warp_sum(lane < warps ? scratch[32 + lane] : 0.f);
}

// THREADS: the block's size.  PRE: with 16-byte pieces, how many pieces of the NEXT row a thread asks for
// while the block works on this one (a block then takes every gridDim.x-th row); 0: one row per block.
template <typename T, int THREADS, int PRE>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS)
rotated_prepare_kernel(const float* qkv, const int* positions, const float* __restrict__ q_weight,
                       const float* __restrict__ k_weight, const float* __restrict__ key_freq,
                       const float* __restrict__ value_freq, const long long* slots, T* __restrict__ q_out, T* k_pool,
                       T* v_pool, int rows, int heads, int kv_heads, int dim, int vdim, int rot, int interleaved,
                       int normalise_values, float eps, float magnitude, int page_size, int write_kv, int chunked) {
  pdl_trigger();
  extern __shared__ __align__(16) float row[];       // [q | k | v], sines and cosines, 64 + kv_heads
  const int wq = heads * dim, wk = kv_heads * dim, wv = kv_heads * vdim;
  const int width = wq + wk + wv;
  float* key_sine = row + width;                     // [rot / 2], then the cosines
  float* key_cosine = key_sine + rot / 2;
  float* value_sine = key_cosine + rot / 2;          // [vdim / 2], then the cosines
  float* value_cosine = value_sine + vdim / 2;
  float* scratch = value_cosine + vdim / 2;
  float* value_scale = scratch + 64;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = THREADS >> 5;
  pdl_wait();

  if (chunked) {
    // Every head starts on a 16-byte piece and turns whole pieces (dim, vdim, rot multiples of 8): the
    // row comes in 16-byte pieces, its sines and cosines are evaluated once for all heads, and a thread
    // takes four consecutive entries at a time (no bank conflicts, 8- or 16-byte stores).
    const int pieces = width >> 2;
    const int key_pairs = rot / 2, value_pairs = value_freq != nullptr ? vdim / 2 : 0;
    // head sizes that are powers of two divide by a shift
    const int dim_shift = (dim & (dim - 1)) == 0 ? __ffs(dim) - 1 : -1;
    const int vdim_shift = (vdim & (vdim - 1)) == 0 ? __ffs(vdim) - 1 : -1;
    float4 ahead[PRE > 0 ? PRE : 1];
    int position_ahead = 0;
    long long slot_ahead = -1;
    auto ask = [&](int r) {
      const float4* src = reinterpret_cast<const float4*>(qkv + (size_t)r * width);
      position_ahead = positions[r];
      if (slots != nullptr) slot_ahead = slots[r];
#pragma unroll
      for (int j = 0; j < PRE; ++j)
        if (threadIdx.x + j * THREADS < pieces) ahead[j] = __ldcg(src + threadIdx.x + j * THREADS);
    };
    if (PRE > 0) ask(blockIdx.x);
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
      if (PRE > 0) {
#pragma unroll
        for (int j = 0; j < PRE; ++j)
          if (threadIdx.x + j * THREADS < pieces) reinterpret_cast<float4*>(row)[threadIdx.x + j * THREADS] = ahead[j];
      } else {
        const float4* src = reinterpret_cast<const float4*>(qkv + (size_t)r * width);
        for (int d = threadIdx.x; d < pieces; d += THREADS) reinterpret_cast<float4*>(row)[d] = __ldcg(src + d);
      }
      const int position = PRE > 0 ? position_ahead : positions[r];
      const long long slot = slots == nullptr ? -1 : PRE > 0 ? slot_ahead : slots[r];
      const bool store = write_kv && slot >= 0;
      const long long page = store ? slot / page_size : 0;
      const int offset = store ? (int)(slot % page_size) : 0;
      for (int i = threadIdx.x; i < key_pairs + value_pairs; i += THREADS) {
        float sine, cosine;
        if (i < key_pairs) {
          sincosf((float)position * key_freq[i], &sine, &cosine);
          key_sine[i] = sine * magnitude;
          key_cosine[i] = cosine * magnitude;
        } else {
          sincosf((float)position * value_freq[i - key_pairs], &sine, &cosine);
          value_sine[i - key_pairs] = sine;
          value_cosine[i - key_pairs] = cosine;
        }
      }
      __syncthreads();
      if (PRE > 0 && r + (int)gridDim.x < rows) ask(r + gridDim.x);
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
      float q_sq = 0.f, k_sq = 0.f;
      for (int d = threadIdx.x; d < (wq >> 2); d += THREADS) {
        const float4 x = reinterpret_cast<const float4*>(row)[d];
        q_sq += fmaf(x.x, x.x, x.y * x.y) + fmaf(x.z, x.z, x.w * x.w);
      }
      for (int d = threadIdx.x; d < (wk >> 2); d += THREADS) {
        const float4 x = reinterpret_cast<const float4*>(row + wq)[d];
        k_sq += fmaf(x.x, x.x, x.y * x.y) + fmaf(x.z, x.z, x.w * x.w);
      }
      block_sum_two(&q_sq, &k_sq, scratch);             // its barriers also publish value_scale
      const float q_scale = q_weight != nullptr ? 1.f / sqrtf(q_sq / (float)wq + eps) : 1.f;
      const float k_scale = k_weight != nullptr ? 1.f / sqrtf(k_sq / (float)wk + eps) : 1.f;

      const int pieces_q = wq >> 2, pieces_k = store ? wk >> 2 : 0, pieces_v = store ? wv >> 2 : 0;
      T* q_row = q_out + (size_t)r * wq;
      // a row's place in its page: head g lies g * page_size * size further on
      T* k_row = k_pool + ((size_t)page * kv_heads * page_size + offset) * dim;
      T* v_row = v_pool + ((size_t)page * kv_heads * page_size + offset) * vdim;
      for (int idx = threadIdx.x; idx < pieces_q + pieces_k + pieces_v; idx += THREADS) {
        if (idx < pieces_q + pieces_k) {
          const bool is_q = idx < pieces_q;
          const int e = (is_q ? idx : idx - pieces_q) << 2;
          const int head = dim_shift >= 0 ? e >> dim_shift : e / dim;
          const int d0 = e - head * dim;
          const float* weight = is_q ? q_weight : k_weight;
          if (weight != nullptr) weight += head * dim;
          const float4 y = turned4(row + (is_q ? e : wq + e) - d0, weight, is_q ? q_scale : k_scale, d0, rot, interleaved,
                                   key_sine, key_cosine);
          if (is_q) store4_as(q_row + e, y);
          else store4_as(k_row + head * (page_size * dim) + d0, y);
        } else {
          const int e = (idx - pieces_q - pieces_k) << 2;
          const int g = vdim_shift >= 0 ? e >> vdim_shift : e / vdim;
          const int d0 = e - g * vdim;
          const float4 y = turned4(row + wq + wk + e - d0, nullptr, value_scale[g], d0, value_freq != nullptr ? vdim : 0,
                                   interleaved, value_sine, value_cosine);
          store4_as(v_row + g * (page_size * vdim) + d0, y);
        }
      }
      __syncthreads();                                  // the next row overwrites what this one read
    }
    return;
  }

  const int r = blockIdx.x;
  const float* src = qkv + (size_t)r * width;
  const int position = positions[r];
  const long long slot = slots != nullptr ? slots[r] : -1;
  const bool store = write_kv && slot >= 0;
  const long long page = store ? slot / page_size : 0;
  const int offset = store ? (int)(slot % page_size) : 0;
  for (int d = threadIdx.x; d < width; d += blockDim.x) row[d] = src[d];
  __syncthreads();

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
  __syncthreads();

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

// The same in pieces of four entries (dim % 8 == 0, n % 8 == 0): the row's sines and cosines are
// evaluated once for all heads; interleaved partners lie inside a piece, and with partners n / 2 apart
// a thread takes a piece and its partner piece together, so nothing is read after another thread wrote it.
template <typename T>
__global__ void __launch_bounds__(256)
turn_heads_chunked_kernel(T* x, const int* positions, const float* __restrict__ freq, int heads, int dim, int n,
                          int interleaved, float sign) {
  pdl_trigger();
  extern __shared__ __align__(16) float tables[];      // n / 2 sines, then n / 2 cosines
  const int half = n / 2;
  float* sine = tables;
  float* cosine = tables + half;
  pdl_wait();
  const int r = blockIdx.x;
  const float position = sign * (float)positions[r];
  T* row = x + (size_t)r * heads * dim;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(position * freq[i], sine + i, cosine + i);
  __syncthreads();
  const int per_head = interleaved ? n >> 2 : half >> 2;
  for (int idx = threadIdx.x; idx < heads * per_head; idx += blockDim.x) {
    const int head = idx / per_head, d0 = (idx - head * per_head) << 2;
    T* h = row + head * dim;
    if (interleaved) {
      const float4 v = load4_as(h + d0);
      const float2 s = *reinterpret_cast<const float2*>(sine + (d0 >> 1)), c = *reinterpret_cast<const float2*>(cosine + (d0 >> 1));
      float4 y;
      rotate_pair(v.x, v.y, s.x, c.x, &y.x, &y.y);
      rotate_pair(v.z, v.w, s.y, c.y, &y.z, &y.w);
      store4_as(h + d0, y);
    } else {
      const float4 u = load4_as(h + d0), v = load4_as(h + d0 + half);
      const float4 s = *reinterpret_cast<const float4*>(sine + d0), c = *reinterpret_cast<const float4*>(cosine + d0);
      float4 y1, y2;
      rotate_pair(u.x, v.x, s.x, c.x, &y1.x, &y2.x);
      rotate_pair(u.y, v.y, s.y, c.y, &y1.y, &y2.y);
      rotate_pair(u.z, v.z, s.z, c.z, &y1.z, &y2.z);
      rotate_pair(u.w, v.w, s.w, c.w, &y1.w, &y2.w);
      store4_as(h + d0, y1);
      store4_as(h + d0 + half, y2);
    }
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
  const size_t shared =
      sizeof(float) * ((size_t)(heads + kv_heads) * dim + (size_t)kv_heads * vdim + rot + vdim + 64 + kv_heads);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  // 16-byte pieces where every head starts on one and turns whole pieces
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int chunked = dim % 8 == 0 && vdim % 8 == 0 && rot % 8 == 0 && aligned(qkv) && aligned(q_out) && aligned(k_pool) &&
                      aligned(v_pool) && aligned(q_weight) && aligned(k_weight);
  // threads by the row's width alone (the sums' order follows the block's size: a row must not see the batch)
  const int row_width = (heads + kv_heads) * dim + kv_heads * vdim;
  auto launch = [&](auto kernel, int threads, bool rows_ahead, auto* q_typed, auto* k_typed, auto* v_typed) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    int grid = rows;
    if (rows_ahead && chunked) {
      // as many blocks as run at once; each takes every grid-th row and asks for its next row early
      int per_sm = 0;
      cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, shared);
      if (err != cudaSuccess) return (int)err;
      grid = std::min(rows, std::max(per_sm, 1) * sm_count());
    }
    launch_kernel(kernel, dim3(grid), dim3(threads), shared, stream, qkv, positions, q_weight, k_weight, key_freq,
                  value_freq, slots, q_typed, k_typed, v_typed, rows, heads, kv_heads, dim, vdim, rot, interleaved,
                  normalise_values, eps, magnitude, page_size, write_kv, chunked);
    return launch_status();
  };
  auto launch_typed = [&](auto* q_typed, auto* k_typed, auto* v_typed) -> int {
    using T = std::remove_pointer_t<decltype(q_typed)>;
    if (row_width <= 4096) return launch(rotated_prepare_kernel<T, 256, 4>, 256, true, q_typed, k_typed, v_typed);
    if (row_width <= 8192) return launch(rotated_prepare_kernel<T, 512, 4>, 512, true, q_typed, k_typed, v_typed);
    return launch(rotated_prepare_kernel<T, 1024, 0>, 1024, false, q_typed, k_typed, v_typed);
  };
  if (dtype == MLR_F32) return launch_typed((float*)q_out, (float*)k_pool, (float*)v_pool);
  if (dtype == MLR_BF16) return launch_typed((bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool);
  return MLR_BAD_DTYPE;
}

// x: [rows, heads, dim] in `dtype`, the first n entries of every head turned in place by
// sign * positions[row] * freq[i] (freq: float32 [n/2]).
MLR_EXPORT int mlr_turn_heads(void* x, const int* positions, const float* freq, int rows, int heads, int dim, int n,
                              int interleaved, float sign, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || dim <= 0 || n <= 0 || n > dim || n % 2 != 0) return MLR_BAD_SIZE;
  const size_t staged = sizeof(float) * (size_t)n;
  if (dim % 8 == 0 && n % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && staged <= 48 * 1024) {
    if (dtype == MLR_F32)
      launch_kernel(turn_heads_chunked_kernel<float>, dim3(rows), dim3(256), staged, stream, (float*)x, positions, freq,
                    heads, dim, n, interleaved, sign);
    else if (dtype == MLR_BF16)
      launch_kernel(turn_heads_chunked_kernel<bf16>, dim3(rows), dim3(256), staged, stream, (bf16*)x, positions, freq,
                    heads, dim, n, interleaved, sign);
    else
      return MLR_BAD_DTYPE;
    return launch_status();
  }
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
