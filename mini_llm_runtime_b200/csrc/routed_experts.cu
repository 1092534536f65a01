// A routed set of small gated feed-forward experts: the router and the per-pair kernels.
//
// mlr_route_experts      one warp per row: logits z = R x in float32 (R float32 [experts, K]),
//                        scores s = softmax(z) (or sigmoid(z)), choice scores c = s + correction; experts
//                        form `groups` equal groups of neighbours, a group's score is its largest choice
//                        score, only experts of the `keep` best groups can be chosen; the `top` largest
//                        choice scores win (ties: the lower index); the weights are the winners' s,
//                        divided by their sum if asked.  chosen int32 [rows, top], weights float32.
// mlr_expert_hidden      for every (row, chosen expert) pair p: hidden[p] = act(Wg_e x) * (Wu_e x), one warp
//                        per output, the dot products split over the lanes in a fixed order.
// mlr_expert_down        out[row] = sum_t weights[row, t] * (Wd_e(t) hidden[row * top + t]) in float32, t
//                        ascending: one warp per output column, the chosen experts one after the other.
// These serve the 32-bit path at every size and the bfloat16 path for steps of few rows (each pair
// streams its expert's matrices once, 16-byte loads); many rows in bfloat16 go through the sorted,
// grouped tensor-core product instead.
// mlr_sort_pairs         counting sort of the pairs by expert for the grouped product: the place of every
//                        pair in expert order, the token of every place, and the list of row tiles.
// mlr_gather_rows_by     xs[place] = x[token of place].
// mlr_combine_pairs      out[row] = sum_t weights[row, t] * y[place of pair (row, t)], t ascending.
#include "common.cuh"

namespace mlr {

constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ float load_as_float(const float* p) { return *p; }
__device__ __forceinline__ float load_as_float(const bf16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_experts_kernel(const T* x, const float* __restrict__ router, const float* __restrict__ correction, int* chosen,
                     float* weights, int rows, int K, int experts, int top, int groups, int keep, int sigmoid_scores,
                     int renormalise) {
  pdl_trigger();
  extern __shared__ float shared[];      // per warp: [experts] scores + [experts] choice scores + [groups]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * ROUTE_WARPS + warp;
  float* score = shared + (size_t)warp * (2 * experts + groups);
  float* choice = score + experts;
  float* group_score = choice + experts;
  pdl_wait();
  if (row >= rows) return;
  const T* xr = x + (size_t)row * K;
  for (int e = 0; e < experts; ++e) {
    const float* w = router + (size_t)e * K;
    float sum = 0.f;
    for (int k = lane; k < K; k += 32) sum = fmaf(w[k], load_as_float(xr + k), sum);
    sum = warp_sum(sum);
    if (lane == 0) score[e] = sum;
  }
  __syncwarp();
  if (sigmoid_scores) {
    for (int e = lane; e < experts; e += 32) score[e] = 1.f / (1.f + expf(-score[e]));
  } else {
    float top_logit = -INFINITY;
    for (int e = lane; e < experts; e += 32) top_logit = fmaxf(top_logit, score[e]);
    top_logit = warp_max(top_logit);
    float total = 0.f;
    for (int e = lane; e < experts; e += 32) {
      const float p = expf(score[e] - top_logit);
      score[e] = p;
      total += p;
    }
    total = warp_sum(total);
    for (int e = lane; e < experts; e += 32) score[e] = score[e] / total;
  }
  for (int e = lane; e < experts; e += 32) choice[e] = score[e] + (correction != nullptr ? correction[e] : 0.f);
  __syncwarp();
  // the best `keep` groups stay; the others' choice scores become minus infinity
  const int size = experts / groups;
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int j = 0; j < size; ++j) best = fmaxf(best, choice[g * size + j]);
      group_score[g] = best;
    }
    __syncwarp();
    // rank of every group: groups with a larger score, or an equal one and a lower index, come first
    for (int g = lane; g < groups; g += 32) {
      int before = 0;
      const float mine = group_score[g];
      for (int o = 0; o < groups; ++o) {
        const float other = group_score[o];
        before += (other > mine || (other == mine && o < g)) ? 1 : 0;
      }
      if (before >= keep)
        for (int j = 0; j < size; ++j) choice[g * size + j] = -INFINITY;
    }
    __syncwarp();
  }
  float weight_sum = 0.f;
  for (int t = 0; t < top; ++t) {
    float best = -INFINITY;
    int best_at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float c = choice[e];
      if (c > best || (c == best && e < best_at && c != -INFINITY)) {
        best = c;
        best_at = e;
      }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_at = __shfl_xor_sync(0xffffffffu, best_at, offset);
      if (other > best || (other == best && other_at < best_at)) {
        best = other;
        best_at = other_at;
      }
    }
    if (best_at == 0x7fffffff) best_at = 0;      // fewer eligible experts than `top` (the host refuses such a config)
    const float w = score[best_at];
    weight_sum += w;
    if (lane == 0) {
      chosen[(size_t)row * top + t] = best_at;
      weights[(size_t)row * top + t] = w;
      choice[best_at] = -INFINITY;
    }
    __syncwarp();
  }
  if (renormalise && lane == 0)
    for (int t = 0; t < top; ++t) weights[(size_t)row * top + t] /= weight_sum;
}

// Dot product of a weight row with a float32 vector in shared memory, split over the lanes of a warp:
// with `wide`, lane l takes the pieces of 8 (bfloat16) or 4 (float32) entries l, l + 32, ..; else single
// entries.  Every lane gets the sum; the order of additions depends on K only.
__device__ __forceinline__ float warp_dot(const bf16* __restrict__ w, const float* x, int K, int lane, bool wide) {
  float sum = 0.f;
  if (wide) {
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(w + k));
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 v = __bfloat1622float2(pairs[j]);
        sum = fmaf(v.x, x[k + 2 * j], sum);
        sum = fmaf(v.y, x[k + 2 * j + 1], sum);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) sum = fmaf(__bfloat162float(w[k]), x[k], sum);
  }
  return warp_sum(sum);
}
__device__ __forceinline__ float warp_dot(const float* __restrict__ w, const float* x, int K, int lane, bool wide) {
  float sum = 0.f;
  if (wide) {
    for (int k = lane * 4; k < K; k += 128) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(w + k));
      sum = fmaf(v.x, x[k], sum);
      sum = fmaf(v.y, x[k + 1], sum);
      sum = fmaf(v.z, x[k + 2], sum);
      sum = fmaf(v.w, x[k + 3], sum);
    }
  } else {
    for (int k = lane; k < K; k += 32) sum = fmaf(w[k], x[k], sum);
  }
  return warp_sum(sum);
}

constexpr int EXPERT_WARPS = 8;
constexpr int HIDDEN_PER_CTA = 32;     // outputs of one CTA of the hidden kernel (4 per warp)
constexpr int DOWN_PER_CTA = 32;

// gate_up: [experts][2 * ff][K] with rows in blocks of `block` gate rows followed by the `block` up rows
// of the same outputs (block == ff: all gate rows first).
template <typename T>
__global__ void __launch_bounds__(EXPERT_WARPS * 32)
expert_hidden_kernel(const T* x, const int* chosen, const T* __restrict__ gate_up, T* hidden, int K, int ff, int top,
                     int block, int act, int wide) {
  pdl_trigger();
  extern __shared__ float xs[];      // [K]
  const int pair = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  const int row = pair / top;
  const int expert = chosen[pair];
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = load_as_float(x + (size_t)row * K + k);
  __syncthreads();
  const T* w = gate_up + (size_t)expert * 2 * ff * K;
  for (int j = blockIdx.y * HIDDEN_PER_CTA + warp; j < min(ff, (blockIdx.y + 1) * HIDDEN_PER_CTA); j += EXPERT_WARPS) {
    const int gate_row = (j / block) * 2 * block + j % block;
    const float gate = warp_dot(w + (size_t)gate_row * K, xs, K, lane, wide != 0);
    const float up = warp_dot(w + (size_t)(gate_row + block) * K, xs, K, lane, wide != 0);
    if (lane == 0) {
      float value;
      if (act == 1) {
        value = 0.5f * gate * (1.f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate))) * up;
      } else {
        value = gate / (1.f + expf(-gate)) * up;
      }
      hidden[(size_t)pair * ff + j] = from_float<T>(value);
    }
  }
}

// down: [experts][N][ff]
template <typename T>
__global__ void __launch_bounds__(EXPERT_WARPS * 32)
expert_down_kernel(const T* hidden, const int* chosen, const float* weights, const T* __restrict__ down, float* out, int N,
                   int ff, int top, int wide) {
  pdl_trigger();
  extern __shared__ float hs[];      // [top][ff]
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  for (int k = threadIdx.x; k < top * ff; k += blockDim.x) hs[k] = load_as_float(hidden + (size_t)row * top * ff + k);
  __syncthreads();
  for (int n = blockIdx.y * DOWN_PER_CTA + warp; n < min(N, (blockIdx.y + 1) * DOWN_PER_CTA); n += EXPERT_WARPS) {
    float total = 0.f;
    for (int t = 0; t < top; ++t) {
      const int expert = chosen[(size_t)row * top + t];
      const float y = warp_dot(down + ((size_t)expert * N + n) * ff, hs + (size_t)t * ff, ff, lane, wide != 0);
      total = fmaf(weights[(size_t)row * top + t], y, total);
    }
    if (lane == 0) out[(size_t)row * N + n] = total;
  }
}

// ---------------------------------------------------------------- sorted form for the grouped product
// One CTA.  place[p]: where pair p lands in expert order; token_of[place]: the row it came from;
// tiles: for every used tile of `tile_rows` rows (expert, first place, end place), then -1 entries up
// to max_tiles.  The order inside an expert's run is not fixed (atomics); every pair's result is
// computed from its own row alone, so the order changes no number.
__global__ void __launch_bounds__(1024)
sort_pairs_kernel(const int* chosen, int* place, int* token_of, int* tiles, int pairs, int top, int experts, int tile_rows,
                  int max_tiles) {
  pdl_trigger();
  extern __shared__ int counts[];        // [experts] counts, [experts + 1] starts, [experts] cursors
  int* starts = counts + experts;
  int* cursor = starts + experts + 1;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  pdl_wait();
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[chosen[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tile = 0;
    for (int e = 0; e < experts; ++e) {
      starts[e] = at;
      cursor[e] = at;
      for (int r = 0; r < counts[e] && tile < max_tiles; r += tile_rows, ++tile) {
        tiles[3 * tile] = e;
        tiles[3 * tile + 1] = at + r;
        tiles[3 * tile + 2] = at + counts[e];
      }
      at += counts[e];
    }
    starts[experts] = at;
    for (; tile < max_tiles; ++tile) {
      tiles[3 * tile] = -1;
      tiles[3 * tile + 1] = 0;
      tiles[3 * tile + 2] = 0;
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int at = atomicAdd(&cursor[chosen[p]], 1);
    place[p] = at;
    token_of[at] = p / top;
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
gather_rows_by_kernel(const T* x, const int* token_of, T* out, int width_bytes) {
  pdl_trigger();
  pdl_wait();
  const int at = blockIdx.x;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(x) + (size_t)token_of[at] * width_bytes;
  uint8_t* dst = reinterpret_cast<uint8_t*>(out) + (size_t)at * width_bytes;
  if (width_bytes % 16 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0) {
    for (int b = threadIdx.x * 16; b < width_bytes; b += blockDim.x * 16)
      *reinterpret_cast<uint4*>(dst + b) = __ldcg(reinterpret_cast<const uint4*>(src + b));
  } else {
    for (int b = threadIdx.x; b < width_bytes; b += blockDim.x) dst[b] = src[b];
  }
}

__global__ void __launch_bounds__(256)
combine_pairs_kernel(const float* y, const int* place, const float* weights, float* out, int N, int top) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float total = 0.f;
    for (int t = 0; t < top; ++t)
      total = fmaf(weights[(size_t)row * top + t], __ldcg(y + (size_t)place[(size_t)row * top + t] * N + n), total);
    out[(size_t)row * N + n] = total;
  }
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// x: [rows, K] in `dtype`; router: float32 [experts, K]; correction: float32 [experts] or null;
// chosen: int32 [rows, top]; weights: float32 [rows, top].
MLR_EXPORT int mlr_route_experts(const void* x, const float* router, const float* correction, int* chosen, float* weights,
                                 int rows, int K, int experts, int top, int groups, int keep, int sigmoid_scores,
                                 int renormalise, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || K <= 0 || experts <= 0 || top <= 0 || groups <= 0 || keep <= 0 || keep > groups || experts % groups != 0 ||
      top > keep * (experts / groups))
    return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * ROUTE_WARPS * (2 * (size_t)experts + groups);
  if (shared > 48 * 1024) return MLR_TOO_LARGE;
  const dim3 grid((rows + ROUTE_WARPS - 1) / ROUTE_WARPS), block(ROUTE_WARPS * 32);
  if (dtype == MLR_F32)
    launch_kernel(route_experts_kernel<float>, grid, block, shared, stream, (const float*)x, router, correction, chosen,
                  weights, rows, K, experts, top, groups, keep, sigmoid_scores, renormalise);
  else if (dtype == MLR_BF16)
    launch_kernel(route_experts_kernel<bf16>, grid, block, shared, stream, (const bf16*)x, router, correction, chosen,
                  weights, rows, K, experts, top, groups, keep, sigmoid_scores, renormalise);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// x: [rows, K]; chosen: int32 [rows * top]; gate_up: [experts, 2 * ff, K]; hidden: [rows * top, ff]; all
// floating tensors in `dtype`.  act: 0 silu, 1 the tanh form of gelu.
MLR_EXPORT int mlr_expert_hidden(const void* x, const int* chosen, const void* gate_up, void* hidden, int rows, int K, int ff,
                                 int top, int block, int act, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || K <= 0 || ff <= 0 || top <= 0 || block <= 0 || ff % block != 0) return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * (size_t)K;
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  const dim3 grid(rows * top, (ff + HIDDEN_PER_CTA - 1) / HIDDEN_PER_CTA), threads(EXPERT_WARPS * 32);
  auto launch = [&](auto kernel, auto* xt, auto* wt, auto* ht, int wide) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, grid, threads, shared, stream, xt, chosen, wt, ht, K, ff, top, block, act, wide);
    return launch_status();
  };
  const bool aligned = ((uintptr_t)gate_up & 15) == 0;
  if (dtype == MLR_F32)
    return launch(expert_hidden_kernel<float>, (const float*)x, (const float*)gate_up, (float*)hidden, aligned && K % 4 == 0);
  if (dtype == MLR_BF16)
    return launch(expert_hidden_kernel<bf16>, (const bf16*)x, (const bf16*)gate_up, (bf16*)hidden, aligned && K % 8 == 0);
  return MLR_BAD_DTYPE;
}

// hidden: [rows * top, ff]; down: [experts, N, ff] in `dtype`; weights: float32 [rows * top]; out: float32 [rows, N].
MLR_EXPORT int mlr_expert_down(const void* hidden, const int* chosen, const float* weights, const void* down, float* out,
                               int rows, int N, int ff, int top, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || N <= 0 || ff <= 0 || top <= 0) return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * (size_t)top * ff;
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  const dim3 grid(rows, (N + DOWN_PER_CTA - 1) / DOWN_PER_CTA), threads(EXPERT_WARPS * 32);
  auto launch = [&](auto kernel, auto* ht, auto* wt, int wide) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, grid, threads, shared, stream, ht, chosen, weights, wt, out, N, ff, top, wide);
    return launch_status();
  };
  const bool aligned = ((uintptr_t)down & 15) == 0;
  if (dtype == MLR_F32) return launch(expert_down_kernel<float>, (const float*)hidden, (const float*)down, aligned && ff % 4 == 0);
  if (dtype == MLR_BF16) return launch(expert_down_kernel<bf16>, (const bf16*)hidden, (const bf16*)down, aligned && ff % 8 == 0);
  return MLR_BAD_DTYPE;
}

// chosen: int32 [pairs]; place: int32 [pairs]; token_of: int32 [pairs]; tiles: int32 [max_tiles, 3].
MLR_EXPORT int mlr_sort_pairs(const int* chosen, int* place, int* token_of, int* tiles, int pairs, int top, int experts,
                              int tile_rows, int max_tiles, cudaStream_t stream) {
  if (pairs == 0) return MLR_OK;
  if (pairs < 0 || top <= 0 || experts <= 0 || tile_rows <= 0 || max_tiles <= 0) return MLR_BAD_SIZE;
  const size_t shared = sizeof(int) * (3 * (size_t)experts + 1);
  if (shared > 48 * 1024) return MLR_TOO_LARGE;
  launch_kernel(sort_pairs_kernel, dim3(1), dim3(1024), shared, stream, chosen, place, token_of, tiles, pairs, top, experts,
                tile_rows, max_tiles);
  return launch_status();
}

MLR_EXPORT int mlr_gather_rows_by(const void* x, const int* token_of, void* out, int places, int width_bytes,
                                  cudaStream_t stream) {
  if (places == 0) return MLR_OK;
  if (places < 0 || width_bytes <= 0) return MLR_BAD_SIZE;
  launch_kernel(gather_rows_by_kernel<uint8_t>, dim3(places), dim3(128), 0, stream, (const uint8_t*)x, token_of,
                (uint8_t*)out, width_bytes);
  return launch_status();
}

MLR_EXPORT int mlr_combine_pairs(const float* y, const int* place, const float* weights, float* out, int rows, int N, int top,
                                 cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || N <= 0 || top <= 0) return MLR_BAD_SIZE;
  launch_kernel(combine_pairs_kernel, dim3(rows), dim3(256), 0, stream, y, place, weights, out, N, top);
  return launch_status();
}
