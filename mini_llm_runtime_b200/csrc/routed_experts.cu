// A routed set of small gated feed-forward experts: the router and the per-pair kernels.
//
// mlr_route_experts      logits z = R x in float32 (R float32 [experts, K]; a CTA per eight rows and eight
//                        experts), then a warp per row: scores s = softmax(z) (or sigmoid(z)), choice scores
//                        c = s + correction; experts
//                        form `groups` equal groups of neighbours, a group's score is the sum of its `group_top`
//                        largest choice scores (1: its largest), only experts of the `keep` best groups can be chosen; the `top` largest
//                        choice scores win (ties: the lower index); the weights are the winners' s,
//                        divided by their sum + renorm_eps if asked.  chosen int32 [rows, top], weights float32.
// mlr_expert_hidden      for every (row, chosen expert) pair p: hidden[p] = act(Wg_e x) * (Wu_e x), a warp
//                        per four outputs, the dot products split over the lanes in a fixed order.
// mlr_expert_down        out[row] = sum_t weights[row, t] * (Wd_e(t) hidden[row * top + t]) in float32, t
//                        ascending: a warp per four output columns, the chosen experts one after the other.
// These serve the 32-bit path at every size and the bfloat16 path for steps of few rows (each pair
// streams its expert's matrices once, 16-byte loads); many rows in bfloat16 go through the sorted,
// grouped tensor-core product instead.
// mlr_sort_pairs         counting sort of the pairs by expert for the grouped product: the place of every
//                        pair in expert order, the token of every place, and the list of row tiles.
// mlr_gather_rows_by     xs[place] = x[token of place].
// mlr_combine_pairs      out[row] = sum_t weights[row, t] * y[place of pair (row, t)], t ascending.
#include "common.cuh"

namespace mlr {

constexpr int ROUTE_WARPS = 8;     // warps of a logits CTA: one expert each
constexpr int ROUTE_ROWS = 8;      // most rows one logits CTA takes (each router entry it loads serves all of them)
constexpr int CHOOSE_WARPS = 4;    // rows of a choosing CTA: one warp each

__device__ __forceinline__ float load_as_float(const float* p) { return *p; }
__device__ __forceinline__ float load_as_float(const bf16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ void unpack(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(pairs[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack(const uint4& raw, float (&v)[4]) {
  v[0] = __uint_as_float(raw.x);
  v[1] = __uint_as_float(raw.y);
  v[2] = __uint_as_float(raw.z);
  v[3] = __uint_as_float(raw.w);
}

// Router logits.  CTA (i, j) takes rows i * rows_per_cta .. and experts j * 8 * E .., E neighbouring
// experts per warp (E = 1 for steps of few rows: more CTAs; E = 4 for many: a row's piece read from
// shared memory serves four experts).  The rows wait in shared memory as float32; lane l multiplies
// the 16-byte pieces l, l + 32, .. of an expert's router row (single entries without `wide`) with
// all the CTA's rows, one running sum per row and expert, so the order of a logit's additions
// depends on K alone: not on the rows beside it, nor on E.
template <typename T, int E>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
router_logits_kernel(const T* x, const float* __restrict__ router, float* logits, int rows, int K, int experts,
                     int rows_per_cta, int wide, int x_wide) {
  pdl_trigger();
  extern __shared__ __align__(16) float xs[];      // [rows_per_cta][K]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = blockIdx.x * rows_per_cta;
  const int live = min(rows_per_cta, rows - row0);
  pdl_wait();
  if (x_wide) {
    constexpr int N = 16 / sizeof(T);
    const int pieces = K / N;
#pragma unroll 4
    for (int idx = threadIdx.x; idx < rows_per_cta * pieces; idx += blockDim.x) {
      const int r = idx / pieces, c = idx - r * pieces;
      float v[N];
      if (r < live) {
        unpack(__ldcg(reinterpret_cast<const uint4*>(x + (size_t)(row0 + r) * K) + c), v);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = 0.f;
      }
      float4* dst = reinterpret_cast<float4*>(xs + (size_t)r * K + (size_t)c * N);
#pragma unroll
      for (int j = 0; j < N; j += 4) dst[j >> 2] = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
  } else {
    for (int idx = threadIdx.x; idx < rows_per_cta * K; idx += blockDim.x) {
      const int r = idx / K;
      xs[idx] = r < live ? load_as_float(x + (size_t)(row0 + r) * K + (idx - r * K)) : 0.f;
    }
  }
  __syncthreads();
  const int e0 = (blockIdx.y * ROUTE_WARPS + warp) * E;
  if (e0 >= experts) return;
  const float* w[E];
#pragma unroll
  for (int i = 0; i < E; ++i) w[i] = router + (size_t)min(e0 + i, experts - 1) * K;   // past the end: the last one again, dropped
  float acc[E][ROUTE_ROWS];
#pragma unroll
  for (int i = 0; i < E; ++i)
#pragma unroll
    for (int r = 0; r < ROUTE_ROWS; ++r) acc[i][r] = 0.f;
  if (wide) {
#pragma unroll 2
    for (int k = lane * 4; k < K; k += 128) {
      float4 wv[E];
#pragma unroll
      for (int i = 0; i < E; ++i) wv[i] = __ldg(reinterpret_cast<const float4*>(w[i] + k));
#pragma unroll
      for (int r = 0; r < ROUTE_ROWS; ++r) {
        if (r < rows_per_cta) {
          const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)r * K + k);
#pragma unroll
          for (int i = 0; i < E; ++i)
            acc[i][r] = fmaf(wv[i].w, xv.w, fmaf(wv[i].z, xv.z, fmaf(wv[i].y, xv.y, fmaf(wv[i].x, xv.x, acc[i][r]))));
        }
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      float wv[E];
#pragma unroll
      for (int i = 0; i < E; ++i) wv[i] = __ldg(w[i] + k);
#pragma unroll
      for (int r = 0; r < ROUTE_ROWS; ++r) {
        if (r < rows_per_cta) {
          const float xv = xs[(size_t)r * K + k];
#pragma unroll
          for (int i = 0; i < E; ++i) acc[i][r] = fmaf(wv[i], xv, acc[i][r]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < E; ++i) {
#pragma unroll
    for (int r = 0; r < ROUTE_ROWS; ++r) {
      if (r < live) {
        const float sum = warp_sum(acc[i][r]);
        if (lane == 0 && e0 + i < experts) logits[(size_t)(row0 + r) * experts + e0 + i] = sum;
      }
    }
  }
}

// The choice, one warp per row, from the row's logits.
__global__ void __launch_bounds__(CHOOSE_WARPS * 32)
choose_experts_kernel(const float* logits, const float* __restrict__ correction, int* chosen, float* weights, int rows,
                      int experts, int top, int groups, int keep, int group_top, int sigmoid_scores, int renormalise,
                      float renorm_eps) {
  pdl_trigger();
  extern __shared__ __align__(16) float shared[];      // per warp: [experts] scores, [experts] choice scores, [groups]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * CHOOSE_WARPS + warp;
  float* score = shared + (size_t)warp * (2 * experts + groups);
  float* choice = score + experts;
  float* group_score = choice + experts;
  pdl_wait();
  if (row >= rows) return;
  if (sigmoid_scores) {
    for (int e = lane; e < experts; e += 32) score[e] = 1.f / (1.f + expf(-__ldcg(logits + (size_t)row * experts + e)));
  } else {
    float top_logit = -INFINITY;
    for (int e = lane; e < experts; e += 32) {
      const float z = __ldcg(logits + (size_t)row * experts + e);
      score[e] = z;
      top_logit = fmaxf(top_logit, z);
    }
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
      // the sum of the group's `group_top` largest choice scores (1: its largest), taken largest first
      float total = 0.f, bound = INFINITY;
      int bound_at = -1;
      for (int n = 0; n < group_top && n < size; ++n) {
        float best = -INFINITY;
        int best_at = size;
        for (int j = 0; j < size; ++j) {
          const float c = choice[g * size + j];
          const bool below = c < bound || (c == bound && j > bound_at);      // not one of those already taken
          if (below && c > best) {
            best = c;
            best_at = j;
          }
        }
        total = n == 0 ? best : total + best;
        bound = best;
        bound_at = best_at;
      }
      group_score[g] = total;
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
      if (c > best) {      // ascending e: of equal scores the lowest index stays
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
    for (int t = 0; t < top; ++t) weights[(size_t)row * top + t] /= (weight_sum + renorm_eps);
}


// R dot products at once of weight rows with one float32 vector in shared memory, split over the lanes
// of a warp: with `wide`, lane l takes the 16-byte pieces l, l + 32, .. of every row (R loads in flight
// per step, the vector's piece read once for all rows); else single entries.  Every lane gets the
// sums; the order of a sum's additions depends on K only.
template <int R, typename T>
__device__ __forceinline__ void warp_dots(const T* const (&rows)[R], const float* x, int K, int lane, bool wide,
                                          float (&out)[R]) {
  constexpr int N = 16 / sizeof(T);
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  if (wide) {
    for (int k = lane * N; k < K; k += 32 * N) {
      uint4 raw[R];
#pragma unroll
      for (int r = 0; r < R; ++r) raw[r] = __ldg(reinterpret_cast<const uint4*>(rows[r] + k));
      float xv[N];
#pragma unroll
      for (int j = 0; j < N; j += 4) {
        const float4 piece = *reinterpret_cast<const float4*>(x + k + j);
        xv[j] = piece.x;
        xv[j + 1] = piece.y;
        xv[j + 2] = piece.z;
        xv[j + 3] = piece.w;
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float wv[N];
        unpack(raw[r], wv);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[r] = fmaf(wv[j], xv[j], acc[r]);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) {
      const float xv = x[k];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = fmaf(load_as_float(rows[r] + k), xv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) out[r] = warp_sum(acc[r]);
}

constexpr int EXPERT_WARPS = 8;
constexpr int PER_WARP = 4;            // outputs a warp computes at once
constexpr int HIDDEN_PER_CTA = EXPERT_WARPS * PER_WARP;
constexpr int DOWN_PER_CTA = EXPERT_WARPS * PER_WARP;

// gate_up: [experts][2 * ff][K] with rows in blocks of `block` gate rows followed by the `block` up rows
// of the same outputs (block == ff: all gate rows first).
template <typename T>
__global__ void __launch_bounds__(EXPERT_WARPS * 32)
expert_hidden_kernel(const T* x, const int* chosen, const T* __restrict__ gate_up, T* hidden, int K, int ff, int top,
                     int block, int act, int wide) {
  pdl_trigger();
  extern __shared__ __align__(16) float xs[];      // [K]
  const int pair = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  const int row = pair / top;
  const int expert = chosen[pair];
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = load_as_float(x + (size_t)row * K + k);
  __syncthreads();
  const T* w = gate_up + (size_t)expert * 2 * ff * K;
  const int j0 = blockIdx.y * HIDDEN_PER_CTA + warp * PER_WARP;
  if (j0 >= ff) return;
  const T* rows[2 * PER_WARP];
#pragma unroll
  for (int i = 0; i < PER_WARP; ++i) {
    const int j = min(j0 + i, ff - 1);          // a row past the end repeats the last one; its result is dropped
    const int gate_row = (j / block) * 2 * block + j % block;
    rows[i] = w + (size_t)gate_row * K;
    rows[PER_WARP + i] = w + (size_t)(gate_row + block) * K;
  }
  float sums[2 * PER_WARP];
  warp_dots<2 * PER_WARP, T>(rows, xs, K, lane, wide != 0, sums);
  if (lane < PER_WARP && j0 + lane < ff) {
    float gate = 0.f, up = 0.f;
#pragma unroll
    for (int i = 0; i < PER_WARP; ++i)
      if (i == lane) {
        gate = sums[i];
        up = sums[PER_WARP + i];
      }
    float value;
    if (act == 1) {
      value = 0.5f * gate * (1.f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate))) * up;
    } else {
      value = gate / (1.f + expf(-gate)) * up;
    }
    hidden[(size_t)pair * ff + j0 + lane] = from_float<T>(value);
  }
}

// down: [experts][N][ff]
template <typename T>
__global__ void __launch_bounds__(EXPERT_WARPS * 32)
expert_down_kernel(const T* hidden, const int* chosen, const float* weights, const T* __restrict__ down, float* out, int N,
                   int ff, int top, int wide) {
  pdl_trigger();
  extern __shared__ __align__(16) float hs[];      // [top][ff], each row padded to a multiple of four
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pitch = (ff + 3) & ~3;
  pdl_wait();
  for (int idx = threadIdx.x; idx < top * ff; idx += blockDim.x) {
    const int t = idx / ff, k = idx - t * ff;
    hs[(size_t)t * pitch + k] = load_as_float(hidden + (size_t)row * top * ff + idx);
  }
  __syncthreads();
  const int n0 = blockIdx.y * DOWN_PER_CTA + warp * PER_WARP;
  if (n0 >= N) return;
  float total[PER_WARP];
#pragma unroll
  for (int i = 0; i < PER_WARP; ++i) total[i] = 0.f;
  for (int t = 0; t < top; ++t) {
    const int expert = chosen[(size_t)row * top + t];
    const T* rows[PER_WARP];
#pragma unroll
    for (int i = 0; i < PER_WARP; ++i) rows[i] = down + ((size_t)expert * N + min(n0 + i, N - 1)) * ff;
    float y[PER_WARP];
    warp_dots<PER_WARP, T>(rows, hs + (size_t)t * pitch, ff, lane, wide != 0, y);
    const float weight = weights[(size_t)row * top + t];
#pragma unroll
    for (int i = 0; i < PER_WARP; ++i) total[i] = fmaf(weight, y[i], total[i]);
  }
  if (lane < PER_WARP && n0 + lane < N) {
    float value = 0.f;
#pragma unroll
    for (int i = 0; i < PER_WARP; ++i)
      if (i == lane) value = total[i];
    out[(size_t)row * N + n0 + lane] = value;
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
// logits: float32 [rows, experts] (scratch); chosen: int32 [rows, top]; weights: float32 [rows, top].
MLR_EXPORT int mlr_route_experts(const void* x, const float* router, const float* correction, float* logits, int* chosen,
                                 float* weights, int rows, int K, int experts, int top, int groups, int keep, int group_top,
                                 int sigmoid_scores, int renormalise, float renorm_eps, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || K <= 0 || experts <= 0 || top <= 0 || groups <= 0 || keep <= 0 || keep > groups || experts % groups != 0 ||
      group_top <= 0 ||
      top > keep * (experts / groups))
    return MLR_BAD_SIZE;
  // as many rows per CTA as there are and fit (each router entry is then loaded once for all of them)
  int rows_per_cta = 1;
  while (rows_per_cta < ROUTE_ROWS && rows_per_cta < rows) rows_per_cta *= 2;
  auto bytes = [&](int r) { return sizeof(float) * (size_t)r * (size_t)K; };
  while (rows_per_cta > 1 && bytes(rows_per_cta) > 64 * 1024) rows_per_cta /= 2;
  const size_t shared = bytes(rows_per_cta);
  const size_t choose_shared = sizeof(float) * CHOOSE_WARPS * (2 * (size_t)experts + groups);
  if (shared > 200 * 1024 || choose_shared > 200 * 1024) return MLR_TOO_LARGE;
  const int wide = K % 4 == 0 && ((uintptr_t)router & 15) == 0;
  const bool many = rows > 8 * ROUTE_ROWS;
  const int per_cta = ROUTE_WARPS * (many ? 4 : 1);
  const dim3 grid((rows + rows_per_cta - 1) / rows_per_cta, (experts + per_cta - 1) / per_cta);
  auto launch = [&](auto kernel, auto* typed) -> int {
    const int x_wide = K % (16 / (int)sizeof(*typed)) == 0 && ((uintptr_t)x & 15) == 0;
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, grid, dim3(ROUTE_WARPS * 32), shared, stream, typed, router, logits, rows, K, experts, rows_per_cta,
                  wide, x_wide);
    return launch_status();
  };
  int status = MLR_BAD_DTYPE;
  if (dtype == MLR_F32)
    status = many ? launch(router_logits_kernel<float, 4>, (const float*)x) : launch(router_logits_kernel<float, 1>, (const float*)x);
  if (dtype == MLR_BF16)
    status = many ? launch(router_logits_kernel<bf16, 4>, (const bf16*)x) : launch(router_logits_kernel<bf16, 1>, (const bf16*)x);
  if (status != MLR_OK) return status;
  if (choose_shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(choose_experts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(choose_experts_kernel, dim3((rows + CHOOSE_WARPS - 1) / CHOOSE_WARPS), dim3(CHOOSE_WARPS * 32), choose_shared,
                stream, (const float*)logits, correction, chosen, weights, rows, experts, top, groups, keep, group_top,
                sigmoid_scores, renormalise, renorm_eps);
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
  const size_t shared = sizeof(float) * (size_t)top * ((ff + 3) & ~3);
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
