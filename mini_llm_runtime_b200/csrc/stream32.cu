// Kernels of decoders whose residual stream is 32-bit floats and whose sublayers are wrapped in
// layer norms on both sides ("sandwich" arrangement).
//
// mlr_embedding_rows32     float32 rows table[ids] * scale of a table in the compute dtype.
// mlr_layer_norm_step      one pass over each row of the stream x that does, in this order, whatever
//                          its arguments ask for:
//                            x += LN(delta; dw, db)      the sublayer output that was still to be added,
//                                                        normalised on its way into the stream
//                            x += offset                 one learned vector for all rows
//                            out = LN(x; w, b)           the input of the next sublayer, compute dtype
//                          LN(v; w, b) = (v - mean) / sqrt(var + eps) * w + b with var the mean of the
//                          squared deviations; all sums in float32 in an order fixed by the width.
// mlr_rms_norm_step        the same pass for sublayers that are normalised on their way into the stream by
//                          an RMS norm (no centering, no bias): x += delta / rms(delta) * dw, then
//                          out = x / rms(x) * w, or the rows of x as they are in the compute dtype when
//                          no w is given (the input of a sublayer that reads the stream itself).
// mlr_normed_mean          out = factor * (a / rms(a) * wa + b / rms(b) * wb) for two float32 inputs.
// mlr_clamped_gate         y = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit) and
//                          u = clamp(up, -limit, limit), on rows of gate/up blocks.
// mlr_scale_inplace        x *= s for float32 x (logit scale).
#include "common.cuh"

#include <type_traits>

namespace mlr {

template <typename T>
__global__ void __launch_bounds__(256)
embedding_rows32_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out, int width,
                        int vocab, float scale) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  id = min(max(id, 0), vocab - 1);
  const T* src = table + (size_t)id * width;
  float* dst = out + (size_t)row * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) dst[d] = to_float(src[d]) * scale;
}

// mean and 1/sqrt(var + eps) of `width` floats in shared memory; every thread gets both.
__device__ __forceinline__ void row_statistics(const float* values, int width, float eps, float* scratch, float* mean_out,
                                               float* rstd_out) {
  float sum = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) sum += values[d];
  const float mean = block_sum(sum, scratch) / (float)width;
  float sq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float c = values[d] - mean;
    sq = fmaf(c, c, sq);
  }
  const float variance = block_sum(sq, scratch) / (float)width;
  *mean_out = mean;
  *rstd_out = 1.f / sqrtf(variance + eps);
}

template <typename T>
__global__ void __launch_bounds__(256)
layer_norm_step_kernel(float* x, const float* delta, const float* __restrict__ dw, const float* __restrict__ db,
                       const float* __restrict__ offset, const float* __restrict__ w, const float* __restrict__ b,
                       T* __restrict__ out, int width, float eps) {
  pdl_trigger();
  extern __shared__ float staged[];      // [width] + 32
  float* scratch = staged + width;
  const size_t base = (size_t)blockIdx.x * width;
  pdl_wait();
  float mean, rstd;
  if (delta != nullptr) {
    for (int d = threadIdx.x; d < width; d += blockDim.x) staged[d] = delta[base + d];
    __syncthreads();
    row_statistics(staged, width, eps, scratch, &mean, &rstd);
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      float v = x[base + d] + fmaf((staged[d] - mean) * rstd, dw[d], db[d]);
      if (offset != nullptr) v += offset[d];
      staged[d] = v;
      x[base + d] = v;
    }
  } else {
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      float v = x[base + d];
      if (offset != nullptr) {
        v += offset[d];
        x[base + d] = v;
      }
      staged[d] = v;
    }
  }
  if (out == nullptr) return;
  __syncthreads();
  row_statistics(staged, width, eps, scratch, &mean, &rstd);
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    out[base + d] = from_float<T>(fmaf((staged[d] - mean) * rstd, w[d], b[d]));
}

// The same with one warp per row and the row in registers (width a multiple of 4, at most CH * 128):
// no barriers, 16-byte accesses.  Lane l holds the float4 pieces l, l + 32, ..
__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(bf16* dst, float4 v) {
  uint2 packed;
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  packed.x = *reinterpret_cast<uint32_t*>(&lo);
  packed.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = packed;
}

template <int CH>
__device__ __forceinline__ void warp_row_statistics(const float4 (&v)[CH], int pieces, int lane, int width, float eps,
                                                    float* mean_out, float* rstd_out) {
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j)
    if (lane + 32 * j < pieces) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  const float mean = warp_sum(sum) / (float)width;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j)
    if (lane + 32 * j < pieces) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      sq += fmaf(a, a, b * b) + fmaf(c, c, d * d);
    }
  *mean_out = mean;
  *rstd_out = 1.f / sqrtf(warp_sum(sq) / (float)width + eps);
}

__device__ __forceinline__ float4 normalised(float4 v, float mean, float rstd, float4 w, float4 b) {
  return make_float4(fmaf((v.x - mean) * rstd, w.x, b.x), fmaf((v.y - mean) * rstd, w.y, b.y),
                     fmaf((v.z - mean) * rstd, w.z, b.z), fmaf((v.w - mean) * rstd, w.w, b.w));
}

template <typename T, int CH>
__global__ void __launch_bounds__(128)
layer_norm_step_warp_kernel(float* x, const float* delta, const float* __restrict__ dw, const float* __restrict__ db,
                            const float* __restrict__ offset, const float* __restrict__ w, const float* __restrict__ b,
                            T* __restrict__ out, int rows, int width, float eps) {
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int pieces = width >> 2;
  pdl_wait();
  if (row >= rows) return;
  const size_t base = (size_t)row * width;
  const float4* x4 = reinterpret_cast<const float4*>(x + base);

  float4 v[CH];
  float mean, rstd;
  if (delta != nullptr) {
    const float4* d4 = reinterpret_cast<const float4*>(delta + base);
#pragma unroll
    for (int j = 0; j < CH; ++j)
      if (lane + 32 * j < pieces) v[j] = __ldcg(d4 + lane + 32 * j);
    warp_row_statistics<CH>(v, pieces, lane, width, eps, &mean, &rstd);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int c = lane + 32 * j;
      if (c < pieces) {
        const float4 add = normalised(v[j], mean, rstd, reinterpret_cast<const float4*>(dw)[c],
                                      reinterpret_cast<const float4*>(db)[c]);
        float4 now = __ldcg(x4 + c);
        now.x += add.x; now.y += add.y; now.z += add.z; now.w += add.w;
        if (offset != nullptr) {
          const float4 o = reinterpret_cast<const float4*>(offset)[c];
          now.x += o.x; now.y += o.y; now.z += o.z; now.w += o.w;
        }
        v[j] = now;
        store4(x + base + 4 * c, now);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const int c = lane + 32 * j;
      if (c < pieces) {
        float4 now = __ldcg(x4 + c);
        if (offset != nullptr) {
          const float4 o = reinterpret_cast<const float4*>(offset)[c];
          now.x += o.x; now.y += o.y; now.z += o.z; now.w += o.w;
          store4(x + base + 4 * c, now);
        }
        v[j] = now;
      }
    }
  }
  if (out == nullptr) return;
  warp_row_statistics<CH>(v, pieces, lane, width, eps, &mean, &rstd);
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = lane + 32 * j;
    if (c < pieces)
      store4(out + base + 4 * c, normalised(v[j], mean, rstd, reinterpret_cast<const float4*>(w)[c],
                                            reinterpret_cast<const float4*>(b)[c]));
  }
}

// Steps of few rows (decoding): one CTA of THREADS threads (128, or more for rows wider than 2,048)
// per row, at most four float4 pieces per thread, and every operand (the row, what is added, the
// norms' vectors) asked for before the first is used, so that the pass costs one trip to memory
// instead of one per phase.
template <int THREADS>
__device__ __forceinline__ float block_sum_of(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = (scratch[0] + scratch[1]) + (scratch[2] + scratch[3]);
#pragma unroll
  for (int i = 4; i < THREADS / 32; i += 4) total += (scratch[i] + scratch[i + 1]) + (scratch[i + 2] + scratch[i + 3]);
  return total;
}

// EARLY: the norms' vectors are asked for before the wait and kept in registers (steps of few rows: one
// trip to memory); otherwise they are read where they are used (many rows: more blocks per SM).
template <typename T, int THREADS, bool EARLY>
__global__ void __launch_bounds__(THREADS)
layer_norm_step_row_kernel(float* x, const float* delta, const float* __restrict__ dw, const float* __restrict__ db,
                           const float* __restrict__ offset, const float* __restrict__ w, const float* __restrict__ b,
                           T* __restrict__ out, int width, float eps) {
  pdl_trigger();
  __shared__ float scratch[THREADS / 32];
  constexpr int CH = 4;
  const int pieces = width >> 2;
  const size_t base = (size_t)blockIdx.x * width;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 dwv[CH], dbv[CH], ov[CH], wv[CH], bv[CH], dv[CH], xv[CH];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    const bool in = c < pieces;
    if (EARLY) {
      dwv[j] = in && delta != nullptr ? reinterpret_cast<const float4*>(dw)[c] : zero;
      dbv[j] = in && delta != nullptr ? reinterpret_cast<const float4*>(db)[c] : zero;
      ov[j] = in && offset != nullptr ? reinterpret_cast<const float4*>(offset)[c] : zero;
      wv[j] = in && out != nullptr ? reinterpret_cast<const float4*>(w)[c] : zero;
      bv[j] = in && out != nullptr ? reinterpret_cast<const float4*>(b)[c] : zero;
    }
  }
  // piece j of a vector: from the registers, or from memory now
  auto piece = [&](const float4 (&kept)[CH], const float* vector, int j) -> float4 {
    if (EARLY) return kept[j];
    const int c = threadIdx.x + THREADS * j;
    return c < pieces ? reinterpret_cast<const float4*>(vector)[c] : zero;
  };
  pdl_wait();
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    const bool in = c < pieces;
    dv[j] = in && delta != nullptr ? __ldcg(reinterpret_cast<const float4*>(delta + base) + c) : zero;
    xv[j] = in ? __ldcg(reinterpret_cast<const float4*>(x + base) + c) : zero;
  }
  if (delta != nullptr) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) sum += (dv[j].x + dv[j].y) + (dv[j].z + dv[j].w);      // pieces past the row are zeros
    const float mean = block_sum_of<THREADS>(sum, scratch) / (float)width;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j)
      if (threadIdx.x + THREADS * j < pieces) {
        const float a = dv[j].x - mean, bb = dv[j].y - mean, c = dv[j].z - mean, d = dv[j].w - mean;
        sq += fmaf(a, a, bb * bb) + fmaf(c, c, d * d);
      }
    const float rstd = 1.f / sqrtf(block_sum_of<THREADS>(sq, scratch) / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const float4 add = normalised(dv[j], mean, rstd, piece(dwv, dw, j), piece(dbv, db, j));
      xv[j].x += add.x; xv[j].y += add.y; xv[j].z += add.z; xv[j].w += add.w;
    }
  }
  if (offset != nullptr) {
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      const float4 o = piece(ov, offset, j);
      xv[j].x += o.x; xv[j].y += o.y; xv[j].z += o.z; xv[j].w += o.w;
    }
  }
  if (delta != nullptr || offset != nullptr) {
#pragma unroll
    for (int j = 0; j < CH; ++j)
      if (threadIdx.x + THREADS * j < pieces) store4(x + base + 4 * (threadIdx.x + THREADS * j), xv[j]);
  }
  if (out == nullptr) return;
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j)
    if (threadIdx.x + THREADS * j < pieces) sum += (xv[j].x + xv[j].y) + (xv[j].z + xv[j].w);
  const float mean = block_sum_of<THREADS>(sum, scratch) / (float)width;
  float sq = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j)
    if (threadIdx.x + THREADS * j < pieces) {
      const float a = xv[j].x - mean, bb = xv[j].y - mean, c = xv[j].z - mean, d = xv[j].w - mean;
      sq += fmaf(a, a, bb * bb) + fmaf(c, c, d * d);
    }
  const float rstd = 1.f / sqrtf(block_sum_of<THREADS>(sq, scratch) / (float)width + eps);
#pragma unroll
  for (int j = 0; j < CH; ++j)
    if (threadIdx.x + THREADS * j < pieces)
      store4(out + base + 4 * (threadIdx.x + THREADS * j), normalised(xv[j], mean, rstd, piece(wv, w, j), piece(bv, b, j)));
}

// 1 / sqrt(mean(v^2) + eps) of `width` floats in shared memory; every thread gets it.
__device__ __forceinline__ float row_inverse_rms(const float* values, int width, float eps, float* scratch) {
  float sq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) sq = fmaf(values[d], values[d], sq);
  return 1.f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
}

template <typename T>
__global__ void __launch_bounds__(256)
rms_norm_step_kernel(float* x, const float* delta, const float* __restrict__ dw, const float* __restrict__ w,
                     T* __restrict__ out, int width, float eps) {
  pdl_trigger();
  extern __shared__ float staged[];      // [width] + 32
  float* scratch = staged + width;
  const size_t base = (size_t)blockIdx.x * width;
  pdl_wait();
  if (delta != nullptr) {
    for (int d = threadIdx.x; d < width; d += blockDim.x) staged[d] = __ldcg(delta + base + d);
    __syncthreads();
    const float rstd = row_inverse_rms(staged, width, eps, scratch);
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      const float v = __ldcg(x + base + d) + staged[d] * rstd * dw[d];
      staged[d] = v;
      x[base + d] = v;
    }
  } else {
    for (int d = threadIdx.x; d < width; d += blockDim.x) staged[d] = __ldcg(x + base + d);
  }
  if (out == nullptr) return;
  if (w == nullptr) {
    for (int d = threadIdx.x; d < width; d += blockDim.x) out[base + d] = from_float<T>(staged[d]);      // own entries
    return;
  }
  __syncthreads();
  const float rstd = row_inverse_rms(staged, width, eps, scratch);
  for (int d = threadIdx.x; d < width; d += blockDim.x) out[base + d] = from_float<T>(staged[d] * rstd * w[d]);
}

__global__ void __launch_bounds__(256)
normed_mean_kernel(const float* a, const float* __restrict__ wa, const float* b, const float* __restrict__ wb,
                   float* __restrict__ out, int width, float eps, float factor) {
  pdl_trigger();
  extern __shared__ float staged[];      // [2 * width] + 32
  float* second = staged + width;
  float* scratch = second + width;
  const size_t base = (size_t)blockIdx.x * width;
  pdl_wait();
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    staged[d] = __ldcg(a + base + d);
    second[d] = __ldcg(b + base + d);
  }
  __syncthreads();
  const float ra = row_inverse_rms(staged, width, eps, scratch);
  const float rb = row_inverse_rms(second, width, eps, scratch);
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    out[base + d] = factor * (staged[d] * ra * wa[d] + second[d] * rb * wb[d]);
}

// The same two for steps of few rows (decoding): one CTA of THREADS threads per row, at most four float4
// pieces per thread, every operand asked for before the first is used (one trip to memory).
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
rms_norm_step_row_kernel(float* x, const float* delta, const float* __restrict__ dw, const float* __restrict__ w,
                         T* __restrict__ out, int width, float eps) {
  pdl_trigger();
  __shared__ float scratch[THREADS / 32];
  constexpr int CH = 4;
  const int pieces = width >> 2;
  const size_t base = (size_t)blockIdx.x * width;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 dwv[CH], wv[CH], dv[CH], xv[CH];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    const bool in = c < pieces;
    dwv[j] = in && delta != nullptr ? reinterpret_cast<const float4*>(dw)[c] : zero;
    wv[j] = in && out != nullptr && w != nullptr ? reinterpret_cast<const float4*>(w)[c] : zero;
  }
  pdl_wait();
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    const bool in = c < pieces;
    dv[j] = in && delta != nullptr ? __ldcg(reinterpret_cast<const float4*>(delta + base) + c) : zero;
    xv[j] = in ? __ldcg(reinterpret_cast<const float4*>(x + base) + c) : zero;
  }
  if (delta != nullptr) {
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) sq += fmaf(dv[j].x, dv[j].x, dv[j].y * dv[j].y) + fmaf(dv[j].z, dv[j].z, dv[j].w * dv[j].w);
    const float rstd = 1.f / sqrtf(block_sum_of<THREADS>(sq, scratch) / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CH; ++j) {
      xv[j].x += dv[j].x * rstd * dwv[j].x; xv[j].y += dv[j].y * rstd * dwv[j].y;
      xv[j].z += dv[j].z * rstd * dwv[j].z; xv[j].w += dv[j].w * rstd * dwv[j].w;
      if (threadIdx.x + THREADS * j < pieces) store4(x + base + 4 * (threadIdx.x + THREADS * j), xv[j]);
    }
  }
  if (out == nullptr) return;
  float rstd = 1.f;
  if (w != nullptr) {
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < CH; ++j) sq += fmaf(xv[j].x, xv[j].x, xv[j].y * xv[j].y) + fmaf(xv[j].z, xv[j].z, xv[j].w * xv[j].w);
    rstd = 1.f / sqrtf(block_sum_of<THREADS>(sq, scratch) / (float)width + eps);
  }
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    if (threadIdx.x + THREADS * j >= pieces) continue;
    float4 o = xv[j];
    if (w != nullptr) o = make_float4(o.x * rstd * wv[j].x, o.y * rstd * wv[j].y, o.z * rstd * wv[j].z, o.w * rstd * wv[j].w);
    store4(out + base + 4 * (threadIdx.x + THREADS * j), o);
  }
}

template <int THREADS>
__global__ void __launch_bounds__(THREADS)
normed_mean_row_kernel(const float* a, const float* __restrict__ wa, const float* b, const float* __restrict__ wb,
                       float* __restrict__ out, int width, float eps, float factor) {
  pdl_trigger();
  __shared__ float scratch[THREADS / 32];
  constexpr int CH = 4;
  const int pieces = width >> 2;
  const size_t base = (size_t)blockIdx.x * width;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 wav[CH], wbv[CH], av[CH], bv[CH];
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    wav[j] = c < pieces ? reinterpret_cast<const float4*>(wa)[c] : zero;
    wbv[j] = c < pieces ? reinterpret_cast<const float4*>(wb)[c] : zero;
  }
  pdl_wait();
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    av[j] = c < pieces ? __ldcg(reinterpret_cast<const float4*>(a + base) + c) : zero;
    bv[j] = c < pieces ? __ldcg(reinterpret_cast<const float4*>(b + base) + c) : zero;
  }
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    sa += fmaf(av[j].x, av[j].x, av[j].y * av[j].y) + fmaf(av[j].z, av[j].z, av[j].w * av[j].w);
    sb += fmaf(bv[j].x, bv[j].x, bv[j].y * bv[j].y) + fmaf(bv[j].z, bv[j].z, bv[j].w * bv[j].w);
  }
  const float ra = 1.f / sqrtf(block_sum_of<THREADS>(sa, scratch) / (float)width + eps);
  const float rb = 1.f / sqrtf(block_sum_of<THREADS>(sb, scratch) / (float)width + eps);
#pragma unroll
  for (int j = 0; j < CH; ++j) {
    const int c = threadIdx.x + THREADS * j;
    if (c >= pieces) continue;
    store4(out + base + 4 * c, make_float4(factor * (av[j].x * ra * wav[j].x + bv[j].x * rb * wbv[j].x),
                                           factor * (av[j].y * ra * wav[j].y + bv[j].y * rb * wbv[j].y),
                                           factor * (av[j].z * ra * wav[j].z + bv[j].z * rb * wbv[j].z),
                                           factor * (av[j].w * ra * wav[j].w + bv[j].w * rb * wbv[j].w)));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
clamped_gate_kernel(const T* x, T* __restrict__ out, long long rows, int inner, int block, float limit, float slope) {
  pdl_trigger();
  pdl_wait();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= rows * inner) return;
  const long long row = index / inner;
  const int column = (int)(index - row * inner);
  const int group = column / block, within = column - group * block;
  const T* source = x + row * 2 * inner + (size_t)group * 2 * block;
  const float g = fminf(to_float(source[within]), limit);
  const float u = fminf(fmaxf(to_float(source[block + within]), -limit), limit);
  out[index] = from_float<T>(g / (1.f + expf(-slope * g)) * (u + 1.f));
}

__global__ void __launch_bounds__(256) scale_inplace_kernel(float* x, long long count, float factor) {
  pdl_trigger();
  pdl_wait();
  const long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (index < count) x[index] *= factor;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

MLR_EXPORT int mlr_embedding_rows32(const int* ids, const void* table, float* out, int rows, int width, int vocab,
                                    float scale, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0 || vocab <= 0) return MLR_BAD_SIZE;
  if (dtype == MLR_F32)
    launch_kernel(embedding_rows32_kernel<float>, dim3(rows), dim3(256), 0, stream, ids, (const float*)table, out, width, vocab, scale);
  else if (dtype == MLR_BF16)
    launch_kernel(embedding_rows32_kernel<bf16>, dim3(rows), dim3(256), 0, stream, ids, (const bf16*)table, out, width, vocab, scale);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

// x: float32 [rows, width], updated in place when delta or offset is given.  delta: float32
// [rows, width] or null (then dw, db are not read).  offset: float32 [width] or null.  out: compute
// dtype [rows, width] or null (then w, b are not read).
MLR_EXPORT int mlr_layer_norm_step(float* x, const float* delta, const float* dw, const float* db, const float* offset,
                                   const float* w, const float* b, void* out, int rows, int width, float eps,
                                   int out_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0) return MLR_BAD_SIZE;
  if ((delta != nullptr && (dw == nullptr || db == nullptr)) || (out != nullptr && (w == nullptr || b == nullptr)))
    return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * ((size_t)width + 32);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool pieces_fit = width % 4 == 0 && aligned(x) && aligned(delta) && aligned(dw) && aligned(db) && aligned(offset) &&
                          aligned(w) && aligned(b) && aligned(out);
  if (pieces_fit && width <= 8192 && (rows <= 64 || width > 2048)) {
    // few rows, or rows too wide for a warp's registers: a CTA per row, all operands asked for at once
    auto launch_row = [&](auto kernel, int threads, auto* typed_out) -> int {
      launch_kernel(kernel, dim3(rows), dim3(threads), 0, stream, x, delta, dw, db, offset, w, b, typed_out, width, eps);
      return launch_status();
    };
    auto launch_typed = [&](auto* typed_out) -> int {
      using T = std::remove_pointer_t<decltype(typed_out)>;
      if (rows <= 64) {
        if (width <= 2048) return launch_row(layer_norm_step_row_kernel<T, 128, true>, 128, typed_out);
        if (width <= 4096) return launch_row(layer_norm_step_row_kernel<T, 256, true>, 256, typed_out);
        return launch_row(layer_norm_step_row_kernel<T, 512, true>, 512, typed_out);
      }
      if (width <= 4096) return launch_row(layer_norm_step_row_kernel<T, 256, false>, 256, typed_out);
      return launch_row(layer_norm_step_row_kernel<T, 512, false>, 512, typed_out);
    };
    if (out_dtype == MLR_F32) return launch_typed((float*)out);
    if (out_dtype == MLR_BF16) return launch_typed((bf16*)out);
    return MLR_BAD_DTYPE;
  }
  if (pieces_fit && width <= 2048) {
    // the row fits a warp's registers
    auto launch_warp = [&](auto kernel, auto* typed_out) -> int {
      launch_kernel(kernel, dim3((rows + 3) / 4), dim3(128), 0, stream, x, delta, dw, db, offset, w, b, typed_out, rows,
                    width, eps);
      return launch_status();
    };
    if (out_dtype == MLR_F32) {
      if (width <= 512) return launch_warp(layer_norm_step_warp_kernel<float, 4>, (float*)out);
      if (width <= 1024) return launch_warp(layer_norm_step_warp_kernel<float, 8>, (float*)out);
      return launch_warp(layer_norm_step_warp_kernel<float, 16>, (float*)out);
    }
    if (out_dtype == MLR_BF16) {
      if (width <= 512) return launch_warp(layer_norm_step_warp_kernel<bf16, 4>, (bf16*)out);
      if (width <= 1024) return launch_warp(layer_norm_step_warp_kernel<bf16, 8>, (bf16*)out);
      return launch_warp(layer_norm_step_warp_kernel<bf16, 16>, (bf16*)out);
    }
    return MLR_BAD_DTYPE;
  }
  auto launch = [&](auto kernel, auto* typed_out) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, dim3(rows), dim3(256), shared, stream, x, delta, dw, db, offset, w, b, typed_out, width, eps);
    return launch_status();
  };
  if (out_dtype == MLR_F32) return launch(layer_norm_step_kernel<float>, (float*)out);
  if (out_dtype == MLR_BF16) return launch(layer_norm_step_kernel<bf16>, (bf16*)out);
  return MLR_BAD_DTYPE;
}

// x: float32 [rows, width], updated in place when delta is given.  delta: float32 [rows, width] or null
// (then dw is not read); dw, w: float32 [width]; out: [rows, width] in out_dtype or null.  With out and no
// w, out receives the rows of x (after the add) as they are.
MLR_EXPORT int mlr_rms_norm_step(float* x, const float* delta, const float* dw, const float* w, void* out, int rows,
                                 int width, float eps, int out_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0 || (delta != nullptr && dw == nullptr)) return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * ((size_t)width + 32);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool few = rows <= 64 && width % 4 == 0 && width <= 8192 && aligned(x) && aligned(delta) && aligned(dw) && aligned(w) &&
                   aligned(out);
  auto launch = [&](auto kernel, auto* typed_out) -> int {
    using T = std::remove_pointer_t<decltype(typed_out)>;
    if (few) {
      if (width <= 2048)
        launch_kernel(rms_norm_step_row_kernel<T, 128>, dim3(rows), dim3(128), 0, stream, x, delta, dw, w, typed_out, width, eps);
      else if (width <= 4096)
        launch_kernel(rms_norm_step_row_kernel<T, 256>, dim3(rows), dim3(256), 0, stream, x, delta, dw, w, typed_out, width, eps);
      else
        launch_kernel(rms_norm_step_row_kernel<T, 512>, dim3(rows), dim3(512), 0, stream, x, delta, dw, w, typed_out, width, eps);
      return launch_status();
    }
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, dim3(rows), dim3(256), shared, stream, x, delta, dw, w, typed_out, width, eps);
    return launch_status();
  };
  if (out_dtype == MLR_F32) return launch(rms_norm_step_kernel<float>, (float*)out);
  if (out_dtype == MLR_BF16) return launch(rms_norm_step_kernel<bf16>, (bf16*)out);
  return MLR_BAD_DTYPE;
}

// a, b, out: float32 [rows, width]; wa, wb: float32 [width].
MLR_EXPORT int mlr_normed_mean(const float* a, const float* wa, const float* b, const float* wb, float* out, int rows,
                               int width, float eps, float factor, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0) return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * (2 * (size_t)width + 32);
  if (shared > 200 * 1024) return MLR_TOO_LARGE;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (rows <= 64 && width % 4 == 0 && width <= 8192 && aligned(a) && aligned(wa) && aligned(b) && aligned(wb) && aligned(out)) {
    if (width <= 2048)
      launch_kernel(normed_mean_row_kernel<128>, dim3(rows), dim3(128), 0, stream, a, wa, b, wb, out, width, eps, factor);
    else if (width <= 4096)
      launch_kernel(normed_mean_row_kernel<256>, dim3(rows), dim3(256), 0, stream, a, wa, b, wb, out, width, eps, factor);
    else
      launch_kernel(normed_mean_row_kernel<512>, dim3(rows), dim3(512), 0, stream, a, wa, b, wb, out, width, eps, factor);
    return launch_status();
  }
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(normed_mean_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(normed_mean_kernel, dim3(rows), dim3(256), shared, stream, a, wa, b, wb, out, width, eps, factor);
  return launch_status();
}

MLR_EXPORT int mlr_clamped_gate(const void* x, void* out, long long rows, int inner, int block, float limit, float slope,
                                int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || inner <= 0 || block <= 0 || inner % block != 0) return MLR_BAD_SIZE;
  const long long blocks = (rows * inner + 255) / 256;
  if (blocks > 0x7fffffffLL) return MLR_TOO_LARGE;
  if (dtype == MLR_F32)
    launch_kernel(clamped_gate_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)x, (float*)out,
                  rows, inner, block, limit, slope);
  else if (dtype == MLR_BF16)
    launch_kernel(clamped_gate_kernel<bf16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const bf16*)x, (bf16*)out,
                  rows, inner, block, limit, slope);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

MLR_EXPORT int mlr_scale_inplace(float* x, long long count, float factor, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  const long long blocks = (count + 255) / 256;
  if (blocks > 0x7fffffffLL) return MLR_TOO_LARGE;
  launch_kernel(scale_inplace_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, count, factor);
  return launch_status();
}
