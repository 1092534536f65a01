// Kernels of a selective state-space mixer with a scalar decay per head (the "state-space duality"
// form): a short causal convolution per channel whose last inputs are carried per request, the
// recurrence itself, and the gated, grouped RMS norm behind it.  Everything here is float32; the
// projections around it are products of their own.
//
// mlr_causal_conv        out[t, c] = act(bias[c] + sum_k w[c, k] u[t - (taps - 1) + k, c]) over the tokens
//                        of each request, the inputs before the step's first token coming from the
//                        request's state [taps - 1, channels] (zeros for a new request), which then
//                        receives the step's last inputs.  act: silu (1) or none (0).
// mlr_state_space_scan   per request, head h and token t, with g(h) = h / (heads / groups):
//                          dt = softplus(dt_raw[t, h] + dt_bias[h]);  a = exp(-exp(A_log[h]) dt)
//                          S <- a S + dt B[t, g] x[t, h]^T            (S: [state, vdim], kept as [vdim, state])
//                          y[t, h] = S^T C[t, g] + D[h] x[t, h]
//                        token by token in a fixed order, so a request's numbers do not depend on how its
//                        tokens were cut into steps.
// mlr_gated_group_norm   out = RMSnorm_parts(y * silu(z)) * weight: the row is cut into `parts` equal parts,
//                        each divided by its own root mean square (eps inside the root).
#include "common.cuh"

#include <type_traits>

namespace mlr {

constexpr int MAX_TAPS = 16;

// The request's new carried inputs: the last taps - 1 inputs of (old carried inputs, the step's rows).
__device__ __forceinline__ void carry_inputs(const float* u, long long u_stride, float* state, int channels, int c,
                                             int q_start, int q_len, int taps) {
  float kept[MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i) {
    if (i < taps - 1) {
      const int t = q_len - (taps - 1) + i;       // relative to the step's first row
      kept[i] = t >= 0 ? __ldcg(u + (size_t)(q_start + t) * u_stride + c) : state[(size_t)(taps - 1 + t) * channels + c];
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_TAPS - 1; ++i)
    if (i < taps - 1) state[(size_t)i * channels + c] = kept[i];
}

constexpr int CONV_TOKENS = 16;     // tokens one thread walks

// grid: (channel blocks, segments, token chunks).  A one-row segment's thread also advances the state;
// longer segments leave that to carry_kernel (their readers and the writer would race otherwise).
__global__ void __launch_bounds__(128)
causal_conv_kernel(const float* u, long long u_stride, const float* __restrict__ weight, const float* __restrict__ bias,
                   float* states, float* out, const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                   const int* __restrict__ seg_slot, int channels, int taps, int act) {
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seg = blockIdx.y;
  float w[MAX_TAPS];
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) w[k] = (k < taps && c < channels) ? weight[(size_t)c * taps + k] : 0.f;
  const float b = (bias != nullptr && c < channels) ? bias[c] : 0.f;
  pdl_wait();
  if (c >= channels) return;
  const int q_start = seg_q_start[seg], q_len = seg_q_len[seg];
  const int t0 = blockIdx.z * CONV_TOKENS;
  if (t0 >= q_len) return;
  float* state = states + (size_t)seg_slot[seg] * (taps - 1) * channels;
  const int count = min(q_len - t0, CONV_TOKENS);
  // every input the thread's tokens need, asked for at once (one trip to memory): the tokens' own and the
  // taps - 1 before them, which for the segment's first tokens come from the carried inputs
  float in[CONV_TOKENS + MAX_TAPS - 1];
#pragma unroll
  for (int i = 0; i < CONV_TOKENS + MAX_TAPS - 1; ++i) {
    in[i] = 0.f;
    if (i < count + taps - 1) {
      const int s = t0 - (taps - 1) + i;
      in[i] = s >= 0 ? __ldcg(u + (size_t)(q_start + s) * u_stride + c) : state[(size_t)(taps - 1 + s) * channels + c];
    }
  }
#pragma unroll
  for (int t = 0; t < CONV_TOKENS; ++t) {
    if (t < count) {
      float sum = b;
#pragma unroll
      for (int k = 0; k < MAX_TAPS; ++k)
        if (k < taps) sum = fmaf(w[k], in[t + k], sum);
      if (act == 1) sum = sum / (1.f + expf(-sum));
      out[(size_t)(q_start + t0 + t) * channels + c] = sum;
    }
  }
  if (q_len == 1) carry_inputs(u, u_stride, state, channels, c, q_start, q_len, taps);
}

__global__ void __launch_bounds__(128)
carry_kernel(const float* u, long long u_stride, float* states, const int* __restrict__ seg_q_start,
             const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot, int channels, int taps) {
  // The kernel behind this one is the recurrence: few blocks that run long.  Brought in while the
  // convolution's thousands of blocks still fill the SMs, its blocks land several to an SM, wherever room
  // appears first, and share that SM's shared-memory pipe for their whole walk (a prompt step of twelve
  // layers: 11.3 ms against 8.7 ms).  So the trigger comes after the wait: the recurrence's blocks are
  // placed on an almost idle GPU, one per SM.
  pdl_wait();
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seg = blockIdx.y;
  if (c >= channels) return;
  const int q_len = seg_q_len[seg];
  if (q_len <= 1) return;
  carry_inputs(u, u_stride, states + (size_t)seg_slot[seg] * (taps - 1) * channels, channels, c, seg_q_start[seg], q_len, taps);
}

constexpr int SCAN_NPT = 16;        // state entries of one value channel a thread holds
constexpr int SCAN_TOKENS = 32;     // tokens staged at once
constexpr int SCAN_THREADS = 128;

struct ScanArgs {
  const float *x, *B, *C, *dt_raw;
  long long x_stride, b_stride, c_stride, dt_stride;
  const float *dt_bias, *A_log, *D;
  float* states;
  float* y;
  const int *seg_q_start, *seg_q_len, *seg_slot;
  int heads, vdim, n, groups;
};

// Asynchronous copies into shared memory (the data never passes through registers, and the thread goes on).
__device__ __forceinline__ void copy_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// SL: threads that share one value channel's state (a power of two; SL * SCAN_NPT >= n).  Lane l of a warp
// holds 16 entries of channel p = l / SL: the pieces of four entries number s, s + SL, s + 2 SL, s + 3 SL with
// s = l % SL (neighbouring threads read neighbouring 16-byte pieces of a staged row: no bank conflicts; with
// 16 entries in a row per thread a quarter warp's reads fell into two banks).
// grid: (segments, heads, value-channel blocks).  The inputs of 32 tokens at a time are staged in shared
// memory by asynchronous copies, the next 32 while these are walked; WIDE: in 16-byte pieces (state size,
// channel block and all row strides multiples of four floats, pointers aligned).
template <int SL, bool WIDE>
__global__ void __launch_bounds__(SCAN_THREADS)
state_space_scan_kernel(ScanArgs a) {
  pdl_trigger();
  extern __shared__ __align__(16) float shared[];
  constexpr int P_CTA = SCAN_THREADS / SL;
  const int N = a.n, P = a.vdim;
  const int buffer = SCAN_TOKENS * (2 * N + P_CTA + 1);      // floats of one staging buffer
  float* decay = shared + 2 * buffer + SCAN_NPT;             // [SCAN_TOKENS]; a last piece may reach past a buffer's end
  float* step = decay + SCAN_TOKENS;                         // [SCAN_TOKENS]
  const int seg = blockIdx.x, head = blockIdx.y;
  const int group = head / (a.heads / a.groups);
  const int s = threadIdx.x % SL, p_local = threadIdx.x / SL;
  const int p = blockIdx.z * P_CTA + p_local;
  const float rate = expf(a.A_log[head]), bias = a.dt_bias[head], skip = a.D[head];
  pdl_wait();
  const int q_start = a.seg_q_start[seg], q_len = a.seg_q_len[seg];

  // rows [t0, t0 + 32) of the segment into buffer `which`: B and C of the head's group, the block's value
  // channels of x, the head's raw step sizes
  auto stage = [&](int t0, int which) {
    float* b_rows = shared + which * buffer;
    float* c_rows = b_rows + SCAN_TOKENS * N;
    float* x_rows = c_rows + SCAN_TOKENS * N;
    float* raw = x_rows + SCAN_TOKENS * P_CTA;
    const int tokens = min(SCAN_TOKENS, q_len - t0);
    const size_t row0 = (size_t)(q_start + t0);
    if (WIDE) {
      const int per_row = N >> 2;
      for (int idx = threadIdx.x; idx < tokens * per_row; idx += SCAN_THREADS) {
        const int t = idx / per_row, n = (idx - t * per_row) << 2;
        copy_async_16(b_rows + t * N + n, a.B + (row0 + t) * a.b_stride + (size_t)group * N + n);
        copy_async_16(c_rows + t * N + n, a.C + (row0 + t) * a.c_stride + (size_t)group * N + n);
      }
      constexpr int X_PIECES = P_CTA / 4;
      for (int idx = threadIdx.x; idx < tokens * X_PIECES; idx += SCAN_THREADS) {
        const int t = idx / X_PIECES, pl = (idx - t * X_PIECES) << 2;
        const int pp = blockIdx.z * P_CTA + pl;
        if (pp < P) copy_async_16(x_rows + t * P_CTA + pl, a.x + (row0 + t) * a.x_stride + (size_t)head * P + pp);
      }
    } else {
      for (int idx = threadIdx.x; idx < tokens * N; idx += SCAN_THREADS) {
        const int t = idx / N, n = idx - t * N;
        copy_async_4(b_rows + idx, a.B + (row0 + t) * a.b_stride + (size_t)group * N + n);
        copy_async_4(c_rows + idx, a.C + (row0 + t) * a.c_stride + (size_t)group * N + n);
      }
      for (int idx = threadIdx.x; idx < tokens * P_CTA; idx += SCAN_THREADS) {
        const int t = idx / P_CTA, pl = idx - t * P_CTA;
        const int pp = blockIdx.z * P_CTA + pl;
        if (pp < P) copy_async_4(x_rows + idx, a.x + (row0 + t) * a.x_stride + (size_t)head * P + pp);
      }
    }
    if (threadIdx.x < tokens) copy_async_4(raw + threadIdx.x, a.dt_raw + (row0 + threadIdx.x) * a.dt_stride + head);
    copy_async_commit();
  };

  stage(0, 0);
  float* state = a.states + (((size_t)a.seg_slot[seg] * a.heads + head) * P + (p < P ? p : 0)) * N;
  auto entry = [&](int i) { return (((i >> 2) * SL + s) << 2) + (i & 3); };      // the state entry a thread's i-th number is
  float S[SCAN_NPT];
#pragma unroll
  for (int i = 0; i < SCAN_NPT; ++i) {
    const int n = entry(i);
    S[i] = (p < P && n < N) ? state[n] : 0.f;
  }
  int which = 0;
  for (int t0 = 0; t0 < q_len; t0 += SCAN_TOKENS, which ^= 1) {
    const int tokens = min(SCAN_TOKENS, q_len - t0);
    const bool more = t0 + SCAN_TOKENS < q_len;
    if (more) stage(t0 + SCAN_TOKENS, which ^ 1);
    if (more) copy_async_wait<1>(); else copy_async_wait<0>();
    __syncthreads();
    const float* b_rows = shared + which * buffer;
    const float* c_rows = b_rows + SCAN_TOKENS * N;
    const float* x_rows = c_rows + SCAN_TOKENS * N;
    const float* raw = x_rows + SCAN_TOKENS * P_CTA;
    if (threadIdx.x < tokens) {
      const float z = raw[threadIdx.x] + bias;
      const float dt = z > 20.f ? z : log1pf(expf(z));
      step[threadIdx.x] = dt;
      decay[threadIdx.x] = expf(-rate * dt);
    }
    __syncthreads();
    // two tokens in flight: the second one's reads and products run under the first one's sums and shuffles
#pragma unroll 2
    for (int t = 0; t < tokens; ++t) {
      const float av = decay[t], xv = p < P ? x_rows[t * P_CTA + p_local] : 0.f;
      const float dx = step[t] * xv;
      const float* bt = b_rows + t * N;
      const float* ct = c_rows + t * N;
      float bv[SCAN_NPT], cv[SCAN_NPT];
      if (WIDE) {
#pragma unroll
        for (int i = 0; i < SCAN_NPT; i += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(bt + entry(i)), c4 = *reinterpret_cast<const float4*>(ct + entry(i));
          bv[i] = b4.x; bv[i + 1] = b4.y; bv[i + 2] = b4.z; bv[i + 3] = b4.w;
          cv[i] = c4.x; cv[i + 1] = c4.y; cv[i + 2] = c4.z; cv[i + 3] = c4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < SCAN_NPT; ++i) {
          const bool in = entry(i) < N;
          bv[i] = in ? bt[entry(i)] : 0.f;
          cv[i] = in ? ct[entry(i)] : 0.f;
        }
      }
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < SCAN_NPT; ++i) {
        if (entry(i) < N) {
          S[i] = fmaf(av, S[i], bv[i] * dx);
          sums[i & 3] = fmaf(S[i], cv[i], sums[i & 3]);
        }
      }
      float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
#pragma unroll
      for (int offset = SL / 2; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (s == 0 && p < P) a.y[(size_t)(q_start + t0 + t) * a.heads * P + (size_t)head * P + p] = fmaf(skip, xv, sum);
    }
    __syncthreads();      // the next turn of the loop stages into this buffer
  }
  if (p < P) {
#pragma unroll
    for (int i = 0; i < SCAN_NPT; ++i) {
      const int n = entry(i);
      if (n < N) state[n] = S[i];
    }
  }
}

// grid: (rows, parts)
template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* y, const float* z, long long z_stride, const float* __restrict__ weight,
                        T* __restrict__ out, int inner, int parts, float eps) {
  pdl_trigger();
  extern __shared__ float staged[];      // [inner / parts] + 32
  const int width = inner / parts;
  float* scratch = staged + width;
  const int row = blockIdx.x, first = blockIdx.y * width;
  pdl_wait();
  float sq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float gate = z == nullptr ? 1.f : __ldcg(z + (size_t)row * z_stride + first + d);
    const float v = __ldcg(y + (size_t)row * inner + first + d) * (z == nullptr ? 1.f : gate / (1.f + expf(-gate)));
    staged[d] = v;
    sq = fmaf(v, v, sq);
  }
  const float rstd = 1.f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    out[(size_t)row * inner + first + d] = from_float<T>(staged[d] * rstd * weight[first + d]);
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// u: float32 rows of `channels` entries spaced u_stride apart; weight: float32 [channels, taps]; bias:
// float32 [channels] or null; states: float32 [slots, taps - 1, channels]; out: float32 [rows, channels].
MLR_EXPORT int mlr_causal_conv(const float* u, long long u_stride, const float* weight, const float* bias, float* states,
                               float* out, const int* seg_q_start, const int* seg_q_len, const int* seg_slot, int segments,
                               int max_q_len, int channels, int taps, int act, cudaStream_t stream) {
  if (segments == 0) return MLR_OK;
  if (segments < 0 || max_q_len <= 0 || channels <= 0 || taps < 2) return MLR_BAD_SIZE;
  if (taps > MAX_TAPS || segments > 65535) return MLR_TOO_LARGE;
  const int chunks = (max_q_len + CONV_TOKENS - 1) / CONV_TOKENS;
  if (chunks > 65535) return MLR_TOO_LARGE;
  launch_kernel(causal_conv_kernel, dim3((channels + 127) / 128, segments, chunks), dim3(128), 0, stream, u, u_stride, weight,
                bias, states, out, seg_q_start, seg_q_len, seg_slot, channels, taps, act);
  int status = launch_status();
  if (status != MLR_OK || max_q_len == 1) return status;
  launch_kernel(carry_kernel, dim3((channels + 127) / 128, segments), dim3(128), 0, stream, u, u_stride, states, seg_q_start,
                seg_q_len, seg_slot, channels, taps);
  return launch_status();
}

// x: float32 rows of heads*vdim entries; B, C: rows of groups*n entries; dt_raw: rows of `heads` entries
// (each with its own row stride); dt_bias, A_log, D: float32 [heads]; states: float32 [slots, heads, vdim, n];
// y: float32 [rows, heads*vdim].
MLR_EXPORT int mlr_state_space_scan(const float* x, long long x_stride, const float* B, long long b_stride, const float* C,
                                    long long c_stride, const float* dt_raw, long long dt_stride, const float* dt_bias,
                                    const float* A_log, const float* D, float* states, float* y, const int* seg_q_start,
                                    const int* seg_q_len, const int* seg_slot, int segments, int heads, int vdim, int n,
                                    int groups, cudaStream_t stream) {
  if (segments == 0) return MLR_OK;
  if (segments < 0 || heads <= 0 || vdim <= 0 || n <= 0 || groups <= 0 || heads % groups != 0) return MLR_BAD_SIZE;
  if (n > 32 * SCAN_NPT || heads > 65535) return MLR_TOO_LARGE;
  ScanArgs a{x, B, C, dt_raw, x_stride, b_stride, c_stride, dt_stride, dt_bias, A_log, D, states, y,
             seg_q_start, seg_q_len, seg_slot, heads, vdim, n, groups};
  int slices = 1;
  while (slices * SCAN_NPT < n) slices *= 2;
  auto multiple = [](long long v) { return v % 4 == 0; };
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool wide = multiple(n) && multiple(vdim) && multiple(x_stride) && multiple(b_stride) && multiple(c_stride) &&
                    aligned(x) && aligned(B) && aligned(C);
  auto launch = [&](auto kernel, int sl) -> int {
    const int p_cta = SCAN_THREADS / sl;
    const size_t shared = sizeof(float) * (2 * (size_t)SCAN_TOKENS * (2 * n + p_cta + 1) + SCAN_NPT + 2 * SCAN_TOKENS);
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, dim3(segments, heads, (vdim + p_cta - 1) / p_cta), dim3(SCAN_THREADS), shared, stream, a);
    return launch_status();
  };
  switch (slices) {
    case 1: return wide ? launch(state_space_scan_kernel<1, true>, 1) : launch(state_space_scan_kernel<1, false>, 1);
    case 2: return wide ? launch(state_space_scan_kernel<2, true>, 2) : launch(state_space_scan_kernel<2, false>, 2);
    case 4: return wide ? launch(state_space_scan_kernel<4, true>, 4) : launch(state_space_scan_kernel<4, false>, 4);
    case 8: return wide ? launch(state_space_scan_kernel<8, true>, 8) : launch(state_space_scan_kernel<8, false>, 8);
    case 16: return wide ? launch(state_space_scan_kernel<16, true>, 16) : launch(state_space_scan_kernel<16, false>, 16);
    default: return wide ? launch(state_space_scan_kernel<32, true>, 32) : launch(state_space_scan_kernel<32, false>, 32);
  }
}

// y: float32 [rows, inner]; z: float32 rows of `inner` entries spaced z_stride apart, or null (no gate);
// weight: float32 [inner]; out: [rows, inner] in out_dtype.
MLR_EXPORT int mlr_gated_group_norm(const float* y, const float* z, long long z_stride, const float* weight, void* out,
                                    int rows, int inner, int parts, float eps, int out_dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || inner <= 0 || parts <= 0 || inner % parts != 0) return MLR_BAD_SIZE;
  const size_t shared = sizeof(float) * ((size_t)inner / parts + 32);
  if (shared > 200 * 1024 || parts > 65535) return MLR_TOO_LARGE;
  auto launch = [&](auto kernel, auto* typed) -> int {
    if (shared > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
    }
    launch_kernel(kernel, dim3(rows, parts), dim3(256), shared, stream, y, z, z_stride, weight, typed, inner, parts, eps);
    return launch_status();
  };
  if (out_dtype == MLR_F32) return launch(gated_group_norm_kernel<float>, (float*)out);
  if (out_dtype == MLR_BF16) return launch(gated_group_norm_kernel<bf16>, (bf16*)out);
  return MLR_BAD_DTYPE;
}
