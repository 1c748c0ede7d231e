// Row kernels of blocks that norm a sublayer's input AND its output ("sandwich" blocks), all with 32-bit math:
//
//   group_norm   x += mult * post_w * groupnorm(delta + bias)   (the sublayer's output, normed, scaled, added)
//                out = pre_w * groupnorm(x)                     (the next sublayer's input)
//                in ONE pass over the row; either half may be missing.  groupnorm cuts a row into equal
//                consecutive parts and divides each by sqrt(mean(part^2) + eps).
//   bias_act     out = act(sum of split-K partials + bias + add)   (epilogue of a biased product)
//   short_conv   out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)  per channel over a request's time axis, the
//                last taps - 1 inputs of every request kept as its state.
//
// Every sum runs in an order that depends on the row alone (not on the batch or on how a prompt was cut).
#include "common.cuh"

// 1 / rms of every group of row[0..D) into inv[0..groups): warp w takes groups w, w + nwarp, ...
__device__ __forceinline__ void group_rms(const float* row, int D, int groups, float eps, float* rms) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int gs = D / groups;
  for (int g = warp; g < groups; g += nwarp) {
    const float* p = row + (size_t)g * gs;
    float s = 0.f;
    for (int i = lane; i < gs; i += 32) s = fmaf(p[i], p[i], s);
    s = warp_sum(s);
    if (lane == 0) rms[g] = sqrtf(s / (float)gs + eps);
  }
}

// One block per row.  Source row r = row_index ? row_index[n] : n (then x is not written back).
template <typename TO>
__global__ void group_norm_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits, long long split_stride,
                                  const float* __restrict__ delta_bias, const float* __restrict__ post_w, int post_groups,
                                  float mult, const float* __restrict__ pre_w, int pre_groups, int pre_norm, float eps,
                                  TO* __restrict__ out, long long ld_out, float* __restrict__ out32,
                                  const int* __restrict__ row_index, int D) {
  JLX_TL(TL_NORM);
  extern __shared__ float smem[];
  float* row = smem;       // [D]
  float* rms = smem + D;   // [max groups]
  const int n = blockIdx.x;
  const size_t r = row_index ? (size_t)row_index[n] : (size_t)n;
  float* xr = x + r * D;
  if (delta) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float s = 0.f;
      for (int z = 0; z < splits; ++z) s += delta[(size_t)z * split_stride + r * D + d];
      if (delta_bias) s += delta_bias[d];
      row[d] = s;
    }
    __syncthreads();
    if (post_w) {
      group_rms(row, D, post_groups, eps, rms);
      __syncthreads();
      const int gs = D / post_groups;
      for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float y = row[d] / rms[d / gs] * post_w[d];
        const float s = fmaf(mult, y, xr[d]);
        row[d] = s;
        if (!row_index) xr[d] = s;
      }
    } else {
      for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float s = xr[d] + mult * row[d];
        row[d] = s;
        if (!row_index) xr[d] = s;
      }
    }
  } else {
    for (int d = threadIdx.x; d < D; d += blockDim.x) row[d] = xr[d];
  }
  if (!out && !out32) return;
  __syncthreads();
  if (pre_norm) {
    group_rms(row, D, pre_groups, eps, rms);
    __syncthreads();
  }
  const int gs = pre_norm ? D / pre_groups : D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float v = row[d];
    if (pre_norm) {
      v = v / rms[d / gs];
      if (pre_w) v *= pre_w[d];
    }
    if (out) out[(size_t)n * ld_out + d] = from_f32<TO>(v);
    if (out32) out32[(size_t)n * D + d] = v;
  }
}

JLX_API int jlx_group_norm(float* x, const float* delta, int splits, long long split_stride, const float* delta_bias,
                           const float* post_w, int post_groups, float mult, const float* pre_w, int pre_groups,
                           int pre_norm, float eps, void* out, int out_dtype, long long ld_out, float* out32,
                           const int* row_index, int N, int D, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0 && splits >= 1, "group_norm: bad sizes N=%d D=%d splits=%d", N, D, splits);
  JLX_REQUIRE(eps > 0.f, "group_norm: eps must be positive");
  JLX_REQUIRE(!post_w || (post_groups >= 1 && D % post_groups == 0), "group_norm: %d groups do not divide the width %d", post_groups, D);
  JLX_REQUIRE(!pre_norm || (pre_groups >= 1 && D % pre_groups == 0), "group_norm: %d groups do not divide the width %d", pre_groups, D);
  JLX_REQUIRE(!out || ld_out >= D, "group_norm: the output's row is shorter than the width");
  if (N == 0) return 0;
  const int g = (post_w && post_groups > pre_groups) ? post_groups : (pre_groups > 1 ? pre_groups : 1);
  const size_t smem = sizeof(float) * ((size_t)D + g);
  JLX_REQUIRE(smem <= 200 * 1024, "group_norm: a row of %d values does not fit into shared memory", D);
  const int threads = D >= 4096 ? 512 : (D >= 1024 ? 256 : 128);
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    if (smem > 48 * 1024)
      JLX_CUDA(cudaFuncSetAttribute(group_norm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    group_norm_kernel<TO><<<N, threads, smem, stream>>>(x, delta, splits, split_stride, delta_bias, post_w, post_groups, mult,
                                                         pre_w, pre_groups, pre_norm, eps, (TO*)out, ld_out, out32, row_index, D);
  });
  JLX_LAUNCH_CHECK("group_norm");
  return 0;
}

// ------------------------------------------------------------------------------------------------ bias + activation
enum { ACT_NONE = 0, ACT_RELU2 = 1, ACT_SILU = 2, ACT_GELU_TANH = 3 };

__device__ __forceinline__ float activate(float z, int act) {
  switch (act) {
    case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    case ACT_SILU: return z / (1.f + expf(-z));
    case ACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    default: return z;
  }
}

template <typename TI, typename TO>
__global__ void bias_act_kernel(const TI* __restrict__ in, int splits, long long split_stride, const float* __restrict__ bias,
                                const float* __restrict__ add, int act, TO* __restrict__ out, int F) {
  JLX_TL(TL_OTHER);
  const size_t i = blockIdx.x;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += to_f32<TI>(in[(size_t)z * split_stride + i * F + f]);
    if (bias) s += bias[f];
    if (add) s += add[i * F + f];
    out[i * F + f] = from_f32<TO>(activate(s, act));
  }
}

JLX_API int jlx_bias_act(const void* in, int in_dtype, int splits, long long split_stride, const float* bias, const float* add,
                         int act, void* out, int out_dtype, int rows, int F, cudaStream_t stream) {
  JLX_REQUIRE(rows >= 0 && F > 0 && splits >= 1, "bias_act: bad sizes rows=%d F=%d splits=%d", rows, F, splits);
  JLX_REQUIRE(splits == 1 || in_dtype == JLX_F32, "bias_act: split-K partials are float32");
  JLX_REQUIRE(act >= ACT_NONE && act <= ACT_GELU_TANH, "bias_act: unknown activation %d", act);
  if (rows == 0) return 0;
  JLX_DISPATCH_DTYPE(in_dtype, TI, JLX_DISPATCH_DTYPE(out_dtype, TO,
      (bias_act_kernel<TI, TO><<<rows, 256, 0, stream>>>((const TI*)in, splits, split_stride, bias, add, act, (TO*)out, F))));
  JLX_LAUNCH_CHECK("bias_act");
  return 0;
}

// ------------------------------------------------------------------------------------------------ short convolution
// h: float32 [N, D] rows of the step's tokens (flattened requests); w: float32 [D, taps]; state: float32
// [slots, taps - 1, D], entry k of a request that holds L tokens being its input at position L - (taps - 1) + k
// (zeros before the start: the slab is zeroed when a request is admitted).
// Blocks 0..N-1 serve one token each, unless the token is among the first taps - 1 of its request's portion: those
// need the state, and block N + r serves them for request r and then moves the state on, one thread per channel
// doing both, so that no block reads a state entry that another block replaces.
#define CONV_MAX_TAPS 16

template <typename TO>
__global__ void short_conv_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ slot_ids,
                                  const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                  TO* __restrict__ out, int N, int D, int taps) {
  JLX_TL(TL_OTHER);
  const int b = blockIdx.x;
  if (b < N) {
    const int r = req_of_token[b];
    if (positions[b] - q_start[r] < taps - 1) return;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float acc = h[(size_t)b * D + d];
      for (int j = 0; j < taps; ++j) acc = fmaf(w[(size_t)d * taps + j], h[(size_t)(b - taps + 1 + j) * D + d], acc);
      out[(size_t)b * D + d] = from_f32<TO>(acc);
    }
    return;
  }
  const int r = b - N;
  const int n0 = cu_q[r], qlen = cu_q[r + 1] - n0;
  float* st = state + (size_t)slot_ids[r] * (taps - 1) * D;
  const int head = qlen < taps - 1 ? qlen : taps - 1;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float old[CONV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k) old[k] = k < taps - 1 ? st[(size_t)k * D + d] : 0.f;
    for (int i = 0; i < head; ++i) {
      float acc = h[(size_t)(n0 + i) * D + d];
      for (int j = 0; j < taps; ++j) {
        const int s = i - taps + 1 + j;  // index within the portion; negative: before it, in the state
        const float v = s >= 0 ? h[(size_t)(n0 + s) * D + d] : old[s + taps - 1];
        acc = fmaf(w[(size_t)d * taps + j], v, acc);
      }
      out[(size_t)(n0 + i) * D + d] = from_f32<TO>(acc);
    }
    for (int k = 0; k < taps - 1; ++k) {
      const int s = qlen - (taps - 1) + k;
      st[(size_t)k * D + d] = s >= 0 ? h[(size_t)(n0 + s) * D + d] : old[s + taps - 1];
    }
  }
}

JLX_API int jlx_short_conv(const float* h, const float* w, float* state, const int* cu_q, const int* q_start,
                           const int* slot_ids, const int* req_of_token, const int* positions, void* out, int out_dtype,
                           int N, int R, int D, int taps, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && R >= 0 && D > 0, "short_conv: bad sizes N=%d R=%d D=%d", N, R, D);
  JLX_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "short_conv: %d taps; supported 1..%d", taps, CONV_MAX_TAPS);
  JLX_REQUIRE(taps == 1 || state, "short_conv: a convolution over more than one tap needs its state");
  if (N == 0) return 0;
  const int blocks = N + (taps > 1 ? R : 0);
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    short_conv_kernel<TO><<<blocks, 256, 0, stream>>>(h, w, state, cu_q, q_start, slot_ids, req_of_token, positions, (TO*)out, N, D, taps);
  });
  JLX_LAUNCH_CHECK("short_conv");
  return 0;
}
