// Row kernels of blocks that norm a sublayer's input AND its output ("sandwich" blocks), all with 32-bit math:
//
//   group_norm   x += mult * post_w * groupnorm(delta + bias)   (the sublayer's output, normed, scaled, added;
//                with post_norm = 0 the norm is left out and post_w is a scale per channel: x += mult * post_w * delta)
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
                                  int post_norm, float mult, const float* __restrict__ pre_w, int pre_groups, int pre_norm, float eps,
                                  TO* __restrict__ out, long long ld_out, float* __restrict__ out32,
                                  const int* __restrict__ row_index, int D) {
  JLX_TL(TL_NORM);
  pdl_launch_dependents_if_small();
  pdl_wait();
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
      if (post_norm) group_rms(row, D, post_groups, eps, rms);
      __syncthreads();
      const int gs = D / post_groups;
      for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float y = post_norm ? row[d] / rms[d / gs] * post_w[d] : row[d] * post_w[d];
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

// Four consecutive outputs as one access (the address is a multiple of 4 elements).
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = o;
}

// The same row, four values per access: for widths and groups that are multiples of 4 and 16-byte aligned tensors.
// Every value goes through the same operations as in the kernel above.
template <typename TO>
__global__ void group_norm_x4_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits, long long split_stride,
                                     const float* __restrict__ delta_bias, const float* __restrict__ post_w, int post_groups,
                                     int post_norm, float mult, const float* __restrict__ pre_w, int pre_groups, int pre_norm, float eps,
                                     TO* __restrict__ out, long long ld_out, float* __restrict__ out32,
                                     const int* __restrict__ row_index, int D) {
  JLX_TL(TL_NORM);
  pdl_launch_dependents_if_small();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  float* row = smem;       // [D]
  float* rms = smem + D;   // [max groups]
  float4* row4 = reinterpret_cast<float4*>(row);
  const int n = blockIdx.x, D4 = D >> 2;
  const size_t r = row_index ? (size_t)row_index[n] : (size_t)n;
  float4* xr4 = reinterpret_cast<float4*>(x + r * D);
  if (delta) {
    for (int d = threadIdx.x; d < D4; d += blockDim.x) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int z = 0; z < splits; ++z) {
        const float4 v = *reinterpret_cast<const float4*>(delta + (size_t)z * split_stride + r * D + 4 * d);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      if (delta_bias) {
        const float4 b = reinterpret_cast<const float4*>(delta_bias)[d];
        s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w;
      }
      row4[d] = s;
    }
    __syncthreads();
    if (post_w) {
      if (post_norm) group_rms(row, D, post_groups, eps, rms);
      __syncthreads();
      const int gs4 = (D / post_groups) >> 2;
      for (int d = threadIdx.x; d < D4; d += blockDim.x) {
        const float rr = rms[d / gs4];
        const float4 v = row4[d], w = reinterpret_cast<const float4*>(post_w)[d], xo = xr4[d];
        float4 s;
        if (post_norm) {
          s.x = fmaf(mult, v.x / rr * w.x, xo.x);
          s.y = fmaf(mult, v.y / rr * w.y, xo.y);
          s.z = fmaf(mult, v.z / rr * w.z, xo.z);
          s.w = fmaf(mult, v.w / rr * w.w, xo.w);
        } else {  // a scale per channel, no norm
          s.x = fmaf(mult, v.x * w.x, xo.x);
          s.y = fmaf(mult, v.y * w.y, xo.y);
          s.z = fmaf(mult, v.z * w.z, xo.z);
          s.w = fmaf(mult, v.w * w.w, xo.w);
        }
        row4[d] = s;
        if (!row_index) xr4[d] = s;
      }
    } else {
      for (int d = threadIdx.x; d < D4; d += blockDim.x) {
        const float4 v = row4[d], xo = xr4[d];
        const float4 s = make_float4(xo.x + mult * v.x, xo.y + mult * v.y, xo.z + mult * v.z, xo.w + mult * v.w);
        row4[d] = s;
        if (!row_index) xr4[d] = s;
      }
    }
  } else {
    for (int d = threadIdx.x; d < D4; d += blockDim.x) row4[d] = xr4[d];
  }
  if (!out && !out32) return;
  __syncthreads();
  if (pre_norm) {
    group_rms(row, D, pre_groups, eps, rms);
    __syncthreads();
  }
  const int gs4 = pre_norm ? (D / pre_groups) >> 2 : D4;
  for (int d = threadIdx.x; d < D4; d += blockDim.x) {
    float4 v = row4[d];
    if (pre_norm) {
      const float rr = rms[d / gs4];
      v.x /= rr; v.y /= rr; v.z /= rr; v.w /= rr;
      if (pre_w) {
        const float4 w = reinterpret_cast<const float4*>(pre_w)[d];
        v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
      }
    }
    if (out) store4<TO>(out + (size_t)n * ld_out + 4 * d, v);
    if (out32) reinterpret_cast<float4*>(out32 + (size_t)n * D)[d] = v;
  }
}

JLX_API int jlx_group_norm(float* x, const float* delta, int splits, long long split_stride, const float* delta_bias,
                           const float* post_w, int post_groups, int post_norm, float mult, const float* pre_w,
                           int pre_groups, int pre_norm, float eps, void* out, int out_dtype, long long ld_out, float* out32,
                           const int* row_index, int N, int D, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0 && splits >= 1, "group_norm: bad sizes N=%d D=%d splits=%d", N, D, splits);
  JLX_REQUIRE(eps > 0.f, "group_norm: eps must be positive");
  if (!post_norm) post_groups = 1;
  JLX_REQUIRE(!post_w || (post_groups >= 1 && D % post_groups == 0), "group_norm: %d groups do not divide the width %d", post_groups, D);
  JLX_REQUIRE(!pre_norm || (pre_groups >= 1 && D % pre_groups == 0), "group_norm: %d groups do not divide the width %d", pre_groups, D);
  JLX_REQUIRE(!out || ld_out >= D, "group_norm: the output's row is shorter than the width");
  if (N == 0) return 0;
  const int g = (post_w && post_groups > pre_groups) ? post_groups : (pre_groups > 1 ? pre_groups : 1);
  const size_t smem = sizeof(float) * ((size_t)D + g + 4);
  JLX_REQUIRE(smem <= 200 * 1024, "group_norm: a row of %d values does not fit into shared memory", D);
  const int threads = D >= 4096 ? 512 : (D >= 1024 ? 256 : 128);
  const bool x4 = (D & 3) == 0 && (!post_w || ((D / post_groups) & 3) == 0) && (!pre_norm || ((D / pre_groups) & 3) == 0) &&
                  (split_stride & 3) == 0 && (ld_out & 3) == 0 &&
                  (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)delta_bias | (uintptr_t)post_w | (uintptr_t)pre_w |
                    (uintptr_t)out | (uintptr_t)out32) & 15) == 0;
  if (x4) {
    JLX_DISPATCH_DTYPE(out_dtype, TO, {
      if (smem > 48 * 1024)
        JLX_CUDA(cudaFuncSetAttribute(group_norm_x4_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      JLX_CUDA(jlx_launch_pdl(group_norm_x4_kernel<TO>, dim3(N), dim3(D >= 8192 ? 512 : (D >= 2048 ? 256 : 128)), smem, stream,
                              x, delta, splits, split_stride, delta_bias, post_w, post_groups, post_norm, mult, pre_w, pre_groups, pre_norm,
                              eps, (TO*)out, ld_out, out32, row_index, D));
    });
    JLX_LAUNCH_CHECK("group_norm");
    return 0;
  }
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    if (smem > 48 * 1024)
      JLX_CUDA(cudaFuncSetAttribute(group_norm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    JLX_CUDA(jlx_launch_pdl(group_norm_kernel<TO>, dim3(N), dim3(threads), smem, stream, x, delta, splits, split_stride, delta_bias,
                            post_w, post_groups, post_norm, mult, pre_w, pre_groups, pre_norm, eps, (TO*)out, ld_out, out32, row_index, D));
  });
  JLX_LAUNCH_CHECK("group_norm");
  return 0;
}

// ------------------------------------------------------------------------------------------------ bias + activation
enum { ACT_NONE = 0, ACT_RELU2 = 1, ACT_SILU = 2, ACT_GELU_TANH = 3, ACT_GELU = 4, ACT_TANH = 5 };

__device__ __forceinline__ float activate(float z, int act) {
  switch (act) {
    case ACT_RELU2: { const float r = fmaxf(z, 0.f); return r * r; }
    case ACT_SILU: return z / (1.f + expf(-z));
    case ACT_GELU: return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));
    case ACT_TANH: return tanhf(z);
    case ACT_GELU_TANH: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    default: return z;
  }
}

template <typename TI, typename TO>
__global__ void bias_act_kernel(const TI* __restrict__ in, int splits, long long split_stride, const float* __restrict__ bias,
                                const float* __restrict__ add, int act, TO* __restrict__ out, int F) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t i = blockIdx.x;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += to_f32<TI>(in[(size_t)z * split_stride + i * F + f]);
    if (bias) s += bias[f];
    if (add) s += add[i * F + f];
    out[i * F + f] = from_f32<TO>(activate(s, act));
  }
}

// The common case: float32 sums in (whole or split-K partials), four values per access.
template <typename TO>
__global__ void bias_act_f32x4_kernel(const float* __restrict__ in, int splits, long long split_stride, const float* __restrict__ bias,
                                      const float* __restrict__ add, int act, TO* __restrict__ out, int F) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const size_t i = blockIdx.x;
  for (int f = threadIdx.x * 4; f < F; f += blockDim.x * 4) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int z = 0; z < splits; ++z) {
      const float4 v = *reinterpret_cast<const float4*>(in + (size_t)z * split_stride + i * F + f);
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + f);
      s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w;
    }
    if (add) {
      const float4 a = *reinterpret_cast<const float4*>(add + i * F + f);
      s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w;
    }
    out[i * F + f] = from_f32<TO>(activate(s.x, act));
    out[i * F + f + 1] = from_f32<TO>(activate(s.y, act));
    out[i * F + f + 2] = from_f32<TO>(activate(s.z, act));
    out[i * F + f + 3] = from_f32<TO>(activate(s.w, act));
  }
}

JLX_API int jlx_bias_act(const void* in, int in_dtype, int splits, long long split_stride, const float* bias, const float* add,
                         int act, void* out, int out_dtype, int rows, int F, cudaStream_t stream) {
  JLX_REQUIRE(rows >= 0 && F > 0 && splits >= 1, "bias_act: bad sizes rows=%d F=%d splits=%d", rows, F, splits);
  JLX_REQUIRE(splits == 1 || in_dtype == JLX_F32, "bias_act: split-K partials are float32");
  JLX_REQUIRE(act >= ACT_NONE && act <= ACT_TANH, "bias_act: unknown activation %d", act);
  if (rows == 0) return 0;
  if (in_dtype == JLX_F32 && (F & 3) == 0 && (split_stride & 3) == 0 &&
      (((uintptr_t)in | (uintptr_t)bias | (uintptr_t)add) & 15) == 0) {
    JLX_DISPATCH_DTYPE(out_dtype, TO,
        JLX_CUDA(jlx_launch_pdl(bias_act_f32x4_kernel<TO>, dim3(rows), dim3(256), 0, stream, (const float*)in, splits, split_stride,
                                bias, add, act, (TO*)out, F)));
    JLX_LAUNCH_CHECK("bias_act");
    return 0;
  }
  JLX_DISPATCH_DTYPE(in_dtype, TI, JLX_DISPATCH_DTYPE(out_dtype, TO,
      JLX_CUDA(jlx_launch_pdl(bias_act_kernel<TI, TO>, dim3(rows), dim3(256), 0, stream, (const TI*)in, splits, split_stride, bias,
                              add, act, (TO*)out, F))));
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
  pdl_launch_dependents_if_small();
  pdl_wait();
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

// The same with four channels per thread (width a multiple of 4, 16-byte aligned tensors); same operations per value.
template <typename TO>
__global__ void short_conv_x4_kernel(const float* __restrict__ h, const float* __restrict__ w, float* __restrict__ state,
                                     const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ slot_ids,
                                     const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                     TO* __restrict__ out, int N, int D, int taps) {
  JLX_TL(TL_OTHER);
  pdl_launch_dependents_if_small();
  pdl_wait();
  const int b = blockIdx.x, D4 = D >> 2;
  auto h4 = [&](int row, int d) { return reinterpret_cast<const float4*>(h + (size_t)row * D)[d]; };
  auto tap = [&](float4& acc, int d, int j, const float4 v) {
    acc.x = fmaf(w[(size_t)(4 * d) * taps + j], v.x, acc.x);
    acc.y = fmaf(w[(size_t)(4 * d + 1) * taps + j], v.y, acc.y);
    acc.z = fmaf(w[(size_t)(4 * d + 2) * taps + j], v.z, acc.z);
    acc.w = fmaf(w[(size_t)(4 * d + 3) * taps + j], v.w, acc.w);
  };
  if (b < N) {
    const int r = req_of_token[b];
    if (positions[b] - q_start[r] < taps - 1) return;
    for (int d = threadIdx.x; d < D4; d += blockDim.x) {
      float4 acc = h4(b, d);
      for (int j = 0; j < taps; ++j) tap(acc, d, j, h4(b - taps + 1 + j, d));
      store4<TO>(out + (size_t)b * D + 4 * d, acc);
    }
    return;
  }
  const int r = b - N;
  const int n0 = cu_q[r], qlen = cu_q[r + 1] - n0;
  float4* st = reinterpret_cast<float4*>(state + (size_t)slot_ids[r] * (taps - 1) * D);
  const int head = qlen < taps - 1 ? qlen : taps - 1;
  for (int d = threadIdx.x; d < D4; d += blockDim.x) {
    float4 old[CONV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k) old[k] = k < taps - 1 ? st[(size_t)k * D4 + d] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = 0; i < head; ++i) {
      float4 acc = h4(n0 + i, d);
      for (int j = 0; j < taps; ++j) {
        const int s = i - taps + 1 + j;
        tap(acc, d, j, s >= 0 ? h4(n0 + s, d) : old[s + taps - 1]);
      }
      store4<TO>(out + (size_t)(n0 + i) * D + 4 * d, acc);
    }
    for (int k = 0; k < taps - 1; ++k) {
      const int s = qlen - (taps - 1) + k;
      st[(size_t)k * D4 + d] = s >= 0 ? h4(n0 + s, d) : old[s + taps - 1];
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
  if ((D & 3) == 0 && (((uintptr_t)h | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
    JLX_DISPATCH_DTYPE(out_dtype, TO, {
      JLX_CUDA(jlx_launch_pdl(short_conv_x4_kernel<TO>, dim3(blocks), dim3(D >= 4096 ? 256 : 128), 0, stream, h, w, state, cu_q, q_start,
                              slot_ids, req_of_token, positions, (TO*)out, N, D, taps));
    });
    JLX_LAUNCH_CHECK("short_conv");
    return 0;
  }
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    JLX_CUDA(jlx_launch_pdl(short_conv_kernel<TO>, dim3(blocks), dim3(256), 0, stream, h, w, state, cu_q, q_start, slot_ids,
                            req_of_token, positions, (TO*)out, N, D, taps));
  });
  JLX_LAUNCH_CHECK("short_conv");
  return 0;
}
