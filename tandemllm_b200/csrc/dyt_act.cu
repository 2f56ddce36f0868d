// Element-wise row kernels: the Dynamic Tanh norm fused with the residual add in front of it, and activations applied
// to a product's rows.
//
//   dyt      residual += delta;  out = tanh(alpha * residual) * w + b      alpha one scalar a norm; no mean, no variance
//   xielu    f(z) = ap z^2 + z / 2 for z > 0,  an (exp(z) - 1 - z) + z / 2 for z <= 0      (ap, an: two numbers a layer)
//
// Everything is computed in 32-bit; only the output is rounded to the compute dtype.
#include "common.cuh"

namespace tl {

// One thread takes `VEC` consecutive elements of an output row. `delta` holds `parts` partial sums [parts][rows, hidden]
// that are added in order (parts 0: nothing is added). With `gather`, output row i is made from row gather[i] and the
// residual is left as it is.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) add_dyt_kernel(float* __restrict__ residual, const float* __restrict__ delta, int parts,
                                                      long long part_stride, const float* __restrict__ weight,
                                                      const float* __restrict__ bias, const float* __restrict__ alpha,
                                                      T* __restrict__ out, const int* __restrict__ gather, int out_rows,
                                                      int hidden) {
  const int per_row = hidden / VEC;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)out_rows * per_row) return;
  const int orow = (int)(i / per_row), c = (int)(i - (long long)orow * per_row) * VEC;
  const int r = gather ? gather[orow] : orow;
  const float a = alpha[0];
  float x[VEC], d[VEC];
  const float* res = residual + (long long)r * hidden + c;
  if constexpr (VEC == 4) {
    const float4 v = *reinterpret_cast<const float4*>(res);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
    x[0] = res[0];
  }
  if (parts > 0) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) d[j] = 0.f;
    for (int s = 0; s < parts; ++s) {
      const float* src = delta + s * part_stride + (long long)r * hidden + c;
      if constexpr (VEC == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        d[0] += v.x; d[1] += v.y; d[2] += v.z; d[3] += v.w;
      } else {
        d[0] += src[0];
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) x[j] += d[j];
    if (!gather) {
      if constexpr (VEC == 4) *reinterpret_cast<float4*>(residual + (long long)r * hidden + c) = make_float4(x[0], x[1], x[2], x[3]);
      else residual[(long long)r * hidden + c] = x[0];
    }
  }
  T* dst = out + (long long)orow * hidden + c;
#pragma unroll
  for (int j = 0; j < VEC; ++j) dst[j] = from_f32<T>(fmaf(tanhf(a * x[j]), weight[c + j], bias[c + j]));
}

template <typename T>
__global__ void __launch_bounds__(256) activation_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, int act,
                                                         float a0, float a1) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_f32<T>(activation(to_f32(in[i]), act, a0, a1));
}

}  // namespace tl

using namespace tl;

extern "C" int tl_add_dyt(float* residual, const float* delta, int parts, long long part_stride, const float* weight,
                          const float* bias, const float* alpha, void* out, const int* gather, int out_rows, int hidden,
                          int dtype, cudaStream_t stream) {
  if (out_rows == 0) return 0;
  TL_REQUIRE(hidden > 0 && parts >= 0 && (parts == 0 || delta), "add_dyt: hidden %d, %d parts", hidden, parts);
  const bool vec = hidden % 4 == 0 && ((uintptr_t)residual % 16) == 0 && (!delta || ((uintptr_t)delta % 16) == 0) &&
                   part_stride % 4 == 0;
  const long long n = (long long)out_rows * (vec ? hidden / 4 : hidden);
  const unsigned blocks = (unsigned)ceil_div64(n, 256);
#define TL_DYT(T_, V_)                                                                                             \
  add_dyt_kernel<T_, V_><<<blocks, 256, 0, stream>>>(residual, delta, parts, part_stride, weight, bias, alpha, (T_*)out, \
                                                     gather, out_rows, hidden)
  if (dtype == TL_FP32) {
    if (vec) TL_DYT(float, 4); else TL_DYT(float, 1);
  } else {
    if (vec) TL_DYT(bf16, 4); else TL_DYT(bf16, 1);
  }
#undef TL_DYT
  TL_LAUNCH_CHECK();
  return 0;
}

// out = act(in) element by element, `act` a code TL_ACT_* with its two constants (xIELU: the two branch factors).
extern "C" int tl_activation(const void* in, void* out, long long n, int act, float a0, float a1, int dtype,
                             cudaStream_t stream) {
  if (n == 0) return 0;
  TL_REQUIRE(act >= 1 && act <= TL_ACT_LAST, "activation %d is not one of 1..%d", act, TL_ACT_LAST);
  const unsigned blocks = (unsigned)ceil_div64(n, 256);
  if (dtype == TL_FP32) activation_kernel<float><<<blocks, 256, 0, stream>>>((const float*)in, (float*)out, n, act, a0, a1);
  else activation_kernel<bf16><<<blocks, 256, 0, stream>>>((const bf16*)in, (bf16*)out, n, act, a0, a1);
  TL_LAUNCH_CHECK();
  return 0;
}
