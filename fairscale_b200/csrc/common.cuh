// Shared device/host helpers for the sm_100a kernels of this library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FSB_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python bindings
enum FsbDtype : int { FSB_F32 = 0, FSB_F16 = 1, FSB_BF16 = 2 };

// Error codes written to a kernel's status word (0 = ok).
enum FsbStatus : int {
  FSB_OK = 0,
  FSB_ERR_WAIT_TIMEOUT = 1,  // a bounded wait ran out; the kernel returned early, its output is invalid
  FSB_ERR_BAD_ARG = 2,
};

namespace fsb {

constexpr int kWarp = 32;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : 0.f;
  if (warp == 0) r = warp_sum(r);
  if (threadIdx.x == 0) scratch[0] = r;
  __syncthreads();
  return scratch[0];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nwarps) ? scratch[threadIdx.x] : -INFINITY;
  if (warp == 0) r = warp_max(r);
  if (threadIdx.x == 0) scratch[0] = r;
  __syncthreads();
  return scratch[0];
}

// ---- scalar conversion between storage types and fp32 ------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- 16-byte vectors of T -----------------------------------------------------------------------
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 raw; T v[N]; };
};

template <typename T> __device__ __forceinline__ Vec16<T> ld16(const T* p) {
  Vec16<T> r;
  r.raw = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <typename T> __device__ __forceinline__ void st16(T* p, const Vec16<T>& x) {
  *reinterpret_cast<uint4*>(p) = x.raw;
}

// erf(x) as an odd polynomial x * P(x^2) of degree 17 on |x| <= 3.5 (least-squares fit on Chebyshev nodes, max error
// 2.1e-4 in fp32), constant beyond.  The GEMM epilogues evaluate it per element: with the libdevice routine, or with
// any formula built on a reciprocal and an exponential, they were bound by the special-function pipe; this one runs
// on the FMA pipe only.  The error is an order of magnitude below the bf16 rounding of the result.
__device__ __forceinline__ float fast_erf(float x) {
  const float ax = fminf(fabsf(x), 3.5f);
  const float t = ax * ax;
  float p = 1.7347794642241373e-08f;
  p = fmaf(p, t, -1.0356023911367276e-06f);
  p = fmaf(p, t, 2.671026157385393e-05f);
  p = fmaf(p, t, -0.0003934614440707046f);
  p = fmaf(p, t, 0.0037059609711284783f);
  p = fmaf(p, t, -0.02383114556013128f);
  p = fmaf(p, t, 0.10964519147478315f);
  p = fmaf(p, t, -0.37479130195833465f);
  p = fmaf(p, t, 1.1282852575734723f);
  return copysignf(fminf(ax * p, 1.f), x);
}
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.f + fast_erf(x * 0.70710678118654752f));
}
// d/dx gelu(x) = Phi(x) + x phi(x): the polynomial erf plus one exponential.
__device__ __forceinline__ float gelu_erf_grad(float x) {
  const float cdf = fmaf(0.5f, fast_erf(x * 0.70710678118654752f), 0.5f);
  return fmaf(x * 0.3989422804014327f, __expf(-0.5f * x * x), cdf);
}

}  // namespace fsb
