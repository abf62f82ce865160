// Multi-tensor Adam for sm_100a: ONE launch updates any number of tensors.
//
// The tensor table lives in global memory (no kernel-argument size limit); a block finds its
// tensor by binary search over the chunk prefix and streams its chunk with 16-byte accesses.
// Supported storage types (runtime-dispatched, the kernel is bandwidth bound):
//   parameters fp32 / fp16 / bf16, gradients fp32 / fp16 / bf16, moments fp32 or scaled fp16,
//   optional low-precision parameter copy (fp16 / bf16) written in the same pass.
// Side outputs: `found_inf` is set when an fp16 moment overflows; the whole update is skipped
// when `*noop_flag != 0` (AMP found-inf) without a host round trip.
//
// Math (fairscale/clib/fused_adam_cuda/fused_adam_cuda_kernel.cu:21-135): g' = g / grad_scale,
// m = b1 m + (1-b1) g', v = b2 v + (1-b2) g'^2, denom = sqrt(v + eps) (mode 0) or sqrt(v) + eps
// (mode 1), p -= step_size * (m / denom + decay * p); step_size carries the bias correction.
// `adamw` switches to decoupled decay: p = p (1 - lr decay) - step_size m / denom.

#include "common.cuh"

namespace fsb {

struct AdamTensor {
  void* p;
  const void* g;
  void* m;
  void* v;
  void* p_copy;         // may be null
  long long numel;
  long long chunk_start;  // index of this tensor's first chunk in the global chunk numbering
  long long pad_;
};

struct AdamArgs {
  const AdamTensor* table;
  int n_tensors;
  int p_dtype, g_dtype, s_dtype, c_dtype;
  float step_size, lr, beta1, beta2, eps, inv_grad_scale, optim_scale, decay;
  int mode, adamw;
  const int* noop_flag;
  int* found_inf;
  const float* inv_scale_dev;  // optional device scalar multiplied into the gradient (AMP unscale / clip)
};

constexpr int ADAM_CHUNK = 8192;   // elements per block
constexpr int ADAM_THREADS = 256;

__device__ __forceinline__ void load4(const void* base, int dtype, long long i, float (&x)[4]) {
  if (dtype == FSB_F32) {
    const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + i);
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
  } else if (dtype == FSB_BF16) {
    const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + i);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(static_cast<const __half*>(base) + i);
    const __half2 a = *reinterpret_cast<const __half2*>(&t.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&t.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  }
}
__device__ __forceinline__ float load1(const void* base, int dtype, long long i) {
  if (dtype == FSB_F32) return static_cast<const float*>(base)[i];
  if (dtype == FSB_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(static_cast<const __half*>(base)[i]);
}
__device__ __forceinline__ void store4(void* base, int dtype, long long i, const float (&x)[4]) {
  if (dtype == FSB_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + i) = make_float4(x[0], x[1], x[2], x[3]);
  } else if (dtype == FSB_BF16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + i) = t;
  } else {
    __half2 a = __floats2half2_rn(x[0], x[1]), b = __floats2half2_rn(x[2], x[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(static_cast<__half*>(base) + i) = t;
  }
}
__device__ __forceinline__ void store1(void* base, int dtype, long long i, float x) {
  if (dtype == FSB_F32) static_cast<float*>(base)[i] = x;
  else if (dtype == FSB_BF16) static_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(x);
  else static_cast<__half*>(base)[i] = __float2half_rn(x);
}

__device__ __forceinline__ void adam_math(float& p, float g, float& m, float& v, const AdamArgs& a, float gmul, bool& overflow) {
  const bool scaled_state = a.s_dtype != FSB_F32;
  g *= gmul;
  float mm = scaled_state ? m / a.optim_scale : m;
  float vv = scaled_state ? v / a.optim_scale : v;
  mm = a.beta1 * mm + (1.f - a.beta1) * g;
  vv = a.beta2 * vv + (1.f - a.beta2) * g * g;
  const float denom = (a.mode == 0) ? sqrtf(vv + a.eps) : sqrtf(vv) + a.eps;
  if (a.adamw) {
    p = p * (1.f - a.lr * a.decay) - a.step_size * (mm / denom);
  } else {
    p = p - a.step_size * (mm / denom + a.decay * p);
  }
  if (scaled_state) {
    m = mm * a.optim_scale;
    v = vv * a.optim_scale;
    if (!isfinite(__half2float(__float2half_rn(m))) || !isfinite(__half2float(__float2half_rn(v)))) overflow = true;
  } else {
    m = mm;
    v = vv;
  }
}

__global__ void __launch_bounds__(ADAM_THREADS) multi_tensor_adam_kernel(AdamArgs a) {
  if (a.noop_flag != nullptr && *a.noop_flag != 0) return;
  // locate the tensor that owns chunk blockIdx.x
  int lo = 0, hi = a.n_tensors - 1;
  const long long chunk = blockIdx.x;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (a.table[mid].chunk_start <= chunk) lo = mid; else hi = mid - 1;
  }
  const AdamTensor t = a.table[lo];
  const long long begin = (chunk - t.chunk_start) * ADAM_CHUNK;
  const long long end = min(begin + (long long)ADAM_CHUNK, t.numel);
  const float gmul = a.inv_grad_scale * (a.inv_scale_dev != nullptr ? *a.inv_scale_dev : 1.f);
  bool overflow = false;

  // 16-byte (fp32) / 8-byte (16-bit) vector path needs every base pointer aligned for 4 elements
  const auto aligned = [](const void* ptr, int dtype) {
    const uintptr_t bytes = (dtype == FSB_F32) ? 16 : 8;
    return ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) % bytes) == 0;
  };
  const bool vec = aligned(t.p, a.p_dtype) && aligned(t.g, a.g_dtype) && aligned(t.m, a.s_dtype) &&
                   aligned(t.v, a.s_dtype) && aligned(t.p_copy, a.c_dtype);
  long long i = begin + 4ll * threadIdx.x;
  if (vec) {
    for (; i + 3 < end; i += 4ll * ADAM_THREADS) {
      float p[4], g[4], m[4], v[4];
      load4(t.p, a.p_dtype, i, p);
      load4(t.g, a.g_dtype, i, g);
      load4(t.m, a.s_dtype, i, m);
      load4(t.v, a.s_dtype, i, v);
#pragma unroll
      for (int k = 0; k < 4; ++k) adam_math(p[k], g[k], m[k], v[k], a, gmul, overflow);
      store4(t.p, a.p_dtype, i, p);
      store4(t.m, a.s_dtype, i, m);
      store4(t.v, a.s_dtype, i, v);
      if (t.p_copy != nullptr) store4(t.p_copy, a.c_dtype, i, p);
    }
    // ragged tail of the chunk (at most 3 elements of the whole tensor)
    if (i < end && i + 3 >= end) {
      for (long long j = i; j < end; ++j) {
        float p = load1(t.p, a.p_dtype, j), g = load1(t.g, a.g_dtype, j), m = load1(t.m, a.s_dtype, j), v = load1(t.v, a.s_dtype, j);
        adam_math(p, g, m, v, a, gmul, overflow);
        store1(t.p, a.p_dtype, j, p); store1(t.m, a.s_dtype, j, m); store1(t.v, a.s_dtype, j, v);
        if (t.p_copy != nullptr) store1(t.p_copy, a.c_dtype, j, p);
      }
    }
  } else {
    for (long long j = begin + threadIdx.x; j < end; j += ADAM_THREADS) {
      float p = load1(t.p, a.p_dtype, j), g = load1(t.g, a.g_dtype, j), m = load1(t.m, a.s_dtype, j), v = load1(t.v, a.s_dtype, j);
      adam_math(p, g, m, v, a, gmul, overflow);
      store1(t.p, a.p_dtype, j, p); store1(t.m, a.s_dtype, j, m); store1(t.v, a.s_dtype, j, v);
      if (t.p_copy != nullptr) store1(t.p_copy, a.c_dtype, j, p);
    }
  }
  if (overflow && a.found_inf != nullptr) *a.found_inf = 1;
}

// Sum of squares of many tensors (one launch) into *out (fp32, must be zeroed by the caller).
struct NormTensor { const void* x; long long numel; long long chunk_start; long long pad_; };

__global__ void __launch_bounds__(ADAM_THREADS) multi_tensor_sumsq_kernel(const NormTensor* table, int n, int dtype, float* out) {
  __shared__ float scratch[32];
  int lo = 0, hi = n - 1;
  const long long chunk = blockIdx.x;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (table[mid].chunk_start <= chunk) lo = mid; else hi = mid - 1;
  }
  const NormTensor t = table[lo];
  const long long begin = (chunk - t.chunk_start) * ADAM_CHUNK;
  const long long end = min(begin + (long long)ADAM_CHUNK, t.numel);
  float acc = 0.f;
  for (long long j = begin + threadIdx.x; j < end; j += ADAM_THREADS) {
    const float x = load1(t.x, dtype, j);
    acc += x * x;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// x[i] *= *scale_dev (clip coefficient computed on the device), any dtype.
__global__ void __launch_bounds__(ADAM_THREADS) multi_tensor_scale_kernel(const NormTensor* table, int n, int dtype, const float* scale_dev, int* found_inf) {
  int lo = 0, hi = n - 1;
  const long long chunk = blockIdx.x;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (table[mid].chunk_start <= chunk) lo = mid; else hi = mid - 1;
  }
  const NormTensor t = table[lo];
  const long long begin = (chunk - t.chunk_start) * ADAM_CHUNK;
  const long long end = min(begin + (long long)ADAM_CHUNK, t.numel);
  const float s = *scale_dev;
  bool bad = false;
  for (long long j = begin + threadIdx.x; j < end; j += ADAM_THREADS) {
    const float x = load1(t.x, dtype, j) * s;
    if (!isfinite(x)) bad = true;
    store1(const_cast<void*>(t.x), dtype, j, x);
  }
  if (bad && found_inf != nullptr) *found_inf = 1;
}

}  // namespace fsb

FSB_API int fsb_adam_chunk_size() { return fsb::ADAM_CHUNK; }

// `table` is a device array of n_tensors records of 8 x int64:
//   {p, g, m, v, p_copy (0 = none), numel, chunk_start, 0};  total_chunks = sum ceil(numel / chunk).
FSB_API int fsb_multi_tensor_adam(const void* table, int n_tensors, long long total_chunks, int p_dtype, int g_dtype,
                                  int s_dtype, int c_dtype, float step_size, float lr, float beta1, float beta2, float eps,
                                  float grad_scale, float optim_scale, float decay, int mode, int adamw,
                                  const int* noop_flag, int* found_inf, const float* inv_scale_dev, cudaStream_t stream) {
  using namespace fsb;
  if (n_tensors <= 0 || total_chunks <= 0) return 0;
  AdamArgs a;
  a.table = static_cast<const AdamTensor*>(table);
  a.n_tensors = n_tensors;
  a.p_dtype = p_dtype; a.g_dtype = g_dtype; a.s_dtype = s_dtype; a.c_dtype = c_dtype;
  a.step_size = step_size; a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps;
  a.inv_grad_scale = 1.f / grad_scale; a.optim_scale = optim_scale; a.decay = decay;
  a.mode = mode; a.adamw = adamw;
  a.noop_flag = noop_flag; a.found_inf = found_inf; a.inv_scale_dev = inv_scale_dev;
  multi_tensor_adam_kernel<<<static_cast<unsigned>(total_chunks), ADAM_THREADS, 0, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// table records: {x, numel, chunk_start, 0}
FSB_API int fsb_multi_tensor_sumsq(const void* table, int n_tensors, long long total_chunks, int dtype, float* out,
                                   cudaStream_t stream) {
  using namespace fsb;
  if (n_tensors <= 0 || total_chunks <= 0) return 0;
  multi_tensor_sumsq_kernel<<<static_cast<unsigned>(total_chunks), ADAM_THREADS, 0, stream>>>(
      static_cast<const NormTensor*>(table), n_tensors, dtype, out);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_multi_tensor_scale(const void* table, int n_tensors, long long total_chunks, int dtype,
                                   const float* scale_dev, int* found_inf, cudaStream_t stream) {
  using namespace fsb;
  if (n_tensors <= 0 || total_chunks <= 0) return 0;
  multi_tensor_scale_kernel<<<static_cast<unsigned>(total_chunks), ADAM_THREADS, 0, stream>>>(
      static_cast<const NormTensor*>(table), n_tensors, dtype, scale_dev, found_inf);
  return static_cast<int>(cudaGetLastError());
}
