// Small bandwidth-bound kernels: embedding gather / scatter-add, GELU, SwiGLU, casts, axpy, softmax.
// All use 16-byte accesses and grid-stride loops sized to the 148 SMs of a B200.

#include "common.cuh"

namespace fsb {

constexpr int EW_THREADS = 256;

__host__ inline int ew_grid(long long work_items) {
  const long long blocks = (work_items + EW_THREADS - 1) / EW_THREADS;
  const long long cap = 148ll * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// out[t, :] = wte[tok[t] - vocab_start, :] (+ wpe[t % seq, :]); rows outside the local vocab slice give zeros.
__global__ void embedding_fwd_kernel(const long long* __restrict__ tok, const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, long long T, int H,
                                     int seq, long long vocab_start, long long vocab_local, float scale) {
  const int nvec = H / 8;
  const long long total = T * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nvec;
    const int j = static_cast<int>(i - t * nvec);
    const long long id = tok[t] - vocab_start;
    Vec16<__nv_bfloat16> o;
    const bool mine = id >= 0 && id < vocab_local;
    if (mine) o = ld16(wte + id * H + j * 8); else o.raw = make_uint4(0, 0, 0, 0);
    if (scale != 1.f || wpe != nullptr) {
      Vec16<__nv_bfloat16> p;
      if (wpe != nullptr) p = ld16(wpe + (t % seq) * H + j * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float v = __bfloat162float(o.v[k]) * scale;
        if (wpe != nullptr) v += __bfloat162float(p.v[k]);
        o.v[k] = __float2bfloat16_rn(v);
      }
    }
    st16(out + t * H + j * 8, o);
  }
}

// dwte[tok[t]-vocab_start, :] += dout[t, :] * scale (fp32 accumulation buffer), dwpe[t % seq, :] += dout[t, :]
__global__ void embedding_bwd_kernel(const long long* __restrict__ tok, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dwte, float* __restrict__ dwpe, long long T, int H, int seq,
                                     long long vocab_start, long long vocab_local, float scale) {
  const int nvec = H / 8;
  const long long total = T * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nvec;
    const int j = static_cast<int>(i - t * nvec);
    const Vec16<__nv_bfloat16> g = ld16(dout + t * H + j * 8);
    const long long id = tok[t] - vocab_start;
    if (id >= 0 && id < vocab_local) {
      float* dst = dwte + id * H + j * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) atomicAdd(dst + k, __bfloat162float(g.v[k]) * scale);
    }
    if (dwpe != nullptr) {
      float* dst = dwpe + (t % seq) * H + j * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) atomicAdd(dst + k, __bfloat162float(g.v[k]));
    }
  }
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<TO>(to_f32<TI>(in[i]) * scale);
}

// fp32 -> bf16 with 16-byte stores (8 elements per thread)
__global__ void cast_f32_bf16_vec_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long nvec, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const float4 a = *reinterpret_cast<const float4*>(in + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(in + i * 8 + 4);
    Vec16<__nv_bfloat16> o;
    o.v[0] = __float2bfloat16_rn(a.x * scale); o.v[1] = __float2bfloat16_rn(a.y * scale);
    o.v[2] = __float2bfloat16_rn(a.z * scale); o.v[3] = __float2bfloat16_rn(a.w * scale);
    o.v[4] = __float2bfloat16_rn(b.x * scale); o.v[5] = __float2bfloat16_rn(b.y * scale);
    o.v[6] = __float2bfloat16_rn(b.z * scale); o.v[7] = __float2bfloat16_rn(b.w * scale);
    st16(out + i * 8, o);
  }
}

// acc_f32[i] = (accumulate ? acc_f32[i] : 0) + src_bf16[i] * scale   (gradient shard accumulation in master precision)
__global__ void accum_bf16_into_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ acc, long long nvec, float scale, int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const Vec16<__nv_bfloat16> s = ld16(src + i * 8);
    float4 a = make_float4(0, 0, 0, 0), b = make_float4(0, 0, 0, 0);
    if (accumulate) { a = *reinterpret_cast<float4*>(acc + i * 8); b = *reinterpret_cast<float4*>(acc + i * 8 + 4); }
    a.x += __bfloat162float(s.v[0]) * scale; a.y += __bfloat162float(s.v[1]) * scale;
    a.z += __bfloat162float(s.v[2]) * scale; a.w += __bfloat162float(s.v[3]) * scale;
    b.x += __bfloat162float(s.v[4]) * scale; b.y += __bfloat162float(s.v[5]) * scale;
    b.z += __bfloat162float(s.v[6]) * scale; b.w += __bfloat162float(s.v[7]) * scale;
    *reinterpret_cast<float4*>(acc + i * 8) = a;
    *reinterpret_cast<float4*>(acc + i * 8 + 4) = b;
  }
}

// mode 0: y = gelu(x); mode 1: dx = dy * gelu'(x)
__global__ void gelu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ out, long long nvec, int mode) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const Vec16<__nv_bfloat16> a = ld16(x + i * 8);
    Vec16<__nv_bfloat16> o;
    if (mode == 0) {
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(gelu_erf(__bfloat162float(a.v[k])));
    } else {
      const Vec16<__nv_bfloat16> d = ld16(dy + i * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(__bfloat162float(d.v[k]) * gelu_erf_grad(__bfloat162float(a.v[k])));
    }
    st16(out + i * 8, o);
  }
}

// gate_up: [rows, 2F] laid out as [gate | up]; y[rows, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ y, long long rows, int F) {
  const int nvec = F / 8;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int j = static_cast<int>(i - r * nvec);
    const Vec16<__nv_bfloat16> g = ld16(gate_up + r * 2 * F + j * 8);
    const Vec16<__nv_bfloat16> u = ld16(gate_up + r * 2 * F + F + j * 8);
    Vec16<__nv_bfloat16> o;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float a = __bfloat162float(g.v[k]);
      o.v[k] = __float2bfloat16_rn(a / (1.f + __expf(-a)) * __bfloat162float(u.v[k]));
    }
    st16(y + r * F + j * 8, o);
  }
}
// d(gate_up)[rows, 2F] from dy[rows, F]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate_up, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dgate_up, long long rows, int F) {
  const int nvec = F / 8;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int j = static_cast<int>(i - r * nvec);
    const Vec16<__nv_bfloat16> g = ld16(gate_up + r * 2 * F + j * 8);
    const Vec16<__nv_bfloat16> u = ld16(gate_up + r * 2 * F + F + j * 8);
    const Vec16<__nv_bfloat16> d = ld16(dy + r * F + j * 8);
    Vec16<__nv_bfloat16> og, ou;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float a = __bfloat162float(g.v[k]), b = __bfloat162float(u.v[k]), dd = __bfloat162float(d.v[k]);
      const float sig = 1.f / (1.f + __expf(-a));
      const float silu = a * sig;
      og.v[k] = __float2bfloat16_rn(dd * b * (sig + silu * (1.f - sig)));
      ou.v[k] = __float2bfloat16_rn(dd * silu);
    }
    st16(dgate_up + r * 2 * F + j * 8, og);
    st16(dgate_up + r * 2 * F + F + j * 8, ou);
  }
}

// y = a + b (bf16), 8 elements per thread
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const Vec16<__nv_bfloat16> x = ld16(a + i * 8), z = ld16(b + i * 8);
    Vec16<__nv_bfloat16> o;
#pragma unroll
    for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(__bfloat162float(x.v[k]) + __bfloat162float(z.v[k]));
    st16(y + i * 8, o);
  }
}

// Row softmax (fp32 math) over bf16 or fp32 rows; one CTA per row. causal_offset >= 0 masks columns
// j > (row % causal_rows) + causal_offset.
template <typename T>
__global__ void __launch_bounds__(256) softmax_kernel(const T* __restrict__ x, T* __restrict__ y, int cols, float scale, int causal_rows, int causal_offset) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * cols;
  T* yr = y + row * cols;
  int limit = cols;
  if (causal_rows > 0) limit = min(cols, static_cast<int>(row % causal_rows) + causal_offset + 1);
  float m = -INFINITY;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) m = fmaxf(m, to_f32<T>(xr[j]) * scale);
  m = block_max(m, scratch);
  float s = 0.f;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) s += __expf(to_f32<T>(xr[j]) * scale - m);
  s = block_sum(s, scratch);
  const float inv = 1.f / s;
  for (int j = threadIdx.x; j < cols; j += blockDim.x)
    yr[j] = from_f32<T>(j < limit ? __expf(to_f32<T>(xr[j]) * scale - m) * inv : 0.f);
}

}  // namespace fsb

FSB_API int fsb_embedding_fwd(const long long* tok, const void* wte, const void* wpe, void* out, long long T, int H, int seq,
                              long long vocab_start, long long vocab_local, float scale, cudaStream_t stream) {
  using namespace fsb;
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  embedding_fwd_kernel<<<ew_grid(T * (H / 8)), EW_THREADS, 0, stream>>>(tok, static_cast<const __nv_bfloat16*>(wte),
      static_cast<const __nv_bfloat16*>(wpe), static_cast<__nv_bfloat16*>(out), T, H, seq > 0 ? seq : 1, vocab_start, vocab_local, scale);
  return static_cast<int>(cudaGetLastError());
}

// dwte / dwpe: zero-initialised fp32 accumulation buffers ([vocab_local, H] / [seq, H]; dwpe may be null)
FSB_API int fsb_embedding_bwd(const long long* tok, const void* dout, float* dwte, float* dwpe, long long T, int H, int seq,
                              long long vocab_start, long long vocab_local, float scale, cudaStream_t stream) {
  using namespace fsb;
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  embedding_bwd_kernel<<<ew_grid(T * (H / 8)), EW_THREADS, 0, stream>>>(tok, static_cast<const __nv_bfloat16*>(dout), dwte, dwpe, T, H,
                                                                         seq > 0 ? seq : 1, vocab_start, vocab_local, scale);
  return static_cast<int>(cudaGetLastError());
}

// out[i] = in[i] * scale with dtype conversion. dtype codes: 0 fp32, 1 fp16, 2 bf16.
FSB_API int fsb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, float scale, cudaStream_t stream) {
  using namespace fsb;
  if (n <= 0) return 0;
  const int grid = ew_grid(n / 4 + 1);
  if (in_dtype == FSB_F32 && out_dtype == FSB_BF16 && n % 8 == 0 && (reinterpret_cast<uintptr_t>(in) % 16 == 0) &&
      (reinterpret_cast<uintptr_t>(out) % 16 == 0)) {
    cast_f32_bf16_vec_kernel<<<ew_grid(n / 8), EW_THREADS, 0, stream>>>(static_cast<const float*>(in), static_cast<__nv_bfloat16*>(out), n / 8, scale);
  }
#define FSB_CAST_CASE(IC, IT, OC, OT) \
  else if (in_dtype == IC && out_dtype == OC) cast_kernel<IT, OT><<<grid, EW_THREADS, 0, stream>>>(static_cast<const IT*>(in), static_cast<OT*>(out), n, scale);
  FSB_CAST_CASE(FSB_F32, float, FSB_BF16, __nv_bfloat16)
  FSB_CAST_CASE(FSB_F32, float, FSB_F16, __half)
  FSB_CAST_CASE(FSB_F32, float, FSB_F32, float)
  FSB_CAST_CASE(FSB_BF16, __nv_bfloat16, FSB_F32, float)
  FSB_CAST_CASE(FSB_F16, __half, FSB_F32, float)
  FSB_CAST_CASE(FSB_BF16, __nv_bfloat16, FSB_BF16, __nv_bfloat16)
  FSB_CAST_CASE(FSB_F16, __half, FSB_F16, __half)
#undef FSB_CAST_CASE
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_accum_bf16_into_f32(const void* src, float* acc, long long n, float scale, int accumulate, cudaStream_t stream) {
  using namespace fsb;
  if (n <= 0) return 0;
  if (n % 8 != 0) return -1;
  accum_bf16_into_f32_kernel<<<ew_grid(n / 8), EW_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), acc, n / 8, scale, accumulate);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_gelu(const void* x, const void* dy, void* out, long long n, int backward, cudaStream_t stream) {
  using namespace fsb;
  if (n <= 0) return 0;
  if (n % 8 != 0) return -1;
  gelu_kernel<<<ew_grid(n / 8), EW_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
                                                         static_cast<__nv_bfloat16*>(out), n / 8, backward);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_swiglu_fwd(const void* gate_up, void* y, long long rows, int F, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (F % 8 != 0) return -1;
  swiglu_fwd_kernel<<<ew_grid(rows * (F / 8)), EW_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(y), rows, F);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_swiglu_bwd(const void* gate_up, const void* dy, void* dgate_up, long long rows, int F, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (F % 8 != 0) return -1;
  swiglu_bwd_kernel<<<ew_grid(rows * (F / 8)), EW_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(gate_up), static_cast<const __nv_bfloat16*>(dy),
                                                                         static_cast<__nv_bfloat16*>(dgate_up), rows, F);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_add_bf16(const void* a, const void* b, void* y, long long n, cudaStream_t stream) {
  using namespace fsb;
  if (n <= 0) return 0;
  if (n % 8 != 0) return -1;
  add_kernel<<<ew_grid(n / 8), EW_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
                                                        static_cast<__nv_bfloat16*>(y), n / 8);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_softmax(const void* x, void* y, long long rows, int cols, int dtype, float scale, int causal_rows, int causal_offset,
                        cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (dtype == FSB_F32) softmax_kernel<float><<<static_cast<unsigned>(rows), 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), cols, scale, causal_rows, causal_offset);
  else if (dtype == FSB_BF16) softmax_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), cols, scale, causal_rows, causal_offset);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}
