// Rotary position embedding on packed QKV, counter-based dropout, and a bounded delay kernel.
//
// * RoPE rotates the interleaved pairs (x[2i], x[2i+1]) of the q and k parts of a packed [B, S, 3, H, D] bf16 tensor
//   by the angle pos * theta^(-2i/D), in place or into a second tensor.  The backward pass is the same kernel with
//   the opposite sign of the angle, so nothing is saved.  The v part is copied (or left alone when in place).
// * Dropout draws its keep mask from Philox4x32-10 keyed by (seed, offset): element e uses counter (offset + e / 4)
//   and word e % 4.  The backward pass regenerates the mask from the same (seed, offset) instead of storing it.
// * The delay kernel keeps one CTA busy for a given number of nanoseconds (capped at one second).  Stream-ordering
//   tests use it where the reference's tests call torch.cuda._sleep
//   (tests/nn/data_parallel/test_fsdp_overlap.py:60-100 in the reference).
//
// These replace ATen elementwise kernels used by the reference's models: nn.Dropout in
// benchmarks/models/transformer_lm.py:38,55,57 and the rotary embedding a Llama-style tensor-parallel model applies
// between its ColumnParallelLinear QKV projection and attention.

#include "common.cuh"

namespace fsb {

constexpr int MISC_THREADS = 256;

__host__ inline int misc_grid(long long work_items) {
  const long long blocks = (work_items + MISC_THREADS - 1) / MISC_THREADS;
  const long long cap = 148ll * 16;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// ------------------------------------------------------------------------------------------------ RoPE
// One thread handles 8 consecutive elements (4 pairs) of one (b, s, which, h) row of D elements.
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, long long B, int S, int H, int D,
                            float log2_theta, float sign, int pos_offset) {
  const int vec_per_row = D / 8;
  const long long rows = B * S * 3 * H;
  const long long total = rows * vec_per_row;
  const float inv_d = 1.f / static_cast<float>(D);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / vec_per_row;
    const int j = static_cast<int>(i - row * vec_per_row);
    const int which = static_cast<int>((row / H) % 3);
    if (which == 2) {  // v: untouched
      if (in != out) st16(out + row * D + j * 8, ld16(in + row * D + j * 8));
      continue;
    }
    const int s = static_cast<int>((row / (3ll * H)) % S) + pos_offset;
    Vec16<__nv_bfloat16> x = ld16(in + row * D + j * 8);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int pair = j * 4 + k;  // frequency index i of the pair (2i, 2i+1)
      const float inv_freq = exp2f(-log2_theta * (2.f * static_cast<float>(pair)) * inv_d);
      float sn, cs;
      sincosf(static_cast<float>(s) * inv_freq, &sn, &cs);
      sn *= sign;
      const float x1 = __bfloat162float(x.v[2 * k]), x2 = __bfloat162float(x.v[2 * k + 1]);
      x.v[2 * k] = __float2bfloat16_rn(x1 * cs - x2 * sn);
      x.v[2 * k + 1] = __float2bfloat16_rn(x1 * sn + x2 * cs);
    }
    st16(out + row * D + j * 8, x);
  }
}

// ------------------------------------------------------------------------------------------------ dropout
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// y = keep ? x * scale : 0 with keep = (random 32-bit word >= threshold), threshold = p * 2^32.
// One thread handles 8 elements: two Philox calls (counters 2v and 2v+1 past `offset`).
__global__ void dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n, uint32_t threshold,
                               float scale, unsigned long long seed, unsigned long long offset) {
  const long long nvec = n / 8;
  const uint2 key = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    const unsigned long long c0 = offset + 2ull * static_cast<unsigned long long>(v);
    const uint4 r0 = philox4x32_10(make_uint4(static_cast<uint32_t>(c0), static_cast<uint32_t>(c0 >> 32), 0u, 0u), key);
    const uint4 r1 = philox4x32_10(make_uint4(static_cast<uint32_t>(c0 + 1), static_cast<uint32_t>((c0 + 1) >> 32), 0u, 0u), key);
    const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    Vec16<__nv_bfloat16> a = ld16(x + v * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) a.v[k] = __float2bfloat16_rn(w[k] >= threshold ? __bfloat162float(a.v[k]) * scale : 0.f);
    st16(y + v * 8, a);
  }
  // tail (n not a multiple of 8): one thread, same counter rule
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long e = nvec * 8; e < n; ++e) {
      const unsigned long long c = offset + static_cast<unsigned long long>(e / 4);
      const uint4 r = philox4x32_10(make_uint4(static_cast<uint32_t>(c), static_cast<uint32_t>(c >> 32), 0u, 0u), key);
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
      y[e] = __float2bfloat16_rn(w[e & 3] >= threshold ? __bfloat162float(x[e]) * scale : 0.f);
    }
  }
}

// ------------------------------------------------------------------------------------------------ delay
__global__ void delay_kernel(unsigned long long ns) {
  const uint64_t t0 = globaltimer_ns();
  while (globaltimer_ns() - t0 < ns) __nanosleep(500);
}

// The same with a dynamic shared-memory footprint, so that each of its CTAs keeps a whole SM from anybody else.
__global__ void delay_wide_kernel(unsigned long long ns) {
  extern __shared__ unsigned char delay_smem[];
  if (threadIdx.x == 0) delay_smem[0] = 0;
  const uint64_t t0 = globaltimer_ns();
  while (globaltimer_ns() - t0 < ns) __nanosleep(500);
}

}  // namespace fsb

// qkv_in / qkv_out: packed [B, S, 3, H, D] bf16 (may be the same pointer); D a multiple of 8.  backward != 0 applies
// the inverse rotation (the gradient of the forward).  pos_offset shifts the position of the first token.
FSB_API int fsb_rope(const void* qkv_in, void* qkv_out, long long B, int S, int H, int D, float theta, int backward, int pos_offset,
                     cudaStream_t stream) {
  using namespace fsb;
  if (B <= 0 || S <= 0 || H <= 0) return 0;
  if (D <= 0 || (D % 8) || theta <= 0.f) return -1;
  const long long total = B * S * 3 * H * (D / 8);
  rope_kernel<<<misc_grid(total), MISC_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(qkv_in),
                                                              reinterpret_cast<__nv_bfloat16*>(qkv_out), B, S, H, D, log2f(theta),
                                                              backward ? -1.f : 1.f, pos_offset);
  return static_cast<int>(cudaGetLastError());
}

// y = dropout(x) for bf16 tensors of n elements (x and y 16-byte aligned; may alias).  The same (seed, offset) gives
// the same mask, which is how the backward pass (called on the output gradient) reuses it.  A call consumes
// ceil(n / 4) Philox counters past `offset`.
FSB_API int fsb_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, unsigned long long offset,
                        cudaStream_t stream) {
  using namespace fsb;
  if (n <= 0) return 0;
  if (!(p >= 0.f) || p >= 1.f) return -1;
  const double thr = static_cast<double>(p) * 4294967296.0;
  const uint32_t threshold = thr >= 4294967295.0 ? 0xFFFFFFFFu : static_cast<uint32_t>(thr);
  dropout_kernel<<<misc_grid((n + 7) / 8), MISC_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                       reinterpret_cast<__nv_bfloat16*>(y), n, threshold,
                                                                       1.f / (1.f - p), seed, offset);
  return static_cast<int>(cudaGetLastError());
}

// Occupies the stream for `ns` nanoseconds (at most one second) with a single thread.
FSB_API int fsb_delay(unsigned long long ns, cudaStream_t stream) {
  if (ns > 1000000000ull) ns = 1000000000ull;
  fsb::delay_kernel<<<1, 1, 0, stream>>>(ns);
  return static_cast<int>(cudaGetLastError());
}

// Takes `ctas` whole SMs (200 KB of shared memory per CTA) for `ns` nanoseconds (at most one second): a stand-in for a
// foreign kernel that leaves a persistent kernel of another stream fewer SMs than its grid has CTAs.
FSB_API int fsb_delay_wide(unsigned long long ns, int ctas, cudaStream_t stream) {
  if (ns > 1000000000ull) ns = 1000000000ull;
  if (ctas < 1 || ctas > 1024) return -1;
  constexpr int kSmem = 200 * 1024;
  cudaError_t e = cudaFuncSetAttribute(fsb::delay_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return static_cast<int>(e);
  fsb::delay_wide_kernel<<<ctas, 32, kSmem, stream>>>(ns);
  return static_cast<int>(cudaGetLastError());
}
