// Collectives over NVLink 5 / NVSwitch peer memory, issued from inside the kernels (no NCCL).
//
// Every rank owns a "symmetric" buffer that all peers have mapped; a kernel receives the table of peer
// pointers and moves data with plain 16-byte loads / stores over NVLink.  Synchronisation between GPUs uses
// one 32-bit flag per (channel, source rank) in a symmetric signal pad: a rank publishes the call's epoch to
// every peer with st.release.sys and polls its own pad with ld.acquire.sys.  Each collective is ONE kernel:
//
//   entry barrier (peers' inputs are ready)  ->  pull / push over NVLink  ->  exit barrier (peers are done
//   with my buffer), so that in-stream ordering on every GPU is enough for the callers.
//
// All polls are bounded: after the wait limit (fsb_comm_set_timeout_ms, default 30 s) without progress the kernel writes FSB_ERR_WAIT_TIMEOUT to its
// status word and returns; the host raises.  No TMA cluster multicast is used anywhere; remote data is read
// with ordinary loads (L1-bypassing) by the CTA that needs it.
//
// These kernels replace the c10d calls of the reference: _all_gather_base / _reduce_scatter_base
// (fairscale/nn/data_parallel/fully_sharded_data_parallel.py:2032-2037,
// fairscale/internal/reduce_scatter_bucketer.py:38-45), all_reduce (nn/model_parallel/mappings.py:42) and
// all_to_all_single (nn/moe/moe_layer.py:29), and fuse the element-wise work that follows them
// (pre/post-divide, fp32 cast, gradient accumulation; MoE slot scatter / weighted combine).

#include "comm_dev.cuh"

#include <cstdlib>

namespace fsb {

// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS) barrier_kernel(CommCtx c) {
  signal_peers(c, c.channel);
  wait_peers(c, c.channel);
}

// out[p * n16 + i] = src_p[i] for every rank p; src pointers address each rank's shard (16-byte units)

// d[i] = s[i] for i in [0, n16): grid-strided, COMM_UNROLL loads in flight per thread before the first store
__device__ __forceinline__ void copy_peer16(uint4* __restrict__ d, const uint4* __restrict__ s, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + (COMM_UNROLL - 1) * stride < n16; i += COMM_UNROLL * stride) {
    uint4 v[COMM_UNROLL];
#pragma unroll
    for (int u = 0; u < COMM_UNROLL; ++u) v[u] = ld_peer16(s + i + u * stride);
#pragma unroll
    for (int u = 0; u < COMM_UNROLL; ++u) d[i + u * stride] = v[u];
  }
  for (; i < n16; i += stride) d[i] = ld_peer16(s + i);
}

__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM)
all_gather_kernel(CommCtx c, PtrTable src, uint4* __restrict__ out, long long n16) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);
  if (!wait_peers(c, c.channel)) return;
  for (int k = 0; k < c.world; ++k) {
    const int p = (c.rank + k) % c.world;  // start with the local shard, then walk the ring
    copy_peer16(out + static_cast<long long>(p) * n16, reinterpret_cast<const uint4*>(src.p[p]), n16);
  }
  exit_barrier(c, c.channel + 1);
}

// Column-interleaved all-gather: every rank holds src_p [rows, cols16] (16-byte units); out is [rows, world * cols16] and
// receives rank p's rows in columns [p * cols16, (p + 1) * cols16): the layout of a gather along the last dimension,
// written directly (no all-gather into a leading axis followed by a transposing copy).
__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM)
all_gather_cols_kernel(CommCtx c, PtrTable src, uint4* __restrict__ out, long long rows, int cols16) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);
  if (!wait_peers(c, c.channel)) return;
  const long long per_rank = rows * cols16;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long out_ld = static_cast<long long>(c.world) * cols16;
  for (int k = 0; k < c.world; ++k) {
    const int p = (c.rank + k) % c.world;
    const uint4* s = reinterpret_cast<const uint4*>(src.p[p]);
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + (COMM_UNROLL - 1) * stride < per_rank; i += COMM_UNROLL * stride) {
      uint4 v[COMM_UNROLL];
#pragma unroll
      for (int u = 0; u < COMM_UNROLL; ++u) v[u] = ld_peer16(s + i + u * stride);
#pragma unroll
      for (int u = 0; u < COMM_UNROLL; ++u) {
        const long long e = i + u * stride, r = e / cols16;
        out[r * out_ld + static_cast<long long>(p) * cols16 + (e - r * cols16)] = v[u];
      }
    }
    for (; i < per_rank; i += stride) {
      const long long r = i / cols16;
      out[r * out_ld + static_cast<long long>(p) * cols16 + (i - r * cols16)] = ld_peer16(s + i);
    }
  }
  exit_barrier(c, c.channel + 1);
}

// out[p-th chunk] = src_p[my chunk]: equal-split all-to-all, chunk = n16 16-byte units
__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM)
all_to_all_kernel(CommCtx c, PtrTable src, uint4* __restrict__ out, long long n16) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);
  if (!wait_peers(c, c.channel)) return;
  for (int k = 0; k < c.world; ++k) {
    const int p = (c.rank + k) % c.world;
    copy_peer16(out + static_cast<long long>(p) * n16, reinterpret_cast<const uint4*>(src.p[p]) + static_cast<long long>(c.rank) * n16, n16);
  }
  exit_barrier(c, c.channel + 1);
}

template <typename T> struct Acc8;  // 16 bytes of T accumulated in fp32
template <> struct Acc8<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void add(float (&a)[8], const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { a[2 * i] += __low2float(h[i]); a[2 * i + 1] += __high2float(h[i]); }
  }
};
template <> struct Acc8<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void add(float (&a)[8], const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { a[2 * i] += __low2float(h[i]); a[2 * i + 1] += __high2float(h[i]); }
  }
};
template <> struct Acc8<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void add(float (&a)[8], const uint4& v) {
    const float* f = reinterpret_cast<const float*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] += f[i];
  }
};

// Reduce-scatter with fused scale / cast / accumulate:
//   out[i] = (accumulate ? out[i] : 0) + scale * sum_p src_p[rank * n + i]
// TI: gradient dtype in the peers' buffers; TO: output dtype (fp32 master-precision shard or TI).
template <typename TI, typename TO>
__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM)
reduce_scatter_kernel(CommCtx c, PtrTable src, TO* __restrict__ out, long long n, float scale, int accumulate, long long base,
                      int active) {
  // `base`: first element of the slice this rank sums (rank * n for a reduce-scatter, 0 for a reduction of the whole
  // buffer to one owner); `active` == 0: this rank only takes part in the two barriers (it is not the owner).
  if (blockIdx.x == 0) signal_peers(c, c.channel);
  if (!wait_peers(c, c.channel)) return;
  constexpr int E = Acc8<TI>::N;
  const long long nvec = active ? n / E : 0;
  if (!active) n = 0;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // two ranks: two vectors per thread and pass, so that a thread still has four peer loads in flight
  if (c.world <= 2) {
    for (; i + stride < nvec; i += 2 * stride) {
      uint4 v[2][2];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (q < c.world) v[u][q] = ld_peer16(reinterpret_cast<const TI*>(src.p[q]) + base + (i + u * stride) * E);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (q < c.world) Acc8<TI>::add(a, v[u][q]);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          float r = a[e] * scale;
          TO* o = out + (i + u * stride) * E + e;
          if (accumulate) r += to_f32<TO>(*o);
          *o = from_f32<TO>(r);
        }
      }
    }
  }
  for (; i < nvec; i += stride) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // peers in groups of COMM_UNROLL (their loads in flight together); fixed summation order (rank 0, 1, ...), so the
    // result does not depend on timing
#pragma unroll
    for (int g = 0; g < kMaxRanks; g += COMM_UNROLL) {
      if (g < c.world) {
        uint4 v[COMM_UNROLL];
#pragma unroll
        for (int q = 0; q < COMM_UNROLL; ++q)
          if (g + q < c.world) v[q] = ld_peer16(reinterpret_cast<const TI*>(src.p[g + q]) + base + i * E);
#pragma unroll
        for (int q = 0; q < COMM_UNROLL; ++q)
          if (g + q < c.world) Acc8<TI>::add(a, v[q]);
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      float r = a[e] * scale;
      TO* o = out + i * E + e;
      if (accumulate) r += to_f32<TO>(*o);
      *o = from_f32<TO>(r);
    }
  }
  // ragged tail (n not a multiple of the vector width)
  for (long long i = nvec * E + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float a = 0.f;
    for (int q = 0; q < c.world; ++q) a += to_f32<TI>(reinterpret_cast<const TI*>(src.p[q])[base + i]);
    float r = a * scale;
    if (accumulate) r += to_f32<TO>(out[i]);
    out[i] = from_f32<TO>(r);
  }
  exit_barrier(c, c.channel + 1);
}

// The summation half of the copy-engine reduce-scatter: every addend already lies in this GPU's memory (src.p[q], q in rank
// order: the own slice where the gradient was produced, the peers' slices where the copy engines put them).
//   out[i] = (accumulate ? out[i] : 0) + scale * sum_q src_q[i]         (fp32 sum, fixed order: bitwise what the pull kernel gives)
template <typename TI, typename TO>
__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM)
local_sum_kernel(PtrTable src, int world, TO* __restrict__ out, long long n, float scale, int accumulate) {
  constexpr int E = Acc8<TI>::N;
  const long long nvec = n / E;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int g = 0; g < kMaxRanks; g += COMM_UNROLL) {
      if (g < world) {
        uint4 v[COMM_UNROLL];
#pragma unroll
        for (int q = 0; q < COMM_UNROLL; ++q)
          if (g + q < world) v[q] = ld_peer16(reinterpret_cast<const TI*>(src.p[g + q]) + i * E);
#pragma unroll
        for (int q = 0; q < COMM_UNROLL; ++q)
          if (g + q < world) Acc8<TI>::add(a, v[q]);
      }
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      float r = a[e] * scale;
      TO* o = out + i * E + e;
      if (accumulate) r += to_f32<TO>(*o);
      *o = from_f32<TO>(r);
    }
  }
  for (long long i = nvec * E + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float a = 0.f;
    for (int q = 0; q < world; ++q) a += to_f32<TI>(reinterpret_cast<const TI*>(src.p[q])[i]);
    float r = a * scale;
    if (accumulate) r += to_f32<TO>(out[i]);
    out[i] = from_f32<TO>(r);
  }
}

// ------------------------------------------------------------------------------------------------
// Reduce-scatter fused with the sharded Adam update (the gradient shard never exists in memory):
//   g[i]  = scale * sum_p src_p[rank * n + i]                      (fp32, fixed summation order)
//   m, v, p updated as in the multi-tensor Adam kernel (adam.cu) on this rank's fp32 master shard,
//   p_copy[i] = bf16 / fp16 (p[i])   written into the symmetric heap, where the next all-gather reads it.
// Side outputs: *gnorm_sq += sum g^2 (for logging / a later clip of the *next* step), *found_inf = 1 on a non-finite g.
// The exit barrier also covers p_copy: no peer reads the new shard before every rank has left the kernel.
// ------------------------------------------------------------------------------------------------
struct AdamHyper {
  float step_size, lr, beta1, beta2, eps, decay;
  int eps_inside_sqrt, adamw;
};

__device__ __forceinline__ void adam_update(float& p, float g, float& m, float& v, const AdamHyper& h) {
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float denom = h.eps_inside_sqrt ? sqrtf(v + h.eps) : sqrtf(v) + h.eps;
  if (h.adamw) p = p * (1.f - h.lr * h.decay) - h.step_size * (m / denom);
  else         p = p - h.step_size * (m / denom + h.decay * p);
}

template <typename TI, typename TC>
__global__ void __launch_bounds__(COMM_THREADS, 8)
reduce_scatter_adam_kernel(CommCtx c, PtrTable src, long long n, float scale, float* __restrict__ p, float* __restrict__ m,
                           float* __restrict__ v, TC* __restrict__ p_copy, AdamHyper h, float* gnorm_sq, int* found_inf) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);
  if (!wait_peers(c, c.channel)) return;
  constexpr int E = Acc8<TI>::N;
  const long long nvec = n / E;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long base = static_cast<long long>(c.rank) * n;
  float sq = 0.f;
  bool bad = false;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int grp = 0; grp < kMaxRanks; grp += COMM_UNROLL) {
      if (grp < c.world) {
        uint4 ld[COMM_UNROLL];
#pragma unroll
        for (int q = 0; q < COMM_UNROLL; ++q)
          if (grp + q < c.world) ld[q] = ld_peer16(reinterpret_cast<const TI*>(src.p[grp + q]) + base + i * E);
#pragma unroll
        for (int q = 0; q < COMM_UNROLL; ++q)
          if (grp + q < c.world) Acc8<TI>::add(g, ld[q]);
      }
    }
#pragma unroll
    for (int half = 0; half < E / 4; ++half) {
      const long long o = i * E + half * 4;
      float4 pp = *reinterpret_cast<const float4*>(p + o), mm = *reinterpret_cast<const float4*>(m + o),
             vv = *reinterpret_cast<const float4*>(v + o);
      float pa[4] = {pp.x, pp.y, pp.z, pp.w}, ma[4] = {mm.x, mm.y, mm.z, mm.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = g[half * 4 + k] * scale;
        sq += gk * gk;
        bad |= !isfinite(gk);
        adam_update(pa[k], gk, ma[k], va[k], h);
      }
      *reinterpret_cast<float4*>(p + o) = make_float4(pa[0], pa[1], pa[2], pa[3]);
      *reinterpret_cast<float4*>(m + o) = make_float4(ma[0], ma[1], ma[2], ma[3]);
      *reinterpret_cast<float4*>(v + o) = make_float4(va[0], va[1], va[2], va[3]);
      if (p_copy != nullptr) {
        TC lo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) lo[k] = from_f32<TC>(pa[k]);
        *reinterpret_cast<uint2*>(p_copy + o) = *reinterpret_cast<const uint2*>(lo);  // 8-byte store (o is a multiple of 4)
      }
    }
  }
  for (long long i = nvec * E + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    float gk = 0.f;
    for (int q = 0; q < c.world; ++q) gk += to_f32<TI>(reinterpret_cast<const TI*>(src.p[q])[base + i]);
    gk *= scale;
    sq += gk * gk;
    bad |= !isfinite(gk);
    float pk = p[i], mk = m[i], vk = v[i];
    adam_update(pk, gk, mk, vk, h);
    p[i] = pk; m[i] = mk; v[i] = vk;
    if (p_copy != nullptr) p_copy[i] = from_f32<TC>(pk);
  }
  if (gnorm_sq != nullptr) {
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) atomicAdd(gnorm_sq, sq);
  }
  if (bad && found_inf != nullptr) *found_inf = 1;
  exit_barrier(c, c.channel + 1);
}

// In-place all-reduce (sum) of every rank's symmetric buffer of n elements, two-shot:
// reduce my chunk from all peers into my buffer, cross-GPU barrier, then pull the other chunks from their owners.
// The grid must be fully resident (its CTAs wait for one another).
template <typename T>
__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM) all_reduce_kernel(CommCtx c, PtrTable bufs, long long n) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);
  if (!wait_peers(c, c.channel)) return;
  constexpr int E = Acc8<T>::N;
  const long long chunk = ((n / E + c.world - 1) / c.world);  // vectors per chunk
  const long long nvec = n / E;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  T* mine = reinterpret_cast<T*>(const_cast<void*>(bufs.p[c.rank]));
  const long long lo = min(static_cast<long long>(c.rank) * chunk, nvec), hi = min(lo + chunk, nvec);
  for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi; i += stride) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int q = 0; q < kMaxRanks; ++q)
      if (q < c.world) Acc8<T>::add(a, ld_peer16(reinterpret_cast<const T*>(bufs.p[q]) + i * E));
    T r[8];
#pragma unroll
    for (int e = 0; e < E; ++e) r[e] = from_f32<T>(a[e]);
    *reinterpret_cast<uint4*>(mine + i * E) = *reinterpret_cast<const uint4*>(r);
  }
  // elements past the last full vector are reduced by rank 0 and fetched by the others below
  if (c.rank == 0) {
    for (long long i = nvec * E + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
      float a = 0.f;
      for (int q = 0; q < c.world; ++q) a += to_f32<T>(reinterpret_cast<const T*>(bufs.p[q])[i]);
      mine[i] = from_f32<T>(a);
    }
  }
  exit_barrier(c, c.channel + 1);  // every rank's chunk is final and nobody still reads stale chunks
  // all CTAs must observe the barrier that the last CTA completed: spin on the pad (monotonic epochs)
  if (!wait_peers(c, c.channel + 1)) return;
  for (int k = 1; k < c.world; ++k) {
    const int p = (c.rank + k) % c.world;
    const long long plo = min(static_cast<long long>(p) * chunk, nvec), phi = min(plo + chunk, nvec);
    const T* s = reinterpret_cast<const T*>(bufs.p[p]);
    for (long long i = plo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < phi; i += stride)
      *reinterpret_cast<uint4*>(mine + i * E) = ld_peer16(s + i * E);
  }
  if (c.rank != 0) {
    const T* s = reinterpret_cast<const T*>(bufs.p[0]);
    for (long long i = nvec * E + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) mine[i] = s[i];
  }
  exit_barrier(c, c.channel + 2);
}

// ------------------------------------------------------------------------------------------------
// MoE routing over peer memory.
// scatter: row t of `x` [T, M] is stored (scaled by w[t] if given) into row dst_row[t] of rank dst_rank[t]'s
//          buffer (remote 16-byte stores); rows with dst_rank < 0 are dropped.
// gather : out[t] (+)= w[t] * row src_row[t] of rank src_rank[t]'s buffer (remote loads).
// One warp moves one row; M % 8 == 0 (bf16).
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(COMM_THREADS, COMM_MIN_CTAS_PER_SM) moe_scatter_rows_kernel(CommCtx c, PtrTable dst, const __nv_bfloat16* __restrict__ x,
                                                                        const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                                                                        const float* __restrict__ w, long long T, int rows_per_token, int M,
                                                                        const int* __restrict__ counts, int E, int C, int n_local) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);  // destinations are zeroed / free
  if (!wait_peers(c, c.channel)) return;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long t = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    const int r = dst_rank[t];
    if (r < 0) continue;
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dst.p[r])) + static_cast<long long>(dst_row[t]) * M;
    const __nv_bfloat16* s = x + (t / rows_per_token) * M;
    const float scale = (w != nullptr) ? w[t] : 1.f;
    for (int j = lane * 8; j < M; j += 256) {
      Vec16<__nv_bfloat16> v = ld16(s + j);
      if (w != nullptr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v.v[k] = __float2bfloat16_rn(__bfloat162float(v.v[k]) * scale);
      }
      st16(d + j, v);
    }
  }
  // Rows that no token of this rank claimed: expert e took slots [0, counts[e] + counts[E + e]) of this rank's C-row
  // segment in its owner's buffer (first choices, then second choices); the rest of the segment is zeroed here, so the
  // owner needs no separate pass over its whole landing buffer.
  if (counts != nullptr) {
    Vec16<__nv_bfloat16> z;
#pragma unroll
    for (int k = 0; k < 8; ++k) z.v[k] = __float2bfloat16_rn(0.f);
    const long long rows = static_cast<long long>(E) * C;
    for (long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; idx < rows; idx += warps) {
      const int e = static_cast<int>(idx / C), slot = static_cast<int>(idx % C);
      if (slot < counts[e] + counts[E + e]) continue;
      const long long row = static_cast<long long>(e % n_local) * (static_cast<long long>(c.world) * C) + static_cast<long long>(c.rank) * C + slot;
      __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(dst.p[e / n_local])) + row * M;
      for (int j = lane * 8; j < M; j += 256) st16(d + j, z);
    }
  }
  exit_barrier(c, c.channel + 1);  // all rows of all ranks have landed
}

// out[token] = sum over its `rows_per_token` routes of w[t] * peer_row(t); dot[t] (optional) = <peer_row(t), g[token]>
__global__ void __launch_bounds__(COMM_THREADS, 8) moe_gather_rows_kernel(CommCtx c, PtrTable src, __nv_bfloat16* __restrict__ out,
                                                                       const int* __restrict__ src_rank, const int* __restrict__ src_row,
                                                                       const float* __restrict__ w, const __nv_bfloat16* __restrict__ g,
                                                                       float* __restrict__ dot, long long tokens, int rows_per_token, int M) {
  if (blockIdx.x == 0) signal_peers(c, c.channel);  // sources are complete
  if (!wait_peers(c, c.channel)) return;
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long tok = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; tok < tokens; tok += warps) {
    float dots[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = lane * 8; j < M; j += 256) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      Vec16<__nv_bfloat16> gv;
      if (g != nullptr) gv = ld16(g + tok * M + j);
      for (int k = 0; k < rows_per_token && k < 4; ++k) {
        const long long t = tok * rows_per_token + k;
        const int r = src_rank[t];
        if (r < 0) continue;
        const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + static_cast<long long>(src_row[t]) * M + j;
        Vec16<__nv_bfloat16> v;
        v.raw = ld_peer16(s);
        const float wt = (w != nullptr) ? w[t] : 1.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float f = __bfloat162float(v.v[e]);
          acc[e] += wt * f;
          if (g != nullptr) dots[k] += f * __bfloat162float(gv.v[e]);
        }
      }
      if (out != nullptr) {
        Vec16<__nv_bfloat16> o;
#pragma unroll
        for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16_rn(acc[e]);
        st16(out + tok * M + j, o);
      }
    }
    if (dot != nullptr) {
      for (int k = 0; k < rows_per_token && k < 4; ++k) {
        const float d = warp_sum(dots[k]);
        if (lane == 0) dot[tok * rows_per_token + k] = d;
      }
    }
  }
  exit_barrier(c, c.channel + 1);  // peers may reuse their buffers
}

}  // namespace fsb

// ------------------------------------------------------------------------------------------------
// C ABI. `pads` / `ptrs`: host arrays of `world` device pointers (peer-mapped). `counter`: zeroed device uint.
// dtype codes: 0 fp32, 1 fp16, 2 bf16. All data pointers 16-byte aligned.
// ------------------------------------------------------------------------------------------------
static fsb::CommCtx make_ctx(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, int* status) {
  fsb::CommCtx c{};
  c.rank = rank; c.world = world; c.epoch = epoch; c.channel = channel;
  for (int i = 0; i < world && i < fsb::kMaxRanks; ++i) c.pads[i] = static_cast<uint32_t*>(pads[i]);
  c.counter = static_cast<unsigned int*>(counter);
  c.status = status;
  c.wait_ns = fsb_host::comm_wait_ns();
  return c;
}
static fsb::PtrTable make_table(void* const* ptrs, int world) {
  fsb::PtrTable t{};
  for (int i = 0; i < world && i < fsb::kMaxRanks; ++i) t.p[i] = ptrs[i];
  return t;
}
// FSB_COMM_MAX_CTAS overrides the CTA cap of the streaming collectives (default: one 128-thread CTA per SM, so that two
// collectives running on different streams still leave room for a persistent GEMM CTA on every SM).
// Collectives that sit on the critical path of their layer (MoE dispatch / combine, all-to-all, the column gather of a
// tensor-parallel output) have nothing to share the SMs with: eight CTAs per SM instead of one.
constexpr int kWideGrid = 148 * 8;
static int comm_grid(long long work_items, int max_blocks) {
  static int cap = -1;
  if (cap < 0) {
    const char* e = getenv("FSB_COMM_MAX_CTAS");
    cap = (e != nullptr && atoi(e) > 0) ? atoi(e) : 0;
  }
  if (cap > 0 && max_blocks != kWideGrid) max_blocks = cap;
  long long b = (work_items + fsb::COMM_THREADS - 1) / fsb::COMM_THREADS;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

FSB_API int fsb_comm_max_ranks() { return fsb::kMaxRanks; }

// Limit of one device-side wait for a peer, for every collective launched from now on (milliseconds; default 30 s).
FSB_API int fsb_comm_set_timeout_ms(long long ms) {
  if (ms <= 0) return -1;
  fsb_host::comm_wait_ns() = static_cast<unsigned long long>(ms) * 1000000ull;
  return 0;
}
FSB_API long long fsb_comm_get_timeout_ms() { return static_cast<long long>(fsb_host::comm_wait_ns() / 1000000ull); }

FSB_API int fsb_comm_barrier(int rank, int world, unsigned epoch, int channel, void* const* pads, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks) return -1;
  fsb::barrier_kernel<<<1, fsb::COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch, channel, pads, nullptr, status));
  return static_cast<int>(cudaGetLastError());
}

// out[world * nbytes] <- every rank's shard (src[p], nbytes each, multiple of 16)
FSB_API int fsb_comm_all_gather(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, void* const* src,
                                void* out, long long nbytes, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks || nbytes % 16) return -1;
  const long long n16 = nbytes / 16;
  fsb::all_gather_kernel<<<comm_grid(n16, 148), fsb::COMM_THREADS, 0, stream>>>(
      make_ctx(rank, world, epoch, channel, pads, counter, status), make_table(src, world), static_cast<uint4*>(out), n16);
  return static_cast<int>(cudaGetLastError());
}

// The same all-gather with the payload moved by the copy engines: flag barrier (peers' shards are final) -> one
// cudaMemcpyAsync per peer from its mapped shard -> flag barrier (peers are done reading mine).  No SM takes part in the
// transfer, so kernels of other streams keep the whole GPU; the price is world + 1 enqueues instead of one.
// Uses epochs `epoch` (entry) and `epoch + 1` (exit) on `channel`: the caller advances its epoch by two.
FSB_API int fsb_comm_all_gather_dma(int rank, int world, unsigned epoch, int channel, void* const* pads, void* const* src, void* out,
                                    long long nbytes, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks) return -1;
  fsb::barrier_kernel<<<1, fsb::COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch, channel, pads, nullptr, status));
  for (int k = 0; k < world; ++k) {
    const int p = (rank + k) % world;  // own shard first, then the ring: the peers' copy engines start on different sources
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(out) + static_cast<long long>(p) * nbytes, src[p], static_cast<size_t>(nbytes),
                                    cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  fsb::barrier_kernel<<<1, fsb::COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch + 1u, channel, pads, nullptr, status));
  return static_cast<int>(cudaGetLastError());
}

// out[rows, world * row_bytes] <- every rank's [rows, row_bytes] tensor, rank p in byte columns [p * row_bytes, ...)
FSB_API int fsb_comm_all_gather_cols(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                                     void* const* src, void* out, long long rows, long long row_bytes, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks || row_bytes % 16 || row_bytes / 16 > 0x7fffffff) return -1;
  const int cols16 = static_cast<int>(row_bytes / 16);
  fsb::all_gather_cols_kernel<<<comm_grid(rows * cols16, kWideGrid), fsb::COMM_THREADS, 0, stream>>>(
      make_ctx(rank, world, epoch, channel, pads, counter, status), make_table(src, world), static_cast<uint4*>(out), rows, cols16);
  return static_cast<int>(cudaGetLastError());
}

// Partial all-gather on the copy engines: byte ranges [lo[i], hi[i]) of the gathered buffer (`world` shards of
// `shard_bytes`) are fetched from the shards that hold them, behind one flag barrier (peers' shards are final).  There is
// no exit barrier: the caller must run a full collective on the same shards (which has one) before any shard changes.
FSB_API int fsb_comm_gather_ranges_dma(int rank, int world, unsigned epoch, int channel, void* const* pads, void* const* src, void* out,
                                       long long shard_bytes, int n_ranges, const long long* lo, const long long* hi, int* status,
                                       cudaStream_t stream) {
  if (world > fsb::kMaxRanks || shard_bytes <= 0) return -1;
  fsb::barrier_kernel<<<1, fsb::COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch, channel, pads, nullptr, status));
  for (int i = 0; i < n_ranges; ++i) {
    long long a = lo[i];
    while (a < hi[i]) {
      const long long p = a / shard_bytes;
      if (p >= world) return -1;
      const long long end = (p + 1) * shard_bytes < hi[i] ? (p + 1) * shard_bytes : hi[i];
      cudaError_t e = cudaMemcpyAsync(static_cast<char*>(out) + a, static_cast<const char*>(src[p]) + (a - p * shard_bytes),
                                      static_cast<size_t>(end - a), cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) return static_cast<int>(e);
      a = end;
    }
  }
  return static_cast<int>(cudaGetLastError());
}

// Stream-ordered 32-bit store by the driver (no kernel, no SM): cuStreamWriteValue32, looked up once.
using stream_write_fn = int (*)(cudaStream_t, unsigned long long, unsigned int, unsigned int);
static stream_write_fn stream_write_entry() {
  static stream_write_fn fn = []() -> stream_write_fn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<stream_write_fn>(f);
  }();
  return fn;
}

FSB_API int fsb_comm_stream_memops_available() { return stream_write_entry() != nullptr ? 1 : 0; }

// The copies of an all-gather, reporting their progress to a consumer that runs concurrently.  Bytes [prio_lo, prio_hi) of
// the gathered buffer go first, in pieces of `piece_bytes`; after piece i is in place flags[i] = flag_value is stored in
// stream order by the driver.  The rest of the buffer follows.
//
// Two phases, because only copies from a PEER are certain to run on a copy engine: a copy within this GPU's own memory
// made no progress while a persistent kernel that fills every SM was waiting for it.
//   phase 0 - the part of [prio_lo, prio_hi) that lies in this rank's own shard.  Enqueue it on the consumer's stream,
//             before the consumer.
//   phase 1 - on a side stream that waits for phase 0: the peers' parts of [prio_lo, prio_hi) with one flag store per
//             piece (cyclically from piece `first_piece` on, flags in sending order), then the peers' parts of the rest, then the rest of the own shard (which may have to wait for the
//             consumer to leave the SMs).  Nothing the consumer waits for needs an SM.
// The caller brackets the two calls with barriers (peers' shards final before / peers done reading after) on the
// consumer's stream.  Returns -2 without stream memory operations.
FSB_API int fsb_comm_gather_flagged_copies(int rank, int world, int phase, void* const* src, void* out, long long shard_bytes,
                                           long long prio_lo, long long prio_hi, long long piece_bytes, int first_piece,
                                           unsigned int* flags, unsigned int flag_value, cudaStream_t stream) {
  const long long total = shard_bytes * world;
  if (world > fsb::kMaxRanks || rank < 0 || rank >= world || shard_bytes <= 0 || piece_bytes <= 0 || prio_lo < 0 || prio_hi > total ||
      prio_lo > prio_hi || first_piece < 0)
    return -1;
  const stream_write_fn write_u32 = stream_write_entry();
  if (write_u32 == nullptr) return -2;
  // copies the part of [a, b) held by the peers (own == false) or by this rank (own == true)
  auto copy_range = [&](long long a, long long b, bool own) -> cudaError_t {
    while (a < b) {
      const long long p = a / shard_bytes;
      const long long end = (p + 1) * shard_bytes < b ? (p + 1) * shard_bytes : b;
      if ((p == rank) == own) {
        cudaError_t e = cudaMemcpyAsync(static_cast<char*>(out) + a, static_cast<const char*>(src[p]) + (a - p * shard_bytes),
                                        static_cast<size_t>(end - a), cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) return e;
      }
      a = end;
    }
    return cudaSuccess;
  };
  if (phase == 0) return static_cast<int>(copy_range(prio_lo, prio_hi, true));
  // pieces go out cyclically from `first_piece` on (ranks start at different pieces: they would otherwise all pull from the
  // owner of the first bytes at once); flags are indexed in sending order
  const int num_pieces = static_cast<int>((prio_hi - prio_lo + piece_bytes - 1) / piece_bytes);
  for (int i = 0; i < num_pieces; ++i) {
    const int q = (first_piece + i) % num_pieces;
    const long long a = prio_lo + static_cast<long long>(q) * piece_bytes;
    cudaError_t e = copy_range(a, a + piece_bytes < prio_hi ? a + piece_bytes : prio_hi, false);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (write_u32(stream, reinterpret_cast<unsigned long long>(flags + i), flag_value, 0u) != 0) return -3;
  }
  cudaError_t e = copy_range(0, prio_lo, false);
  if (e == cudaSuccess) e = copy_range(prio_hi, total, false);
  if (e == cudaSuccess) e = copy_range(0, prio_lo, true);
  if (e == cudaSuccess) e = copy_range(prio_hi, total, true);
  return static_cast<int>(e);
}

// All-gather of equal row blocks (`shard_bytes` each; block p of `out` is rank p's) whose progress a concurrently running
// consumer follows: blocks arrive this rank's own first, then rank + 1, ... cyclically, each in pieces of `piece_bytes`, and
// flags[k * pieces_per_block + j] = flag_value is stored in stream order once piece j of the k-th arriving block is in
// place.  Two phases for the reason given above (copies within this GPU do not overlap a persistent kernel):
//   phase 0 - own block + its flags, on the consumer's stream before the consumer;
//   phase 1 - the peers' blocks on the copy engines of a side stream that waits for phase 0.
// The caller provides the barriers around the two calls.  Returns -2 without stream memory operations.
FSB_API int fsb_comm_gather_blocks_flagged(int rank, int world, int phase, void* const* src, void* out, long long shard_bytes,
                                           long long piece_bytes, unsigned int* flags, unsigned int flag_value, cudaStream_t stream) {
  if (world > fsb::kMaxRanks || rank < 0 || rank >= world || shard_bytes <= 0 || piece_bytes <= 0) return -1;
  const stream_write_fn write_u32 = stream_write_entry();
  if (write_u32 == nullptr) return -2;
  const int pps = static_cast<int>((shard_bytes + piece_bytes - 1) / piece_bytes);
  const int k_lo = phase == 0 ? 0 : 1, k_hi = phase == 0 ? 1 : world;
  for (int k = k_lo; k < k_hi; ++k) {
    const int p = (rank + k) % world;
    char* dst = static_cast<char*>(out) + static_cast<long long>(p) * shard_bytes;
    const char* from = static_cast<const char*>(src[p]);
    for (int j = 0; j < pps; ++j) {
      const long long a = static_cast<long long>(j) * piece_bytes;
      const long long n = a + piece_bytes < shard_bytes ? piece_bytes : shard_bytes - a;
      if (dst + a != from + a) {
        cudaError_t e = cudaMemcpyAsync(dst + a, from + a, static_cast<size_t>(n), cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) return static_cast<int>(e);
      }
      if (write_u32(stream, reinterpret_cast<unsigned long long>(flags + k * pps + j), flag_value, 0u) != 0) return -3;
    }
  }
  return 0;
}

FSB_API int fsb_comm_all_to_all(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, void* const* src,
                                void* out, long long chunk_bytes, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks || chunk_bytes % 16) return -1;
  const long long n16 = chunk_bytes / 16;
  fsb::all_to_all_kernel<<<comm_grid(n16, kWideGrid), fsb::COMM_THREADS, 0, stream>>>(
      make_ctx(rank, world, epoch, channel, pads, counter, status), make_table(src, world), static_cast<uint4*>(out), n16);
  return static_cast<int>(cudaGetLastError());
}

// out[n] (out_dtype) = (accumulate ? out : 0) + scale * sum_p src[p][rank * n + i]   (src in in_dtype)
static int launch_reduce(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, void* const* src,
                         int in_dtype, void* out, int out_dtype, long long n, float scale, int accumulate, long long base, int active,
                         int* status, cudaStream_t stream) {
  using namespace fsb;
  const CommCtx c = make_ctx(rank, world, epoch, channel, pads, counter, status);
  const PtrTable t = make_table(src, world);
  const int grid = active ? comm_grid(n / 8, 148) : 1;
#define FSB_RS(IC, IT, OC, OT)                                                                                          \
  if (in_dtype == IC && out_dtype == OC) {                                                                              \
    reduce_scatter_kernel<IT, OT><<<grid, COMM_THREADS, 0, stream>>>(c, t, static_cast<OT*>(out), n, scale, accumulate, base, active); \
    return static_cast<int>(cudaGetLastError());                                                                        \
  }
  FSB_RS(FSB_BF16, __nv_bfloat16, FSB_F32, float)
  FSB_RS(FSB_BF16, __nv_bfloat16, FSB_BF16, __nv_bfloat16)
  FSB_RS(FSB_F16, __half, FSB_F32, float)
  FSB_RS(FSB_F16, __half, FSB_F16, __half)
  FSB_RS(FSB_F32, float, FSB_F32, float)
#undef FSB_RS
  return -1;
}

FSB_API int fsb_comm_reduce_scatter(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                                    void* const* src, int in_dtype, void* out, int out_dtype, long long n, float scale, int accumulate,
                                    int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks) return -1;
  if ((n * (in_dtype == FSB_F32 ? 4 : 2)) % 16) return -1;  // each rank's chunk must start 16-byte aligned
  return launch_reduce(rank, world, epoch, channel, pads, counter, src, in_dtype, out, out_dtype, n, scale, accumulate,
                       static_cast<long long>(rank) * n, 1, status, stream);
}

// Reduce-scatter with the transport on the copy engines: flag barrier (peers' gradients are final) -> one cudaMemcpyAsync
// per peer that brings its copy of this rank's slice into `stage` ((world - 1) * n elements of in_dtype, ordinary device
// memory) -> flag barrier (peers are done reading this rank's buffer) -> a short local kernel that sums the world addends
// in rank order, scales, casts and accumulates exactly like the pull kernel.  While the slices travel no SM is involved, so
// GEMMs of other streams keep the whole GPU; the sum touches the SMs for the time it takes to stream world * n elements
// from local memory.  Uses epochs `epoch` and `epoch + 1` on `channel`.
FSB_API int fsb_comm_reduce_scatter_dma(int rank, int world, unsigned epoch, int channel, void* const* pads, void* const* src,
                                        int in_dtype, void* stage, void* out, int out_dtype, long long n, float scale, int accumulate,
                                        int* status, cudaStream_t stream) {
  using namespace fsb;
  if (world > kMaxRanks) return -1;
  const long long es = in_dtype == FSB_F32 ? 4 : 2;
  if ((n * es) % 16) return -1;
  barrier_kernel<<<1, COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch, channel, pads, nullptr, status));
  const void* addend[kMaxRanks];
  for (int k = 1; k < world; ++k) {
    const int p = (rank + k) % world;  // the ring: at any moment the ranks read from different sources
    char* dst = static_cast<char*>(stage) + static_cast<long long>(k - 1) * n * es;
    cudaError_t e = cudaMemcpyAsync(dst, static_cast<const char*>(src[p]) + static_cast<long long>(rank) * n * es, static_cast<size_t>(n * es),
                                    cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    addend[p] = dst;
  }
  addend[rank] = static_cast<const char*>(src[rank]) + static_cast<long long>(rank) * n * es;
  barrier_kernel<<<1, COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch + 1u, channel, pads, nullptr, status));
  PtrTable t{};
  for (int q = 0; q < world; ++q) t.p[q] = addend[q];
  const int grid = comm_grid(n / 8, 148 * 4);
#define FSB_LS(IC, IT, OC, OT)                                                                                          \
  if (in_dtype == IC && out_dtype == OC) {                                                                              \
    local_sum_kernel<IT, OT><<<grid, COMM_THREADS, 0, stream>>>(t, world, static_cast<OT*>(out), n, scale, accumulate); \
    return static_cast<int>(cudaGetLastError());                                                                        \
  }
  FSB_LS(FSB_BF16, __nv_bfloat16, FSB_F32, float)
  FSB_LS(FSB_BF16, __nv_bfloat16, FSB_BF16, __nv_bfloat16)
  FSB_LS(FSB_F16, __half, FSB_F32, float)
  FSB_LS(FSB_F16, __half, FSB_F16, __half)
  FSB_LS(FSB_F32, float, FSB_F32, float)
#undef FSB_LS
  return -1;
}

// Sum of every rank's symmetric buffer bufs[p] (n elements of `dtype`) into rank `owner`'s buffer, in place and scaled; the
// other ranks' buffers are left as they are.  The owner pulls; the others only take part in the two barriers (peers'
// buffers final before, owner done reading after).  ZeRO-2's reduction of a gradient bucket to the rank that owns it.
FSB_API int fsb_comm_reduce_to(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, void* const* bufs,
                               int dtype, long long n, float scale, int owner, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks || owner < 0 || owner >= world) return -1;
  return launch_reduce(rank, world, epoch, channel, pads, counter, bufs, dtype, bufs[rank], dtype, n, scale, 0, 0, rank == owner ? 1 : 0,
                       status, stream);
}

// Every rank but `owner` copies the owner's symmetric buffer into `out` (nbytes) on the copy engines, between two flag
// barriers (owner's buffer final before, everybody done reading after).  ZeRO-1's publication of the updated parameters
// of one owner.  Uses epochs `epoch` and `epoch + 1` on `channel`.
FSB_API int fsb_comm_broadcast_dma(int rank, int world, unsigned epoch, int channel, void* const* pads, void* const* src, void* out,
                                   long long nbytes, int owner, int* status, cudaStream_t stream) {
  if (world > fsb::kMaxRanks || owner < 0 || owner >= world) return -1;
  fsb::barrier_kernel<<<1, fsb::COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch, channel, pads, nullptr, status));
  if (rank != owner && out != src[owner]) {
    cudaError_t e = cudaMemcpyAsync(out, src[owner], static_cast<size_t>(nbytes), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  fsb::barrier_kernel<<<1, fsb::COMM_THREADS, 0, stream>>>(make_ctx(rank, world, epoch + 1u, channel, pads, nullptr, status));
  return static_cast<int>(cudaGetLastError());
}

// Fused reduce-scatter + Adam on this rank's shard.  src: every rank's flat gradient (in_dtype, world * n elements, in the
// symmetric heap); p / m / v: fp32 shards of n elements; p_copy (copy_dtype bf16 / fp16, may be null): the compute-dtype
// shard.  n * sizeof(in_dtype) must be a multiple of 16 and p / m / v 16-byte aligned.
FSB_API int fsb_comm_reduce_scatter_adam(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                                         void* const* src, int in_dtype, long long n, float scale, float* p, float* m, float* v,
                                         void* p_copy, int copy_dtype, float step_size, float lr, float beta1, float beta2, float eps,
                                         float decay, int eps_inside_sqrt, int adamw, float* gnorm_sq, int* found_inf, int* status,
                                         cudaStream_t stream) {
  using namespace fsb;
  if (world > kMaxRanks) return -1;
  if ((n * (in_dtype == FSB_F32 ? 4 : 2)) % 16) return -1;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) return -1;
  const CommCtx c = make_ctx(rank, world, epoch, channel, pads, counter, status);
  const PtrTable t = make_table(src, world);
  const AdamHyper h{step_size, lr, beta1, beta2, eps, decay, eps_inside_sqrt, adamw};
  const int grid = comm_grid(n / 8, 148);
#define FSB_RSA(IC, IT, CC, CT)                                                                                               \
  if (in_dtype == IC && (p_copy == nullptr || copy_dtype == CC)) {                                                            \
    reduce_scatter_adam_kernel<IT, CT><<<grid, COMM_THREADS, 0, stream>>>(c, t, n, scale, p, m, v, static_cast<CT*>(p_copy), h, \
                                                                          gnorm_sq, found_inf);                               \
    return static_cast<int>(cudaGetLastError());                                                                             \
  }
  FSB_RSA(FSB_BF16, __nv_bfloat16, FSB_BF16, __nv_bfloat16)
  FSB_RSA(FSB_F16, __half, FSB_F16, __half)
  FSB_RSA(FSB_F32, float, FSB_BF16, __nv_bfloat16)
  FSB_RSA(FSB_F32, float, FSB_F16, __half)
#undef FSB_RSA
  return -1;
}

// in-place sum over ranks of every rank's symmetric buffer bufs[p] (n elements)
FSB_API int fsb_comm_all_reduce(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, void* const* bufs,
                                int dtype, long long n, int* status, cudaStream_t stream) {
  using namespace fsb;
  if (world > kMaxRanks) return -1;
  const CommCtx c = make_ctx(rank, world, epoch, channel, pads, counter, status);
  const PtrTable t = make_table(bufs, world);
  // The CTAs of this kernel wait for one another, so it is launched cooperatively: the runtime starts it only when
  // the whole grid can be resident at once, whatever else is running on the device.
  int grid = comm_grid(n / 8 / world + 1, 132);
  CommCtx cc = c;
  PtrTable tt = t;
  long long nn = n;
  void* args[] = {&cc, &tt, &nn};
  const void* fn = nullptr;
  if (dtype == FSB_BF16) fn = reinterpret_cast<const void*>(all_reduce_kernel<__nv_bfloat16>);
  else if (dtype == FSB_F16) fn = reinterpret_cast<const void*>(all_reduce_kernel<__half>);
  else if (dtype == FSB_F32) fn = reinterpret_cast<const void*>(all_reduce_kernel<float>);
  else return -1;
  return static_cast<int>(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(COMM_THREADS), args, 0, stream));
}

FSB_API int fsb_comm_moe_scatter_rows(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                                      void* const* dst, const void* x, const int* dst_rank, const int* dst_row, const float* w,
                                      long long T, int rows_per_token, int M, const int* counts, int E, int C, int n_local,
                                      int* status, cudaStream_t stream) {
  using namespace fsb;
  if (world > kMaxRanks || M % 8) return -1;
  if (counts != nullptr && (E < 1 || C < 1 || n_local < 1 || E != n_local * world)) return -1;
  moe_scatter_rows_kernel<<<comm_grid(T * 32, kWideGrid), COMM_THREADS, 0, stream>>>(
      make_ctx(rank, world, epoch, channel, pads, counter, status), make_table(dst, world), static_cast<const __nv_bfloat16*>(x),
      dst_rank, dst_row, w, T, rows_per_token, M, counts, E, C, n_local);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_comm_moe_gather_rows(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                                     void* const* src, void* out, const int* src_rank, const int* src_row, const float* w,
                                     const void* g, float* dot, long long tokens, int rows_per_token, int M, int* status,
                                     cudaStream_t stream) {
  using namespace fsb;
  if (world > kMaxRanks || M % 8 || rows_per_token > 4) return -1;
  moe_gather_rows_kernel<<<comm_grid(tokens * 32, kWideGrid), COMM_THREADS, 0, stream>>>(
      make_ctx(rank, world, epoch, channel, pads, counter, status), make_table(src, world), static_cast<__nv_bfloat16*>(out), src_rank,
      src_row, w, static_cast<const __nv_bfloat16*>(g), dot, tokens, rows_per_token, M);
  return static_cast<int>(cudaGetLastError());
}
