// Index part of GShard top-2 gating: first / second expert of every token and the token's slot in that expert's buffer.
//
//   idx1[s] = argmax_e logits[s, e]                       (first maximum, like torch.argmax)
//   idx2[s] = argmax_{e != idx1[s]} logits[s, e] + noise[s, e]
//   loc1[s] = number of tokens s' < s with idx1[s'] == idx1[s]
//   loc2[s] = (tokens whose first choice is idx2[s]) + number of tokens s' < s with idx2[s'] == idx2[s]
//   count1[e] = tokens whose first choice is e
//
// The reference builds these from one-hot [S, E] int64 matrices and two cumulative sums over S
// (fairscale/nn/moe/top2gate.py:50-66); here it is three small launches: per-token argmax + per-block histograms,
// a scan of the block histograms, and a ranking pass (warp match + shared-memory prefix).  The differentiable part
// (softmax, gate values, auxiliary loss) is the pair of kernels at the end of this file.

#include "common.cuh"

namespace fsb {

constexpr int T2_THREADS = 256;
constexpr int T2_WARPS = T2_THREADS / 32;
constexpr int T2_MAX_E = 512;

template <typename T> __device__ __forceinline__ float t2_load(const T* p, long long i) { return static_cast<float>(p[i]); }
template <> __device__ __forceinline__ float t2_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(T2_THREADS) top2_choose_kernel(const T* __restrict__ logits, const float* __restrict__ noise, int S, int E,
                                                                 int* __restrict__ idx1, int* __restrict__ idx2,
                                                                 int* __restrict__ block_counts) {
  __shared__ int hist[2][T2_MAX_E];
  for (int e = threadIdx.x; e < 2 * E; e += T2_THREADS) hist[e / E][e % E] = 0;
  __syncthreads();
  const int s = blockIdx.x * T2_THREADS + threadIdx.x;
  if (s < S) {
    const long long base = static_cast<long long>(s) * E;
    float best = -INFINITY;
    int i1 = 0;
    for (int e = 0; e < E; ++e) {
      const float v = t2_load(logits, base + e);
      if (v > best) { best = v; i1 = e; }
    }
    float best2 = -INFINITY;
    int i2 = (i1 == 0) ? 1 : 0;
    for (int e = 0; e < E; ++e) {
      if (e == i1) continue;
      const float v = t2_load(logits, base + e) + noise[base + e];
      if (v > best2) { best2 = v; i2 = e; }
    }
    idx1[s] = i1;
    idx2[s] = i2;
    atomicAdd(&hist[0][i1], 1);
    atomicAdd(&hist[1][i2], 1);
  }
  __syncthreads();
  int* out = block_counts + static_cast<long long>(blockIdx.x) * 2 * E;
  for (int e = threadIdx.x; e < 2 * E; e += T2_THREADS) out[e] = hist[e / E][e % E];
}

// exclusive scan over blocks, in place; totals[2][E] receives the column sums
__global__ void top2_scan_kernel(int* __restrict__ block_counts, int n_blocks, int E, int* __restrict__ totals) {
  for (int c = threadIdx.x; c < 2 * E; c += blockDim.x) {
    int run = 0;
    for (int b = 0; b < n_blocks; ++b) {
      int* p = block_counts + static_cast<long long>(b) * 2 * E + c;
      const int v = *p;
      *p = run;
      run += v;
    }
    totals[c] = run;
  }
}

__global__ void __launch_bounds__(T2_THREADS) top2_rank_kernel(const int* __restrict__ idx1, const int* __restrict__ idx2,
                                                               const int* __restrict__ block_offsets, const int* __restrict__ totals,
                                                               int S, int E, int* __restrict__ loc1, int* __restrict__ loc2) {
  __shared__ int warp_cnt[2][T2_WARPS][T2_MAX_E];  // tokens of each warp per expert, then exclusive prefix over warps
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 2 * T2_WARPS * E; i += T2_THREADS) {
    const int k = i / (T2_WARPS * E), r = i - k * T2_WARPS * E;
    warp_cnt[k][r / E][r % E] = 0;
  }
  __syncthreads();
  const int s = blockIdx.x * T2_THREADS + threadIdx.x;
  const bool valid = s < S;
  const int e1 = valid ? idx1[s] : -1 - lane, e2 = valid ? idx2[s] : -1 - lane;  // distinct dummies never match
  const unsigned lt = (1u << lane) - 1u;
  const unsigned m1 = __match_any_sync(0xffffffffu, e1), m2 = __match_any_sync(0xffffffffu, e2);
  const int r1 = __popc(m1 & lt), r2 = __popc(m2 & lt);
  if (valid && r1 == 0) warp_cnt[0][warp][e1] = __popc(m1);  // first lane of each group records the group size
  if (valid && r2 == 0) warp_cnt[1][warp][e2] = __popc(m2);
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * E; i += T2_THREADS) {  // exclusive prefix over the warps of the block
    const int k = i / E, e = i - k * E;
    int run = 0;
    for (int w = 0; w < T2_WARPS; ++w) {
      const int v = warp_cnt[k][w][e];
      warp_cnt[k][w][e] = run;
      run += v;
    }
  }
  __syncthreads();
  if (valid) {
    const int* off = block_offsets + static_cast<long long>(blockIdx.x) * 2 * E;
    loc1[s] = off[e1] + warp_cnt[0][warp][e1] + r1;
    loc2[s] = totals[e2] + off[E + e2] + warp_cnt[1][warp][e2] + r2;  // second choices queue behind all first choices
  }
}

// ------------------------------------------------------------------------------------------------ gate values
// The differentiable part of the gate in one pass per direction (one warp per token, softmax in fp32 registers).
//
// forward:  p = softmax(logits[s, :]);  g_k = p[idx_k] * keep_k;  denom = max(g_1 + g_2, eps);  gate[s, k] = g_k / denom;
//           me_sum[e] += p[e]   (column sums, one atomic per CTA and expert).  l_aux = mean_e(me_sum[e] / S * ce[e]).
// backward: dp[e] = d_l_aux * ce[e] / (E * S)  (+ the quotient rule of the two kept gates at idx_1, idx_2);
//           d_logits[s, e] = p[e] * (dp[e] - sum_j p[j] dp[j]).
// loc_k < capacity decides keep_k, as in the index kernels' consumer.
constexpr int GV_THREADS = 256;
constexpr int GV_PER_LANE = T2_MAX_E / 32;

template <typename T>
__device__ __forceinline__ void gv_softmax(const T* __restrict__ row, int E, int lane, float (&p)[GV_PER_LANE]) {
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    p[j] = e < E ? t2_load(row, e) : -INFINITY;
    mx = fmaxf(mx, p[j]);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j) {
    p[j] = (lane + 32 * j) < E ? __expf(p[j] - mx) : 0.f;
    sum += p[j];
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j) p[j] *= inv;
}

// value of element `e` of a row distributed as p[j] on lane (e % 32), j = e / 32
__device__ __forceinline__ float gv_pick(const float (&p)[GV_PER_LANE], int e, int lane) {
  float v = 0.f;
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j)
    if (j == (e >> 5)) v = p[j];
  return __shfl_sync(0xffffffffu, v, e & 31);
}

template <typename T>
__global__ void __launch_bounds__(GV_THREADS) top2_gate_fwd_kernel(const T* __restrict__ logits, int S, int E, const int* __restrict__ idx1,
                                                                   const int* __restrict__ idx2, const int* __restrict__ loc1,
                                                                   const int* __restrict__ loc2, int capacity, float eps,
                                                                   const int* __restrict__ count1, float* __restrict__ gate,
                                                                   float* __restrict__ me_sum, float* __restrict__ l_aux,
                                                                   unsigned int* __restrict__ ticket) {
  __shared__ float col[T2_MAX_E];
  __shared__ bool last;
  for (int e = threadIdx.x; e < E; e += GV_THREADS) col[e] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps_total = gridDim.x * (GV_THREADS / 32);
  float acc[GV_PER_LANE];
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j) acc[j] = 0.f;
  for (int s = blockIdx.x * (GV_THREADS / 32) + warp; s < S; s += warps_total) {
    float p[GV_PER_LANE];
    gv_softmax(logits + static_cast<long long>(s) * E, E, lane, p);
#pragma unroll
    for (int j = 0; j < GV_PER_LANE; ++j) acc[j] += p[j];
    const int i1 = idx1[s], i2 = idx2[s];
    const float g1 = loc1[s] < capacity ? gv_pick(p, i1, lane) : 0.f;
    const float g2 = loc2[s] < capacity ? gv_pick(p, i2, lane) : 0.f;
    if (lane == 0) {
      const float denom = fmaxf(g1 + g2, eps);
      gate[2 * static_cast<long long>(s)] = g1 / denom;
      gate[2 * static_cast<long long>(s) + 1] = g2 / denom;
    }
  }
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j)
    if (lane + 32 * j < E) atomicAdd(&col[lane + 32 * j], acc[j]);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += GV_THREADS) atomicAdd(&me_sum[e], col[e]);
  // the last CTA to get here has every column sum in front of it: l_aux = mean_e(me[e] * ce[e])
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last) {
    __threadfence();
    float part = 0.f;
    for (int e = threadIdx.x; e < E; e += GV_THREADS) part += __ldcg(&me_sum[e]) * static_cast<float>(count1[e]);
    for (int e = threadIdx.x; e < E; e += GV_THREADS) col[e] = 0.f;
    __syncthreads();
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) atomicAdd(&col[0], part);
    __syncthreads();
    if (threadIdx.x == 0) {
      l_aux[0] = col[0] / (static_cast<float>(E) * static_cast<float>(S) * static_cast<float>(S));
      *ticket = 0u;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(GV_THREADS) top2_gate_bwd_kernel(const T* __restrict__ logits, int S, int E, const int* __restrict__ idx1,
                                                                   const int* __restrict__ idx2, const int* __restrict__ loc1,
                                                                   const int* __restrict__ loc2, int capacity, float eps,
                                                                   const float* __restrict__ d_gate, const float* __restrict__ d_l_aux,
                                                                   const int* __restrict__ count1, T* __restrict__ d_logits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps_total = gridDim.x * (GV_THREADS / 32);
  const float aux = d_l_aux != nullptr ? d_l_aux[0] / (static_cast<float>(E) * static_cast<float>(S) * static_cast<float>(S)) : 0.f;
  float dp_aux[GV_PER_LANE];  // d_l_aux * ce[e] / (E * S), ce[e] = count1[e] / S
#pragma unroll
  for (int j = 0; j < GV_PER_LANE; ++j) dp_aux[j] = (lane + 32 * j) < E ? aux * static_cast<float>(count1[lane + 32 * j]) : 0.f;
  for (int s = blockIdx.x * (GV_THREADS / 32) + warp; s < S; s += warps_total) {
    float p[GV_PER_LANE];
    gv_softmax(logits + static_cast<long long>(s) * E, E, lane, p);
    const int i1 = idx1[s], i2 = idx2[s];
    const bool k1 = loc1[s] < capacity, k2 = loc2[s] < capacity;
    const float g1 = k1 ? gv_pick(p, i1, lane) : 0.f;
    const float g2 = k2 ? gv_pick(p, i2, lane) : 0.f;
    const float dg1 = d_gate[2 * static_cast<long long>(s)], dg2 = d_gate[2 * static_cast<long long>(s) + 1];
    float d1, d2;  // gradients of the two kept probabilities
    const float sum = g1 + g2;
    if (sum > eps) {
      const float inv2 = 1.f / (sum * sum);
      d1 = g2 * (dg1 - dg2) * inv2;
      d2 = g1 * (dg2 - dg1) * inv2;
    } else {
      d1 = dg1 / eps;
      d2 = dg2 / eps;
    }
    if (!k1) d1 = 0.f;
    if (!k2) d2 = 0.f;
    float dp[GV_PER_LANE];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < GV_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      dp[j] = dp_aux[j] + (e == i1 ? d1 : 0.f) + (e == i2 ? d2 : 0.f);
      dot += p[j] * dp[j];
    }
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    T* out = d_logits + static_cast<long long>(s) * E;
#pragma unroll
    for (int j = 0; j < GV_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < E) out[e] = static_cast<T>(p[j] * (dp[j] - dot));
    }
  }
}

}  // namespace fsb

// logits: [S, E] fp32 (dtype 0) or bf16 (dtype 2); noise: fp32 [S, E]; idx1 / idx2 / loc1 / loc2: int32 [S];
// workspace: int32 [ceil(S / 256) * 2 * E]; totals: int32 [2 * E] (totals[e] = count of first choices of expert e).
FSB_API int fsb_top2_workspace_ints(int S, int E) { return ((S + fsb::T2_THREADS - 1) / fsb::T2_THREADS) * 2 * E; }

FSB_API int fsb_top2_route(const void* logits, int dtype, const float* noise, int S, int E, int* idx1, int* idx2, int* loc1, int* loc2,
                           int* workspace, int* totals, cudaStream_t stream) {
  using namespace fsb;
  if (S <= 0) return 0;
  if (E < 2 || E > T2_MAX_E) return -1;
  const int blocks = (S + T2_THREADS - 1) / T2_THREADS;
  if (dtype == FSB_F32) top2_choose_kernel<float><<<blocks, T2_THREADS, 0, stream>>>(static_cast<const float*>(logits), noise, S, E, idx1, idx2, workspace);
  else if (dtype == FSB_BF16) top2_choose_kernel<__nv_bfloat16><<<blocks, T2_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), noise, S, E, idx1, idx2, workspace);
  else return -1;
  top2_scan_kernel<<<1, 256, 0, stream>>>(workspace, blocks, E, totals);
  top2_rank_kernel<<<blocks, T2_THREADS, 0, stream>>>(idx1, idx2, workspace, totals, S, E, loc1, loc2);
  return static_cast<int>(cudaGetLastError());
}

static int gv_grid(int S) {
  const int per_cta = fsb::GV_THREADS / 32;
  int g = (S + per_cta - 1) / per_cta;
  return g < 1 ? 1 : (g > 148 * 4 ? 148 * 4 : g);
}

// gate[S, 2] (fp32), l_aux (one fp32) and me_sum[E] (fp32 scratch) from logits [S, E] (fp32 / bf16) and the index kernels' output.
// me_sum and *ticket must be zero on entry (the kernel leaves the ticket at zero again).
FSB_API int fsb_top2_gate_fwd(const void* logits, int dtype, int S, int E, const int* idx1, const int* idx2, const int* loc1, const int* loc2,
                              int capacity, float eps, const int* count1, float* gate, float* me_sum, float* l_aux, unsigned int* ticket,
                              cudaStream_t stream) {
  using namespace fsb;
  if (E < 2 || E > T2_MAX_E || S < 1) return -1;
  if (dtype == FSB_F32)
    top2_gate_fwd_kernel<float><<<gv_grid(S), GV_THREADS, 0, stream>>>(static_cast<const float*>(logits), S, E, idx1, idx2, loc1, loc2, capacity,
                                                                        eps, count1, gate, me_sum, l_aux, ticket);
  else if (dtype == FSB_BF16)
    top2_gate_fwd_kernel<__nv_bfloat16><<<gv_grid(S), GV_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), S, E, idx1, idx2, loc1,
                                                                                loc2, capacity, eps, count1, gate, me_sum, l_aux, ticket);
  else return -1;
  return static_cast<int>(cudaGetLastError());
}

// d_logits[S, E] (dtype of logits) from d_gate[S, 2] (fp32) and d_l_aux (one fp32 on the device, may be null)
FSB_API int fsb_top2_gate_bwd(const void* logits, int dtype, int S, int E, const int* idx1, const int* idx2, const int* loc1, const int* loc2,
                              int capacity, float eps, const float* d_gate, const float* d_l_aux, const int* count1, void* d_logits,
                              cudaStream_t stream) {
  using namespace fsb;
  if (E < 2 || E > T2_MAX_E || S < 1) return -1;
  if (dtype == FSB_F32)
    top2_gate_bwd_kernel<float><<<gv_grid(S), GV_THREADS, 0, stream>>>(static_cast<const float*>(logits), S, E, idx1, idx2, loc1, loc2, capacity,
                                                                        eps, d_gate, d_l_aux, count1, static_cast<float*>(d_logits));
  else if (dtype == FSB_BF16)
    top2_gate_bwd_kernel<__nv_bfloat16><<<gv_grid(S), GV_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), S, E, idx1, idx2, loc1,
                                                                                loc2, capacity, eps, d_gate, d_l_aux, count1,
                                                                                static_cast<__nv_bfloat16*>(d_logits));
  else return -1;
  return static_cast<int>(cudaGetLastError());
}
