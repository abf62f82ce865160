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
// (softmax, gate values, auxiliary loss) stays in PyTorch.

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
