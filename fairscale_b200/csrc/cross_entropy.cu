// Softmax cross-entropy over bf16 logits with fp32 math.
//
// Forward: one CTA per token row, one streaming pass (online max / sum) over the vocabulary with
// 16-byte loads; writes the per-row loss and log-sum-exp.  Backward: one pass that turns the logits
// into d(logits) = (softmax - onehot) * g in place or into a separate buffer.  The [tokens, vocab]
// matrix is therefore read twice and written once in total.
// The vocab-parallel variant returns each rank's (max, sum-exp at that max, target logit) triple so
// the caller can combine them with ONE 3-vector all-reduce instead of the three all-reduces of
// fairscale/nn/model_parallel/cross_entropy.py:35,62-71.

#include "common.cuh"

namespace fsb {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_update(float& m, float& s, float x) {
  if (x > m) { s = s * __expf(m - x) + 1.f; m = x; } else { s += __expf(x - m); }
}

// stats_out (optional): per row {max, sumexp(at max), target_logit or 0 if target outside [v0, v0+V)}
__global__ void __launch_bounds__(CE_THREADS) ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                            float* __restrict__ loss, float* __restrict__ lse_out, float* __restrict__ stats_out,
                                                            int V, long long ld, long long vocab_start, long long ignore_index) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  const int nvec = V / 8;
  for (int j = threadIdx.x; j < nvec; j += CE_THREADS) {
    const Vec16<__nv_bfloat16> t = ld16(lr + j * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) online_update(m, s, __bfloat162float(t.v[k]));
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) online_update(m, s, __bfloat162float(lr[j]));
  const float gmax = block_max(m, scratch);
  const float contrib = (m == -INFINITY) ? 0.f : s * __expf(m - gmax);
  const float gsum = block_sum(contrib, scratch);
  if (threadIdx.x == 0) {
    const long long tgt = targets[row];
    const long long local = tgt - vocab_start;
    const bool mine = tgt != ignore_index && local >= 0 && local < V;
    const float tl = mine ? __bfloat162float(lr[local]) : 0.f;
    const float lse = gmax + __logf(gsum);
    if (lse_out != nullptr) lse_out[row] = lse;
    if (loss != nullptr) loss[row] = (tgt == ignore_index) ? 0.f : (lse - tl);
    if (stats_out != nullptr) {
      stats_out[row * 3 + 0] = gmax;
      stats_out[row * 3 + 1] = gsum;
      stats_out[row * 3 + 2] = tl;
    }
  }
}

// dlogits[row, j] = (exp(logit - lse[row]) - [j == target]) * gscale[row-independent scalar] * gout[row or scalar]
__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                                                            const float* __restrict__ lse, const float* __restrict__ grad_out, int grad_is_scalar,
                                                            float scale, __nv_bfloat16* __restrict__ dlogits, int V, long long ld,
                                                            long long vocab_start, long long ignore_index) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * ld;
  __nv_bfloat16* dr = dlogits + row * ld;
  const long long tgt = targets[row];
  const float g = (tgt == ignore_index) ? 0.f : scale * (grad_is_scalar ? grad_out[0] : grad_out[row]);
  const float l = lse[row];
  const long long local = tgt - vocab_start;
  const int nvec = V / 8;
  for (int j = threadIdx.x; j < nvec; j += CE_THREADS) {
    const Vec16<__nv_bfloat16> t = ld16(lr + j * 8);
    Vec16<__nv_bfloat16> o;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float p = __expf(__bfloat162float(t.v[k]) - l);
      if (j * 8 + k == local) p -= 1.f;
      o.v[k] = __float2bfloat16_rn(p * g);
    }
    st16(dr + j * 8, o);
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
    float p = __expf(__bfloat162float(lr[j]) - l);
    if (j == local) p -= 1.f;
    dr[j] = __float2bfloat16_rn(p * g);
  }
}

}  // namespace fsb

// logits: bf16 [rows, V] with row stride ld (ld % 8 == 0 and base 16-byte aligned for the vector path).
FSB_API int fsb_ce_fwd(const void* logits, const long long* targets, float* loss, float* lse, float* stats, long long rows,
                       int V, long long ld, long long vocab_start, long long ignore_index, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (ld % 8 != 0) return -1;
  ce_fwd_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets, loss, lse,
                                                                         stats, V, ld, vocab_start, ignore_index);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_ce_bwd(const void* logits, const long long* targets, const float* lse, const float* grad_out, int grad_is_scalar,
                       float scale, void* dlogits, long long rows, int V, long long ld, long long vocab_start,
                       long long ignore_index, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (ld % 8 != 0) return -1;
  ce_bwd_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets, lse, grad_out,
                                                                         grad_is_scalar, scale, static_cast<__nv_bfloat16*>(dlogits), V, ld,
                                                                         vocab_start, ignore_index);
  return static_cast<int>(cudaGetLastError());
}
