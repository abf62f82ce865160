// LayerNorm / RMSNorm forward and backward for bf16 activations, fp32 statistics.
//
// Forward: one CTA per row, the row is read once with 16-byte loads, kept in registers, reduced
// (mean / variance) and written once; mean and rstd are saved for backward.
// Backward: same one-pass structure for dx; dgamma / dbeta are accumulated per CTA over a strip of
// rows into fp32 partials [n_strips, H], reduced by a second small kernel (no atomics, so the
// result is deterministic).
// Replaces nn.LayerNorm in the reference's benchmark models (benchmarks/models/transformer_lm.py:109-110).

#include "common.cuh"

namespace fsb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 4;  // block-per-row path: up to 4 x 8 bf16 per thread -> H <= 8192
constexpr int NORM_WARPS = 4;    // warp-per-row path: rows handled per CTA

// ---- warp-per-row kernels (H <= 4096): a lane keeps VPL 16-byte vectors of the row in registers, all
// reductions are warp shuffles, no shared memory and no block barriers.
template <bool RMS, int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32) norm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                                                        const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                                                        float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                        long long rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = H / 8;
  const __nv_bfloat16* xr = x + row * H;
  float v[VPL][8];
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < VPL; ++it) {
    const int j = lane + it * 32;
    if (j < nvec) {
      const Vec16<__nv_bfloat16> t = ld16(xr + j * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) { v[it][k] = __bfloat162float(t.v[k]); sum += v[it][k]; }
    }
  }
  const float mean = RMS ? 0.f : warp_sum(sum) / H;
  float sq = 0.f;
#pragma unroll
  for (int it = 0; it < VPL; ++it) {
    const int j = lane + it * 32;
    if (j < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) { const float d = v[it][k] - mean; sq += d * d; }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / H + eps);
  if (lane == 0) {
    if (!RMS && mean_out != nullptr) mean_out[row] = mean;
    if (rstd_out != nullptr) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + row * H;
#pragma unroll
  for (int it = 0; it < VPL; ++it) {
    const int j = lane + it * 32;
    if (j < nvec) {
      const Vec16<__nv_bfloat16> g = ld16(gamma + j * 8);
      Vec16<__nv_bfloat16> o;
      if (!RMS && beta != nullptr) {
        const Vec16<__nv_bfloat16> b = ld16(beta + j * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          o.v[k] = __float2bfloat16_rn((v[it][k] - mean) * rstd * __bfloat162float(g.v[k]) + __bfloat162float(b.v[k]));
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn((v[it][k] - mean) * rstd * __bfloat162float(g.v[k]));
      }
      st16(yr + j * 8, o);
    }
  }
}

// dx only (dgamma / dbeta come from norm_dparam_partial_kernel)
template <bool RMS, int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32) norm_bwd_dx_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                           const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                                                                           const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                                                           long long rows, int H) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = H / 8;
  const float mean = RMS ? 0.f : mean_in[row];
  const float rstd = rstd_in[row];
  float xh[VPL][8], wdy[VPL][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int it = 0; it < VPL; ++it) {
    const int j = lane + it * 32;
    if (j < nvec) {
      const Vec16<__nv_bfloat16> tx = ld16(x + row * H + j * 8);
      const Vec16<__nv_bfloat16> td = ld16(dy + row * H + j * 8);
      const Vec16<__nv_bfloat16> tg = ld16(gamma + j * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        xh[it][k] = (__bfloat162float(tx.v[k]) - mean) * rstd;
        wdy[it][k] = __bfloat162float(td.v[k]) * __bfloat162float(tg.v[k]);
        s1 += wdy[it][k];
        s2 += wdy[it][k] * xh[it][k];
      }
    }
  }
  s1 = RMS ? 0.f : warp_sum(s1) / H;
  s2 = warp_sum(s2) / H;
#pragma unroll
  for (int it = 0; it < VPL; ++it) {
    const int j = lane + it * 32;
    if (j < nvec) {
      Vec16<__nv_bfloat16> o;
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(rstd * (wdy[it][k] - s1 - xh[it][k] * s2));
      st16(dx + row * H + j * 8, o);
    }
  }
}

// dx and the dgamma / dbeta partials in one pass over dy and x (H <= 2048).  Persistent: a warp walks rows
// blockIdx.x * 4 + warp, + 4 * gridDim.x, ...; a lane owns the same VPL x 8 columns in every row, so it accumulates
// their dgamma / dbeta contributions in registers.  dy and x stay packed in registers between the statistics pass and
// the output pass.  At the end the four warps of a CTA are summed through shared memory and the CTA writes one
// partial row: dgamma_part / dbeta_part are [gridDim.x, H].
template <bool RMS, int VPL>
__global__ void __launch_bounds__(NORM_WARPS * 32, 2) norm_bwd_fused_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                            const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                                                                            const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                                                            float* __restrict__ dgamma_part, float* __restrict__ dbeta_part,
                                                                            long long rows, int H) {
  extern __shared__ float fused_red[];  // [NORM_WARPS][H]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = H / 8;
  float dg[VPL][8], db[VPL][8];
#pragma unroll
  for (int it = 0; it < VPL; ++it) {
#pragma unroll
    for (int k = 0; k < 8; ++k) { dg[it][k] = 0.f; db[it][k] = 0.f; }
  }
  for (long long row = static_cast<long long>(blockIdx.x) * NORM_WARPS + warp; row < rows; row += static_cast<long long>(gridDim.x) * NORM_WARPS) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    Vec16<__nv_bfloat16> tx[VPL], td[VPL];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int it = 0; it < VPL; ++it) {
      const int j = lane + it * 32;
      if (j < nvec) {
        tx[it] = ld16(x + row * H + j * 8);
        td[it] = ld16(dy + row * H + j * 8);
      }
    }
#pragma unroll
    for (int it = 0; it < VPL; ++it) {
      const int j = lane + it * 32;
      if (j < nvec) {
        const Vec16<__nv_bfloat16> tg = ld16(gamma + j * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (__bfloat162float(tx[it].v[k]) - mean) * rstd;
          const float w = __bfloat162float(td[it].v[k]) * __bfloat162float(tg.v[k]);
          s1 += w;
          s2 = fmaf(w, xh, s2);
        }
      }
    }
    s1 = RMS ? 0.f : warp_sum(s1) / H;
    s2 = warp_sum(s2) / H;
#pragma unroll
    for (int it = 0; it < VPL; ++it) {
      const int j = lane + it * 32;
      if (j < nvec) {
        const Vec16<__nv_bfloat16> tg = ld16(gamma + j * 8);
        Vec16<__nv_bfloat16> o;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float xh = (__bfloat162float(tx[it].v[k]) - mean) * rstd;
          const float d = __bfloat162float(td[it].v[k]);
          const float w = d * __bfloat162float(tg.v[k]);
          o.v[k] = __float2bfloat16_rn(rstd * (w - s1 - xh * s2));
          dg[it][k] = fmaf(d, xh, dg[it][k]);
          if (!RMS) db[it][k] += d;
        }
        st16(dx + row * H + j * 8, o);
      }
    }
  }
  // the CTA's partial row: sum of its four warps, dgamma first and dbeta second through the same buffer
#pragma unroll 1
  for (int which = 0; which < (RMS ? 1 : 2); ++which) {
    float* out = which == 0 ? dgamma_part : dbeta_part;
    if (out == nullptr) break;  // uniform
    __syncthreads();
#pragma unroll
    for (int it = 0; it < VPL; ++it) {
      const int j = lane + it * 32;
      if (j < nvec) {
#pragma unroll
        for (int k = 0; k < 8; ++k) fused_red[warp * H + j * 8 + k] = which == 0 ? dg[it][k] : db[it][k];
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < H; c += NORM_WARPS * 32) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < NORM_WARPS; ++w) acc += fused_red[w * H + c];
      out[static_cast<long long>(blockIdx.x) * H + c] = acc;
    }
  }
}

// Partial column sums of dy * xhat (-> dgamma) and dy (-> dbeta) over a strip of rows.
// grid = (ceil(H / 256), strips), block = (32, 8): a thread owns 8 consecutive columns.
template <bool RMS>
__global__ void __launch_bounds__(256) norm_dparam_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                  const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                                                  float* __restrict__ dgamma_part, float* __restrict__ dbeta_part,
                                                                  long long rows, int H) {
  const int col0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const bool active = col0 < H;
  float dg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, db[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (long long r = blockIdx.y * 8 + threadIdx.y; active && r < rows; r += static_cast<long long>(gridDim.y) * 8) {
    const float mean = RMS ? 0.f : mean_in[r];
    const float rstd = rstd_in[r];
    const Vec16<__nv_bfloat16> tx = ld16(x + r * H + col0);
    const Vec16<__nv_bfloat16> td = ld16(dy + r * H + col0);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float d = __bfloat162float(td.v[k]);
      dg[k] += d * (__bfloat162float(tx.v[k]) - mean) * rstd;
      db[k] += d;
    }
  }
  __shared__ float red[2][8][32][9];
#pragma unroll
  for (int k = 0; k < 8; ++k) { red[0][threadIdx.y][threadIdx.x][k] = dg[k]; red[1][threadIdx.y][threadIdx.x][k] = db[k]; }
  __syncthreads();
  if (threadIdx.y < 2 && active) {
    const int which = threadIdx.y;
    if (which == 1 && (RMS || dbeta_part == nullptr)) return;
    float* out = (which == 0 ? dgamma_part : dbeta_part) + static_cast<long long>(blockIdx.y) * H + col0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float s = 0.f;
#pragma unroll
      for (int yy = 0; yy < 8; ++yy) s += red[which][yy][threadIdx.x][k];
      out[k] = s;
    }
  }
}

template <bool RMS>
__global__ void __launch_bounds__(NORM_THREADS) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                                                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float scratch[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  __nv_bfloat16* yr = y + row * H;
  const int nvec = H / 8;
  float v[NORM_MAX_VEC][8];
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < NORM_MAX_VEC; ++it) {
    const int j = threadIdx.x + it * NORM_THREADS;
    if (j < nvec) {
      const Vec16<__nv_bfloat16> t = ld16(xr + j * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) { v[it][k] = __bfloat162float(t.v[k]); sum += v[it][k]; }
    }
  }
  float mean = 0.f;
  if (!RMS) mean = block_sum(sum, scratch) / H;
  float sq = 0.f;
#pragma unroll
  for (int it = 0; it < NORM_MAX_VEC; ++it) {
    const int j = threadIdx.x + it * NORM_THREADS;
    if (j < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) { const float d = v[it][k] - mean; sq += d * d; }
    }
  }
  const float var = block_sum(sq, scratch) / H;
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (!RMS && mean_out != nullptr) mean_out[row] = mean;
    if (rstd_out != nullptr) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int it = 0; it < NORM_MAX_VEC; ++it) {
    const int j = threadIdx.x + it * NORM_THREADS;
    if (j < nvec) {
      const Vec16<__nv_bfloat16> g = ld16(gamma + j * 8);
      Vec16<__nv_bfloat16> o;
      if (!RMS && beta != nullptr) {
        const Vec16<__nv_bfloat16> b = ld16(beta + j * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          o.v[k] = __float2bfloat16_rn((v[it][k] - mean) * rstd * __bfloat162float(g.v[k]) + __bfloat162float(b.v[k]));
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn((v[it][k] - mean) * rstd * __bfloat162float(g.v[k]));
      }
      st16(yr + j * 8, o);
    }
  }
}

// Block-per-row dx (H > 4096).
template <bool RMS>
__global__ void __launch_bounds__(NORM_THREADS) norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                   const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                                                                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, int H) {
  __shared__ float scratch[32];
  const int nvec = H / 8;
  const long long row = blockIdx.x;
  const float mean = RMS ? 0.f : mean_in[row];
  const float rstd = rstd_in[row];
  float xh[NORM_MAX_VEC][8], wdy[NORM_MAX_VEC][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int it = 0; it < NORM_MAX_VEC; ++it) {
    const int j = threadIdx.x + it * NORM_THREADS;
    if (j < nvec) {
      const Vec16<__nv_bfloat16> tx = ld16(x + row * H + j * 8);
      const Vec16<__nv_bfloat16> td = ld16(dy + row * H + j * 8);
      const Vec16<__nv_bfloat16> tg = ld16(gamma + j * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        xh[it][k] = (__bfloat162float(tx.v[k]) - mean) * rstd;
        wdy[it][k] = __bfloat162float(td.v[k]) * __bfloat162float(tg.v[k]);
        s1 += wdy[it][k];
        s2 += wdy[it][k] * xh[it][k];
      }
    }
  }
  if (!RMS) s1 = block_sum(s1, scratch) / H; else s1 = 0.f;
  s2 = block_sum(s2, scratch) / H;
#pragma unroll
  for (int it = 0; it < NORM_MAX_VEC; ++it) {
    const int j = threadIdx.x + it * NORM_THREADS;
    if (j < nvec) {
      Vec16<__nv_bfloat16> o;
#pragma unroll
      for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(rstd * (wdy[it][k] - s1 - xh[it][k] * s2));
      st16(dx + row * H + j * 8, o);
    }
  }
}

// out[c] = sum_r part[r, c]  (fp32 partials -> bf16 or fp32 result).  block = (32 columns, 8 row groups): a thread
// adds rows ty, ty + 8, ... of its column in a fixed order, the eight sums are combined through shared memory.
__global__ void __launch_bounds__(256) column_reduce_kernel(const float* __restrict__ part, int rows, int H, __nv_bfloat16* out_bf16, float* out_f32) {
  __shared__ float red[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (c < H) {
#pragma unroll 4
    for (int r = threadIdx.y; r < rows; r += 8) acc += part[static_cast<long long>(r) * H + c];
  }
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) t += red[y][threadIdx.x];
    if (out_bf16 != nullptr) out_bf16[c] = __float2bfloat16_rn(t);
    if (out_f32 != nullptr) out_f32[c] = t;
  }
}

// Column sums of a bf16 matrix [rows, H] (bias gradient): strip partials then reduce.
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, long long rows, int H, float* __restrict__ part) {
  // block = 32 x 8 threads; a block handles 256 columns (8 per thread along x) for a strip of rows
  const int col0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const bool active = col0 < H;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (long long r = blockIdx.y * 8 + threadIdx.y; active && r < rows; r += static_cast<long long>(gridDim.y) * 8) {
    const Vec16<__nv_bfloat16> t = ld16(x + r * H + col0);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += __bfloat162float(t.v[k]);
  }
  __shared__ float red[8][32][9];
#pragma unroll
  for (int k = 0; k < 8; ++k) red[threadIdx.y][threadIdx.x][k] = acc[k];
  __syncthreads();
  if (threadIdx.y == 0 && active) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float s = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) s += red[y][threadIdx.x][k];
      part[static_cast<long long>(blockIdx.y) * H + col0 + k] = s;
    }
  }
}

}  // namespace fsb

// H must be a multiple of 8 and <= 8192. mean/rstd are fp32 [rows]. rms != 0 selects RMSNorm
// (beta and mean ignored).
template <bool RMS>
static void launch_norm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* g, const __nv_bfloat16* b, __nv_bfloat16* y, float* mean,
                            float* rstd, long long rows, int H, float eps, cudaStream_t stream) {
  using namespace fsb;
  const unsigned grid = static_cast<unsigned>((rows + NORM_WARPS - 1) / NORM_WARPS);
  const int vpl = (H / 8 + 31) / 32;
  if (vpl <= 2)       norm_fwd_warp_kernel<RMS, 2><<<grid, NORM_WARPS * 32, 0, stream>>>(x, g, b, y, mean, rstd, rows, H, eps);
  else if (vpl <= 4)  norm_fwd_warp_kernel<RMS, 4><<<grid, NORM_WARPS * 32, 0, stream>>>(x, g, b, y, mean, rstd, rows, H, eps);
  else if (vpl <= 8)  norm_fwd_warp_kernel<RMS, 8><<<grid, NORM_WARPS * 32, 0, stream>>>(x, g, b, y, mean, rstd, rows, H, eps);
  else if (vpl <= 16) norm_fwd_warp_kernel<RMS, 16><<<grid, NORM_WARPS * 32, 0, stream>>>(x, g, b, y, mean, rstd, rows, H, eps);
  else norm_fwd_kernel<RMS><<<static_cast<unsigned>(rows), NORM_THREADS, 0, stream>>>(x, g, b, y, mean, rstd, H, eps);
}

template <bool RMS>
static void launch_norm_bwd_dx(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* g, const float* mean,
                               const float* rstd, __nv_bfloat16* dx, long long rows, int H, cudaStream_t stream) {
  using namespace fsb;
  const unsigned grid = static_cast<unsigned>((rows + NORM_WARPS - 1) / NORM_WARPS);
  const int vpl = (H / 8 + 31) / 32;
  if (vpl <= 2)       norm_bwd_dx_warp_kernel<RMS, 2><<<grid, NORM_WARPS * 32, 0, stream>>>(dy, x, g, mean, rstd, dx, rows, H);
  else if (vpl <= 4)  norm_bwd_dx_warp_kernel<RMS, 4><<<grid, NORM_WARPS * 32, 0, stream>>>(dy, x, g, mean, rstd, dx, rows, H);
  else if (vpl <= 8)  norm_bwd_dx_warp_kernel<RMS, 8><<<grid, NORM_WARPS * 32, 0, stream>>>(dy, x, g, mean, rstd, dx, rows, H);
  else norm_bwd_dx_kernel<RMS><<<static_cast<unsigned>(rows), NORM_THREADS, 0, stream>>>(dy, x, g, mean, rstd, dx, H);
}

FSB_API int fsb_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                         long long rows, int H, float eps, int rms, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H > 8 * NORM_THREADS * NORM_MAX_VEC) return -1;
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  auto* gg = static_cast<const __nv_bfloat16*>(gamma);
  auto* bb = static_cast<const __nv_bfloat16*>(beta);
  auto* yy = static_cast<__nv_bfloat16*>(y);
  if (rms) launch_norm_fwd<true>(xx, gg, bb, yy, mean, rstd, rows, H, eps, stream);
  else     launch_norm_fwd<false>(xx, gg, bb, yy, mean, rstd, rows, H, eps, stream);
  return static_cast<int>(cudaGetLastError());
}

// Rows of fp32 partials the backward needs room for: the fused kernel (H <= 2048) writes one row per CTA of its
// persistent grid (two CTAs per SM, never more CTAs than groups of four rows), the two-kernel path at most 48.
constexpr int NORM_FUSED_MAX_H = 2048;
constexpr int NORM_FUSED_MAX_CTAS = 2 * 148;

static int norm_bwd_fused_ctas(long long rows) {
  const long long want = (rows + fsb::NORM_WARPS - 1) / fsb::NORM_WARPS;
  return static_cast<int>(want < 1 ? 1 : (want > NORM_FUSED_MAX_CTAS ? NORM_FUSED_MAX_CTAS : want));
}
static int norm_bwd_split_strips(long long rows) {
  const long long want = (rows + 7) / 8;
  return static_cast<int>(want < 1 ? 1 : (want > 48 ? 48 : want));
}

FSB_API int fsb_norm_bwd_num_strips(long long rows) {
  const int a = norm_bwd_fused_ctas(rows), b = norm_bwd_split_strips(rows);
  return a > b ? a : b;
}

template <bool RMS>
static void launch_norm_bwd_fused(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* g, const float* mean, const float* rstd,
                                  __nv_bfloat16* dx, float* pg, float* pb, long long rows, int H, int ctas, cudaStream_t stream) {
  using namespace fsb;
  const size_t smem = static_cast<size_t>(NORM_WARPS) * H * sizeof(float);  // <= 32 KB
  const int vpl = (H / 8 + 31) / 32;
  if (vpl <= 2)      norm_bwd_fused_kernel<RMS, 2><<<ctas, NORM_WARPS * 32, smem, stream>>>(dy, x, g, mean, rstd, dx, pg, pb, rows, H);
  else if (vpl <= 4) norm_bwd_fused_kernel<RMS, 4><<<ctas, NORM_WARPS * 32, smem, stream>>>(dy, x, g, mean, rstd, dx, pg, pb, rows, H);
  else               norm_bwd_fused_kernel<RMS, 8><<<ctas, NORM_WARPS * 32, smem, stream>>>(dy, x, g, mean, rstd, dx, pg, pb, rows, H);
}

// partials: fp32 workspace of 2 * n_strips * H floats (n_strips from fsb_norm_bwd_num_strips).
// dgamma / dbeta are bf16 [H] outputs (dbeta may be null, and is ignored for RMSNorm).
FSB_API int fsb_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, void* dx,
                         void* dgamma, void* dbeta, float* partials, long long rows, int H, int rms, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H > 8 * NORM_THREADS * NORM_MAX_VEC) return -1;
  const bool fused = H <= NORM_FUSED_MAX_H;
  const int strips = fused ? norm_bwd_fused_ctas(rows) : norm_bwd_split_strips(rows);
  float* pg = partials;
  float* pb = partials + static_cast<long long>(strips) * H;
  auto* d = static_cast<const __nv_bfloat16*>(dy);
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  auto* gg = static_cast<const __nv_bfloat16*>(gamma);
  auto* o = static_cast<__nv_bfloat16*>(dx);
  const bool want_beta = !rms && dbeta != nullptr;
  if (fused) {
    if (rms) launch_norm_bwd_fused<true>(d, xx, gg, mean, rstd, o, pg, nullptr, rows, H, strips, stream);
    else     launch_norm_bwd_fused<false>(d, xx, gg, mean, rstd, o, pg, want_beta ? pb : nullptr, rows, H, strips, stream);
  } else {
    dim3 block(32, 8), grid((H / 8 + 31) / 32, strips);
    if (rms) {
      launch_norm_bwd_dx<true>(d, xx, gg, mean, rstd, o, rows, H, stream);
      norm_dparam_partial_kernel<true><<<grid, block, 0, stream>>>(d, xx, mean, rstd, pg, nullptr, rows, H);
    } else {
      launch_norm_bwd_dx<false>(d, xx, gg, mean, rstd, o, rows, H, stream);
      norm_dparam_partial_kernel<false><<<grid, block, 0, stream>>>(d, xx, mean, rstd, pg, want_beta ? pb : nullptr, rows, H);
    }
  }
  const dim3 threads(32, 8);
  const int blocks = (H + 31) / 32;
  column_reduce_kernel<<<blocks, threads, 0, stream>>>(pg, strips, H, static_cast<__nv_bfloat16*>(dgamma), nullptr);
  if (want_beta) column_reduce_kernel<<<blocks, threads, 0, stream>>>(pb, strips, H, static_cast<__nv_bfloat16*>(dbeta), nullptr);
  return static_cast<int>(cudaGetLastError());
}

FSB_API int fsb_colsum_num_strips(long long rows) {
  const long long want = (rows + 63) / 64;
  return static_cast<int>(want < 1 ? 1 : (want > 48 ? 48 : want));
}

// out[c] = sum_r x[r, c]; x bf16 [rows, H] (H % 8 == 0); partials fp32 [n_strips, H]; out bf16 [H].
FSB_API int fsb_colsum(const void* x, long long rows, int H, float* partials, void* out, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0 || H <= 0) return 0;
  if (H % 8 != 0) return -1;
  const int strips = fsb_colsum_num_strips(rows);
  dim3 block(32, 8), grid((H / 8 + 31) / 32, strips);
  colsum_partial_kernel<<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), rows, H, partials);
  const dim3 threads(32, 8);
  const int blocks = (H + 31) / 32;
  column_reduce_kernel<<<blocks, threads, 0, stream>>>(partials, strips, H, static_cast<__nv_bfloat16*>(out), nullptr);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free column sum (declared in fsb_no_alloc.h; no counterpart in the reference library).
// The strip partials go to a fixed array in device memory instead of a workspace from the caller.
// ---------------------------------------------------------------------------------------------------------
#include <mutex>

#include "fsb_no_alloc.h"

namespace {
constexpr int kStaticStrips = 48;   // upper bound of fsb_colsum_num_strips
constexpr int kMaxDevices = 64;
static __device__ __align__(256) float g_colsum_scratch[kStaticStrips * FSB_COLSUM_STATIC_MAX_H];
float* g_colsum_scratch_ptr[kMaxDevices] = {};
std::mutex g_colsum_scratch_mutex;

// Device address of the scratch array on the current device; resolved once per device.
int colsum_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return FSB_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_colsum_scratch_mutex);
  if (g_colsum_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return FSB_NOALLOC_ERR_SYMBOL;
    }
    g_colsum_scratch_ptr[dev] = p;
  }
  *out = g_colsum_scratch_ptr[dev];
  return 0;
}
}  // namespace

FSB_API int fsb_colsum_static_max_h(void) { return FSB_COLSUM_STATIC_MAX_H; }

FSB_API const char* fsb_colsum_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case FSB_NOALLOC_ERR_SHAPE: return "fsb_colsum_static: H must be a multiple of 8";
    case FSB_NOALLOC_ERR_TOO_LARGE: return "fsb_colsum_static: H exceeds FSB_COLSUM_STATIC_MAX_H (8192); call fsb_colsum with a caller-provided workspace";
    case FSB_NOALLOC_ERR_DEVICE: return "fsb_colsum_static: device ordinal beyond the 64 devices the library tracks";
    case FSB_NOALLOC_ERR_SYMBOL: return "fsb_colsum_static: could not resolve the built-in workspace on this device";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "fsb_colsum_static: unknown error";
  }
}

FSB_API int fsb_colsum_static(const void* x, long long rows, int H, void* out, cudaStream_t stream) {
  using namespace fsb;
  if (rows <= 0 || H <= 0) return 0;
  if (H % 8 != 0) return FSB_NOALLOC_ERR_SHAPE;
  if (H > FSB_COLSUM_STATIC_MAX_H) return FSB_NOALLOC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = colsum_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  const int strips = fsb_colsum_num_strips(rows);  // <= kStaticStrips
  dim3 block(32, 8), grid((H / 8 + 31) / 32, strips);
  // every (strip, column < H) element read by the reduction below is written here first: no clearing needed
  colsum_partial_kernel<<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), rows, H, scratch);
  const dim3 threads(32, 8);
  const int blocks = (H + 31) / 32;
  column_reduce_kernel<<<blocks, threads, 0, stream>>>(scratch, strips, H, static_cast<__nv_bfloat16*>(out), nullptr);
  return static_cast<int>(cudaGetLastError());
}
