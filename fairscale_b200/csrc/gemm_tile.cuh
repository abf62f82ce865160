// Pieces shared by the tcgen05 GEMM kernels: tile constants, the shared-memory layout of the operand ring,
// the L2-friendly tile order and the fused epilogue that drains one TMEM accumulator into global memory.
#pragma once

#include "sm100.cuh"

namespace fsb {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // 64 bf16 = 128 B = one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int GEMM_THREADS = 192;

enum Epilogue : int {
  EPI_NONE = 0,           // C = acc
  EPI_BIAS = 1,           // C = acc + bias[n]
  EPI_BIAS_GELU = 2,      // C = gelu(acc + bias[n]);  aux_out (optional) = acc + bias[n]
  EPI_BIAS_RESIDUAL = 3,  // C = acc + bias[n] + aux[m,n]
  EPI_DGELU = 4,          // C = acc * gelu'(aux[m,n])
  EPI_RESIDUAL = 5,       // C = acc + aux[m,n]
};

struct GemmParams {
  void* C;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux;
  __nv_bfloat16* aux_out;
  int M, N, K;
  int ldc, ld_aux;
  int a_mn_major, b_mn_major;
  int epilogue;
  int out_f32;       // C is fp32 (else bf16)
  int accumulate_c;  // C += result (fp32 output only)
  int* status;
  // batched (grouped) products: `batch` independent problems of the same shape; element strides between them
  int batch;
  long long stride_c, stride_aux, stride_bias;
  // dynamic tile scheduler of the CTA-pair kernel: sched[0] = next tile to hand out, sched[1] = pairs that have finished
  // (both zero before the launch; the last pair to finish resets them)
  unsigned int* sched;
  // Optional arrival flags of the B operand (CTA-pair kernel, B K-major with contiguous rows): the operand is being
  // written by somebody else (copy engines gathering a sharded weight) while the kernel runs.  Bytes
  // [i * b_piece_bytes, (i + 1) * b_piece_bytes) of B are valid once b_ready[i] >= b_ready_epoch (epochs only grow).
  // Pieces are sent cyclically starting with piece b_first_piece (ranks start at different pieces, so that they do not
  // all pull from the same source at once) and flags are indexed in sending order: piece q raises
  // b_ready[(q - b_first_piece) mod b_num_pieces].  Tiles are visited N-major in the same cyclic order.
  const unsigned int* b_ready;
  unsigned int b_ready_epoch;
  long long b_piece_bytes;
  unsigned long long b_wait_ns;
  int b_first_piece, b_num_pieces;
  // Optional arrival flags of the A operand (CTA-pair kernel, A K-major): A is the concatenation of `a_num_shards` row
  // blocks of `a_shard_rows` rows that arrive block by block, block `a_first_shard` first (it is this rank's own), then
  // the following ones cyclically, each in pieces of `a_piece_rows` rows.  Piece j of the k-th arriving block is valid
  // once a_ready[k * pieces_per_block + j] >= a_ready_epoch; flags are raised in that order.  Tiles are visited M-major
  // in arrival order.  Waits are bounded by b_wait_ns.
  const unsigned int* a_ready;
  unsigned int a_ready_epoch;
  int a_shard_rows, a_piece_rows, a_first_shard, a_num_shards;
};

// Parameters of problem `b` of a batch (pointers advanced; everything else shared).
__device__ __forceinline__ GemmParams gemm_params_of_batch(const GemmParams& p, int b) {
  GemmParams q = p;
  if (p.out_f32) q.C = reinterpret_cast<float*>(p.C) + b * p.stride_c;
  else           q.C = reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.stride_c;
  if (p.bias != nullptr) q.bias = p.bias + b * p.stride_bias;
  if (p.aux != nullptr) q.aux = p.aux + b * p.stride_aux;
  if (p.aux_out != nullptr) q.aux_out = p.aux_out + b * p.stride_aux;
  return q;
}

template <int BLOCK_N>
struct SmemLayout {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int EPI_OFFSET = BAR_OFFSET + 256;     // 4 KB of epilogue staging per epilogue warp (4 warps)
  static constexpr int TOTAL = EPI_OFFSET + 4 * 4096 + 1024;  // + slack for 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Groups of 16 M-tiles walk N together, so concurrently running CTAs share A and B slabs in L2.
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

// Drain one accumulator (this warp's 32 lanes x BLOCK_N columns starting at TMEM address t_base) through the
// fused epilogue into global memory. `row` is the global output row owned by this thread.
template <int BLOCK_N>
__device__ __forceinline__ void epilogue_rows(uint32_t t_base, int row, int n0, const GemmParams& p) {
  const bool row_ok = row < p.M;
  const bool vec_ok = (p.ldc % 8 == 0) && (p.ld_aux % 8 == 0);
#pragma unroll 1
  for (int c = 0; c < BLOCK_N / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_base + static_cast<uint32_t>(c * 32), r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (!row_ok || col0 >= p.N) continue;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    const bool full = vec_ok && (col0 + 32 <= p.N);
    const int epi = p.epilogue;
    if (epi == EPI_BIAS || epi == EPI_BIAS_GELU || epi == EPI_BIAS_RESIDUAL) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
    }
    if (epi == EPI_BIAS_GELU) {
      if (p.aux_out != nullptr) {
        __nv_bfloat16* po = p.aux_out + static_cast<size_t>(row) * p.ld_aux + col0;
        if (full) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            Vec16<__nv_bfloat16> o;
#pragma unroll
            for (int i = 0; i < 8; ++i) o.v[i] = __float2bfloat16_rn(v[q * 8 + i]);
            st16(po + q * 8, o);
          }
        } else {
          for (int i = 0; i < 32 && col0 + i < p.N; ++i) po[i] = __float2bfloat16_rn(v[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = gelu_erf(v[i]);
    } else if (epi == EPI_BIAS_RESIDUAL || epi == EPI_RESIDUAL || epi == EPI_DGELU) {
      const __nv_bfloat16* pa = p.aux + static_cast<size_t>(row) * p.ld_aux + col0;
      float a[32];
      if (full) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          Vec16<__nv_bfloat16> x = ld16(pa + q * 8);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[q * 8 + i] = __bfloat162float(x.v[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) a[i] = (col0 + i < p.N) ? __bfloat162float(pa[i]) : 0.f;
      }
      if (epi == EPI_DGELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= gelu_erf_grad(a[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += a[i];
      }
    }
    if (p.out_f32) {
      float* pc = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
      if (p.accumulate_c) {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) pc[i] += v[i];
      } else if (col0 + 32 <= p.N && (p.ldc % 4 == 0)) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(pc + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
      } else {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) pc[i] = v[i];
      }
    } else {
      __nv_bfloat16* pc = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
      if (full) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          Vec16<__nv_bfloat16> o;
#pragma unroll
          for (int i = 0; i < 8; ++i) o.v[i] = __float2bfloat16_rn(v[q * 8 + i]);
          st16(pc + q * 8, o);
        }
      } else {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) pc[i] = __float2bfloat16_rn(v[i]);
      }
    }
  }
}


// ------------------------------------------------------------------------------------------------
// Coalesced epilogue for bf16 outputs.  A warp owns 32 accumulator rows (one TMEM lane quadrant) and walks its
// columns in slabs of 64.  Thread = row when it reads TMEM and does the math, but global memory is touched
// with 8 lanes per row (8 x 16 B = one 128-byte line, 4 rows per instruction): the slab is transposed through a
// warp-private, XOR-swizzled 4 KB staging buffer in shared memory, in both directions (aux in, C / aux_out out).
// `stage` is this warp's buffer; ncols is a multiple of 64.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t epi_swz(int row, int chunk) {  // byte offset of 16-byte chunk `chunk` of `row`
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// global [32 rows x 64 cols] bf16 slab -> staging (coalesced reads)
__device__ __forceinline__ void epi_slab_load(uint8_t* stage, const __nv_bfloat16* g, int ld, int row0, int col0, int M, int N, int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rr = it * 4 + (lane >> 3);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + rr < M && col0 + cc * 8 < N) v = *reinterpret_cast<const uint4*>(g + static_cast<size_t>(row0 + rr) * ld + col0 + cc * 8);
    *reinterpret_cast<uint4*>(stage + epi_swz(rr, cc)) = v;
  }
}
// The same slab in two steps: global -> registers (issued early, e.g. before the accumulator is ready, so the DRAM
// latency overlaps other work) and registers -> staging.
__device__ __forceinline__ void epi_slab_prefetch(uint4 (&pre)[8], const __nv_bfloat16* g, int ld, int row0, int col0, int M, int N, int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rr = it * 4 + (lane >> 3);
    pre[it] = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + rr < M && col0 + cc * 8 < N) pre[it] = __ldcg(reinterpret_cast<const uint4*>(g + static_cast<size_t>(row0 + rr) * ld + col0 + cc * 8));
  }
}
__device__ __forceinline__ void epi_slab_commit(uint8_t* stage, const uint4 (&pre)[8], int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) *reinterpret_cast<uint4*>(stage + epi_swz(it * 4 + (lane >> 3), cc)) = pre[it];
}
__device__ __forceinline__ bool epilogue_needs_aux(int epi) { return epi == EPI_BIAS_RESIDUAL || epi == EPI_RESIDUAL || epi == EPI_DGELU; }

// staging -> global [32 rows x 64 cols] bf16 slab (coalesced writes)
__device__ __forceinline__ void epi_slab_store(const uint8_t* stage, __nv_bfloat16* g, int ld, int row0, int col0, int M, int N, int lane) {
  const int cc = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rr = it * 4 + (lane >> 3);
    if (row0 + rr < M && col0 + cc * 8 < N)
      *reinterpret_cast<uint4*>(g + static_cast<size_t>(row0 + rr) * ld + col0 + cc * 8) = *reinterpret_cast<const uint4*>(stage + epi_swz(rr, cc));
  }
}
// this thread's row of the slab: 64 floats -> staging as bf16
__device__ __forceinline__ void epi_row_to_stage(uint8_t* stage, const float (&v)[64], int lane) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    Vec16<__nv_bfloat16> o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = __float2bfloat16_rn(v[c * 8 + i]);
    *reinterpret_cast<uint4*>(stage + epi_swz(lane, c)) = o.raw;
  }
}

// `pre` holds the aux slab of the first 64 columns when the epilogue reads aux (see epi_slab_prefetch; the caller loads
// it before it waits for the accumulator); the slabs after the first are prefetched here while the previous one drains.
__device__ __forceinline__ void epilogue_rows_coalesced(uint32_t t_base, int row0, int n0, int ncols, const GemmParams& p, uint8_t* stage, int lane,
                                                        uint4 (&pre)[8]) {
  const int epi = p.epilogue;
  const bool needs_aux = epilogue_needs_aux(epi);
  for (int c0 = 0; c0 < ncols; c0 += 64) {
    const int col0 = n0 + c0;
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(t_base + static_cast<uint32_t>(c0), r0);
    tmem_ld_32x32(t_base + static_cast<uint32_t>(c0 + 32), r1);
    if (needs_aux && col0 < p.N) epi_slab_commit(stage, pre, lane);  // overlaps the TMEM load
    tmem_ld_wait();
    if (col0 >= p.N) continue;  // warp-uniform
    float v[64];
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] = __uint_as_float(r0[i]); v[32 + i] = __uint_as_float(r1[i]); }
    if (epi == EPI_BIAS || epi == EPI_BIAS_GELU || epi == EPI_BIAS_RESIDUAL) {
      if ((reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (col0 + c * 8 < p.N) {
            const Vec16<__nv_bfloat16> b = ld16(p.bias + col0 + c * 8);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[c * 8 + i] += __bfloat162float(b.v[i]);
          }
        }
      } else {  // a bias that is a view into a flat parameter may start at any element
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
      }
    }
    if (needs_aux) {
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        Vec16<__nv_bfloat16> a;
        a.raw = *reinterpret_cast<const uint4*>(stage + epi_swz(lane, c));
        if (epi == EPI_DGELU) {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c * 8 + i] *= gelu_erf_grad(__bfloat162float(a.v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c * 8 + i] += __bfloat162float(a.v[i]);
        }
      }
      __syncwarp();
      if (c0 + 64 < ncols && col0 + 64 < p.N) epi_slab_prefetch(pre, p.aux, p.ld_aux, row0, col0 + 64, p.M, p.N, lane);
    }
    if (epi == EPI_BIAS_GELU) {
      if (p.aux_out != nullptr) {
        epi_row_to_stage(stage, v, lane);
        __syncwarp();
        epi_slab_store(stage, p.aux_out, p.ld_aux, row0, col0, p.M, p.N, lane);
        __syncwarp();
      }
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = gelu_erf(v[i]);
    }
    epi_row_to_stage(stage, v, lane);
    __syncwarp();
    epi_slab_store(stage, reinterpret_cast<__nv_bfloat16*>(p.C), p.ldc, row0, col0, p.M, p.N, lane);
    __syncwarp();
  }
}

// bf16 output with 16-byte aligned rows: the layouts the coalesced epilogue handles
__device__ __forceinline__ bool epilogue_can_coalesce(const GemmParams& p) {
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(p.C) | reinterpret_cast<uintptr_t>(p.aux) | reinterpret_cast<uintptr_t>(p.aux_out);
  return !p.out_f32 && (p.ldc % 8 == 0) && (p.ld_aux % 8 == 0) && (p.N % 8 == 0) && (ptrs & 15u) == 0;
}

}  // namespace fsb
