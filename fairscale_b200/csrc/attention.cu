// Causal flash attention (forward + backward) on tcgen05 / TMEM for packed QKV.
//
//   qkv : bf16 [B, S, 3, H, D]   (the output of the fused QKV projection, untouched)
//   o   : bf16 [B, S, H, D]      lse : fp32 [B, H, S]   (natural-log sum-exp of the scaled scores)
//
// All tiles are fetched straight from the packed tensor with per-CTA TMA loads (no permute / contiguous /
// cat glue kernels) and every product runs on the tensor cores with fp32 accumulators in TMEM:
//
//   forward (one CTA per 128 query rows)       S = Q K^T -> online softmax -> O += P V
//   backward dQ (one CTA per 128 query rows)   S = Q K^T, dP = dO V^T -> dS -> dQ += dS K
//   backward dK/dV (one CTA per 128 key rows)  S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T -> dV += P^T dO, dK += dS^T Q
//
// Thread roles per CTA (320 threads): warp 0 TMA producer, warp 1 MMA issuer (+TMEM allocation), warps 2..9
// "softmax" threads: two threads per accumulator row (TMEM lane == row; warps w and w+4 share a lane quadrant and
// take half of the columns each, so every scheduler has two warps to interleave), which do the exponentials in
// registers and hand the bf16 probabilities back to the tensor cores through 128-byte-swizzled shared memory.
// A K-major tile [rows, 64] and an MN-major tile of the same bytes differ only in the MMA descriptor, so each
// streamed tile is loaded once and used both as a "transposed" and a "plain" operand.
// Every mbarrier wait is bounded (see sm100.cuh).
//
// Replaces nn.MultiheadAttention / bmm+softmax in the reference's models
// (benchmarks/models/transformer_lm.py:107,150-152,169-183).

#include "sm100.cuh"

#include <cstdlib>

namespace fsb {

constexpr int ATT_THREADS = 320;  // TMA warp + MMA warp + 8 compute warps (two per TMEM lane quadrant, half the columns each)
constexpr int ATT_BM = 128;  // rows owned by a CTA (TMEM lanes)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct AttnParams {
  int B, S, H, D;
  float scale;        // softmax scale (1/sqrt(D))
  __nv_bfloat16* o;   // fwd out / bwd in   [B*S, H*D]
  float* lse;         // [B, H, S]
  const float* delta; // [2, B, H, S]: scale * rowsum(dO * O), then the base-2 lse (both written by attn_delta_kernel)
  __nv_bfloat16* dqkv;  // [B*S, 3*H*D]
  int* status;
  unsigned long long* trace;  // optional timeline of CTA (0,0,0) of the forward kernel: [role][iteration][4] ns stamps
};

#define ATT_TRACE(role, j, k)                                                                                       \
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 64)                     \
    p.trace[((role) * 64 + (j)) * 4 + (k)] = globaltimer_ns();

// byte offset of (row, 16-byte chunk) inside a 128-byte-swizzled [rows x 64 bf16] slab
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

__device__ __forceinline__ float ex2_approx(float x) {  // 2^x on the MUFU pipe, one instruction
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// K-major operand descriptor for k-step `ks` (16 elements) of a tile made of [rows x 64] slabs of `slab_bytes`
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int ks, uint32_t slab_bytes) {
  return make_smem_desc(base + static_cast<uint32_t>(ks >> 2) * slab_bytes + static_cast<uint32_t>(ks & 3) * 32u, 16u, 1024u);
}
// MN-major operand descriptor: the tile is [k_rows x 64] slabs (one per 64 MN elements, `slab_bytes` apart);
// k-step `ks` covers 16 k_rows = 2048 bytes.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int ks, uint32_t slab_bytes) {
  return make_smem_desc(base + static_cast<uint32_t>(ks) * 2048u, slab_bytes, 1024u);
}

struct AttnBars {
  uint64_t stat_full;     // stationary tiles landed
  uint64_t str_full[3];   // streamed stage landed (first operand)
  uint64_t str2_full[2];  // streamed stage landed (second operand)
  uint64_t str_empty[3];  // streamed stage free again (forward: the V half of the stage)
  uint64_t k_empty[2];    // forward: K half of the stage free again (released as soon as S = Q K^T has read it)
  uint64_t s_full[2];     // score accumulator(s) ready in TMEM
  uint64_t s_empty[2];    // score accumulator(s) drained by the softmax threads
  uint64_t p_full;        // probabilities / dS written to shared memory
  uint64_t acc_done;      // accumulate-type MMAs of the iteration finished (P buffer + accumulators free)
  uint64_t acc_done2[2];  // dQ kernel: the same, alternating with the double-buffered dS tile
  uint64_t p_full2[2];    // backward kernels: dS (dQ kernel) / P^T and dS^T (dK/dV kernel) buffer b written.  One barrier per buffer: with a single one the threads could
                          // complete the phase of step u+1 (other buffer) before the MMA warp had observed step u
  uint64_t stat_empty;    // backward (persistent): the item's last products that read the stationary tiles have completed
  uint64_t acc_free;      // backward (persistent): the 8 compute warps have read the item's output accumulators
  uint32_t tmem_slot;
  int abort_flag;
};

struct PairXch {            // forward only: row statistics exchanged between the two threads of a row
  float xch[2][2][ATT_BM];  // [parity][column half][row]
  int xflag[2][2][ATT_BM];  // sequence number of the value in xch (0 = nothing yet)
};

// The two threads of a row swap one float through shared memory.  `seq` (> 0) must differ between consecutive uses of
// a parity slot.  The wait is a bounded poll, not a hardware barrier, so a thread that gave up after a timeout
// elsewhere cannot strand its partner.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool pair_exchange(PairXch* bars, int parity, int half, int row, int seq, float mine, float& other,
                                              volatile int* abort_flag) {
  *reinterpret_cast<volatile float*>(&bars->xch[parity][half][row]) = mine;
  __threadfence_block();
  *reinterpret_cast<volatile int*>(&bars->xflag[parity][half][row]) = seq;
  const volatile int* theirs = &bars->xflag[parity][half ^ 1][row];
  if (*theirs != seq) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (*theirs != seq) {
      if (((++spins) & 127u) == 0u) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > kWaitLimitNs) {
          *abort_flag = 1;
          return false;
        }
      }
    }
  }
  __threadfence_block();
  other = *reinterpret_cast<volatile float*>(&bars->xch[parity][half ^ 1][row]);
  return true;
}

__device__ __forceinline__ void attn_init_bars(AttnBars* b) {
  mbar_init(&b->stat_full, 1);
  mbar_init(&b->str_full[2], 1);
  mbar_init(&b->str_empty[2], 1);
  for (int i = 0; i < 2; ++i) {
    mbar_init(&b->str_full[i], 1);
    mbar_init(&b->str2_full[i], 1);
    mbar_init(&b->str_empty[i], 1);
    mbar_init(&b->k_empty[i], 1);
    mbar_init(&b->s_full[i], 1);
    mbar_init(&b->s_empty[i], 8);
  }
  mbar_init(&b->p_full, 8);
  mbar_init(&b->acc_done, 1);
  mbar_init(&b->acc_done2[0], 1);
  mbar_init(&b->acc_done2[1], 1);
  mbar_init(&b->p_full2[0], 8);
  mbar_init(&b->p_full2[1], 8);
  mbar_init(&b->stat_empty, 1);
  mbar_init(&b->acc_free, 8);
  b->abort_flag = 0;
  fence_barrier_init();
}

__device__ __forceinline__ void attn_teardown(AttnBars* bars, int warp, uint32_t tmem_base, uint32_t ncols, int* status) {
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, FSB_ERR_WAIT_TIMEOUT | (bars->abort_flag << 8));
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, ncols);
  }
}

// Row maximum / exponentials of 64 columns (starting at column `col0`) of a score row held in registers.  Eight
// independent accumulators keep the dependent chains short.
template <bool DIAG>
__device__ __forceinline__ float fwd_row_max(const uint32_t (&sr)[2][32], int col0, int row) {
  float m[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) m[k] = -INFINITY;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float v = __uint_as_float(sr[c][i]);
      if (!DIAG || (col0 + c * 32 + i) <= row) m[i & 7] = fmaxf(m[i & 7], v);
    }
  }
  return fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7])));
}

template <bool DIAG>
__device__ __forceinline__ float fwd_row_exp(const uint32_t (&sr)[2][32], int col0, int row, float sl2, float mb, uint32_t (&pk)[32]) {
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p0 = ex2_approx(fmaf(__uint_as_float(sr[c][i]), sl2, -mb));
      float p1 = ex2_approx(fmaf(__uint_as_float(sr[c][i + 1]), sl2, -mb));
      if (DIAG) {
        if (col0 + c * 32 + i > row) p0 = 0.f;
        if (col0 + c * 32 + i + 1 > row) p1 = 0.f;
      }
      acc[(i >> 1) & 7] += p0 + p1;
      pk[c * 16 + (i >> 1)] = pack_bf16(p0, p1);
    }
  }
  return ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
}

// =================================================================================================
// Forward
// =================================================================================================
template <int D>
struct FwdSmem {
  static constexpr int TILE = ATT_BM * D * 2;  // one [128 x D] bf16 tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;           // 2 stages
  static constexpr int V_OFF = 3 * TILE;       // 2 stages
  static constexpr int P_OFF = 5 * TILE;       // [128 x 128] bf16
  static constexpr int BAR_OFF = P_OFF + ATT_BM * 128 * 2;
  static constexpr int XCH_OFF = BAR_OFF + 256;
  static constexpr int TOTAL = XCH_OFF + 4096 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_qkv, AttnParams p) {
  using L = FwdSmem<D>;
  constexpr int SLABS = D / 64;
  constexpr uint32_t SLAB = ATT_BM * 128;  // bytes of a [128 x 64] slab
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  AttnBars* bars = reinterpret_cast<AttnBars*>(smem + L::BAR_OFF);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = p.S / ATT_BM;
  const int qt = n_qt - 1 - blockIdx.x;  // heavy (long) rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_kv = qt + 1;
  const int HD = p.H * D;
  const int row0 = b * p.S + qt * ATT_BM;
  constexpr uint32_t TMEM_COLS = 512;  // S0 [0,128) S1 [128,256) O [256, 256+D)

  if (threadIdx.x == 0) {
    attn_init_bars(bars);
    tma_prefetch_desc(&tm_qkv);
  }
  PairXch* xch = reinterpret_cast<PairXch*>(smem + L::XCH_OFF);
  for (int i = threadIdx.x; i < 2 * 2 * ATT_BM; i += ATT_THREADS) (&xch->xflag[0][0][0])[i] = 0;
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars->stat_full, L::TILE);
#pragma unroll
      for (int c = 0; c < SLABS; ++c) tma_load_2d(smem + L::Q_OFF + c * SLAB, &tm_qkv, &bars->stat_full, h * D + c * 64, row0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&bars->k_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag)) break;
        ATT_TRACE(0, j, 0)
        const int krow = b * p.S + j * ATT_BM;
        mbar_expect_tx(&bars->str_full[st], L::TILE);
#pragma unroll
        for (int c = 0; c < SLABS; ++c)
          tma_load_2d(smem + L::K_OFF + st * L::TILE + c * SLAB, &tm_qkv, &bars->str_full[st], HD + h * D + c * 64, krow);
        if (!mbar_wait(&bars->str_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag)) break;
        ATT_TRACE(0, j, 1)
        mbar_expect_tx(&bars->str2_full[st], L::TILE);
#pragma unroll
        for (int c = 0; c < SLABS; ++c)
          tma_load_2d(smem + L::V_OFF + st * L::TILE + c * SLAB, &tm_qkv, &bars->str2_full[st], 2 * HD + h * D + c * 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(ATT_BM, 128, true, false, false);  // Q K^T : both K-major
      const uint32_t idesc_o = make_idesc_f16(ATT_BM, D, true, false, true);     // P V   : V is MN-major
      const uint32_t sq = smem_u32(smem + L::Q_OFF), sp = smem_u32(smem + L::P_OFF);
      bool ok = mbar_wait(&bars->stat_full, 0, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&bars->str_full[st], (j >> 1) & 1, abort_flag)) return false;
        ATT_TRACE(1, j, 0)
        if (!mbar_wait(&bars->s_empty[st], ((j >> 1) & 1) ^ 1u, abort_flag)) return false;
        ATT_TRACE(1, j, 1)
        tc_fence_after_sync();
        const uint32_t sk = smem_u32(smem + L::K_OFF + st * L::TILE);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16_ss(tmem_base + st * 128, desc_kmajor(sq, ks, SLAB), desc_kmajor(sk, ks, SLAB), idesc_s, ks != 0);
        umma_commit(&bars->s_full[st]);
        umma_commit(&bars->k_empty[st]);  // the K tile can be refilled while the softmax and P V of this step run
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) { if (!issue_s(j + 1)) { ok = false; break; } }
        const int st = j & 1;
        if (!mbar_wait(&bars->p_full, j & 1, abort_flag)) { ok = false; break; }
        ATT_TRACE(1, j, 2)
        if (!mbar_wait(&bars->str2_full[st], (j >> 1) & 1, abort_flag)) { ok = false; break; }
        ATT_TRACE(1, j, 3)
        tc_fence_after_sync();
        const uint32_t sv = smem_u32(smem + L::V_OFF + st * L::TILE);
#pragma unroll
        for (int ks = 0; ks < 128 / 16; ++ks)
          umma_f16_ss(tmem_base + 256, desc_kmajor(sp, ks, SLAB), desc_mnmajor(sv, ks, SLAB), idesc_o, (j | ks) != 0);
        umma_commit(&bars->str_empty[st]);
        umma_commit(&bars->acc_done);
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;   // which 64 of the 128 score columns (and which D/2 of the output columns)
    const int row = quad * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's share of the row sum
    uint8_t* sp = smem + L::P_OFF;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int st = j & 1;
      if (!mbar_wait(&bars->s_full[st], (j >> 1) & 1, abort_flag)) { ok = false; break; }
      if (warp == 2 && lane == 0) { ATT_TRACE(2, j, 0) }
      tc_fence_after_sync();
      const uint32_t ts = tmem_base + st * 128 + half * 64 + lane_off;
      const bool diag = (j == qt);
      uint32_t sr[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld_32x32(ts + c * 32, sr[c]);
      tmem_ld_wait();
      if (warp == 2 && lane == 0) { ATT_TRACE(3, j, 0) }
      // Tiles below the diagonal need no mask; only the last tile of a CTA pays for the comparisons.
      float mx, other;
      if (!diag) mx = fwd_row_max<false>(sr, half * 64, row); else mx = fwd_row_max<true>(sr, half * 64, row);
      if (warp == 2 && lane == 0) { ATT_TRACE(3, j, 1) }
      if (!__all_sync(0xffffffffu, pair_exchange(xch, j & 1, half, row, j + 1, mx, other, abort_flag))) { ok = false; break; }
      if (warp == 2 && lane == 0) { ATT_TRACE(3, j, 2) }
      mx = fmaxf(mx, other);
      // Keep the old maximum while the new one is at most 2^8 above it: the probabilities stay well inside the
      // bf16 / fp32 range and O needs no rescaling (the final 1 / l normalisation uses the same maximum).
      float m_new = fmaxf(m_run, mx);
      if (m_run != -INFINITY && (m_new - m_run) * sl2 <= 8.f) m_new = m_run;
      const float alpha = (m_run == -INFINITY) ? 0.f : ex2_approx((m_run - m_new) * sl2);
      const float mb = m_new * sl2;
      uint32_t pk[32];
      float rs;
      if (!diag) rs = fwd_row_exp<false>(sr, half * 64, row, sl2, mb, pk); else rs = fwd_row_exp<true>(sr, half * 64, row, sl2, mb, pk);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_empty[st]);
      if (warp == 2 && lane == 0) { ATT_TRACE(2, j, 1) }
      // O and the P buffer belong to the previous P V product until it has completed
      if (j > 0) {
        if (!mbar_wait(&bars->acc_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
        if (warp == 2 && lane == 0) { ATT_TRACE(2, j, 2) }
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < D / 64; ++c) {
            const uint32_t to = tmem_base + 256 + lane_off + half * (D / 2) + c * 32;
            uint32_t r[32];
            tmem_ld_32x32(to, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) { lo[i] = r[i]; hi[i] = r[16 + i]; }
            tmem_st_32x16(to, lo);
            tmem_st_32x16(to + 16, hi);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {  // this thread's 8 chunks of 8 bf16 = its half of the row of P
        const uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(sp + half * SLAB + swz(row, ch)) = v;
      }
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
      if (warp == 2 && lane == 0) { ATT_TRACE(2, j, 3) }
      l_run = l_run * alpha + rs;
      m_run = m_new;
    }
    if (ok && mbar_wait(&bars->acc_done, (n_kv - 1) & 1, abort_flag)) {
      tc_fence_after_sync();
      float l_other = 0.f;
      const bool got = __all_sync(0xffffffffu, pair_exchange(xch, n_kv & 1, half, row, n_kv + 1, l_run, l_other, abort_flag));
      const float l_tot = l_run + l_other;
      const float inv = got ? 1.f / l_tot : 0.f;
      __nv_bfloat16* orow = p.o + static_cast<size_t>(row0 + row) * HD + h * D + half * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + 256 + lane_off + half * (D / 2) + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
          v.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
          v.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
          v.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = v;
        }
      }
      if (half == 0 && p.lse != nullptr)
        p.lse[(static_cast<size_t>(b) * p.H + h) * p.S + qt * ATT_BM + row] = (m_run * sl2 + log2f(l_tot)) * LN2;
    }
  }
  attn_teardown(bars, warp, tmem_base, TMEM_COLS, p.status);
}

// dS for 32 columns (starting at key column `col0` of the 128-key tile) of one row:
// P = 2^(s * sl2 - lse2), dS = P * (dP * scale - delta * scale)
template <bool DIAG>
__device__ __forceinline__ void dq_cols32(const uint32_t (&rs)[32], const uint32_t (&rp)[32], int col0, int row, float sl2,
                                          float lse2, float scale, float delta_s, uint32_t (&pk)[16]) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float p0 = ex2_approx(fmaf(__uint_as_float(rs[i]), sl2, -lse2));
    float p1 = ex2_approx(fmaf(__uint_as_float(rs[i + 1]), sl2, -lse2));
    if (DIAG) {
      if (col0 + i > row) p0 = 0.f;
      if (col0 + i + 1 > row) p1 = 0.f;
    }
    pk[i >> 1] = pack_bf16(p0 * fmaf(__uint_as_float(rp[i]), scale, -delta_s), p1 * fmaf(__uint_as_float(rp[i + 1]), scale, -delta_s));
  }
}

// =================================================================================================
// Backward, dQ: one CTA per 128 query rows; streams K and V tiles and consumes them in two steps of 64 keys, so that
// S / dP fit TMEM twice and the products of step u+1 overlap the exponentials of step u.
// =================================================================================================
template <int D>
struct DqSmem {
  static constexpr int TILE = ATT_BM * D * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int DO_OFF = TILE;
  static constexpr int K_OFF = 2 * TILE;   // 2 stages
  static constexpr int V_OFF = 4 * TILE;   // 2 stages
  static constexpr int DS_OFF = 6 * TILE;  // two [128 x 64] bf16 buffers
  static constexpr int BAR_OFF = DS_OFF + ATT_BM * 128 * 2;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qkv, const __grid_constant__ CUtensorMap tm_do, AttnParams p) {
  using L = DqSmem<D>;
  constexpr int SLABS = D / 64;
  constexpr uint32_t SLAB = ATT_BM * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  AttnBars* bars = reinterpret_cast<AttnBars*>(smem + L::BAR_OFF);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // warp-uniform
  // Persistent: one CTA per SM walks the work items (one 128-row query tile of one head), long rows first, dealt
  // round-robin; TMEM, barriers and the K / V ring live for the whole kernel (running counters give the phases).
  const int n_qt = p.S / ATT_BM;
  const int HB = p.H * p.B;
  const int n_items = n_qt * HB;
  const int HD = p.H * D;
  constexpr uint32_t TMEM_COLS = 512;  // buffer b: S [128 b, +64) dP [128 b + 64, +64); dQ [256, 256+D)

  if (threadIdx.x == 0) {
    attn_init_bars(bars);
    tma_prefetch_desc(&tm_qkv);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, bars->tmem_slot, 0);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t jt = 0, it = 0;  // key tiles / items so far
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
        const int qt = n_qt - 1 - item / HB;
        const int hb = item % HB;
        const int h = hb % p.H, b = hb / p.H;
        const int n_kv = qt + 1;
        const int row0 = b * p.S + qt * ATT_BM;
        if (!mbar_wait(&bars->stat_empty, (it & 1u) ^ 1u, abort_flag, 33)) { ok = false; break; }
        mbar_expect_tx(&bars->stat_full, 2 * L::TILE);
#pragma unroll
        for (int c = 0; c < SLABS; ++c) {
          tma_load_2d(smem + L::Q_OFF + c * SLAB, &tm_qkv, &bars->stat_full, h * D + c * 64, row0);
          tma_load_2d(smem + L::DO_OFF + c * SLAB, &tm_do, &bars->stat_full, h * D + c * 64, row0);
        }
        for (int j = 0; j < n_kv; ++j, ++jt) {
          const int st = jt & 1;
          if (!mbar_wait(&bars->str_empty[st], ((jt >> 1) & 1u) ^ 1u, abort_flag, 34)) { ok = false; break; }
          const int krow = b * p.S + j * ATT_BM;
          mbar_expect_tx(&bars->str_full[st], 2 * L::TILE);
#pragma unroll
          for (int c = 0; c < SLABS; ++c) {
            tma_load_2d(smem + L::K_OFF + st * L::TILE + c * SLAB, &tm_qkv, &bars->str_full[st], HD + h * D + c * 64, krow);
            tma_load_2d(smem + L::V_OFF + st * L::TILE + c * SLAB, &tm_qkv, &bars->str_full[st], 2 * HD + h * D + c * 64, krow);
          }
        }
      }
    }
  } else if (warp == 1) {
    // MMA issuer: all lanes run the loop, one elected lane issues each group
    const uint32_t idesc_s = make_idesc_f16(ATT_BM, 64, true, false, false);
    const uint32_t idesc_q = make_idesc_f16(ATT_BM, D, true, false, true);  // dS K : K tile read MN-major
    const uint32_t sq = smem_u32(smem + L::Q_OFF), sdo = smem_u32(smem + L::DO_OFF), sds = smem_u32(smem + L::DS_OFF);
    uint32_t jt0 = 0, ut0 = 0, it = 0;  // key tiles / steps of earlier items, items so far
    bool ok = true;
    // step u = key tile u / 2, keys [64 (u & 1), +64) of it; S and dP of step u go to accumulator buffer u & 1
    auto issue_sp = [&](int u, int n_steps) -> bool {
      const uint32_t jt = jt0 + (u >> 1), ut = ut0 + u;
      const int hh = u & 1, st = jt & 1, buf = u & 1;
      if (hh == 0 && !mbar_wait_warp(&bars->str_full[st], (jt >> 1) & 1u, abort_flag, 35)) return false;
      if (!mbar_wait_warp(&bars->s_empty[buf], ((ut >> 1) & 1u) ^ 1u, abort_flag, 36)) return false;
      tc_fence_after_sync();
      const uint32_t sk = smem_u32(smem + L::K_OFF + st * L::TILE) + hh * 8192u;  // rows 64 hh .. of every slab
      const uint32_t sv = smem_u32(smem + L::V_OFF + st * L::TILE) + hh * 8192u;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16_ss(tmem_base + buf * 128, desc_kmajor(sq, ks, SLAB), desc_kmajor(sk, ks, SLAB), idesc_s, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16_ss(tmem_base + buf * 128 + 64, desc_kmajor(sdo, ks, SLAB), desc_kmajor(sv, ks, SLAB), idesc_s, ks != 0);
        umma_commit(&bars->s_full[buf]);
        if (u == n_steps - 1) umma_commit(&bars->stat_empty);  // the item's last use of Q and dO
      }
      __syncwarp();
      return true;
    };
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      const int qt = n_qt - 1 - item / HB;
      const int n_steps = 2 * (qt + 1);
      if (!mbar_wait_warp(&bars->stat_full, it & 1u, abort_flag, 37)) { ok = false; break; }
      ok = issue_sp(0, n_steps);
      for (int u = 0; u < n_steps && ok; ++u) {
        if (u + 1 < n_steps) { if (!issue_sp(u + 1, n_steps)) { ok = false; break; } }
        const uint32_t jt = jt0 + (u >> 1), ut = ut0 + u;
        const int hh = u & 1, st = jt & 1, buf = u & 1;
        // the dQ accumulator still belongs to the previous item until its threads have read it
        if (u == 0 && !mbar_wait_warp(&bars->acc_free, (it & 1u) ^ 1u, abort_flag, 38)) { ok = false; break; }
        if (!mbar_wait_warp(&bars->p_full2[buf], (ut >> 1) & 1u, abort_flag, 39)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t sk = smem_u32(smem + L::K_OFF + st * L::TILE);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 64 / 16; ++ks)
            umma_f16_ss(tmem_base + 256, desc_kmajor(sds + buf * 16384u, ks, SLAB), desc_mnmajor(sk, hh * 4 + ks, SLAB), idesc_q, (u | ks) != 0);
          if (hh == 1) umma_commit(&bars->str_empty[st]);
          umma_commit(&bars->acc_done2[buf]);
        }
        __syncwarp();
      }
      jt0 += static_cast<uint32_t>(n_steps >> 1);
      ut0 += static_cast<uint32_t>(n_steps);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // which 64 score columns / which D/2 output columns
    const int row = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    uint8_t* sds = smem + L::DS_OFF;
    uint32_t ut0 = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int qt = n_qt - 1 - item / HB;
      const int hb = item % HB;
      const int h = hb % p.H, b = hb / p.H;
      const int n_steps = 2 * (qt + 1);
      const int row0 = b * p.S + qt * ATT_BM;
      const size_t stat_idx = (static_cast<size_t>(b) * p.H + h) * p.S + qt * ATT_BM + row;
      const float lse2 = p.delta[static_cast<size_t>(p.B) * p.H * p.S + stat_idx];  // base-2 lse, written by the delta kernel
      const float delta_s = p.delta[stat_idx];                                       // scale * rowsum(dO * O)
      for (int u = 0; u < n_steps && ok; ++u) {
        const uint32_t ut = ut0 + u;
        const int j = u >> 1, hh = u & 1, buf = u & 1;
        if (!mbar_wait(&bars->s_full[buf], (ut >> 1) & 1u, abort_flag, 40)) { ok = false; break; }
        tc_fence_after_sync();
        const bool diag = (j == qt);
        uint32_t pk[16];
        {
          uint32_t rs[32], rp[32];
          tmem_ld_32x32(tmem_base + buf * 128 + lane_off + half * 32, rs);
          tmem_ld_32x32(tmem_base + buf * 128 + 64 + lane_off + half * 32, rp);
          tmem_ld_wait();
          if (!diag) dq_cols32<false>(rs, rp, hh * 64 + half * 32, row, sl2, lse2, p.scale, delta_s, pk);
          else       dq_cols32<true>(rs, rp, hh * 64 + half * 32, row, sl2, lse2, p.scale, delta_s, pk);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_empty[buf]);
        if (ut >= 2) {  // the dQ product that read this dS buffer two steps ago
          if (!mbar_wait(&bars->acc_done2[buf], ((ut >> 1) - 1u) & 1u, abort_flag, 41)) { ok = false; break; }
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(sds + buf * 16384 + swz(row, half * 4 + ch)) = v;
        }
        fence_proxy_async();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full2[buf]);
      }
      if (!ok) break;
      const uint32_t ul = ut0 + static_cast<uint32_t>(n_steps) - 1u;  // the item's last step
      if (!mbar_wait(&bars->acc_done2[ul & 1u], (ul >> 1) & 1u, abort_flag, 42)) { ok = false; break; }
      tc_fence_after_sync();
      __nv_bfloat16* drow = p.dqkv + static_cast<size_t>(row0 + row) * (3 * HD) + h * D + half * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + 256 + lane_off + half * (D / 2) + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
          v.y = pack_bf16(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
          v.z = pack_bf16(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
          v.w = pack_bf16(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
          *reinterpret_cast<uint4*>(drow + c * 32 + q * 8) = v;
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_free);
      ut0 += static_cast<uint32_t>(n_steps);
    }
  }
  attn_teardown(bars, warp, tmem_base, TMEM_COLS, p.status);
}

// P^T and dS^T for one key row against 32 queries (`qa0` = sequence index of the first); the per-query statistics come
// in 16-byte broadcast loads.
template <bool DIAG>
__device__ __forceinline__ void dkv_row(const uint32_t (&rs)[32], const uint32_t (&rp)[32], const float* __restrict__ lse2,
                                        const float* __restrict__ delta_s, int qa0, int key, float sl2, float scale,
                                        uint32_t (&pp)[16], uint32_t (&pd)[16]) {
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 l = __ldg(reinterpret_cast<const float4*>(lse2 + i));
    const float4 e = __ldg(reinterpret_cast<const float4*>(delta_s + i));
    const float lv[4] = {l.x, l.y, l.z, l.w}, ev[4] = {e.x, e.y, e.z, e.w};
    float pr[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      pr[k] = ex2_approx(fmaf(__uint_as_float(rs[i + k]), sl2, -lv[k]));
      if (DIAG && key > qa0 + i + k) pr[k] = 0.f;
    }
    pp[i >> 1] = pack_bf16(pr[0], pr[1]);
    pp[(i >> 1) + 1] = pack_bf16(pr[2], pr[3]);
    pd[i >> 1] = pack_bf16(pr[0] * fmaf(__uint_as_float(rp[i]), scale, -ev[0]), pr[1] * fmaf(__uint_as_float(rp[i + 1]), scale, -ev[1]));
    pd[(i >> 1) + 1] = pack_bf16(pr[2] * fmaf(__uint_as_float(rp[i + 2]), scale, -ev[2]), pr[3] * fmaf(__uint_as_float(rp[i + 3]), scale, -ev[3]));
  }
}

// =================================================================================================
// Backward, dK / dV: one CTA per 128 key rows; streams 64-row Q / dO sub-tiles.
// =================================================================================================
constexpr int KV_QSUB = 64;

template <int D>
struct DkvSmem {
  static constexpr int TILE = ATT_BM * D * 2;     // K or V tile
  static constexpr int QTILE = KV_QSUB * D * 2;   // Q or dO sub-tile
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE;
  static constexpr int STAGES = 3;                             // Q / dO sub-tiles in flight
  static constexpr int Q_OFF = 2 * TILE;
  static constexpr int DO_OFF = 2 * TILE + STAGES * QTILE;
  static constexpr int PT_BYTES = ATT_BM * KV_QSUB * 2;          // [128 keys x 64 q] bf16
  static constexpr int PT_OFF = 2 * TILE + 2 * STAGES * QTILE;  // P^T, two buffers: the threads fill one while the
  static constexpr int DST_OFF = PT_OFF + 2 * PT_BYTES;         // tensor cores still read the other; dS^T likewise
  static constexpr int BAR_OFF = DST_OFF + 2 * PT_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_do, AttnParams p) {
  using L = DkvSmem<D>;
  constexpr int SLABS = D / 64;
  constexpr uint32_t SLAB = ATT_BM * 128;    // [128 x 64] slab of K / V / P^T / dS^T
  constexpr uint32_t QSLAB = KV_QSUB * 128;  // [64 x 64] slab of Q / dO
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  AttnBars* bars = reinterpret_cast<AttnBars*>(smem + L::BAR_OFF);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // warp-uniform
  // Persistent: one CTA per SM walks the work items (one 128-row key tile of one head); small key tiles see the most
  // query sub-tiles and come first.  Every item has an even number of sub-tiles, so the accumulator buffer of a
  // sub-tile is its running index & 1 as well.
  const int n_kt = p.S / ATT_BM;
  const int HB = p.H * p.B;
  const int n_items = n_kt * HB;
  const int HD = p.H * D;
  // S^T / dP^T are double-buffered so the products of sub-tile t+1 run while the threads work on sub-tile t:
  // buffer 0: S^T [0,64) dP^T [64,128); buffer 1: S^T [384,448) dP^T [448,512); dV [128,128+D); dK [256,256+D)
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    attn_init_bars(bars);
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, bars->tmem_slot, 0);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t tt = 0, it = 0;  // sub-tiles / items so far
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
        const int kt = item / HB;
        const int hb = item % HB;
        const int h = hb % p.H, b = hb / p.H;
        const int krow0 = b * p.S + kt * ATT_BM;
        const int first_sub = kt * (ATT_BM / KV_QSUB);
        const int n_sub = p.S / KV_QSUB - first_sub;
        if (!mbar_wait(&bars->stat_empty, (it & 1u) ^ 1u, abort_flag, 65)) { ok = false; break; }
        mbar_expect_tx(&bars->stat_full, 2 * L::TILE);
#pragma unroll
        for (int c = 0; c < SLABS; ++c) {
          tma_load_2d(smem + L::K_OFF + c * SLAB, &tm_kv, &bars->stat_full, HD + h * D + c * 64, krow0);
          tma_load_2d(smem + L::V_OFF + c * SLAB, &tm_kv, &bars->stat_full, 2 * HD + h * D + c * 64, krow0);
        }
        for (int t = 0; t < n_sub; ++t, ++tt) {
          const int st = tt % L::STAGES;
          if (!mbar_wait(&bars->str_empty[st], ((tt / L::STAGES) & 1u) ^ 1u, abort_flag, 66)) { ok = false; break; }
          const int qrow = b * p.S + (first_sub + t) * KV_QSUB;
          mbar_expect_tx(&bars->str_full[st], 2 * L::QTILE);
#pragma unroll
          for (int c = 0; c < SLABS; ++c) {
            tma_load_2d(smem + L::Q_OFF + st * L::QTILE + c * QSLAB, &tm_q, &bars->str_full[st], h * D + c * 64, qrow);
            tma_load_2d(smem + L::DO_OFF + st * L::QTILE + c * QSLAB, &tm_do, &bars->str_full[st], h * D + c * 64, qrow);
          }
        }
      }
    }
  } else if (warp == 1) {
    // MMA issuer: all lanes run the loop, one elected lane issues each group
    const uint32_t idesc_s = make_idesc_f16(ATT_BM, KV_QSUB, true, false, false);  // K Q^T, V dO^T
    const uint32_t idesc_a = make_idesc_f16(ATT_BM, D, true, false, true);         // P^T dO, dS^T Q (B MN-major)
    const uint32_t sk = smem_u32(smem + L::K_OFF), sv = smem_u32(smem + L::V_OFF);
    const uint32_t spt = smem_u32(smem + L::PT_OFF), sdst = smem_u32(smem + L::DST_OFF);
    uint32_t tt0 = 0, it = 0;
    bool ok = true;
    // S^T(t) = K Q_t^T and dP^T(t) = V dO_t^T into accumulator buffer t & 1
    auto issue_sp = [&](int t, int n_sub) -> bool {
      const uint32_t tt = tt0 + t;
      const int st = tt % L::STAGES, buf = t & 1;
      if (!mbar_wait_warp(&bars->str_full[st], (tt / L::STAGES) & 1u, abort_flag, 67)) return false;
      if (!mbar_wait_warp(&bars->s_empty[buf], ((tt >> 1) & 1u) ^ 1u, abort_flag, 68)) return false;
      tc_fence_after_sync();
      const uint32_t sq = smem_u32(smem + L::Q_OFF + st * L::QTILE);
      const uint32_t sdo = smem_u32(smem + L::DO_OFF + st * L::QTILE);
      const uint32_t t_s = tmem_base + (buf ? 384u : 0u), t_p = tmem_base + (buf ? 448u : 64u);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16_ss(t_s, desc_kmajor(sk, ks, SLAB), desc_kmajor(sq, ks, QSLAB), idesc_s, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16_ss(t_p, desc_kmajor(sv, ks, SLAB), desc_kmajor(sdo, ks, QSLAB), idesc_s, ks != 0);
        umma_commit(&bars->s_full[buf]);
        if (t == n_sub - 1) umma_commit(&bars->stat_empty);  // the item's last use of the K and V tiles
      }
      __syncwarp();
      return true;
    };
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      const int kt = item / HB;
      const int n_sub = p.S / KV_QSUB - kt * (ATT_BM / KV_QSUB);
      if (!mbar_wait_warp(&bars->stat_full, it & 1u, abort_flag, 69)) { ok = false; break; }
      ok = issue_sp(0, n_sub);
      for (int t = 0; t < n_sub && ok; ++t) {
        if (t + 1 < n_sub) { if (!issue_sp(t + 1, n_sub)) { ok = false; break; } }
        const uint32_t tt = tt0 + t;
        const int st = tt % L::STAGES;
        const uint32_t sq = smem_u32(smem + L::Q_OFF + st * L::QTILE);
        const uint32_t sdo = smem_u32(smem + L::DO_OFF + st * L::QTILE);
        // dK / dV still belong to the previous item until its threads have read them
        if (t == 0 && !mbar_wait_warp(&bars->acc_free, (it & 1u) ^ 1u, abort_flag, 70)) { ok = false; break; }
        const int buf = t & 1;
        if (!mbar_wait_warp(&bars->p_full2[buf], (tt >> 1) & 1u, abort_flag, 71)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t pbuf = static_cast<uint32_t>(buf) * L::PT_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < KV_QSUB / 16; ++ks)
            umma_f16_ss(tmem_base + 128, desc_kmajor(spt + pbuf, ks, SLAB), desc_mnmajor(sdo, ks, QSLAB), idesc_a, (t | ks) != 0);
#pragma unroll
          for (int ks = 0; ks < KV_QSUB / 16; ++ks)
            umma_f16_ss(tmem_base + 256, desc_kmajor(sdst + pbuf, ks, SLAB), desc_mnmajor(sq, ks, QSLAB), idesc_a, (t | ks) != 0);
          umma_commit(&bars->str_empty[st]);
          umma_commit(&bars->acc_done2[buf]);
        }
        __syncwarp();
      }
      tt0 += static_cast<uint32_t>(n_sub);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // which 32 of the 64 queries of a sub-tile / which D/2 output columns
    const int row = quad * 32 + lane;  // key row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    uint8_t* spt = smem + L::PT_OFF;
    uint8_t* sdst = smem + L::DST_OFF;
    uint32_t tt0 = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int kt = item / HB;
      const int hb = item % HB;
      const int h = hb % p.H, b = hb / p.H;
      const int krow0 = b * p.S + kt * ATT_BM;
      const int first_sub = kt * (ATT_BM / KV_QSUB);
      const int n_sub = p.S / KV_QSUB - first_sub;
      const float* delta_bh = p.delta + (static_cast<size_t>(b) * p.H + h) * p.S;   // scale * rowsum(dO * O)
      const float* lse2_bh = delta_bh + static_cast<size_t>(p.B) * p.H * p.S;        // base-2 lse
      for (int t = 0; t < n_sub && ok; ++t) {
        const uint32_t tt = tt0 + t;
        const int buf = t & 1;
        if (!mbar_wait(&bars->s_full[buf], (tt >> 1) & 1u, abort_flag, 72)) { ok = false; break; }
        tc_fence_after_sync();
        const int qa0 = (first_sub + t) * KV_QSUB + half * 32;  // first query (sequence index) this thread handles
        const int key = kt * ATT_BM + row;                      // this thread's key (sequence index)
        const bool diag = qa0 < (kt + 1) * ATT_BM;              // may overlap the diagonal block
        uint32_t pp[16], pd[16];
        {
          uint32_t rs[32], rp[32];
          tmem_ld_32x32(tmem_base + (buf ? 384u : 0u) + lane_off + half * 32, rs);
          tmem_ld_32x32(tmem_base + (buf ? 448u : 64u) + lane_off + half * 32, rp);
          tmem_ld_wait();
          if (!diag) dkv_row<false>(rs, rp, lse2_bh + qa0, delta_bh + qa0, qa0, key, sl2, p.scale, pp, pd);
          else       dkv_row<true>(rs, rp, lse2_bh + qa0, delta_bh + qa0, qa0, key, sl2, p.scale, pp, pd);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_empty[buf]);
        if (tt >= 2) {  // the accumulate products that read this P^T / dS^T buffer two sub-tiles ago
          if (!mbar_wait(&bars->acc_done2[buf], ((tt >> 1) - 1u) & 1u, abort_flag, 73)) { ok = false; break; }
        }
        uint8_t* pt = spt + buf * L::PT_BYTES;
        uint8_t* dst = sdst + buf * L::PT_BYTES;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {  // 32 query columns = 4 chunks of 8 bf16
          *reinterpret_cast<uint4*>(pt + swz(row, half * 4 + ch)) = make_uint4(pp[ch * 4], pp[ch * 4 + 1], pp[ch * 4 + 2], pp[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(dst + swz(row, half * 4 + ch)) = make_uint4(pd[ch * 4], pd[ch * 4 + 1], pd[ch * 4 + 2], pd[ch * 4 + 3]);
        }
        fence_proxy_async();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full2[buf]);
      }
      if (!ok) break;
      const uint32_t tl = tt0 + static_cast<uint32_t>(n_sub) - 1u;  // the item's last sub-tile
      if (!mbar_wait(&bars->acc_done2[tl & 1u], (tl >> 1) & 1u, abort_flag, 74)) { ok = false; break; }
      tc_fence_after_sync();
      __nv_bfloat16* base = p.dqkv + static_cast<size_t>(krow0 + row) * (3 * HD) + h * D + half * (D / 2);
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {  // 0: dK (TMEM cols 256..), 1: dV (cols 128..)
        const uint32_t tcol = (which == 0 ? 256u : 128u) + static_cast<uint32_t>(half * (D / 2));
        __nv_bfloat16* drow = base + (which == 0 ? HD : 2 * HD);
#pragma unroll 1
        for (int c = 0; c < D / 64; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + tcol + lane_off + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            v.y = pack_bf16(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            v.z = pack_bf16(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            v.w = pack_bf16(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            *reinterpret_cast<uint4*>(drow + c * 32 + q * 8) = v;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_free);
      tt0 += static_cast<uint32_t>(n_sub);
    }
  }
  attn_teardown(bars, warp, tmem_base, TMEM_COLS, p.status);
}

// delta[b, h, s] = scale * sum_d dO[b, s, h, d] * O[b, s, h, d].  D / 8 lanes share one (token, head) pair (16 bytes per
// lane and tensor), so a warp covers 256 / D pairs per step and keeps several independent loads in flight.
// Also writes the base-2 log-sum-exp right behind it: delta[B*H*S + i] = lse[i] * log2(e).
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                         const float* __restrict__ lse, float* __restrict__ delta, float scale, int B,
                                                         int S, int H, int D) {
  const int lanes_per = D >> 3;             // 8 or 16
  const int lane = threadIdx.x & 31;
  const int sub = lane / lanes_per, sl = lane - sub * lanes_per;
  const int pairs_per_warp = 32 / lanes_per;
  const long long total = static_cast<long long>(B) * S * H;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long base = warp * pairs_per_warp; base < total; base += n_warps * pairs_per_warp) {
    const long long pair = base + sub;  // (token, head) index in [B*S, H] order == element offset / D
    float acc = 0.f;
    if (pair < total) {
      const Vec16<__nv_bfloat16> a = ld16(o + pair * D + sl * 8), c = ld16(d_o + pair * D + sl * 8);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += __bfloat162float(a.v[k]) * __bfloat162float(c.v[k]);
    }
    for (int off = lanes_per >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sl == 0 && pair < total) {
      const long long tok = pair / H;
      const int h = static_cast<int>(pair - tok * H);
      const long long bb = tok / S, ss = tok - bb * S;
      const long long idx = (bb * H + h) * S + ss;
      delta[idx] = acc * scale;
      delta[total + idx] = lse[idx] * LOG2E;
    }
  }
}

}  // namespace fsb

// ------------------------------------------------------------------------------------------------
// C ABI.  S must be a multiple of 128, D in {64, 128}; all tensors contiguous, 16-byte aligned.
// ------------------------------------------------------------------------------------------------
template <typename K>
static int set_smem(K kernel, int bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}
// Each CTA allocates all 512 TMEM columns, so two CTAs must never share an SM: ask for more than half of the
// SM's shared memory even when the tiles need less (D = 64).
static constexpr int kMinSmem = 120 * 1024;
static inline int one_cta_smem(int bytes) { return bytes < kMinSmem ? kMinSmem : bytes; }

FSB_API int fsb_attn_fwd_pingpong(const void* qkv, void* o, float* lse, int B, int S, int H, int D, float scale, int* status,
                                  cudaStream_t stream);

// Debug aid: copies (and clears) the bit set of wait sites that were blocked when an attention kernel aborted.
FSB_API int fsb_attn_wait_sites(unsigned int* out8) {
  unsigned int zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbol(out8, fsb::g_blocked_wait_sites, sizeof(zero));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(fsb::g_blocked_wait_sites, zero, sizeof(zero));
  return static_cast<int>(e);
}

FSB_API int fsb_last_tensor_map_result() { return fsb_host::last_encode_result(); }

// Debug aid: when set to a device buffer of 4 * 64 * 4 uint64, the forward kernel's CTA (0,0,0) records nanosecond
// time stamps of its producer / MMA / softmax roles per key tile.  Pass nullptr to switch it off again.
static unsigned long long* g_attn_trace = nullptr;
FSB_API int fsb_attn_set_trace(void* buf) {
  g_attn_trace = static_cast<unsigned long long*>(buf);
  return 0;
}

FSB_API int fsb_attn_fwd(const void* qkv, void* o, float* lse, int B, int S, int H, int D, float scale, int* status,
                         cudaStream_t stream) {
  using namespace fsb;
  if (S % ATT_BM != 0 || (D != 64 && D != 128)) return -1;
  // Two query tiles per CTA in ping-pong, persistent (attention_fwd_pingpong.cu), when the sequence is a multiple of
  // 256; FSB_ATTN_FWD=classic keeps the one-tile kernel below (also used while a timeline trace is being recorded).
  static int pingpong = -1;
  if (pingpong < 0) {
    const char* e = getenv("FSB_ATTN_FWD");
    pingpong = (e != nullptr && e[0] == 'c') ? 0 : 1;
  }
  if (pingpong == 1 && S % (2 * ATT_BM) == 0 && g_attn_trace == nullptr) return fsb_attn_fwd_pingpong(qkv, o, lse, B, S, H, D, scale, status, stream);
  CUtensorMap tm;
  if (!fsb_host::encode_2d_16bit(&tm, qkv, (uint64_t)3 * H * D, (uint64_t)B * S, (uint64_t)3 * H * D, 64, ATT_BM)) return -1;
  AttnParams p{};
  p.B = B; p.S = S; p.H = H; p.D = D; p.scale = scale;
  p.o = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = status; p.trace = g_attn_trace;
  dim3 grid(S / ATT_BM, H, B);
  if (D == 128) {
    set_smem(attn_fwd_kernel<128>, FwdSmem<128>::TOTAL);
    attn_fwd_kernel<128><<<grid, ATT_THREADS, FwdSmem<128>::TOTAL, stream>>>(tm, p);
  } else {
    set_smem(attn_fwd_kernel<64>, one_cta_smem(FwdSmem<64>::TOTAL));
    attn_fwd_kernel<64><<<grid, ATT_THREADS, one_cta_smem(FwdSmem<64>::TOTAL), stream>>>(tm, p);
  }
  return static_cast<int>(cudaGetLastError());
}

// dqkv receives dQ, dK and dV in the packed layout of qkv.  delta: fp32 workspace [B, H, S].
FSB_API int fsb_attn_bwd(const void* qkv, const void* o, const void* d_o, const float* lse, float* delta, void* dqkv, int B, int S,
                         int H, int D, float scale, int* status, cudaStream_t stream) {
  using namespace fsb;
  if (S % ATT_BM != 0 || (D != 64 && D != 128)) return -1;
  CUtensorMap tm_qkv128, tm_do128, tm_qkv64, tm_do64;
  if (!fsb_host::encode_2d_16bit(&tm_qkv128, qkv, (uint64_t)3 * H * D, (uint64_t)B * S, (uint64_t)3 * H * D, 64, ATT_BM)) return -2;
  if (!fsb_host::encode_2d_16bit(&tm_do128, d_o, (uint64_t)H * D, (uint64_t)B * S, (uint64_t)H * D, 64, ATT_BM)) return -3;
  if (!fsb_host::encode_2d_16bit(&tm_qkv64, qkv, (uint64_t)3 * H * D, (uint64_t)B * S, (uint64_t)3 * H * D, 64, KV_QSUB)) return -4;
  if (!fsb_host::encode_2d_16bit(&tm_do64, d_o, (uint64_t)H * D, (uint64_t)B * S, (uint64_t)H * D, 64, KV_QSUB)) return -5;
  AttnParams p{};
  p.B = B; p.S = S; p.H = H; p.D = D; p.scale = scale;
  p.o = const_cast<__nv_bfloat16*>(static_cast<const __nv_bfloat16*>(o));
  p.lse = const_cast<float*>(lse); p.delta = delta; p.dqkv = static_cast<__nv_bfloat16*>(dqkv); p.status = status;
  p.trace = g_attn_trace;
  {
    const long long pairs = static_cast<long long>(B) * S * H;
    const int threads = 256;
    long long blocks = (pairs * (D / 8) + threads - 1) / threads;  // one step per warp at most ...
    if (blocks > 148 * 16) blocks = 148 * 16;                       // ... but no more CTAs than keep every SM busy
    attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(o),
                                                                             static_cast<const __nv_bfloat16*>(d_o), lse, delta, scale, B, S, H, D);
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_items = (S / ATT_BM) * H * B;
  const dim3 grid(n_items < sms ? n_items : sms);  // persistent: one CTA per SM walks the work items
  if (D == 128) {
    set_smem(attn_bwd_dq_kernel<128>, DqSmem<128>::TOTAL);
    set_smem(attn_bwd_dkv_kernel<128>, DkvSmem<128>::TOTAL);
    attn_bwd_dkv_kernel<128><<<grid, ATT_THREADS, DkvSmem<128>::TOTAL, stream>>>(tm_qkv128, tm_qkv64, tm_do64, p);
    attn_bwd_dq_kernel<128><<<grid, ATT_THREADS, DqSmem<128>::TOTAL, stream>>>(tm_qkv128, tm_do128, p);
  } else {
    set_smem(attn_bwd_dq_kernel<64>, one_cta_smem(DqSmem<64>::TOTAL));
    set_smem(attn_bwd_dkv_kernel<64>, one_cta_smem(DkvSmem<64>::TOTAL));
    attn_bwd_dkv_kernel<64><<<grid, ATT_THREADS, one_cta_smem(DkvSmem<64>::TOTAL), stream>>>(tm_qkv128, tm_qkv64, tm_do64, p);
    attn_bwd_dq_kernel<64><<<grid, ATT_THREADS, one_cta_smem(DqSmem<64>::TOTAL), stream>>>(tm_qkv128, tm_do128, p);
  }
  return static_cast<int>(cudaGetLastError());
}
