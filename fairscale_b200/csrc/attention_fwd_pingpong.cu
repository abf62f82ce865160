// Causal flash-attention forward with two query tiles per CTA in ping-pong and the probabilities kept in TMEM.
//
//   qkv : bf16 [B, S, 3, H, D] (packed, read by TMA)      o : bf16 [B, S, H, D]      lse : fp32 [B, H, S]
//
// One CTA owns 256 query rows as two 128-row tiles A and B.  The tensor cores alternate between the tiles, so the
// softmax of one tile runs while the products of the other are in flight:
//
//   tensor pipe :  S_A(j)  S_B(j) | PV_A(j-1) S_A(j) ... ->  PV_A(j)  S_A(j+1)  PV_B(j)  S_B(j+1)  PV_A(j+1) ...
//   softmax A   :          [ softmax A(j) ............ ]              [ softmax A(j+1) ............ ]
//   softmax B   :                    [ softmax B(j) ............ ]              [ softmax B(j+1) ..... ]
//
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 softmax of tile A, warps 6-9
// softmax of tile B; one thread per query row (TMEM lane), so the row maximum and row sum need no exchange.
// TMEM (512 columns): S_A [0,128)  S_B [128,256)  O_A [256,256+D)  O_B [384,384+D).  The bf16 probabilities overwrite
// the first 64 columns of their own score tile (two values per 32-bit column) and feed P V as the TMEM A operand of
// tcgen05.mma, so they never pass through shared memory.  The tensor pipe executes in issue order: S_t(j+1) is issued
// after PV_t(j) and therefore cannot overwrite P_t(j) early.
// Tile A skips the last key tile of the item (it lies wholly above A's diagonal).  Every mbarrier wait is bounded.
//
// The kernel is persistent: one CTA per SM walks a list of work items (256 query rows of one head), longest rows first,
// dealt round-robin.  TMEM, barriers and the K / V ring live for the whole kernel, and the next item's query tiles are
// loaded as soon as the last Q K^T products of the current item have completed, i.e. during its final softmax and
// output write.  (With one CTA per item an SM sat idle for 7-10 us between consecutive CTAs - launch, 197 KB of shared
// memory, TMEM allocation - which was a third of the kernel's run time.)
//
// Replaces nn.MultiheadAttention / bmm+softmax in the reference's models
// (benchmarks/models/transformer_lm.py:107,150-152,169-183).

#include "sm100.cuh"

namespace fsb {
namespace pp {

constexpr int THREADS = 320;
constexpr int BM = 128;          // rows of a query tile == TMEM lanes
constexpr int BN = 128;          // keys per step
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct Params {
  int B, S, H, D;
  float scale;
  __nv_bfloat16* o;
  float* lse;
  int* status;
  unsigned long long* trace;  // optional timeline of CTA (0,0,0): [role][step][4] nanosecond stamps
};

// role 0: MMA issuer, 1: softmax of tile A (warp 2, lane 0), 2: softmax of tile B (warp 6, lane 0)
#define PP_TRACE(role, j, k)                                                                              \
  if (p.trace != nullptr && blockIdx.x == 0 && (j) < 32 && (threadIdx.x & 31) == 0)                            \
    p.trace[((role) * 32 + (j)) * 4 + (k)] = globaltimer_ns();

struct Bars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2];
  uint64_t v_full[2], v_empty[2];
  uint64_t s_full[2];   // per query tile: scores of the current step are in TMEM
  uint64_t p_full[2];   // per query tile: probabilities written (4 warp arrivals)
  uint64_t o_done[2];   // per query tile: P V of the current step has completed
  uint64_t q_empty;     // the item's last Q K^T products have completed: the query tiles may be replaced
  uint64_t o_free[2];   // per query tile: the softmax warps have read the item's output accumulator (4 warp arrivals)
  uint32_t tmem_slot;
  int abort_flag;
};

template <int D>
struct Smem {
  static constexpr int TILE = BM * D * 2;
  static constexpr int Q_OFF = 0;            // two query tiles
  static constexpr int K_OFF = 2 * TILE;     // two stages
  static constexpr int V_OFF = 4 * TILE;     // two stages
  static constexpr int BAR_OFF = 6 * TILE;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// K-major operand: [rows x 64] slabs of `slab_bytes`; k-step ks covers 16 elements (32 bytes inside the swizzle row)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int ks, uint32_t slab_bytes) {
  return make_smem_desc(base + static_cast<uint32_t>(ks >> 2) * slab_bytes + static_cast<uint32_t>(ks & 3) * 32u, 16u, 1024u);
}
// MN-major operand: the same bytes read as [k_rows x 64] slabs; k-step ks covers 16 k_rows = 2048 bytes
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int ks, uint32_t slab_bytes) {
  return make_smem_desc(base + static_cast<uint32_t>(ks) * 2048u, slab_bytes, 1024u);
}

template <bool DIAG>
__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32], int col0, int row, float m) {
  float a[4] = {m, m, m, m};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    if (!DIAG || (col0 + i) <= row) a[i & 3] = fmaxf(a[i & 3], __uint_as_float(r[i]));
  }
  return fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
}

template <bool DIAG>
__device__ __forceinline__ float chunk_exp(const uint32_t (&r)[32], int col0, int row, float sl2, float mb, uint32_t (&pk)[16]) {
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float p0 = ex2_approx(fmaf(__uint_as_float(r[i]), sl2, -mb));
    float p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), sl2, -mb));
    if (DIAG) {
      if (col0 + i > row) p0 = 0.f;
      if (col0 + i + 1 > row) p1 = 0.f;
    }
    acc[(i >> 1) & 3] += p0 + p1;
    pk[i >> 1] = pack_bf16(p0, p1);
  }
  return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_pingpong_kernel(const __grid_constant__ CUtensorMap tm_qkv, Params p) {
  using L = Smem<D>;
  constexpr int SLABS = D / 64;
  constexpr uint32_t SLAB = BM * 128;  // bytes of a [128 x 64] bf16 slab
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + L::BAR_OFF);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;  // warp-uniform
  // Work items (256 query rows of one head) ordered longest first and dealt round-robin to the persistent CTAs: every
  // role of the CTA walks the same list.  item -> (q2, h, b): all heads of the longest rows come first.
  const int n_q2 = p.S / (2 * BM);
  const int HB = p.H * p.B;
  const int n_items = n_q2 * HB;
  const int HD = p.H * D;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->p_full[i], 4);
      mbar_init(&bars->o_done[i], 1);
      mbar_init(&bars->o_free[i], 4);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_qkv);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t kt = 0;  // key tiles loaded so far (selects the K / V stage and its phase)
      uint32_t it = 0;  // items started so far
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
        const int q2 = n_q2 - 1 - item / HB;
        const int hb = item % HB;
        const int h = hb % p.H, b = hb / p.H;
        const int n_kv = 2 * q2 + 2;
        const int row0 = b * p.S + q2 * 2 * BM;
        // the query tiles of the previous item are free once its last Q K^T products have completed
        if (!mbar_wait(&bars->q_empty, (it & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        mbar_expect_tx(&bars->q_full, 2 * L::TILE);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int c = 0; c < SLABS; ++c)
            tma_load_2d(smem + L::Q_OFF + t * L::TILE + c * SLAB, &tm_qkv, &bars->q_full, h * D + c * 64, row0 + t * BM);
        for (int j = 0; j < n_kv; ++j, ++kt) {
          const int st = kt & 1;
          const uint32_t par = ((kt >> 1) & 1u) ^ 1u;
          const int krow = b * p.S + j * BN;
          if (!mbar_wait(&bars->k_empty[st], par, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&bars->k_full[st], L::TILE);
#pragma unroll
          for (int c = 0; c < SLABS; ++c)
            tma_load_2d(smem + L::K_OFF + st * L::TILE + c * SLAB, &tm_qkv, &bars->k_full[st], HD + h * D + c * 64, krow);
          if (!mbar_wait(&bars->v_empty[st], par, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&bars->v_full[st], L::TILE);
#pragma unroll
          for (int c = 0; c < SLABS; ++c)
            tma_load_2d(smem + L::V_OFF + st * L::TILE + c * SLAB, &tm_qkv, &bars->v_full[st], 2 * HD + h * D + c * 64, krow);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (all lanes run the loop, one is elected per group)
    const uint32_t idesc_s = make_idesc_f16(BM, BN, true, false, false);  // Q K^T: both K-major
    const uint32_t idesc_o = make_idesc_f16(BM, D, true, false, true);    // P V: P from TMEM, V MN-major
    const uint32_t sq = smem_u32(smem + L::Q_OFF);
    uint32_t kt0 = 0;          // key tiles consumed by earlier items
    uint32_t cs[2] = {0, 0};   // steps issued so far per query tile (phase of p_full)
    uint32_t it = 0;
    bool ok = true;
    auto issue_s = [&](int t, uint32_t kt) -> bool {
      const int st = kt & 1;
      if (!mbar_wait_warp(&bars->k_full[st], (kt >> 1) & 1u, abort_flag)) return false;
      tc_fence_after_sync();
      const uint32_t sk = smem_u32(smem + L::K_OFF + st * L::TILE);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16_ss(tmem_base + t * 128, desc_kmajor(sq + t * L::TILE, ks, SLAB), desc_kmajor(sk, ks, SLAB), idesc_s, ks != 0);
        umma_commit(&bars->s_full[t]);
      }
      __syncwarp();
      return true;
    };
    auto issue_pv = [&](int t, uint32_t kt, bool first) -> bool {
      if (!mbar_wait_warp(&bars->p_full[t], cs[t] & 1u, abort_flag)) return false;
      tc_fence_after_sync();
      const uint32_t sv = smem_u32(smem + L::V_OFF + (kt & 1) * L::TILE);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)
          umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + ks * 8, desc_mnmajor(sv, ks, SLAB), idesc_o, (!first || ks != 0) ? 1u : 0u);
        umma_commit(&bars->o_done[t]);
      }
      __syncwarp();
      ++cs[t];
      return true;
    };
    auto commit = [&](uint64_t* bar) {
      if (elect_one()) umma_commit(bar);
      __syncwarp();
    };
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      const int q2 = n_q2 - 1 - item / HB;
      const int n_kv = 2 * q2 + 2;  // key tiles seen by tile B; tile A sees one less (its last one is wholly masked)
      const int n_a = n_kv - 1;
      if (!mbar_wait_warp(&bars->q_full, it & 1u, abort_flag)) { ok = false; break; }
      ok = issue_s(0, kt0);
      if (ok) ok = issue_s(1, kt0);
      if (ok) commit(&bars->k_empty[kt0 & 1]);
      if (ok && n_kv == 1) commit(&bars->q_empty);
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t kt = kt0 + j;
        const int st = kt & 1;
        if (!mbar_wait_warp(&bars->v_full[st], (kt >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (item == static_cast<int>(blockIdx.x)) { PP_TRACE(0, j, 0); }
        if (p.trace != nullptr && item == 0 && j < 32 && lane == 0) p.trace[384 + j] = clock64();
        if (j == 0) {
          // the output accumulators still belong to the previous item until its softmax warps have read them
          if (!mbar_wait_warp(&bars->o_free[0], (it & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait_warp(&bars->o_free[1], (it & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        }
        if (j < n_a) {
          if (!issue_pv(0, kt, j == 0)) { ok = false; break; }
          if (item == static_cast<int>(blockIdx.x)) { PP_TRACE(0, j, 1); }
          if (j + 1 < n_a && !issue_s(0, kt + 1)) { ok = false; break; }
        }
        if (item == static_cast<int>(blockIdx.x)) { PP_TRACE(0, j, 2); }
        if (!issue_pv(1, kt, j == 0)) { ok = false; break; }
        if (item == static_cast<int>(blockIdx.x)) { PP_TRACE(0, j, 3); }
        commit(&bars->v_empty[st]);
        if (j + 1 < n_kv) {
          if (!issue_s(1, kt + 1)) { ok = false; break; }
          commit(&bars->k_empty[(kt + 1) & 1]);
          if (j + 2 == n_kv) commit(&bars->q_empty);  // that was the item's last use of the query tiles
        }
      }
      kt0 += n_kv;
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: one thread per query row
    const int t = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t ts = tmem_base + t * 128 + lane_off;        // scores; probabilities overwrite columns [0, 64)
    const uint32_t to = tmem_base + 256 + t * 128 + lane_off;  // output accumulator
    const float sl2 = p.scale * LOG2E;
    uint32_t cs = 0;  // steps of this tile so far, over all items (phase of s_full / o_done)
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const int q2 = n_q2 - 1 - item / HB;
      const int hb = item % HB;
      const int h = hb % p.H, b = hb / p.H;
      const int n_kv = 2 * q2 + 2;
      const int n_it = t == 0 ? n_kv - 1 : n_kv;
      const int row0 = b * p.S + q2 * 2 * BM;
      const bool traced = (item == static_cast<int>(blockIdx.x)) && quad == 2;
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n_it && ok; ++j, ++cs) {
        if (!mbar_wait(&bars->s_full[t], cs & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        if (traced) { PP_TRACE(1 + t, j, 0); }
        const bool diag = (j == n_it - 1);
        uint32_t r0[32], r1[32];
        // pass 1: row maximum
        float mx = -INFINITY;
        tmem_ld_32x32(ts, r0);
        tmem_ld_32x32(ts + 32, r1);
        tmem_ld_wait();
        if (!diag) { mx = chunk_max<false>(r0, 0, row, mx); mx = chunk_max<false>(r1, 32, row, mx); }
        else       { mx = chunk_max<true>(r0, 0, row, mx);  mx = chunk_max<true>(r1, 32, row, mx); }
        tmem_ld_32x32(ts + 64, r0);
        tmem_ld_32x32(ts + 96, r1);
        tmem_ld_wait();
        if (!diag) { mx = chunk_max<false>(r0, 64, row, mx); mx = chunk_max<false>(r1, 96, row, mx); }
        else       { mx = chunk_max<true>(r0, 64, row, mx);  mx = chunk_max<true>(r1, 96, row, mx); }
        // keep the old maximum while the new one is at most 2^8 above it: no rescaling of O, values stay in range
        float m_new = fmaxf(m_run, mx);
        if (m_run != -INFINITY && (m_new - m_run) * sl2 <= 8.f) m_new = m_run;
        const float alpha = (m_run == -INFINITY) ? 0.f : ex2_approx((m_run - m_new) * sl2);
        const float mb = m_new * sl2;
        if (traced) { PP_TRACE(1 + t, j, 1); }
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // O_t belongs to P V of step j-1 until that has completed (it has: S_t(j) was issued behind it)
          if (!mbar_wait(&bars->o_done[t], (cs - 1u) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(to + c * 32, r);
            tmem_ld_wait();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              lo[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              hi[i] = __float_as_uint(__uint_as_float(r[16 + i]) * alpha);
            }
            tmem_st_32x16(to + c * 32, lo);
            tmem_st_32x16(to + c * 32 + 16, hi);
          }
        }
        if (traced) { PP_TRACE(1 + t, j, 2); }
        // pass 2: exponentials; chunk c of 32 keys becomes 16 packed columns at [16 c, 16 c + 16), always behind the reads
        float rs = 0.f;
        uint32_t pk[16];
        tmem_ld_32x32(ts, r0);
        tmem_ld_32x32(ts + 32, r1);
        tmem_ld_wait();
        if (!diag) rs += chunk_exp<false>(r0, 0, row, sl2, mb, pk); else rs += chunk_exp<true>(r0, 0, row, sl2, mb, pk);
        tmem_ld_32x32(ts + 64, r0);  // in flight during the next exponentials
        tmem_st_32x16(ts, pk);
        if (!diag) rs += chunk_exp<false>(r1, 32, row, sl2, mb, pk); else rs += chunk_exp<true>(r1, 32, row, sl2, mb, pk);
        tmem_ld_32x32(ts + 96, r1);
        tmem_st_32x16(ts + 16, pk);
        tmem_ld_wait();
        if (!diag) rs += chunk_exp<false>(r0, 64, row, sl2, mb, pk); else rs += chunk_exp<true>(r0, 64, row, sl2, mb, pk);
        tmem_st_32x16(ts + 32, pk);
        if (!diag) rs += chunk_exp<false>(r1, 96, row, sl2, mb, pk); else rs += chunk_exp<true>(r1, 96, row, sl2, mb, pk);
        tmem_st_32x16(ts + 48, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[t]);
        if (traced) { PP_TRACE(1 + t, j, 3); }
        l_run = l_run * alpha + rs;
        m_run = m_new;
      }
      if (!ok) break;
      // epilogue of the item: normalise and store this thread's output row, then hand the accumulator back
      if (!mbar_wait(&bars->o_done[t], (cs - 1u) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const float inv = 1.f / l_run;
      __nv_bfloat16* orow = p.o + static_cast<size_t>(row0 + t * BM + row) * HD + h * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(to + c * 32, r);
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
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->o_free[t]);
      if (p.lse != nullptr)
        p.lse[(static_cast<size_t>(b) * p.H + h) * p.S + q2 * 2 * BM + t * BM + row] = (m_run * sl2 + log2f(l_run)) * LN2;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (bars->abort_flag) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, FSB_ERR_WAIT_TIMEOUT);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace pp
}  // namespace fsb

// C ABI.  S must be a multiple of 256 and D in {64, 128}; returns -1 otherwise (the caller falls back to the
// one-tile-per-CTA forward).  Tensors are contiguous and 16-byte aligned.
// Debug aid: a device buffer of 416 uint64 receives nanosecond stamps [role][step][4] of the first item of CTA 0 and, from
// entry 384, the issuer's clock64 per step; nullptr switches it off.
static unsigned long long* g_pp_trace = nullptr;
FSB_API int fsb_attn_pp_set_trace(void* buf) {
  g_pp_trace = static_cast<unsigned long long*>(buf);
  return 0;
}

FSB_API int fsb_attn_fwd_pingpong(const void* qkv, void* o, float* lse, int B, int S, int H, int D, float scale, int* status,
                                  cudaStream_t stream) {
  using namespace fsb;
  using namespace fsb::pp;
  if (S % (2 * BM) != 0 || (D != 64 && D != 128)) return -1;
  CUtensorMap tm;
  if (!fsb_host::encode_2d_16bit(&tm, qkv, (uint64_t)3 * H * D, (uint64_t)B * S, (uint64_t)3 * H * D, 64, BM)) return -1;
  Params p{};
  p.B = B; p.S = S; p.H = H; p.D = D; p.scale = scale;
  p.o = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = status; p.trace = g_pp_trace;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_items = (S / (2 * BM)) * H * B;
  const dim3 grid(n_items < sms ? n_items : sms);  // persistent: one CTA per SM walks the work items
  // each CTA allocates all 512 TMEM columns, so two CTAs must never share an SM: ask for more than half of its shared memory
  constexpr int kMinSmem = 120 * 1024;
  if (D == 128) {
    constexpr int smem = Smem<128>::TOTAL;
    cudaFuncSetAttribute(attn_fwd_pingpong_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attn_fwd_pingpong_kernel<128><<<grid, THREADS, smem, stream>>>(tm, p);
  } else {
    constexpr int smem = Smem<64>::TOTAL < kMinSmem ? kMinSmem : Smem<64>::TOTAL;
    cudaFuncSetAttribute(attn_fwd_pingpong_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attn_fwd_pingpong_kernel<64><<<grid, THREADS, smem, stream>>>(tm, p);
  }
  return static_cast<int>(cudaGetLastError());
}
