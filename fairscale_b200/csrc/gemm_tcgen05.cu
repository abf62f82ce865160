// bf16 GEMM on the 5th-generation tensor cores (tcgen05) with fused epilogues.
//
//   C[M,N] = epilogue( sum_k A(m,k) * B(n,k) )        fp32 accumulation in TMEM
//
// A and B are bf16 and can each be stored K-major ([rows, K], K contiguous) or MN-major
// ([K, rows], rows contiguous); this covers the three products of a linear layer without any
// transposed copy:
//   forward  Y  = X  W^T : A = X  (K-major),  B = W  (K-major)
//   dgrad    dX = dY W   : A = dY (K-major),  B = W  (MN-major, stored [N_out... see gemm.py)
//   wgrad    dW = dY^T X : A = dY (MN-major), B = X  (MN-major)
//
// Structure: persistent kernel, one CTA per SM, 192 threads.
//   warp 0      TMA producer: 128-byte-swizzled 64-wide K slabs of A and B into a 4-stage smem ring
//   warp 1      allocates TMEM (2 x BLOCK_N fp32 columns) and issues tcgen05.mma (one elected lane)
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (each warp its 32-lane quadrant),
//               apply bias / GELU / GELU' / residual, convert and store; overlaps the next tile's
//               main loop because the accumulator is double-buffered in TMEM.
// All loads are per-CTA TMA loads of this GPU's own memory. Every mbarrier wait is bounded.
//
// Replaces the cuBLAS calls behind F.linear in the reference
// (fairscale/nn/model_parallel/layers.py:290,380 and every nn.Linear of its benchmark models).

#include "gemm_tile.cuh"

#include <cstdlib>
#include <mutex>

namespace fsb {

// BATCHED: the tensor maps are 3-D (K / MN, rows, problem) and a tile index also selects the problem; used for the
// local experts of an MoE layer (equal capacity per expert), where one launch replaces a Python loop of GEMMs.
template <int BLOCK_N, bool BATCHED>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
  using L = SmemLayout<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);  // warp-uniform
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per_problem = tiles_m * tiles_n;
  const int num_tiles = tiles_per_problem * (BATCHED ? p.batch : 1);
  const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
  auto load_tile = [&](void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    if (BATCHED) tma_load_3d(dst, map, bar, x, y, z);
    else         tma_load_2d(dst, map, bar, x, y);
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BLOCK_N);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int pb = BATCHED ? tile / tiles_per_problem : 0;
        int tm, tn;
        tile_coords(tile - pb * tiles_per_problem, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BLOCK_M, n0 = tn * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if (!p.a_mn_major) {
            load_tile(sa, &tmap_a, &full_bar[stage], k0, m0, pb);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / 64; ++j) load_tile(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0, pb);
          }
          if (!p.b_mn_major) {
            load_tile(sb, &tmap_b, &full_bar[stage], k0, n0, pb);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j) load_tile(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0, pb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (all lanes run the loop, one elected lane issues)
    {
      const uint32_t idesc = make_idesc_f16(BLOCK_M, BLOCK_N, true, p.a_mn_major != 0, p.b_mn_major != 0);
      // K-major: LBO unused, SBO 1024; UMMA_K advance = 32 B inside the swizzle row.
      // MN-major: LBO = 8192 (next 64 MN elements), SBO 1024; UMMA_K advance = 16 k-rows = 2048 B.
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u, b_kstep = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_warp(&tmem_empty_bar[acc], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
              const uint64_t adesc = make_smem_desc(sa + k * a_kstep, a_lbo, 1024u);
              const uint64_t bdesc = make_smem_desc(sb + k * b_kstep, b_lbo, 1024u);
              umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);  // frees the smem slot once these MMAs have read it
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (elect_one()) umma_commit(&tmem_full_bar[acc]);
        __syncwarp();
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int pb = BATCHED ? tile / tiles_per_problem : 0;
      int tm, tn;
      tile_coords(tile - pb * tiles_per_problem, tiles_m, tiles_n, tm, tn);
      const int row = tm * BLOCK_M + quad * 32 + lane;
      const int n0 = tn * BLOCK_N;
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + static_cast<uint32_t>(acc * BLOCK_N) + (static_cast<uint32_t>(quad * 32) << 16);
      const GemmParams pt = BATCHED ? gemm_params_of_batch(p, pb) : p;
      uint4 pre[8];
      if (epilogue_can_coalesce(pt) && epilogue_needs_aux(pt.epilogue)) epi_slab_prefetch(pre, pt.aux, pt.ld_aux, row - lane, n0, pt.M, pt.N, lane);
      if (epilogue_can_coalesce(pt)) epilogue_rows_coalesced(t_base, row - lane, n0, BLOCK_N, pt, smem + L::EPI_OFFSET + quad * 4096, lane, pre);
      else                           epilogue_rows<BLOCK_N>(t_base, row, n0, pt);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out: report, give in-flight TMA copies time to land, then release TMEM and leave
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, FSB_ERR_WAIT_TIMEOUT);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BLOCK_N);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (two SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2. Each CTA stages only its 128 rows of A and its 128 columns of B, so the
// shared-memory traffic per MMA drops by a third and 6 stages fit. CTA 0 (the leader) issues the MMAs;
// both CTAs load with their own per-CTA TMA (nothing is broadcast), and both drain their half of the
// accumulator. Barriers: full[] lives in the leader and counts both CTAs' bytes; empty[] and tmem_full[]
// exist in both CTAs and are signalled by two commits (local + peer); tmem_empty[] lives in the leader
// and collects the 8 epilogue warps of the pair.
// ------------------------------------------------------------------------------------------------
constexpr int PAIR_BLOCK_N = 256;
constexpr int PAIR_HALF_N = 128;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_SCHED_DEPTH = 4;                      // tile indices in flight between the scheduler and its readers
constexpr int PAIR_EPI_WARPS = 8;                        // two per TMEM lane quadrant, 128 columns each
constexpr int PAIR_THREADS = 64 + 32 * PAIR_EPI_WARPS;   // producer warp + MMA warp + epilogue warps

struct PairSmem {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;      // 16 KB: this CTA's 128 rows
  static constexpr int B_BYTES = PAIR_HALF_N * BLOCK_K * 2;  // 16 KB: this CTA's 128 columns
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = PAIR_STAGES * STAGE_BYTES;           // 4 KB of staging per epilogue warp
  static constexpr int BAR_OFFSET = EPI_OFFSET + PAIR_EPI_WARPS * 4096;
  // No slack for re-aligning the base: the kernel has no static shared memory, so its dynamic window starts 1024-byte
  // aligned (checked at run time).  With the 1 KB the hardware reserves per CTA this leaves 2816 bytes of the SM's
  // 228 KB, enough for two of the 128-thread communication CTAs (1 KB reserve + 8 bytes each) to stay resident beside
  // a GEMM CTA; a third would keep the next GEMM CTA off the SM.
  static constexpr int TOTAL = BAR_OFFSET + 256;
};

__device__ __forceinline__ void pair_tile_coords(const GemmParams& p, int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  if (p.b_ready != nullptr) {  // N-major in sending order of the pieces of B: every M tile of the rows that arrive first
    const int lin = tile / tiles_m;
    tm = tile - lin * tiles_m;
    // first tile that starts inside the first piece sent (rounded up: the tile before it needs the piece sent last)
    const long long tile_bytes = static_cast<long long>(PAIR_BLOCK_N) * p.K * 2;
    const int rot = static_cast<int>((static_cast<long long>(p.b_first_piece) * p.b_piece_bytes + tile_bytes - 1) / tile_bytes);
    tn = (lin + rot) % tiles_n;
  } else if (p.a_ready != nullptr) {  // M-major in arrival order of the row blocks of A, this rank's own block first
    const int lin = tile / tiles_n;
    tn = tile - lin * tiles_n;
    // first tile that starts inside this rank's own block (rounded up: a tile that straddles the block's start also needs
    // rows of the block that arrives last, so it is visited last)
    const int rot = static_cast<int>((static_cast<long long>(p.a_first_shard) * p.a_shard_rows + 2 * BLOCK_M - 1) / (2 * BLOCK_M));
    tm = (lin + rot) % tiles_m;
  } else {
    tile_coords(tile, tiles_m, tiles_n, tm, tn);
  }
}

// Wait until bytes [lo, hi) of the B operand have arrived (see GemmParams::b_ready).  Flags are raised in sending order by
// one stream, so a raised flag vouches for every piece sent before it: `upto` caches the highest sending index seen.
// Returns false when the wait limit ran out.
__device__ __forceinline__ bool wait_b_pieces(const GemmParams& p, long long lo, long long hi, int& upto, volatile int* abort_flag) {
  const int first = static_cast<int>(lo / p.b_piece_bytes), last = static_cast<int>((hi - 1) / p.b_piece_bytes);
  bool waited = false;
  for (int q = first; q <= last; ++q) {
    const int i = (q - p.b_first_piece + p.b_num_pieces) % p.b_num_pieces;  // sending index of piece q
    if (i <= upto) continue;
    const uint64_t t0 = globaltimer_ns();
    unsigned int v;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.b_ready + i) : "memory");
      if (static_cast<int>(v - p.b_ready_epoch) >= 0) break;
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > p.b_wait_ns) {
        if (*abort_flag == 0) *abort_flag = 10;
        return false;
      }
      __nanosleep(200);
    }
    upto = i;
    waited = true;
  }
  if (waited) asm volatile("fence.proxy.async;" ::: "memory");  // the arrived bytes before this thread's TMA reads of them
  return true;
}

// Wait until rows [r0, r1) of the A operand have arrived (see GemmParams::a_ready).  Flags are raised in index order by
// one stream, so a raised flag vouches for every lower index: `upto` caches the highest index seen.
__device__ __forceinline__ bool wait_a_rows(const GemmParams& p, int r0, int r1, int& upto, volatile int* abort_flag) {
  const int pps = (p.a_shard_rows + p.a_piece_rows - 1) / p.a_piece_rows;
  bool waited = false;
  int r = r0;
  while (r < r1) {
    const int shard = r / p.a_shard_rows, in_shard = r - shard * p.a_shard_rows;
    const int k = (shard - p.a_first_shard + p.a_num_shards) % p.a_num_shards;
    const int j = in_shard / p.a_piece_rows;
    const int idx = k * pps + j;
    if (idx > upto) {
      const uint64_t t0 = globaltimer_ns();
      unsigned int v;
      while (true) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.a_ready + idx) : "memory");
        if (static_cast<int>(v - p.a_ready_epoch) >= 0) break;
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > p.b_wait_ns) {
          if (*abort_flag == 0) *abort_flag = 11;
          return false;
        }
        __nanosleep(200);
      }
      upto = idx;
      waited = true;
    }
    int next = shard * p.a_shard_rows + (j + 1) * p.a_piece_rows;  // first row of the next piece
    const int shard_end = (shard + 1) * p.a_shard_rows;
    if (next > shard_end) next = shard_end;
    r = next;
  }
  if (waited) asm volatile("fence.proxy.async;" ::: "memory");  // the arrived rows before this thread's TMA reads of them
  return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_bf16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
  using L = PairSmem;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0u) {  // same for every thread of the pair: nothing has been set up yet
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, FSB_ERR_BAD_ARG);
    return;
  }

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + PAIR_STAGES;
  uint64_t* tmem_full_bar = empty_bar + PAIR_STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* sched_full = tmem_empty_bar + 2;           // [PAIR_SCHED_DEPTH] in every CTA: the slot holds a tile index
  uint64_t* sched_empty = sched_full + PAIR_SCHED_DEPTH;  // [PAIR_SCHED_DEPTH] in the leader: every reader has taken it
  volatile int* sched_tile = reinterpret_cast<volatile int*>(sched_empty + PAIR_SCHED_DEPTH);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int*>(sched_tile) + PAIR_SCHED_DEPTH);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);  // warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
  const int tiles_n = (p.N + PAIR_BLOCK_N - 1) / PAIR_BLOCK_N;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 2 * PAIR_EPI_WARPS);  // the epilogue warps of both CTAs of the pair
    }
    for (int q = 0; q < PAIR_SCHED_DEPTH; ++q) {
      mbar_init(&sched_full[q], 1);
      mbar_init(&sched_empty[q], 2 + 2 * PAIR_EPI_WARPS);  // the peer's producer, the MMA warp, all epilogue warps of the pair
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.b_ready != nullptr) {
      // The first piece of B arrives only after every peer has entered the gather, which can be long after this kernel
      // started (rank skew).  Wait for it here, under the long limit, before any of the pipeline's short waits counts.
      int upto = -1;
      const long long first_byte = static_cast<long long>(p.b_first_piece) * p.b_piece_bytes;
      wait_b_pieces(p, first_byte, first_byte + 1, upto, abort_flag);
    }
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * PAIR_BLOCK_N);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, *tmem_slot, 0);

  // Tiles are handed out at run time: the leader's producer takes the next index from a counter in global memory and
  // publishes it (or -1 at the end) to both CTAs through a small ring; every role reads the ring in order.  An SM that
  // is slowed down or taken by a kernel of another stream (a collective) then simply works off fewer tiles, instead of
  // holding back the tiles a static schedule would have given it.
  // Reader side: wait for slot q, take the index, hand the slot back to the leader.
  auto take_tile = [&](int q, uint32_t qphase, int site) -> int {
    if (!mbar_wait_cluster(&sched_full[q], qphase, abort_flag, site)) return -2;
    const int t = sched_tile[q];
    mbar_arrive_cluster(map_to_cta(smem_u32(&sched_empty[q]), 0));
    return t;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int q = 0;
      uint32_t qphase = 0;
      bool ok = true;
      // Leader: `cur` is the tile to load now (already published), `nxt` the one after it.  Indices are published one
      // tile ahead, so the other roles find theirs without waiting, and fetched one more tile ahead, so the atomic's
      // round trip hides behind a whole tile of loads.
      auto publish = [&](int t) -> bool {
        if (!mbar_wait(&sched_empty[q], qphase ^ 1u, abort_flag, 2)) return false;
        sched_tile[q] = t;
        st_shared_cluster_u32(map_to_cta(smem_u32(const_cast<int*>(&sched_tile[q])), 1), static_cast<uint32_t>(t));
        mbar_arrive_cluster(map_to_cta(smem_u32(&sched_full[q]), 0));
        mbar_arrive_cluster(map_to_cta(smem_u32(&sched_full[q]), 1));
        if (++q == PAIR_SCHED_DEPTH) { q = 0; qphase ^= 1u; }
        return true;
      };
      int cur = -1, nxt = -1;
      int b_upto = -1;  // highest B piece known to have arrived
      if (leader) {
        cur = static_cast<int>(atomicAdd(&p.sched[0], 1u));
        if (cur >= num_tiles) cur = -1;
        ok = publish(cur);
        if (cur >= 0) nxt = static_cast<int>(atomicAdd(&p.sched[0], 1u));
      }
      while (ok) {
        int tile;
        if (leader) {
          tile = cur;
          if (tile >= 0) {
            const int nt = nxt < num_tiles ? nxt : -1;
            if (!publish(nt)) break;
            cur = nt;
            if (nt >= 0) nxt = static_cast<int>(atomicAdd(&p.sched[0], 1u));  // used one tile from now
          }
        } else {
          tile = take_tile(q, qphase, 3);
          if (++q == PAIR_SCHED_DEPTH) { q = 0; qphase ^= 1u; }
        }
        if (tile < 0) break;
        int tm, tn;
        pair_tile_coords(p, tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * 2 * BLOCK_M + static_cast<int>(rank) * BLOCK_M;
        const int n0 = tn * PAIR_BLOCK_N + static_cast<int>(rank) * PAIR_HALF_N;
        if (p.b_ready != nullptr && n0 < p.N) {
          const long long row_bytes = static_cast<long long>(p.K) * 2;
          const int n1 = n0 + PAIR_HALF_N < p.N ? n0 + PAIR_HALF_N : p.N;
          if (!wait_b_pieces(p, n0 * row_bytes, n1 * row_bytes, b_upto, abort_flag)) break;
        }
        if (p.a_ready != nullptr && m0 < p.M) {
          if (!wait_a_rows(p, m0, m0 + BLOCK_M < p.M ? m0 + BLOCK_M : p.M, b_upto, abort_flag)) break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, 4)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * L::STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * BLOCK_K;
          if (!p.a_mn_major) {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_M / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmap_a, bar, m0 + j * 64, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < PAIR_HALF_N / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmap_b, bar, n0 + j * 64, k0);
          }
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (leader) {
        // the last pair to get here has seen every pair's final fetch: put the counters back for the next launch
        __threadfence();
        if (atomicAdd(&p.sched[1], 1u) == static_cast<unsigned int>(num_pairs - 1)) {
          p.sched[0] = 0u;
          p.sched[1] = 0u;
          __threadfence();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only; all lanes run the loop,
    // one elected lane issues, so that addresses and descriptors stay warp-uniform)
    if (leader) {
      const uint32_t idesc = make_idesc_f16(2 * BLOCK_M, PAIR_BLOCK_N, true, p.a_mn_major != 0, p.b_mn_major != 0);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u, b_kstep = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      int q = 0;
      uint32_t qphase = 0;
      bool ok = true;
      while (ok) {
        int tile = 0;
        if (lane == 0) tile = take_tile(q, qphase, 5);
        tile = __shfl_sync(0xffffffffu, tile, 0);
        if (++q == PAIR_SCHED_DEPTH) { q = 0; qphase ^= 1u; }
        if (tile < 0) break;
        if (!mbar_wait_warp(&tmem_empty_bar[acc], acc_phase ^ 1u, abort_flag, 6)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * PAIR_BLOCK_N);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_warp(&full_bar[stage], phase, abort_flag, 7)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
              const uint64_t adesc = make_smem_desc(sa + k * a_kstep, a_lbo, 1024u);
              const uint64_t bdesc = make_smem_desc(sb + k * b_kstep, b_lbo, 1024u);
              umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit_pair(map_to_cta(eb, 0));
            umma_commit_pair(map_to_cta(eb, 1));
          }
          __syncwarp();
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        const uint32_t fb = smem_u32(&tmem_full_bar[acc]);
        if (elect_one()) {
          umma_commit_pair(map_to_cta(fb, 0));
          umma_commit_pair(map_to_cta(fb, 1));
        }
        __syncwarp();
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const int quad = warp & 3;            // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;     // which 128 columns of the 256 this warp drains
    uint8_t* stage = smem + L::EPI_OFFSET + (warp - 2) * 4096;
    const bool coalesce = epilogue_can_coalesce(p);
    int acc = 0;
    uint32_t acc_phase = 0;
    int q = 0;
    uint32_t qphase = 0;
    bool ok = true;
    while (ok) {
      int tile = 0;
      if (lane == 0) tile = take_tile(q, qphase, 8);
      tile = __shfl_sync(0xffffffffu, tile, 0);
      if (++q == PAIR_SCHED_DEPTH) { q = 0; qphase ^= 1u; }
      if (tile < 0) break;
      int tm, tn;
      pair_tile_coords(p, tile, tiles_m, tiles_n, tm, tn);
      const int row0 = tm * 2 * BLOCK_M + static_cast<int>(rank) * BLOCK_M + quad * 32;
      const int n0 = tn * PAIR_BLOCK_N + half * (PAIR_BLOCK_N / 2);
      uint4 pre[8];
      if (coalesce && epilogue_needs_aux(p.epilogue) && n0 < p.N) epi_slab_prefetch(pre, p.aux, p.ld_aux, row0, n0, p.M, p.N, lane);
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, 9)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + static_cast<uint32_t>(acc * PAIR_BLOCK_N + half * (PAIR_BLOCK_N / 2)) +
                              (static_cast<uint32_t>(quad * 32) << 16);
      if (coalesce) epilogue_rows_coalesced(t_base, row0, n0, PAIR_BLOCK_N / 2, p, stage, lane, pre);
      else          epilogue_rows<PAIR_BLOCK_N / 2>(t_base, row0 + lane, n0, p);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, FSB_ERR_WAIT_TIMEOUT | (*abort_flag << 8));
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();  // neither CTA leaves while its partner may still signal its barriers or read its smem
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 2 * PAIR_BLOCK_N);
  }
}

}  // namespace fsb

// Counter pairs of the dynamic tile scheduler: a ring of slots per device, one slot per launch, so that GEMMs running
// at the same time on different streams never share a counter.  A slot is all zero whenever no kernel is using it (the
// kernel resets it), hence 64 launches would have to be in flight at once on one device before two could collide.
static unsigned int* next_sched_slot(int di) {
  constexpr int kSlots = 64;
  static std::mutex mu;
  static unsigned int* base[64] = {nullptr};
  static unsigned int seq[64] = {0};
  std::lock_guard<std::mutex> lock(mu);
  if (base[di] == nullptr) {
    void* ptr = nullptr;
    if (cudaMalloc(&ptr, kSlots * 2 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    if (cudaMemset(ptr, 0, kSlots * 2 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    base[di] = static_cast<unsigned int*>(ptr);
  }
  return base[di] + 2 * ((seq[di]++) % kSlots);
}

// C ABI ------------------------------------------------------------------------------------------
// lda / ldb: elements between consecutive rows of the *stored* matrix ([rows,K] when K-major,
// [K,rows] when MN-major). All leading dimensions must be multiples of 8; pointers 16-byte aligned.
// Returns 0 on success, a cudaError_t value, or -1 for an argument / tensor-map problem.
static int gemm_bf16_impl(const void* A, const void* B, void* C, const void* bias, const void* aux, void* aux_out,
                          int M, int N, int K, int lda, int ldb, int ldc, int ld_aux, int a_mn_major, int b_mn_major,
                          int epilogue, int out_f32, int accumulate_c, int max_ctas, int* status, cudaStream_t stream,
                          const unsigned int* b_ready, unsigned int b_ready_epoch, long long b_piece_bytes, unsigned long long b_wait_ns,
                          const unsigned int* a_ready = nullptr, int a_shard_rows = 0, int a_piece_rows = 0, int a_first_shard = 0,
                          int a_num_shards = 0, int b_first_piece = 0);

FSB_API int fsb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* aux, void* aux_out,
                          int M, int N, int K, int lda, int ldb, int ldc, int ld_aux, int a_mn_major, int b_mn_major,
                          int epilogue, int out_f32, int accumulate_c, int max_ctas, int* status, cudaStream_t stream) {
  return gemm_bf16_impl(A, B, C, bias, aux, aux_out, M, N, K, lda, ldb, ldc, ld_aux, a_mn_major, b_mn_major, epilogue, out_f32,
                        accumulate_c, max_ctas, status, stream, nullptr, 0u, 0, 0ull);
}

// C[M, N] = epilogue(A[M, K] * B^T + bias) with B ([N, K], rows contiguous: ldb == K) arriving while the kernel runs:
// ready[i] >= ready_epoch means bytes [i * piece_bytes, (i + 1) * piece_bytes) of B are in place (see GemmParams::b_ready).
// Pieces are sent cyclically from `first_piece` on and flags are indexed in sending order.
// Needs the CTA-pair kernel (M, N >= 256); returns -1 otherwise.  wait_ms bounds every wait for a piece.
FSB_API int fsb_gemm_bf16_streamed_b(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda, int ldc,
                                     int epilogue, const unsigned int* ready, unsigned int ready_epoch, long long piece_bytes,
                                     int first_piece, long long wait_ms, int* status, cudaStream_t stream) {
  if (M < 256 || N < 256 || ready == nullptr || piece_bytes <= 0) return -1;
  if (epilogue != fsb::EPI_NONE && epilogue != fsb::EPI_BIAS) return -1;
  if (first_piece < 0) return -1;
  return gemm_bf16_impl(A, B, C, bias, nullptr, nullptr, M, N, K, lda, K, ldc, ldc, 0, 0, epilogue, 0, 0, 0, status, stream, ready,
                        ready_epoch, piece_bytes, static_cast<unsigned long long>(wait_ms > 0 ? wait_ms : 30000) * 1000000ull, nullptr, 0, 0,
                        0, 0, first_piece);
}

// C[M, N] = epilogue(A * B^T + bias) with A ([M, K], rows contiguous) arriving while the kernel runs, row block by row block
// (see GemmParams::a_ready): the all-gather of a sequence-parallel activation consumed by the product it feeds.
// B is [N, K] (ldb) or, with b_mn_major, [K, N].  Needs the CTA-pair kernel (M, N >= 256); returns -1 otherwise.
FSB_API int fsb_gemm_bf16_streamed_a(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int ldb, int ldc,
                                     int b_mn_major, int epilogue, const unsigned int* ready, unsigned int ready_epoch, int shard_rows,
                                     int piece_rows, int first_shard, int num_shards, long long wait_ms, int* status, cudaStream_t stream) {
  if (M < 256 || N < 256 || ready == nullptr || shard_rows <= 0 || piece_rows <= 0 || num_shards <= 0 || shard_rows * num_shards != M) return -1;
  if (first_shard < 0 || first_shard >= num_shards) return -1;
  if (epilogue != fsb::EPI_NONE && epilogue != fsb::EPI_BIAS && epilogue != fsb::EPI_BIAS_GELU) return -1;
  return gemm_bf16_impl(A, B, C, bias, nullptr, nullptr, M, N, K, K, ldb, ldc, ldc, 0, b_mn_major, epilogue, 0, 0, 0, status, stream, nullptr,
                        ready_epoch, 0, static_cast<unsigned long long>(wait_ms > 0 ? wait_ms : 30000) * 1000000ull, ready, shard_rows,
                        piece_rows, first_shard, num_shards);
}

static int gemm_bf16_impl(const void* A, const void* B, void* C, const void* bias, const void* aux, void* aux_out,
                          int M, int N, int K, int lda, int ldb, int ldc, int ld_aux, int a_mn_major, int b_mn_major,
                          int epilogue, int out_f32, int accumulate_c, int max_ctas, int* status, cudaStream_t stream,
                          const unsigned int* b_ready, unsigned int b_ready_epoch, long long b_piece_bytes, unsigned long long b_wait_ns,
                          const unsigned int* a_ready, int a_shard_rows, int a_piece_rows, int a_first_shard, int a_num_shards,
                          int b_first_piece) {
  using namespace fsb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -1;
  if (accumulate_c && !out_f32) return -1;

  const int block_n = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  bool ok = true;
  if (!a_mn_major) ok &= fsb_host::encode_2d_16bit(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M);
  else             ok &= fsb_host::encode_2d_16bit(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 64, BLOCK_K);
  if (!b_mn_major) ok &= fsb_host::encode_2d_16bit(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, block_n);
  else             ok &= fsb_host::encode_2d_16bit(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K);
  if (!ok) return -1;

  GemmParams p;
  p.C = C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux = reinterpret_cast<const __nv_bfloat16*>(aux);
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ld_aux = ld_aux > 0 ? ld_aux : ldc;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.epilogue = epilogue; p.out_f32 = out_f32; p.accumulate_c = accumulate_c;
  p.status = status;
  p.batch = 1; p.stride_c = p.stride_aux = p.stride_bias = 0;
  p.sched = nullptr;
  p.b_ready = b_ready; p.b_ready_epoch = b_ready_epoch; p.b_piece_bytes = b_piece_bytes; p.b_wait_ns = b_wait_ns;
  p.b_num_pieces = b_piece_bytes > 0 ? static_cast<int>((static_cast<long long>(N) * K * 2 + b_piece_bytes - 1) / b_piece_bytes) : 1;
  p.b_first_piece = b_ready != nullptr ? b_first_piece % p.b_num_pieces : 0;
  p.a_ready = a_ready; p.a_ready_epoch = b_ready_epoch; p.a_shard_rows = a_shard_rows; p.a_piece_rows = a_piece_rows;
  p.a_first_shard = a_first_shard; p.a_num_shards = a_num_shards;

  int dev = 0;
  cudaGetDevice(&dev);
  static int num_sms_cache[64] = {0};
  static bool attr_set[64][2] = {{false}};
  const int di = dev & 63;
  if (num_sms_cache[di] == 0) cudaDeviceGetAttribute(&num_sms_cache[di], cudaDevAttrMultiProcessorCount, dev);
  const int num_sms = num_sms_cache[di];
  const int tiles = ((M + BLOCK_M - 1) / BLOCK_M) * ((N + block_n - 1) / block_n);
  int grid = tiles < num_sms ? tiles : num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;

  cudaError_t err;
  static int pair_mode = -1;  // FSB_GEMM_PAIR=0 disables the CTA-pair kernel
  if (pair_mode < 0) {
    const char* e = getenv("FSB_GEMM_PAIR");
    pair_mode = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if ((b_ready != nullptr || a_ready != nullptr) && !(pair_mode == 1 && M >= 256 && N >= 256 && max_ctas == 0)) return -1;
  if (pair_mode == 1 && M >= 256 && N >= 256 && max_ctas == 0) {
    // the B map's box is this CTA's 128 columns (K-major) / 64 (MN-major, unchanged)
    if (!b_mn_major && !fsb_host::encode_2d_16bit(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, PAIR_HALF_N)) return -1;
    static bool pair_attr_set[64] = {false};
    if (!pair_attr_set[di]) {
      cudaFuncSetAttribute(gemm_bf16_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL);
      pair_attr_set[di] = true;
    }
    const int pair_tiles = ((M + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) * ((N + PAIR_BLOCK_N - 1) / PAIR_BLOCK_N);
    const int max_pairs = num_sms / 2;
    const int pairs = pair_tiles < max_pairs ? pair_tiles : max_pairs;
    p.sched = next_sched_slot(di);
    if (p.sched == nullptr) return -1;
    gemm_bf16_tcgen05_pair_kernel<<<2 * pairs, PAIR_THREADS, PairSmem::TOTAL, stream>>>(ta, tb, p);
    return static_cast<int>(cudaGetLastError());
  }
  if (block_n == 256) {
    if (!attr_set[di][0]) {
      cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<256>::TOTAL);
      attr_set[di][0] = true;
    }
    gemm_bf16_tcgen05_kernel<256, false><<<grid, GEMM_THREADS, SmemLayout<256>::TOTAL, stream>>>(ta, tb, p);
  } else {
    if (!attr_set[di][1]) {
      cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<128>::TOTAL);
      attr_set[di][1] = true;
    }
    gemm_bf16_tcgen05_kernel<128, false><<<grid, GEMM_THREADS, SmemLayout<128>::TOTAL, stream>>>(ta, tb, p);
  }
  err = cudaGetLastError();
  return static_cast<int>(err);
}

// `batch` independent products of one shape in a single launch (the local experts of an MoE layer):
//   C[b] = epilogue( A[b] * B[b]^T ),  b = 0 .. batch-1
// stride_*: elements between consecutive problems (stride_bias may be 0 for a shared bias).  Layout flags, leading
// dimensions and epilogues as for fsb_gemm_bf16.  Rows of a problem never leak into the next one: the tensor maps are
// three-dimensional, so a tile that overhangs M or N reads zeros.
FSB_API int fsb_gemm_bf16_batched(const void* A, const void* B, void* C, const void* bias, const void* aux, void* aux_out, int batch,
                                  int M, int N, int K, int lda, int ldb, int ldc, int ld_aux, long long stride_a, long long stride_b,
                                  long long stride_c, long long stride_aux, long long stride_bias, int a_mn_major, int b_mn_major,
                                  int epilogue, int out_f32, int accumulate_c, int* status, cudaStream_t stream) {
  using namespace fsb;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (stride_a % 8) || (stride_b % 8) || (reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return -1;
  if (accumulate_c && !out_f32) return -1;
  const int block_n = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  bool ok = true;
  if (!a_mn_major) ok &= fsb_host::encode_3d_16bit(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, (uint64_t)lda, (uint64_t)stride_a, BLOCK_K, BLOCK_M, 1);
  else             ok &= fsb_host::encode_3d_16bit(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)batch, (uint64_t)lda, (uint64_t)stride_a, 64, BLOCK_K, 1);
  if (!b_mn_major) ok &= fsb_host::encode_3d_16bit(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)batch, (uint64_t)ldb, (uint64_t)stride_b, BLOCK_K, block_n, 1);
  else             ok &= fsb_host::encode_3d_16bit(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)batch, (uint64_t)ldb, (uint64_t)stride_b, 64, BLOCK_K, 1);
  if (!ok) return -1;
  GemmParams p;
  p.C = C;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.aux = reinterpret_cast<const __nv_bfloat16*>(aux);
  p.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ld_aux = ld_aux > 0 ? ld_aux : ldc;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.epilogue = epilogue; p.out_f32 = out_f32; p.accumulate_c = accumulate_c;
  p.status = status;
  p.sched = nullptr;
  p.b_ready = nullptr; p.b_ready_epoch = 0; p.b_piece_bytes = 0; p.b_wait_ns = 0; p.b_first_piece = 0; p.b_num_pieces = 1;
  p.a_ready = nullptr; p.a_ready_epoch = 0; p.a_shard_rows = p.a_piece_rows = p.a_first_shard = p.a_num_shards = 0;
  p.batch = batch; p.stride_c = stride_c; p.stride_aux = stride_aux > 0 ? stride_aux : stride_c; p.stride_bias = stride_bias;
  int dev = 0, num_sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = static_cast<long long>(batch) * ((M + BLOCK_M - 1) / BLOCK_M) * ((N + block_n - 1) / block_n);
  const int grid = tiles < num_sms ? static_cast<int>(tiles) : num_sms;
  static bool attr_set_dev[64][2] = {{false}};  // the attribute is per device
  bool* attr_set = attr_set_dev[dev & 63];
  if (block_n == 256) {
    if (!attr_set[0]) {
      cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<256>::TOTAL);
      attr_set[0] = true;
    }
    gemm_bf16_tcgen05_kernel<256, true><<<grid, GEMM_THREADS, SmemLayout<256>::TOTAL, stream>>>(ta, tb, p);
  } else {
    if (!attr_set[1]) {
      cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<128>::TOTAL);
      attr_set[1] = true;
    }
    gemm_bf16_tcgen05_kernel<128, true><<<grid, GEMM_THREADS, SmemLayout<128>::TOTAL, stream>>>(ta, tb, p);
  }
  return static_cast<int>(cudaGetLastError());
}
