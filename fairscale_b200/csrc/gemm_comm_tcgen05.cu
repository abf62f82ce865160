// Tensor-parallel GEMMs fused with their collective, one kernel each, over NVLink peer memory.
//
//   ag_gemm :  C[M, N] = concat_r(A_r)[M, K] * B[N, K]^T           all-gather -> GEMM
//              (A is sharded by rows: rank r owns the Mc = M / world rows of chunk r)
//   gemm_rs :  Out[Mc, N] = sum_r ( A_r[M, Kr] * B_r[N, Kr]^T )[rows of my chunk]     GEMM -> reduce-scatter
//
// Both are persistent kernels whose first `n_comm` CTAs move data while the remaining CTAs run the tcgen05
// main loop of gemm_tcgen05.cu (TMA producer warp / MMA warp / 4 epilogue warps, accumulators double-buffered
// in TMEM).  Tiles are ordered chunk by chunk so that communication of one chunk overlaps the math of another:
//
//   ag_gemm  the GEMM CTAs start with the rows this rank already owns; meanwhile the copy CTAs pull the peers'
//            chunks (16-byte L1-bypassing peer loads, remote chunks in ring order) into the local gather
//            buffer and publish one counter per chunk; a producer warp waits for that counter (bounded) before
//            the first TMA load of a chunk.  Every remote byte crosses NVLink once; TMA only ever reads this
//            GPU's own memory.  The gather buffer is kept: backward needs the gathered activations.
//   gemm_rs  rank r computes the chunks in the order r+1, r+2, ..., r (its own last) and writes bf16 partial
//            tiles to its symmetric staging buffer; the epilogue warp that completes a chunk raises a flag
//            in the owner's signal pad (st.release.sys).  The owner's reduce CTAs wait for each peer's flag
//            (bounded) and bulk-copy that peer's partial rows into a local receive buffer while the tensor-core
//            CTAs are still busy.  When a CTA of either kind runs out of work it joins the final pass,
//            out = own partial + received partials (fixed order, fp32) + bias, which therefore runs on every SM.
//
// Cross-GPU ordering uses the epoch flags of comm_dev.cuh; an exit barrier keeps a rank's buffers alive until
// every peer is done reading them.  No TMA multicast, no cluster launch.  Replaces all-gather + F.linear and
// F.linear + all-reduce of the reference's tensor-parallel layers
// (fairscale/nn/model_parallel/layers.py:290,380-382; mappings.py:42-78).

#include "comm_dev.cuh"
#include "gemm_tile.cuh"

namespace fsb {

constexpr int FUSED_BLOCK_N = 256;
// dynamic shared memory of both kernels: operand ring + barriers (SmemLayout) + 4 KB of epilogue staging per epilogue warp
constexpr int FUSED_EPI_OFFSET = SmemLayout<FUSED_BLOCK_N>::EPI_OFFSET;
constexpr int FUSED_SMEM = SmemLayout<FUSED_BLOCK_N>::TOTAL;

constexpr int kMaxNTiles = 64;  // N tiles of the weight-gather GEMM (N <= 16384)

struct FusedParams {
  CommCtx c;
  PtrTable peer;          // ag: every rank's A shard; rs: every rank's staging buffer [M, N]
  uint4* gather;          // ag: local gather buffer [M, K]
  uint32_t* counts;       // per-chunk counters in local memory (monotonic across calls)
  uint32_t target;        // value a chunk counter reaches when the chunk is complete in this call
  uint32_t target_comm;   // rs: value counts[kMaxRanks] reaches when every reduce CTA has folded in all peers
  long long chunk16;      // 16-byte units per chunk (ag: Mc * K * 2 / 16; rs: Mc * N * 2 / 16)
  float* acc;             // rs: local receive buffers, (world - 1) x [Mc, N] bf16 (one per peer, in arrival order)
  __nv_bfloat16* out;     // rs: result [Mc, N]
  const __nv_bfloat16* out_bias;  // rs: bias added once after the reduction (may be null)
  int n_comm;             // CTAs [0, n_comm) communicate, the rest compute
  int Mc;                 // rows per chunk
  // weight-gather GEMM (MODE 2): the B operand is a row range of a flat buffer that arrives shard by shard.
  // N-tile visited o-th: order[o]; it may start once chunks need_lo[tn] .. need_hi[tn] (rank ids) have landed.
  int local_first;        // copy CTAs move the local shard first (its tiles start almost at once)
  uint8_t order[kMaxNTiles], need_lo[kMaxNTiles], need_hi[kMaxNTiles];
};

__device__ __forceinline__ bool wait_counter(const uint32_t* ctr, uint32_t target, volatile int* abort_flag, unsigned long long wait_ns) {
  const uint64_t t0 = globaltimer_ns();
  while (static_cast<int32_t>(ld_acquire_gpu(ctr) - target) < 0) {
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > wait_ns) {
      *abort_flag = 1;
      return false;
    }
    __nanosleep(128);
  }
  return true;
}

// The tcgen05 main loop shared by both kernels.  MODE 0: ag_gemm, MODE 1: gemm_rs.
template <int MODE>
__device__ __forceinline__ void fused_gemm_cta(const CUtensorMap& tmap_a_local, const CUtensorMap& tmap_a, const CUtensorMap& tmap_b,
                                               const GemmParams& p, const FusedParams& f, uint8_t* smem) {
  constexpr int BLOCK_N = FUSED_BLOCK_N;
  using L = SmemLayout<BLOCK_N>;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full_bar = empty_bar + STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);  // warp-uniform
  const int lane = threadIdx.x & 31;
  const int g = blockIdx.x - f.n_comm, G = gridDim.x - f.n_comm;
  const int world = f.c.world, rank = f.c.rank;

  const int tiles_mc = (MODE == 2) ? (p.M + BLOCK_M - 1) / BLOCK_M : f.Mc / BLOCK_M;  // MODE 2: all M tiles
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per_chunk = tiles_mc * tiles_n;
  const int num_tiles = (MODE == 2) ? tiles_per_chunk : tiles_per_chunk * world;
  const int num_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
  // chunk visited k-th: ag starts at home, rs ends at home
  auto chunk_of = [&](int k) { return (rank + k + (MODE == 1 ? 1 : 0)) % world; };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 4);
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_chunk = -1;
      for (int tile = g; tile < num_tiles && ok; tile += G) {
        const int k = (MODE == 2) ? 0 : tile / tiles_per_chunk;
        const int chunk = (MODE == 2) ? rank : chunk_of(k);
        int tm, tn;
        if (MODE == 2) {
          // all M tiles of one N tile run back to back (its weight rows stay in L2), N tiles in arrival order
          tn = f.order[tile / tiles_mc];
          tm = tile % tiles_mc;
          if (ready_chunk != tn) {
            for (int cnk = f.need_lo[tn]; cnk <= f.need_hi[tn] && ok; ++cnk)
              if (!wait_counter(f.counts + cnk, f.target, abort_flag, f.c.wait_ns)) ok = false;
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");  // the copy CTAs' stores before this thread's TMA reads
            ready_chunk = tn;
          }
        } else {
          tile_coords(tile - k * tiles_per_chunk, tiles_mc, tiles_n, tm, tn);
        }
        const int n0 = tn * BLOCK_N;
        const bool local_a = (MODE == 0) && (chunk == rank);
        const int m0 = (MODE == 2) ? tm * BLOCK_M : (local_a ? tm * BLOCK_M : chunk * f.Mc + tm * BLOCK_M);
        if (MODE == 0 && !local_a && ready_chunk != chunk) {
          // the copy CTAs publish a chunk with generic-proxy stores; order them before this thread's TMA reads
          if (!wait_counter(f.counts + chunk, f.target, abort_flag, f.c.wait_ns)) { ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");
          ready_chunk = chunk;
        }
        const CUtensorMap* ta = (local_a || MODE == 2) ? &tmap_a_local : &tmap_a;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          tma_load_2d(sa, ta, &full_bar[stage], k0, m0);
          if (!p.b_mn_major) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j) tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // MMA issuer: all lanes run the loop (warp-uniform addresses and descriptors), one elected lane issues
    {
      const uint32_t idesc = make_idesc_f16(BLOCK_M, BLOCK_N, true, false, p.b_mn_major != 0);
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t b_kstep = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = g; tile < num_tiles && ok; tile += G) {
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
              const uint64_t adesc = make_smem_desc(sa + k * 32u, 16u, 1024u);
              const uint64_t bdesc = make_smem_desc(sb + k * b_kstep, b_lbo, 1024u);
              umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);
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
    const int quad = warp & 3;
    const bool coalesce = epilogue_can_coalesce(p);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = g; tile < num_tiles && ok; tile += G) {
      const int k = (MODE == 2) ? 0 : tile / tiles_per_chunk;
      const int chunk = (MODE == 2) ? 0 : chunk_of(k);
      int tm, tn;
      if (MODE == 2) { tn = f.order[tile / tiles_mc]; tm = tile % tiles_mc; }
      else           { tile_coords(tile - k * tiles_per_chunk, tiles_mc, tiles_n, tm, tn); }
      const int row = (MODE == 2 ? 0 : chunk * f.Mc) + tm * BLOCK_M + quad * 32 + lane;
      const int n0 = tn * BLOCK_N;
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_base = tmem_base + static_cast<uint32_t>(acc * BLOCK_N) + (static_cast<uint32_t>(quad * 32) << 16);
      uint4 pre[8];  // the fused kernels' epilogues read no aux operand
      if (coalesce) epilogue_rows_coalesced(t_base, row - lane, n0, BLOCK_N, p, smem + FUSED_EPI_OFFSET + quad * 4096, lane, pre);
      else          epilogue_rows<BLOCK_N>(t_base, row, n0, p);
      tc_fence_before_sync();
      if (MODE == 1) {
        // publish this warp's share of the tile; the warp that completes the chunk tells its owner.  __syncwarp orders
        // the lanes' stores before lane 0's system-scope fence, which is cumulative over them.
        __syncwarp();
        if (lane == 0) {
          __threadfence_system();
          const uint32_t prev = atomicAdd(f.counts + chunk, 1u);
          if (prev + 1u == f.target) {
            __threadfence_system();
            st_release_sys(f.c.pads[chunk] + f.c.channel * kMaxRanks + rank, f.c.epoch);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
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

// ------------------------------------------------------------------------------------------------ ag_gemm
// Copy engine of a communication CTA: a ring of COPY_BUFS shared-memory buffers of COPY_PIECE bytes, filled by untiled
// bulk loads (which may read a peer's memory) and drained by bulk stores or by the CTA's threads.  One thread drives
// it, so ~190 KB are in flight per CTA whatever the NVLink latency, instead of a few 16-byte loads per thread.
constexpr int COPY_PIECE = 32 * 1024;
constexpr int COPY_BUFS = 6;  // 192 KB: the operand ring of the compute CTAs, which a communication CTA does not use

struct CopyJob { int chunk; long long off; uint32_t bytes; };

// n-th piece this CTA moves: chunks are visited in `order` (k = 0 .. n_chunks-1 -> chunk id), pieces strided by n_comm
__device__ __forceinline__ CopyJob copy_job(int n, int per_cta, long long chunk_bytes, int n_comm, int cta) {
  CopyJob j;
  j.chunk = n / per_cta;  // index into the visiting order
  const long long q = cta + static_cast<long long>(n % per_cta) * n_comm;
  j.off = q * COPY_PIECE;
  const long long left = chunk_bytes - j.off;
  j.bytes = static_cast<uint32_t>(left < COPY_PIECE ? left : COPY_PIECE);
  return j;
}

__device__ __forceinline__ void ag_copy_cta(const FusedParams& f, uint8_t* smem) {
  const CommCtx& c = f.c;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + COPY_BUFS * COPY_PIECE);
  __shared__ int copy_abort;
  if (threadIdx.x == 0) {
    copy_abort = 0;
    for (int i = 0; i < COPY_BUFS; ++i) mbar_init(&full[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (blockIdx.x == 0) signal_peers(c, c.channel);  // my shard is ready (stream order) -> peers may read it
  if (!wait_peers(c, c.channel)) return;
  const long long chunk_bytes = f.chunk16 * 16;
  const long long pieces = (chunk_bytes + COPY_PIECE - 1) / COPY_PIECE;
  const int cta = blockIdx.x;
  const int per_cta = cta < pieces ? static_cast<int>((pieces - cta + f.n_comm - 1) / f.n_comm) : 0;
  const int n_jobs = per_cta * c.world;
  if (threadIdx.x == 0 && per_cta > 0) {
    volatile int* abort_flag = &copy_abort;
    // visiting order: remote chunks in ring order, the local copy last (nothing waits for it) - or first, when the
    // consumers also read the local chunk from the gather buffer (weight-gather GEMM)
    auto chunk_id = [&](int k) { return (c.rank + (f.local_first ? 0 : 1) + k) % c.world; };
    auto issue_load = [&](int n) {
      const CopyJob j = copy_job(n, per_cta, chunk_bytes, f.n_comm, cta);
      const int b = n % COPY_BUFS;
      const uint8_t* src = static_cast<const uint8_t*>(f.peer.p[chunk_id(j.chunk)]) + j.off;
      mbar_expect_tx(&full[b], j.bytes);
      bulk_load_1d(smem + b * COPY_PIECE, src, j.bytes, &full[b]);
    };
    for (int n = 0; n < COPY_BUFS - 1 && n < n_jobs; ++n) issue_load(n);
    bool ok = true;
    for (int n = 0; n < n_jobs && ok; ++n) {
      const CopyJob j = copy_job(n, per_cta, chunk_bytes, f.n_comm, cta);
      const int b = n % COPY_BUFS;
      if (!mbar_wait(&full[b], (n / COPY_BUFS) & 1, abort_flag)) { ok = false; break; }
      uint8_t* dst = reinterpret_cast<uint8_t*>(f.gather) + static_cast<long long>(chunk_id(j.chunk)) * chunk_bytes + j.off;
      bulk_store_1d(dst, smem + b * COPY_PIECE, j.bytes);
      tma_store_commit();
      if (n + COPY_BUFS - 1 < n_jobs) {
        tma_store_wait_read<1>();  // the store issued one job ago has drained its buffer: refill it
        issue_load(n + COPY_BUFS - 1);
      }
      if ((n + 1) % per_cta == 0) {  // last piece of a chunk for this CTA: publish it
        tma_store_wait<0>();
        fence_proxy_async_all();
        __threadfence();
        atomicAdd(f.counts + chunk_id(j.chunk), 1u);
      }
    }
    if (!ok && c.status != nullptr) atomicExch(c.status, FSB_ERR_WAIT_TIMEOUT);
    tma_store_wait<0>();
  } else if (threadIdx.x == 0) {
    for (int k = 0; k < c.world; ++k) atomicAdd(f.counts + k, 1u);  // nothing to copy: still counted as a publisher
  }
  __syncthreads();
  exit_barrier_n(c, c.channel + 1, static_cast<unsigned int>(f.n_comm));  // peers are done reading my shard
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a_local, const __grid_constant__ CUtensorMap tmap_a_gather,
               const __grid_constant__ CUtensorMap tmap_b, GemmParams p, FusedParams f) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (static_cast<int>(blockIdx.x) < f.n_comm) {
    ag_copy_cta(f, smem);
    return;
  }
  fused_gemm_cta<0>(tmap_a_local, tmap_a_gather, tmap_b, p, f, smem);
}

// ------------------------------------------------------------------------------------------------ weight-gather GEMM
// C[M, N] = epilogue( A[M, K] * W^T ) where W [N, K] is a row range of a flat parameter whose shards are being
// all-gathered by the SAME kernel: the copy CTAs pull every rank's shard into the local full-parameter buffer (kept for
// the unit's other products and for backward) and publish one counter per shard; a compute CTA starts an N tile as soon
// as the shards holding its weight rows have landed.  N tiles are visited in arrival order, the local shard first.
__global__ void __launch_bounds__(GEMM_THREADS, 1)
wag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, GemmParams p, FusedParams f) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (static_cast<int>(blockIdx.x) < f.n_comm) {
    ag_copy_cta(f, smem);
    return;
  }
  fused_gemm_cta<2>(tmap_a, tmap_a, tmap_w, p, f, smem);
}

// ------------------------------------------------------------------------------------------------ gemm_rs
__device__ __forceinline__ void unpack8(const uint4& v, float (&o)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { o[2 * i] = __low2float(h[i]); o[2 * i + 1] = __high2float(h[i]); }
}

// Peers' partials of my chunk -> local receive buffers (one per peer, bf16), with the same bulk-copy engine as the
// all-gather: thread 0 waits for a peer's flag, then streams that peer's rows through the shared-memory ring into
// recv[k].  Nothing is added here; the final pass sums the buffers in a fixed order.  Returns false after a timeout.
__device__ __forceinline__ bool rs_pull_cta(const FusedParams& f, uint8_t* smem) {
  const CommCtx& c = f.c;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + COPY_BUFS * COPY_PIECE);
  __shared__ int red_abort;
  if (threadIdx.x == 0) {
    red_abort = 0;
    for (int i = 0; i < COPY_BUFS; ++i) mbar_init(&full[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort_flag = &red_abort;
  const long long chunk_bytes = f.chunk16 * 16;
  const long long pieces = (chunk_bytes + COPY_PIECE - 1) / COPY_PIECE;
  const int cta = blockIdx.x;
  const int per_cta = cta < pieces ? static_cast<int>((pieces - cta + f.n_comm - 1) / f.n_comm) : 0;
  const int n_jobs = per_cta * (c.world - 1);
  if (threadIdx.x == 0 && per_cta > 0) {
    auto peer_of = [&](int k) { return (c.rank - 1 - k + 2 * c.world) % c.world; };  // the order in which peers finish my chunk
    int flag_seen = -1;
    bool ok = true;
    auto issue_load = [&](int n) -> bool {
      const CopyJob j = copy_job(n, per_cta, chunk_bytes, f.n_comm, cta);
      if (j.chunk > flag_seen) {
        const uint32_t* flag = c.pads[c.rank] + c.channel * kMaxRanks + peer_of(j.chunk);
        const uint64_t t0 = globaltimer_ns();
        while (static_cast<int32_t>(ld_acquire_sys(flag) - c.epoch) < 0) {
          if (globaltimer_ns() - t0 > c.wait_ns) {
            *abort_flag = 1;
            return false;
          }
          __nanosleep(128);
        }
        flag_seen = j.chunk;
      }
      const int b = n % COPY_BUFS;
      const uint8_t* src = static_cast<const uint8_t*>(f.peer.p[peer_of(j.chunk)]) + static_cast<long long>(c.rank) * chunk_bytes + j.off;
      mbar_expect_tx(&full[b], j.bytes);
      bulk_load_1d(smem + b * COPY_PIECE, src, j.bytes, &full[b]);
      return true;
    };
    int issued = 0;
    for (; issued < COPY_BUFS - 1 && issued < n_jobs && ok; ++issued) ok = issue_load(issued);
    for (int n = 0; n < n_jobs && ok; ++n) {
      const CopyJob j = copy_job(n, per_cta, chunk_bytes, f.n_comm, cta);
      const int b = n % COPY_BUFS;
      if (!mbar_wait(&full[b], (n / COPY_BUFS) & 1, abort_flag)) { ok = false; break; }
      uint8_t* dst = reinterpret_cast<uint8_t*>(f.acc) + static_cast<long long>(j.chunk) * chunk_bytes + j.off;
      bulk_store_1d(dst, smem + b * COPY_PIECE, j.bytes);
      tma_store_commit();
      if (issued < n_jobs) {
        tma_store_wait_read<1>();  // the store issued one job ago has drained its buffer: refill it
        ok = issue_load(issued++);
      }
    }
    tma_store_wait<0>();
    fence_proxy_async_all();
    if (!ok) {
      *abort_flag = 1;
      if (c.status != nullptr) atomicExch(c.status, FSB_ERR_WAIT_TIMEOUT);
    }
  }
  __syncthreads();
  const bool ok = (*abort_flag == 0);
  __threadfence();
  if (threadIdx.x == 0) atomicAdd(f.counts + kMaxRanks, 1u);
  exit_barrier_n(c, c.channel + 1, static_cast<unsigned int>(f.n_comm));  // peers are done reading my staging buffer
  return ok;
}

// out = my own partial chunk + the peers' partials (receive buffers, fixed order) + bias, on every CTA of the grid once
// its other work is done.
__device__ __forceinline__ void rs_final_pass(const FusedParams& f, int N) {
  __shared__ int final_ok;
  if (threadIdx.x == 0) {
    int dummy_abort = 0;
    bool ok = wait_counter(f.counts + f.c.rank, f.target, &dummy_abort, f.c.wait_ns);               // my own chunk is complete
    if (ok && f.c.world > 1) ok = wait_counter(f.counts + kMaxRanks, f.target_comm, &dummy_abort, f.c.wait_ns);  // peers' rows have landed
    if (!ok && f.c.status != nullptr) atomicExch(f.c.status, FSB_ERR_WAIT_TIMEOUT);
    final_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!final_ok) return;
  const uint4* own = reinterpret_cast<const uint4*>(f.peer.p[f.c.rank]) + static_cast<long long>(f.c.rank) * f.chunk16;
  const uint4* recv = reinterpret_cast<const uint4*>(f.acc);
  const int n16_row = N / 8;
  const int n_peers = f.c.world - 1;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = 4;  // independent 16-byte loads in flight per thread and source: the pass is latency-bound otherwise
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < f.chunk16; i0 += U * stride) {
    uint4 raw[U];
    float v[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      raw[u] = (i < f.chunk16) ? __ldcg(own + i) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) unpack8(raw[u], v[u]);
    for (int k = 0; k < n_peers; ++k) {
      const uint4* rk = recv + static_cast<long long>(k) * f.chunk16;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        raw[u] = (i < f.chunk16) ? __ldcg(rk + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float x[8];
        unpack8(raw[u], x);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[u][e] += x[e];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= f.chunk16) continue;
      if (f.out_bias != nullptr) {
        float b[8];
        unpack8(*reinterpret_cast<const uint4*>(f.out_bias + static_cast<int>(i % n16_row) * 8), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[u][e] += b[e];
      }
      Vec16<__nv_bfloat16> o;
#pragma unroll
      for (int e = 0; e < 8; ++e) o.v[e] = __float2bfloat16_rn(v[u][e]);
      st16(f.out + i * 8, o);
    }
  }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p, FusedParams f) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (static_cast<int>(blockIdx.x) < f.n_comm) {
    if (f.c.world > 1 && !rs_pull_cta(f, smem)) return;
  } else {
    fused_gemm_cta<1>(tmap_a, tmap_a, tmap_b, p, f, smem);
  }
  rs_final_pass(f, p.N);
}

}  // namespace fsb

// C ABI ------------------------------------------------------------------------------------------
static fsb::CommCtx fused_ctx(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter, int* status) {
  fsb::CommCtx c{};
  c.rank = rank; c.world = world; c.epoch = epoch; c.channel = channel;
  for (int i = 0; i < world && i < fsb::kMaxRanks; ++i) c.pads[i] = static_cast<uint32_t*>(pads[i]);
  c.counter = static_cast<unsigned int*>(counter);
  c.status = status;
  c.wait_ns = fsb_host::comm_wait_ns();
  return c;
}

static int fused_grid(int n_comm, int tiles, int* grid_out) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (n_comm < 1 || n_comm >= sms) return -1;
  int gemm_ctas = sms - n_comm;  // every CTA must be resident at once: the compute CTAs wait for the copy CTAs
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  *grid_out = n_comm + gemm_ctas;
  return 0;
}

// C[M, N] (bf16, ldc) = epilogue( gather(A)[M, K] * B^T ).  a_peers[r]: rank r's shard [Mc, K] (contiguous, in the
// symmetric heap); a_local: this rank's shard; gather: local [M, K] buffer that receives every chunk.
// B is [N, K] (K-major) or [K, N] (b_mn_major).  counts: `world` uint32 in local memory, zero at first use;
// target: cumulative n_comm * (number of calls that used `counts`), this call included.
FSB_API int fsb_ag_gemm_bf16(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                             void* const* a_peers, const void* a_local, void* gather, const void* B, void* C, const void* bias,
                             void* aux_out, int M, int N, int K, int ldb, int ldc, int b_mn_major, int epilogue, void* counts,
                             unsigned target, int n_comm, int* status, cudaStream_t stream) {
  using namespace fsb;
  if (world < 1 || world > kMaxRanks || M % world) return -1;
  const int Mc = M / world;
  if (Mc % BLOCK_M || K % 8 || ldb % 8 || ldc % 8) return -1;
  if (epilogue != EPI_NONE && epilogue != EPI_BIAS && epilogue != EPI_BIAS_GELU) return -1;
  CUtensorMap tl, tg, tb;
  bool ok = fsb_host::encode_2d_16bit(&tl, a_local, (uint64_t)K, (uint64_t)Mc, (uint64_t)K, BLOCK_K, BLOCK_M);
  ok &= fsb_host::encode_2d_16bit(&tg, gather, (uint64_t)K, (uint64_t)M, (uint64_t)K, BLOCK_K, BLOCK_M);
  if (!b_mn_major) ok &= fsb_host::encode_2d_16bit(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, FUSED_BLOCK_N);
  else             ok &= fsb_host::encode_2d_16bit(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K);
  if (!ok) return -1;
  GemmParams p{};
  p.C = C; p.bias = static_cast<const __nv_bfloat16*>(bias); p.aux = nullptr; p.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ld_aux = ldc; p.a_mn_major = 0; p.b_mn_major = b_mn_major;
  p.epilogue = epilogue; p.out_f32 = 0; p.accumulate_c = 0; p.status = status; p.batch = 1;
  FusedParams f{};
  f.c = fused_ctx(rank, world, epoch, channel, pads, counter, status);
  for (int i = 0; i < world; ++i) f.peer.p[i] = a_peers[i];
  f.gather = static_cast<uint4*>(gather);
  f.counts = static_cast<uint32_t*>(counts);
  f.target = target;
  f.chunk16 = static_cast<long long>(Mc) * K * 2 / 16;
  f.n_comm = n_comm; f.Mc = Mc;
  int grid = 0;
  const int tiles = (M / BLOCK_M) * ((N + FUSED_BLOCK_N - 1) / FUSED_BLOCK_N);
  if (fused_grid(n_comm, tiles, &grid) != 0) return -1;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_set[64] = {false};  // the attribute is per device
  if (!attr_set[dev & 63]) {
    cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FUSED_SMEM);
    attr_set[dev & 63] = true;
  }
  ag_gemm_kernel<<<grid, GEMM_THREADS, FUSED_SMEM, stream>>>(tl, tg, tb, p, f);
  return static_cast<int>(cudaGetLastError());
}

// Weight-gather GEMM (FSDP: the all-gather of a unit's flat parameter fused with the first product that consumes it).
//   shard_peers[r]: rank r's shard of the flat parameter (shard_elems bf16, in the symmetric heap)
//   full: local buffer of world * shard_elems bf16 that receives every shard (the gathered flat parameter)
//   W = full + w_offset, [N, K] row-major (w_offset and K multiples of 8);  C[M, N] = epilogue(A[M, K] W^T + bias)
// bias (optional) must already be valid (it is NOT awaited).  counts / target as for fsb_ag_gemm_bf16.
FSB_API int fsb_wag_gemm_bf16(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                              void* const* shard_peers, long long shard_elems, void* full, long long w_offset, const void* A,
                              void* C, const void* bias, void* aux_out, int M, int N, int K, int lda, int ldc, int epilogue,
                              void* counts, unsigned target, int n_comm, int* status, cudaStream_t stream) {
  using namespace fsb;
  if (world < 1 || world > kMaxRanks || K % 8 || lda % 8 || ldc % 8 || w_offset % 8 || (shard_elems * 2) % 16) return -1;
  if (epilogue != EPI_NONE && epilogue != EPI_BIAS && epilogue != EPI_BIAS_GELU) return -1;
  const int tiles_n = (N + FUSED_BLOCK_N - 1) / FUSED_BLOCK_N;
  if (tiles_n > kMaxNTiles || w_offset + static_cast<long long>(N) * K > shard_elems * world) return -1;
  const __nv_bfloat16* W = static_cast<const __nv_bfloat16*>(full) + w_offset;
  CUtensorMap ta, tw;
  bool ok = fsb_host::encode_2d_16bit(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M);
  ok &= fsb_host::encode_2d_16bit(&tw, W, (uint64_t)K, (uint64_t)N, (uint64_t)K, BLOCK_K, FUSED_BLOCK_N);
  if (!ok) return -1;
  GemmParams p{};
  p.C = C; p.bias = static_cast<const __nv_bfloat16*>(bias); p.aux = nullptr; p.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ld_aux = ldc; p.a_mn_major = 0; p.b_mn_major = 0;
  p.epilogue = epilogue; p.out_f32 = 0; p.accumulate_c = 0; p.status = status; p.batch = 1;
  FusedParams f{};
  f.c = fused_ctx(rank, world, epoch, channel, pads, counter, status);
  for (int i = 0; i < world; ++i) f.peer.p[i] = shard_peers[i];
  f.gather = static_cast<uint4*>(full);
  f.counts = static_cast<uint32_t*>(counts);
  f.target = target;
  f.chunk16 = shard_elems * 2 / 16;
  f.n_comm = n_comm; f.Mc = 0; f.local_first = 1;
  // plan: which shards an N tile needs and in which order the tiles become runnable (shard r arrives (r - rank) mod
  // world-th; a tile is runnable when its last shard is)
  int ready_pos[kMaxNTiles];
  for (int tn = 0; tn < tiles_n; ++tn) {
    const long long first = w_offset + static_cast<long long>(tn) * FUSED_BLOCK_N * K;
    const int rows = (tn + 1) * FUSED_BLOCK_N <= N ? FUSED_BLOCK_N : N - tn * FUSED_BLOCK_N;
    const long long last = first + static_cast<long long>(rows) * K - 1;
    const int lo = static_cast<int>(first / shard_elems), hi = static_cast<int>(last / shard_elems);
    f.need_lo[tn] = static_cast<uint8_t>(lo);
    f.need_hi[tn] = static_cast<uint8_t>(hi);
    int pos = 0;
    for (int c = lo; c <= hi; ++c) {
      const int q = (c - rank + world) % world;
      if (q > pos) pos = q;
    }
    ready_pos[tn] = pos;
  }
  int filled = 0;
  for (int pos = 0; pos < world; ++pos)
    for (int tn = 0; tn < tiles_n; ++tn)
      if (ready_pos[tn] == pos) f.order[filled++] = static_cast<uint8_t>(tn);
  int grid = 0;
  const int tiles = ((M + BLOCK_M - 1) / BLOCK_M) * tiles_n;
  if (fused_grid(n_comm, tiles, &grid) != 0) return -1;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_set[64] = {false};
  if (!attr_set[dev & 63]) {
    cudaFuncSetAttribute(wag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FUSED_SMEM);
    attr_set[dev & 63] = true;
  }
  wag_gemm_kernel<<<grid, GEMM_THREADS, FUSED_SMEM, stream>>>(ta, tw, p, f);
  return static_cast<int>(cudaGetLastError());
}

// out[Mc, N] (bf16) = sum over ranks of (A[M, K] * B^T)[my chunk's rows] (+ out_bias).  stage_peers[r]: rank r's
// staging buffer [M, N] bf16 in the symmetric heap (this rank writes stage_peers[rank]); acc: local receive buffers,
// (world - 1) * Mc * N bf16;
// counts: kMaxRanks + 1 uint32; target as for ag_gemm but counting 4 * tiles-per-chunk arrivals per call;
// target_comm: cumulative n_comm over the calls (with world > 1) that used `counts`.
FSB_API int fsb_gemm_rs_bf16(int rank, int world, unsigned epoch, int channel, void* const* pads, void* counter,
                             void* const* stage_peers, const void* A, const void* B, void* out, const void* out_bias, void* acc,
                             int M, int N, int K, int lda, int ldb, int b_mn_major, void* counts, unsigned target,
                             unsigned target_comm, int n_comm, int* status, cudaStream_t stream) {
  using namespace fsb;
  if (world < 1 || world > kMaxRanks || M % world) return -1;
  const int Mc = M / world;
  if (Mc % BLOCK_M || N % 8 || lda % 8 || ldb % 8) return -1;
  CUtensorMap ta, tb;
  bool ok = fsb_host::encode_2d_16bit(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BLOCK_K, BLOCK_M);
  if (!b_mn_major) ok &= fsb_host::encode_2d_16bit(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BLOCK_K, FUSED_BLOCK_N);
  else             ok &= fsb_host::encode_2d_16bit(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 64, BLOCK_K);
  if (!ok) return -1;
  GemmParams p{};
  p.C = const_cast<void*>(stage_peers[rank]);
  p.M = M; p.N = N; p.K = K; p.ldc = N; p.ld_aux = N; p.a_mn_major = 0; p.b_mn_major = b_mn_major;
  p.epilogue = EPI_NONE; p.out_f32 = 0; p.accumulate_c = 0; p.status = status; p.batch = 1;
  FusedParams f{};
  f.c = fused_ctx(rank, world, epoch, channel, pads, counter, status);
  for (int i = 0; i < world; ++i) f.peer.p[i] = stage_peers[i];
  f.counts = static_cast<uint32_t*>(counts);
  f.target = target;
  f.target_comm = target_comm;
  f.chunk16 = static_cast<long long>(Mc) * N * 2 / 16;
  f.acc = static_cast<float*>(acc);
  f.out = static_cast<__nv_bfloat16*>(out);
  f.out_bias = static_cast<const __nv_bfloat16*>(out_bias);
  f.n_comm = n_comm; f.Mc = Mc;
  int grid = 0;
  const int tiles = (M / BLOCK_M) * ((N + FUSED_BLOCK_N - 1) / FUSED_BLOCK_N);
  if (fused_grid(n_comm, tiles, &grid) != 0) return -1;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool attr_set[64] = {false};  // the attribute is per device
  if (!attr_set[dev & 63]) {
    cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FUSED_SMEM);
    attr_set[dev & 63] = true;
  }
  gemm_rs_kernel<<<grid, GEMM_THREADS, FUSED_SMEM, stream>>>(ta, tb, p, f);
  return static_cast<int>(cudaGetLastError());
}

// arrivals per chunk and call that fsb_gemm_rs_bf16 counts (the caller accumulates `target` with it)
FSB_API int fsb_gemm_rs_arrivals(int M, int N, int world) {
  using namespace fsb;
  if (world < 1 || M % world || (M / world) % BLOCK_M) return -1;
  return 4 * (M / world / BLOCK_M) * ((N + FUSED_BLOCK_N - 1) / FUSED_BLOCK_N);
}
