// Column-parallel encoder GEMM for all layers in one persistent launch (sm_100a).
//
//   C[l][m, n] = sum_k A[l][m, k] * B[l][n, k] + bias[l][n]          (bf16 in, fp32 accumulate, bf16 out)
//
// A = token activations [L, M, K], B = encoder weights [L, N, K] (both K-major), C = pre-activations.
// Counterpart of the reference's per-layer F.linear calls (clt/models/parallel.py:286 through
// clt/models/encoder.py:101).
//
// Structure: one CTA per SM, 6 warps.  Warp 0 feeds a 4-stage shared-memory ring with TMA tile loads
// (no cluster multicast: every CTA fetches its own tiles), warp 1 issues tcgen05.mma 128x256x16 into one
// of two 256-column TMEM accumulators, warps 2-5 drain the other accumulator with tcgen05.ld, add the
// bias and store bf16.  Tiles are ordered m-fastest so CTAs that run together share the weight tile in L2.
// Every mbarrier wait is bounded; on a timeout the CTA records STATUS_WAIT_TIMEOUT, drains its copies,
// frees its TMEM and returns.
#include <cstdlib>

#include "common.cuh"

namespace clt {

namespace gemm {
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzled row
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t B_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
// ring + 1024 B alignment slack + barriers/bias
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 4 * 4096 + 1024 + 4096;  // ring + epilogue staging + slack + barriers
}  // namespace gemm

// Epilogue of one 32-row slab (one warp, lane = row): TMEM -> registers -> + bias -> bf16 -> shared staging
// tile of 32 rows x 64 columns in the 128-byte-swizzled layout -> one TMA store per 64 columns.  Writing
// full rows through TMA instead of 16 bytes per lane and row keeps the L1/shared data pipe, which the tensor
// core's operand reads share, almost free.  `stage` is this warp's 4 KB buffer (1024-byte aligned).
constexpr int kEpiCols = 64;
constexpr uint32_t kEpiStageBytes = 32 * kEpiCols * 2;

// With `colacc` (shared, [2][BN] floats: sums and sums of squares per tile column) the slab's column statistics
// of the rounded bf16 values are read back from the staging tile (each lane owns two adjacent columns) and
// added up over the tile's four slabs; `nrows` masks the rows beyond the matrix.
__device__ __forceinline__ void epilogue_slab(uint32_t taddr, const CUtensorMap* map_c, uint8_t* stage, const float* bias_s,
                                              int bn, int n_base, int m_base, int l, int lane, float* colacc, int bn_full, int nrows) {
  for (int c = 0; c < bn / kEpiCols; ++c) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(taddr + c * kEpiCols, r0);
    tmem_ld_32x32(taddr + c * kEpiCols + 32, r1);
    if (lane == 0) bulk_wait_read<0>();  // the previous store has read the staging tile
    __syncwarp();
    tmem_ld_wait();
    const float4* b4 = reinterpret_cast<const float4*>(bias_s + c * kEpiCols);
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // 16-byte chunk j of this lane's row: columns [8j, 8j + 8)
      const uint32_t* r = j < 4 ? &r0[8 * j] : &r1[8 * (j - 4)];
      const float4 ba = b4[2 * j], bb = b4[2 * j + 1];
      uint4 q;
      q.x = pack_t16x2(__uint_as_float(r[0]) + ba.x, __uint_as_float(r[1]) + ba.y);
      q.y = pack_t16x2(__uint_as_float(r[2]) + ba.z, __uint_as_float(r[3]) + ba.w);
      q.z = pack_t16x2(__uint_as_float(r[4]) + bb.x, __uint_as_float(r[5]) + bb.y);
      q.w = pack_t16x2(__uint_as_float(r[6]) + bb.z, __uint_as_float(r[7]) + bb.w);
      *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = q;
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(map_c, stage, n_base + c * kEpiCols, m_base, l);
      bulk_commit();
    }
    if (colacc != nullptr) {
      float s0 = 0.f, s1 = 0.f, q0 = 0.f, q1 = 0.f;
      const uint32_t chunk = uint32_t(lane >> 2), inner = uint32_t(lane & 3) * 4u;
#pragma unroll 8
      for (int r = 0; r < 32; ++r) {
        if (r < nrows) {
          const uint32_t u = *reinterpret_cast<const uint32_t*>(stage + r * 128 + ((chunk ^ uint32_t(r & 7)) << 4) + inner);
          const float a = t16_lo(u), b = t16_hi(u);
          s0 += a; q0 = fmaf(a, a, q0);
          s1 += b; q1 = fmaf(b, b, q1);
        }
      }
      const int col = c * kEpiCols + 2 * lane;
      atomicAdd(&colacc[col], s0); atomicAdd(&colacc[col + 1], s1);
      atomicAdd(&colacc[bn_full + col], q0); atomicAdd(&colacc[bn_full + col + 1], q1);
    }
  }
}

// Per-tile column statistics -> global partials [L][row blocks of 128][N][2], then cleared for the next tile.
__device__ __forceinline__ void flush_tile_stats(float* colacc, int bn_full, float* tile_stats, int l, int row_block, int row_blocks,
                                                 int n_base, int N, int etid) {
  for (int j = etid; j < bn_full; j += 128) {
    const int n = n_base + j;
    if (n < N && row_block < row_blocks) {
      float2* dst = reinterpret_cast<float2*>(tile_stats) + (1LL * l * row_blocks + row_block) * N + n;
      *dst = make_float2(colacc[j], colacc[bn_full + j]);
    }
    colacc[j] = 0.f;
    colacc[bn_full + j] = 0.f;
  }
}

struct GemmShared {
  uint64_t full[gemm::STAGES];
  uint64_t empty[gemm::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_ok;
  alignas(16) float bias[gemm::BN];
  float colacc[2 * gemm::BN];
};

__global__ void __launch_bounds__(gemm::NUM_THREADS, 1)
encoder_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const t16* __restrict__ bias,
                    int L, int M, int N, int K, long long ldc, long long layer_stride_c, int* __restrict__ status,
                    float* __restrict__ tile_stats) {
  using namespace gemm;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = tiles + size_t(STAGES) * STAGE_BYTES;  // four 4 KB staging tiles, 1024-byte aligned
  GemmShared* sh = reinterpret_cast<GemmShared*>(epi_stage + 4 * kEpiStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_kb = (K + BK - 1) / BK;
  const long long total_tiles = 1LL * L * tiles_m * tiles_n;
  volatile int* abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->tmem_full[b], 1);
      mbar_init(&sh->tmem_empty[b], 4);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  for (int j = threadIdx.x; j < 2 * BN; j += NUM_THREADS) sh->colacc[j] = 0.f;
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int mt = int(t % tiles_m);
        const int nt = int((t / tiles_m) % tiles_n);
        const int l = int(t / (1LL * tiles_m * tiles_n));
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&sh->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&sh->full[s], STAGE_BYTES);
          uint8_t* a_dst = tiles + size_t(s) * STAGE_BYTES;
          tma_load_3d(a_dst, &map_a, &sh->full[s], kb * BK, mt * BM, l);
          tma_load_3d(a_dst + A_BYTES, &map_b, &sh->full[s], kb * BK, nt * BN, l);
        }
      }
      if (!ok) {
        // Give the copies already issued a bounded chance to land before the CTA retires.
        const uint32_t issued = it;
        const uint32_t first = issued > STAGES ? issued - STAGES : 0;
        for (uint32_t j = first; j < issued; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(&sh->full[j % STAGES], (j / STAGES) & 1)) {
            if (clock64() - start > kWaitTimeoutCycles) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
        const uint32_t buf = local_tile & 1;
        const uint32_t tph = (local_tile >> 1) & 1;
        if (!mbar_wait(&sh->tmem_empty[buf], tph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&sh->full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + size_t(s) * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = umma_desc_kmajor_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance 16 elements (32 bytes) along K inside the swizzled row: +2 in 16-byte units
            umma_bf16_ss(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, (kb | k) != 0);
          }
          tc_commit(&sh->empty[s]);  // frees the stage when these MMAs have read it
        }
        if (ok) tc_commit(&sh->tmem_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int etid = (warp - 2) * 32 + lane;
    const int row_blocks = (M + 127) / 128;
    int prev_l = -1, prev_rb = 0, prev_n = 0;
    uint32_t local_tile = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
      const int mt = int(t % tiles_m);
      const int nt = int((t / tiles_m) % tiles_n);
      const int l = int(t / (1LL * tiles_m * tiles_n));
      const uint32_t buf = local_tile & 1;
      const uint32_t tph = (local_tile >> 1) & 1;
      named_barrier_sync(1, 128);  // previous tile's bias reads and column sums are done
      if (tile_stats != nullptr && prev_l >= 0) flush_tile_stats(sh->colacc, BN, tile_stats, prev_l, prev_rb, row_blocks, prev_n, N, etid);
      prev_l = l; prev_rb = mt; prev_n = nt * BN;
      for (int j = etid; j < BN; j += 128) {
        const int n = nt * BN + j;
        sh->bias[j] = (bias != nullptr && n < N) ? t16_to_float(bias[1LL * l * N + n]) : 0.f;
      }
      // One thread performs the bounded wait and publishes the outcome, so the four warps always
      // take the same branch and nobody is left alone at a named barrier.
      if (etid == 0) sh->epi_ok = mbar_wait(&sh->tmem_full[buf], tph, abort_flag) ? 1 : 0;
      named_barrier_sync(1, 128);
      if (!sh->epi_ok) { ok = false; break; }
      tc_fence_after();
      const int m_base = mt * BM + quarter * 32;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quarter * 32) << 16);
      if (m_base < M) epilogue_slab(taddr, &map_c, epi_stage + (warp - 2) * kEpiStageBytes, sh->bias, min(BN, ((N - nt * BN + kEpiCols - 1) / kEpiCols) * kEpiCols), nt * BN, m_base, l, lane,
                                    tile_stats != nullptr ? sh->colacc : nullptr, BN, min(32, M - m_base));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
    }
    if (ok && tile_stats != nullptr && prev_l >= 0) {
      named_barrier_sync(1, 128);
      flush_tile_stats(sh->colacc, BN, tile_stats, prev_l, prev_rb, row_blocks, prev_n, N, etid);
    }
  }

  if (warp >= 2 && lane == 0) bulk_wait_all();  // output stores of this warp are complete
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh->abort_flag && status != nullptr) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ CTA-pair variant (cta_group::2)
// Two CTAs of a cluster work on one 256 x 256 tile: each loads its own 128 rows of A and one half (128 rows)
// of the weight tile, the leader CTA issues tcgen05.mma with cta_group::2 (M = 256), which reads the operand
// halves from both CTAs' shared memory and writes 128 accumulator rows into each CTA's TMEM.  Per CTA and
// k-step this moves 32 KB from L2 instead of 48 KB for the same number of MMA cycles, and the ring holds six
// stages instead of four.  No multicast loads: tcgen05.commit is the only multicast (barrier arrivals).
//
//   full[s]        leader only: armed by the leader's producer for the bytes of both CTAs
//   empty[s]       both CTAs: commit (multicast) after the MMAs of the stage
//   tmem_full[b]   both CTAs: commit (multicast) after the tile's last MMA
//   tmem_empty[b]  leader only: 8 arrivals, four epilogue warps of each CTA
namespace gemm2 {
constexpr int BM = 128;       // rows per CTA; the pair covers 256
constexpr int BN = 256;
constexpr int BN_HALF = 128;  // weight rows loaded per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t B_BYTES = BN_HALF * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 4 * 4096 + 1024 + 4096;
}  // namespace gemm2

struct GemmPairShared {
  uint64_t full[gemm2::STAGES];
  uint64_t empty[gemm2::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_ok;
  alignas(16) float bias[gemm2::BN];
  float colacc[2 * gemm2::BN];
};

__global__ void __launch_bounds__(gemm2::NUM_THREADS, 1)
encoder_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, const t16* __restrict__ bias,
                         int L, int M, int N, int K, long long ldc, long long layer_stride_c, int* __restrict__ status,
                         float* __restrict__ tile_stats) {
  using namespace gemm2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = tiles + size_t(STAGES) * STAGE_BYTES;
  GemmPairShared* sh = reinterpret_cast<GemmPairShared*>(epi_stage + 4 * kEpiStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (N + BN - 1) / BN;
  const int num_kb = (K + BK - 1) / BK;
  const long long total_tiles = 1LL * L * tiles_m * tiles_n;
  volatile int* abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->tmem_full[b], 1);
      mbar_init(&sh->tmem_empty[b], 8);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  for (int j = threadIdx.x; j < 2 * BN; j += NUM_THREADS) sh->colacc[j] = 0.f;
  if (warp == 1) {
    tmem_alloc_pair(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (long long t = pair; t < total_tiles && ok; t += npairs) {
        const int mt = int(t % tiles_m);
        const int nt = int((t / tiles_m) % tiles_n);
        const int l = int(t / (1LL * tiles_m * tiles_n));
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&sh->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_expect_tx(&sh->full[s], 2 * STAGE_BYTES);
          const uint32_t full_leader = mapa_shared(smem_u32(&sh->full[s]), 0);
          uint8_t* a_dst = tiles + size_t(s) * STAGE_BYTES;
          tma_load_3d_pair(a_dst, &map_a, full_leader, kb * BK, (mt * 2 + int(cta_rank)) * BM, l);
          tma_load_3d_pair(a_dst + A_BYTES, &map_b, full_leader, kb * BK, nt * BN + int(cta_rank) * BN_HALF, l);
        }
      }
      // Copies still in flight are counted on the leader's barriers, which the MMA thread consumes; a CTA
      // that gave up waits below (cluster barrier) until its partner is done as well.
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (long long t = pair; t < total_tiles && ok; t += npairs, ++local_tile) {
        const uint32_t buf = local_tile & 1;
        const uint32_t tph = (local_tile >> 1) & 1;
        if (!mbar_wait(&sh->tmem_empty[buf], tph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&sh->full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + size_t(s) * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = umma_desc_kmajor_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_ss_pair(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, (kb | k) != 0);
          tc_commit_pair(&sh->empty[s], 3);  // frees the stage in both CTAs
        }
        if (ok) tc_commit_pair(&sh->tmem_full[buf], 3);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const int etid = (warp - 2) * 32 + lane;
    const int row_blocks = (M + 127) / 128;
    int prev_l = -1, prev_rb = 0, prev_n = 0;
    uint32_t local_tile = 0;
    bool ok = true;
    for (long long t = pair; t < total_tiles && ok; t += npairs, ++local_tile) {
      const int mt = int(t % tiles_m);
      const int nt = int((t / tiles_m) % tiles_n);
      const int l = int(t / (1LL * tiles_m * tiles_n));
      const uint32_t buf = local_tile & 1;
      const uint32_t tph = (local_tile >> 1) & 1;
      named_barrier_sync(1, 128);
      if (tile_stats != nullptr && prev_l >= 0) flush_tile_stats(sh->colacc, BN, tile_stats, prev_l, prev_rb, row_blocks, prev_n, N, etid);
      prev_l = l; prev_rb = mt * 2 + int(cta_rank); prev_n = nt * BN;
      for (int j = etid; j < BN; j += 128) {
        const int n = nt * BN + j;
        sh->bias[j] = (bias != nullptr && n < N) ? t16_to_float(bias[1LL * l * N + n]) : 0.f;
      }
      if (etid == 0) sh->epi_ok = mbar_wait(&sh->tmem_full[buf], tph, abort_flag) ? 1 : 0;
      named_barrier_sync(1, 128);
      if (!sh->epi_ok) { ok = false; break; }
      tc_fence_after();
      const int m_base = (mt * 2 + int(cta_rank)) * BM + quarter * 32;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quarter * 32) << 16);
      if (m_base < M) epilogue_slab(taddr, &map_c, epi_stage + (warp - 2) * kEpiStageBytes, sh->bias, min(BN, ((N - nt * BN + kEpiCols - 1) / kEpiCols) * kEpiCols), nt * BN, m_base, l, lane,
                                    tile_stats != nullptr ? sh->colacc : nullptr, BN, min(32, M - m_base));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&sh->tmem_empty[buf]), 0));  // the leader's barrier
    }
    if (ok && tile_stats != nullptr && prev_l >= 0) {
      named_barrier_sync(1, 128);
      flush_tile_stats(sh->colacc, BN, tile_stats, prev_l, prev_rb, row_blocks, prev_n, N, etid);
    }
  }

  if (warp >= 2 && lane == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA retires (or frees TMEM) while the other may still use its memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh->abort_flag && status != nullptr) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [layers, rows, K] bf16, K contiguous; box = [1, box_rows, 64] with the 128-byte swizzle.
static bool make_kmajor_map(CUtensorMap* map, const void* base, int layers, int rows, int K, long long row_stride_elems,
                            long long layer_stride_elems, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {cuuint64_t(K), cuuint64_t(rows), cuuint64_t(layers)};
  cuuint64_t strides[2] = {cuuint64_t(row_stride_elems) * 2, cuuint64_t(layer_stride_elems) * 2};
  cuuint32_t box[3] = {cuuint32_t(gemm::BK), cuuint32_t(box_rows), 1};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = enc(map, (CLT_T16_IS_HALF ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16), 3, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace clt

// Returns 0 on success, a negative value when the arguments cannot be handled (the caller raises).
// tile_stats (optional): [L][ceil(M / 128)][N][2] fp32, receives per 128-row block and column the sum and the sum of
// squares of the stored (bf16-rounded) outputs; every element is written, nothing has to be cleared.
extern "C" int CLT_FN(clt_encoder_gemm)(const void* A, const void* B, const void* bias, void* C, int L, int M, int N, int K,
                                long long ldc, long long layer_stride_c, int* status, float* tile_stats, int num_sms, cudaStream_t stream) {
  using namespace clt;
  if (K % 8 != 0 || ldc % 8 != 0 || layer_stride_c % 8 != 0) return -1;  // 16-byte TMA strides / vector stores
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -2;
  CUtensorMap map_a, map_b, map_c;
  if (!make_kmajor_map(&map_a, A, L, M, K, K, 1LL * M * K, gemm::BM)) return -3;
  // output map: [L, M, N] with 64-column x 32-row boxes (one epilogue slab store), clipped at M and N
  if (!make_kmajor_map(&map_c, C, L, M, N, ldc, layer_stride_c, 32)) return -3;
  // ---- CTA pairs when the problem has full 256-row tiles and the device can co-schedule clusters of two
  static int pair_clusters = -1;  // co-resident clusters of two, probed once
  if (pair_clusters < 0) {
    pair_clusters = 0;
    if (cudaFuncSetAttribute(encoder_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm2::SMEM_BYTES)) == cudaSuccess) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(2 * num_sms);
      probe.blockDim = dim3(gemm2::NUM_THREADS);
      probe.dynamicSmemBytes = gemm2::SMEM_BYTES;
      cudaLaunchAttribute pattr[1];
      pattr[0].id = cudaLaunchAttributeClusterDimension;
      pattr[0].val.clusterDim.x = 2; pattr[0].val.clusterDim.y = 1; pattr[0].val.clusterDim.z = 1;
      probe.attrs = pattr;
      probe.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, encoder_gemm_pair_kernel, &probe) == cudaSuccess && n > 0) pair_clusters = n;
      else (void)cudaGetLastError();
    } else {
      (void)cudaGetLastError();
    }
  }
  const long long pair_tiles = 1LL * L * ((M + 2 * gemm2::BM - 1) / (2 * gemm2::BM)) * ((N + gemm2::BN - 1) / gemm2::BN);
  // CLT_GEMM_SINGLE_CTA=1 keeps the single-CTA 128x256 kernel for every shape (for comparisons)
  static const bool force_single = [] { const char* e = getenv("CLT_GEMM_SINGLE_CTA"); return e != nullptr && e[0] == '1'; }();
  if (pair_clusters > 0 && !force_single && M >= 2 * gemm2::BM && pair_tiles > 0) {
    if (!make_kmajor_map(&map_b, B, L, N, K, K, 1LL * N * K, gemm2::BN_HALF)) return -3;
    const int clusters = int(pair_tiles < pair_clusters ? pair_tiles : pair_clusters);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(gemm2::NUM_THREADS);
    cfg.dynamicSmemBytes = gemm2::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const t16* bias_p = static_cast<const t16*>(bias);
    if (cudaLaunchKernelEx(&cfg, encoder_gemm_pair_kernel, map_a, map_b, map_c, bias_p, L, M, N, K, ldc, layer_stride_c, status, tile_stats) != cudaSuccess)
      return -5;
    return 0;
  }
  if (!make_kmajor_map(&map_b, B, L, N, K, K, 1LL * N * K, gemm::BN)) return -3;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(encoder_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm::SMEM_BYTES)) != cudaSuccess) return -4;
    attr_set = true;
  }
  const long long tiles = 1LL * L * ((M + gemm::BM - 1) / gemm::BM) * ((N + gemm::BN - 1) / gemm::BN);
  if (tiles == 0) return 0;
  const int grid = int(tiles < num_sms ? tiles : num_sms);
  encoder_gemm_kernel<<<grid, gemm::NUM_THREADS, gemm::SMEM_BYTES, stream>>>(
      map_a, map_b, map_c, static_cast<const t16*>(bias), L, M, N, K, ldc, layer_stride_c, status, tile_stats);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
