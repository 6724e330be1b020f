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
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024 + 2048;
}  // namespace gemm

struct GemmShared {
  uint64_t full[gemm::STAGES];
  uint64_t empty[gemm::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_ok;
  float bias[gemm::BN];
};

__global__ void __launch_bounds__(gemm::NUM_THREADS, 1)
encoder_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ C,
                    int L, int M, int N, int K, long long ldc, long long layer_stride_c, int* __restrict__ status) {
  using namespace gemm;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmShared* sh = reinterpret_cast<GemmShared*>(tiles + size_t(STAGES) * STAGE_BYTES);

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
    uint32_t local_tile = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
      const int mt = int(t % tiles_m);
      const int nt = int((t / tiles_m) % tiles_n);
      const int l = int(t / (1LL * tiles_m * tiles_n));
      const uint32_t buf = local_tile & 1;
      const uint32_t tph = (local_tile >> 1) & 1;
      named_barrier_sync(1, 128);  // previous tile's bias reads are done
      for (int j = etid; j < BN; j += 128) {
        const int n = nt * BN + j;
        sh->bias[j] = (bias != nullptr && n < N) ? __bfloat162float(bias[1LL * l * N + n]) : 0.f;
      }
      // One thread performs the bounded wait and publishes the outcome, so the four warps always
      // take the same branch and nobody is left alone at a named barrier.
      if (etid == 0) sh->epi_ok = mbar_wait(&sh->tmem_full[buf], tph, abort_flag) ? 1 : 0;
      named_barrier_sync(1, 128);
      if (!sh->epi_ok) { ok = false; break; }
      tc_fence_after();
      const int m = mt * BM + quarter * 32 + lane;
      __nv_bfloat16* crow = C + 1LL * l * layer_stride_c + 1LL * m * ldc + 1LL * nt * BN;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int n0 = nt * BN + c * 32;
        if (m < M && n0 < N) {
          uint32_t packed[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float v0 = __uint_as_float(r[2 * j]) + sh->bias[c * 32 + 2 * j];
            const float v1 = __uint_as_float(r[2 * j + 1]) + sh->bias[c * 32 + 2 * j + 1];
            packed[j] = pack_bf16x2(v0, v1);
          }
          if (n0 + 32 <= N) {
            uint4* dst = reinterpret_cast<uint4*>(crow + c * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          } else {
            const __nv_bfloat16* pv = reinterpret_cast<const __nv_bfloat16*>(packed);
            for (int j = 0; j < 32 && n0 + j < N; ++j) crow[c * 32 + j] = pv[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
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
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace clt

// Returns 0 on success, a negative value when the arguments cannot be handled (the caller raises).
extern "C" int clt_encoder_gemm(const void* A, const void* B, const void* bias, void* C, int L, int M, int N, int K,
                                long long ldc, long long layer_stride_c, int* status, int num_sms, cudaStream_t stream) {
  using namespace clt;
  if (K % 8 != 0 || ldc % 8 != 0 || layer_stride_c % 8 != 0) return -1;  // 16-byte TMA strides / vector stores
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -2;
  CUtensorMap map_a, map_b;
  if (!make_kmajor_map(&map_a, A, L, M, K, K, 1LL * M * K, gemm::BM)) return -3;
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
      map_a, map_b, static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(C), L, M, N, K, ldc, layer_stride_c, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
