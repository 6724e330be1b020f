// Tensor-parallel data plane over peer memory (NVLink 5 / NVSwitch), sm_100a.
//
// The reference sums every (source, target) decoder output with an NCCL all-reduce - 78 of them per forward
// for a 12-layer model - and gathers full activations with all_gather (clt/models/parallel.py:143,197).
// Here the cross-rank traffic of a training step is two pushes through symmetric memory:
//
//   1. the sparse decode kernel stores each token's partial reconstruction straight into the staging slot of
//      the rank that owns the token (reduce-scatter by push, overlapped with the decode itself);
//   2. owner_reduce_loss_kernel sums the W staged slots of its tokens, adds the bias, forms the residual, the
//      squared-error sums and the bf16 gradient seed, and stores the seed rows into every peer's buffer
//      (all-gather by push, bf16 instead of fp32).
//
// peer_barrier_kernel orders the two phases across GPUs: release-store of a sequence number into every peer's
// flag word, then a bounded acquire-spin on the own flag words.  A wait that runs out records
// STATUS_WAIT_TIMEOUT and returns; nothing spins forever.  Plain peer loads/stores only (no multicast loads).
#include "common.cuh"

namespace clt {

constexpr int kMaxRanks = 8;

struct PeerTable {
  int world;
  int rank;
  void* ptr[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags[r] points at rank r's flag array [slots][world]; every rank writes `seq` into slot/rank position of
// every peer and waits until all peers wrote theirs.  One CTA of at least `world` threads.
// `timeout_cycles`: the phase barriers of the training step use kWaitTimeoutCycles (the ranks reach them within
// microseconds of one another); the staging barriers wait for a peer's data loader and are given a longer limit.
__global__ void peer_barrier_kernel(PeerTable flags, int slot, uint32_t seq, int* __restrict__ status, long long timeout_cycles) {
  const int tid = threadIdx.x;
  __threadfence_system();
  if (tid < flags.world) {
    uint32_t* dst = static_cast<uint32_t*>(flags.ptr[tid]) + slot * flags.world + flags.rank;
    st_release_sys_u32(dst, seq);
    const uint32_t* mine = static_cast<const uint32_t*>(flags.ptr[flags.rank]) + slot * flags.world + tid;
    const long long start = clock64();
    while (ld_acquire_sys_u32(mine) != seq) {
      if (clock64() - start > timeout_cycles) {
        atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __threadfence_system();
}

// stage: this rank's staging area [world][L][rows_per_rank][d] fp32 (slot w = partial sums pushed by rank w).
// gs_peers[q]: rank q's gradient-seed buffer [L][B][d] bf16.  This rank owns token rows
// [rank * rows_per_rank, ...).  grid = (blocks, L).
__global__ void __launch_bounds__(256) owner_reduce_loss_kernel(const float* __restrict__ stage, PeerTable gs_peers,
                                                                  const float* __restrict__ bias_sum,
                                                                  const float* __restrict__ addend,
                                                                  const t16* __restrict__ target,
                                                                  const float* __restrict__ sigma, float* __restrict__ yhat_out,
                                                                  double* __restrict__ sq_err, int L, int B, int d,
                                                                  int rows_per_rank, float* __restrict__ ctl) {
  const int t = blockIdx.y;
  const float loss_scale = ctl != nullptr ? ctl[SC_LOSS_SCALE] : 1.f;
  bool bad = false;
  const int world = gs_peers.world, rank = gs_peers.rank;
  const int row_base = rank * rows_per_rank;
  const int nrows = max(0, min(rows_per_rank, B - row_base));
  const int vec_per_row = d / 8;
  const long long nvec = 1LL * nrows * vec_per_row;
  const long long slot_stride = 1LL * L * rows_per_rank * d;
  float sq = 0.f;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < nvec; i += 1LL * gridDim.x * blockDim.x) {
    const int lrow = int(i / vec_per_row);
    const int e0 = int(i - 1LL * lrow * vec_per_row) * 8;
    const long long soff = (1LL * t * rows_per_rank + lrow) * d + e0;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    for (int w = 0; w < world; ++w) {
      const float4 a0 = __ldcs(reinterpret_cast<const float4*>(stage + w * slot_stride + soff));
      const float4 a1 = __ldcs(reinterpret_cast<const float4*>(stage + w * slot_stride + soff) + 1);
      v[0] += a0.x; v[1] += a0.y; v[2] += a0.z; v[3] += a0.w; v[4] += a1.x; v[5] += a1.y; v[6] += a1.z; v[7] += a1.w;
    }
    const int row = row_base + lrow;
    const long long off = (1LL * t * B + row) * d + e0;
    const uint4 tv = *reinterpret_cast<const uint4*>(target + off);
    const uint32_t u[4] = {tv.x, tv.y, tv.z, tv.w};
    float g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] += bias_sum[1LL * t * d + e0 + j];
      if (addend) v[j] += addend[off + j];
      const float y = (j & 1) ? t16_hi(u[j >> 1]) : t16_lo(u[j >> 1]);
      const float sg = sigma ? sigma[1LL * t * d + e0 + j] : 1.f;
      const float r = (v[j] - y) * sg;
      sq = fmaf(r, r, sq);
      g[j] = r * sg * loss_scale;
      bad |= !(fabsf(g[j]) <= kT16Max);
    }
    uint4 gv;
    gv.x = pack_t16x2(g[0], g[1]); gv.y = pack_t16x2(g[2], g[3]); gv.z = pack_t16x2(g[4], g[5]); gv.w = pack_t16x2(g[6], g[7]);
    for (int q = 0; q < world; ++q)  // all-gather by push: the seed rows land in every rank's buffer
      *reinterpret_cast<uint4*>(static_cast<t16*>(gs_peers.ptr[q]) + off) = gv;
    if (yhat_out) {
      float4* dst = reinterpret_cast<float4*>(yhat_out + off);
      dst[0] = make_float4(v[0], v[1], v[2], v[3]);
      dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  __shared__ float red[8];
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
    if (tot != 0.f) atomicAdd(&sq_err[t], double(tot));
  }
  if (bad && ctl != nullptr) atomicOr(reinterpret_cast<int*>(ctl) + SC_FOUND_INF, 1);
}

}  // namespace clt

using namespace clt;

struct CltPeerTable {
  int world;
  int rank;
  void* ptr[8];
};
static PeerTable to_table(const CltPeerTable* a) {
  PeerTable t;
  t.world = a->world; t.rank = a->rank;
  for (int i = 0; i < kMaxRanks; ++i) t.ptr[i] = a->ptr[i];
  return t;
}

#if !CLT_T16_IS_HALF
extern "C" int clt_peer_barrier(const CltPeerTable* flags, int slot, unsigned int seq, int* status, long long timeout_cycles,
                                cudaStream_t st) {
  if (flags->world <= 1) return 0;
  peer_barrier_kernel<<<1, 32, 0, st>>>(to_table(flags), slot, seq, status, timeout_cycles > 0 ? timeout_cycles : kWaitTimeoutCycles);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#endif

extern "C" int CLT_FN(clt_owner_reduce_loss)(const float* stage, const CltPeerTable* gs_peers, const float* bias_sum, const float* addend,
                                     const void* target, const float* sigma, float* yhat_out, double* sq_err, int L, int B, int d,
                                     int rows_per_rank, float* ctl, cudaStream_t st) {
  if (d % 8 != 0) return -1;
  dim3 grid(148, L);
  owner_reduce_loss_kernel<<<grid, 256, 0, st>>>(stage, to_table(gs_peers), bias_sum, addend, static_cast<const t16*>(target),
                                                 sigma, yhat_out, sq_err, L, B, d, rows_per_rank, ctl);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
