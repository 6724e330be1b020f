// Shared device helpers for the sm_100a kernels: PTX wrappers for mbarrier / TMA /
// tcgen05, bounded waits, status codes and small math utilities.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---------------------------------------------------------------------------------------------------------
// 16-bit storage type of weights / activations.  Every translation unit is compiled twice: once for bf16
// (namespace clt, C symbols clt_*) and once with -DCLT_HALF for fp16 (namespace clt_h, C symbols clt_*_h),
// through one-line wrapper files that define CLT_HALF and include the .cu file.
#ifdef CLT_HALF
#define CLT_NS clt_h
#define CLT_FN(name) name##_h
#define CLT_T16_IS_HALF 1
#else
#define CLT_NS clt
#define CLT_FN(name) name
#define CLT_T16_IS_HALF 0
#endif
#define clt CLT_NS

namespace clt {

#if CLT_T16_IS_HALF
using t16 = __half;
using t16x2 = __half2;
constexpr float kT16Max = 65504.f;
#else
using t16 = __nv_bfloat16;
using t16x2 = __nv_bfloat162;
constexpr float kT16Max = 3.3895313892515355e38f;
#endif

// Status words written by kernels into a caller-provided int32 buffer.  The host reads
// them after the step; nothing traps or spins forever.
enum StatusCode : int {
  STATUS_OK = 0,
  STATUS_WAIT_TIMEOUT = 1,       // a bounded wait (mbarrier / peer flag) ran out
  STATUS_CAPACITY = 2,           // an output list did not fit its buffer
  STATUS_SELECT_RANGE = 3,       // threshold not inside the histogram range
  STATUS_TIE_OVERFLOW = 4,       // more ties at the cut than the tie buffer holds
  STATUS_BOUNDS = 5,             // debug build (-DCLT_DEBUG_BOUNDS): an index or peer offset was out of range; the access was skipped
};

// Index checks of the debug build.  Compute-sanitizer is not available everywhere these kernels run, so the build with
// -DCLT_DEBUG_BOUNDS checks the indices that come from data (entry lists, token ids, peer ranks and offsets) before they
// are used: a bad one records STATUS_BOUNDS, the site code and the offending value in the status words 0, 2 and 3 and the
// access is skipped - nothing traps and nothing is read or written out of range.  In the regular build the check
// compiles to `true`.
#ifdef CLT_DEBUG_BOUNDS
__device__ __forceinline__ bool clt_in_bounds(long long idx, long long limit, int* status, int site) {
  if (idx >= 0 && idx < limit) return true;
  if (status != nullptr && atomicCAS(status, STATUS_OK, STATUS_BOUNDS) == STATUS_OK) {
    status[2] = site;
    status[3] = int(idx);
  }
  return false;
}
#else
__device__ __forceinline__ bool clt_in_bounds(long long, long long, int*, int) { return true; }
#endif

// ~1 s at 2 GHz; every spin-wait in this library gives up after this many cycles.
constexpr long long kWaitTimeoutCycles = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the wait ran out or another role of the CTA already
// gave up (abort flag in shared memory); the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
    // a batch of polls between looks at the clock and the abort flag keeps the common case cheap
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kWaitTimeoutCycles) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// --------------------------------------------------------------------- TMA
// Tiled bulk tensor load, 3-D, no multicast: each CTA fetches its own tile.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Untiled bulk copy global -> shared (1-D), no multicast: both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// L2 eviction policies for streams that are touched once (evict_first) and for data that is re-read (evict_last).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_load_1d_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_store_1d_hint(void* gdst, const void* smem_src, uint32_t bytes, uint64_t policy) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
               ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_u32(smem_src)), "r"(bytes), "l"(policy)
               : "memory");
}
// Untiled bulk copy shared -> global, tracked by the issuing thread's bulk async-groups.
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's committed groups still have to read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
// Waits until all of this thread's committed groups are complete (writes performed).
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Tiled bulk tensor store shared -> global, 3-D (clipped at the tensor's bounds), tracked by bulk async-groups.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ----------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives row (lane base + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------- CTA pairs (cluster of two, tcgen05 cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load issued by either CTA of a pair into its own shared memory; the bytes are counted on the mbarrier
// at `mbar_cluster_addr` (the leader CTA's).  No multicast: every CTA fetches its own tile.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t mbar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(mbar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives on the barrier at this shared-memory offset in every CTA of `cta_mask` once the MMAs issued so far
// by this thread are complete.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}
// D (+)= A * B over a CTA pair: M = 256 (128 rows per CTA), each CTA holds its A rows and half of B's rows at
// the same shared-memory offsets; issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 tile whose rows are 128 bytes
// (64 elements) with the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version of this architecture
  d |= static_cast<uint64_t>(2) << 61;                      // layout type: 128-byte swizzle
  return d;
}
// Instruction descriptor: 16-bit x 16-bit -> fp32 (operand format 0 = fp16, 1 = bf16), both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(CLT_T16_IS_HALF ? 0 : 1) << 7) | (static_cast<uint32_t>(CLT_T16_IS_HALF ? 0 : 1) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
// Same with the A operand MN-major (bit 15) and / or the B operand MN-major (bit 16).
__host__ __device__ constexpr uint32_t umma_idesc_t16(int m, int n, int a_mn_major, int b_mn_major) {
  return umma_idesc_bf16(m, n) | (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16);
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ------------------------------------------------------------------- math
// real bf16 (optimizer moments may be bf16 whatever the weight type is)
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
// the build's 16-bit type
#if CLT_T16_IS_HALF
__device__ __forceinline__ uint32_t pack_t16x2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float t16_lo(uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu))); }
__device__ __forceinline__ float t16_hi(uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16))); }
__device__ __forceinline__ float t16_to_float(t16 v) { return __half2float(v); }
__device__ __forceinline__ t16 float_to_t16(float v) { return __float2half_rn(v); }
__device__ __forceinline__ t16 float_to_t16_rd(float v) { return __float2half_rd(v); }
__device__ __forceinline__ t16x2 make_t16x2(t16 a, t16 b) { return __halves2half2(a, b); }
// 0xFFFF in every half where a >= b (false for NaN)
__device__ __forceinline__ uint32_t t16x2_ge_mask(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("set.ge.u32.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
#else
__device__ __forceinline__ uint32_t pack_t16x2(float lo, float hi) { return pack_bf16x2(lo, hi); }
__device__ __forceinline__ float t16_lo(uint32_t v) { return bf16_lo(v); }
__device__ __forceinline__ float t16_hi(uint32_t v) { return bf16_hi(v); }
__device__ __forceinline__ float t16_to_float(t16 v) { return __bfloat162float(v); }
__device__ __forceinline__ t16 float_to_t16(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ t16 float_to_t16_rd(float v) { return __float2bfloat16_rd(v); }
__device__ __forceinline__ t16x2 make_t16x2(t16 a, t16 b) { return __halves2bfloat162(a, b); }
__device__ __forceinline__ uint32_t t16x2_ge_mask(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("set.ge.u32.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
#endif

// Monotone map float -> uint32 (larger float => larger key); NaN sorts above +inf.
__device__ __forceinline__ uint32_t float_to_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// ------------------------------------------------------------------- step control block
// 16 32-bit words in device memory that steer the optimizer kernels of a step without a host round trip.
// step_control_kernel (step.cu) fills it after the loss is known; every Adam kernel reads it.
enum StepCtl : int {
  SC_SKIP = 0,          // int: non-zero -> the optimizer kernels return without touching anything
  SC_INV_SCALE = 1,     // float: 1 / loss scale, multiplies every term derived from the gradient seed
  SC_LOSS_SCALE = 2,    // float: loss scale the gradient seed of this step is multiplied with (1 unless fp16)
  SC_GROWTH = 3,        // int: steps since the loss scale last changed
  SC_FOUND_INF = 4,     // int: set by the loss kernels when the gradient seed left the 16-bit range or is NaN
  SC_GRAD_NORM_SQ = 5,  // float: squared gradient norm gathered by the norm pre-pass (gradient clipping)
  SC_CLIP = 6,          // float: clip coefficient, multiplies every row gradient
  SC_SKIPPED = 7,       // int: number of skipped steps so far
  SC_SIZE = 16,
};
struct StepScales {
  float inv_scale, clip;
  bool skip;
};
__device__ __forceinline__ StepScales read_step_ctl(const float* ctl) {
  StepScales s;
  s.inv_scale = 1.f; s.clip = 1.f; s.skip = false;
  if (ctl != nullptr) {
    s.skip = __float_as_int(__ldg(ctl + SC_SKIP)) != 0;
    s.inv_scale = __ldg(ctl + SC_INV_SCALE);
    s.clip = __ldg(ctl + SC_CLIP);
  }
  return s;
}

// ------------------------------------------------------------------- cross-rank exchange of small vectors
constexpr int kMaxPeers = 8;
// peers[r] points at rank r's exchange area: [rounds][world][slot_elems] uint32 data plus one flag word per
// (round, source rank).  A round may be used once per launch sequence; `seq` grows with every step.
struct Exchange {
  int world;
  int rank;
  uint32_t* peers[kMaxPeers];
  uint32_t* flags[kMaxPeers];
  int slot_elems;
  uint32_t seq;
};
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// All-gather of `n` 32-bit words per rank (one CTA): every rank stores its words into slot [round][rank] of every
// peer, raises flag [round][rank] there and waits (bounded) for all peers' flags in its own area.  Afterwards rank
// q's words are at exchange_slot(ex, round, q).  Returns false on a timeout.  Because every rank waits for every
// other rank's flag, the call is also a barrier: all device work that a rank completed before its call (earlier
// kernels of the stream included) is visible to the ranks that return from theirs.
__device__ __forceinline__ const uint32_t* exchange_slot(const Exchange& ex, int round, int q) {
  return ex.peers[ex.rank] + (size_t(round) * ex.world + q) * ex.slot_elems;
}
__device__ __forceinline__ bool exchange_gather(const Exchange& ex, int round, const uint32_t* vals, int n, int* timeout_flag_smem) {
  if (ex.world <= 1) return true;
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int p = 0; p < ex.world; ++p) {
    uint32_t* dst = ex.peers[p] + (size_t(round) * ex.world + ex.rank) * ex.slot_elems;
    for (int i = tid; i < n; i += nt) dst[i] = vals[i];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < ex.world) st_release_sys(ex.flags[tid] + size_t(round) * ex.world + ex.rank, ex.seq);
  if (tid < ex.world) {
    const uint32_t* f = ex.flags[ex.rank] + size_t(round) * ex.world + tid;
    const long long start = clock64();
    while (ld_acquire_sys(f) != ex.seq) {
      if (clock64() - start > kWaitTimeoutCycles) { *timeout_flag_smem = 1; break; }
    }
  }
  __syncthreads();
  return *timeout_flag_smem == 0;
}

}  // namespace clt
