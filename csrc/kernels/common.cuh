// Shared device helpers for the sm_100a kernels: vector loads, warp/block
// reductions, mbarrier / TMA / tcgen05 PTX wrappers, bounded waits.
//
// Every spin-wait in this library is bounded: a wait that does not finish
// within its budget records a code in a status word and the kernel drains and
// returns instead of spinning forever.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PB_API extern "C" __attribute__((visibility("default")))

namespace pb {

// One-time launcher set-up keyed by device. cudaFuncSetAttribute (the opt-in to more than
// 48 KB of dynamic shared memory) and occupancy queries apply to the device that is current
// when they are made, and one process may drive several GPUs, so a plain `static bool` would
// leave every device after the first without the attribute. Usage:
//   static DeviceOnce once;  if (once.need()) { ...set-up...; once.done(); }
// Host threads may race on the first call of a device: the set-up is idempotent, the bits are
// set with atomic read-modify-write builtins.
struct DeviceOnce {
  unsigned long long bits[4] = {0ull, 0ull, 0ull, 0ull};   // up to 256 device ordinals
  static int current() {
    int dev = 0;
    cudaGetDevice(&dev);
    return dev < 0 ? 0 : (dev & 255);
  }
  bool need() const {
    const int d = current();
    return ((__atomic_load_n(&bits[d >> 6], __ATOMIC_ACQUIRE) >> (d & 63)) & 1ull) == 0ull;
  }
  void done() {
    const int d = current();
    __atomic_fetch_or(&bits[d >> 6], 1ull << (d & 63), __ATOMIC_RELEASE);
  }
};

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ---------------------------------------------------------------------------
// status codes written by kernels that gave up on a bounded wait
// ---------------------------------------------------------------------------
enum : int {
  PB_OK = 0,
  PB_TIMEOUT_MBAR = 1,   // an mbarrier phase never completed
  PB_TIMEOUT_FLAG = 2,   // a peer / host flag never reached its value
  PB_BAD_ARG = 3,
};

// ---------------------------------------------------------------------------
// Debug bounds checks (the -DPB_DEBUG_BOUNDS build of the library).
//
// Indices that come from data (a target token, a routed row, a peer rank, a sequence position)
// are checked before the access they feed: the first violation of a launch records
// (kernel id, index, limit) in a device-side record and the access is skipped, so the kernel
// finishes and the context stays usable. The host reads and clears the record with
// pb_debug_bounds_read. In the normal build PB_BOUNDS_OK() is the constant `true`.
// ---------------------------------------------------------------------------
enum : int {
  PB_K_SOFTCAP_CE = 1, PB_K_MOE_PERMUTE = 2, PB_K_MOE_COMBINE = 3, PB_K_MOE_COMBINE_BWD = 4,
  PB_K_EP_DISPATCH = 5, PB_K_EP_COMBINE = 6, PB_K_ROPE = 7, PB_K_LATENT = 8, PB_K_EP_PULL = 9,
};
#ifdef PB_DEBUG_BOUNDS
struct BoundsRecord {
  int kernel, hits;
  long long index, limit;
};
// one record per translation unit (no relocatable device code in this build); every file that
// checks exports a reader with PB_DEFINE_BOUNDS_READER and the host polls them all
static __device__ BoundsRecord g_bounds_record = {0, 0, 0, 0};
static inline int bounds_read_tu(long long* out4) {
  BoundsRecord r;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyFromSymbol(&r, g_bounds_record, sizeof(r));
  if (e != cudaSuccess) return static_cast<int>(e);
  out4[0] = r.kernel; out4[1] = r.hits; out4[2] = r.index; out4[3] = r.limit;
  const BoundsRecord z = {0, 0, 0, 0};
  return static_cast<int>(cudaMemcpyToSymbol(g_bounds_record, &z, sizeof(z)));
}
#define PB_DEFINE_BOUNDS_READER(tu) \
  PB_API int pb_debug_bounds_read_##tu(long long* out4) { return ::pb::bounds_read_tu(out4); }
__device__ __forceinline__ bool bounds_ok(int kernel, long long index, long long limit) {
  if (index >= 0 && index < limit) return true;
  if (atomicAdd(&g_bounds_record.hits, 1) == 0) {
    g_bounds_record.kernel = kernel;
    g_bounds_record.index = index;
    g_bounds_record.limit = limit;
  }
  return false;
}
#define PB_BOUNDS_OK(kernel, index, limit) (::pb::bounds_ok((kernel), (index), (limit)))
#else
#define PB_BOUNDS_OK(kernel, index, limit) (true)
#define PB_DEFINE_BOUNDS_READER(tu)
#endif

// ---------------------------------------------------------------------------
// small math / packing helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_to_f32(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ bf16 f32_to_bf16(float x) { return __float2bfloat16_rn(x); }

struct alignas(16) bf16x8 {
  bf162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `scratch` must hold 33 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ---------------------------------------------------------------------------
// shared-memory address / mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Iteration budget of one bounded mbarrier wait. try_wait itself blocks for a
// hardware-defined slice (order of a microsecond), so this is seconds at most.
#ifndef PB_MBAR_SPIN_LIMIT
#define PB_MBAR_SPIN_LIMIT (1u << 22)
#endif

// Bounded wait. Returns false (and latches *status) if the budget ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
  for (uint32_t it = 0; it < PB_MBAR_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && status != nullptr &&
        *reinterpret_cast<volatile int*>(status) != PB_OK)
      return false;  // someone else already gave up: drain fast
  }
  if (status != nullptr) atomicCAS(status, PB_OK, PB_TIMEOUT_MBAR);
  return false;
}

// Same contract with the non-blocking probe: test_wait returns at once, so a waiter notices
// the phase flip within a few cycles instead of after try_wait's suspend slice. For the short
// dependent hops of a latency chain (softmax rows <-> MMA issue); keep try_wait where the wait
// is long and the warp should stay out of the issue slots.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
#ifndef PB_MBAR_TEST_LIMIT
#define PB_MBAR_TEST_LIMIT (1u << 27)
#endif
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, int* status) {
  for (uint32_t it = 0; it < PB_MBAR_TEST_LIMIT; ++it) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((it & 0xFFFFu) == 0xFFFFu && status != nullptr &&
        *reinterpret_cast<volatile int*>(status) != PB_OK)
      return false;
  }
  if (status != nullptr) atomicCAS(status, PB_OK, PB_TIMEOUT_MBAR);
  return false;
}

// ---------------------------------------------------------------------------
// TMA (tiled bulk tensor copies), no cluster multicast anywhere
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const void* tmap, const void* smem_src, int32_t x,
                                             int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* smem_src, int32_t x,
                                             int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(tmap)),
      "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// L2 policy for data that is written once and not read again by this kernel (output tiles):
// its lines are the first to go, so they do not push the operand panels out of the cache.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_store_3d_hint(const void* tmap, const void* smem_src, int32_t x,
                                                  int32_t y, int32_t z, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], "
      "[%1], %5;" ::"l"(reinterpret_cast<uint64_t>(tmap)),
      "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05 (5th-gen tensor cores, accumulators in tensor memory)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the whole CTA.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same for 8-bit float operands (e4m3/e5m2), fp32 accumulate.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from tensor memory (bf16 packed), B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Make the mbarrier track completion of all MMAs issued so far by this thread.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// ---------------------------------------------------------------------------
// CTA pairs (cta_group::2): two CTAs of a cluster run one 256-row MMA, each holding half of the
// rows of A and of the accumulator and half of the columns of B. The even CTA issues the MMAs.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_smem_addr` in CTA `cta` of this cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// Bounded wait that also acquires what CTAs of the whole cluster released before arriving.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int* status) {
  for (uint32_t it = 0; it < PB_MBAR_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 1023u) == 1023u && status != nullptr &&
        *reinterpret_cast<volatile int*>(status) != PB_OK)
      return false;
  }
  if (status != nullptr) atomicCAS(status, PB_OK, PB_TIMEOUT_MBAR);
  return false;
}
// Tile load of a CTA pair: the bytes land in this CTA's shared memory, the completion is
// counted on the barrier at `bar_cluster_addr`, which may live in the peer CTA.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const void* tmap,
                                                 uint32_t bar_cluster_addr, int32_t x, int32_t y,
                                                 int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Completion of the pair's MMAs issued so far arrives on the barrier at the same shared-memory
// offset in every CTA of `cta_mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane
// (taddr.lane + t), columns taddr.col .. +31.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Instruction descriptor, kind::f16 / kind::f8f6f4, dense, fp32 accumulate.
//   [4,6) D format (1 = f32)   [7,10) A format   [10,13) B format
//   bit 15 A is MN-major       bit 16 B is MN-major
//   [17,23) N >> 3             [24,29) M >> 4
// kind::f16 formats: 0 = f16, 1 = bf16.  kind::f8f6f4: 0 = e4m3, 1 = e5m2.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt_a, uint32_t fmt_b, uint32_t M,
                                                  uint32_t N, uint32_t a_mn_major,
                                                  uint32_t b_mn_major) {
  return (1u << 4) | (fmt_a << 7) | (fmt_b << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile.
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1   [61,64) swizzle (2 = 128B)
__device__ __forceinline__ uint64_t make_sdesc_sw128(uint32_t saddr, uint32_t lbo_bytes,
                                                     uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// The same descriptor split into its two 32-bit words. Only the low word (start address,
// leading byte offset) changes between the MMAs of a tile, and only by a constant, so an
// issuing thread that keeps `lo` in a register spends one add per operand per MMA:
//   lo' = lo + (byte_offset >> 4)      (valid inside the 256 KB shared-memory window)
__device__ __forceinline__ uint32_t sdesc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t sdesc_hi_sw128(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ void umma_f16_words(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi,
                                               uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Pair form of umma_f16_words (cta_group::2, issued by the even CTA).
__device__ __forceinline__ void umma_f16_pair_words(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi,
                                                    uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                    uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------------------
// system-scope flags for peer / host signalling
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Wait until *flag >= want or `budget_ns` elapsed. Returns false on time-out.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want,
                                             uint64_t budget_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (ld_acquire_sys(flag) < want) {
    if ((++it & 63u) == 0) {
      if (globaltimer_ns() - t0 > budget_ns) {
        if (status != nullptr) atomicCAS(status, PB_OK, PB_TIMEOUT_FLAG);
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}

}  // namespace pb
