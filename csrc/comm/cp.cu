// Context-parallel delta-rule state hand-off over peer memory.
//
// A rank that holds one slice of a long sequence summarises it, per (batch, head), as an affine
// map of the 128 x 128 fp32 state:  S_out = P S_in + R.  The state entering rank r is the
// composition of the maps of ranks 0..r-1 (forward), and the state gradient leaving rank r is
// the composition of the transposed maps of ranks N-1..r+1 (backward):
//
//   forward   S = S0;   for q = 0 .. r-1:     S = P_q S + R_q
//   backward  G = 0;    for q = N-1 .. r+1:   G = P_q^T G + R_q     (R_q then holds the local
//                                                                    state gradient)
//
// pb_cp_push stores this rank's (P, R) into slot [rank] of every rank that needs it (plain
// peer stores over NVLink), fences, and the last CTA to finish raises this rank's flag on those
// peers. pb_cp_compose waits (bounded) for the flags of the ranks it depends on and composes the
// prefix in fp32 on the CUDA cores, one CTA per (batch, head). No collective library call and no
// host round trip sits between a rank's local scan and the scan with the true incoming state.
//
// Reference: parallel/context.py delta-state hand-off of the reference (host-side gather +
// compose); the peer-memory protocol is this library's own.
#include "common.cuh"

namespace pb {
namespace cp {

constexpr int D = 128;
constexpr int MAT = D * D;          // floats per matrix
constexpr int MAX_RANKS = 8;

struct Peers {
  void* p[MAX_RANKS];
};

// Layout of each rank's symmetric buffer:
//   uint32 flags[2][MAX_RANKS]  (direction, source rank)            at byte 0   (64 bytes used)
//   uint32 done_counter[2]                                          at byte 64
//   float  slots[MAX_RANKS][2][bh][MAT]                             at byte 256
__device__ __forceinline__ float* slot_ptr(void* base, int src, int which, int bh_count, int bh) {
  return reinterpret_cast<float*>(static_cast<uint8_t*>(base) + 256) +
         ((static_cast<size_t>(src) * 2 + which) * bh_count + bh) * MAT;
}

__global__ void cp_push_kernel(const float* __restrict__ P, const float* __restrict__ R, Peers peers,
                               int rank, int world, int bh_count, int reverse, uint32_t epoch) {
  const size_t n4 = static_cast<size_t>(bh_count) * MAT / 4;
  const int lo = reverse ? 0 : rank + 1, hi = reverse ? rank : world;   // target ranks [lo, hi)
  for (int q = lo; q < hi; ++q) {
    float4* dp = reinterpret_cast<float4*>(slot_ptr(peers.p[q], rank, 0, bh_count, 0));
    float4* dr = reinterpret_cast<float4*>(slot_ptr(peers.p[q], rank, 1, bh_count, 0));
    const float4* sp = reinterpret_cast<const float4*>(P);
    const float4* sr = reinterpret_cast<const float4*>(R);
    for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      dp[i] = sp[i];
      dr[i] = sr[i];
    }
  }
  // every store of this CTA is visible system-wide before the CTA counts itself done
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(peers.p[rank]) + 64) + reverse;
    const uint32_t prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;   // ready for the next push on this stream
      __threadfence_system();
      for (int q = lo; q < hi; ++q) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(peers.p[q]) + reverse * MAX_RANKS + rank;
        st_release_sys(flag, epoch);
      }
    }
  }
}

// One CTA per (batch, head), 256 threads, each owning an 8 x 8 block of the state.
// Shared memory: the state (64 KB) and the current P (64 KB).
__global__ void __launch_bounds__(256, 1)
cp_compose_kernel(void* local, const float* __restrict__ s0, float* __restrict__ out, int rank,
                  int world, int bh_count, int reverse, uint32_t epoch, uint64_t budget_ns,
                  int* status) {
  extern __shared__ float smem[];
  float* st = smem;           // [D][D] state, row-major
  float* pm = smem + MAT;     // [D][D] current P (row-major; read transposed when reverse)
  __shared__ int ok_flag;
  const int bh = blockIdx.x;
  const int first = reverse ? world - 1 : 0, last = reverse ? rank + 1 : rank - 1, step = reverse ? -1 : 1;
  const int n_src = reverse ? world - 1 - rank : rank;
  if (threadIdx.x == 0) {
    bool ok = true;
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(local) + reverse * MAX_RANKS;
    for (int i = 0, q = first; i < n_src && ok; ++i, q += step)
      ok = wait_flag_ge(flags + q, epoch, budget_ns, status);
    ok_flag = ok ? 1 : 0;
  }
  __syncthreads();
  if (!ok_flag) return;   // status is latched; the output is left untouched

  const int tr = (threadIdx.x >> 4) * 8, tc = (threadIdx.x & 15) * 8;   // this thread's 8 x 8 block
  for (int i = threadIdx.x; i < MAT / 4; i += 256)
    reinterpret_cast<float4*>(st)[i] =
        s0 != nullptr ? reinterpret_cast<const float4*>(s0 + static_cast<size_t>(bh) * MAT)[i]
                      : make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();
  for (int i = 0, q = first; i < n_src; ++i, q += step) {
    const float* Pq = slot_ptr(local, q, 0, bh_count, bh);
    const float* Rq = slot_ptr(local, q, 1, bh_count, bh);
    for (int j = threadIdx.x; j < MAT / 4; j += 256)
      reinterpret_cast<float4*>(pm)[j] = reinterpret_cast<const float4*>(Pq)[j];
    __syncthreads();
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
      for (int b = 0; b < 8; ++b) acc[a][b] = Rq[(tr + a) * D + tc + b];
    for (int k = 0; k < D; ++k) {
      float pa[8], sb[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) pa[a] = reverse ? pm[k * D + tr + a] : pm[(tr + a) * D + k];
#pragma unroll
      for (int b = 0; b < 8; ++b) sb[b] = st[k * D + tc + b];
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = fmaf(pa[a], sb[b], acc[a][b]);
    }
    __syncthreads();   // everyone has finished reading the old state
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
      for (int b = 0; b < 8; ++b) st[(tr + a) * D + tc + b] = acc[a][b];
    __syncthreads();
  }
  for (int i = threadIdx.x; i < MAT / 4; i += 256)
    reinterpret_cast<float4*>(out + static_cast<size_t>(bh) * MAT)[i] = reinterpret_cast<float4*>(st)[i];
}

static Peers make_peers(void* const* ptrs, int world) {
  Peers p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < world ? ptrs[i] : nullptr;
  return p;
}

}  // namespace cp
}  // namespace pb

using namespace pb;

// Bytes of symmetric memory each rank needs for `bh` (batch x head) states.
PB_API long pb_cp_buffer_bytes(int bh) {
  return 256 + static_cast<long>(cp::MAX_RANKS) * 2 * bh * cp::MAT * 4;
}

// Publish this rank's (P, R), fp32 [bh, 128, 128] each, to the ranks after it (reverse = 0) or
// before it (reverse = 1). `epoch` must grow by one per call and direction.
PB_API int pb_cp_push(const void* P, const void* R, void* const* buf_ptrs, int rank, int world, int bh,
                      int reverse, int epoch, cudaStream_t st) {
  if (world < 1 || world > cp::MAX_RANKS || rank < 0 || rank >= world || bh <= 0 || epoch <= 0)
    return PB_BAD_ARG;
  const int targets = reverse ? rank : world - 1 - rank;
  if (targets == 0) return 0;
  const int grid = 64;
  cp::cp_push_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(P), static_cast<const float*>(R),
                                           cp::make_peers(buf_ptrs, world), rank, world, bh, reverse,
                                           static_cast<uint32_t>(epoch));
  return static_cast<int>(cudaGetLastError());
}

// out [bh, 128, 128] = composition of the maps this rank depends on, applied to s0 (or zero).
// Waits at most budget_ns for each source rank's flag to reach `epoch`; on expiry *status is set
// to PB_TIMEOUT_FLAG and `out` is not written.
PB_API int pb_cp_compose(void* local_buf, const void* s0, void* out, int rank, int world, int bh,
                         int reverse, int epoch, long budget_ns, int* status, cudaStream_t st) {
  if (world < 1 || world > cp::MAX_RANKS || rank < 0 || rank >= world || bh <= 0 || epoch <= 0)
    return PB_BAD_ARG;
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  const int smem = 2 * cp::MAT * 4;
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(cp::cp_compose_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  cp::cp_compose_kernel<<<bh, 256, smem, st>>>(local_buf, static_cast<const float*>(s0),
                                               static_cast<float*>(out), rank, world, bh, reverse,
                                               static_cast<uint32_t>(epoch),
                                               static_cast<uint64_t>(budget_ns), status);
  return static_cast<int>(cudaGetLastError());
}
