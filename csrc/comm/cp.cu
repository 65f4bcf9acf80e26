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

// ---------------------------------------------------------------------------------------
// Chain mode: the sequence is cut into 2 * world half-slices and rank r holds half-slices r and
// 2 * world - 1 - r (zig-zag), so that causal attention costs every rank the same. The state
// chain then visits 2 * world positions. Every rank stores both of its maps into EVERY rank's
// buffer at their chain positions,
//   maps[direction][which = P, R][row = b * heads + h][position][128 x 128]   at byte 256 + ...
// and raises its flag there; once all flags are up each rank folds the whole chain locally
// (pb_delta_compose over 2 * world maps) and keeps the two states it needs. Local map index:
// (b * 2 + half) * heads + h, i.e. the two half-slices of a sequence are batch entries.
// Chain flags live at byte 128 (uint32 [2][MAX_RANKS]), the push counters at byte 72.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float* chain_ptr(void* base, int dir, int which, int rows, int world,
                                            int row, int pos) {
  const size_t per_which = static_cast<size_t>(rows) * 2 * world * MAT;
  return reinterpret_cast<float*>(static_cast<uint8_t*>(base) + 256) +
         (static_cast<size_t>(dir) * 2 + which) * per_which +
         (static_cast<size_t>(row) * 2 * world + pos) * MAT;
}

__global__ void cp_push_chain_kernel(const float* __restrict__ P, const float* __restrict__ R,
                                     Peers peers, int rank, int world, int batch, int heads,
                                     int reverse, uint32_t epoch) {
  const int rows = batch * heads;
  const size_t per_map4 = MAT / 4;
  const size_t n4 = static_cast<size_t>(rows) * 2 * per_map4;      // float4 per tensor (P or R)
  for (int q = 0; q < world; ++q) {
    for (size_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      const int local = static_cast<int>(i / per_map4);              // (b * 2 + half) * heads + h
      const size_t within = i % per_map4;
      const int h = local % heads, bhalf = local / heads;
      const int half = bhalf & 1, b = bhalf >> 1;
      const int pos = half == 0 ? rank : 2 * world - 1 - rank;
      const int row = b * heads + h;
      reinterpret_cast<float4*>(chain_ptr(peers.p[q], reverse, 0, rows, world, row, pos))[within] =
          reinterpret_cast<const float4*>(P)[i];
      reinterpret_cast<float4*>(chain_ptr(peers.p[q], reverse, 1, rows, world, row, pos))[within] =
          reinterpret_cast<const float4*>(R)[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(peers.p[rank]) + 72) + reverse;
    const uint32_t prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;
      __threadfence_system();
      for (int q = 0; q < world; ++q) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(peers.p[q]) + 128) +
                         reverse * MAX_RANKS + rank;
        st_release_sys(flag, epoch);
      }
    }
  }
}

// Bounded wait for every rank's chain flag of this epoch; a timeout latches the status word.
__global__ void cp_wait_chain_kernel(void* local, int world, int reverse, uint32_t epoch,
                                     uint64_t budget_ns, int* status) {
  const uint32_t* flags = reinterpret_cast<const uint32_t*>(static_cast<uint8_t*>(local) + 128) +
                          reverse * MAX_RANKS;
  bool ok = true;
  for (int q = 0; q < world && ok; ++q) ok = wait_flag_ge(flags + q, epoch, budget_ns, status);
  __threadfence_system();
}

// ---------------------------------------------------------------------------------------
// Keys / values of a zig-zag split sequence. Every rank stages its two half-slices of K and V
// ([K half 0 | K half 1 | V half 0 | V half 1], half_bytes each) in symmetric memory; after a
// barrier each rank pulls all of them into its own natural-order K and V (plain 16-byte loads
// from the peers' memory, no library call), which the attention kernel then reads locally.
// The gradients come back the other way: every rank's attention backward leaves dK, dV for the
// whole prefix it saw in its own symmetric buffer ([dK | dV], full_elems bf16 each); the owner
// of a half-slice sums the peers' rows in rank order in fp32. Rank q has rows for chain position
// p iff p <= 2 * world - 1 - q.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
cp_kv_gather_kernel(Peers stage, uint4* __restrict__ k_dst, uint4* __restrict__ v_dst, int world,
                    size_t half16) {
  const size_t per_rank = 4 * half16;
  const size_t total = per_rank * world;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int q = static_cast<int>(i / per_rank);
    const size_t w = i % per_rank;
    const int part = static_cast<int>(w / half16);      // 0, 1: K halves; 2, 3: V halves
    const size_t off = w % half16;
    const int pos = (part & 1) == 0 ? q : 2 * world - 1 - q;
    const uint4 v = reinterpret_cast<const uint4*>(stage.p[q])[w];
    (part < 2 ? k_dst : v_dst)[static_cast<size_t>(pos) * half16 + off] = v;
  }
}

__global__ void __launch_bounds__(256)
cp_kv_reduce_kernel(Peers full, bf16* __restrict__ dk_out, bf16* __restrict__ dv_out, int rank,
                    int world, size_t half_elems, size_t full_elems) {
  const size_t half8 = half_elems / 8;
  const size_t total = 4 * half8;                        // dK half 0, dK half 1, dV half 0, dV half 1
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int part = static_cast<int>(i / half8);
    const size_t off = i % half8;
    const int half = part & 1, which = part >> 1;
    const int pos = half == 0 ? rank : 2 * world - 1 - rank;
    const int last = min(world - 1, 2 * world - 1 - pos);    // ranks 0 .. last hold these rows
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    bf16x8 v[MAX_RANKS];
#pragma unroll
    for (int q = 0; q < MAX_RANKS; ++q)
      if (q <= last)
        v[q] = reinterpret_cast<const bf16x8*>(static_cast<const bf16*>(full.p[q]) +
                                               which * full_elems + pos * half_elems)[off];
#pragma unroll
    for (int q = 0; q < MAX_RANKS; ++q)
      if (q <= last) {
        float f[8];
        unpack8(v[q], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    reinterpret_cast<bf16x8*>(which == 0 ? dk_out : dv_out)[static_cast<size_t>(half) * half8 + off] =
        pack8(acc);
  }
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

// ---- chain mode (zig-zag split) ----
PB_API long pb_cp_chain_bytes(int rows, int world) {
  return 256 + 2L * 2 * rows * 2 * world * cp::MAT * 4;
}

// P, R: fp32 [(batch * 2 + half) * heads + h][128][128]: this rank's two half-slices per sequence.
PB_API int pb_cp_push_chain(const void* P, const void* R, void* const* buf_ptrs, int rank, int world,
                            int batch, int heads, int reverse, int epoch, cudaStream_t st) {
  if (world < 1 || world > cp::MAX_RANKS || rank < 0 || rank >= world || batch <= 0 || heads <= 0 ||
      epoch <= 0)
    return PB_BAD_ARG;
  cp::cp_push_chain_kernel<<<96, 256, 0, st>>>(static_cast<const float*>(P), static_cast<const float*>(R),
                                               cp::make_peers(buf_ptrs, world), rank, world, batch,
                                               heads, reverse, static_cast<uint32_t>(epoch));
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_cp_wait_chain(void* local_buf, int world, int reverse, int epoch, long budget_ns,
                            int* status, cudaStream_t st) {
  if (world < 1 || world > cp::MAX_RANKS || epoch <= 0) return PB_BAD_ARG;
  cp::cp_wait_chain_kernel<<<1, 1, 0, st>>>(local_buf, world, reverse, static_cast<uint32_t>(epoch),
                                            static_cast<uint64_t>(budget_ns), status);
  return static_cast<int>(cudaGetLastError());
}

// stage_ptrs: every rank's staging buffer; half_bytes a multiple of 16.
PB_API int pb_cp_kv_gather(void* const* stage_ptrs, void* k_dst, void* v_dst, int world,
                           long half_bytes, cudaStream_t st) {
  if (world < 1 || world > cp::MAX_RANKS || half_bytes <= 0 || half_bytes % 16) return PB_BAD_ARG;
  cp::cp_kv_gather_kernel<<<148 * 4, 256, 0, st>>>(cp::make_peers(stage_ptrs, world),
                                                   static_cast<uint4*>(k_dst), static_cast<uint4*>(v_dst),
                                                   world, static_cast<size_t>(half_bytes / 16));
  return static_cast<int>(cudaGetLastError());
}

// full_ptrs: every rank's [dK | dV] buffer (full_elems bf16 each); dk_out / dv_out: bf16
// [2 halves][half_elems] of this rank.
PB_API int pb_cp_kv_reduce(void* const* full_ptrs, void* dk_out, void* dv_out, int rank, int world,
                           long half_elems, long full_elems, cudaStream_t st) {
  if (world < 1 || world > cp::MAX_RANKS || rank < 0 || rank >= world || half_elems <= 0 ||
      half_elems % 8 || full_elems < 2L * world * half_elems)
    return PB_BAD_ARG;
  cp::cp_kv_reduce_kernel<<<148 * 4, 256, 0, st>>>(cp::make_peers(full_ptrs, world),
                                                   static_cast<bf16*>(dk_out), static_cast<bf16*>(dv_out),
                                                   rank, world, static_cast<size_t>(half_elems),
                                                   static_cast<size_t>(full_elems));
  return static_cast<int>(cudaGetLastError());
}
