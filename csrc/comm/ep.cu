// Expert-parallel token exchange over symmetric memory (one process per GPU, NVLink peer
// loads / stores; no library collective on the path).
//
// Rank r owns experts [r * El, (r + 1) * El). Per MoE layer and direction:
//
//   pb_ep_layout    every rank reads all ranks' per-expert pair counts (peer loads) and
//                   derives, identically everywhere, each owner's receive layout: expert
//                   segments on 128-row boundaries, inside a segment the rows of source 0,
//                   then source 1, ... It emits the owner-side tables for the grouped GEMMs
//                   (segment offsets, row totals, padded lengths, expert of each 128-row block)
//                   and the sender-side table send_base[e] = first row of my pairs for expert e
//                   in its owner's buffer. Needing more rows than the buffers hold latches
//                   PB_EP_OVERFLOW in the status word and the excess pairs are dropped.
//   pb_ep_dispatch  push: every local (token, slot) row (x gate, in the backward) is stored
//                   straight into the owner's receive buffer (16-byte peer stores) and its
//                   (owner, row) is remembered
//   pb_ep_combine   pull: out[t] = sum_s gate[t, s] * ybuf_owner(t, s)[row(t, s)] by peer loads
//   pb_ep_rowdot / pb_ep_pull_scalar   gate gradient: the owner forms <y_row, dy_row>, the
//                   source reads it back and divides by the gate it scaled dy with
//
// Ordering between the phases is the caller's bounded device barrier (pb_barrier_all).
// Reference semantics: kernels/__init__.py ep_dispatch / ep_combine of the reference
// (token -> expert-owner exchange with stable ordering); the data path is this library's own.
#include "common.cuh"

#include <cuda_fp8.h>

namespace pb {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_E = 512;
constexpr int PB_EP_OVERFLOW = 4;

struct EpPeers {
  void* p[EP_MAX_RANKS];
};

// counts.p[s]: int [E] = pairs of source s per global expert. One block.
__global__ void ep_layout_kernel(EpPeers counts, int rank, int world, int E, int max_rows,
                                 int* __restrict__ expert_off,   // [El + 1]
                                 int* __restrict__ totals,       // [El]
                                 int* __restrict__ k_len,        // [El]
                                 int* __restrict__ mblk_group,   // [max_rows / 128]
                                 int* __restrict__ send_base,    // [E]
                                 int* __restrict__ blk_expect,   // [max_rows / 128] or null
                                 int* status) {
  __shared__ int tot[EP_MAX_E];      // pairs per expert over all sources
  __shared__ int before[EP_MAX_E];   // pairs of sources < rank
  __shared__ int seg[EP_MAX_E + 1];  // segment start of expert e inside its owner's buffer
  const int El = E / world;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < world; ++s) {
      const int c = __ldcv(static_cast<const int*>(counts.p[s]) + e);
      if (s < rank) b += c;
      t += c;
    }
    tot[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < world) {          // one thread per owner: aligned prefix over its experts
    const int q = threadIdx.x;
    int run = 0;
    for (int j = 0; j < El; ++j) {
      seg[q * El + j] = run;
      run += (tot[q * El + j] + 127) / 128 * 128;
    }
    if (q == rank) seg[E] = run;
    if (run > max_rows && status != nullptr) atomicCAS(status, 0, PB_EP_OVERFLOW);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) send_base[e] = seg[e] + before[e];
  const int mine = rank * El;
  const int used = min(seg[E], max_rows / 128 * 128);
  for (int j = threadIdx.x; j <= El; j += blockDim.x) {
    const int start = (j < El) ? seg[mine + j] : seg[E];
    expert_off[j] = min(start, used);
    if (j < El) {
      const int end = min(start + (tot[mine + j] + 127) / 128 * 128, used);
      totals[j] = max(0, min(tot[mine + j], used - min(start, used)));
      k_len[j] = max(0, end - min(start, used));
    }
  }
  for (int m = threadIdx.x; m < max_rows / 128; m += blockDim.x) {
    const int row = m * 128;
    int g = -1;
    if (row < used) {
      int lo = 0, hi = El;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg[mine + mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    mblk_group[m] = g;
    if (blk_expect != nullptr) {
      // rows of this block that senders will store (the rest is padding the owner zeroes)
      int want = 0;
      if (g >= 0) {
        const int start = seg[mine + g];
        const int valid_end = min(start + tot[mine + g], used);
        want = max(0, min(row + 128, valid_end) - row);
      }
      blk_expect[m] = want;
    }
  }
}

// One warp per local pair. local_off: my own 128-padded placement offsets (from the local
// stable sort), row_of_local its rows; dest row = send_base[e] + (row_of_local - local_off[e]).
__global__ void ep_dispatch_kernel(const bf16* __restrict__ src, long ld_src,
                                   const int* __restrict__ ids, const int* __restrict__ row_of_local,
                                   const int* __restrict__ local_off, const int* __restrict__ send_base,
                                   const float* __restrict__ scale, int n_pairs, int k, int d, int El,
                                   int max_rows, EpPeers xbuf, int* __restrict__ dest_rank,
                                   int* __restrict__ dest_row) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_pairs) return;
  const int e = ids[w];
  const int q = e / El;
  const int row = send_base[e] + (row_of_local[w] - local_off[e]);
  const bool ok = row < max_rows && PB_BOUNDS_OK(PB_K_EP_DISPATCH, q, EP_MAX_RANKS) &&
                  PB_BOUNDS_OK(PB_K_EP_DISPATCH, row, max_rows);
  if (lane == 0) {
    dest_rank[w] = q;
    dest_row[w] = ok ? row : -1;
  }
  if (!ok) return;
  const bf16* s = src + static_cast<size_t>(w / k) * ld_src;
  bf16* o = static_cast<bf16*>(xbuf.p[q]) + static_cast<size_t>(row) * d;
  const float g = scale ? scale[w] : 1.f;
  // eight 16-byte loads of the row in flight per lane before the first (possibly remote) store:
  // a 2048-wide row costs one memory latency instead of eight
  for (int c0 = lane * 8; c0 < d; c0 += 2048) {
    bf16x8 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (c0 + u * 256 < d) v[u] = *reinterpret_cast<const bf16x8*>(s + c0 + u * 256);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + u * 256 >= d) continue;
      if (scale) {
        float f[8];
        unpack8(v[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= g;
        v[u] = pack8(f);
      }
      *reinterpret_cast<bf16x8*>(o + c0 + u * 256) = v[u];
    }
  }
}

// four floats -> four e4m3 bytes (round to nearest even, saturating), little-endian
__device__ __forceinline__ uint32_t ep_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// FP8 on the wire: the sender quantises each row to e4m3 in 1 x 128 blocks (scale = amax / 448,
// 1 for an all-zero block; the same rule and rounding as the row quantiser of the FP8 GEMM) and
// stores 16 payload bytes per lane plus one fp32 scale per block straight into the owner's
// receive buffers: xq [max_rows, d] bytes and xs [d / 128, max_rows] floats, the layout the
// grouped FP8 GEMM reads. Half the NVLink bytes of a bf16 dispatch and no quantiser pass on
// the owner. One warp per local pair; a lane covers 16 consecutive elements, eight lanes a block.
__global__ void ep_dispatch_fp8_kernel(const bf16* __restrict__ src, long ld_src,
                                       const int* __restrict__ ids, const int* __restrict__ row_of_local,
                                       const int* __restrict__ local_off, const int* __restrict__ send_base,
                                       int n_pairs, int k, int d, int El, int max_rows, EpPeers xq,
                                       EpPeers xs, EpPeers arrived, int* __restrict__ dest_rank,
                                       int* __restrict__ dest_row) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_pairs) return;
  const int e = ids[w];
  const int q = e / El;
  const int row = send_base[e] + (row_of_local[w] - local_off[e]);
  const bool ok = row < max_rows;
  if (lane == 0) {
    dest_rank[w] = q;
    dest_row[w] = ok ? row : -1;
  }
  if (!ok) return;
  const bf16* s = src + static_cast<size_t>(w / k) * ld_src;
  uint8_t* oq = static_cast<uint8_t*>(xq.p[q]) + static_cast<size_t>(row) * d;
  float* os = static_cast<float*>(xs.p[q]);
  // Every lane runs every iteration (the shuffles below name the whole warp); lanes past the
  // end of a row narrower than 512 elements only take part in the shuffles. d is a multiple
  // of 128, so the eight lanes of a block are active or idle together.
  for (int c0 = 0; c0 < d; c0 += 512) {
    const int c = c0 + lane * 16;
    const bool active = c < d;
    float f[16];
    if (active) {
      unpack8(*reinterpret_cast<const bf16x8*>(s + c), f);
      unpack8(*reinterpret_cast<const bf16x8*>(s + c + 8), f + 8);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) f[j] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    if (!active) continue;
    const float scale = amax > 0.f ? amax / 448.f : 1.f;
    uint4 pk;
    pk.x = ep_e4m3x4(__fdiv_rn(f[0], scale), __fdiv_rn(f[1], scale), __fdiv_rn(f[2], scale), __fdiv_rn(f[3], scale));
    pk.y = ep_e4m3x4(__fdiv_rn(f[4], scale), __fdiv_rn(f[5], scale), __fdiv_rn(f[6], scale), __fdiv_rn(f[7], scale));
    pk.z = ep_e4m3x4(__fdiv_rn(f[8], scale), __fdiv_rn(f[9], scale), __fdiv_rn(f[10], scale), __fdiv_rn(f[11], scale));
    pk.w = ep_e4m3x4(__fdiv_rn(f[12], scale), __fdiv_rn(f[13], scale), __fdiv_rn(f[14], scale), __fdiv_rn(f[15], scale));
    *reinterpret_cast<uint4*>(oq + c) = pk;
    if ((lane & 7) == 0) os[static_cast<size_t>(c >> 7) * max_rows + row] = scale;
  }
  if (arrived.p[q] != nullptr) {
    // fused mode: tell the owner's GEMM that one more row of this 128-row block has landed.
    // Every lane's stores are ordered before the count (fence, warp barrier, then the add).
    __threadfence_system();
    __syncwarp();
    if (lane == 0) atomicAdd_system(static_cast<unsigned int*>(arrived.p[q]) + (row >> 7), 1u);
  }
}

// padding rows of the FP8 receive buffers: zero payload, unit scale (they dequantise to 0);
// one block per local expert
__global__ void ep_zero_pad_fp8_kernel(uint8_t* __restrict__ xq, float* __restrict__ xs, int d,
                                       int max_rows, const int* __restrict__ expert_off,
                                       const int* __restrict__ totals) {
  const int e = blockIdx.x;
  const int lo = expert_off[e] + totals[e], hi = expert_off[e + 1];
  const size_t n16 = static_cast<size_t>(hi - lo) * d / 16;
  uint4* p = reinterpret_cast<uint4*>(xq + static_cast<size_t>(lo) * d);
  for (size_t i = threadIdx.x; i < n16; i += blockDim.x) p[i] = make_uint4(0u, 0u, 0u, 0u);
  const int nkb = d / 128;
  for (int i = threadIdx.x; i < (hi - lo) * nkb; i += blockDim.x)
    xs[static_cast<size_t>(i / (hi - lo)) * max_rows + lo + i % (hi - lo)] = 1.f;
}

// out[t] = sum_s gate * ybuf[dest_rank][dest_row] (+ add[t]); one warp per token.
// The (rank, row, gate) of the token's k slots are read once; per 256-column step all k peer
// loads of a lane are issued before the first is used, so a warp has k x 16 bytes per lane in
// flight over NVLink instead of one load at a time (the pull is latency-bound otherwise).
constexpr int EP_MAX_K = 8;
__global__ void __launch_bounds__(256) ep_combine_kernel(EpPeers ybuf, const int* __restrict__ dest_rank,
                                                         const int* __restrict__ dest_row,
                                                         const float* __restrict__ gates,
                                                         const bf16* __restrict__ add, int T, int k, int d,
                                                         bf16* __restrict__ out) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  const bf16* src[EP_MAX_K];
  float g[EP_MAX_K];
#pragma unroll
  for (int s = 0; s < EP_MAX_K; ++s) {
    src[s] = nullptr;
    g[s] = 0.f;
    if (s < k) {
      const size_t i = static_cast<size_t>(t) * k + s;
      const int row = dest_row[i];
      const int q = dest_rank[i];
      if (row >= 0 && PB_BOUNDS_OK(PB_K_EP_COMBINE, q, EP_MAX_RANKS)) {
        src[s] = static_cast<const bf16*>(ybuf.p[q]) + static_cast<size_t>(row) * d;
        g[s] = gates ? gates[i] : 1.f;
      }
    }
  }
  for (int c = lane * 8; c < d; c += 256) {
    uint4 raw[EP_MAX_K];
#pragma unroll
    for (int s = 0; s < EP_MAX_K; ++s)
      if (src[s] != nullptr) raw[s] = __ldcv(reinterpret_cast<const uint4*>(src[s] + c));
    float acc[8];
    if (add != nullptr) unpack8(*reinterpret_cast<const bf16x8*>(add + static_cast<size_t>(t) * d + c), acc);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
#pragma unroll
    for (int s = 0; s < EP_MAX_K; ++s) {
      if (src[s] == nullptr) continue;
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(&raw[s]), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(g[s], f[j], acc[j]);
    }
    *reinterpret_cast<bf16x8*>(out + static_cast<size_t>(t) * d + c) = pack8(acc);
  }
}

// dot[r] = <a[r], b[r]> for r < *rows_used; one warp per row
__global__ void ep_rowdot_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b,
                                 const int* __restrict__ rows_used, int d, float* __restrict__ dot) {
  const int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (r >= *rows_used) return;
  float acc = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    float f[8], g[8];
    unpack8(*reinterpret_cast<const bf16x8*>(a + static_cast<size_t>(r) * d + c), f);
    unpack8(*reinterpret_cast<const bf16x8*>(b + static_cast<size_t>(r) * d + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(f[j], g[j], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) dot[r] = acc;
}

// out[i] = dotbuf[dest_rank[i]][dest_row[i]] / div[i]
__global__ void ep_pull_scalar_kernel(EpPeers dotbuf, const int* __restrict__ dest_rank,
                                      const int* __restrict__ dest_row, const float* __restrict__ div,
                                      int n, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int row = dest_row[i];
  float v = 0.f;
  if (row >= 0) {
    v = __ldcv(static_cast<const float*>(dotbuf.p[dest_rank[i]]) + row);
    const float g = div ? div[i] : 1.f;
    v = (fabsf(g) > 1e-20f) ? v / g : 0.f;
  }
  out[i] = v;
}

}  // namespace pb

using namespace pb;

static EpPeers make_peers(void* const* ptrs, int world) {
  EpPeers p;
  for (int i = 0; i < EP_MAX_RANKS; ++i) p.p[i] = i < world ? ptrs[i] : nullptr;
  return p;
}

// blk_expect (may be null): rows each 128-row block of this rank's receive buffer will get.
PB_API int pb_ep_layout(void* const* count_ptrs, int rank, int world, int E, int max_rows,
                        int* expert_off, int* totals, int* k_len, int* mblk_group, int* send_base,
                        int* blk_expect, int* status, cudaStream_t st) {
  if (world <= 0 || world > EP_MAX_RANKS || E <= 0 || E > EP_MAX_E || E % world != 0 ||
      max_rows % 128 != 0)
    return PB_BAD_ARG;
  ep_layout_kernel<<<1, 512, 0, st>>>(make_peers(count_ptrs, world), rank, world, E, max_rows,
                                      expert_off, totals, k_len, mblk_group, send_base, blk_expect,
                                      status);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_ep_dispatch(const void* src, long ld_src, const int* ids, const int* row_of_local,
                          const int* local_off, const int* send_base, const float* scale,
                          int n_pairs, int k, int d, int El, int max_rows, void* const* xbuf_ptrs,
                          int world, int* dest_rank, int* dest_row, cudaStream_t st) {
  if (n_pairs <= 0 || d % 8 != 0 || El <= 0) return PB_BAD_ARG;
  const int grid = static_cast<int>((static_cast<long>(n_pairs) * 32 + 255) / 256);
  ep_dispatch_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(src), ld_src, ids, row_of_local,
                                           local_off, send_base, scale, n_pairs, k, d, El, max_rows,
                                           make_peers(xbuf_ptrs, world), dest_rank, dest_row);
  return static_cast<int>(cudaGetLastError());
}

// The FP8-on-the-wire dispatch: xq_ptrs / xs_ptrs are every rank's receive buffers (e4m3 bytes
// [max_rows, d]; fp32 scales [d / 128, max_rows]). d a multiple of 128. arrived_ptrs (may be
// null): every rank's per-128-row-block arrival counters for the fused grouped GEMM
// (pb_gemm_fp8_grouped_arrive); with it no barrier is needed between dispatch and GEMM.
PB_API int pb_ep_dispatch_fp8(const void* src, long ld_src, const int* ids, const int* row_of_local,
                              const int* local_off, const int* send_base, int n_pairs, int k, int d,
                              int El, int max_rows, void* const* xq_ptrs, void* const* xs_ptrs,
                              void* const* arrived_ptrs, int world, int* dest_rank, int* dest_row,
                              cudaStream_t st) {
  if (n_pairs <= 0 || d % 128 != 0 || El <= 0 || (ld_src % 8) != 0) return PB_BAD_ARG;
  const int grid = static_cast<int>((static_cast<long>(n_pairs) * 32 + 255) / 256);
  EpPeers arr;
  for (int i = 0; i < EP_MAX_RANKS; ++i)
    arr.p[i] = (arrived_ptrs != nullptr && i < world) ? arrived_ptrs[i] : nullptr;
  ep_dispatch_fp8_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(src), ld_src, ids, row_of_local,
                                               local_off, send_base, n_pairs, k, d, El, max_rows,
                                               make_peers(xq_ptrs, world), make_peers(xs_ptrs, world),
                                               arr, dest_rank, dest_row);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_ep_zero_pad_fp8(void* xq, float* xs, int d, int max_rows, const int* expert_off,
                              const int* totals, int El, cudaStream_t st) {
  if (El <= 0 || d % 128 != 0) return PB_BAD_ARG;
  ep_zero_pad_fp8_kernel<<<El, 256, 0, st>>>(static_cast<uint8_t*>(xq), xs, d, max_rows, expert_off,
                                             totals);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_ep_combine(void* const* ybuf_ptrs, int world, const int* dest_rank,
                         const int* dest_row, const float* gates, const void* add, int T, int k, int d,
                         void* out, cudaStream_t st) {
  if (T <= 0 || d % 8 != 0 || k < 1 || k > EP_MAX_K) return PB_BAD_ARG;
  const int grid = static_cast<int>((static_cast<long>(T) * 32 + 255) / 256);
  ep_combine_kernel<<<grid, 256, 0, st>>>(make_peers(ybuf_ptrs, world), dest_rank, dest_row, gates,
                                          static_cast<const bf16*>(add), T, k, d,
                                          static_cast<bf16*>(out));
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_ep_rowdot(const void* a, const void* b, const int* rows_used, int max_rows, int d,
                        float* dot, cudaStream_t st) {
  if (max_rows <= 0 || d % 8 != 0) return PB_BAD_ARG;
  const int grid = static_cast<int>((static_cast<long>(max_rows) * 32 + 255) / 256);
  ep_rowdot_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(a), static_cast<const bf16*>(b),
                                         rows_used, d, dot);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_ep_pull_scalar(void* const* dot_ptrs, int world, const int* dest_rank,
                             const int* dest_row, const float* div, int n, float* out,
                             cudaStream_t st) {
  if (n <= 0) return PB_BAD_ARG;
  ep_pull_scalar_kernel<<<(n + 255) / 256, 256, 0, st>>>(make_peers(dot_ptrs, world), dest_rank,
                                                         dest_row, div, n, out);
  return static_cast<int>(cudaGetLastError());
}

PB_DEFINE_BOUNDS_READER(ep)
