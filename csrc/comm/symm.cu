// Symmetric memory over CUDA IPC and the fused compute+collective kernels that
// run on it (one process per GPU, every rank holds every peer's base pointer).
//
//   pb_barrier_all           device-side barrier over peer flags, bounded wait
//   pb_reduce_to_owner       gradient reduce-scatter by ownership: the owner reads
//                            every rank's fp32 gradient slice over NVLink, folds them
//                            in rank order (fp32 left fold: bitwise reproducible, the
//                            determinism contract of parallel/fsdp.py:161-190 in the
//                            reference), writes the sum locally and emits its
//                            sum-of-squares partials for the global-norm clip
//   pb_publish_scalar / pb_sum_slots   all-gather + ordered sum of one float per rank
//   pb_adamw_bcast / pb_muon_apply_bcast   optimizer update fused with the parameter
//                            all-gather: the refreshed bf16 weights are stored
//                            straight into every peer's working copy (16-byte P2P
//                            stores), no separate collective
//
// Peer traffic is plain loads/stores on peer pointers. No TMA from peer memory, no
// multicast. Flags use release/acquire at system scope; every wait is bounded.
#include "common.cuh"

namespace pb {

constexpr int MAX_RANKS = 8;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

// flags layout on every rank: uint32 [slots][MAX_RANKS]; slot s, entry r = last epoch
// at which rank r arrived at barrier slot s.
__global__ void barrier_all_kernel(PeerPtrs flags, int rank, int world, int slot, uint32_t epoch,
                                   uint64_t budget_ns, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    uint32_t* peer = static_cast<uint32_t*>(flags.p[t]) + slot * MAX_RANKS + rank;
    st_release_sys(peer, epoch);
    const uint32_t* mine = static_cast<const uint32_t*>(flags.p[rank]) + slot * MAX_RANKS + t;
    wait_flag_ge(mine, epoch, budget_ns, status);
    __threadfence_system();
  }
}

// W > 0: the number of ranks is a compile-time constant, so the W loads of an element are all in
// flight before the first add (the fold itself stays in rank order). W == 0: any rank count.
template <int W>
__global__ void __launch_bounds__(256) reduce_to_owner_kernel(PeerPtrs grads, long lo, long n,
                                                              int world, float* __restrict__ out,
                                                              float* __restrict__ partial) {
  __shared__ float scratch[33];
  float ss = 0.f;
  const long n4 = n >> 2;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 acc;
    if (W > 0) {
      float4 v[W > 0 ? W : 1];
#pragma unroll
      for (int r = 0; r < W; ++r)
        v[r] = __ldcv(reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + lo) + i);
      acc = v[0];
#pragma unroll
      for (int r = 1; r < W; ++r) {
        acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
      }
    } else {
      acc = __ldcv(reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[0]) + lo) + i);
      for (int r = 1; r < world; ++r) {
        const float4 v =
            __ldcv(reinterpret_cast<const float4*>(static_cast<const float*>(grads.p[r]) + lo) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    reinterpret_cast<float4*>(out + lo)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (blockIdx.x == 0) {
    for (long i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) {
      float acc = __ldcv(static_cast<const float*>(grads.p[0]) + lo + i);
      for (int r = 1; r < world; ++r) acc += __ldcv(static_cast<const float*>(grads.p[r]) + lo + i);
      out[lo + i] = acc;
      ss += acc * acc;
    }
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

__global__ void fold_partials_scalar_kernel(const float* __restrict__ partial, int nparts,
                                            float* __restrict__ out, int accumulate) {
  float s = 0.f;
  for (int b = threadIdx.x; b < nparts; b += 32) s += partial[b];
  s = warp_sum(s);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

__global__ void publish_scalar_kernel(PeerPtrs slots, int rank, int world,
                                      const float* __restrict__ val) {
  const int t = threadIdx.x;
  if (t < world) {
    static_cast<float*>(slots.p[t])[rank] = *val;
    __threadfence_system();
  }
}
__global__ void sum_slots_kernel(const float* slots, int world, float* out) {
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += __ldcv(slots + r);  // rank order: same bits everywhere
    out[0] = s;
  }
}

__device__ __forceinline__ float clip_scale_dev(const float* gnorm_sq, float clip) {
  if (gnorm_sq == nullptr || clip <= 0.f) return 1.f;
  const float n = sqrtf(fmaxf(*gnorm_sq, 0.f));
  return n > clip ? clip / (n + 1e-6f) : 1.f;
}

// AdamW on [lo, lo+n) of the slab; bf16 result stored into every rank's copy.
__global__ void __launch_bounds__(256) adamw_bcast_kernel(
    float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
    float* __restrict__ v, PeerPtrs lp, int world, long lo, long n, float lr, float b1, float b2,
    float eps, float wd, float inv_bc1, float inv_bc2, const float* __restrict__ gnorm_sq,
    float clip, float gscale) {
  const float s = clip_scale_dev(gnorm_sq, clip) * gscale;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = lo + i * 8;
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gi = g[e + j] * s;
      const float mi = b1 * m[e + j] + (1.f - b1) * gi;
      const float vi = b2 * v[e + j] + (1.f - b2) * gi * gi;
      m[e + j] = mi;
      v[e + j] = vi;
      const float pi = p[e + j] * (1.f - lr * wd) - lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
      p[e + j] = pi;
      o[j] = pi;
    }
    const bf16x8 pk = pack8(o);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<bf16x8*>(static_cast<bf16*>(lp.p[r]) + e) = pk;
  }
}

// p -= lr (scale O + wd p) on [lo, lo+n); bf16 result stored into every rank's copy.
__global__ void __launch_bounds__(256) muon_apply_bcast_kernel(float* __restrict__ p,
                                                               const bf16* __restrict__ o,
                                                               PeerPtrs lp, int world, long lo,
                                                               long n, float lr, float scale,
                                                               float wd) {
  const long n8 = n >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = lo + i * 8;
    float ov[8], q[8];
    unpack8(*reinterpret_cast<const bf16x8*>(o + i * 8), ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pi = p[e + j];
      q[j] = pi - lr * (scale * ov[j] + wd * pi);
      p[e + j] = q[j];
    }
    const bf16x8 pk = pack8(q);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<bf16x8*>(static_cast<bf16*>(lp.p[r]) + e) = pk;
  }
}

static inline int cgrid(long n, int per_thread) {
  long g = (n / per_thread + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

static PeerPtrs make_peers(void* const* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}

}  // namespace pb

using namespace pb;

PB_API int pb_symm_alloc(long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*out, 0, static_cast<size_t>(bytes)));
}
PB_API int pb_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }
PB_API int pb_ipc_get_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(out64, &h, sizeof(h));
  return 0;
}
PB_API int pb_ipc_open_handle(const void* h64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, h64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
PB_API int pb_ipc_close_handle(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }
PB_API int pb_ipc_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// Every rank calls this with the same (slot, epoch); returns when all have arrived or
// latches PB_TIMEOUT_FLAG into *status after budget_ns.
PB_API int pb_barrier_all(void* const* flag_ptrs, int rank, int world, int slot, int epoch,
                          long budget_ns, int* status, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || slot < 0) return PB_BAD_ARG;
  if (budget_ns <= 0 || budget_ns > 60000000000L) return PB_BAD_ARG;
  barrier_all_kernel<<<1, 32, 0, st>>>(make_peers(flag_ptrs, world), rank, world, slot,
                                       static_cast<uint32_t>(epoch),
                                       static_cast<uint64_t>(budget_ns), status);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_reduce_nparts(long n) {
  const int g = cgrid(n, 16);
  return g;
}

// out[lo:lo+n] = sum over ranks (rank order) of grads[r][lo:lo+n]; sumsq (+)= |out slice|^2.
// scratch: pb_reduce_nparts(n) floats. `out` may be this rank's own gradient buffer.
PB_API int pb_reduce_to_owner(void* const* grad_ptrs, int world, long lo, long n, void* out,
                              void* scratch, void* sumsq, int accumulate, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || (lo & 3) != 0) return PB_BAD_ARG;
  if (n <= 0) return 0;
  const int g = pb_reduce_nparts(n);
  const PeerPtrs pp = make_peers(grad_ptrs, world);
  float* out_ = static_cast<float*>(out);
  float* scr_ = static_cast<float*>(scratch);
  switch (world) {
    case 2: reduce_to_owner_kernel<2><<<g, 256, 0, st>>>(pp, lo, n, world, out_, scr_); break;
    case 4: reduce_to_owner_kernel<4><<<g, 256, 0, st>>>(pp, lo, n, world, out_, scr_); break;
    case 8: reduce_to_owner_kernel<8><<<g, 256, 0, st>>>(pp, lo, n, world, out_, scr_); break;
    default: reduce_to_owner_kernel<0><<<g, 256, 0, st>>>(pp, lo, n, world, out_, scr_); break;
  }
  fold_partials_scalar_kernel<<<1, 32, 0, st>>>(static_cast<const float*>(scratch), g,
                                                static_cast<float*>(sumsq), accumulate);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_publish_scalar(void* const* slot_ptrs, int rank, int world, const void* val,
                             cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS) return PB_BAD_ARG;
  publish_scalar_kernel<<<1, 32, 0, st>>>(make_peers(slot_ptrs, world), rank, world,
                                          static_cast<const float*>(val));
  return static_cast<int>(cudaGetLastError());
}
PB_API int pb_sum_slots(const void* slots, int world, void* out, cudaStream_t st) {
  sum_slots_kernel<<<1, 32, 0, st>>>(static_cast<const float*>(slots), world,
                                     static_cast<float*>(out));
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_adamw_bcast(void* p, const void* g, void* m, void* v, void* const* lp_ptrs,
                          int world, long lo, long n, float lr, float b1, float b2, float eps,
                          float wd, int step, const void* gnorm_sq, float clip, float gscale,
                          cudaStream_t st) {
  if (step < 1 || world < 1 || world > MAX_RANKS || (lo & 7) != 0 || (n & 7) != 0) return PB_BAD_ARG;
  if (n == 0) return 0;
  const float inv_bc1 = 1.f / (1.f - powf(b1, static_cast<float>(step)));
  const float inv_bc2 = 1.f / (1.f - powf(b2, static_cast<float>(step)));
  adamw_bcast_kernel<<<cgrid(n, 16), 256, 0, st>>>(
      static_cast<float*>(p), static_cast<const float*>(g), static_cast<float*>(m),
      static_cast<float*>(v), make_peers(lp_ptrs, world), world, lo, n, lr, b1, b2, eps, wd,
      inv_bc1, inv_bc2, static_cast<const float*>(gnorm_sq), clip, gscale);
  return static_cast<int>(cudaGetLastError());
}

// `o` points at the orthogonalised update of the slice itself (element 0 = element lo).
PB_API int pb_muon_apply_bcast(void* p, const void* o, void* const* lp_ptrs, int world, long lo,
                               long n, float lr, float scale, float wd, cudaStream_t st) {
  if (world < 1 || world > MAX_RANKS || (lo & 7) != 0 || (n & 7) != 0) return PB_BAD_ARG;
  if (n == 0) return 0;
  muon_apply_bcast_kernel<<<cgrid(n, 16), 256, 0, st>>>(
      static_cast<float*>(p), static_cast<const bf16*>(o), make_peers(lp_ptrs, world), world, lo,
      n, lr, scale, wd);
  return static_cast<int>(cudaGetLastError());
}
