// ZeRO-3 parameter sharding over symmetric memory (one process per GPU).
//
// The bf16 working weights of a group of matrices (one transformer layer, the embedding
// table, the unembedding) form a "blob" of L elements; rank q keeps elements
// [q * L / N, (q + 1) * L / N) of every blob in its shard region, nothing else.
//
//   pb_shard_gather       all-gather of one blob into a local landing buffer: every rank
//                         pulls its peers' chunks with 16-byte loads over NVLink (its own
//                         chunk is a local copy). Run on a side stream one layer ahead of the
//                         compute, so the transfer hides behind the previous layer's kernels.
//   pb_muon_apply_table   Moonlight update of a batch of owned matrices (fp32 masters held
//                         by the owner only) whose refreshed bf16 values are stored straight
//                         to where they live: the one rank holding that part of the blob
//                         (sharded), every rank (replicated small weights) or this rank only
//                         (expert-parallel weights). The parameter all-gather of a
//                         replicated design becomes one store per element.
//   pb_adamw_table        the same for a range of the AdamW slab.
//
// Reference contract: parallel/fsdp.py:145-158 (gather = concatenation of the shards in rank
// order) and :193-222 (bf16 working view + fp32 master view, shard first, cast second).
// Peer traffic is plain loads / stores on peer pointers; ordering against the consumers is the
// caller's bounded device barrier.
#include "common.cuh"

namespace pb {

constexpr int FS_MAX_RANKS = 8;

struct FsPeers {
  void* p[FS_MAX_RANKS];
};

// where a weight's bf16 copy lives: chunk > 0: sharded blob, element P of the blob is on rank
// P / chunk at base + P % chunk; chunk == 0: replicated, every rank at base + t; chunk < 0: this
// rank only at base + t. `pos` is the weight's first element inside its blob.
struct FsDest {
  long pos, chunk, base;
};

__device__ __forceinline__ void fs_store8(const FsPeers& lp, const FsDest& d, long t, int world,
                                          int rank, const bf16x8& v) {
  if (d.chunk > 0) {
    const long P = d.pos + t;
    const int r = static_cast<int>(P / d.chunk);
    *reinterpret_cast<bf16x8*>(static_cast<bf16*>(lp.p[r]) + d.base + (P - r * d.chunk)) = v;
  } else if (d.chunk == 0) {
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<bf16x8*>(static_cast<bf16*>(lp.p[r]) + d.base + t) = v;
  } else {
    *reinterpret_cast<bf16x8*>(static_cast<bf16*>(lp.p[rank]) + d.base + t) = v;
  }
}

// dst[q * chunk + t] = shard_q[shard_off + t]
__global__ void __launch_bounds__(256) shard_gather_kernel(FsPeers shards, long shard_off,
                                                           long chunk, bf16* __restrict__ dst,
                                                           int world, int rank) {
  const long v_per = chunk >> 3;                 // 16-byte vectors per chunk
  const long total = v_per * world;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  // four loads in flight per thread
  for (; i + 3 * stride < total; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long j = i + u * stride;
      const int q = static_cast<int>(j / v_per);
      const long t = j - q * v_per;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const bf16*>(shards.p[q]) + shard_off) + t;
      v[u] = __ldcv(src);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) reinterpret_cast<uint4*>(dst)[i + u * stride] = v[u];
  }
  for (; i < total; i += stride) {
    const int q = static_cast<int>(i / v_per);
    const long t = i - q * v_per;
    reinterpret_cast<uint4*>(dst)[i] =
        __ldcv(reinterpret_cast<const uint4*>(static_cast<const bf16*>(shards.p[q]) + shard_off) + t);
  }
}

// blockIdx.y = matrix j of the batch (n elements each, back to back in p and o)
__global__ void __launch_bounds__(256) muon_apply_table_kernel(float* __restrict__ p,
                                                               const bf16* __restrict__ o, long n,
                                                               float lr, float scale, float wd,
                                                               const FsDest* __restrict__ table,
                                                               FsPeers lp, int world, int rank) {
  const FsDest d = table[blockIdx.y];
  p += static_cast<long>(blockIdx.y) * n;
  o += static_cast<long>(blockIdx.y) * n;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = i * 8;
    float ov[8], q[8];
    unpack8(*reinterpret_cast<const bf16x8*>(o + e), ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pi = p[e + j];
      q[j] = pi - lr * (scale * ov[j] + wd * pi);
      p[e + j] = q[j];
    }
    fs_store8(lp, d, e, world, rank, pack8(q));
  }
}

__device__ __forceinline__ float fs_clip_scale(const float* gnorm_sq, float clip) {
  if (gnorm_sq == nullptr || clip <= 0.f) return 1.f;
  const float n = sqrtf(fmaxf(*gnorm_sq, 0.f));
  return n > clip ? clip / (n + 1e-6f) : 1.f;
}

// AdamW on n elements: p, m, v are the owner's state (element 0 = first element of the range),
// g the gradient of the same range.
__global__ void __launch_bounds__(256) adamw_table_kernel(
    float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
    float* __restrict__ v, long n, float lr, float b1, float b2, float eps, float wd,
    float inv_bc1, float inv_bc2, const float* __restrict__ gnorm_sq, float clip, float gscale,
    FsDest d, FsPeers lp, int world, int rank) {
  const float s = fs_clip_scale(gnorm_sq, clip) * gscale;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = i * 8;
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
    fs_store8(lp, d, e, world, rank, pack8(o));
  }
}

static FsPeers fs_peers(void* const* ptrs, int world) {
  FsPeers pp;
  for (int i = 0; i < FS_MAX_RANKS; ++i) pp.p[i] = i < world ? ptrs[i] : nullptr;
  return pp;
}
static inline int fs_grid(long n, int per_thread, int cap) {
  long g = (n / per_thread + 255) / 256;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace pb

using namespace pb;

// dst (L = chunk * world bf16 elements, 16-byte aligned) = concatenation over ranks of
// shard_ptrs[q][shard_off : shard_off + chunk]. chunk and shard_off multiples of 8.
// max_ctas bounds the grid so the copy shares the GPU with the compute it overlaps (0: default).
PB_API int pb_shard_gather(void* const* shard_ptrs, long shard_off, long chunk, void* dst,
                           int world, int rank, int max_ctas, cudaStream_t st) {
  if (world < 1 || world > FS_MAX_RANKS || rank < 0 || rank >= world || chunk <= 0 ||
      (chunk & 7) != 0 || (shard_off & 7) != 0 || (reinterpret_cast<uintptr_t>(dst) & 15) != 0)
    return PB_BAD_ARG;
  const int cap = max_ctas > 0 ? max_ctas : 148 * 2;
  shard_gather_kernel<<<fs_grid((chunk >> 3) * world, 4, cap), 256, 0, st>>>(
      fs_peers(shard_ptrs, world), shard_off, chunk, static_cast<bf16*>(dst), world, rank);
  return static_cast<int>(cudaGetLastError());
}

// p, o: nb matrices of n elements each (n a multiple of 8); table: nb FsDest entries (device).
PB_API int pb_muon_apply_table(void* p, const void* o, long n, int nb, float lr, float scale,
                               float wd, const void* table, void* const* lp_ptrs, int world,
                               int rank, cudaStream_t st) {
  if (world < 1 || world > FS_MAX_RANKS || rank < 0 || rank >= world || (n & 7) != 0 ||
      table == nullptr)
    return PB_BAD_ARG;
  if (nb <= 0 || n == 0) return 0;
  for (int j0 = 0; j0 < nb; j0 += 32768) {
    const int cnt = nb - j0 < 32768 ? nb - j0 : 32768;
    muon_apply_table_kernel<<<dim3(fs_grid(n, 16, 148 * 4), cnt), 256, 0, st>>>(
        static_cast<float*>(p) + static_cast<long>(j0) * n,
        static_cast<const bf16*>(o) + static_cast<long>(j0) * n, n, lr, scale, wd,
        static_cast<const FsDest*>(table) + j0, fs_peers(lp_ptrs, world), world, rank);
  }
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_adamw_table(void* p, const void* g, void* m, void* v, long n, float lr, float b1,
                          float b2, float eps, float wd, int step, const void* gnorm_sq,
                          float clip, float gscale, long pos, long chunk, long base,
                          void* const* lp_ptrs, int world, int rank, cudaStream_t st) {
  if (step < 1 || world < 1 || world > FS_MAX_RANKS || rank < 0 || rank >= world || (n & 7) != 0 ||
      (pos & 7) != 0 || (base & 7) != 0 || (chunk > 0 && (chunk & 7) != 0))
    return PB_BAD_ARG;
  if (n == 0) return 0;
  const float inv_bc1 = 1.f / (1.f - powf(b1, static_cast<float>(step)));
  const float inv_bc2 = 1.f / (1.f - powf(b2, static_cast<float>(step)));
  FsDest d;
  d.pos = pos; d.chunk = chunk; d.base = base;
  adamw_table_kernel<<<fs_grid(n, 16, 148 * 8), 256, 0, st>>>(
      static_cast<float*>(p), static_cast<const float*>(g), static_cast<float*>(m),
      static_cast<float*>(v), n, lr, b1, b2, eps, wd, inv_bc1, inv_bc2,
      static_cast<const float*>(gnorm_sq), clip, gscale, d, fs_peers(lp_ptrs, world), world, rank);
  return static_cast<int>(cudaGetLastError());
}
