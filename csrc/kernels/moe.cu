// Mixture-of-experts routing and token movement (sm_100a).
//
//   route        sigmoid scores, stable top-k (ties -> lower expert), gates = top / sum(top)
//   count/scan/place   a stable counting sort of the (token, slot) pairs by expert that gives
//                each pair its row in the expert-grouped buffer; expert segments start on
//                128-row boundaries so a segment is a whole number of GEMM row blocks
//   permute      gather token rows into the grouped buffer (optionally scaled by the gate: the
//                backward of combine), zeroing the padding rows
//   combine      out[t] = sum_s gate[t, s] * y[row(t, s)]  (gate = 1: backward of permute)
//   combine_bwd  dgate[t, s] = <y[row(t, s)], dout[t]>
//   route_bwd    gradient of the gates w.r.t. the router logits
//
// Row placement is a pure function of the expert ids (no atomics decide an order), so the
// grouped GEMMs and their weight gradients are bit-reproducible run to run.
//
// Reference semantics: model/__init__.py:485-598 of the reference (sigmoid router, top-k,
// gate normalisation with a 1e-9 floor); the grouped data path is this library's own.
#include "common.cuh"

namespace pb {
namespace moe {

constexpr int TOK_PER_BLOCK = 256;   // tokens per block of the counting sort
constexpr int MAX_E = 512;
constexpr int MAX_K = 32;

// One warp per token. logits: [T, E] fp32. bias: [E] or null (selection only).
// PER = experts per lane the instantiation is unrolled for (2 covers 64 experts: a quarter of
// the compare / select work of the 512-expert form for the same result).
template <int PER>
__global__ void route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                             int T, int E, int k, float* __restrict__ probs, int* __restrict__ ids,
                             float* __restrict__ gates) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + static_cast<size_t>(warp) * E;
  float p[PER], s[PER];
  const int per = (E + 31) / 32;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    if (i < per && e < E) {
      p[i] = 1.f / (1.f + expf(-row[e]));
      s[i] = p[i] + (bias ? bias[e] : 0.f);
      probs[static_cast<size_t>(warp) * E + e] = p[i];
    } else {
      p[i] = 0.f;
      s[i] = -INFINITY;
    }
  }
  float mine = 0.f;   // lane j keeps the probability of the j-th pick
  float sum = 0.f;
  for (int j = 0; j < k; ++j) {
    // best remaining (score, lowest index) of this lane, then across the warp
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (i < per && s[i] > bv) { bv = s[i]; be = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    // owner lane retires the winner and reports its probability
    float pv = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (i * 32 + lane == be) { pv = p[i]; s[i] = -INFINITY; }
    pv = __shfl_sync(0xffffffffu, pv, be & 31);
    if (lane == j) mine = pv;
    sum += pv;
    if (lane == 0) ids[static_cast<size_t>(warp) * k + j] = be;
  }
  const float inv = 1.f / fmaxf(sum, 1e-9f);
  if (lane < k) gates[static_cast<size_t>(warp) * k + lane] = mine * inv;
}

// Gradient of gates w.r.t. logits. dgates, gates: [T, k]; probs: [T, E]; dlogits: [T, E] (zeroed
// here except at the selected experts).
__global__ void route_bwd_kernel(const float* __restrict__ dgates, const float* __restrict__ gates,
                                 const float* __restrict__ probs, const int* __restrict__ ids, int T,
                                 int E, int k, float* __restrict__ dlogits) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  float* drow = dlogits + static_cast<size_t>(warp) * E;
  for (int e = lane; e < E; e += 32) drow[e] = 0.f;
  __syncwarp();
  if (lane == 0) {
    const size_t o = static_cast<size_t>(warp) * k;
    float sum = 0.f, dot = 0.f;
    for (int j = 0; j < k; ++j) {
      sum += probs[static_cast<size_t>(warp) * E + ids[o + j]];
      dot += dgates[o + j] * gates[o + j];
    }
    if (sum > 1e-9f) {
      const float inv = 1.f / sum;
      for (int j = 0; j < k; ++j) {
        const int e = ids[o + j];
        const float p = probs[static_cast<size_t>(warp) * E + e];
        drow[e] = (dgates[o + j] - dot) * inv * p * (1.f - p);
      }
    }
  }
}

// per-block histogram of expert ids. block_counts: [nblocks, E]
__global__ void count_kernel(const int* __restrict__ ids, int n_pairs, int pairs_per_block, int E,
                             int* __restrict__ block_counts) {
  __shared__ int hist[MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int lo = blockIdx.x * pairs_per_block;
  const int hi = min(lo + pairs_per_block, n_pairs);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) atomicAdd(&hist[ids[i]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    block_counts[static_cast<size_t>(blockIdx.x) * E + e] = hist[e];
}

// One block. Turns block_counts into exclusive per-block bases, and writes
//   expert_off[e] (128-aligned segment starts, expert_off[E] = rows in use), totals[e],
//   k_len[e] = padded segment length, mblk_group[m] for m < max_mblk (-1 beyond the data).
__global__ void scan_kernel(int* __restrict__ block_counts, int nblocks, int E,
                            int* __restrict__ expert_off, int* __restrict__ totals,
                            int* __restrict__ k_len, int* __restrict__ mblk_group, int max_mblk) {
  __shared__ int tot[MAX_E];
  __shared__ int off[MAX_E + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < nblocks; ++b) {
      const int c = block_counts[static_cast<size_t>(b) * E + e];
      block_counts[static_cast<size_t>(b) * E + e] = run;
      run += c;
    }
    tot[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      run += (tot[e] + 127) / 128 * 128;
    }
    off[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    expert_off[e] = off[e];
    if (e < E) {
      totals[e] = tot[e];
      k_len[e] = off[e + 1] - off[e];
    }
  }
  for (int m = threadIdx.x; m < max_mblk; m += blockDim.x) {
    const int row = m * 128;
    int g = -1;
    if (row < off[E]) {
      int lo = 0, hi = E;   // last e with off[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (off[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    mblk_group[m] = g;
  }
}

// One warp per block of pairs walks them in order; row_of[i] = expert_off + block base + rank.
__global__ void place_kernel(const int* __restrict__ ids, int n_pairs, int pairs_per_block, int E,
                             const int* __restrict__ block_base, const int* __restrict__ expert_off,
                             int* __restrict__ row_of) {
  __shared__ int run[MAX_E];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32)
    run[e] = expert_off[e] + block_base[static_cast<size_t>(blockIdx.x) * E + e];
  __syncwarp();
  const int lo = blockIdx.x * pairs_per_block;
  const int hi = min(lo + pairs_per_block, n_pairs);
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const bool on = i < hi;
    const int e = on ? ids[i] : -1 - lane;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    int start = 0;
    if (on) start = run[e];
    __syncwarp();
    if (on) {
      row_of[i] = start + rank;
      if (rank == __popc(same) - 1) run[e] = start + rank + 1;   // last of its group advances
    }
    __syncwarp();
  }
}

// dst[row_of[t, s]] = scale * src[t]; one warp per pair. d % 8 == 0.
__global__ void permute_kernel(const bf16* __restrict__ src, const int* __restrict__ row_of,
                               const float* __restrict__ scale, int n_pairs, int k, int d, long ld_src,
                               bf16* __restrict__ dst, long dst_rows) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_pairs) return;
  const bf16* s = src + static_cast<size_t>(w / k) * ld_src;
  if (!PB_BOUNDS_OK(PB_K_MOE_PERMUTE, row_of[w], dst_rows)) return;
  bf16* o = dst + static_cast<size_t>(row_of[w]) * d;
  const float g = scale ? scale[w] : 1.f;
  for (int c = lane * 8; c < d; c += 256) {
    bf16x8 v = *reinterpret_cast<const bf16x8*>(s + c);
    if (scale) {
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= g;
      v = pack8(f);
    }
    *reinterpret_cast<bf16x8*>(o + c) = v;
  }
}

// zero rows [expert_off[e] + totals[e], expert_off[e + 1]) ; one block per expert
__global__ void zero_pad_kernel(bf16* __restrict__ buf, int d, const int* __restrict__ expert_off,
                                const int* __restrict__ totals) {
  const int e = blockIdx.x;
  const int lo = expert_off[e] + totals[e], hi = expert_off[e + 1];
  const size_t n8 = static_cast<size_t>(hi - lo) * d / 8;
  bf16x8 z;
#pragma unroll
  for (int j = 0; j < 4; ++j) z.v[j] = __floats2bfloat162_rn(0.f, 0.f);
  bf16x8* p = reinterpret_cast<bf16x8*>(buf + static_cast<size_t>(lo) * d);
  for (size_t i = threadIdx.x; i < n8; i += blockDim.x) p[i] = z;
}

// out[t] = sum_s gate[t, s] * y[row_of[t, s]] (+ add[t]); one warp per token, fp32 accumulate.
__global__ void combine_kernel(const bf16* __restrict__ y, const int* __restrict__ row_of,
                               const float* __restrict__ gates, const bf16* __restrict__ add, int T,
                               int k, int d, bf16* __restrict__ out, long y_rows) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane * 8; c < d; c += 256) {
    float acc[8];
    if (add != nullptr) unpack8(*reinterpret_cast<const bf16x8*>(add + static_cast<size_t>(t) * d + c), acc);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int s = 0; s < k; ++s) {
      const size_t i = static_cast<size_t>(t) * k + s;
      const float g = gates ? gates[i] : 1.f;
      float f[8];
      if (!PB_BOUNDS_OK(PB_K_MOE_COMBINE, row_of[i], y_rows)) continue;
      unpack8(*reinterpret_cast<const bf16x8*>(y + static_cast<size_t>(row_of[i]) * d + c), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(g, f[j], acc[j]);
    }
    *reinterpret_cast<bf16x8*>(out + static_cast<size_t>(t) * d + c) = pack8(acc);
  }
}

// dgates[t, s] = <y[row_of[t, s]], dout[t]> ; one warp per pair
__global__ void combine_bwd_kernel(const bf16* __restrict__ y, const bf16* __restrict__ dout,
                                   const int* __restrict__ row_of, int n_pairs, int k, int d,
                                   float* __restrict__ dgates) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= n_pairs) return;
  const bf16* a = y + static_cast<size_t>(row_of[w]) * d;
  const bf16* b = dout + static_cast<size_t>(w / k) * d;
  float acc = 0.f;
  for (int c = lane * 8; c < d; c += 256) {
    float f[8], g[8];
    unpack8(*reinterpret_cast<const bf16x8*>(a + c), f);
    unpack8(*reinterpret_cast<const bf16x8*>(b + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(f[j], g[j], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) dgates[w] = acc;
}

}  // namespace moe
}  // namespace pb

using namespace pb;

static inline int warps_grid(long warps, int threads) {
  return static_cast<int>((warps * 32 + threads - 1) / threads);
}

PB_API int pb_moe_route(const float* logits, const float* bias, int T, int E, int k, float* probs,
                        int* ids, float* gates, cudaStream_t st) {
  if (T <= 0 || E <= 0 || E > moe::MAX_E || k <= 0 || k > moe::MAX_K || k > E) return PB_BAD_ARG;
  const int per = (E + 31) / 32;
  const int grid = warps_grid(T, 256);
  if (per <= 2) moe::route_kernel<2><<<grid, 256, 0, st>>>(logits, bias, T, E, k, probs, ids, gates);
  else if (per <= 4) moe::route_kernel<4><<<grid, 256, 0, st>>>(logits, bias, T, E, k, probs, ids, gates);
  else if (per <= 8) moe::route_kernel<8><<<grid, 256, 0, st>>>(logits, bias, T, E, k, probs, ids, gates);
  else moe::route_kernel<moe::MAX_E / 32><<<grid, 256, 0, st>>>(logits, bias, T, E, k, probs, ids, gates);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_moe_route_bwd(const float* dgates, const float* gates, const float* probs,
                            const int* ids, int T, int E, int k, float* dlogits, cudaStream_t st) {
  if (T <= 0 || E <= 0 || k <= 0) return PB_BAD_ARG;
  moe::route_bwd_kernel<<<warps_grid(T, 256), 256, 0, st>>>(dgates, gates, probs, ids, T, E, k, dlogits);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_moe_sort_nblocks(int n_pairs, int k) {
  const int per = moe::TOK_PER_BLOCK * k;
  return (n_pairs + per - 1) / per;
}

// Rows for the (token, slot) pairs grouped by expert. ids: [n_pairs] expert of each pair in
// token-major order; scratch: nblocks * E ints. Outputs: row_of [n_pairs]; expert_off [E + 1];
// totals [E]; k_len [E]; mblk_group [max_mblk].
PB_API int pb_moe_sort(const int* ids, int n_pairs, int k, int E, int* scratch, int* row_of,
                       int* expert_off, int* totals, int* k_len, int* mblk_group, int max_mblk,
                       cudaStream_t st) {
  if (n_pairs <= 0 || E <= 0 || E > moe::MAX_E || k <= 0) return PB_BAD_ARG;
  const int per = moe::TOK_PER_BLOCK * k;
  const int nblocks = (n_pairs + per - 1) / per;
  moe::count_kernel<<<nblocks, 256, 0, st>>>(ids, n_pairs, per, E, scratch);
  moe::scan_kernel<<<1, 512, 0, st>>>(scratch, nblocks, E, expert_off, totals, k_len, mblk_group,
                                      max_mblk);
  moe::place_kernel<<<nblocks, 32, 0, st>>>(ids, n_pairs, per, E, scratch, expert_off, row_of);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_moe_permute(const void* src, const int* row_of, const float* scale, int n_pairs, int k,
                          int d, long ld_src, void* dst, const int* expert_off, const int* totals,
                          int E, cudaStream_t st) {
  if (n_pairs <= 0 || d % 8 != 0) return PB_BAD_ARG;
  // rows of dst: the worst case the placement sizes its buffers for
  const long dst_rows = (static_cast<long>(n_pairs) + static_cast<long>(E > 0 ? E : 1) * 127 + 127) / 128 * 128;
  moe::permute_kernel<<<warps_grid(n_pairs, 256), 256, 0, st>>>(
      static_cast<const bf16*>(src), row_of, scale, n_pairs, k, d, ld_src, static_cast<bf16*>(dst),
      dst_rows);
  if (expert_off != nullptr)
    moe::zero_pad_kernel<<<E, 256, 0, st>>>(static_cast<bf16*>(dst), d, expert_off, totals);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_moe_zero_pad(void* buf, int d, const int* expert_off, const int* totals, int E,
                           cudaStream_t st) {
  if (E <= 0 || d % 8 != 0) return PB_BAD_ARG;
  moe::zero_pad_kernel<<<E, 256, 0, st>>>(static_cast<bf16*>(buf), d, expert_off, totals);
  return static_cast<int>(cudaGetLastError());
}

// y_rows: rows of y (the bound the debug build checks row_of against; 0 = unknown).
PB_API int pb_moe_combine(const void* y, const int* row_of, const float* gates, const void* add,
                          int T, int k, int d, void* out, long y_rows, cudaStream_t st) {
  if (T <= 0 || d % 8 != 0) return PB_BAD_ARG;
  moe::combine_kernel<<<warps_grid(T, 256), 256, 0, st>>>(
      static_cast<const bf16*>(y), row_of, gates, static_cast<const bf16*>(add), T, k, d,
      static_cast<bf16*>(out), y_rows > 0 ? y_rows : (1L << 62));
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_moe_combine_bwd(const void* y, const void* dout, const int* row_of, int n_pairs, int k,
                              int d, float* dgates, cudaStream_t st) {
  if (n_pairs <= 0 || d % 8 != 0) return PB_BAD_ARG;
  moe::combine_bwd_kernel<<<warps_grid(n_pairs, 256), 256, 0, st>>>(
      static_cast<const bf16*>(y), static_cast<const bf16*>(dout), row_of, n_pairs, k, d, dgates);
  return static_cast<int>(cudaGetLastError());
}

PB_DEFINE_BOUNDS_READER(moe)
