// Fused optimizer kernels over flat fp32 master buffers (sm_100a, HBM-bound):
// deterministic sum of squares, global-norm clip factor, AdamW, Muon momentum
// (Nesterov) + Frobenius normalisation into the bf16 Newton-Schulz input, and
// the Moonlight / Jordan parameter update that also refreshes the bf16 copy.
//
// Math: train/__init__.py adamw_update (:503-539), muon_update (:346-374),
// muon_transfer_step (:401-458), grad clip (:917-928) of the reference.
#include "common.cuh"

namespace pb {

// partial[b] = sum over this block's grid-stride slice of x^2
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const float* __restrict__ x, long n,
                                                            float* __restrict__ partial) {
  __shared__ float scratch[33];
  float s = 0.f;
  const long n4 = n >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 v = x4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0)
    for (long i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) s += x[i] * x[i];
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256) sumsq_partial_bf16_kernel(const bf16* __restrict__ x,
                                                                 long n,
                                                                 float* __restrict__ partial) {
  __shared__ float scratch[33];
  float s = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float v = bf16_to_f32(x[i]);
    s += v * v;
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] (+)= sum_b partial[b], fixed order, one warp.
__global__ void fold_scalar_kernel(const float* __restrict__ partial, int nparts,
                                   float* __restrict__ out, int accumulate) {
  float s = 0.f;
  for (int b = threadIdx.x; b < nparts; b += 32) s += partial[b];
  // fixed-shape butterfly: deterministic for a fixed nparts
  s = warp_sum(s);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

// out[j] = sum_b partial[j * nparts + b] for every matrix j = blockIdx.x: one warp each, the
// same fixed order as fold_scalar_kernel.
__global__ void fold_rows_kernel(const float* __restrict__ partial, int nparts,
                                 float* __restrict__ out) {
  const float* p = partial + static_cast<long>(blockIdx.x) * nparts;
  float s = 0.f;
  for (int b = threadIdx.x; b < nparts; b += 32) s += p[b];
  s = warp_sum(s);
  if (threadIdx.x == 0) out[blockIdx.x] = s;
}

// scale = clip / (norm + 1e-6) if norm > clip else 1   (clip <= 0: 1)
__device__ __forceinline__ float clip_scale(const float* gnorm_sq, float clip) {
  if (gnorm_sq == nullptr || clip <= 0.f) return 1.f;
  const float n = sqrtf(fmaxf(*gnorm_sq, 0.f));
  return n > clip ? clip / (n + 1e-6f) : 1.f;
}

__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p,
                                                    const float* __restrict__ g,
                                                    float* __restrict__ m, float* __restrict__ v,
                                                    bf16* __restrict__ p_lp, long n, float lr,
                                                    float b1, float b2, float eps, float wd,
                                                    float inv_bc1, float inv_bc2,
                                                    const float* __restrict__ gnorm_sq,
                                                    float clip, float gscale) {
  const float s = clip_scale(gnorm_sq, clip) * gscale;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gi = g[i] * s;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float step = (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
    const float pi = p[i] * (1.f - lr * wd) - lr * step;
    p[i] = pi;
    if (p_lp != nullptr) p_lp[i] = f32_to_bf16(pi);
  }
}

// m = beta*m + s*g;  partial sums of nesterov^2 with nesterov = s*g + beta*m.
// blockIdx.y selects one of gridDim.y equally sized matrices laid out back to back; the
// partials of matrix j are partial[j * gridDim.x .. (j + 1) * gridDim.x).
__global__ void __launch_bounds__(256) muon_momentum_kernel(const float* __restrict__ g,
                                                            float* __restrict__ m, long n,
                                                            float beta,
                                                            const float* __restrict__ gnorm_sq,
                                                            float clip, float gscale,
                                                            float* __restrict__ partial) {
  __shared__ float scratch[33];
  const float s = clip_scale(gnorm_sq, clip) * gscale;
  g += static_cast<long>(blockIdx.y) * n;
  m += static_cast<long>(blockIdx.y) * n;
  partial += static_cast<long>(blockIdx.y) * gridDim.x;
  float acc = 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gi = g[i] * s;
    const float mi = beta * m[i] + gi;
    m[i] = mi;
    const float nes = gi + beta * mi;
    acc += nes * nes;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}
// x0 = bf16(nesterov / |nesterov|_F) (zeros if the norm is below 1e-7)
__global__ void __launch_bounds__(256) muon_normalize_kernel(const float* __restrict__ g,
                                                             const float* __restrict__ m,
                                                             bf16* __restrict__ x0, long n,
                                                             float beta,
                                                             const float* __restrict__ gnorm_sq,
                                                             float clip, float gscale,
                                                             const float* __restrict__ nes_sq) {
  const float s = clip_scale(gnorm_sq, clip) * gscale;
  g += static_cast<long>(blockIdx.y) * n;
  m += static_cast<long>(blockIdx.y) * n;
  x0 += static_cast<long>(blockIdx.y) * n;
  const float fro = sqrtf(fmaxf(nes_sq[blockIdx.y], 0.f));
  const float inv = fro > 1e-7f ? 1.f / fro : 0.f;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float nes = g[i] * s + beta * m[i];
    x0[i] = f32_to_bf16(nes * inv);
  }
}
// p = p - lr * (scale * O + wd * p); p_lp = bf16(p)
__global__ void __launch_bounds__(256) muon_apply_kernel(float* __restrict__ p,
                                                         const bf16* __restrict__ o,
                                                         bf16* __restrict__ p_lp, long n, float lr,
                                                         float scale, float wd) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float pi = p[i];
    const float q = pi - lr * (scale * bf16_to_f32(o[i]) + wd * pi);
    p[i] = q;
    if (p_lp != nullptr) p_lp[i] = f32_to_bf16(q);
  }
}

// y = bf16(x * scale) ; plain cast helpers for the flat buffers
__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, bf16* __restrict__ y, long n,
                                     float scale) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    y[i] = f32_to_bf16(x[i] * scale);
}
// acc_f32 += scale * x_bf16
__global__ void axpy_bf16_f32_kernel(const bf16* __restrict__ x, float* __restrict__ acc, long n,
                                     float scale) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    acc[i] += scale * bf16_to_f32(x[i]);
}
// out[c][r] = in[r][c] (bf16), 32x32 tiles through shared memory
__global__ void transpose_bf16_kernel(const bf16* __restrict__ in, bf16* __restrict__ out,
                                      int rows, int cols) {
  __shared__ bf16 tile[32][33];
  const int bx = blockIdx.x * 32, by = blockIdx.y * 32;
  const size_t boff = static_cast<size_t>(blockIdx.z) * rows * cols;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = by + j, c = bx + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[boff + static_cast<size_t>(r) * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int c = bx + j, r = by + threadIdx.x;
    if (r < rows && c < cols) out[boff + static_cast<size_t>(c) * rows + r] = tile[threadIdx.x][j];
  }
}

// QK-clip on observed logits. max_logit[h] is the largest scaled attention logit query head h
// produced during the step; a head over `tau` has its logits pulled back to tau by scaling the
// rows of its query projection and of its key projection. Query heads that share a key head
// (G per group): the key rows take fk = sqrt(min(1, tau / max over the group)), query head h
// takes min(1, tau / max_h) / fk, so every head's logits scale by exactly min(1, tau / max_h).
// One block per weight row; rows [row0, row0 + rows) of the (heads * dh, cols) matrix are in
// `master` (fp32, may be null) and `lp` (bf16, may be null).
__global__ void __launch_bounds__(256) qk_clip_rescale_kernel(float* __restrict__ master,
                                                              bf16* __restrict__ lp, int rows,
                                                              int cols, int dh, int group,
                                                              int n_q_heads, int is_k, long row0,
                                                              const float* __restrict__ max_logit,
                                                              float tau) {
  const long r = blockIdx.x;
  if (r >= rows) return;
  const int head = static_cast<int>((row0 + r) / dh);
  const int kv = is_k ? head : head / group;
  float mg = 0.f;
  for (int j = 0; j < group; ++j) {
    const int h = kv * group + j;
    if (h < n_q_heads) mg = fmaxf(mg, max_logit[h]);
  }
  const float fk = sqrtf(mg > tau ? tau / mg : 1.f);
  float f = fk;
  if (!is_k) {
    const float mh = max_logit[head];
    f = (mh > tau ? tau / mh : 1.f) / fk;
  }
  if (f == 1.f) return;
  const long base = r * static_cast<long>(cols);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    if (master != nullptr) {
      const float v = master[base + c] * f;
      master[base + c] = v;
      if (lp != nullptr) lp[base + c] = f32_to_bf16(v);
    } else if (lp != nullptr) {
      lp[base + c] = f32_to_bf16(bf16_to_f32(lp[base + c]) * f);
    }
  }
}

// 64-bit position-weighted checksum of a flat buffer of 32-bit words (silent-data-corruption
// probe: every replica of a shard must produce the same value). Partials are combined with
// integer adds, so the result does not depend on the grid.
__global__ void __launch_bounds__(256) checksum_u32_kernel(const uint32_t* __restrict__ x, long n,
                                                           unsigned long long* __restrict__ out) {
  unsigned long long acc = 0ull;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const unsigned long long w = x[i];
    acc += (w + 0x9E3779B97F4A7C15ull) * (static_cast<unsigned long long>(i) * 2ull + 1ull);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(out, acc);
}

static inline int ogrid(long n, int per_thread = 4) {
  long g = (n / per_thread + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace pb

using namespace pb;

#define PB_SUMSQ_MAX_PARTS 1184

PB_API int pb_sumsq_nparts(long n) {
  const int g = ogrid(n);
  return g < PB_SUMSQ_MAX_PARTS ? g : PB_SUMSQ_MAX_PARTS;
}

// out[0] (+)= sum(x^2). scratch: pb_sumsq_nparts(n) floats.
PB_API int pb_sumsq_f32(const void* x, long n, void* scratch, void* out, int accumulate,
                        cudaStream_t st) {
  const int g = pb_sumsq_nparts(n);
  sumsq_partial_kernel<<<g, 256, 0, st>>>(static_cast<const float*>(x), n,
                                          static_cast<float*>(scratch));
  fold_scalar_kernel<<<1, 32, 0, st>>>(static_cast<const float*>(scratch), g,
                                       static_cast<float*>(out), accumulate);
  return cudaGetLastError();
}
PB_API int pb_sumsq_bf16(const void* x, long n, void* scratch, void* out, int accumulate,
                         cudaStream_t st) {
  const int g = pb_sumsq_nparts(n);
  sumsq_partial_bf16_kernel<<<g, 256, 0, st>>>(static_cast<const bf16*>(x), n,
                                               static_cast<float*>(scratch));
  fold_scalar_kernel<<<1, 32, 0, st>>>(static_cast<const float*>(scratch), g,
                                       static_cast<float*>(out), accumulate);
  return cudaGetLastError();
}

PB_API int pb_adamw(void* p, const void* g, void* m, void* v, void* p_lp, long n, float lr,
                    float b1, float b2, float eps, float wd, int step, const void* gnorm_sq,
                    float clip, float gscale, cudaStream_t st) {
  if (step < 1) return PB_BAD_ARG;
  const float inv_bc1 = 1.f / (1.f - powf(b1, static_cast<float>(step)));
  const float inv_bc2 = 1.f / (1.f - powf(b2, static_cast<float>(step)));
  adamw_kernel<<<ogrid(n), 256, 0, st>>>(
      static_cast<float*>(p), static_cast<const float*>(g), static_cast<float*>(m),
      static_cast<float*>(v), static_cast<bf16*>(p_lp), n, lr, b1, b2, eps, wd, inv_bc1, inv_bc2,
      static_cast<const float*>(gnorm_sq), clip, gscale);
  return cudaGetLastError();
}

// Momentum + Nesterov + Frobenius-normalised bf16 Newton-Schulz input.
// scratch: pb_sumsq_nparts(n) + 1 floats (the last one receives |nesterov|^2).
PB_API int pb_muon_prepare(const void* g, void* m, void* x0, long n, float beta,
                           const void* gnorm_sq, float clip, float gscale, void* scratch,
                           cudaStream_t st) {
  const int parts = pb_sumsq_nparts(n);
  float* part = static_cast<float*>(scratch);
  float* nes_sq = part + parts;
  muon_momentum_kernel<<<parts, 256, 0, st>>>(static_cast<const float*>(g),
                                              static_cast<float*>(m), n, beta,
                                              static_cast<const float*>(gnorm_sq), clip, gscale,
                                              part);
  fold_scalar_kernel<<<1, 32, 0, st>>>(part, parts, nes_sq, 0);
  muon_normalize_kernel<<<ogrid(n), 256, 0, st>>>(
      static_cast<const float*>(g), static_cast<const float*>(m), static_cast<bf16*>(x0), n, beta,
      static_cast<const float*>(gnorm_sq), clip, gscale, nes_sq);
  return cudaGetLastError();
}

// The same over `nb` matrices of `n` elements each, back to back in g, m and x0: three
// launches for the whole shape class instead of three per matrix, bit-identical results.
// scratch: nb * (pb_sumsq_nparts(n) + 1) floats.
PB_API int pb_muon_prepare_batched(const void* g, void* m, void* x0, long n, int nb, float beta,
                                   const void* gnorm_sq, float clip, float gscale, void* scratch,
                                   cudaStream_t st) {
  if (nb <= 0 || n <= 0) return PB_BAD_ARG;
  const int parts = pb_sumsq_nparts(n);
  float* part = static_cast<float*>(scratch);
  float* nes_sq = part + static_cast<long>(parts) * nb;
  for (int j0 = 0; j0 < nb; j0 += 32768) {      // gridDim.y limit is 65535
    const int cnt = nb - j0 < 32768 ? nb - j0 : 32768;
    const float* gj = static_cast<const float*>(g) + static_cast<long>(j0) * n;
    float* mj = static_cast<float*>(m) + static_cast<long>(j0) * n;
    bf16* xj = static_cast<bf16*>(x0) + static_cast<long>(j0) * n;
    float* pj = part + static_cast<long>(j0) * parts;
    muon_momentum_kernel<<<dim3(parts, cnt), 256, 0, st>>>(gj, mj, n, beta,
                                                         static_cast<const float*>(gnorm_sq),
                                                         clip, gscale, pj);
    fold_rows_kernel<<<cnt, 32, 0, st>>>(pj, parts, nes_sq + j0);
    muon_normalize_kernel<<<dim3(ogrid(n), cnt), 256, 0, st>>>(
        gj, mj, xj, n, beta, static_cast<const float*>(gnorm_sq), clip, gscale, nes_sq + j0);
  }
  return cudaGetLastError();
}

PB_API int pb_muon_apply(void* p, const void* o, void* p_lp, long n, float lr, float scale,
                         float wd, cudaStream_t st) {
  muon_apply_kernel<<<ogrid(n), 256, 0, st>>>(static_cast<float*>(p), static_cast<const bf16*>(o),
                                              static_cast<bf16*>(p_lp), n, lr, scale, wd);
  return cudaGetLastError();
}

// See qk_clip_rescale_kernel. rows / row0 select a row range of the projection (a row shard);
// `group` = query heads per key head; is_k = 1 for the key projection (heads = key heads).
PB_API int pb_qk_clip_rescale(void* master, void* lp, int rows, int cols, int dh, int group,
                              int n_q_heads, int is_k, long row0, const void* max_logit,
                              float tau, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (cols <= 0 || dh <= 0 || group <= 0 || n_q_heads <= 0 || tau <= 0.f || max_logit == nullptr ||
      (master == nullptr && lp == nullptr))
    return PB_BAD_ARG;
  qk_clip_rescale_kernel<<<rows, 256, 0, st>>>(static_cast<float*>(master), static_cast<bf16*>(lp),
                                               rows, cols, dh, group, n_q_heads, is_k, row0,
                                               static_cast<const float*>(max_logit), tau);
  return cudaGetLastError();
}

// out[0] (uint64, zeroed here) = checksum of n 32-bit words at x.
PB_API int pb_checksum_u32(const void* x, long n, void* out, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(out, 0, 8, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (n > 0)
    checksum_u32_kernel<<<ogrid(n), 256, 0, st>>>(static_cast<const uint32_t*>(x), n,
                                                  static_cast<unsigned long long*>(out));
  return cudaGetLastError();
}

PB_API int pb_cast_f32_bf16(const void* x, void* y, long n, float scale, cudaStream_t st) {
  cast_f32_bf16_kernel<<<ogrid(n), 256, 0, st>>>(static_cast<const float*>(x),
                                                 static_cast<bf16*>(y), n, scale);
  return cudaGetLastError();
}
PB_API int pb_axpy_bf16_f32(const void* x, void* acc, long n, float scale, cudaStream_t st) {
  axpy_bf16_f32_kernel<<<ogrid(n), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                 static_cast<float*>(acc), n, scale);
  return cudaGetLastError();
}
PB_API int pb_transpose_bf16(const void* in, void* out, int batch, int rows, int cols,
                             cudaStream_t st) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
  transpose_bf16_kernel<<<grid, dim3(32, 8), 0, st>>>(static_cast<const bf16*>(in),
                                                      static_cast<bf16*>(out), rows, cols);
  return cudaGetLastError();
}
