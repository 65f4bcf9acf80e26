// Latent Jacobi step (one sweep of the in-sequence latent-slot solve), the memory-bound parts.
//
//   rows      <- hidden[b, slot_start - 1 + j, :]                 (gather, j < K)
//   a         <- silu(rows W1^T) W2^T                             (tcgen05 GEMMs, gemm.cu)
//   new[b, s] <- embeds[b, s]           for s outside the slots   (copy, fused with ...)
//   new[b, slot_start + j] <- rmsnorm(a[b K + j]) * w             (... normalise + scatter)
//
// The copy of the embeddings is needed anyway (the sweep must not overwrite its input), so the
// normalisation and the scatter ride along in that one pass over [B, S, d].
// Reference semantics: model/__init__.py _apply_latent_adapter (silu MLP + rms_norm); the
// in-sequence slot layout is this library's own.
#include "common.cuh"

namespace pb {

// one warp per gathered row; d % 8 == 0
__global__ void latent_gather_kernel(const bf16* __restrict__ src, bf16* __restrict__ rows, int B,
                                     int S, int d, int start, int K) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= B * K) return;
  const int b = w / K, j = w % K;
  const bf16x8* s = reinterpret_cast<const bf16x8*>(src + (static_cast<size_t>(b) * S + start + j) * d);
  bf16x8* o = reinterpret_cast<bf16x8*>(rows + static_cast<size_t>(w) * d);
  for (int i = lane; i < d / 8; i += 32) o[i] = s[i];
}

// rows (B*K, d) added into / written to positions start .. start+K of a zero or existing tensor
__global__ void latent_scatter_kernel(const bf16* __restrict__ rows, bf16* __restrict__ dst, int B,
                                      int S, int d, int start, int K) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= B * K) return;
  const int b = w / K, j = w % K;
  const bf16x8* s = reinterpret_cast<const bf16x8*>(rows + static_cast<size_t>(w) * d);
  bf16x8* o = reinterpret_cast<bf16x8*>(dst + (static_cast<size_t>(b) * S + start + j) * d);
  for (int i = lane; i < d / 8; i += 32) o[i] = s[i];
}

// one warp per sequence position: copy, or normalise the matching adapter row
__global__ void latent_norm_scatter_kernel(const bf16* __restrict__ a, const float* __restrict__ w,
                                           const bf16* __restrict__ embeds, bf16* __restrict__ out,
                                           float* __restrict__ rstd, int B, int S, int d, int start,
                                           int K, float eps) {
  const long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long>(B) * S) return;
  const int b = static_cast<int>(row / S), s = static_cast<int>(row % S);
  bf16x8* o = reinterpret_cast<bf16x8*>(out + row * d);
  if (s < start || s >= start + K) {
    const bf16x8* e = reinterpret_cast<const bf16x8*>(embeds + row * d);
    for (int i = lane; i < d / 8; i += 32) o[i] = e[i];
    return;
  }
  const int r = b * K + (s - start);
  const bf16x8* src = reinterpret_cast<const bf16x8*>(a + static_cast<size_t>(r) * d);
  float ss = 0.f;
  for (int i = lane; i < d / 8; i += 32) {
    float f[8];
    unpack8(src[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
  }
  ss = warp_sum(ss);
  const float rs = rsqrtf(ss / d + eps);
  if (lane == 0) rstd[r] = rs;
  for (int i = lane; i < d / 8; i += 32) {
    float f[8];
    unpack8(src[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = f[k] * rs * w[8 * i + k];
    o[i] = pack8(f);
  }
}

__global__ void silu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long n8) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = f[k] * sigmoidf_(f[k]);
    reinterpret_cast<bf16x8*>(y)[i] = pack8(f);
  }
}
__global__ void silu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                bf16* __restrict__ dx, long n8) {
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float f[8], g[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], f);
    unpack8(reinterpret_cast<const bf16x8*>(dy)[i], g);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = sigmoidf_(f[k]);
      g[k] *= s * (1.f + f[k] * (1.f - s));
    }
    reinterpret_cast<bf16x8*>(dx)[i] = pack8(g);
  }
}

}  // namespace pb

using namespace pb;

static bool bad_slots(int B, int S, int d, int start, int K) {
  return B <= 0 || S <= 0 || d <= 0 || d % 8 != 0 || K <= 0 || start < 0 || start + K > S;
}

// rows[b K + j, :] = src[b, start + j, :]   (src: [B, S, d] bf16)
PB_API int pb_latent_gather(const void* src, void* rows, int B, int S, int d, int start, int K,
                            cudaStream_t st) {
  if (bad_slots(B, S, d, start, K)) return PB_BAD_ARG;
  latent_gather_kernel<<<(B * K * 32 + 255) / 256, 256, 0, st>>>(
      static_cast<const bf16*>(src), static_cast<bf16*>(rows), B, S, d, start, K);
  return static_cast<int>(cudaGetLastError());
}

// dst[b, start + j, :] = rows[b K + j, :]   (other positions of dst are left as they are)
PB_API int pb_latent_scatter(const void* rows, void* dst, int B, int S, int d, int start, int K,
                             cudaStream_t st) {
  if (bad_slots(B, S, d, start, K)) return PB_BAD_ARG;
  latent_scatter_kernel<<<(B * K * 32 + 255) / 256, 256, 0, st>>>(
      static_cast<const bf16*>(rows), static_cast<bf16*>(dst), B, S, d, start, K);
  return static_cast<int>(cudaGetLastError());
}

// out = embeds with positions start .. start+K replaced by rmsnorm(a) * w; rstd: fp32 [B K]
PB_API int pb_latent_norm_scatter(const void* a, const void* w, const void* embeds, void* out,
                                  void* rstd, int B, int S, int d, int start, int K, float eps,
                                  cudaStream_t st) {
  if (bad_slots(B, S, d, start, K)) return PB_BAD_ARG;
  const long warps = static_cast<long>(B) * S;
  latent_norm_scatter_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, st>>>(
      static_cast<const bf16*>(a), static_cast<const float*>(w), static_cast<const bf16*>(embeds),
      static_cast<bf16*>(out), static_cast<float*>(rstd), B, S, d, start, K, eps);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_silu_fwd(const void* x, void* y, long n, cudaStream_t st) {
  if (n <= 0 || n % 8 != 0) return PB_BAD_ARG;
  const long n8 = n / 8;
  const int grid = static_cast<int>(n8 / 256 + 1 < 148 * 8 ? n8 / 256 + 1 : 148 * 8);
  silu_fwd_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<bf16*>(y), n8);
  return static_cast<int>(cudaGetLastError());
}
PB_API int pb_silu_bwd(const void* dy, const void* x, void* dx, long n, cudaStream_t st) {
  if (n <= 0 || n % 8 != 0) return PB_BAD_ARG;
  const long n8 = n / 8;
  const int grid = static_cast<int>(n8 / 256 + 1 < 148 * 8 ? n8 / 256 + 1 : 148 * 8);
  silu_bwd_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(dy), static_cast<const bf16*>(x),
                                        static_cast<bf16*>(dx), n8);
  return static_cast<int>(cudaGetLastError());
}
