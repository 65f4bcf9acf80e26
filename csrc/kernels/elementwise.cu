// HBM-bound fused elementwise / row kernels of the training step (sm_100a):
// RMSNorm (+residual) fwd/bwd, RoPE, SwiGLU, L2-norm of q/k heads, and the
// fused soft-cap + cross-entropy forward/backward over vocabulary rows.
//
// Math follows the reference model: rms_norm (model/__init__.py:305-310),
// _apply_rope interleaved pairs (model/__init__.py:337-359), _swiglu
// (model/__init__.py:547-549), _l2_normalize (model/__init__.py:201-203),
// soft_cap + cross_entropy (train/__init__.py:561-604).
#include <cuda_fp8.h>

#include "common.cuh"

namespace pb {

// ---------------------------------------------------------------------------
// RMSNorm forward. One warp per row. Optional residual add:
//   h = x (+ res);  y = h * rsqrt(mean(h^2) + eps) * w
// h_out (may alias x) receives h when res != nullptr.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128) rmsnorm_fwd_kernel(const bf16* __restrict__ x,
                                                          const bf16* __restrict__ res,
                                                          const float* __restrict__ w,
                                                          bf16* __restrict__ y, bf16* h_out,
                                                          float* __restrict__ rstd_out, int rows,
                                                          int d, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = static_cast<size_t>(row) * d;
  const int nvec = d >> 3;
  float ss = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    float f[8];
    bf16x8 p = *reinterpret_cast<const bf16x8*>(x + base + v * 8);
    unpack8(p, f);
    if (res != nullptr) {
      float g[8];
      bf16x8 q = *reinterpret_cast<const bf16x8*>(res + base + v * 8);
      unpack8(q, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      p = pack8(f);
      unpack8(p, f);  // the norm sees the rounded residual stream
      *reinterpret_cast<bf16x8*>(h_out + base + v * 8) = p;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  const bf16* src = (res != nullptr) ? h_out : x;
  for (int v = lane; v < nvec; v += 32) {
    float f[8];
    bf16x8 p = *reinterpret_cast<const bf16x8*>(src + base + v * 8);
    unpack8(p, f);
    const float4 w0 = *reinterpret_cast<const float4*>(w + v * 8);
    const float4 w1 = *reinterpret_cast<const float4*>(w + v * 8 + 4);
    f[0] *= rstd * w0.x; f[1] *= rstd * w0.y; f[2] *= rstd * w0.z; f[3] *= rstd * w0.w;
    f[4] *= rstd * w1.x; f[5] *= rstd * w1.y; f[6] *= rstd * w1.z; f[7] *= rstd * w1.w;
    *reinterpret_cast<bf16x8*>(y + base + v * 8) = pack8(f);
  }
}

// d = 256 NV (NV <= 8): the row lives in registers between the two passes and every load of the
// row is issued before the first use. Same arithmetic as rmsnorm_fwd_kernel.
// q_out / s_out (may be null): the normalised row also leaves as e4m3 with one fp32 scale per
// 128 columns, q [rows, d] bytes and s [d / 128, rows] floats, the operand layout of the
// block-scaled FP8 GEMM. The bf16-rounded values are what is quantised (scale = amax / 448, 1 for
// an all-zero block, true division), so the bytes equal those of the stand-alone row quantiser
// run over y. A 128-column block is the 8 elements of 16 consecutive lanes.
__device__ __forceinline__ uint32_t rms_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}
template <int NV, bool Q>
__global__ void __launch_bounds__(128) rmsnorm_fwd_reg_kernel(
    const bf16* __restrict__ x, const bf16* __restrict__ res, const float* __restrict__ w,
    bf16* __restrict__ y, bf16* h_out, float* __restrict__ rstd_out, int rows, float eps,
    uint8_t* __restrict__ q_out, float* __restrict__ s_out) {
  constexpr int d = NV * 256;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = static_cast<size_t>(row) * d;
  bf16x8 px[NV], pr[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    px[v] = *reinterpret_cast<const bf16x8*>(x + base + (v * 32 + lane) * 8);
    if (res != nullptr) pr[v] = *reinterpret_cast<const bf16x8*>(res + base + (v * 32 + lane) * 8);
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    float f[8];
    unpack8(px[v], f);
    if (res != nullptr) {
      float g[8];
      unpack8(pr[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      px[v] = pack8(f);
      unpack8(px[v], f);  // the norm sees the rounded residual stream
      *reinterpret_cast<bf16x8*>(h_out + base + (v * 32 + lane) * 8) = px[v];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(d) + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int col = (v * 32 + lane) * 8;
    float f[8];
    unpack8(px[v], f);
    const float4 w0 = *reinterpret_cast<const float4*>(w + col);
    const float4 w1 = *reinterpret_cast<const float4*>(w + col + 4);
    f[0] *= rstd * w0.x; f[1] *= rstd * w0.y; f[2] *= rstd * w0.z; f[3] *= rstd * w0.w;
    f[4] *= rstd * w1.x; f[5] *= rstd * w1.y; f[6] *= rstd * w1.z; f[7] *= rstd * w1.w;
    const bf16x8 out = pack8(f);
    *reinterpret_cast<bf16x8*>(y + base + col) = out;
    if (Q) {
      unpack8(out, f);                      // quantise what was stored
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = amax > 0.f ? amax / 448.f : 1.f;
      uint2 pk;
      pk.x = rms_e4m3x4(__fdiv_rn(f[0], scale), __fdiv_rn(f[1], scale), __fdiv_rn(f[2], scale), __fdiv_rn(f[3], scale));
      pk.y = rms_e4m3x4(__fdiv_rn(f[4], scale), __fdiv_rn(f[5], scale), __fdiv_rn(f[6], scale), __fdiv_rn(f[7], scale));
      *reinterpret_cast<uint2*>(q_out + base + col) = pk;
      if ((lane & 15) == 0) s_out[static_cast<size_t>(col >> 7) * rows + row] = scale;
    }
  }
}

// ---------------------------------------------------------------------------
// RMSNorm backward, d <= 2048. Persistent: a CTA of 256 threads walks groups of four rows with
// a grid stride; thread t owns columns [8 t, 8 t + 8) of every row, so its share of dw stays
// in eight registers for the whole kernel and is written once, as row blockIdx.x of
// `dw_partial`. The loads of all four rows are issued before the first use, and the four row
// dots share one block reduction (one __syncthreads per group; the scratch is double-buffered).
//   xh = h * rstd;  g = dy * w;  dx = rstd * (g - xh * mean(g * xh)) (+ dres)
// A second kernel folds the partial rows in a fixed order (deterministic).
// ---------------------------------------------------------------------------
constexpr int RMS_BWD_ROWS = 4;
constexpr int RMS_BWD_SMEM = 2 * RMS_BWD_ROWS * 3 * 256 * 16;   // two groups x rows x {dy, h, dres} x 4 KB

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// The next group of rows is copied into shared memory (cp.async, each thread its own 16 bytes
// per row and tensor, so no barrier guards the data) while the current group is reduced, so the
// loads never drain at the per-group barrier.
__global__ void __launch_bounds__(256, 2) rmsnorm_bwd_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ h, const float* __restrict__ w,
    const float* __restrict__ rstd_in, const bf16* __restrict__ dres, bf16* __restrict__ dx,
    float* __restrict__ dw_partial, int rows, int d) {
  constexpr int R = RMS_BWD_ROWS;
  extern __shared__ __align__(16) uint8_t rms_stage[];   // [2][R][3][256] x 16 bytes
  __shared__ float red[2][R][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = threadIdx.x * 8;
  const bool on = col < d;
  float ww[8], acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { ww[i] = 0.f; acc[i] = 0.f; }
  if (on) {
    const float4 w0 = *reinterpret_cast<const float4*>(w + col);
    const float4 w1 = *reinterpret_cast<const float4*>(w + col + 4);
    ww[0] = w0.x; ww[1] = w0.y; ww[2] = w0.z; ww[3] = w0.w;
    ww[4] = w1.x; ww[5] = w1.y; ww[6] = w1.z; ww[7] = w1.w;
  }
  const float inv_d = 1.f / static_cast<float>(d);
  auto slot = [&](int buf, int r, int which) -> bf16x8* {
    return reinterpret_cast<bf16x8*>(rms_stage) + ((buf * R + r) * 3 + which) * 256 + threadIdx.x;
  };
  auto issue = [&](long row0, int buf) {
    if (on) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const long row = row0 + r;
        if (row < rows) {
          const size_t off = static_cast<size_t>(row) * d + col;
          cp_async_16(slot(buf, r, 0), dy + off);
          cp_async_16(slot(buf, r, 1), h + off);
          if (dres != nullptr) cp_async_16(slot(buf, r, 2), dres + off);
        }
      }
    }
    cp_async_commit();
  };
  const long stride = static_cast<long>(gridDim.x) * R;
  int buf = 0;
  long row0 = static_cast<long>(blockIdx.x) * R;
  if (row0 < rows) issue(row0, 0);
  for (; row0 < rows; row0 += stride) {
    if (row0 + stride < rows) {
      issue(row0 + stride, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    bf16x8 pdy[R], ph[R];
    float rs[R], dot[R];
    bool valid[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const long row = row0 + r;
      valid[r] = on && row < rows;
      rs[r] = row < rows ? rstd_in[row] : 0.f;
      dot[r] = 0.f;
      if (valid[r]) {
        pdy[r] = *slot(buf, r, 0);
        ph[r] = *slot(buf, r, 1);
        float a[8], b[8];
        unpack8(pdy[r], a);
        unpack8(ph[r], b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = b[i] * rs[r];
          dot[r] += a[i] * ww[i] * xhat;
          acc[i] += a[i] * xhat;
        }
      }
      dot[r] = warp_sum(dot[r]);
      if (lane == 0) red[buf][r][warp] = dot[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (!valid[r]) continue;
      float tot = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) tot += red[buf][r][k];
      tot *= inv_d;
      float a[8], b[8], o[8];
      unpack8(pdy[r], a);
      unpack8(ph[r], b);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rs[r] * (a[i] * ww[i] - b[i] * rs[r] * tot);
      if (dres != nullptr) {
        float q[8];
        unpack8(*slot(buf, r, 2), q);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += q[i];
      }
      *reinterpret_cast<bf16x8*>(dx + static_cast<size_t>(row0 + r) * d + col) = pack8(o);
    }
    buf ^= 1;
  }
  if (on) {
    float* out = dw_partial + static_cast<size_t>(blockIdx.x) * d + col;
    *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(out + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// Generic-width fallback (any d % 8 == 0): one CTA per row at a time, smem dw.
__global__ void __launch_bounds__(256) rmsnorm_bwd_generic_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ h, const float* __restrict__ w,
    const float* __restrict__ rstd_in, const bf16* __restrict__ dres, bf16* __restrict__ dx,
    float* __restrict__ dw_partial, int rows, int d) {
  extern __shared__ float sm[];  // [d] dw + 33 scratch
  float* sdw = sm;
  float* scratch = sm + d;
  for (int c = threadIdx.x; c < d; c += blockDim.x) sdw[c] = 0.f;
  __syncthreads();
  const float inv_d = 1.f / static_cast<float>(d);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * d;
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float xhat = bf16_to_f32(h[base + c]) * rstd;
      const float a = bf16_to_f32(dy[base + c]);
      dot += a * w[c] * xhat;
      sdw[c] += a * xhat;
    }
    dot = block_sum(dot, scratch) * inv_d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
      const float xhat = bf16_to_f32(h[base + c]) * rstd;
      float o = rstd * (bf16_to_f32(dy[base + c]) * w[c] - xhat * dot);
      if (dres != nullptr) o += bf16_to_f32(dres[base + c]);
      dx[base + c] = f32_to_bf16(o);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    dw_partial[static_cast<size_t>(blockIdx.x) * d + c] = sdw[c];
}

// dw[c] (+)= sum_p partial[p][c], p in increasing order.
__global__ void fold_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                     int nparts, int d, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<size_t>(p) * d + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ---------------------------------------------------------------------------
// RoPE, interleaved (even, odd) pairs, in place. x: [tokens, heads, D].
// pos[t] is the position of token t (nullptr: t % seq_len). rot_pairs pairs
// are rotated, the rest pass through. inverse != 0 applies the transpose.
// ---------------------------------------------------------------------------
__global__ void rope_kernel(bf16* __restrict__ x, const int* __restrict__ pos, long tokens,
                            int heads, int D, int rot_pairs, int seq_len, float base,
                            int inverse) {
  // One thread per (token, group of four pairs): the angles depend on the token and the pair
  // only, so sine and cosine are computed once and reused for every head of the token.
  const int vec_per_head = D >> 3;
  const int rot_vecs = (rot_pairs + 3) >> 2;          // vectors that hold a rotated pair
  const long total = tokens * rot_vecs;
  const float rot_dim = static_cast<float>(rot_pairs * 2);
  const float log2_base = log2f(base);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % rot_vecs);
    const long t = i / rot_vecs;
    const int pair0 = v * 4;
    const float p = pos != nullptr ? static_cast<float>(pos[t])
                                   : static_cast<float>(t % seq_len);
    float sn[4], cs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pr = pair0 + j;
      const float inv_freq = exp2f(-2.f * static_cast<float>(pr) / rot_dim * log2_base);
      float s_, c_;
      sincosf(p * inv_freq, &s_, &c_);
      if (inverse) s_ = -s_;
      if (pr >= rot_pairs) { s_ = 0.f; c_ = 1.f; }   // pass-through pair
      sn[j] = s_; cs[j] = c_;
    }
    bf16x8* ptr = reinterpret_cast<bf16x8*>(x) + (t * heads) * vec_per_head + v;
    int h = 0;
    for (; h + 4 <= heads; h += 4) {        // four heads' loads in flight
      bf16x8 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = ptr[static_cast<long>(h + u) * vec_per_head];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float f[8];
        unpack8(q[u], f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float e = f[2 * j], o = f[2 * j + 1];
          f[2 * j] = e * cs[j] - o * sn[j];
          f[2 * j + 1] = e * sn[j] + o * cs[j];
        }
        ptr[static_cast<long>(h + u) * vec_per_head] = pack8(f);
      }
    }
    for (; h < heads; ++h) {
      float f[8];
      unpack8(ptr[static_cast<long>(h) * vec_per_head], f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = f[2 * j], o = f[2 * j + 1];
        f[2 * j] = e * cs[j] - o * sn[j];
        f[2 * j + 1] = e * sn[j] + o * cs[j];
      }
      ptr[static_cast<long>(h) * vec_per_head] = pack8(f);
    }
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on a fused [rows, 2H] projection: out = silu(gu[:, :H]) * gu[:, H:]
// ---------------------------------------------------------------------------
// rows_dev (may be null): device-side row count; rows beyond it are left untouched. Buffers
// sized for a worst case (expert-parallel receive buffers) then cost only what is in use.
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long rows,
                                  int H, const int* __restrict__ rows_dev) {
  if (rows_dev != nullptr) rows = min(rows, static_cast<long>(*rows_dev));
  const int vph = H >> 3;
  const long total = rows * vph;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vph;
    const int c = static_cast<int>(i % vph) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * H + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * H + H + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * sigmoidf_(g[j]) * u[j];
    *reinterpret_cast<bf16x8*>(out + r * H + c) = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu,
                                  bf16* __restrict__ dgu, long rows, int H,
                                  const int* __restrict__ rows_dev) {
  if (rows_dev != nullptr) rows = min(rows, static_cast<long>(*rows_dev));
  const int vph = H >> 3;
  const long total = rows * vph;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / vph;
    const int c = static_cast<int>(i % vph) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * H + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * H + H + c), u);
    unpack8(*reinterpret_cast<const bf16x8*>(dout + r * H + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sigmoidf_(g[j]);
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    *reinterpret_cast<bf16x8*>(dgu + r * 2 * H + c) = pack8(dg);
    *reinterpret_cast<bf16x8*>(dgu + r * 2 * H + H + c) = pack8(du);
  }
}

// ---------------------------------------------------------------------------
// L2 normalisation of head vectors, in place. x: [nvec, D], one warp each.
//   xn = x / max(|x|, eps);   inv_norm[nvec] saved for the backward.
// Backward (in place on dxn): dx = inv * (dxn - xn * <xn, dxn>)
// (exact when |x| > eps; when clamped the projection term is dropped.)
// ---------------------------------------------------------------------------
__global__ void l2norm_fwd_kernel(bf16* __restrict__ x, float* __restrict__ inv_norm, long nvec,
                                  int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long vec = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (vec >= nvec) return;
  bf16* p = x + vec * D;
  float ss = 0.f;
  for (int c = lane * 4; c < D; c += 128) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(p + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(p + c + 2));
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
  }
  ss = warp_sum(ss);
  const float n = sqrtf(ss);
  const float inv = 1.f / fmaxf(n, eps);
  if (lane == 0) inv_norm[vec] = n > eps ? inv : -inv;  // sign marks the clamped case
  for (int c = lane * 4; c < D; c += 128) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(p + c));
    float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(p + c + 2));
    *reinterpret_cast<bf162*>(p + c) = __floats2bfloat162_rn(a.x * inv, a.y * inv);
    *reinterpret_cast<bf162*>(p + c + 2) = __floats2bfloat162_rn(b.x * inv, b.y * inv);
  }
}
__global__ void l2norm_bwd_kernel(bf16* __restrict__ dxn, const bf16* __restrict__ xn,
                                  const float* __restrict__ inv_norm, long nvec, int D) {
  const int lane = threadIdx.x & 31;
  const long vec = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (vec >= nvec) return;
  bf16* g = dxn + vec * D;
  const bf16* y = xn + vec * D;
  float dot = 0.f;
  for (int c = lane * 4; c < D; c += 128) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(g + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(g + c + 2));
    const float2 ya = __bfloat1622float2(*reinterpret_cast<const bf162*>(y + c));
    const float2 yb = __bfloat1622float2(*reinterpret_cast<const bf162*>(y + c + 2));
    dot += a.x * ya.x + a.y * ya.y + b.x * yb.x + b.y * yb.y;
  }
  dot = warp_sum(dot);
  float inv = inv_norm[vec];
  if (inv < 0.f) { inv = -inv; dot = 0.f; }
  for (int c = lane * 4; c < D; c += 128) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const bf162*>(g + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const bf162*>(g + c + 2));
    const float2 ya = __bfloat1622float2(*reinterpret_cast<const bf162*>(y + c));
    const float2 yb = __bfloat1622float2(*reinterpret_cast<const bf162*>(y + c + 2));
    *reinterpret_cast<bf162*>(g + c) =
        __floats2bfloat162_rn(inv * (a.x - ya.x * dot), inv * (a.y - ya.y * dot));
    *reinterpret_cast<bf162*>(g + c + 2) =
        __floats2bfloat162_rn(inv * (b.x - yb.x * dot), inv * (b.y - yb.y * dot));
  }
}

// D == 128 (the head width of every shipped model): half a warp per vector, one 16-byte access
// per lane, eight vectors per warp with all their loads issued before the first reduction.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__global__ void __launch_bounds__(256) l2norm128_fwd_kernel(bf16* __restrict__ x,
                                                            float* __restrict__ inv_norm,
                                                            long nvec, float eps) {
  const int lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
  const long wstride = static_cast<long>(gridDim.x) * (blockDim.x >> 5) * 8;
  for (long v0 = (blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5)) * 8;
       v0 < nvec; v0 += wstride) {
    bf16x8 p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long vec = v0 + j * 2 + half;
      if (vec < nvec) p[j] = *reinterpret_cast<const bf16x8*>(x + vec * 128 + l16 * 8);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long vec = v0 + j * 2 + half;
      float f[8];
      float ss = 0.f;
      if (vec < nvec) {
        unpack8(p[j], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
      ss = half_warp_sum(ss);
      if (vec < nvec) {
        const float n = sqrtf(ss);
        const float inv = 1.f / fmaxf(n, eps);
        if (l16 == 0) inv_norm[vec] = n > eps ? inv : -inv;
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= inv;
        *reinterpret_cast<bf16x8*>(x + vec * 128 + l16 * 8) = pack8(f);
      }
    }
  }
}
__global__ void __launch_bounds__(256) l2norm128_bwd_kernel(bf16* __restrict__ dxn,
                                                            const bf16* __restrict__ xn,
                                                            const float* __restrict__ inv_norm,
                                                            long nvec) {
  const int lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
  const long wstride = static_cast<long>(gridDim.x) * (blockDim.x >> 5) * 8;
  for (long v0 = (blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5)) * 8;
       v0 < nvec; v0 += wstride) {
    bf16x8 pg[4], py[4];
    float invs[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long vec = v0 + j * 2 + half;
      if (vec < nvec) {
        pg[j] = *reinterpret_cast<const bf16x8*>(dxn + vec * 128 + l16 * 8);
        py[j] = *reinterpret_cast<const bf16x8*>(xn + vec * 128 + l16 * 8);
        invs[j] = inv_norm[vec];
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long vec = v0 + j * 2 + half;
      float g[8], y[8];
      float dot = 0.f;
      if (vec < nvec) {
        unpack8(pg[j], g);
        unpack8(py[j], y);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += g[i] * y[i];
      }
      dot = half_warp_sum(dot);
      if (vec < nvec) {
        float inv = invs[j];
        if (inv < 0.f) { inv = -inv; dot = 0.f; }
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = inv * (g[i] - y[i] * dot);
        *reinterpret_cast<bf16x8*>(dxn + vec * 128 + l16 * 8) = pack8(g);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Fused soft-cap + cross-entropy, forward and backward in one launch.
// logits: [rows, V] bf16, overwritten with d(loss)/d(logits).
//   c = cap * tanh(x / cap)   (cap <= 0: c = x)
//   loss_row = wt[row] * (logsumexp(c) - c[target]);  wt carries mask / denom
//   dx = wt * (softmax(c) - onehot) * (1 - (c/cap)^2)
// One CTA per row; the row is read from HBM once and re-read from L2.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(512) softcap_ce_kernel(bf16* __restrict__ logits,
                                                         const int* __restrict__ targets,
                                                         const float* __restrict__ wt,
                                                         float* __restrict__ loss_rows,
                                                         float* __restrict__ lse_rows, int V,
                                                         float cap, int write_grad) {
  __shared__ float scratch[33];
  const long row = blockIdx.x;
  bf16* p = logits + row * V;
  const float w = wt[row];
  const int tgt = targets[row];
  const int nvec = V >> 3;
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  if (w == 0.f) {
    // masked row: zero gradient, zero loss, nothing to reduce
    if (write_grad) {
      bf16x8 z;
      for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) reinterpret_cast<bf16x8*>(p)[v] = z;
    }
    if (threadIdx.x == 0) {
      loss_rows[row] = 0.f;
      if (lse_rows != nullptr) lse_rows[row] = 0.f;
    }
    return;
  }
  float shift;
  if (cap > 0.f) {
    shift = cap;  // capped logits are bounded by cap: no max pass needed
  } else {
    float m = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8(reinterpret_cast<const bf16x8*>(p)[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, f[i]);
    }
    shift = block_max(m, scratch);
  }
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(p)[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float c = cap > 0.f ? cap * tanh_fast(f[i] * inv_cap) : f[i];
      s += __expf(c - shift);
    }
  }
  s = block_sum(s, scratch);
  // a target outside the vocabulary would read (and below, write) outside the row
  const float xt = PB_BOUNDS_OK(PB_K_SOFTCAP_CE, tgt, V) ? bf16_to_f32(p[tgt]) : 0.f;
  const float ct = cap > 0.f ? cap * tanh_fast(xt * inv_cap) : xt;
  const float lse = __logf(s) + shift;
  if (threadIdx.x == 0) {
    loss_rows[row] = w * (lse - ct);
    if (lse_rows != nullptr) lse_rows[row] = lse;
  }
  if (!write_grad) return;
  const float inv_s = 1.f / s;
  __syncthreads();  // the target element is read above before anyone overwrites it
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(p)[v], f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float t = cap > 0.f ? tanh_fast(f[i] * inv_cap) : 0.f;
      const float c = cap > 0.f ? cap * t : f[i];
      float g = __expf(c - shift) * inv_s;
      if (v * 8 + i == tgt) g -= 1.f;
      g *= w;
      if (cap > 0.f) g *= (1.f - t * t);
      f[i] = g;
    }
    reinterpret_cast<bf16x8*>(p)[v] = pack8(f);
  }
}

// out[i] = sigmoid(x[i]) (bf16 -> bf16), dx = dy * s * (1 - s)
__global__ void sigmoid_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long n) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x)
    y[i] = f32_to_bf16(sigmoidf_(bf16_to_f32(x[i])));
}

static inline int grid_for(long total, int block, int cap = 148 * 16) {
  long g = (total + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace pb

using namespace pb;

// 1 when the library was built with -DPB_DEBUG_BOUNDS.
PB_API int pb_debug_bounds_enabled() {
#ifdef PB_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// Readers of the per-file violation records: pb_debug_bounds_read_<file>(out4), out4 (host, four
// 64-bit values) = {kernel id, violations since the last read, index, limit} of the first recorded
// violation of that file's kernels; the call clears the record and synchronises the device.
PB_DEFINE_BOUNDS_READER(elementwise)

static int rmsnorm_fwd_impl(const void* x, const void* res, const void* w, void* y, void* h_out,
                            void* rstd, void* q, void* scales, int rows, int d, float eps,
                            cudaStream_t st);

PB_API int pb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out,
                          void* rstd, int rows, int d, float eps, cudaStream_t st) {
  return rmsnorm_fwd_impl(x, res, w, y, h_out, rstd, nullptr, nullptr, rows, d, eps, st);
}

// The same with the FP8 image of y for the GEMM that follows: q [rows, d] e4m3 bytes, scales
// [d / 128, rows] fp32. d a multiple of 256, at most 2048 (the register-resident kernel).
PB_API int pb_rmsnorm_fwd_fp8(const void* x, const void* res, const void* w, void* y, void* h_out,
                              void* rstd, void* q, void* scales, int rows, int d, float eps,
                              cudaStream_t st) {
  if (q == nullptr || scales == nullptr || d % 256 != 0 || d > 2048) return PB_BAD_ARG;
  return rmsnorm_fwd_impl(x, res, w, y, h_out, rstd, q, scales, rows, d, eps, st);
}

static int rmsnorm_fwd_impl(const void* x, const void* res, const void* w, void* y, void* h_out,
                            void* rstd, void* q, void* scales, int rows, int d, float eps,
                            cudaStream_t st) {
  if (d % 8 != 0 || rows <= 0) return PB_BAD_ARG;
  const int wpb = 4;
  if (d % 256 == 0 && d <= 2048) {
    uint8_t* q_ = static_cast<uint8_t*>(q);
    float* sc_ = static_cast<float*>(scales);
    const bf16* x_ = static_cast<const bf16*>(x);
    const bf16* r_ = static_cast<const bf16*>(res);
    const float* w_ = static_cast<const float*>(w);
    bf16* y_ = static_cast<bf16*>(y);
    bf16* h_ = static_cast<bf16*>(h_out);
    float* s_ = static_cast<float*>(rstd);
    const int grid = (rows + wpb - 1) / wpb;
    switch (d / 256) {
#define PB_CASE(NV)                                                                              \
  case NV:                                                                                       \
    if (q_ != nullptr)                                                                           \
      rmsnorm_fwd_reg_kernel<NV, true><<<grid, wpb * 32, 0, st>>>(x_, r_, w_, y_, h_, s_, rows,  \
                                                                  eps, q_, sc_);                 \
    else                                                                                         \
      rmsnorm_fwd_reg_kernel<NV, false><<<grid, wpb * 32, 0, st>>>(x_, r_, w_, y_, h_, s_, rows, \
                                                                   eps, nullptr, nullptr);       \
    break;
      PB_CASE(1) PB_CASE(2) PB_CASE(3) PB_CASE(4) PB_CASE(5) PB_CASE(6) PB_CASE(7) PB_CASE(8)
#undef PB_CASE
    }
    return cudaGetLastError();
  }
  rmsnorm_fwd_kernel<<<(rows + wpb - 1) / wpb, wpb * 32, 0, st>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(res), static_cast<const float*>(w),
      static_cast<bf16*>(y), static_cast<bf16*>(h_out), static_cast<float*>(rstd), rows, d, eps);
  return cudaGetLastError();
}

// Number of partial rows rmsnorm_bwd writes (scratch must hold that many x d floats).
PB_API int pb_rmsnorm_bwd_nparts(int rows, int d) {
  const bool cols = d <= 2048;              // the column-owner kernel: two CTAs per SM
  int g = cols ? 148 * 2 : 148 * 4;
  const int per = cols ? RMS_BWD_ROWS : 1;
  const int need = (rows + per - 1) / per;
  return need < g ? (need < 1 ? 1 : need) : g;
}

PB_API int pb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const void* rstd,
                          const void* dres, void* dx, void* dw, void* scratch, int accumulate,
                          int rows, int d, cudaStream_t st) {
  if (d % 8 != 0 || rows <= 0) return PB_BAD_ARG;
  const int grid = pb_rmsnorm_bwd_nparts(rows, d);
  const bf16* dy_ = static_cast<const bf16*>(dy);
  const bf16* h_ = static_cast<const bf16*>(h);
  const float* w_ = static_cast<const float*>(w);
  const float* r_ = static_cast<const float*>(rstd);
  const bf16* dr_ = static_cast<const bf16*>(dres);
  bf16* dx_ = static_cast<bf16*>(dx);
  float* part = static_cast<float*>(scratch);
  if (d <= 2048) {
    static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
    if (attr_once.need()) {
      cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           RMS_BWD_SMEM);
      attr_once.done();
    }
    rmsnorm_bwd_kernel<<<grid, 256, RMS_BWD_SMEM, st>>>(dy_, h_, w_, r_, dr_, dx_, part, rows, d);
  } else {
    const size_t smem = (d + 33) * sizeof(float);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(rmsnorm_bwd_generic_kernel,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    rmsnorm_bwd_generic_kernel<<<grid, 256, smem, st>>>(dy_, h_, w_, r_, dr_, dx_, part, rows, d);
  }
  fold_partials_kernel<<<(d + 255) / 256, 256, 0, st>>>(part, static_cast<float*>(dw), grid, d,
                                                        accumulate);
  return cudaGetLastError();
}

PB_API int pb_rope(void* x, const void* pos, long tokens, int heads, int D, int rot_pairs,
                   int seq_len, float base, int inverse, cudaStream_t st) {
  if (D % 8 != 0) return PB_BAD_ARG;
  const long total = tokens * ((rot_pairs + 3) / 4);
  if (total <= 0) return 0;
  rope_kernel<<<grid_for(total, 128), 128, 0, st>>>(static_cast<bf16*>(x),
                                                    static_cast<const int*>(pos), tokens, heads,
                                                    D, rot_pairs, seq_len, base, inverse);
  return cudaGetLastError();
}

PB_API int pb_swiglu_fwd(const void* gu, void* out, long rows, int H, cudaStream_t st) {
  if (H % 8 != 0) return PB_BAD_ARG;
  swiglu_fwd_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, st>>>(
      static_cast<const bf16*>(gu), static_cast<bf16*>(out), rows, H, nullptr);
  return cudaGetLastError();
}
// The same over the first min(rows, *rows_dev) rows (rows_dev: a device int).
PB_API int pb_swiglu_fwd_dyn(const void* gu, void* out, long rows, int H, const int* rows_dev,
                             cudaStream_t st) {
  if (H % 8 != 0) return PB_BAD_ARG;
  swiglu_fwd_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, st>>>(
      static_cast<const bf16*>(gu), static_cast<bf16*>(out), rows, H, rows_dev);
  return cudaGetLastError();
}
PB_API int pb_swiglu_bwd_dyn(const void* dout, const void* gu, void* dgu, long rows, int H,
                             const int* rows_dev, cudaStream_t st) {
  if (H % 8 != 0) return PB_BAD_ARG;
  swiglu_bwd_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, st>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(gu), static_cast<bf16*>(dgu), rows,
      H, rows_dev);
  return cudaGetLastError();
}

// dst[0 : n) = src[0 : n) rows of row_bytes each, n = min(max_rows, *rows_dev): a copy of the
// part of a worst-case-sized buffer that is in use (16-byte vectors; row_bytes % 16 == 0).
__global__ void __launch_bounds__(256) copy_rows_dyn_kernel(const uint4* __restrict__ src,
                                                            uint4* __restrict__ dst, long vec_per_row,
                                                            long max_rows,
                                                            const int* __restrict__ rows_dev) {
  const long rows = min(max_rows, static_cast<long>(*rows_dev));
  const long total = rows * vec_per_row;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  for (; i + 3 * stride < total; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < total; i += stride) dst[i] = src[i];
}
PB_API int pb_copy_rows_dyn(const void* src, void* dst, long row_bytes, long max_rows,
                            const int* rows_dev, cudaStream_t st) {
  if (row_bytes <= 0 || row_bytes % 16 != 0 || max_rows <= 0 || rows_dev == nullptr ||
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) != 0)
    return PB_BAD_ARG;
  copy_rows_dyn_kernel<<<grid_for(max_rows * (row_bytes / 16), 256 * 4), 256, 0, st>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), row_bytes / 16, max_rows, rows_dev);
  return cudaGetLastError();
}
PB_API int pb_swiglu_bwd(const void* dout, const void* gu, void* dgu, long rows, int H,
                         cudaStream_t st) {
  if (H % 8 != 0) return PB_BAD_ARG;
  swiglu_bwd_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, st>>>(
      static_cast<const bf16*>(dout), static_cast<const bf16*>(gu), static_cast<bf16*>(dgu), rows,
      H, nullptr);
  return cudaGetLastError();
}

PB_API int pb_l2norm_fwd(void* x, void* inv_norm, long nvec, int D, float eps, cudaStream_t st) {
  if (D % 4 != 0) return PB_BAD_ARG;
  if (D == 128 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const long warps = (nvec + 7) / 8;
    l2norm128_fwd_kernel<<<grid_for((warps + 7) / 8, 1, 148 * 8), 256, 0, st>>>(
        static_cast<bf16*>(x), static_cast<float*>(inv_norm), nvec, eps);
    return cudaGetLastError();
  }
  const int wpb = 8;
  l2norm_fwd_kernel<<<static_cast<unsigned>((nvec + wpb - 1) / wpb), wpb * 32, 0, st>>>(
      static_cast<bf16*>(x), static_cast<float*>(inv_norm), nvec, D, eps);
  return cudaGetLastError();
}
PB_API int pb_l2norm_bwd(void* dxn, const void* xn, const void* inv_norm, long nvec, int D,
                         cudaStream_t st) {
  if (D % 4 != 0) return PB_BAD_ARG;
  if (D == 128 && ((reinterpret_cast<uintptr_t>(dxn) | reinterpret_cast<uintptr_t>(xn)) & 15) == 0) {
    const long warps = (nvec + 7) / 8;
    l2norm128_bwd_kernel<<<grid_for((warps + 7) / 8, 1, 148 * 8), 256, 0, st>>>(
        static_cast<bf16*>(dxn), static_cast<const bf16*>(xn),
        static_cast<const float*>(inv_norm), nvec);
    return cudaGetLastError();
  }
  const int wpb = 8;
  l2norm_bwd_kernel<<<static_cast<unsigned>((nvec + wpb - 1) / wpb), wpb * 32, 0, st>>>(
      static_cast<bf16*>(dxn), static_cast<const bf16*>(xn),
      static_cast<const float*>(inv_norm), nvec, D);
  return cudaGetLastError();
}

PB_API int pb_softcap_ce(void* logits, const void* targets, const void* wt, void* loss_rows,
                         void* lse_rows, long rows, int V, float cap, int write_grad,
                         cudaStream_t st) {
  if (V % 8 != 0 || rows <= 0) return PB_BAD_ARG;
  softcap_ce_kernel<<<static_cast<unsigned>(rows), 512, 0, st>>>(
      static_cast<bf16*>(logits), static_cast<const int*>(targets),
      static_cast<const float*>(wt), static_cast<float*>(loss_rows),
      static_cast<float*>(lse_rows), V, cap, write_grad);
  return cudaGetLastError();
}

PB_API int pb_sigmoid(const void* x, void* y, long n, cudaStream_t st) {
  sigmoid_fwd_kernel<<<grid_for(n, 256), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                       static_cast<bf16*>(y), n);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the path where they need
// the kernel: code running inside a memory pool that owns the whole device, a
// runtime that pre-plans every byte before it starts (inference servers, real-time
// loops), or a plug-in that is only handed its input and output buffers. The
// regular entry point pb_rmsnorm_bwd needs a caller-provided scratch buffer for the
// per-CTA partial sums of dw; this variant keeps that scratch in a fixed
// file-scope device array instead, so the caller passes inputs and outputs only.
//
// Limits and rules (also stated in pb200_noalloc.h):
//  * d <= PB_NOALLOC_MAX_D (2048) and d % 8 == 0; larger widths are rejected with
//    PB_BAD_ARG and nothing is launched.
//  * The array (PB_NOALLOC_MAX_PARTS x PB_NOALLOC_MAX_D floats, about 2.3 MiB) is
//    part of the library image: every GPU that loads the library holds it until
//    the process exits.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current). Make that first call before
//    any stream capture begins on the device.
//  * All calls on a device share the one array. The kernel overwrites every partial
//    row it later folds, so nothing needs clearing between calls, but two calls
//    that overlap on the GPU (different streams) race on it: serialise them.
// ---------------------------------------------------------------------------
#define PB_NOALLOC_MAX_D 2048
// widths up to 2048 run the column-owner kernel, whose grid is at most two CTAs per SM
#define PB_NOALLOC_MAX_PARTS (148 * 2)
#define PB_NOALLOC_MAX_DEVICES 64

static __device__ __align__(256) float g_noalloc_rms_partials[PB_NOALLOC_MAX_PARTS * PB_NOALLOC_MAX_D];

// Host-side cache of the array's device address, one slot per device ordinal.
// (In host code the symbol name is only a handle; the address must be queried.)
static float* g_noalloc_addr[PB_NOALLOC_MAX_DEVICES] = {nullptr};

PB_API int pb_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const void* rstd,
                                  const void* dres, void* dx, void* dw, int accumulate, int rows,
                                  int d, cudaStream_t st) {
  if (rows <= 0 || d <= 0 || d % 8 != 0 || d > PB_NOALLOC_MAX_D) return PB_BAD_ARG;
  const int nparts = pb_rmsnorm_bwd_nparts(rows, d);
  if (nparts > PB_NOALLOC_MAX_PARTS) return PB_BAD_ARG;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= PB_NOALLOC_MAX_DEVICES) return PB_BAD_ARG;
  float* scratch = __atomic_load_n(&g_noalloc_addr[dev], __ATOMIC_ACQUIRE);
  if (scratch == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_rms_partials);
    if (e != cudaSuccess) return static_cast<int>(e);
    scratch = static_cast<float*>(ptr);
    __atomic_store_n(&g_noalloc_addr[dev], scratch, __ATOMIC_RELEASE);
  }
  return pb_rmsnorm_bwd(dy, h, w, rstd, dres, dx, dw, scratch, accumulate, rows, d, st);
}

PB_API int pb_rmsnorm_bwd_noalloc_max_d() { return PB_NOALLOC_MAX_D; }
