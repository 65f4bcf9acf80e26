// Block-scaled FP8 (e4m3) GEMM on tcgen05 and the quantisers that feed it (sm_100a).
//
//   C[M, N] (bf16) = sum over K-blocks kb of  sa[kb, m] * sb[n / 128, kb] * (Aq_kb . Bq_kb^T)
//
// Aq [M, K] e4m3 with one fp32 scale per row per 128 contraction elements (stored
// [K / 128, M] so a warp reads consecutive rows), Bq [N, K] e4m3 with one scale per
// 128 x 128 block. Exactly the arithmetic of quantise -> dequantise -> fp32 matmul, with the
// dequantisation applied to the 128-deep partial products instead of to the operands.
//
// One CTA per SM, persistent over 128 x 256 output tiles:
//   warp 0   TMA producer: per K-block a 128 x 128 B tile of A and a 256 x 128 B tile of B
//            (128 bytes per row = one swizzle atom), 4-stage ring
//   warp 1   MMA issuer: four kind::f8f6f4 MMAs (M 128, N 256, K 32) per K-block into one of
//            two 256-column tensor-memory accumulators, fresh (not accumulated) per K-block
//   warps 2-9  promotion + epilogue, two groups of four warps, one per 128-column half (one B
//            scale each): every thread owns one output row of its half; per K-block it reads
//            the 128 partial sums from tensor memory (two 64-column batches per wait), scales
//            them by sa * sb and adds them to 128 fp32 registers with packed two-wide FMAs
//            (fma.rn.f32x2: the promotion is bound by FMA issue slots); after the last K-block the
//            row goes out as bf16 through a swizzled staging slab and TMA stores
// Grouped mode (mixture-of-experts): row block m multiplies expert mblk_group[m] of a
// [groups, N, K] weight tensor with scales [groups, N / 128, K / 128]; negative = skip.
//
// Quantisers: pb_fp8_quant_rows (1 x 128 blocks, writes q and the [K / 128, M] scales) and
// pb_fp8_quant_blocks (128 x 128 blocks). scale = amax / 448, or 1 for an all-zero block.
//
// Reference semantics: kernels/__init__.py fp8_quantize / fp8_linear of the reference
// (block 128, e4m3, scale = amax / 448).
#include <cuda.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace pb {

int make_tmap_3d(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                 uint32_t box_inner, uint32_t box_outer);
int num_sms();

namespace f8 {

constexpr int BM = 128, BN = 256, BK = 128, HALF = 128;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 8 * 4096;
constexpr int THREADS = 320;
constexpr int SMEM_TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;

struct Params {
  int M, N, K;
  const float* sa;     // [K / 128, M]
  const float* sb;     // [groups, ceil(N / 128), K / 128]
  const int* mblk_group;
  int* status;
  // Fused expert-parallel dispatch (null otherwise): the rows of A and their scales are being
  // stored into this GPU's memory by the other ranks' dispatch kernels while this kernel runs.
  // blk_arrived[m] counts the rows of 128-row block m that have landed (the senders add to it
  // with release semantics after each row), blk_expect[m] is how many will; the TMA producer
  // takes a block only once it is complete. TMA reads this GPU's own memory only.
  const uint32_t* blk_arrived;
  const int* blk_expect;
  uint64_t wait_budget_ns;
};

// Two fp32 FMAs in one instruction (fma.rn.f32x2): a0 += s * x0, a1 += s * x1, each rounded
// like fmaf. The promotion is bound by FMA issue slots, and this halves them.
__device__ __forceinline__ void fma2(float& a0, float& a1, float s, uint32_t x0, uint32_t x1) {
  asm("{\n\t.reg .b64 pa, pb, pc;\n\t"
      "mov.b64 pa, {%0, %1};\n\t"
      "mov.b64 pb, {%3, %4};\n\t"
      "mov.b64 pc, {%2, %2};\n\t"
      "fma.rn.f32x2 pa, pc, pb, pa;\n\t"
      "mov.b64 {%0, %1}, pa;\n\t}"
      : "+f"(a0), "+f"(a1)
      : "f"(s), "r"(x0), "r"(x1));
}

// PROBE 0 is the product. The others exist only in the debug build of the library and time
// parts of the kernel (their output is not the product's): 1 = no promotion (loads, MMAs and
// the per-K-block accumulator hand-over only), 2 = accumulation in place with one hand-over
// per tile (the ceiling of this tile shape and operand feed), 3 = promotion FMAs without the
// tensor-memory loads, 4 = tensor-memory loads without the FMAs.
template <int PROBE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smA = smem;
  uint8_t* smB = smem + STAGES * A_BYTES;
  uint8_t* smEpi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int nkb = p.K / BK;
  const long total = static_cast<long>(num_m) * num_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 256);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // n-major inside groups of 8 row blocks, like the bf16 kernel: B tiles stay in L2
  auto coords = [&](long t, int& m_blk, int& n_blk) {
    const int r = static_cast<int>(t);
    const int group = 8 * num_n;
    const int first_m = (r / group) * 8;
    const int gsz = min(num_m - first_m, 8);
    m_blk = first_m + (r % group) % gsz;
    n_blk = (r % group) / gsz;
  };
  auto group_of = [&](int m_blk) { return p.mblk_group ? p.mblk_group[m_blk] : 0; };

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (long t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int m_blk, n_blk;
        coords(t, m_blk, n_blk);
        const int g = group_of(m_blk);
        if (g < 0) continue;
        if (p.blk_arrived != nullptr) {
          const int want = p.blk_expect[m_blk];
          if (want > 0) {
            if (!wait_flag_ge(p.blk_arrived + m_blk, static_cast<uint32_t>(want), p.wait_budget_ns,
                              p.status)) { ok = false; break; }
            // the rows were written by peers' ordinary stores; the bulk loads below read
            // through the asynchronous proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, p.status)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
          tma_load_3d(smA + s * A_BYTES, &tmA, &full[s], kb * BK, m_blk * BM, 0);
          tma_load_3d(smB + s * B_BYTES, &tmB, &full[s], kb * BK, n_blk * BN, g);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(0, 0, BM, BN, 0, 0);   // e4m3 x e4m3, both K-major
      int s = 0;
      uint32_t ph = 0;
      uint32_t it = 0;        // K-blocks issued so far: picks the accumulator and its phase
      bool ok = true;
      for (long t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int m_blk, n_blk;
        coords(t, m_blk, n_blk);
        if (group_of(m_blk) < 0) continue;
        for (int kb = 0; kb < nkb; it += (PROBE == 2 ? (kb == nkb - 1) : 1), ++kb) {
          const int acc = it & 1;
          if ((PROBE != 2 || kb == 0) && !mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, p.status)) { ok = false; break; }
          if (!mbar_wait(&full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smA + s * A_BYTES);
          const uint32_t b_addr = smem_u32(smB + s * B_BYTES);
#pragma unroll
          for (int j = 0; j < BK / 32; ++j)
            umma_f8(tmem_base + acc * BN, make_sdesc_sw128(a_addr + j * 32, 16, 1024),
                    make_sdesc_sw128(b_addr + j * 32, 16, 1024), idesc,
                    (j > 0 || (PROBE == 2 && kb > 0)) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (PROBE != 2 || kb == nkb - 1) umma_commit(&tfull[acc]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;            // tensor-memory lane quarter of this warp
    const int half = (warp - 2) >> 2;  // which 128 columns of the tile
    const int n_sb = p.K / BK;
    const int n_sb_rows = (p.N + HALF - 1) / HALF;
    uint32_t it = 0;
    bool ok = true;
    uint8_t* buf = smEpi + (warp - 2) * 4096;
    for (long t = blockIdx.x; t < total && ok; t += gridDim.x) {
      int m_blk, n_blk;
      coords(t, m_blk, n_blk);
      const int g = group_of(m_blk);
      if (g < 0) continue;
      const int row = m_blk * BM + q * 32 + lane;
      const int srow = min(row, p.M - 1);
      const int sb_row = min(n_blk * 2 + half, n_sb_rows - 1);
      const float* sb = p.sb + (static_cast<size_t>(g) * n_sb_rows + sb_row) * n_sb;
      float acc[HALF];
#pragma unroll
      for (int i = 0; i < HALF; ++i) acc[i] = 0.f;
      // Scale of the K-block in hand, loaded one block ahead so its latency hides behind the
      // previous block's promotion. In the fused-dispatch mode a peer may still be writing the
      // scales when the tile starts: the first one is then read only after the first accumulator
      // is full, which implies that the whole row block (payload and scales) has landed.
      const float* sa_row = p.sa + srow;
      float scale_cur = 0.f;
      bool have = false;
      if (p.blk_arrived == nullptr) {
        scale_cur = __ldcg(sa_row) * sb[0];
        have = true;
      }
      for (int kb = 0; kb < (PROBE == 2 ? 1 : nkb); ++kb, ++it) {
        const int a = it & 1;
        if (!mbar_wait(&tfull[a], (it >> 1) & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        if (!have) scale_cur = __ldcg(sa_row + static_cast<size_t>(kb) * p.M) * sb[kb];
        const float scale = scale_cur;
        if (kb + 1 < nkb) {
          scale_cur = __ldcg(sa_row + static_cast<size_t>(kb + 1) * p.M) * sb[kb + 1];
          have = true;
        }
        const uint32_t t_addr =
            tmem_base + a * BN + half * HALF + (static_cast<uint32_t>(q * 32) << 16);
        if constexpr (PROBE == 0) {
#pragma unroll
          for (int c = 0; c < HALF; c += 64) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(t_addr + c, r0);
            tmem_ld_32x32b_x32(t_addr + c + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              fma2(acc[c + i], acc[c + i + 1], scale, r0[i], r0[i + 1]);
              fma2(acc[c + 32 + i], acc[c + 32 + i + 1], scale, r1[i], r1[i + 1]);
            }
          }
        } else if constexpr (PROBE == 3) {
          const float v = __uint_as_float(0x3f800000u + (kb & 3));
#pragma unroll
          for (int i = 0; i < HALF; ++i) acc[i] = fmaf(scale, v + i, acc[i]);
        } else if constexpr (PROBE == 4) {
#pragma unroll
          for (int c = 0; c < HALF; c += 64) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(t_addr + c, r0);
            tmem_ld_32x32b_x32(t_addr + c + 32, r1);
            tmem_ld_wait();
            acc[c] = fmaf(scale, __uint_as_float(r0[0]) + __uint_as_float(r1[31]), acc[c]);
          }
        } else {
          acc[0] += scale + __uint_as_float(t_addr & 1u);
        }
        tc_fence_before();
        mbar_arrive(&tempty[a]);
      }
      if (!ok) break;
      // row -> bf16 -> 64-column slabs in the TMA swizzle layout -> bulk tensor stores
      const int y0 = m_blk * BM + q * 32;
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) {
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        uint8_t* rowp = buf + lane * 128;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          bf16x8 pk;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            pk.v[j] = __floats2bfloat162_rn(acc[sl * 64 + 8 * i + 2 * j], acc[sl * 64 + 8 * i + 2 * j + 1]);
          *reinterpret_cast<bf16x8*>(rowp + ((i ^ (lane & 7)) << 4)) = pk;
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int x0 = n_blk * BN + half * HALF + sl * 64;
        if (lane == 0 && x0 < p.N && y0 < p.M) tma_store_3d(&tmC, buf, x0, y0, 0);
        if (lane == 0) tma_store_commit();
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let copies in flight land
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------ quantisers
__device__ __forceinline__ uint32_t to_e4m3x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// One warp per row; a lane covers 16 consecutive elements (two 16-byte loads, one 16-byte
// store), eight lanes one 128-element block, so a warp moves 512 elements per step. Every lane
// runs every step (the shuffles name the whole warp); K is a multiple of 128, so the eight lanes
// of a block are active or idle together.
// rows_dev (may be null): device-side count of the rows in use; the scale table keeps its row
// stride M whatever that count.
__device__ __forceinline__ uint4 quant16(const float (&f)[16], bool active, float* scale_out) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(f[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  *scale_out = scale;
  uint4 pk = make_uint4(0u, 0u, 0u, 0u);
  if (active) {
    // true division (not a reciprocal multiply): ties must round as in x / scale
    pk.x = to_e4m3x4(__fdiv_rn(f[0], scale), __fdiv_rn(f[1], scale), __fdiv_rn(f[2], scale), __fdiv_rn(f[3], scale));
    pk.y = to_e4m3x4(__fdiv_rn(f[4], scale), __fdiv_rn(f[5], scale), __fdiv_rn(f[6], scale), __fdiv_rn(f[7], scale));
    pk.z = to_e4m3x4(__fdiv_rn(f[8], scale), __fdiv_rn(f[9], scale), __fdiv_rn(f[10], scale), __fdiv_rn(f[11], scale));
    pk.w = to_e4m3x4(__fdiv_rn(f[12], scale), __fdiv_rn(f[13], scale), __fdiv_rn(f[14], scale), __fdiv_rn(f[15], scale));
  }
  return pk;
}

__global__ void __launch_bounds__(256) quant_rows_kernel(const bf16* __restrict__ x, long ld, int M,
                                                         int K, uint8_t* __restrict__ q,
                                                         float* __restrict__ scales,
                                                         const int* __restrict__ rows_dev) {
  const int lane = threadIdx.x & 31;
  const int m_eff = rows_dev != nullptr ? min(M, *rows_dev) : M;
  const long warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  for (long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < m_eff;
       row += warps) {
    const bf16* src = x + static_cast<size_t>(row) * ld;
    for (int c0 = 0; c0 < K; c0 += 512) {
      const int c = c0 + lane * 16;
      const bool active = c < K;
      float f[16];
      if (active) {
        unpack8(*reinterpret_cast<const bf16x8*>(src + c), f);
        unpack8(*reinterpret_cast<const bf16x8*>(src + c + 8), f + 8);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = 0.f;
      }
      float scale;
      const uint4 pk = quant16(f, active, &scale);
      if (active) {
        *reinterpret_cast<uint4*>(q + static_cast<size_t>(row) * K + c) = pk;
        if ((lane & 7) == 0) scales[static_cast<size_t>(c >> 7) * M + row] = scale;
      }
    }
  }
}

// SwiGLU fused with the row quantiser: h = silu(gate) * up is written as bf16 (the backward
// and the weight gradient of the next product need it) and, from those bf16 values, as e4m3 +
// 1 x 128 scales for the FP8 product that consumes it. One pass over gu instead of a SwiGLU
// pass and a quantiser pass. gu [rows, 2H] (gate | up), H a multiple of 128.
__global__ void __launch_bounds__(256) swiglu_quant_kernel(const bf16* __restrict__ gu,
                                                           bf16* __restrict__ h, int M, int H,
                                                           uint8_t* __restrict__ q,
                                                           float* __restrict__ scales,
                                                           const int* __restrict__ rows_dev) {
  const int lane = threadIdx.x & 31;
  const int m_eff = rows_dev != nullptr ? min(M, *rows_dev) : M;
  const long warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  for (long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < m_eff;
       row += warps) {
    const bf16* src = gu + static_cast<size_t>(row) * 2 * H;
    for (int c0 = 0; c0 < H; c0 += 512) {
      const int c = c0 + lane * 16;
      const bool active = c < H;
      float f[16];
      if (active) {
        float g[16], u[16];
        unpack8(*reinterpret_cast<const bf16x8*>(src + c), g);
        unpack8(*reinterpret_cast<const bf16x8*>(src + c + 8), g + 8);
        unpack8(*reinterpret_cast<const bf16x8*>(src + H + c), u);
        unpack8(*reinterpret_cast<const bf16x8*>(src + H + c + 8), u + 8);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float s = 1.f / (1.f + __expf(-g[j]));
          // quantise what the bf16 copy holds, so both forms of h agree
          f[j] = bf16_to_f32(f32_to_bf16(g[j] * s * u[j]));
        }
        if (h != nullptr) {                  // callers that keep only the e4m3 rows pass null
          bf16* dst = h + static_cast<size_t>(row) * H + c;
          *reinterpret_cast<bf16x8*>(dst) = pack8(f);
          *reinterpret_cast<bf16x8*>(dst + 8) = pack8(f + 8);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) f[j] = 0.f;
      }
      float scale;
      const uint4 pk = quant16(f, active, &scale);
      if (active) {
        *reinterpret_cast<uint4*>(q + static_cast<size_t>(row) * H + c) = pk;
        if ((lane & 7) == 0) scales[static_cast<size_t>(c >> 7) * M + row] = scale;
      }
    }
  }
}

// y[row, :] = bf16(e4m3(q[row, :]) * scale of its 1 x 128 block); one warp per row, a lane
// covers 16 consecutive elements (one 16-byte load, two 16-byte stores)
__global__ void __launch_bounds__(256) dequant_rows_kernel(const uint8_t* __restrict__ q,
                                                           const float* __restrict__ scales,
                                                           long ld_s, int M, int K,
                                                           bf16* __restrict__ y,
                                                           const int* __restrict__ rows_dev) {
  const int lane = threadIdx.x & 31;
  const int m_eff = rows_dev != nullptr ? min(M, *rows_dev) : M;
  const long warps = (static_cast<long>(gridDim.x) * blockDim.x) >> 5;
  for (long row = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < m_eff;
       row += warps) {
    // four column groups (2048 elements of the row) per pass: their payload and scale loads are
    // all issued before the first conversion, so a pass costs one memory latency, not four
    for (int c0 = 0; c0 < K; c0 += 2048) {
      uint4 raw[4];
      float sc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 512 + lane * 16;
        if (c < K) {
          raw[u] = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(row) * K + c);
          sc[u] = scales[static_cast<size_t>(c >> 7) * ld_s + row];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 512 + lane * 16;
        if (c >= K) continue;
        const float s = sc[u];
        const uint32_t w4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float f[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(
                static_cast<__nv_fp8x2_storage_t>((w4[j] >> (16 * hh)) & 0xffffu), __NV_E4M3);
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            f[4 * j + 2 * hh] = v.x * s;
            f[4 * j + 2 * hh + 1] = v.y * s;
          }
        }
        bf16* dst = y + static_cast<size_t>(row) * K + c;
        *reinterpret_cast<bf16x8*>(dst) = pack8(f);
        *reinterpret_cast<bf16x8*>(dst + 8) = pack8(f + 8);
      }
    }
  }
}

// One CTA (256 threads) per 128 x 128 block of a [N, K] matrix (edges clipped).
// q / scales may be null when only `deq` is wanted. deq (may be null): bf16 [N, K] image of the
// quantised block, e4m3(w / scale) * scale: the operand the FP8 GEMM really multiplied, which is
// what the backward of an FP8 linear differentiates against.
__global__ void __launch_bounds__(256)
quant_blocks_kernel(const bf16* __restrict__ w, long ld, int N, int K, uint8_t* __restrict__ q,
                    float* __restrict__ scales, bf16* __restrict__ deq) {
  // The 128 x 128 block is read once: thread t keeps 16 consecutive elements of four rows
  // (rows t / 8 + 32 i, columns 16 (t % 8) ..) in registers across the block-wide maximum.
  __shared__ float red[33];
  const int nb = blockIdx.y, kb = blockIdx.x;
  const int r0 = nb * 128 + (threadIdx.x >> 3), c = kb * 128 + (threadIdx.x & 7) * 16;
  const bool vec_ok = (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  float v[4][16];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 32 * i;
    if (r < N && c < K) {                      // K is a multiple of 128: the 16 columns are in range
      const bf16* src = w + static_cast<size_t>(r) * ld + c;
      if (vec_ok) {
        unpack8(*reinterpret_cast<const bf16x8*>(src), v[i]);
        unpack8(*reinterpret_cast<const bf16x8*>(src + 8), v[i] + 8);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[i][j] = __bfloat162float(src[j]);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    }
  }
  amax = block_max(amax, red);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 32 * i;
    if (r >= N || c >= K) continue;
    uint32_t pk[4];
#pragma unroll
    for (int g = 0; g < 4; ++g)
      pk[g] = to_e4m3x4(__fdiv_rn(v[i][4 * g], scale), __fdiv_rn(v[i][4 * g + 1], scale),
                        __fdiv_rn(v[i][4 * g + 2], scale), __fdiv_rn(v[i][4 * g + 3], scale));
    if (q != nullptr)
      *reinterpret_cast<uint4*>(q + static_cast<size_t>(r) * K + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    if (deq != nullptr) {
      float f[16];
#pragma unroll
      for (int g = 0; g < 4; ++g)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(
              static_cast<__nv_fp8x2_storage_t>((pk[g] >> (16 * hh)) & 0xffffu), __NV_E4M3);
          const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&h2));
          f[4 * g + 2 * hh] = t.x * scale;
          f[4 * g + 2 * hh + 1] = t.y * scale;
        }
      bf16* dst = deq + static_cast<size_t>(r) * K + c;
      *reinterpret_cast<bf16x8*>(dst) = pack8(f);
      *reinterpret_cast<bf16x8*>(dst + 8) = pack8(f + 8);
    }
  }
  if (threadIdx.x == 0 && scales != nullptr) scales[static_cast<size_t>(nb) * gridDim.x + kb] = scale;
}

}  // namespace f8
}  // namespace pb

using namespace pb;

// x [M, K] bf16 (row stride ld, K % 128 == 0) -> q [M, K] e4m3, scales [K / 128, M] fp32.
PB_API int pb_fp8_quant_rows(const void* x, long ld, int M, int K, void* q, float* scales,
                             cudaStream_t st) {
  if (M <= 0 || K <= 0 || K % 128 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return PB_BAD_ARG;
  long blocks = (static_cast<long>(M) * 32 + 255) / 256;
  // one warp per row, no grid-stride cap: measured 10 % faster than a persistent grid
  f8::quant_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const bf16*>(x), ld, M, K, static_cast<uint8_t*>(q), scales, nullptr);
  return static_cast<int>(cudaGetLastError());
}
// The same over the first min(M, *rows_dev) rows (rows_dev: a device int).
PB_API int pb_fp8_quant_rows_dyn(const void* x, long ld, int M, int K, void* q, float* scales,
                                 const int* rows_dev, cudaStream_t st) {
  if (M <= 0 || K <= 0 || K % 128 != 0 || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
    return PB_BAD_ARG;
  long blocks = (static_cast<long>(M) * 32 + 255) / 256;
  f8::quant_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const bf16*>(x), ld, M, K, static_cast<uint8_t*>(q), scales, rows_dev);
  return static_cast<int>(cudaGetLastError());
}

// h [M, H] bf16 = silu(gu[:, :H]) * gu[:, H:], and its e4m3 rows q [M, H] with scales
// [H / 128, M], in one pass. H a multiple of 128; rows_dev (may be null): device row count.
PB_API int pb_swiglu_quant(const void* gu, void* h, int M, int H, void* q, float* scales,
                           const int* rows_dev, cudaStream_t st) {
  if (M <= 0 || H <= 0 || H % 128 != 0) return PB_BAD_ARG;
  long blocks = (static_cast<long>(M) * 32 + 255) / 256;
  f8::swiglu_quant_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const bf16*>(gu), static_cast<bf16*>(h), M, H, static_cast<uint8_t*>(q), scales,
      rows_dev);
  return static_cast<int>(cudaGetLastError());
}

// q [M, K] e4m3 with scales [K / 128, ld_s] (ld_s >= M: the row stride of the scale table)
// -> y [M, K] bf16. The straight-through backward of an FP8 product uses these values.
PB_API int pb_fp8_dequant_rows(const void* q, const float* scales, long ld_s, int M, int K, void* y,
                               const int* rows_dev, cudaStream_t st) {
  if (M <= 0 || K <= 0 || K % 128 != 0 || ld_s < M) return PB_BAD_ARG;
  long blocks = (static_cast<long>(M) * 32 + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  f8::dequant_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const uint8_t*>(q), scales, ld_s, M, K, static_cast<bf16*>(y), rows_dev);
  return static_cast<int>(cudaGetLastError());
}

// w [groups * N, K] bf16 (K % 128 == 0, N % 128 == 0 when groups > 1) -> q e4m3 same shape,
// scales [groups * ceil(N / 128), K / 128].
PB_API int pb_fp8_quant_blocks(const void* w, long ld, int rows, int K, void* q, float* scales,
                               cudaStream_t st) {
  if (rows <= 0 || K <= 0 || K % 128 != 0 || ld % 4 != 0) return PB_BAD_ARG;
  dim3 grid(K / 128, (rows + 127) / 128);
  f8::quant_blocks_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(w), ld, rows, K,
                                                static_cast<uint8_t*>(q), scales, nullptr);
  return static_cast<int>(cudaGetLastError());
}

// out [rows, K] bf16 = the 128 x 128 block quantisation of w applied and undone (e4m3 rounding at
// the block's scale): the weight an FP8 linear really used. Same shape rules as
// pb_fp8_quant_blocks.
PB_API int pb_fp8_fakequant_blocks(const void* w, long ld, int rows, int K, void* out,
                                   cudaStream_t st) {
  if (rows <= 0 || K <= 0 || K % 128 != 0 || ld % 4 != 0 || out == nullptr) return PB_BAD_ARG;
  dim3 grid(K / 128, (rows + 127) / 128);
  f8::quant_blocks_kernel<<<grid, 256, 0, st>>>(static_cast<const bf16*>(w), ld, rows, K, nullptr,
                                                nullptr, static_cast<bf16*>(out));
  return static_cast<int>(cudaGetLastError());
}

// C [M, N] bf16 = block-scaled Aq [M, K] x Bq [groups, N, K]^T. K % 128 == 0, N % 8 == 0.
// sa [K / 128, M]; sb [groups, ceil(N / 128), K / 128]; mblk_group null (groups == 1) or one
// int per 128-row block of A / C.
template <int PROBE = 0>
static int gemm_fp8_launch(const void* Aq, const float* sa, const void* Bq, const float* sb,
                           void* C, int M, int N, int K, int groups, long ldc,
                           const int* mblk_group, int* status, int max_ctas,
                           const uint32_t* blk_arrived, const int* blk_expect, long budget_ns,
                           cudaStream_t st);

PB_API int pb_gemm_fp8_blockscaled(const void* Aq, const float* sa, const void* Bq, const float* sb,
                                   void* C, int M, int N, int K, int groups, long ldc,
                                   const int* mblk_group, int* status, int max_ctas,
                                   cudaStream_t st) {
  return gemm_fp8_launch(Aq, sa, Bq, sb, C, M, N, K, groups, ldc, mblk_group, status, max_ctas,
                         nullptr, nullptr, 0, st);
}

// The grouped product fused with the arrival of its rows: Aq / sa are a receive buffer that the
// other ranks' dispatch kernels are still filling. blk_arrived (uint32 per 128-row block, in
// memory the senders can reach, zero before the senders start) is incremented once per landed
// row; blk_expect (int per block) is the number of rows each block will receive. A row block is
// loaded only when complete; a block that does not complete within budget_ns latches
// PB_TIMEOUT_FLAG in *status and the kernel drains.
PB_API int pb_gemm_fp8_grouped_arrive(const void* Aq, const float* sa, const void* Bq, const float* sb,
                                      void* C, int M, int N, int K, int groups, long ldc,
                                      const int* mblk_group, const void* blk_arrived,
                                      const int* blk_expect, long budget_ns, int* status,
                                      cudaStream_t st) {
  if (blk_arrived == nullptr || blk_expect == nullptr || budget_ns <= 0 || mblk_group == nullptr)
    return PB_BAD_ARG;
  return gemm_fp8_launch(Aq, sa, Bq, sb, C, M, N, K, groups, ldc, mblk_group, status, 0,
                         static_cast<const uint32_t*>(blk_arrived), blk_expect, budget_ns, st);
}

#ifdef PB_DEBUG_BOUNDS
// Debug build only: the timing probes of gemm_fp8_kernel (1 no promotion, 2 accumulation in
// place, 3 FMAs only, 4 tensor-memory loads only). C receives values that are not the product.
PB_API int pb_gemm_fp8_probe(const void* Aq, const float* sa, const void* Bq, const float* sb,
                             void* C, int M, int N, int K, long ldc, int probe, int* status,
                             cudaStream_t st) {
  switch (probe) {
    case 1: return gemm_fp8_launch<1>(Aq, sa, Bq, sb, C, M, N, K, 1, ldc, nullptr, status, 0, nullptr, nullptr, 0, st);
    case 2: return gemm_fp8_launch<2>(Aq, sa, Bq, sb, C, M, N, K, 1, ldc, nullptr, status, 0, nullptr, nullptr, 0, st);
    case 3: return gemm_fp8_launch<3>(Aq, sa, Bq, sb, C, M, N, K, 1, ldc, nullptr, status, 0, nullptr, nullptr, 0, st);
    case 4: return gemm_fp8_launch<4>(Aq, sa, Bq, sb, C, M, N, K, 1, ldc, nullptr, status, 0, nullptr, nullptr, 0, st);
    default: return PB_BAD_ARG;
  }
}
#endif

template <int PROBE>
static int gemm_fp8_launch(const void* Aq, const float* sa, const void* Bq, const float* sb,
                           void* C, int M, int N, int K, int groups, long ldc,
                           const int* mblk_group, int* status, int max_ctas,
                           const uint32_t* blk_arrived, const int* blk_expect, long budget_ns,
                           cudaStream_t st) {
  using namespace f8;
  if (M <= 0 || N <= 0 || K <= 0 || K % BK != 0 || groups <= 0 || (ldc * 2) % 16 != 0)
    return PB_BAD_ARG;
  if (groups > 1 && (mblk_group == nullptr || N % HALF != 0)) return PB_BAD_ARG;
  if (groups == 1 && blk_arrived != nullptr && N % HALF != 0) return PB_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(Aq) & 15) || (reinterpret_cast<uintptr_t>(Bq) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return PB_BAD_ARG;
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel<PROBE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  CUtensorMap tmA, tmB, tmC;
  int r = make_tmap_3d(&tmA, Aq, 1, K, M, 1, K, 0, BK, BM);
  if (r != 0) return 1000 + r;
  r = make_tmap_3d(&tmB, Bq, 1, K, N, groups, K, static_cast<uint64_t>(N) * K, BK, BN);
  if (r != 0) return 2000 + r;
  r = make_tmap_3d(&tmC, C, 2, N, M, 1, ldc, 0, 64, 32);
  if (r != 0) return 3000 + r;
  Params p;
  p.M = M; p.N = N; p.K = K;
  p.sa = sa; p.sb = sb; p.mblk_group = mblk_group; p.status = status;
  p.blk_arrived = blk_arrived; p.blk_expect = blk_expect;
  p.wait_budget_ns = static_cast<uint64_t>(budget_ns);
  const long tiles = static_cast<long>((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = static_cast<int>(tiles);
  gemm_fp8_kernel<PROBE><<<grid, THREADS, SMEM_TOTAL, st>>>(tmA, tmB, tmC, p);
  return static_cast<int>(cudaGetLastError());
}
