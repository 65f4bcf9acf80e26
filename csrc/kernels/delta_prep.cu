// Chunk-local WY operands of the delta rule on tcgen05 (sm_100a), one fused kernel.
//
// For every chunk of 64 tokens of one (batch, head) it forms, from the K / Q / V rows and
// the write strengths beta, everything the state walk consumes:
//
//   G = K K^T                      A  = diag(beta) tril(G, -1)       T = (I + A)^-1
//   A' = T diag(beta)              W  = A' K        U^ = A' V        M = tril(Q K^T)
//
// K, Q and V are read by TMA straight out of the projection outputs ([batch * seq,
// heads * 128], no per-chunk copies); G and Q K^T are two tcgen05.mma products with their
// accumulators in tensor memory; the unit-lower-triangular inverse is an fp32 forward
// substitution with one column per thread (operand rows broadcast from shared memory as
// 16-byte loads); A' goes back to shared memory as a 128-byte-swizzled bf16 operand for
// the two products W and U^; every result leaves by a TMA store. Two CTAs of 64 threads
// share an SM (256 tensor-memory columns each), so one chunk's substitution overlaps the
// other's loads, products and stores.
//
// Reference semantics: kernels/__init__.py:357-376 of the reference (per-token delta-rule
// recurrence); the chunked WY algebra and this kernel are this library's own.
#include <cuda.h>

#include "common.cuh"

namespace pb {

int make_tmap_3d(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                 uint32_t box_inner, uint32_t box_outer);

namespace dprep {

constexpr int C = 64, D = 128;
constexpr int KT = 0, QT = 16384, VT = 32768, AF = 49152, AP = 65536, BARS = 73728;
constexpr int SMEM_BYTES = 100 * 1024;  // also keeps residency at two CTAs per SM
constexpr int TMEM_COLS = 256;

struct Params {
  int n_chunks;   // chunks per sequence
  int heads;
  int seq_len;    // tokens per sequence (multiple of 64)
  int total;      // batch * heads * n_chunks
  const void* beta;  // [batch, seq, heads]
  int beta_f32;
  int* status;
};

__device__ __forceinline__ void st_swz(uint8_t* tile, int row, int c16, const bf16x8& v) {
  *reinterpret_cast<bf16x8*>(tile + row * 128 + ((c16 ^ (row & 7)) << 4)) = v;
}

// Row `row` of a 64-column fp32 accumulator block -> bf16 [64][64] swizzled tile, keeping
// columns <= limit (limit = 63 keeps all).
__device__ __forceinline__ void row_to_tile(uint32_t taddr, uint8_t* tile, int row, int limit) {
#pragma unroll 1
  for (int c = 0; c < 64; c += 32) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c, v);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (c + 8 * i + j <= limit) ? __uint_as_float(v[8 * i + j]) : 0.f;
      st_swz(tile, row, (c >> 3) + i, pack8(f));
    }
  }
}

__global__ void __launch_bounds__(64, 2)
delta_prep_fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmW,
                      const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmM,
                      const __grid_constant__ CUtensorMap tmAP, const __grid_constant__ CUtensorMap tmT,
                      const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BARS);
  uint64_t* full = bars;
  uint64_t* mma1 = bars + 1;
  uint64_t* mma2 = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  float4* af4 = reinterpret_cast<float4*>(smem + AF);

  const int r = threadIdx.x, warp = r >> 5;
  if (r == 0) {
    mbar_init(full, 1); mbar_init(mma1, 1); mbar_init(mma2, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t id_kk64 = make_idesc(1, 1, 128, 64, 0, 0);    // A, B K-major, N = 64
  const uint32_t id_kn = make_idesc(1, 1, 128, 128, 0, 1);     // A K-major, B MN-major
  const uint32_t kt = smem_u32(smem + KT), qt = smem_u32(smem + QT), vt = smem_u32(smem + VT);
  const uint32_t ap = smem_u32(smem + AP);

  uint32_t ph = 0;
  for (int g = blockIdx.x; g < p.total; g += gridDim.x, ph ^= 1) {
    const int seq = g / p.n_chunks, n = g - seq * p.n_chunks;
    const int b = seq / p.heads, h = seq - b * p.heads;
    const int row0 = b * p.seq_len + n * C;   // token row of the projection outputs
    const int x0 = h * D;
    if (r == 0) {
      tma_store_wait_read<0>();  // earlier stores have drained the tiles about to be refilled
      mbar_arrive_expect_tx(full, 3 * 16384);
      tma_load_3d(smem + KT, &tmK, full, x0, row0, 0);
      tma_load_3d(smem + KT + 8192, &tmK, full, x0 + 64, row0, 0);
      tma_load_3d(smem + QT, &tmQ, full, x0, row0, 0);
      tma_load_3d(smem + QT + 8192, &tmQ, full, x0 + 64, row0, 0);
      tma_load_3d(smem + VT, &tmV, full, x0, row0, 0);
      tma_load_3d(smem + VT + 8192, &tmV, full, x0 + 64, row0, 0);
    }
    const size_t bidx = (static_cast<size_t>(row0) + r) * p.heads + h;
    const float beta = p.beta_f32 ? static_cast<const float*>(p.beta)[bidx]
                                  : bf16_to_f32(static_cast<const bf16*>(p.beta)[bidx]);
    bool ok = true;
    if (r == 0) {
      ok = mbar_wait(full, ph, p.status);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < 8; ++j)     // G = K K^T -> columns [0, 64)
          umma_f16(tmem, make_sdesc_sw128(kt + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024),
                   make_sdesc_sw128(kt + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024), id_kk64, j > 0);
#pragma unroll
        for (int j = 0; j < 8; ++j)     // Q K^T -> columns [64, 128)
          umma_f16(tmem + 64, make_sdesc_sw128(qt + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024),
                   make_sdesc_sw128(kt + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024), id_kk64, j > 0);
        umma_commit(mma1);
      }
    }
    ok = mbar_wait_spin(mma1, ph, p.status) && ok;
    if (!__syncthreads_and(ok)) break;
    tc_fence_after();

    // A = diag(beta) tril(G, -1), fp32, rows in 16-byte pieces at position (piece ^ (row & 15))
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(lane_addr + c, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float4 a;
        a.x = (c + 4 * i + 0 < r) ? beta * __uint_as_float(v[4 * i + 0]) : 0.f;
        a.y = (c + 4 * i + 1 < r) ? beta * __uint_as_float(v[4 * i + 1]) : 0.f;
        a.z = (c + 4 * i + 2 < r) ? beta * __uint_as_float(v[4 * i + 2]) : 0.f;
        a.w = (c + 4 * i + 3 < r) ? beta * __uint_as_float(v[4 * i + 3]) : 0.f;
        af4[r * 16 + (((c >> 2) + i) ^ (r & 15))] = a;
      }
    }
    // M = tril(Q K^T) -> the Q tile's first half (the products that read Q are complete)
    row_to_tile(lane_addr + 64, smem + QT, r, r);
    __syncthreads();

    // column r of T = (I + A)^-1 by forward substitution
    float t[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      float a0 = (i == r) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int c = 0; c < (i + 3) / 4; ++c) {
        const float4 a = af4[i * 16 + (c ^ (i & 15))];
        if (4 * c + 0 < i) a0 = fmaf(-a.x, t[4 * c + 0], a0);
        if (4 * c + 1 < i) a1 = fmaf(-a.y, t[4 * c + 1], a1);
        if (4 * c + 2 < i) a2 = fmaf(-a.z, t[4 * c + 2], a2);
        if (4 * c + 3 < i) a3 = fmaf(-a.w, t[4 * c + 3], a3);
      }
      t[i] = (a0 + a1) + (a2 + a3);
    }
    // T -> the Q tile's second half, A' = T diag(beta) -> operand tile (element (i, r) each)
    {
      uint8_t* tt = smem + QT + 8192;
      uint8_t* at = smem + AP;
      const int sub = (r & 7) * 2, c16 = r >> 3;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const int off = i * 128 + ((c16 ^ (i & 7)) << 4) + sub;
        *reinterpret_cast<bf16*>(tt + off) = f32_to_bf16(t[i]);
        *reinterpret_cast<bf16*>(at + off) = f32_to_bf16(t[i] * beta);
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tc_fence_after();
#pragma unroll
      for (int j = 0; j < 4; ++j)       // W = A' K -> columns [0, 128)
        umma_f16(tmem, make_sdesc_sw128(ap + j * 32, 16, 1024),
                 make_sdesc_sw128(kt + j * 2048, 8192, 1024), id_kn, j > 0);
#pragma unroll
      for (int j = 0; j < 4; ++j)       // U^ = A' V -> columns [128, 256)
        umma_f16(tmem + 128, make_sdesc_sw128(ap + j * 32, 16, 1024),
                 make_sdesc_sw128(vt + j * 2048, 8192, 1024), id_kn, j > 0);
      umma_commit(mma2);
      tma_store_3d(&tmM, smem + QT, 0, g * C, 0);
      tma_store_3d(&tmT, smem + QT + 8192, 0, g * C, 0);
      tma_store_3d(&tmAP, smem + AP, 0, g * C, 0);
      tma_store_commit();
    }
    ok = mbar_wait_spin(mma2, ph, p.status);
    if (!__syncthreads_and(ok)) break;
    tc_fence_after();
    // W -> K tile, U^ -> V tile (both products have finished reading them), then out
    row_to_tile(lane_addr + 0, smem + KT, r, 63);
    row_to_tile(lane_addr + 64, smem + KT + 8192, r, 63);
    row_to_tile(lane_addr + 128, smem + VT, r, 63);
    row_to_tile(lane_addr + 192, smem + VT + 8192, r, 63);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tma_store_3d(&tmW, smem + KT, 0, g * C, 0);
      tma_store_3d(&tmW, smem + KT + 8192, 64, g * C, 0);
      tma_store_3d(&tmU, smem + VT, 0, g * C, 0);
      tma_store_3d(&tmU, smem + VT + 8192, 64, g * C, 0);
      tma_store_commit();
    }
  }
  if (r == 0) tma_store_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------
// Backward of the chunk-local part. Given, per chunk, the gradients the state walk hands
// back (dW, -dU, dM = dO U^T before masking, and the walk's own contributions to dQ and dK)
// it produces dq, dk, dv (token-major, like q / k / v) and dbeta:
//
//   dA' = dW K^T - (-dU) V^T... (dU^ = dU)          dV = A'^T dU          dK += A'^T dW
//   dbeta_j += sum_i dA'_ij T_ij                     dA = -T^T (dA' A'^T)
//   dbeta_i += sum_{j<i} dA_ij G_ij                  dG = diag(beta) tril(dA, -1)
//   dK += (dG + dG^T) K + tril(dM)^T Q               dQ += tril(dM) K
//
// Eleven tcgen05 products in four passes with 64-row operands; the 64 x 64 intermediates
// go through one shared-memory tile, re-used as K-major or MN-major operand as needed, so
// no transposes are materialised. The column sum for dbeta is the diagonal of dA'^T T,
// also a tensor-core product.
namespace bwd {
constexpr int DW = 0, NDU = 16384, KTB = 32768, VQ = 49152, APB = 65536, TT = 73728, DM = 81920,
              TMP = 90112, BARSB = 98304;
constexpr int SMEM_BWD = 108 * 1024;
}  // namespace bwd

struct BwdParams {
  int n_chunks, heads, seq_len, total;
  const void* beta;    // [batch, seq, heads]
  int beta_f32;
  const bf16* dq_add;  // [total][64][128] or null: the walk's dQ = dO S^T
  const bf16* dk_add;  // [total][64][128] or null: the walk's dK = U dS'^T
  void* dbeta;         // [batch, seq, heads], same type as beta
  int* status;
};

__device__ __forceinline__ void ld_row32(uint32_t taddr, float* f) {
  uint32_t v[32];
  tmem_ld_32x32b_x32(taddr, v);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
}

// 128 accumulator columns of row `row` (+ an optional bf16 global row, times `sign`) ->
// two swizzled [64][64] bf16 tiles 8 KB apart
__device__ __forceinline__ void row128_to_tiles(uint32_t taddr, uint8_t* tiles, int row, float sign,
                                                const bf16* add) {
#pragma unroll 1
  for (int c = 0; c < 128; c += 32) {
    float f[32];
    ld_row32(taddr + c, f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = sign * f[8 * i + j];
      if (add != nullptr) {
        float a[8];
        unpack8(*reinterpret_cast<const bf16x8*>(add + c + 8 * i), a);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += a[j];
      }
      const int col = c + 8 * i;
      st_swz(tiles + (col >> 6) * 8192, row, (col & 63) >> 3, pack8(o));
    }
  }
}

__global__ void __launch_bounds__(64, 2)
delta_prep_bwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDW,
                      const __grid_constant__ CUtensorMap tmNDU, const __grid_constant__ CUtensorMap tmDM,
                      const __grid_constant__ CUtensorMap tmAP, const __grid_constant__ CUtensorMap tmT,
                      const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
                      const __grid_constant__ CUtensorMap tmDV, const BwdParams p) {
  using namespace bwd;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BARSB);
  uint64_t* full = bars;
  uint64_t* fullq = bars + 1;
  uint64_t* mma = bars + 2;   // [4]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int r = threadIdx.x, warp = r >> 5;
  if (r == 0) {
    mbar_init(full, 1); mbar_init(fullq, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&mma[i], 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDW); tma_prefetch_desc(&tmNDU); tma_prefetch_desc(&tmDM);
    tma_prefetch_desc(&tmAP); tma_prefetch_desc(&tmT);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t id_kk64 = make_idesc(1, 1, 128, 64, 0, 0);
  const uint32_t id_mm64 = make_idesc(1, 1, 128, 64, 1, 1);
  const uint32_t id_kn = make_idesc(1, 1, 128, 128, 0, 1);
  const uint32_t id_mm = make_idesc(1, 1, 128, 128, 1, 1);
  const uint32_t dw = smem_u32(smem + DW), ndu = smem_u32(smem + NDU), kt = smem_u32(smem + KTB);
  const uint32_t vq = smem_u32(smem + VQ), ap = smem_u32(smem + APB), tt = smem_u32(smem + TT);
  const uint32_t dm = smem_u32(smem + DM), tmp = smem_u32(smem + TMP);
  // operand descriptors: 128-wide K-major (8 steps), 64-wide K-major (4), MN-major (4)
  auto k128 = [](uint32_t base, int j) {
    return make_sdesc_sw128(base + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024);
  };
  auto k64 = [](uint32_t base, int j) { return make_sdesc_sw128(base + j * 32, 16, 1024); };
  auto mn = [](uint32_t base, int j) { return make_sdesc_sw128(base + j * 2048, 8192, 1024); };

  uint32_t ph = 0;
  for (int g = blockIdx.x; g < p.total; g += gridDim.x, ph ^= 1) {
    const int seq = g / p.n_chunks, n = g - seq * p.n_chunks;
    const int b = seq / p.heads, h = seq - b * p.heads;
    const int row0 = b * p.seq_len + n * C;
    const int x0 = h * D;
    const int crow = g * C;
    if (r == 0) {
      tma_store_wait_read<0>();
      mbar_arrive_expect_tx(full, 4 * 16384 + 3 * 8192);
      tma_load_3d(smem + DW, &tmDW, full, 0, crow, 0);
      tma_load_3d(smem + DW + 8192, &tmDW, full, 64, crow, 0);
      tma_load_3d(smem + NDU, &tmNDU, full, 0, crow, 0);
      tma_load_3d(smem + NDU + 8192, &tmNDU, full, 64, crow, 0);
      tma_load_3d(smem + KTB, &tmK, full, x0, row0, 0);
      tma_load_3d(smem + KTB + 8192, &tmK, full, x0 + 64, row0, 0);
      tma_load_3d(smem + VQ, &tmV, full, x0, row0, 0);
      tma_load_3d(smem + VQ + 8192, &tmV, full, x0 + 64, row0, 0);
      tma_load_3d(smem + APB, &tmAP, full, 0, crow, 0);
      tma_load_3d(smem + TT, &tmT, full, 0, crow, 0);
      tma_load_3d(smem + DM, &tmDM, full, 0, crow, 0);
    }
    const size_t bidx = (static_cast<size_t>(row0) + r) * p.heads + h;
    const float beta = p.beta_f32 ? static_cast<const float*>(p.beta)[bidx]
                                  : bf16_to_f32(static_cast<const bf16*>(p.beta)[bidx]);
    bool ok = true;
    // ---- pass 1: dA' parts and dV ----
    if (r == 0) {
      ok = mbar_wait(full, ph, p.status);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < 8; ++j) umma_f16(tmem + 0, k128(dw, j), k128(kt, j), id_kk64, j > 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) umma_f16(tmem + 64, k128(ndu, j), k128(vq, j), id_kk64, j > 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f16(tmem + 128, mn(ap, j), mn(ndu, j), id_mm, j > 0);
        umma_commit(&mma[0]);
      }
    }
    ok = mbar_wait_spin(&mma[0], ph, p.status) && ok;
    if (!__syncthreads_and(ok)) break;
    tc_fence_after();
    if (r == 0) {   // V is consumed: bring Q into its place
      mbar_arrive_expect_tx(fullq, 16384);
      tma_load_3d(smem + VQ, &tmQ, fullq, x0, row0, 0);
      tma_load_3d(smem + VQ + 8192, &tmQ, fullq, x0 + 64, row0, 0);
    }
    // dV = -(A'^T (-dU)) -> staged over the -dU tile
    row128_to_tiles(lane_addr + 128, smem + NDU, r, -1.f, nullptr);
    // dA' = dW K^T - (-dU) V^T -> operand tile
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
      float a[32], s[32];
      ld_row32(lane_addr + c, a);
      ld_row32(lane_addr + 64 + c, s);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = a[8 * i + j] - s[8 * i + j];
        st_swz(smem + TMP, r, (c >> 3) + i, pack8(o));
      }
    }
    // tril(dM) in place (row r keeps columns <= r)
#pragma unroll
    for (int c16 = 0; c16 < 8; ++c16) {
      bf16x8* cell = reinterpret_cast<bf16x8*>(smem + DM + r * 128 + ((c16 ^ (r & 7)) << 4));
      if (8 * c16 + 7 > r) {
        float f[8];
        unpack8(*cell, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) if (8 * c16 + j > r) f[j] = 0.f;
        *cell = pack8(f);
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- pass 2: X = dA' A'^T, Y = dA'^T T (diagonal = dbeta part), dK = A'^T dW ----
    if (r == 0) {
      tc_fence_after();
      tma_store_3d(&tmDV, smem + NDU, x0, row0, 0);
      tma_store_3d(&tmDV, smem + NDU + 8192, x0 + 64, row0, 0);
      tma_store_commit();
#pragma unroll
      for (int j = 0; j < 4; ++j) umma_f16(tmem + 0, k64(tmp, j), k64(ap, j), id_kk64, j > 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) umma_f16(tmem + 64, mn(tmp, j), mn(tt, j), id_mm64, j > 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) umma_f16(tmem + 128, mn(ap, j), mn(dw, j), id_mm, j > 0);
      umma_commit(&mma[1]);
    }
    ok = mbar_wait_spin(&mma[1], ph, p.status);
    if (!__syncthreads_and(ok)) break;
    tc_fence_after();
    float dbeta = 0.f;
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
      float x[32], y[32];
      ld_row32(lane_addr + c, x);
      ld_row32(lane_addr + 64 + c, y);
#pragma unroll
      for (int i = 0; i < 32; ++i) if (c + i == r) dbeta = y[i];
#pragma unroll
      for (int i = 0; i < 4; ++i) st_swz(smem + TMP, r, (c >> 3) + i, pack8(x + 8 * i));
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- pass 3: -dA = T^T X, G = K K^T ----
    if (r == 0) {
      tc_fence_after();
#pragma unroll
      for (int j = 0; j < 4; ++j) umma_f16(tmem + 0, mn(tt, j), mn(tmp, j), id_mm64, j > 0);
#pragma unroll
      for (int j = 0; j < 8; ++j) umma_f16(tmem + 64, k128(kt, j), k128(kt, j), id_kk64, j > 0);
      umma_commit(&mma[2]);
    }
    ok = mbar_wait_spin(&mma[2], ph, p.status);
    if (!__syncthreads_and(ok)) break;
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
      float na[32], gk[32];
      ld_row32(lane_addr + c, na);
      ld_row32(lane_addr + 64 + c, gk);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const bool low = c + 8 * i + j < r;
          const float da = low ? -na[8 * i + j] : 0.f;
          dbeta = fmaf(da, low ? gk[8 * i + j] : 0.f, dbeta);
          o[j] = beta * da;
        }
        st_swz(smem + TMP, r, (c >> 3) + i, pack8(o));
      }
    }
    if (p.beta_f32) static_cast<float*>(p.dbeta)[bidx] = dbeta;
    else static_cast<bf16*>(p.dbeta)[bidx] = f32_to_bf16(dbeta);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- pass 4: dK += dG K + dG^T K + tril(dM)^T Q ; dQ = tril(dM) K ----
    if (r == 0) {
      ok = mbar_wait(fullq, ph, p.status);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f16(tmem + 128, k64(tmp, j), mn(kt, j), id_kn, 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f16(tmem + 128, mn(tmp, j), mn(kt, j), id_mm, 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f16(tmem + 128, mn(dm, j), mn(vq, j), id_mm, 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f16(tmem + 0, k64(dm, j), mn(kt, j), id_kn, j > 0);
        umma_commit(&mma[3]);
      }
      tma_store_wait_read<0>();   // dV has left the tile dK is staged in
    }
    ok = mbar_wait_spin(&mma[3], ph, p.status) && ok;
    if (!__syncthreads_and(ok)) break;
    tc_fence_after();
    {
      const size_t off = (static_cast<size_t>(crow) + r) * D;
      row128_to_tiles(lane_addr + 0, smem + DW, r, 1.f, p.dq_add ? p.dq_add + off : nullptr);
      row128_to_tiles(lane_addr + 128, smem + NDU, r, 1.f, p.dk_add ? p.dk_add + off : nullptr);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (r == 0) {
      tma_store_3d(&tmDQ, smem + DW, x0, row0, 0);
      tma_store_3d(&tmDQ, smem + DW + 8192, x0 + 64, row0, 0);
      tma_store_3d(&tmDK, smem + NDU, x0, row0, 0);
      tma_store_3d(&tmDK, smem + NDU + 8192, x0 + 64, row0, 0);
      tma_store_commit();
    }
  }
  if (r == 0) tma_store_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace dprep
}  // namespace pb

using namespace pb;

// q, k, v: bf16 [batch * seq_len, ld] row-major with head h at columns [128 h, 128 h + 128)
// (ld >= heads * 128, a multiple of 8); beta: [batch, seq_len, heads], fp32 or bf16.
// Outputs, chunk g = (b * heads + h) * n_chunks + n: W, U^ [g][64][128]; M, A', T [g][64][64].
PB_API int pb_delta_prep_fwd(const void* q, const void* k, const void* v, const void* beta,
                             int beta_f32, void* W, void* Uhat, void* M, void* Ap, void* T,
                             int batch, int seq_len, int heads, int ld, int* status,
                             int max_ctas, cudaStream_t st) {
  using namespace dprep;
  if (batch <= 0 || heads <= 0 || seq_len <= 0 || seq_len % C != 0 || ld < heads * D || ld % 8)
    return PB_BAD_ARG;
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(delta_prep_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  Params p;
  p.n_chunks = seq_len / C; p.heads = heads; p.seq_len = seq_len;
  p.total = batch * heads * p.n_chunks;
  p.beta = beta; p.beta_f32 = beta_f32; p.status = status;
  const uint64_t tok = static_cast<uint64_t>(batch) * seq_len;
  const uint64_t rows = static_cast<uint64_t>(p.total) * C;
  CUtensorMap tK, tQ, tV, tW, tU, tM, tA, tT;
  int r = 0;
  r |= make_tmap_3d(&tK, k, 2, static_cast<uint64_t>(heads) * D, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tQ, q, 2, static_cast<uint64_t>(heads) * D, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tV, v, 2, static_cast<uint64_t>(heads) * D, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tW, W, 2, D, rows, 1, D, 0, 64, C);
  r |= make_tmap_3d(&tU, Uhat, 2, D, rows, 1, D, 0, 64, C);
  r |= make_tmap_3d(&tM, M, 2, C, rows, 1, C, 0, 64, C);
  r |= make_tmap_3d(&tA, Ap, 2, C, rows, 1, C, 0, 64, C);
  r |= make_tmap_3d(&tT, T, 2, C, rows, 1, C, 0, 64, C);
  if (r != 0) return 1000 + r;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = 2 * sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > p.total) grid = p.total;
  delta_prep_fwd_kernel<<<grid, 64, SMEM_BYTES, st>>>(tK, tQ, tV, tW, tU, tM, tA, tT, p);
  return static_cast<int>(cudaGetLastError());
}

// Backward of pb_delta_prep_fwd. dW, ndU (= -dU), dq_add, dk_add: [total][64][128] bf16;
// dM (unmasked dO U^T), Ap, T: [total][64][64] bf16; dq, dk, dv: like q / k / v;
// dbeta: like beta. dq_add / dk_add may be null.
PB_API int pb_delta_prep_bwd(const void* q, const void* k, const void* v, const void* beta,
                             int beta_f32, const void* Ap, const void* T, const void* dW,
                             const void* ndU, const void* dM, const void* dq_add,
                             const void* dk_add, void* dq, void* dk, void* dv, void* dbeta,
                             int batch, int seq_len, int heads, int ld, int* status,
                             int max_ctas, cudaStream_t st) {
  using namespace dprep;
  if (batch <= 0 || heads <= 0 || seq_len <= 0 || seq_len % C != 0 || ld < heads * D || ld % 8)
    return PB_BAD_ARG;
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(delta_prep_bwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         bwd::SMEM_BWD);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  BwdParams p;
  p.n_chunks = seq_len / C; p.heads = heads; p.seq_len = seq_len;
  p.total = batch * heads * p.n_chunks;
  p.beta = beta; p.beta_f32 = beta_f32;
  p.dq_add = static_cast<const bf16*>(dq_add);
  p.dk_add = static_cast<const bf16*>(dk_add);
  p.dbeta = dbeta; p.status = status;
  const uint64_t tok = static_cast<uint64_t>(batch) * seq_len;
  const uint64_t rows = static_cast<uint64_t>(p.total) * C;
  const uint64_t hd = static_cast<uint64_t>(heads) * D;
  CUtensorMap tK, tQ, tV, tDW, tNDU, tDM, tA, tT, tDQ, tDK, tDV;
  int r = 0;
  r |= make_tmap_3d(&tK, k, 2, hd, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tQ, q, 2, hd, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tV, v, 2, hd, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tDW, dW, 2, D, rows, 1, D, 0, 64, C);
  r |= make_tmap_3d(&tNDU, ndU, 2, D, rows, 1, D, 0, 64, C);
  r |= make_tmap_3d(&tDM, dM, 2, C, rows, 1, C, 0, 64, C);
  r |= make_tmap_3d(&tA, Ap, 2, C, rows, 1, C, 0, 64, C);
  r |= make_tmap_3d(&tT, T, 2, C, rows, 1, C, 0, 64, C);
  r |= make_tmap_3d(&tDQ, dq, 2, hd, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tDK, dk, 2, hd, tok, 1, ld, 0, 64, C);
  r |= make_tmap_3d(&tDV, dv, 2, hd, tok, 1, ld, 0, 64, C);
  if (r != 0) return 1000 + r;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = 2 * sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > p.total) grid = p.total;
  delta_prep_bwd_kernel<<<grid, 64, bwd::SMEM_BWD, st>>>(tK, tQ, tV, tDW, tNDU, tDM, tA, tT, tDQ,
                                                           tDK, tDV, p);
  return static_cast<int>(cudaGetLastError());
}
