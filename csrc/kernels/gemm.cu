// Persistent warp-specialised bf16 GEMM on the 5th-gen tensor cores (sm_100a).
//
//   C[b] = alpha * A[b] * B[b]^T + beta * D[b]
//
// A is logically [M, K], B logically [N, K]. Either operand may be stored
// K-major (row-major as written) or MN-major (the transpose, contraction index
// outermost): that covers y = x W^T, dx = dy W, dW = dy^T x and the
// Newton-Schulz products without materialising a transpose.
//
// Structure per CTA (one per SM, persistent over a swizzled tile order):
//   warp 0     TMA producer: cp.async.bulk.tensor tiles, 128B swizzle, into a
//              STAGES-deep shared-memory ring guarded by full/empty mbarriers
//   warp 1     allocates tensor memory; one lane issues tcgen05.mma
//              (128 x BN x 16 per instruction), tcgen05.commit frees ring slots
//              and publishes the accumulator
//   warps 2-5  epilogue: tcgen05.ld the fp32 accumulator (two accumulators in
//              tensor memory so the next tile's main loop overlaps), scale,
//              add D, convert, store
// No cluster launch and no multicast: safe in multi-GPU code.
#include <cuda.h>

#include "common.cuh"

namespace pb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row

struct GemmParams {
  int M, N, K, batch;
  void* C;
  const void* D;
  long ldc, strideC, ldd, strideD;
  float alpha, beta;
  int out_f32, d_f32;
  int a_mn, b_mn;
  int tma_store;  // epilogue stages tiles in shared memory and stores them with TMA
  int m_group;    // row blocks per rasterisation group (all column blocks of a group before the next)
  int* status;
  // Grouped modes (both null for the plain GEMM):
  //  mblk_group[m_blk]: rows of A / C are grouped (128-aligned) and row block m_blk multiplies
  //    batch entry mblk_group[m_blk] of B (negative: the block is padding and is skipped).
  //  k_off / k_len[b]: batch entry b contracts over rows [k_off[b], k_off[b] + k_len[b]) of the
  //    two MN-major operands, which are shared by all entries (k_len a multiple of 64; 0 skips).
  const int* mblk_group;
  const int* k_off;
  const int* k_len;
  // All-gather mode (ag_ready null for every other GEMM): B is this rank's full-size copy of a
  // matrix whose rows [q R, (q + 1) R) are owned by rank q. Two copier warps per CTA pull the
  // other ranks' rows from their buffers (ag_src[q], same layout) into B in 8-row items, ring
  // order starting after this rank, and add the rows they landed to ag_ready[n_blk]; the TMA
  // producer of a tile waits until its panel holds ag_epoch x (remote rows of the panel).
  // Tiles walk the panels in the same ring order, all row blocks of a panel before the next.
  const void* ag_src[8];
  void* ag_dst;
  uint32_t* ag_ready;
  long ag_ld;
  int ag_rank, ag_world, ag_rows_per_rank;
  uint32_t ag_epoch;
  uint64_t ag_budget_ns;
};

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int EPI_BYTES = 4 * 2 * 4096;  // per epilogue warp: two 32-row x 128 B slabs
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

// One warp's share of a finished accumulator: 32 rows (tensor-memory lanes of `t_addr`) x BN
// columns, scaled, D added, converted and stored. `y0` is the matrix row of lane 0, `n0` the
// first column, `my_epi_base` the warp's 8 KB staging area for the TMA-store path; the warp
// handles tile columns [col_lo, col_hi) (multiples of 64).
template <int BN>
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, const CUtensorMap* tmC,
                                              uint32_t t_addr, uint8_t* my_epi_base, int b, int y0,
                                              int n0, int lane, int col_lo = 0, int col_hi = BN) {
  const int row = y0 + lane;
  const bool row_ok = row < p.M;
  const size_t c_off = static_cast<size_t>(b) * p.strideC + static_cast<size_t>(row) * p.ldc;
  const size_t d_off = static_cast<size_t>(b) * p.strideD + static_cast<size_t>(row) * p.ldd;
  if (p.tma_store) {
    // Stage 32 rows x 128 bytes per warp in the TMA swizzle layout, then one bulk
    // tensor store per slab: coalesced, asynchronous, clipped at the matrix edge.
    uint8_t* my_epi = my_epi_base;
    const int cols_per_slab = p.out_f32 ? 32 : 64;
    const uint64_t evict_first = l2_policy_evict_first();
    const int halves = cols_per_slab / 32;
#pragma unroll 1
    for (int sl = col_lo / cols_per_slab; sl * cols_per_slab < col_hi; ++sl) {
      const int x0 = n0 + sl * cols_per_slab;
      uint8_t* buf = my_epi + (sl & 1) * 4096;
      // the whole slab is requested from tensor memory before the wait for the staging buffer,
      // so the two latencies overlap
      uint32_t ra[32], rb[32];
      tmem_ld_32x32b_x32(t_addr + sl * cols_per_slab, ra);
      if (halves == 2) tmem_ld_32x32b_x32(t_addr + sl * cols_per_slab + 32, rb);
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
      tmem_ld_wait();
      auto chunk = [&](const uint32_t (&r)[32], const int hf) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        const int col0 = x0 + hf * 32;
        if (p.D != nullptr && row_ok && col0 < p.N) {
          const bool full_chunk = (col0 + 32 <= p.N);
          if (p.d_f32) {
            const float* dp = static_cast<const float*>(p.D) + d_off + col0;
            if (full_chunk && (p.ldd % 4 == 0)) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 d4 = reinterpret_cast<const float4*>(dp)[i];
                v[4 * i] += p.beta * d4.x; v[4 * i + 1] += p.beta * d4.y;
                v[4 * i + 2] += p.beta * d4.z; v[4 * i + 3] += p.beta * d4.w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) v[i] += p.beta * dp[i];
            }
          } else {
            const bf16* dp = static_cast<const bf16*>(p.D) + d_off + col0;
            if (full_chunk && (p.ldd % 8 == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float f[8];
                unpack8(reinterpret_cast<const bf16x8*>(dp)[i], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[8 * i + j] += p.beta * f[j];
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) v[i] += p.beta * bf16_to_f32(dp[i]);
            }
          }
        }
        uint8_t* rowp = buf + lane * 128;
        if (p.out_f32) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(rowp + ((i ^ (lane & 7)) << 4)) =
                make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            bf16x8 pk;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              pk.v[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
            *reinterpret_cast<bf16x8*>(rowp + (((hf * 4 + i) ^ (lane & 7)) << 4)) = pk;
          }
        }
      };
      chunk(ra, 0);
      if (halves == 2) chunk(rb, 1);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && x0 < p.N && y0 < p.M) tma_store_3d_hint(tmC, buf, x0, y0, b, evict_first);
      if (lane == 0) tma_store_commit();
    }
  } else
#pragma unroll 1
  for (int c = col_lo; c < col_hi; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_addr + c, r);
    tmem_ld_wait();
    const int col0 = n0 + c;
    if (row_ok && col0 < p.N) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
      const bool full_chunk = (col0 + 32 <= p.N);
      // All indexing below is compile-time so v stays in registers; ragged
      // edges use the same unrolled loops with a per-element predicate.
      if (p.D != nullptr) {
        if (p.d_f32) {
          const float* dp = static_cast<const float*>(p.D) + d_off + col0;
          if (full_chunk && (p.ldd % 4 == 0)) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 d4 = reinterpret_cast<const float4*>(dp)[i];
              v[4 * i] += p.beta * d4.x; v[4 * i + 1] += p.beta * d4.y;
              v[4 * i + 2] += p.beta * d4.z; v[4 * i + 3] += p.beta * d4.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += p.beta * dp[i];
          }
        } else {
          const bf16* dp = static_cast<const bf16*>(p.D) + d_off + col0;
          if (full_chunk && (p.ldd % 8 == 0)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float f[8];
              unpack8(reinterpret_cast<const bf16x8*>(dp)[i], f);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[8 * i + j] += p.beta * f[j];
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) v[i] += p.beta * bf16_to_f32(dp[i]);
          }
        }
      }
      if (p.out_f32) {
        float* cp = static_cast<float*>(p.C) + c_off + col0;
        if (full_chunk && (p.ldc % 4 == 0)) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(cp)[i] =
                make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) cp[i] = v[i];
        }
      } else {
        bf16* cp = static_cast<bf16*>(p.C) + c_off + col0;
        if (full_chunk && (p.ldc % 8 == 0)) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            bf16x8 pk;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              pk.v[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
            reinterpret_cast<bf16x8*>(cp)[i] = pk;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) cp[i] = f32_to_bf16(v[i]);
        }
      }
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(256, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smA = smem;
  uint8_t* smB = smem + STAGES * S::A_BYTES;
  uint8_t* smEpi = smem + STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES + S::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = num_m * num_n;
  const long total_tiles = static_cast<long>(tiles_per_batch) * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
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

  auto tile_coords = [&](long t, int& b, int& m_blk, int& n_blk) {
    b = static_cast<int>(t / tiles_per_batch);
    const int r = static_cast<int>(t % tiles_per_batch);
    if (p.ag_ready != nullptr) {   // panels in ring order from this rank's first panel
      m_blk = r % num_m;
      n_blk = ((p.ag_rank * p.ag_rows_per_rank) / BN + r / num_m) % num_n;
      return;
    }
    const int group = p.m_group * num_n;
    const int g = r / group;
    const int first_m = g * p.m_group;
    const int gsz = min(num_m - first_m, p.m_group);
    m_blk = first_m + (r % group) % gsz;
    n_blk = (r % group) / gsz;
  };
  // operand batch indices, first contraction row and contraction blocks of a tile
  auto tile_group = [&](int b, int m_blk, int& b_a, int& b_b, int& k_base, int& nkb) {
    b_a = b; b_b = b; k_base = 0; nkb = num_kb;
    if (p.mblk_group != nullptr) {
      b_b = p.mblk_group[m_blk];
      return b_b >= 0;
    }
    if (p.k_len != nullptr) {
      b_a = b_b = 0;
      k_base = p.k_off[b];
      nkb = p.k_len[b] / BK;
      return nkb > 0;
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, m_blk, n_blk;
        tile_coords(t, b, m_blk, n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        int b_a, b_b, k_base, nkb;
        if (!tile_group(b, m_blk, b_a, b_b, k_base, nkb)) continue;
        if (p.ag_ready != nullptr) {
          // rows of this panel that other ranks own must have landed in B
          const int lo = max(n0, p.ag_rank * p.ag_rows_per_rank);
          const int hi = min(min(n0 + BN, p.N), (p.ag_rank + 1) * p.ag_rows_per_rank);
          const int remote = min(n0 + BN, p.N) - n0 - max(hi - lo, 0);
          if (remote > 0) {
            if (!wait_flag_ge(p.ag_ready + n_blk, p.ag_epoch * static_cast<uint32_t>(remote),
                              p.ag_budget_ns, p.status)) { ok = false; break; }
            // the rows were written by ordinary stores; the bulk loads below read through the
            // asynchronous proxy
            asm volatile("fence.proxy.async.global;" ::: "memory");
          }
        }
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, p.status)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[s], S::STAGE_BYTES);
          uint8_t* a_dst = smA + s * S::A_BYTES;
          uint8_t* b_dst = smB + s * S::B_BYTES;
          const int k0 = k_base + kb * BK;
          if (!p.a_mn) {
            tma_load_3d(a_dst, &tmA, &full[s], k0, m0, b_a);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(a_dst + c * 8192, &tmA, &full[s], m0 + c * 64, k0, b_a);
          }
          if (!p.b_mn) {
            tma_load_3d(b_dst, &tmB, &full[s], k0, n0, b_b);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(b_dst + c * 8192, &tmB, &full[s], n0 + c * 64, k0, b_b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 1, BM, BN, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u);
      // descriptor words hoisted out of the loops: high words constant, low words
      // (stage base + step * j) in 16-byte units, so the issue loop is a handful of instructions
      constexpr uint32_t HI = sdesc_hi_sw128(1024);
      const uint32_t a_lo0 = sdesc_lo(smem_u32(smA), p.a_mn ? 8192 : 16);
      const uint32_t b_lo0 = sdesc_lo(smem_u32(smB), p.b_mn ? 8192 : 16);
      const uint32_t a_step = (p.a_mn ? 2048u : 32u) >> 4, b_step = (p.b_mn ? 2048u : 32u) >> 4;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int nkb = num_kb;
        if (p.mblk_group != nullptr || p.k_len != nullptr) {
          int b, m_blk, n_blk, b_a, b_b, k_base;
          tile_coords(t, b, m_blk, n_blk);
          if (!tile_group(b, m_blk, b_a, b_b, k_base, nkb)) continue;
        }
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait_spin(&full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(s) * (S::A_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(s) * (S::B_BYTES >> 4);
          // K-major: 16 elements = 32 bytes along the swizzled row.
          // MN-major: 16 k-rows = two 8-row groups of 1024 bytes.
#pragma unroll
          for (int j = 0; j < BK / 16; ++j)
            umma_f16_words(d_tmem, a_lo + j * a_step, HI, b_lo + j * b_step, HI, idesc,
                           (kb > 0 || j > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else if (warp >= 6) {
    // ------------------- all-gather copier (idle in every other mode) -------------------
    if (p.ag_ready != nullptr) {
      const int R = p.ag_rows_per_rank;
      const int items_per_rank = (R + 7) / 8;
      const long n_items = static_cast<long>(p.ag_world - 1) * items_per_rank;
      const int vec_per_row = p.K / 8;   // 16-byte vectors
      for (long it = static_cast<long>(blockIdx.x) * 2 + (warp - 6); it < n_items;
           it += static_cast<long>(gridDim.x) * 2) {
        const int src = (p.ag_rank + 1 + static_cast<int>(it / items_per_rank)) % p.ag_world;
        const int r0 = src * R + static_cast<int>(it % items_per_rank) * 8;
        const int nrows = min(8, (src + 1) * R - r0);
        const bf16x8* sp = static_cast<const bf16x8*>(p.ag_src[src]);
        bf16x8* dp = static_cast<bf16x8*>(p.ag_dst);
        for (int rr = 0; rr < nrows; ++rr) {
          const size_t base = (static_cast<size_t>(r0 + rr) * p.ag_ld) / 8;
          int j = lane;
          for (; j + 96 < vec_per_row; j += 128) {   // four peer loads in flight per lane
            const bf16x8 a = sp[base + j], b = sp[base + j + 32], c = sp[base + j + 64],
                         d = sp[base + j + 96];
            dp[base + j] = a; dp[base + j + 32] = b; dp[base + j + 64] = c; dp[base + j + 96] = d;
          }
          for (; j < vec_per_row; j += 32) dp[base + j] = sp[base + j];
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(p.ag_ready + r0 / BN, static_cast<uint32_t>(nrows));
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int acc = 0;
    uint32_t acc_ph = 0;
    bool ok = true;
    for (long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int b, m_blk, n_blk;
      tile_coords(t, b, m_blk, n_blk);
      const int n0 = n_blk * BN;
      {
        int b_a, b_b, k_base, nkb;
        if (!tile_group(b, m_blk, b_a, b_b, k_base, nkb)) continue;
      }
      if (!mbar_wait(&tfull[acc], acc_ph, p.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      epilogue_rows<BN>(p, &tmC, t_addr, smEpi + (warp - 2) * 8192, b, m_blk * BM + q * 32, n0, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
  }

  if (warp >= 2 && warp < 6 && lane == 0) tma_store_wait<0>();  // staged tiles must be read out before exit
  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    // A wait ran out somewhere: give copies that may still be in flight a
    // bounded moment to land before shared memory is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair variant (plain and batched products only): a cluster of two CTAs on neighbouring SMs
// computes one 256 x 256 tile with tcgen05.mma.cta_group::2. Each CTA loads its 128 rows of A and
// its 128 of the tile's 256 rows of B, so a k-block costs each SM 32 KB of shared-memory reads
// instead of 48 KB: the operand reads of the single-CTA 128 x 256 tile take three quarters of the
// shared-memory bandwidth, and the epilogue's staging traffic competes for the rest.
//   even CTA: warp 0 loads, warp 1 lane 0 issues the pair's MMAs, warps 2-9 drain rows 0..127
//   odd CTA:  warp 0 loads (completions counted on the even CTA's barrier), warps 2-9 drain
//             rows 128..255 from its own tensor memory
// (eight epilogue warps, two per tensor-memory lane quarter: with four, draining a 256-column
// accumulator took longer than a K = 2048 main loop)
// Barriers: full[s] lives in the even CTA (2 x stage bytes); empty[s] and tfull[a] exist in both
// and are signalled by one tcgen05.commit to both CTAs; tempty[a] lives in the even CTA and
// collects the sixteen epilogue warps of the pair. Loads carry no cluster multicast.
// ---------------------------------------------------------------------------
struct Gemm2Smem {
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = 128 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 5;
  static constexpr int EPI_WARPS = 8;
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * 4096;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
  static constexpr int THREADS = (2 + EPI_WARPS) * 32;
};

__global__ void __launch_bounds__(Gemm2Smem::THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using S = Gemm2Smem;
  constexpr int STAGES = S::STAGES;
  constexpr int BN = 256, BM2 = 256;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared-memory window starts at the same offset in both CTAs, so the aligned
  // carve-up below is identical in the pair (the pair MMA addresses both by one descriptor)
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* smA = smem;
  uint8_t* smB = smem + STAGES * S::A_BYTES;
  uint8_t* smEpi = smem + STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * S::STAGE_BYTES + S::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: even CTA (issues the MMAs), 1: odd CTA
  const long pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_m = (p.M + BM2 - 1) / BM2;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = num_m * num_n;
  const long total_tiles = static_cast<long>(tiles_per_batch) * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 2 * S::EPI_WARPS);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    // Each CTA allocates all 512 columns of its own SM (one CTA per SM by shared-memory size), so
    // both accumulators start at column 0 in either CTA and one address serves the pair's MMA.
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  cluster_sync_all();      // barriers of both CTAs initialised before any remote arrival
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coords = [&](long t, int& b, int& m_blk, int& n_blk) {
    b = static_cast<int>(t / tiles_per_batch);
    const int r = static_cast<int>(t % tiles_per_batch);
    const int group = p.m_group * num_n;
    const int g = r / group;
    const int first_m = g * p.m_group;
    const int gsz = min(num_m - first_m, p.m_group);
    m_blk = first_m + (r % group) % gsz;
    n_blk = (r % group) / gsz;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (long t = pair; t < total_tiles && ok; t += n_pairs) {
        int b, m_blk, n_blk;
        tile_coords(t, b, m_blk, n_blk);
        const int m0 = m_blk * BM2 + static_cast<int>(rank) * 128;
        const int n0 = n_blk * BN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, p.status)) { ok = false; break; }
          if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * S::STAGE_BYTES);
          const uint32_t bar = cluster_map(smem_u32(&full[s]), 0);
          uint8_t* a_dst = smA + s * S::A_BYTES;
          uint8_t* b_dst = smB + s * S::B_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_3d_pair(a_dst, &tmA, bar, k0, m0, b);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_3d_pair(a_dst + c * 8192, &tmA, bar, m0 + c * 64, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d_pair(b_dst, &tmB, bar, k0, n0, b);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tma_load_3d_pair(b_dst + c * 8192, &tmB, bar, n0 + c * 64, k0, b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA) ------------------------------
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(1, 1, BM2, BN, p.a_mn ? 1u : 0u, p.b_mn ? 1u : 0u);
      // One issuing thread feeds both tensor cores: a k-block is four MMAs of 128 cycles each,
      // so everything between two MMAs is kept to a few instructions. The descriptors' high
      // words are constants; the low words are (stage base + step * j), all in 16-byte units.
      constexpr uint32_t HI = sdesc_hi_sw128(1024);
      const uint32_t a_lo0 = sdesc_lo(smem_u32(smA), p.a_mn ? 8192 : 16);
      const uint32_t b_lo0 = sdesc_lo(smem_u32(smB), p.b_mn ? 8192 : 16);
      const uint32_t a_step = (p.a_mn ? 2048u : 32u) >> 4, b_step = (p.b_mn ? 2048u : 32u) >> 4;
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 0;
      bool ok = true;
      for (long t = pair; t < total_tiles && ok; t += n_pairs) {
        if (!mbar_wait_cluster(&tempty[acc], acc_ph ^ 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_spin(&full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + static_cast<uint32_t>(s) * (S::A_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + static_cast<uint32_t>(s) * (S::B_BYTES >> 4);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j)
            umma_f16_pair_words(d_tmem, a_lo + j * a_step, HI, b_lo + j * b_step, HI, idesc,
                                (kb > 0 || j > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s], 3);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull[acc], 3);
        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_ph = 0;
    const uint32_t tempty0 = cluster_map(smem_u32(&tempty[0]), 0);
    for (long t = pair; t < total_tiles; t += n_pairs) {
      int b, m_blk, n_blk;
      tile_coords(t, b, m_blk, n_blk);
      if (!mbar_wait(&tfull[acc], acc_ph, p.status)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      // two warps per lane quarter: warps 2-5 drain columns 0..127, warps 6-9 columns 128..255
      const int c_lo = warp < 6 ? 0 : 128;
      epilogue_rows<BN>(p, &tmC, t_addr, smEpi + (warp - 2) * 8192, b,
                        m_blk * BM2 + static_cast<int>(rank) * 128 + q * 32, n_blk * BN, lane, c_lo,
                        c_lo + 128);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + acc * 8);
      if (++acc == 2) { acc = 0; acc_ph ^= 1; }
    }
  }

  if (warp >= 2 && lane == 0) tma_store_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  // neither CTA leaves (or frees tensor memory) while its peer may still signal its barriers,
  // read its operand tiles or write its accumulators
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 3-D map over a [batch][outer][inner] bf16 (or 1-byte) tensor, 128B swizzle.
int make_tmap_3d(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                 uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {ld_elems * elem_bytes,
                           (batch > 1 ? batch_stride_elems : ld_elems * outer) * elem_bytes};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                   : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUresult r =
      fn(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

static int g_num_sms = 0;
int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                const GemmParams& p, int max_ctas,
                cudaStream_t st) {
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmSmem<BN>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  const long tiles =
      static_cast<long>((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = static_cast<int>(tiles);
  gemm_bf16_kernel<BN><<<grid, 256, GemmSmem<BN>::TOTAL, st>>>(tmA, tmB, tmC, p);
  return static_cast<int>(cudaGetLastError());
}

// Launch of the CTA-pair kernel: clusters of two, as many pairs as can be resident.
int launch_gemm2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                 const GemmParams& p, int max_ctas, cudaStream_t st) {
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  static int max_pairs = 0;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(Gemm2Smem::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Gemm2Smem::TOTAL;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(gemm2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Gemm2Smem::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    cfg.gridDim = dim3(num_sms() & ~1, 1, 1);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm2_bf16_kernel, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); n = num_sms() / 2; }
    max_pairs = n > 0 ? n : num_sms() / 2;
    if (max_pairs > num_sms() / 2) max_pairs = num_sms() / 2;
    attr_once.done();
  }
  const long tiles = static_cast<long>((p.M + 255) / 256) * ((p.N + 255) / 256) * p.batch;
  long pairs = max_pairs;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) pairs = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm2_bf16_kernel, tmA, tmB, tmC, p);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

int gemm2_pairs_resident() { return num_sms() / 2; }

}  // namespace pb

using namespace pb;

static int g_gemm_variant = 0;
// Kernel-variant selection (the default, 0, picks by shape): bit 0 forces the 128-wide tile,
// bit 2 the direct-store epilogue, bit 3 keeps every product on the single-CTA kernel. Every
// variant computes the same product; the tests run them against each other.
PB_API int pb_gemm_set_variant(int flags) {
  if (flags & ~(1 | 4 | 8)) return PB_BAD_ARG;
  g_gemm_variant = flags;
  return 0;
}

// C = alpha * A * B^T + beta * D.  See the header comment for the layouts.
//   a_mn == 0: A stored [M, K] with row stride lda;  a_mn == 1: stored [K, M], row stride lda
//   b_mn == 0: B stored [N, K] with row stride ldb;  b_mn == 1: stored [K, N], row stride ldb
// Strides are in elements. Base pointers 16-byte aligned, lda/ldb multiples of 8.
// `status` (device int, may be null) latches a non-zero code if a bounded wait ran out.
// `max_ctas` > 0 limits the persistent grid (leaves SMs for a concurrent kernel).
static int gemm_impl(const void* A, const void* B, void* C, const void* D, int M, int N, int K,
                     int batch, long lda, long ldb, long ldc, long ldd, long strideA,
                     long strideB, long strideC, long strideD, int a_mn, int b_mn, int out_f32,
                     int d_f32, float alpha, float beta, int* status, int max_ctas,
                     cudaStream_t st, const int* mblk_group, int b_batch, const int* k_off,
                     const int* k_len);

// all-gather arguments of the call in progress (host side, set only by pb_gemm_bf16_ag)
struct AgArgs {
  const void* src[8];
  uint32_t* ready;
  int rank, world, rows_per_rank;
  uint32_t epoch;
  uint64_t budget_ns;
};
static thread_local const AgArgs* g_ag = nullptr;

// C = A W^T where W [N, K] is sharded by rows over `world` ranks and gathered by the kernel
// itself: w_ptrs[q] is rank q's full-size buffer (its own rows valid), w_ptrs[rank] doubles as the
// local destination. ready: uint32 [ceil(N / 256)] on this GPU, zero before the first call and
// owned by this weight; epoch counts the calls (1, 2, ...). N / world must be a multiple of 8,
// N > 128. Peers must not rewrite their rows while the call runs.
PB_API int pb_gemm_bf16_ag(const void* A, void* const* w_ptrs, void* C, int M, int N, int K, long lda,
                           long ldw, long ldc, int rank, int world, void* ready, int epoch,
                           long budget_ns, int* status, cudaStream_t st) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || N % world != 0 ||
      (N / world) % 8 != 0 || N <= 128 || K % 8 != 0 || epoch <= 0 || ready == nullptr)
    return PB_BAD_ARG;
  AgArgs a;
  for (int i = 0; i < 8; ++i) a.src[i] = i < world ? w_ptrs[i] : nullptr;
  a.ready = static_cast<uint32_t*>(ready);
  a.rank = rank; a.world = world; a.rows_per_rank = N / world;
  a.epoch = static_cast<uint32_t>(epoch);
  a.budget_ns = static_cast<uint64_t>(budget_ns);
  g_ag = &a;
  const int rc = gemm_impl(A, w_ptrs[rank], C, nullptr, M, N, K, 1, lda, ldw, ldc, ldc, 0, 0, 0, 0, 0, 0,
                           0, 0, 1.f, 0.f, status, 0, st, nullptr, 0, nullptr, nullptr);
  g_ag = nullptr;
  return rc;
}

PB_API int pb_gemm_bf16(const void* A, const void* B, void* C, const void* D, int M, int N, int K,
                        int batch, long lda, long ldb, long ldc, long ldd, long strideA,
                        long strideB, long strideC, long strideD, int a_mn, int b_mn, int out_f32,
                        int d_f32, float alpha, float beta, int* status, int max_ctas,
                        cudaStream_t st) {
  return gemm_impl(A, B, C, D, M, N, K, batch, lda, ldb, ldc, ldd, strideA, strideB, strideC,
                   strideD, a_mn, b_mn, out_f32, d_f32, alpha, beta, status, max_ctas, st, nullptr,
                   0, nullptr, nullptr);
}

// Grouped product for mixture-of-experts layers: C[rows of block m] = A[rows] * B[g(m)]^T,
// A [M, K] and C [M, N] with their rows grouped by expert in 128-row blocks, B [groups, N, K]
// (or [groups, K, N] with b_mn); mblk_group (device, one int per 128-row block) names the
// group of each block, negative = padding block, skipped (its C rows are left untouched).
PB_API int pb_gemm_bf16_grouped(const void* A, const void* B, void* C, int M, int N, int K,
                                int groups, long lda, long ldb, long ldc, long strideB, int b_mn,
                                const int* mblk_group, int* status, int max_ctas,
                                cudaStream_t st) {
  if (groups <= 0 || mblk_group == nullptr) return PB_BAD_ARG;
  return gemm_impl(A, B, C, nullptr, M, N, K, 1, lda, ldb, ldc, 0, 0, strideB, 0, 0, 0, b_mn, 0, 0,
                   1.f, 0.f, status, max_ctas, st, mblk_group, groups, nullptr, nullptr);
}

// Grouped weight gradient: for every group g, C[g] (+)= A[rows_g]^T * B[rows_g] where
// rows_g = [k_off[g], k_off[g] + k_len[g]) of the row-grouped A [R, M] and B [R, N] (k_len a
// multiple of 64, device arrays). C, D: [groups, M, N]; beta = 1 with D = C accumulates.
// Groups with k_len 0 are skipped (C left untouched).
PB_API int pb_gemm_bf16_grouped_wgrad(const void* A, const void* B, void* C, const void* D, int M,
                                      int N, int R, int groups, long lda, long ldb, long ldc,
                                      long strideC, int out_f32, int d_f32, float beta,
                                      const int* k_off, const int* k_len, int* status,
                                      int max_ctas, cudaStream_t st) {
  if (groups <= 0 || k_off == nullptr || k_len == nullptr) return PB_BAD_ARG;
  return gemm_impl(A, B, C, D, M, N, R, groups, lda, ldb, ldc, ldc, 0, 0, strideC, strideC, 1, 1,
                   out_f32, d_f32, 1.f, beta, status, max_ctas, st, nullptr, 0, k_off, k_len);
}

static int gemm_impl(const void* A, const void* B, void* C, const void* D, int M, int N, int K,
                     int batch, long lda, long ldb, long ldc, long ldd, long strideA,
                     long strideB, long strideC, long strideD, int a_mn, int b_mn, int out_f32,
                     int d_f32, float alpha, float beta, int* status, int max_ctas,
                     cudaStream_t st, const int* mblk_group, int b_batch, const int* k_off,
                     const int* k_len) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return PB_BAD_ARG;
  if ((lda % 8) != 0 || (ldb % 8) != 0) return PB_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return PB_BAD_ARG;
  if (batch > 1 && k_len == nullptr && ((strideA % 8) != 0 || (strideB % 8) != 0))
    return PB_BAD_ARG;
  // operand batch counts: shared 2-D operands in the grouped weight gradient, per-group B
  // in the grouped forward product
  const int batch_a = (k_len != nullptr) ? 1 : batch;
  const int batch_b = (k_len != nullptr) ? 1 : (mblk_group != nullptr ? b_batch : batch);
  if (mblk_group != nullptr && (strideB % 8) != 0) return PB_BAD_ARG;
  const bool bn256 = N > 128 && !(g_gemm_variant & 1);
  // CTA pairs (256 x 256 tiles) for plain and batched products; grouped and all-gather modes and
  // limited grids stay on one CTA. A pair tile covers two single-CTA tiles, so the waves fill
  // alike, except when the last row block is at most half a pair tile: then the pair kernel
  // needs enough tiles for that waste not to matter.
  const long pair_tiles = static_cast<long>((M + 255) / 256) * ((N + 255) / 256) * batch;
  const int m_tail = M % 256;
  const bool pair = bn256 && mblk_group == nullptr && k_len == nullptr && g_ag == nullptr &&
                    !(g_gemm_variant & 8) && M > 128 && (max_ctas <= 0 || max_ctas >= num_sms()) &&
                    (m_tail == 0 || m_tail > 128 || pair_tiles >= 2 * gemm2_pairs_resident());
  const int BN = bn256 ? 256 : 128;
  CUtensorMap tmA, tmB;
  int r;
  if (!a_mn)
    r = make_tmap_3d(&tmA, A, 2, K, M, batch_a, lda, strideA, BK, BM);
  else
    r = make_tmap_3d(&tmA, A, 2, M, K, batch_a, lda, strideA, 64, BK);
  if (r != 0) return 1000 + r;
  if (!b_mn)
    r = make_tmap_3d(&tmB, B, 2, K, N, batch_b, ldb, strideB, BK, pair ? 128 : BN);
  else
    r = make_tmap_3d(&tmB, B, 2, N, K, batch_b, ldb, strideB, 64, BK);
  if (r != 0) return 2000 + r;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.C = C; p.D = D;
  p.ldc = ldc; p.strideC = strideC; p.ldd = ldd; p.strideD = strideD;
  p.alpha = alpha; p.beta = beta;
  p.out_f32 = out_f32; p.d_f32 = d_f32;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.status = status;
  {
    // Rasterisation: the A panels of a group of row blocks stay in L2 while the B panels stream
    // past them once per group, so B is read from DRAM (row blocks / group) times. The group is
    // as tall as lets its A panels take about 48 MB of the 126 MB L2, and at least 8 blocks so
    // that a wave of tiles stays near-square when the panels are too long to be resident.
    const long panel_bytes = static_cast<long>(pair ? 256 : BM) * K * 2;
    long g = (48L << 20) / (panel_bytes > 0 ? panel_bytes : 1);
    if (g < 8) g = 8;
    if (g > 64) g = 64;
    // a B that fits in L2 next to the group is not re-read whatever the group: keep the wave square
    if (static_cast<long>(N) * K * 2 <= (32L << 20)) g = 8;
    p.m_group = static_cast<int>(g);
  }
  p.mblk_group = mblk_group; p.k_off = k_off; p.k_len = k_len;
  p.ag_ready = nullptr;
  if (g_ag != nullptr) {
    for (int i = 0; i < 8; ++i) p.ag_src[i] = g_ag->src[i];
    p.ag_dst = const_cast<void*>(B);
    p.ag_ready = g_ag->ready; p.ag_ld = ldb;
    p.ag_rank = g_ag->rank; p.ag_world = g_ag->world; p.ag_rows_per_rank = g_ag->rows_per_rank;
    p.ag_epoch = g_ag->epoch; p.ag_budget_ns = g_ag->budget_ns;
  }
  // TMA-store epilogue when the output rows are 16-byte aligned; else direct stores.
  const int cbytes = out_f32 ? 4 : 2;
  CUtensorMap tmC = tmA;
  p.tma_store = 0;
  if (!(g_gemm_variant & 4) && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      (ldc * cbytes) % 16 == 0 && (batch == 1 || (strideC * cbytes) % 16 == 0)) {
    if (make_tmap_3d(&tmC, C, cbytes, N, M, batch, ldc, strideC, out_f32 ? 32 : 64, 32) == 0)
      p.tma_store = 1;
  }
  if (pair) return launch_gemm2(tmA, tmB, tmC, p, max_ctas, st);
  return bn256 ? launch_gemm<256>(tmA, tmB, tmC, p, max_ctas, st)
               : launch_gemm<128>(tmA, tmB, tmC, p, max_ctas, st);
}
