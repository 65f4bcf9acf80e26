// Chunked delta-rule state scan on tcgen05 (sm_100a), forward and backward.
//
// The chunk-local WY operands (W = T b K, U^ = T b V, M = tril(Q K^T)) do not depend
// on the running state; what is sequential is, per (batch, head), the walk over
// chunks of 64 tokens with the 128 x 128 fp32 state S:
//
//   forward   Y = W S            U = U^ - Y          O = Q S + M U      S += K^T U
//   backward  dU = M^T dO + K dS                     dS += Q^T dO - W^T dU
//
// One CTA owns one (batch, head) sequence. The state lives in tensor memory for the
// whole walk (fp32, 128 lanes x 128 columns); every product is a tcgen05.mma with
// M = 128, N = 128; the bf16 image of the state and of U that the MMAs consume as
// their B operand is rewritten in shared memory each chunk in the 128-byte-swizzled
// layout TMA itself produces; Q/K/W/M and U^ (or dO) tiles arrive by TMA through a
// two-stage ring, and every output leaves by a TMA store from shared memory. Tiles with 64 token rows are used as 128-row A operands: the upper 64
// accumulator rows are then meaningless and are never read.
//
// warps 0-3: tensor-memory <-> registers <-> shared/global (lane = state row or token)
// warp 4   : MMA issue (one lane)          warp 5: TMA producer (one lane)
//
// Reference semantics: kernels/__init__.py:357-376 (per-token recurrence, post-update
// read) of the reference; the chunked algebra is this library's own.
#include <cuda.h>

#include "common.cuh"

namespace pb {

int make_tmap_3d(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                 uint32_t box_inner, uint32_t box_outer);

namespace dscan {

constexpr int C = 64;    // tokens per chunk
constexpr int D = 128;   // head dim (keys and values)
constexpr int TILE_W = 0, TILE_Q = 16384, TILE_K = 32768, TILE_M = 49152, TILE_DO = 57344;
constexpr int STAGE_BYTES = 57344 + 16384;  // W, Q, K (16 KB each), M (8 KB), U^ or dO (16 KB)
constexpr int XB_BYTES = 32768, UB_BYTES = 16384, OB_BYTES = 16384;
constexpr int TMEM_COLS = 512;
constexpr uint32_t COL_X = 0, COL_Y = 128, COL_O = 256;

struct Params {
  int n_chunks;        // chunks per sequence
  int n_seq;           // batch * heads
  int n_seg;           // segments per sequence: CTA (seq, seg) walks n_chunks / n_seg chunks from
                       //   x_init[seq * n_seg + seg] and leaves x_final[seq * n_seg + seg]
  int summary;         // 1: only the segment's affine map is wanted. Nothing but x_final is
                       //   written, the output products are skipped. Forward launches two CTAs
                       //   per segment: CTA half 0 starts from zero (x_final <- R, the state the
                       //   segment adds), half 1 from the identity with U^ = 0 (p_final <- P, the
                       //   linear part). Backward launches half 0 only (its linear part is P^T).
  float* p_final;      // [n_seq * n_seg, 128, 128], summary forward only
  int heads;           // > 0: Q, K, O and dO live in [batch * seq_len, ld] (head h at columns 128 h)
  int seq_len;         //      instead of the per-chunk layout
  const float* x_init; // [n_seq, 128, 128] or null (zeros)
  float* x_final;      // [n_seq, 128, 128] or null
  int* status;
};

template <bool BWD>
struct Smem {
  static constexpr int STAGE = STAGE_BYTES;
  static constexpr int XB = 2 * STAGE;
  static constexpr int UB = XB + XB_BYTES;
  static constexpr int OB = UB + UB_BYTES;
  static constexpr int BARS = OB + OB_BYTES;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

// 16-byte store of 8 bf16 into a [rows][64 n] 128B-swizzled MN-major operand chunk.
__device__ __forceinline__ void st_swz(uint8_t* chunk_base, int krow, int c16, const bf16x8& v) {
  *reinterpret_cast<bf16x8*>(chunk_base + krow * 128 + ((c16 ^ (krow & 7)) << 4)) = v;
}

template <bool BWD>
__global__ void __launch_bounds__(192, 1)
delta_scan_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQ,
                  const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmM,
                  const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmXB,
                  const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmO,
                  const Params p) {
  using S = Smem<BWD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* xb = smem + S::XB;
  uint8_t* ub = smem + S::UB;
  uint8_t* ob = smem + S::OB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BARS);
  uint64_t* full = bars;          // [2]
  uint64_t* empty = bars + 2;     // [2]
  uint64_t* x_ready = bars + 4;
  uint64_t* y_done = bars + 5;
  uint64_t* u_ready = bars + 6;
  uint64_t* o_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = p.n_seq * p.n_seg;
  const int half = static_cast<int>(blockIdx.x) / n_units;      // 1: the identity-start CTA
  const int unit = static_cast<int>(blockIdx.x) % n_units;      // seq * n_seg + seg
  const int seq = unit / p.n_seg;
  const int N = p.n_chunks / p.n_seg;                           // chunks this CTA walks
  const int n0 = (unit % p.n_seg) * N;                          // its first chunk
  const int NT = p.n_chunks;
  const bool sum = p.summary != 0;
  const bool lin = sum && half == 1;                            // linear part only: U^ = 0
  const bool tokmaj = p.heads > 0;
  const int tok0 = tokmaj ? (seq / p.heads) * p.seq_len : seq * NT * C;  // first token row
  const int tx = tokmaj ? (seq % p.heads) * D : 0;

  if (threadIdx.x == 0) {
    mbar_init(&full[0], 1); mbar_init(&full[1], 1);
    mbar_init(&empty[0], 1); mbar_init(&empty[1], 1);
    mbar_init(x_ready, 128); mbar_init(u_ready, 128);
    mbar_init(y_done, 1); mbar_init(o_done, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmM);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 5) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      // a forward summary needs neither Q nor M (no output product), its linear half no U^
      const bool need_qm = BWD || !sum;
      const bool need_fifth = BWD || !lin;
      const uint32_t stage_tx = 32768u + (need_qm ? 24576u : 0u) + (need_fifth ? 16384u : 0u);
      for (int it = 0; it < N; ++it) {
        const int n = n0 + (BWD ? (N - 1 - it) : it);
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, p.status)) break;
        mbar_arrive_expect_tx(&full[s], stage_tx);
        uint8_t* st = smem + s * S::STAGE;
        const int row = (seq * NT + n) * C;
        const int trow = tok0 + n * C;
        tma_load_3d(st + TILE_W, &tmW, &full[s], 0, row, 0);
        tma_load_3d(st + TILE_W + 8192, &tmW, &full[s], 64, row, 0);
        tma_load_3d(st + TILE_K, &tmK, &full[s], tx, trow, 0);
        tma_load_3d(st + TILE_K + 8192, &tmK, &full[s], tx + 64, trow, 0);
        if (need_qm) {
          tma_load_3d(st + TILE_Q, &tmQ, &full[s], tx, trow, 0);
          tma_load_3d(st + TILE_Q + 8192, &tmQ, &full[s], tx + 64, trow, 0);
          tma_load_3d(st + TILE_M, &tmM, &full[s], 0, row, 0);
        }
        if (BWD) {
          tma_load_3d(st + TILE_DO, &tmDO, &full[s], tx, trow, 0);
          tma_load_3d(st + TILE_DO + 8192, &tmDO, &full[s], tx + 64, trow, 0);
        } else if (need_fifth) {
          tma_load_3d(st + TILE_DO, &tmDO, &full[s], 0, row, 0);
          tma_load_3d(st + TILE_DO + 8192, &tmDO, &full[s], 64, row, 0);
        }
      }
    }
  } else if (warp == 4) {
    // -------------------------------- MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t id_kn = make_idesc(1, 1, 128, 128, 0, 1);  // A K-major, B MN-major
      const uint32_t id_nn = make_idesc(1, 1, 128, 128, 1, 1);  // A MN-major, B MN-major
      const uint32_t xb_a = smem_u32(xb), ub_a = smem_u32(ub);
      for (int it = 0; it < N; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1, cph = it & 1;
        const uint32_t st = smem_u32(smem + s * S::STAGE);
        if (!mbar_wait(&full[s], ph, p.status)) break;
        if (!mbar_wait_spin(x_ready, cph, p.status)) break;
        tc_fence_after();
        if (!BWD) {
          // Y = W X ; O = Q X
#pragma unroll
          for (int j = 0; j < 8; ++j)
            umma_f16(tmem + COL_Y,
                     make_sdesc_sw128(st + TILE_W + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024),
                     make_sdesc_sw128(xb_a + j * 2048, 16384, 1024), id_kn, j > 0);
          umma_commit(y_done);
          if (!sum) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              umma_f16(tmem + COL_O,
                       make_sdesc_sw128(st + TILE_Q + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024),
                       make_sdesc_sw128(xb_a + j * 2048, 16384, 1024), id_kn, j > 0);
          }
        } else {
          // Y = M^T dO + K X
#pragma unroll
          for (int j = 0; j < 4; ++j)
            umma_f16(tmem + COL_Y, make_sdesc_sw128(st + TILE_M + j * 2048, 8192, 1024),
                     make_sdesc_sw128(st + TILE_DO + j * 2048, 8192, 1024), id_nn, j > 0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            umma_f16(tmem + COL_Y,
                     make_sdesc_sw128(st + TILE_K + (j >> 2) * 8192 + (j & 3) * 32, 16, 1024),
                     make_sdesc_sw128(xb_a + j * 2048, 16384, 1024), id_kn, 1);
          umma_commit(y_done);
          // X += Q^T dO   (independent of dU: keeps the tensor core busy meanwhile)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            umma_f16(tmem + COL_X, make_sdesc_sw128(st + TILE_Q + j * 2048, 8192, 1024),
                     make_sdesc_sw128(st + TILE_DO + j * 2048, 8192, 1024), id_nn, 1);
        }
        if (!mbar_wait_spin(u_ready, cph, p.status)) break;
        tc_fence_after();
        if (!BWD) {
          // O += M U ; X += K^T U
          if (!sum) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              umma_f16(tmem + COL_O, make_sdesc_sw128(st + TILE_M + j * 32, 16, 1024),
                       make_sdesc_sw128(ub_a + j * 2048, 8192, 1024), id_kn, 1);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            umma_f16(tmem + COL_X, make_sdesc_sw128(st + TILE_K + j * 2048, 8192, 1024),
                     make_sdesc_sw128(ub_a + j * 2048, 8192, 1024), id_nn, 1);
        } else {
          // X += W^T (-dU)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            umma_f16(tmem + COL_X, make_sdesc_sw128(st + TILE_W + j * 2048, 8192, 1024),
                     make_sdesc_sw128(ub_a + j * 2048, 8192, 1024), id_nn, 1);
        }
        umma_commit(o_done);
        umma_commit(&empty[s]);
      }
    }
  } else {
    // ------------------------- state / token row threads -------------------------
    // Every result leaves through shared memory and a TMA store (coalesced, asynchronous):
    // the bf16 state image is stored from the very tile the MMAs read, U / -dU from the
    // operand tile, O from a staging tile. Thread 0 issues and tracks the stores.
    const int r = threadIdx.x;  // 0..127: tensor-memory lane = state row (or token row < 64)
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    auto sync_rows = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    {
      const float* x0 = (p.x_init && !sum) ? p.x_init + (static_cast<size_t>(unit) * D + r) * D : nullptr;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i)
          v[i] = x0 ? __float_as_uint(x0[c + i]) : ((lin && c + i == r) ? __float_as_uint(1.f) : 0u);
        tmem_st_32x32b_x32(lane_addr + COL_X + c, v);
      }
      tmem_st_wait();
    }
    // rows of the previous chunk's output: tensor memory -> staging tile
    auto stage_out = [&]() {
      if (!BWD && !sum && r < C) {
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(lane_addr + COL_O + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            bf16x8 pk;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              pk.v[j] = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]),
                                              __uint_as_float(v[8 * i + 2 * j + 1]));
            const int col = c + 8 * i;
            st_swz(ob + (col >> 6) * 8192, r, (col & 63) >> 3, pk);
          }
        }
      }
    };
    bool ok = true;
    for (int it = 0; it < N && ok; ++it) {
      const int n = n0 + (BWD ? (N - 1 - it) : it);
      const uint32_t cph = it & 1;
      const int g = seq * NT + n;
      if (it > 0) {
        if (!mbar_wait_spin(o_done, cph ^ 1, p.status)) { ok = false; break; }
        tc_fence_after();
      }
      // all earlier bulk stores have finished reading xb / ub / ob before they are rewritten
      if (r == 0) tma_store_wait_read<0>();
      sync_rows();
      if (it > 0) stage_out();
      // bf16 image of the state entering this chunk
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + COL_X + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          bf16x8 pk;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            pk.v[j] = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]),
                                            __uint_as_float(v[8 * i + 2 * j + 1]));
          const int col = c + 8 * i;
          st_swz(xb + (col >> 6) * 16384, r, (col & 63) >> 3, pk);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(x_ready);
      sync_rows();
      if (r == 0 && !sum) {
        if (!BWD && it > 0) {
          const int prow = tok0 + (n - 1) * C;
          tma_store_3d(&tmO, ob, tx, prow, 0);
          tma_store_3d(&tmO, ob + 8192, tx + 64, prow, 0);
        }
        tma_store_3d(&tmXB, xb, 0, g * D, 0);
        tma_store_3d(&tmXB, xb + 16384, 64, g * D, 0);
        tma_store_commit();
      }
      if (!mbar_wait_spin(y_done, cph, p.status)) { ok = false; break; }
      tc_fence_after();
      if (r < C) {
        const uint8_t* uh = smem + (it & 1) * S::STAGE + TILE_DO;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(lane_addr + COL_Y + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = __uint_as_float(v[8 * i + j]);
            const int col = c + 8 * i;
            if (!BWD && !lin) {
              float uhv[8];
              unpack8(*reinterpret_cast<const bf16x8*>(uh + (col >> 6) * 8192 + r * 128 +
                                                       ((((col & 63) >> 3) ^ (r & 7)) << 4)),
                      uhv);
#pragma unroll
              for (int j = 0; j < 8; ++j) y[j] = uhv[j] - y[j];  // U = U^ - W S
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) y[j] = -y[j];          // operand (and output) is -dU
            }
            bf16x8 pk;
#pragma unroll
            for (int j = 0; j < 4; ++j) pk.v[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
            st_swz(ub + (col >> 6) * 8192, r, (col & 63) >> 3, pk);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(u_ready);
      sync_rows();
      if (r == 0 && !sum) {
        tma_store_3d(&tmU, ub, 0, g * C, 0);
        tma_store_3d(&tmU, ub + 8192, 64, g * C, 0);
        tma_store_commit();
      }
    }
    // drain: last chunk's output rows and the final state
    if (ok && N > 0) {
      if (mbar_wait_spin(o_done, (N - 1) & 1, p.status)) {
        tc_fence_after();
        if (r == 0) tma_store_wait_read<0>();
        sync_rows();
        stage_out();
        fence_proxy_async_smem();
        sync_rows();
        if (r == 0 && !BWD && !sum) {
          const int prow = tok0 + (n0 + N - 1) * C;
          tma_store_3d(&tmO, ob, tx, prow, 0);
          tma_store_3d(&tmO, ob + 8192, tx + 64, prow, 0);
          tma_store_commit();
        }
        float* fin = lin ? p.p_final : p.x_final;
        if (fin != nullptr) {
          float* xf = fin + (static_cast<size_t>(unit) * D + r) * D;
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(lane_addr + COL_X + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(xf + c)[i] =
                  make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                              __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
          }
        }
      }
    }
    if (r == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <bool BWD>
int launch(const void* W, const void* Q, const void* K, const void* M, const void* fifth,
           void* xb_out, void* u_out, void* o_out, int ld, const Params& p, cudaStream_t st) {
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<BWD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Smem<BWD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  const uint64_t G = static_cast<uint64_t>(p.n_seq) * p.n_chunks;
  const uint64_t rows = G * C;
  CUtensorMap tW, tQ, tK, tM, tD, tXB, tU, tO;
  int r = 0;
  // token-major tensors: [batch * seq_len, ld]; per-chunk tensors: [G * 64, 128]
  const bool tokmaj = p.heads > 0;
  const uint64_t t_inner = tokmaj ? static_cast<uint64_t>(p.heads) * D : D;
  const uint64_t t_ld = tokmaj ? static_cast<uint64_t>(ld) : D;
  r |= make_tmap_3d(&tW, W, 2, D, rows, 1, D, 0, 64, C);
  r |= make_tmap_3d(&tQ, Q, 2, t_inner, rows * D / t_inner, 1, t_ld, 0, 64, C);
  r |= make_tmap_3d(&tK, K, 2, t_inner, rows * D / t_inner, 1, t_ld, 0, 64, C);
  r |= make_tmap_3d(&tM, M, 2, C, rows, 1, C, 0, 64, C);
  if (BWD) r |= make_tmap_3d(&tD, fifth, 2, t_inner, rows * D / t_inner, 1, t_ld, 0, 64, C);
  else r |= make_tmap_3d(&tD, fifth, 2, D, rows, 1, D, 0, 64, C);
  r |= make_tmap_3d(&tXB, xb_out, 2, D, G * D, 1, D, 0, 64, D);
  r |= make_tmap_3d(&tU, u_out, 2, D, rows, 1, D, 0, 64, C);
  if (BWD) r |= make_tmap_3d(&tO, u_out, 2, D, rows, 1, D, 0, 64, C);
  else r |= make_tmap_3d(&tO, o_out, 2, t_inner, rows * D / t_inner, 1, t_ld, 0, 64, C);
  if (r != 0) return 1000 + r;
  const int ctas = p.n_seq * p.n_seg * ((p.summary && !BWD) ? 2 : 1);
  delta_scan_kernel<BWD><<<ctas, 192, Smem<BWD>::TOTAL, st>>>(tW, tQ, tK, tM, tD, tXB, tU, tO, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dscan
}  // namespace pb

using namespace pb;

// Forward walk. All per-chunk tensors are row-major [(n_seq * n_chunks * 64), 128]
// bf16 (M: [.., 64]), chunk g = seq * n_chunks + n occupying rows [64 g, 64 g + 64).
// With heads > 0, Q, K and out (and dO in the backward walk) are instead token-major
// [batch * n_chunks * 64, ld] with head h = seq % heads at columns [128 h, 128 h + 128).
//   out   <- O            u_out <- U            xb_out[g] <- bf16(S entering chunk g)
//   x_init / x_final: fp32 [n_seq, 128, 128] (x_init may be null = zero state)
static int scan_args_ok(int n_seq, int n_chunks, int heads, int ld, int n_seg) {
  if (n_seq <= 0 || n_chunks <= 0 || heads < 0 || n_seg <= 0 || n_chunks % n_seg != 0) return 0;
  if (heads > 0 && (n_seq % heads != 0 || ld < heads * dscan::D || ld % 8 != 0)) return 0;
  return 1;
}
static dscan::Params scan_params(int n_seq, int n_chunks, int heads, int n_seg, int summary,
                                 const void* x_init, void* x_final, void* p_final, int* status) {
  dscan::Params p;
  p.n_chunks = n_chunks; p.n_seq = n_seq; p.n_seg = n_seg; p.summary = summary;
  p.heads = heads; p.seq_len = n_chunks * dscan::C;
  p.x_init = static_cast<const float*>(x_init);
  p.x_final = static_cast<float*>(x_final);
  p.p_final = static_cast<float*>(p_final);
  p.status = status;
  return p;
}

PB_API int pb_delta_scan_fwd(const void* W, const void* Uhat, const void* Q, const void* K,
                             const void* M, void* out, void* u_out, void* xb_out,
                             const void* x_init, void* x_final, int n_seq, int n_chunks,
                             int heads, int ld, int* status, cudaStream_t st) {
  if (!scan_args_ok(n_seq, n_chunks, heads, ld, 1)) return PB_BAD_ARG;
  return dscan::launch<false>(W, Q, K, M, Uhat, xb_out, u_out, out, ld,
                              scan_params(n_seq, n_chunks, heads, 1, 0, x_init, x_final, nullptr, status), st);
}

// The same walk with every sequence cut into n_seg segments of n_chunks / n_seg chunks, one CTA
// per segment. x_init / x_final: fp32 [n_seq * n_seg, 128, 128], the state entering / leaving
// each segment (x_init comes from pb_delta_scan_summary_fwd + pb_delta_compose).
PB_API int pb_delta_scan_fwd_seg(const void* W, const void* Uhat, const void* Q, const void* K,
                                 const void* M, void* out, void* u_out, void* xb_out,
                                 const void* x_init, void* x_final, int n_seq, int n_chunks,
                                 int n_seg, int heads, int ld, int* status, cudaStream_t st) {
  if (!scan_args_ok(n_seq, n_chunks, heads, ld, n_seg) || x_init == nullptr) return PB_BAD_ARG;
  return dscan::launch<false>(W, Q, K, M, Uhat, xb_out, u_out, out, ld,
                              scan_params(n_seq, n_chunks, heads, n_seg, 0, x_init, x_final, nullptr, status), st);
}

// Affine map of every segment, S_out = P S_in + R, without outputs: r_out, p_out fp32
// [n_seq * n_seg, 128, 128]. Two CTAs per segment (one per map), three products per chunk
// instead of six, no stores but the two maps.
PB_API int pb_delta_scan_summary_fwd(const void* W, const void* Uhat, const void* K, void* r_out,
                                     void* p_out, int n_seq, int n_chunks, int n_seg, int heads,
                                     int ld, int* status, cudaStream_t st) {
  if (!scan_args_ok(n_seq, n_chunks, heads, ld, n_seg) || r_out == nullptr || p_out == nullptr)
    return PB_BAD_ARG;
  // Q, M and the output maps are never touched in this mode; W stands in so that the tensor
  // maps are valid objects.
  return dscan::launch<false>(W, K, K, W, Uhat, const_cast<void*>(W), const_cast<void*>(W),
                              const_cast<void*>(K), ld,
                              scan_params(n_seq, n_chunks, heads, n_seg, 1, nullptr, r_out, p_out, status), st);
}

// Backward walk (chunks in reverse). x_init = gradient of the final state (or null),
//   ndu_out <- -dU (note the sign)
//   dxb_out[g] <- bf16(dS leaving chunk g, i.e. before chunk g is applied)
//   x_final <- gradient of the initial state
PB_API int pb_delta_scan_bwd(const void* W, const void* Q, const void* K, const void* M,
                             const void* dO, void* ndu_out, void* dxb_out, const void* x_init,
                             void* x_final, int n_seq, int n_chunks, int heads, int ld,
                             int* status, cudaStream_t st) {
  if (!scan_args_ok(n_seq, n_chunks, heads, ld, 1)) return PB_BAD_ARG;
  return dscan::launch<true>(W, Q, K, M, dO, dxb_out, ndu_out, nullptr, ld,
                             scan_params(n_seq, n_chunks, heads, 1, 0, x_init, x_final, nullptr, status), st);
}

// Segmented backward walk: x_init = gradient of the state leaving each segment, x_final =
// gradient of the state entering it, both fp32 [n_seq * n_seg, 128, 128].
PB_API int pb_delta_scan_bwd_seg(const void* W, const void* Q, const void* K, const void* M,
                                 const void* dO, void* ndu_out, void* dxb_out, const void* x_init,
                                 void* x_final, int n_seq, int n_chunks, int n_seg, int heads,
                                 int ld, int* status, cudaStream_t st) {
  if (!scan_args_ok(n_seq, n_chunks, heads, ld, n_seg) || x_init == nullptr) return PB_BAD_ARG;
  return dscan::launch<true>(W, Q, K, M, dO, dxb_out, ndu_out, nullptr, ld,
                             scan_params(n_seq, n_chunks, heads, n_seg, 0, x_init, x_final, nullptr, status), st);
}

// What each segment's backward walk adds to the state gradient when it starts from zero
// (g_out fp32 [n_seq * n_seg, 128, 128]); the linear part is the transpose of the forward P.
PB_API int pb_delta_scan_summary_bwd(const void* W, const void* Q, const void* K, const void* M,
                                     const void* dO, void* g_out, int n_seq, int n_chunks,
                                     int n_seg, int heads, int ld, int* status, cudaStream_t st) {
  if (!scan_args_ok(n_seq, n_chunks, heads, ld, n_seg) || g_out == nullptr) return PB_BAD_ARG;
  return dscan::launch<true>(W, Q, K, M, dO, const_cast<void*>(W), const_cast<void*>(W), nullptr, ld,
                             scan_params(n_seq, n_chunks, heads, n_seg, 1, nullptr, g_out, nullptr, status), st);
}

// ---------------------------------------------------------------------------
// Sequential composition of the segments' affine maps (fp32 on the CUDA cores; 128^3 per step).
//   forward  S <- s0 (or 0); for j = 0 .. n_seg-1:  s_in[j] <- S;  S <- P_j S + R_j;   s_fin <- S
//            p_tot (optional) <- P_{n-1} ... P_0
//   reverse  G <- s0 (or 0); for j = n_seg-1 .. 0:  s_in[j] <- G;  G <- P_j^T G + R_j; s_fin <- G
// One CTA per (sequence, 16-column slab): columns of the state never mix.
// ---------------------------------------------------------------------------
namespace pb {
namespace dcomp {
constexpr int D = 128, SLAB = 16, LDP = D + 1;
constexpr int SMEM = (D * LDP + D * (SLAB + 1)) * 4;
// 256 threads: thread t owns row t / 2 and eight of the slab's sixteen columns. The whole P_j
// (64 KB) is staged in shared memory once per segment: one round of coalesced loads, then
// 128 x 8 fused multiply-adds per thread with no further global traffic.
__global__ void __launch_bounds__(256)
compose_kernel(const float* __restrict__ P, const float* __restrict__ R,
               const float* __restrict__ s0, float* __restrict__ s_in, float* __restrict__ s_fin,
               float* __restrict__ p_tot, int n_seg, int reverse, int slabs_state) {
  extern __shared__ float sm[];
  float (*pt)[LDP] = reinterpret_cast<float (*)[LDP]>(sm);                  // pt[r][k]
  float (*cur)[SLAB + 1] = reinterpret_cast<float (*)[SLAB + 1]>(sm + D * LDP);
  const int seq = blockIdx.y;
  const bool on_p = static_cast<int>(blockIdx.x) >= slabs_state;    // this CTA folds P itself
  const int col0 = (on_p ? blockIdx.x - slabs_state : blockIdx.x) * SLAB;
  const int r = threadIdx.x >> 1, c0 = (threadIdx.x & 1) * 8;
  const size_t mat = static_cast<size_t>(D) * D;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float v = 0.f;
    if (on_p) v = (r == col0 + c0 + c) ? 1.f : 0.f;
    else if (s0 != nullptr) v = s0[seq * mat + r * D + col0 + c0 + c];
    cur[r][c0 + c] = v;
  }
  for (int step = 0; step < n_seg; ++step) {
    const int j = reverse ? n_seg - 1 - step : step;
    const float* Pj = P + (static_cast<size_t>(seq) * n_seg + j) * mat;
    const float* Rj = R + (static_cast<size_t>(seq) * n_seg + j) * mat;
    // pt[r'][k] = P[r'][k] (forward) or P[k][r'] (reverse); global reads are row-contiguous
    for (int i = threadIdx.x; i < D * D / 4; i += 256) {
      const float4 v = reinterpret_cast<const float4*>(Pj)[i];
      const int a = (i * 4) / D, b = (i * 4) % D;
      if (!reverse) { pt[a][b] = v.x; pt[a][b + 1] = v.y; pt[a][b + 2] = v.z; pt[a][b + 3] = v.w; }
      else { pt[b][a] = v.x; pt[b + 1][a] = v.y; pt[b + 2][a] = v.z; pt[b + 3][a] = v.w; }
    }
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = on_p ? 0.f : Rj[r * D + col0 + c0 + c];
    __syncthreads();                       // pt and cur (previous step / initial) are in place
    if (!on_p && s_in != nullptr) {
      float* o = s_in + (static_cast<size_t>(seq) * n_seg + j) * mat + r * D + col0 + c0;
#pragma unroll
      for (int c = 0; c < 8; ++c) o[c] = cur[r][c0 + c];
    }
#pragma unroll 8
    for (int k = 0; k < D; ++k) {
      const float pv = pt[r][k];
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = fmaf(pv, cur[k][c0 + c], acc[c]);
    }
    __syncthreads();                       // every thread has finished reading cur and pt
#pragma unroll
    for (int c = 0; c < 8; ++c) cur[r][c0 + c] = acc[c];
  }
  __syncthreads();
  float* fin = on_p ? p_tot : s_fin;
  if (fin != nullptr) {
    float* o = fin + seq * mat + r * D + col0 + c0;
#pragma unroll
    for (int c = 0; c < 8; ++c) o[c] = cur[r][c0 + c];
  }
}
}  // namespace dcomp
}  // namespace pb

PB_API int pb_delta_compose(const void* P, const void* R, const void* s0, void* s_in, void* s_fin,
                            void* p_tot, int n_seq, int n_seg, int reverse, cudaStream_t st) {
  if (n_seq <= 0 || n_seg <= 0 || P == nullptr || R == nullptr) return PB_BAD_ARG;
  if (p_tot != nullptr && reverse) return PB_BAD_ARG;
  const int slabs = pb::dcomp::D / pb::dcomp::SLAB;
  dim3 grid(p_tot != nullptr ? 2 * slabs : slabs, n_seq);
  static pb::DeviceOnce attr_once;
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(pb::dcomp::compose_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, pb::dcomp::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  pb::dcomp::compose_kernel<<<grid, 256, pb::dcomp::SMEM, st>>>(
      static_cast<const float*>(P), static_cast<const float*>(R), static_cast<const float*>(s0),
      static_cast<float*>(s_in), static_cast<float*>(s_fin), static_cast<float*>(p_tot), n_seg,
      reverse, slabs);
  return static_cast<int>(cudaGetLastError());
}
