// Causal softmax attention with grouped KV heads on tcgen05 (sm_100a), head dim 128.
//
// Forward (flash-style, one CTA per 128 query rows of one head):
//   S = Q K_j^T  (tensor memory, double-buffered)      P = exp2(S c - m)   (registers, one
//   O += P V_j   (tensor memory)                                             query row per thread)
// The running maximum is only raised when it would grow by more than 2^8 (the rescale of O is a
// tensor-memory read-modify-write, so it is skipped while the stale maximum is safe); the final
// O / l and the log-sum-exp use the maximum actually applied, which keeps the result exact.
//
// Backward, two kernels sharing one skeleton (no atomics, deterministic):
//   dQ  : CTA = 128 query rows; streams 64-key tiles   S = Q K^T, dP = dO V^T, dS = P (dP - delta) c
//         dQ += dS K
//   dKV : CTA = 128 key rows of one KV head; streams 64-query tiles of every query head of the
//         group  S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q
// Every streamed tile is used twice from the same shared-memory image: as the K-major B operand
// of the score product and as the MN-major B operand of the gradient product.
//
// warps 0-3: one tensor-memory lane (= row) per thread; warp 4: MMA issue; warp 5: TMA producer.
// All tensors are token-major: Q/O/dO/dQ [batch * seq, ldq] with head h at columns 128 h,
// K/V/dK/dV [batch * seq, ldkv] with KV head g at columns 128 g. seq must be a multiple of 256 (forward) / 128 (backward).
//
// Reference semantics: model/__init__.py gqa/mla attention (softmax(q k^T / sqrt(d)) v with a
// causal mask) of the reference; the tiling is this library's own.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"

namespace pb {

int make_tmap_3d(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t batch, uint64_t ld_elems, uint64_t batch_stride_elems,
                 uint32_t box_inner, uint32_t box_outer);

namespace attn {

constexpr int D = 128;
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units

// Optional cycle accounting of the forward row warps (compile with -DPB_ATTN_PROF): thread 0 of
// each warpgroup adds the clocks it spent in each phase of a block to a device array.
#ifdef PB_ATTN_PROF
__device__ unsigned long long g_attn_prof[8];
#define PB_PROF_START long long prof_t = clock64();
#define PB_PROF(i)                                                                  \
  if (r == 0) {                                                                     \
    const long long prof_n = clock64();                                             \
    atomicAdd(&g_attn_prof[i], static_cast<unsigned long long>(prof_n - prof_t));  \
    prof_t = prof_n;                                                                \
  }
#else
#define PB_PROF_START
#define PB_PROF(i)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 16-byte store of 8 bf16 into a [rows][64] 128B-swizzled chunk (row pitch 128 bytes).
__device__ __forceinline__ void st_swz(uint8_t* chunk_base, int row, int c16, const bf16x8& v) {
  *reinterpret_cast<bf16x8*>(chunk_base + row * 128 + ((c16 ^ (row & 7)) << 4)) = v;
}
__device__ __forceinline__ bf16x8 pack_bf16x8(const float* f) {
  bf16x8 pk;
#pragma unroll
  for (int j = 0; j < 4; ++j) pk.v[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return pk;
}
__device__ __forceinline__ void sync_rows() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Warp-uniform bounded wait: the row warps run warp-collective tensor-memory loads, so either
// every lane goes on or none does.
__device__ __forceinline__ bool wait_all(uint64_t* bar, uint32_t parity, int* status) {
  return __all_sync(0xffffffffu, mbar_wait_spin(bar, parity, status));
}

// ------------------------------------------------------------------------------ forward
namespace fwd {
// shared memory: Q (two 128-row tiles), three K/V stages of 64 keys, two P buffers per tile
constexpr int Q_OFF = 0, KV_OFF = 65536, KV_STAGES = 3, KV_STAGE = 32768;
constexpr int P_OFF = KV_OFF + KV_STAGES * KV_STAGE, BARS = P_OFF + 65536;
constexpr int SMEM = BARS + 512 + 1024;
constexpr uint32_t COL_S = 0, COL_O = 256, TMEM_COLS = 512;   // S[tile][buf] 64 cols, O[tile] 128

struct Params {
  int seq, heads, kv_heads;   // seq: query rows per batch entry
  int seq_kv, q_off;          // key rows per batch entry; global position of query row 0
  float scale_log2;   // softmax scale * log2(e)
  float* lse2;        // [batch, heads, seq], log2 domain
  float* rowmax;      // [batch, heads, seq] largest scaled logit of the row, or null
  int* status;
};

// One CTA = 256 query rows of one head: two 128-row tiles, each owned by one warpgroup
// (warps 0-3 and 4-7) so that one group's exponentials overlap the other's tensor-core work.
// Keys and values arrive in blocks of 64.  warps 8 and 9: MMA issue for tile 0 and tile 1 (a
// single issuing thread cannot keep up with 24 small MMAs per block), warp 10: TMA producer.
__global__ void __launch_bounds__(352, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BARS);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [4]
  uint64_t* kv_empty = bars + 5;   // [4]
  uint64_t* s_done = bars + 9;     // [tile][buf]
  uint64_t* s_free = bars + 13;    // [tile][buf]
  uint64_t* p_ready = bars + 17;   // [tile]
  uint64_t* o_done = bars + 19;    // [tile][buf]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 26);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cb = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.heads / p.kv_heads);
  const int gb = cb + p.q_off / 256;   // position of this CTA's rows among all keys
  const int row0 = b * p.seq + cb * 256;
  const int nj1 = 4 * gb + 4;     // 64-key blocks seen by tile 1; tile 0 sees nj1 - 2

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 2); }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&s_done[i], 1); mbar_init(&s_free[i], 4); mbar_init(&o_done[i], 1);
    }
    mbar_init(&p_ready[0], 4); mbar_init(&p_ready[1], 4);   // one arrival per warp
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 10) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 65536);
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(smem + Q_OFF + t * 32768, &tmQ, q_full, h * D, row0 + t * 128, 0);
        tma_load_3d(smem + Q_OFF + t * 32768 + 16384, &tmQ, q_full, h * D + 64, row0 + t * 128, 0);
      }
      for (int j = 0; j < nj1; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int krow = b * p.seq_kv + j * 64;
        if (!mbar_wait(&kv_empty[s], ph ^ 1, p.status)) break;
        mbar_arrive_expect_tx(&kv_full[s], KV_STAGE);
        uint8_t* st = smem + KV_OFF + s * KV_STAGE;
        tma_load_3d(st, &tmK, &kv_full[s], g * D, krow, 0);
        tma_load_3d(st + 8192, &tmK, &kv_full[s], g * D + 64, krow, 0);
        tma_load_3d(st + 16384, &tmV, &kv_full[s], g * D, krow, 0);
        tma_load_3d(st + 16384 + 8192, &tmV, &kv_full[s], g * D + 64, krow, 0);
      }
    }
  } else if (warp >= 8) {
    if (lane == 0) {
      const int t = warp - 8;                                     // the tile this thread issues for
      const int nj = nj1 - (t == 0 ? 2 : 0);
      const uint32_t id_s = make_idesc(1, 1, 128, 64, 0, 0);     // S = Q K^T, N = 64 keys
      const uint32_t id_o = make_idesc(1, 1, 128, 128, 0, 1);    // O += P V, V MN-major
      constexpr uint32_t HI = sdesc_hi_sw128(1024);
      // descriptor low words are kept in registers: one add per operand per MMA
      const uint32_t q_lo = sdesc_lo(smem_u32(smem + Q_OFF + t * 32768), 16);
      const uint32_t p_lo0 = sdesc_lo(smem_u32(smem + P_OFF + t * 32768), 16);
      const uint32_t kv0 = smem_u32(smem + KV_OFF);
      const uint32_t d_o = tmem + COL_O + t * 128;
      bool ok = mbar_wait_spin(q_full, 0, p.status);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES;
        const int sb = t * 2 + (j & 1);
        if (!mbar_wait_spin(&kv_full[s], (j / KV_STAGES) & 1, p.status)) return false;
        if (!mbar_wait_spin(&s_free[sb], ((j >> 1) & 1) ^ 1, p.status)) return false;
        tc_fence_after();
        const uint32_t k_lo = sdesc_lo(kv0 + s * KV_STAGE, 16);
        const uint32_t d = tmem + COL_S + sb * 64;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj)
          umma_f16_words(d, q_lo + (((jj >> 2) * 16384 + (jj & 3) * 32) >> 4), HI,
                         k_lo + (((jj >> 2) * 8192 + (jj & 3) * 32) >> 4), HI, id_s, jj > 0);
        umma_commit(&s_done[sb]);
        return true;
      };
      // the scores run two blocks ahead of the P V products, so neither the row warps nor
      // the P V issue ever wait for a K/V tile that is still in flight
      if (ok) ok = issue_s(0);
      if (ok && nj > 1) ok = issue_s(1);
      for (int j = 0; j < nj && ok; ++j) {
        const int s = j % KV_STAGES;
        if (!mbar_wait_spin(&p_ready[t], j & 1, p.status)) break;
        tc_fence_after();
        const uint32_t v_lo = sdesc_lo(kv0 + s * KV_STAGE + 16384, 8192);
        const uint32_t p_lo = p_lo0 + (((j & 1) * 16384) >> 4);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          umma_f16_words(d_o, p_lo + ((jj * 32) >> 4), HI, v_lo + ((jj * 2048) >> 4), HI, id_o,
                         (j > 0) || (jj > 0));
        umma_commit(&o_done[t * 2 + (j & 1)]);
        umma_commit(&kv_empty[s]);   // needs both tiles' commits (tile 0 skips the last two blocks,
                                     // whose stages are never refilled)
        if (j + 2 < nj && !issue_s(j + 2)) break;
      }
    }
  } else {
    const int t = warp >> 2;               // tile / warpgroup
    const int r = threadIdx.x & 127;       // query row of the tile = tensor-memory lane
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int qpos = gb * 256 + t * 128 + r;     // global position (for the causal mask)
    const int q0 = gb * 256 + t * 128;
    const int nj = nj1 - (t == 0 ? 2 : 0);
    auto sync_group = [&] {
      if (t == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
      else asm volatile("bar.sync 2, 128;" ::: "memory");
    };
    float m_used = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nj && ok; ++j) {
      const int sb = t * 2 + (j & 1);
      const uint32_t ph = (j >> 1) & 1;
      const bool edge = j * 64 + 63 > q0;
      PB_PROF_START
      if (!wait_all(&s_done[sb], ph, p.status)) { ok = false; break; }
      tc_fence_after();
      PB_PROF(0)
      uint32_t v[64];
      tmem_ld_32x32b_x32(lane_addr + COL_S + sb * 64, v);
      tmem_ld_32x32b_x32(lane_addr + COL_S + sb * 64 + 32, v + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);   // the scores are in registers now
      PB_PROF(1)
      if (edge) {   // only the blocks on the diagonal pay for the mask
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (j * 64 + i > qpos) v[i] = 0xff800000u;   // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      m_true = fmaxf(m_true, mx);
      PB_PROF(2)
      if (j == 0) {
        m_used = mx;
      } else if (__any_sync(0xffffffffu, mx > m_used + RESCALE_THRESHOLD)) {
        // raise the applied maximum: O of this tile must be idle (previous P V finished)
        if (!wait_all(&o_done[t * 2 + ((j - 1) & 1)], ((j - 1) >> 1) & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const float m_new = fmaxf(m_used, mx);
        const float alpha = ex2(m_used - m_new);
        l *= alpha;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(lane_addr + COL_O + t * 128 + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x32(lane_addr + COL_O + t * 128 + c, o);
        }
        tmem_st_wait();
        m_used = m_new;
      }
      PB_PROF(3)
      // P buffer j & 1 was last read by the P V product of block j - 2, which this thread's
      // issuer queued before S(j): the completed s_done wait above already covers it
      uint8_t* pbuf = smem + P_OFF + t * 32768 + (j & 1) * 16384;
      const float neg_m = -m_used;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // one fused multiply-add and one exponential per score; masked entries are -inf -> 0
          f[k] = ex2(fmaf(__uint_as_float(v[8 * i + k]), p.scale_log2, neg_m));
          l4[k & 3] += f[k];
        }
        st_swz(pbuf, r, i, pack_bf16x8(f));
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      PB_PROF(4)
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
      PB_PROF(5)
#ifdef PB_ATTN_PROF
      if (r == 0) atomicAdd(&g_attn_prof[6], 1ull);
#endif
    }
    if (ok && wait_all(&o_done[t * 2 + ((nj - 1) & 1)], ((nj - 1) >> 1) & 1, p.status)) {
      tc_fence_after();
      uint8_t* obuf = smem + P_OFF + t * 32768;   // both P buffers of the tile, now idle
      const float inv = 1.f / l;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(lane_addr + COL_O + t * 128 + c, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] = __uint_as_float(o[8 * i + k]) * inv;
          const int col = c + 8 * i;
          st_swz(obuf + (col >> 6) * 16384, r, (col & 63) >> 3, pack_bf16x8(f));
        }
      }
      const size_t vi = (static_cast<size_t>(b) * p.heads + h) * p.seq + cb * 256 + t * 128 + r;
      p.lse2[vi] = m_used + log2f(l);
      if (p.rowmax != nullptr) p.rowmax[vi] = m_true * 0.6931471805599453f;
      fence_proxy_async_smem();
      sync_group();
      if (r == 0) {
        tma_store_3d(&tmO, obuf, h * D, row0 + t * 128, 0);
        tma_store_3d(&tmO, obuf + 16384, h * D + 64, row0 + t * 128, 0);
        tma_store_commit();
        tma_store_wait<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies in flight land
    __syncthreads();
  }
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}
}  // namespace fwd

// ----------------------------------------------------------------------------- backward
namespace bwd {
constexpr int RA_OFF = 0, RB_OFF = 32768, ST_OFF = 65536;       // stages: T1 16 KB + T2 16 KB
constexpr int DS_OFF = ST_OFF + 2 * 32768, PT_OFF = DS_OFF + 2 * 16384;
constexpr int VEC_OFF = PT_OFF + 2 * 16384, BARS = VEC_OFF + 2 * 512;
constexpr int SMEM = BARS + 256 + 1024;
constexpr uint32_t COL_X1 = 0, COL_X2 = 128, COL_ACC1 = 256, COL_ACC2 = 384, TMEM_COLS = 512;

struct Params {
  int seq, heads, kv_heads, n_blk;  // seq: query rows per batch entry; n_blk: 128-row blocks of the grid
  int seq_kv, q_off;                // key rows per batch entry; global position of query row 0
  float scale_log2, scale;
  const float* lse2;    // [batch, heads, seq]
  const float* delta;   // [batch, heads, seq]  rowsum(dO * O)
  int* status;
};

// DKV = false: resident Q, dO (one head); streams K, V tiles; output dQ.
// DKV = true : resident K, V (one KV head); streams Q, dO tiles of the group; outputs dK, dV.
// Two warpgroups (warps 0-3, 4-7) take the streamed tiles alternately, each with its own score
// buffers in tensor memory and its own dS / P^T operand buffers, and accumulate into the same
// gradient accumulators.  MMA issue is spread over three warps because one thread cannot issue
// 20+ small MMAs per tile fast enough: warp 8 the first score product, warp 9 the second,
// warp 10 the gradient accumulations; warp 11: TMA producer.
template <bool DKV>
__global__ void __launch_bounds__(384, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmRA, const __grid_constant__ CUtensorMap tmRB,
                const __grid_constant__ CUtensorMap tmT1, const __grid_constant__ CUtensorMap tmT2,
                const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BARS);
  uint64_t* r_full = bars;
  uint64_t* t_full = bars + 1;    // [2]
  uint64_t* t_empty = bars + 3;   // [2]
  uint64_t* x_done = bars + 5;    // [2]
  uint64_t* x_free = bars + 7;    // [2]
  uint64_t* pd_ready = bars + 9;  // [2]
  uint64_t* pd_free = bars + 11;  // [2]
  uint64_t* acc_done = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.heads / p.kv_heads;
  const int b = blockIdx.z;
  // dQ: heavy blocks are the late query blocks; dKV: the early key blocks.
  const int blk = DKV ? static_cast<int>(blockIdx.x) : p.n_blk - 1 - static_cast<int>(blockIdx.x);
  const int hy = blockIdx.y;                       // query head (dQ) or KV head (dKV)
  const int g = DKV ? hy : hy / group;
  // dQ: blk is a local query block, streamed tiles are global key tiles 0 .. diagonal.
  // dKV: blk is a global key block, streamed tiles are the local query tiles at or after it.
  const int gblk = DKV ? blk : blk + p.q_off / 128;
  const int q_off64 = p.q_off / 64;
  const int t_first = DKV ? max(0, 2 * blk - q_off64) : 0;
  const int t_count = DKV ? max(0, p.seq / 64 - t_first) : 2 * gblk + 2;
  const int n_it = DKV ? group * t_count : t_count;
  const int row0 = b * (DKV ? p.seq_kv : p.seq) + blk * 128;
  const int t_seq = DKV ? p.seq : p.seq_kv;        // rows per batch entry of the streamed tensors

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], 1);
      mbar_init(&x_done[i], 2); mbar_init(&x_free[i], 4);    // two issuing threads; one arrival per row warp
      mbar_init(&pd_ready[i], 4); mbar_init(&pd_free[i], 1);
    }
    mbar_init(acc_done, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmRA); tma_prefetch_desc(&tmRB);
    tma_prefetch_desc(&tmT1); tma_prefetch_desc(&tmT2);
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 11) {
    if (lane == 0) {
      const int rx = (DKV ? g : hy) * D;
      // A key block that no local query sees streams nothing: its resident tiles are not
      // loaded either, because their buffers are the staging of the all-zero stores and no one
      // would wait for the loads to land first.
      if (n_it > 0) {
        mbar_arrive_expect_tx(r_full, 65536);
        tma_load_3d(smem + RA_OFF, &tmRA, r_full, rx, row0, 0);
        tma_load_3d(smem + RA_OFF + 16384, &tmRA, r_full, rx + 64, row0, 0);
        tma_load_3d(smem + RB_OFF, &tmRB, r_full, rx, row0, 0);
        tma_load_3d(smem + RB_OFF + 16384, &tmRB, r_full, rx + 64, row0, 0);
      }
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int t = t_first + (DKV ? it % t_count : it);
        const int tx = (DKV ? g * group + it / t_count : g) * D;
        const int trow = b * t_seq + t * 64;
        if (!mbar_wait(&t_empty[s], ph ^ 1, p.status)) break;
        mbar_arrive_expect_tx(&t_full[s], 32768);
        uint8_t* st = smem + ST_OFF + s * 32768;
        tma_load_3d(st, &tmT1, &t_full[s], tx, trow, 0);
        tma_load_3d(st + 8192, &tmT1, &t_full[s], tx + 64, trow, 0);
        tma_load_3d(st + 16384, &tmT2, &t_full[s], tx, trow, 0);
        tma_load_3d(st + 16384 + 8192, &tmT2, &t_full[s], tx + 64, trow, 0);
      }
    }
  } else if (warp == 8 || warp == 9) {
    // score products: warp 8 issues X1 = RA T1^T, warp 9 issues X2 = RB T2^T
    if (lane == 0) {
      const int which = warp - 8;
      const uint32_t id_x = make_idesc(1, 1, 128, 64, 0, 0);     // A K-major, B K-major, N = 64
      constexpr uint32_t HI = sdesc_hi_sw128(1024);
      const uint32_t r_lo = sdesc_lo(smem_u32(smem + (which == 0 ? RA_OFF : RB_OFF)), 16);
      const uint32_t st0 = smem_u32(smem + ST_OFF + which * 16384);
      const uint32_t col = which == 0 ? COL_X1 : COL_X2;
      bool ok = n_it == 0 || mbar_wait_spin(r_full, 0, p.status);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait_spin(&t_full[s], ph, p.status)) break;
        if (!mbar_wait_spin(&x_free[s], ph ^ 1, p.status)) break;
        tc_fence_after();
        const uint32_t t_lo = sdesc_lo(st0 + s * 32768, 16);
        const uint32_t d = tmem + col + s * 64;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj)
          umma_f16_words(d, r_lo + (((jj >> 2) * 16384 + (jj & 3) * 32) >> 4), HI,
                         t_lo + (((jj >> 2) * 8192 + (jj & 3) * 32) >> 4), HI, id_x, jj > 0);
        umma_commit(&x_done[s]);
      }
    }
  } else if (warp == 10) {
    // gradient accumulations, all from this one thread so that they stay ordered
    if (lane == 0) {
      const uint32_t id_acc = make_idesc(1, 1, 128, 128, 0, 1);  // A K-major, B MN-major
      constexpr uint32_t HI = sdesc_hi_sw128(1024);
      const uint32_t st0 = smem_u32(smem + ST_OFF);
      const uint32_t ds_lo0 = sdesc_lo(smem_u32(smem + DS_OFF), 16);
      const uint32_t pt_lo0 = sdesc_lo(smem_u32(smem + PT_OFF), 16);
      int it = 0;
      for (; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait_spin(&pd_ready[s], ph, p.status)) break;
        tc_fence_after();
        // the streamed tiles again, now as MN-major B operands (64-wide chunks 8 KB apart)
        const uint32_t t1_mn = sdesc_lo(st0 + s * 32768, 8192), t2_mn = t1_mn + (16384 >> 4);
        const uint32_t ds_lo = ds_lo0 + ((s * 16384) >> 4), pt_lo = pt_lo0 + ((s * 16384) >> 4);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          umma_f16_words(tmem + COL_ACC1, ds_lo + ((jj * 32) >> 4), HI, t1_mn + ((jj * 2048) >> 4),
                         HI, id_acc, (it > 0) || (jj > 0));
        if (DKV) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            umma_f16_words(tmem + COL_ACC2, pt_lo + ((jj * 32) >> 4), HI,
                           t2_mn + ((jj * 2048) >> 4), HI, id_acc, (it > 0) || (jj > 0));
        }
        // the score products of this tile finished before the row warps could signal pd_ready,
        // so the completion of these MMAs releases the whole stage
        umma_commit(&t_empty[s]);
        umma_commit(&pd_free[s]);
      }
      if (it == n_it) umma_commit(acc_done);
    }
  } else {
    const int wg = warp >> 2;          // warpgroup = score buffer = parity of its iterations
    const int r = threadIdx.x & 127;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    auto sync_group = [&] {
      if (wg == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
      else asm volatile("bar.sync 2, 128;" ::: "memory");
    };
    const int pos = gblk * 128 + r;   // global query position (dQ) or key position (dKV) of this row
    float row_lse = 0.f, row_delta = 0.f;
    if (!DKV) {
      const size_t vi = (static_cast<size_t>(b) * p.heads + hy) * p.seq + blk * 128 + r;
      row_lse = p.lse2[vi];
      row_delta = p.delta[vi];
    }
    // dKV: per-column log-sum-exp and delta of the streamed query tile, prefetched one
    // iteration ahead by threads 0..63 (lse) and 64..127 (delta).
    auto vec_src = [&](int it) -> const float* {
      const int t = t_first + it % t_count;
      const int h = g * group + it / t_count;
      const float* base = (r < 64) ? p.lse2 : p.delta;
      return base + (static_cast<size_t>(b) * p.heads + h) * p.seq + t * 64 + (r & 63);
    };
    float vec_next = (DKV && wg < n_it) ? *vec_src(wg) : 0.f;
    bool ok = true;
    for (int it = wg; it < n_it && ok; it += 2) {
      const int s = wg;
      const uint32_t ph = (it >> 1) & 1;
      const int t = t_first + (DKV ? it % t_count : it);
      float* vec = reinterpret_cast<float*>(smem + VEC_OFF + s * 512);
      if (DKV) {
        sync_group();        // the group's readers of the previous tile are done
        vec[r] = vec_next;   // [0,64) lse2, [64,128) delta
        if (it + 2 < n_it) vec_next = *vec_src(it + 2);
        sync_group();
      }
      if (!wait_all(&x_done[s], ph, p.status)) { ok = false; break; }
      if (!wait_all(&pd_free[s], ph ^ 1, p.status)) { ok = false; break; }
      tc_fence_after();
      // mask: dQ rows are queries, columns keys (key > query is masked);
      //       dKV rows are keys, columns queries (query < key is masked)
      const int tg = DKV ? t + q_off64 : t;     // global index of the streamed tile
      const bool edge = DKV ? (tg * 64 < gblk * 128 + 127) : (tg * 64 + 63 > gblk * 128);
      uint8_t* dsb = smem + DS_OFF + s * 16384;
      uint8_t* ptb = smem + PT_OFF + s * 16384;
      auto tile_rows = [&](auto EDGE) {
#pragma unroll 1
        for (int c = 0; c < 64; c += 32) {
          uint32_t x1[32], x2[32];
          tmem_ld_32x32b_x32(lane_addr + COL_X1 + s * 64 + c, x1);
          tmem_ld_32x32b_x32(lane_addr + COL_X2 + s * 64 + c, x2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float pf[8], df[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int col = c + 8 * i + k;
              const float lse = DKV ? vec[col] : row_lse;
              const float dl = DKV ? vec[64 + col] : row_delta;
              float pr = ex2(fmaf(__uint_as_float(x1[8 * i + k]), p.scale_log2, -lse));
              if (decltype(EDGE)::value) {
                const int other = tg * 64 + col;
                const bool masked = DKV ? (other < pos) : (other > pos);
                if (masked) pr = 0.f;
              }
              pf[k] = pr;
              df[k] = pr * ((__uint_as_float(x2[8 * i + k]) - dl) * p.scale);
            }
            const int c16 = (c >> 3) + i;
            st_swz(dsb, r, c16, pack_bf16x8(df));
            if (DKV) st_swz(ptb, r, c16, pack_bf16x8(pf));
          }
        }
      };
      if (edge) tile_rows(std::true_type{});
      else tile_rows(std::false_type{});
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&x_free[s]);
        mbar_arrive(&pd_ready[s]);
      }
    }
    // every row thread gets here (no early exit above), so the group barriers below are safe
    if (wait_all(acc_done, 0, p.status) && ok) {
      tc_fence_after();
      // resident tiles are no longer read: reuse them as the staging for the TMA stores.
      // dKV: group 0 drains dK, group 1 drains dV.  dQ: each group drains 64 columns.
      uint8_t* stage = smem + ((DKV && wg == 1) ? RB_OFF : RA_OFF);
      const uint32_t col0 = (DKV && wg == 1) ? COL_ACC2 : COL_ACC1;
      const int c_lo = DKV ? 0 : wg * 64, c_hi = DKV ? D : wg * 64 + 64;
#pragma unroll 1
      for (int c = c_lo; c < c_hi; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(lane_addr + col0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float f[8];
#pragma unroll
          // a key block with no local query at or after it gets an all-zero gradient
          for (int k = 0; k < 8; ++k) f[k] = n_it > 0 ? __uint_as_float(v[8 * i + k]) : 0.f;
          const int col = c + 8 * i;
          st_swz(stage + (col >> 6) * 16384, r, (col & 63) >> 3, pack_bf16x8(f));
        }
      }
      fence_proxy_async_smem();
      sync_group();
      if (r == 0) {
        const int ox = (DKV ? g : hy) * D;
        if (DKV) {
          const CUtensorMap* tm = wg == 0 ? &tmO1 : &tmO2;
          tma_store_3d(tm, stage, ox, row0, 0);
          tma_store_3d(tm, stage + 16384, ox + 64, row0, 0);
        } else {
          tma_store_3d(&tmO1, stage + wg * 16384, ox + wg * 64, row0, 0);
        }
        tma_store_commit();
        tma_store_wait<0>();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != PB_OK) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// delta[b, h, s] = sum_d dO * O  (one warp per row)
__global__ void attn_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout,
                                  float* __restrict__ delta, int rows, int seq, int heads, int ldo,
                                  int lddo) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= rows * heads) return;
  const int tok = w / heads, h = w % heads;
  const bf16* po = o + static_cast<size_t>(tok) * ldo + h * D + lane * 4;
  const bf16* pd = dout + static_cast<size_t>(tok) * lddo + h * D + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(po), d = *reinterpret_cast<const uint2*>(pd);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&d);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(a2[i]), y = __bfloat1622float2(d2[i]);
    acc += x.x * y.x + x.y * y.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const int bb = tok / seq, s = tok % seq;
    delta[(static_cast<size_t>(bb) * heads + h) * seq + s] = acc;
  }
}
}  // namespace bwd

static bool bad_geometry(int batch, int seq, int heads, int kv_heads, int ldq, int ldkv) {
  return batch <= 0 || seq <= 0 || seq % 128 != 0 || heads <= 0 || kv_heads <= 0 ||
         heads % kv_heads != 0 || ldq < heads * D || ldkv < kv_heads * D || ldq % 8 != 0 ||
         ldkv % 8 != 0;
}

}  // namespace attn
}  // namespace pb

using namespace pb;

// out = softmax(scale * Q K^T + causal mask) V.  q/out: [batch * seq, ldq / ldo] bf16 with head h
// at columns [128 h, 128 h + 128); k/v: [batch * seq_kv, ldkv] with KV head g likewise.
// Query row i of a batch entry sits at global position q_off + i and sees keys 0 .. q_off + i
// (q_off = 0 and seq_kv = seq is ordinary causal attention; a context-parallel rank passes its
// slice of the queries, the gathered keys and its offset). seq, q_off multiples of 256;
// seq_kv >= q_off + seq, a multiple of 128.
// lse2: fp32 [batch, heads, seq], log2 of the softmax denominator plus the applied maximum.
// rowmax (optional): fp32 [batch, heads, seq], the largest scaled logit of each row.
PB_API int pb_attn_fwd_cp(const void* q, const void* k, const void* v, void* out, void* lse2,
                          void* rowmax, int batch, int seq, int seq_kv, int q_off, int heads,
                          int kv_heads, int ldq, int ldkv, int ldo, float scale, int* status,
                          cudaStream_t st) {
  using namespace attn;
  if (bad_geometry(batch, seq, heads, kv_heads, ldq, ldkv) || ldo < heads * D || ldo % 8 != 0 ||
      seq % 256 != 0 || !(scale > 0.f) || q_off < 0 || q_off % 256 != 0 || seq_kv % 128 != 0 ||
      seq_kv < q_off + seq)
    return PB_BAD_ARG;
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(fwd::attn_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, fwd::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  const uint64_t rows = static_cast<uint64_t>(batch) * seq, krows = static_cast<uint64_t>(batch) * seq_kv;
  CUtensorMap tQ, tK, tV, tO;
  int r = 0;
  r |= make_tmap_3d(&tQ, q, 2, static_cast<uint64_t>(heads) * D, rows, 1, ldq, 0, 64, 128);
  r |= make_tmap_3d(&tK, k, 2, static_cast<uint64_t>(kv_heads) * D, krows, 1, ldkv, 0, 64, 64);
  r |= make_tmap_3d(&tV, v, 2, static_cast<uint64_t>(kv_heads) * D, krows, 1, ldkv, 0, 64, 64);
  r |= make_tmap_3d(&tO, out, 2, static_cast<uint64_t>(heads) * D, rows, 1, ldo, 0, 64, 128);
  if (r != 0) return 1000 + r;
  fwd::Params p;
  p.seq = seq; p.heads = heads; p.kv_heads = kv_heads;
  p.seq_kv = seq_kv; p.q_off = q_off;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = static_cast<float*>(lse2);
  p.rowmax = static_cast<float*>(rowmax);
  p.status = status;
  fwd::attn_fwd_kernel<<<dim3(seq / 256, heads, batch), 352, fwd::SMEM, st>>>(tQ, tK, tV, tO, p);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_attn_fwd(const void* q, const void* k, const void* v, void* out, void* lse2,
                       void* rowmax, int batch, int seq, int heads, int kv_heads, int ldq, int ldkv,
                       int ldo, float scale, int* status, cudaStream_t st) {
  return pb_attn_fwd_cp(q, k, v, out, lse2, rowmax, batch, seq, seq, 0, heads, kv_heads, ldq, ldkv,
                        ldo, scale, status, st);
}

// Gradients of pb_attn_fwd_cp. delta: fp32 scratch [batch, heads, seq] (written here).
// dq: [batch * seq, ldq]; dk, dv: [batch * seq_kv, ldkv] (all bf16, fully overwritten; key rows
// that no local query sees get zeros).
PB_API int pb_attn_bwd_cp(const void* q, const void* k, const void* v, const void* out,
                          const void* dout, const void* lse2, void* delta, void* dq, void* dk,
                          void* dv, int batch, int seq, int seq_kv, int q_off, int heads,
                          int kv_heads, int ldq, int ldkv, int ldo, float scale, int* status,
                          cudaStream_t st) {
  using namespace attn;
  if (bad_geometry(batch, seq, heads, kv_heads, ldq, ldkv) || ldo < heads * D || ldo % 8 != 0 ||
      !(scale > 0.f) || q_off < 0 || q_off % 128 != 0 || seq_kv % 128 != 0 || seq_kv < q_off + seq)
    return PB_BAD_ARG;
  static pb::DeviceOnce attr_once;   // per device: the attribute belongs to the current GPU
  if (attr_once.need()) {
    cudaError_t e = cudaFuncSetAttribute(bwd::attn_bwd_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bwd::SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(bwd::attn_bwd_kernel<true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, bwd::SMEM);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_once.done();
  }
  const uint64_t rows = static_cast<uint64_t>(batch) * seq, krows = static_cast<uint64_t>(batch) * seq_kv;
  const uint64_t qi = static_cast<uint64_t>(heads) * D, ki = static_cast<uint64_t>(kv_heads) * D;
  {
    const long long warps = static_cast<long long>(rows) * heads;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    bwd::attn_delta_kernel<<<blocks, 256, 0, st>>>(
        static_cast<const bf16*>(out), static_cast<const bf16*>(dout), static_cast<float*>(delta),
        static_cast<int>(rows), seq, heads, ldo, ldo);
  }
  bwd::Params p;
  p.seq = seq; p.heads = heads; p.kv_heads = kv_heads;
  p.seq_kv = seq_kv; p.q_off = q_off;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse2 = static_cast<const float*>(lse2);
  p.delta = static_cast<const float*>(delta);
  p.status = status;
  int r = 0;
  {
    // dQ: resident Q, dO (128-row boxes); streamed K, V (64-row boxes)
    CUtensorMap tQ, tDO, tK, tV, tDQ;
    r |= make_tmap_3d(&tQ, q, 2, qi, rows, 1, ldq, 0, 64, 128);
    r |= make_tmap_3d(&tDO, dout, 2, qi, rows, 1, ldo, 0, 64, 128);
    r |= make_tmap_3d(&tK, k, 2, ki, krows, 1, ldkv, 0, 64, 64);
    r |= make_tmap_3d(&tV, v, 2, ki, krows, 1, ldkv, 0, 64, 64);
    r |= make_tmap_3d(&tDQ, dq, 2, qi, rows, 1, ldq, 0, 64, 128);
    if (r != 0) return 1000 + r;
    p.n_blk = seq / 128;
    bwd::attn_bwd_kernel<false><<<dim3(p.n_blk, heads, batch), 384, bwd::SMEM, st>>>(
        tQ, tDO, tK, tV, tDQ, tDQ, p);
  }
  {
    // dK, dV: resident K, V (every key block of the gathered keys); streamed local Q, dO
    CUtensorMap tK, tV, tQ, tDO, tDK, tDV;
    r |= make_tmap_3d(&tK, k, 2, ki, krows, 1, ldkv, 0, 64, 128);
    r |= make_tmap_3d(&tV, v, 2, ki, krows, 1, ldkv, 0, 64, 128);
    r |= make_tmap_3d(&tQ, q, 2, qi, rows, 1, ldq, 0, 64, 64);
    r |= make_tmap_3d(&tDO, dout, 2, qi, rows, 1, ldo, 0, 64, 64);
    r |= make_tmap_3d(&tDK, dk, 2, ki, krows, 1, ldkv, 0, 64, 128);
    r |= make_tmap_3d(&tDV, dv, 2, ki, krows, 1, ldkv, 0, 64, 128);
    if (r != 0) return 2000 + r;
    p.n_blk = seq_kv / 128;
    bwd::attn_bwd_kernel<true><<<dim3(p.n_blk, kv_heads, batch), 384, bwd::SMEM, st>>>(
        tK, tV, tQ, tDO, tDK, tDV, p);
  }
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_attn_bwd(const void* q, const void* k, const void* v, const void* out,
                       const void* dout, const void* lse2, void* delta, void* dq, void* dk,
                       void* dv, int batch, int seq, int heads, int kv_heads, int ldq, int ldkv,
                       int ldo, float scale, int* status, cudaStream_t st) {
  return pb_attn_bwd_cp(q, k, v, out, dout, lse2, delta, dq, dk, dv, batch, seq, seq, 0, heads,
                        kv_heads, ldq, ldkv, ldo, scale, status, st);
}

#ifdef PB_ATTN_PROF
PB_API int pb_attn_prof_read(unsigned long long* out8, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out8, attn::g_attn_prof, sizeof(unsigned long long) * 8);
  if (e == cudaSuccess && reset) {
    unsigned long long z[8] = {};
    e = cudaMemcpyToSymbol(attn::g_attn_prof, z, sizeof z);
  }
  return static_cast<int>(e);
}
#endif
