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
    ok = mbar_wait(mma1, ph, p.status) && ok;
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
    ok = mbar_wait(mma2, ph, p.status);
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(delta_prep_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set = true;
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
