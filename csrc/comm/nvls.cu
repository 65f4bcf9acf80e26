// NVLS (NVLink SHARP) multicast memory and the kernels that use it: the in-switch variants of
// the broadcast and reduce paths, next to the peer-to-peer ones of symm.cu.
//
// A multicast object spans one physical allocation per GPU of the group. Through its multicast
// address, one `multimem.st` is replicated by the NVSwitch into every GPU's allocation (a
// broadcast that costs the sender one store instead of one per peer) and one
// `multimem.ld_reduce` returns the sum over every GPU's copy, reduced inside the switch.
//
//   pb_nvls_supported        does this device (and driver) offer multicast objects
//   pb_nvls_create / import  rank 0 creates the object and exports a POSIX file descriptor;
//                            the other ranks import the descriptor they were passed
//   pb_nvls_add_device       every rank adds its device (all must, before any bind)
//   pb_nvls_bind_map         allocate this GPU's physical memory, map it (unicast address),
//                            bind it to the object, map the object (multicast address)
//   pb_nvls_free             unmap, unbind, release
//   pb_mm_muon_apply / pb_mm_adamw   optimizer update fused with the parameter broadcast:
//                            one multimem.st per 16 bytes lands in every rank's bf16 copy
//   pb_mm_allreduce_f32      two-shot all-reduce: this rank's slice is reduced by
//                            multimem.ld_reduce and the sum is written back to every rank by
//                            multimem.st (order of the additions is the switch's: the fast,
//                            order-free variant; pb_reduce_to_owner is the rank-ordered one)
//
// Availability is a run-time fact (driver, fabric permissions): every entry point returns an
// error code instead of aborting and the callers fall back to the peer-to-peer kernels.
// No TMA and no cluster multicast is involved anywhere in this file.
// Reference: the reference only plans in-switch collectives (spec/05-training-system.md:11-16).
#include <cuda.h>
#include <unistd.h>

#include "common.cuh"

namespace pb {
namespace nvls {

struct Api {
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  CUresult (*CtxGetDevice)(CUdevice*);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                               size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                      CUmulticastGranularity_flags);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                        unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                         CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                           CUmemAllocationHandleType);
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                          CUmemAllocationGranularity_flags);
  bool ok;
};

static bool load_one(const char* name, void** out) {
  cudaDriverEntryPointQueryResult q;
  void* ptr = nullptr;
  if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || ptr == nullptr)
    return false;
  *out = ptr;
  return true;
}

static const Api* api() {
  static Api a;
  static int state = 0;   // 0 not tried, 1 ok, 2 missing
  if (state == 0) {
    bool ok = true;
#define PB_LOAD(field, sym) ok = load_one(sym, reinterpret_cast<void**>(&a.field)) && ok
    PB_LOAD(DeviceGetAttribute, "cuDeviceGetAttribute");
    PB_LOAD(CtxGetDevice, "cuCtxGetDevice");
    PB_LOAD(MulticastCreate, "cuMulticastCreate");
    PB_LOAD(MulticastAddDevice, "cuMulticastAddDevice");
    PB_LOAD(MulticastBindMem, "cuMulticastBindMem");
    PB_LOAD(MulticastUnbind, "cuMulticastUnbind");
    PB_LOAD(MulticastGetGranularity, "cuMulticastGetGranularity");
    PB_LOAD(MemCreate, "cuMemCreate");
    PB_LOAD(MemRelease, "cuMemRelease");
    PB_LOAD(MemAddressReserve, "cuMemAddressReserve");
    PB_LOAD(MemAddressFree, "cuMemAddressFree");
    PB_LOAD(MemMap, "cuMemMap");
    PB_LOAD(MemUnmap, "cuMemUnmap");
    PB_LOAD(MemSetAccess, "cuMemSetAccess");
    PB_LOAD(MemExportToShareableHandle, "cuMemExportToShareableHandle");
    PB_LOAD(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    PB_LOAD(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
#undef PB_LOAD
    a.ok = ok;
    state = ok ? 1 : 2;
  }
  return state == 1 ? &a : nullptr;
}

// One multicast-backed allocation of this rank.
struct Buffer {
  CUmemGenericAllocationHandle mc = 0, mem = 0;
  CUdeviceptr uc_ptr = 0, mc_ptr = 0;
  size_t size = 0;
  CUdevice dev = 0;
  int world = 0;
  bool bound = false, uc_mapped = false, mc_mapped = false, have_mc = false, have_mem = false;
};

static CUmulticastObjectProp mc_prop(int world, size_t size) {
  CUmulticastObjectProp p = {};
  p.numDevices = static_cast<unsigned>(world);
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  p.flags = 0;
  return p;
}

static int rc_of(CUresult r) { return r == CUDA_SUCCESS ? 0 : 10000 + static_cast<int>(r); }

constexpr int MM_MAX_GRID = 148 * 8;
static inline int mm_grid(long n, int per_thread) {
  long g = (n / per_thread + 255) / 256;
  if (g > MM_MAX_GRID) g = MM_MAX_GRID;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_add_v4(const void* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}

__device__ __forceinline__ float mm_clip_scale(const float* gnorm_sq, float clip) {
  if (gnorm_sq == nullptr || clip <= 0.f) return 1.f;
  const float n = sqrtf(fmaxf(*gnorm_sq, 0.f));
  return n > clip ? clip / (n + 1e-6f) : 1.f;
}

// p -= lr (scale O + wd p) on n elements; bf16 result broadcast through the multicast address.
__global__ void __launch_bounds__(256) mm_muon_apply_kernel(float* __restrict__ p,
                                                            const bf16* __restrict__ o,
                                                            bf16* mc_lp, long n, float lr,
                                                            float scale, float wd) {
  const long n8 = n >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = i * 8;
    float ov[8], q[8];
    unpack8(*reinterpret_cast<const bf16x8*>(o + e), ov);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pi = p[e + j];
      q[j] = pi - lr * (scale * ov[j] + wd * pi);
      p[e + j] = q[j];
    }
    const bf16x8 pk = pack8(q);
    multimem_st_v4(mc_lp + e, *reinterpret_cast<const uint4*>(&pk));
  }
}

__global__ void __launch_bounds__(256) mm_adamw_kernel(
    float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
    float* __restrict__ v, bf16* mc_lp, long n, float lr, float b1, float b2, float eps, float wd,
    float inv_bc1, float inv_bc2, const float* __restrict__ gnorm_sq, float clip, float gscale) {
  const float s = mm_clip_scale(gnorm_sq, clip) * gscale;
  const long n8 = n >> 3;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long e = i * 8;
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gi = g[e + j] * s;
      const float mi = b1 * m[e + j] + (1.f - b1) * gi;
      const float vi = b2 * v[e + j] + (1.f - b2) * gi * gi;
      m[e + j] = mi;
      v[e + j] = vi;
      const float pi = p[e + j] * (1.f - lr * wd) - lr * (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
      p[e + j] = pi;
      o[j] = pi;
    }
    const bf16x8 pk = pack8(o);
    multimem_st_v4(mc_lp + e, *reinterpret_cast<const uint4*>(&pk));
  }
}

// mc[lo : lo + n) (fp32) <- sum over the ranks' copies, written to every rank.
__global__ void __launch_bounds__(256) mm_allreduce_f32_kernel(float* mc, long lo, long n) {
  const long n4 = n >> 2;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  // four in-switch reductions in flight per thread before the first write-back
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = multimem_ld_reduce_add_v4(mc + lo + (i + u * stride) * 4);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      multimem_st_v4(mc + lo + (i + u * stride) * 4, *reinterpret_cast<const uint4*>(&s[u]));
  }
  for (; i < n4; i += stride) {
    float* a = mc + lo + i * 4;
    const float4 s = multimem_ld_reduce_add_v4(a);
    multimem_st_v4(a, *reinterpret_cast<const uint4*>(&s));
  }
}

}  // namespace nvls
}  // namespace pb

using namespace pb;
using namespace pb::nvls;

// *out = 1 when the current device and driver offer multicast objects.
PB_API int pb_nvls_supported(int* out) {
  *out = 0;
  const Api* a = api();
  if (a == nullptr) return 0;
  CUdevice dev;
  if (a->CtxGetDevice(&dev) != CUDA_SUCCESS) {
    cudaFree(nullptr);   // make the primary context current, then ask again
    if (a->CtxGetDevice(&dev) != CUDA_SUCCESS) return 0;
  }
  int v = 0;
  if (a->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  *out = v ? 1 : 0;
  return 0;
}

// Size actually used for `bytes` on a group of `world` devices (multicast granularity).
PB_API long pb_nvls_rounded_size(long bytes, int world) {
  const Api* a = api();
  if (a == nullptr || bytes <= 0) return -1;
  CUmulticastObjectProp p = mc_prop(world, static_cast<size_t>(bytes));
  size_t gran = 0;
  if (a->MulticastGetGranularity(&gran, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS ||
      gran == 0)
    return -1;
  return static_cast<long>((static_cast<size_t>(bytes) + gran - 1) / gran * gran);
}

static Buffer* new_buffer(const Api* a, long size, int world) {
  Buffer* b = new Buffer();
  b->size = static_cast<size_t>(size);
  b->world = world;
  if (a->CtxGetDevice(&b->dev) != CUDA_SUCCESS) {
    cudaFree(nullptr);
    if (a->CtxGetDevice(&b->dev) != CUDA_SUCCESS) { delete b; return nullptr; }
  }
  return b;
}

// Rank 0: create the multicast object of `size` bytes (pb_nvls_rounded_size) for `world` devices
// and export it as a file descriptor to hand to the other ranks (the caller closes it).
PB_API int pb_nvls_create(long size, int world, int* fd_out, void** handle_out) {
  const Api* a = api();
  if (a == nullptr || size <= 0 || world < 2) return PB_BAD_ARG;
  Buffer* b = new_buffer(a, size, world);
  if (b == nullptr) return PB_BAD_ARG;
  CUmulticastObjectProp p = mc_prop(world, b->size);
  CUresult r = a->MulticastCreate(&b->mc, &p);
  if (r != CUDA_SUCCESS) { delete b; return rc_of(r); }
  b->have_mc = true;
  int fd = -1;
  r = a->MemExportToShareableHandle(&fd, b->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { a->MemRelease(b->mc); delete b; return rc_of(r); }
  *fd_out = fd;
  *handle_out = b;
  return 0;
}

PB_API int pb_nvls_import(int fd, long size, int world, void** handle_out) {
  const Api* a = api();
  if (a == nullptr || size <= 0 || world < 2 || fd < 0) return PB_BAD_ARG;
  Buffer* b = new_buffer(a, size, world);
  if (b == nullptr) return PB_BAD_ARG;
  CUresult r = a->MemImportFromShareableHandle(&b->mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) { delete b; return rc_of(r); }
  b->have_mc = true;
  *handle_out = b;
  return 0;
}

PB_API int pb_nvls_close_fd(int fd) { return fd >= 0 ? close(fd) : 0; }

PB_API int pb_nvls_add_device(void* handle) {
  const Api* a = api();
  Buffer* b = static_cast<Buffer*>(handle);
  if (a == nullptr || b == nullptr) return PB_BAD_ARG;
  return rc_of(a->MulticastAddDevice(b->mc, b->dev));
}

// After every rank has added its device: physical memory, unicast mapping, bind, multicast
// mapping. *local_out is this GPU's copy (zero-filled), *mc_out the multicast address.
PB_API int pb_nvls_bind_map(void* handle, void** local_out, void** mc_out) {
  const Api* a = api();
  Buffer* b = static_cast<Buffer*>(handle);
  if (a == nullptr || b == nullptr) return PB_BAD_ARG;
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = b->dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemAccessDesc acc = {};
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUresult r = a->MemCreate(&b->mem, b->size, &prop, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  b->have_mem = true;
  r = a->MemAddressReserve(&b->uc_ptr, b->size, 0, 0, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  r = a->MemMap(b->uc_ptr, b->size, 0, b->mem, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  b->uc_mapped = true;
  r = a->MemSetAccess(b->uc_ptr, b->size, &acc, 1);
  if (r != CUDA_SUCCESS) return rc_of(r);
  cudaError_t e = cudaMemset(reinterpret_cast<void*>(b->uc_ptr), 0, b->size);
  if (e != cudaSuccess) return static_cast<int>(e);
  r = a->MulticastBindMem(b->mc, 0, b->mem, 0, b->size, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  b->bound = true;
  r = a->MemAddressReserve(&b->mc_ptr, b->size, 0, 0, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  r = a->MemMap(b->mc_ptr, b->size, 0, b->mc, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  b->mc_mapped = true;
  r = a->MemSetAccess(b->mc_ptr, b->size, &acc, 1);
  if (r != CUDA_SUCCESS) return rc_of(r);
  *local_out = reinterpret_cast<void*>(b->uc_ptr);
  *mc_out = reinterpret_cast<void*>(b->mc_ptr);
  return 0;
}

// Safe at any stage of the set-up. Call it on every rank, with no kernel of any rank still
// using the buffer (synchronise and meet first).
PB_API int pb_nvls_free(void* handle) {
  const Api* a = api();
  Buffer* b = static_cast<Buffer*>(handle);
  if (a == nullptr || b == nullptr) return PB_BAD_ARG;
  if (b->mc_mapped) a->MemUnmap(b->mc_ptr, b->size);
  if (b->mc_ptr) a->MemAddressFree(b->mc_ptr, b->size);
  if (b->bound) a->MulticastUnbind(b->mc, b->dev, 0, b->size);
  if (b->uc_mapped) a->MemUnmap(b->uc_ptr, b->size);
  if (b->uc_ptr) a->MemAddressFree(b->uc_ptr, b->size);
  if (b->have_mem) a->MemRelease(b->mem);
  if (b->have_mc) a->MemRelease(b->mc);
  delete b;
  return 0;
}

// `p`, `o`: the n-element slice itself (element 0 = first element of the slice); `mc_lp`: the
// multicast address of the same slice of the bf16 copy. n a multiple of 8, addresses 16-byte
// aligned.
PB_API int pb_mm_muon_apply(void* p, const void* o, void* mc_lp, long n, float lr, float scale,
                            float wd, cudaStream_t st) {
  if ((n & 7) != 0 || (reinterpret_cast<uintptr_t>(mc_lp) & 15) != 0) return PB_BAD_ARG;
  if (n == 0) return 0;
  mm_muon_apply_kernel<<<mm_grid(n, 16), 256, 0, st>>>(static_cast<float*>(p),
                                                       static_cast<const bf16*>(o),
                                                       static_cast<bf16*>(mc_lp), n, lr, scale, wd);
  return static_cast<int>(cudaGetLastError());
}

PB_API int pb_mm_adamw(void* p, const void* g, void* m, void* v, void* mc_lp, long n, float lr,
                       float b1, float b2, float eps, float wd, int step, const void* gnorm_sq,
                       float clip, float gscale, cudaStream_t st) {
  if (step < 1 || (n & 7) != 0 || (reinterpret_cast<uintptr_t>(mc_lp) & 15) != 0) return PB_BAD_ARG;
  if (n == 0) return 0;
  const float inv_bc1 = 1.f / (1.f - powf(b1, static_cast<float>(step)));
  const float inv_bc2 = 1.f / (1.f - powf(b2, static_cast<float>(step)));
  mm_adamw_kernel<<<mm_grid(n, 16), 256, 0, st>>>(
      static_cast<float*>(p), static_cast<const float*>(g), static_cast<float*>(m),
      static_cast<float*>(v), static_cast<bf16*>(mc_lp), n, lr, b1, b2, eps, wd, inv_bc1, inv_bc2,
      static_cast<const float*>(gnorm_sq), clip, gscale);
  return static_cast<int>(cudaGetLastError());
}

// In-switch all-reduce of this rank's slice [lo, lo + n) of an fp32 buffer whose multicast
// address is mc: afterwards every rank's copy holds the sum there. lo, n multiples of 4. The
// ranks' slices together cover the buffer; a barrier before (inputs written) and after (all
// slices done) is the caller's.
PB_API int pb_mm_allreduce_f32(void* mc, long lo, long n, cudaStream_t st) {
  if ((lo & 3) != 0 || (n & 3) != 0 || (reinterpret_cast<uintptr_t>(mc) & 15) != 0) return PB_BAD_ARG;
  if (n == 0) return 0;
  mm_allreduce_f32_kernel<<<mm_grid(n, 8), 256, 0, st>>>(static_cast<float*>(mc), lo, n);
  return static_cast<int>(cudaGetLastError());
}
