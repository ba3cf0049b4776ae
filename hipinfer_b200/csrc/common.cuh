// Shared helpers of the sm_100a kernels: element types, error reporting, reductions.
//
// Every launcher is `extern "C" int hb_*(..., cudaStream_t)`: 0 on success, a negative code
// with a message in hb_last_error() otherwise (the reference prints and exits on a CUDA
// error, src/hip_compat.h:95-97, and returns -1 on bad arguments, src/api.cu:1827-1839).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define HB_EXPORT extern "C" __attribute__((visibility("default")))

enum { HB_F32 = 0, HB_BF16 = 1 };

void hb_set_error(const char* fmt, ...);

#define HB_FAIL(...)            \
  do {                          \
    hb_set_error(__VA_ARGS__);  \
    return -1;                  \
  } while (0)

#define HB_CHECK_LAUNCH(name)                                               \
  do {                                                                      \
    cudaError_t e_ = cudaGetLastError();                                    \
    if (e_ != cudaSuccess) HB_FAIL("%s: %s", name, cudaGetErrorString(e_)); \
  } while (0)

__device__ __forceinline__ float hb_to_float(float v) { return v; }
__device__ __forceinline__ float hb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T hb_from_float(float v);
template <> __device__ __forceinline__ float hb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 hb_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float hb_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float hb_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block in a fixed order (lane tree, then warps 0..n-1 in sequence); every thread
// gets the result. `sh` holds at least 32 floats.
__device__ __forceinline__ float hb_block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = hb_warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; i++) t += sh[i];
  return t;
}

// Four consecutive elements as one 16-byte (fp32) or 8-byte (bf16) access.
__device__ __forceinline__ float4 hb_load4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 hb_load4(const __nv_bfloat16* p) {
  const uint2 r = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&r.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&r.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void hb_store4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void hb_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 r;
  r.x = *(uint32_t*)&a;
  r.y = *(uint32_t*)&b;
  *(uint2*)p = r;
}

// Calls f.template operator()<TA, TB>() for the element types named by two dtype codes.
#define HB_DISPATCH_2(da, db, NAME, ...)                                                     \
  do {                                                                                       \
    if ((da) == HB_F32 && (db) == HB_F32) { using TA = float; using TB = float; __VA_ARGS__; }                      \
    else if ((da) == HB_F32 && (db) == HB_BF16) { using TA = float; using TB = __nv_bfloat16; __VA_ARGS__; }        \
    else if ((da) == HB_BF16 && (db) == HB_F32) { using TA = __nv_bfloat16; using TB = float; __VA_ARGS__; }        \
    else if ((da) == HB_BF16 && (db) == HB_BF16) { using TA = __nv_bfloat16; using TB = __nv_bfloat16; __VA_ARGS__; } \
    else HB_FAIL("%s: unknown dtype code %d/%d", NAME, (int)(da), (int)(db));                \
  } while (0)

#define HB_DISPATCH_1(da, NAME, ...)                                        \
  do {                                                                      \
    if ((da) == HB_F32) { using TA = float; __VA_ARGS__; }                  \
    else if ((da) == HB_BF16) { using TA = __nv_bfloat16; __VA_ARGS__; }    \
    else HB_FAIL("%s: unknown dtype code %d", NAME, (int)(da));             \
  } while (0)

// ---------------------------------------------------------------------------------------
// A timing build (-DHB_TL): kernels leave globaltimer stamps of their last launch, per translation
// unit, in slot `id`: phase 0 entry, 1 the dependency wait over, 2 inputs loaded (block 0), 3 the
// end of the block that ended last. Compiled out otherwise.
// ---------------------------------------------------------------------------------------
#ifdef HB_TL
#define HB_TL_DEFINE(tu)                                                                                  \
  static __device__ unsigned long long hb_tl_buf[32 * 4];                                                 \
  HB_EXPORT int hb_tl_dump_##tu(unsigned long long* out) {                                                \
    return cudaMemcpyFromSymbol(out, hb_tl_buf, sizeof(hb_tl_buf)) == cudaSuccess ? 0 : -1;               \
  }
#define HB_TL_MARK(id, ph) hb_tl_mark(hb_tl_buf, id, ph, 0)
#define HB_TL_MARK_T(id, ph, thread) hb_tl_mark(hb_tl_buf, id, ph, thread)
__device__ __forceinline__ void hb_tl_mark(unsigned long long* buf, int id, int ph, int thread) {
  if (threadIdx.x != thread) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  if (ph == 3) atomicMax(&buf[id * 4 + 3], t);
  else if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0) buf[id * 4 + ph] = t;
}
#else
#define HB_TL_DEFINE(tu)
#define HB_TL_MARK(id, ph)
#define HB_TL_MARK_T(id, ph, thread)
#endif

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch: a kernel launched with hb_launch() may start while the kernel
// before it in the stream is still running. It calls hb_pdl_launch() at once (so that ITS
// successor can be staged as early) and hb_pdl_wait() before its first access to anything an
// earlier kernel wrote or still reads; only work on constants (weights, its own shared memory,
// barriers, tensor memory) may come before the wait. hb_pdl_wait() returns when the preceding
// kernel has finished and its writes are visible. With g_hb_pdl == 0 launches are ordinary.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void hb_pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void hb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

extern int g_hb_pdl;

// The same for a kernel whose blocks form clusters of `cluster` (the grid a multiple of it in every dimension).
template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                            dim3 cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_hb_pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_hb_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
