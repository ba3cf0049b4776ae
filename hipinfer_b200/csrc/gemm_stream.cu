// The decode-step matrix product on the 5th-generation tensor cores, operands swapped:
// C^T[N, M] = W[N,K] A[M,K]^T. The 128 weight rows of a CTA are the M side of tcgen05.mma, the
// few token rows (padded to NT = 16, 32 or 64) its N side, so no tensor-core work is wasted on
// padding and every weight byte is read from HBM once, by TMA, through a four-deep pipeline;
// several CTAs share an SM, which keeps close to 200 KB of loads in flight per SM. The
// accumulator (128 lanes x NT columns of tensor memory) comes back with tcgen05.ld: lane = output
// column n, so a warp's stores for one token are 128 contiguous bytes.
//
// A CTA owns 128 output columns and one slice of K; the number of slices depends on (N, K)
// only, never on M, so a token's result does not depend on what else is in the batch. Slices
// leave fp32 partials [slice][token][column]; the CTA that finishes a column block last adds
// them in slice order and applies the epilogue (store fp32 / store bf16 / add into the fp32
// residual / SwiGLU over gate and up columns interleaved by 16), then zeroes the counter.
// Epilogue ST_SLICES leaves the slices where they are for the kernel that consumes the result
// (the next norm, the rotation: gemm_stream_consumers.cu), which adds them in the same order:
// one kernel and one round trip through memory less between two products.
// It replaces gemv_kernel and gemm_skinny_kernel of the reference (src/kernels.cuh:164, 911).
// All waits are bounded.
#include "tc_common.cuh"

HB_TL_DEFINE(stream)

enum { ST_F32 = 0, ST_BF16 = 1, ST_ADD_F32 = 2, ST_SWIGLU_BF16 = 3, ST_SLICES = 4 };
constexpr int ST_ROWS = 128, ST_BK = 64, ST_W_BYTES = ST_ROWS * ST_BK * 2;

// DEEP: the pipeline of a product that is not split along K (many column blocks): six stages,
// two CTAs per SM; otherwise four (three for 64 tokens) and three CTAs per SM.
template <int NT, bool DEEP> struct StreamCfg {
  static constexpr int STAGE = ST_W_BYTES + NT * ST_BK * 2;
  static constexpr int STAGES = DEEP ? (NT <= 32 ? 6 : 4) : (NT <= 32 ? 4 : 3);
  static constexpr int BAR = STAGES * STAGE;
  static constexpr int TOTAL = BAR + 256 + 1024;
  static constexpr int TMEM_COLS = NT < 32 ? 32 : NT;
};

__device__ __forceinline__ void stream_store(int epi, void* C, long ldc, int m, int n, int N, float v, float v_up, bool lower_half) {
  // lower_half: this column is a gate column (n % 32 < 16); v_up is the matching up column's value
  if (epi == ST_SWIGLU_BF16) {
    if (lower_half && n < N) ((__nv_bfloat16*)C)[(size_t)m * ldc + (n >> 5) * 16 + (n & 15)] =
        __float2bfloat16_rn(v / (1.f + __expf(-v)) * v_up);
  } else if (n < N) {
    if (epi == ST_BF16) ((__nv_bfloat16*)C)[(size_t)m * ldc + n] = __float2bfloat16_rn(v);
    else if (epi == ST_ADD_F32) ((float*)C)[(size_t)m * ldc + n] += v;
    else ((float*)C)[(size_t)m * ldc + n] = v;
  }
}

template <int NT, bool DEEP>
__global__ void __launch_bounds__(192) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w,
                                                          const __grid_constant__ CUtensorMap map_x, void* C, long ldc,
                                                          int M, int N, int K, int kslice, float* ws, int* counters,
                                                          int epi, int* status, int defer) {
  using S = StreamCfg<NT, DEEP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + S::BAR);
  uint64_t* empty = full + S::STAGES;
  uint64_t* done = empty + S::STAGES;
  uint32_t* tmem_slot = (uint32_t*)(done + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* is_last = (int*)(tmem_slot + 2);

  hb_pdl_launch();
  HB_TL_MARK(0, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x, sp = blockIdx.y, ksplit = gridDim.y, NP = gridDim.x * ST_ROWS;
  const int n0 = nb * ST_ROWS, k_begin = sp * kslice, k_end = min(K, k_begin + kslice);
  const int num_kb = (k_end - k_begin + ST_BK - 1) / ST_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; s++) { hb_mbar_init(&full[s], 1); hb_mbar_init(&empty[s], 1); }
    hb_mbar_init(done, 1);
    *abort_flag = 0;
    hb_fence_barrier_init();
  }
  if (warp == 5) {
    hb_tmem_alloc(tmem_slot, S::TMEM_COLS);
    hb_tmem_relinquish();
  }
  if (warp == 4 && lane == 0) { hb_tma_prefetch_desc(&map_w); hb_tma_prefetch_desc(&map_x); }
  hb_tc_fence_before();
  __syncthreads();
  hb_tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      // the weights do not depend on the kernel before this one: the first stages' weight tiles
      // are requested before the wait, the activations after it
      const int pre = num_kb < S::STAGES ? num_kb : S::STAGES;
      for (int kb = 0; kb < pre; kb++) {
        hb_mbar_expect_tx(&full[kb], S::STAGE);
        hb_tma_load_2d(smem + kb * S::STAGE, &map_w, &full[kb], k_begin + kb * ST_BK, n0);
      }
      hb_pdl_wait();
      HB_TL_MARK_T(0, 1, 128);
      for (int kb = 0; kb < pre; kb++)
        hb_tma_load_2d(smem + kb * S::STAGE + ST_W_BYTES, &map_x, &full[kb], k_begin + kb * ST_BK, 0);
      for (int kb = pre; kb < num_kb; kb++) {
        const uint32_t s = kb % S::STAGES, ph = (kb / S::STAGES) & 1;
        if (!hb_mbar_wait(&empty[s], ph ^ 1, abort_flag)) break;
        hb_mbar_expect_tx(&full[s], S::STAGE);
        hb_tma_load_2d(smem + s * S::STAGE, &map_w, &full[s], k_begin + kb * ST_BK, n0);
        hb_tma_load_2d(smem + s * S::STAGE + ST_W_BYTES, &map_x, &full[s], k_begin + kb * ST_BK, 0);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = hb_umma_idesc_bf16(ST_ROWS, NT);
      bool ok = true;
      for (int kb = 0; kb < num_kb; kb++) {
        const uint32_t s = kb % S::STAGES, ph = (kb / S::STAGES) & 1;
        if (!hb_mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
        hb_tc_fence_after();
        const uint64_t dw = hb_umma_desc_k128(hb_smem_u32(smem + s * S::STAGE));
        const uint64_t dx = hb_umma_desc_k128(hb_smem_u32(smem + s * S::STAGE + ST_W_BYTES));
#pragma unroll
        for (int k = 0; k < ST_BK / 16; k++) hb_umma_bf16(tmem_base, dw + 2 * k, dx + 2 * k, idesc, (kb | k) != 0);
        hb_umma_commit(&empty[s]);
      }
      if (ok) hb_umma_commit(done);
    }
  } else {
    // epilogue warps: lane = output column n0 + 32 * warp + lane, v[m] = token m
    const bool ok = hb_mbar_wait(done, 0, abort_flag);
    hb_tc_fence_after();
    hb_pdl_wait();  // before the first access to memory that earlier kernels wrote or still read
    HB_TL_MARK(0, 2);   // (thread 0 is an epilogue thread: the product is done)
    float v[NT];
#pragma unroll
    for (int c = 0; c < NT / 16; c++) hb_tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + c * 16, v + 16 * c);
    const int n = n0 + warp * 32 + lane;
    if (ksplit == 1 && epi != ST_SLICES) {
#pragma unroll
      for (int m = 0; m < NT; m++) {
        if (m < M) {
          const float up = __shfl_down_sync(0xffffffffu, v[m], 16);
          if (ok) stream_store(epi, C, ldc, m, n, N, v[m], up, (lane & 16) == 0);
        }
      }
    } else if (ok) {
#pragma unroll
      for (int m = 0; m < NT; m++)
        if (m < M) ws[((size_t)sp * NT + m) * NP + n] = v[m];
    }
    hb_tc_fence_before();
  }

  HB_TL_MARK(0, 3);
  if (ksplit > 1 && !defer) __threadfence();   // only the block that adds the slices in here has to see the others' partials
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    hb_tmem_dealloc(tmem_base, S::TMEM_COLS);
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    __nanosleep(100000);
  }
  if (ksplit == 1 || defer) return;  // defer: stream_reduce_kernel adds the slices, with the whole GPU

  if (threadIdx.x == 0) *is_last = atomicAdd(&counters[nb], 1) == ksplit - 1;
  __syncthreads();
  if (!*is_last) return;
  __threadfence();
  // four consecutive columns per thread, the slices' loads issued four at a time, added in slice order
  const size_t slice_stride = (size_t)NT * NP;
  for (int i = threadIdx.x; i < (ST_ROWS / 4) * M; i += 192) {
    const int m = i / (ST_ROWS / 4), nl = (i - m * (ST_ROWS / 4)) * 4, n = n0 + nl;
    const bool gate = (nl & 16) == 0, swiglu = epi == ST_SWIGLU_BF16;
    if (n >= N || (swiglu && !gate)) continue;
    const float* p = ws + (size_t)m * NP + n;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), up = acc;
    int sl = 0;
    for (; sl + 4 <= ksplit; sl += 4) {
      float4 a[4], u[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        a[j] = __ldcg((const float4*)(p + (sl + j) * slice_stride));
        if (swiglu) u[j] = __ldcg((const float4*)(p + (sl + j) * slice_stride + 16));
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        acc.x += a[j].x; acc.y += a[j].y; acc.z += a[j].z; acc.w += a[j].w;
        if (swiglu) { up.x += u[j].x; up.y += u[j].y; up.z += u[j].z; up.w += u[j].w; }
      }
    }
    for (; sl < ksplit; sl++) {
      const float4 a = __ldcg((const float4*)(p + sl * slice_stride));
      acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
      if (swiglu) {
        const float4 u = __ldcg((const float4*)(p + sl * slice_stride + 16));
        up.x += u.x; up.y += u.y; up.z += u.z; up.w += u.w;
      }
    }
    stream_store(epi, C, ldc, m, n, N, acc.x, up.x, gate);
    stream_store(epi, C, ldc, m, n + 1, N, acc.y, up.y, gate);
    stream_store(epi, C, ldc, m, n + 2, N, acc.z, up.z, gate);
    stream_store(epi, C, ldc, m, n + 3, N, acc.w, up.w, gate);
  }
  if (threadIdx.x == 0) counters[nb] = 0;
}

// The slices' partial sums added in slice order and the epilogue applied, four columns per thread,
// over the whole output at once. With many token rows this is much more work than one CTA per
// column block should do at the end of the product kernel, so it runs as a kernel of its own.
__global__ void __launch_bounds__(256) stream_reduce_kernel(const float* __restrict__ ws, void* C, long ldc, int M, int N,
                                                            int NP, int NT, int ksplit, int epi) {
  hb_pdl_launch();
  HB_TL_MARK(5, 0);
  hb_pdl_wait();
  HB_TL_MARK(5, 1);
  const int per_row = NP >> 2;
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)M * per_row) return;
  const int m = (int)(idx / per_row), n = (int)(idx - (long)m * per_row) * 4;
  const bool gate = (n & 16) == 0, swiglu = epi == ST_SWIGLU_BF16;
  if (n >= N || (swiglu && !gate)) return;
  const size_t slice_stride = (size_t)NT * NP;
  const float* p = ws + (size_t)m * NP + n;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), up = acc;
  int sl = 0;
  for (; sl + 4 <= ksplit; sl += 4) {
    float4 a[4], u[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      a[j] = __ldcg((const float4*)(p + (sl + j) * slice_stride));
      if (swiglu) u[j] = __ldcg((const float4*)(p + (sl + j) * slice_stride + 16));
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      acc.x += a[j].x; acc.y += a[j].y; acc.z += a[j].z; acc.w += a[j].w;
      if (swiglu) { up.x += u[j].x; up.y += u[j].y; up.z += u[j].z; up.w += u[j].w; }
    }
  }
  for (; sl < ksplit; sl++) {
    const float4 a = __ldcg((const float4*)(p + sl * slice_stride));
    acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
    if (swiglu) {
      const float4 u = __ldcg((const float4*)(p + sl * slice_stride + 16));
      up.x += u.x; up.y += u.y; up.z += u.z; up.w += u.w;
    }
  }
  stream_store(epi, C, ldc, m, n, N, acc.x, up.x, gate);
  stream_store(epi, C, ldc, m, n + 1, N, acc.y, up.y, gate);
  stream_store(epi, C, ldc, m, n + 2, N, acc.z, up.z, gate);
  stream_store(epi, C, ldc, m, n + 3, N, acc.w, up.w, gate);
  HB_TL_MARK(5, 3);
}

// The split of K for an [N, K] weight: a function of the weight's shape alone.
static void stream_plan(int N, int K, int sms, int* kslice, int* ksplit) {
  const int n_blocks = (N + ST_ROWS - 1) / ST_ROWS;
  int want = (3 * sms) / n_blocks;
  int max_split = K / 256;               // a slice is at least 256 deep, and there are at most 16
  if (max_split > 16) max_split = 16;
  if (want > max_split) want = max_split;
  if (want < 1) want = 1;
  int ks = (K + want - 1) / want;
  ks = (ks + ST_BK - 1) / ST_BK * ST_BK;
  *kslice = ks;
  *ksplit = (K + ks - 1) / ks;
}

HB_EXPORT int hb_gemm_stream_plan(int N, int K, int* kslice, int* ksplit, long* ws_floats_per_token, int* n_blocks) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  stream_plan(N, K, sms, kslice, ksplit);
  *n_blocks = (N + ST_ROWS - 1) / ST_ROWS;
  *ws_floats_per_token = (long)(*ksplit) * (*n_blocks) * ST_ROWS;   // not needed when ksplit is 1, except for ST_SLICES
  return 0;
}

template <int NT, bool DEEP>
static int launch_stream(const CUtensorMap& mw, const CUtensorMap& mx, void* C, long ldc, int M, int N, int K, int kslice,
                         int ksplit, int n_blocks, float* ws, int* counters, int epi, int* status, cudaStream_t s) {
  // from 8 token rows on (measured) the slices are added by a kernel of its own; ST_SLICES leaves them to the consumer
  const int defer = epi == ST_SLICES || (ksplit > 1 && M >= 8);
  using S = StreamCfg<NT, DEEP>;
  auto kern = gemm_stream_kernel<NT, DEEP>;
  static bool configured[64] = {};      // the attribute belongs to a device: set once on each
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_stream: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  cudaError_t e = hb_launch(kern, dim3(n_blocks, ksplit), 192, S::TOTAL, s, mw, mx, C, ldc, M, N, K, kslice, ws, counters,
                            epi, status, defer);
  if (e != cudaSuccess) HB_FAIL("hb_gemm_stream: %s", cudaGetErrorString(e));
  if (defer && epi != ST_SLICES) {
    const int NP = n_blocks * ST_ROWS;
    const long items = (long)M * (NP / 4);
    e = hb_launch(stream_reduce_kernel, (unsigned)((items + 255) / 256), 256, 0, s, (const float*)ws, C, ldc, M, N, NP, NT,
                  ksplit, epi);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_stream: %s", cudaGetErrorString(e));
  }
  return 0;
}

// C per `epi` (0 fp32, 1 bf16, 2 fp32 +=, 3 bf16 SwiGLU [M, N/2]) for M <= 64. ws: at least
// ksplit * n_blocks * 128 * NT floats when ksplit > 1 (NT = M rounded up to 16, 32 or 64);
// counters: n_blocks ints, all zero (left zero). Calls sharing ws/counters must not overlap.
// epi 4: C is not touched; ws keeps the slices [ksplit][NT][n_blocks * 128] (also when ksplit is 1).
HB_EXPORT int hb_gemm_stream(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int N, int K,
                             int epi, float* ws, long ws_floats, int* counters, int n_counters, int* status,
                             cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) HB_FAIL("hb_gemm_stream: M = %d is beyond 64 rows", M);
  if (K <= 0 || (K & 7)) HB_FAIL("hb_gemm_stream: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  if (epi < 0 || epi > 4) HB_FAIL("hb_gemm_stream: unknown epilogue %d", epi);
  if (epi == ST_SWIGLU_BF16 && (N & 31)) HB_FAIL("hb_gemm_stream: SwiGLU needs N = %d to be a multiple of 32", N);
  if (!status) HB_FAIL("hb_gemm_stream: no status word");
  int kslice, ksplit, n_blocks;
  long per_token;
  hb_gemm_stream_plan(N, K, &kslice, &ksplit, &per_token, &n_blocks);
  const int NT = M <= 16 ? 16 : M <= 32 ? 32 : 64;
  if ((ksplit > 1 || epi == ST_SLICES) && (!ws || ws_floats < per_token * NT))
    HB_FAIL("hb_gemm_stream: workspace of %ld floats, %ld needed", ws_floats, per_token * NT);
  if (ksplit > 1 && (!counters || n_counters < n_blocks)) HB_FAIL("hb_gemm_stream: %d counters, %d needed", n_counters, n_blocks);
  CUtensorMap mw, mx;
  if (hb_make_tensor_map_bf16(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, ST_ROWS)) return -1;
  if (hb_make_tensor_map_bf16(&mx, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, (uint32_t)NT)) return -1;
  int r;
#define HB_ST_ARGS mw, mx, C, ldc, M, N, K, kslice, ksplit, n_blocks, ws, counters, epi, status, s
  if (ksplit == 1) {
    if (NT == 16) r = launch_stream<16, true>(HB_ST_ARGS);
    else if (NT == 32) r = launch_stream<32, true>(HB_ST_ARGS);
    else r = launch_stream<64, true>(HB_ST_ARGS);
  } else {
    if (NT == 16) r = launch_stream<16, false>(HB_ST_ARGS);
    else if (NT == 32) r = launch_stream<32, false>(HB_ST_ARGS);
    else r = launch_stream<64, false>(HB_ST_ARGS);
  }
#undef HB_ST_ARGS
  if (r) return r;
  HB_CHECK_LAUNCH("hb_gemm_stream");
  return 0;
}

// Finish a product that was left as slices (epi 4): C per `epi` (0 to 3) from ws, for the same M, N, K.
HB_EXPORT int hb_gemm_stream_finish(const float* ws, void* C, long ldc, int M, int N, int K, int epi, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (epi < 0 || epi > 3) HB_FAIL("hb_gemm_stream_finish: unknown epilogue %d", epi);
  int kslice, ksplit, n_blocks;
  long per_token;
  hb_gemm_stream_plan(N, K, &kslice, &ksplit, &per_token, &n_blocks);
  const int NT = M <= 16 ? 16 : M <= 32 ? 32 : 64, NP = n_blocks * ST_ROWS;
  const long items = (long)M * (NP / 4);
  cudaError_t e = hb_launch(stream_reduce_kernel, (unsigned)((items + 255) / 256), 256, 0, s, ws, C, ldc, M, N, NP, NT,
                            ksplit, epi);
  if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_finish: %s", cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------------------------------
// hb_gemm_stream_static: the same product for callers that must not allocate (declared in
// gemm_stream_static.h). The split-K partial sums and the per-block counters live in two
// file-scope device arrays instead of a caller-provided workspace.
// ---------------------------------------------------------------------------------------
#include "gemm_stream_static.h"

static __device__ __align__(256) float g_static_ws[HB_STATIC_WS_FLOATS];
static __device__ __align__(256) int g_static_counters[HB_STATIC_COUNTERS];

// The arrays' device addresses, looked up once per device. In host code the names above are
// host-side stand-ins, not device addresses, so they are never passed to a kernel directly.
static float* g_static_ws_ptr[HB_STATIC_MAX_DEVICES];
static int* g_static_cnt_ptr[HB_STATIC_MAX_DEVICES];

HB_EXPORT int hb_gemm_stream_static(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int N,
                                    int K, int epi, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_static: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= HB_STATIC_MAX_DEVICES) HB_FAIL("hb_gemm_stream_static: device %d is beyond %d", dev, HB_STATIC_MAX_DEVICES);
  if (!g_static_ws_ptr[dev]) {  // first call on this device (it is the current one): not inside a stream capture
    void *pw = nullptr, *pc = nullptr;
    e = cudaGetSymbolAddress(&pw, g_static_ws);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_static: address of the scratch array: %s", cudaGetErrorString(e));
    e = cudaGetSymbolAddress(&pc, g_static_counters);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_static: address of the counter array: %s", cudaGetErrorString(e));
    g_static_cnt_ptr[dev] = (int*)pc;
    g_static_ws_ptr[dev] = (float*)pw;
  }
  if (M > 64) HB_FAIL("hb_gemm_stream_static: M = %d is beyond 64 rows", M);
  if (K <= 0 || (K & 7)) HB_FAIL("hb_gemm_stream_static: K = %d must be a positive multiple of 8", K);
  if (epi < 0 || epi > 3) HB_FAIL("hb_gemm_stream_static: unknown epilogue %d (0 to 3)", epi);
  if (epi == ST_SWIGLU_BF16 && (N & 31)) HB_FAIL("hb_gemm_stream_static: SwiGLU needs N = %d to be a multiple of 32", N);
  if (!status) HB_FAIL("hb_gemm_stream_static: no status word");
  int kslice, ksplit, n_blocks;
  long per_token;
  hb_gemm_stream_plan(N, K, &kslice, &ksplit, &per_token, &n_blocks);
  const int NT = M <= 16 ? 16 : M <= 32 ? 32 : 64;
  if (ksplit == 1) per_token = 0;   // a product that is not split needs no scratch
  if (per_token * NT > (long)HB_STATIC_WS_FLOATS)
    HB_FAIL("hb_gemm_stream_static: M = %d, N = %d, K = %d need %ld floats of scratch; the static array holds %ld", M, N, K,
            per_token * NT, (long)HB_STATIC_WS_FLOATS);
  if (ksplit > 1 && n_blocks > HB_STATIC_COUNTERS)
    HB_FAIL("hb_gemm_stream_static: N = %d needs %d block counters; the static array holds %d", N, n_blocks, HB_STATIC_COUNTERS);
  if (ksplit > 1) {
    // every call shares the arrays and finds what the last one left: the counters this call uses must start at zero
    e = cudaMemsetAsync(g_static_cnt_ptr[dev], 0, sizeof(int) * n_blocks, s);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_static: clearing the counters: %s", cudaGetErrorString(e));
  }
  return hb_gemm_stream(A, lda, W, ldw, C, ldc, M, N, K, epi, g_static_ws_ptr[dev], (long)HB_STATIC_WS_FLOATS,
                        g_static_cnt_ptr[dev], ksplit > 1 ? HB_STATIC_COUNTERS : n_blocks, status, s);
}
