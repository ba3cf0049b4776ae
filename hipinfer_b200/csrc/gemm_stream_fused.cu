// Decode-step products with their neighbours fused in, for up to 16 token rows:
//
//   mode 0:  act = SwiGLU( RMSNorm(x) Wgu^T )                      (norm + gate/up + activation)
//   mode 1:  q, k, v = RMSNorm(x) Wqkv^T; rotary on q and k; q to q_out, k and v to their page slots
//
// The product itself is gemm_stream.cu's: 128 weight rows are the M side of tcgen05.mma, the
// token rows its N side, weights streamed once by TMA, K split by a factor that depends on the
// weight's shape only, partial sums added in slice order by the CTA that finishes a column
// block last. What is new: the activation operand is not loaded but MADE here. While the weight
// tiles are in flight, the four epilogue warps read the fp32 residual rows, compute
// r = rsqrt(mean(x^2) + eps) in fp32 (one warp per token, fixed order), and write
// bf16(w * (x * r)) for this CTA's slice of K straight into shared memory in the 128-byte-swizzled
// K-major layout that tcgen05.mma reads. The last CTA of a column block then applies the
// activation or the rotation to the summed columns (a column block is one or two whole heads,
// so a rotary pair (d, d + D/2) lies inside it) and writes q, or the cache page slot, directly.
// The reference fuses the same neighbours into its GEMV (gemv_kernel NORM prologue and EPI 2 / 3,
// src/kernels.cuh:182-200, 264-278). Every wait is bounded.
#include "tc_common.cuh"

constexpr int FS_ROWS = 128, FS_BK = 64, FS_NT = 16, FS_STAGES = 4;  // at most; three when the slice's activations are large
constexpr int FS_W_BYTES = FS_ROWS * FS_BK * 2, FS_X_TILE = FS_NT * FS_BK * 2;

struct FusedArgs {
  const float* x; long ldx; const int* rows;   // residual stream [*, K] fp32; rows: optional gather of the M rows
  const void* norm_w; int norm_w_bf16; float eps;
  int mode;                                    // 0 SwiGLU, 1 rotary + cache write
  __nv_bfloat16* out; long ldo;                // act [M, N/2] (mode 0) or q [M, Hq*D] (mode 1)
  const int* pos; const int* slot_map; const float2* table;
  __nv_bfloat16* kc; __nv_bfloat16* vc;
  int Hq, Hkv, D, page_size;
};

__device__ __forceinline__ void fs_bar_epilogue() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ float4 fs_load_w4(const void* w, int bf16, int k) {
  if (bf16) {
    const uint2 r = *(const uint2*)((const __nv_bfloat16*)w + k);
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&r.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&r.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
  return *(const float4*)((const float*)w + k);
}

__global__ void __launch_bounds__(192) gemm_stream_fused_kernel(const __grid_constant__ CUtensorMap map_w, const FusedArgs a,
                                                                int M, int N, int K, int kslice, int stages, float* ws,
                                                                int* counters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int kb_max = (kslice + FS_BK - 1) / FS_BK;
  uint8_t* xr = smem + stages * FS_W_BYTES;                    // [kb_max][16][64] bf16, swizzled tiles
  uint64_t* full = (uint64_t*)(xr + kb_max * FS_X_TILE);
  uint64_t* empty = full + FS_STAGES;
  uint64_t* done = empty + FS_STAGES;
  uint64_t* xready = done + 1;
  uint32_t* tmem_slot = (uint32_t*)(xready + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  int* is_last = (int*)(tmem_slot + 2);
  float* rinv = (float*)(tmem_slot + 4);                        // [16]

  hb_pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = blockIdx.x, sp = blockIdx.y, ksplit = gridDim.y, NP = gridDim.x * FS_ROWS;
  const int n0 = nb * FS_ROWS, k_begin = sp * kslice, k_end = min(K, k_begin + kslice);
  const int num_kb = (k_end - k_begin + FS_BK - 1) / FS_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < FS_STAGES; s++) { hb_mbar_init(&full[s], 1); hb_mbar_init(&empty[s], 1); }
    hb_mbar_init(done, 1);
    hb_mbar_init(xready, 128);
    *abort_flag = 0;
    hb_fence_barrier_init();
  }
  if (warp == 5) {
    hb_tmem_alloc(tmem_slot, 32);
    hb_tmem_relinquish();
  }
  if (warp == 4 && lane == 0) hb_tma_prefetch_desc(&map_w);
  hb_tc_fence_before();
  __syncthreads();
  hb_tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {  // weights only: they do not depend on the kernel before this one
      for (int kb = 0; kb < num_kb; kb++) {
        const uint32_t s = kb % stages, ph = (kb / stages) & 1;
        if (!hb_mbar_wait(&empty[s], ph ^ 1, abort_flag)) break;
        hb_mbar_expect_tx(&full[s], FS_W_BYTES);
        hb_tma_load_2d(smem + s * FS_W_BYTES, &map_w, &full[s], k_begin + kb * FS_BK, n0);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = hb_umma_idesc_bf16(FS_ROWS, FS_NT);
      bool ok = hb_mbar_wait(xready, 0, abort_flag);
      for (int kb = 0; kb < num_kb && ok; kb++) {
        const uint32_t s = kb % stages, ph = (kb / stages) & 1;
        if (!hb_mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
        hb_tc_fence_after();
        const uint64_t dw = hb_umma_desc_k128(hb_smem_u32(smem + s * FS_W_BYTES));
        const uint64_t dx = hb_umma_desc_k128(hb_smem_u32(xr + kb * FS_X_TILE));
#pragma unroll
        for (int k = 0; k < FS_BK / 16; k++) hb_umma_bf16(tmem_base, dw + 2 * k, dx + 2 * k, idesc, (kb | k) != 0);
        hb_umma_commit(&empty[s]);
      }
      if (ok) hb_umma_commit(done);
    }
  } else {
    // ---- the four epilogue warps first make the normalised activations of this slice
    hb_pdl_wait();
    const int tid = threadIdx.x;
    for (int m = warp; m < M; m += 4) {  // one warp per token, lanes stride the row, fixed order
      const float* row = a.x + (size_t)(a.rows ? a.rows[m] : m) * a.ldx;
      float ss = 0.f;
#pragma unroll 8
      for (int i = lane; i < (K >> 2); i += 32) {
        const float4 v = *(const float4*)(row + 4 * i);
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
      }
      ss = hb_warp_sum(ss);
      if (lane == 0) rinv[m] = rsqrtf(ss / (float)K + a.eps);
    }
    fs_bar_epilogue();
    const int cpr = num_kb * 8;  // 16-byte chunks per token row in this slice
    for (int idx = tid; idx < FS_NT * cpr; idx += 128) {
      const int m = idx / cpr, cc = idx - m * cpr, kb = cc >> 3, c = cc & 7, k = k_begin + cc * 8;
      uint4 packed = make_uint4(0, 0, 0, 0);
      if (m < M && k < K) {
        const float* row = a.x + (size_t)(a.rows ? a.rows[m] : m) * a.ldx + k;
        const float4 x0 = *(const float4*)row, x1 = *(const float4*)(row + 4);
        const float4 w0 = fs_load_w4(a.norm_w, a.norm_w_bf16, k), w1 = fs_load_w4(a.norm_w, a.norm_w_bf16, k + 4);
        const float r = rinv[m];
        packed.x = hb_pack_bf16(w0.x * (x0.x * r), w0.y * (x0.y * r));
        packed.y = hb_pack_bf16(w0.z * (x0.z * r), w0.w * (x0.w * r));
        packed.z = hb_pack_bf16(w1.x * (x1.x * r), w1.y * (x1.y * r));
        packed.w = hb_pack_bf16(w1.z * (x1.z * r), w1.w * (x1.w * r));
      }
      const uint32_t dst = hb_smem_u32(xr + kb * FS_X_TILE) + m * 128 + ((c ^ (m & 7)) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed.x), "r"(packed.y), "r"(packed.z), "r"(packed.w) : "memory");
    }
    hb_fence_proxy_async();  // these generic-proxy writes are read by the tensor core's async proxy
    hb_mbar_arrive(xready);

    // ---- then the accumulator: lane = output column n0 + 32 * warp + lane, v[m] = token m
    const bool ok = hb_mbar_wait(done, 0, abort_flag);
    hb_tc_fence_after();
    float v[FS_NT];
    hb_tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16), v);
    const int n = n0 + warp * 32 + lane;
    if (ok) {
#pragma unroll
      for (int m = 0; m < FS_NT; m++)
        if (m < M) ws[((size_t)sp * FS_NT + m) * NP + n] = v[m];
    }
    hb_tc_fence_before();
  }

  __threadfence();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    hb_tmem_dealloc(tmem_base, 32);
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    __nanosleep(100000);
  }
  if (threadIdx.x == 0) *is_last = atomicAdd(&counters[nb], 1) == ksplit - 1;
  __syncthreads();
  if (!*is_last) return;
  __threadfence();

  const size_t slice_stride = (size_t)FS_NT * NP;
  if (a.mode == 0) {
    // SwiGLU: gate columns nl % 32 < 16, the matching up column 16 further; four columns per thread
    for (int i = threadIdx.x; i < (FS_ROWS / 4) * M; i += 192) {
      const int m = i / (FS_ROWS / 4), nl = (i - m * (FS_ROWS / 4)) * 4, n = n0 + nl;
      if (n >= N || (nl & 16)) continue;
      const float* p = ws + (size_t)m * NP + n;
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
      for (int sl = 0; sl < ksplit; sl++) {
        const float4 gg = __ldcg((const float4*)(p + sl * slice_stride)), uu = __ldcg((const float4*)(p + sl * slice_stride + 16));
        g.x += gg.x; g.y += gg.y; g.z += gg.z; g.w += gg.w;
        u.x += uu.x; u.y += uu.y; u.z += uu.z; u.w += uu.w;
      }
      __nv_bfloat16* o = a.out + (size_t)m * a.ldo + (n >> 5) * 16 + (n & 15);
      uint2 r;
      r.x = hb_pack_bf16(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
      r.y = hb_pack_bf16(g.z / (1.f + __expf(-g.z)) * u.z, g.w / (1.f + __expf(-g.w)) * u.w);
      *(uint2*)o = r;
    }
  } else {
    // rotary + cache write: a thread takes four pairs (j..j+3, j + D/2 ..) of one head of one token
    const int D = a.D, half = D >> 1, heads = FS_ROWS / D, qph = half >> 2;  // quads of pairs per head
    for (int i = threadIdx.x; i < M * heads * qph; i += 192) {
      const int m = i / (heads * qph), rem = i - m * (heads * qph), hl = rem / qph, j = (rem - hl * qph) * 4;
      const int n1 = n0 + hl * D + j, hh = (n0 + hl * D) / D;
      if (n1 >= N) continue;
      const float* p = ws + (size_t)m * NP + n1;
      float4 x1 = make_float4(0.f, 0.f, 0.f, 0.f), x2 = x1;
      for (int sl = 0; sl < ksplit; sl++) {
        const float4 aa = __ldcg((const float4*)(p + sl * slice_stride)), bb = __ldcg((const float4*)(p + sl * slice_stride + half));
        x1.x += aa.x; x1.y += aa.y; x1.z += aa.z; x1.w += aa.w;
        x2.x += bb.x; x2.y += bb.y; x2.z += bb.z; x2.w += bb.w;
      }
      __nv_bfloat16* dst;
      if (hh < a.Hq + a.Hkv) {
        const float2* cs = a.table + (size_t)a.pos[m] * half + j;
        const float4 c01 = *(const float4*)cs, c23 = *(const float4*)(cs + 2);
        float4 y1, y2;
        y1.x = __fsub_rn(__fmul_rn(x1.x, c01.x), __fmul_rn(x2.x, c01.y)); y2.x = __fadd_rn(__fmul_rn(x2.x, c01.x), __fmul_rn(x1.x, c01.y));
        y1.y = __fsub_rn(__fmul_rn(x1.y, c01.z), __fmul_rn(x2.y, c01.w)); y2.y = __fadd_rn(__fmul_rn(x2.y, c01.z), __fmul_rn(x1.y, c01.w));
        y1.z = __fsub_rn(__fmul_rn(x1.z, c23.x), __fmul_rn(x2.z, c23.y)); y2.z = __fadd_rn(__fmul_rn(x2.z, c23.x), __fmul_rn(x1.z, c23.y));
        y1.w = __fsub_rn(__fmul_rn(x1.w, c23.z), __fmul_rn(x2.w, c23.w)); y2.w = __fadd_rn(__fmul_rn(x2.w, c23.z), __fmul_rn(x1.w, c23.w));
        x1 = y1; x2 = y2;
      }
      if (hh < a.Hq) {
        dst = a.out + (size_t)m * a.ldo + hh * D + j;
      } else {
        const int slot = a.slot_map ? a.slot_map[m] : -1;
        if (slot < 0) continue;
        const size_t page = slot / a.page_size, off = slot % a.page_size;
        const bool is_k = hh < a.Hq + a.Hkv;
        const int hk = is_k ? hh - a.Hq : hh - a.Hq - a.Hkv;
        dst = (is_k ? a.kc : a.vc) + ((page * a.Hkv + hk) * a.page_size + off) * D + j;
      }
      uint2 r1, r2;
      r1.x = hb_pack_bf16(x1.x, x1.y); r1.y = hb_pack_bf16(x1.z, x1.w);
      r2.x = hb_pack_bf16(x2.x, x2.y); r2.y = hb_pack_bf16(x2.z, x2.w);
      *(uint2*)dst = r1;
      *(uint2*)(dst + half) = r2;
    }
  }
  if (threadIdx.x == 0) counters[nb] = 0;
}

extern "C" int hb_gemm_stream_plan(int N, int K, int* kslice, int* ksplit, long* ws_floats_per_token, int* n_blocks);

// Can the fused kernel take this product? (the K slice's activations must fit beside the weight stages)
HB_EXPORT int hb_gemm_stream_fused_supported(int M, int N, int K) {
  if (M <= 0 || M > FS_NT || K <= 0 || (K & 7) || N <= 0) return 0;
  int kslice, ksplit, n_blocks;
  long per_token;
  hb_gemm_stream_plan(N, K, &kslice, &ksplit, &per_token, &n_blocks);
  return kslice <= 1024;
}

// mode 0: out = act [M, N/2] bf16. mode 1: out = q [M, Hq*D] bf16, k/v to kc/vc at slot_map
// (cache layout [page][kv head][page_size][D]); needs 128 % D == 0 and N == (Hq + 2 Hkv) D a
// multiple of 128. x: fp32 rows (gathered through `rows` when given), K a multiple of 8, ldx of 4.
// ws: ksplit * n_blocks * 128 * 16 floats; counters: n_blocks ints, zero (left zero).
HB_EXPORT int hb_gemm_stream_fused(const float* x, long ldx, const int* rows, const void* norm_w, int norm_w_dt, float eps,
                                   const void* W, long ldw, int M, int N, int K, int mode, void* out, long ldo,
                                   const int* pos, const int* slot_map, const void* table, void* kc, void* vc, int Hq,
                                   int Hkv, int D, int page_size, float* ws, long ws_floats, int* counters,
                                   int n_counters, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (!hb_gemm_stream_fused_supported(M, N, K)) HB_FAIL("hb_gemm_stream_fused: M = %d, N = %d, K = %d are not supported", M, N, K);
  if ((ldx & 3) || ((uintptr_t)x & 15) || ((uintptr_t)norm_w & 15)) HB_FAIL("hb_gemm_stream_fused: x and the norm weight must be 16-byte aligned");
  if (norm_w_dt != HB_F32 && norm_w_dt != HB_BF16) HB_FAIL("hb_gemm_stream_fused: unknown norm weight type %d", norm_w_dt);
  if (mode == 0) {
    if ((N & 31) || (ldo & 3)) HB_FAIL("hb_gemm_stream_fused: SwiGLU needs N = %d a multiple of 32", N);
  } else if (mode == 1) {
    if (D <= 0 || FS_ROWS % D || (D & 7) || N != (Hq + 2 * Hkv) * D || N % FS_ROWS || (ldo & 3))
      HB_FAIL("hb_gemm_stream_fused: rotary epilogue needs head_dim %d to divide 128 and N = %d = (Hq + 2 Hkv) D, a multiple of 128", D, N);
    if (!pos || !table) HB_FAIL("hb_gemm_stream_fused: rotary epilogue needs positions and a table");
  } else {
    HB_FAIL("hb_gemm_stream_fused: unknown mode %d", mode);
  }
  if (!status) HB_FAIL("hb_gemm_stream_fused: no status word");
  int kslice, ksplit, n_blocks;
  long per_token;
  hb_gemm_stream_plan(N, K, &kslice, &ksplit, &per_token, &n_blocks);
  const long need = (long)ksplit * n_blocks * FS_ROWS * FS_NT;
  if (!ws || ws_floats < need) HB_FAIL("hb_gemm_stream_fused: workspace of %ld floats, %ld needed", ws_floats, need);
  if (!counters || n_counters < n_blocks) HB_FAIL("hb_gemm_stream_fused: %d counters, %d needed", n_counters, n_blocks);
  CUtensorMap mw;
  if (hb_make_tensor_map_bf16(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, FS_ROWS)) return -1;
  FusedArgs a;
  a.x = x; a.ldx = ldx; a.rows = rows; a.norm_w = norm_w; a.norm_w_bf16 = norm_w_dt == HB_BF16; a.eps = eps;
  a.mode = mode; a.out = (__nv_bfloat16*)out; a.ldo = ldo; a.pos = pos; a.slot_map = slot_map; a.table = (const float2*)table;
  a.kc = (__nv_bfloat16*)kc; a.vc = (__nv_bfloat16*)vc; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.page_size = page_size;
  const int kb_max = (kslice + FS_BK - 1) / FS_BK;
  const int stages = kb_max <= 4 ? 4 : 3;   // keeps three CTAs on an SM when the slice's activations take more room
  const size_t smem = (size_t)stages * FS_W_BYTES + (size_t)kb_max * FS_X_TILE + 256 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_fused: %s", cudaGetErrorString(e));
    configured = true;
  }
  cudaError_t e = hb_launch(gemm_stream_fused_kernel, dim3(n_blocks, ksplit), 192, smem, s, mw, a, M, N, K, kslice, stages,
                            ws, counters, status);
  if (e != cudaSuccess) HB_FAIL("hb_gemm_stream_fused: %s", cudaGetErrorString(e));
  HB_CHECK_LAUNCH("hb_gemm_stream_fused");
  return 0;
}
