// The bandwidth-bound matrix product of decode steps: C[M,N] = A[M,K] W[N,K]^T for M <= 64
// rows. Every weight is read from HBM exactly once, straight from global memory into the
// A-fragments of warp MMAs (m16n8k16: 16 weight rows x 8 tokens), 16 bytes per load; the few
// activation rows sit in shared memory and are reused by all eight warps of the CTA. Replaces
// gemv_kernel and gemm_skinny_kernel of the reference (src/kernels.cuh:164, 911), from which
// the idea of permuting k inside a fragment is taken: a lane's 8 consecutive weights of one
// row feed two MMAs, and the activation fragment uses the same assignment of k to slots.
//
// A CTA owns 128 output columns (8 warps x 16 weight rows) and one slice of K. The number of
// slices is a function of (N, K) only, never of M or the batch, so a token's arithmetic is the
// same whatever runs beside it. Slices leave fp32 partial sums in a workspace; the CTA that
// finishes a column block last adds them in slice order 0, 1, 2, ... (so the result does not
// depend on which CTA came last), applies the epilogue and zeroes the block's counter again.
// Epilogues as in gemm_tc.cu: fp32 store, bf16 store, add into fp32, SwiGLU over gate/up
// columns interleaved by 16.
#include "tc_common.cuh"

enum { SK_F32 = 0, SK_BF16 = 1, SK_ADD_F32 = 2, SK_SWIGLU_BF16 = 3 };

constexpr int SK_ROWS = 128;   // weight rows (output columns) per CTA
constexpr int SK_XC = 512;     // activation chunk along K held in shared memory
constexpr int SK_XS = SK_XC * 2 + 64;  // bytes between activation rows: 64 bytes of padding keep 16-byte reads conflict-free

template <int MT>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const __nv_bfloat16* __restrict__ A, long lda,
                                                          const __nv_bfloat16* __restrict__ W, long ldw, void* C,
                                                          long ldc, int M, int N, int K, int kslice, float* ws,
                                                          int* counters, int epi) {
  constexpr int MP = MT * 8;
  extern __shared__ __align__(16) uint8_t xs[];  // [MP][SK_XS]
  __shared__ int is_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nb = blockIdx.x, sp = blockIdx.y, ksplit = gridDim.y;
  const int NP = gridDim.x * SK_ROWS;
  const int n0 = nb * SK_ROWS + warp * 16;
  const __nv_bfloat16* w0 = W + (size_t)min(n0 + g, N - 1) * ldw;
  const __nv_bfloat16* w1 = W + (size_t)min(n0 + g + 8, N - 1) * ldw;
  const int k_begin = sp * kslice, k_end = min(K, k_begin + kslice);
  float d[MT][4];
#pragma unroll
  for (int j = 0; j < MT; j++) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;

  for (int kc = k_begin; kc < k_end; kc += SK_XC) {
    const int clen = min(SK_XC, k_end - kc);
    __syncthreads();
    for (int i = tid; i < MP * (SK_XC / 8); i += 256) {
      const int m = i / (SK_XC / 8), c = i - m * (SK_XC / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < M && c * 8 < clen) v = *(const uint4*)(A + (size_t)m * lda + kc + c * 8);
      *(uint4*)(xs + m * SK_XS + c * 16) = v;
    }
    __syncthreads();
    for (int kk = 0; kk < clen; kk += 128) {
      uint4 wa[4], wb[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int k = kk + u * 32 + t * 8;
        if (k < clen) {
          wa[u] = hb_ldg_stream(w0 + kc + k);
          wb[u] = hb_ldg_stream(w1 + kc + k);
        } else {
          wa[u] = wb[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int k = kk + u * 32 + t * 8;
#pragma unroll
        for (int j = 0; j < MT; j++) {
          const uint4 xv = *(const uint4*)(xs + (8 * j + g) * SK_XS + k * 2);
          const uint32_t a0[4] = {wa[u].x, wb[u].x, wa[u].y, wb[u].y}, b0[2] = {xv.x, xv.y};
          hb_mma_16816(d[j], a0, b0);
          const uint32_t a1[4] = {wa[u].z, wb[u].z, wa[u].w, wb[u].w}, b1[2] = {xv.z, xv.w};
          hb_mma_16816(d[j], a1, b1);
        }
      }
    }
  }

  // partial sums of this slice: ws[slice][column][token]
  float* base = ws + ((size_t)sp * NP + n0) * MP;
#pragma unroll
  for (int j = 0; j < MT; j++) {
    *(float2*)(base + (size_t)g * MP + 8 * j + 2 * t) = make_float2(d[j][0], d[j][1]);
    *(float2*)(base + (size_t)(g + 8) * MP + 8 * j + 2 * t) = make_float2(d[j][2], d[j][3]);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(&counters[nb], 1) == ksplit - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();

  const float* col0 = ws + (size_t)nb * SK_ROWS * MP;
  const size_t slice_stride = (size_t)NP * MP;
  if (epi == SK_SWIGLU_BF16) {
    __nv_bfloat16* out = (__nv_bfloat16*)C;
    for (int i = tid; i < (SK_ROWS / 2) * M; i += 256) {
      const int m = i / (SK_ROWS / 2), p = i - m * (SK_ROWS / 2);
      const int nl = (p >> 4) * 32 + (p & 15), n = nb * SK_ROWS + nl;
      if (n + 16 >= N) continue;
      float gsum = 0.f, usum = 0.f;
      for (int s = 0; s < ksplit; s++) {
        gsum += __ldcg(col0 + s * slice_stride + (size_t)nl * MP + m);
        usum += __ldcg(col0 + s * slice_stride + (size_t)(nl + 16) * MP + m);
      }
      out[(size_t)m * ldc + (n >> 5) * 16 + (n & 15)] = __float2bfloat16_rn(gsum / (1.f + __expf(-gsum)) * usum);
    }
  } else {
    for (int i = tid; i < SK_ROWS * M; i += 256) {
      const int m = i / SK_ROWS, nl = i - m * SK_ROWS, n = nb * SK_ROWS + nl;
      if (n >= N) continue;
      float acc = 0.f;
      for (int s = 0; s < ksplit; s++) acc += __ldcg(col0 + s * slice_stride + (size_t)nl * MP + m);
      if (epi == SK_BF16) ((__nv_bfloat16*)C)[(size_t)m * ldc + n] = __float2bfloat16_rn(acc);
      else if (epi == SK_ADD_F32) ((float*)C)[(size_t)m * ldc + n] += acc;
      else ((float*)C)[(size_t)m * ldc + n] = acc;
    }
  }
  if (tid == 0) counters[nb] = 0;
}

// The split of K for an [N, K] weight: a function of the weight's shape alone.
static void skinny_plan(int N, int K, int sms, int* kslice, int* ksplit) {
  const int n_blocks = (N + SK_ROWS - 1) / SK_ROWS;
  int want = (3 * sms + n_blocks - 1) / n_blocks;          // about three CTAs per SM over the whole grid
  const int max_split = (K + 255) / 256;                    // a slice is at least 256 deep
  if (want > max_split) want = max_split;
  if (want < 1) want = 1;
  int ks = (K + want - 1) / want;
  ks = (ks + 127) / 128 * 128;                              // whole 128-element steps
  *kslice = ks;
  *ksplit = (K + ks - 1) / ks;
}

HB_EXPORT int hb_gemm_skinny_plan(int N, int K, int* kslice, int* ksplit, long* ws_floats_per_token_row, int* n_blocks) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  skinny_plan(N, K, sms, kslice, ksplit);
  *n_blocks = (N + SK_ROWS - 1) / SK_ROWS;
  *ws_floats_per_token_row = (long)(*ksplit) * (*n_blocks) * SK_ROWS;
  return 0;
}

// C per `epi` (0 fp32, 1 bf16, 2 fp32 +=, 3 bf16 SwiGLU [M, N/2]). ws: at least
// ksplit * n_blocks * 128 * roundup(M, 8) floats; counters: n_blocks ints, all zero (left zero).
// Calls that share ws/counters must not overlap on the device.
HB_EXPORT int hb_gemm_skinny(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int N, int K,
                             int epi, float* ws, long ws_floats, int* counters, int n_counters, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) HB_FAIL("hb_gemm_skinny: M = %d is beyond 64 rows", M);
  if (K <= 0 || (K & 7) || (lda & 7) || (ldw & 7)) HB_FAIL("hb_gemm_skinny: K = %d and the row strides must be multiples of 8", K);
  if (((uintptr_t)A & 15) || ((uintptr_t)W & 15)) HB_FAIL("hb_gemm_skinny: operands must be 16-byte aligned");
  if (epi == SK_SWIGLU_BF16 && (N & 31)) HB_FAIL("hb_gemm_skinny: SwiGLU needs N = %d to be a multiple of 32", N);
  if (epi < 0 || epi > 3) HB_FAIL("hb_gemm_skinny: unknown epilogue %d", epi);
  int kslice, ksplit, n_blocks;
  long per_row;
  hb_gemm_skinny_plan(N, K, &kslice, &ksplit, &per_row, &n_blocks);
  const int MT = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
  if (ws_floats < per_row * MT * 8) HB_FAIL("hb_gemm_skinny: workspace of %ld floats, %ld needed", ws_floats, per_row * MT * 8);
  if (n_counters < n_blocks) HB_FAIL("hb_gemm_skinny: %d counters, %d needed", n_counters, n_blocks);
  dim3 grid(n_blocks, ksplit);
  const __nv_bfloat16 *a = (const __nv_bfloat16*)A, *w = (const __nv_bfloat16*)W;
  const size_t smem = (size_t)MT * 8 * SK_XS;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * SK_XS);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_skinny: %s", cudaGetErrorString(e));
    configured = true;
  }
  switch (MT) {
    case 1: gemm_skinny_kernel<1><<<grid, 256, smem, s>>>(a, lda, w, ldw, C, ldc, M, N, K, kslice, ws, counters, epi); break;
    case 2: gemm_skinny_kernel<2><<<grid, 256, smem, s>>>(a, lda, w, ldw, C, ldc, M, N, K, kslice, ws, counters, epi); break;
    case 4: gemm_skinny_kernel<4><<<grid, 256, smem, s>>>(a, lda, w, ldw, C, ldc, M, N, K, kslice, ws, counters, epi); break;
    default: gemm_skinny_kernel<8><<<grid, 256, smem, s>>>(a, lda, w, ldw, C, ldc, M, N, K, kslice, ws, counters, epi); break;
  }
  HB_CHECK_LAUNCH("hb_gemm_skinny");
  return 0;
}
