// The plain kernels: every operation of the model in true 32-bit arithmetic (FFMA, expf, no
// tensor cores, no reduced-precision matrix mode), templated on the element types so that the
// same code also serves bfloat16 storage where no faster kernel applies. Sizes are runtime
// arguments; nothing here knows a model.
//
// What each replaces in the reference (src/kernels.cuh): embed_kernel 1877, rmsnorm_kernel 110,
// gemv_kernel 164 / gemm_mma_kernel 585 (as one plain tiled product), silu_mul 100,
// rope_cache_kernel 1126 (here over pages), flash_prefill_mma_kernel 1335 and
// decode_attn_mma_kernel 1681 (here one split-key kernel for any row), argmax_kernel 1925.
#include "common.cuh"

#include <stdarg.h>

static thread_local char g_err[512];
void hb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}
HB_EXPORT const char* hb_last_error() { return g_err; }
HB_EXPORT int hb_core_abi_version() { return 1; }
int g_hb_pdl = 1;
HB_EXPORT void hb_set_pdl(int on) { g_hb_pdl = on; }

// ---------------------------------------------------------------------------------------
// Embedding: out[i, :] = table[tok[i], :] into the 32-bit residual stream.
// ---------------------------------------------------------------------------------------
template <typename TE>
__global__ void embed_kernel(const TE* __restrict__ table, const int* __restrict__ tok, float* __restrict__ out, int H) {
  hb_pdl_launch();
  hb_pdl_wait();
  const TE* src = table + (size_t)tok[blockIdx.x] * H;
  float* dst = out + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = hb_to_float(src[i]);
}

HB_EXPORT int hb_embed(const void* table, int table_dt, const int* tok, float* out, int T, int H, cudaStream_t s) {
  if (T <= 0) return 0;
  HB_DISPATCH_1(table_dt, "hb_embed", (hb_launch(embed_kernel<TA>, T, 256, 0, s, (const TA*)table, tok, out, H)));
  HB_CHECK_LAUNCH("hb_embed");
  return 0;
}

// ---------------------------------------------------------------------------------------
// RMSNorm: y = w * (x * rsqrt(mean(x^2) + eps)); x is the 32-bit residual stream, the sum of
// squares, the mean and the scaling are 32-bit, the result is rounded once. `rows` (optional)
// picks the input row of each output row.
// ---------------------------------------------------------------------------------------
template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ y,
                               const int* __restrict__ rows, int H, float eps) {
  __shared__ float sh[32];
  const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* xr = x + r * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  const float inv = rsqrtf(hb_block_sum(ss, sh) / (float)H + eps);
  TO* yr = y + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = hb_from_float<TO>(hb_to_float(w[i]) * (xr[i] * inv));
}

// The same with 16-byte accesses and the row held in registers between the two passes
// (H a multiple of 4, at most 256 * 4 * NV elements). The sum runs over the same per-thread
// partial sums whatever M is.
template <typename TW, typename TO, int NV>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                                          TO* __restrict__ y, const int* __restrict__ rows, int H,
                                                          float eps) {
  __shared__ float sh[32];
  hb_pdl_launch();
  hb_pdl_wait();
  const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* xr = x + r * H;
  const int nvec = H >> 2;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int c = threadIdx.x + i * 256;
    v[i] = c < nvec ? hb_load4(xr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  const float inv = rsqrtf(hb_block_sum(ss, sh) / (float)H + eps);
  TO* yr = y + (size_t)blockIdx.x * H;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      const float4 ww = hb_load4(w + 4 * c);
      hb_store4(yr + 4 * c, make_float4(ww.x * (v[i].x * inv), ww.y * (v[i].y * inv), ww.z * (v[i].z * inv),
                                        ww.w * (v[i].w * inv)));
    }
  }
}

HB_EXPORT int hb_rmsnorm(const float* x, const void* w, int w_dt, void* y, int y_dt, const int* rows, int M, int H,
                         float eps, cudaStream_t s) {
  if (M <= 0) return 0;
  const bool aligned = !(((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15);
  if ((H & 3) == 0 && H <= 8192 && aligned) {
    if (H <= 2048) {
      HB_DISPATCH_2(w_dt, y_dt, "hb_rmsnorm",
                    (hb_launch(rmsnorm_vec_kernel<TA, TB, 2>, M, 256, 0, s, x, (const TA*)w, (TB*)y, rows, H, eps)));
    } else {
      HB_DISPATCH_2(w_dt, y_dt, "hb_rmsnorm",
                    (hb_launch(rmsnorm_vec_kernel<TA, TB, 8>, M, 256, 0, s, x, (const TA*)w, (TB*)y, rows, H, eps)));
    }
    HB_CHECK_LAUNCH("hb_rmsnorm");
    return 0;
  }
  HB_DISPATCH_2(w_dt, y_dt, "hb_rmsnorm",
                (rmsnorm_kernel<TA, TB><<<M, 256, 0, s>>>(x, (const TA*)w, (TB*)y, rows, H, eps)));
  HB_CHECK_LAUNCH("hb_rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Plain matrix product C[M,N] = A[M,K] W[N,K]^T, W row-major with K contiguous as the
// reference stores weights (src/api.cu:81-83). 64x64 tile, 16 deep, 4x4 outputs per thread,
// one FFMA chain per output running k = 0..K-1 in order: an output's value does not depend on
// M, on the tile it lies in, or on anything else in the batch.
// EPI 0: C = acc;  EPI 1: C += acc (32-bit C: the residual stream).
// ---------------------------------------------------------------------------------------
template <typename TA, typename TW, typename TC, int EPI>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, long lda, const TW* __restrict__ W,
                                                        long ldw, TC* __restrict__ C, long ldc, int M, int N, int K) {
  __shared__ float As[16][68], Ws[16][68];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m_blk = blockIdx.y * 64, n_blk = blockIdx.x * 64;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (m_blk + lr < M && k < K) ? hb_to_float(A[(size_t)(m_blk + lr) * lda + k]) : 0.f;
      Ws[lk + i][lr] = (n_blk + lr < N && k < K) ? hb_to_float(W[(size_t)(n_blk + lr) * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m_blk + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n_blk + tx * 4 + j;
      if (n >= N) continue;
      TC* c = C + (size_t)m * ldc + n;
      if (EPI == 1) *c = hb_from_float<TC>(hb_to_float(*c) + acc[i][j]);
      else *c = hb_from_float<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW>
static int gemm_simt_launch(const void* A, long lda, const void* W, long ldw, void* C, int c_dt, long ldc, int M, int N,
                            int K, int epi, cudaStream_t s) {
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (epi == 1) {
    if (c_dt != HB_F32) HB_FAIL("hb_gemm_simt: accumulating into C needs a 32-bit C");
    gemm_simt_kernel<TA, TW, float, 1><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, ldw, (float*)C, ldc, M, N, K);
  } else if (c_dt == HB_F32) {
    gemm_simt_kernel<TA, TW, float, 0><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, ldw, (float*)C, ldc, M, N, K);
  } else if (c_dt == HB_BF16) {
    gemm_simt_kernel<TA, TW, __nv_bfloat16, 0><<<grid, 256, 0, s>>>((const TA*)A, lda, (const TW*)W, ldw,
                                                                    (__nv_bfloat16*)C, ldc, M, N, K);
  } else {
    HB_FAIL("hb_gemm_simt: unknown C dtype code %d", c_dt);
  }
  return 0;
}

HB_EXPORT int hb_gemm_simt(const void* A, int a_dt, long lda, const void* W, int w_dt, long ldw, void* C, int c_dt,
                           long ldc, int M, int N, int K, int epi, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) HB_FAIL("hb_gemm_simt: K must be positive");
  if (epi != 0 && epi != 1) HB_FAIL("hb_gemm_simt: unknown epilogue %d", epi);
  if ((M + 63) / 64 > 65535) HB_FAIL("hb_gemm_simt: M = %d is beyond the grid limit", M);
  int r = -1;
  HB_DISPATCH_2(a_dt, w_dt, "hb_gemm_simt", (r = gemm_simt_launch<TA, TB>(A, lda, W, ldw, C, c_dt, ldc, M, N, K, epi, s)));
  if (r) return r;
  HB_CHECK_LAUNCH("hb_gemm_simt");
  return 0;
}

// ---------------------------------------------------------------------------------------
// SwiGLU over a gate/up matrix whose columns are interleaved in groups of `grp`
// (grp gate columns, grp up columns, ...): act[m, i] = silu(g) * u, silu(g) = g / (1 + e^-g).
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gu, long ld_gu, TO* __restrict__ act, long ld_act, int I, int grp) {
  const TI* row = gu + (size_t)blockIdx.y * ld_gu;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= I) return;
  const int b = i / grp, j = i - b * grp;
  const float g = hb_to_float(row[(size_t)b * 2 * grp + j]), u = hb_to_float(row[(size_t)b * 2 * grp + grp + j]);
  act[(size_t)blockIdx.y * ld_act + i] = hb_from_float<TO>(g / (1.f + expf(-g)) * u);
}

HB_EXPORT int hb_swiglu(const void* gu, int gu_dt, long ld_gu, void* act, int act_dt, long ld_act, int M, int I, int grp,
                        cudaStream_t s) {
  if (M <= 0) return 0;
  if (grp <= 0 || I % grp) HB_FAIL("hb_swiglu: width %d is not a multiple of the interleave group %d", I, grp);
  if (M > 65535) HB_FAIL("hb_swiglu: M = %d is beyond the grid limit", M);
  dim3 grid((I + 255) / 256, M);
  HB_DISPATCH_2(gu_dt, act_dt, "hb_swiglu",
                (swiglu_kernel<TA, TB><<<grid, 256, 0, s>>>((const TA*)gu, ld_gu, (TB*)act, ld_act, I, grp)));
  HB_CHECK_LAUNCH("hb_swiglu");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Rotary table: (cos, sin) of angle = float(p) * inv_freq[i], the angle a 32-bit product, the
// functions evaluated in double (src/api.cu:1430-1441), kept in 32-bit.
// ---------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float2* __restrict__ table, int n_pos, int half) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_pos * half) return;
  const int p = idx / half, i = idx - p * half;
  const float angle = __fmul_rn((float)p, inv_freq[i]);
  double sn, cs;
  sincos((double)angle, &sn, &cs);
  table[idx] = make_float2((float)cs, (float)sn);
}

HB_EXPORT int hb_rope_table(const float* inv_freq, void* table, int n_pos, int half, cudaStream_t s) {
  if (n_pos <= 0 || half <= 0) return 0;
  const long n = (long)n_pos * half;
  rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(inv_freq, (float2*)table, n_pos, half);
  HB_CHECK_LAUNCH("hb_rope_table");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Rotary position encoding of q and k (half-split pairs (d, d + rot/2) over the first `rot`
// dimensions of each head, the rest passed through), and the cache write: rotated k and raw v
// go to the page slot of their token. Cache layout [page][kv head][page_size][D].
// A negative slot writes nothing (a layer that reads another layer's cache).
// ---------------------------------------------------------------------------------------
template <typename TI, typename TQ, typename TC>
__global__ void rope_kv_kernel(const TI* __restrict__ qkv, long ld, const int* __restrict__ pos,
                               const int* __restrict__ slot_map, const float2* __restrict__ table, TQ* __restrict__ q_out,
                               TC* __restrict__ kc, TC* __restrict__ vc, int Hq, int Hkv, int D, int rot, int page_size) {
  const int t = blockIdx.x, half = rot >> 1;
  const TI* base = qkv + (size_t)t * ld;
  const float2* cs = table + (size_t)pos[t] * half;
  const int slot = slot_map ? slot_map[t] : -1;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  for (int i = threadIdx.x; i < (Hq + Hkv) * D; i += blockDim.x) {
    const int hh = i / D, d = i - hh * D;
    if (hh >= Hq && slot < 0) break;
    float y;
    if (d < rot) {
      const int j = d < half ? d : d - half;
      const float x1 = hb_to_float(base[hh * D + j]), x2 = hb_to_float(base[hh * D + j + half]);
      const float2 c = cs[j];
      y = d < half ? __fsub_rn(__fmul_rn(x1, c.x), __fmul_rn(x2, c.y)) : __fadd_rn(__fmul_rn(x2, c.x), __fmul_rn(x1, c.y));
    } else {
      y = hb_to_float(base[i]);
    }
    if (hh < Hq) q_out[(size_t)t * Hq * D + i] = hb_from_float<TQ>(y);
    else kc[((page * Hkv + (hh - Hq)) * page_size + off) * D + d] = hb_from_float<TC>(y);
  }
  if (slot < 0) return;
  const TI* v = base + (size_t)(Hq + Hkv) * D;
  for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
    const int h = i / D, d = i - h * D;
    vc[((page * Hkv + h) * page_size + off) * D + d] = hb_from_float<TC>(hb_to_float(v[i]));
  }
}

// The same four elements at a time (rotary over the whole head, head_dim a multiple of 8).
template <typename TI, typename TQ, typename TC>
__global__ void __launch_bounds__(256) rope_kv_vec_kernel(const TI* __restrict__ qkv, long ld, const int* __restrict__ pos,
                                                          const int* __restrict__ slot_map, const float2* __restrict__ table,
                                                          TQ* __restrict__ q_out, TC* __restrict__ kc, TC* __restrict__ vc,
                                                          int Hq, int Hkv, int D, int page_size) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.x, half = D >> 1, hv = half >> 2;  // hv: groups of 4 pairs per head
  const TI* base = qkv + (size_t)t * ld;
  const float2* cs = table + (size_t)pos[t] * half;
  const int slot = slot_map ? slot_map[t] : -1;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const int n_rot = (slot >= 0 ? Hq + Hkv : Hq) * hv;
  for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
    const int hh = i / hv, j = (i - hh * hv) * 4;
    const float4 x1 = hb_load4(base + hh * D + j), x2 = hb_load4(base + hh * D + half + j);
    const float4 c01 = *(const float4*)(cs + j), c23 = *(const float4*)(cs + j + 2);  // (cos, sin) pairs
    float4 y1, y2;
    y1.x = __fsub_rn(__fmul_rn(x1.x, c01.x), __fmul_rn(x2.x, c01.y)); y2.x = __fadd_rn(__fmul_rn(x2.x, c01.x), __fmul_rn(x1.x, c01.y));
    y1.y = __fsub_rn(__fmul_rn(x1.y, c01.z), __fmul_rn(x2.y, c01.w)); y2.y = __fadd_rn(__fmul_rn(x2.y, c01.z), __fmul_rn(x1.y, c01.w));
    y1.z = __fsub_rn(__fmul_rn(x1.z, c23.x), __fmul_rn(x2.z, c23.y)); y2.z = __fadd_rn(__fmul_rn(x2.z, c23.x), __fmul_rn(x1.z, c23.y));
    y1.w = __fsub_rn(__fmul_rn(x1.w, c23.z), __fmul_rn(x2.w, c23.w)); y2.w = __fadd_rn(__fmul_rn(x2.w, c23.z), __fmul_rn(x1.w, c23.w));
    if (hh < Hq) {
      TQ* dst = q_out + (size_t)t * Hq * D + hh * D + j;
      hb_store4(dst, y1);
      hb_store4(dst + half, y2);
    } else {
      TC* dst = kc + ((page * Hkv + (hh - Hq)) * page_size + off) * D + j;
      hb_store4(dst, y1);
      hb_store4(dst + half, y2);
    }
  }
  if (slot < 0) return;
  const TI* v = base + (size_t)(Hq + Hkv) * D;
  const int dv = D >> 2;
  for (int i = threadIdx.x; i < Hkv * dv; i += blockDim.x) {
    const int h = i / dv, d = (i - h * dv) * 4;
    hb_store4(vc + ((page * Hkv + h) * page_size + off) * D + d, hb_load4(v + h * D + d));
  }
}

HB_EXPORT int hb_rope_kv(const void* qkv, int qkv_dt, long ld, const int* pos, const int* slot_map, const void* table,
                         void* q_out, int q_dt, void* kc, void* vc, int cache_dt, int T, int Hq, int Hkv, int D, int rot,
                         int page_size, cudaStream_t s) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > D || (rot & 1)) HB_FAIL("hb_rope_kv: rotary width %d must be even and at most head_dim %d", rot, D);
  if (q_dt != cache_dt) HB_FAIL("hb_rope_kv: q and the cache must have the same element type");
  const bool aligned = !(((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)table) & 15);
  if (rot == D && (D & 7) == 0 && (ld & 3) == 0 && aligned) {
    HB_DISPATCH_2(qkv_dt, q_dt, "hb_rope_kv",
                  (hb_launch(rope_kv_vec_kernel<TA, TB, TB>, T, 256, 0, s, (const TA*)qkv, ld, pos, slot_map,
                             (const float2*)table, (TB*)q_out, (TB*)kc, (TB*)vc, Hq, Hkv, D, page_size)));
    HB_CHECK_LAUNCH("hb_rope_kv");
    return 0;
  }
  HB_DISPATCH_2(qkv_dt, q_dt, "hb_rope_kv",
                (rope_kv_kernel<TA, TB, TB><<<T, 256, 0, s>>>((const TA*)qkv, ld, pos, slot_map, (const float2*)table,
                                                              (TB*)q_out, (TB*)kc, (TB*)vc, Hq, Hkv, D, rot, page_size)));
  HB_CHECK_LAUNCH("hb_rope_kv");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Attention of single rows over the paged cache. One block per (key chunk, kv head, row):
// the G query heads of a kv head share one pass over its keys (src/kernels.cuh:1501-1508).
// Row t of request r at position p sees keys max(0, p - window + 1) .. p (window 0: all), the
// causal mask on absolute positions of src/kernels.cuh:1416-1418. Keys are cut into chunks of
// `chunk` ABSOLUTE positions, so how a row's keys are split depends on its position alone,
// never on the batch (the reference picks its split count from the batch size,
// src/api.cu:643-646). Scores, max, sum, exp and the value sums are 32-bit. A row that spans
// one chunk is finished here; otherwise partial (acc, max, sum) go to the workspace and
// attn_merge_kernel combines the chunks in ascending order.
// ---------------------------------------------------------------------------------------
template <typename TQ, typename TC>
__global__ void __launch_bounds__(128) attn_rows_kernel(
    const TQ* __restrict__ q, const TC* __restrict__ kc, const TC* __restrict__ vc, const int* __restrict__ bt,
    int bt_stride, const int* __restrict__ row_req, const int* __restrict__ pos, TQ* __restrict__ out,
    float* __restrict__ part_acc, float* __restrict__ part_ml, int Hq, int Hkv, int D, int page_size, int window,
    float scale, int chunk, int S) {
  extern __shared__ float smem[];
  const int t = blockIdx.z, h = blockIdx.y, s = blockIdx.x, G = Hq / Hkv;
  const int p = pos[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int s_lo = lo / chunk, s_hi = p / chunk;
  if (s < s_lo || s > s_hi) return;
  const int k0 = max(s * chunk, lo), k1 = min((s + 1) * chunk, p + 1), nk = k1 - k0;
  float* qs = smem;               // [G][D]
  float* sc = smem + G * D;       // [G][chunk]
  float* ml = sc + G * chunk;     // [G][2]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const TQ* qrow = q + ((size_t)t * Hq + (size_t)h * G) * D;
  for (int i = tid; i < G * D; i += 128) qs[i] = hb_to_float(qrow[i]) * scale;
  __syncthreads();
  const int* table = bt + (size_t)row_req[t] * bt_stride;
  for (int j = tid; j < nk; j += 128) {
    const int kp = k0 + j;
    const size_t page = table[kp / page_size];
    const TC* kr = kc + ((page * Hkv + h) * page_size + kp % page_size) * D;
    for (int g = 0; g < G; g++) {
      float a = 0.f;
      for (int d = 0; d < D; d++) a = fmaf(qs[g * D + d], hb_to_float(kr[d]), a);
      sc[g * chunk + j] = a;
    }
  }
  __syncthreads();
  for (int g = warp; g < G; g += 4) {
    float m = -INFINITY;
    for (int j = lane; j < nk; j += 32) m = fmaxf(m, sc[g * chunk + j]);
    m = hb_warp_max(m);
    float l = 0.f;
    for (int j = lane; j < nk; j += 32) {
      const float e = expf(sc[g * chunk + j] - m);
      sc[g * chunk + j] = e;
      l += e;
    }
    l = hb_warp_sum(l);
    if (lane == 0) { ml[2 * g] = m; ml[2 * g + 1] = l; }
  }
  __syncthreads();
  const bool whole = s_lo == s_hi;
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i - g * D;
    float a = 0.f;
    for (int j = 0; j < nk; j++) {
      const int kp = k0 + j;
      const size_t page = table[kp / page_size];
      a = fmaf(sc[g * chunk + j], hb_to_float(vc[((page * Hkv + h) * page_size + kp % page_size) * D + d]), a);
    }
    const size_t head = (size_t)t * Hq + (size_t)h * G + g;
    if (whole) out[head * D + d] = hb_from_float<TQ>(a / ml[2 * g + 1]);
    else part_acc[(head * S + s) * D + d] = a;
  }
  if (!whole && tid < G) {
    const size_t head = (size_t)t * Hq + (size_t)h * G + tid;
    part_ml[(head * S + s) * 2] = ml[2 * tid];
    part_ml[(head * S + s) * 2 + 1] = ml[2 * tid + 1];
  }
}

template <typename TQ>
__global__ void attn_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                  const int* __restrict__ pos, TQ* __restrict__ out, int Hq, int D, int window, int chunk,
                                  int S, const int* __restrict__ row_req, const int* __restrict__ q_len, int row_limit) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.y, hq = blockIdx.x;
  if (q_len && q_len[row_req[t]] >= row_limit) return;
  const int p = pos[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int s_lo = lo / chunk, s_hi = p / chunk;
  if (s_lo == s_hi) return;
  const size_t head = (size_t)t * Hq + hq;
  float m = -INFINITY;
  for (int s = s_lo; s <= s_hi; s++) m = fmaxf(m, part_ml[(head * S + s) * 2]);
  float l = 0.f;
  for (int s = s_lo; s <= s_hi; s++) l += part_ml[(head * S + s) * 2 + 1] * expf(part_ml[(head * S + s) * 2] - m);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s = s_lo; s <= s_hi; s++) a += part_acc[(head * S + s) * D + d] * expf(part_ml[(head * S + s) * 2] - m);
    out[head * D + d] = hb_from_float<TQ>(a / l);
  }
}

// Workspace (floats) that hb_attn_rows needs for T rows whose largest position is max_pos.
HB_EXPORT long hb_attn_rows_workspace(int T, int Hq, int D, int max_pos, int chunk) {
  const long S = max_pos / chunk + 1;
  return S <= 1 ? 0 : (long)T * Hq * S * (D + 2);
}

HB_EXPORT int hb_attn_rows(const void* q, int q_dt, const void* kc, const void* vc, int cache_dt, const int* bt,
                           int bt_stride, const int* row_req, const int* pos, void* out, float* workspace, int T, int Hq,
                           int Hkv, int D, int page_size, int window, float scale, int chunk, int max_pos,
                           cudaStream_t s) {
  if (T <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv) HB_FAIL("hb_attn_rows: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
  if (chunk <= 0 || chunk % 32) HB_FAIL("hb_attn_rows: chunk %d must be a positive multiple of 32", chunk);
  if (q_dt != cache_dt) HB_FAIL("hb_attn_rows: q and the cache must have the same element type");
  const int G = Hq / Hkv, S = max_pos / chunk + 1;
  const size_t smem = ((size_t)G * D + (size_t)G * chunk + 2 * G) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_attn_rows: group %d x head_dim %d x chunk %d needs %zu bytes of shared memory", G, D, chunk, smem);
  if (T > 65535 || Hkv > 65535) HB_FAIL("hb_attn_rows: %d rows / %d kv heads are beyond the grid limit", T, Hkv);
  if (S > 1 && !workspace) HB_FAIL("hb_attn_rows: rows that span %d chunks need a workspace", S);
  float* part_acc = workspace;
  float* part_ml = workspace ? workspace + (size_t)T * Hq * S * D : nullptr;
  dim3 grid(S, Hkv, T);
  HB_DISPATCH_1(q_dt, "hb_attn_rows", {
    auto kern = attn_rows_kernel<TA, TA>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) HB_FAIL("hb_attn_rows: %s", cudaGetErrorString(e));
    }
    kern<<<grid, 128, smem, s>>>((const TA*)q, (const TA*)kc, (const TA*)vc, bt, bt_stride, row_req, pos, (TA*)out,
                                 part_acc, part_ml, Hq, Hkv, D, page_size, window, scale, chunk, S);
    if (S > 1) {
      dim3 mg(Hq, T);
      hb_launch(attn_merge_kernel<TA>, mg, 64, 0, s, (const float*)part_acc, (const float*)part_ml, pos, (TA*)out, Hq, D, window,
                chunk, S, (const int*)nullptr, (const int*)nullptr, 0);
    }
  });
  HB_CHECK_LAUNCH("hb_attn_rows");
  return 0;
}

// Finishes rows that span several key chunks from partials laid out as hb_attn_rows leaves them
// (for attention kernels of other libraries that write the same partials).
HB_EXPORT int hb_attn_merge(float* workspace, const int* pos, void* out, int out_dt, int T, int Hq, int D, int window,
                            int chunk, int max_pos, const int* row_req, const int* q_len, int row_limit, cudaStream_t s) {
  const int S = max_pos / chunk + 1;
  if (T <= 0 || S <= 1) return 0;
  if (!workspace) HB_FAIL("hb_attn_merge: no workspace");
  float* part_acc = workspace;
  float* part_ml = workspace + (size_t)T * Hq * S * D;
  dim3 mg(Hq, T);
  HB_DISPATCH_1(out_dt, "hb_attn_merge",
                (hb_launch(attn_merge_kernel<TA>, mg, 64, 0, s, (const float*)part_acc, (const float*)part_ml, pos, (TA*)out, Hq,
                           D, window, chunk, S, row_req, q_len, row_limit)));
  HB_CHECK_LAUNCH("hb_attn_merge");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Sampling from 32-bit logits. temperature 0: the largest value, the lowest index on ties, NaN
// above every number, index 0 when all are -inf (the reference's rules, src/kernels.cuh:1883-1913). temperature > 0: arg max of logit / temperature + Gumbel noise,
// the noise a counter-based hash of (seed, position, index), so a draw does not depend on what
// else is in the batch.
// ---------------------------------------------------------------------------------------
// A candidate (value, index) as one 64-bit key whose unsigned order is the rule above, so that the
// choice over any split of a row is a plain maximum: the high word is the value's bits made
// monotone (negative floats inverted, the others with the sign bit set; -0 counts as +0; every NaN
// becomes the largest word), the low word is ~index, so of equal values the lower index wins. Key 0
// stands for "no candidate" and lies below every real key.
__device__ __forceinline__ unsigned long long pick_key(float v, int i) {
  uint32_t hi;
  if (v != v) {
    hi = 0xFFFFFFFFu;
  } else {
    const uint32_t b = __float_as_uint(v + 0.0f);
    hi = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
  return ((unsigned long long)hi << 32) | (uint32_t)~(uint32_t)i;
}
__device__ __forceinline__ int pick_index(unsigned long long key) { return key ? (int)~(uint32_t)key : 0; }
// The largest key of the block in thread 0 (`sh`: one slot per warp).
__device__ __forceinline__ unsigned long long pick_block_max(unsigned long long key, unsigned long long* sh) {
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
    key = other > key ? other : key;
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) sh[w] = key;
  __syncthreads();
  if (w == 0) {
    key = lane < nw ? sh[lane] : 0ull;
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
      key = other > key ? other : key;
    }
  }
  return key;
}
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float sample_uniform(uint32_t seed, uint32_t position, uint32_t index) {
  uint32_t h = mix32(seed ^ 0x9E3779B9u);
  h = mix32(h ^ (position * 0x85EBCA6Bu));
  h = mix32(h ^ (index * 0xC2B2AE35u));
  return ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

// Entries [s * slice, (s + 1) * slice) of row blockIdx.y. One slice (best null): its best index goes to out[row]. Several:
// the slice's best key meets the others' in best[row] by an atomic maximum (the order of the arrivals does not matter: the
// keys are totally ordered), and the block that arrives last writes the row's index and leaves best[row] and count[row]
// zero for the next call: no second kernel.
__global__ void __launch_bounds__(1024) sample_slice_kernel(const float* __restrict__ logits, long ld, int V, int slice,
                                                            const float* __restrict__ temperature,
                                                            const uint32_t* __restrict__ seed, const int* __restrict__ position,
                                                            unsigned long long* __restrict__ best, int* __restrict__ count,
                                                            int* __restrict__ out) {
  __shared__ unsigned long long sh[32];
  hb_pdl_launch();
  hb_pdl_wait();
  const int row = blockIdx.y, s = blockIdx.x;
  const float* l = logits + (size_t)row * ld;
  const float temp = temperature ? temperature[row] : 0.f;
  const uint32_t sd = seed ? seed[row] : 0u, ps = position ? (uint32_t)position[row] : 0u;
  const int i0 = s * slice, i1 = min(V, i0 + slice);
  unsigned long long key = 0ull;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
    float v = l[i];
    if (temp > 0.f) v = v / temp - logf(-logf(sample_uniform(sd, ps, (uint32_t)i)));
    const unsigned long long k = pick_key(v, i);
    key = k > key ? k : key;
  }
  key = pick_block_max(key, sh);
  if (threadIdx.x == 0) {
    if (!best) {
      out[row] = pick_index(key);
    } else {
      atomicMax(&best[row], key);
      __threadfence();
      if (atomicAdd(&count[row], 1) == (int)gridDim.x - 1) {     // every slice of the row has arrived
        __threadfence();
        out[row] = pick_index(atomicExch(&best[row], 0ull));
        count[row] = 0;
      }
    }
  }
}

// Slices per row that hb_sample uses for a vocabulary of V.
HB_EXPORT int hb_sample_slices(int V) { return V <= 4096 ? 1 : (V + 2047) / 2048 > 128 ? 128 : (V + 2047) / 2048; }

// workspace (needed when hb_sample_slices(V) > 1): 12 bytes a row, 8-byte aligned, all zero; the call leaves it zero.
// Calls that share it must not overlap.
HB_EXPORT int hb_sample(const float* logits, long ld, int rows, int V, const float* temperature, const uint32_t* seed,
                        const int* position, int* out, void* workspace, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (V <= 0) HB_FAIL("hb_sample: empty vocabulary");
  const int n = hb_sample_slices(V);
  if (rows > 65535) HB_FAIL("hb_sample: %d rows are beyond the grid limit", rows);
  if (((uintptr_t)workspace & 7) != 0) HB_FAIL("hb_sample: the workspace must be 8-byte aligned");
  if (n == 1 || !workspace) {
    hb_launch(sample_slice_kernel, dim3(1, rows), 1024, 0, s, logits, ld, V, V, temperature, seed, position,
              (unsigned long long*)nullptr, (int*)nullptr, out);
  } else {
    unsigned long long* best = (unsigned long long*)workspace;     // rows keys, then rows counters
    const int slice = (V + n - 1) / n;
    hb_launch(sample_slice_kernel, dim3(n, rows), 256, 0, s, logits, ld, V, slice, temperature, seed, position, best,
              (int*)(best + rows), out);
  }
  HB_CHECK_LAUNCH("hb_sample");
  return 0;
}

// ---------------------------------------------------------------------------------------
// tokens[i] = src[map[i]] where map[i] >= 0: rows of a step whose token was sampled on the
// device by the step before and has not been to the host.
// ---------------------------------------------------------------------------------------
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src, const int* __restrict__ map, int n) {
  hb_pdl_launch();
  hb_pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && map[i] >= 0) tokens[i] = src[map[i]];
}

HB_EXPORT int hb_feed_tokens(int* tokens, const int* src, const int* map, int n, cudaStream_t s) {
  if (n <= 0) return 0;
  hb_launch(feed_tokens_kernel, (n + 127) / 128, 128, 0, s, tokens, src, map, n);
  HB_CHECK_LAUNCH("hb_feed_tokens");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Element-type conversion of a dense array (weights of another storage type, test helpers).
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = hb_from_float<TO>(hb_to_float(in[i]));
}

HB_EXPORT int hb_convert(const void* in, int in_dt, void* out, int out_dt, long n, cudaStream_t s) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256);
  HB_DISPATCH_2(in_dt, out_dt, "hb_convert", (convert_kernel<TA, TB><<<blocks, 256, 0, s>>>((const TA*)in, (TB*)out, (size_t)n)));
  HB_CHECK_LAUNCH("hb_convert");
  return 0;
}
