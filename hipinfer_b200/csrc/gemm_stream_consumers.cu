// Kernels that take the result of a decode-step product as the K slices it was computed in
// (gemm_stream.cu, epilogue ST_SLICES: ws[slice][token][column], fp32) and add the slices
// themselves, in slice order, as the separate reduction would have:
//   add_rmsnorm_slices_kernel: x += sum of slices (the residual stream), y = RMSNorm(x) w
//   rope_kv_slices_kernel:     q/k/v = sum of slices, rotation of q and k, cache write
// A decode step is a chain of small kernels that each wait for the one before; every kernel
// taken out of the chain saves its start-up and the round trip of its result through memory
// (the reference folds the norm and the residual into its matrix-vector kernels for the same
// reason, src/kernels.cuh:164-330).
#include "common.cuh"

HB_TL_DEFINE(consumers)

// The sum over the slices of four consecutive columns, added in slice order. All loads are
// asked for before the first is used (up to 16 slices; the kernels here are short chains of
// round trips to L2, and every round trip saved is most of a microsecond).
constexpr int SL_MAX = 16;
__device__ __forceinline__ float4 slices_sum4(const float* __restrict__ p, int ksplit, long slice_stride) {
  float4 a[SL_MAX];
#pragma unroll
  for (int j = 0; j < SL_MAX; j++)
    if (j < ksplit) a[j] = __ldcg((const float4*)(p + j * slice_stride));
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int j = 0; j < SL_MAX; j++)
    if (j < ksplit) { acc.x += a[j].x; acc.y += a[j].y; acc.z += a[j].z; acc.w += a[j].w; }
  for (int sl = SL_MAX; sl < ksplit; sl++) {
    const float4 v = __ldcg((const float4*)(p + sl * slice_stride));
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  return acc;
}

// One block of 512 threads per row; the row stays in registers between the sum of squares and
// the scaling (H a multiple of 4, at most 512 * 4 * NV). With `rows` (a gather of some rows, as before the
// output head) x itself is left as it is: two entries may name the same row.
template <int NV>
__global__ void __launch_bounds__(512) add_rmsnorm_slices_kernel(float* __restrict__ x, long ldx, const float* __restrict__ ws,
                                                                 int ksplit, long slice_stride, long row_stride,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ y, const int* __restrict__ rows,
                                                                 int H, float eps) {
  __shared__ float sh[32];
  hb_pdl_launch();
  const int tl = rows ? 2 : ksplit <= 8 ? 0 : 1;
  HB_TL_MARK(tl, 0);
  const int nvec = H >> 2;
  float4 ww[NV];
#pragma unroll
  for (int i = 0; i < NV; i++) {   // the norm's weight does not depend on the kernel ahead
    const int c = threadIdx.x + i * 512;
    ww[i] = c < nvec ? hb_load4(w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  hb_pdl_wait();
  HB_TL_MARK(tl, 1);
  const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* xr = x + r * ldx;
  const float* pr = ws + r * row_stride;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int c = threadIdx.x + i * 512;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < nvec) {
      const float4 o = hb_load4(xr + 4 * c), a = slices_sum4(pr + 4 * c, ksplit, slice_stride);
      v[i] = make_float4(o.x + a.x, o.y + a.y, o.z + a.z, o.w + a.w);
      if (!rows) hb_store4(xr + 4 * c, v[i]);
    }
    ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
  }
  HB_TL_MARK(tl, 2);
  const float inv = rsqrtf(hb_block_sum(ss, sh) / (float)H + eps);
  __nv_bfloat16* yr = y + (size_t)blockIdx.x * H;
#pragma unroll
  for (int i = 0; i < NV; i++) {
    const int c = threadIdx.x + i * 512;
    if (c < nvec)
      hb_store4(yr + 4 * c, make_float4(ww[i].x * (v[i].x * inv), ww[i].y * (v[i].y * inv), ww[i].z * (v[i].z * inv),
                                        ww[i].w * (v[i].w * inv)));
  }
  HB_TL_MARK(tl, 3);
}

// x [M, H] fp32 (row stride ldx) += the slices; y [M or n_rows, H] bf16 = RMSNorm of the sum times w.
HB_EXPORT int hb_add_rmsnorm_slices(float* x, long ldx, const float* ws, int ksplit, long slice_stride, long row_stride,
                                    const void* w, void* y, const int* rows, int M, int H, float eps, cudaStream_t s) {
  if (M <= 0) return 0;
  if ((H & 3) || H > 8192) HB_FAIL("hb_add_rmsnorm_slices: width %d must be a multiple of 4 and at most 8192", H);
  if (((uintptr_t)x | (uintptr_t)ws | (uintptr_t)w | (uintptr_t)y) & 15 || (ldx & 3) || (row_stride & 3) || (slice_stride & 3))
    HB_FAIL("hb_add_rmsnorm_slices: pointers and strides must be multiples of 16 bytes");
  if (ksplit < 1) HB_FAIL("hb_add_rmsnorm_slices: %d slices", ksplit);
  const __nv_bfloat16* ww = (const __nv_bfloat16*)w;
  __nv_bfloat16* yy = (__nv_bfloat16*)y;
  if (H <= 2048) hb_launch(add_rmsnorm_slices_kernel<1>, M, 512, 0, s, x, ldx, ws, ksplit, slice_stride, row_stride, ww, yy, rows, H, eps);
  else if (H <= 4096) hb_launch(add_rmsnorm_slices_kernel<2>, M, 512, 0, s, x, ldx, ws, ksplit, slice_stride, row_stride, ww, yy, rows, H, eps);
  else hb_launch(add_rmsnorm_slices_kernel<4>, M, 512, 0, s, x, ldx, ws, ksplit, slice_stride, row_stride, ww, yy, rows, H, eps);
  HB_CHECK_LAUNCH("hb_add_rmsnorm_slices");
  return 0;
}

// The rotation and cache write of rope_kv_vec_kernel (core library) on the sum of the slices:
// row t holds [q (Hq D); k (Hkv D); v (Hkv D)]; the pair (j, j + D/2) of every q and k head is
// turned by the angle of (pos[t], j) from the table of (cos, sin); q goes to q_out, k and v to
// the cache at slot_map[t] (a negative slot or no map: nothing is stored). blockIdx.y shares a
// row's heads among several blocks.
__global__ void __launch_bounds__(256) rope_kv_slices_kernel(const float* __restrict__ ws, int ksplit, long slice_stride,
                                                             long row_stride, const int* __restrict__ pos,
                                                             const int* __restrict__ slot_map,
                                                             const float2* __restrict__ table,
                                                             __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ kc,
                                                             __nv_bfloat16* __restrict__ vc, int Hq, int Hkv, int D,
                                                             int page_size) {
  hb_pdl_launch();
  const int t = blockIdx.x, half = D >> 1, hv = half >> 2;  // hv: groups of 4 pairs per head
  const float2* cs = table + (size_t)pos[t] * half;         // positions and slots are the step's own input
  const int slot = slot_map ? slot_map[t] : -1;
  HB_TL_MARK(3, 0);
  hb_pdl_wait();
  HB_TL_MARK(3, 1);
  const float* base = ws + (size_t)t * row_stride;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const int n_rot = (slot >= 0 ? Hq + Hkv : Hq) * hv, dv = D >> 2;
  const int n_all = n_rot + (slot >= 0 ? Hkv * dv : 0);
  for (int i = blockIdx.y * 256 + threadIdx.x; i < n_all; i += 256 * gridDim.y) {
    if (i < n_rot) {
      const int hh = i / hv, j = (i - hh * hv) * 4;
      const float4 x1 = slices_sum4(base + hh * D + j, ksplit, slice_stride);
      const float4 x2 = slices_sum4(base + hh * D + half + j, ksplit, slice_stride);
      const float4 c01 = *(const float4*)(cs + j), c23 = *(const float4*)(cs + j + 2);  // (cos, sin) pairs
      float4 y1, y2;
      y1.x = __fsub_rn(__fmul_rn(x1.x, c01.x), __fmul_rn(x2.x, c01.y)); y2.x = __fadd_rn(__fmul_rn(x2.x, c01.x), __fmul_rn(x1.x, c01.y));
      y1.y = __fsub_rn(__fmul_rn(x1.y, c01.z), __fmul_rn(x2.y, c01.w)); y2.y = __fadd_rn(__fmul_rn(x2.y, c01.z), __fmul_rn(x1.y, c01.w));
      y1.z = __fsub_rn(__fmul_rn(x1.z, c23.x), __fmul_rn(x2.z, c23.y)); y2.z = __fadd_rn(__fmul_rn(x2.z, c23.x), __fmul_rn(x1.z, c23.y));
      y1.w = __fsub_rn(__fmul_rn(x1.w, c23.z), __fmul_rn(x2.w, c23.w)); y2.w = __fadd_rn(__fmul_rn(x2.w, c23.z), __fmul_rn(x1.w, c23.w));
      __nv_bfloat16* dst = hh < Hq ? q_out + (size_t)t * Hq * D + hh * D + j
                                   : kc + ((page * Hkv + (hh - Hq)) * page_size + off) * D + j;
      hb_store4(dst, y1);
      hb_store4(dst + half, y2);
    } else {
      const int k = i - n_rot, h = k / dv, d = (k - h * dv) * 4;
      hb_store4(vc + ((page * Hkv + h) * page_size + off) * D + d,
                slices_sum4(base + (size_t)(Hq + Hkv) * D + h * D + d, ksplit, slice_stride));
    }
  }
  HB_TL_MARK(3, 3);
}

// Rotary over the whole head only (D a multiple of 8); q_out and the cache are bf16.
HB_EXPORT int hb_rope_kv_slices(const float* ws, int ksplit, long slice_stride, long row_stride, const int* pos,
                                const int* slot_map, const void* table, void* q_out, void* kc, void* vc, int T, int Hq,
                                int Hkv, int D, int page_size, cudaStream_t s) {
  if (T <= 0) return 0;
  if (D & 7) HB_FAIL("hb_rope_kv_slices: head_dim %d must be a multiple of 8", D);
  if (((uintptr_t)ws | (uintptr_t)q_out | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)table) & 15 || (row_stride & 3) || (slice_stride & 3))
    HB_FAIL("hb_rope_kv_slices: pointers and strides must be multiples of 16 bytes");
  if (ksplit < 1) HB_FAIL("hb_rope_kv_slices: %d slices", ksplit);
  const int items = (Hq + Hkv) * (D >> 3) + Hkv * (D >> 2);
  const int ny = T > 128 ? 1 : (items + 255) / 256;     // few rows: a row's heads are shared among several blocks
  hb_launch(rope_kv_slices_kernel, dim3(T, ny), 256, 0, s, ws, ksplit, slice_stride, row_stride, pos, slot_map,
            (const float2*)table, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, Hq, Hkv, D, page_size);
  HB_CHECK_LAUNCH("hb_rope_kv_slices");
  return 0;
}
