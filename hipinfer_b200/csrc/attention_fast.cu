// Attention over the paged bf16 cache, the fast kernels.
//
// attn_decode_kernel: rows with few queries (decode tokens, short portions). One block per
// (key chunk, kv head, row); the G query heads of the kv head share one pass over its keys and
// values (src/kernels.cuh:1501-1508 does the same on a contiguous cache), 16-byte loads, each
// key read once for all G heads, each value read once for all G heads. Keys are cut into chunks
// of ABSOLUTE positions, so the split of a row depends on its position alone. Scores, softmax
// and the value sums are fp32; partial (acc, max, sum) of rows that span several chunks go to a
// workspace and are merged in ascending chunk order by attn_merge_kernel of the core library.
#include "tc_common.cuh"

constexpr int AD_THREADS = 128;

// Byte offset of 16-byte chunk c of key row `row` in a [keys][D] bf16 tile, swizzled so that both
// a thread-per-row walk and a lanes-across-a-row walk are free of bank conflicts.
template <int D> __device__ __forceinline__ uint32_t ad_swz(int row, int c) {
  constexpr int CH = D / 8;
  return (uint32_t)(row * (D * 2) + ((c ^ (CH == 4 ? ((row >> 1) & 3) : (row & 7))) << 4));
}

template <int D, int G>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
    const int* __restrict__ bt, int bt_stride, const int* __restrict__ row_req, const int* __restrict__ pos,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml, int Hq, int Hkv,
    int page_size, int window, float scale, int chunk, int S, const int* __restrict__ q_len, int row_limit) {
  constexpr int CH = D / 8;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the whole key chunk and the whole value chunk are requested at once (cp.async), so a block
  // has up to 2 * chunk * D * 2 bytes in flight; scores and sums follow
  const uint32_t sK = hb_smem_u32(smem_raw), sV = sK + chunk * D * 2;
  float* qs = (float*)(smem_raw + 2 * chunk * D * 2);  // [G][D], scaled
  float* sc = qs + G * D;                              // [G][chunk]
  float* ml = sc + G * chunk;                          // [G][2]
  float* red = ml + 2 * G;                             // [4 warps][G][D]
  hb_pdl_launch();
  hb_pdl_wait();
  const int t = blockIdx.z, h = blockIdx.y, s = blockIdx.x;
  if (q_len && q_len[row_req[t]] >= row_limit) return;  // a long portion: the flash kernel's
  const int p = pos[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int s_lo = lo / chunk, s_hi = p / chunk;
  if (s < s_lo || s > s_hi) return;
  const int k0 = max(s * chunk, lo), k1 = min((s + 1) * chunk, p + 1), nk = k1 - k0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = bt + (size_t)row_req[t] * bt_stride;
  for (int i = tid; i < nk * CH; i += AD_THREADS) {
    const int r = i / CH, c = i - r * CH, kp = k0 + r;
    const size_t page = table[kp / page_size];
    hb_cp_async16(sK + ad_swz<D>(r, c), kc + ((page * Hkv + h) * page_size + kp % page_size) * D + c * 8);
  }
  hb_cp_async_commit();
  for (int i = tid; i < nk * CH; i += AD_THREADS) {
    const int r = i / CH, c = i - r * CH, kp = k0 + r;
    const size_t page = table[kp / page_size];
    hb_cp_async16(sV + ad_swz<D>(r, c), vc + ((page * Hkv + h) * page_size + kp % page_size) * D + c * 8);
  }
  hb_cp_async_commit();
  const __nv_bfloat16* qrow = q + ((size_t)t * Hq + (size_t)h * G) * D;
  for (int i = tid; i < G * D; i += AD_THREADS) qs[i] = __bfloat162float(qrow[i]) * scale;
  hb_cp_async_wait<1>();
  __syncthreads();

  // scores: one key per thread, all G heads from one pass over the key's D elements
  for (int j = tid; j < nk; j += AD_THREADS) {
    float a[G];
#pragma unroll
    for (int g = 0; g < G; g++) a[g] = 0.f;
#pragma unroll
    for (int i = 0; i < CH; i++) {
      uint4 kv;
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(kv.x), "=r"(kv.y), "=r"(kv.z), "=r"(kv.w) : "r"(sK + ad_swz<D>(j, i)));
      const __nv_bfloat162* k2 = (const __nv_bfloat162*)&kv;
      float kf[8];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float2 f = __bfloat1622float2(k2[e]);
        kf[2 * e] = f.x;
        kf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int g = 0; g < G; g++) {
        const float4 q0 = *(const float4*)(qs + g * D + i * 8), q1 = *(const float4*)(qs + g * D + i * 8 + 4);
        a[g] = fmaf(q0.x, kf[0], a[g]); a[g] = fmaf(q0.y, kf[1], a[g]);
        a[g] = fmaf(q0.z, kf[2], a[g]); a[g] = fmaf(q0.w, kf[3], a[g]);
        a[g] = fmaf(q1.x, kf[4], a[g]); a[g] = fmaf(q1.y, kf[5], a[g]);
        a[g] = fmaf(q1.z, kf[6], a[g]); a[g] = fmaf(q1.w, kf[7], a[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; g++) sc[g * chunk + j] = a[g];
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
  hb_cp_async_wait<0>();
  __syncthreads();

  // values: D/8 lanes share a key's row, so a warp takes 32 / (D/8) keys per pass and each value
  // is read once for all G heads; lanes, then warps, are summed in a fixed order
  constexpr int TPK = D / 8, KPW = 32 / TPK;
  const int kq = lane / TPK, dc = lane % TPK;
  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; g++)
#pragma unroll
    for (int e = 0; e < 8; e++) acc[g][e] = 0.f;
#pragma unroll 4
  for (int j = warp * KPW + kq; j < nk; j += 4 * KPW) {
    uint4 raw;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "r"(sV + ad_swz<D>(j, dc)));
    const __nv_bfloat162* v2 = (const __nv_bfloat162*)&raw;
    float vf[8];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float2 f = __bfloat1622float2(v2[e]);
      vf[2 * e] = f.x;
      vf[2 * e + 1] = f.y;
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float pj = sc[g * chunk + j];
#pragma unroll
      for (int e = 0; e < 8; e++) acc[g][e] = fmaf(pj, vf[e], acc[g][e]);
    }
  }
#pragma unroll
  for (int g = 0; g < G; g++)
#pragma unroll
    for (int e = 0; e < 8; e++) {
      float a = acc[g][e];
#pragma unroll
      for (int o = TPK; o < 32; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (kq == 0) red[(warp * G + g) * D + dc * 8 + e] = a;
    }
  __syncthreads();
  const bool whole = s_lo == s_hi;
  for (int i = tid; i < G * D; i += AD_THREADS) {
    const int g = i / D;
    const float a = ((red[i] + red[G * D + i]) + red[2 * G * D + i]) + red[3 * G * D + i];
    const size_t head = (size_t)t * Hq + (size_t)h * G + g;
    if (whole) out[head * D + (i - g * D)] = __float2bfloat16_rn(a / ml[2 * g + 1]);
    else part_acc[(head * S + s) * D + (i - g * D)] = a;
  }
  if (!whole && tid < G) {
    const size_t head = (size_t)t * Hq + (size_t)h * G + tid;
    part_ml[(head * S + s) * 2] = ml[2 * tid];
    part_ml[(head * S + s) * 2 + 1] = ml[2 * tid + 1];
  }
}

template <int D>
static int launch_decode(int G, dim3 grid, size_t smem, cudaStream_t st, const __nv_bfloat16* q, const __nv_bfloat16* kc,
                         const __nv_bfloat16* vc, const int* bt, int bt_stride, const int* row_req, const int* pos,
                         __nv_bfloat16* out, float* pa, float* pm, int Hq, int Hkv, int page_size, int window, float scale,
                         int chunk, int S, const int* q_len, int row_limit) {
#define HB_AD_CASE(GG)                                                                                              \
  case GG:                                                                                                          \
    {                                                                                                               \
      static bool configured = false;                                                                               \
      if (!configured) {                                                                                            \
        cudaFuncSetAttribute(attn_decode_kernel<D, GG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);   \
        configured = true;                                                                                          \
      }                                                                                                             \
    }                                                                                                               \
    hb_launch(attn_decode_kernel<D, GG>, grid, AD_THREADS, smem, st, q, kc, vc, bt, bt_stride, row_req, pos, out, pa, pm, \
              Hq, Hkv, page_size, window, scale, chunk, S, q_len, row_limit);                                        \
    return 0;
  switch (G) {
    HB_AD_CASE(1) HB_AD_CASE(2) HB_AD_CASE(3) HB_AD_CASE(4) HB_AD_CASE(5) HB_AD_CASE(6) HB_AD_CASE(7) HB_AD_CASE(8)
  }
#undef HB_AD_CASE
  return 1;
}

// Does the decode kernel take these sizes? (head_dim 32, 64 or 128; group up to 8)
HB_EXPORT int hb_attn_decode_supported(int Hq, int Hkv, int D) {
  return Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 8 && (D == 32 || D == 64 || D == 128);
}

// Partials layout as hb_attn_rows of the core library: workspace = part_acc [T, Hq, S, D] then
// part_ml [T, Hq, S, 2], S = max_pos / chunk + 1; rows spanning several chunks are finished by
// hb_attn_merge (core library) with the same chunk. With q_len given, rows of requests whose
// portion has row_limit rows or more are skipped (the flash kernel computes those).
HB_EXPORT int hb_attn_decode(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                             const int* row_req, const int* pos, void* out, float* workspace, int T, int Hq, int Hkv,
                             int D, int page_size, int window, float scale, int chunk, int max_pos, const int* q_len,
                             int row_limit, cudaStream_t st) {
  if (T <= 0) return 0;
  if (!hb_attn_decode_supported(Hq, Hkv, D)) HB_FAIL("hb_attn_decode: %d/%d heads of %d are not supported", Hq, Hkv, D);
  if (chunk <= 0 || chunk % 32) HB_FAIL("hb_attn_decode: chunk %d must be a positive multiple of 32", chunk);
  if (T > 65535 || Hkv > 65535) HB_FAIL("hb_attn_decode: %d rows / %d kv heads are beyond the grid limit", T, Hkv);
  const int G = Hq / Hkv, S = max_pos / chunk + 1;
  if (S > 1 && !workspace) HB_FAIL("hb_attn_decode: rows that span %d chunks need a workspace", S);
  const size_t smem = 2 * (size_t)chunk * D * 2 + ((size_t)G * D + (size_t)G * chunk + 2 * G + 4 * (size_t)G * D) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_attn_decode: %zu bytes of shared memory (chunk %d, head_dim %d)", smem, chunk, D);
  float* pa = workspace;
  float* pm = workspace ? workspace + (size_t)T * Hq * S * D : nullptr;
  dim3 grid(S, Hkv, T);
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)kc, *vv = (const __nv_bfloat16*)vc;
  int r = 1;
  if (D == 32) r = launch_decode<32>(G, grid, smem, st, qq, kk, vv, bt, bt_stride, row_req, pos, (__nv_bfloat16*)out, pa, pm, Hq, Hkv, page_size, window, scale, chunk, S, q_len, row_limit);
  else if (D == 64) r = launch_decode<64>(G, grid, smem, st, qq, kk, vv, bt, bt_stride, row_req, pos, (__nv_bfloat16*)out, pa, pm, Hq, Hkv, page_size, window, scale, chunk, S, q_len, row_limit);
  else if (D == 128) r = launch_decode<128>(G, grid, smem, st, qq, kk, vv, bt, bt_stride, row_req, pos, (__nv_bfloat16*)out, pa, pm, Hq, Hkv, page_size, window, scale, chunk, S, q_len, row_limit);
  if (r) HB_FAIL("hb_attn_decode: no kernel for group %d", G);
  HB_CHECK_LAUNCH("hb_attn_decode");
  return 0;
}
