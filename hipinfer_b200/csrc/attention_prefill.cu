// Causal flash attention of prompt portions over the paged bf16 cache (head_dim 64 or 128).
//
// One CTA = 64 consecutive query rows of one request and one query head (4 warps x 16 rows).
// It walks the request's keys in tiles of 64 ABSOLUTE positions, gathered page by page through
// the block table with cp.async into swizzled shared memory (double-buffered), S = Q K^T and
// O += P V on warp MMAs (m16n8k16, bf16 in, fp32 out), online softmax in fp32 in the exp2 domain,
// P rounded to bf16 before P V, as the reference does (src/kernels.cuh:1335-1482, 1456). The
// mask is on absolute positions: key kp is visible to a query at qp iff kp <= qp (and
// kp > qp - window when there is a window) (src/kernels.cuh:1416-1418). Because tiles are cut at
// absolute positions and a row's running max and sum are its own, a row's result does not
// depend on how the prompt was cut into portions or on what else is in the batch.
//
// Requests whose portion has fewer than `min_rows` rows are left to the row kernel.
#include "tc_common.cuh"

#ifndef HB_FP_MINB
#define HB_FP_MINB 4
#endif
constexpr int FP_BQ = 64, FP_BKV = 64, FP_THREADS = 128;

template <int D> __device__ __forceinline__ uint32_t fp_swz(int row, int chunk) {
  return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

// Copies keys [k_base, k_base + 64) of kv head h into a [64][D] swizzled tile; rows outside
// [k_first, k_last] are zeroed (their pages may have been given back, or not exist yet).
template <int D>
__device__ __forceinline__ void fp_load_tile(uint32_t tile, const __nv_bfloat16* __restrict__ cache,
                                             const int* __restrict__ table, int Hkv, int h, int page_size, int k_base,
                                             int k_first, int k_last, int tid) {
  constexpr int CH = D / 8;
  for (int i = tid; i < FP_BKV * CH; i += FP_THREADS) {
    const int r = i / CH, c = i - r * CH, kp = k_base + r;
    const uint32_t dst = tile + fp_swz<D>(r, c);
    if (kp >= k_first && kp <= k_last) {
      const size_t page = table[kp / page_size];
      hb_cp_async16(dst, cache + ((page * Hkv + h) * page_size + kp % page_size) * D + c * 8);
    } else {
      asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
    }
  }
}

template <int D>
__global__ void __launch_bounds__(FP_THREADS, HB_FP_MINB) flash_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
    const int* __restrict__ bt, int bt_stride, const int* __restrict__ q_start, const int* __restrict__ q_len,
    const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int page_size, int window,
    float scale_log2, int min_rows) {
  constexpr int CH = D / 8, KS = D / 16, NT_O = D / 8, TILE = FP_BKV * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  // the last query tiles of a portion have the most keys to walk: they are started first
  // blocks start in the order of blockIdx.x, then y: all heads' heaviest query tile first, then the next one
  // (longest work first: with the query tile fastest, the last head's heaviest tile would start last and run alone)
  const int req = blockIdx.z, hq = blockIdx.x, qt = gridDim.y - 1 - blockIdx.y;
  const int n_rows = q_len[req];
  if (n_rows < min_rows || qt * FP_BQ >= n_rows) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int h = hq / (Hq / Hkv);
  const int row0 = q_start[req] + qt * FP_BQ, rows_here = min(FP_BQ, n_rows - qt * FP_BQ);
  const int p_first = ctx_len[req] + qt * FP_BQ, p_last = p_first + rows_here - 1;
  const int* table = bt + (size_t)req * bt_stride;
  const uint32_t sQ = hb_smem_u32(smem), sK = sQ + FP_BQ * D * 2, sV = sK + 2 * TILE;

  // Q tile (rows past the portion's end are zero)
  for (int i = tid; i < FP_BQ * CH; i += FP_THREADS) {
    const int r = i / CH, c = i - r * CH;
    const uint32_t dst = sQ + fp_swz<D>(r, c);
    if (r < rows_here) hb_cp_async16(dst, q + ((size_t)(row0 + r) * Hq + hq) * D + c * 8);
    else asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
  }
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int kt_lo = lo / FP_BKV, kt_hi = p_last / FP_BKV;
  fp_load_tile<D>(sK, kc, table, Hkv, h, page_size, kt_lo * FP_BKV, lo, p_last, tid);
  fp_load_tile<D>(sV, vc, table, Hkv, h, page_size, kt_lo * FP_BKV, lo, p_last, tid);
  hb_cp_async_commit();
  hb_cp_async_wait<0>();
  __syncthreads();

  uint32_t qf[KS][4];
  {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KS; kk++)
      hb_ldmatrix_x4(qf[kk], sQ + fp_swz<D>(warp * 16 + (mi & 1) * 8 + r, kk * 2 + (mi >> 1)));
  }
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  // positions of this thread's two rows (rows past the end take the last row's position; never stored)
  const int r_a = warp * 16 + g, r_b = r_a + 8;
  const int qp_a = p_first + min(r_a, rows_here - 1), qp_b = p_first + min(r_b, rows_here - 1);

  for (int kt = kt_lo; kt <= kt_hi; kt++) {
    const int buf = (kt - kt_lo) & 1;
    if (kt < kt_hi) {  // prefetch the next tile into the other buffer
      fp_load_tile<D>(sK + (buf ^ 1) * TILE, kc, table, Hkv, h, page_size, (kt + 1) * FP_BKV, lo, p_last, tid);
      fp_load_tile<D>(sV + (buf ^ 1) * TILE, vc, table, Hkv, h, page_size, (kt + 1) * FP_BKV, lo, p_last, tid);
    }
    hb_cp_async_commit();
    const uint32_t tK = sK + buf * TILE, tV = sV + buf * TILE;
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int kk = 0; kk < KS; kk++) {
#pragma unroll
        for (int np = 0; np < 4; np++) {  // pairs of 8-key tiles
          uint32_t b[4];
          hb_ldmatrix_x4(b, tK + fp_swz<D>(np * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1)));
          hb_mma_16816(s[2 * np], qf[kk], b);
          hb_mma_16816(s[2 * np + 1], qf[kk], b + 2);
        }
      }
    }
    // mask on absolute positions, then the online softmax update of the two rows
    const int k_base = kt * FP_BKV;
    const bool need_mask = k_base + FP_BKV - 1 > p_first || (window > 0 && k_base < p_last - window + 1);
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; i++) {
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int kp = k_base + i * 8 + 2 * t + e;
        if (need_mask) {
          const bool va = kp <= qp_a && (window <= 0 || kp > qp_a - window);
          const bool vb = kp <= qp_b && (window <= 0 || kp > qp_b - window);
          if (!va) s[i][e] = -INFINITY;
          if (!vb) s[i][2 + e] = -INFINITY;
        }
        mx_a = fmaxf(mx_a, s[i][e]);
        mx_b = fmaxf(mx_b, s[i][2 + e]);
      }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m0, mx_a * scale_log2), mn_b = fmaxf(m1, mx_b * scale_log2);
    const float sub_a = mn_a == -INFINITY ? 0.f : mn_a, sub_b = mn_b == -INFINITY ? 0.f : mn_b;
    const float corr_a = hb_exp2(m0 - sub_a), corr_b = hb_exp2(m1 - sub_b);
    m0 = mn_a; m1 = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
    uint32_t pf[4][4];  // P as A-fragments: 4 steps of 16 keys
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const float p0 = hb_exp2(s[i][0] * scale_log2 - sub_a), p1 = hb_exp2(s[i][1] * scale_log2 - sub_a);
      const float p2 = hb_exp2(s[i][2] * scale_log2 - sub_b), p3 = hb_exp2(s[i][3] * scale_log2 - sub_b);
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      pf[i >> 1][(i & 1) * 2] = hb_pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = hb_pack_bf16(p2, p3);
    }
    l0 = l0 * corr_a + sum_a;
    l1 = l1 * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < NT_O; i++) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int j2 = 0; j2 < 4; j2++) {
#pragma unroll
        for (int cp = 0; cp < NT_O / 2; cp++) {
          uint32_t b[4];
          hb_ldmatrix_x4_trans(b, tV + fp_swz<D>(j2 * 16 + (mi & 1) * 8 + r, cp * 2 + (mi >> 1)));
          hb_mma_16816(o[2 * cp], pf[j2], b);
          hb_mma_16816(o[2 * cp + 1], pf[j2], b + 2);
        }
      }
    }
    hb_cp_async_wait<0>();
    __syncthreads();
  }

  // the row sums are spread over the four lanes of a quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv_a = 1.f / l0, inv_b = 1.f / l1;
#pragma unroll
  for (int i = 0; i < NT_O; i++) {
    const int d = i * 8 + 2 * t;
    if (r_a < rows_here)
      *(uint32_t*)(out + ((size_t)(row0 + r_a) * Hq + hq) * D + d) = hb_pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
    if (r_b < rows_here)
      *(uint32_t*)(out + ((size_t)(row0 + r_b) * Hq + hq) * D + d) = hb_pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
  }
}

HB_EXPORT int hb_flash_prefill_supported(int Hq, int Hkv, int D) {
  return Hkv > 0 && Hq % Hkv == 0 && (D == 64 || D == 128);
}

// q, out [T, Hq, D] bf16; caches [page, Hkv, page_size, D] bf16; per request: q_start, q_len,
// ctx_len (tokens cached before this step) and a block table row. Requests with fewer than
// min_rows rows are skipped. max_q_len: the longest portion (sizes the grid).
HB_EXPORT int hb_flash_prefill(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                               const int* q_start, const int* q_len, const int* ctx_len, void* out, int R, int max_q_len,
                               int Hq, int Hkv, int D, int page_size, int window, float scale, int min_rows,
                               cudaStream_t st) {
  if (R <= 0 || max_q_len <= 0) return 0;
  if (!hb_flash_prefill_supported(Hq, Hkv, D)) HB_FAIL("hb_flash_prefill: %d/%d heads of %d are not supported", Hq, Hkv, D);
  if (R > 65535 || max_q_len > 65535 * FP_BQ) HB_FAIL("hb_flash_prefill: %d requests / portions of %d rows are beyond the grid limit", R, max_q_len);
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(Hq, (max_q_len + FP_BQ - 1) / FP_BQ, R);
  const size_t smem = (size_t)(FP_BQ + 4 * FP_BKV) * D * 2;
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)kc, *vv = (const __nv_bfloat16*)vc;
  if (D == 64) {
    flash_prefill_kernel<64><<<grid, FP_THREADS, smem, st>>>(qq, kk, vv, bt, bt_stride, q_start, q_len, ctx_len,
                                                             (__nv_bfloat16*)out, Hq, Hkv, page_size, window, scale_log2, min_rows);
  } else {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(flash_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) HB_FAIL("hb_flash_prefill: %s", cudaGetErrorString(e));
      configured = true;
    }
    flash_prefill_kernel<128><<<grid, FP_THREADS, smem, st>>>(qq, kk, vv, bt, bt_stride, q_start, q_len, ctx_len,
                                                              (__nv_bfloat16*)out, Hq, Hkv, page_size, window, scale_log2, min_rows);
  }
  HB_CHECK_LAUNCH("hb_flash_prefill");
  return 0;
}
