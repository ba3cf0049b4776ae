// Attention over the paged bf16 cache, the fast kernels.
//
// attn_decode_kernel: rows with few queries (decode tokens, short portions). One block per
// (key chunk, kv head, row); the G query heads of the kv head share one pass over its keys and
// values. Keys are cut into chunks of ABSOLUTE positions, so the split of a row depends on its
// position alone. Softmax and the value sums are fp32; partial (acc, max, sum) of rows that span
// several chunks go to a workspace and are merged in ascending chunk order by the block of the
// row and kv head that finishes last.
#include "tc_common.cuh"

HB_TL_DEFINE(attn)

#ifndef HB_AD_TMA
#define HB_AD_TMA 1
#endif
#ifndef HB_AD_THREADS
#define HB_AD_THREADS 128
#endif
constexpr int AD_THREADS = HB_AD_THREADS, AD_WARPS = AD_THREADS / 32;
static int g_ad_cluster_rows = 8;    // rows of a step up to which a row's chunk blocks run as one cluster (see CL below); measured:
                                     // 4 % faster steps at 1 and 8 rows, 2 % slower at 16, 12 % slower at 32 (clusters are placed as gangs)
HB_EXPORT void hb_attn_decode_set_cluster_rows(int rows) { g_ad_cluster_rows = rows; }

// Byte offset of 16-byte chunk c of key row `row` in a [keys][D] bf16 tile (D = 64 or 128): the
// swizzle that makes ldmatrix of eight consecutive rows free of bank conflicts.
template <int D> __device__ __forceinline__ uint32_t ad_swz(int row, int c) {
  return (uint32_t)(row * (D * 2) + ((c ^ (row & 7)) << 4));
}

// The same for a tile that TMA wrote: per 64 columns a [keys][128 bytes] block in the 128-byte
// swizzle (16-byte chunk ^ (row & 7)); head_dim 128 is two such blocks, half_stride bytes apart.
template <int D, bool TMA> __device__ __forceinline__ uint32_t ad_off(int row, int c, uint32_t half_stride) {
  if constexpr (TMA) return (uint32_t)((c >> 3) * half_stride + row * 128 + (((c & 7) ^ (row & 7)) << 4));
  else return ad_swz<D>(row, c);
}

// Rows [r_lo, r_hi) of the tile (row r = key k0 + r) by cp.async, page by page: the page
// numbers of four pages are read first, then every thread copies its 16-byte pieces of them.
template <int D>
__device__ __forceinline__ void ad_load_rows(const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                                             const int* __restrict__ table, int Hkv, int h, int page_size, int k0,
                                             int r_lo, int r_hi, uint32_t sK, uint32_t sV, int tid) {
  constexpr int CH = D / 8;
  if (r_lo >= r_hi) return;
  const int pg_lo = (k0 + r_lo) / page_size, pg_hi = (k0 + r_hi - 1) / page_size, pieces = page_size * CH;
  for (int pg0 = pg_lo; pg0 <= pg_hi; pg0 += 4) {
    int pid[4];
#pragma unroll
    for (int j = 0; j < 4; j++) pid[j] = pg0 + j <= pg_hi ? __ldg(table + pg0 + j) : 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (pg0 + j > pg_hi) break;
      const size_t base = ((size_t)pid[j] * Hkv + h) * page_size * D;
      const int r_page = (pg0 + j) * page_size - k0;   // tile row of the page's first key
      for (int i = tid; i < pieces; i += AD_THREADS) {
        const int rr = i / CH, c = i % CH, r = r_page + rr;
        if (r < r_lo || r >= r_hi) continue;
        const uint32_t off = ad_swz<D>(r, c);
        hb_cp_async16(sK + off, kc + base + (size_t)rr * D + c * 8);
        hb_cp_async16(sV + off, vc + base + (size_t)rr * D + c * 8);
      }
    }
  }
}


// One block = one (key chunk, kv head, row). The chunk's keys and values are requested at once
// with cp.async into swizzled shared memory; each warp then takes 64 keys: S = Q K^T and
// O = P V on warp MMAs with the G query heads of the kv head as the rows of the 16-row tile
// (src/kernels.cuh:1681-1869 does the same on a contiguous cache), softmax in fp32 in the exp2
// domain, P rounded to bf16 before P V. The warps' (max, sum, O) are combined in warp order.
//
// Keys below ctx_len[request] were written by earlier steps, and the step's positions and block
// tables by a copy that ended before the step's first kernel began: a block asks for those keys
// and values BEFORE it waits for the kernel ahead of it (which writes this step's keys), so that
// under programmatic dependent launch the cache streams in while the projections still run.
// A row that spans several chunks is finished by the block that ends last (a counter per
// (row, kv head), left at zero again): it adds the chunks' partials in ascending chunk order.
//
// TMA: the tile comes by cp.async.bulk.tensor, one box per page and 64 columns, asked for by lane 0
// of the warp that will use it and awaited on that warp's own mbarrier (bounded). The copy engine
// keeps far more bytes in flight than 16-byte loads from 128 threads can: this is the kernel for
// whole pages (no window, page size 8 to 64); the other one takes the rest.
//
// RW (TMA only): rows of shared memory a warp has for its 64 keys. 64: the whole chunk lies in shared memory. 32
// (head_dim 128): a warp walks its keys in two passes through 32 rows, asking for the second half when it is done
// with the first: a block holds 64 KB instead of 128 KB of keys and values and three blocks share an SM instead
// of one, which keeps more bytes in flight; the warps' partial results then lie over the keys (after a barrier).
// KW (TMA only): keys of the chunk a warp owns (chunk / 4): 64, or 128 (head_dim 64: chunks of 512 keys, two passes
// through 64 rows: half as many blocks and partial results, and a step of 8 requests fits the SMs at once).
// SR (TMA only): rows of shared memory a warp has: RW (it asks for the keys of a pass when it is done with the pass
// before) or KW (all its keys are asked for at the start: 128 KB a block, for launches of so few blocks that every one
// has an SM of its own; the passes and their arithmetic are the same).
// CL (TMA only): the chunk blocks of a (row, kv head) are one thread-block cluster (the grid's x extent, at most 8). A
// block leaves its partial result in its own shared memory, the cluster meets at a barrier, and the block of the
// row's first chunk adds the partials through distributed shared memory, in the same order and with the same
// arithmetic as the merge through memory below: fence, counter and the partials' round trip through L2 (4 of a
// layer's 11 us at 8 requests) become two cluster barriers. Blocks without keys only pass the barriers.
template <int D, int G, bool TMA, int RW, int KW, int SR, bool CL>
__global__ void __launch_bounds__(AD_THREADS) attn_decode_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, int* __restrict__ status,
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
    const int* __restrict__ bt, int bt_stride, const int* __restrict__ row_req, const int* __restrict__ pos,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml, int Hq, int Hkv,
    int page_size, int window, float scale_log2, int chunk, int S, const int* __restrict__ q_len, int row_limit,
    const int* __restrict__ ctx_len, int* __restrict__ counters) {
  constexpr int CH = D / 8, KS = D / 16, NT_O = D / 8, WK = 64;  // WK: keys per warp pass
  extern __shared__ __align__(128) uint8_t smem_dyn[];
  uint8_t* smem_raw = TMA ? (uint8_t*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023) : smem_dyn;   // the swizzle wants 1 KB
  static_assert((RW == WK && KW == WK) || (TMA && (RW == 32 || RW == 64) && KW % RW == 0), "a warp's keys and rows");
  static_assert(SR == RW || SR == KW, "a warp's rows of shared memory: one pass or all its keys");
  constexpr int NSUB = KW / RW;                                         // passes of a warp over its keys
  const int tile_rows = TMA ? AD_WARPS * SR : chunk;                    // key rows of shared memory
  const uint32_t sK = hb_smem_u32(smem_raw), sV = sK + tile_rows * D * 2, sQ = sV + tile_rows * D * 2;
  const uint32_t hs = (uint32_t)tile_rows * 128;                        // bytes between the 64-column halves of a TMA tile
  float* red_o = NSUB == 1 ? (float*)(smem_raw + 2 * tile_rows * D * 2 + 16 * D * 2) : (float*)smem_raw;  // [warps][G][D]
  float* red_ml = red_o + AD_WARPS * G * D;                             // [warps][G][2]
  __shared__ int is_last;
  __shared__ __align__(8) uint64_t bars[AD_WARPS];
  __shared__ int abort_flag;
  __shared__ __align__(16) float cl_acc[CL ? G * D : 1];     // CL: this block's partial result, read by the merging block
  __shared__ __align__(8) float cl_ml[CL ? G * 2 : 2];
  hb_pdl_launch();
  HB_TL_MARK(0, 0);
  const int t = blockIdx.z, h = blockIdx.y, s = blockIdx.x;
  // row_req null: a step of single decode rows, row t being request t (and its position the length its request had):
  // one round trip to memory less before the keys can be asked for
  const int rq = row_req ? row_req[t] : t;
  const int p = pos[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int s_lo = lo / chunk, s_hi = p / chunk;
  if ((q_len && q_len[rq] >= row_limit) || s < s_lo || s > s_hi) {  // a long portion (the flash kernel's), or no keys here
    if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0) hb_pdl_wait();  // the grid never ends before the one ahead of it
    if constexpr (CL) { hb_cluster_sync(); hb_cluster_sync(); }      // the cluster's two barriers, as every block of it
    return;
  }
  const int k0 = max(s * chunk, lo), k1 = min((s + 1) * chunk, p + 1), nk = k1 - k0;
  const int n_old = ctx_len ? max(0, min(k1, row_req ? ctx_len[rq] : p) - k0) : 0;   // rows of the tile from earlier steps
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  const int* table = bt + (size_t)rq * bt_stride;
  bool loaded = true;
  if constexpr (TMA) {
    // whole pages: row r of the tile is key s * chunk + r; warp w owns rows 64 w .. 64 w + 63
    if (tid == 0) {
      for (int w = 0; w < AD_WARPS; w++) hb_mbar_init(&bars[w], 2);
      abort_flag = 0;
      hb_fence_barrier_init();
    }
    __syncthreads();
    // warp w's keys are KW w .. KW w + KW - 1 of the chunk; its rows of shared memory SR w .. SR w + SR - 1 hold the
    // first SR of them now
    const int r_w = warp * KW, rb = warp * SR, page_bytes = page_size * D * 2 * 2;   // a page's keys and values of one kv head
    const int pages_w = r_w < nk ? min(SR / page_size, (nk - r_w + page_size - 1) / page_size) : 0;
    const int old_w = min(pages_w, max(0, n_old - r_w) / page_size);  // pages wholly from earlier steps
    const int page0 = (k0 + r_w) / page_size;
    if (pages_w > 0) {
      // rows of this warp beyond its last page are never written: the values there must be finite (they meet P = 0;
      // in a second pass they are values of the first)
      for (int i = (rb + pages_w * page_size) * CH + lane; i < (rb + SR) * CH; i += 32)
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(sV + ad_off<D, true>(i / CH, i % CH, hs)), "r"(0u) : "memory");
      if (lane == 0) {
        hb_mbar_expect_tx(&bars[warp], (uint32_t)(old_w * page_bytes));
        for (int j = 0; j < old_w; j++) {
          const int row = (__ldg(table + page0 + j) * Hkv + h) * page_size, dst = (rb + j * page_size) * 128;
#pragma unroll
          for (int hf = 0; hf < D / 64; hf++) {
            hb_tma_load_2d(smem_raw + hf * hs + dst, &map_k, &bars[warp], hf * 64, row);
            hb_tma_load_2d(smem_raw + tile_rows * D * 2 + hf * hs + dst, &map_v, &bars[warp], hf * 64, row);
          }
        }
      }
    }
    hb_pdl_wait();
    HB_TL_MARK(0, 1);
    if (pages_w > 0 && lane == 0) {   // the pages that hold this step's keys
      hb_mbar_expect_tx(&bars[warp], (uint32_t)((pages_w - old_w) * page_bytes));
      for (int j = old_w; j < pages_w; j++) {
        const int row = (__ldg(table + page0 + j) * Hkv + h) * page_size, dst = (rb + j * page_size) * 128;
#pragma unroll
        for (int hf = 0; hf < D / 64; hf++) {
          hb_tma_load_2d(smem_raw + hf * hs + dst, &map_k, &bars[warp], hf * 64, row);
          hb_tma_load_2d(smem_raw + tile_rows * D * 2 + hf * hs + dst, &map_v, &bars[warp], hf * 64, row);
        }
      }
    }
  } else {
  const int rows_pad = (nk + WK - 1) / WK * WK;  // rows the warps will touch; the tail is zeroed
  for (int i = nk * CH + tid; i < rows_pad * CH; i += AD_THREADS) {
    const uint32_t off = ad_swz<D>(i / CH, i % CH);
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(sK + off), "r"(0u) : "memory");
    asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(sV + off), "r"(0u) : "memory");
  }
  ad_load_rows<D>(kc, vc, table, Hkv, h, page_size, k0, 0, n_old, sK, sV, tid);
  hb_cp_async_commit();
  hb_pdl_wait();
  ad_load_rows<D>(kc, vc, table, Hkv, h, page_size, k0, n_old, nk, sK, sV, tid);   // this step's keys
  hb_cp_async_commit();
  }
  // Q tile [16][D]: rows 0..G-1 are the heads of this kv head, the rest zero
  for (int i = tid; i < 16 * CH; i += AD_THREADS) {
    const int r = i / CH, c = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *(const uint4*)(q + ((size_t)t * Hq + (size_t)h * G + r) * D + c * 8);
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(sQ + ad_swz<D>(r, c)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
  if constexpr (!TMA) hb_cp_async_wait<0>();
  __syncthreads();
  if constexpr (TMA) {
    if (warp * KW < nk) loaded = hb_mbar_wait(&bars[warp], 0, &abort_flag);
    if (!loaded && lane == 0) atomicExch(status, 1);   // the result is not valid; the host raises
  }
  const int* table_w = table;   // (the loop below asks for a warp's second half itself)
  HB_TL_MARK(0, 2);

  float m_run = -INFINITY, l_run = 0.f;  // of row g (a head when g < G), over this warp's keys
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  uint32_t qf[KS][4];
  {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KS; kk++) hb_ldmatrix_x4(qf[kk], sQ + ad_swz<D>((mi & 1) * 8 + r, kk * 2 + (mi >> 1)));
  }
  for (int pass = 0;; pass++) {
    // keys kb .. kb + RW - 1 of the chunk, in rows rb .. of shared memory
    const int kb = TMA ? warp * KW + pass * RW : warp * WK + pass * AD_WARPS * WK;
    if (kb >= nk || (TMA && pass >= NSUB)) break;
    const int rb = TMA ? warp * SR + (SR == RW ? 0 : pass * RW) : kb;
    if constexpr (TMA && NSUB > 1 && SR == RW) {
      if (pass > 0) {   // the second half of the warp's keys goes where the first was: every lane is done reading it
        __syncwarp();
        const int pages = min(RW / page_size, (nk - kb + page_size - 1) / page_size), page0 = (k0 + kb) / page_size;
        if (lane == 0) {
          hb_fence_proxy_async();
          hb_mbar_expect_tx(&bars[warp], (uint32_t)(pages * page_size * D * 2 * 2));
          hb_mbar_arrive(&bars[warp]);   // the barrier counts two arrivals a phase
          for (int j = 0; j < pages; j++) {
            const int row = (__ldg(table_w + page0 + j) * Hkv + h) * page_size, dst = (rb + j * page_size) * 128;
#pragma unroll
            for (int hf = 0; hf < D / 64; hf++) {
              hb_tma_load_2d(smem_raw + hf * hs + dst, &map_k, &bars[warp], hf * 64, row);
              hb_tma_load_2d(smem_raw + tile_rows * D * 2 + hf * hs + dst, &map_v, &bars[warp], hf * 64, row);
            }
          }
        }
        if (loaded) loaded = hb_mbar_wait(&bars[warp], pass & 1, &abort_flag);
        if (!loaded) {
          if (lane == 0) atomicExch(status, 1);
          break;
        }
      }
    }
    float sc[RW / 8][4];
#pragma unroll
    for (int i = 0; i < RW / 8; i++) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int kk = 0; kk < KS; kk++) {
#pragma unroll
        for (int np = 0; np < RW / 16; np++) {
          uint32_t b[4];
          hb_ldmatrix_x4(b, sK + ad_off<D, TMA>(rb + np * 16 + (mi >> 1) * 8 + r, kk * 2 + (mi & 1), hs));
          hb_mma_16816(sc[2 * np], qf[kk], b);
          hb_mma_16816(sc[2 * np + 1], qf[kk], b + 2);
        }
      }
    }
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < RW / 8; i++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        if (kb + i * 8 + 2 * tq + e >= nk) sc[i][e] = -INFINITY;
        mx = fmaxf(mx, sc[i][e]);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_run, mx * scale_log2);   // mx is a real score here: a pass never runs without a visible key
    const float corr = hb_exp2(m_run - mn);
    m_run = mn;
    float sum = 0.f;
    uint32_t pf[RW / 16][4];
#pragma unroll
    for (int i = 0; i < RW / 8; i++) {
      const float p0 = hb_exp2(sc[i][0] * scale_log2 - mn), p1 = hb_exp2(sc[i][1] * scale_log2 - mn);
      sum += p0 + p1;
      pf[i >> 1][(i & 1) * 2] = hb_pack_bf16(p0, p1);
      pf[i >> 1][(i & 1) * 2 + 1] = 0u;  // rows 8..15 of the tile are padding
    }
    l_run = l_run * corr + sum;
#pragma unroll
    for (int i = 0; i < NT_O; i++) { o[i][0] *= corr; o[i][1] *= corr; }
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int j2 = 0; j2 < RW / 16; j2++) {
#pragma unroll
        for (int cp = 0; cp < NT_O / 2; cp++) {
          uint32_t b[4];
          hb_ldmatrix_x4_trans(b, sV + ad_off<D, TMA>(rb + j2 * 16 + (mi & 1) * 8 + r, cp * 2 + (mi >> 1), hs));
          hb_mma_16816(o[2 * cp], pf[j2], b);
          hb_mma_16816(o[2 * cp + 1], pf[j2], b + 2);
        }
      }
    }
  }
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if constexpr (NSUB > 1) __syncthreads();   // the partial results lie over the keys: every warp is done with them
  if (g < G) {
#pragma unroll
    for (int i = 0; i < NT_O; i++) {
      red_o[(warp * G + g) * D + i * 8 + 2 * tq] = o[i][0];
      red_o[(warp * G + g) * D + i * 8 + 2 * tq + 1] = o[i][1];
    }
    if (tq == 0) { red_ml[(warp * G + g) * 2] = m_run; red_ml[(warp * G + g) * 2 + 1] = l_run; }
  }
  __syncthreads();
  // the warps' partial results, in warp order; (max, sum) leave in the natural-log domain
  const bool whole = s_lo == s_hi;
  for (int i = tid; i < G * D; i += AD_THREADS) {
    const int gg = i / D, d = i - gg * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < AD_WARPS; w++) m = fmaxf(m, red_ml[(w * G + gg) * 2]);
    float a = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < AD_WARPS; w++) {
      const float f = hb_exp2(red_ml[(w * G + gg) * 2] - m);  // 0 for a warp without keys
      a += red_o[(w * G + gg) * D + d] * f;
      l += red_ml[(w * G + gg) * 2 + 1] * f;
    }
    const size_t head = (size_t)t * Hq + (size_t)h * G + gg;
    if (whole) {
      out[head * D + d] = __float2bfloat16_rn(a / l);
    } else if constexpr (CL) {
      cl_acc[i] = a;
      if (d == 0) { cl_ml[gg * 2] = m * 0.6931471805599453f; cl_ml[gg * 2 + 1] = l; }
    } else {
      part_acc[(head * S + s) * D + d] = a;
      if (d == 0) {
        part_ml[(head * S + s) * 2] = m * 0.6931471805599453f;
        part_ml[(head * S + s) * 2 + 1] = l;
      }
    }
  }
  HB_TL_MARK(1, 3);   // slot 1: the end of the chunk work; slot 0: the end of the merge
  if constexpr (CL) {
    hb_cluster_sync();                                     // every block's partial is in its shared memory, visible cluster-wide
    if (!whole && s == s_lo) {
      const int nc = s_hi - s_lo + 1;
      const uint32_t acc_l = hb_smem_u32(cl_acc), ml_l = hb_smem_u32(cl_ml);
      for (int i = tid; i < G * D; i += AD_THREADS) {
        const int gg = i / D;
        float mv[8], lv[8], av[8];                         // a cluster has at most 8 blocks
#pragma unroll
        for (int c = 0; c < 8; c++)
          if (c < nc) {
            uint32_t ra, rm;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(acc_l + (uint32_t)i * 4), "r"((uint32_t)(s_lo + c)));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rm) : "r"(ml_l + (uint32_t)gg * 8), "r"((uint32_t)(s_lo + c)));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(av[c]) : "r"(ra) : "memory");
            asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(mv[c]), "=f"(lv[c]) : "r"(rm) : "memory");
          }
        float m = -INFINITY, a = 0.f, l = 0.f;
#pragma unroll
        for (int c = 0; c < 8; c++)
          if (c < nc) m = fmaxf(m, mv[c]);
#pragma unroll
        for (int c = 0; c < 8; c++)
          if (c < nc) {
            const float f = expf(mv[c] - m);
            l += lv[c] * f;
            a += av[c] * f;
          }
        out[((size_t)t * Hq + (size_t)h * G + gg) * D + (i - gg * D)] = __float2bfloat16_rn(a / l);
      }
    }
    hb_cluster_sync();                                     // no block leaves while its partial may still be read
    HB_TL_MARK(0, 3);
    return;
  }
  if (whole) return;
  // the block of this (row, kv head) that ends last adds the chunks, lowest first
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* cnt = counters + (size_t)t * Hkv + h;
    const int last = atomicAdd(cnt, 1) == s_hi - s_lo;
    if (last) *cnt = 0;
    is_last = last;
  }
  __syncthreads();
  if (!is_last) return;
  // the others' partials were made visible (their fence) before their count; they are read from L2 below
  const int nc = s_hi - s_lo + 1;
  constexpr int PER = 2;   // (head, column) pairs of a thread whose loads are in flight together
  if (nc <= 16) {   // every load of a group of pairs asked for before the first is used: one round trip to L2 a group
   for (int i0 = tid; i0 < G * D; i0 += PER * AD_THREADS) {
    float2 v[PER][16];
    float acc[PER][16];
#pragma unroll
    for (int k = 0; k < PER; k++) {
      const int i = i0 + k * AD_THREADS, gg = i / D, d = i - gg * D;
      if (i < G * D) {
        const size_t head = (size_t)t * Hq + (size_t)h * G + gg;
        const float2* ml = (const float2*)part_ml + head * S + s_lo;
        const float* pa = part_acc + (head * S + s_lo) * D + d;
#pragma unroll
        for (int c = 0; c < 16; c++)
          if (c < nc) { v[k][c] = __ldcg(ml + c); acc[k][c] = __ldcg(pa + (size_t)c * D); }
      }
    }
#pragma unroll
    for (int k = 0; k < PER; k++) {
      const int i = i0 + k * AD_THREADS, gg = i / D, d = i - gg * D;
      if (i < G * D) {
        float m = -INFINITY, a = 0.f, l = 0.f;
#pragma unroll
        for (int c = 0; c < 16; c++)
          if (c < nc) m = fmaxf(m, v[k][c].x);
#pragma unroll
        for (int c = 0; c < 16; c++)
          if (c < nc) {
            const float f = expf(v[k][c].x - m);
            l += v[k][c].y * f;
            a += acc[k][c] * f;
          }
        out[((size_t)t * Hq + (size_t)h * G + gg) * D + d] = __float2bfloat16_rn(a / l);
      }
    }
   }
  } else {
    for (int i = tid; i < G * D; i += AD_THREADS) {
      const int gg = i / D, d = i - gg * D;
      const size_t head = (size_t)t * Hq + (size_t)h * G + gg;
      const float2* ml = (const float2*)part_ml + head * S + s_lo;
      const float* pa = part_acc + (head * S + s_lo) * D + d;
      float m = -INFINITY, a = 0.f, l = 0.f;
      for (int c = 0; c < nc; c++) m = fmaxf(m, __ldcg(ml + c).x);
      for (int c = 0; c < nc; c++) {
        const float2 v = __ldcg(ml + c);
        const float f = expf(v.x - m);
        l += v.y * f;
        a += __ldcg(pa + (size_t)c * D) * f;
      }
      out[head * D + d] = __float2bfloat16_rn(a / l);
    }
  }
  HB_TL_MARK(0, 3);
}

template <int D, bool TMA, int RW, int KW, int SR, bool CL = false>
static int launch_decode(int G, dim3 grid, size_t smem, cudaStream_t st, const CUtensorMap& mk, const CUtensorMap& mv,
                         int* status, const __nv_bfloat16* q, const __nv_bfloat16* kc, const __nv_bfloat16* vc,
                         const int* bt, int bt_stride, const int* row_req, const int* pos, __nv_bfloat16* out, float* pa,
                         float* pm, int Hq, int Hkv, int page_size, int window, float scale, int chunk, int S,
                         const int* q_len, int row_limit, const int* ctx_len, int* counters) {
#define HB_AD_CASE(GG)                                                                                              \
  case GG:                                                                                                          \
    {                                                                                                               \
      static bool configured = false;                                                                               \
      if (!configured) {                                                                                            \
        cudaFuncSetAttribute(attn_decode_kernel<D, GG, TMA, RW, KW, SR, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
        configured = true;                                                                                          \
      }                                                                                                             \
    }                                                                                                               \
    if (CL)                                                                                                         \
      hb_launch_cluster(attn_decode_kernel<D, GG, TMA, RW, KW, SR, CL>, grid, AD_THREADS, smem, st, dim3(grid.x, 1, 1), mk, mv, status, \
                        q, kc, vc, bt, bt_stride, row_req, pos, out, pa, pm, Hq, Hkv, page_size, window, scale, chunk, S,    \
                        q_len, row_limit, ctx_len, counters);                                                       \
    else                                                                                                            \
      hb_launch(attn_decode_kernel<D, GG, TMA, RW, KW, SR, CL>, grid, AD_THREADS, smem, st, mk, mv, status, q, kc, vc, bt, bt_stride, \
                row_req, pos, out, pa, pm, Hq, Hkv, page_size, window, scale, chunk, S, q_len, row_limit, ctx_len,  \
                counters);                                                                                          \
    return 0;
  switch (G) {
    HB_AD_CASE(1) HB_AD_CASE(2) HB_AD_CASE(3) HB_AD_CASE(4) HB_AD_CASE(5) HB_AD_CASE(6) HB_AD_CASE(7) HB_AD_CASE(8)
  }
#undef HB_AD_CASE
  return 1;
}

// Does the decode kernel take these sizes? (head_dim 64 or 128; group up to 8)
HB_EXPORT int hb_attn_decode_supported(int Hq, int Hkv, int D) {
  return Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 8 && (D == 64 || D == 128);
}

// Partials layout as hb_attn_rows of the core library: workspace = part_acc [T, Hq, S, D] then
// part_ml [T, Hq, S, 2], S = max_pos / chunk + 1; `counters` are T * Hkv ints that are zero
// between calls (needed when S > 1). With q_len given, rows of requests whose portion has
// row_limit rows or more are skipped (the flash kernel computes those). ctx_len (per request,
// or null): the tokens that were in the cache before this step; their keys may be read before
// the kernel ahead in the stream has ended. row_req null: row t is request t's only row. n_pages: the pages the cache holds (its first
// extent); status: the word a bounded wait that ran out sets to 1. With both, no window, a chunk
// of 256 (or of 512 at head_dim 64) and pages of 8 to 64 tokens the keys and values come by TMA.
HB_EXPORT int hb_attn_decode(const void* q, const void* kc, const void* vc, long n_pages, const int* bt, int bt_stride,
                             const int* row_req, const int* pos, void* out, float* workspace, int* counters, int T,
                             int Hq, int Hkv, int D, int page_size, int window, float scale, int chunk, int max_pos,
                             const int* q_len, int row_limit, const int* ctx_len, int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (!hb_attn_decode_supported(Hq, Hkv, D)) HB_FAIL("hb_attn_decode: %d/%d heads of %d are not supported", Hq, Hkv, D);
  if (chunk <= 0 || chunk % 32) HB_FAIL("hb_attn_decode: chunk %d must be a positive multiple of 32", chunk);
  if (T > 65535 || Hkv > 65535 || max_pos / chunk + 1 > 65535) HB_FAIL("hb_attn_decode: %d rows / %d kv heads / %d chunks are beyond the grid limit", T, Hkv, max_pos / chunk + 1);
  const int G = Hq / Hkv, S = max_pos / chunk + 1;
  if (S > 1 && (!workspace || !counters)) HB_FAIL("hb_attn_decode: rows that span %d chunks need a workspace and counters", S);
  if (chunk % 64) HB_FAIL("hb_attn_decode: chunk %d must be a multiple of 64", chunk);
  const long cache_rows = n_pages * Hkv * page_size;
  const bool tma = HB_AD_TMA && status && n_pages > 0 && window == 0 && page_size % 8 == 0 && page_size <= 64 &&
                   64 % page_size == 0 && cache_rows < (1L << 31) && !(((uintptr_t)kc | (uintptr_t)vc) & 15) &&
                   (chunk == AD_WARPS * 64 || (chunk == AD_WARPS * 128 && D == 64));
  // by TMA a block has 4 x RW rows of keys and values. head_dim 128 with pages of at most 32 tokens: a warp's 64 keys
  // in two passes through 32 rows (64 KB a block, three blocks an SM instead of one). head_dim 64 with chunks of 512
  // keys: a warp's 128 keys in two passes through 64 rows (64 KB a block as with chunks of 256). In both the warps'
  // partial results lie over the keys at the end.
  const bool halves = tma && D == 128 && page_size <= 32, wide = tma && chunk == AD_WARPS * 128;
  // so few blocks that each has an SM of its own: all the keys of a chunk of 512 at once (the same passes)
  static int n_sm = 0;
  if (!n_sm) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n_sm = 1;
  }
  const bool resident = wide && (long)S * Hkv * T <= n_sm;
  const int rw = halves ? 32 : resident ? 128 : 64;
  const size_t smem = tma ? 2 * (size_t)(AD_WARPS * rw) * D * 2 + 16 * (size_t)D * 2 + 1024 +
                                (halves || wide ? 0 : AD_WARPS * (size_t)G * (D + 2) * sizeof(float))
                          : 2 * (size_t)chunk * D * 2 + 16 * (size_t)D * 2 + AD_WARPS * (size_t)G * (D + 2) * sizeof(float);
  if (smem > 200 * 1024) HB_FAIL("hb_attn_decode: %zu bytes of shared memory (chunk %d, head_dim %d)", smem, chunk, D);
  float* pa = workspace;
  float* pm = workspace ? workspace + (size_t)T * Hq * S * D : nullptr;
  dim3 grid(S, Hkv, T);
  const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)kc, *vv = (const __nv_bfloat16*)vc;
  CUtensorMap mk, mv;
  memset(&mk, 0, sizeof(mk));
  memset(&mv, 0, sizeof(mv));
  if (tma) {   // the cache as [pages * kv heads * page_size rows][D], a box = one page of one kv head, 64 columns
    if (hb_make_tensor_map_bf16(&mk, kc, (uint64_t)cache_rows, (uint64_t)D, (uint64_t)D, (uint32_t)page_size)) return -1;
    if (hb_make_tensor_map_bf16(&mv, vc, (uint64_t)cache_rows, (uint64_t)D, (uint64_t)D, (uint32_t)page_size)) return -1;
  }
  const float sl2 = scale * 1.4426950408889634f;
  int r = 1;
#define HB_AD_ARGS G, grid, smem, st, mk, mv, status, qq, kk, vv, bt, bt_stride, row_req, pos, (__nv_bfloat16*)out, pa, pm, Hq, Hkv, \
                   page_size, window, sl2, chunk, S, q_len, row_limit, ctx_len, counters
  // a step of few rows whose chunks fit one cluster: the chunks' partial results meet in distributed shared memory
  const bool cl = tma && S >= 2 && S <= 8 && T <= g_ad_cluster_rows;
  if (D == 64 && resident && cl) r = launch_decode<64, true, 64, 128, 128, true>(HB_AD_ARGS);
  else if (D == 64 && wide && cl) r = launch_decode<64, true, 64, 128, 64, true>(HB_AD_ARGS);
  else if (halves && cl) r = launch_decode<128, true, 32, 64, 32, true>(HB_AD_ARGS);
  else if (D == 64 && resident) r = launch_decode<64, true, 64, 128, 128>(HB_AD_ARGS);
  else if (D == 64 && wide) r = launch_decode<64, true, 64, 128, 64>(HB_AD_ARGS);
  else if (D == 64) r = tma ? launch_decode<64, true, 64, 64, 64>(HB_AD_ARGS) : launch_decode<64, false, 64, 64, 64>(HB_AD_ARGS);
  else if (halves) r = launch_decode<128, true, 32, 64, 32>(HB_AD_ARGS);
  else if (D == 128) r = tma ? launch_decode<128, true, 64, 64, 64>(HB_AD_ARGS) : launch_decode<128, false, 64, 64, 64>(HB_AD_ARGS);
#undef HB_AD_ARGS
  if (r) HB_FAIL("hb_attn_decode: no kernel for group %d", G);
  HB_CHECK_LAUNCH("hb_attn_decode");
  return 0;
}
