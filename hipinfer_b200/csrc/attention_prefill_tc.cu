// Causal flash attention of prompt portions on the 5th-generation tensor cores (head_dim 64 or 128).
//
// One CTA = 128 consecutive query rows of one request and one query head; it walks the
// request's keys in tiles of 128 ABSOLUTE positions. Six warps:
//   warp 4 (one thread)  TMA: the Q tile once, then per tile the K pages and the V pages, each
//                        page one box of the cache's tensor map (128-byte swizzle, no multicast);
//   warp 5 (one thread)  tcgen05.mma: S = Q K^T into tensor memory, and, once the softmax
//                        warps have written P, O_tile = P V (V is read as an MN-major operand
//                        straight from its [key][d] page layout);
//   warps 0-3            softmax: a thread owns one query ROW: it reads its row of S from
//                        tensor memory (no shuffles for max or sum), masks on absolute positions,
//                        exponentiates in the exp2 domain in fp32, writes P as bf16 into shared
//                        memory in the swizzled K-major layout the tensor core reads. The output
//                        row stays in tensor memory over all the tiles (the products accumulate);
//                        it is in units of 2^m, where m follows the row's maximum lazily: only a
//                        maximum that exceeds m by more than 8 raises it, and only then is the row
//                        read, rescaled and written back.
// K and V are double-buffered in shared memory, S and P single. A CTA takes 256 columns of tensor
// memory (S 128, O head_dim), 113 KB of shared memory at head_dim 64 and 114 registers a thread (a
// row of S is read in two halves of 64, the first one twice: once for the maximum, once for the
// exponentials), so that TWO CTAs share an SM: while the softmax of one keeps the
// special-function unit busy, the other stores P or waits for the
// tensor core. Because tiles are cut at absolute
// positions and a row's running max and sum are its own, a row's result does not depend on how
// the prompt was cut or on what else is in the batch. Replaces flash_prefill_mma_kernel of the
// reference (src/kernels.cuh:1335-1482). Every wait is bounded.
#include "tc_common.cuh"

constexpr int FT_BM = 128, FT_BN = 128;
constexpr int FT_TILE = 128 * 64 * 2;  // one [128][64] bf16 tile: 16 KB; a [128][head_dim] operand is head_dim / 64 of them, 64 columns each

// MN-major operand with the 128-byte swizzle: 64 contiguous elements of the MN dimension per row,
// eight K rows per 1,024-byte group (stride SBO); further MN atoms would lie LBO apart (one here).
__device__ __forceinline__ uint64_t ft_desc_mn128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(FT_TILE >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor as hb_umma_idesc_bf16, with B read MN-major.
__host__ __device__ constexpr uint32_t ft_idesc_b_mn(int M, int N) { return hb_umma_idesc_bf16(M, N) | (1u << 16); }


struct FtBars {
  uint64_t q_full, k_full[2], k_free[2], v_full[2], v_free[2], s_full, s_free, o_full, p_full, p_free;
  uint32_t tmem_slot;
  int abort_flag;
};

// Buffers that alternate tile by tile: index i & 1, phase (i >> 1) & 1.
#define FT_B(i) ((i) & 1)
#define FT_PH(i) (((i) >> 1) & 1)

// head_dim 128: operands of two 64-column tiles each, the output tile 128 columns wide (192 KB of
// shared memory: one CTA per SM).
template <int FT_D>
__global__ void __launch_bounds__(FT_D == 64 ? 256 : 192, FT_D == 64 ? 2 : 1) flash_prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ bt, int bt_stride, const int* __restrict__ q_start,
    const int* __restrict__ q_len, const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, int Hq, int Hkv,
    int page_size, int window, float scale_log2, int min_rows, int* status) {
  // the 128-byte swizzle wants the tiles on 1 KB boundaries; with no room for slack (two CTAs an SM) the
  // dynamic shared memory itself has to start on one, which is checked below
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int NH = FT_D / 64, OPND = NH * FT_TILE;   // 64-column tiles and bytes of a [128][head_dim] operand
  uint8_t* sQ = smem;                  // [128][head_dim]
  uint8_t* sK = sQ + OPND;             // two stages of [128 keys][head_dim]
  uint8_t* sV = sK + 2 * OPND;         // two stages of [128 keys][head_dim]
  uint8_t* sP = sV + 2 * OPND;         // two K blocks of [128 rows][64 keys]
  FtBars* bar = (FtBars*)(sP + 2 * FT_TILE);
  volatile int* abort_flag = &bar->abort_flag;

  // the last query tiles of a portion have the most keys to walk: they are started first
  // blocks start in the order of blockIdx.x, then y: all heads' heaviest query tile first, then the next one
  // (longest work first: with the query tile fastest, the last head's heaviest tile would start last and run alone)
  const int req = blockIdx.z, hq = blockIdx.x, qt = gridDim.y - 1 - blockIdx.y;
  // the step's own metadata (lengths, tables) was copied before the step's first kernel began; everything else
  // that an earlier kernel wrote is read after hb_pdl_wait() below
  hb_pdl_launch();
  const int n_rows = q_len[req];
  if (n_rows < min_rows || qt * FT_BM >= n_rows) {
    if ((blockIdx.x | blockIdx.y | blockIdx.z) == 0) hb_pdl_wait();   // the grid never ends before the one ahead of it
    return;
  }
  if (hb_smem_u32(smem) & 1023) {   // never seen; the tiles would not be where the tensor core expects them
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = hq / (Hq / Hkv);
  const int row0 = q_start[req] + qt * FT_BM, rows_here = min(FT_BM, n_rows - qt * FT_BM);
  const int p_first = ctx_len[req] + qt * FT_BM, p_last = p_first + rows_here - 1;
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int kt_lo = lo / FT_BN, kt_hi = p_last / FT_BN, n_tiles = kt_hi - kt_lo + 1;
  const int* table = bt + (size_t)req * bt_stride;

  if (threadIdx.x == 0) {
    hb_mbar_init(&bar->q_full, 1);
    for (int b = 0; b < 2; b++) {
      hb_mbar_init(&bar->k_full[b], 1); hb_mbar_init(&bar->k_free[b], 1);
      hb_mbar_init(&bar->v_full[b], 1); hb_mbar_init(&bar->v_free[b], 1);
    }
    hb_mbar_init(&bar->o_full, 1);
    hb_mbar_init(&bar->p_full, 128); hb_mbar_init(&bar->p_free, 1);
    hb_mbar_init(&bar->s_full, 1); hb_mbar_init(&bar->s_free, 128);
    bar->abort_flag = 0;
    hb_fence_barrier_init();
  }
  // masked keys of a last, ragged tile are never loaded: what the tensor core reads in their place
  // must be finite (P is exactly 0 there, and 0 * NaN would poison the row)
  for (int i = threadIdx.x; i < 4 * OPND / 16; i += 192) ((uint4*)sK)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 5) {
    hb_tmem_alloc(&bar->tmem_slot, 256);
    hb_tmem_relinquish();
  }
  if (warp == 4 && lane == 0) { hb_tma_prefetch_desc(&map_q); hb_tma_prefetch_desc(&map_k); hb_tma_prefetch_desc(&map_v); }
  hb_fence_proxy_async();
  hb_tc_fence_before();
  __syncthreads();
  hb_tc_fence_after();
  const uint32_t tmem_s = bar->tmem_slot, tmem_o = tmem_s + FT_BN;  // S: 128 columns, O: head_dim columns
  hb_pdl_wait();   // barriers, shared and tensor memory were set up while the kernel ahead was still running

  if (warp == 4) {  // ---------------- TMA: lane l brings page l of the tile (the page ids come in one load)
    if (lane == 0) {
      hb_mbar_expect_tx(&bar->q_full, OPND);
#pragma unroll
      for (int hf = 0; hf < NH; hf++) hb_tma_load_2d(sQ + hf * FT_TILE, &map_q, &bar->q_full, hq * FT_D + hf * 64, row0);
    }
    for (int i = 0; i < n_tiles; i++) {
      const int k_base = (kt_lo + i) * FT_BN, b = FT_B(i);
      const int first_page = max(k_base, lo) / page_size, last_page = min(k_base + FT_BN - 1, p_last) / page_size;
      const int np = last_page - first_page + 1;
      const uint32_t bytes = (uint32_t)np * page_size * FT_D * 2;
      const int pg = first_page + lane;
      const int row = lane < np ? (table[pg] * Hkv + h) * page_size : 0;
      const int off = b * OPND + (pg * page_size - k_base) * 128;   // rows of 128 bytes in each 64-column tile
      int ok = 1;
      if (lane == 0) {
        ok = hb_mbar_wait(&bar->k_free[b], FT_PH(i) ^ 1, abort_flag);
        if (ok) hb_mbar_expect_tx(&bar->k_full[b], bytes);
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane < np) {
#pragma unroll
        for (int hf = 0; hf < NH; hf++) hb_tma_load_2d(sK + off + hf * FT_TILE, &map_k, &bar->k_full[b], hf * 64, row);
      }
      if (lane == 0) {
        ok = hb_mbar_wait(&bar->v_free[b], FT_PH(i) ^ 1, abort_flag);
        if (ok) hb_mbar_expect_tx(&bar->v_full[b], bytes);
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (lane < np) {
#pragma unroll
        for (int hf = 0; hf < NH; hf++) hb_tma_load_2d(sV + off + hf * FT_TILE, &map_v, &bar->v_full[b], hf * 64, row);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {  // ---------------- tensor cores: S_i is issued before O_{i-1}, so it overlaps the softmax of tile i - 1
      constexpr uint32_t idesc_s = hb_umma_idesc_bf16(FT_BM, FT_BN), idesc_o = ft_idesc_b_mn(FT_BM, FT_D);
      bool ok = hb_mbar_wait(&bar->q_full, 0, abort_flag);
      for (int i = 0; i <= n_tiles && ok; i++) {
        if (i < n_tiles) {
          const int b = FT_B(i);
          if (!hb_mbar_wait(&bar->k_full[b], FT_PH(i), abort_flag) || !hb_mbar_wait(&bar->s_free, (i & 1) ^ 1, abort_flag)) break;
          hb_tc_fence_after();
#pragma unroll
          for (int k = 0; k < FT_D / 16; k++) {   // 16 columns a step: four steps in each 64-column tile
            const uint64_t dq = hb_umma_desc_k128(hb_smem_u32(sQ + (k >> 2) * FT_TILE)) + 2 * (k & 3);
            const uint64_t dk = hb_umma_desc_k128(hb_smem_u32(sK + b * OPND + (k >> 2) * FT_TILE)) + 2 * (k & 3);
            hb_umma_bf16(tmem_s, dq, dk, idesc_s, k != 0);
          }
          hb_umma_commit(&bar->s_full);
          hb_umma_commit(&bar->k_free[b]);
        }
        if (i > 0) {
          const int j = i - 1, b = FT_B(j);
          if (!hb_mbar_wait(&bar->p_full, j & 1, abort_flag) || !hb_mbar_wait(&bar->v_full[b], FT_PH(j), abort_flag)) break;
          hb_tc_fence_after();
#pragma unroll
          for (int k = 0; k < FT_BN / 16; k++) {
            const uint64_t dp = hb_umma_desc_k128(hb_smem_u32(sP + (k >> 2) * FT_TILE)) + 2 * (k & 3);
            const uint64_t dv = ft_desc_mn128(hb_smem_u32(sV + b * OPND + k * 16 * 128));   // 16 keys on; the second 64 columns lie FT_TILE further (the descriptor's leading offset)
            hb_umma_bf16(tmem_o, dp, dv, idesc_o, j != 0 || k != 0);   // O stays in tensor memory over all the tiles
          }
          hb_umma_commit(&bar->o_full);
          hb_umma_commit(&bar->v_free[b]);
          hb_umma_commit(&bar->p_free);
        }
      }
    }
  } else {  // ---------------- softmax: thread = query row
    const int r = warp * 32 + lane;
    const int qp = p_first + min(r, rows_here - 1);  // rows past the portion's end are computed, never stored
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    // The output row accumulates in tensor memory over all the tiles, in units of 2^m_run. m_run follows the
    // row's maximum lazily: it is raised (and the row of O rescaled, which has to wait for the product of the
    // tile before) only when a tile's maximum exceeds it by more than FT_SLACK, so P <= 2^FT_SLACK; the sum
    // l_run is in the same units, and O / l_run is exact whichever maxima were used.
    constexpr float FT_SLACK = 8.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;   // every wait's outcome is made uniform over the warp: the tensor-memory accesses below are warp-wide
    for (int i = 0; i < n_tiles && ok; i++) {
      const int k_base = (kt_lo + i) * FT_BN;
      const bool need_mask = k_base + FT_BN - 1 > p_first || (window > 0 && k_base < p_last - window + 1);
      if (!__all_sync(0xffffffffu, hb_mbar_wait(&bar->s_full, i & 1, abort_flag))) { ok = false; break; }
      hb_tc_fence_after();
      // the row of S in two halves of 64 keys, the first one read twice (once for the maximum, once for the
      // exponentials): 128 registers a thread is all that lets a new CTA start beside one that is still
      // running (see the launch bounds). A softmax warp is alone on its scheduler: four independent chains
      // for the maximum and for the sum, and the mask only where one is needed
      uint32_t sr[64];
      const int hi_j = qp - k_base, lo_j = window > 0 ? qp - window - k_base : -1;  // key j of the tile is visible iff lo_j < j <= hi_j
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int hh = 0; hh < 2; hh++) {
        hb_tmem_ld64_nowait(tmem_s + lane_base + hh * 64, sr);
        hb_tmem_ld_wait();
        hb_tmem_ld_fence64(sr);
        if (need_mask) {
#pragma unroll
          for (int j = 0; j < 64; j++) {
            const float v = (j + hh * 64 <= hi_j && j + hh * 64 > lo_j) ? __uint_as_float(sr[j]) : -INFINITY;
            sr[j] = __float_as_uint(v);
            mx4[j & 3] = fmaxf(mx4[j & 3], v);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; j++) mx4[j & 3] = fmaxf(mx4[j & 3], __uint_as_float(sr[j]));
        }
      }
      const float m_tile = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const bool grow = m_tile > m_run + FT_SLACK;   // also the first tile with a visible key: m_run is -inf
      float corr = 1.f;
      if (grow) {
        corr = hb_exp2(m_run - m_tile);   // 0 while nothing has been summed
        m_run = m_tile;
      }
      const float sub = m_run == -INFINITY ? 0.f : m_run;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      // the exponentials: keys 64-127 are still in the registers (masked), keys 0-63 are read again
#pragma unroll
      for (int hh = 1; hh >= 0; hh--) {
        if (hh == 0) {
          hb_tmem_ld64_nowait(tmem_s + lane_base, sr);
          hb_tmem_ld_wait();
          hb_tmem_ld_fence64(sr);
          hb_tc_fence_before();
          hb_mbar_arrive(&bar->s_free);  // the last read of S: the scores of the next tile may overwrite it
          if (need_mask) {
#pragma unroll
            for (int j = 0; j < 64; j++)
              if (!(j <= hi_j && j > lo_j)) sr[j] = __float_as_uint(-INFINITY);
          }
        }
#pragma unroll
        for (int j = 0; j < 64; j += 2) {  // masked scores are -inf: 2^-inf = 0
          const float p0 = hb_exp2(fmaf(__uint_as_float(sr[j]), scale_log2, -sub));
          const float p1 = hb_exp2(fmaf(__uint_as_float(sr[j + 1]), scale_log2, -sub));
          sum4[(j >> 1) & 3] += p0 + p1;
          sr[j >> 1] = hb_pack_bf16(p0, p1);
        }
        if (hh == 1) {
          if (!__all_sync(0xffffffffu, hb_mbar_wait(&bar->p_free, (i & 1) ^ 1, abort_flag))) { ok = false; break; }
        }
        // 64 keys = eight 16-byte chunks of this row in K block hh of P
#pragma unroll
        for (int cc = 0; cc < 8; cc++) {
          const uint32_t dst = hb_smem_u32(sP + hh * FT_TILE) + r * 128 + ((cc ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(sr[4 * cc]), "r"(sr[4 * cc + 1]),
                       "r"(sr[4 * cc + 2]), "r"(sr[4 * cc + 3]) : "memory");
        }
      }
      if (!ok) break;
      l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      // a raised maximum: the rows of O so far, which the product of the tile before has to have finished writing
      // (it is the only one that can still be running: the scores of this tile were committed after the one before it)
      if (i > 0 && __any_sync(0xffffffffu, grow)) {
        if (!__all_sync(0xffffffffu, hb_mbar_wait(&bar->o_full, (i - 1) & 1, abort_flag))) { ok = false; break; }
        hb_tc_fence_after();
#pragma unroll
        for (int hf = 0; hf < NH; hf++) {
          hb_tmem_ld64_nowait(tmem_o + hf * 64 + lane_base, sr);
          hb_tmem_ld_wait();
          hb_tmem_ld_fence64(sr);
#pragma unroll
          for (int d = 0; d < 64; d++) sr[d] = __float_as_uint(__uint_as_float(sr[d]) * corr);
          hb_tmem_st64(tmem_o + hf * 64 + lane_base, sr);
        }
        hb_tmem_st_wait();
      }
      hb_tc_fence_before();
      hb_fence_proxy_async();
      hb_mbar_arrive(&bar->p_full);
    }
    if (ok && __all_sync(0xffffffffu, hb_mbar_wait(&bar->o_full, (n_tiles - 1) & 1, abort_flag))) {
      hb_tc_fence_after();
      const float inv = 1.f / l_run;
      __nv_bfloat16* dst = out + ((size_t)(row0 + r) * Hq + hq) * FT_D;
#pragma unroll
      for (int hf = 0; hf < NH; hf++) {
        uint32_t orr[64];
        hb_tmem_ld64_nowait(tmem_o + hf * 64 + lane_base, orr);
        hb_tmem_ld_wait();
        hb_tmem_ld_fence64(orr);
        if (r < rows_here) {
#pragma unroll
          for (int d = 0; d < 64; d += 8) {
            uint4 w;
            w.x = hb_pack_bf16(__uint_as_float(orr[d]) * inv, __uint_as_float(orr[d + 1]) * inv);
            w.y = hb_pack_bf16(__uint_as_float(orr[d + 2]) * inv, __uint_as_float(orr[d + 3]) * inv);
            w.z = hb_pack_bf16(__uint_as_float(orr[d + 4]) * inv, __uint_as_float(orr[d + 5]) * inv);
            w.w = hb_pack_bf16(__uint_as_float(orr[d + 6]) * inv, __uint_as_float(orr[d + 7]) * inv);
            *(uint4*)(dst + hf * 64 + d) = w;
          }
        }
      }
    }
  }

  hb_tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    __nanosleep(100000);
  }
  if (warp == 5) {
    __syncwarp();
    hb_tmem_dealloc(tmem_s, 256);
  }
}

HB_EXPORT int hb_flash_prefill_tc_supported(int Hq, int Hkv, int D, int page_size) {
  return Hkv > 0 && Hq % Hkv == 0 && (D == 64 || D == 128) && page_size >= 8 && page_size <= FT_BN && (page_size & (page_size - 1)) == 0;
}

// q, out [T, Hq, D] bf16; caches [num_pages, Hkv, page_size, D] bf16 (D 64 or 128); per request q_start, q_len,
// ctx_len and a block table row, as hb_flash_prefill. Requests with fewer than min_rows rows are
// skipped. `status` is set to 1 if a bounded wait ran out.
HB_EXPORT int hb_flash_prefill_tc(const void* q, const void* kc, const void* vc, long num_pages, const int* bt, int bt_stride,
                                  const int* q_start, const int* q_len, const int* ctx_len, void* out, int T, int R,
                                  int max_q_len, int Hq, int Hkv, int D, int page_size, int window, float scale,
                                  int min_rows, int* status, cudaStream_t st) {
  if (R <= 0 || max_q_len <= 0 || T <= 0) return 0;
  if (!hb_flash_prefill_tc_supported(Hq, Hkv, D, page_size))
    HB_FAIL("hb_flash_prefill_tc: %d/%d heads of %d with pages of %d are not supported", Hq, Hkv, D, page_size);
  if (R > 65535 || max_q_len > 65535 * FT_BM) HB_FAIL("hb_flash_prefill_tc: %d requests / portions of %d rows are beyond the grid limit", R, max_q_len);
  if (!status) HB_FAIL("hb_flash_prefill_tc: no status word");
  CUtensorMap mq, mk, mv;
  if (hb_make_tensor_map_bf16(&mq, q, (uint64_t)T, (uint64_t)Hq * D, (uint64_t)Hq * D, FT_BM)) return -1;
  const uint64_t rows = (uint64_t)num_pages * Hkv * page_size;
  if (hb_make_tensor_map_bf16(&mk, kc, rows, (uint64_t)D, (uint64_t)D, (uint32_t)page_size)) return -1;
  if (hb_make_tensor_map_bf16(&mv, vc, rows, (uint64_t)D, (uint64_t)D, (uint32_t)page_size)) return -1;
  dim3 grid(Hq, (max_q_len + FT_BM - 1) / FT_BM, R);
  const float sl2 = scale * 1.4426950408889634f;
  cudaError_t e;
  if (D == 64) {
    const size_t smem = 7 * (size_t)FT_TILE + sizeof(FtBars);   // 113 KB: two CTAs an SM
    static bool configured = false;
    if (!configured) {
      e = cudaFuncSetAttribute(flash_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) HB_FAIL("hb_flash_prefill_tc: %s", cudaGetErrorString(e));
      configured = true;
    }
    e = hb_launch(flash_prefill_tc_kernel<64>, grid, 192, smem, st, mq, mk, mv, bt, bt_stride, q_start, q_len, ctx_len,
                  (__nv_bfloat16*)out, Hq, Hkv, page_size, window, sl2, min_rows, status);
  } else {
    const size_t smem = 12 * (size_t)FT_TILE + sizeof(FtBars);  // Q, 2 K, 2 V of 32 KB each and P: 192 KB
    static bool configured = false;
    if (!configured) {
      e = cudaFuncSetAttribute(flash_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) HB_FAIL("hb_flash_prefill_tc: %s", cudaGetErrorString(e));
      configured = true;
    }
    e = hb_launch(flash_prefill_tc_kernel<128>, grid, 192, smem, st, mq, mk, mv, bt, bt_stride, q_start, q_len, ctx_len,
                  (__nv_bfloat16*)out, Hq, Hkv, page_size, window, sl2, min_rows, status);
  }
  if (e != cudaSuccess) HB_FAIL("hb_flash_prefill_tc: %s", cudaGetErrorString(e));
  HB_CHECK_LAUNCH("hb_flash_prefill_tc");
  return 0;
}
