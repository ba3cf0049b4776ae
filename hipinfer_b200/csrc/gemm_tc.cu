// C[M,N] = A[M,K] W[N,K]^T on the 5th-generation tensor cores: bf16 operands brought into
// shared memory by TMA (128-byte swizzle, K-major, no multicast), tcgen05.mma issued by one
// thread, fp32 accumulators in tensor memory, read back with tcgen05.ld for the epilogue.
//
// One persistent CTA per SM walks tiles of 128 x BN; six warps: 0-3 epilogue (each owns the
// 32 TMEM lanes it may touch), 4 the TMA producer, 5 the MMA issuer and TMEM owner. The
// accumulator is double-buffered in TMEM, so the epilogue of one tile overlaps the main loop
// of the next. K runs in blocks of 64 in ascending order for every tile: an output's value does
// not depend on M or on which tile it lies in.
//
// Epilogues: store fp32 / store bf16 / add into the fp32 residual stream (the reference's
// epilogue 1, src/kernels.cuh:881-889) / SwiGLU over gate and up columns interleaved in groups
// of 16 (its epilogue 2, src/kernels.cuh:850-863). Replaces gemm_mma_kernel (src/kernels.cuh:585).
// A fifth epilogue rotates a q/k/v product and writes q and the cache pages (EPI_ROPE_KV below).
// Every mbarrier wait is bounded; a wait that runs out raises the status word and the kernel
// drains and returns.
#include "tc_common.cuh"

enum { EPI_F32 = 0, EPI_BF16 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3, EPI_ROPE_KV = 4 };

// EPI_ROPE_KV: the product is a q/k/v projection of heads of 64; the epilogue rotates the q and k heads (half-split
// pairs (d, d + 32), the angles from a table of (cos, sin) per position) and writes q as bf16 [M, Hq * 64], k and v
// into their pages of the cache; nothing goes to C. What rope_kv_vec_kernel does from an fp32 copy of the product,
// product by product in the same fp32 operations (src/kernels.cuh:127-136, 1126-1150 rotate and store in one kernel too).
struct RopeEpi {
  const int* pos;         // [M] position of each row
  const int* slot_map;    // [M] page * page_size + offset of each row's token in the cache, -1: not stored; or null
  const float2* table;    // [positions][32] (cos, sin)
  __nv_bfloat16 *q_out, *kc, *vc;
  int Hq, Hkv, page_size;
};

constexpr int BM = 128, BK = 64;
#ifndef HB_GEMM_PAIR
#define HB_GEMM_PAIR 1
#endif
#ifndef HB_GEMM_TMA_STORE
#define HB_GEMM_TMA_STORE 1
#endif

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + slack to align the base to 1024
  // with the epilogue through TMA stores: two 32 x 32 fp32 boxes per epilogue warp, 1 KB aligned, after the barriers
  static constexpr int STAGING_OFFSET = (BAR_OFFSET + 256 + 1023) / 1024 * 1024;
  static constexpr int TOTAL_TS = STAGING_OFFSET + 4 * 2 * 4096 + 1024;
};

template <int EPI>
__device__ __forceinline__ void epilogue_store(const float* v, void* C, long ldc, int row, int col0, int M, int N) {
  // v: 32 consecutive columns col0.. of `row`
  if (row >= M) return;
  if (EPI == EPI_SWIGLU_BF16) {
    // columns [0,16) gate, [16,32) up of outputs (col0/2) .. +15
    __nv_bfloat16* out = (__nv_bfloat16*)C + (size_t)row * ldc + (col0 >> 1);
    const int n_out = N >> 1, o0 = col0 >> 1;
    __align__(16) __nv_bfloat16 r[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const float g = v[j], u = v[16 + j];
      r[j] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
    }
    if (o0 + 16 <= n_out && ((ldc & 7) == 0)) {
      *(uint4*)(out) = *(const uint4*)(r);
      *(uint4*)(out + 8) = *(const uint4*)(r + 8);
    } else {
      for (int j = 0; j < 16 && o0 + j < n_out; j++) out[j] = r[j];
    }
  } else if (EPI == EPI_BF16) {
    __nv_bfloat16* out = (__nv_bfloat16*)C + (size_t)row * ldc + col0;
    if (col0 + 32 <= N && ((ldc & 7) == 0)) {
      __align__(16) __nv_bfloat16 r[32];
#pragma unroll
      for (int j = 0; j < 32; j++) r[j] = __float2bfloat16_rn(v[j]);
#pragma unroll
      for (int j = 0; j < 4; j++) *(uint4*)(out + 8 * j) = *(const uint4*)(r + 8 * j);
    } else {
      for (int j = 0; j < 32 && col0 + j < N; j++) out[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* out = (float*)C + (size_t)row * ldc + col0;
    if (col0 + 32 <= N && ((ldc & 3) == 0)) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (EPI == EPI_ADD_F32) {
          const float4 c = *(const float4*)(out + 4 * j);
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        *(float4*)(out + 4 * j) = o;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < N; j++) out[j] = EPI == EPI_ADD_F32 ? out[j] + v[j] : v[j];
    }
  }
}

// One head of 64 columns of one row (x1: columns 0-31, x2: 32-63) of a q/k/v product: rotated if it is a q or k
// head, then 128 bytes of bf16 to q_out or to the row's place in the cache. The products and sums are single fp32
// operations in the order of rope_kv_vec_kernel, so both paths give the same bits.
__device__ __forceinline__ void rope_head_store(float* x1, float* x2, int head, int row, bool live, const float2* cs,
                                                int slot, const RopeEpi& rp) {
  __nv_bfloat16* dst = nullptr;
  if (head < rp.Hq) {
    dst = rp.q_out + ((size_t)row * rp.Hq + head) * 64;
  } else if (slot >= 0) {
    const size_t page = slot / rp.page_size, off = slot % rp.page_size;
    const bool is_k = head < rp.Hq + rp.Hkv;
    dst = (is_k ? rp.kc : rp.vc) + ((page * rp.Hkv + (head - rp.Hq - (is_k ? 0 : rp.Hkv))) * rp.page_size + off) * 64;
  }
  if (!live || !dst) return;
  if (head < rp.Hq + rp.Hkv) {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float4 c = *(const float4*)(cs + j);   // (cos, sin) of pairs j and j + 1
      const float a0 = x1[j], b0 = x2[j], a1 = x1[j + 1], b1 = x2[j + 1];
      x1[j] = __fsub_rn(__fmul_rn(a0, c.x), __fmul_rn(b0, c.y));
      x2[j] = __fadd_rn(__fmul_rn(b0, c.x), __fmul_rn(a0, c.y));
      x1[j + 1] = __fsub_rn(__fmul_rn(a1, c.z), __fmul_rn(b1, c.w));
      x2[j + 1] = __fadd_rn(__fmul_rn(b1, c.z), __fmul_rn(a1, c.w));
    }
  }
#pragma unroll
  for (int j = 0; j < 4; j++) {
    *(uint4*)(dst + 8 * j) = make_uint4(hb_pack_bf16(x1[8 * j], x1[8 * j + 1]), hb_pack_bf16(x1[8 * j + 2], x1[8 * j + 3]),
                                        hb_pack_bf16(x1[8 * j + 4], x1[8 * j + 5]), hb_pack_bf16(x1[8 * j + 6], x1[8 * j + 7]));
    *(uint4*)(dst + 32 + 8 * j) = make_uint4(hb_pack_bf16(x2[8 * j], x2[8 * j + 1]), hb_pack_bf16(x2[8 * j + 2], x2[8 * j + 3]),
                                             hb_pack_bf16(x2[8 * j + 4], x2[8 * j + 5]), hb_pack_bf16(x2[8 * j + 6], x2[8 * j + 7]));
  }
}

// 32 accumulator columns (chunk c of the tile at column n0) of 32 rows, one row a lane, through this warp's two
// 4 KB boxes of swizzled shared memory and out by a TMA tensor store (or reduce). PER chunks fill one box of
// 128-byte rows: 1 (fp32), 2 (bf16), 4 (SwiGLU: 16 outputs each). row0: the first of the warp's 32 rows in C.
template <int EPI>
__device__ __forceinline__ void ts_chunk(const float* v, int c, int n0, int N, int row0, uint8_t* boxes, int lane,
                                         const CUtensorMap* map_c) {
  constexpr int PER = EPI == EPI_SWIGLU_BF16 ? 4 : EPI == EPI_BF16 ? 2 : 1;
  uint8_t* box = boxes + ((c / PER) & 1) * 4096;
  if (c % PER == 0) {
    if (lane == 0) hb_tma_store_wait_read<1>();   // the store that last read this box is done with it
    __syncwarp();
  }
  const uint32_t b = hb_smem_u32(box) + lane * 128;
  if constexpr (EPI == EPI_SWIGLU_BF16) {
    uint32_t r[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float g0 = v[2 * j], g1 = v[2 * j + 1];
      r[j] = hb_pack_bf16(g0 / (1.f + __expf(-g0)) * v[16 + 2 * j], g1 / (1.f + __expf(-g1)) * v[17 + 2 * j]);
    }
#pragma unroll
    for (int j = 0; j < 2; j++)
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(b + ((((c % PER) * 2 + j) ^ (lane & 7)) << 4)),
                   "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3]) : "memory");
  } else if constexpr (EPI == EPI_BF16) {
#pragma unroll
    for (int j = 0; j < 4; j++)
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(b + ((((c % PER) * 4 + j) ^ (lane & 7)) << 4)),
                   "r"(hb_pack_bf16(v[8 * j], v[8 * j + 1])), "r"(hb_pack_bf16(v[8 * j + 2], v[8 * j + 3])),
                   "r"(hb_pack_bf16(v[8 * j + 4], v[8 * j + 5])), "r"(hb_pack_bf16(v[8 * j + 6], v[8 * j + 7])) : "memory");
  } else {
#pragma unroll
    for (int j = 0; j < 8; j++)
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(b + ((j ^ (lane & 7)) << 4)), "f"(v[4 * j]),
                   "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
  }
  if ((c + 1) % PER == 0 || n0 + (c + 1) * 32 >= N) {   // the box is full, or the tensor ends here
    hb_fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      // first column of the box in the output: accumulator column / 2 for SwiGLU
      const int x = EPI == EPI_SWIGLU_BF16 ? (n0 >> 1) + (c / PER) * 64 : n0 + (c / PER) * (PER * 32);
      if (EPI == EPI_ADD_F32) hb_tma_reduce_add_2d(map_c, box, x, row0);
      else hb_tma_store_2d(map_c, box, x, row0);
      hb_tma_store_commit();
    }
  }
}

// TS: results leave through shared memory and TMA: a warp writes 32 rows x 128 bytes in
// the 128-byte swizzle (no bank conflicts) and one lane sends the box as a tensor store, or,
// for the add into the residual stream, as a tensor REDUCE (the add happens at the memory side:
// the SM never reads C). Rows are whole 128-byte lines, and the next box is read from tensor
// memory while the last one is on its way.
template <int BN, int STAGES, int EPI, bool TS>
__global__ void __launch_bounds__(192, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                         const __grid_constant__ CUtensorMap map_w,
                                                         const __grid_constant__ CUtensorMap map_c, void* C, long ldc,
                                                         int M, int N, int K, int* status, const RopeEpi rp) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + S::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  hb_pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN, num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { hb_mbar_init(&full[s], 1); hb_mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; b++) { hb_mbar_init(&tmem_full[b], 1); hb_mbar_init(&tmem_empty[b], 4); }
    *abort_flag = 0;
    hb_fence_barrier_init();
  }
  if (warp == 5) {
    hb_tmem_alloc(tmem_slot, BN == 192 ? 512 : 2 * BN);   // a power of two
    hb_tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    hb_tma_prefetch_desc(&map_a);
    hb_tma_prefetch_desc(&map_w);
    if (TS) hb_tma_prefetch_desc(&map_c);
  }
  hb_tc_fence_before();
  __syncthreads();
  hb_tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  hb_pdl_wait();   // barriers and tensor memory were set up while the kernel ahead was still running

  if (warp == 4) {
    if (lane == 0) {  // ---------------- TMA producer
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!hb_mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          hb_mbar_expect_tx(&full[s], S::STAGE_BYTES);
          hb_tma_load_2d(smem + s * S::STAGE_BYTES, &map_a, &full[s], kb * BK, m0);
          hb_tma_load_2d(smem + s * S::STAGE_BYTES + S::A_BYTES, &map_w, &full[s], kb * BK, n0);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {  // ---------------- MMA issuer
      constexpr uint32_t idesc = hb_umma_idesc_bf16(BM, BN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tile_i++) {
        const uint32_t buf = tile_i & 1, aph = (tile_i >> 1) & 1;
        if (!hb_mbar_wait(&tmem_empty[buf], aph ^ 1, abort_flag)) break;
        hb_tc_fence_after();
        const uint32_t d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!hb_mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          hb_tc_fence_after();
          const uint64_t da = hb_umma_desc_k128(hb_smem_u32(smem + s * S::STAGE_BYTES));
          const uint64_t db = hb_umma_desc_k128(hb_smem_u32(smem + s * S::STAGE_BYTES + S::A_BYTES));
#pragma unroll
          for (int k = 0; k < BK / 16; k++) hb_umma_bf16(d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          hb_umma_commit(&empty[s]);
        }
        if (ok) hb_umma_commit(&tmem_full[buf]);
      }
    }
  } else {  // ---------------- epilogue warps 0..3
    uint32_t tile_i = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, tile_i++) {
      const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
      const uint32_t buf = tile_i & 1, aph = (tile_i >> 1) & 1;
      if (!hb_mbar_wait(&tmem_full[buf], aph, abort_flag)) break;
      hb_tc_fence_after();
      const int row = m0 + warp * 32 + lane;
      const uint32_t t0 = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BN;
      if constexpr (EPI == EPI_ROPE_KV) {
        const bool live = row < M;
        const float2* cs = rp.table + (size_t)(live ? rp.pos[row] : 0) * 32;
        const int slot = live && rp.slot_map ? rp.slot_map[row] : -1;
#pragma unroll 1
        for (int hd = 0; hd < BN / 64; hd++) {   // a head = two chunks of 32 columns
          float x1[32], x2[32];
          hb_tmem_ld32(t0 + hd * 64, x1);
          hb_tmem_ld32(t0 + hd * 64 + 32, x2);
          if (n0 + hd * 64 >= N) continue;
          rope_head_store(x1, x2, (n0 >> 6) + hd, row, live, cs, slot, rp);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
          float v[32];
          hb_tmem_ld32(t0 + c * 32, v);
          if (n0 + c * 32 >= N) continue;
          if constexpr (TS) {
            ts_chunk<EPI>(v, c, n0, N, m0 + warp * 32, smem + S::STAGING_OFFSET + warp * 8192, lane, &map_c);
          } else {
            epilogue_store<EPI>(v, C, ldc, row, n0 + c * 32, M, N);
          }
        }
      }
      hb_tc_fence_before();
      __syncwarp();
      if (lane == 0) hb_mbar_arrive(&tmem_empty[buf]);
    }
    if (TS && lane == 0) hb_tma_store_wait_all();   // before the shared memory is given up and the kernel ends
  }

  hb_tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    __nanosleep(100000);  // let copies that may still be in flight land before the shared memory is given up
  }
  if (warp == 5) {
    __syncwarp();
    hb_tmem_dealloc(tmem_base, BN == 192 ? 512 : 2 * BN);
  }
}

// ---------------------------------------------------------------------------------------
// The same product by CTA PAIRS (clusters of two, cta_group::2): a pair works on a 256 x 256
// tile; each CTA loads its 128 rows of A and its 128 of the tile's 256 weight rows (the tensor
// cores read the other half from the partner's shared memory, so a CTA moves 32 KB of operands
// per 64-deep block instead of 48 KB), and holds its 128 rows of the accumulator in its own
// tensor memory. One thread of the even CTA issues the MMAs; its commits arrive on the barriers
// of both CTAs; the loaders of both CTAs count their bytes on the even CTA's barriers; the odd
// CTA's epilogue warps free the accumulator by arriving on the even CTA's barrier. Results
// leave through the TMA-store epilogue. K runs in blocks of 64 in ascending order as above.
// ---------------------------------------------------------------------------------------
template <int STAGES>
struct PairSmem {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = 128 * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int STAGING_OFFSET = (BAR_OFFSET + 256 + 1023) / 1024 * 1024;
  static constexpr int TOTAL = STAGING_OFFSET + 4 * 2 * 4096 + 1024;
};

template <int STAGES, int EPI>
__global__ void __launch_bounds__(192, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                              const __grid_constant__ CUtensorMap map_w,
                                                              const __grid_constant__ CUtensorMap map_c, int M, int N, int K,
                                                              int* status) {
  using S = PairSmem<STAGES>;
  constexpr int BN = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // the same offset in both CTAs
  uint64_t* full = (uint64_t*)(smem + S::BAR_OFFSET);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  hb_pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = hb_cluster_ctarank();                 // 0: issues the MMAs, owns the barriers the loads count on
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (M + 255) / 256, n_tiles = (N + BN - 1) / BN, num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { hb_mbar_init(&full[s], 1); hb_mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; b++) { hb_mbar_init(&tmem_full[b], 1); hb_mbar_init(&tmem_empty[b], 8); }   // four epilogue warps of each CTA
    *abort_flag = 0;
    hb_fence_barrier_init();
  }
  if (warp == 5) {
    hb_tmem_alloc_pair(tmem_slot, 512);
    hb_tmem_relinquish_pair();
  }
  if (warp == 4 && lane == 0) { hb_tma_prefetch_desc(&map_a); hb_tma_prefetch_desc(&map_w); hb_tma_prefetch_desc(&map_c); }
  hb_tc_fence_before();
  __syncthreads();
  hb_cluster_sync();   // the partner's barriers exist before anything is signalled across
  hb_tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  hb_pdl_wait();

  if (warp == 4) {
    if (lane == 0) {  // ---------------- TMA producer of this CTA's halves
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        const int m0 = (tile % m_tiles) * 256 + rank * 128, n0 = (tile / m_tiles) * BN + rank * 128;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!hb_mbar_wait(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          if (rank == 0) hb_mbar_expect_tx(&full[s], 2 * S::STAGE_BYTES);   // both CTAs' bytes
          const uint32_t bar = hb_mapa(&full[s], 0);
          hb_tma_load_2d_pair(smem + s * S::STAGE_BYTES, &map_a, bar, kb * BK, m0);
          hb_tma_load_2d_pair(smem + s * S::STAGE_BYTES + S::A_BYTES, &map_w, bar, kb * BK, n0);
        }
      }
      // the last commits still arrive on this CTA's barriers: wait for them before the shared memory is given up
      for (uint32_t j = it > STAGES ? it - STAGES : 0; j < it && ok; j++)
        ok = hb_mbar_wait(&empty[j % STAGES], (j / STAGES) & 1, abort_flag);
    }
  } else if (warp == 5) {
    if (lane == 0 && rank == 0) {  // ---------------- MMA issuer of the pair
      constexpr uint32_t idesc = hb_umma_idesc_bf16(256, BN);
      uint32_t it = 0, tile_i = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs, tile_i++) {
        const uint32_t buf = tile_i & 1, aph = (tile_i >> 1) & 1;
        if (!hb_mbar_wait(&tmem_empty[buf], aph ^ 1, abort_flag)) break;
        hb_tc_fence_after();
        const uint32_t d = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!hb_mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          hb_tc_fence_after();
          const uint64_t da = hb_umma_desc_k128(hb_smem_u32(smem + s * S::STAGE_BYTES));
          const uint64_t db = hb_umma_desc_k128(hb_smem_u32(smem + s * S::STAGE_BYTES + S::A_BYTES));
#pragma unroll
          for (int k = 0; k < BK / 16; k++) hb_umma_bf16_pair(d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          hb_umma_commit_pair(&empty[s]);
        }
        if (ok) hb_umma_commit_pair(&tmem_full[buf]);
      }
    }
  } else {  // ---------------- epilogue warps 0..3: this CTA's 128 rows of the tile
    uint32_t tile_i = 0;
    for (int tile = pair; tile < num_tiles; tile += n_pairs, tile_i++) {
      const int m0 = (tile % m_tiles) * 256 + rank * 128, n0 = (tile / m_tiles) * BN;
      const uint32_t buf = tile_i & 1, aph = (tile_i >> 1) & 1;
      if (!hb_mbar_wait(&tmem_full[buf], aph, abort_flag)) break;
      hb_tc_fence_after();
      const uint32_t t0 = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        float v[32];
        hb_tmem_ld32(t0 + c * 32, v);
        if (n0 + c * 32 >= N) continue;
        ts_chunk<EPI>(v, c, n0, N, m0 + warp * 32, smem + S::STAGING_OFFSET + warp * 8192, lane, &map_c);
      }
      hb_tc_fence_before();
      __syncwarp();
      if (lane == 0) hb_mbar_arrive_remote(hb_mapa(&tmem_empty[buf], 0));
    }
    if (lane == 0) hb_tma_store_wait_all();
  }

  hb_tc_fence_before();
  __syncthreads();
  hb_cluster_sync();   // neither CTA leaves while the other may still signal it or read its shared memory
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    __nanosleep(100000);
  }
  if (warp == 5) {
    __syncwarp();
    hb_tmem_dealloc_pair(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int hb_make_tensor_map_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                            uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) HB_FAIL("cuTensorMapEncodeTiled is not available from this driver");
  if (((uintptr_t)base & 15) || (row_stride_elems * 2) % 16)
    HB_FAIL("tensor map: base %p and row stride %llu elements must be 16-byte aligned", base,
            (unsigned long long)row_stride_elems);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_elems * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) HB_FAIL("cuTensorMapEncodeTiled failed with code %d (rows %llu, cols %llu)", (int)r,
                                 (unsigned long long)rows, (unsigned long long)cols);
  return 0;
}

// A 2-D fp32 tensor map [rows, cols] with a box of 32 x 32 (128-byte rows) and the 128-byte swizzle: for stores.
static int hb_make_tensor_map_f32_box32(CUtensorMap* out, void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) HB_FAIL("cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_elems * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) HB_FAIL("cuTensorMapEncodeTiled (fp32 output) failed with code %d (rows %llu, cols %llu)", (int)r,
                                 (unsigned long long)rows, (unsigned long long)cols);
  return 0;
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, int STAGES, int EPI, bool TS>
static int launch_gemm_tc_ts(const CUtensorMap& ma, const CUtensorMap& mw, const CUtensorMap& mc, void* C, long ldc, int M,
                             int N, int K, int* status, cudaStream_t s, const RopeEpi& rp = RopeEpi()) {
  using S = GemmSmem<BN, STAGES>;
  constexpr int smem = TS ? S::TOTAL_TS : S::TOTAL;
  auto kern = gemm_tc_kernel<BN, STAGES, EPI, TS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaError_t e = hb_launch(kern, grid, 192, smem, s, ma, mw, mc, C, ldc, M, N, K, status, rp);
  if (e != cudaSuccess) HB_FAIL("hb_gemm_tc: %s", cudaGetErrorString(e));
  return 0;
}

// fp32 results go out through TMA stores where C allows it (16-byte aligned base and rows)
template <int BN, int STAGES, int EPI>
static int launch_gemm_tc(const CUtensorMap& ma, const CUtensorMap& mw, void* C, long ldc, int M, int N, int K,
                          int* status, cudaStream_t s) {
  CUtensorMap mc;
  memset(&mc, 0, sizeof(mc));
  if constexpr (EPI == EPI_F32 || EPI == EPI_ADD_F32) {
    if (HB_GEMM_TMA_STORE && !((uintptr_t)C & 15) && (ldc & 3) == 0) {
      if (hb_make_tensor_map_f32_box32(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc)) return -1;
      return launch_gemm_tc_ts<BN, STAGES, EPI, true>(ma, mw, mc, C, ldc, M, N, K, status, s);
    }
  } else {
    if (HB_GEMM_TMA_STORE && !((uintptr_t)C & 15) && (ldc & 7) == 0) {   // bf16 [M, N] or [M, N / 2]: boxes of 32 rows x 64 columns
      const uint64_t cols = EPI == EPI_SWIGLU_BF16 ? (uint64_t)N / 2 : (uint64_t)N;
      if (hb_make_tensor_map_bf16(&mc, C, (uint64_t)M, cols, (uint64_t)ldc, 32)) return -1;
      return launch_gemm_tc_ts<BN, STAGES, EPI, true>(ma, mw, mc, C, ldc, M, N, K, status, s);
    }
  }
  return launch_gemm_tc_ts<BN, STAGES, EPI, false>(ma, mw, mc, C, ldc, M, N, K, status, s);
}

// The CTA-pair kernel: C must be addressable by TMA stores (16-byte aligned base and rows).
template <int EPI>
static int launch_gemm_pair(const CUtensorMap& ma, const void* W, long ldw, void* C, long ldc, int M, int N, int K, int* status,
                            cudaStream_t s) {
  using S = PairSmem<6>;
  CUtensorMap mw, mc;
  if (hb_make_tensor_map_bf16(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128)) return -1;
  if (EPI == EPI_F32 || EPI == EPI_ADD_F32) {
    if (((uintptr_t)C & 15) || (ldc & 3)) HB_FAIL("hb_gemm_tc: the CTA-pair kernel needs a 16-byte aligned C");
    if (hb_make_tensor_map_f32_box32(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc)) return -1;
  } else {
    if (((uintptr_t)C & 15) || (ldc & 7)) HB_FAIL("hb_gemm_tc: the CTA-pair kernel needs a 16-byte aligned C");
    const uint64_t cols = EPI == EPI_SWIGLU_BF16 ? (uint64_t)N / 2 : (uint64_t)N;
    if (hb_make_tensor_map_bf16(&mc, C, (uint64_t)M, cols, (uint64_t)ldc, 32)) return -1;
  }
  auto kern = gemm_tc_pair_kernel<6, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) HB_FAIL("hb_gemm_tc: %s", cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256), pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  cudaError_t e = hb_launch_cluster(kern, dim3(2 * pairs), 192, S::TOTAL, s, dim3(2, 1, 1), ma, mw, mc, M, N, K, status);
  if (e != cudaSuccess) HB_FAIL("hb_gemm_tc: %s", cudaGetErrorString(e));
  return 0;
}

template <int BN, int STAGES>
static int dispatch_epi(int epi, const CUtensorMap& ma, const CUtensorMap& mw, void* C, long ldc, int M, int N, int K,
                        int* status, cudaStream_t s) {
  switch (epi) {
    case EPI_F32: return launch_gemm_tc<BN, STAGES, EPI_F32>(ma, mw, C, ldc, M, N, K, status, s);
    case EPI_BF16: return launch_gemm_tc<BN, STAGES, EPI_BF16>(ma, mw, C, ldc, M, N, K, status, s);
    case EPI_ADD_F32: return launch_gemm_tc<BN, STAGES, EPI_ADD_F32>(ma, mw, C, ldc, M, N, K, status, s);
    case EPI_SWIGLU_BF16: return launch_gemm_tc<BN, STAGES, EPI_SWIGLU_BF16>(ma, mw, C, ldc, M, N, K, status, s);
  }
  HB_FAIL("hb_gemm_tc: unknown epilogue %d", epi);
}

// C (+)= A W^T. A [M, K] bf16 (row stride lda), W [N, K] bf16 (row stride ldw); C per `epi`:
// 0 fp32 [M, N], 1 bf16 [M, N], 2 fp32 += , 3 bf16 [M, N/2] = SwiGLU over 16-interleaved gate/up
// columns. `status` is a device-visible word that is set to 1 if a wait ran out.
// tile_n: 128, 192 (fp32 results) or 256; 512: 256 x 256 tiles by CTA pairs; 0: chosen from M, N and C's alignment.
// An output's value is the same whichever is taken.
HB_EXPORT int hb_gemm_tc(const void* A, long lda, const void* W, long ldw, void* C, long ldc, int M, int N, int K,
                         int epi, int tile_n, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7)) HB_FAIL("hb_gemm_tc: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  if (epi == EPI_SWIGLU_BF16 && (N & 31)) HB_FAIL("hb_gemm_tc: SwiGLU needs N = %d to be a multiple of 32", N);
  if (!status) HB_FAIL("hb_gemm_tc: no status word");
  if (tile_n == 0) {
    // 128 x 256 tiles feed the tensor cores best (a narrower tile reads more operand bytes per flop: measured
    // 1.1 times the time per column at 192, 1.35 times at 128); a narrower one is taken when it fills the
    // SMs' rounds better. An output's value is the same for every tile width.
    const long mt = (M + BM - 1) / BM, sms = sm_count();
    auto cost = [&](int bn, double per_col) { return (double)((mt * ((N + bn - 1) / bn) + sms - 1) / sms) * bn * per_col; };
    tile_n = 256;
    double best = cost(256, 1.0);
    if ((epi == EPI_F32 || epi == EPI_ADD_F32) && cost(192, 1.1) < best) { tile_n = 192; best = cost(192, 1.1); }
    if (cost(128, 1.35) < best) tile_n = 128;
    // where the 256-wide tile is the choice, CTA pairs on 256 x 256 tiles do the same work with a third less
    // operand traffic per CTA (measured 0 to 14 % faster, never slower), given two row halves and a C that TMA can store to
    const bool c_ok = !((uintptr_t)C & 15) && (ldc & ((epi == EPI_F32 || epi == EPI_ADD_F32) ? 3 : 7)) == 0;
    if (HB_GEMM_PAIR && tile_n == 256 && M > 128 && c_ok) tile_n = 512;
  }
  if (tile_n == 512) {   // 256 x 256 tiles by CTA pairs
    CUtensorMap ma;
    if (hb_make_tensor_map_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return -1;
    int r;
    switch (epi) {
      case EPI_F32: r = launch_gemm_pair<EPI_F32>(ma, W, ldw, C, ldc, M, N, K, status, s); break;
      case EPI_BF16: r = launch_gemm_pair<EPI_BF16>(ma, W, ldw, C, ldc, M, N, K, status, s); break;
      case EPI_ADD_F32: r = launch_gemm_pair<EPI_ADD_F32>(ma, W, ldw, C, ldc, M, N, K, status, s); break;
      case EPI_SWIGLU_BF16: r = launch_gemm_pair<EPI_SWIGLU_BF16>(ma, W, ldw, C, ldc, M, N, K, status, s); break;
      default: HB_FAIL("hb_gemm_tc: unknown epilogue %d", epi);
    }
    if (r) return r;
    HB_CHECK_LAUNCH("hb_gemm_tc");
    return 0;
  }
  if (tile_n != 128 && tile_n != 256 && !(tile_n == 192 && (epi == EPI_F32 || epi == EPI_ADD_F32)))
    HB_FAIL("hb_gemm_tc: tile_n must be 128 or 256 (or 192 with an fp32 result, or 512 for CTA pairs)");
  CUtensorMap ma, mw;
  if (hb_make_tensor_map_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return -1;
  if (hb_make_tensor_map_bf16(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)tile_n)) return -1;
  int r;
  if (tile_n == 256) r = dispatch_epi<256, 4>(epi, ma, mw, C, ldc, M, N, K, status, s);
  else if (tile_n == 128) r = dispatch_epi<128, 6>(epi, ma, mw, C, ldc, M, N, K, status, s);
  else r = epi == EPI_F32 ? launch_gemm_tc<192, 4, EPI_F32>(ma, mw, C, ldc, M, N, K, status, s)
                          : launch_gemm_tc<192, 4, EPI_ADD_F32>(ma, mw, C, ldc, M, N, K, status, s);
  if (r) return r;
  HB_CHECK_LAUNCH("hb_gemm_tc");
  return 0;
}

// q/k/v projection with rotation and cache write in the epilogue (EPI_ROPE_KV): A [M, K] bf16, W [(Hq + 2 Hkv) * 64, K]
// bf16 with the rows q heads, k heads, v heads; pos [M]; slot_map [M] or null (then only q is written); table
// [positions][32] (cos, sin) fp32; q_out [M, Hq * 64] bf16; caches [pages, Hkv, page_size, 64] bf16. Heads of 64 only.
HB_EXPORT int hb_gemm_tc_rope_kv(const void* A, long lda, const void* W, long ldw, int M, int K, const int* pos,
                                 const int* slot_map, const void* table, void* q_out, void* kc, void* vc, int Hq, int Hkv,
                                 int D, int page_size, int* status, cudaStream_t s) {
  if (M <= 0) return 0;
  if (D != 64) HB_FAIL("hb_gemm_tc_rope_kv: heads of %d (64 only)", D);
  if (Hq <= 0 || Hkv <= 0 || page_size <= 0) HB_FAIL("hb_gemm_tc_rope_kv: %d/%d heads, pages of %d", Hq, Hkv, page_size);
  if (K <= 0 || (K & 7)) HB_FAIL("hb_gemm_tc_rope_kv: K = %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
  if (!status || !pos || !table || !q_out) HB_FAIL("hb_gemm_tc_rope_kv: a null argument");
  if (slot_map && (!kc || !vc)) HB_FAIL("hb_gemm_tc_rope_kv: a slot map without caches");
  if (((uintptr_t)q_out | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)table) & 15) HB_FAIL("hb_gemm_tc_rope_kv: q, caches and table must be 16-byte aligned");
  const int N = (Hq + 2 * Hkv) * 64;
  CUtensorMap ma, mw, mc;
  memset(&mc, 0, sizeof(mc));
  if (hb_make_tensor_map_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return -1;
  if (hb_make_tensor_map_bf16(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 192)) return -1;
  RopeEpi rp;
  rp.pos = pos; rp.slot_map = slot_map; rp.table = (const float2*)table;
  rp.q_out = (__nv_bfloat16*)q_out; rp.kc = (__nv_bfloat16*)kc; rp.vc = (__nv_bfloat16*)vc;
  rp.Hq = Hq; rp.Hkv = Hkv; rp.page_size = page_size;
  if (launch_gemm_tc_ts<192, 4, EPI_ROPE_KV, false>(ma, mw, mc, nullptr, 0, M, N, K, status, s, rp)) return -1;
  HB_CHECK_LAUNCH("hb_gemm_tc_rope_kv");
  return 0;
}
