// Products of a FEW token rows (1 to 16: decode steps of small batches, short portions) with a
// weight matrix, in the shape the reference gives its decode GEMVs (src/kernels.cuh:164-281:
// norm in the prologue, rotation + cache write / residual add / SwiGLU in the epilogue, no split
// of K), so that a decoder layer is five kernels: q/k/v, attention, o, gate/up, down.
//
// A block owns whole output rows: a tile of 16 weight rows over ALL of K, so nothing is summed
// across blocks and the epilogue finishes the job: no partial sums in memory, no reduction
// kernel, no second pass over the residual. Every weight byte is read from HBM once, by the
// bulk-copy engine (cp.async.bulk: one copy of 2 KB per weight row and K chunk, into padded rows
// of shared memory so that the 16-byte fragment loads meet no bank twice), through a ring of
// stages. The 32 lanes of one producer warp issue the copies, a lane per row, each with its
// addresses in registers: measured on this GPU, one thread that loops over a stage's copies
// (or divides to find an address) hands the engine a copy every 45 ns, a third of what HBM
// delivers, and copies of 1 KB stay at 4 TB/s however they are issued. The ring is filled
// BEFORE the kernel waits for the kernel ahead of it (weights do not depend on it), so under
// programmatic dependent launch the weights of a product stream in while the one before it
// still runs; the norm's weight is staged in shared memory before the wait as well. Four
// consumer warps split a chunk's K among them and multiply with warp MMAs (m16n8k16, bf16 in,
// fp32 accumulate: the weight rows are the MMA's M side, the 8 or 16 token rows its N side);
// the op is bound by HBM, its arithmetic is a few hundred MMAs a block (21 cycles of latency
// and 8 cycles an MMA here, measured). The warps' sums meet in shared memory, added in warp order.
//
// Input modes.  A_BF16: the token rows are bf16 activations and stream through the ring beside
// the weights (lanes 16.. of the producer warp).  A_NORM: the token rows are the fp32 residual
// stream; all eight warps compute their RMSNorm (sum of squares, rsqrt, times the norm's weight,
// all in fp32, rounded once to bf16) into shared memory after the wait, a warp per row, every
// load of a row in flight at once. Each block reads M x K floats from L2 for that, which is why
// this path ends at 16 rows.
//
// Tiles and epilogues.  A tile's rows 8..15 are the partners of its rows 0..7, and the MMA
// thread that holds accumulator row g also holds row g + 8:  ROPE_KV: the rows are
// [q heads; k heads; v heads] of a fused projection; a tile holds 8 dimensions j of one head and
// their rotation partners j + D/2, turns q and k by the row's (cos, sin) and writes q and the
// row's place in the K and V pages.  SWIGLU: 8 gate rows and their 8 up rows (the matrix
// alternates 16 gate and 16 up rows): out (bf16) = silu(gate) * up.  ADD: 16 consecutive rows,
// out (fp32) += .  Tile t walks its chunks of K starting at chunk t % chunks (blocks that run
// side by side read different columns).
// A token's result depends on its own row alone (its column of the MMA), never on the batch,
// and is the same bits among 8 and among 16 rows. All waits are bounded.
#include "tc_common.cuh"

HB_TL_DEFINE(rows)

enum { RW_A_BF16 = 0, RW_A_NORM = 1, RW_A_SCALED = 2 };
enum { RW_ROPE_KV = 0, RW_ADD = 1, RW_SWIGLU = 2 };
constexpr int RW_R = 16;                         // weight rows of a tile: one m16 MMA tile
constexpr int RW_KC = 1024;                      // K elements of a stage: a copy brings 2 KB of one row
constexpr int RW_PAD = 64;                       // a row's stride is 16 words beyond a multiple of 32: 16-byte fragment loads of eight rows meet no bank twice
constexpr int RW_ROWB = RW_KC * 2 + RW_PAD;      // bytes of a padded row of a stage
constexpr int RW_CONSUMERS = 4, RW_WARPS = 8, RW_THREADS = RW_WARPS * 32;   // warps 0..3 multiply, warp 4 issues the copies; all eight normalise

struct RowsArgs {
  const void* A; long lda;               // A_BF16: bf16 [M, K]; A_NORM: fp32 residual [M, K]
  const __nv_bfloat16* norm_w; float eps;
  const __nv_bfloat16* W; long ldw;
  int M, N, K, n_tiles, stages;
  void* out; long ldo;                   // ADD: fp32 [M, N]; SWIGLU: bf16 [M, N / 2]
  const int* pos; const int* slot_map; const float2* table;   // ROPE_KV
  __nv_bfloat16 *q_out, *kc, *vc;
  int Hq, Hkv, D, page_size;
  int* status;
  // ADD, optional: what the NEXT norm's consumer wants, made while the new residual values are in registers:
  // xb [M, N] bf16 = x_new * next_w (not yet divided by the row's RMS), ssq_part [N / 16][16] = each tile's share of sum(x_new^2)
  const __nv_bfloat16* next_w; __nv_bfloat16* xb; long ldxb; float* ssq_part;
  // A_SCALED: A is such an xb; the row's 1 / RMS comes from ssq_part (n_parts tiles) and is applied in the epilogue
  int n_parts;
};

__device__ __forceinline__ void rw_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(hb_smem_u32(dst)), "l"((uint64_t)src), "r"(bytes), "r"(hb_smem_u32(bar)) : "memory");
}
// D[16x8] += A[16x16] B[16x8], bf16 in, fp32 accumulate. Not volatile: the compiler is free to move the fragment
// loads of later steps ahead of it.
__device__ __forceinline__ void rw_mma(float* d, const uint32_t* a, const uint32_t* b) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void rw_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(RW_CONSUMERS * 32) : "memory"); }

// Weight row that row r (0..15) of tile t holds. ADD: 16 consecutive rows. ROPE_KV: the rotation pairs of 8 dimensions of
// one head, rows 0..7 the dimensions j0.., rows 8..15 their partners j0 + D/2... SWIGLU: 8 gate rows and, as rows 8..15,
// their 8 up rows (the matrix alternates 16 gate rows and 16 up rows). Either way the thread of an MMA that holds
// accumulator row g also holds row g + 8: the pair meets in one thread.
template <int EPI>
__device__ __forceinline__ long rw_row(const RowsArgs& a, int t, int r) {
  if constexpr (EPI == RW_ROPE_KV) {
    const int per_head = a.D >> 4, hh = t / per_head, j0 = (t - hh * per_head) * 8;
    return (long)hh * a.D + j0 + (r & 7) + (r >> 3) * (a.D >> 1);
  } else if constexpr (EPI == RW_SWIGLU) {
    return (long)(t >> 1) * 32 + (t & 1) * 8 + (r & 7) + (r >> 3) * 16;
  } else {
    return (long)t * RW_R + r;
  }
}

template <int MT, int A_MODE, int EPI>
__global__ void __launch_bounds__(RW_THREADS, 2) rows_product_kernel(const RowsArgs a) {
  constexpr int NTILES = MT / 8;
  constexpr bool STREAM_A = A_MODE == RW_A_BF16;     // the token rows come through the ring; else they lie in shared memory (xs)
  constexpr int W_STAGE = RW_R * RW_ROWB, A_STAGE = STREAM_A ? MT * RW_ROWB : 0, STAGE = W_STAGE + A_STAGE;
  extern __shared__ __align__(128) uint8_t smem[];
  const int stages = a.stages;
  uint8_t* ring = smem;
  float* red = (float*)(smem + (size_t)stages * STAGE);                        // [consumers][16][MT]
  uint8_t* xs = (uint8_t*)(red + RW_CONSUMERS * RW_R * MT);                    // A_NORM, A_SCALED: [MT][K * 2 + 64]
  const int xs_rowb = a.K * 2 + RW_PAD;
  uint8_t* wsm = xs + (!STREAM_A ? (size_t)MT * xs_rowb : 0);                 // A_NORM: the norm's weight, [K] bf16
  uint64_t* full = (uint64_t*)(wsm + (A_MODE == RW_A_NORM ? (size_t)a.K * 2 : 0));
  uint64_t* empty = full + stages;
  uint64_t* xbar = empty + stages;                                            // A_SCALED: the token rows have arrived in xs
  uint64_t* rbar = xbar + 1;                                                  // A_SCALED: rs is written
  __shared__ int abort_word;
  __shared__ float rs[16];               // A_SCALED: 1 / RMS of the token rows
  volatile int* abort_flag = &abort_word;

  hb_pdl_launch();
  HB_TL_MARK(EPI * 3 + 0, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunks = (a.K + RW_KC - 1) / RW_KC;
  const int my_tiles = blockIdx.x < a.n_tiles ? (a.n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
  const int total = my_tiles * chunks;                                         // (tile, chunk) units of this block, in order
  const bool producer = warp == RW_CONSUMERS;
  // Lane r < 16 of the producer warp brings weight row r of every unit, lane 16 + m activation row m (A_BF16). A copy is
  // one instruction of one lane with everything it needs in registers: a thread that loops over a stage's copies, or
  // divides to find its addresses, hands the copy engine far less than the memory can deliver (measured: 2 to 3 TB/s).
  constexpr int ARRIVALS = STREAM_A ? 32 : 16;
  const bool w_lane = lane < RW_R, a_lane = STREAM_A && lane >= 16 && lane - 16 < a.M;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; s++) { hb_mbar_init(&full[s], ARRIVALS); hb_mbar_init(&empty[s], RW_CONSUMERS); }
    hb_mbar_init(xbar, 1);
    hb_mbar_init(rbar, RW_WARPS - RW_CONSUMERS - 1);
    *abort_flag = 0;
    hb_fence_barrier_init();
  }
  if constexpr (A_MODE == RW_A_NORM)      // the norm's weight is a constant: it is in shared memory before the wait
    for (int i = threadIdx.x; i < (a.K >> 3); i += RW_THREADS) ((uint4*)wsm)[i] = __ldg((const uint4*)a.norm_w + i);
  __syncthreads();

  // producer state: the unit (tile index ti, chunk c) it issues next, its stage and that stage's parity
  int p_ti = 0, p_c = 0, p_s = 0, p_par = 0, p_u = 0, p_first = 0;
  const uint8_t* p_src = nullptr;       // this lane's row of the current tile (weights) or of the activations
  bool p_valid = false;
  auto p_tile = [&]() {                 // called when a tile begins
    const int t = blockIdx.x + p_ti * gridDim.x;
    p_first = t % chunks;               // the chunk order turns with the tile (see the consumers)
    if (w_lane) {
      const long row = rw_row<EPI>(a, t, lane);
      p_valid = row < a.N;
      p_src = (const uint8_t*)(a.W + row * a.ldw);
    }
  };
  if (producer) {
    if (a_lane) { p_valid = true; p_src = (const uint8_t*)((const __nv_bfloat16*)a.A + (long)(lane - 16) * a.lda); }
    p_tile();
  }
  // Issues this lane's copy of the current unit (arming the stage's barrier for its bytes first) when `mine`, and
  // moves on to the next unit either way.
  auto p_issue = [&](bool mine, bool arrive) {
    int cc = p_c + p_first;
    if (cc >= chunks) cc -= chunks;
    const int k0 = cc * RW_KC;
    const uint32_t bytes = (uint32_t)(min(RW_KC, a.K - k0) * 2);
    if (arrive) {
      if (mine && p_valid) {
        hb_mbar_expect_tx(&full[p_s], bytes);
        rw_bulk_load(ring + (size_t)p_s * STAGE + (w_lane ? lane * RW_ROWB : W_STAGE + (lane - 16) * RW_ROWB),
                     p_src + (size_t)k0 * 2, bytes, &full[p_s]);
      } else if (mine) {
        hb_mbar_arrive(&full[p_s]);
      }
    }
    p_u++;
    if (++p_s == stages) { p_s = 0; p_par ^= 1; }
    if (++p_c == chunks) { p_c = 0; p_ti++; p_tile(); }
  };
  // weights do not depend on the kernel ahead: the ring is filled before the wait, the activation rows after it
  const int pre = total < stages ? total : stages;
  if (producer && w_lane)
    for (int u = 0; u < pre; u++) p_issue(true, true);
  hb_pdl_wait();
  HB_TL_MARK(EPI * 3 + 0, 1);
  if (producer && !w_lane) {
    if (STREAM_A)
      for (int u = 0; u < pre; u++) p_issue(true, true);
    else
      for (int u = 0; u < pre; u++) p_issue(false, false);      // (idle lanes keep the same counters)
  }

  if constexpr (A_MODE == RW_A_SCALED) {
    // the token rows (already times the norm's weight, bf16) come into xs by bulk copy, a lane of the producer warp per row
    if (producer && lane == 0) hb_mbar_expect_tx(xbar, (uint32_t)(a.M * a.K * 2));
    __syncwarp();
    if (producer && lane < a.M)
      rw_bulk_load(xs + (size_t)lane * xs_rowb, (const __nv_bfloat16*)a.A + (long)lane * a.lda, (uint32_t)(a.K * 2), xbar);
    // the rows' sums of squares were left in pieces, one per tile of the product that wrote the residual: the three warps
    // that neither multiply nor copy add them, a row at a time in a fixed order, while the others go on; the epilogue
    // waits for them (rbar). Eight loads of a lane are in flight at once.
    if (warp > RW_CONSUMERS) {
      for (int m = warp - RW_CONSUMERS - 1; m < a.M; m += RW_WARPS - RW_CONSUMERS - 1) {
        float ss = 0.f;
        for (int p0 = lane; p0 < a.n_parts; p0 += 32 * 8) {
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; j++) v[j] = p0 + 32 * j < a.n_parts ? __ldcg(a.ssq_part + (size_t)(p0 + 32 * j) * 16 + m) : 0.f;
#pragma unroll
          for (int j = 0; j < 8; j++) ss += v[j];
        }
        ss = hb_warp_sum(ss);
        if (lane == 0) rs[m] = rsqrtf(ss / (float)a.K + a.eps);
      }
      __syncwarp();
      if (lane == 0) hb_mbar_arrive(rbar);
    }
  }
  if constexpr (A_MODE == RW_A_NORM) {
    // RMSNorm of the token rows into shared memory, a warp per row (all eight warps): x * rsqrt(mean(x^2) + eps) * w,
    // in fp32, rounded once
    const float* X = (const float*)a.A;
    for (int m = warp; m < a.M; m += RW_THREADS / 32) {
      const float* xr = X + (long)m * a.lda;
      constexpr int XV = 16;                                 // float4 a lane keeps: rows of up to 2,048 in one pass
      const int nv = a.K >> 2;                               // K is a multiple of 32
      const uint2* wv = (const uint2*)wsm;                   // four bf16 weights a load, from shared memory
      uint8_t* row = xs + (size_t)m * xs_rowb;
      float ss = 0.f;
      auto scaled = [&](float4 q, uint2 w, float inv) {
        const float2 w01 = __bfloat1622float2(*(const __nv_bfloat162*)&w.x), w23 = __bfloat1622float2(*(const __nv_bfloat162*)&w.y);
        return make_float4(w01.x * (q.x * inv), w01.y * (q.y * inv), w23.x * (q.z * inv), w23.y * (q.w * inv));
      };
      if (nv <= XV * 32) {
        float4 keep[XV];                                     // every load of the row is asked for before the first is used
#pragma unroll
        for (int i = 0; i < XV; i++) {
          const int v = lane + 32 * i;
          keep[i] = v < nv ? __ldcg((const float4*)xr + v) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < XV; i++)
          ss = fmaf(keep[i].x, keep[i].x, fmaf(keep[i].y, keep[i].y, fmaf(keep[i].z, keep[i].z, fmaf(keep[i].w, keep[i].w, ss))));
        ss = hb_warp_sum(ss);
        HB_TL_MARK(EPI * 3 + 2, 0);
        const float inv = rsqrtf(ss / (float)a.K + a.eps);
#pragma unroll
        for (int h = 0; h < XV; h += 8) {                     // eight weights to registers, then their eight stores
          uint2 wk[8];
#pragma unroll
          for (int i = 0; i < 8; i++) wk[i] = lane + 32 * (h + i) < nv ? wv[lane + 32 * (h + i)] : make_uint2(0u, 0u);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int v = lane + 32 * (h + i);
            if (v < nv) hb_store4((__nv_bfloat16*)row + 4 * v, scaled(keep[h + i], wk[i], inv));
          }
        }
      } else {
        for (int v = lane; v < nv; v += 32) {
          const float4 q = __ldcg((const float4*)xr + v);
          ss = fmaf(q.x, q.x, fmaf(q.y, q.y, fmaf(q.z, q.z, fmaf(q.w, q.w, ss))));
        }
        ss = hb_warp_sum(ss);
        const float inv = rsqrtf(ss / (float)a.K + a.eps);
        for (int v0 = lane; v0 < nv; v0 += 32 * 8) {         // eight loads in flight, then their stores
          float4 q[8];
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int v = v0 + 32 * i;
            q[i] = v < nv ? __ldcg((const float4*)xr + v) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int v = v0 + 32 * i;
            if (v < nv) hb_store4((__nv_bfloat16*)row + 4 * v, scaled(q[i], wv[v], inv));
          }
        }
      }
    }
    HB_TL_MARK(EPI * 3 + 2, 1);
    __syncthreads();
  }
  HB_TL_MARK(EPI * 3 + 0, 2);

  if (warp >= RW_CONSUMERS) {
    // ---------------- producer warp: refill a stage as soon as the consumers are done with it
    if (producer && (w_lane || STREAM_A))
      while (p_u < total) {
        if (!hb_mbar_wait(&empty[p_s], (uint32_t)p_par ^ 1, abort_flag)) break;
        p_issue(true, true);
      }
  } else {
    // ---------------- consumers: each takes every fourth 16-wide step of K
    const int g = lane >> 2, tq = lane & 3;
    int s = 0, par = 0;
    bool ok = true;      // false once a wait of this warp gave up; the warp still passes every barrier of the block
    if constexpr (A_MODE == RW_A_SCALED) ok = hb_mbar_wait(xbar, 0, abort_flag);
    for (int ti = 0; ti < my_tiles; ti++) {
      const int t = blockIdx.x + ti * gridDim.x;
      // The steps of a tile go to SETS independent accumulators in turn (added up at the end): the MMAs of a round do
      // not wait for one another. The same number for 8 and 16 token rows, so that a row's sum has one order.
      constexpr int SETS = 4;
      // What the epilogue reads from memory does not depend on the product: it is asked for now and has come by then.
      // ADD: a thread's (at most two) old residual values and next-norm weights; ROPE_KV: its row's (cos, sin) and slot.
      constexpr int EPI_ITEMS = (EPI == RW_ADD ? RW_R : 8) * MT, EPI_PER = (EPI_ITEMS + RW_CONSUMERS * 32 - 1) / (RW_CONSUMERS * 32);
      float pre_x[EPI_PER], pre_w[EPI_PER];
      float2 pre_cs[EPI_PER];
      int pre_slot[EPI_PER];
#pragma unroll
      for (int e = 0; e < EPI_PER; e++) {
        const int i = (int)threadIdx.x + e * RW_CONSUMERS * 32;
        pre_x[e] = 0.f; pre_w[e] = 0.f; pre_cs[e] = make_float2(1.f, 0.f); pre_slot[e] = -1;
        if constexpr (EPI == RW_ADD) {
          const int m = i >> 4, r = i & 15;
          const long n = (long)t * RW_R + r;
          if (i < EPI_ITEMS && m < a.M && n < a.N) {
            pre_x[e] = __ldcg((const float*)a.out + (long)m * a.ldo + n);
            if (a.next_w) pre_w[e] = __bfloat162float(a.next_w[n]);
          }
        } else if constexpr (EPI == RW_ROPE_KV) {
          const int m = i >> 3, j = i & 7, per_head = a.D >> 4, hh = t / per_head, d = (t - hh * per_head) * 8 + j;
          if (i < EPI_ITEMS && m < a.M) {
            if (hh < a.Hq + a.Hkv) pre_cs[e] = a.table[(size_t)a.pos[m] * (a.D >> 1) + d];
            if (hh >= a.Hq && a.slot_map) pre_slot[e] = a.slot_map[m];
          }
        }
      }
      float acc[SETS][NTILES][4];
#pragma unroll
      for (int e = 0; e < SETS; e++)
#pragma unroll
        for (int j = 0; j < NTILES; j++) acc[e][j][0] = acc[e][j][1] = acc[e][j][2] = acc[e][j][3] = 0.f;
      const int c_first = t % chunks;
      for (int c = 0; c < chunks; c++) {
        const int s_now = s, par_now = par;
        if (++s == stages) { s = 0; par ^= 1; }
        if (!ok || !hb_mbar_wait(&full[s_now], (uint32_t)par_now, abort_flag)) { ok = false; continue; }
        if (ti == 0 && c == 0) HB_TL_MARK(EPI * 3 + 1, 0);
        const uint8_t* ws = ring + (size_t)s_now * STAGE;
        // Tile t walks its chunks of K starting at chunk t % chunks. Were all blocks to read the same 2 KB columns of
        // their rows at the same time, the requests would meet in one half of the memory system (measured: half the
        // bandwidth for any row stride of 4 KB or more); turned against each other they spread over all of it. The
        // order of a row's sum depends on its tile, that is on the row itself, never on the batch.
        const int cc = c + c_first >= chunks ? c + c_first - chunks : c + c_first;
        const int k0 = cc * RW_KC, steps = min(RW_KC, a.K - k0) >> 4;
        // A thread reads 16 bytes (8 consecutive k) of its weight rows g and g + 8 and of its token rows: two MMA steps
        // worth. The MMA's k slots of a thread (2 tq, 2 tq + 1, 2 tq + 8, 2 tq + 9) are filled, for both operands alike,
        // with k = 8 tq + {0, 1, 2, 3} in the first step and 8 tq + {4, 5, 6, 7} in the second: a sum over k does not
        // care in which slot a k sits, and three 16-byte loads feed two MMAs instead of twelve 4-byte ones.
        const uint8_t* a_base = ws + g * RW_ROWB + tq * 16;
        const uint8_t* b_base = !STREAM_A ? xs + (size_t)g * xs_rowb + (size_t)k0 * 2 + tq * 16
                                                    : ws + W_STAGE + g * RW_ROWB + tq * 16;
        const size_t b_rows8 = !STREAM_A ? (size_t)8 * xs_rowb : (size_t)8 * RW_ROWB;
        const int blocks32 = steps >> 1;
        auto round = [&](int kb, int e0) {       // 32 of K: three 16-byte loads a token tile, two MMAs
          const uint4 lo = *(const uint4*)(a_base + kb * 64), hi = *(const uint4*)(a_base + 8 * RW_ROWB + kb * 64);
          const uint32_t af0[4] = {lo.x, hi.x, lo.y, hi.y}, af1[4] = {lo.z, hi.z, lo.w, hi.w};
#pragma unroll
          for (int j = 0; j < NTILES; j++) {
            const uint4 bv = *(const uint4*)(b_base + j * b_rows8 + kb * 64);
            const uint32_t bf0[2] = {bv.x, bv.y}, bf1[2] = {bv.z, bv.w};
            rw_mma(acc[e0][j], af0, bf0);
            rw_mma(acc[e0 + 1][j], af1, bf1);
          }
        };
        constexpr int ROUNDS = RW_KC / 32 / RW_CONSUMERS;
        if (blocks32 == RW_KC / 32) {            // a whole chunk: no branch between the rounds, their loads go out together
#pragma unroll
          for (int r = 0; r < ROUNDS; r++) round(r * RW_CONSUMERS + warp, (2 * r) % SETS);
        } else {
#pragma unroll
          for (int r = 0; r < ROUNDS; r++)
            if (r * RW_CONSUMERS + warp < blocks32) round(r * RW_CONSUMERS + warp, (2 * r) % SETS);
        }
        if (ti == 0 && c == 0) HB_TL_MARK(EPI * 3 + 2, 2);
        __syncwarp();
        if (lane == 0) hb_mbar_arrive(&empty[s_now]);
      }
      if (ti == 0) HB_TL_MARK(EPI * 3 + 1, 1);
      // the warps' partial sums: red[warp][row][token]
      float* mine = red + warp * RW_R * MT;
#pragma unroll
      for (int j = 0; j < NTILES; j++) {
        const int col = j * 8 + tq * 2;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < SETS; e++) { v[0] += acc[e][j][0]; v[1] += acc[e][j][1]; v[2] += acc[e][j][2]; v[3] += acc[e][j][3]; }
        *(float2*)(mine + g * MT + col) = make_float2(v[0], v[1]);
        *(float2*)(mine + (g + 8) * MT + col) = make_float2(v[2], v[3]);
      }
      if constexpr (A_MODE == RW_A_SCALED)
        if (ti == 0 && !hb_mbar_wait(rbar, 0, abort_flag)) ok = false;
      rw_consumer_sync();
      const int tid = *abort_flag ? RW_THREADS : (int)threadIdx.x;      // a block that gave up stores nothing
      auto total_of = [&](int r, int m) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < RW_CONSUMERS; w++) v += red[(w * RW_R + r) * MT + m];
        return v;
      };
      auto scale_of = [&](int m) { return A_MODE == RW_A_SCALED ? rs[m] : 1.f; };
      if constexpr (EPI == RW_ADD) {
#pragma unroll
        for (int e = 0; e < EPI_PER; e++) {
          const int i = tid + e * RW_CONSUMERS * 32;
          if (i >= RW_R * MT) break;
          const int m = i >> 4, r = i & 15;
          const long n = (long)t * RW_R + r;
          float xn = 0.f;
          if (m < a.M && n < a.N) {
            xn = pre_x[e] + total_of(r, m);
            ((float*)a.out)[(long)m * a.ldo + n] = xn;
            if (a.next_w) a.xb[(long)m * a.ldxb + n] = __float2bfloat16_rn(xn * pre_w[e]);
          }
          if (a.next_w) {               // the 16 lanes that hold a row's 16 columns add their squares, in a fixed order
            float sq = xn * xn;
            sq += __shfl_xor_sync(0xffffffffu, sq, 8);
            sq += __shfl_xor_sync(0xffffffffu, sq, 4);
            sq += __shfl_xor_sync(0xffffffffu, sq, 2);
            sq += __shfl_xor_sync(0xffffffffu, sq, 1);
            if (r == 0 && m < a.M) a.ssq_part[(size_t)t * 16 + m] = sq;
          }
        }
      } else if constexpr (EPI == RW_SWIGLU) {
        for (int i = tid; i < 8 * MT; i += RW_CONSUMERS * 32) {
          const int m = i >> 3, j = i & 7;
          if (m < a.M && rw_row<EPI>(a, t, 8 + j) < a.N) {
            const float gt = total_of(j, m) * scale_of(m), up = total_of(8 + j, m) * scale_of(m);
            ((__nv_bfloat16*)a.out)[(long)m * a.ldo + (long)t * 8 + j] = __float2bfloat16_rn(gt / (1.f + __expf(-gt)) * up);
          }
        }
      } else {
        const int half = a.D >> 1, per_head = a.D >> 4;
        const int hh = t / per_head, d0 = (t - hh * per_head) * 8;
#pragma unroll
        for (int e = 0; e < EPI_PER; e++) {
          const int i = tid + e * RW_CONSUMERS * 32;
          if (i >= 8 * MT) break;
          const int m = i >> 3, j = i & 7, d = d0 + j;
          if (m >= a.M) continue;
          const float x1 = total_of(j, m) * scale_of(m), x2 = total_of(8 + j, m) * scale_of(m);
          float y1 = x1, y2 = x2;
          if (hh < a.Hq + a.Hkv) {
            const float2 cs = pre_cs[e];
            y1 = __fsub_rn(__fmul_rn(x1, cs.x), __fmul_rn(x2, cs.y));
            y2 = __fadd_rn(__fmul_rn(x2, cs.x), __fmul_rn(x1, cs.y));
          }
          __nv_bfloat16* dst;
          if (hh < a.Hq) {
            dst = a.q_out + ((long)m * a.Hq + hh) * a.D + d;
          } else {
            const int slot = pre_slot[e];
            if (slot < 0) continue;
            const long page = slot / a.page_size, off = slot % a.page_size;
            const bool is_k = hh < a.Hq + a.Hkv;
            const int h = is_k ? hh - a.Hq : hh - a.Hq - a.Hkv;
            dst = (is_k ? a.kc : a.vc) + ((page * a.Hkv + h) * a.page_size + off) * a.D + d;
          }
          dst[0] = __float2bfloat16_rn(y1);
          dst[half] = __float2bfloat16_rn(y2);
        }
      }
      if (ti == 0) HB_TL_MARK(EPI * 3 + 1, 2);
      rw_consumer_sync();         // red is written again by the next tile
    }
  }
  HB_TL_MARK(EPI * 3 + 0, 3);
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(a.status, 1);
    __nanosleep(100000);          // copies that were asked for may still be landing in this block's shared memory
  }
}

// ---------------------------------------------------------------------------------------
// Shared memory a block may take, in KB, by epilogue: the ring gets what the fixed parts leave. About half an SM
// where the next product's blocks should find room beside this one's (they fill their rings while this one runs);
// the SwiGLU product, the largest of a layer, takes more stages instead.
static int g_rows_budget_kb[4] = {104, 104, 176, 156};   // ROPE_KV, ADD, SWIGLU, ADD with a K of more than two stages
HB_EXPORT void hb_rows_set_budget(int epi, int kb) {
  if (epi >= 0 && epi < 4 && kb >= 32 && kb <= 220) g_rows_budget_kb[epi] = kb;
}
constexpr size_t RW_SMEM_MAX = 220 * 1024;

template <int MT, int A_MODE> static size_t rows_fixed_bytes(int K) {
  return (size_t)RW_CONSUMERS * RW_R * MT * 4 + (A_MODE != RW_A_BF16 ? (size_t)MT * (K * 2 + RW_PAD) : 0) +
         (A_MODE == RW_A_NORM ? (size_t)K * 2 : 0) + 256;
}

template <int MT, int A_MODE, int EPI>
static int rows_launch(RowsArgs a, cudaStream_t s) {
  constexpr int R = RW_R;
  constexpr size_t STAGE = R * RW_ROWB + (A_MODE == RW_A_BF16 ? MT * RW_ROWB : 0);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t fixed = rows_fixed_bytes<MT, A_MODE>(a.K);
  a.n_tiles = (a.N + R - 1) / R;
  // a deep ring of one block per SM, unless there are more tiles than SMs and fewer than two rounds of them: then
  // two smaller blocks share an SM, so that every tile streams from the start (a second round would double the time)
  const bool deep = a.n_tiles <= sms || a.n_tiles >= 2 * sms;
  const size_t budget = (size_t)g_rows_budget_kb[EPI == RW_ADD ? (a.K > 2 * RW_KC && deep ? 3 : 1) : EPI == RW_SWIGLU && !deep ? 1 : EPI] * 1024;
  if (fixed + 2 * (STAGE + 16) > RW_SMEM_MAX) HB_FAIL("hb_rows: K = %d with %d token rows does not fit shared memory", a.K, MT);
  int stages = fixed + 2 * (STAGE + 16) > budget ? 2 : (int)((budget - fixed) / (STAGE + 16));
  if (stages > 12) stages = 12;
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * (STAGE + 16);
  auto kern = rows_product_kernel<MT, A_MODE, EPI>;
  static bool configured[64] = {};      // the attribute belongs to a device: set once on each
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RW_SMEM_MAX);
    if (e != cudaSuccess) HB_FAIL("hb_rows: %s", cudaGetErrorString(e));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int grid = a.n_tiles < 2 * sms ? a.n_tiles : sms;      // few tiles: a block each; many: one block per SM walks them
  cudaError_t e = hb_launch(kern, dim3(grid), RW_THREADS, smem, s, a);
  if (e != cudaSuccess) HB_FAIL("hb_rows: %s", cudaGetErrorString(e));
  return 0;
}

static int rows_check(const char* what, const RowsArgs& a, bool norm) {
  if (a.M < 1 || a.M > 16) HB_FAIL("%s: %d token rows (1 to 16)", what, a.M);
  if (a.K <= 0 || (a.K & 31)) HB_FAIL("%s: K = %d must be a positive multiple of 32", what, a.K);
  if ((a.ldw & 7) || ((uintptr_t)a.W & 15)) HB_FAIL("%s: weight rows must start on 16-byte boundaries", what);
  if (norm) {
    if ((a.lda & 3) || ((uintptr_t)a.A & 15) || ((uintptr_t)a.norm_w & 7)) HB_FAIL("%s: the residual rows must start on 16-byte boundaries", what);
  } else if ((a.lda & 7) || ((uintptr_t)a.A & 15)) {
    HB_FAIL("%s: activation rows must start on 16-byte boundaries", what);
  }
  if (!a.status) HB_FAIL("%s: no status word", what);
  return 0;
}

// q, k (rotated by the row's angle) and v of x's RMSNorm times a fused [q; k; v] weight: q to q_out [M, Hq D] bf16, k and v
// to their page slots (cache layout [page, Hkv, page_size, D]; slot_map null or a negative slot: not stored).
// x fp32 [M, K] (row stride ldx), norm_w bf16 [K], W bf16 [(Hq + 2 Hkv) D, K], table (cos, sin) fp32 [positions, D / 2].
HB_EXPORT int hb_rows_norm_qkv_rope(const float* x, long ldx, const void* norm_w, float eps, const void* W, long ldw, int M,
                                    int K, const int* pos, const int* slot_map, const void* table, void* q_out, void* kc,
                                    void* vc, int Hq, int Hkv, int D, int page_size, int* status, cudaStream_t s) {
  RowsArgs a = {};
  a.A = x; a.lda = ldx; a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps; a.W = (const __nv_bfloat16*)W; a.ldw = ldw;
  a.M = M; a.N = (Hq + 2 * Hkv) * D; a.K = K; a.pos = pos; a.slot_map = slot_map; a.table = (const float2*)table;
  a.q_out = (__nv_bfloat16*)q_out; a.kc = (__nv_bfloat16*)kc; a.vc = (__nv_bfloat16*)vc;
  a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.page_size = page_size; a.status = status;
  if (M <= 0) return 0;
  if (rows_check("hb_rows_norm_qkv_rope", a, true)) return -1;
  if (D < 16 || (D & 15)) HB_FAIL("hb_rows_norm_qkv_rope: head_dim %d must be a multiple of 16", D);
  if (!pos || !table || !q_out || (slot_map && (!kc || !vc))) HB_FAIL("hb_rows_norm_qkv_rope: a null argument");
  return M <= 8 ? rows_launch<8, RW_A_NORM, RW_ROPE_KV>(a, s) : rows_launch<16, RW_A_NORM, RW_ROPE_KV>(a, s);
}

// out fp32 [M, N] (row stride ldo) += act [M, K] (bf16) W[N, K]^T. With next_w (bf16 [N], the weight of the norm that reads
// `out` next): also xb [M, N] bf16 (row stride ldxb) = out * next_w, and ssq_part [ceil(N / 16)][16] floats = each 16-column
// tile's share of the rows' sums of squares; hb_rows_scaled_* take those in place of the residual rows.
HB_EXPORT int hb_rows_add(const void* act, long lda, const void* W, long ldw, float* out, long ldo, int M, int N, int K,
                          const void* next_w, void* xb, long ldxb, float* ssq_part, int* status, cudaStream_t s) {
  RowsArgs a = {};
  a.A = act; a.lda = lda; a.W = (const __nv_bfloat16*)W; a.ldw = ldw; a.M = M; a.N = N; a.K = K; a.out = out; a.ldo = ldo;
  a.status = status; a.next_w = (const __nv_bfloat16*)next_w; a.xb = (__nv_bfloat16*)xb; a.ldxb = ldxb; a.ssq_part = ssq_part;
  if (M <= 0 || N <= 0) return 0;
  if (rows_check("hb_rows_add", a, false)) return -1;
  if (next_w && (!xb || !ssq_part)) HB_FAIL("hb_rows_add: next_w without xb and ssq_part");
  return M <= 8 ? rows_launch<8, RW_A_BF16, RW_ADD>(a, s) : rows_launch<16, RW_A_BF16, RW_ADD>(a, s);
}

// hb_rows_norm_qkv_rope with the normalisation prepared by the product that wrote the residual (hb_rows_add with next_w):
// xb [M, K] bf16 = x * norm_w and ssq_part [n_parts][16] in place of x and norm_w; 1 / RMS is applied in the epilogue.
HB_EXPORT int hb_rows_scaled_qkv_rope(const void* xb, long ldxb, const float* ssq_part, int n_parts, float eps, const void* W,
                                      long ldw, int M, int K, const int* pos, const int* slot_map, const void* table,
                                      void* q_out, void* kc, void* vc, int Hq, int Hkv, int D, int page_size, int* status,
                                      cudaStream_t s) {
  RowsArgs a = {};
  a.A = xb; a.lda = ldxb; a.ssq_part = (float*)ssq_part; a.n_parts = n_parts; a.eps = eps; a.W = (const __nv_bfloat16*)W; a.ldw = ldw;
  a.M = M; a.N = (Hq + 2 * Hkv) * D; a.K = K; a.pos = pos; a.slot_map = slot_map; a.table = (const float2*)table;
  a.q_out = (__nv_bfloat16*)q_out; a.kc = (__nv_bfloat16*)kc; a.vc = (__nv_bfloat16*)vc;
  a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.page_size = page_size; a.status = status;
  if (M <= 0) return 0;
  if (rows_check("hb_rows_scaled_qkv_rope", a, false)) return -1;
  if (D < 16 || (D & 15)) HB_FAIL("hb_rows_scaled_qkv_rope: head_dim %d must be a multiple of 16", D);
  if (!ssq_part || n_parts * 16 != K) HB_FAIL("hb_rows_scaled_qkv_rope: %d pieces of the sums of squares for a width of %d", n_parts, K);
  if (!pos || !table || !q_out || (slot_map && (!kc || !vc))) HB_FAIL("hb_rows_scaled_qkv_rope: a null argument");
  return M <= 8 ? rows_launch<8, RW_A_SCALED, RW_ROPE_KV>(a, s) : rows_launch<16, RW_A_SCALED, RW_ROPE_KV>(a, s);
}

// hb_rows_norm_swiglu with the normalisation prepared the same way.
HB_EXPORT int hb_rows_scaled_swiglu(const void* xb, long ldxb, const float* ssq_part, int n_parts, float eps, const void* W,
                                    long ldw, void* out, long ldo, int M, int N, int K, int* status, cudaStream_t s) {
  RowsArgs a = {};
  a.A = xb; a.lda = ldxb; a.ssq_part = (float*)ssq_part; a.n_parts = n_parts; a.eps = eps; a.W = (const __nv_bfloat16*)W; a.ldw = ldw;
  a.M = M; a.N = N; a.K = K; a.out = out; a.ldo = ldo; a.status = status;
  if (M <= 0 || N <= 0) return 0;
  if (rows_check("hb_rows_scaled_swiglu", a, false)) return -1;
  if (N & 31) HB_FAIL("hb_rows_scaled_swiglu: N = %d must be a multiple of 32 (gate and up rows in groups of 16)", N);
  if (!ssq_part || n_parts * 16 != K) HB_FAIL("hb_rows_scaled_swiglu: %d pieces of the sums of squares for a width of %d", n_parts, K);
  return M <= 8 ? rows_launch<8, RW_A_SCALED, RW_SWIGLU>(a, s) : rows_launch<16, RW_A_SCALED, RW_SWIGLU>(a, s);
}

// out bf16 [M, N / 2] = silu(gate) * up of x's RMSNorm times W [N, K], whose rows alternate 16 gate rows and their 16 up rows.
HB_EXPORT int hb_rows_norm_swiglu(const float* x, long ldx, const void* norm_w, float eps, const void* W, long ldw,
                                  void* out, long ldo, int M, int N, int K, int* status, cudaStream_t s) {
  RowsArgs a = {};
  a.A = x; a.lda = ldx; a.norm_w = (const __nv_bfloat16*)norm_w; a.eps = eps; a.W = (const __nv_bfloat16*)W; a.ldw = ldw;
  a.M = M; a.N = N; a.K = K; a.out = out; a.ldo = ldo; a.status = status;
  if (M <= 0 || N <= 0) return 0;
  if (rows_check("hb_rows_norm_swiglu", a, true)) return -1;
  if (N & 31) HB_FAIL("hb_rows_norm_swiglu: N = %d must be a multiple of 32 (gate and up rows in groups of 16)", N);
  return M <= 8 ? rows_launch<8, RW_A_NORM, RW_SWIGLU>(a, s) : rows_launch<16, RW_A_NORM, RW_SWIGLU>(a, s);
}

// Whether the norm-in-the-prologue kernels take a width K with M token rows (the normalised rows lie in shared memory).
HB_EXPORT int hb_rows_norm_supported(int M, int K) {
  if (M < 1 || M > 16 || K <= 0 || (K & 31)) return 0;
  const size_t fixed = M <= 8 ? rows_fixed_bytes<8, RW_A_NORM>(K) : rows_fixed_bytes<16, RW_A_NORM>(K);
  return fixed + 2 * (RW_R * RW_ROWB + 16) <= RW_SMEM_MAX ? 1 : 0;
}
