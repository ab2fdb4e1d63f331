// BF16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operands staged by TMA).
//
// One kernel template covers the three products a linear layer needs (the reference gets them from
// cuBLASLt: linear_forward / linear_backward_inp / linear_backward_weight, train/gpt_kernels.cuh:165-194):
//     fwd  out[M,N]  = x[M,K]    . W[N,K]^T     A K-major,  B K-major,  bf16 store
//     dX   dx[M,K]   = dout[M,N] . W[N,K]       A K-major,  B MN-major, bf16 store
//     dW   dW[N,K]  += dout[M,N]^T . x[M,K]     A MN-major, B MN-major, fp32 red.add (split-K over tokens)
// "D[m,n] = sum_k A(m,k) B(n,k)" with each operand either K-major (k contiguous in memory) or MN-major.
//
// Structure: persistent CTAs (one per SM), 192 threads = 1 TMA-producer warp, 1 MMA-issuer warp (a single
// elected thread issues tcgen05.mma), 4 epilogue warps.  Tile 128 x BN x 64 with a multi-stage shared-memory
// ring guarded by full/empty mbarriers; two TMEM accumulators (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.  Every mbarrier wait is bounded: on expiry the kernel records an error
// word, frees its TMEM and returns.
#include "../tc.cuh"

#include <cstdio>
#include <map>
#include <array>
#include <mutex>
#include <tuple>
#include <vector>


namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

enum { EPI_BF16 = 0, EPI_F32_ADD = 1 };

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;   // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;   // 16/32 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int STAGING_BYTES = 4 * 2 * 4096;  // 4 epilogue warps x 2 buffers x [32 rows x 128 B]
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES + 1024;  // +1024 alignment slack
};

// All-gather fused into the GEMM (FSDP): four extra warps per CTA pull 16 KB pieces of the sharded parameter unit from
// the owning ranks' memory (peer loads over NVLink) into the local gather slot and publish a per-piece flag; the TMA
// producer of a tile waits (bounded) for the pieces that hold its rows of B.  Needs all CTAs co-resident: the kernel
// is started with a cooperative launch.
struct GatherArgs {
  const uint4* const* src;   // device array [world]: base of each rank's shard of this unit
  uint4* dst;                // local gather slot (start of the unit)
  long shard_vec;            // 16-byte vectors per shard
  long b_lo_vec, b_hi_vec;   // vector range of the B matrix inside the unit
  long b_row_vec;            // vectors per row of B (K-major B: pitch; used to map a tile's rows to pieces)
  int* flags;                // one int per piece, device memory of this GPU, monotonically increasing epochs
  int* ctr;                  // [0] completed launches (epoch = ctr[0] + 1), [1] CTAs done in this launch
  int world;
  int piece_vec;             // vectors per piece
  long spin_limit_ns;
};

struct GemmArgs {
  void* out;
  int M, N, K;       // logical problem: D[M,N], reduction K
  int ldo;           // output row pitch in elements
  int tiles_m, tiles_n, splits, kb_per_split, kb_total;
  int a3d, b3d;      // MN-major operand fetched through a 3-D tensor map (one TMA per stage) instead of 64-wide 2-D boxes
  int streamk;       // pair kernel, fp32 add epilogue: every cluster (group) takes an equal contiguous share of all (tile, k-block) units
  int sk_group, sk_group_m;   // stream-K group size (tiles along the short dimension) and whether that dimension is M
  int nt_fast;       // static schedule: consecutive work items walk N first (tiles in flight share rows of A) instead of M
  // optional rotary embedding in the bf16 epilogue (pair kernel): output columns [0, rope_cols) are heads of 64 columns
  // whose halves (i, i + 32) are rotated by the angle table row (output row % rope_T)
  const float* cosT;
  const float* sinT;
  int rope_T, rope_cols;
  // optional SwiGLU in the bf16 epilogue (pair kernel, forward product with N = 2 * sw_I = [gate | up] columns): a pair
  // tile holds gate columns [nt*128, +128) in accumulator columns 0..127 and the matching up columns in 128..255 (the
  // leader CTA stages the gate rows of W, its peer the up rows), so silu(gate) * up is formed where both are at hand
  // and written to sw_out[M, sw_I] beside the [gate | up] output that backward needs
  bf16* sw_out;
  int sw_I;
  float out_scale;   // 8-bit form: accumulators are multiplied by this (1 / (activation scale * weight scale))
  // optional learned-position add in the bf16 epilogue (pair kernel): out[r, c] += pos[r % pos_period, c], pos is
  // [pos_period, N] bf16 (the vision tower's patch embedding: positions repeat every n_patch rows)
  const bf16* pos;
  int pos_period;
  // optional row-dot in the bf16 epilogue (pair kernel, the attention output projection's input gradient D = dO[M, H*64]):
  // dl_out[(b*H + h)*T + t] = sum over the 64 columns of head h of D[row, .] * dl_o[row, .] with row = b*T + t, taken on the
  // fp32 accumulators - the "delta" term of the attention backward, which otherwise costs a pass over dO and O
  const bf16* dl_o;
  float* dl_out;
  int dl_T, dl_H;
};

// Work items of one cluster of the pair kernel.  Static mode: items c, c + nclusters, ... of tiles x splits.
// Stream-K mode: the tiles' k-blocks are laid end to end (tile-major) and cut into nclusters equal ranges, so a cluster
// gets at most a tail piece of one tile, whole tiles, and a head piece of another; every piece is add-reduced into the
// fp32 output, which is what the split-K epilogue does anyway.
struct WorkItem { int mt, nt, kb0, kb1; };
struct WorkIter {
  int t, step, total, tiles_m, tiles_n, kb_per_split, kb_total;
  int member, G, grouped_m;     // stream-K: this cluster's tile index along the grouped dimension
  long u, u1;
  bool sk, nt_fast;
  __device__ WorkIter(const GemmArgs& g, int cid, int ncl)
      : t(cid), step(ncl), total(g.tiles_m * g.tiles_n * g.splits), tiles_m(g.tiles_m), tiles_n(g.tiles_n),
        kb_per_split(g.kb_per_split), kb_total(g.kb_total), sk(g.streamk != 0), nt_fast(g.nt_fast != 0) {
    // Stream-K in groups: the G tiles that share the wide operand (same index along the long dimension) are given to G
    // neighbouring clusters with IDENTICAL (long-dimension tile, k-block) ranges, so that operand is fetched from DRAM
    // once and found in L2 by the other members; the narrow operand is small enough to live in L2.
    G = g.sk_group > 0 ? g.sk_group : 1;
    grouped_m = g.sk_group_m;
    const int ngroups = ncl / G, grp = cid / G;
    member = cid % G;
    const int long_tiles = G == 1 ? g.tiles_m * g.tiles_n : (grouped_m ? g.tiles_n : g.tiles_m);   // G == 1: every tile on its own
    const long units = (long)long_tiles * g.kb_total;
    if (sk && grp < ngroups) {
      u = units * grp / ngroups;
      u1 = units * (grp + 1) / ngroups;
    } else {
      u = u1 = 0;
    }
  }
  __device__ bool next(WorkItem& w) {
    if (sk) {
      if (u >= u1) return false;
      const int lt = (int)(u / kb_total);
      w.kb0 = (int)(u % kb_total);
      w.kb1 = (int)min((long)kb_total, w.kb0 + (u1 - u));
      if (G == 1) { w.mt = lt % tiles_m; w.nt = lt / tiles_m; }
      else if (grouped_m) { w.mt = member; w.nt = lt; }
      else { w.mt = lt; w.nt = member; }
      u += w.kb1 - w.kb0;
      return true;
    }
    if (t >= total) return false;
    const int sp = t / (tiles_m * tiles_n);
    if (nt_fast) { w.nt = t % tiles_n; w.mt = (t / tiles_n) % tiles_m; }
    else { w.mt = t % tiles_m; w.nt = (t / tiles_m) % tiles_n; }
    w.kb0 = sp * kb_per_split; w.kb1 = min(w.kb0 + kb_per_split, kb_total);
    t += step;
    return true;
  }
};

__device__ __forceinline__ bool wait_piece(const int* flag, int epoch, long limit_ns) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  if (v >= epoch) return true;
  const uint64_t t0 = tc::globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; i++) {
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v >= epoch) return true;
      __nanosleep(64);
    }
    if ((long)(tc::globaltimer_ns() - t0) > limit_ns) { mlb_set_error(MLB_ERR_FLAG_TIMEOUT, 0x6a7); return false; }
  }
}

template <int BN, bool A_MN, bool B_MN, int EPI, bool GATHER = false>
__global__ void __launch_bounds__(GEMM_THREADS + (GATHER ? 128 : 0), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmD, const GemmArgs g, const GatherArgs ga) {
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * S::STAGE_BYTES;
  uint64_t* full = (uint64_t*)(staging + S::STAGING_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = g.tiles_m * g.tiles_n * g.splits;
  int g_epoch = 0;
  if (GATHER) g_epoch = *((volatile int*)ga.ctr) + 1;   // every CTA reads it before the last one to finish bumps it

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; i++) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], 4); }
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tmA);
    tc::tma_prefetch_desc(&tmB);
    tc::tma_prefetch_desc(&tmD);
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, 2 * BN);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (!GATHER) mlb_pdl_sync();   // set-up done; operands written by the previous kernel are read from here on

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (tc::elect_one()) {
      int stage = 0, phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int mt = t % g.tiles_m, nt = (t / g.tiles_m) % g.tiles_n, sp = t / (g.tiles_m * g.tiles_n);
        const int m0 = mt * BM, n0 = nt * BN;
        const int kb0 = sp * g.kb_per_split, kb1 = min(kb0 + g.kb_per_split, g.kb_total);
        if (GATHER) {
          // rows [n0, n0+BN) of a K-major B live in a contiguous vector range of the unit; an MN-major B needs all of it
          long lo = ga.b_lo_vec, hi = ga.b_hi_vec;
          if (!B_MN) { lo = ga.b_lo_vec + (long)n0 * ga.b_row_vec; hi = min(ga.b_hi_vec, lo + (long)BN * ga.b_row_vec); }
          for (long pc = lo / ga.piece_vec; pc <= (hi - 1) / ga.piece_vec && ok; pc++)
            ok = wait_piece(ga.flags + pc, g_epoch, ga.spin_limit_ns);
          asm volatile("fence.proxy.async;" ::: "memory");   // peer data landed by generic stores, read next by TMA
          if (!ok) break;
        }
        for (int kb = kb0; kb < kb1; kb++) {
          if (!tc::mbar_wait(&empty[stage], phase ^ 1, 1)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          tc::mbar_expect_tx(&full[stage], S::STAGE_BYTES);
          if (!A_MN) {
            tc::tma_load_2d(sA, &tmA, &full[stage], kb * BK, m0);
          } else {
#pragma unroll
            if (g.a3d) tc::tma_load_3d(sA, &tmA, &full[stage], 0, kb * BK, m0 / 64);
            else
              for (int c = 0; c < BM / 64; c++) tc::tma_load_2d(sA + c * 8192, &tmA, &full[stage], m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tc::tma_load_2d(sB, &tmB, &full[stage], kb * BK, n0);
          } else {
#pragma unroll
            if (g.b3d) tc::tma_load_3d(sB, &tmB, &full[stage], 0, kb * BK, n0 / 64);
            else
              for (int c = 0; c < BN / 64; c++) tc::tma_load_2d(sB + c * 8192, &tmB, &full[stage], n0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (tc::elect_one()) {
      constexpr uint32_t idesc = tc::idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
        const int sp = t / (g.tiles_m * g.tiles_n);
        const int kb0 = sp * g.kb_per_split, kb1 = min(kb0 + g.kb_per_split, g.kb_total);
        const int acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, 2)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb++) {
          if (!tc::mbar_wait(&full[stage], phase, 3)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sA = tc::smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sB = sA + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            const uint64_t da = A_MN ? tc::smem_desc_sw128(sA + k * 2048, 8192, 1024) : tc::smem_desc_sw128(sA + k * 32, 16, 1024);
            const uint64_t db = B_MN ? tc::smem_desc_sw128(sB + k * 2048, 8192, 1024) : tc::smem_desc_sw128(sB + k * 32, 16, 1024);
            tc::mma_bf16_ss(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc::mma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc::mma_commit(&acc_full[acc]);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    // Each warp owns 32 accumulator rows (its TMEM lane group).  A 128-byte-wide slab of those rows (64 bf16 or
    // 32 fp32 columns) is converted into a swizzled 4 KB staging buffer and handed to TMA: a tiled store for bf16
    // outputs, an fp32 add-reduce for split-K weight gradients.  Two buffers per warp keep one transfer in flight;
    // TMA clips rows / columns beyond the matrix.
    const int lg = warp & 3;  // TMEM lane group this warp may read
    uint8_t* my_stage = staging + lg * 8192;
    constexpr int SLAB_COLS = (EPI == EPI_BF16) ? 64 : 32;
    int it = 0, slab = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
      const int mt = t % g.tiles_m, nt = (t / g.tiles_m) % g.tiles_n;
      const int m0 = mt * BM, n0 = nt * BN;
      const int acc = it & 1, acc_phase = (it >> 1) & 1;
      if (!tc::mbar_wait(&acc_full[acc], acc_phase, 4)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(lg * 32) << 16) + acc * BN;
      const bool rows_live = (m0 + lg * 32) < g.M;
#pragma unroll 1
      for (int c = 0; c < BN / SLAB_COLS; c++) {
        uint8_t* buf = my_stage + (slab & 1) * 4096;
        uint32_t r[32], r2[32];
        tc::tmem_ld32(taddr + c * SLAB_COLS, r);
        if (EPI == EPI_BF16) tc::tmem_ld32(taddr + c * SLAB_COLS + 32, r2);
        tc::tmem_ld_wait();
        const int col0 = n0 + c * SLAB_COLS;
        if (!rows_live || col0 >= g.N) continue;   // warp-uniform
        if (lane == 0) tc::tma_wait_group_read<1>();   // the transfer that last used this buffer has read it
        __syncwarp();
        uint8_t* rowp = buf + lane * 128;
        if (EPI == EPI_BF16) {
#pragma unroll
          for (int v = 0; v < 8; v++) {
            const uint32_t* src = (v < 4) ? &r[v * 8] : &r2[(v - 4) * 8];
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(src[0]), __uint_as_float(src[1]));
            pk.y = pack_bf16(__uint_as_float(src[2]), __uint_as_float(src[3]));
            pk.z = pack_bf16(__uint_as_float(src[4]), __uint_as_float(src[5]));
            pk.w = pack_bf16(__uint_as_float(src[6]), __uint_as_float(src[7]));
            *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = pk;
          }
        } else {
#pragma unroll
          for (int v = 0; v < 8; v++) {
            uint4 pk = make_uint4(r[v * 4 + 0], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = pk;
          }
        }
        tc::fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (EPI == EPI_BF16) tc::tma_store_2d(&tmD, buf, col0, m0 + lg * 32);
          else tc::tma_reduce_add_2d(&tmD, buf, col0, m0 + lg * 32);
          tc::tma_commit_group();
        }
        slab++;   // counts issued transfers only, so the two buffers strictly alternate
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[acc]);
    }
    if (lane == 0) tc::tma_wait_group<0>();   // all stores / reductions of this warp have completed
  }
  if (GATHER && warp >= 6) {
    // ---------------------------------------------------------------- gather warps (6..9)
    const int gt = threadIdx.x - GEMM_THREADS;            // 0..127
    const long total_vec = ga.shard_vec * ga.world;
    const long n_pieces = (total_vec + ga.piece_vec - 1) / ga.piece_vec;
    for (long pc = blockIdx.x; pc < n_pieces; pc += gridDim.x) {
      const long v0 = pc * ga.piece_vec, v1 = min(total_vec, v0 + ga.piece_vec);
      for (long v = v0 + gt; v < v1; v += 128) {
        const int w = (int)(v / ga.shard_vec);
        const uint4* sp = ga.src[w] + (v - (long)w * ga.shard_vec);
        uint4 x;
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w) : "l"(sp) : "memory");
        ga.dst[v] = x;
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (gt == 0) asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(ga.flags + pc), "r"(g_epoch) : "memory");
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (GATHER && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ga.ctr + 1, 1) == (int)gridDim.x - 1) { ga.ctr[1] = 0; ga.ctr[0] = g_epoch; }
  }
  if (warp == 1) tc::tmem_dealloc(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------ CTA-pair variant (cta_group::2)
// A 1-CTA 128x256 tile needs 48 KB of operands per 64-deep K step, more than an SM can pull from L2 in the ~512 cycles
// the MMAs of that step take.  Here two CTAs of a cluster share a 256 x 256 tile: each stages its 128 rows of A and
// 128 of the 256 rows of B (32 KB per step and SM, a third less L2 traffic per FLOP), the leader issues
// tcgen05.mma.cta_group::2 with M = 256, and each CTA drains its own 128 TMEM lanes x 256 columns.
//   full[s]      leader only: one arrive.expect_tx by the leader's producer for BOTH CTAs' bytes; both producers' TMA
//                loads complete on it
//   empty[s]     one per CTA; the leader's MMA thread commits to both
//   acc_full[a]  one per CTA; committed to both
//   acc_empty[a] leader only, 8 arrivals: the four epilogue warps of each CTA (the peer's arrive remotely)
// Persistent: cluster c handles pair-tiles c, c + nclusters, ...; all waits are bounded as in the 1-CTA kernel, and both
// CTAs meet at a cluster barrier before TMEM is released so neither outlives remote accesses to it.
template <int EMODE>
struct Gemm2Smem {
  static constexpr int A_BYTES = 128 * BK * 2;    // this CTA's rows of A
  static constexpr int B_BYTES = 128 * BK * 2;    // this CTA's half of B
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = EMODE == 0 ? 5 : 6;
  static constexpr int BUFS = EMODE == 0 ? 2 : 1;               // staging buffers per epilogue warp
  static constexpr int STAGING_BYTES = 8 * BUFS * 4096;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES + 1024;
};
constexpr int GEMM2_THREADS = 64 + 8 * 32;   // producer warp, MMA warp, eight epilogue warps

// One warp writes a slab of 32 rows x 64 bf16 (lane = row, pk = that row's 64 values packed in pairs) through its
// swizzled 4 KB staging buffer to out[m0 + row, col0 .. col0 + 63]: four full 128-byte rows per store instruction.
__device__ __forceinline__ void slab_store_bf16(uint8_t* buf, int lane, const uint32_t (&pk)[32], bf16* out, int ldo, int m0,
                                                int col0, int M, int ncols) {
  uint8_t* rowp = buf + lane * 128;
#pragma unroll
  for (int v = 0; v < 8; v++)
    *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = make_uint4(pk[v * 4], pk[v * 4 + 1], pk[v * 4 + 2], pk[v * 4 + 3]);
  __syncwarp();
  const int ch = lane & 7, gcol = col0 + ch * 8;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = i * 4 + (lane >> 3);
    const uint4 v = *reinterpret_cast<const uint4*>(buf + row * 128 + ((ch ^ (row & 7)) << 4));
    if (m0 + row < M && gcol < ncols) *reinterpret_cast<uint4*>(out + (size_t)(m0 + row) * ldo + gcol) = v;
  }
  __syncwarp();   // the buffer is rewritten by the next slab
}
__device__ __forceinline__ void scale64(uint32_t (&r)[32], uint32_t (&r2)[32], float s) {
#pragma unroll
  for (int i = 0; i < 32; i++) {
    r[i] = __float_as_uint(__uint_as_float(r[i]) * s);
    r2[i] = __float_as_uint(__uint_as_float(r2[i]) * s);
  }
}
__device__ __forceinline__ void pack64(const uint32_t (&r)[32], const uint32_t (&r2)[32], uint32_t (&pk)[32]) {
#pragma unroll
  for (int i = 0; i < 16; i++) {
    pk[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    pk[16 + i] = pack_bf16(__uint_as_float(r2[2 * i]), __uint_as_float(r2[2 * i + 1]));
  }
}

// Epilogue: eight warps per CTA; warp w reads TMEM lanes 32*(w%4).. (the lane group the hardware lets it read) and one
// 128-column half of the accumulator.  A slab of 32 rows x 128 bytes goes through a swizzled staging buffer, then
//   EMODE 0: TMA tiled store / fp32 add-reduce (two buffers per warp, one transfer in flight)
//   EMODE 1: the warp itself writes it out, four full 128-byte rows per instruction (st.global.v4 / red.global.add.v4.f32)
// Register budget: the ten warps land three on two of the SM's four sub-partitions (16 K registers each).  At 160
// registers per thread those three warps leave 1 K registers, room for one 32-register warp of a small kernel from
// another stream (the gradient-bucket kernels that run behind backward use 128-thread CTAs for that reason); at the 168
// the compiler takes when left alone nothing else fits on the SM and such a kernel and this one exclude each other.
// F8: both operands are E4M3 bytes, K-major; a 128-byte shared-memory row then holds 128 elements of K, one stage 128
// of K (four K = 32 instructions), and the accumulators are multiplied by g.out_scale (the product of the two dequant
// scales) on their way out.  Everything else - tiles, ring, barriers, epilogue - is shared with the bf16 form.
// POS: the learned-position add of GemmArgs::pos is compiled in (its own instantiation, so that the register allocation of
// the plain kernels is not affected).
template <bool A_MN, bool B_MN, int EPI, int EMODE, bool F8 = false, bool POS = false, bool DELTA = false>
__global__ void __cluster_dims__(2, 1, 1) __maxnreg__(160)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmD, const GemmArgs g) {
  static_assert(!F8 || (!A_MN && !B_MN && EPI == EPI_BF16), "the 8-bit form is a forward product: K-major operands, bf16 out");
  constexpr int KSTEP = F8 ? 128 : BK;     // elements of K per stage
  using S = Gemm2Smem<EMODE>;
  constexpr int STAGES = S::STAGES;
  constexpr int BN = 256, PM = 256;    // pair tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + STAGES * S::STAGE_BYTES;
  uint64_t* full = (uint64_t*)(staging + S::STAGING_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();          // 0 = leader
  const int cid = (int)tc::cluster_id_x(), ncl = (int)tc::cluster_count_x();

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; i++) { tc::mbar_init(&acc_full[i], 1); tc::mbar_init(&acc_empty[i], 16); }
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tmA);
    tc::tma_prefetch_desc(&tmB);
    if (EMODE == 0) tc::tma_prefetch_desc(&tmD);
  }
  if (warp == 1) tc::tmem_alloc_pair(tmem_slot, 2 * BN);
  tc::tc_fence_before();
  tc::cluster_sync();      // barriers of both CTAs initialised, TMEM of both allocated
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  mlb_pdl_sync();          // set-up done; operands written by the previous kernel are read from here on

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (one per CTA)
    if (tc::elect_one()) {
      int stage = 0, phase = 0;
      bool ok = true;
      WorkIter iter(g, cid, ncl);
      WorkItem w;
      while (ok && iter.next(w)) {
        const int m0 = w.mt * PM + (int)rank * 128;
        // SwiGLU form: tile nt pairs gate rows [nt*128, +128) of W (leader) with up rows [I + nt*128, +128) (peer)
        const int n0 = g.sw_out ? (w.nt * 128 + (int)rank * g.sw_I) : (w.nt * BN + (int)rank * 128);
        for (int kb = w.kb0; kb < w.kb1; kb++) {
          if (!tc::mbar_wait(&empty[stage], phase ^ 1, 0x21)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          const uint32_t bar = tc::mapa_u32(tc::smem_u32(&full[stage]), 0);
          if (rank == 0) tc::mbar_expect_tx(&full[stage], 2 * S::STAGE_BYTES);
          if (!A_MN) {
            tc::tma_load_2d_pair(sA, &tmA, bar, kb * KSTEP, m0);
          } else {
            if (g.a3d) tc::tma_load_3d_pair(sA, &tmA, bar, 0, kb * BK, m0 / 64);
            else
              for (int c = 0; c < 2; c++) tc::tma_load_2d_pair(sA + c * 8192, &tmA, bar, m0 + c * 64, kb * BK);
          }
          if (!B_MN) {
            tc::tma_load_2d_pair(sB, &tmB, bar, kb * KSTEP, n0);
          } else {
            if (g.b3d) tc::tma_load_3d_pair(sB, &tmB, bar, 0, kb * BK, n0 / 64);
            else
              for (int c = 0; c < 2; c++) tc::tma_load_2d_pair(sB + c * 8192, &tmB, bar, n0 + c * 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    if (rank == 0 && tc::elect_one()) {
      constexpr uint32_t idesc = F8 ? tc::idesc_e4m3(PM, BN) : tc::idesc_bf16(PM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0, phase = 0, it = 0;
      bool ok = true;
      WorkIter iter(g, cid, ncl);
      WorkItem w;
      for (; ok && iter.next(w); it++) {
        const int kb0 = w.kb0, kb1 = w.kb1;
        const int acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!tc::mbar_wait(&acc_empty[acc], acc_phase ^ 1, 0x22)) { ok = false; break; }
        tc::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb++) {
          if (!tc::mbar_wait(&full[stage], phase, 0x23)) { ok = false; break; }
          tc::tc_fence_after();
          const uint32_t sA = tc::smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sB = sA + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            const uint64_t da = A_MN ? tc::smem_desc_sw128(sA + k * 2048, 8192, 1024) : tc::smem_desc_sw128(sA + k * 32, 16, 1024);
            const uint64_t db = B_MN ? tc::smem_desc_sw128(sB + k * 2048, 8192, 1024) : tc::smem_desc_sw128(sB + k * 32, 16, 1024);
            if (F8) tc::mma_e4m3_ss_pair(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else tc::mma_bf16_ss_pair(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc::mma_commit_pair(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc::mma_commit_pair(&acc_full[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..9 of each CTA)
    const int lg = warp & 3, half = (warp - 2) >> 2;
    uint8_t* my_stage = staging + (warp - 2) * (S::BUFS * 4096);
    constexpr int SLAB_COLS = (EPI == EPI_BF16) ? 64 : 32;
    constexpr int SLABS = 128 / SLAB_COLS;       // per warp and tile
    constexpr int ELEM = (EPI == EPI_BF16) ? 2 : 4;
    int it = 0, slab = 0;
    bool ok = true;
    WorkIter iter(g, cid, ncl);
    WorkItem w;
    for (; ok && iter.next(w); it++) {
      const int m0 = w.mt * PM + (int)rank * 128 + lg * 32, n0 = w.nt * BN + half * 128;
      const int acc = it & 1, acc_phase = (it >> 1) & 1;
      if (!tc::mbar_wait(&acc_full[acc], acc_phase, 0x24)) { ok = false; break; }
      tc::tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(lg * 32) << 16) + acc * BN + half * 128;
      const bool rows_live = m0 < g.M;
      if (EPI == EPI_BF16 && EMODE == 1 && g.sw_out != nullptr) {
        // this warp: columns [half*64, +64) of the tile's gate block and of its up block; gate and up go out rounded to
        // bf16, and silu(gate) * up is computed from those rounded values (what a separate pass over the output reads)
        const uint32_t tg = tmem_base + ((uint32_t)(lg * 32) << 16) + acc * BN + half * 64;
        const int cg = w.nt * 128 + half * 64;                 // column of the gate slab; the up slab sits sw_I further
        uint32_t gp[32], up[32];
        {
          uint32_t r[32], r2[32];
          tc::tmem_ld32(tg, r);
          tc::tmem_ld32(tg + 32, r2);
          tc::tmem_ld_wait();
          if (F8) scale64(r, r2, g.out_scale);
          pack64(r, r2, gp);
          tc::tmem_ld32(tg + 128, r);
          tc::tmem_ld32(tg + 160, r2);
          tc::tmem_ld_wait();
          if (F8) scale64(r, r2, g.out_scale);
          pack64(r, r2, up);
        }
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive_cluster(tc::mapa_u32(tc::smem_u32(&acc_empty[acc]), 0));   // accumulator is in registers
        if (rows_live) {
          bf16* o = (bf16*)g.out;
          slab_store_bf16(my_stage, lane, gp, o, g.ldo, m0, cg, g.M, g.sw_I);
          slab_store_bf16(my_stage, lane, up, o + g.sw_I, g.ldo, m0, cg, g.M, g.sw_I);
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const float g0 = __uint_as_float(gp[i] << 16), g1 = __uint_as_float(gp[i] & 0xffff0000u);
            const float u0 = __uint_as_float(up[i] << 16), u1 = __uint_as_float(up[i] & 0xffff0000u);
            gp[i] = pack_bf16(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
          }
          slab_store_bf16(my_stage, lane, gp, g.sw_out, g.sw_I, m0, cg, g.M, g.sw_I);
        }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < SLABS; c++) {
        uint8_t* buf = my_stage + (EMODE == 0 ? (slab & 1) * 4096 : 0);
        uint32_t r[32], r2[32];
        tc::tmem_ld32(taddr + c * SLAB_COLS, r);
        if (EPI == EPI_BF16) tc::tmem_ld32(taddr + c * SLAB_COLS + 32, r2);
        tc::tmem_ld_wait();
        const int col0 = n0 + c * SLAB_COLS;
        if (!rows_live || col0 >= g.N) continue;   // warp-uniform
        if (EMODE == 0) {
          if (lane == 0) tc::tma_wait_group_read<1>();   // the transfer that last used this buffer has read it
          __syncwarp();
        }
        uint8_t* rowp = buf + lane * 128;
        if (EPI == EPI_BF16) {
          if (F8) scale64(r, r2, g.out_scale);
          if (POS && g.pos != nullptr && m0 + lane < g.M) {
            // this lane's row of the position table, columns col0 .. col0 + 63 (clipped to N): eight 16-byte loads
            const bf16* prow = g.pos + (size_t)((m0 + lane) % g.pos_period) * g.N + col0;
#pragma unroll
            for (int v = 0; v < 8; v++) {
              if (col0 + v * 8 < g.N) {
                const uint4 pv = __ldg(reinterpret_cast<const uint4*>(prow) + v);
                const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                  uint32_t* d = (v < 4) ? &r[v * 8 + 2 * e] : &r2[(v - 4) * 8 + 2 * e];
                  d[0] = __float_as_uint(__uint_as_float(d[0]) + __uint_as_float(pw[e] << 16));
                  d[1] = __float_as_uint(__uint_as_float(d[1]) + __uint_as_float(pw[e] & 0xffff0000u));
                }
              }
            }
          }
          if (DELTA && g.dl_o != nullptr && m0 + lane < g.M) {
            // the slab is one head of this lane's row: dot of its 64 fp32 values with the forward pass's attention output
            const bf16* orow = g.dl_o + (size_t)(m0 + lane) * g.N + col0;
            float acc_d = 0.f;
#pragma unroll
            for (int v = 0; v < 8; v++) {
              const uint4 ov = __ldg(reinterpret_cast<const uint4*>(orow) + v);
              const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
              const uint32_t* d = (v < 4) ? &r[v * 8] : &r2[(v - 4) * 8];
#pragma unroll
              for (int e = 0; e < 4; e++) {
                acc_d = fmaf(__uint_as_float(d[2 * e]), __uint_as_float(ow[e] << 16), acc_d);
                acc_d = fmaf(__uint_as_float(d[2 * e + 1]), __uint_as_float(ow[e] & 0xffff0000u), acc_d);
              }
            }
            const int row = m0 + lane, bb = row / g.dl_T;
            g.dl_out[((size_t)bb * g.dl_H + (col0 >> 6)) * g.dl_T + (row - bb * g.dl_T)] = acc_d;
          }
          if (g.cosT != nullptr && col0 < g.rope_cols) {   // warp-uniform; the slab is one head: r = first half, r2 = second
            const int t = (m0 + lane) % g.rope_T;
            const float4* c4 = reinterpret_cast<const float4*>(g.cosT + (size_t)t * 32);
            const float4* s4 = reinterpret_cast<const float4*>(g.sinT + (size_t)t * 32);
#pragma unroll
            for (int q = 0; q < 8; q++) {
              const float4 c = __ldg(c4 + q), sn = __ldg(s4 + q);
              const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
              for (int e = 0; e < 4; e++) {
                const float x0 = __uint_as_float(r[q * 4 + e]), x1 = __uint_as_float(r2[q * 4 + e]);
                r[q * 4 + e] = __float_as_uint(x0 * cc[e] - x1 * ss[e]);
                r2[q * 4 + e] = __float_as_uint(x1 * cc[e] + x0 * ss[e]);
              }
            }
          }
#pragma unroll
          for (int v = 0; v < 8; v++) {
            const uint32_t* src = (v < 4) ? &r[v * 8] : &r2[(v - 4) * 8];
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(src[0]), __uint_as_float(src[1]));
            pk.y = pack_bf16(__uint_as_float(src[2]), __uint_as_float(src[3]));
            pk.z = pack_bf16(__uint_as_float(src[4]), __uint_as_float(src[5]));
            pk.w = pack_bf16(__uint_as_float(src[6]), __uint_as_float(src[7]));
            *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = pk;
          }
        } else {
#pragma unroll
          for (int v = 0; v < 8; v++) {
            uint4 pk = make_uint4(r[v * 4 + 0], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = pk;
          }
        }
        if (EMODE == 0) {
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (EPI == EPI_BF16) tc::tma_store_2d(&tmD, buf, col0, m0);
            else tc::tma_reduce_add_2d(&tmD, buf, col0, m0);
            tc::tma_commit_group();
          }
        } else {
          __syncwarp();
          const int ch = lane & 7, gcol = col0 + ch * (16 / ELEM);
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int row = i * 4 + (lane >> 3);
            const uint4 v = *reinterpret_cast<const uint4*>(buf + row * 128 + ((ch ^ (row & 7)) << 4));
            if (m0 + row < g.M && gcol < g.N) {
              uint8_t* dst = (uint8_t*)g.out + ((size_t)(m0 + row) * g.ldo + gcol) * ELEM;
              if (EPI == EPI_BF16) {
                *reinterpret_cast<uint4*>(dst) = v;
              } else {
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v.x)),
                             "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                             : "memory");
              }
            }
          }
          __syncwarp();   // the buffer is rewritten by the next slab
        }
        slab++;
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive_cluster(tc::mapa_u32(tc::smem_u32(&acc_empty[acc]), 0));
    }
    if (EMODE == 0 && lane == 0) tc::tma_wait_group<0>();
  }
  tc::tc_fence_before();
  tc::cluster_sync();      // no CTA frees TMEM or exits while its peer may still signal or read it
  if (warp == 1) tc::tmem_dealloc_pair(tmem_base, 2 * BN);
}

// ------------------------------------------------------------------ SIMT fallback (any shape / alignment)
// D[m,n] = sum_k A[m*sam + k*sak] * B[n*sbn + k*sbk]; 64x64 tile, 16x16 threads, 4x4 per thread.
template <int EPI>
__global__ void __launch_bounds__(256) gemm_simt_kernel(void* out, const bf16* __restrict__ A, const bf16* __restrict__ B,
                                                        int M, int N, int K, long sam, long sak, long sbn, long sbk, int ldo) {
  __shared__ float sA[16][65], sB[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      int kk, mm;
      if (sak == 1) { kk = i & 15; mm = i >> 4; } else { mm = i & 63; kk = i >> 6; }
      int gm = m0 + mm, gk = k0 + kk;
      sA[kk][mm] = (gm < M && gk < K) ? __bfloat162float(A[gm * sam + gk * sak]) : 0.f;
    }
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      int kk, nn;
      if (sbk == 1) { kk = i & 15; nn = i >> 4; } else { nn = i & 63; kk = i >> 6; }
      int gn = n0 + nn, gk = k0 + kk;
      sB[kk][nn] = (gn < N && gk < K) ? __bfloat162float(B[gn * sbn + gk * sbk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; kk++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = sA[kk][ty * 4 + i]; b[i] = sB[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; i++)
    for (int j = 0; j < 4; j++) {
      int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < M && gn < N) {
        if (EPI == EPI_BF16) ((bf16*)out)[(size_t)gm * ldo + gn] = __float2bfloat16(acc[i][j]);
        else ((float*)out)[(size_t)gm * ldo + gn] += acc[i][j];
      }
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

std::mutex g_tmap_mu;
typedef std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t, int> TmapKey;
std::map<TmapKey, CUtensorMap*> g_tmaps;
// The cache is keyed on base pointers.  A training step uses a few hundred distinct (pointer, shape) pairs; a caller
// whose allocator hands out ever new addresses would grow it without bound, so it is emptied when it reaches this many
// entries.  The maps themselves are never freed before that point is long past: kernels receive them BY VALUE
// (__grid_constant__ parameters), so a launch that is still queued does not read this memory; entries dropped here are
// parked on a retired list that is released at the following reset.
constexpr size_t TMAP_CACHE_MAX = 8192;
std::vector<CUtensorMap*> g_tmaps_retired;
void tmap_cache_trim_locked() {
  if (g_tmaps.size() < TMAP_CACHE_MAX) return;
  for (CUtensorMap* m : g_tmaps_retired) delete m;
  g_tmaps_retired.clear();
  for (auto& kv : g_tmaps)
    if (kv.second) g_tmaps_retired.push_back(kv.second);
  g_tmaps.clear();
}

}  // namespace

bool mlb_make_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                   uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  if (((uintptr_t)base & 15) || ((pitch_elems * elem_bytes) & 15) || box_cols * elem_bytes != 128) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : (elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

const CUtensorMap* mlb_tmap_cached(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                                   uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  TmapKey key(base, rows, cols, pitch_elems, box_rows, box_cols, elem_bytes);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) return it->second;
  tmap_cache_trim_locked();
  CUtensorMap* m = new CUtensorMap;
  if (!mlb_make_tmap(m, base, rows, cols, pitch_elems, box_rows, box_cols, elem_bytes)) { delete m; return nullptr; }
  g_tmaps[key] = m;
  return m;
}

const CUtensorMap* mlb_tmap_mn3d_cached(const void* base, uint64_t k_rows, uint64_t mn_cols, uint64_t pitch_elems, uint32_t chunks) {
  EncodeTiledFn enc = get_encode();
  if (!enc || (mn_cols % 64) != 0 || ((uintptr_t)base & 15) || ((pitch_elems * 2) & 15)) return nullptr;
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  TmapKey key(base, k_rows, mn_cols, pitch_elems, chunks, 0xffffffffu, -3);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) return it->second;
  tmap_cache_trim_locked();
  CUtensorMap* m = new CUtensorMap;
  cuuint64_t dims[3] = {64, k_rows, mn_cols / 64};
  cuuint64_t strides[2] = {pitch_elems * 2, 128};
  cuuint32_t box[3] = {64, 64, chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { delete m; g_tmaps[key] = nullptr; return nullptr; }
  g_tmaps[key] = m;
  return m;
}

namespace {

int g_use_3d = 1;            // tuning hook: 0 = always use 64-wide 2-D boxes for MN-major operands
int g_num_sms = 0;
int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

int g_force_simt = 0;        // test hook: route everything through the SIMT kernel
int g_max_ctas = 0;          // 0 = one CTA per SM; >0 caps the persistent grid (leaves SMs to a concurrent kernel)
int g_force_splits = 0;      // tuning hook: >0 overrides the split-K heuristic of the weight-gradient GEMM

template <int BN, bool A_MN, bool B_MN, int EPI>
int launch_tc(const CUtensorMap* tmA, const CUtensorMap* tmB, const CUtensorMap* tmD, const GemmArgs& g, cudaStream_t st) {
  auto kern = gemm_tc_kernel<BN, A_MN, B_MN, EPI>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  int total = g.tiles_m * g.tiles_n * g.splits;
  int cap = g_max_ctas > 0 ? g_max_ctas : num_sms();
  int grid = total < cap ? total : cap;
  GatherArgs none{};
  return (int)mlb_launch_tmem(kern, dim3(grid), dim3(GEMM_THREADS), GemmSmem<BN>::TOTAL, st, *tmA, *tmB, *tmD, g, none);
}

// CTA-pair kernel: one cluster of two CTAs per SM pair; the grid is sized from the number of clusters that can be
// resident at once (a GPC with an odd number of usable SMs leaves one without a partner), so the static tile
// schedule never waits for a second wave of CTAs.
int g_use_pairs = 1;         // tuning hook: 0 = always the 1-CTA kernel
int g_tile_order = 0;        // tuning hook: 0 = by operand size, 1 = M first, 2 = N first
int g_sk_groups = 1;         // tuning hook: 0 = stream-K without groups (one linear range per cluster)
int g_streamk = 1;           // tuning hook: weight-gradient products cut into equal k-block ranges per cluster
int g_epi_mode = 1;          // tuning hook: pair kernel's epilogue, 0 = TMA store / reduce, 1 = coalesced stores by the warps
int g_small_tiles = 1;       // tuning hook: 0 = never trade the CTA-pair tile for 128 x 128 tiles on small problems
template <bool A_MN, bool B_MN, int EPI, int EMODE, bool POS = false, bool DELTA = false>
int launch_tc2(const CUtensorMap* tmA, const CUtensorMap* tmB, const CUtensorMap* tmD, const GemmArgs& g, cudaStream_t st) {
  using Gemm2Smem = Gemm2Smem<EMODE>;
  auto kern = gemm_tc2_kernel<A_MN, B_MN, EPI, EMODE, false, POS, DELTA>;
  static int max_clusters = -1;
  if (max_clusters < 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Smem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms() & ~1);
    cfg.blockDim = dim3(GEMM2_THREADS);
    cfg.dynamicSmemBytes = Gemm2Smem::TOTAL;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = num_sms() / 2; }
    max_clusters = n < num_sms() / 2 ? n : num_sms() / 2;
  }
  int total = g.streamk ? g.tiles_m * g.tiles_n * g.kb_total : g.tiles_m * g.tiles_n * g.splits;
  int cap = max_clusters;
  if (g_max_ctas > 0 && g_max_ctas / 2 < cap) cap = g_max_ctas / 2 > 0 ? g_max_ctas / 2 : 1;
  int clusters = total < cap ? total : cap;
  return (int)mlb_launch_tmem(kern, dim3(2 * clusters), dim3(GEMM2_THREADS), Gemm2Smem::TOTAL, st, *tmA, *tmB, *tmD, g);
}
int pair_clusters() { return (g_max_ctas > 0 ? g_max_ctas : num_sms()) / 2; }

// Cooperative launch of the gather variant (all CTAs must be co-resident because tiles wait on other CTAs' pieces).
template <int BN, bool B_MN>
int launch_tc_gather(const CUtensorMap* tmA, const CUtensorMap* tmB, const CUtensorMap* tmD, GemmArgs g, GatherArgs ga, cudaStream_t st) {
  auto kern = gemm_tc_kernel<BN, false, B_MN, EPI_BF16, true>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  int total = g.tiles_m * g.tiles_n * g.splits;
  int cap = g_max_ctas > 0 ? g_max_ctas : num_sms();
  int grid = total < cap ? total : cap;
  CUtensorMap a = *tmA, b = *tmB, d = *tmD;
  void* args[] = {&a, &b, &d, &g, &ga};
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(GEMM_THREADS + 128), args, GemmSmem<BN>::TOTAL, st);
  return (int)e;
}

// Generic entry: D[M,N] (+)= sum_k A(m,k) B(n,k).
// A_MN=false: A is [M,K] row-major with pitch lda.  A_MN=true: A is stored [K,M] row-major with pitch lda.
// Same for B with N.  EPI_BF16 stores bf16; EPI_F32_ADD accumulates into fp32.
struct RopeEpi { const float* cosT; const float* sinT; int T, cols; };
struct SwigluEpi { bf16* out; int I; };
struct PosEpi { const bf16* pos; int period; };
struct DeltaEpi { const bf16* o; float* out; int T, H; };
template <bool A_MN, bool B_MN, int EPI>
int gemm_dispatch_impl(void* out, int ldo, const bf16* A, int lda, const bf16* B, int ldb, int M, int N, int K, cudaStream_t st,
                       const RopeEpi* rope = nullptr, const SwigluEpi* swi = nullptr, const PosEpi* pe = nullptr,
                       const DeltaEpi* dl = nullptr) {
  bool aligned = ((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0) && (lda % 8 == 0) && (ldb % 8 == 0) &&
                 ((uintptr_t)out % 16 == 0) && (ldo % 8 == 0) && (N % 8 == 0) && M > 0 && N > 0 && K > 0;
  // MN-major operands are fetched in 64-wide chunks along M/N: the global extent must be a multiple of 8 elements
  // (16 bytes) for the tensor map; out-of-range chunks are zero-filled by TMA.
  if (A_MN) aligned = aligned && (M % 8 == 0);
  if (B_MN) aligned = aligned && (N % 8 == 0);
  if (!A_MN || !B_MN) aligned = aligned && (K % 8 == 0);
  if (rope && (g_force_simt || !aligned || get_encode() == nullptr)) return -7;   // caller rotates separately
  if (swi && (g_force_simt || !aligned || get_encode() == nullptr || g_epi_mode != 1 || !g_use_pairs || A_MN || B_MN ||
              EPI != EPI_BF16 || N != 2 * swi->I || swi->I % 128 != 0 || M <= 128 || ((uintptr_t)swi->out & 15)))
    return -7;                                                                       // caller runs the separate kernel
  if (pe && (g_force_simt || !aligned || get_encode() == nullptr || g_epi_mode != 1 || !g_use_pairs || EPI != EPI_BF16 || M <= 128 ||
             N <= 128 || N % 8 != 0 || ((uintptr_t)pe->pos & 15) || pe->period < 1))
    return -7;
  if (dl && (g_force_simt || !aligned || get_encode() == nullptr || g_epi_mode != 1 || !g_use_pairs || A_MN || !B_MN || EPI != EPI_BF16 ||
             M <= 128 || N <= 128 || N != dl->H * 64 || M % dl->T != 0 || ((uintptr_t)dl->o & 15)))
    return -7;                                                                       // caller runs the separate kernels
  if (g_force_simt || !aligned || get_encode() == nullptr) {
    dim3 grid(ceil_div_i(N, 64), ceil_div_i(M, 64));
    long sam = A_MN ? 1 : lda, sak = A_MN ? lda : 1, sbn = B_MN ? 1 : ldb, sbk = B_MN ? ldb : 1;
    gemm_simt_kernel<EPI><<<grid, 256, 0, st>>>(out, A, B, M, N, K, sam, sak, sbn, sbk, ldo);
    return (int)cudaGetLastError();
  }
  // Tile shape.  Large products run on CTA pairs (256 x 256 per SM pair: least operand traffic per FLOP).  When such tiles
  // are too few to occupy the machine (a skinny output at a small token count, e.g. M = 2048, N = 768: 24 pair tiles for
  // 74 SM pairs) the 1-CTA kernel with 128 x 128 tiles has the same multiply rate per SM and four times as many tiles.
  // Estimated cycles: waves x (k-blocks x cycles per k-block + a fixed cost per tile for ramp and epilogue); the 128-wide
  // tile pays ~25 % more per k-block for its operand traffic.
  int BN = (N > 128) ? 256 : 128;
  bool pairs = g_use_pairs && BN == 256 && M > 128;   // 256 x 256 tile shared by a CTA pair
  if (pairs && !rope && !swi && !pe && !dl && g_small_tiles) {
    const long kb = ceil_div_i(K, BK);
    const long pt = (long)ceil_div_i(M, 256) * ceil_div_i(N, 256), ct = (long)ceil_div_i(M, 128) * ceil_div_i(N, 128);
    const long pc = pair_clusters(), sm = g_max_ctas > 0 ? g_max_ctas : num_sms();
    double cost_pair, cost_c128;
    if (EPI == EPI_F32_ADD) {       // both forms split the reduction to fill the machine
      cost_pair = (double)pt * kb / pc * 512.0 + 4000.0;
      cost_c128 = (double)ct * kb / sm * 320.0 + 3000.0;
      if (ct * kb / 8 < sm) cost_c128 = 1e30;      // too little work per CTA even at the smallest split
    } else {
      cost_pair = (double)((pt + pc - 1) / pc) * (kb * 512.0 + 2000.0);
      cost_c128 = (double)((ct + sm - 1) / sm) * (kb * 320.0 + 2000.0);
    }
    if (cost_c128 < 0.8 * cost_pair) { pairs = false; BN = 128; }
  }
  if (rope && !(pairs && rope->cols % 64 == 0 && N % 64 == 0)) return -7;
  GemmArgs g;
  g.cosT = rope ? rope->cosT : nullptr; g.sinT = rope ? rope->sinT : nullptr;
  g.rope_T = rope ? rope->T : 1; g.rope_cols = rope ? rope->cols : 0;
  g.sw_out = swi ? swi->out : nullptr; g.sw_I = swi ? swi->I : 0; g.out_scale = 1.f;
  g.pos = pe ? pe->pos : nullptr; g.pos_period = pe ? pe->period : 1;
  g.dl_o = dl ? dl->o : nullptr; g.dl_out = dl ? dl->out : nullptr; g.dl_T = dl ? dl->T : 1; g.dl_H = dl ? dl->H : 1;
  g.out = out; g.M = M; g.N = N; g.K = K; g.ldo = ldo;
  g.tiles_m = ceil_div_i(M, pairs ? 256 : BM);
  g.tiles_n = swi ? swi->I / 128 : ceil_div_i(N, BN);
  g.kb_total = ceil_div_i(K, BK);
  g.splits = 1;
  if (EPI == EPI_F32_ADD) {
    // split the reduction so the persistent grid is filled: choose the split count with the best last-wave fill
    int tiles = g.tiles_m * g.tiles_n, sms = pairs ? pair_clusters() : (g_max_ctas > 0 ? g_max_ctas : num_sms());
    int best = 1;
    double best_eff = 0;
    for (int s = 1; s <= 32; s++) {
      if (g.kb_total / s < 8 && s > 1) break;
      long w = (long)tiles * s;
      double eff = (double)w / ((double)((w + sms - 1) / sms) * sms);
      if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
    }
    g.splits = best;
    if (g_force_splits > 0) g.splits = g_force_splits;
  }
  g.kb_per_split = ceil_div_i(g.kb_total, g.splits);
  g.splits = ceil_div_i(g.kb_total, g.kb_per_split);
  g.a3d = g.b3d = 0;
  g.streamk = (pairs && EPI == EPI_F32_ADD && g_streamk && g_force_splits == 0) ? 1 : 0;
  // Tiles in flight should share the operand that does not fit in L2: walk N first when A is the larger one.
  g.nt_fast = (g_tile_order == 2) ? 1 : (g_tile_order == 1 ? 0 : ((long)M > (long)N ? 1 : 0));
  g.sk_group = 1; g.sk_group_m = 0;
  if (g.streamk) {
    // group along the dimension with fewer tiles (its operand is the narrow one); at most 4 members, else plain stream-K
    const int short_tiles = g.tiles_m < g.tiles_n ? g.tiles_m : g.tiles_n;
    if (g_sk_groups && short_tiles <= 4 && short_tiles >= 1 && pair_clusters() >= 4 * short_tiles) { g.sk_group = short_tiles; g.sk_group_m = g.tiles_m < g.tiles_n ? 1 : 0; }
  }
  const CUtensorMap* tmA = nullptr;
  const CUtensorMap* tmB = nullptr;
  if (A_MN && g_use_3d) { tmA = mlb_tmap_mn3d_cached(A, K, M, lda, BM / 64); g.a3d = tmA != nullptr; }
  const int b_rows = pairs ? 128 : BN;   // rows of B one CTA stages
  if (B_MN && g_use_3d) { tmB = mlb_tmap_mn3d_cached(B, K, N, ldb, b_rows / 64); g.b3d = tmB != nullptr; }
  if (!tmA) tmA = A_MN ? mlb_tmap_cached(A, K, M, lda, 64, 64) : mlb_tmap_cached(A, M, K, lda, BM, 64);
  if (!tmB) tmB = B_MN ? mlb_tmap_cached(B, K, N, ldb, 64, 64) : mlb_tmap_cached(B, N, K, ldb, b_rows, 64);
  const CUtensorMap* tmD = (EPI == EPI_BF16) ? mlb_tmap_cached(out, M, N, ldo, 32, 64, 2) : mlb_tmap_cached(out, M, N, ldo, 32, 32, 4);
  if (!tmA || !tmB || !tmD) return -2;
  if constexpr (!A_MN && !B_MN && EPI == EPI_BF16) {
    if (pairs && pe) return launch_tc2<false, false, EPI_BF16, 1, true>(tmA, tmB, tmD, g, st);
  }
  if constexpr (!A_MN && B_MN && EPI == EPI_BF16) {
    if (dl) return pairs ? launch_tc2<false, true, EPI_BF16, 1, false, true>(tmA, tmB, tmD, g, st) : -7;
  }
  if (pairs && g_epi_mode == 0) return launch_tc2<A_MN, B_MN, EPI, 0>(tmA, tmB, tmD, g, st);
  if (pairs) return launch_tc2<A_MN, B_MN, EPI, 1>(tmA, tmB, tmD, g, st);
  if (BN == 256) return launch_tc<256, A_MN, B_MN, EPI>(tmA, tmB, tmD, g, st);
  return launch_tc<128, A_MN, B_MN, EPI>(tmA, tmB, tmD, g, st);
}

// ------------------------------------------------------------------ plan cache + autotune (ENTROPY_AUTOTUNE, train/gemm.cuh)
// The reference times the library's top-k algorithms per GEMM shape and caches the winner.  Here the candidates are
// this file's own forms: tile (CTA-pair tiles forced / chosen by the cost model / 1-CTA kernel), order of the tiles
// in flight (M first / N first), epilogue (TMA store or reduce / coalesced stores by the warps) and, for the fp32
// add-reduce products, stream-K on / off and its grouping.  With autotuning on, the first call of a shape outside
// graph capture runs every candidate a few times on the call's own operands (add-reduce products into a scratch
// output), keeps the fastest in a per-process cache, and every call of that shape then runs with its plan.
struct GemmPlan { int tile, order, epi, streamk, skg; float us; };
int g_autotune = 0;
static std::map<std::array<int, 7>, GemmPlan> g_plans;
static std::mutex g_plans_mu;
struct PlanScope {      // applies a plan to the tuning globals for one dispatch
  int pairs, small, order, epi, sk, skg;
  explicit PlanScope(const GemmPlan& p) : pairs(g_use_pairs), small(g_small_tiles), order(g_tile_order), epi(g_epi_mode), sk(g_streamk), skg(g_sk_groups) {
    g_use_pairs = p.tile != 2; g_small_tiles = p.tile == 1; g_tile_order = p.order; g_epi_mode = p.epi; g_streamk = p.streamk; g_sk_groups = p.skg;
  }
  ~PlanScope() { g_use_pairs = pairs; g_small_tiles = small; g_tile_order = order; g_epi_mode = epi; g_streamk = sk; g_sk_groups = skg; }
};
template <bool A_MN, bool B_MN, int EPI>
int gemm_dispatch(void* out, int ldo, const bf16* A, int lda, const bf16* B, int ldb, int M, int N, int K, cudaStream_t st,
                  const RopeEpi* rope = nullptr, const SwigluEpi* swi = nullptr, const PosEpi* pe = nullptr) {
  if (!g_autotune || g_force_simt) return gemm_dispatch_impl<A_MN, B_MN, EPI>(out, ldo, A, lda, B, ldb, M, N, K, st, rope, swi, pe);
  const std::array<int, 7> key = {(A_MN ? 4 : 0) | (B_MN ? 2 : 0) | (EPI == EPI_F32_ADD ? 1 : 0), M, N, K,
                                  (rope ? 1 : 0) | (swi ? 2 : 0) | (pe ? 4 : 0), ldo, lda * 131 + ldb};
  GemmPlan plan{};
  bool have = false;
  {
    std::lock_guard<std::mutex> lk(g_plans_mu);
    auto it = g_plans.find(key);
    if (it != g_plans.end()) { plan = it->second; have = true; }
  }
  if (!have) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return gemm_dispatch_impl<A_MN, B_MN, EPI>(out, ldo, A, lda, B, ldb, M, N, K, st, rope, swi, pe);   // no timing inside a capture
    }
    void* tune_out = out;
    void* scratch = nullptr;
    if (EPI == EPI_F32_ADD) {      // the candidates must not add to the caller's accumulator
      if (cudaMalloc(&scratch, (size_t)M * ldo * sizeof(float)) != cudaSuccess) { cudaGetLastError(); scratch = nullptr; }
      tune_out = scratch;
    }
    plan = GemmPlan{1, 0, 1, 1, 1, 0.f};       // the static heuristics
    if (tune_out != nullptr) {
      cudaEvent_t e0, e1;
      cudaEventCreate(&e0);
      cudaEventCreate(&e1);
      float best = 1e30f;
      const bool fixed_epi = rope || swi || pe;      // these epilogues exist in one form only
      for (int tile = 0; tile < (fixed_epi ? 1 : 3); tile++)
        for (int order = 1; order <= 2; order++)
          for (int epi = fixed_epi ? 1 : 0; epi < 2; epi++)
            for (int sk = (EPI == EPI_F32_ADD) ? 0 : 1; sk < 2; sk++)
              for (int skg = (EPI == EPI_F32_ADD && sk) ? 0 : 1; skg < 2; skg++) {
                GemmPlan c{fixed_epi ? 1 : tile, order, epi, sk, skg, 0.f};
                PlanScope scope(c);
                if (gemm_dispatch_impl<A_MN, B_MN, EPI>(tune_out, ldo, A, lda, B, ldb, M, N, K, st, rope, swi, pe) != 0) { cudaGetLastError(); continue; }
                cudaEventRecord(e0, st);
                int rc = 0;
                for (int i = 0; i < 3 && rc == 0; i++) rc = gemm_dispatch_impl<A_MN, B_MN, EPI>(tune_out, ldo, A, lda, B, ldb, M, N, K, st, rope, swi, pe);
                cudaEventRecord(e1, st);
                if (cudaEventSynchronize(e1) != cudaSuccess || rc != 0) { cudaGetLastError(); continue; }
                float ms = 0.f;
                cudaEventElapsedTime(&ms, e0, e1);
                c.us = ms * 1000.f / 3.f;
                if (c.us < best) { best = c.us; plan = c; }
              }
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
    }
    if (scratch) cudaFree(scratch);
    std::lock_guard<std::mutex> lk(g_plans_mu);
    g_plans[key] = plan;
  }
  PlanScope scope(plan);
  return gemm_dispatch_impl<A_MN, B_MN, EPI>(out, ldo, A, lda, B, ldb, M, N, K, st, rope, swi, pe);
}

// 8-bit forward product on the CTA-pair kernel: out[M,N] (bf16) = out_scale * x8[M,K] . W8[N,K]^T, operands E4M3 bytes.
int gemm_fp8_dispatch(void* out, int ldo, const uint8_t* A, int lda, const uint8_t* B, int ldb, int M, int N, int K, float out_scale,
                      cudaStream_t st, const SwigluEpi* swi, const RopeEpi* rope = nullptr) {
  const bool ok = ((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0) && (lda % 16 == 0) && (ldb % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                  (ldo % 8 == 0) && (N % 8 == 0) && (K % 16 == 0) && M > 128 && N > 128 && K > 0 && get_encode() != nullptr &&
                  g_use_pairs && g_epi_mode == 1 && !g_force_simt;
  if (!ok) return -7;
  if (swi && (N != 2 * swi->I || swi->I % 128 != 0 || ((uintptr_t)swi->out & 15))) return -7;
  if (rope && !(rope->cols % 64 == 0 && N % 64 == 0)) return -7;
  GemmArgs g;
  g.cosT = rope ? rope->cosT : nullptr; g.sinT = rope ? rope->sinT : nullptr;
  g.rope_T = rope ? rope->T : 1; g.rope_cols = rope ? rope->cols : 0;
  g.sw_out = swi ? swi->out : nullptr; g.sw_I = swi ? swi->I : 0; g.out_scale = out_scale;
  g.pos = nullptr; g.pos_period = 1; g.dl_o = nullptr; g.dl_out = nullptr; g.dl_T = 1; g.dl_H = 1;
  g.out = out; g.M = M; g.N = N; g.K = K; g.ldo = ldo;
  g.tiles_m = ceil_div_i(M, 256);
  g.tiles_n = swi ? swi->I / 128 : ceil_div_i(N, 256);
  g.kb_total = ceil_div_i(K, 128);
  g.splits = 1; g.kb_per_split = g.kb_total; g.a3d = g.b3d = 0; g.streamk = 0; g.sk_group = 1; g.sk_group_m = 0;
  g.nt_fast = (g_tile_order == 2) ? 1 : (g_tile_order == 1 ? 0 : ((long)M > (long)N ? 1 : 0));
  const CUtensorMap* tmA = mlb_tmap_cached(A, M, K, lda, 128, 128, 1);
  const CUtensorMap* tmB = mlb_tmap_cached(B, N, K, ldb, 128, 128, 1);
  const CUtensorMap* tmD = mlb_tmap_cached(out, M, N, ldo, 32, 64, 2);
  if (!tmA || !tmB || !tmD) return -2;
  using Smem = Gemm2Smem<1>;
  auto kern = gemm_tc2_kernel<false, false, EPI_BF16, 1, true>;
  static int max_clusters = -1;
  if (max_clusters < 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_sms() & ~1);
    cfg.blockDim = dim3(GEMM2_THREADS);
    cfg.dynamicSmemBytes = Smem::TOTAL;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n <= 0) { cudaGetLastError(); n = num_sms() / 2; }
    max_clusters = n < num_sms() / 2 ? n : num_sms() / 2;
  }
  int total = g.tiles_m * g.tiles_n;
  int cap = max_clusters;
  if (g_max_ctas > 0 && g_max_ctas / 2 < cap) cap = g_max_ctas / 2 > 0 ? g_max_ctas / 2 : 1;
  int clusters = total < cap ? total : cap;
  return (int)mlb_launch_tmem(kern, dim3(2 * clusters), dim3(GEMM2_THREADS), Smem::TOTAL, st, *tmA, *tmB, *tmD, g);
}

}  // namespace

// out[M,N] (bf16) = out_scale * x8[M,K] . W8[N,K]^T with E4M3 operands (tcgen05.mma kind::f8f6f4): the reference's opt-in
// 8-bit forward (linear_forward_fp8, train/gpt_kernels.cuh:171-176, scalar dequant scales :103-112).  Returns -7
// (nothing launched) for shapes the CTA-pair kernel does not take (M, N > 128; K and the pitches multiples of 16).
MLB_API int mlb_linear_fwd_fp8(void* out, const void* x8, const void* W8, int M, int N, int K, int ldo, int ldx, int ldw, float out_scale,
                               cudaStream_t st) {
  return gemm_fp8_dispatch(out, ldo, (const uint8_t*)x8, ldx, (const uint8_t*)W8, ldw, M, N, K, out_scale, st, nullptr);
}
// The QKV product in 8 bits with the rotary embedding in the epilogue (see mlb_linear_fwd_rope).
MLB_API int mlb_linear_fwd_fp8_rope(void* out, const void* x8, const void* W8, int M, int N, int K, int ldo, int ldx, int ldw, float out_scale,
                                    const float* cosT, const float* sinT, int T, int rope_cols, cudaStream_t st) {
  RopeEpi r{cosT, sinT, T, rope_cols};
  return gemm_fp8_dispatch(out, ldo, (const uint8_t*)x8, ldx, (const uint8_t*)W8, ldw, M, N, K, out_scale, st, nullptr, &r);
}
// The gate|up product in 8 bits with silu(gate) * up from the epilogue (see mlb_linear_fwd_swiglu).
MLB_API int mlb_linear_fwd_fp8_swiglu(void* gu, void* sw, const void* x8, const void* W8, int M, int I, int K, int ldgu, int ldx, int ldw,
                                      float out_scale, cudaStream_t st) {
  SwigluEpi e{(bf16*)sw, I};
  return gemm_fp8_dispatch(gu, ldgu, (const uint8_t*)x8, ldx, (const uint8_t*)W8, ldw, M, 2 * I, K, out_scale, st, &e);
}

// out[M,N] = x[M,K] . W[N,K]^T
MLB_API int mlb_linear_fwd(void* out, const void* x, const void* W, int M, int N, int K, int ldo, int ldx, int ldw, cudaStream_t st) {
  return gemm_dispatch<false, false, EPI_BF16>(out, ldo, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, st);
}
// out[M,N] = x[M,K] . W[N,K]^T, then rotary embedding on output columns [0, rope_cols): heads of 64 columns, halves
// (i, i + 32) rotated by the angle of position (row % T); cosT / sinT are [T, 32] fp32.  Returns -7 (nothing launched)
// when the shape does not take the CTA-pair tensor-core path; the caller then runs the plain product and rotates.
MLB_API int mlb_linear_fwd_rope(void* out, const void* x, const void* W, int M, int N, int K, int ldo, int ldx, int ldw,
                                const float* cosT, const float* sinT, int T, int rope_cols, cudaStream_t st) {
  RopeEpi r{cosT, sinT, T, rope_cols};
  return gemm_dispatch<false, false, EPI_BF16>(out, ldo, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, st, &r);
}
// gu[M, 2I] = x[M,K] . W[2I,K]^T with W = [W_gate; W_up], and sw[M, I] = silu(gu[:, :I]) * gu[:, I:] from the same
// accumulators (rounded to bf16 first, so sw equals what the separate SwiGLU kernel computes from gu).  Returns -7
// (nothing launched) when the shape does not take the CTA-pair path (I must be a multiple of 128, M > 128).
MLB_API int mlb_linear_fwd_swiglu(void* gu, void* sw, const void* x, const void* W, int M, int I, int K, int ldgu, int ldx, int ldw,
                                  cudaStream_t st) {
  SwigluEpi e{(bf16*)sw, I};
  return gemm_dispatch<false, false, EPI_BF16>(gu, ldgu, (const bf16*)x, ldx, (const bf16*)W, ldw, M, 2 * I, K, st, nullptr, &e);
}
// out[M,N] = x[M,K] . W[N,K]^T + pos[row % period, :]: the vision tower's patch embedding with the learned positions added
// on the fp32 accumulators in the epilogue (the reference runs linear_forward + add_posembed_k, train/gpt.cu:861-863).
// Returns -7 (nothing launched) when the shape does not take the CTA-pair path (M, N > 128).
MLB_API int mlb_linear_fwd_posembed(void* out, const void* x, const void* W, const void* pos, int period, int M, int N, int K, int ldo,
                                    int ldx, int ldw, cudaStream_t st) {
  PosEpi e{(const bf16*)pos, period};
  return gemm_dispatch<false, false, EPI_BF16>(out, ldo, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, st, nullptr, nullptr, &e);
}
// dx[M,K] = dout[M,N] . W[N,K]      (GEMM view: D[M,K], reduction N; B(n=k_in, k=n_out) is MN-major)
MLB_API int mlb_linear_dx(void* dx, const void* dout, const void* W, int M, int N, int K, int lddx, int lddo, int ldw, cudaStream_t st) {
  return gemm_dispatch<false, true, EPI_BF16>(dx, lddx, (const bf16*)dout, lddo, (const bf16*)W, ldw, M, K, N, st);
}
// dx = dout . W as mlb_linear_dx, for the attention output projection: also delta[b, h, t] = sum_c dx[row, h*64 + c] * o[row, h*64 + c]
// (row = b*T + t, o = the forward pass's attention output [M, H*64]) from the epilogue.  -7: the shape does not take this
// path, nothing was launched.
MLB_API int mlb_linear_dx_delta(void* dx, const void* dout, const void* W, const void* o, float* delta, int T, int H, int M, int N, int K,
                                int lddx, int lddo, int ldw, cudaStream_t st) {
  if (K != H * 64 || lddx != K) return -7;
  DeltaEpi e{(const bf16*)o, delta, T, H};
  return gemm_dispatch_impl<false, true, EPI_BF16>(dx, lddx, (const bf16*)dout, lddo, (const bf16*)W, ldw, M, K, N, st, nullptr, nullptr, nullptr, &e);
}
// dW[N,K] += dout[M,N]^T . x[M,K]   (GEMM view: D[N,K], reduction M; both operands MN-major)
MLB_API int mlb_linear_dw(void* dW, const void* dout, const void* x, int M, int N, int K, int lddw, int lddo, int ldx, cudaStream_t st) {
  return gemm_dispatch<true, true, EPI_F32_ADD>(dW, lddw, (const bf16*)dout, lddo, (const bf16*)x, ldx, N, K, M, st);
}

// General entry: D[M,N] = sum_k A(m,k) B(n,k), bf16 store (accumulate = 0) or fp32 += (accumulate = 1).
//   a_mn = 0: A stored [M,K] (K contiguous, pitch lda);  a_mn = 1: A stored [K,M] (M contiguous, pitch lda); same for B with N.
MLB_API int mlb_gemm(void* out, const void* A, const void* B, int M, int N, int K, int ldo, int lda, int ldb, int a_mn, int b_mn,
                     int accumulate, cudaStream_t st) {
  const bf16* a = (const bf16*)A;
  const bf16* b = (const bf16*)B;
  const int sel = (a_mn ? 4 : 0) | (b_mn ? 2 : 0) | (accumulate ? 1 : 0);
  switch (sel) {
    case 0: return gemm_dispatch<false, false, EPI_BF16>(out, ldo, a, lda, b, ldb, M, N, K, st);
    case 1: return gemm_dispatch<false, false, EPI_F32_ADD>(out, ldo, a, lda, b, ldb, M, N, K, st);
    case 2: return gemm_dispatch<false, true, EPI_BF16>(out, ldo, a, lda, b, ldb, M, N, K, st);
    case 3: return gemm_dispatch<false, true, EPI_F32_ADD>(out, ldo, a, lda, b, ldb, M, N, K, st);
    case 4: return gemm_dispatch<true, false, EPI_BF16>(out, ldo, a, lda, b, ldb, M, N, K, st);
    case 5: return gemm_dispatch<true, false, EPI_F32_ADD>(out, ldo, a, lda, b, ldb, M, N, K, st);
    case 6: return gemm_dispatch<true, true, EPI_BF16>(out, ldo, a, lda, b, ldb, M, N, K, st);
    default: return gemm_dispatch<true, true, EPI_F32_ADD>(out, ldo, a, lda, b, ldb, M, N, K, st);
  }
}

// out[M,N] = x[M,K] . W[N,K]^T where W lies inside a sharded parameter unit that this launch also all-gathers:
//   unit_dst    local gather slot (start of the unit, 16-byte aligned), W == unit_dst + w_off_elems
//   src_ptrs    device array [world] of the ranks' shard bases; every shard holds shard_elems bf16 (multiple of 8)
//   flags       device ints, one per 16 KB piece of the unit (zero-initialised once); ctr: two device ints (zeroed once)
// When the kernel has finished, the WHOLE unit is present in unit_dst (not only W).
MLB_API int mlb_linear_fwd_gather(void* out, const void* x, int M, int N, int K, int ldo, int ldx, void* unit_dst,
                                  long w_off_elems, const void* src_ptrs, long shard_elems, int world, int* flags, int* ctr,
                                  double spin_limit_s, cudaStream_t st) {
  const bf16* W = (const bf16*)unit_dst + w_off_elems;
  const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)out % 16 == 0) && (ldx % 8 == 0) &&
                       (ldo % 8 == 0) && (K % 8 == 0) && (N % 8 == 0) && (shard_elems % 8 == 0) && (w_off_elems % 8 == 0) &&
                       get_encode() != nullptr;
  if (!aligned) return -6;
  const int BN = (N > 128) ? 256 : 128;
  GemmArgs g;
  g.out = out; g.M = M; g.N = N; g.K = K; g.ldo = ldo;
  g.tiles_m = ceil_div_i(M, BM); g.tiles_n = ceil_div_i(N, BN); g.kb_total = ceil_div_i(K, BK);
  g.splits = 1; g.kb_per_split = g.kb_total; g.a3d = g.b3d = 0; g.streamk = 0; g.sk_group = 1; g.sk_group_m = 0; g.nt_fast = 0;
  g.cosT = g.sinT = nullptr; g.rope_T = 1; g.rope_cols = 0; g.sw_out = nullptr; g.sw_I = 0; g.out_scale = 1.f; g.pos = nullptr; g.pos_period = 1; g.dl_o = nullptr; g.dl_out = nullptr; g.dl_T = 1; g.dl_H = 1;
  GatherArgs ga;
  ga.src = (const uint4* const*)src_ptrs; ga.dst = (uint4*)unit_dst; ga.shard_vec = shard_elems / 8;
  ga.b_lo_vec = w_off_elems / 8; ga.b_hi_vec = (w_off_elems + (long)N * K) / 8; ga.b_row_vec = K / 8;
  ga.flags = flags; ga.ctr = ctr; ga.world = world; ga.piece_vec = 1024; ga.spin_limit_ns = (long)(spin_limit_s * 1e9);
  const CUtensorMap* tmA = mlb_tmap_cached(x, M, K, ldx, BM, 64);
  const CUtensorMap* tmB = mlb_tmap_cached(W, N, K, K, BN, 64);
  const CUtensorMap* tmD = mlb_tmap_cached(out, M, N, ldo, 32, 64, 2);
  if (!tmA || !tmB || !tmD) return -2;
  if (BN == 256) return launch_tc_gather<256, false>(tmA, tmB, tmD, g, ga, st);
  return launch_tc_gather<128, false>(tmA, tmB, tmD, g, ga, st);
}

// ------------------------------------------------------------------ tensor-pipe micro-benchmark
// One CTA per SM; one thread issues `reps` groups of four tcgen05.mma (M = 128, K = 16 each, N given) on resident
// shared-memory (or TMEM, for A) operands and waits for their completion: cycles[blockIdx.x] = SM cycles for all of them.
namespace {
template <int N, bool A_TMEM>
__global__ void __launch_bounds__(128, 1) mma_probe_kernel(long long* cycles, int reps) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bar = (uint64_t*)(smem + 16384 + 32768);
  uint32_t* slot = (uint32_t*)(bar + 1);
  for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { tc::mbar_init(bar, 1); tc::mbar_fence_init(); }
  if (threadIdx.x < 32) tc::tmem_alloc(slot, 512);
  tc::fence_async_smem();
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = tc::idesc_bf16(128, N, 0, 0);
    const uint32_t sA = tc::smem_u32(smem), sB = sA + 16384;
    const long long t0 = clock64();
    for (int r = 0; r < reps; r++) {
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const uint64_t db = tc::smem_desc_sw128(sB + k * 32, 16, 1024);
        if (A_TMEM) tc::mma_bf16_ts(tmem, tmem + 256 + k * 8, db, idesc, 1u);
        else tc::mma_bf16_ss(tmem, tc::smem_desc_sw128(sA + k * 32, 16, 1024), db, idesc, 1u);
      }
    }
    tc::mma_commit(bar);
    tc::mbar_wait(bar, 0, 0x70);
    cycles[blockIdx.x] = clock64() - t0;
  }
  tc::tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tc::tmem_dealloc(tmem, 512);
}
}  // namespace
// N in {64, 128, 256}; a_tmem: A operand from TMEM instead of shared memory.  `cycles` holds one int64 per SM.
MLB_API int mlb_mma_probe(long long* cycles, int N, int a_tmem, int reps, cudaStream_t st) {
  const int smem = 16384 + 32768 + 64 + 1024;
#define PROBE(NN, TS)                                                                                         \
  {                                                                                                           \
    cudaFuncSetAttribute(mma_probe_kernel<NN, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);        \
    mma_probe_kernel<NN, TS><<<num_sms(), 128, smem, st>>>(cycles, reps);                                     \
  }
  if (N == 64 && !a_tmem) PROBE(64, false)
  else if (N == 64) PROBE(64, true)
  else if (N == 128 && !a_tmem) PROBE(128, false)
  else if (N == 128) PROBE(128, true)
  else if (N == 256 && !a_tmem) PROBE(256, false)
  else if (N == 256) PROBE(256, true)
  else return -1;
#undef PROBE
  return (int)cudaGetLastError();
}

MLB_API int mlb_tmap_cache_size() { std::lock_guard<std::mutex> lk(g_tmap_mu); return (int)g_tmaps.size(); }
MLB_API void mlb_gemm_force_simt(int on) { g_force_simt = on; }
MLB_API void mlb_gemm_set_max_ctas(int n) { g_max_ctas = n; }
MLB_API void mlb_gemm_set_splits(int n) { g_force_splits = n; }
MLB_API void mlb_gemm_use_3d_maps(int on) { g_use_3d = on; }
MLB_API void mlb_gemm_use_pairs(int on) { g_use_pairs = on; }
// 1: time this file's GEMM forms per shape on first use and keep the fastest (see GemmPlan); 0: static heuristics
MLB_API void mlb_gemm_autotune(int on) { g_autotune = on; }
MLB_API int mlb_gemm_plan_count() { std::lock_guard<std::mutex> lk(g_plans_mu); return (int)g_plans.size(); }
// plan i of the cache in iteration order: {form bits, M, N, K, tile, order, epilogue, stream-K, groups, microseconds}
MLB_API int mlb_gemm_plan_get(int i, int* out10) {
  std::lock_guard<std::mutex> lk(g_plans_mu);
  if (i < 0 || i >= (int)g_plans.size()) return -1;
  auto it = g_plans.begin();
  std::advance(it, i);
  out10[0] = it->first[0]; out10[1] = it->first[1]; out10[2] = it->first[2]; out10[3] = it->first[3];
  out10[4] = it->second.tile; out10[5] = it->second.order; out10[6] = it->second.epi; out10[7] = it->second.streamk;
  out10[8] = it->second.skg; out10[9] = (int)it->second.us;
  return 0;
}
MLB_API void mlb_gemm_epilogue_mode(int m) { g_epi_mode = m; }
MLB_API void mlb_gemm_small_tiles(int on) { g_small_tiles = on; }
MLB_API void mlb_gemm_streamk(int on) { g_streamk = on; }
MLB_API void mlb_gemm_tile_order(int mode) { g_tile_order = mode; }
MLB_API void mlb_gemm_streamk_groups(int on) { g_sk_groups = on; }

MLB_DEFINE_ERROR_WORD(gemm)
