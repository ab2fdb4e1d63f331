// Causal flash attention, forward and backward, on tcgen05 tensor cores with TMEM accumulators.
//
// Replaces the reference's cuDNN-frontend SDPA graphs (train/attn_cudnn.cuh:31-128).  Like them it reads Q, K and V
// strided straight out of qkv[B,T,3C] (one TMA tensor map over the [B*T, 3C] matrix; a head is a 64- or 128-column
// window), writes O into atty[B,T,C], saves the per-row log-sum-exp, and in backward writes dQ, dK, dV strided into
// dqkv[B,T,3C].  Scale 1/sqrt(hd), causal over the whole sequence, no dropout.
//
// Forward, one CTA (128 threads) per 128-query tile: S = Q K^T by tcgen05.mma into TMEM, each thread owns one query
// row (TMEM lane) for the online softmax, P is written bf16 into 128B-swizzled shared memory and fed back as the A
// operand of O_blk = P V (V consumed MN-major, i.e. untransposed), O is rescaled in registers.
// Backward, two kernels that each own their accumulators in TMEM (no atomics, deterministic):
//   dK/dV kernel per 128-key tile:  S^T = K Q^T, dP^T = V dO^T, P^T and dS^T to shared memory, dV += P^T dO, dK += dS^T Q.
//   dQ kernel per 128-query tile:   S = Q K^T, dP = dO V^T, dS to shared memory, dQ += dS K.
// RoPE's backward rotation of dQ/dK can be applied in the epilogue (each thread holds a full head row).
// Head sizes other than 64/128 (or unaligned strides) use a plain SIMT implementation further down.
#include "../tc.cuh"
#include <algorithm>
#include <mutex>
#include <queue>
#include <vector>

MLB_DEFINE_ERROR_WORD(attn)

namespace {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int TILE_BYTES = 128 * 64 * 2;  // one [128 rows x 64 bf16] swizzled chunk = 16 KB

// K-major view of a [128 x (64*chunks)] tile: k-step ks covers 16 elements of the contraction dimension.
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int ks) {
  return tc::smem_desc_sw128(base + (ks >> 2) * TILE_BYTES + (ks & 3) * 32, 16, 1024);
}
// The same descriptors with the address arithmetic left to the caller: base + (byte offset >> 4).  K-major: +2 per
// 16-element k-step inside a 64-column chunk, + TILE_BYTES/16 per chunk; MN-major: +128 per 16-row k-step.
__device__ __forceinline__ uint64_t desc_base_k(uint32_t base) { return tc::smem_desc_sw128(base, 16, 1024); }
__device__ __forceinline__ uint64_t desc_base_mn(uint32_t base) { return tc::smem_desc_sw128(base, TILE_BYTES, 1024); }
// MN-major view of a [128 contraction rows x (64*chunks)] tile: k-step ks covers 16 rows.
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int ks) {
  return tc::smem_desc_sw128(base + ks * 2048, TILE_BYTES, 1024);
}
// Byte offset of element (row r, column c) in a K-major swizzled [128 x 128] bf16 tile made of two 64-column chunks;
// c must be a multiple of 8 (16-byte unit).
__device__ __forceinline__ uint32_t sw_off(int r, int c) {
  return (uint32_t)((c >> 6) * TILE_BYTES + r * 128 + ((((c & 63) >> 3) ^ (r & 7)) << 4));
}

struct AttnArgs {
  int B, T, H, hd;
  float scale;
  bf16* out;          // fwd: atty ; bwd: dqkv
  float* lse;         // [B,H,T]
  const float* delta; // [B,H,T] (bwd)
  const float* cosT;  // optional fused RoPE-backward tables [T, hd/2]
  const float* sinT;
  bf16* dq_part;       // fused backward: dQ partial tiles [B][nq(nq+1)/2 (query tile i, key tile kt <= i)][128][C]
  int variant;         // forward tuning switch (see the kernel)
  long long* timeline; // optional: SM cycle stamps of CTA (0,0,0) of the fused backward, eight per (query block) step
  const int* sched;    // forward over tile pairs: per CTA the work items in order, -1 terminated; nullptr = round robin
  int sched_stride;    // entries per CTA in `sched`
  int dynamic;         // persistent kernels: draw the work items from the device counter instead
  int out_tma;         // forward over tile pairs: O leaves through a staging tile and TMA stores (needs T % 128 == 0)
};

// ================================================================== forward
// Warp-specialised: 16 softmax warps + 1 control warp (one thread of it issues every TMA load and tcgen05.mma).
// Softmax warp w reads TMEM lane group (w & 3) and score-column quarter (w >> 2): four threads share a query row, each
// owning 32 of the 128 score columns and HD/4 of the output columns.  Scores, P tiles and P.V results are all double
// buffered (TMEM: S0 S1 O0 O1), so the control warp runs two key blocks ahead and the softmax warps never wait for an
// MMA they have just enabled: the accumulation O += P_j V_j is folded in one iteration late.
constexpr int ATT_SOFTMAX_WARPS = 16;
constexpr int ATT_THREADS = (ATT_SOFTMAX_WARPS + 1) * 32;

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// packed fp32x2 arithmetic (two lanes per instruction on sm_100) and 3-input max
__device__ __forceinline__ uint64_t pk2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

template <int HD>
struct FwdSmem {
  static constexpr int CH = HD / 64;
  static constexpr int VBUF = (HD == 64) ? 2 : 1;
  static constexpr int QBUF = (HD == 64) ? 2 : 1;
  static constexpr int Q = 0;                                   // QBUF buffers
  static constexpr int K = Q + QBUF * CH * TILE_BYTES;          // 2 slots
  static constexpr int V = K + 2 * CH * TILE_BYTES;             // VBUF slots
  static constexpr int P = V + VBUF * CH * TILE_BYTES;          // 2 buffers x [128 x 128] bf16
  static constexpr int RED = P + 2 * 2 * TILE_BYTES;            // 3 x 4 x 128 floats: per-quarter row maxima (x2) / sums
  static constexpr int BAR = RED + 6144;
  static constexpr int TOTAL = BAR + 256 + 1024;
};

// Work item = one 128-query tile of one (sample, head).  Items are numbered heaviest first (most key blocks) and dealt
// round-robin to the persistent CTAs; both warp roles walk the same sequence.
struct FwdItem {
  int w, li, qt, b, h, nkb;
  bool valid;
  __device__ __forceinline__ void set(int w_, int li_, int total, int nq, int BH, int H) {
    w = w_; li = li_; valid = w_ < total;
    if (valid) {
      qt = nq - 1 - w_ / BH;
      const int bh = w_ % BH;
      b = bh / H; h = bh % H;
      nkb = qt + 1;
    } else {
      qt = b = h = 0; nkb = 1;
    }
  }
};
struct FwdCursor {   // position of one key block in the flattened (item, block) sequence of this CTA
  FwdItem it;
  int j;
  __device__ __forceinline__ void advance(int total, int nq, int BH, int H, int stride) {
    if (!it.valid) return;
    if (++j >= it.nkb) { it.set(it.w + stride, it.li + 1, total, nq, BH, H); j = 0; }
  }
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm, const AttnArgs a) {
  using S = FwdSmem<HD>;
  constexpr int CH = HD / 64, OC = HD / 4, VBUF = S::VBUF, QBUF = S::QBUF;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + S::BAR);
  uint64_t *bar_q = bars, *bar_k = bars + 2, *bar_v = bars + 4, *bar_s = bars + 6, *bar_p = bars + 8, *bar_o = bars + 10;
  uint32_t* tmem_slot = (uint32_t*)(bars + 12);
  volatile int* s_abort = (volatile int*)(bars + 13);   // set by the first wait that runs out; later waits are skipped
  float* s_red = (float*)(smem + S::RED);
  {   // an earlier CTA already gave up on a wait: do not queue more 4 s waits behind it (CTA-uniform decision)
    __shared__ int s_skip;
    if (threadIdx.x == 0) s_skip = *(volatile int*)&g_mlb_error;
    __syncthreads();
    if (s_skip != 0) return;
  }

  const int nq = (a.T + 127) / 128;
  const int BH = a.B * a.H, total = nq * BH, stride = gridDim.x;
  const int C = a.H * HD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < 2; i++) {
      tc::mbar_init(&bar_q[i], 1); tc::mbar_init(&bar_k[i], 1); tc::mbar_init(&bar_v[i], 1); tc::mbar_init(&bar_s[i], 1);
      tc::mbar_init(&bar_p[i], ATT_SOFTMAX_WARPS); tc::mbar_init(&bar_o[i], 1);
    }
    *s_abort = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tm);
  }
  if (warp == ATT_SOFTMAX_WARPS) tc::tmem_alloc(tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_o = tmem + 256;   // O buffers at +256 and +256+HD
  // Bounded, sticky wait: after the first expiry in this CTA every later wait returns at once, and all threads keep
  // executing the same sequence of arrivals / named barriers, so nobody is left waiting for a thread that gave up.
  auto wait = [&](uint64_t* bar, uint32_t phase, int where) -> bool {
    if (*s_abort) return false;
    if (!tc::mbar_wait(bar, phase, where)) { *s_abort = 1; return false; }
    return true;
  };

  if (warp == ATT_SOFTMAX_WARPS) {
    // ---------------------------------------------------------------- control warp
    // Everything is indexed by g, the running number of the key block in this CTA's flattened sequence:
    // K slot / score buffer / P buffer / O buffer = g & 1, V slot = g % VBUF, Q buffer = (local item number) % QBUF.
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = tc::idesc_bf16(128, HD, 0, 1);
      auto load_q = [&](const FwdItem& it) {
        const int qb = it.li % QBUF;
        tc::mbar_expect_tx(&bar_q[qb], CH * TILE_BYTES);
        for (int c = 0; c < CH; c++)
          tc::tma_load_2d(smem + S::Q + (qb * CH + c) * TILE_BYTES, &tm, &bar_q[qb], it.h * HD + c * 64, it.b * a.T + it.qt * 128);
      };
      auto load_k = [&](const FwdCursor& c, int g) {
        const int sl = g & 1;
        tc::mbar_expect_tx(&bar_k[sl], CH * TILE_BYTES);
        for (int x = 0; x < CH; x++)
          tc::tma_load_2d(smem + S::K + (sl * CH + x) * TILE_BYTES, &tm, &bar_k[sl], C + c.it.h * HD + x * 64, c.it.b * a.T + c.j * 128);
      };
      auto load_v = [&](const FwdCursor& c, int g) {
        const int sl = g % VBUF;
        tc::mbar_expect_tx(&bar_v[sl], CH * TILE_BYTES);
        for (int x = 0; x < CH; x++)
          tc::tma_load_2d(smem + S::V + (sl * CH + x) * TILE_BYTES, &tm, &bar_v[sl], 2 * C + c.it.h * HD + x * 64, c.it.b * a.T + c.j * 128);
      };
      auto issue_s = [&](const FwdCursor& c, int g) {   // S(g) = Q K^T into score buffer g & 1
        const uint32_t sQ = tc::smem_u32(smem + S::Q + (c.it.li % QBUF) * CH * TILE_BYTES);
        const uint32_t sK = tc::smem_u32(smem + S::K + (g & 1) * CH * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(tmem + (g & 1) * 128, desc_k(sQ, ks), desc_k(sK, ks), idesc_s, ks > 0);
      };
      FwdCursor c0, c1, c2;
      c0.it.set(blockIdx.x, 0, total, nq, BH, a.H); c0.j = 0;
      c1 = c0; c1.advance(total, nq, BH, a.H, stride);
      c2 = c1; c2.advance(total, nq, BH, a.H, stride);
      int pending_q_w = -1, pending_q_li = 0;   // Q tile to prefetch as soon as its buffer's previous S MMAs are known complete
      // ---- prologue: first two key blocks
      load_q(c0.it);
      load_k(c0, 0);
      load_v(c0, 0);
      if (c1.it.valid) {
        load_k(c1, 1);
        if (VBUF == 2) load_v(c1, 1);
        if (c1.it.li != c0.it.li && QBUF == 2) load_q(c1.it);
      }
      if (wait(&bar_q[0], 0, 10) && wait(&bar_k[0], 0, 11)) { tc::tc_fence_after(); issue_s(c0, 0); }
      tc::mma_commit(&bar_s[0]);
      if (c1.it.valid) {
        bool okq = true;
        if (c1.it.li != c0.it.li) {
          if (QBUF == 1) {   // single Q buffer: S(0) must be done before the next item's Q may land
            okq = wait(&bar_s[0], 0, 12);
            if (okq) load_q(c1.it);
          }
          okq = okq && wait(&bar_q[c1.it.li % QBUF], (c1.it.li / QBUF) & 1, 10);
        }
        if (okq && wait(&bar_k[1], 0, 11)) { tc::tc_fence_after(); issue_s(c1, 1); }
        tc::mma_commit(&bar_s[1]);
      }
      int q_loaded_li = c1.it.valid ? c1.it.li : c0.it.li;   // highest local item whose Q load has been issued
      if (QBUF == 2) {   // the item after the last loaded one can be prefetched once its buffer is free
        FwdItem nx;
        nx.set(blockIdx.x + (q_loaded_li + 1) * stride, q_loaded_li + 1, total, nq, BH, a.H);
        if (nx.valid) { pending_q_w = nx.w; pending_q_li = nx.li; }
      }
      for (int g = 0; c0.it.valid; g++) {
        const int sl = g & 1, ph = (g >> 1) & 1;
        // (a) S(g) is complete (so is every earlier S): K slot g&1 can take the key block two ahead, and a pending Q
        //     prefetch whose buffer was last read by an item that ended at or before g can go out
        const bool s_done = wait(&bar_s[sl], ph, 12);
        if (s_done && c2.it.valid) load_k(c2, g + 2);
        if (s_done && QBUF == 2 && pending_q_w >= 0 && pending_q_li - 2 < c0.it.li + (c0.j == c0.it.nkb - 1 ? 1 : 0)) {
          // buffer (pending_q_li & 1) was used by local item pending_q_li - 2, all of whose blocks are <= g here
          FwdItem nx;
          nx.set(pending_q_w, pending_q_li, total, nq, BH, a.H);
          load_q(nx);
          q_loaded_li = pending_q_li;
          pending_q_w = -1;
        }
        // (b) P(g) written (and S(g) fully read) -> O_blk(g) = P V
        if (wait(&bar_p[sl], ph, 13) && wait(&bar_v[g % VBUF], (g / VBUF) & 1, 14)) {
          tc::tc_fence_after();
          const uint32_t sP = tc::smem_u32(smem + S::P + sl * 2 * TILE_BYTES);
          const uint32_t sV = tc::smem_u32(smem + S::V + (g % VBUF) * CH * TILE_BYTES);
#pragma unroll
          for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ss(t_o + sl * HD, desc_k(sP, ks), desc_mn(sV, ks), idesc_o, ks > 0);
        }
        tc::mma_commit(&bar_o[sl]);
        // (c) score buffer g&1 is free: S(g+2), possibly the first block of a later item
        if (c2.it.valid) {
          bool okq = true;
          if (c2.j == 0) {
            if (c2.it.li > q_loaded_li) {
              // not prefetched (single Q buffer, or the prefetch condition never became true): the buffer's previous user
              // ends at block g+1, whose S was issued in the previous iteration
              okq = wait(&bar_s[(g + 1) & 1], ((g + 1) >> 1) & 1, 12);
              if (okq) { load_q(c2.it); q_loaded_li = c2.it.li; if (pending_q_li == c2.it.li) pending_q_w = -1; }
            }
            okq = okq && wait(&bar_q[c2.it.li % QBUF], (c2.it.li / QBUF) & 1, 10);
            if (QBUF == 2 && pending_q_w < 0) {
              FwdItem nx;
              nx.set(c2.it.w + stride, c2.it.li + 1, total, nq, BH, a.H);
              if (nx.valid && nx.li > q_loaded_li) { pending_q_w = nx.w; pending_q_li = nx.li; }
            }
          }
          if (okq && wait(&bar_k[sl], ((g + 2) >> 1) & 1, 15)) { tc::tc_fence_after(); issue_s(c2, g + 2); }
          tc::mma_commit(&bar_s[sl]);
        }
        // (d) V slot free once P V of block g has completed
        const FwdCursor& cv = (VBUF == 2) ? c2 : c1;
        if (cv.it.valid && wait(&bar_o[sl], ph, 16)) load_v(cv, g + VBUF);
        c0 = c1; c1 = c2; c2.advance(total, nq, BH, a.H, stride);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int lg = warp & 3, cq = warp >> 2, row = lg * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    const uint64_t sl2x2 = pk2(sl2, sl2);
    int g = 0;
    uint32_t r[32];
    bool have_scores = false;
    FwdItem it;
    it.set(blockIdx.x, 0, total, nq, BH, a.H);
    for (; it.valid; it.set(it.w + stride, it.li + 1, total, nq, BH, a.H)) {
      const int qrow = it.qt * 128 + row;
      float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
      float o[OC];
#pragma unroll
      for (int i = 0; i < OC; i++) o[i] = 0.f;
      auto fold = [&](int gb, float alpha) {   // O = O * alpha + (P V) of block gb
        if (OC == 16) {
          uint32_t ro[16];
          tc::tmem_ld16(t_o + (gb & 1) * HD + lane_addr + cq * 16, ro);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; i++) o[i] = o[i] * alpha + __uint_as_float(ro[i]);
        } else {
          uint32_t ro[32];
          tc::tmem_ld32(t_o + (gb & 1) * HD + lane_addr + cq * 32, ro);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) o[i % OC] = o[i % OC] * alpha + __uint_as_float(ro[i]);
        }
        tc::tc_fence_before();
      };
      for (int j = 0; j < it.nkb; j++, g++) {
        const int sl = g & 1;
        const int kc0 = j * 128 + cq * 32;
        if (!have_scores) {   // first block of this CTA: nothing was prefetched
          wait(&bar_s[sl], (g >> 1) & 1, 17);
          tc::tc_fence_after();
          tc::tmem_ld32(tmem + sl * 128 + lane_addr + cq * 32, r);
          tc::tmem_ld_wait();
          have_scores = true;
        }
        float mx = -INFINITY;
        if (j == it.qt) {
#pragma unroll
          for (int i = 0; i < 32; i++)
            if (kc0 + i > qrow) r[i] = 0xff800000u;   // -inf: masked by causality
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        float* red = s_red + sl * 512;
        red[cq * 128 + row] = mx;
        named_bar_sync(1 + lg, 128);
        mx = fmaxf(fmaxf(red[row], red[128 + row]), fmaxf(red[256 + row], red[384 + row]));
        const float m_new = fmaxf(m, mx * sl2);   // finite: key 0 is visible to every query
        const float alpha = exp2f(m - m_new);     // exp2(-inf) = 0 on the first block
        const uint64_t nm2 = pk2(-m_new, -m_new);
        uint64_t rs2 = pk2(0.f, 0.f);
        uint8_t* pbuf = smem + S::P + sl * 2 * TILE_BYTES;
#pragma unroll
        for (int v8 = 0; v8 < 4; v8++) {
          uint32_t pw[4];
#pragma unroll
          for (int x = 0; x < 4; x++) {
            const int e = v8 * 8 + 2 * x;
            float z0, z1;
            upk2(fma2(pk2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), sl2x2, nm2), z0, z1);
            const float p0 = exp2f(z0), p1 = exp2f(z1);
            rs2 = add2(rs2, pk2(p0, p1));
            pw[x] = pack_bf16(p0, p1);
          }
          *reinterpret_cast<uint4*>(pbuf + sw_off(row, cq * 32 + v8 * 8)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        }
        tc::fence_async_smem();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&bar_p[sl]);
        float rs_lo, rs_hi;
        upk2(rs2, rs_lo, rs_hi);
        l = l * alpha + (rs_lo + rs_hi);
        m = m_new;
        // the score registers are free again: start fetching the next block's scores (this item's or the next item's)
        // so that the TMEM latency hides behind the fold below
        const bool more = (j + 1 < it.nkb) || (it.w + stride < total);
        if (more) {
          wait(&bar_s[(g + 1) & 1], ((g + 1) >> 1) & 1, 17);
          tc::tc_fence_after();
          tc::tmem_ld32(tmem + ((g + 1) & 1) * 128 + lane_addr + cq * 32, r);
        } else {
          have_scores = false;
        }
        if (j > 0) {   // fold in the previous block, whose P V product had a whole softmax to complete
          wait(&bar_o[(g - 1) & 1], ((g - 1) >> 1) & 1, 18);
          tc::tc_fence_after();
          fold(g - 1, alpha_prev);     // its tcgen05.wait::ld also covers the score prefetch
        } else if (more) {
          tc::tmem_ld_wait();
        }
        alpha_prev = alpha;
      }
      wait(&bar_o[(g - 1) & 1], ((g - 1) >> 1) & 1, 19);
      tc::tc_fence_after();
      fold(g - 1, alpha_prev);
      // combine the four partial row sums (third exchange buffer: the max buffers may already be in use by a fast warp
      // of the next item), normalise, store
      float* red = s_red + 1024;
      named_bar_sync(1 + lg, 128);   // everyone in the row group has finished reading the previous item's sums
      red[cq * 128 + row] = l;
      named_bar_sync(1 + lg, 128);
      const float L = red[row] + red[128 + row] + red[256 + row] + red[384 + row];
      if (!*s_abort && qrow < a.T) {
        const float inv = 1.f / L;
        bf16* dst = a.out + ((size_t)(it.b * a.T + qrow)) * C + it.h * HD + cq * OC;
#pragma unroll
        for (int v8 = 0; v8 < OC / 8; v8++) {
          uint4 pk;
          pk.x = pack_bf16(o[v8 * 8 + 0] * inv, o[v8 * 8 + 1] * inv); pk.y = pack_bf16(o[v8 * 8 + 2] * inv, o[v8 * 8 + 3] * inv);
          pk.z = pack_bf16(o[v8 * 8 + 4] * inv, o[v8 * 8 + 5] * inv); pk.w = pack_bf16(o[v8 * 8 + 6] * inv, o[v8 * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(dst + v8 * 8) = pk;
        }
        if (cq == 0) a.lse[((size_t)it.b * a.H + it.h) * a.T + qrow] = (m + log2f(L)) * LN2;
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == ATT_SOFTMAX_WARPS) tc::tmem_dealloc(tmem, TMEM_COLS);
}

// ================================================================== forward, head size 64: one thread per query row
// A persistent CTA works on PAIRS of 128-query tiles of one (sample, head): tile 0 is owned by warps 0-3, tile 1 by
// warps 4-7 (thread = one query row: no cross-thread reductions, no shared-memory exchange), warp 8 issues tile 0's
// MMAs, warp 10 tile 1's, warp 9 every TMA load.  Per key block j and tile t:   S_t = Q_t K_j^T (TMEM) -> p = exp2(s*c - m) in 32-column chunks
// straight out of TMEM -> P_t written as packed bf16 into its own TMEM columns (the A operand of the next MMA never
// touches shared memory, and the next block's scores can be issued before P_t V_j) -> O_t += P_t V_j.
// Where O lives and what m is depends on the variant (template MODE):
//   1  O_blk = P V is folded into 64 fp32 registers per row after every block with the usual running-max rescale;
//   2  O accumulates in TMEM over the item's blocks; m is the maximum of an EARLIER block as long as no row of the warp
//      has grown past it by more than 2^8 (then p <= 256, harmless in bf16 / fp32), and only when one has are O (in
//      place, TMEM load / multiply / store) and l rescaled - rare after the first blocks;
//   3  as 2, but the row maximum is tracked inside the exponential pass and a block is redone the exact way when the
//      threshold is passed (the default: one TMEM read of the scores per block instead of two).
// The two tiles share K_j / V_j (one load per 256 queries) and run out of phase: while one tile's threads compute
// exponentials the tensor core works for the other tile.  Both tiles walk the same key blocks; the block past tile
// 0's diagonal is fully masked for it (its threads compute nothing; modes 2 and 3 skip its P V).
// A CTA's items come from a balanced schedule built on the host (attn_schedule), the finished O rows leave through a
// swizzled staging tile and one TMA store per warp.
// mbarriers per tile: bar_s S complete (commit) | bar_sc S read out of TMEM (4 warps; in mode 3 half way through the
// block, so that the next block's Q K^T is issued under the rest of the exponentials) | bar_p P stored (4 warps) |
// bar_o P V complete (commit) | bar_of O_blk folded (4 warps, mode 1 only).  K has 3 slots, V 4, Q 2 buffers: each is a
// ring with a "full" barrier (TMA bytes) and a "released" barrier on which the 8 softmax warps arrive when they have
// seen the MMAs that read the slot complete (Q K^T for K and Q, P V for V).
// What the cycle stamps showed about the issuing threads: every tcgen05.mma and every tcgen05.commit costs its thread
// ~75 cycles whatever the product's size, so 12 MMAs and 2 commits per key block and tile are ~1000 cycles of one
// thread; with a single thread for both tiles that chain (3200 cycles per key block, never waiting) was the kernel's
// pace.
// The one-pass variant writes P as the upper halves of the fp32 exponentials (one byte-permute per pair instead of a
// rounding conversion; equal speed when measured, kept for its single instruction).  Cutting off 16 mantissa bits loses
// 2^-8 / mantissa of the value, 0.28 % on average over mantissas; the exponentials are therefore taken of
// z + log2(1.0028), which centres the error of P, and the row sum (of the same, unrounded values) is divided by 1.0028
// once per row.  Error of O against an fp32 reference: 2.1e-3 relative Frobenius (a bf16 rounding of the reference
// itself: 1.6e-3), mean signed error below 1e-5.
constexpr float P_BIAS_LOG2 = 0.0040339f;     // log2(1.0028)
constexpr float P_BIAS_INV = 0.99720782f;     // 1 / 1.0028
__device__ __forceinline__ uint32_t pack_hi16(float lo, float hi) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
  return r;
}
// ------------------------------------------------------------------ work items from a device counter
// Alternative to the host-built table: the CTAs of a launch draw item numbers 0, 1, 2, ... (heaviest first) from a
// counter in device memory.  One thread per CTA (the loader) draws - always ahead of where the CTA is working, since it
// needs the next items for its prefetches - and publishes what it drew in a shared-memory ring (value, then sequence
// number); every other role of the CTA reads its li-th item from the ring and waits, bounded, if it is not there yet.
// A CTA that finds the counter exhausted publishes -1 from then on.  The last CTA to leave resets the counters, so
// there is nothing to zero between launches (or graph replays); one launch per kernel kind may be in flight on a device.
// A shape met for the first time needs no table then (none can be built during graph capture).  Off by default: a CTA
// has to claim its next item while it still works on the current one (the prefetches need it), which costs the balance
// more than the table's fixed assignment does - 4 us per forward and 10 us per backward call alone, 0.3 ms per step
// next to the gradient kernels that run behind backward on 4 GPUs.
__device__ int g_attn_ctr[4];      // [2 * kind]: next item, [2 * kind + 1]: CTAs that have left
struct ItemRing {
  volatile int* val;   // [64]
  volatile int* seq;   // [64]: li + 1 once item li has been published; seq[64]: index of the first -1 item (INT_MAX until known)
  int published;       // publisher only
  __device__ __forceinline__ int draw(int li, int kind, int total) {          // publisher thread
    while (published <= li) {
      if (published >= seq[64]) { published = li + 1; break; }              // exhausted: nothing more to draw or publish
      int w = atomicAdd(&g_attn_ctr[2 * kind], 1);
      if (w >= total) { seq[64] = published; __threadfence_block(); published = li + 1; break; }
      val[published & 63] = w;
      __threadfence_block();
      seq[published & 63] = published + 1;
      published++;
    }
    return li >= seq[64] ? -1 : val[li & 63];
  }
  __device__ __forceinline__ int read(int li, volatile int* abort_flag) const {     // everyone else
    for (long spin = 0; spin < (1L << 26); spin++) {
      if (seq[li & 63] == li + 1) return val[li & 63];
      if (li >= seq[64]) return -1;
      if (*abort_flag) return -1;
    }
    mlb_set_error(MLB_ERR_MBAR_TIMEOUT, 0x7f);
    *abort_flag = 1;
    return -1;
  }
};
__device__ __forceinline__ void attn_ctr_leave(int kind) {        // one thread per CTA, after the CTA's last draw
  __threadfence();
  if (atomicAdd(&g_attn_ctr[2 * kind + 1], 1) == (int)gridDim.x - 1) {
    g_attn_ctr[2 * kind] = 0;
    g_attn_ctr[2 * kind + 1] = 0;
    __threadfence();
  }
}
struct Fwd2Smem {
  static constexpr int Q = 0;                          // 2 buffers x 2 tiles
  static constexpr int KN = 3;                         // K slots; V has one more
  static constexpr int K = Q + 4 * TILE_BYTES;
  static constexpr int V = K + KN * TILE_BYTES;
  static constexpr int OST = V + (KN + 1) * TILE_BYTES;   // O staging: 8 warps x [32 rows x 128 B] bf16, swizzled
  static constexpr int BAR = OST + 2 * TILE_BYTES;
  static constexpr int SCHED = BAR + 256;                 // this CTA's first 64 work items
  static constexpr int TOTAL = SCHED + 768 + 1024;             // SCHED: 64 items, or a ring of 64 (value, sequence number) + end marker
};
constexpr int FWD2_THREADS = 11 * 32;   // 8 softmax warps, MMA warp of tile 0, loader warp, MMA warp of tile 1

struct Fwd2Step {   // one key block of one item in this CTA's flattened sequence
  int w, li, p, b, h, nkb, j;
  bool valid;
  __device__ __forceinline__ void set_item(int w_, int li_, int total, int npair, int nq, int BH, int H) {
    w = w_; li = li_; valid = w_ >= 0 && w_ < total; j = 0;
    if (valid) {
      p = npair - 1 - w_ / BH;                 // heaviest pairs first
      const int bh = w_ % BH;
      b = bh / H; h = bh % H;
      nkb = min(2 * p + 2, nq);
    } else {
      p = b = h = 0; nkb = 1;
    }
  }
  template <class F>   // item_at(li): this CTA's li-th work item or -1
  __device__ __forceinline__ void advance(F&& item_at, int total, int npair, int nq, int BH, int H) {
    if (!valid) return;
    if (++j >= nkb) set_item(item_at(li + 1), li + 1, total, npair, nq, BH, H);
  }
};

// MODE 1: O folded into registers every block | 2: O in TMEM, lazy rescale, two passes | 3: the same in one pass.
// (Measured without gain on top of mode 3 and taken out again: 4, 6 or 8 of every 16 exponential pairs as a cubic on the
// FMA pipe instead of the special-function unit - equal, 3 % and 5 % slower although the pure exponential chunks got
// shorter; fp16 exponentials two at a time; tile 1 started half a block behind tile 0; the MMA and loader threads
// sleeping between barrier probes.)
template <int MODE, bool DYN = false>
__global__ void __maxnreg__(160) attn_fwd_rows_tc_kernel(const __grid_constant__ CUtensorMap tm, const __grid_constant__ CUtensorMap tm_out,
                                                                           const AttnArgs a) {
  mlb_pdl_sync();
  using S = Fwd2Smem;
  constexpr bool LAZY = MODE >= 2;
  constexpr int HD = 64;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + S::BAR);
  constexpr int KN = S::KN, VN = S::KN + 1;
  uint64_t *bar_q = bars /*[2]*/, *bar_s = bars + 2 /*[2]*/, *bar_p = bars + 4 /*[2]*/, *bar_o = bars + 6 /*[2]*/, *bar_of = bars + 8 /*[2]*/,
           *bar_k = bars + 10 /*[KN]*/, *bar_v = bars + 10 + KN /*[VN]*/;
  // slot released: both tiles' MMAs that read it have completed (one arrival per softmax warp, which saw them complete)
  uint64_t *bar_kf = bars + 10 + KN + VN /*[KN]*/, *bar_vf = bar_kf + KN /*[VN]*/, *bar_qf = bar_vf + VN /*[2]*/;
  uint64_t* bar_sc = bar_qf + 2 /*[2]*/;     // S_t read out by its four softmax warps
  uint32_t* tmem_slot = (uint32_t*)(bar_sc + 2);
  volatile int* s_abort = (volatile int*)(bar_sc + 3);
  static_assert((10 + 2 * (KN + VN) + 2 + 2 + 2) * 8 <= 256, "barrier area");
  {
    __shared__ int s_skip;
    if (threadIdx.x == 0) s_skip = *(volatile int*)&g_mlb_error;
    __syncthreads();
    if (s_skip != 0) return;
  }
  const int nq = (a.T + 127) / 128, npair = (nq + 1) / 2;
  const int BH = a.B * a.H, total = npair * BH, stride = gridDim.x;
  const int C = a.H * HD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // This CTA's sequence of work items (item w = pair p of (sample, head) bh, heaviest pairs first): from the host's
  // balanced schedule if there is one, else round robin over the grid.  The rows of the schedule end with -1 entries.
  const int* srow = a.sched ? a.sched + (size_t)blockIdx.x * a.sched_stride : nullptr;
  int* s_sched = (int*)(smem + S::SCHED);     // the row's first 64 entries: a global load at an item boundary stalls
  if (srow && tid < 64) s_sched[tid] = tid < a.sched_stride ? __ldg(srow + tid) : -1;   // its warp for a DRAM latency
  constexpr bool dyn = DYN;
  ItemRing ring{(volatile int*)s_sched, (volatile int*)s_sched + 64, 0};
  if (dyn && tid <= 64) s_sched[64 + tid] = tid < 64 ? 0 : 0x7fffffff;
  const bool publisher = warp == 9 && lane == 0;
  auto item_at = [&](int li) -> int {
    if (dyn) return publisher ? ring.draw(li, 0, total) : ring.read(li, s_abort);
    if (srow) return li < 64 ? s_sched[li] : __ldg(srow + li);
    const int x = blockIdx.x + li * stride;
    return x < total ? x : -1;
  };

  if (tid == 0) {
    for (int i = 0; i < 2; i++) {
      tc::mbar_init(&bar_q[i], 1); tc::mbar_init(&bar_s[i], 1); tc::mbar_init(&bar_o[i], 1);
      tc::mbar_init(&bar_p[i], 4); tc::mbar_init(&bar_of[i], 4);
    }
    for (int i = 0; i < KN; i++) { tc::mbar_init(&bar_k[i], 1); tc::mbar_init(&bar_kf[i], 8); }
    for (int i = 0; i < VN; i++) { tc::mbar_init(&bar_v[i], 1); tc::mbar_init(&bar_vf[i], 8); }
    for (int i = 0; i < 2; i++) { tc::mbar_init(&bar_qf[i], 8); tc::mbar_init(&bar_sc[i], 4); }
    *s_abort = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tm);
    tc::tma_prefetch_desc(&tm_out);
  }
  if (warp == 8) tc::tmem_alloc(tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;     // S0 @0, S1 @128, P0 @256, P1 @320 (bf16 pairs), O0 @384, O1 @448
  auto wait = [&](uint64_t* bar, uint32_t phase, int where) -> bool {
    if (tc::mbar_try(bar, phase)) return true;      // the common case costs one probe
    if (*s_abort) return false;
    if (!tc::mbar_wait(bar, phase, where)) { *s_abort = 1; return false; }
    return true;
  };

  if (warp == 9) {
    // ---------------------------------------------------------------- loader warp: every TMA load (and the index arithmetic)
    if (lane == 0) {
      auto load_q = [&](const Fwd2Step& s) {
        const int qb = s.li & 1;
        tc::mbar_expect_tx(&bar_q[qb], 2 * TILE_BYTES);
        for (int t = 0; t < 2; t++)
          tc::tma_load_2d(smem + S::Q + (qb * 2 + t) * TILE_BYTES, &tm, &bar_q[qb], s.h * HD, s.b * a.T + (2 * s.p + t) * 128);
      };
      // Block n goes into K slot n % KN and V slot n % VN once the previous tenant's readers are done.  Every slot is a
      // ring of its own (full barrier / released barrier), so no wait here can be overtaken by two phases however far
      // one tile runs ahead of the other.
      auto load_kv = [&](const Fwd2Step& s, int n) {
        if (n >= KN) wait(&bar_kf[n % KN], (n / KN + 1) & 1, 70);
        tc::mbar_expect_tx(&bar_k[n % KN], TILE_BYTES);
        tc::tma_load_2d(smem + S::K + (n % KN) * TILE_BYTES, &tm, &bar_k[n % KN], C + s.h * HD, s.b * a.T + s.j * 128);
        if (n >= VN) wait(&bar_vf[n % VN], (n / VN + 1) & 1, 71);
        tc::mbar_expect_tx(&bar_v[n % VN], TILE_BYTES);
        tc::tma_load_2d(smem + S::V + (n % VN) * TILE_BYTES, &tm, &bar_v[n % VN], 2 * C + s.h * HD, s.b * a.T + s.j * 128);
      };
      Fwd2Step c0, c3;      // steps g and g + KN
      c0.set_item(item_at(0), 0, total, npair, nq, BH, a.H);
      c3 = c0;
      if (c0.valid) {
        load_q(c0);
        Fwd2Step nx;
        nx.set_item(item_at(1), 1, total, npair, nq, BH, a.H);
        if (nx.valid) load_q(nx);          // the second item's Q goes into the other buffer right away
        for (int i = 0; i < KN; i++) {
          if (c3.valid) load_kv(c3, i);
          c3.advance(item_at, total, npair, nq, BH, a.H);
        }
      }
      for (int g = 0; c0.valid; g++) {
        if (c3.valid) load_kv(c3, g + KN);
        if (c0.j == c0.nkb - 1) {
          // once this item's MMAs are done its Q buffer takes the item after next
          Fwd2Step nx;
          nx.set_item(item_at(c0.li + 2), c0.li + 2, total, npair, nq, BH, a.H);
          if (nx.valid) {
            wait(&bar_qf[c0.li & 1], (c0.li >> 1) & 1, 72);
            load_q(nx);
          }
        }
        c0.advance(item_at, total, npair, nq, BH, a.H);
        c3.advance(item_at, total, npair, nq, BH, a.H);
      }
    }
  } else if (warp == 8 || warp == 10) {
    // ---------------------------------------------------------------- MMA warps: one issuing thread per tile (warp 8: tile
    // 0, warp 10: tile 1).  A single thread for both tiles was the kernel's pace: its serial chain of waits, descriptor
    // arithmetic and issues took ~3200 cycles per key block, all of it busy.  Slot and phase counters are kept
    // incrementally (no division on this thread).
    if (lane == 0) {
      const int t = warp == 8 ? 0 : 1;
      constexpr uint32_t idesc_s = tc::idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_o = tc::idesc_bf16(128, HD, 0, 1);     // A = P (TMEM, K-major), B = V (MN-major)
      constexpr uint64_t TILE_D = TILE_BYTES >> 4;     // one tile further, in descriptor address units
      const uint64_t dq0 = desc_base_k(tc::smem_u32(smem + S::Q)) + (uint64_t)t * TILE_D, dk0 = desc_base_k(tc::smem_u32(smem + S::K));
      const uint64_t dv0 = desc_base_mn(tc::smem_u32(smem + S::V));
      const uint32_t d_s = tmem + t * 128, d_p = tmem + 256 + t * 64, d_o = tmem + 384 + t * HD;
      int li = 0, j = 0, w = item_at(0), w_next = item_at(1);   // the next item's index is fetched an item ahead
      auto item_nkb = [&](int w_) { return min(2 * (npair - 1 - w_ / BH) + 2, nq); };
      bool valid = w >= 0;
      int nkb = valid ? item_nkb(w) : 0;
      int qt_t = valid ? 2 * (npair - 1 - w / BH) + t : 0;      // this tile's diagonal block in the current item
      if (valid) {
        const bool ok0 = wait(&bar_q[0], 0, 60) && wait(&bar_k[0], 0, 61);
        if (ok0) {
          tc::tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < 4; ks++) tc::mma_bf16_ss(d_s, dq0 + ks * 2, dk0 + ks * 2, idesc_s, ks > 0);
        }
        tc::mma_commit(&bar_s[t]);
      }
      int k1 = 1 % KN, k1p = 0;     // slot and phase parity of key block g + 1
      int vs = 0, vp = 0;           // of value block g
      for (int g = 0; valid; g++) {
        // next step: same item, or the first block of this CTA's next item
        int nli = li, nj = j + 1, nw = w;
        if (nj >= nkb) { nli = li + 1; nj = 0; nw = w_next; }
        const bool has_next = nw >= 0;
        bool next_ok = has_next;
        if (has_next) {
          next_ok = wait(&bar_k[k1], k1p, 62);
          if (next_ok && nj == 0) next_ok = wait(&bar_q[nli & 1], (nli >> 1) & 1, 63);
        }
        const uint64_t dqn = dq0 + (uint64_t)((nli & 1) * 2) * TILE_D, dkn = dk0 + (uint64_t)k1 * TILE_D;
        const uint64_t dvg = dv0 + (uint64_t)vs * TILE_D;
        if (has_next) {                              // the next scores as soon as S_t(g) has been read out
          const bool sc_ok = wait(&bar_sc[t], g & 1, 73);
          if (sc_ok && next_ok) {
            tc::tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ks++) tc::mma_bf16_ss(d_s, dqn + ks * 2, dkn + ks * 2, idesc_s, ks > 0);
          }
          tc::mma_commit(&bar_s[t]);
        }
        const bool v_ok = wait(&bar_v[vs], vp, 64);
        bool go = wait(&bar_p[t], g & 1, 65);        // P_t(g) is in TMEM
        if constexpr (!LAZY) {
          if (go && g > 0) go = wait(&bar_of[t], (g - 1) & 1, 66);   // O_blk_t(g-1) has been folded
        }
        // LAZY: a block past the tile's diagonal (tile 0's last one) adds nothing to the accumulated O and is not multiplied
        if (go && v_ok && !(LAZY && j > qt_t)) {
          tc::tc_fence_after();
          // LAZY: O accumulates in TMEM over the item's key blocks (the softmax warps rescale it in place when needed)
          const bool acc0 = LAZY && j > 0;
#pragma unroll
          for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ts(d_o, d_p + ks * 8, dvg + ks * 128, idesc_o, ks > 0 || acc0);
        }
        tc::mma_commit(&bar_o[t]);
        if (nj == 0 && has_next) { nkb = item_nkb(nw); qt_t = 2 * (npair - 1 - nw / BH) + t; w_next = item_at(nli + 1); }
        li = nli; j = nj; w = nw; valid = has_next;
        if (++k1 == KN) { k1 = 0; k1p ^= 1; }
        if (++vs == VN) { vs = 0; vp ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: tile t = warp >> 2
    const int t = warp >> 2, lg = warp & 3, row = lg * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
    const uint32_t t_s = tmem + t * 128 + lane_addr, t_p = tmem + 256 + t * 64 + lane_addr, t_o = tmem + 384 + t * HD + lane_addr;
    const float sl2 = a.scale * LOG2E;
    const uint64_t sl2x2 = pk2(sl2, sl2);
    int g = 0;
    // first 16 blocks of CTA 0: thread 0 (tile 0) and thread 128 (tile 1), 8 stamps per block, tile 1 behind tile 0's 128
    long long* tl = (a.timeline && blockIdx.x == 0 && (tid & 127) == 0) ? a.timeline + (tid >> 7) * 128 : nullptr;
    Fwd2Step it;
    it.set_item(item_at(0), 0, total, npair, nq, BH, a.H);
    for (; it.valid; it.set_item(item_at(it.li + 1), it.li + 1, total, npair, nq, BH, a.H)) {
      const int qt = 2 * it.p + t, qrow = qt * 128 + row;
      float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
      float o[LAZY ? 1 : HD];
#pragma unroll
      for (int i = 0; i < (LAZY ? 1 : HD); i++) o[i] = 0.f;
      auto fold = [&](float alpha) {   // O = O * alpha + (P V) of the previous block
        if constexpr (!LAZY) {
          uint32_t r0[32], r1[32];
          tc::tmem_ld32(t_o, r0);
          tc::tmem_ld32(t_o + 32, r1);
          tc::tmem_ld_wait();
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_of[t]);
#pragma unroll
          for (int i = 0; i < 32; i++) {
            o[i] = o[i] * alpha + __uint_as_float(r0[i]);
            o[32 + i] = o[32 + i] * alpha + __uint_as_float(r1[i]);
          }
        }
      };
      auto rescale = [&](float alpha) {   // LAZY: O (TMEM, sum over the blocks so far) *= alpha, in place
#pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t r[32], w0[16], w1[16];
          tc::tmem_ld32(t_o + c * 32, r);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; i++) {
            w0[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            w1[i] = __float_as_uint(__uint_as_float(r[16 + i]) * alpha);
          }
          tc::tmem_st16(t_o + c * 32, w0);
          tc::tmem_st16(t_o + c * 32 + 16, w1);
        }
      };
      // The slots' release barriers are arrived on from here (one lane per warp, 8 warps) rather than by tcgen05.commit:
      // every tcgen05 instruction costs its issuing thread ~75 cycles, and that thread's chain sets the block time.
      auto s_seen = [&](int j) {          // Q K^T of block g has completed: its K slot, and after an item's last block Q
        if (lane == 0) {
          tc::mbar_arrive(&bar_kf[g % KN]);
          if (j == it.nkb - 1) tc::mbar_arrive(&bar_qf[it.li & 1]);
        }
      };
      for (int j = 0; j < it.nkb; j++, g++) {
        if constexpr (MODE == 3) {
          // One pass per key block: exponentials against the reference maximum of an earlier block while the row
          // maximum of this block is tracked next to them; only if some row of the warp has grown past the reference by
          // more than 2^8 is the block redone the exact way (row maximum first, O and l rescaled, exponentials again).
          // The first block of an item always takes the exact way.  j, qt and the votes are uniform over the warp.
          if (tl && g < 16) tl[g * 8 + 0] = clock64();
          wait(&bar_s[t], g & 1, 67);
          tc::tc_fence_after();
          s_seen(j);
          if (tl && g < 16) tl[g * 8 + 1] = clock64();
          const bool diag = (j == qt);
          const int kc0 = j * 128;
          bool p_free = (j == 0);        // P's columns are free once the previous block's P V has completed
          auto free_p = [&]() {
            if (!p_free) {
              wait(&bar_o[t], (g - 1) & 1, 68);
              tc::tc_fence_after();
              if (lane == 0) tc::mbar_arrive(&bar_vf[(g - 1) % VN]);     // P V of block g-1 is done with its V slot
              p_free = true;
            }
          };
          auto release_s = [&]() {       // this warp's rows of S(g) have been read out of TMEM (or are not needed)
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&bar_sc[t]);
          };
          if (j > qt) {                  // past the diagonal: every key of this block is masked for every row of the tile;
            release_s();                 // the MMA thread skips its P V
            free_p();
          } else {
            bool exact = (j == 0);
            auto mask = [&](int c, uint32_t (&r)[32]) {
              if (diag) {
#pragma unroll
                for (int i = 0; i < 32; i++)
                  if (kc0 + c * 32 + i > qrow) r[i] = 0xff800000u;     // exp2(-inf) = 0
              }
            };
            for (int attempt = 0; attempt < 2; attempt++) {
              if (exact) {
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                  uint32_t r[32];
                  tc::tmem_ld32(t_s + c * 32, r);
                  tc::tmem_ld_wait();
                  mask(c, r);
#pragma unroll
                  for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                }
                const float m_new = fmaxf(m, mx * sl2);   // finite: key 0 is visible to every query
                if (j > 0) {
                  const float alpha = ex2_approx(m - m_new);
                  l *= alpha;
                  free_p();
                  rescale(alpha);
                }
                m = m_new;
              }
              const uint64_t nm2 = pk2(P_BIAS_LOG2 - m, P_BIAS_LOG2 - m);
              uint64_t rs2 = pk2(0.f, 0.f);
              float mx = -INFINITY;
              // exponentials of one 32-column chunk held in registers; track: the row maximum is followed next to them
              auto exps = [&](uint32_t (&r)[32], uint32_t (&pw)[16], auto track) {
#pragma unroll
                for (int x = 0; x < 16; x++) {
                  float z0, z1;
                  if constexpr (decltype(track)::value) mx = max3(mx, __uint_as_float(r[2 * x]), __uint_as_float(r[2 * x + 1]));
                  upk2(fma2(pk2(__uint_as_float(r[2 * x]), __uint_as_float(r[2 * x + 1])), sl2x2, nm2), z0, z1);
                  const float p0 = ex2_approx(z0), p1 = ex2_approx(z1);
                  rs2 = add2(rs2, pk2(p0, p1));
                  pw[x] = pack_hi16(p0, p1);
                }
              };
              // The scores leave TMEM ahead of the arithmetic: chunks 2 and 3 are in registers when chunks 0 and 1 are
              // done, and S is handed back to the MMA thread there - the next block's Q K^T runs under the second half
              // of this block's exponentials instead of after them.
              uint32_t ra[32], rb[32], pw0[16], pw1[16];
              tc::tmem_ld32(t_s, ra);
              tc::tmem_ld_wait();
              mask(0, ra);
              tc::tmem_ld32(t_s + 32, rb);
              exps(ra, pw0, std::true_type{});
              if (tl && g < 16) tl[g * 8 + 2] = clock64();     // mode 3: stamps 2..5 = chunks done
              tc::tmem_ld_wait();
              mask(1, rb);
              tc::tmem_ld32(t_s + 64, ra);
              free_p();
              tc::tmem_st16(t_p, pw0);
              exps(rb, pw1, std::true_type{});
              tc::tmem_st16(t_p + 16, pw1);
              if (tl && g < 16) tl[g * 8 + 3] = clock64();
              tc::tmem_ld32(t_s + 96, rb);
              tc::tmem_ld_wait();
              mask(2, ra);
              mask(3, rb);
              if (!exact) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  mx = max3(mx, __uint_as_float(ra[i]), __uint_as_float(ra[i + 1]));
                  mx = max3(mx, __uint_as_float(rb[i]), __uint_as_float(rb[i + 1]));
                }
                if (__any_sync(0xffffffffu, mx * sl2 - m > 8.f)) {
                  exact = true;           // S has not been handed back: this attempt's P is overwritten, its row sum dropped
                  continue;
                }
              }
              release_s();
              exps(ra, pw0, std::false_type{});
              tc::tmem_st16(t_p + 32, pw0);
              if (tl && g < 16) tl[g * 8 + 4] = clock64();
              exps(rb, pw1, std::false_type{});
              tc::tmem_st16(t_p + 48, pw1);
              if (tl && g < 16) tl[g * 8 + 5] = clock64();
              float rs_lo, rs_hi;
              upk2(rs2, rs_lo, rs_hi);
              l += rs_lo + rs_hi;
              break;
            }
          }
          tc::tmem_st_wait();
          tc::tc_fence_before();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bar_p[t]);
          if (tl && g < 16) tl[g * 8 + 6] = clock64();
          continue;
        }
        if (tl && g < 16) tl[g * 8 + 0] = clock64();
        wait(&bar_s[t], g & 1, 67);
        tc::tc_fence_after();
        s_seen(j);
        if (tl && g < 16) tl[g * 8 + 1] = clock64();
        float alpha = 1.f;
        bool resc = false;
        const bool masked = j > qt;      // past the diagonal: every key of this block is masked for every row of the tile
        const bool diag = (j == qt);
        const int kc0 = j * 128;
        float m_new = m;
        if (!masked) {
          // pass 1: row maximum
          float mx = -INFINITY;
#pragma unroll
          for (int c = 0; c < 4; c++) {
            uint32_t r[32];
            tc::tmem_ld32(t_s + c * 32, r);
            tc::tmem_ld_wait();
            if (diag) {
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (kc0 + c * 32 + i > qrow) r[i] = 0xff800000u;
            }
#pragma unroll
            for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          }
          m_new = fmaxf(m, mx * sl2);               // finite: key 0 is visible to every query
          if constexpr (LAZY) {
            // The exponentials keep the reference maximum of an earlier block while no row of this warp has grown past
            // it by more than 2^8 (p <= 256 is harmless in bf16 / fp32); only then is O rescaled, for the whole warp
            // (the TMEM accesses are warp-wide).  `masked` and j are the same for the whole warp.
            if (j == 0) {
              m = m_new;
            } else if (__any_sync(0xffffffffu, m_new - m > 8.f)) {
              resc = true;
              alpha = ex2_approx(m - m_new);
              l *= alpha;
              m = m_new;
            }
            m_new = m;
          } else {
            alpha = ex2_approx(m - m_new);            // exp2(-inf) = 0 on the first block
          }
        }
        if (tl && g < 16) tl[g * 8 + 2] = clock64();
        if (j > 0) {   // the previous block's P V has had the whole row-maximum pass to complete; P's columns are free after it
          wait(&bar_o[t], (g - 1) & 1, 68);
          tc::tc_fence_after();
          if (lane == 0) tc::mbar_arrive(&bar_vf[(g - 1) % VN]);
          if (tl && g < 16) tl[g * 8 + 5] = clock64();
          if constexpr (LAZY) {
            if (resc) rescale(alpha);
          } else {
            fold(alpha_prev);
          }
          if (tl && g < 16) tl[g * 8 + 6] = clock64();
        }
        if (masked) {
          uint32_t z[16];
#pragma unroll
          for (int i = 0; i < 16; i++) z[i] = 0u;
#pragma unroll
          for (int c = 0; c < 4; c++) tc::tmem_st16(t_p + c * 16, z);
        } else {
          const uint64_t nm2 = pk2(-m_new, -m_new);
          uint64_t rs2 = pk2(0.f, 0.f);
          // pass 2: exponentials, row sum, P as bf16 pairs into its own TMEM columns
#pragma unroll
          for (int c = 0; c < 4; c++) {
            uint32_t r[32], pw[16];
            tc::tmem_ld32(t_s + c * 32, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int x = 0; x < 16; x++) {
              float z0, z1;
              upk2(fma2(pk2(__uint_as_float(r[2 * x]), __uint_as_float(r[2 * x + 1])), sl2x2, nm2), z0, z1);
              float p0 = ex2_approx(z0), p1 = ex2_approx(z1);
              if (diag) {
                if (kc0 + c * 32 + 2 * x > qrow) p0 = 0.f;
                if (kc0 + c * 32 + 2 * x + 1 > qrow) p1 = 0.f;
              }
              rs2 = add2(rs2, pk2(p0, p1));
              pw[x] = pack_bf16(p0, p1);
            }
            tc::tmem_st16(t_p + c * 16, pw);
          }
          float rs_lo, rs_hi;
          upk2(rs2, rs_lo, rs_hi);
          l = LAZY ? l + (rs_lo + rs_hi) : l * alpha + (rs_lo + rs_hi);
          m = m_new;
        }
        if (tl && g < 16) tl[g * 8 + 3] = clock64();
        tc::tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) { tc::mbar_arrive(&bar_sc[t]); tc::mbar_arrive(&bar_p[t]); }
        if (tl && g < 16) tl[g * 8 + 4] = clock64();
        alpha_prev = alpha;
      }
      wait(&bar_o[t], (g - 1) & 1, 69);
      tc::tc_fence_after();
      if (lane == 0) tc::mbar_arrive(&bar_vf[(g - 1) % VN]);
      fold(alpha_prev);
      if constexpr (MODE == 3) l *= P_BIAS_INV;
      const float inv = 1.f / l;
      const bool store = !*s_abort && qrow < a.T;
      bf16* dst = a.out + ((size_t)(it.b * a.T + qrow)) * C + it.h * HD;
      if constexpr (LAZY) {
        // the accumulated O leaves TMEM here; the next item's first P V (accumulate off) is ordered behind these loads
        // by this warp's arrival on bar_p for that block.  With whole tiles (T a multiple of 128) the bf16 rows go
        // through a swizzled staging tile and leave with one TMA store per warp: a store instruction whose lanes hit 32
        // different lines keeps the load/store unit busy for tens of cycles, eight of them per thread.
        uint8_t* stage = smem + S::OST + warp * 4096;
        if (a.out_tma) {
          if (lane == 0) tc::tma_wait_group_read<0>();      // the previous item's rows have been read out of the staging tile
          __syncwarp();
        }
  #pragma unroll
        for (int c = 0; c < 2; c++) {
          uint32_t r[32];
          tc::tmem_ld32(t_o + c * 32, r);
          tc::tmem_ld_wait();
#pragma unroll
          for (int v8 = 0; v8 < 4; v8++) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(r[v8 * 8 + 0]) * inv, __uint_as_float(r[v8 * 8 + 1]) * inv);
            pk.y = pack_bf16(__uint_as_float(r[v8 * 8 + 2]) * inv, __uint_as_float(r[v8 * 8 + 3]) * inv);
            pk.z = pack_bf16(__uint_as_float(r[v8 * 8 + 4]) * inv, __uint_as_float(r[v8 * 8 + 5]) * inv);
            pk.w = pack_bf16(__uint_as_float(r[v8 * 8 + 6]) * inv, __uint_as_float(r[v8 * 8 + 7]) * inv);
            if (a.out_tma) *reinterpret_cast<uint4*>(stage + lane * 128 + (((c * 4 + v8) ^ (lane & 7)) << 4)) = pk;
            else if (store) *reinterpret_cast<uint4*>(dst + c * 32 + v8 * 8) = pk;
          }
        }
          if (a.out_tma) {
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0 && !*s_abort && qt * 128 < a.T) {   // (an odd number of query tiles leaves the last pair's second tile empty)
            tc::tma_store_2d(&tm_out, stage, it.h * HD, it.b * a.T + qt * 128 + lg * 32);
            tc::tma_commit_group();
          }
        }
      } else if (store) {
#pragma unroll
        for (int v8 = 0; v8 < HD / 8; v8++) {
          uint4 pk;
          pk.x = pack_bf16(o[v8 * 8 + 0] * inv, o[v8 * 8 + 1] * inv); pk.y = pack_bf16(o[v8 * 8 + 2] * inv, o[v8 * 8 + 3] * inv);
          pk.z = pack_bf16(o[v8 * 8 + 4] * inv, o[v8 * 8 + 5] * inv); pk.w = pack_bf16(o[v8 * 8 + 6] * inv, o[v8 * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(dst + v8 * 8) = pk;
        }
      }
      if (store) {
        a.lse[((size_t)it.b * a.H + it.h) * a.T + qrow] = (m + log2f(l)) * LN2;
      }
      if (tl && g <= 16) tl[(g - 1) * 8 + 7] = clock64();     // stamp 7 of an item's last block: its epilogue is done
    }
    if (lane == 0) tc::tma_wait_group<0>();     // this warp's TMA stores of O have completed before the CTA's shared memory goes
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 8) tc::tmem_dealloc(tmem, TMEM_COLS);
  if (dyn && tid == 0) attn_ctr_leave(0);
}

// ================================================================== backward: delta = rowsum(dO * O)
__global__ void attn_delta_k(float* __restrict__ delta, const bf16* __restrict__ dout, const bf16* __restrict__ out, int B, int T,
                             int H, int hd) {
  mlb_pdl_sync();
  // one group of hd/8 consecutive lanes per (row, head): 16-byte loads, shuffle reduction inside the group.  The host
  // launches this kernel only when B*T*H*hd/8 fits 31 bits, so all index arithmetic is 32-bit (a 64-bit division by
  // a run-time value costs more instructions than the rest of the thread's work).
  const unsigned gsz = (unsigned)hd >> 3;  // lanes per head (8 for hd=64, 16 for hd=128); a power of two <= 32 on this path
  const unsigned tid = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned gidx = tid / gsz, gl = tid % gsz;
  const unsigned total = (unsigned)B * T * H;
  float s = 0.f;
  if (gidx < total) {
    const size_t e = (size_t)gidx * hd + gl * 8;
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(out + e));
    const uint4 d = __ldcs(reinterpret_cast<const uint4*>(dout + e));
    const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      s = fmaf(__uint_as_float(wa[i] << 16), __uint_as_float(wd[i] << 16), s);
      s = fmaf(__uint_as_float(wa[i] & 0xffff0000u), __uint_as_float(wd[i] & 0xffff0000u), s);
    }
  }
  for (unsigned o = gsz >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (gidx < total && gl == 0) {
    const unsigned h = gidx % (unsigned)H, bt = gidx / (unsigned)H;
    const unsigned b = bt / (unsigned)T, t = bt % (unsigned)T;
    delta[((size_t)b * H + h) * T + t] = s;
  }
}
__global__ void attn_delta_scalar_k(float* __restrict__ delta, const bf16* __restrict__ dout, const bf16* __restrict__ out, int B,
                                    int T, int H, int hd) {
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long)B * T * H) return;
  const int h = w % H;
  const long bt = w / H;
  const bf16* po = out + bt * (long)H * hd + h * hd;
  const bf16* pd = dout + bt * (long)H * hd + h * hd;
  float s = 0.f;
  for (int i = lane; i < hd; i += 32) s += __bfloat162float(po[i]) * __bfloat162float(pd[i]);
  s = warp_sum(s);
  const int b = bt / T, t = bt % T;
  if (lane == 0) delta[((long)b * H + h) * T + t] = s;
}

// Epilogue helper for the backward kernels: one warp moves 64 accumulator columns of its 32 rows from TMEM to
// dst as bf16: columns [c0, c0+32) and [c0 + HD/2, c0 + HD/2 + 32), which are exactly RoPE's rotation pairs
// (i, i + HD/2).  With tables given, RoPE's backward rotation (d0' = d0 c + d1 s, d1' = d1 c - d0 s) is applied.
template <int HD>
__device__ __forceinline__ void store_pairs_rope(bf16* dst_row, uint32_t taddr, int c0, bool live, const float* cosT,
                                                 const float* sinT, int t, float out_scale = 1.f) {
  uint32_t ra[32], rb[32];
  tc::tmem_ld32(taddr + c0, ra);
  tc::tmem_ld32(taddr + c0 + HD / 2, rb);
  tc::tmem_ld_wait();
  if (!live) return;
  float x0[32], x1[32];
#pragma unroll
  for (int i = 0; i < 32; i++) { x0[i] = __uint_as_float(ra[i]) * out_scale; x1[i] = __uint_as_float(rb[i]) * out_scale; }
  if (cosT) {
    const float* c = cosT + (size_t)t * (HD / 2) + c0;
    const float* s = sinT + (size_t)t * (HD / 2) + c0;
#pragma unroll
    for (int i = 0; i < 32; i++) {
      const float d0 = x0[i], d1 = x1[i], cc = c[i], ss = s[i];
      x0[i] = d0 * cc + d1 * ss;
      x1[i] = d1 * cc - d0 * ss;
    }
  }
#pragma unroll
  for (int v8 = 0; v8 < 4; v8++) {
    uint4 pa, pb;
    pa.x = pack_bf16(x0[v8 * 8 + 0], x0[v8 * 8 + 1]); pa.y = pack_bf16(x0[v8 * 8 + 2], x0[v8 * 8 + 3]);
    pa.z = pack_bf16(x0[v8 * 8 + 4], x0[v8 * 8 + 5]); pa.w = pack_bf16(x0[v8 * 8 + 6], x0[v8 * 8 + 7]);
    pb.x = pack_bf16(x1[v8 * 8 + 0], x1[v8 * 8 + 1]); pb.y = pack_bf16(x1[v8 * 8 + 2], x1[v8 * 8 + 3]);
    pb.z = pack_bf16(x1[v8 * 8 + 4], x1[v8 * 8 + 5]); pb.w = pack_bf16(x1[v8 * 8 + 6], x1[v8 * 8 + 7]);
    *reinterpret_cast<uint4*>(dst_row + c0 + v8 * 8) = pa;
    *reinterpret_cast<uint4*>(dst_row + c0 + HD / 2 + v8 * 8) = pb;
  }
}

constexpr int BWD_THREADS = 512;

// ================================================================== backward: dK, dV (one CTA per 128-key tile)
// 512 threads; thread (row = key, quarter cq) handles 32 of the 128 query columns of S^T / dP^T.  The MMAs of the next
// query block are queued right behind the dV/dK MMAs of the current one, so one commit covers both.
template <int HD>
struct BwdKVSmem {
  static constexpr int CH = HD / 64;
  static constexpr int NBUF = (HD == 64) ? 2 : 1;
  static constexpr int K = 0;
  static constexpr int V = K + CH * TILE_BYTES;
  static constexpr int Q = V + CH * TILE_BYTES;                 // NBUF buffers
  static constexpr int DO = Q + NBUF * CH * TILE_BYTES;         // NBUF buffers
  static constexpr int PT = DO + NBUF * CH * TILE_BYTES;
  static constexpr int DST = PT + 2 * TILE_BYTES;
  static constexpr int STAT = DST + 2 * TILE_BYTES;             // lse[128], delta[128] floats
  static constexpr int BAR = STAT + 1024;
  static constexpr int TOTAL = BAR + 128 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_kv_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv,
                                                                        const __grid_constant__ CUtensorMap tm_do,
                                                                        const AttnArgs a) {
  using S = BwdKVSmem<HD>;
  constexpr int CH = HD / 64, NBUF = S::NBUF;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + S::BAR);
  uint64_t *bar_kv = bars, *bar_q = bars + 1 /*[2]*/, *bar_s = bars + 3, *bar_d = bars + 4;
  uint32_t* tmem_slot = (uint32_t*)(bars + 5);
  float* s_lse = (float*)(smem + S::STAT);
  float* s_delta = s_lse + 128;

  const int nq = (a.T + 127) / 128;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kt * 128;
  const int C = a.H * HD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = warp & 3, cq = warp >> 2, row = lg * 32 + lane;
  const int row0 = b * a.T;

  if (tid == 0) {
    tc::mbar_init(bar_kv, 1); tc::mbar_init(&bar_q[0], 1); tc::mbar_init(&bar_q[1], 1);
    tc::mbar_init(bar_s, 1); tc::mbar_init(bar_d, 1);
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tm_qkv);
    tc::tma_prefetch_desc(&tm_do);
  }
  if (warp == 0) tc::tmem_alloc(tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_st = tmem, t_dpt = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 256 + HD;
  const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
  constexpr uint32_t idesc_s = tc::idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_d = tc::idesc_bf16(128, HD, 0, 1);
  const uint32_t sK = tc::smem_u32(smem + S::K), sV = tc::smem_u32(smem + S::V);
  const uint32_t sPT = tc::smem_u32(smem + S::PT), sDST = tc::smem_u32(smem + S::DST);

  auto load_q_do = [&](int i, int buf) {
    tc::mbar_expect_tx(&bar_q[buf], 2 * CH * TILE_BYTES);
    for (int c = 0; c < CH; c++) {
      tc::tma_load_2d(smem + S::Q + (buf * CH + c) * TILE_BYTES, &tm_qkv, &bar_q[buf], h * HD + c * 64, row0 + i * 128);
      tc::tma_load_2d(smem + S::DO + (buf * CH + c) * TILE_BYTES, &tm_do, &bar_q[buf], h * HD + c * 64, row0 + i * 128);
    }
  };
  auto issue_scores = [&](int buf) {   // S^T = K Q^T and dP^T = V dO^T for the block in `buf`
    const uint32_t sQ = tc::smem_u32(smem + S::Q + buf * CH * TILE_BYTES), sDO = tc::smem_u32(smem + S::DO + buf * CH * TILE_BYTES);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(t_st, desc_k(sK, ks), desc_k(sQ, ks), idesc_s, ks > 0);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(t_dpt, desc_k(sV, ks), desc_k(sDO, ks), idesc_s, ks > 0);
  };
  const int n_it = nq - kt;
  if (tid == 0) {
    tc::mbar_expect_tx(bar_kv, 2 * CH * TILE_BYTES);
    for (int c = 0; c < CH; c++) {
      tc::tma_load_2d(smem + S::K + c * TILE_BYTES, &tm_qkv, bar_kv, C + h * HD + c * 64, row0 + k0);
      tc::tma_load_2d(smem + S::V + c * TILE_BYTES, &tm_qkv, bar_kv, 2 * C + h * HD + c * 64, row0 + k0);
    }
    load_q_do(kt, 0);
    if (tc::mbar_wait(bar_kv, 0, 20) && tc::mbar_wait(&bar_q[0], 0, 21)) {
      tc::tc_fence_after();
      issue_scores(0);
    }
    tc::mma_commit(bar_s);
  }
  const float sl2 = a.scale * LOG2E;
  const int krow = k0 + row;
  bool ok = true;
  for (int it = 0; it < n_it; it++) {
    const int i = kt + it, q0 = i * 128;
    const int buf = (NBUF == 2) ? (it & 1) : 0;
    if (tid < 256) {   // per-query statistics of this block (queries past the sequence end contribute nothing)
      const int q = q0 + (tid & 127);
      const size_t si = ((size_t)b * a.H + h) * a.T + q;
      if (tid < 128) s_lse[tid] = (q < a.T) ? a.lse[si] * LOG2E : INFINITY;
      else s_delta[tid - 128] = (q < a.T) ? a.delta[si] : 0.f;
    }
    __syncthreads();
    if (!tc::mbar_wait(bar_s, it & 1, 22)) { ok = false; break; }
    tc::tc_fence_after();
    // every MMA issued so far has completed: the other Q/dO buffer (read by the previous dV/dK) can be refilled
    if (NBUF == 2 && tid == 0 && it + 1 < n_it) load_q_do(i + 1, buf ^ 1);
    const bool diag = (it == 0);
    {
      uint32_t rs[32], rd[32];
      tc::tmem_ld32(t_st + lane_addr + cq * 32, rs);
      tc::tmem_ld32(t_dpt + lane_addr + cq * 32, rd);
      tc::tmem_ld_wait();
#pragma unroll
      for (int v8 = 0; v8 < 4; v8++) {
        float p[8], ds[8];
#pragma unroll
        for (int x = 0; x < 8; x++) {
          const int qc = cq * 32 + v8 * 8 + x;
          float pv = exp2f(__uint_as_float(rs[v8 * 8 + x]) * sl2 - s_lse[qc]);
          if (diag && (q0 + qc) < krow) pv = 0.f;
          p[x] = pv;
          ds[x] = pv * (__uint_as_float(rd[v8 * 8 + x]) - s_delta[qc]) * a.scale;
        }
        uint4 pk, dk;
        pk.x = pack_bf16(p[0], p[1]); pk.y = pack_bf16(p[2], p[3]); pk.z = pack_bf16(p[4], p[5]); pk.w = pack_bf16(p[6], p[7]);
        dk.x = pack_bf16(ds[0], ds[1]); dk.y = pack_bf16(ds[2], ds[3]); dk.z = pack_bf16(ds[4], ds[5]); dk.w = pack_bf16(ds[6], ds[7]);
        const uint32_t off = sw_off(row, cq * 32 + v8 * 8);
        *reinterpret_cast<uint4*>(smem + S::PT + off) = pk;
        *reinterpret_cast<uint4*>(smem + S::DST + off) = dk;
      }
    }
    tc::fence_async_smem();
    tc::tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc::tc_fence_after();
      const uint32_t sQ = tc::smem_u32(smem + S::Q + buf * CH * TILE_BYTES), sDO = tc::smem_u32(smem + S::DO + buf * CH * TILE_BYTES);
#pragma unroll
      for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ss(t_dv, desc_k(sPT, ks), desc_mn(sDO, ks), idesc_d, (it > 0 || ks > 0));
#pragma unroll
      for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ss(t_dk, desc_k(sDST, ks), desc_mn(sQ, ks), idesc_d, (it > 0 || ks > 0));
      if (it + 1 < n_it) {
        bool ready = true;
        if (NBUF == 1) {   // single buffer: dV/dK must finish reading Q/dO before the next block is loaded over them
          tc::mma_commit(bar_d);
          ready = tc::mbar_wait(bar_d, it & 1, 23);
          if (ready) load_q_do(i + 1, 0);
        }
        const int nb = (NBUF == 2) ? (buf ^ 1) : 0;
        const int nphase = (NBUF == 2) ? (((it + 1) >> 1) & 1) : ((it + 1) & 1);
        if (ready && tc::mbar_wait(&bar_q[nb], nphase, 24)) {
          tc::tc_fence_after();
          issue_scores(nb);
        }
      }
      tc::mma_commit(bar_s);
    }
  }
  if (ok) ok = tc::mbar_wait(bar_s, n_it & 1, 25);   // dV / dK of the last block are complete
  tc::tc_fence_after();
  if (ok) {
    // jobs: HD/64 column-pair slabs for dK (with RoPE) then HD/64 for dV; one job per quarter-group of warps
    constexpr int JOBS = HD / 64;
    if (cq < 2 * JOBS) {
      const bool is_k = cq < JOBS;
      const int pass = is_k ? cq : cq - JOBS;
      bf16* dst = a.out + ((size_t)(row0 + krow)) * 3 * C + (is_k ? C : 2 * C) + h * HD;
      store_pairs_rope<HD>(dst, (is_k ? t_dk : t_dv) + lane_addr, pass * 32, krow < a.T, is_k ? a.cosT : nullptr,
                           is_k ? a.sinT : nullptr, krow);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
}

// ================================================================== backward, head size 64: ONE kernel, five GEMMs
// Persistent CTAs, one per SM; a work item is one 128-key tile of a (sample, head) and loops over the query tiles
// i >= its own; the items of a CTA come from a balanced schedule built on the host (attn_schedule).  Per query block:
//     S^T = K Q^T, dP^T = V dO^T                            (two MMAs into TMEM)
//     P^T = exp2(S^T*c - lse), dS^T = P^T (dP^T - delta)    (512 threads, packed f32x2 math)
//     dV += P^T dO   (P^T stays in TMEM as the bf16 A operand),   dK += dS^T Q,   dQ_i = dS K   (dS^T in shared memory)
// The pipeline keeps the tensor core and the element-wise warps busy at the same time:
//   * as soon as the element-wise warps have S^T / dP^T of block j in registers they release the TMEM columns and the
//     control thread issues the score MMAs of block j+1 (Q / dO tiles are triple buffered so they are already there);
//   * the exponentials of block j+1 are computed while dV / dK / dQ of block j run; only the stores of P^T / dS^T wait
//     for those MMAs (one TMEM region, one shared-memory tile);
//   * dQ_j is a partial sum over key tiles.  fp32 add-reduces into one accumulator (TMA or vector red) ran into the
//     L2's atomic throughput (32 KB per block and SM); instead every (query tile, key tile) pair owns a bf16 tile of a
//     partial buffer, written with plain stores right after block j+1's operands are handed over, and a second
//     kernel adds the partials of a query row in fp32 in key-tile order (deterministic), applies the scale and RoPE's
//     backward rotation and writes bf16 dQ.
// Warps: 8 element-wise (TMEM lane group x 64-query half), 4 drain (dQ partial tiles, dK / dV epilogue), 2 MMA issuers (scores / gradients), 1 loader.
// mbarriers: bar_s scores complete (commit) | bar_free S^T/dP^T read out (8 warps) | bar_p P^T/dS^T stored (8 warps) |
// bar_dv dV MMAs complete (commit: P^T may be overwritten) | bar_d[2] dV/dK/dQ MMAs complete (commit, alternating so
// that a waiter two blocks behind cannot mistake a phase) | bar_dqf dQ read out (4 warps) | bar_epi dK/dV of a key tile read out (4 warps).
struct BwdFusedSmem {
  static constexpr int K = 0;
  static constexpr int V = K + TILE_BYTES;
  static constexpr int Q = V + TILE_BYTES;               // 3 buffers
  static constexpr int DO = Q + 3 * TILE_BYTES;          // 3 buffers
  static constexpr int DST = DO + 3 * TILE_BYTES;        // 2 buffers x [128 keys x 128 queries] bf16
  static constexpr int DQS = DST + 4 * TILE_BYTES;       // dQ staging: 4 drain warps x [32 rows x 128 B] bf16, swizzled
  static constexpr int STAT = DQS + TILE_BYTES;          // 8 warps x (-lse*log2e [64], -delta [64])
  static constexpr int BAR = STAT + 4096;
  static constexpr int SCHED = BAR + 256;                // this CTA's first 64 work items
  static constexpr int TOTAL = SCHED + 768 + 1024;             // SCHED: 64 items, or a ring of 64 (value, sequence number) + end marker
};

constexpr int BWDF_E_WARPS = 8;       // element-wise warps: TMEM lane group (w & 3) x 64-query column half (w >> 2)
constexpr int BWDF_D_WARPS = 4;       // drain warps: dQ partial tiles and the dK / dV epilogue, one TMEM lane group each
// Warp w runs on scheduler w % 4.  Warp 12 stays idle so that the two MMA warps (13, 14) and the loader warp (15) land on
// schedulers 1, 2 and 3: every scheduler then carries two element-wise warps, one drain warp and at most one light warp.
constexpr int BWDF_SCORE_WARP = BWDF_E_WARPS + BWDF_D_WARPS + 1;  // issues S^T / dP^T (scheduler 1)
constexpr int BWDF_CTRL_WARP = BWDF_E_WARPS + BWDF_D_WARPS + 2;   // issues dV / dK / dQ (scheduler 2)
constexpr int BWDF_LOAD_WARP = BWDF_CTRL_WARP + 1;                // issues every TMA load
constexpr int BWDF_THREADS = (BWDF_LOAD_WARP + 1) * 32;

template <bool DYN>
__global__ void __maxnreg__(120) attn_bwd_fused_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv,
                                                                            const __grid_constant__ CUtensorMap tm_do,
                                                                            const __grid_constant__ CUtensorMap tm_dq, const AttnArgs a) {
  mlb_pdl_sync();
  using S = BwdFusedSmem;
  constexpr int HD = 64;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + S::BAR);
  uint64_t *bar_kv = bars, *bar_q = bars + 1 /*[3]*/, *bar_s = bars + 4, *bar_free = bars + 5, *bar_p = bars + 6, *bar_dv = bars + 7,
           *bar_dqf = bars + 8, *bar_epi = bars + 9, *bar_d = bars + 12 /*[2]: block blk completes bar_d[blk & 1]*/;
  uint32_t* tmem_slot = (uint32_t*)(bars + 10);
  volatile int* s_abort = (volatile int*)(bars + 11);
  float* s_stat = (float*)(smem + S::STAT);   // [8 warps][-lse*log2e x64 | -delta x64]
  {
    __shared__ int s_skip;
    if (threadIdx.x == 0) s_skip = *(volatile int*)&g_mlb_error;
    __syncthreads();
    if (s_skip != 0) return;
  }
  const int nq = (a.T + 127) / 128;
  const int C = a.H * HD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Persistent CTAs: work item w = key tile kt = w / (B*H) of (sample, head) w % (B*H), so the items are in descending
  // cost order (a key tile meets the nq - kt query tiles at or after it).  A CTA's items come from the host's balanced
  // schedule (rows end with -1 entries; the first 64 are copied to shared memory), else round robin over the grid.
  const int BH = a.B * a.H, total = nq * BH;
  const int* srow = a.sched ? a.sched + (size_t)blockIdx.x * a.sched_stride : nullptr;
  int* s_sched = (int*)(smem + S::SCHED);
  if (srow && tid < 64) s_sched[tid] = tid < a.sched_stride ? __ldg(srow + tid) : -1;
  struct Item { int kt, b, h, row0; bool valid; };
  constexpr bool dyn = DYN;
  ItemRing ring{(volatile int*)s_sched, (volatile int*)s_sched + 64, 0};
  if (dyn && tid <= 64) s_sched[64 + tid] = tid < 64 ? 0 : 0x7fffffff;
  const bool publisher = warp == BWDF_LOAD_WARP && lane == 0;
  auto item_at = [&](int li) -> Item {
    int w;
    if (dyn) w = publisher ? ring.draw(li, 1, total) : ring.read(li, s_abort);
    else if (srow) w = li < 64 ? s_sched[li] : __ldg(srow + li);
    else { w = blockIdx.x + li * gridDim.x; if (w >= total) w = -1; }
    Item r;
    r.valid = w >= 0;
    if (!r.valid) w = 0;
    r.kt = w / BH;
    const int bh = w - r.kt * BH;
    r.b = bh / a.H;
    r.h = bh - r.b * a.H;
    r.row0 = r.b * a.T;
    return r;
  };

  if (tid == 0) {
    tc::mbar_init(bar_kv, 1);
    for (int i = 0; i < 3; i++) tc::mbar_init(&bar_q[i], 1);
    tc::mbar_init(bar_s, 1); tc::mbar_init(bar_dv, 1); tc::mbar_init(&bar_d[0], 1); tc::mbar_init(&bar_d[1], 1);
    tc::mbar_init(bar_free, BWDF_E_WARPS); tc::mbar_init(bar_p, BWDF_E_WARPS);
    tc::mbar_init(bar_dqf, BWDF_D_WARPS); tc::mbar_init(bar_epi, BWDF_D_WARPS);
    *s_abort = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tm_qkv);
    tc::tma_prefetch_desc(&tm_do);
    tc::tma_prefetch_desc(&tm_dq);
  }
  if (warp == BWDF_CTRL_WARP) tc::tmem_alloc(tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // S^T 128 | dP^T 128 | P^T (bf16 pairs) 64 | dV 64 | dK 64 | dQ 64
  const uint32_t t_st = tmem, t_dpt = tmem + 128, t_pt = tmem + 256, t_dv = tmem + 320, t_dk = tmem + 384, t_dq = tmem + 448;
  auto wait = [&](uint64_t* bar, uint32_t phase, int where) -> bool {
    if (tc::mbar_try(bar, phase)) return true;
    if (*s_abort) return false;
    if (!tc::mbar_wait(bar, phase, where)) { *s_abort = 1; return false; }
    return true;
  };
  long long* tl = (a.timeline && blockIdx.x == 0 && lane == 0) ? a.timeline : nullptr;

  if (warp == BWDF_LOAD_WARP) {
    // ---------------------------------------------------------------- loader warp: every TMA load
    if (lane == 0) {
      auto load_kv = [&](const Item& w) {
        tc::mbar_expect_tx(bar_kv, 2 * TILE_BYTES);
        tc::tma_load_2d(smem + S::K, &tm_qkv, bar_kv, C + w.h * HD, w.row0 + w.kt * 128);
        tc::tma_load_2d(smem + S::V, &tm_qkv, bar_kv, 2 * C + w.h * HD, w.row0 + w.kt * 128);
      };
      auto load_q_do = [&](const Item& w, int i, int g) {          // g: running block number, buffer g % 3
        const int buf = g % 3;
        tc::mbar_expect_tx(&bar_q[buf], 2 * TILE_BYTES);
        tc::tma_load_2d(smem + S::Q + buf * TILE_BYTES, &tm_qkv, &bar_q[buf], w.h * HD, w.row0 + i * 128);
        tc::tma_load_2d(smem + S::DO + buf * TILE_BYTES, &tm_do, &bar_q[buf], w.h * HD, w.row0 + i * 128);
      };
      int blk = 0;
      Item cur = item_at(0);
      if (cur.valid) {
        load_kv(cur);
        load_q_do(cur, cur.kt, 0);
        if (nq - cur.kt > 1) load_q_do(cur, cur.kt + 1, 1);
      }
      for (int li = 0; cur.valid; li++) {
        const int kt = cur.kt;
        const int n_it = nq - kt;
        for (int it = 0; it < n_it; it++, blk++) {
          // the tiles of block it+2 go where block it-1's were: its dV / dK MMAs must have finished reading them
          // (every completion of bar_d is observed, so this thread's parity never falls a whole period behind)
          if (blk > 0) wait(&bar_d[(blk - 1) & 1], ((blk - 1) >> 1) & 1, 43);
          if (it + 2 < n_it) load_q_do(cur, kt + it + 2, blk + 2);
        }
        const Item nx = item_at(li + 1);
        if (nx.valid) {
          // every MMA of this key tile is complete: K, V and all Q / dO buffers are free for the next item
          wait(&bar_d[(blk - 1) & 1], ((blk - 1) >> 1) & 1, 44);
          load_kv(nx);
          load_q_do(nx, nx.kt, blk);
          if (nq - nx.kt > 1) load_q_do(nx, nx.kt + 1, blk + 1);
        }
        cur = nx;
      }
    }
  } else if (warp == BWDF_CTRL_WARP || warp == BWDF_SCORE_WARP) {
    // ---------------------------------------------------------------- two MMA warps: waits, tcgen05.mma, commits, nothing else
    // Every tcgen05.mma / commit costs its issuing thread ~75 cycles whatever the product's size: 32 MMAs and two commits
    // per query block from ONE thread were 2700 of the block's 3500 cycles, never waiting.  The 8 score MMAs have
    // their own issuing thread, so they go out while the 24 gradient MMAs of the previous block are still being issued.
    // (Descriptors are formed by adding small constants to per-buffer bases.)
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc::idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_d = tc::idesc_bf16(128, HD, 0, 1);    // A K-major (P^T in TMEM / dS^T), B MN-major (dO / Q)
      constexpr uint32_t idesc_q = tc::idesc_bf16(128, HD, 1, 1);    // A MN-major (dS^T read as dS), B MN-major (K)
      constexpr uint64_t TILE_D = TILE_BYTES >> 4;
      const uint64_t dKk = desc_base_k(tc::smem_u32(smem + S::K)), dVk = desc_base_k(tc::smem_u32(smem + S::V));
      const uint64_t dQk = desc_base_k(tc::smem_u32(smem + S::Q)), dDOk = desc_base_k(tc::smem_u32(smem + S::DO));
      const uint64_t dQmn = desc_base_mn(tc::smem_u32(smem + S::Q)), dDOmn = desc_base_mn(tc::smem_u32(smem + S::DO));
      const uint64_t dKmn = desc_base_mn(tc::smem_u32(smem + S::K));
      const uint64_t dSTk = desc_base_k(tc::smem_u32(smem + S::DST)), dSTmn = desc_base_mn(tc::smem_u32(smem + S::DST));
      auto issue_scores = [&](int buf, uint32_t q_phase) {
        if (!wait(&bar_q[buf], q_phase, 41)) return;
        tc::tc_fence_after();
        const uint64_t o = (uint64_t)buf * TILE_D;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(t_st, dKk + ks * 2, dQk + o + ks * 2, idesc_s, ks > 0);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(t_dpt, dVk + ks * 2, dDOk + o + ks * 2, idesc_s, ks > 0);
      };
      int blk = 0, buf = 0, q_use = 0;     // buffer blk % 3 and how many times it has been filled before (blk / 3)
      if (warp == BWDF_SCORE_WARP) {
        // the score products: S^T / dP^T of block j+1 as soon as block j's have been read out of TMEM
        for (int item = 0;; item++) {
          const Item cur = item_at(item);
          if (!cur.valid) break;
          const int n_it = nq - cur.kt;
          if (wait(bar_kv, item & 1, 40)) issue_scores(buf, q_use & 1);
          tc::mma_commit(bar_s);
          for (int it = 0; it < n_it; it++, blk++) {
            int nbuf = buf + 1, nq_use = q_use;
            if (nbuf == 3) { nbuf = 0; nq_use++; }
            // S^T / dP^T of this block are in registers: the score MMAs of the next block may overwrite them
            wait(bar_free, blk & 1, 42);
            if (it + 1 < n_it) {
              tc::tc_fence_after();
              issue_scores(nbuf, nq_use & 1);
              tc::mma_commit(bar_s);
            }
            buf = nbuf; q_use = nq_use;
          }
        }
      } else {
        // the gradient products of block j once P^T / dS^T are stored
        for (int item = 0;; item++) {
          const Item cur = item_at(item);
          if (!cur.valid) break;
          const int n_it = nq - cur.kt;
          for (int it = 0; it < n_it; it++, blk++) {
            bool go = wait(bar_p, blk & 1, 45);     // P^T in TMEM, dS^T in shared memory
            if (tl) tl[blk * 8 + 5] = clock64();
            if (it == 0) go = wait(bar_kv, item & 1, 40) && go;       // (seen by the score thread long ago; this thread reads K too)
            go = wait(&bar_q[buf], q_use & 1, 41) && go;
            if (it == 0 && item > 0) go = wait(bar_epi, (item - 1) & 1, 46) && go;   // previous tile's dK / dV have been read out
            const bool dv_go = go;
            if (go) {
              tc::tc_fence_after();
              const uint64_t o = (uint64_t)buf * TILE_D;
              const uint64_t od = (uint64_t)(blk & 1) * 2 * TILE_D;     // dS^T buffer of this block
              const uint32_t acc = it > 0;
#pragma unroll
              for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ts(t_dv, t_pt + ks * 8, dDOmn + o + ks * 128, idesc_d, acc | (ks > 0));
              tc::mma_commit(bar_dv);       // P^T's columns are free for the next block while dK and dQ are still going
#pragma unroll
              for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ss(t_dk, dSTk + od + (ks >> 2) * TILE_D + (ks & 3) * 2, dQmn + o + ks * 128, idesc_d, acc | (ks > 0));
              if (blk > 0) go = wait(bar_dqf, (blk - 1) & 1, 47);   // the previous dQ tile has left TMEM
              if (go) {
                tc::tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ss(t_dq, dSTmn + od + ks * 128, dKmn + ks * 128, idesc_q, ks > 0);
              }
            }
            if (!dv_go) tc::mma_commit(bar_dv);     // (aborting: keep the barrier's phases in step)
            tc::mma_commit(&bar_d[blk & 1]);
            if (tl) tl[blk * 8 + 6] = clock64();
            if (++buf == 3) { buf = 0; q_use++; }
          }
        }
      }
    }
  } else if (warp < BWDF_E_WARPS) {
    // ---------------------------------------------------------------- 8 element-wise warps
    const int lg = warp & 3, ch = warp >> 2, row = lg * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
    const float sl2 = a.scale * LOG2E;
    const uint64_t sl2x2 = pk2(sl2, sl2);
    // per-query statistics: each warp keeps the 64 queries of its column half in a private shared-memory slot
    // (-lse*log2e, -delta; queries past the end give P = 0).  Lane l fetches queries l and l+32 of the NEXT block while
    // this block is processed, so neither the load latency nor a CTA-wide barrier sits between two blocks.
    float* my_stat = s_stat + warp * 128;
    auto fetch_stat = [&](const Item& w, int i, float (&l)[2], float (&d)[2]) {
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int q = i * 128 + ch * 64 + u * 32 + lane;
        const size_t si = ((size_t)w.b * a.H + w.h) * a.T + q;
        l[u] = (q < a.T) ? a.lse[si] : INFINITY;
        d[u] = (q < a.T) ? a.delta[si] : 0.f;
      }
    };
    int blk = 0;
    for (int item = 0;; item++) {
      const Item cur = item_at(item);
      if (!cur.valid) break;
      const int kt = cur.kt;
      const int k0 = kt * 128, krow = k0 + row;
      const int n_it = nq - kt;
      float st_l[2], st_d[2];
      fetch_stat(cur, kt, st_l, st_d);
      for (int it = 0; it < n_it; it++, blk++) {
        const int i = kt + it, q0 = i * 128;
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 2; u++) {
          my_stat[u * 32 + lane] = -st_l[u] * LOG2E;
          my_stat[64 + u * 32 + lane] = -st_d[u];
        }
        __syncwarp();
        if (it + 1 < n_it) fetch_stat(cur, i + 1, st_l, st_d);
        if (tl && warp == 0) tl[blk * 8 + 0] = clock64();
        wait(bar_s, blk & 1, 48);          // S^T, dP^T of this block are complete
        tc::tc_fence_after();
        if (tl && warp == 0) tl[blk * 8 + 1] = clock64();
        // dS^T of this block goes into the shared-memory tile that block blk-2's dK / dQ MMAs read
        if (blk >= 2) wait(&bar_d[blk & 1], ((blk >> 1) + 1) & 1, 51);
        uint32_t pw[2][16];
        const bool diag = (it == 0);
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          uint32_t rs[32], rd[32];
          const int c0 = ch * 64 + hf * 32;      // first query column of this pass
          tc::tmem_ld32(t_st + lane_addr + c0, rs);
          tc::tmem_ld32(t_dpt + lane_addr + c0, rd);
          tc::tmem_ld_wait();
          if (hf == 1) {
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar_free);
          }
#pragma unroll
          for (int v8 = 0; v8 < 4; v8++) {
            const int qc = c0 + v8 * 8;
            const float* sn = my_stat + hf * 32 + v8 * 8;
            float nl[8], nd[8];
            uint32_t dw[4];
            *reinterpret_cast<float4*>(nl) = *reinterpret_cast<const float4*>(sn);
            *reinterpret_cast<float4*>(nl + 4) = *reinterpret_cast<const float4*>(sn + 4);
            *reinterpret_cast<float4*>(nd) = *reinterpret_cast<const float4*>(sn + 64);
            *reinterpret_cast<float4*>(nd + 4) = *reinterpret_cast<const float4*>(sn + 68);
#pragma unroll
            for (int x = 0; x < 4; x++) {
              const int e = v8 * 8 + 2 * x;
              float z0, z1;
              upk2(fma2(pk2(__uint_as_float(rs[e]), __uint_as_float(rs[e + 1])), sl2x2, pk2(nl[2 * x], nl[2 * x + 1])), z0, z1);
              float p0 = ex2_approx(z0), p1 = ex2_approx(z1);
              if (diag) {
                if (q0 + qc + 2 * x < krow) p0 = 0.f;
                if (q0 + qc + 2 * x + 1 < krow) p1 = 0.f;
              }
              const uint64_t t2 = add2(pk2(__uint_as_float(rd[e]), __uint_as_float(rd[e + 1])), pk2(nd[2 * x], nd[2 * x + 1]));
              float d0, d1;
              upk2(mul2(pk2(p0, p1), t2), d0, d1);
              pw[hf][v8 * 4 + x] = pack_bf16(p0, p1);
              dw[x] = pack_bf16(d0, d1);
            }
            // dS^T goes straight into the buffer that block blk-2 used: only the two TMEM stores of P^T are left to do
            // once the previous block's dV MMAs are out of the way
            *reinterpret_cast<uint4*>(smem + S::DST + (blk & 1) * 2 * TILE_BYTES + sw_off(row, qc)) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
          }
        }
        tc::fence_async_smem();
        if (tl && warp == 0) tl[blk * 8 + 2] = clock64();
        // P^T's TMEM columns belong to the previous block's dV MMAs until they complete
        if (blk > 0) { wait(bar_dv, (blk - 1) & 1, 49); tc::tc_fence_after(); }
        if (tl && warp == 0) tl[blk * 8 + 3] = clock64();
        tc::tmem_st16(t_pt + lane_addr + ch * 32, pw[0]);
        tc::tmem_st16(t_pt + lane_addr + ch * 32 + 16, pw[1]);
        tc::tmem_st_wait();

        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(bar_p);
        if (tl && warp == 0) tl[blk * 8 + 4] = clock64();
      }
    }
  } else if (warp < BWDF_E_WARPS + BWDF_D_WARPS) {
    // ---------------------------------------------------------------- 4 drain warps
    // dQ partial of (query block i, this key tile): TMEM -> bf16 -> its own tile of the partial buffer (a full 128-byte
    // row per thread; no atomics, the finishing kernel adds the key tiles' partials in a fixed order); after the last
    // block of a key tile also dK (scaled, RoPE backward) and dV.
    const int lg = warp & 3, row = lg * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
    const int npairs = nq * (nq + 1) / 2;
    uint8_t* stage = smem + S::DQS + lg * 4096;
    if (warp != BWDF_E_WARPS) tl = nullptr;
    int blk = 0;
    for (int item = 0;; item++) {
      const Item cur = item_at(item);
      if (!cur.valid) break;
      const int kt = cur.kt, b = cur.b, h = cur.h, row0 = cur.row0;
      const int krow = kt * 128 + row;
      const int n_it = nq - kt;
      for (int it = 0; it < n_it; it++, blk++) {
        const int i = kt + it;
        wait(&bar_d[blk & 1], (blk >> 1) & 1, 50);          // dV, dK, dQ MMAs of this block are complete
        tc::tc_fence_after();
        uint32_t r0[32], r1[32];
        tc::tmem_ld32(t_dq + lane_addr, r0);
        tc::tmem_ld32(t_dq + lane_addr + 32, r1);
        tc::tmem_ld_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(bar_dqf);
        // bf16 rows go through a swizzled staging tile and leave with ONE TMA store per warp: per-lane stores to 32
        // different lines would occupy the load/store unit that the element-wise warps need at the same moment
        if (lane == 0) tc::tma_wait_group_read<0>();      // the previous tile has been read out of the staging buffer
        __syncwarp();
        uint8_t* rowp = stage + lane * 128;
#pragma unroll
        for (int v = 0; v < 8; v++) {
          const uint32_t* src = (v < 4) ? &r0[v * 8] : &r1[(v - 4) * 8];
          uint4 pk;
          pk.x = pack_bf16(__uint_as_float(src[0]), __uint_as_float(src[1]));
          pk.y = pack_bf16(__uint_as_float(src[2]), __uint_as_float(src[3]));
          pk.z = pack_bf16(__uint_as_float(src[4]), __uint_as_float(src[5]));
          pk.w = pack_bf16(__uint_as_float(src[6]), __uint_as_float(src[7]));
          *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = pk;
        }
        tc::fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          tc::tma_store_2d(&tm_dq, stage, h * HD, (int)((((long)b * npairs + (i * (i + 1) / 2 + kt)) * 128) + lg * 32));
          tc::tma_commit_group();
        }
        if (tl && warp == BWDF_E_WARPS) tl[blk * 8 + 7] = clock64();
      }
      // the wait above covered the last block: dV and dK of this key tile are final
      {
        bf16* dk = a.out + ((size_t)(row0 + krow)) * 3 * C + C + h * HD;
        store_pairs_rope<HD>(dk, t_dk + lane_addr, 0, !*s_abort && krow < a.T, a.cosT, a.sinT, krow, a.scale);
        store_pairs_rope<HD>(dk + C, t_dv + lane_addr, 0, !*s_abort && krow < a.T, nullptr, nullptr, krow, 1.f);
      }
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(bar_epi);
    }
    if (lane == 0) tc::tma_wait_group<0>();     // every partial tile of this warp has been written
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == BWDF_CTRL_WARP) tc::tmem_dealloc(tmem, TMEM_COLS);
  if (dyn && tid == 0) attn_ctr_leave(1);
}

// dQ partial tiles -> bf16 Q slice of dqkv[rows, 3C]: sum over the key tiles kt <= i of query tile i (fp32, fixed
// order), times `scale`, optional RoPE backward.  One thread per (row, head, group of 16 rotation pairs); the partial
// layout is [B][i(i+1)/2 + kt][128][C] bf16.
__global__ void __launch_bounds__(256) attn_dq_finish_k(bf16* __restrict__ dqkv, const bf16* __restrict__ part, long rows, int T, int H,
                                                        int hd, float scale, const float* __restrict__ cosT,
                                                        const float* __restrict__ sinT) {
  mlb_pdl_sync();
  const int h2 = hd >> 1, gph = h2 >> 4, gpr = H * gph;   // groups of 16 pairs per head / per row
  // rows * gpr fits 31 bits (checked by the host): 32-bit index arithmetic
  const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (unsigned)rows * gpr) return;
  const unsigned r = idx / (unsigned)gpr;
  const int g = idx % (unsigned)gpr, h = g / gph, v = g % gph;
  const int t = r % (unsigned)T, C = H * hd;
  const long b = r / (unsigned)T;
  const int nq = (T + 127) / 128, npairs = nq * (nq + 1) / 2, i = t >> 7;
  const bf16* base = part + ((b * npairs + (long)i * (i + 1) / 2) * 128 + (t & 127)) * C + h * hd + v * 16;
  float x0[16], x1[16];
#pragma unroll
  for (int k = 0; k < 16; k++) { x0[k] = 0.f; x1[k] = 0.f; }
#pragma unroll 2
  for (int kt = 0; kt <= i; kt++) {
    const uint4* p0 = reinterpret_cast<const uint4*>(base + (long)kt * 128 * C);
    const uint4* p1 = reinterpret_cast<const uint4*>(base + (long)kt * 128 * C + h2);
    const uint4 a0 = __ldcs(p0), a1 = __ldcs(p0 + 1), b0 = __ldcs(p1), b1 = __ldcs(p1 + 1);
    const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int k = 0; k < 8; k++) {
      x0[2 * k] += __uint_as_float(wa[k] << 16); x0[2 * k + 1] += __uint_as_float(wa[k] & 0xffff0000u);
      x1[2 * k] += __uint_as_float(wb[k] << 16); x1[2 * k + 1] += __uint_as_float(wb[k] & 0xffff0000u);
    }
  }
#pragma unroll
  for (int k = 0; k < 16; k++) { x0[k] *= scale; x1[k] *= scale; }
  if (cosT) {
    const float4* c4 = reinterpret_cast<const float4*>(cosT + (long)t * h2 + v * 16);
    const float4* s4 = reinterpret_cast<const float4*>(sinT + (long)t * h2 + v * 16);
#pragma unroll
    for (int i4 = 0; i4 < 4; i4++) {
      const float4 c = c4[i4], sn = s4[i4];
      const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float d0 = x0[4 * i4 + k], d1 = x1[4 * i4 + k];
        x0[4 * i4 + k] = d0 * cc[k] + d1 * ss[k];
        x1[4 * i4 + k] = d1 * cc[k] - d0 * ss[k];
      }
    }
  }
  bf16* o0 = dqkv + (long)r * 3L * C + h * hd + v * 16;
#pragma unroll
  for (int i2 = 0; i2 < 2; i2++) {
    uint4 w0, w1;
    w0.x = pack_bf16(x0[8 * i2], x0[8 * i2 + 1]); w0.y = pack_bf16(x0[8 * i2 + 2], x0[8 * i2 + 3]);
    w0.z = pack_bf16(x0[8 * i2 + 4], x0[8 * i2 + 5]); w0.w = pack_bf16(x0[8 * i2 + 6], x0[8 * i2 + 7]);
    w1.x = pack_bf16(x1[8 * i2], x1[8 * i2 + 1]); w1.y = pack_bf16(x1[8 * i2 + 2], x1[8 * i2 + 3]);
    w1.z = pack_bf16(x1[8 * i2 + 4], x1[8 * i2 + 5]); w1.w = pack_bf16(x1[8 * i2 + 6], x1[8 * i2 + 7]);
    *reinterpret_cast<uint4*>(o0 + 8 * i2) = w0;
    *reinterpret_cast<uint4*>(o0 + h2 + 8 * i2) = w1;
  }
}

// ================================================================== backward: dQ (one CTA per 128-query tile)
template <int HD>
struct BwdQSmem {
  static constexpr int CH = HD / 64;
  static constexpr int NBUF = (HD == 64) ? 2 : 1;
  static constexpr int Q = 0;
  static constexpr int DO = Q + CH * TILE_BYTES;
  static constexpr int K = DO + CH * TILE_BYTES;               // NBUF
  static constexpr int V = K + NBUF * CH * TILE_BYTES;         // NBUF
  static constexpr int DS = V + NBUF * CH * TILE_BYTES;
  static constexpr int BAR = DS + 2 * TILE_BYTES;
  static constexpr int TOTAL = BAR + 128 + 1024;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_q_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv,
                                                                       const __grid_constant__ CUtensorMap tm_do,
                                                                       const AttnArgs a) {
  using S = BwdQSmem<HD>;
  constexpr int CH = HD / 64, NBUF = S::NBUF;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + S::BAR);
  uint64_t *bar_q = bars, *bar_kv = bars + 1 /*[2]*/, *bar_s = bars + 3, *bar_d = bars + 4;
  uint32_t* tmem_slot = (uint32_t*)(bars + 5);

  const int nq = (a.T + 127) / 128;
  const int qt = nq - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = qt * 128;
  const int C = a.H * HD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lg = warp & 3, cq = warp >> 2, row = lg * 32 + lane;
  const int row0 = b * a.T;

  if (tid == 0) {
    tc::mbar_init(bar_q, 1); tc::mbar_init(&bar_kv[0], 1); tc::mbar_init(&bar_kv[1], 1);
    tc::mbar_init(bar_s, 1); tc::mbar_init(bar_d, 1);
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tm_qkv);
    tc::tma_prefetch_desc(&tm_do);
  }
  if (warp == 0) tc::tmem_alloc(tmem_slot, TMEM_COLS);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dq = tmem + 256;
  const uint32_t lane_addr = (uint32_t)(lg * 32) << 16;
  constexpr uint32_t idesc_s = tc::idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_d = tc::idesc_bf16(128, HD, 0, 1);
  const uint32_t sQ = tc::smem_u32(smem + S::Q), sDO = tc::smem_u32(smem + S::DO), sDS = tc::smem_u32(smem + S::DS);

  auto load_kv = [&](int j, int buf) {
    tc::mbar_expect_tx(&bar_kv[buf], 2 * CH * TILE_BYTES);
    for (int c = 0; c < CH; c++) {
      tc::tma_load_2d(smem + S::K + (buf * CH + c) * TILE_BYTES, &tm_qkv, &bar_kv[buf], C + h * HD + c * 64, row0 + j * 128);
      tc::tma_load_2d(smem + S::V + (buf * CH + c) * TILE_BYTES, &tm_qkv, &bar_kv[buf], 2 * C + h * HD + c * 64, row0 + j * 128);
    }
  };
  auto issue_scores = [&](int buf) {   // S = Q K^T and dP = dO V^T for the key block in `buf`
    const uint32_t sK = tc::smem_u32(smem + S::K + buf * CH * TILE_BYTES), sV = tc::smem_u32(smem + S::V + buf * CH * TILE_BYTES);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(t_s, desc_k(sQ, ks), desc_k(sK, ks), idesc_s, ks > 0);
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) tc::mma_bf16_ss(t_dp, desc_k(sDO, ks), desc_k(sV, ks), idesc_s, ks > 0);
  };
  const int nkb = qt + 1;
  if (tid == 0) {
    tc::mbar_expect_tx(bar_q, 2 * CH * TILE_BYTES);
    for (int c = 0; c < CH; c++) {
      tc::tma_load_2d(smem + S::Q + c * TILE_BYTES, &tm_qkv, bar_q, h * HD + c * 64, row0 + q0);
      tc::tma_load_2d(smem + S::DO + c * TILE_BYTES, &tm_do, bar_q, h * HD + c * 64, row0 + q0);
    }
    load_kv(0, 0);
    if (tc::mbar_wait(bar_q, 0, 30) && tc::mbar_wait(&bar_kv[0], 0, 31)) {
      tc::tc_fence_after();
      issue_scores(0);
    }
    tc::mma_commit(bar_s);
  }
  const float sl2 = a.scale * LOG2E;
  const int qrow = q0 + row;
  const size_t si = ((size_t)b * a.H + h) * a.T + qrow;
  const float lse2 = (qrow < a.T) ? a.lse[si] * LOG2E : INFINITY;
  const float delta = (qrow < a.T) ? a.delta[si] : 0.f;
  bool ok = true;
  for (int j = 0; j < nkb; j++) {
    const int buf = (NBUF == 2) ? (j & 1) : 0;
    const int k0 = j * 128;
    if (!tc::mbar_wait(bar_s, j & 1, 32)) { ok = false; break; }
    tc::tc_fence_after();
    if (NBUF == 2 && tid == 0 && j + 1 < nkb) load_kv(j + 1, buf ^ 1);
    const bool diag = (j == qt);
    {
      uint32_t rs[32], rd[32];
      tc::tmem_ld32(t_s + lane_addr + cq * 32, rs);
      tc::tmem_ld32(t_dp + lane_addr + cq * 32, rd);
      tc::tmem_ld_wait();
#pragma unroll
      for (int v8 = 0; v8 < 4; v8++) {
        float ds[8];
#pragma unroll
        for (int x = 0; x < 8; x++) {
          const int kcol = k0 + cq * 32 + v8 * 8 + x;
          float pv = exp2f(__uint_as_float(rs[v8 * 8 + x]) * sl2 - lse2);
          if (diag && kcol > qrow) pv = 0.f;
          ds[x] = pv * (__uint_as_float(rd[v8 * 8 + x]) - delta) * a.scale;
        }
        uint4 dk;
        dk.x = pack_bf16(ds[0], ds[1]); dk.y = pack_bf16(ds[2], ds[3]); dk.z = pack_bf16(ds[4], ds[5]); dk.w = pack_bf16(ds[6], ds[7]);
        *reinterpret_cast<uint4*>(smem + S::DS + sw_off(row, cq * 32 + v8 * 8)) = dk;
      }
    }
    tc::fence_async_smem();
    tc::tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc::tc_fence_after();
      const uint32_t sK = tc::smem_u32(smem + S::K + buf * CH * TILE_BYTES);
#pragma unroll
      for (int ks = 0; ks < 8; ks++) tc::mma_bf16_ss(t_dq, desc_k(sDS, ks), desc_mn(sK, ks), idesc_d, (j > 0 || ks > 0));
      if (j + 1 < nkb) {
        bool ready = true;
        if (NBUF == 1) {
          tc::mma_commit(bar_d);
          ready = tc::mbar_wait(bar_d, j & 1, 33);
          if (ready) load_kv(j + 1, 0);
        }
        const int nb = (NBUF == 2) ? (buf ^ 1) : 0;
        const int nphase = (NBUF == 2) ? (((j + 1) >> 1) & 1) : ((j + 1) & 1);
        if (ready && tc::mbar_wait(&bar_kv[nb], nphase, 34)) {
          tc::tc_fence_after();
          issue_scores(nb);
        }
      }
      tc::mma_commit(bar_s);
    }
  }
  if (ok) ok = tc::mbar_wait(bar_s, nkb & 1, 35);
  tc::tc_fence_after();
  if (ok && cq < HD / 64) {
    bf16* dst = a.out + ((size_t)(row0 + qrow)) * 3 * C + h * HD;
    store_pairs_rope<HD>(dst, t_dq + lane_addr, cq * 32, qrow < a.T, a.cosT, a.sinT, qrow);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, TMEM_COLS);
}

// ================================================================== SIMT fallback (any head size <= 256, any T)
// One block per (query row, head, sample); scores kept in shared memory.
// `last` = index of the last key a query sees: the query's own position (causal) or T - 1 (bidirectional, the vision
// encoder's attention).
__global__ void attn_fwd_simt_k(bf16* __restrict__ out, float* __restrict__ lse, const bf16* __restrict__ qkv, int B, int T, int H,
                                int hd, float scale, int causal = 1) {
  extern __shared__ float sc[];  // T scores + 32 reduce
  float* red = sc + T;
  const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, C = H * hd;
  const int last = causal ? i : T - 1;
  const bf16* q = qkv + ((size_t)(b * T + i)) * 3 * C + h * hd;
  float mx = -INFINITY;
  for (int j = threadIdx.x; j <= last; j += blockDim.x) {
    const bf16* k = qkv + ((size_t)(b * T + j)) * 3 * C + C + h * hd;
    float s = 0.f;
    for (int d = 0; d < hd; d++) s += __bfloat162float(q[d]) * __bfloat162float(k[d]);
    s *= scale;
    sc[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int j = threadIdx.x; j <= last; j += blockDim.x) { float p = __expf(sc[j] - mx); sc[j] = p; sum += p; }
  sum = block_sum(sum, red);
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j <= last; j++) acc += sc[j] * __bfloat162float(qkv[((size_t)(b * T + j)) * 3 * C + 2 * C + h * hd + d]);
    out[((size_t)(b * T + i)) * C + h * hd + d] = __float2bfloat16(acc / sum);
  }
  if (threadIdx.x == 0) lse[((size_t)b * H + h) * T + i] = mx + __logf(sum);
}
// dQ for query i.
__global__ void attn_bwd_q_simt_k(bf16* __restrict__ dqkv, const bf16* __restrict__ dout, const bf16* __restrict__ qkv,
                                  const float* __restrict__ lse, const float* __restrict__ delta, int B, int T, int H, int hd,
                                  float scale, int causal = 1) {
  extern __shared__ float sc[];
  const int i = blockIdx.x, h = blockIdx.y, b = blockIdx.z, C = H * hd;
  const int last = causal ? i : T - 1;
  const bf16* q = qkv + ((size_t)(b * T + i)) * 3 * C + h * hd;
  const bf16* dO = dout + ((size_t)(b * T + i)) * C + h * hd;
  const float L = lse[((size_t)b * H + h) * T + i], D = delta[((size_t)b * H + h) * T + i];
  for (int j = threadIdx.x; j <= last; j += blockDim.x) {
    const bf16* k = qkv + ((size_t)(b * T + j)) * 3 * C + C + h * hd;
    const bf16* v = k + C;
    float s = 0.f, dp = 0.f;
    for (int d = 0; d < hd; d++) {
      s += __bfloat162float(q[d]) * __bfloat162float(k[d]);
      dp += __bfloat162float(dO[d]) * __bfloat162float(v[d]);
    }
    sc[j] = __expf(s * scale - L) * (dp - D) * scale;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j <= last; j++) acc += sc[j] * __bfloat162float(qkv[((size_t)(b * T + j)) * 3 * C + C + h * hd + d]);
    dqkv[((size_t)(b * T + i)) * 3 * C + h * hd + d] = __float2bfloat16(acc);
  }
}
// dK, dV for key j.
__global__ void attn_bwd_kv_simt_k(bf16* __restrict__ dqkv, const bf16* __restrict__ dout, const bf16* __restrict__ qkv,
                                   const float* __restrict__ lse, const float* __restrict__ delta, int B, int T, int H, int hd,
                                   float scale, int causal = 1) {
  extern __shared__ float sc[];  // p[T], ds[T]
  float* sp = sc;
  float* sds = sc + T;
  const int j = blockIdx.x, h = blockIdx.y, b = blockIdx.z, C = H * hd;
  const int first = causal ? j : 0;      // first query that sees key j
  const bf16* k = qkv + ((size_t)(b * T + j)) * 3 * C + C + h * hd;
  const bf16* v = k + C;
  for (int i = first + threadIdx.x; i < T; i += blockDim.x) {
    const bf16* q = qkv + ((size_t)(b * T + i)) * 3 * C + h * hd;
    const bf16* dO = dout + ((size_t)(b * T + i)) * C + h * hd;
    float s = 0.f, dp = 0.f;
    for (int d = 0; d < hd; d++) {
      s += __bfloat162float(q[d]) * __bfloat162float(k[d]);
      dp += __bfloat162float(dO[d]) * __bfloat162float(v[d]);
    }
    const size_t si = ((size_t)b * H + h) * T + i;
    const float p = __expf(s * scale - lse[si]);
    sp[i] = p;
    sds[i] = p * (dp - delta[si]) * scale;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float dk = 0.f, dv = 0.f;
    for (int i = first; i < T; i++) {
      dk += sds[i] * __bfloat162float(qkv[((size_t)(b * T + i)) * 3 * C + h * hd + d]);
      dv += sp[i] * __bfloat162float(dout[((size_t)(b * T + i)) * C + h * hd + d]);
    }
    dqkv[((size_t)(b * T + j)) * 3 * C + C + h * hd + d] = __float2bfloat16(dk);
    dqkv[((size_t)(b * T + j)) * 3 * C + 2 * C + h * hd + d] = __float2bfloat16(dv);
  }
}

int g_attn_force_simt = 0;
int g_attn_dynamic = 0;
int g_fwd_rows = 3;   // head size 64: 1 / 2 / 3 = thread-per-row forward over tile pairs (variants at the launch), 0 = four-threads-per-row forward

template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

bool tc_ok(const void* qkv, const void* other, int H, int hd) {
  const int C = H * hd;
  return !g_attn_force_simt && (hd == 64 || hd == 128) && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)other % 16 == 0) && (C % 8 == 0);
}

}  // namespace

static long long* g_timeline = nullptr;
MLB_API void mlb_attn_force_simt(int on) { g_attn_force_simt = on; }
MLB_API void mlb_attn_fwd_mode(int rows) { g_fwd_rows = rows; }
// 1: the persistent attention kernels draw their work items from a device counter (see ItemRing); 0: host-built table
MLB_API void mlb_attn_dynamic(int on) { g_attn_dynamic = on; }
// Diagnostic: device buffer of at least 8 * (query blocks per CTA) int64 that CTA (0,0,0) of the fused backward fills
// with SM cycle stamps, eight per block: element-wise warp 0 before / after the score wait, after its exponentials,
// after the previous block's MMAs completed, after P^T / dS^T are stored; control thread when it saw P^T and when the
// block's MMAs were issued; first drain warp when the dQ partial was stored.  nullptr switches it off.
MLB_API void mlb_attn_set_timeline(void* buf) { g_timeline = (long long*)buf; }

// Balanced static schedules for the persistent attention kernels.  Work items (forward: pair p of a (sample, head);
// backward: key tile kt of a (sample, head); both numbered so that the cost falls with the item number; cost = the item's
// 128x128 blocks plus a fixed part for loads, pipeline refill and epilogue) go one by one to the CTA with the least work
// so far.  Forward, B=16 H=12 T=1024, 148 CTAs: round robin leaves the slowest CTA with 30 key-block steps where the
// average is 26, this assignment gets 26.  Backward: 768 equal CTAs of 9 blocks each ran as 5.2 waves (54 blocks on the
// slowest SM); 1536 single-tile items scheduled this way give 47.  The table lives in device memory, one row of `stride`
// entries per CTA, -1 terminated (with room for a look-ahead of two items), cached per shape; it is built with a
// blocking copy, so while the stream is being captured into a graph and the shape is new, nullptr is returned and the
// kernels fall back to round robin.
struct AttnSchedule { int kind, dev, B, H, T, grid, stride; int* table; };
static std::mutex g_sched_mu;
static std::vector<AttnSchedule> g_sched;
static int g_fwd_balance = 1;
MLB_API void mlb_attn_fwd_balance(int on) { g_fwd_balance = on; }   // (both directions)
static const int* attn_schedule(int kind /*0 forward pairs, 1 backward key tiles*/, int B, int H, int T, int grid, int* stride_out,
                                cudaStream_t st) {
  if (!g_fwd_balance) return nullptr;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(g_sched_mu);
  for (const AttnSchedule& e : g_sched)
    if (e.kind == kind && e.dev == dev && e.B == B && e.H == H && e.T == T && e.grid == grid) { *stride_out = e.stride; return e.table; }
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return nullptr;
  const int nq = (T + 127) / 128, npair = (nq + 1) / 2, BH = B * H;
  const int total = (kind == 0 ? npair : nq) * BH;
  std::vector<std::vector<int>> rows(grid);
  using Bin = std::pair<long, int>;     // (work so far in quarter blocks, CTA)
  std::priority_queue<Bin, std::vector<Bin>, std::greater<Bin>> heap;
  for (int c = 0; c < grid; c++) heap.push({0, c});
  for (int w = 0; w < total; w++) {     // items are in descending cost order by construction
    long cost;
    if (kind == 0) cost = 4L * std::min(2 * (npair - 1 - w / BH) + 2, nq) + 2;
    else cost = 4L * (nq - w / BH) + 3;
    Bin b = heap.top();
    heap.pop();
    rows[b.second].push_back(w);
    heap.push({b.first + cost, b.second});
  }
  size_t longest = 0;
  for (const auto& r : rows) longest = std::max(longest, r.size());
  const int stride = (int)longest + 3;
  std::vector<int> host((size_t)grid * stride, -1);
  for (int c = 0; c < grid; c++) std::copy(rows[c].begin(), rows[c].end(), host.begin() + (size_t)c * stride);
  int* table = nullptr;
  if (cudaMalloc(&table, host.size() * sizeof(int)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (cudaMemcpy(table, host.data(), host.size() * sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(table);
    return nullptr;
  }
  g_sched.push_back({kind, dev, B, H, T, grid, stride, table});
  *stride_out = stride;
  return table;
}

// out[B,T,C], lse[B,H,T] from qkv[B,T,3C].
MLB_API int mlb_attn_fwd(void* out, float* lse, const void* qkv, int B, int T, int H, int hd, cudaStream_t st) {
  const int C = H * hd;
  const float scale = 1.0f / sqrtf((float)hd);
  if (tc_ok(qkv, out, H, hd)) {
    const CUtensorMap* tm = mlb_tmap_cached(qkv, (uint64_t)B * T, 3 * C, 3 * C, 128, 64);
    if (!tm) return -2;
    AttnArgs a{B, T, H, hd, scale, (bf16*)out, lse, nullptr, nullptr, nullptr, nullptr, g_fwd_rows, g_timeline};
    const long items = (long)((T + 127) / 128) * H * B;
    int sms = 0, devid = 0;
    cudaGetDevice(&devid);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, devid);
    if (sms <= 0) sms = 148;
    dim3 grid((unsigned)(items < sms ? items : sms));   // persistent: one CTA per SM walks its share of the tiles
    if (hd == 64 && g_fwd_rows) {
      // mode 1: O folded into registers every block; 2: O accumulated in TMEM, rescaled only when a row maximum grows by
      // more than 2^8; 3: as 2 with the row maximum tracked inside the exponential pass (one pass per key block)
      const long pairs = (long)(((T + 127) / 128 + 1) / 2) * H * B;
      const dim3 grid2((unsigned)(pairs < sms ? pairs : sms));
      a.dynamic = (g_attn_dynamic && g_fwd_rows != 1 && g_fwd_rows != 2) ? 1 : 0;      // (the default variant only)
      a.sched = (pairs > sms && !a.dynamic) ? attn_schedule(0, B, H, T, (int)grid2.x, &a.sched_stride, st) : nullptr;
      const CUtensorMap* to = (T % 128 == 0 && g_fwd_rows >= 2) ? mlb_tmap_cached(out, (uint64_t)B * T, C, C, 32, 64, 2) : nullptr;
      a.out_tma = to != nullptr;
      if (!to) to = tm;      // unused by the kernel then
#define MLB_FWD2(MODE)                                                                                                             \
  {                                                                                                                            \
    static int once = set_smem(attn_fwd_rows_tc_kernel<MODE>, Fwd2Smem::TOTAL);                                          \
    (void)once;                                                                                                                \
    mlb_launch_tmem(attn_fwd_rows_tc_kernel<MODE>, grid2, dim3(FWD2_THREADS), Fwd2Smem::TOTAL, st, *tm, *to, a);              \
  }
      if (a.dynamic && g_fwd_rows != 1 && g_fwd_rows != 2) {
        static int once = set_smem(attn_fwd_rows_tc_kernel<3, true>, Fwd2Smem::TOTAL);
        (void)once;
        mlb_launch_tmem(attn_fwd_rows_tc_kernel<3, true>, grid2, dim3(FWD2_THREADS), Fwd2Smem::TOTAL, st, *tm, *to, a);
      } else {
        switch (g_fwd_rows) {
          case 1: MLB_FWD2(1) break;
          case 2: MLB_FWD2(2) break;
          default: MLB_FWD2(3) break;
        }
      }
#undef MLB_FWD2
    } else if (hd == 64) {
      static int once = set_smem(attn_fwd_tc_kernel<64>, FwdSmem<64>::TOTAL);
      (void)once;
      attn_fwd_tc_kernel<64><<<grid, ATT_THREADS, FwdSmem<64>::TOTAL, st>>>(*tm, a);
    } else {
      static int once = set_smem(attn_fwd_tc_kernel<128>, FwdSmem<128>::TOTAL);
      (void)once;
      attn_fwd_tc_kernel<128><<<grid, ATT_THREADS, FwdSmem<128>::TOTAL, st>>>(*tm, a);
    }
    return (int)cudaGetLastError();
  }
  if (hd > 256) return -4;
  attn_fwd_simt_k<<<dim3(T, H, B), 128, (T + 32) * sizeof(float), st>>>((bf16*)out, lse, (const bf16*)qkv, B, T, H, hd, scale);
  return (int)cudaGetLastError();
}

// Bidirectional (no causal mask) attention for short sequences such as a vision encoder's patch tokens: the scalar
// kernels, any T and head size <= 256.  Same layouts as mlb_attn_fwd / mlb_attn_bwd; delta is scratch of B*H*T floats.
MLB_API int mlb_attn_bidir_fwd(void* out, float* lse, const void* qkv, int B, int T, int H, int hd, cudaStream_t st) {
  if (hd > 256 || (size_t)(T + 32) * sizeof(float) > 48 * 1024) return -4;
  attn_fwd_simt_k<<<dim3(T, H, B), 128, (T + 32) * sizeof(float), st>>>((bf16*)out, lse, (const bf16*)qkv, B, T, H, hd, 1.0f / sqrtf((float)hd), 0);
  return (int)cudaGetLastError();
}
MLB_API int mlb_attn_bidir_bwd(void* dqkv, const void* dout, const void* qkv, const void* out, const float* lse, float* delta, int B, int T,
                               int H, int hd, cudaStream_t st) {
  if (hd > 256 || (size_t)2 * T * sizeof(float) > 48 * 1024) return -4;
  const float scale = 1.0f / sqrtf((float)hd);
  const long heads = (long)B * T * H;
  attn_delta_scalar_k<<<(unsigned)((heads * 32 + 255) / 256), 256, 0, st>>>(delta, (const bf16*)dout, (const bf16*)out, B, T, H, hd);
  attn_bwd_q_simt_k<<<dim3(T, H, B), 128, T * sizeof(float), st>>>((bf16*)dqkv, (const bf16*)dout, (const bf16*)qkv, lse, delta, B, T, H, hd, scale, 0);
  attn_bwd_kv_simt_k<<<dim3(T, H, B), 128, 2 * T * sizeof(float), st>>>((bf16*)dqkv, (const bf16*)dout, (const bf16*)qkv, lse, delta, B, T, H, hd, scale, 0);
  return (int)cudaGetLastError();
}

// Bytes of dQ-partial scratch the fused backward needs for this shape (0: no fused backward for it).
MLB_API long mlb_attn_bwd_scratch_bytes(int B, int T, int H, int hd) {
  if (hd != 64) return 0;
  const long nq = (T + 127) / 128;
  return (long)B * (nq * (nq + 1) / 2) * 128 * H * hd * 2;
}

// dqkv[B,T,3C] from dout[B,T,C], qkv, out, lse.  `delta` is scratch of B*H*T floats.  `dq_part` (optional) is scratch of
// mlb_attn_bwd_scratch_bytes() bytes whose contents do not matter: with it and head size 64 the fused
// single-kernel backward runs; without it the two-kernel backward (dK/dV kernel + dQ kernel) runs.  If cosT/sinT are given, RoPE's
// backward rotation is applied to dQ and dK before they are stored (tensor-core path only; returns 1 if it was applied,
// 0 if the caller still has to rotate, <0 or a CUDA error code > 1 on failure).
// have_delta != 0: `delta` already holds rowsum(dO * O) per (sample, head, query) - written by the epilogue of the GEMM
// that produced dO (mlb_linear_dx_delta) - and the pass over dO and O is skipped.
static int attn_bwd_impl(void* dqkv, const void* dout, const void* qkv, const void* out, const float* lse, float* delta, void* dq_part,
                         int B, int T, int H, int hd, const float* cosT, const float* sinT, int have_delta, cudaStream_t st);
MLB_API int mlb_attn_bwd(void* dqkv, const void* dout, const void* qkv, const void* out, const float* lse, float* delta, void* dq_part,
                         int B, int T, int H, int hd, const float* cosT, const float* sinT, cudaStream_t st) {
  return attn_bwd_impl(dqkv, dout, qkv, out, lse, delta, dq_part, B, T, H, hd, cosT, sinT, 0, st);
}
MLB_API int mlb_attn_bwd_have_delta(void* dqkv, const void* dout, const void* qkv, const void* out, const float* lse, float* delta,
                                    void* dq_part, int B, int T, int H, int hd, const float* cosT, const float* sinT, cudaStream_t st) {
  return attn_bwd_impl(dqkv, dout, qkv, out, lse, delta, dq_part, B, T, H, hd, cosT, sinT, 1, st);
}
static int attn_bwd_impl(void* dqkv, const void* dout, const void* qkv, const void* out, const float* lse, float* delta, void* dq_part,
                         int B, int T, int H, int hd, const float* cosT, const float* sinT, int have_delta, cudaStream_t st) {
  const int C = H * hd;
  const float scale = 1.0f / sqrtf((float)hd);
  if (!have_delta) {
    const long heads = (long)B * T * H;
    const int gsz = hd / 8;
    const bool vec = (hd % 8 == 0) && heads * gsz < (1L << 31) && gsz <= 32 && (gsz & (gsz - 1)) == 0 && ((uintptr_t)dout % 16 == 0) && ((uintptr_t)out % 16 == 0);
    if (vec) mlb_launch(attn_delta_k, dim3((unsigned)((heads * gsz + 255) / 256)), dim3(256), 0, st, delta, (const bf16*)dout, (const bf16*)out, B, T, H, hd);
    else attn_delta_scalar_k<<<(unsigned)((heads * 32 + 255) / 256), 256, 0, st>>>(delta, (const bf16*)dout, (const bf16*)out, B, T, H, hd);
  }
  if (tc_ok(qkv, dout, H, hd) && ((uintptr_t)dqkv % 16 == 0)) {
    const CUtensorMap* tq = mlb_tmap_cached(qkv, (uint64_t)B * T, 3 * C, 3 * C, 128, 64);
    const CUtensorMap* td = mlb_tmap_cached(dout, (uint64_t)B * T, C, C, 128, 64);
    if (!tq || !td) return -2;
    AttnArgs a{B, T, H, hd, scale, (bf16*)dqkv, const_cast<float*>(lse), delta, cosT, sinT, (bf16*)dq_part, 0, g_timeline};
    dim3 grid((T + 127) / 128, H, B);
    if (hd == 64 && dq_part != nullptr && ((uintptr_t)dq_part % 16 == 0) && (long)B * T * H * (hd / 32) < (1L << 31)) {
      // single fused kernel + dQ finish; the partial buffer is [B * nq(nq+1)/2 * 128 rows, C] bf16
      const long nqh = (T + 127) / 128;
      const CUtensorMap* tpart = mlb_tmap_cached(dq_part, (uint64_t)B * (nqh * (nqh + 1) / 2) * 128, C, C, 32, 64, 2);
      if (!tpart) return -2;
      static int o0 = set_smem(attn_bwd_fused_tc_kernel<false>, BwdFusedSmem::TOTAL);
      static int o1 = set_smem(attn_bwd_fused_tc_kernel<true>, BwdFusedSmem::TOTAL);
      (void)o0; (void)o1;
      // persistent CTAs, one per SM, over the (key tile, sample, head) items
      int sms = 0, devid = 0;
      cudaGetDevice(&devid);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, devid);
      if (sms <= 0) sms = 148;
      const long n_items = nqh * H * B;
      dim3 grid_f((unsigned)(n_items < sms ? n_items : sms));
      a.dynamic = g_attn_dynamic;
      a.sched = (n_items > sms && !a.dynamic) ? attn_schedule(1, B, H, T, (int)grid_f.x, &a.sched_stride, st) : nullptr;
      if (a.dynamic) mlb_launch_tmem(attn_bwd_fused_tc_kernel<true>, grid_f, dim3(BWDF_THREADS), BwdFusedSmem::TOTAL, st, *tq, *td, *tpart, a);
      else mlb_launch_tmem(attn_bwd_fused_tc_kernel<false>, grid_f, dim3(BWDF_THREADS), BwdFusedSmem::TOTAL, st, *tq, *td, *tpart, a);
      const long groups = (long)B * T * H * (hd / 32);
      mlb_launch(attn_dq_finish_k, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, st, (bf16*)dqkv, (const bf16*)dq_part, (long)B * T, T, H, hd, scale, cosT, sinT);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return (int)e + 1000;
      return cosT ? 1 : 0;
    }
    if (hd == 64) {
      static int o1 = set_smem(attn_bwd_kv_tc_kernel<64>, BwdKVSmem<64>::TOTAL);
      static int o2 = set_smem(attn_bwd_q_tc_kernel<64>, BwdQSmem<64>::TOTAL);
      (void)o1; (void)o2;
      attn_bwd_kv_tc_kernel<64><<<grid, BWD_THREADS, BwdKVSmem<64>::TOTAL, st>>>(*tq, *td, a);
      attn_bwd_q_tc_kernel<64><<<grid, BWD_THREADS, BwdQSmem<64>::TOTAL, st>>>(*tq, *td, a);
    } else {
      static int o1 = set_smem(attn_bwd_kv_tc_kernel<128>, BwdKVSmem<128>::TOTAL);
      static int o2 = set_smem(attn_bwd_q_tc_kernel<128>, BwdQSmem<128>::TOTAL);
      (void)o1; (void)o2;
      attn_bwd_kv_tc_kernel<128><<<grid, BWD_THREADS, BwdKVSmem<128>::TOTAL, st>>>(*tq, *td, a);
      attn_bwd_q_tc_kernel<128><<<grid, BWD_THREADS, BwdQSmem<128>::TOTAL, st>>>(*tq, *td, a);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e + 1000;
    return cosT ? 1 : 0;
  }
  if (hd > 256) return -4;
  attn_bwd_q_simt_k<<<dim3(T, H, B), 128, T * sizeof(float), st>>>((bf16*)dqkv, (const bf16*)dout, (const bf16*)qkv, lse, delta, B, T, H,
                                                                  hd, scale);
  attn_bwd_kv_simt_k<<<dim3(T, H, B), 128, 2 * T * sizeof(float), st>>>((bf16*)dqkv, (const bf16*)dout, (const bf16*)qkv, lse, delta, B,
                                                                       T, H, hd, scale);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e + 1000;
  return 0;
}
