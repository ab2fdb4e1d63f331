// In-kernel collectives over NVLink peer memory, fused with the optimizer.
//
// ddp_bucket_kernel replaces, for one gradient bucket, the reference's chain
//     cast_f2b -> ncclAllReduce -> cast_b2f_scale -> adamw           (train/gpt.cu:310-328, :348-367)
// with ONE kernel and no library collective.  Every rank runs it on the same bucket:
//   1. entry barrier: flags in every peer's symmetric flag array tell that the peer's gradients of this bucket are final;
//   2. this rank owns 1/world of the bucket: it loads that shard of the fp32 gradients from every rank's buffer
//      (plain peer loads over NVLink/NVSwitch), sums them in fp32 in rank order (deterministic, tighter than a bf16
//      all-reduce), applies the 1/(world*accum) mean and the AdamW update to its shard of master / m / v, and stores the
//      new bf16 parameters into every rank's parameter buffer (peer stores);
//   3. exit barrier: the last CTA to finish signals every peer and waits for their signals, so when the kernel ends all
//      peers have stopped reading this rank's gradients and this rank's parameters are complete.
// The same kernel with world = 1 is a fused mean-scale + AdamW.  Reduce-scatter + sharded AdamW for ZeRO-style
// sharding is the same kernel with `bcast` = 0 (parameters stay sharded).
// Every wait on a peer flag is bounded (the caller passes the limit; the engine's default is 20 s, tests pass a fraction
// of a second): on expiry the kernel records MLB_ERR_FLAG_TIMEOUT and returns.
#include "../common.cuh"

MLB_DEFINE_ERROR_WORD(comm)

namespace {

constexpr int MAX_WORLD = 16;

struct BucketArgs {
  float* const* grads;       // device array [world]: base of each rank's flat fp32 gradient buffer
  bf16* const* params;       // device array [world]: base of each rank's flat bf16 parameter buffer
  int* const* flags;         // device array [world]: base of each rank's flag array: [2][max_buckets][MAX_WORLD] ints
  float* master;
  float* m;
  float* v;
  int* done_counter;         // local, 2 * max_buckets ints, 0 between launches: [bucket] CTAs that finished the update,
                             // [max_buckets + bucket] CTAs that finished the bf16 staging copy
  int* epoch_ctr;            // local, one int per bucket: number of completed launches.  The epoch of a launch is
                             // epoch_ctr[bucket] + 1, read from memory so that a replayed CUDA graph advances it.
  long off, n;               // bucket range in elements
  int rank, world, bucket, max_buckets, bcast;
  float lr, b1, b2, eps, wd, inv_bc1, inv_bc2, scale;
  const float* dev_hyper;    // optional {lr, 1/bc1, 1/bc2, scale} in device memory (CUDA-graph replay)
  float* grads_mc;           // optional NVLS multicast address of the gradient buffers: the switch sums all ranks' values
  bf16* params_mc;           // optional NVLS multicast address of the parameter buffers: one store reaches every rank
  bf16* const* gstage;       // bf16 reduction: device array [world] of the ranks' bf16 staging copies of the gradients
  bf16* gstage_mc;           // ... and their multicast address
  long spin_limit_ns;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {   // system-scope relaxed load: never served from a stale L1 line
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits until *flag >= epoch.  Returns false (after recording the error) if that takes longer than limit_ns.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, long limit_ns, int detail) {
  if (ld_acquire_sys(flag) >= epoch) return true;
  const uint64_t t0 = gtimer();
  for (;;) {
    for (int i = 0; i < 64; i++) {
      if (ld_acquire_sys(flag) >= epoch) return true;
      __nanosleep(100);
    }
    if ((long)(gtimer() - t0) > limit_ns) {
      mlb_set_error(MLB_ERR_FLAG_TIMEOUT, detail);
      return false;
    }
  }
}

// Gradient source of the reduction:
//   GM_F32_PEER  fp32 gradients, one plain peer load per rank, summed in rank order (deterministic, exact mean)
//   GM_F32_MC    fp32 gradients through the NVLink multicast address: the switch returns the sum over all ranks
//   GM_BF16_PEER bf16 staging copies (written by phase 0 of this kernel), peer loads, fp32 accumulation
//   GM_BF16_MC   bf16 staging copies through the multicast address, fp32 accumulation inside the switch
enum { GM_F32_PEER = 0, GM_F32_MC = 1, GM_BF16_PEER = 2, GM_BF16_MC = 3 };

__device__ __forceinline__ uint4 ld_peer_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void acc_bf16x2(float& a, float& b, uint32_t u) {
  a += __uint_as_float(u << 16);
  b += __uint_as_float(u & 0xffff0000u);
}

// 4 consecutive gradient elements starting at absolute element e (e % 4 == 0), summed over the ranks.
template <int GM>
__device__ __forceinline__ float4 load_grad_sum4(const BucketArgs& a, long e, int W) {
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
  if (GM == GM_F32_MC) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(g.x), "=f"(g.y), "=f"(g.z), "=f"(g.w) : "l"(a.grads_mc + e) : "memory");
  } else if (GM == GM_F32_PEER) {
#pragma unroll 4
    for (int w = 0; w < W; w++) {
      const float4 t = ld_peer_f4(a.grads[w] + e);
      g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
    }
  }
  return g;
}
// 8 consecutive gradient elements (e % 8 == 0) from the bf16 staging copies.
template <int GM>
__device__ __forceinline__ void load_grad_sum8(const BucketArgs& a, long e, int W, float (&g)[8]) {
#pragma unroll
  for (int j = 0; j < 8; j++) g[j] = 0.f;
  if (GM == GM_BF16_MC) {
    uint4 u;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(a.gstage_mc + e) : "memory");
    acc_bf16x2(g[0], g[1], u.x); acc_bf16x2(g[2], g[3], u.y); acc_bf16x2(g[4], g[5], u.z); acc_bf16x2(g[6], g[7], u.w);
  } else {
#pragma unroll 4
    for (int w = 0; w < W; w++) {
      const uint4 u = ld_peer_u4(a.gstage[w] + e);
      acc_bf16x2(g[0], g[1], u.x); acc_bf16x2(g[2], g[3], u.y); acc_bf16x2(g[4], g[5], u.z); acc_bf16x2(g[6], g[7], u.w);
    }
  }
}

// AdamW on 4 elements at e; writes master / m / v and returns the packed bf16 parameters.
__device__ __forceinline__ uint2 adamw4(const BucketArgs& a, long e, const float* g, float lr, float inv_bc1, float inv_bc2, float scale) {
  float4 mm = *reinterpret_cast<const float4*>(a.m + e);
  float4 vv = *reinterpret_cast<const float4*>(a.v + e);
  float4 p = *reinterpret_cast<const float4*>(a.master + e);
  float* mp = &mm.x; float* vp = &vv.x; float* pp = &p.x;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const float gj = g[j] * scale;
    mp[j] = a.b1 * mp[j] + (1.f - a.b1) * gj;
    vp[j] = a.b2 * vp[j] + (1.f - a.b2) * gj * gj;
    pp[j] -= lr * (mp[j] * inv_bc1 / (sqrtf(vp[j] * inv_bc2) + a.eps) + a.wd * pp[j]);
  }
  *reinterpret_cast<float4*>(a.m + e) = mm;
  *reinterpret_cast<float4*>(a.v + e) = vv;
  *reinterpret_cast<float4*>(a.master + e) = p;
  uint2 o;
  o.x = pack_bf16(p.x, p.y);
  o.y = pack_bf16(p.z, p.w);
  return o;
}
__device__ __forceinline__ void store_params4(const BucketArgs& a, long e, uint2 o, int W) {
  if (a.bcast && a.params_mc) {
    asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(a.params_mc + e), "r"(o.x), "r"(o.y) : "memory");
  } else if (a.bcast) {
#pragma unroll 4
    for (int w = 0; w < W; w++) *reinterpret_cast<uint2*>(a.params[w] + e) = o;
  } else {
    *reinterpret_cast<uint2*>(a.params[a.rank] + e) = o;
  }
}

// Lean form: 128 threads and at most 32 registers per thread, no shared memory.  That is one warp per SM sub-partition
// with 1 K registers each, which is what a resident CTA of the persistent tensor-core kernels (GEMM, attention: capped
// at 160 / 120 registers for this purpose) leaves free; so bucket kernels launched behind backward on a second stream
// share SMs with those kernels instead of keeping whole SMs - and with them clusters of a statically scheduled
// persistent grid - waiting.
// The body uses NO shared memory (block-wide decisions go through __syncthreads_and / __syncthreads_or): a tensor-core
// CTA leaves less than 2 KB of an SM's shared memory free, and a CTA that declares even one shared variable is charged
// a full allocation unit on top of the per-CTA reserve, so it would not fit beside one.
template <int GM>
__device__ __forceinline__ void ddp_bucket_body(const BucketArgs& a) {
  const int W = a.world;
  const int epoch = *((volatile int*)(a.epoch_ctr + a.bucket)) + 1;   // every CTA reads it before the last one bumps it
  int* my_flags = a.flags[a.rank];
  int* ready_row = my_flags + (0 * a.max_buckets + a.bucket) * MAX_WORLD;   // ready_row[w] written by rank w
  int* done_row = my_flags + (1 * a.max_buckets + a.bucket) * MAX_WORLD;
  // ---- 0. bf16 reduction: this rank's fp32 gradients of the whole bucket are rounded into its staging copy, which is
  //         what the peers (or the switch) read; the last CTA to finish the copy opens the entry barrier
  if (GM == GM_BF16_PEER || GM == GM_BF16_MC) {
    const long nv = a.n / 8;                         // buckets of this mode are multiples of 8 elements, 32-byte aligned
    bf16* st = a.gstage[a.rank];
    const float* gr = a.grads[a.rank];
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
      const long e = a.off + i * 8;
      const float4 x = *reinterpret_cast<const float4*>(gr + e), y = *reinterpret_cast<const float4*>(gr + e + 4);
      uint4 o;
      o.x = pack_bf16(x.x, x.y); o.y = pack_bf16(x.z, x.w); o.z = pack_bf16(y.x, y.y); o.w = pack_bf16(y.z, y.w);
      *reinterpret_cast<uint4*>(st + e) = o;
    }
    __threadfence_system();
    __syncthreads();
    int last = 0;
    if (threadIdx.x == 0) last = (atomicAdd(a.done_counter + a.max_buckets + a.bucket, 1) == (int)gridDim.x - 1);
    if (__syncthreads_or(last)) {
      if (threadIdx.x == 0) a.done_counter[a.max_buckets + a.bucket] = 0;
      if (threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(a.flags[threadIdx.x] + (0 * a.max_buckets + a.bucket) * MAX_WORLD + a.rank, epoch);
      }
    }
  } else if (blockIdx.x == 0 && threadIdx.x < W) {
    // ---- 1. entry barrier: gradients of this bucket are final on this rank (stream order), tell every peer
    __threadfence_system();
    st_release_sys(a.flags[threadIdx.x] + (0 * a.max_buckets + a.bucket) * MAX_WORLD + a.rank, epoch);
  }
  int seen = 1;
  if (threadIdx.x < W) seen = wait_flag(ready_row + threadIdx.x, epoch, a.spin_limit_ns, (a.bucket << 8) | threadIdx.x) ? 1 : 0;
  const bool ok = __syncthreads_and(seen) != 0;
  // ---- 2. reduce-scatter + mean + AdamW on this rank's shard, parameters stored to every rank
  if (ok) {
    float lr = a.lr, inv_bc1 = a.inv_bc1, inv_bc2 = a.inv_bc2, scale = a.scale;
    if (a.dev_hyper) { lr = a.dev_hyper[0]; inv_bc1 = a.dev_hyper[1]; inv_bc2 = a.dev_hyper[2]; scale = a.dev_hyper[3]; }
    constexpr int VEC = (GM == GM_BF16_PEER || GM == GM_BF16_MC) ? 8 : 4;
    const long chunk = ((a.n + W - 1) / W + VEC - 1) & ~(long)(VEC - 1);      // shard length, multiple of VEC elements
    const long lo = a.off + (long)a.rank * chunk;
    const long hi = min(a.off + a.n, lo + chunk);
    const long nvec = (hi > lo) ? (hi - lo) / VEC : 0;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
      const long e = lo + i * VEC;
      if (VEC == 4) {
        const float4 g = load_grad_sum4<GM>(a, e, W);
        store_params4(a, e, adamw4(a, e, &g.x, lr, inv_bc1, inv_bc2, scale), W);
      } else {
        float g[8];
        load_grad_sum8<GM>(a, e, W, g);
        store_params4(a, e, adamw4(a, e, g, lr, inv_bc1, inv_bc2, scale), W);
        store_params4(a, e + 4, adamw4(a, e + 4, g + 4, lr, inv_bc1, inv_bc2, scale), W);
      }
    }
    // scalar tail (fp32 peer mode only; the other modes are refused by the host for sizes that leave one)
    if (GM == GM_F32_PEER && blockIdx.x == 0 && threadIdx.x == 0) {
      for (long e = lo + nvec * 4; e < hi; e++) {
        float g = 0.f;
        for (int w = 0; w < W; w++) g += *((volatile float*)(a.grads[w] + e));
        g *= scale;
        float mj = a.b1 * a.m[e] + (1.f - a.b1) * g, vj = a.b2 * a.v[e] + (1.f - a.b2) * g * g, pj = a.master[e];
        pj -= lr * (mj * inv_bc1 / (sqrtf(vj * inv_bc2) + a.eps) + a.wd * pj);
        a.m[e] = mj; a.v[e] = vj; a.master[e] = pj;
        for (int w = 0; w < W; w++)
          if (a.bcast || w == a.rank) a.params[w][e] = __float2bfloat16(pj);
      }
    }
  }
  // ---- 3. exit barrier (last CTA of this rank)
  __threadfence_system();
  __syncthreads();
  int last = 0;
  if (threadIdx.x == 0) last = (atomicAdd(a.done_counter + a.bucket, 1) == (int)gridDim.x - 1);
  if (!__syncthreads_or(last)) return;
  if (threadIdx.x == 0) { a.done_counter[a.bucket] = 0; a.epoch_ctr[a.bucket] = epoch; }
  if (threadIdx.x < W) {
    __threadfence_system();
    int* peer_flags = a.flags[threadIdx.x];
    st_release_sys(peer_flags + (1 * a.max_buckets + a.bucket) * MAX_WORLD + a.rank, epoch);
    if (ok) wait_flag(done_row + threadIdx.x, epoch, a.spin_limit_ns, 0x8000 | (a.bucket << 8) | threadIdx.x);
  }
}
// lean: capped at 32 registers for launches that share SMs with the backward pass; the other form lets the compiler keep
// every peer's load in flight and is used when the kernel has the machine to itself (the last bucket, un-overlapped runs)
template <int GM>
__global__ void __maxnreg__(32) ddp_bucket_lean_kernel(const BucketArgs a) { ddp_bucket_body<GM>(a); }
template <int GM>
__global__ void __launch_bounds__(256) ddp_bucket_kernel(const BucketArgs a) { ddp_bucket_body<GM>(a); }

// All-gather by peer loads: dst[w*chunk_bytes ...] = shard of rank w, for every w; 16-byte vectors, system-scope loads.
// No barrier is needed here: the producer of the shards (the reduce-scatter + AdamW kernel of the previous step) ends
// with a barrier across all ranks, and this kernel is ordered after it on the same stream.
// 31 registers and no shared memory: with 128-thread CTAs and the largest shared-memory split (set at launch) its CTAs fit
// beside those of the persistent tensor-core kernels, see ddp_bucket_lean_kernel.
__global__ void __maxnreg__(32) allgather_pull_kernel(uint4* __restrict__ dst, const uint4* const* __restrict__ src,
                                                      long chunk_vec, int world) {
  const long total = chunk_vec * world;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int w = (int)(i / chunk_vec);
    const long j = i - (long)w * chunk_vec;
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src[w] + j) : "memory");
    dst[i] = v;
  }
}

// Co-residency probe (micro-benchmark hook): a small kernel without shared memory, at most 32 registers per thread, that
// keeps its CTAs busy for `dur_ns` - mode 0 by watching the clock, modes 1 / 2 by streaming `n4` float4 of `buf` through
// x = x * 1.0000001f over and over (default caching / evict-first hints) - so that its effect on a tensor-core kernel
// running at the same time on another stream can be measured.  CARVE selects the shared-memory split it asks for.
template <bool CARVE>
__global__ void __maxnreg__(32) corun_probe_kernel(float4* buf, long n4, long dur_ns, int mode) {
  const uint64_t t0 = gtimer();
  if (mode == 0) {
    while ((long)(gtimer() - t0) < dur_ns) __nanosleep(200);
    return;
  }
  for (;;) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
      float4 x;
      if (mode == 2) asm volatile("ld.global.cs.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w) : "l"(buf + i));
      else x = buf[i];
      x.x *= 1.0000001f; x.y *= 1.0000001f; x.z *= 1.0000001f; x.w *= 1.0000001f;
      if (mode == 2) asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(buf + i), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
      else buf[i] = x;
      if ((i & 0xfff) == 0 && (long)(gtimer() - t0) >= dur_ns) return;
    }
    if ((long)(gtimer() - t0) >= dur_ns) return;
  }
}

// Test hook: waits (bounded) on a flag that nothing sets, to exercise the timeout path on one GPU.
__global__ void flag_timeout_probe_kernel(const int* flag, int epoch, long limit_ns, int* result) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *result = wait_flag(flag, epoch, limit_ns, 0x7777) ? 1 : 2;
}

}  // namespace

MLB_API int mlb_comm_max_world() { return MAX_WORLD; }

// One bucket of the fused data-parallel gradient step.  Pointer arrays live in device memory (world entries each).
//   gmode        GM_* above.  The multicast modes need the matching multicast address; the bf16 modes need the staging
//                pointer table (and `done_counter` 2 * max_buckets ints long), off and n multiples of 8.
//   ctas         grid size (256 threads each); lean != 0 selects the 32-register form (see above)
MLB_API int mlb_ddp_bucket2(const void* grads_ptrs, const void* params_ptrs, const void* flags_ptrs, float* master, float* m, float* v,
                            int* done_counter, int* epoch_ctr, long off, long n, int rank, int world, int bucket, int max_buckets,
                            int bcast, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float scale,
                            const float* dev_hyper, int ctas, double spin_limit_s, float* grads_mc, void* params_mc,
                            const void* gstage_ptrs, void* gstage_mc, int gmode, int lean, cudaStream_t st) {
  if (world < 1 || world > MAX_WORLD || bucket < 0 || bucket >= max_buckets) return -1;
  if ((off & 3) != 0) return -5;   // float4 path needs 16-byte aligned bucket starts
  if (gmode == GM_F32_MC && grads_mc == nullptr) return -8;
  if ((gmode == GM_BF16_PEER || gmode == GM_BF16_MC) && (gstage_ptrs == nullptr || (off & 7) != 0 || (n & 7) != 0)) return -8;
  if (gmode == GM_BF16_MC && gstage_mc == nullptr) return -8;
  if (gmode == GM_F32_MC && (n & 3) != 0) return -8;
  BucketArgs a;
  a.grads = (float* const*)grads_ptrs; a.params = (bf16* const*)params_ptrs; a.flags = (int* const*)flags_ptrs;
  a.master = master; a.m = m; a.v = v; a.done_counter = done_counter; a.epoch_ctr = epoch_ctr;
  a.off = off; a.n = n; a.rank = rank; a.world = world; a.bucket = bucket; a.max_buckets = max_buckets;
  a.bcast = bcast; a.lr = lr; a.b1 = b1; a.b2 = b2; a.eps = eps; a.wd = wd; a.inv_bc1 = 1.f / bc1; a.inv_bc2 = 1.f / bc2;
  a.scale = scale; a.dev_hyper = dev_hyper; a.grads_mc = grads_mc; a.params_mc = (bf16*)params_mc; a.spin_limit_ns = (long)(spin_limit_s * 1e9);
  a.gstage = (bf16* const*)gstage_ptrs; a.gstage_mc = (bf16*)gstage_mc;
  const long chunk = ((n + world - 1) / world + 7) & ~7L;
  long want = (chunk / 4 + 127) / 128;
  if (want < 1) want = 1;
  if (ctas < 1) ctas = 64;
  const int grid = (int)(want < ctas ? want : ctas);
  // An SM's split between L1 and shared memory is fixed while CTAs are resident on it.  The tensor-core kernels need the
  // largest shared-memory split; a bucket CTA that got onto an idle SM first with the default (L1-heavy) split would keep
  // their CTAs (and with them whole clusters of a persistent grid) waiting until it leaves.  So these kernels ask for
  // the largest shared-memory split too, although they use none.
#define MLB_BUCKET_CASE(GMV)                                                                                              \
  case GMV: {                                                                                                             \
    static bool carve = false;                                                                                            \
    if (!carve) {                                                                                                         \
      cudaFuncSetAttribute(ddp_bucket_lean_kernel<GMV>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared); \
      cudaFuncSetAttribute(ddp_bucket_kernel<GMV>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);      \
      carve = true;                                                                                                       \
    }                                                                                                                     \
    if (lean) ddp_bucket_lean_kernel<GMV><<<grid, 128, 0, st>>>(a);                                                       \
    else ddp_bucket_kernel<GMV><<<grid, 256, 0, st>>>(a);                                                                 \
    break;                                                                                                                \
  }
  switch (gmode) {
    MLB_BUCKET_CASE(GM_F32_PEER)
    MLB_BUCKET_CASE(GM_F32_MC)
    MLB_BUCKET_CASE(GM_BF16_PEER)
    MLB_BUCKET_CASE(GM_BF16_MC)
    default: return -1;
  }
#undef MLB_BUCKET_CASE
  return (int)cudaGetLastError();
}

// The fp32 form (peer loads, or the multicast address when one is given); `ctas` counts 512-thread blocks as before.
MLB_API int mlb_ddp_bucket(const void* grads_ptrs, const void* params_ptrs, const void* flags_ptrs, float* master, float* m, float* v,
                           int* done_counter, int* epoch_ctr, long off, long n, int rank, int world, int bucket, int max_buckets,
                           int bcast, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float scale,
                           const float* dev_hyper, int ctas, double spin_limit_s, float* grads_mc, void* params_mc,
                           cudaStream_t st) {
  return mlb_ddp_bucket2(grads_ptrs, params_ptrs, flags_ptrs, master, m, v, done_counter, epoch_ctr, off, n, rank, world, bucket,
                         max_buckets, bcast, lr, b1, b2, eps, wd, bc1, bc2, scale, dev_hyper, ctas < 1 ? 64 : 2 * ctas, spin_limit_s,
                         grads_mc, params_mc, nullptr, nullptr, (grads_mc != nullptr && (n & 3) == 0) ? GM_F32_MC : GM_F32_PEER, 0, st);
}

// dst (local) <- concatenation of the `world` shards whose device pointers are in src_ptrs (device array); every shard
// is chunk_bytes long (a multiple of 16).
// `threads` per CTA: 128 for a launch that shares SMs with compute kernels, 512 for one that has the machine.
MLB_API int mlb_allgather_pull2(void* dst, const void* src_ptrs, long chunk_bytes, int world, int ctas, int threads, cudaStream_t st) {
  if ((chunk_bytes & 15) != 0 || world < 1 || threads < 32 || threads > 1024) return -1;
  static bool carve = false;
  if (!carve) {
    cudaFuncSetAttribute(allgather_pull_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    carve = true;
  }
  const long chunk_vec = chunk_bytes / 16;
  long want = (chunk_vec * world + threads - 1) / threads;
  if (want < 1) want = 1;
  if (ctas < 1) ctas = 32;
  allgather_pull_kernel<<<(int)(want < ctas ? want : ctas), threads, 0, st>>>((uint4*)dst, (const uint4* const*)src_ptrs, chunk_vec, world);
  return (int)cudaGetLastError();
}
MLB_API int mlb_allgather_pull(void* dst, const void* src_ptrs, long chunk_bytes, int world, int ctas, cudaStream_t st) {
  return mlb_allgather_pull2(dst, src_ptrs, chunk_bytes, world, ctas, 512, st);
}

MLB_API int mlb_corun_probe(float* buf, long n_floats, double dur_s, int mode, int ctas, int threads, int max_shared_carveout, cudaStream_t st) {
  if (dur_s > 0.05) dur_s = 0.05;          // a probe, not a load generator: 50 ms at most
  if (max_shared_carveout) {
    cudaFuncSetAttribute(corun_probe_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    corun_probe_kernel<true><<<ctas, threads, 0, st>>>((float4*)buf, n_floats / 4, (long)(dur_s * 1e9), mode);
  } else {
    corun_probe_kernel<false><<<ctas, threads, 0, st>>>((float4*)buf, n_floats / 4, (long)(dur_s * 1e9), mode);
  }
  return (int)cudaGetLastError();
}

// Runs the bounded flag wait against `flag` (device memory, never written) and stores 1 (seen) or 2 (timed out) in *result.
MLB_API int mlb_flag_timeout_probe(const int* flag, int epoch, double limit_s, int* result, cudaStream_t st) {
  flag_timeout_probe_kernel<<<1, 32, 0, st>>>(flag, epoch, (long)(limit_s * 1e9), result);
  return (int)cudaGetLastError();
}
