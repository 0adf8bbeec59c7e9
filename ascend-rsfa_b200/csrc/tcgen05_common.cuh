// Pieces shared by the tcgen05 attention kernels: wait tags, debug trace hooks, packed-math
// helpers, register re-budgeting and the host-side TMA map construction.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace rsfa {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
#ifndef RSFA_SUM_LIMIT
#define RSFA_SUM_LIMIT 32768.0f
#endif
#ifndef RSFA_HEADROOM
#define RSFA_HEADROOM 6.0f
#endif
// The reference maximum of a row is placed this many log2 units ABOVE the largest score seen when
// it is set, so P starts at <= 2^-6 and a row can grow by 21 log2 units before anything has to be
// rescaled.  fp16 keeps full precision down to 2^-14, i.e. for weights down to 2^-8 of the row's
// largest, and denormals (absolute error 2^-19 of the largest weight) below that.  On benchmark configuration
// cfg2 (N(0,1) inputs, sm_scale 0.5: near one-hot rows) 0.6 % of the warp-steps still took the
// careful path with a headroom of 4; 4 -> 6 -> 8 gave 1171 -> 1194 -> 1206 TFLOP/s there.
constexpr float kHeadroomLog2 = RSFA_HEADROOM;
// Bound on the sum of the exponentials of one 64-key half of a row (and thereby on every P value
// of it; all terms are non-negative) above which the softmax leaves its fast path; fp16 holds
// 65504.
constexpr float kSumLimit = RSFA_SUM_LIMIT;

// Wait-site tags (reported in the status word when a wait runs out).
enum : int {
  kTagQEmpty = 1, kTagKvEmpty = 2, kTagQFull = 3, kTagKvFull = 4, kTagPFull = 5, kTagSFull = 6, kTagOFull = 7,
  kTagSched = 8, kTagPvDone = 10
};

// Debug builds (-DRSFA_TRACE) log (clock, code) pairs per role for CTA 0; the product build
// compiles this away.
#ifdef RSFA_TRACE
constexpr int kTraceCap = 4096;
#define RSFA_TRACE_DECL(role_) \
  unsigned long long* trace_buf = (p.trace != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0) ? p.trace + (role_) * 2 * kTraceCap : nullptr; \
  int trace_n = 0
#define RSFA_TRACE_EV(code_)                                         \
  do {                                                               \
    if (trace_buf != nullptr && trace_n < kTraceCap) {               \
      trace_buf[2 * trace_n] = static_cast<unsigned long long>(clock64()); \
      trace_buf[2 * trace_n + 1] = static_cast<unsigned long long>(code_); \
      ++trace_n;                                                     \
    }                                                                \
  } while (0)
#else
#define RSFA_TRACE_DECL(role_) do {} while (0)
#define RSFA_TRACE_EV(code_) do {} while (0)
#endif

struct TmaMaps {
  CUtensorMap q, k, v, o;
};

// Work items = (batch * head, block of Q rows), numbered head-major so that the CTAs working on one head
// find its K/V in L2; with the causal mask the blocks of a head come heaviest (last rows) first.  The items
// of the last `tail_heads` heads are numbered differently when the mask makes their sizes differ: block-major
// (the heaviest block of each of those heads, then the next lighter one of each, ...), so that the queue ends
// on the lightest items of the launch instead of on a whole head, heaviest block included, and the CTAs
// finish together.
struct SchedInfo {
  int total_items;
  int items_per_head;  // blocks of Q rows per head
  int tail_first;      // first item of the block-major tail (== total_items: no tail)
  int tail_heads;
  int split_items;     // separate-P kernel: the last so many items are handed out as two single Q tiles each
};

// `sched.total_items` and `sched.items_per_head` set: the tail covers about two items per CTA.
inline void sched_set_tail(SchedInfo& sched, int heads, int causal, int grid) {
  sched.tail_first = sched.total_items;
  sched.tail_heads = 0;
  sched.split_items = 0;
  if (causal != 0 && sched.items_per_head > 1) {
    int th = (2 * grid + sched.items_per_head - 1) / sched.items_per_head;
    if (th > heads) th = heads;
    sched.tail_heads = th;
    sched.tail_first = (heads - th) * sched.items_per_head;
  }
}

// work item -> (batch * head, block of Q rows)
__device__ __forceinline__ void sched_decode(const SchedInfo& sched, int causal, int item, int& bh, int& blk) {
  if (item < sched.tail_first) {
    bh = item / sched.items_per_head;
    blk = item - bh * sched.items_per_head;
    if (causal) blk = sched.items_per_head - 1 - blk;
  } else {
    const int r = item - sched.tail_first;
    const int rank = r / sched.tail_heads;            // 0 = heaviest block
    bh = sched.tail_first / sched.items_per_head + (r - rank * sched.tail_heads);
    blk = sched.items_per_head - 1 - rank;
  }
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}

template <bool kBf16>
__device__ __forceinline__ void unpack2(uint32_t v, float& lo, float& hi) {
  if constexpr (kBf16) {
    lo = __uint_as_float(v << 16);
    hi = __uint_as_float(v & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    lo = f.x;
    hi = f.y;
  }
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// Two fp32 lanes in one 64-bit register: Blackwell's packed FFMA2 / FADD2 halve the issue slots
// of the scale-and-subtract and of the row sum.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}


// Careful version of the softmax of 64 keys (half a 128-key tile, or one 64-key tile), used once a
// kernel's fast loop has found that a P value might leave the 16-bit range.  It is deliberately
// NOT inlined and is called only from code behind the fast loop: inside the fast loop even a call
// to it slowed every step by 5 %.
// The scores of the half are still intact in tensor memory (P has not been written over them), so
// they are loaded again: true row maximum, new reference (with headroom) for rows that exceeded
// the old one, l and (if `rescale`) this thread's row of O_t brought to the new reference, then
// exp2 / sum / pack and the tcgen05.st of P.  Returns {new reference, l + this half's sum}.
// `limit` = last visible score of the half (63 if none is masked).  All 32 lanes call it together.
template <int D, bool kBf16>
__device__ __noinline__ uint64_t softmax_half_careful(uint32_t t_s, uint32_t t_p, uint32_t t_o, int limit,
                                                      float scale_log2, float headroom, float m_used, float l,
                                                      int rescale) {
  uint32_t a[32], b[32];
  tmem_ld_x32(t_s, a);
  tmem_ld_x32(t_s + 32, b);
  tmem_wait_ld();
  reg_fence_x32(a);
  reg_fence_x32(b);
  if (limit < 63) {
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      if (c > limit) a[c] = 0xff800000u;
      if (c + 32 > limit) b[c] = 0xff800000u;
    }
  }
  float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    mx[0] = max3(mx[0], __uint_as_float(a[c]), __uint_as_float(a[c + 1]));
    mx[1] = max3(mx[1], __uint_as_float(a[c + 2]), __uint_as_float(a[c + 3]));
    mx[2] = max3(mx[2], __uint_as_float(b[c]), __uint_as_float(b[c + 1]));
    mx[3] = max3(mx[3], __uint_as_float(b[c + 2]), __uint_as_float(b[c + 3]));
  }
  const float mb = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
  float alpha = 1.f;
  if (mb > m_used) {
    const float m_new = mb + headroom;
    alpha = ex2((m_used - m_new) * scale_log2);
    l *= alpha;
    m_used = m_new;
  }
  if (rescale && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t o[32];
      tmem_ld_x32(t_o + c0, o);
      tmem_wait_ld();
      reg_fence_x32(o);
#pragma unroll
      for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
      tmem_st_x32(t_o + c0, o);
    }
  }
  const float neg_m = -m_used * scale_log2;
  float h0 = 0.f, h1 = 0.f;
  uint32_t pk[32];
#pragma unroll
  for (int c = 0; c < 32; c += 2) {
    const float e0 = ex2(fmaf(__uint_as_float(a[c]), scale_log2, neg_m));
    const float e1 = ex2(fmaf(__uint_as_float(a[c + 1]), scale_log2, neg_m));
    const float e2 = ex2(fmaf(__uint_as_float(b[c]), scale_log2, neg_m));
    const float e3 = ex2(fmaf(__uint_as_float(b[c + 1]), scale_log2, neg_m));
    h0 += e0 + e1;
    h1 += e2 + e3;
    pk[c >> 1] = pack2<kBf16>(e0, e1);
    pk[16 + (c >> 1)] = pack2<kBf16>(e2, e3);
  }
  tmem_st_x32(t_p, pk);
  return pack_f32x2(m_used, l + (h0 + h1));
}

// Epilogue of one warp: its 32 rows of O (kCols fp32 columns in tensor memory at `t_o`, one row per
// lane) times inv_l, as 16-bit values, to global memory.  The rows go through the warp's own 4 KB of
// 128-byte-swizzled staging (`stage`, 1024-byte aligned) and one TMA store per 64 columns: a thread owns
// a whole row, so direct stores would touch 32 different lines per instruction, and per-warp staging needs
// no synchronisation wider than a warp.  `map_o` describes O with boxes of 64 columns x 32 rows; rows past
// the end of the tensor are clipped by the store, and `any_row` = false (all 32 rows past the end) stores
// nothing.  All 32 lanes call it together; the caller waits for the stores before the CTA exits
// (tma_store_wait_all by lane 0).  kBufs = 2: `stage` holds two such 4 KB buffers used in turn, so that
// a store reads one while the next 64 columns are written to the other.
template <int kCols, bool kBf16, int kBufs = 1>
__device__ __forceinline__ void store_o_rows(uint32_t t_o, float inv_l, uint32_t stage, int lane,
                                             const CUtensorMap* map_o, int row_first, int h, int b, bool any_row) {
  const bool issuer = (lane == 0);
#pragma unroll 1
  for (int c0 = 0; c0 < kCols; c0 += 64) {
    uint32_t o0[32], o1[32];
    tmem_ld_x32(t_o + c0, o0);
    tmem_ld_x32(t_o + c0 + 32, o1);
    tmem_wait_ld();
    reg_fence_x32(o0);
    reg_fence_x32(o1);
    // the store that last read this staging buffer is done with it
    if (issuer) tma_store_wait_read_but<kBufs - 1>();
    __syncwarp();
    const uint32_t buf = stage + (kBufs == 1 ? 0u : static_cast<uint32_t>((c0 >> 6) % kBufs) * 4096u);
    const uint32_t row_addr = buf + lane * 128;
    const uint32_t sw = static_cast<uint32_t>(lane & 7);
#pragma unroll
    for (int c = 0; c < 32; c += 8) {
      st_shared_v4(row_addr + (((c >> 3) ^ sw) << 4),
                   pack2<kBf16>(__uint_as_float(o0[c + 0]) * inv_l, __uint_as_float(o0[c + 1]) * inv_l),
                   pack2<kBf16>(__uint_as_float(o0[c + 2]) * inv_l, __uint_as_float(o0[c + 3]) * inv_l),
                   pack2<kBf16>(__uint_as_float(o0[c + 4]) * inv_l, __uint_as_float(o0[c + 5]) * inv_l),
                   pack2<kBf16>(__uint_as_float(o0[c + 6]) * inv_l, __uint_as_float(o0[c + 7]) * inv_l));
      st_shared_v4(row_addr + ((((c >> 3) + 4) ^ sw) << 4),
                   pack2<kBf16>(__uint_as_float(o1[c + 0]) * inv_l, __uint_as_float(o1[c + 1]) * inv_l),
                   pack2<kBf16>(__uint_as_float(o1[c + 2]) * inv_l, __uint_as_float(o1[c + 3]) * inv_l),
                   pack2<kBf16>(__uint_as_float(o1[c + 4]) * inv_l, __uint_as_float(o1[c + 5]) * inv_l),
                   pack2<kBf16>(__uint_as_float(o1[c + 6]) * inv_l, __uint_as_float(o1[c + 7]) * inv_l));
    }
    fence_proxy_async();
    __syncwarp();
    if (issuer && any_row) {
      tma_store_4d(map_o, buf, c0, row_first, h, b);
      tma_store_commit();
    }
  }
}

// Register budgets per warpgroup after the common set-up of the 384-thread kernels (the launch
// allocates 168 per thread): two softmax warpgroups and the warpgroup of the TMA / MMA warps.
// setmaxnreg.inc can only take registers that another warpgroup of the same CTA has released with
// setmaxnreg.dec: an increase that asks for more than was released waits for ever (it did, with
// 208 / 96).  D = 128: 200 / 104 (184 / 136 and 168 / 168 measure the same: the softmax does not need
// more than 168); D = 64: 208 / 80 (200 / 104 is 6 % slower there).
template <int D>
struct RegBudget {
  static constexpr int kLaunch = 168;
  static constexpr int kSoftmax = (D == 128) ? 200 : 208;
  static constexpr int kOther = (D == 128) ? 104 : 80;
  static_assert(128 * (kLaunch - kOther) >= 2 * 128 * (kSoftmax - kLaunch),
                "the softmax warpgroups can only take what the third warpgroup releases");
};
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// Last act of a CTA of a persistent kernel (one thread, after the CTA's final barrier): count the CTA as
// finished in word [1] of the work queue; the CTA that completes the count puts both words back
// to zero.  Every CTA's own additions to word [0] are behind it by then, so the pair is zero again
// when the grid has exited - also when the CTAs left early through the wait-expired path.
__device__ __forceinline__ void queue_retire(unsigned int* queue) {
  __threadfence();
  if (atomicAdd(queue + 1, 1u) == gridDim.x - 1) {
    queue[0] = 0u;
    queue[1] = 0u;
    __threadfence();
  }
}

// ---------------------------------------------------------------- host side
// Launch of a persistent kernel, with programmatic stream serialisation when `pdl` is set: the
// kernel may then begin its set-up (barriers, tensor-memory allocation, descriptor prefetch) while
// the kernel in front of it on the stream drains, and waits in griddep_wait() before it touches
// global memory.
template <typename Kernel, typename... Args>
cudaError_t launch_persistent(Kernel kern, int grid, int threads, size_t smem, cudaStream_t stream, bool pdl,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned int>(grid));
  cfg.blockDim = dim3(static_cast<unsigned int>(threads));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static std::atomic<EncodeTiledFn> fn{nullptr};
  EncodeTiledFn f = fn.load(std::memory_order_acquire);
  if (f == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      f = reinterpret_cast<EncodeTiledFn>(ptr);
      fn.store(f, std::memory_order_release);
    }
  }
  return f;
}

// [B,H,S,D] tensor, 16-bit elements, as a 4-D map (D, S, H, B) with boxes of 64 x `box_rows`.
bool make_map(CUtensorMap* map, const void* base, const FwdParams& p, const int64_t* st, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(p.D), static_cast<cuuint64_t>(p.S),
                              static_cast<cuuint64_t>(p.H), static_cast<cuuint64_t>(p.B)};
  // A dimension of extent 1 may carry any stride (PyTorch leaves whatever the view had): the
  // encoder wants multiples of 16 bytes, so such a dimension gets the dense stride instead.
  auto stride_bytes = [&](int64_t s, int extent, int64_t dense) {
    return static_cast<cuuint64_t>(((extent > 1 && s > 0) ? s : dense) * 2);
  };
  const cuuint64_t strides[3] = {stride_bytes(st[2], p.S, p.D), stride_bytes(st[1], p.H, static_cast<int64_t>(p.S) * p.D),
                                 stride_bytes(st[0], p.B, static_cast<int64_t>(p.H) * p.S * p.D)};
  const cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(box_rows), 1u, 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = enc(map, p.bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace
}  // namespace rsfa
