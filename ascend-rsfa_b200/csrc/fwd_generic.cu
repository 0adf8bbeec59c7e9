// Generic FlashAttention-2 forward for sm_100a on the legacy tensor path
// (mma.sync m16n8k16, fp32 accumulate): the counterpart of the reference's
// single-tile kernels _attn_fwd_small and _attn_fwd_small_causal
// (ascend_rsfa/flash_attention_forward.py:26-159), which are latency- and
// HBM-bound.  The dispatcher sends it the smallest tiles - head dimension 16 at
// S <= 128, sequences of at most 64 keys at D <= 64 - where it measures faster
// than the tcgen05 kernels, and every shape with a non-positive sm_scale, which
// those are not built for.  It accepts any S >= 1, any D in {16,32,64,128,256} and
// any strides with a contiguous innermost dimension (the "force_path" option runs
// it on every shape: the parity tests compare the two families that way); rows and
// keys past S are predicated, which the reference does not do.
//
// One CTA = 4 warps = 64 query rows; each warp owns 16 rows and sweeps the keys
// in tiles of kBN with the online-softmax recurrence of _attn_fwd_inner
// (:184-224): scale, running max, p = exp(s - m) rounded to the input type before
// the second product (:211), l and acc rescaled by alpha (:217-223).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace rsfa {
namespace {

constexpr int kBM = 64;
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int D>
struct GenericCfg {
  static constexpr int kBN = (D >= 256) ? 32 : 64;
  static constexpr int kLd = D + 8;  // padded row, in elements: shifts rows by 16 B across banks
  static constexpr int kSmemBytes = (kBM + 2 * kBN) * kLd * 2;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <bool kBf16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

// Copy `rows` x D 16-bit elements (row stride `stride` elements) into padded shared
// memory; rows at or past `valid_rows` are zero-filled.
template <int D, int kLd>
__device__ __forceinline__ void load_tile(uint16_t* smem, const uint16_t* gmem, int64_t stride,
                                          int rows, int valid_rows) {
  constexpr int kVecPerRow = D / 8;
  for (int idx = threadIdx.x; idx < rows * kVecPerRow; idx += kThreads) {
    const int r = idx / kVecPerRow;
    const int c = (idx % kVecPerRow) * 8;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < valid_rows) val = *reinterpret_cast<const uint4*>(gmem + r * stride + c);
    *reinterpret_cast<uint4*>(smem + r * kLd + c) = val;
  }
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads) fwd_generic_kernel(const FwdParams p) {
  using Cfg = GenericCfg<D>;
  constexpr int kBN = Cfg::kBN;
  constexpr int kLd = Cfg::kLd;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint16_t* sQ = reinterpret_cast<uint16_t*>(smem_raw);
  uint16_t* sK = sQ + kBM * kLd;
  uint16_t* sV = sK + kBN * kLd;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // One linear grid index = (head, row block): gridDim.y stops at 65535, the number of heads does not.
  const int S = p.S;
  const int row_blocks = (S + kBM - 1) / kBM;
  const int bh = blockIdx.x / row_blocks;
  const int b = bh / p.H;
  const int h = bh % p.H;
  const int m0 = (blockIdx.x - bh * row_blocks) * kBM;

  const uint16_t* gq = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_stride[0] + h * p.q_stride[1];
  const uint16_t* gk = reinterpret_cast<const uint16_t*>(p.k) + b * p.k_stride[0] + h * p.k_stride[1];
  const uint16_t* gv = reinterpret_cast<const uint16_t*>(p.v) + b * p.v_stride[0] + h * p.v_stride[1];
  uint16_t* go = reinterpret_cast<uint16_t*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1];

  load_tile<D, kLd>(sQ, gq + static_cast<int64_t>(m0) * p.q_stride[2], p.q_stride[2], kBM, S - m0);

  const float scale_log2 = p.sm_scale * kLog2e;
  // Row ownership inside the m16n8 accumulator: c0,c1 -> row lane/4, c2,c3 -> row lane/4 + 8.
  const int row_lo = m0 + warp * 16 + (lane >> 2);
  const int row_hi = row_lo + 8;

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  const int kv_end = p.causal ? min(S, m0 + kBM) : S;
  for (int n0 = 0; n0 < kv_end; n0 += kBN) {
    __syncthreads();  // previous tile fully consumed (also orders the Q load on the first pass)
    load_tile<D, kLd>(sK, gk + static_cast<int64_t>(n0) * p.k_stride[2], p.k_stride[2], kBN, S - n0);
    load_tile<D, kLd>(sV, gv + static_cast<int64_t>(n0) * p.v_stride[2], p.v_stride[2], kBN, S - n0);
    __syncthreads();

    // ---- scores: 16 rows x kBN keys per warp
    float s[kBN / 8][4];
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 16 + (lane >> 4) * 8;
        ldmatrix_x4(a, static_cast<uint32_t>(__cvta_generic_to_shared(sQ + r * kLd + c)));
      }
#pragma unroll
      for (int nt = 0; nt < kBN / 16; ++nt) {
        uint32_t bfrag[4];
        const int r = nt * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(bfrag, static_cast<uint32_t>(__cvta_generic_to_shared(sK + r * kLd + c)));
        mma_16816<kBf16>(s[2 * nt], a, bfrag[0], bfrag[1]);
        mma_16816<kBf16>(s[2 * nt + 1], a, bfrag[2], bfrag[3]);
      }
    }

    // ---- scale (to log2 units), mask, running max
    const bool need_mask = (n0 + kBN > S) || (p.causal && n0 + kBN > m0 + warp * 16);
    float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[i][e] * scale_log2;
        if (need_mask) {
          const int col = n0 + i * 8 + (lane & 3) * 2 + (e & 1);
          const int row = (e < 2) ? row_lo : row_hi;
          if (col >= S || (p.causal && col > row)) x = -INFINITY;
        }
        s[i][e] = x;
        if (e < 2) tmax_lo = fmaxf(tmax_lo, x); else tmax_hi = fmaxf(tmax_hi, x);
      }
    }
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
    const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
    // A row with nothing visible yet keeps m = -inf; use 0 as the subtrahend so no inf-inf appears.
    const float ms_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo;
    const float ms_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    const float alpha_lo = exp2f(m_lo - ms_lo), alpha_hi = exp2f(m_hi - ms_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;

    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t pfrag[kBN / 8][2];
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) {
      const float p0 = exp2f(s[i][0] - ms_lo), p1 = exp2f(s[i][1] - ms_lo);
      const float p2 = exp2f(s[i][2] - ms_hi), p3 = exp2f(s[i][3] - ms_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pfrag[i][0] = pack2<kBf16>(p0, p1);
      pfrag[i][1] = pack2<kBf16>(p2, p3);
    }
    l_lo = l_lo * alpha_lo + sum_lo;  // partial sums: the quad is reduced once, in the epilogue
    l_hi = l_hi * alpha_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      acc[i][0] *= alpha_lo;
      acc[i][1] *= alpha_lo;
      acc[i][2] *= alpha_hi;
      acc[i][3] *= alpha_hi;
    }

    // ---- acc += P V
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      const uint32_t a[4] = {pfrag[2 * kk][0], pfrag[2 * kk][1], pfrag[2 * kk + 1][0],
                             pfrag[2 * kk + 1][1]};
#pragma unroll
      for (int dt = 0; dt < D / 16; ++dt) {
        uint32_t bfrag[4];
        const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = dt * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(bfrag, static_cast<uint32_t>(__cvta_generic_to_shared(sV + r * kLd + c)));
        mma_16816<kBf16>(acc[2 * dt], a, bfrag[0], bfrag[1]);
        mma_16816<kBf16>(acc[2 * dt + 1], a, bfrag[2], bfrag[3]);
      }
    }
  }

  // ---- epilogue: O = acc / l, lse = m + log l (natural log; :400-404)
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = 1.f / l_lo, inv_hi = 1.f / l_hi;
  const int col0 = (lane & 3) * 2;
  if (row_lo < S) {
    uint16_t* dst = go + static_cast<int64_t>(row_lo) * p.o_stride[2];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + col0) = pack2<kBf16>(acc[i][0] * inv_lo, acc[i][1] * inv_lo);
    if (p.lse != nullptr && (lane & 3) == 0)
      p.lse[static_cast<int64_t>(bh) * S + row_lo] = m_lo * kLn2 + logf(l_lo);
  }
  if (row_hi < S) {
    uint16_t* dst = go + static_cast<int64_t>(row_hi) * p.o_stride[2];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + col0) = pack2<kBf16>(acc[i][2] * inv_hi, acc[i][3] * inv_hi);
    if (p.lse != nullptr && (lane & 3) == 0)
      p.lse[static_cast<int64_t>(bh) * S + row_hi] = m_hi * kLn2 + logf(l_hi);
  }
}

template <int D, bool kBf16>
cudaError_t launch_one(const FwdParams& p, cudaStream_t stream) {
  using Cfg = GenericCfg<D>;
  auto kern = fwd_generic_kernel<D, kBf16>;
  static std::atomic<unsigned long long> smem_done{0};   // per kernel instantiation, bit per device
  cudaError_t e = set_dynamic_smem_once(smem_done, reinterpret_cast<const void*>(kern), Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  const long long blocks = generic_grid_blocks(p.B, p.H, p.S);
  if (blocks > 2147483647LL) return cudaErrorInvalidConfiguration;
  kern<<<static_cast<unsigned int>(blocks), kThreads, Cfg::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

template <int D>
cudaError_t launch_dtype(const FwdParams& p, cudaStream_t stream) {
  return p.bf16 ? launch_one<D, true>(p, stream) : launch_one<D, false>(p, stream);
}

}  // namespace

long long generic_grid_blocks(int B, int H, int S) {
  return static_cast<long long>(B) * H * ((S + kBM - 1) / kBM);
}

cudaError_t launch_fwd_generic(const FwdParams& p, cudaStream_t stream, long long* launches) {
  cudaError_t e;
  switch (p.D) {
    case 16: e = launch_dtype<16>(p, stream); break;
    case 32: e = launch_dtype<32>(p, stream); break;
    case 64: e = launch_dtype<64>(p, stream); break;
    case 128: e = launch_dtype<128>(p, stream); break;
    case 256: e = launch_dtype<256>(p, stream); break;
    default: return cudaErrorInvalidValue;
  }
  if (e == cudaSuccess) *launches += 1;
  return e;
}

}  // namespace rsfa
