// FlashAttention-2 forward for head dimension 256 on B200 (sm_100a).
//
// Same building blocks as the D <= 128 kernel (tcgen05 MMAs, accumulators in tensor memory, TMA
// staging, atomic work queue), different shape: at D = 256 the output accumulator alone takes 256
// of the 512 TMEM columns per 128 rows, so a CTA owns ONE Q tile of 128 rows and overlaps work by
// double-buffering S instead of ping-ponging two Q tiles:
//   S[j & 1] = Q K_j^T        keys in tiles of 64: 16 MMAs of 128x64x16, both operands in smem
//   softmax warps             S[j & 1] -> P_j (16-bit, written over S[j & 1])
//   O += P_j V_j              4 MMAs of 128x256x16, A = P_j from TMEM, B = V_j MN-major
// QK^T of tile j+2 is issued right after PV of tile j, so the tensor pipe works on tile j+1, j+2
// while the softmax warps are on tile j+1.  TMEM columns: S[0] [0,64)  S[1] [64,128)  O [128,384).
// Shared memory: Q 64 KB + 4 ring slots of 32 KB (K and V tiles of 64 keys).
//
// It covers the reference's D = 256 shapes (ascend_rsfa/flash_attention_forward.py:653-661 lists
// them in its tile table; the kernels are the same _attn_fwd / _run_causal_split, :271-541).
//
// Roles: warps 0..3 softmax (one thread per row), warp 4 TMA producer, warp 5 MMA issuer.
#include "tcgen05_common.cuh"

namespace rsfa {
namespace {

constexpr int kD = 256;
constexpr int kRows = 128;      // Q rows per CTA (= TMEM lanes)
constexpr int kKeys = 64;       // keys per K/V tile
constexpr int kThreads256 = 192;
constexpr int kTmaWarp256 = 4;
constexpr int kMmaWarp256 = 5;
constexpr int kStages256 = 4;
constexpr int kBoxes256 = kD / 64;
constexpr int kQBoxBytes256 = kRows * 128;           // 16 KB
constexpr int kQBytes256 = kBoxes256 * kQBoxBytes256; // 64 KB
constexpr int kKvBoxBytes256 = kKeys * 128;          // 8 KB
constexpr int kKvBytes256 = kBoxes256 * kKvBoxBytes256;  // 32 KB
constexpr int kColS256 = 0;     // S[b] at kColS256 + 64 * b
constexpr int kColO256 = 128;
constexpr int kNumBarriers256 = 2 + 2 * kStages256 + 2 + 2 + 2 + 4;
constexpr int kSmemBytes256 = kQBytes256 + kStages256 * kKvBytes256 + 1024 + kNumBarriers256 * 8 + 64;

__device__ __forceinline__ int num_kv_tiles_256(int row0, int S, int causal) {
  if (row0 >= S) return 0;
  const int last_key = causal ? min(S, row0 + kRows) : S;  // exclusive
  return (last_key + kKeys - 1) / kKeys;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads256, 1)
fwd_tcgen05_d256_kernel(const __grid_constant__ TmaMaps maps, const FwdParams p, const SchedInfo sched) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sKV = sQ + kQBytes256;
  const uint32_t sBar = sKV + kStages256 * kKvBytes256;
  const uint32_t bar_q_full = sBar;
  const uint32_t bar_q_empty = sBar + 8u;
  auto bar_kv_full = [&](int s) { return sBar + 8u * (2 + s); };
  auto bar_kv_empty = [&](int s) { return sBar + 8u * (2 + kStages256 + s); };
  auto bar_s_full = [&](int b) { return sBar + 8u * (2 + 2 * kStages256 + b); };
  auto bar_p_full = [&](int b) { return sBar + 8u * (4 + 2 * kStages256 + b); };
  const uint32_t bar_pv_done = sBar + 8u * (6 + 2 * kStages256);   // one completion per key tile
  const uint32_t bar_o_full = bar_pv_done + 8u;                    // one completion per work item
  const uint32_t bar_sched_full0 = bar_o_full + 8u;                // 2 slots
  const uint32_t bar_sched_empty0 = bar_sched_full0 + 16u;         // 2 slots
  const uint32_t misc = sBar + 8u * kNumBarriers256;
  uint8_t* misc_ptr = smem_raw + (misc - smem_u32(smem_raw));
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc_ptr);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc_ptr + 4);
  volatile int* sched_ring = reinterpret_cast<volatile int*>(misc_ptr + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t wait_ns = p.wait_limit_ns;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    for (int s = 0; s < kStages256; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_s_full(b), 1);
      mbar_init(bar_p_full(b), kRows);
      mbar_init(bar_sched_full0 + 8u * b, 1);
      mbar_init(bar_sched_empty0 + 8u * b, 1 + 4);  // MMA lane + one lane per softmax warp
    }
    mbar_init(bar_pv_done, 1);
    mbar_init(bar_o_full, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kMmaWarp256) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), 512);
    tmem_relinquish();
  }
  if (warp == kTmaWarp256 && lane == 0) {
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int S = p.S;
  const int items_per_head = sched.items_per_head;
  auto decode = [&](int item, int& bh, int& row0) {
    bh = item / items_per_head;
    int blk = item - bh * items_per_head;
    if (p.causal) blk = items_per_head - 1 - blk;   // heaviest block first inside a head
    row0 = blk * kRows;
  };

  if (warp == kTmaWarp256) {
    // ================================================================ producer
    // Ring order = consumption order of the MMA warp: K_0, K_1, then V_j, K_{j+2} for j = 0, 1, ...
    if (lane == 0) {
      uint32_t kv_count = 0, item_count = 0;
      bool ok = true;
      while (ok) {
        const int slot = item_count & 1;
        ok = mbar_wait(bar_sched_empty0 + 8u * slot, ((item_count >> 1) & 1) ^ 1, abort_flag, wait_ns, kTagSched);
        if (!ok) break;
        const int item = static_cast<int>(atomicAdd(p.tile_counter, 1u));
        sched_ring[slot] = item;
        __threadfence_block();
        mbar_arrive(bar_sched_full0 + 8u * slot);
        if (item >= sched.total_items) break;
        int bh, row0;
        decode(item, bh, row0);
        const int b = bh / p.H, h = bh - b * p.H;
        const int n = num_kv_tiles_256(row0, S, p.causal);
        auto load_kv = [&](const CUtensorMap* map, int j) -> bool {
          const uint32_t s = kv_count % kStages256;
          const uint32_t ph = (kv_count / kStages256) & 1;
          if (!mbar_wait(bar_kv_empty(s), ph ^ 1, abort_flag, wait_ns, kTagKvEmpty)) return false;
          mbar_arrive_expect_tx(bar_kv_full(s), kKvBytes256);
          for (int bx = 0; bx < kBoxes256; ++bx)
            tma_load_4d(sKV + s * kKvBytes256 + bx * kKvBoxBytes256, map, bar_kv_full(s), bx * 64, j * kKeys, h, b);
          ++kv_count;
          return true;
        };
        // K_0 (and K_1) before Q: their slots free up while the previous item drains.
        ok = load_kv(&maps.k, 0);
        if (ok && n > 1) ok = load_kv(&maps.k, 1);
        if (ok) ok = mbar_wait(bar_q_empty, (item_count & 1) ^ 1, abort_flag, wait_ns, kTagQEmpty);
        if (ok) {
          mbar_arrive_expect_tx(bar_q_full, kQBytes256);
          for (int bx = 0; bx < kBoxes256; ++bx)
            tma_load_4d(sQ + bx * kQBoxBytes256, &maps.q, bar_q_full, bx * 64, row0, h, b);
        }
        for (int j = 0; ok && j < n; ++j) {
          ok = load_kv(&maps.v, j);
          if (ok && j + 2 < n) ok = load_kv(&maps.k, j + 2);
        }
        ++item_count;
      }
    }
  } else if (warp == kMmaWarp256) {
    // ============================================================== MMA issuer
    {
      // Every lane runs this role with identical control flow; only the tcgen05 instructions are
      // issued by one elected lane.
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      auto wait_all = [&](uint32_t bar, uint32_t parity, int tag) -> bool {
        const bool r = mbar_wait(bar, parity, abort_flag, wait_ns, tag);
        return __all_sync(0xffffffffu, r) != 0;
      };
      constexpr uint32_t idesc_qk = make_idesc_f16(kRows, kKeys, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(kRows, kD, kBf16, false, true);
      const uint64_t desc_q0 = make_smem_desc_sw128(sQ, 16, 1024);
      const uint64_t desc_k0 = make_smem_desc_sw128(sKV, 16, 1024);
      const uint64_t desc_v0 = make_smem_desc_sw128(sKV, kKvBoxBytes256, 1024);
      RSFA_TRACE_DECL(2);
      uint32_t kv_count = 0, item_count = 0;
      uint32_t p_count[2] = {0, 0};
      bool ok = true;
      while (ok) {
        const int slot = item_count & 1;
        ok = wait_all(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, kTagSched);
        if (!ok) break;
        const int item = __shfl_sync(0xffffffffu, sched_ring[slot], 0);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sched_empty0 + 8u * slot);
        if (item >= sched.total_items) break;
        int bh, row0;
        decode(item, bh, row0);
        const int n = num_kv_tiles_256(row0, S, p.causal);

        // S[buf] = Q K^T: K-major operands; 16 elements of D per step = 32 B inside a swizzle row,
        // four steps per 64-column box.
        auto issue_qk = [&](int buf, uint32_t kslot) {
          const uint64_t kd = desc_k0 + static_cast<uint64_t>((kslot * kKvBytes256) >> 4);
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks) {
            const uint32_t off_q = ((ks >> 2) * kQBoxBytes256 + (ks & 3) * 32) >> 4;
            const uint32_t off_k = ((ks >> 2) * kKvBoxBytes256 + (ks & 3) * 32) >> 4;
            umma_ss_elect(tmem_u + kColS256 + 64 * buf, desc_q0 + off_q, kd + off_k, idesc_qk, ks > 0 ? 1u : 0u);
          }
        };
        // O (+)= P V: A = P in TMEM (8 columns per 16 keys), B = V MN-major, N = 256 spans the four
        // 64-column boxes (kKvBoxBytes256 apart), 16 keys = two 8-row atoms of 1024 B.
        auto issue_pv = [&](int buf, uint32_t vslot, bool accumulate) {
          const uint64_t vd = desc_v0 + static_cast<uint64_t>((vslot * kKvBytes256) >> 4);
#pragma unroll
          for (int ks = 0; ks < kKeys / 16; ++ks) {
            umma_ts_elect(tmem_u + kColO256, tmem_u + kColS256 + 64 * buf + ks * 8, vd + ((ks * 2048) >> 4),
                    idesc_pv, (accumulate || ks > 0) ? 1u : 0u);
          }
        };
        auto wait_kv = [&](uint32_t idx) -> bool {
          return wait_all(bar_kv_full(idx % kStages256), (idx / kStages256) & 1, kTagKvFull);
        };

        ok = wait_all(bar_q_full, item_count & 1, kTagQFull);
        if (!ok) break;
        uint32_t idx = kv_count;       // next ring entry to consume
        // prologue: S[0] = Q K_0^T, S[1] = Q K_1^T
        for (int j = 0; ok && j < 2 && j < n; ++j) {
          ok = wait_kv(idx);
          if (!ok) break;
          tc_fence_after_sync();
          issue_qk(j, idx % kStages256);
          umma_commit_elect(bar_s_full(j));
          umma_commit_elect(bar_kv_empty(idx % kStages256));
          ++idx;
        }
        if (!ok) break;
        if (n <= 2) umma_commit_elect(bar_q_empty);   // Q is dead after its last QK^T
        for (int j = 0; ok && j < n; ++j) {
          const int buf = j & 1;
          ok = wait_kv(idx);                     // V_j
          if (!ok) break;
          RSFA_TRACE_EV(0x6000 + j);   // V present
          ok = wait_all(bar_p_full(buf), p_count[buf] & 1, kTagPFull);
          if (!ok) break;
          ++p_count[buf];
          tc_fence_after_sync();
          RSFA_TRACE_EV(0x1000 + j);   // P seen
          issue_pv(buf, idx % kStages256, j > 0);
          RSFA_TRACE_EV(0x2000 + j);   // PV issued
          umma_commit_elect(bar_pv_done);
          umma_commit_elect(bar_kv_empty(idx % kStages256));
          if (j == n - 1) umma_commit_elect(bar_o_full);
          ++idx;
          if (j + 2 < n) {
            ok = wait_kv(idx);                   // K_{j+2}
            if (!ok) break;
            tc_fence_after_sync();
            RSFA_TRACE_EV(0x3000 + j);   // K(j+2) present
            issue_qk(buf, idx % kStages256);     // S[buf] is free: PV_j above consumed P_j in order
            RSFA_TRACE_EV(0x5000 + j);   // QK(j+2) issued
            umma_commit_elect(bar_s_full(buf));
            umma_commit_elect(bar_kv_empty(idx % kStages256));
            if (j + 3 == n) umma_commit_elect(bar_q_empty);
            ++idx;
          }
        }
        if (!ok) break;
        kv_count = idx;
        ++item_count;
      }
    }
  } else {
    // ========================================================== softmax warps
    const int row_in_tile = warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + kColO256;
    const float scale_log2 = p.sm_scale * kLog2e;
    uint32_t item_count = 0, o_count = 0, pv_count = 0;
    uint32_t s_count[2] = {0, 0};
    bool ok = true;
#ifdef RSFA_TRACE
    unsigned long long* trace_buf = (p.trace != nullptr && blockIdx.x == 0 && warp == 0 && lane == 0) ? p.trace : nullptr;
    int trace_n = 0;
#endif
    while (ok) {
      const int slot = item_count & 1;
      ok = mbar_wait(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, abort_flag, wait_ns, kTagSched);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int item = sched_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sched_empty0 + 8u * slot);
      if (item >= sched.total_items) break;
      ++item_count;
      int bh, row0;
      decode(item, bh, row0);
      const int row = row0 + row_in_tile;
      const int n = num_kv_tiles_256(row0, S, p.causal);

      float m_used = -INFINITY;
      float l = 0.f;
      for (int j = 0; j < n; ++j) {
        const int buf = j & 1;
        const uint32_t tS = tmem_base + lane_base + kColS256 + 64 * buf;
        ok = mbar_wait(bar_s_full(buf), s_count[buf] & 1, abort_flag, wait_ns, kTagSFull);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_count[buf];
        tc_fence_after_sync();
        RSFA_TRACE_EV(0x1000 + j);   // S seen

        uint32_t s0[32], s1[32];
        tmem_ld_x32(tS + 0, s0);
        tmem_ld_x32(tS + 32, s1);
        tmem_wait_ld();
        reg_fence_x32(s0);
        reg_fence_x32(s1);

        const int n0 = j * kKeys;
        const bool masked = (n0 + kKeys > S) || (p.causal && n0 + kKeys > row0 + 1);
        if (masked) {
          int limit = S - 1 - n0;
          if (p.causal) limit = min(limit, row - n0);
          const uint32_t ninf = 0xff800000u;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c > limit) s0[c] = ninf;
            if (c + 32 > limit) s1[c] = ninf;
          }
        }
        float mb;
        {
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            mx[0] = max3(mx[0], __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
            mx[1] = max3(mx[1], __uint_as_float(s0[c + 2]), __uint_as_float(s0[c + 3]));
            mx[2] = max3(mx[2], __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
            mx[3] = max3(mx[3], __uint_as_float(s1[c + 2]), __uint_as_float(s1[c + 3]));
          }
          mb = fmaxf(max3(mx[0], mx[1], mx[2]), mx[3]);
        }
        // With 64-key tiles the upper rows of the Q tile see nothing of the second diagonal tile:
        // such a row keeps its reference max (moving it towards 0 could underflow l).
        const bool nothing_visible = (mb == -INFINITY);

        float alpha = 1.f;
        bool grow = false;
        if (j == 0) {
          m_used = nothing_visible ? 0.f : mb;
        } else if (!nothing_visible && (mb - m_used) * scale_log2 > kRescaleThreshold) {
          alpha = ex2((m_used - mb) * scale_log2);
          l *= alpha;
          m_used = mb;
          grow = true;
        }
        if (__any_sync(0xffffffffu, grow)) {
          // Unlike the two-tile kernel, QK^T of this tile was issued before PV of the previous one,
          // so O may still be written: wait for PV_{j-1} (completion number pv_count + j - 1).
          ok = mbar_wait(bar_pv_done, (pv_count + j - 1) & 1, abort_flag, wait_ns, kTagOFull);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll 1
          for (int c0 = 0; c0 < kD; c0 += 32) {
            uint32_t o[32];
            tmem_ld_x32(tO + c0, o);
            tmem_wait_ld();
            reg_fence_x32(o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            tmem_st_x32(tO + c0, o);
          }
        }

        RSFA_TRACE_EV(0x3000 + j);   // max done
        const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
        const float neg_m = -m_used * scale_log2;
        const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
        uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
        uint32_t pk[32];   // all 64 keys are packed first, then stored with one tcgen05.st
        auto exp_pack = [&](uint32_t (&sv)[32], int base) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            float x0, x1, x2, x3;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, neg_m2), x0, x1);
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3])), scale2, neg_m2), x2, x3);
            const float e0 = ex2(x0), e1 = ex2(x1), e2 = ex2(x2), e3 = ex2(x3);
            sum_a = add_f32x2(sum_a, pack_f32x2(e0, e1));
            sum_b = add_f32x2(sum_b, pack_f32x2(e2, e3));
            pk[base + (c >> 1)] = pack2<kBf16>(e0, e1);
            pk[base + (c >> 1) + 1] = pack2<kBf16>(e2, e3);
          }
        };
        exp_pack(s0, 0);
        exp_pack(s1, 16);
        tmem_st_x32(tS, pk);
        {
          float a0, a1;
          unpack_f32x2(add_f32x2(sum_a, sum_b), a0, a1);
          l += a0 + a1;
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar_p_full(buf));
        RSFA_TRACE_EV(0x5000 + j);   // P handed over
      }
      if (!ok) break;
      pv_count += n;

      // ---- epilogue
      ok = mbar_wait(bar_o_full, o_count & 1, abort_flag, wait_ns, kTagOFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ++o_count;
      tc_fence_after_sync();
      RSFA_TRACE_EV(0x6000);   // O seen
      const float inv_l = 1.f / l;
      const int b = bh / p.H, h = bh - b * p.H;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1] +
                       static_cast<int64_t>(row) * p.o_stride[2];
#pragma unroll 1
      for (int c0 = 0; c0 < kD; c0 += 32) {
        uint32_t o[32];
        tmem_ld_x32(tO + c0, o);
        tmem_wait_ld();
        reg_fence_x32(o);
        if (row < S) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 v4;
            v4.x = pack2<kBf16>(__uint_as_float(o[c + 0]) * inv_l, __uint_as_float(o[c + 1]) * inv_l);
            v4.y = pack2<kBf16>(__uint_as_float(o[c + 2]) * inv_l, __uint_as_float(o[c + 3]) * inv_l);
            v4.z = pack2<kBf16>(__uint_as_float(o[c + 4]) * inv_l, __uint_as_float(o[c + 5]) * inv_l);
            v4.w = pack2<kBf16>(__uint_as_float(o[c + 6]) * inv_l, __uint_as_float(o[c + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c0 + c) = v4;
          }
        }
      }
      if (p.lse != nullptr && row < S)
        p.lse[static_cast<int64_t>(bh) * S + row] = m_used * p.sm_scale + logf(l);
      tc_fence_before_sync();
      RSFA_TRACE_EV(0x7000);   // epilogue done
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == kMmaWarp256) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(p.status, 0, *abort_flag);
}

template <bool kBf16>
cudaError_t launch_d256(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  TmaMaps maps;
  if (!make_map(&maps.q, p.q, p, p.q_stride, kRows) || !make_map(&maps.k, p.k, p, p.k_stride, kKeys) ||
      !make_map(&maps.v, p.v, p, p.v_stride, kKeys))
    return cudaErrorInvalidValue;
  SchedInfo sched;
  sched.items_per_head = (p.S + kRows - 1) / kRows;
  sched.total_items = sched.items_per_head * p.B * p.H;
  auto kern = fwd_tcgen05_d256_kernel<kBf16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes256);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(p.tile_counter, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return e;
  const int grid = sched.total_items < sm_count ? sched.total_items : sm_count;
  kern<<<grid, kThreads256, kSmemBytes256, stream>>>(maps, p, sched);
  e = cudaGetLastError();
  if (e == cudaSuccess) *launches += 1;
  return e;
}

}  // namespace

cudaError_t launch_fwd_tcgen05_d256(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  return p.bf16 ? launch_d256<true>(p, sm_count, stream, launches) : launch_d256<false>(p, sm_count, stream, launches);
}

}  // namespace rsfa
