// FlashAttention-2 forward for B200 (sm_100a), head dimension 64: "separate P" kernel.
//
// It replaces the reference's D = 64 specialisation _attn_fwd_inner_d64_nc
// (ascend_rsfa/flash_attention_forward.py:229-267, selected at :375-382) and the generic loop
// _attn_fwd_inner (:163-226) / the causal split (:408-541) for D = 64.
//
// At D = 64 the exponentials, not the MMAs, bound a 128 x 128 tile (MUFU 1024 clk, tensor pipe
// 640), and tensor memory has 128 columns to spare: two S tiles (256) and two O tiles (128) leave
// room for P in columns of its own.  S_t is then free again as soon as the softmax warps have
// loaded it into registers, so the MMA warp computes S_t(j+1) while the softmax of tile j is still
// running: the softmax -> PV -> QK^T(next) chain with its hand-over latencies (about 1300 clk per
// tile and step at this size) is off the softmax warps' critical path and they run back to back.
//
// Roles (384 threads): warps 0..3 softmax of Q tile 0, 4..7 softmax of Q tile 1 (one thread per
// row), warp 8 TMA producer, warps 9 and 10 MMA issuers of Q tile 0 and 1, warp 11 idle.
// TMEM columns: S_0 [0,128)  S_1 [128,256)  O_0 [256,320)  O_1 [320,384)  P_0 [384,448)  P_1 [448,512).
// Per key tile j (128 keys) and Q tile t:
//   S_t = Q_t K_j^T          4 MMAs 128 x 128 x 16, operands in shared memory
//   softmax group t          tcgen05.ld S_t, release S_t, exp2 against the row's reference, row
//                            sum, sum check, wait until PV of tile j-1 has read P_t, tcgen05.st P_t
//   O_t += P_t V_j           8 MMAs 128 x 64 x 16, A = P_t from TMEM, B = V_j MN-major
// The softmax keeps no per-tile row maximum (see softmax_half_careful in tcgen05_common.cuh for
// the scheme): P is taken against a reference fixed at the first key tile, and a check of each
// tile's row sums says whether a P value may have left the 16-bit range.  Because S_t is gone by
// the time that check can fail, the fast loop cannot repair a tile.  A work item with a failed
// check is therefore run a second time by the same CTA, as its next item (only the Q tile whose
// check failed: the other one's rows are right and written), with the "safe" loop:
// that one checks each 64-key half while its scores are still in registers and, when a half is
// over the limit, moves the rows' reference up by a whole number of binary orders and brings l,
// the tile's first half and O_t along (about a sixth slower per step, so it is not the default).
// A CTA that has had to repeat more than one item in kBailOneIn stops trying the fast loop.
// Everything is local to the CTA: no list in global memory, no second launch.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "../../include/rsfa.h"
#include "tcgen05_common.cuh"

namespace rsfa {
namespace {

constexpr int kD = 64;
constexpr int kRows = 128;     // rows per Q tile (= TMEM lanes)
constexpr int kKeys = 128;     // keys per K/V tile
constexpr int kTiles = 2;      // Q tiles per CTA
constexpr int kThreadsSp = 384;
constexpr int kTmaWarpSp = 8;
constexpr int kMmaWarpSp0 = 9;  // warps 9, 10: one issuer per Q tile
constexpr int kStagesSp = 6;
constexpr int kBailOneIn = 4;        // a CTA gives up on the fast loop when more than 1 item in 4 had to be repeated,
constexpr int kBailMin = 2;          // ... and at least this many were
// A work item in the scheduler ring: its number, a flag "run it with the safe loop", and with that flag the
// Q tiles to run (bit 28 + t): a repeat only runs the Q tile(s) whose check failed.
constexpr int kSafeItem = 1 << 30;
constexpr int kTileBit0 = 28;
// ... and a flag "fast loop, but only the Q tiles named": the halves of the items of a last, thin wave
constexpr int kMaskedItem = 1 << 27;
constexpr int kItemMask = kMaskedItem - 1;
constexpr int kQBytes = kRows * kD * 2;      // 16 KB
constexpr int kKvBytes = kKeys * kD * 2;     // 16 KB
constexpr int kStageBytesSp = kRows * 128;   // epilogue staging per Q tile: 128 rows x 64 columns
__host__ __device__ constexpr int kColS(int t) { return t * 128; }
__host__ __device__ constexpr int kColO(int t) { return 256 + t * kD; }
__host__ __device__ constexpr int kColP(int t) { return 384 + t * 64; }
// barriers: q_full, q_empty, s_full, s_free, p_full, p_free, o_full per tile; ring; scheduler
constexpr int kNumBarriersSp = 7 * kTiles + 2 * kStagesSp + 4;
constexpr int kSmemBytesSp = kTiles * kQBytes + kStagesSp * kKvBytes + kTiles * kStageBytesSp + 1024 +
                             kNumBarriersSp * 8 + 64;

__device__ __forceinline__ int num_kv_tiles_sp(int row0, int S, int causal) {
  if (row0 >= S) return 0;
  const int last_key = causal ? min(S, row0 + kRows) : S;  // exclusive
  return (last_key + kKeys - 1) / kKeys;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreadsSp, 1)
fwd_tcgen05_sp_kernel(const __grid_constant__ TmaMaps maps, const FwdParams p, const SchedInfo sched) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles: 1024-byte alignment
  const uint32_t sQ = smem_base;
  const uint32_t sKV = sQ + kTiles * kQBytes;
  const uint32_t sStage = sKV + kStagesSp * kKvBytes;
  const uint32_t sBar = sStage + kTiles * kStageBytesSp;
  auto bar_q_full = [&](int t) { return sBar + 8u * t; };
  auto bar_q_empty = [&](int t) { return sBar + 8u * (kTiles + t); };
  auto bar_s_full = [&](int t) { return sBar + 8u * (2 * kTiles + t); };
  auto bar_s_free = [&](int t) { return sBar + 8u * (3 * kTiles + t); };
  auto bar_p_full = [&](int t) { return sBar + 8u * (4 * kTiles + t); };
  auto bar_p_free = [&](int t) { return sBar + 8u * (5 * kTiles + t); };
  auto bar_o_full = [&](int t) { return sBar + 8u * (6 * kTiles + t); };
  auto bar_kv_full = [&](int s) { return sBar + 8u * (7 * kTiles + s); };
  auto bar_kv_empty = [&](int s) { return sBar + 8u * (7 * kTiles + kStagesSp + s); };
  const uint32_t bar_sched_full0 = sBar + 8u * (7 * kTiles + 2 * kStagesSp);   // 2 slots
  const uint32_t bar_sched_empty0 = bar_sched_full0 + 16u;                     // 2 slots
  const uint32_t misc = sBar + 8u * kNumBarriersSp;
  // misc words: [0] TMEM base, [1] abort flag, [2..3] scheduler ring, [4..5] Q tiles (bit t) of this ring
  // slot's item that failed a sum check (set by their softmax warps before they give the slot back)
  uint8_t* misc_ptr = smem_raw + (misc - smem_u32(smem_raw));
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc_ptr);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc_ptr + 4);
  volatile int* sched_ring = reinterpret_cast<volatile int*>(misc_ptr + 8);
  volatile int* item_failed = reinterpret_cast<volatile int*>(misc_ptr + 16);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t wait_ns = p.wait_limit_ns;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    item_failed[0] = 0;
    item_failed[1] = 0;
    for (int t = 0; t < kTiles; ++t) {
      mbar_init(bar_q_full(t), 1);
      mbar_init(bar_q_empty(t), 1);
      mbar_init(bar_s_full(t), 1);
      mbar_init(bar_s_free(t), 4);        // one lane of each softmax warp of the tile
      mbar_init(bar_p_full(t), kRows);
      mbar_init(bar_p_free(t), 1);
      mbar_init(bar_o_full(t), 1);
    }
    for (int s = 0; s < kStagesSp; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), kTiles);  // both MMA warps release a slot
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sched_full0 + 8u * s, 1);
      // the MMA warps give a slot back when they have read it, the softmax warps (one lane each) only
      // when they are done with the item: a free slot means that its item's sum checks are known
      mbar_init(bar_sched_empty0 + 8u * s, kTiles + kTiles * 4);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kMmaWarpSp0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), 512);
    tmem_relinquish();
  }
  if (warp == kTmaWarpSp && lane == 0) {
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    tma_prefetch_desc(&maps.o);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  // Only this CTA's shared and tensor memory so far; global memory waits for what is in front on the stream.
  griddep_wait();

  const int S = p.S;
  // work item -> (head, first row).  Causal: heaviest (last) row block first.
  auto decode = [&](int item, int& bh, int& row0) {
    int blk;
    sched_decode(sched, p.causal, item, bh, blk);
    row0 = blk * (kTiles * kRows);
  };

  // setmaxnreg is warpgroup-aligned: every warp of a warpgroup must execute the SAME instruction,
  // so the third warpgroup lowers its budget before it splits into roles.
  if (warp >= kTmaWarpSp) {
    setmaxnreg_dec<RegBudget<kD>::kOther>();
    if (warp == kTmaWarpSp) {
      // ================================================================ producer
      if (lane == 0) {
        uint32_t kv_count = 0, item_count = 0;
        int dispatched[2] = {0, 0};        // item of each ring slot
        int n_fast = 0, n_failed = 0;      // items tried with the fast loop / of those, repeated
        bool queue_empty = false;
        bool ok = true;
        while (ok) {
          const int slot = item_count & 1;
          ok = mbar_wait(bar_sched_empty0 + 8u * slot, ((item_count >> 1) & 1) ^ 1, abort_flag, wait_ns, kTagSched);
          if (!ok) break;
          // The item that had this slot (two items ago) is finished.  If one of its sum checks failed,
          // it is the next item, with the safe loop; else the queue's next one (the first item of a CTA
          // is its own index: grid <= number of items), fast unless this CTA has given up on that.
          int item = sched.total_items;
          auto take_failed = [&](int sl) {
            const int tiles = item_failed[sl];
            if (tiles != 0) {
              item_failed[sl] = 0;
              ++n_failed;
              item = dispatched[sl] | kSafeItem | (tiles << kTileBit0);
            }
          };
          if (item_count >= 2) take_failed(slot);
          if (item == sched.total_items && !queue_empty) {
            // the queue counts whole items first, then two halves for each of the last split_items items
            const int q = (item_count == 0) ? static_cast<int>(blockIdx.x)
                                            : static_cast<int>(atomicAdd(p.tile_counter, 1u) + gridDim.x);
            const int n_whole = sched.total_items - sched.split_items;
            if (q >= sched.total_items + sched.split_items) {
              queue_empty = true;
              griddep_launch_dependents();   // the queue is empty: the kernel behind this one may set up
            } else {
              int tiles = (1 << kTiles) - 1;
              item = q;
              if (q >= n_whole) {
                item = n_whole + ((q - n_whole) >> 1);
                tiles = 1 << ((q - n_whole) & 1);
              }
              if (n_failed >= kBailMin && n_failed * kBailOneIn > n_fast) {
                item |= kSafeItem | (tiles << kTileBit0);
              } else {
                if (q >= n_whole) item |= kMaskedItem | (tiles << kTileBit0);
                ++n_fast;
              }
            }
          }
          if (item == sched.total_items && item_count >= 1) {
            // Nothing left to hand out, but the item in the other slot is still running and may fail:
            // wait for it (the wait the next dispatch would have done) before the CTA is told to leave.
            ok = mbar_wait(bar_sched_empty0 + 8u * (slot ^ 1), (((item_count + 1) >> 1) & 1) ^ 1, abort_flag, wait_ns,
                           kTagSched);
            if (!ok) break;
            take_failed(slot ^ 1);
          }
          dispatched[slot] = item & kItemMask;
          sched_ring[slot] = item;
          __threadfence_block();
          mbar_arrive(bar_sched_full0 + 8u * slot);
          if (item == sched.total_items) break;
          int bh, row0;
          decode(item & kItemMask, bh, row0);
          const int b = bh / p.H, h = bh - b * p.H;
          int nmax = 0;
          for (int t = 0; t < kTiles; ++t) nmax = max(nmax, num_kv_tiles_sp(row0 + t * kRows, S, p.causal));
          auto load_q = [&](int t) -> bool {
            if (!mbar_wait(bar_q_empty(t), (item_count & 1) ^ 1, abort_flag, wait_ns, kTagQEmpty)) return false;
            mbar_arrive_expect_tx(bar_q_full(t), kQBytes);
            tma_load_4d(sQ + t * kQBytes, &maps.q, bar_q_full(t), 0, row0 + t * kRows, h, b);
            return true;
          };
          auto load_kv = [&](const CUtensorMap* map, int j) -> bool {
            const uint32_t s = kv_count % kStagesSp;
            const uint32_t ph = (kv_count / kStagesSp) & 1;
            if (!mbar_wait(bar_kv_empty(s), ph ^ 1, abort_flag, wait_ns, kTagKvEmpty)) return false;
            mbar_arrive_expect_tx(bar_kv_full(s), kKvBytes);
            tma_load_4d(sKV + s * kKvBytes, map, bar_kv_full(s), 0, j * kKeys, h, b);
            ++kv_count;
            return true;
          };
          // K_0 / V_0 first: their ring slots free up while the previous item drains, whereas the
          // Q buffers are released only once that item's last QK^T MMA has finished.
          if (nmax > 0) ok = load_kv(&maps.k, 0);
          if (ok && nmax > 0) ok = load_kv(&maps.v, 0);
          for (int t = 0; ok && t < kTiles; ++t) ok = load_q(t);
          for (int j = 1; ok && j < nmax; ++j) {
            ok = load_kv(&maps.k, j);
            if (ok) ok = load_kv(&maps.v, j);
          }
          ++item_count;
        }
      }
    } else if (warp < kMmaWarpSp0 + kTiles) {
      // ============================================================ MMA issuers, one warp per Q tile
      // Every lane runs this role with identical control flow; only the tcgen05 instructions are
      // issued by one elected lane.  Both warps walk the same ring entries; a slot is free again
      // when both have committed it.
      const int t = warp - kMmaWarpSp0;
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      auto wait_all = [&](uint32_t bar, uint32_t parity, int tag) -> bool {
        return mbar_wait_warp(bar, parity, abort_flag, wait_ns, tag);
      };
      constexpr uint32_t idesc_qk = make_idesc_f16(kRows, kKeys, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(kRows, kD, kBf16, false, true);
      const uint64_t desc_q = make_smem_desc_sw128(sQ + t * kQBytes, 16, 1024);
      const uint64_t desc_k0 = make_smem_desc_sw128(sKV, 16, 1024);
      const uint64_t desc_v0 = make_smem_desc_sw128(sKV, kKvBytes, 1024);
      uint32_t kv_count = 0, item_count = 0;
      uint32_t sf_count = 0, p_count = 0;   // phases of s_free / p_full of this tile: one per key tile
      bool ok = true;
      while (ok) {
        const int slot = item_count & 1;
        ok = wait_all(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, kTagSched);
        if (!ok) break;
        const int entry = __shfl_sync(0xffffffffu, sched_ring[slot], 0);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sched_empty0 + 8u * slot);
        if (entry == sched.total_items) break;
        const int item = entry & kItemMask;   // fast or safe: the same MMAs
        // a repeat may leave this Q tile out: it then only gives its operands back
        const bool tile_runs = (entry & (kSafeItem | kMaskedItem)) == 0 || ((entry >> (kTileBit0 + t)) & 1) != 0;
        int bh, row0;
        decode(item, bh, row0);
        int nmax = 0;
        for (int tt = 0; tt < kTiles; ++tt) nmax = max(nmax, num_kv_tiles_sp(row0 + tt * kRows, S, p.causal));
        const int n = tile_runs ? num_kv_tiles_sp(row0 + t * kRows, S, p.causal) : 0;
        // S_t = Q_t K^T: both operands K-major in one 64-column box; 16 elements of D per step
        // = 32 B inside the 128-byte swizzle row.
        // MMAs and the commits behind them go out from ONE elected region (an elect.sync and a
        // branch per instruction cost the warp more than the instruction); commit = 0: none.
        auto issue_qk = [&](uint32_t kslot, uint32_t commit_a, uint32_t commit_b) {
          const uint64_t kd = desc_k0 + static_cast<uint64_t>((kslot * kKvBytes) >> 4);
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < kD / 16; ++ks)
              umma_ss(tmem_u + kColS(t), desc_q + ((ks * 32) >> 4), kd + ((ks * 32) >> 4), idesc_qk, ks > 0 ? 1u : 0u);
            if (commit_a != 0) umma_commit(commit_a);
            if (commit_b != 0) umma_commit(commit_b);
          }
          __syncwarp();
        };
        // O_t (+)= P_t V: A = P_t in TMEM (16 keys = 8 columns per step), B = V MN-major:
        // 16 keys per step = two 8-row atoms of 1024 B.
        auto issue_pv = [&](uint32_t vslot, bool accumulate, uint32_t commit_a, uint32_t commit_b) {
          const uint64_t vd = desc_v0 + static_cast<uint64_t>((vslot * kKvBytes) >> 4);
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < kKeys / 16; ++ks)
              umma_ts(tmem_u + kColO(t), tmem_u + kColP(t) + ks * 8, vd + ((ks * 2048) >> 4), idesc_pv,
                      (accumulate || ks > 0) ? 1u : 0u);
            if (commit_a != 0) umma_commit(commit_a);
            if (commit_b != 0) umma_commit(commit_b);
          }
          __syncwarp();
        };
        auto wait_kv = [&](uint32_t idx) -> bool {
          return wait_all(bar_kv_full(idx % kStagesSp), (idx / kStagesSp) & 1, kTagKvFull);
        };

        ok = wait_all(bar_q_full(t), item_count & 1, kTagQFull);
        if (!ok) break;
        const uint32_t base = kv_count;   // K_j at base + 2j, V_j at base + 2j + 1
        if (nmax > 0) {
          ok = wait_kv(base);
          if (!ok) break;
          tc_fence_after_sync();
          // S_t is free: the previous item's last P was produced after its S had been read.
          if (n > 0)
            issue_qk(base % kStagesSp, bar_s_full(t), n <= 1 ? bar_q_empty(t) : 0u);
          else
            umma_commit_elect(bar_q_empty(t));
          umma_commit_elect(bar_kv_empty(base % kStagesSp));
        }
        for (int j = 0; ok && j < nmax; ++j) {
          const uint32_t vidx = base + 2 * j + 1;
          const uint32_t kidx = base + 2 * j + 2;
          // next S first: it only needs the softmax warps to have loaded S_t(j)
          if (j + 1 < nmax) {
            ok = wait_kv(kidx);
            if (!ok) break;
            if (j + 1 < n) {
              ok = wait_all(bar_s_free(t), (sf_count + j) & 1, kTagSFull);
              if (!ok) break;
              tc_fence_after_sync();
              issue_qk(kidx % kStagesSp, bar_s_full(t), j + 2 == n ? bar_q_empty(t) : 0u);
            }
            umma_commit_elect(bar_kv_empty(kidx % kStagesSp));
          }
          ok = wait_kv(vidx);
          if (!ok) break;
          if (j < n) {
            ok = wait_all(bar_p_full(t), (p_count + j) & 1, kTagPFull);
            if (!ok) break;
            tc_fence_after_sync();
            issue_pv(vidx % kStagesSp, j > 0, bar_p_free(t), j == n - 1 ? bar_o_full(t) : 0u);
          }
          umma_commit_elect(bar_kv_empty(vidx % kStagesSp));
        }
        if (!ok) break;
        kv_count += 2 * nmax;
        sf_count += n;
        p_count += n;
        ++item_count;
      }
    }
  } else {
    // ========================================================== softmax groups
    setmaxnreg_inc<RegBudget<kD>::kSoftmax>();
    const int t = warp >> 2;                   // Q tile of this group
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + kColS(t);
    const uint32_t tO = tmem_base + lane_base + kColO(t);
    const uint32_t tP = tmem_base + lane_base + kColP(t);
    const float scale_log2 = p.sm_scale * kLog2e;
    const float headroom = kHeadroomLog2 / scale_log2;   // in raw score units (sm_scale > 0 on this path)
    uint32_t item_count = 0, s_count = 0, o_count = 0, pf_count = 0;
    bool ok = true;

    // One work item of this Q tile: key tiles, then the epilogue.  kSafe = false is the fast loop (one
    // sum check per key tile; returns true if one failed: the item's output is then undefined and the
    // item has to be run again), kSafe = true the loop that repairs a failed check in place.
    auto run_item = [&](auto safe_tag, int item) __attribute__((always_inline)) -> bool {
      constexpr bool kSafe = decltype(safe_tag)::value;
      int bh, row0;
      decode(item, bh, row0);
      const int tile_row0 = row0 + t * kRows;
      const int row = tile_row0 + row_in_tile;
      const int n_tiles = num_kv_tiles_sp(tile_row0, S, p.causal);
      if (n_tiles == 0) return false;

      // Row state: x = s * scale_log2 + neg_m is the exponent of a score against the row's reference
      // (first key tile's maximum + headroom; the safe loop moves it up when a check fails), l = sum of P.
      float neg_m = 0.f;
      float l = 0.f;
      bool overflow = false;
      for (int j = 0; j < n_tiles; ++j) {
        ok = mbar_wait_warp(bar_s_full(t), s_count & 1, abort_flag, wait_ns, kTagSFull);
        if (!ok) break;
        ++s_count;
        tc_fence_after_sync();

        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld_x32(tS + 0, s0);
        tmem_ld_x32(tS + 32, s1);
        tmem_ld_x32(tS + 64, s2);
        tmem_ld_x32(tS + 96, s3);
        tmem_wait_ld();
        reg_fence_x32(s0);
        reg_fence_x32(s1);
        reg_fence_x32(s2);
        reg_fence_x32(s3);
        // S_t is in registers: the MMA warp may compute the next one over it.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free(t));

        // masked tile: the one crossing the diagonal, or the ragged end of the sequence
        const int n0 = j * kKeys;
        const bool masked = (n0 + kKeys > S) || (p.causal && n0 + kKeys > tile_row0 + 1);
        if (masked) {
          int limit = S - 1 - n0;                           // last visible column of this tile
          if (p.causal) limit = min(limit, row - n0);
          const uint32_t ninf = 0xff800000u;
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (c > limit) s0[c] = ninf;
            if (c + 32 > limit) s1[c] = ninf;
            if (c + 64 > limit) s2[c] = ninf;
            if (c + 96 > limit) s3[c] = ninf;
          }
        }
        if (j == 0) {
          float mx[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) mx[i] = -INFINITY;
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            mx[0] = max3(mx[0], __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
            mx[1] = max3(mx[1], __uint_as_float(s0[c + 2]), __uint_as_float(s0[c + 3]));
            mx[2] = max3(mx[2], __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
            mx[3] = max3(mx[3], __uint_as_float(s1[c + 2]), __uint_as_float(s1[c + 3]));
            mx[4] = max3(mx[4], __uint_as_float(s2[c]), __uint_as_float(s2[c + 1]));
            mx[5] = max3(mx[5], __uint_as_float(s2[c + 2]), __uint_as_float(s2[c + 3]));
            mx[6] = max3(mx[6], __uint_as_float(s3[c]), __uint_as_float(s3[c + 1]));
            mx[7] = max3(mx[7], __uint_as_float(s3[c + 2]), __uint_as_float(s3[c + 3]));
          }
          float mb = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]));
          if (mb == -INFINITY) mb = 0.f;  // only rows past S can get here; keep them finite
          neg_m = -(mb + headroom) * scale_log2;
        }
        const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
        uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
        uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
        // exp2, row sum and 16-bit packing of 32 scores into pk[base .. base+16)
        auto exp_pack = [&](uint32_t (&sv)[32], uint32_t (&pk)[32], int base) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            const uint64_t xa = fma_f32x2(pack_f32x2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), scale2, neg_m2);
            const uint64_t xb = fma_f32x2(pack_f32x2(__uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3])), scale2, neg_m2);
            float x0, x1, x2, x3;
            unpack_f32x2(xa, x0, x1);
            unpack_f32x2(xb, x2, x3);
            const float e0 = ex2(x0), e1 = ex2(x1), e2 = ex2(x2), e3 = ex2(x3);
            sum_a = add_f32x2(sum_a, pack_f32x2(e0, e1));
            sum_b = add_f32x2(sum_b, pack_f32x2(e2, e3));
            pk[base + (c >> 1)] = pack2<kBf16>(e0, e1);
            pk[base + (c >> 1) + 1] = pack2<kBf16>(e2, e3);
          }
        };
        auto take_sum = [&]() -> float {
          float a0, a1;
          unpack_f32x2(add_f32x2(sum_a, sum_b), a0, a1);
          sum_a = pack_f32x2(0.f, 0.f);
          sum_b = sum_a;
          return a0 + a1;
        };
        uint32_t pk0[32], pk1[32];
        if constexpr (!kSafe) {
          exp_pack(s0, pk0, 0);
          exp_pack(s1, pk0, 16);
          exp_pack(s2, pk1, 0);
          exp_pack(s3, pk1, 16);
          const float h = take_sum();
          // Every P value is bounded by the sum; !(h <= limit) also catches NaN and +inf.
          if (__any_sync(0xffffffffu, !(h <= kSumLimit))) overflow = true;
          l += h;
        } else {
          // A half (64 keys) whose sum is over the limit may hold values beyond the 16-bit range.  Its
          // scores are still in registers: the rows concerned move their reference up by a whole
          // number of binary orders, so that the half's maximum sits `headroom` below it again; l,
          // this tile's first half (already packed: the factor is a power of two, so this is exact
          // short of underflow) and O_t follow, and the half is computed again.  Rows that were fine
          // go through it with a factor of one.  All 32 lanes run it together.
          auto repair = [&](uint32_t (&sx)[32], uint32_t (&sy)[32], uint32_t (&pk)[32], bool second, float& h_this,
                            float& h_first) -> bool {
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              mx[0] = max3(mx[0], __uint_as_float(sx[c]), __uint_as_float(sx[c + 1]));
              mx[1] = max3(mx[1], __uint_as_float(sx[c + 2]), __uint_as_float(sx[c + 3]));
              mx[2] = max3(mx[2], __uint_as_float(sy[c]), __uint_as_float(sy[c + 1]));
              mx[3] = max3(mx[3], __uint_as_float(sy[c + 2]), __uint_as_float(sy[c + 3]));
            }
            const float mb = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            float shift = 0.f;
            if (!(h_this <= kSumLimit)) shift = ceilf(fmaf(mb, scale_log2, neg_m) + kHeadroomLog2);
            if (!(shift >= 0.f)) shift = 0.f;   // NaN scores: nothing sensible to do, and nothing to get stuck in
            const float alpha = shift <= 126.f ? __int_as_float((127 - static_cast<int>(shift)) << 23) : 0.f;
            neg_m -= shift;
            neg_m2 = pack_f32x2(neg_m, neg_m);
            l *= alpha;
            if (second) {
              h_first *= alpha;
#pragma unroll
              for (int c = 0; c < 32; ++c) {
                float f0, f1;
                unpack2<kBf16>(pk0[c], f0, f1);
                pk0[c] = pack2<kBf16>(f0 * alpha, f1 * alpha);
              }
            }
            if (j > 0) {
              // O_t holds the key tiles before this one, complete once the PV MMAs of tile j-1 are
              if (!mbar_wait_warp(bar_p_free(t), (pf_count + j - 1) & 1, abort_flag, wait_ns, kTagPvDone)) return false;
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
            exp_pack(sx, pk, 0);
            exp_pack(sy, pk, 16);
            h_this = take_sum();
            return true;
          };
          exp_pack(s0, pk0, 0);
          exp_pack(s1, pk0, 16);
          float h0 = take_sum();
          if (__any_sync(0xffffffffu, !(h0 <= kSumLimit))) {
            float none = 0.f;
            ok = repair(s0, s1, pk0, false, h0, none);
            if (!ok) break;
          }
          exp_pack(s2, pk1, 0);
          exp_pack(s3, pk1, 16);
          float h1 = take_sum();
          if (__any_sync(0xffffffffu, !(h1 <= kSumLimit))) {
            ok = repair(s2, s3, pk1, true, h1, h0);
            if (!ok) break;
          }
          l += h0 + h1;
        }
        // P_t still belongs to the PV MMAs of the previous key tile until they have completed.
        if (j > 0) {
          ok = mbar_wait_warp(bar_p_free(t), (pf_count + j - 1) & 1, abort_flag, wait_ns, kTagPvDone);
          if (!ok) break;
          tc_fence_after_sync();
        }
        tmem_st_x32(tP, pk0);
        tmem_st_x32(tP + 32, pk1);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar_p_full(t));
      }
      if (!ok) return false;
      pf_count += n_tiles;

      // ---- epilogue: O_t / l -> global, lse = reference + log l
      ok = mbar_wait_warp(bar_o_full(t), o_count & 1, abort_flag, wait_ns, kTagOFull);
      if (!ok) return false;
      ++o_count;
      tc_fence_after_sync();
      const float inv_l = 1.f / l;
      const int b = bh / p.H, h = bh - b * p.H;
      // A repeated item writes the rows its first attempt wrote: those stores must have landed first.
      if (kSafe && lane == 0) tma_store_wait_all();
      // O_t / l -> global memory: each warp stages and stores its own 32 rows (store_o_rows)
      {
        const int wq = warp & 3;
        store_o_rows<kD, kBf16>(tO, inv_l, sStage + t * kStageBytesSp + wq * 4096, lane, &maps.o,
                                tile_row0 + wq * 32, h, b, tile_row0 + wq * 32 < S);
      }
      if (p.lse != nullptr && row < S)
        p.lse[static_cast<int64_t>(bh) * S + row] = -neg_m * kLn2 + logf(l);
      tc_fence_before_sync();
      return overflow;
    };

    while (ok) {
      const int slot = item_count & 1;
      ok = mbar_wait_warp(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, abort_flag, wait_ns, kTagSched);
      if (!ok) break;
      const int item = sched_ring[slot];
      if (item == sched.total_items) break;
      ++item_count;
      bool failed = false;
      if ((item & (kSafeItem | kMaskedItem)) == 0 || ((item >> (kTileBit0 + t)) & 1) != 0) {
        if ((item & kSafeItem) == 0)
          failed = run_item(std::false_type{}, item & kItemMask);
        else
          run_item(std::true_type{}, item & kItemMask);
      }
      if (!ok) break;
      // Done with the item: the ring slot goes back, with the news if this Q tile has to be run again.
      __syncwarp();
      if (lane == 0) {
        if (failed) atomicOr(const_cast<int*>(item_failed) + slot, 1 << t);
        mbar_arrive(bar_sched_empty0 + 8u * slot);
      }
    }
    if (lane == 0) tma_store_wait_all();   // the last TMA stores must be complete before the CTA exits
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag != 0) {
    // Give copies and MMAs still in flight time to land before shared memory and TMEM go away.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == kMmaWarpSp0) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0) {
    if (*abort_flag != 0) atomicCAS(p.status, 0, *abort_flag);
    queue_retire(p.tile_counter);
  }
}

}  // namespace

template <bool kBf16>
static cudaError_t launch_sp_one(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  TmaMaps maps;
  if (!make_map(&maps.q, p.q, p, p.q_stride, kRows) || !make_map(&maps.k, p.k, p, p.k_stride, kKeys) ||
      !make_map(&maps.v, p.v, p, p.v_stride, kKeys) || !make_map(&maps.o, p.o, p, p.o_stride, 32))
    return cudaErrorInvalidValue;
  SchedInfo sched;
  sched.items_per_head = (p.S + kTiles * kRows - 1) / (kTiles * kRows);
  sched.total_items = sched.items_per_head * p.B * p.H;
  if (!tcgen05_sp_fits(p)) return cudaErrorInvalidValue;
  auto kern = fwd_tcgen05_sp_kernel<kBf16>;
  static std::atomic<unsigned long long> smem_done{0};   // per kernel instantiation, bit per device
  cudaError_t e = set_dynamic_smem_once(smem_done, reinterpret_cast<const void*>(kern), kSmemBytesSp);
  if (e != cudaSuccess) return e;
  // No memset of the work queue: the last CTA of the launch that used it before put it back to zero.
  // Items of equal size (no causal mask) in a last wave that fills at most half the grid, or fewer items
  // than half the grid altogether, are handed out as single Q tiles: a lone tile takes 0.55 of the time of
  // the pair, so the launch ends that much sooner.
  int split = 0;
  if (!p.causal) {
    if (2 * sched.total_items <= sm_count) {
      split = sched.total_items;
    } else if (sched.total_items > sm_count) {
      const int r = sched.total_items % sm_count;
      if (r > 0 && 2 * r <= sm_count) split = r;
    }
  }
  const int n_queue = sched.total_items + split;
  const int grid = n_queue < sm_count ? n_queue : sm_count;
  sched_set_tail(sched, p.B * p.H, p.causal, grid);
  sched.split_items = split;
  e = launch_persistent(kern, grid, kThreadsSp, kSmemBytesSp, stream, p.pdl != 0, maps, p, sched);
  if (e == cudaSuccess) *launches += 1;
  return e;
}

bool tcgen05_sp_fits(const FwdParams& p) {
  const long long items = static_cast<long long>((p.S + kTiles * kRows - 1) / (kTiles * kRows)) * p.B * p.H;
  return items < kItemMask;   // the scheduler ring keeps flags in the bits above
}

cudaError_t launch_fwd_tcgen05_sp(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  if (p.D > kD) return cudaErrorInvalidValue;   // D < 64: zero columns from the tensor maps
  return p.bf16 ? launch_sp_one<true>(p, sm_count, stream, launches)
                : launch_sp_one<false>(p, sm_count, stream, launches);
}

}  // namespace rsfa
