// FlashAttention-2 forward for B200 (sm_100a): warp-specialised, persistent,
// tcgen05 tensor cores with accumulators in tensor memory, operands staged by TMA.
//
// It replaces the reference's tiled kernels: _attn_fwd with _attn_fwd_inner and
// _attn_fwd_inner_d64_nc (ascend_rsfa/flash_attention_forward.py:163-404) and the
// two-launch causal split _run_causal_split / _attn_fwd_split_inner (:408-541).
// Where the reference runs the unmasked prefix and the masked diagonal as two
// launches that pass l, m and an fp16 copy of the accumulator through global
// memory (:338-368), this kernel runs both tile kinds in one sweep — an unmasked
// loop body for prefix tiles and a masked one for the tile that crosses the
// diagonal (or the ragged end of the sequence) — with the state in registers and
// the accumulator in tensor memory.
//
// One CTA owns kNT query tiles of 128 rows ("Q tiles") of one (batch, head) and
// sweeps the keys in tiles of 128.  Roles:
//   warps 0..3   softmax group 0: one thread per row of Q tile 0
//   warps 4..7   softmax group 1: one thread per row of Q tile 1
//   warp  8      TMA producer (one lane): Q tiles once per work item, K/V tiles
//                through a ring of kStages shared-memory slots
//   warp  9      MMA issuer (one lane) and owner of the TMEM allocation
//   warps 10,11  idle; they complete the third warpgroup so that register budgets can be moved
//                between warpgroups with setmaxnreg (softmax threads keep a whole row in registers)
// Per key tile j and Q tile t:
//   S_t = Q_t K_j^T          tcgen05.mma, both operands from shared memory
//   softmax group t          tcgen05.ld S_t -> exp2 against the row's reference (set
//                            from the first key tile, with headroom), row sum -> P_t
//                            (16-bit) written back over S_t with tcgen05.st.  No row
//                            maximum per tile: a warp whose sum check says a P value
//                            might overflow redoes that tile in a careful path that
//                            moves the reference and rescales its O_t rows in TMEM
//                            (the reference's "rescale skipping", :466-487, taken to
//                            "rescale only when it must")
//   O_t += P_t V_j           tcgen05.mma, A from TMEM, B = V_j as an MN-major operand
// The two Q tiles alternate on the tensor pipe, so the MMAs of one overlap the
// softmax of the other.  TMEM columns: S_0 [0,128)  S_1 [128,256)  O_0 [256,256+D)
// O_1 [256+D, 256+2D).
//
// Work items (batch*head, 256-row block) are handed out through an atomic
// counter; a CTA keeps fetching until the queue is empty.  Causal items are
// ordered heaviest first inside each head; items of one head are adjacent so the
// CTAs working on them share its K and V through L2.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "../../include/rsfa.h"
#include "tcgen05_common.cuh"

namespace rsfa {
namespace {

constexpr int kTileM = 128;   // rows per Q tile (= TMEM lanes)
constexpr int kTileN = 128;   // keys per K/V tile
constexpr int kNT = 2;        // Q tiles per CTA
constexpr int kNumThreads = 384;  // 3 warpgroups: softmax 0, softmax 1, {TMA, MMA, 2 idle warps}
constexpr int kTmaWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kTmemCols = 512;

template <int D>
struct Cfg {
  static constexpr int kBoxes = D / 64;                       // 64-column TMA boxes per row
  static constexpr int kQTileBytes = kTileM * D * 2;
  static constexpr int kKvTileBytes = kTileN * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 6;
  static constexpr int kQBoxBytes = kTileM * 128;             // 128 rows x 128 B
  static constexpr int kKvBoxBytes = kTileN * 128;
  static constexpr int kStageBytes = kTileM * 128;            // epilogue staging: 128 rows x 64 columns
  static constexpr int kNumBarriers = 2 * kNT + 2 * kStages + 6 * kNT + 4;
  static constexpr int kSmemBytes = kNT * kQTileBytes + kStages * kKvTileBytes + kNT * kStageBytes + 1024 /*align*/ +
                                    kNumBarriers * 8 + 64;
  __host__ __device__ static constexpr int kColS(int t) { return t * kTileN; }
  __host__ __device__ static constexpr int kColO(int t) { return 2 * kTileN + t * D; }
};

// Number of key tiles Q tile (row0 .. row0+127) has to visit.
__device__ __forceinline__ int num_kv_tiles(int row0, int S, int causal) {
  if (row0 >= S) return 0;
  const int last_key = causal ? min(S, row0 + kTileM) : S;  // exclusive
  return (last_key + kTileN - 1) / kTileN;
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kNumThreads, 1)
fwd_tcgen05_kernel(const __grid_constant__ TmaMaps maps, const FwdParams p, const SchedInfo sched) {
  using C = Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sKV = sQ + kNT * C::kQTileBytes;
  const uint32_t sStage = sKV + C::kStages * C::kKvTileBytes;   // one staging buffer per softmax group
  const uint32_t sBar = sStage + kNT * C::kStageBytes;
  // barrier addresses
  auto bar_q_full = [&](int t) { return sBar + 8u * t; };
  auto bar_q_empty = [&](int t) { return sBar + 8u * (kNT + t); };
  auto bar_kv_full = [&](int s) { return sBar + 8u * (2 * kNT + s); };
  auto bar_kv_empty = [&](int s) { return sBar + 8u * (2 * kNT + C::kStages + s); };
  auto bar_s_full = [&](int t) { return sBar + 8u * (2 * kNT + 2 * C::kStages + t); };
  // P_t is handed to the MMA warp in two halves of 64 keys so the first PV MMAs start early.
  auto bar_p_full = [&](int t, int half) { return sBar + 8u * (3 * kNT + 2 * C::kStages + 2 * t + half); };
  auto bar_o_full = [&](int t) { return sBar + 8u * (5 * kNT + 2 * C::kStages + t); };
  // completion of the PV MMAs of a tile's first 64 keys (waited on only by the softmax slow path)
  auto bar_pv0_done = [&](int t) { return sBar + 8u * (7 * kNT + 2 * C::kStages + t); };
  const uint32_t bar_sched_full0 = sBar + 8u * (8 * kNT + 2 * C::kStages);  // 2 slots
  const uint32_t bar_sched_empty0 = bar_sched_full0 + 16u;                   // 2 slots
  const uint32_t misc = sBar + 8u * C::kNumBarriers;
  // misc words: [0] TMEM base, [1] abort flag, [2..3] scheduler ring
  uint8_t* misc_ptr = smem_raw + (misc - smem_u32(smem_raw));
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc_ptr);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc_ptr + 4);
  volatile int* sched_ring = reinterpret_cast<volatile int*>(misc_ptr + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t wait_ns = p.wait_limit_ns;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < kNT; ++t) {
      mbar_init(bar_q_full(t), 1);
      mbar_init(bar_q_empty(t), 1);
      mbar_init(bar_s_full(t), 1);
      mbar_init(bar_p_full(t, 0), kTileM);
      mbar_init(bar_p_full(t, 1), kTileM);
      mbar_init(bar_o_full(t), 1);
      mbar_init(bar_pv0_done(t), 1);
    }
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sched_full0 + 8u * s, 1);
      mbar_init(bar_sched_empty0 + 8u * s, 1 + kNT * 4);  // MMA lane + one lane per softmax warp
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), kTmemCols);
    tmem_relinquish();
  }
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    tma_prefetch_desc(&maps.o);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  // Everything above touched only this CTA's shared and tensor memory; from here on global memory
  // is read and written, which has to wait for the kernel in front of this one on the stream.
  griddep_wait();

  const int S = p.S;
  // work item -> (head, first row).  Causal: heaviest (last) row block first.
  auto decode = [&](int item, int& bh, int& row0) {
    int blk;
    sched_decode(sched, p.causal, item, bh, blk);
    row0 = blk * (kNT * kTileM);
  };

  // setmaxnreg is warpgroup-aligned: every warp of a warpgroup must execute the SAME instruction,
  // so the third warpgroup lowers its budget before it splits into roles.
  if (warp >= kTmaWarp) {
    setmaxnreg_dec<RegBudget<D>::kOther>();
  if (warp > kMmaWarp) {
    // idle warps of the third warpgroup
  } else if (warp == kTmaWarp) {
    // ================================================================ producer
    if (lane == 0) {
      RSFA_TRACE_DECL(3);
      uint32_t kv_count = 0;   // K/V tiles loaded so far (ring position)
      uint32_t item_count = 0; // work items started so far
      bool ok = true;
      while (ok) {
        // fetch the next work item and publish it to the other roles
        const int slot = item_count & 1;
        ok = mbar_wait(bar_sched_empty0 + 8u * slot, ((item_count >> 1) & 1) ^ 1, abort_flag, wait_ns,
                       kTagSched);
        if (!ok) break;
        // The first item of a CTA is its own index (the grid is never larger than the number of items): no
        // round trip to the queue stands before the first loads.  The queue hands out the items behind those.
        const int item = (item_count == 0) ? static_cast<int>(blockIdx.x)
                                           : static_cast<int>(atomicAdd(p.tile_counter, 1u) + gridDim.x);
        sched_ring[slot] = item;
        __threadfence_block();
        mbar_arrive(bar_sched_full0 + 8u * slot);
        if (item >= sched.total_items) {
          griddep_launch_dependents();   // the queue is empty: the next kernel on the stream may set up
          break;
        }
        int bh, row0;
        decode(item, bh, row0);
        const int b = bh / p.H, h = bh - b * p.H;
        int nmax = 0;
        for (int t = 0; t < kNT; ++t) nmax = max(nmax, num_kv_tiles(row0 + t * kTileM, S, p.causal));

        auto load_q = [&](int t) -> bool {
          if (!mbar_wait(bar_q_empty(t), (item_count & 1) ^ 1, abort_flag, wait_ns, kTagQEmpty)) return false;
          RSFA_TRACE_EV(0x100 + t);
          mbar_arrive_expect_tx(bar_q_full(t), C::kQTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sQ + t * C::kQTileBytes + bx * C::kQBoxBytes, &maps.q, bar_q_full(t), bx * 64,
                        row0 + t * kTileM, h, b);
          return true;
        };
        auto load_kv = [&](const CUtensorMap* map, int j) -> bool {
          if (static_cast<int>(kv_count) == p.test_drop_load) {   // test hook: this tile is never announced
            ++kv_count;
            return true;
          }
          const uint32_t s = kv_count % C::kStages;
          const uint32_t ph = (kv_count / C::kStages) & 1;
          if (!mbar_wait(bar_kv_empty(s), ph ^ 1, abort_flag, wait_ns, kTagKvEmpty)) return false;
          RSFA_TRACE_EV(0x200 + j);
          mbar_arrive_expect_tx(bar_kv_full(s), C::kKvTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sKV + s * C::kKvTileBytes + bx * C::kKvBoxBytes, map, bar_kv_full(s), bx * 64,
                        j * kTileN, h, b);
          ++kv_count;
          return true;
        };
        // K_0 first: its ring slot frees up while the previous item drains.  Then the Q tiles, which
        // wait for that item's last QK^T, and only then V_0, whose slot frees up last of all: behind
        // V_0 the Q loads, which come from DRAM, started 2000 clk later than they could.
        if (nmax > 0) ok = load_kv(&maps.k, 0);
        if (ok) ok = load_q(0);
        if (ok) ok = load_q(1);
        if (ok && nmax > 0) ok = load_kv(&maps.v, 0);
        for (int j = 1; ok && j < nmax; ++j) {
          ok = load_kv(&maps.k, j);
          if (ok) ok = load_kv(&maps.v, j);
        }
        ++item_count;
      }
    }
  } else if (warp == kMmaWarp) {
    // ============================================================== MMA issuer
    {
      // Every lane runs this role with identical control flow; only the tcgen05 instructions are
      // issued by one elected lane.
      const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      auto wait_all = [&](uint32_t bar, uint32_t parity, int tag) -> bool {
        return mbar_wait_warp(bar, parity, abort_flag, wait_ns, tag);
      };
      constexpr uint32_t idesc_qk = make_idesc_f16(kTileM, kTileN, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(kTileM, D, kBf16, false, true);
      RSFA_TRACE_DECL(2);
      const uint64_t desc_q0 = make_smem_desc_sw128(sQ, 16, 1024);
      const uint64_t desc_k0 = make_smem_desc_sw128(sKV, 16, 1024);
      const uint64_t desc_v0 = make_smem_desc_sw128(sKV, C::kKvBoxBytes, 1024);
      uint32_t kv_count = 0, item_count = 0;
      uint32_t p_count[kNT] = {0, 0};
      bool ok = true;
      while (ok) {
        const int slot = item_count & 1;
        ok = wait_all(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, kTagSched);
        if (!ok) break;
        const int item = __shfl_sync(0xffffffffu, sched_ring[slot], 0);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sched_empty0 + 8u * slot);
        if (item >= sched.total_items) break;
        RSFA_TRACE_EV(0xa000);   // item known
        int bh, row0;
        decode(item, bh, row0);
        int n[kNT];
        int nmax = 0;
        for (int t = 0; t < kNT; ++t) {
          n[t] = num_kv_tiles(row0 + t * kTileM, S, p.causal);
          nmax = max(nmax, n[t]);
        }
        // S_t = Q_t K^T : both operands K-major, 64-column boxes, 8-row atoms of 1024 B.  A step
        // of 16 along D moves the start address by 32 B inside the 128-byte swizzle row.
        // The MMAs of one operand pair and the commits that follow them are issued from ONE elected
        // region: an elect.sync and a branch per instruction cost the issuing warp more than the
        // instruction (batched: +3 % at D = 128, +4 % at D = 64).  A commit of 0 means none.
        auto issue_qk = [&](int t, uint32_t kslot, uint32_t commit_a, uint32_t commit_b, uint32_t commit_c = 0u,
                            uint32_t commit_d = 0u) {
          const uint64_t qd = desc_q0 + static_cast<uint64_t>((t * C::kQTileBytes) >> 4);
          const uint64_t kd = desc_k0 + static_cast<uint64_t>((kslot * C::kKvTileBytes) >> 4);
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint32_t off_q = ((ks >> 2) * C::kQBoxBytes + (ks & 3) * 32) >> 4;
              const uint32_t off_k = ((ks >> 2) * C::kKvBoxBytes + (ks & 3) * 32) >> 4;
              umma_ss(tmem_u + C::kColS(t), qd + off_q, kd + off_k, idesc_qk, ks > 0 ? 1u : 0u);
            }
            if (commit_a != 0) umma_commit(commit_a);
            if (commit_b != 0) umma_commit(commit_b);
            if (commit_c != 0) umma_commit(commit_c);
            if (commit_d != 0) umma_commit(commit_d);
          }
          __syncwarp();
        };
        // O_t (+)= P_t V : A = P_t in TMEM (16 keys = 8 columns per step), B = V MN-major:
        // 16 keys per step = two 8-row atoms (stride 1024 B), 64-column boxes kKvBoxBytes apart.
        auto issue_pv = [&](int t, uint32_t vslot, bool accumulate, int ks_begin, int ks_end, uint32_t commit_a) {
          const uint64_t vd = desc_v0 + static_cast<uint64_t>((vslot * C::kKvTileBytes) >> 4);
          if (elect_one()) {
#pragma unroll
            for (int ks = ks_begin; ks < ks_end; ++ks)
              umma_ts(tmem_u + C::kColO(t), tmem_u + C::kColS(t) + ks * 8, vd + ((ks * 2048) >> 4), idesc_pv,
                      (accumulate || ks > 0) ? 1u : 0u);
            if (commit_a != 0) umma_commit(commit_a);
          }
          __syncwarp();
        };
        auto wait_kv = [&](uint32_t idx) -> bool {
          return wait_all(bar_kv_full(idx % C::kStages), (idx / C::kStages) & 1, kTagKvFull);
        };

        for (int t = 0; ok && t < kNT; ++t)
          ok = wait_all(bar_q_full(t), item_count & 1, kTagQFull);
        if (!ok) break;
        RSFA_TRACE_EV(0xa100);   // Q present
        const uint32_t base = kv_count;  // K_j at base + 2j, V_j at base + 2j + 1
        if (nmax > 0) {
          ok = wait_kv(base);
          if (!ok) break;
          tc_fence_after_sync();
          RSFA_TRACE_EV(0xa200);   // K_0 present
          for (int t = 0; t < kNT; ++t) {
            // Q_t is dead once its last QK^T MMA has run: release it so the next item's Q load
            // overlaps the rest of this item.
            if (n[t] > 0)
              issue_qk(t, base % C::kStages, bar_s_full(t), n[t] <= 1 ? bar_q_empty(t) : 0u);
            else
              umma_commit_elect(bar_q_empty(t));
          }
          umma_commit_elect(bar_kv_empty(base % C::kStages));
        }
        // Steady state, kept free of everything the end of an item needs: while both tiles have key tiles
        // left after step j, every step is V_j, then per tile PV(j) in two halves and QK^T(j+1).  The MMA
        // warp is the pacemaker of the CTA: an extra test or call in this loop shows up in every step.
        const int n_lean = min(n[0], n[1]) - 1;
        int j0 = 0;
        for (; ok && j0 < n_lean; ++j0) {
          const uint32_t vidx = base + 2 * j0 + 1;
          const uint32_t kidx = base + 2 * j0 + 2;
          const uint32_t vslot = vidx % C::kStages, kslot = kidx % C::kStages;
          ok = wait_kv(vidx);
          if (!ok) break;
          RSFA_TRACE_EV(0x6000 + j0);                  // V_j present
#pragma unroll
          for (int t = 0; t < kNT; ++t) {
            ok = wait_all(bar_p_full(t, 0), p_count[t] & 1, kTagPFull);
            if (!ok) break;
            tc_fence_after_sync();
            RSFA_TRACE_EV(0x1000 + (t << 8) + j0);   // P half 0 seen
            issue_pv(t, vslot, j0 > 0, 0, kTileN / 32, bar_pv0_done(t));
            RSFA_TRACE_EV(0x2000 + (t << 8) + j0);   // PV half 0 issued
            ok = wait_all(bar_p_full(t, 1), p_count[t] & 1, kTagPFull);
            if (!ok) break;
            ++p_count[t];
            tc_fence_after_sync();
            RSFA_TRACE_EV(0x3000 + (t << 8) + j0);   // P half 1 seen
            issue_pv(t, vslot, true, kTileN / 32, kTileN / 16, 0u);
            RSFA_TRACE_EV(0x4000 + (t << 8) + j0);   // PV half 1 issued
            if (t == 0) {
              ok = wait_kv(kidx);
              if (!ok) break;
              tc_fence_after_sync();
            }
            RSFA_TRACE_EV(0x9000 + (t << 8) + j0);   // K ready
            // behind the last MMAs of the step that read V_j and K_{j+1} the release of both slots rides along
            issue_qk(t, kslot, bar_s_full(t), j0 + 2 == n[t] ? bar_q_empty(t) : 0u,
                     t == kNT - 1 ? bar_kv_empty(vslot) : 0u, t == kNT - 1 ? bar_kv_empty(kslot) : 0u);
            RSFA_TRACE_EV(0x5000 + (t << 8) + j0);   // QK(j+1) and its commits issued
          }
          RSFA_TRACE_EV(0x7000 + j0);   // iteration end
        }
        if (!ok) break;
        // The last steps of the item, in which a tile may run out of key tiles (both at once without the
        // causal mask, one a step before the other with it).
        for (int j = j0; ok && j < nmax; ++j) {
          const uint32_t vidx = base + 2 * j + 1;
          const uint32_t kidx = base + 2 * j + 2;
          ok = wait_kv(vidx);
          if (!ok) break;
          RSFA_TRACE_EV(0x6000 + j);                  // V_j present
          bool k_ready = false, folded = false;
          for (int t = 0; ok && t < kNT; ++t) {
            if (j < n[t]) {
              ok = wait_all(bar_p_full(t, 0), p_count[t] & 1, kTagPFull);
              if (!ok) break;
              tc_fence_after_sync();
              RSFA_TRACE_EV(0x1000 + (t << 8) + j);   // P half 0 seen
              issue_pv(t, vidx % C::kStages, j > 0, 0, kTileN / 32, bar_pv0_done(t));
              RSFA_TRACE_EV(0x2000 + (t << 8) + j);   // PV half 0 issued
              ok = wait_all(bar_p_full(t, 1), p_count[t] & 1, kTagPFull);
              if (!ok) break;
              ++p_count[t];
              tc_fence_after_sync();
              RSFA_TRACE_EV(0x3000 + (t << 8) + j);   // P half 1 seen
              issue_pv(t, vidx % C::kStages, true, kTileN / 32, kTileN / 16, j == n[t] - 1 ? bar_o_full(t) : 0u);
              RSFA_TRACE_EV(0x4000 + (t << 8) + j);   // PV half 1 issued
            }
            if (j + 1 < n[t]) {
              if (!k_ready) {
                ok = wait_kv(kidx);
                if (!ok) break;
                tc_fence_after_sync();
                k_ready = true;
              }
              RSFA_TRACE_EV(0x9000 + (t << 8) + j);   // K ready
              folded = (t == kNT - 1);   // the last MMAs of the step: the release of both slots rides along
              issue_qk(t, kidx % C::kStages, bar_s_full(t), j + 2 == n[t] ? bar_q_empty(t) : 0u,
                       folded ? bar_kv_empty(vidx % C::kStages) : 0u, folded ? bar_kv_empty(kidx % C::kStages) : 0u);
              RSFA_TRACE_EV(0x5000 + (t << 8) + j);   // QK(j+1) and its commits issued
            }
          }
          if (!ok) break;
          if (j + 1 < nmax && !k_ready) {  // tile loaded for a Q tile that did not need it: still consume it
            ok = wait_kv(kidx);
            if (!ok) break;
          }
          if (!folded)
            umma_commit2_elect(bar_kv_empty(vidx % C::kStages), j + 1 < nmax ? bar_kv_empty(kidx % C::kStages) : 0u);
          RSFA_TRACE_EV(0x7000 + j);   // iteration end
        }
        if (!ok) break;
        kv_count += 2 * nmax;
        ++item_count;
      }
    }
  }
  } else {
    // ========================================================== softmax groups
    setmaxnreg_inc<RegBudget<D>::kSoftmax>();
    const int t = warp >> 2;                   // Q tile of this group
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + C::kColS(t);
    const uint32_t tO = tmem_base + lane_base + C::kColO(t);
    const float scale_log2 = p.sm_scale * kLog2e;
    const float headroom = kHeadroomLog2 / scale_log2;   // in raw score units (sm_scale > 0 on this path)
    uint32_t item_count = 0, s_count = 0, o_count = 0;
    bool ok = true;
#ifdef RSFA_TRACE
    unsigned long long* trace_buf = (p.trace != nullptr && blockIdx.x == 0 && lane == 0)
                                        ? p.trace + ((warp & 3) == 0 ? t : 4 + warp) * 2 * kTraceCap : nullptr;
    int trace_n = 0;
#endif
    while (ok) {
      const int slot = item_count & 1;
      ok = mbar_wait_warp(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, abort_flag, wait_ns, kTagSched);
      if (!ok) break;
      const int item = sched_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sched_empty0 + 8u * slot);
      if (item >= sched.total_items) break;
      ++item_count;
      int bh, row0;
      decode(item, bh, row0);
      const int tile_row0 = row0 + t * kTileM;
      const int row = tile_row0 + row_in_tile;
      const int n_tiles = num_kv_tiles(tile_row0, S, p.causal);
      if (n_tiles == 0) continue;

      // The reference maximum m_used of a row is set from the first key tile (plus headroom) and is
      // NOT recomputed per tile: a tile is exponentiated against the current reference straight
      // away.  Only when the sum of a 64-key half exceeds kSumLimit (every P value of the half is
      // bounded by that sum, so none can have left the 16-bit range otherwise) does the warp leave
      // this loop and finish the work item in the careful loop below, which redoes that half and
      // handles the remaining key tiles with a row maximum per half.  This replaces the per-tile
      // maximum of the reference's loop (:196-203) and its "rescale only when the maximum moved"
      // (:466-487) by "rescale only when it must".
      float m_used = -INFINITY;  // reference, in raw score units
      float l = 0.f;
      int j = 0;
      while (j < n_tiles) {
      int careful_half = -1;     // >= 0: the half of key tile j that failed the check
      for (; j < n_tiles; ++j) {
        ok = mbar_wait_warp(bar_s_full(t), s_count & 1, abort_flag, wait_ns, kTagSFull);
        if (!ok) break;
        ++s_count;
        tc_fence_after_sync();
        RSFA_TRACE_EV(0x1000 + j);   // S seen

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
        RSFA_TRACE_EV(0x2000 + j);   // S in registers

        // masked tile: the one crossing the diagonal, or the ragged end of the sequence
        const int n0 = j * kTileN;
        const bool masked = (n0 + kTileN > S) || (p.causal && n0 + kTileN > tile_row0 + 1);
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
          m_used = mb + headroom;
        }
        RSFA_TRACE_EV(0x3000 + j);   // reference ready
        const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
        const float neg_m = -m_used * scale_log2;
        const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
        uint64_t sum_a, sum_b;
        // exp2, row sum and 16-bit packing of 32 scores into pk[base .. base+16).  The packed
        // values of one half (64 keys) are collected first and stored with a single tcgen05.st:
        // a store issued per 32 scores would make the next chunk's arithmetic wait on it, because
        // the registers it reads cannot be overwritten until the (slow) TMEM store has taken them.
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
        auto exp_half = [&](uint32_t (&sa)[32], uint32_t (&sb)[32], uint32_t (&pk)[32]) -> float {
          sum_a = pack_f32x2(0.f, 0.f);
          sum_b = sum_a;
          exp_pack(sa, pk, 0);
          exp_pack(sb, pk, 16);
          float a0, a1;
          unpack_f32x2(add_f32x2(sum_a, sum_b), a0, a1);
          return a0 + a1;
        };
        {
          uint32_t pk[32];
          const float h = exp_half(s0, s1, pk);
          // !(h <= limit) also catches NaN and +inf.  Nothing of this half has been stored yet.
          if (__any_sync(0xffffffffu, !(h <= kSumLimit))) {
            careful_half = 0;
            break;
          }
          l += h;
          RSFA_TRACE_EV(0xb000);   // half 0 computed
          tmem_st_x32(tS, pk);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(bar_p_full(t, 0));
          RSFA_TRACE_EV(0x4000 + j);   // half 0 handed over
        }
        {
          uint32_t pk[32];
          const float h = exp_half(s2, s3, pk);
          if (__any_sync(0xffffffffu, !(h <= kSumLimit))) {
            careful_half = 1;
            break;
          }
          l += h;
          RSFA_TRACE_EV(0xb001);   // half 1 computed
          tmem_st_x32(tS + 32, pk);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(bar_p_full(t, 1));
        }
        RSFA_TRACE_EV(0x5000 + j);   // half 1 handed over
      }
      if (!ok) break;
      if (careful_half >= 0) {
        // Finish key tile j half by half with the scores loaded again from tensor memory (P has
        // not been written over the half that failed the check, nor over the one behind it), then
        // go back to the fast loop.  The PV MMAs of the tile's first half accumulate into O_t, so
        // the second half waits for them before it may rescale O_t.
        RSFA_TRACE_EV(0xc000 + j);
        const int n0 = j * kTileN;
        int limit = S - 1 - n0;                             // last visible column of this tile
        if (p.causal) limit = min(limit, row - n0);
        for (int half = careful_half; half < 2; ++half) {
          if (half == 1) {
            ok = mbar_wait_warp(bar_pv0_done(t), (s_count - 1) & 1, abort_flag, wait_ns, kTagPvDone);
            if (!ok) break;
            tc_fence_after_sync();
          }
          // half 0: O_t is quiescent, S_t(j) complete implies every earlier MMA of this tile completed
          const uint64_t r = softmax_half_careful<D, kBf16>(tS + 64 * half, tS + 32 * half, tO, limit - 64 * half,
                                                            scale_log2, headroom, m_used, l,
                                                            (j > 0 || half > 0) ? 1 : 0);
          unpack_f32x2(r, m_used, l);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(bar_p_full(t, half));
        }
        if (!ok) break;
        ++j;
      }
      }
      if (!ok) break;

      // ---- epilogue: O_t / l -> global, lse = m + log l
      ok = mbar_wait_warp(bar_o_full(t), o_count & 1, abort_flag, wait_ns, kTagOFull);
      if (!ok) break;
      ++o_count;
      tc_fence_after_sync();
      RSFA_TRACE_EV(0x6000);         // O complete seen
      const float inv_l = 1.f / l;
      const int b = bh / p.H, h = bh - b * p.H;
      // O_t / l -> global memory: each warp stages and stores its own 32 rows (store_o_rows)
      {
        const int wq = warp & 3;
        store_o_rows<D, kBf16>(tO, inv_l, sStage + t * C::kStageBytes + wq * 4096, lane, &maps.o, tile_row0 + wq * 32, h, b,
                               tile_row0 + wq * 32 < S);
      }
      if (p.lse != nullptr && row < S)
        p.lse[static_cast<int64_t>(bh) * S + row] = m_used * p.sm_scale + logf(l);
      tc_fence_before_sync();
      RSFA_TRACE_EV(0x7000);         // epilogue done
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
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
  if (threadIdx.x == 0) {
    if (*abort_flag != 0) atomicCAS(p.status, 0, *abort_flag);
    queue_retire(p.tile_counter);
  }
}

template <int D, bool kBf16>
cudaError_t launch_one(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  using C = Cfg<D>;
  TmaMaps maps;
  if (!make_map(&maps.q, p.q, p, p.q_stride, kTileM) || !make_map(&maps.k, p.k, p, p.k_stride, kTileN) ||
      !make_map(&maps.v, p.v, p, p.v_stride, kTileN) || !make_map(&maps.o, p.o, p, p.o_stride, 32))
    return cudaErrorInvalidValue;
  SchedInfo sched;
  sched.items_per_head = (p.S + kNT * kTileM - 1) / (kNT * kTileM);
  sched.total_items = sched.items_per_head * p.B * p.H;
  auto kern = fwd_tcgen05_kernel<D, kBf16>;
  static std::atomic<unsigned long long> smem_done{0};   // per kernel instantiation, bit per device
  cudaError_t e = set_dynamic_smem_once(smem_done, reinterpret_cast<const void*>(kern), C::kSmemBytes);
  if (e != cudaSuccess) return e;
  // No memset of the work queue: the last CTA of the launch that used it before put it back to zero.
  const int grid = sched.total_items < sm_count ? sched.total_items : sm_count;
  sched_set_tail(sched, p.B * p.H, p.causal, grid);
  e = launch_persistent(kern, grid, kNumThreads, C::kSmemBytes, stream, p.pdl != 0, maps, p, sched);
  if (e == cudaSuccess) *launches += 1;
  return e;
}

}  // namespace

// D = 16 and 32 run on the D = 64 kernels: the tensor maps describe the real D columns, the 64-column
// boxes read zeros past them (Q, K: nothing added to the scores; V: output columns that the clipped
// store never writes), so the kernels need no variant of their own.
bool tcgen05_supports(int S, int D, float sm_scale) {
  return (D == 16 || D == 32 || D == 64 || D == 128 || D == 256) && S >= 1 && sm_scale > 0.f;
}

namespace {
struct TileRow {
  int s_min, s_max, d, causal, bm, bn;
};
const TileRow kTileTable[] = {
#include "tile_table.inc"
};
}  // namespace

void tcgen05_resolve_tile(int S, int D, int causal, int req_bm, int req_bn, int variant, int* bm, int* bn) {
  if (D < 64) D = 64;   // served by the D = 64 kernels
  *bm = 128;
  if (D == 256) {  // one instantiation only
    *bn = 64;
    return;
  }
  if (variant == 0 || variant == 1 || (variant == 2 && D == 64)) {
    *bn = variant == 1 ? 64 : 128;
    return;
  }
  if (req_bm == 128 && (req_bn == 128 || req_bn == 64)) {  // an instantiated tile: honour the request
    *bn = req_bn;
    return;
  }
  *bn = 128;
  for (const TileRow& r : kTileTable) {
    if (S >= r.s_min && S <= r.s_max && D == r.d && (causal != 0) == (r.causal != 0)) {
      *bm = r.bm;
      *bn = r.bn;
      return;
    }
  }
}

cudaError_t launch_fwd_tcgen05(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  // D = 256 exists only in the double-buffered family (its accumulator leaves room for one Q tile).
  if (p.tile_n == 64 || p.D == 256) return launch_fwd_tcgen05_db(p, sm_count, stream, launches);
  if (p.D == 128) return p.bf16 ? launch_one<128, true>(p, sm_count, stream, launches)
                                : launch_one<128, false>(p, sm_count, stream, launches);
  if (p.D <= 64) {
    // D = 64 (and below): the separate-P kernel, unless single-buffered S is forced.  A single key
    // tile (S <= 128) leaves nothing to overlap: this file's kernel then.
    if (p.variant != 0 && (p.S > kTileN || p.variant == 2) && tcgen05_sp_fits(p))
      return launch_fwd_tcgen05_sp(p, sm_count, stream, launches);
    return p.bf16 ? launch_one<64, true>(p, sm_count, stream, launches)
                  : launch_one<64, false>(p, sm_count, stream, launches);
  }
  return cudaErrorInvalidValue;
}

}  // namespace rsfa

// ------------------------------------------------------------------------------------------
// rsfa_fwd_noalloc: the tcgen05 kernel for callers that must not allocate device memory.
//
// rsfa_fwd keeps its work-queue counter and status word in a buffer the library obtains with
// cudaMalloc on first use.  Some callers cannot tolerate that: an inference server that hands
// all device memory to its own arena at start-up and treats any later cudaMalloc as a fault, a
// hard-real-time loop in which an allocation (which may synchronise the device) breaks the
// latency budget, or a plugin loaded into a process whose memory is accounted by someone else.
// For them the same kernel runs here with its scratch in a fixed, statically allocated block of
// device memory that is part of the library image.
namespace rsfa {
namespace {

// The whole scratch: words 0 and 1 = work queue (items handed out, CTAs finished), word 2 = status
// word, rest unused.  Every GPU that loads the library holds these 256 bytes until the process exits.
constexpr int kStaticScratchBytes = 256;
static __device__ __align__(256) unsigned int g_static_scratch[kStaticScratchBytes / sizeof(unsigned int)];

// Largest problem the entry point accepts: the queue counter is one 32-bit word of the block and
// every CTA adds to it once more after the queue is empty, so items + CTAs must stay below 2^31.
constexpr long long kNoAllocMaxItems = 1ll << 30;

struct NoAllocDevice {
  bool ready = false;
  unsigned int* scratch = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
};
std::mutex g_noalloc_mu;
NoAllocDevice g_noalloc_dev[64];

// Once per device, with that device current.  In host code `g_static_scratch` is only a handle:
// the address the kernel needs comes from cudaGetSymbolAddress.
int noalloc_setup(int device, NoAllocDevice** out) {
  if (device < 0 || device >= 64) return RSFA_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  NoAllocDevice& d = g_noalloc_dev[device];
  if (!d.ready) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
      cudaGetLastError();
      return RSFA_ERR_NO_DEVICE;
    }
    if (major != 10) return RSFA_ERR_NO_DEVICE;
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return RSFA_ERR_CUDA;
    }
    d.scratch = static_cast<unsigned int*>(ptr);
    d.sm_count = sms;
    d.ready = true;
  }
  *out = &d;
  return RSFA_OK;
}

}  // namespace

int* noalloc_status_word(int device) {
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  const NoAllocDevice& d = g_noalloc_dev[device];
  return d.ready ? reinterpret_cast<int*>(d.scratch + 2) : nullptr;
}
}  // namespace rsfa

extern "C" int rsfa_fwd_noalloc(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                                int S, int D, const int64_t* strides, int causal, float sm_scale, int dtype,
                                void* stream) {
  using namespace rsfa;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || strides == nullptr)
    return RSFA_ERR_INVALID_ARGUMENT;
  if (B < 1 || H < 1 || S < 1) return RSFA_ERR_INVALID_ARGUMENT;
  if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256) return RSFA_ERR_INVALID_ARGUMENT;
  if (dtype != RSFA_DTYPE_F16 && dtype != RSFA_DTYPE_BF16) return RSFA_ERR_INVALID_ARGUMENT;
  if (!(sm_scale == sm_scale)) return RSFA_ERR_INVALID_ARGUMENT;
  const void* ptrs[4] = {q, k, v, o};
  for (int t = 0; t < 4; ++t) {
    if ((reinterpret_cast<uintptr_t>(ptrs[t]) & 15u) != 0) return RSFA_ERR_INVALID_ARGUMENT;
    const int64_t* st = strides + 4 * t;
    if (st[3] != 1) return RSFA_ERR_INVALID_ARGUMENT;
    const int extent[3] = {B, H, S};
    for (int i = 0; i < 3; ++i)
      if (extent[i] > 1 && (st[i] < D || (st[i] & 7) != 0)) return RSFA_ERR_INVALID_ARGUMENT;
  }
  // Only the tcgen05 kernel uses scratch; shapes it is not built for have no variant here.
  if (!tcgen05_supports(S, D, sm_scale)) return RSFA_ERR_UNSUPPORTED;
  const int rows_per_item = (D == 256) ? kTileM : kNT * kTileM;   // both families use 256-row items at D <= 128
  const long long items = static_cast<long long>(B) * H * ((S + rows_per_item - 1) / rows_per_item);
  if (items > kNoAllocMaxItems) return RSFA_ERR_TOO_LARGE;

  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_NO_DEVICE;
  }
  NoAllocDevice* d = nullptr;
  const int rc = noalloc_setup(device, &d);
  if (rc != RSFA_OK) return rc;

  FwdParams p;
  p.q = q;
  p.k = k;
  p.v = v;
  p.o = o;
  p.lse = lse;
  p.B = B;
  p.H = H;
  p.S = S;
  p.D = D;
  for (int i = 0; i < 3; ++i) {
    p.q_stride[i] = strides[0 + i];
    p.k_stride[i] = strides[4 + i];
    p.v_stride[i] = strides[8 + i];
    p.o_stride[i] = strides[12 + i];
  }
  p.causal = causal ? 1 : 0;
  p.sm_scale = sm_scale;
  p.bf16 = (dtype == RSFA_DTYPE_BF16) ? 1 : 0;
  {
    int bm = 0, bn = 0;
    tcgen05_resolve_tile(S, D, causal, 0, 0, -1, &bm, &bn);   // no tile request here: the table decides
    p.tile_n = bn;
  }
  p.tile_counter = d->scratch;      // words 0 and 1, cleared on `stream` below
  p.status = reinterpret_cast<int*>(d->scratch + 2);
  p.wait_limit_ns = option_wait_limit_ns();
  p.pdl = 0;                        // a memset precedes the kernel on the stream: nothing to overlap with
  p.test_drop_load = option_test_drop_load();
  p.variant = -1;
#ifdef RSFA_TRACE
  p.trace = nullptr;
#endif
  // The block keeps whatever the last call left (a kernel puts its queue back to zero when it ends,
  // but a call that was cut short may not have): a fresh call starts from zero queue words and "ok".
  if (cudaMemsetAsync(d->scratch, 0, 3 * sizeof(unsigned int), static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_CUDA;
  }
  long long launches = 0;
  const cudaError_t e = launch_fwd_tcgen05(p, d->sm_count, static_cast<cudaStream_t>(stream), &launches);
  count_launches(launches);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_CUDA;
  }
  return RSFA_OK;
}
