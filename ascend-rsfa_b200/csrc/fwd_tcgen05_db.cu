// FlashAttention-2 forward for B200 (sm_100a), "double-buffered S" kernel family.
//
// Replaces the reference's tiled kernels _attn_fwd / _attn_fwd_inner(_d64_nc) and the causal
// split _run_causal_split (ascend_rsfa/flash_attention_forward.py:163-541) in one launch.
//
// A CTA owns kNT Q tiles of 128 rows of one (batch, head) and sweeps the keys in tiles of 64.
// Each Q tile has TWO S buffers in tensor memory, so the MMA warp computes S for key tile j+2
// while the softmax warps are still on tile j+1: the softmax -> PV -> QK^T dependency chain of a
// single-buffered design is cut, the tensor pipe and the softmax warps each run back to back.
//   S_t[j & 1] = Q_t K_j^T    D/16 MMAs of 128 x 64 x 16, both operands in shared memory
//   softmax group t           tcgen05.ld S -> mask (diagonal / ragged tiles) -> exp2 against the
//                             row's reference -> row sum -> sum check -> P_j (16-bit) over
//                             S_t[j & 1]; a failed check redoes the tile carefully (new reference,
//                             rescale of O_t in TMEM)
//   O_t += P_j V_j            4 MMAs of 128 x D x 16, A = P_j from TMEM, B = V_j MN-major
// One MMA-issuing warp per Q tile: a wait on an mbarrier costs the issuing warp about 100 cycles
// even when it is already satisfied and a tcgen05.mma about 40, so one warp cannot feed both tiles.
// TMEM columns: S_t[b] at 128 t + 64 b, O_t at 128 kNT + D t (kNT = 2 for D <= 128, 1 for D = 256).
// Shared memory: Q tiles + a ring of K/V tiles of 64 keys filled by TMA (128-byte swizzle).
// Roles: warps [0, 4 kNT) softmax (one thread per row), then one TMA warp and kNT MMA warps.
// D = 256 differs in three ways (see DbCfg): Q travels through the K/V ring and is copied into the
// 128 spare tensor-memory columns by the MMA warp (tcgen05.cp), QK^T reads it from there (A in
// tensor memory, only K from shared memory), and warps 8-11 do the epilogue so that the single
// softmax group can go on to the next work item at once.
// Work items (batch*head, block of 128 kNT rows) come from an atomic queue, head-major, causal
// blocks heaviest first inside a head.
#include "tcgen05_common.cuh"

namespace rsfa {
namespace {

constexpr int kRowsDb = 128;   // rows per Q tile (= TMEM lanes)
constexpr int kKeysDb = 64;    // keys per K/V tile

template <int D, int NT>
struct DbCfg {
  static constexpr int kBoxes = D / 64;
  static constexpr int kQBoxBytes = kRowsDb * 128;
  static constexpr int kQTileBytes = kBoxes * kQBoxBytes;
  static constexpr int kKvBoxBytes = kKeysDb * 128;
  static constexpr int kKvBytes = kBoxes * kKvBoxBytes;
  // A ring slot holds a PAIR of tiles that the MMA warps consume together: (K_0, K_1) first,
  // then (V_j, K_{j+2}) for j = 0, 1, ... - one full/empty barrier pair per slot.
  static constexpr int kSlotBytes = 2 * kKvBytes;
  static constexpr int kStages = (D == 256) ? 3 : (D == 128 ? 4 : 6);
  // D = 256 has a warpgroup of its own for the epilogue (warps 8-11; a warp reads the tensor-memory
  // lanes 32 * (warp % 4) ...): the single softmax group goes straight on to the next work item and
  // the O store runs beside that item's first key tiles.  Warps 6 and 7 have no role.
  static constexpr bool kEpi = (D == 256);
  static constexpr int kEpiWarp0 = 8;
  static constexpr int kThreads = kEpi ? 384 : 32 * (4 * NT + 1 + NT);
  static constexpr int kTmaWarp = 4 * NT;
  static constexpr int kMmaWarp0 = 4 * NT + 1;   // one MMA warp per Q tile
  // q_full, q_empty, pv_done, o_full per tile; s_full, p_full per (tile, buffer); ring; scheduler
  // epilogue staging: 128 rows x 64 columns, twice at D = 256 (four chunks per row; the shared
  // memory is there once Q has no buffer of its own)
  static constexpr int kStageBufs = (D == 256) ? 2 : 1;
  static constexpr int kStageBytes = kStageBufs * kRowsDb * 128;
  static constexpr int kNumBarriers = 4 * NT + 4 * NT + NT + 2 * kStages + 4 + 2;
  // D = 256 leaves 128 tensor-memory columns free: Q lives there as the A operand of QK^T.  Those
  // MMAs then read only K from shared memory (with both operands there, N = 64 took 65 clk instead
  // of 32 and the MMA warp was the limit), and Q needs no shared-memory buffer of its own: it comes
  // through the ring as the first entry of a work item, the MMA warp copies it into tensor memory
  // with tcgen05.cp, and its 64 KB are a third ring slot (with two slots the delivery of the K/V
  // pairs was the next limit).
  static constexpr bool kQTmem = (D == 256);
  static constexpr int kQSmemBytes = kQTmem ? 0 : NT * kQTileBytes;
  __host__ __device__ static constexpr int col_q() { return 128 * NT + D * NT; }
  static_assert(!kQTmem || (NT == 1 && kQTileBytes == kSlotBytes), "Q travels through a ring slot");
  static constexpr int kSmemBytes = kQSmemBytes + kStages * kSlotBytes + NT * kStageBytes + 1024 + kNumBarriers * 8 + 128 + 512;
  __host__ __device__ static constexpr int col_s(int t, int b) { return 128 * t + 64 * b; }
  __host__ __device__ static constexpr int col_o(int t) { return 128 * NT + D * t; }
};

__device__ __forceinline__ int num_kv_tiles_db(int row0, int S, int causal) {
  if (row0 >= S) return 0;
  const int last_key = causal ? min(S, row0 + kRowsDb) : S;  // exclusive
  return (last_key + kKeysDb - 1) / kKeysDb;
}

template <int D, int NT, bool kBf16>
__global__ void __launch_bounds__(DbCfg<D, NT>::kThreads, 1)
fwd_tcgen05_db_kernel(const __grid_constant__ TmaMaps maps, const FwdParams p, const SchedInfo sched) {
  using C = DbCfg<D, NT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sKV = sQ + C::kQSmemBytes;
  const uint32_t sStage = sKV + C::kStages * C::kSlotBytes;   // one staging buffer per softmax group
  const uint32_t sBar = sStage + NT * C::kStageBytes;
  auto bar_q_full = [&](int t) { return sBar + 8u * t; };
  auto bar_q_empty = [&](int t) { return sBar + 8u * (NT + t); };
  auto bar_pv_done = [&](int t) { return sBar + 8u * (2 * NT + t); };   // one completion per key tile
  auto bar_o_full = [&](int t) { return sBar + 8u * (3 * NT + t); };    // one completion per work item
  auto bar_s_full = [&](int t, int b) { return sBar + 8u * (4 * NT + 2 * t + b); };
  auto bar_p_full = [&](int t, int b) { return sBar + 8u * (6 * NT + 2 * t + b); };
  auto bar_kv_full = [&](int s) { return sBar + 8u * (8 * NT + s); };
  auto bar_kv_empty = [&](int s) { return sBar + 8u * (8 * NT + C::kStages + s); };
  const uint32_t bar_sched_full0 = sBar + 8u * (9 * NT + 2 * C::kStages);  // 2 slots
  const uint32_t bar_sched_empty0 = bar_sched_full0 + 16u;                 // 2 slots
  // D = 256: softmax group -> epilogue warps (1 / l of every row is in s_inv_l), epilogue warps -> MMA
  // warp and softmax group (O has been read, s_inv_l may be written again)
  const uint32_t bar_epi_ready = bar_sched_empty0 + 16u;
  const uint32_t bar_o_free = bar_epi_ready + 8u;
  const uint32_t misc = sBar + 8u * C::kNumBarriers;
  uint8_t* misc_ptr = smem_raw + (misc - smem_u32(smem_raw));
  volatile uint32_t* tmem_base_slot = reinterpret_cast<volatile uint32_t*>(misc_ptr);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc_ptr + 4);
  volatile int* sched_ring = reinterpret_cast<volatile int*>(misc_ptr + 8);
  volatile float* s_inv_l = reinterpret_cast<volatile float*>(misc_ptr + 128);   // kRowsDb values

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t wait_ns = p.wait_limit_ns;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < NT; ++t) {
      mbar_init(bar_q_full(t), 1);
      mbar_init(bar_q_empty(t), 1);
      mbar_init(bar_pv_done(t), 1);
      mbar_init(bar_o_full(t), 1);
      for (int b = 0; b < 2; ++b) {
        mbar_init(bar_s_full(t, b), 1);
        mbar_init(bar_p_full(t, b), kRowsDb);
      }
    }
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), NT);   // one commit per MMA warp
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sched_full0 + 8u * s, 1);
      // one lane per MMA warp, per softmax warp and per epilogue warp
      mbar_init(bar_sched_empty0 + 8u * s, NT + 4 * NT + (C::kEpi ? 4 : 0));
    }
    mbar_init(bar_epi_ready, kRowsDb);
    mbar_init(bar_o_free, 4);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == C::kMmaWarp0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), 512);
    tmem_relinquish();
  }
  if (warp == C::kTmaWarp && lane == 0) {
    tma_prefetch_desc(&maps.q);
    tma_prefetch_desc(&maps.k);
    tma_prefetch_desc(&maps.v);
    tma_prefetch_desc(&maps.o);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  // Only this CTA's shared and tensor memory so far; global memory waits for the kernel in front.
  griddep_wait();

  const int S = p.S;
  auto decode = [&](int item, int& bh, int& row0) {
    int blk;
    sched_decode(sched, p.causal, item, bh, blk);
    row0 = blk * (NT * kRowsDb);
  };

  if (warp == C::kTmaWarp) {
    // ================================================================ producer
    if (lane == 0) {
      RSFA_TRACE_DECL(3);
      uint32_t kv_count = 0, item_count = 0;
      bool ok = true;
      // D = 256: Q reaches the softmax warps through the ring, and at a work-item boundary everything
      // waits for it (2 us from HBM).  So the Q tile of the NEXT item is sent on its way to L2 as early as
      // the item is known: without the causal mask the next item is claimed while this one starts (all
      // items take equally long, claiming one ahead costs no balance); with it, when it is claimed
      // anyway, which is still two key tiles before its load can be issued.
      int claimed = -1;
      auto prefetch_q = [&](int it) {
        if (it >= sched.total_items) return;
        int pbh, prow0;
        decode(it, pbh, prow0);
        const int pb = pbh / p.H, ph = pbh - pb * p.H;
        for (int bx = 0; bx < C::kBoxes; ++bx) tma_prefetch_l2_4d(&maps.q, bx * 64, prow0, ph, pb);
      };
      while (ok) {
        const int slot = item_count & 1;
        ok = mbar_wait(bar_sched_empty0 + 8u * slot, ((item_count >> 1) & 1) ^ 1, abort_flag, wait_ns, kTagSched);
        if (!ok) break;
        int item = claimed;
        claimed = -1;
        if (item < 0) {
          // the first item of a CTA is its own index (grid <= number of items), the queue hands out the rest
          item = (item_count == 0) ? static_cast<int>(blockIdx.x)
                                   : static_cast<int>(atomicAdd(p.tile_counter, 1u) + gridDim.x);
          if (C::kQTmem) prefetch_q(item);
        }
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
        for (int t = 0; t < NT; ++t) nmax = max(nmax, num_kv_tiles_db(row0 + t * kRowsDb, S, p.causal));
        // one ring entry: tile A (K_0 or V_j) and, when it exists, tile B (K_1 or K_{j+2})
        auto load_pair = [&](const CUtensorMap* map_a, int ja, bool has_b, int jb) -> bool {
          const uint32_t s = kv_count % C::kStages;
          const uint32_t ph = (kv_count / C::kStages) & 1;
          if (!mbar_wait(bar_kv_empty(s), ph ^ 1, abort_flag, wait_ns, kTagKvEmpty)) return false;
          RSFA_TRACE_EV(0x200 + ja);
          mbar_arrive_expect_tx(bar_kv_full(s), has_b ? C::kSlotBytes : C::kKvBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sKV + s * C::kSlotBytes + bx * C::kKvBoxBytes, map_a, bar_kv_full(s), bx * 64, ja * kKeysDb, h, b);
          if (has_b) {
            for (int bx = 0; bx < C::kBoxes; ++bx)
              tma_load_4d(sKV + s * C::kSlotBytes + C::kKvBytes + bx * C::kKvBoxBytes, &maps.k, bar_kv_full(s), bx * 64,
                          jb * kKeysDb, h, b);
          }
          ++kv_count;
          return true;
        };
        if constexpr (C::kQTmem) {
          if (!p.causal) {
            claimed = static_cast<int>(atomicAdd(p.tile_counter, 1u) + gridDim.x);
            prefetch_q(claimed);
          }
          // Q is the first ring entry of the item
          const uint32_t s = kv_count % C::kStages;
          const uint32_t ph = (kv_count / C::kStages) & 1;
          ok = mbar_wait(bar_kv_empty(s), ph ^ 1, abort_flag, wait_ns, kTagKvEmpty);
          if (!ok) break;
          RSFA_TRACE_EV(0x100);
          mbar_arrive_expect_tx(bar_kv_full(s), C::kQTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sKV + s * C::kSlotBytes + bx * C::kQBoxBytes, &maps.q, bar_kv_full(s), bx * 64, row0, h, b);
          ++kv_count;
        }
        // (K_0, K_1) before the Q tiles: ring slots free up while the previous item drains,
        // whereas a Q buffer is released only when that item's last QK^T on it has finished.
        ok = load_pair(&maps.k, 0, nmax > 1, 1);
        for (int t = 0; !C::kQTmem && ok && t < NT; ++t) {
          ok = mbar_wait(bar_q_empty(t), (item_count & 1) ^ 1, abort_flag, wait_ns, kTagQEmpty);
          if (!ok) break;
          RSFA_TRACE_EV(0x100 + t);
          mbar_arrive_expect_tx(bar_q_full(t), C::kQTileBytes);
          for (int bx = 0; bx < C::kBoxes; ++bx)
            tma_load_4d(sQ + t * C::kQTileBytes + bx * C::kQBoxBytes, &maps.q, bar_q_full(t), bx * 64,
                        row0 + t * kRowsDb, h, b);
        }
        for (int j = 0; ok && j < nmax; ++j) ok = load_pair(&maps.v, j, j + 2 < nmax, j + 2);
        ++item_count;
      }
    }
  } else if (warp >= C::kMmaWarp0 && warp < C::kMmaWarp0 + NT) {
    // ============================================================== MMA issuers, one warp per Q tile
    // Every lane runs this role with identical control flow (operands stay in uniform registers);
    // only the tcgen05 instructions are issued by one elected lane.  Both warps walk the same
    // sequence of ring entries; a slot is free again when both have committed it.
    const int t = warp - C::kMmaWarp0;
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    auto wait_all = [&](uint32_t bar, uint32_t parity, int tag) -> bool {
      return mbar_wait_warp(bar, parity, abort_flag, wait_ns, tag);
    };
    constexpr uint32_t idesc_qk = make_idesc_f16(kRowsDb, kKeysDb, kBf16, false, false);
    constexpr uint32_t idesc_pv = make_idesc_f16(kRowsDb, D, kBf16, false, true);
    RSFA_TRACE_DECL(2);
#ifdef RSFA_TRACE
    if (t != 0) trace_buf = nullptr;
#endif
    const uint64_t desc_q = make_smem_desc_sw128(sQ + t * C::kQTileBytes, 16, 1024);
    const uint64_t desc_k0 = make_smem_desc_sw128(sKV, 16, 1024);
    const uint64_t desc_v0 = make_smem_desc_sw128(sKV, C::kKvBoxBytes, 1024);
    const uint32_t col_o = tmem_u + C::col_o(t);
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
      int nmax = 0;
      for (int tt = 0; tt < NT; ++tt) nmax = max(nmax, num_kv_tiles_db(row0 + tt * kRowsDb, S, p.causal));
      const int n = num_kv_tiles_db(row0 + t * kRowsDb, S, p.causal);
      // S_t[buf] = Q_t K^T: K-major operands; 16 elements of D per step = 32 B inside a swizzle
      // row, four steps per 64-column box.  `koff` = byte offset of the K tile in the ring.
      // MMAs and the commits behind them go out from ONE elected region (an elect.sync and a branch
      // per instruction cost the warp more than the instruction); commit = 0: none.
      auto issue_qk = [&](int buf, uint32_t koff, uint32_t commit_a, uint32_t commit_b) {
        const uint64_t kd = desc_k0 + static_cast<uint64_t>(koff >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off_q = ((ks >> 2) * C::kQBoxBytes + (ks & 3) * 32) >> 4;
            const uint32_t off_k = ((ks >> 2) * C::kKvBoxBytes + (ks & 3) * 32) >> 4;
            if constexpr (C::kQTmem)
              umma_ts(tmem_u + C::col_s(t, buf), tmem_u + C::col_q() + ks * 8, kd + off_k, idesc_qk, ks > 0 ? 1u : 0u);
            else
              umma_ss(tmem_u + C::col_s(t, buf), desc_q + off_q, kd + off_k, idesc_qk, ks > 0 ? 1u : 0u);
          }
          if (commit_a != 0) umma_commit(commit_a);
          if (commit_b != 0) umma_commit(commit_b);
        }
        __syncwarp();
      };
      // O_t (+)= P V: A = P in TMEM (8 columns per 16 keys), B = V MN-major, N = D spans D/64
      // boxes (kKvBoxBytes apart), 16 keys = two 8-row atoms of 1024 B.
      auto issue_pv = [&](int buf, uint32_t voff, bool accumulate, uint32_t commit_a, uint32_t commit_b) {
        const uint64_t vd = desc_v0 + static_cast<uint64_t>(voff >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < kKeysDb / 16; ++ks)
            umma_ts(col_o, tmem_u + C::col_s(t, buf) + ks * 8, vd + ((ks * 2048) >> 4), idesc_pv,
                    (accumulate || ks > 0) ? 1u : 0u);
          if (commit_a != 0) umma_commit(commit_a);
          if (commit_b != 0) umma_commit(commit_b);
        }
        __syncwarp();
      };

      if constexpr (C::kQTmem) {
        // Q arrives as the first ring entry of the item.  This warp copies it into tensor memory
        // itself (tcgen05.cp: 16 elements of D = eight columns per instruction, the same shared-memory
        // slabs an SS-form MMA would read); the copies run in order behind the last item's MMAs and in
        // front of the QK^T issued below, and the slot is free again when they are complete.
        const uint32_t qs = kv_count % C::kStages;
        ok = wait_all(bar_kv_full(qs), (kv_count / C::kStages) & 1, kTagQFull);
        if (!ok) break;
        tc_fence_after_sync();
        RSFA_TRACE_EV(0x4000);   // Q present
        const uint64_t qd = desc_k0 + static_cast<uint64_t>((qs * C::kSlotBytes) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks)
            tmem_cp_128x256b(tmem_u + C::col_q() + ks * 8, qd + (((ks >> 2) * C::kQBoxBytes + (ks & 3) * 32) >> 4));
          umma_commit(bar_kv_empty(qs));
        }
        __syncwarp();
        ++kv_count;
      } else {
        ok = wait_all(bar_q_full(t), item_count & 1, kTagQFull);
        if (!ok) break;
      }
      // entry 0: (K_0, K_1) -> S_t[0], S_t[1]
      {
        const uint32_t s = kv_count % C::kStages;
        ok = wait_all(bar_kv_full(s), (kv_count / C::kStages) & 1, kTagKvFull);
        if (!ok) break;
        tc_fence_after_sync();
        RSFA_TRACE_EV(0x60ff);   // (K_0, K_1) present
        for (int j = 0; j < 2; ++j) {
          if (j < n) issue_qk(j, s * C::kSlotBytes + j * C::kKvBytes, bar_s_full(t, j), 0u);
        }
        RSFA_TRACE_EV(0x50ff);   // QK^T 0 and 1 issued
        // Q_t is dead after its last QK^T
        umma_commit2_elect((n <= 2 && !C::kQTmem) ? bar_q_empty(t) : 0u, bar_kv_empty(s));
        ++kv_count;
      }
      // entry j + 1: (V_j, K_{j+2})
      for (int j = 0; ok && j < nmax; ++j) {
        const int buf = j & 1;
        const uint32_t s = kv_count % C::kStages;
        ok = wait_all(bar_kv_full(s), (kv_count / C::kStages) & 1, kTagKvFull);
        if (!ok) break;
        RSFA_TRACE_EV(0x6000 + j);   // entry present
        if (j < n) {
          ok = wait_all(bar_p_full(t, buf), p_count[buf] & 1, kTagPFull);
          if (!ok) break;
          ++p_count[buf];
          tc_fence_after_sync();
          RSFA_TRACE_EV(0x1000 + j);   // P seen
          if (C::kEpi && j == 0 && item_count > 0) {
            // the first PV of an item overwrites O: the epilogue warps must have read the last one
            ok = wait_all(bar_o_free, (item_count - 1) & 1, kTagOFull);
            if (!ok) break;
            tc_fence_after_sync();
            RSFA_TRACE_EV(0x3000 + j);   // O free seen
          }
          issue_pv(buf, s * C::kSlotBytes, j > 0, bar_pv_done(t), j == n - 1 ? bar_o_full(t) : 0u);
          RSFA_TRACE_EV(0x2000 + j);   // PV issued
        }
        if (j + 2 < n) {
          // S_t[buf] is free: PV above consumed P_j in order
          issue_qk(buf, s * C::kSlotBytes + C::kKvBytes, bar_s_full(t, buf),
                   (j + 3 == n && !C::kQTmem) ? bar_q_empty(t) : 0u);
          RSFA_TRACE_EV(0x5000 + j);   // QK(j+2) issued
        }
        umma_commit_elect(bar_kv_empty(s));
        ++kv_count;
      }
      if (!ok) break;
      ++item_count;
    }
  } else if (warp < 4 * NT) {
    // ========================================================== softmax groups
    const int t = warp >> 2;   // Q tile of this group
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tO = tmem_base + lane_base + C::col_o(t);
    const float scale_log2 = p.sm_scale * kLog2e;
    const float headroom = kHeadroomLog2 / scale_log2;   // in raw score units (sm_scale > 0 on this path)
    uint32_t item_count = 0, o_count = 0, pv_count = 0;
    uint32_t s_count[2] = {0, 0};
    bool ok = true;
#ifdef RSFA_TRACE
    unsigned long long* trace_buf = (p.trace != nullptr && blockIdx.x == 0 && (warp & 3) == 0 && lane == 0)
                                        ? p.trace + t * 2 * kTraceCap : nullptr;
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
      const int tile_row0 = row0 + t * kRowsDb;
      const int row = tile_row0 + row_in_tile;
      const int n = num_kv_tiles_db(tile_row0, S, p.causal);
      if (n == 0) continue;

      // As in the 128-key kernel: the row's reference is set from the first key tile (plus
      // headroom) and a tile is exponentiated against it straight away; only when the sum check
      // says that a P value might leave the 16-bit range is that tile redone by
      // softmax_half_careful, which moves the reference and rescales this thread's row of O_t.
      float m_used = -INFINITY;   // reference, raw score units
      float l = 0.f;
      int j = 0;
      while (j < n) {
        bool careful = false;
        for (; j < n; ++j) {
          const int buf = j & 1;
          const uint32_t tS = tmem_base + lane_base + C::col_s(t, buf);
          ok = mbar_wait_warp(bar_s_full(t, buf), s_count[buf] & 1, abort_flag, wait_ns, kTagSFull);
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

          // masked tile: one that crosses the diagonal, or the ragged end of the sequence
          const int n0 = j * kKeysDb;
          const bool masked = (n0 + kKeysDb > S) || (p.causal && n0 + kKeysDb > tile_row0 + 1);
          if (masked) {
            int limit = S - 1 - n0;   // last visible column of this tile
            if (p.causal) limit = min(limit, row - n0);
            const uint32_t ninf = 0xff800000u;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              if (c > limit) s0[c] = ninf;
              if (c + 32 > limit) s1[c] = ninf;
            }
          }
          if (j == 0) {
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              mx[0] = max3(mx[0], __uint_as_float(s0[c]), __uint_as_float(s0[c + 1]));
              mx[1] = max3(mx[1], __uint_as_float(s0[c + 2]), __uint_as_float(s0[c + 3]));
              mx[2] = max3(mx[2], __uint_as_float(s1[c]), __uint_as_float(s1[c + 1]));
              mx[3] = max3(mx[3], __uint_as_float(s1[c + 2]), __uint_as_float(s1[c + 3]));
            }
            float mb = fmaxf(max3(mx[0], mx[1], mx[2]), mx[3]);
            if (mb == -INFINITY) mb = 0.f;   // only rows past S can get here; keep them finite
            m_used = mb + headroom;
          }
          RSFA_TRACE_EV(0x3000 + j);   // reference ready

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
          float a0, a1;
          unpack_f32x2(add_f32x2(sum_a, sum_b), a0, a1);
          const float h = a0 + a1;
          // !(h <= limit) also catches NaN and +inf.  Nothing of this tile has been stored yet.
          if (__any_sync(0xffffffffu, !(h <= kSumLimit))) {
            careful = true;
            break;
          }
          l += h;
          tmem_st_x32(tS, pk);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(bar_p_full(t, buf));
          RSFA_TRACE_EV(0x5000 + j);   // P handed over
        }
        if (!ok) break;
        if (careful) {
          // Redo key tile j with its scores loaded again from tensor memory, then go back to the
          // fast loop.  QK^T of this tile was issued before PV of the previous one, so O_t may
          // still be written: wait for PV_{j-1} (completion number pv_count + j - 1 of this tile).
          const int buf = j & 1;
          const uint32_t tS = tmem_base + lane_base + C::col_s(t, buf);
          if (j > 0) {
            ok = mbar_wait_warp(bar_pv_done(t), (pv_count + j - 1) & 1, abort_flag, wait_ns, kTagOFull);
            if (!ok) break;
            tc_fence_after_sync();
          }
          const int n0 = j * kKeysDb;
          int limit = S - 1 - n0;
          if (p.causal) limit = min(limit, row - n0);
          const uint64_t r = softmax_half_careful<D, kBf16>(tS, tS, tO, limit, scale_log2, headroom, m_used, l,
                                                            j > 0 ? 1 : 0);
          unpack_f32x2(r, m_used, l);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(bar_p_full(t, buf));
          ++j;
        }
      }
      if (!ok) break;
      pv_count += n;
      if constexpr (C::kEpi) {
        // ---- the epilogue warps store O: they get 1 / l; lse = m + log l is written here
        if (o_count > 0) {   // they are done with the item before (long ago, as a rule)
          ok = mbar_wait_warp(bar_o_free, (o_count - 1) & 1, abort_flag, wait_ns, kTagOFull);
          if (!ok) break;
        }
        ++o_count;
        s_inv_l[row_in_tile] = 1.f / l;
        mbar_arrive(bar_epi_ready);
        if (p.lse != nullptr && row < S)
          p.lse[static_cast<int64_t>(bh) * S + row] = m_used * p.sm_scale + logf(l);
        RSFA_TRACE_EV(0x7000);   // item handed to the epilogue warps
      }
      if constexpr (C::kEpi) continue;
      // ---- epilogue: O_t / l -> global, lse = m + log l (natural log; :400-404)
      ok = mbar_wait_warp(bar_o_full(t), o_count & 1, abort_flag, wait_ns, kTagOFull);
      if (!ok) break;
      ++o_count;
      tc_fence_after_sync();
      RSFA_TRACE_EV(0x6000);   // O seen
      const float inv_l = 1.f / l;
      const int b = bh / p.H, h = bh - b * p.H;
      // O_t / l -> global memory: each warp stages and stores its own 32 rows (store_o_rows)
      {
        const int wq = warp & 3;
        store_o_rows<D, kBf16, C::kStageBufs>(tO, inv_l, sStage + t * C::kStageBytes + wq * (4096 * C::kStageBufs), lane,
                                              &maps.o, tile_row0 + wq * 32, h, b, tile_row0 + wq * 32 < S);
      }
      if (p.lse != nullptr && row < S)
        p.lse[static_cast<int64_t>(bh) * S + row] = m_used * p.sm_scale + logf(l);
      tc_fence_before_sync();
      RSFA_TRACE_EV(0x7000);   // epilogue done
    }
    if (lane == 0) tma_store_wait_all();   // the last TMA stores must be complete before the CTA exits
  } else if (C::kEpi && warp >= C::kEpiWarp0) {
    // ============================================================== epilogue warps (D = 256)
    // Follow the scheduler like the other roles; per item: wait for 1 / l from the softmax group and
    // for the last PV, store O / l (store_o_rows), tell the MMA warp that O may be overwritten.
    const int wq = warp & 3;
    const uint32_t tO = tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + C::col_o(0);
    uint32_t item_count = 0;
    bool ok = true;
    RSFA_TRACE_DECL(1);
#ifdef RSFA_TRACE
    if (wq != 0) trace_buf = nullptr;
#endif
    while (ok) {
      const int slot = item_count & 1;
      ok = mbar_wait_warp(bar_sched_full0 + 8u * slot, (item_count >> 1) & 1, abort_flag, wait_ns, kTagSched);
      if (!ok) break;
      const int item = sched_ring[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sched_empty0 + 8u * slot);
      if (item >= sched.total_items) break;
      int bh, row0;
      decode(item, bh, row0);
      const int b = bh / p.H, h = bh - b * p.H;
      ok = mbar_wait_warp(bar_epi_ready, item_count & 1, abort_flag, wait_ns, kTagOFull);
      if (!ok) break;
      const float inv_l = s_inv_l[wq * 32 + lane];
      RSFA_TRACE_EV(0xe000);   // 1 / l seen
      ok = mbar_wait_warp(bar_o_full(0), item_count & 1, abort_flag, wait_ns, kTagOFull);
      if (!ok) break;
      tc_fence_after_sync();
      RSFA_TRACE_EV(0x6000);   // O seen
      store_o_rows<D, kBf16, C::kStageBufs>(tO, inv_l, sStage + wq * (4096 * C::kStageBufs), lane, &maps.o, row0 + wq * 32,
                                            h, b, row0 + wq * 32 < S);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_o_free);
      RSFA_TRACE_EV(0x7000);   // epilogue done
      ++item_count;
    }
    if (lane == 0) tma_store_wait_all();
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
  if (warp == C::kMmaWarp0) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0) {
    if (*abort_flag != 0) atomicCAS(p.status, 0, *abort_flag);
    queue_retire(p.tile_counter);
  }
}

template <int D, int NT, bool kBf16>
cudaError_t launch_db(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  using C = DbCfg<D, NT>;
  TmaMaps maps;
  if (!make_map(&maps.q, p.q, p, p.q_stride, kRowsDb) || !make_map(&maps.k, p.k, p, p.k_stride, kKeysDb) ||
      !make_map(&maps.v, p.v, p, p.v_stride, kKeysDb) || !make_map(&maps.o, p.o, p, p.o_stride, 32))
    return cudaErrorInvalidValue;
  SchedInfo sched;
  sched.items_per_head = (p.S + NT * kRowsDb - 1) / (NT * kRowsDb);
  sched.total_items = sched.items_per_head * p.B * p.H;
  auto kern = fwd_tcgen05_db_kernel<D, NT, kBf16>;
  static std::atomic<unsigned long long> smem_done{0};   // per kernel instantiation, bit per device
  cudaError_t e = set_dynamic_smem_once(smem_done, reinterpret_cast<const void*>(kern), C::kSmemBytes);
  if (e != cudaSuccess) return e;
  // No memset of the work queue: the last CTA of the launch that used it before put it back to zero.
  const int grid = sched.total_items < sm_count ? sched.total_items : sm_count;
  sched_set_tail(sched, p.B * p.H, p.causal, grid);
  e = launch_persistent(kern, grid, C::kThreads, C::kSmemBytes, stream, p.pdl != 0, maps, p, sched);
  if (e == cudaSuccess) *launches += 1;
  return e;
}

}  // namespace

cudaError_t launch_fwd_tcgen05_db(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches) {
  switch (p.D < 64 ? 64 : p.D) {
    case 64: return p.bf16 ? launch_db<64, 2, true>(p, sm_count, stream, launches) : launch_db<64, 2, false>(p, sm_count, stream, launches);
    case 128: return p.bf16 ? launch_db<128, 2, true>(p, sm_count, stream, launches) : launch_db<128, 2, false>(p, sm_count, stream, launches);
    case 256: return p.bf16 ? launch_db<256, 1, true>(p, sm_count, stream, launches) : launch_db<256, 1, false>(p, sm_count, stream, launches);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace rsfa
