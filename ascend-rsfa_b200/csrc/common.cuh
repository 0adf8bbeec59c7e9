// Types shared by the kernels and the C-ABI dispatcher.
#pragma once
#include <atomic>
#include <cstdint>
#include <cuda_runtime.h>

namespace rsfa {

// One attention problem as the kernels see it: raw pointers plus element strides.
struct FwdParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;  // may be null
  int B, H, S, D;
  int64_t q_stride[3];  // batch, head, row (the innermost stride is 1)
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int causal;
  float sm_scale;
  int bf16;
  int tile_n;   // keys per tile on the tcgen05 path: 128 (single-buffered S) or 64 (double-buffered S)
  int variant;  // the "tcgen05_variant" option: -1 automatic, 0 / 1 / 2 force a kernel of the family
  int* status;                 // device status word, never null
  // Work queue of the persistent kernels: word [0] hands out work items, word [1] counts the CTAs
  // that have finished.  Both are zero before a launch; the CTA that finishes last puts them back
  // to zero, so the next launch that gets this pair needs no memset in front of it.
  unsigned int* tile_counter;
  unsigned long long wait_limit_ns;
  int pdl;             // 1: launch with programmatic stream serialisation (the "pdl" option)
  // Test hook (the "test_drop_load" option, -1 = off): the producer of the 128-key tcgen05 kernel
  // leaves out its n-th K/V tile load together with the barrier arrival that announces it.  Nothing
  // is in flight for that tile and no address is touched; the consumer's bounded wait simply runs
  // out, which is how the tests reach the wait-expired path on a healthy GPU.
  int test_drop_load;
#ifdef RSFA_TRACE
  unsigned long long* trace;  // debug builds only: per-role event log of CTA 0
#endif
};

// Raises a kernel's dynamic shared-memory limit once per device instead of on every call (the
// attribute stays with the function in that device's context).  `done` is a bit mask by device
// ordinal, one per kernel instantiation (a static of the launcher that owns the kernel).
inline cudaError_t set_dynamic_smem_once(std::atomic<unsigned long long>& done, const void* kern, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && ((done.load(std::memory_order_acquire) >> dev) & 1ull)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  return e;
}

// Launchers implemented in the kernel translation units.  Each returns a cudaError_t
// from the launch itself and bumps *launches by the number of kernels it started.
cudaError_t launch_fwd_generic(const FwdParams& p, cudaStream_t stream, long long* launches);
// CTAs the short-sequence kernel launches: one per (batch, head, block of 64 query rows), all on grid.x.
long long generic_grid_blocks(int B, int H, int S);
cudaError_t launch_fwd_tcgen05(const FwdParams& p, int sm_count, cudaStream_t stream,
                               long long* launches);
// The double-buffered-S family (D = 64, 128, 256), selected by launch_fwd_tcgen05.
cudaError_t launch_fwd_tcgen05_db(const FwdParams& p, int sm_count, cudaStream_t stream,
                                  long long* launches);
// The D = 64 kernel with P in tensor-memory columns of its own (fwd_tcgen05_sp.cu), selected by launch_fwd_tcgen05.
cudaError_t launch_fwd_tcgen05_sp(const FwdParams& p, int sm_count, cudaStream_t stream, long long* launches);
// Whether a problem's work items can be numbered in that kernel's scheduler ring (fewer than 2^27).
bool tcgen05_sp_fits(const FwdParams& p);
// Tile the tcgen05 family runs for a problem: the requested (block_m, block_n) when that tile is
// instantiated for D, otherwise the tile table's row for (S, D, causal).  `variant` = -1 lets the
// request / table decide, 0 forces 128-key tiles with single-buffered S, 1 forces 64-key tiles (D <= 128
// only), 2 forces 128-key tiles with the separate-P kernel where it exists (D = 64).
void tcgen05_resolve_tile(int S, int D, int causal, int req_bm, int req_bn, int variant, int* bm, int* bn);
// Adds to the process-wide kernel-launch counter behind rsfa_launch_count().
void count_launches(long long n);
// Current values of the "wait_limit_ms" (in ns), "pdl" and "test_drop_load" options.
unsigned long long option_wait_limit_ns();
int option_pdl();
int option_test_drop_load();
// Device address of the status word in the static scratch block of rsfa_fwd_noalloc on `device`, or
// null while that entry point has not been used there.
int* noalloc_status_word(int device);
// True when the tcgen05 kernel is instantiated for this head dimension.
bool tcgen05_supports(int S, int D, float sm_scale);

}  // namespace rsfa
