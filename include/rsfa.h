/*
 * rsfa.h — C ABI of the B200 FlashAttention-2 forward library (librsfa_b200.so).
 *
 * The library is the device side of the Python operator
 *   ascend_rsfa.flash_attention_forward.attention(q, k, v, causal, sm_scale, BLOCK_M, BLOCK_N)
 * and of get_tiling(batch, heads, seq, head_dim, causal).  All tensors are
 * [B, H, S, D] with 16-bit elements; all pointers are plain device (or, where
 * stated, host) addresses; sizes are ints; nothing here depends on PyTorch.
 * Every function returns RSFA_OK (0) or a negative RSFA_ERR_* code and never
 * aborts the process.  rsfa_strerror() names a code.
 *
 * Citations of the form file:line point into the reference project
 * (ascend_rsfa/flash_attention_forward.py unless another file is named).
 */
#ifndef RSFA_H_
#define RSFA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RSFA_API __attribute__((visibility("default")))
#else
#define RSFA_API
#endif

#define RSFA_OK 0
#define RSFA_ERR_INVALID_ARGUMENT (-1) /* bad shape, stride, alignment, tile or dtype           */
#define RSFA_ERR_UNSUPPORTED (-2)      /* legal for the reference, not built here               */
#define RSFA_ERR_CUDA (-3)             /* a CUDA runtime / driver call failed                   */
#define RSFA_ERR_DEVICE_STATUS (-4)    /* a kernel reported a non-zero status (bounded wait...) */
#define RSFA_ERR_NO_DEVICE (-5)        /* no CUDA device, or not an sm_100 device               */
#define RSFA_ERR_TOO_LARGE (-6)        /* beyond rsfa_fwd_noalloc's fixed scratch, or > 2^31-1 CTAs */

#define RSFA_DTYPE_F16 0
#define RSFA_DTYPE_BF16 1

/* Kernel families a call can be routed to (see rsfa_select_path). */
#define RSFA_PATH_GENERIC 0 /* mma.sync kernel: any S, D in {16,32,64,128,256}; the smallest tiles, scale <= 0 */
#define RSFA_PATH_TCGEN05 1 /* warp-specialised tcgen05 / TMEM / TMA kernel                         */

/*
 * Forward attention on device tensors.  Replaces _attention.forward (:547-616)
 * with everything it dispatches to: _attn_fwd_small / _attn_fwd_small_causal
 * (:26-159), _attn_fwd with _attn_fwd_inner / _attn_fwd_inner_d64_nc (:163-404)
 * and the two-launch causal split _run_causal_split (:493-541).
 *
 *   q, k, v, o   device pointers, element (b,h,s,d) at base + b*st[0] + h*st[1] + s*st[2] + d*st[3]
 *   lse          optional device pointer to B*H*S floats (contiguous): m + log(l) per row in
 *                natural-log units (:400-404); may be NULL.  Written for causal calls too.
 *   strides      16 element strides: q[4], k[4], v[4], o[4].  The innermost stride must be 1, the
 *                others multiples of 8 elements, and the base pointers 16-byte aligned.
 *   causal       0/1; the mask keeps key j <= query i, square and aligned top-left (:153, :194).
 *   sm_scale     multiplies q.k before the softmax (:84, :199).
 *   block_m/n    the reference's BLOCK_M / BLOCK_N.  Results do not depend on them; they are a
 *                request that is honoured when such a tile is instantiated and otherwise replaced
 *                by the table's choice (rsfa_get_tiling).  Must be positive.
 *   dtype        RSFA_DTYPE_F16 or RSFA_DTYPE_BF16 (:698 tests one bf16 case).
 *   stream       a cudaStream_t (NULL = default stream).  The call is asynchronous like the
 *                reference's kernel launches; it does not synchronise.
 *
 * Concurrency: calls on different streams of one device may overlap on the GPU.  Every call is one
 * kernel launch and takes a work queue of its own out of 1024 per device (the kernel puts it back to
 * zero when it ends); nothing else in device memory is shared between calls except the status word,
 * which is per device.
 *
 * Errors: D outside {16,32,64,128,256} or mismatched (the reference asserts, :551-554), B/H/S < 1,
 * misaligned pointers or strides -> RSFA_ERR_INVALID_ARGUMENT.  A device status left by an earlier
 * launch on the same device is reported by rsfa_device_status, not here.
 */
RSFA_API int rsfa_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
             int B, int H, int S, int D, const int64_t* strides,
             int causal, float sm_scale, int block_m, int block_n, int dtype, void* stream);

/*
 * The same operator on HOST buffers (contiguous [B,H,S,D]); the library stages heads through the
 * device in slabs, overlapping host->device copies, kernels and device->host copies on its own
 * streams, and returns when o_host (and lse_host, if not NULL) is complete.  This is the call the
 * reference's harness makes when its tensors start on the host: tensor creation + attention() +
 * synchronize (benchmarks/run_final_benchmark.py:104-124).  Buffers may be pageable; pinned
 * buffers copy faster.  `device` is the CUDA ordinal to use.  Calls for one device share its staging
 * buffers and streams: issue them one at a time per device (different devices are independent).
 */
RSFA_API int rsfa_fwd_host(const void* q_host, const void* k_host, const void* v_host, void* o_host,
                  float* lse_host, int B, int H, int S, int D, int causal, float sm_scale,
                  int block_m, int block_n, int dtype, int device);

/*
 * rsfa_fwd for callers that must not allocate device memory.  It has no counterpart in the
 * reference; it exists for hosts where a cudaMalloc inside an operator call is not acceptable:
 * servers that give all device memory to their own arena at start-up, latency-critical loops in
 * which an allocation may stall the device, plugins whose memory is accounted by the embedding
 * process.  rsfa_fwd keeps its work-queue counter and status word in a buffer it cudaMallocs on
 * first use; this entry point runs the same tcgen05 kernel with that scratch in a 256-byte block
 * of static device memory inside the library (held by every GPU that loads the library until the
 * process exits) and calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Arguments as rsfa_fwd, without block_m / block_n: the tile table decides, so either tcgen05
 * kernel family may run, as in rsfa_fwd (64-key tiles at D = 256 and for short causal sequences,
 * 128-key tiles otherwise, the separate-P kernel at D <= 64).
 * Every in-kernel wait is bounded by the "wait_limit_ms" option, as in rsfa_fwd.  Limits: only
 * shapes the tcgen05 kernels are built for (sm_scale > 0; D = 16 and 32 run on the D = 64 kernel) -> otherwise
 * RSFA_ERR_UNSUPPORTED; at most 2^30 work items (B * H * ceil(S / 256), or ceil(S / 128) at D = 256), because the queue counter
 * is a single 32-bit word of the block -> otherwise RSFA_ERR_TOO_LARGE.
 *
 * The first call on a device looks up the device address of the static block (one
 * cudaGetSymbolAddress with that device current); make that first call outside any stream
 * capture.  All calls on a device share the one block, which keeps the previous call's contents:
 * each call clears the work queue and the status word on `stream` before its kernel, so calls on
 * one stream are safe back to back, but two calls whose kernels can overlap on the GPU (different
 * streams, no dependency) race on the queue and must be ordered by the caller.  A bounded wait
 * that runs out leaves the output incomplete and a code in the block's status word, which
 * rsfa_device_status reports together with rsfa_fwd's (the next rsfa_fwd_noalloc call clears it).
 */
RSFA_API int rsfa_fwd_noalloc(const void* q, const void* k, const void* v, void* o, float* lse,
                              int B, int H, int S, int D, const int64_t* strides,
                              int causal, float sm_scale, int dtype, void* stream);

/*
 * Tile lookup.  Replaces get_tiling (:624-665): the reference keys a 32-entry dict by the full
 * (Z, H, N_CTX, HEAD_DIM, causal) tuple and raises KeyError otherwise; here the table is keyed by
 * (S, D, causal) only, any B and H are accepted, and only tiles that are instantiated are returned.
 */
RSFA_API int rsfa_get_tiling(int B, int H, int S, int D, int causal, int* block_m, int* block_n);

/*
 * Which kernel family rsfa_fwd would use for this problem, and the tile it would run
 * (after snapping block_m/block_n).  Counterpart of the dispatch in _attention.forward (:564-610).
 * tile_m / tile_n may be NULL.  The tcgen05 kernels run every shape with sm_scale > 0 except head
 * dimension 16 at S <= 128 and sequences of at most 64 keys at D <= 64, which the short-sequence
 * kernel serves (measured per call; the batch size does not enter).
 */
RSFA_API int rsfa_select_path(int S, int D, int causal, float sm_scale, int block_m, int block_n, int dtype,
                     int* path, int* tile_m, int* tile_n);

/*
 * Number of work items rsfa_fwd splits this problem into: (batch, head, block of query rows) units
 * that the persistent tcgen05 kernels hand out through their queue (256 rows each, 128 at D = 256),
 * or the CTAs of the short-sequence kernel (64 rows each, all on grid.x, so the count may exceed
 * 65535).  Counterpart of NUM_BLOCKS = cdiv(N_CTX, BLOCK_M) * Z * H (:289-294).  Needs no device.
 */
RSFA_API int rsfa_work_items(int B, int H, int S, int D, int causal, float sm_scale, long long* items);

/*
 * Number of streaming multiprocessors of a device: the grid size of the persistent kernel.
 * Replaces get_num_compute_cores (:19-21).  Returns the count (> 0) or a negative error.
 */
RSFA_API int rsfa_sm_count(int device);

/*
 * Synchronise `device` and return the status word its kernels share (this call allocates nothing
 * and reads only the scratch that rsfa_fwd or rsfa_fwd_noalloc has already set up on the device): RSFA_OK, or
 * RSFA_ERR_DEVICE_STATUS with the raw word in *raw (if not NULL): (1 << 16) | tag, where tag names
 * the wait that ran out.  Reading clears the word.  rsfa_fwd itself returns RSFA_OK for a call
 * whose kernel later gives up (the launch is asynchronous) and the output of that call is then
 * incomplete: callers that care call this function at their synchronisation points, or set the
 * "check_status" option, under which every rsfa_fwd copies the word to the host behind its kernels
 * and the next rsfa_fwd on that device returns RSFA_ERR_DEVICE_STATUS without launching once a
 * non-zero word has arrived (this function then reports and clears it).
 * The reference has no counterpart: its kernels cannot time out.
 */
RSFA_API int rsfa_device_status(int device, int* raw);

/* Count of kernels this library has launched in this process (all devices). */
RSFA_API long long rsfa_launch_count(void);

/*
 * Tuning / test knobs.  Names: "force_path" (-1 auto, 0 generic, 1 tcgen05),
 * "wait_limit_ms" (bound of every in-kernel wait, default 2000), "tcgen05_variant" (-1: the requested tile if
 * instantiated, else the tile table, and at D = 64 with 128-key tiles the separate-P kernel followed
 * by a second launch over the work items it could not finish; 0 / 1 force the single-buffered 128-key /
 * double-buffered 64-key kernel for D <= 128; 2 forces 128-key tiles with the separate-P kernel where
 * it exists), "host_slab_heads"
 * (heads per staging slab of rsfa_fwd_host, 0 = automatic), "pdl" (1, the default: the tcgen05 kernels
 * are launched with programmatic stream serialisation, so the set-up of a launch overlaps the tail of
 * the kernel in front of it on the stream; they wait for that kernel before touching global memory),
 * "check_status" (0 / 1, see rsfa_device_status), "test_drop_load" (-1 = off; n >= 0: every CTA of the
 * 128-key tcgen05 kernel leaves out its n-th K/V tile load and the barrier arrival that announces it,
 * so that a bounded wait runs out - for tests of the wait-expired path; the output of such a call
 * is incomplete).
 * rsfa_get_option also answers "workspace_devices": the number of devices on which rsfa_fwd has
 * created its workspace (0 in a process that has only used rsfa_fwd_noalloc).
 * Unknown names -> RSFA_ERR_INVALID_ARGUMENT.
 */
RSFA_API int rsfa_set_option(const char* name, long long value);
RSFA_API long long rsfa_get_option(const char* name);

RSFA_API const char* rsfa_strerror(int code);

/* major*10000 + minor*100 + patch */
RSFA_API int rsfa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RSFA_H_ */
