// C ABI of librsfa_b200.so: argument validation, kernel selection, per-device
// workspace, the tile table and the host-buffer entry point.  The host side of
// the reference for this path is _attention.forward and get_tiling
// (ascend_rsfa/flash_attention_forward.py:547-665); see include/rsfa.h for the
// contract of every function.
#include <atomic>
#include <cstring>
#include <mutex>

#include <cuda_runtime.h>

#include "../../include/rsfa.h"
#include "common.cuh"

namespace {

constexpr int kMaxDevices = 64;
constexpr int kCounterSlots = 1024;  // one work queue (two words) per launch in flight

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  unsigned int* counters = nullptr;  // kCounterSlots work queues of two words (see FwdParams::tile_counter)
  int* status = nullptr;
  int* status_mirror = nullptr;      // pinned host copy of the status word (the "check_status" option)
  unsigned next_slot = 0;
  // staging buffers of rsfa_fwd_host (grow-only)
  void* stage[2][4] = {{nullptr, nullptr, nullptr, nullptr}, {nullptr, nullptr, nullptr, nullptr}};
  float* stage_lse[2] = {nullptr, nullptr};
  size_t stage_bytes = 0;
  size_t stage_lse_bytes = 0;
  cudaStream_t streams[2] = {nullptr, nullptr};
};

std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
std::atomic<long long> g_launches{0};
std::atomic<long long> g_force_path{-1};
std::atomic<long long> g_wait_limit_ms{2000};
std::atomic<long long> g_host_slab_heads{0};
std::atomic<long long> g_tcgen05_variant{-1};
std::atomic<long long> g_pdl{1};
std::atomic<long long> g_test_drop_load{-1};
std::atomic<long long> g_check_status{0};
#ifdef RSFA_TRACE
std::atomic<long long> g_trace_ptr{0};
#endif

int ensure_device(int device, DeviceState** out) {
  if (device < 0 || device >= kMaxDevices) return RSFA_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& d = g_dev[device];
  if (!d.ready) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
      cudaGetLastError();
      return RSFA_ERR_NO_DEVICE;
    }
    if (prop.major != 10) return RSFA_ERR_NO_DEVICE;  // the kernels are built for sm_100a only
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess) return RSFA_ERR_CUDA;
    if (cudaSetDevice(device) != cudaSuccess) return RSFA_ERR_CUDA;
    cudaError_t e = cudaMalloc(&d.counters, 2 * kCounterSlots * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&d.status, sizeof(int));
    if (e == cudaSuccess) e = cudaHostAlloc(&d.status_mirror, sizeof(int), cudaHostAllocDefault);
    if (e == cudaSuccess) *d.status_mirror = 0;
    if (e == cudaSuccess) e = cudaMemset(d.counters, 0, 2 * kCounterSlots * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(d.status, 0, sizeof(int));
    cudaSetDevice(prev);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return RSFA_ERR_CUDA;
    }
    d.sm_count = prop.multiProcessorCount;
    d.cc_major = prop.major;
    d.ready = true;
  }
  *out = &d;
  return RSFA_OK;
}

bool valid_head_dim(int D) { return D == 16 || D == 32 || D == 64 || D == 128 || D == 256; }

// Kernel family by shape.  The tcgen05 kernels take everything they are instantiated for (sm_scale > 0)
// except the smallest tiles: head dimension 16, and sequences of at most 64 keys at D <= 64, stay on
// the short-sequence kernel, the counterpart of the reference's single-tile kernels for N_CTX <= 128
// (:564).  Measured per call, host clock around call + synchronise / 4096 heads back to back:
//   S = 128 D = 128: 34 against 44 us at 128 heads, 93 against 346 us at 4096 (HBM rate against not);
//   S = 128 D = 64: 33 against 41 us; D = 256: 34 against 52 us; S = 128 D = 32: 66 against 107 us at 4096;
//   S = 64 D = 64: 32 against 34 us at 128 heads but 78 against 74 us at 4096; S = 64 D = 32: 77 against 38 us;
//   D = 16: 66 against 59 us at 4096 heads, 32 against 29 us at 2.
// The batch size does not enter: since a launch sets itself up under the tail of the one before, claims
// its first work item without the queue and needs no memset, the tcgen05 kernel starts as fast as
// the small one.
int choose_path(int S, int D, float sm_scale) {
  const long long forced = g_force_path.load();
  const bool tc_ok = rsfa::tcgen05_supports(S, D, sm_scale);
  if (forced == RSFA_PATH_GENERIC) return RSFA_PATH_GENERIC;
  if (forced == RSFA_PATH_TCGEN05 && tc_ok) return RSFA_PATH_TCGEN05;
  if (!tc_ok) return RSFA_PATH_GENERIC;
  if (S > 128) return RSFA_PATH_TCGEN05;
  return (D >= 32 && !(S <= 64 && D <= 64)) ? RSFA_PATH_TCGEN05 : RSFA_PATH_GENERIC;
}

// Tile a call runs: on the tcgen05 path the request is honoured when instantiated, otherwise the
// tile table decides; the generic kernel has one tile per head dimension.
void tile_of_path(int path, int S, int D, int causal, int req_bm, int req_bn, int* bm, int* bn) {
  if (path == RSFA_PATH_TCGEN05) {
    rsfa::tcgen05_resolve_tile(S, D, causal, req_bm, req_bn, static_cast<int>(g_tcgen05_variant.load()), bm, bn);
  } else {
    *bm = 64;
    *bn = (D >= 256) ? 32 : 64;
  }
}

}  // namespace

namespace rsfa {
void count_launches(long long n) { g_launches.fetch_add(n); }
unsigned long long option_wait_limit_ns() {
  return static_cast<unsigned long long>(g_wait_limit_ms.load()) * 1000000ull;
}
int option_pdl() { return static_cast<int>(g_pdl.load()); }
int option_test_drop_load() { return static_cast<int>(g_test_drop_load.load()); }
}  // namespace rsfa

extern "C" {

int rsfa_version(void) { return 100; }

const char* rsfa_strerror(int code) {
  switch (code) {
    case RSFA_OK: return "ok";
    case RSFA_ERR_INVALID_ARGUMENT: return "invalid argument (shape, stride, alignment, tile or dtype)";
    case RSFA_ERR_UNSUPPORTED: return "unsupported configuration";
    case RSFA_ERR_CUDA: return "CUDA call failed";
    case RSFA_ERR_DEVICE_STATUS: return "a kernel reported a non-zero device status (bounded wait expired)";
    case RSFA_ERR_NO_DEVICE: return "no usable sm_100 CUDA device";
    case RSFA_ERR_TOO_LARGE: return "problem too large: beyond the fixed scratch of the allocation-free entry point, or more CTAs than a grid holds";
    default: return "unknown error code";
  }
}

long long rsfa_launch_count(void) { return g_launches.load(); }

int rsfa_set_option(const char* name, long long value) {
  if (name == nullptr) return RSFA_ERR_INVALID_ARGUMENT;
  if (std::strcmp(name, "force_path") == 0) {
    if (value < -1 || value > 1) return RSFA_ERR_INVALID_ARGUMENT;
    g_force_path.store(value);
    return RSFA_OK;
  }
  if (std::strcmp(name, "wait_limit_ms") == 0) {
    if (value < 1 || value > 60000) return RSFA_ERR_INVALID_ARGUMENT;
    g_wait_limit_ms.store(value);
    return RSFA_OK;
  }
#ifdef RSFA_TRACE
  if (std::strcmp(name, "trace_ptr") == 0) {
    g_trace_ptr.store(value);
    return RSFA_OK;
  }
#endif
  if (std::strcmp(name, "tcgen05_variant") == 0) {
    if (value < -1 || value > 2) return RSFA_ERR_INVALID_ARGUMENT;
    g_tcgen05_variant.store(value);
    return RSFA_OK;
  }
  if (std::strcmp(name, "host_slab_heads") == 0) {
    if (value < 0) return RSFA_ERR_INVALID_ARGUMENT;
    g_host_slab_heads.store(value);
    return RSFA_OK;
  }
  if (std::strcmp(name, "pdl") == 0) {
    if (value < 0 || value > 1) return RSFA_ERR_INVALID_ARGUMENT;
    g_pdl.store(value);
    return RSFA_OK;
  }
  if (std::strcmp(name, "check_status") == 0) {
    if (value < 0 || value > 1) return RSFA_ERR_INVALID_ARGUMENT;
    g_check_status.store(value);
    return RSFA_OK;
  }
  if (std::strcmp(name, "test_drop_load") == 0) {
    if (value < -1 || value > 1000000) return RSFA_ERR_INVALID_ARGUMENT;
    g_test_drop_load.store(value);
    return RSFA_OK;
  }
  return RSFA_ERR_INVALID_ARGUMENT;
}

long long rsfa_get_option(const char* name) {
  if (name == nullptr) return RSFA_ERR_INVALID_ARGUMENT;
  if (std::strcmp(name, "force_path") == 0) return g_force_path.load();
  if (std::strcmp(name, "wait_limit_ms") == 0) return g_wait_limit_ms.load();
  if (std::strcmp(name, "host_slab_heads") == 0) return g_host_slab_heads.load();
  if (std::strcmp(name, "tcgen05_variant") == 0) return g_tcgen05_variant.load();
  if (std::strcmp(name, "pdl") == 0) return g_pdl.load();
  if (std::strcmp(name, "check_status") == 0) return g_check_status.load();
  if (std::strcmp(name, "test_drop_load") == 0) return g_test_drop_load.load();
  if (std::strcmp(name, "workspace_devices") == 0) {   // read-only: devices on which rsfa_fwd has made its workspace
    std::lock_guard<std::mutex> lock(g_mu);
    long long n = 0;
    for (int i = 0; i < kMaxDevices; ++i) n += g_dev[i].ready ? 1 : 0;
    return n;
  }
  return RSFA_ERR_INVALID_ARGUMENT;
}

int rsfa_sm_count(int device) {
  int major = 0, sms = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_NO_DEVICE;
  }
  return major == 10 ? sms : RSFA_ERR_NO_DEVICE;   // the kernels are built for sm_100a only
}

int rsfa_select_path(int S, int D, int causal, float sm_scale, int block_m, int block_n, int dtype,
                     int* path, int* tile_m, int* tile_n) {
  if (path == nullptr || S < 1 || !valid_head_dim(D) || block_m < 1 || block_n < 1 ||
      (dtype != RSFA_DTYPE_F16 && dtype != RSFA_DTYPE_BF16))
    return RSFA_ERR_INVALID_ARGUMENT;
  *path = choose_path(S, D, sm_scale);
  int bm, bn;
  tile_of_path(*path, S, D, causal, block_m, block_n, &bm, &bn);
  if (tile_m != nullptr) *tile_m = bm;
  if (tile_n != nullptr) *tile_n = bn;
  return RSFA_OK;
}

int rsfa_get_tiling(int B, int H, int S, int D, int causal, int* block_m, int* block_n) {
  if (block_m == nullptr || block_n == nullptr || B < 1 || H < 1 || S < 1 || !valid_head_dim(D))
    return RSFA_ERR_INVALID_ARGUMENT;
  // The tile of the kernel family the shape runs on (sm_scale is taken as positive here): a row of
  // the tile table on the tcgen05 path, the short-sequence kernel's single tile otherwise.
  const int path = choose_path(S, D, 1.0f);
  tile_of_path(path, S, D, causal, 0, 0, block_m, block_n);
  return RSFA_OK;
}

int rsfa_work_items(int B, int H, int S, int D, int causal, float sm_scale, long long* items) {
  if (items == nullptr || B < 1 || H < 1 || S < 1 || !valid_head_dim(D)) return RSFA_ERR_INVALID_ARGUMENT;
  const long long heads = static_cast<long long>(B) * H;
  if (choose_path(S, D, sm_scale) == RSFA_PATH_GENERIC) {
    *items = rsfa::generic_grid_blocks(B, H, S);
  } else {
    const int rows = (D == 256) ? 128 : 256;   // query rows per work item of the tcgen05 kernels
    *items = heads * ((S + rows - 1) / rows);
  }
  (void)causal;   // masked row blocks are still work items (lighter ones)
  return RSFA_OK;
}

int rsfa_device_status(int device, int* raw) {
  if (device < 0 || device >= kMaxDevices) return RSFA_ERR_INVALID_ARGUMENT;
  // Looks only at what exists: the workspace of rsfa_fwd if a call has created it, the static block
  // of rsfa_fwd_noalloc if that has been used.  It allocates nothing itself.
  DeviceState* d = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_dev[device].ready) d = &g_dev[device];
  }
  int* na = rsfa::noalloc_status_word(device);
  int prev = 0;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_NO_DEVICE;
  }
  int word = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess && d != nullptr) {
    e = cudaMemcpy(&word, d->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && word != 0) e = cudaMemset(d->status, 0, sizeof(int));
    *d->status_mirror = 0;
  }
  if (e == cudaSuccess && na != nullptr) {
    int word_na = 0;
    e = cudaMemcpy(&word_na, na, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && word_na != 0) {
      e = cudaMemset(na, 0, sizeof(int));
      if (word == 0) word = word_na;
    }
  }
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_CUDA;
  }
  if (raw != nullptr) *raw = word;
  return word == 0 ? RSFA_OK : RSFA_ERR_DEVICE_STATUS;
}

int rsfa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int S, int D,
             const int64_t* strides, int causal, float sm_scale, int block_m, int block_n, int dtype,
             void* stream) {
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || strides == nullptr)
    return RSFA_ERR_INVALID_ARGUMENT;
  if (B < 1 || H < 1 || S < 1 || !valid_head_dim(D)) return RSFA_ERR_INVALID_ARGUMENT;
  if (block_m < 1 || block_n < 1) return RSFA_ERR_INVALID_ARGUMENT;
  if (dtype != RSFA_DTYPE_F16 && dtype != RSFA_DTYPE_BF16) return RSFA_ERR_INVALID_ARGUMENT;
  if (!(sm_scale == sm_scale)) return RSFA_ERR_INVALID_ARGUMENT;  // NaN
  const void* ptrs[4] = {q, k, v, o};
  for (int t = 0; t < 4; ++t) {
    if ((reinterpret_cast<uintptr_t>(ptrs[t]) & 15u) != 0) return RSFA_ERR_INVALID_ARGUMENT;
    const int64_t* st = strides + 4 * t;
    if (st[3] != 1) return RSFA_ERR_INVALID_ARGUMENT;
    const int extent[3] = {B, H, S};
    for (int i = 0; i < 3; ++i) {
      if (extent[i] > 1 && (st[i] < D || (st[i] & 7) != 0)) return RSFA_ERR_INVALID_ARGUMENT;
    }
  }
  if (static_cast<long long>(B) * H > 2147483647LL / 4) return RSFA_ERR_INVALID_ARGUMENT;

  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_NO_DEVICE;
  }
  DeviceState* d = nullptr;
  const int rc = ensure_device(device, &d);
  if (rc != RSFA_OK) return rc;

  rsfa::FwdParams p;
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
  p.status = d->status;
  const bool check_status = g_check_status.load() != 0;
  if (check_status && *static_cast<volatile int*>(d->status_mirror) != 0) {
    // A kernel of an earlier call left a non-zero status word and its copy has reached the host:
    // this call is not launched; rsfa_device_status() reports the word and clears it.
    return RSFA_ERR_DEVICE_STATUS;
  }
  {
    std::lock_guard<std::mutex> lock(g_mu);
    p.tile_counter = d->counters + 2 * (d->next_slot++ % kCounterSlots);
  }
  p.wait_limit_ns = rsfa::option_wait_limit_ns();
  p.pdl = rsfa::option_pdl();
  p.test_drop_load = rsfa::option_test_drop_load();
#ifdef RSFA_TRACE
  p.trace = reinterpret_cast<unsigned long long*>(g_trace_ptr.load());
#endif
  p.variant = static_cast<int>(g_tcgen05_variant.load());

  long long launches = 0;
  cudaError_t e;
  const int path = choose_path(S, D, sm_scale);
  // one CTA per (head, block of 64 rows), all on grid.x, whose limit is 2^31 - 1
  if (path == RSFA_PATH_GENERIC && rsfa::generic_grid_blocks(B, H, S) > 2147483647LL) return RSFA_ERR_TOO_LARGE;
  {
    int bm = 0, bn = 0;
    tile_of_path(path, S, D, causal, block_m, block_n, &bm, &bn);
    p.tile_n = bn;
  }
  if (path == RSFA_PATH_TCGEN05)
    e = rsfa::launch_fwd_tcgen05(p, d->sm_count, static_cast<cudaStream_t>(stream), &launches);
  else
    e = rsfa::launch_fwd_generic(p, static_cast<cudaStream_t>(stream), &launches);
  g_launches.fetch_add(launches);
  if (e == cudaSuccess && check_status) {
    // The status word follows the kernels to the host on the same stream; the next call looks at it.
    if (cudaMemcpyAsync(d->status_mirror, d->status, sizeof(int), cudaMemcpyDeviceToHost,
                        static_cast<cudaStream_t>(stream)) != cudaSuccess)
      cudaGetLastError();
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_CUDA;
  }
  return RSFA_OK;
}

int rsfa_fwd_host(const void* q_host, const void* k_host, const void* v_host, void* o_host, float* lse_host,
                  int B, int H, int S, int D, int causal, float sm_scale, int block_m, int block_n, int dtype,
                  int device) {
  if (q_host == nullptr || k_host == nullptr || v_host == nullptr || o_host == nullptr)
    return RSFA_ERR_INVALID_ARGUMENT;
  if (B < 1 || H < 1 || S < 1 || !valid_head_dim(D) || block_m < 1 || block_n < 1)
    return RSFA_ERR_INVALID_ARGUMENT;
  if (dtype != RSFA_DTYPE_F16 && dtype != RSFA_DTYPE_BF16) return RSFA_ERR_INVALID_ARGUMENT;
  DeviceState* d = nullptr;
  int rc = ensure_device(device, &d);
  if (rc != RSFA_OK) return rc;
  int prev = 0;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) return RSFA_ERR_CUDA;

  const long long heads = static_cast<long long>(B) * H;
  const size_t head_bytes = static_cast<size_t>(S) * D * 2;
  // Slab size: enough heads to fill the device several times over, small enough that the first
  // kernel starts early; at most 1 GiB per staged tensor.
  long long slab = g_host_slab_heads.load();
  if (slab <= 0) {
    slab = (heads + 7) / 8;
    const long long cap = static_cast<long long>((1ull << 30) / head_bytes);
    if (slab > cap) slab = cap;
    if (slab < 1) slab = 1;
  }
  if (slab > heads) slab = heads;
  const size_t need = static_cast<size_t>(slab) * head_bytes;
  const size_t need_lse = static_cast<size_t>(slab) * S * sizeof(float);

  cudaError_t e = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    for (int s = 0; s < 2 && e == cudaSuccess; ++s)
      if (d->streams[s] == nullptr) e = cudaStreamCreateWithFlags(&d->streams[s], cudaStreamNonBlocking);
    if (e == cudaSuccess && d->stage_bytes < need) {
      for (int s = 0; s < 2; ++s)
        for (int t = 0; t < 4; ++t) {
          if (d->stage[s][t] != nullptr) cudaFree(d->stage[s][t]);
          d->stage[s][t] = nullptr;
          if (e == cudaSuccess) e = cudaMalloc(&d->stage[s][t], need);
        }
      d->stage_bytes = (e == cudaSuccess) ? need : 0;
    }
    if (e == cudaSuccess && lse_host != nullptr && d->stage_lse_bytes < need_lse) {
      for (int s = 0; s < 2; ++s) {
        if (d->stage_lse[s] != nullptr) cudaFree(d->stage_lse[s]);
        d->stage_lse[s] = nullptr;
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&d->stage_lse[s]), need_lse);
      }
      d->stage_lse_bytes = (e == cudaSuccess) ? need_lse : 0;
    }
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaSetDevice(prev);
    return RSFA_ERR_CUDA;
  }

  // Heads are independent, so a slab is treated as a [1, n, S, D] problem.
  int result = RSFA_OK;
  int turn = 0;
  for (long long h0 = 0; h0 < heads && result == RSFA_OK; h0 += slab, turn ^= 1) {
    const long long n = (heads - h0 < slab) ? (heads - h0) : slab;
    const size_t bytes = static_cast<size_t>(n) * head_bytes;
    const size_t off = static_cast<size_t>(h0) * head_bytes;
    cudaStream_t st = d->streams[turn];
    const void* src[3] = {q_host, k_host, v_host};
    for (int t = 0; t < 3 && e == cudaSuccess; ++t)
      e = cudaMemcpyAsync(d->stage[turn][t], static_cast<const char*>(src[t]) + off, bytes,
                          cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) break;
    const int64_t sd = static_cast<int64_t>(S) * D;
    const int64_t strides[16] = {n * sd, sd, D, 1, n * sd, sd, D, 1, n * sd, sd, D, 1, n * sd, sd, D, 1};
    float* lse_dev = (lse_host != nullptr) ? d->stage_lse[turn] : nullptr;
    result = rsfa_fwd(d->stage[turn][0], d->stage[turn][1], d->stage[turn][2], d->stage[turn][3], lse_dev, 1,
                      static_cast<int>(n), S, D, strides, causal, sm_scale, block_m, block_n, dtype, st);
    if (result != RSFA_OK) break;
    e = cudaMemcpyAsync(static_cast<char*>(o_host) + off, d->stage[turn][3], bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && lse_host != nullptr)
      e = cudaMemcpyAsync(lse_host + static_cast<size_t>(h0) * S, lse_dev, static_cast<size_t>(n) * S * sizeof(float),
                          cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) break;
  }
  for (int s = 0; s < 2; ++s) {
    const cudaError_t es = cudaStreamSynchronize(d->streams[s]);
    if (e == cudaSuccess) e = es;
  }
  cudaSetDevice(prev);
  if (result != RSFA_OK) return result;
  if (e != cudaSuccess) {
    cudaGetLastError();
    return RSFA_ERR_CUDA;
  }
  return RSFA_OK;
}

}  // extern "C"
