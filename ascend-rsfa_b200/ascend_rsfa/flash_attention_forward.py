"""FlashAttention-2 forward for NVIDIA B200 behind the ASCEND-RSFA operator API.

Drop-in for the reference module of the same name
(ascend_rsfa/flash_attention_forward.py): the same names, argument order and
return types —

    attention(q, k, v, causal, sm_scale, BLOCK_M, BLOCK_N) -> o        (:622)
    get_tiling(batch, heads, seq, head_dim, causal) -> (BLOCK_M, BLOCK_N)  (:624)
    class _attention(torch.autograd.Function)                           (:547)
    get_num_compute_cores()                                             (:19)

— on [B, H, S, D] fp16 (or bf16) CUDA tensors.  The work is done by hand-written
sm_100a kernels in librsfa_b200.so, reached through its C ABI with ctypes; this
file only validates, allocates the output like the reference does
(``torch.empty_like(q)``, :558) and passes raw pointers, strides and the current
CUDA stream.  There is no Triton, no PyTorch math and no CPU path here: without
the library, or on a non-CUDA tensor, the call raises.

Differences from the reference, all on purpose:
* BLOCK_M / BLOCK_N are a request.  Results never depend on them (true of the
  reference too); a tile that is not instantiated is replaced by the table's.
* get_tiling is keyed by (seq, head_dim, causal) and accepts any batch / heads,
  where the reference raises KeyError outside its 32 listed tuples (:665).
* Sequence lengths that are not a multiple of the tile are handled (the
  reference silently assumes divisibility), and the causal call also produces
  the log-sum-exp (the reference writes it on the non-causal path only, :400-404).
"""
import ctypes

import torch

from . import _capi

_lib = _capi.load()

DEVICE = "cuda"
_DTYPES = {torch.float16: _capi.RSFA_DTYPE_F16, torch.bfloat16: _capi.RSFA_DTYPE_BF16}

# The raw handle of the current stream without building a torch.cuda.Stream object (3 us per call,
# a tenth of a short-sequence call); the public route is the fallback.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _current_stream(index):
    if _raw_stream is not None:
        return _raw_stream(index)
    return torch.cuda.current_stream(index).cuda_stream


# ctypes stride arrays of dense [B, H, S, D] problems, by shape: building one costs 2 us
_dense_strides = {}


def _strides_of(qd, kd, vd, o):
    if qd.is_contiguous() and kd.is_contiguous() and vd.is_contiguous() and o.is_contiguous():
        arr = _dense_strides.get(qd.shape)
        if arr is None:
            if len(_dense_strides) > 256:
                _dense_strides.clear()
            arr = _dense_strides[qd.shape] = (ctypes.c_int64 * 16)(*(tuple(o.stride()) * 4))
        return arr
    return (ctypes.c_int64 * 16)(*qd.stride(), *kd.stride(), *vd.stride(), *o.stride())


def get_num_compute_cores():
    """SM count of the current CUDA device (the reference returns the AI-core count, :19-21)."""
    n = _lib.rsfa_sm_count(torch.cuda.current_device())
    if n <= 0:
        _capi.check(n, "rsfa_sm_count")
    return n


def _dense(t):
    """The C ABI wants a unit innermost stride, the other strides multiples of 8 elements and a
    16-byte aligned base; anything else is copied once."""
    if t.is_contiguous() and t.shape[-1] % 8 == 0 and t.data_ptr() % 16 == 0:
        return t                      # the usual case, decided without walking the strides
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0
    if ok:
        D = t.shape[-1]
        for dim in range(3):
            if t.shape[dim] > 1 and (t.stride(dim) % 8 != 0 or t.stride(dim) < D):
                ok = False
    return t if ok else t.contiguous()


def _forward(q, k, v, causal, sm_scale, BM, BN, want_lse):
    assert q.shape[-1] == k.shape[-1] and k.shape[-1] == v.shape[-1]
    assert q.shape[-1] in {16, 32, 64, 128, 256}
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k, v must share one [B, H, S, D] shape")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("attention() needs CUDA tensors: this build has no CPU path")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must all be float16 or all bfloat16")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must live on one device")
    Z, H, N_CTX, HEAD_DIM = q.shape
    if q.numel() == 0:
        # an empty batch, head count or sequence: nothing to launch (the C ABI itself wants B, H, S >= 1)
        return (torch.empty_like(q),
                torch.empty((Z, H, N_CTX), dtype=torch.float32, device=q.device) if want_lse else None)
    qd, kd, vd = _dense(q.detach()), _dense(k.detach()), _dense(v.detach())
    o = torch.empty_like(qd)
    if not (o.stride(-1) == 1 and all(o.shape[i] == 1 or o.stride(i) % 8 == 0 for i in range(3))):
        o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    M = torch.empty((Z, H, N_CTX), dtype=torch.float32, device=q.device) if want_lse else None
    strides = _strides_of(qd, kd, vd, o)
    args = (qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), M.data_ptr() if M is not None else None,
            Z, H, N_CTX, HEAD_DIM, strides, 1 if causal else 0, float(sm_scale), int(BM), int(BN),
            _DTYPES[q.dtype])
    # rsfa_fwd launches on the CURRENT device; switching costs microseconds, so only when needed
    if q.device.index == torch.cuda.current_device():
        rc = _lib.rsfa_fwd(*args, _current_stream(q.device.index))
    else:
        with torch.cuda.device(q.device):
            rc = _lib.rsfa_fwd(*args, _current_stream(q.device.index))
    if rc != 0:
        _capi.check(rc, "rsfa_fwd")
    return o, M


# ============================================================================
# The class name `_attention` is part of the reference's frozen surface (:545).
# ============================================================================
class _attention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, BM, BN):
        # The reference keeps the log-sum-exp for a backward pass it does not have (:400-404, :616);
        # with no backward here either it is not computed on this path: attention_with_lse() returns it.
        o, _ = _forward(q, k, v, causal, sm_scale, BM, BN, want_lse=False)
        ctx.save_for_backward(q, k, v, o)
        ctx.sm_scale = sm_scale
        ctx.HEAD_DIM = q.shape[-1]
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("the reference ships no backward pass; neither does this build")


# ============================================================================
# The name `attention` is part of the reference's frozen surface (:620).
# ============================================================================
attention = _attention.apply


def attention_with_lse(q, k, v, causal, sm_scale, BM=128, BN=128):
    """attention() that also returns the [B, H, S] fp32 log-sum-exp m + log(l) (:400-404)."""
    return _forward(q, k, v, causal, sm_scale, BM, BN, want_lse=True)


def get_tiling(Z, H, N_CTX, HEAD_DIM, causal):
    """Return (BLOCK_M, BLOCK_N) for the given problem shape from the per-(S, D, causal) tile
    table.  Any batch and head count is accepted; ValueError for an impossible shape."""
    bm, bn = ctypes.c_int(0), ctypes.c_int(0)
    rc = _lib.rsfa_get_tiling(int(Z), int(H), int(N_CTX), int(HEAD_DIM), 1 if causal else 0,
                              ctypes.byref(bm), ctypes.byref(bn))
    _capi.check(rc, "rsfa_get_tiling")
    return bm.value, bn.value


def select_path(N_CTX, HEAD_DIM, causal, sm_scale, BM=128, BN=128, dtype=torch.float16):
    """(path, tile_m, tile_n) the library would use: path 0 = short-sequence / generic mma.sync
    kernel, 1 = tcgen05 kernel."""
    path, tm, tn = ctypes.c_int(0), ctypes.c_int(0), ctypes.c_int(0)
    rc = _lib.rsfa_select_path(int(N_CTX), int(HEAD_DIM), 1 if causal else 0, float(sm_scale), int(BM),
                               int(BN), _DTYPES[dtype], ctypes.byref(path), ctypes.byref(tm),
                               ctypes.byref(tn))
    _capi.check(rc, "rsfa_select_path")
    return path.value, tm.value, tn.value


def attention_host(q, k, v, causal, sm_scale, BM=128, BN=128, device=0, out=None):
    """attention() for tensors that live in HOST memory (ideally pinned): the library streams
    slabs of heads through the device, overlapping the copies in both directions with the
    kernels, and returns a host tensor.  Blocks until the result is complete."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("attention_host() takes CPU tensors")
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k, v must share one [B, H, S, D] shape")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must all be float16 or all bfloat16")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    Z, H, N_CTX, HEAD_DIM = q.shape
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=q.is_pinned())
    if q.numel() == 0:
        return out
    rc = _lib.rsfa_fwd_host(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), None,
                            Z, H, N_CTX, HEAD_DIM, 1 if causal else 0, float(sm_scale), int(BM), int(BN),
                            _DTYPES[q.dtype], int(device))
    _capi.check(rc, "rsfa_fwd_host")
    return out


def device_status(device=None):
    """Synchronise and raise RuntimeError if a kernel left a non-zero status (a bounded wait ran
    out).  Returns None otherwise."""
    dev = torch.cuda.current_device() if device is None else int(device)
    raw = ctypes.c_int(0)
    rc = _lib.rsfa_device_status(dev, ctypes.byref(raw))
    if rc == _capi.RSFA_ERR_DEVICE_STATUS:
        raise RuntimeError("device status 0x%x: %s" % (raw.value & 0xffffffff, _capi.strerror(rc)))
    _capi.check(rc, "rsfa_device_status")


def work_items(Z, H, N_CTX, HEAD_DIM, causal, sm_scale):
    """Units of work a call is split into: (batch, head, block of query rows) items of the persistent
    tcgen05 kernels, or CTAs of the short-sequence kernel (the reference's NUM_BLOCKS, :289-294)."""
    n = ctypes.c_longlong(0)
    _capi.check(_lib.rsfa_work_items(int(Z), int(H), int(N_CTX), int(HEAD_DIM), 1 if causal else 0, float(sm_scale),
                                     ctypes.byref(n)), "rsfa_work_items")
    return n.value


def launch_count():
    """Kernels launched by the library in this process."""
    return int(_lib.rsfa_launch_count())


def set_option(name, value):
    _capi.check(_lib.rsfa_set_option(name.encode(), int(value)), "rsfa_set_option(%s)" % name)
