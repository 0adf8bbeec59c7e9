"""CPU oracle for the FlashAttention-2 forward path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 PyTorch on the CPU, the arithmetic of the
reference operator ``ascend_rsfa.flash_attention_forward.attention``.  Only the
test-suite, the smoke check and the ``cpu_baseline`` / ``--impl reference`` legs
of the benchmark may import it; the product path never does.

Parity status: pinned by tolerance.  The reference stores no golden tensors; its
own tests compare against a closed vendor operator at atol = rtol = 1e-2
(ascend_rsfa/flash_attention_forward.py:736-738,
benchmarks/run_correctness_test.py:142-148).  The fixtures under
``tests/golden`` were produced by running the reference's own kernels on the CPU
through the Triton interpreter (see ``tests/golden/make_golden.py``) and this
oracle is checked against them.

What is restated, with the reference lines it follows:

* ``attention_fp32``      softmax(q k^T * sm_scale [+ causal mask]) v — the
  single-tile kernels are this formula verbatim
  (flash_attention_forward.py:84-88 non-causal, :150-158 causal); the mask keeps
  ``row >= col`` (:153, :194, :439), square and aligned top-left.
* ``attention_online``    the tiled online-softmax recurrence
  (:184-224: scale, running max, ``p = exp(qk - m)``, ``p`` rounded to the input
  dtype before the second product (:211), ``l = l*alpha + sum p`` (:217-219),
  ``acc = acc*alpha + p v`` (:221-223)) and the epilogue ``acc / l`` with
  ``lse = m + log l`` (:400-404).  It exists to show the recurrence and the
  plain formula agree, and that results do not depend on (BLOCK_M, BLOCK_N).
"""
from __future__ import annotations

import math
import torch


def _check(q, k, v):
    if q.dim() != 4 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k, v must share one [B, H, S, D] shape")


def attention_fp32(q, k, v, causal, sm_scale, return_lse=False, heads_per_chunk=None):
    """softmax(q k^T * sm_scale [+ mask]) v in fp32, one (b, h) chunk at a time.

    Inputs of any float dtype on the CPU; returns fp32 ``[B, H, S, D]`` (and the
    natural-log row normaliser ``[B, H, S]`` when ``return_lse``).  The S x S
    score matrix is materialised per chunk of heads so memory stays bounded
    (S = 8192 -> 256 MiB per head).
    """
    _check(q, k, v)
    B, H, S, D = q.shape
    qf = q.reshape(B * H, S, D)
    kf = k.reshape(B * H, S, D)
    vf = v.reshape(B * H, S, D)
    out = torch.empty((B * H, S, D), dtype=torch.float32)
    lse = torch.empty((B * H, S), dtype=torch.float32) if return_lse else None
    if heads_per_chunk is None:
        heads_per_chunk = max(1, (1 << 26) // max(1, S * S))
    mask = None
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool).tril_().logical_not_()
    for lo in range(0, B * H, heads_per_chunk):
        hi = min(B * H, lo + heads_per_chunk)
        s = torch.matmul(qf[lo:hi].float(), kf[lo:hi].float().transpose(-1, -2))
        s.mul_(float(sm_scale))
        if mask is not None:
            s.masked_fill_(mask, float("-inf"))
        m = s.amax(dim=-1, keepdim=True)
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        out[lo:hi] = torch.matmul(p / l, vf[lo:hi].float())
        if return_lse:
            lse[lo:hi] = (m + torch.log(l)).squeeze(-1)
    out = out.reshape(B, H, S, D)
    if return_lse:
        return out, lse.reshape(B, H, S)
    return out


def attention_online(q, k, v, causal, sm_scale, block_m, block_n, return_lse=False):
    """The tiled recurrence, block by block, with P rounded to the input dtype.

    Pure-Python loops over tiles: meant for small shapes only.  Ragged edges
    (S not a multiple of the tile) are handled by clipping the tile, which the
    reference does not do (it assumes divisibility).
    """
    _check(q, k, v)
    B, H, S, D = q.shape
    dt = q.dtype
    out = torch.empty((B, H, S, D), dtype=torch.float32)
    lse = torch.empty((B, H, S), dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            qf, kf, vf = q[b, h].float(), k[b, h].float(), v[b, h].float()
            for m0 in range(0, S, block_m):
                m1 = min(S, m0 + block_m)
                rows = torch.arange(m0, m1)
                m_i = torch.full((m1 - m0,), float("-inf"))
                l_i = torch.zeros(m1 - m0)
                acc = torch.zeros(m1 - m0, D)
                hi = min(S, m1) if causal else S
                for n0 in range(0, hi, block_n):
                    n1 = min(hi, n0 + block_n)
                    s = qf[m0:m1] @ kf[n0:n1].T * float(sm_scale)
                    if causal:
                        cols = torch.arange(n0, n1)
                        s = s.masked_fill(rows[:, None] < cols[None, :], float("-inf"))
                    m_new = torch.maximum(m_i, s.amax(dim=-1))
                    p = torch.exp(s - m_new[:, None])
                    alpha = torch.exp(m_i - m_new)
                    l_i = l_i * alpha + p.sum(dim=-1)
                    acc = acc * alpha[:, None] + p.to(dt).float() @ vf[n0:n1]
                    m_i = m_new
                out[b, h, m0:m1] = acc / l_i[:, None]
                lse[b, h, m0:m1] = m_i + torch.log(l_i)
    if return_lse:
        return out, lse
    return out


def error_metrics(out, ref, atol=1e-2, rtol=1e-2):
    """max / mean absolute error, allclose at the reference's tolerance, and a
    separate finiteness flag (the reference's ``equal_nan=True`` would let
    NaN == NaN pass, run_correctness_test.py:148)."""
    o = out.detach().float().cpu()
    r = ref.detach().float().cpu()
    diff = (o - r).abs()
    return {
        "max_abs": float(diff.max()) if diff.numel() else 0.0,
        "mean_abs": float(diff.mean()) if diff.numel() else 0.0,
        "finite": bool(torch.isfinite(o).all()),
        "allclose": bool(torch.allclose(o, r, atol=atol, rtol=rtol)),
    }


# Benchmark configurations: (B, H, S, D, sm_scale, input multiplier).
CONFIGS = {
    "cfg1": (1, 2, 128, 64, 0.5, 1.0),
    "cfg2": (128, 8, 2048, 128, 0.5, 1.0),
    "cfg3": (64, 8, 1024, 256, 1.0 / 16.0, 1.0),
    "cfg4": (16, 16, 4096, 128, 1.0 / math.sqrt(128.0), 1.0),
    "cfg5": (4, 32, 8192, 64, 0.125, 2.0),
}


def make_inputs(B, H, S, D, seed=42, std=1.0, dtype=torch.float16, device="cpu"):
    """Seeded i.i.d. N(0, std) q, k, v, generated in fp32 on the CPU and cast."""
    g = torch.Generator().manual_seed(int(seed))
    ts = []
    for _ in range(3):
        t = torch.randn((B, H, S, D), generator=g, dtype=torch.float32)
        if std != 1.0:
            t.mul_(std)
        ts.append(t.to(dtype).to(device))
    return tuple(ts)


def attention_flops(B, H, S, D, causal):
    """4 B H S^2 D, halved for causal (the figure the roofline uses)."""
    f = 4.0 * B * H * S * S * D
    return f / 2.0 if causal else f
