"""Generate golden vectors by running the REFERENCE's own kernels on the CPU.

Run in a container that has the reference checkout and upstream Triton:

    python tests/golden/make_golden.py <path to the reference checkout>

The reference's kernels are TritonAscend programs; upstream Triton's CPU
interpreter (TRITON_INTERPRET=1) executes them when three shims are in place:
an empty ``torch_npu`` module, a fixed core count instead of the NPU query, and
``tl.max`` without TritonAscend's ``propagate_nan`` keyword.  Nothing of the
reference is copied: its file is loaded from where it lies and only called.

Each case writes ``<name>.npz`` with fp16 q, k, v, the reference output o and
the call arguments.  The cases cover every dispatch branch of the reference
(flash_attention_forward.py:564-610): single-tile non-causal, single-tile
causal, tiled non-causal (with the D=64 inner loop and the general one), and
the prefix/diagonal causal split.
"""
import importlib.util
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch


def load_reference(root):
    sys.modules.setdefault("torch_npu", types.ModuleType("torch_npu"))
    import triton.language as tl

    if not getattr(tl.max, "_rsfa_shim", False):
        orig = tl.max

        def _max(*a, propagate_nan=None, **kw):
            return orig(*a, **kw)

        _max._rsfa_shim = True
        tl.max = _max
    path = os.path.join(root, "ascend_rsfa", "flash_attention_forward.py")
    spec = importlib.util.spec_from_file_location("reference_fa", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.get_num_compute_cores = lambda: 4
    return mod


# name, B, H, S, D, causal, sm_scale, BM, BN, seed, std
CASES = [
    ("cfg1_noncausal", 1, 2, 128, 64, False, 0.5, 64, 64, 42, 1.0),
    ("cfg1_causal", 1, 2, 128, 64, True, 0.5, 64, 64, 42, 1.0),
    ("small_causal_s64", 1, 2, 64, 64, True, 0.5, 64, 16, 20, 0.5),
    ("tiled_noncausal_d64", 1, 2, 256, 64, False, 0.5, 64, 32, 20, 0.5),
    ("tiled_noncausal_d128", 1, 1, 256, 128, False, 0.5, 64, 128, 42, 1.0),
    ("split_causal_d128", 1, 1, 256, 128, True, 0.5, 128, 64, 42, 1.0),
    ("split_causal_d32", 1, 2, 128, 32, True, 0.25, 32, 32, 7, 1.0),
]


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    root = sys.argv[1]
    mod = load_reference(root)
    here = os.path.dirname(os.path.abspath(__file__))
    for name, B, H, S, D, causal, scale, bm, bn, seed, std in CASES:
        g = torch.Generator().manual_seed(seed)
        q, k, v = [(torch.randn((B, H, S, D), generator=g) * std).half() for _ in range(3)]
        o = mod.attention(q, k, v, causal, scale, bm, bn)
        assert torch.isfinite(o.float()).all(), name
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            q=q.numpy(), k=k.numpy(), v=v.numpy(), o=o.numpy(),
            causal=np.array(causal), sm_scale=np.array(scale, dtype=np.float64),
            block_m=np.array(bm), block_n=np.array(bn),
        )
        print(name, tuple(o.shape), "ok")


if __name__ == "__main__":
    main()
