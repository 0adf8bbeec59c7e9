"""Build librsfa_b200.so for sm_100a with nvcc, in-tree.

    python ascend-rsfa_b200/build.py [--force] [--verbose] [--trace]

The library lands beside the Python module that loads it
(ascend_rsfa/librsfa_b200.so) together with a stamp file holding a hash of the
sources, headers and compiler flags it was built from; a rebuild happens when
that hash no longer matches (file times are not consulted: the built library
travels with the source tree, and a checkout can carry any times), or with
--force.

--trace builds a separate debug library, ascend_rsfa/librsfa_b200_trace.so, with
-DRSFA_TRACE: the kernels of CTA 0 then log (clock, event code) pairs per role
into a buffer given through the "trace_ptr" option.  The per-role cycle tables
under profiles/ come from that build; the product library has no trace code.
"""
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "ascend_rsfa", "librsfa_b200.so")
OUT_TRACE = os.path.join(HERE, "ascend_rsfa", "librsfa_b200_trace.so")
SOURCES = ["rsfa_api.cu", "fwd_generic.cu", "fwd_tcgen05.cu", "fwd_tcgen05_db.cu", "fwd_tcgen05_sp.cu"]
HEADERS = ["common.cuh", "ptx_sm100.cuh", "tcgen05_common.cuh", "tile_table.inc", os.path.join("..", "..", "include", "rsfa.h")]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-cudart", "static",
]


def find_nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def source_hash(flags):
    """Hash of everything the library is made from: sources, headers, flags."""
    h = hashlib.sha256()
    for f in SOURCES + HEADERS:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read() + b"\0")
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def stale(out, flags):
    stamp = out + ".stamp"
    if not (os.path.exists(out) and os.path.exists(stamp)):
        return True
    with open(stamp) as fh:
        return fh.read().strip() != source_hash(flags)


def build(force=False, verbose=False, trace=False):
    out = OUT_TRACE if trace else OUT
    flags = FLAGS + (["-DRSFA_TRACE"] if trace else [])
    if not force and not stale(out, flags):
        return out
    nvcc = find_nvcc()
    objs = []
    build_dir = os.path.join(HERE, "build", "trace" if trace else "product")
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        cmd = [nvcc] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        log, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(log)
        if pr.returncode != 0:
            raise RuntimeError("nvcc failed on " + src)
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
            "-Xcompiler", "-fPIC", "-o", out] + objs
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link failed")
    with open(out + ".stamp", "w") as fh:
        fh.write(source_hash(flags) + "\n")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
