"""Build libpa_b200.so (hand-written CUDA for sm_100a) in-tree with nvcc.

    python build.py [--force] [--verbose] [--core]

The .so lands next to csrc/ (git-ignored).

--core builds libpa_b200_core.so from the CORE sources only: the page table, the small decoder ops with the fp32 linear
layer, sampling, and the ragged-batch sequence ops (norm / token shift / recurrence, differential and latent attention,
routed experts, masked softmax attention, matrix-state recurrences).  It is what the config-driven models need; a first run in a fresh checkout compiles this and no more.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libpa_b200.so")
OUT_CORE = os.path.join(HERE, "libpa_b200_core.so")
CORE = ("page_table.cu", "decoder_ops.cu", "linear_tf32x3.cu", "sampling.cu", "seq_ops.cu", "diff_attention.cu",
        "latent_attention.cu", "masked_attention.cu", "recurrence_ops.cu", "moe_ops.cu")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3",
    "--expt-relaxed-constexpr",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
    "-ccbin", "/usr/bin/g++",
]


def sources(core=False):
    if core:
        return [os.path.join(CSRC, f) for f in CORE]
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(out=OUT, core=False):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = sources(core) + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return any(os.path.getmtime(p) > t for p in deps)


def ensure_core(verbose=False):
    """The library a config-driven model needs: the full one when it is there and current, else the core one (built now
    if missing or older than its sources)."""
    if not _stale(OUT, False):
        return OUT
    return build(verbose=verbose, core=True)


def build(force=False, verbose=False, core=False):
    OUT = OUT_CORE if core else globals()["OUT"]
    if not force and not _stale(OUT, core):
        return OUT
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    objs, procs = [], []
    for src in sources(core):
        obj = os.path.join(HERE, "build", os.path.basename(src) + ".o")
        objs.append(obj)
        cmd = [NVCC, *FLAGS, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = f"{OUT}.{os.getpid()}.tmp"   # linked aside and renamed: a concurrent process never loads half a file
    subprocess.check_call([NVCC, "-shared", "-o", tmp, *objs, "-cudart", "static", "-ccbin", "/usr/bin/g++"])
    os.replace(tmp, OUT)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, core="--core" in sys.argv))
