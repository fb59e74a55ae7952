"""Build libfa_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: python flash-attention-rdna3_b200/build.py [--force] [--verbose] [--prof] [--debug-bounds]

Each .cu file is compiled to an object only when it or a header is newer than the object, then all
objects are linked into fa_b200/libfa_b200.so next to the Python package that loads it.

--prof builds a second library, fa_b200/libfa_b200_prof.so, with -DFA_PROF: the tensor-core forward, backward and decode
kernels then count, per CTA and role, the cycles spent in each phase of their loops (csrc/fa_prof.cuh) and the library
exports fa_debug_read_prof / fa_debug_read_prof_bwd / fa_debug_read_prof_decode, which copy the counters to the host. It is a tuning aid: the
product library carries none of it, and nothing loads the profiling library unless a script points
fa_b200._lib.LIB_PATH at it.

--debug-bounds builds fa_b200/libfa_b200_debug.so with -DFA_DEBUG_BOUNDS: every tiled TMA load checks its coordinates
and destination (alignment of the innermost coordinate, no negative head / batch coordinate) before it is issued,
prints a violation and skips the copy (csrc/fa_sm100.cuh). compute-sanitizer is not available everywhere these kernels
are developed; this is the substitute for the one class of mistake that faults the GPU instead of giving wrong numbers.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
OUT = os.path.join(HERE, "fa_b200", "libfa_b200.so")
SOURCES = ["fa_api.cu", "fa_simt.cu", "fa_tiled_fwd.cu", "fa_tiled_dq.cu", "fa_tiled_dkdv.cu", "fa_decode.cu", "fa_tiny.cu", "fa_fwd_sm100.cu", "fa_bwd_sm100.cu", "fa_wide_sm100.cu", "fa_decode_sm100.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc():
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _newest_header():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(HERE, "..", "include", "fa_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False, prof=False, debug_bounds=False):
    global OBJ, OUT
    if prof:
        OBJ = os.path.join(HERE, "build", "prof")
        OUT = os.path.join(HERE, "fa_b200", "libfa_b200_prof.so")
    if debug_bounds:
        OBJ = os.path.join(HERE, "build", "debug")
        OUT = os.path.join(HERE, "fa_b200", "libfa_b200_debug.so")
    os.makedirs(OBJ, exist_ok=True)
    header_time = _newest_header()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), header_time)
        if stale:
            cmd = [_nvcc(), *NVCC_FLAGS, *(["-DFA_PROF"] if prof else []),
                   *(["-DFA_DEBUG_BOUNDS"] if debug_bounds else []), "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append((src, cmd))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"--- {name}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}")
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in SOURCES]
    if jobs or not os.path.exists(OUT):
        cmd = [_nvcc(), "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, prof="--prof" in sys.argv,
                debug_bounds="--debug-bounds" in sys.argv))
