"""Builds libstrictb200.so in-tree with nvcc for sm_100a (no other architecture, no JIT).

    python -m strict_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libstrictb200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
HOST_CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-ccbin", HOST_CXX,
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def source_id():
    """sha256 over the library's sources and its header (file names and contents, sorted): the build
    stamps it into the library (strictb200_build_id) so that a run can say which sources its binary
    was made from."""
    import hashlib
    h = hashlib.sha256()
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cpp", ".cuh", ".h"))]
    files.append(os.path.join(HERE, "..", "include", "strictb200.h"))
    for path in files:
        h.update(os.path.basename(path).encode() + b"\0")
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "strictb200.h"))
    jobs = []
    objs = []
    sid = source_id()
    stamp = os.path.join(OBJ, "build_id.txt")
    stamped = open(stamp).read().strip() if os.path.exists(stamp) else ""
    for src in sources():
        obj = os.path.join(OBJ, src.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        is_id = src == "build_id.cpp"  # the one file that carries the stamp: rebuilt whenever any source changed
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers) or (is_id and stamped != sid):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + (['-DSB_BUILD_ID="%s"' % sid] if is_id else []) + \
                  ["-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode:
                sys.stderr.write(" ".join(cmd[-4:]) + "\n" + r.stdout + r.stderr)
            if r.returncode:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    with open(stamp, "w") as f:
        f.write(sid + "\n")
    if force or jobs or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-ccbin", HOST_CXX, "-o", LIB] + objs + ["-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
