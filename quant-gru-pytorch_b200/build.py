"""Build csrc/ into libqgru_b200.so with nvcc for sm_100a (cross-compiles without a GPU).

Every source is compiled to an object of its own (in parallel; only sources that changed, or
all of them when a header changed) and the objects are linked into the shared library."""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
_CSRC = os.path.join(_HERE, "csrc")
_OBJ = os.path.join(_HERE, "build")
SOURCES = ["qgru_api.cu", "qgru_gemm_tc.cu", "qgru_rec_mma.cu", "qgru_rec_cluster.cu", "qgru_rec_c64.cu", "qgru_float.cu",
           "qgru_hist.cu", "qgru_backward.cu", "qgru_probe.cu", "qgru_host.cc"]
OUT = os.path.join(_HERE, "libqgru_b200.so")


def _headers_mtime():
    deps = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC) if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(_ROOT, "include", "qgru.h"))
    deps.append(os.path.abspath(__file__))
    return max(os.path.getmtime(d) for d in deps)


def _obj(src):
    return os.path.join(_OBJ, src + ".o")


def _stale_sources(force):
    hdr = _headers_mtime()
    out = []
    for s in SOURCES:
        o = _obj(s)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(hdr, os.path.getmtime(os.path.join(_CSRC, s))):
            out.append(s)
    return out


def build(force=False, verbose=False):
    """Compile what is out of date and link.  Returns the .so path."""
    stale = _stale_sources(force)
    if not stale and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(_obj(s)) for s in SOURCES):
        return OUT
    os.makedirs(_OBJ, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    base = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
            "-Xcompiler", "-fPIC,-fvisibility=hidden,-ffp-contract=off",
            "-I" + os.path.join(_ROOT, "include"), "-I" + _CSRC]
    if verbose:
        base += ["-Xptxas", "-v"]

    def compile_one(s):
        return s, subprocess.run(base + ["-c", os.path.join(_CSRC, s), "-o", _obj(s)], capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(stale)))) as pool:
        results = list(pool.map(compile_one, stale))
    for s, res in results:
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n" + res.stdout + res.stderr)
        if verbose:
            print(res.stderr)
    res = subprocess.run([nvcc, "-shared", "-o", OUT + ".tmp"] + [_obj(s) for s in SOURCES] + ["-lcudart"],
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    os.replace(OUT + ".tmp", OUT)
    return OUT


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
