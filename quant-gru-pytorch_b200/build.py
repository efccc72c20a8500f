"""Build csrc/ into libqgru_b200.so with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
SOURCES = ["qgru_api.cu", "qgru_gemm_tc.cu", "qgru_rec_mma.cu", "qgru_rec_cluster.cu", "qgru_float.cu", "qgru_hist.cu", "qgru_backward.cu", "qgru_host.cc"]
OUT = os.path.join(_HERE, "libqgru_b200.so")


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(_HERE, "csrc", f) for f in os.listdir(os.path.join(_HERE, "csrc"))]
    deps.append(os.path.join(_ROOT, "include", "qgru.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile the library if any source is newer than it.  Returns the .so path."""
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-Xcompiler", "-fPIC,-fvisibility=hidden,-ffp-contract=off", "-shared",
           "-I" + os.path.join(_ROOT, "include"), "-I" + os.path.join(_HERE, "csrc")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(_HERE, "csrc", s) for s in SOURCES]
    cmd += ["-o", OUT + ".tmp", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    os.replace(OUT + ".tmp", OUT)
    if verbose:
        print(res.stderr)
    return OUT


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
