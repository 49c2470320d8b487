"""Builds the CUDA library in-tree: jatai_b200/libjatai_b200.so (sm_100a only)."""
import os
import subprocess
import sys

AQUI = os.path.dirname(os.path.abspath(__file__))
FONTE = os.path.join(AQUI, "csrc", "jatai_b200.cu")
SAIDA = os.path.join(AQUI, "libjatai_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-shared", "-Xcompiler", "-fPIC"]


def fontes():
    d = os.path.join(AQUI, "csrc")
    return [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith((".cu", ".cuh"))]


def desatualizada():
    if not os.path.exists(SAIDA):
        return True
    t = os.path.getmtime(SAIDA)
    return any(os.path.getmtime(f) > t for f in fontes())


def build(force=False, verbose=False):
    """Compile if a source is newer than the library.  Raises if nvcc fails."""
    if not force and not desatualizada():
        return SAIDA
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + [FONTE, "-o", SAIDA]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return SAIDA


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
