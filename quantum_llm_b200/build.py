"""Builds libqllm_b200.so (sm_100a) in-tree with nvcc.  No JIT cache is used, so
the library travels with the source tree."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libqllm_b200.so")
SOURCES = ["kernels_basic.cu", "kernels_attention.cu", "kernels_attention_q4h.cu", "kernels_attention_q4h_tc.cu", "kernels_attention_q8.cu", "kernels_attention_f16.cu", "kernels_sampler.cu", "kernels_sampler_full.cu", "kernels_presence.cu", "kernels_fused.cu", "kernels_moe.cu", "gemv_mma.cu",
           "provider.cu", "c_api_kernels.cu", "no_alloc.cu", "descriptor.cpp", "pack.cpp"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-fmad=false", "-ccbin", "/usr/bin/g++"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "qllm_b200.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objects, procs = [], []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(objdir, os.path.splitext(src)[0] + ".o")
        objects.append(obj)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc, *FLAGS, "-c", path, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objects):
        subprocess.run([nvcc, "-shared", "-o", LIB, *objects, "-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
