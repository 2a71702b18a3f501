"""Builds libcatena_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch extension).

    python catena-lang_b200/build.py [--force] [--verbose]

Host code is compiled with -ffp-contract=off and device code with --fmad=false: the determinism
contract of the reference's own build (catena-lang/src/runtime/artifact.rs:59-80).  The device
arithmetic additionally uses explicitly rounded intrinsics, so the flags are a second line of
defence rather than the only one.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libcatena_b200.so")
SOURCES = ["core.cu", "map_reduce.cu", "map_program.cu", "map_jit.cu", "int_programs.cu", "gemm_f32.cu", "gemm_tc.cu", "gemm_tc2.cu", "attn_decode.cu", "attn_decode_tc.cu", "llama.cu", "llama_decode_fused.cu", "attn_prefill_tc.cu", "programs.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--std=c++17", "--fmad=false",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-fno-fast-math,-Wall,-Wno-unused-function",
    "-Xptxas", "-v",
]


def _newest_source_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(HERE, "..", "include", "catena_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force=False, verbose=False):
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= _newest_source_mtime():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        elif verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [nvcc, "-shared", "-o", OUT, *objs, "-lcudart"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
