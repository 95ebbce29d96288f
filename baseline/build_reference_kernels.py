"""Compile the reference's own CUDA kernels, unmodified, for sm_100a into one shared library.

    python baseline/build_reference_kernels.py --src <checkout of AIxSpace/llmgen> [--out baseline/_ref]

The files are the list of the reference's build script (build.zig: CUDA_SRC), compiled with its flags
(-O3 -std=c++17) except for the architecture, which is sm_100a here and sm_86 there.  Their entry points are
plain `extern "C"` functions with no Zig in them, so the library can be loaded with ctypes.  It is a
comparator for `bench.py --kernels` (same B200, same inputs, same timing loop) and for the fixtures under
tests/golden/; nothing of the product loads it.  The output folder is not tracked.
"""
import argparse
import os
import subprocess
import sys

CUDA_SRC = ["cuda_context.cu", "embedding/embedding.cu", "memory/memcpy.cu", "memory/memory.cu", "linear/linear.cu",
            "norm/norm_final.cu", "arithmetic/add_v1.cu", "arithmetic/mul_v1.cu", "activation/silu_v1.cu",
            "softmax/softmax.cu", "shape/shape.cu", "rope/rope_v1.cu", "attention/attention.cu", "sample/sample.cu"]
LIB_NAME = "libllmgen_ref_kernels.so"


def build(src: str, out: str, nvcc: str = "nvcc") -> str:
    root = os.path.join(src, "src", "backend", "cuda")
    missing = [f for f in CUDA_SRC if not os.path.isfile(os.path.join(root, f))]
    if missing:
        raise SystemExit(f"{root}: not the reference's CUDA backend (missing {', '.join(missing)})")
    os.makedirs(out, exist_ok=True)
    objects = []
    for f in CUDA_SRC:
        obj = os.path.join(out, f.replace("/", "_") + ".o")
        cmd = [nvcc, "-c", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               os.path.join(root, f), "-o", obj]
        print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objects.append(obj)
    lib = os.path.join(out, LIB_NAME)
    cmd = [nvcc, "-shared", "-o", lib] + objects + ["-lcublas"]
    print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    for obj in objects:
        os.remove(obj)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", default=os.environ.get("LLMGEN_REFERENCE", ""), help="checkout of the reference")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref"))
    args = ap.parse_args()
    if not args.src:
        sys.exit("give --src (or LLMGEN_REFERENCE): the folder of the reference's checkout")
    print("built", build(args.src, args.out))
