"""Three rates of the device that the kernels' rooflines rest on, measured by small programs of their own:

    mma_rate   cycles per `tcgen05.mma` of 128 x N x 16 issued back to back (N = 64, 128, 256)
    tma_rate   bytes per clock and SM that TMA tile loads bring from L2 into shared memory, against the bytes and
               the number of boxes per stage of the ring, on one SM and on all
    exp_rate   cycles per exponential and thread in the second pass of a softmax (fma, ex2, sum, pack, store) with 4, 8
               and 16 warps an SM, and with part of the exponentials computed by a cubic on the FMA pipe

    python baseline/device_rates.py [--out FOLDER]        (needs nvcc and a B200; `bench.py --rates` calls it)

The programs include the package's own tcgen05.cuh (mbarrier, TMA and MMA wrappers, bounded waits); nothing of the
product loads them.
"""
import argparse
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.normpath(os.path.join(HERE, "..", "llmgen_b200", "csrc"))
PROGRAMS = ("mma_rate", "tma_rate", "exp_rate")


def build(out: str, nvcc: str = "nvcc"):
    os.makedirs(out, exist_ok=True)
    paths = []
    for name in PROGRAMS:
        exe = os.path.join(out, name)
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-I", CSRC,
               "-o", exe, os.path.join(HERE, "device_rates", name + ".cu"), "-lcuda"]
        subprocess.run(cmd, check=True)
        paths.append(exe)
    return paths


def run(out: str = "") -> str:
    with tempfile.TemporaryDirectory() as tmp:
        text = []
        for exe in build(out or tmp):
            text.append(subprocess.run([exe], check=True, capture_output=True, text=True, timeout=300).stdout)
    return "".join(text)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="", help="keep the programs in this folder")
    args = ap.parse_args()
    sys.stdout.write(run(args.out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
