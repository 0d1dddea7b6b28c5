"""Compiles the CUDA and host libraries in-tree with nvcc / g++ (sm_100a only)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))


def build(verbose=False, jobs=None):
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", os.path.join(HERE, "csrc"), f"-j{jobs}", "all"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("building the CUDA extension failed (see the compiler output above)")
    for name in ("libgreta_cuda.so",):
        if not os.path.exists(os.path.join(HERE, name)):
            raise RuntimeError(f"{name} was not produced")


if __name__ == "__main__":
    build(verbose=True)
