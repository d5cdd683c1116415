"""In-tree build of the CUDA library and the host programs (sm_100a only).

    python -m lantern_b200.build            # build what is out of date
    python -m lantern_b200.build --force

nvcc cross-compiles without a GPU.  Outputs: lantern_b200/liblantern_b200.so (C ABI of include/lantern_b200.h) and
lantern_b200/liblantern_b200_hosts.so (the host programs of lantern_b200/hosts linked against it).
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "liblantern_b200.so")
HOSTS = os.path.join(HERE, "liblantern_b200_hosts.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, log=None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        sys.stderr.write(p.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return p.stdout


def build_all(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "lantern_b200.h"))
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))
    jobs = []
    for s in sources:
        stem = os.path.splitext(s)[0]
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ, stem + ".o")
        if force or _newer(obj, [src] + headers):
            jobs.append(([NVCC] + NVCC_FLAGS + ["-c", src, "-o", obj], os.path.join(OBJ, stem + ".ptxas.log")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        for out in ex.map(lambda j: _run(*j), jobs):
            if verbose:
                print(out)
    objs = [os.path.join(OBJ, os.path.splitext(s)[0] + ".o") for s in sources]
    if force or jobs or _newer(LIB, objs):
        _run([NVCC, "-shared", "-o", LIB] + objs + ["-ldl", "-lpthread"])
    hsrc = os.path.join(HERE, "hosts", "models.cpp")
    hdeps = [hsrc, os.path.join(HERE, "hosts", "tape.hpp"), os.path.join(HERE, "hosts", "loader.hpp"), LIB] + headers[-1:]
    if force or _newer(HOSTS, hdeps):
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-o", HOSTS, hsrc, "-L" + HERE, "-llantern_b200",
              "-Wl,-rpath,$ORIGIN"])
    return LIB, HOSTS


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB, HOSTS)
