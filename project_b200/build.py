"""Builds libgatzk_b200.so in-tree with nvcc for sm_100a (no JIT cache, no cmake)."""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libgatzk_b200.so")
TUNING_LIB_PATH = os.path.join(HERE, "libgatzk_b200_tuning.so")
FLOW_LIB_PATH = os.path.join(HERE, "libgatzk_b200_flow.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "gatzk_b200.h"))
    headers.append(os.path.join(HERE, "host", "bounded_wait.hpp"))  # included by comm.cu
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(obj)
        path = os.path.join(CSRC, src)
        if force or _stale(obj, [path] + headers):
            jobs.append((path, obj))

    def compile_one(job):
        path, obj = job
        proc = subprocess.run([nvcc, *NVCC_FLAGS, "-c", path, "-o", obj], capture_output=True, text=True)
        return path, proc

    with ThreadPoolExecutor(max_workers=8) as pool:
        for path, proc in pool.map(compile_one, jobs):
            if verbose or proc.returncode != 0:
                sys.stderr.write(f"== {os.path.basename(path)}\n{proc.stderr}\n")
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on {path}")
    if jobs or not os.path.exists(LIB_PATH):
        subprocess.run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], check=True)
    # measurement aids (the integer-pipe ceiling) live in a library of their own
    tuning_src = os.path.join(CSRC, "tuning", "mac_peak.cu")
    if force or _stale(TUNING_LIB_PATH, [tuning_src] + headers):
        subprocess.run([nvcc, *NVCC_FLAGS[:-2], "-shared", tuning_src, "-o", TUNING_LIB_PATH], check=True)
    # the commit + prove flow: plain C++ host code over the C ABI of the library above
    host = os.path.join(HERE, "host")
    flow_deps = [os.path.join(host, f) for f in ("flow_gpu.cpp", "prover_flow.hpp", "prover_flow_tail.hpp", "prover_flow_quotients.hpp", "flow_c_impl.hpp", "proof_codec.hpp", "host_forward.hpp")]
    flow_deps += [os.path.join(os.path.dirname(HERE), "include", f) for f in ("gatzk_b200.h", "gatzk_b200_flow.h")]
    if force or _stale(FLOW_LIB_PATH, flow_deps + [LIB_PATH]):
        subprocess.run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wextra", flow_deps[0], "-o", FLOW_LIB_PATH,
                        f"-L{HERE}", "-lgatzk_b200", "-Wl,-rpath,$ORIGIN"], check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
