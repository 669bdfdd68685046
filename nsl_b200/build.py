"""Builds nsl_b200/libnslq_b200.so in-tree with nvcc for sm_100a only."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnslq_b200.so")

SOURCES = ["abi.cu", "act_quant.cu", "ternary_gemv.cu", "ternary_decode_sm100.cu", "ternary_gemm_sm100.cu", "w4a16_gemv.cu", "w4a16_gemm_sm100.cu", "w4a16_decode_sm100.cu", "noalloc.cu", "shard_comm.cu", "decode_attention.cu", "decode_glue.cu", "pack_at_load.cu", "bitnet_loader.cu", "nsl_shims.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--fmad=true", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
    "-Xptxas", "-v", "-Xptxas", "-warn-spills",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "nslq_b200.h"))
    deps.append(os.path.join(HERE, "..", "include", "nsl_shims.h"))
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source into one shared library.  Returns its path."""
    if not force and not needs_build():
        return LIB
    objs = []
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    log = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(HERE, "build", src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-ccbin", "/usr/bin/g++", "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env,
                                            text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        log.append("== %s ==\n%s" % (src, out))
        if p.returncode != 0:
            failed = True
    with open(os.path.join(HERE, "build", "ptxas.log"), "w") as f:
        f.write("\n".join(log))
    if failed or verbose:
        sys.stderr.write("\n".join(log))
    if failed:
        raise RuntimeError("nvcc failed; see nsl_b200/build/ptxas.log")
    cmd = [_nvcc(), "-shared", "-ccbin", "/usr/bin/g++", "-o", LIB, *objs, "-lcudart", "-ldl"]
    subprocess.check_call(cmd, env=env)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
