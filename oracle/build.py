"""Build recipe for the CPU checker (test infrastructure, not product code).

`build_oracle()` compiles oracle/ldn_oracle.c into oracle/_build/libldn_oracle.so with gcc + OpenMP.
`build_ref()` (only where the upstream checkout is present) compiles the reference's own CUDA
sources, where they lie, together with oracle/ref_shim.cu into oracle/_ref/libldn_ref.so so that GPU
tests can compare against the reference's kernels themselves.  No reference source is copied.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libldn_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libldn_ref.so")
# the upstream checkout, if there is one: named by LDN_REFERENCE_ROOT, else a `reference` directory beside this repository
REF_ROOT = os.environ.get("LDN_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "ldn_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
    cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-fno-fast-math",
           "-ffp-contract=off", "-o", ORACLE_SO, src, "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def ref_available():
    return os.path.isdir(os.path.join(REF_ROOT, "core", "cuda"))


def build_ref(force=False):
    """Compile the reference's .cu files in place (read-only) plus our extern "C" shim."""
    if not ref_available():
        return REF_SO if os.path.exists(REF_SO) else None
    cu_dir = os.path.join(REF_ROOT, "core", "cuda")
    srcs = [os.path.join(cu_dir, f) for f in
            ("norm_dist_cuda.cu", "inf_dist_cuda.cu", "bound_inf_dist_cuda.cu")]
    shim = os.path.join(HERE, "ref_shim.cu")
    if not force and _newer(REF_SO, srcs + [shim]):
        return REF_SO
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    objs = []
    procs = []
    for s in srcs + [shim]:
        o = os.path.join(os.path.dirname(REF_SO), os.path.basename(s) + ".o")
        objs.append(o)
        cmd = ["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-I", cu_dir, "-c", s, "-o", o]
        procs.append(subprocess.Popen(cmd))
    for p in procs:
        if p.wait() != 0:
            raise RuntimeError("reference build failed")
    subprocess.run(["nvcc", "-shared", "-o", REF_SO] + objs + ["-lcudart"], check=True)
    for o in objs:
        os.remove(o)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_ref(force="--force" in sys.argv))
