"""Builds the kernel library (every .cu of this folder) with nvcc for sm_100a.

The library is one shared object with a C ABI, loaded through ctypes: no Python headers and
no torch headers are compiled, so a first build takes well under a minute.  It is kept in
`_build/` beside the sources, stamped with a hash of the sources and flags; a stale or missing
library is rebuilt at the first call that needs it, with a progress line per file.  If the
source folder cannot be written, the build goes to a per-user temporary folder.
"""
import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libedgelm_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _say(msg):
    print(f"[edgelm_b200 build] {msg}", file=sys.stderr, flush=True)


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _stamp():
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def find_nvcc():
    for cand in (os.environ.get("EDGELM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("edgelm_b200: nvcc not found (looked at $EDGELM_NVCC, PATH and /usr/local/cuda/bin); "
                       "the CUDA kernels cannot be built and there is no other path")


def _build_dir():
    d = os.path.join(CSRC, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"edgelm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build_if_needed=True, verbose=False):
    """Path of an up-to-date kernel library, building it when needed."""
    stamp = _stamp()
    for d in (os.path.join(CSRC, "_build"), os.path.join(tempfile.gettempdir(), f"edgelm_b200_build_{os.getuid()}")):
        lib, st = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.txt")
        if os.path.exists(lib) and os.path.exists(st) and open(st).read().strip() == stamp:
            return lib
    if not build_if_needed:
        raise RuntimeError("edgelm_b200: the kernel library is not built")
    return build(verbose=verbose)


def _compile_one(nvcc, src, obj, extra):
    cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
    t0 = time.time()
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    return src, r.returncode, r.stdout, time.time() - t0


def build(verbose=False, ptxas_info=False):
    """Compile every source (in parallel) and link; returns the library's path."""
    nvcc = find_nvcc()
    d = _build_dir()
    srcs = sources()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {d} (first call only)")
    objs, failed = [], []
    t0 = time.time()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = []
        for s in srcs:
            obj = os.path.join(d, s[:-3] + ".o")
            objs.append(obj)
            futs.append(ex.submit(_compile_one, nvcc, s, obj, extra))
        for fu in concurrent.futures.as_completed(futs):
            src, rc, out, dt = fu.result()
            _say(f"  {src}: {'ok' if rc == 0 else 'FAILED'} in {dt:.1f} s ({time.time() - t0:.0f} s since start)")
            if rc != 0:
                failed.append((src, out))
            elif (verbose or ptxas_info) and out.strip():
                print(out, file=sys.stderr)
    if failed:
        raise RuntimeError("edgelm_b200: nvcc failed:\n" + "\n".join(f"--- {s}\n{o}" for s, o in failed))
    tmp_lib = os.path.join(d, f".{LIB_NAME}.{os.getpid()}")
    r = subprocess.run([nvcc, "-shared", "-o", tmp_lib] + objs + ["-lcudart_static", "-ldl", "-lrt", "-lpthread"],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("edgelm_b200: link failed:\n" + r.stdout)
    lib = os.path.join(d, LIB_NAME)
    os.replace(tmp_lib, lib)  # atomic: another process never sees half a library
    with open(os.path.join(d, "stamp.txt"), "w") as f:
        f.write(_stamp())
    _say(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


if __name__ == "__main__":
    build(verbose=True, ptxas_info="--ptxas" in sys.argv)
