"""Builds and loads the CUDA library (libpulpnn_b200.so and the two drop-in shims).

The library is compiled in-tree with nvcc for sm_100a only. Loading never falls back to
anything: if the shared object is missing, or there is no GPU when a kernel is called, the
caller gets an error.
"""
import ctypes as C
import hashlib
import os
import re
import shlex
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
INCLUDE = os.path.join(ROOT, "include")
MAIN_SO = os.path.join(LIBDIR, "libpulpnn_b200.so")
DROPIN_SO = {32: os.path.join(LIBDIR, "libpulpnn_b200_32.so"),
             64: os.path.join(LIBDIR, "libpulpnn_b200_64.so")}

CU_SOURCES = ["context.cu", "conv_generic.cu", "depthwise.cu", "pool_add.cu", "entry_points.cu",
              "igemm_tc.cu", "net.cu", "depthwise_hwc3x3.cu",
              "conv_smallcin.cu", "depthwise_chw3x3.cu", "depthwise_hwc3x3_tma.cu",
              "conv_smallcin_tc.cu", "layout.cu", "subbyte.cu", "diagnostics.cu", "dwpw_fused.cu", "igemm_tc2.cu", "gemm_fewrows.cu", "dwpw_tcdw.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build_library(verbose=False, force=False):
    """Compile every .cu for sm_100a and link the three shared objects (in-tree).

    PULPNN_NVCC_FLAGS in the environment adds compiler flags (e.g. -DPULPNN_TRACE, the timing trace of
    igemm_tc.cu); such objects are kept apart from the ordinary ones, and the library is relinked
    whenever the flags differ from those of the library on disk."""
    os.makedirs(LIBDIR, exist_ok=True)
    extra = shlex.split(os.environ.get("PULPNN_NVCC_FLAGS", ""))
    objdir = OBJDIR + ("_" + hashlib.sha1(" ".join(extra).encode()).hexdigest()[:8] if extra else "")
    os.makedirs(objdir, exist_ok=True)
    stamp = os.path.join(LIBDIR, "nvcc_flags.txt")
    previous = open(stamp).read() if os.path.exists(stamp) else ""
    if previous != " ".join(extra):
        force_link = True
    else:
        force_link = False
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    sources = [s for s in CU_SOURCES if os.path.exists(os.path.join(CSRC, s))]

    def compile_one(src):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        path = os.path.join(CSRC, src)
        if not force and _newer(obj, [path] + headers):
            return obj
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=4) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or force_link or not _newer(MAIN_SO, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", MAIN_SO] + objs
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        with open(stamp, "w") as f:
            f.write(" ".join(extra))
    dropin_src = os.path.join(CSRC, "dropin.c")
    for bits, so in DROPIN_SO.items():
        if force or not _newer(so, [dropin_src, MAIN_SO] + headers):
            cmd = ["gcc", "-std=gnu11", "-O2", "-fPIC", "-shared", "-DPULPNN_BN_BITS=%d" % bits,
                   dropin_src, "-o", so, "-L" + LIBDIR, "-lpulpnn_b200", "-Wl,-rpath,$ORIGIN"]
            if verbose:
                print(" ".join(cmd), flush=True)
            subprocess.run(cmd, check=True)
    return MAIN_SO


def declared_symbols():
    """Every function name that include/*.h declares (after preprocessing)."""
    names = set()
    for hdr, defs in (("pulpnn_b200.h", []), ("pulpnn_b200_dropin.h", ["-DPULPNN_BN_BITS=32"])):
        out = subprocess.run(["gcc", "-E", "-P"] + defs + [os.path.join(INCLUDE, hdr)], check=True,
                             capture_output=True, text=True).stdout
        for m in re.finditer(r"\b(pulp_nn_\w+|pulpnn_\w+)\s*\(", out):
            names.add(m.group(1))
    return sorted(names)


_lib = None


def load_library():
    """dlopen libpulpnn_b200.so. Raises if it has not been built: there is no other path."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(MAIN_SO):
        raise RuntimeError(
            "%s is missing: build it with `python __graft_entry__.py` (needs nvcc). "
            "This package has no CPU or PyTorch fallback." % MAIN_SO)
    _lib = C.CDLL(MAIN_SO, mode=C.RTLD_GLOBAL)
    _lib.pulpnn_last_error_message.restype = C.c_char_p
    _lib.pulpnn_launch_count.restype = C.c_ulonglong
    _lib.pulpnn_net_create.restype = C.c_void_p
    _lib.pulpnn_net_layer_output_bytes.restype = C.c_size_t
    _lib.pulpnn_net_launches_per_run.restype = C.c_ulonglong
    _lib.pulpnn_net_layer_kernel.restype = C.c_char_p
    return _lib


def load_dropin(bits):
    load_library()
    return C.CDLL(DROPIN_SO[bits])
