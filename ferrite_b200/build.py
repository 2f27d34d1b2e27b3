"""In-tree build of the native libraries.

``libferrite_b200_kernels.so``  - every sm_100a CUDA kernel behind a C ABI (nvcc)
``_runtime*.so``                - the C++ host runtime: planner, radix cache, page/state pools,
                                  CPU golden ops (pybind11, g++)

Both land inside the package directory so they travel with a source snapshot.  A build id
(hash of the sources) is compiled into each library and checked at load time, the same
defence against stale binaries the reference keeps with its same-source gate
(``crates/ferrite-kernel/build.rs:133-215``).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "ferrite_b200"
KDIR = ROOT / "csrc" / "kernels"
RDIR = ROOT / "csrc" / "runtime"
BUILD = ROOT / "build"
KLIB = PKG / "libferrite_b200_kernels.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _hash(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def kernel_sources():
    return sorted(KDIR.glob("*.cu"))


def kernel_build_id() -> str:
    return _hash(list(KDIR.glob("*.cu")) + list(KDIR.glob("*.cuh")))


def _run(cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, **kw)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def build_kernels(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    bid = kernel_build_id()
    stamp = BUILD / "kernels.id"
    if not force and KLIB.exists() and stamp.exists() and stamp.read_text() == bid:
        return KLIB
    BUILD.mkdir(exist_ok=True)
    idsrc = BUILD / "build_id.cu"
    idsrc.write_text('extern "C" __attribute__((visibility("default"))) const char* fb_build_id() '
                     '{ return "%s"; }\n' % bid)
    srcs = kernel_sources() + [idsrc]
    flags = list(NVCC_FLAGS) + ["-I", str(KDIR)]
    if ptxas_v:
        flags += ["-Xptxas", "-v"]

    def one(src: Path):
        obj = BUILD / (src.stem + ".o")
        hfile = BUILD / (src.stem + ".hash")
        dep = _hash([src] + list(KDIR.glob("*.cuh")))
        if not force and obj.exists() and hfile.exists() and hfile.read_text() == dep:
            return obj, ""
        log = _run(["nvcc", *flags, "-c", str(src), "-o", str(obj)])
        hfile.write_text(dep)
        return obj, log

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        res = list(ex.map(one, srcs))
    if verbose or ptxas_v:
        for _, log in res:
            if log.strip():
                print(log)
    _run(["nvcc", "-shared", "-o", str(KLIB), *[str(o) for o, _ in res], "-lcudart", "-lcuda"])
    stamp.write_text(bid)
    return KLIB


def runtime_sources():
    return sorted(RDIR.glob("*.cpp")) + sorted((ROOT / "csrc" / "golden").glob("*.cpp"))


def runtime_path() -> Path:
    return PKG / ("_runtime" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_runtime(force: bool = False) -> Path:
    import pybind11
    srcs = runtime_sources()
    out = runtime_path()
    if not srcs:
        return out
    hdrs = list(RDIR.glob("*.h")) + list((ROOT / "csrc" / "golden").glob("*.h"))
    bid = _hash(srcs + hdrs)
    stamp = BUILD / "runtime.id"
    if not force and out.exists() and stamp.exists() and stamp.read_text() == bid:
        return out
    BUILD.mkdir(exist_ok=True)
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(RDIR),
           "-I", str(ROOT / "csrc" / "golden")]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", '-DFB_RUNTIME_BUILD_ID="%s"' % bid]

    def one(src: Path):
        obj = BUILD / ("rt_" + src.stem + ".o")
        hfile = BUILD / ("rt_" + src.stem + ".hash")
        dep = _hash([src] + hdrs)
        if not force and obj.exists() and hfile.exists() and hfile.read_text() == dep:
            return obj
        _run(["g++", *flags, *inc, "-c", str(src), "-o", str(obj)])
        hfile.write_text(dep)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(one, srcs))
    _run(["g++", "-shared", "-pthread", "-o", str(out), *[str(o) for o in objs]])
    stamp.write_text(bid)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_runtime(force)


if __name__ == "__main__":
    f = "--force" in sys.argv
    v = "-v" in sys.argv
    k = build_kernels(force=f, verbose=v, ptxas_v="--ptxas" in sys.argv)
    r = build_runtime(force=f)
    print("built", k, r)
