"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

The library is built with nvcc the first time it is needed and kept beside the
sources (``_build/``), or in a per-user temporary folder when the checkout
cannot be written.  Its file name carries a hash of the sources and flags, so a
changed source never runs stale code.  There is no fallback: without nvcc or
with a failing compile the error is raised.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xcompiler", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def sources() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _nvcc() -> str:
    for candidate in (os.environ.get("FIELDRUN_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise BuildError("nvcc was not found (looked at $FIELDRUN_B200_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of fieldrun_b200 cannot be built and there is no other path")


def source_hash() -> str:
    h = hashlib.sha256()
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(HERE, name), "rb") as handle:
            h.update(handle.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    override = os.environ.get("FIELDRUN_B200_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(HERE, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"fieldrun_b200_build_{os.getuid()}"))
    for path in candidates:
        try:
            os.makedirs(path, exist_ok=True)
            probe = os.path.join(path, f".write_probe_{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return path
        except OSError:
            continue
    raise BuildError(f"no writable folder for the compiled kernels among {candidates}")


def library_path(create_dir: bool = True) -> str:
    tag = source_hash()
    in_tree = os.path.join(HERE, "_build", f"libfieldrun_b200_{tag}.so")
    if os.path.isfile(in_tree) or not create_dir:
        return in_tree
    return os.path.join(_build_dir(), f"libfieldrun_b200_{tag}.so")


def _say(message: str) -> None:
    print(f"[fieldrun_b200] {message}", file=sys.stderr, flush=True)


def build(verbose: bool = True, ptxas_info: bool = False) -> str:
    """Compile if needed and return the path of the shared library."""
    target = library_path()
    if os.path.isfile(target):
        return target
    nvcc = _nvcc()
    out_dir = os.path.dirname(target)
    tag = source_hash()
    files = sources()
    started = time.time()
    if verbose:
        _say(f"compiling {len(files)} CUDA sources for sm_100a into {out_dir} (first use; takes a minute or two)")

    def compile_one(name: str) -> tuple[str, str]:
        obj = os.path.join(out_dir, f"{name[:-3]}_{tag}.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", HERE, "-c", os.path.join(HERE, name), "-o", obj]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
        return obj, proc.stderr

    objects: list[str] = []
    logs: list[str] = []
    workers = max(1, min(len(files), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
        futures = {pool.submit(compile_one, name): name for name in files}
        done = 0
        for future in concurrent.futures.as_completed(futures):
            obj, log = future.result()
            objects.append(obj)
            logs.append(log)
            done += 1
            if verbose:
                _say(f"  compiled {futures[future]} ({done}/{len(files)}, {time.time() - started:.0f} s)")
    partial = target + f".tmp{os.getpid()}"
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", partial, *sorted(objects), "-lcudart"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking the kernels failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(partial, target)
    for name in os.listdir(out_dir):                       # libraries of older sources
        if name.startswith("libfieldrun_b200_") and name.endswith(".so") and name != os.path.basename(target):
            try:
                os.remove(os.path.join(out_dir, name))
            except OSError:
                pass
    for obj in objects:
        try:
            os.remove(obj)
        except OSError:
            pass
    if verbose:
        _say(f"built {os.path.basename(target)} in {time.time() - started:.0f} s")
    if ptxas_info:
        sys.stderr.write("\n".join(logs))
    return target


if __name__ == "__main__":
    print(build(ptxas_info="--ptxas" in sys.argv))
