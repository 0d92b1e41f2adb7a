"""Builds the CUDA kernels for sm_100a into one shared library, in the source tree.

The kernels are plain CUDA with `extern "C"` entry points (no torch headers), so
nvcc compiles each file in seconds and Python calls them through ctypes.  The
library is built at first use: into `csrc/_build/` beside the sources, or, when
that folder cannot be written, into a per-user folder under the temporary
directory.  A stamp file holds a hash of the sources and flags; a matching stamp
means the library is current.  While nvcc runs, a progress line is printed every
few seconds.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libmachserve_b200_kernels.so"
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]
# No fast-math flag on purpose: expf, rsqrtf and division keep their accurate forms.


# Other builds of the same sources: a name, the flags it adds, and a build folder of its own beside the plain one.
# "timeline": the kernels of a decoding step stamp the device clock at their start, when their wait for the preceding
# kernel returns and at their end (launch.cuh); read by machserve_b200/timeline.py.
FLAVORS = {"timeline": ["-DMS_TIMELINE"]}


class BuildError(RuntimeError):
    pass


def sources():
    return sorted(CSRC.glob("*.cu"))


def _flags(flavor) -> list:
    if flavor is None:
        return list(NVCC_FLAGS)
    if flavor not in FLAVORS:
        raise BuildError(f"unknown build flavor '{flavor}' (known: {', '.join(sorted(FLAVORS))})")
    return NVCC_FLAGS + FLAVORS[flavor]


def _fingerprint(flavor=None) -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(_flags(flavor)).encode())
    return h.hexdigest()[:16]


def find_nvcc() -> str:
    for cand in (
        os.environ.get("NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH, $CUDA_HOME/bin and /usr/local/cuda/bin)")


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def _folder(flavor) -> str:
    return "_build" if flavor is None else f"_build_{flavor}"


def build_dir(flavor=None) -> Path:
    override = os.environ.get("MACHSERVE_B200_BUILD_DIR")
    if override:
        p = Path(override) if flavor is None else Path(override) / flavor
        if not _writable_dir(p):
            raise BuildError(f"MACHSERVE_B200_BUILD_DIR={override} cannot be written")
        return p
    in_tree = CSRC / _folder(flavor)
    if _writable_dir(in_tree):
        return in_tree
    p = Path(tempfile.gettempdir()) / f"machserve_b200{_folder(flavor)}_{os.getuid()}"
    if not _writable_dir(p):
        raise BuildError(f"neither {in_tree} nor {p} can be written; set MACHSERVE_B200_BUILD_DIR")
    return p


def _say(msg: str) -> None:
    print(f"[machserve_b200] {msg}", file=sys.stderr, flush=True)


def library_path(verbose: bool = True, flavor=None) -> Path:
    """The path of the current library (of the plain build, or of a flavor), building it first if it is missing or stale."""
    in_tree = CSRC / _folder(flavor)
    fp = _fingerprint(flavor)
    # a current library that came with the tree is used even when the tree is read-only
    if (in_tree / LIB_NAME).is_file() and (in_tree / "stamp").is_file() and (in_tree / "stamp").read_text() == fp:
        return in_tree / LIB_NAME
    out = build_dir(flavor)
    lib, stamp = out / LIB_NAME, out / "stamp"
    with open(out / "lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if lib.is_file() and stamp.is_file() and stamp.read_text() == fp:
                return lib
            _compile(out, lib, verbose, _flags(flavor))
            stamp.write_text(fp)
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _compile(out: Path, lib: Path, verbose: bool, flags) -> None:
    nvcc = find_nvcc()
    srcs = sources()
    if not srcs:
        raise BuildError(f"no .cu files under {CSRC}")
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out} (first use only)")
    procs = []
    for src in srcs:
        obj = out / (src.stem + ".o")
        log = open(out / (src.stem + ".log"), "w")
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        procs.append((src, obj, log, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT)))
    last = time.time()
    while True:
        running = [p for p in procs if p[3].poll() is None]
        if not running:
            break
        if verbose and time.time() - last >= 5.0:
            _say(f"  nvcc: {len(procs) - len(running)}/{len(procs)} files done after {time.time() - t0:.0f} s")
            last = time.time()
        time.sleep(0.1)
    failed = []
    for src, obj, log, proc in procs:
        log.close()
        if proc.returncode != 0:
            failed.append(f"{src.name}:\n{(out / (src.stem + '.log')).read_text()[-4000:]}")
    if failed:
        raise BuildError("nvcc failed:\n" + "\n".join(failed))
    tmp = out / (LIB_NAME + f".tmp{os.getpid()}")
    link = [nvcc, "-shared", "-o", str(tmp), *[str(p[1]) for p in procs]]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise BuildError("link failed:\n" + r.stdout[-4000:])
    os.replace(tmp, lib)
    if verbose:
        _say(f"kernels built in {time.time() - t0:.0f} s")


if __name__ == "__main__":
    print(library_path())
