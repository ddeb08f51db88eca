"""In-tree native build: CUDA kernels (sm_100a only) and host C++ into two shared objects.

  recml_b200/lib/librecml_cuda.so   every file under csrc/cuda/*.cu
  recml_b200/lib/librecml_host.so   every file under csrc/host, csrc/data, csrc/ckpt (*.cpp)

Objects are rebuilt only when a source (or a header next to it) changed, judged by a
content hash stored beside the library, so a tree whose libraries were built elsewhere
loads them without invoking a compiler.  Kernels export plain `extern "C"` launchers that
take raw pointers and a stream; Python binds them with ctypes (`recml_b200.ops._lib`).
"""
from __future__ import annotations

import concurrent.futures
import glob
import hashlib
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
LIB_DIR = os.path.join(ROOT, "recml_b200", "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-Wall"]

# Checked builds (separate object and library names, so they never mix with the optimised ones):
#   RECML_DEBUG=1                       kernels and host code compiled with -DRECML_DEBUG: buffers handed to
#                                       kernels carry canary words that are verified after the launch, and
#                                       device-side index checks that the optimised build leaves out are on
#   RECML_SANITIZE=address,undefined    host library built with the named compiler sanitizers (run Python with
#                                       LD_PRELOAD=$(gcc -print-file-name=libasan.so))
DEBUG = os.environ.get("RECML_DEBUG", "0") not in ("", "0")
SANITIZE = os.environ.get("RECML_SANITIZE", "")
_SUFFIX = ("_dbg" if DEBUG else "") + ("_san" if SANITIZE else "")
if DEBUG:
  NVCC_FLAGS = NVCC_FLAGS + ["-DRECML_DEBUG=1"]
  CXX_FLAGS = CXX_FLAGS + ["-DRECML_DEBUG=1"]
if SANITIZE:
  CXX_FLAGS = [f for f in CXX_FLAGS if f != "-O3"] + ["-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={SANITIZE}"]


def _nvcc() -> str:
  return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _digest(paths: list[str], extra: str = "") -> str:
  h = hashlib.sha256(extra.encode())
  for p in sorted(paths):
    h.update(os.path.relpath(p, ROOT).encode())
    with open(p, "rb") as f:
      h.update(f.read())
  return h.hexdigest()


def _sources():
  cu = sorted(glob.glob(os.path.join(CSRC, "cuda", "*.cu")))
  cu_hdr = sorted(glob.glob(os.path.join(CSRC, "cuda", "*.cuh")) + glob.glob(os.path.join(CSRC, "cuda", "*.h")))
  cpp, cpp_hdr = [], []
  for d in ("host", "data", "ckpt"):
    cpp += sorted(glob.glob(os.path.join(CSRC, d, "*.cpp")))
    cpp_hdr += sorted(glob.glob(os.path.join(CSRC, d, "*.h")))
  return cu, cu_hdr, cpp, cpp_hdr


def cuda_lib_path() -> str:
  return os.path.join(LIB_DIR, f"librecml_cuda{'_dbg' if DEBUG else ''}.so")


def _read_text(path: str) -> str:
  with open(path) as f:
    return f.read()


def host_lib_path() -> str:
  return os.path.join(LIB_DIR, f"librecml_host{_SUFFIX}.so")


def _run(cmd: list[str]) -> None:
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"command failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def _compile_all(srcs, hdrs, compiler_cmd, tag) -> tuple[list[str], bool]:
  os.makedirs(OBJ_DIR, exist_ok=True)
  # the flags are part of the key: another RECML_SANITIZE value or a debug build never reuses these objects
  hdr_digest = _digest(hdrs, tag + "|" + " ".join(NVCC_FLAGS if tag == "cuda" else CXX_FLAGS))
  jobs, objs = [], []
  for src in srcs:
    obj = os.path.join(OBJ_DIR, os.path.basename(src) + (_SUFFIX if tag == "host" else ("_dbg" if DEBUG else "")) + ".o")
    stamp = obj + ".sha"
    want = _digest([src], hdr_digest)
    objs.append(obj)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == want:
      continue
    jobs.append((src, obj, stamp, want))
  def one(job):
    src, obj, stamp, want = job
    _run(compiler_cmd(src, obj))
    with open(stamp, "w") as f:
      f.write(want)
  with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
    list(ex.map(one, jobs))
  return objs, bool(jobs)


def build_host(verbose: bool = False, force: bool = False) -> dict[str, str]:
  """Builds only the C++ host library (machines without nvcc: CI, CPU-only test runs)."""
  return build(verbose=verbose, force=force, only=("host",))


def build(verbose: bool = False, force: bool = False, only: tuple[str, ...] = ("cuda", "host")) -> dict[str, str]:
  """Builds whatever is out of date and returns the library paths."""
  os.makedirs(LIB_DIR, exist_ok=True)
  cu, cu_hdr, cpp, cpp_hdr = _sources()
  out = {}
  for name, srcs, hdrs, lib, comp, link in (
      ("cuda", cu, cu_hdr, cuda_lib_path(),
       lambda s, o: [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(CSRC, "cuda"), "-c", s, "-o", o],
       lambda objs, lib: [_nvcc(), "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]),
      ("host", cpp, cpp_hdr, host_lib_path(),
       lambda s, o: ["g++", *CXX_FLAGS, "-I", CSRC, "-c", s, "-o", o],
       lambda objs, lib: ["g++", "-shared", "-pthread", "-o", lib, *objs, "-lz", "-ldl",
                          *([f"-fsanitize={SANITIZE}"] if SANITIZE else [])])):
    if not srcs or name not in only:
      continue
    want = _digest(srcs + hdrs, name + "|" + " ".join(NVCC_FLAGS if name == "cuda" else CXX_FLAGS))
    stamp = lib + ".sha"
    if not force and os.path.exists(lib) and os.path.exists(stamp) and _read_text(stamp) == want:
      out[name] = lib
      continue
    if name == "cuda" and not os.path.exists(_nvcc()):
      raise RuntimeError("nvcc not found and librecml_cuda.so is missing or stale")
    if verbose:
      print(f"[recml_b200] building {os.path.basename(lib)} ...", file=sys.stderr)
    objs, _ = _compile_all(srcs, hdrs, comp, name)
    _run(link(objs, lib))
    with open(stamp, "w") as f:
      f.write(want)
    out[name] = lib
  return out


if __name__ == "__main__":
  print(build(verbose=True, force="--force" in sys.argv))
