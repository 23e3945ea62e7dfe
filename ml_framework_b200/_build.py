"""In-tree build of ``libmlfb200.so`` (CUDA kernels + C++ runtime) for sm_100a.

The library has a plain C ABI (see ``csrc/mlf_api.h``) and is loaded with ``ctypes``; it links
only against the CUDA runtime, so it builds in seconds with ``nvcc`` and needs no GPU to
compile. Objects are cached under ``ml_framework_b200/_build/`` and rebuilt when a source or
any header changes.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
LIB_PATH = PKG_DIR / "libmlfb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3",
    "--expt-relaxed-constexpr", "--use_fast_math",
    "-Xptxas", "-v",
    "-DMLF_BUILD",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _sources() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")))


def _headers_digest() -> str:
    h = hashlib.sha1()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(nvcc: str, src: Path, obj: Path, log: Path) -> tuple[Path, int, str]:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    return src, r.returncode, r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every source under ``csrc/`` for sm_100a and link ``libmlfb200.so``."""
    nvcc = _nvcc()
    obj_dir = BUILD_DIR / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)
    stamp = BUILD_DIR / "headers.sha1"
    digest = _headers_digest()
    headers_changed = force or (not stamp.exists()) or stamp.read_text() != digest
    jobs = []
    objs = []
    for src in _sources():
        rel = src.relative_to(CSRC)
        obj = obj_dir / ("_".join(rel.with_suffix("").parts) + ".o")
        objs.append(obj)
        if headers_changed or not obj.exists() or obj.stat().st_mtime < src.stat().st_mtime:
            jobs.append((src, obj, obj.with_suffix(".log")))
    failed = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, l) for s, o, l in jobs]
            for f in futs:
                src, rc, out = f.result()
                if verbose or rc != 0:
                    sys.stderr.write(f"[mlf build] {src.relative_to(CSRC)} rc={rc}\n{out}\n")
                if rc != 0:
                    failed.append(src)
    if failed:
        raise RuntimeError(f"nvcc failed for: {', '.join(str(s) for s in failed)}")
    stamp.write_text(digest)
    need_link = bool(jobs) or not LIB_PATH.exists()
    if need_link:
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        os.replace(tmp, LIB_PATH)
    DIGEST_PATH.write_text(_tree_digest())
    return LIB_PATH


DIGEST_PATH = PKG_DIR / "libmlfb200.so.digest"


def _tree_digest() -> str:
    """Digest of every source and header under ``csrc/`` and of the compiler flags."""
    h = hashlib.sha1()
    for p in sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def stale() -> bool:
    """True when the built library does not correspond to the sources under ``csrc/`` (by content, so that a copy
    of the tree with fresh time stamps is not taken for a change)."""
    if not LIB_PATH.exists() or not DIGEST_PATH.exists():
        return True
    return DIGEST_PATH.read_text().strip() != _tree_digest()


def resource_report() -> str:
    """ptxas register / spill / shared-memory lines of the last build, per source."""
    out = []
    for log in sorted((BUILD_DIR / "obj").glob("*.log")):
        lines = [l for l in log.read_text().splitlines() if "registers" in l or "spill" in l or "Compiling entry" in l]
        if lines:
            out.append(f"== {log.stem}")
            out.extend(lines)
    return "\n".join(out)


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(p)
    if "-r" in sys.argv:
        print(resource_report())
