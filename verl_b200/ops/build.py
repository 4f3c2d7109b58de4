"""In-tree build of the sm_100a native library ``verl_b200/ops/_C.so``.

CUDA sources under ``csrc/`` are plain CUDA (no torch headers) and export C launchers; a single
``bindings.cpp`` adapts them to ``torch.ops.verl_b200.*``.  Objects are cached by content hash in
``verl_b200/ops/_build`` so an unchanged tree loads without invoking a compiler.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

OPS_DIR = Path(__file__).resolve().parent
CSRC = OPS_DIR / "csrc"
BUILD = OPS_DIR / "_build"
LIB = OPS_DIR / "_C.so"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _hash(paths, extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd, log: Path) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.write_text(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({' '.join(cmd[:3])} ...):\n{proc.stdout[-4000:]}")


def sources():
    cu = sorted(CSRC.glob("*.cu"))
    cpp = sorted(CSRC.glob("*.cpp"))
    hdr = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    return cu, cpp, hdr


def is_current() -> bool:
    stamp = BUILD / "stamp.json"
    if not LIB.exists() or not stamp.exists():
        return False
    cu, cpp, hdr = sources()
    try:
        return json.loads(stamp.read_text()).get("hash") == _hash(cu + cpp + hdr, " ".join(NVCC_FLAGS))
    except Exception:
        return False


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link ``_C.so``. Returns the library path."""
    cu, cpp, hdr = sources()
    if not force and is_current():
        return LIB
    from torch.utils import cpp_extension as ce
    import torch

    BUILD.mkdir(exist_ok=True)
    hdr_hash = _hash(hdr, " ".join(NVCC_FLAGS))
    jobs = []
    objs = []
    for src in cu:
        obj = BUILD / (src.stem + ".o")
        tag = BUILD / (src.stem + ".hash")
        want = _hash([src], hdr_hash)
        objs.append(obj)
        if obj.exists() and tag.exists() and tag.read_text() == want and not force:
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, BUILD / (src.stem + ".log"), tag, want))
    inc = []
    for p in ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(cuda=True):
        inc += ["-I", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in cpp:
        obj = BUILD / (src.stem + ".o")
        tag = BUILD / (src.stem + ".hash")
        want = _hash([src], hdr_hash + torch.__version__)
        objs.append(obj)
        if obj.exists() and tag.exists() and tag.read_text() == want and not force:
            continue
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
               *inc, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, BUILD / (src.stem + ".log"), tag, want))

    def work(job):
        cmd, log, tag, want = job
        _run(cmd, log)
        tag.write_text(want)
        if verbose:
            print(f"[build] {log.stem} ok", file=sys.stderr)

    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as ex:
        list(ex.map(work, jobs))

    libdirs = ce.library_paths(device_type="cuda") if "device_type" in ce.library_paths.__code__.co_varnames else ce.library_paths(cuda=True)
    link = ["g++", "-shared", "-o", str(LIB), *[str(o) for o in objs]]
    for d in libdirs:
        link += ["-L", d, f"-Wl,-rpath,{d}"]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    _run(link, BUILD / "link.log")
    (BUILD / "stamp.json").write_text(json.dumps({"hash": _hash(cu + cpp + hdr, " ".join(NVCC_FLAGS))}))
    return LIB


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output (registers, spills, shared memory) of the last build."""
    out = []
    for log in sorted(BUILD.glob("*.log")):
        txt = log.read_text()
        if "ptxas info" in txt:
            out.append(f"== {log.stem}\n" + "\n".join(l for l in txt.splitlines() if "ptxas info" in l or "Function properties" in l or "bytes stack" in l))
    return "\n".join(out)


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(path)
    if "--report" in sys.argv:
        print(ptxas_report())
