"""Build the product libraries in-tree with nvcc for sm_100a.

  build()        libkllm_b200.so   every .cu under csrc/ (the C-ABI of include/kllm_b200.h and kllm_seq.h)
  build_seq()    libkllm_seq.so    only the sequence-batch engine (csrc/seq_*.cu + runtime.cu): what a batched
                                   model needs, without the single-sequence decoder's kernels
  build_seq_tools()                kuiper_trace / kuiper_generate linked against libkllm_seq.so with plain g++

Used by __graft_entry__.build(), tests, bench.py and bin/trace_run.  No JIT cache: the .so files land in
kuiperllama_b200/lib/ so they travel to the GPU box with the repo snapshot.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libkllm_b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources():
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*")) + list((PKG.parent / "include").glob("*.h"))):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ into one shared library; no-op when up to date."""
    LIBDIR.mkdir(exist_ok=True)
    stamp = LIBDIR / ".stamp"
    fp = _fingerprint()
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == fp:
        return LIB
    objs = []
    objdir = LIBDIR / "obj"
    objdir.mkdir(exist_ok=True)
    common = [nvcc_path(), "-std=c++17", "-O3", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC",
              "-I", str(PKG.parent / "include")]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in _sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", str(src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        text = out.decode(errors="replace")
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"[kllm build] {src.name} FAILED\n{text}\n")
        elif verbose or text.strip():
            sys.stderr.write(f"[kllm build] {src.name}\n{text}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc_path(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs)])
    stamp.write_text(fp)
    return LIB


# ---- the sequence-batch engine alone ------------------------------------------------------------------------------
SEQ_LIB = LIBDIR / "libkllm_seq.so"
KUIPER = PKG / "kuiper"
SEQ_TOOLS_DIR = KUIPER / "_build" / "seq"
# host sources of the batched-model side: the allocator, the model-folder readers, the scheduler, and every model
# family registered with KLLM_REGISTER_SEQUENCE_MODEL
SEQ_HOST_SOURCES = ["source/base/alloc.cpp", "source/base/buffer.cpp", "source/model/safetensors.cpp",
                    "source/model/sequence_model.cpp", "source/model/fobolorn.cpp",
                    "source/model/kikunex.cpp", "source/model/vurazen.cpp", "source/model/bukuvik.cpp"]
SEQ_TOOLS = ["kuiper_trace", "kuiper_generate"]
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))


def _seq_sources():
    return [CSRC / "runtime.cu"] + sorted(CSRC.glob("seq_*.cu"))


def _hash_files(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()


class _Lock:
    """One build at a time per checkout (several runners may start together)."""

    def __init__(self, path: Path):
        self.path = path

    def __enter__(self):
        import fcntl
        self.f = open(self.path, "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        self.f.close()


def _run_all(cmds, what):
    procs = [(c, subprocess.Popen(c, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)) for c in cmds]
    failed = False
    for c, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"[kllm build] {' '.join(map(str, c))} FAILED\n{out.decode(errors='replace')}\n")
    if failed:
        raise RuntimeError(f"{what} failed")


def build_seq(force: bool = False) -> Path:
    """Compile the sequence-batch engine into libkllm_seq.so; no-op when up to date."""
    LIBDIR.mkdir(exist_ok=True)
    with _Lock(LIBDIR / ".seq.lock"):
        stamp = LIBDIR / ".seq.stamp"
        fp = _hash_files(list(CSRC.glob("seq_*")) + [CSRC / "runtime.cu", CSRC / "kllm_host.h"] +
                         list((PKG.parent / "include").glob("*.h")))
        if not force and SEQ_LIB.exists() and stamp.exists() and stamp.read_text() == fp:
            return SEQ_LIB
        objdir = LIBDIR / "obj_seq"
        objdir.mkdir(exist_ok=True)
        common = [nvcc_path(), "-std=c++17", "-O3", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC",
                  "-I", str(PKG.parent / "include")]
        objs = [objdir / (src.stem + ".o") for src in _seq_sources()]
        _run_all([common + ["-c", str(src), "-o", str(obj)] for src, obj in zip(_seq_sources(), objs)], "nvcc")
        subprocess.check_call([nvcc_path(), *ARCH, "-shared", "-o", str(SEQ_LIB), *map(str, objs)])
        stamp.write_text(fp)
    return SEQ_LIB


def build_seq_tools(force: bool = False) -> Path:
    """kuiper_trace and kuiper_generate for batched models, linked against libkllm_seq.so (g++, no CMake)."""
    lib = build_seq(force)
    SEQ_TOOLS_DIR.mkdir(parents=True, exist_ok=True)
    with _Lock(SEQ_TOOLS_DIR / ".lock"):
        stamp = SEQ_TOOLS_DIR / ".stamp"
        srcs = [KUIPER / s for s in SEQ_HOST_SOURCES]
        tools = [KUIPER / "tools" / (t + ".cpp") for t in SEQ_TOOLS]
        fp = _hash_files(srcs + tools + list((KUIPER / "include").rglob("*.h")) +
                         list((PKG.parent / "include").glob("*.h"))) + lib.read_bytes()[:0].hex() + \
            str(lib.stat().st_mtime_ns)
        if not force and stamp.exists() and stamp.read_text() == fp and \
                all((SEQ_TOOLS_DIR / t).exists() for t in SEQ_TOOLS):
            return SEQ_TOOLS_DIR
        cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
        inc = ["-I", str(KUIPER / "include"), "-I", str(PKG.parent / "include"), "-I", str(CUDA_HOME / "include"),
               "-I", str(PKG / "third_party" / "miniglog")]
        flags = [cxx, "-std=c++20", "-O2", "-fPIC", *inc]
        objs = [SEQ_TOOLS_DIR / (s.stem + ".o") for s in srcs]
        _run_all([flags + ["-c", str(s), "-o", str(o)] for s, o in zip(srcs, objs)], "g++")
        link = ["-L", str(LIBDIR), "-lkllm_seq", "-L", str(CUDA_HOME / "lib64"), "-lcudart", "-lpthread",
                f"-Wl,-rpath,{LIBDIR}", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}"]
        _run_all([flags + [str(t), *map(str, objs), "-o", str(SEQ_TOOLS_DIR / t.stem), *link] for t in tools], "g++")
        stamp.write_text(fp)
    return SEQ_TOOLS_DIR


if __name__ == "__main__":
    if "--seq" in sys.argv:
        print(build_seq_tools(force="--force" in sys.argv))
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
