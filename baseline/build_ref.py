"""Builds the UNMODIFIED reference sources out of tree into ``baseline/_ref/``.

``libref_train.a`` holds the reference's library targets oil_core, oil_math, oil_format, oil_kernel, oil_model,
oil_inference, oil_tokenizer and oil_trainer exactly as its CMakeLists.txt lists them (CMakeLists.txt:41-153), with the one
translation unit of oil_trainer that cannot compile on Linux left out (src/hf_streamer.cpp includes <windows.h> and WinHTTP
unconditionally; nothing else in the trainer refers to it). ``ref_train_bench`` links ``baseline/ref_train_bench.cpp``
against it, ``ref_quant_oracle`` links ``baseline/ref_quant_oracle.cpp`` (codebook wire form and the whole-tensor
codebook checkpoint, for the format tests). Flags are the reference's own GCC Release flags with AVX2 (cmake/compiler.cmake:30-47) minus ``-march=native``,
so that a binary built on one machine runs on another x86-64 host with AVX2.

    python baseline/build_ref.py [--reference /path/to/InNova]
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
TARGETS = ["oil_core", "oil_math", "oil_format", "oil_kernel", "oil_model", "oil_inference", "oil_tokenizer", "oil_trainer"]
LEFT_OUT = {"src/hf_streamer.cpp"}
FLAGS = ["-std=c++20", "-O3", "-DNDEBUG", "-mavx2", "-mavx", "-mbmi2", "-mfma", "-fPIC", "-w", "-pthread"]


def reference_root(argv=None) -> Path:
    argv = sys.argv if argv is None else argv
    if "--reference" in argv:
        return Path(argv[argv.index("--reference") + 1])
    return Path(os.environ.get("INNOVA_REFERENCE", "/root/reference"))


def target_sources(ref: Path, target: str):
    text = (ref / "CMakeLists.txt").read_text()
    m = re.search(r"add_library\(%s\s+([^)]*)\)" % re.escape(target), text)
    if not m:
        raise RuntimeError("target %s not found in the reference's CMakeLists.txt" % target)
    return [s for s in m.group(1).split() if s.endswith(".cpp") and s not in LEFT_OUT]


def _config_header(ref: Path, inc: Path):
    """oil_config.h as CMake's configure_file would write it with OIL_AVX2 on and the GPU back-ends off."""
    src = (ref / "oil_config.h.in").read_text()
    out = []
    for line in src.splitlines():
        m = re.match(r"#cmakedefine (\w+)", line)
        if m:
            out.append("#define %s" % m.group(1) if m.group(1) == "OIL_AVX2" else "/* #undef %s */" % m.group(1))
        else:
            out.append(line)
    inc.mkdir(parents=True, exist_ok=True)
    (inc / "oil_config.h").write_text("\n".join(out) + "\n")


def build(ref: Path | None = None, force: bool = False) -> Path:
    ref = ref or reference_root()
    exe = OUT / "ref_train_bench"
    driver = HERE / "ref_train_bench.cpp"
    oracle = HERE / "ref_quant_oracle.cpp"
    if exe.exists() and (OUT / "ref_quant_oracle").exists() and not force and exe.stat().st_mtime > driver.stat().st_mtime and \
            (OUT / "ref_quant_oracle").stat().st_mtime > oracle.stat().st_mtime:
        return exe
    if not (ref / "CMakeLists.txt").exists():
        raise RuntimeError("reference sources not found at %s" % ref)
    cxx = shutil.which("g++")
    if cxx is None:
        raise RuntimeError("g++ not found")
    obj = OUT / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    _config_header(ref, OUT / "cfg")
    inc = ["-I", str(ref / "include"), "-I", str(OUT / "cfg"), "-I", str(ref)]
    srcs = [s for t in TARGETS for s in target_sources(ref, t)]

    def cc(s):
        o = obj / (s.replace("/", "_") + ".o")
        if force or not o.exists():
            r = subprocess.run([cxx, *FLAGS, *inc, "-c", str(ref / s), "-o", str(o)], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("reference source %s failed to compile:\n%s" % (s, r.stderr[-2000:]))
        return o

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(cc, srcs))
    lib = OUT / "libref_train.a"
    if lib.exists():
        lib.unlink()
    subprocess.run(["ar", "rcs", str(lib), *map(str, objs)], check=True)
    for src, out in ((driver, exe), (HERE / "ref_quant_oracle.cpp", OUT / "ref_quant_oracle")):
        r = subprocess.run([cxx, *FLAGS, *inc, str(src), str(lib), "-o", str(out)], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("%s failed to link:\n%s" % (src.name, r.stderr[-3000:]))
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
