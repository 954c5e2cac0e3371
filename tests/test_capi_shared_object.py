"""liboil_capi.so exports the reference's five C entry points; a C program links against it and generates text."""
import os
import shutil
import subprocess
import sys
import sysconfig

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C_MAIN = r"""
#include <stdio.h>
#include <string.h>
#include "oil_capi.h"
int main(int argc, char** argv) {
  OilModel* bad = oil_model_load("/nonexistent/model.oil");
  if (bad != NULL || strlen(oil_last_error()) == 0) { printf("FAIL missing file accepted\n"); return 1; }
  OilModel* m = oil_model_load(argv[1]);
  if (!m) { printf("FAIL load: %s\n", oil_last_error()); return 2; }
  char* a = oil_generate(m, "the quick", 6);
  if (!a) { printf("FAIL generate: %s\n", oil_last_error()); return 3; }
  char* b = oil_generate(m, "the quick", 6);
  if (!b || strcmp(a, b) != 0) { printf("FAIL greedy generations differ\n"); return 4; }
  if (strlen(oil_last_error()) != 0) { printf("FAIL stale error\n"); return 5; }
  printf("OK [%s]\n", a);
  oil_free_string(a);
  oil_free_string(b);
  if (oil_generate(NULL, "x", 1) != NULL || strlen(oil_last_error()) == 0) { printf("FAIL null model\n"); return 6; }
  oil_model_free(m);
  oil_model_free(NULL);
  return 0;
}
"""


def test_c_program_loads_and_generates(tmp_path):
    from innova_b200 import build
    so = build.build_capi()
    cc = shutil.which("gcc") or shutil.which("cc")
    if so is None or cc is None:
        pytest.skip("no Python development files or no C compiler")
    syms = subprocess.run(["nm", "-D", str(so)], capture_output=True, text=True).stdout
    for name in ("oil_model_load", "oil_model_free", "oil_generate", "oil_free_string", "oil_last_error"):
        assert f" T {name}" in syms
    # a tiny model trained by the CLI
    corpus = tmp_path / "c.txt"
    corpus.write_text("the quick brown fox jumps over the lazy dog. " * 100)
    model = str(tmp_path / "m.oil")
    r = subprocess.run([sys.executable, "-m", "innova_b200.cli.train", "--model", model, "--data", str(corpus), "--batch-size", "4",
                        "--seq-length", "32", "--hidden-size", "32", "--num-layers", "1", "--num-heads", "1", "--max-steps", "5", "--device", "cpu",
                        "--vocab-size", "256"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    (tmp_path / "main.c").write_text(C_MAIN)
    exe = str(tmp_path / "capi_test")
    libdir = os.path.dirname(str(so))
    r = subprocess.run([cc, str(tmp_path / "main.c"), "-I", os.path.join(ROOT, "innova_b200", "csrc", "capi"), "-L", libdir, "-loil_capi",
                        f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{sysconfig.get_config_var('LIBDIR')}", "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    env = dict(os.environ, INNOVA_B200_PYTHON=sys.executable, INNOVA_B200_ROOT=ROOT, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([exe, model], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and r.stdout.startswith("OK ["), r.stdout + r.stderr
