import shutil

import pytest
import torch

from innova_b200.utils.code_gen import KINDS, CodeGenerator, CodeTemplate, KernelSpec

needs_nvcc = pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not on PATH")


def test_sources_templates_and_cache(tmp_path):
    cg = CodeGenerator(str(tmp_path))
    k = cg.specialize_for_shape("rms_norm", M=64, N=768)
    assert k.spec.threads == 128 and "constexpr int N = 768" in k.source_code and k.function_name in k.source_code
    assert cg.specialize_for_shape("rms_norm", M=64, N=768) is k and len(cg.get_all_kernels()) == 1
    e = cg.specialize_for_shape("silu", N=1001)
    assert e.spec.vec == 1 and "__expf" in e.source_code
    assert "x * 0.5f" in cg.generate_kernel_for_shape(KernelSpec("scale", N=16, scale=0.5))
    cg.register_template(CodeTemplate("double", "out = 2x", "float @NAME@(float x) { return @FACTOR@ * x; }", ["FACTOR", "NAME"], "custom"))
    assert cg.apply_template("double", {"NAME": "f", "FACTOR": 2}) == "float f(float x) { return 2 * x; }"
    with pytest.raises(KeyError):
        cg.apply_template("double", {"NAME": "f"})
    assert "double" in cg.get_available_templates()
    src = cg.generate_full_source(cg.get_all_kernels())
    assert src.startswith("#include") and cg.save_source(str(tmp_path / "all.cu"), src)
    cg.record_timing("attention", 3.0); cg.record_timing("norm", 0.2)
    slow = cg.identify_slow_paths(1.0)
    assert [p.op_name for p in slow] == ["attention"] and slow[0].priority == 3
    assert len(cg.variants(KernelSpec("relu", N=1024))) == 9 and "#pragma unroll 4" in cg.generate_unrolled_loop("i", 0, 8, 4, "x += i;")


@needs_nvcc
def test_every_kind_compiles_for_sm100a(tmp_path):
    cg = CodeGenerator(str(tmp_path))
    kernels = [cg.generate_optimized_kernel(KernelSpec(kind, M=96, N=160, K=64)) for kind in KINDS]
    so = cg.compile_code(cg.generate_full_source(kernels))
    assert so is not None, cg.last_error
    assert cg.compile_code("extern \"C\" __global__ void broken( { }") is None and "error" in cg.last_error


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["gelu", "add", "scale", "rms_norm", "layer_norm", "softmax", "embedding_lookup", "quantize_dequantize", "gemm"])
def test_gpu_generated_kernels_match_pytorch(tmp_path, kind):
    cg = CodeGenerator(str(tmp_path))
    k = cg.generate_optimized_kernel(KernelSpec(kind, M=100, N=1000 if kind not in ("gemm",) else 72, K=200, scale=0.25))
    r = cg.validate(k, iters=3)
    assert r.compiles and r.runs and r.correctness_pass, (kind, r)
    assert r.runtime_ms > 0 and k.validated


@pytest.mark.gpu
def test_gpu_auto_optimize_picks_a_correct_variant(tmp_path):
    cg = CodeGenerator(str(tmp_path))
    best = cg.auto_optimize([KernelSpec("silu", N=1 << 20)])
    assert len(best) == 1 and best[0].validated and best[0].benchmark_ms > 0


def test_named_generators_and_format_dispatch(tmp_path):
    cg = CodeGenerator(str(tmp_path))
    assert "constexpr int M = 64, N = 96, K = 32" in cg.generate_gemm(64, 96, 32) and "rsqrtf(s2 / N" in cg.generate_rms_norm(768)
    assert "mean" in cg.generate_layer_norm(512) and "__expf(v[j] - mx)" in cg.generate_softmax(1000)
    for gen, expr in ((cg.generate_relu, "fmaxf(x, 0.f)"), (cg.generate_silu, "__expf(-x)"), (cg.generate_gelu, "tanhf"), (cg.generate_add, "x + y"),
                      (cg.generate_mul, "x * y"), (cg.generate_residual_add, "x + y")):
        assert expr in gen(4096)
    assert "x * 0.25f" in cg.generate_scale(1000, 0.25) and "x * 3.0f" in cg.generate_scale(1000, 3.0)       # one kernel per scale value
    assert "32000 - 1" in cg.generate_embedding_lookup(32000, 256) and "(256 - 1)" in cg.generate_quantize_dequantize(4096, 64, 256)
    src = cg.generate_format_dispatch("gemv", ["OIL4", "OIL8"])
    assert 'extern "C" int gemv_oil4(' in src and "case 3: return gemv_oil4(w, x, y, n, stream);  // OIL4" in src and "default: return -1;" in src
    assert cg.generate_format_branch("gemv", "OIL8", 512).startswith("if (format == 4) return gemv_oil8(w, x, y, 512L, stream);")
    assert cg.generate_includes(["cmath", "vector"]) == "#include <cmath>\n#include <vector>\n"
    assert cg.generate_loop_header("i", 0, 10) == "for (long i = 0; i < 10; ++i)" and cg.generate_loop_header("i", 0, 10, "4").endswith("i += 4)")
    assert cg.generate_if_block("x > 0", "y = x;\nz = y;", 1) == "  if (x > 0) {\n    y = x;\n    z = y;\n  }\n"


@needs_nvcc
def test_format_dispatch_source_compiles_as_host_code(tmp_path):
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    cg = CodeGenerator(str(tmp_path))
    src = cg.generate_format_dispatch("gemv", ["OIL1", "OIL4", "OIL8", "OIL32"])
    path = tmp_path / "dispatch.cpp"
    path.write_text(src)
    assert subprocess.run(["g++", "-std=c++17", "-c", "-o", str(tmp_path / "d.o"), str(path)], capture_output=True).returncode == 0
