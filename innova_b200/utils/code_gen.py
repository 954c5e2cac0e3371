"""Kernel source generator and validator: CUDA C++ for sm_100a, specialised per shape.

Reference behaviour covered (include/oil/code_gen.h:12-188): ``KernelSpec`` -> source text for the operator kinds
(elementwise activations and arithmetic, RMS / layer norm, softmax, embedding lookup, quantise-dequantise, a GEMM),
templates with placeholders, an unroll / vector-width choice per shape, ``validate`` (compile, run, compare against a
reference, time), a kernel cache, ``identify_slow_paths`` / ``improve_slow_path`` / ``auto_optimize`` (try the variants,
keep the fastest that is still correct) and ``generate_full_source`` / ``save_source``. The reference emits C++ with
AVX2 / AVX-512 / NEON intrinsics; the targets here are CUDA variants (elements per thread, threads per block, rows per
block), compiled by ``nvcc -gencode arch=compute_100a,code=sm_100a``. Compilation works without a GPU; running and
timing need one.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import tempfile
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

ELEMENTWISE = {
    "relu": "fmaxf(x, 0.f)",
    "silu": "x / (1.f + __expf(-x))",
    "gelu": "0.5f * x * (1.f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)))",
    "add": "x + y",
    "mul": "x * y",
    "residual_add": "x + y",
    "scale": "x * {scale}f",
}
KINDS = tuple(ELEMENTWISE) + ("rms_norm", "layer_norm", "softmax", "embedding_lookup", "quantize_dequantize", "gemm")


@dataclass
class KernelSpec:
    kind: str = "relu"
    M: int = 0              # rows (norms, softmax, gemm, embedding: tokens)
    N: int = 0              # row length / elements / gemm N
    K: int = 0              # gemm reduction length
    vec: int = 4            # elements per thread and step (1, 2, 4)
    threads: int = 256
    scale: float = 1.0
    block: int = 32         # quantisation block
    levels: int = 16        # quantisation levels
    name: str = ""


@dataclass
class GeneratedKernel:
    spec: KernelSpec
    source_code: str
    function_name: str
    validated: bool = False
    compiled: bool = False
    benchmark_ms: float = 0.0
    error_message: str = ""
    library: Optional[str] = None


@dataclass
class CodeValidationResult:
    syntax_valid: bool = False
    compiles: bool = False
    runs: bool = False
    correctness_pass: bool = False
    max_error: float = 0.0
    error_message: str = ""
    runtime_ms: float = 0.0


@dataclass
class SlowPath:
    op_name: str
    current_time_ms: float
    target_time_ms: float
    current_kernel: str = ""
    priority: int = 0


@dataclass
class CodeTemplate:
    name: str
    description: str
    template_code: str
    placeholders: List[str]
    kind: str


_HEADER = "#include <cuda_runtime.h>\n#include <stdint.h>\n#include <math.h>\n"

_T_ELEMENTWISE = """
extern "C" __global__ void __launch_bounds__(@THREADS@) @NAME@_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, long n) {
  const long stride = (long)gridDim.x * blockDim.x * @VEC@;
  for (long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * @VEC@; i < n; i += stride) {
#pragma unroll
    for (int j = 0; j < @VEC@; ++j) {
      if (i + j < n) {
        const float x = a[i + j];
        const float y = b ? b[i + j] : 0.f;
        (void)y;
        out[i + j] = @EXPR@;
      }
    }
  }
}
extern "C" int @NAME@(const float* a, const float* b, float* out, long n, void* stream) {
  long blocks = (n + @THREADS@ * @VEC@ - 1) / (@THREADS@ * @VEC@);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  @NAME@_kernel<<<(int)blocks, @THREADS@, 0, (cudaStream_t)stream>>>(a, b, out, n);
  return (int)cudaGetLastError();
}
"""

_T_ROW = """
// one warp per row of @N@ elements: the row is read once into registers, reduced with shuffles, written once
extern "C" __global__ void __launch_bounds__(@THREADS@) @NAME@_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out, int rows) {
  constexpr int N = @N@, PER = (N + 31) / 32;
  const int row = blockIdx.x * (@THREADS@ / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v[PER];
  float s1 = 0.f, s2 = 0.f, mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int c = j * 32 + lane;
    v[j] = c < N ? x[(long)row * N + c] : (@IS_SOFTMAX@ ? -INFINITY : 0.f);
    if (c < N) { s1 += v[j]; s2 += v[j] * v[j]; mx = fmaxf(mx, v[j]); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
@BODY@
}
extern "C" int @NAME@(const float* x, const float* w, float* out, int rows, void* stream) {
  const int per_block = @THREADS@ / 32;
  @NAME@_kernel<<<(rows + per_block - 1) / per_block, @THREADS@, 0, (cudaStream_t)stream>>>(x, w, out, rows);
  return (int)cudaGetLastError();
}
"""

_BODY = {
    "rms_norm": """  const float r = rsqrtf(s2 / N + 1e-5f);
#pragma unroll
  for (int j = 0; j < PER; ++j) { const int c = j * 32 + lane; if (c < N) out[(long)row * N + c] = v[j] * r * w[c]; }""",
    "layer_norm": """  const float mean = s1 / N, r = rsqrtf(fmaxf(s2 / N - mean * mean, 0.f) + 1e-5f);
#pragma unroll
  for (int j = 0; j < PER; ++j) { const int c = j * 32 + lane; if (c < N) out[(long)row * N + c] = (v[j] - mean) * r * w[c]; }""",
    "softmax": """  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) { v[j] = __expf(v[j] - mx); sum += (j * 32 + lane < N) ? v[j] : 0.f; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
  for (int j = 0; j < PER; ++j) { const int c = j * 32 + lane; if (c < N) out[(long)row * N + c] = v[j] / sum; }""",
}

_T_EMBED = """
extern "C" __global__ void @NAME@_kernel(const int* __restrict__ ids, const float* __restrict__ table, float* __restrict__ out, int tokens) {
  constexpr int D = @N@;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < (long)tokens * D; i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / D), d = (int)(i % D);
    const int id = min(max(ids[t], 0), @M@ - 1);
    out[i] = table[(long)id * D + d];
  }
}
extern "C" int @NAME@(const int* ids, const float* table, float* out, int tokens, void* stream) {
  @NAME@_kernel<<<148 * 4, @THREADS@, 0, (cudaStream_t)stream>>>(ids, table, out, tokens);
  return (int)cudaGetLastError();
}
"""

_T_QDQ = """
// block-@BLOCK@ abs-max scaling to @LEVELS@ uniform levels and back (one warp per block when @BLOCK@ == 32)
extern "C" __global__ void @NAME@_kernel(const float* __restrict__ x, float* __restrict__ out, long n) {
  const long nblk = (n + @BLOCK@ - 1) / @BLOCK@;
  for (long b = (long)blockIdx.x * blockDim.x + threadIdx.x; b < nblk; b += (long)gridDim.x * blockDim.x) {
    float amax = 0.f;
    for (int j = 0; j < @BLOCK@ && b * @BLOCK@ + j < n; ++j) amax = fmaxf(amax, fabsf(x[b * @BLOCK@ + j]));
    const float step = amax > 0.f ? 2.f * amax / (@LEVELS@ - 1) : 1.f;
    for (int j = 0; j < @BLOCK@ && b * @BLOCK@ + j < n; ++j) {
      const float q = rintf((x[b * @BLOCK@ + j] + amax) / step);
      out[b * @BLOCK@ + j] = q * step - amax;
    }
  }
}
extern "C" int @NAME@(const float* x, float* out, long n, void* stream) {
  @NAME@_kernel<<<148 * 2, @THREADS@, 0, (cudaStream_t)stream>>>(x, out, n);
  return (int)cudaGetLastError();
}
"""

_T_GEMM = """
// C[M, N] = A[M, K] * B[N, K]^T, fp32, @TILE@ x @TILE@ shared-memory tiles (a shape-specialised fallback; the framework's
// bf16 GEMMs are the tcgen05 kernels)
extern "C" __global__ void @NAME@_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C) {
  constexpr int M = @M@, N = @N@, K = @K@, T = @TILE@;
  __shared__ float sa[T][T + 1], sb[T][T + 1];
  const int tx = threadIdx.x, ty = threadIdx.y, row = blockIdx.y * T + ty, col = blockIdx.x * T + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += T) {
    sa[ty][tx] = (row < M && k0 + tx < K) ? A[(long)row * K + k0 + tx] : 0.f;
    sb[ty][tx] = (blockIdx.x * T + ty < N && k0 + tx < K) ? B[(long)(blockIdx.x * T + ty) * K + k0 + tx] : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < T; ++k) acc += sa[ty][k] * sb[tx][k];
    __syncthreads();
  }
  if (row < M && col < N) C[(long)row * N + col] = acc;
}
extern "C" int @NAME@(const float* A, const float* B, float* C, void* stream) {
  dim3 grid((@N@ + @TILE@ - 1) / @TILE@, (@M@ + @TILE@ - 1) / @TILE@), block(@TILE@, @TILE@);
  @NAME@_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(A, B, C);
  return (int)cudaGetLastError();
}
"""


def _fill(template: str, **vals) -> str:
    for k, v in vals.items():
        template = template.replace(f"@{k}@", str(v))
    return template


class CodeGenerator:
    NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-lineinfo"]

    def __init__(self, work_dir: Optional[str] = None):
        self.work_dir = work_dir or tempfile.mkdtemp(prefix="inv_codegen_")
        self.kernel_cache: Dict[str, GeneratedKernel] = {}
        self.templates: Dict[str, CodeTemplate] = {}
        self.timings: Dict[str, float] = {}        # op name -> measured ms (fed by the caller or by validate)
        for kind, tmpl in (("elementwise", _T_ELEMENTWISE), ("row", _T_ROW), ("embedding_lookup", _T_EMBED), ("quantize_dequantize", _T_QDQ),
                           ("gemm", _T_GEMM)):
            ph = sorted(set(p for p in __import__("re").findall(r"@(\w+)@", tmpl)))
            self.register_template(CodeTemplate(kind, f"default {kind} template", tmpl, ph, kind))

    # ------------------------------------------------------------------ templates
    def register_template(self, t: CodeTemplate):
        self.templates[t.name] = t

    def get_available_templates(self) -> List[str]:
        return sorted(self.templates)

    def apply_template(self, name: str, values: Dict[str, object]) -> str:
        t = self.templates[name]
        missing = [p for p in t.placeholders if p not in values]
        if missing:
            raise KeyError(f"template {name}: no value for {missing}")
        return _fill(t.template_code, **values)

    # ------------------------------------------------------------------ generation
    def make_function_name(self, s: KernelSpec) -> str:
        return s.name or f"gen_{s.kind}_m{s.M}_n{s.N}_k{s.K}_v{s.vec}_t{s.threads}"

    def generate_unrolled_loop(self, var: str, start: int, end: int, unroll: int, body: str) -> str:
        return f"#pragma unroll {unroll}\nfor (int {var} = {start}; {var} < {end}; ++{var}) {{\n  {body}\n}}\n"

    def generate_kernel_for_shape(self, s: KernelSpec) -> str:
        name = self.make_function_name(s)
        if s.kind in ELEMENTWISE:
            return self.apply_template("elementwise", {"NAME": name, "THREADS": s.threads, "VEC": s.vec, "EXPR": ELEMENTWISE[s.kind].format(scale=repr(float(s.scale)))})
        if s.kind in _BODY:
            return self.apply_template("row", {"NAME": name, "THREADS": s.threads, "N": s.N, "IS_SOFTMAX": int(s.kind == "softmax"), "BODY": _BODY[s.kind]})
        if s.kind == "embedding_lookup":
            return self.apply_template("embedding_lookup", {"NAME": name, "THREADS": s.threads, "N": s.N, "M": s.M})
        if s.kind == "quantize_dequantize":
            return self.apply_template("quantize_dequantize", {"NAME": name, "THREADS": s.threads, "BLOCK": s.block, "LEVELS": s.levels})
        if s.kind == "gemm":
            return self.apply_template("gemm", {"NAME": name, "M": s.M, "N": s.N, "K": s.K, "TILE": 16 if s.vec <= 2 else 32})
        raise ValueError(f"unknown kernel kind {s.kind}")

    def generate_optimized_kernel(self, s: KernelSpec) -> GeneratedKernel:
        name = self.make_function_name(s)
        if name not in self.kernel_cache:
            self.kernel_cache[name] = GeneratedKernel(s, self.generate_kernel_for_shape(s), name)
        return self.kernel_cache[name]

    def specialize_for_shape(self, kind: str, M: int = 0, N: int = 0, K: int = 0) -> GeneratedKernel:
        """Vector width from the divisibility of the length, threads from the row length."""
        n = N or M
        vec = 4 if n % 4 == 0 else (2 if n % 2 == 0 else 1)
        threads = 128 if (kind in _BODY and N <= 1024) else 256
        return self.generate_optimized_kernel(KernelSpec(kind, M, N, K, vec=vec, threads=threads))

    # -- one generator per operator, as the reference names them (include/oil/code_gen.h:103-121); each returns source text
    def generate_gemm(self, M: int, N: int, K: int) -> str:
        return self.specialize_for_shape("gemm", M, N, K).source_code

    def generate_rms_norm(self, dim: int) -> str:
        return self.specialize_for_shape("rms_norm", 0, dim).source_code

    def generate_layer_norm(self, dim: int) -> str:
        return self.specialize_for_shape("layer_norm", 0, dim).source_code

    def generate_softmax(self, dim: int) -> str:
        return self.specialize_for_shape("softmax", 0, dim).source_code

    def generate_relu(self, n: int) -> str:
        return self.specialize_for_shape("relu", 0, n).source_code

    def generate_silu(self, n: int) -> str:
        return self.specialize_for_shape("silu", 0, n).source_code

    def generate_gelu(self, n: int) -> str:
        return self.specialize_for_shape("gelu", 0, n).source_code

    def generate_add(self, n: int) -> str:
        return self.specialize_for_shape("add", 0, n).source_code

    def generate_mul(self, n: int) -> str:
        return self.specialize_for_shape("mul", 0, n).source_code

    def generate_residual_add(self, n: int) -> str:
        return self.specialize_for_shape("residual_add", 0, n).source_code

    def generate_scale(self, n: int, scale_val: float) -> str:
        vec = 4 if n % 4 == 0 else (2 if n % 2 == 0 else 1)
        return self.generate_optimized_kernel(KernelSpec("scale", 0, n, 0, vec=vec, scale=scale_val,
                                                         name=f"gen_scale_n{n}_s{abs(hash(float(scale_val))) % 10 ** 8}")).source_code

    def generate_embedding_lookup(self, vocab_size: int, embed_dim: int) -> str:
        return self.specialize_for_shape("embedding_lookup", vocab_size, embed_dim).source_code

    def generate_quantize_dequantize(self, n: int, block: int = 32, levels: int = 16) -> str:
        return self.generate_optimized_kernel(KernelSpec("quantize_dequantize", 0, n, 0, block=block, levels=levels,
                                                         name=f"gen_qdq_n{n}_b{block}_l{levels}")).source_code

    def generate_format_dispatch(self, op_name: str, formats: Sequence[str]) -> str:
        """A host function ``<op>_dispatch(format, ...)`` that switches on the weight format id and calls ``<op>_<format>``
        (declared ``extern "C"``; the caller links the per-format kernels). Unknown ids return -1."""
        from ..formats import oil
        decl = "".join(f'extern "C" int {op_name}_{f.lower()}(const void* w, const float* x, float* y, long n, void* stream);\n' for f in formats)
        cases = "".join(f"    case {oil.format_id(f)}: return {op_name}_{f.lower()}(w, x, y, n, stream);  // {f}\n" for f in formats)
        return (f"{decl}extern \"C\" int {op_name}_dispatch(int format, const void* w, const float* x, float* y, long n, void* stream) {{\n"
                f"  switch (format) {{\n{cases}    default: return -1;\n  }}\n}}\n")

    def generate_format_branch(self, op_name: str, fmt: str, dim: int) -> str:
        from ..formats import oil
        return f"if (format == {oil.format_id(fmt)}) return {op_name}_{fmt.lower()}(w, x, y, {int(dim)}L, stream);  // {fmt}\n"

    def generate_includes(self, includes: Sequence[str]) -> str:
        return "".join(f"#include <{h}>\n" for h in includes)

    def generate_loop_header(self, var: str, start: int, end: int, step: str = "1") -> str:
        inc = f"++{var}" if step == "1" else f"{var} += {step}"
        return f"for (long {var} = {start}; {var} < {end}; {inc})"

    def generate_if_block(self, condition: str, body: str, indent_level: int = 1) -> str:
        pad = "  " * indent_level
        return f"{pad}if ({condition}) {{\n{self.generate_block(body, indent_level + 1)}{pad}}}\n"

    def generate_block(self, body: str, indent_level: int) -> str:
        pad = "  " * indent_level
        return "".join(pad + line + "\n" for line in body.strip("\n").split("\n"))

    def generate_full_source(self, kernels: Sequence[GeneratedKernel]) -> str:
        return _HEADER + "".join(k.source_code for k in kernels)

    def save_source(self, path: str, source: str) -> bool:
        open(path, "w").write(source)
        return True

    def get_kernel(self, name: str) -> GeneratedKernel:
        return self.kernel_cache[name]

    def get_all_kernels(self) -> List[GeneratedKernel]:
        return list(self.kernel_cache.values())

    def clear_kernels(self):
        self.kernel_cache.clear()

    # ------------------------------------------------------------------ validation
    def compile_code(self, source: str, out_path: Optional[str] = None) -> Optional[str]:
        """nvcc -shared for sm_100a. Returns the library path, or None (``last_error`` holds the compiler output)."""
        tag = hashlib.sha1(source.encode()).hexdigest()[:16]
        cu, so = os.path.join(self.work_dir, tag + ".cu"), out_path or os.path.join(self.work_dir, tag + ".so")
        if os.path.exists(so):
            return so
        open(cu, "w").write(source if source.startswith("#include") else _HEADER + source)
        p = subprocess.run(["nvcc", *self.NVCC_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", so, cu], capture_output=True, text=True)
        self.last_error = p.stderr
        return so if p.returncode == 0 else None

    def _reference(self, s: KernelSpec, args):
        import torch.nn.functional as F
        k = s.kind
        if k in ELEMENTWISE:
            x, y = args
            return {"relu": lambda: x.relu(), "silu": lambda: F.silu(x), "gelu": lambda: F.gelu(x, approximate="tanh"), "add": lambda: x + y,
                    "mul": lambda: x * y, "residual_add": lambda: x + y, "scale": lambda: x * s.scale}[k]()
        if k == "rms_norm":
            x, w = args
            return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + 1e-5) * w
        if k == "layer_norm":
            x, w = args
            return F.layer_norm(x, (s.N,), w, None, 1e-5)
        if k == "softmax":
            return args[0].softmax(-1)
        if k == "embedding_lookup":
            ids, table = args
            return table[ids.long()]
        if k == "gemm":
            return args[0] @ args[1].t()
        raise ValueError(k)

    def validate(self, kernel: GeneratedKernel, iters: int = 20) -> CodeValidationResult:
        """Compiles; on a GPU also runs against the PyTorch reference and times the kernel with CUDA events."""
        res = CodeValidationResult()
        so = self.compile_code(_HEADER + kernel.source_code)
        res.syntax_valid = res.compiles = so is not None
        kernel.compiled, kernel.library = res.compiles, so
        if not res.compiles:
            res.error_message = kernel.error_message = self.last_error
            return res
        if not torch.cuda.is_available():
            return res
        s, dev = kernel.spec, torch.device("cuda")
        fn = getattr(ctypes.CDLL(so), kernel.function_name)
        g = torch.Generator(device=dev).manual_seed(0)
        rows = s.M or 64
        if s.kind in ELEMENTWISE:
            n = s.N or s.M or (1 << 20)
            x, y = torch.randn(n, device=dev, generator=g), torch.randn(n, device=dev, generator=g)
            out = torch.empty_like(x)
            call = lambda: fn(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_long(n), None)
            ref = self._reference(s, (x, y))
        elif s.kind in _BODY:
            x, w = torch.randn(rows, s.N, device=dev, generator=g), torch.rand(s.N, device=dev, generator=g) + 0.5
            out = torch.empty_like(x)
            call = lambda: fn(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(rows), None)
            ref = self._reference(s, (x, w))
        elif s.kind == "embedding_lookup":
            ids = torch.randint(0, s.M, (256,), device=dev, dtype=torch.int32, generator=g)
            table = torch.randn(s.M, s.N, device=dev, generator=g)
            out = torch.empty(256, s.N, device=dev)
            call = lambda: fn(ctypes.c_void_p(ids.data_ptr()), ctypes.c_void_p(table.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(256), None)
            ref = self._reference(s, (ids, table))
        elif s.kind == "quantize_dequantize":
            n = max(s.block, (s.N or 1 << 16) // s.block * s.block)      # whole blocks, so that the check below can view them
            x = torch.randn(n, device=dev, generator=g)
            out = torch.empty_like(x)
            call = lambda: fn(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_long(n), None)
            ref = None
        else:
            A, B = torch.randn(s.M, s.K, device=dev, generator=g), torch.randn(s.N, s.K, device=dev, generator=g)
            out = torch.empty(s.M, s.N, device=dev)
            call = lambda: fn(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()), ctypes.c_void_p(out.data_ptr()), None)
            ref = self._reference(s, (A, B))
        torch.cuda.synchronize()
        rc = call()
        torch.cuda.synchronize()
        res.runs = rc == 0
        if ref is not None:
            res.max_error = float((out - ref).abs().max() / ref.abs().max().clamp_min(1e-6))
            res.correctness_pass = res.runs and res.max_error < 2e-3
        else:          # quantise-dequantise: the error is bounded by half a step of the block's grid
            step = 2 * x.view(-1, s.block).abs().amax(-1, keepdim=True) / (s.levels - 1)
            res.max_error = float(((out - x).view(-1, s.block).abs() / step.clamp_min(1e-12)).max())
            res.correctness_pass = res.runs and res.max_error <= 0.5 + 1e-3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        res.runtime_ms = kernel.benchmark_ms = e0.elapsed_time(e1) / iters
        kernel.validated = res.correctness_pass
        self.timings[kernel.function_name] = res.runtime_ms
        return res

    # ------------------------------------------------------------------ optimisation loop
    def record_timing(self, op_name: str, ms: float):
        self.timings[op_name] = ms

    def identify_slow_paths(self, threshold_ms: float = 1.0) -> List[SlowPath]:
        slow = [SlowPath(n, t, threshold_ms, n, int(t / threshold_ms)) for n, t in self.timings.items() if t > threshold_ms]
        return sorted(slow, key=lambda p: -p.priority)

    def variants(self, s: KernelSpec) -> List[KernelSpec]:
        out = []
        for vec in (1, 2, 4):
            for threads in (128, 256, 512):
                if s.kind in _BODY and vec != s.vec:
                    continue       # the row kernels have no vector width
                out.append(KernelSpec(s.kind, s.M, s.N, s.K, vec, threads, s.scale, s.block, s.levels))
        return out

    def improve_slow_path(self, base: KernelSpec) -> GeneratedKernel:
        """Validates every variant of the spec and returns the fastest correct one (the first that compiles without a GPU)."""
        best = None
        for v in self.variants(base):
            k = self.generate_optimized_kernel(v)
            r = self.validate(k)
            if not r.compiles:
                continue
            if not torch.cuda.is_available():
                return k
            if r.correctness_pass and (best is None or k.benchmark_ms < best.benchmark_ms):
                best = k
        return best

    def auto_optimize(self, specs: Sequence[KernelSpec]) -> List[GeneratedKernel]:
        return [k for k in (self.improve_slow_path(s) for s in specs) if k is not None]
