"""Run-time compiled sm_100a kernels: CUDA source -> ``nvcc -cubin`` -> cached cubin + manifest -> driver-API module -> launch on the
current PyTorch stream.

Two layers:

``compile_cubin`` / ``JitModule``   source text is hashed together with the flags; ``<cache>/<name>-<hash>.cubin`` and a JSON manifest
                                    (entry points, architecture, flags, source hash, registers / shared memory as reported by
                                    ``ptxas -v``) are written once and reused.  The cache directory defaults to ``_ext/jit`` inside the
                                    package, so kernels compiled ahead of time travel with the tree; ``SUROGATE_JIT_CACHE`` moves it.
                                    Loading goes through the CUDA driver API (``cuModuleLoadData`` / ``cuModuleGetFunction`` /
                                    ``cuLaunchKernel``) on PyTorch's context and stream: no host compiler, no Python extension build.
``ElementwiseOp``                   a generator for fused element-wise ops with hand-written derivatives: one forward kernel and one
                                    backward kernel over 8-wide bf16 / 4-wide fp32 vectors, wrapped in an autograd function.  Model
                                    families whose activations are not among the fixed kernels (squared ReLU, tanh soft-cap, GeGLU,
                                    clamped GLU) get a single-pass CUDA kernel from a two-line description (``runtime/torch_fns.py``).

Parity: surogate/kernels/jit_compile.py + csrc/src/runtime/jit/jit_kernel_loader.* (AOT-compiled Triton / CuTe-DSL cubins with JSON
manifests loaded through the driver API).  Here the kernel language is CUDA C++ for sm_100a and the compiler is nvcc.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
import re
import subprocess
import tempfile
import threading
from dataclasses import dataclass
from typing import Any, Dict, List, Sequence, Tuple

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo"]
_lock = threading.Lock()


def cache_dir() -> str:
    d = os.environ.get("SUROGATE_JIT_CACHE") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_ext", "jit")
    os.makedirs(d, exist_ok=True)
    return d


def nvcc_path() -> str:
    home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    p = os.path.join(home, "bin", "nvcc")
    return p if os.path.exists(p) else "nvcc"


@dataclass
class Manifest:
    name: str
    entries: List[str]
    arch: str
    flags: List[str]
    source_sha256: str
    cubin: str
    resources: Dict[str, Dict[str, int]]

    def to_json(self) -> Dict[str, Any]:
        return dict(self.__dict__)


def _parse_ptxas(log: str) -> Dict[str, Dict[str, int]]:
    out: Dict[str, Dict[str, int]] = {}
    cur = None
    for line in log.splitlines():
        m = re.search(r"Compiling entry function '(\w+)'", line)
        if m:
            cur = m.group(1)
            out[cur] = {}
            continue
        if cur and "Used" in line:
            r = re.search(r"Used (\d+) registers", line)
            s = re.search(r"(\d+) bytes smem", line)
            out[cur]["registers"] = int(r.group(1)) if r else 0
            out[cur]["shared_bytes"] = int(s.group(1)) if s else 0
        if cur and "bytes spill stores" in line:
            sp = re.search(r"(\d+) bytes spill stores", line)
            out[cur]["spill_store_bytes"] = int(sp.group(1)) if sp else 0
    return out


def compile_cubin(name: str, source: str, extra_flags: Sequence[str] = ()) -> Manifest:
    """Compile (or find in the cache) and return the manifest.  Works without a GPU: nvcc cross-compiles."""
    flags = list(BASE_FLAGS) + list(extra_flags)
    h = hashlib.sha256((source + "\0" + " ".join(ARCH_FLAGS + flags)).encode()).hexdigest()
    base = os.path.join(cache_dir(), f"{name}-{h[:16]}")
    with _lock:
        if os.path.exists(base + ".cubin") and os.path.exists(base + ".json"):
            with open(base + ".json") as f:
                return Manifest(**json.load(f))
        with tempfile.TemporaryDirectory() as td:
            src = os.path.join(td, name + ".cu")
            with open(src, "w") as f:
                f.write(source)
            tmp_out = os.path.join(td, name + ".cubin")
            cmd = [nvcc_path(), "-cubin", *ARCH_FLAGS, *flags, "-Xptxas", "-v", "-o", tmp_out, src]
            p = subprocess.run(cmd, capture_output=True, text=True)
            if p.returncode != 0:
                raise RuntimeError(f"nvcc failed for JIT kernel '{name}':\n{p.stderr[-4000:]}")
            entries = re.findall(r'extern\s+"C"\s+__global__\s+void\s+(?:__launch_bounds__\([^)]*\)\s*)?(\w+)', source)
            man = Manifest(name, entries, "sm_100a", flags, h, os.path.basename(base + ".cubin"), _parse_ptxas(p.stderr))
            _move(tmp_out, base + ".cubin")
            with open(base + ".json.tmp", "w") as f:
                json.dump(man.to_json(), f, indent=1)
            os.replace(base + ".json.tmp", base + ".json")
            return man


def _move(src: str, dst: str) -> None:
    import shutil

    shutil.copyfile(src, dst + ".tmp")
    os.replace(dst + ".tmp", dst)


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver call failed with error {int(err)} ({err})")
    return res[1] if len(res) == 2 else res[1:]


class JitModule:
    """A loaded cubin.  ``launch(entry, grid, block, args, arg_types)`` enqueues on PyTorch's current stream."""

    def __init__(self, manifest: Manifest):
        import torch
        from cuda.bindings import driver

        self.manifest, self.driver = manifest, driver
        torch.cuda.current_stream()          # makes sure PyTorch's primary context exists and is current on this thread
        with open(os.path.join(cache_dir(), manifest.cubin), "rb") as f:
            self._image = f.read()
        self.module = _check(driver.cuModuleLoadData(self._image))
        self.functions: Dict[str, Any] = {}

    def function(self, entry: str):
        fn = self.functions.get(entry)
        if fn is None:
            fn = self.functions[entry] = _check(self.driver.cuModuleGetFunction(self.module, entry.encode()))
        return fn

    def launch(self, entry: str, grid: Tuple[int, int, int], block: Tuple[int, int, int], args: Sequence[Any], arg_types: Sequence[Any], shared_bytes: int = 0) -> None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
        _check(self.driver.cuLaunchKernel(self.function(entry), *grid, *block, shared_bytes, stream, (tuple(args), tuple(arg_types)), 0))


_modules: Dict[Any, JitModule] = {}


def load(name: str, source: str, extra_flags: Sequence[str] = ()) -> JitModule:
    import torch

    man = compile_cubin(name, source, extra_flags)
    key = (man.source_sha256, torch.cuda.current_device())      # a module belongs to the context (device) it was loaded into
    m = _modules.get(key)
    if m is None:
        m = _modules[key] = JitModule(man)
    return m


# ------------------------------------------------------------------------------------------------------- element-wise generator

_PRELUDE = r"""
#include <cuda_bf16.h>
#include <stdint.h>
template <typename T> struct Vec;
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* t = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 v = __bfloat1622float2(t[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
        uint4 raw;
        __nv_bfloat162* t = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) t[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};
template <> struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* f) { const float4 v = *reinterpret_cast<const float4*>(p); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
    static __device__ __forceinline__ void store(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
"""


def _kernel(entry: str, ctype: str, ins: Sequence[str], outs: Sequence[str], body: str, consts: Sequence[str]) -> str:
    params = ", ".join([f"const {ctype}* __restrict__ p_{n}" for n in ins] + [f"{ctype}* __restrict__ p_{n}" for n in outs] + [f"float {c}" for c in consts] + ["size_t n"])
    loads = "\n".join(f"        float v_{n}[V::N]; V::load(p_{n} + i, v_{n});" for n in ins)
    decl = "\n".join(f"        float v_{n}[V::N];" for n in outs)
    bind_in = " ".join(f"const float {n} = v_{n}[k];" for n in ins)
    bind_out = " ".join(f"float {n};" for n in outs)
    write = " ".join(f"v_{n}[k] = {n};" for n in outs)
    stores = "\n".join(f"        V::store(p_{n} + i, v_{n});" for n in outs)
    return f"""
extern "C" __global__ void __launch_bounds__(256) {entry}({params}) {{
    using V = Vec<{ctype}>;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * V::N;
    for (size_t i = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * V::N; i < n; i += stride) {{
{loads}
{decl}
#pragma unroll
        for (int k = 0; k < V::N; ++k) {{
            {bind_in} {bind_out}
            {body}
            {write}
        }}
{stores}
    }}
}}
"""


class ElementwiseOp:
    """``ElementwiseOp("relu2", ("x",), "y = x > 0.f ? x * x : 0.f;", {"x": "dx = x > 0.f ? 2.f * x * dy : 0.f;"})``.

    ``forward`` assigns ``y`` from the inputs; each ``backward[name]`` assigns ``d<name>`` from the inputs and ``dy``.  ``consts`` are
    float scalars passed at call time (e.g. a soft-cap value).  Tensors must be contiguous, of one dtype (bf16 or fp32), with a number
    of elements that is a multiple of the vector width; anything else takes the PyTorch fallback given as ``reference``."""

    def __init__(self, name: str, inputs: Sequence[str], forward: str, backward: Dict[str, str], consts: Sequence[str] = (), reference=None):
        self.name, self.inputs, self.forward, self.backward, self.consts, self.reference = name, tuple(inputs), forward, dict(backward), tuple(consts), reference
        self._fn = None

    def source(self) -> str:
        src = _PRELUDE
        for ctype, tag in (("__nv_bfloat16", "bf16"), ("float", "f32")):
            src += _kernel(f"{self.name}_fwd_{tag}", ctype, self.inputs, ("y",), self.forward, self.consts)
            body = "\n            ".join(self.backward[n] for n in self.inputs if n in self.backward)
            src += _kernel(f"{self.name}_bwd_{tag}", ctype, self.inputs + ("dy",), tuple("d" + n for n in self.inputs if n in self.backward), body, self.consts)
        return src

    def compile(self) -> Manifest:
        return compile_cubin("ew_" + self.name, self.source())

    def _launch(self, entry: str, tensors, consts, n: int, width: int) -> None:
        mod = load("ew_" + self.name, self.source())
        blocks = max(1, min((n // width + 255) // 256, 148 * 8))
        args = [t.data_ptr() for t in tensors] + [float(c) for c in consts] + [n]
        types = [ctypes.c_void_p] * len(tensors) + [ctypes.c_float] * len(consts) + [ctypes.c_size_t]
        mod.launch(entry, (blocks, 1, 1), (256, 1, 1), args, types)

    def supported(self, tensors) -> bool:
        import torch

        t0 = tensors[0]
        width = 8 if t0.dtype == torch.bfloat16 else 4
        return (t0.is_cuda and t0.dtype in (torch.bfloat16, torch.float32) and t0.numel() % width == 0 and t0.numel() > 0
                and all(t.is_cuda and t.dtype == t0.dtype and t.shape == t0.shape for t in tensors))

    def __call__(self, *tensors, **consts):
        import torch

        cvals = [consts[c] for c in self.consts]
        if not self.supported(tensors):
            if self.reference is None:
                raise RuntimeError(f"JIT element-wise op '{self.name}' needs equal-shaped contiguous CUDA bf16 / fp32 tensors")
            return self.reference(*tensors, **consts)
        if self._fn is None:
            op = self

            class Fn(torch.autograd.Function):
                @staticmethod
                def forward(ctx, cv, *xs):
                    xs = tuple(x.contiguous() for x in xs)
                    tag, width = ("bf16", 8) if xs[0].dtype == torch.bfloat16 else ("f32", 4)
                    y = torch.empty_like(xs[0])
                    op._launch(f"{op.name}_fwd_{tag}", list(xs) + [y], cv, y.numel(), width)
                    ctx.save_for_backward(*xs)
                    ctx.cv = cv
                    return y

                @staticmethod
                def backward(ctx, dy):
                    xs = ctx.saved_tensors
                    tag, width = ("bf16", 8) if xs[0].dtype == torch.bfloat16 else ("f32", 4)
                    wanted = [n for n in op.inputs if n in op.backward]
                    grads = {n: torch.empty_like(xs[0]) for n in wanted}
                    op._launch(f"{op.name}_bwd_{tag}", list(xs) + [dy.contiguous()] + [grads[n] for n in wanted], ctx.cv, xs[0].numel(), width)
                    return (None,) + tuple(grads.get(n) for n in op.inputs)

            self._fn = Fn
        return self._fn.apply(cvals, *tensors)


# Ops used by the model families (runtime/torch_fns.py)
def _relu2_ref(x):
    import torch.nn.functional as F

    return F.relu(x).square()


def _softcap_ref(x, cap):
    import torch

    return torch.tanh(x.float() / cap).mul(cap).to(x.dtype)


def _geglu_ref(g, u):
    import torch.nn.functional as F

    return F.gelu(g.float(), approximate="tanh").to(g.dtype) * u


RELU2 = ElementwiseOp("relu2", ("x",), "y = x > 0.f ? x * x : 0.f;", {"x": "dx = x > 0.f ? 2.f * x * dy : 0.f;"}, reference=_relu2_ref)
SOFTCAP = ElementwiseOp("softcap", ("x",), "y = cap * tanhf(x / cap);", {"x": "{ const float t = tanhf(x / cap); dx = dy * (1.f - t * t); }"}, consts=("cap",),
                        reference=_softcap_ref)
GEGLU_TANH = ElementwiseOp(
    "geglu_tanh", ("g", "u"),
    "{ const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g); y = 0.5f * g * (1.f + tanhf(c)) * u; }",
    {"g": "{ const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g); const float t = tanhf(c);"
          " dg = dy * u * (0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * g * g)); }",
     "u": "{ const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g); du = dy * 0.5f * g * (1.f + tanhf(c)); }"}, reference=_geglu_ref)
ALL_OPS = (RELU2, SOFTCAP, GEGLU_TANH)


def precompile_all() -> List[Manifest]:
    """Compile every built-in JIT op into the cache (called by the build entry point, so the cubins travel with the tree)."""
    return [op.compile() for op in ALL_OPS]
