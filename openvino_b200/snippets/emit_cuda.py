"""CUDA emitter of a snippet: linear IR -> one sm_100a kernel, built with nvcc and kept in a cache directory.

Two shapes of kernel come out of one linear IR:

* no reduction: a flat element-wise kernel. A thread handles ``VEC`` neighbouring columns of one row with 16-byte
  loads and stores (8 values of a 16-bit type, 4 of fp32) when every input is contiguous or broadcast along the row,
  pointers and row strides are 16-byte aligned and ``cols % VEC == 0``; the scalar instance of the same body serves
  everything else;
* with reductions: one CTA per row (grid-stride over rows); every stage of the loop structure is one pass of the CTA
  over the row, reductions finish with a warp-shuffle + shared-memory block reduction, per-row values live in
  registers between the passes.

All arithmetic is fp32; loads widen, stores narrow. The text depends only on the structure of the snippet (operation
sequence, attributes, element types, broadcast kinds), so equal layers of a network share one compiled kernel: the
cache key is the hash of the text. Role of the reference's generator / emitters
(src/common/snippets/src/generator.cpp, src/plugins/intel_cpu/src/emitters/snippets/x64/jit_kernel_emitter.cpp).
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import threading
from pathlib import Path
from typing import Dict, List, Sequence

from .lowered import COL, FULL, LinearIR
from .op_table import OPS, REDUCTIONS, _f

_CTYPE = {"f32": "float", "f16": "__half", "bf16": "__nv_bfloat16", "boolean": "unsigned char", "u8": "unsigned char"}
_ESIZE = {"f32": 4, "f16": 2, "bf16": 2, "boolean": 1, "u8": 1}
MAX_IO = 12
KEPT_ITERS = (1, 2, 4)

_PRELUDE = r"""
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <math.h>
struct Args { const void* in[%(max_io)d]; void* out[%(max_io)d]; long long rs[%(max_io)d]; long long cs[%(max_io)d]; long long rows; long long cols; };
__device__ __forceinline__ float tanh_fast(float x) { float y; asm("tanh.approx.f32 %%0, %%1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float widen(float v) { return v; }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float widen(unsigned char v) { return v ? 1.0f : 0.0f; }
__device__ __forceinline__ void narrow(float& d, float v) { d = v; }
__device__ __forceinline__ void narrow(__half& d, float v) { d = __float2half_rn(v); }
__device__ __forceinline__ void narrow(__nv_bfloat16& d, float v) { d = __float2bfloat16_rn(v); }
__device__ __forceinline__ void narrow(unsigned char& d, float v) { d = v != 0.0f ? 1 : 0; }
template <int BYTES>
__device__ __forceinline__ void copy_bytes(void* d, const void* s) {
    if constexpr (BYTES %% 16 == 0) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
    } else if constexpr (BYTES == 8) {
        *reinterpret_cast<uint2*>(d) = *reinterpret_cast<const uint2*>(s);
    } else if constexpr (BYTES == 4) {
        *reinterpret_cast<unsigned*>(d) = *reinterpret_cast<const unsigned*>(s);
    } else {
#pragma unroll
        for (int i = 0; i < BYTES; ++i) reinterpret_cast<unsigned char*>(d)[i] = reinterpret_cast<const unsigned char*>(s)[i];
    }
}
// conversions of a whole vector: two values per instruction for the 16-bit types
template <class T, int VEC>
__device__ __forceinline__ void widen_all(const T* src, float* dst) {
    if constexpr (sizeof(T) == 2 && VEC %% 2 == 0) {
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            float2 f;
            if constexpr (sizeof(T) == 2 && __is_same(T, __half)) f = __half22float2(reinterpret_cast<const __half2*>(src)[i]);
            else f = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[i]);
            dst[2 * i] = f.x;
            dst[2 * i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[i] = widen(src[i]);
    }
}
template <class T, int VEC>
__device__ __forceinline__ void narrow_all(T* dst, const float* src) {
    if constexpr (sizeof(T) == 2 && VEC %% 2 == 0) {
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
            if constexpr (__is_same(T, __half)) reinterpret_cast<__half2*>(dst)[i] = __floats2half2_rn(src[2 * i], src[2 * i + 1]);
            else reinterpret_cast<__nv_bfloat162*>(dst)[i] = __floats2bfloat162_rn(src[2 * i], src[2 * i + 1]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) narrow(dst[i], src[i]);
    }
}
// VEC values of one input for columns c .. c+VEC-1 of row r: one 16-byte (or narrower) load when the input runs along
// the row, one scalar load repeated when it is constant along the row
template <class T, int VEC>
__device__ __forceinline__ void load_vec(const void* base, long long rs, long long cs, long long r, long long c, float* dst) {
    const T* p = reinterpret_cast<const T*>(base) + r * rs;
    if (cs == 0) {
        const float v = widen(p[0]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[i] = v;
    } else if constexpr (VEC == 1) {
        dst[0] = widen(p[c * cs]);
    } else {
        alignas(16) T tmp[VEC];
        copy_bytes<VEC * (int)sizeof(T)>(tmp, p + c);
        widen_all<T, VEC>(tmp, dst);
    }
}
template <class T, int VEC>
__device__ __forceinline__ void store_vec(void* base, long long r, long long cols, long long c, const float* src) {
    T* p = reinterpret_cast<T*>(base) + r * cols + c;
    if constexpr (VEC == 1) {
        narrow(p[0], src[0]);
    } else {
        alignas(16) T tmp[VEC];
        narrow_all<T, VEC>(tmp, src);
        copy_bytes<VEC * (int)sizeof(T)>(p, tmp);
    }
}
__device__ __forceinline__ float block_sum(float v, float* sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();                         // the buffer may still be read from the reduction before
    if ((threadIdx.x & 31) == 0) sm[w] = v;
    __syncthreads();
    v = 0.0f;
    for (int i = 0; i < nw; ++i) v += sm[i];          // every thread sums the same values in the same order
    return v;
}
__device__ __forceinline__ float block_max(float v, float* sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sm[w] = v;
    __syncthreads();
    v = -INFINITY;
    for (int i = 0; i < nw; ++i) v = fmaxf(v, sm[i]);
    return v;
}
"""


def _name(lir: LinearIR, lp, i: int, lane: str) -> str:
    e = lir.exprs[i]
    if e.domain == COL:
        return "c%d" % i
    return "r%d[%s]" % (lp.regs[i], lane)


def _col_stmt(lir: LinearIR, i: int) -> str:
    """Statement computing a per-row value (declared at row scope)."""
    e = lir.exprs[i]
    if e.kind == "scalar":
        return "const float c%d = %s;" % (i, _f(e.value))
    if e.kind == "inv_cols":
        return "const float c%d = 1.0f / (float)a.cols;" % i
    if e.kind == "param":
        t = _CTYPE[lir.in_types[e.index]]
        return "const float c%d = widen(reinterpret_cast<const %s*>(a.in[%d])[r * a.rs[%d]]);" % (i, t, e.index, e.index)
    return "const float c%d = %s;" % (i, OPS[e.op].cuda(e.attrs, *["c%d" % a for a in e.args]))


def _loop_body(lir: LinearIR, lp, indent: str, kept: bool = False) -> List[str]:
    """Statements of one pass for VEC columns starting at c (registers are float[VEC] arrays). In ``kept`` mode values
    of earlier passes are read back from the per-thread arrays k<id>[it] and values that later passes need are saved."""
    out = []
    nregs = 1 + max(lp.regs.values()) if lp.regs else 0
    for k in range(nregs):
        out.append("%sfloat r%d[VEC];" % (indent, k))
    for i in lp.body:
        e = lir.exprs[i]
        if kept and i in lp.readback:
            out.append("%s_Pragma(\"unroll\") for (int i = 0; i < VEC; ++i) r%d[i] = k%d[it][i];" % (indent, lp.regs[i], i))
            continue
        if e.kind == "param":
            t = _CTYPE[lir.in_types[e.index]]
            out.append("%sload_vec<%s, VEC>(a.in[%d], a.rs[%d], a.cs[%d], r, c, r%d);" % (indent, t, e.index, e.index, e.index, lp.regs[i]))
        else:
            args = [_name(lir, lp, a_, "i") for a_ in e.args]
            out.append("%s_Pragma(\"unroll\") for (int i = 0; i < VEC; ++i) r%d[i] = %s;" % (indent, lp.regs[i], OPS[e.op].cuda(e.attrs, *args)))
        if kept and i in lir.kept and e.stage == lp.index:
            out.append("%s_Pragma(\"unroll\") for (int i = 0; i < VEC; ++i) k%d[it][i] = r%d[i];" % (indent, i, lp.regs[i]))
    for rd in lp.reduces:
        src = lir.exprs[rd].args[0]
        comb = REDUCTIONS[lir.exprs[rd].op][2]("acc%d" % rd, _name(lir, lp, src, "i"))
        out.append("%s_Pragma(\"unroll\") for (int i = 0; i < VEC; ++i) acc%d = %s;" % (indent, rd, comb))
    for s in lp.stores:
        t = _CTYPE[lir.out_types[s.output]]
        out.append("%sstore_vec<%s, VEC>(a.out[%d], r, a.cols, c, r%d);" % (indent, t, s.output, lp.regs[s.value]))
    return out


def generate_source(lir: LinearIR) -> str:
    # all streams 16 bits wide: approximate transcendentals are below the resolution of what is stored
    fast = all(_ESIZE[t] <= 2 for t in lir.in_types + lir.out_types) and any(t in ("f16", "bf16") for t in lir.out_types)
    for e in lir.exprs:
        if e.kind == "op":
            e.attrs = dict(e.attrs, _fast=fast)
    src = [_PRELUDE % {"max_io": MAX_IO}]
    src.append("template <int VEC> __device__ __forceinline__ void run(const Args& a) {")
    if not lir.has_reduce:
        lp = lir.loops[0]
        src.append("    const long long per_row = a.cols / VEC, total = a.rows * per_row;")
        src.append("    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {")
        src.append("        const long long r = t / per_row, c = (t - r * per_row) * VEC;")
        for i in lp.prologue:
            src.append("        " + _col_stmt(lir, i))
        src.extend(_loop_body(lir, lp, "        "))
        src.append("    }")
    else:
        src.append("    __shared__ float sm[32];")
        src.append("    for (long long r = blockIdx.x; r < a.rows; r += gridDim.x) {")
        for lp in lir.loops:
            for i in lp.prologue:
                src.append("        " + _col_stmt(lir, i))
            for rd in lp.reduces:
                src.append("        float acc%d = %s;" % (rd, _f(REDUCTIONS[lir.exprs[rd].op][0])))
            if lp.body:
                src.append("        for (long long c = (long long)threadIdx.x * VEC; c < a.cols; c += (long long)blockDim.x * VEC) {")
                src.extend(_loop_body(lir, lp, "            "))
                src.append("        }")
            for rd in lp.reduces:
                src.append("        const float c%d = %s(acc%d, sm);" % (rd, REDUCTIONS[lir.exprs[rd].op][3], rd))
        for i in lir.epilogue:
            src.append("        " + _col_stmt(lir, i))
        for s in lir.stores:
            if s.domain == COL:
                t = _CTYPE[lir.out_types[s.output]]
                src.append("        if (threadIdx.x == 0) narrow(reinterpret_cast<%s*>(a.out[%d])[r], c%d);" % (t, s.output, s.value))
        src.append("    }")
    src.append("}")
    use_kept = bool(lir.has_reduce and lir.kept and lir.loops_kept)
    if use_kept:
        # the same passes with the reused values held in registers: ITERS iterations of the CTA cover a row
        src.append("template <int VEC, int ITERS> __device__ __forceinline__ void run_kept(const Args& a) {")
        src.append("    __shared__ float sm[32];")
        src.append("    for (long long r = blockIdx.x; r < a.rows; r += gridDim.x) {")
        for i in lir.kept:
            src.append("        float k%d[ITERS][VEC];" % i)
        for lp in lir.loops_kept:
            for i in lp.prologue:
                src.append("        " + _col_stmt(lir, i))
            for rd in lp.reduces:
                src.append("        float acc%d = %s;" % (rd, _f(REDUCTIONS[lir.exprs[rd].op][0])))
            if lp.body:
                src.append("        _Pragma(\"unroll\") for (int it = 0; it < ITERS; ++it) {")
                src.append("            const long long c = ((long long)it * blockDim.x + threadIdx.x) * VEC;")
                src.append("            if (c < a.cols) {")
                src.extend(_loop_body(lir, lp, "                ", kept=True))
                src.append("            }")
                src.append("        }")
            for rd in lp.reduces:
                src.append("        const float c%d = %s(acc%d, sm);" % (rd, REDUCTIONS[lir.exprs[rd].op][3], rd))
        for i in lir.epilogue:
            src.append("        " + _col_stmt(lir, i))
        for s_ in lir.stores:
            if s_.domain == COL:
                t = _CTYPE[lir.out_types[s_.output]]
                src.append("        if (threadIdx.x == 0) narrow(reinterpret_cast<%s*>(a.out[%d])[r], c%d);" % (t, s_.output, s_.value))
        src.append("    }")
        src.append("}")
        for it in KEPT_ITERS:
            src.append("extern \"C\" __global__ void __launch_bounds__(256) snippet_vec_k%d(Args a) { run_kept<%d, %d>(a); }" % (it, vec_width(lir), it))
    src.append("extern \"C\" __global__ void __launch_bounds__(256) snippet_vec(Args a) { run<%d>(a); }" % vec_width(lir))
    src.append("extern \"C\" __global__ void __launch_bounds__(256) snippet_scalar(Args a) { run<1>(a); }")
    src.append("extern \"C\" int snippet_launch(const Args* a, int variant, int grid, int block, void* stream) {")
    src.append("    // variant: 0 scalar, 1 vector, 2 + n vector with kept values and KEPT_ITERS[n] iterations per row")
    src.append("    switch (variant) {")
    src.append("        case 0: snippet_scalar<<<grid, block, 0, (cudaStream_t)stream>>>(*a); break;")
    src.append("        case 1: snippet_vec<<<grid, block, 0, (cudaStream_t)stream>>>(*a); break;")
    if use_kept:
        for n_, it in enumerate(KEPT_ITERS):
            src.append("        case %d: snippet_vec_k%d<<<grid, block, 0, (cudaStream_t)stream>>>(*a); break;" % (2 + n_, it))
    src.append("        default: return (int)cudaErrorInvalidValue;")
    src.append("    }")
    src.append("    return (int)cudaGetLastError();")
    src.append("}")
    return "\n".join(src) + "\n"


def vec_width(lir: LinearIR) -> int:
    """Columns per thread of the vector instance: 16 bytes of the widest 16-bit stream, 4 values when fp32 is involved."""
    sizes = [_ESIZE[t] for t in lir.in_types + lir.out_types]
    return 4 if 4 in sizes else 8


def cache_dir() -> Path:
    d = Path(os.environ.get("OVB_SNIPPETS_CACHE") or (Path.home() / ".cache" / "openvino_b200" / "snippets"))
    d.mkdir(parents=True, exist_ok=True)
    return d


class _ArgsStruct(ctypes.Structure):
    _fields_ = [("inp", ctypes.c_void_p * MAX_IO), ("out", ctypes.c_void_p * MAX_IO), ("rs", ctypes.c_longlong * MAX_IO), ("cs", ctypes.c_longlong * MAX_IO),
                ("rows", ctypes.c_longlong), ("cols", ctypes.c_longlong)]


_LOADED: Dict[str, "CudaKernel"] = {}
_BUILD_LOCK = threading.Lock()


class CudaKernel:
    """A compiled snippet: ``launch`` takes device pointers, strides in elements and the 2-D extent."""

    def __init__(self, lir: LinearIR):
        self.lir = lir
        self.vec = vec_width(lir)
        self.source = generate_source(lir)
        self.key = hashlib.sha256(self.source.encode()).hexdigest()[:24]
        self._lib = None

    @staticmethod
    def get(lir: LinearIR) -> "CudaKernel":
        k = CudaKernel(lir)
        with _BUILD_LOCK:
            have = _LOADED.get(k.key)
            if have is not None:
                return have
            k._build()
            _LOADED[k.key] = k
        return k

    def _build(self) -> None:
        from ..build import _nvcc
        d = cache_dir()
        so, cu = d / ("snippet_%s.so" % self.key), d / ("snippet_%s.cu" % self.key)
        if not so.exists():
            cu.write_text(self.source)
            tmp = d / ("snippet_%s.%d.tmp.so" % (self.key, os.getpid()))
            cmd = [_nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-shared", "-Xcompiler", "-fPIC", "-cudart", "static",
                   "-o", str(tmp), str(cu)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError("snippet kernel failed to build:\n%s\n%s" % (res.stderr[-2000:], self.source))
            os.replace(tmp, so)          # atomic: other processes either see the finished file or none
        self._lib = ctypes.CDLL(str(so))
        self._lib.snippet_launch.argtypes = [ctypes.POINTER(_ArgsStruct), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        self._lib.snippet_launch.restype = ctypes.c_int

    def launch(self, in_ptrs: Sequence[int], in_rs: Sequence[int], in_cs: Sequence[int], out_ptrs: Sequence[int], rows: int, cols: int, stream: int, sm_count: int = 148) -> None:
        a = _ArgsStruct()
        for i, (p, rs, cs) in enumerate(zip(in_ptrs, in_rs, in_cs)):
            a.inp[i], a.rs[i], a.cs[i] = p, rs, cs
        for i, p in enumerate(out_ptrs):
            a.out[i] = p
        a.rows, a.cols = rows, cols
        v = self.vec
        esz_in = [_ESIZE[t] for t in self.lir.in_types]
        vec_ok = cols % v == 0 and all(p % 16 == 0 for p in out_ptrs) and all(
            cs == 0 or (cs == 1 and p % 16 == 0 and (rs * e) % 16 == 0) for p, rs, cs, e in zip(in_ptrs, in_rs, in_cs, esz_in)) and \
            all((cols * _ESIZE[t]) % 16 == 0 for t in self.lir.out_types)
        width = v if vec_ok else 1
        variant = 1 if vec_ok else 0
        if self.lir.has_reduce:
            block = 256 if cols >= 256 * width else max(32, ((cols // width + 31) // 32) * 32)
            grid = max(1, min(rows, sm_count * 8))
            if vec_ok and self.lir.kept and self.lir.loops_kept:
                need = -(-cols // (block * width))            # iterations of the CTA over one row
                for n_, it in enumerate(KEPT_ITERS):
                    if it >= need:
                        variant = 2 + n_
                        break
        else:
            block = 256
            grid = max(1, min((rows * (cols // width) + block - 1) // block, sm_count * 16))
        rc = self._lib.snippet_launch(ctypes.byref(a), variant, int(grid), int(block), ctypes.c_void_p(stream))
        if rc != 0:
            raise RuntimeError("snippet kernel launch failed with CUDA error %d" % rc)
