"""ctypes front-end of ``libovb_cuda.so`` (the hand-written sm_100a kernel library).

Tensors are ``torch.Tensor`` objects used as typed device buffers: torch supplies the
allocator and the CUDA stream, every computation below runs in this repository's own kernels.
There is no eager/PyTorch fallback: if the library cannot be loaded, calls raise.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import threading
from pathlib import Path
from typing import Optional

import torch

_PKG = Path(__file__).resolve().parent.parent
# OVB_CUDA_LIB names another build of the kernel library (a build with different compile-time tuning switches, say)
_LIB_PATH = Path(os.environ["OVB_CUDA_LIB"]) if os.environ.get("OVB_CUDA_LIB") else _PKG / "lib" / "libovb_cuda.so"

W_BF16, W_U4, W_U8, W_F16, W_F8 = 0, 1, 2, 3, 4
ACT_NONE, ACT_GELU_ERF, ACT_RELU, ACT_SILU, ACT_SWIGLU, ACT_GELU_TANH = 0, 1, 2, 3, 4, 5

STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "bad argument seen on device",
                4: "local flag wait timed out", 5: "index out of range (debug build; the access was skipped)"}


class GemmArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p), ("bias", C.c_void_p), ("residual", C.c_void_p),
        ("scales", C.c_void_p), ("zps", C.c_void_p), ("ws", C.c_void_p), ("counters", C.c_void_p),
        ("ws_bytes", C.c_int64),
        ("T", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("ldx", C.c_int), ("ldo", C.c_int), ("ldr", C.c_int),
        ("group_size", C.c_int), ("wmode", C.c_int), ("act", C.c_int), ("out_f32", C.c_int),
        ("splits", C.c_int), ("block_t", C.c_int), ("w_tiled", C.c_int),
        ("comm", C.c_void_p), ("w_kb_stride", C.c_int),
        ("group_offsets", C.c_void_p), ("num_groups", C.c_int), ("group_mode", C.c_int),
    ]


class PaArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("past_lens", C.c_void_p), ("subsequence_begins", C.c_void_p), ("block_indices", C.c_void_p),
        ("block_indices_begins", C.c_void_p), ("scratch", C.c_void_p),
        ("B", C.c_int), ("T", C.c_int), ("Hq", C.c_int), ("Hkv", C.c_int), ("D", C.c_int),
        ("ldq", C.c_int), ("block_size", C.c_int), ("max_context_len", C.c_int), ("max_q_len", C.c_int),
        ("sliding_window", C.c_int), ("scale", C.c_float),
        ("kv_u8", C.c_int), ("k_meta", C.c_void_p), ("v_meta", C.c_void_p),
    ]


_lib = None
_lock = threading.Lock()


class KernelLibraryError(RuntimeError):
    pass


def lib():
    """Load (building first if the sources are newer) and return the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists() or os.environ.get("OVB_REBUILD") == "1":
            from .. import build as _build
            _build.build_cuda()
        if not _LIB_PATH.exists():
            raise KernelLibraryError("libovb_cuda.so is missing and could not be built: %s" % _LIB_PATH)
        l = C.CDLL(str(_LIB_PATH))
        l.ovb_last_error.restype = C.c_char_p
        l.ovb_status_ptr.restype = C.c_void_p
        l.ovb_gemm_ws_bytes.restype = C.c_int64
        l.ovb_pa_scratch_bytes.restype = C.c_int64
        l.ovb_gemm.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        l.ovb_paged_attention.argtypes = [C.POINTER(PaArgs), C.c_void_p]
        l.ovb_status_read.argtypes = [C.c_void_p]
        _lib = l
        if os.environ.get("OVB_CC_COLLECT"):       # conditional compilation, analysing stage: statistics at shutdown
            from ..utils import cc as _cc   # noqa: F401
    return _lib


def available() -> bool:
    return torch.cuda.is_available()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelLibraryError("%s failed (%d): %s" % (what, rc, lib().ovb_last_error().decode()))


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def read_status() -> int:
    """Device status word: 0 = ok. Synchronises the current stream and clears the word."""
    return int(lib().ovb_status_read(C.c_void_p(_stream())))


def set_peer_spin_limit(polls: int) -> int:
    """Polls (about 0.25 us apart) a kernel waits for a peer GPU before it gives up with status 2; 0 = default (about 1 s).
    Returns the previous value."""
    fn = lib().ovb_set_peer_spin_limit
    fn.restype = C.c_uint
    return int(fn(C.c_uint(int(polls))))


def debug_bounds_enabled() -> bool:
    """True when the loaded kernel library is the bounds-checking debug build (``OVB_CUDA_LIB=.../libovb_cuda_dbg.so``)."""
    return bool(lib().ovb_debug_bounds_enabled())


def debug_set_limits(kv_blocks: int = 0, vocab: int = 0) -> None:
    """Debug build: the limits that block ids / cache slots / token ids read by kernels are checked against (0 = unknown)."""
    _check(lib().ovb_debug_set_limits(C.c_int(int(kv_blocks)), C.c_int(int(vocab))), "ovb_debug_set_limits")


def check_status(what: str = "kernel") -> None:
    s = read_status()
    if s != 0:
        raise KernelLibraryError("%s reported device status %d (%s)" % (what, s, STATUS_NAMES.get(s, "?")))


# ------------------------------------------------------------------------------------------ workspace
class Workspace:
    """Scratch memory shared by the kernels of one device/stream: split-K partials + counters,
    decode-attention split-KV partials. Allocated once, reused by every call (calls that overlap on
    the GPU must use different workspaces)."""

    def __init__(self, device, gemm_bytes: int = 64 << 20, pa_bytes: int = 64 << 20):
        self.device = device
        self.gemm_ws = torch.empty(gemm_bytes // 4, dtype=torch.float32, device=device)
        self.counters = torch.zeros(int(lib().ovb_gemm_num_counters()), dtype=torch.int32, device=device)
        self.pa_scratch = torch.empty(pa_bytes // 4, dtype=torch.float32, device=device)


_default_ws: dict = {}


def default_workspace(device) -> Workspace:
    key = torch.device(device).index or 0
    if key not in _default_ws:
        _default_ws[key] = Workspace(torch.device("cuda", key))
    return _default_ws[key]


# ------------------------------------------------------------------------------------------ weights
class PackedWeight:
    """A FullyConnected weight in the layout the GEMM kernel reads.

    mode W_BF16/W_F16: ``w`` is [N, K] 16-bit (optionally tile-packed).  mode W_U4: ``w`` is the tile-packed
    nibble stream, ``scales`` is the [K/group, N, 2] bf16 table of (scale, 16 + zero_point) pairs.
    mode W_U8: ``w`` [N, K] u8, the pairs hold the zero point itself.
    """

    def __init__(self, mode, w, N, K, scales=None, zps=None, group_size=0, bias=None, tiled=False, kb_stride=0):
        self.mode, self.w, self.N, self.K = mode, w, N, K
        self.scales, self.zps, self.group_size, self.bias = scales, zps, group_size, bias
        self.tiled = tiled
        self.kb_stride = kb_stride     # > 0: this weight is a window into a larger tile-packed one

    def window(self, n0: int, n: int, k0: int = 0, k: Optional[int] = None) -> "PackedWeight":
        """Rows [n0, n0 + n) and columns [k0, k0 + k) of a tile-packed 16-bit weight as a weight of its own (no copy):
        one expert of a stack of experts. Offsets and sizes are multiples of the tile (128 rows, 64 columns)."""
        k = self.K - k0 if k is None else k
        assert self.tiled and self.mode in (W_BF16, W_F16) and self.bias is None
        assert n0 % 128 == 0 and n % 128 == 0 and k0 % 64 == 0 and k % 64 == 0 and n0 + n <= self.N and k0 + k <= self.K
        stride = self.kb_stride or self.K // 64
        first_chunk = (n0 // 128) * stride + k0 // 64
        return PackedWeight(self.mode, self.w[first_chunk * 8192:], n, k, tiled=True, kb_stride=stride)

    @staticmethod
    def from_dense(w: torch.Tensor, bias=None, tiled: bool = True) -> "PackedWeight":
        """16-bit [N, K] weight. ``tiled`` re-packs it into tile-contiguous, pre-swizzled 16 KB chunks (one
        bulk copy per k-block); K must then be a multiple of 64, otherwise the row-major form is kept."""
        assert w.dim() == 2 and w.dtype in (torch.bfloat16, torch.float16)
        mode = W_BF16 if w.dtype == torch.bfloat16 else W_F16
        N, Kd = w.shape
        w = w.contiguous()
        if tiled and Kd % 64 == 0:
            out = torch.empty(((N + 127) // 128) * 128 * Kd, dtype=w.dtype, device=w.device)
            _check(lib().ovb_pack_w16(C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int(N), C.c_int(Kd),
                                      C.c_void_p(_stream())), "ovb_pack_w16")
            return PackedWeight(mode, out, N, Kd, bias=bias, tiled=True)
        return PackedWeight(mode, w, N, Kd, bias=bias)

    @staticmethod
    def from_ir_u4(w_ir: torch.Tensor, scales_ir: torch.Tensor, zps_ir: Optional[torch.Tensor], N: int, K: int,
                   group_size: int, zp_is_u8: bool = False, bias=None) -> "PackedWeight":
        """w_ir: uint8 [N*K/2] LSB-first nibbles (IR layout); scales_ir fp16 [N, G]; zps_ir packed u4 [N*G/2]
        (or uint8 [N, G] when zp_is_u8) or None for the symmetric i4-style offset 8."""
        dev = w_ir.device
        G = K // group_size
        w_out = torch.empty(((N + 127) // 128) * (K // 64) * 4608, dtype=torch.uint8, device=dev)
        # the kernel copies the pairs of 128 rows at a time: keep 128 pairs of slack behind the table
        s_out = torch.zeros(G * N * 2 + 256, dtype=torch.bfloat16, device=dev)
        rc = lib().ovb_pack_u4(C.c_void_p(w_ir.data_ptr()), C.c_void_p(scales_ir.data_ptr()),
                               C.c_void_p(_ptr(zps_ir)), C.c_int(1 if zp_is_u8 else 0), C.c_void_p(w_out.data_ptr()),
                               C.c_void_p(s_out.data_ptr()), C.c_void_p(None), C.c_int(N), C.c_int(K),
                               C.c_int(group_size), C.c_void_p(_stream()))
        _check(rc, "ovb_pack_u4")
        return PackedWeight(W_U4, w_out, N, K, s_out, None, group_size, bias)

    @staticmethod
    def from_ir_u8(w_ir: torch.Tensor, scales_ir: torch.Tensor, zps_ir: Optional[torch.Tensor], N: int, K: int,
                   group_size: int, bias=None) -> "PackedWeight":
        G = K // group_size
        s = scales_ir.reshape(N, G).float().t().contiguous().to(torch.bfloat16)
        if zps_ir is None:
            z = torch.full((G, N), 128.0, dtype=torch.bfloat16, device=w_ir.device)
        else:
            z = zps_ir.reshape(N, G).float().t().contiguous().to(torch.bfloat16)
        sz = torch.stack([s, z], dim=-1).contiguous()      # [G, N, 2] pairs
        sz = torch.cat([sz.reshape(-1), torch.zeros(256, dtype=sz.dtype, device=sz.device)])   # slack for 128-row copies
        return PackedWeight(W_U8, w_ir.contiguous(), N, K, sz, None, group_size, bias)

    @staticmethod
    def from_f8_block(w8: torch.Tensor, block_scales: torch.Tensor, N: int, K: int, block: int = 128, bias=None) -> "PackedWeight":
        """fp8 e4m3 weight [N, K] (uint8 or float8 storage) with one fp32 scale per ``block`` x ``block`` tile
        (``block_scales`` [ceil(N/block), K/block]): dequantised weight = fp8 value * scale of its tile.
        The kernel reads the scales as a (k-group, row) table of bf16 values that already carry the 2^120 exponent
        shift of its byte-to-bf16 conversion."""
        assert block == 128 and K % block == 0
        w8 = w8.view(torch.uint8).reshape(N, K).contiguous()
        G = K // block
        s = block_scales.float().reshape(-1, G)                                     # [N/128, G]
        per_row = s.repeat_interleave(block, dim=0)[:N]                             # [N, G]
        scaled = (per_row.t().contiguous() * float(2.0 ** 120)).to(torch.bfloat16)  # [G, N]
        sz = torch.stack([scaled, torch.zeros_like(scaled)], dim=-1).contiguous()
        sz = torch.cat([sz.reshape(-1), torch.zeros(256, dtype=sz.dtype, device=sz.device)])   # slack for 128-row copies
        return PackedWeight(W_F8, w8, N, K, sz, None, block, bias)


# ------------------------------------------------------------------------------------------ ops
def gemm(x: torch.Tensor, w: PackedWeight, out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         act: int = ACT_NONE, out_f32: bool = False, ws: Optional[Workspace] = None, splits: int = 0,
         block_t: int = 0, comm=None) -> torch.Tensor:
    """out[T, N] = act(x[T, K] @ dequant(W)^T + bias) + residual  on the tcgen05 GEMM.

    ``comm`` (a ``parallel.comm.CommStruct``): sum the product over the tensor-parallel ranks inside the epilogue."""
    assert x.dim() == 2 and x.stride(1) == 1
    T, K = x.shape
    assert K == w.K, (K, w.K)
    if out is None:
        out = torch.empty((T, w.N // 2 if act == ACT_SWIGLU else w.N), dtype=torch.float32 if out_f32 else x.dtype, device=x.device)
    if ws is None:
        ws = default_workspace(x.device)
    a = GemmArgs()
    a.x, a.w, a.out = x.data_ptr(), w.w.data_ptr(), out.data_ptr()
    a.bias = _ptr(w.bias)
    a.residual = _ptr(residual)
    a.scales, a.zps = _ptr(w.scales), _ptr(w.zps)
    a.ws, a.counters, a.ws_bytes = ws.gemm_ws.data_ptr(), ws.counters.data_ptr(), ws.gemm_ws.numel() * 4
    a.T, a.N, a.K = T, w.N, K
    a.ldx, a.ldo = x.stride(0), out.stride(0)
    a.ldr = residual.stride(0) if residual is not None else 0
    a.group_size = w.group_size
    a.wmode, a.act, a.out_f32 = w.mode, act, 1 if out_f32 else 0
    a.splits, a.block_t = splits, block_t
    a.w_kb_stride = int(getattr(w, "kb_stride", 0) or 0)
    a.w_tiled = 1 if (w.tiled and w.mode in (W_BF16, W_F16)) else 0
    a.comm = C.addressof(comm) if comm is not None else None
    _check(lib().ovb_gemm(C.byref(a), C.c_void_p(_stream())), "ovb_gemm")
    return out


def rmsnorm(x, gamma, eps, residual=None, out=None, residual_out=None):
    rows, cols = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().ovb_rmsnorm(C.c_void_p(x.data_ptr()), C.c_void_p(_ptr(residual)), C.c_void_p(gamma.data_ptr()),
                             C.c_void_p(out.data_ptr()), C.c_void_p(_ptr(residual_out)), C.c_int(rows), C.c_int(cols),
                             C.c_float(eps), C.c_void_p(_stream())), "ovb_rmsnorm")
    return out


def selective_ssm(A, dt, Bm, x, Cm, state):
    """Selective state-space scan over fp32 tensors: A [H], dt [B, L, H], Bm / Cm [B, L, G, S], x [B, L, H, P], state [B, H, P, S].
    Returns (y [B, L, H, P], new state); ``state`` itself is left as it was."""
    B, L, H, P = x.shape
    G, S = Bm.shape[2], Bm.shape[3]
    args = [t.float().contiguous() for t in (A, dt, Bm, x, Cm)]
    new_state = state.float().contiguous().clone()
    y = torch.empty((B, L, H, P), dtype=torch.float32, device=x.device)
    _check(lib().ovb_selective_ssm(*(C.c_void_p(t.data_ptr()) for t in args), C.c_void_p(new_state.data_ptr()), C.c_void_p(y.data_ptr()),
                                   C.c_int(B), C.c_int(L), C.c_int(H), C.c_int(P), C.c_int(G), C.c_int(S), C.c_void_p(_stream())), "ovb_selective_ssm")
    return y, new_state


def gated_delta_rule(q, k, v, gate, beta, state):
    """Gated delta rule over fp32 tensors: q / k [B, L, Hq, Dk] (already scaled / normalised), v [B, L, Hv, Dv], gate / beta [B, L, Hv],
    state [B, Hv, Dk, Dv]. Returns (y [B, L, Hv, Dv], new state)."""
    B, L, Hq, Dk = q.shape
    Hv, Dv = v.shape[2], v.shape[3]
    args = [t.float().contiguous() for t in (q, k, v, gate, beta)]
    new_state = state.float().contiguous().clone()
    y = torch.empty((B, L, Hv, Dv), dtype=torch.float32, device=q.device)
    _check(lib().ovb_gated_delta_rule(*(C.c_void_p(t.data_ptr()) for t in args), C.c_void_p(new_state.data_ptr()), C.c_void_p(y.data_ptr()),
                                      C.c_int(B), C.c_int(L), C.c_int(Hq), C.c_int(Hv), C.c_int(Dk), C.c_int(Dv), C.c_void_p(_stream())), "ovb_gated_delta_rule")
    return y, new_state


def layernorm(x, gamma, beta, eps, residual=None, out=None):
    rows, cols = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().ovb_layernorm(C.c_void_p(x.data_ptr()), C.c_void_p(_ptr(residual)), C.c_void_p(gamma.data_ptr()),
                               C.c_void_p(beta.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int(rows), C.c_int(cols),
                               C.c_float(eps), C.c_int(1 if x.dtype == torch.float16 else 0), C.c_void_p(_stream())),
           "ovb_layernorm")
    return out


def silu_mul(gu, out=None, nrows: Optional[torch.Tensor] = None):
    """silu(gate) * up over [rows, 2F] -> [rows, F]; ``nrows`` (int32 device tensor) limits the rows without a host read."""
    rows, F2 = gu.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((rows, F), dtype=gu.dtype, device=gu.device)
    _check(lib().ovb_silu_mul_counted(C.c_void_p(gu.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int(rows), C.c_int(F),
                                      C.c_void_p(nrows.data_ptr() if nrows is not None else None), C.c_void_p(_stream())), "ovb_silu_mul")
    return out


def pick_block_t(T: int) -> int:
    """Row-tile height the GEMM picks for T rows (16 .. 256)."""
    for bt in (16, 32, 64, 128):
        if T <= bt:
            return bt
    return 256


def act_quant_fp8(x: torch.Tensor):
    """bf16 [rows, cols] -> (e4m3 bytes [rows, cols] uint8, fp32 scales [rows, cols / 128]); x ~ q * scale per group of 128."""
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.uint8, device=x.device)
    s = torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
    _check(lib().ovb_act_quant_fp8(C.c_void_p(x.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(s.data_ptr()), C.c_int(rows), C.c_int(cols),
                                   C.c_void_p(_stream())), "ovb_act_quant_fp8")
    return q, s


def kv_block_copy(k_cache: torch.Tensor, v_cache: torch.Tensor, src_blocks: torch.Tensor, dst_blocks: torch.Tensor) -> None:
    """Copy whole blocks (first dimension of the caches) src -> dst in both caches; int32 block lists on the device."""
    n = int(src_blocks.numel())
    block_bytes = k_cache[0].numel() * k_cache.element_size()
    _check(lib().ovb_kv_block_copy(C.c_void_p(k_cache.data_ptr()), C.c_void_p(v_cache.data_ptr()), C.c_void_p(src_blocks.data_ptr()),
                                   C.c_void_p(dst_blocks.data_ptr()), C.c_int(n), C.c_int64(block_bytes), C.c_void_p(_stream())), "ovb_kv_block_copy")


def lora_apply(x: torch.Tensor, a: "PackedWeight", b: "PackedWeight", y: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """y + alpha * (x @ A^T) @ B^T with both products on the tcgen05 GEMM (A [r, K], B [N, r] packed with ``from_dense``);
    the second GEMM adds ``y`` in its epilogue. Role of the reference's lora_{ref,opt}.cl kernels."""
    h = gemm(x, a)
    if alpha != 1.0:
        h = h * alpha
    return gemm(h, b, residual=y)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[F, K] gate and up projections -> [2F, K] in the row order of the fused SwiGLU epilogue (``ACT_SWIGLU``): every
    128-row tile holds 64 gate rows followed by the 64 up rows of the same channels. F must be a multiple of 64."""
    F, Kd = gate.shape
    assert up.shape == gate.shape and F % 64 == 0
    return torch.stack([gate.reshape(F // 64, 64, Kd), up.reshape(F // 64, 64, Kd)], dim=1).reshape(2 * F, Kd)


def wait_flag(flag: torch.Tensor, value: int, max_polls: int = 1 << 16, result: Optional[torch.Tensor] = None) -> None:
    """Queue a bounded device-side wait for ``flag[0] >= value`` (int32 tensor); a time-out shows in the status word."""
    _check(lib().ovb_comm_wait_flag(C.c_void_p(flag.data_ptr()), C.c_int(value), C.c_uint(max_polls), C.c_void_p(_ptr(result)),
                                    C.c_void_p(_stream())), "ovb_comm_wait_flag")


def sample_gumbel(logits: torch.Tensor, temperature: float, seed: int = 0, step: Optional[torch.Tensor] = None, vocab_offset: int = 0,
                  out: Optional[torch.Tensor] = None, out_max: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Temperature sampling by perturbed arg-max over bf16 ``logits`` [rows, V] (a vocabulary shard starting at
    ``vocab_offset``); returns local token indices (int32) and, in ``out_max``, the perturbed maxima."""
    rows, V = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib().ovb_sample_gumbel(C.c_void_p(logits.data_ptr()), C.c_int(logits.stride(0)), C.c_int(rows), C.c_int(V), C.c_int(vocab_offset),
                                   C.c_float(temperature), C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), C.c_void_p(_ptr(step)),
                                   C.c_void_p(out.data_ptr()), C.c_void_p(_ptr(out_max)), C.c_void_p(_stream())), "ovb_sample_gumbel")
    return out


def conv2d(x: torch.Tensor, w: "PackedWeight", kernel, strides, pads_begin, pads_end, dilations, act: int = ACT_NONE) -> torch.Tensor:
    """2-D convolution of a 16-bit NCHW tensor as im2col + tcgen05 GEMM; ``w`` packs the filters as [O, Kpad] with
    k = (c*kh + r)*kw + s (``pack_conv_weight``). Returns NCHW (a permuted view of the GEMM's [B*Ho*Wo, O] output)."""
    B, Cin, H, W = x.shape
    kh, kw = kernel
    Ho = (H + pads_begin[0] + pads_end[0] - dilations[0] * (kh - 1) - 1) // strides[0] + 1
    Wo = (W + pads_begin[1] + pads_end[1] - dilations[1] * (kw - 1) - 1) // strides[1] + 1
    x = x.contiguous()
    cols = torch.empty((B * Ho * Wo, w.K), dtype=x.dtype, device=x.device)
    _check(lib().ovb_im2col(C.c_void_p(x.data_ptr()), C.c_void_p(cols.data_ptr()), C.c_int(B), C.c_int(Cin), C.c_int(H), C.c_int(W),
                            C.c_int(kh), C.c_int(kw), C.c_int(strides[0]), C.c_int(strides[1]), C.c_int(pads_begin[0]), C.c_int(pads_begin[1]),
                            C.c_int(dilations[0]), C.c_int(dilations[1]), C.c_int(Ho), C.c_int(Wo), C.c_int(w.K), C.c_void_p(_stream())), "ovb_im2col")
    out = gemm(cols, w, act=act)
    return out.view(B, Ho, Wo, w.N).permute(0, 3, 1, 2)


def pack_conv_weight(w: torch.Tensor, bias=None) -> "PackedWeight":
    """[O, C, kh, kw] 16-bit filters -> GEMM weight [O, Kpad], Kpad = C*kh*kw rounded up to 64."""
    O = w.shape[0]
    flat = w.reshape(O, -1)
    Kd = flat.shape[1]
    Kpad = (Kd + 63) // 64 * 64
    if Kpad != Kd:
        flat = torch.nn.functional.pad(flat, (0, Kpad - Kd))
    return PackedWeight.from_dense(flat.contiguous(), bias=bias)


def sample(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0, seed: int = 0, step: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Draw one token per row of bf16 ``logits`` [rows, V]; ``step``: device int32 word mixed into the random stream."""
    rows, V = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(lib().ovb_sample(C.c_void_p(logits.data_ptr()), C.c_int(logits.stride(0)), C.c_int(rows), C.c_int(V), C.c_float(temperature),
                            C.c_int(top_k), C.c_float(top_p), C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF), C.c_void_p(_ptr(step)),
                            C.c_void_p(out.data_ptr()), C.c_void_p(_stream())), "ovb_sample")
    return out


def bump(counter: torch.Tensor) -> None:
    _check(lib().ovb_bump(C.c_void_p(counter.data_ptr()), C.c_void_p(_stream())), "ovb_bump")


def moe_route_topk(logits: torch.Tensor, k: int, out=None) -> torch.Tensor:
    """logits [T, E] fp32 -> dense routing weights [T, E] fp32 (softmax, top-k, renormalised)."""
    T, E = logits.shape
    if out is None:
        out = torch.empty((T, E), dtype=torch.float32, device=logits.device)
    _check(lib().ovb_moe_route_topk(C.c_void_p(logits.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int(T), C.c_int(E), C.c_int(k),
                                    C.c_void_p(_stream())), "ovb_moe_route_topk")
    return out


def moe_silu_mul_scale(gu: torch.Tensor, weights: torch.Tensor, F: int, nloc: int, e0: int, out=None) -> torch.Tensor:
    rows = gu.shape[0]
    E = weights.shape[1]
    if out is None:
        out = torch.empty((rows, nloc * F), dtype=gu.dtype, device=gu.device)
    _check(lib().ovb_moe_silu_mul_scale(C.c_void_p(gu.data_ptr()), C.c_void_p(weights.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int(rows),
                                        C.c_int(F), C.c_int(nloc), C.c_int(E), C.c_int(e0), C.c_void_p(_stream())), "ovb_moe_silu_mul_scale")
    return out


def moe_group(route: torch.Tensor, e0: int, nloc: int, idx: torch.Tensor, counts: torch.Tensor) -> None:
    """Token lists of the local experts e0 .. e0+nloc-1: idx [nloc, >=T] int32 (token order), counts [nloc] int32."""
    T, E = route.shape
    _check(lib().ovb_moe_group(C.c_void_p(route.data_ptr()), C.c_int(T), C.c_int(E), C.c_int(e0), C.c_int(nloc), C.c_void_p(idx.data_ptr()),
                               C.c_int(idx.stride(0)), C.c_void_p(counts.data_ptr()), C.c_void_p(_stream())), "ovb_moe_group")


def moe_positions(route: torch.Tensor, e0: int, nloc: int, pos: torch.Tensor, counts: torch.Tensor) -> None:
    """pos [T, nloc] int32: position of every token in the row list of each local expert (-1: not routed there); counts [nloc]."""
    T, E = route.shape
    _check(lib().ovb_moe_positions(C.c_void_p(route.data_ptr()), C.c_int(T), C.c_int(E), C.c_int(e0), C.c_int(nloc), C.c_void_p(pos.data_ptr()),
                                   C.c_void_p(counts.data_ptr()), C.c_void_p(_stream())), "ovb_moe_positions")


def moe_gather_sorted(x: torch.Tensor, pos: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor, xg: torch.Tensor) -> None:
    """Rows of ``x`` copied into ``xg`` sorted by expert; ``offsets`` [nloc + 1] receives the experts' row ranges."""
    T, H = x.shape
    _check(lib().ovb_moe_gather_sorted(C.c_void_p(x.data_ptr()), C.c_void_p(pos.data_ptr()), C.c_void_p(counts.data_ptr()), C.c_void_p(offsets.data_ptr()),
                                       C.c_void_p(xg.data_ptr()), C.c_int(T), C.c_int(H), C.c_int(pos.shape[1]), C.c_int(xg.shape[0]),
                                       C.c_void_p(_stream())), "ovb_moe_gather_sorted")


def moe_combine_sorted(y: torch.Tensor, route: torch.Tensor, pos: torch.Tensor, offsets: torch.Tensor, dst: torch.Tensor, e0: int, accumulate: bool) -> None:
    """dst[t] (+)= sum over local experts of route[t, e] * y[row of (t, e)] (expert order, deterministic)."""
    T, E = route.shape
    _check(lib().ovb_moe_combine_sorted(C.c_void_p(y.data_ptr()), C.c_void_p(route.data_ptr()), C.c_void_p(pos.data_ptr()), C.c_void_p(offsets.data_ptr()),
                                        C.c_void_p(dst.data_ptr()), C.c_int(T), C.c_int(y.shape[1]), C.c_int(E), C.c_int(e0), C.c_int(pos.shape[1]),
                                        C.c_int(dst.stride(0)), C.c_int(1 if accumulate else 0), C.c_int(y.shape[0]), C.c_void_p(_stream())),
           "ovb_moe_combine_sorted")


def gemm_grouped(x: torch.Tensor, w: PackedWeight, offsets: torch.Tensor, num_groups: int, mode: int, out: torch.Tensor, act: int = ACT_NONE,
                 ws: Optional[Workspace] = None, block_t: int = 0) -> torch.Tensor:
    """One launch for all groups (experts): rows [offsets[g], offsets[g + 1]) of ``x`` times weight g of the stack ``w``.
    mode 1: ``w`` is [num_groups * N, K] (stacked along N); mode 2: ``w`` is [N, num_groups * K] (stacked along K).
    ``offsets`` is an int32 device tensor written by an earlier kernel; nothing is read back to the host."""
    assert x.dim() == 2 and x.stride(1) == 1 and offsets.dtype == torch.int32 and offsets.numel() >= num_groups + 1
    cap, K = x.shape
    N = w.N // num_groups if mode == 1 else w.N
    assert (K == w.K if mode == 1 else K * num_groups == w.K), (K, w.K, mode)
    if ws is None:
        ws = default_workspace(x.device)
    a = GemmArgs()
    a.x, a.w, a.out = x.data_ptr(), w.w.data_ptr(), out.data_ptr()
    a.bias = None
    a.residual = None
    a.scales, a.zps = _ptr(w.scales), _ptr(w.zps)
    a.ws, a.counters, a.ws_bytes = ws.gemm_ws.data_ptr(), ws.counters.data_ptr(), ws.gemm_ws.numel() * 4
    a.T, a.N, a.K = cap, N, K
    a.ldx, a.ldo, a.ldr = x.stride(0), out.stride(0), 0
    a.group_size = w.group_size
    a.wmode, a.act, a.out_f32 = w.mode, act, 0
    a.splits, a.block_t = 1, block_t
    a.w_kb_stride = 0
    a.w_tiled = 1 if (w.tiled and w.mode in (W_BF16, W_F16)) else 0
    a.comm = None
    a.group_offsets, a.num_groups, a.group_mode = offsets.data_ptr(), num_groups, mode
    _check(lib().ovb_gemm(C.byref(a), C.c_void_p(_stream())), "ovb_gemm (grouped)")
    return out


def moe_silu_mul_rows(gu: torch.Tensor, route: torch.Tensor, idx: torch.Tensor, e: int, out: torch.Tensor) -> torch.Tensor:
    rows, F2 = gu.shape
    _check(lib().ovb_moe_silu_mul_rows(C.c_void_p(gu.data_ptr()), C.c_void_p(route.data_ptr()), C.c_void_p(idx.data_ptr()), C.c_void_p(out.data_ptr()),
                                       C.c_int(rows), C.c_int(F2 // 2), C.c_int(route.shape[1]), C.c_int(e), C.c_void_p(_stream())), "ovb_moe_silu_mul_rows")
    return out


def moe_scatter_add(src: torch.Tensor, idx: torch.Tensor, dst: torch.Tensor) -> None:
    rows, H = src.shape
    _check(lib().ovb_moe_scatter_add(C.c_void_p(src.data_ptr()), C.c_void_p(idx.data_ptr()), C.c_void_p(dst.data_ptr()), C.c_int(rows), C.c_int(H),
                                     C.c_int(dst.stride(0)), C.c_void_p(_stream())), "ovb_moe_scatter_add")


def add(a, b, out=None):
    if out is None:
        out = torch.empty_like(a)
    _check(lib().ovb_add(C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(out.data_ptr()),
                         C.c_int64(a.numel()), C.c_void_p(_stream())), "ovb_add")
    return out


def embedding(ids, table, out=None):
    rows = ids.numel()
    vocab, cols = table.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=table.dtype, device=table.device)
    _check(lib().ovb_embedding(C.c_void_p(ids.data_ptr()), C.c_int(1 if ids.dtype == torch.int32 else 0),
                               C.c_void_p(table.data_ptr()), C.c_void_p(out.data_ptr()),
                               C.c_int(rows), C.c_int(cols), C.c_int(vocab), C.c_void_p(_stream())), "ovb_embedding")
    return out


def argmax(logits, out=None, out_max=None):
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int64, device=logits.device)
    _check(lib().ovb_argmax(C.c_void_p(logits.data_ptr()), C.c_int(logits.stride(0)), C.c_int(rows), C.c_int(vocab),
                            C.c_void_p(out.data_ptr()), C.c_int(1 if out.dtype == torch.int32 else 0),
                            C.c_void_p(_ptr(out_max)), C.c_void_p(_stream())), "ovb_argmax")
    return out


def resolve_ids(ids, tok_src, last_token):
    _check(lib().ovb_resolve_ids(C.c_void_p(ids.data_ptr()), C.c_void_p(tok_src.data_ptr()),
                                 C.c_void_p(last_token.data_ptr()), C.c_int(ids.numel()), C.c_void_p(_stream())),
           "ovb_resolve_ids")


def scatter_tokens(tokens, tok_dst, last_token):
    _check(lib().ovb_scatter_tokens(C.c_void_p(tokens.data_ptr()), C.c_void_p(tok_dst.data_ptr()),
                                    C.c_void_p(last_token.data_ptr()), C.c_int(tokens.numel()), C.c_void_p(_stream())),
           "ovb_scatter_tokens")


def rope_kv_write(qkv, positions, slot_map, k_cache, v_cache, Hq, Hkv, D, theta, block_size):
    T = qkv.shape[0]
    _check(lib().ovb_rope_kv_write(C.c_void_p(qkv.data_ptr()), C.c_void_p(positions.data_ptr()),
                                   C.c_void_p(slot_map.data_ptr()), C.c_void_p(k_cache.data_ptr()),
                                   C.c_void_p(v_cache.data_ptr()), C.c_int(T), C.c_int(Hq), C.c_int(Hkv), C.c_int(D),
                                   C.c_float(theta), C.c_int(block_size), C.c_void_p(_stream())), "ovb_rope_kv_write")


def rope_kv_write_u8(qkv, positions, slot_map, k_cache, v_cache, k_meta, v_meta, Hq, Hkv, D, theta, block_size):
    """RoPE on the query / key heads of ``qkv`` and the write of the new key / value rows into a u8 cache: rows are
    quantised per (token, head); ``k_meta`` / ``v_meta`` [num_blocks, Hkv, block_size, 2] fp16 receive (scale, zero point)."""
    T = qkv.shape[0]
    assert k_cache.dtype == torch.uint8 and k_meta.dtype == torch.float16
    _check(lib().ovb_rope_kv_write_u8(C.c_void_p(qkv.data_ptr()), C.c_void_p(positions.data_ptr()), C.c_void_p(slot_map.data_ptr()),
                                      C.c_void_p(k_cache.data_ptr()), C.c_void_p(v_cache.data_ptr()), C.c_void_p(k_meta.data_ptr()),
                                      C.c_void_p(v_meta.data_ptr()), C.c_int(T), C.c_int(Hq), C.c_int(Hkv), C.c_int(D), C.c_float(theta),
                                      C.c_int(block_size), C.c_void_p(_stream())), "ovb_rope_kv_write_u8")


def paged_attention(q, k_cache, v_cache, past_lens, subsequence_begins, block_indices, block_indices_begins, Hq, Hkv, D,
                    scale=None, max_context_len=0, max_q_len=0, sliding_window=0, block_size=16, out=None, ws=None, k_meta=None, v_meta=None):
    """q: [T, >=Hq*D] (row pitch = q.stride(0)); caches [num_blocks, Hkv, block_size, D] (16-bit, or uint8 with the
    (scale, zero point) tables ``k_meta`` / ``v_meta``)."""
    T = q.shape[0]
    B = past_lens.numel()
    if out is None:
        out = torch.empty((T, Hq * D), dtype=q.dtype, device=q.device)
    if ws is None:
        ws = default_workspace(q.device)
    a = PaArgs()
    a.q, a.out, a.k_cache, a.v_cache = q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    a.past_lens, a.subsequence_begins = past_lens.data_ptr(), subsequence_begins.data_ptr()
    a.block_indices, a.block_indices_begins = block_indices.data_ptr(), block_indices_begins.data_ptr()
    need = int(lib().ovb_pa_scratch_bytes(C.c_int(B), C.c_int(Hq), C.c_int(D), C.c_int(max_context_len)))
    a.scratch = ws.pa_scratch.data_ptr() if need <= ws.pa_scratch.numel() * 4 else None
    a.B, a.T, a.Hq, a.Hkv, a.D = B, T, Hq, Hkv, D
    a.ldq = q.stride(0)
    a.block_size, a.max_context_len, a.max_q_len = block_size, max_context_len, max_q_len
    a.sliding_window = sliding_window
    a.scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if k_cache.dtype == torch.uint8:
        assert k_meta is not None and v_meta is not None
        a.kv_u8, a.k_meta, a.v_meta = 1, k_meta.data_ptr(), v_meta.data_ptr()
    _check(lib().ovb_paged_attention(C.byref(a), C.c_void_p(_stream())), "ovb_paged_attention")
    return out


def sdpa_dense(q, k, v, B, S, H, D, ld, scale=None, causal=False, out=None):
    """q/k/v: views into [B*S, ld] buffers (head h at column h*D); out [B*S, H*D]."""
    if out is None:
        out = torch.empty((B * S, H * D), dtype=q.dtype, device=q.device)
    sc = scale if scale is not None else 1.0 / math.sqrt(D)
    _check(lib().ovb_sdpa_dense(C.c_void_p(q.data_ptr()), C.c_void_p(k.data_ptr()), C.c_void_p(v.data_ptr()),
                                C.c_void_p(out.data_ptr()), C.c_int(B), C.c_int(S), C.c_int(H), C.c_int(D), C.c_int(ld),
                                C.c_float(sc), C.c_int(1 if q.dtype == torch.float16 else 0), C.c_int(1 if causal else 0),
                                C.c_void_p(_stream())), "ovb_sdpa_dense")
    return out
