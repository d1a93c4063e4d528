"""Tensor-parallel communicator: one process per GPU, peers reach each other's memory over NVLink.

Every rank owns a *symmetric heap*: one device allocation with the same layout on all ranks, exported as a CUDA
IPC handle and mapped by every peer (handles travel through ``torch.distributed``; NCCL or gloo only carry the
64-byte handles, never tensor data). The kernels of the library then read and write peers' heaps directly:

* ``gemm_allreduce``  - the row-parallel GEMM with the all-reduce (+ residual add) fused into its epilogue:
  tiles are pushed to peers as soon as they leave the tensor core, tile by tile (ovb_gemm with ``comm``).
* ``argmax_combine``  - greedy sampling over vocabulary shards.
* ``all_reduce``      - small bf16 tensors that live in the heap.

Heap layout (byte offsets are the same on every rank): step counter, flag words per call site, one-shot staging
(two alternating buffers), two-shot staging, then tensors handed out by ``alloc`` (the residual streams).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch

from ..ops import cuda as K

MAX_RANKS = 8
ARGMAX_ROWS_CAP = 1024
NVLS_FLAG_STRIDE = 16      # kNvlsFlagStride of the kernels


class CommStruct(C.Structure):
    """Mirror of ``ovb_comm`` (csrc/cuda/ovb_cuda.h)."""

    _fields_ = [
        ("rank", C.c_int), ("world", C.c_int),
        ("heap", C.c_void_p * MAX_RANKS),
        ("heap_bytes", C.c_int64),
        ("epoch_off", C.c_int64), ("flags_off", C.c_int64), ("flags_per_site", C.c_int64),
        ("stage1_off", C.c_int64), ("stage1_bytes", C.c_int64), ("stage2_off", C.c_int64), ("stage2_bytes", C.c_int64),
        ("num_sites", C.c_int), ("site", C.c_int), ("mode", C.c_int),
        ("mc_base", C.c_void_p), ("nvls_flags_off", C.c_int64), ("nvls_flags_per_site", C.c_int64),
        ("stage3_off", C.c_int64), ("stage3_bytes", C.c_int64),
    ]


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


class HeapLayout:
    """Offsets of the fixed areas inside the symmetric heap; pure arithmetic, shared by every rank."""

    def __init__(self, world: int, hidden: int, max_tokens: int, num_sites: int, tensor_bytes: int):
        self.world, self.hidden, self.max_tokens, self.num_sites = world, hidden, max_tokens, num_sites
        tiles_max = (hidden // 128) * ((max_tokens + 255) // 256 + 1)
        self.flags_per_site = max(tiles_max * (world + 1), 64 + 2 * world * ARGMAX_ROWS_CAP * 2)
        self.epoch_off = 0
        self.flags_off = 256
        off = self.flags_off + num_sites * self.flags_per_site * 4
        self.stage1_off = _round_up(off, 1024)
        self.stage1_bytes = _round_up(2 * world * 128 * hidden * 2, 1024)        # one-shot (T <= 128): flag-carrying packets, 2x the tile bytes
        self.stage2_off = self.stage1_off + 2 * self.stage1_bytes
        # two-shot: every tile has one owner; rounding the tiles per owner up costs at most `world` extra tiles
        self.stage2_bytes = _round_up(2 * (_round_up(max_tokens, 256) * hidden + world * 256 * 128) * 2, 1024)    # packets: 2x
        # staging of the stand-alone all-reduce (two alternating buffers of its own)
        self.stage3_off = _round_up(self.stage2_off + self.stage2_bytes, 1024)
        self.stage3_bytes = self.stage1_bytes
        # barrier words of the in-switch (NVLS) collectives: 16 int32 per tile of a fused GEMM / CTA of an all-reduce
        self.nvls_flags_per_site = max(tiles_max, 148) * NVLS_FLAG_STRIDE
        self.nvls_flags_off = _round_up(self.stage3_off + 2 * self.stage3_bytes, 1024)
        self.tensors_off = _round_up(self.nvls_flags_off + num_sites * self.nvls_flags_per_site * 4, 1024)
        self.heap_bytes = self.tensors_off + _round_up(tensor_bytes, 1024)


class PeerCommunicator:
    def __init__(self, rank: int, world: int, device, group=None):
        assert 1 <= world <= MAX_RANKS
        self.rank, self.world, self.device, self.group = rank, world, torch.device(device), group
        self.layout: Optional[HeapLayout] = None
        self._base = 0
        self._peer_ptrs: List[int] = []
        self._bump = 0
        self._structs = {}
        self._keep = []
        self._any_bufs = {}
        self.mc_ptr = 0           # multicast mapping of the heap (NVLS), 0 = none
        self._symm = None

    # ------------------------------------------------------------------ set-up (collective)
    def setup(self, hidden: int, max_tokens: int, num_layers: int, tensor_bytes: int) -> None:
        """Allocate this rank's heap and map every peer's. Call on all ranks with equal arguments.

        Two ways to get the heap. Preferred: ``torch.distributed._symmetric_memory`` (driver virtual-memory allocations
        exchanged between the processes), which on an NVSwitch machine also binds the heaps to one NVLink multicast
        object: ``mc_ptr`` then addresses all ranks' heaps at once and the collectives reduce inside the switch. Otherwise
        (``OVB_NVLS=0`` or ``NCCL_NVLS_ENABLE=0`` in the environment, or the set-up failing on any rank): a plain device
        allocation exported as a CUDA IPC handle, and the peer-store protocols. A job whose ranks may leave while others
        keep running uses the second form: a rank must not die while its memory is bound to a multicast object."""
        import torch.distributed as dist
        num_sites = 2 * num_layers + 3          # two fused GEMMs per layer, argmax, two alternating all-reduce sites
        self.layout = HeapLayout(self.world, hidden, max_tokens, num_sites, tensor_bytes)
        lib = K.lib()
        self._declare(lib)
        self.mc_ptr = 0
        self._symm = None
        want_nvls = os.environ.get("OVB_NVLS", "1") != "0" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0" and self.world in (2, 4, 8)
        if want_nvls:
            ok, err = 1, ""
            try:
                self._setup_symmetric()
            except Exception as e:            # noqa: BLE001 - any failure means "use the IPC heap", on every rank
                ok, err = 0, "%s: %s" % (type(e).__name__, e)
            flags = [None] * self.world
            dist.all_gather_object(flags, (ok, err), group=self.group)
            if not all(f[0] for f in flags):
                self._symm, self._base, self._peer_ptrs, self.mc_ptr = None, 0, [], 0
                from ..utils import log as _log
                _log.warn("comm", "symmetric-memory heap unavailable (%s); using the CUDA IPC heap and peer stores"
                          % "; ".join(f[1] for f in flags if not f[0])[:300])
        if not self._base:
            self._setup_ipc(lib)
        self._bump = self.layout.tensors_off
        dist.barrier(group=self.group)
        # peer mappings are released before the CUDA context goes away at interpreter exit (or at openvino_b200.shutdown())
        import weakref
        from ..utils.shutdown import register_shutdown_callback
        ref = weakref.ref(self)
        register_shutdown_callback(lambda: ref() and ref().close(), "PeerCommunicator.close")

    def _setup_symmetric(self) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = self.group if self.group is not None else dist.group.WORLD
        with torch.cuda.device(self.device):
            t = symm.empty(self.layout.heap_bytes, dtype=torch.uint8, device=self.device)
            t.zero_()
            torch.cuda.synchronize(self.device)
            hdl = symm.rendezvous(t, group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != t.data_ptr():
            raise RuntimeError("unexpected symmetric-memory handle (%d pointers)" % len(ptrs))
        self._symm = (t, hdl)               # keeps the allocation and the mappings alive
        self._base, self._peer_ptrs = ptrs[self.rank], ptrs
        self.mc_ptr = int(getattr(hdl, "multicast_ptr", 0) or 0)

    def _setup_ipc(self, lib) -> None:
        import torch.distributed as dist
        with torch.cuda.device(self.device):
            base = C.c_void_p()
            K._check(lib.ovb_comm_alloc(C.c_int64(self.layout.heap_bytes), C.byref(base)), "ovb_comm_alloc")
            self._base = base.value
            handle = (C.c_ubyte * 64)()
            K._check(lib.ovb_comm_export(C.c_void_p(self._base), handle), "ovb_comm_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=self.group)
            self._peer_ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    self._peer_ptrs.append(self._base)
                    continue
                buf = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                p = C.c_void_p()
                K._check(lib.ovb_comm_open(buf, C.byref(p)), "ovb_comm_open")
                self._peer_ptrs.append(p.value)

    @staticmethod
    def _declare(lib) -> None:
        lib.ovb_comm_alloc.argtypes = [C.c_int64, C.POINTER(C.c_void_p)]
        lib.ovb_comm_export.argtypes = [C.c_void_p, C.c_void_p]
        lib.ovb_comm_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        lib.ovb_comm_close.argtypes = [C.c_void_p]
        lib.ovb_comm_free.argtypes = [C.c_void_p]
        lib.ovb_comm_step_begin.argtypes = [C.POINTER(CommStruct), C.c_void_p]
        lib.ovb_comm_argmax_combine.argtypes = [C.POINTER(CommStruct), C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.ovb_comm_allreduce_bf16.argtypes = [C.POINTER(CommStruct), C.c_void_p, C.c_int64, C.c_void_p]
        lib.ovb_comm_allreduce.argtypes = [C.POINTER(CommStruct), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]

    def close(self) -> None:
        if not self._base:
            return
        lib = K.lib()
        torch.cuda.synchronize(self.device)
        if self._symm is not None:          # torch owns the allocation and the mappings
            self._symm, self._base, self._peer_ptrs, self.mc_ptr = None, 0, [], 0
            return
        for r, p in enumerate(self._peer_ptrs):
            if r != self.rank and p:
                lib.ovb_comm_close(C.c_void_p(p))
        lib.ovb_comm_free(C.c_void_p(self._base))
        self._base, self._peer_ptrs = 0, []

    # ------------------------------------------------------------------ heap tensors
    def alloc(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """A tensor inside the symmetric heap (same offset on every rank when every rank allocates in the same order)."""
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        off = _round_up(self._bump, 256)
        if off + nbytes > self.layout.heap_bytes:
            raise RuntimeError("symmetric heap exhausted: %d bytes wanted at offset %d of %d" % (nbytes, off, self.layout.heap_bytes))
        self._bump = off + nbytes
        t = _wrap_device_memory(self._base + off, nbytes, self.device).view(dtype).reshape(tuple(shape))
        self._keep.append(t)
        return t

    def in_heap(self, t: torch.Tensor) -> bool:
        return self._base <= t.data_ptr() < self._base + self.layout.heap_bytes

    # ------------------------------------------------------------------ collectives
    def struct(self, site: int, mode: int = 0) -> CommStruct:
        key = (site, mode)
        s = self._structs.get(key)
        if s is None:
            L = self.layout
            s = CommStruct()
            s.rank, s.world = self.rank, self.world
            for r in range(self.world):
                s.heap[r] = self._peer_ptrs[r]
            s.heap_bytes = L.heap_bytes
            s.epoch_off, s.flags_off, s.flags_per_site = L.epoch_off, L.flags_off, L.flags_per_site
            s.stage1_off, s.stage1_bytes, s.stage2_off, s.stage2_bytes = L.stage1_off, L.stage1_bytes, L.stage2_off, L.stage2_bytes
            s.num_sites, s.site, s.mode = L.num_sites, site, mode
            s.mc_base = self.mc_ptr or None
            s.nvls_flags_off, s.nvls_flags_per_site = L.nvls_flags_off, L.nvls_flags_per_site
            s.stage3_off, s.stage3_bytes = L.stage3_off, L.stage3_bytes
            self._structs[key] = s
        return s

    def step_begin(self) -> None:
        K._check(K.lib().ovb_comm_step_begin(C.byref(self.struct(0)), C.c_void_p(K._stream())), "ovb_comm_step_begin")

    def recover(self) -> int:
        """After a step in which a rank reported a peer time-out (or did not take part): bring the ranks' step numbers back
        together. Every rank calls this between steps, with nothing of its own in flight: the step numbers are compared on
        the host and every rank moves to one past the largest, so that flags and packet tags of the abandoned step can never
        satisfy a later wait; the local completion counter of the fused kernels and the device status word are cleared.
        Returns the new step number. (The reference's sub-memory manager has no recovery: a lost rank ends the process
        group, src/plugins/intel_cpu/src/sub_memory_manager.hpp.)"""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        epoch = _wrap_device_memory(self._base + self.layout.epoch_off, 4, self.device).view(torch.int32)
        mine = torch.tensor([int(epoch.item())], dtype=torch.int64, device=self.device if dist.get_backend(self.group) == "nccl" else "cpu")
        dist.all_reduce(mine, op=dist.ReduceOp.MAX, group=self.group)
        new = int(mine.item()) + 1
        epoch.fill_(new)
        K.default_workspace(self.device).counters.zero_()
        K.read_status()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        return new

    def gemm_allreduce(self, x: torch.Tensor, w: "K.PackedWeight", h: torch.Tensor, ws, site: int, mode: int = 0) -> None:
        """h += sum over ranks of x @ W_shard^T (h replicated, must live in the heap)."""
        K.gemm(x, w, out=h, residual=h, ws=ws, comm=self.struct(site, mode))

    def argmax_combine(self, ids: torch.Tensor, max_vals: torch.Tensor, shard_size: int) -> None:
        site = self.layout.num_sites - 3
        K._check(K.lib().ovb_comm_argmax_combine(C.byref(self.struct(site)), C.c_void_p(ids.data_ptr()), C.c_void_p(max_vals.data_ptr()),
                                                 C.c_int(ids.numel()), C.c_int(shard_size), C.c_void_p(K._stream())), "ovb_comm_argmax_combine")

    _DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

    def all_reduce(self, t: torch.Tensor, site: Optional[int] = None) -> None:
        """In-place sum over the ranks of a heap tensor (fp32, fp16 or bf16; a multiple of 16 bytes)."""
        assert t.dtype in self._DTYPES and t.is_contiguous() and self.in_heap(t)
        site = self.layout.num_sites - 1 if site is None else site
        K._check(K.lib().ovb_comm_allreduce(C.byref(self.struct(site)), C.c_void_p(t.data_ptr()), C.c_int64(t.numel()), C.c_int(self._DTYPES[t.dtype]),
                                            C.c_void_p(K._stream())), "ovb_comm_allreduce")

    def all_reduce_any(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over the ranks of any device tensor (fp32 / fp16 / bf16): staged through a heap tensor that grows on demand
        (every rank calls with the same sizes in the same order, so the heap offsets agree). Returns a new tensor."""
        assert x.dtype in self._DTYPES
        per = 16 // x.element_size()
        n = x.numel()
        padded = (n + per - 1) // per * per
        key = x.dtype
        buf = self._any_bufs.get(key)
        if buf is None or buf.numel() < padded:
            buf = self.alloc((max(padded, 1 << 20),), x.dtype)
            self._any_bufs[key] = buf
        stage = buf[:padded]
        if padded != n:
            stage[n:].zero_()
        stage[:n].copy_(x.reshape(-1))
        self.all_reduce_large(stage)
        return stage[:n].clone().reshape(x.shape)

    def all_reduce_large(self, t: torch.Tensor) -> int:
        """Sum a heap tensor of any size over the ranks, in pieces that fit the one-shot staging area. Every piece gets
        a step number of its own (the flags of a call site hold step numbers) and the pieces alternate between two call
        sites, i.e. between the two staging buffers: a rank that runs ahead writes into the buffer its peers are not
        reading. A last bump keeps later users of the step number apart from these flags. Returns the launches made."""
        assert t.dtype in self._DTYPES and t.is_contiguous() and self.in_heap(t)
        L = self.layout
        if self.mc_ptr:
            # in-switch reduction works in place on the heap tensor: no staging, so no pieces
            self.step_begin()
            self.all_reduce(t)
            return 2
        per = 16 // t.element_size()
        max_elems = (((L.stage3_bytes // self.world) & ~15) // t.element_size()) & ~(per - 1)
        flat = t.view(-1)
        n, i, k = flat.numel(), 0, 0
        while i < n:
            m = min(max_elems, n - i)
            self.step_begin()
            self.all_reduce(flat[i:i + m], site=L.num_sites - 1 - (k & 1))
            i += m
            k += 1
        self.step_begin()
        return 2 * k + 1


class _DeviceMemory:
    """Exposes raw device memory through ``__cuda_array_interface__`` so that torch can view it without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def _wrap_device_memory(ptr: int, nbytes: int, device) -> torch.Tensor:
    with torch.cuda.device(device):
        return torch.as_tensor(_DeviceMemory(ptr, nbytes), device=device)
