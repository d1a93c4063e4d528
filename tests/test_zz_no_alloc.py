"""The allocation-free decode attention entry point, called through its exported C symbol.

``ovb_paged_attention_decode_static`` (declared in csrc/cuda/ovb_cuda_static.h) keeps its split-KV scratch in a
fixed device array inside the library. The test calls the symbol with ctypes, twice in a row on batches of
different shape (so the second call meets the leftovers of the first), and compares each result with
``ovb_paged_attention`` given a caller-allocated scratch. A batch beyond the static size must be refused
before anything is launched. The file name keeps this module last in collection order; it also passes when
run alone in a fresh process.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 * 1024 * 1024


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _decode_batch(past_lens, Hq, Hkv, D, block_size, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    B = len(past_lens)
    nblocks = [(p + 1 + block_size - 1) // block_size for p in past_lens]
    total = sum(nblocks)
    begins = [0]
    for n in nblocks:
        begins.append(begins[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).to(torch.int32).cuda()
    return dict(
        q=torch.randn(B, Hq * D, device="cuda", generator=g).to(torch.bfloat16),
        k_cache=torch.randn(total, Hkv, block_size, D, device="cuda", generator=g).to(torch.bfloat16),
        v_cache=torch.randn(total, Hkv, block_size, D, device="cuda", generator=g).to(torch.bfloat16),
        past_lens=i32(past_lens), subsequence_begins=i32(list(range(B + 1))), block_indices=perm, block_indices_begins=i32(begins),
        B=B, Hq=Hq, Hkv=Hkv, D=D, block_size=block_size, max_context_len=max(past_lens) + 1)


def _reference_decode(batch):
    """Plain PyTorch fp32 decode attention over the paged cache (one query token per sequence)."""
    B, Hq, Hkv, D, bs = batch["B"], batch["Hq"], batch["Hkv"], batch["D"], batch["block_size"]
    q = batch["q"].float().view(B, Hq, D)
    out = torch.empty(B, Hq, D, device="cuda")
    begins = batch["block_indices_begins"].tolist()
    for b in range(B):
        n = int(batch["past_lens"][b]) + 1
        blocks = batch["block_indices"][begins[b]:begins[b + 1]].long()
        keys = batch["k_cache"][blocks].float().permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n]
        vals = batch["v_cache"][blocks].float().permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n]
        keys = keys.repeat_interleave(Hq // Hkv, 0)
        vals = vals.repeat_interleave(Hq // Hkv, 0)
        p = torch.softmax(torch.einsum("hd,hnd->hn", q[b], keys) / math.sqrt(D), -1)
        out[b] = torch.einsum("hn,hnd->hd", p, vals)
    return out.view(B, Hq * D)


def _args(k, batch, out, scratch_ptr):
    a = k.PaArgs()
    a.q, a.out = batch["q"].data_ptr(), out.data_ptr()
    a.k_cache, a.v_cache = batch["k_cache"].data_ptr(), batch["v_cache"].data_ptr()
    a.past_lens, a.subsequence_begins = batch["past_lens"].data_ptr(), batch["subsequence_begins"].data_ptr()
    a.block_indices, a.block_indices_begins = batch["block_indices"].data_ptr(), batch["block_indices_begins"].data_ptr()
    a.scratch = scratch_ptr
    a.B = a.T = batch["B"]
    a.Hq, a.Hkv, a.D = batch["Hq"], batch["Hkv"], batch["D"]
    a.ldq = batch["q"].stride(0)
    a.block_size, a.max_context_len, a.max_q_len = batch["block_size"], batch["max_context_len"], 1
    a.sliding_window = 0
    a.scale = 1.0 / math.sqrt(batch["D"])
    return a


@pytest.fixture(scope="module")
def k():
    from openvino_b200.ops import cuda as mod
    lib = mod.lib()
    fn = lib.ovb_paged_attention_decode_static          # the exported C symbol
    fn.argtypes = [C.POINTER(mod.PaArgs), C.c_void_p]
    fn.restype = C.c_int
    lib.ovb_last_error.restype = C.c_char_p
    return mod


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row(k):
    lib = k.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # first: long contexts, many KV splits; second: another shape with fewer splits, run right after
    shapes = [([1500, 40, 2047, 700], 8, 2), ([300, 5, 129], 32, 8)]
    for seed, (past_lens, Hq, Hkv) in enumerate(shapes):
        batch = _decode_batch(past_lens, Hq, Hkv, 128, 16, seed)
        need = int(lib.ovb_pa_scratch_bytes(C.c_int(batch["B"]), C.c_int(Hq), C.c_int(128), C.c_int(batch["max_context_len"])))
        assert need <= STATIC_SCRATCH_BYTES
        want = torch.zeros(batch["B"], Hq * 128, device="cuda", dtype=torch.bfloat16)
        caller_scratch = torch.empty(need // 4, device="cuda", dtype=torch.float32)
        rc = lib.ovb_paged_attention(C.byref(_args(k, batch, want, caller_scratch.data_ptr())), stream)
        assert rc == 0, lib.ovb_last_error()
        got = torch.zeros_like(want)
        rc = lib.ovb_paged_attention_decode_static(C.byref(_args(k, batch, got, None)), stream)
        assert rc == 0, lib.ovb_last_error()
        torch.cuda.synchronize()
        assert want.float().abs().sum().item() > 0
        assert _rel_err(got, want) < 1e-2
        assert _rel_err(got, _reference_decode(batch)) < 2e-2
        # The point of the entry point: a call takes no device memory, neither from the driver nor from PyTorch's
        # caching allocator. (The very first call on a device may load the library's device code; this one is later.)
        out2 = torch.zeros_like(want)
        args2 = _args(k, batch, out2, None)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        torch_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        rc = lib.ovb_paged_attention_decode_static(C.byref(args2), stream)
        torch.cuda.synchronize()
        assert rc == 0, lib.ovb_last_error()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before
        assert torch.equal(out2, got)


def test_batch_beyond_the_static_size_is_refused(k):
    lib = k.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    batch = _decode_batch([3] * 64, 32, 8, 128, 16, 3)          # 64 x 32 heads needs about 34 MB
    out = torch.full((64, 32 * 128), 7.0, device="cuda", dtype=torch.bfloat16)
    rc = lib.ovb_paged_attention_decode_static(C.byref(_args(k, batch, out, None)), stream)
    assert rc < 0
    msg = lib.ovb_last_error().decode()
    assert "static" in msg and str(STATIC_SCRATCH_BYTES) in msg
    torch.cuda.synchronize()
    assert (out == 7.0).all()                                   # nothing was launched
    # prefill batches are not what this entry point is for
    a = _args(k, _decode_batch([3, 3], 8, 2, 128, 16, 4), out, None)
    a.max_q_len = 2
    assert lib.ovb_paged_attention_decode_static(C.byref(a), stream) < 0
    # nor shapes that the split-KV decode kernel does not serve (they would never touch the scratch)
    a = _args(k, _decode_batch([3, 3], 8, 2, 128, 16, 4), out, None)
    a.block_size = 32
    assert lib.ovb_paged_attention_decode_static(C.byref(a), stream) < 0
    assert "block size" in lib.ovb_last_error().decode()
