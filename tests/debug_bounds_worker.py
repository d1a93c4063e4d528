"""Runs under the bounds-checking debug build of the kernels (OVB_CUDA_LIB=.../libovb_cuda_dbg.so): indices beyond the
declared limits are reported through the status word and the access is skipped. Every tensor here is allocated larger
than the declared limit, so the indices used would stay inside device allocations even without the checks."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from openvino_b200.ops import cuda as K   # noqa: E402


def main():
    assert K.debug_bounds_enabled(), "the debug kernel library is not the one that was loaded"
    dev = "cuda"
    Hq, Hkv, D, bs = 8, 2, 128, 16
    declared, allocated = 8, 16                     # the host declares 8 cache blocks; the tensors hold 16
    K.debug_set_limits(kv_blocks=declared, vocab=100)
    kc = torch.randn(allocated, Hkv, bs, D, device=dev).to(torch.bfloat16)
    vc = torch.randn_like(kc)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    q = torch.randn(2, Hq * D, device=dev).to(torch.bfloat16)
    past, sb, bib = i32([40, 20]), i32([0, 1, 2]), i32([0, 3, 5])

    def decode(blocks):
        K.paged_attention(q, kc, vc, past, sb, i32(blocks), bib, Hq, Hkv, D, max_context_len=41, max_q_len=1)
        return K.read_status()

    assert decode([0, 1, 2, 3, 4]) == 0
    assert decode([0, 1, 11, 3, 4]) == 5            # block 11 >= 8 declared blocks
    assert decode([5, 6, 7, 3, 4]) == 0             # the status word was cleared by the read; the context is fine

    # cache write: a slot beyond the declared cache is reported and not written
    qkv = torch.randn(3, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16)
    before = kc.clone()
    K.rope_kv_write(qkv, i32([0, 1, 2]), i32([5, declared * bs + 7, 9]), kc, vc, Hq, Hkv, D, 10000.0, bs)
    assert K.read_status() == 5
    blk, off = (declared * bs + 7) // bs, (declared * bs + 7) % bs
    assert torch.equal(kc[blk, :, off], before[blk, :, off])          # the out-of-range row stayed untouched
    assert not torch.equal(kc[0, :, 5], before[0, :, 5])              # the valid rows were written
    K.rope_kv_write(qkv, i32([0, 1, 2]), i32([5, 6, -1]), kc, vc, Hq, Hkv, D, 10000.0, bs)
    assert K.read_status() == 0                                       # a negative slot means "do not write": not an error

    # token ids beyond the vocabulary
    table = torch.randn(128, 64, device=dev).to(torch.bfloat16)       # declared vocabulary: 100 rows
    out = torch.empty(3, 64, device=dev, dtype=torch.bfloat16)
    K.embedding(i32([1, 2, 3]), table[:100], out=out)
    assert K.read_status() == 0
    K.embedding(i32([1, 105, 3]), table[:100], out=out)
    assert K.read_status() == 5 and torch.equal(out[1], table[0])     # reported, row 0 read instead
    print("DEBUG_BOUNDS_OK", flush=True)


if __name__ == "__main__":
    main()
