"""Tensor parallelism: heap layout arithmetic on CPU; the fused GEMM + all-reduce and the TP model on 2 GPUs."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

from openvino_b200.parallel.comm import CommStruct, HeapLayout


def test_heap_layout_is_disjoint_and_large_enough():
    for world, hidden, tokens, layers in ((2, 4096, 8192, 32), (8, 4096, 8192, 32), (4, 8192, 4096, 80), (2, 256, 256, 2)):
        L = HeapLayout(world, hidden, tokens, 2 * layers + 2, tensor_bytes=tokens * hidden * 2)
        areas = [(L.epoch_off, 4), (L.flags_off, L.num_sites * L.flags_per_site * 4), (L.stage1_off, 2 * L.stage1_bytes),
                 (L.stage2_off, L.stage2_bytes), (L.stage3_off, 2 * L.stage3_bytes),
                 (L.nvls_flags_off, L.num_sites * L.nvls_flags_per_site * 4), (L.tensors_off, L.heap_bytes - L.tensors_off)]
        for (a, n), (b, _) in zip(areas, areas[1:]):
            assert a + n <= b
        assert L.heap_bytes - L.tensors_off >= tokens * hidden * 2
        # one-shot: T <= 128 -> one token tile per weight tile
        tiles = hidden // 128
        # (flag-carrying packets take twice the bytes of the bf16 tiles)
        assert 2 * world * tiles * 128 * 128 * 2 <= L.stage1_bytes
        # two-shot: worst case T = tokens with 256-token tiles
        t_tiles = (tokens + 255) // 256
        total = tiles * t_tiles
        assert 2 * world * ((total + world - 1) // world) * 256 * 128 * 2 <= L.stage2_bytes
        assert total * (world + 1) <= L.flags_per_site
        # in-switch protocol: plain bf16 tiles in the same staging areas, 16 barrier words per tile
        assert tiles * 128 * 128 * 2 <= L.stage1_bytes and total * 256 * 128 * 2 <= L.stage2_bytes
        assert total * 16 <= L.nvls_flags_per_site and 148 * 16 <= L.nvls_flags_per_site
        for off in (L.stage1_off, L.stage2_off, L.tensors_off):
            assert off % 256 == 0


def test_comm_struct_matches_the_c_layout():
    # int rank, world; void* heap[8]; int64 x 8; int x 3 (+ padding to 8); void* mc_base; int64 x 4
    assert C.sizeof(CommStruct) == 8 + 64 + 8 * 8 + 16 + 8 + 4 * 8
    assert CommStruct.heap.offset == 8 and CommStruct.heap_bytes.offset == 72 and CommStruct.num_sites.offset == 136
    assert CommStruct.mc_base.offset == 152 and CommStruct.stage3_bytes.offset == 184


def _run_tp_worker(world: int, nvls: bool, port: int):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    # nvls False: CUDA IPC heap + peer stores (no multicast object is ever bound); True: symmetric memory + in-switch reduction
    env = dict(os.environ, OVB_NVLS="1" if nvls else "0")
    if not nvls:
        env["NCCL_NVLS_ENABLE"] = "0"
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
                        "--master-port", str(port), worker], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "TP_WORKER_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])
    return r.stdout


@pytest.mark.gpu
def test_tensor_parallel_on_two_gpus():
    out = _run_tp_worker(2, False, 29671)
    assert "nvls=0" in out


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_in_switch_reduction(world):
    _run_tp_worker(world, True, 29672 + world)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [4, 8])
def test_tensor_parallel_peer_stores_beyond_two_gpus(world):
    _run_tp_worker(world, False, 29682 + world)


@pytest.mark.gpu
@pytest.mark.parametrize("world,env", [(2, {"OVB_NVLS": "0", "NCCL_NVLS_ENABLE": "0"}), (2, {"OVB_COMM_NVLS_MODES": "3"}), (8, {})])
def test_fused_gemm_all_reduce_at_serving_shapes(world, env):
    """The fused GEMM + all-reduce at the shapes of an 8B model (T = 64 and T = 8192, more tiles than one wave of CTAs, so
    the reducer CTAs and the two-shot owners take part): sum over the ranks against GEMM + fp32 all-reduce, and the same
    bits on every rank. The benchmark module verifies every shape it times and exits non-zero on a mismatch."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
                        "--master-port", str(29690 + world), "-m", "openvino_b200.parallel.bench_fused", "--iters", "3", "--warmup", "1"],
                       capture_output=True, text=True, timeout=900, env=dict(os.environ, **env))
    assert r.returncode == 0 and "FUSED_ALLREDUCE_MISMATCH" not in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])
    import json
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(rows) >= 3 and all(x["ranks_identical"] and x["rel_err_vs_fp32_allreduce"] < 2e-2 for x in rows)


@pytest.mark.gpu
def test_peer_that_never_posts_times_out_and_the_ranks_recover():
    """Failure detection without a GPU fault: a rank skips one fused step, the other rank's kernel reports
    STATUS_PEER_TIMEOUT after a short bounded wait, both keep their contexts, resynchronise on the host and run on."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, OVB_NVLS="0", NCCL_NVLS_ENABLE="0")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_timeout_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29699", worker], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "TP_TIMEOUT_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-3000:])
