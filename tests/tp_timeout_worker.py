"""Ranks of the peer-time-out test (tests/test_tensor_parallel.py): rank 1 sits out one fused GEMM + all-reduce, rank 0's
kernel gives up after a short wait and reports STATUS_PEER_TIMEOUT through the status word; both ranks then resynchronise
their step numbers on the host and the next step works. Plain peer loads / stores on the CUDA IPC heap (no multicast
object is bound), so a rank that stays away cannot disturb the other GPU."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from openvino_b200.ops import cuda as K   # noqa: E402
from openvino_b200.parallel.comm import PeerCommunicator   # noqa: E402
from openvino_b200.utils import quant   # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    world = dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    H, Kd, T = 256, 256, 32
    comm = PeerCommunicator(rank, world, dev)
    comm.setup(hidden=H, max_tokens=256, num_layers=2, tensor_bytes=(256 + 8) * H * 2 + 4096)
    assert not comm.mc_ptr, "this test runs on the IPC heap (OVB_NVLS=0)"
    ws = K.default_workspace(dev)
    h = comm.alloc((T, H))
    torch.manual_seed(rank)
    x = torch.randn(T, Kd, device=dev, dtype=torch.bfloat16)
    packed, s, z = quant.random_u4_weight(H, Kd, 128, dev, seed=rank)
    pw = K.PackedWeight.from_ir_u4(packed, s, quant.pack_u4(z), H, Kd, 128)

    def step(site):
        h.zero_()
        comm.step_begin()
        comm.gemm_allreduce(x, pw, h, ws, site)
        return K.read_status()

    def reference():
        ref = K.gemm(x, pw, out_f32=True, ws=ws)
        dist.all_reduce(ref)
        return ref

    assert step(0) == 0
    ref = reference()
    assert float((h.float() - ref).norm() / ref.norm()) < 2e-2
    dist.barrier()

    # one rank stays away from a step: the other one's wait runs out after a few milliseconds instead of a second
    K.set_peer_spin_limit(20000)
    status = step(1) if rank == 0 else 0
    K.set_peer_spin_limit(0)
    if rank == 0:
        assert status == 2, "expected STATUS_PEER_TIMEOUT, got %d" % status
    torch.cuda.synchronize()
    # the context is alive on both ranks; the host protocol brings the step numbers back together
    new_step = comm.recover()
    assert step(0) == 0 and step(1) == 0
    assert float((h.float() - ref).norm() / ref.norm()) < 2e-2
    dist.barrier()
    if rank == 0:
        print("TP_TIMEOUT_OK world=%d resynchronised at step %d" % (world, new_step), flush=True)
    comm.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
