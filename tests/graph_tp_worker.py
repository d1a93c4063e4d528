"""Ranks of tests/test_graph_tp.py: every rank partitions BERT-tiny for itself, runs its shard on the CPU device and
compares with the unpartitioned model (gloo all-reduce between the ranks). With OVB_GRAPH_TP_DEVICE=CUDA the shards run on
one GPU per rank and the AllReduce nodes use the package's peer-memory all-reduce."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import openvino_b200 as ov   # noqa: E402
from openvino_b200 import _ovcore as _c   # noqa: E402
from openvino_b200.models.torch_zoo import bert_tiny   # noqa: E402
from openvino_b200.parallel.graph_tp import tensor_parallel_partition   # noqa: E402


def main():
    on_gpu = os.environ.get("OVB_GRAPH_TP_DEVICE", "CPU") == "CUDA"
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if on_gpu else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    net = bert_tiny().eval()
    ids = torch.randint(0, 100, (2, 16))
    mask = torch.ones(2, 16, dtype=torch.int64)
    typ = torch.zeros(2, 16, dtype=torch.int64)
    with torch.no_grad():
        want = net(ids, mask, typ).numpy()
    m = ov.convert_model(net, example_input=(ids, mask, typ))
    rm = m.clone()
    _c.run_moc_transformations(rm._m, True)
    _c.run_llm_fusions(rm._m)
    n_fc = sum(1 for n in rm.get_ops() if n.get_type_name() == "FullyConnected")
    inserted = tensor_parallel_partition(rm, rank, world)
    layers = sum(1 for n in rm.get_ops() if n.get_type_name() == "ScaledDotProductAttention")
    assert inserted == 2 * layers, (inserted, layers)
    # every sharded weight is 1/world of the original
    sizes = sorted(int(np.prod(n.input_value(1).get_shape())) for n in rm.get_ops() if n.get_type_name() == "FullyConnected")
    assert len(sizes) == n_fc
    device = "CUDA.%d" % torch.cuda.current_device() if on_gpu else "CPU"
    out = ov.compile_model(rm, device)([ids.numpy(), mask.numpy(), typ.numpy()])[0]
    err = np.linalg.norm(out - want) / np.linalg.norm(want)
    assert err < (2e-2 if on_gpu else 1e-4), err
    if on_gpu:
        from openvino_b200.runtime import cuda_plugin
        assert cuda_plugin._GRAPH_COMMS, "the AllReduce nodes did not use the peer-memory communicator"
    dist.barrier()
    if rank == 0:
        print("GRAPH_TP_OK world=%d all_reduces=%d err=%.2e" % (world, inserted, err))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
