"""Host and device topology queries.

CPU side: the native core reads sysfs (sockets, NUMA nodes, physical / hyper-threaded / efficient cores, ISA flags) and
derives stream counts from a performance hint - the queries of ``openvino.runtime`` system_conf
(src/inference/dev_api/openvino/runtime/system_conf.hpp: get_number_of_cpu_cores, get_num_numa_nodes,
with_cpu_x86_avx2, get_proc_type_table ...). GPU side: the CUDA devices of this process with memory, SM count and the
peer-access matrix that the tensor-parallel communicator needs.
"""
from __future__ import annotations

from typing import Dict, List

from .. import _ovcore as _c

ALL_PROC, MAIN_CORE_PROC, EFFICIENT_CORE_PROC, HYPER_THREADING_PROC, PROC_NUMA_NODE_ID, PROC_SOCKET_ID = range(6)


def cpu_topology(root: str = "/"):
    """Topology of the machine (``root`` lets tests point at a directory that mimics /sys and /proc)."""
    return _c.host_cpu_topology() if root == "/" else _c.read_cpu_topology(root)


def get_number_of_cpu_cores(big_cores_only: bool = False) -> int:
    t = cpu_topology()
    row = t.proc_type_table[0]
    return row[MAIN_CORE_PROC] if big_cores_only else row[MAIN_CORE_PROC] + row[EFFICIENT_CORE_PROC]


def get_number_of_logical_cpu_cores(big_cores_only: bool = False) -> int:
    row = cpu_topology().proc_type_table[0]
    return row[MAIN_CORE_PROC] + row[HYPER_THREADING_PROC] if big_cores_only else row[ALL_PROC]


def get_num_numa_nodes() -> int:
    return cpu_topology().numa_nodes


def get_num_sockets() -> int:
    return cpu_topology().sockets


def get_proc_type_table() -> List[List[int]]:
    return [list(r) for r in cpu_topology().proc_type_table]


def is_cpu_map_available() -> bool:
    return len(cpu_topology().cpu_mapping_table) > 0


def _flag(*names) -> bool:
    t = cpu_topology()
    return any(t.has(n) for n in names)


def with_cpu_x86_sse42() -> bool: return _flag("sse4_2")
def with_cpu_x86_avx() -> bool: return _flag("avx")
def with_cpu_x86_avx2() -> bool: return _flag("avx2")
def with_cpu_x86_avx512f() -> bool: return _flag("avx512f")
def with_cpu_x86_avx512_core() -> bool: return _flag("avx512f") and _flag("avx512bw") and _flag("avx512vl") and _flag("avx512dq")
def with_cpu_x86_avx512_core_vnni() -> bool: return with_cpu_x86_avx512_core() and _flag("avx512_vnni")
def with_cpu_x86_bfloat16() -> bool: return _flag("avx512_bf16")
def with_cpu_x86_avx512_core_amx() -> bool: return _flag("amx_tile") and _flag("amx_int8", "amx_bf16")
def with_cpu_neon_fp16() -> bool: return _flag("asimdhp", "fphp")
def with_cpu_sve() -> bool: return _flag("sve")


def streams_for_hint(hint: str = "LATENCY", num_streams: int = 0, num_threads: int = 0, root: str = "/"):
    """-> (streams, threads per stream) the CPU device uses for ``PERFORMANCE_HINT=hint``."""
    return _c.plan_streams(cpu_topology(root), str(hint), int(num_streams), int(num_threads))


def gpu_topology() -> List[Dict]:
    """One entry per visible CUDA device: name, memory, SM count, compute capability and which peers it can map."""
    import sys
    torch = sys.modules.get("torch")
    if torch is None:
        import torch
    if not torch.cuda.is_available():
        return []
    n = torch.cuda.device_count()
    out = []
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        peers = [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)]
        out.append(dict(index=i, name=p.name, total_memory=p.total_memory, multi_processor_count=p.multi_processor_count,
                        compute_capability=(p.major, p.minor), peers=peers))
    return out
