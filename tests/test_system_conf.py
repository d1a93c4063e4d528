"""CPU topology tables from a sysfs-like tree; stream planning per performance hint."""
import os

import openvino_b200 as ov
from openvino_b200 import _ovcore as _c
from openvino_b200.runtime import system_conf as sc


def _machine(root, sockets, cores_per_socket, smt, numa_per_socket=1, little=0, flags="fpu sse4_2 avx avx2 avx512f"):
    """Write /sys + /proc files of a machine: processor ids are socket-major, hyper-thread siblings in the upper half."""
    cpu = root / "sys/devices/system/cpu"
    node = root / "sys/devices/system/node"
    n_cores = sockets * cores_per_socket
    total = n_cores * smt
    (cpu).mkdir(parents=True)
    (cpu / "online").write_text("0-%d\n" % (total - 1))
    numa = {}
    for p in range(total):
        core = p % n_cores
        s = core // cores_per_socket
        d = cpu / ("cpu%d" % p)
        (d / "topology").mkdir(parents=True)
        (d / "cpufreq").mkdir()
        (d / "topology/physical_package_id").write_text("%d\n" % s)
        (d / "topology/core_id").write_text("%d\n" % (core % cores_per_socket))
        is_little = (core % cores_per_socket) >= cores_per_socket - little
        (d / "cpufreq/cpuinfo_max_freq").write_text("%d\n" % (2600000 if is_little else 5000000))
        per_node = cores_per_socket // numa_per_socket
        numa.setdefault(s * numa_per_socket + (core % cores_per_socket) // per_node, []).append(p)
    for k, procs in numa.items():
        (node / ("node%d" % k)).mkdir(parents=True)
        (node / ("node%d" % k) / "cpulist").write_text(",".join(map(str, procs)) + "\n")
    (root / "proc").mkdir()
    (root / "proc/cpuinfo").write_text("processor\t: 0\nflags\t\t: %s\n" % flags)
    return str(root)


def test_two_socket_server_with_smt(tmp_path):
    root = _machine(tmp_path, sockets=2, cores_per_socket=16, smt=2, numa_per_socket=2)
    t = _c.read_cpu_topology(root)
    assert (t.sockets, t.numa_nodes, t.cores, t.processors) == (2, 4, 32, 64)
    total = t.proc_type_table[0]
    assert total[sc.ALL_PROC] == 64 and total[sc.MAIN_CORE_PROC] == 32 and total[sc.HYPER_THREADING_PROC] == 32 and total[sc.EFFICIENT_CORE_PROC] == 0
    assert total[sc.PROC_NUMA_NODE_ID] == -1 and total[sc.PROC_SOCKET_ID] == -1
    rows = t.proc_type_table[1:]
    assert len(rows) == 4 and all(r[sc.ALL_PROC] == 16 and r[sc.MAIN_CORE_PROC] == 8 for r in rows)
    assert sorted((r[sc.PROC_SOCKET_ID], r[sc.PROC_NUMA_NODE_ID]) for r in rows) == [(0, 0), (0, 1), (1, 2), (1, 3)]
    assert len(t.cpu_mapping_table) == 64 and t.has("avx512f") and not t.has("amx_tile")
    # LATENCY: one stream on one socket's cores; THROUGHPUT: streams of four cores
    assert sc.streams_for_hint("LATENCY", root=root) == (1, 16)
    assert sc.streams_for_hint("THROUGHPUT", root=root) == (8, 4)
    assert sc.streams_for_hint("THROUGHPUT", num_streams=3, root=root) == (3, 10)


def test_hybrid_client_cpu(tmp_path):
    root = _machine(tmp_path, sockets=1, cores_per_socket=12, smt=1, little=4)
    t = _c.read_cpu_topology(root)
    total = t.proc_type_table[0]
    assert total[sc.MAIN_CORE_PROC] == 8 and total[sc.EFFICIENT_CORE_PROC] == 4 and len(t.proc_type_table) == 1
    assert total[sc.PROC_SOCKET_ID] == 0


def test_host_queries_and_cpu_list():
    assert _c.parse_cpu_list("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    assert sc.get_number_of_logical_cpu_cores() >= sc.get_number_of_cpu_cores() >= 1
    assert sc.get_num_numa_nodes() >= 1 and sc.get_num_sockets() >= 1
    assert isinstance(sc.with_cpu_x86_avx2(), bool) and sc.is_cpu_map_available()
    assert isinstance(sc.gpu_topology(), list)
