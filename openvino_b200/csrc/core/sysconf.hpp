// Host CPU topology: sockets, NUMA nodes, physical cores, hyper-threads, core types, ISA flags.
//
// Role of src/inference/src/os/lin/lin_system_conf.cpp (parse_processor_info_linux, the proc_type_table / cpu_mapping_table
// pair) and src/inference/src/system_conf.cpp (with_cpu_x86_* and get_number_of_* queries). The tables are built from a
// sysfs-style directory tree so that tests can describe a machine with plain files.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace ovc {

// columns of a proc_type_table row
enum ProcCol { ALL_PROC = 0, MAIN_CORE_PROC, EFFICIENT_CORE_PROC, HYPER_THREADING_PROC, PROC_NUMA_NODE_ID, PROC_SOCKET_ID, PROC_TABLE_COLS };
// columns of a cpu_mapping_table row
enum CpuCol { CPU_MAP_PROCESSOR_ID = 0, CPU_MAP_NUMA_NODE_ID, CPU_MAP_SOCKET_ID, CPU_MAP_CORE_ID, CPU_MAP_CORE_TYPE, CPU_MAP_GROUP_ID, CPU_MAP_USED_FLAG, CPU_MAP_COLS };

struct CpuTopology {
    int sockets = 0, numa_nodes = 0, cores = 0, processors = 0;
    std::vector<std::vector<int>> proc_type_table;   // row 0: whole machine; then one row per (socket, numa node) when there are several
    std::vector<std::vector<int>> cpu_mapping_table; // one row per logical processor
    std::vector<std::string> flags;                  // ISA flags of /proc/cpuinfo ("avx2", "avx512f", "amx_tile", ...)
    bool has(const std::string& flag) const;
};

// `root` is "/" on a real machine: files read are <root>/sys/devices/system/cpu/{online,cpuN/topology/*,cpuN/cpufreq/cpuinfo_max_freq},
// <root>/sys/devices/system/node/nodeN/cpulist and <root>/proc/cpuinfo.
CpuTopology read_cpu_topology(const std::string& root = "/");
const CpuTopology& host_cpu_topology();              // cached read of the running machine
std::vector<int> parse_cpu_list(const std::string& s);   // "0-3,8,10-11" -> {0,1,2,3,8,10,11}

// Streams for a performance hint: LATENCY -> one stream over the cores of one socket; THROUGHPUT -> streams of `threads_per_stream`
// physical cores (reference: get_streams_info_table, src/plugins/intel_cpu/src/cpu_streams_calculation.cpp).
struct StreamsPlan { int num_streams = 1; int threads_per_stream = 1; };
StreamsPlan plan_streams(const CpuTopology& t, const std::string& hint, int requested_streams, int requested_threads);

}  // namespace ovc
