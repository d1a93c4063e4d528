#include "sysconf.hpp"

#include <algorithm>
#include <fstream>
#include <mutex>
#include <set>
#include <sstream>
#include <thread>

namespace ovc {

namespace {

bool read_line(const std::string& path, std::string& out) {
    std::ifstream f(path);
    if (!f) return false;
    std::getline(f, out);
    return true;
}
bool read_int(const std::string& path, long& v) {
    std::string s;
    if (!read_line(path, s) || s.empty()) return false;
    try { v = std::stol(s); } catch (...) { return false; }
    return true;
}

}  // namespace

std::vector<int> parse_cpu_list(const std::string& s) {
    std::vector<int> out;
    std::stringstream ss(s);
    std::string part;
    while (std::getline(ss, part, ',')) {
        if (part.empty()) continue;
        const size_t dash = part.find('-');
        try {
            if (dash == std::string::npos) out.push_back(std::stoi(part));
            else for (int i = std::stoi(part.substr(0, dash)), e = std::stoi(part.substr(dash + 1)); i <= e; ++i) out.push_back(i);
        } catch (...) {}
    }
    return out;
}

bool CpuTopology::has(const std::string& flag) const { return std::find(flags.begin(), flags.end(), flag) != flags.end(); }

CpuTopology read_cpu_topology(const std::string& root_in) {
    std::string root = root_in;
    if (!root.empty() && root.back() == '/') root.pop_back();
    const std::string cpu_dir = root + "/sys/devices/system/cpu";
    CpuTopology t;
    std::string online;
    std::vector<int> cpus;
    if (read_line(cpu_dir + "/online", online)) cpus = parse_cpu_list(online);
    if (cpus.empty()) {                       // no sysfs: fall back to the processor count
        const int n = std::max(1u, std::thread::hardware_concurrency());
        for (int i = 0; i < n; ++i) cpus.push_back(i);
    }
    // NUMA node of every processor
    std::map<int, int> numa_of;
    for (int node = 0; node < 1024; ++node) {
        std::string list;
        if (!read_line(root + "/sys/devices/system/node/node" + std::to_string(node) + "/cpulist", list)) {
            if (node > 8 && numa_of.empty()) break;
            if (node > 64) break;
            continue;
        }
        for (int c : parse_cpu_list(list)) numa_of[c] = node;
    }
    // per processor: socket, core id, max frequency (core type: the fastest class is "main", slower ones "efficient")
    struct P { int id, socket, core, numa; long freq; };
    std::vector<P> procs;
    long max_freq = 0;
    for (int c : cpus) {
        P p{c, 0, c, numa_of.count(c) ? numa_of[c] : 0, 0};
        long v;
        const std::string base = cpu_dir + "/cpu" + std::to_string(c);
        if (read_int(base + "/topology/physical_package_id", v)) p.socket = (int)std::max(0l, v);
        if (read_int(base + "/topology/core_id", v)) p.core = (int)v;
        if (read_int(base + "/cpufreq/cpuinfo_max_freq", v)) p.freq = v;
        max_freq = std::max(max_freq, p.freq);
        procs.push_back(p);
    }
    std::set<int> sockets, numas;
    std::map<std::pair<int, int>, int> first_of_core;     // (socket, core) -> dense core index
    for (auto& p : procs) {
        sockets.insert(p.socket);
        numas.insert(p.numa);
    }
    t.sockets = (int)sockets.size();
    t.numa_nodes = (int)numas.size();
    t.processors = (int)procs.size();
    // rows: [0] total, then per (socket, numa) group when more than one group exists
    std::map<std::pair<int, int>, std::vector<int>> groups;
    for (auto& p : procs) {
        const auto key = std::make_pair(p.socket, p.core);
        const bool first = !first_of_core.count(key);
        if (first) first_of_core[key] = (int)first_of_core.size();
        const bool efficient = max_freq > 0 && p.freq > 0 && p.freq * 100 < max_freq * 80;   // clearly slower class of core
        const int type = first ? (efficient ? EFFICIENT_CORE_PROC : MAIN_CORE_PROC) : HYPER_THREADING_PROC;
        t.cpu_mapping_table.push_back({p.id, p.numa, p.socket, first_of_core[key], type, first_of_core[key], -1});
        auto& row = groups[{p.socket, p.numa}];
        if (row.empty()) row.assign(PROC_TABLE_COLS, 0);
        row[ALL_PROC] += 1;
        row[type] += 1;
        row[PROC_NUMA_NODE_ID] = p.numa;
        row[PROC_SOCKET_ID] = p.socket;
    }
    t.cores = (int)first_of_core.size();
    std::vector<int> total(PROC_TABLE_COLS, 0);
    for (auto& g : groups)
        for (int c = ALL_PROC; c <= HYPER_THREADING_PROC; ++c) total[c] += g.second[c];
    total[PROC_NUMA_NODE_ID] = groups.size() > 1 ? -1 : groups.begin()->second[PROC_NUMA_NODE_ID];
    total[PROC_SOCKET_ID] = groups.size() > 1 ? -1 : groups.begin()->second[PROC_SOCKET_ID];
    t.proc_type_table.push_back(total);
    if (groups.size() > 1)
        for (auto& g : groups) t.proc_type_table.push_back(g.second);
    // ISA flags
    std::ifstream ci(root + "/proc/cpuinfo");
    std::string line;
    while (std::getline(ci, line)) {
        if (line.rfind("flags", 0) == 0 || line.rfind("Features", 0) == 0) {
            const size_t colon = line.find(':');
            std::stringstream ss(colon == std::string::npos ? "" : line.substr(colon + 1));
            std::string f;
            while (ss >> f) t.flags.push_back(f);
            break;
        }
    }
    return t;
}

const CpuTopology& host_cpu_topology() {
    static CpuTopology t;
    static std::once_flag once;
    std::call_once(once, [] { t = read_cpu_topology("/"); });
    return t;
}

StreamsPlan plan_streams(const CpuTopology& t, const std::string& hint, int requested_streams, int requested_threads) {
    StreamsPlan p;
    const auto& total = t.proc_type_table.at(0);
    int cores = total[MAIN_CORE_PROC] + total[EFFICIENT_CORE_PROC];
    if (cores <= 0) cores = std::max(1, t.processors);
    if (requested_threads > 0) cores = std::min(cores, requested_threads);
    if (requested_streams > 0) {
        p.num_streams = std::min(requested_streams, cores);
        p.threads_per_stream = std::max(1, cores / p.num_streams);
        return p;
    }
    if (hint == "THROUGHPUT" || hint == "CUMULATIVE_THROUGHPUT") {
        // streams of four cores (at least one stream per NUMA node)
        const int per = cores >= 8 ? 4 : (cores >= 4 ? 2 : 1);
        p.num_streams = std::max(std::max(1, t.numa_nodes), cores / per);
        p.threads_per_stream = std::max(1, cores / p.num_streams);
    } else {
        // LATENCY: one stream on the cores of one socket (crossing sockets costs more than it brings)
        int socket_cores = cores;
        if (t.proc_type_table.size() > 1) {
            std::map<int, int> per_socket;
            for (size_t r = 1; r < t.proc_type_table.size(); ++r)
                per_socket[t.proc_type_table[r][PROC_SOCKET_ID]] += t.proc_type_table[r][MAIN_CORE_PROC] + t.proc_type_table[r][EFFICIENT_CORE_PROC];
            socket_cores = 0;
            for (auto& kv : per_socket) socket_cores = std::max(socket_cores, kv.second);
        }
        p.num_streams = 1;
        p.threads_per_stream = std::max(1, std::min(cores, socket_cores));
    }
    return p;
}

}  // namespace ovc
