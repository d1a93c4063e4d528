// IR (.xml/.bin) serialisation entry points of the native core.
#pragma once
#include "graph.hpp"

namespace ovc {

struct SerializeOptions {
    int version = 11;
    bool deterministic = false;   // omit names (used for hashing / cache keys)
};

void serialize_model(const Model& m, std::string& xml, std::string& bin, const SerializeOptions& opt = {});
ModelPtr deserialize_model(const std::string& xml, BufferPtr weights);
ModelPtr read_model_files(const std::string& xml_path, const std::string& bin_path = "");
void save_model_files(const Model& m, const std::string& xml_path, const std::string& bin_path = "", const SerializeOptions& opt = {});
uint64_t model_hash(const Model& m);

}  // namespace ovc
