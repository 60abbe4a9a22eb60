// Shared host-side declarations of the puppygrad_b200 library.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "puppygrad_b200.h"

namespace pg {

// Stores the message for pg_last_error_message() on this thread and returns `code`.
int set_error(int code, const std::string& msg);
void clear_error();
const char* last_error_cstr();

// ---- minimal JSON value (config.json and the safetensors header) ----
struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  bool num_is_integer = false;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* get(const std::string& key) const;
};
// Returns false and fills `err` on malformed input.
bool parse_json(const char* data, size_t len, Json* out, std::string* err);

// ---- safetensors container (the format of the `safetensors` crate, version 0.7.0) ----
struct TensorEntry {
  std::string dtype;
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;  // byte offsets into the data section
};
struct SafeTensorsFile {
  std::vector<uint8_t> bytes;   // whole file
  size_t data_start = 0;        // offset of the data section
  std::map<std::string, TensorEntry> tensors;
  const uint8_t* data(const TensorEntry& e) const { return bytes.data() + data_start + e.begin; }
};
// Reads and parses `path`. Errors are returned as PG_ASSET with a message.
int read_safetensors(const std::string& path, SafeTensorsFile* out);

// ---- config ----
int validate_config(const pg_gpt2_config& cfg);
int load_config_json(const std::string& path, pg_gpt2_config* out);

// Host copy of the weights in the ABI's tensor order, with validated lengths.
struct HostWeights {
  std::vector<const float*> ptrs;
  std::vector<uint64_t> lens;
  std::vector<std::vector<float>> owned;  // backing store when loaded from a file
};
int validate_weight_lens(const pg_gpt2_config& cfg, const uint64_t* lens, uint64_t n_tensors);
int load_weights_safetensors(const std::string& path, const pg_gpt2_config& cfg, HostWeights* out);

}  // namespace pg
