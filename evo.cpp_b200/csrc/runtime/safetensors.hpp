// Strict read-only view of an evo2-runtime-v1 Safetensors artifact: a single
// .safetensors file or a sharded directory / model.safetensors.index.json.
// Follows upstream's container contract (docs/model-format.md:31-127,
// src/model_format.cpp): 8-byte little-endian header length, JSON header,
// dense payload with contiguous non-overlapping tensors, dtypes F32 / BF16 /
// F8_E4M3, typed string metadata with s:/u:/f:/b:/l:/x: prefixes.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace evob {

enum class TensorType { kF32, kBF16, kE4M3 };

struct TensorView {
  std::string name;
  TensorType type = TensorType::kF32;
  std::vector<std::size_t> shape;
  const unsigned char *data = nullptr;
  std::size_t bytes = 0;
  std::size_t elements() const {
    std::size_t n = 1;
    for (const std::size_t d : shape) n *= d;
    return n;
  }
};

class ModelFile {
 public:
  ~ModelFile();
  ModelFile(const ModelFile &) = delete;
  ModelFile &operator=(const ModelFile &) = delete;

  // Returns evo_status; message through evob::last_error().
  static int open(const std::string &path, std::shared_ptr<ModelFile> *out);

  const TensorView *find(const std::string &name) const;
  const std::vector<TensorView> &tensors() const { return tensors_; }
  const std::string *metadata(const std::string &key) const;
  std::size_t payload_bytes() const { return payload_bytes_; }

  // Typed metadata accessors; missing key or wrong prefix -> kModelFormat.
  int get_string(const std::string &key, std::string *out) const;
  int get_u64(const std::string &key, std::size_t *out) const;
  int get_f64(const std::string &key, double *out) const;
  int get_bool(const std::string &key, bool *out) const;
  int get_list(const std::string &key, std::vector<std::size_t> *out) const;

 private:
  ModelFile() = default;
  int open_shard(const std::string &path, bool first);
  struct Mapping {
    void *address = nullptr;
    std::size_t length = 0;
  };
  std::vector<Mapping> mappings_;
  std::vector<TensorView> tensors_;
  std::map<std::string, std::size_t> index_;
  std::map<std::string, std::string> metadata_;
  std::size_t payload_bytes_ = 0;
};

}  // namespace evob
