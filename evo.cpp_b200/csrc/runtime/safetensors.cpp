#include "safetensors.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>

#include "../common.cuh"

namespace evob {
namespace {

// ---- a small JSON reader (objects, arrays, strings, integers, literals)
struct Json {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool boolean = false;
  double number = 0;
  std::string text;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> members;  // insertion order
  const Json *get(const std::string &key) const {
    for (const auto &m : members)
      if (m.first == key) return &m.second;
    return nullptr;
  }
};

class JsonParser {
 public:
  JsonParser(const char *begin, const char *end) : p_(begin), end_(end) {}
  bool parse(Json *out) {
    skip();
    if (!value(out, 0)) return false;
    skip();
    return p_ == end_;
  }

 private:
  const char *p_, *end_;
  void skip() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool literal(const char *word) {
    const std::size_t n = std::strlen(word);
    if (static_cast<std::size_t>(end_ - p_) < n || std::memcmp(p_, word, n) != 0) return false;
    p_ += n;
    return true;
  }
  bool string(std::string *out) {
    if (p_ >= end_ || *p_ != '"') return false;
    ++p_;
    out->clear();
    while (p_ < end_ && *p_ != '"') {
      if (*p_ == '\\') {
        if (++p_ >= end_) return false;
        switch (*p_) {
          case '"': out->push_back('"'); break;
          case '\\': out->push_back('\\'); break;
          case '/': out->push_back('/'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'n': out->push_back('\n'); break;
          case 'r': out->push_back('\r'); break;
          case 't': out->push_back('\t'); break;
          case 'u': {
            if (end_ - p_ < 5) return false;
            unsigned code = 0;
            for (int i = 1; i <= 4; ++i) {
              const char c = p_[i];
              code <<= 4;
              if (c >= '0' && c <= '9') code |= c - '0';
              else if (c >= 'a' && c <= 'f') code |= c - 'a' + 10;
              else if (c >= 'A' && c <= 'F') code |= c - 'A' + 10;
              else return false;
            }
            p_ += 4;
            if (code < 0x80) out->push_back(static_cast<char>(code));
            else if (code < 0x800) {
              out->push_back(static_cast<char>(0xc0 | (code >> 6)));
              out->push_back(static_cast<char>(0x80 | (code & 0x3f)));
            } else {
              out->push_back(static_cast<char>(0xe0 | (code >> 12)));
              out->push_back(static_cast<char>(0x80 | ((code >> 6) & 0x3f)));
              out->push_back(static_cast<char>(0x80 | (code & 0x3f)));
            }
            break;
          }
          default: return false;
        }
        ++p_;
      } else {
        out->push_back(*p_++);
      }
    }
    if (p_ >= end_) return false;
    ++p_;
    return true;
  }
  bool value(Json *out, const int depth) {
    if (depth > 16 || p_ >= end_) return false;
    if (*p_ == '{') {
      out->kind = Json::kObject;
      ++p_;
      skip();
      if (p_ < end_ && *p_ == '}') { ++p_; return true; }
      for (;;) {
        std::string key;
        skip();
        if (!string(&key)) return false;
        skip();
        if (p_ >= end_ || *p_ != ':') return false;
        ++p_;
        skip();
        Json member;
        if (!value(&member, depth + 1)) return false;
        out->members.emplace_back(std::move(key), std::move(member));
        skip();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == '}') { ++p_; return true; }
        return false;
      }
    }
    if (*p_ == '[') {
      out->kind = Json::kArray;
      ++p_;
      skip();
      if (p_ < end_ && *p_ == ']') { ++p_; return true; }
      for (;;) {
        Json item;
        skip();
        if (!value(&item, depth + 1)) return false;
        out->items.push_back(std::move(item));
        skip();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == ']') { ++p_; return true; }
        return false;
      }
    }
    if (*p_ == '"') {
      out->kind = Json::kString;
      return string(&out->text);
    }
    if (literal("true")) { out->kind = Json::kBool; out->boolean = true; return true; }
    if (literal("false")) { out->kind = Json::kBool; return true; }
    if (literal("null")) { out->kind = Json::kNull; return true; }
    const char *start = p_;
    while (p_ < end_ && (std::strchr("+-0123456789.eE", *p_) != nullptr)) ++p_;
    if (p_ == start) return false;
    out->kind = Json::kNumber;
    out->number = std::strtod(std::string(start, p_).c_str(), nullptr);
    return true;
  }
};

bool ends_with(const std::string &s, const std::string &suffix) {
  return s.size() >= suffix.size() &&
         s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

bool is_directory(const std::string &path) {
  struct stat st;
  return stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

std::string directory_of(const std::string &path) {
  const std::size_t slash = path.find_last_of('/');
  return slash == std::string::npos ? "." : path.substr(0, slash);
}

}  // namespace

ModelFile::~ModelFile() {
  for (const Mapping &m : mappings_)
    if (m.address != nullptr) munmap(m.address, m.length);
}

int ModelFile::open_shard(const std::string &path, const bool first) {
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) return fail(kIo, "cannot open model file: " + path);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) {
    ::close(fd);
    return fail(kModelFormat, "model file is truncated: " + path);
  }
  const std::size_t length = static_cast<std::size_t>(st.st_size);
  void *address = mmap(nullptr, length, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (address == MAP_FAILED) return fail(kIo, "cannot map model file: " + path);
  mappings_.push_back({address, length});
  const auto *bytes = static_cast<const unsigned char *>(address);
  std::uint64_t header_length = 0;
  for (int i = 0; i < 8; ++i) header_length |= static_cast<std::uint64_t>(bytes[i]) << (8 * i);
  if (header_length == 0 || header_length > length - 8 || header_length % 8 != 0 ||
      header_length > (1ULL << 28))
    return fail(kModelFormat, "Safetensors header length is invalid: " + path);
  Json header;
  const char *json_begin = reinterpret_cast<const char *>(bytes + 8);
  if (!JsonParser(json_begin, json_begin + header_length).parse(&header) ||
      header.kind != Json::kObject)
    return fail(kModelFormat, "Safetensors header is not valid JSON: " + path);
  const unsigned char *payload = bytes + 8 + header_length;
  const std::size_t payload_length = length - 8 - header_length;

  std::map<std::string, std::string> shard_metadata;
  struct Entry { TensorView view; std::size_t begin, end; };
  std::vector<Entry> entries;
  for (const auto &[name, value] : header.members) {
    if (name == "__metadata__") {
      if (value.kind != Json::kObject)
        return fail(kModelFormat, "Safetensors __metadata__ must be an object");
      for (const auto &[key, item] : value.members) {
        if (item.kind != Json::kString)
          return fail(kModelFormat, "Safetensors metadata values must be strings");
        shard_metadata[key] = item.text;
      }
      continue;
    }
    const Json *dtype = value.get("dtype"), *shape = value.get("shape"),
               *offsets = value.get("data_offsets");
    if (value.kind != Json::kObject || dtype == nullptr || shape == nullptr ||
        offsets == nullptr || dtype->kind != Json::kString || shape->kind != Json::kArray ||
        offsets->kind != Json::kArray || offsets->items.size() != 2)
      return fail(kModelFormat, "tensor entry is malformed: " + name);
    Entry entry;
    entry.view.name = name;
    std::size_t element = 0;
    if (dtype->text == "F32") { entry.view.type = TensorType::kF32; element = 4; }
    else if (dtype->text == "BF16") { entry.view.type = TensorType::kBF16; element = 2; }
    else if (dtype->text == "F8_E4M3") { entry.view.type = TensorType::kE4M3; element = 1; }
    else return fail(kModelFormat, "unsupported tensor dtype " + dtype->text + ": " + name);
    if (shape->items.empty() || shape->items.size() > 8)
      return fail(kModelFormat, "tensor rank is unsupported: " + name);
    std::size_t elements = 1;
    for (const Json &d : shape->items) {
      if (d.kind != Json::kNumber || d.number < 1 || d.number != static_cast<double>(
                                                          static_cast<std::size_t>(d.number)))
        return fail(kModelFormat, "tensor dimensions must be positive: " + name);
      entry.view.shape.push_back(static_cast<std::size_t>(d.number));
      elements *= entry.view.shape.back();
    }
    entry.begin = static_cast<std::size_t>(offsets->items[0].number);
    entry.end = static_cast<std::size_t>(offsets->items[1].number);
    if (entry.end < entry.begin || entry.end > payload_length ||
        entry.end - entry.begin != elements * element)
      return fail(kModelFormat, "tensor byte range does not match its shape: " + name);
    entry.view.data = payload + entry.begin;
    entry.view.bytes = entry.end - entry.begin;
    entries.push_back(std::move(entry));
  }
  std::sort(entries.begin(), entries.end(),
            [](const Entry &a, const Entry &b) { return a.begin < b.begin; });
  std::size_t cursor = 0;
  for (const Entry &entry : entries) {
    if (entry.begin != cursor)
      return fail(kModelFormat, "tensor payload has a hole or an overlap at " + entry.view.name);
    cursor = entry.end;
  }
  if (cursor != payload_length)
    return fail(kModelFormat, "model file has trailing or missing payload bytes: " + path);
  if (first) metadata_ = shard_metadata;
  else if (shard_metadata != metadata_)
    return fail(kModelFormat, "shard metadata differs between files");
  for (Entry &entry : entries) {
    if (index_.count(entry.view.name) != 0)
      return fail(kModelFormat, "tensor appears twice: " + entry.view.name);
    index_[entry.view.name] = tensors_.size();
    tensors_.push_back(std::move(entry.view));
  }
  payload_bytes_ += payload_length;
  return kOk;
}

int ModelFile::open(const std::string &path, std::shared_ptr<ModelFile> *out) {
  if (out == nullptr || path.empty()) return fail(kInvalidArgument, "model path is empty");
  std::shared_ptr<ModelFile> file(new ModelFile());
  std::string index_path;
  if (is_directory(path)) {
    struct stat st;
    if (stat((path + "/model.safetensors.index.json").c_str(), &st) == 0)
      index_path = path + "/model.safetensors.index.json";
    else {
      const int status = file->open_shard(path + "/model.safetensors", true);
      if (status != kOk) return status;
    }
  } else if (ends_with(path, ".index.json")) {
    index_path = path;
  } else {
    const int status = file->open_shard(path, true);
    if (status != kOk) return status;
  }
  if (!index_path.empty()) {
    std::ifstream stream(index_path);
    if (!stream) return fail(kIo, "cannot open model index: " + index_path);
    std::stringstream buffer;
    buffer << stream.rdbuf();
    const std::string text = buffer.str();
    Json index;
    if (!JsonParser(text.data(), text.data() + text.size()).parse(&index) ||
        index.kind != Json::kObject)
      return fail(kModelFormat, "model index is not valid JSON");
    const Json *map = index.get("weight_map");
    if (map == nullptr || map->kind != Json::kObject || map->members.empty())
      return fail(kModelFormat, "model index has no weight_map");
    std::vector<std::string> shards;
    for (const auto &[name, shard] : map->members) {
      if (shard.kind != Json::kString || shard.text.find('/') != std::string::npos)
        return fail(kModelFormat, "model index shard name is invalid");
      if (std::find(shards.begin(), shards.end(), shard.text) == shards.end())
        shards.push_back(shard.text);
    }
    std::sort(shards.begin(), shards.end());
    const std::string base = directory_of(index_path);
    for (std::size_t i = 0; i < shards.size(); ++i) {
      const int status = file->open_shard(base + "/" + shards[i], i == 0);
      if (status != kOk) return status;
    }
    for (const auto &[name, shard] : map->members)
      if (file->index_.count(name) == 0)
        return fail(kModelFormat, "indexed tensor is missing from its shard: " + name);
    if (map->members.size() != file->tensors_.size())
      return fail(kModelFormat, "shards hold tensors the index does not list");
    const Json *meta = index.get("metadata");
    const Json *total = meta != nullptr ? meta->get("total_size") : nullptr;
    if (total != nullptr && total->kind == Json::kNumber &&
        static_cast<std::size_t>(total->number) != file->payload_bytes_)
      return fail(kModelFormat, "model index total_size does not match the shards");
  }
  *out = std::move(file);
  return kOk;
}

const TensorView *ModelFile::find(const std::string &name) const {
  const auto it = index_.find(name);
  return it == index_.end() ? nullptr : &tensors_[it->second];
}

const std::string *ModelFile::metadata(const std::string &key) const {
  const auto it = metadata_.find(key);
  return it == metadata_.end() ? nullptr : &it->second;
}

namespace {
int typed(const ModelFile &file, const std::string &key, const char prefix,
          std::string *payload) {
  const std::string *raw = file.metadata(key);
  if (raw == nullptr) return fail(kModelFormat, "required metadata is missing: " + key);
  if (raw->size() < 2 || (*raw)[0] != prefix || (*raw)[1] != ':')
    return fail(kModelFormat, "metadata has the wrong type: " + key);
  *payload = raw->substr(2);
  return kOk;
}
bool parse_u64(const std::string &text, std::size_t *out) {
  if (text.empty() || text.size() > 20 || (text.size() > 1 && text[0] == '0')) return false;
  std::size_t value = 0;
  for (const char c : text) {
    if (c < '0' || c > '9') return false;
    value = value * 10 + static_cast<std::size_t>(c - '0');
  }
  *out = value;
  return true;
}
}  // namespace

int ModelFile::get_string(const std::string &key, std::string *out) const {
  return typed(*this, key, 's', out);
}
int ModelFile::get_u64(const std::string &key, std::size_t *out) const {
  std::string text;
  const int status = typed(*this, key, 'u', &text);
  if (status != kOk) return status;
  if (!parse_u64(text, out)) return fail(kModelFormat, "metadata is not a canonical integer: " + key);
  return kOk;
}
int ModelFile::get_f64(const std::string &key, double *out) const {
  std::string text;
  const int status = typed(*this, key, 'f', &text);
  if (status != kOk) return status;
  if (text.size() != 16) return fail(kModelFormat, "metadata is not an F64 bit pattern: " + key);
  std::uint64_t bits = 0;
  for (const char c : text) {
    bits <<= 4;
    if (c >= '0' && c <= '9') bits |= static_cast<std::uint64_t>(c - '0');
    else if (c >= 'a' && c <= 'f') bits |= static_cast<std::uint64_t>(c - 'a' + 10);
    else return fail(kModelFormat, "metadata is not an F64 bit pattern: " + key);
  }
  std::memcpy(out, &bits, 8);
  return kOk;
}
int ModelFile::get_bool(const std::string &key, bool *out) const {
  std::string text;
  const int status = typed(*this, key, 'b', &text);
  if (status != kOk) return status;
  if (text != "0" && text != "1") return fail(kModelFormat, "metadata is not a boolean: " + key);
  *out = text == "1";
  return kOk;
}
int ModelFile::get_list(const std::string &key, std::vector<std::size_t> *out) const {
  std::string text;
  const int status = typed(*this, key, 'l', &text);
  if (status != kOk) return status;
  out->clear();
  if (text.empty()) return kOk;
  std::size_t start = 0;
  while (start <= text.size()) {
    const std::size_t comma = text.find(',', start);
    const std::string item = text.substr(start, comma == std::string::npos ? std::string::npos : comma - start);
    std::size_t value = 0;
    if (!parse_u64(item, &value)) return fail(kModelFormat, "metadata is not an integer list: " + key);
    out->push_back(value);
    if (comma == std::string::npos) break;
    start = comma + 1;
  }
  return kOk;
}

}  // namespace evob
