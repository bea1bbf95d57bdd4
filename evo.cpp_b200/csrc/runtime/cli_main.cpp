// `evo` command-line driver for the CUDA path: run / score / bench / embed, written
// against the public C ABI only (include/evo/evo.h + evo_b200.h).  Mirrors the
// surface of upstream's CUDA CLI (src/cli.cpp:98-173,
// src/cuda/inference_cli.cpp:199-263, 341-700, 1310-1345): the same
// sub-commands and legacy flag form, score JSONL fields, bench JSONL schema
// (include/evo/benchmark.hpp, src/benchmark.cpp:41-100), raw-byte generation on
// stdout and one `evo_metrics {...}` line on stderr; `embed` writes one NPY v1
// F32 matrix per record plus an embeddings.jsonl manifest into an empty or new
// directory (src/cuda/inference_cli.cpp:278-337, 972-1108).  Exit code = evo_status.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <limits>
#include <memory>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "../../../include/evo/evo.h"
#include "../../../include/evo/evo_b200.h"

namespace {

struct Options {
  std::string command = "run", model, prompt, input, profile = "exact", output_format = "raw",
              name = "generated", output, pooling = "none";
  size_t layer = static_cast<size_t>(-1);
  std::vector<int32_t> gpus{0};
  size_t tokens = 0, context = 4096, warmup = 1, repetitions = 5, top_k = 1;
  float temperature = 1.0F, top_p = 1.0F;
  uint64_t seed = 0;
  bool allow_fixture = false;
  // variant-score: inline (--sequence --position --ref --alt) or file form (--vcf --reference)
  std::string sequence, reference_allele, alternate_allele, strand = "both", normalization = "sum";
  std::string vcf_path, reference_path;
  // serve
  size_t workers = 4, max_queue = 64;
  // generation / scoring diagnostics (upstream src/cli.cpp:166-172): how many prompt tokens the cached
  // prefill takes before the rest is teacher-forced through decode; token, logit and block-output dumps
  size_t force_prompt_threshold = 0;  // 0: not given
  bool dump_tokens = false;
  std::string dump_logits_path, dump_layer_path;
  size_t dump_layer = static_cast<size_t>(-1);
  size_t position = 0, window = 0;
};

struct Record {
  std::string name, format;
  std::string bytes;
};

[[noreturn]] void die(const int code, const std::string &message) {
  std::cerr << "evo: " << message << '\n';
  std::exit(code);
}

void check(const evo_status status, const char *what) {
  if (status != EVO_STATUS_OK) die(static_cast<int>(status), std::string(what) + ": " + evo_last_error());
}

double seconds_since(const std::chrono::steady_clock::time_point start) {
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
}

void json_string(std::ostream &out, const std::string &text) {
  out.put('"');
  for (const unsigned char c : text) {
    if (c == '"' || c == '\\') out << '\\' << c;
    else if (c < 0x20 || c >= 0x7f)  // bytes above ASCII as their Latin-1 code points: the line stays valid UTF-8
      out << "\\u" << std::hex << std::setw(4) << std::setfill('0') << int(c) << std::dec << std::setfill(' ');
    else out.put(static_cast<char>(c));
  }
  out.put('"');
}

// FASTA ('>'), strict four-line FASTQ ('@') or one raw record; CRLF is
// normalised; white space inside a sequence line is an error
// (upstream include/evo/sequence_io.hpp:22-29, docs/sequence-inputs.md:16-33).
std::vector<Record> read_records(const std::string &path, const size_t limit) {
  std::ifstream file(path, std::ios::binary);
  if (!file) die(EVO_STATUS_IO, "cannot open input: " + path);
  std::vector<std::string> lines;
  for (std::string line; std::getline(file, line);) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    lines.push_back(line);
  }
  while (!lines.empty() && lines.back().empty()) lines.pop_back();
  if (lines.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "input holds no sequence");
  const auto validate = [&](const std::string &sequence) {
    for (const unsigned char c : sequence)
      if (c == ' ' || c == '\t') die(EVO_STATUS_INVALID_ARGUMENT, "white space inside a sequence line");
    if (sequence.size() > limit)
      die(EVO_STATUS_INVALID_ARGUMENT, "sequence exceeds --ctx " + std::to_string(limit));
  };
  std::vector<Record> records;
  if (lines[0][0] == '>') {
    for (const std::string &line : lines) {
      if (!line.empty() && line[0] == '>') records.push_back({line.substr(1), "fasta", ""});
      else records.back().bytes += line;
    }
  } else if (lines[0][0] == '@') {
    if (lines.size() % 4 != 0) die(EVO_STATUS_INVALID_ARGUMENT, "FASTQ input is not a multiple of four lines");
    for (size_t i = 0; i < lines.size(); i += 4) {
      if (lines[i].empty() || lines[i][0] != '@' || lines[i + 2].empty() || lines[i + 2][0] != '+' ||
          lines[i + 1].size() != lines[i + 3].size())
        die(EVO_STATUS_INVALID_ARGUMENT, "malformed FASTQ record");
      records.push_back({lines[i].substr(1), "fastq", lines[i + 1]});
    }
  } else {
    Record record{"sequence", "raw", ""};
    for (const std::string &line : lines) record.bytes += line;
    records.push_back(record);
  }
  for (const Record &record : records) {
    if (record.bytes.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "empty sequence record");
    validate(record.bytes);
  }
  return records;
}

uint64_t fnv1a64(const std::string &bytes) {
  uint64_t hash = 1469598103934665603ULL;
  for (const unsigned char c : bytes) {
    hash ^= c;
    hash *= 1099511628211ULL;
  }
  return hash;
}

// Value of `key` in a flat JSON object (one request per line): strings are
// unescaped for \" \\ \n \t \/ and \uXXXX below 0x100, numbers are returned as
// their text.  Returns false when the key is absent.
bool json_field(const std::string &line, const std::string &key, std::string *value) {
  const std::string needle = '"' + key + '"';
  size_t at = 0;
  while ((at = line.find(needle, at)) != std::string::npos) {
    size_t cursor = at + needle.size();
    while (cursor < line.size() && (line[cursor] == ' ' || line[cursor] == '\t')) ++cursor;
    if (cursor >= line.size() || line[cursor] != ':') {
      at += needle.size();
      continue;
    }
    ++cursor;
    while (cursor < line.size() && (line[cursor] == ' ' || line[cursor] == '\t')) ++cursor;
    value->clear();
    if (cursor < line.size() && line[cursor] == '"') {
      for (++cursor; cursor < line.size() && line[cursor] != '"'; ++cursor) {
        if (line[cursor] != '\\' || cursor + 1 >= line.size()) {
          value->push_back(line[cursor]);
          continue;
        }
        const char escaped = line[++cursor];
        if (escaped == 'n') value->push_back('\n');
        else if (escaped == 't') value->push_back('\t');
        else if (escaped == 'u' && cursor + 4 < line.size()) {
          value->push_back(static_cast<char>(std::stoul(line.substr(cursor + 1, 4), nullptr, 16) & 0xffU));
          cursor += 4;
        } else value->push_back(escaped);
      }
    } else {
      while (cursor < line.size() && line[cursor] != ',' && line[cursor] != '}' && line[cursor] != ' ')
        value->push_back(line[cursor++]);
    }
    return true;
  }
  return false;
}

struct Collected {
  std::vector<float> logits;
  size_t rows = 0, columns = 0;
};

evo_status collect(const float *logits, size_t rows, size_t columns, size_t, void *user) {
  auto *sink = static_cast<Collected *>(user);
  sink->logits.insert(sink->logits.end(), logits, logits + rows * columns);
  sink->rows += rows;
  sink->columns = columns;
  return EVO_STATUS_OK;
}

// log-softmax of one target in double precision over F32 logits
// (upstream src/cuda/inference_cli.cpp:199-224).
double log_probability(const float *logits, const size_t vocab, const uint32_t target) {
  float maximum = -std::numeric_limits<float>::infinity();
  for (size_t i = 0; i < vocab; ++i) {
    if (!std::isfinite(logits[i])) die(EVO_STATUS_INTERNAL, "model produced a non-finite score logit");
    maximum = std::max(maximum, logits[i]);
  }
  double normalizer = 0.0;
  for (size_t i = 0; i < vocab; ++i)
    normalizer += std::exp(static_cast<double>(logits[i]) - static_cast<double>(maximum));
  return static_cast<double>(logits[target]) - static_cast<double>(maximum) - std::log(normalizer);
}

struct Matrix {
  std::vector<float> values;
  size_t rows = 0, columns = 0;
};

evo_status collect_matrix(const float *values, size_t rows, size_t columns, size_t, const evo_embedding_result_info *,
                          void *user) {
  auto *matrix = static_cast<Matrix *>(user);
  matrix->values.insert(matrix->values.end(), values, values + rows * columns);
  matrix->rows += rows;
  matrix->columns = columns;
  return EVO_STATUS_OK;
}

// NPY format version 1.0: magic, version, little-endian header length, a Python
// dict literal padded with spaces so the data starts on a 64-byte boundary.
void write_npy(const std::filesystem::path &path, const Matrix &matrix) {
  std::ostringstream dict;
  dict << "{'descr': '<f4', 'fortran_order': False, 'shape': (" << matrix.rows << ", " << matrix.columns << "), }";
  std::string header = dict.str();
  const size_t unpadded = 10 + header.size() + 1;
  header.append((64 - unpadded % 64) % 64, ' ');
  header.push_back('\n');
  std::ofstream out(path, std::ios::binary | std::ios::trunc);
  const unsigned char prefix[10] = {0x93, 'N', 'U', 'M', 'P', 'Y', 1, 0,
                                    static_cast<unsigned char>(header.size() & 0xff),
                                    static_cast<unsigned char>(header.size() >> 8)};
  out.write(reinterpret_cast<const char *>(prefix), 10);
  out.write(header.data(), static_cast<std::streamsize>(header.size()));
  out.write(reinterpret_cast<const char *>(matrix.values.data()),
            static_cast<std::streamsize>(matrix.values.size() * sizeof(float)));
  if (!out) die(EVO_STATUS_IO, "cannot write '" + path.string() + "'");
}

Options parse(int argc, char **argv) {
  Options o;
  int first = 1;
  if (argc > 1 && argv[1][0] != '-') {
    o.command = argv[1];
    first = 2;
  }
  const auto value = [&](int &i) -> std::string {
    if (i + 1 >= argc) die(EVO_STATUS_INVALID_ARGUMENT, std::string("missing value for ") + argv[i]);
    return argv[++i];
  };
  for (int i = first; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "-m" || a == "--model") o.model = value(i);
    else if (a == "-p" || a == "--prompt") o.prompt = value(i);
    else if (a == "-n") o.tokens = std::stoull(value(i));
    else if (a == "--input") o.input = value(i);
    else if (a == "--score") { o.command = "score"; o.input = value(i); }
    else if (a == "--ctx") o.context = std::stoull(value(i));
    else if (a == "--profile") o.profile = value(i);
    else if (a == "--backend") { if (value(i) == "cpu") die(EVO_STATUS_UNSUPPORTED, "this build provides the CUDA backend only"); }
    else if (a == "--temp") o.temperature = std::stof(value(i));
    else if (a == "--top-k") o.top_k = std::stoull(value(i));
    else if (a == "--top-p") o.top_p = std::stof(value(i));
    else if (a == "--seed") o.seed = std::stoull(value(i));
    else if (a == "--warmup") o.warmup = std::stoull(value(i));
    else if (a == "--repetitions") o.repetitions = std::stoull(value(i));
    else if (a == "--output-format") o.output_format = value(i);
    else if (a == "--name") o.name = value(i);
    else if (a == "--output") o.output = value(i);
    else if (a == "--layer") o.layer = std::stoull(value(i));
    else if (a == "--pooling") o.pooling = value(i);
    else if (a == "--allow-test-fixture") o.allow_fixture = true;
    else if (a == "--force-prompt-threshold") {
      const std::string text = value(i);
      char *end = nullptr;
      const unsigned long long parsed = std::strtoull(text.c_str(), &end, 10);
      if (text.empty() || text[0] < '0' || text[0] > '9' || *end != '\0' || parsed < 1 || parsed > 1048576ULL)
        die(EVO_STATUS_INVALID_ARGUMENT, "--force-prompt-threshold must be an integer in [1, 1048576]");
      o.force_prompt_threshold = static_cast<size_t>(parsed);
    } else if (a == "--dump-tokens") o.dump_tokens = true;
    else if (a == "--dump-logits") {
      o.dump_logits_path = value(i);
      if (o.dump_logits_path.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "--dump-logits path must not be empty");
    } else if (a == "--dump-layer") {
      const std::string spec = value(i);
      const size_t colon = spec.find(':');
      char *end = nullptr;
      const unsigned long long layer = std::strtoull(spec.c_str(), &end, 10);
      if (colon == std::string::npos || colon == 0 || colon + 1 >= spec.size() || end != spec.c_str() + colon ||
          spec[0] < '0' || spec[0] > '9')
        die(EVO_STATUS_INVALID_ARGUMENT, "--dump-layer must be a nonnegative INDEX:PATH");
      o.dump_layer = static_cast<size_t>(layer);
      o.dump_layer_path = spec.substr(colon + 1);
    }
    else if (a == "--sequence") o.sequence = value(i);
    else if (a == "--vcf") o.vcf_path = value(i);
    else if (a == "--workers" || a == "--max-batch") o.workers = std::stoull(value(i));
    else if (a == "--max-queue") o.max_queue = std::stoull(value(i));
    else if (a == "--reference") o.reference_path = value(i);
    else if (a == "--position") o.position = std::stoull(value(i));
    else if (a == "--ref") o.reference_allele = value(i);
    else if (a == "--alt") o.alternate_allele = value(i);
    else if (a == "--window") o.window = std::stoull(value(i));
    else if (a == "--strand") o.strand = value(i);
    else if (a == "--normalization") o.normalization = value(i);
    else if (a == "--gpu") {
      o.gpus.clear();
      std::stringstream list(value(i));
      for (std::string item; std::getline(list, item, ',');) o.gpus.push_back(std::stoi(item));
    } else if (a == "--version") { std::cout << evo_version_string() << '\n'; std::exit(0); }
    else if (a == "--help" || a == "-h") {
      std::cout << "usage:\n  evo run -m MODEL -p DNA -n TOKENS [--ctx N --gpu 0,1 --profile exact|b200-tc|b200-fp8|fast-q8-kv]\n"
                   "          [--force-prompt-threshold N --dump-tokens --dump-logits PATH --dump-layer INDEX:PATH]\n"
                   "  evo score -m MODEL --input FASTA_FASTQ_OR_TEXT [--dump-tokens --dump-logits PATH --dump-layer INDEX:PATH]\n"
                   "  evo bench -m MODEL --input FASTA_FASTQ_OR_TEXT [--warmup N --repetitions N]\n"
                   "  evo embed -m MODEL --input FASTA_FASTQ_OR_TEXT --output DIR --layer N "
                   "--pooling none|mean|last\n"
                   "  evo variant-score -m MODEL --sequence DNA --position POS --ref REF --alt ALT "
                   "[--window N --strand forward|reverse|both --normalization sum|mean]\n"
                   "  evo serve -m MODEL [--workers N --max-queue M --ctx N --profile ...] < requests.jsonl\n"
                   "  evo variant-score -m MODEL --vcf VARIANTS.vcf[.gz] --reference GENOME.fa "
                   "[--window N --strand ... --normalization ...]\n";
      std::exit(0);
    } else die(EVO_STATUS_INVALID_ARGUMENT, "unknown option " + a);
  }
  if (o.model.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "a model path is required (-m)");
  const bool generation = o.command == "run";
  if (o.force_prompt_threshold != 0 && !generation)
    die(EVO_STATUS_INVALID_ARGUMENT, "--force-prompt-threshold is only valid for generation");
  if ((!o.dump_logits_path.empty() || !o.dump_layer_path.empty()) && !generation && o.command != "score")
    die(EVO_STATUS_INVALID_ARGUMENT, "--dump-logits and --dump-layer are valid for generation and scoring only");
  if (o.profile != "exact" && o.profile != "b200-tc" && o.profile != "b200-fp8" && o.profile != "fast-q8-kv")
    die(EVO_STATUS_UNSUPPORTED, "profile must be exact, b200-tc, b200-fp8 or fast-q8-kv");
  return o;
}

struct Metrics {
  double load_seconds = 0, prefill_seconds = 0, decode_seconds = 0, teacher_force_seconds = 0;
  size_t prefill_tokens = 0, decode_tokens = 0, teacher_force_tokens = 0, retained_logits_peak_bytes = 0;
};

void print_tokens(const std::string &label, const std::string &bytes) {
  std::cerr << "tokens " << label << "=[";
  for (size_t i = 0; i < bytes.size(); ++i) std::cerr << (i ? "," : "") << int(static_cast<unsigned char>(bytes[i]));
  std::cerr << "]\n";
}

// One prefill whose block output `layer` goes to an NPY file (upstream --dump-layer INDEX:PATH, the
// block-output tap): the sequence has to fit one activation chunk.  cached selects the exact
// cached-generation arithmetic (generation) or the ordinary prefill (scoring).
struct LayerDumpSink {
  std::filesystem::path path;
  Collected logits;
};
evo_status write_layer_dump(size_t, int32_t, const float *values, size_t rows, size_t columns, void *user) {
  Matrix matrix;
  matrix.values.assign(values, values + rows * columns);
  matrix.rows = rows;
  matrix.columns = columns;
  write_npy(static_cast<LayerDumpSink *>(user)->path, matrix);
  return EVO_STATUS_OK;
}
evo_status collect_beside_dump(const float *logits, size_t rows, size_t columns, size_t offset, void *user) {
  return collect(logits, rows, columns, offset, &static_cast<LayerDumpSink *>(user)->logits);
}
Collected prefill_with_layer_dump(evo_context *context, const std::string &bytes, const Options &o, const bool cached) {
  if (bytes.size() > evo_b200_context_activation_capacity(context))
    die(EVO_STATUS_INVALID_ARGUMENT, "--dump-layer is unavailable when prefill spans multiple activation chunks");
  evo_batch *batch = nullptr;
  check(evo_batch_create(1, &batch), "batch");
  check(evo_batch_add_sequence(batch, reinterpret_cast<const uint8_t *>(bytes.data()), bytes.size()), "batch");
  LayerDumpSink sink;
  sink.path = o.dump_layer_path;
  const evo_b200_dump_request request{o.dump_layer, EVO_B200_DUMP_BLOCK_OUTPUT};
  const evo_status status = evo_b200_context_prefill_with_dumps(context, batch, &request, 1, cached ? 1 : 0,
                                                                write_layer_dump, collect_beside_dump, &sink);
  evo_batch_free(batch);
  check(status, "prefill with --dump-layer");
  return sink.logits;
}

evo_context *new_context(const evo_model *model, const Options &o) {
  evo_context_params params = evo_context_default_params();
  params.context_size = o.context;
  if (o.profile == "b200-tc") params.flags |= EVO_CONTEXT_FLAG_B200_TENSORCORE_FP8;
  if (o.profile == "b200-fp8") params.flags |= EVO_CONTEXT_FLAG_B200_FP8_FFN;
  if (o.profile == "fast-q8-kv") params.flags |= EVO_CONTEXT_FLAG_FAST_Q8_KV;
  evo_context *context = nullptr;
  check(evo_context_create(model, &params, &context), "context");
  return context;
}

Collected prefill(evo_context *context, const std::string &bytes) {
  evo_batch *batch = nullptr;
  check(evo_batch_create(1, &batch), "batch");
  check(evo_batch_add_sequence(batch, reinterpret_cast<const uint8_t *>(bytes.data()), bytes.size()),
        "batch");
  Collected sink;
  const evo_status status = evo_context_prefill(context, batch, collect, &sink);
  evo_batch_free(batch);
  check(status, "prefill");
  return sink;
}

void print_metrics(const Metrics &m, const Options &o, const evo_context *context) {
  const auto rate = [](const size_t n, const double s) { return s > 0 ? static_cast<double>(n) / s : 0.0; };
  std::cerr << "evo_metrics {\"model_load_seconds\":" << std::setprecision(9) << m.load_seconds
            << ",\"prefill_tokens\":" << m.prefill_tokens << ",\"prefill_seconds\":" << m.prefill_seconds
            << ",\"prefill_tokens_per_second\":" << rate(m.prefill_tokens, m.prefill_seconds)
            << ",\"teacher_force_tokens\":" << m.teacher_force_tokens << ",\"teacher_force_seconds\":"
            << m.teacher_force_seconds << ",\"teacher_force_tokens_per_second\":"
            << rate(m.teacher_force_tokens, m.teacher_force_seconds)
            << ",\"decode_tokens\":" << m.decode_tokens << ",\"decode_seconds\":" << m.decode_seconds
            << ",\"decode_tokens_per_second\":" << rate(m.decode_tokens, m.decode_seconds)
            << ",\"kv_cache\":\"" << (o.profile == "fast-q8-kv" ? "q8_paged" : "bf16_contiguous")
            << "\",\"profile\":\"" << o.profile
            << "\",\"retained_logits_peak_bytes\":" << m.retained_logits_peak_bytes << ",\"gpus\":[";
  const size_t stages = context == nullptr ? 0 : evo_b200_context_stage_count(context);
  for (size_t i = 0; i < stages; ++i) {
    evo_b200_stage_info info{};
    info.struct_size = sizeof(info);
    if (evo_b200_context_stage_info(context, i, &info) != EVO_STATUS_OK) break;
    std::cerr << (i ? "," : "") << "{\"device\":" << info.device << ",\"layers\":[" << info.layer_begin
              << ',' << info.layer_end << "],\"weights_bytes\":" << info.weight_bytes
              << ",\"cache_bytes\":" << info.cache_bytes << ",\"arena_bytes\":" << info.arena_bytes << '}';
  }
  std::cerr << "]}\n";
}


// Sum (or mean) of next-token log-likelihoods of one window, as `evo score`
// computes them (upstream src/cuda/inference_cli.cpp:762-799 scores both windows
// of a strand with its sequence scorer).
struct WindowScore {
  double log_likelihood = 0.0;
  size_t scored_tokens = 0;
};

WindowScore score_window(const evo_model *model, const Options &o, const std::string &bytes, const size_t vocab,
                         Metrics *metrics, evo_context **last_context) {
  if (*last_context != nullptr) evo_context_free(*last_context);
  *last_context = new_context(model, o);
  const auto start = std::chrono::steady_clock::now();
  const Collected out = prefill(*last_context, bytes);
  metrics->prefill_seconds += seconds_since(start);
  metrics->prefill_tokens += bytes.size();
  WindowScore score;
  for (size_t t = 0; t + 1 < bytes.size(); ++t)
    score.log_likelihood += log_probability(out.logits.data() + t * vocab, vocab,
                                            static_cast<unsigned char>(bytes[t + 1]));
  score.scored_tokens = bytes.size() - 1;
  return score;
}

std::string reverse_complement_of(const std::string &sequence) {
  std::string out(sequence.size(), '\0');
  check(evo_b200_reverse_complement(sequence.data(), sequence.size(), out.data()), "reverse complement");
  return out;
}

}  // namespace

int main(int argc, char **argv) {
  const Options o = parse(argc, argv);
  Metrics metrics;
  evo_model_params mp = evo_model_default_params();
  mp.backend = EVO_BACKEND_CUDA;
  mp.devices = o.gpus.data();
  mp.device_count = o.gpus.size();
  if (o.allow_fixture) mp.flags |= EVO_MODEL_FLAG_TEST_ONLY_ALLOW_SYNTHETIC;
  evo_model *model = nullptr;
  const auto load_start = std::chrono::steady_clock::now();
  check(evo_model_load(o.model.c_str(), &mp, &model), "model");
  metrics.load_seconds = seconds_since(load_start);
  const size_t vocab = evo_model_vocab_size(model);
  evo_context *last_context = nullptr;

  if (o.command == "score") {
    if (o.input.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "score needs --input");
    const bool dumping = !o.dump_logits_path.empty() || !o.dump_layer_path.empty();
    size_t processed = 0;
    for (const Record &record : read_records(o.input, o.context)) {
      if (processed++ != 0 && dumping)
        die(EVO_STATUS_INVALID_ARGUMENT, "--dump-logits and --dump-layer require a score input with exactly one record");
      if (o.dump_tokens) print_tokens(record.name, record.bytes);
      if (record.bytes.size() < 2) die(EVO_STATUS_INVALID_ARGUMENT, "scoring needs at least two tokens");
      if (last_context != nullptr) evo_context_free(last_context);
      last_context = new_context(model, o);
      const auto start = std::chrono::steady_clock::now();
      const Collected out = o.dump_layer_path.empty() ? prefill(last_context, record.bytes)
                                                      : prefill_with_layer_dump(last_context, record.bytes, o, false);
      metrics.prefill_seconds += seconds_since(start);
      metrics.prefill_tokens += record.bytes.size();
      if (!o.dump_logits_path.empty()) {
        Matrix all;
        all.values = out.logits;
        all.rows = record.bytes.size();
        all.columns = vocab;
        write_npy(o.dump_logits_path, all);
        metrics.retained_logits_peak_bytes = std::max(metrics.retained_logits_peak_bytes, out.logits.size() * sizeof(float));
      }
      std::vector<double> scores;
      for (size_t t = 0; t + 1 < record.bytes.size(); ++t)
        scores.push_back(log_probability(out.logits.data() + t * vocab, vocab,
                                         static_cast<unsigned char>(record.bytes[t + 1])));
      double total = 0.0;
      for (const double s : scores) total += s;
      const double mean = total / static_cast<double>(scores.size());
      const double perplexity = std::exp(-mean);
      std::cout << "{\"name\":";
      json_string(std::cout, record.name);
      std::cout << ",\"input_format\":\"" << record.format << "\",\"backend\":\"cuda\",\"profile\":\""
                << o.profile << "\",\"model_id\":";
      const std::string id = evo_model_id(model);
      if (id.empty()) std::cout << "null"; else json_string(std::cout, id);
      std::cout << ",\"tokens\":" << record.bytes.size() << ",\"scored_tokens\":" << scores.size()
                << ",\"log_likelihood\":" << std::setprecision(17) << total
                << ",\"mean_log_likelihood\":" << mean << ",\"perplexity\":";
      if (std::isfinite(perplexity)) std::cout << perplexity; else std::cout << "null";
      std::cout << ",\"token_log_likelihoods\":[";
      for (size_t i = 0; i < scores.size(); ++i) std::cout << (i ? "," : "") << scores[i];
      std::cout << "]}\n";
    }
  } else if (o.command == "embed") {
    if (o.input.empty() || o.output.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "embed needs --input and --output");
    if (o.layer == static_cast<size_t>(-1)) die(EVO_STATUS_INVALID_ARGUMENT, "embed needs --layer");
    if (o.pooling != "none" && o.pooling != "mean" && o.pooling != "last")
      die(EVO_STATUS_INVALID_ARGUMENT, "--pooling must be none, mean or last");
    namespace fs = std::filesystem;
    const fs::path directory{o.output};
    std::error_code error;
    if (fs::exists(directory, error)) {
      if (error || !fs::is_directory(directory, error))
        die(EVO_STATUS_INVALID_ARGUMENT, "embedding output exists and is not a directory: '" + o.output + "'");
      if (fs::directory_iterator(directory, error) != fs::directory_iterator{})
        die(EVO_STATUS_INVALID_ARGUMENT, "embedding output directory must be empty: '" + o.output + "'");
    } else if (error || !fs::create_directories(directory, error) || error) {
      die(EVO_STATUS_IO, "cannot create embedding output directory '" + o.output + "'");
    }
    std::ofstream manifest(directory / "embeddings.jsonl", std::ios::binary | std::ios::trunc);
    if (!manifest) die(EVO_STATUS_IO, "cannot open embedding manifest");
    size_t record_index = 0;
    for (const Record &record : read_records(o.input, o.context)) {
      if (record.bytes.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "embedding record '" + record.name + "' is empty");
      if (last_context != nullptr) evo_context_free(last_context);
      last_context = new_context(model, o);
      evo_batch *batch = nullptr;
      check(evo_batch_create(1, &batch), "batch");
      check(evo_batch_add_sequence(batch, reinterpret_cast<const uint8_t *>(record.bytes.data()),
                                   record.bytes.size()), "batch");
      evo_embedding_options options = evo_embedding_default_options();
      options.layer = o.layer;
      options.pooling = o.pooling.c_str();
      Matrix matrix;
      const auto start = std::chrono::steady_clock::now();
      const evo_status status = evo_context_embed_ex(last_context, batch, &options, collect_matrix, &matrix);
      evo_batch_free(batch);
      check(status, "embed");
      metrics.prefill_seconds += seconds_since(start);
      metrics.prefill_tokens += record.bytes.size();
      std::ostringstream filename;
      filename << std::setw(6) << std::setfill('0') << record_index << ".npy";
      write_npy(directory / filename.str(), matrix);
      manifest << "{\"record_index\":" << record_index << ",\"name\":";
      json_string(manifest, record.name);
      manifest << ",\"input_format\":\"" << record.format << "\",\"file\":";
      json_string(manifest, filename.str());
      manifest << ",\"source_tokens\":" << record.bytes.size() << ",\"shape\":[" << matrix.rows << ','
               << matrix.columns << "],\"layer\":" << o.layer << ",\"point\":\"block_output\",\"pooling\":\""
               << o.pooling << "\",\"dtype\":\"float32\",\"backend\":\"cuda\",\"profile\":\"" << o.profile
               << "\",\"test_fixture\":" << (o.allow_fixture ? "true" : "false") << ",\"model_id\":";
      const std::string id = evo_model_id(model);
      if (id.empty()) manifest << "null"; else json_string(manifest, id);
      manifest << "}\n";
      manifest.flush();
      if (!manifest) die(EVO_STATUS_IO, "cannot write the embedding manifest");
      ++record_index;
    }
  } else if (o.command == "variant-score") {
    // Upstream's variant-effect driver (src/cuda/inference_cli.cpp:801-975): per allele,
    // delta = LL(alternate window) - LL(reference window) per strand, averaged over strands; the
    // alleles come from the command line or from a VCF whose windows are cut out of a reference FASTA.
    const bool from_files = !o.vcf_path.empty() || !o.reference_path.empty();
    if (from_files) {
      if (o.vcf_path.empty() || o.reference_path.empty())
        die(EVO_STATUS_INVALID_ARGUMENT, "variant-score needs --vcf and --reference together");
      if (!o.sequence.empty() || o.position != 0 || !o.reference_allele.empty() || !o.alternate_allele.empty())
        die(EVO_STATUS_INVALID_ARGUMENT, "--vcf/--reference cannot be combined with --sequence/--position/--ref/--alt");
    } else if (o.sequence.empty() || o.position == 0 || o.reference_allele.empty() || o.alternate_allele.empty()) {
      die(EVO_STATUS_INVALID_ARGUMENT, "variant-score needs --sequence, --position (1-based), --ref and --alt, "
                                       "or --vcf and --reference");
    }
    if (o.strand != "forward" && o.strand != "reverse" && o.strand != "both")
      die(EVO_STATUS_INVALID_ARGUMENT, "--strand must be one of forward, reverse, or both");
    if (o.normalization != "sum" && o.normalization != "mean")
      die(EVO_STATUS_INVALID_ARGUMENT, "--normalization must be one of sum or mean");
    const size_t window_tokens = o.window == 0 ? o.context : o.window;
    if (window_tokens > o.context) die(EVO_STATUS_INVALID_ARGUMENT, "--window must not exceed --ctx");
    // `sequence` holds the allele at 1-based `position`; `offset` is where sequence[0] sits on its
    // contig (0 for the inline form); `vcf` is null for the inline form
    const auto score_variant = [&](const std::string &sequence, const size_t position, const std::string &ref_allele,
                                   const std::string &alt_allele, const size_t offset,
                                   const evo_b200_vcf_record *vcf) -> evo_status {
      evo_b200_variant_window window{};
      window.struct_size = sizeof(window);
      std::string reference(window_tokens, '\0'), alternate(window_tokens, '\0');
      const evo_status made = evo_b200_variant_window_make(
          sequence.data(), sequence.size(), position, ref_allele.data(), ref_allele.size(), alt_allele.data(),
          alt_allele.size(), window_tokens, &window, reference.data(), alternate.data(), window_tokens);
      if (made != EVO_STATUS_OK) return made;
      reference.resize(window.reference_length);
      alternate.resize(window.alternate_length);
      struct Strand {
        const char *name;
        WindowScore reference, alternate;
        double delta;
      };
      std::vector<Strand> strands;
      const auto score_strand = [&](const char *name, const std::string &ref, const std::string &alt) {
        Strand strand{name, score_window(model, o, ref, vocab, &metrics, &last_context),
                      score_window(model, o, alt, vocab, &metrics, &last_context), 0.0};
        if (o.normalization == "mean") {
          strand.reference.log_likelihood /= static_cast<double>(strand.reference.scored_tokens);
          strand.alternate.log_likelihood /= static_cast<double>(strand.alternate.scored_tokens);
        }
        strand.delta = strand.alternate.log_likelihood - strand.reference.log_likelihood;
        strands.push_back(strand);
      };
      if (o.strand != "reverse") score_strand("+", reference, alternate);
      if (o.strand != "forward") score_strand("-", reverse_complement_of(reference), reverse_complement_of(alternate));
      double aggregate = 0.0;
      for (const Strand &strand : strands) aggregate += strand.delta;
      aggregate /= static_cast<double>(strands.size());
      std::cout << "{\"source\":\"" << (vcf == nullptr ? "inline" : "vcf") << '"';
      if (vcf != nullptr) {
        std::cout << ",\"record_index\":" << vcf->record_index << ",\"allele_index\":" << vcf->allele_index
                  << ",\"vcf_line\":" << vcf->line_number << ",\"id\":";
        json_string(std::cout, vcf->id);
        std::cout << ",\"contig\":";
        json_string(std::cout, vcf->contig);
      }
      std::cout << ",\"position\":" << (vcf == nullptr ? position : vcf->position_1based)
                << ",\"position_coordinate_system\":\"" << (vcf == nullptr ? "1-based" : "VCF-1-based")
                << "\",\"reference\":";
      json_string(std::cout, ref_allele);
      std::cout << ",\"alternate\":";
      json_string(std::cout, alt_allele);
      std::cout << ",\"window\":{\"start\":" << offset + window.reference_start << ",\"end\":"
                << offset + window.reference_end << ",\"coordinate_system\":\"0-based-half-open\"";
      if (vcf != nullptr) {
        std::cout << ",\"contig\":";
        json_string(std::cout, vcf->contig);
      }
      std::cout << ",\"reference_sequence\":";
      json_string(std::cout, reference);
      std::cout << ",\"alternate_sequence\":";
      json_string(std::cout, alternate);
      std::cout << ",\"reference_tokens\":" << reference.size() << ",\"alternate_tokens\":" << alternate.size()
                << "},\"normalization\":\"" << (o.normalization == "sum" ? "sum_log_likelihood" : "mean_log_likelihood")
                << "\",\"backend\":\"cuda\",\"profile\":\"" << o.profile << "\",\"test_fixture\":"
                << (o.allow_fixture ? "true" : "false") << ",\"model_id\":";
      const std::string id = evo_model_id(model);
      if (id.empty()) std::cout << "null"; else json_string(std::cout, id);
      std::cout << ",\"strands\":[" << std::setprecision(17);
      for (size_t i = 0; i < strands.size(); ++i) {
        const Strand &strand = strands[i];
        std::cout << (i ? "," : "") << "{\"strand\":\"" << strand.name << "\",\"reference_log_likelihood\":"
                  << strand.reference.log_likelihood << ",\"alternate_log_likelihood\":"
                  << strand.alternate.log_likelihood << ",\"reference_scored_tokens\":"
                  << strand.reference.scored_tokens << ",\"alternate_scored_tokens\":"
                  << strand.alternate.scored_tokens << ",\"delta\":" << strand.delta << '}';
      }
      std::cout << "],\"aggregation\":\"" << (strands.size() == 1 ? "single_strand" : "mean_across_strands")
                << "\",\"score\":" << aggregate << "}\n";
      return EVO_STATUS_OK;
    };
    if (!from_files) {
      check(score_variant(o.sequence, o.position, o.reference_allele, o.alternate_allele, 0, nullptr),
            "variant window");
    } else {
      evo_b200_reference *genome = nullptr;
      check(evo_b200_reference_open(o.reference_path.c_str(), &genome), "reference FASTA");
      struct Walk {
        evo_b200_reference *genome;
        size_t window_tokens;
        const decltype(score_variant) *score;
      } walk{genome, window_tokens, &score_variant};
      const evo_status streamed = evo_b200_vcf_stream(
          o.vcf_path.c_str(),
          [](const evo_b200_vcf_record *record, void *user) -> evo_status {
            const Walk &w = *static_cast<const Walk *>(user);
            std::string slice(w.window_tokens, '\0');
            size_t start = 0, end = 0;
            const std::string ref = record->reference, alt = record->alternate;
            const evo_status cut = evo_b200_reference_window(w.genome, record->contig, record->position_1based,
                                                             ref.data(), ref.size(), alt.data(), alt.size(),
                                                             w.window_tokens, &start, &end, nullptr, slice.data(),
                                                             slice.size());
            if (cut != EVO_STATUS_OK) {
              std::cerr << "evo: VCF line " << record->line_number << ": " << evo_last_error() << '\n';
              return cut;
            }
            slice.resize(end - start);
            return (*w.score)(slice, record->position_1based - start, ref, alt, start, record);
          },
          &walk);
      evo_b200_reference_free(genome);
      if (streamed != EVO_STATUS_OK) die(static_cast<int>(streamed), std::string("variant-score: ") + evo_last_error());
    }
  } else if (o.command == "bench") {
    if (o.input.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "bench needs --input");
    if (o.repetitions == 0) die(EVO_STATUS_INVALID_ARGUMENT, "--repetitions must be positive");
    const Record record = read_records(o.input, o.context).front();
    std::vector<double> samples;
    for (size_t i = 0; i < o.warmup + o.repetitions; ++i) {
      if (last_context != nullptr) evo_context_free(last_context);
      last_context = new_context(model, o);
      const auto start = std::chrono::steady_clock::now();
      prefill(last_context, record.bytes);
      const double seconds = seconds_since(start);
      if (i >= o.warmup) {
        samples.push_back(seconds);
        metrics.prefill_seconds += seconds;
        metrics.prefill_tokens += record.bytes.size();
      }
    }
    std::vector<double> sorted = samples;
    std::sort(sorted.begin(), sorted.end());
    const double median = sorted.size() % 2 ? sorted[sorted.size() / 2]
                                            : 0.5 * (sorted[sorted.size() / 2 - 1] + sorted[sorted.size() / 2]);
    std::ostringstream hash;
    hash << "fnv1a64:" << std::hex << std::setw(16) << std::setfill('0') << fnv1a64(record.bytes);
    std::cout << "{\"schema_version\":1,\"command\":\"bench\",\"model_path\":";
    json_string(std::cout, o.model);
    std::cout << ",\"model_id\":";
    const std::string id = evo_model_id(model);
    if (id.empty()) std::cout << "null"; else json_string(std::cout, id);
    std::cout << ",\"architecture\":";
    json_string(std::cout, evo_model_architecture(model));
    std::cout << ",\"artifact_profile\":";
    json_string(std::cout, evo_model_profile(model));
    std::cout << ",\"execution_profile\":\"" << o.profile << "\",\"backend\":\"cuda\",\"input\":{\"path\":";
    json_string(std::cout, o.input);
    std::cout << ",\"name\":";
    json_string(std::cout, record.name);
    std::cout << ",\"format\":\"" << record.format << "\",\"identity\":\"" << hash.str()
              << "\"},\"context_size\":" << o.context << ",\"warmup\":" << o.warmup
              << ",\"repetitions\":" << o.repetitions << ",\"tokens\":" << record.bytes.size()
              << ",\"timing_scope\":\"prefill_with_host_logits\",\"samples_seconds\":["
              << std::setprecision(17);
    for (size_t i = 0; i < samples.size(); ++i) std::cout << (i ? "," : "") << samples[i];
    std::cout << "],\"statistic\":\"median\",\"median_seconds\":" << median
              << ",\"median_tokens_per_second\":" << static_cast<double>(record.bytes.size()) / median
              << "}\n";
  } else if (o.command == "serve") {
    // The serving loop of upstream's `evo serve` (src/server.cpp) without its HTTP transport: one
    // JSON request per input line, one JSON response per request as it completes (not in input
    // order), on a pool of contexts that share the model's weights.
    //   {"id":"a","op":"score","sequence":"ACGT..."}
    //   {"id":"b","op":"generate","prompt":"ACGT","tokens":16,"temperature":1,"top_k":1,"top_p":1,"seed":0}
    evo_b200_scheduler_params sp{};
    sp.struct_size = sizeof(sp);
    sp.workers = o.workers;
    sp.maximum_queue = std::max(o.max_queue, o.workers);
    sp.context_size = o.context;
    if (o.profile == "b200-tc") sp.context_flags |= EVO_CONTEXT_FLAG_B200_TENSORCORE_FP8;
    if (o.profile == "b200-fp8") sp.context_flags |= EVO_CONTEXT_FLAG_B200_FP8_FFN;
    if (o.profile == "fast-q8-kv") sp.context_flags |= EVO_CONTEXT_FLAG_FAST_Q8_KV;
    evo_b200_scheduler *scheduler = nullptr;
    check(evo_b200_scheduler_create(model, &sp, &scheduler), "scheduler");
    struct Pending {
      std::string id, op;
      std::mutex *output;
    };
    std::mutex output;
    const auto respond = [](uint64_t, const evo_b200_request_result *r, void *user) {
      std::unique_ptr<Pending> pending(static_cast<Pending *>(user));
      std::ostringstream line;
      line << "{\"id\":";
      json_string(line, pending->id);
      line << ",\"op\":";
      json_string(line, pending->op);
      if (r->cancelled) {
        line << ",\"error\":{\"code\":\"cancelled\",\"message\":\"request was cancelled\"}";
      } else if (r->status != EVO_STATUS_OK) {
        line << ",\"error\":{\"code\":\"" << evo_status_name(r->status) << "\",\"message\":";
        json_string(line, r->error);
        line << '}';
      } else if (pending->op == "score") {
        line << std::setprecision(17) << ",\"tokens\":" << r->scored_tokens + 1 << ",\"scored_tokens\":"
             << r->scored_tokens << ",\"log_likelihood\":" << r->log_likelihood << ",\"mean_log_likelihood\":"
             << r->log_likelihood / static_cast<double>(r->scored_tokens);
      } else {
        line << ",\"generated\":";
        json_string(line, std::string(reinterpret_cast<const char *>(r->generated), r->generated_length));
      }
      line << std::setprecision(6) << ",\"queue_seconds\":" << r->queue_seconds << ",\"run_seconds\":"
           << r->run_seconds << "}\n";
      std::lock_guard<std::mutex> lock(*pending->output);
      std::cout << line.str();
      std::cout.flush();
    };
    size_t line_number = 0;
    for (std::string line; std::getline(std::cin, line);) {
      ++line_number;
      if (line.empty()) continue;
      auto pending = std::make_unique<Pending>();
      pending->output = &output;
      if (!json_field(line, "id", &pending->id)) pending->id = std::to_string(line_number);
      std::string payload, number;
      evo_b200_request request{};
      request.struct_size = sizeof(request);
      request.sampler = evo_sampler_default_params();
      const bool has_op = json_field(line, "op", &pending->op);
      const auto refuse = [&](const char *code, const std::string &message) {
        std::lock_guard<std::mutex> lock(output);
        std::cout << "{\"id\":";
        json_string(std::cout, pending->id);
        std::cout << ",\"error\":{\"code\":\"" << code << "\",\"message\":";
        json_string(std::cout, message);
        std::cout << "}}\n";
        std::cout.flush();
      };
      if (has_op && pending->op == "score" && json_field(line, "sequence", &payload)) {
        request.kind = EVO_B200_REQUEST_SCORE;
      } else if (has_op && pending->op == "generate" && json_field(line, "prompt", &payload)) {
        request.kind = EVO_B200_REQUEST_GENERATE;
        try {
          if (json_field(line, "tokens", &number)) request.new_tokens = std::stoull(number);
          if (json_field(line, "temperature", &number)) request.sampler.temperature = std::stof(number);
          if (json_field(line, "top_k", &number)) request.sampler.top_k = std::stoull(number);
          if (json_field(line, "top_p", &number)) request.sampler.top_p = std::stof(number);
          if (json_field(line, "seed", &number)) request.sampler.seed = std::stoull(number);
        } catch (const std::exception &) {
          refuse("invalid_argument", "a numeric request field cannot be parsed");
          continue;
        }
      } else {
        refuse("invalid_argument", "a request needs \"op\":\"score\" with \"sequence\" or \"op\":\"generate\" with \"prompt\"");
        continue;
      }
      request.sequence = reinterpret_cast<const uint8_t *>(payload.data());
      request.length = payload.size();
      uint64_t ticket = 0;
      Pending *const raw = pending.get();
      const evo_status submitted = evo_b200_scheduler_submit(scheduler, &request, respond, raw, &ticket);
      if (submitted != EVO_STATUS_OK) refuse(evo_status_name(submitted), evo_last_error());
      else if (ticket == 0) refuse("busy", "the request queue is full");
      else pending.release();  // owned by the completion now
    }
    evo_b200_scheduler_wait_idle(scheduler);
    evo_b200_scheduler_metrics totals{};
    totals.struct_size = sizeof(totals);
    check(evo_b200_scheduler_read_metrics(scheduler, &totals), "scheduler metrics");
    std::cerr << "{\"scheduler\":{\"submitted\":" << totals.submitted << ",\"rejected\":" << totals.rejected
              << ",\"completed\":" << totals.completed << ",\"failed\":" << totals.failed << ",\"cancelled\":"
              << totals.cancelled << ",\"queue_peak\":" << totals.queue_peak << ",\"active_peak\":"
              << totals.active_peak << ",\"workers\":" << o.workers << "}}\n";
    evo_b200_scheduler_free(scheduler);
  } else if (o.command == "run") {
    if (o.prompt.empty()) die(EVO_STATUS_INVALID_ARGUMENT, "run needs a prompt (-p)");
    if (o.prompt.size() + o.tokens > o.context)
      die(EVO_STATUS_INVALID_ARGUMENT, "prompt plus generated tokens exceed --ctx");
    evo_sampler_params sp = evo_sampler_default_params();
    sp.temperature = o.temperature;
    sp.top_k = o.top_k;
    sp.top_p = o.top_p;
    sp.seed = o.seed;
    evo_sampler *sampler = nullptr;
    check(evo_sampler_create(&sp, &sampler), "sampler");
    last_context = new_context(model, o);
    if (o.dump_tokens) print_tokens("prompt", o.prompt);
    // Upstream's generation pass (src/cuda/inference_cli.cpp:436-470): the first tokens of the prompt - all of
    // it up to min(3000, activation capacity) unless --force-prompt-threshold says otherwise - run as one
    // exact cached prefill, the rest of the prompt is teacher-forced through decode.
    const size_t capacity = evo_b200_context_activation_capacity(last_context);
    const size_t threshold = o.force_prompt_threshold != 0 ? o.force_prompt_threshold : std::min<size_t>(3000, capacity);
    const size_t prefilled = std::min(o.prompt.size(), threshold);
    if (prefilled > capacity)
      die(EVO_STATUS_INVALID_ARGUMENT, "prompt prefill: exact cached prefill must fit one activation chunk; lower "
                                       "--force-prompt-threshold to at most " + std::to_string(capacity));
    auto start = std::chrono::steady_clock::now();
    Collected out;
    if (!o.dump_layer_path.empty()) {
      out = prefill_with_layer_dump(last_context, o.prompt.substr(0, prefilled), o, true);
    } else {
      std::vector<uint32_t> ids(prefilled);
      for (size_t i = 0; i < prefilled; ++i) ids[i] = static_cast<unsigned char>(o.prompt[i]);
      check(evo_b200_context_prefill_tokens(last_context, ids.data(), ids.size(), EVO_B200_PREFILL_CACHED, collect, &out),
            "prompt prefill");
    }
    metrics.prefill_seconds = seconds_since(start);
    metrics.prefill_tokens = prefilled;
    std::vector<float> logits(out.logits.end() - static_cast<std::ptrdiff_t>(vocab), out.logits.end());
    start = std::chrono::steady_clock::now();
    for (size_t i = prefilled; i < o.prompt.size(); ++i) {
      Collected step;
      check(evo_context_decode(last_context, static_cast<unsigned char>(o.prompt[i]), collect, &step),
            "teacher-forced prompt token");
      logits = step.logits;
      ++metrics.teacher_force_tokens;
    }
    metrics.teacher_force_seconds = seconds_since(start);
    Matrix dumped;  // --dump-logits: the logits every sampling step saw, [generated tokens, vocabulary]
    dumped.columns = vocab;
    std::string generated;
    start = std::chrono::steady_clock::now();
    for (size_t i = 0; i < o.tokens; ++i) {
      if (!o.dump_logits_path.empty()) {
        dumped.values.insert(dumped.values.end(), logits.begin(), logits.end());
        ++dumped.rows;
      }
      uint32_t token = 0;
      check(evo_sampler_sample(sampler, logits.data(), vocab, &token), "sample");
      uint8_t byte = 0;
      check(evo_model_decode_token(model, token, &byte), "decode token");
      generated.push_back(static_cast<char>(byte));
      if (i + 1 == o.tokens) break;
      Collected step;
      check(evo_context_decode(last_context, token, collect, &step), "decode");
      logits = step.logits;
      ++metrics.decode_tokens;
    }
    metrics.decode_seconds = seconds_since(start);
    if (!o.dump_logits_path.empty()) {
      write_npy(o.dump_logits_path, dumped);
      metrics.retained_logits_peak_bytes = dumped.values.size() * sizeof(float);
    }
    if (o.output_format == "fasta") std::cout << '>' << o.name << '\n' << generated << '\n';
    else std::cout << generated;
    std::cout.flush();
    evo_sampler_free(sampler);
  } else {
    die(EVO_STATUS_UNSUPPORTED, "unknown command " + o.command + " (run, score, bench, embed, variant-score, serve)");
  }
  print_metrics(metrics, o, last_context);
  if (last_context != nullptr) evo_context_free(last_context);
  evo_model_free(model);
  return 0;
}
