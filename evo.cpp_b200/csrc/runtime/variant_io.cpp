// VCF stream and indexed reference FASTA for the variant-effect driver
// (contract: upstream include/evo/variant_io.hpp:13-45; messages follow
// src/variant_io.cpp:168-352 so that callers see the same diagnostics).
#include "variant_io.hpp"

#include <fcntl.h>
#include <unistd.h>
#include <zlib.h>

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cstring>
#include <limits>
#include <memory>
#include <vector>

#include "../common.cuh"
#include "variant.hpp"

namespace evob {
namespace {

constexpr std::size_t kMaxLineBytes = std::size_t{16} << 20;

// Next line of a (possibly gzip-compressed) stream without its terminator.
// Returns 1 for a line, 0 at the end of the input, -1 on a read error or a
// line longer than kMaxLineBytes.
int next_line(gzFile file, std::string *line) {
  line->clear();
  char buffer[1 << 16];
  while (gzgets(file, buffer, sizeof(buffer)) != nullptr) {
    const std::size_t got = std::strlen(buffer);
    line->append(buffer, got);
    if (line->size() > kMaxLineBytes) return -1;
    if (got != 0 && buffer[got - 1] == '\n') {
      line->pop_back();
      if (!line->empty() && line->back() == '\r') line->pop_back();
      return 1;
    }
  }
  int code = 0;
  gzerror(file, &code);
  if (code != Z_OK && code != Z_STREAM_END) return -1;
  if (line->empty()) return 0;
  if (line->back() == '\r') line->pop_back();
  return 1;  // last line without a terminator
}

std::vector<std::string_view> split(const std::string_view text, const char separator) {
  std::vector<std::string_view> parts;
  std::size_t begin = 0;
  for (;;) {
    const std::size_t end = text.find(separator, begin);
    if (end == std::string_view::npos) {
      parts.push_back(text.substr(begin));
      return parts;
    }
    parts.push_back(text.substr(begin, end - begin));
    begin = end + 1;
  }
}

int parse_position(const std::string_view text, std::size_t *value) {
  if (text.empty()) return fail(kInvalidArgument, "VCF POS must be a positive integer");
  std::size_t parsed = 0;
  for (const char c : text) {
    if (c < '0' || c > '9') return fail(kInvalidArgument, "VCF POS must be a positive integer");
    const std::size_t digit = static_cast<std::size_t>(c - '0');
    if (parsed > (std::numeric_limits<std::size_t>::max() - digit) / 10)
      return fail(kInvalidArgument, "VCF POS overflows size_t");
    parsed = parsed * 10 + digit;
  }
  if (parsed == 0) return fail(kInvalidArgument, "VCF POS must be a positive integer");
  *value = parsed;
  return kOk;
}

// Re-raises the current error text with the line it belongs to.
int at_line(const int status, const std::size_t line_number) {
  const std::string text = last_error();
  const std::size_t colon = text.find(": ");
  return fail(status, (colon == std::string::npos ? text : text.substr(colon + 2)) + " at line " +
                          std::to_string(line_number));
}

}  // namespace

int stream_vcf_file(const std::string &path, const std::function<int(const VcfRecord &)> &callback) {
  if (path.empty()) return fail(kInvalidArgument, "VCF path must not be empty");
  if (!callback) return fail(kInvalidArgument, "VCF callback must not be empty");
  gzFile file = path == "-" ? gzdopen(dup(0), "rb") : gzopen(path.c_str(), "rb");
  if (file == nullptr) return fail(kIo, "cannot open " + path + ": " + std::strerror(errno));
  struct Close {
    gzFile file;
    ~Close() { gzclose(file); }
  } close{file};
  static const char *const kColumns[] = {"#CHROM", "POS", "ID", "REF", "ALT", "QUAL", "FILTER", "INFO"};
  bool saw_columns = false;
  std::size_t record_index = 0, line_number = 0;
  std::string line;
  for (;;) {
    const int got = next_line(file, &line);
    if (got < 0) return fail(kIo, "cannot read a VCF line at line " + std::to_string(line_number + 1));
    if (got == 0) break;
    ++line_number;
    if (line.empty()) return fail(kInvalidArgument, "VCF has an empty line at " + std::to_string(line_number));
    if (line.compare(0, 2, "##") == 0) continue;
    if (line.front() == '#') {
      const auto header = split(line, '\t');
      bool matches = header.size() >= 8;
      for (std::size_t i = 0; matches && i < 8; ++i) matches = header[i] == kColumns[i];
      if (!matches)
        return fail(kInvalidArgument, "VCF has an unsupported header at line " + std::to_string(line_number));
      if (saw_columns)
        return fail(kInvalidArgument, "VCF repeats the #CHROM header at line " + std::to_string(line_number));
      saw_columns = true;
      continue;
    }
    if (!saw_columns)
      return fail(kInvalidArgument,
                  "VCF data appears before the #CHROM header at line " + std::to_string(line_number));
    const auto fields = split(line, '\t');
    if (fields.size() < 8 || fields[0].empty() || fields[2].empty() || fields[3].empty() || fields[4].empty())
      return fail(kInvalidArgument,
                  "VCF record has fewer than 8 valid fields at line " + std::to_string(line_number));
    std::size_t position = 0;
    int status = parse_position(fields[1], &position);
    if (status == kOk) status = validate_iupac_dna(fields[3], "VCF REF");
    if (status != kOk) return at_line(status, line_number);
    const auto alternates = split(fields[4], ',');
    for (std::size_t allele = 0; allele < alternates.size(); ++allele) {
      status = validate_iupac_dna(alternates[allele], "VCF ALT");
      if (status != kOk) return at_line(status, line_number);
      VcfRecord record;
      record.contig = std::string(fields[0]);
      record.id = std::string(fields[2]);
      record.reference = std::string(fields[3]);
      record.alternate = std::string(alternates[allele]);
      record.position_1based = position;
      record.record_index = record_index;
      record.allele_index = allele;
      record.line_number = line_number;
      status = callback(record);
      if (status != kOk) return status;
    }
    ++record_index;
  }
  if (!saw_columns) return fail(kInvalidArgument, "VCF is missing #CHROM header");
  if (record_index == 0) return fail(kInvalidArgument, "VCF contains no records");
  return kOk;
}

// ---------------------------------------------------------------- reference
ReferenceFasta::~ReferenceFasta() {
  if (descriptor_ >= 0) ::close(descriptor_);
}

int ReferenceFasta::open(const std::string &path, ReferenceFasta **out) {
  if (out == nullptr) return fail(kInvalidArgument, "reference output is null");
  *out = nullptr;
  if (path.empty() || path == "-")
    return fail(kInvalidArgument, "reference FASTA must be a reusable file path");
  const int descriptor = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (descriptor < 0) return fail(kIo, "cannot open " + path + ": " + std::strerror(errno));
  std::unique_ptr<ReferenceFasta> reference(new ReferenceFasta());
  reference->descriptor_ = descriptor;
  unsigned char magic[2] = {0, 0};
  if (::pread(descriptor, magic, 2, 0) == 2 && magic[0] == 0x1f && magic[1] == 0x8b)
    return fail(kUnsupported, "reference FASTA is gzip-compressed: random access needs the plain file");

  std::vector<char> block(std::size_t{4} << 20);
  std::uint64_t offset = 0;           // file offset of block[0]
  std::size_t line_number = 1;
  bool line_start = true, in_header = false, name_done = false, have_header = false;
  std::string name;
  Contig *current = nullptr;
  std::size_t line_bases = 0;         // bases seen on the current sequence line
  std::uint64_t line_offset = 0;      // file offset where the current line began
  bool short_line_seen = false;       // a line narrower than the first one ended: it must be the last
  const auto end_sequence_line = [&](const std::uint64_t next_line_offset) -> int {
    if (current == nullptr) return kOk;
    if (line_bases == 0) {  // a blank line carries nothing, but only the end of a contig may have one
      if (current->line_bases != 0) short_line_seen = true;
      return kOk;
    }
    if (short_line_seen || (current->line_bases != 0 && line_bases > current->line_bases))
      return fail(kInvalidArgument, "reference FASTA lines of contig '" + name +
                                        "' differ in width before its last line (line " +
                                        std::to_string(line_number) + "): random access needs uniform lines");
    if (current->line_bases == 0) {
      current->offset = line_offset;
      current->line_bases = line_bases;
      current->line_bytes = static_cast<std::size_t>(next_line_offset - line_offset);
    } else if (line_bases < current->line_bases ||
               static_cast<std::size_t>(next_line_offset - line_offset) != current->line_bytes) {
      short_line_seen = true;
    }
    current->length += line_bases;
    return kOk;
  };
  for (;;) {
    const ssize_t got = ::pread(descriptor, block.data(), block.size(), static_cast<off_t>(offset));
    if (got < 0) return fail(kIo, "cannot read " + path + ": " + std::strerror(errno));
    if (got == 0) break;
    for (ssize_t i = 0; i < got; ++i) {
      const char c = block[static_cast<std::size_t>(i)];
      const std::uint64_t here = offset + static_cast<std::uint64_t>(i);
      if (line_start) {
        line_start = false;
        line_offset = here;
        line_bases = 0;
        if (c == '>') {
          in_header = true;
          name_done = false;
          name.clear();
          continue;
        }
      }
      if (c == '\n') {
        if (in_header) {
          if (name.empty())
            return fail(kInvalidArgument,
                        "reference FASTA has an empty header at line " + std::to_string(line_number));
          if (reference->contigs_.count(name) != 0)
            return fail(kInvalidArgument, "reference FASTA contains duplicate contig '" + name + "'");
          current = &reference->contigs_[name];
          short_line_seen = false;
          have_header = true;
          in_header = false;
        } else {
          const int status = end_sequence_line(here + 1);
          if (status != kOk) return status;
        }
        line_start = true;
        ++line_number;
        continue;
      }
      if (in_header) {
        if (c == ' ' || c == '\t' || c == '\r') name_done = true;
        if (!name_done) name.push_back(c);
        continue;
      }
      if (c == '\r') continue;  // counted in line_bytes, not in the bases
      if (std::isspace(static_cast<unsigned char>(c)) != 0)
        return fail(kInvalidArgument,
                    "reference FASTA contains whitespace at line " + std::to_string(line_number));
      if (!have_header)
        return fail(kInvalidArgument, "reference FASTA sequence appears before a header at line " +
                                          std::to_string(line_number));
      ++line_bases;
    }
    offset += static_cast<std::uint64_t>(got);
  }
  if (!line_start && !in_header) {
    // last line without a terminator: give it the first line's terminator width for the geometry check
    const std::size_t terminator = current != nullptr && current->line_bases != 0
                                       ? current->line_bytes - current->line_bases : 1;
    const int status = end_sequence_line(offset + terminator);
    if (status != kOk) return status;
  }
  if (!have_header) return fail(kInvalidArgument, "reference input is not FASTA");
  *out = reference.release();
  return kOk;
}

int ReferenceFasta::contig_length(const std::string_view contig, std::size_t *length) const {
  const auto found = contigs_.find(contig);
  if (found == contigs_.end())
    return fail(kInvalidArgument, "reference FASTA has no contig '" + std::string(contig) + "'");
  if (length != nullptr) *length = found->second.length;
  return kOk;
}

int ReferenceFasta::fetch(const std::string_view contig, const std::size_t start, const std::size_t end,
                          std::string *bases) const {
  if (bases == nullptr) return fail(kInvalidArgument, "reference fetch output is null");
  bases->clear();
  const auto found = contigs_.find(contig);
  if (found == contigs_.end())
    return fail(kInvalidArgument, "reference FASTA has no contig '" + std::string(contig) + "'");
  const Contig &c = found->second;
  if (start > end || end > c.length)
    return fail(kInvalidArgument, "reference range lies outside contig '" + std::string(contig) + "'");
  if (start == end) return kOk;
  // byte span that holds the bases, line terminators included
  const std::uint64_t first = c.offset + (start / c.line_bases) * c.line_bytes + start % c.line_bases;
  const std::uint64_t last = c.offset + ((end - 1) / c.line_bases) * c.line_bytes + (end - 1) % c.line_bases + 1;
  std::string raw(static_cast<std::size_t>(last - first), '\0');
  std::size_t filled = 0;
  while (filled < raw.size()) {
    const ssize_t got = ::pread(descriptor_, raw.data() + filled, raw.size() - filled,
                                static_cast<off_t>(first + filled));
    if (got <= 0) return fail(kIo, "reference FASTA changed since it was indexed");
    filled += static_cast<std::size_t>(got);
  }
  bases->reserve(end - start);
  for (const char ch : raw)
    if (ch != '\n' && ch != '\r') bases->push_back(ch);
  if (bases->size() != end - start) return fail(kIo, "reference FASTA changed since it was indexed");
  return kOk;
}

int ReferenceFasta::slice(const std::string_view contig, const std::size_t position_1based,
                          const std::string_view reference, const std::string_view alternate,
                          const std::size_t maximum_tokens, ReferenceSlice *output) const {
  if (output == nullptr) return fail(kInvalidArgument, "reference slice output is null");
  *output = ReferenceSlice{};
  if (contig.empty()) return fail(kInvalidArgument, "reference contig must not be empty");
  int status = validate_iupac_dna(reference, "reference allele");
  if (status == kOk) status = validate_iupac_dna(alternate, "alternate allele");
  if (status != kOk) return status;
  if (position_1based == 0) return fail(kInvalidArgument, "reference position must be positive");
  const std::size_t start = position_1based - 1;
  if (reference.size() > std::numeric_limits<std::size_t>::max() - start)
    return fail(kInvalidArgument, "reference allele coordinates overflow");
  const std::size_t allele_end = start + reference.size();
  const std::size_t core = std::max(reference.size(), alternate.size());
  if (maximum_tokens < core || maximum_tokens < 2)
    return fail(kInvalidArgument, "variant window must fit both alleles and at least two tokens");
  std::size_t length = 0;
  status = contig_length(contig, &length);
  if (status != kOk) return status;
  if (start > length || reference.size() > length - start)
    return fail(kInvalidArgument, "VCF REF extends beyond reference contig '" + std::string(contig) + "'");
  std::string present;
  status = fetch(contig, start, allele_end, &present);
  if (status != kOk) return status;
  if (present != reference)
    return fail(kInvalidArgument, "VCF REF does not match reference contig '" + std::string(contig) +
                                      "' at 1-based position " + std::to_string(position_1based));
  // half the flank budget on each side; what one side cannot use goes to the other
  const std::size_t budget = maximum_tokens - core;
  std::size_t left = std::min(start, budget / 2);
  const std::size_t right_available = length - allele_end;
  std::size_t right = std::min(right_available, budget - left);
  std::size_t spare = budget - left - right;
  const std::size_t more_left = std::min(start - left, spare);
  left += more_left;
  spare -= more_left;
  right += std::min(right_available - right, spare);
  output->contig = std::string(contig);
  output->start = start - left;
  output->end = allele_end + right;
  output->contig_length = length;
  return fetch(contig, output->start, output->end, &output->sequence);
}

}  // namespace evob
