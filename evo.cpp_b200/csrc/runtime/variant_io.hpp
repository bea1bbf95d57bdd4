// File inputs of the variant-effect driver: a VCF stream and random access to
// a reference FASTA.  Contract of upstream include/evo/variant_io.hpp:13-45
// (src/variant_io.cpp): one callback per ALT allele of every VCF record,
// plain or gzip input; the scoring window around an allele is as much flank as
// the token budget allows, half on each side, a side that runs out of contig
// ceding its share to the other (src/variant_io.cpp:313-327).
//
// Upstream re-reads the FASTA twice for every allele.  Here the file is
// scanned once into an in-memory index (contig -> offset, length, line
// geometry: what a .fai holds) and every window is one positioned read.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <string>
#include <string_view>

namespace evob {

struct VcfRecord {
  std::string contig, id, reference, alternate;
  std::size_t position_1based = 0;
  std::size_t record_index = 0;  // data line, counted from 0
  std::size_t allele_index = 0;  // position inside the ALT list
  std::size_t line_number = 0;   // 1-based line of the file
};

// Calls `callback` once per ALT allele; a non-kOk return stops the stream and
// is returned.  "-" reads standard input.  Symbolic and breakend alleles are
// refused (IUPAC DNA only).
int stream_vcf_file(const std::string &path, const std::function<int(const VcfRecord &)> &callback);

struct ReferenceSlice {
  std::string contig, sequence;
  std::size_t start = 0, end = 0;  // 0-based half-open span of `sequence` on the contig
  std::size_t contig_length = 0;
};

class ReferenceFasta {
 public:
  ~ReferenceFasta();
  // Scans `path` (plain FASTA, every sequence line of a contig but the last of
  // the same width) once.  kOk or a status with the message set.
  static int open(const std::string &path, ReferenceFasta **out);
  std::size_t contig_count() const { return contigs_.size(); }
  // Length of `contig`, or kInvalidArgument when the file has none of that name.
  int contig_length(std::string_view contig, std::size_t *length) const;
  // Bases [start, end) of `contig`.
  int fetch(std::string_view contig, std::size_t start, std::size_t end, std::string *bases) const;
  // The scoring window of upstream's fetch_reference_slice: checks that the
  // contig holds `reference` at `position_1based`, then cuts at most
  // `maximum_tokens` bases around the allele.
  int slice(std::string_view contig, std::size_t position_1based, std::string_view reference,
            std::string_view alternate, std::size_t maximum_tokens, ReferenceSlice *output) const;

 private:
  struct Contig {
    std::uint64_t offset = 0;      // file offset of the first base
    std::size_t length = 0;        // bases
    std::size_t line_bases = 0;    // bases per full line
    std::size_t line_bytes = 0;    // bytes per full line including the terminator
  };
  ReferenceFasta() = default;
  int descriptor_ = -1;
  std::map<std::string, Contig, std::less<>> contigs_;
};

}  // namespace evob
