// Variant-effect scoring windows: host-side sequence logic shared by the
// `evo variant-score` driver and the C ABI (evo_b200_variant_window,
// evo_b200_reverse_complement).  Behaviour follows upstream src/variant.cpp:
// IUPAC validation (:69-84), reverse complement with case kept (:11-66, 86-101)
// and the flank budget of make_variant_window (:103-174).
#pragma once

#include <cstddef>
#include <string>
#include <string_view>

namespace evob {

struct VariantWindow {
  std::string reference, alternate;  // window with the reference / alternate allele in place
  std::size_t reference_start = 0;   // 0-based half-open span of the window on the input sequence
  std::size_t reference_end = 0;
  std::size_t variant_offset = 0;    // offset of the allele inside either window
};

// Complement of one IUPAC DNA letter (case kept); 0 for anything else.
char iupac_complement(char letter) noexcept;

// kOk, or kInvalidArgument with the message set (fail()).
int validate_iupac_dna(std::string_view sequence, std::string_view label);
int reverse_complement(std::string_view sequence, std::string *output);
int make_variant_window(std::string_view sequence, std::size_t position_1based, std::string_view reference,
                        std::string_view alternate, std::size_t maximum_tokens, VariantWindow *output);

}  // namespace evob
