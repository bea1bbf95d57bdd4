#include "variant.hpp"

#include <algorithm>

#include <string>
#include <utility>

#include "../common.cuh"

namespace evob {

char iupac_complement(const char letter) noexcept {
  // pairs of the IUPAC nucleotide code; S, W and N are their own complements
  static constexpr char kFrom[] = "ACGTRYSWKMBDHVN";
  static constexpr char kTo[] = "TGCAYRSWMKVHDBN";
  const bool lower = letter >= 'a' && letter <= 'z';
  const char upper = lower ? static_cast<char>(letter - 'a' + 'A') : letter;
  for (std::size_t i = 0; kFrom[i] != '\0'; ++i)
    if (kFrom[i] == upper) return lower ? static_cast<char>(kTo[i] - 'A' + 'a') : kTo[i];
  return 0;
}

int validate_iupac_dna(const std::string_view sequence, const std::string_view label) {
  if (sequence.empty()) return fail(kInvalidArgument, std::string(label) + " must not be empty");
  for (std::size_t i = 0; i < sequence.size(); ++i)
    if (iupac_complement(sequence[i]) == 0)
      return fail(kInvalidArgument,
                  std::string(label) + " contains non-IUPAC DNA byte at offset " + std::to_string(i));
  return kOk;
}

int reverse_complement(const std::string_view sequence, std::string *const output) {
  if (output == nullptr) return fail(kInvalidArgument, "reverse-complement output is null");
  const int status = validate_iupac_dna(sequence, "sequence");
  if (status != kOk) return status;
  output->assign(sequence.size(), '\0');
  for (std::size_t i = 0; i < sequence.size(); ++i)
    (*output)[sequence.size() - 1 - i] = iupac_complement(sequence[i]);
  return kOk;
}

int make_variant_window(const std::string_view sequence, const std::size_t position_1based,
                        const std::string_view reference, const std::string_view alternate,
                        const std::size_t maximum_tokens, VariantWindow *const output) {
  if (output == nullptr) return fail(kInvalidArgument, "variant window output is null");
  *output = VariantWindow{};
  int status = validate_iupac_dna(sequence, "reference sequence");
  if (status == kOk) status = validate_iupac_dna(reference, "reference allele");
  if (status == kOk) status = validate_iupac_dna(alternate, "alternate allele");
  if (status != kOk) return status;
  if (position_1based == 0)
    return fail(kInvalidArgument, "variant position is 1-based and must be positive");
  const std::size_t start = position_1based - 1;
  if (start > sequence.size() || reference.size() > sequence.size() - start)
    return fail(kInvalidArgument, "reference allele extends beyond the supplied sequence");
  if (sequence.substr(start, reference.size()) != reference)
    return fail(kInvalidArgument, "reference allele does not match the supplied sequence at 1-based position " +
                                      std::to_string(position_1based));
  const std::size_t core = std::max(reference.size(), alternate.size());
  if (maximum_tokens < core || maximum_tokens < 2)
    return fail(kInvalidArgument, "variant window must fit both alleles and at least two tokens");
  // Flanks: half of what the longer allele leaves on the left, the rest on the
  // right; whatever one side cannot use goes to the other.
  const std::size_t end = start + reference.size();
  const std::size_t left_room = start, right_room = sequence.size() - end;
  const std::size_t budget = maximum_tokens - core;
  std::size_t left = std::min(left_room, budget / 2);
  std::size_t right = std::min(right_room, budget - left);
  const std::size_t more_left = std::min(left_room - left, budget - left - right);
  left += more_left;
  right += std::min(right_room - right, budget - left - right);

  VariantWindow window;
  window.reference_start = start - left;
  window.reference_end = end + right;
  window.variant_offset = left;
  const std::string_view left_flank = sequence.substr(start - left, left);
  const std::string_view right_flank = sequence.substr(end, right);
  for (const auto &[target, allele] : {std::pair<std::string *, std::string_view>{&window.reference, reference},
                                       std::pair<std::string *, std::string_view>{&window.alternate, alternate}}) {
    target->reserve(left + allele.size() + right);
    target->append(left_flank).append(allele).append(right_flank);
  }
  if (window.reference.size() < 2 || window.alternate.size() < 2)
    return fail(kInvalidArgument, "reference and alternate windows must each contain two tokens");
  *output = std::move(window);
  return kOk;
}

}  // namespace evob
