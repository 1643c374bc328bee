// Additions to the reference's operator surface.  Everything here is optional and
// defaults to the reference's behaviour.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/zkllm_b200.h"

namespace zkllm {

// random_vec() draws from std::random_device like the reference
// (fr-tensor.cu:16-24) unless a seed is set here or in the environment variable
// ZKLLM_CHALLENGE_SEED; a seeded stream makes whole driver runs reproducible.
void seed_challenges(uint64_t seed);
void unseed_challenges();

// The reference computes the round polynomials of zkFC::prove and tLookup::prove
// and the G1 elements of Commitment::me_open and then drops them.  When a sink is
// installed, every prover appends what it produced.
struct Transcript {
    struct Entry {
        std::string label;                 // e.g. "zkip", "tLookup", "me_open"
        std::vector<zkb_fr_t> scalars;     // round-polynomial coefficients, claims
        std::vector<zkb_g1_t> points;      // G1 proof elements
    };
    std::vector<Entry> entries;
};
void set_transcript_sink(Transcript* sink);   // nullptr = off (default)
Transcript* transcript_sink();

// Throws std::runtime_error(msg) when a C-ABI call failed; dimension and
// verifier failures carry the reference's message text.
void check(int rc);

}  // namespace zkllm
