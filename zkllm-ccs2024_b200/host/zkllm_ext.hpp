// Additions to the reference's operator surface.  Everything here is optional and
// defaults to the reference's behaviour.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/zkllm_b200.h"

struct Weight;   // commitment.cuh
struct Claim;    // proof.cuh

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

// Resident files: with `on`, loadbin / savebin (ioutils) keep a device copy of every file they
// touch, up to limit_bytes in total (0 = keep the current limit, 24 GiB at first; least recently
// used files go first), and a later loadbin of an unchanged file copies from the device instead of
// reading the disk.  Off by default, like the reference, which reads every file again; turning it
// off releases the copies.  `zkllm-driver batch` turns it on.
struct ResidentStats {
    unsigned long long loads_from_disk = 0, loads_from_device = 0, bytes_from_disk = 0, bytes_from_device = 0, saved_files = 0;
};
void set_resident_files(bool on, size_t limit_bytes = 0);
ResidentStats resident_stats();

// Deferred writes: with `on`, savebin (and so every save / save_int / save_long) copies the tensor to a page-locked
// host buffer and returns; a writer thread puts it on disk.  flush_saves() returns when every such file is complete
// and throws if a write failed; loading a file that is still being written waits for it.  Off by default, like the
// reference, whose savebin returns with the file written.  `zkllm-driver batch` turns it on and flushes before it
// answers a line.
void set_deferred_saves(bool on);
void flush_saves();

// verifyWeightClaim (proof.cuh) in two halves: add() starts the opening of a weight commitment at a claim's point and
// returns; finish() waits for every opening started, compares each with its claim (throwing the reference's
// "verifyWeightClaim: opening != c.claim") and prints the reference's "Opening complete" line per opening.  Between the
// two the caller goes on proving: an opening keeps the multipliers busy, a lookup proof the memory.  The Weight must
// outlive finish(); the destructor waits without checking (use finish()).
class WeightOpenings {
public:
    WeightOpenings();
    ~WeightOpenings();
    WeightOpenings(const WeightOpenings&) = delete;
    WeightOpenings& operator=(const WeightOpenings&) = delete;
    void add(const ::Weight& w, const ::Claim& c);
    void finish();
private:
    struct Pending;
    std::vector<Pending*> pending_;
};

// Throws std::runtime_error(msg) when a C-ABI call failed; dimension and
// verifier failures carry the reference's message text.
void check(int rc);

}  // namespace zkllm
