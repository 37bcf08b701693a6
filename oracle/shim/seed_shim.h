// Force-included (-include) ahead of every reference source when building oracle/_ref.
// The reference draws every PRNG seed from std::random_device (cahel-main/include/prng.cuh:12-23)
// and has no seeding API.  This header swaps that type for a logged, deterministic word
// stream so the harness knows exactly which 64-byte seeds each call consumed.
// Test infrastructure only; nothing here is part of the product.
#pragma once
#include <cstdint>
#include <random>
#include <string>

extern "C" uint32_t lb_shim_next_word(void);

namespace std {
struct lb_seeded_random_device {
    typedef unsigned int result_type;
    lb_seeded_random_device() {}
    explicit lb_seeded_random_device(const std::string &) {}
    explicit lb_seeded_random_device(const char *) {}
    static constexpr result_type min() { return 0u; }
    static constexpr result_type max() { return 0xFFFFFFFFu; }
    result_type operator()() { return lb_shim_next_word(); }
    double entropy() const { return 32.0; }
};
} // namespace std

#define random_device lb_seeded_random_device
