// Stand-in for the one OpenFHE header the reference's secretkey.cu includes.  It only
// provides the few names that file touches, and its "Gaussian" polynomial is all zeros,
// so decryption in the checker build adds no noise-flooding term and is deterministic.
// Test infrastructure: used when compiling the reference sources into oracle/_ref.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <vector>

namespace lbcrypto {

struct NativeInteger {
    uint64_t v;
    NativeInteger(uint64_t x = 0) : v(x) {}
};

enum Format { EVALUATION = 0, COEFFICIENT = 1 };

struct ShimValues {
    std::vector<uint64_t> d;
    const uint64_t &at(size_t i) const { return d.at(i); }
};

struct ShimPoly {
    ShimValues vals;
    const ShimValues &GetValues() const { return vals; }
};

struct DCRTPoly {
    struct DggType {
        explicit DggType(double) {}
    };
    struct Params {
        size_t order;
        std::vector<NativeInteger> moduli;
        Params(size_t o, const std::vector<NativeInteger> &m) : order(o), moduli(m) {}
    };
    std::vector<ShimPoly> elems;
    DCRTPoly(const DggType &, const std::shared_ptr<Params> &p, Format)
    {
        elems.resize(p->moduli.size());
        for (auto &e : elems) e.vals.d.assign(p->order / 2, 0);
    }
    const std::vector<ShimPoly> &GetAllElements() const { return elems; }
};

} // namespace lbcrypto
