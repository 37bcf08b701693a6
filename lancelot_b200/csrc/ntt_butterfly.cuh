// The modular butterflies of the transform kernels (ntt.cu), shared with the register-only
// rate probe of the diagnostics (diag.cu).
#pragma once
#include "modarith.cuh"

namespace lb {

// Butterfly variants, chosen per prime:
//   integer, strict: Shoup product on the integer multiplier with a three-multiplication high part
//                    (shoup_lazy4), values kept in [0, 8q);
//   integer, lazy:   the prime is below 2^58, so x may grow by 2q per stage over all seventeen
//                    possible stages (bound 35q < 2^64) and the per-butterfly conditional
//                    subtraction is dropped; the closing pass reduces once;
//   FP64:            primes below 2^47, the whole butterfly on the FP64 pipe (f64_mulmod): eight
//                    double-precision operations and nothing on the integer pipes.  The 64-bit
//                    words then hold the bit patterns of integer-valued doubles; in this mode the
//                    scalars q and q2 of the butterfly functions carry double(q) and double(1 / q);
//   FP64, tight:     the same butterflies for primes of [2^47, 2^50).  The multiplicand of a butterfly
//                    must stay below 2^51 (hardly more than 2q here) and a value grows by up to 0.75 q
//                    per stage, so every element is brought back to the residue nearest zero when a
//                    pass loads it (|v| <= q / 2, at most 2q before the third stage) and once more
//                    inside a pass of four stages.
// Every variant leaves the same canonical residues in memory.
enum { kIntStrict = 0, kIntLazy = 1, kF64Tight = 2, kF64 = 3 };
LB_D constexpr bool is_f64_mode(const int mode) { return mode == kF64 || mode == kF64Tight; }

LB_D int butterfly_mode(const u64 q)
{
    if (q < kF64PrimeLimit) return kF64;
    if (q < kF64TightPrimeLimit) return kF64Tight;
    return (q >> 58) == 0 ? kIntLazy : kIntStrict;
}

// the two scalars the butterflies of a mode take: (q, 2q), or (double(q), double(1 / q)) as bit patterns
template <int MODE>
LB_D u64 bf_scalar_q(const u64 q) { return is_f64_mode(MODE) ? bits_of((double)q) : q; }
template <int MODE>
LB_D u64 bf_scalar_q2(const u64 q) { return is_f64_mode(MODE) ? bits_of(1.0 / (double)q) : q << 1; }

template <int MODE>
LB_D void fwd_bf(u64 &x, u64 &y, const ulonglong2 w, const u64 q, const u64 q2)
{
    if (is_f64_mode(MODE)) {
        const double xd = f64_of(x), r = f64_mulmod(f64_of(y), f64_of(w.x), f64_of(w.y), f64_of(q));
        y = bits_of(__dadd_rn(xd, -r));
        x = bits_of(__dadd_rn(xd, r));
        return;
    }
    if (MODE == kIntStrict) {
        // values below 8q between stages: x is brought below 4q, the product is below 4q (shoup_lazy4)
        const u64 q4 = q2 << 1;
        x = csub(x, q4);
        const u64 t = shoup_lazy4(y, w.x, w.y, q);
        y = x + q4 - t;
        x = x + t;
        return;
    }
    const u64 t = shoup_lazy(y, w.x, w.y, q);
    y = x + q2 - t;
    x = x + t;
}

// inverse butterfly kinds: the integer Shoup product, or all on the FP64 pipe
// kInvF64Tight: kInvF64 for primes of [2^47, 2^50): the sums double per stage and the difference that is multiplied
// must stay below 2^51, so the values are centred when a pass loads them and again after every second stage
enum { kInvInt = 0, kInvF64Tight = 1, kInvF64 = 2 };
LB_D constexpr bool is_inv_f64(const int im) { return im == kInvF64 || im == kInvF64Tight; }

LB_D int inverse_mode(const u64 q) { return q < kF64PrimeLimit ? kInvF64 : q < kF64TightPrimeLimit ? kInvF64Tight : kInvInt; }
template <int IM>
LB_D u64 inv_scalar_q(const u64 q) { return is_inv_f64(IM) ? bits_of((double)q) : q; }
template <int IM>
LB_D u64 inv_scalar_q2(const u64 q) { return is_inv_f64(IM) ? bits_of(1.0 / (double)q) : q << 1; }

template <int IM>
LB_D void inv_bf(u64 &x, u64 &y, const ulonglong2 w, const u64 q, const u64 q2)
{
    if (is_inv_f64(IM)) {
        // the sum doubles its magnitude per stage: the passes reduce where 2^51 comes into reach
        const double xd = f64_of(x), yd = f64_of(y);
        x = bits_of(__dadd_rn(xd, yd));
        y = bits_of(f64_mulmod(__dadd_rn(xd, -yd), f64_of(w.x), f64_of(w.y), f64_of(q)));
        return;
    }
    // values below 4q between stages: the sum is brought back below 4q, the product is below 4q (shoup_lazy4)
    const u64 q4 = q2 << 1;
    const u64 s = csub(x + y, q4);
    const u64 d = x + q4 - y; // below 8q
    x = s;
    y = shoup_lazy4(d, w.x, w.y, q);
}

} // namespace lb
