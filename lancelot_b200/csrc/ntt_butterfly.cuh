// The modular butterflies of the transform kernels (ntt.cu), shared with the register-only
// rate probe of the diagnostics (diag.cu).
#pragma once
#include "modarith.cuh"

namespace lb {

// Butterfly variants, chosen per prime:
//   integer, strict: Shoup product on the integer multiplier, values kept in [0, 4q);
//   integer, lazy:   the prime is below 2^58, so x may grow by 2q per stage over all seventeen
//                    possible stages (bound 35q < 2^64) and the per-butterfly conditional
//                    subtraction is dropped; the closing pass reduces once;
//   FP64, strict / lazy: primes below 2^50 / 2^46, quotient estimated on the FP64 pipe
//                    (fp_mul_signed), which takes the 64 x 64 -> 128 bit product off the
//                    integer multiplier, the pipe that bounds these kernels.
// Every variant leaves the same canonical residues in memory.
enum { kIntStrict = 0, kIntLazy = 1, kFpStrict = 2, kFpLazy = 3 };

LB_D int butterfly_mode(const u64 q)
{
    if (q < kFpLazyLimit) return kFpLazy;
    if (q < kFpPrimeLimit) return kFpStrict;
    return (q >> 58) == 0 ? kIntLazy : kIntStrict;
}

template <int MODE>
LB_D void fwd_bf(u64 &x, u64 &y, const ulonglong2 w, const u64 q, const u64 q2)
{
    if (MODE == kIntStrict || MODE == kFpStrict) x = csub(x, q2);
    if (MODE == kFpStrict || MODE == kFpLazy) {
        const u64 r = fp_mul_signed(y, w.x, w.y, q), xq = x + q; // r in (-q, q)
        y = xq - r;
        x = xq + r;
    } else {
        const u64 t = shoup_lazy(y, w.x, w.y, q);
        y = x + q2 - t;
        x = x + t;
    }
}

template <bool FP>
LB_D void inv_bf(u64 &x, u64 &y, const ulonglong2 w, const u64 q, const u64 q2)
{
    const u64 s = csub(x + y, q2);
    const u64 d = x + q2 - y; // below 4q
    x = s;
    y = FP ? fp_mul_signed(d, w.x, w.y, q) + q : shoup_lazy(d, w.x, w.y, q);
}

} // namespace lb
