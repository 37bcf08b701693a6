// 64-bit modular arithmetic shared by host precompute and device kernels.
//
// Device code keeps residues lazily reduced inside a kernel (forward butterflies in
// [0,4q), inverse in [0,2q)) and always stores the canonical residue in [0,q), which is
// what every stage of the reference library leaves in memory
// (cahel-main/src/ntt/fntt_2d.cu:860-866, cahel-main/include/uintmodmath.cuh:112-259).
#pragma once
#include <cstdint>

namespace lb {

typedef uint64_t u64;
typedef unsigned __int128 u128;

#if defined(__CUDACC__)
#define LB_HD __host__ __device__ __forceinline__
#define LB_D __device__ __forceinline__
#else
#define LB_HD inline
#define LB_D inline
#endif

// ---- host-only helpers (precompute) ---------------------------------------------------
#if defined(__x86_64__) && !defined(__CUDA_ARCH__)
// 128-by-64 division in one instruction; valid whenever the high half is below q
inline u64 h_div128(u64 hi, u64 lo, u64 q, u64 *rem)
{
    u64 quo, r;
    __asm__("divq %4" : "=a"(quo), "=d"(r) : "a"(lo), "d"(hi), "r"(q) : "cc");
    *rem = r;
    return quo;
}
inline u64 h_mulmod(u64 a, u64 b, u64 q)
{
    if (a >= q) a %= q;
    if (b >= q) b %= q;
    const u128 p = (u128)a * b;
    u64 r;
    h_div128((u64)(p >> 64), (u64)p, q, &r);
    return r;
}
#else
inline u64 h_mulmod(u64 a, u64 b, u64 q) { return (u64)((u128)a * b % q); }
#endif
inline u64 h_powmod(u64 b, u64 e, u64 q)
{
    u64 r = 1 % q;
    b %= q;
    for (; e; e >>= 1) {
        if (e & 1) r = h_mulmod(r, b, q);
        b = h_mulmod(b, b, q);
    }
    return r;
}
inline u64 h_invmod(u64 a, u64 q) { return h_powmod(a % q, q - 2, q); } // q prime
#if defined(__x86_64__) && !defined(__CUDA_ARCH__)
inline u64 h_shoup(u64 w, u64 q)
{
    if (w >= q) return (u64)(((u128)w << 64) / q);
    u64 r;
    return h_div128(w, 0, q, &r);
}
#else
inline u64 h_shoup(u64 w, u64 q) { return (u64)(((u128)w << 64) / q); }
#endif

// ---- the FP64 pipe in the transform kernels -----------------------------------------------------
// Primes below 2^50: the whole butterfly runs on the FP64 pipe.  Residues travel through the
// transform as integer-valued doubles (their bit patterns sit in the same 64-bit words), products
// are formed error-free with fused multiply-adds.  Below 2^47 values may grow over all forward stages
// without a reduction (13 q < 2^51); from 2^47 up they are centred once per pass (ntt_butterfly.cuh).
// Their twiddle entries are (double(w), double(w / q)).
constexpr u64 kF64TightPrimeLimit = u64(1) << 50; // below it the butterflies run on the FP64 pipe: 2q stays below 2^51
constexpr u64 kF64PrimeLimit = u64(1) << 47;

inline u64 h_bits_of(double d)
{
    u64 bits;
    static_assert(sizeof(bits) == sizeof(d), "double is 64 bits");
    __builtin_memcpy(&bits, &d, sizeof(bits));
    return bits;
}
inline u64 h_fp_quot(u64 w, u64 q)
{
    return h_bits_of((double)w / (double)q); // both exact in double, so the quotient is correctly rounded
}
// the two words of a twiddle-table entry for the power w of a root modulo prime q
// (primes below 2^50 run their butterflies on the FP64 pipe: the power as a double, and its quotient by q)
inline u64 h_twiddle_value(u64 w, u64 q) { return q < kF64TightPrimeLimit ? h_bits_of((double)w) : w; }
inline u64 h_twiddle_quot(u64 w, u64 q) { return q < kF64TightPrimeLimit ? h_fp_quot(w, q) : h_shoup(w, q); }

#if defined(__CUDACC__)
// ---- device arithmetic ----------------------------------------------------------------

// ---- residues as integer-valued doubles (primes below 2^50) --------------------------------------
LB_D double f64_of(u64 bits) { return __longlong_as_double((long long)bits); }
LB_D u64 bits_of(double d) { return (u64)__double_as_longlong(d); }
// an integer below 2^52 as a double: its bits under the exponent of 2^52, minus 2^52
LB_D double f64_from_u52(u64 x) { return __dadd_rn(__longlong_as_double((long long)(x | 0x4330000000000000ull)), -4503599627370496.0); }
// back: a double holding an integer of [0, 2^52)
LB_D u64 u52_from_f64(double d) { return (u64)__double_as_longlong(__dadd_rn(d, 4503599627370496.0)) & 0x000FFFFFFFFFFFFFull; }

// r = y w - Q q with Q the integer nearest to y w / q: r is congruent to y w and |r| <= 0.75 q.
// Needs integer-valued |y| < 2^51, w < q < 2^47, wq = double(w / q).  y w is split error-free into
// h + l (l = fma(y, w, -h) is exact); Q comes from one fused multiply-add into 1.5 * 2^52, whose
// rounding is the rounding to an integer (|y wq| < 2^51 keeps the sum inside [2^52, 2^53)); the
// estimate is off by at most 0.5 + 2^-2.  h - Q q = (y w - Q q) - l is an integer below 2^50 in
// magnitude, so the second fused multiply-add is exact, and so is the final sum.
LB_D double f64_mulmod(const double y, const double w, const double wq, const double q)
{
    const double h = __dmul_rn(y, w);
    const double l = __fma_rn(y, w, -h);
    const double Q = __dadd_rn(__fma_rn(y, wq, 6755399441055744.0), -6755399441055744.0);
    return __dadd_rn(__fma_rn(-Q, q, h), l);
}
// the residue of an integer-valued |v| < 2^52 nearest to zero: |result| <= q / 2 (+ rounding of 1 / q)
LB_D double f64_centre(const double v, const double q, const double qinv)
{
    const double Q = __dadd_rn(__fma_rn(v, qinv, 6755399441055744.0), -6755399441055744.0);
    return __fma_rn(-Q, q, v);
}
// the canonical residue in [0, q) as an integer
LB_D u64 f64_canon(const double v, const double q, const double qinv)
{
    const double r = f64_centre(v, q, qinv);
    return u52_from_f64(r < 0.0 ? __dadd_rn(r, q) : r);
}

// x * w mod q in [0, 2q) for any 64-bit x, given ws = floor(w 2^64 / q), w < q.
LB_D u64 shoup_lazy(u64 x, u64 w, u64 ws, u64 q)
{
    u64 hi = __umul64hi(x, ws);
    return x * w - hi * q;
}

// The same with the high product formed from three 32 x 32 multiplications instead of four: the quotient comes out at
// most two too small (the product of the low halves and the carries of the cross terms are dropped, each worth less
// than one), so the result is congruent to x w and lies in [0, 4q).  For the butterflies, which only need a bound.
LB_D u64 shoup_lazy4(u64 x, u64 w, u64 ws, u64 q)
{
    const unsigned xh = (unsigned)(x >> 32), xl = (unsigned)x, sh = (unsigned)(ws >> 32), sl = (unsigned)ws;
    const u64 hi = (u64)xh * sh + __umulhi(xh, sl) + __umulhi(xl, sh);
    return x * w - hi * q;
}

LB_D u64 shoup_mul(u64 x, u64 w, u64 ws, u64 q)
{
    u64 r = shoup_lazy(x, w, ws, q);
    return r >= q ? r - q : r;
}

LB_D u64 csub(u64 x, u64 q) { return x >= q ? x - q : x; }

LB_D u64 add_mod(u64 a, u64 b, u64 q) { return csub(a + b, q); }
LB_D u64 sub_mod(u64 a, u64 b, u64 q) { return a >= b ? a - b : a + q - b; }

// x mod q for any 64-bit x, bhi = floor(2^64 / q)
LB_D u64 barrett64(u64 x, u64 q, u64 bhi)
{
    u64 s = __umul64hi(x, bhi);
    u64 r = x - s * q;
    return r >= q ? r - q : r;
}

struct u128d {
    u64 lo, hi;
};

LB_D u128d mul_wide(u64 a, u64 b)
{
    u128d r;
    r.lo = a * b;
    r.hi = __umul64hi(a, b);
    return r;
}

// acc += a * b; the 128-bit integer type lets the compiler share partial products between the
// two halves and keep the additions on the carry chain
LB_D void mac_wide(u128d &acc, u64 a, u64 b)
{
    const u128 s = ((u128)acc.hi << 64 | acc.lo) + (u128)a * b;
    acc.lo = (u64)s;
    acc.hi = (u64)(s >> 64);
}

// (hi:lo) mod q with the two-word ratio floor(2^128 / q) = (r1:r0); exact for q < 2^62.
LB_D u64 barrett128(u128d z, u64 q, u64 r0, u64 r1)
{
    // quotient estimate: floor(z * ratio / 2^128), dropping the lowest partial product
    u64 carry = __umul64hi(z.lo, r0);
    u64 t_lo = z.lo * r1;
    u64 t_hi = __umul64hi(z.lo, r1);
    u64 s = t_lo + carry;
    u64 c1 = t_hi + (s < t_lo);
    u64 u_lo = z.hi * r0;
    u64 u_hi = __umul64hi(z.hi, r0);
    u64 s2 = s + u_lo;
    u64 c2 = u_hi + (s2 < u_lo);
    u64 qhat = z.hi * r1 + c1 + c2;
    u64 r = z.lo - qhat * q;
    // the estimate is short by at most 2
    r = csub(r, q << 1);
    return csub(r, q);
}

LB_D u64 mul_mod(u64 a, u64 b, u64 q, u64 r0, u64 r1) { return barrett128(mul_wide(a, b), q, r0, r1); }
#endif

// Per-modulus constants as laid out in device memory (one entry per prime of QP).
struct ModConst {
    u64 q;
    u64 r0, r1;      // floor(2^128 / q), low and high word
    u64 ninv, ninvs; // N^-1 mod q and its Shoup quotient
    u64 iw1n, iw1ns; // psi^-bitrev(1) * N^-1 (last inverse stage fused with the scaling)
    u64 pad;
};

} // namespace lb
