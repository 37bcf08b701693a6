// Host-side parameter generation and constant tables for the CKKS path.
//
// Everything here is a deterministic function of (N, modulus list, special-prime count,
// Galois elements) and must reproduce the reference library's choices exactly, because
// ciphertext bit-exactness depends on identical primes, roots and conversion constants:
//   primes          cahel-main/src/modulus.cu:93-125, cahel-main/src/util/numth.cu:209-235
//   roots / tables  cahel-main/src/util/ntt.cu:32-80, cahel-main/src/util/numth.cu:311-333
//   modulus chain   cahel-main/src/context.cu:352-403
//   RNS constants   cahel-main/src/util/rns.cu:218-270,374-431,433-556
//   Galois tables   cahel-main/include/galois.cuh:22-75,155-192
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "modarith.cuh"

namespace lb {

bool is_prime(u64 n);
// Primes p = 1 mod 2N of exactly `bit_size` bits, largest first.
std::vector<u64> get_primes(u64 N, int bit_size, int count);
// One prime per requested bit size; equal sizes receive distinct primes, largest first.
std::vector<u64> coeff_modulus_create(u64 N, const std::vector<int> &bit_sizes);
u64 minimal_primitive_root(u64 degree, u64 q);
uint32_t bit_reverse(uint32_t x, int bits);
uint32_t galois_elt_from_step(int step, u64 N);
// Upper bound on the total coefficient-modulus bit count for 128-bit classical security
// (cahel-main/include/util/hestdparms.h), 0 when N is outside the table.
int max_bit_count_tc128(u64 N);

// Constants of one data level (size_l data limbs in use).
struct LevelConst {
    int size_l = 0, beta = 0;
    std::vector<u64> qlast_inv, qlast_inv_s; // [size_l-1]  q_last^-1 mod q_r (+ Shoup)
    std::vector<u64> p_inv, p_inv_s;         // [size_l]    P^-1 mod q_r
    // mod-up, per source limb i: (Q_digit / q_i)^-1 mod q_i
    std::vector<u64> hat_inv, hat_inv_s; // [size_l]
    // mod-up matrix: for digit j, output row r of QlP (0..size_l+size_p-1, own rows unused),
    // input i in the digit: (Q_digit / q_i) mod modulus(r).   index ((j*LP + r)*alpha + i)
    std::vector<u64> hat_mod;
    // mod-down: (P / p_i)^-1 mod p_i  [size_p], and (P / p_i) mod q_r  [size_l][size_p]
    std::vector<u64> phat_inv, phat_inv_s;
    std::vector<u64> phat_mod;
};

struct HostParams {
    int logN = 0;
    u64 N = 0;
    int size_QP = 0, size_Q = 0, size_P = 0;
    std::vector<u64> q, psi;
    std::vector<ModConst> mc;             // [size_QP]
    std::vector<u64> tw, itw;             // [size_QP][N][2]  (value, Shoup quotient or, below 2^50, the double value / q), index m + k
    std::vector<uint32_t> galois_elts;    // as given by the caller
    std::vector<uint32_t> perm;           // [n_elts][N]
    std::vector<LevelConst> level;        // index = size_l (1..size_Q); [0] unused
    std::vector<u64> p_mod_q, p_mod_q_s;  // [size_Q]  P mod q_r (key generation)
    std::string error;

    bool init(int logN, const std::vector<u64> &moduli, int size_P, const std::vector<uint32_t> &elts);
    int table_index(int size_l, int row) const { return row < size_l ? row : size_Q + (row - size_l); }
};

} // namespace lb
