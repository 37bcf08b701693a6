#include "params.h"

#include <algorithm>
#include <map>

namespace lb {

bool is_prime(u64 n)
{
    // Miller-Rabin with the first twelve prime bases is exact for every 64-bit integer.
    static const u64 bases[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
    if (n < 2) return false;
    for (u64 b : bases) {
        if (n == b) return true;
        if (n % b == 0) return false;
    }
    u64 d = n - 1;
    int s = 0;
    while ((d & 1) == 0) {
        d >>= 1;
        ++s;
    }
    for (u64 b : bases) {
        u64 x = h_powmod(b, d, n);
        if (x == 1 || x == n - 1) continue;
        bool witness = true;
        for (int i = 1; i < s && witness; ++i) {
            x = h_mulmod(x, x, n);
            if (x == n - 1) witness = false;
        }
        if (witness) return false;
    }
    return true;
}

std::vector<u64> get_primes(u64 N, int bit_size, int count)
{
    std::vector<u64> out;
    const u64 step = 2 * N;
    const u64 floor_value = u64(1) << (bit_size - 1);
    for (u64 cand = (u64(1) << bit_size) - step + 1; (int)out.size() < count && cand > floor_value; cand -= step)
        if (is_prime(cand)) out.push_back(cand);
    if ((int)out.size() < count) out.clear();
    return out;
}

std::vector<u64> coeff_modulus_create(u64 N, const std::vector<int> &bit_sizes)
{
    std::map<int, int> wanted;
    for (int b : bit_sizes) ++wanted[b];
    std::map<int, std::vector<u64>> pool;
    for (auto &kv : wanted) {
        pool[kv.first] = get_primes(N, kv.first, kv.second);
        if (pool[kv.first].empty()) return {};
    }
    std::map<int, size_t> next;
    std::vector<u64> result;
    for (int b : bit_sizes) result.push_back(pool[b][next[b]++]);
    return result;
}

u64 minimal_primitive_root(u64 degree, u64 q)
{
    if ((q - 1) % degree != 0) return 0;
    const u64 cofactor = (q - 1) / degree;
    u64 gen = 0;
    for (u64 x = 2; x < q && gen == 0; ++x) {
        u64 r = h_powmod(x, cofactor, q);
        if (h_powmod(r, degree / 2, q) == q - 1) gen = r;
    }
    // every primitive root is an odd power of gen; walk them all and keep the smallest
    const u64 sq = h_mulmod(gen, gen, q);
    u64 best = gen, cur = gen;
    for (u64 i = 1; i < degree / 2; ++i) {
        cur = h_mulmod(cur, sq, q);
        best = std::min(best, cur);
    }
    return best;
}

uint32_t bit_reverse(uint32_t x, int bits)
{
    if (bits <= 0) return 0;
    x = ((x >> 1) & 0x55555555u) | ((x & 0x55555555u) << 1);
    x = ((x >> 2) & 0x33333333u) | ((x & 0x33333333u) << 2);
    x = ((x >> 4) & 0x0F0F0F0Fu) | ((x & 0x0F0F0F0Fu) << 4);
    x = ((x >> 8) & 0x00FF00FFu) | ((x & 0x00FF00FFu) << 8);
    x = (x >> 16) | (x << 16);
    return x >> (32 - bits);
}

uint32_t galois_elt_from_step(int step, u64 N)
{
    const uint32_t m = (uint32_t)(2 * N);
    if (step == 0) return m - 1; // conjugation
    int s = step > 0 ? step : (int)(N / 2) + step; // right rotation by k == left rotation by N/2 - k
    u64 e = 1;
    for (int i = 0; i < s; ++i) e = (e * 5) & (m - 1);
    return (uint32_t)e;
}

int max_bit_count_tc128(u64 N)
{
    switch (N) {
    case 1024: return 27;
    case 2048: return 54;
    case 4096: return 109;
    case 8192: return 218;
    case 16384: return 438;
    case 32768: return 881;
    case 65536: return 1777;
    case 131072: return 3576;
    default: return 0;
    }
}

static u64 prod_mod(const std::vector<u64> &factors, int skip, u64 q)
{
    u64 r = 1 % q;
    for (int i = 0; i < (int)factors.size(); ++i)
        if (i != skip) r = h_mulmod(r, factors[i] % q, q);
    return r;
}

bool HostParams::init(int logN_, const std::vector<u64> &moduli, int size_P_, const std::vector<uint32_t> &elts)
{
    logN = logN_;
    N = u64(1) << logN;
    size_QP = (int)moduli.size();
    size_P = size_P_;
    size_Q = size_QP - size_P;
    if (logN < 4 || logN > 17) { error = "poly_modulus_degree is invalid"; return false; }
    if (size_QP < 1 || size_QP > 64) { error = "coeff_modulus size is invalid"; return false; }
    if (size_P < 0 || size_Q < 1) { error = "special_modulus_size is invalid"; return false; }
    q = moduli;
    for (int i = 0; i < size_QP; ++i) {
        // 60 bits at most, as CoeffModulus::Create hands them out (cahel-main/src/modulus.cu:93-125); the lazy ranges
        // of the kernels (differences below 2^61, sums of 63 products in 128 bits, eight residues in 64) rely on it
        if (q[i] >> 60) { error = "coeff_modulus primes must be below 2^60"; return false; }
        for (int j = 0; j < i; ++j)
            if (q[i] == q[j]) { error = "coeff_modulus primes must be distinct"; return false; }
    }

    psi.resize(size_QP);
    mc.resize(size_QP);
    tw.assign((size_t)size_QP * N * 2, 0);
    itw.assign((size_t)size_QP * N * 2, 0);
    for (int m = 0; m < size_QP; ++m) {
        const u64 p = q[m];
        if (!is_prime(p)) { error = "coeff_modulus entries must be prime"; return false; }
        psi[m] = minimal_primitive_root(2 * N, p);
        if (psi[m] == 0) { error = "invalid modulus: no primitive 2N-th root"; return false; }
        const u64 ipsi = h_invmod(psi[m], p);
        u64 *t = &tw[(size_t)m * N * 2], *it = &itw[(size_t)m * N * 2];
        u64 pw = 1, ipw = 1, ipw_at_1 = 1; // ipw_at_1: the inverse table's entry 1 as an integer (psi^-(N/2))
        for (u64 i = 0; i < N; ++i) {
            const uint32_t r = bit_reverse((uint32_t)i, logN);
            if (r == 1) ipw_at_1 = ipw;
            t[2 * r] = h_twiddle_value(pw, p);
            t[2 * r + 1] = h_twiddle_quot(pw, p);
            it[2 * r] = h_twiddle_value(ipw, p);
            it[2 * r + 1] = h_twiddle_quot(ipw, p);
            pw = h_mulmod(pw, psi[m], p);
            ipw = h_mulmod(ipw, ipsi, p);
        }
        ModConst &c = mc[m];
        c.q = p;
        const u128 ratio = (~u128(0)) / p; // floor((2^128 - 1) / p) == floor(2^128 / p) for odd p > 1
        c.r0 = (u64)ratio;
        c.r1 = (u64)(ratio >> 64);
        c.ninv = h_invmod(N % p, p);
        c.ninvs = h_shoup(c.ninv, p);
        c.iw1n = h_mulmod(ipw_at_1, c.ninv, p);
        c.iw1ns = h_shoup(c.iw1n, p);
        c.pad = 0;
    }

    galois_elts = elts;
    perm.assign(elts.size() * N, 0);
    for (size_t e = 0; e < elts.size(); ++e) {
        if ((elts[e] & 1u) == 0 || elts[e] >= 2 * N) { error = "Galois element is not valid"; return false; }
        for (u64 i = 0; i < N; ++i) {
            const uint32_t rev = bit_reverse((uint32_t)(N + i), logN + 1);
            const u64 raw = ((u64)elts[e] * rev) >> 1 & (N - 1);
            perm[e * N + i] = bit_reverse((uint32_t)raw, logN);
        }
    }

    std::vector<u64> special(q.begin() + size_Q, q.end());
    p_mod_q.resize(size_Q);
    p_mod_q_s.resize(size_Q);
    for (int r = 0; r < size_Q; ++r) {
        p_mod_q[r] = prod_mod(special, -1, q[r]);
        p_mod_q_s[r] = h_shoup(p_mod_q[r], q[r]);
    }

    level.assign(size_Q + 1, LevelConst());
    for (int L = 1; L <= size_Q; ++L) {
        LevelConst &lc = level[L];
        lc.size_l = L;
        const u64 ql = q[L - 1];
        for (int r = 0; r + 1 < L; ++r) {
            lc.qlast_inv.push_back(h_invmod(ql % q[r], q[r]));
            lc.qlast_inv_s.push_back(h_shoup(lc.qlast_inv.back(), q[r]));
        }
        if (size_P == 0) continue;
        const int alpha = size_P, LP = L + size_P;
        lc.beta = (L + alpha - 1) / alpha;
        for (int r = 0; r < L; ++r) {
            lc.p_inv.push_back(h_invmod(p_mod_q[r], q[r]));
            lc.p_inv_s.push_back(h_shoup(lc.p_inv.back(), q[r]));
        }
        lc.hat_inv.assign(L, 0);
        lc.hat_inv_s.assign(L, 0);
        lc.hat_mod.assign((size_t)lc.beta * LP * alpha, 0);
        for (int j = 0; j < lc.beta; ++j) {
            const int s = j * alpha, e = std::min(L, s + alpha);
            std::vector<u64> digit(q.begin() + s, q.begin() + e);
            for (int i = s; i < e; ++i) {
                lc.hat_inv[i] = h_invmod(prod_mod(digit, i - s, q[i]), q[i]);
                lc.hat_inv_s[i] = h_shoup(lc.hat_inv[i], q[i]);
                for (int r = 0; r < LP; ++r) {
                    const u64 mr = q[table_index(L, r)];
                    lc.hat_mod[((size_t)j * LP + r) * alpha + (i - s)] = prod_mod(digit, i - s, mr);
                }
            }
        }
        lc.phat_inv.resize(size_P);
        lc.phat_inv_s.resize(size_P);
        lc.phat_mod.assign((size_t)L * size_P, 0);
        for (int i = 0; i < size_P; ++i) {
            const u64 pi = special[i];
            lc.phat_inv[i] = h_invmod(prod_mod(special, i, pi), pi);
            lc.phat_inv_s[i] = h_shoup(lc.phat_inv[i], pi);
            for (int r = 0; r < L; ++r) lc.phat_mod[(size_t)r * size_P + i] = prod_mod(special, i, q[r]);
        }
    }
    return true;
}

} // namespace lb
