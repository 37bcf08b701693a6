/*
 * CPU restatement of CAHEL's CKKS encrypted-aggregation path (TEST INFRASTRUCTURE).
 *
 * This file is the checker, never the product: only tests, the smoke entry and the
 * benchmark's cpu_baseline / reference legs may load it.  It restates, in plain C with
 * 128-bit integers, the mathematical definition of every step that the reference
 * library (cahel-main) runs on the GPU.  Every stage output of the reference is the
 * canonical residue in [0,q), so a different internal schedule is bit-identical as
 * long as the same primes, roots, digit partition, approximate base conversion and
 * operation order are used.  Each function cites the reference file:line it follows.
 *
 * Parity pin: scalar known answers from cahel-main/unittest/util (checked in
 * tests/test_oracle_kat.py) and fixtures produced by running the reference library
 * itself on a GPU (tests/golden, produced by oracle/ref_harness.cu).
 *
 * Layouts (cahel-main/include/ciphertext.h:7, plaintext.h:11):
 *   polynomial  [limb][N] u64,  ciphertext [poly][limb][N],  key pair [2][size_QP][N],
 *   switch key  [dnum][2][size_QP][N],  mod-up digits [beta][size_Ql+size_P][N].
 * In a QlP buffer the special limbs follow the Ql data limbs; their modulus/table
 * index is size_Q + i (cahel-main/src/eval_key_switch.cu:27).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef uint64_t u64;
typedef unsigned __int128 u128;

#define ORC_MAX_MOD 64
#define ORC_MAX_ELTS 64

typedef struct orc_ctx {
    int logN;
    size_t N;
    int size_QP, size_Q, size_P;
    u64 q[ORC_MAX_MOD];
    u64 psi[ORC_MAX_MOD];
    u64 *w[ORC_MAX_MOD], *ws[ORC_MAX_MOD];   /* psi^bitrev(i) and its Shoup quotient */
    u64 *iw[ORC_MAX_MOD], *iws[ORC_MAX_MOD]; /* psi^-bitrev(i) and quotient          */
    int n_elts;
    uint32_t elts[ORC_MAX_ELTS];
    uint32_t *perm[ORC_MAX_ELTS];
} orc_ctx;

/* ---------------------------------------------------------------- scalar helpers */

static inline u64 mulmod(u64 a, u64 b, u64 q) { return (u64)((u128)a * b % q); }
static inline u64 addmod(u64 a, u64 b, u64 q) { u64 s = a + b; return s >= q ? s - q : s; }
static inline u64 submod(u64 a, u64 b, u64 q) { return a >= b ? a - b : a + q - b; }

u64 orc_mulmod(u64 a, u64 b, u64 q) { return mulmod(a, b, q); }

u64 orc_powmod(u64 b, u64 e, u64 q)
{
    u64 r = 1 % q;
    b %= q;
    while (e) {
        if (e & 1) r = mulmod(r, b, q);
        b = mulmod(b, b, q);
        e >>= 1;
    }
    return r;
}

/* q prime */
u64 orc_invmod(u64 a, u64 q) { return orc_powmod(a % q, q - 2, q); }

/* floor(w * 2^64 / q): the quotient half of a Shoup operand
 * (cahel-main/include/util/uintarithsmallmod.h MultiplyUIntModOperand::set_quotient). */
u64 orc_shoup(u64 w, u64 q) { return (u64)(((u128)w << 64) / q); }

static inline u64 mulmod_shoup(u64 x, u64 w, u64 ws, u64 q)
{
    u64 hi = (u64)(((u128)x * ws) >> 64);
    u64 r = x * w - hi * q;
    return r >= q ? r - q : r;
}

/* Deterministic Miller-Rabin, exact below 2^64.  The reference's test is the
 * randomised one (cahel-main/src/util/numth.cu:160-206); both accept exactly the primes. */
int orc_is_prime(u64 n)
{
    static const u64 small[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
    if (n < 2) return 0;
    for (size_t i = 0; i < sizeof(small) / sizeof(small[0]); i++) {
        if (n == small[i]) return 1;
        if (n % small[i] == 0) return 0;
    }
    u64 d = n - 1;
    int r = 0;
    while (!(d & 1)) { d >>= 1; r++; }
    for (size_t i = 0; i < sizeof(small) / sizeof(small[0]); i++) {
        u64 x = orc_powmod(small[i], d, n);
        if (x == 1 || x == n - 1) continue;
        int comp = 1;
        for (int j = 1; j < r; j++) {
            x = mulmod(x, x, n);
            if (x == n - 1) { comp = 0; break; }
        }
        if (comp) return 0;
    }
    return 1;
}

/* cahel-main/src/util/numth.cu:209-235 get_primes: candidates 2^b - 2N*k + 1, k = 1,2,..,
 * descending, stop at 2^(b-1).  Returns how many were found. */
int orc_get_primes(u64 N, int bit_size, int count, u64 *out)
{
    u64 factor = 2 * N;
    u64 value = ((u64)1 << bit_size) - factor + 1;
    u64 lower = (u64)1 << (bit_size - 1);
    int found = 0;
    while (found < count && value > lower) {
        if (orc_is_prime(value)) out[found++] = value;
        value -= factor;
    }
    return found;
}

/* cahel-main/src/modulus.cu:93-125 CoeffModulus::Create: a bit size requested m times
 * receives the m largest qualifying primes, handed out largest first in request order. */
int orc_coeff_modulus_create(u64 N, const int *bit_sizes, int n, u64 *out)
{
    int used[64] = {0};
    for (int i = 0; i < n; i++) {
        int b = bit_sizes[i];
        int cnt = 0;
        for (int j = 0; j < n; j++) cnt += (bit_sizes[j] == b);
        u64 tmp[ORC_MAX_MOD];
        if (orc_get_primes(N, b, cnt, tmp) != cnt) return -1;
        out[i] = tmp[used[b]++];
    }
    return 0;
}

static uint32_t bitrev(uint32_t x, int bits)
{
    uint32_t r = 0;
    for (int i = 0; i < bits; i++) r |= ((x >> i) & 1u) << (bits - 1 - i);
    return r;
}
uint32_t orc_bitrev(uint32_t x, int bits) { return bitrev(x, bits); }

/* cahel-main/src/util/numth.cu:311-333: numerically smallest primitive 2N-th root. */
u64 orc_minimal_primitive_root(u64 degree, u64 q)
{
    if ((q - 1) % degree) return 0;
    u64 quo = (q - 1) / degree, root = 0;
    for (u64 x = 2; x < q; x++) {
        u64 r = orc_powmod(x, quo, q);
        if (orc_powmod(r, degree >> 1, q) == q - 1) { root = r; break; }
    }
    u64 gsq = mulmod(root, root, q), cur = root, best = root;
    for (u64 i = 0; i < degree / 2; i++) {
        if (cur < best) best = cur;
        cur = mulmod(cur, gsq, q);
    }
    return best;
}

/* ---------------------------------------------------------------- context */

/* cahel-main/include/galois.cuh:42-57: NTT-domain permutation table of one element. */
static void build_perm(uint32_t *tab, uint32_t elt, int logN)
{
    uint32_t N = 1u << logN;
    for (uint32_t i = 0; i < N; i++) {
        uint32_t rev = bitrev(N + i, logN + 1);
        u64 raw = ((u64)elt * rev) >> 1;
        raw &= (N - 1);
        tab[i] = bitrev((uint32_t)raw, logN);
    }
}

/* cahel-main/include/galois.cuh:155-192 get_elts_from_steps */
uint32_t orc_elt_from_step(int step, u64 N)
{
    uint32_t n = (uint32_t)N, m = 2 * n;
    if (step == 0) return m - 1;
    int neg = step < 0;
    uint32_t pos = (uint32_t)abs(step);
    int s = neg ? (int)(n >> 1) - (int)pos : (int)pos;
    u64 e = 1;
    while (s--) e = (e * 5) & (m - 1);
    return (uint32_t)e;
}

/* Tables follow cahel-main/src/util/ntt.cu:32-80: root_powers[bitrev(i)] = psi^i.  The
 * inverse table here holds psi^-i (the reference stores psi^-i / 2 and halves in every
 * butterfly; the transform is the same exact inverse map). */
orc_ctx *orc_create(int logN, const u64 *moduli, int size_QP, int size_P, const uint32_t *elts, int n_elts)
{
    orc_ctx *c = (orc_ctx *)calloc(1, sizeof(orc_ctx));
    c->logN = logN;
    c->N = (size_t)1 << logN;
    c->size_QP = size_QP;
    c->size_P = size_P;
    c->size_Q = size_QP - size_P;
    size_t N = c->N;
    for (int m = 0; m < size_QP; m++) {
        u64 q = moduli[m];
        c->q[m] = q;
        u64 psi = orc_minimal_primitive_root(2 * N, q);
        if (!psi) { free(c); return NULL; }
        c->psi[m] = psi;
        u64 ipsi = orc_invmod(psi, q);
        c->w[m] = (u64 *)malloc(N * 8); c->ws[m] = (u64 *)malloc(N * 8);
        c->iw[m] = (u64 *)malloc(N * 8); c->iws[m] = (u64 *)malloc(N * 8);
        u64 p = 1, ip = 1;
        for (size_t i = 0; i < N; i++) {
            uint32_t r = bitrev((uint32_t)i, logN);
            c->w[m][r] = p; c->ws[m][r] = orc_shoup(p, q);
            c->iw[m][r] = ip; c->iws[m][r] = orc_shoup(ip, q);
            p = mulmod(p, psi, q);
            ip = mulmod(ip, ipsi, q);
        }
    }
    c->n_elts = n_elts;
    for (int i = 0; i < n_elts; i++) {
        c->elts[i] = elts[i];
        c->perm[i] = (uint32_t *)malloc(N * 4);
        build_perm(c->perm[i], elts[i], logN);
    }
    return c;
}

void orc_destroy(orc_ctx *c)
{
    if (!c) return;
    for (int m = 0; m < c->size_QP; m++) { free(c->w[m]); free(c->ws[m]); free(c->iw[m]); free(c->iws[m]); }
    for (int i = 0; i < c->n_elts; i++) free(c->perm[i]);
    free(c);
}

u64 orc_get_modulus(const orc_ctx *c, int i) { return c->q[i]; }
u64 orc_get_psi(const orc_ctx *c, int i) { return c->psi[i]; }
const uint32_t *orc_get_perm(const orc_ctx *c, int i) { return c->perm[i]; }
const u64 *orc_get_twiddles(const orc_ctx *c, int mod, int inverse) { return inverse ? c->iw[mod] : c->w[mod]; }

/* table index of limb r of a QlP-shaped buffer with L data limbs */
static inline int tix(const orc_ctx *c, int L, int r) { return r < L ? r : c->size_Q + (r - L); }

/* ---------------------------------------------------------------- NTT */

/* Forward negacyclic NTT, cahel-main/src/ntt/ntt_1d.cu:38-74 + butterfly.cuh:10-20:
 * for m = 1,2,..,N/2, t = N/(2m): (x,y) = (a[2kt+j], a[2kt+j+t]) -> (x + w y, x - w y),
 * w = psi^bitrev(m+k).  Natural order in, bit-reversed order out, canonical residues. */
void orc_ntt_fwd(const orc_ctx *c, u64 *a, int mod)
{
    size_t N = c->N;
    u64 q = c->q[mod];
    const u64 *w = c->w[mod], *ws = c->ws[mod];
    for (size_t m = 1, t = N >> 1; m < N; m <<= 1, t >>= 1) {
        for (size_t k = 0; k < m; k++) {
            u64 W = w[m + k], Ws = ws[m + k];
            u64 *x = a + 2 * k * t, *y = x + t;
            for (size_t j = 0; j < t; j++) {
                u64 v = mulmod_shoup(y[j], W, Ws, q);
                u64 u = x[j];
                x[j] = addmod(u, v, q);
                y[j] = submod(u, v, q);
            }
        }
    }
}

/* Inverse, cahel-main/src/ntt/ntt_1d.cu:129-171 + butterfly.cuh:29-43: for m = N/2,..,1:
 * (x,y) -> ((x + y)/2, (x - y) w^-1 / 2).  Bit-reversed in, natural order out. */
void orc_ntt_inv(const orc_ctx *c, u64 *a, int mod)
{
    size_t N = c->N;
    u64 q = c->q[mod];
    const u64 *w = c->iw[mod], *ws = c->iws[mod];
    u64 half = (q + 1) >> 1; /* 2^-1 mod q */
    u64 halfs = orc_shoup(half, q);
    for (size_t m = N >> 1, t = 1; m >= 1; m >>= 1, t <<= 1) {
        for (size_t k = 0; k < m; k++) {
            u64 W = w[m + k], Ws = ws[m + k];
            u64 *x = a + 2 * k * t, *y = x + t;
            for (size_t j = 0; j < t; j++) {
                u64 u = x[j], v = y[j];
                x[j] = mulmod_shoup(addmod(u, v, q), half, halfs, q);
                y[j] = mulmod_shoup(mulmod_shoup(submod(u, v, q), W, Ws, q), half, halfs, q);
            }
        }
    }
}

/* Rows of (size_l data limbs + size_p special limbs), repeated n_groups times. */
void orc_ntt_rows(const orc_ctx *c, u64 *data, int n_groups, int size_l, int size_p, int inverse)
{
    int per = size_l + size_p;
    long total = (long)n_groups * per;
#pragma omp parallel for schedule(dynamic)
    for (long r = 0; r < total; r++) {
        int mod = tix(c, size_l, (int)(r % per));
        if (inverse) orc_ntt_inv(c, data + (size_t)r * c->N, mod);
        else orc_ntt_fwd(c, data + (size_t)r * c->N, mod);
    }
}

/* ---------------------------------------------------------------- element-wise (cahel-main/src/polymath.cu:16-227) */

/* op: 0 add, 1 sub, 2 mul, 3 negate(a) ; rows = n_polys*L limbs, limb r uses modulus r % L */
void orc_poly_op(const orc_ctx *c, int op, int L, int n_polys, const u64 *a, const u64 *b, u64 *out)
{
    size_t N = c->N;
#pragma omp parallel for
    for (int r = 0; r < n_polys * L; r++) {
        u64 q = c->q[r % L];
        const u64 *x = a + (size_t)r * N, *y = b ? b + (size_t)r * N : NULL;
        u64 *o = out + (size_t)r * N;
        for (size_t i = 0; i < N; i++) {
            switch (op) {
            case 0: o[i] = addmod(x[i], y[i], q); break;
            case 1: o[i] = submod(x[i], y[i], q); break;
            case 2: o[i] = mulmod(x[i], y[i], q); break;
            default: o[i] = x[i] ? q - x[i] : 0; break;
            }
        }
    }
}

/* cahel-main/src/polymath.cu:531-566 tensor_prod_2x2_rns_poly: (a0,a1)x(b0,b1) -> (a0b0, a0b1+a1b0, a1b1) */
void orc_tensor(const orc_ctx *c, int L, const u64 *a, const u64 *b, u64 *out)
{
    size_t N = c->N, S = (size_t)L * N;
#pragma omp parallel for
    for (int r = 0; r < L; r++) {
        u64 q = c->q[r];
        for (size_t i = 0; i < N; i++) {
            size_t k = (size_t)r * N + i;
            u64 a0 = a[k], a1 = a[S + k], b0 = b[k], b1 = b[S + k];
            out[k] = mulmod(a0, b0, q);
            out[S + k] = addmod(mulmod(a0, b1, q), mulmod(a1, b0, q), q);
            out[2 * S + k] = mulmod(a1, b1, q);
        }
    }
}

/* cahel-main/src/polymath.cu:568-600 tensor_square_2x2_rns_poly: (a0^2, 2 a0 a1, a1^2) */
void orc_square(const orc_ctx *c, int L, const u64 *a, u64 *out) { orc_tensor(c, L, a, a, out); }

/* ---------------------------------------------------------------- Galois (cahel-main/src/galois.cu:20-29) */

void orc_galois(const orc_ctx *c, int elt_idx, int n_limbs, const u64 *in, u64 *out)
{
    size_t N = c->N;
    const uint32_t *tab = c->perm[elt_idx];
    for (int r = 0; r < n_limbs; r++)
        for (size_t i = 0; i < N; i++) out[(size_t)r * N + i] = in[(size_t)r * N + tab[i]];
}

/* ---------------------------------------------------------------- base conversion */

/* Approximate fast base conversion (no overflow correction) from the primes listed in
 * in_idx to prime q_out: sum_i [x_i * (B/b_i)^-1]_{b_i} * ((B/b_i) mod q_out) mod q_out.
 * cahel-main/src/rns_bconv.cu:47-79 (phase 1), :166-199 (phase 2), host constants
 * cahel-main/src/util/rns.cu:218-270,374-431.  src limbs are in coefficient form. */
static void bconv(const orc_ctx *c, const int *in_idx, int n_in, const u64 *const *src, int out_mod, u64 *dst)
{
    size_t N = c->N;
    u64 qo = c->q[out_mod];
    u64 hatinv[ORC_MAX_MOD], hat_mod_out[ORC_MAX_MOD];
    for (int i = 0; i < n_in; i++) {
        u64 bi = c->q[in_idx[i]];
        u64 h = 1 % bi, ho = 1 % qo;
        for (int j = 0; j < n_in; j++) {
            if (j == i) continue;
            h = mulmod(h, c->q[in_idx[j]] % bi, bi);
            ho = mulmod(ho, c->q[in_idx[j]] % qo, qo);
        }
        hatinv[i] = orc_invmod(h, bi);
        hat_mod_out[i] = ho;
    }
    for (size_t k = 0; k < N; k++) {
        u128 acc = 0;
        for (int i = 0; i < n_in; i++) {
            u64 t = mulmod(src[i][k], hatinv[i], c->q[in_idx[i]]);
            acc += (u128)t * hat_mod_out[i];
        }
        dst[k] = (u64)(acc % qo);
    }
}

/* cahel-main/src/rns_bconv.cu:668-792 DRNSTool::modup.  cks [L][N] in NTT form ->
 * out [beta][L+P][N] in NTT form; digit j = limbs [j*alpha, min((j+1)*alpha, L)).
 * alpha == 1 takes `x mod r` of the canonical coefficient (rns_bconv.cu:562-585), which
 * equals the general formula for a one-prime base.  Own limbs keep the NTT input. */
void orc_modup(const orc_ctx *c, int L, const u64 *cks, u64 *out)
{
    size_t N = c->N;
    int P = c->size_P, alpha = P, LP = L + P;
    int beta = (L + alpha - 1) / alpha;
    u64 *coef = (u64 *)malloc((size_t)L * N * 8);
    memcpy(coef, cks, (size_t)L * N * 8);
    orc_ntt_rows(c, coef, 1, L, 0, 1);
    for (int j = 0; j < beta; j++) {
        int s = j * alpha, e = s + alpha < L ? s + alpha : L;
        int idx[ORC_MAX_MOD];
        const u64 *src[ORC_MAX_MOD];
        for (int i = s; i < e; i++) { idx[i - s] = i; src[i - s] = coef + (size_t)i * N; }
        u64 *dj = out + (size_t)j * LP * N;
#pragma omp parallel for
        for (int r = 0; r < LP; r++) {
            u64 *d = dj + (size_t)r * N;
            if (r >= s && r < e) { memcpy(d, cks + (size_t)r * N, N * 8); continue; }
            int mod = tix(c, L, r);
            bconv(c, idx, e - s, src, mod, d);
            orc_ntt_fwd(c, d, mod);
        }
    }
    free(coef);
}

/* cahel-main/src/eval_key_switch.cu:13-76: cx_t[r] = sum_j digit_j[r] * evk_j.t[r] mod r.
 * evk: [dnum][2][size_QP][N] (b then a).  out: [2][L+P][N]. */
void orc_inner_product(const orc_ctx *c, int L, const u64 *digits, const u64 *evk, u64 *out)
{
    size_t N = c->N;
    int P = c->size_P, LP = L + P, QP = c->size_QP;
    int beta = (L + P - 1) / P;
#pragma omp parallel for
    for (int r = 0; r < LP; r++) {
        int mod = tix(c, L, r);
        u64 q = c->q[mod];
        for (size_t k = 0; k < N; k++) {
            u128 a0 = 0, a1 = 0; /* beta <= 64 products below 2^120 fit 128 bits */
            for (int j = 0; j < beta; j++) {
                u64 d = digits[((size_t)j * LP + r) * N + k];
                const u64 *key = evk + (size_t)j * 2 * QP * N;
                a0 += (u128)d * key[(size_t)mod * N + k];
                a1 += (u128)d * key[((size_t)QP + mod) * N + k];
            }
            out[(size_t)r * N + k] = (u64)(a0 % q);
            out[((size_t)LP + r) * N + k] = (u64)(a1 % q);
        }
    }
}

/* cahel-main/src/rns_bconv.cu:965-1053 moddown_from_NTT (and :871-944 moddown, which is
 * the same map): delta = BConv_{P->Ql}(INTT(cx[P limbs])); out_i = (cx_i - NTT(delta)_i) P^-1 mod q_i
 * (cahel-main/src/ntt/ntt_moddown.cu:244-252).  cx [L+P][N] NTT -> out [L][N] NTT. */
void orc_moddown(const orc_ctx *c, int L, const u64 *cx, u64 *out)
{
    size_t N = c->N;
    int P = c->size_P;
    u64 *pc = (u64 *)malloc((size_t)P * N * 8);
    memcpy(pc, cx + (size_t)L * N, (size_t)P * N * 8);
    int idx[ORC_MAX_MOD];
    const u64 *src[ORC_MAX_MOD];
    for (int i = 0; i < P; i++) {
        idx[i] = c->size_Q + i;
        orc_ntt_inv(c, pc + (size_t)i * N, idx[i]);
        src[i] = pc + (size_t)i * N;
    }
#pragma omp parallel for
    for (int r = 0; r < L; r++) {
        u64 q = c->q[r];
        u64 pinv = 1;
        for (int i = 0; i < P; i++) pinv = mulmod(pinv, c->q[c->size_Q + i] % q, q);
        pinv = orc_invmod(pinv, q);
        u64 *delta = (u64 *)malloc(N * 8);
        bconv(c, idx, P, src, r, delta);
        orc_ntt_fwd(c, delta, r);
        for (size_t k = 0; k < N; k++)
            out[(size_t)r * N + k] = mulmod(submod(cx[(size_t)r * N + k], delta[k], q), pinv, q);
        free(delta);
    }
    free(pc);
}

/* cahel-main/src/eval_key_switch.cu:80-216 switch_key_inplace: ct[2][L][N] += moddown(<modup(cks), evk>) */
void orc_keyswitch(const orc_ctx *c, int L, u64 *ct, const u64 *cks, const u64 *evk)
{
    size_t N = c->N;
    int P = c->size_P, LP = L + P, beta = (L + P - 1) / P;
    u64 *dig = (u64 *)malloc((size_t)beta * LP * N * 8);
    u64 *cx = (u64 *)malloc((size_t)2 * LP * N * 8);
    u64 *md = (u64 *)malloc((size_t)L * N * 8);
    orc_modup(c, L, cks, dig);
    orc_inner_product(c, L, dig, evk, cx);
    for (int i = 0; i < 2; i++) {
        orc_moddown(c, L, cx + (size_t)i * LP * N, md);
        orc_poly_op(c, 0, L, 1, ct + (size_t)i * L * N, md, ct + (size_t)i * L * N);
    }
    free(dig); free(cx); free(md);
}

/* cahel-main/src/evaluate.cu:2019-2056: ct3 [3][L][N] -> (c0,c1) += KS(c2); result in ct3[0..1] */
void orc_relinearize(const orc_ctx *c, int L, u64 *ct3, const u64 *rlk)
{
    orc_keyswitch(c, L, ct3, ct3 + (size_t)2 * L * c->N, rlk);
}

/* cahel-main/src/rns.cu:507-570 divide_and_round_q_last_ntt (floors; no rounding term):
 * r = INTT(c_last); c'_j = (c_j - NTT_j(r mod q_j)) q_last^-1 mod q_j.  in [k][L][N] -> out [k][L-1][N] */
void orc_rescale(const orc_ctx *c, int L, int n_polys, const u64 *in, u64 *out)
{
    size_t N = c->N;
    u64 ql = c->q[L - 1];
    for (int p = 0; p < n_polys; p++) {
        const u64 *src = in + (size_t)p * L * N;
        u64 *last = (u64 *)malloc(N * 8);
        memcpy(last, src + (size_t)(L - 1) * N, N * 8);
        orc_ntt_inv(c, last, L - 1);
#pragma omp parallel for
        for (int r = 0; r < L - 1; r++) {
            u64 q = c->q[r], inv = orc_invmod(ql % q, q);
            u64 *t = (u64 *)malloc(N * 8);
            for (size_t k = 0; k < N; k++) t[k] = last[k] % q;
            orc_ntt_fwd(c, t, r);
            u64 *d = out + ((size_t)p * (L - 1) + r) * N;
            for (size_t k = 0; k < N; k++) d[k] = mulmod(submod(src[(size_t)r * N + k], t[k], q), inv, q);
            free(t);
        }
        free(last);
    }
}

/* cahel-main/src/evaluate.cu:2253-2300 mod_switch_drop_to_next: keep the first L-1 limbs of each polynomial */
void orc_drop_last(const orc_ctx *c, int L, int n_polys, const u64 *in, u64 *out)
{
    size_t N = c->N;
    for (int p = 0; p < n_polys; p++)
        memcpy(out + (size_t)p * (L - 1) * N, in + (size_t)p * L * N, (size_t)(L - 1) * N * 8);
}

/* cahel-main/src/evaluate.cu:2631-2686 apply_galois_inplace: permute first, then key switch
 * the permuted c1; ct [2][L][N] in place. */
void orc_rotate(const orc_ctx *c, int L, u64 *ct, int elt_idx, const u64 *glk)
{
    size_t S = (size_t)L * c->N;
    u64 *t0 = (u64 *)malloc(S * 8), *t1 = (u64 *)malloc(S * 8);
    orc_galois(c, elt_idx, L, ct, t0);
    orc_galois(c, elt_idx, L, ct + S, t1);
    memcpy(ct, t0, S * 8);
    memset(ct + S, 0, S * 8);
    orc_keyswitch(c, L, ct, t1, glk);
    free(t0); free(t1);
}

/* cahel-main/src/evaluate.cu:2412-2629 hoisting_inplace: modup(c1) once, then per step permute
 * every digit, inner product with that step's key, accumulate in QlP; two moddowns;
 * c0' = sum sigma(c0) + cx0, c1' = cx1.  glks[i] is the key of elt_idx[i]. */
void orc_hoisting(const orc_ctx *c, int L, u64 *ct, int n_steps, const int *elt_idx, const u64 *const *glks)
{
    size_t N = c->N, S = (size_t)L * N;
    int P = c->size_P, LP = L + P, beta = (L + P - 1) / P;
    u64 *dig = (u64 *)malloc((size_t)beta * LP * N * 8);
    u64 *pdig = (u64 *)malloc((size_t)beta * LP * N * 8);
    u64 *acc = (u64 *)calloc((size_t)2 * LP * N, 8);
    u64 *tmp = (u64 *)malloc((size_t)2 * LP * N * 8);
    u64 *acc0 = (u64 *)calloc(S, 8), *t0 = (u64 *)malloc(S * 8);
    orc_modup(c, L, ct + S, dig);
    for (int s = 0; s < n_steps; s++) {
        orc_galois(c, elt_idx[s], L, ct, t0);
        orc_poly_op(c, 0, L, 1, acc0, t0, acc0);
        /* limbs of a QlP buffer: galois is modulus independent */
        orc_galois(c, elt_idx[s], beta * LP, dig, pdig);
        orc_inner_product(c, L, pdig, glks[s], tmp);
        for (int i = 0; i < 2; i++)
            for (int r = 0; r < LP; r++) {
                u64 q = c->q[tix(c, L, r)];
                u64 *a = acc + ((size_t)i * LP + r) * N, *b = tmp + ((size_t)i * LP + r) * N;
                for (size_t k = 0; k < N; k++) a[k] = addmod(a[k], b[k], q);
            }
    }
    orc_moddown(c, L, acc, t0);
    orc_poly_op(c, 0, L, 1, acc0, t0, ct);
    orc_moddown(c, L, acc + (size_t)LP * N, ct + S);
    free(dig); free(pdig); free(acc); free(tmp); free(acc0); free(t0);
}

/* ---------------------------------------------------------------- PRNG + samplers (cahel-main/src/prng.cu) */

static inline uint32_t rotl(uint32_t u, int s) { return (u << s) | (u >> (32 - s)); }
static inline uint32_t ld32(const uint8_t *p) { return (uint32_t)p[0] | (uint32_t)p[1] << 8 | (uint32_t)p[2] << 16 | (uint32_t)p[3] << 24; }

#define QR(a, b, cc, d)            \
    x[b] ^= rotl(x[a] + x[d], 7);  \
    x[cc] ^= rotl(x[b] + x[a], 9); \
    x[d] ^= rotl(x[cc] + x[b], 13); \
    x[a] ^= rotl(x[d] + x[cc], 18);

/* cahel-main/src/prng.cu:16-138: words 0..7 = seed bytes 0..31, words 8,9 = nonce,
 * words 10..15 = seed bytes 32..55; ten Salsa20 double rounds; feed-forward add. */
void orc_prng_block(const uint8_t *seed, u64 nonce, uint32_t out[16])
{
    uint32_t x[16], j[16];
    for (int i = 0; i < 8; i++) j[i] = ld32(seed + 4 * i);
    j[8] = (uint32_t)nonce;
    j[9] = (uint32_t)(nonce >> 32);
    for (int i = 0; i < 6; i++) j[10 + i] = ld32(seed + 32 + 4 * i);
    memcpy(x, j, sizeof(x));
    for (int r = 0; r < 10; r++) {
        QR(0, 4, 8, 12) QR(5, 9, 13, 1) QR(10, 14, 2, 6) QR(15, 3, 7, 11)
        QR(0, 1, 2, 3) QR(5, 6, 7, 4) QR(10, 11, 8, 9) QR(15, 12, 13, 14)
    }
    for (int i = 0; i < 16; i++) out[i] = x[i] + j[i];
}

/* kind 0: ternary (prng.cu:143-165), kind 1: centred binomial error (prng.cu:219-242).
 * The nonce is the coefficient index, so every limb carries the same small value.
 * rows: size_l data limbs then size_p special limbs. */
void orc_sample_small(const orc_ctx *c, int kind, const uint8_t *seed, int size_l, int size_p, u64 *out)
{
    size_t N = c->N;
    int rows = size_l + size_p;
#pragma omp parallel for
    for (size_t k = 0; k < N; k++) {
        uint32_t b[16];
        orc_prng_block(seed, k, b);
        int v;
        if (kind == 0) {
            v = (int)((b[0] & 0xFF) % 3) - 1;
        } else {
            uint32_t w0 = b[0], w1 = b[1];
            v = __builtin_popcount(w0 & 0xFF) + __builtin_popcount((w0 >> 8) & 0xFF) + __builtin_popcount((w0 >> 16) & 0x1F)
                - __builtin_popcount((w0 >> 24) & 0xFF) - __builtin_popcount(w1 & 0xFF) - __builtin_popcount((w1 >> 8) & 0x1F);
        }
        for (int r = 0; r < rows; r++) {
            u64 q = c->q[tix(c, size_l, r)];
            out[(size_t)r * N + k] = v < 0 ? q - (u64)(-v) : (u64)v;
        }
    }
}

/* cahel-main/src/prng.cu:176-208 sample_uniform_poly: block t serves coefficients 8t..8t+7 of
 * the flat [rows][N] array; a word above the largest multiple of q is rejected and the
 * whole block is redrawn with nonce t + tries*N*rows (already accepted words stay). */
void orc_sample_uniform(const orc_ctx *c, const uint8_t *seed, int size_l, int size_p, u64 *out)
{
    size_t N = c->N;
    int rows = size_l + size_p;
    size_t blocks = (N >> 3) * rows;
#pragma omp parallel for
    for (size_t t = 0; t < blocks; t++) {
        int r = (int)(t / (N >> 3));
        u64 q = c->q[tix(c, size_l, r)];
        u64 max_multiple = UINT64_MAX - (UINT64_MAX % q) - 1;
        uint32_t b[16];
        orc_prng_block(seed, t, b);
        u64 tries = 1;
        for (int i = 0; i < 8; i++) {
            u64 v = (u64)b[2 * i] | (u64)b[2 * i + 1] << 32;
            while (v > max_multiple) {
                orc_prng_block(seed, t + tries * N * rows, b);
                tries++;
                v = (u64)b[2 * i] | (u64)b[2 * i + 1] << 32;
            }
            out[t * 8 + i] = v % q;
        }
    }
}

/* ---------------------------------------------------------------- keys, encryption, decryption (cahel-main/src/secretkey.cu) */

/* :254-283 gen_secretkey: sk = NTT(ternary) over all QP limbs */
void orc_gen_sk(const orc_ctx *c, const uint8_t *seed, u64 *sk)
{
    orc_sample_small(c, 0, seed, c->size_Q, c->size_P, sk);
    orc_ntt_rows(c, sk, 1, c->size_Q, c->size_P, 0);
}

/* :451-515 encrypt_zero_symmetric at the key level: (b, a) = (-(a s + e), a), e from seed_e,
 * a from seed_a sampled directly in NTT form.  pk [2][QP][N]. */
void orc_gen_pk(const orc_ctx *c, const u64 *sk, const uint8_t *seed_e, const uint8_t *seed_a, u64 *pk)
{
    size_t N = c->N;
    int QP = c->size_QP;
    u64 *e = (u64 *)malloc((size_t)QP * N * 8);
    orc_sample_small(c, 1, seed_e, c->size_Q, c->size_P, e);
    orc_ntt_rows(c, e, 1, c->size_Q, c->size_P, 0);
    u64 *a = pk + (size_t)QP * N;
    orc_sample_uniform(c, seed_a, c->size_Q, c->size_P, a);
    for (int r = 0; r < QP; r++) {
        u64 q = c->q[r];
        for (size_t k = 0; k < N; k++) {
            size_t i = (size_t)r * N + k;
            u64 v = addmod(mulmod(a[i], sk[i], q), e[i], q);
            pk[i] = v ? q - v : 0;
        }
    }
    free(e);
}

/* :328-372 generate_one_kswitch_key + polymath.cu:320-337: dnum fresh key pairs, then
 * evk_j.b[limb] += (P mod q_limb) * skp[limb] for the limbs of digit j.
 * seeds: [dnum][2][64] (error seed, uniform seed per pair).  out [dnum][2][QP][N]. */
void orc_gen_ksk(const orc_ctx *c, const u64 *sk, const u64 *skp, const uint8_t *seeds, u64 *out)
{
    size_t N = c->N;
    int QP = c->size_QP, P = c->size_P, alpha = P, dnum = c->size_Q / P;
    for (int j = 0; j < dnum; j++) {
        u64 *key = out + (size_t)j * 2 * QP * N;
        orc_gen_pk(c, sk, seeds + (size_t)j * 128, seeds + (size_t)j * 128 + 64, key);
        for (int r = j * alpha; r < (j + 1) * alpha; r++) {
            u64 q = c->q[r], pm = 1;
            for (int i = 0; i < P; i++) pm = mulmod(pm, c->q[c->size_Q + i] % q, q);
            for (size_t k = 0; k < N; k++) {
                size_t i = (size_t)r * N + k;
                key[i] = addmod(key[i], mulmod(pm, skp[i], q), q);
            }
        }
    }
}

/* :47-170 asymmetric encryption of zero at the key level followed by moddown to the
 * first data level: u ternary (seed_u); e0 == e1 from the single seed_e (:78-98);
 * c_i = pk_i u + e_i over QP; then divide by P.  ct [2][Q][N]. */
void orc_encrypt_zero_asym(const orc_ctx *c, const u64 *pk, const uint8_t *seed_u, const uint8_t *seed_e, u64 *ct)
{
    size_t N = c->N;
    int QP = c->size_QP, Q = c->size_Q, P = c->size_P;
    u64 *u = (u64 *)malloc((size_t)QP * N * 8), *e = (u64 *)malloc((size_t)QP * N * 8);
    u64 *cx = (u64 *)malloc((size_t)QP * N * 8);
    orc_sample_small(c, 0, seed_u, Q, P, u);
    orc_ntt_rows(c, u, 1, Q, P, 0);
    orc_sample_small(c, 1, seed_e, Q, P, e);
    orc_ntt_rows(c, e, 1, Q, P, 0);
    for (int p = 0; p < 2; p++) {
        for (int r = 0; r < QP; r++) {
            u64 q = c->q[r];
            for (size_t k = 0; k < N; k++) {
                size_t i = (size_t)r * N + k;
                cx[i] = addmod(mulmod(u[i], pk[(size_t)p * QP * N + i], q), e[i], q);
            }
        }
        orc_moddown(c, Q, cx, ct + (size_t)p * Q * N);
    }
    free(u); free(e); free(cx);
}

/* :594-654 ckks_decrypt without the noise-flooding term: pt = c0 + c1 s + c2 s^2.  sk [QP][N]. */
void orc_decrypt(const orc_ctx *c, int L, int n_polys, const u64 *ct, const u64 *sk, u64 *pt)
{
    size_t N = c->N;
#pragma omp parallel for
    for (int r = 0; r < L; r++) {
        u64 q = c->q[r];
        for (size_t k = 0; k < N; k++) {
            size_t i = (size_t)r * N + k;
            u64 s = sk[i], sp = s, acc = ct[i];
            for (int p = 1; p < n_polys; p++) {
                acc = addmod(acc, mulmod(ct[(size_t)p * L * N + i], sp, q), q);
                sp = mulmod(sp, s, q);
            }
            pt[i] = acc;
        }
    }
}

/* ---------------------------------------------------------------- encoder (cahel-main/src/ckks.cu, fft.cu, croots.cu, rns_base.cu) */

typedef struct { double x, y; } cplx;

/* cuCmul with each part contracted into one rounded product and one fused multiply-add, which is how
 * the device compiler emits cahel-main/src/fft.cu:12-41 under its default -fmad=true.  Which product of
 * the imaginary part is the rounded one differs between the reference's two inverse-FFT kernels: the
 * multi-stage kernel that runs the first eleven stages (fft.cu:194-268, SWITCH_POINT = 2048) rounds
 * a.x * b.y (first_kernel != 0), the per-stage kernel (fft.cu:279-344) rounds a.y * b.x.  Pinned by the
 * reference-made plaintexts at scale 2^50 (fixtures n4096_s50, n8192_s50, n65536_a8). */
#define ORC_IFFT_FIRST_KERNEL_STAGES 11
static inline cplx cmul2(cplx a, cplx b, int first_kernel)
{
    cplx r;
    r.x = fma(a.x, b.x, -(a.y * b.y));
    r.y = first_kernel ? fma(a.y, b.x, a.x * b.y) : fma(a.x, b.y, a.y * b.x);
    return r;
}
static inline cplx cmul(cplx a, cplx b) { return cmul2(a, b, 0); }

/* cahel-main/src/croots.cu:14-66: one eighth of the M-th roots from polar(), the rest by symmetry */
static cplx croot(size_t index, size_t M)
{
    static const double PI = 3.1415926535897932384626433832795028842;
    index &= M - 1;
    cplx r;
    if (index <= M / 8) {
        double th = 2 * PI * (double)index / (double)M;
        r.x = cos(th); r.y = sin(th);
        return r;
    } else if (index <= M / 4) {
        cplx t = croot(M / 4 - index, M);
        r.x = t.y; r.y = t.x;
        return r;
    } else if (index <= M / 2) {
        cplx t = croot(M / 2 - index, M);
        r.x = 0.0 - t.x; r.y = 0.0 - (-t.y);
        return r;
    } else if (index <= 3 * M / 4) {
        cplx t = croot(index - M / 2, M);
        r.x = 0.0 - t.x; r.y = 0.0 - t.y;
        return r;
    } else {
        cplx t = croot(M - index, M);
        r.x = t.x; r.y = -t.y;
        return r;
    }
}

void orc_croot(size_t index, size_t M, double *out) { cplx r = croot(index, M); out[0] = r.x; out[1] = r.y; }

/* twiddle index of butterfly group k at a stage with 2^logPairs pairs (fft.cu:216-222) */
static inline uint32_t psi_index(const uint32_t *group, uint32_t k, int logPairs, int logn, int logRatio, uint32_t M)
{
    uint32_t rev = logn > 1 ? bitrev(k << logPairs, logn - 1) : 0;
    uint32_t p = group[rev];
    p <<= (logPairs + logRatio);
    return p & (M - 1);
}

static uint32_t *rot_group(size_t N)
{
    size_t half = N >> 2;
    if (half == 0) half = 1;
    uint32_t *g = (uint32_t *)malloc(half * 4), pos = 1, M = (uint32_t)(2 * N);
    for (size_t i = 0; i < half; i++) { g[i] = pos; pos = (pos * 5) & (M - 1); }
    return g;
}

/* cahel-main/src/ckks.cu:104-209 encode_internal.  values: n_values complex numbers (re,im
 * pairs), sparse_slots a power of two >= n_values, output plaintext [L][N] in NTT form.
 * Special inverse FFT per fft.cu:194-344 (stride 1 first, scale/n folded into the last stage),
 * rounding and residues per rns_base.cu:121-156. */
void orc_encode(const orc_ctx *c, int L, const double *values, size_t n_values, size_t sparse_slots, double scale, u64 *pt)
{
    size_t N = c->N, n = sparse_slots;
    uint32_t M = (uint32_t)(2 * N);
    int logn = 0;
    while (((size_t)1 << logn) < n) logn++;
    int logRatio = (c->logN + 1) - logn - 2;
    cplx *a = (cplx *)calloc(n, sizeof(cplx));
    for (size_t i = 0; i < n; i++) {
        uint32_t d = bitrev((uint32_t)i, logn);
        if (i < n_values) { a[d].x = values[2 * i]; a[d].y = values[2 * i + 1]; }
    }
    uint32_t *group = rot_group(N);
    double fix = scale / (double)n;
    for (int iter = logn - 1; iter >= 0; iter--) {
        int logPairs = logn - iter - 1;
        uint32_t pairs = 1u << logPairs;
        for (uint32_t tid = 0; tid < n / 2; tid++) {
            uint32_t k = tid >> logPairs, j = tid & (pairs - 1), g = 2 * k * pairs + j;
            uint32_t pi = psi_index(group, k, logPairs, logn, logRatio, M);
            cplx w = croot(M - pi, M);
            cplx x0 = a[g], x1 = a[g + pairs], s0, s1;
            s0.x = x0.x + x1.x; s0.y = x0.y + x1.y;
            s1.x = x0.x - x1.x; s1.y = x0.y - x1.y;
            s1 = cmul2(s1, w, logPairs < ORC_IFFT_FIRST_KERNEL_STAGES);
            if (iter == 0 && fix != 0.0) { s0.x *= fix; s0.y *= fix; s1.x *= fix; s1.y *= fix; }
            a[g] = s0; a[g + pairs] = s1;
        }
    }
    size_t ratio = (N / 2) / n;
    memset(pt, 0, (size_t)L * N * 8);
    for (int r = 0; r < L; r++) {
        u64 q = c->q[r];
        for (size_t id = 0; id < 2 * n; id++) {
            double v = id < n ? round(a[id].x) : round(a[id - n].y);
            int negv = signbit(v);
            double av = fabs(v);
            u64 red;
            if (av < 18446744073709551616.0) red = (u64)av % q;
            else {
                u64 lo = (u64)fmod(av, 18446744073709551616.0), hi = (u64)(av / 18446744073709551616.0);
                red = (u64)((((u128)hi << 64) | lo) % q);
            }
            if (negv) red = q - red; /* the reference stores q for a negative zero; canonicalised below */
            pt[(size_t)r * N + id * ratio] = red;
        }
    }
    /* a rounded -0.0 yields the non-canonical residue q in the reference too
     * (rns_base.cu:147-149); the NTT reduces it, so the transformed plaintext agrees. */
    for (int r = 0; r < L; r++)
        for (size_t k = 0; k < N; k++)
            if (pt[(size_t)r * N + k] == c->q[r]) pt[(size_t)r * N + k] = 0;
    orc_ntt_rows(c, pt, 1, L, 0, 0);
    free(a); free(group);
}

/* cahel-main/src/ckks.cu:292-465 decode_internal: INTT, centred CRT composition
 * (rns_base.cu:325-459), times 1/scale, special forward FFT (fft.cu:54-182), bit reversal.
 * The composition is carried out exactly with Garner mixed radix and converted to a long
 * double, which is at least as accurate as the reference's per-word double accumulation. */
void orc_decode(const orc_ctx *c, int L, const u64 *pt, double scale, size_t sparse_slots, double *out)
{
    size_t N = c->N, n = sparse_slots;
    uint32_t M = (uint32_t)(2 * N);
    int logn = 0;
    while (((size_t)1 << logn) < n) logn++;
    int logRatio = (c->logN + 1) - logn - 2;
    u64 *p = (u64 *)malloc((size_t)L * N * 8);
    memcpy(p, pt, (size_t)L * N * 8);
    orc_ntt_rows(c, p, 1, L, 0, 1);
    size_t ratio = (N / 2) / n;
    cplx *a = (cplx *)calloc(n, sizeof(cplx));
    /* Garner mixed radix x = v0 + v1 q0 + v2 q0 q1 + ..., evaluated exactly in multi-word
     * integers, centred against Q/2, and only then converted to floating point. */
    int W = L + 1;
    u64 Qw[ORC_MAX_MOD + 1], Qh[ORC_MAX_MOD + 1], radw[ORC_MAX_MOD][ORC_MAX_MOD + 1];
    memset(Qw, 0, sizeof(Qw));
    Qw[0] = 1;
    for (int r = 0; r < L; r++) {
        memcpy(radw[r], Qw, sizeof(u64) * W);
        u64 carry = 0;
        for (int i = 0; i < W; i++) { u128 t = (u128)Qw[i] * c->q[r] + carry; Qw[i] = (u64)t; carry = (u64)(t >> 64); }
    }
    for (int i = 0; i < W; i++) Qh[i] = (Qw[i] >> 1) | (i + 1 < W ? Qw[i + 1] << 63 : 0);
    u64 ginv[ORC_MAX_MOD];
    for (int r = 0; r < L; r++) {
        u64 q = c->q[r], radix = 1;
        for (int s = 0; s < r; s++) radix = mulmod(radix, c->q[s] % q, q);
        ginv[r] = orc_invmod(radix, q);
    }
    for (size_t id = 0; id < 2 * n; id++) {
        u64 v[ORC_MAX_MOD];
        for (int r = 0; r < L; r++) {
            u64 q = c->q[r];
            u64 t = p[(size_t)r * N + id * ratio] % q;
            u64 acc = 0, radix = 1;
            for (int s = 0; s < r; s++) {
                acc = addmod(acc, mulmod(v[s] % q, radix, q), q);
                radix = mulmod(radix, c->q[s] % q, q);
            }
            v[r] = mulmod(submod(t, acc, q), ginv[r], q);
        }
        u64 x[ORC_MAX_MOD + 1];
        memset(x, 0, sizeof(u64) * W);
        for (int r = 0; r < L; r++) {
            u64 carry = 0;
            for (int i = 0; i < W; i++) {
                u128 t = (u128)radw[r][i] * v[r] + x[i] + carry;
                x[i] = (u64)t; carry = (u64)(t >> 64);
            }
        }
        int ge = 1; /* x >= ceil(Q/2)?  (upper_half_threshold = (Q+1)/2, cahel-main/src/context.cu:305-312) */
        for (int i = W - 1; i >= 0; i--) {
            if (x[i] != Qh[i]) { ge = x[i] > Qh[i]; break; }
        }
        int neg = 0;
        if (ge) { /* compare is against floor(Q/2); Q odd so x > floor(Q/2) <=> x >= (Q+1)/2 */
            int eq = 1;
            for (int i = 0; i < W; i++) eq &= (x[i] == Qh[i]);
            if (!eq) {
                neg = 1;
                u64 borrow = 0;
                for (int i = 0; i < W; i++) {
                    u128 t = (u128)Qw[i] - x[i] - borrow;
                    x[i] = (u64)t; borrow = (u64)(t >> 64) & 1;
                }
            }
        }
        long double val = 0.0L, rad = 1.0L;
        for (int i = 0; i < W; i++) { val += (long double)x[i] * rad; rad *= 18446744073709551616.0L; }
        if (neg) val = -val;
        double d = (double)(val / (long double)scale);
        if (id < n) a[id].x = d; else a[id - n].y = d;
    }
    uint32_t *group = rot_group(N);
    for (int iter = 0; iter < logn; iter++) {
        int logPairs = logn - iter - 1;
        uint32_t pairs = 1u << logPairs;
        for (uint32_t tid = 0; tid < n / 2; tid++) {
            uint32_t k = tid >> logPairs, j = tid & (pairs - 1), g = 2 * k * pairs + j;
            uint32_t pi = psi_index(group, k, logPairs, logn, logRatio, M);
            cplx w = croot(pi, M);
            cplx x0 = a[g], x1 = cmul(a[g + pairs], w);
            a[g].x = x0.x + x1.x; a[g].y = x0.y + x1.y;
            a[g + pairs].x = x0.x - x1.x; a[g + pairs].y = x0.y - x1.y;
        }
    }
    for (size_t i = 0; i < n; i++) {
        uint32_t d = bitrev((uint32_t)i, logn);
        out[2 * d] = a[i].x; out[2 * d + 1] = a[i].y;
    }
    free(p); free(a); free(group);
}

/* coefficient-domain output of the encoder's inverse FFT (before rounding), for
 * tests that want to look at near-half rounding cases */
size_t orc_N(const orc_ctx *c) { return c->N; }

/* ---------------------------------------------------------------- batched forms for the timed CPU baseline
 * The same functions over a batch of independent items, one OpenMP thread per item; the inner loops of the
 * functions above then run serially (nested parallel regions are off by default).  This is how a CPU
 * implementation would use its cores on the Krum workload: parallel over ciphertexts and pairs, not over
 * the three or four limbs of one polynomial. */
#ifdef _OPENMP
#include <omp.h>
int orc_max_threads(void) { return omp_get_max_threads(); }
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
#else
int orc_max_threads(void) { return 1; }
void orc_set_threads(int n) { (void)n; }
#endif

/* values [batch][slots] doubles, seeds [batch][2][64] (ternary, error) -> ct [batch][2][size_Q][N] */
void orc_encode_encrypt_batch(const orc_ctx *c, const u64 *pk, const double *values, size_t slots, double scale, const uint8_t *seeds,
                              int batch, u64 *ct)
{
    size_t N = c->N;
    int Q = c->size_Q;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < batch; b++) {
        u64 *pt = (u64 *)malloc((size_t)Q * N * 8);
        double *v = (double *)malloc(slots * 2 * sizeof(double));
        for (size_t i = 0; i < slots; i++) { v[2 * i] = values[(size_t)b * slots + i]; v[2 * i + 1] = 0.0; }
        orc_encode(c, Q, v, slots, slots, scale, pt);
        u64 *out = ct + (size_t)b * 2 * Q * N;
        orc_encrypt_zero_asym(c, pk, seeds + (size_t)b * 128, seeds + (size_t)b * 128 + 64, out);
        orc_poly_op(c, 0, Q, 1, out, pt, out);
        free(pt); free(v);
    }
}

/* acc[b] += (y[b] - x[b])^2 for a batch of ciphertext pairs: x, y [batch][2][L][N], acc [batch][3][L][N] */
void orc_pair_chunk_batch(const orc_ctx *c, int L, const u64 *x, const u64 *y, u64 *acc, int batch)
{
    size_t N = c->N;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < batch; b++) {
        u64 *d = (u64 *)malloc((size_t)2 * L * N * 8), *sq = (u64 *)malloc((size_t)3 * L * N * 8);
        orc_poly_op(c, 1, L, 2, y + (size_t)b * 2 * L * N, x + (size_t)b * 2 * L * N, d);
        orc_tensor(c, L, d, d, sq);
        orc_poly_op(c, 0, L, 3, acc + (size_t)b * 3 * L * N, sq, acc + (size_t)b * 3 * L * N);
        free(d); free(sq);
    }
}

/* acc[b] += x[b] (x) mask for a batch of ciphertexts: x [batch][2][L][N], mask [2][L][N], acc [batch][3][L][N]
 * (the per-client step of the mask multiplication, lancelot-main-GPU/utils/byzantine_fl.py:401-409) */
void orc_mask_chunk_batch(const orc_ctx *c, int L, const u64 *x, const u64 *mask, u64 *acc, int batch)
{
    size_t N = c->N;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < batch; b++) {
        u64 *t = (u64 *)malloc((size_t)3 * L * N * 8);
        orc_tensor(c, L, x + (size_t)b * 2 * L * N, mask, t);
        orc_poly_op(c, 0, L, 3, acc + (size_t)b * 3 * L * N, t, acc + (size_t)b * 3 * L * N);
        free(t);
    }
}

/* relinearize + rescale of a batch: ct3 [batch][3][L][N] (clobbered) -> out [batch][2][L-1][N] */
void orc_relin_rescale_batch(const orc_ctx *c, int L, u64 *ct3, const u64 *rlk, u64 *out, int batch)
{
    size_t N = c->N;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < batch; b++) {
        u64 *ct = ct3 + (size_t)b * 3 * L * N;
        orc_relinearize(c, L, ct, rlk);
        orc_rescale(c, L, 2, ct, out + (size_t)b * 2 * (L - 1) * N);
    }
}

/* multiply + relinearize + rescale of a batch: x, y [batch][2][L][N] -> out [batch][2][L-1][N] */
void orc_hmult_batch(const orc_ctx *c, int L, const u64 *x, const u64 *y, const u64 *rlk, u64 *out, int batch)
{
    size_t N = c->N;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < batch; b++) {
        u64 *ct = (u64 *)malloc((size_t)3 * L * N * 8);
        orc_tensor(c, L, x + (size_t)b * 2 * L * N, y + (size_t)b * 2 * L * N, ct);
        orc_relinearize(c, L, ct, rlk);
        orc_rescale(c, L, 2, ct, out + (size_t)b * 2 * (L - 1) * N);
        free(ct);
    }
}

/* ct[b] <- rot(ct[b]) for a batch [batch][2][L][N] with one Galois key */
void orc_rotate_batch(const orc_ctx *c, int L, u64 *ct, int elt_idx, const u64 *glk, int batch)
{
    size_t N = c->N;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < batch; b++) orc_rotate(c, L, ct + (size_t)b * 2 * L * N, elt_idx, glk);
}

/* forward then inverse transform of a batch of polynomials [batch][size_l][N], one thread per limb */
void orc_ntt_roundtrip_batch(const orc_ctx *c, u64 *data, int batch, int size_l)
{
    orc_ntt_rows(c, data, batch, size_l, 0, 0);
    orc_ntt_rows(c, data, batch, size_l, 0, 1);
}
