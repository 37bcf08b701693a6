// Keyed pseudo-random sampling, key generation arithmetic and public-key encryption.
//
// The block function and the three samplers must reproduce the reference bit for bit
// (cahel-main/src/prng.cu:16-242): sixteen little-endian words, words 0..7 and 10..15 from
// the 64-byte seed, words 8,9 the nonce, ten Salsa20 double rounds, feed-forward add.
// The reference recomputes the same block once per limb for the small samplers; here one
// thread computes a coefficient's block once and writes every limb.
#include "context.h"

namespace lb {

constexpr int kSampThreads = 256;

struct Seed {
    uint32_t w[16];
};

LB_D uint32_t rotl32(uint32_t v, int s) { return __funnelshift_l(v, v, s); }

#define LB_QR(a, b, c, d)          \
    x[b] ^= rotl32(x[a] + x[d], 7);  \
    x[c] ^= rotl32(x[b] + x[a], 9);  \
    x[d] ^= rotl32(x[c] + x[b], 13); \
    x[a] ^= rotl32(x[d] + x[c], 18);

LB_D void prng_block(const uint32_t *__restrict__ seed, const u64 nonce, uint32_t (&x)[16])
{
    uint32_t j[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) j[i] = seed[i];
    j[8] = (uint32_t)nonce;
    j[9] = (uint32_t)(nonce >> 32);
#pragma unroll
    for (int i = 0; i < 6; ++i) j[10 + i] = seed[8 + i];
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = j[i];
    // unrolled in full: the small samplers use one or two words of the block, and only then can the compiler drop
    // the quarter rounds of the last double round that do not reach them
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        LB_QR(0, 4, 8, 12) LB_QR(5, 9, 13, 1) LB_QR(10, 14, 2, 6) LB_QR(15, 3, 7, 11)
        LB_QR(0, 1, 2, 3) LB_QR(5, 6, 7, 4) LB_QR(10, 11, 8, 9) LB_QR(15, 12, 13, 14)
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] += j[i];
}

// kind 0: ternary in {-1,0,1} from byte 0 mod 3 (prng.cu:143-165)
// kind 1: centred binomial from 21 + 21 bits of bytes 0..5 (prng.cu:219-242)
LB_D int small_value(const int kind, const uint32_t w0, const uint32_t w1)
{
    if (kind == 0) return (int)((w0 & 0xFFu) % 3u) - 1;
    return __popc(w0 & 0x1FFFFFu) - (__popc(w0 >> 24) + __popc(w1 & 0x1FFFu));
}

// out[b][rows][N]; seeds[b][16] words; every row carries the same small polynomial
__global__ void __launch_bounds__(kSampThreads) sample_small_kernel(u64 *__restrict__ out, const uint32_t *__restrict__ seeds,
                                                                    const int seed_stride, const ModConst *__restrict__ mc, const int kind,
                                                                    const int logN, const int size_l, const int size_p,
                                                                    const int size_Q, const long total)
{
    const int rows = size_l + size_p;
    const long n_mask = (1L << logN) - 1;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long b = i >> logN, k = i & n_mask;
        uint32_t x[16];
        prng_block(seeds + seed_stride * b, (u64)k, x);
        const int v = small_value(kind, x[0], x[1]);
        u64 *o = out + ((b * rows) << logN) + k;
        for (int r = 0; r < rows; ++r) {
            const u64 q = mc[r < size_l ? r : size_Q + (r - size_l)].q;
            o[(long)r << logN] = v < 0 ? q - (u64)(-v) : (u64)v;
        }
    }
}

// prng.cu:176-208: block t covers coefficients 8t..8t+7 of the flat [rows][N] array; a word
// above the largest multiple of q redraws the whole block with nonce t + tries * N * rows.
__global__ void __launch_bounds__(kSampThreads) sample_uniform_kernel(u64 *__restrict__ out, const uint32_t *__restrict__ seeds,
                                                                      const int seed_stride, const ModConst *__restrict__ mc, const int logN,
                                                                      const int size_l, const int size_p, const int size_Q,
                                                                      const long total, const long out_stride)
{
    const int rows = size_l + size_p;
    const long blocks_per_poly = ((long)rows << logN) >> 3;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long b = i / blocks_per_poly, t = i - b * blocks_per_poly;
        const int r = (int)(t >> (logN - 3));
        const ModConst m = mc[r < size_l ? r : size_Q + (r - size_l)];
        const u64 max_multiple = ~0ull - barrett64(~0ull, m.q, m.r1) - 1;
        uint32_t x[16];
        prng_block(seeds + seed_stride * b, (u64)t, x);
        u64 tries = 1;
        u64 *o = out + b * out_stride + (t << 3);
#pragma unroll 1
        for (int w = 0; w < 8; ++w) {
            u64 v = (u64)x[2 * w] | (u64)x[2 * w + 1] << 32;
            while (v > max_multiple) {
                prng_block(seeds + seed_stride * b, (u64)t + tries * (u64)((long)rows << logN), x);
                ++tries;
                v = (u64)x[2 * w] | (u64)x[2 * w + 1] << 32;
            }
            o[w] = barrett64(v, m.q, m.r1);
        }
    }
}

// the same small polynomial as one signed byte per coefficient (|value| <= 21)
__global__ void __launch_bounds__(kSampThreads) sample_small_i8_kernel(signed char *__restrict__ out, const uint32_t *__restrict__ seeds,
                                                                       const int seed_stride, const int kind, const int logN,
                                                                       const long total)
{
    const long n_mask = (1L << logN) - 1;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long b = i >> logN, k = i & n_mask;
        uint32_t x[16];
        prng_block(seeds + seed_stride * b, (u64)k, x);
        out[i] = (signed char)small_value(kind, x[0], x[1]);
    }
}

static inline int grid_for(const Context *ctx, long items)
{
    long need = (items + kSampThreads - 1) / kSampThreads;
    const long cap = (long)ctx->sm_count * 16;
    return (int)(need < 1 ? 1 : (need < cap ? need : cap));
}

int sample_small(Context *ctx, int kind, const uint32_t *d_seeds, int seed_stride, int batch, int size_l, int size_p, u64 *out, cudaStream_t stream)
{
    const long total = (long)batch << ctx->hp.logN;
    if (total == 0) return LB_OK;
    count_launch("sample_small_kernel", stream, 8.0 * total * (size_l + size_p));
    sample_small_kernel<<<grid_for(ctx, total), kSampThreads, 0, stream>>>(out, d_seeds, seed_stride, ctx->d_mc, kind, ctx->hp.logN, size_l, size_p,
                                                                          ctx->hp.size_Q, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

int sample_uniform(Context *ctx, const uint32_t *d_seeds, int seed_stride, int batch, int size_l, int size_p, u64 *out, cudaStream_t stream,
                   long out_stride)
{
    const long total = ((long)batch * (size_l + size_p) << ctx->hp.logN) >> 3;
    if (total == 0) return LB_OK;
    if (out_stride <= 0) out_stride = (long)(size_l + size_p) << ctx->hp.logN; // polynomials back to back
    count_launch("sample_uniform_kernel", stream);
    sample_uniform_kernel<<<grid_for(ctx, total), kSampThreads, 0, stream>>>(out, d_seeds, seed_stride, ctx->d_mc, ctx->hp.logN, size_l, size_p,
                                                                            ctx->hp.size_Q, total, out_stride);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- key generation arithmetic (cahel-main/src/secretkey.cu:322-372,451-515) ---------------

// b = -(a s + e) over all QP limbs
__global__ void __launch_bounds__(kSampThreads) pk_combine_kernel(u64 *__restrict__ b, const u64 *__restrict__ a,
                                                                  const u64 *__restrict__ s, const u64 *__restrict__ e,
                                                                  const ModConst *__restrict__ mc, const int logN, const long total)
{
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const ModConst m = mc[(int)(i >> logN)];
        u128d acc = mul_wide(a[i], s[i]);
        acc.lo += e[i];
        acc.hi += acc.lo < e[i];
        const u64 v = barrett128(acc, m.q, m.r0, m.r1);
        b[i] = v ? m.q - v : 0;
    }
}

// evk_j.b[limb] += (P mod q_limb) * s'[limb] for the limbs of digit j (polymath.cu:320-337)
__global__ void __launch_bounds__(kSampThreads) ksk_add_kernel(u64 *__restrict__ key, const u64 *__restrict__ skp,
                                                               const u64 *__restrict__ pmod, const u64 *__restrict__ pmod_s,
                                                               const ModConst *__restrict__ mc, const int logN, const int alpha,
                                                               const long key_stride, const long total)
{
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int r = (int)(i >> logN);
        const int j = r / alpha;
        const u64 q = mc[r].q;
        u64 *dst = key + j * key_stride + i;
        *dst = add_mod(*dst, shoup_mul(skp[i], pmod[r], pmod_s[r], q), q);
    }
}

int gen_public_key(Context *ctx, const u64 *sk, const uint32_t *d_seed_e, const uint32_t *d_seed_a, u64 *pk, u64 *scratch,
                   cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const long poly = (long)hp.size_QP << hp.logN;
    int rc;
    if ((rc = sample_small(ctx, 1, d_seed_e, 16, 1, hp.size_Q, hp.size_P, scratch, stream))) return rc;
    NttJob j;
    j.src = scratch;
    j.dst = scratch;
    j.n_groups = 1;
    j.per_group = hp.size_QP;
    j.size_l = hp.size_Q;
    if ((rc = ntt_forward(ctx, j, stream))) return rc;
    if ((rc = sample_uniform(ctx, d_seed_a, 16, 1, hp.size_Q, hp.size_P, pk + poly, stream))) return rc;
    count_launch("pk_combine_kernel", stream);
    pk_combine_kernel<<<grid_for(ctx, poly), kSampThreads, 0, stream>>>(pk, pk + poly, sk, scratch, ctx->d_mc, hp.logN, poly);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

int gen_switch_key(Context *ctx, const u64 *sk, const u64 *skp, const uint32_t *d_seeds, u64 *out, u64 *scratch, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const int dnum = hp.size_Q / hp.size_P;
    const long poly = (long)hp.size_QP << hp.logN;
    for (int j = 0; j < dnum; ++j) {
        int rc = gen_public_key(ctx, sk, d_seeds + 32 * j, d_seeds + 32 * j + 16, out + 2 * poly * j, scratch, stream);
        if (rc) return rc;
    }
    const long total = (long)hp.size_Q << hp.logN;
    count_launch("ksk_add_kernel", stream);
    ksk_add_kernel<<<grid_for(ctx, total), kSampThreads, 0, stream>>>(out, skp, ctx->d_p_mod_q, ctx->d_p_mod_q_s, ctx->d_mc, hp.logN,
                                                                     hp.size_P, 2 * poly, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// The same two steps for a batch of key pairs / switch keys (grid y): pair t is (b, a) = (pairs + t * 2 poly, + poly),
// its error e + t * poly; switch key k is dnum consecutive pairs and takes the target skp + k * poly.
__global__ void __launch_bounds__(kSampThreads) pk_combine_batch_kernel(u64 *__restrict__ pairs, const u64 *__restrict__ s,
                                                                        const u64 *__restrict__ e, const ModConst *__restrict__ mc,
                                                                        const int logN, const long poly)
{
    u64 *b = pairs + (long)blockIdx.y * 2 * poly;
    const u64 *a = b + poly, *eb = e + (long)blockIdx.y * poly;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < poly; i += (long)gridDim.x * blockDim.x) {
        const ModConst m = mc[(int)(i >> logN)];
        u128d acc = mul_wide(a[i], s[i]);
        acc.lo += eb[i];
        acc.hi += acc.lo < eb[i];
        const u64 v = barrett128(acc, m.q, m.r0, m.r1);
        b[i] = v ? m.q - v : 0;
    }
}

__global__ void __launch_bounds__(kSampThreads) ksk_add_batch_kernel(u64 *__restrict__ keys, const u64 *__restrict__ skp,
                                                                     const u64 *__restrict__ pmod, const u64 *__restrict__ pmod_s,
                                                                     const ModConst *__restrict__ mc, const int logN, const int alpha,
                                                                     const long key_words, const long poly, const long total)
{
    u64 *key = keys + (long)blockIdx.y * key_words;
    const u64 *target = skp + (long)blockIdx.y * poly;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int r = (int)(i >> logN);
        const int j = r / alpha;
        const u64 q = mc[r].q;
        u64 *dst = key + j * 2 * poly + i;
        *dst = add_mod(*dst, shoup_mul(target[i], pmod[r], pmod_s[r], q), q);
    }
}

// n switch keys at once: the streams, and so the keys, are those of n calls of gen_switch_key with seeds
// d_seeds + k * 32 * dnum, but every step is one launch over all keys and digits instead of one per key and digit.
// targets: [n][QP][N]; out: [n][dnum][2][QP][N]; scratch: n * dnum polynomials.
int gen_switch_keys(Context *ctx, const u64 *sk, const u64 *targets, int n, const uint32_t *d_seeds, u64 *out, u64 *scratch,
                    cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const int dnum = hp.size_Q / hp.size_P;
    const long poly = (long)hp.size_QP << hp.logN;
    const int pairs = n * dnum;
    if (pairs == 0) return LB_OK;
    if (pairs > 65535) { set_error("too many switch keys in one call"); return LB_ERR_INVALID_ARG; }
    int rc;
    if ((rc = sample_small(ctx, 1, d_seeds, 32, pairs, hp.size_Q, hp.size_P, scratch, stream))) return rc;
    NttJob j;
    j.src = scratch;
    j.dst = scratch;
    j.n_groups = pairs;
    j.per_group = hp.size_QP;
    j.size_l = hp.size_Q;
    if ((rc = ntt_forward(ctx, j, stream))) return rc;
    if ((rc = sample_uniform(ctx, d_seeds + 16, 32, pairs, hp.size_Q, hp.size_P, out + poly, stream, 2 * poly))) return rc;
    long gx = (poly + kSampThreads - 1) / kSampThreads;
    const long cap = (long)ctx->sm_count * 16;
    if (gx > cap) gx = cap;
    count_launch("pk_combine_kernel", stream);
    pk_combine_batch_kernel<<<dim3((unsigned)gx, (unsigned)pairs), kSampThreads, 0, stream>>>(out, sk, scratch, ctx->d_mc, hp.logN, poly);
    LB_CUDA(cudaGetLastError());
    const long total = (long)hp.size_Q << hp.logN;
    count_launch("ksk_add_kernel", stream);
    ksk_add_batch_kernel<<<dim3((unsigned)grid_for(ctx, total), (unsigned)n), kSampThreads, 0, stream>>>(
        out, targets, ctx->d_p_mod_q, ctx->d_p_mod_q_s, ctx->d_mc, hp.logN, hp.size_P, (long)dnum * 2 * poly, poly, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- public-key encryption (cahel-main/src/secretkey.cu:47-170) -----------------------------

// cx[b][p][QP][N] = pk[p] * u[b] + e[b]   (u and e already in NTT form; e0 == e1)
__global__ void __launch_bounds__(kSampThreads) encrypt_combine_kernel(u64 *__restrict__ cx, const u64 *__restrict__ pk,
                                                                       const u64 *__restrict__ u, const u64 *__restrict__ e,
                                                                       const ModConst *__restrict__ mc, const int logN,
                                                                       const long poly, const long total)
{
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long b = i / poly, k = i - b * poly;
        const ModConst m = mc[(int)(k >> logN)];
        const u64 uu = u[i], ee = e[i];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            u128d acc = mul_wide(uu, pk[p * poly + k]);
            acc.lo += ee;
            acc.hi += acc.lo < ee;
            cx[(2 * b + p) * poly + k] = barrett128(acc, m.q, m.r0, m.r1);
        }
    }
}

size_t encrypt_workspace_bytes(const Context *ctx, int batch)
{
    const HostParams &hp = ctx->hp;
    // u,e [2][batch][QP][N] + cx [batch][2][QP][N] + special-limb coefficients [2 batch][P][N] + seeds
    return ((size_t)batch * (4 * hp.size_QP + 2 * hp.size_P) << hp.logN) * 8 + (size_t)batch * 128 + 256;
}

// ct[b][2][Q][N] = moddown(pk u + e) (+ pt[b] on the first polynomial)
// pt_is_coeff: the plaintext rows are in coefficient form and are folded into the mod-down
// transform ((cx - NTT(delta - P m)) P^-1 equals (cx - NTT(delta)) P^-1 + NTT(m) word for word)
int encrypt_asymmetric(Context *ctx, const u64 *pk, const u64 *pt, int pt_is_coeff, const uint8_t *host_seeds, int batch, u64 *ct,
                       cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    if (hp.size_P < 1) { set_error("public-key encryption needs a special prime"); return LB_ERR_INVALID_ARG; }
    const int QP = hp.size_QP, Q = hp.size_Q, P = hp.size_P;
    const long poly = (long)QP << hp.logN;
    int rc = ctx->ensure_workspace(encrypt_workspace_bytes(ctx, batch));
    if (rc) return rc;
    u64 *u = reinterpret_cast<u64 *>(ctx->ws);
    u64 *e = u + batch * poly;
    u64 *cx = e + batch * poly;
    u64 *pc = cx + 2 * batch * poly;
    uint32_t *seeds = reinterpret_cast<uint32_t *>(pc + (((size_t)2 * batch * P) << hp.logN));
    // seeds arrive as [batch][2][64 bytes]: (ternary seed, error seed) per ciphertext
    LB_CUDA(cudaMemcpyAsync(seeds, host_seeds, (size_t)batch * 128, cudaMemcpyHostToDevice, stream));
    const bool fold_e = (P == 1); // one special prime: the error never needs its own transforms
    const long total = batch * poly;
    if (fold_e) {
        // u and e stay signed bytes: the transforms that consume them reduce them into their primes while loading
        const long n_small = (long)batch << hp.logN;
        count_launch("sample_small_i8_kernel", stream, (double)n_small);
        sample_small_i8_kernel<<<grid_for(ctx, n_small), kSampThreads, 0, stream>>>(reinterpret_cast<signed char *>(u), seeds, 32, 0, hp.logN,
                                                                                   n_small);
        LB_CUDA(cudaGetLastError());
        count_launch("sample_small_i8_kernel", stream, (double)n_small);
        sample_small_i8_kernel<<<grid_for(ctx, n_small), kSampThreads, 0, stream>>>(reinterpret_cast<signed char *>(e), seeds + 16, 32, 1,
                                                                                   hp.logN, n_small);
        LB_CUDA(cudaGetLastError());
        // u's transform stores its products with the two key polynomials straight away: cx[b][p][QP][N] = pk[p] * NTT(u[b])
        NttJob j;
        j.small = reinterpret_cast<const signed char *>(u);
        j.dst = cx;
        j.n_groups = batch;
        j.per_group = QP;
        j.size_l = Q;
        j.dst_outer = 2 * QP;
        j.mul2 = pk;
        if ((rc = ntt_forward(ctx, j, stream))) return rc;
    } else {
        if ((rc = sample_small(ctx, 0, seeds, 32, batch, Q, P, u, stream))) return rc;
        if ((rc = sample_small(ctx, 1, seeds + 16, 32, batch, Q, P, e, stream))) return rc;
        NttJob j;
        j.src = u;
        j.dst = u;
        j.n_groups = 2 * batch; // u and e are adjacent
        j.per_group = QP;
        j.size_l = Q;
        if ((rc = ntt_forward(ctx, j, stream))) return rc;
        count_launch("encrypt_combine_kernel", stream);
        encrypt_combine_kernel<<<grid_for(ctx, total), kSampThreads, 0, stream>>>(cx, pk, u, e, ctx->d_mc, hp.logN, poly, total);
        LB_CUDA(cudaGetLastError());
    }
    // moddown of 2*batch polynomials from QP to Q
    const DevLevel &dl = ctx->d_level[Q];
    NttJob inv;
    inv.src = cx;
    inv.dst = pc;
    inv.n_groups = 2 * batch;
    inv.per_group = P;
    inv.size_l = 0;
    inv.src_group_stride = QP;
    inv.src_row_off = Q;
    inv.dst_group_stride = P;
    inv.fold = P > 1 ? dl.pfold : nullptr;
    if ((rc = ntt_inverse(ctx, inv, stream))) return rc;
    NttJob fwd;
    fwd.src = pc;
    fwd.dst = ct;
    fwd.n_groups = 2 * batch;
    fwd.per_group = Q;
    fwd.size_l = Q;
    fwd.src_group_stride = P;
    fwd.dst_group_stride = Q;
    fwd.bconv_n = P;
    fwd.bconv_mat = P > 1 ? dl.phat_mod : nullptr;
    fwd.mat_row_stride = P;
    fwd.aux = cx;
    fwd.aux_group_stride = QP;
    fwd.scal = dl.p_inv;
    fwd.scal_s = dl.p_inv_s;
    fwd.split = 2;
    if (fold_e) {
        fwd.esmall = reinterpret_cast<const signed char *>(e);
        fwd.esmall_p = hp.q[Q];
    }
    if (pt && pt_is_coeff) {
        fwd.presub = pt;
        fwd.presub_outer = Q;
        fwd.presub_inner = 1;
        fwd.presub_scal = ctx->d_p_mod_q;
        fwd.presub_scal_s = ctx->d_p_mod_q_s;
    } else {
        fwd.add = pt;
        fwd.add_group_stride = 0;
        fwd.add_outer = Q;
        fwd.add_inner = pt ? 1 : 0;
    }
    return ntt_forward(ctx, fwd, stream);
}

} // namespace lb
