// Hybrid key switching, rescale, rotation and hoisted rotation sums.
//
// Reference flow (cahel-main/src/eval_key_switch.cu:80-216): modup (INTT, per-digit base
// conversion, per-digit NTT) -> inner product with the key -> two moddowns (INTT of the
// special limbs, base conversion, NTT, (cx - delta) P^-1) -> add to the ciphertext; about
// fourteen launches with every intermediate written to HBM.
//
// Here the base conversions live inside the forward transform's load stage and the
// moddown / rescale closing arithmetic (and the final addition to the ciphertext) inside
// its store stage, so a key switch is five launches:
//   1 INTT of the L input limbs (mod-up scaling folded into the closing constants)
//   2 NTT of all beta x (L + P) digit limbs with the base conversion fused into the load;
//     a digit's own limbs are never copied: the inner product reads them from the input
//   3 inner product over digits (128-bit lazy accumulation, one reduction per output)
//   4 INTT of the 2 x P special limbs (mod-down scaling folded in)
//   5 NTT of 2 x L limbs: load = P->Ql conversion, store = (cx - delta) P^-1 + ct
#include "context.h"

namespace lb {

constexpr int kKsThreads = 256;
constexpr int kMaxSteps = 32;

struct KsWs {
    u64 *coef, *digits, *cx, *pc, *tmp;
};

// rows of N words a key switch of `batch` ciphertexts needs:
// coef[b][L] + digits[b][beta][LP] + cx[b][2][LP] + pc[b][2][P] + tmp[b][3][L]
static size_t ks_rows(const Context *ctx, int L)
{
    const HostParams &hp = ctx->hp;
    const size_t P = hp.size_P, LP = L + P, beta = hp.level[L].beta;
    return L + beta * LP + 2 * LP + 2 * P + 3 * (size_t)L;
}

size_t keyswitch_workspace_bytes(const Context *ctx, int L) { return ks_rows(ctx, L) * ctx->hp.N * sizeof(u64); }

static int get_ws(Context *ctx, int L, int batch, KsWs &w)
{
    const HostParams &hp = ctx->hp;
    const size_t N = hp.N, P = hp.size_P, LP = L + P, B = batch;
    const size_t beta = hp.level[L].beta;
    int rc = ctx->ensure_workspace(ks_rows(ctx, L) * N * sizeof(u64) * B);
    if (rc) return rc;
    u64 *p = reinterpret_cast<u64 *>(ctx->ws);
    w.coef = p; p += B * L * N;
    w.digits = p; p += B * beta * LP * N;
    w.cx = p; p += B * 2 * LP * N;
    w.pc = p; p += B * 2 * P * N;
    w.tmp = p;
    return LB_OK;
}

// ciphertexts per pass so that the scratch stays below ~2 GiB
static int sub_batch(const Context *ctx, int L, int batch)
{
    const size_t per = ks_rows(ctx, L) * ctx->hp.N * sizeof(u64);
    size_t cap = (size_t(2) << 30) / per;
    if (cap < 1) cap = 1;
    return (size_t)batch < cap ? batch : (int)cap;
}

static int check_level(const Context *ctx, int L)
{
    if (ctx->hp.size_P < 1) { set_error("key switching needs at least one special prime"); return LB_ERR_INVALID_ARG; }
    if (L < 1 || L > ctx->hp.size_Q) { set_error("ciphertext level is out of range"); return LB_ERR_INVALID_ARG; }
    if (ctx->hp.size_Q % ctx->hp.size_P != 0) {
        // the reference sizes keys by floor(size_Q / size_P) digits but switches with ceil(size_Ql / size_P)
        set_error("special_modulus_size must divide the number of data primes");
        return LB_ERR_INVALID_ARG;
    }
    return LB_OK;
}

// ---- step 1+2: mod-up (cahel-main/src/rns_bconv.cu:668-792) -----------------------------
// cks: polynomial b at row b * cks_stride

static int modup_into(Context *ctx, int L, int batch, const u64 *cks, long cks_stride, u64 *coef, u64 *digits, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const int P = hp.size_P, LP = L + P, alpha = P, beta = hp.level[L].beta;
    const DevLevel &dl = ctx->d_level[L];
    NttJob inv;
    inv.src = cks;
    inv.dst = coef;
    inv.n_groups = batch;
    inv.per_group = L;
    inv.size_l = L;
    inv.src_group_stride = cks_stride;
    inv.dst_group_stride = L;
    inv.fold = alpha > 1 ? dl.fold : nullptr;
    int rc = ntt_inverse(ctx, inv, stream);
    if (rc) return rc;
    NttJob fwd;
    fwd.src = coef;
    fwd.dst = digits;
    fwd.n_groups = batch * beta;
    fwd.per_group = LP;
    fwd.split = beta;
    fwd.size_l = L;
    fwd.src_outer = L;
    fwd.dst_group_stride = LP;
    fwd.digit_alpha = alpha;
    fwd.bconv_n = alpha;
    fwd.bconv_mat = alpha > 1 ? dl.hat_mod : nullptr;
    fwd.mat_group_stride = (long)LP * alpha;
    fwd.mat_row_stride = alpha;
    return ntt_forward(ctx, fwd, stream);
}

// ---- step 3: inner product (cahel-main/src/eval_key_switch.cu:13-76; with a gather and a
// loop over steps it is also the hoisting accumulation of cahel-main/src/evaluate.cu:2572-2599)

struct IpArgs {
    const u64 *evk[kMaxSteps];
    const uint32_t *perm[kMaxSteps];
    int n_steps;
};

// grid: x over the coefficients of a limb (two per thread without a gather, one with), y = limb of
// QlP, z = blocks of ciphertexts (four with a gather, two without); no index division, 16-byte accesses on the streaming path.  A thread
// applies every key word it loads to all ciphertexts of its block: the keys (and the permutation tables of a hoisting) come
// from L2 once per block of ciphertexts instead of once per ciphertext, which was what bounded the hoisting sum
// (15 steps x 2 digits of key per ciphertext: 17 GB of L2 reads per launch at 190 ciphertexts).
template <bool GATHER>
constexpr int ip_cts() { return GATHER ? 4 : 2; }
template <bool GATHER>
__global__ void __launch_bounds__(kKsThreads) inner_product_kernel(const u64 *__restrict__ digits, const u64 *__restrict__ own,
                                                                   const long own_stride, u64 *__restrict__ cx,
                                                                   const ModConst *__restrict__ mc, const IpArgs args, const int logN,
                                                                   const int L, const int LP, const int size_Q, const int size_QP,
                                                                   const int alpha, const int beta, const int batch)
{
    constexpr int V = GATHER ? 1 : 2, B = ip_cts<GATHER>();
    const long per_ct = (long)LP << logN;
    const int r = blockIdx.y;
    const int tbl = r < L ? r : size_Q + (r - L);
    const ModConst m = mc[tbl];
    const int own_digit = r < L ? r / alpha : -1;
    const long n = 1L << logN;
    for (long b0 = (long)blockIdx.z * B; b0 < batch; b0 += (long)gridDim.z * B) {
        const int nb = (int)min((long)B, batch - b0);
        for (long k = ((long)blockIdx.x * blockDim.x + threadIdx.x) * V; k < n; k += (long)gridDim.x * blockDim.x * V) {
            u128d a0[B][V], a1[B][V];
            u64 r0[B][V], r1[B][V];
#pragma unroll
            for (int c = 0; c < B; ++c) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    a0[c][v] = a1[c][v] = u128d{0, 0};
                    r0[c][v] = r1[c][v] = 0;
                }
            }
            // one term = one digit of one step; the operands of term t + 1 are requested before term t is multiplied,
            // so the loads of a term have the whole multiply-accumulate of its predecessor to arrive in
            struct Term {
                u64 k0[V], k1[V], d[B][V];
            };
            auto fetch = [&](const int t) {
                Term x;
                const int s = t / beta, j = t - s * beta;
                const u64 *key = args.evk[s];
                const long kk = GATHER && args.perm[s] ? (long)args.perm[s][k] : k;
                const u64 *kb = key + ((((long)j * 2) * size_QP + tbl) << logN) + k;
                if (GATHER) {
                    x.k0[0] = kb[0];
                    x.k1[0] = kb[(long)size_QP << logN];
                } else {
                    const ulonglong2 kv0 = *reinterpret_cast<const ulonglong2 *>(kb);
                    const ulonglong2 kv1 = *reinterpret_cast<const ulonglong2 *>(kb + ((long)size_QP << logN));
                    x.k0[0] = kv0.x; x.k0[V - 1] = kv0.y;
                    x.k1[0] = kv1.x; x.k1[V - 1] = kv1.y;
                }
#pragma unroll
                for (int c = 0; c < B; ++c) {
                    if (c < nb) {
                        const long b = b0 + c;
                        const u64 *src = (j == own_digit) ? own + ((b * own_stride) << logN) + ((long)r << logN)
                                                          : digits + b * beta * per_ct + (((long)j * LP + r) << logN);
                        if (GATHER) {
                            x.d[c][0] = src[kk];
                        } else {
                            const ulonglong2 dv = *reinterpret_cast<const ulonglong2 *>(src + k);
                            x.d[c][0] = dv.x; x.d[c][V - 1] = dv.y;
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < V; ++v) x.d[c][v] = 0;
                    }
                }
                return x;
            };
            const int n_terms = args.n_steps * beta;
            int pending = 0;
            Term cur = fetch(0);
            for (int t = 0; t < n_terms; ++t) {
                const Term nxt = t + 1 < n_terms ? fetch(t + 1) : cur;
#pragma unroll
                for (int c = 0; c < B; ++c) {
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        mac_wide(a0[c][v], cur.d[c][v], cur.k0[v]);
                        mac_wide(a1[c][v], cur.d[c][v], cur.k1[v]);
                    }
                }
                if (++pending == 32) {
#pragma unroll
                    for (int c = 0; c < B; ++c) {
#pragma unroll
                        for (int v = 0; v < V; ++v) {
                            r0[c][v] = add_mod(r0[c][v], barrett128(a0[c][v], m.q, m.r0, m.r1), m.q);
                            r1[c][v] = add_mod(r1[c][v], barrett128(a1[c][v], m.q, m.r0, m.r1), m.q);
                            a0[c][v] = a1[c][v] = u128d{0, 0};
                        }
                    }
                    pending = 0;
                }
                cur = nxt;
            }
#pragma unroll
            for (int c = 0; c < B; ++c) {
                if (c < nb) {
                    u64 *o0 = cx + 2 * (b0 + c) * per_ct + ((long)r << logN) + k, *o1 = o0 + per_ct;
#pragma unroll
                    for (int v = 0; v < V; ++v) {
                        r0[c][v] = add_mod(r0[c][v], barrett128(a0[c][v], m.q, m.r0, m.r1), m.q);
                        r1[c][v] = add_mod(r1[c][v], barrett128(a1[c][v], m.q, m.r0, m.r1), m.q);
                    }
                    if (GATHER) {
                        o0[0] = r0[c][0];
                        o1[0] = r1[c][0];
                    } else {
                        *reinterpret_cast<ulonglong2 *>(o0) = make_ulonglong2(r0[c][0], r0[c][V - 1]);
                        *reinterpret_cast<ulonglong2 *>(o1) = make_ulonglong2(r1[c][0], r1[c][V - 1]);
                    }
                }
            }
        }
    }
}

static int inner_product_steps(Context *ctx, int L, int batch, const u64 *digits, const u64 *own, long own_stride, const IpArgs &args,
                               u64 *cx, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const int LP = L + hp.size_P;
    bool gather = false;
    for (int s = 0; s < args.n_steps; ++s) gather = gather || args.perm[s] != nullptr;
    const long per_thread = gather ? 1 : 2;
    long gx = ((long)hp.N / per_thread + kKsThreads - 1) / kKsThreads;
    if (gx < 1) gx = 1;
    const int per_block = gather ? ip_cts<true>() : ip_cts<false>();
    const int zb = (batch + per_block - 1) / per_block;
    const dim3 grid((unsigned)gx, (unsigned)LP, (unsigned)(zb < 65535 ? zb : 65535));
    // digits (beta rows per output row, the own limbs included), both key polynomials per step and digit, two outputs
    count_launch("inner_product_kernel", stream,
                 8.0 * hp.N * LP * batch * (double)hp.level[L].beta + 8.0 * hp.N * LP * 2.0 * hp.level[L].beta * args.n_steps +
                     8.0 * hp.N * LP * 2.0 * batch);
    if (gather)
        inner_product_kernel<true><<<grid, kKsThreads, 0, stream>>>(digits, own, own_stride, cx, ctx->d_mc, args, hp.logN, L, LP, hp.size_Q,
                                                                   hp.size_QP, hp.size_P, hp.level[L].beta, batch);
    else
        inner_product_kernel<false><<<grid, kKsThreads, 0, stream>>>(digits, own, own_stride, cx, ctx->d_mc, args, hp.logN, L, LP, hp.size_Q,
                                                                    hp.size_QP, hp.size_P, hp.level[L].beta, batch);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- step 4+5: mod-down (cahel-main/src/rns_bconv.cu:965-1053, ntt_moddown.cu:244-252) -----
// cx: [batch][ppc][LP][N]; polynomial (b, p) goes to out + (b * out_outer + p * out_inner) rows

struct Placement {
    long outer, inner; // row strides between ciphertexts and between the polynomials of one
};

static int moddown_into(Context *ctx, int L, int batch, int ppc, const u64 *cx, u64 *pc, u64 *out, Placement po, const u64 *add,
                        Placement pa, int add_inner, cudaStream_t stream, const u64 *add1 = nullptr, long add1_outer = 0)
{
    const HostParams &hp = ctx->hp;
    const int P = hp.size_P, LP = L + P;
    const DevLevel &dl = ctx->d_level[L];
    NttJob inv;
    inv.src = cx;
    inv.dst = pc;
    inv.n_groups = batch * ppc;
    inv.per_group = P;
    inv.size_l = 0; // every row is a special limb
    inv.src_group_stride = LP;
    inv.src_row_off = L;
    inv.dst_group_stride = P;
    inv.fold = P > 1 ? dl.pfold : nullptr;
    int rc = ntt_inverse(ctx, inv, stream);
    if (rc) return rc;
    NttJob fwd;
    fwd.src = pc;
    fwd.dst = out;
    fwd.n_groups = batch * ppc;
    fwd.per_group = L;
    fwd.split = ppc;
    fwd.size_l = L;
    fwd.src_group_stride = P;
    fwd.dst_group_stride = po.inner;
    fwd.dst_outer = po.outer;
    fwd.bconv_n = P;
    fwd.bconv_mat = P > 1 ? dl.phat_mod : nullptr;
    fwd.mat_group_stride = 0;
    fwd.mat_row_stride = P;
    fwd.aux = cx;
    fwd.aux_group_stride = LP;
    fwd.scal = dl.p_inv;
    fwd.scal_s = dl.p_inv_s;
    fwd.add = add;
    fwd.add_group_stride = pa.inner;
    fwd.add_outer = pa.outer;
    fwd.add_inner = add ? add_inner : 0;
    fwd.add1 = add1;
    fwd.add1_outer = add1_outer;
    return ntt_forward(ctx, fwd, stream);
}

// ---- public pieces ----------------------------------------------------------------------

int modup(Context *ctx, int L, const u64 *cks, u64 *digits, cudaStream_t stream)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    KsWs w;
    if ((rc = get_ws(ctx, L, 1, w))) return rc;
    if ((rc = modup_into(ctx, L, 1, cks, L, w.coef, digits, stream))) return rc;
    // materialise the digit's own limbs for callers that want the reference layout
    const HostParams &hp = ctx->hp;
    const int LP = L + hp.size_P, alpha = hp.size_P;
    for (int j = 0; j < hp.level[L].beta; ++j) {
        const int s = j * alpha, e = s + alpha < L ? s + alpha : L;
        LB_CUDA(cudaMemcpyAsync(digits + ((size_t)j * LP + s) * hp.N, cks + (size_t)s * hp.N, (size_t)(e - s) * hp.N * 8,
                                cudaMemcpyDeviceToDevice, stream));
    }
    return LB_OK;
}

int inner_product(Context *ctx, int L, const u64 *digits, const u64 *cks, const u64 *evk, u64 *cx, cudaStream_t stream)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    IpArgs args = {};
    args.evk[0] = evk;
    args.perm[0] = nullptr;
    args.n_steps = 1;
    return inner_product_steps(ctx, L, 1, digits, cks, L, args, cx, stream);
}

int moddown(Context *ctx, int L, const u64 *cx, u64 *out, cudaStream_t stream)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    KsWs w;
    if ((rc = get_ws(ctx, L, 1, w))) return rc;
    return moddown_into(ctx, L, 1, 1, cx, w.pc, out, Placement{L, L}, nullptr, Placement{0, 0}, 0, stream);
}

// out(b, p) = (p < add_inner ? add(b, p) : 0) + moddown(<modup(cks_b), evk>)_p for a batch of ciphertexts
static int keyswitch_batch(Context *ctx, int L, int batch, const u64 *cks, long cks_stride, const u64 *evk, const u64 *add,
                           Placement pa, int add_inner, u64 *out, Placement po, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const int step = sub_batch(ctx, L, batch);
    for (int b0 = 0; b0 < batch; b0 += step) {
        const int nb = batch - b0 < step ? batch - b0 : step;
        KsWs w;
        int rc = get_ws(ctx, L, nb, w);
        if (rc) return rc;
        const u64 *cks_b = cks + ((size_t)b0 * cks_stride << hp.logN);
        if ((rc = modup_into(ctx, L, nb, cks_b, cks_stride, w.coef, w.digits, stream))) return rc;
        IpArgs args = {};
        args.evk[0] = evk;
        args.n_steps = 1;
        if ((rc = inner_product_steps(ctx, L, nb, w.digits, cks_b, cks_stride, args, w.cx, stream))) return rc;
        const u64 *add_b = add ? add + ((size_t)b0 * pa.outer << hp.logN) : nullptr;
        u64 *out_b = out + ((size_t)b0 * po.outer << hp.logN);
        if ((rc = moddown_into(ctx, L, nb, 2, w.cx, w.pc, out_b, po, add_b, pa, add_inner, stream))) return rc;
    }
    return LB_OK;
}

int keyswitch(Context *ctx, int L, const u64 *cks, const u64 *evk, const u64 *add0, const u64 *add1, u64 *out, cudaStream_t stream)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    const size_t poly = (size_t)L * ctx->hp.N;
    if (add0 && add1 && add1 != add0 + poly) { set_error("addends must be the two polynomials of one ciphertext"); return LB_ERR_INVALID_ARG; }
    if (!add0 && add1) { set_error("an addend for the second polynomial alone is not supported"); return LB_ERR_INVALID_ARG; }
    return keyswitch_batch(ctx, L, 1, cks, L, evk, add0, Placement{2L * L, L}, add0 ? (add1 ? 2 : 1) : 0, out, Placement{2L * L, L}, stream);
}

// cahel-main/src/evaluate.cu:2019-2056, for `batch` size-3 ciphertexts stored back to back
int relinearize(Context *ctx, int L, int batch, u64 *ct3, const u64 *rlk, cudaStream_t stream)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    const size_t poly = (size_t)L * ctx->hp.N;
    const Placement p3{3L * L, L};
    return keyswitch_batch(ctx, L, batch, ct3 + 2 * poly, 3L * L, rlk, ct3, p3, 2, ct3, p3, stream);
}

// cahel-main/src/rns.cu:544-570 (floors): two launches for all polynomials.
// Polynomial p of ciphertext b sits at row b * in_outer + p * L of `in`; the output is dense
// [batch][ppc][L-1][N].
int rescale(Context *ctx, int L, int batch, int ppc, const u64 *in, long in_outer, u64 *out, cudaStream_t stream)
{
    if (L < 2 || L > ctx->hp.size_Q) { set_error("cannot rescale: no next level"); return LB_ERR_INVALID_ARG; }
    const int n_polys = batch * ppc;
    int rc = ctx->ensure_workspace((size_t)n_polys * ctx->hp.N * 8);
    if (rc) return rc;
    u64 *last = reinterpret_cast<u64 *>(ctx->ws);
    NttJob inv;
    inv.src = in;
    inv.dst = last;
    inv.n_groups = n_polys;
    inv.per_group = 1;
    inv.split = ppc;
    inv.size_l = 1;
    inv.tbl_off = L - 1;
    inv.src_group_stride = L;
    inv.src_outer = in_outer;
    inv.src_row_off = L - 1;
    inv.dst_group_stride = 1;
    if ((rc = ntt_inverse(ctx, inv, stream))) return rc;
    const DevLevel &dl = ctx->d_level[L];
    NttJob fwd;
    fwd.src = last;
    fwd.dst = out;
    fwd.n_groups = n_polys;
    fwd.per_group = L - 1;
    fwd.split = ppc;
    fwd.size_l = L - 1;
    fwd.src_group_stride = 1;
    fwd.dst_group_stride = L - 1;
    fwd.bconv_n = 1;
    fwd.aux = in;
    fwd.aux_group_stride = L;
    fwd.aux_outer = in_outer;
    fwd.scal = dl.qlast_inv;
    fwd.scal_s = dl.qlast_inv_s;
    return ntt_forward(ctx, fwd, stream);
}

// cahel-main/src/evaluate.cu:2631-2686 for a batch of size-2 ciphertexts stored back to back:
// permute both polynomials, then switch the permuted c1
int rotate(Context *ctx, int L, int batch, u64 *ct, int elt_idx, const u64 *glk, cudaStream_t stream, bool accumulate)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    const HostParams &hp = ctx->hp;
    const int step = sub_batch(ctx, L, batch);
    const size_t poly = (size_t)L * hp.N;
    const Placement p2{2L * L, L};
    for (int b0 = 0; b0 < batch; b0 += step) {
        const int nb = batch - b0 < step ? batch - b0 : step;
        KsWs w;
        if ((rc = get_ws(ctx, L, nb, w))) return rc;
        u64 *ct_b = ct + 2 * poly * b0;
        // accumulate: the image of c0 takes c0 along, and the closing transform adds the old c1 to the new one
        if (accumulate) rc = poly_galois_plus_c0(ctx, elt_idx, L, nb, ct_b, w.tmp, stream);
        else rc = poly_galois(ctx, elt_idx, 2L * L * nb, ct_b, w.tmp, stream);
        if (rc) return rc;
        if ((rc = modup_into(ctx, L, nb, w.tmp + poly, 2L * L, w.coef, w.digits, stream))) return rc;
        IpArgs args = {};
        args.evk[0] = glk;
        args.n_steps = 1;
        if ((rc = inner_product_steps(ctx, L, nb, w.digits, w.tmp + poly, 2L * L, args, w.cx, stream))) return rc;
        if ((rc = moddown_into(ctx, L, nb, 2, w.cx, w.pc, ct_b, p2, w.tmp, p2, 1, stream, accumulate ? ct_b + poly : nullptr, 2L * L)))
            return rc;
    }
    return LB_OK;
}

// sum over steps of the permuted c0 (cahel-main/src/evaluate.cu:2560-2568); c0 of ciphertext b at row b * ct_stride
__global__ void __launch_bounds__(kKsThreads) galois_sum_kernel(const u64 *__restrict__ src, const long ct_stride, u64 *__restrict__ dst,
                                                                const ModConst *__restrict__ mc, const IpArgs args, const int logN,
                                                                const int L, const long total, const int plus_self)
{
    const long n_mask = (1L << logN) - 1;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long row = i >> logN, k = i & n_mask;
        const long b = row / L, r = row - b * L;
        const u64 q = mc[r].q;
        const u64 *s0 = src + ((b * ct_stride + r) << logN);
        u64 acc = plus_self ? s0[k] : 0;
        for (int s = 0; s < args.n_steps; ++s) acc = add_mod(acc, s0[args.perm[s][k]], q);
        dst[i] = acc;
    }
}

// cahel-main/src/evaluate.cu:2412-2629 for a batch of size-2 ciphertexts stored back to back:
// one mod-up, per step a permuted inner product, two mod-downs
int hoisting(Context *ctx, int L, int batch, u64 *ct, int n_steps, const int *elt_idx, const u64 *const *glks, cudaStream_t stream,
             bool accumulate)
{
    int rc = check_level(ctx, L);
    if (rc) return rc;
    if (n_steps < 1 || n_steps > kMaxSteps) { set_error("hoisting supports 1 to 32 steps per call"); return LB_ERR_INVALID_ARG; }
    const HostParams &hp = ctx->hp;
    IpArgs args = {};
    args.n_steps = n_steps;
    for (int s = 0; s < n_steps; ++s) {
        if (elt_idx[s] < 0 || elt_idx[s] >= (int)hp.galois_elts.size()) { set_error("Galois key not present in hoisting"); return LB_ERR_LOGIC; }
        args.evk[s] = glks[s];
        args.perm[s] = ctx->d_perm + ((size_t)elt_idx[s] << hp.logN);
    }
    const int step = sub_batch(ctx, L, batch);
    const size_t poly = (size_t)L * hp.N;
    for (int b0 = 0; b0 < batch; b0 += step) {
        const int nb = batch - b0 < step ? batch - b0 : step;
        KsWs w;
        if ((rc = get_ws(ctx, L, nb, w))) return rc;
        u64 *ct_b = ct + 2 * poly * b0;
        if ((rc = modup_into(ctx, L, nb, ct_b + poly, 2L * L, w.coef, w.digits, stream))) return rc;
        if ((rc = inner_product_steps(ctx, L, nb, w.digits, ct_b + poly, 2L * L, args, w.cx, stream))) return rc;
        const long total = ((long)L << hp.logN) * nb;
        long blocks = (total + kKsThreads - 1) / kKsThreads;
        const long cap = (long)ctx->sm_count * 16;
        if (blocks > cap) blocks = cap;
        count_launch("galois_sum_kernel", stream);
        galois_sum_kernel<<<(int)blocks, kKsThreads, 0, stream>>>(ct_b, 2L * L, w.tmp, ctx->d_mc, args, hp.logN, L, total, accumulate ? 1 : 0);
        LB_CUDA(cudaGetLastError());
        if ((rc = moddown_into(ctx, L, nb, 2, w.cx, w.pc, ct_b, Placement{2L * L, L}, w.tmp, Placement{L, L}, 1, stream,
                               accumulate ? ct_b + poly : nullptr, 2L * L)))
            return rc;
    }
    return LB_OK;
}

} // namespace lb
