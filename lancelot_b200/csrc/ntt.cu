// Batched negacyclic NTT / inverse NTT over RNS limbs for sm_100a.
//
// Mathematical definition (must equal the reference's, cahel-main/src/ntt/ntt_1d.cu:38-74,
// :129-171 and butterfly.cuh:10-43; its production path is the two-kernel radix-8 pair in
// cahel-main/src/ntt/fntt_2d.cu:8,126,872 and intt_2d.cu:8,103,693):
//   forward: stages m = 1,2,..,N/2, butterfly (x,y) -> (x + w y, x - w y), w = psi^bitrev(m+k);
//            natural order in, bit-reversed order out, canonical residues out.
//   inverse: the exact inverse map (the reference halves in every butterfly; here N^-1 is
//            folded into the last stage).
//
// Schedule (new): ONE kernel per transform and one pass over HBM.  A limb of N = 2^16
// coefficients (512 KiB) does not fit one SM, so a thread-block cluster of C = N / 8192 CTAs
// owns a limb.  The first log2(C) stages run in registers on coalesced strided global loads;
// their outputs are scattered to the owning CTA through distributed shared memory; each
// CTA then finishes an independent 8192-point transform in its own shared memory with
// register-blocked radix-8 passes and writes its contiguous part of the result with
// 16-byte stores.  The inverse mirrors this (contiguous loads, local passes, DSMEM gather,
// last log2(C) stages in registers, coalesced strided stores).  Algorithmic traffic is
// 16 bytes per coefficient per transform; twiddles (16 B each, value + Shoup quotient) are
// read through L2.
#include <cooperative_groups.h>

#include "context.h"
#include "ntt_butterfly.cuh"

namespace cg = cooperative_groups;

namespace lb {

// Launch shape: threads per CTA, CTAs per SM the register allocation aims at, and log2 of the points one
// CTA keeps in shared memory (8192 points: 64 KiB + padding, three CTAs per SM).  Register passes take at most
// three stages (radix 8).
constexpr int kNttThreads = 256;
constexpr int kNttMinBlocks = 3;
constexpr int kMaxLocalLog = 13;
constexpr int kMaxRadixLog = 3;

struct NttK {
    const u64 *src;
    u64 *dst;
    const ulonglong2 *tw;
    const ModConst *mc;
    int logN, per_group, split, size_l, size_Q, tbl_off;
    long src_group_stride, dst_group_stride, aux_group_stride, add_group_stride;
    long src_outer, dst_outer, aux_outer, add_outer;
    int src_row_off, skip_lo, skip_hi;
    int bconv_n, digit_alpha, add_inner;
    const u64 *bconv_mat;
    long mat_group_stride, mat_row_stride;
    const u64 *aux, *scal, *scal_s, *add, *fold;
    const u64 *add1; // addend rows of the groups with inner == 1, if they sit elsewhere (see NttJob::add1)
    long add1_outer;
    const u64 *mul2; // forward epilogue: two products per row (see NttJob::mul2)
    const u64 *presub, *presub_scal, *presub_scal_s;
    const signed char *esmall;
    const signed char *small;
    u64 esmall_p;
    long presub_outer;
    int presub_inner;
    int npass;
    int nwide; // passes whose butterflies cross warp chunks (forward: the first nwide, inverse: the last nwide)
    int wlog;  // log2 of the contiguous chunk one warp owns in the other passes
    unsigned char S[8];
};

// one spare word per 16 keeps the stride-8 and stride-1 passes off the same banks
LB_D int sidx(int i) { return i + (i >> 4); }

// S consecutive forward stages on 2^S register values; stage u uses twiddle (t0 << u) + block
template <int S, int MODE>
LB_D void fwd_core(u64 (&v)[1 << S], const ulonglong2 *__restrict__ tw, const unsigned t0, const u64 q, const u64 q2)
{
#pragma unroll
    for (int u = 0; u < S; ++u) {
        const int half = 1 << (S - 1 - u);
        if (MODE == kF64Tight && u == 3) { // three stages since the values were centred: centre them again
#pragma unroll
            for (int i = 0; i < (1 << S); ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q), f64_of(q2)));
        }
#pragma unroll
        for (int b = 0; b < (1 << u); ++b) {
            const ulonglong2 w = __ldg(tw + ((t0 << u) + b));
#pragma unroll
            for (int i = 0; i < half; ++i) fwd_bf<MODE>(v[b * 2 * half + i], v[b * 2 * half + i + half], w, q, q2);
        }
    }
}

// S consecutive inverse stages; stage u pairs distance 2^u and uses twiddle (tb >> u) + block.
// CLOSE: the last of them is the transform's last stage and carries the N^-1 scaling; it leaves
// canonical residues (as integers in every mode).  In kInvF64 mode q, q2 carry double(q), double(1 / q)
// and (cn, cns), (cw, cws) the closing constants and their quotients by q, all as doubles.
template <int S, bool CLOSE, int IM>
LB_D void inv_core(u64 (&v)[1 << S], const ulonglong2 *__restrict__ itw, const unsigned tb, const u64 q, const u64 q2,
                   const u64 cn, const u64 cns, const u64 cw, const u64 cws)
{
#pragma unroll
    for (int u = 0; u < S; ++u) {
        const int dist = 1 << u;
        if (IM == kInvF64Tight && u > 0 && (u & 1) == 0) { // two stages since the values were centred
#pragma unroll
            for (int i = 0; i < (1 << S); ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q), f64_of(q2)));
        }
#pragma unroll
        for (int b = 0; b < (1 << (S - 1 - u)); ++b) {
            if (CLOSE && u == S - 1) {
#pragma unroll
                for (int i = 0; i < dist; ++i) {
                    u64 &x = v[b * 2 * dist + i], &y = v[b * 2 * dist + i + dist];
                    if (is_inv_f64(IM)) {
                        const double xd = f64_of(x), yd = f64_of(y), qd = f64_of(q), qi = f64_of(q2);
                        x = f64_canon(f64_mulmod(__dadd_rn(xd, yd), f64_of(cn), f64_of(cns), qd), qd, qi);
                        y = f64_canon(f64_mulmod(__dadd_rn(xd, -yd), f64_of(cw), f64_of(cws), qd), qd, qi);
                    } else {
                        const u64 s = x + y, d = x + (q2 << 1) - y; // inputs below 4q
                        x = shoup_mul(s, cn, cns, q);
                        y = shoup_mul(d, cw, cws, q);
                    }
                }
            } else {
                const ulonglong2 w = __ldg(itw + ((tb >> u) + b));
#pragma unroll
                for (int i = 0; i < dist; ++i) inv_bf<IM>(v[b * 2 * dist + i], v[b * 2 * dist + i + dist], w, q, q2);
            }
        }
    }
}

template <int R>
LB_D void load_contig(u64 (&v)[R], const u64 *p)
{
    if (R == 1) {
        v[0] = p[0];
    } else {
#pragma unroll
        for (int i = 0; i < R; i += 2) {
            const ulonglong2 t = *reinterpret_cast<const ulonglong2 *>(p + i);
            v[i] = t.x;
            v[i + 1] = t.y;
        }
    }
}

template <int R>
LB_D void store_contig(const u64 (&v)[R], u64 *p)
{
#pragma unroll
    for (int i = 0; i < R; i += 2) *reinterpret_cast<ulonglong2 *>(p + i) = make_ulonglong2(v[i], v[i + 1]);
}

// ---- forward --------------------------------------------------------------------------

// Where a transform input comes from: a plain row, one row reduced into this row's prime,
// or an approximate fast base conversion of up to alpha rows (cahel-main/src/rns_bconv.cu:
// 562-623 for mod-up, :847-866 and :166-199 for mod-down), evaluated while loading.
struct FwdIn {
    const u64 *src;
    const u64 *mat;
    const u64 *sub; // optional: the loaded value becomes value - sub[k] * sub_w (plaintext folded into a mod-down)
    const signed char *es; // optional small error polynomial e of an encryption (see the encrypt path)
    const signed char *small; // the input itself as signed bytes (then src is not read)
    int n, logN;
    u64 q, r0, r1, sub_w, sub_ws, es_p;
};

LB_D u64 load_in(const FwdIn &in, const int idx)
{
    u64 v;
    if (in.small) {
        const int ev = in.small[idx];
        v = ev < 0 ? in.q - (u64)(-ev) : (u64)ev;
    } else if (in.n == 0) {
        v = in.src[idx];
    } else if (in.mat == nullptr) {
        u64 x = in.src[idx];
        if (in.es) {
            // x is INTT(pk u) on the special prime p: add e mod p first (INTT is linear, so this is the
            // special limb of pk u + e), convert, then take e off again on this prime, because the
            // caller's aux rows hold pk u without e:  (pk u + e) - NTT(delta) = pk u - NTT(delta - e)
            const int ev = in.es[idx];
            x = add_mod(x, ev < 0 ? in.es_p - (u64)(-ev) : (u64)ev, in.es_p);
            v = barrett64(x, in.q, in.r1);
            v = sub_mod(v, ev < 0 ? in.q - (u64)(-ev) : (u64)ev, in.q);
        } else {
            v = barrett64(x, in.q, in.r1);
        }
    } else {
        u128d acc;
        acc.lo = 0;
        acc.hi = 0;
        for (int i = 0; i < in.n; ++i) mac_wide(acc, in.src[((size_t)i << in.logN) + idx], __ldg(in.mat + i));
        v = barrett128(acc, in.q, in.r0, in.r1);
    }
    if (in.sub) v = sub_mod(v, shoup_mul(in.sub[idx], in.sub_w, in.sub_ws, in.q), in.q);
    return v;
}

struct FwdEpi {
    const u64 *aux; // nullptr: plain store
    const u64 *add; // optional addend
    u64 scal, scal_s;
    // optional: instead of the transform itself, store its products with two fixed rows (the two polynomials of a
    // public key): dst <- NTT(x) * mul0, dst + dst1_off <- NTT(x) * mul1
    const u64 *mul0, *mul1;
    long dst1_off;
    u64 r0, r1; // floor(2^128 / q) for those products
};

// Work split of one register pass.  A pass whose largest butterfly span exceeds a warp's chunk
// is shared out over the whole CTA; in every other pass a warp keeps to the groups of its own
// contiguous 2^wlog-point chunk, so that consecutive such passes only need a warp-level barrier.
struct PassSplit {
    int first, end, step;
};

template <int S>
LB_D PassSplit pass_split(const int logn_loc, const int wlog)
{
    PassSplit ps;
    if (wlog < 0) {
        ps.first = threadIdx.x;
        ps.end = 1 << (logn_loc - S);
        ps.step = kNttThreads;
    } else {
        const int gpw = 1 << (wlog - S), warp = threadIdx.x >> 5;
        ps.first = warp * gpw + (threadIdx.x & 31);
        ps.end = (warp + 1) * gpw;
        ps.step = 32;
    }
    return ps;
}

template <int S, int MODE>
LB_D void fwd_pass(u64 *sm, const bool from_global, u64 *gdst, const FwdIn &in, const int logn_loc, const int logt,
                   const unsigned cc, const ulonglong2 *tw, const u64 q, const u64 q2, const FwdEpi &epi, const int wlog)
{
    constexpr int R = 1 << S;
    const int logst = logt - (S - 1);
    const int logm0 = logn_loc - 1 - logt;
    const PassSplit ps = pass_split<S>(logn_loc, wlog);
    for (int g = ps.first; g < ps.end; g += ps.step) {
        const int lo = g & ((1 << logst) - 1), hi = g >> logst;
        const int base = (hi << (logt + 1)) + lo;
        u64 v[R];
        if (from_global) {
#pragma unroll
            for (int i = 0; i < R; ++i) v[i] = load_in(in, base + (i << logst));
            if (is_f64_mode(MODE)) {
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = bits_of(f64_from_u52(v[i]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) v[i] = sm[sidx(base + (i << logst))];
        }
        if (MODE == kF64Tight) {
#pragma unroll
            for (int i = 0; i < R; ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q), f64_of(q2)));
        }
        fwd_core<S, MODE>(v, tw, (cc << logm0) + hi, q, q2);
        if (gdst) { // closing pass: logst == 0, the 2^S results are contiguous
            const u64 qi = in.q; // the prime as an integer (q, q2 are the butterflies' scalars)
            if (is_f64_mode(MODE)) {
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = f64_canon(f64_of(v[i]), f64_of(q), f64_of(q2));
            } else if (MODE == kIntLazy) {
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = barrett64(v[i], qi, in.r1);
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = csub(csub(csub(v[i], q2 << 1), q2), q);
            }
            if (epi.aux) {
                u64 t[R];
                load_contig<R>(t, epi.aux + base);
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = shoup_mul(sub_mod(t[i], v[i], qi), epi.scal, epi.scal_s, qi);
                if (epi.add) {
                    load_contig<R>(t, epi.add + base);
#pragma unroll
                    for (int i = 0; i < R; ++i) v[i] = add_mod(v[i], t[i], qi);
                }
            }
            if (epi.mul0) {
                u64 t[R], w[R];
                load_contig<R>(t, epi.mul1 + base);
#pragma unroll
                for (int i = 0; i < R; ++i) w[i] = mul_mod(v[i], t[i], qi, epi.r0, epi.r1);
                store_contig<R>(w, gdst + epi.dst1_off + base);
                load_contig<R>(t, epi.mul0 + base);
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = mul_mod(v[i], t[i], qi, epi.r0, epi.r1);
            }
            store_contig<R>(v, gdst + base);
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) sm[sidx(base + (i << logst))] = v[i];
        }
    }
}

template <int MODE>
LB_D void fwd_pass_any(const int S, u64 *sm, const bool from_global, u64 *gdst, const FwdIn &in, const int logn_loc, const int logt,
                       const unsigned cc, const ulonglong2 *tw, const u64 q, const u64 q2, const FwdEpi &epi, const int wlog)
{
    if (S == 3) fwd_pass<3, MODE>(sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog);
    else if (S == 2) fwd_pass<2, MODE>(sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog);
    else fwd_pass<1, MODE>(sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog);
}

// Everything a forward CTA derives from its row index: where the limb comes from, which prime
// and tables it uses, and what the closing pass does with the result.
struct FwdRow {
    FwdIn in;
    FwdEpi epi;
    u64 *dst;
    const ulonglong2 *tw;
    u64 q;
    int mode;
};

// false: this row has nothing to transform (uniform over the cluster that owns the row)
LB_D bool fwd_row_setup(const NttK &a, const int row, FwdRow &r)
{
    const int grp = row / a.per_group, rr = row - grp * a.per_group;
    if (rr >= a.skip_lo && rr < a.skip_hi) return false;
    const int go = grp / a.split, gi = grp - go * a.split;
    int n_in = a.bconv_n;
    size_t src_row = (size_t)go * a.src_outer + a.src_row_off;
    const u64 *mat = a.bconv_mat;
    if (a.digit_alpha > 0) {
        const int s = gi * a.digit_alpha;
        const int e = min(s + a.digit_alpha, a.size_l);
        if (rr >= s && rr < e) return false; // the digit's own limbs stay in NTT form
        src_row += s;
        n_in = e - s;
        if (mat) mat += (size_t)gi * a.mat_group_stride;
    } else {
        src_row += (size_t)gi * a.src_group_stride;
    }
    if (n_in == 0) src_row += rr;
    if (mat) mat += (size_t)rr * a.mat_row_stride;
    const int tbl = rr < a.size_l ? rr + a.tbl_off : a.size_Q + (rr - a.size_l);
    const ModConst mc = a.mc[tbl];
    const int logN = a.logN;
    r.q = mc.q;
    r.tw = a.tw + ((size_t)tbl << logN);
    FwdIn &in = r.in;
    in.n = n_in;
    in.logN = logN;
    in.q = mc.q;
    in.r0 = mc.r0;
    in.r1 = mc.r1;
    in.src = a.src + (src_row << logN);
    in.mat = mat;
    in.sub = (a.presub && gi < a.presub_inner) ? a.presub + (((size_t)go * a.presub_outer + rr) << logN) : nullptr;
    in.sub_w = in.sub ? a.presub_scal[rr] : 0;
    in.sub_ws = in.sub ? a.presub_scal_s[rr] : 0;
    in.es = a.esmall ? a.esmall + ((size_t)go << logN) : nullptr;
    in.small = a.small ? a.small + ((size_t)grp << logN) : nullptr;
    in.es_p = a.esmall_p;
    r.mode = butterfly_mode(mc.q);
    r.dst = a.dst + (((size_t)go * a.dst_outer + (size_t)gi * a.dst_group_stride + rr) << logN);
    FwdEpi &epi = r.epi;
    epi.aux = a.aux ? a.aux + (((size_t)go * a.aux_outer + (size_t)gi * a.aux_group_stride + rr) << logN) : nullptr;
    epi.add = (a.add && gi < a.add_inner) ? a.add + (((size_t)go * a.add_outer + (size_t)gi * a.add_group_stride + rr) << logN) : nullptr;
    if (a.add1 && gi == 1) epi.add = a.add1 + (((size_t)go * a.add1_outer + rr) << logN);
    epi.scal = a.aux ? a.scal[rr] : 0;
    epi.scal_s = a.aux ? a.scal_s[rr] : 0;
    epi.mul0 = a.mul2 ? a.mul2 + ((size_t)rr << logN) : nullptr;
    epi.mul1 = a.mul2 ? a.mul2 + ((size_t)(a.per_group + rr) << logN) : nullptr;
    epi.dst1_off = (long)a.per_group << logN;
    epi.r0 = mc.r0;
    epi.r1 = mc.r1;
    return true;
}

template <int LOGC>
__global__ void __launch_bounds__(kNttThreads, kNttMinBlocks) ntt_fwd_kernel(const NttK a)
{
    extern __shared__ __align__(16) u64 sm[];
    constexpr int C = 1 << LOGC;
    FwdRow fr;
    if (!fwd_row_setup(a, blockIdx.x >> LOGC, fr)) return;
    const FwdIn &in = fr.in;
    FwdEpi &epi = fr.epi;
    u64 *dst = fr.dst;
    const ulonglong2 *tw = fr.tw;
    const int mode = fr.mode;
    // the butterflies' two scalars: (q, 2q), or (double(q), double(1 / q)) when they run on the FP64 pipe
    const u64 q = is_f64_mode(mode) ? bf_scalar_q<kF64>(fr.q) : fr.q, q2 = is_f64_mode(mode) ? bf_scalar_q2<kF64>(fr.q) : fr.q << 1;
    const int logn_loc = a.logN - LOGC, n_loc = 1 << logn_loc;

    unsigned c = 0;
    if constexpr (LOGC > 0) {
        cg::cluster_group cluster = cg::this_cluster();
        c = cluster.block_rank();
        // Every CTA of the cluster must be running before its shared memory is written; the
        // first loads and butterflies do not touch it, so only the first scatter waits.
        cluster.barrier_arrive();
        u64 *remote[C];
#pragma unroll
        for (int k = 0; k < C; ++k) remote[k] = cluster.map_shared_rank(sm, k);
        const int share = n_loc >> LOGC;
        auto column = [&](const int jj, const bool first) {
            const int j = c * share + jj;
            u64 v[C];
#pragma unroll
            for (int k = 0; k < C; ++k) v[k] = load_in(in, j + k * n_loc);
            if (is_f64_mode(mode)) {
#pragma unroll
                for (int k = 0; k < C; ++k) v[k] = bits_of(f64_from_u52(v[k]));
            }
            if (mode == kF64Tight) {
#pragma unroll
                for (int k = 0; k < C; ++k) v[k] = bits_of(f64_centre(f64_of(v[k]), f64_of(q), f64_of(q2)));
            }
            switch (mode) {
            case kF64: fwd_core<LOGC, kF64>(v, tw, 1u, q, q2); break;
            case kF64Tight: fwd_core<LOGC, kF64Tight>(v, tw, 1u, q, q2); break;
            case kIntLazy: fwd_core<LOGC, kIntLazy>(v, tw, 1u, q, q2); break;
            default: fwd_core<LOGC, kIntStrict>(v, tw, 1u, q, q2); break;
            }
            if (first) cluster.barrier_wait();
#pragma unroll
            for (int k = 0; k < C; ++k) remote[k][sidx(j)] = v[k];
        };
        if ((int)threadIdx.x < share) column(threadIdx.x, true);
        else cluster.barrier_wait();
        for (int jj = threadIdx.x + kNttThreads; jj < share; jj += kNttThreads) column(jj, false);
        cluster.sync(); // all scatters into this CTA have landed; from here on it only touches its own memory
        const size_t off = (size_t)c * n_loc;
        if (epi.aux) epi.aux += off;
        if (epi.add) epi.add += off;
        if (epi.mul0) { epi.mul0 += off; epi.mul1 += off; }
    }

    int logt = logn_loc - 1;
    const unsigned cc = C + c;
    for (int p = 0; p < a.npass; ++p) {
        const int S = a.S[p];
        const bool from_global = (LOGC == 0 && p == 0);
        u64 *gdst = (p == a.npass - 1) ? dst + (size_t)c * n_loc : nullptr;
        const int wlog = p < a.nwide ? -1 : a.wlog;
        switch (mode) {
        case kF64: fwd_pass_any<kF64>(S, sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog); break;
        case kF64Tight: fwd_pass_any<kF64Tight>(S, sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog); break;
        case kIntLazy: fwd_pass_any<kIntLazy>(S, sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog); break;
        default: fwd_pass_any<kIntStrict>(S, sm, from_global, gdst, in, logn_loc, logt, cc, tw, q, q2, epi, wlog); break;
        }
        logt -= S;
        if (p + 1 < a.npass) {
            if (wlog < 0) __syncthreads();
            else __syncwarp();
        }
    }
}

// ---- inverse --------------------------------------------------------------------------

// Stages a run of FP64 inverse butterflies may take before the sums, which double per stage, must be brought
// back to the residue nearest zero: operands of a butterfly stay below 2^50 (their difference below 2^51).
// `fresh`: the run starts from canonical residues below 2^bits; otherwise from |v| <= 2^(bits - 1).
struct F64Run {
    int bits, since, allowed;
    LB_D explicit F64Run(const u64 q) : bits(0), since(0), allowed(0)
    {
        while (bits < 64 && (q >> bits) != 0) ++bits; // q < 2^bits
        allowed = 51 - bits;
    }
    // true: reduce before the next `stages` stages
    LB_D bool before(const int stages)
    {
        const bool reduce = since + stages > allowed;
        if (reduce) {
            since = 0;
            allowed = 52 - bits;
        }
        since += stages;
        return reduce;
    }
};

// IM == kInvF64: `reduce` asks for the centred reduction of the loaded values (see F64Run)
template <int S, bool CLOSE, int IM>
LB_D void inv_pass(u64 *sm, const u64 *gsrc, u64 *gdst, const int logn_loc, const int logt, const unsigned cc,
                   const ulonglong2 *itw, const u64 q, const u64 q2, const u64 cn, const u64 cns, const u64 cw,
                   const u64 cws, const int wlog, const bool reduce)
{
    constexpr int R = 1 << S;
    const int logst = logt;
    const int logm0 = logn_loc - 1 - logt;
    const PassSplit ps = pass_split<S>(logn_loc, wlog);
    for (int g = ps.first; g < ps.end; g += ps.step) {
        const int lo = g & ((1 << logst) - 1), hi = g >> logst;
        const int base = (hi << (logst + S)) + lo;
        u64 v[R];
        if (gsrc) { // opening pass: logst == 0, contiguous
            load_contig<R>(v, gsrc + base);
            if (is_inv_f64(IM)) {
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = bits_of(f64_from_u52(v[i]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) v[i] = sm[sidx(base + (i << logst))];
        }
        if ((IM == kInvF64 && reduce && !gsrc) || IM == kInvF64Tight) {
#pragma unroll
            for (int i = 0; i < R; ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q), f64_of(q2)));
        }
        inv_core<S, CLOSE, IM>(v, itw, (cc << logm0) + (hi << (S - 1)), q, q2, cn, cns, cw, cws);
        if (gdst) {
#pragma unroll
            for (int i = 0; i < R; ++i) gdst[base + (i << logst)] = v[i];
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) sm[sidx(base + (i << logst))] = v[i];
        }
    }
}

template <bool CLOSE, int IM>
LB_D void inv_pass_any(const int S, u64 *sm, const u64 *gsrc, u64 *gdst, const int logn_loc, const int logt, const unsigned cc,
                       const ulonglong2 *itw, const u64 q, const u64 q2, const u64 cn, const u64 cns, const u64 cw, const u64 cws,
                       const int wlog, const bool reduce)
{
    if (S == 3) inv_pass<3, CLOSE, IM>(sm, gsrc, gdst, logn_loc, logt, cc, itw, q, q2, cn, cns, cw, cws, wlog, reduce);
    else if (S == 2) inv_pass<2, CLOSE, IM>(sm, gsrc, gdst, logn_loc, logt, cc, itw, q, q2, cn, cns, cw, cws, wlog, reduce);
    else inv_pass<1, CLOSE, IM>(sm, gsrc, gdst, logn_loc, logt, cc, itw, q, q2, cn, cns, cw, cws, wlog, reduce);
}

// The closing constants of an inverse transform for the butterflies' mode: integers with their Shoup quotients,
// or (kInvF64) the constants and their quotients by q as doubles.
struct InvConst {
    u64 q, q2, cn, cns, cw, cws;
};
LB_D InvConst inv_constants(const int im, const u64 q, const u64 cn, const u64 cns, const u64 cw, const u64 cws)
{
    InvConst k;
    if (is_inv_f64(im)) {
        const double qd = (double)q;
        k.q = bits_of(qd);
        k.q2 = bits_of(1.0 / qd);
        k.cn = bits_of((double)cn);
        k.cns = bits_of((double)cn / qd);
        k.cw = bits_of((double)cw);
        k.cws = bits_of((double)cw / qd);
    } else {
        k.q = q; k.q2 = q << 1; k.cn = cn; k.cns = cns; k.cw = cw; k.cws = cws;
    }
    return k;
}

template <int LOGC>
__global__ void __launch_bounds__(kNttThreads, kNttMinBlocks) ntt_inv_kernel(const NttK a)
{
    extern __shared__ __align__(16) u64 sm[];
    constexpr int C = 1 << LOGC;
    const int row = blockIdx.x >> LOGC;
    const int grp = row / a.per_group, rr = row - grp * a.per_group;
    if (rr >= a.skip_lo && rr < a.skip_hi) return;
    const int tbl = rr < a.size_l ? rr + a.tbl_off : a.size_Q + (rr - a.size_l);
    const ModConst mc = a.mc[tbl];
    const u64 q = mc.q, q2 = q << 1;
    const int logN = a.logN, logn_loc = logN - LOGC, n_loc = 1 << logn_loc;
    const ulonglong2 *itw = a.tw + ((size_t)tbl << logN);
    const int go = grp / a.split, gi = grp - go * a.split;
    const u64 *src = a.src + (((size_t)go * a.src_outer + (size_t)gi * a.src_group_stride + rr + a.src_row_off) << logN);
    u64 *dst = a.dst + (((size_t)go * a.dst_outer + (size_t)gi * a.dst_group_stride + rr) << logN);
    u64 cn = mc.ninv, cns = mc.ninvs, cw = mc.iw1n, cws = mc.iw1ns;
    if (a.fold) {
        const u64 *f = a.fold + 4 * rr;
        cn = f[0]; cns = f[1]; cw = f[2]; cws = f[3];
    }
    unsigned c = 0;
    if constexpr (LOGC > 0) c = cg::this_cluster().block_rank();
    const unsigned cc = C + c;
    const int im = inverse_mode(q);
    const InvConst ic = inv_constants(im, q, cn, cns, cw, cws);
    F64Run run(q);
    int logt = 0;
    for (int p = 0; p < a.npass; ++p) {
        const int S = a.S[p];
        const u64 *gsrc = (p == 0) ? src + (size_t)c * n_loc : nullptr;
        const bool closing = (LOGC == 0 && p == a.npass - 1);
        u64 *gdst = closing ? dst : nullptr;
        const int wlog = p >= a.npass - a.nwide ? -1 : a.wlog;
        if (p > 0) {
            if (wlog < 0) __syncthreads();
            else __syncwarp();
        }
        const bool red = run.before(S);
        if (im == kInvF64) {
            if (closing) inv_pass_any<true, kInvF64>(S, sm, gsrc, gdst, logn_loc, logt, cc, itw, ic.q, ic.q2, ic.cn, ic.cns, ic.cw, ic.cws, wlog, red);
            else inv_pass_any<false, kInvF64>(S, sm, gsrc, gdst, logn_loc, logt, cc, itw, ic.q, ic.q2, ic.cn, ic.cns, ic.cw, ic.cws, wlog, red);
        } else if (im == kInvF64Tight) {
            if (closing) inv_pass_any<true, kInvF64Tight>(S, sm, gsrc, gdst, logn_loc, logt, cc, itw, ic.q, ic.q2, ic.cn, ic.cns, ic.cw, ic.cws, wlog, true);
            else inv_pass_any<false, kInvF64Tight>(S, sm, gsrc, gdst, logn_loc, logt, cc, itw, ic.q, ic.q2, ic.cn, ic.cns, ic.cw, ic.cws, wlog, true);
        } else {
            if (closing) inv_pass_any<true, kInvInt>(S, sm, gsrc, gdst, logn_loc, logt, cc, itw, q, q2, cn, cns, cw, cws, wlog, false);
            else inv_pass_any<false, kInvInt>(S, sm, gsrc, gdst, logn_loc, logt, cc, itw, q, q2, cn, cns, cw, cws, wlog, false);
        }
        logt += S;
    }
    if constexpr (LOGC > 0) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync(); // all local transforms of the cluster are in shared memory (and every peer is running)
        const u64 *remote[C];
#pragma unroll
        for (int k = 0; k < C; ++k) remote[k] = cluster.map_shared_rank(sm, k);
        const int share = n_loc >> LOGC;
        const bool red = run.before(LOGC);
        for (int jj = threadIdx.x; jj < share; jj += kNttThreads) {
            const int j = c * share + jj;
            u64 v[C];
#pragma unroll
            for (int kk = 0; kk < C; ++kk) v[kk] = remote[kk][sidx(j)];
            if (im == kInvF64) {
                if (red) {
#pragma unroll
                    for (int kk = 0; kk < C; ++kk) v[kk] = bits_of(f64_centre(f64_of(v[kk]), f64_of(ic.q), f64_of(ic.q2)));
                }
                inv_core<LOGC, true, kInvF64>(v, itw, C / 2, ic.q, ic.q2, ic.cn, ic.cns, ic.cw, ic.cws);
            } else if (im == kInvF64Tight) {
#pragma unroll
                for (int kk = 0; kk < C; ++kk) v[kk] = bits_of(f64_centre(f64_of(v[kk]), f64_of(ic.q), f64_of(ic.q2)));
                inv_core<LOGC, true, kInvF64Tight>(v, itw, C / 2, ic.q, ic.q2, ic.cn, ic.cns, ic.cw, ic.cws);
            } else {
                inv_core<LOGC, true, kInvInt>(v, itw, C / 2, q, q2, cn, cns, cw, cws);
            }
#pragma unroll
            for (int kk = 0; kk < C; ++kk) dst[j + kk * n_loc] = v[kk];
        }
        cluster.sync(); // shared memory stays alive until every peer has read it
    }
}

// ---- fixed schedule for rings of 8192 points and more ---------------------------------------------
// Every production ring degree leaves 8192 points per CTA, so the local transform is always the
// same thirteen stages.  With the stage numbers known at compile time the index arithmetic of a
// register group collapses to one shared-memory address plus immediate offsets, and the split
//   first pass : log2(C) + 1 stages on strided global loads (the cluster stages and the first
//                local one), scattered through distributed shared memory,
//   pass A     : local stages with spans 2048, 1024, 512 (CTA-wide),
//   passes B-D : spans 256..1 inside each warp's 1024-point chunk (warp barriers only),
// makes every register pass a radix-8 one: five passes instead of six.  The inverse mirrors it.
constexpr int kHalfLoc = 4096;                                // points per half of a CTA's part
constexpr int kHalfLocPad = kHalfLoc + (kHalfLoc >> 4);        // the same distance in padded shared memory

// offset of element i of a register group in padded shared memory; the group's elements are
// 2^LOGST apart and its base has zero bits where the element index goes
template <int LOGST>
LB_D constexpr int pad_off(const int i)
{
    return LOGST >= 4 ? (i << LOGST) + (i << (LOGST - 4)) : LOGST == 3 ? 8 * i + (i >> 1) : i;
}

LB_D uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
LB_D uint32_t map_to_cta(const uint32_t addr, const unsigned rank)
{
    uint32_t r;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
LB_D void st_cluster(const uint32_t addr, const u64 v) { asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory"); }
LB_D u64 ld_cluster(const uint32_t addr)
{
    u64 v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}

// group index of iteration `it` (0..3): shared out over the CTA, or inside the warp's own chunk
template <bool WIDE>
LB_D int fixed_group(const int it)
{
    return WIDE ? (int)threadIdx.x + 256 * it : (int)((threadIdx.x >> 5) << 7) + (int)(threadIdx.x & 31) + 32 * it;
}

// PLAIN: the input is the limb itself and the output is stored as it is, so none of the fused
// conversions is compiled in (sixteen inlined copies of the input ones make the instruction stream
// of this pass miss the cache).
template <int LOGC, int MODE, bool PLAIN>
LB_D void fwd_first_fixed(u64 *sm, const FwdIn &in, const unsigned c, const ulonglong2 *tw, const u64 bq, const u64 bq2)
{
    constexpr int F = LOGC + 1, R0 = 1 << F, COLS = kHalfLoc >> LOGC;
    const uint32_t sbase = smem_addr(sm);
    const u64 q = in.q; // the prime as an integer for the loaders; bq, bq2 are the butterflies' scalars
    for (int col = threadIdx.x; col < COLS; col += 256) {
        const int j = c * COLS + col;
        u64 v[R0];
        if (PLAIN) {
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = in.src[j + k * kHalfLoc];
        } else if (in.small) {
            // the small polynomial of an encryption as signed bytes, the same for every prime
            int ev[R0];
#pragma unroll
            for (int k = 0; k < R0; ++k) ev[k] = in.small[j + k * kHalfLoc];
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = ev[k] < 0 ? q - (u64)(-ev[k]) : (u64)ev[k];
        } else if (in.n == 0 && in.sub == nullptr) {
            // a plain row in the instantiation with fused parts (its epilogue is what this launch is after)
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = in.src[j + k * kHalfLoc];
        } else if (in.n == 1 && in.mat == nullptr) {
            // One source row reduced into this prime (every conversion of a chain with one special
            // prime).  The branches on the optional parts stay outside the loops so that all loads
            // of a part are in flight together; inside load_in each element would wait for its own.
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = in.src[j + k * kHalfLoc];
            if (in.es) {
                int ev[R0];
#pragma unroll
                for (int k = 0; k < R0; ++k) ev[k] = in.es[j + k * kHalfLoc];
#pragma unroll
                for (int k = 0; k < R0; ++k) {
                    const u64 x = add_mod(v[k], ev[k] < 0 ? in.es_p - (u64)(-ev[k]) : (u64)ev[k], in.es_p);
                    v[k] = sub_mod(barrett64(x, q, in.r1), ev[k] < 0 ? q - (u64)(-ev[k]) : (u64)ev[k], q);
                }
            } else {
#pragma unroll
                for (int k = 0; k < R0; ++k) v[k] = barrett64(v[k], q, in.r1);
            }
            if (in.sub) {
#pragma unroll
                for (int h = 0; h < R0; h += 8) {
                    u64 t[R0 < 8 ? R0 : 8];
#pragma unroll
                    for (int k = 0; k < (R0 < 8 ? R0 : 8); ++k) t[k] = in.sub[j + (h + k) * kHalfLoc];
#pragma unroll
                    for (int k = 0; k < (R0 < 8 ? R0 : 8); ++k) v[h + k] = sub_mod(v[h + k], shoup_mul(t[k], in.sub_w, in.sub_ws, q), q);
                }
            }
        } else if (in.mat != nullptr && in.sub == nullptr) {
            // base conversion of several source rows: four outputs share one walk over the rows, so four
            // loads are in flight per row instead of one
            constexpr int G = R0 < 4 ? R0 : 4;
#pragma unroll
            for (int h = 0; h < R0; h += G) {
                u128d acc[G];
#pragma unroll
                for (int k = 0; k < G; ++k) acc[k] = u128d{0, 0};
                for (int i = 0; i < in.n; ++i) {
                    const u64 m = __ldg(in.mat + i);
                    const u64 *row = in.src + ((size_t)i << in.logN) + j;
#pragma unroll
                    for (int k = 0; k < G; ++k) mac_wide(acc[k], row[(h + k) * kHalfLoc], m);
                }
#pragma unroll
                for (int k = 0; k < G; ++k) v[h + k] = barrett128(acc[k], q, in.r0, in.r1);
            }
        } else {
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = load_in(in, j + k * kHalfLoc);
        }
        if (is_f64_mode(MODE)) {
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = bits_of(f64_from_u52(v[k]));
        }
        if (MODE == kF64Tight) {
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = bits_of(f64_centre(f64_of(v[k]), f64_of(bq), f64_of(bq2)));
        }
        fwd_core<F, MODE>(v, tw, 1u, bq, bq2);
        const int s0 = sidx(j);
        if constexpr (LOGC == 0) {
            sm[s0] = v[0];
            sm[s0 + kHalfLocPad] = v[1];
        } else {
            // every CTA of the cluster must be running before its shared memory is written
            if (col == (int)threadIdx.x) cg::this_cluster().barrier_wait();
#pragma unroll
            for (int r = 0; r < (1 << LOGC); ++r) {
                const uint32_t ra = map_to_cta(sbase + 8u * s0, r);
                st_cluster(ra, v[2 * r]);
                st_cluster(ra + 8u * kHalfLocPad, v[2 * r + 1]);
            }
        }
    }
}

// three forward stages starting at span 2^LOGT
// q, q2: the butterflies' scalars; qi, r1: the prime as an integer and floor(2^64 / q) for the closing pass
template <int LOGT, int MODE, bool PLAIN = false>
LB_D void fwd_pass_fixed(u64 *sm, u64 *gdst, const unsigned cc, const ulonglong2 *tw, const u64 q, const u64 q2, const u64 qi,
                         const u64 r1, const FwdEpi &epi)
{
    constexpr int LOGST = LOGT - 2;
    constexpr bool WIDE = LOGT + 1 > 10, CLOSING = LOGST == 0;
    for (int it = 0; it < 4; ++it) {
        const int g = fixed_group<WIDE>(it);
        const int lo = g & ((1 << LOGST) - 1), hi = g >> LOGST;
        const int base = (hi << (LOGT + 1)) + lo;
        u64 *p = sm + sidx(base);
        u64 v[8];
        u64 t[8];
        if (CLOSING && !PLAIN && epi.aux) load_contig<8>(t, epi.aux + base); // in flight during the butterflies
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = p[pad_off<LOGST>(i)];
        if (MODE == kF64Tight) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q), f64_of(q2)));
        }
        fwd_core<3, MODE>(v, tw, (cc << (12 - LOGT)) + hi, q, q2);
        if constexpr (CLOSING) {
            if (is_f64_mode(MODE)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = f64_canon(f64_of(v[i]), f64_of(q), f64_of(q2));
            } else if (MODE == kIntLazy) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = barrett64(v[i], qi, r1);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = csub(csub(csub(v[i], q2 << 1), q2), q);
            }
            if (!PLAIN && epi.aux) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = shoup_mul(sub_mod(t[i], v[i], qi), epi.scal, epi.scal_s, qi);
                if (epi.add) {
                    load_contig<8>(t, epi.add + base);
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = add_mod(v[i], t[i], qi);
                }
            }
            if (!PLAIN && epi.mul0) {
                u64 w[8];
                load_contig<8>(t, epi.mul1 + base);
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = mul_mod(v[i], t[i], qi, epi.r0, epi.r1);
                store_contig<8>(w, gdst + epi.dst1_off + base);
                load_contig<8>(t, epi.mul0 + base);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = mul_mod(v[i], t[i], qi, epi.r0, epi.r1);
            }
            store_contig<8>(v, gdst + base);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) p[pad_off<LOGST>(i)] = v[i];
        }
    }
}

template <int LOGC, int MODE, bool PLAIN>
LB_D void fwd_body_fixed(u64 *sm, const FwdRow &fr, const unsigned c)
{
    const u64 q = bf_scalar_q<MODE>(fr.q), q2 = bf_scalar_q2<MODE>(fr.q);
    const unsigned cc = (1u << LOGC) + c;
    fwd_first_fixed<LOGC, MODE, PLAIN>(sm, fr.in, c, fr.tw, q, q2);
    if constexpr (LOGC > 0) cg::this_cluster().sync(); // all scatters into this CTA have landed
    else __syncthreads();
    fwd_pass_fixed<11, MODE>(sm, nullptr, cc, fr.tw, q, q2, fr.q, fr.in.r1, fr.epi);
    __syncthreads();
    fwd_pass_fixed<8, MODE>(sm, nullptr, cc, fr.tw, q, q2, fr.q, fr.in.r1, fr.epi);
    __syncwarp();
    fwd_pass_fixed<5, MODE>(sm, nullptr, cc, fr.tw, q, q2, fr.q, fr.in.r1, fr.epi);
    __syncwarp();
    fwd_pass_fixed<2, MODE, PLAIN>(sm, fr.dst + (size_t)c * (2 * kHalfLoc), cc, fr.tw, q, q2, fr.q, fr.in.r1, fr.epi);
}

template <int LOGC, bool PLAIN>
__global__ void __launch_bounds__(256, kNttMinBlocks) ntt_fwd_fixed_kernel(const NttK a)
{
    extern __shared__ __align__(16) u64 sm[];
    FwdRow fr;
    if (!fwd_row_setup(a, blockIdx.x >> LOGC, fr)) return;
    unsigned c = 0;
    if constexpr (LOGC > 0) {
        c = cg::this_cluster().block_rank();
        cg::this_cluster().barrier_arrive();
        const size_t off = (size_t)c * (2 * kHalfLoc);
        if (fr.epi.aux) fr.epi.aux += off;
        if (fr.epi.add) fr.epi.add += off;
        if (fr.epi.mul0) { fr.epi.mul0 += off; fr.epi.mul1 += off; }
    }
    switch (fr.mode) {
    case kF64: fwd_body_fixed<LOGC, kF64, PLAIN>(sm, fr, c); break;
    case kF64Tight: fwd_body_fixed<LOGC, kF64Tight, PLAIN>(sm, fr, c); break;
    case kIntLazy: fwd_body_fixed<LOGC, kIntLazy, PLAIN>(sm, fr, c); break;
    default: fwd_body_fixed<LOGC, kIntStrict, PLAIN>(sm, fr, c); break;
    }
}

// three inverse stages starting at distance 2^LOGT
template <int LOGT, int IM>
LB_D void inv_pass_fixed(u64 *sm, const u64 *gsrc, const unsigned cc, const ulonglong2 *itw, const u64 q, const u64 q2, const bool reduce)
{
    constexpr bool WIDE = LOGT + 3 > 10, OPENING = LOGT == 0;
    for (int it = 0; it < 4; ++it) {
        const int g = fixed_group<WIDE>(it);
        const int lo = g & ((1 << LOGT) - 1), hi = g >> LOGT;
        const int base = (hi << (LOGT + 3)) + lo;
        u64 *p = sm + sidx(base);
        u64 v[8];
        if constexpr (OPENING) {
            load_contig<8>(v, gsrc + base);
            if (is_inv_f64(IM)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = bits_of(f64_from_u52(v[i]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = p[pad_off<LOGT>(i)];
        }
        if ((IM == kInvF64 && reduce && !OPENING) || IM == kInvF64Tight) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q), f64_of(q2)));
        }
        inv_core<3, false, IM>(v, itw, (cc << (12 - LOGT)) + (hi << 2), q, q2, 0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) p[pad_off<LOGT>(i)] = v[i];
    }
}

template <int LOGC, int IM>
LB_D void inv_last_fixed(u64 *sm, u64 *dst, const unsigned c, const ulonglong2 *itw, const u64 q, const u64 q2, const u64 cn,
                         const u64 cns, const u64 cw, const u64 cws, const bool reduce)
{
    constexpr int F = LOGC + 1, R0 = 1 << F, COLS = kHalfLoc >> LOGC;
    const uint32_t sbase = smem_addr(sm);
    for (int col = threadIdx.x; col < COLS; col += 256) {
        const int j = c * COLS + col;
        const int s0 = sidx(j);
        u64 v[R0];
        if constexpr (LOGC == 0) {
            v[0] = sm[s0];
            v[1] = sm[s0 + kHalfLocPad];
        } else {
#pragma unroll
            for (int r = 0; r < (1 << LOGC); ++r) {
                const uint32_t ra = map_to_cta(sbase + 8u * s0, r);
                v[2 * r] = ld_cluster(ra);
                v[2 * r + 1] = ld_cluster(ra + 8u * kHalfLocPad);
            }
        }
        if ((IM == kInvF64 && reduce) || IM == kInvF64Tight) {
#pragma unroll
            for (int k = 0; k < R0; ++k) v[k] = bits_of(f64_centre(f64_of(v[k]), f64_of(q), f64_of(q2)));
        }
        inv_core<F, true, IM>(v, itw, 1u << LOGC, q, q2, cn, cns, cw, cws);
#pragma unroll
        for (int k = 0; k < R0; ++k) dst[j + k * kHalfLoc] = v[k];
    }
}

template <int LOGC, int IM>
LB_D void inv_body_fixed(u64 *sm, const u64 *src, u64 *dst, const unsigned c, const ulonglong2 *itw, const u64 qi, const u64 cn_i,
                         const u64 cns_i, const u64 cw_i, const u64 cws_i)
{
    const InvConst k = inv_constants(IM, qi, cn_i, cns_i, cw_i, cws_i);
    const u64 q = k.q, q2 = k.q2;
    const unsigned cc = (1u << LOGC) + c;
    F64Run run(qi);
    const bool r0 = run.before(3), r1 = run.before(3), r2 = run.before(3), r3 = run.before(3), r4 = run.before(LOGC + 1);
    (void)r0; // the opening pass reads canonical residues
    inv_pass_fixed<0, IM>(sm, src + (size_t)c * (2 * kHalfLoc), cc, itw, q, q2, false);
    __syncwarp();
    inv_pass_fixed<3, IM>(sm, nullptr, cc, itw, q, q2, r1);
    __syncwarp();
    inv_pass_fixed<6, IM>(sm, nullptr, cc, itw, q, q2, r2);
    __syncthreads();
    inv_pass_fixed<9, IM>(sm, nullptr, cc, itw, q, q2, r3);
    if constexpr (LOGC > 0) cg::this_cluster().sync(); // every local transform of the cluster is in shared memory
    else __syncthreads();
    inv_last_fixed<LOGC, IM>(sm, dst, c, itw, q, q2, k.cn, k.cns, k.cw, k.cws, r4);
    if constexpr (LOGC > 0) cg::this_cluster().sync(); // shared memory stays alive until every peer has read it
}

template <int LOGC>
__global__ void __launch_bounds__(256, kNttMinBlocks) ntt_inv_fixed_kernel(const NttK a)
{
    extern __shared__ __align__(16) u64 sm[];
    const int row = blockIdx.x >> LOGC;
    const int grp = row / a.per_group, rr = row - grp * a.per_group;
    if (rr >= a.skip_lo && rr < a.skip_hi) return;
    const int tbl = rr < a.size_l ? rr + a.tbl_off : a.size_Q + (rr - a.size_l);
    const ModConst mc = a.mc[tbl];
    const int logN = a.logN;
    const ulonglong2 *itw = a.tw + ((size_t)tbl << logN);
    const int go = grp / a.split, gi = grp - go * a.split;
    const u64 *src = a.src + (((size_t)go * a.src_outer + (size_t)gi * a.src_group_stride + rr + a.src_row_off) << logN);
    u64 *dst = a.dst + (((size_t)go * a.dst_outer + (size_t)gi * a.dst_group_stride + rr) << logN);
    u64 cn = mc.ninv, cns = mc.ninvs, cw = mc.iw1n, cws = mc.iw1ns;
    if (a.fold) {
        const u64 *f = a.fold + 4 * rr;
        cn = f[0]; cns = f[1]; cw = f[2]; cws = f[3];
    }
    unsigned c = 0;
    if constexpr (LOGC > 0) c = cg::this_cluster().block_rank();
    if (mc.q < kF64PrimeLimit) inv_body_fixed<LOGC, kInvF64>(sm, src, dst, c, itw, mc.q, cn, cns, cw, cws);
    else if (mc.q < kF64TightPrimeLimit) inv_body_fixed<LOGC, kInvF64Tight>(sm, src, dst, c, itw, mc.q, cn, cns, cw, cws);
    else inv_body_fixed<LOGC, kInvInt>(sm, src, dst, c, itw, mc.q, cn, cns, cw, cws);
}

// ---- launchers ------------------------------------------------------------------------

// Splits `stages` into as few register passes of at most R stages as possible, evenly.
static int split_even(int stages, int R, unsigned char *out)
{
    const int count = (stages + R - 1) / R;
    int n = 0;
    for (int i = 0; i < count; ++i) {
        const int s = (stages + (count - i) - 1) / (count - i);
        out[n++] = (unsigned char)s;
        stages -= s;
    }
    return n;
}

struct PassPlan {
    int npass, nwide, wlog;
    unsigned char S[8];
};

static PassPlan plan_passes(int logn_loc, bool forward)
{
    // The log2(warps) stages whose butterflies span more than one warp's chunk run as
    // CTA-wide passes; the rest stay inside a warp's contiguous chunk.  Of those, the pass
    // that touches global memory with contiguous per-thread data (forward: last, inverse:
    // first) takes the largest radix.  Short transforms keep every pass CTA-wide.
    const int R = kMaxRadixLog;
    int lw = 0;
    while ((32 << lw) < kNttThreads) ++lw;
    PassPlan pl;
    unsigned char wide[8], mid[8];
    int nw = 0, local = logn_loc;
    pl.wlog = -1;
    if (logn_loc - lw >= 8) {
        local = logn_loc - lw;
        pl.wlog = local;
        nw = split_even(lw, R, wide);
    }
    const int edge = local >= R ? R : local;
    const int nm = split_even(local - edge, R, mid);
    int n = 0;
    if (forward) {
        for (int i = 0; i < nw; ++i) pl.S[n++] = wide[i];
        for (int i = 0; i < nm; ++i) pl.S[n++] = mid[i];
        pl.S[n++] = (unsigned char)edge;
    } else {
        pl.S[n++] = (unsigned char)edge;
        for (int i = nm - 1; i >= 0; --i) pl.S[n++] = mid[i];
        for (int i = nw - 1; i >= 0; --i) pl.S[n++] = wide[i];
    }
    pl.npass = n;
    pl.nwide = nw;
    if (pl.wlog < 0) pl.nwide = n; // every pass CTA-wide
    return pl;
}

template <int LOGC>
static int launch(bool forward, bool fixed, const NttK &k, int rows, size_t smem, cudaStream_t stream, double bytes)
{
    auto kern = forward ? ntt_fwd_kernel<LOGC> : ntt_inv_kernel<LOGC>;
    int which = 0;
    const bool plain = k.bconv_n == 0 && k.digit_alpha == 0 && !k.presub && !k.esmall && !k.small && !k.aux && !k.mul2;
    if constexpr (LOGC <= 3) {
        if (fixed) {
            kern = !forward ? ntt_inv_fixed_kernel<LOGC> : plain ? ntt_fwd_fixed_kernel<LOGC, true> : ntt_fwd_fixed_kernel<LOGC, false>;
            which = plain ? 2 : 1;
        }
    }
    // function attributes belong to the device the kernel image is loaded on
    static bool configured[64][2][3] = {};
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    bool &done = configured[dev & 63][forward][which];
    if (!done) {
        // largest request any ring degree makes: 8192 points plus one pad word per 16
        LB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
        if (LOGC > 3) LB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        done = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows << LOGC);
    cfg.blockDim = dim3(kNttThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1 << LOGC;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch(!forward ? "ntt_inv_kernel" : plain ? "ntt_fwd_kernel(plain input)" : "ntt_fwd_kernel(fused input)", stream, bytes);
    LB_CUDA(cudaLaunchKernelEx(&cfg, kern, k));
    return LB_OK;
}

static int run(Context *ctx, const NttJob &job, bool forward, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    const int rows = job.n_groups * job.per_group;
    if (rows <= 0) return LB_OK;
    NttK k;
    k.src = job.src;
    k.dst = job.dst;
    k.tw = forward ? ctx->d_tw : ctx->d_itw;
    k.mc = ctx->d_mc;
    k.logN = hp.logN;
    k.per_group = job.per_group;
    k.size_l = job.size_l;
    k.size_Q = hp.size_Q;
    k.tbl_off = job.tbl_off;
    k.split = job.split > 0 ? job.split : 1;
    k.src_group_stride = job.src_group_stride >= 0 ? job.src_group_stride : job.per_group;
    k.dst_group_stride = job.dst_group_stride >= 0 ? job.dst_group_stride : job.per_group;
    k.aux_group_stride = job.aux_group_stride >= 0 ? job.aux_group_stride : job.per_group;
    k.add_group_stride = job.add_group_stride >= 0 ? job.add_group_stride : job.per_group;
    k.src_outer = job.src_outer >= 0 ? job.src_outer : k.split * k.src_group_stride;
    k.dst_outer = job.dst_outer >= 0 ? job.dst_outer : k.split * k.dst_group_stride;
    k.aux_outer = job.aux_outer >= 0 ? job.aux_outer : k.split * k.aux_group_stride;
    k.add_outer = job.add_outer >= 0 ? job.add_outer : k.split * k.add_group_stride;
    k.src_row_off = job.src_row_off;
    k.skip_lo = job.skip_lo;
    k.skip_hi = job.skip_hi;
    k.bconv_n = job.bconv_n;
    k.digit_alpha = job.digit_alpha;
    k.add_inner = job.add_inner;
    k.add1 = job.add1;
    k.add1_outer = job.add1_outer;
    k.bconv_mat = job.bconv_mat;
    k.mat_group_stride = job.mat_group_stride;
    k.mat_row_stride = job.mat_row_stride;
    k.aux = job.aux;
    k.scal = job.scal;
    k.scal_s = job.scal_s;
    k.add = job.add;
    k.fold = job.fold;
    k.mul2 = job.mul2;
    k.presub = job.presub;
    k.esmall = job.esmall;
    k.small = job.small;
    k.esmall_p = job.esmall_p;
    k.presub_scal = job.presub_scal;
    k.presub_scal_s = job.presub_scal_s;
    k.presub_outer = job.presub_outer >= 0 ? job.presub_outer : job.per_group;
    k.presub_inner = job.presub ? job.presub_inner : 0;
    const int logc = hp.logN > kMaxLocalLog ? hp.logN - kMaxLocalLog : 0;
    const int logn_loc = hp.logN - logc;
    const PassPlan pl = plan_passes(logn_loc, forward);
    k.npass = pl.npass;
    k.nwide = pl.nwide;
    k.wlog = pl.wlog;
    for (int i = 0; i < pl.npass; ++i) k.S[i] = pl.S[i];
    const size_t n_loc = size_t(1) << logn_loc;
    const size_t smem = (n_loc + (n_loc >> 4) + 2) * sizeof(u64);
    const bool fixed = logn_loc == 13; // rings of 8192 points and more take the fixed-schedule kernels
    // algorithmic bytes of this launch (diagnostics): rows written once; plain rows read once; fused loaders read the
    // group's source rows once per group, plus the rows the epilogue and the prologue fold in
    const double limb = 8.0 * (double)hp.N;
    const int live = job.per_group - (job.skip_hi > job.skip_lo ? job.skip_hi - job.skip_lo : 0);
    const double out_rows = (double)job.n_groups * live;
    double bytes = out_rows * limb;
    if (job.digit_alpha > 0) bytes += (double)job.n_groups * job.digit_alpha * limb;
    else if (job.bconv_n > 0) bytes += (double)job.n_groups * job.bconv_n * limb;
    else if (job.small) bytes += (double)job.n_groups * (double)hp.N; // one byte per coefficient and group
    else bytes += out_rows * limb;
    const double outer = (double)job.n_groups / k.split;
    if (job.aux) bytes += out_rows * limb;
    if (job.add) bytes += outer * (job.add_inner < k.split ? job.add_inner : k.split) * live * limb;
    if (job.add1) bytes += outer * live * limb;
    if (job.presub) bytes += outer * (k.presub_inner < k.split ? k.presub_inner : k.split) * live * limb;
    if (job.esmall) bytes += outer * (double)hp.N;
    if (job.mul2) bytes += out_rows * limb + 2.0 * job.per_group * limb; // a second output row per row, the two fixed rows once
    switch (logc) {
    case 0: return launch<0>(forward, fixed, k, rows, smem, stream, bytes);
    case 1: return launch<1>(forward, fixed, k, rows, smem, stream, bytes);
    case 2: return launch<2>(forward, fixed, k, rows, smem, stream, bytes);
    case 3: return launch<3>(forward, fixed, k, rows, smem, stream, bytes);
    case 4: return launch<4>(forward, fixed, k, rows, smem, stream, bytes);
    default: set_error("poly_modulus_degree above 65536 is not supported"); return LB_ERR_INVALID_ARG;
    }
}

int ntt_forward(Context *ctx, const NttJob &job, cudaStream_t stream) { return run(ctx, job, true, stream); }
int ntt_inverse(Context *ctx, const NttJob &job, cudaStream_t stream) { return run(ctx, job, false, stream); }

} // namespace lb
