// CKKS encoder: canonical-embedding special FFT in double precision plus RNS decompose /
// compose (cahel-main/src/ckks.cu:104-209,292-465, fft.cu:54-344, rns_base.cu:121-156,325-459).
//
// Encoding is bit-sensitive: a coefficient is round()ed after the inverse FFT, so the
// butterfly expression shapes of the reference are kept exactly (x0 + x1, (x0 - x1) * w with
// the complex product's difference/sum contracted into one fused multiply-add each, scale/n
// multiplied in after the last stage).  Only the schedule differs: one kernel per batch of
// messages, a thread-block cluster per message, local stages in shared memory, the last
// log2(C) stages through distributed shared memory, and the rounding + residue step fused
// into the final store, instead of one global pass per stage plus a host round trip.
#include <cooperative_groups.h>

#include "context.h"

namespace cg = cooperative_groups;

namespace lb {

constexpr int kFftThreads = 256;
constexpr int kFftLocalLog = 12; // 4096 complex points (64 KiB + padding) per CTA

struct cplx {
    double x, y;
};

LB_D cplx c_add(cplx a, cplx b) { return {__dadd_rn(a.x, b.x), __dadd_rn(a.y, b.y)}; }
LB_D cplx c_sub(cplx a, cplx b) { return {__dsub_rn(a.x, b.x), __dsub_rn(a.y, b.y)}; }
// cuCmul as the device compiler contracts it in the reference's kernels: one rounded product feeding one fused
// multiply-add per part.  Which product of the imaginary part is the rounded one differs between the reference's two
// inverse-FFT kernels: the multi-stage kernel that runs the first eleven stages (cahel-main/src/fft.cu:194-268,
// SWITCH_POINT = 2048) rounds a.x * b.y, the per-stage kernel of the later stages (fft.cu:279-344) rounds a.y * b.x.
// Plaintexts at scale 2^50, whose largest coefficients keep two or three bits below the rounding point, pin this
// (reference-made fixtures n4096_s50, n8192_s50, n65536_a8).
constexpr int kRefIfftFirstKernelStages = 11;
LB_D cplx c_mul(cplx a, cplx b, const bool first_kernel_stage = false)
{
    cplx r;
    r.x = __fma_rn(a.x, b.x, -__dmul_rn(a.y, b.y));
    r.y = first_kernel_stage ? __fma_rn(a.y, b.x, __dmul_rn(a.x, b.y)) : __fma_rn(a.x, b.y, __dmul_rn(a.y, b.x));
    return r;
}

LB_D int fidx(int i) { return i + (i >> 4); }

struct EncK {
    const void *values; // [batch][value_stride] of dtype
    int dtype;          // 0 double real, 1 float real, 2 complex double
    long value_stride;  // elements between messages
    int n_values;
    u64 *pt;            // [batch][size_l][N]
    const double2 *roots;
    const uint32_t *group;
    const double2 *tw; // stage-ordered copy of the twiddles (see Context::d_ifft_tw), or nullptr
    const ModConst *mc;
    int logN, logn, size_l;
    double fix;
    double too_large;
    int *status;
    int npass;
    unsigned char S[8];
};

LB_D cplx load_value(const EncK &a, const long msg, const unsigned idx)
{
    cplx v = {0.0, 0.0};
    if (idx < (unsigned)a.n_values) {
        if (a.dtype == 0) v.x = reinterpret_cast<const double *>(a.values)[msg * a.value_stride + idx];
        else if (a.dtype == 1) v.x = (double)reinterpret_cast<const float *>(a.values)[msg * a.value_stride + idx];
        else {
            const double2 t = reinterpret_cast<const double2 *>(a.values)[msg * a.value_stride + idx];
            v.x = t.x;
            v.y = t.y;
        }
    }
    return v;
}

// twiddle of butterfly group k at stage u (pairs = 2^u): fft.cu:216-222
LB_D cplx ifft_twiddle(const EncK &a, const unsigned k, const int u)
{
    if (a.tw) { // one load instead of two dependent ones
        const unsigned n = 1u << a.logn;
        const double2 w = __ldg(a.tw + (n - (n >> u)) + k);
        return {w.x, w.y};
    }
    const int logRatio = a.logN + 1 - a.logn - 2;
    const unsigned M = 2u << a.logN;
    const unsigned rev = a.logn > 1 ? (__brev(k << u) >> (33 - a.logn)) : 0u;
    unsigned p = a.group[rev];
    p <<= (u + logRatio);
    p &= M - 1;
    const double2 w = a.roots[M - p];
    return {w.x, w.y};
}

// round, reduce into every prime, and store coefficient `pos` of the plaintext (rns_base.cu:121-156)
LB_D void emit_coeff(const EncK &a, u64 *pt_msg, const unsigned pos, const double value)
{
    const double r = round(value);
    const bool neg = signbit(r);
    const double av = fabs(r);
    // ceil(log2(av)) + 1 >= total bit count  <=>  av > 2^(total - 2)   (ckks.cu:185-191)
    if (av > a.too_large) atomicOr(a.status, 1);
    const long N = 1L << a.logN;
    if (av < 18446744073709551616.0) {
        const u64 m = (u64)av;
        for (int l = 0; l < a.size_l; ++l) {
            const ModConst mc = a.mc[l];
            u64 t = barrett64(m, mc.q, mc.r1);
            if (neg && t) t = mc.q - t;
            pt_msg[l * N + pos] = t;
        }
    } else {
        u128d z;
        z.lo = (u64)fmod(av, 18446744073709551616.0);
        z.hi = (u64)(av / 18446744073709551616.0);
        for (int l = 0; l < a.size_l; ++l) {
            const ModConst mc = a.mc[l];
            u64 t = barrett128(z, mc.q, mc.r0, mc.r1);
            if (neg && t) t = mc.q - t;
            pt_msg[l * N + pos] = t;
        }
    }
}

template <int S>
LB_D void ifft_pass(cplx *sm, const EncK &a, const long msg, const bool first, const bool last_global, u64 *pt_msg,
                    const int logn_loc, const int logt, const unsigned c, const int ratio_log)
{
    constexpr int R = 1 << S;
    const int groups = 1 << (logn_loc - S);
    for (int g = threadIdx.x; g < groups; g += kFftThreads) {
        const int lo = g & ((1 << logt) - 1), hi = g >> logt;
        const int base = (hi << (logt + S)) + lo;
        cplx v[R];
        if (first) { // logt == 0: the bit-reversal placement is folded into the load
            const unsigned gbase = (c << logn_loc) + base;
            // the type switch sits outside the element loop so that the R loads are in flight together
            unsigned idx[R];
#pragma unroll
            for (int i = 0; i < R; ++i) idx[i] = __brev(gbase + i) >> (32 - a.logn);
            if (a.dtype == 1) {
                const float *f = reinterpret_cast<const float *>(a.values) + msg * a.value_stride;
                float t[R];
#pragma unroll
                for (int i = 0; i < R; ++i) t[i] = idx[i] < (unsigned)a.n_values ? f[idx[i]] : 0.0f;
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = {(double)t[i], 0.0};
            } else if (a.dtype == 0) {
                const double *f = reinterpret_cast<const double *>(a.values) + msg * a.value_stride;
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = {idx[i] < (unsigned)a.n_values ? f[idx[i]] : 0.0, 0.0};
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i) v[i] = load_value(a, msg, idx[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) v[i] = sm[fidx(base + (i << logt))];
        }
#pragma unroll
        for (int s = 0; s < S; ++s) {
            const int u = logt + s;
            const int dist = 1 << s;
#pragma unroll
            for (int b = 0; b < (1 << (S - 1 - s)); ++b) {
                // global butterfly group index of this pair
                const unsigned k = ((c << logn_loc) >> (u + 1)) + (hi << (S - 1 - s)) + b;
                const cplx w = ifft_twiddle(a, k, u);
                const bool early = u < kRefIfftFirstKernelStages; // uniform over the CTA
#pragma unroll
                for (int i = 0; i < dist; ++i) {
                    cplx &x0 = v[b * 2 * dist + i], &x1 = v[b * 2 * dist + i + dist];
                    const cplx s0 = c_add(x0, x1), s1 = c_sub(x0, x1);
                    x0 = s0;
                    x1 = c_mul(s1, w, early);
                }
            }
        }
        if (last_global) { // single-CTA transform: this pass holds the final stage
            const unsigned n = 1u << a.logn;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const unsigned e = base + (i << logt);
                cplx z = v[i];
                if (a.fix != 0.0) {
                    z.x = __dmul_rn(z.x, a.fix);
                    z.y = __dmul_rn(z.y, a.fix);
                }
                emit_coeff(a, pt_msg, e << ratio_log, z.x);
                emit_coeff(a, pt_msg, (e + n) << ratio_log, z.y);
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; ++i) sm[fidx(base + (i << logt))] = v[i];
        }
    }
}

// fills the stage-ordered twiddle table from the root table: the same values, found once
__global__ void ifft_twiddle_table_kernel(EncK a, double2 *out)
{
    const unsigned n = 1u << a.logn;
    a.tw = nullptr;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i + 1 < n; i += gridDim.x * blockDim.x) {
        // stage u holds the entries [n - (n >> u), n - (n >> (u + 1)))
        int u = 0;
        while (i >= n - (n >> (u + 1))) ++u;
        const unsigned k = i - (n - (n >> u));
        const cplx w = ifft_twiddle(a, k, u);
        out[i] = make_double2(w.x, w.y);
    }
}

template <int LOGC>
__global__ void __launch_bounds__(kFftThreads) encode_ifft_kernel(const EncK a)
{
    extern __shared__ __align__(16) unsigned char smraw[];
    cplx *sm = reinterpret_cast<cplx *>(smraw);
    constexpr int C = 1 << LOGC;
    const long msg = blockIdx.x >> LOGC;
    const int logn_loc = a.logn - LOGC, n_loc = 1 << logn_loc;
    const int ratio_log = (a.logN - 1) - a.logn;
    u64 *pt_msg = a.pt + ((msg * a.size_l) << a.logN);
    unsigned c = 0;
    if constexpr (LOGC > 0) {
        c = cg::this_cluster().block_rank();
        cg::this_cluster().sync();
    }
    int logt = 0;
    for (int p = 0; p < a.npass; ++p) {
        const int S = a.S[p];
        const bool last_global = (LOGC == 0 && p == a.npass - 1);
        if (p > 0) __syncthreads();
        if (S == 3) ifft_pass<3>(sm, a, msg, p == 0, last_global, pt_msg, logn_loc, logt, c, ratio_log);
        else if (S == 2) ifft_pass<2>(sm, a, msg, p == 0, last_global, pt_msg, logn_loc, logt, c, ratio_log);
        else ifft_pass<1>(sm, a, msg, p == 0, last_global, pt_msg, logn_loc, logt, c, ratio_log);
        logt += S;
    }
    if constexpr (LOGC > 0) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const cplx *remote[C];
#pragma unroll
        for (int k = 0; k < C; ++k) remote[k] = cluster.map_shared_rank(sm, k);
        const int share = n_loc >> LOGC;
        const unsigned n = 1u << a.logn;
        for (int jj = threadIdx.x; jj < share; jj += kFftThreads) {
            const int j = c * share + jj;
            cplx v[C];
#pragma unroll
            for (int k = 0; k < C; ++k) v[k] = remote[k][fidx(j)];
#pragma unroll
            for (int s = 0; s < LOGC; ++s) {
                const int u = logn_loc + s;
                const int dist = 1 << s;
#pragma unroll
                for (int b = 0; b < (1 << (LOGC - 1 - s)); ++b) {
                    // element j + kk * n_loc with kk = b * 2 * dist + i: group index (j + kk n_loc) >> (u + 1) = b
                    const cplx w = ifft_twiddle(a, (unsigned)b, u);
#pragma unroll
                    for (int i = 0; i < dist; ++i) {
                        cplx &x0 = v[b * 2 * dist + i], &x1 = v[b * 2 * dist + i + dist];
                        const cplx s0 = c_add(x0, x1), s1 = c_sub(x0, x1);
                        x0 = s0;
                        x1 = c_mul(s1, w);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < C; ++k) {
                const unsigned e = j + k * n_loc;
                cplx z = v[k];
                if (a.fix != 0.0) {
                    z.x = __dmul_rn(z.x, a.fix);
                    z.y = __dmul_rn(z.y, a.fix);
                }
                emit_coeff(a, pt_msg, e << ratio_log, z.x);
                emit_coeff(a, pt_msg, (e + n) << ratio_log, z.y);
            }
        }
        cluster.sync();
    }
}

static int plan(int logn_loc, unsigned char *S)
{
    // first pass (contiguous, gathers the input) at radix 8 when possible, then radix 8 / 4
    int n = 0, rem = logn_loc;
    while (rem > 0) {
        int s = rem >= 3 ? 3 : rem;
        if (rem == 4) s = 2;
        S[n++] = (unsigned char)s;
        rem -= s;
    }
    return n;
}

template <int LOGC>
static int launch_encode(const EncK &k, int batch, size_t smem, cudaStream_t stream)
{
    auto kern = encode_ifft_kernel<LOGC>;
    static bool configured = false;
    if (!configured) {
        LB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)batch << LOGC);
    cfg.blockDim = dim3(kFftThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1 << LOGC;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch("encode_ifft_kernel", stream);
    LB_CUDA(cudaLaunchKernelEx(&cfg, kern, k));
    return LB_OK;
}

// values -> plaintexts [batch][size_l][N] in NTT form
int encode(Context *ctx, int size_l, const void *values, int dtype, long value_stride, int n_values, int sparse_slots, int batch,
           double scale, u64 *pt, int *d_status, int skip_ntt, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    int logn = 0;
    while ((1 << logn) < sparse_slots) ++logn;
    if ((1 << logn) != sparse_slots || sparse_slots < 2 || (u64)sparse_slots > hp.N / 2) {
        set_error("single value encoding is not available / slot count must be a power of two up to N/2");
        return LB_ERR_INVALID_ARG;
    }
    if (n_values > sparse_slots) { set_error("values_size is too large"); return LB_ERR_INVALID_ARG; }
    int total_bits = 0;
    for (int l = 0; l < size_l; ++l) total_bits += 64 - __builtin_clzll(hp.q[l]);
    // the reference bounds by the bit count of the product; the sum of prime bit counts is within size_l of it
    {
        long double prod = 1.0L;
        for (int l = 0; l < size_l; ++l) prod *= (long double)hp.q[l];
        int e = 0;
        frexpl(prod, &e);
        total_bits = e;
    }
    if (scale <= 0 || ((int)log2(scale) + 1 >= total_bits)) { set_error("scale out of bounds"); return LB_ERR_INVALID_ARG; }
    if (batch <= 0) return LB_OK;
    if ((u64)sparse_slots < hp.N / 2)
        LB_CUDA(cudaMemsetAsync(pt, 0, ((size_t)batch * size_l << hp.logN) * 8, stream));
    EncK k;
    k.values = values;
    k.dtype = dtype;
    k.value_stride = value_stride;
    k.n_values = n_values;
    k.pt = pt;
    k.roots = ctx->d_croots;
    k.group = ctx->d_rot_group;
    k.tw = nullptr;
    k.mc = ctx->d_mc;
    k.logN = hp.logN;
    k.logn = logn;
    if (!ctx->d_ifft_tw[logn]) {
        // one table per slot count, built once and kept with the context; the build is synchronous so that a
        // later encode on another stream never reads a table still being filled
        double2 *tbl = nullptr;
        LB_CUDA(cudaMalloc((void **)&tbl, sizeof(double2) << logn));
        ctx->owned.push_back(tbl);
        count_launch("ifft_twiddle_table_kernel", stream);
        ifft_twiddle_table_kernel<<<(unsigned)(((1u << logn) + 255) / 256), 256, 0, stream>>>(k, tbl);
        LB_CUDA(cudaGetLastError());
        LB_CUDA(cudaStreamSynchronize(stream));
        ctx->d_ifft_tw[logn] = tbl;
    }
    k.tw = ctx->d_ifft_tw[logn];
    k.size_l = size_l;
    k.fix = scale / (double)sparse_slots;
    k.too_large = ldexp(1.0, total_bits - 2);
    k.status = d_status;
    const int logc = logn > kFftLocalLog ? logn - kFftLocalLog : 0;
    const int logn_loc = logn - logc;
    k.npass = plan(logn_loc, k.S);
    const size_t n_loc = size_t(1) << logn_loc;
    const size_t smem = (n_loc + (n_loc >> 4) + 2) * sizeof(cplx);
    int rc;
    switch (logc) {
    case 0: rc = launch_encode<0>(k, batch, smem, stream); break;
    case 1: rc = launch_encode<1>(k, batch, smem, stream); break;
    case 2: rc = launch_encode<2>(k, batch, smem, stream); break;
    case 3: rc = launch_encode<3>(k, batch, smem, stream); break;
    default: set_error("slot count above 32768 is not supported"); return LB_ERR_INVALID_ARG;
    }
    if (rc) return rc;
    if (skip_ntt) return LB_OK; // coefficient form, for an encryption that folds the plaintext in
    NttJob j;
    j.src = pt;
    j.dst = pt;
    j.n_groups = batch;
    j.per_group = size_l;
    j.size_l = size_l;
    return ntt_forward(ctx, j, stream);
}

// ---- decode -----------------------------------------------------------------------------

constexpr int kMaxComposeLimbs = 32; // the constants travel as a kernel argument (17 KiB at 32 limbs, below the 32 KiB limit)

struct ComposeConst {
    u64 radix[kMaxComposeLimbs][kMaxComposeLimbs + 1]; // q_0 ... q_{r-1} as a multi-word integer
    u64 Q[kMaxComposeLimbs + 1], Qhalf[kMaxComposeLimbs + 1];
    u64 ginv[kMaxComposeLimbs], ginv_s[kMaxComposeLimbs];
    u64 radix_mod[kMaxComposeLimbs][kMaxComposeLimbs]; // (q_0...q_{s-1}) mod q_r
};

// Exact centred CRT composition by Garner's mixed radix, then one conversion to double.
// (The reference accumulates word by word in double, rns_base.cu:325-459; both are within
// an ulp of the true quotient, and decoding is compared by tolerance.)
__global__ void __launch_bounds__(256) compose_kernel(cplx *__restrict__ out, const u64 *__restrict__ coef,
                                                      const ModConst *__restrict__ mc, const ComposeConst cc, const int logN,
                                                      const int logn, const int size_l, const double inv_scale)
{
    const unsigned n = 1u << logn;
    const int ratio_log = (logN - 1) - logn;
    const int W = size_l + 1;
    coef += ((size_t)blockIdx.y * size_l) << logN;
    out += (size_t)blockIdx.y * n;
    for (unsigned id = blockIdx.x * blockDim.x + threadIdx.x; id < 2 * n; id += gridDim.x * blockDim.x) {
        u64 v[kMaxComposeLimbs];
        for (int r = 0; r < size_l; ++r) {
            const ModConst m = mc[r];
            const u64 t = coef[((size_t)r << logN) + ((size_t)id << ratio_log)];
            u64 acc = 0;
            for (int s = 0; s < r; ++s) acc = add_mod(acc, mul_mod(barrett64(v[s], m.q, m.r1), cc.radix_mod[r][s], m.q, m.r0, m.r1), m.q);
            v[r] = shoup_mul(sub_mod(t, acc, m.q), cc.ginv[r], cc.ginv_s[r], m.q);
        }
        u64 x[kMaxComposeLimbs + 1];
        for (int i = 0; i < W; ++i) x[i] = 0;
        for (int r = 0; r < size_l; ++r) {
            u64 carry = 0;
            for (int i = 0; i < W; ++i) {
                u128d t = mul_wide(cc.radix[r][i], v[r]);
                t.lo += x[i];
                t.hi += t.lo < x[i];
                t.lo += carry;
                t.hi += t.lo < carry;
                x[i] = t.lo;
                carry = t.hi;
            }
        }
        bool gt = false, decided = false;
        for (int i = W - 1; i >= 0 && !decided; --i)
            if (x[i] != cc.Qhalf[i]) { gt = x[i] > cc.Qhalf[i]; decided = true; }
        if (gt) { // x > floor(Q/2): represent x - Q
            u64 borrow = 0;
            for (int i = 0; i < W; ++i) {
                const u64 a = cc.Q[i], b = x[i];
                const u64 d = a - b - borrow;
                borrow = (a < b) || (a == b && borrow);
                x[i] = d;
            }
        }
        // only the non-zero words count: with many limbs 2^(64 i) leaves the range of a double long before the
        // words of a centred coefficient stop being zero, and 0 * inf would poison the sum
        double val = 0.0;
        for (int i = 0; i < W; ++i)
            if (x[i]) val += ldexp((double)x[i], 64 * i);
        if (gt) val = -val;
        val *= inv_scale;
        if (id < n) out[id].x = val;
        else out[id - n].y = val;
    }
}

// one forward stage over global memory (fft.cu:54-182): (x0, x1) <- (x0 + w x1, x0 - w x1)
__global__ void __launch_bounds__(256) fft_stage_kernel(cplx *__restrict__ a, const double2 *__restrict__ roots,
                                                        const uint32_t *__restrict__ group, const int logN, const int logn,
                                                        const int u)
{
    const unsigned half = 1u << (logn - 1);
    const int logRatio = logN + 1 - logn - 2;
    const unsigned M = 2u << logN;
    a += (size_t)blockIdx.y << logn;
    for (unsigned tid = blockIdx.x * blockDim.x + threadIdx.x; tid < half; tid += gridDim.x * blockDim.x) {
        const unsigned pairs = 1u << u;
        const unsigned k = tid >> u, j = tid & (pairs - 1), g = 2 * k * pairs + j;
        const unsigned rev = logn > 1 ? (__brev(k << u) >> (33 - logn)) : 0u;
        unsigned p = group[rev];
        p <<= (u + logRatio);
        p &= M - 1;
        const double2 w2 = roots[p];
        const cplx w = {w2.x, w2.y};
        const cplx x0 = a[g], x1 = c_mul(a[g + pairs], w);
        a[g] = c_add(x0, x1);
        a[g + pairs] = c_sub(x0, x1);
    }
}

__global__ void __launch_bounds__(256) bitrev_out_kernel(cplx *__restrict__ out, const cplx *__restrict__ in, const int logn)
{
    const unsigned n = 1u << logn;
    out += (size_t)blockIdx.y << logn;
    in += (size_t)blockIdx.y << logn;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[__brev(i) >> (32 - logn)] = in[i];
}

size_t decode_workspace_bytes(const Context *ctx, int size_l, int batch)
{
    return (((size_t)size_l << ctx->hp.logN) + ctx->hp.N) * 8 * batch + 256;
}

// plaintext [size_l][N] (NTT form) -> sparse_slots complex doubles on the device
int decode(Context *ctx, int size_l, int batch, const u64 *pt, double scale, int sparse_slots, double *out_complex, cudaStream_t stream)
{
    const HostParams &hp = ctx->hp;
    if (size_l > kMaxComposeLimbs) { set_error("decode supports at most 32 limbs"); return LB_ERR_INVALID_ARG; }
    int logn = 0;
    while ((1 << logn) < sparse_slots) ++logn;
    if ((1 << logn) != sparse_slots || sparse_slots < 2 || (u64)sparse_slots > hp.N / 2) {
        set_error("slot count must be a power of two between 2 and N/2");
        return LB_ERR_INVALID_ARG;
    }
    if (scale <= 0) { set_error("scale out of bounds"); return LB_ERR_INVALID_ARG; }
    int rc = ctx->ensure_workspace(decode_workspace_bytes(ctx, size_l, batch));
    if (rc) return rc;
    u64 *coef = reinterpret_cast<u64 *>(ctx->ws);
    cplx *buf = reinterpret_cast<cplx *>(coef + (((size_t)size_l * batch) << hp.logN));
    NttJob inv;
    inv.src = pt;
    inv.dst = coef;
    inv.n_groups = batch;
    inv.per_group = size_l;
    inv.size_l = size_l;
    if ((rc = ntt_inverse(ctx, inv, stream))) return rc;
    ComposeConst cc;
    memset(&cc, 0, sizeof(cc));
    const int W = size_l + 1;
    u64 Q[kMaxComposeLimbs + 1] = {1};
    for (int r = 0; r < size_l; ++r) {
        for (int i = 0; i < W; ++i) cc.radix[r][i] = Q[i];
        u64 carry = 0;
        for (int i = 0; i < W; ++i) {
            const u128 t = (u128)Q[i] * hp.q[r] + carry;
            Q[i] = (u64)t;
            carry = (u64)(t >> 64);
        }
        u64 radix = 1;
        for (int s = 0; s < r; ++s) {
            cc.radix_mod[r][s] = radix;
            radix = h_mulmod(radix, hp.q[s] % hp.q[r], hp.q[r]);
        }
        cc.ginv[r] = h_invmod(radix, hp.q[r]);
        cc.ginv_s[r] = h_shoup(cc.ginv[r], hp.q[r]);
    }
    for (int i = 0; i < W; ++i) {
        cc.Q[i] = Q[i];
        cc.Qhalf[i] = (Q[i] >> 1) | (i + 1 < W ? Q[i + 1] << 63 : 0);
    }
    const unsigned n = (unsigned)sparse_slots;
    count_launch("compose_kernel", stream);
    compose_kernel<<<dim3((2 * n + 255) / 256, batch), 256, 0, stream>>>(buf, coef, ctx->d_mc, cc, hp.logN, logn, size_l, 1.0 / scale);
    LB_CUDA(cudaGetLastError());
    for (int iter = 0; iter < logn; ++iter) {
        const int u = logn - iter - 1;
        count_launch("fft_stage_kernel", stream);
        fft_stage_kernel<<<dim3((n / 2 + 255) / 256, batch), 256, 0, stream>>>(buf, ctx->d_croots, ctx->d_rot_group, hp.logN, logn, u);
    }
    LB_CUDA(cudaGetLastError());
    count_launch("bitrev_out_kernel", stream);
    bitrev_out_kernel<<<dim3((n + 255) / 256, batch), 256, 0, stream>>>(reinterpret_cast<cplx *>(out_complex), buf, logn);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

} // namespace lb
