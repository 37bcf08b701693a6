// Element-wise RNS polynomial kernels: HBM-streaming integer work, two coefficients per
// thread through 16-byte loads, grids sized in multiples of the SM count.
// They replace the one-launch-per-polynomial kernels of cahel-main/src/polymath.cu:16-227
// (add/sub/negate/multiply), :531-600 (2x2 tensor and square), cahel-main/src/galois.cu:20-29
// (NTT-domain automorphism) and the per-chunk sub / square / add sequence of the Krum inner
// loop (lancelot-main-GPU/utils/byzantine_fl.py:221-223).
#include "context.h"

namespace lb {

constexpr int kPolyThreads = 256;

static inline int grid_for(const Context *ctx, long work_items, int per_block)
{
    long need = (work_items + per_block - 1) / per_block;
    long cap = (long)ctx->sm_count * 16;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// ---- add / sub / mul / neg --------------------------------------------------------------

template <int OP>
__global__ void __launch_bounds__(kPolyThreads) binary_kernel(const ulonglong2 *__restrict__ a, const ulonglong2 *__restrict__ b,
                                                              ulonglong2 *__restrict__ out, const ModConst *__restrict__ mc,
                                                              const int size_l, const int log_half_n, const long total)
{
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const int row = (int)(i >> log_half_n);
        const ModConst m = mc[row % size_l];
        const ulonglong2 x = a[i];
        ulonglong2 y = make_ulonglong2(0, 0), r;
        if (OP != OP_NEG && OP != OP_REDUCE) y = b[i];
        if (OP == OP_ADD) {
            r.x = add_mod(x.x, y.x, m.q);
            r.y = add_mod(x.y, y.y, m.q);
        } else if (OP == OP_SUB) {
            r.x = sub_mod(x.x, y.x, m.q);
            r.y = sub_mod(x.y, y.y, m.q);
        } else if (OP == OP_MUL) {
            r.x = mul_mod(x.x, y.x, m.q, m.r0, m.r1);
            r.y = mul_mod(x.y, y.y, m.q, m.r0, m.r1);
        } else if (OP == OP_REDUCE) {
            // any 64-bit word, e.g. a plain sum of residues, back to its canonical residue
            r.x = barrett128(u128d{x.x, 0}, m.q, m.r0, m.r1);
            r.y = barrett128(u128d{x.y, 0}, m.q, m.r0, m.r1);
        } else {
            r.x = x.x ? m.q - x.x : 0;
            r.y = x.y ? m.q - x.y : 0;
        }
        out[i] = r;
    }
}

int poly_binary(Context *ctx, int op, int size_l, long rows, const u64 *a, const u64 *b, u64 *out, cudaStream_t stream)
{
    if (rows <= 0) return LB_OK;
    const int log_half_n = ctx->hp.logN - 1;
    const long total = rows << log_half_n;
    const int grid = grid_for(ctx, total, kPolyThreads);
    const ulonglong2 *pa = reinterpret_cast<const ulonglong2 *>(a), *pb = reinterpret_cast<const ulonglong2 *>(b);
    ulonglong2 *po = reinterpret_cast<ulonglong2 *>(out);
    count_launch("binary_kernel", stream);
    switch (op) {
    case OP_ADD: binary_kernel<OP_ADD><<<grid, kPolyThreads, 0, stream>>>(pa, pb, po, ctx->d_mc, size_l, log_half_n, total); break;
    case OP_SUB: binary_kernel<OP_SUB><<<grid, kPolyThreads, 0, stream>>>(pa, pb, po, ctx->d_mc, size_l, log_half_n, total); break;
    case OP_MUL: binary_kernel<OP_MUL><<<grid, kPolyThreads, 0, stream>>>(pa, pb, po, ctx->d_mc, size_l, log_half_n, total); break;
    case OP_NEG: binary_kernel<OP_NEG><<<grid, kPolyThreads, 0, stream>>>(pa, pb, po, ctx->d_mc, size_l, log_half_n, total); break;
    case OP_REDUCE: binary_kernel<OP_REDUCE><<<grid, kPolyThreads, 0, stream>>>(pa, pb, po, ctx->d_mc, size_l, log_half_n, total); break;
    default: set_error("unknown element-wise operation"); return LB_ERR_INVALID_ARG;
    }
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- tensor product ---------------------------------------------------------------------

LB_D u64 tensor_mid(u64 a0, u64 b1, u64 a1, u64 b0, const ModConst &m)
{
    u128d acc = mul_wide(a0, b1);
    mac_wide(acc, a1, b0);
    return barrett128(acc, m.q, m.r0, m.r1);
}

__global__ void __launch_bounds__(kPolyThreads) tensor_kernel(const ulonglong2 *__restrict__ a, const ulonglong2 *__restrict__ b,
                                                              ulonglong2 *__restrict__ out, const ModConst *__restrict__ mc,
                                                              const int size_l, const int log_half_n, const long per_ct,
                                                              const long total)
{
    // per_ct = size_l * N / 2 vector elements per polynomial
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long ct = i / per_ct, e = i - ct * per_ct;
        const ModConst m = mc[(int)(e >> log_half_n)];
        const ulonglong2 a0 = a[ct * 2 * per_ct + e], a1 = a[ct * 2 * per_ct + per_ct + e];
        const ulonglong2 b0 = b[ct * 2 * per_ct + e], b1 = b[ct * 2 * per_ct + per_ct + e];
        ulonglong2 d0, d1, d2;
        d0.x = mul_mod(a0.x, b0.x, m.q, m.r0, m.r1);
        d0.y = mul_mod(a0.y, b0.y, m.q, m.r0, m.r1);
        d1.x = tensor_mid(a0.x, b1.x, a1.x, b0.x, m);
        d1.y = tensor_mid(a0.y, b1.y, a1.y, b0.y, m);
        d2.x = mul_mod(a1.x, b1.x, m.q, m.r0, m.r1);
        d2.y = mul_mod(a1.y, b1.y, m.q, m.r0, m.r1);
        out[ct * 3 * per_ct + e] = d0;
        out[ct * 3 * per_ct + per_ct + e] = d1;
        out[ct * 3 * per_ct + 2 * per_ct + e] = d2;
    }
}

int poly_tensor(Context *ctx, int size_l, int batch, const u64 *a, const u64 *b, u64 *out, cudaStream_t stream)
{
    if (batch <= 0) return LB_OK;
    const int log_half_n = ctx->hp.logN - 1;
    const long per_ct = (long)size_l << log_half_n;
    const long total = per_ct * batch;
    count_launch("tensor_kernel", stream);
    tensor_kernel<<<grid_for(ctx, total, kPolyThreads), kPolyThreads, 0, stream>>>(
        reinterpret_cast<const ulonglong2 *>(a), reinterpret_cast<const ulonglong2 *>(b), reinterpret_cast<ulonglong2 *>(out),
        ctx->d_mc, size_l, log_half_n, per_ct, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- Galois automorphism in NTT form ---------------------------------------------------

__global__ void __launch_bounds__(kPolyThreads) galois_kernel(const u64 *__restrict__ src, u64 *__restrict__ dst,
                                                              const uint32_t *__restrict__ perm, const int logN, const long total)
{
    const long n_mask = (1L << logN) - 1;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long row = i >> logN;
        dst[i] = src[(row << logN) + perm[i & n_mask]];
    }
}

// ciphertexts [batch][2][L][N]: dst = image of src under the automorphism, the first polynomial plus itself
__global__ void __launch_bounds__(kPolyThreads) galois_plus_c0_kernel(const u64 *__restrict__ src, u64 *__restrict__ dst,
                                                                      const uint32_t *__restrict__ perm, const ModConst *__restrict__ mc,
                                                                      const int logN, const int L, const long total)
{
    const long n_mask = (1L << logN) - 1;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long row = i >> logN;
        const int r = (int)(row % (2 * L));
        const u64 v = src[(row << logN) + perm[i & n_mask]];
        dst[i] = r < L ? add_mod(v, src[i], mc[r].q) : v;
    }
}

// out[g] = sum of the items in[idx] listed for group g (the reference's add_many over a chosen subset):
// items are n_rows limbs each, row r uses prime r % size_l; lists in CSR form on the device
__global__ void __launch_bounds__(kPolyThreads) sum_groups_kernel(const ulonglong2 *__restrict__ in, ulonglong2 *__restrict__ out,
                                                                  const int *__restrict__ offsets, const int *__restrict__ indices,
                                                                  const ModConst *__restrict__ mc, const int size_l, const int log_half_n,
                                                                  const long item)
{
    const int g = blockIdx.y;
    const int lo = offsets[g], hi = offsets[g + 1];
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < item; i += (long)gridDim.x * blockDim.x) {
        const u64 q = mc[(int)((i >> log_half_n) % size_l)].q;
        ulonglong2 r = make_ulonglong2(0, 0);
        for (int t = lo; t < hi; ++t) {
            const ulonglong2 v = in[(long)indices[t] * item + i];
            r.x = add_mod(r.x, v.x, q);
            r.y = add_mod(r.y, v.y, q);
        }
        out[(long)g * item + i] = r;
    }
}

int poly_sum_groups(Context *ctx, int size_l, long n_rows, int n_groups, const int *h_offsets, const int *h_indices, const u64 *in,
                    u64 *out, cudaStream_t stream)
{
    if (n_groups <= 0) return LB_OK;
    const int n_idx = h_offsets[n_groups];
    const size_t bytes = ((size_t)n_groups + 1 + n_idx) * sizeof(int);
    int rc = ctx->ensure_workspace(bytes);
    if (rc) return rc;
    int *d = reinterpret_cast<int *>(ctx->ws);
    LB_CUDA(cudaMemcpyAsync(d, h_offsets, ((size_t)n_groups + 1) * sizeof(int), cudaMemcpyHostToDevice, stream));
    if (n_idx) LB_CUDA(cudaMemcpyAsync(d + n_groups + 1, h_indices, (size_t)n_idx * sizeof(int), cudaMemcpyHostToDevice, stream));
    const long item = (n_rows << ctx->hp.logN) / 2;
    long gx = (item + kPolyThreads - 1) / kPolyThreads;
    if (gx > 4096) gx = 4096;
    count_launch("sum_groups_kernel", stream);
    sum_groups_kernel<<<dim3((unsigned)gx, (unsigned)n_groups), kPolyThreads, 0, stream>>>(
        reinterpret_cast<const ulonglong2 *>(in), reinterpret_cast<ulonglong2 *>(out), d, d + n_groups + 1, ctx->d_mc, size_l,
        ctx->hp.logN - 1, item);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

int poly_galois(Context *ctx, int elt_idx, long rows, const u64 *src, u64 *dst, cudaStream_t stream)
{
    if (elt_idx < 0 || elt_idx >= (int)ctx->hp.galois_elts.size()) {
        set_error("Galois key not present");
        return LB_ERR_LOGIC;
    }
    const long total = rows << ctx->hp.logN;
    count_launch("galois_kernel", stream);
    galois_kernel<<<grid_for(ctx, total, kPolyThreads), kPolyThreads, 0, stream>>>(
        src, dst, ctx->d_perm + ((size_t)elt_idx << ctx->hp.logN), ctx->hp.logN, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

int poly_galois_plus_c0(Context *ctx, int elt_idx, int L, int batch, const u64 *src, u64 *dst, cudaStream_t stream)
{
    if (elt_idx < 0 || elt_idx >= (int)ctx->hp.galois_elts.size()) {
        set_error("Galois key not present");
        return LB_ERR_LOGIC;
    }
    const long total = ((long)batch * 2 * L) << ctx->hp.logN;
    count_launch("galois_kernel", stream);
    galois_plus_c0_kernel<<<grid_for(ctx, total, kPolyThreads), kPolyThreads, 0, stream>>>(
        src, dst, ctx->d_perm + ((size_t)elt_idx << ctx->hp.logN), ctx->d_mc, ctx->hp.logN, L, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- Krum inner loop: acc += sum_c (b_c - a_c)^2 as a size-3 ciphertext ---------------------

constexpr int kKrumThreads = 128;

// One thread owns two coefficients of one limb and walks a slice of the chunks with 128-bit
// lazy accumulators (products of residues below 2^61 leave room for 64 terms between
// reductions).  The chunk axis is cut into gridDim.y slices so that a pair keeps every SM
// busy even though one polynomial only has L * N / 2 vector elements; slices > 1 write
// partial sums that krum_reduce_kernel adds.
__global__ void __launch_bounds__(kKrumThreads) krum_accumulate_kernel(const ulonglong2 *__restrict__ a, const ulonglong2 *__restrict__ b,
                                                                       ulonglong2 *__restrict__ out, const ModConst *__restrict__ mc,
                                                                       const int log_half_n, const long per_poly,
                                                                       const long stride_a, const long stride_b,
                                                                       const int n_chunks, const int accumulate)
{
    const int slices = gridDim.y, slice = blockIdx.y;
    const int c_lo = (int)(((long)n_chunks * slice) / slices), c_hi = (int)(((long)n_chunks * (slice + 1)) / slices);
    ulonglong2 *dst = out + (long)slice * 3 * per_poly;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < per_poly; e += (long)gridDim.x * blockDim.x) {
        const ModConst m = mc[(int)(e >> log_half_n)];
        u64 r0x = 0, r0y = 0, r1x = 0, r1y = 0, r2x = 0, r2y = 0;
        for (int c0 = c_lo; c0 < c_hi; c0 += 64) {
            const int c1 = min(c0 + 64, c_hi);
            u128d s0x = {0, 0}, s0y = {0, 0}, s1x = {0, 0}, s1y = {0, 0}, s2x = {0, 0}, s2y = {0, 0};
#pragma unroll 4
            for (int c = c0; c < c1; ++c) {
                const ulonglong2 a0 = __ldcs(a + c * stride_a + e), a1 = __ldcs(a + c * stride_a + per_poly + e);
                const ulonglong2 b0 = __ldcs(b + c * stride_b + e), b1 = __ldcs(b + c * stride_b + per_poly + e);
                const u64 x0 = sub_mod(b0.x, a0.x, m.q), y0 = sub_mod(b0.y, a0.y, m.q);
                const u64 x1 = sub_mod(b1.x, a1.x, m.q), y1 = sub_mod(b1.y, a1.y, m.q);
                mac_wide(s0x, x0, x0);
                mac_wide(s0y, y0, y0);
                mac_wide(s1x, x0, x1);
                mac_wide(s1y, y0, y1);
                mac_wide(s2x, x1, x1);
                mac_wide(s2y, y1, y1);
            }
            r0x = add_mod(r0x, barrett128(s0x, m.q, m.r0, m.r1), m.q);
            r0y = add_mod(r0y, barrett128(s0y, m.q, m.r0, m.r1), m.q);
            r1x = add_mod(r1x, barrett128(s1x, m.q, m.r0, m.r1), m.q);
            r1y = add_mod(r1y, barrett128(s1y, m.q, m.r0, m.r1), m.q);
            r2x = add_mod(r2x, barrett128(s2x, m.q, m.r0, m.r1), m.q);
            r2y = add_mod(r2y, barrett128(s2y, m.q, m.r0, m.r1), m.q);
        }
        // middle term is 2 x0 x1
        r1x = add_mod(r1x, r1x, m.q);
        r1y = add_mod(r1y, r1y, m.q);
        if (accumulate && slices == 1) {
            const ulonglong2 o0 = dst[e], o1 = dst[per_poly + e], o2 = dst[2 * per_poly + e];
            r0x = add_mod(r0x, o0.x, m.q); r0y = add_mod(r0y, o0.y, m.q);
            r1x = add_mod(r1x, o1.x, m.q); r1y = add_mod(r1y, o1.y, m.q);
            r2x = add_mod(r2x, o2.x, m.q); r2y = add_mod(r2y, o2.y, m.q);
        }
        dst[e] = make_ulonglong2(r0x, r0y);
        dst[per_poly + e] = make_ulonglong2(r1x, r1y);
        dst[2 * per_poly + e] = make_ulonglong2(r2x, r2y);
    }
}

// acc (+)= sum over slices of partial[slice]; total = 3 * per_poly vector elements
__global__ void __launch_bounds__(kPolyThreads) krum_reduce_kernel(const ulonglong2 *__restrict__ partial, ulonglong2 *__restrict__ acc,
                                                                   const ModConst *__restrict__ mc, const int log_half_n,
                                                                   const int size_l, const long total, const int slices,
                                                                   const int accumulate)
{
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const u64 q = mc[(int)((i >> log_half_n) % size_l)].q;
        ulonglong2 r = accumulate ? acc[i] : make_ulonglong2(0, 0);
        for (int s = 0; s < slices; ++s) {
            const ulonglong2 p = partial[(long)s * total + i];
            r.x = add_mod(r.x, p.x, q);
            r.y = add_mod(r.y, p.y, q);
        }
        acc[i] = r;
    }
}

int krum_accumulate(Context *ctx, int size_l, int n_chunks, const u64 *a, const u64 *b, long chunk_stride_a,
                    long chunk_stride_b, u64 *acc, int accumulate, cudaStream_t stream)
{
    const int log_half_n = ctx->hp.logN - 1;
    const long per_poly = (long)size_l << log_half_n;
    const long blocks = (per_poly + kKrumThreads - 1) / kKrumThreads;
    // enough slices for about eight resident blocks per SM, at least four chunks per slice
    long slices = ((long)ctx->sm_count * 8 + blocks - 1) / blocks;
    if (slices > n_chunks / 4) slices = n_chunks / 4;
    if (slices > 32) slices = 32;
    if (slices < 1) slices = 1;
    ulonglong2 *dst = reinterpret_cast<ulonglong2 *>(acc);
    if (slices > 1) {
        int rc = ctx->ensure_workspace((size_t)slices * 3 * per_poly * sizeof(ulonglong2));
        if (rc) return rc;
        dst = reinterpret_cast<ulonglong2 *>(ctx->ws);
    }
    count_launch("krum_accumulate_kernel", stream);
    krum_accumulate_kernel<<<dim3((unsigned)blocks, (unsigned)slices), kKrumThreads, 0, stream>>>(
        reinterpret_cast<const ulonglong2 *>(a), reinterpret_cast<const ulonglong2 *>(b), dst, ctx->d_mc, log_half_n, per_poly,
        chunk_stride_a / 2, chunk_stride_b / 2, n_chunks, accumulate);
    LB_CUDA(cudaGetLastError());
    if (slices > 1) {
        const long total = 3 * per_poly;
        count_launch("krum_reduce_kernel", stream);
        krum_reduce_kernel<<<grid_for(ctx, total, kPolyThreads), kPolyThreads, 0, stream>>>(
            dst, reinterpret_cast<ulonglong2 *>(acc), ctx->d_mc, log_half_n, size_l, total, (int)slices, accumulate);
        LB_CUDA(cudaGetLastError());
    }
    return LB_OK;
}

// ---- tiled Krum inner loop ------------------------------------------------------------------------
// A round needs the sum for every pair of clients, so the one-pair kernel reads each client once
// per partner.  A tile keeps the current chunk of up to six clients in registers and produces up
// to eight pair sums from it: a triangle (all pairs inside one set of NA clients, NB == 0) or a
// rectangle (every client of set A against every client of set B).  Pair p of a triangle is
// (0,1),(0,2),..,(1,2),..; of a rectangle a * NB + b.  HBM reads per pair drop from two clients to
// (NA + NB) / (NA * NB), 0.75 for the 2 x 4 rectangle.

constexpr int kTileMaxIn = 6, kTileMaxPairs = 8;

struct KrumTileArgs {
    const u64 *in[kTileMaxIn];
    u64 *out[kTileMaxPairs];
};

// Work split.  An item is one chunk of one unit; a unit is kTileSeg consecutive coefficients of one limb.  Items are
// ordered by unit, then chunk, and every item carries its limb's cost weight (the 128-bit integer path of a 60-bit
// prime is bound by its arithmetic, the FP64 path of a 40-bit one by its loads).  The grid is one CTA per SM, and CTA b takes the items whose
// running cost lies in [total b / G, total (b + 1) / G): every CTA gets the same amount of work whatever the number
// of units, and no wave of CTAs runs half empty.  A CTA's range cuts at most its first and its last unit; the sums
// of such a partial piece go to a scratch slot of the CTA (slot 0: the piece starts the CTA's range, slot 1: any
// later one) and a second, small kernel adds the pieces of each cut unit mod q.  Units that lie inside one CTA's
// range are stored directly.
//
// Data movement: one thread per coefficient, and every thread feeds itself.  Thread t copies word t of either
// polynomial of every client of the tile for the item a ring's length ahead with asynchronous 8-byte copies
// (cp.async, global to shared memory without passing registers; a warp's copies of one row are 256 contiguous
// bytes) into its own slots of a ring of shared-memory stages, and waits only for its own oldest copy group before it
// reads them.  No thread ever reads another thread's slot, so the loop has no barrier of any kind, nothing to spin on
// and nothing that could hang; with kTileRingBytes of copies in flight per SM the loads run at the rate of HBM while
// eight warps do the arithmetic.  (A ring filled by bulk copies of the tensor memory accelerator, cp.async.bulk with
// mbarriers, was built and measured first: one CTA got one item per microsecond out of it whatever the depth of the
// ring, 3.7 TB/s at one CTA per SM against 6.8 TB/s for this ring.)
//
// Arithmetic: the limb's prime picks the pipe.  60-bit primes keep differences in (0, 2q) and sum them in 128 bits
// (reduced in place every 63 chunks).  Primes below 2^41 (the 40-bit primes of Lancelot's chain) take the FP64 pipe.
// Every operand x < 2^41 is split ONCE per client into x = h 2^21 + l (l < 2^21, h < 2^20), each half planted in the
// mantissa of a double with exponent 2^52 (two integer instructions and no conversion); the difference of two such
// doubles is the exact signed difference of the halves, so a pair costs no integer work at all: four subtractions
// give d = dh 2^21 + dl with |dl| < 2^21, |dh| < 2^20, every product of two halves is below 2^42 in magnitude and
// exact, and a double accumulator takes 2048 of them before 2^53 comes into reach.  Per pair
//   sum (d0)^2      = LL0 + 2^22 LH0 + 2^42 HH0      (LH0 = sum of l0 h0, counted twice)
//   sum d0 d1       = LL1 + 2^21 X1  + 2^42 HH1      (X1 = sum of l0 h1 + h0 l1)
//   sum (d1)^2      = LL2 + 2^22 LH2 + 2^42 HH2
// are rebuilt as exact 128-bit integers at the end of a window and reduced mod q.  Ten fused multiply-adds and four
// subtractions per pair, chunk and coefficient replace twelve 32 x 32 -> 64 bit multiplications, their carry chains
// and the 64-bit subtractions.
constexpr int kTileSeg = 256;                        // coefficients per unit = threads per CTA
constexpr int kTileThreads = kTileSeg;
constexpr int kTileMaxStages = 16;
constexpr int kTileRingBytes = 160 * 1024; // shared memory the ring may take: the copies in flight per SM
constexpr int kTileMaxLimbs = 64;
constexpr u64 kTileF64PrimeLimit = u64(1) << 41;
constexpr int kTileF64Window = 2048;

// stages of the ring for a tile of n_in clients: what fits kTileRingBytes at full segments
constexpr int tile_stages(const int n_in)
{
    const int s = kTileRingBytes / (2 * n_in * kTileSeg * 8);
    return s < 2 ? 2 : s > kTileMaxStages ? kTileMaxStages : s;
}

struct TilePlan {
    long cost_base[kTileMaxLimbs + 1]; // running cost in front of limb l's items
    int weight[kTileMaxLimbs];
    int size_l, n_chunks, segs_per_limb, seg;
    long n_items;
};

LB_D uint32_t tile_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 8 bytes global -> shared without passing registers; completion is awaited per group of copies
LB_D void cp_async8(const uint32_t dst, const void *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory"); }
LB_D void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
LB_D void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// first item of CTA b of G: the item at which the running cost reaches total * b / G
LB_D long tile_boundary(const TilePlan &pl, const int b, const int G)
{
    if (b <= 0) return 0;
    if (b >= G) return pl.n_items;
    const long t = pl.cost_base[pl.size_l] / G * b + pl.cost_base[pl.size_l] % G * b / G;
    int l = 0;
    while (l + 1 < pl.size_l && pl.cost_base[l + 1] <= t) ++l;
    const long per_limb = (long)pl.segs_per_limb * pl.n_chunks;
    return per_limb * l + (t - pl.cost_base[l] + pl.weight[l] - 1) / pl.weight[l];
}

// the two polynomials' residues of one client as halves planted in doubles of exponent 2^52
struct TileOperand {
    double l0, h0, l1, h1;
};
LB_D double tile_planted(const unsigned v) { return __hiloint2double(0x43300000, (int)v); }
LB_D TileOperand tile_operand(const u64 x0, const u64 x1)
{
    TileOperand r;
    r.l0 = tile_planted((unsigned)x0 & 0x1FFFFFu);
    r.h0 = tile_planted((unsigned)(x0 >> 21));
    r.l1 = tile_planted((unsigned)x1 & 0x1FFFFFu);
    r.h1 = tile_planted((unsigned)(x1 >> 21));
    return r;
}
// (ll + mid 2^shift + hh 2^42) mod q for integer-valued doubles below 2^53 in magnitude; the total may be negative
LB_D u64 tile_fold(const double ll, const double mid, const int shift, const double hh, const ModConst &m)
{
    const __int128 t = (__int128)__double2ll_rn(ll) + (__int128)__double2ll_rn(mid) * ((__int128)1 << shift) +
                       (__int128)__double2ll_rn(hh) * ((__int128)1 << 42);
    const bool neg = t < 0;
    const unsigned __int128 a = neg ? (unsigned __int128)(-t) : (unsigned __int128)t;
    const u64 r = barrett128(u128d{(u64)a, (u64)(a >> 64)}, m.q, m.r0, m.r1);
    return neg && r ? m.q - r : r;
}

// stage layout: row (client i, polynomial t) at words [(2 i + t) * seg, +seg)
template <int NA, int NB>
__global__ void __launch_bounds__(kTileThreads, 1) krum_tile_kernel(const __grid_constant__ KrumTileArgs args, const __grid_constant__ TilePlan pl,
                                                                    const ModConst *__restrict__ mc, const int logn, const long per_poly,
                                                                    const long chunk_stride, u64 *__restrict__ scratch)
{
    constexpr int NI = NA + NB, NP = NB ? NA * NB : NA * (NA - 1) / 2, STAGES = tile_stages(NI);
    extern __shared__ __align__(128) u64 tile_sm[];
    const int seg = pl.seg, n_chunks = pl.n_chunks, segs = pl.segs_per_limb;
    const int G = gridDim.x, cta = blockIdx.x;
    const int t = threadIdx.x;
    if (t >= seg) return; // rings of fewer than kTileSeg coefficients; the kernel has no barrier
    const long lo = tile_boundary(pl, cta, G), hi = tile_boundary(pl, cta + 1, G);
    const unsigned row_bytes = (unsigned)(seg * sizeof(u64)), stage_bytes = 2 * NI * row_bytes;
    const uint32_t sm_t = tile_smem(tile_sm) + (uint32_t)t * 8u;
    auto unit_offset = [&](const long unit) { // first coefficient of the unit, plus this thread's
        const int limb = (int)(unit / segs);
        return ((long)limb << logn) + (unit - (long)limb * segs) * seg + t;
    };

    // ---- this thread's copies: the ring is filled up front; then one item is requested per item read ----
    long p_left = hi - lo, p_unit = lo / n_chunks;
    int p_c = (int)(lo - p_unit * n_chunks), p_s = 0;
    long p_off = p_c * chunk_stride + unit_offset(p_unit);
    auto produce = [&]() {
        if (p_left > 0) {
            const uint32_t dst = sm_t + (uint32_t)p_s * stage_bytes;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const u64 *src = args.in[i] + p_off;
                cp_async8(dst + (uint32_t)(2 * i) * row_bytes, src);
                cp_async8(dst + (uint32_t)(2 * i + 1) * row_bytes, src + per_poly);
            }
            --p_left;
            p_off += chunk_stride;
            if (++p_c == n_chunks) {
                p_c = 0;
                ++p_unit;
                if (p_left > 0) p_off = unit_offset(p_unit);
            }
            if (++p_s == STAGES) p_s = 0;
        }
        cp_async_commit(); // one group per call, empty at the tail, so the group count below stays fixed
    };
#pragma unroll 1
    for (int i = 0; i < STAGES - 1; ++i) produce();

    {
        int s = 0;
        // requests the item a ring's length ahead, waits for this thread's copies of the next item, returns its rows
        auto acquire = [&]() -> const u64 * {
            produce();
            cp_async_wait<STAGES - 1>();
            return tile_sm + (size_t)s * (2 * NI * seg) + t;
        };
        auto release = [&]() {
            if (++s == STAGES) s = 0;
        };

        long it = lo;
        long unit = lo / n_chunks;
        int c = (int)(lo - unit * n_chunks);
        while (it < hi) {
            // one piece: chunks [c, c_end) of this unit
            const int c_end = (int)min((long)n_chunks, (long)c + (hi - it));
            const int limb = (int)(unit / segs);
            const ModConst m = mc[limb];
            const long e = ((long)limb << logn) + (unit - (long)limb * segs) * seg + t;
            // where this piece's sums go: the whole unit is final; a cut piece goes to this CTA's slot and is added
            // up by krum_tile_combine_kernel
            const bool whole = c == 0 && c_end == n_chunks;
            u64 *const piece = scratch + ((size_t)cta * 2 + (it == lo ? 0 : 1)) * (NP * 3) * seg + t;
            auto emit = [&](const int p, u64 v0, u64 v1, u64 v2, const bool add) {
                u64 *const d = whole ? args.out[p] + e : piece + (size_t)(p * 3) * seg;
                const long st = whole ? per_poly : (long)seg;
                v1 = add_mod(v1, v1, m.q); // middle term is 2 x0 x1
                if (add) { // a later window of a piece of more than kTileF64Window chunks
                    v0 = add_mod(v0, d[0], m.q);
                    v1 = add_mod(v1, d[st], m.q);
                    v2 = add_mod(v2, d[2 * st], m.q);
                }
                d[0] = v0;
                d[st] = v1;
                d[2 * st] = v2;
            };
            if (m.q < kTileF64PrimeLimit) {
                for (int w0 = c; w0 < c_end; w0 += kTileF64Window) {
                    const int w1 = min(w0 + kTileF64Window, c_end);
                    double ll0[NP], lh0[NP], hh0[NP], ll1[NP], x1[NP], hh1[NP], ll2[NP], lh2[NP], hh2[NP];
#pragma unroll
                    for (int p = 0; p < NP; ++p) ll0[p] = lh0[p] = hh0[p] = ll1[p] = x1[p] = hh1[p] = ll2[p] = lh2[p] = hh2[p] = 0.0;
                    auto pair = [&](const int p, const TileOperand &a, const TileOperand &b) {
                        const double dl0 = __dsub_rn(b.l0, a.l0), dh0 = __dsub_rn(b.h0, a.h0);
                        const double dl1 = __dsub_rn(b.l1, a.l1), dh1 = __dsub_rn(b.h1, a.h1);
                        ll0[p] = __fma_rn(dl0, dl0, ll0[p]);
                        lh0[p] = __fma_rn(dl0, dh0, lh0[p]);
                        hh0[p] = __fma_rn(dh0, dh0, hh0[p]);
                        ll1[p] = __fma_rn(dl0, dl1, ll1[p]);
                        x1[p] = __fma_rn(dl0, dh1, x1[p]);
                        x1[p] = __fma_rn(dh0, dl1, x1[p]);
                        hh1[p] = __fma_rn(dh0, dh1, hh1[p]);
                        ll2[p] = __fma_rn(dl1, dl1, ll2[p]);
                        lh2[p] = __fma_rn(dl1, dh1, lh2[p]);
                        hh2[p] = __fma_rn(dh1, dh1, hh2[p]);
                    };
                    for (int cc = w0; cc < w1; ++cc) {
                        const u64 *row = acquire();
                        TileOperand a[NA];
#pragma unroll
                        for (int i = 0; i < NA; ++i) a[i] = tile_operand(row[(2 * i) * seg], row[(2 * i + 1) * seg]);
                        if (NB) {
#pragma unroll
                            for (int j = 0; j < NB; ++j) {
                                const TileOperand b = tile_operand(row[(2 * (NA + j)) * seg], row[(2 * (NA + j) + 1) * seg]);
#pragma unroll
                                for (int i = 0; i < NA; ++i) pair(i * NB + j, a[i], b);
                            }
                        } else {
                            int p = 0;
#pragma unroll
                            for (int i = 0; i < NA; ++i) {
#pragma unroll
                                for (int j = i + 1; j < NA; ++j, ++p) pair(p, a[i], a[j]);
                            }
                        }
                        release();
                    }
                    {
#pragma unroll
                        for (int p = 0; p < NP; ++p)
                            emit(p, tile_fold(ll0[p], lh0[p], 22, hh0[p], m), tile_fold(ll1[p], x1[p], 21, hh1[p], m),
                                 tile_fold(ll2[p], lh2[p], 22, hh2[p], m), w0 != c);
                    }
                }
            } else {
                // 128-bit running sums; every 63 chunks they are reduced in place, which leaves room for
                // 63 more products of differences below 2^61
                u128d s0[NP], s1[NP], s2[NP];
#pragma unroll
                for (int p = 0; p < NP; ++p) s0[p] = s1[p] = s2[p] = u128d{0, 0};
                for (int w0 = c; w0 < c_end; w0 += 63) {
                    const int w1 = min(w0 + 63, c_end);
                    for (int cc = w0; cc < w1; ++cc) {
                        const u64 *row = acquire();
                        int p = 0;
#pragma unroll
                        for (int i = 0; i < NA; ++i) {
                            const u64 a0 = row[(2 * i) * seg], a1 = row[(2 * i + 1) * seg];
#pragma unroll
                            for (int j = NB ? NA : i + 1; j < NI; ++j, ++p) {
                                // differences left in (0, 2q): 63 products below 2^122 and a residue fit 128 bits
                                const u64 d0 = row[(2 * j) * seg] + m.q - a0, d1 = row[(2 * j + 1) * seg] + m.q - a1;
                                mac_wide(s0[p], d0, d0);
                                mac_wide(s1[p], d0, d1);
                                mac_wide(s2[p], d1, d1);
                            }
                        }
                        release();
                    }
#pragma unroll
                    for (int p = 0; p < NP; ++p) {
                        s0[p] = u128d{barrett128(s0[p], m.q, m.r0, m.r1), 0};
                        s1[p] = u128d{barrett128(s1[p], m.q, m.r0, m.r1), 0};
                        s2[p] = u128d{barrett128(s2[p], m.q, m.r0, m.r1), 0};
                    }
                }
#pragma unroll
                for (int p = 0; p < NP; ++p) emit(p, s0[p].lo, s1[p].lo, s2[p].lo, false);
            }
            it += c_end - c;
            c = c_end;
            if (c == n_chunks) c = 0, ++unit;
        }
    }
}

// adds the pieces of every unit that more than one CTA of krum_tile_kernel worked on; one CTA per unit.  Thread 0 walks
// the CTAs that share the unit (a handful) and lists their scratch slots, every thread then adds its coefficient.
constexpr int kTileListed = 64, kTileMaxGrid = 1024;
__global__ void __launch_bounds__(kTileSeg) krum_tile_combine_kernel(const __grid_constant__ KrumTileArgs args, const __grid_constant__ TilePlan pl,
                                                                     const ModConst *__restrict__ mc, const int logn, const long per_poly,
                                                                     const u64 *__restrict__ scratch, const int G, const int n_pairs)
{
    __shared__ int listed[kTileListed];
    __shared__ int n_listed, next_cta; // next_cta < 0: nothing (left) to add
    __shared__ long bound[kTileMaxGrid + 1]; // first item of every CTA of krum_tile_kernel (the divisions, done side by side)
    const int seg = pl.seg, n_chunks = pl.n_chunks, segs = pl.segs_per_limb;
    const int t = (int)threadIdx.x < seg ? threadIdx.x : 0;
    const long unit = blockIdx.x;
    const int limb = (int)(unit / segs);
    const u64 q = mc[limb].q;
    const long e = ((long)limb << logn) + (unit - (long)limb * segs) * seg + t;
    const long first = unit * n_chunks, last = first + n_chunks;
    const int n_words = n_pairs * 3;
    for (int b = threadIdx.x; b <= G; b += blockDim.x) bound[b] = tile_boundary(pl, b, G);
    __syncthreads();
    if (threadIdx.x == 0) {
        next_cta = 0;
        if (n_chunks > 0) {
            // the CTA that holds the unit's first item: the last one that starts at or before it
            int lo = 0, hi = G - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (bound[mid] <= first) lo = mid;
                else hi = mid - 1;
            }
            next_cta = bound[lo + 1] >= last ? -2 : lo; // -2: one CTA had the whole unit and stored it
        }
    }
    u64 acc[kTileMaxPairs * 3];
#pragma unroll
    for (int w = 0; w < kTileMaxPairs * 3; ++w) acc[w] = 0;
    for (;;) {
        if (threadIdx.x == 0) {
            int n = 0, b = next_cta;
            if (n_chunks == 0) b = -1; // no chunks: the sums are zero
            while (b >= 0 && b < G && n < kTileListed) {
                const long blo = bound[b];
                if (blo >= last) {
                    b = -1;
                    break;
                }
                const long plo = max(blo, first), phi = min(bound[b + 1], last);
                if (plo < phi) listed[n++] = b * 2 + (plo == blo ? 0 : 1);
                ++b;
            }
            n_listed = n;
            next_cta = b >= G ? -1 : b;
        }
        __syncthreads();
        const int n = n_listed, more = next_cta;
        if (more == -2) return;
        for (int i = 0; i < n; ++i) {
            const u64 *src = scratch + (size_t)listed[i] * n_words * seg + t;
#pragma unroll
            for (int w = 0; w < kTileMaxPairs * 3; ++w)
                if (w < n_words) acc[w] = add_mod(acc[w], src[(size_t)w * seg], q);
        }
        __syncthreads();
        if (more < 0) break;
    }
    if ((int)threadIdx.x < seg) {
#pragma unroll
        for (int w = 0; w < kTileMaxPairs * 3; ++w)
            if (w < n_words) args.out[w / 3][(w % 3) * per_poly + e] = acc[w];
    }
}

template <int NA, int NB>
static int launch_tile(Context *ctx, const KrumTileArgs &args, int size_l, int n_chunks, long chunk_stride, cudaStream_t stream)
{
    constexpr int NP = NB ? NA * NB : NA * (NA - 1) / 2;
    const int logn = ctx->hp.logN;
    const long per_poly = (long)size_l << logn;
    if (size_l > kTileMaxLimbs) {
        set_error("a Krum tile takes at most 64 limbs");
        return LB_ERR_INVALID_ARG;
    }
    TilePlan pl = {};
    pl.seg = (1 << logn) < kTileSeg ? (1 << logn) : kTileSeg;
    pl.segs_per_limb = (1 << logn) / pl.seg;
    pl.size_l = size_l;
    pl.n_chunks = n_chunks;
    const long per_limb = (long)pl.segs_per_limb * n_chunks;
    pl.n_items = per_limb * size_l;
    for (int l = 0; l < size_l; ++l) {
        // measured on B200: an item of the FP64 path takes the time of its loads (2 units per client), one of the
        // integer path the time of its arithmetic (3 units per pair) where that is more
        const int loads = 2 * (NA + NB), sums = 3 * NP;
        pl.weight[l] = ctx->hp.q[l] < kTileF64PrimeLimit ? loads : (sums > loads ? sums : loads);
        pl.cost_base[l + 1] = pl.cost_base[l] + per_limb * pl.weight[l];
    }
    const size_t smem = (size_t)tile_stages(NA + NB) * 2 * (NA + NB) * pl.seg * sizeof(u64);
    static int ctas_per_sm[64] = {};
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    if (!ctas_per_sm[dev & 63]) {
        const size_t most = (size_t)tile_stages(NA + NB) * 2 * (NA + NB) * kTileSeg * sizeof(u64); // full segments
        LB_CUDA(cudaFuncSetAttribute(krum_tile_kernel<NA, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most));
        int occ = 0;
        LB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, krum_tile_kernel<NA, NB>, kTileThreads, most));
        ctas_per_sm[dev & 63] = occ > 0 ? occ : 1;
    }
    long G = (long)ctas_per_sm[dev & 63] * ctx->sm_count;
    if (G > kTileMaxGrid) G = kTileMaxGrid;
    if (G > pl.n_items) G = pl.n_items > 0 ? pl.n_items : 1;
    int rc = ctx->ensure_workspace((size_t)G * 2 * NP * 3 * pl.seg * sizeof(u64));
    if (rc) return rc;
    u64 *scratch = reinterpret_cast<u64 *>(ctx->ws);
    if (pl.n_items > 0) {
        count_launch("krum_tile_kernel", stream, 8.0 * per_poly * ((double)(NA + NB) * 2 * n_chunks + 3.0 * NP));
        krum_tile_kernel<NA, NB><<<(unsigned)G, kTileThreads, smem, stream>>>(args, pl, ctx->d_mc, logn, per_poly, chunk_stride, scratch);
        LB_CUDA(cudaGetLastError());
    }
    count_launch("krum_tile_combine_kernel", stream);
    krum_tile_combine_kernel<<<(unsigned)(size_l * pl.segs_per_limb), kTileSeg, 0, stream>>>(args, pl, ctx->d_mc, logn, per_poly, scratch, (int)G, NP);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

int krum_accumulate_tile(Context *ctx, int size_l, int n_chunks, int n_a, const u64 *const *a, int n_b, const u64 *const *b,
                         long chunk_stride, u64 *const *out, cudaStream_t stream)
{
    const int n_pairs = n_b ? n_a * n_b : n_a * (n_a - 1) / 2;
    const bool ok = n_b == 0 ? (n_a >= 2 && n_a <= 4) : (n_a >= 1 && n_a <= 2 && n_b >= 1 && n_b <= 4);
    if (!ok) {
        set_error("a Krum tile is a triangle of 2..4 clients or a rectangle of 1..2 by 1..4 clients");
        return LB_ERR_INVALID_ARG;
    }
    KrumTileArgs args = {};
    for (int i = 0; i < n_a; ++i) args.in[i] = a[i];
    for (int i = 0; i < n_b; ++i) args.in[n_a + i] = b[i];
    for (int p = 0; p < n_pairs; ++p) args.out[p] = out[p];
    int rc = LB_OK;
    switch (n_a * 8 + n_b) {
    case 2 * 8 + 0: rc = launch_tile<2, 0>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 3 * 8 + 0: rc = launch_tile<3, 0>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 4 * 8 + 0: rc = launch_tile<4, 0>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 1: rc = launch_tile<1, 1>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 2: rc = launch_tile<1, 2>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 3: rc = launch_tile<1, 3>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 4: rc = launch_tile<1, 4>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 2 * 8 + 1: rc = launch_tile<2, 1>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 2 * 8 + 2: rc = launch_tile<2, 2>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 2 * 8 + 3: rc = launch_tile<2, 3>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    default: rc = launch_tile<2, 4>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    }
    return rc;
}

// ---- mask multiplication: out[c] = sum_k ct_k[c] (x) mask_k as size-3 ciphertexts -------------
// (lancelot-main-GPU/utils/byzantine_fl.py:401-409: per chunk, multiply every client's ciphertext
// with that client's mask ciphertext and add the products)

constexpr int kMaxMaskClients = 64;

struct MaskArgs {
    const ulonglong2 *ct[kMaxMaskClients]; // client k, chunk c at ct[k] + c * chunk_stride
    int n_clients;
};

__global__ void __launch_bounds__(kKrumThreads) mask_accumulate_kernel(const MaskArgs args, const ulonglong2 *__restrict__ masks,
                                                                       ulonglong2 *__restrict__ out, const ModConst *__restrict__ mc,
                                                                       const int log_half_n, const long per_poly,
                                                                       const long chunk_stride)
{
    const long c = blockIdx.y;
    ulonglong2 *dst = out + c * 3 * per_poly;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < per_poly; e += (long)gridDim.x * blockDim.x) {
        const ModConst m = mc[(int)(e >> log_half_n)];
        u64 r0x = 0, r0y = 0, r1x = 0, r1y = 0, r2x = 0, r2y = 0;
        for (int k0 = 0; k0 < args.n_clients; k0 += 32) {
            const int k1 = min(k0 + 32, args.n_clients);
            u128d s0x = {0, 0}, s0y = {0, 0}, s1x = {0, 0}, s1y = {0, 0}, s2x = {0, 0}, s2y = {0, 0};
#pragma unroll 2
            for (int k = k0; k < k1; ++k) {
                const ulonglong2 *a = args.ct[k] + c * chunk_stride;
                const ulonglong2 *b = masks + (long)k * 2 * per_poly;
                const ulonglong2 a0 = __ldcs(a + e), a1 = __ldcs(a + per_poly + e);
                const ulonglong2 b0 = b[e], b1 = b[per_poly + e];
                mac_wide(s0x, a0.x, b0.x);
                mac_wide(s0y, a0.y, b0.y);
                mac_wide(s1x, a0.x, b1.x);
                mac_wide(s1x, a1.x, b0.x);
                mac_wide(s1y, a0.y, b1.y);
                mac_wide(s1y, a1.y, b0.y);
                mac_wide(s2x, a1.x, b1.x);
                mac_wide(s2y, a1.y, b1.y);
            }
            r0x = add_mod(r0x, barrett128(s0x, m.q, m.r0, m.r1), m.q);
            r0y = add_mod(r0y, barrett128(s0y, m.q, m.r0, m.r1), m.q);
            r1x = add_mod(r1x, barrett128(s1x, m.q, m.r0, m.r1), m.q);
            r1y = add_mod(r1y, barrett128(s1y, m.q, m.r0, m.r1), m.q);
            r2x = add_mod(r2x, barrett128(s2x, m.q, m.r0, m.r1), m.q);
            r2y = add_mod(r2y, barrett128(s2y, m.q, m.r0, m.r1), m.q);
        }
        dst[e] = make_ulonglong2(r0x, r0y);
        dst[per_poly + e] = make_ulonglong2(r1x, r1y);
        dst[2 * per_poly + e] = make_ulonglong2(r2x, r2y);
    }
}

int mask_accumulate(Context *ctx, int size_l, int n_clients, int n_chunks, const u64 *const *client_cts, long chunk_stride,
                    const u64 *masks, u64 *out, cudaStream_t stream)
{
    if (n_clients < 1 || n_clients > kMaxMaskClients) { set_error("mask multiplication supports 1 to 64 clients per call"); return LB_ERR_INVALID_ARG; }
    if (n_chunks <= 0) return LB_OK;
    MaskArgs args;
    args.n_clients = n_clients;
    for (int k = 0; k < n_clients; ++k) args.ct[k] = reinterpret_cast<const ulonglong2 *>(client_cts[k]);
    const int log_half_n = ctx->hp.logN - 1;
    const long per_poly = (long)size_l << log_half_n;
    long blocks = (per_poly + kKrumThreads - 1) / kKrumThreads;
    // every client's ciphertext read once, one size-3 sum per chunk written
    count_launch("mask_accumulate_kernel", stream, 8.0 * (size_l << ctx->hp.logN) * n_chunks * (2.0 * n_clients + 3.0));
    mask_accumulate_kernel<<<dim3((unsigned)blocks, (unsigned)n_chunks), kKrumThreads, 0, stream>>>(
        args, reinterpret_cast<const ulonglong2 *>(masks), reinterpret_cast<ulonglong2 *>(out), ctx->d_mc, log_half_n, per_poly,
        chunk_stride / 2);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

// ---- level drop and decryption ---------------------------------------------------------

int poly_drop_last(Context *ctx, int size_l, int n_polys, const u64 *in, u64 *out, cudaStream_t stream)
{
    const size_t N = ctx->hp.N;
    LB_CUDA(cudaMemcpy2DAsync(out, (size_t)(size_l - 1) * N * 8, in, (size_t)size_l * N * 8, (size_t)(size_l - 1) * N * 8,
                              n_polys, cudaMemcpyDeviceToDevice, stream));
    return LB_OK;
}

// cahel-main/src/secretkey.cu:594-631 without the noise-flooding term
__global__ void __launch_bounds__(kPolyThreads) decrypt_kernel(const u64 *__restrict__ ct, const u64 *__restrict__ sk,
                                                               u64 *__restrict__ pt, const ModConst *__restrict__ mc,
                                                               const int logN, const int n_polys, const long per_poly, const long total)
{
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
        const long b = idx / per_poly, i = idx - b * per_poly;
        const ModConst m = mc[(int)(i >> logN)];
        const u64 *c = ct + b * n_polys * per_poly;
        const u64 s = sk[i];
        u64 sp = s, r = c[i];
        for (int p = 1; p < n_polys; ++p) {
            r = add_mod(r, mul_mod(c[p * per_poly + i], sp, m.q, m.r0, m.r1), m.q);
            sp = mul_mod(sp, s, m.q, m.r0, m.r1);
        }
        pt[idx] = r;
    }
}

int poly_decrypt(Context *ctx, int size_l, int n_polys, int batch, const u64 *ct, const u64 *sk, u64 *pt, cudaStream_t stream)
{
    const long per_poly = (long)size_l << ctx->hp.logN;
    const long total = per_poly * batch;
    count_launch("decrypt_kernel", stream);
    decrypt_kernel<<<grid_for(ctx, total, kPolyThreads), kPolyThreads, 0, stream>>>(ct, sk, pt, ctx->d_mc, ctx->hp.logN, n_polys,
                                                                                    per_poly, total);
    LB_CUDA(cudaGetLastError());
    return LB_OK;
}

} // namespace lb
