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

constexpr int kTileThreads = 128;
constexpr int kTileMaxIn = 6, kTileMaxPairs = 8;

struct KrumTileArgs {
    const u64 *in[kTileMaxIn];
    u64 *out[kTileMaxPairs];
};

template <int NA, int NB>
__global__ void __launch_bounds__(kTileThreads, 3) krum_tile_kernel(const KrumTileArgs args, const ModConst *__restrict__ mc, const int logn,
                                                                    const long per_poly, const long chunk_stride, const int n_chunks)
{
    constexpr int NI = NA + NB, NP = NB ? NA * NB : NA * (NA - 1) / 2;
    // chunks a thread keeps in flight: as many as the accumulators of the shape leave registers for
    constexpr int kTileUnroll = NP <= 4 ? 3 : NP <= 6 ? 2 : 1;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < per_poly; e += (long)gridDim.x * blockDim.x) {
        const ModConst m = mc[(int)(e >> logn)];
        // 128-bit running sums; every 63 chunks they are reduced in place, which leaves room for
        // 63 more products of differences below 2^61
        u128d s0[NP], s1[NP], s2[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) s0[p] = s1[p] = s2[p] = u128d{0, 0};
        for (int c0 = 0; c0 < n_chunks; c0 += 63) {
            const int c1 = min(c0 + 63, n_chunks);
#pragma unroll(kTileUnroll)
            for (int c = c0; c < c1; ++c) {
                u64 v0[NI], v1[NI];
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const u64 *base = args.in[i] + c * chunk_stride + e;
                    v0[i] = __ldcs(base);
                    v1[i] = __ldcs(base + per_poly);
                }
                int p = 0;
#pragma unroll
                for (int i = 0; i < NA; ++i) {
#pragma unroll
                    for (int j = NB ? NA : i + 1; j < NI; ++j, ++p) {
                        // differences left in (0, 2q): 63 products below 2^122 and a residue fit 128 bits
                        const u64 x0 = v0[j] + m.q - v0[i], x1 = v1[j] + m.q - v1[i];
                        mac_wide(s0[p], x0, x0);
                        mac_wide(s1[p], x0, x1);
                        mac_wide(s2[p], x1, x1);
                    }
                }
            }
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                s0[p] = u128d{barrett128(s0[p], m.q, m.r0, m.r1), 0};
                s1[p] = u128d{barrett128(s1[p], m.q, m.r0, m.r1), 0};
                s2[p] = u128d{barrett128(s2[p], m.q, m.r0, m.r1), 0};
            }
        }
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            u64 *dst = args.out[p];
            dst[e] = s0[p].lo;
            dst[per_poly + e] = add_mod(s1[p].lo, s1[p].lo, m.q); // middle term is 2 x0 x1
            dst[2 * per_poly + e] = s2[p].lo;
        }
    }
}

template <int NA, int NB>
static void launch_tile(Context *ctx, const KrumTileArgs &args, int size_l, int n_chunks, long chunk_stride, cudaStream_t stream)
{
    const long per_poly = (long)size_l << ctx->hp.logN;
    const long blocks = (per_poly + kTileThreads - 1) / kTileThreads;
    count_launch("krum_tile_kernel", stream, 8.0 * per_poly * ((double)(NA + NB) * 2 * n_chunks + 3.0 * (NB ? NA * NB : NA * (NA - 1) / 2)));
    krum_tile_kernel<NA, NB><<<(unsigned)blocks, kTileThreads, 0, stream>>>(args, ctx->d_mc, ctx->hp.logN, per_poly, chunk_stride, n_chunks);
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
    switch (n_a * 8 + n_b) {
    case 2 * 8 + 0: launch_tile<2, 0>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 3 * 8 + 0: launch_tile<3, 0>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 4 * 8 + 0: launch_tile<4, 0>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 1: launch_tile<1, 1>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 2: launch_tile<1, 2>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 3: launch_tile<1, 3>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 1 * 8 + 4: launch_tile<1, 4>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 2 * 8 + 1: launch_tile<2, 1>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 2 * 8 + 2: launch_tile<2, 2>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    case 2 * 8 + 3: launch_tile<2, 3>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    default: launch_tile<2, 4>(ctx, args, size_l, n_chunks, chunk_stride, stream); break;
    }
    LB_CUDA(cudaGetLastError());
    return LB_OK;
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
    count_launch("mask_accumulate_kernel", stream);
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
