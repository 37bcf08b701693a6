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

// Data movement: a CTA owns kTileThreads consecutive coefficients of one limb.  Per chunk it needs one 1 KiB
// segment of either polynomial of every client of the tile; an elected thread fetches them with bulk asynchronous
// copies (cp.async.bulk, the 1-D form of the tensor memory accelerator; this GPU's own memory, no multicast) into a
// ring of kTileStages shared-memory stages, each guarded by an mbarrier that counts the bytes.  Nothing of this sits
// in registers, so three stages of up to 12 KiB per CTA are in flight ahead of the arithmetic at three CTAs per SM,
// which is what the HBM latency asks for; the threads read their operands from shared memory when they need them.
//
// Arithmetic: the limb's prime picks the pipe.  60-bit primes keep differences in (0, 2q) and sum them in 128 bits
// (reduced in place every 63 chunks).  Primes below 2^41 (the 40-bit primes of Lancelot's chain) take the FP64
// pipe: a difference d = b - a of two residues (|d| < 2^41) is split into d = h 2^21 + l with 0 <= l < 2^21 and
// |h| <= 2^20, both exact as doubles; every product of two halves is below 2^42 in magnitude and exact, and a double
// accumulator takes 2048 of them before 2^53 comes into reach.  Per pair
//   sum (d0)^2      = LL0 + 2^22 LH0 + 2^42 HH0      (LH0 = sum of l0 h0, counted twice)
//   sum d0 d1       = LL1 + 2^21 X1  + 2^42 HH1      (X1 = sum of l0 h1 + h0 l1)
//   sum (d1)^2      = LL2 + 2^22 LH2 + 2^42 HH2
// are rebuilt as exact 128-bit integers at the end of a window and reduced mod q.  Ten fused multiply-adds per
// pair, chunk and coefficient replace twelve 32 x 32 -> 64 bit multiplications and their carry chains.
constexpr u64 kTileF64PrimeLimit = u64(1) << 41;
constexpr int kTileF64Window = 2048;
constexpr int kTileStages = 4;
constexpr unsigned kTileSpinLimit = 1u << 24; // polls of an mbarrier before the kernel gives up and raises status bit 1

LB_D uint32_t tile_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
LB_D void mbar_init(const uint32_t bar, const unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
LB_D void mbar_expect_tx(const uint32_t bar, const unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
LB_D bool mbar_try_wait(const uint32_t bar, const unsigned parity)
{
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// global -> this CTA's shared memory, completion counted in bytes on the mbarrier; both addresses 16-byte aligned,
// size a multiple of 16
LB_D void bulk_load(const uint32_t dst, const void *src, const unsigned bytes, const uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

struct TileHalves {
    double l, h;
};
// a signed difference |d| < 2^41 as d = h 2^21 + l with 0 <= l < 2^21
LB_D TileHalves tile_split(const long long d)
{
    TileHalves r;
    r.l = __dadd_rn(__hiloint2double(0x43300000, (int)((unsigned)d & 0x1FFFFFu)), -4503599627370496.0);
    // h in [-2^20, 2^20): biased by 2^20 into an unsigned word, the bias taken off again as a double
    r.h = __dadd_rn(__hiloint2double(0x43300000, (int)((unsigned)(d >> 21) + 0x100000u)), -(4503599627370496.0 + 1048576.0));
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
__global__ void __launch_bounds__(kTileThreads, (NA + NB > 4 ? 2 : 3)) krum_tile_kernel(const KrumTileArgs args, const ModConst *__restrict__ mc, const int logn,
                                                                    const long per_poly, const long chunk_stride, const int n_chunks,
                                                                    int *__restrict__ status)
{
    constexpr int NI = NA + NB, NP = NB ? NA * NB : NA * (NA - 1) / 2;
    extern __shared__ __align__(128) u64 tile_sm[];
    __shared__ __align__(8) unsigned long long bars[kTileStages];
    const int seg = min(kTileThreads, 1 << logn);              // coefficients per CTA
    const int blocks_per_limb = (1 << logn) / seg;
    const int limb = blockIdx.x / blocks_per_limb;
    const long e0 = ((long)limb << logn) + (long)(blockIdx.x - limb * blocks_per_limb) * seg; // first coefficient of this CTA
    const ModConst m = mc[limb];
    const unsigned stage_bytes = (unsigned)(2 * NI * seg * sizeof(u64));
    const uint32_t sm_base = tile_smem(tile_sm), bar_base = tile_smem(bars);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < kTileStages; ++s) mbar_init(bar_base + 8u * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](const int c) { // thread 0: fetch chunk c into stage c % kTileStages
        const int s = c % kTileStages;
        const uint32_t bar = bar_base + 8u * s, dst = sm_base + (uint32_t)s * stage_bytes;
        mbar_expect_tx(bar, stage_bytes);
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const u64 *src = args.in[i] + c * chunk_stride + e0;
            bulk_load(dst + (uint32_t)((2 * i) * seg * 8), src, (unsigned)(seg * 8), bar);
            bulk_load(dst + (uint32_t)((2 * i + 1) * seg * 8), src + per_poly, (unsigned)(seg * 8), bar);
        }
    };
    if (threadIdx.x == 0) {
        for (int c = 0; c < kTileStages && c < n_chunks; ++c) issue(c);
    }
    const bool active = (int)threadIdx.x < seg;
    const int t = active ? threadIdx.x : 0;
    const bool f64 = m.q < kTileF64PrimeLimit;
    bool failed = false;

    // one chunk: waits for its stage, hands the operands of pair (i, j) to `pair`, releases the stage
    auto chunk = [&](const int c, auto &&pair) {
        const int s = c % kTileStages;
        const uint32_t bar = bar_base + 8u * s;
        const unsigned parity = (unsigned)(c / kTileStages) & 1u;
        unsigned polls = 0;
        bool gave_up = false;
        while (!mbar_try_wait(bar, parity)) {
            if (++polls > kTileSpinLimit) { // a copy that never lands: give up, say so, leave without touching the data
                gave_up = true;
                break;
            }
        }
        failed = __syncthreads_or(gave_up); // the whole CTA goes on or leaves together
        if (!failed) {
            const u64 *row = tile_sm + (size_t)s * (2 * NI * seg) + t;
            int p = 0;
#pragma unroll
            for (int i = 0; i < NA; ++i) {
#pragma unroll
                for (int j = NB ? NA : i + 1; j < NI; ++j, ++p)
                    pair(p, row[(2 * i) * seg], row[(2 * i + 1) * seg], row[(2 * j) * seg], row[(2 * j + 1) * seg]);
            }
        }
        __syncthreads(); // every thread has read the stage (or given up) before it is refilled
        if (threadIdx.x == 0 && !failed && c + kTileStages < n_chunks) issue(c + kTileStages);
    };

    const long e = e0 + t;
    if (f64) {
        u64 r0[NP], r1[NP], r2[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) r0[p] = r1[p] = r2[p] = 0;
        for (int c0 = 0; c0 < n_chunks && !failed; c0 += kTileF64Window) {
            const int c1 = min(c0 + kTileF64Window, n_chunks);
            double ll0[NP], lh0[NP], hh0[NP], ll1[NP], x1[NP], hh1[NP], ll2[NP], lh2[NP], hh2[NP];
#pragma unroll
            for (int p = 0; p < NP; ++p) ll0[p] = lh0[p] = hh0[p] = ll1[p] = x1[p] = hh1[p] = ll2[p] = lh2[p] = hh2[p] = 0.0;
            for (int c = c0; c < c1 && !failed; ++c) {
                chunk(c, [&](const int p, const u64 a0, const u64 a1, const u64 b0, const u64 b1) {
                    const TileHalves d0 = tile_split((long long)(b0 - a0)), d1 = tile_split((long long)(b1 - a1));
                    ll0[p] = __fma_rn(d0.l, d0.l, ll0[p]);
                    lh0[p] = __fma_rn(d0.l, d0.h, lh0[p]);
                    hh0[p] = __fma_rn(d0.h, d0.h, hh0[p]);
                    ll1[p] = __fma_rn(d0.l, d1.l, ll1[p]);
                    x1[p] = __fma_rn(d0.l, d1.h, x1[p]);
                    x1[p] = __fma_rn(d0.h, d1.l, x1[p]);
                    hh1[p] = __fma_rn(d0.h, d1.h, hh1[p]);
                    ll2[p] = __fma_rn(d1.l, d1.l, ll2[p]);
                    lh2[p] = __fma_rn(d1.l, d1.h, lh2[p]);
                    hh2[p] = __fma_rn(d1.h, d1.h, hh2[p]);
                });
            }
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                r0[p] = add_mod(r0[p], tile_fold(ll0[p], lh0[p], 22, hh0[p], m), m.q);
                r1[p] = add_mod(r1[p], tile_fold(ll1[p], x1[p], 21, hh1[p], m), m.q);
                r2[p] = add_mod(r2[p], tile_fold(ll2[p], lh2[p], 22, hh2[p], m), m.q);
            }
        }
        if (active && !failed) {
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                u64 *dst = args.out[p];
                dst[e] = r0[p];
                dst[per_poly + e] = add_mod(r1[p], r1[p], m.q); // middle term is 2 x0 x1
                dst[2 * per_poly + e] = r2[p];
            }
        }
    } else {
        // 128-bit running sums; every 63 chunks they are reduced in place, which leaves room for
        // 63 more products of differences below 2^61
        u128d s0[NP], s1[NP], s2[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) s0[p] = s1[p] = s2[p] = u128d{0, 0};
        for (int c0 = 0; c0 < n_chunks && !failed; c0 += 63) {
            const int c1 = min(c0 + 63, n_chunks);
            for (int c = c0; c < c1 && !failed; ++c) {
                chunk(c, [&](const int p, const u64 a0, const u64 a1, const u64 b0, const u64 b1) {
                    // differences left in (0, 2q): 63 products below 2^122 and a residue fit 128 bits
                    const u64 x0 = b0 + m.q - a0, x1 = b1 + m.q - a1;
                    mac_wide(s0[p], x0, x0);
                    mac_wide(s1[p], x0, x1);
                    mac_wide(s2[p], x1, x1);
                });
            }
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                s0[p] = u128d{barrett128(s0[p], m.q, m.r0, m.r1), 0};
                s1[p] = u128d{barrett128(s1[p], m.q, m.r0, m.r1), 0};
                s2[p] = u128d{barrett128(s2[p], m.q, m.r0, m.r1), 0};
            }
        }
        if (active && !failed) {
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                u64 *dst = args.out[p];
                dst[e] = s0[p].lo;
                dst[per_poly + e] = add_mod(s1[p].lo, s1[p].lo, m.q); // middle term is 2 x0 x1
                dst[2 * per_poly + e] = s2[p].lo;
            }
        }
    }
    if (failed && threadIdx.x == 0) atomicOr(status, 2);
}

template <int NA, int NB>
static int launch_tile(Context *ctx, const KrumTileArgs &args, int size_l, int n_chunks, long chunk_stride, cudaStream_t stream)
{
    const long per_poly = (long)size_l << ctx->hp.logN;
    const int seg = (1 << ctx->hp.logN) < kTileThreads ? (1 << ctx->hp.logN) : kTileThreads;
    const long blocks = (long)size_l * ((1L << ctx->hp.logN) / seg);
    const size_t smem = (size_t)kTileStages * 2 * (NA + NB) * seg * sizeof(u64);
    static bool configured[64] = {};
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        LB_CUDA(cudaFuncSetAttribute(krum_tile_kernel<NA, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(kTileStages * 2 * 6 * kTileThreads * sizeof(u64))));
        configured[dev & 63] = true;
    }
    count_launch("krum_tile_kernel", stream, 8.0 * per_poly * ((double)(NA + NB) * 2 * n_chunks + 3.0 * (NB ? NA * NB : NA * (NA - 1) / 2)));
    krum_tile_kernel<NA, NB><<<(unsigned)blocks, kTileThreads, smem, stream>>>(args, ctx->d_mc, ctx->hp.logN, per_poly, chunk_stride, n_chunks,
                                                                               ctx->d_status);
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
