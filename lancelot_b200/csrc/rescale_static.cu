// Rescale without any device allocation.
//
// Some callers of this library must not allocate device memory while they work: code
// that runs between the capture calls of a CUDA graph, a serving loop whose memory was
// budgeted up front so that nothing else may grow, or a host framework that owns the
// allocator and forbids foreign cudaMalloc calls on its device.  The regular rescale keeps its
// scratch (the last limb of every polynomial in coefficient form) in the context's
// workspace, which is grown with cudaMalloc on demand.  This variant keeps that scratch in
// a fixed array that is part of the library image instead, so the call itself never
// allocates or frees anything.
//
// Price: every GPU that loads the library holds the array (kStaticWords * 8 bytes = 1.5 MiB)
// until the process exits, the size is capped, and all calls on one device share the one
// array, so two calls that overlap on the GPU (different streams) race.
#include <atomic>

#include "context.h"

namespace lb {

// room for three polynomials of ring degree 65536 (or six of 32768, ...)
constexpr size_t kStaticWords = 3 * 65536;
static __device__ __align__(256) u64 g_rescale_scratch[kStaticWords];

constexpr int kMaxDevices = 64;
// device address of g_rescale_scratch per device; the symbol itself is only a host-side
// handle and must never be handed to a kernel
static std::atomic<u64 *> g_scratch_addr[kMaxDevices]; // two host threads may resolve it at once: both store the same value

// Resolves the array's address on the current device once.  Not an allocation: the array
// already exists in the loaded module.  Do this before any stream capture starts.
static int static_scratch(u64 **out)
{
    int dev = 0;
    LB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("device ordinal out of range for the allocation-free rescale");
        return LB_ERR_INVALID_ARG;
    }
    u64 *addr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!addr) {
        void *p = nullptr;
        LB_CUDA(cudaGetSymbolAddress(&p, g_rescale_scratch));
        addr = static_cast<u64 *>(p);
        g_scratch_addr[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return LB_OK;
}

size_t rescale_static_max_words() { return kStaticWords; }

// Same arithmetic as rescale() in keyswitch.cu (cahel-main/src/rns.cu:544-570), scratch in
// the static array.  The inverse transform overwrites every scratch word the forward pass
// reads, so nothing has to be cleared between calls.
int rescale_static(Context *ctx, int L, int n_polys, const u64 *in, u64 *out, cudaStream_t stream)
{
    if (L < 2 || L > ctx->hp.size_Q) { set_error("cannot rescale: no next level"); return LB_ERR_INVALID_ARG; }
    if (n_polys < 1 || (size_t)n_polys * ctx->hp.N > kStaticWords) {
        set_error("allocation-free rescale: n_polys * N exceeds the static scratch of 196608 words");
        return LB_ERR_INVALID_ARG;
    }
    u64 *last = nullptr;
    int rc = static_scratch(&last);
    if (rc) return rc;
    NttJob inv;
    inv.src = in;
    inv.dst = last;
    inv.n_groups = n_polys;
    inv.per_group = 1;
    inv.size_l = 1;
    inv.tbl_off = L - 1;
    inv.src_group_stride = L;
    inv.src_row_off = L - 1;
    inv.dst_group_stride = 1;
    if ((rc = ntt_inverse(ctx, inv, stream))) return rc;
    const DevLevel &dl = ctx->d_level[L];
    NttJob fwd;
    fwd.src = last;
    fwd.dst = out;
    fwd.n_groups = n_polys;
    fwd.per_group = L - 1;
    fwd.size_l = L - 1;
    fwd.src_group_stride = 1;
    fwd.dst_group_stride = L - 1;
    fwd.bconv_n = 1;
    fwd.aux = in;
    fwd.aux_group_stride = L;
    fwd.scal = dl.qlast_inv;
    fwd.scal_s = dl.qlast_inv_s;
    return ntt_forward(ctx, fwd, stream);
}

} // namespace lb
