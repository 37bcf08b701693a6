#include "context.h"

#include <cmath>
#include <cstring>
#include <mutex>

namespace lb {

static thread_local std::string g_error;

void set_error(const std::string &msg) { g_error = msg; }

const std::string &last_error() { return g_error; }

int cuda_fail(cudaError_t e, const char *what)
{
    g_error = std::string("CUDA error: ") + cudaGetErrorString(e) + " in " + what;
    (void)cudaGetLastError(); // a rejected launch must not poison the next call's error check
    return LB_ERR_CUDA;
}

// One scratch block per device survives its context: a caller that builds a fresh context
// every round (as the reference's Krum driver does) then pays for cudaMalloc / cudaFree of
// gigabytes only once per process.
constexpr int kMaxCachedDevices = 64;
static std::mutex g_ws_mu; // guards the two arrays below
static void *g_ws_cache[kMaxCachedDevices];
static size_t g_ws_cache_bytes[kMaxCachedDevices];

int Context::ensure_workspace(size_t bytes)
{
    if (bytes <= ws_bytes) return LB_OK;
    void *cached = nullptr;
    size_t cached_bytes = 0;
    if (device >= 0 && device < kMaxCachedDevices) {
        std::lock_guard<std::mutex> lock(g_ws_mu);
        if (g_ws_cache[device] && g_ws_cache_bytes[device] >= bytes) {
            cached = g_ws_cache[device];
            cached_bytes = g_ws_cache_bytes[device];
            g_ws_cache[device] = nullptr;
            g_ws_cache_bytes[device] = 0;
        }
    }
    if (cached) {
        // work queued on the previous block (if any) must finish before it is dropped
        if (ws) {
            LB_CUDA(cudaDeviceSynchronize());
            LB_CUDA(cudaFree(ws));
        }
        ws = cached;
        ws_bytes = cached_bytes;
        return LB_OK;
    }
    // the old block may still be in use by work queued earlier
    LB_CUDA(cudaDeviceSynchronize());
    if (ws) LB_CUDA(cudaFree(ws));
    ws = nullptr;
    ws_bytes = 0;
    const size_t want = bytes + bytes / 4;
    cudaError_t e = cudaMalloc(&ws, want);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("out of device memory for the workspace");
        return LB_ERR_NO_MEMORY;
    }
    ws_bytes = want;
    return LB_OK;
}

template <class T>
static int upload(Context *ctx, T **dst, const T *src, size_t count)
{
    *dst = nullptr;
    if (count == 0) return LB_OK;
    LB_CUDA(cudaMalloc((void **)dst, count * sizeof(T)));
    ctx->owned.push_back(*dst);
    LB_CUDA(cudaMemcpy(*dst, src, count * sizeof(T), cudaMemcpyHostToDevice));
    return LB_OK;
}

// Complex 2N-th roots of unity exactly as the reference encoder derives them: one eighth
// from std::polar, the rest by symmetry (cahel-main/src/croots.cu:27-66).
static void complex_root(size_t index, size_t M, double &re, double &im)
{
    static const double PI = 3.1415926535897932384626433832795028842;
    index &= M - 1;
    if (index <= M / 8) {
        const double th = 2 * PI * (double)index / (double)M;
        re = std::cos(th);
        im = std::sin(th);
    } else if (index <= M / 4) {
        complex_root(M / 4 - index, M, im, re);
    } else if (index <= M / 2) {
        complex_root(M / 2 - index, M, re, im);
        re = 0.0 - re;
        im = 0.0 - (-im);
    } else if (index <= 3 * M / 4) {
        complex_root(index - M / 2, M, re, im);
        re = 0.0 - re;
        im = 0.0 - im;
    } else {
        complex_root(M - index, M, re, im);
        im = -im;
    }
}

// Destroyed contexts are parked with their device tables instead of being freed: the tables
// depend only on (device, ring degree, primes, Galois elements), and a caller that builds a
// fresh context for every round (as the reference's Krum driver does) otherwise repeats the
// host precompute, some fifty allocations and their uploads each time.
constexpr size_t kMaxParked = 4;
static std::mutex g_parked_mu;
static std::vector<Context *> g_parked;

static void release_tables(Context *ctx)
{
    for (void *p : ctx->owned) cudaFree(p);
    delete ctx;
}

static Context *take_parked(int logN, const std::vector<u64> &moduli, int size_P, const std::vector<uint32_t> &elts, int device)
{
    std::lock_guard<std::mutex> lock(g_parked_mu);
    for (size_t i = 0; i < g_parked.size(); ++i) {
        Context *c = g_parked[i];
        if (c->device == device && c->hp.logN == logN && c->hp.size_P == size_P && c->hp.q == moduli && c->hp.galois_elts == elts) {
            g_parked.erase(g_parked.begin() + i);
            return c;
        }
    }
    return nullptr;
}

int context_create(int logN, const std::vector<u64> &moduli, int size_P, const std::vector<uint32_t> &elts, int device,
                   Context **out)
{
    *out = nullptr;
    if (Context *parked = take_parked(logN, moduli, size_P, elts, device)) {
        cudaError_t pe = cudaSetDevice(device);
        if (pe == cudaSuccess) pe = cudaMemset(parked->d_status, 0, 256);
        if (pe != cudaSuccess) {
            release_tables(parked);
            return cuda_fail(pe, "reviving a parked context");
        }
        *out = parked;
        return LB_OK;
    }
    Context *ctx = new Context();
    if (!ctx->hp.init(logN, moduli, size_P, elts)) {
        set_error(ctx->hp.error);
        delete ctx;
        return LB_ERR_INVALID_ARG;
    }
    ctx->device = device;
    int rc = LB_OK;
    auto fail = [&](int code) {
        for (void *p : ctx->owned) cudaFree(p);
        delete ctx;
        return code;
    };
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaSetDevice"));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(cuda_fail(e, "cudaGetDeviceProperties"));
    if (prop.major < 9) {
        set_error("this library needs thread-block clusters (compute capability 10.0)");
        return fail(LB_ERR_LOGIC);
    }
    ctx->sm_count = prop.multiProcessorCount;
    const HostParams &hp = ctx->hp;
    const size_t N = hp.N;
    if ((rc = upload(ctx, &ctx->d_mc, hp.mc.data(), hp.mc.size()))) return fail(rc);
    if ((rc = upload(ctx, &ctx->d_tw, reinterpret_cast<const ulonglong2 *>(hp.tw.data()), hp.tw.size() / 2))) return fail(rc);
    if ((rc = upload(ctx, &ctx->d_itw, reinterpret_cast<const ulonglong2 *>(hp.itw.data()), hp.itw.size() / 2))) return fail(rc);
    if ((rc = upload(ctx, &ctx->d_perm, hp.perm.data(), hp.perm.size()))) return fail(rc);
    if ((rc = upload(ctx, &ctx->d_p_mod_q, hp.p_mod_q.data(), hp.p_mod_q.size()))) return fail(rc);
    if ((rc = upload(ctx, &ctx->d_p_mod_q_s, hp.p_mod_q_s.data(), hp.p_mod_q_s.size()))) return fail(rc);
    ctx->d_level.resize(hp.size_Q + 1);
    for (int L = 1; L <= hp.size_Q; ++L) {
        const LevelConst &lc = hp.level[L];
        DevLevel &d = ctx->d_level[L];
        if ((rc = upload(ctx, &d.qlast_inv, lc.qlast_inv.data(), lc.qlast_inv.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.qlast_inv_s, lc.qlast_inv_s.data(), lc.qlast_inv_s.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.p_inv, lc.p_inv.data(), lc.p_inv.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.p_inv_s, lc.p_inv_s.data(), lc.p_inv_s.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.hat_inv, lc.hat_inv.data(), lc.hat_inv.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.hat_inv_s, lc.hat_inv_s.data(), lc.hat_inv_s.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.hat_mod, lc.hat_mod.data(), lc.hat_mod.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.phat_inv, lc.phat_inv.data(), lc.phat_inv.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.phat_inv_s, lc.phat_inv_s.data(), lc.phat_inv_s.size()))) return fail(rc);
        if ((rc = upload(ctx, &d.phat_mod, lc.phat_mod.data(), lc.phat_mod.size()))) return fail(rc);
        if (hp.size_P > 0) {
            std::vector<u64> fold((size_t)L * 4), pfold((size_t)hp.size_P * 4);
            for (int r = 0; r < L; ++r) {
                const ModConst &m = hp.mc[r];
                fold[4 * r + 0] = h_mulmod(m.ninv, lc.hat_inv[r], m.q);
                fold[4 * r + 1] = h_shoup(fold[4 * r + 0], m.q);
                fold[4 * r + 2] = h_mulmod(m.iw1n, lc.hat_inv[r], m.q);
                fold[4 * r + 3] = h_shoup(fold[4 * r + 2], m.q);
            }
            for (int i = 0; i < hp.size_P; ++i) {
                const ModConst &m = hp.mc[hp.size_Q + i];
                pfold[4 * i + 0] = h_mulmod(m.ninv, lc.phat_inv[i], m.q);
                pfold[4 * i + 1] = h_shoup(pfold[4 * i + 0], m.q);
                pfold[4 * i + 2] = h_mulmod(m.iw1n, lc.phat_inv[i], m.q);
                pfold[4 * i + 3] = h_shoup(pfold[4 * i + 2], m.q);
            }
            if ((rc = upload(ctx, &d.fold, fold.data(), fold.size()))) return fail(rc);
            if ((rc = upload(ctx, &d.pfold, pfold.data(), pfold.size()))) return fail(rc);
        }
    }
    // encoder tables (cahel-main/src/ckks.cu:34-102)
    {
        const size_t M = 2 * N;
        std::vector<double> roots(2 * M);
        for (size_t i = 0; i < M; ++i) complex_root(i, M, roots[2 * i], roots[2 * i + 1]);
        if ((rc = upload(ctx, &ctx->d_croots, reinterpret_cast<const double2 *>(roots.data()), M))) return fail(rc);
        const size_t quarter = N / 4 ? N / 4 : 1;
        std::vector<uint32_t> group(quarter);
        uint32_t pos = 1;
        for (size_t i = 0; i < quarter; ++i) {
            group[i] = pos;
            pos = (uint32_t)(((u64)pos * 5) & (M - 1));
        }
        if ((rc = upload(ctx, &ctx->d_rot_group, group.data(), group.size()))) return fail(rc);
    }
    {
        e = cudaMalloc((void **)&ctx->d_status, 256);
        if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMalloc"));
        ctx->owned.push_back(ctx->d_status);
        e = cudaMemset(ctx->d_status, 0, 256);
        if (e != cudaSuccess) return fail(cuda_fail(e, "cudaMemset"));
    }
    *out = ctx;
    return LB_OK;
}

void context_destroy(Context *ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->ws) {
        const int d = ctx->device;
        void *drop = ctx->ws;
        if (d >= 0 && d < kMaxCachedDevices) {
            std::lock_guard<std::mutex> lock(g_ws_mu);
            if (ctx->ws_bytes > g_ws_cache_bytes[d]) {
                drop = g_ws_cache[d];
                g_ws_cache[d] = ctx->ws;
                g_ws_cache_bytes[d] = ctx->ws_bytes;
            }
        }
        if (drop) cudaFree(drop);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
    }
    Context *evicted = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_parked_mu);
        g_parked.push_back(ctx);
        if (g_parked.size() > kMaxParked) {
            evicted = g_parked.front();
            g_parked.erase(g_parked.begin());
        }
    }
    if (evicted) {
        cudaSetDevice(evicted->device);
        release_tables(evicted);
        cudaSetDevice(ctx->device);
    }
}

} // namespace lb
