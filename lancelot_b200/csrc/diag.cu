// Diagnostics for benchmarks (include/lancelot_b200_diag.h): launch counter, per-kernel device
// times of whatever the library launches while the timer is on, and the register-only butterfly
// rate probe.  Nothing here is on the compute path; with the timer off a launch costs one
// counter increment.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/lancelot_b200_diag.h"
#include "context.h"
#include "ntt_butterfly.cuh"

namespace lb {

// the transform kernels' launch shape (ntt.cu): the probe runs at their occupancy
constexpr int kNttThreads = 256;
constexpr int kNttMinBlocks = 3;

static unsigned long long g_launches = 0;
unsigned long long launch_count() { return g_launches; }

// ---- kernel timer ---------------------------------------------------------------------------
// While enabled, an event is recorded on the launching stream in front of every kernel of this
// library.  A kernel's time is the span to the next event on the same stream (the next launch, or
// the closing event the report records), so copies and idle gaps between two launches count towards
// the first.  One stream at a time is timed correctly: a launch on another stream closes the
// current span with an event on the previous stream.
constexpr int kMaxMarks = 1 << 15;
struct Mark {
    const char *name;
    cudaEvent_t ev;
    cudaStream_t stream;
    double bytes;
};
static std::mutex g_diag_mu;
static bool g_timing = false;
static std::vector<cudaEvent_t> g_pool;
static std::vector<Mark> g_marks;
static bool g_overflow = false;

void count_launch(const char *name, cudaStream_t stream, double bytes)
{
    ++g_launches;
    if (!g_timing) return;
    std::lock_guard<std::mutex> lock(g_diag_mu);
    if ((int)g_marks.size() >= kMaxMarks) {
        g_overflow = true;
        return;
    }
    cudaEvent_t ev;
    if (g_marks.size() < g_pool.size()) {
        ev = g_pool[g_marks.size()];
    } else {
        if (cudaEventCreate(&ev) != cudaSuccess) return;
        g_pool.push_back(ev);
    }
    cudaEventRecord(ev, stream);
    g_marks.push_back(Mark{name ? name : "other", ev, stream, bytes});
}

// ---- arithmetic ceiling probe -------------------------------------------------------------------
// The same forward butterfly as the transform kernels, on registers only (no shared or global
// memory traffic inside the loop), at the transform kernels' occupancy.  Its rate is the ceiling
// the modular arithmetic of that butterfly variant sets for any NTT schedule on this GPU; one
// limb of N points needs (N/2) log2 N butterflies for 16 N bytes of traffic.
template <int MODE>
__global__ void __launch_bounds__(kNttThreads, kNttMinBlocks) butterfly_probe_kernel(u64 *out, const u64 q, const u64 w0, const u64 ws0,
                                                                                       const int iters)
{
    u64 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (u64)threadIdx.x * 8 + i + blockIdx.x;
    if (is_f64_mode(MODE)) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = bits_of(f64_from_u52(v[i]));
    }
    const u64 q2 = bf_scalar_q2<MODE>(q), q1 = bf_scalar_q<MODE>(q);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            const int half = 4 >> s;
#pragma unroll
            for (int b = 0; b < (1 << s); ++b) {
                // twiddles that differ per thread and stage, so that nothing is hoisted out of the loop
                const ulonglong2 w = is_f64_mode(MODE) ? make_ulonglong2(bits_of(f64_of(w0) + (double)(threadIdx.x + b)), bits_of(f64_of(ws0) * (double)(1 + s)))
                                                  : make_ulonglong2(w0 + threadIdx.x + b, ws0 + threadIdx.x + s);
#pragma unroll
                for (int i = 0; i < half; ++i) fwd_bf<MODE>(v[b * 2 * half + i], v[b * 2 * half + i + half], w, q1, q2);
            }
        }
        // keep the lazy ranges bounded, as the closing reduction does
        if (MODE == kIntLazy) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] &= 0x03FFFFFFFFFFFFFFull;
        }
        if (is_f64_mode(MODE)) { // one centred reduction per element and radix-8 pass: what the tight variant does
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = bits_of(f64_centre(f64_of(v[i]), f64_of(q1), f64_of(q2)));
        }
    }
    u64 acc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc ^= v[i];
    out[(size_t)blockIdx.x * blockDim.x + threadIdx.x] = acc;
}

// mode: 0 integer strict, 1 integer lazy, 2 all on the FP64 pipe at a 50-bit prime, 3 all on the FP64 pipe at a 40-bit prime,
// -1 the variant the context's first prime takes.
int probe_butterfly_rate(Context *ctx, int mode, double *butterflies_per_second)
{
    if (mode < 0) {
        const u64 q0 = ctx->hp.q[0];
        mode = q0 < kF64PrimeLimit ? kF64 : q0 < kF64TightPrimeLimit ? kF64Tight : (q0 >> 58) == 0 ? kIntLazy : kIntStrict;
    }
    if (mode > kF64) {
        set_error("butterfly variant must be 0..3 or -1");
        return LB_ERR_INVALID_ARG;
    }
    const int blocks = ctx->sm_count * kNttMinBlocks, iters = 2000;
    int rc = ctx->ensure_workspace((size_t)blocks * kNttThreads * sizeof(u64));
    if (rc) return rc;
    u64 *out = reinterpret_cast<u64 *>(ctx->ws);
    // any odd modulus of the variant's size gives the variant's instruction stream
    static const u64 size_of_mode[4] = {(u64(1) << 60) - 93, (u64(1) << 57) - 13, (u64(1) << 50) - 27, (u64(1) << 40) - 87};
    const u64 q = size_of_mode[mode], w = h_twiddle_value(q / 3, q), ws = h_twiddle_quot(q / 3, q);
    cudaEvent_t e0, e1;
    LB_CUDA(cudaEventCreate(&e0));
    LB_CUDA(cudaEventCreate(&e1));
    float best = 1e30f;
    for (int rep = 0; rep < 4; ++rep) {
        LB_CUDA(cudaEventRecord(e0, 0));
        count_launch("butterfly_probe_kernel", nullptr);
        switch (mode) {
        case kIntStrict: butterfly_probe_kernel<kIntStrict><<<blocks, kNttThreads>>>(out, q, w, ws, iters); break;
        case kIntLazy: butterfly_probe_kernel<kIntLazy><<<blocks, kNttThreads>>>(out, q, w, ws, iters); break;
        case kF64Tight: butterfly_probe_kernel<kF64Tight><<<blocks, kNttThreads>>>(out, q, w, ws, iters); break;
        default: butterfly_probe_kernel<kF64><<<blocks, kNttThreads>>>(out, q, w, ws, iters); break;
        }
        LB_CUDA(cudaEventRecord(e1, 0));
        LB_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        LB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *butterflies_per_second = (double)blocks * kNttThreads * iters * 12.0 / (best * 1e-3);
    return LB_OK;
}


} // namespace lb

using namespace lb;

extern "C" {

unsigned long long lb_launch_count(void) { return launch_count(); }

int lb_diag_kernel_timing(int enable)
{
    std::lock_guard<std::mutex> lock(g_diag_mu);
    g_marks.clear();
    g_overflow = false;
    g_timing = enable != 0;
    return LB_OK;
}

int lb_diag_kernel_report(char *buf, size_t capacity)
{
    std::lock_guard<std::mutex> lock(g_diag_mu);
    if (!buf || capacity < 64) {
        set_error("report buffer is too small");
        return LB_ERR_INVALID_ARG;
    }
    struct Row {
        const char *name;
        long launches;
        double ms, bytes;
    };
    std::vector<Row> rows;
    if (!g_marks.empty()) {
        cudaEvent_t last;
        LB_CUDA(cudaEventCreateWithFlags(&last, cudaEventDefault));
        LB_CUDA(cudaEventRecord(last, g_marks.back().stream));
        LB_CUDA(cudaEventSynchronize(last));
        for (size_t i = 0; i < g_marks.size(); ++i) {
            cudaEvent_t end = i + 1 < g_marks.size() ? g_marks[i + 1].ev : last;
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, g_marks[i].ev, end) != cudaSuccess) {
                (void)cudaGetLastError();
                ms = 0.f;
            }
            size_t r = 0;
            while (r < rows.size() && std::strcmp(rows[r].name, g_marks[i].name)) ++r;
            if (r == rows.size()) rows.push_back(Row{g_marks[i].name, 0, 0.0, 0.0});
            rows[r].launches += 1;
            rows[r].ms += ms;
            rows[r].bytes += g_marks[i].bytes;
        }
        cudaEventDestroy(last);
    }
    size_t off = 0;
    auto put = [&](const char *fmt, auto... a) {
        if (off < capacity) {
            int n = std::snprintf(buf + off, capacity - off, fmt, a...);
            if (n > 0) off += (size_t)n;
        }
    };
    put("{");
    for (size_t r = 0; r < rows.size(); ++r)
        put("%s\"%s\": {\"launches\": %ld, \"ms\": %.4f, \"bytes\": %.0f}", r ? ", " : "", rows[r].name, rows[r].launches, rows[r].ms,
            rows[r].bytes);
    put("%s\"_overflow\": %s}", rows.empty() ? "" : ", ", g_overflow ? "true" : "false");
    g_marks.clear();
    if (off >= capacity) {
        set_error("report buffer is too small");
        return LB_ERR_INVALID_ARG;
    }
    return LB_OK;
}

int lb_probe_butterfly_rate(lb_context *h, int variant, double *butterflies_per_second)
{
    Context *c = lb_context_impl(h);
    if (!c || !butterflies_per_second) {
        set_error("context or destination is null");
        return LB_ERR_INVALID_ARG;
    }
    LB_CUDA(cudaSetDevice(c->device));
    return probe_butterfly_rate(c, variant, butterflies_per_second);
}

} // extern "C"
