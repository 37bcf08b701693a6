// Fixture generator: drives the UNMODIFIED reference library (cahel-main, compiled by
// oracle/Makefile.ref) through the CKKS chain on a GPU and records, for every stage,
// the SHA-256 of the device buffer plus its first words.  The seeds every call consumed
// are logged by the force-included seed shim, so the CPU restatement and the product
// library can replay the same keys and ciphertexts and must reproduce the same digests.
//
// Test infrastructure only.
// Usage: ref_harness <out.json> [--cases a,b,...] [--dump dir [--dump-only stage,...]] [--time timings.json]
//   --cases  run only the named parameter sets (default: all of them)
//   --dump   also write the raw bytes of every (or only the named) recorded stage to <dir>/<case>.<stage>.bin
//   --time   also time the reference's own operations with CUDA events and write them as JSON
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "cahel.h"

using namespace cahel;

// ---- logged deterministic word stream behind std::random_device --------------------------
static std::vector<uint32_t> g_words;
static uint64_t g_state = 0x243F6A8885A308D3ull;

extern "C" uint32_t lb_shim_next_word(void)
{
    // splitmix64
    g_state += 0x9E3779B97F4A7C15ull;
    uint64_t z = g_state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    uint32_t w = (uint32_t)(z >> 16);
    g_words.push_back(w);
    return w;
}

// ---- SHA-256 ---------------------------------------------------------------------------
struct Sha256 {
    uint32_t h[8];
    uint8_t buf[64];
    uint64_t len = 0;
    size_t fill = 0;
    Sha256()
    {
        static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
        memcpy(h, init, sizeof(h));
    }
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t *p)
    {
        static const uint32_t k[64] = {
            0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be,
            0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa,
            0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85,
            0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3,
            0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f,
            0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
        uint32_t w[64];
        for (int i = 0; i < 16; i++) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; i++) {
            uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; i++) {
            uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25), ch = (e & f) ^ (~e & g);
            uint32_t t1 = hh + S1 + ch + k[i] + w[i];
            uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22), mj = (a & b) ^ (a & c) ^ (b & c);
            uint32_t t2 = S0 + mj;
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const void *data, size_t n)
    {
        const uint8_t *p = (const uint8_t *)data;
        len += n;
        while (n) {
            size_t take = 64 - fill < n ? 64 - fill : n;
            memcpy(buf + fill, p, take);
            fill += take; p += take; n -= take;
            if (fill == 64) { block(buf); fill = 0; }
        }
    }
    std::string hex()
    {
        uint64_t bits = len * 8;
        uint8_t pad = 0x80;
        update(&pad, 1);
        uint8_t z = 0;
        while (fill != 56) update(&z, 1);
        uint8_t lb[8];
        for (int i = 0; i < 8; i++) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(lb, 8);
        char out[65];
        for (int i = 0; i < 8; i++) snprintf(out + 8 * i, 9, "%08x", h[i]);
        return std::string(out);
    }
};

// ---- recording ---------------------------------------------------------------------------
static std::ostringstream g_json;
static bool g_first = true;
static std::string g_dump_dir;
static std::vector<std::string> g_dump_only; // stage names to dump (empty: every stage)
static std::string g_case;

static void record_host(const std::string &name, const void *data, size_t bytes, bool is_double = false)
{
    Sha256 s;
    s.update(data, bytes);
    if (!g_first) g_json << ",\n";
    g_first = false;
    g_json << "    \"" << name << "\": {\"bytes\": " << bytes << ", \"sha256\": \"" << s.hex() << "\", \"head\": [";
    size_t n = bytes / 8 < 8 ? bytes / 8 : 8;
    for (size_t i = 0; i < n; i++) {
        if (i) g_json << ", ";
        if (is_double) {
            char b[64];
            snprintf(b, sizeof(b), "%.17g", ((const double *)data)[i]);
            g_json << b;
        } else {
            g_json << "\"" << ((const uint64_t *)data)[i] << "\"";
        }
    }
    g_json << "]}";
    if (!g_dump_dir.empty() && (g_dump_only.empty() || std::find(g_dump_only.begin(), g_dump_only.end(), name) != g_dump_only.end())) {
        std::ofstream f(g_dump_dir + "/" + g_case + "." + name + ".bin", std::ios::binary);
        f.write((const char *)data, bytes);
    }
}

static void record_dev(const std::string &name, const uint64_t *dev, size_t count)
{
    std::vector<uint64_t> h(count);
    CUDA_CHECK(cudaMemcpy(h.data(), dev, count * 8, cudaMemcpyDeviceToHost));
    record_host(name, h.data(), count * 8);
}

// seeds consumed since `from`: groups of 16 words, each group stored in reverse draw order
// (cahel-main/include/prng.cuh:15-21 fills its buffer from the back)
static void record_seeds(const std::string &name, size_t from)
{
    std::vector<uint32_t> out;
    size_t n = g_words.size() - from;
    for (size_t g = 0; g + 16 <= n; g += 16)
        for (int i = 15; i >= 0; i--) out.push_back(g_words[from + g + i]);
    if (!g_first) g_json << ",\n";
    g_first = false;
    g_json << "    \"" << name << "\": {\"seed_words\": [";
    for (size_t i = 0; i < out.size(); i++) g_json << (i ? ", " : "") << out[i];
    g_json << "]}";
}

// the byte stream of an object's own save(): digest of everything, and for ciphertexts also of
// everything before the trailing 64-byte seed buffer (whose content the library never defines
// for ciphertexts it did not seed-compress) plus that tail itself
template <class T>
static void record_stream(const std::string &name, T &obj, bool has_seed_tail)
{
    std::ostringstream os(std::ios::binary);
    obj.save(os);
    const std::string b = os.str();
    record_host(name, b.data(), b.size());
    if (has_seed_tail && b.size() >= 64) {
        record_host(name + "_body", b.data(), b.size() - 64);
        record_host(name + "_tail", b.data() + b.size() - 64, 64);
    }
}

// message slot i = (i * 2654435761 mod 2^32) / 2^31 - 1, exactly representable
static std::vector<double> message(size_t n, uint32_t salt)
{
    std::vector<double> v(n);
    for (size_t i = 0; i < n; i++) {
        uint32_t x = (uint32_t)((i + salt) * 2654435761u);
        v[i] = (double)x / 2147483648.0 - 1.0;
    }
    return v;
}

static std::vector<std::string> g_only;
static bool g_first_case = true;

static bool wanted(const std::string &name)
{
    return g_only.empty() || std::find(g_only.begin(), g_only.end(), name) != g_only.end();
}

// naf_step: a rotation step that has no key of its own, so that rotate_vector goes through the
// non-adjacent-form decomposition (0 = skip)
static void run_case(const std::string &name, size_t n, const std::vector<int> &bits, size_t size_P, double scale,
                     const std::vector<int> &steps, int naf_step = 0)
{
    if (!wanted(name)) return;
    g_case = name;
    g_first = true;
    g_json << (g_first_case ? "" : ",\n") << "  \"" << name << "\": {\n";
    g_first_case = false;
    EncryptionParameters parms(scheme_type::ckks);
    parms.set_poly_modulus_degree(n);
    auto moduli = CoeffModulus::Create(n, bits);
    parms.set_coeff_modulus(moduli);
    parms.set_special_modulus_size(size_P);
    auto elts = get_elts_from_steps(steps, n);
    parms.set_galois_elts(elts);
    {
        std::vector<uint64_t> mv;
        for (auto &m : moduli) mv.push_back(m.value());
        record_host("moduli", mv.data(), mv.size() * 8);
        std::vector<uint64_t> ev(elts.begin(), elts.end());
        record_host("galois_elts", ev.data(), ev.size() * 8);
    }
    CAHELGPUContext context(parms, true, sec_level_type::none);
    const size_t size_QP = moduli.size(), size_Q = size_QP - size_P, dnum = size_Q / size_P;

    size_t mark = g_words.size();
    CAHELGPUSecretKey sk(parms);
    sk.gen_secretkey(context);
    record_seeds("seed_sk", mark);
    record_dev("sk", sk.secret_key_array(), size_QP * n);

    mark = g_words.size();
    CAHELGPUPublicKey pk(context);
    sk.gen_publickey(context, pk);
    record_seeds("seed_pk", mark);
    record_dev("pk", pk.pk_.data(), 2 * size_QP * n);

    mark = g_words.size();
    CAHELGPURelinKey rlk(context);
    sk.gen_relinkey(context, rlk);
    record_seeds("seed_rlk", mark);
    for (size_t j = 0; j < dnum; j++) record_dev("rlk" + std::to_string(j), rlk.public_keys_[j].pk_.data(), 2 * size_QP * n);

    mark = g_words.size();
    CAHELGPUGaloisKey glk(context);
    sk.create_galois_keys(context, glk);
    record_seeds("seed_glk", mark);
    for (size_t e = 0; e < elts.size(); e++)
        for (size_t j = 0; j < dnum; j++)
            record_dev("glk" + std::to_string(e) + "_" + std::to_string(j), glk.relin_keys_[e].public_keys_[j].pk_.data(), 2 * size_QP * n);

    CAHELGPUCKKSEncoder encoder(context);
    const size_t slots = encoder.slot_count();
    auto m1 = message(slots, 1), m2 = message(slots, 77);
    CAHELGPUPlaintext pt1(context), pt2(context);
    encoder.encode(context, m1, scale, pt1);
    encoder.encode(context, m2, scale, pt2);
    record_dev("pt1", pt1.data(), size_Q * n);
    record_dev("pt2", pt2.data(), size_Q * n);

    mark = g_words.size();
    CAHELGPUCiphertext ct1(context), ct2(context);
    pk.encrypt_asymmetric(context, pt1, ct1, false);
    pk.encrypt_asymmetric(context, pt2, ct2, false);
    record_seeds("seed_enc", mark);
    record_dev("ct1", ct1.data(), 2 * size_Q * n);
    record_dev("ct2", ct2.data(), 2 * size_Q * n);
    record_stream("stream_pt1", pt1, false);
    record_stream("stream_ct1", ct1, true);
    record_stream("stream_pk", pk, true);
    record_stream("stream_rlk", rlk, false);
    record_stream("stream_glk", glk, false);

    CAHELGPUCiphertext diff(context), prod(context);
    sub(context, ct2, ct1, diff);
    record_dev("sub", diff.data(), 2 * size_Q * n);
    multiply(context, ct1, ct2, prod);
    record_dev("mul", prod.data(), 3 * size_Q * n);
    CAHELGPUCiphertext sq(diff);
    square_inplace(context, sq);
    record_dev("square", sq.data(), 3 * size_Q * n);

    relinearize_inplace(context, prod, rlk);
    record_dev("relin", prod.data(), 2 * size_Q * n);
    rescale_to_next_inplace(context, prod);
    const size_t L2 = size_Q - 1;
    record_dev("rescale", prod.data(), 2 * L2 * n);
    prod.set_scale(scale);
    record_stream("stream_rescaled", prod, true);

    CAHELGPUCiphertext rot(context);
    rotate_vector(context, prod, steps[0], glk, rot);
    record_dev("rotate", rot.data(), 2 * L2 * n);

    if (naf_step) {
        CAHELGPUCiphertext rn(context);
        rotate_vector(context, prod, naf_step, glk, rn);
        record_dev("rotate_naf", rn.data(), 2 * L2 * n);
    }

    CAHELGPUCiphertext hoist = hoisting(context, prod, glk, steps);
    record_dev("hoisting", hoist.data(), 2 * L2 * n);

    // second level down when the chain allows it (exercises a partial last digit)
    if (L2 >= 2) {
        CAHELGPUCiphertext low(prod);
        mod_switch_to_next_inplace(context, low);
        record_dev("drop", low.data(), 2 * (L2 - 1) * n);
        CAHELGPUCiphertext rot2(context);
        rotate_vector(context, low, steps[0], glk, rot2);
        record_dev("rotate_low", rot2.data(), 2 * (L2 - 1) * n);
    }

    CAHELGPUPlaintext dec(context);
    sk.decrypt(context, hoist, dec);
    record_dev("decrypt", dec.data(), L2 * n);
    std::vector<cuDoubleComplex> out;
    encoder.decode(context, dec, out);
    record_host("decode", out.data(), out.size() * sizeof(cuDoubleComplex), true);

    g_json << "\n  }";
}

// ---- the reference's own operations timed with CUDA events -------------------------------
static std::ostringstream g_time_json;
static bool g_time_first_case = true;

template <class F, class G>
static double median_ms(int reps, G &&prepare, F &&op)
{
    cudaEvent_t a, b;
    CUDA_CHECK(cudaEventCreate(&a));
    CUDA_CHECK(cudaEventCreate(&b));
    std::vector<float> ms;
    for (int r = 0; r < reps + 2; r++) {
        prepare();
        CUDA_CHECK(cudaDeviceSynchronize());
        CUDA_CHECK(cudaEventRecord(a, 0));
        op();
        CUDA_CHECK(cudaEventRecord(b, 0));
        CUDA_CHECK(cudaEventSynchronize(b));
        float t;
        CUDA_CHECK(cudaEventElapsedTime(&t, a, b));
        if (r >= 2) ms.push_back(t);  // two untimed warm-up runs
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    std::sort(ms.begin(), ms.end());
    return ms[ms.size() / 2];
}

// Median milliseconds of each operation of cahel-main/examples/7_performance.cu:540-757 (host call to result on
// the device, legacy default stream as the reference uses it), plus the per-chunk body of the Krum driver
// (lancelot-main-GPU/utils/byzantine_fl.py:201-223) and the plain forward / inverse transform of all data limbs.
static void time_case(const std::string &name, size_t n, const std::vector<int> &bits, size_t size_P, double scale,
                      const std::vector<int> &steps, int reps)
{
    if (!wanted(name)) return;
    EncryptionParameters parms(scheme_type::ckks);
    parms.set_poly_modulus_degree(n);
    auto moduli = CoeffModulus::Create(n, bits);
    parms.set_coeff_modulus(moduli);
    parms.set_special_modulus_size(size_P);
    parms.set_galois_elts(get_elts_from_steps(steps, n));
    CAHELGPUContext context(parms, true, sec_level_type::none);
    const size_t size_Q = moduli.size() - size_P;
    CAHELGPUSecretKey sk(parms);
    sk.gen_secretkey(context);
    CAHELGPUPublicKey pk(context);
    sk.gen_publickey(context, pk);
    CAHELGPURelinKey rlk(context);
    sk.gen_relinkey(context, rlk);
    CAHELGPUGaloisKey glk(context);
    sk.create_galois_keys(context, glk);
    CAHELGPUCKKSEncoder encoder(context);
    auto m1 = message(encoder.slot_count(), 1), m2 = message(encoder.slot_count(), 77);
    CAHELGPUPlaintext pt1(context), pt2(context);
    CAHELGPUCiphertext ct1(context), ct2(context), work(context), work2(context), acc(context);
    auto nothing = [] {};
    std::vector<std::pair<std::string, double>> out;
    out.push_back({"keygen_all", median_ms(3, nothing, [&] {
                       CAHELGPUSecretKey s2(parms);
                       s2.gen_secretkey(context);
                       CAHELGPUPublicKey p2(context);
                       s2.gen_publickey(context, p2);
                       CAHELGPURelinKey r2(context);
                       s2.gen_relinkey(context, r2);
                       CAHELGPUGaloisKey g2(context);
                       s2.create_galois_keys(context, g2);
                   })});
    out.push_back({"encode", median_ms(reps, nothing, [&] { encoder.encode(context, m1, scale, pt1); })});
    encoder.encode(context, m2, scale, pt2);
    out.push_back({"encrypt", median_ms(reps, nothing, [&] { pk.encrypt_asymmetric(context, pt1, ct1, false); })});
    pk.encrypt_asymmetric(context, pt2, ct2, false);
    out.push_back({"sub", median_ms(reps, nothing, [&] { sub(context, ct2, ct1, work); })});
    out.push_back({"multiply", median_ms(reps, nothing, [&] { multiply(context, ct1, ct2, work); })});
    out.push_back({"square_inplace", median_ms(reps, [&] { work2 = ct1; }, [&] { square_inplace(context, work2); })});
    acc = work2;
    out.push_back({"add_inplace_size3", median_ms(reps, nothing, [&] { add_inplace(context, acc, work2); })});
    // one chunk of one pair as the reference's driver runs it: two encodes, two encryptions, sub, square, add
    out.push_back({"krum_pair_chunk", median_ms(reps, nothing, [&] {
                       encoder.encode(context, m1, scale, pt1);
                       encoder.encode(context, m2, scale, pt2);
                       pk.encrypt_asymmetric(context, pt1, ct1, false);
                       pk.encrypt_asymmetric(context, pt2, ct2, false);
                       sub(context, ct2, ct1, work2);
                       square_inplace(context, work2);
                       add_inplace(context, acc, work2);
                   })});
    out.push_back({"relinearize", median_ms(reps, [&] { work2 = work; }, [&] { relinearize_inplace(context, work2, rlk); })});
    out.push_back({"multiply_relin_rescale", median_ms(reps, nothing, [&] {
                       multiply(context, ct1, ct2, work2);
                       relinearize_inplace(context, work2, rlk);
                       rescale_to_next_inplace(context, work2);
                   })});
    multiply(context, ct1, ct2, work);
    relinearize_inplace(context, work, rlk);
    out.push_back({"rescale", median_ms(reps, [&] { work2 = work; }, [&] { rescale_to_next_inplace(context, work2); })});
    out.push_back({"rotate_vector", median_ms(reps, nothing, [&] { rotate_vector(context, ct1, steps[0], glk, work2); })});
    if (steps.size() > 1)
        out.push_back({"hoisting_" + std::to_string(steps.size()), median_ms(reps, nothing, [&] { work2 = hoisting(context, ct1, glk, steps); })});
    out.push_back({"ntt_forward_data_limbs", median_ms(reps, nothing, [&] {
                       nwt_2d_radix8_forward_inplace(ct1.data(), context.gpu_rns_tables(), size_Q, 0);
                   })});
    out.push_back({"ntt_inverse_data_limbs", median_ms(reps, nothing, [&] {
                       nwt_2d_radix8_backward_inplace(ct1.data(), context.gpu_rns_tables(), size_Q, 0);
                   })});
    CAHELGPUPlaintext dec(context);
    out.push_back({"decrypt", median_ms(reps, nothing, [&] { sk.decrypt(context, ct2, dec); })});
    std::vector<cuDoubleComplex> vals;
    out.push_back({"decode", median_ms(reps, nothing, [&] { encoder.decode(context, dec, vals); })});

    g_time_json << (g_time_first_case ? "" : ",\n") << "  \"" << name << "\": {\"n\": " << n << ", \"size_Q\": " << size_Q
                << ", \"size_P\": " << size_P << ", \"reps\": " << reps << ", \"ms\": {";
    g_time_first_case = false;
    for (size_t i = 0; i < out.size(); i++) {
        char b[64];
        snprintf(b, sizeof(b), "%.4f", out[i].second);
        g_time_json << (i ? ", " : "") << "\"" << out[i].first << "\": " << b;
    }
    g_time_json << "}}";
}

static std::vector<int> range_steps(int lo, int hi)
{
    std::vector<int> v;
    for (int i = lo; i <= hi; i++) v.push_back(i);
    return v;
}

int main(int argc, char **argv)
{
    if (argc < 2) {
        fprintf(stderr, "usage: %s out.json [--cases a,b,...] [--dump dir [--dump-only stage,...]] [--time timings.json]\n", argv[0]);
        return 2;
    }
    std::string time_out;
    for (int i = 2; i < argc; i++) {
        std::string a = argv[i];
        if (a == "--cases" && i + 1 < argc) {
            std::stringstream ss(argv[++i]);
            std::string item;
            while (std::getline(ss, item, ',')) g_only.push_back(item);
        } else if (a == "--dump" && i + 1 < argc) {
            g_dump_dir = argv[++i];
        } else if (a == "--dump-only" && i + 1 < argc) {
            std::stringstream ss(argv[++i]);
            std::string item;
            while (std::getline(ss, item, ',')) g_dump_only.push_back(item);
        } else if (a == "--time" && i + 1 < argc) {
            time_out = argv[++i];
        } else {
            fprintf(stderr, "unknown argument %s\n", a.c_str());
            return 2;
        }
    }
    const double s40 = 1099511627776.0, s50 = 1125899906842624.0;
    // 60 + 23 x 50 data bits and 8 x 60 special bits: the hybrid key-switching benchmark shape (alpha 8, dnum 3)
    std::vector<int> wide = {60};
    for (int i = 0; i < 23; i++) wide.push_back(50);
    for (int i = 0; i < 8; i++) wide.push_back(60);
    g_json << "{\n";
    try {
        // Lancelot's own chain shape {60,40,40 | 60}, alpha = 1, at the smallest 2-D NTT size
        run_case("n4096_a1", 4096, {60, 40, 40, 60}, 1, s40, {1, 2, 3});
        // the ring degree of the primitive-chain benchmark configuration
        run_case("n8192_a1", 8192, {60, 40, 40, 60}, 1, s40, {1, 2, 3});
        // alpha = 2, dnum = 3: generic base-conversion path and, one level down, a partial digit
        run_case("n4096_a2", 4096, {50, 40, 40, 40, 40, 40, 50, 50}, 2, s40, {1, 5});
        // the ring degrees of the two Krum benchmark configurations, with a rotation (5 = 4 + 1) that has no key
        run_case("n32768_a1", 32768, {60, 40, 40, 60}, 1, s40, {1, 2, 4}, 5);
        run_case("n65536_a1", 65536, {60, 40, 40, 60}, 1, s40, {1, 2, 4}, 5);
        // the hybrid key-switching benchmark configuration
        run_case("n65536_a8", 65536, wide, 8, s50, {1, 4}, 5);
        // scale 2^50 leaves two or three bits below the rounding point of the largest coefficients, so these plaintexts
        // pin the encoder's floating-point order: slots = 2048 runs the single-kernel inverse FFT, 4096 adds one
        // stage kernel (cahel-main/src/fft.cu:407-449)
        run_case("n4096_s50", 4096, {60, 60, 60}, 1, s50, {1});
        run_case("n8192_s50", 8192, {60, 60, 60}, 1, s50, {1});
    } catch (const std::exception &e) {
        fprintf(stderr, "reference threw: %s\n", e.what());
        return 1;
    }
    g_json << "\n}\n";
    {
        std::ofstream f(argv[1]);
        f << g_json.str();
    }
    if (!time_out.empty()) {
        g_time_json << "{\n";
        try {
            time_case("n8192_a1", 8192, {60, 40, 40, 60}, 1, s40, range_steps(1, 15), 20);
            time_case("n32768_a1", 32768, {60, 40, 40, 60}, 1, s40, range_steps(1, 15), 20);
            time_case("n65536_a1", 65536, {60, 40, 40, 60}, 1, s40, range_steps(1, 15), 20);
            time_case("n65536_a8", 65536, wide, 8, s50, {1}, 10);
        } catch (const std::exception &e) {
            fprintf(stderr, "reference threw while timing: %s\n", e.what());
            return 1;
        }
        g_time_json << "\n}\n";
        std::ofstream f(time_out);
        f << g_time_json.str();
    }
    return 0;
}
