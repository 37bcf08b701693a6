// The primitive-chain configuration written against the C++ layer the way
// cahel-main/examples/4_ckks_basics.cu writes it against the reference: encode, encrypt,
// multiply, relinearize, rescale, rotate, hoisting, decrypt, decode; results must match the
// plaintext computation within 1e-3 (cahel-main/examples/example.h:14-19).  Exit code 0 = pass.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>

#include "cahel_b200.hpp"

using namespace cahel;

static double max_err(const std::vector<double> &got, const std::vector<double> &want)
{
    double e = 0;
    for (size_t i = 0; i < want.size(); ++i) e = std::fmax(e, std::fabs(got[i] - want[i]));
    return e;
}

// host-only mode: cpp_api_check --parms-id N size_P chain_index q0 q1 ...  prints the 32 digest bytes in hex
static int print_parms_id(int argc, char **argv)
{
    if (argc < 6) return 2;
    const size_t n = std::strtoull(argv[2], nullptr, 10), size_p = std::strtoull(argv[3], nullptr, 10), chain = std::strtoull(argv[4], nullptr, 10);
    std::vector<uint64_t> moduli;
    for (int i = 5; i < argc; ++i) moduli.push_back(std::strtoull(argv[i], nullptr, 10));
    const size_t size_q = moduli.size() - size_p;
    const auto id = cahel_b200::parms_id_of(n, moduli, size_p, chain == 0 ? moduli.size() : size_q - (chain - 1));
    const unsigned char *b = reinterpret_cast<const unsigned char *>(id.data());
    for (int i = 0; i < 32; ++i) printf("%02x", b[i]);
    printf("\n");
    return 0;
}

static std::vector<uint64_t> words_of(const uint64_t *dev, size_t n)
{
    std::vector<uint64_t> h(n);
    cudaMemcpy(h.data(), dev, n * 8, cudaMemcpyDeviceToHost);
    return h;
}

int main(int argc, char **argv)
{
    if (argc > 1 && std::string(argv[1]) == "--parms-id") return print_parms_id(argc, argv);
    try {
        const size_t n = 8192, slots = n / 2;
        EncryptionParameters parms(scheme_type::ckks);
        parms.set_poly_modulus_degree(n);
        parms.set_coeff_modulus(CoeffModulus::Create(n, {60, 40, 40, 60}));
        parms.set_special_modulus_size(1);
        parms.set_galois_elts(get_elts_from_steps({1, 2, 3}, n));
        CAHELGPUContext context(parms, true, sec_level_type::tc128);
        CAHELGPUSecretKey sk(parms);
        sk.gen_secretkey(context);
        CAHELGPUPublicKey pk(context);
        sk.gen_publickey(context, pk);
        CAHELGPURelinKey rlk(context);
        sk.gen_relinkey(context, rlk);
        CAHELGPUGaloisKey glk(context);
        sk.create_galois_keys(context, glk);
        CAHELGPUCKKSEncoder encoder(context);
        const double scale = std::pow(2.0, 40);
        std::vector<double> x(slots), y(slots), xy(slots);
        for (size_t i = 0; i < slots; ++i) {
            x[i] = std::sin(0.37 * i);
            y[i] = std::cos(0.11 * i);
            xy[i] = x[i] * y[i];
        }
        CAHELGPUPlaintext px(context), py(context);
        encoder.encode(context, x, scale, px);
        encoder.encode(context, y, scale, py);
        CAHELGPUCiphertext cx(context), cy(context);
        pk.encrypt_asymmetric(context, px, cx);
        pk.encrypt_asymmetric(context, py, cy);
        multiply_inplace(context, cx, cy);
        relinearize_inplace(context, cx, rlk);
        rescale_to_next_inplace(context, cx);
        double e1 = max_err(encoder.decode(context, sk.decrypt(context, cx)), xy);
        CAHELGPUCiphertext rot(context);
        rotate_vector(context, cx, 1, glk, rot);
        std::vector<double> want(slots);
        for (size_t i = 0; i < slots; ++i) want[i] = xy[(i + 1) % slots];
        double e2 = max_err(encoder.decode(context, sk.decrypt(context, rot)), want);
        CAHELGPUCiphertext h = hoisting(context, cx, glk, {1, 2, 3});
        for (size_t i = 0; i < slots; ++i) want[i] = xy[(i + 1) % slots] + xy[(i + 2) % slots] + xy[(i + 3) % slots];
        double e3 = max_err(encoder.decode(context, sk.decrypt(context, h)), want);
        bool threw = false;
        try {
            relinearize_inplace(context, cy, rlk); // size 2: must be refused like the reference does
        } catch (const std::invalid_argument &) {
            threw = true;
        }
        // streams in the reference's layout: several objects in one stream, loaded back word for word
        std::stringstream wire(std::ios::in | std::ios::out | std::ios::binary);
        px.save(context, wire);
        cx.save(context, wire);
        pk.save(context, wire);
        CAHELGPUPlaintext px2;
        CAHELGPUCiphertext cx2;
        CAHELGPUPublicKey pk2;
        px2.load(context, wire);
        cx2.load(context, wire);
        pk2.load(context, wire);
        const size_t limbs2 = (size_t)context.size_l(cx.chain_index());
        bool same = words_of(px2.data(), 3 * n) == words_of(px.data(), 3 * n) &&
                    words_of(cx2.data(), 2 * limbs2 * n) == words_of(cx.data(), 2 * limbs2 * n) &&
                    words_of(pk2.pk_.get(), 2 * 4 * n) == words_of(pk.pk_.get(), 2 * 4 * n) && cx2.chain_index() == cx.chain_index() &&
                    cx2.size() == 2 && cx2.scale() == cx.scale() && px2.scale() == px.scale();
        bool refused_stream = false;
        try {
            std::stringstream bad(wire.str().substr(1), std::ios::in | std::ios::binary); // shifted: parms_id cannot match
            CAHELGPUPlaintext p3;
            p3.load(context, bad);
        } catch (const std::invalid_argument &) {
            refused_stream = true;
        }
        // relinearization and Galois key streams: saved, loaded, and the loaded keys give the same ciphertext words
        std::stringstream kwire(std::ios::in | std::ios::out | std::ios::binary);
        rlk.save(context, kwire);
        glk.save(context, kwire);
        CAHELGPURelinKey rlk2;
        CAHELGPUGaloisKey glk2;
        rlk2.load(context, kwire);
        glk2.load(context, kwire);
        CAHELGPUCiphertext m1(context), m2(context);
        {
            CAHELGPUCiphertext a(context), b(context);
            pk.encrypt_asymmetric(context, px, a);
            pk.encrypt_asymmetric(context, py, b);
            multiply(context, a, b, m1);
            m2 = m1;
            relinearize_inplace(context, m1, rlk);
            relinearize_inplace(context, m2, rlk2);
            rotate_vector_inplace(context, m1, 2, glk);
            rotate_vector_inplace(context, m2, 2, glk2);
        }
        const bool keys_same = words_of(m1.data(), 2 * 3 * n) == words_of(m2.data(), 2 * 3 * n);
        // steady state: a loop of evaluator calls takes its blocks from the pool, not from the driver
        const size_t allocs_before = cahel_b200::DevicePool::instance().device_allocations();
        for (int it = 0; it < 20; ++it) {
            CAHELGPUCiphertext t(context), r(context);
            multiply(context, cx2, cx2, t);
            relinearize_inplace(context, t, rlk);
            rotate_vector(context, t, 1, glk, r);
            CAHELGPUCiphertext hs = hoisting(context, r, glk, {1, 2, 3});
            (void)encoder.decode(context, sk.decrypt(context, hs));
        }
        const size_t new_allocs = cahel_b200::DevicePool::instance().device_allocations() - allocs_before;
        // the first pass may still meet sizes it has not seen; twenty passes must not keep allocating
        const bool pooled = new_allocs <= 8 && cahel_b200::DevicePool::instance().reuses() > 100;
        if (const char *path = std::getenv("CPP_API_CHECK_STREAM")) {
            std::ofstream f(path, std::ios::binary);
            const std::string b = wire.str();
            f.write(b.data(), (std::streamsize)b.size());
        }
        printf("multiply %.3g rotate %.3g hoisting %.3g refused %d streams %d bad-stream-refused %d key-streams %d pooled %d (new device allocations %zu)\n",
               e1, e2, e3, (int)threw, (int)same, (int)refused_stream, (int)keys_same, (int)pooled, new_allocs);
        return (e1 < 1e-3 && e2 < 1e-3 && e3 < 1e-3 && threw && same && refused_stream && keys_same && pooled) ? 0 : 1;
    } catch (const std::exception &e) {
        printf("exception: %s\n", e.what());
        return 2;
    }
}
