// The primitive-chain configuration written against the C++ layer the way
// cahel-main/examples/4_ckks_basics.cu writes it against the reference: encode, encrypt,
// multiply, relinearize, rescale, rotate, hoisting, decrypt, decode; results must match the
// plaintext computation within 1e-3 (cahel-main/examples/example.h:14-19).  Exit code 0 = pass.
#include <cstdio>

#include "cahel_b200.hpp"

using namespace cahel;

static double max_err(const std::vector<double> &got, const std::vector<double> &want)
{
    double e = 0;
    for (size_t i = 0; i < want.size(); ++i) e = std::fmax(e, std::fabs(got[i] - want[i]));
    return e;
}

int main()
{
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
        printf("multiply %.3g rotate %.3g hoisting %.3g refused %d\n", e1, e2, e3, (int)threw);
        return (e1 < 1e-3 && e2 < 1e-3 && e3 < 1e-3 && threw) ? 0 : 1;
    } catch (const std::exception &e) {
        printf("exception: %s\n", e.what());
        return 2;
    }
}
