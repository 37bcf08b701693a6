// C++ host layer with CAHEL's names and signatures over the C ABI (lancelot_b200.h).
//
// It mirrors the CKKS part of cahel-main/include/{cahel,context,gpucontext,ciphertext,plaintext,
// secretkey,ckks,evaluate}.h: same type names, same argument order (context first, output last and
// mutated in place), value semantics (deep copy on copy), std::invalid_argument for parameter /
// level / scale mismatches and std::logic_error for missing keys or CUDA failures
// (cahel-main/include/common.h:50-62).  Header only; link against liblancelot_b200.so and cudart.
// The pybind module of the reference (cahel-main/python/src/binding.cu) compiles against these
// classes unchanged for the CKKS entry points it exports.
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <array>
#include <functional>
#include <istream>
#include <map>
#include <memory>
#include <ostream>
#include <random>
#include <stdexcept>
#include <vector>

#include "lancelot_b200.h"

namespace cahel {

enum class scheme_type : std::uint8_t { none = 0x0, bgv = 0x1, bfv = 0x2, ckks = 0x3 };
enum class mul_tech_type : std::uint8_t { none = 0x0, behz = 0x1, hps = 0x2, hps_overq = 0x3, hps_overq_leveled = 0x4 };
enum class sec_level_type : int { none = 0, tc128 = 128, tc192 = 192, tc256 = 256 };

class Modulus {
public:
    Modulus(std::uint64_t v = 0) : value_(v) {}
    std::uint64_t value() const { return value_; }

private:
    std::uint64_t value_;
};

struct CoeffModulus {
    // cahel-main/src/modulus.cu:93-125
    static std::vector<Modulus> Create(std::size_t poly_modulus_degree, std::vector<int> bit_sizes)
    {
        std::vector<std::uint64_t> out(bit_sizes.size());
        int rc = lb_coeff_modulus_create(poly_modulus_degree, bit_sizes.data(), (int)bit_sizes.size(), out.data());
        if (rc == LB_ERR_INVALID_ARG) throw std::invalid_argument(lb_last_error());
        if (rc != LB_OK) throw std::logic_error(lb_last_error());
        return std::vector<Modulus>(out.begin(), out.end());
    }
};

class EncryptionParameters {
public:
    explicit EncryptionParameters(scheme_type scheme) : scheme_(scheme) {}
    void set_mul_tech(mul_tech_type t) { mul_tech_ = t; }
    void set_poly_modulus_degree(std::size_t n) { n_ = n; }
    void set_special_modulus_size(std::size_t k) { special_ = k; }
    void set_galois_elts(const std::vector<std::uint32_t> &e) { elts_ = e; }
    void set_coeff_modulus(const std::vector<Modulus> &m) { moduli_ = m; }
    scheme_type scheme() const { return scheme_; }
    std::size_t poly_modulus_degree() const { return n_; }
    std::size_t special_modulus_size() const { return special_; }
    const std::vector<Modulus> &coeff_modulus() const { return moduli_; }
    const std::vector<std::uint32_t> &galois_elts() const { return elts_; }

private:
    scheme_type scheme_;
    mul_tech_type mul_tech_ = mul_tech_type::none;
    std::size_t n_ = 0, special_ = 1;
    std::vector<Modulus> moduli_;
    std::vector<std::uint32_t> elts_;
};

} // namespace cahel

// cahel-main/include/galois.cuh:155-192
inline std::vector<std::uint32_t> get_elts_from_steps(const std::vector<int> &steps, std::size_t coeff_count)
{
    std::vector<std::uint32_t> out(steps.size());
    int rc = lb_galois_elts_from_steps(steps.data(), (int)steps.size(), coeff_count, out.data());
    if (rc != LB_OK) throw std::invalid_argument(lb_last_error());
    return out;
}

namespace cahel_b200 {

inline void check(int rc)
{
    if (rc == LB_OK) return;
    if (rc == LB_ERR_INVALID_ARG) throw std::invalid_argument(lb_last_error());
    throw std::logic_error(lb_last_error());
}

inline void cuda_check(cudaError_t e)
{
    if (e != cudaSuccess) throw std::logic_error(std::string("CUDA error: ") + cudaGetErrorString(e));
}

// Seeds: the reference reads std::random_device for every key and encryption
// (cahel-main/include/prng.cuh:12-23).  A replacement source makes runs reproducible.
using SeedSource = std::function<void(std::uint8_t *out, std::size_t n_seeds)>;
inline void system_seeds(std::uint8_t *out, std::size_t n)
{
    std::random_device rd("/dev/urandom");
    for (std::size_t i = 0; i < n * 16; ++i) {
        std::uint32_t w = rd();
        std::memcpy(out + 4 * i, &w, 4);
    }
}
inline SeedSource &seed_source()
{
    static SeedSource src = system_seeds;
    return src;
}
inline void set_seed_source(SeedSource s) { seed_source() = s ? std::move(s) : SeedSource(system_seeds); }
inline void reset_seed_source() { seed_source() = system_seeds; }
inline std::vector<std::uint8_t> seeds(std::size_t n)
{
    std::vector<std::uint8_t> s(64 * n);
    seed_source()(s.data(), n);
    return s;
}

// Device blocks are recycled instead of being handed back to the driver: like the reference's global memory pool
// (cahel-main/include/mempool.cuh:471-492,600-606), a container that goes out of scope returns its block to a
// free list, bucketed by size (powers of two from 256 bytes), and the next container of that bucket takes it
// without a cudaMalloc / cudaFree (both synchronise the device).  Every call of this layer runs on the default
// stream, so a recycled block is never handed out while earlier work on it is still queued behind later work.
// Single-threaded use, like the reference's pool.  trim() frees what is cached.
class DevicePool {
public:
    static DevicePool &instance()
    {
        static DevicePool pool;
        return pool;
    }
    static std::size_t bucket_bytes(std::size_t bytes)
    {
        std::size_t b = 256;
        while (b < bytes) b <<= 1;
        return b;
    }
    void *take(std::size_t bytes)
    {
        const std::size_t b = bucket_bytes(bytes);
        int dev = 0;
        cuda_check(cudaGetDevice(&dev));
        auto &list = free_[{dev, b}];
        if (!list.empty()) {
            void *p = list.back();
            list.pop_back();
            cached_ -= b;
            ++reused_;
            return p;
        }
        void *p = nullptr;
        cudaError_t e = cudaMalloc(&p, b);
        if (e != cudaSuccess) { // give cached blocks back to the driver and try once more
            (void)cudaGetLastError();
            trim();
            cuda_check(cudaMalloc(&p, b));
        }
        ++allocated_;
        owner_[p] = {dev, b};
        return p;
    }
    void give(void *p)
    {
        auto it = owner_.find(p);
        if (it == owner_.end()) return;
        free_[it->second].push_back(p);
        cached_ += it->second.second;
    }
    void trim()
    {
        for (auto &kv : free_) {
            for (void *p : kv.second) {
                owner_.erase(p);
                cudaFree(p);
            }
            kv.second.clear();
        }
        cached_ = 0;
    }
    std::size_t device_allocations() const { return allocated_; }
    std::size_t reuses() const { return reused_; }
    std::size_t cached_bytes() const { return cached_; }
    ~DevicePool() { trim(); }

private:
    DevicePool() = default;
    std::map<std::pair<int, std::size_t>, std::vector<void *>> free_;
    std::map<void *, std::pair<int, std::size_t>> owner_;
    std::size_t cached_ = 0, allocated_ = 0, reused_ = 0;
};

// device array of 64-bit words with value semantics, backed by the pool
class DeviceWords {
public:
    DeviceWords() = default;
    explicit DeviceWords(std::size_t n) { resize(n); }
    DeviceWords(const DeviceWords &o) { *this = o; }
    DeviceWords(DeviceWords &&o) noexcept : p_(o.p_), n_(o.n_), cap_(o.cap_) { o.p_ = nullptr; o.n_ = 0; o.cap_ = 0; }
    DeviceWords &operator=(const DeviceWords &o)
    {
        if (this != &o) {
            resize(o.n_);
            if (n_) cuda_check(cudaMemcpyAsync(p_, o.p_, n_ * 8, cudaMemcpyDeviceToDevice, nullptr));
        }
        return *this;
    }
    DeviceWords &operator=(DeviceWords &&o) noexcept
    {
        if (this != &o) {
            release();
            p_ = o.p_; n_ = o.n_; cap_ = o.cap_;
            o.p_ = nullptr; o.n_ = 0; o.cap_ = 0;
        }
        return *this;
    }
    ~DeviceWords() { release(); }
    // contents are not kept; a block whose bucket already fits is reused as it is
    void resize(std::size_t n)
    {
        if (n == n_) return;
        if (n && p_ && DevicePool::bucket_bytes(n * 8) == cap_) {
            n_ = n;
            return;
        }
        release();
        if (n) {
            cap_ = DevicePool::bucket_bytes(n * 8);
            p_ = static_cast<std::uint64_t *>(DevicePool::instance().take(n * 8));
        }
        n_ = n;
    }
    std::uint64_t *get() const { return p_; }
    std::size_t size() const { return n_; }

private:
    void release()
    {
        if (p_) DevicePool::instance().give(p_);
        p_ = nullptr;
        n_ = 0;
        cap_ = 0;
    }
    std::uint64_t *p_ = nullptr;
    std::size_t n_ = 0, cap_ = 0;
};

} // namespace cahel_b200

// ---- byte streams in the reference's own format ----------------------------------------------
namespace cahel {
using parms_id_type = std::array<std::uint64_t, 4>;
}

namespace cahel_b200 {

// BLAKE2b (RFC 7693), unkeyed, 32-byte digest: the hash behind the reference's parms_id
// (cahel-main/include/util/hash.h:22-38)
inline cahel::parms_id_type blake2b_256(const std::uint8_t *in, std::size_t len)
{
    static const std::uint64_t iv[8] = {0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL, 0xa54ff53a5f1d36f1ULL,
                                        0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL, 0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};
    static const std::uint8_t sigma[12][16] = {
        {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
        {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
        {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
        {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
        {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0},
        {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3}};
    auto rotr = [](std::uint64_t x, int n) { return (x >> n) | (x << (64 - n)); };
    std::uint64_t h[8];
    for (int i = 0; i < 8; ++i) h[i] = iv[i];
    h[0] ^= 0x01010000ULL ^ 32; // digest length 32, no key, fanout = depth = 1
    auto compress = [&](const std::uint8_t *block, std::uint64_t t, bool last) {
        std::uint64_t m[16], v[16];
        for (int i = 0; i < 16; ++i) {
            m[i] = 0;
            for (int b = 7; b >= 0; --b) m[i] = (m[i] << 8) | block[8 * i + b];
        }
        for (int i = 0; i < 8; ++i) {
            v[i] = h[i];
            v[i + 8] = iv[i];
        }
        v[12] ^= t;
        if (last) v[14] = ~v[14];
        auto g = [&](int a, int b, int c, int d, std::uint64_t x, std::uint64_t y) {
            v[a] = v[a] + v[b] + x; v[d] = rotr(v[d] ^ v[a], 32);
            v[c] = v[c] + v[d];     v[b] = rotr(v[b] ^ v[c], 24);
            v[a] = v[a] + v[b] + y; v[d] = rotr(v[d] ^ v[a], 16);
            v[c] = v[c] + v[d];     v[b] = rotr(v[b] ^ v[c], 63);
        };
        for (int r = 0; r < 12; ++r) {
            const std::uint8_t *s = sigma[r];
            g(0, 4, 8, 12, m[s[0]], m[s[1]]);   g(1, 5, 9, 13, m[s[2]], m[s[3]]);
            g(2, 6, 10, 14, m[s[4]], m[s[5]]);  g(3, 7, 11, 15, m[s[6]], m[s[7]]);
            g(0, 5, 10, 15, m[s[8]], m[s[9]]);  g(1, 6, 11, 12, m[s[10]], m[s[11]]);
            g(2, 7, 8, 13, m[s[12]], m[s[13]]); g(3, 4, 9, 14, m[s[14]], m[s[15]]);
        }
        for (int i = 0; i < 8; ++i) h[i] ^= v[i] ^ v[i + 8];
    };
    std::uint8_t block[128];
    std::size_t off = 0;
    while (len - off > 128) {
        compress(in + off, off + 128, false);
        off += 128;
    }
    std::memset(block, 0, sizeof(block));
    std::memcpy(block, in + off, len - off);
    compress(block, len, true);
    return {h[0], h[1], h[2], h[3]};
}

// parms_id of a chain level (cahel-main/include/util/encryptionparams.h:337-381): scheme, N, number of
// special primes, every prime of the key level, the primes in use at the level, and a zero plain modulus
inline cahel::parms_id_type parms_id_of(std::size_t n, const std::vector<std::uint64_t> &moduli, std::size_t size_p, std::size_t size_l_or_all)
{
    std::vector<std::uint64_t> w = {3 /* scheme_type::ckks */, (std::uint64_t)n, (std::uint64_t)size_p};
    w.insert(w.end(), moduli.begin(), moduli.end());
    w.insert(w.end(), moduli.begin(), moduli.begin() + size_l_or_all);
    w.push_back(0);
    return blake2b_256(reinterpret_cast<const std::uint8_t *>(w.data()), w.size() * 8); // little-endian host, as the reference assumes
}

template <class T>
inline void put(std::ostream &s, const T &v) { s.write(reinterpret_cast<const char *>(&v), sizeof(T)); }
template <class T>
inline T get(std::istream &s)
{
    T v{};
    s.read(reinterpret_cast<char *>(&v), sizeof(T));
    if (!s) throw std::runtime_error("I/O error");
    return v;
}

inline void put_words(std::ostream &s, const std::uint64_t *dev, std::size_t n)
{
    std::vector<std::uint64_t> h(n);
    if (n) cuda_check(cudaMemcpy(h.data(), dev, n * 8, cudaMemcpyDeviceToHost));
    put<std::uint64_t>(s, n);
    s.write(reinterpret_cast<const char *>(h.data()), (std::streamsize)(n * 8));
    if (!s) throw std::runtime_error("I/O error");
}

inline void get_words(std::istream &s, DeviceWords &dst, std::size_t expect)
{
    if (get<std::uint64_t>(s) != expect) throw std::invalid_argument("stream does not match the context");
    std::vector<std::uint64_t> h(expect);
    s.read(reinterpret_cast<char *>(h.data()), (std::streamsize)(expect * 8));
    if (!s) throw std::runtime_error("I/O error");
    dst.resize(expect);
    if (expect) cuda_check(cudaMemcpy(dst.get(), h.data(), expect * 8, cudaMemcpyHostToDevice));
}

} // namespace cahel_b200

// ---- context and containers -------------------------------------------------------------------

// cahel-main/include/gpucontext.h:15-136.  chain index 0 = key level, 1 = first data level,
// each further index drops one prime (cahel-main/src/context.cu:352-403).
struct CAHELGPUContext {
    lb_context *lb_handle_ = nullptr;
    std::size_t poly_degree_ = 0, size_QP_ = 0, size_P_ = 0, size_Q_ = 0;
    std::vector<std::uint64_t> moduli_;
    std::vector<std::uint32_t> galois_elts_;
    bool expand_mod_chain_ = true;

    CAHELGPUContext(const cahel::EncryptionParameters &parms, bool expand_mod_chain = true,
                    cahel::sec_level_type sec_level = cahel::sec_level_type::tc128, int device = -1)
    {
        if (parms.scheme() != cahel::scheme_type::ckks) throw std::invalid_argument("unsupported scheme");
        poly_degree_ = parms.poly_modulus_degree();
        int log_n = 0;
        while ((std::size_t(1) << log_n) < poly_degree_) ++log_n;
        if (poly_degree_ < 16 || (std::size_t(1) << log_n) != poly_degree_) throw std::invalid_argument("invalid poly_modulus_degree");
        for (auto &m : parms.coeff_modulus()) moduli_.push_back(m.value());
        size_QP_ = moduli_.size();
        size_P_ = size_QP_ > 1 ? parms.special_modulus_size() : 0;
        size_Q_ = size_QP_ - size_P_;
        galois_elts_ = parms.galois_elts();
        expand_mod_chain_ = expand_mod_chain;
        if (device < 0) cahel_b200::cuda_check(cudaGetDevice(&device));
        cahel_b200::check(lb_context_create(log_n, moduli_.data(), (int)size_QP_, (int)size_P_, galois_elts_.data(),
                                            (int)galois_elts_.size(), sec_level != cahel::sec_level_type::none, device, &lb_handle_));
    }
    CAHELGPUContext(const CAHELGPUContext &) = delete;
    CAHELGPUContext &operator=(const CAHELGPUContext &) = delete;
    ~CAHELGPUContext() { lb_context_destroy(lb_handle_); }

    std::size_t max_chain() const { return expand_mod_chain_ ? size_Q_ : 1; }
    int size_l(std::size_t chain_index) const
    {
        if (chain_index == 0) return (int)size_Q_;
        if (chain_index > max_chain()) throw std::invalid_argument("chain_index is out of range");
        return (int)(size_Q_ - (chain_index - 1));
    }
    int total_bits(std::size_t chain_index) const
    {
        long double p = 1.0L;
        const std::size_t n = chain_index == 0 ? size_QP_ : (std::size_t)size_l(chain_index);
        for (std::size_t i = 0; i < n; ++i) p *= (long double)moduli_[i];
        int e = 0;
        std::frexp(p, &e);
        return e;
    }
    int elt_index(std::uint32_t elt) const
    {
        for (std::size_t i = 0; i < galois_elts_.size(); ++i)
            if (galois_elts_[i] == elt) return (int)i;
        return -1;
    }
    cahel::parms_id_type parms_id(std::size_t chain_index) const
    {
        return cahel_b200::parms_id_of(poly_degree_, moduli_, size_P_, chain_index == 0 ? size_QP_ : (std::size_t)size_l(chain_index));
    }
};

// cahel-main/include/plaintext.h:11
struct CAHELGPUPlaintext {
    cahel_b200::DeviceWords data_;
    std::size_t chain_index_ = 0, coeff_modulus_size_ = 0, poly_modulus_degree_ = 0;
    double scale_ = 1.0;
    bool is_ntt_form_ = true;
    CAHELGPUPlaintext() = default;
    explicit CAHELGPUPlaintext(const CAHELGPUContext &) {}
    std::uint64_t *data() const { return data_.get(); }
    std::size_t &chain_index() { return chain_index_; }
    std::size_t chain_index() const { return chain_index_; }
    double &scale() { return scale_; }
    double scale() const { return scale_; }
    bool is_ntt_form() const { return is_ntt_form_; }
    // cahel-main/include/plaintext.h:109-213, byte for byte.  The reference's save() takes no context
    // because its containers keep the parms_id; these look it up in the context.
    void save(const CAHELGPUContext &context, std::ostream &stream) const
    {
        const std::size_t limbs = (std::size_t)context.size_l(chain_index_), n = context.poly_degree_;
        cahel_b200::put(stream, context.parms_id(chain_index_));
        cahel_b200::put<std::uint64_t>(stream, limbs);
        cahel_b200::put<std::uint64_t>(stream, chain_index_);
        cahel_b200::put<std::uint64_t>(stream, n);
        cahel_b200::put(stream, scale_);
        cahel_b200::put_words(stream, data_.get(), limbs * n);
    }
    void load(const CAHELGPUContext &context, std::istream &stream)
    {
        const auto id = cahel_b200::get<cahel::parms_id_type>(stream);
        const auto limbs = cahel_b200::get<std::uint64_t>(stream), chain = cahel_b200::get<std::uint64_t>(stream),
                   n = cahel_b200::get<std::uint64_t>(stream);
        const double scale = cahel_b200::get<double>(stream);
        if (n != context.poly_degree_ || chain > context.max_chain() || limbs != (std::uint64_t)context.size_l(chain) ||
            id != context.parms_id(chain))
            throw std::invalid_argument("plaintext data is invalid");
        cahel_b200::get_words(stream, data_, limbs * n);
        chain_index_ = chain; coeff_modulus_size_ = limbs; poly_modulus_degree_ = n; scale_ = scale; is_ntt_form_ = true;
    }
};

// cahel-main/include/ciphertext.h:7
struct CAHELGPUCiphertext {
    cahel_b200::DeviceWords data_;
    std::size_t size_ = 0, chain_index_ = 0, coeff_modulus_size_ = 0, poly_modulus_degree_ = 0;
    double scale_ = 1.0;
    bool is_ntt_form_ = true;
    CAHELGPUCiphertext() = default;
    explicit CAHELGPUCiphertext(const CAHELGPUContext &) {}
    std::uint64_t *data() const { return data_.get(); }
    std::size_t size() const { return size_; }
    std::size_t &chain_index() { return chain_index_; }
    std::size_t chain_index() const { return chain_index_; }
    double &scale() { return scale_; }
    double scale() const { return scale_; }
    void set_scale(double s) { scale_ = s; }
    bool is_ntt_form() const { return is_ntt_form_; }
    // ciphertext.h:303-351: new shape; the words are left for the caller to fill
    void resize(const CAHELGPUContext &context, std::size_t chain_index, std::size_t size)
    {
        size_ = size;
        chain_index_ = chain_index;
        coeff_modulus_size_ = (std::size_t)context.size_l(chain_index);
        poly_modulus_degree_ = context.poly_degree_;
        data_.resize(size_ * coeff_modulus_size_ * poly_modulus_degree_);
    }
    // cahel-main/include/ciphertext.h:174-292, byte for byte (the trailing 64-byte seed block is zero,
    // as the reference leaves it); see CAHELGPUPlaintext::save for the context argument
    void save(const CAHELGPUContext &context, std::ostream &stream) const
    {
        const std::size_t limbs = (std::size_t)context.size_l(chain_index_), n = context.poly_degree_;
        cahel_b200::put(stream, context.parms_id(chain_index_));
        cahel_b200::put(stream, is_ntt_form_);
        cahel_b200::put<std::uint64_t>(stream, chain_index_);
        cahel_b200::put<std::uint64_t>(stream, size_);
        cahel_b200::put<std::uint64_t>(stream, n);
        cahel_b200::put<std::uint64_t>(stream, limbs);
        cahel_b200::put(stream, scale_);
        cahel_b200::put_words(stream, data_.get(), size_ * limbs * n);
        const char seed[64] = {0};
        stream.write(seed, sizeof(seed));
        if (!stream) throw std::runtime_error("I/O error");
    }
    void load(const CAHELGPUContext &context, std::istream &stream)
    {
        const auto id = cahel_b200::get<cahel::parms_id_type>(stream);
        const bool ntt = cahel_b200::get<bool>(stream);
        const auto chain = cahel_b200::get<std::uint64_t>(stream), size = cahel_b200::get<std::uint64_t>(stream),
                   n = cahel_b200::get<std::uint64_t>(stream), limbs = cahel_b200::get<std::uint64_t>(stream);
        const double scale = cahel_b200::get<double>(stream);
        if (n != context.poly_degree_ || chain > context.max_chain() || limbs != (std::uint64_t)context.size_l(chain) || size < 2 ||
            id != context.parms_id(chain))
            throw std::invalid_argument("ciphertext data is invalid");
        cahel_b200::get_words(stream, data_, size * limbs * n);
        char seed[64];
        stream.read(seed, sizeof(seed));
        if (!stream) throw std::runtime_error("I/O error");
        size_ = size; chain_index_ = chain; coeff_modulus_size_ = limbs; poly_modulus_degree_ = n; scale_ = scale; is_ntt_form_ = ntt;
    }
};

struct CAHELGPUPublicKey {
    cahel_b200::DeviceWords pk_;
    CAHELGPUPublicKey() = default;
    explicit CAHELGPUPublicKey(const CAHELGPUContext &) {}
    // cahel-main/include/secretkey.h:54-60: the pair as a size-2 ciphertext over all primes; the reference
    // writes the key level's parms_id with chain index 1 and scale 1
    void save(const CAHELGPUContext &context, std::ostream &stream) const
    {
        if (!pk_.size()) throw std::logic_error("public key has not been generated");
        const std::size_t n = context.poly_degree_;
        cahel_b200::put(stream, context.parms_id(0));
        cahel_b200::put(stream, true);
        cahel_b200::put<std::uint64_t>(stream, 1);
        cahel_b200::put<std::uint64_t>(stream, 2);
        cahel_b200::put<std::uint64_t>(stream, n);
        cahel_b200::put<std::uint64_t>(stream, context.size_QP_);
        cahel_b200::put(stream, 1.0);
        cahel_b200::put_words(stream, pk_.get(), 2 * context.size_QP_ * n);
        const char seed[64] = {0};
        stream.write(seed, sizeof(seed));
        if (!stream) throw std::runtime_error("I/O error");
    }
    void load(const CAHELGPUContext &context, std::istream &stream)
    {
        const auto id = cahel_b200::get<cahel::parms_id_type>(stream);
        (void)cahel_b200::get<bool>(stream);
        (void)cahel_b200::get<std::uint64_t>(stream);
        const auto size = cahel_b200::get<std::uint64_t>(stream), n = cahel_b200::get<std::uint64_t>(stream),
                   limbs = cahel_b200::get<std::uint64_t>(stream);
        (void)cahel_b200::get<double>(stream);
        if (n != context.poly_degree_ || limbs != context.size_QP_ || size != 2 || id != context.parms_id(0))
            throw std::invalid_argument("public key data is invalid");
        cahel_b200::get_words(stream, pk_, 2 * limbs * n);
        char seed[64];
        stream.read(seed, sizeof(seed));
        if (!stream) throw std::runtime_error("I/O error");
    }
    // cahel-main/src/secretkey.cu:179-249; only plaintexts of the first data level, like the reference
    void encrypt_asymmetric(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, CAHELGPUCiphertext &cipher,
                            bool save_seed = false) const
    {
        (void)save_seed;
        if (!pk_.size()) throw std::logic_error("public key has not been generated");
        if (!plain.is_ntt_form()) throw std::invalid_argument("CKKS plain must be in NTT form");
        if (plain.chain_index() != 1) throw std::invalid_argument("asymmetric encryption expects a plaintext at the first data level");
        cipher.resize(context, 1, 2);
        auto s = cahel_b200::seeds(2);
        cahel_b200::check(lb_encrypt_asymmetric(context.lb_handle_, pk_.get(), plain.data(), s.data(), 1, cipher.data(), nullptr));
        cipher.scale() = plain.scale();
    }
    CAHELGPUCiphertext encrypt_asymmetric(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, bool save_seed = false) const
    {
        CAHELGPUCiphertext c(context);
        encrypt_asymmetric(context, plain, c, save_seed);
        return c;
    }
};

struct CAHELGPURelinKey {
    cahel_b200::DeviceWords keys_; // [dnum][2][size_QP][N]
    CAHELGPURelinKey() = default;
    explicit CAHELGPURelinKey(const CAHELGPUContext &) {}
    // cahel-main/include/secretkey.h:212-256: key-level parms_id, generated flag, pair count, then every key pair as a
    // size-2 ciphertext stream over all primes with chain index 0 and scale 1 (seed block zero)
    void save(const CAHELGPUContext &context, std::ostream &stream) const
    {
        if (!keys_.size()) throw std::logic_error("relinearization key has not been generated");
        const std::size_t n = context.poly_degree_, pair = 2 * context.size_QP_ * n, dnum = keys_.size() / pair;
        cahel_b200::put(stream, context.parms_id(0));
        cahel_b200::put(stream, true);
        cahel_b200::put<std::uint64_t>(stream, dnum);
        for (std::size_t j = 0; j < dnum; ++j) {
            cahel_b200::put(stream, context.parms_id(0));
            cahel_b200::put(stream, true);
            cahel_b200::put<std::uint64_t>(stream, 0);
            cahel_b200::put<std::uint64_t>(stream, 2);
            cahel_b200::put<std::uint64_t>(stream, n);
            cahel_b200::put<std::uint64_t>(stream, context.size_QP_);
            cahel_b200::put(stream, 1.0);
            cahel_b200::put_words(stream, keys_.get() + j * pair, pair);
            const char seed[64] = {0};
            stream.write(seed, sizeof(seed));
        }
        if (!stream) throw std::runtime_error("I/O error");
    }
    void load(const CAHELGPUContext &context, std::istream &stream)
    {
        const std::size_t n = context.poly_degree_, pair = 2 * context.size_QP_ * n;
        const auto id = cahel_b200::get<cahel::parms_id_type>(stream);
        (void)cahel_b200::get<bool>(stream);
        const auto dnum = cahel_b200::get<std::uint64_t>(stream);
        if (id != context.parms_id(0) || dnum != context.size_Q_ / context.size_P_) throw std::invalid_argument("relinearization key data is invalid");
        cahel_b200::DeviceWords all(dnum * pair), one;
        for (std::uint64_t j = 0; j < dnum; ++j) {
            const auto pid = cahel_b200::get<cahel::parms_id_type>(stream);
            (void)cahel_b200::get<bool>(stream);
            (void)cahel_b200::get<std::uint64_t>(stream);
            const auto size = cahel_b200::get<std::uint64_t>(stream), pn = cahel_b200::get<std::uint64_t>(stream),
                       limbs = cahel_b200::get<std::uint64_t>(stream);
            (void)cahel_b200::get<double>(stream);
            if (pid != id || size != 2 || pn != n || limbs != context.size_QP_) throw std::invalid_argument("relinearization key data is invalid");
            cahel_b200::get_words(stream, one, pair);
            cahel_b200::cuda_check(cudaMemcpy(all.get() + j * pair, one.get(), pair * 8, cudaMemcpyDeviceToDevice));
            char seed[64];
            stream.read(seed, sizeof(seed));
            if (!stream) throw std::runtime_error("I/O error");
        }
        keys_ = std::move(all);
    }
};

struct CAHELGPUGaloisKey {
    std::vector<CAHELGPURelinKey> relin_keys_; // one per Galois element of the context
    CAHELGPUGaloisKey() = default;
    explicit CAHELGPUGaloisKey(const CAHELGPUContext &) {}
    // cahel-main/include/secretkey.h:354-400: key-level parms_id, generated flag, key count, then one
    // relinearization-key stream per Galois element
    void save(const CAHELGPUContext &context, std::ostream &stream) const
    {
        if (relin_keys_.empty()) throw std::logic_error("Galois keys have not been generated");
        cahel_b200::put(stream, context.parms_id(0));
        cahel_b200::put(stream, true);
        cahel_b200::put<std::uint64_t>(stream, relin_keys_.size());
        for (const auto &k : relin_keys_) k.save(context, stream);
    }
    void load(const CAHELGPUContext &context, std::istream &stream)
    {
        const auto id = cahel_b200::get<cahel::parms_id_type>(stream);
        (void)cahel_b200::get<bool>(stream);
        const auto count = cahel_b200::get<std::uint64_t>(stream);
        if (id != context.parms_id(0) || count != context.galois_elts_.size()) throw std::invalid_argument("Galois key data is invalid");
        std::vector<CAHELGPURelinKey> keys(count);
        for (auto &k : keys) k.load(context, stream);
        relin_keys_ = std::move(keys);
    }
};

// cahel-main/include/secretkey.h, src/secretkey.cu:254-654
struct CAHELGPUSecretKey {
    std::vector<cahel_b200::DeviceWords> powers_; // s, s^2, ... at the key level
    explicit CAHELGPUSecretKey(const cahel::EncryptionParameters &) {}

    void gen_secretkey(const CAHELGPUContext &context)
    {
        powers_.assign(1, cahel_b200::DeviceWords(context.size_QP_ * context.poly_degree_));
        auto s = cahel_b200::seeds(1);
        cahel_b200::check(lb_gen_secret_key(context.lb_handle_, s.data(), powers_[0].get(), nullptr));
    }
    const std::uint64_t *secret_key_array() const
    {
        if (powers_.empty()) throw std::logic_error("cannot generate keys for unspecified secret key");
        return powers_[0].get();
    }
    const std::uint64_t *power(const CAHELGPUContext &context, std::size_t k)
    {
        secret_key_array();
        while (powers_.size() < k) {
            cahel_b200::DeviceWords next(context.size_QP_ * context.poly_degree_);
            cahel_b200::check(lb_multiply_poly_key_level(context.lb_handle_, powers_.back().get(), powers_[0].get(), next.get(), nullptr));
            powers_.push_back(std::move(next));
        }
        return powers_[k - 1].get();
    }
    void gen_publickey(const CAHELGPUContext &context, CAHELGPUPublicKey &pk, bool save_seed = true) const
    {
        (void)save_seed;
        pk.pk_.resize(2 * context.size_QP_ * context.poly_degree_);
        auto s = cahel_b200::seeds(2);
        cahel_b200::check(lb_gen_public_key(context.lb_handle_, secret_key_array(), s.data(), s.data() + 64, pk.pk_.get(), nullptr));
    }
    void gen_switch_key(const CAHELGPUContext &context, const std::uint64_t *target, CAHELGPURelinKey &out) const
    {
        const std::size_t dnum = context.size_Q_ / context.size_P_;
        out.keys_.resize(dnum * 2 * context.size_QP_ * context.poly_degree_);
        auto s = cahel_b200::seeds(2 * dnum);
        cahel_b200::check(lb_gen_switch_key(context.lb_handle_, secret_key_array(), target, s.data(), out.keys_.get(), nullptr));
    }
    void gen_relinkey(const CAHELGPUContext &context, CAHELGPURelinKey &rlk, bool save_seed = false)
    {
        (void)save_seed;
        gen_switch_key(context, power(context, 2), rlk);
    }
    void create_galois_keys(const CAHELGPUContext &context, CAHELGPUGaloisKey &glk, bool save_seed = false) const
    {
        (void)save_seed;
        glk.relin_keys_.assign(context.galois_elts_.size(), CAHELGPURelinKey());
        cahel_b200::DeviceWords rotated(context.size_QP_ * context.poly_degree_);
        for (std::size_t i = 0; i < context.galois_elts_.size(); ++i) {
            cahel_b200::check(lb_galois_permute(context.lb_handle_, (int)i, (int)context.size_QP_, secret_key_array(), rotated.get(), nullptr));
            gen_switch_key(context, rotated.get(), glk.relin_keys_[i]);
        }
    }
    // cahel-main/src/secretkey.cu:451-560: (c0, c1) = (-(a s + e) + pt, a) at the plaintext's level
    void encrypt_symmetric(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, CAHELGPUCiphertext &cipher,
                           bool save_seed = false) const
    {
        (void)save_seed;
        if (!plain.is_ntt_form()) throw std::invalid_argument("CKKS plain must be in NTT form");
        const int L = context.size_l(plain.chain_index());
        const std::size_t poly = (std::size_t)L * context.poly_degree_;
        cipher.resize(context, plain.chain_index(), 2);
        auto s = cahel_b200::seeds(2);
        cahel_b200::DeviceWords e(poly);
        std::uint64_t *c0 = cipher.data(), *a = cipher.data() + poly;
        cahel_b200::check(lb_sample_error(context.lb_handle_, s.data(), L, 0, e.get(), nullptr));
        cahel_b200::check(lb_ntt_forward(context.lb_handle_, e.get(), 1, L, 0, nullptr));
        cahel_b200::check(lb_sample_uniform(context.lb_handle_, s.data() + 64, L, 0, a, nullptr));
        // the first L limbs of the key-level secret are its data-level limbs
        cahel_b200::check(lb_multiply_poly(context.lb_handle_, L, 1, a, secret_key_array(), c0, nullptr));
        cahel_b200::check(lb_add(context.lb_handle_, L, 1, c0, e.get(), c0, nullptr));
        cahel_b200::check(lb_negate(context.lb_handle_, L, 1, c0, c0, nullptr));
        cahel_b200::check(lb_add(context.lb_handle_, L, 1, c0, plain.data(), c0, nullptr));
        cipher.scale() = plain.scale();
    }
    CAHELGPUCiphertext encrypt_symmetric(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, bool save_seed = false) const
    {
        CAHELGPUCiphertext c(context);
        encrypt_symmetric(context, plain, c, save_seed);
        return c;
    }
    // ckks_decrypt without the noise-flooding term
    void decrypt(const CAHELGPUContext &context, const CAHELGPUCiphertext &cipher, CAHELGPUPlaintext &plain)
    {
        if (!cipher.is_ntt_form()) throw std::invalid_argument("encrypted must be in NTT form");
        const int L = context.size_l(cipher.chain_index());
        power(context, cipher.size() > 1 ? cipher.size() - 1 : 1);
        plain.data_.resize((std::size_t)L * context.poly_degree_);
        if (cipher.size() <= 2) {
            cahel_b200::check(lb_decrypt(context.lb_handle_, L, (int)cipher.size(), cipher.data(), secret_key_array(), plain.data(), nullptr));
        } else {
            // c0 + sum_p c_p s^p with the key-level powers (the kernel's own s^p would use data-level strides)
            const std::size_t poly = (std::size_t)L * context.poly_degree_;
            cahel_b200::cuda_check(cudaMemcpy(plain.data(), cipher.data(), poly * 8, cudaMemcpyDeviceToDevice));
            cahel_b200::DeviceWords tmp(poly);
            for (std::size_t p = 1; p < cipher.size(); ++p) {
                cahel_b200::check(lb_multiply_poly(context.lb_handle_, L, 1, cipher.data() + p * poly, power(context, p), tmp.get(), nullptr));
                cahel_b200::check(lb_add(context.lb_handle_, L, 1, plain.data(), tmp.get(), plain.data(), nullptr));
            }
        }
        plain.chain_index() = cipher.chain_index();
        plain.scale() = cipher.scale();
        plain.coeff_modulus_size_ = (std::size_t)L;
        plain.poly_modulus_degree_ = context.poly_degree_;
    }
    CAHELGPUPlaintext decrypt(const CAHELGPUContext &context, const CAHELGPUCiphertext &cipher)
    {
        CAHELGPUPlaintext p(context);
        decrypt(context, cipher, p);
        return p;
    }
};

// cahel-main/include/ckks.h, src/ckks.cu
struct CAHELGPUCKKSEncoder {
    std::size_t slots_ = 0, sparse_slots_ = 0;
    explicit CAHELGPUCKKSEncoder(const CAHELGPUContext &context) : slots_(context.poly_degree_ / 2) {}
    std::size_t slot_count() const { return slots_; }
    void reset_sparse_slots() { sparse_slots_ = 0; }

    void encode(const CAHELGPUContext &context, const std::vector<double> &values, std::size_t chain_index, double scale,
                CAHELGPUPlaintext &destination)
    {
        if (values.size() > slots_) throw std::invalid_argument("values_size is too large");
        if (sparse_slots_ == 0) {
            sparse_slots_ = 1;
            while (sparse_slots_ < values.size()) sparse_slots_ <<= 1;
        } else if (values.size() > sparse_slots_) {
            throw std::invalid_argument("values_size exceeds previous message length");
        }
        if (sparse_slots_ < 2) throw std::invalid_argument("single value encoding is not available");
        const int L = context.size_l(chain_index);
        cahel_b200::DeviceWords staging(values.size() + 1); // pooled scratch: one word per double
        double *d_vals = reinterpret_cast<double *>(staging.get());
        cahel_b200::cuda_check(cudaMemcpy(d_vals, values.data(), values.size() * sizeof(double), cudaMemcpyHostToDevice));
        destination.data_.resize((std::size_t)L * context.poly_degree_);
        int rc = lb_encode(context.lb_handle_, L, d_vals, 0, values.size(), (int)values.size(), (int)sparse_slots_, 1, scale,
                           destination.data(), nullptr);
        if (rc == LB_OK) rc = lb_check_status(context.lb_handle_, nullptr);
        cahel_b200::check(rc);
        destination.chain_index() = chain_index;
        destination.scale() = scale;
        destination.coeff_modulus_size_ = (std::size_t)L;
        destination.poly_modulus_degree_ = context.poly_degree_;
    }
    void encode(const CAHELGPUContext &context, const std::vector<double> &values, double scale, CAHELGPUPlaintext &destination)
    {
        encode(context, values, 1, scale, destination);
    }
    CAHELGPUPlaintext encode(const CAHELGPUContext &context, const std::vector<double> &values, double scale)
    {
        CAHELGPUPlaintext p(context);
        encode(context, values, 1, scale, p);
        return p;
    }
    CAHELGPUPlaintext encode(const CAHELGPUContext &context, const std::vector<double> &values, std::size_t chain_index, double scale)
    {
        CAHELGPUPlaintext p(context);
        encode(context, values, chain_index, scale, p);
        return p;
    }
    void decode(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, std::vector<double> &destination)
    {
        if (!plain.is_ntt_form()) throw std::invalid_argument("plain is not in NTT form");
        if (sparse_slots_ == 0) sparse_slots_ = slots_;
        const int L = context.size_l(plain.chain_index());
        cahel_b200::DeviceWords staging(sparse_slots_ * 2); // pooled scratch for the complex slots
        double *d_out = reinterpret_cast<double *>(staging.get());
        int rc = lb_decode(context.lb_handle_, L, plain.data(), plain.scale(), (int)sparse_slots_, d_out, nullptr);
        std::vector<double> host(2 * sparse_slots_);
        if (rc == LB_OK) cahel_b200::cuda_check(cudaMemcpy(host.data(), d_out, host.size() * sizeof(double), cudaMemcpyDeviceToHost));
        cahel_b200::check(rc);
        destination.resize(sparse_slots_);
        for (std::size_t i = 0; i < sparse_slots_; ++i) destination[i] = host[2 * i];
    }
    std::vector<double> decode(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain)
    {
        std::vector<double> out;
        decode(context, plain, out);
        return out;
    }
};

// ---- evaluator (cahel-main/include/evaluate.h, src/evaluate.cu, src/eval_key_switch.cu) -----------

namespace cahel_b200 {
inline bool same_scale(double x, double y) { return std::fabs(x - y) <= 1e-9 * std::fmax(std::fmax(std::fabs(x), std::fabs(y)), 1.0); }
inline void check_same_level(const CAHELGPUCiphertext &a, const CAHELGPUCiphertext &b)
{
    if (a.chain_index() != b.chain_index()) throw std::invalid_argument("encrypted1 and encrypted2 parameter mismatch");
    if (a.is_ntt_form() != b.is_ntt_form()) throw std::invalid_argument("NTT form mismatch");
    if (!same_scale(a.scale(), b.scale())) throw std::invalid_argument("scale mismatch");
}
// cahel-main/include/context.h:644-660
inline void check_scale(const CAHELGPUContext &context, double scale, std::size_t chain_index)
{
    if (scale <= 0 || (int)std::log2(scale) >= context.total_bits(chain_index)) throw std::invalid_argument("scale out of bounds");
}
inline void addsub_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &a, const CAHELGPUCiphertext &b, bool add)
{
    check_same_level(a, b);
    const int L = context.size_l(a.chain_index());
    const std::size_t poly = (std::size_t)L * context.poly_degree_;
    const std::size_t k = a.size() < b.size() ? a.size() : b.size();
    if (a.size() < b.size()) { // the result takes the larger size: extra polynomials are (+/-) b's
        CAHELGPUCiphertext grown = b;
        if (!add) check(lb_negate(context.lb_handle_, L, (int)b.size(), b.data(), grown.data(), nullptr));
        check((add ? lb_add : lb_sub)(context.lb_handle_, L, (int)k, a.data(), b.data(), grown.data(), nullptr));
        grown.scale() = a.scale();
        a = std::move(grown);
        return;
    }
    (void)poly;
    check((add ? lb_add : lb_sub)(context.lb_handle_, L, (int)k, a.data(), b.data(), a.data(), nullptr));
}
} // namespace cahel_b200

inline void negate_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted)
{
    cahel_b200::check(lb_negate(context.lb_handle_, context.size_l(encrypted.chain_index()), (int)encrypted.size(), encrypted.data(),
                                encrypted.data(), nullptr));
}
inline void negate(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, CAHELGPUCiphertext &destination)
{
    destination = encrypted;
    negate_inplace(context, destination);
}
inline void add_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2)
{
    cahel_b200::addsub_inplace(context, encrypted1, encrypted2, true);
}
inline void add(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2,
                CAHELGPUCiphertext &destination)
{
    if (&destination == &encrypted2 && &destination != &encrypted1) {
        add_inplace(context, destination, encrypted1);
        return;
    }
    if (&destination != &encrypted1) destination = encrypted1;
    add_inplace(context, destination, encrypted2);
}
inline void sub_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2)
{
    cahel_b200::addsub_inplace(context, encrypted1, encrypted2, false);
}
// destination = encrypted1 - encrypted2 (cahel-main/include/evaluate.h:52-61)
inline void sub(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2,
                CAHELGPUCiphertext &destination)
{
    if (&destination == &encrypted2 && &destination != &encrypted1) {
        CAHELGPUCiphertext tmp = encrypted1;
        sub_inplace(context, tmp, encrypted2);
        destination = std::move(tmp);
        return;
    }
    if (&destination != &encrypted1) destination = encrypted1;
    sub_inplace(context, destination, encrypted2);
}
inline void add_many(const CAHELGPUContext &context, const std::vector<CAHELGPUCiphertext> &encrypteds, CAHELGPUCiphertext &destination)
{
    if (encrypteds.empty()) throw std::invalid_argument("encrypteds cannot be empty");
    CAHELGPUCiphertext acc = encrypteds[0];
    for (std::size_t i = 1; i < encrypteds.size(); ++i) add_inplace(context, acc, encrypteds[i]);
    destination = std::move(acc);
}
inline void add_plain_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, const CAHELGPUPlaintext &plain)
{
    if (encrypted.chain_index() != plain.chain_index()) throw std::invalid_argument("encrypted and plain parameter mismatch");
    if (!cahel_b200::same_scale(encrypted.scale(), plain.scale())) throw std::invalid_argument("scale mismatch");
    cahel_b200::check(lb_add(context.lb_handle_, context.size_l(encrypted.chain_index()), 1, encrypted.data(), plain.data(), encrypted.data(), nullptr));
}
inline void sub_plain_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, const CAHELGPUPlaintext &plain)
{
    if (encrypted.chain_index() != plain.chain_index()) throw std::invalid_argument("encrypted and plain parameter mismatch");
    if (!cahel_b200::same_scale(encrypted.scale(), plain.scale())) throw std::invalid_argument("scale mismatch");
    cahel_b200::check(lb_sub(context.lb_handle_, context.size_l(encrypted.chain_index()), 1, encrypted.data(), plain.data(), encrypted.data(), nullptr));
}
inline void multiply_plain_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, const CAHELGPUPlaintext &plain)
{
    if (encrypted.chain_index() != plain.chain_index()) throw std::invalid_argument("encrypted and plain parameter mismatch");
    cahel_b200::check_scale(context, encrypted.scale() * plain.scale(), encrypted.chain_index());
    const int L = context.size_l(encrypted.chain_index());
    const std::size_t poly = (std::size_t)L * context.poly_degree_;
    for (std::size_t p = 0; p < encrypted.size(); ++p)
        cahel_b200::check(lb_multiply_poly(context.lb_handle_, L, 1, encrypted.data() + p * poly, plain.data(), encrypted.data() + p * poly, nullptr));
    encrypted.scale() *= plain.scale();
}
// ckks_multiply (cahel-main/src/evaluate.cu:447-500) for two size-2 ciphertexts
inline void multiply_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2)
{
    if (encrypted1.chain_index() != encrypted2.chain_index()) throw std::invalid_argument("encrypted1 and encrypted2 parameter mismatch");
    if (encrypted1.size() != 2 || encrypted2.size() != 2) throw std::invalid_argument("only size-2 ciphertexts can be multiplied on this path");
    cahel_b200::check_scale(context, encrypted1.scale() * encrypted2.scale(), encrypted1.chain_index());
    CAHELGPUCiphertext out(context);
    out.resize(context, encrypted1.chain_index(), 3);
    cahel_b200::check(lb_multiply(context.lb_handle_, context.size_l(encrypted1.chain_index()), 1, encrypted1.data(), encrypted2.data(), out.data(), nullptr));
    out.scale() = encrypted1.scale() * encrypted2.scale();
    encrypted1 = std::move(out);
}
inline void multiply(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2,
                     CAHELGPUCiphertext &destination)
{
    CAHELGPUCiphertext tmp = encrypted1;
    multiply_inplace(context, tmp, encrypted2);
    destination = std::move(tmp);
}
inline void square_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted)
{
    CAHELGPUCiphertext copy = encrypted;
    multiply_inplace(context, encrypted, copy);
}
// cahel-main/src/evaluate.cu:2019-2056
inline void relinearize_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, const CAHELGPURelinKey &relin_keys)
{
    if (encrypted.size() != 3) throw std::invalid_argument("destination_size must be 3");
    if (!relin_keys.keys_.size()) throw std::invalid_argument("relin_keys is not valid for encryption parameters");
    const int L = context.size_l(encrypted.chain_index());
    cahel_b200::check(lb_relinearize(context.lb_handle_, L, encrypted.data(), relin_keys.keys_.get(), nullptr));
    CAHELGPUCiphertext out(context);
    out.resize(context, encrypted.chain_index(), 2);
    cahel_b200::cuda_check(cudaMemcpy(out.data(), encrypted.data(), out.data_.size() * 8, cudaMemcpyDeviceToDevice));
    out.scale() = encrypted.scale();
    encrypted = std::move(out);
}
inline void multiply_and_relin_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted1, const CAHELGPUCiphertext &encrypted2,
                                       const CAHELGPURelinKey &relin_keys)
{
    multiply_inplace(context, encrypted1, encrypted2);
    relinearize_inplace(context, encrypted1, relin_keys);
}
// cahel-main/src/evaluate.cu:2059,2307-2361
inline void rescale_to_next_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted)
{
    if (encrypted.chain_index() >= context.max_chain()) throw std::invalid_argument("end of modulus switching chain reached");
    const int L = context.size_l(encrypted.chain_index());
    CAHELGPUCiphertext out(context);
    out.resize(context, encrypted.chain_index() + 1, encrypted.size());
    cahel_b200::check(lb_rescale(context.lb_handle_, L, (int)encrypted.size(), encrypted.data(), out.data(), nullptr));
    out.scale() = encrypted.scale() / (double)context.moduli_[L - 1];
    encrypted = std::move(out);
}
// mod_switch_drop_to_next / mod_switch_to_inplace (cahel-main/src/evaluate.cu:2200-2300)
inline void mod_switch_to_next_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted)
{
    if (encrypted.chain_index() >= context.max_chain()) throw std::invalid_argument("end of modulus switching chain reached");
    const int L = context.size_l(encrypted.chain_index());
    CAHELGPUCiphertext out(context);
    out.resize(context, encrypted.chain_index() + 1, encrypted.size());
    cahel_b200::check(lb_mod_switch_drop(context.lb_handle_, L, (int)encrypted.size(), encrypted.data(), out.data(), nullptr));
    out.scale() = encrypted.scale();
    encrypted = std::move(out);
}
inline void mod_switch_to_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, std::size_t chain_index)
{
    if (encrypted.chain_index() > chain_index) throw std::invalid_argument("cannot switch to higher level modulus");
    while (encrypted.chain_index() < chain_index) mod_switch_to_next_inplace(context, encrypted);
}
// cahel-main/src/evaluate.cu:2631-2686
inline void apply_galois_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, std::size_t galois_elt_index,
                                 const CAHELGPUGaloisKey &galois_keys)
{
    if (encrypted.size() > 2) throw std::invalid_argument("encrypted size must be 2");
    if (galois_elt_index >= galois_keys.relin_keys_.size()) throw std::logic_error("Galois key not present");
    cahel_b200::check(lb_rotate(context.lb_handle_, context.size_l(encrypted.chain_index()), encrypted.data(), (int)galois_elt_index,
                                galois_keys.relin_keys_[galois_elt_index].keys_.get(), nullptr));
}
// rotate_internal (cahel-main/src/evaluate.cu:2364-2410): a direct key, else the non-adjacent form of the step
inline void rotate_vector_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, int step, const CAHELGPUGaloisKey &galois_key)
{
    if (step == 0) return;
    const int idx = context.elt_index(get_elts_from_steps({step}, context.poly_degree_)[0]);
    if (idx >= 0) {
        apply_galois_inplace(context, encrypted, (std::size_t)idx, galois_key);
        return;
    }
    std::vector<int> parts;
    {
        bool sign = step < 0;
        int v = std::abs(step);
        for (int i = 0; v; ++i) {
            int zi = (v & 1) ? 2 - (v & 3) : 0;
            v = (v - zi) >> 1;
            if (zi) parts.push_back((sign ? -zi : zi) * (1 << i)); // least significant first, the order the reference applies
        }
    }
    if (parts.size() == 1) throw std::invalid_argument("Galois key not present");
    for (int s : parts)
        if ((std::size_t)std::abs(s) != context.poly_degree_ / 2) rotate_vector_inplace(context, encrypted, s, galois_key);
}
inline void rotate_vector(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, int step, const CAHELGPUGaloisKey &galois_key,
                          CAHELGPUCiphertext &destination)
{
    destination = encrypted;
    rotate_vector_inplace(context, destination, step, galois_key);
}
// cahel-main/src/evaluate.cu:2412-2629
inline void hoisting_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &ct, const CAHELGPUGaloisKey &glk, const std::vector<int> &steps)
{
    if (ct.size() > 2) throw std::invalid_argument("ciphertext size must be 2");
    auto elts = get_elts_from_steps(steps, context.poly_degree_);
    std::vector<int> idx;
    std::vector<const std::uint64_t *> keys;
    for (auto e : elts) {
        int i = context.elt_index(e);
        if (i < 0) throw std::logic_error("Galois key not present in hoisting");
        idx.push_back(i);
        keys.push_back(glk.relin_keys_[(std::size_t)i].keys_.get());
    }
    cahel_b200::check(lb_hoisting(context.lb_handle_, context.size_l(ct.chain_index()), ct.data(), (int)idx.size(), idx.data(), keys.data(), nullptr));
}
inline CAHELGPUCiphertext hoisting(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, const CAHELGPUGaloisKey &glk,
                                   const std::vector<int> &steps)
{
    CAHELGPUCiphertext out = encrypted;
    hoisting_inplace(context, out, glk, steps);
    return out;
}

// ---- out-of-place forms and the remaining names of cahel-main/include/evaluate.h -------------------------------
// (the reference writes them as copy + in-place call, evaluate.h:35-61,120-160,383-400,566-600)
inline void add_plain(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, const CAHELGPUPlaintext &plain,
                      CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    add_plain_inplace(context, destination, plain);
}
inline void sub_plain(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, const CAHELGPUPlaintext &plain,
                      CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    sub_plain_inplace(context, destination, plain);
}
inline void multiply_plain(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, const CAHELGPUPlaintext &plain,
                           CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    multiply_plain_inplace(context, destination, plain);
}
inline void square(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    square_inplace(context, destination);
}
inline void relinearize(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, const CAHELGPURelinKey &relin_keys,
                        CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    relinearize_inplace(context, destination, relin_keys);
}
inline void rescale_to_next(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    rescale_to_next_inplace(context, destination);
}
inline void mod_switch_to_next(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    mod_switch_to_next_inplace(context, destination);
}
inline void mod_switch_to(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, CAHELGPUCiphertext &destination,
                          std::size_t chain_index)
{
    if (&destination != &encrypted) destination = encrypted;
    mod_switch_to_inplace(context, destination, chain_index);
}
// plaintexts in NTT form drop their last limb like ciphertexts do (cahel-main/src/evaluate.cu:2253-2300)
inline void mod_switch_to_next_inplace(const CAHELGPUContext &context, CAHELGPUPlaintext &plain)
{
    if (plain.chain_index() >= context.max_chain()) throw std::invalid_argument("end of modulus switching chain reached");
    const int L = context.size_l(plain.chain_index());
    cahel_b200::DeviceWords out((std::size_t)(L - 1) * context.poly_degree_);
    cahel_b200::check(lb_mod_switch_drop(context.lb_handle_, L, 1, plain.data(), out.get(), nullptr));
    plain.data_ = std::move(out);
    plain.chain_index() += 1;
    plain.coeff_modulus_size_ = (std::size_t)(L - 1);
}
inline void mod_switch_to_inplace(const CAHELGPUContext &context, CAHELGPUPlaintext &plain, std::size_t chain_index)
{
    if (plain.chain_index() > chain_index) throw std::invalid_argument("cannot switch to higher level modulus");
    while (plain.chain_index() < chain_index) mod_switch_to_next_inplace(context, plain);
}
inline void mod_switch_to_next(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, CAHELGPUPlaintext &destination)
{
    if (&destination != &plain) destination = plain;
    mod_switch_to_next_inplace(context, destination);
}
inline void mod_switch_to(const CAHELGPUContext &context, const CAHELGPUPlaintext &plain, CAHELGPUPlaintext &destination, std::size_t chain_index)
{
    if (&destination != &plain) destination = plain;
    mod_switch_to_inplace(context, destination, chain_index);
}
inline void apply_galois(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, std::size_t galois_elt_index,
                         const CAHELGPUGaloisKey &galois_keys, CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    apply_galois_inplace(context, destination, galois_elt_index, galois_keys);
}
// conjugation is the Galois element 2N - 1 (cahel-main/include/evaluate.h:577-600)
inline void complex_conjugate_inplace(const CAHELGPUContext &context, CAHELGPUCiphertext &encrypted, const CAHELGPUGaloisKey &galois_key)
{
    const int idx = context.elt_index((std::uint32_t)(2 * context.poly_degree_ - 1));
    if (idx < 0) throw std::logic_error("Galois key not present");
    apply_galois_inplace(context, encrypted, (std::size_t)idx, galois_key);
}
inline void complex_conjugate(const CAHELGPUContext &context, const CAHELGPUCiphertext &encrypted, const CAHELGPUGaloisKey &galois_key,
                              CAHELGPUCiphertext &destination)
{
    if (&destination != &encrypted) destination = encrypted;
    complex_conjugate_inplace(context, destination, galois_key);
}
// Names the reference exports for its BFV / BGV schemes or that fall outside the encrypted-aggregation path; they
// exist so that code written against the reference still links, and refuse at run time.
inline void rotate_rows_inplace(const CAHELGPUContext &, CAHELGPUCiphertext &, int, const CAHELGPUGaloisKey &)
{
    throw std::logic_error("unsupported scheme: rotate_rows is a BFV / BGV operation");
}
inline void rotate_rows(const CAHELGPUContext &, const CAHELGPUCiphertext &, int, const CAHELGPUGaloisKey &, CAHELGPUCiphertext &)
{
    throw std::logic_error("unsupported scheme: rotate_rows is a BFV / BGV operation");
}
inline void rotate_columns_inplace(const CAHELGPUContext &, CAHELGPUCiphertext &, const CAHELGPUGaloisKey &)
{
    throw std::logic_error("unsupported scheme: rotate_columns is a BFV / BGV operation");
}
inline void rotate_columns(const CAHELGPUContext &, const CAHELGPUCiphertext &, const CAHELGPUGaloisKey &, CAHELGPUCiphertext &)
{
    throw std::logic_error("unsupported scheme: rotate_columns is a BFV / BGV operation");
}
inline void exponentiate_inplace(const CAHELGPUContext &, CAHELGPUCiphertext &, std::uint64_t, const CAHELGPURelinKey &)
{
    throw std::logic_error("exponentiate is not part of the encrypted-aggregation path");
}
inline void exponentiate(const CAHELGPUContext &, const CAHELGPUCiphertext &, std::uint64_t, const CAHELGPURelinKey &, CAHELGPUCiphertext &)
{
    throw std::logic_error("exponentiate is not part of the encrypted-aggregation path");
}
inline void multiply_many(const CAHELGPUContext &, std::vector<CAHELGPUCiphertext> &, const CAHELGPURelinKey &, CAHELGPUCiphertext &)
{
    throw std::logic_error("multiply_many is not part of the encrypted-aggregation path");
}
