// extern "C" surface declared in include/lancelot_b200.h.  Argument validation lives here
// (the kernels trust their launchers); nothing below ever computes on the CPU.
#include <algorithm>
#include <cstring>
#include <vector>

#include "context.h"

namespace lb {
const std::string &last_error();
int context_create(int logN, const std::vector<u64> &moduli, int size_P, const std::vector<uint32_t> &elts, int device,
                   Context **out);
void context_destroy(Context *ctx);
} // namespace lb

using namespace lb;

struct lb_context {
    Context *c;
};

static inline Context *C(lb_context *h) { return h ? h->c : nullptr; }
namespace lb {
Context *lb_context_impl(lb_context *h) { return h ? h->c : nullptr; }
} // namespace lb
static inline const Context *C(const lb_context *h) { return h ? h->c : nullptr; }
static inline cudaStream_t S(void *s) { return reinterpret_cast<cudaStream_t>(s); }

#define REQUIRE(cond, msg)             \
    do {                               \
        if (!(cond)) {                 \
            set_error(msg);            \
            return LB_ERR_INVALID_ARG; \
        }                              \
    } while (0)

static int bind(lb_context *h)
{
    if (!h || !h->c) {
        set_error("context is null");
        return LB_ERR_INVALID_ARG;
    }
    LB_CUDA(cudaSetDevice(h->c->device));
    return LB_OK;
}

static int level_ok(const Context *c, int size_l)
{
    REQUIRE(size_l >= 1 && size_l <= c->hp.size_Q, "size_l is out of range for this context");
    return LB_OK;
}

extern "C" {

const char *lb_last_error(void) { return last_error().c_str(); }

int lb_coeff_modulus_create(uint64_t n, const int *bit_sizes, int count, uint64_t *out)
{
    REQUIRE(bit_sizes && out && count >= 1 && count <= 64, "bit_sizes is invalid");
    REQUIRE(n >= 16 && n <= 131072 && (n & (n - 1)) == 0, "poly_modulus_degree is invalid");
    std::vector<int> bits(bit_sizes, bit_sizes + count);
    for (int b : bits) REQUIRE(b >= 2 && b <= 60, "bit_sizes is invalid");
    std::vector<u64> m = coeff_modulus_create(n, bits);
    if (m.empty()) {
        set_error("failed to find enough qualifying primes");
        return LB_ERR_LOGIC;
    }
    std::memcpy(out, m.data(), sizeof(u64) * count);
    return LB_OK;
}

int lb_galois_elts_from_steps(const int *steps, int count, uint64_t n, uint32_t *out)
{
    REQUIRE(steps && out && count >= 0, "steps is invalid");
    for (int i = 0; i < count; ++i) {
        const long a = steps[i] < 0 ? -(long)steps[i] : steps[i];
        REQUIRE(a < (long)(n >> 1), "step count too large");
        out[i] = galois_elt_from_step(steps[i], n);
    }
    return LB_OK;
}

uint64_t lb_minimal_primitive_root(uint64_t degree, uint64_t modulus) { return minimal_primitive_root(degree, modulus); }

int lb_max_bit_count_tc128(uint64_t n) { return max_bit_count_tc128(n); }

int lb_context_create(int log_n, const uint64_t *moduli, int n_moduli, int special, const uint32_t *elts, int n_elts,
                      int check_tc128, int device, lb_context **out)
{
    REQUIRE(out, "out is null");
    *out = nullptr;
    REQUIRE(moduli && n_moduli >= 1 && n_moduli <= 64, "coeff_modulus size is invalid");
    REQUIRE(n_elts >= 0 && (n_elts == 0 || elts), "galois_elts is invalid");
    std::vector<u64> m(moduli, moduli + n_moduli);
    std::vector<uint32_t> e(elts, elts + n_elts);
    if (check_tc128) {
        int bits = 0;
        for (u64 v : m) bits += 64 - __builtin_clzll(v);
        const int bound = max_bit_count_tc128(u64(1) << log_n);
        REQUIRE(bound > 0 && bits <= bound, "invalid parameters_insecure");
    }
    Context *c = nullptr;
    int rc = context_create(log_n, m, special, e, device, &c);
    if (rc) return rc;
    *out = new lb_context{c};
    return LB_OK;
}

void lb_context_destroy(lb_context *h)
{
    if (!h) return;
    context_destroy(h->c);
    delete h;
}

int lb_context_get_modulus(const lb_context *h, int i, uint64_t *out)
{
    const Context *c = C(h);
    REQUIRE(c && out && i >= 0 && i < c->hp.size_QP, "modulus index is out of range");
    *out = c->hp.q[i];
    return LB_OK;
}

int lb_context_get_root(const lb_context *h, int i, uint64_t *out)
{
    const Context *c = C(h);
    REQUIRE(c && out && i >= 0 && i < c->hp.size_QP, "modulus index is out of range");
    *out = c->hp.psi[i];
    return LB_OK;
}

int lb_context_get_galois_table(const lb_context *h, int e, uint32_t *out)
{
    const Context *c = C(h);
    REQUIRE(c && out && e >= 0 && e < (int)c->hp.galois_elts.size(), "Galois element index is out of range");
    std::memcpy(out, &c->hp.perm[(size_t)e * c->hp.N], c->hp.N * sizeof(uint32_t));
    return LB_OK;
}

int lb_context_reserve_workspace(lb_context *h, size_t bytes)
{
    int rc = bind(h);
    if (rc) return rc;
    return C(h)->ensure_workspace(bytes);
}

size_t lb_keyswitch_workspace_bytes(const lb_context *h, int size_l)
{
    const Context *c = C(h);
    if (!c || size_l < 1 || size_l > c->hp.size_Q || c->hp.size_P < 1) return 0;
    return keyswitch_workspace_bytes(c, size_l);
}

static int ntt_rows(lb_context *h, uint64_t *data, int n_groups, int size_l, int size_p, bool fwd, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    Context *c = C(h);
    REQUIRE(data || n_groups == 0, "data is null");
    REQUIRE(n_groups >= 0 && size_l >= 0 && size_l <= c->hp.size_Q && size_p >= 0 && size_p <= c->hp.size_P && size_l + size_p >= 1,
            "limb counts are out of range for this context");
    NttJob job;
    job.src = data;
    job.dst = data;
    job.n_groups = n_groups;
    job.per_group = size_l + size_p;
    job.size_l = size_l;
    return fwd ? ntt_forward(c, job, S(stream)) : ntt_inverse(c, job, S(stream));
}

int lb_ntt_forward(lb_context *h, uint64_t *data, int n_groups, int size_l, int size_p, void *stream)
{
    return ntt_rows(h, data, n_groups, size_l, size_p, true, stream);
}

int lb_ntt_inverse(lb_context *h, uint64_t *data, int n_groups, int size_l, int size_p, void *stream)
{
    return ntt_rows(h, data, n_groups, size_l, size_p, false, stream);
}

static int binary(lb_context *h, int op, int size_l, int n_polys, const uint64_t *a, const uint64_t *b, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(n_polys >= 0 && a && out && (b || op == OP_NEG || op == OP_REDUCE), "operand is null");
    return poly_binary(C(h), op, size_l, (long)n_polys * size_l, a, b, out, S(stream));
}

int lb_add(lb_context *h, int size_l, int n, const uint64_t *a, const uint64_t *b, uint64_t *out, void *s) { return binary(h, OP_ADD, size_l, n, a, b, out, s); }
int lb_sub(lb_context *h, int size_l, int n, const uint64_t *a, const uint64_t *b, uint64_t *out, void *s) { return binary(h, OP_SUB, size_l, n, a, b, out, s); }
int lb_multiply_poly(lb_context *h, int size_l, int n, const uint64_t *a, const uint64_t *b, uint64_t *out, void *s) { return binary(h, OP_MUL, size_l, n, a, b, out, s); }
int lb_negate(lb_context *h, int size_l, int n, const uint64_t *a, uint64_t *out, void *s) { return binary(h, OP_NEG, size_l, n, a, nullptr, out, s); }
int lb_reduce_mod(lb_context *h, int size_l, int n, const uint64_t *a, uint64_t *out, void *s) { return binary(h, OP_REDUCE, size_l, n, a, nullptr, out, s); }

int lb_sum_groups(lb_context *h, int size_l, int n_polys, int n_groups, const int *offsets, const int *indices, int n_items,
                  const uint64_t *in, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(offsets && in && out && n_polys >= 1 && n_groups >= 0, "operand is null");
    if (n_groups == 0) return LB_OK;
    REQUIRE(n_groups <= 65535, "too many groups");
    REQUIRE(offsets[0] == 0, "offsets must start at 0");
    for (int g = 0; g < n_groups; ++g) REQUIRE(offsets[g + 1] >= offsets[g], "offsets must not decrease");
    REQUIRE(offsets[n_groups] == 0 || indices, "operand is null");
    for (int t = 0; t < offsets[n_groups]; ++t) REQUIRE(indices[t] >= 0 && indices[t] < n_items, "item index is out of range");
    return poly_sum_groups(C(h), size_l, (long)n_polys * size_l, n_groups, offsets, indices, in, out, S(stream));
}

int lb_multiply_poly_key_level(lb_context *h, const uint64_t *a, const uint64_t *b, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(a && b && out, "operand is null");
    // at the key level the limb list is Q || P, which is also the table order
    return poly_binary(C(h), OP_MUL, C(h)->hp.size_QP, C(h)->hp.size_QP, a, b, out, S(stream));
}

int lb_multiply(lb_context *h, int size_l, int batch, const uint64_t *a, const uint64_t *b, uint64_t *out3, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(a && b && out3 && batch >= 0, "operand is null");
    REQUIRE(out3 != a && out3 != b, "the size-3 result cannot alias an input");
    return poly_tensor(C(h), size_l, batch, a, b, out3, S(stream));
}

int lb_square(lb_context *h, int size_l, int batch, const uint64_t *a, uint64_t *out3, void *stream)
{
    return lb_multiply(h, size_l, batch, a, a, out3, stream);
}

int lb_mod_switch_drop(lb_context *h, int size_l, int n_polys, const uint64_t *in, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(size_l >= 2 && size_l <= C(h)->hp.size_Q, "end of modulus switching chain reached");
    REQUIRE(in && out && n_polys >= 1, "operand is null");
    return poly_drop_last(C(h), size_l, n_polys, in, out, S(stream));
}

int lb_galois_permute(lb_context *h, int elt, int n_limbs, const uint64_t *in, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(in && out && in != out && n_limbs >= 0, "operand is null or aliased");
    return poly_galois(C(h), elt, n_limbs, in, out, S(stream));
}

int lb_modup(lb_context *h, int size_l, const uint64_t *cks, uint64_t *digits, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(cks && digits, "operand is null");
    return modup(C(h), size_l, cks, digits, S(stream));
}

int lb_keyswitch_inner_product(lb_context *h, int size_l, const uint64_t *digits, const uint64_t *evk, uint64_t *cx, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(digits && evk && cx, "operand is null");
    // digits carries its own limbs here, so the "own" source is the digit buffer itself:
    // pass a pointer the kernel never dereferences differently by materialising the rows
    Context *c = C(h);
    if ((rc = level_ok(c, size_l))) return rc;
    // own limbs of digit j sit at digits[j][j*alpha ..]; gather them into the workspace tail
    const HostParams &hp = c->hp;
    const int LP = size_l + hp.size_P, alpha = hp.size_P;
    REQUIRE(alpha >= 1, "key switching needs at least one special prime");
    if ((rc = c->ensure_workspace(keyswitch_workspace_bytes(c, size_l)))) return rc;
    u64 *own = reinterpret_cast<u64 *>(c->ws); // the coefficient scratch is free at this point
    for (int j = 0; j < hp.level[size_l].beta; ++j) {
        const int s = j * alpha, e = s + alpha < size_l ? s + alpha : size_l;
        LB_CUDA(cudaMemcpyAsync(own + (size_t)s * hp.N, digits + ((size_t)j * LP + s) * hp.N, (size_t)(e - s) * hp.N * 8,
                                cudaMemcpyDeviceToDevice, S(stream)));
    }
    return inner_product(c, size_l, digits, own, evk, cx, S(stream));
}

int lb_moddown(lb_context *h, int size_l, const uint64_t *cx, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(cx && out, "operand is null");
    return moddown(C(h), size_l, cx, out, S(stream));
}

int lb_keyswitch(lb_context *h, int size_l, uint64_t *ct, const uint64_t *cks, const uint64_t *evk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct && cks && evk, "operand is null");
    const size_t poly = (size_t)size_l * C(h)->hp.N;
    return keyswitch(C(h), size_l, cks, evk, ct, ct + poly, ct, S(stream));
}

int lb_relinearize(lb_context *h, int size_l, uint64_t *ct3, const uint64_t *rlk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct3 && rlk, "operand is null");
    return relinearize(C(h), size_l, 1, ct3, rlk, S(stream));
}

int lb_relinearize_batch(lb_context *h, int size_l, int batch, uint64_t *ct3, const uint64_t *rlk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct3 && rlk && batch >= 0, "operand is null");
    if (batch == 0) return LB_OK;
    return relinearize(C(h), size_l, batch, ct3, rlk, S(stream));
}

int lb_rescale(lb_context *h, int size_l, int n_polys, const uint64_t *in, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(in && out && n_polys >= 1, "operand is null");
    return rescale(C(h), size_l, n_polys, 1, in, size_l, out, S(stream));
}

int lb_rescale_strided(lb_context *h, int size_l, int batch, int polys_per_ct, const uint64_t *in, size_t ct_stride, uint64_t *out,
                       void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(in && out && batch >= 0 && polys_per_ct >= 1, "operand is null");
    REQUIRE(ct_stride % C(h)->hp.N == 0, "ciphertext stride must be a whole number of limbs");
    if (batch == 0) return LB_OK;
    return rescale(C(h), size_l, batch, polys_per_ct, in, (long)(ct_stride / C(h)->hp.N), out, S(stream));
}

int lb_rescale_no_alloc(lb_context *h, int size_l, int n_polys, const uint64_t *in, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(in && out, "operand is null");
    return rescale_static(C(h), size_l, n_polys, in, out, S(stream));
}

size_t lb_rescale_no_alloc_max_words(void) { return rescale_static_max_words(); }

int lb_rotate(lb_context *h, int size_l, uint64_t *ct, int elt, const uint64_t *glk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct && glk, "operand is null");
    return rotate(C(h), size_l, 1, ct, elt, glk, S(stream));
}

int lb_rotate_batch(lb_context *h, int size_l, int batch, uint64_t *ct, int elt, const uint64_t *glk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct && glk && batch >= 0, "operand is null");
    if (batch == 0) return LB_OK;
    return rotate(C(h), size_l, batch, ct, elt, glk, S(stream));
}

int lb_hoisting(lb_context *h, int size_l, uint64_t *ct, int n_steps, const int *elts, const uint64_t *const *keys, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct && elts && keys, "operand is null");
    return hoisting(C(h), size_l, 1, ct, n_steps, elts, keys, S(stream));
}

int lb_hoisting_batch(lb_context *h, int size_l, int batch, uint64_t *ct, int n_steps, const int *elts, const uint64_t *const *keys,
                      void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(ct && elts && keys && batch >= 0, "operand is null");
    if (batch == 0) return LB_OK;
    return hoisting(C(h), size_l, batch, ct, n_steps, elts, keys, S(stream));
}

int lb_krum_accumulate(lb_context *h, int size_l, int n_chunks, const uint64_t *a, const uint64_t *b, size_t sa, size_t sb,
                       uint64_t *acc, int accumulate, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(a && b && acc && n_chunks >= 0, "operand is null");
    REQUIRE(sa % 2 == 0 && sb % 2 == 0, "chunk strides must be even");
    return krum_accumulate(C(h), size_l, n_chunks, a, b, (long)sa, (long)sb, acc, accumulate, S(stream));
}

int lb_krum_accumulate_tile(lb_context *h, int size_l, int n_chunks, int n_a, const uint64_t *const *a, int n_b,
                            const uint64_t *const *b, size_t chunk_stride, uint64_t *const *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(a && out && (b || n_b == 0) && n_chunks >= 0, "operand is null");
    REQUIRE(n_a >= 1 && n_a <= 4 && n_b >= 0 && n_b <= 4, "tile shape is out of range");
    for (int i = 0; i < n_a; ++i) REQUIRE(a[i], "operand is null");
    for (int i = 0; i < n_b; ++i) REQUIRE(b[i], "operand is null");
    const int n_pairs = n_b ? n_a * n_b : n_a * (n_a - 1) / 2;
    for (int i = 0; i < n_pairs && i < 8; ++i) REQUIRE(out[i], "operand is null");
    return krum_accumulate_tile(C(h), size_l, n_chunks, n_a, a, n_b, b, (long)chunk_stride, out, S(stream));
}

// The pair list of a round as tiles of lb_krum_accumulate_tile.  Clients are blocked by index in groups of four; a
// diagonal block whose pairs are all the pairs of its clients is one triangle, anything else is cut into rectangles of
// one or two first clients that share their set of second clients.
int lb_krum_pair_sums(lb_context *h, int size_l, int n_clients, const uint64_t *const *cts, int n_chunks, size_t chunk_stride,
                      int n_pairs, const int *pairs, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(cts && out && (pairs || n_pairs == 0) && n_chunks >= 0 && n_pairs >= 0 && n_clients >= 0, "operand is null");
    for (int p = 0; p < n_pairs; ++p) {
        const int i = pairs[2 * p], j = pairs[2 * p + 1];
        REQUIRE(i >= 0 && i < j && j < n_clients, "a pair is (i, j) with 0 <= i < j < n_clients");
        REQUIRE(cts[i] && cts[j], "operand is null");
    }
    constexpr int W = 4;
    const size_t acc_words = (size_t)3 * size_l * C(h)->hp.N;
    const int n_blocks = (n_clients + W - 1) / W;
    // slot[i * n_clients + j] = index of pair (i, j) in the caller's list, -1 if absent (a pair listed twice is refused)
    std::vector<int> slot((size_t)n_clients * n_clients, -1);
    for (int p = 0; p < n_pairs; ++p) {
        int &sl = slot[(size_t)pairs[2 * p] * n_clients + pairs[2 * p + 1]];
        REQUIRE(sl < 0, "a pair is listed twice");
        sl = p;
    }
    auto launch = [&](const std::vector<int> &rows, const std::vector<int> &cols) -> int {
        const uint64_t *a[4], *b[4];
        uint64_t *o[8];
        const int na = (int)rows.size(), nb = (int)cols.size();
        for (int r = 0; r < na; ++r) a[r] = cts[rows[r]];
        for (int c = 0; c < nb; ++c) b[c] = cts[cols[c]];
        int n = 0;
        if (nb == 0) {
            for (int r = 0; r < na; ++r)
                for (int c = r + 1; c < na; ++c) o[n++] = out + (size_t)slot[(size_t)rows[r] * n_clients + rows[c]] * acc_words;
        } else {
            for (int r = 0; r < na; ++r)
                for (int c = 0; c < nb; ++c) o[n++] = out + (size_t)slot[(size_t)rows[r] * n_clients + cols[c]] * acc_words;
        }
        return krum_accumulate_tile(C(h), size_l, n_chunks, na, a, nb, nb ? b : nullptr, (long)chunk_stride, o, S(stream));
    };
    for (int ga = 0; ga < n_blocks; ++ga) {
        for (int gb = ga; gb < n_blocks; ++gb) {
            // the block's pairs by first client
            std::vector<int> first;
            std::vector<std::vector<int>> second;
            int count = 0;
            std::vector<char> seen(n_clients, 0);
            std::vector<int> members;
            for (int i = ga * W; i < (ga + 1) * W && i < n_clients; ++i) {
                std::vector<int> cols;
                for (int j = gb * W; j < (gb + 1) * W && j < n_clients; ++j)
                    if (j > i && slot[(size_t)i * n_clients + j] >= 0) {
                        cols.push_back(j);
                        if (!seen[i]) seen[i] = 1, members.push_back(i);
                        if (!seen[j]) seen[j] = 1, members.push_back(j);
                    }
                if (!cols.empty()) {
                    first.push_back(i);
                    count += (int)cols.size();
                    second.push_back(cols);
                }
            }
            if (count == 0) continue;
            const int m = (int)members.size();
            if (ga == gb && count == m * (m - 1) / 2) {
                std::sort(members.begin(), members.end());
                if ((rc = launch(members, {}))) return rc;
                continue;
            }
            for (size_t k = 0; k < first.size();) {
                if (k + 1 < first.size() && second[k + 1] == second[k]) {
                    if ((rc = launch({first[k], first[k + 1]}, second[k]))) return rc;
                    k += 2;
                } else {
                    if ((rc = launch({first[k]}, second[k]))) return rc;
                    k += 1;
                }
            }
        }
    }
    return LB_OK;
}

// byzantine_fl.py:244-273 for a batch of pair sums: relinearize_inplace, rescale_to_next_inplace, hoisting over
// the first steps added to the ciphertext, then rotate_vector + add_inplace for every further step
int lb_krum_scores(lb_context *h, int size_l, int n_pairs, uint64_t *acc, const uint64_t *relin_key, int n_first, const int *first_elts,
                   const uint64_t *const *first_keys, int n_pow, const int *pow_elts, const uint64_t *const *pow_keys, uint64_t *scores,
                   void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(size_l >= 2, "the pair sums must have a level to rescale to");
    REQUIRE(acc && relin_key && scores && n_pairs >= 0 && n_first >= 0 && n_pow >= 0, "operand is null");
    REQUIRE((n_first == 0 || (first_elts && first_keys)) && (n_pow == 0 || (pow_elts && pow_keys)), "operand is null");
    if (n_pairs == 0) return LB_OK;
    Context *c = C(h);
    cudaStream_t st = S(stream);
    const int L = size_l - 1;
    if ((rc = relinearize(c, size_l, n_pairs, acc, relin_key, st))) return rc;
    if ((rc = rescale(c, size_l, n_pairs, 2, acc, 3L * size_l, scores, st))) return rc;
    // scores += hoisting(scores), scores += rotate(scores, step): the sums are formed inside the key switch's closing
    // transform (no copy of the batch, no separate addition)
    if (n_first > 0 && (rc = hoisting(c, L, n_pairs, scores, n_first, first_elts, first_keys, st, true))) return rc;
    for (int k = 0; k < n_pow; ++k)
        if ((rc = rotate(c, L, n_pairs, scores, pow_elts[k], pow_keys[k], st, true))) return rc;
    return LB_OK;
}

int lb_decrypt(lb_context *h, int size_l, int n_polys, const uint64_t *ct, const uint64_t *sk, uint64_t *pt, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(ct && sk && pt && n_polys >= 1, "operand is null");
    return poly_decrypt(C(h), size_l, n_polys, 1, ct, sk, pt, S(stream));
}

int lb_decrypt_batch(lb_context *h, int size_l, int n_polys, int batch, const uint64_t *ct, const uint64_t *sk, uint64_t *pt, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(ct && sk && pt && n_polys >= 1 && batch >= 0, "operand is null");
    if (batch == 0) return LB_OK;
    return poly_decrypt(C(h), size_l, n_polys, batch, ct, sk, pt, S(stream));
}

int lb_mask_accumulate(lb_context *h, int size_l, int n_clients, int n_chunks, const uint64_t *const *client_cts, size_t chunk_stride,
                       const uint64_t *masks, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(client_cts && masks && out && n_chunks >= 0, "operand is null");
    REQUIRE(chunk_stride % 2 == 0, "chunk stride must be even");
    return mask_accumulate(C(h), size_l, n_clients, n_chunks, client_cts, (long)chunk_stride, masks, out, S(stream));
}

// ---- samplers, keys, encryption ------------------------------------------------------------

static int stage_seeds(Context *c, const uint8_t *host_seeds, int n_seeds, uint32_t **d_seeds, u64 **scratch, size_t scratch_words,
                       cudaStream_t stream)
{
    // layout of the context scratch: [seeds][scratch_words]
    const size_t seed_bytes = ((size_t)n_seeds * 64 + 255) / 256 * 256;
    int rc = c->ensure_workspace(seed_bytes + scratch_words * 8);
    if (rc) return rc;
    *d_seeds = reinterpret_cast<uint32_t *>(c->ws);
    if (scratch) *scratch = reinterpret_cast<u64 *>(reinterpret_cast<uint8_t *>(c->ws) + seed_bytes);
    LB_CUDA(cudaMemcpyAsync(*d_seeds, host_seeds, (size_t)n_seeds * 64, cudaMemcpyHostToDevice, stream));
    return LB_OK;
}

int lb_sample_ternary(lb_context *h, const uint8_t *seed, int size_l, int size_p, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(seed && out, "operand is null");
    uint32_t *ds;
    if ((rc = stage_seeds(C(h), seed, 1, &ds, nullptr, 0, S(stream)))) return rc;
    return sample_small(C(h), 0, ds, 16, 1, size_l, size_p, out, S(stream));
}

int lb_sample_error(lb_context *h, const uint8_t *seed, int size_l, int size_p, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(seed && out, "operand is null");
    uint32_t *ds;
    if ((rc = stage_seeds(C(h), seed, 1, &ds, nullptr, 0, S(stream)))) return rc;
    return sample_small(C(h), 1, ds, 16, 1, size_l, size_p, out, S(stream));
}

int lb_sample_uniform(lb_context *h, const uint8_t *seed, int size_l, int size_p, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(seed && out, "operand is null");
    REQUIRE(C(h)->hp.logN >= 3, "ring degree too small");
    uint32_t *ds;
    if ((rc = stage_seeds(C(h), seed, 1, &ds, nullptr, 0, S(stream)))) return rc;
    return sample_uniform(C(h), ds, 16, 1, size_l, size_p, out, S(stream));
}

int lb_gen_secret_key(lb_context *h, const uint8_t *seed, uint64_t *sk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(seed && sk, "operand is null");
    Context *c = C(h);
    uint32_t *ds;
    if ((rc = stage_seeds(c, seed, 1, &ds, nullptr, 0, S(stream)))) return rc;
    if ((rc = sample_small(c, 0, ds, 16, 1, c->hp.size_Q, c->hp.size_P, sk, S(stream)))) return rc;
    NttJob j;
    j.src = sk;
    j.dst = sk;
    j.n_groups = 1;
    j.per_group = c->hp.size_QP;
    j.size_l = c->hp.size_Q;
    return ntt_forward(c, j, S(stream));
}

int lb_gen_public_key(lb_context *h, const uint64_t *sk, const uint8_t *seed_error, const uint8_t *seed_uniform, uint64_t *pk, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(sk && seed_error && seed_uniform && pk, "operand is null");
    Context *c = C(h);
    uint8_t both[128];
    memcpy(both, seed_error, 64);
    memcpy(both + 64, seed_uniform, 64);
    uint32_t *ds;
    u64 *scratch;
    if ((rc = stage_seeds(c, both, 2, &ds, &scratch, (size_t)c->hp.size_QP << c->hp.logN, S(stream)))) return rc;
    // the staged copy must not be overwritten by `both` going out of scope: pageable copies complete before return
    return gen_public_key(c, sk, ds, ds + 16, pk, scratch, S(stream));
}

int lb_gen_switch_key(lb_context *h, const uint64_t *sk, const uint64_t *sk_target, const uint8_t *seeds, uint64_t *out, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(sk && sk_target && seeds && out, "operand is null");
    Context *c = C(h);
    REQUIRE(c->hp.size_P >= 1 && c->hp.size_Q % c->hp.size_P == 0, "special_modulus_size must divide the number of data primes");
    const int dnum = c->hp.size_Q / c->hp.size_P;
    uint32_t *ds;
    u64 *scratch;
    if ((rc = stage_seeds(c, seeds, 2 * dnum, &ds, &scratch, (size_t)c->hp.size_QP << c->hp.logN, S(stream)))) return rc;
    return gen_switch_key(c, sk, sk_target, ds, out, scratch, S(stream));
}

int lb_gen_galois_keys(lb_context *h, const uint64_t *sk, int n_keys, const int *elt_indices, const uint8_t *seeds, uint64_t *out,
                       void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(sk && seeds && out && n_keys >= 0 && (elt_indices || n_keys == 0), "operand is null");
    if (n_keys == 0) return LB_OK;
    Context *c = C(h);
    REQUIRE(c->hp.size_P >= 1 && c->hp.size_Q % c->hp.size_P == 0, "special_modulus_size must divide the number of data primes");
    for (int k = 0; k < n_keys; ++k)
        REQUIRE(elt_indices[k] >= 0 && elt_indices[k] < (int)c->hp.galois_elts.size(), "Galois element index is out of range");
    const int dnum = c->hp.size_Q / c->hp.size_P;
    const size_t poly = (size_t)c->hp.size_QP << c->hp.logN;
    uint32_t *ds;
    u64 *scratch;
    // scratch: the rotated secret keys [n][QP][N], then one error polynomial per key and digit
    if ((rc = stage_seeds(c, seeds, 2 * dnum * n_keys, &ds, &scratch, poly * (size_t)n_keys * (1 + dnum), S(stream)))) return rc;
    u64 *targets = scratch, *errors = scratch + poly * n_keys;
    for (int k = 0; k < n_keys; ++k)
        if ((rc = poly_galois(c, elt_indices[k], c->hp.size_QP, sk, targets + poly * k, S(stream)))) return rc;
    return gen_switch_keys(c, sk, targets, n_keys, ds, out, errors, S(stream));
}

int lb_encrypt_asymmetric(lb_context *h, const uint64_t *pk, const uint64_t *pt, const uint8_t *seeds, int batch, uint64_t *ct, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(pk && seeds && ct && batch >= 0, "operand is null");
    if (batch == 0) return LB_OK;
    return encrypt_asymmetric(C(h), pk, pt, 0, seeds, batch, ct, S(stream));
}

int lb_encode_encrypt(lb_context *h, const uint64_t *pk, const void *values, int dtype, size_t value_stride, int n_values,
                      int sparse_slots, int batch, double scale, const uint8_t *seeds, uint64_t *ct, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    REQUIRE(pk && seeds && ct && batch >= 0 && (values || n_values == 0), "operand is null");
    REQUIRE(dtype >= 0 && dtype <= 2, "unknown value type");
    if (batch == 0) return LB_OK;
    Context *c = C(h);
    const int Q = c->hp.size_Q;
    // coefficient-form plaintexts live behind the encryption scratch
    const size_t enc_bytes = (encrypt_workspace_bytes(c, batch) + 255) / 256 * 256;
    const size_t pt_bytes = ((size_t)batch * Q << c->hp.logN) * 8;
    if ((rc = c->ensure_workspace(enc_bytes + pt_bytes))) return rc;
    u64 *pt = reinterpret_cast<u64 *>(reinterpret_cast<uint8_t *>(c->ws) + enc_bytes);
    if ((rc = encode(c, Q, values, dtype, (long)value_stride, n_values, sparse_slots, batch, scale, pt, c->d_status, 1, S(stream)))) return rc;
    return encrypt_asymmetric(c, pk, pt, 1, seeds, batch, ct, S(stream));
}

// ---- encoder ------------------------------------------------------------------------------

int lb_encode(lb_context *h, int size_l, const void *values, int dtype, size_t value_stride, int n_values, int sparse_slots, int batch,
              double scale, uint64_t *pt, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE((values || n_values == 0) && pt && batch >= 0 && n_values >= 0, "values cannot be null");
    REQUIRE(dtype >= 0 && dtype <= 2, "unknown value type");
    return encode(C(h), size_l, values, dtype, (long)value_stride, n_values, sparse_slots, batch, scale, pt, C(h)->d_status, 0, S(stream));
}

int lb_decode(lb_context *h, int size_l, const uint64_t *pt, double scale, int sparse_slots, double *out_complex, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(pt && out_complex, "destination cannot be null");
    return decode(C(h), size_l, 1, pt, scale, sparse_slots, out_complex, S(stream));
}

int lb_decode_batch(lb_context *h, int size_l, int batch, const uint64_t *pt, double scale, int sparse_slots, double *out_complex, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    if ((rc = level_ok(C(h), size_l))) return rc;
    REQUIRE(pt && out_complex && batch >= 0, "destination cannot be null");
    if (batch == 0) return LB_OK;
    return decode(C(h), size_l, batch, pt, scale, sparse_slots, out_complex, S(stream));
}

int lb_check_status(lb_context *h, void *stream)
{
    int rc = bind(h);
    if (rc) return rc;
    int flags = 0;
    LB_CUDA(cudaMemcpyAsync(&flags, C(h)->d_status, sizeof(int), cudaMemcpyDeviceToHost, S(stream)));
    LB_CUDA(cudaStreamSynchronize(S(stream)));
    if (flags) {
        LB_CUDA(cudaMemsetAsync(C(h)->d_status, 0, sizeof(int), S(stream)));
        if (flags & 1) {
            set_error("encoded values are too large");
            return LB_ERR_INVALID_ARG;
        }
        set_error("device-side status flag raised");
        return LB_ERR_LOGIC;
    }
    return LB_OK;
}

} // extern "C"
