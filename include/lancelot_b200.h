/*
 * lancelot_b200 - C ABI of the B200 (sm_100a) CKKS encrypted-aggregation path.
 *
 * This is the boundary a binding of the reference's C++ API (cahel-main/include/*.h) or of
 * its Python module (cahel-main/python/src/binding.cu) calls instead of launching the
 * reference's own kernels.  Plain pointers and sizes only.  Unless stated otherwise every
 * `uint64_t *` argument is DEVICE memory holding residues in [0, q) in the reference's
 * layouts (cahel-main/include/ciphertext.h:7, plaintext.h:11):
 *
 *   polynomial  [limb][N]            ciphertext  [poly][limb][N]
 *   key pair    [2][size_QP][N]      switch key  [dnum][2][size_QP][N]   (b then a)
 *   mod-up      [beta][size_l + size_P][N]
 *
 * `size_l` is the number of data primes of the operand's level (size_Q at chain index 1,
 * one fewer per rescale).  All calls are asynchronous on `stream` (a cudaStream_t passed as
 * void *, NULL = default stream) and return 0 on success or one of the LB_ERR_* codes; the
 * message of the last failure on the calling thread is available from lb_last_error().
 * LB_ERR_INVALID_ARG marks the conditions where the reference throws std::invalid_argument,
 * LB_ERR_LOGIC / LB_ERR_CUDA where it throws std::logic_error (cahel-main/include/common.h:50-62).
 * The library never falls back to the CPU: without a usable GPU every compute call fails.
 *
 * Every call on a context uses that context's scratch workspace and tables; calls on one context
 * must therefore be issued on ONE stream (or be ordered by the caller with events).  Use one context
 * per concurrent stream.  A call makes the context's device current for the calling thread.
 * Benchmark diagnostics (launch counter, per-kernel timer, butterfly-rate probe) are declared in
 * lancelot_b200_diag.h and are not part of this boundary.
 */
#ifndef LANCELOT_B200_H
#define LANCELOT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LB_API __attribute__((visibility("default")))
#else
#define LB_API
#endif

#define LB_OK 0
#define LB_ERR_INVALID_ARG 1
#define LB_ERR_LOGIC 2
#define LB_ERR_CUDA 3
#define LB_ERR_NO_MEMORY 4

typedef struct lb_context lb_context;

LB_API const char *lb_last_error(void);

/* ---- host-only parameter helpers (no GPU needed) ---------------------------------------- */

/* cahel::CoeffModulus::Create (cahel-main/src/modulus.cu:93-125; pyCAHEL coeff_modulus_create,
 * binding.cu:34): one NTT-friendly prime per requested bit size, largest first. */
LB_API int lb_coeff_modulus_create(uint64_t poly_modulus_degree, const int *bit_sizes, int count, uint64_t *out_moduli);
/* get_elts_from_steps (cahel-main/include/galois.cuh:155-192; binding.cu:77). */
LB_API int lb_galois_elts_from_steps(const int *steps, int count, uint64_t poly_modulus_degree, uint32_t *out_elts);
/* Minimal primitive 2N-th root used for the NTT tables (cahel-main/src/util/numth.cu:311-333). */
LB_API uint64_t lb_minimal_primitive_root(uint64_t degree, uint64_t modulus);
/* CoeffModulus::MaxBitCount for sec_level_type::tc128 (cahel-main/include/util/hestdparms.h:16-38). */
LB_API int lb_max_bit_count_tc128(uint64_t poly_modulus_degree);

/* ---- context (replaces CAHELGPUContext, cahel-main/include/gpucontext.h:15-136) ------------ */

/* moduli: the key-level list Q || P as returned by lb_coeff_modulus_create; the last
 * special_modulus_size entries are the special primes.  galois_elts may be NULL.
 * check_tc128 != 0 rejects parameter sets above the 128-bit bound like
 * cahel-main/src/context.cu:181-186. */
LB_API int lb_context_create(int log_n, const uint64_t *moduli, int n_moduli, int special_modulus_size,
                      const uint32_t *galois_elts, int n_galois_elts, int check_tc128, int device, lb_context **out);
LB_API void lb_context_destroy(lb_context *ctx);
/* host copies of context constants */
LB_API int lb_context_get_modulus(const lb_context *ctx, int index, uint64_t *out);
LB_API int lb_context_get_root(const lb_context *ctx, int index, uint64_t *out);
LB_API int lb_context_get_galois_table(const lb_context *ctx, int elt_index, uint32_t *out_host_table);
/* The context owns one scratch block that grows on demand (device synchronisation + cudaMalloc when it
 * does).  Reserving the largest size up front keeps every later call allocation-free. */
LB_API int lb_context_reserve_workspace(lb_context *ctx, size_t bytes);
/* bytes of context-owned scratch a key switch at this level uses */
LB_API size_t lb_keyswitch_workspace_bytes(const lb_context *ctx, int size_l);

/* ---- negacyclic NTT (cahel-main/src/ntt/fntt_2d.cu:872, intt_2d.cu:693) --------------------- */

/* data: n_groups x (size_l + size_p) limbs; inside a group the first size_l limbs use data
 * primes 0..size_l-1 and the next size_p the special primes.  In place. */
LB_API int lb_ntt_forward(lb_context *ctx, uint64_t *data, int n_groups, int size_l, int size_p, void *stream);
LB_API int lb_ntt_inverse(lb_context *ctx, uint64_t *data, int n_groups, int size_l, int size_p, void *stream);

/* ---- element-wise evaluator ops (cahel-main/src/evaluate.cu:15,42,199; polymath.cu:16-227) ---- */

/* out = a (+|-|*) b over n_polys polynomials of size_l limbs each; out may alias a or b. */
LB_API int lb_add(lb_context *ctx, int size_l, int n_polys, const uint64_t *a, const uint64_t *b, uint64_t *out, void *stream);
LB_API int lb_sub(lb_context *ctx, int size_l, int n_polys, const uint64_t *a, const uint64_t *b, uint64_t *out, void *stream);
LB_API int lb_multiply_poly(lb_context *ctx, int size_l, int n_polys, const uint64_t *a, const uint64_t *b, uint64_t *out, void *stream);
/* out[g][n_polys][size_l][N] = sum of the items in[i][n_polys][size_l][N] with i in indices[offsets[g] .. offsets[g+1])
 * (add_many, cahel-main/src/evaluate.cu:177-197, over chosen subsets in one launch: the per-client sums of the
 * Krum driver, lancelot-main-GPU/utils/byzantine_fl.py:333-346).  offsets [n_groups + 1] and indices are HOST arrays;
 * an empty group gives zeros. */
LB_API int lb_sum_groups(lb_context *ctx, int size_l, int n_polys, int n_groups, const int *offsets, const int *indices, int n_items,
                  const uint64_t *in, uint64_t *out, void *stream);
/* element-wise product of two key-level polynomials [size_QP][N] (compute_secret_key_array, cahel-main/src/secretkey.cu:285-320) */
LB_API int lb_multiply_poly_key_level(lb_context *ctx, const uint64_t *a, const uint64_t *b, uint64_t *out, void *stream);
LB_API int lb_negate(lb_context *ctx, int size_l, int n_polys, const uint64_t *a, uint64_t *out, void *stream);
/* out = a mod q per limb for ANY 64-bit words a (out may alias a).  The reference has no such call: its additions
 * reduce one by one (cahel-main/src/polymath.cu:16-60).  It closes a plain 64-bit sum of residues, such as the
 * reduce-scatter of per-GPU partial pair sums in the Krum driver, in one pass. */
LB_API int lb_reduce_mod(lb_context *ctx, int size_l, int n_polys, const uint64_t *a, uint64_t *out, void *stream);
/* ckks_multiply / ckks_square (cahel-main/src/evaluate.cu:447,1433): batch of size-2 ciphertexts -> size-3 */
LB_API int lb_multiply(lb_context *ctx, int size_l, int batch, const uint64_t *a, const uint64_t *b, uint64_t *out3, void *stream);
LB_API int lb_square(lb_context *ctx, int size_l, int batch, const uint64_t *a, uint64_t *out3, void *stream);
/* mod_switch_drop_to_next (cahel-main/src/evaluate.cu:2253): drop the last limb of every polynomial */
LB_API int lb_mod_switch_drop(lb_context *ctx, int size_l, int n_polys, const uint64_t *in, uint64_t *out, void *stream);
/* apply_galois_ntt (cahel-main/src/galois.cu:153) on n_limbs limbs */
LB_API int lb_galois_permute(lb_context *ctx, int elt_index, int n_limbs, const uint64_t *in, uint64_t *out, void *stream);

/* ---- key switching (cahel-main/src/eval_key_switch.cu:80-216, rns_bconv.cu:668,965) ---------- */

LB_API int lb_modup(lb_context *ctx, int size_l, const uint64_t *cks, uint64_t *digits, void *stream);
LB_API int lb_keyswitch_inner_product(lb_context *ctx, int size_l, const uint64_t *digits, const uint64_t *evk, uint64_t *cx, void *stream);
LB_API int lb_moddown(lb_context *ctx, int size_l, const uint64_t *cx, uint64_t *out, void *stream);
/* switch_key_inplace: ct[2][size_l][N] += KS(cks) */
LB_API int lb_keyswitch(lb_context *ctx, int size_l, uint64_t *ct, const uint64_t *cks, const uint64_t *evk, void *stream);
/* relinearize_inplace (cahel-main/src/evaluate.cu:2019): ct3[3][size_l][N]; result in the first two polynomials */
LB_API int lb_relinearize(lb_context *ctx, int size_l, uint64_t *ct3, const uint64_t *relin_key, void *stream);
/* rescale_to_next (cahel-main/src/evaluate.cu:2059,2307; rns.cu:544): in [n_polys][size_l][N] -> out [n_polys][size_l-1][N] */
LB_API int lb_rescale(lb_context *ctx, int size_l, int n_polys, const uint64_t *in, uint64_t *out, void *stream);
/* rescale of the first polys_per_ct polynomials of `batch` ciphertexts that sit ct_stride words apart
 * (e.g. the two result polynomials of relinearized size-3 ciphertexts); out is dense [batch][polys_per_ct][size_l-1][N] */
LB_API int lb_rescale_strided(lb_context *ctx, int size_l, int batch, int polys_per_ct, const uint64_t *in, size_t ct_stride,
                       uint64_t *out, void *stream);
/* No counterpart in the reference.  Same result as lb_rescale, for callers that must not
 * allocate device memory while they run (work issued while a CUDA graph is being captured,
 * serving processes with a fixed memory budget, hosts that own the device allocator):
 * the scratch lives in a fixed 1.5 MiB array inside the library image instead of the
 * context's growable workspace, so this call performs no cudaMalloc / cudaFree.
 * Limits: n_polys * N <= lb_rescale_no_alloc_max_words() (196608), otherwise
 * LB_ERR_INVALID_ARG.  The first call on a device looks up the array's address; make that
 * call before any stream capture begins.  All calls on a device share the array, so
 * calls that overlap on the GPU (different streams) race; calls on one stream do not. */
LB_API int lb_rescale_no_alloc(lb_context *ctx, int size_l, int n_polys, const uint64_t *in, uint64_t *out, void *stream);
LB_API size_t lb_rescale_no_alloc_max_words(void);
/* apply_galois_inplace / rotate_vector for one Galois element that has a key (cahel-main/src/evaluate.cu:2364,2631) */
LB_API int lb_rotate(lb_context *ctx, int size_l, uint64_t *ct, int elt_index, const uint64_t *galois_key, void *stream);
/* hoisting_inplace (cahel-main/src/evaluate.cu:2412): ct <- sum over steps of rot(ct, step).
 * galois_keys: HOST array of n_steps device pointers, key of elt_indices[i] at [i]. */
LB_API int lb_hoisting(lb_context *ctx, int size_l, uint64_t *ct, int n_steps, const int *elt_indices,
                const uint64_t *const *galois_keys, void *stream);

/* Batched forms: `batch` ciphertexts stored back to back ([batch][3][size_l][N] for
 * relinearize, [batch][2][size_l][N] for rotate / hoisting), all switched with the same key.
 * The reference has no batch axis (one ciphertext per call, cahel-main/include/evaluate.h);
 * the Krum driver needs one to keep 190 independent pair results in flight. */
LB_API int lb_relinearize_batch(lb_context *ctx, int size_l, int batch, uint64_t *ct3, const uint64_t *relin_key, void *stream);
LB_API int lb_rotate_batch(lb_context *ctx, int size_l, int batch, uint64_t *ct, int elt_index, const uint64_t *galois_key, void *stream);
LB_API int lb_hoisting_batch(lb_context *ctx, int size_l, int batch, uint64_t *ct, int n_steps, const int *elt_indices,
                      const uint64_t *const *galois_keys, void *stream);

/* ---- Krum pairwise distance inner loop (lancelot-main-GPU/utils/byzantine_fl.py:201-223) ------- */

/* acc[3][size_l][N] (+)= sum over chunks c of square(b_c - a_c); a, b: chunk c of a client at
 * a + c * chunk_stride (in uint64 units), each chunk a size-2 ciphertext. */
LB_API int lb_krum_accumulate(lb_context *ctx, int size_l, int n_chunks, const uint64_t *a, const uint64_t *b,
                       size_t chunk_stride_a, size_t chunk_stride_b, uint64_t *acc, int accumulate, void *stream);

/* The same sums for several client pairs from one pass over their ciphertexts.  a / b / out are HOST
 * arrays of device pointers; every client's chunk c sits chunk_stride words after chunk c - 1.
 * n_b == 0: triangle, all pairs inside the 2..4 clients of a, in the order (0,1),(0,2),..,(1,2),..;
 * n_b > 0: rectangle, 1..2 clients of a against 1..4 clients of b, pair a_i, b_j at index i * n_b + j.
 * out[p][3][size_l][N] = sum over chunks of square(second - first) for pair p (overwritten). */
LB_API int lb_krum_accumulate_tile(lb_context *ctx, int size_l, int n_chunks, int n_a, const uint64_t *const *a, int n_b,
                            const uint64_t *const *b, size_t chunk_stride, uint64_t *const *out, void *stream);

/* The pair sums of a round in one call: out[p][3][size_l][N] = sum over chunks of square(ct_j - ct_i) for
 * pairs[2p] = i < pairs[2p+1] = j (the loop over pairs and chunks of byzantine_fl.py:466-514 with the diagonal left
 * out).  cts: HOST array of n_clients device pointers (only the clients that occur in a pair are read), chunk c of a
 * client chunk_stride words after chunk c - 1; pairs: HOST array.  The call covers the list with the tiles of
 * lb_krum_accumulate_tile that read the least (triangles of four clients, two clients against four). */
LB_API int lb_krum_pair_sums(lb_context *ctx, int size_l, int n_clients, const uint64_t *const *cts, int n_chunks, size_t chunk_stride,
                      int n_pairs, const int *pairs, uint64_t *out, void *stream);
/* From pair sums to score ciphertexts (byzantine_fl.py:244-273) for a batch: relinearize_inplace and
 * rescale_to_next_inplace of acc [n_pairs][3][size_l][N] (overwritten), scores <- result [n_pairs][2][size_l-1][N],
 * scores += hoisting(scores, first steps), then scores += rotate(scores, step) for every further step in order.
 * first_keys / pow_keys: HOST arrays of device pointers to the Galois keys of first_elts / pow_elts (indices into
 * the context's Galois elements). */
LB_API int lb_krum_scores(lb_context *ctx, int size_l, int n_pairs, uint64_t *acc, const uint64_t *relin_key, int n_first,
                   const int *first_elts, const uint64_t *const *first_keys, int n_pow, const int *pow_elts,
                   const uint64_t *const *pow_keys, uint64_t *scores, void *stream);

/* Mask multiplication of the aggregation phase (lancelot-main-GPU/utils/byzantine_fl.py:371-429):
 * out[c][3][size_l][N] = sum over clients k of ct_k[c] (x) mask_k (ckks_multiply + add_inplace per client
 * in the reference).  client_cts: HOST array of n_clients device pointers, chunk c of client k at
 * client_cts[k] + c * chunk_stride words; masks: [n_clients][2][size_l][N]. */
LB_API int lb_mask_accumulate(lb_context *ctx, int size_l, int n_clients, int n_chunks, const uint64_t *const *client_cts,
                       size_t chunk_stride, const uint64_t *masks, uint64_t *out, void *stream);

/* ---- decryption (cahel-main/src/secretkey.cu:594-654 without the noise-flooding term) --------- */

LB_API int lb_decrypt(lb_context *ctx, int size_l, int n_polys, const uint64_t *ct, const uint64_t *secret_key, uint64_t *pt, void *stream);
/* `batch` ciphertexts of n_polys polynomials each, stored back to back -> pt[batch][size_l][N] */
LB_API int lb_decrypt_batch(lb_context *ctx, int size_l, int n_polys, int batch, const uint64_t *ct, const uint64_t *secret_key, uint64_t *pt, void *stream);

/* ---- samplers and keys (cahel-main/src/prng.cu:143-242, secretkey.cu:254-515) -----------------
 * The reference draws a fresh 64-byte seed from the operating system for every call
 * (cahel-main/include/prng.cuh:12-23); here the caller supplies the seeds (HOST pointers),
 * which is what makes results reproducible and comparable bit for bit. */

LB_API int lb_sample_ternary(lb_context *ctx, const uint8_t *seed, int size_l, int size_p, uint64_t *out, void *stream);
LB_API int lb_sample_error(lb_context *ctx, const uint8_t *seed, int size_l, int size_p, uint64_t *out, void *stream);
LB_API int lb_sample_uniform(lb_context *ctx, const uint8_t *seed, int size_l, int size_p, uint64_t *out, void *stream);
/* gen_secretkey (secretkey.cu:254): sk[size_QP][N] = NTT(ternary) */
LB_API int lb_gen_secret_key(lb_context *ctx, const uint8_t *seed, uint64_t *sk, void *stream);
/* gen_publickey (secretkey.cu:322,451): pk[2][size_QP][N] = (-(a s + e), a) */
LB_API int lb_gen_public_key(lb_context *ctx, const uint64_t *sk, const uint8_t *seed_error, const uint8_t *seed_uniform, uint64_t *pk, void *stream);
/* generate_one_kswitch_key (secretkey.cu:328): out[dnum][2][size_QP][N]; sk_target is s^2 for
 * a relinearization key, the permuted secret for a Galois key; seeds[dnum][2][64] (error, uniform) */
LB_API int lb_gen_switch_key(lb_context *ctx, const uint64_t *sk, const uint64_t *sk_target, const uint8_t *seeds, uint64_t *out, void *stream);
/* create_galois_keys (cahel-main/src/secretkey.cu:374-449) for several Galois elements of the context in one call:
 * out[k][dnum][2][size_QP][N] = the switch key from sk rotated by element elt_indices[k] to sk, generated from
 * seeds[k][2 dnum][64] exactly as lb_galois_permute + lb_gen_switch_key generate it, with every step launched once
 * for all keys and digits. */
LB_API int lb_gen_galois_keys(lb_context *ctx, const uint64_t *sk, int n_keys, const int *elt_indices, const uint8_t *seeds,
                       uint64_t *out, void *stream);
/* encrypt_asymmetric (secretkey.cu:47-249) for a batch: ct[b][2][size_Q][N] = moddown(pk u + e) + (pt[b], 0).
 * seeds[b][2][64] = (ternary seed, error seed); pt may be NULL (encryption of zero). */
LB_API int lb_encrypt_asymmetric(lb_context *ctx, const uint64_t *pk, const uint64_t *pt, const uint8_t *seeds, int batch, uint64_t *ct, void *stream);

/* ---- CKKS encoder (cahel-main/src/ckks.cu:104-209,292-465) ---------------------------------- */

/* values: DEVICE array [batch][value_stride] of dtype 0 = double (real), 1 = float (real),
 * 2 = complex double; the first n_values of each message are encoded into sparse_slots
 * slots at `scale`; pt[batch][size_l][N] in NTT form.  Values that do not fit the modulus
 * raise a device flag reported by lb_check_status (the reference throws invalid_argument). */
LB_API int lb_encode(lb_context *ctx, int size_l, const void *values, int dtype, size_t value_stride, int n_values, int sparse_slots,
              int batch, double scale, uint64_t *pt, void *stream);
/* lb_encode followed by lb_encrypt_asymmetric for a batch, bit-identical to the two calls, with
 * the plaintext kept in coefficient form and folded into the encryption's mod-down transform
 * (three transforms and one round trip through HBM fewer per ciphertext): ct[batch][2][size_Q][N] */
LB_API int lb_encode_encrypt(lb_context *ctx, const uint64_t *pk, const void *values, int dtype, size_t value_stride, int n_values,
                      int sparse_slots, int batch, double scale, const uint8_t *seeds, uint64_t *ct, void *stream);
/* out_complex: DEVICE array of sparse_slots (re, im) pairs */
LB_API int lb_decode(lb_context *ctx, int size_l, const uint64_t *pt, double scale, int sparse_slots, double *out_complex, void *stream);
/* pt[batch][size_l][N] -> out_complex[batch][sparse_slots] (re, im) pairs */
LB_API int lb_decode_batch(lb_context *ctx, int size_l, int batch, const uint64_t *pt, double scale, int sparse_slots, double *out_complex, void *stream);
/* Synchronises the stream and reports (then clears) conditions kernels could only flag. */
LB_API int lb_check_status(lb_context *ctx, void *stream);

#ifdef __cplusplus
}
#endif
#endif
