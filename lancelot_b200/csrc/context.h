// Device-resident context: constant tables uploaded once, a reusable workspace, and the
// launch helpers every kernel file shares.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "../../include/lancelot_b200.h"
#include "params.h"

namespace lb {

struct DevLevel {
    u64 *qlast_inv = nullptr, *qlast_inv_s = nullptr;
    u64 *p_inv = nullptr, *p_inv_s = nullptr;
    u64 *hat_inv = nullptr, *hat_inv_s = nullptr, *hat_mod = nullptr;
    u64 *phat_inv = nullptr, *phat_inv_s = nullptr, *phat_mod = nullptr;
    // inverse-NTT closing constants with the mod-up factor folded in: N^-1 * hat_inv and
    // psi^-bitrev(1) * N^-1 * hat_inv (value, Shoup quotient) per limb
    u64 *fold = nullptr; // [size_l][4]
    // same for the special limbs with phat_inv folded in: [size_p][4]
    u64 *pfold = nullptr;
};

struct Context {
    HostParams hp;
    int device = 0;
    int sm_count = 0;
    ModConst *d_mc = nullptr;
    ulonglong2 *d_tw = nullptr, *d_itw = nullptr;
    uint32_t *d_perm = nullptr;
    u64 *d_p_mod_q = nullptr, *d_p_mod_q_s = nullptr;
    std::vector<DevLevel> d_level;
    // encoder tables
    double2 *d_croots = nullptr; // [2N] complex roots of unity
    uint32_t *d_rot_group = nullptr; // [N/4] powers of 5 mod 2N
    // inverse-FFT twiddles of the encoder in the order its stages use them, one table per log2(slots), each built
    // on first use: entry (n - (n >> u)) + k is the twiddle of butterfly group k at stage u
    double2 *d_ifft_tw[20] = {};
    int *d_status = nullptr;         // sticky device-side condition flags (bit 0: encoded values are too large)
    // scratch owned by the context, grown on demand between operations
    void *ws = nullptr;
    size_t ws_bytes = 0;
    std::vector<void *> owned; // device allocations released with the context

    int ensure_workspace(size_t bytes);
};

void set_error(const std::string &msg);
// every kernel launch of this library goes through this (diag.cu): counted always, timed per kernel name while
// the diagnostic timer is on
// algorithmic_bytes: what the launch must read and write at least (each datum once, tables excluded), 0 = not stated
void count_launch(const char *kernel_name, cudaStream_t stream, double algorithmic_bytes = 0.0);
unsigned long long launch_count();
struct Context;
Context *lb_context_impl(lb_context *h); // the context behind a C-ABI handle (capi.cu)
int cuda_fail(cudaError_t e, const char *what);

#define LB_CUDA(call)                                         \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
    } while (0)

// ---- kernels (one launcher per step; all asynchronous on `stream`) ----------------------

struct NttJob {
    // Rows are limbs of N residues.  Row r belongs to group g = r / per_group at position
    // rr = r % per_group; a group is further addressed as (outer, inner) = (g / split, g % split)
    // so that batches of multi-polynomial ciphertexts map without copies:
    //   row offset of a group in X = outer * X_outer + inner * X_group_stride      (X = src, dst, aux, add)
    const u64 *src = nullptr;
    u64 *dst = nullptr;
    int n_groups = 1;
    int per_group = 1;
    int split = 1;
    int size_l = 1;      // rows [0,size_l) use table tbl_off + row, the rest size_Q + (row - size_l)
    int tbl_off = 0;
    long src_group_stride = -1, dst_group_stride = -1; // inner strides in rows; -1: per_group
    long src_outer = -1, dst_outer = -1;               // outer strides in rows; -1: split * inner stride
    int src_row_off = 0;   // first source row inside a group
    int skip_lo = 0, skip_hi = 0; // rows [skip_lo, skip_hi) of each group are left untouched
    // Forward prologue (fast base conversion fused into the load): the transform input of
    // row rr is  sum_{i < bconv_n} src_row(i)[k] * mat[i]  mod q_rr,  where src_row(i) is row
    // src_row_off + i of the group's source block.  mat == nullptr means all-ones with
    // bconv_n == 1, i.e. "x mod q_rr" of a single source row.
    int bconv_n = 0;
    const u64 *bconv_mat = nullptr;     // entries of row rr start at (digit * mat_group_stride + rr * mat_row_stride)
    long mat_group_stride = 0, mat_row_stride = 0;
    int digit_alpha = 0; // > 0: mod-up mode.  inner = digit j of ciphertext `outer`: source rows
                         // [j*alpha, min((j+1)*alpha, size_l)) of the outer block (the inner stride of
                         // src is not used), and the digit's own rows are skipped
    // Forward prologue, second part: x <- x - presub[k] * presub_scal[rr] for groups with inner < presub_inner;
    // presub rows are [outer][per_group][N] in coefficient form (a plaintext folded into the mod-down of an encryption)
    const u64 *presub = nullptr, *presub_scal = nullptr, *presub_scal_s = nullptr;
    long presub_outer = -1;
    int presub_inner = 0;
    // Encryption only (one special prime): esmall[outer][N] is the small error polynomial as signed bytes;
    // the single source row is (INTT(pk u) on p); the load forms ((x + e) mod p) mod q_rr - e
    const signed char *esmall = nullptr;
    u64 esmall_p = 0;
    // The transform input itself as signed bytes, small[group][N]: every row of a group transforms the same small
    // polynomial (the ternary u of an encryption), reduced into the row's prime by the load; src is not read
    const signed char *small = nullptr;
    // Forward epilogue: dst = (aux - NTT(x)) * scal[rr] (+ add), the closing step of mod-down and rescale
    const u64 *aux = nullptr;
    long aux_group_stride = -1, aux_outer = -1;
    const u64 *scal = nullptr, *scal_s = nullptr;
    const u64 *add = nullptr; // optional addend rows; only groups with inner < add_inner have one
    long add_group_stride = -1, add_outer = -1;
    int add_inner = 0;
    // the addend rows of the groups with inner == 1 when they sit in another buffer: add1 + outer * add1_outer rows
    // (the second polynomial of ciphertexts that a rotation is added to in place); may alias dst
    const u64 *add1 = nullptr;
    long add1_outer = 0;
    // Forward epilogue, alternative: mul2[2][per_group][N] are two fixed rows per row position (the two polynomials of a
    // public key); group g stores NTT(x) * mul2[0] at dst rows (go * dst_outer + rr) and NTT(x) * mul2[1] per_group rows
    // further on, so dst_outer = 2 * per_group lays the products out as [group][2][per_group][N]
    const u64 *mul2 = nullptr;
    // Inverse epilogue: closing constants per row replaced by fold[rr][4]
    const u64 *fold = nullptr;
};

int ntt_forward(Context *ctx, const NttJob &job, cudaStream_t stream);
int ntt_inverse(Context *ctx, const NttJob &job, cudaStream_t stream);
int probe_butterfly_rate(Context *ctx, int mode, double *butterflies_per_second);

// element-wise kernels (poly.cu).  Rows are limbs of N residues; row r uses prime r % size_l.
enum PolyOp { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_NEG = 3, OP_REDUCE = 4 };
int poly_binary(Context *ctx, int op, int size_l, long rows, const u64 *a, const u64 *b, u64 *out, cudaStream_t stream);
// out[3][L][N] = a[2][L][N] (x) b[2][L][N], batched over `batch` ciphertexts
int poly_tensor(Context *ctx, int size_l, int batch, const u64 *a, const u64 *b, u64 *out, cudaStream_t stream);
// dst[i] = src[perm[i]] for `rows` limbs
int poly_galois(Context *ctx, int elt_idx, long rows, const u64 *src, u64 *dst, cudaStream_t stream);
// the same for ciphertexts [batch][2][L][N], with the first polynomial of each added to its own image
int poly_galois_plus_c0(Context *ctx, int elt_idx, int L, int batch, const u64 *src, u64 *dst, cudaStream_t stream);
int poly_sum_groups(Context *ctx, int size_l, long n_rows, int n_groups, const int *h_offsets, const int *h_indices, const u64 *in,
                    u64 *out, cudaStream_t stream);
// acc[3][L][N] (+)= sum_c square(b_c - a_c) over n_chunks ciphertext pairs [2][L][N]
int krum_accumulate(Context *ctx, int size_l, int n_chunks, const u64 *a, const u64 *b, long chunk_stride_a,
                    long chunk_stride_b, u64 *acc, int accumulate, cudaStream_t stream);
int krum_accumulate_tile(Context *ctx, int size_l, int n_chunks, int n_a, const u64 *const *a, int n_b, const u64 *const *b,
                         long chunk_stride, u64 *const *out, cudaStream_t stream);
// drop the last limb of each polynomial: in [polys][L][N] -> out [polys][L-1][N]
int poly_drop_last(Context *ctx, int size_l, int n_polys, const u64 *in, u64 *out, cudaStream_t stream);
// pt = c0 + c1 s + c2 s^2 ...
int poly_decrypt(Context *ctx, int size_l, int n_polys, int batch, const u64 *ct, const u64 *sk, u64 *pt, cudaStream_t stream);
// out[c][3][L][N] = sum over clients k of ct_k[c] (x) mask_k; client_cts: host array of device pointers
int mask_accumulate(Context *ctx, int size_l, int n_clients, int n_chunks, const u64 *const *client_cts, long chunk_stride,
                    const u64 *masks, u64 *out, cudaStream_t stream);

// key switching (keyswitch.cu); all buffers in NTT form, evk [dnum][2][size_QP][N]
size_t keyswitch_workspace_bytes(const Context *ctx, int size_l);
// ct[2][L][N]: out_i = (add_i ? add_i : 0) + moddown(<modup(cks), evk>)_i ; add0/add1 may alias out
int keyswitch(Context *ctx, int size_l, const u64 *cks, const u64 *evk, const u64 *add0, const u64 *add1, u64 *out,
              cudaStream_t stream);
int relinearize(Context *ctx, int size_l, int batch, u64 *ct3, const u64 *rlk, cudaStream_t stream);
int rescale(Context *ctx, int size_l, int batch, int polys_per_ct, const u64 *in, long in_outer_rows, u64 *out, cudaStream_t stream);
// accumulate: ct <- ct + rotation (sum of rotations) of ct instead of ct <- rotation
int rotate(Context *ctx, int size_l, int batch, u64 *ct, int elt_idx, const u64 *glk, cudaStream_t stream, bool accumulate = false);
int rescale_static(Context *ctx, int size_l, int n_polys, const u64 *in, u64 *out, cudaStream_t stream); // rescale_static.cu
size_t rescale_static_max_words();
int hoisting(Context *ctx, int size_l, int batch, u64 *ct, int n_steps, const int *elt_idx, const u64 *const *glks,
             cudaStream_t stream, bool accumulate = false);
// exposed pieces of the key switch for per-stage parity tests
int modup(Context *ctx, int size_l, const u64 *cks, u64 *digits, cudaStream_t stream);
int inner_product(Context *ctx, int size_l, const u64 *digits, const u64 *cks, const u64 *evk, u64 *cx, cudaStream_t stream);
int moddown(Context *ctx, int size_l, const u64 *cx, u64 *out, cudaStream_t stream);

// samplers, key generation, encryption (sampler.cu).  d_seeds: device words, 16 per seed.
int sample_small(Context *ctx, int kind, const uint32_t *d_seeds, int seed_stride, int batch, int size_l, int size_p, u64 *out,
                 cudaStream_t stream);
int sample_uniform(Context *ctx, const uint32_t *d_seeds, int seed_stride, int batch, int size_l, int size_p, u64 *out,
                   cudaStream_t stream, long out_stride = 0);
int gen_public_key(Context *ctx, const u64 *sk, const uint32_t *d_seed_e, const uint32_t *d_seed_a, u64 *pk, u64 *scratch,
                   cudaStream_t stream);
int gen_switch_key(Context *ctx, const u64 *sk, const u64 *skp, const uint32_t *d_seeds, u64 *out, u64 *scratch, cudaStream_t stream);
int gen_switch_keys(Context *ctx, const u64 *sk, const u64 *targets, int n, const uint32_t *d_seeds, u64 *out, u64 *scratch,
                    cudaStream_t stream);
size_t encrypt_workspace_bytes(const Context *ctx, int batch);
// encoder (encoder.cu)
int encode(Context *ctx, int size_l, const void *values, int dtype, long value_stride, int n_values, int sparse_slots, int batch,
           double scale, u64 *pt, int *d_status, int skip_ntt, cudaStream_t stream);
int decode(Context *ctx, int size_l, int batch, const u64 *pt, double scale, int sparse_slots, double *out_complex, cudaStream_t stream);
int encrypt_asymmetric(Context *ctx, const u64 *pk, const u64 *pt, int pt_is_coeff, const uint8_t *host_seeds, int batch, u64 *ct,
                       cudaStream_t stream);

} // namespace lb
