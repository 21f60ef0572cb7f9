/*
 * ckks_oracle.h - CPU restatement of the reference's CKKS key-switching / NTT path.
 *
 * TEST INFRASTRUCTURE ONLY. This library is the checker for the CUDA product: only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark may load it. The
 * product library never links, imports or executes anything in this directory.
 *
 * Parity status: PINNED. Every function below was checked, limb hash by limb hash, against
 * outputs of the unmodified reference library (built by oracle/Makefile into oracle/_ref and
 * driven by oracle/ref_harness.cu on a B200); the recorded outputs live in tests/golden/.
 * The reference's own tests hold no limb-level golden vectors (they only round-trip or
 * decrypt-and-compare), so co-running the reference is the pin.
 *
 * Every function cites the reference file:line (paths relative to the reference checkout)
 * whose arithmetic it restates. All data is uint64 residues, layout [poly][limb][N].
 */
#ifndef CKKS_ORACLE_H
#define CKKS_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORA_MAX_LIMBS 64

/* ---- scalar helpers -------------------------------------------------------------------- */
uint64_t ora_mulmod(uint64_t a, uint64_t b, uint64_t q);
uint64_t ora_powmod(uint64_t a, uint64_t e, uint64_t q);
uint64_t ora_invmod(uint64_t a, uint64_t q);
int ora_is_prime(uint64_t v);
/* src/host/modulus.cu:80-111 + src/host/numth.cu:207-232: primes per requested bit size,
 * searched downward from 2^bits - 2N + 1 in steps of 2N; each bit size hands out its primes
 * smallest-first. Returns 0 on success. */
int ora_create_coeff_modulus(size_t N, const int *bit_sizes, size_t count, uint64_t *out);
/* src/host/numth.cu:309-332: smallest primitive degree-th root of unity mod q. */
uint64_t ora_minimal_primitive_root(uint64_t degree, uint64_t q);
/* bit reversal over `bits` bits */
uint32_t ora_bitrev(uint32_t x, int bits);

/* ---- deterministic synthetic data ------------------------------------------------------- */
/* Index-addressed uniform generator: element i of stream `seed` is the first of the draws
 * mix(seed,i,0), mix(seed,i,1), ... (masked to bitlen(q) bits) that is < q. Exactly uniform
 * in [0,q), independent of evaluation order. */
uint64_t ora_uniform_at(uint64_t seed, uint64_t i, uint64_t q);
void ora_fill_uniform(uint64_t *dst, size_t n, uint64_t q, uint64_t seed);
/* Fills n_limbs limbs of a [..][N] buffer: limb l takes prime primes[l] and stream
 * (case_seed << 40) ^ (buf << 16) ^ (limb0 + l). The reference harness, the tests and the
 * benchmark all build their synthetic ciphertexts and keys through this one rule. */
void ora_fill_limbs(uint64_t *dst, size_t N, const uint64_t *primes, size_t n_limbs,
                    uint64_t case_seed, uint64_t buf, uint64_t limb0);
/* order-independent 64-bit content hash of one limb: sum_i mix64(x_i ^ mix64(i+1)) */
uint64_t ora_limb_hash(const uint64_t *x, size_t n);

/* ---- context ---------------------------------------------------------------------------- */
typedef struct ora_ctx ora_ctx;
/* primes[0..size_QP): Q primes first, then the size_P special primes (src/context.cu:125-168) */
ora_ctx *ora_ctx_create(size_t N, const uint64_t *primes, size_t size_QP, size_t size_P);
void ora_ctx_destroy(ora_ctx *c);
size_t ora_ctx_N(const ora_ctx *c);
/* table accessors, for comparing the product's tables word for word (src/host/ntt.cu:11-56) */
const uint64_t *ora_ctx_twiddle(const ora_ctx *c, size_t prime_idx);
const uint64_t *ora_ctx_itwiddle(const ora_ctx *c, size_t prime_idx);
uint64_t ora_ctx_root(const ora_ctx *c, size_t prime_idx);
/* number of digits at level with `size_Ql` Q-limbs: ceil(size_Ql / size_P) (src/rns.cu:149) */
size_t ora_beta(const ora_ctx *c, size_t size_Ql);

/* ---- transforms (src/ntt/ntt_1d.cu:17-76,194-256; include/butterfly.cuh:17-71) ---------- */
/* in place over n_limbs limbs starting at physical prime index first_prime */
void ora_ntt_forward(const ora_ctx *c, uint64_t *data, size_t n_limbs, size_t first_prime);
void ora_ntt_inverse(const ora_ctx *c, uint64_t *data, size_t n_limbs, size_t first_prime);

/* ---- key switching ------------------------------------------------------------------------ */
/* src/rns_bconv.cu:530-628. in: c2[size_Ql][N] NTT form. out: [beta][size_Ql+size_P][N]. */
void ora_modup(const ora_ctx *c, size_t size_Ql, const uint64_t *c2, uint64_t *out);
/* src/eval_key_switch.cu:175-230. digits [beta][size_Ql+size_P][N]; evk[d] -> [2][size_QP][N];
 * out [2][size_Ql+size_P][N]. */
void ora_ks_inner_prod(const ora_ctx *c, size_t size_Ql, const uint64_t *digits,
                       const uint64_t *const *evk, uint64_t *out);
/* src/rns_bconv.cu:776-828. cx [size_Ql+size_P][N] (left untouched) -> out [size_Ql][N]. */
void ora_moddown(const ora_ctx *c, size_t size_Ql, const uint64_t *cx, uint64_t *out);
/* src/eval_key_switch.cu:294-381: ct[2][size_Ql][N] += ModDown(<ModUp(c2), evk>). */
void ora_keyswitch(const ora_ctx *c, size_t size_Ql, const uint64_t *c2,
                   const uint64_t *const *evk, uint64_t *ct);

/* ---- evaluator pieces --------------------------------------------------------------------- */
/* src/polymath.cu:463-498 (tensor_prod_2x2_rns_poly): a,b [2][l][N] -> out [3][l][N] */
void ora_tensor_mul(const ora_ctx *c, size_t size_Ql, const uint64_t *a, const uint64_t *b,
                    uint64_t *out);
/* src/evaluate.cu:1061-1104 + 1342-1374: out[2][l][N] = relin(a*b) */
void ora_multiply_and_relin(const ora_ctx *c, size_t size_Ql, const uint64_t *a,
                            const uint64_t *b, const uint64_t *const *rlk, uint64_t *out);
/* src/rns.cu:1128-1183: in [n_poly][l][N] -> out [n_poly][l-1][N], floor-style RNS rescale */
void ora_rescale(const ora_ctx *c, size_t size_Ql, size_t n_poly, const uint64_t *in,
                 uint64_t *out);
void ora_rescale_rounded(const ora_ctx *c, size_t size_Ql, size_t n_poly, const uint64_t *in, uint64_t *out);
/* include/galois.cuh:16-49 */
uint32_t ora_galois_elt_from_step(int step, size_t N);
/* include/galois.cuh:98-113: NTT-domain gather table, dst[i] = src[perm[i]] */
void ora_galois_perm(size_t N, uint32_t galois_elt, uint32_t *perm);
/* src/evaluate.cu:1607-1656: permute c0,c1 then key-switch the permuted c1. ct [2][l][N] in/out */
void ora_apply_galois(const ora_ctx *c, size_t size_Ql, uint32_t galois_elt,
                      const uint64_t *const *ksk, uint64_t *ct);
/* src/evaluate.cu:1929-2082: one ModUp, then per step permute extended digits.
 * ksk[s] -> pointer table (beta entries) of the key for elts[s]; outs[s] -> [2][l][N]. */
void ora_hoist_rotations(const ora_ctx *c, size_t size_Ql, const uint64_t *ct,
                         const uint32_t *elts, size_t n_steps,
                         const uint64_t *const *const *ksk, uint64_t *const *outs);
void ora_hoisting_sum(const ora_ctx *c, size_t size_Ql, const uint64_t *ct, const uint32_t *elts, size_t n_steps,
                      const uint64_t *const *const *ksk, uint64_t *out);
/* src/bsgs.cu:51-96: acc_k = sum_b pt_b (.) baby_b[k], reduced after every term.
 * pts[b] -> [l][N]; babies[b] -> [2][l][N]; out [2][l][N]. */
void ora_bsgs_mac(const ora_ctx *c, size_t size_Ql, size_t M, const uint64_t *const *pts,
                  const uint64_t *const *babies, uint64_t *out);
/* src/bootstrap.cu:660-686 + forward NTT: signed centred int64[N] -> [size_Ql][N] NTT form */
void ora_expand_single_chain(const ora_ctx *c, size_t size_Ql, const int64_t *coeffs, uint64_t *out);
/* src/polymath.cu:17-180 elementwise helpers over [n_limbs][N] starting at prime 0 */
void ora_add(const ora_ctx *c, size_t n_limbs, const uint64_t *a, const uint64_t *b, uint64_t *o);
void ora_sub(const ora_ctx *c, size_t n_limbs, const uint64_t *a, const uint64_t *b, uint64_t *o);
void ora_mul(const ora_ctx *c, size_t n_limbs, const uint64_t *a, const uint64_t *b, uint64_t *o);

/* number of OpenMP threads the oracle will use */
int ora_num_threads(void);
void ora_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
