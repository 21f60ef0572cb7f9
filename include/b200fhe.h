/*
 * b200fhe.h - C ABI of libb200fhe.so: CKKS hybrid key switching and the negacyclic NTT under it,
 * hand-written for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a binding of the reference library would call instead of the reference's
 * own CUDA path. Each entry point names the reference interface it replaces (paths relative to the
 * reference checkout). Conventions:
 *   - every function returns 0 on success, a negative B2_E* code on a caller error, a positive
 *     value (cudaError_t) on a CUDA failure; b2_last_error() gives the message for this thread;
 *   - all `d_*` pointers are DEVICE pointers to uint64 residues laid out [poly][limb][N]
 *     (coefficient index contiguous), limbs ordered like the context's primes: the reference's
 *     layout (include/ciphertext.h:161-163), so buffers interchange byte for byte; they must be
 *     32-byte aligned (the transforms use 256-bit accesses; B2_EINVAL otherwise - cudaMalloc and
 *     torch allocations are);
 *   - NTT-form data is in the bit-reversed order the reference's forward transform produces;
 *   - `size_Ql` is the number of Q limbs the operand holds (chain index k of the reference holds
 *     size_Q - (k - 1) limbs, src/context.cu:145-168);
 *   - nothing allocates behind the caller's back: scratch comes in as `d_ws` / `ws_bytes`
 *     (size from b2_workspace_bytes); `stream` is a cudaStream_t passed as void*;
 *   - calls are asynchronous on `stream`; there is no CPU fallback - without a CUDA device
 *     b2_ctx_create fails.
 */
#ifndef B200FHE_H
#define B200FHE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_EINVAL (-1)  /* bad argument (size, level, null pointer)              */
#define B2_ESIZE (-2)   /* polynomial degree or limb count outside what is built */
#define B2_EWS (-3)     /* workspace too small                                   */
#define B2_ENOMEM (-4)  /* host allocation failed                                */
#define B2_ENOKEY (-5)  /* Galois element has no permutation table               */

typedef struct b2_ctx b2_ctx;

const char *b2_last_error(void);
int b2_version(void);

/* replaces CoeffModulus::Create (src/host/modulus.cu:80-111; python/src/binding.cu:56) */
int b2_create_coeff_modulus(size_t N, const int *bit_sizes, size_t count, uint64_t *primes_out);

/* replaces PhantomContext(params) (src/context.cu:125-232; python/src/binding.cu:72):
 * primes[0..size_QP) = Q primes then the size_P special primes. Builds every table of every
 * level on the host and uploads it to `device`. N in [2^12, 2^17]. */
int b2_ctx_create(size_t N, const uint64_t *primes, size_t size_QP, size_t size_P, int device,
                  b2_ctx **out);
void b2_ctx_destroy(b2_ctx *ctx);
size_t b2_ctx_N(const b2_ctx *ctx);
size_t b2_ctx_size_Q(const b2_ctx *ctx);
size_t b2_ctx_size_P(const b2_ctx *ctx);
/* number of digits at a level: ceil(size_Ql / size_P) (src/rns.cu:149) */
size_t b2_ctx_beta(const b2_ctx *ctx, size_t size_Ql);
/* host copies of the tables, for word-for-word checks against src/host/ntt.cu:11-56:
 * which = 0 forward twiddles, 1 inverse twiddles, 2 forward Shoup words, 3 inverse Shoup words */
int b2_ctx_get_table(const b2_ctx *ctx, int which, size_t prime_idx, uint64_t *host_out);

/* scratch bytes for an operation at a level. op: one of B2_OP_* */
#define B2_OP_MODUP 1
#define B2_OP_MODDOWN 2
#define B2_OP_KEYSWITCH 3
#define B2_OP_RESCALE 4
#define B2_OP_MUL_RELIN 5
#define B2_OP_ROTATE 6
#define B2_OP_HOIST 7
size_t b2_workspace_bytes(const b2_ctx *ctx, int op, size_t size_Ql);

/* replaces nwt_2d_radix8_forward_inplace / _backward_inplace (src/ntt/fntt_2d.cu:665-709,
 * src/ntt/intt_2d.cu:769-813): in place over n_limbs limbs; limb i uses prime first_prime + i. */
int b2_ntt_forward(b2_ctx *ctx, uint64_t *d_data, size_t n_limbs, size_t first_prime, void *stream);
int b2_ntt_inverse(b2_ctx *ctx, uint64_t *d_data, size_t n_limbs, size_t first_prime, void *stream);

/* replaces DRNSTool::modup (src/rns_bconv.cu:530-628):
 * d_c2 [size_Ql][N] (NTT form) -> d_out [beta][size_Ql + size_P][N] (NTT form) */
int b2_modup(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_c2, uint64_t *d_out, void *d_ws,
             size_t ws_bytes, void *stream);

/* replaces key_switch_inner_prod (src/eval_key_switch.cu:265-291):
 * d_digits [beta][size_Ql+size_P][N]; evk[d] = device pointer to digit d of the key,
 * [2][size_QP][N] at key level (include/secretkey.h:116-226); d_out [2][size_Ql+size_P][N] */
int b2_ks_inner_prod(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_digits,
                     const uint64_t *const *evk, size_t n_evk, uint64_t *d_out, void *stream);

/* replaces DRNSTool::moddown_from_NTT (src/rns_bconv.cu:776-828) for n_poly polynomials at once:
 * d_cx [n_poly][size_Ql+size_P][N] (its P limbs are overwritten) -> d_out [n_poly][size_Ql][N] */
int b2_moddown(b2_ctx *ctx, size_t size_Ql, size_t n_poly, uint64_t *d_cx, uint64_t *d_out,
               void *d_ws, size_t ws_bytes, void *stream);

/* replaces keyswitch_inplace (src/eval_key_switch.cu:294-381):
 * d_ct [2][size_Ql][N] += ModDown(<ModUp(d_c2), evk>) */
int b2_keyswitch(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_c2, const uint64_t *const *evk,
                 size_t n_evk, uint64_t *d_ct, void *d_ws, size_t ws_bytes, void *stream);

/* keyswitch_inplace (src/eval_key_switch.cu:294-381) for `batch` ciphertexts switched with ONE key (a batch of
 * relinearisations, or of rotations by one step): set b reads d_c2 + b * c2_stride limbs and updates
 * d_ct + b * ct_stride limbs ([2][size_Ql][N] each); strides in limbs of N words. Every kernel is one launch over the
 * batch where the fused pipeline applies (N = 2^16), else the key switches run one after another. Same limbs as
 * `batch` calls of b2_keyswitch. d_ws: b2_keyswitch_batch_workspace_bytes(). */
size_t b2_keyswitch_batch_workspace_bytes(const b2_ctx *ctx, size_t size_Ql, size_t batch);
int b2_keyswitch_batch(b2_ctx *ctx, size_t size_Ql, size_t batch, const uint64_t *d_c2, size_t c2_stride,
                       const uint64_t *const *evk, size_t n_evk, uint64_t *d_ct, size_t ct_stride,
                       void *d_ws, size_t ws_bytes, void *stream);

/* multiply_and_relin (src/evaluate.cu:1061-1104) and, rescale != 0, rescale_to_next (src/evaluate.cu:1413-1464) for
 * `batch` ciphertext pairs with ONE relinearisation key, every kernel one launch over the batch. Pair b reads
 * d_a + b * a_stride and d_b + b * b_stride limbs ([2][size_Ql][N] each) and writes d_out + b * out_stride limbs:
 * [2][size_Ql][N], or [2][size_Ql-1][N] after the rescale. Same limbs as b2_multiply_and_relin followed by b2_rescale. */
size_t b2_multiply_relin_batch_workspace_bytes(const b2_ctx *ctx, size_t size_Ql, size_t batch);
int b2_multiply_relin_rescale_batch(b2_ctx *ctx, size_t size_Ql, size_t batch, const uint64_t *d_a, size_t a_stride,
                                    const uint64_t *d_b, size_t b_stride, const uint64_t *const *rlk, size_t n_evk,
                                    uint64_t *d_out, size_t out_stride, int rescale, void *d_ws, size_t ws_bytes,
                                    void *stream);

/* replaces special_fft_backward / special_fft_forward with their bit reversals (src/fft.cu:90-346, src/ckks.cu:97-105, 176-183):
 * n = N/2 complex doubles; d_rot uint32 [n] = 5^j mod 2N, d_ksi complex double [2N + 1] = exp(2 pi i k / 2N).
 * inverse = 1 (encode): d_vals (overwritten) -> d_out = preimage of the embedding times scale; inverse = 0 (decode):
 * d_vals -> d_out = slot values times scale. d_vals and d_out must not overlap. */
int b2_special_fft(b2_ctx *ctx, void *d_vals, void *d_out, const uint32_t *d_rot, const void *d_ksi, int inverse,
                   double scale, void *stream);
/* the rounding step of encode_internal (src/ckks.cu:107-131): N/2 complex doubles -> int64 [N] signed coefficients
 * (real parts first, then imaginary parts); spread them over the limbs with b2_expand_signed */
int b2_encode_round(b2_ctx *ctx, const void *d_u, int64_t *d_coeffs, void *stream);
/* replaces DBaseConverter::compose_array (src/rns_base.cu:173-234): coefficient-form residues d_res [size_Ql][N] -> N/2
 * complex doubles (centred value times inv_scale; coefficient k real part of entry k, k + N/2 its imaginary part).
 * d_tab: 64-bit words hat [l][l] (Q/q_i) | inv [l] ((Q/q_i)^-1 mod q_i) | Q [l] | floor(Q/2) [l], little endian */
int b2_decode_compose(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_res, const uint64_t *d_tab, double inv_scale,
                      void *d_out, void *stream);

/* replaces sample_uniform_poly / sample_error_poly / sample_ternary_poly (src/prng.cu:142-240): polynomials drawn on the
 * device from a ChaCha20 keystream (32-byte key, 12-byte nonce, both host pointers read at call time; never reuse a pair).
 * kind 0: uniform residues, d_out uint64 [n_limbs][N] for primes first_prime ..; kind 1: centred binomial, 21 coin pairs;
 * kind 2: uniform ternary; kinds 1 and 2 write int64 [N] signed coefficients (spread them with b2_expand_signed). */
int b2_sample(b2_ctx *ctx, int kind, const uint8_t *key32, const uint8_t *nonce12, size_t first_prime, size_t n_limbs,
              void *d_out, void *stream);

/* replaces bgv_ckks_multiply's tensor product (src/evaluate.cu:345-397, src/polymath.cu:463-540):
 * d_a, d_b [2][size_Ql][N] -> d_out [3][size_Ql][N] */
int b2_tensor_mul(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_a, const uint64_t *d_b,
                  uint64_t *d_out, void *stream);

/* replaces multiply_and_relin_inplace for CKKS (src/evaluate.cu:1061-1104, 1342-1374):
 * d_out [2][size_Ql][N] = relinearise(d_a * d_b) */
int b2_multiply_and_relin(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_a, const uint64_t *d_b,
                          const uint64_t *const *rlk, size_t n_evk, uint64_t *d_out, void *d_ws,
                          size_t ws_bytes, void *stream);

/* replaces divide_and_round_q_last_ntt under rescale_to_next (src/rns.cu:1128-1183,
 * src/evaluate.cu:1413-1464): d_in [n_poly][size_Ql][N] -> d_out [n_poly][size_Ql-1][N] */
int b2_rescale(b2_ctx *ctx, size_t size_Ql, size_t n_poly, const uint64_t *d_in, uint64_t *d_out,
               void *d_ws, size_t ws_bytes, void *stream);

/* b2_rescale with the remainder of the dropped prime taken centred, so that every coefficient is
 * rounded to nearest instead of floored. No counterpart in the reference (its rescale, src/rns.cu:
 * 1128-1183, adds no rounding offset); the bootstrapping pipeline uses it because the half-unit bias
 * of flooring, summed over all coefficients, is what limits the precision of EvalRound. Same
 * arguments and workspace as b2_rescale. */
int b2_rescale_rounded(b2_ctx *ctx, size_t size_Ql, size_t n_poly, const uint64_t *d_in,
                       uint64_t *d_out, void *d_ws, size_t ws_bytes, void *stream);

/* No counterpart in the reference (which takes every scratch buffer from cudaMallocAsync).
 * Same result as b2_rescale, for callers that cannot supply scratch and must not allocate: a
 * process whose device memory is already fully reserved by another allocator, or a thread that
 * may not enter an allocating CUDA call at that point. The scratch is a 1.5 MiB array inside the
 * library image (3 polynomials x 65536 coefficients, held by every GPU that loads the library);
 * larger requests return B2_ESIZE. The entry point calls no cudaMalloc/cudaFree and no
 * allocating library routine. The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress with that device current); make that first call at set-up, before any
 * stream capture. All calls share the one array and it keeps the previous call's contents (every
 * word read is written first, so nothing needs clearing): two calls that overlap on the GPU -
 * different streams, or different contexts on one device - race on it; serialise them. */
int b2_rescale_static(b2_ctx *ctx, size_t size_Ql, size_t n_poly, const uint64_t *d_in,
                      uint64_t *d_out, void *stream);

/* replaces get_elt_from_step (include/galois.cuh:16-49); returns 0 when the step is out of range */
uint32_t b2_galois_elt_from_step(int step, size_t N);
/* replaces PhantomGaloisTool's table construction (include/galois.cuh:98-113): makes the
 * NTT-domain gather table of one Galois element resident on the device (idempotent) */
int b2_galois_prepare(b2_ctx *ctx, uint32_t galois_elt);
/* replaces PhantomGaloisTool::apply_galois_ntt (src/galois.cu:11-18, 86-102):
 * d_dst[l][i] = d_src[l][perm[i]] over n_limbs limbs (d_dst != d_src) */
int b2_galois_permute(b2_ctx *ctx, uint32_t galois_elt, const uint64_t *d_src, uint64_t *d_dst,
                      size_t n_limbs, void *stream);

/* replaces apply_galois_with_ksk / rotate (src/evaluate.cu:1607-1730): d_out may alias d_ct.
 * d_out [2][size_Ql][N] = key-switched automorphism of d_ct */
int b2_apply_galois(b2_ctx *ctx, size_t size_Ql, uint32_t galois_elt, const uint64_t *d_ct,
                    const uint64_t *const *ksk, size_t n_evk, uint64_t *d_out, void *d_ws,
                    size_t ws_bytes, void *stream);

/* replaces hoisting_inplace (src/evaluate.cu:1732-1927): d_out [2][size_Ql][N] = the SUM over the n_steps Galois
 * elements of the rotated d_ct, from one ModUp of c1 and one ModDown per polynomial (ksk and workspace as for
 * b2_hoist_rotations; d_out must not alias d_ct) */
int b2_hoisting_sum(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_ct, const uint32_t *elts, size_t n_steps,
                    const uint64_t *const *ksk, size_t n_evk, uint64_t *d_out, void *d_ws, size_t ws_bytes,
                    void *stream);

/* Rotations that are summed afterwards (the giant steps of a BSGS linear transform) can share one ModDown.
 * No counterpart in the reference, which runs apply_galois per giant (src/bootstrap.cu:1290-1340):
 *   b2_apply_galois_accumulate: d_acc [2][size_Ql][N] (+)= (perm(c0), 0) + Q limbs of <ModUp(perm(c1)), key> * P^-1,
 *                               d_accP [2][size_P][N] (+)= P limbs of the same inner product;
 *                               first != 0 starts a new sum (both accumulators are overwritten);
 *   b2_keyswitch_finish:        d_acc -= NTT(BConv(INTT(d_accP)) * P^-1); d_accP is consumed.
 * One accumulate + finish equals b2_apply_galois bit for bit. Workspace: B2_OP_ROTATE bytes for accumulate,
 * 2 * size_Ql limbs for finish. */
int b2_apply_galois_accumulate(b2_ctx *ctx, size_t size_Ql, uint32_t galois_elt, const uint64_t *d_ct,
                               const uint64_t *const *ksk, size_t n_evk, uint64_t *d_acc, uint64_t *d_accP,
                               int first, void *d_ws, size_t ws_bytes, void *stream);
int b2_keyswitch_finish(b2_ctx *ctx, size_t size_Ql, uint64_t *d_accP, uint64_t *d_acc, void *d_ws,
                        size_t ws_bytes, void *stream);

/* replaces hoist_rotations (src/evaluate.cu:1929-2082): one ModUp of c1 shared by n_steps
 * automorphisms. ksk[s * n_evk + d] = digit d of the key of elts[s]; d_outs[s] -> [2][size_Ql][N] */
int b2_hoist_rotations(b2_ctx *ctx, size_t size_Ql, const uint64_t *d_ct, const uint32_t *elts,
                       size_t n_steps, const uint64_t *const *ksk, size_t n_evk,
                       uint64_t *const *d_outs, void *d_ws, size_t ws_bytes, void *stream);

/* replaces mac_accumulate_kernel (src/bsgs.cu:51-96): d_out [2][size_Ql][N] =
 * sum_b pts[b] (.) babies[b], pts[b] -> [size_Ql][N], babies[b] -> [2][size_Ql][N] (device ptrs) */
int b2_bsgs_mac(b2_ctx *ctx, size_t size_Ql, size_t M, const uint64_t *const *pts,
                const uint64_t *const *babies, uint64_t *d_out, void *stream);

/* the same for 1 to 4 giants in one launch (no counterpart in the reference): d_outs[g] = sum_b pts[g * M + b] (.) babies[b],
 * a null pts entry skips that term. The babies are read once per launch instead of once per giant.
 * pts, babies, d_outs are DEVICE arrays of device pointers. */
int b2_bsgs_mac_multi(b2_ctx *ctx, size_t size_Ql, size_t M, size_t n_giants, const uint64_t *const *pts,
                      const uint64_t *const *babies, uint64_t *const *d_outs, void *stream);

/* replaces expand_single_chain_to_full and the per-diagonal expansion inside the BSGS driver
 * (src/single_chain_plaintext.cu:93-192, src/bsgs.cu:282-315, src/bootstrap.cu:660-686):
 * d_signed int64[N] (signed, centred coefficients, device) -> d_out [size_Ql][N] in NTT form */
int b2_expand_single_chain(b2_ctx *ctx, size_t size_Ql, const int64_t *d_signed, uint64_t *d_out,
                           void *stream);

/* M of them in one go (what the BSGS driver does per giant step, src/bsgs.cu:282-315):
 * d_signed int64[M][N] -> d_out [M][size_Ql][N] in NTT form, two launches for the expansion and two for all transforms */
int b2_expand_single_chain_batch(b2_ctx *ctx, size_t size_Ql, size_t M, const int64_t *d_signed, uint64_t *d_out,
                                 void *stream);

/* the same over any limb range [first_prime, first_prime + n_limbs), optionally left in coefficient
 * form: what the samplers and the encoder of the reference do per limb when they reduce a small
 * signed value into every prime (src/rns_base.cu:49-73, src/prng.cu:142-240) */
int b2_expand_signed(b2_ctx *ctx, size_t first_prime, size_t n_limbs, const int64_t *d_signed,
                     uint64_t *d_out, int to_ntt, void *stream);

/* replaces add/sub/multiply_rns_poly (src/polymath.cu:17-180) over [n_limbs][N], limb i on prime i;
 * op: 0 add, 1 sub, 2 multiply, 3 negate (d_b ignored). d_out may alias an input. */
int b2_poly_op(b2_ctx *ctx, int op, size_t n_limbs, const uint64_t *d_a, const uint64_t *d_b,
               uint64_t *d_out, void *stream);

/* b2_poly_op over a whole ciphertext [n_poly][size_Ql][N] in one launch (limb t of polynomial p on prime t).
 * op 0 add, 1 sub: d_b is a ciphertext of the same shape; op 2: d_b is ONE polynomial [size_Ql][N] (a
 * plaintext) multiplied into every polynomial (multiply_plain, src/evaluate.cu:1150-1200); op 3 negate. */
int b2_ct_op(b2_ctx *ctx, int op, size_t size_Ql, size_t n_poly, const uint64_t *d_a, const uint64_t *d_b,
             uint64_t *d_out, void *stream);
/* every polynomial of a ciphertext times the per-limb integer h_scalars[i] (see b2_poly_scalar, op 1) */
int b2_ct_scalar(b2_ctx *ctx, size_t size_Ql, size_t n_poly, const uint64_t *d_a, const uint64_t *h_scalars,
                 uint64_t *d_out, void *stream);

/* d_out [n_poly][size_Ql][N] = sum_t term_t * h_scalars[t][limb]  (+ h_const[limb] on polynomial 0, may be NULL):
 * the weighted sums of Chebyshev basis ciphertexts in EvalMod, which the reference forms with one
 * multiply_plain by an encoded constant vector and one add per term (src/evalmod.cu:287-334). Term t is a
 * ciphertext with h_term_limbs[t] >= size_Ql limbs per polynomial (only its first size_Ql are read).
 * All h_* arrays live on the host; at most 8 terms and 32 limbs. */
int b2_ct_lincomb(b2_ctx *ctx, size_t size_Ql, size_t n_poly, size_t n_terms, const uint64_t *const *h_terms,
                  const uint32_t *h_term_limbs, const uint64_t *h_scalars, const uint64_t *h_const,
                  uint64_t *d_out, void *stream);

/* per-limb integer constants over [n_limbs][N], limb i on prime i: op 0 adds h_scalars[i] to every
 * value of limb i (in NTT form that is adding the constant polynomial h_scalars[i]); op 1 multiplies
 * limb i by h_scalars[i] (replaces multiply_scalar_per_tower_kernel, src/bootstrap.cu:1535-1565).
 * h_scalars is a HOST array of n_limbs (<= 64) reduced residues. d_out may alias d_a. */
int b2_poly_scalar(b2_ctx *ctx, int op, size_t n_limbs, const uint64_t *d_a, const uint64_t *h_scalars,
                   uint64_t *d_out, void *stream);

/* RNS-limb sharding of one key switch over `world` GPUs (no counterpart in the reference, which
 * has no multi-GPU path; replaces keyswitch_inplace, src/eval_key_switch.cu:294-381, on a slice).
 * Rank r owns the Q limbs [r l/world, (r+1) l/world) and the P limbs [r alpha/world, (r+1) alpha/world).
 * b2_ctx_set_shard builds this rank's lists (synchronises the device; call at set-up).
 * b2_shard_limbs: out4 = {first Q limb, Q count, first P limb, P count} at a level.
 * b2_shard_keyswitch_phase runs the rank-local part of phase 0, 1 or 2; between the phases the
 * caller all-gathers, over all ranks, (after 0) the l limbs at d_ws[0 .. l N) and (after 1) the
 * 2 alpha limbs at d_ws[(l + beta (l+alpha)) N ..), laid out [2][alpha][N]. Buffers are full size on
 * every rank; only the owned limbs of d_c2, evk and d_ct are read, only the owned limbs of d_ct
 * are updated. */
int b2_ctx_set_shard(b2_ctx *ctx, int rank, int world);
int b2_shard_limbs(const b2_ctx *ctx, size_t size_Ql, uint32_t *out4);
int b2_shard_keyswitch_phase(b2_ctx *ctx, size_t size_Ql, int phase, const uint64_t *d_c2,
                             const uint64_t *const *evk, size_t n_evk, uint64_t *d_ct, void *d_ws,
                             size_t ws_bytes, void *stream);

/* Exchange buffers for the limb-sharded pipeline on one node (no counterpart in the reference): device memory with a 64-byte
 * CUDA IPC handle (b2_peer_alloc), a peer's mapping of it (b2_peer_open / b2_peer_close), and an asynchronous copy into it on
 * a stream (b2_peer_copy: DMA over NVLink, no kernel). The caller orders a consumer after every peer's copies (a collective
 * barrier on the same stream does). */
int b2_peer_alloc(size_t bytes, void **d_ptr, uint8_t *handle64);
int b2_peer_open(const uint8_t *handle64, void **d_ptr);
int b2_peer_close(void *d_ptr);
int b2_peer_free(void *d_ptr);
int b2_peer_copy(void *d_dst, const void *d_src, size_t bytes, void *stream);

/* The same three phases for `batch` ciphertexts at once, all switched with one key: d_c2 [batch][size_Ql][N], d_ct
 * [batch][2][size_Ql][N]. Every kernel of a phase is one launch over the whole batch, so a rank that owns an eighth of the
 * limbs still fills its GPU. Workspace (b2_shard_batch_workspace_bytes), in limbs of N words:
 *   T   [size_Ql][batch]           scaled coefficient form of c2; this rank's Q limbs are one contiguous block
 *   CXP [alpha][2][batch]          P limbs of both polynomials; this rank's P limbs are one contiguous block
 *   UP  [batch][beta][size_Ql + alpha]
 * so the caller needs ONE all-gather of T after phase 0 and ONE of CXP after phase 1. Needs the tensor-core base
 * conversion (the default where alpha <= 8). No counterpart in the reference, which has no multi-GPU path. */
size_t b2_shard_batch_workspace_bytes(const b2_ctx *ctx, size_t size_Ql, size_t batch);
int b2_shard_keyswitch_phase_batch(b2_ctx *ctx, size_t size_Ql, int phase, size_t batch, const uint64_t *d_c2,
                                   const uint64_t *const *evk, size_t n_evk, uint64_t *d_ct, void *d_ws,
                                   size_t ws_bytes, void *stream);

/* Measurement hooks (no counterpart in the reference, which times with CUDATimer around whole
 * calls, include/cuda_wrapper.cuh:191-283). b2_launch_count: kernels launched by this library in
 * this process so far. b2_profile_start/stop: while on, every kernel launch is bracketed by CUDA
 * events on its own stream; stop synchronises the device and returns, per kernel name (names
 * joined by ';'), the summed duration in ms and the number of launches. */
uint64_t b2_launch_count(void);
/* b2_device_status: synchronises the context's device and returns in *status the status word its kernels
 * set (0: nothing happened; bit 0: a bounded wait inside a kernel - the tensor-core base conversion waiting
 * for its MMA - ran out and that tile's outputs were not written). No counterpart in the reference, whose
 * kernels have no device-side wait. */
int b2_device_status(b2_ctx *ctx, uint32_t *status);
int b2_profile_start(b2_ctx *ctx);
int b2_profile_stop(b2_ctx *ctx, char *names, size_t names_cap, float *total_ms, uint32_t *launches,
                    size_t cap, size_t *n_out);

#ifdef __cplusplus
}
#endif
#endif
