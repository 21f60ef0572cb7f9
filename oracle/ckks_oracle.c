/*
 * ckks_oracle.c - CPU restatement of the reference's CKKS key-switching / NTT path.
 * TEST INFRASTRUCTURE ONLY (see ckks_oracle.h). Plain C11 + OpenMP over limbs.
 *
 * Every kernel of the reference on this path writes canonical residues in [0,q), so the
 * restatement is free to use the simplest arithmetic (unsigned __int128 products, '%'):
 * what must match is the tables (primes, minimal roots, bit-reversed twiddle order), the
 * digit partition and the ORDER of the approximate base conversions.
 */
#include "ckks_oracle.h"

#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef unsigned __int128 u128;

/* ------------------------------------------------------------------------------------------ */
/* scalar helpers                                                                               */
/* ------------------------------------------------------------------------------------------ */
uint64_t ora_mulmod(uint64_t a, uint64_t b, uint64_t q) { return (uint64_t)(((u128)a * b) % q); }

uint64_t ora_powmod(uint64_t a, uint64_t e, uint64_t q) {
    uint64_t r = 1 % q;
    a %= q;
    while (e) {
        if (e & 1) r = ora_mulmod(r, a, q);
        a = ora_mulmod(a, a, q);
        e >>= 1;
    }
    return r;
}

/* q prime */
uint64_t ora_invmod(uint64_t a, uint64_t q) { return ora_powmod(a, q - 2, q); }

static inline uint64_t addmod(uint64_t a, uint64_t b, uint64_t q) {
    uint64_t s = a + b;
    return s >= q ? s - q : s;
}
static inline uint64_t submod(uint64_t a, uint64_t b, uint64_t q) { return a >= b ? a - b : a + q - b; }

/* Deterministic Miller-Rabin for 64-bit values. The reference (src/host/numth.cu:118-205)
 * runs a probabilistic Miller-Rabin; both agree on primality for every input. */
int ora_is_prime(uint64_t v) {
    static const uint64_t bases[12] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
    if (v < 2) return 0;
    for (int i = 0; i < 12; i++) {
        if (v == bases[i]) return 1;
        if (v % bases[i] == 0) return 0;
    }
    uint64_t d = v - 1;
    int r = 0;
    while ((d & 1) == 0) { d >>= 1; r++; }
    for (int i = 0; i < 12; i++) {
        uint64_t x = ora_powmod(bases[i], d, v);
        if (x == 1 || x == v - 1) continue;
        int comp = 1;
        for (int j = 1; j < r; j++) {
            x = ora_mulmod(x, x, v);
            if (x == v - 1) { comp = 0; break; }
        }
        if (comp) return 0;
    }
    return 1;
}

/* src/host/numth.cu:207-232 (get_primes) driven as in src/host/modulus.cu:80-111 (Create). */
int ora_create_coeff_modulus(size_t N, const int *bit_sizes, size_t count, uint64_t *out) {
    if (count > ORA_MAX_LIMBS) return -1;
    uint64_t factor = 2 * (uint64_t)N;
    /* for each distinct bit size: the list of the first k qualifying primes, descending */
    for (size_t i = 0; i < count; i++) out[i] = 0;
    for (int bits = 2; bits <= 60; bits++) {
        size_t need = 0;
        for (size_t i = 0; i < count; i++) need += (bit_sizes[i] == bits);
        if (!need) continue;
        uint64_t found[ORA_MAX_LIMBS];
        size_t nf = 0;
        uint64_t value = ((uint64_t)1 << bits);
        if (value < factor) return -2;
        value = value - factor + 1;
        uint64_t lower = (uint64_t)1 << (bits - 1);
        while (nf < need && value > lower) {
            if (ora_is_prime(value)) found[nf++] = value;
            if (value < factor) break;
            value -= factor;
        }
        if (nf < need) return -3;
        /* Create pops from the back: the smallest found prime goes to the first request */
        for (size_t i = 0; i < count; i++)
            if (bit_sizes[i] == bits) out[i] = found[--nf];
    }
    for (size_t i = 0; i < count; i++)
        if (!out[i]) return -4;
    return 0;
}

/* src/host/numth.cu:309-332. The reference starts from a random primitive root and walks all
 * odd powers keeping the minimum; the minimum over the whole set does not depend on the start. */
uint64_t ora_minimal_primitive_root(uint64_t degree, uint64_t q) {
    if ((q - 1) % degree) return 0;
    uint64_t cof = (q - 1) / degree, root = 0;
    for (uint64_t g = 2; g < q; g++) {
        uint64_t r = ora_powmod(g, cof, q);
        if (ora_powmod(r, degree >> 1, q) == q - 1) { root = r; break; }
    }
    uint64_t sq = ora_mulmod(root, root, q), cur = root, best = root;
    for (uint64_t i = 0; i < degree / 2; i++) {
        if (cur < best) best = cur;
        cur = ora_mulmod(cur, sq, q);
    }
    return best;
}

uint32_t ora_bitrev(uint32_t x, int bits) {
    uint32_t r = 0;
    for (int i = 0; i < bits; i++) r |= ((x >> i) & 1u) << (bits - 1 - i);
    return r;
}

/* ------------------------------------------------------------------------------------------ */
/* synthetic data                                                                               */
/* ------------------------------------------------------------------------------------------ */
static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

uint64_t ora_uniform_at(uint64_t seed, uint64_t i, uint64_t q) {
    int bits = 64 - __builtin_clzll(q);
    uint64_t mask = bits >= 64 ? ~0ULL : (((uint64_t)1 << bits) - 1);
    uint64_t base = mix64(seed * 0x9E3779B97F4A7C15ULL + 0x632BE59BD9B4E019ULL) + i * 0xD1342543DE82EF95ULL;
    for (uint64_t k = 0;; k++) {
        uint64_t v = mix64(base + k * 0x9E3779B97F4A7C15ULL) & mask;
        if (v < q) return v;
    }
}

void ora_fill_uniform(uint64_t *dst, size_t n, uint64_t q, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) dst[i] = ora_uniform_at(seed, i, q);
}

void ora_fill_limbs(uint64_t *dst, size_t N, const uint64_t *primes, size_t n_limbs,
                    uint64_t case_seed, uint64_t buf, uint64_t limb0) {
    for (size_t l = 0; l < n_limbs; l++)
        ora_fill_uniform(dst + l * N, N, primes[l], (case_seed << 40) ^ (buf << 16) ^ (limb0 + l));
}

uint64_t ora_limb_hash(const uint64_t *x, size_t n) {
    uint64_t h = 0;
    for (size_t i = 0; i < n; i++) h += mix64(x[i] ^ mix64((uint64_t)i + 1));
    return h;
}

/* ------------------------------------------------------------------------------------------ */
/* context                                                                                      */
/* ------------------------------------------------------------------------------------------ */
struct ora_ctx {
    size_t N;
    int logN;
    size_t size_QP, size_Q, size_P;
    uint64_t q[ORA_MAX_LIMBS];
    uint64_t root[ORA_MAX_LIMBS];
    uint64_t ninv[ORA_MAX_LIMBS];
    uint64_t *tw[ORA_MAX_LIMBS];  /* tw[br(i)] = psi^i            (src/host/ntt.cu:22-33) */
    uint64_t *itw[ORA_MAX_LIMBS]; /* itw[br(i)] = psi^-i; itw[1] *= N^-1 (src/host/ntt.cu:35-55) */
};

ora_ctx *ora_ctx_create(size_t N, const uint64_t *primes, size_t size_QP, size_t size_P) {
    if (size_QP > ORA_MAX_LIMBS || size_P >= size_QP || (N & (N - 1)) || N < 2) return NULL;
    ora_ctx *c = (ora_ctx *)calloc(1, sizeof(ora_ctx));
    c->N = N;
    c->logN = __builtin_ctzll(N);
    c->size_QP = size_QP;
    c->size_P = size_P;
    c->size_Q = size_QP - size_P;
    int bad = 0;
#pragma omp parallel for schedule(dynamic)
    for (size_t l = 0; l < size_QP; l++) {
        uint64_t q = primes[l];
        c->q[l] = q;
        uint64_t psi = ora_minimal_primitive_root(2 * N, q);
        if (!psi) { bad = 1; continue; }
        uint64_t ipsi = ora_invmod(psi, q);
        c->root[l] = psi;
        c->ninv[l] = ora_invmod(N % q, q);
        c->tw[l] = (uint64_t *)malloc(N * sizeof(uint64_t));
        c->itw[l] = (uint64_t *)malloc(N * sizeof(uint64_t));
        uint64_t p = psi, ip = ipsi;
        c->tw[l][0] = 1;
        c->itw[l][0] = 1;
        for (size_t i = 1; i < N; i++) {
            uint32_t r = ora_bitrev((uint32_t)i, c->logN);
            c->tw[l][r] = p;
            c->itw[l][r] = ip;
            p = ora_mulmod(p, psi, q);
            ip = ora_mulmod(ip, ipsi, q);
        }
        if (N > 1) c->itw[l][1] = ora_mulmod(c->itw[l][1], c->ninv[l], q);
    }
    if (bad) { ora_ctx_destroy(c); return NULL; }
    return c;
}

void ora_ctx_destroy(ora_ctx *c) {
    if (!c) return;
    for (size_t l = 0; l < c->size_QP; l++) { free(c->tw[l]); free(c->itw[l]); }
    free(c);
}
size_t ora_ctx_N(const ora_ctx *c) { return c->N; }
const uint64_t *ora_ctx_twiddle(const ora_ctx *c, size_t i) { return c->tw[i]; }
const uint64_t *ora_ctx_itwiddle(const ora_ctx *c, size_t i) { return c->itw[i]; }
uint64_t ora_ctx_root(const ora_ctx *c, size_t i) { return c->root[i]; }
size_t ora_beta(const ora_ctx *c, size_t size_Ql) { return (size_Ql + c->size_P - 1) / c->size_P; }

/* physical prime index of logical limb t of a [size_Ql + size_P] buffer
 * (src/eval_key_switch.cu:181-182; src/ntt/fntt_2d.cu:440-443) */
static inline size_t phys(const ora_ctx *c, size_t size_Ql, size_t t) {
    return t < size_Ql ? t : c->size_Q + (t - size_Ql);
}

/* ------------------------------------------------------------------------------------------ */
/* transforms                                                                                   */
/* ------------------------------------------------------------------------------------------ */
/* src/ntt/ntt_1d.cu:41-60 with include/butterfly.cuh:17-40: Cooley-Tukey, natural order in,
 * bit-reversed out, twiddle index m+k. */
static void ntt_fwd_limb(uint64_t *x, size_t N, uint64_t q, const uint64_t *tw) {
    size_t t = N >> 1;
    for (size_t m = 1; m < N; m <<= 1, t >>= 1) {
        for (size_t k = 0; k < m; k++) {
            uint64_t w = tw[m + k];
            uint64_t *a = x + 2 * k * t, *b = a + t;
            for (size_t j = 0; j < t; j++) {
                uint64_t u = a[j], v = ora_mulmod(b[j], w, q);
                a[j] = addmod(u, v, q);
                b[j] = submod(u, v, q);
            }
        }
    }
}

/* src/ntt/ntt_1d.cu:221-244 with include/butterfly.cuh:42-71: Gentleman-Sande, bit-reversed
 * in, natural out. The last stage uses itw[1] (which already carries N^-1) on the y outputs
 * and multiplies the x outputs by N^-1 (include/ntt_radix8_tmpl.cuh:566-568). */
static void ntt_inv_limb(uint64_t *x, size_t N, uint64_t q, const uint64_t *itw, uint64_t ninv) {
    size_t t = 1;
    for (size_t m = N >> 1; m >= 1; m >>= 1, t <<= 1) {
        for (size_t k = 0; k < m; k++) {
            uint64_t w = itw[m + k];
            uint64_t *a = x + 2 * k * t, *b = a + t;
            for (size_t j = 0; j < t; j++) {
                uint64_t u = a[j], v = b[j];
                uint64_t s = addmod(u, v, q);
                a[j] = (m == 1) ? ora_mulmod(s, ninv, q) : s;
                b[j] = ora_mulmod(submod(u, v, q), w, q);
            }
        }
    }
}

void ora_ntt_forward(const ora_ctx *c, uint64_t *data, size_t n_limbs, size_t first_prime) {
#pragma omp parallel for schedule(dynamic)
    for (size_t l = 0; l < n_limbs; l++)
        ntt_fwd_limb(data + l * c->N, c->N, c->q[first_prime + l], c->tw[first_prime + l]);
}

void ora_ntt_inverse(const ora_ctx *c, uint64_t *data, size_t n_limbs, size_t first_prime) {
#pragma omp parallel for schedule(dynamic)
    for (size_t l = 0; l < n_limbs; l++)
        ntt_inv_limb(data + l * c->N, c->N, c->q[first_prime + l], c->itw[first_prime + l],
                     c->ninv[first_prime + l]);
}

/* ------------------------------------------------------------------------------------------ */
/* base conversion pieces                                                                       */
/* ------------------------------------------------------------------------------------------ */
/* (prod_{k in set, k != skip} m_k) mod p ; set given as physical prime indices */
static uint64_t punctured_prod_mod(const ora_ctx *c, const size_t *set, size_t n, size_t skip, uint64_t p) {
    uint64_t r = 1 % p;
    for (size_t k = 0; k < n; k++)
        if (k != skip) r = ora_mulmod(r, c->q[set[k]] % p, p);
    return r;
}

/* Fast (approximate) base conversion of the residues in[i][*] (i over `iset`, coefficient form)
 * to one output prime p:  sum_i (in_i * hatinv_i mod m_i) * (hat_i mod p) mod p.
 * src/rns_bconv.cu:40-60 (scale), :143-168 / :455-485 (accumulate in 128 bits, one reduction;
 * include/rns_bconv.cuh:112-125). `scaled` says the inputs already carry hatinv_i. */
static void bconv_to_prime(const ora_ctx *c, const size_t *iset, size_t ni, const uint64_t *const *in,
                           int scaled, uint64_t p, uint64_t *out) {
    uint64_t hatinv[ORA_MAX_LIMBS], hatp[ORA_MAX_LIMBS];
    for (size_t i = 0; i < ni; i++) {
        uint64_t mi = c->q[iset[i]];
        hatinv[i] = ora_invmod(punctured_prod_mod(c, iset, ni, i, mi), mi);
        hatp[i] = punctured_prod_mod(c, iset, ni, i, p);
    }
    for (size_t j = 0; j < c->N; j++) {
        u128 acc = 0; /* the reference keeps a 128-bit sum; reduce as we go, same value mod p */
        for (size_t i = 0; i < ni; i++) {
            uint64_t y = scaled ? in[i][j] : ora_mulmod(in[i][j], hatinv[i], c->q[iset[i]]);
            acc = (acc + (u128)y * hatp[i]) % p;
        }
        out[j] = (uint64_t)acc;
    }
}

/* src/rns_bconv.cu:530-628 (alpha > 1 path; alpha == 1 at :432-453 is the same formula with a
 * one-term sum). Digit d = limbs [alpha*d, min(alpha*(d+1), size_Ql)). */
void ora_modup(const ora_ctx *c, size_t size_Ql, const uint64_t *c2, uint64_t *out) {
    size_t N = c->N, alpha = c->size_P, beta = ora_beta(c, size_Ql), size_QlP = size_Ql + alpha;
    uint64_t *t = (uint64_t *)malloc(size_Ql * N * sizeof(uint64_t));
    memcpy(t, c2, size_Ql * N * sizeof(uint64_t));
    ora_ntt_inverse(c, t, size_Ql, 0); /* :558 nwt_2d_radix8_backward_scale (scale folded below) */
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (size_t d = 0; d < beta; d++) {
        for (size_t tl = 0; tl < size_QlP; tl++) {
            size_t start = alpha * d, end = start + alpha < size_Ql ? start + alpha : size_Ql;
            uint64_t *dst = out + (d * size_QlP + tl) * N;
            if (tl >= start && tl < end) { /* :563-564 modup_copy_partQl_kernel */
                memcpy(dst, c2 + tl * N, N * sizeof(uint64_t));
                continue;
            }
            size_t iset[ORA_MAX_LIMBS];
            const uint64_t *in[ORA_MAX_LIMBS];
            for (size_t i = start; i < end; i++) { iset[i - start] = i; in[i - start] = t + i * N; }
            size_t pp = phys(c, size_Ql, tl);
            bconv_to_prime(c, iset, end - start, in, 0, c->q[pp], dst); /* :610-613 */
            ntt_fwd_limb(dst, N, c->q[pp], c->tw[pp]);                  /* :618-620 */
        }
    }
    free(t);
}

/* src/eval_key_switch.cu:175-230: 128-bit accumulate over the digits, one Barrett at the end
 * (reduction_threshold != 0 on this path, :355-356). */
void ora_ks_inner_prod(const ora_ctx *c, size_t size_Ql, const uint64_t *digits,
                       const uint64_t *const *evk, uint64_t *out) {
    size_t N = c->N, alpha = c->size_P, beta = ora_beta(c, size_Ql), size_QlP = size_Ql + alpha;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (size_t k = 0; k < 2; k++) {
        for (size_t tl = 0; tl < size_QlP; tl++) {
            size_t pp = phys(c, size_Ql, tl);
            uint64_t q = c->q[pp];
            uint64_t *dst = out + (k * size_QlP + tl) * N;
            for (size_t j = 0; j < N; j++) {
                u128 acc = 0;
                for (size_t d = 0; d < beta; d++) {
                    uint64_t x = digits[(d * size_QlP + tl) * N + j];
                    uint64_t e = evk[d][(k * c->size_QP + pp) * N + j];
                    acc = (acc + (u128)x * e) % q;
                }
                dst[j] = (uint64_t)acc;
            }
        }
    }
}

/* src/rns_bconv.cu:776-828: INTT of the P limbs, P -> Q_l conversion (bConv_BEHZ, :212-229),
 * forward NTT, (cx - delta) * P^-1 (include/ntt_radix8_tmpl.cuh:203-233). */
void ora_moddown(const ora_ctx *c, size_t size_Ql, const uint64_t *cx, uint64_t *out) {
    size_t N = c->N, alpha = c->size_P;
    uint64_t *z = (uint64_t *)malloc(alpha * N * sizeof(uint64_t));
    memcpy(z, cx + size_Ql * N, alpha * N * sizeof(uint64_t));
    ora_ntt_inverse(c, z, alpha, c->size_Q);
    size_t iset[ORA_MAX_LIMBS];
    const uint64_t *in[ORA_MAX_LIMBS];
    for (size_t i = 0; i < alpha; i++) { iset[i] = c->size_Q + i; in[i] = z + i * N; }
#pragma omp parallel for schedule(dynamic)
    for (size_t j = 0; j < size_Ql; j++) {
        uint64_t q = c->q[j];
        uint64_t *delta = out + j * N;
        bconv_to_prime(c, iset, alpha, in, 0, q, delta);
        ntt_fwd_limb(delta, N, q, c->tw[j]);
        uint64_t P = 1;
        for (size_t i = 0; i < alpha; i++) P = ora_mulmod(P, c->q[c->size_Q + i] % q, q);
        uint64_t Pinv = ora_invmod(P, q); /* src/rns.cu:100-138 bigPInv_mod_q */
        for (size_t i = 0; i < N; i++)
            delta[i] = ora_mulmod(submod(cx[j * N + i], delta[i], q), Pinv, q);
    }
    free(z);
}

/* src/eval_key_switch.cu:294-381 */
void ora_keyswitch(const ora_ctx *c, size_t size_Ql, const uint64_t *c2,
                   const uint64_t *const *evk, uint64_t *ct) {
    size_t N = c->N, alpha = c->size_P, beta = ora_beta(c, size_Ql), size_QlP = size_Ql + alpha;
    uint64_t *up = (uint64_t *)malloc(beta * size_QlP * N * sizeof(uint64_t));
    uint64_t *cx = (uint64_t *)malloc(2 * size_QlP * N * sizeof(uint64_t));
    uint64_t *dn = (uint64_t *)malloc(size_Ql * N * sizeof(uint64_t));
    ora_modup(c, size_Ql, c2, up);
    ora_ks_inner_prod(c, size_Ql, up, evk, cx);
    for (size_t k = 0; k < 2; k++) {
        ora_moddown(c, size_Ql, cx + k * size_QlP * N, dn);
        ora_add(c, size_Ql, ct + k * size_Ql * N, dn, ct + k * size_Ql * N); /* :376-378 add_to_ct_kernel */
    }
    free(up); free(cx); free(dn);
}

/* ------------------------------------------------------------------------------------------ */
/* evaluator pieces                                                                             */
/* ------------------------------------------------------------------------------------------ */
void ora_add(const ora_ctx *c, size_t n_limbs, const uint64_t *a, const uint64_t *b, uint64_t *o) {
#pragma omp parallel for schedule(static)
    for (size_t l = 0; l < n_limbs; l++)
        for (size_t i = 0; i < c->N; i++) o[l * c->N + i] = addmod(a[l * c->N + i], b[l * c->N + i], c->q[l]);
}
void ora_sub(const ora_ctx *c, size_t n_limbs, const uint64_t *a, const uint64_t *b, uint64_t *o) {
#pragma omp parallel for schedule(static)
    for (size_t l = 0; l < n_limbs; l++)
        for (size_t i = 0; i < c->N; i++) o[l * c->N + i] = submod(a[l * c->N + i], b[l * c->N + i], c->q[l]);
}
void ora_mul(const ora_ctx *c, size_t n_limbs, const uint64_t *a, const uint64_t *b, uint64_t *o) {
#pragma omp parallel for schedule(static)
    for (size_t l = 0; l < n_limbs; l++)
        for (size_t i = 0; i < c->N; i++) o[l * c->N + i] = ora_mulmod(a[l * c->N + i], b[l * c->N + i], c->q[l]);
}

/* src/polymath.cu:463-498: d0 = a0 b0, d2 = a1 b1, d1 = (a0+a1)(b0+b1) - d0 - d2 */
void ora_tensor_mul(const ora_ctx *c, size_t size_Ql, const uint64_t *a, const uint64_t *b, uint64_t *out) {
    size_t N = c->N, S = size_Ql * N;
#pragma omp parallel for schedule(static)
    for (size_t l = 0; l < size_Ql; l++) {
        uint64_t q = c->q[l];
        for (size_t i = 0; i < N; i++) {
            size_t o = l * N + i;
            uint64_t a0 = a[o], a1 = a[S + o], b0 = b[o], b1 = b[S + o];
            uint64_t d0 = ora_mulmod(a0, b0, q), d2 = ora_mulmod(a1, b1, q);
            uint64_t d1 = ora_mulmod(addmod(a0, a1, q), addmod(b0, b1, q), q);
            out[o] = d0;
            out[S + o] = submod(submod(d1, d0, q), d2, q);
            out[2 * S + o] = d2;
        }
    }
}

void ora_multiply_and_relin(const ora_ctx *c, size_t size_Ql, const uint64_t *a, const uint64_t *b,
                            const uint64_t *const *rlk, uint64_t *out) {
    size_t S = size_Ql * c->N;
    uint64_t *t = (uint64_t *)malloc(3 * S * sizeof(uint64_t));
    ora_tensor_mul(c, size_Ql, a, b, t);
    memcpy(out, t, 2 * S * sizeof(uint64_t));
    ora_keyswitch(c, size_Ql, t + 2 * S, rlk, out); /* src/evaluate.cu:1342-1374 */
    free(t);
}

/* src/rns.cu:1128-1183: r = INTT(c_last); out_j = (c_j - NTT(r mod q_j)) * q_last^-1 mod q_j.
 * No rounding offset is added anywhere in that function. */
void ora_rescale(const ora_ctx *c, size_t size_Ql, size_t n_poly, const uint64_t *in, uint64_t *out) {
    size_t N = c->N, last = size_Ql - 1;
    uint64_t qlast = c->q[last];
    for (size_t p = 0; p < n_poly; p++) {
        const uint64_t *ci = in + p * size_Ql * N;
        uint64_t *co = out + p * last * N;
        uint64_t *r = (uint64_t *)malloc(N * sizeof(uint64_t));
        memcpy(r, ci + last * N, N * sizeof(uint64_t));
        ntt_inv_limb(r, N, qlast, c->itw[last], c->ninv[last]);
#pragma omp parallel for schedule(dynamic)
        for (size_t j = 0; j < last; j++) {
            uint64_t q = c->q[j], inv = ora_invmod(qlast % q, q);
            uint64_t *d = co + j * N;
            for (size_t i = 0; i < N; i++) d[i] = r[i] % q;
            ntt_fwd_limb(d, N, q, c->tw[j]);
            for (size_t i = 0; i < N; i++) d[i] = ora_mulmod(submod(ci[j * N + i], d[i], q), inv, q);
        }
        free(r);
    }
}

/* The same with the remainder of the dropped prime taken centred (v > q_last/2 stands for v - q_last),
 * so that coefficients are rounded to nearest. Not in the reference: it states what
 * b2_rescale_rounded computes, for the parity test of that entry point. */
void ora_rescale_rounded(const ora_ctx *c, size_t size_Ql, size_t n_poly, const uint64_t *in, uint64_t *out) {
    size_t N = c->N, last = size_Ql - 1;
    uint64_t qlast = c->q[last], half = qlast >> 1;
    for (size_t p = 0; p < n_poly; p++) {
        const uint64_t *ci = in + p * size_Ql * N;
        uint64_t *co = out + p * last * N;
        uint64_t *r = (uint64_t *)malloc(N * sizeof(uint64_t));
        memcpy(r, ci + last * N, N * sizeof(uint64_t));
        ntt_inv_limb(r, N, qlast, c->itw[last], c->ninv[last]);
#pragma omp parallel for schedule(dynamic)
        for (size_t j = 0; j < last; j++) {
            uint64_t q = c->q[j], inv = ora_invmod(qlast % q, q);
            uint64_t *d = co + j * N;
            for (size_t i = 0; i < N; i++) d[i] = r[i] > half ? submod(r[i] % q, qlast % q, q) : r[i] % q;
            ntt_fwd_limb(d, N, q, c->tw[j]);
            for (size_t i = 0; i < N; i++) d[i] = ora_mulmod(submod(ci[j * N + i], d[i], q), inv, q);
        }
        free(r);
    }
}

/* include/galois.cuh:16-49 */
uint32_t ora_galois_elt_from_step(int step, size_t N) {
    uint32_t n = (uint32_t)N, m = 2 * n;
    if (step == 0) return m - 1;
    int neg = step < 0;
    uint32_t pos = (uint32_t)(neg ? -step : step);
    if (pos >= (n >> 1)) return 0; /* the reference throws "step count too large" */
    uint32_t s = neg ? (n >> 1) - pos : pos;
    uint64_t e = 1;
    while (s--) e = (e * 5) & (m - 1);
    return (uint32_t)e;
}

/* include/galois.cuh:98-113 */
void ora_galois_perm(size_t N, uint32_t galois_elt, uint32_t *perm) {
    int logN = __builtin_ctzll(N);
    for (size_t i = N; i < 2 * N; i++) {
        uint32_t rev = ora_bitrev((uint32_t)i, logN + 1);
        uint64_t raw = (((uint64_t)galois_elt * rev) >> 1) & (N - 1);
        perm[i - N] = ora_bitrev((uint32_t)raw, logN);
    }
}

static void gather(const uint64_t *src, const uint32_t *perm, size_t n_limbs, size_t N, uint64_t *dst) {
#pragma omp parallel for schedule(static)
    for (size_t l = 0; l < n_limbs; l++)
        for (size_t i = 0; i < N; i++) dst[l * N + i] = src[l * N + perm[i]];
}

/* src/evaluate.cu:1607-1656: c0 <- perm(c0); c1 <- 0; key-switch perm(c1) into (c0, c1). */
void ora_apply_galois(const ora_ctx *c, size_t size_Ql, uint32_t galois_elt, const uint64_t *const *ksk,
                      uint64_t *ct) {
    size_t N = c->N, S = size_Ql * N;
    uint32_t *perm = (uint32_t *)malloc(N * sizeof(uint32_t));
    uint64_t *t = (uint64_t *)malloc(2 * S * sizeof(uint64_t));
    ora_galois_perm(N, galois_elt, perm);
    gather(ct, perm, size_Ql, N, t);
    gather(ct + S, perm, size_Ql, N, t + S);
    memcpy(ct, t, S * sizeof(uint64_t));
    memset(ct + S, 0, S * sizeof(uint64_t));
    ora_keyswitch(c, size_Ql, t + S, ksk, ct);
    free(perm); free(t);
}

/* src/evaluate.cu:1929-2082: ModUp(c1) once (:2013-2014); per step gather c0 and every extended
 * digit (:2036-2045), inner product, two ModDowns, c0_out = perm(c0) + cx0, c1_out = cx1. */
void ora_hoist_rotations(const ora_ctx *c, size_t size_Ql, const uint64_t *ct, const uint32_t *elts,
                         size_t n_steps, const uint64_t *const *const *ksk, uint64_t *const *outs) {
    size_t N = c->N, alpha = c->size_P, beta = ora_beta(c, size_Ql), size_QlP = size_Ql + alpha, S = size_Ql * N;
    uint64_t *up = (uint64_t *)malloc(beta * size_QlP * N * sizeof(uint64_t));
    uint64_t *pup = (uint64_t *)malloc(beta * size_QlP * N * sizeof(uint64_t));
    uint64_t *cx = (uint64_t *)malloc(2 * size_QlP * N * sizeof(uint64_t));
    uint64_t *pc0 = (uint64_t *)malloc(S * sizeof(uint64_t));
    uint64_t *dn = (uint64_t *)malloc(S * sizeof(uint64_t));
    uint32_t *perm = (uint32_t *)malloc(N * sizeof(uint32_t));
    ora_modup(c, size_Ql, ct + S, up);
    for (size_t s = 0; s < n_steps; s++) {
        ora_galois_perm(N, elts[s], perm);
        gather(ct, perm, size_Ql, N, pc0);
        gather(up, perm, beta * size_QlP, N, pup);
        ora_ks_inner_prod(c, size_Ql, pup, ksk[s], cx);
        ora_moddown(c, size_Ql, cx, dn);
        ora_add(c, size_Ql, pc0, dn, outs[s]);
        ora_moddown(c, size_Ql, cx + size_QlP * N, outs[s] + S);
    }
    free(up); free(pup); free(cx); free(pc0); free(dn); free(perm);
}

/* src/evaluate.cu:1732-1927 (hoisting_inplace): ModUp(c1) once (:1826-1829); per step gather c0 and every extended
 * digit, inner product, everything summed - c0 over Q_l (:1861-1863), the inner products over Q_l and P (:1876-1882);
 * then one ModDown per polynomial (:1885-1888); out0 = sum perm(c0) + cx0, out1 = cx1 (:1895-1906). */
void ora_hoisting_sum(const ora_ctx *c, size_t size_Ql, const uint64_t *ct, const uint32_t *elts, size_t n_steps,
                      const uint64_t *const *const *ksk, uint64_t *out) {
    size_t N = c->N, alpha = c->size_P, beta = ora_beta(c, size_Ql), size_QlP = size_Ql + alpha, S = size_Ql * N;
    uint64_t *up = (uint64_t *)malloc(beta * size_QlP * N * sizeof(uint64_t));
    uint64_t *pup = (uint64_t *)malloc(beta * size_QlP * N * sizeof(uint64_t));
    uint64_t *cx = (uint64_t *)malloc(2 * size_QlP * N * sizeof(uint64_t));
    uint64_t *acc = (uint64_t *)calloc(2 * size_QlP * N, sizeof(uint64_t));
    uint64_t *acc0 = (uint64_t *)calloc(S, sizeof(uint64_t));
    uint64_t *pc0 = (uint64_t *)malloc(S * sizeof(uint64_t));
    uint64_t *dn = (uint64_t *)malloc(S * sizeof(uint64_t));
    uint32_t *perm = (uint32_t *)malloc(N * sizeof(uint32_t));
    ora_modup(c, size_Ql, ct + S, up);
    for (size_t s = 0; s < n_steps; s++) {
        ora_galois_perm(N, elts[s], perm);
        gather(ct, perm, size_Ql, N, pc0);
        ora_add(c, size_Ql, acc0, pc0, acc0);
        gather(up, perm, beta * size_QlP, N, pup);
        ora_ks_inner_prod(c, size_Ql, pup, ksk[s], cx);
        for (size_t k = 0; k < 2; k++)
            for (size_t t = 0; t < size_QlP; t++) {
                uint64_t q = c->q[t < size_Ql ? t : c->size_Q + (t - size_Ql)];
                uint64_t *a = acc + (k * size_QlP + t) * N;
                const uint64_t *x = cx + (k * size_QlP + t) * N;
                for (size_t i = 0; i < N; i++) a[i] = addmod(a[i], x[i], q);
            }
    }
    ora_moddown(c, size_Ql, acc, dn);
    ora_add(c, size_Ql, acc0, dn, out);
    ora_moddown(c, size_Ql, acc + size_QlP * N, out + S);
    free(up); free(pup); free(cx); free(acc); free(acc0); free(pc0); free(dn); free(perm);
}

/* src/bsgs.cu:51-96 */
void ora_bsgs_mac(const ora_ctx *c, size_t size_Ql, size_t M, const uint64_t *const *pts,
                  const uint64_t *const *babies, uint64_t *out) {
    size_t N = c->N, S = size_Ql * N;
#pragma omp parallel for schedule(static)
    for (size_t l = 0; l < size_Ql; l++) {
        uint64_t q = c->q[l];
        for (size_t i = 0; i < N; i++) {
            size_t o = l * N + i;
            uint64_t a0 = 0, a1 = 0;
            for (size_t b = 0; b < M; b++) {
                uint64_t p = pts[b][o];
                a0 = addmod(a0, ora_mulmod(p, babies[b][o], q), q);
                a1 = addmod(a1, ora_mulmod(p, babies[b][S + o], q), q);
            }
            out[o] = a0;
            out[S + o] = a1;
        }
    }
}

/* src/bootstrap.cu:660-686 (light_pt_expand_per_tower_kernel) followed by the forward NTT of
 * src/bsgs.cu:308-314 / src/single_chain_plaintext.cu:93-192 */
void ora_expand_single_chain(const ora_ctx *c, size_t size_Ql, const int64_t *coeffs, uint64_t *out) {
    size_t N = c->N;
#pragma omp parallel for schedule(dynamic)
    for (size_t l = 0; l < size_Ql; l++) {
        uint64_t q = c->q[l];
        uint64_t *d = out + l * N;
        for (size_t i = 0; i < N; i++) {
            int64_t v = coeffs[i];
            uint64_t mag = v >= 0 ? (uint64_t)v : (uint64_t)0 - (uint64_t)v;
            uint64_t r = mag % q;
            d[i] = (v >= 0 || r == 0) ? r : q - r;
        }
        ntt_fwd_limb(d, N, q, c->tw[l]);
    }
}

/* Fixes the number of OpenMP threads the oracle uses from now on, whatever OMP_NUM_THREADS said when the
 * library was loaded (launchers such as torchrun export OMP_NUM_THREADS=1). n < 1 leaves it unchanged. */
void ora_set_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int ora_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
