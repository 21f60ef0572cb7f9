// ntt_kernels.cuh - two-pass negacyclic NTT / INTT over RNS limbs for sm_100a.
//
// Decomposition. N = N1 * N2 (N1 = 2^LOG_A rows, N2 = 2^LOG_B columns of the row-major limb).
//   forward:  pass A = first LOG_A Cooley-Tukey stages = N2 independent N1-point transforms down
//             the columns; pass B = last LOG_B stages = N1 independent N2-point transforms on the
//             contiguous rows. Natural order in, bit-reversed order out, twiddle index m + k
//             (the reference's convention: src/ntt/ntt_1d.cu:41-60, src/host/ntt.cu:22-33).
//   inverse:  the mirror image with Gentleman-Sande butterflies, rows first.
// One kernel template serves both passes: a CTA owns C sub-transforms of T points, every thread
// keeps EPT = 16 (or 8) residues in registers and runs R1 stages, exchanges once through padded
// shared memory, runs the remaining R2 stages and stores. A limb therefore crosses global memory
// twice per transform (the intermediate of the two passes stays in the 126 MB L2).
//
// Twiddle index algebra (P = 1 for the column pass, P = N1 + row for the row pass):
//   forward, local stage s (0-based inside the T-point sub-transform), pair group k':
//       index = (P << s) + k'
//   inverse, local stage with gap 2^u, pair group k':
//       index = ((T >> (u + 1)) * P) + k'
// Lazy ranges: forward keeps [0,4q), inverse keeps [0,2q); the last pass stores canonical values.
#pragma once
#include <type_traits>
#include "modarith.cuh"

namespace b2 {

struct Mod {
    uint64_t q, r0, r1, pad;  // r = floor(2^128 / q)
};

// One job = one limb transform: where the limb lives and which prime's tables it uses.
// x = slot in the transform's own buffer, y = prime index, z/w = extra slots for epilogues.
// Inverse transforms read limb x of src and write limb w of dst (z selects the final scaling).
using Job = uint4;

// resident threads per SM the pass kernels are compiled for (register cap = 65536 / this)
#ifndef B2_NTT_RESIDENT_THREADS
#define B2_NTT_RESIDENT_THREADS 768
#endif
// (a pass whose threads hold 32 residues each - the 512-point pass of N = 2^17 - gets twice the registers: half the threads)
constexpr int ntt_min_blocks(int threads, int residues_per_thread = 16) {
    return (B2_NTT_RESIDENT_THREADS / (residues_per_thread > 16 ? 2 : 1)) / threads > 0 ? (B2_NTT_RESIDENT_THREADS / (residues_per_thread > 16 ? 2 : 1)) / threads : 1;
}

struct NttArgs {
    const uint64_t *src;  // limb `slot` at src + slot * N
    uint64_t *dst;
    const Job *jobs;       // nullptr: slot = job, prime = first_prime + job
    uint32_t first_prime;
    uint32_t logN;
    const W2 *tw;          // [size_QP][N] {w, shoup(w)}
    const Mod *mod;        // [size_QP]
    const W2 *fin;         // inverse only: [idx][2] = {scale of the x outputs, last-stage twiddle}
    uint32_t period;       // without a job list: limb j uses prime first_prime + j % period (0: + j), a batch of polynomials
    // forward column pass with SRC != 0 (rescale): limb job.x is not read from its own slot but made on the fly from
    // slot job.x / src_div of src, whose words are residues mod src_q, reduced into the limb's prime
    uint32_t src_div;
    uint64_t src_q;
    // A batch of polynomial sets in one launch (the two-pass kernels only): blockIdx.y = set b, and limb slot s of set b
    // lives at slot s * (lm1 + 1) + b * bs of the buffer. Zero-initialised fields mean one set, slots as they are.
    // Batch-major buffers [b][slots] use lm1 = 0, bs = slots per set; limb-major ones [slot][b] use lm1 = batch - 1, bs = 1.
    uint32_t src_lm1, src_bs, dst_lm1, dst_bs;
};

// The sets of a batched launch are the slow grid dimension. With the sets fastest (the CTAs of all sets on one tile next to
// one another, sharing its twiddles in L2) the row passes ran as fast and the column passes 8 % slower on B200.
__device__ __forceinline__ uint32_t set_idx(const NttArgs &) { return blockIdx.y; }
__device__ __forceinline__ uint32_t work_idx(const NttArgs &) { return blockIdx.x; }
__device__ __forceinline__ size_t src_slot(const NttArgs &a, uint32_t slot) { return (size_t)slot * (a.src_lm1 + 1) + (size_t)set_idx(a) * a.src_bs; }
__device__ __forceinline__ size_t dst_slot(const NttArgs &a, uint32_t slot) { return (size_t)slot * (a.dst_lm1 + 1) + (size_t)set_idx(a) * a.dst_bs; }

__device__ __forceinline__ Job get_job(const NttArgs &a, uint32_t j) {
    if (a.jobs) return a.jobs[j];
    const uint32_t p = a.first_prime + (a.period ? j % a.period : j);
    return make_uint4(j, p, p, j);
}

// 256-bit global accesses (sm_100): one lane moves a whole 32-byte sector, so a thread that owns a run of
// consecutive residues touches every sector once instead of twice with 16-byte accesses. p: 32-byte aligned.
struct u64x4 {
    uint64_t a, b, c, d;
};
__device__ __forceinline__ u64x4 ld256(const uint64_t *p) {
    u64x4 v;
    asm("ld.global.v4.u64 {%0, %1, %2, %3}, [%4];" : "=l"(v.a), "=l"(v.b), "=l"(v.c), "=l"(v.d) : "l"(p));
    return v;
}
__device__ __forceinline__ void st256(uint64_t *p, uint64_t a, uint64_t b, uint64_t c, uint64_t d) {
    asm volatile("st.global.v4.u64 [%0], {%1, %2, %3, %4};" ::"l"(p), "l"(a), "l"(b), "l"(c), "l"(d) : "memory");
}

// ---- epilogues of the last forward (row) pass ---------------------------------------------------
// The row pass leaves every thread with E consecutive canonical residues starting at limb offset o.
// An epilogue first preloads whatever else it needs for those positions (before the butterflies, so
// the loads are in flight while the ALUs work) and then finishes and stores them.
__host__ __device__ inline bool aligned32(const void *p) { return ((uintptr_t)p & 31) == 0; }

struct EpiStore {
    uint64_t *dst;
    bool aligned() const { return true; }  // dst is the transform's own output, checked by the launcher
    template <int E> struct Regs {};
    __device__ __forceinline__ void init(const NttArgs &a, const Job &job, size_t N) { dst = a.dst + dst_slot(a, job.x) * N; }
    template <int E> __device__ __forceinline__ void preload(Regs<E> &, size_t) const {}
    template <int E> __device__ __forceinline__ void finish(const Regs<E> &, size_t o, uint64_t (&x)[E], uint64_t) const {
#pragma unroll
        for (int i = 0; i < E; i += 4) st256(dst + o + i, x[i], x[i + 1], x[i + 2], x[i + 3]);
    }
};

// out[job.w] = (ACCUM ? out[job.w] : 0) + (minuend[job.z] - v) * k[prime]
// ModDown (src/rns_bconv.cu:820-821 with include/ntt_radix8_tmpl.cuh:203-233) followed by the
// add-to-ciphertext (:763-769) when ACCUM; rescale (src/rns.cu:1146-1158) without.
template <bool ACCUM>
struct EpiSubMul {
    const uint64_t *minuend;  // [slots][N]
    uint64_t *out;            // [slots][N]
    const W2 *k;              // per prime
    uint32_t m_bs = 0, o_bs = 0;  // batch strides in limbs (set b of a batched launch: see NttArgs)
    const uint64_t *m_ = nullptr;
    uint64_t *o_ = nullptr;
    W2 kk = W2{0, 0};
    bool aligned() const { return aligned32(minuend) && aligned32(out); }
    template <int E> struct Regs {
        u64x4 m[E / 4];
        u64x4 acc[ACCUM ? E / 4 : 1];
    };
    __device__ __forceinline__ void init(const NttArgs &a, const Job &job, size_t N) {
        m_ = minuend + ((size_t)job.z + (size_t)set_idx(a) * m_bs) * N;
        o_ = out + ((size_t)job.w + (size_t)set_idx(a) * o_bs) * N;
        kk = k[job.y];
    }
    template <int E> __device__ __forceinline__ void preload(Regs<E> &r, size_t o) const {
#pragma unroll
        for (int i = 0; i < E / 4; i++) {
            r.m[i] = ld256(m_ + o + 4 * i);
            if (ACCUM) r.acc[i] = ld256(o_ + o + 4 * i);
        }
    }
    template <int E> __device__ __forceinline__ void finish(const Regs<E> &r, size_t o, uint64_t (&x)[E], uint64_t q) const {
#pragma unroll
        for (int i = 0; i < E / 4; i++) {
            uint64_t r0 = mul_shoup(sub_mod(r.m[i].a, x[4 * i], q), kk, q);
            uint64_t r1 = mul_shoup(sub_mod(r.m[i].b, x[4 * i + 1], q), kk, q);
            uint64_t r2 = mul_shoup(sub_mod(r.m[i].c, x[4 * i + 2], q), kk, q);
            uint64_t r3 = mul_shoup(sub_mod(r.m[i].d, x[4 * i + 3], q), kk, q);
            if (ACCUM) {
                r0 = add_mod(r.acc[i].a, r0, q);
                r1 = add_mod(r.acc[i].b, r1, q);
                r2 = add_mod(r.acc[i].c, r2, q);
                r3 = add_mod(r.acc[i].d, r3, q);
            }
            st256(o_ + o + 4 * i, r0, r1, r2, r3);
        }
    }
};

// out[job.w] -= v  (the fused key switch: the inner-product kernel has already left
// ct + cx * P^-1 in `out`, and the ModDown matrix carries P^-1, so only the subtraction remains)
struct EpiSubFrom {
    uint64_t *out;
    uint32_t bs = 0;  // batch stride of `out` in limbs (set b of a batched launch: see NttArgs)
    uint64_t *o_ = nullptr;
    bool aligned() const { return aligned32(out); }
    template <int E> struct Regs {
        u64x4 u[E / 4];
    };
    __device__ __forceinline__ void init(const NttArgs &a, const Job &job, size_t N) { o_ = out + ((size_t)job.w + (size_t)set_idx(a) * bs) * N; }
    template <int E> __device__ __forceinline__ void preload(Regs<E> &r, size_t o) const {
#pragma unroll
        for (int i = 0; i < E / 4; i++) r.u[i] = ld256(o_ + o + 4 * i);
    }
    template <int E> __device__ __forceinline__ void finish(const Regs<E> &r, size_t o, uint64_t (&x)[E], uint64_t q) const {
#pragma unroll
        for (int i = 0; i < E / 4; i++)
            st256(o_ + o + 4 * i, sub_mod(r.u[i].a, x[4 * i], q), sub_mod(r.u[i].b, x[4 * i + 1], q), sub_mod(r.u[i].c, x[4 * i + 2], q),
                  sub_mod(r.u[i].d, x[4 * i + 3], q));
    }
};

template <int LOG_T, int RC>
__device__ __forceinline__ int pad_idx(int e) { return e + (e >> RC); }

// ================================================================================================
// arithmetic policies
// ================================================================================================
// On B200 a 32x32->64-bit integer multiply issues at a quarter of the rate of a double-precision
// FMA (measured: ~16 vs 64 lanes per clock per SM), and a 64-bit Shoup product needs six of them.
// Primes below 2^41 therefore run their butterflies in FP64: residues are held as doubles with
// exact integer values, a modular product is
//     h = y*w,  l = fma(y,w,-h)            (h + l = y*w exactly)
//     c = rint(y * (w/q))                  (quotient estimate, off by at most one)
//     r = fma(-c, q, h) + l                (exact: |h - c q| < 2^53), r = y*w (mod q), |r| < q
// and a butterfly costs 8 FP64 instructions and no integer multiply. Ranges: a forward stage grows
// a residue by < q (|x| < 17q after 16 stages); an inverse stage doubles the bound and every pass
// renormalises once, so products never see |y| >= 2^50. Results are converted back to canonical
// uint64 at the end, so outputs are bit-identical to the integer path.
// Larger primes use 64-bit Shoup/Harvey butterflies; below 2^46 without any conditional
// subtraction (forward: < 33q after 16 stages; inverse: < 2^17 q), above with one per butterfly.
constexpr uint64_t FP_LIMIT = 1ull << 41;
constexpr uint64_t WIDE_LIMIT = 1ull << 46;
constexpr double FP_MAGIC = 6755399441055744.0;  // 1.5 * 2^52: (v + M) - M = rint(v) for |v| < 2^51
constexpr double FP_2_52 = 4503599627370496.0;

template <bool WIDE>
struct ArithInt {
    using T = uint64_t;
    using Tw = W2;
    struct K {
        uint64_t q, q2, r1;
        int logN;
    };
    __device__ __forceinline__ static K make(const Mod &md, int logN) { return K{md.q, 2 * md.q, md.r1, logN}; }
    __device__ __forceinline__ static Tw ldtw(const W2 *tw, size_t idx, const K &) { return ldg_w2(tw + idx); }
    __device__ __forceinline__ static Tw ldfin(const W2 *p, const K &) { return ldg_w2(p); }
    __device__ __forceinline__ static T from_u64(uint64_t v, const K &) { return v; }
    __device__ __forceinline__ static T from_raw(uint64_t v) { return v; }
    __device__ __forceinline__ static uint64_t to_raw(T v) { return v; }
    __device__ __forceinline__ static void ct(T &a, T &b, W2 w, const K &k) {
        if (WIDE) {
            const uint64_t t = mul_shoup_lazy(b, w, k.q);
            b = a + k.q2 - t;
            a = a + t;
        } else {
            ct_bfly(a, b, w, k.q, k.q2);
        }
    }
    // g = number of stages of the whole inverse transform already done
    __device__ __forceinline__ static void gs(T &a, T &b, W2 w, const K &k, int g) {
        if (WIDE) {
            const uint64_t d = a - b + (k.q << (g + 1));
            a = a + b;
            b = mul_shoup_lazy(d, w, k.q);
        } else {
            gs_bfly(a, b, w, k.q, k.q2);
        }
    }
    __device__ __forceinline__ static void gs_last(T &a, T &b, W2 sx, W2 sy, const K &k) {
        const uint64_t s = a + b;
        const uint64_t d = a - b + (WIDE ? (k.q << k.logN) : k.q2);
        a = mul_shoup(s, sx, k.q);
        b = mul_shoup(d, sy, k.q);
    }
    __device__ __forceinline__ static T pass_end(T v, const K &) { return v; }  // nothing to renormalise
    __device__ __forceinline__ static uint64_t canon_fwd(T v, const K &k) {
        return WIDE ? barrett64(v, k.q, k.r1) : csub(csub(v, k.q2), k.q);
    }
    __device__ __forceinline__ static uint64_t canon_inv(T v, const K &) { return v; }  // gs_last is canonical
};

struct ArithFp {
    using T = double;
    struct Tw {
        double w, wq;  // w and w / q
    };
    struct K {
        double q, qinv;
        int logN;
    };
    // table entry i of an FP64 prime is one double (8 bytes); w / q is rebuilt as w * (1/q), whose
    // relative error of 2^-52 is far inside the slack of the quotient estimate
    __device__ __forceinline__ static Tw ldtw(const W2 *tw, size_t idx, const K &k) {
        const double w = __ldg(reinterpret_cast<const double *>(tw) + idx);
        return Tw{w, __dmul_rn(w, k.qinv)};
    }
    __device__ __forceinline__ static Tw ldfin(const W2 *p, const K &) {
        const W2 v = ldg_w2(p);
        return Tw{__longlong_as_double((long long)v.w), __longlong_as_double((long long)v.ws)};
    }
    __device__ __forceinline__ static K make(const Mod &md, int logN) {
        const double q = (double)md.q;
        return K{q, 1.0 / q, logN};
    }
    __device__ __forceinline__ static T from_u64(uint64_t v, const K &) {
        return __dsub_rn(__longlong_as_double((long long)(v | 0x4330000000000000ull)), FP_2_52);
    }
    __device__ __forceinline__ static T from_raw(uint64_t v) { return __longlong_as_double((long long)v); }
    __device__ __forceinline__ static uint64_t to_raw(T v) { return (uint64_t)__double_as_longlong(v); }
    __device__ __forceinline__ static T mulmod(T y, Tw w, const K &k) {
        const double wd = w.w, wq = w.wq;
        const double h = __dmul_rn(y, wd);
        const double l = __fma_rn(y, wd, -h);
        const double c = __dsub_rn(__fma_rn(y, wq, FP_MAGIC), FP_MAGIC);
        return __dadd_rn(__fma_rn(-c, k.q, h), l);
    }
    __device__ __forceinline__ static T reduce(T v, const K &k) {
        const double c = __dsub_rn(__fma_rn(v, k.qinv, FP_MAGIC), FP_MAGIC);
        return __fma_rn(-c, k.q, v);
    }
    __device__ __forceinline__ static void ct(T &a, T &b, Tw w, const K &k) {
        const double t = mulmod(b, w, k);
        b = __dsub_rn(a, t);
        a = __dadd_rn(a, t);
    }
    __device__ __forceinline__ static void gs(T &a, T &b, Tw w, const K &k, int) {
        const double d = __dsub_rn(a, b);
        a = __dadd_rn(a, b);
        b = mulmod(d, w, k);
    }
    __device__ __forceinline__ static void gs_last(T &a, T &b, Tw sx, Tw sy, const K &k) {
        const double s = __dadd_rn(a, b), d = __dsub_rn(a, b);
        a = mulmod(s, sx, k);
        b = mulmod(d, sy, k);
    }
    __device__ __forceinline__ static T pass_end(T v, const K &k) { return reduce(v, k); }
    __device__ __forceinline__ static uint64_t to_canon(T v, const K &k) {  // |v| < q
        if (v < 0.0) v = __dadd_rn(v, k.q);
        return (uint64_t)__double_as_longlong(__dadd_rn(v, FP_2_52)) & 0x000FFFFFFFFFFFFFull;
    }
    __device__ __forceinline__ static uint64_t canon_fwd(T v, const K &k) { return to_canon(reduce(v, k), k); }
    __device__ __forceinline__ static uint64_t canon_inv(T v, const K &k) { return to_canon(v, k); }
};

// ---- stage runners: compile-time recursion keeps every register index a constant --------------
// forward: E residues x[], local stages S..R-1 of this stage group; twiddle index
// (P << (shift + S)) + (k0 << S) + g.
template <class A, int S, int R, int E>
__device__ __forceinline__ void ct_stages(typename A::T (&x)[E], const W2 *tw, size_t P, int shift, size_t k0, const typename A::K &k) {
    if constexpr (S < R) {
        constexpr int half = E >> (S + 1);
#pragma unroll
        for (int g = 0; g < (1 << S); g++) {
            const typename A::Tw w = A::ldtw(tw, (P << (shift + S)) + (k0 << S) + g, k);
#pragma unroll
            for (int j = 0; j < half; j++) A::ct(x[g * 2 * half + j], x[g * 2 * half + j + half], w, k);
        }
        ct_stages<A, S + 1, R, E>(x, tw, P, shift, k0, k);
    }
}

// inverse: local stages U..R-1 (gap 2^U); twiddle index (m0 >> U) * P + (k0 >> U) + g with
// m0 = sub-transform size >> (1 + stages already done), k0 = first pair group of this thread at
// U = 0. g0 = stages of the whole transform already done.
template <class A, int U, int R, int E>
__device__ __forceinline__ void gs_stages(typename A::T (&x)[E], const W2 *tw, size_t P, int m0, size_t k0, int g0, const typename A::K &k) {
    if constexpr (U < R) {
        constexpr int gap = 1 << U;
#pragma unroll
        for (int g = 0; g < (E >> (U + 1)); g++) {
            const typename A::Tw w = A::ldtw(tw, (size_t)(m0 >> U) * P + (k0 >> U) + g, k);
#pragma unroll
            for (int j = 0; j < gap; j++) A::gs(x[g * 2 * gap + j], x[g * 2 * gap + j + gap], w, k, g0 + U);
        }
        gs_stages<A, U + 1, R, E>(x, tw, P, m0, k0, g0, k);
    }
}

// ================================================================================================
// forward pass: R1 strided stages, exchange, R2 contiguous stages
// FIRST: the input holds canonical residues (else the raw lazy values of the previous pass)
// ================================================================================================
// STAGED: the tile's input already sits in `sm` itself, dense ([e][c] for the column pass, [c][e] for the row
// pass), put there by asynchronous copies; it is read into registers, and after a barrier the same buffer
// serves as the exchange buffer.
// SRC (column pass only): 1 = the input word reduced into the limb's prime, 2 = its centred representative
// (word - src_q when the word exceeds src_q / 2) reduced: the remainder a rescale subtracts, floor or nearest.
template <class A, int LOG_T, int R1, int R2, int LOG_C, bool COLS, bool LAST, class Epi, bool STAGED = false, int SRC = 0>
__device__ __forceinline__ void fwd_body(const NttArgs &a, const Epi &epi, uint64_t *sm, const Job &job, const Mod &md, uint32_t tile) {
    using T = typename A::T;
    static_assert(SRC == 0 || (COLS && !STAGED), "the on-the-fly source belongs to the plain column pass");
    constexpr bool FIRST = COLS;
    constexpr int TT = 1 << LOG_T, E1 = 1 << R1, E2 = 1 << R2, C = 1 << LOG_C;
    constexpr int EPT = E1 > E2 ? E1 : E2;
    constexpr int THREADS = C * TT / EPT;
    constexpr int TPAD = TT + (TT >> R2);
    const size_t N = (size_t)1 << a.logN;
    const typename A::K k = A::make(md, (int)a.logN);
    const W2 *tw = a.tw + (size_t)job.y * N;
    const uint64_t *src = a.src + src_slot(a, SRC ? job.x / a.src_div : job.x) * N;
    const size_t estride = COLS ? (N >> LOG_T) : 1;
    const size_t cstride = COLS ? 1 : TT;
    const size_t base = COLS ? (size_t)tile * C : (size_t)tile * C * TT;
    const uint32_t n1 = (uint32_t)(N >> LOG_T);  // number of sub-transforms per limb
    const int tid = threadIdx.x;
    const uint64_t src_half = SRC == 2 ? a.src_q >> 1 : 0, src_q_red = SRC == 2 ? barrett64(a.src_q, md.q, md.r1) : 0;

    // ---- stage group 1 ---------------------------------------------------------------------------
#pragma unroll
    for (int gi = 0; gi < EPT / E1; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / E2);
        const int elo = COLS ? (gid / C) : (gid % E2);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        T x[E1];
        const uint64_t *p = src + base + (size_t)c * cstride + (size_t)elo * estride;
#pragma unroll
        for (int i = 0; i < E1; i++) {
            const int e = elo + i * E2;
            uint64_t v = STAGED ? sm[COLS ? (e * C + c) : (c * TT + e)] : p[(size_t)i * E2 * estride];
            if (SRC) {
                const uint64_t word = v;
                v = barrett64(word, md.q, md.r1);
                if (SRC == 2 && word > src_half) v = sub_mod(v, src_q_red, md.q);
            }
            x[i] = FIRST ? A::from_u64(v, k) : A::from_raw(v);
        }
        if (STAGED) {
            static_assert(!STAGED || E1 == EPT, "staged input wants one register group per thread");
            __syncthreads();  // every staged value is in registers: the buffer may now take the exchange
        }
        ct_stages<A, 0, R1, E1>(x, tw, P, 0, 0, k);
#pragma unroll
        for (int i = 0; i < E1; i++) {
            const int pe = pad_idx<LOG_T, R2>(elo + i * E2);
            sm[COLS ? (pe * C + c) : (c * TPAD + pe)] = A::to_raw(x[i]);
        }
    }
    __syncthreads();
    // ---- stage group 2 ---------------------------------------------------------------------------
    Epi e = epi;
    if (LAST) e.init(a, job, N);
    uint64_t *dst = a.dst + dst_slot(a, job.x) * N;
#pragma unroll
    for (int gi = 0; gi < EPT / E2; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / E1);
        const int ehi = COLS ? (gid / C) : (gid % E1);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        const size_t o = base + (size_t)c * cstride + (size_t)ehi * E2 * estride;
        typename Epi::template Regs<E2> regs;
        if (LAST) e.template preload<E2>(regs, o);
        T x[E2];
#pragma unroll
        for (int i = 0; i < E2; i++) {
            const int pe = pad_idx<LOG_T, R2>(ehi * E2 + i);
            x[i] = A::from_raw(sm[COLS ? (pe * C + c) : (c * TPAD + pe)]);
        }
        ct_stages<A, 0, R2, E2>(x, tw, P, R1, ehi, k);
        if (LAST) {
            static_assert(!LAST || !COLS, "the last forward pass is the row pass");
            uint64_t y[E2];
#pragma unroll
            for (int i = 0; i < E2; i++) y[i] = A::canon_fwd(x[i], k);
            e.template finish<E2>(regs, o, y, md.q);
        } else {
#pragma unroll
            for (int i = 0; i < E2; i++) dst[o + (size_t)i * estride] = A::to_raw(x[i]);
        }
    }
}

template <int LOG_T, int R1, int R2, int LOG_C, bool COLS, bool LAST, class Epi, int SRC = 0>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) / (1 << (R1 > R2 ? R1 : R2)), ntt_min_blocks((1 << (LOG_C + LOG_T)) / (1 << (R1 > R2 ? R1 : R2)), 1 << (R1 > R2 ? R1 : R2)))
ntt_fwd_pass(NttArgs a, Epi epi) {
    static_assert(R1 + R2 == LOG_T, "stage split");
    constexpr int TT = 1 << LOG_T, C = 1 << LOG_C;
    __shared__ uint64_t sm[C * (TT + (TT >> R2))];
    const uint32_t tiles = (uint32_t)(((size_t)1 << a.logN) >> (LOG_T + LOG_C));
    const uint32_t jobi = work_idx(a) / tiles, tile = work_idx(a) % tiles;
    const Job job = get_job(a, jobi);
    const Mod md = a.mod[job.y];
    if (md.q < FP_LIMIT) fwd_body<ArithFp, LOG_T, R1, R2, LOG_C, COLS, LAST, Epi, false, SRC>(a, epi, sm, job, md, tile);
    else if (md.q < WIDE_LIMIT) fwd_body<ArithInt<true>, LOG_T, R1, R2, LOG_C, COLS, LAST, Epi, false, SRC>(a, epi, sm, job, md, tile);
    else fwd_body<ArithInt<false>, LOG_T, R1, R2, LOG_C, COLS, LAST, Epi, false, SRC>(a, epi, sm, job, md, tile);
}

// ================================================================================================
// Last forward (row) pass of ModUp fused with the key-switch inner product, for the limbs on FP64 primes.
// A CTA owns one tile of one output limb t and walks the digits: the digit that holds limb t itself contributes the
// NTT-form input as it is, every other digit's limb t is finished here (row pass of its column-pass output) and never
// stored. Both polynomials of the key are multiplied in and accumulated in FP64 (|sum| < beta q), reduced once, and
// ct[k][t] += sum_k * P^-1 as the stand-alone inner-product kernel does. Same residues as that kernel.
// ================================================================================================
#define B2_MAC_MAX_BETA 8
struct MacArgs {
    const uint64_t *own;                   // NTT-form input of ModUp, [l][N]
    const uint64_t *evk[B2_MAC_MAX_BETA];  // digit d: [2][size_QP][N]
    uint64_t *ct;                          // [2][l][N]
    uint64_t *cxp;                         // [2][alpha][N]: the P limbs of the inner product
    const W2 *pinv;                        // per prime: P^-1 {w, shoup}
    const W2 *fin;                         // per prime, for the integer path: P^-1 * 2^64 mod q (Q), 2^64 mod p (P)
    uint32_t l, lP, alpha, beta, size_Q, size_QP, acc_p;
    uint32_t interleave;                   // consecutive CTAs walk the limbs of one tile (else the tiles of one limb)
    // a batched launch (one key for every set): set b = blockIdx.x, so that the CTAs which read the same key tile run next
    // to one another and all but the first find it in L2; its digits, NTT-form input, ciphertext and P limbs start
    // b * dig_bs / own_bs / ct_bs / cxp_bs limbs further
    uint32_t dig_bs, own_bs, ct_bs, cxp_bs;  // (with the sets as the slow dimension instead the pass took 30.7 instead of 27.8 us per key switch)
    uint32_t p_first, first_limb;          // the grid covers p_first P limbs, then the Q limbs from first_limb on
    uint32_t p_off;                        // index of the first of those P limbs (a rank's slice under limb sharding; else 0)
    // P limb i of polynomial k of set b lands at limb slot i * cxp_i + k * cxp_k + b * cxp_bs of cxp: [set][2][alpha] is
    // (1, alpha, 2 alpha), the limb-major exchange buffer [alpha][2][sets] is (2 sets, sets, 1)
    uint32_t cxp_i, cxp_k;
};

__device__ __forceinline__ u64x4 ld256_cs(const uint64_t *p) {  // streaming: the key is read once
    u64x4 v;
    asm("ld.global.cs.v4.u64 {%0, %1, %2, %3}, [%4];" : "=l"(v.a), "=l"(v.b), "=l"(v.c), "=l"(v.d) : "l"(p));
    return v;
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int KEEP>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(KEEP) : "memory");
}

// bytes of dynamic shared memory the kernel wants: the exchange buffer and one digit's two key polynomials for the tile
template <int LOG_T, int R, int LOG_C>
constexpr size_t mac_smem_bytes() {
    return (size_t)((1 << LOG_C) * ((1 << LOG_T) + ((1 << LOG_T) >> R)) + 2 * (1 << (LOG_C + LOG_T))) * 8;
}

// How the fused pass multiplies a finished digit residue into a key word and sums over the digits, per arithmetic.
// FP64 primes: the signed products (below q in magnitude) are summed as doubles and reduced once.
// Integer primes: a Montgomery product y * key * 2^-64 (four 64-bit multiplies, no correction step: the key word is
// below q, so any 64-bit y gives a value below 2q) summed in one 64-bit word - 128-bit accumulators for sixteen residues
// times two polynomials would not fit the register file, and a Barrett reduction per product costs twice the multiplies.
// The factor 2^-64 is undone by the constant of the final multiplication (MacArgs::fin).
template <class A> struct MacAcc;
template <> struct MacAcc<ArithFp> {
    using T = double;
    using K = ArithFp::K;
    struct C {};
    __device__ __forceinline__ static C make(const Mod &) { return C{}; }
    __device__ __forceinline__ static T zero() { return 0.0; }
    __device__ __forceinline__ static double operand(double y, const K &k) { return ArithFp::reduce(y, k); }
    __device__ __forceinline__ static void mac(T &acc, double y, uint64_t key, const K &k, const C &) {
        const double w = ArithFp::from_u64(key, k);
        acc = __dadd_rn(acc, ArithFp::mulmod(y, ArithFp::Tw{w, __dmul_rn(w, k.qinv)}, k));
    }
    // canonical residue of the sum
    __device__ __forceinline__ static uint64_t finish(T acc, W2, const K &k, const C &) { return ArithFp::canon_fwd(acc, k); }
};
template <bool WIDE> struct MacAcc<ArithInt<WIDE>> {
    using T = uint64_t;
    using K = typename ArithInt<WIDE>::K;
    struct C {
        uint64_t q, q2, ninv;  // ninv = -q^-1 mod 2^64
        bool tight;            // 2 * beta * q could pass 2^64: keep the sum below 2q after every term
    };
    __device__ __forceinline__ static C make(const Mod &md) {
        uint64_t x = md.q;  // q * q = 1 mod 8; every Newton step doubles the valid bits
#pragma unroll
        for (int i = 0; i < 5; i++) x *= 2 - md.q * x;
        return C{md.q, 2 * md.q, 0 - x, (md.q >> 59) != 0};
    }
    __device__ __forceinline__ static T zero() { return 0; }
    __device__ __forceinline__ static uint64_t operand(uint64_t y, const K &) { return y; }  // lazy values (below 2^63) do
    __device__ __forceinline__ static void mac(T &acc, uint64_t y, uint64_t key, const K &, const C &c) {
        const uint64_t lo = y * key, hi = __umul64hi(y, key);
        const uint64_t m = lo * c.ninv;
        // (y key + m q) / 2^64: the low words cancel, carrying one unless lo is zero
        acc += hi + __umul64hi(m, c.q) + (lo != 0);
        if (c.tight) acc = csub(acc, c.q2);
    }
    // sum * 2^-64 times the limb's closing constant, canonical
    __device__ __forceinline__ static uint64_t finish(T acc, W2 fin, const K &, const C &c) { return mul_shoup(acc, fin, c.q); }
};

// One tile of one output limb t (logical index: Q limbs 0 .. l-1, then the P limbs) through all digits.
template <class A, int LOG_T, int R, int LOG_C>
__device__ __forceinline__ void mac_body(const NttArgs &a, const MacArgs &m, uint64_t *sm, uint64_t *kb, uint32_t t, uint32_t pp, uint32_t tile,
                                         uint32_t bset, const Mod &md) {
    using T = typename A::T;
    using Acc = MacAcc<A>;
    constexpr int TT = 1 << LOG_T, E = 1 << R, C = 1 << LOG_C;
    constexpr int TPAD = TT + (TT >> R), THREADS = (C * TT) >> R;
    static_assert(E == 16, "the key staging below gives every thread eight 16-byte chunks per polynomial");
    const size_t N = (size_t)1 << a.logN;
    const typename A::K k = A::make(md, (int)a.logN);
    const W2 *tw = a.tw + (size_t)pp * N;
    const uint32_t n1 = (uint32_t)(N >> LOG_T);
    const int tid = threadIdx.x;
    const int c = tid / E, e = tid % E;  // sub-transform of the tile, register group within it (both stage groups)
    const uint32_t P = n1 + tile * C + c;
    const size_t base = (size_t)tile * C * TT;
    const size_t o = base + (size_t)c * TT + (size_t)e * E;  // this thread's E consecutive outputs: tid * 16 into the tile
    const uint32_t own_d = t < m.l ? t / m.alpha : 0xFFFFFFFFu;  // a P limb belongs to no digit
    const typename Acc::C mc = Acc::make(md);
    typename Acc::T acc0[E], acc1[E];
#pragma unroll
    for (int i = 0; i < E; i++) acc0[i] = acc1[i] = Acc::zero();
    for (uint32_t d = 0; d < m.beta; d++) {
        // The digit's key tile starts its way from HBM now (cp.async, L1 bypassed: the key is read once) and is waited for
        // only after this digit's butterflies: a thread's eight 16-byte chunks of a polynomial are XOR-swizzled inside its
        // 128-byte row so that the 128-bit reads below are free of bank conflicts.
        {
            const uint64_t *g0 = m.evk[d] + (size_t)pp * N + base, *g1 = g0 + (size_t)m.size_QP * N;
#pragma unroll
            for (int g = tid; g < C * TT / 2; g += THREADS) {
                const int owner = g >> 3, chunk = g & 7, off = owner * 16 + ((chunk ^ (owner & 7)) << 1);
                cp_async16(kb + off, g0 + 2 * g);
                cp_async16(kb + C * TT + off, g1 + 2 * g);
            }
            cp_async_commit();
        }
        T y[E];
        if (d == own_d) {
#pragma unroll
            for (int i = 0; i < E; i += 4) {
                const u64x4 v = ld256(m.own + ((size_t)bset * m.own_bs + t) * N + o + i);
                y[i] = A::from_u64(v.a, k), y[i + 1] = A::from_u64(v.b, k), y[i + 2] = A::from_u64(v.c, k), y[i + 3] = A::from_u64(v.d, k);
            }
        } else {
            const uint64_t *src = a.src + ((size_t)bset * m.dig_bs + (size_t)d * m.lP + t) * N + base + (size_t)c * TT + e;
#pragma unroll
            for (int i = 0; i < E; i++) y[i] = A::from_raw(src[i * E]);
            ct_stages<A, 0, R, E>(y, tw, P, 0, 0, k);
#pragma unroll
            for (int i = 0; i < E; i++) sm[c * TPAD + pad_idx<LOG_T, R>(e + i * E)] = A::to_raw(y[i]);
            __syncthreads();
#pragma unroll
            for (int i = 0; i < E; i++) y[i] = A::from_raw(sm[c * TPAD + pad_idx<LOG_T, R>(e * E + i)]);
            ct_stages<A, 0, R, E>(y, tw, P, R, e, k);
#pragma unroll
            for (int i = 0; i < E; i++) y[i] = Acc::operand(y[i], k);
        }
        cp_async_wait<0>();
        __syncthreads();  // every thread's share of the key tile has landed
#pragma unroll
        for (int i = 0; i < E; i += 2) {
            const int off = tid * 16 + (((i >> 1) ^ (tid & 7)) << 1);
            const ulonglong2 u = *reinterpret_cast<const ulonglong2 *>(kb + off), v = *reinterpret_cast<const ulonglong2 *>(kb + C * TT + off);
            Acc::mac(acc0[i], y[i], u.x, k, mc);
            Acc::mac(acc0[i + 1], y[i + 1], u.y, k, mc);
            Acc::mac(acc1[i], y[i], v.x, k, mc);
            Acc::mac(acc1[i + 1], y[i + 1], v.y, k, mc);
        }
        __syncthreads();  // the key tile and the exchange buffer are free for the next digit
    }
    const uint64_t q = md.q;
    if (t < m.l) {
        // a Q limb: ct[k][t] += sum * P^-1. FP64 sums are canonical first and take P^-1; integer sums carry 2^-64 and
        // take P^-1 * 2^64 in the same single multiplication.
        constexpr bool FP = std::is_same<A, ArithFp>::value;
        const W2 pi = FP ? m.pinv[pp] : m.fin[pp];
        uint64_t *c0 = m.ct + ((size_t)bset * m.ct_bs + t) * N + o, *c1 = c0 + (size_t)m.l * N;
#pragma unroll
        for (int i = 0; i < E; i += 4) {
            const u64x4 u = ld256(c0 + i), v = ld256(c1 + i);
            uint64_t r[4], s[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                r[j] = Acc::finish(acc0[i + j], pi, k, mc);
                s[j] = Acc::finish(acc1[i + j], pi, k, mc);
                if (FP) r[j] = mul_shoup(r[j], pi, q), s[j] = mul_shoup(s[j], pi, q);
            }
            st256(c0 + i, add_mod(u.a, r[0], q), add_mod(u.b, r[1], q), add_mod(u.c, r[2], q), add_mod(u.d, r[3], q));
            st256(c1 + i, add_mod(v.a, s[0], q), add_mod(v.b, s[1], q), add_mod(v.c, s[2], q), add_mod(v.d, s[3], q));
        }
    } else {
        // a P limb: kept (or, acc_p, added to what is there) in the compact buffer [2][alpha][N] for the ModDown that
        // follows; the closing constant of an integer prime is 2^64 mod p
        const W2 fin = m.fin[pp];
        uint64_t *p0 = m.cxp + ((size_t)bset * m.cxp_bs + (size_t)(t - m.l) * m.cxp_i) * N + o, *p1 = p0 + (size_t)m.cxp_k * N;
#pragma unroll
        for (int i = 0; i < E; i += 4) {
            uint64_t r[4], s[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                r[j] = Acc::finish(acc0[i + j], fin, k, mc);
                s[j] = Acc::finish(acc1[i + j], fin, k, mc);
            }
            if (m.acc_p) {
                const u64x4 u = ld256(p0 + i), v = ld256(p1 + i);
                r[0] = add_mod(r[0], u.a, q), r[1] = add_mod(r[1], u.b, q), r[2] = add_mod(r[2], u.c, q), r[3] = add_mod(r[3], u.d, q);
                s[0] = add_mod(s[0], v.a, q), s[1] = add_mod(s[1], v.b, q), s[2] = add_mod(s[2], v.c, q), s[3] = add_mod(s[3], v.d, q);
            }
            st256(p0 + i, r[0], r[1], r[2], r[3]);
            st256(p1 + i, s[0], s[1], s[2], s[3]);
        }
    }
}

template <int LOG_T, int R, int LOG_C>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) >> R, 3) ntt_fwd_rows_mac(NttArgs a, const __grid_constant__ MacArgs m) {
    static_assert(2 * R == LOG_T, "equal stage groups: one register group per thread in both");
    constexpr int TT = 1 << LOG_T, C = 1 << LOG_C;
    constexpr int TPAD = TT + (TT >> R);
    extern __shared__ __align__(16) uint64_t mac_smem[];
    uint64_t *sm = mac_smem;             // [C][TPAD] exchange buffer of the row pass
    uint64_t *kb = mac_smem + C * TPAD;  // [2][C * TT] the tile of both key polynomials of the digit in hand
    const uint32_t tiles = (uint32_t)(((size_t)1 << a.logN) >> (LOG_T + LOG_C));
    // the P limbs (60-bit primes: the long CTAs) go first so that they do not form the tail of the grid
    const uint32_t n_limbs = gridDim.y / tiles, bset = blockIdx.x;
    const uint32_t i = m.interleave ? blockIdx.y % n_limbs : blockIdx.y / tiles, tile = m.interleave ? blockIdx.y / n_limbs : blockIdx.y % tiles;
    const uint32_t t = i < m.p_first ? m.l + m.p_off + i : m.first_limb + (i - m.p_first);
    const uint32_t pp = t < m.l ? t : m.size_Q + (t - m.l);  // the limb's prime
    const Mod md = a.mod[pp];
    if (md.q < FP_LIMIT) mac_body<ArithFp, LOG_T, R, LOG_C>(a, m, sm, kb, t, pp, tile, bset, md);
    else if (md.q < WIDE_LIMIT) mac_body<ArithInt<true>, LOG_T, R, LOG_C>(a, m, sm, kb, t, pp, tile, bset, md);
    else mac_body<ArithInt<false>, LOG_T, R, LOG_C>(a, m, sm, kb, t, pp, tile, bset, md);
}

// ================================================================================================
// inverse pass: RA contiguous stages, exchange, RB strided stages
// ================================================================================================
template <class A, int LOG_T, int RA, int RB, int LOG_C, bool COLS, bool LAST, bool STAGED = false>
__device__ __forceinline__ void inv_body(const NttArgs &a, uint64_t *sm, const Job &job, const Mod &md, uint32_t tile) {
    using T = typename A::T;
    constexpr bool FIRST = !COLS;
    constexpr int TT = 1 << LOG_T, EA = 1 << RA, EB = 1 << RB, C = 1 << LOG_C;
    constexpr int EPT = EA > EB ? EA : EB;
    constexpr int THREADS = C * TT / EPT;
    constexpr int TPAD = TT + (TT >> RA);
    const size_t N = (size_t)1 << a.logN;
    const typename A::K k = A::make(md, (int)a.logN);
    const W2 *tw = a.tw + (size_t)job.y * N;
    const uint64_t *src = a.src + src_slot(a, FIRST ? job.x : job.w) * N;  // the second pass works in place on dst
    uint64_t *dst = a.dst + dst_slot(a, job.w) * N;
    const size_t estride = COLS ? (N >> LOG_T) : 1;
    const size_t cstride = COLS ? 1 : TT;
    const size_t base = COLS ? (size_t)tile * C : (size_t)tile * C * TT;
    const uint32_t n1 = (uint32_t)(N >> LOG_T);
    const int tid = threadIdx.x;
    // stages of the whole transform done before this pass: the row pass comes first
    const int g_pass = COLS ? ((int)a.logN - LOG_T) : 0;

    // ---- stage group 1: contiguous runs of EA residues ----------------------------------------------
#pragma unroll
    for (int gi = 0; gi < EPT / EA; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / EB);
        const int ehi = COLS ? (gid / C) : (gid % EB);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        T x[EA];
        const uint64_t *p = src + base + (size_t)c * cstride + (size_t)ehi * EA * estride;
        if (STAGED) {
            static_assert(!STAGED || EA == EPT, "staged input wants one register group per thread");
#pragma unroll
            for (int i = 0; i < EA; i++) {
                const int e = ehi * EA + i;
                const uint64_t v = sm[COLS ? (e * C + c) : (c * TT + e)];
                x[i] = FIRST ? A::from_u64(v, k) : A::from_raw(v);
            }
            __syncthreads();
        } else if (COLS) {
#pragma unroll
            for (int i = 0; i < EA; i++) {
                const uint64_t v = p[(size_t)i * estride];
                x[i] = FIRST ? A::from_u64(v, k) : A::from_raw(v);
            }
        } else {
#pragma unroll
            for (int i = 0; i < EA; i += 4) {
                const u64x4 v = ld256(p + i);
                x[i] = FIRST ? A::from_u64(v.a, k) : A::from_raw(v.a);
                x[i + 1] = FIRST ? A::from_u64(v.b, k) : A::from_raw(v.b);
                x[i + 2] = FIRST ? A::from_u64(v.c, k) : A::from_raw(v.c);
                x[i + 3] = FIRST ? A::from_u64(v.d, k) : A::from_raw(v.d);
            }
        }
        gs_stages<A, 0, RA, EA>(x, tw, P, TT >> 1, (size_t)ehi * (EA >> 1), g_pass, k);
#pragma unroll
        for (int i = 0; i < EA; i++) {
            const int pe = pad_idx<LOG_T, RA>(ehi * EA + i);
            sm[COLS ? (pe * C + c) : (c * TPAD + pe)] = A::to_raw(x[i]);
        }
    }
    __syncthreads();
    // ---- stage group 2: stride EA ---------------------------------------------------------------------
#pragma unroll
    for (int gi = 0; gi < EPT / EB; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / EA);
        const int elo = COLS ? (gid / C) : (gid % EA);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        T x[EB];
#pragma unroll
        for (int i = 0; i < EB; i++) {
            const int pe = pad_idx<LOG_T, RA>(elo + i * EA);
            x[i] = A::from_raw(sm[COLS ? (pe * C + c) : (c * TPAD + pe)]);
        }
        gs_stages<A, 0, (LAST ? RB - 1 : RB), EB>(x, tw, P, TT >> (RA + 1), 0, g_pass + RA, k);
        uint64_t *o = dst + base + (size_t)c * cstride + (size_t)elo * estride;
        if (LAST) {
            // last stage of the whole transform (twiddle index 1): the x outputs take the scale,
            // the y outputs a twiddle that already carries it (src/host/ntt.cu:53-55,
            // include/ntt_radix8_tmpl.cuh:566-568); callers fold further per-limb factors in.
            constexpr int gap = EB / 2;
            const typename A::Tw sx = A::ldfin(a.fin + 2 * (size_t)job.z, k);
            const typename A::Tw sy = A::ldfin(a.fin + 2 * (size_t)job.z + 1, k);
#pragma unroll
            for (int j = 0; j < gap; j++) A::gs_last(x[j], x[j + gap], sx, sy, k);
#pragma unroll
            for (int i = 0; i < EB; i++) o[(size_t)i * EA * estride] = A::canon_inv(x[i], k);
        } else {
#pragma unroll
            for (int i = 0; i < EB; i++) o[(size_t)i * EA * estride] = A::to_raw(A::pass_end(x[i], k));
        }
    }
}

template <int LOG_T, int RA, int RB, int LOG_C, bool COLS, bool LAST>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) / (1 << (RA > RB ? RA : RB)), ntt_min_blocks((1 << (LOG_C + LOG_T)) / (1 << (RA > RB ? RA : RB)), 1 << (RA > RB ? RA : RB)))
ntt_inv_pass(NttArgs a) {
    static_assert(RA + RB == LOG_T, "stage split");
    constexpr int TT = 1 << LOG_T, C = 1 << LOG_C;
    __shared__ uint64_t sm[C * (TT + (TT >> RA))];
    const uint32_t tiles = (uint32_t)(((size_t)1 << a.logN) >> (LOG_T + LOG_C));
    const uint32_t jobi = work_idx(a) / tiles, tile = work_idx(a) % tiles;
    const Job job = get_job(a, jobi);
    const Mod md = a.mod[job.y];
    if (md.q < FP_LIMIT) inv_body<ArithFp, LOG_T, RA, RB, LOG_C, COLS, LAST>(a, sm, job, md, tile);
    else if (md.q < WIDE_LIMIT) inv_body<ArithInt<true>, LOG_T, RA, RB, LOG_C, COLS, LAST>(a, sm, job, md, tile);
    else inv_body<ArithInt<false>, LOG_T, RA, RB, LOG_C, COLS, LAST>(a, sm, job, md, tile);
}

// ================================================================================================
// pipelined passes: a resident CTA walks over several tiles, and while it transforms one tile the next one
// is already on its way from global memory into the second shared-memory buffer (cp.async, 16 bytes per
// copy, L1 bypassed). The plain kernels above have bytes in flight only during the load phase of each CTA,
// which bounds them near 2.5 TB/s; here every resident CTA always has a whole tile in flight.
// ================================================================================================
// tile `tile` of limb slot `slot` of src -> dense buffer ([e][c] or [c][e])
template <int LOG_T, int LOG_C, bool COLS, int THREADS>
__device__ __forceinline__ void stage_tile(uint64_t *buf, const uint64_t *src, size_t N, uint32_t slot, uint32_t tile) {
    constexpr int TT = 1 << LOG_T, C = 1 << LOG_C;
    constexpr int GRAN = C * TT / 2;  // 16-byte granules per tile
    const uint64_t *s = src + (size_t)slot * N + (COLS ? (size_t)tile * C : (size_t)tile * C * TT);
#pragma unroll
    for (int g = threadIdx.x; g < GRAN; g += THREADS) {
        if (COLS) {
            const int row = g / (C / 2), part = g % (C / 2);
            cp_async16(buf + row * C + part * 2, s + (size_t)row * (N >> LOG_T) + part * 2);
        } else {
            cp_async16(buf + g * 2, s + (size_t)g * 2);
        }
    }
}

template <int LOG_T, int R1, int R2, int LOG_C, bool COLS, bool LAST, class Epi>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) / (1 << (R1 > R2 ? R1 : R2)), ntt_min_blocks((1 << (LOG_C + LOG_T)) / (1 << (R1 > R2 ? R1 : R2))))
ntt_fwd_pipe(NttArgs a, Epi epi, uint32_t total) {
    static_assert(R1 == R2, "pipelined passes are built for equal stage groups");
    constexpr int TT = 1 << LOG_T, C = 1 << LOG_C, THREADS = (C * TT) >> R1;
    __shared__ __align__(16) uint64_t buf[2][C * (TT + (TT >> R2))];
    const size_t N = (size_t)1 << a.logN;
    const uint32_t tiles = (uint32_t)(N >> (LOG_T + LOG_C));
    uint32_t item = blockIdx.x;
    if (item < total) stage_tile<LOG_T, LOG_C, COLS, THREADS>(buf[0], a.src, N, get_job(a, item / tiles).x, item % tiles);
    cp_async_commit();
    for (uint32_t it = 0; item < total; it++, item += gridDim.x) {
        const uint32_t nxt = item + gridDim.x;
        if (nxt < total) stage_tile<LOG_T, LOG_C, COLS, THREADS>(buf[(it + 1) & 1], a.src, N, get_job(a, nxt / tiles).x, nxt % tiles);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        uint64_t *sm = buf[it & 1];
        const Job job = get_job(a, item / tiles);
        const Mod md = a.mod[job.y];
        const uint32_t tile = item % tiles;
        if (md.q < FP_LIMIT) fwd_body<ArithFp, LOG_T, R1, R2, LOG_C, COLS, LAST, Epi, true>(a, epi, sm, job, md, tile);
        else if (md.q < WIDE_LIMIT) fwd_body<ArithInt<true>, LOG_T, R1, R2, LOG_C, COLS, LAST, Epi, true>(a, epi, sm, job, md, tile);
        else fwd_body<ArithInt<false>, LOG_T, R1, R2, LOG_C, COLS, LAST, Epi, true>(a, epi, sm, job, md, tile);
        __syncthreads();  // the buffer is refilled two iterations from now, by the prefetch of the next one
    }
    cp_async_wait<0>();
}

template <int LOG_T, int RA, int RB, int LOG_C, bool COLS, bool LAST>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) / (1 << (RA > RB ? RA : RB)), ntt_min_blocks((1 << (LOG_C + LOG_T)) / (1 << (RA > RB ? RA : RB))))
ntt_inv_pipe(NttArgs a, uint32_t total) {
    static_assert(RA == RB, "pipelined passes are built for equal stage groups");
    constexpr int TT = 1 << LOG_T, C = 1 << LOG_C, THREADS = (C * TT) >> RA;
    constexpr bool FIRST = !COLS;
    __shared__ __align__(16) uint64_t buf[2][C * (TT + (TT >> RA))];
    const size_t N = (size_t)1 << a.logN;
    const uint32_t tiles = (uint32_t)(N >> (LOG_T + LOG_C));
    uint32_t item = blockIdx.x;
    if (item < total) {
        const Job j0 = get_job(a, item / tiles);
        stage_tile<LOG_T, LOG_C, COLS, THREADS>(buf[0], a.src, N, FIRST ? j0.x : j0.w, item % tiles);
    }
    cp_async_commit();
    for (uint32_t it = 0; item < total; it++, item += gridDim.x) {
        const uint32_t nxt = item + gridDim.x;
        if (nxt < total) {
            const Job jn = get_job(a, nxt / tiles);
            stage_tile<LOG_T, LOG_C, COLS, THREADS>(buf[(it + 1) & 1], a.src, N, FIRST ? jn.x : jn.w, nxt % tiles);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        uint64_t *sm = buf[it & 1];
        const Job job = get_job(a, item / tiles);
        const Mod md = a.mod[job.y];
        const uint32_t tile = item % tiles;
        if (md.q < FP_LIMIT) inv_body<ArithFp, LOG_T, RA, RB, LOG_C, COLS, LAST, true>(a, sm, job, md, tile);
        else if (md.q < WIDE_LIMIT) inv_body<ArithInt<true>, LOG_T, RA, RB, LOG_C, COLS, LAST, true>(a, sm, job, md, tile);
        else inv_body<ArithInt<false>, LOG_T, RA, RB, LOG_C, COLS, LAST, true>(a, sm, job, md, tile);
        __syncthreads();
    }
    cp_async_wait<0>();
}

}  // namespace b2

// ================================================================================================
// single-launch transforms for N = 2^16 on a thread-block cluster
// ================================================================================================
// A cluster of 8 CTAs owns one limb (256 x 256 residues, 512 KiB). The two passes exchange through
// distributed shared memory instead of global memory: every CTA keeps a 256 x 32 (forward: its
// column block after the column pass) or 32 x 256 (inverse: its row block after the row pass)
// slab of 64 KiB in shared memory, the cluster synchronises with the hardware cluster barrier, and
// the second pass gathers its inputs from the eight slabs. A limb therefore crosses global memory
// once in and once out. No flag or spin wait is involved: cluster.sync() is the only rendezvous
// and every thread of every CTA reaches it unconditionally.
#include <cooperative_groups.h>

namespace b2 {
namespace cg = cooperative_groups;

constexpr int CL_SIZE = 8;        // CTAs per cluster
constexpr int CL_THREADS = 256;   // two tile groups of 128 threads
constexpr int CL_SLAB = 256 * 32; // residues per slab
constexpr int CL_EX = 8 * (256 + 16);
constexpr size_t CL_SMEM = (size_t)(CL_SLAB + 2 * CL_EX) * 8;

// slab indexing with a rotation of the 8-column groups by (row >> 4): rows 16 apart fall into
// different bank groups, which is what the two access patterns below need
__device__ __forceinline__ int slab_fwd(int row, int col32) { return row * 32 + ((col32 + 8 * (row >> 4)) & 31); }
__device__ __forceinline__ int slab_inv(int row32, int col) { return row32 * 256 + (col ^ (8 * ((row32 >> 4) & 1))); }

template <class A, class Epi>
__device__ __forceinline__ void fwd_cluster_body(const NttArgs &a, const Epi &epi, uint64_t *smem, const Job &job, const Mod &md) {
    using T = typename A::T;
    constexpr int LOG_T = 8, R1 = 4, R2 = 4, E = 16, C = 8, TPAD = 256 + 16;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const size_t N = 65536;
    const typename A::K k = A::make(md, 16);
    const W2 *tw = a.tw + (size_t)job.y * N;
    const uint64_t *src = a.src + (size_t)job.x * N;
    uint64_t *slab = smem;
    const int tg = threadIdx.x >> 7, t = threadIdx.x & 127;
    uint64_t *ex = smem + CL_SLAB + tg * CL_EX;

    // ---- column pass on this CTA's 32 columns: 4 tiles of 8, two at a time -------------------
#pragma unroll 1
    for (int it = 0; it < 2; it++) {
        const int ti = it * 2 + tg;
        const int c = t % C, e_lo = t / C;
        T x[E];
        const uint64_t *p = src + (size_t)e_lo * 256 + rank * 32 + ti * 8 + c;
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = A::from_u64(p[(size_t)i * 16 * 256], k);
        ct_stages<A, 0, R1, E>(x, tw, 1, 0, 0, k);
#pragma unroll
        for (int i = 0; i < E; i++) ex[pad_idx<LOG_T, R2>(e_lo + i * 16) * C + c] = A::to_raw(x[i]);
        __syncthreads();
        const int e_hi = t / C;
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = A::from_raw(ex[pad_idx<LOG_T, R2>(e_hi * 16 + i) * C + c]);
        ct_stages<A, 0, R2, E>(x, tw, 1, R1, e_hi, k);
#pragma unroll
        for (int i = 0; i < E; i++) slab[slab_fwd(e_hi * 16 + i, ti * 8 + c)] = A::to_raw(x[i]);
        __syncthreads();
    }
    cluster.sync();
    // ---- row pass on this CTA's 32 rows, inputs gathered from the eight slabs -------------------
    Epi e = epi;
    e.init(a, job, N);
    (void)TPAD;
#pragma unroll 1
    for (int it = 0; it < 2; it++) {
        const int ti = it * 2 + tg;
        const int ch = t / 16, e_lo = t % 16;
        const int row = rank * 32 + ti * 8 + ch;
        const uint32_t P = 256u + (uint32_t)row;
        T x[E];
#pragma unroll
        for (int i = 0; i < E; i++) {
            const int col = e_lo + 16 * i;
            const uint64_t *peer = cluster.map_shared_rank(slab, col >> 5);
            x[i] = A::from_raw(peer[slab_fwd(row, col & 31)]);
        }
        ct_stages<A, 0, R1, E>(x, tw, P, 0, 0, k);
#pragma unroll
        for (int i = 0; i < E; i++) ex[ch * TPAD + pad_idx<LOG_T, R2>(e_lo + i * 16)] = A::to_raw(x[i]);
        __syncthreads();
        const int e_hi = t % 16;
        const size_t o = (size_t)row * 256 + (size_t)e_hi * 16;
        typename Epi::template Regs<E> regs;
        e.template preload<E>(regs, o);
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = A::from_raw(ex[ch * TPAD + pad_idx<LOG_T, R2>(e_hi * 16 + i)]);
        ct_stages<A, 0, R2, E>(x, tw, P, R1, e_hi, k);
        uint64_t y[E];
#pragma unroll
        for (int i = 0; i < E; i++) y[i] = A::canon_fwd(x[i], k);
        e.template finish<E>(regs, o, y, md.q);
        __syncthreads();
    }
    cluster.sync();  // nobody leaves while a peer may still read its slab
}

template <class Epi>
__global__ void __cluster_dims__(CL_SIZE, 1, 1) __launch_bounds__(CL_THREADS, 2) ntt_fwd_cluster(NttArgs a, Epi epi) {
    extern __shared__ __align__(16) uint64_t cl_smem[];
    const Job job = get_job(a, blockIdx.x / CL_SIZE);
    const Mod md = a.mod[job.y];
    if (md.q < FP_LIMIT) fwd_cluster_body<ArithFp, Epi>(a, epi, cl_smem, job, md);
    else if (md.q < WIDE_LIMIT) fwd_cluster_body<ArithInt<true>, Epi>(a, epi, cl_smem, job, md);
    else fwd_cluster_body<ArithInt<false>, Epi>(a, epi, cl_smem, job, md);
}

template <class A>
__device__ __forceinline__ void inv_cluster_body(const NttArgs &a, uint64_t *smem, const Job &job, const Mod &md) {
    using T = typename A::T;
    constexpr int LOG_T = 8, RA = 4, RB = 4, E = 16, C = 8, TPAD = 256 + 16;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const size_t N = 65536;
    const typename A::K k = A::make(md, 16);
    const W2 *tw = a.tw + (size_t)job.y * N;
    const uint64_t *src = a.src + (size_t)job.x * N;
    uint64_t *dst = a.dst + (size_t)job.w * N;
    uint64_t *slab = smem;
    const int tg = threadIdx.x >> 7, t = threadIdx.x & 127;
    uint64_t *ex = smem + CL_SLAB + tg * CL_EX;

    // ---- row pass on this CTA's 32 rows (bit-reversed input, contiguous) ------------------------
#pragma unroll 1
    for (int it = 0; it < 2; it++) {
        const int ti = it * 2 + tg;
        const int ch = t / 16, e_hi = t % 16;
        const int row32 = ti * 8 + ch;
        const uint32_t P = 256u + (uint32_t)(rank * 32 + row32);
        T x[E];
        const uint64_t *p = src + (size_t)(rank * 32 + row32) * 256 + (size_t)e_hi * 16;
#pragma unroll
        for (int i = 0; i < E; i += 2) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(p + i);
            x[i] = A::from_u64(v.x, k);
            x[i + 1] = A::from_u64(v.y, k);
        }
        gs_stages<A, 0, RA, E>(x, tw, P, 128, (size_t)e_hi * 8, 0, k);
#pragma unroll
        for (int i = 0; i < E; i++) ex[ch * TPAD + pad_idx<LOG_T, RA>(e_hi * 16 + i)] = A::to_raw(x[i]);
        __syncthreads();
        const int e_lo = t % 16;
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = A::from_raw(ex[ch * TPAD + pad_idx<LOG_T, RA>(e_lo + i * 16)]);
        gs_stages<A, 0, RB, E>(x, tw, P, 128 >> RA, 0, RA, k);
#pragma unroll
        for (int i = 0; i < E; i++) slab[slab_inv(row32, e_lo + 16 * i)] = A::to_raw(A::pass_end(x[i], k));
        __syncthreads();
    }
    cluster.sync();
    // ---- column pass on this CTA's 32 columns, inputs gathered from the eight slabs ----------------
#pragma unroll 1
    for (int it = 0; it < 2; it++) {
        const int ti = it * 2 + tg;
        const int c = t % C, e_hi = t / C;
        const int col = rank * 32 + ti * 8 + c;
        T x[E];
        {
            const uint64_t *peer = cluster.map_shared_rank(slab, e_hi >> 1);
#pragma unroll
            for (int i = 0; i < E; i++) x[i] = A::from_raw(peer[slab_inv((e_hi & 1) * 16 + i, col)]);
        }
        gs_stages<A, 0, RA, E>(x, tw, 1, 128, (size_t)e_hi * 8, 8, k);
#pragma unroll
        for (int i = 0; i < E; i++) ex[pad_idx<LOG_T, RA>(e_hi * 16 + i) * C + c] = A::to_raw(x[i]);
        __syncthreads();
        const int e_lo = t / C;
#pragma unroll
        for (int i = 0; i < E; i++) x[i] = A::from_raw(ex[pad_idx<LOG_T, RA>(e_lo + i * 16) * C + c]);
        gs_stages<A, 0, RB - 1, E>(x, tw, 1, 128 >> RA, 0, 8 + RA, k);
        const typename A::Tw sx = A::ldfin(a.fin + 2 * (size_t)job.z, k);
        const typename A::Tw sy = A::ldfin(a.fin + 2 * (size_t)job.z + 1, k);
#pragma unroll
        for (int j = 0; j < E / 2; j++) A::gs_last(x[j], x[j + E / 2], sx, sy, k);
        uint64_t *o = dst + (size_t)e_lo * 256 + col;
#pragma unroll
        for (int i = 0; i < E; i++) o[(size_t)i * 16 * 256] = A::canon_inv(x[i], k);
        __syncthreads();
    }
    cluster.sync();
}

__global__ void __cluster_dims__(CL_SIZE, 1, 1) __launch_bounds__(CL_THREADS, 2) ntt_inv_cluster(NttArgs a) {
    extern __shared__ __align__(16) uint64_t cl_smem[];
    const Job job = get_job(a, blockIdx.x / CL_SIZE);
    const Mod md = a.mod[job.y];
    if (md.q < FP_LIMIT) inv_cluster_body<ArithFp>(a, cl_smem, job, md);
    else if (md.q < WIDE_LIMIT) inv_cluster_body<ArithInt<true>>(a, cl_smem, job, md);
    else inv_cluster_body<ArithInt<false>>(a, cl_smem, job, md);
}

}  // namespace b2
