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
#include "modarith.cuh"

namespace b2 {

struct Mod {
    uint64_t q, r0, r1, pad;  // r = floor(2^128 / q)
};

// One job = one limb transform: where the limb lives and which prime's tables it uses.
// x = slot in the transform's own buffer, y = prime index, z/w = extra slots for epilogues.
using Job = uint4;

struct NttArgs {
    const uint64_t *src;  // limb `slot` at src + slot * N
    uint64_t *dst;
    const Job *jobs;       // nullptr: slot = job, prime = first_prime + job
    uint32_t first_prime;
    uint32_t logN;
    const W2 *tw;          // [size_QP][N] {w, shoup(w)}
    const Mod *mod;        // [size_QP]
    const W2 *fin;         // inverse only: [idx][2] = {scale of the x outputs, last-stage twiddle}
};

__device__ __forceinline__ Job get_job(const NttArgs &a, uint32_t j) {
    if (a.jobs) return a.jobs[j];
    return make_uint4(j, a.first_prime + j, a.first_prime + j, 0);
}

// ---- epilogues of the last forward pass ------------------------------------------------------
// Each receives canonical values and decides where they go.
struct EpiStore {
    uint64_t *dst;
    __device__ __forceinline__ void init(const NttArgs &a, const Job &job, size_t N) { dst = a.dst + (size_t)job.x * N; }
    __device__ __forceinline__ void put(size_t i, uint64_t v, uint64_t) const { dst[i] = v; }
    __device__ __forceinline__ void put2(size_t i, uint64_t v0, uint64_t v1, uint64_t) const {
        *reinterpret_cast<ulonglong2 *>(dst + i) = make_ulonglong2(v0, v1);
    }
};

// out[job.w] = acc[job.w] + (minuend[job.z] - v) * k[prime]   (ModDown + add-to-ciphertext:
// src/rns_bconv.cu:820-821 with include/ntt_radix8_tmpl.cuh:203-233, then :763-769), or without
// the accumulate (rescale: src/rns.cu:1146-1158).
template <bool ACCUM>
struct EpiSubMul {
    const uint64_t *minuend;  // [slots][N]
    uint64_t *out;            // [slots][N]
    const W2 *k;              // per prime
    const uint64_t *m_;
    uint64_t *o_;
    W2 kk;
    __device__ __forceinline__ void init(const NttArgs &, const Job &job, size_t N) {
        m_ = minuend + (size_t)job.z * N;
        o_ = out + (size_t)job.w * N;
        kk = k[job.y];
    }
    __device__ __forceinline__ uint64_t one(size_t i, uint64_t v, uint64_t q) const {
        uint64_t r = mul_shoup(sub_mod(m_[i], v, q), kk, q);
        if (ACCUM) r = add_mod(o_[i], r, q);
        return r;
    }
    __device__ __forceinline__ void put(size_t i, uint64_t v, uint64_t q) const { o_[i] = one(i, v, q); }
    __device__ __forceinline__ void put2(size_t i, uint64_t v0, uint64_t v1, uint64_t q) const {
        ulonglong2 m = *reinterpret_cast<const ulonglong2 *>(m_ + i);
        uint64_t r0 = mul_shoup(sub_mod(m.x, v0, q), kk, q);
        uint64_t r1 = mul_shoup(sub_mod(m.y, v1, q), kk, q);
        if (ACCUM) {
            ulonglong2 o = *reinterpret_cast<const ulonglong2 *>(o_ + i);
            r0 = add_mod(o.x, r0, q);
            r1 = add_mod(o.y, r1, q);
        }
        *reinterpret_cast<ulonglong2 *>(o_ + i) = make_ulonglong2(r0, r1);
    }
};

template <int LOG_T, int RC>
__device__ __forceinline__ int pad_idx(int e) { return e + (e >> RC); }


// ---- stage runners: compile-time recursion keeps every register index a constant --------------
// forward: E residues x[], local stages S..R-1 of this round; twiddle index = tw0 + ((k0 << S) + g)
// where tw0 = P << (stage offset) is folded by the caller through `shift`.
template <int S, int R, int E>
__device__ __forceinline__ void ct_stages(uint64_t (&x)[E], const W2 *tw, size_t P, int shift, size_t k0, uint64_t q, uint64_t q2) {
    if constexpr (S < R) {
        constexpr int half = E >> (S + 1);
#pragma unroll
        for (int g = 0; g < (1 << S); g++) {
            const W2 w = ldg_w2(tw + (P << (shift + S)) + (k0 << S) + g);
#pragma unroll
            for (int j = 0; j < half; j++) ct_bfly(x[g * 2 * half + j], x[g * 2 * half + j + half], w, q, q2);
        }
        ct_stages<S + 1, R, E>(x, tw, P, shift, k0, q, q2);
    }
}

// inverse: local stages U..R-1 (gap 2^U); twiddle index = (m0 >> U) * P + (k0 >> U) + g with
// m0 = sub-transform size >> (1 + stages already done), k0 = first pair group of this thread at U = 0.
template <int U, int R, int E>
__device__ __forceinline__ void gs_stages(uint64_t (&x)[E], const W2 *tw, size_t P, int m0, size_t k0, uint64_t q, uint64_t q2) {
    if constexpr (U < R) {
        constexpr int gap = 1 << U;
#pragma unroll
        for (int g = 0; g < (E >> (U + 1)); g++) {
            const W2 w = ldg_w2(tw + (size_t)(m0 >> U) * P + (k0 >> U) + g);
#pragma unroll
            for (int j = 0; j < gap; j++) gs_bfly(x[g * 2 * gap + j], x[g * 2 * gap + j + gap], w, q, q2);
        }
        gs_stages<U + 1, R, E>(x, tw, P, m0, k0, q, q2);
    }
}

// ================================================================================================
// forward pass: R1 strided stages, exchange, R2 contiguous stages
// ================================================================================================
template <int LOG_T, int R1, int R2, int LOG_C, bool COLS, bool LAST, class Epi>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) / (1 << (R1 > R2 ? R1 : R2)))
ntt_fwd_pass(NttArgs a, Epi epi) {
    static_assert(R1 + R2 == LOG_T, "stage split");
    constexpr int T = 1 << LOG_T, E1 = 1 << R1, E2 = 1 << R2, C = 1 << LOG_C;
    constexpr int EPT = E1 > E2 ? E1 : E2;
    constexpr int THREADS = C * T / EPT;
    constexpr int TPAD = T + (T >> R2);
    __shared__ uint64_t sm[C * TPAD];

    const size_t N = (size_t)1 << a.logN;
    const uint32_t tiles = (uint32_t)(N >> (LOG_T + LOG_C));
    const uint32_t jobi = blockIdx.x / tiles, tile = blockIdx.x % tiles;
    const Job job = get_job(a, jobi);
    const Mod md = a.mod[job.y];
    const uint64_t q = md.q, q2 = 2 * md.q;
    const W2 *tw = a.tw + (size_t)job.y * N;
    const uint64_t *src = a.src + (size_t)job.x * N;
    const size_t estride = COLS ? (N >> LOG_T) : 1;
    const size_t cstride = COLS ? 1 : T;
    const size_t base = COLS ? (size_t)tile * C : (size_t)tile * C * T;
    const uint32_t n1 = (uint32_t)(N >> LOG_T);  // number of sub-transforms per limb
    const int tid = threadIdx.x;

    // ---- round 1 ---------------------------------------------------------------------------
#pragma unroll
    for (int gi = 0; gi < EPT / E1; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / E2);
        const int elo = COLS ? (gid / C) : (gid % E2);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        uint64_t x[E1];
        const uint64_t *p = src + base + (size_t)c * cstride + (size_t)elo * estride;
#pragma unroll
        for (int i = 0; i < E1; i++) x[i] = p[(size_t)i * E2 * estride];
        ct_stages<0, R1, E1>(x, tw, P, 0, 0, q, q2);
#pragma unroll
        for (int i = 0; i < E1; i++) {
            const int pe = pad_idx<LOG_T, R2>(elo + i * E2);
            sm[COLS ? (pe * C + c) : (c * TPAD + pe)] = x[i];
        }
    }
    __syncthreads();
    // ---- round 2 ---------------------------------------------------------------------------
    Epi e = epi;
    if (LAST) e.init(a, job, N);
    uint64_t *dst = a.dst + (size_t)job.x * N;
#pragma unroll
    for (int gi = 0; gi < EPT / E2; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / E1);
        const int ehi = COLS ? (gid / C) : (gid % E1);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        uint64_t x[E2];
#pragma unroll
        for (int i = 0; i < E2; i++) {
            const int pe = pad_idx<LOG_T, R2>(ehi * E2 + i);
            x[i] = sm[COLS ? (pe * C + c) : (c * TPAD + pe)];
        }
        ct_stages<0, R2, E2>(x, tw, P, R1, ehi, q, q2);
        const size_t o = base + (size_t)c * cstride + (size_t)ehi * E2 * estride;
        if (LAST) {
#pragma unroll
            for (int i = 0; i < E2; i++) x[i] = csub(csub(x[i], q2), q);
            if (COLS) {
#pragma unroll
                for (int i = 0; i < E2; i++) e.put(o + (size_t)i * estride, x[i], q);
            } else {
#pragma unroll
                for (int i = 0; i < E2; i += 2) e.put2(o + i, x[i], x[i + 1], q);
            }
        } else {
#pragma unroll
            for (int i = 0; i < E2; i++) dst[o + (size_t)i * estride] = x[i];
        }
    }
}

// ================================================================================================
// inverse pass: RA contiguous stages, exchange, RB strided stages
// ================================================================================================
template <int LOG_T, int RA, int RB, int LOG_C, bool COLS, bool LAST>
__global__ void __launch_bounds__((1 << (LOG_C + LOG_T)) / (1 << (RA > RB ? RA : RB)))
ntt_inv_pass(NttArgs a) {
    static_assert(RA + RB == LOG_T, "stage split");
    constexpr int T = 1 << LOG_T, EA = 1 << RA, EB = 1 << RB, C = 1 << LOG_C;
    constexpr int EPT = EA > EB ? EA : EB;
    constexpr int THREADS = C * T / EPT;
    constexpr int TPAD = T + (T >> RA);
    __shared__ uint64_t sm[C * TPAD];

    const size_t N = (size_t)1 << a.logN;
    const uint32_t tiles = (uint32_t)(N >> (LOG_T + LOG_C));
    const uint32_t jobi = blockIdx.x / tiles, tile = blockIdx.x % tiles;
    const Job job = get_job(a, jobi);
    const Mod md = a.mod[job.y];
    const uint64_t q = md.q, q2 = 2 * md.q;
    const W2 *tw = a.tw + (size_t)job.y * N;
    const uint64_t *src = a.src + (size_t)job.x * N;
    uint64_t *dst = a.dst + (size_t)job.x * N;
    const size_t estride = COLS ? (N >> LOG_T) : 1;
    const size_t cstride = COLS ? 1 : T;
    const size_t base = COLS ? (size_t)tile * C : (size_t)tile * C * T;
    const uint32_t n1 = (uint32_t)(N >> LOG_T);
    const int tid = threadIdx.x;

    // ---- round 1: contiguous runs of EA residues ----------------------------------------------
#pragma unroll
    for (int gi = 0; gi < EPT / EA; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / EB);
        const int ehi = COLS ? (gid / C) : (gid % EB);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        uint64_t x[EA];
        const uint64_t *p = src + base + (size_t)c * cstride + (size_t)ehi * EA * estride;
        if (COLS) {
#pragma unroll
            for (int i = 0; i < EA; i++) x[i] = p[(size_t)i * estride];
        } else {
#pragma unroll
            for (int i = 0; i < EA; i += 2) {
                ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(p + i);
                x[i] = v.x;
                x[i + 1] = v.y;
            }
        }
        gs_stages<0, RA, EA>(x, tw, P, T >> 1, (size_t)ehi * (EA >> 1), q, q2);
#pragma unroll
        for (int i = 0; i < EA; i++) {
            const int pe = pad_idx<LOG_T, RA>(ehi * EA + i);
            sm[COLS ? (pe * C + c) : (c * TPAD + pe)] = x[i];
        }
    }
    __syncthreads();
    // ---- round 2: stride EA ---------------------------------------------------------------------
#pragma unroll
    for (int gi = 0; gi < EPT / EB; gi++) {
        const int gid = tid + gi * THREADS;
        const int c = COLS ? (gid % C) : (gid / EA);
        const int elo = COLS ? (gid / C) : (gid % EA);
        const uint32_t P = COLS ? 1u : (n1 + tile * C + c);
        uint64_t x[EB];
#pragma unroll
        for (int i = 0; i < EB; i++) {
            const int pe = pad_idx<LOG_T, RA>(elo + i * EA);
            x[i] = sm[COLS ? (pe * C + c) : (c * TPAD + pe)];
        }
        gs_stages<0, (LAST ? RB - 1 : RB), EB>(x, tw, P, T >> (RA + 1), 0, q, q2);
        if (LAST) {
            // last stage of the whole transform (twiddle index 1): the x outputs take the scale,
            // the y outputs a twiddle that already carries it (src/host/ntt.cu:53-55,
            // include/ntt_radix8_tmpl.cuh:566-568); callers fold further per-limb factors in.
            constexpr int gap = EB / 2;
            const W2 sx = ldg_w2(a.fin + 2 * (size_t)job.z);
            const W2 sy = ldg_w2(a.fin + 2 * (size_t)job.z + 1);
#pragma unroll
            for (int j = 0; j < gap; j++) {
                const uint64_t sm_ = x[j] + x[j + gap];
                const uint64_t df_ = x[j] - x[j + gap] + q2;
                x[j] = mul_shoup(sm_, sx, q);
                x[j + gap] = mul_shoup(df_, sy, q);
            }
        }
        uint64_t *o = dst + base + (size_t)c * cstride + (size_t)elo * estride;
#pragma unroll
        for (int i = 0; i < EB; i++) o[(size_t)i * EA * estride] = x[i];
    }
}

}  // namespace b2
