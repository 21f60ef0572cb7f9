// b200fhe.cu - context, kernels and C ABI of libb200fhe.so (see include/b200fhe.h).
//
// Device data layout: ciphertext buffers are the reference's [poly][limb][N] uint64 arrays.
// Tables live in one context: per prime {q, floor(2^128/q)}; forward and inverse twiddles as
// interleaved {w, shoup(w)} pairs, [size_QP][N] each (64 MiB at N = 2^16 with 32 primes); and per
// level (number of Q limbs l) one "plan": job lists for every transform of the key switch,
// base-conversion matrices per digit and the constants folded into the inverse transform.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200fhe.h"
#include "ntt_kernels.cuh"
#include "sampler.cuh"
#include "encoder.cuh"
#include "bconv_tc.cuh"

using namespace b2;
typedef unsigned __int128 u128_t;

// ------------------------------------------------------------------------------------------------
// error handling
// ------------------------------------------------------------------------------------------------
static thread_local std::string g_err;
static int fail(int code, const std::string &msg) {
    g_err = msg;
    return code;
}
#define CUDA_TRY(expr)                                                                            \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess)                                                                    \
            return fail((int)e_, std::string(#expr) + ": " + cudaGetErrorString(e_));             \
    } while (0)
#define LAUNCH_CHECK(name)                                                                        \
    do {                                                                                          \
        cudaError_t e_ = cudaGetLastError();                                                      \
        if (e_ != cudaSuccess) return fail((int)e_, std::string(name) + ": " + cudaGetErrorString(e_)); \
    } while (0)

#include <atomic>
static std::atomic<uint64_t> g_launches{0};

extern "C" const char *b2_last_error(void) { return g_err.c_str(); }
extern "C" uint64_t b2_launch_count(void) { return g_launches.load(); }
extern "C" int b2_version(void) { return 1; }

// ------------------------------------------------------------------------------------------------
// host number theory (own statement of src/host/numth.cu, modulus.cu, ntt.cu, rns.cu semantics)
// ------------------------------------------------------------------------------------------------
static inline uint64_t h_mulmod(uint64_t a, uint64_t b, uint64_t q) { return (uint64_t)((u128_t)a * b % q); }
static uint64_t h_powmod(uint64_t a, uint64_t e, uint64_t q) {
    uint64_t r = 1;
    a %= q;
    for (; e; e >>= 1) {
        if (e & 1) r = h_mulmod(r, a, q);
        a = h_mulmod(a, a, q);
    }
    return r;
}
static inline uint64_t h_invmod(uint64_t a, uint64_t q) { return h_powmod(a % q, q - 2, q); }
static inline uint64_t h_shoup(uint64_t w, uint64_t q) { return (uint64_t)(((u128_t)w << 64) / q); }
static inline W2 h_w2(uint64_t w, uint64_t q) { return W2{w, h_shoup(w, q)}; }
// Transform constants as the kernels want them for this prime: {w, shoup(w)} for the integer
// butterflies, the bit patterns of {double(w), double(w/q)} for primes on the FP64 path.
static inline W2 h_tw_enc(uint64_t w, uint64_t q) {
    if (q >= b2::FP_LIMIT) return h_w2(w, q);
    const double wd = (double)w, wq = (double)w / (double)q;
    W2 r;
    memcpy(&r.w, &wd, 8);
    memcpy(&r.ws, &wq, 8);
    return r;
}

static bool h_is_prime(uint64_t v) {
    static const uint64_t wit[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
    if (v < 2) return false;
    for (uint64_t p : wit) {
        if (v == p) return true;
        if (v % p == 0) return false;
    }
    uint64_t d = v - 1;
    int r = 0;
    while (!(d & 1)) d >>= 1, r++;
    for (uint64_t a : wit) {
        uint64_t x = h_powmod(a, d, v);
        if (x == 1 || x == v - 1) continue;
        bool composite = true;
        for (int i = 1; i < r && composite; i++) {
            x = h_mulmod(x, x, v);
            if (x == v - 1) composite = false;
        }
        if (composite) return false;
    }
    return true;
}

extern "C" int b2_create_coeff_modulus(size_t N, const int *bit_sizes, size_t count, uint64_t *out) {
    if (!bit_sizes || !out || count == 0 || count > 64) return fail(B2_EINVAL, "create_coeff_modulus: bad count");
    if (N < 2 || (N & (N - 1)) || N > 131072) return fail(B2_EINVAL, "create_coeff_modulus: poly_modulus_degree is invalid");
    for (size_t i = 0; i < count; i++)
        if (bit_sizes[i] < 2 || bit_sizes[i] > 60) return fail(B2_EINVAL, "create_coeff_modulus: bit_sizes is invalid");
    const uint64_t step = 2 * (uint64_t)N;
    std::map<int, std::vector<uint64_t>> table;
    for (size_t i = 0; i < count; i++) table[bit_sizes[i]];
    for (auto &kv : table) {
        size_t need = std::count(bit_sizes, bit_sizes + count, kv.first);
        uint64_t top = (uint64_t)1 << kv.first, low = top >> 1;
        if (top < step) return fail(B2_EINVAL, "create_coeff_modulus: failed to find enough qualifying primes");
        for (uint64_t v = top - step + 1; kv.second.size() < need && v > low; v -= step) {
            if (h_is_prime(v)) kv.second.push_back(v);
            if (v < step) break;
        }
        if (kv.second.size() < need) return fail(B2_EINVAL, "create_coeff_modulus: failed to find enough qualifying primes");
    }
    // every bit size hands out its primes smallest-first
    for (size_t i = 0; i < count; i++) {
        auto &v = table[bit_sizes[i]];
        out[i] = v.back();
        v.pop_back();
    }
    return B2_OK;
}

// smallest primitive 2N-th root of unity mod q (0 if none)
static uint64_t h_min_root(uint64_t degree, uint64_t q) {
    if ((q - 1) % degree) return 0;
    uint64_t cof = (q - 1) / degree, r = 0;
    for (uint64_t g = 2; g < q && !r; g++) {
        uint64_t c = h_powmod(g, cof, q);
        if (h_powmod(c, degree / 2, q) == q - 1) r = c;
    }
    uint64_t sq = h_mulmod(r, r, q), cur = r, best = r;
    for (uint64_t i = 0; i < degree / 2; i++) {
        best = std::min(best, cur);
        cur = h_mulmod(cur, sq, q);
    }
    return best;
}

static inline uint32_t h_bitrev(uint32_t x, int bits) {
    uint32_t r = 0;
    for (int i = 0; i < bits; i++) r |= ((x >> i) & 1u) << (bits - 1 - i);
    return r;
}

// ------------------------------------------------------------------------------------------------
// context
// ------------------------------------------------------------------------------------------------
struct BconvGroup {
    uint32_t in_slot0;   // first input limb (slot in the source buffer)
    uint32_t ni;         // number of input limbs
    uint32_t mat_off;    // offset (in u64) of this group's [n_out][ni] matrix
    uint32_t out_begin;  // first entry of this group in the output list
    uint32_t n_out;
    uint32_t out_slot_base;  // added to every output slot
    uint32_t copy_dst_slot0; // ModUp: where the digit's own limbs are copied to
    uint32_t in_pieces;      // 21-bit pieces needed to hold an input residue (2 below 2^42, else 3)
};

// One base conversion launch in tensor-core form: job list (grid.y), the groups and byte images they index
struct TcSet {
    const TcJob *jobs = nullptr;
    const TcGroup *groups = nullptr;
    const uint8_t *images = nullptr;
    uint32_t n_jobs = 0, jobs_per_poly = 0, max_alloc = 32;
};

struct LevelPlan {
    uint32_t l = 0, beta = 0;
    // offsets into the level blob (device), counts
    Job *jobs_up_intt = nullptr;   // l
    Job *jobs_up_ntt = nullptr;    // n_up_ntt
    uint32_t n_up_ntt = 0;
    Job *jobs_up_rows = nullptr;   // the jobs of jobs_up_ntt whose limb is not on an FP64 prime of Q (fused inner product)
    uint32_t n_up_rows = 0;
    uint32_t n_wideQ = 0;          // leading Q limbs on primes >= 2^41
    bool mac_ok = false;           // Q limbs [n_wideQ, l) all on FP64 primes: the fused row pass + inner product applies
    Job *jobs_dn_intt = nullptr;   // 2*alpha (poly-major), prefix alpha for one polynomial
    Job *jobs_dn_ntt = nullptr;    // 2*l
    Job *jobs_dnf_intt = nullptr;  // fused key switch: P limbs live compactly in [2][alpha][N]
    Job *jobs_dnf_ntt = nullptr;   // 2*l, epilogue subtracts from the ciphertext
    BconvGroup *grp_dnf = nullptr; // 2
    Job *jobs_rs_intt = nullptr;   // 3 (one per polynomial)
    Job *jobs_rs_ntt = nullptr;    // 3*(l-1)
    W2 *fin_up = nullptr;          // [l][2]
    W2 *qlast_inv = nullptr;       // [size_QP] indexed by prime (valid j < l-1)
    BconvGroup *grp_up = nullptr;  // beta
    uint2 *outs_up = nullptr;      // (slot, prime) list, beta groups concatenated
    uint64_t *mat_up = nullptr;
    double *matd_up = nullptr;     // mat_up as 21-bit pieces of (entry * 2^64 mod p), [..][3]
    BconvGroup *grp_dn = nullptr;  // 2 (one per polynomial)
    uint2 *outs_dn = nullptr;      // l entries shared by both groups
    BconvGroup *grp_rs = nullptr;  // 3
    uint2 *outs_rs = nullptr;      // l-1
    void *blob = nullptr;
    TcSet tc_up, tc_dn, tc_dnf;    // tensor-core form of the ModUp / ModDown / fused-ModDown conversions
    void *tc_blob = nullptr;
};

struct b2_ctx {
    int device = 0;
    size_t N = 0;
    int logN = 0;
    size_t size_QP = 0, size_Q = 0, size_P = 0;
    std::vector<uint64_t> q;
    std::vector<W2> h_tw, h_itw;  // host copies [size_QP][N]
    Mod *d_mod = nullptr;
    W2 *d_tw = nullptr, *d_itw = nullptr;
    W2 *d_fin_plain = nullptr;  // [size_QP][2] = {N^-1, itw[1]}
    W2 *d_fin_P = nullptr;      // [size_P][2]  = the same times (P/p_i)^-1 mod p_i
    W2 *d_Pinv = nullptr;       // [size_QP] indexed by prime (valid for Q primes): P^-1 mod q_j
    W2 *d_macfin = nullptr;     // [size_QP] closing constant of the fused inner product's Montgomery sums: P^-1 * 2^64 mod q_j, 2^64 mod p_i
    uint64_t *d_mat_dn = nullptr;  // [size_Q][size_P]: (P/p_i) mod q_j
    uint64_t *d_mat_dn_pinv = nullptr;  // the same times P^-1 mod q_j (fused key switch)
    uint64_t *d_one = nullptr;     // [size_QP] ones: the [n_out][1] "matrix" of the rescale reduction
    double *d_matd_dn = nullptr, *d_matd_dn_pinv = nullptr, *d_matd_one = nullptr;  // FP64 piece forms
    struct RedcMeta {
        uint64_t p, ninv;  // ninv = -p^-1 mod 2^64
        uint32_t pieces, pad;
        uint64_t pad2;
        double cw[4], cwq[4];  // p < 2^42: 2^(21 w) mod p for w = 1..4, and the same divided by p
    };
    RedcMeta *d_redc = nullptr;    // [size_QP]
    bool bconv_fp = false;         // every digit satisfies sum(q_i) < 2^64 and alpha <= 8
    bool bconv_tc = false;         // base conversions on the tensor cores (alpha <= 8, primes above 2^16; off with B2_BCONV=fp|int)
    bool bconv_int = false;        // B2_BCONV=int: force the 128-bit integer kernel
    int tc_wg = 4;                 // warpgroups per CTA of the tensor-core conversion (B2_BCONV_WG = 1, 2, 4)
    bool tc_simple = false;        // B2_BCONV_TC_SIMPLE=1: one CTA per tile instead of the persistent pipelined kernel
    bool tc_serial_ld = false;     // B2_BCONV_SERIAL_LD=1: the epilogue waits for every TMEM load before it reduces (no load in flight)
    uint32_t tc_max_groups = 16;   // B2_BCONV_GROUPS: column groups per conversion job (8: at most 128 TMEM columns, four CTAs per SM)
    uint32_t *d_err = nullptr;     // device status word: set by a kernel whose bounded wait ran out
    std::vector<uint64_t> h_mat_dn, h_mat_dn_pinv;  // host copies of the ModDown matrices [size_Q][size_P]
    bool use_cluster = false;      // N = 2^16: single-launch transforms on 8-CTA clusters
    bool use_pipe = false;         // N = 2^16: persistent passes with asynchronous double-buffered tile loads
    bool mac_interleave = false;   // B2_KS_FUSED_ORDER=1: consecutive CTAs of the fused pass walk limbs, not tiles (measured slower)
    // The fused pass may also take the limbs on primes of 41 bits and more (q0 and P at the usual parameters): 10 launches
    // instead of 12 and no stored digits at all. Measured on B200 at N = 2^16, l = 24: single calls lose 4 % of their
    // four-stream throughput to it (the stand-alone inner product is memory-bound and hides behind other streams' transforms;
    // fused, it is integer-multiply work) though a lone key switch gains 8 us; batched calls gain 1 %. So it is on for
    // batched calls and off for single ones unless B2_KS_FUSED_WIDE = 0 | 1 says otherwise.
    int mac_wide = -1;
    bool use_mac = false;          // N = 2^16: ModUp's last forward pass carries the inner product (off with B2_KS_FUSED_IP=0)
    int sm_count = 148;
    // RNS-limb sharding of one ciphertext over `shard_world` GPUs: this rank's slice of every list
    int shard_rank = 0, shard_world = 1;
    struct ShardPlan {
        uint32_t q0 = 0, nq = 0, p0 = 0, np = 0, n_up_ntt = 0;
        Job *jobs_up_ntt = nullptr, *jobs_dn_intt = nullptr, *jobs_dn_ntt = nullptr;
        BconvGroup *grp_up = nullptr, *grp_dn = nullptr;
        uint2 *outs_up = nullptr, *outs_dn = nullptr;
        uint64_t *mat_up = nullptr, *mat_dn = nullptr;
        double *matd_up = nullptr, *matd_dn = nullptr;
        void *blob = nullptr;
        TcSet tc_up, tc_dn;
        // the batched phases keep the P limbs of a batch as [P limb][polynomial][set]: this rank's P limbs are one
        // contiguous block, so the exchange before ModDown is a single all-gather
        Job *jobs_dn_intt_b = nullptr;
        TcSet tc_dn_b;
        void *tc_blob = nullptr;
    };
    std::vector<ShardPlan> shard;  // index l; empty until b2_ctx_set_shard
    std::vector<LevelPlan> plan;   // index l (1..size_Q)
    std::map<uint32_t, uint32_t *> galois;  // elt -> device gather table
    std::mutex mu;
    // optional per-kernel timing: CUDA events recorded around every launch on the launching stream
    bool profiling = false;
    struct ProfRec {
        const char *name;
        cudaEvent_t e0, e1;
    };
    std::vector<ProfRec> prof;
};

// Brackets one kernel launch: counts it and, when profiling is on, records events around it.
struct LaunchScope {
    b2_ctx *c;
    cudaStream_t s;
    int idx = -1;
    LaunchScope(const b2_ctx *ctx, cudaStream_t st, const char *name) : c(const_cast<b2_ctx *>(ctx)), s(st) {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (c->profiling) {
            b2_ctx::ProfRec r{name, nullptr, nullptr};
            cudaEventCreate(&r.e0);
            cudaEventCreate(&r.e1);
            cudaEventRecord(r.e0, s);
            c->prof.push_back(r);
            idx = (int)c->prof.size() - 1;
        }
    }
    ~LaunchScope() {
        if (idx >= 0) cudaEventRecord(c->prof[idx].e1, s);
    }
};

template <typename T>
static T *blob_take(char *&cur, size_t count) {
    uintptr_t p = (reinterpret_cast<uintptr_t>(cur) + 15) & ~uintptr_t(15);
    cur = reinterpret_cast<char *>(p + count * sizeof(T));
    return reinterpret_cast<T *>(p);
}

static inline uint32_t phys_prime(const b2_ctx *c, size_t l, size_t t) { return (uint32_t)(t < l ? t : c->size_Q + (t - l)); }

// product of the primes in [s, e) except index `skip`, mod p
static uint64_t punctured(const std::vector<uint64_t> &q, size_t s, size_t e, size_t skip, uint64_t p) {
    uint64_t r = 1 % p;
    for (size_t k = s; k < e; k++)
        if (k != skip) r = h_mulmod(r, q[k] % p, p);
    return r;
}

// 21-bit pieces (as doubles) of a matrix entry: the operand form of the FP64 base conversion
static inline void h_pieces(uint64_t m, uint64_t p, double *out3) {
    // outputs below 2^42 are reduced in FP64 (no Montgomery factor); larger ones by Montgomery reduction
    const uint64_t v = p < (1ull << 42) ? m % p : (uint64_t)((((u128_t)m) << 64) % p);
    out3[0] = (double)(v & 0x1FFFFF);
    out3[1] = (double)((v >> 21) & 0x1FFFFF);
    out3[2] = (double)(v >> 42);
}
static inline uint32_t h_npieces(uint64_t q) { return q < (1ull << 42) ? 2u : 3u; }

// uploads what a TcBuild holds as one blob and points the sets' job lists (given as [first job, count) ranges) into it
static int tc_upload(const TcBuild &b, void **blob, std::initializer_list<std::pair<TcSet *, std::pair<uint32_t, uint32_t>>> sets) {
    const size_t jb = (b.jobs.size() * sizeof(TcJob) + 255) & ~size_t(255), gb = (b.groups.size() * sizeof(TcGroup) + 255) & ~size_t(255);
    const size_t total = jb + gb + b.images.size() + 256;
    if (cudaMalloc(blob, total) != cudaSuccess) return fail(B2_ENOMEM, "cudaMalloc(tensor-core conversion plan) failed");
    char *base = (char *)*blob;
    cudaError_t e = cudaMemcpy(base, b.jobs.data(), b.jobs.size() * sizeof(TcJob), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(base + jb, b.groups.data(), b.groups.size() * sizeof(TcGroup), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(base + jb + gb, b.images.data(), b.images.size(), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail((int)e, "cudaMemcpy(tensor-core conversion plan) failed");
    for (auto &s : sets) {
        TcSet *ts = s.first;
        ts->jobs = (const TcJob *)base + s.second.first;
        ts->n_jobs = s.second.second;
        ts->groups = (const TcGroup *)(base + jb);
        ts->images = (const uint8_t *)(base + jb + gb);
        ts->max_alloc = 32;
        for (uint32_t j = 0; j < s.second.second; j++) ts->max_alloc = std::max(ts->max_alloc, b.jobs[s.second.first + j].alloc_cols);
    }
    return B2_OK;
}

static int build_level(b2_ctx *c, size_t l) {
    const size_t N = c->N, alpha = c->size_P, sQ = c->size_Q;
    const size_t beta = (l + alpha - 1) / alpha, lP = l + alpha;
    LevelPlan &pl = c->plan[l];
    pl.l = (uint32_t)l;
    pl.beta = (uint32_t)beta;
    const size_t n_up_ntt = beta * lP - l;
    const size_t mat_up_words = beta * lP * alpha;
    // host staging mirrors the device blob
    size_t bytes = 64 + sizeof(Job) * (l + 2 * n_up_ntt + 4 * alpha + 4 * l + 3 + 3 * l) + sizeof(W2) * (2 * l + c->size_QP) +
                   sizeof(BconvGroup) * (beta + 4 + 3) + sizeof(uint2) * (n_up_ntt + l + l) + 8 * mat_up_words * 4 + 16 * 24;
    std::vector<char> host(bytes, 0);
    char *cur = host.data();
    auto *jobs_up_intt = blob_take<Job>(cur, l);
    auto *jobs_up_ntt = blob_take<Job>(cur, n_up_ntt);
    auto *jobs_up_rows = blob_take<Job>(cur, n_up_ntt);
    auto *jobs_dn_intt = blob_take<Job>(cur, 2 * alpha);
    auto *jobs_dn_ntt = blob_take<Job>(cur, 2 * l);
    auto *jobs_dnf_intt = blob_take<Job>(cur, 2 * alpha);
    auto *jobs_dnf_ntt = blob_take<Job>(cur, 2 * l);
    auto *grp_dnf = blob_take<BconvGroup>(cur, 2);
    auto *jobs_rs_intt = blob_take<Job>(cur, 3);
    auto *jobs_rs_ntt = blob_take<Job>(cur, 3 * l);
    auto *fin_up = blob_take<W2>(cur, 2 * l);
    auto *qlast_inv = blob_take<W2>(cur, c->size_QP);
    auto *grp_up = blob_take<BconvGroup>(cur, beta);
    auto *outs_up = blob_take<uint2>(cur, n_up_ntt);
    auto *mat_up = blob_take<uint64_t>(cur, mat_up_words);
    auto *matd_up = blob_take<double>(cur, mat_up_words * 3);
    auto *grp_dn = blob_take<BconvGroup>(cur, 2);
    auto *outs_dn = blob_take<uint2>(cur, l);
    auto *grp_rs = blob_take<BconvGroup>(cur, 3);
    auto *outs_rs = blob_take<uint2>(cur, l);
    const size_t used = cur - host.data();
    if (used > bytes) return fail(B2_ENOMEM, "level blob overflow");

    // ---- ModUp (src/rns_bconv.cu:530-628; constants src/rns.cu:149-189) ----
    size_t up_i = 0, mat_off = 0;
    for (size_t d = 0; d < beta; d++) {
        const size_t s = alpha * d, e = std::min(s + alpha, l), ni = e - s;
        uint32_t in_pieces = 2;
        for (size_t i = s; i < e; i++) in_pieces = std::max(in_pieces, h_npieces(c->q[i]));
        grp_up[d] = BconvGroup{(uint32_t)s, (uint32_t)ni, (uint32_t)mat_off, (uint32_t)up_i, (uint32_t)(lP - ni),
                               (uint32_t)(d * lP), (uint32_t)(d * lP + s), in_pieces};
        for (size_t i = s; i < e; i++) {
            const uint64_t qi = c->q[i];
            const uint64_t hatinv = h_invmod(punctured(c->q, s, e, i, qi), qi);
            // INTT's final-stage constants with (Q_d/q_i)^-1 folded in
            const uint64_t ninv = h_invmod(N % qi, qi);
            fin_up[2 * i] = h_tw_enc(h_mulmod(ninv, hatinv, qi), qi);
            fin_up[2 * i + 1] = h_tw_enc(h_mulmod(c->h_itw[i * N + 1].w, hatinv, qi), qi);
            jobs_up_intt[i] = make_uint4((uint32_t)i, (uint32_t)i, (uint32_t)i, (uint32_t)i);
        }
        for (size_t t = 0; t < lP; t++) {
            if (t >= s && t < e) continue;
            const uint32_t pp = phys_prime(c, l, t);
            jobs_up_ntt[up_i] = make_uint4((uint32_t)(d * lP + t), pp, 0, 0);
            outs_up[up_i] = make_uint2((uint32_t)t, pp);
            for (size_t i = s; i < e; i++) {
                mat_up[mat_off] = punctured(c->q, s, e, i, c->q[pp]);
                h_pieces(mat_up[mat_off], c->q[pp], matd_up + 3 * mat_off);
                mat_off++;
            }
            up_i++;
        }
    }
    // limbs whose last forward pass can carry the inner product: Q limbs on FP64 primes behind a prefix of wide ones
    size_t n_wide = 0;
    while (n_wide < l && c->q[n_wide] >= b2::FP_LIMIT) n_wide++;
    bool mac_ok = n_wide < l && beta <= B2_MAC_MAX_BETA;
    for (size_t i = n_wide; i < l; i++) mac_ok = mac_ok && c->q[i] < b2::FP_LIMIT;
    size_t n_up_rows = 0;
    for (size_t j = 0; j < n_up_ntt; j++) {
        const size_t t = jobs_up_ntt[j].x % lP;
        if (t < n_wide || t >= l) jobs_up_rows[n_up_rows++] = jobs_up_ntt[j];
    }
    // ---- ModDown (src/rns_bconv.cu:776-828) ----
    uint32_t p_pieces = 2;
    for (size_t i = 0; i < alpha; i++) p_pieces = std::max(p_pieces, h_npieces(c->q[sQ + i]));
    for (size_t k = 0; k < 2; k++) {
        for (size_t i = 0; i < alpha; i++)
            jobs_dn_intt[k * alpha + i] = make_uint4((uint32_t)(k * lP + l + i), (uint32_t)(sQ + i), (uint32_t)i, (uint32_t)(k * lP + l + i));
        for (size_t j = 0; j < l; j++)
            jobs_dn_ntt[k * l + j] = make_uint4((uint32_t)(k * l + j), (uint32_t)j, (uint32_t)(k * lP + j), (uint32_t)(k * l + j));
        grp_dn[k] = BconvGroup{(uint32_t)(k * lP + l), (uint32_t)alpha, 0, 0, (uint32_t)l, (uint32_t)(k * l), 0, p_pieces};
        for (size_t i = 0; i < alpha; i++)
            jobs_dnf_intt[k * alpha + i] = make_uint4((uint32_t)(k * alpha + i), (uint32_t)(sQ + i), (uint32_t)i, (uint32_t)(k * alpha + i));
        for (size_t j = 0; j < l; j++)
            jobs_dnf_ntt[k * l + j] = make_uint4((uint32_t)(k * l + j), (uint32_t)j, 0, (uint32_t)(k * l + j));
        grp_dnf[k] = BconvGroup{(uint32_t)(k * alpha), (uint32_t)alpha, 0, 0, (uint32_t)l, (uint32_t)(k * l), 0, p_pieces};
    }
    for (size_t j = 0; j < l; j++) outs_dn[j] = make_uint2((uint32_t)j, (uint32_t)j);
    // ---- rescale (src/rns.cu:1128-1183; constants src/rns.cu:66-95) ----
    if (l >= 2) {
        const uint64_t ql = c->q[l - 1];
        for (size_t j = 0; j + 1 < l; j++) {
            qlast_inv[j] = h_w2(h_invmod(ql % c->q[j], c->q[j]), c->q[j]);
            outs_rs[j] = make_uint2((uint32_t)j, (uint32_t)j);
        }
        for (size_t p = 0; p < 3; p++) {
            jobs_rs_intt[p] = make_uint4((uint32_t)(p * l + l - 1), (uint32_t)(l - 1), (uint32_t)(l - 1), (uint32_t)p);
            for (size_t j = 0; j + 1 < l; j++)
                jobs_rs_ntt[p * (l - 1) + j] =
                    make_uint4((uint32_t)(p * (l - 1) + j), (uint32_t)j, (uint32_t)(p * l + j), (uint32_t)(p * (l - 1) + j));
            grp_rs[p] = BconvGroup{(uint32_t)p, 1, 0, 0, (uint32_t)(l - 1), (uint32_t)(p * (l - 1)), 0, h_npieces(ql)};
        }
    }
    if (cudaMalloc(&pl.blob, used) != cudaSuccess) return fail(B2_ENOMEM, "cudaMalloc(level plan) failed");
    cudaError_t e = cudaMemcpy(pl.blob, host.data(), used, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail((int)e, "cudaMemcpy(level plan) failed");
    auto dev = [&](const void *hp) { return (char *)pl.blob + ((const char *)hp - host.data()); };
    pl.jobs_up_intt = (Job *)dev(jobs_up_intt);
    pl.jobs_up_ntt = (Job *)dev(jobs_up_ntt);
    pl.n_up_ntt = (uint32_t)n_up_ntt;
    pl.jobs_up_rows = (Job *)dev(jobs_up_rows);
    pl.n_up_rows = (uint32_t)n_up_rows;
    pl.n_wideQ = (uint32_t)n_wide;
    pl.mac_ok = mac_ok;
    pl.jobs_dn_intt = (Job *)dev(jobs_dn_intt);
    pl.jobs_dn_ntt = (Job *)dev(jobs_dn_ntt);
    pl.jobs_dnf_intt = (Job *)dev(jobs_dnf_intt);
    pl.jobs_dnf_ntt = (Job *)dev(jobs_dnf_ntt);
    pl.grp_dnf = (BconvGroup *)dev(grp_dnf);
    pl.jobs_rs_intt = (Job *)dev(jobs_rs_intt);
    pl.jobs_rs_ntt = (Job *)dev(jobs_rs_ntt);
    pl.fin_up = (W2 *)dev(fin_up);
    pl.qlast_inv = (W2 *)dev(qlast_inv);
    pl.grp_up = (BconvGroup *)dev(grp_up);
    pl.outs_up = (uint2 *)dev(outs_up);
    pl.mat_up = (uint64_t *)dev(mat_up);
    pl.matd_up = (double *)dev(matd_up);
    pl.grp_dn = (BconvGroup *)dev(grp_dn);
    pl.outs_dn = (uint2 *)dev(outs_dn);
    pl.grp_rs = (BconvGroup *)dev(grp_rs);
    pl.outs_rs = (uint2 *)dev(outs_rs);
    if (c->bconv_tc) {
        // the same conversions as tensor-core jobs: ModUp digits, then ModDown of up to two polynomials with the plain
        // matrix (cx layout [2][lP]) and with the P^-1-carrying one (compact P limbs [2][alpha])
        TcBuild tb;
        tb.max_groups = c->tc_max_groups;
        std::vector<TcSpecOut> outs;
        uint32_t n_up = 0, n_dn = 0, n_dnf = 0;
        for (size_t d = 0; d < beta; d++) {
            const BconvGroup &g = grp_up[d];
            outs.clear();
            for (uint32_t j = 0; j < g.n_out; j++) {
                const uint2 o = outs_up[g.out_begin + j];
                outs.push_back(TcSpecOut{g.out_slot_base + o.x, c->q[o.y], mat_up + g.mat_off + (size_t)j * g.ni});
            }
            n_up += tb.add(g.in_slot0, g.ni, g.copy_dst_slot0, outs);
        }
        uint32_t per_poly = 0;
        for (int fused = 0; fused < 2; fused++)
            for (size_t k = 0; k < 2; k++) {
                const BconvGroup &g = fused ? grp_dnf[k] : grp_dn[k];
                const std::vector<uint64_t> &m = fused ? c->h_mat_dn_pinv : c->h_mat_dn;
                outs.clear();
                for (size_t j = 0; j < l; j++) outs.push_back(TcSpecOut{g.out_slot_base + (uint32_t)j, c->q[j], m.data() + j * alpha});
                per_poly = tb.add(g.in_slot0, g.ni, 0xFFFFFFFFu, outs);
                (fused ? n_dnf : n_dn) += per_poly;
            }
        if (!tb.ok) return fail(B2_EINVAL, "tensor-core base conversion: unsupported prime in the chain");
        int rc = tc_upload(tb, &pl.tc_blob, {{&pl.tc_up, {0u, n_up}}, {&pl.tc_dn, {n_up, n_dn}}, {&pl.tc_dnf, {n_up + n_dn, n_dnf}}});
        if (rc) return rc;
        pl.tc_up.jobs_per_poly = n_up;
        pl.tc_dn.jobs_per_poly = pl.tc_dnf.jobs_per_poly = per_poly;
    }
    return B2_OK;
}

extern "C" void b2_ctx_destroy(b2_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaFree(c->d_mod);
    cudaFree(c->d_tw);
    cudaFree(c->d_itw);
    cudaFree(c->d_fin_plain);
    cudaFree(c->d_fin_P);
    cudaFree(c->d_Pinv);
    cudaFree(c->d_macfin);
    cudaFree(c->d_mat_dn);
    cudaFree(c->d_mat_dn_pinv);
    cudaFree(c->d_one);
    cudaFree(c->d_matd_dn);
    cudaFree(c->d_matd_dn_pinv);
    cudaFree(c->d_matd_one);
    cudaFree(c->d_redc);
    for (auto &pl : c->plan) {
        cudaFree(pl.blob);
        cudaFree(pl.tc_blob);
    }
    cudaFree(c->d_err);
    for (auto &sp : c->shard) {
        cudaFree(sp.blob);
        cudaFree(sp.tc_blob);
    }
    for (auto &kv : c->galois) cudaFree(kv.second);
    delete c;
}

extern "C" int b2_ctx_create(size_t N, const uint64_t *primes, size_t size_QP, size_t size_P, int device, b2_ctx **out) {
    if (!primes || !out) return fail(B2_EINVAL, "ctx_create: null argument");
    *out = nullptr;
    if (N < 4096 || N > 131072 || (N & (N - 1))) return fail(B2_ESIZE, "ctx_create: poly_modulus_degree must be a power of two in [4096, 131072]");
    if (size_QP < 2 || size_QP > 64) return fail(B2_ESIZE, "ctx_create: the coefficient modulus must hold 2..64 primes");
    if (size_P < 1 || size_P >= size_QP) return fail(B2_EINVAL, "ctx_create: special_modulus_size must be in [1, size_QP)");
    if (size_P > 16) return fail(B2_ESIZE, "ctx_create: special_modulus_size above 16 is not built");
    int ndev = 0;
    cudaError_t de = cudaGetDeviceCount(&ndev);
    if (de != cudaSuccess || ndev == 0) return fail(de != cudaSuccess ? (int)de : (int)cudaErrorNoDevice, "ctx_create: no CUDA device (this library has no CPU path)");
    if (device < 0 || device >= ndev) return fail(B2_EINVAL, "ctx_create: bad device index");
    CUDA_TRY(cudaSetDevice(device));

    b2_ctx *c = new b2_ctx();
    c->device = device;
    c->N = N;
    c->logN = __builtin_ctzll(N);
    c->size_QP = size_QP;
    c->size_P = size_P;
    c->size_Q = size_QP - size_P;
    c->q.assign(primes, primes + size_QP);
    for (size_t i = 0; i < size_QP; i++) {
        const uint64_t q = c->q[i];
        if (q < 2 || (q >> 61) || !h_is_prime(q) || (q - 1) % (2 * N)) {
            delete c;
            return fail(B2_EINVAL, "ctx_create: every modulus must be a prime = 1 (mod 2N) of at most 61 bits");
        }
        for (size_t j = 0; j < i; j++)
            if (c->q[j] == q) {
                delete c;
                return fail(B2_EINVAL, "ctx_create: moduli must be distinct");
            }
    }
    // ---- twiddles: tw[br(i)] = psi^i, itw[br(i)] = psi^-i, itw[1] *= N^-1 (src/host/ntt.cu:11-56)
    c->h_tw.resize(size_QP * N);
    c->h_itw.resize(size_QP * N);
    std::vector<Mod> mods(size_QP);
    std::vector<W2> fin_plain(2 * size_QP);
    std::vector<uint32_t> br(N);
    for (size_t i = 0; i < N; i++) br[i] = h_bitrev((uint32_t)i, c->logN);
#pragma omp parallel for schedule(dynamic)
    for (size_t l = 0; l < size_QP; l++) {
        const uint64_t q = c->q[l];
        const uint64_t psi = h_min_root(2 * N, q), ipsi = h_invmod(psi, q);
        W2 *tw = c->h_tw.data() + l * N, *itw = c->h_itw.data() + l * N;
        uint64_t p = psi, ip = ipsi;
        tw[0] = h_w2(1, q);
        itw[0] = h_w2(1, q);
        for (size_t i = 1; i < N; i++) {
            tw[br[i]] = h_w2(p, q);
            itw[br[i]] = h_w2(ip, q);
            p = h_mulmod(p, psi, q);
            ip = h_mulmod(ip, ipsi, q);
        }
        const uint64_t ninv = h_invmod(N % q, q);
        itw[1] = h_w2(h_mulmod(itw[1].w, ninv, q), q);
        fin_plain[2 * l] = h_w2(ninv, q);
        fin_plain[2 * l + 1] = itw[1];
        // floor(2^128 / q) as two words
        u128_t hi = ((u128_t)1 << 64);  // 2^64
        uint64_t r1 = (uint64_t)(hi / q);
        u128_t rem = hi % q;
        uint64_t r0 = (uint64_t)((rem << 64) / q);
        mods[l] = Mod{q, r0, r1, 0};
    }
    // ---- P-related constants (src/rns.cu:100-138, 192-194) ----
    const size_t sQ = c->size_Q, sP = size_P;
    std::vector<W2> fin_P(2 * sP), Pinv(size_QP, W2{0, 0});
    std::vector<uint64_t> mat_dn(sQ * sP), mat_dn_pinv(sQ * sP);
    for (size_t i = 0; i < sP; i++) {
        const uint64_t p = c->q[sQ + i];
        const uint64_t hatinv = h_invmod(punctured(c->q, sQ, size_QP, sQ + i, p), p);
        fin_P[2 * i] = h_tw_enc(h_mulmod(fin_plain[2 * (sQ + i)].w, hatinv, p), p);
        fin_P[2 * i + 1] = h_tw_enc(h_mulmod(fin_plain[2 * (sQ + i) + 1].w, hatinv, p), p);
    }
    for (size_t j = 0; j < sQ; j++) {
        const uint64_t qj = c->q[j];
        uint64_t P = 1;
        for (size_t i = 0; i < sP; i++) {
            P = h_mulmod(P, c->q[sQ + i] % qj, qj);
            mat_dn[j * sP + i] = punctured(c->q, sQ, size_QP, sQ + i, qj);
        }
        Pinv[j] = h_w2(h_invmod(P, qj), qj);
        for (size_t i = 0; i < sP; i++) mat_dn_pinv[j * sP + i] = h_mulmod(mat_dn[j * sP + i], Pinv[j].w, qj);
    }
    const std::vector<uint64_t> ones(size_QP, 1);
    std::vector<double> matd_dn(3 * sQ * sP), matd_dn_pinv(3 * sQ * sP), matd_one(3 * size_QP);
    std::vector<b2_ctx::RedcMeta> redc(size_QP);
    for (size_t j = 0; j < sQ; j++)
        for (size_t i = 0; i < sP; i++) {
            h_pieces(mat_dn[j * sP + i], c->q[j], &matd_dn[3 * (j * sP + i)]);
            h_pieces(mat_dn_pinv[j * sP + i], c->q[j], &matd_dn_pinv[3 * (j * sP + i)]);
        }
    for (size_t j = 0; j < size_QP; j++) {
        h_pieces(1, c->q[j], &matd_one[3 * j]);
        uint64_t inv = 1;  // Newton: inv = q^-1 mod 2^64
        for (int it = 0; it < 6; it++) inv *= 2 - c->q[j] * inv;
        redc[j] = b2_ctx::RedcMeta{c->q[j], (uint64_t)(0 - inv), h_npieces(c->q[j]), 0, 0, {0, 0, 0, 0}, {0, 0, 0, 0}};
        for (int w = 1; w <= 4; w++) {
            const uint64_t cw = h_powmod(2, 21 * w, c->q[j]);
            redc[j].cw[w - 1] = (double)cw;
            redc[j].cwq[w - 1] = (double)cw / (double)c->q[j];
        }
    }
    // the FP64 base conversion needs sum_i(in_i * M_i) < p * 2^64: every digit's primes must sum
    // below 2^64 (true for up to 8 primes of 61 bits, 16 of 60); otherwise the integer kernel runs
    c->bconv_fp = sP <= 8;
    for (size_t s0 = 0; s0 < size_QP && c->bconv_fp; s0 += sP) {
        u128_t sum = 0;
        for (size_t i = s0; i < std::min(s0 + sP, size_QP); i++) sum += c->q[i];
        if (sum >> 64) c->bconv_fp = false;
    }
    auto up = [&](void **dptr, const void *src, size_t bytes) -> cudaError_t {
        cudaError_t e = cudaMalloc(dptr, bytes);
        if (e != cudaSuccess) return e;
        return cudaMemcpy(*dptr, src, bytes, cudaMemcpyHostToDevice);
    };
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = up((void **)&c->d_mod, mods.data(), sizeof(Mod) * size_QP);
    {
        // device copies carry the per-prime encoding (FP64 constants for small primes)
        std::vector<W2> enc(size_QP * N);
        for (int which = 0; which < 2; which++) {
            const std::vector<W2> &src = which ? c->h_itw : c->h_tw;
#pragma omp parallel for schedule(static)
            for (size_t l = 0; l < size_QP; l++) {
                if (c->q[l] < b2::FP_LIMIT) {  // FP64 primes: one double per entry in the front half
                    double *dd = reinterpret_cast<double *>(&enc[l * N]);
                    for (size_t i = 0; i < N; i++) dd[i] = (double)src[l * N + i].w;
                    for (size_t i = N; i < 2 * N; i++) dd[i] = 0.0;
                } else {
                    for (size_t i = 0; i < N; i++) enc[l * N + i] = src[l * N + i];
                }
            }
            if (e == cudaSuccess) e = up(which ? (void **)&c->d_itw : (void **)&c->d_tw, enc.data(), sizeof(W2) * size_QP * N);
        }
        std::vector<W2> fp(2 * size_QP);
        for (size_t l = 0; l < size_QP; l++) {
            fp[2 * l] = h_tw_enc(fin_plain[2 * l].w, c->q[l]);
            fp[2 * l + 1] = h_tw_enc(fin_plain[2 * l + 1].w, c->q[l]);
        }
        if (e == cudaSuccess) e = up((void **)&c->d_fin_plain, fp.data(), sizeof(W2) * 2 * size_QP);
    }
    if (e == cudaSuccess) e = up((void **)&c->d_fin_P, fin_P.data(), sizeof(W2) * 2 * sP);
    if (e == cudaSuccess) e = up((void **)&c->d_Pinv, Pinv.data(), sizeof(W2) * size_QP);
    {
        std::vector<W2> macfin(size_QP);
        for (size_t j = 0; j < size_QP; j++) {
            const uint64_t r64 = (uint64_t)((((unsigned __int128)1) << 64) % c->q[j]);
            macfin[j] = h_w2(j < sQ ? h_mulmod(Pinv[j].w, r64, c->q[j]) : r64, c->q[j]);
        }
        if (e == cudaSuccess) e = up((void **)&c->d_macfin, macfin.data(), sizeof(W2) * size_QP);
    }
    if (e == cudaSuccess) e = up((void **)&c->d_mat_dn, mat_dn.data(), 8 * sQ * sP);
    if (e == cudaSuccess) e = up((void **)&c->d_mat_dn_pinv, mat_dn_pinv.data(), 8 * sQ * sP);
    if (e == cudaSuccess) e = up((void **)&c->d_one, ones.data(), 8 * size_QP);
    if (e == cudaSuccess) e = up((void **)&c->d_matd_dn, matd_dn.data(), 8 * matd_dn.size());
    if (e == cudaSuccess) e = up((void **)&c->d_matd_dn_pinv, matd_dn_pinv.data(), 8 * matd_dn_pinv.size());
    if (e == cudaSuccess) e = up((void **)&c->d_matd_one, matd_one.data(), 8 * matd_one.size());
    if (e == cudaSuccess) e = up((void **)&c->d_redc, redc.data(), sizeof(b2_ctx::RedcMeta) * size_QP);
    if (e != cudaSuccess) {
        b2_ctx_destroy(c);
        return fail((int)e, std::string("ctx_create: table upload failed: ") + cudaGetErrorString(e));
    }
    // B2_NTT_CLUSTER=1 selects the single-launch cluster transforms at N = 2^16. They are bit-exact
    // but measured slower than the two-launch transforms on B200 (register pressure, two CTAs per
    // SM), so they stay opt-in.
    c->h_mat_dn = mat_dn;
    c->h_mat_dn_pinv = mat_dn_pinv;
    {
        // B2_BCONV selects the base-conversion kernel: "tc" (default: tensor cores), "fp" (FP64 pieces), "int" (128-bit integers)
        const char *env_bc = getenv("B2_BCONV");
        const std::string bc = env_bc ? env_bc : "tc";
        bool tc_ok = sP <= 8;
        for (size_t i = 0; i < size_QP; i++) tc_ok = tc_ok && c->q[i] > (1ull << 16);
        c->bconv_tc = tc_ok && bc == "tc";
        c->bconv_int = bc == "int";
        const char *env_wg = getenv("B2_BCONV_WG");
        c->tc_wg = env_wg ? atoi(env_wg) : 4;
        if (c->tc_wg != 1 && c->tc_wg != 2 && c->tc_wg != 4) c->tc_wg = 4;
        const char *env_sld = getenv("B2_BCONV_SERIAL_LD");
        c->tc_serial_ld = env_sld && env_sld[0] == '1';
        const char *env_groups = getenv("B2_BCONV_GROUPS");
        if (env_groups && atoi(env_groups) >= 1 && atoi(env_groups) <= 16) c->tc_max_groups = (uint32_t)atoi(env_groups);
        const char *env_simple = getenv("B2_BCONV_TC_SIMPLE");
        c->tc_simple = env_simple && env_simple[0] == '1';
        if (cudaMalloc((void **)&c->d_err, 4) != cudaSuccess || cudaMemset(c->d_err, 0, 4) != cudaSuccess) {
            b2_ctx_destroy(c);
            return fail(B2_ENOMEM, "ctx_create: cudaMalloc(status word) failed");
        }
        if (c->logN == 16) {
            // per device: the fused row pass stages a key tile next to its exchange buffer (49 KB, above the 48 KB default)
            // <8, 4, 3> = the row-pass configuration of N = 2^16 (PassCfg<8>, asserted where the kernel is launched)
            cudaError_t em = cudaFuncSetAttribute(ntt_fwd_rows_mac<8, 4, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)mac_smem_bytes<8, 4, 3>());
            if (em != cudaSuccess) {
                b2_ctx_destroy(c);
                return fail((int)em, std::string("ctx_create: cudaFuncSetAttribute(ntt_fwd_rows_mac): ") + cudaGetErrorString(em));
            }
        }
        if (c->bconv_tc) {
            // per device: the conversion asks for more dynamic shared memory than it uses (see tc_smem_request)
            cudaError_t ea = cudaFuncSetAttribute(bconv_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_MAX_REQUEST);
            if (ea == cudaSuccess) ea = cudaFuncSetAttribute(bconv_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_MAX_REQUEST);
            if (ea == cudaSuccess) ea = cudaFuncSetAttribute(bconv_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_MAX_REQUEST);
            if (ea == cudaSuccess) ea = cudaFuncSetAttribute(bconv_tc_persist<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_MAX_REQUEST);
            if (ea == cudaSuccess) ea = cudaFuncSetAttribute(bconv_tc_persist<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_MAX_REQUEST);
            if (ea == cudaSuccess) ea = cudaFuncSetAttribute(bconv_tc_persist<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_MAX_REQUEST);
            if (ea != cudaSuccess) {
                b2_ctx_destroy(c);
                return fail((int)ea, std::string("ctx_create: cudaFuncSetAttribute(bconv_tc_kernel): ") + cudaGetErrorString(ea));
            }
        }
    }
    const char *env_cl = getenv("B2_NTT_CLUSTER");
    c->use_cluster = (c->logN == 16) && env_cl && env_cl[0] == '1';
    const char *env_pipe = getenv("B2_NTT_PIPE");
    c->use_pipe = (c->logN == 16) && env_pipe && env_pipe[0] == '1';
    const char *env_mac = getenv("B2_KS_FUSED_IP");
    if (const char *e = getenv("B2_KS_FUSED_WIDE")) c->mac_wide = e[0] != '0' ? 1 : 0;
    if (const char *e = getenv("B2_KS_FUSED_ORDER")) c->mac_interleave = e[0] == '1';
    c->use_mac = (c->logN == 16) && !c->use_cluster && !c->use_pipe && !(env_mac && env_mac[0] == '0');
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, c->device);
    if (c->sm_count < 1) c->sm_count = 148;
    c->plan.resize(sQ + 1);
    for (size_t l = 1; l <= sQ; l++) {
        int rc = build_level(c, l);
        if (rc != B2_OK) {
            b2_ctx_destroy(c);
            return rc;
        }
    }
    *out = c;
    return B2_OK;
}

extern "C" size_t b2_ctx_N(const b2_ctx *c) { return c ? c->N : 0; }
extern "C" size_t b2_ctx_size_Q(const b2_ctx *c) { return c ? c->size_Q : 0; }
extern "C" size_t b2_ctx_size_P(const b2_ctx *c) { return c ? c->size_P : 0; }
extern "C" size_t b2_ctx_beta(const b2_ctx *c, size_t l) { return c ? (l + c->size_P - 1) / c->size_P : 0; }

extern "C" int b2_ctx_get_table(const b2_ctx *c, int which, size_t prime_idx, uint64_t *host_out) {
    if (!c || !host_out || prime_idx >= c->size_QP || which < 0 || which > 3) return fail(B2_EINVAL, "ctx_get_table: bad argument");
    const W2 *t = ((which & 1) ? c->h_itw.data() : c->h_tw.data()) + prime_idx * c->N;
    for (size_t i = 0; i < c->N; i++) host_out[i] = (which & 2) ? t[i].ws : t[i].w;
    return B2_OK;
}

// ------------------------------------------------------------------------------------------------
// transform launchers
// ------------------------------------------------------------------------------------------------
// stage split per polynomial degree: {LOG_A (column pass), LOG_B (row pass)}
template <int LOG_T> struct PassCfg;
// LOG_C: sub-transforms per CTA in the row pass; LOG_CC: columns per CTA in the column pass (2^LOG_CC * 8 bytes is
// the contiguous run a row of the tile covers: 128 bytes, one full line, at LOG_CC = 4)
#ifndef B2_NTT_LOG_CC8
#define B2_NTT_LOG_CC8 3
#endif
// 512-point sub-transforms (the row pass of N = 2^17): 4 + 5 stages, 32 residues per thread in the second group
template <> struct PassCfg<9> { static constexpr int R_STRIDED = 4, R_CONTIG = 5, LOG_C = 2, LOG_CC = 3; };
template <> struct PassCfg<8> { static constexpr int R_STRIDED = 4, R_CONTIG = 4, LOG_C = 3, LOG_CC = B2_NTT_LOG_CC8; };
template <> struct PassCfg<7> { static constexpr int R_STRIDED = 3, R_CONTIG = 4, LOG_C = 4, LOG_CC = 4; };
template <> struct PassCfg<6> { static constexpr int R_STRIDED = 3, R_CONTIG = 3, LOG_C = 4, LOG_CC = 4; };

template <int LOG_T, bool COLS = false>
static constexpr int pass_threads() {
    using P = PassCfg<LOG_T>;
    return (1 << ((COLS ? P::LOG_CC : P::LOG_C) + LOG_T)) >> (P::R_STRIDED > P::R_CONTIG ? P::R_STRIDED : P::R_CONTIG);
}

// grid of a pipelined pass: every CTA gets the same number of tiles (as far as divisibility allows)
static uint32_t pipe_grid(const b2_ctx *c, uint32_t total) {
    const uint32_t slots = (uint32_t)c->sm_count * 6;
    const uint32_t per_cta = (total + slots - 1) / slots;
    return (total + per_cta - 1) / per_cta;
}

// grid of a two-pass transform kernel over `work` tiles and `batch` sets
static dim3 pass_grid(NttArgs &, uint32_t work, uint32_t batch) { return dim3(work, batch); }

template <int LOG_A, int LOG_B, class Epi, int SRC = 0>
static void launch_fwd(const b2_ctx *c, const NttArgs &a, uint32_t njobs, const Epi &epi, cudaStream_t s, uint32_t batch = 1) {
    using A = PassCfg<LOG_A>;
    using B = PassCfg<LOG_B>;
    const uint32_t N = 1u << a.logN;
    if constexpr (LOG_A == 8 && LOG_B == 8 && SRC == 0) {
        if (c->use_pipe) {
            const uint32_t total = njobs * (N >> (LOG_A + A::LOG_C));
            {
                LaunchScope ls(c, s, "ntt_fwd_cols");
                ntt_fwd_pipe<LOG_A, A::R_STRIDED, A::R_CONTIG, A::LOG_C, true, false, EpiStore>
                    <<<pipe_grid(c, total), pass_threads<LOG_A>(), 0, s>>>(a, EpiStore{}, total);  // the pipelined passes keep 8 columns
            }
            NttArgs b = a;
            b.src = a.dst;
            LaunchScope ls(c, s, "ntt_fwd_rows");
            ntt_fwd_pipe<LOG_B, B::R_STRIDED, B::R_CONTIG, B::LOG_C, false, true, Epi><<<pipe_grid(c, total), pass_threads<LOG_B>(), 0, s>>>(b, epi, total);
            return;
        }
    }
    {
        NttArgs a1 = a;
        const dim3 grid = pass_grid(a1, njobs * (N >> (LOG_A + A::LOG_CC)), batch);
        LaunchScope ls(c, s, "ntt_fwd_cols");
        ntt_fwd_pass<LOG_A, A::R_STRIDED, A::R_CONTIG, A::LOG_CC, true, false, EpiStore, SRC><<<grid, pass_threads<LOG_A, true>(), 0, s>>>(a1, EpiStore{});
    }
    NttArgs b = a;
    b.src = a.dst;  // second pass works in place on the first pass's output
    b.src_lm1 = a.dst_lm1, b.src_bs = a.dst_bs;
    const dim3 grid = pass_grid(b, njobs * (N >> (LOG_B + B::LOG_C)), batch);
    LaunchScope ls(c, s, "ntt_fwd_rows");
    ntt_fwd_pass<LOG_B, B::R_STRIDED, B::R_CONTIG, B::LOG_C, false, true, Epi><<<grid, pass_threads<LOG_B>(), 0, s>>>(b, epi);
}

template <int LOG_A, int LOG_B>
static void launch_inv(const b2_ctx *c, const NttArgs &a, uint32_t njobs, cudaStream_t s, uint32_t batch = 1) {
    using A = PassCfg<LOG_A>;
    using B = PassCfg<LOG_B>;
    const uint32_t N = 1u << a.logN;
    if constexpr (LOG_A == 8 && LOG_B == 8) {
        if (c->use_pipe) {
            const uint32_t total = njobs * (N >> (LOG_B + B::LOG_C));
            {
                LaunchScope ls(c, s, "ntt_inv_rows");
                ntt_inv_pipe<LOG_B, B::R_CONTIG, B::R_STRIDED, B::LOG_C, false, false><<<pipe_grid(c, total), pass_threads<LOG_B>(), 0, s>>>(a, total);
            }
            NttArgs b = a;
            b.src = a.dst;
            LaunchScope ls(c, s, "ntt_inv_cols");
            ntt_inv_pipe<LOG_A, A::R_CONTIG, A::R_STRIDED, A::LOG_C, true, true><<<pipe_grid(c, total), pass_threads<LOG_A>(), 0, s>>>(b, total);
            return;
        }
    }
    {
        NttArgs a1 = a;
        const dim3 grid = pass_grid(a1, njobs * (N >> (LOG_B + B::LOG_C)), batch);
        LaunchScope ls(c, s, "ntt_inv_rows");
        ntt_inv_pass<LOG_B, B::R_CONTIG, B::R_STRIDED, B::LOG_C, false, false><<<grid, pass_threads<LOG_B>(), 0, s>>>(a1);
    }
    NttArgs b = a;
    b.src = a.dst;
    b.src_lm1 = a.dst_lm1, b.src_bs = a.dst_bs;
    const dim3 grid = pass_grid(b, njobs * (N >> (LOG_A + A::LOG_CC)), batch);
    LaunchScope ls(c, s, "ntt_inv_cols");
    ntt_inv_pass<LOG_A, A::R_CONTIG, A::R_STRIDED, A::LOG_CC, true, true><<<grid, pass_threads<LOG_A, true>(), 0, s>>>(b);
}

// SRC != 0: the column pass makes limb job.x from slot job.x / src_div of src (words mod src_q) instead of reading it
// A batched launch: `batch` polynomial sets, slot s of set b at s * (lm1 + 1) + b * bs of the source / destination
struct BatchDims {
    uint32_t batch = 1, src_lm1 = 0, src_bs = 0, dst_lm1 = 0, dst_bs = 0;
};

template <class Epi, int SRC = 0>
static int run_fwd(const b2_ctx *c, const uint64_t *src, uint64_t *dst, const Job *jobs, uint32_t njobs, uint32_t first_prime,
                   const Epi &epi, cudaStream_t s, uint32_t period = 0, uint32_t src_div = 0, uint64_t src_q = 0, const BatchDims &bd = BatchDims{}) {
    if (njobs == 0) return B2_OK;
    if (!aligned32(src) || !aligned32(dst) || !epi.aligned()) return fail(B2_EINVAL, "device buffers must be 32-byte aligned (256-bit accesses)");
    NttArgs a{src, dst, jobs, first_prime, (uint32_t)c->logN, c->d_tw, c->d_mod, nullptr, period, src_div, src_q, bd.src_lm1, bd.src_bs, bd.dst_lm1, bd.dst_bs};
    if (bd.batch != 1 && (c->use_cluster || c->use_pipe)) return fail(B2_EINVAL, "batched transforms need the two-pass kernels");
    if (SRC != 0 && (c->use_cluster || src_div == 0)) return fail(B2_EINVAL, "the on-the-fly source needs the two-pass transform");
    if (c->use_cluster) {
        // the attribute belongs to the (function, device) pair; setting it is cheap, so it is set on every launch path
        // rather than remembered per thread (a thread may drive contexts on several devices)
        CUDA_TRY(cudaFuncSetAttribute(ntt_fwd_cluster<Epi>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CL_SMEM));
        LaunchScope ls(c, s, "ntt_fwd_cluster");
        ntt_fwd_cluster<Epi><<<njobs * CL_SIZE, CL_THREADS, CL_SMEM, s>>>(a, epi);
        LAUNCH_CHECK("ntt_fwd_cluster");
        return B2_OK;
    }
    switch (c->logN) {
        case 17: launch_fwd<8, 9, Epi, SRC>(c, a, njobs, epi, s, bd.batch); break;
        case 16: launch_fwd<8, 8, Epi, SRC>(c, a, njobs, epi, s, bd.batch); break;
        case 15: launch_fwd<7, 8, Epi, SRC>(c, a, njobs, epi, s, bd.batch); break;
        case 14: launch_fwd<7, 7, Epi, SRC>(c, a, njobs, epi, s, bd.batch); break;
        case 13: launch_fwd<6, 7, Epi, SRC>(c, a, njobs, epi, s, bd.batch); break;
        case 12: launch_fwd<6, 6, Epi, SRC>(c, a, njobs, epi, s, bd.batch); break;
        default: return fail(B2_ESIZE, "unsupported polynomial degree");
    }
    LAUNCH_CHECK("ntt_fwd_pass");
    return B2_OK;
}

static int run_inv(const b2_ctx *c, const uint64_t *src, uint64_t *dst, const Job *jobs, uint32_t njobs, uint32_t first_prime,
                   const W2 *fin, cudaStream_t s, const BatchDims &bd = BatchDims{}) {
    if (njobs == 0) return B2_OK;
    if (!aligned32(src) || !aligned32(dst)) return fail(B2_EINVAL, "device buffers must be 32-byte aligned (256-bit accesses)");
    NttArgs a{src, dst, jobs, first_prime, (uint32_t)c->logN, c->d_itw, c->d_mod, fin, 0, 0, 0, bd.src_lm1, bd.src_bs, bd.dst_lm1, bd.dst_bs};
    if (bd.batch != 1 && (c->use_cluster || c->use_pipe)) return fail(B2_EINVAL, "batched transforms need the two-pass kernels");
    if (c->use_cluster) {
        CUDA_TRY(cudaFuncSetAttribute(ntt_inv_cluster, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CL_SMEM));
        LaunchScope ls(c, s, "ntt_inv_cluster");
        ntt_inv_cluster<<<njobs * CL_SIZE, CL_THREADS, CL_SMEM, s>>>(a);
        LAUNCH_CHECK("ntt_inv_cluster");
        return B2_OK;
    }
    switch (c->logN) {
        case 17: launch_inv<8, 9>(c, a, njobs, s, bd.batch); break;
        case 16: launch_inv<8, 8>(c, a, njobs, s, bd.batch); break;
        case 15: launch_inv<7, 8>(c, a, njobs, s, bd.batch); break;
        case 14: launch_inv<7, 7>(c, a, njobs, s, bd.batch); break;
        case 13: launch_inv<6, 7>(c, a, njobs, s, bd.batch); break;
        case 12: launch_inv<6, 6>(c, a, njobs, s, bd.batch); break;
        default: return fail(B2_ESIZE, "unsupported polynomial degree");
    }
    LAUNCH_CHECK("ntt_inv_pass");
    return B2_OK;
}

// ------------------------------------------------------------------------------------------------
// base conversion, inner product, elementwise kernels
// ------------------------------------------------------------------------------------------------
// Fast base conversion (src/rns_bconv.cu:143-168, 455-485): for every coefficient n and every output
// prime p_j of the group:  out_j[n] = (sum_i in_i[n] * M[j][i]) mod p_j, the sum kept in 128 bits
// and reduced once. One thread owns two adjacent coefficients, loads their ni inputs once and walks
// all outputs, so the inputs cross HBM once and every store is a coalesced 16-byte write.
// gridDim.y = group (digit of ModUp / polynomial of ModDown). COPY: also copies the group's own
// limbs from `copy_src` (the NTT-form input) into the output buffer (src/rns_bconv.cu:522-528).
struct BconvOut {
    uint64_t q, r0, r1, slot;
};

template <int MAX_NI, bool COPY>
__global__ void __launch_bounds__(128) bconv_kernel(const uint64_t *__restrict__ in, uint64_t *__restrict__ out,
                                                    const uint64_t *__restrict__ copy_src, const BconvGroup *groups,
                                                    const uint2 *outs, const uint64_t *mats, const Mod *mod, uint32_t N) {
    extern __shared__ __align__(16) uint64_t s_raw[];
    const BconvGroup g = groups[blockIdx.y];
    BconvOut *s_out = reinterpret_cast<BconvOut *>(s_raw);          // [n_out]
    uint64_t *s_mat = s_raw + 4 * (size_t)g.n_out;                  // [n_out][ni]
    const uint64_t *mat = mats + g.mat_off;
    for (uint32_t i = threadIdx.x; i < g.n_out * g.ni; i += blockDim.x) s_mat[i] = mat[i];
    for (uint32_t j = threadIdx.x; j < g.n_out; j += blockDim.x) {
        const uint2 o = outs[g.out_begin + j];
        const Mod md = mod[o.y];
        s_out[j] = BconvOut{md.q, md.r0, md.r1, (uint64_t)(g.out_slot_base + o.x)};
    }
    __syncthreads();
    const uint32_t n = 2 * (blockIdx.x * blockDim.x + threadIdx.x);
    if (n >= N) return;
    uint64_t y0[MAX_NI], y1[MAX_NI];
#pragma unroll
    for (int i = 0; i < MAX_NI; i++) {
        if (i < (int)g.ni) {
            ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(in + (size_t)(g.in_slot0 + i) * N + n);
            y0[i] = v.x;
            y1[i] = v.y;
            if (COPY) {
                ulonglong2 cv = *reinterpret_cast<const ulonglong2 *>(copy_src + (size_t)(g.in_slot0 + i) * N + n);
                *reinterpret_cast<ulonglong2 *>(out + (size_t)(g.copy_dst_slot0 + i) * N + n) = cv;
            }
        } else {
            y0[i] = y1[i] = 0;
        }
    }
    auto one = [&](uint32_t j) {
        const BconvOut o = s_out[j];
        const uint64_t *m = s_mat + j * g.ni;
        u128 a0{0, 0}, a1{0, 0};
#pragma unroll
        for (int i = 0; i < MAX_NI; i++) {
            if (i < (int)g.ni) {
                const uint64_t mm = m[i];
                mac128(a0, y0[i], mm);
                mac128(a1, y1[i], mm);
            }
        }
        *reinterpret_cast<ulonglong2 *>(out + o.slot * N + n) =
            make_ulonglong2(barrett128(a0, o.q, o.r0, o.r1), barrett128(a1, o.q, o.r0, o.r1));
    };
    uint32_t j = 0;
    for (; j + 1 < g.n_out; j += 2) {
        one(j);
        one(j + 1);
    }
    if (j < g.n_out) one(j);
}

// FP64 form of the same base conversion. On B200 a 64-bit-result integer multiply issues at a quarter
// of the FP64 FMA rate, so the products are done on 21-bit pieces held as doubles: an input residue
// y = y0 + y1 2^21 + y2 2^42 and a matrix entry m (stored as pieces of m * 2^64 mod p) give nine
// exact products below 2^42; five accumulators collect them by weight (sums stay below 2^48, exact),
// are recombined into one 128-bit integer and Montgomery-reduced (the 2^-64 of the reduction cancels
// the 2^64 folded into the matrix). The result is the same residue the integer kernel produces.
// One coefficient per thread; the inputs live in registers, the matrix pieces in shared memory.
struct BconvMetaS {
    uint64_t p, ninv, slot;
    uint32_t pieces, pad;
    double cw[4], cwq[4];
    double pd, pinv;
};

// y * c mod p in FP64 for |y| < 2^50, c < p < 2^42 (the product of ntt_kernels.cuh's ArithFp)
__device__ __forceinline__ double fp_mulmod(double y, double c, double cq, double p) {
    const double h = __dmul_rn(y, c);
    const double l = __fma_rn(y, c, -h);
    const double k = __dsub_rn(__fma_rn(y, cq, b2::FP_MAGIC), b2::FP_MAGIC);
    return __dadd_rn(__fma_rn(-k, p, h), l);
}

static_assert(sizeof(BconvMetaS) == 14 * 8, "shared-memory layout of the base conversion");

template <int INP, int OUTP>
__device__ __forceinline__ void bconv_acc(const double (&yp)[8][3], const double *m, uint32_t ni, double (&A)[5]) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        if (i < (int)ni) {
#pragma unroll
            for (int b = 0; b < OUTP; b++) {
                const double mb = m[3 * i + b];
#pragma unroll
                for (int a = 0; a < INP; a++) A[a + b] = __fma_rn(yp[i][a], mb, A[a + b]);
            }
        }
    }
}

template <int INP, bool COPY>
__device__ __forceinline__ void bconv_fp_body(const uint64_t *__restrict__ in, uint64_t *__restrict__ out, const uint64_t *__restrict__ copy_src,
                                              const BconvGroup &g, const BconvMetaS *s_meta, const double *s_m, uint32_t N, uint32_t n) {
    double yp[8][3];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        if (i < (int)g.ni) {
            const uint64_t y = in[(size_t)(g.in_slot0 + i) * N + n];
            if (COPY) out[(size_t)(g.copy_dst_slot0 + i) * N + n] = copy_src[(size_t)(g.in_slot0 + i) * N + n];
            const uint64_t magic = 0x4330000000000000ull;
            yp[i][0] = __dsub_rn(__longlong_as_double((long long)((y & 0x1FFFFF) | magic)), 4503599627370496.0);
            yp[i][1] = __dsub_rn(__longlong_as_double((long long)(((y >> 21) & 0x1FFFFF) | magic)), 4503599627370496.0);
            yp[i][2] = INP == 3 ? __dsub_rn(__longlong_as_double((long long)((y >> 42) | magic)), 4503599627370496.0) : 0.0;
        } else {
            yp[i][0] = yp[i][1] = yp[i][2] = 0.0;
        }
    }
    for (uint32_t j = 0; j < g.n_out; j++) {
        const BconvMetaS o = s_meta[j];
        const double *m = s_m + 3 * (size_t)j * g.ni;
        double A[5] = {0.0, 0.0, 0.0, 0.0, 0.0};
        if (o.pieces == 2) {
            // small output prime: sum_w A_w 2^(21 w) mod p entirely in FP64 (A_w exact, below 2^48)
            bconv_acc<INP, 2>(yp, m, g.ni, A);
            const double pd = o.pd, pinv = o.pinv;
            double r = A[0];
#pragma unroll
            for (int w = 1; w <= INP; w++) r = __dadd_rn(r, fp_mulmod(A[w], o.cw[w - 1], o.cwq[w - 1], pd));
            r = __fma_rn(-__dsub_rn(__fma_rn(r, pinv, b2::FP_MAGIC), b2::FP_MAGIC), pd, r);
            if (r < 0.0) r = __dadd_rn(r, pd);
            out[o.slot * N + n] = (uint64_t)__double_as_longlong(__dadd_rn(r, 4503599627370496.0)) & 0x000FFFFFFFFFFFFFull;
            continue;
        }
        bconv_acc<INP, 3>(yp, m, g.ni, A);
        // exact integers below 2^48 -> one 128-bit value
        unsigned __int128 V = 0;
#pragma unroll
        for (int w = 4; w >= 0; w--) {
            const uint64_t u = (uint64_t)__double_as_longlong(__dadd_rn(A[w], 4503599627370496.0)) & 0x000FFFFFFFFFFFFFull;
            V = (V << 21) + u;
        }
        // Montgomery reduction: (V + m p) / 2^64 with m = V_lo * (-p^-1); V < p 2^64 so the result is < 2p
        const uint64_t vlo = (uint64_t)V, vhi = (uint64_t)(V >> 64);
        const uint64_t mm = vlo * o.ninv;
        uint64_t r = vhi + __umul64hi(mm, o.p) + (vlo != 0 ? 1 : 0);
        r = csub(r, o.p);
        out[o.slot * N + n] = r;
    }
}

template <bool COPY>
__global__ void __launch_bounds__(128) bconv_fp_kernel(const uint64_t *__restrict__ in, uint64_t *__restrict__ out,
                                                       const uint64_t *__restrict__ copy_src, const BconvGroup *groups, const uint2 *outs,
                                                       const double *matd, const b2_ctx::RedcMeta *redc, uint32_t N) {
    extern __shared__ __align__(16) uint64_t s_raw[];
    const BconvGroup g = groups[blockIdx.y];
    BconvMetaS *s_meta = reinterpret_cast<BconvMetaS *>(s_raw);                      // [n_out]
    double *s_m = reinterpret_cast<double *>(s_raw + 14 * (size_t)g.n_out);          // [n_out][ni][3]
    const double *mat = matd + 3 * (size_t)g.mat_off;
    for (uint32_t i = threadIdx.x; i < 3 * g.n_out * g.ni; i += blockDim.x) s_m[i] = mat[i];
    for (uint32_t j = threadIdx.x; j < g.n_out; j += blockDim.x) {
        const uint2 o = outs[g.out_begin + j];
        const b2_ctx::RedcMeta r = redc[o.y];
        BconvMetaS m{r.p, r.ninv, (uint64_t)(g.out_slot_base + o.x), r.pieces, 0, {}, {}, (double)r.p, 1.0 / (double)r.p};
        for (int w = 0; w < 4; w++) {
            m.cw[w] = r.cw[w];
            m.cwq[w] = r.cwq[w];
        }
        s_meta[j] = m;
    }
    __syncthreads();
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    if (g.in_pieces == 2) bconv_fp_body<2, COPY>(in, out, copy_src, g, s_meta, s_m, N, n);
    else bconv_fp_body<3, COPY>(in, out, copy_src, g, s_meta, s_m, N, n);
}

struct EvkPtrs {
    const uint64_t *p[64];
};

// A batch of inner products in one launch (FUSED form): blockIdx.y = set b. Digits, the NTT-form input and the ciphertext
// of set b start b * dig_bs / own_bs / ct_bs limbs further; P limb i of polynomial k lands at slot
// (i * p_mul_i + k * p_mul_k) * (p_lm1 + 1) + b * p_bs of the P-limb buffer. One set: {0, 0, 0, 1, alpha, 0, 0}.
struct IpBatch {
    uint32_t dig_bs, own_bs, ct_bs, p_mul_i, p_mul_k, p_lm1, p_bs;
};

// Key-switch inner product (src/eval_key_switch.cu:175-230): for logical limb t (physical prime pp)
//   acc[k][t][n] = (sum_d digits[d][t][n] * evk[d][k][pp][n]) mod q_pp,   k = 0, 1
// accumulated in 128 bits and reduced once. Pure streaming: two coefficients per thread, 16-byte
// loads, every load of a thread issued before the first multiply.
// FUSED = false: out[k][t] = acc (the reference's cx buffer, [2][l+alpha][N]).
// FUSED = true (whole key switch): Q limbs go straight into the ciphertext as
//   ct[k][t] += acc * P^-1  and only the P limbs are kept, compactly, in outP [2][alpha][N];
// together with a ModDown matrix that carries P^-1 this equals ct + (acc - delta) * P^-1.
// ACCP (with FUSED): the P limbs are added to what outP already holds, so that several key switches share
// one ModDown ("double hoisting": the Q limbs accumulate in ct anyway).
template <int MAX_BETA, bool FUSED, bool ACCP = false>
__global__ void __launch_bounds__(256) ks_inner_prod_kernel(const uint64_t *__restrict__ digits, const uint64_t *__restrict__ own,
                                                           EvkPtrs evk, uint64_t *__restrict__ out, uint64_t *__restrict__ ct,
                                                           const W2 *__restrict__ pinv, const Mod *mod, const b2_ctx::RedcMeta *redc,
                                                           uint32_t N, uint32_t l, uint32_t lP, uint32_t size_Q, uint32_t size_QP,
                                                           uint32_t beta, uint4 own_range, const IpBatch ib, const uint32_t *__restrict__ perm) {
    // perm (optional): the digits are read through the NTT-domain permutation of a Galois element, digit[perm[n]] - hoisted
    // rotations, whose permuted copy of the ModUp digits is then never written (src/evaluate.cu:2041-2045 permutes into a buffer)
    // own_range = (first Q limb, number of Q limbs, first P limb, number of P limbs) this launch
    // covers: everything on one GPU, the rank's slice under RNS-limb sharding
    // The sets are the slow grid dimension: with the sets fastest (the CTAs that read one piece of the key next to one another) this
    // kernel ran 13 % slower on B200.
    digits += (size_t)blockIdx.y * ib.dig_bs * N;
    if (own) own += (size_t)blockIdx.y * ib.own_bs * N;
    if (FUSED) ct += (size_t)blockIdx.y * ib.ct_bs * N;
    const size_t jdx = 2 * ((size_t)blockIdx.x * blockDim.x + threadIdx.x);
    if (jdx >= (size_t)(own_range.y + own_range.w) * N) return;
    const uint32_t jl = (uint32_t)(jdx / N), n = (uint32_t)(jdx % N);
    const uint32_t t = jl < own_range.y ? own_range.x + jl : l + own_range.z + (jl - own_range.y);
    const size_t idx = (size_t)t * N + n;
    const uint32_t pp = t < l ? t : size_Q + (t - l);
    const Mod md = mod[pp];
    // `own` (optional): the NTT-form input of ModUp; limb t of digit t / alpha is that input itself
    // (src/rns_bconv.cu:522-528), so the digit buffer need not hold a copy of it
    const uint32_t own_d = (own && t < l) ? t / (lP - l) : 0xFFFFFFFFu;
    const uint2 p2 = perm ? *reinterpret_cast<const uint2 *>(perm + n) : make_uint2(0, 0);
    if (md.q < b2::FP_LIMIT) {
        // Small prime (uniform over the block): digits and key words are below 2^41, so each product
        // is four exact FP64 FMAs on 21-bit pieces instead of five wide integer multiplies, and the
        // reduction of sum_w A_w 2^(21 w) stays in FP64 too. Same residues as the integer path.
        const b2_ctx::RedcMeta rm = redc[pp];
        const double qd = (double)md.q, qinv = 1.0 / qd;
        double A[4][3];
#pragma unroll
        for (int o = 0; o < 4; o++) A[o][0] = A[o][1] = A[o][2] = 0.0;
        auto lo = [](uint64_t v) { return __dsub_rn(__longlong_as_double((long long)((v & 0x1FFFFF) | 0x4330000000000000ull)), 4503599627370496.0); };
        auto hi = [](uint64_t v) { return __dsub_rn(__longlong_as_double((long long)((v >> 21) | 0x4330000000000000ull)), 4503599627370496.0); };
        for (uint32_t d = 0; d < beta; d++) {
            ulonglong2 x;
            if (perm) {
                const uint64_t *dg = digits + ((size_t)d * lP + t) * N;
                x = make_ulonglong2(dg[p2.x], dg[p2.y]);
            } else {
                x = (d == own_d) ? *reinterpret_cast<const ulonglong2 *>(own + (size_t)t * N + n)
                                 : *reinterpret_cast<const ulonglong2 *>(digits + ((size_t)d * lP + t) * N + n);
            }
            const uint64_t *e = evk.p[d] + (size_t)pp * N + n;
            const ulonglong2 e0 = __ldcs(reinterpret_cast<const ulonglong2 *>(e));
            const ulonglong2 e1 = __ldcs(reinterpret_cast<const ulonglong2 *>(e + (size_t)size_QP * N));
            const double xl[2] = {lo(x.x), lo(x.y)}, xh[2] = {hi(x.x), hi(x.y)};
            const double el[4] = {lo(e0.x), lo(e0.y), lo(e1.x), lo(e1.y)}, eh[4] = {hi(e0.x), hi(e0.y), hi(e1.x), hi(e1.y)};
#pragma unroll
            for (int o = 0; o < 4; o++) {
                const int c = o & 1;
                A[o][0] = __fma_rn(xl[c], el[o], A[o][0]);
                A[o][1] = __fma_rn(xl[c], eh[o], __fma_rn(xh[c], el[o], A[o][1]));
                A[o][2] = __fma_rn(xh[c], eh[o], A[o][2]);
            }
        }
        uint64_t r[4];
        const W2 pi = FUSED && t < l ? pinv[pp] : W2{0, 0};
        const double pid = (double)pi.w, piq = __dmul_rn(pid, qinv);
#pragma unroll
        for (int o = 0; o < 4; o++) {
            double v = __dadd_rn(A[o][0], __dadd_rn(fp_mulmod(A[o][1], rm.cw[0], rm.cwq[0], qd), fp_mulmod(A[o][2], rm.cw[1], rm.cwq[1], qd)));
            if (FUSED && t < l) v = fp_mulmod(v, pid, piq, qd);          // times P^-1 (|v| < 2^50)
            else v = __fma_rn(-__dsub_rn(__fma_rn(v, qinv, b2::FP_MAGIC), b2::FP_MAGIC), qd, v);
            if (v < 0.0) v = __dadd_rn(v, qd);
            r[o] = (uint64_t)__double_as_longlong(__dadd_rn(v, 4503599627370496.0)) & 0x000FFFFFFFFFFFFFull;
        }
        if (!FUSED) {
            *reinterpret_cast<ulonglong2 *>(out + idx) = make_ulonglong2(r[0], r[1]);
            *reinterpret_cast<ulonglong2 *>(out + (size_t)lP * N + idx) = make_ulonglong2(r[2], r[3]);
        } else if (t < l) {
            uint64_t *c0 = ct + idx, *c1 = ct + (size_t)l * N + idx;
            const ulonglong2 u0 = *reinterpret_cast<const ulonglong2 *>(c0), u1 = *reinterpret_cast<const ulonglong2 *>(c1);
            *reinterpret_cast<ulonglong2 *>(c0) = make_ulonglong2(add_mod(u0.x, r[0], md.q), add_mod(u0.y, r[1], md.q));
            *reinterpret_cast<ulonglong2 *>(c1) = make_ulonglong2(add_mod(u1.x, r[2], md.q), add_mod(u1.y, r[3], md.q));
        } else {
            const size_t o = ((size_t)(t - l) * ib.p_mul_i * (ib.p_lm1 + 1) + (size_t)blockIdx.y * ib.p_bs) * N + n;
            const size_t o1 = o + (size_t)ib.p_mul_k * (ib.p_lm1 + 1) * N;
            if (ACCP) {
                const ulonglong2 p0 = *reinterpret_cast<const ulonglong2 *>(out + o), p1 = *reinterpret_cast<const ulonglong2 *>(out + o1);
                r[0] = add_mod(r[0], p0.x, md.q), r[1] = add_mod(r[1], p0.y, md.q), r[2] = add_mod(r[2], p1.x, md.q), r[3] = add_mod(r[3], p1.y, md.q);
            }
            *reinterpret_cast<ulonglong2 *>(out + o) = make_ulonglong2(r[0], r[1]);
            *reinterpret_cast<ulonglong2 *>(out + o1) = make_ulonglong2(r[2], r[3]);
        }
        return;
    }
    u128 a00{0, 0}, a01{0, 0}, a10{0, 0}, a11{0, 0};
    for (uint32_t d0 = 0; d0 < beta; d0 += MAX_BETA) {
        ulonglong2 x[MAX_BETA], e0[MAX_BETA], e1[MAX_BETA];
#pragma unroll
        for (int i = 0; i < MAX_BETA; i++) {
            if (d0 + i < beta) {
                if (perm) {
                    const uint64_t *dg = digits + ((size_t)(d0 + i) * lP + t) * N;
                    x[i] = make_ulonglong2(dg[p2.x], dg[p2.y]);
                } else {
                    x[i] = (d0 + i == own_d) ? *reinterpret_cast<const ulonglong2 *>(own + (size_t)t * N + n)
                                             : *reinterpret_cast<const ulonglong2 *>(digits + ((size_t)(d0 + i) * lP + t) * N + n);
                }
                const uint64_t *e = evk.p[d0 + i] + (size_t)pp * N + n;
                e0[i] = __ldcs(reinterpret_cast<const ulonglong2 *>(e));
                e1[i] = __ldcs(reinterpret_cast<const ulonglong2 *>(e + (size_t)size_QP * N));
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_BETA; i++) {
            if (d0 + i < beta) {
                mac128(a00, x[i].x, e0[i].x);
                mac128(a01, x[i].y, e0[i].y);
                mac128(a10, x[i].x, e1[i].x);
                mac128(a11, x[i].y, e1[i].y);
            }
        }
    }
    uint64_t r00 = barrett128(a00, md.q, md.r0, md.r1), r01 = barrett128(a01, md.q, md.r0, md.r1);
    uint64_t r10 = barrett128(a10, md.q, md.r0, md.r1), r11 = barrett128(a11, md.q, md.r0, md.r1);
    if (!FUSED) {
        *reinterpret_cast<ulonglong2 *>(out + idx) = make_ulonglong2(r00, r01);
        *reinterpret_cast<ulonglong2 *>(out + (size_t)lP * N + idx) = make_ulonglong2(r10, r11);
    } else if (t < l) {
        const W2 pi = pinv[pp];
        uint64_t *c0 = ct + idx, *c1 = ct + (size_t)l * N + idx;
        const ulonglong2 u0 = *reinterpret_cast<const ulonglong2 *>(c0), u1 = *reinterpret_cast<const ulonglong2 *>(c1);
        *reinterpret_cast<ulonglong2 *>(c0) =
            make_ulonglong2(add_mod(u0.x, mul_shoup(r00, pi, md.q), md.q), add_mod(u0.y, mul_shoup(r01, pi, md.q), md.q));
        *reinterpret_cast<ulonglong2 *>(c1) =
            make_ulonglong2(add_mod(u1.x, mul_shoup(r10, pi, md.q), md.q), add_mod(u1.y, mul_shoup(r11, pi, md.q), md.q));
    } else {
        const size_t o = ((size_t)(t - l) * ib.p_mul_i * (ib.p_lm1 + 1) + (size_t)blockIdx.y * ib.p_bs) * N + n;
        const size_t o1 = o + (size_t)ib.p_mul_k * (ib.p_lm1 + 1) * N;
        if (ACCP) {
            const ulonglong2 p0 = *reinterpret_cast<const ulonglong2 *>(out + o), p1 = *reinterpret_cast<const ulonglong2 *>(out + o1);
            r00 = add_mod(r00, p0.x, md.q), r01 = add_mod(r01, p0.y, md.q), r10 = add_mod(r10, p1.x, md.q), r11 = add_mod(r11, p1.y, md.q);
        }
        *reinterpret_cast<ulonglong2 *>(out + o) = make_ulonglong2(r00, r01);
        *reinterpret_cast<ulonglong2 *>(out + o1) = make_ulonglong2(r10, r11);
    }
}

// HMult tensor product (src/polymath.cu:463-498): d0 = a0 b0, d2 = a1 b1, d1 = (a0+a1)(b0+b1) - d0 - d2
// d0, d1 go to out[0..2S), d2 to out2[0..S): the relinearising caller keeps d2 in scratch and the rest in its result
// A batch in one launch: blockIdx.y = pair b, whose operands, result and d2 start b * bs.x / .y / .z / .w limbs further.
__global__ void __launch_bounds__(256) tensor_mul_kernel(const uint64_t *__restrict__ a, const uint64_t *__restrict__ b, uint64_t *__restrict__ out,
                                                        uint64_t *__restrict__ out2, const Mod *mod, uint32_t N, uint32_t l, uint4 bs) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t S = (size_t)l * N;
    if (idx >= S) return;
    a += (size_t)blockIdx.y * bs.x * N, b += (size_t)blockIdx.y * bs.y * N, out += (size_t)blockIdx.y * bs.z * N, out2 += (size_t)blockIdx.y * bs.w * N;
    const Mod md = mod[idx / N];
    const uint64_t q = md.q;
    const uint64_t a0 = a[idx], a1 = a[S + idx], b0 = b[idx], b1 = b[S + idx];
    u128 p{0, 0};
    mac128(p, a0, b0);
    const uint64_t d0 = barrett128(p, q, md.r0, md.r1);
    p = u128{0, 0};
    mac128(p, a1, b1);
    const uint64_t d2 = barrett128(p, q, md.r0, md.r1);
    p = u128{0, 0};
    mac128(p, add_mod(a0, a1, q), add_mod(b0, b1, q));
    const uint64_t d1 = barrett128(p, q, md.r0, md.r1);
    out[idx] = d0;
    out[S + idx] = sub_mod(sub_mod(d1, d0, q), d2, q);
    out2[idx] = d2;
}

// src/polymath.cu:17-180
// `period` limbs per polynomial: limb t of the buffer uses prime t % period, so one launch covers a whole
// ciphertext. b_wrap: the second operand is one polynomial shared by all (a plaintext).
__global__ void __launch_bounds__(256) poly_op_kernel(int op, const uint64_t *a, const uint64_t *b, uint64_t *out, const Mod *mod,
                                                     uint32_t N, uint32_t n_limbs, uint32_t period, int b_wrap) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_limbs * N) return;
    const Mod md = mod[(idx / N) % period];
    const uint64_t q = md.q, x = a[idx];
    const size_t bi = b_wrap ? idx % ((size_t)period * N) : idx;
    uint64_t r;
    if (op == 0) r = add_mod(x, b[bi], q);
    else if (op == 1) r = sub_mod(x, b[bi], q);
    else if (op == 2) {
        u128 p{0, 0};
        mac128(p, x, b[bi]);
        r = barrett128(p, q, md.r0, md.r1);
    } else r = x ? q - x : 0;
    out[idx] = r;
}

// Per-limb integer constants (src/bootstrap.cu:1535-1565, multiply_scalar_per_tower_kernel; adding
// a constant polynomial c to NTT-form data adds c to every value of the limb).
struct ScalarTab { uint64_t v[64]; };
__global__ void __launch_bounds__(256) poly_scalar_kernel(int op, const uint64_t *a, ScalarTab tab, uint64_t *out, const Mod *mod,
                                                        uint32_t N, uint32_t n_limbs, uint32_t period) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_limbs * N) return;
    const uint32_t limb = (uint32_t)((idx / N) % period);
    const Mod md = mod[limb];
    const uint64_t q = md.q, x = a[idx], s = tab.v[limb];
    uint64_t r;
    if (op == 0) r = add_mod(x, s, q);
    else {
        u128 p{0, 0};
        mac128(p, x, s);
        r = barrett128(p, q, md.r0, md.r1);
    }
    out[idx] = r;
}

// NTT-domain automorphism (src/galois.cu:11-18): dst[l][i] = src[l][perm[i]].
// Optional second operand pair so that c0 and c1 (or several digit buffers) go in one launch.
__global__ void __launch_bounds__(256) galois_gather_kernel(const uint64_t *__restrict__ src, uint64_t *__restrict__ dst,
                                                           const uint32_t *__restrict__ perm, uint32_t N, uint32_t n_limbs) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_limbs * N) return;
    const size_t limb = idx / N;
    dst[idx] = src[limb * N + perm[idx % N]];
}

// The automorphism of a ciphertext (c0, c1) as a rotation needs it: perm(c0) goes straight into the result (added to it
// when ACC: rotations that are summed), perm(c1) into the scratch the key switch reads. limbs [0, l) are c0, [l, 2l) c1.
template <bool ACC>
__global__ void __launch_bounds__(256) galois_split_kernel(const uint64_t *__restrict__ src, uint64_t *__restrict__ dst0, uint64_t *__restrict__ dst1,
                                                          const uint32_t *__restrict__ perm, const Mod *mod, uint32_t N, uint32_t l) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t S = (size_t)l * N;
    if (idx >= 2 * S) return;
    const size_t limb = idx / N;
    const uint64_t v = src[limb * N + perm[idx % N]];
    if (limb >= l) {
        dst1[idx - S] = v;
    } else if (ACC) {
        dst0[idx] = add_mod(dst0[idx], v, mod[limb].q);
    } else {
        dst0[idx] = v;
    }
}

// Single-chain plaintext expansion (src/bootstrap.cu:660-686, light_pt_expand_per_tower_kernel):
// one signed, centred int64 coefficient vector -> its residue in each of n_limbs primes.
__global__ void __launch_bounds__(256) expand_signed_kernel(const int64_t *__restrict__ src, uint64_t *__restrict__ dst, const Mod *mod, uint32_t N,
                                                           uint32_t n_limbs, uint32_t first_prime) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_limbs * N) return;
    const Mod md = mod[first_prime + idx / N];
    const int64_t c = src[idx % N];
    const uint64_t mag = c >= 0 ? (uint64_t)c : (uint64_t)0 - (uint64_t)c;
    u128 v{mag, 0};
    const uint64_t r = barrett128(v, md.q, md.r0, md.r1);
    dst[idx] = (c >= 0 || r == 0) ? r : md.q - r;
}

// Centred remainder of the dropped limb, reduced into every remaining prime: with it the rescale
// rounds to nearest instead of flooring. r: [n_poly][N] coefficient form mod q_last.
__global__ void __launch_bounds__(256) rescale_centre_kernel(const uint64_t *__restrict__ r, uint64_t *__restrict__ out, const Mod *mod, uint32_t N,
                                                            uint32_t n_out, uint32_t n_poly) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_poly * n_out * N) return;
    const uint32_t i = (uint32_t)(idx % N), j = (uint32_t)((idx / N) % n_out), p = (uint32_t)(idx / ((size_t)N * n_out));
    const Mod md = mod[j];
    const uint64_t ql = mod[n_out].q, half = ql >> 1;
    const uint64_t v = r[(size_t)p * N + i];
    uint64_t d = barrett64(v, md.q, md.r1);
    if (v > half) d = sub_mod(d, barrett64(ql, md.q, md.r1), md.q);  // v - q_last, the negative representative
    out[idx] = d;
}

// out = sum_t x_t * s_t (+ c on polynomial 0): per-limb integer weights, one reduction per value. The terms may
// sit at higher levels than the output (more limbs per polynomial): lt[t] is term t's limb count.
#define B2_LINCOMB_MAX_TERMS 8
#define B2_LINCOMB_MAX_LIMBS 32
struct LincombArgs {
    const uint64_t *x[B2_LINCOMB_MAX_TERMS];
    uint32_t lt[B2_LINCOMB_MAX_TERMS];
    uint64_t s[B2_LINCOMB_MAX_TERMS][B2_LINCOMB_MAX_LIMBS];
    uint64_t c[B2_LINCOMB_MAX_LIMBS];
};
__global__ void __launch_bounds__(256) lincomb_kernel(const __grid_constant__ LincombArgs a, uint64_t *out, const Mod *mod, uint32_t N, uint32_t l,
                                                     uint32_t n_poly, uint32_t n_terms) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_poly * l * N) return;
    const uint32_t i = (uint32_t)(idx % N), limb = (uint32_t)((idx / N) % l), p = (uint32_t)(idx / ((size_t)N * l));
    const Mod md = mod[limb];
    u128 acc{p == 0 ? a.c[limb] : 0, 0};
    for (uint32_t t = 0; t < n_terms; t++) mac128(acc, a.x[t][((size_t)p * a.lt[t] + limb) * N + i], a.s[t][limb]);
    out[idx] = barrett128(acc, md.q, md.r0, md.r1);
}

// M signed coefficient vectors at once: src [M][N] -> dst [M][l][N] (limb j of every polynomial on prime j)
__global__ void __launch_bounds__(256) expand_signed_batch_kernel(const int64_t *__restrict__ src, uint64_t *__restrict__ dst, const Mod *mod, uint32_t N,
                                                                 uint32_t l, uint32_t M) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)M * l * N) return;
    const uint32_t i = (uint32_t)(idx % N), limb = (uint32_t)((idx / N) % l), m = (uint32_t)(idx / ((size_t)N * l));
    const Mod md = mod[limb];
    const int64_t c = src[(size_t)m * N + i];
    const uint64_t mag = c >= 0 ? (uint64_t)c : (uint64_t)0 - (uint64_t)c;
    u128 v{mag, 0};
    const uint64_t r = barrett128(v, md.q, md.r0, md.r1);
    dst[idx] = (c >= 0 || r == 0) ? r : md.q - r;
}

struct MacPtrs {
    const uint64_t *const *pts;
    const uint64_t *const *babies;
};

// BSGS giant-step multiply-accumulate (src/bsgs.cu:51-96): out_k = sum_b pt_b (.) baby_b[k].
// The reference reduces after every term; the sum of canonical products is the same residue.
__global__ void __launch_bounds__(256) bsgs_mac_kernel(const uint64_t *const *pts, const uint64_t *const *babies, uint64_t *out, const Mod *mod,
                                                      uint32_t N, uint32_t l, uint32_t M) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t S = (size_t)l * N;
    if (idx >= S) return;
    const Mod md = mod[idx / N];
    u128 a0{0, 0}, a1{0, 0};
    uint32_t pending = 0;
    uint64_t r0 = 0, r1 = 0;
    for (uint32_t b = 0; b < M; b++) {
        const uint64_t p = pts[b][idx];
        mac128(a0, p, babies[b][idx]);
        mac128(a1, p, babies[b][S + idx]);
        if (++pending == 32) {  // 32 products of two 61-bit values stay below 2^128
            a0 = u128{barrett128(a0, md.q, md.r0, md.r1), 0};
            a1 = u128{barrett128(a1, md.q, md.r0, md.r1), 0};
            pending = 1;
        }
    }
    r0 = barrett128(a0, md.q, md.r0, md.r1);
    r1 = barrett128(a1, md.q, md.r0, md.r1);
    out[idx] = r0;
    out[S + idx] = r1;
}

// Up to four giants at once: every baby value is loaded once and multiplied into each giant's own plaintext, so the
// babies (two thirds of the bytes of the single-giant kernel) cross HBM once per group instead of once per giant.
// pts[g * M + b] may be null: that giant has no diagonal for baby b.
template <int G>
__global__ void __launch_bounds__(256) bsgs_mac_multi_kernel(const uint64_t *const *pts, const uint64_t *const *babies, uint64_t *const *outs,
                                                            const Mod *mod, uint32_t N, uint32_t l, uint32_t M, uint32_t n_g) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t S = (size_t)l * N;
    if (idx >= S) return;
    const Mod md = mod[idx / N];
    u128 a[G][2];
#pragma unroll
    for (int g = 0; g < G; g++) a[g][0] = a[g][1] = u128{0, 0};
    uint32_t pending = 0;
    for (uint32_t b = 0; b < M; b++) {
        const uint64_t *bb = babies[b];
        const uint64_t y0 = bb[idx], y1 = bb[S + idx];
#pragma unroll
        for (int g = 0; g < G; g++) {
            const uint64_t *pp = g < (int)n_g ? pts[(size_t)g * M + b] : nullptr;
            if (pp) {
                const uint64_t p = pp[idx];
                mac128(a[g][0], p, y0);
                mac128(a[g][1], p, y1);
            }
        }
        if (++pending == 32) {  // 32 products of two 61-bit values stay below 2^128
#pragma unroll
            for (int g = 0; g < G; g++) {
                a[g][0] = u128{barrett128(a[g][0], md.q, md.r0, md.r1), 0};
                a[g][1] = u128{barrett128(a[g][1], md.q, md.r0, md.r1), 0};
            }
            pending = 1;
        }
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (g < (int)n_g) {
            uint64_t *o = outs[g];
            o[idx] = barrett128(a[g][0], md.q, md.r0, md.r1);
            o[S + idx] = barrett128(a[g][1], md.q, md.r0, md.r1);
        }
    }
}

// Shared memory a conversion CTA asks for: what it uses, or enough that no more CTAs fit on an SM (228 KB) than its
// 512 TMEM columns can serve, whichever is larger - so tcgen05.alloc finds its columns free and never waits.
static uint32_t tc_smem_request(uint32_t alloc_cols, uint32_t used) {
    const uint32_t fit = 512 / alloc_cols;
    return std::max(used, TC_SM_SMEM / (fit + 1));
}

// n_jobs: how many of the set's jobs to run (ModDown of one polynomial runs the first half)
static int run_bconv_tc(const b2_ctx *c, bool copy, const uint64_t *in, uint64_t *out, const uint64_t *copy_src, const TcSet &tc, uint32_t n_jobs,
                        cudaStream_t s, const TcBatch *tbp = nullptr) {
    const uint32_t N = (uint32_t)c->N;
    if (n_jobs == 0) return B2_OK;
    if (copy && !copy_src) return fail(B2_EINVAL, "base conversion: missing copy source");
    TcBatch tb = tbp ? *tbp : TcBatch{1, 0, 0, 0, 0, 0};
    tb.serial_ld = c->tc_serial_ld ? 1u : 0u;
    if (tb.batch != 1 && (copy || c->tc_simple)) return fail(B2_EINVAL, "a batched base conversion runs on the persistent kernel, without the own-limb copy");
    LaunchScope ls(c, s, "bconv");
    // without the copy the jobs' copy slots are ignored by handing the kernel a null source
    const uint64_t *cs = copy ? copy_src : nullptr;
    if (c->tc_simple) {
        const dim3 grid(N / 128, n_jobs);
        const uint32_t smem = tc_smem_request(tc.max_alloc, TC_SMEM_BYTES);
        switch (c->tc_wg) {
            case 1: bconv_tc_kernel<1><<<grid, 128, smem, s>>>(in, out, cs, tc.jobs, tc.groups, tc.images, N, c->d_err); break;
            case 4: bconv_tc_kernel<4><<<grid, 512, smem, s>>>(in, out, cs, tc.jobs, tc.groups, tc.images, N, c->d_err); break;
            default: bconv_tc_kernel<2><<<grid, 256, smem, s>>>(in, out, cs, tc.jobs, tc.groups, tc.images, N, c->d_err); break;
        }
        LAUNCH_CHECK("bconv_tc_kernel");
        return B2_OK;
    }
    // persistent CTAs: as many as stay resident (TMEM columns, threads), each walking its share of the (job, tile) items
    const uint32_t threads = 128u * (uint32_t)c->tc_wg;
    const uint32_t fit = std::min(512u / tc.max_alloc, 2048u / threads);
    const uint32_t total = n_jobs * (N / 128) * tb.batch;
    const uint32_t grid = std::min(total, fit * (uint32_t)c->sm_count);
    const uint32_t smem = tc_smem_request(tc.max_alloc, TCP_SMEM_BYTES);
    switch (c->tc_wg) {
        case 1: bconv_tc_persist<1><<<grid, 128, smem, s>>>(in, out, cs, tc.jobs, tc.groups, tc.images, N, n_jobs, tc.max_alloc, c->d_err, tb); break;
        case 2: bconv_tc_persist<2><<<grid, 256, smem, s>>>(in, out, cs, tc.jobs, tc.groups, tc.images, N, n_jobs, tc.max_alloc, c->d_err, tb); break;
        default: bconv_tc_persist<4><<<grid, 512, smem, s>>>(in, out, cs, tc.jobs, tc.groups, tc.images, N, n_jobs, tc.max_alloc, c->d_err, tb); break;
    }
    LAUNCH_CHECK("bconv_tc_persist");
    return B2_OK;
}

static int run_bconv(const b2_ctx *c, bool copy, const uint64_t *in, uint64_t *out, const uint64_t *copy_src, const BconvGroup *groups,
                     uint32_t n_groups, const uint2 *outs, const uint64_t *mats, const double *matd, uint32_t max_ni, uint32_t max_out,
                     bool in3, cudaStream_t s, const TcSet *tc = nullptr, uint32_t tc_jobs = 0) {
    const uint32_t N = (uint32_t)c->N;
    if (max_ni > 16) return fail(B2_ESIZE, "special_modulus_size above 16 is not built");
    if (c->bconv_tc && tc && tc->jobs) return run_bconv_tc(c, copy, in, out, copy_src, *tc, tc_jobs ? tc_jobs : tc->n_jobs, s);
    LaunchScope ls(c, s, "bconv");
    if (c->bconv_fp && matd && !c->bconv_int) {
        dim3 grid(N / 128, n_groups);
        const size_t smem = (size_t)max_out * sizeof(BconvMetaS) + (size_t)max_out * 24 * 8;
        (void)in3;
        if (copy) bconv_fp_kernel<true><<<grid, 128, smem, s>>>(in, out, copy_src, groups, outs, matd, c->d_redc, N);
        else bconv_fp_kernel<false><<<grid, 128, smem, s>>>(in, out, copy_src, groups, outs, matd, c->d_redc, N);
        LAUNCH_CHECK("bconv_fp_kernel");
        return B2_OK;
    }
    dim3 grid(N / 2 / 128, n_groups);
    const size_t smem = ((size_t)max_ni + 4) * max_out * 8;
    if (copy) {
        if (max_ni <= 8) bconv_kernel<8, true><<<grid, 128, smem, s>>>(in, out, copy_src, groups, outs, mats, c->d_mod, N);
        else bconv_kernel<16, true><<<grid, 128, smem, s>>>(in, out, copy_src, groups, outs, mats, c->d_mod, N);
    } else {
        if (max_ni <= 8) bconv_kernel<8, false><<<grid, 128, smem, s>>>(in, out, copy_src, groups, outs, mats, c->d_mod, N);
        else bconv_kernel<16, false><<<grid, 128, smem, s>>>(in, out, copy_src, groups, outs, mats, c->d_mod, N);
    }
    LAUNCH_CHECK("bconv_kernel");
    return B2_OK;
}

// ------------------------------------------------------------------------------------------------
// C ABI: operations
// ------------------------------------------------------------------------------------------------
#define CHECK_CTX(c)                                                       \
    if (!(c)) return fail(B2_EINVAL, "null context");                      \
    CUDA_TRY(cudaSetDevice((c)->device));
#define CHECK_LEVEL(c, l)                                                                          \
    if ((l) < 1 || (l) > (c)->size_Q) return fail(B2_EINVAL, "size_Ql must be in [1, size_Q]");

static inline size_t limb_bytes(const b2_ctx *c) { return c->N * 8; }

extern "C" size_t b2_workspace_bytes(const b2_ctx *c, int op, size_t l) {
    if (!c || l < 1 || l > c->size_Q) return 0;
    const size_t a = c->size_P, beta = (l + a - 1) / a, lP = l + a, L = limb_bytes(c);
    switch (op) {
        case B2_OP_MODUP: return l * L;
        case B2_OP_MODDOWN: return 3 * l * L;
        case B2_OP_KEYSWITCH: return (l + beta * lP + 2 * lP) * L;
        case B2_OP_RESCALE: return 3 * L;
        case B2_OP_MUL_RELIN: return (l + beta * lP + 2 * lP + 3 * l) * L;
        case B2_OP_ROTATE: return (l + beta * lP + 2 * lP + 2 * l) * L;
        case B2_OP_HOIST: return (l + 2 * beta * lP + 2 * lP + l) * L;
        default: return 0;
    }
}

extern "C" int b2_ntt_forward(b2_ctx *c, uint64_t *d, size_t n_limbs, size_t first_prime, void *stream) {
    CHECK_CTX(c);
    if (!d || first_prime + n_limbs > c->size_QP) return fail(B2_EINVAL, "ntt_forward: limb range outside the modulus chain");
    return run_fwd(c, d, d, nullptr, (uint32_t)n_limbs, (uint32_t)first_prime, EpiStore{}, (cudaStream_t)stream);
}

extern "C" int b2_ntt_inverse(b2_ctx *c, uint64_t *d, size_t n_limbs, size_t first_prime, void *stream) {
    CHECK_CTX(c);
    if (!d || first_prime + n_limbs > c->size_QP) return fail(B2_EINVAL, "ntt_inverse: limb range outside the modulus chain");
    return run_inv(c, d, d, nullptr, (uint32_t)n_limbs, (uint32_t)first_prime, c->d_fin_plain, (cudaStream_t)stream);
}

// ModUp into `out`; `t` = l limbs of scratch for the scaled coefficient form
static int modup_impl(b2_ctx *c, size_t l, const uint64_t *c2, uint64_t *out, uint64_t *t, bool copy_own, cudaStream_t s) {
    const LevelPlan &pl = c->plan[l];
    int rc = run_inv(c, c2, t, pl.jobs_up_intt, (uint32_t)l, 0, pl.fin_up, s);
    if (rc) return rc;
    rc = run_bconv(c, copy_own, t, out, c2, pl.grp_up, pl.beta, pl.outs_up, pl.mat_up, pl.matd_up, (uint32_t)c->size_P, (uint32_t)(l + c->size_P), true, s, &pl.tc_up);
    if (rc) return rc;
    return run_fwd(c, out, out, pl.jobs_up_ntt, pl.n_up_ntt, 0, EpiStore{}, s);
}

extern "C" int b2_modup(b2_ctx *c, size_t l, const uint64_t *d_c2, uint64_t *d_out, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_c2 || !d_out || !d_ws) return fail(B2_EINVAL, "modup: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_MODUP, l)) return fail(B2_EWS, "modup: workspace too small");
    return modup_impl(c, l, d_c2, d_out, (uint64_t *)d_ws, true, (cudaStream_t)stream);
}

// fused = false: out = cx [2][lP][N]. fused = true: Q limbs accumulate into ct, out = [2][alpha][N].
static int inner_prod_impl(b2_ctx *c, size_t l, const uint64_t *digits, const uint64_t *own, const uint64_t *const *evk, size_t n_evk,
                           uint64_t *out, uint64_t *ct, bool fused, cudaStream_t s, const uint4 *range = nullptr, bool acc_p = false,
                           uint32_t batch = 1, const IpBatch *ipb = nullptr, const uint32_t *perm = nullptr) {
    const size_t beta = c->plan[l].beta, lP = l + c->size_P;
    if (perm && own) return fail(B2_EINVAL, "a permuted inner product reads every limb from the digit buffer");
    if (n_evk < beta) return fail(B2_EINVAL, "key has fewer digits than this level needs");
    if (beta > 64) return fail(B2_ESIZE, "more than 64 digits");
    EvkPtrs ep;
    for (size_t d = 0; d < beta; d++) {
        if (!evk[d]) return fail(B2_EINVAL, "null evaluation-key digit");
        ep.p[d] = evk[d];
    }
    const uint4 rg = range ? *range : make_uint4(0, (uint32_t)l, 0, (uint32_t)c->size_P);
    const size_t pairs = (size_t)(rg.y + rg.w) * c->N / 2;
    if (pairs == 0) return B2_OK;
    if (batch != 1 && (!fused || !ipb)) return fail(B2_EINVAL, "a batched inner product runs in the fused form");
    const dim3 grid((unsigned)((pairs + 255) / 256), batch);
    const IpBatch ib = ipb ? *ipb : IpBatch{0, 0, 0, 1, (uint32_t)c->size_P, 0, 0};
    LaunchScope ls(c, s, "ks_inner_prod");
    if (fused && acc_p)
        ks_inner_prod_kernel<3, true, true><<<grid, 256, 0, s>>>(digits, own, ep, out, ct, c->d_Pinv, c->d_mod, c->d_redc, (uint32_t)c->N, (uint32_t)l,
                                                               (uint32_t)lP, (uint32_t)c->size_Q, (uint32_t)c->size_QP, (uint32_t)beta, rg, ib, perm);
    else if (fused)
        ks_inner_prod_kernel<3, true><<<grid, 256, 0, s>>>(digits, own, ep, out, ct, c->d_Pinv, c->d_mod, c->d_redc, (uint32_t)c->N, (uint32_t)l, (uint32_t)lP,
                                                         (uint32_t)c->size_Q, (uint32_t)c->size_QP, (uint32_t)beta, rg, ib, perm);
    else
        ks_inner_prod_kernel<3, false><<<grid, 256, 0, s>>>(digits, own, ep, out, nullptr, nullptr, c->d_mod, c->d_redc, (uint32_t)c->N, (uint32_t)l, (uint32_t)lP,
                                                          (uint32_t)c->size_Q, (uint32_t)c->size_QP, (uint32_t)beta, rg, ib, perm);
    LAUNCH_CHECK("ks_inner_prod_kernel");
    return B2_OK;
}

extern "C" int b2_ks_inner_prod(b2_ctx *c, size_t l, const uint64_t *d_digits, const uint64_t *const *evk, size_t n_evk, uint64_t *d_out,
                                void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_digits || !evk || !d_out) return fail(B2_EINVAL, "ks_inner_prod: null pointer");
    return inner_prod_impl(c, l, d_digits, nullptr, evk, n_evk, d_out, nullptr, false, (cudaStream_t)stream);
}

// ModDown of n_poly (1 or 2) polynomials held in cx [n_poly][l+alpha][N].
// ACCUM: out += result (the add_to_ct step of the key switch), else out = result.
// delta: n_poly * l limbs of scratch.
static int moddown_impl(b2_ctx *c, size_t l, size_t n_poly, uint64_t *cx, uint64_t *out, uint64_t *delta, bool accum, cudaStream_t s) {
    const LevelPlan &pl = c->plan[l];
    const size_t a = c->size_P;
    int rc = run_inv(c, cx, cx, pl.jobs_dn_intt, (uint32_t)(n_poly * a), 0, c->d_fin_P, s);
    if (rc) return rc;
    rc = run_bconv(c, false, cx, delta, nullptr, pl.grp_dn, (uint32_t)n_poly, pl.outs_dn, c->d_mat_dn, c->d_matd_dn, (uint32_t)a, (uint32_t)l, true, s, &pl.tc_dn,
                   (uint32_t)n_poly * pl.tc_dn.jobs_per_poly);
    if (rc) return rc;
    if (accum) {
        EpiSubMul<true> epi{cx, out, c->d_Pinv};
        return run_fwd(c, delta, delta, pl.jobs_dn_ntt, (uint32_t)(n_poly * l), 0, epi, s);
    }
    EpiSubMul<false> epi{cx, out, c->d_Pinv};
    return run_fwd(c, delta, delta, pl.jobs_dn_ntt, (uint32_t)(n_poly * l), 0, epi, s);
}

extern "C" int b2_moddown(b2_ctx *c, size_t l, size_t n_poly, uint64_t *d_cx, uint64_t *d_out, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_cx || !d_out || !d_ws) return fail(B2_EINVAL, "moddown: null pointer");
    if (n_poly < 1 || n_poly > 2) return fail(B2_EINVAL, "moddown: n_poly must be 1 or 2");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_MODDOWN, l)) return fail(B2_EWS, "moddown: workspace too small");
    return moddown_impl(c, l, n_poly, d_cx, d_out, (uint64_t *)d_ws, false, (cudaStream_t)stream);
}

// Everything after ModUp, fused: ct += ModDown(<digits, evk>).
// The inner product adds acc * P^-1 into the Q limbs of ct and keeps only the P limbs (cxP,
// [2][alpha][N]); their inverse transform, the base conversion with the P^-1-carrying matrix and a
// forward transform whose epilogue subtracts from ct finish the job. `delta`: 2*l limbs of scratch.
static int ks_tail_fused(b2_ctx *c, size_t l, const uint64_t *digits, const uint64_t *own, const uint64_t *const *evk, size_t n_evk, uint64_t *ct,
                         uint64_t *cxP, uint64_t *delta, cudaStream_t s, const uint32_t *perm = nullptr) {
    const LevelPlan &pl = c->plan[l];
    const size_t a = c->size_P;
    int rc = inner_prod_impl(c, l, digits, own, evk, n_evk, cxP, ct, true, s, nullptr, false, 1, nullptr, perm);
    if (rc) return rc;
    rc = run_inv(c, cxP, cxP, pl.jobs_dnf_intt, (uint32_t)(2 * a), 0, c->d_fin_P, s);
    if (rc) return rc;
    rc = run_bconv(c, false, cxP, delta, nullptr, pl.grp_dnf, 2, pl.outs_dn, c->d_mat_dn_pinv, c->d_matd_dn_pinv, (uint32_t)a, (uint32_t)l, true, s, &pl.tc_dnf);
    if (rc) return rc;
    return run_fwd(c, delta, delta, pl.jobs_dnf_ntt, (uint32_t)(2 * l), 0, EpiSubFrom{ct}, s);
}

// ModUp and inner product of the fused key switch with the FP64 limbs' inner product inside the last forward pass.
// Applies at N = 2^16 when the level's Q limbs are FP64 primes behind a prefix of wide ones; *done tells whether it ran.
// ct [2][l][N] += (inner product) * P^-1 on the Q limbs; cxP [2][alpha][N] = (acc_p: +=) the P limbs of the inner product.
// A batch of key switches with one key, every kernel one launch over the batch: set b's input, ciphertext, and its scratch
// blocks t [l], up [beta][l+alpha], cxP [2][alpha] start b * c2_bs / ct_bs / l / beta (l+alpha) / 2 alpha limbs further.
struct KsBatch {
    uint32_t batch = 1, c2_bs = 0, ct_bs = 0;
};

static int modup_inner_fused(b2_ctx *c, size_t l, const uint64_t *c2, const uint64_t *const *evk, size_t n_evk, uint64_t *ct, uint64_t *cxP,
                             uint64_t *t, uint64_t *up, bool acc_p, cudaStream_t s, bool *done, const KsBatch &kb = KsBatch{}) {
    const size_t N = c->N, lP = l + c->size_P, beta = c->plan[l].beta;
    const LevelPlan &pl = c->plan[l];
    *done = false;
    const bool wide = (c->mac_wide < 0 ? kb.batch > 1 : c->mac_wide == 1) && beta <= B2_MAC_MAX_BETA;
    if (!(c->use_mac && (pl.mac_ok || wide) && n_evk >= beta && aligned32(c2) && aligned32(ct) && aligned32(up) && aligned32(cxP))) return B2_OK;
    {
        // ModUp up to the column pass for every limb; the row pass is stored only for the limbs the stand-alone inner
        // product still handles (wide Q primes and P); for the FP64 limbs of Q it runs inside ntt_fwd_rows_mac
        using Cfg = PassCfg<8>;
        const uint32_t B = kb.batch, per = (uint32_t)(beta * lP), a2 = (uint32_t)(2 * c->size_P);
        const bool batched = B != 1;
        if (batched && (!c->bconv_tc || c->tc_simple || !pl.tc_up.jobs || !pl.tc_dnf.jobs)) return B2_OK;  // the caller falls back to one key switch at a time
        int rc = run_inv(c, c2, t, pl.jobs_up_intt, (uint32_t)l, 0, pl.fin_up, s, BatchDims{B, 0, kb.c2_bs, 0, (uint32_t)l});
        if (rc) return rc;
        if (batched) {
            const TcBatch tb{B, 0, (uint32_t)l, 0, per, c->tc_serial_ld ? 1u : 0u};
            rc = run_bconv_tc(c, false, t, up, nullptr, pl.tc_up, pl.tc_up.n_jobs, s, &tb);
        } else {
            rc = run_bconv(c, false, t, up, c2, pl.grp_up, pl.beta, pl.outs_up, pl.mat_up, pl.matd_up, (uint32_t)c->size_P, (uint32_t)lP, true, s, &pl.tc_up);
        }
        if (rc) return rc;
        NttArgs a{up, up, pl.jobs_up_ntt, 0, (uint32_t)c->logN, c->d_tw, c->d_mod, nullptr, 0};
        a.src_bs = a.dst_bs = batched ? per : 0;
        {
            NttArgs a1 = a;
            const dim3 grid = pass_grid(a1, pl.n_up_ntt * (uint32_t)(N >> (8 + Cfg::LOG_CC)), B);
            LaunchScope ls(c, s, "ntt_fwd_cols");
            ntt_fwd_pass<8, Cfg::R_STRIDED, Cfg::R_CONTIG, Cfg::LOG_CC, true, false, EpiStore><<<grid, pass_threads<8, true>(), 0, s>>>(a1, EpiStore{});
            LAUNCH_CHECK("ntt_fwd_pass");
        }
        // the limbs on 60-bit primes (q0, P) either ride on the fused pass too (integer arithmetic) or, mac_wide off,
        // keep the stored row pass and the stand-alone inner product
        if (!wide && pl.n_up_rows) {
            NttArgs b = a;
            b.jobs = pl.jobs_up_rows;
            const dim3 grid = pass_grid(b, pl.n_up_rows * (uint32_t)(N >> (8 + Cfg::LOG_C)), B);
            LaunchScope ls(c, s, "ntt_fwd_rows");
            ntt_fwd_pass<8, Cfg::R_STRIDED, Cfg::R_CONTIG, Cfg::LOG_C, false, true, EpiStore><<<grid, pass_threads<8>(), 0, s>>>(b, EpiStore{});
            LAUNCH_CHECK("ntt_fwd_pass");
        }
        if (!wide) {
            const uint4 rest = make_uint4(0, pl.n_wideQ, 0, (uint32_t)c->size_P);
            const IpBatch ib{per, kb.c2_bs, kb.ct_bs, 1, (uint32_t)c->size_P, 0, a2};
            rc = inner_prod_impl(c, l, up, c2, evk, n_evk, cxP, ct, true, s, &rest, acc_p, B, batched ? &ib : nullptr);
            if (rc) return rc;
        }
        {
            MacArgs m{};
            m.own = c2;
            for (size_t d = 0; d < beta; d++) {
                if (!evk[d]) return fail(B2_EINVAL, "null evaluation-key digit");
                m.evk[d] = evk[d];
            }
            m.ct = ct, m.cxp = cxP, m.pinv = c->d_Pinv, m.fin = c->d_macfin;
            m.l = (uint32_t)l, m.lP = (uint32_t)lP, m.alpha = (uint32_t)c->size_P, m.beta = (uint32_t)beta;
            m.size_Q = (uint32_t)c->size_Q, m.size_QP = (uint32_t)c->size_QP;
            m.first_limb = wide ? 0 : pl.n_wideQ, m.p_first = wide ? (uint32_t)c->size_P : 0, m.acc_p = acc_p ? 1 : 0;
            m.interleave = c->mac_interleave ? 1 : 0;
            m.dig_bs = per, m.own_bs = kb.c2_bs, m.ct_bs = kb.ct_bs, m.cxp_bs = a2;
            m.p_off = 0, m.cxp_i = 1, m.cxp_k = (uint32_t)c->size_P;
            const uint32_t n_limbs = (uint32_t)l - m.first_limb + m.p_first;
            LaunchScope ls(c, s, "ntt_fwd_rows_mac");
            static_assert(Cfg::R_STRIDED == Cfg::R_CONTIG, "the fused pass wants equal stage groups");
            static_assert(Cfg::R_CONTIG == 4 && Cfg::LOG_C == 3, "b2_ctx_create raises the shared-memory limit of this instantiation");
            ntt_fwd_rows_mac<8, Cfg::R_CONTIG, Cfg::LOG_C>
                <<<dim3(B, n_limbs * (uint32_t)(N >> (8 + Cfg::LOG_C))), pass_threads<8>(), mac_smem_bytes<8, Cfg::R_CONTIG, Cfg::LOG_C>(), s>>>(a, m);
            LAUNCH_CHECK("ntt_fwd_rows_mac");
        }
    }
    *done = true;
    return B2_OK;
}

// ws layout of the key switch: t [l] | up [beta][lP] | cxP [2][alpha]; delta reuses `up`
static int keyswitch_impl(b2_ctx *c, size_t l, const uint64_t *c2, const uint64_t *const *evk, size_t n_evk, uint64_t *ct, uint64_t *ws,
                          cudaStream_t s) {
    const size_t N = c->N, lP = l + c->size_P, beta = c->plan[l].beta;
    uint64_t *t = ws, *up = t + l * N, *cxP = up + beta * lP * N;
    const LevelPlan &pl = c->plan[l];
    bool done = false;
    int rc = modup_inner_fused(c, l, c2, evk, n_evk, ct, cxP, t, up, false, s, &done);
    if (rc) return rc;
    if (done) {
        const size_t ap = c->size_P;
        rc = run_inv(c, cxP, cxP, pl.jobs_dnf_intt, (uint32_t)(2 * ap), 0, c->d_fin_P, s);
        if (rc) return rc;
        rc = run_bconv(c, false, cxP, up, nullptr, pl.grp_dnf, 2, pl.outs_dn, c->d_mat_dn_pinv, c->d_matd_dn_pinv, (uint32_t)ap, (uint32_t)l, true, s, &pl.tc_dnf);
        if (rc) return rc;
        return run_fwd(c, up, up, pl.jobs_dnf_ntt, (uint32_t)(2 * l), 0, EpiSubFrom{ct}, s);
    }
    rc = modup_impl(c, l, c2, up, t, false, s);  // the inner product reads the own limbs from c2
    if (rc) return rc;
    return ks_tail_fused(c, l, up, c2, evk, n_evk, ct, cxP, up, s);
}

extern "C" int b2_keyswitch(b2_ctx *c, size_t l, const uint64_t *d_c2, const uint64_t *const *evk, size_t n_evk, uint64_t *d_ct, void *d_ws,
                            size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_c2 || !evk || !d_ct || !d_ws) return fail(B2_EINVAL, "keyswitch: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_KEYSWITCH, l)) return fail(B2_EWS, "keyswitch: workspace too small");
    return keyswitch_impl(c, l, d_c2, evk, n_evk, d_ct, (uint64_t *)d_ws, (cudaStream_t)stream);
}

extern "C" size_t b2_keyswitch_batch_workspace_bytes(const b2_ctx *c, size_t l, size_t batch) {
    if (!c || l < 1 || l > c->size_Q || batch < 1) return 0;
    const size_t a = c->size_P, beta = (l + a - 1) / a, lP = l + a;
    return batch * (l + 2 * a + beta * lP) * limb_bytes(c);
}

// `batch` key switches with ONE key: ct_b [2][l][N] += ModDown(<ModUp(c2_b), key>), set b's input at d_c2 + b * c2_stride
// limbs and its ciphertext at d_ct + b * ct_stride limbs. Where the fused pipeline applies (N = 2^16, tensor-core base
// conversion) every kernel is one launch over the whole batch - 10 to 12 launches for the batch instead of per key
// switch, grids that fill the GPU at every level, and the key read from HBM once per batch: the fused inner product
// puts the sets that share a key tile next to one another in the grid, so all but the first find it in L2. Elsewhere the
// key switches run one after another on the same stream. Workspace: t [batch][l] | up [batch][beta][l+alpha] | cxP [batch][2][alpha].
static int keyswitch_batch_impl(b2_ctx *c, size_t l, size_t batch, const uint64_t *d_c2, size_t c2_stride, const uint64_t *const *evk, size_t n_evk,
                                  uint64_t *d_ct, size_t ct_stride, void *d_ws, cudaStream_t s) {
    const LevelPlan &pl = c->plan[l];
    const size_t N = c->N, a = c->size_P, lP = l + a, beta = pl.beta;
    const uint32_t B = (uint32_t)batch, per = (uint32_t)(beta * lP);
    uint64_t *t = (uint64_t *)d_ws, *up = t + batch * l * N, *cxP = up + batch * per * N;
    bool done = false;
    int rc = B2_OK;
    if (batch > 1) {
        rc = modup_inner_fused(c, l, d_c2, evk, n_evk, d_ct, cxP, t, up, false, s, &done, KsBatch{B, (uint32_t)c2_stride, (uint32_t)ct_stride});
        if (rc) return rc;
    }
    if (!done) {
        // one at a time, each in its own block of the workspace
        const size_t one = l + beta * lP + 2 * a;
        for (size_t b = 0; b < batch; b++) {
            rc = keyswitch_impl(c, l, d_c2 + b * c2_stride * N, evk, n_evk, d_ct + b * ct_stride * N, (uint64_t *)d_ws + b * one * N, s);
            if (rc) return rc;
        }
        return B2_OK;
    }
    // ModDown of the P limbs of both polynomials of every set; delta takes the front of each set's `up` block
    rc = run_inv(c, cxP, cxP, pl.jobs_dnf_intt, (uint32_t)(2 * a), 0, c->d_fin_P, s, BatchDims{B, 0, (uint32_t)(2 * a), 0, (uint32_t)(2 * a)});
    if (rc) return rc;
    const TcBatch tb{B, 0, (uint32_t)(2 * a), 0, per, 0};
    rc = run_bconv_tc(c, false, cxP, up, nullptr, pl.tc_dnf, pl.tc_dnf.n_jobs, s, &tb);
    if (rc) return rc;
    return run_fwd(c, up, up, pl.jobs_dnf_ntt, (uint32_t)(2 * l), 0, EpiSubFrom{d_ct, (uint32_t)ct_stride}, s, 0, 0, 0, BatchDims{B, 0, per, 0, per});
}

extern "C" int b2_keyswitch_batch(b2_ctx *c, size_t l, size_t batch, const uint64_t *d_c2, size_t c2_stride, const uint64_t *const *evk, size_t n_evk,
                                  uint64_t *d_ct, size_t ct_stride, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_c2 || !evk || !d_ct || !d_ws || batch < 1 || batch > 65535) return fail(B2_EINVAL, "keyswitch_batch: bad argument");
    if (c2_stride < l || ct_stride < 2 * l || c2_stride > 0xFFFFFFFFull || ct_stride > 0xFFFFFFFFull)
        return fail(B2_EINVAL, "keyswitch_batch: a set's stride is smaller than the set");
    if (ws_bytes < b2_keyswitch_batch_workspace_bytes(c, l, batch)) return fail(B2_EWS, "keyswitch_batch: workspace too small");
    return keyswitch_batch_impl(c, l, batch, d_c2, c2_stride, evk, n_evk, d_ct, ct_stride, d_ws, (cudaStream_t)stream);
}

extern "C" int b2_tensor_mul(b2_ctx *c, size_t l, const uint64_t *d_a, const uint64_t *d_b, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_a || !d_b || !d_out) return fail(B2_EINVAL, "tensor_mul: null pointer");
    const size_t n = l * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "tensor_mul");
    tensor_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_a, d_b, d_out, d_out + 2 * n, c->d_mod, (uint32_t)c->N, (uint32_t)l, make_uint4(0, 0, 0, 0));
    LAUNCH_CHECK("tensor_mul_kernel");
    return B2_OK;
}

extern "C" int b2_multiply_and_relin(b2_ctx *c, size_t l, const uint64_t *d_a, const uint64_t *d_b, const uint64_t *const *rlk, size_t n_evk,
                                     uint64_t *d_out, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_a || !d_b || !rlk || !d_out || !d_ws) return fail(B2_EINVAL, "multiply_and_relin: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_MUL_RELIN, l)) return fail(B2_EWS, "multiply_and_relin: workspace too small");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t S = l * c->N;
    uint64_t *t3 = (uint64_t *)d_ws, *ws = t3 + 3 * S;
    {
        // d0, d1 straight into the result, d2 into scratch for the key switch (every thread reads its own position of
        // the operands before it writes, so the result may alias an operand)
        LaunchScope ls(c, s, "tensor_mul");
        tensor_mul_kernel<<<(unsigned)((S + 255) / 256), 256, 0, s>>>(d_a, d_b, d_out, t3 + 2 * S, c->d_mod, (uint32_t)c->N, (uint32_t)l, make_uint4(0, 0, 0, 0));
        LAUNCH_CHECK("tensor_mul_kernel");
    }
    return keyswitch_impl(c, l, t3 + 2 * S, rlk, n_evk, d_out, ws, s);
}

// Second half of a rescale. r [n_poly][N]: the dropped limb of every polynomial in coefficient form. Every remaining
// limb j gets (in_j - NTT_j(rem mod q_j)) * q_last^-1 with rem = r (MODE 1, the reference's floor: src/rns.cu:1128-1183)
// or its centred representative (MODE 2, round to nearest). The forward column pass reduces r into q_j as it loads, so
// the (l-1) reduced copies are never written out; the one-launch and pipelined transform variants have no such load and
// go through a reduction kernel first.
template <int MODE>
static int rescale_tail(const b2_ctx *c, size_t l, size_t n_poly, const uint64_t *r, const uint64_t *d_in, uint64_t *d_out, cudaStream_t s) {
    const LevelPlan &pl = c->plan[l];
    EpiSubMul<false> epi{d_in, d_out, pl.qlast_inv};
    const uint32_t njobs = (uint32_t)(n_poly * (l - 1));
    if (!c->use_cluster && !c->use_pipe) return run_fwd<EpiSubMul<false>, MODE>(c, r, d_out, pl.jobs_rs_ntt, njobs, 0, epi, s, 0, (uint32_t)(l - 1), c->q[l - 1]);
    if (MODE == 1) {
        // r mod q_j for every remaining prime: a base conversion with one input and the matrix [1]
        int rc = run_bconv(c, false, r, d_out, nullptr, pl.grp_rs, (uint32_t)n_poly, pl.outs_rs, c->d_one, c->d_matd_one, 1, (uint32_t)(l - 1), true, s);
        if (rc) return rc;
    } else {
        const size_t n = n_poly * (l - 1) * c->N;
        LaunchScope ls(c, s, "rescale_centre");
        rescale_centre_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(r, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)(l - 1), (uint32_t)n_poly);
        LAUNCH_CHECK("rescale_centre_kernel");
    }
    return run_fwd(c, d_out, d_out, pl.jobs_rs_ntt, njobs, 0, epi, s);
}

extern "C" int b2_rescale(b2_ctx *c, size_t l, size_t n_poly, const uint64_t *d_in, uint64_t *d_out, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (l < 2) return fail(B2_EINVAL, "rescale: no prime left to drop");
    if (n_poly < 1 || n_poly > 3) return fail(B2_EINVAL, "rescale: n_poly must be in [1, 3]");
    if (!d_in || !d_out || !d_ws) return fail(B2_EINVAL, "rescale: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_RESCALE, l)) return fail(B2_EWS, "rescale: workspace too small");
    cudaStream_t s = (cudaStream_t)stream;
    const LevelPlan &pl = c->plan[l];
    uint64_t *r = (uint64_t *)d_ws;  // [n_poly][N] coefficient form of the dropped limbs
    {
        // dropped limb of every polynomial in one launch pair: limb p*l + l-1 of the input -> limb p of r
        int rc = run_inv(c, d_in, r, pl.jobs_rs_intt, (uint32_t)n_poly, 0, c->d_fin_plain, s);
        if (rc) return rc;
    }
    return rescale_tail<1>(c, l, n_poly, r, d_in, d_out, s);
}

extern "C" int b2_rescale_rounded(b2_ctx *c, size_t l, size_t n_poly, const uint64_t *d_in, uint64_t *d_out, void *d_ws, size_t ws_bytes,
                                  void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (l < 2) return fail(B2_EINVAL, "rescale_rounded: no prime left to drop");
    if (n_poly < 1 || n_poly > 3) return fail(B2_EINVAL, "rescale_rounded: n_poly must be in [1, 3]");
    if (!d_in || !d_out || !d_ws) return fail(B2_EINVAL, "rescale_rounded: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_RESCALE, l)) return fail(B2_EWS, "rescale_rounded: workspace too small");
    cudaStream_t s = (cudaStream_t)stream;
    const LevelPlan &pl = c->plan[l];
    uint64_t *r = (uint64_t *)d_ws;
    {
        // dropped limb of every polynomial in one launch pair: limb p*l + l-1 of the input -> limb p of r
        int rc = run_inv(c, d_in, r, pl.jobs_rs_intt, (uint32_t)n_poly, 0, c->d_fin_plain, s);
        if (rc) return rc;
    }
    return rescale_tail<2>(c, l, n_poly, r, d_in, d_out, s);
}

extern "C" size_t b2_multiply_relin_batch_workspace_bytes(const b2_ctx *c, size_t l, size_t batch) {
    if (!c || l < 1 || l > c->size_Q || batch < 1) return 0;
    return batch * (3 * l + 2) * limb_bytes(c) + b2_keyswitch_batch_workspace_bytes(c, l, batch);
}

// HMult + relinearise (+ rescale) of `batch` ciphertext pairs with ONE relinearisation key, every kernel one launch over
// the batch: tensor product, b2_keyswitch_batch's pipeline, and - rescale != 0 - the drop of the last prime
// (src/evaluate.cu:1061-1104, 1413-1464). Pair b reads d_a + b * a_stride and d_b + b * b_stride limbs ([2][l][N] each)
// and writes d_out + b * out_stride limbs: [2][l][N], or [2][l-1][N] after the rescale. Same limbs as b2_multiply_and_relin
// followed by b2_rescale. Workspace: prod [batch][3][l] | r [batch][2] | the key switch's.
extern "C" int b2_multiply_relin_rescale_batch(b2_ctx *c, size_t l, size_t batch, const uint64_t *d_a, size_t a_stride, const uint64_t *d_b,
                                               size_t b_stride, const uint64_t *const *rlk, size_t n_evk, uint64_t *d_out, size_t out_stride,
                                               int rescale, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_a || !d_b || !rlk || !d_out || !d_ws || batch < 1 || batch > 65535) return fail(B2_EINVAL, "multiply_relin_rescale_batch: bad argument");
    if (rescale && l < 2) return fail(B2_EINVAL, "multiply_relin_rescale_batch: no prime left to drop");
    const size_t out_limbs = 2 * (rescale ? l - 1 : l);
    if (a_stride < 2 * l || b_stride < 2 * l || out_stride < out_limbs || a_stride > 0xFFFFFFFFull || b_stride > 0xFFFFFFFFull || out_stride > 0xFFFFFFFFull)
        return fail(B2_EINVAL, "multiply_relin_rescale_batch: a pair's stride is smaller than the pair");
    if (ws_bytes < b2_multiply_relin_batch_workspace_bytes(c, l, batch)) return fail(B2_EWS, "multiply_relin_rescale_batch: workspace too small");
    if (!aligned32(d_a) || !aligned32(d_b) || !aligned32(d_out) || !aligned32(d_ws)) return fail(B2_EINVAL, "device buffers must be 32-byte aligned (256-bit accesses)");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t N = c->N, S = l * N;
    const uint32_t B = (uint32_t)batch;
    uint64_t *prod = (uint64_t *)d_ws, *r = prod + batch * 3 * S, *ws = r + batch * 2 * N;
    {
        LaunchScope ls(c, s, "tensor_mul");
        tensor_mul_kernel<<<dim3((unsigned)((S + 255) / 256), B), 256, 0, s>>>(d_a, d_b, prod, prod + 2 * S, c->d_mod, (uint32_t)N, (uint32_t)l,
                                                                             make_uint4((uint32_t)a_stride, (uint32_t)b_stride, (uint32_t)(3 * l), (uint32_t)(3 * l)));
        LAUNCH_CHECK("tensor_mul_kernel");
    }
    int rc = keyswitch_batch_impl(c, l, batch, prod + 2 * S, 3 * l, rlk, n_evk, prod, 3 * l, ws, s);
    if (rc) return rc;
    if (!rescale) {
        for (size_t b = 0; b < batch; b++)
            CUDA_TRY(cudaMemcpyAsync(d_out + b * out_stride * N, prod + b * 3 * S, 2 * S * 8, cudaMemcpyDeviceToDevice, s));
        return B2_OK;
    }
    if (c->use_cluster || c->use_pipe) {
        for (size_t b = 0; b < batch; b++) {
            rc = run_inv(c, prod + b * 3 * S, r, c->plan[l].jobs_rs_intt, 2, 0, c->d_fin_plain, s);
            if (rc) return rc;
            rc = rescale_tail<1>(c, l, 2, r, prod + b * 3 * S, d_out + b * out_stride * N, s);
            if (rc) return rc;
        }
        return B2_OK;
    }
    const LevelPlan &pl = c->plan[l];
    // the dropped limb of both polynomials of every pair, then every remaining limb (in_j - NTT_j(r mod q_j)) * q_last^-1
    rc = run_inv(c, prod, r, pl.jobs_rs_intt, 2, 0, c->d_fin_plain, s, BatchDims{B, 0, (uint32_t)(3 * l), 0, 2});
    if (rc) return rc;
    EpiSubMul<false> epi{prod, d_out, pl.qlast_inv};
    epi.m_bs = (uint32_t)(3 * l), epi.o_bs = (uint32_t)out_stride;
    return run_fwd<EpiSubMul<false>, 1>(c, r, d_out, pl.jobs_rs_ntt, (uint32_t)(2 * (l - 1)), 0, epi, s, 0, (uint32_t)(l - 1), c->q[l - 1],
                                         BatchDims{B, 0, 2, 0, (uint32_t)out_stride});
}

// ------------------------------------------------------------------------------------------------
// rescale without any caller-provided or allocated scratch
// ------------------------------------------------------------------------------------------------
// Some callers can hand over inputs and outputs but no scratch buffer and must not allocate one:
// a process whose device memory has been reserved up front by another allocator (so a late
// cudaMalloc fails), or a host thread that is not allowed to enter an allocating CUDA call at
// that point. For them the coefficient-form copies of the dropped limbs live in a fixed array
// that is part of the library image: B2_STATIC_RESCALE_MAX_POLY polynomials of at most
// B2_STATIC_RESCALE_MAX_N coefficients, 1.5 MiB, held by every GPU that loads the library until
// the process exits.
#define B2_STATIC_RESCALE_MAX_N 65536
#define B2_STATIC_RESCALE_MAX_POLY 3
static __device__ __align__(256) uint64_t g_rescale_scratch[B2_STATIC_RESCALE_MAX_POLY * B2_STATIC_RESCALE_MAX_N];

// In host code the symbol above is only a handle, not a device address. The address is looked up
// once per device (with that device current) and cached.
static std::mutex g_scratch_mu;
static uint64_t *g_scratch_ptr[64] = {nullptr};

static int rescale_scratch_for_device(int device, uint64_t **out) {
    if (device < 0 || device >= 64) return fail(B2_EINVAL, "rescale_static: device index out of range");
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_rescale_scratch);
        if (e != cudaSuccess) return fail((int)e, std::string("rescale_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        g_scratch_ptr[device] = static_cast<uint64_t *>(p);
    }
    *out = g_scratch_ptr[device];
    return B2_OK;
}

extern "C" int b2_rescale_static(b2_ctx *c, size_t l, size_t n_poly, const uint64_t *d_in, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (l < 2) return fail(B2_EINVAL, "rescale_static: no prime left to drop");
    if (!d_in || !d_out) return fail(B2_EINVAL, "rescale_static: null pointer");
    if (n_poly < 1 || n_poly > B2_STATIC_RESCALE_MAX_POLY)
        return fail(B2_ESIZE, "rescale_static: n_poly exceeds the built-in scratch (at most 3 polynomials)");
    if (c->N > B2_STATIC_RESCALE_MAX_N)
        return fail(B2_ESIZE, "rescale_static: polynomial degree exceeds the built-in scratch (at most 65536 coefficients)");
    uint64_t *r = nullptr;
    int rc = rescale_scratch_for_device(c->device, &r);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const LevelPlan &pl = c->plan[l];
    // every word of r that is read below is written first by the inverse transforms, so nothing
    // left over from an earlier call needs clearing
    for (size_t p = 0; p < n_poly; p++) {
        rc = run_inv(c, d_in + (p * l + l - 1) * c->N, r + p * c->N, nullptr, 1, (uint32_t)(l - 1), c->d_fin_plain, s);
        if (rc) return rc;
    }
    return rescale_tail<1>(c, l, n_poly, r, d_in, d_out, s);
}

extern "C" uint32_t b2_galois_elt_from_step(int step, size_t N) {
    const uint32_t n = (uint32_t)N, m = 2 * n;
    if (step == 0) return m - 1;
    const bool neg = step < 0;
    const uint32_t pos = (uint32_t)(neg ? -(int64_t)step : step);
    if (pos >= (n >> 1)) return 0;
    uint32_t k = neg ? (n >> 1) - pos : pos;
    uint64_t e = 1;
    while (k--) e = (e * 5) & (m - 1);
    return (uint32_t)e;
}

static int galois_table(b2_ctx *c, uint32_t elt, const uint32_t **out) {
    std::lock_guard<std::mutex> lk(c->mu);
    auto it = c->galois.find(elt);
    if (it != c->galois.end()) {
        *out = it->second;
        return B2_OK;
    }
    if (!(elt & 1) || elt >= 2 * c->N) return fail(B2_EINVAL, "Galois element must be odd and below 2N");
    const size_t N = c->N;
    std::vector<uint32_t> perm(N);
    for (size_t i = 0; i < N; i++) {
        const uint32_t rev = h_bitrev((uint32_t)(i + N), c->logN + 1);
        const uint64_t raw = (((uint64_t)elt * rev) >> 1) & (N - 1);
        perm[i] = h_bitrev((uint32_t)raw, c->logN);
    }
    uint32_t *d = nullptr;
    CUDA_TRY(cudaMalloc(&d, N * 4));
    CUDA_TRY(cudaMemcpy(d, perm.data(), N * 4, cudaMemcpyHostToDevice));
    c->galois[elt] = d;
    *out = d;
    return B2_OK;
}

extern "C" int b2_galois_prepare(b2_ctx *c, uint32_t elt) {
    CHECK_CTX(c);
    const uint32_t *t;
    return galois_table(c, elt, &t);
}

static int gather_impl(b2_ctx *c, const uint32_t *perm, const uint64_t *src, uint64_t *dst, size_t n_limbs, cudaStream_t s) {
    const size_t n = n_limbs * c->N;
    LaunchScope ls(c, s, "galois_gather");
    galois_gather_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, perm, (uint32_t)c->N, (uint32_t)n_limbs);
    LAUNCH_CHECK("galois_gather_kernel");
    return B2_OK;
}

static int gather_split_impl(b2_ctx *c, const uint32_t *perm, const uint64_t *src, uint64_t *dst0, uint64_t *dst1, size_t l, bool acc, cudaStream_t s) {
    const size_t n = 2 * l * c->N;
    LaunchScope ls(c, s, "galois_gather");
    if (acc) galois_split_kernel<true><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst0, dst1, perm, c->d_mod, (uint32_t)c->N, (uint32_t)l);
    else galois_split_kernel<false><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst0, dst1, perm, c->d_mod, (uint32_t)c->N, (uint32_t)l);
    LAUNCH_CHECK("galois_split_kernel");
    return B2_OK;
}

// tables must exist before an asynchronous sequence starts: creating one synchronises
static int galois_lookup(b2_ctx *c, uint32_t elt, const uint32_t **out) {
    std::lock_guard<std::mutex> lk(c->mu);
    auto it = c->galois.find(elt);
    if (it == c->galois.end()) return fail(B2_ENOKEY, "Galois elt not present: call b2_galois_prepare first");
    *out = it->second;
    return B2_OK;
}

extern "C" int b2_galois_permute(b2_ctx *c, uint32_t elt, const uint64_t *d_src, uint64_t *d_dst, size_t n_limbs, void *stream) {
    CHECK_CTX(c);
    if (!d_src || !d_dst || d_src == d_dst) return fail(B2_EINVAL, "galois_permute: needs distinct source and destination");
    const uint32_t *perm;
    int rc = galois_lookup(c, elt, &perm);
    if (rc) return rc;
    return gather_impl(c, perm, d_src, d_dst, n_limbs, (cudaStream_t)stream);
}

extern "C" int b2_apply_galois(b2_ctx *c, size_t l, uint32_t elt, const uint64_t *d_ct, const uint64_t *const *ksk, size_t n_evk, uint64_t *d_out,
                               void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_ct || !ksk || !d_out || !d_ws) return fail(B2_EINVAL, "apply_galois: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_ROTATE, l)) return fail(B2_EWS, "apply_galois: workspace too small");
    const uint32_t *perm;
    int rc = galois_lookup(c, elt, &perm);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t S = l * c->N;
    uint64_t *p = (uint64_t *)d_ws, *ws = p + 2 * S;  // permuted c0 | permuted c1
    // (c0, c1) <- (perm(c0), 0) + key switch of perm(c1)   (src/evaluate.cu:1644-1655)
    const bool apart = d_out + 2 * S <= d_ct || d_ct + 2 * S <= d_out;
    if (apart) {
        rc = gather_split_impl(c, perm, d_ct, d_out, p + S, l, false, s);  // perm(c0) lands in the result
        if (rc) return rc;
    } else {
        rc = gather_impl(c, perm, d_ct, p, 2 * l, s);  // both polynomials: limb index only selects the row
        if (rc) return rc;
        CUDA_TRY(cudaMemcpyAsync(d_out, p, S * 8, cudaMemcpyDeviceToDevice, s));
    }
    CUDA_TRY(cudaMemsetAsync(d_out + S, 0, S * 8, s));
    return keyswitch_impl(c, l, p + S, ksk, n_evk, d_out, ws, s);
}

// Rotations whose results are summed share one ModDown: each call adds perm(c0) + (inner product) * P^-1 on the Q limbs
// of d_acc and the P limbs of the inner product to d_accP; b2_keyswitch_finish converts the P limbs once.
extern "C" int b2_apply_galois_accumulate(b2_ctx *c, size_t l, uint32_t elt, const uint64_t *d_ct, const uint64_t *const *ksk, size_t n_evk,
                                          uint64_t *d_acc, uint64_t *d_accP, int first, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_ct || !ksk || !d_acc || !d_accP || !d_ws) return fail(B2_EINVAL, "apply_galois_accumulate: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_ROTATE, l)) return fail(B2_EWS, "apply_galois_accumulate: workspace too small");
    const uint32_t *perm;
    int rc = galois_lookup(c, elt, &perm);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t N = c->N, S = l * N, lP = l + c->size_P, beta = c->plan[l].beta;
    uint64_t *p = (uint64_t *)d_ws, *t = p + 2 * S, *up = t + S;  // permuted c0 | permuted c1 | t | up
    if (d_acc + 2 * S <= d_ct || d_ct + 2 * S <= d_acc) {
        // perm(c0) straight into (or onto) the accumulator, perm(c1) into scratch: one launch
        rc = gather_split_impl(c, perm, d_ct, d_acc, p + S, l, !first, s);
        if (rc) return rc;
        if (first) CUDA_TRY(cudaMemsetAsync(d_acc + S, 0, S * 8, s));
    } else {
        rc = gather_impl(c, perm, d_ct, p, 2 * l, s);
        if (rc) return rc;
        if (first) {
            CUDA_TRY(cudaMemcpyAsync(d_acc, p, S * 8, cudaMemcpyDeviceToDevice, s));
            CUDA_TRY(cudaMemsetAsync(d_acc + S, 0, S * 8, s));
        } else {
            rc = b2_poly_op(c, 0, l, d_acc, p, d_acc, stream);
            if (rc) return rc;
        }
    }
    (void)beta;
    (void)lP;
    bool done = false;
    rc = modup_inner_fused(c, l, p + S, ksk, n_evk, d_acc, d_accP, t, up, !first, s, &done);
    if (rc || done) return rc;
    rc = modup_impl(c, l, p + S, up, t, false, s);
    if (rc) return rc;
    return inner_prod_impl(c, l, up, p + S, ksk, n_evk, d_accP, d_acc, true, s, nullptr, !first);
}

extern "C" int b2_keyswitch_finish(b2_ctx *c, size_t l, uint64_t *d_accP, uint64_t *d_acc, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_accP || !d_acc || !d_ws) return fail(B2_EINVAL, "keyswitch_finish: null pointer");
    if (ws_bytes < 2 * l * c->N * sizeof(uint64_t)) return fail(B2_EWS, "keyswitch_finish: workspace too small (2 * size_Ql limbs)");
    cudaStream_t s = (cudaStream_t)stream;
    const LevelPlan &pl = c->plan[l];
    const size_t a = c->size_P;
    uint64_t *delta = (uint64_t *)d_ws;
    int rc = run_inv(c, d_accP, d_accP, pl.jobs_dnf_intt, (uint32_t)(2 * a), 0, c->d_fin_P, s);
    if (rc) return rc;
    rc = run_bconv(c, false, d_accP, delta, nullptr, pl.grp_dnf, 2, pl.outs_dn, c->d_mat_dn_pinv, c->d_matd_dn_pinv, (uint32_t)a, (uint32_t)l, true, s, &pl.tc_dnf);
    if (rc) return rc;
    return run_fwd(c, delta, delta, pl.jobs_dnf_ntt, (uint32_t)(2 * l), 0, EpiSubFrom{d_acc}, s);
}

extern "C" int b2_hoist_rotations(b2_ctx *c, size_t l, const uint64_t *d_ct, const uint32_t *elts, size_t n_steps, const uint64_t *const *ksk,
                                  size_t n_evk, uint64_t *const *d_outs, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_ct || !elts || !ksk || !d_outs || !d_ws) return fail(B2_EINVAL, "hoist_rotations: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_HOIST, l)) return fail(B2_EWS, "hoist_rotations: workspace too small");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t N = c->N, lP = l + c->size_P, beta = c->plan[l].beta, S = l * N;
    std::vector<const uint32_t *> perms(n_steps);
    for (size_t i = 0; i < n_steps; i++) {
        int rc = galois_lookup(c, elts[i], &perms[i]);
        if (rc) return rc;
    }
    // ws: t [l] | up [beta][lP] | pup [beta][lP] | cx [2][lP] | pc0 [l]
    uint64_t *t = (uint64_t *)d_ws, *up = t + S, *pup = up + beta * lP * N, *cx = pup + beta * lP * N, *pc0 = cx + 2 * lP * N;
    int rc = modup_impl(c, l, d_ct + S, up, t, true, s);  // ModUp(c1) once (src/evaluate.cu:2013-2014)
    if (rc) return rc;
    for (size_t i = 0; i < n_steps; i++) {
        if (!d_outs[i]) return fail(B2_EINVAL, "hoist_rotations: null output");
        rc = gather_impl(c, perms[i], d_ct, pc0, l, s);
        if (rc) return rc;
        // c0_out = perm(c0) + ModDown(cx0); c1_out = ModDown(cx1). The digits are permuted AFTER ModUp
        // (src/evaluate.cu:2041-2045): the inner product reads them through the permutation, `pup` only serves as delta
        CUDA_TRY(cudaMemcpyAsync(d_outs[i], pc0, S * 8, cudaMemcpyDeviceToDevice, s));
        CUDA_TRY(cudaMemsetAsync(d_outs[i] + S, 0, S * 8, s));
        rc = ks_tail_fused(c, l, up, nullptr, ksk + i * n_evk, n_evk, d_outs[i], cx, pup, s, perms[i]);
        if (rc) return rc;
    }
    return B2_OK;
}

// hoisting_inplace (src/evaluate.cu:1732-1927): the SUM of n_steps rotations from one ModUp and one ModDown pair.
extern "C" int b2_hoisting_sum(b2_ctx *c, size_t l, const uint64_t *d_ct, const uint32_t *elts, size_t n_steps, const uint64_t *const *ksk,
                               size_t n_evk, uint64_t *d_out, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_ct || !elts || !ksk || !d_out || !d_ws || n_steps == 0) return fail(B2_EINVAL, "hoisting_sum: bad argument");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_HOIST, l)) return fail(B2_EWS, "hoisting_sum: workspace too small");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t N = c->N, a = c->size_P, lP = l + a, beta = c->plan[l].beta, S = l * N;
    const LevelPlan &pl = c->plan[l];
    std::vector<const uint32_t *> perms(n_steps);
    for (size_t i = 0; i < n_steps; i++) {
        int rc = galois_lookup(c, elts[i], &perms[i]);
        if (rc) return rc;
    }
    // ws: t [l] | up [beta][lP] | pup [beta][lP] | accP [2][alpha] + delta [2][l] (the 2*lP limbs of cx) | pc0 [l]
    uint64_t *t = (uint64_t *)d_ws, *up = t + S, *pup = up + beta * lP * N /* unused: the digits are read through the permutation */, *accP = pup + beta * lP * N, *delta = accP + 2 * a * N,
             *pc0 = accP + 2 * lP * N;
    int rc = modup_impl(c, l, d_ct + S, up, t, true, s);
    if (rc) return rc;
    for (size_t i = 0; i < n_steps; i++) {
        rc = gather_impl(c, perms[i], d_ct, i == 0 ? d_out : pc0, l, s);
        if (rc) return rc;
        if (i == 0) CUDA_TRY(cudaMemsetAsync(d_out + S, 0, S * 8, s));
        else if ((rc = b2_poly_op(c, 0, l, d_out, pc0, d_out, stream))) return rc;
        rc = inner_prod_impl(c, l, up, nullptr, ksk + i * n_evk, n_evk, accP, d_out, true, s, nullptr, i > 0, 1, nullptr, perms[i]);
        if (rc) return rc;
    }
    rc = run_inv(c, accP, accP, pl.jobs_dnf_intt, (uint32_t)(2 * a), 0, c->d_fin_P, s);
    if (rc) return rc;
    rc = run_bconv(c, false, accP, delta, nullptr, pl.grp_dnf, 2, pl.outs_dn, c->d_mat_dn_pinv, c->d_matd_dn_pinv, (uint32_t)a, (uint32_t)l, true, s, &pl.tc_dnf);
    if (rc) return rc;
    return run_fwd(c, delta, delta, pl.jobs_dnf_ntt, (uint32_t)(2 * l), 0, EpiSubFrom{d_out}, s);
}

extern "C" int b2_bsgs_mac(b2_ctx *c, size_t l, size_t M, const uint64_t *const *pts, const uint64_t *const *babies, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!pts || !babies || !d_out || M == 0) return fail(B2_EINVAL, "bsgs_mac: bad argument");
    const size_t n = l * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "bsgs_mac");
    bsgs_mac_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(pts, babies, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)l, (uint32_t)M);
    LAUNCH_CHECK("bsgs_mac_kernel");
    return B2_OK;
}

extern "C" int b2_bsgs_mac_multi(b2_ctx *c, size_t l, size_t M, size_t n_giants, const uint64_t *const *pts, const uint64_t *const *babies,
                                 uint64_t *const *outs, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!pts || !babies || !outs || M == 0 || n_giants < 1 || n_giants > 4) return fail(B2_EINVAL, "bsgs_mac_multi: bad argument (1 to 4 giants)");
    const size_t n = l * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "bsgs_mac");
    bsgs_mac_multi_kernel<4><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(pts, babies, outs, c->d_mod, (uint32_t)c->N, (uint32_t)l,
                                                                                            (uint32_t)M, (uint32_t)n_giants);
    LAUNCH_CHECK("bsgs_mac_multi_kernel");
    return B2_OK;
}

extern "C" int b2_expand_signed(b2_ctx *c, size_t first_prime, size_t n_limbs, const int64_t *d_signed, uint64_t *d_out, int to_ntt,
                                void *stream) {
    CHECK_CTX(c);
    if (!d_signed || !d_out) return fail(B2_EINVAL, "expand_signed: null pointer");
    if (n_limbs < 1 || first_prime + n_limbs > c->size_QP) return fail(B2_EINVAL, "expand_signed: limb range outside the modulus chain");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = n_limbs * c->N;
    {
        LaunchScope ls(c, s, "expand_signed");
        expand_signed_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_signed, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)n_limbs,
                                                                        (uint32_t)first_prime);
        LAUNCH_CHECK("expand_signed_kernel");
    }
    if (!to_ntt) return B2_OK;
    return run_fwd(c, d_out, d_out, nullptr, (uint32_t)n_limbs, (uint32_t)first_prime, EpiStore{}, s);
}

// The encoder's transform (encoder.cuh): n = N/2 complex values, rot = 5^j mod 2N (uint32 [n]), ksi = exp(2 pi i k / 2N)
// (double2 [2N + 1]). inverse = 1 (encode): d_vals (natural order, overwritten) -> d_out = the embedding's preimage times
// `scale`; inverse = 0 (decode): d_vals -> d_out = slot values times `scale`. d_vals and d_out must not overlap.
extern "C" int b2_special_fft(b2_ctx *c, void *d_vals, void *d_out, const uint32_t *d_rot, const void *d_ksi, int inverse, double scale, void *stream) {
    CHECK_CTX(c);
    if (!d_vals || !d_out || !d_rot || !d_ksi || d_vals == d_out) return fail(B2_EINVAL, "special_fft: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t n = (uint32_t)(c->N / 2), M = (uint32_t)(2 * c->N), logn = (uint32_t)c->logN - 1;
    double2 *v = (double2 *)d_vals, *o = (double2 *)d_out;
    LaunchScope ls(c, s, "special_fft");
    if (inverse) {
        for (uint32_t len = n; len >= 2; len >>= 1)
            b2::cfft_stage_kernel<<<(n / 2 + 255) / 256, 256, 0, s>>>(v, n, len, d_rot, (const double2 *)d_ksi, M, 1);
        b2::cfft_bitrev_kernel<<<(n + 255) / 256, 256, 0, s>>>(o, v, n, logn, scale);
    } else {
        b2::cfft_bitrev_kernel<<<(n + 255) / 256, 256, 0, s>>>(o, v, n, logn, scale);
        for (uint32_t len = 2; len <= n; len <<= 1)
            b2::cfft_stage_kernel<<<(n / 2 + 255) / 256, 256, 0, s>>>(o, n, len, d_rot, (const double2 *)d_ksi, M, 0);
    }
    LAUNCH_CHECK("special_fft kernels");
    return B2_OK;
}

// d_u: N/2 complex values (the scaled preimage, every part below 2^62 in magnitude) -> d_coeffs int64 [N]: coefficient k =
// round(Re u_k), coefficient k + N/2 = round(Im u_k) (src/ckks.cu:97-131 before the decomposition into limbs)
extern "C" int b2_encode_round(b2_ctx *c, const void *d_u, int64_t *d_coeffs, void *stream) {
    CHECK_CTX(c);
    if (!d_u || !d_coeffs) return fail(B2_EINVAL, "encode_round: null pointer");
    const uint32_t n = (uint32_t)(c->N / 2);
    LaunchScope ls(c, (cudaStream_t)stream, "encode_round");
    b2::encode_round_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const double2 *)d_u, n, d_coeffs);
    LAUNCH_CHECK("encode_round_kernel");
    return B2_OK;
}

// CRT composition of a coefficient-form plaintext of l limbs (src/rns_base.cu:173-234): d_res [l][N] -> d_out N/2 complex
// values (coefficient k in the real part of entry k, coefficient k + N/2 in its imaginary part), centred and multiplied by
// inv_scale. d_tab: the level's constants as 64-bit little-endian words, hat [l][l] | inv [l] | Q [l] | floor(Q/2) [l].
extern "C" int b2_decode_compose(b2_ctx *c, size_t l, const uint64_t *d_res, const uint64_t *d_tab, double inv_scale, void *d_out, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_res || !d_tab || !d_out) return fail(B2_EINVAL, "decode_compose: null pointer");
    if (l > (size_t)b2::B2_CRT_MAX_LIMBS) return fail(B2_ESIZE, "decode_compose: more than 64 limbs");
    LaunchScope ls(c, (cudaStream_t)stream, "decode_compose");
    b2::decode_compose_kernel<<<(unsigned)((c->N + 127) / 128), 128, 0, (cudaStream_t)stream>>>(d_res, d_tab, c->d_mod, (uint32_t)c->N, (uint32_t)l, inv_scale,
                                                                                              (double2 *)d_out);
    LAUNCH_CHECK("decode_compose_kernel");
    return B2_OK;
}

// Sampling on the device from a ChaCha20 keystream (sampler.cuh): kind 0 = uniform residues of n_limbs limbs starting at prime
// first_prime (d_out uint64 [n_limbs][N]), kind 1 = centred-binomial error, kind 2 = uniform ternary (d_out int64 [N], signed
// coefficients for b2_expand_signed). key: 32 bytes, nonce: 12 bytes, both read on the host at call time; a (key, nonce) pair
// must never be used for two draws.
extern "C" int b2_sample(b2_ctx *c, int kind, const uint8_t *key32, const uint8_t *nonce12, size_t first_prime, size_t n_limbs, void *d_out,
                         void *stream) {
    CHECK_CTX(c);
    if (!key32 || !nonce12 || !d_out || kind < 0 || kind > 2) return fail(B2_EINVAL, "sample: bad argument");
    if (kind == 0 && (n_limbs < 1 || first_prime + n_limbs > c->size_QP)) return fail(B2_EINVAL, "sample: limb range outside the modulus chain");
    b2::ChaChaKey k;
    memcpy(k.k, key32, 32);
    memcpy(k.n, nonce12, 12);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t blocks = (kind == 0 ? n_limbs : 1) * (c->N / 8);
    if (blocks * (size_t)(b2::B2_SAMPLE_RESERVE + 1) > 0xFFFFFFFFull) return fail(B2_ESIZE, "sample: the draw does not fit the block counter");
    LaunchScope ls(c, s, "sample");
    if (kind == 0)
        b2::sample_uniform_kernel<<<(unsigned)((blocks + 127) / 128), 128, 0, s>>>((uint64_t *)d_out, k, c->d_mod, (uint32_t)first_prime, (uint32_t)c->N,
                                                                                  (uint32_t)blocks);
    else
        b2::sample_small_kernel<<<(unsigned)((blocks + 127) / 128), 128, 0, s>>>((int64_t *)d_out, k, kind, (uint32_t)blocks);
    LAUNCH_CHECK("sample kernel");
    return B2_OK;
}

extern "C" int b2_expand_single_chain(b2_ctx *c, size_t l, const int64_t *d_signed, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    return b2_expand_signed(c, 0, l, d_signed, d_out, 1, stream);
}

extern "C" int b2_expand_single_chain_batch(b2_ctx *c, size_t l, size_t M, const int64_t *d_signed, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (!d_signed || !d_out || M == 0) return fail(B2_EINVAL, "expand_single_chain_batch: bad argument");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = M * l * c->N;
    {
        LaunchScope ls(c, s, "expand_signed");
        expand_signed_batch_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_signed, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)l, (uint32_t)M);
        LAUNCH_CHECK("expand_signed_batch_kernel");
    }
    return run_fwd(c, d_out, d_out, nullptr, (uint32_t)(M * l), 0, EpiStore{}, s, (uint32_t)l);
}

extern "C" int b2_poly_op(b2_ctx *c, int op, size_t n_limbs, const uint64_t *d_a, const uint64_t *d_b, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    if (op < 0 || op > 3 || !d_a || !d_out || (op != 3 && !d_b) || n_limbs < 1 || n_limbs > c->size_QP) return fail(B2_EINVAL, "poly_op: bad argument");
    const size_t n = n_limbs * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "poly_op");
    poly_op_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(op, d_a, d_b, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)n_limbs,
                                                                                   (uint32_t)n_limbs, 0);
    LAUNCH_CHECK("poly_op_kernel");
    return B2_OK;
}

extern "C" int b2_ct_op(b2_ctx *c, int op, size_t l, size_t n_poly, const uint64_t *d_a, const uint64_t *d_b, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    if (op < 0 || op > 3 || !d_a || !d_out || (op != 3 && !d_b) || l < 1 || l > c->size_QP || n_poly < 1 || n_poly > 3)
        return fail(B2_EINVAL, "ct_op: bad argument");
    const size_t n = n_poly * l * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "poly_op");
    poly_op_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(op, d_a, d_b, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)(n_poly * l),
                                                                                   (uint32_t)l, op == 2);
    LAUNCH_CHECK("poly_op_kernel");
    return B2_OK;
}

extern "C" int b2_poly_scalar(b2_ctx *c, int op, size_t n_limbs, const uint64_t *d_a, const uint64_t *h_scalars, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    if (op < 0 || op > 1 || !d_a || !d_out || !h_scalars || n_limbs < 1 || n_limbs > c->size_QP || n_limbs > 64)
        return fail(B2_EINVAL, "poly_scalar: bad argument");
    ScalarTab tab;
    for (size_t i = 0; i < n_limbs; i++) {
        if (h_scalars[i] >= c->q[i]) return fail(B2_EINVAL, "poly_scalar: scalar not reduced");
        tab.v[i] = h_scalars[i];
    }
    const size_t n = n_limbs * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "poly_scalar");
    poly_scalar_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(op, d_a, tab, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)n_limbs,
                                                                                       (uint32_t)n_limbs);
    LAUNCH_CHECK("poly_scalar_kernel");
    return B2_OK;
}

extern "C" int b2_ct_scalar(b2_ctx *c, size_t l, size_t n_poly, const uint64_t *d_a, const uint64_t *h_scalars, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    if (!d_a || !d_out || !h_scalars || l < 1 || l > c->size_QP || l > 64 || n_poly < 1 || n_poly > 3) return fail(B2_EINVAL, "ct_scalar: bad argument");
    ScalarTab tab;
    for (size_t i = 0; i < l; i++) {
        if (h_scalars[i] >= c->q[i]) return fail(B2_EINVAL, "ct_scalar: scalar not reduced");
        tab.v[i] = h_scalars[i];
    }
    const size_t n = n_poly * l * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "poly_scalar");
    poly_scalar_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(1, d_a, tab, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)(n_poly * l),
                                                                                       (uint32_t)l);
    LAUNCH_CHECK("poly_scalar_kernel");
    return B2_OK;
}

extern "C" int b2_ct_lincomb(b2_ctx *c, size_t l, size_t n_poly, size_t n_terms, const uint64_t *const *h_terms, const uint32_t *h_term_limbs,
                             const uint64_t *h_scalars, const uint64_t *h_const, uint64_t *d_out, void *stream) {
    CHECK_CTX(c);
    if (!h_terms || !h_term_limbs || !h_scalars || !d_out || l < 1 || l > c->size_QP || l > B2_LINCOMB_MAX_LIMBS || n_poly < 1 || n_poly > 3 ||
        n_terms < 1 || n_terms > B2_LINCOMB_MAX_TERMS)
        return fail(B2_EINVAL, "ct_lincomb: bad argument (at most 8 terms and 32 limbs)");
    LincombArgs a;
    memset(&a, 0, sizeof(a));
    for (size_t t = 0; t < n_terms; t++) {
        if (!h_terms[t] || h_term_limbs[t] < l) return fail(B2_EINVAL, "ct_lincomb: a term is missing or below the output level");
        a.x[t] = h_terms[t];
        a.lt[t] = h_term_limbs[t];
        for (size_t i = 0; i < l; i++) {
            if (h_scalars[t * l + i] >= c->q[i]) return fail(B2_EINVAL, "ct_lincomb: scalar not reduced");
            a.s[t][i] = h_scalars[t * l + i];
        }
    }
    for (size_t i = 0; i < l && h_const; i++) {
        if (h_const[i] >= c->q[i]) return fail(B2_EINVAL, "ct_lincomb: constant not reduced");
        a.c[i] = h_const[i];
    }
    const size_t n = n_poly * l * c->N;
    LaunchScope ls(c, (cudaStream_t)stream, "lincomb");
    lincomb_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, d_out, c->d_mod, (uint32_t)c->N, (uint32_t)l, (uint32_t)n_poly,
                                                                                   (uint32_t)n_terms);
    LAUNCH_CHECK("lincomb_kernel");
    return B2_OK;
}

// ------------------------------------------------------------------------------------------------
// per-kernel timing for the benchmark
// ------------------------------------------------------------------------------------------------
extern "C" int b2_device_status(b2_ctx *c, uint32_t *status) {
    CHECK_CTX(c);
    if (!status) return fail(B2_EINVAL, "device_status: null pointer");
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemcpy(status, c->d_err, 4, cudaMemcpyDeviceToHost));
    return B2_OK;
}

extern "C" int b2_profile_start(b2_ctx *c) {
    CHECK_CTX(c);
    for (auto &r : c->prof) {
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    c->prof.clear();
    c->profiling = true;
    return B2_OK;
}

extern "C" int b2_profile_stop(b2_ctx *c, char *names, size_t names_cap, float *total_ms, uint32_t *launches, size_t cap, size_t *n_out) {
    CHECK_CTX(c);
    if (!names || !total_ms || !launches || !n_out) return fail(B2_EINVAL, "profile_stop: null pointer");
    c->profiling = false;
    CUDA_TRY(cudaDeviceSynchronize());
    std::vector<std::string> order;
    std::map<std::string, std::pair<float, uint32_t>> agg;
    for (auto &r : c->prof) {
        float ms = 0;
        cudaEventElapsedTime(&ms, r.e0, r.e1);
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
        if (!agg.count(r.name)) order.push_back(r.name);
        agg[r.name].first += ms;
        agg[r.name].second += 1;
    }
    c->prof.clear();
    std::string joined;
    size_t n = 0;
    for (auto &nm : order) {
        if (n >= cap) break;
        joined += nm + ";";
        total_ms[n] = agg[nm].first;
        launches[n] = agg[nm].second;
        n++;
    }
    if (joined.size() + 1 > names_cap) return fail(B2_EINVAL, "profile_stop: name buffer too small");
    memcpy(names, joined.c_str(), joined.size() + 1);
    *n_out = n;
    return B2_OK;
}

// ------------------------------------------------------------------------------------------------
// RNS-limb sharding of one key switch over several GPUs
// ------------------------------------------------------------------------------------------------
// Rank r of G owns the Q limbs [r l / G, (r+1) l / G) and the P limbs [r alpha / G, (r+1) alpha / G)
// of every buffer. Transforms, the inner product and all elementwise work are limb-local; the two
// base conversions need every input limb of a coefficient, so the caller all-gathers (NCCL) between
// the phases below:
//   phase 0: t[own Q] = INTT(c2[own Q]) * (Q_d/q_i)^-1          -> all-gather t (l limbs)
//   phase 1: up[d][own] = NTT(bconv_d(t)); inner product on the own limbs: ct[own Q] += acc P^-1,
//            cxP[k][own P] = INTT(acc) * (P/p_i)^-1               -> all-gather cxP (2 alpha limbs)
//   phase 2: ct[own Q] -= NTT(bconv(cxP) with the P^-1-carrying matrix)
// The results on the own limbs are the same residues the unsharded key switch produces.
static void shard_range(size_t n, int rank, int world, uint32_t *begin, uint32_t *count) {
    const size_t b = n * (size_t)rank / world, e = n * (size_t)(rank + 1) / world;
    *begin = (uint32_t)b;
    *count = (uint32_t)(e - b);
}

static int build_shard_level(b2_ctx *c, size_t l) {
    const size_t alpha = c->size_P, sQ = c->size_Q, beta = (l + alpha - 1) / alpha, lP = l + alpha;
    b2_ctx::ShardPlan &sp = c->shard[l];
    shard_range(l, c->shard_rank, c->shard_world, &sp.q0, &sp.nq);
    shard_range(alpha, c->shard_rank, c->shard_world, &sp.p0, &sp.np);
    auto owned = [&](size_t t) { return t < l ? (t >= sp.q0 && t < sp.q0 + sp.nq) : (t - l >= sp.p0 && t - l < sp.p0 + sp.np); };
    std::vector<Job> jobs_up, jobs_di, jobs_dn, jobs_di_b;
    std::vector<BconvGroup> grp_up(beta), grp_dn(2);
    std::vector<uint2> outs_up, outs_dn;
    std::vector<uint64_t> mat_up, mat_dn;
    std::vector<double> matd_up, matd_dn;
    uint32_t p_pieces = 2;
    for (size_t i = 0; i < alpha; i++) p_pieces = std::max(p_pieces, h_npieces(c->q[sQ + i]));
    for (size_t d = 0; d < beta; d++) {
        const size_t s0 = alpha * d, e0 = std::min(s0 + alpha, l), ni = e0 - s0;
        uint32_t in_pieces = 2;
        for (size_t i = s0; i < e0; i++) in_pieces = std::max(in_pieces, h_npieces(c->q[i]));
        const uint32_t begin = (uint32_t)outs_up.size(), moff = (uint32_t)mat_up.size();
        for (size_t t = 0; t < lP; t++) {
            if ((t >= s0 && t < e0) || !owned(t)) continue;
            const uint32_t pp = phys_prime(c, l, t);
            jobs_up.push_back(make_uint4((uint32_t)(d * lP + t), pp, 0, 0));
            outs_up.push_back(make_uint2((uint32_t)t, pp));
            for (size_t i = s0; i < e0; i++) {
                const uint64_t m = punctured(c->q, s0, e0, i, c->q[pp]);
                double pc[3];
                h_pieces(m, c->q[pp], pc);
                mat_up.push_back(m);
                matd_up.insert(matd_up.end(), pc, pc + 3);
            }
        }
        grp_up[d] = BconvGroup{(uint32_t)s0, (uint32_t)ni, moff, begin, (uint32_t)outs_up.size() - begin, (uint32_t)(d * lP),
                               (uint32_t)(d * lP + s0), in_pieces};
    }
    for (size_t j = sp.q0; j < sp.q0 + sp.nq; j++) {
        outs_dn.push_back(make_uint2((uint32_t)j, (uint32_t)j));
        const uint64_t qj = c->q[j];
        uint64_t P = 1;
        for (size_t i = 0; i < alpha; i++) P = h_mulmod(P, c->q[sQ + i] % qj, qj);
        const uint64_t Pinv = h_invmod(P, qj);
        for (size_t i = 0; i < alpha; i++) {
            const uint64_t m = h_mulmod(punctured(c->q, sQ, c->size_QP, sQ + i, qj), Pinv, qj);
            double pc[3];
            h_pieces(m, qj, pc);
            mat_dn.push_back(m);
            matd_dn.insert(matd_dn.end(), pc, pc + 3);
        }
    }
    for (size_t k = 0; k < 2; k++) {
        for (size_t i = sp.p0; i < sp.p0 + sp.np; i++) {
            jobs_di.push_back(make_uint4((uint32_t)(k * alpha + i), (uint32_t)(sQ + i), (uint32_t)i, (uint32_t)(k * alpha + i)));
            jobs_di_b.push_back(make_uint4((uint32_t)(2 * i + k), (uint32_t)(sQ + i), (uint32_t)i, (uint32_t)(2 * i + k)));
        }
        for (size_t j = sp.q0; j < sp.q0 + sp.nq; j++)
            jobs_dn.push_back(make_uint4((uint32_t)(k * l + j), (uint32_t)j, 0, (uint32_t)(k * l + j)));
        grp_dn[k] = BconvGroup{(uint32_t)(k * alpha), (uint32_t)alpha, 0, 0, sp.nq, (uint32_t)(k * l), 0, p_pieces};
    }
    sp.n_up_ntt = (uint32_t)jobs_up.size();
    // one blob
    auto al = [](size_t b) { return (b + 255) & ~size_t(255); };
    const size_t sz[] = {al(jobs_up.size() * sizeof(Job)), al(jobs_di.size() * sizeof(Job)), al(jobs_dn.size() * sizeof(Job)),
                         al(grp_up.size() * sizeof(BconvGroup)), al(grp_dn.size() * sizeof(BconvGroup)), al(outs_up.size() * sizeof(uint2)),
                         al(outs_dn.size() * sizeof(uint2)), al(mat_up.size() * 8), al(mat_dn.size() * 8), al(matd_up.size() * 8),
                         al(matd_dn.size() * 8), al(jobs_di_b.size() * sizeof(Job))};
    const void *srcs[] = {jobs_up.data(), jobs_di.data(), jobs_dn.data(), grp_up.data(), grp_dn.data(), outs_up.data(),
                          outs_dn.data(), mat_up.data(), mat_dn.data(), matd_up.data(), matd_dn.data(), jobs_di_b.data()};
    const size_t raw[] = {jobs_up.size() * sizeof(Job), jobs_di.size() * sizeof(Job), jobs_dn.size() * sizeof(Job),
                          grp_up.size() * sizeof(BconvGroup), grp_dn.size() * sizeof(BconvGroup), outs_up.size() * sizeof(uint2),
                          outs_dn.size() * sizeof(uint2), mat_up.size() * 8, mat_dn.size() * 8, matd_up.size() * 8, matd_dn.size() * 8,
                          jobs_di_b.size() * sizeof(Job)};
    size_t total = 256;
    for (size_t x : sz) total += x;
    CUDA_TRY(cudaMalloc(&sp.blob, total));
    char *base = (char *)sp.blob;
    void *dptr[12];
    size_t off = 0;
    for (int i = 0; i < 12; i++) {
        dptr[i] = base + off;
        if (raw[i]) CUDA_TRY(cudaMemcpy(dptr[i], srcs[i], raw[i], cudaMemcpyHostToDevice));
        off += sz[i];
    }
    sp.jobs_up_ntt = (Job *)dptr[0];
    sp.jobs_dn_intt = (Job *)dptr[1];
    sp.jobs_dn_ntt = (Job *)dptr[2];
    sp.grp_up = (BconvGroup *)dptr[3];
    sp.grp_dn = (BconvGroup *)dptr[4];
    sp.outs_up = (uint2 *)dptr[5];
    sp.outs_dn = (uint2 *)dptr[6];
    sp.mat_up = (uint64_t *)dptr[7];
    sp.mat_dn = (uint64_t *)dptr[8];
    sp.matd_up = (double *)dptr[9];
    sp.matd_dn = (double *)dptr[10];
    sp.jobs_dn_intt_b = (Job *)dptr[11];
    if (c->bconv_tc) {
        // tensor-core jobs over the rank's outputs (a rank may own no output of a digit, or no Q limb at all)
        TcBuild tb;
        tb.max_groups = c->tc_max_groups;
        std::vector<TcSpecOut> outs;
        uint32_t n_up = 0, n_dn = 0, n_dn_b = 0;
        for (size_t d = 0; d < beta; d++) {
            const BconvGroup &g = grp_up[d];
            if (g.n_out == 0) continue;
            outs.clear();
            for (uint32_t j = 0; j < g.n_out; j++) {
                const uint2 o = outs_up[g.out_begin + j];
                outs.push_back(TcSpecOut{g.out_slot_base + o.x, c->q[o.y], mat_up.data() + g.mat_off + (size_t)j * g.ni});
            }
            n_up += tb.add(g.in_slot0, g.ni, 0xFFFFFFFFu, outs);
        }
        for (size_t k = 0; k < 2 && sp.nq; k++) {
            outs.clear();
            for (uint32_t j = 0; j < sp.nq; j++) outs.push_back(TcSpecOut{(uint32_t)(k * l) + sp.q0 + j, c->q[sp.q0 + j], mat_dn.data() + (size_t)j * alpha});
            n_dn += tb.add((uint32_t)(k * alpha), (uint32_t)alpha, 0xFFFFFFFFu, outs);
        }
        for (size_t k = 0; k < 2 && sp.nq; k++) {  // the same conversion reading P limb i of polynomial k at slot 2 i + k
            outs.clear();
            for (uint32_t j = 0; j < sp.nq; j++) outs.push_back(TcSpecOut{(uint32_t)(k * l) + sp.q0 + j, c->q[sp.q0 + j], mat_dn.data() + (size_t)j * alpha});
            n_dn_b += tb.add((uint32_t)k, (uint32_t)alpha, 0xFFFFFFFFu, outs, 2);
        }
        if (!tb.ok) return fail(B2_EINVAL, "tensor-core base conversion: unsupported prime in the chain");
        if (n_up + n_dn) {
            int rc = tc_upload(tb, &sp.tc_blob, {{&sp.tc_up, {0u, n_up}}, {&sp.tc_dn, {n_up, n_dn}}, {&sp.tc_dn_b, {n_up + n_dn, n_dn_b}}});
            if (rc) return rc;
        }
    }
    return B2_OK;
}

extern "C" int b2_ctx_set_shard(b2_ctx *c, int rank, int world) {
    CHECK_CTX(c);
    if (world < 1 || rank < 0 || rank >= world) return fail(B2_EINVAL, "set_shard: rank must be in [0, world)");
    CUDA_TRY(cudaDeviceSynchronize());
    for (auto &sp : c->shard) {
        cudaFree(sp.blob);
        cudaFree(sp.tc_blob);
    }
    c->shard.clear();
    c->shard_rank = rank;
    c->shard_world = world;
    c->shard.resize(c->size_Q + 1);
    for (size_t l = 1; l <= c->size_Q; l++) {
        int rc = build_shard_level(c, l);
        if (rc) return rc;
    }
    return B2_OK;
}

extern "C" int b2_shard_limbs(const b2_ctx *c, size_t l, uint32_t *out4) {
    if (!c || !out4 || l < 1 || l > c->size_Q) return fail(B2_EINVAL, "shard_limbs: bad argument");
    if (c->shard.empty()) return fail(B2_EINVAL, "shard_limbs: call b2_ctx_set_shard first");
    const b2_ctx::ShardPlan &sp = c->shard[l];
    out4[0] = sp.q0;
    out4[1] = sp.nq;
    out4[2] = sp.p0;
    out4[3] = sp.np;
    return B2_OK;
}

extern "C" int b2_shard_keyswitch_phase(b2_ctx *c, size_t l, int phase, const uint64_t *d_c2, const uint64_t *const *evk, size_t n_evk,
                                        uint64_t *d_ct, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (c->shard.empty()) return fail(B2_EINVAL, "shard_keyswitch_phase: call b2_ctx_set_shard first");
    if (!d_c2 || !evk || !d_ct || !d_ws) return fail(B2_EINVAL, "shard_keyswitch_phase: null pointer");
    if (ws_bytes < b2_workspace_bytes(c, B2_OP_KEYSWITCH, l)) return fail(B2_EWS, "shard_keyswitch_phase: workspace too small");
    cudaStream_t s = (cudaStream_t)stream;
    const LevelPlan &pl = c->plan[l];
    const b2_ctx::ShardPlan &sp = c->shard[l];
    const size_t N = c->N, a = c->size_P, lP = l + a, beta = pl.beta;
    uint64_t *t = (uint64_t *)d_ws, *up = t + l * N, *cxP = up + beta * lP * N;
    int rc;
    switch (phase) {
        case 0:
            return run_inv(c, d_c2, t, pl.jobs_up_intt + sp.q0, sp.nq, 0, pl.fin_up, s);
        case 1: {
            rc = run_bconv(c, false, t, up, d_c2, sp.grp_up, (uint32_t)beta, sp.outs_up, sp.mat_up, sp.matd_up, (uint32_t)a, (uint32_t)lP, true, s, &sp.tc_up);
            if (rc) return rc;
            rc = run_fwd(c, up, up, sp.jobs_up_ntt, sp.n_up_ntt, 0, EpiStore{}, s);
            if (rc) return rc;
            const uint4 rg = make_uint4(sp.q0, sp.nq, sp.p0, sp.np);
            rc = inner_prod_impl(c, l, up, d_c2, evk, n_evk, cxP, d_ct, true, s, &rg);
            if (rc) return rc;
            return run_inv(c, cxP, cxP, sp.jobs_dn_intt, 2 * sp.np, 0, c->d_fin_P, s);
        }
        case 2:
            if (sp.nq == 0) return B2_OK;
            rc = run_bconv(c, false, cxP, up, nullptr, sp.grp_dn, 2, sp.outs_dn, sp.mat_dn, sp.matd_dn, (uint32_t)a, (uint32_t)l, true, s, &sp.tc_dn);
            if (rc) return rc;
            return run_fwd(c, up, up, sp.jobs_dn_ntt, 2 * sp.nq, 0, EpiSubFrom{d_ct}, s);
        default:
            return fail(B2_EINVAL, "shard_keyswitch_phase: phase must be 0, 1 or 2");
    }
}

// Exchange buffers that the other ranks of one node can write: device memory with a CUDA IPC handle, the peers' mappings of
// it, and plain asynchronous copies into them. The limb-sharded pipeline pushes a rank's block of the exchanged limbs into every
// peer's buffer with these copies (DMA engines over NVLink, no SM involved, so they overlap the transforms of other batches),
// where an all-gather kernel would compete with those transforms for SMs. No kernel of this library reads or writes peer
// memory; nothing here waits on the device.
extern "C" int b2_peer_alloc(size_t bytes, void **d_ptr, uint8_t *handle64) {
    if (!d_ptr || !handle64 || bytes == 0) return fail(B2_EINVAL, "peer_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    CUDA_TRY(cudaMalloc(d_ptr, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, *d_ptr);
    if (e != cudaSuccess) {
        cudaFree(*d_ptr);
        *d_ptr = nullptr;
        return fail((int)e, std::string("peer_alloc: cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    }
    memcpy(handle64, &h, 64);
    return B2_OK;
}

extern "C" int b2_peer_open(const uint8_t *handle64, void **d_ptr) {
    if (!handle64 || !d_ptr) return fail(B2_EINVAL, "peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    CUDA_TRY(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return B2_OK;
}

extern "C" int b2_peer_close(void *d_ptr) {
    if (!d_ptr) return B2_OK;
    CUDA_TRY(cudaIpcCloseMemHandle(d_ptr));
    return B2_OK;
}

extern "C" int b2_peer_free(void *d_ptr) {
    if (!d_ptr) return B2_OK;
    CUDA_TRY(cudaFree(d_ptr));
    return B2_OK;
}

// bytes from this GPU's memory into a peer's mapped buffer (or any two device addresses of the process), on `stream`
extern "C" int b2_peer_copy(void *d_dst, const void *d_src, size_t bytes, void *stream) {
    if (!d_dst || !d_src) return fail(B2_EINVAL, "peer_copy: null pointer");
    if (bytes == 0) return B2_OK;
    CUDA_TRY(cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    return B2_OK;
}

extern "C" size_t b2_shard_batch_workspace_bytes(const b2_ctx *c, size_t l, size_t batch) {
    if (!c || l < 1 || l > c->size_Q || batch < 1) return 0;
    const size_t a = c->size_P, beta = (l + a - 1) / a, lP = l + a;
    return batch * (l + 2 * a + beta * lP) * limb_bytes(c);
}

// The three phases for `batch` ciphertexts at once (one key for all of them): every kernel of a phase is one launch over the
// whole batch, so a rank that owns an eighth of the limbs still fills the GPU. Workspace, in limbs:
//   T   [l][batch]            scaled coefficient form of c2, limb-major: this rank's Q limbs are one contiguous block
//   CXP [alpha][2][batch]     P limbs of both polynomials, limb-major likewise
//   UP  [batch][beta][l+alpha]  ModUp digits (its front also holds ModDown's delta)
// The caller all-gathers T after phase 0 and CXP after phase 1 (one collective each).
extern "C" int b2_shard_keyswitch_phase_batch(b2_ctx *c, size_t l, int phase, size_t batch, const uint64_t *d_c2, const uint64_t *const *evk,
                                              size_t n_evk, uint64_t *d_ct, void *d_ws, size_t ws_bytes, void *stream) {
    CHECK_CTX(c);
    CHECK_LEVEL(c, l);
    if (c->shard.empty()) return fail(B2_EINVAL, "shard_keyswitch_phase_batch: call b2_ctx_set_shard first");
    if (!d_c2 || !evk || !d_ct || !d_ws || batch < 1 || batch > 65535) return fail(B2_EINVAL, "shard_keyswitch_phase_batch: bad argument");
    if (ws_bytes < b2_shard_batch_workspace_bytes(c, l, batch)) return fail(B2_EWS, "shard_keyswitch_phase_batch: workspace too small");
    if (!c->bconv_tc || c->tc_simple) return fail(B2_EINVAL, "shard_keyswitch_phase_batch: needs the persistent tensor-core base conversion");
    cudaStream_t s = (cudaStream_t)stream;
    const LevelPlan &pl = c->plan[l];
    const b2_ctx::ShardPlan &sp = c->shard[l];
    const size_t N = c->N, a = c->size_P, lP = l + a, beta = pl.beta;
    const uint32_t B = (uint32_t)batch, per = (uint32_t)(beta * lP);
    uint64_t *T = (uint64_t *)d_ws, *CXP = T + l * batch * N, *UP = CXP + 2 * a * batch * N;
    int rc;
    switch (phase) {
        case 0:
            return run_inv(c, d_c2, T, pl.jobs_up_intt + sp.q0, sp.nq, 0, pl.fin_up, s, BatchDims{B, 0, (uint32_t)l, B - 1, 1});
        case 1: {
            const TcBatch tb{B, B - 1, 1, 0, per, 0};
            if (sp.tc_up.jobs) {
                rc = run_bconv_tc(c, false, T, UP, nullptr, sp.tc_up, sp.tc_up.n_jobs, s, &tb);
                if (rc) return rc;
            }
            const bool fused = c->use_mac && beta <= B2_MAC_MAX_BETA && n_evk >= beta && (sp.nq + sp.np) > 0;
            if (fused) {
                // column pass of the rank's digit limbs, then the row pass with the inner product inside it (every limb of the
                // rank's slice: its P limbs first), as the one-GPU batched key switch does; the P limbs go straight into the
                // limb-major exchange buffer
                using Cfg = PassCfg<8>;
                NttArgs na{UP, UP, sp.jobs_up_ntt, 0, (uint32_t)c->logN, c->d_tw, c->d_mod, nullptr, 0};
                na.src_bs = na.dst_bs = per;
                if (sp.n_up_ntt) {
                    LaunchScope ls(c, s, "ntt_fwd_cols");
                    ntt_fwd_pass<8, Cfg::R_STRIDED, Cfg::R_CONTIG, Cfg::LOG_CC, true, false, EpiStore>
                        <<<dim3(sp.n_up_ntt * (uint32_t)(N >> (8 + Cfg::LOG_CC)), B), pass_threads<8, true>(), 0, s>>>(na, EpiStore{});
                    LAUNCH_CHECK("ntt_fwd_pass");
                }
                MacArgs m{};
                m.own = d_c2;
                for (size_t d = 0; d < beta; d++) {
                    if (!evk[d]) return fail(B2_EINVAL, "null evaluation-key digit");
                    m.evk[d] = evk[d];
                }
                m.ct = d_ct, m.cxp = CXP, m.pinv = c->d_Pinv, m.fin = c->d_macfin;
                m.l = (uint32_t)l, m.lP = (uint32_t)lP, m.alpha = (uint32_t)a, m.beta = (uint32_t)beta;
                m.size_Q = (uint32_t)c->size_Q, m.size_QP = (uint32_t)c->size_QP;
                m.first_limb = sp.q0, m.p_first = sp.np, m.p_off = sp.p0, m.acc_p = 0, m.interleave = 0;
                m.dig_bs = per, m.own_bs = (uint32_t)l, m.ct_bs = (uint32_t)(2 * l);
                m.cxp_i = 2 * B, m.cxp_k = B, m.cxp_bs = 1;
                LaunchScope ls(c, s, "ntt_fwd_rows_mac");
                ntt_fwd_rows_mac<8, Cfg::R_CONTIG, Cfg::LOG_C>
                    <<<dim3(B, (sp.nq + sp.np) * (uint32_t)(N >> (8 + Cfg::LOG_C))), pass_threads<8>(), mac_smem_bytes<8, Cfg::R_CONTIG, Cfg::LOG_C>(), s>>>(na, m);
                LAUNCH_CHECK("ntt_fwd_rows_mac");
            } else {
                rc = run_fwd(c, UP, UP, sp.jobs_up_ntt, sp.n_up_ntt, 0, EpiStore{}, s, 0, 0, 0, BatchDims{B, 0, per, 0, per});
                if (rc) return rc;
                const uint4 rg = make_uint4(sp.q0, sp.nq, sp.p0, sp.np);
                const IpBatch ib{per, (uint32_t)l, (uint32_t)(2 * l), 2, 1, B - 1, 1};
                rc = inner_prod_impl(c, l, UP, d_c2, evk, n_evk, CXP, d_ct, true, s, &rg, false, B, &ib);
                if (rc) return rc;
            }
            return run_inv(c, CXP, CXP, sp.jobs_dn_intt_b, 2 * sp.np, 0, c->d_fin_P, s, BatchDims{B, B - 1, 1, B - 1, 1});
        }
        case 2: {
            if (sp.nq == 0) return B2_OK;
            const TcBatch tb{B, B - 1, 1, 0, per, 0};
            rc = run_bconv_tc(c, false, CXP, UP, nullptr, sp.tc_dn_b, sp.tc_dn_b.n_jobs, s, &tb);
            if (rc) return rc;
            return run_fwd(c, UP, UP, sp.jobs_dn_ntt, 2 * sp.nq, 0, EpiSubFrom{d_ct, (uint32_t)(2 * l)}, s, 0, 0, 0, BatchDims{B, 0, per, 0, per});
        }
        default:
            return fail(B2_EINVAL, "shard_keyswitch_phase_batch: phase must be 0, 1 or 2");
    }
}
