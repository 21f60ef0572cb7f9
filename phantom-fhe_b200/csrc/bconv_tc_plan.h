// bconv_tc_plan.h - data structures and host-side planning of the tensor-core base conversion (kernel: bconv_tc.cuh).
// Plain C++: also compiled by the CPU test-suite, which emulates the matrix product on the byte images built here.
//
// The conversion (src/rns_bconv.cu:143-168, 455-485; include/rns_bconv.cuh:112-125)
//     out_j[n] = (sum_i y_i[n] * M_ji) mod p_j,      i < ni <= 8 inputs, j over the group's outputs
// is one small u8 x u8 -> s32 matrix product per tile of 128 coefficients:
//   * a residue is its own little-endian bytes, y_i = sum_a 2^(8a) y_{i,a}, so the eight uint64 input
//     limbs of a coefficient ARE the K = 64 bytes of its row of A (row = coefficient, k = 8 i + a);
//   * the weight of the input byte is folded into the matrix modulo the output prime:
//         sum_i y_i M_ji  =  sum_{i,a} y_{i,a} * (2^(8a) M_ji mod p_j)      (mod p_j),
//     and that constant, below p_j, is split into its nb_j bytes: column (j, b) of B holds byte b;
//   * D[n][(j,b)] = sum_k A[n][k] B[k][(j,b)] < 64 * 255^2 < 2^22 is exact in int32, and
//         V_j = sum_b D[n][(j,b)] 2^(8b)  =  out_j[n]  (mod p_j),   V_j < 2^(8 nb_j + 14.01).
// The epilogue shift-adds nb_j (4 to 8) int32 words into one 64- or 96-bit integer and reduces it once:
// quotient estimate from the top 32 bits times a 32-bit reciprocal (never above the true quotient, at most
// one below), one conditional subtraction. Canonical residues are unique, so the limbs equal those of the
// integer and FP64 kernels bit for bit.
//
// Outputs are packed into groups of 16 accumulator columns holding floor(16 / nb) outputs of equal byte count nb;
// a job (a digit of ModUp, a polynomial of ModDown) has at most 16 groups = 256 columns. A and B are laid out in
// the canonical K-major no-swizzle form of the sm_100 shared-memory matrix descriptor (8-row x 16-byte core matrices):
//     offset(row, k) = (row / 8) * 512 + (k / 16) * 128 + (row % 8) * 16 + k % 16.
#pragma once
#include <algorithm>
#include <cstdint>
#include <utility>
#include <vector>

#if defined(__CUDACC__)
#define B2_HD __host__ __device__ __forceinline__
#else
#define B2_HD inline
#endif

namespace b2 {

struct TcOut {
    uint64_t p;     // output prime
    uint32_t mu;    // floor(2^(8 nb + 15) / p)
    uint32_t slot;  // output limb (absolute slot in the output buffer)
};
struct TcGroup {
    uint32_t nb;       // bytes per output of this group (4..8)
    uint32_t n_valid;  // outputs present (1 .. 16 / nb)
    uint32_t pad0, pad1;
    TcOut o[4];
};
struct TcJob {
    uint32_t in_slot0, ni;     // first input limb, number of input limbs (<= 8)
    uint32_t copy_dst_slot0;   // ModUp: where the digit's own limbs are copied to (0xFFFFFFFF: no copy)
    uint32_t n_groups;         // column groups (<= 16)
    uint32_t img_off;          // byte offset of the B image (n_groups * 1024 bytes)
    uint32_t grp_off;          // first TcGroup of the job
    uint32_t alloc_cols;       // TMEM columns to allocate: power of two >= max(32, 16 n_groups)
    uint32_t in_stride1;       // input limb i sits at slot in_slot0 + i * (in_stride1 + 1)
};
static_assert(sizeof(TcOut) == 16 && sizeof(TcGroup) == 80 && sizeof(TcJob) == 32, "device layouts");

// byte offset of element (row, k) of a K-major no-swizzle operand with K = 64 bytes
B2_HD uint32_t tc_operand_offset(uint32_t row, uint32_t k) { return (row / 8) * 512 + (k / 16) * 128 + (row % 8) * 16 + k % 16; }

// sum_b c[b] 2^(8b) mod p for NB words below 2^22 each; mu = floor(2^(8 NB + 15) / p)
template <int NB>
B2_HD uint64_t tc_reduce(const uint32_t *c, uint64_t p, uint32_t mu) {
    static_assert(NB >= 4 && NB <= 8, "4 to 8 bytes per output prime");
    constexpr int SH = 8 * NB - 17;  // V >> SH fits 32 bits
    const uint32_t x0 = c[0] + (c[1] << 8), x1 = c[2] + (c[3] << 8);
    uint64_t vlo;  // V mod 2^64
    uint32_t vh;   // V >> SH
    if constexpr (NB <= 6) {
        const uint32_t x2 = NB == 4 ? 0u : (NB == 5 ? c[4] : c[4] + (c[5] << 8));
        vlo = (uint64_t)x0 + ((uint64_t)x1 << 16) + ((uint64_t)x2 << 32);
        vh = (uint32_t)(vlo >> SH);
    } else {
        const uint32_t x2 = c[4] + (c[5] << 8), x3 = NB == 7 ? c[6] : c[6] + (c[7] << 8);
        const uint64_t a = (uint64_t)x0 + ((uint64_t)x1 << 16), b = (uint64_t)x2 + ((uint64_t)x3 << 16);
        const uint64_t mid = (a >> 32) + b;  // V >> 32, below 2^47
        vlo = (a & 0xFFFFFFFFull) | (mid << 32);
        vh = (uint32_t)(mid >> (SH - 32));
    }
    const uint32_t qhat = (uint32_t)(((uint64_t)vh * mu) >> 32);
    const uint64_t r = vlo - (uint64_t)qhat * p;  // true value in [0, 2p), below 2^62: the wrap-around is harmless
    return r >= p ? r - p : r;
}

// tc_reduce with the prime as two words and the last subtraction chosen by the sign of (r - p): r < 2p < 2^62
template <int NB>
B2_HD uint64_t tc_reduce_dev(const uint32_t *c, uint32_t p_lo, uint32_t p_hi, uint32_t mu) {
    constexpr int SH = 8 * NB - 17;
    const uint32_t x0 = c[0] + (c[1] << 8), x1 = c[2] + (c[3] << 8);
    uint64_t vlo;
    uint32_t vh;
    if constexpr (NB <= 6) {
        const uint32_t x2 = NB == 4 ? 0u : (NB == 5 ? c[4] : c[4] + (c[5] << 8));
        vlo = (uint64_t)x1 * 65536u + x0;               // one wide multiply-add
        vlo += (uint64_t)x2 << 32;                      // touches the high word only
        vh = (uint32_t)(vlo >> SH);
    } else {
        const uint32_t x2 = c[4] + (c[5] << 8), x3 = NB == 7 ? c[6] : c[6] + (c[7] << 8);
        const uint64_t a = (uint64_t)x1 * 65536u + x0, b = (uint64_t)x3 * 65536u + x2;
        const uint64_t mid = (a >> 32) + b;
        vlo = (a & 0xFFFFFFFFull) | (mid << 32);
        vh = (uint32_t)(mid >> (SH - 32));
    }
    const uint32_t qhat = (uint32_t)(((uint64_t)vh * mu) >> 32);
    const uint64_t p = ((uint64_t)p_hi << 32) | p_lo;
    const uint64_t r = vlo - ((uint64_t)qhat * p_lo + ((uint64_t)(qhat * p_hi) << 32));
    const uint64_t t = r - p;
    return (int64_t)t < 0 ? r : t;
}

struct TcSpecOut {
    uint32_t slot;        // absolute output limb
    uint64_t p;           // its prime
    const uint64_t *row;  // M[j][0..ni)
};

static inline uint32_t tc_nbytes(uint64_t p) { return std::max(4u, (uint32_t)((64 - __builtin_clzll(p) + 7) / 8)); }

struct TcBuild {
    std::vector<TcJob> jobs;
    std::vector<TcGroup> groups;
    std::vector<uint8_t> images;
    bool ok = true;
    uint32_t max_groups = 16;  // column groups per job: 16 -> up to 256 TMEM columns (two CTAs per SM), 8 -> 128 (four)
    // One conversion (a digit, a polynomial): outputs are packed, in order, into 16-column groups of equal byte count;
    // more than max_groups groups are dealt evenly over further jobs on the same inputs. Returns the number of jobs added.
    uint32_t add(uint32_t in_slot0, uint32_t ni, uint32_t copy_dst, const std::vector<TcSpecOut> &outs, uint32_t in_stride = 1) {
        if (ni < 1 || ni > 8 || outs.empty()) {
            ok = false;
            return 0;
        }
        uint32_t added = 0;
        size_t i = 0;
        // groups the outputs need in all -> jobs of equal size
        uint32_t total_groups = 0;
        for (size_t k = 0; k < outs.size();) {
            const uint32_t nb = tc_nbytes(outs[k].p), opg = 16 / nb;
            uint32_t cnt = 0;
            while (k < outs.size() && cnt < opg && tc_nbytes(outs[k].p) == nb) cnt++, k++;
            total_groups++;
        }
        const uint32_t cap = std::max(1u, std::min(max_groups, 16u));
        const uint32_t n_split = (total_groups + cap - 1) / cap, per_job = (total_groups + n_split - 1) / n_split;
        while (i < outs.size()) {
            TcJob job{in_slot0, ni, added == 0 ? copy_dst : 0xFFFFFFFFu, 0, (uint32_t)images.size(), (uint32_t)groups.size(), 32, in_stride - 1};
            std::vector<std::pair<size_t, uint32_t>> placed;  // (output index, first column) of this job
            while (i < outs.size() && job.n_groups < per_job) {
                const uint32_t nb = tc_nbytes(outs[i].p), opg = 16 / nb;
                TcGroup g{};
                g.nb = nb;
                while (i < outs.size() && g.n_valid < opg && tc_nbytes(outs[i].p) == nb) {
                    const uint64_t p = outs[i].p;
                    const unsigned __int128 mu = ((unsigned __int128)1 << (8 * nb + 15)) / p;
                    if (p <= (1ull << 16) || (mu >> 32)) ok = false;
                    g.o[g.n_valid] = TcOut{p, (uint32_t)mu, outs[i].slot};
                    placed.push_back({i, 16 * job.n_groups + g.n_valid * nb});
                    g.n_valid++;
                    i++;
                }
                groups.push_back(g);
                job.n_groups++;
            }
            const size_t img0 = images.size();
            images.resize(img0 + (size_t)job.n_groups * 1024, 0);
            for (auto &pl : placed) {
                const TcSpecOut &o = outs[pl.first];
                const uint32_t nb = tc_nbytes(o.p);
                for (uint32_t ii = 0; ii < ni; ii++)
                    for (uint32_t a = 0; a < 8; a++) {
                        const uint64_t e = (uint64_t)((((unsigned __int128)(o.row[ii] % o.p)) << (8 * a)) % o.p);
                        const uint32_t k = 8 * ii + a;
                        for (uint32_t b = 0; b < nb; b++) {
                            const uint32_t row = pl.second + b;
                            images[img0 + tc_operand_offset(row, k)] = (uint8_t)(e >> (8 * b));
                        }
                    }
            }
            uint32_t cols = 32;
            while (cols < 16 * job.n_groups) cols <<= 1;
            job.alloc_cols = cols;
            jobs.push_back(job);
            added++;
        }
        return added;
    }
};

}  // namespace b2
