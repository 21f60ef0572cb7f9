// CPU emulation of the tensor-core base conversion: builds the byte images and group tables with the library's own
// planner (phantom-fhe_b200/csrc/bconv_tc_plan.h), forms A from the raw bytes of the input residues exactly as the
// kernel does, computes D = A x B in int32 from the operand layout the matrix descriptors describe, runs the kernel's
// reduction and compares every output with (sum_i y_i M_ji) mod p_j computed in 128-bit integers.
// Usage: bconv_tc_emul <seed>; prints "ok <cases>" or the first mismatch.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "bconv_tc_plan.h"

typedef unsigned __int128 u128;
static uint64_t rng_state;
static uint64_t rnd() {
    uint64_t z = (rng_state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static uint64_t rnd_odd_bits(int bits) { return ((rnd() >> (64 - bits)) | (1ull << (bits - 1)) | 1ull); }

static uint32_t g_max_groups = 16;
static int run_case(int ni, const std::vector<int> &in_bits, const std::vector<int> &out_bits, bool extremes) {
    std::vector<uint64_t> q(ni), p(out_bits.size());
    for (int i = 0; i < ni; i++) q[i] = rnd_odd_bits(in_bits[i]);
    std::vector<uint64_t> mat(out_bits.size() * ni);
    std::vector<b2::TcSpecOut> outs;
    for (size_t j = 0; j < out_bits.size(); j++) {
        p[j] = rnd_odd_bits(out_bits[j]);
        for (int i = 0; i < ni; i++) mat[j * ni + i] = extremes ? p[j] - 1 : rnd() % p[j];
        outs.push_back(b2::TcSpecOut{(uint32_t)(100 + j), p[j], &mat[j * ni]});
    }
    b2::TcBuild tb;
    tb.max_groups = g_max_groups;
    const uint32_t n_jobs = tb.add(3, (uint32_t)ni, 0xFFFFFFFFu, outs);
    if (!tb.ok || n_jobs == 0) return printf("planner refused a valid case\n"), 1;
    const int ROWS = 128;
    std::vector<uint64_t> y((size_t)ni * ROWS);
    for (int i = 0; i < ni; i++)
        for (int r = 0; r < ROWS; r++) y[(size_t)i * ROWS + r] = (extremes || r == 0) ? q[i] - 1 : (r == 1 ? 0 : rnd() % q[i]);
    // A exactly as the kernel stores it
    std::vector<uint8_t> A(128 * 64, 0);
    for (int r = 0; r < ROWS; r++)
        for (int i = 0; i < 8; i++) {
            const uint64_t v = i < ni ? y[(size_t)i * ROWS + r] : 0;
            memcpy(&A[(r >> 3) * 512 + (i >> 1) * 128 + (r & 7) * 16 + (i & 1) * 8], &v, 8);
        }
    std::vector<char> seen(out_bits.size(), 0);
    for (uint32_t jb = 0; jb < n_jobs; jb++) {
        const b2::TcJob &job = tb.jobs[jb];
        if (job.n_groups < 1 || job.n_groups > g_max_groups || job.alloc_cols < 16 * job.n_groups || (job.alloc_cols & (job.alloc_cols - 1)) || job.alloc_cols < 32 ||
            job.alloc_cols > 512 || (job.img_off & 15))
            return printf("bad job header\n"), 1;
        const uint8_t *B = tb.images.data() + job.img_off;
        for (uint32_t g = 0; g < job.n_groups; g++) {
            const b2::TcGroup &G = tb.groups[job.grp_off + g];
            if (G.nb < 4 || G.nb > 8 || G.n_valid < 1 || G.n_valid > 16 / G.nb) return printf("bad group header\n"), 1;
            for (int r = 0; r < ROWS; r++) {
                uint32_t c[16];
                for (int col = 0; col < 16; col++) {
                    uint32_t acc = 0;
                    for (int k = 0; k < 64; k++) acc += (uint32_t)A[b2::tc_operand_offset(r, k)] * B[b2::tc_operand_offset(16 * g + col, k)];
                    if (acc >= (1u << 22)) return printf("accumulator out of range\n"), 1;
                    c[col] = acc;
                }
                for (uint32_t o = 0; o < G.n_valid; o++) {
                    const b2::TcOut &m = G.o[o];
                    uint64_t got;
                    switch (G.nb) {
                        case 4: got = b2::tc_reduce<4>(&c[o * 4], m.p, m.mu); break;
                        case 5: got = b2::tc_reduce<5>(&c[o * 5], m.p, m.mu); break;
                        case 6: got = b2::tc_reduce<6>(&c[o * 6], m.p, m.mu); break;
                        case 7: got = b2::tc_reduce<7>(&c[o * 7], m.p, m.mu); break;
                        default: got = b2::tc_reduce<8>(&c[o * 8], m.p, m.mu); break;
                    }
                    uint64_t lean;
                    const uint32_t plo = (uint32_t)m.p, phi = (uint32_t)(m.p >> 32);
                    switch (G.nb) {
                        case 4: lean = b2::tc_reduce_dev<4>(&c[o * 4], plo, phi, m.mu); break;
                        case 5: lean = b2::tc_reduce_dev<5>(&c[o * 5], plo, phi, m.mu); break;
                        case 6: lean = b2::tc_reduce_dev<6>(&c[o * 6], plo, phi, m.mu); break;
                        case 7: lean = b2::tc_reduce_dev<7>(&c[o * 7], plo, phi, m.mu); break;
                        default: lean = b2::tc_reduce_dev<8>(&c[o * 8], plo, phi, m.mu); break;
                    }
                    if (lean != got) return printf("the two forms of the reduction disagree\n"), 1;
                    const size_t j = m.slot - 100;
                    if (j >= out_bits.size() || m.p != p[j]) return printf("bad output record\n"), 1;
                    seen[j] = 1;
                    u128 want = 0;
                    for (int i = 0; i < ni; i++) want += (u128)y[(size_t)i * ROWS + r] * mat[j * ni + i];
                    if (got != (uint64_t)(want % p[j])) return printf("mismatch: ni=%d nb=%u row=%d out=%zu\n", ni, G.nb, r, j), 1;
                }
            }
        }
    }
    for (char s : seen)
        if (!s) return printf("an output was never produced\n"), 1;
    return 0;
}

int main(int argc, char **argv) {
    rng_state = argc > 1 ? strtoull(argv[1], nullptr, 10) : 1;
    int cases = 0;
    // the headline shapes: ModDown (8 x 60-bit in; 60-bit + 23 x 40-bit out), ModUp digits
    std::vector<int> p60(8, 60), p40(8, 40);
    std::vector<int> dn_out{60};
    for (int i = 0; i < 23; i++) dn_out.push_back(40);
    std::vector<int> up0_out(16, 40), up1_out{60};
    for (int i = 0; i < 8; i++) up0_out.push_back(60);
    for (int i = 0; i < 15; i++) up1_out.push_back(40);
    for (int i = 0; i < 8; i++) up1_out.push_back(60);
    std::vector<int> in_d0{60, 40, 40, 40, 40, 40, 40, 40};
    for (uint32_t mg : {16u, 8u, 3u}) {   // column groups per job: the default, the four-CTAs-per-SM split, a tiny one
        g_max_groups = mg;
        for (int ex = 0; ex < 2; ex++) {
            if (run_case(8, p60, dn_out, ex) || run_case(8, in_d0, up0_out, ex) || run_case(8, p40, up1_out, ex)) return 1;
            cases += 3;
        }
    }
    g_max_groups = 16;
    // every byte count, ragged inputs, more outputs than one job holds, 61-bit primes
    for (int bits = 17; bits <= 61; bits++) {
        std::vector<int> out(5, bits);
        out.push_back(61);
        out.push_back(17 + (bits * 7) % 45);
        for (int ni = 1; ni <= 8; ni += (bits % 3) + 1) {
            std::vector<int> in(ni, 17 + (bits * 11 + ni * 5) % 45);
            in[0] = 61;
            if (run_case(ni, in, out, bits & 1)) return 1;
            cases++;
        }
    }
    std::vector<int> many;
    for (int i = 0; i < 70; i++) many.push_back(i % 2 ? 60 : 36);
    if (run_case(8, p60, many, false) || run_case(3, std::vector<int>{50, 50, 50}, many, true)) return 1;
    cases += 2;
    printf("ok %d\n", cases);
    return 0;
}
