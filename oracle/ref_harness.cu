// ref_harness.cu - drives the UNMODIFIED reference library (oracle/_ref/libPhantom.so) on
// synthetic limbs and records per-limb content hashes of every stage of the key-switching
// path. TEST INFRASTRUCTURE ONLY: its JSON output is what tests/golden/ holds and what pins the
// CPU oracle (ckks_oracle.c, compiled into this binary for the data generator and the hash).
//
// usage: ref_harness --logn 12 --bits 50,36,36,36,36,36,50,50 --special 2 --level 6 --seed 7
//                    --steps 1,2,-1 --out case.json [--time ITERS [--threads T]]
//        ref_harness --bootstrap DIR [--boot-dense 1]   the reference's own bootstrap on its test's chain (N = 2^16):
//                    milliseconds, its decode's error, and the key / result / message files for decoding elsewhere
//        ref_harness --selftest 1 --logn .. --bits .. --special ..   encode -> decode and encrypt -> decrypt -> decode
// Needs a CUDA device (the reference has no CPU path for any of this).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <algorithm>
#include <atomic>
#include <chrono>
#include <fstream>
#include <functional>
#include <random>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "phantom.h"
#include "bsgs.h"
#include "bootstrap.h"
#include "ckks_oracle.h"

using namespace phantom;
using namespace phantom::arith;
using namespace phantom::util;

static std::vector<int> parse_ints(const char *s) {
    std::vector<int> v;
    std::stringstream ss(s);
    std::string tok;
    while (std::getline(ss, tok, ',')) if (!tok.empty()) v.push_back(atoi(tok.c_str()));
    return v;
}

struct Rec { std::string name; std::vector<uint64_t> hashes; };
static std::vector<Rec> g_recs;
static std::vector<std::pair<std::string, double>> g_times;

static void record(const std::string &name, const uint64_t *dev, size_t n_limbs, size_t N) {
    std::vector<uint64_t> h(n_limbs * N);
    cudaDeviceSynchronize();
    cudaMemcpy(h.data(), dev, n_limbs * N * sizeof(uint64_t), cudaMemcpyDeviceToHost);
    Rec r;
    r.name = name;
    for (size_t l = 0; l < n_limbs; l++) r.hashes.push_back(ora_limb_hash(h.data() + l * N, N));
    g_recs.push_back(r);
}

template<typename T> static void put(std::ostream &os, T v) { os.write(reinterpret_cast<const char *>(&v), sizeof(T)); }

// serialised ciphertext header, include/ciphertext.h:173-191
static void put_ct_header(std::ostream &os, size_t chain, size_t size, size_t N, size_t limbs, double scale) {
    put<size_t>(os, chain); put<size_t>(os, size); put<size_t>(os, N); put<size_t>(os, limbs);
    put<double>(os, scale); put<uint64_t>(os, 1); put<size_t>(os, 1);
    put<bool>(os, true); put<bool>(os, false);
}

// ciphertext [size][limbs][N] with synthetic limbs of buffer id `buf`
static PhantomCiphertext make_ct(const std::vector<uint64_t> &primes, size_t chain, size_t size, size_t N,
                                 size_t limbs, double scale, uint64_t seed, uint64_t buf) {
    std::stringstream ss;
    put_ct_header(ss, chain, size, N, limbs, scale);
    std::vector<uint64_t> d(size * limbs * N);
    for (size_t p = 0; p < size; p++)
        ora_fill_limbs(d.data() + p * limbs * N, N, primes.data(), limbs, seed, buf, p * limbs);
    ss.write(reinterpret_cast<const char *>(d.data()), d.size() * sizeof(uint64_t));
    PhantomCiphertext ct;
    ct.load(ss);
    return ct;
}

// relin-style key: dnum public keys, each [2][size_QP][N] at chain 0 (include/secretkey.h:192-226)
static void put_relin_key(std::ostream &os, const std::vector<uint64_t> &primes, size_t dnum, size_t N,
                          uint64_t seed, uint64_t buf0) {
    size_t size_QP = primes.size();
    put<size_t>(os, dnum);
    std::vector<uint64_t> d(2 * size_QP * N);
    for (size_t i = 0; i < dnum; i++) {
        put_ct_header(os, 0, 2, N, size_QP, 1.0);
        for (size_t p = 0; p < 2; p++)
            ora_fill_limbs(d.data() + p * size_QP * N, N, primes.data(), size_QP, seed, buf0 + i, p * size_QP);
        os.write(reinterpret_cast<const char *>(d.data()), d.size() * sizeof(uint64_t));
    }
}

static double time_us(const std::function<void()> &op, int warm, int iters) {
    cudaStream_t s = cudaStreamPerThread;
    for (int i = 0; i < warm; i++) op();
    cudaStreamSynchronize(s);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0, s);
    for (int i = 0; i < iters; i++) op();
    cudaEventRecord(e1, s);
    cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    return ms * 1000.0 / iters;
}

// ---- the reference's bootstrap on the chain of its own round-trip test (test/bootstrap_test.cu:517-662): same parameters
// (N = 2^16, 58 | 40x4 | 58x12 | 29x3 | P 58x4, encapsulation weight 128, 2^15 real slots uniform in (-0.5, 0.5) from
// mt19937_64(0xB007B007), scale 2^40, input left on two primes); dense: the test's default secret, else weight 128 as
// python/examples/bootstrap.py. Writes DIR/boot_sk.bin, boot_ct.bin (the refreshed ciphertext), boot_msg.bin (doubles).
static int run_bootstrap(const std::string &dir, bool dense) {
    const size_t log_n = 16, N = size_t(1) << log_n, HW = 128;
    const double user_scale = std::pow(2.0, 40);
    EncryptionParameters parms(scheme_type::ckks);
    parms.set_poly_modulus_degree(N);
    parms.set_special_modulus_size(4);
    std::vector<int> bits{58};
    bits.insert(bits.end(), 4, 40);
    bits.insert(bits.end(), 12, 58);
    bits.insert(bits.end(), 3, 29);
    bits.insert(bits.end(), 4, 58);
    parms.set_coeff_modulus(CoeffModulus::Create(N, bits));
    auto c2s = build_c2s_diagonals((int) log_n, {5, 5, 5});
    auto s2c = build_s2c_diagonals((int) log_n, {5, 5, 5});
    std::vector<int> steps = c2s_required_rotation_steps(c2s, (int) (N >> 1));
    for (int v : c2s_required_rotation_steps(s2c, (int) (N >> 1))) steps.push_back(v);
    std::sort(steps.begin(), steps.end());
    steps.erase(std::unique(steps.begin(), steps.end()), steps.end());
    auto elts = get_elts_from_steps(steps, N);
    elts.push_back((uint32_t) (2 * N - 1));
    parms.set_galois_elts(elts);
    PhantomContext context(parms);
    PhantomSecretKey sk;
    if (dense) sk = PhantomSecretKey(context);
    else sk.generate_sparse(context, HW);
    PhantomCKKSEncoder encoder(context);
    auto t0 = std::chrono::steady_clock::now();
    BootstrapKey bk = create_bootstrap_key(context, encoder, sk, HW, 9, user_scale);
    cudaDeviceSynchronize();
    const double keygen_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    const size_t slots = encoder.slot_count();
    std::mt19937_64 rng(0xB007B007UL);
    std::uniform_real_distribution<double> dist(-0.5, 0.5);
    std::vector<double> msg(slots);
    std::vector<cuDoubleComplex> z(slots);
    for (size_t i = 0; i < slots; i++) { msg[i] = dist(rng); z[i] = make_cuDoubleComplex(msg[i], 0.0); }
    PhantomPlaintext pt;
    encoder.encode(context, z, user_scale, pt);
    PhantomCiphertext ct;
    sk.encrypt_symmetric(context, pt, ct);
    mod_switch_to_inplace(context, ct, context.total_parm_size() - 2);
    PhantomCiphertext out = bootstrap(context, encoder, ct, bk, user_scale);   // warm-up: tables, allocations
    cudaDeviceSynchronize();
    std::vector<double> ms;
    for (int it = 0; it < 3; it++) {
        auto b0 = std::chrono::steady_clock::now();
        out = bootstrap(context, encoder, ct, bk, user_scale);
        cudaDeviceSynchronize();
        ms.push_back(1e3 * std::chrono::duration<double>(std::chrono::steady_clock::now() - b0).count());
    }
    std::sort(ms.begin(), ms.end());
    PhantomPlaintext dec;
    sk.decrypt(context, out, dec);
    std::vector<cuDoubleComplex> got;
    encoder.decode(context, dec, got);
    double max_err = 0, sum = 0;
    for (size_t i = 0; i < slots; i++) { const double e = std::fabs(got[i].x - msg[i]); max_err = std::max(max_err, e); sum += e; }
    {
        std::ofstream f1(dir + "/boot_sk.bin", std::ios::binary), f2(dir + "/boot_ct.bin", std::ios::binary), f3(dir + "/boot_msg.bin", std::ios::binary);
        sk.save(f1);
        out.save(f2);
        f3.write(reinterpret_cast<const char *>(msg.data()), msg.size() * sizeof(double));
    }
    printf("{\"reference_bootstrap\": {\"secret\": \"%s\", \"ms_median\": %.3f, \"ms_min\": %.3f, \"keygen_s\": %.2f, \"out_chain_index\": %zu, "
           "\"out_limbs\": %zu, \"out_scale_log2\": %.3f, \"own_decode_max_err\": %.6e, \"own_decode_mean_err\": %.6e, \"cuda\": \"%s\"}}\n",
           dense ? "dense" : "sparse128", ms[1], ms[0], keygen_s, out.chain_index(), out.coeff_modulus_size(), std::log2(out.scale()),
           max_err, sum / slots, cudaGetErrorString(cudaGetLastError()));
    return 0;
}

// encode -> decode, and encode -> encrypt -> decrypt -> decode, with the reference's own encoder: where its decode goes wrong
static int run_selftest(int logn, const std::vector<int> &bits, int special) {
    const size_t N = size_t(1) << logn;
    EncryptionParameters parms(scheme_type::ckks);
    parms.set_poly_modulus_degree(N);
    parms.set_coeff_modulus(CoeffModulus::Create(N, bits));
    parms.set_special_modulus_size(special);
    PhantomContext context(parms);
    PhantomCKKSEncoder encoder(context);
    const size_t slots = encoder.slot_count();
    std::vector<cuDoubleComplex> z(slots), got;
    for (size_t j = 0; j < slots; j++) z[j] = make_cuDoubleComplex(cos((double) j), sin(2.0 * j) / 2);
    auto err = [&](const std::vector<cuDoubleComplex> &g) {
        double e = 0;
        for (size_t j = 0; j < slots; j++) e = std::max(e, std::hypot(g[j].x - z[j].x, g[j].y - z[j].y));
        return e;
    };
    const double scale = 1099511627776.0;
    for (size_t chain = 1; chain < context.total_parm_size(); chain += 2) {
        PhantomPlaintext pt;
        encoder.encode(context, z, scale, pt, chain);
        encoder.decode(context, pt, got);
        printf("selftest: chain %zu (%zu limbs) encode->decode max error %.3e\n", chain, context.get_context_data(chain).parms().coeff_modulus().size(), err(got));
    }
    PhantomSecretKey sk(context);
    PhantomPlaintext pt;
    encoder.encode(context, z, scale, pt);
    PhantomCiphertext ct;
    sk.encrypt_symmetric(context, pt, ct);
    PhantomPlaintext dec;
    sk.decrypt(context, ct, dec);
    encoder.decode(context, dec, got);
    printf("selftest: encrypt->decrypt->decode max error %.3e (plaintext chain %zu scale 2^%.1f)\n", err(got), dec.chain_index(), std::log2(dec.scale()));
    PhantomPlaintext dec2 = sk.decrypt(context, ct);
    encoder.decode(context, dec2, got);
    printf("selftest: decrypt (returning form) ->decode max error %.3e (plaintext chain %zu scale 2^%.1f)\n", err(got), dec2.chain_index(), std::log2(dec2.scale()));
    return 0;
}

int main(int argc, char **argv) {
    int logn = 12, special = 2, level = -1, time_iters = 0, n_threads = 0, selftest = 0, boot_dense = 0;
    std::string boot_dir;
    std::vector<int> bsgs;  // {baby steps M, giant steps G}: also run the BSGS matrix-vector driver
    uint64_t seed = 1;
    std::vector<int> bits = {50, 36, 36, 36, 36, 36, 50, 50}, steps = {1, 2, -1};
    std::string out = "case.json", interop_write, interop_read, interop_prefix = "b2";
    for (int i = 1; i + 1 < argc; i += 2) {
        std::string k = argv[i];
        const char *v = argv[i + 1];
        if (k == "--logn") logn = atoi(v);
        else if (k == "--bits") bits = parse_ints(v);
        else if (k == "--special") special = atoi(v);
        else if (k == "--level") level = atoi(v);
        else if (k == "--seed") seed = strtoull(v, nullptr, 10);
        else if (k == "--steps") steps = parse_ints(v);
        else if (k == "--out") out = v;
        else if (k == "--bsgs") bsgs = parse_ints(v);
        else if (k == "--interop-write") interop_write = v;
        else if (k == "--interop-read") interop_read = v;
        else if (k == "--interop-prefix") interop_prefix = v;
        else if (k == "--time") time_iters = atoi(v);
        else if (k == "--threads") n_threads = atoi(v);
        else if (k == "--selftest") selftest = atoi(v);
        else if (k == "--bootstrap") boot_dir = v;
        else if (k == "--boot-dense") boot_dense = atoi(v);
        else { fprintf(stderr, "unknown arg %s\n", argv[i]); return 2; }
    }
    if (!boot_dir.empty()) return run_bootstrap(boot_dir, boot_dense != 0);
    if (selftest) return run_selftest(logn, bits, special);
    const size_t N = size_t(1) << logn;
    const size_t size_QP = bits.size(), size_P = special, size_Q = size_QP - size_P;
    const size_t l = level < 0 ? size_Q : size_t(level);   // number of Q limbs of the data
    const size_t chain = size_Q - l + 1;                      // src/context.cu:145-168
    const size_t beta = (l + size_P - 1) / size_P, lP = l + size_P;

    std::vector<uint32_t> elts;
    for (int s : steps) elts.push_back(get_elt_from_step(s, N));

    EncryptionParameters parms(scheme_type::ckks);
    parms.set_poly_modulus_degree(N);
    auto mods = CoeffModulus::Create(N, bits);
    parms.set_coeff_modulus(mods);
    parms.set_special_modulus_size(size_P);
    parms.set_galois_elts(elts);
    PhantomContext context(parms);
    const auto &s = cudaStreamPerThread;

    std::vector<uint64_t> primes;
    for (auto &m : mods) primes.push_back(m.value());

    // ---- host tables of the reference against the oracle's, word for word ------------------
    int tables_ok = 1;
    {
        std::vector<uint64_t> op(size_QP);
        if (ora_create_coeff_modulus(N, bits.data(), size_QP, op.data()) != 0 || op != primes) tables_ok = 0;
        ora_ctx *oc = ora_ctx_create(N, primes.data(), size_QP, size_P);
        auto &tabs = context.get_context_data(0).small_ntt_tables();
        for (size_t i = 0; i < size_QP && oc; i++) {
            auto &t = tabs->get_ntt_at(i);
            if (memcmp(t.get_from_root_powers().data(), ora_ctx_twiddle(oc, i), N * 8)) tables_ok = 0;
            if (memcmp(t.get_from_inv_root_powers().data(), ora_ctx_itwiddle(oc, i), N * 8)) tables_ok = 0;
        }
        if (!oc) tables_ok = 0;
        ora_ctx_destroy(oc);
    }

    // ---- NTT forward / inverse over all size_QP limbs --------------------------------------
    {
        std::vector<uint64_t> h(size_QP * N);
        ora_fill_limbs(h.data(), N, primes.data(), size_QP, seed, 50, 0);
        auto d = make_cuda_auto_ptr<uint64_t>(size_QP * N, s);
        cudaMemcpy(d.get(), h.data(), h.size() * 8, cudaMemcpyHostToDevice);
        nwt_2d_radix8_forward_inplace(d.get(), context.gpu_rns_tables(), size_QP, 0, s);
        record("ntt_fwd", d.get(), size_QP, N);
        cudaMemcpy(d.get(), h.data(), h.size() * 8, cudaMemcpyHostToDevice);
        nwt_2d_radix8_backward_inplace(d.get(), context.gpu_rns_tables(), size_QP, 0, s);
        record("ntt_inv", d.get(), size_QP, N);
        if (time_iters) {
            g_times.push_back({"ntt_fwd_us", time_us([&] {
                nwt_2d_radix8_forward_inplace(d.get(), context.gpu_rns_tables(), size_QP, 0, s); }, 10, time_iters)});
            g_times.push_back({"ntt_inv_us", time_us([&] {
                nwt_2d_radix8_backward_inplace(d.get(), context.gpu_rns_tables(), size_QP, 0, s); }, 10, time_iters)});
        }
    }

    // ---- keys ---------------------------------------------------------------------------------
    // relin key: buffers 10.. ; Galois key for elts[e]: buffers 100 + 8 e ..
    PhantomRelinKey rlk;
    { std::stringstream ss; put_relin_key(ss, primes, beta, N, seed, 10); rlk.load(ss); }
    PhantomGaloisKey glk;
    {
        std::stringstream ss;
        put<size_t>(ss, elts.size());
        for (size_t e = 0; e < elts.size(); e++) put_relin_key(ss, primes, beta, N, seed, 100 + 8 * e);
        glk.load(ss);
    }

    const double scale = 1099511627776.0; // 2^40
    // ---- interchange with the other library through save()/load() bytes --------------------------------
    // message: slot j = cos(j) + i sin(2j)/2. --interop-write DIR: the reference makes a secret key,
    // encodes, encrypts and saves ref_sk.bin / ref_ct.bin. --interop-read DIR: the reference loads
    // b2_sk.bin / b2_ct.bin written by the other library, decrypts, decodes and prints the error.
    if (!interop_write.empty() || !interop_read.empty()) {
        PhantomCKKSEncoder encoder(context);
        const size_t slots = encoder.slot_count();
        std::vector<cuDoubleComplex> z(slots);
        for (size_t j = 0; j < slots; j++) z[j] = make_cuDoubleComplex(cos((double) j), sin(2.0 * j) / 2);
        if (!interop_write.empty()) {
            PhantomSecretKey sk(context);
            PhantomPlaintext pt;
            encoder.encode(context, z, scale, pt);
            PhantomCiphertext ct;
            sk.encrypt_symmetric(context, pt, ct);
            std::ofstream f1(interop_write + "/ref_sk.bin", std::ios::binary), f2(interop_write + "/ref_ct.bin", std::ios::binary);
            sk.save(f1);
            ct.save(f2);
            // a relinearisation key cut down to the digits chain index 3 reads (src/secretkey.cu:301-352)
            PhantomRelinKey rlk = sk.gen_relinkey(context);
            const size_t full = rlk.dnum();
            rlk.mod_drop_to_inplace(context, 3);
            std::ofstream f3(interop_write + "/ref_rlk_trunc.bin", std::ios::binary);
            rlk.save(f3);
            printf("interop: wrote ref_sk.bin ref_ct.bin ref_rlk_trunc.bin (%zu of %zu digits)\n", rlk.dnum(), full);
        }
        if (!interop_read.empty()) {
            std::ifstream f1(interop_read + "/" + interop_prefix + "_sk.bin", std::ios::binary), f2(interop_read + "/" + interop_prefix + "_ct.bin", std::ios::binary);
            if (!f1 || !f2) { fprintf(stderr, "interop: b2 files missing\n"); return 3; }
            PhantomSecretKey sk;
            sk.load(f1);
            PhantomCiphertext ct;
            ct.load(f2);
            // the decrypted plaintext is integer work: print its per-limb hashes, the caller compares them
            // with its own decryption of the same bytes
            PhantomPlaintext pt = sk.decrypt(context, ct);
            const size_t lim = ct.coeff_modulus_size();
            std::vector<uint64_t> h(lim * N);
            cudaDeviceSynchronize();
            cudaMemcpy(h.data(), pt.data(), h.size() * 8, cudaMemcpyDeviceToHost);
            printf("interop-plain:");
            for (size_t i = 0; i < lim; i++) printf(" %016llx", (unsigned long long) ora_limb_hash(h.data() + i * N, N));
            printf("\n");
            return 0;
        }
        return 0;
    }
    auto &tool = context.get_context_data(chain).gpu_rns_tool();

    // ---- the three stages of the key switch, separately ---------------------------------------
    {
        std::vector<uint64_t> h(l * N);
        ora_fill_limbs(h.data(), N, primes.data(), l, seed, 3, 0);
        auto c2 = make_cuda_auto_ptr<uint64_t>(l * N, s);
        cudaMemcpy(c2.get(), h.data(), h.size() * 8, cudaMemcpyHostToDevice);
        auto up = make_cuda_auto_ptr<uint64_t>(beta * lP * N, s);
        tool.modup(up.get(), c2.get(), context.gpu_rns_tables(), scheme_type::ckks, s);
        record("modup", up.get(), beta * lP, N);
        auto cx = make_cuda_auto_ptr<uint64_t>(2 * lP * N, s);
        key_switch_inner_prod(cx.get(), up.get(), rlk.public_keys_ptr(), tool, context.gpu_rns_tables().modulus(), 15, s);
        record("inner_prod", cx.get(), 2 * lP, N);
        if (time_iters) {
            g_times.push_back({"modup_us", time_us([&] {
                tool.modup(up.get(), c2.get(), context.gpu_rns_tables(), scheme_type::ckks, s); }, 5, time_iters)});
            g_times.push_back({"inner_prod_us", time_us([&] {
                key_switch_inner_prod(cx.get(), up.get(), rlk.public_keys_ptr(), tool,
                                      context.gpu_rns_tables().modulus(), 15, s); }, 5, time_iters)});
            auto cx2 = make_cuda_auto_ptr<uint64_t>(2 * lP * N, s);
            g_times.push_back({"moddown_x2_us", time_us([&] {
                cudaMemcpyAsync(cx2.get(), cx.get(), 2 * lP * N * 8, cudaMemcpyDeviceToDevice, s);
                tool.moddown_from_NTT(cx2.get(), cx2.get(), context.gpu_rns_tables(), scheme_type::ckks, s);
                tool.moddown_from_NTT(cx2.get() + lP * N, cx2.get() + lP * N, context.gpu_rns_tables(),
                                      scheme_type::ckks, s); }, 5, time_iters)});
        }
        for (size_t k = 0; k < 2; k++)
            tool.moddown_from_NTT(cx.get() + k * lP * N, cx.get() + k * lP * N, context.gpu_rns_tables(),
                                  scheme_type::ckks, s);
        record("moddown0", cx.get(), l, N);
        record("moddown1", cx.get() + lP * N, l, N);

        // whole key switch into a synthetic 2-poly ciphertext (buffer 1)
        PhantomCiphertext ct = make_ct(primes, chain, 2, N, l, scale, seed, 1);
        cudaMemcpy(c2.get(), h.data(), h.size() * 8, cudaMemcpyHostToDevice);
        keyswitch_inplace(context, ct, c2.get(), rlk, true, s);
        record("keyswitch", ct.data(), 2 * l, N);
        if (time_iters) {
            g_times.push_back({"keyswitch_us", time_us([&] {
                keyswitch_inplace(context, ct, c2.get(), rlk, true, s); }, 5, time_iters)});
            if (n_threads > 1) {
                // the same call from n_threads host threads, each on its own per-thread default stream with its own ciphertext and
                // input: keyswitch_mt_us = wall time per round of n_threads concurrent key switches
                std::vector<std::thread> th;
                std::atomic<int> ready{0};
                std::atomic<bool> go{false};
                std::vector<double> secs(n_threads, 0.0);
                for (int t = 0; t < n_threads; t++)
                    th.emplace_back([&, t] {
                        const auto &ts = cudaStreamPerThread;
                        PhantomCiphertext my = make_ct(primes, chain, 2, N, l, scale, seed, 1);
                        auto my_c2 = make_cuda_auto_ptr<uint64_t>(l * N, ts);
                        cudaMemcpyAsync(my_c2.get(), h.data(), h.size() * 8, cudaMemcpyHostToDevice, ts);
                        for (int i = 0; i < 5; i++) keyswitch_inplace(context, my, my_c2.get(), rlk, true, ts);
                        cudaStreamSynchronize(ts);
                        ready++;
                        while (!go.load()) std::this_thread::yield();
                        auto b0 = std::chrono::steady_clock::now();
                        for (int i = 0; i < time_iters; i++) keyswitch_inplace(context, my, my_c2.get(), rlk, true, ts);
                        cudaStreamSynchronize(ts);
                        secs[t] = std::chrono::duration<double>(std::chrono::steady_clock::now() - b0).count();
                    });
                while (ready.load() < n_threads) std::this_thread::yield();
                go = true;
                for (auto &t : th) t.join();
                g_times.push_back({"keyswitch_mt_us", 1e6 * *std::max_element(secs.begin(), secs.end()) / time_iters});
                g_times.push_back({"keyswitch_mt_threads", (double) n_threads});
            }
        }
    }

    // ---- HMult + relin, rescale ---------------------------------------------------------------
    {
        PhantomCiphertext a = make_ct(primes, chain, 2, N, l, scale, seed, 1);
        PhantomCiphertext b = make_ct(primes, chain, 2, N, l, scale, seed, 2);
        PhantomCiphertext m(a);
        multiply_and_relin_inplace(context, m, b, rlk);
        record("mul_relin", m.data(), 2 * l, N);
        if (l >= 2) {
            PhantomCiphertext r = rescale_to_next(context, m);
            record("mul_relin_rescale", r.data(), 2 * (l - 1), N);
            PhantomCiphertext ra = rescale_to_next(context, a);
            record("rescale", ra.data(), 2 * (l - 1), N);
        }
        if (time_iters) {
            PhantomCiphertext scratch(a);
            g_times.push_back({"mul_relin_us", time_us([&] {
                scratch = a; multiply_and_relin_inplace(context, scratch, b, rlk); }, 5, time_iters)});
            if (l >= 2)
                g_times.push_back({"mul_relin_rescale_us", time_us([&] {
                    scratch = a; multiply_and_relin_inplace(context, scratch, b, rlk);
                    rescale_to_next_inplace(context, scratch); }, 5, time_iters)});
        }
    }

    // ---- rotations ------------------------------------------------------------------------------
    {
        PhantomCiphertext a = make_ct(primes, chain, 2, N, l, scale, seed, 1);
        for (size_t e = 0; e < elts.size(); e++) {
            PhantomCiphertext r(a);
            apply_galois_inplace(context, r, elts[e], glk);
            record("rotate_" + std::to_string(steps[e]), r.data(), 2 * l, N);
        }
        auto outs = hoist_rotations(context, a, glk, steps);
        for (size_t e = 0; e < outs.size(); e++)
            record("hoist_" + std::to_string(steps[e]), outs[e].data(), 2 * l, N);
        {
            // hoisting_inplace: the SUM of the rotations, one ModUp and one ModDown pair for all steps
            PhantomCiphertext h(a);
            hoisting_inplace(context, h, glk, steps);
            record("hoisting_sum", h.data(), 2 * l, N);
        }
        if (time_iters) {
            PhantomCiphertext r(a);
            g_times.push_back({"rotate_us", time_us([&] {
                r = a; apply_galois_inplace(context, r, elts[0], glk); }, 5, time_iters)});
            g_times.push_back({"hoist_rotations_us", time_us([&] {
                auto o = hoist_rotations(context, a, glk, steps); }, 2, time_iters / 4 + 1)});
        }
    }
    // ---- BSGS matrix-vector driver on synthetic single-chain plaintexts ----------------------------
    // diagonal d = signed centred coefficients in [-2^39, 2^39): uniform draw of stream
    // (seed << 40) ^ ((3000 + d) << 16) below 2^40, minus 2^39. Needs --steps 1,2,..,M/2,M.
    if (bsgs.size() == 2) {
        const size_t M = bsgs[0], G = bsgs[1];
        BsgsDiagonals diags;
        diags.d_pad = M * G;
        diags.baby_steps = M;
        diags.giant_steps = G;
        std::vector<uint64_t> u(N);
        for (size_t d = 0; d < M * G; d++) {
            SingleChainPlaintext scp;
            scp.coeffs = PinnedHostInt64Buffer(N);
            scp.scale = scale;
            ora_fill_uniform(u.data(), N, uint64_t(1) << 40, (seed << 40) ^ (uint64_t(3000 + d) << 16));
            for (size_t i = 0; i < N; i++) scp.coeffs.data()[i] = (int64_t) u[i] - (int64_t(1) << 39);
            diags.diagonals.push_back(std::move(scp));
        }
        PhantomCiphertext x = make_ct(primes, chain, 2, N, l, scale, seed, 1);
        PhantomCiphertext y = bsgs_matmul_preencoded(context, glk, x, diags);
        record("bsgs", y.data(), 2 * (l - 1), N);
        PhantomPlaintext full = expand_single_chain_to_full(context, diags.diagonals[0], chain);
        record("expand_single_chain", full.data(), l, N);
        if (time_iters)
            g_times.push_back({"bsgs_us", time_us([&] { auto r = bsgs_matmul_preencoded(context, glk, x, diags); }, 2, time_iters / 4 + 1)});
    }
    cudaDeviceSynchronize();
    cudaError_t err = cudaGetLastError();

    // ---- JSON ---------------------------------------------------------------------------------
    FILE *f = fopen(out.c_str(), "w");
    if (!f) { perror("open out"); return 1; }
    fprintf(f, "{\n \"logn\": %d, \"special\": %zu, \"level\": %zu, \"seed\": %llu, \"chain_index\": %zu,\n",
            logn, size_P, l, (unsigned long long) seed, chain);
    fprintf(f, " \"bits\": ["); for (size_t i = 0; i < bits.size(); i++) fprintf(f, "%s%d", i ? "," : "", bits[i]); fprintf(f, "],\n");
    fprintf(f, " \"steps\": ["); for (size_t i = 0; i < steps.size(); i++) fprintf(f, "%s%d", i ? "," : "", steps[i]); fprintf(f, "],\n");
    fprintf(f, " \"bsgs\": ["); for (size_t i = 0; i < bsgs.size(); i++) fprintf(f, "%s%d", i ? "," : "", bsgs[i]); fprintf(f, "],\n");
    fprintf(f, " \"elts\": ["); for (size_t i = 0; i < elts.size(); i++) fprintf(f, "%s%u", i ? "," : "", elts[i]); fprintf(f, "],\n");
    fprintf(f, " \"primes\": ["); for (size_t i = 0; i < primes.size(); i++) fprintf(f, "%s%llu", i ? "," : "", (unsigned long long) primes[i]); fprintf(f, "],\n");
    fprintf(f, " \"host_tables_match_oracle\": %s,\n \"cuda_error\": \"%s\",\n", tables_ok ? "true" : "false", cudaGetErrorString(err));
    fprintf(f, " \"times_us\": {");
    for (size_t i = 0; i < g_times.size(); i++) fprintf(f, "%s\"%s\": %.3f", i ? ", " : "", g_times[i].first.c_str(), g_times[i].second);
    fprintf(f, "},\n \"hashes\": {\n");
    for (size_t i = 0; i < g_recs.size(); i++) {
        fprintf(f, "  \"%s\": [", g_recs[i].name.c_str());
        for (size_t j = 0; j < g_recs[i].hashes.size(); j++)
            fprintf(f, "%s\"%016llx\"", j ? "," : "", (unsigned long long) g_recs[i].hashes[j]);
        fprintf(f, "]%s\n", i + 1 < g_recs.size() ? "," : "");
    }
    fprintf(f, " }\n}\n");
    fclose(f);
    printf("wrote %s (%zu records, tables_ok=%d, cuda=%s)\n", out.c_str(), g_recs.size(), tables_ok, cudaGetErrorString(err));
    return (tables_ok && err == cudaSuccess) ? 0 : 1;
}
