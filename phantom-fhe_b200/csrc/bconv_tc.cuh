// bconv_tc.cuh - fast base conversion on the sm_100a tensor cores (tcgen05.mma kind::i8, accumulators in TMEM).
// The formulation, the data structures and the host-side planning are in bconv_tc_plan.h.
//
// CTA = 128 coefficients (M = 128: TMEM lane = coefficient) x one job. The threads put the tile's input limbs into
// shared memory as the rows of A (the raw 8 bytes of each residue) and copy the job's ready-made B image next to it;
// one thread issues two MMAs (K = 2 x 32, N = 16 * groups <= 256) and commits them to an mbarrier; every warp then
// reads its 32 TMEM lanes (tcgen05.ld 32x32b: one coefficient per thread, 16 columns = one output group at a time),
// reduces and stores 8-byte words that are contiguous across the warp. 128 * WG threads: warp w reads lanes
// 32 (w % 4) .. +31 and warpgroup w / 4 takes every WG-th column group.
// No multicast, no cluster; the only wait (MMA completion) is bounded and reports through a status word instead of
// spinning forever; TMEM is released on every path.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "bconv_tc_plan.h"

namespace b2 {

constexpr uint32_t TC_SMEM_A = 128 * 64;            // one tile of A
constexpr uint32_t TC_SMEM_B = 256 * 64;            // largest B image
constexpr uint32_t TC_SMEM_CTRL = TC_SMEM_A + TC_SMEM_B;
constexpr uint32_t TC_SMEM_BYTES = TC_SMEM_CTRL + 32;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;        // polls of the MMA barrier before giving up
constexpr uint32_t TC_SM_SMEM = 233472;             // shared memory of one SM (228 KB)
constexpr uint32_t TC_SMEM_MAX_REQUEST = TC_SM_SMEM / 2;

__device__ __forceinline__ uint32_t tc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: K-major, no swizzle, LBO = 128 B, SBO = 512 B, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(128u >> 4) << 16) | ((uint64_t)(512u >> 4) << 32) | ((uint64_t)1 << 46);
}

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 16 consecutive accumulator columns of this thread's TMEM lane; the wait is part of the same statement so
// that no use of the registers can be scheduled ahead of it
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&c)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]), "=r"(c[4]), "=r"(c[5]), "=r"(c[6]), "=r"(c[7]), "=r"(c[8]), "=r"(c[9]),
          "=r"(c[10]), "=r"(c[11]), "=r"(c[12]), "=r"(c[13]), "=r"(c[14]), "=r"(c[15])
        : "r"(taddr)
        : "memory");
}

// the same load without the wait, and the wait as a statement that owns the registers: a group's planes can be on their way
// while the previous group is reduced
__device__ __forceinline__ void tc_ld16_nowait(uint32_t taddr, uint32_t (&c)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]), "=r"(c[4]), "=r"(c[5]), "=r"(c[6]), "=r"(c[7]), "=r"(c[8]), "=r"(c[9]),
          "=r"(c[10]), "=r"(c[11]), "=r"(c[12]), "=r"(c[13]), "=r"(c[14]), "=r"(c[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld(uint32_t (&c)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]), "+r"(c[4]), "+r"(c[5]), "+r"(c[6]), "+r"(c[7]), "+r"(c[8]), "+r"(c[9]),
                   "+r"(c[10]), "+r"(c[11]), "+r"(c[12]), "+r"(c[13]), "+r"(c[14]), "+r"(c[15])
                 :
                 : "memory");
}

template <int NB>
__device__ __forceinline__ void tc_group_outputs(const uint32_t (&c)[16], const TcGroup *g, uint32_t n_valid, uint64_t *__restrict__ out, size_t N,
                                                 uint32_t n) {
    constexpr int OPG = 16 / NB;
#pragma unroll
    for (int o = 0; o < OPG; o++) {
        if (o < (int)n_valid) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(&g->o[o]));
            const uint64_t p = (uint64_t)raw.x | ((uint64_t)raw.y << 32);
            out[(size_t)raw.w * N + n] = tc_reduce<NB>(&c[o * NB], p, raw.z);
        }
    }
}


// ---- lean epilogue of the persistent kernel ------------------------------------------------------------------------
// One output as the epilogue wants it, 16 bytes in shared memory (one LDS.128): prime, reciprocal, and the output
// limb's first element (slot * N); 0xFFFFFFFF marks a slot of a group that holds no output (p = 1 keeps its
// arithmetic harmless), so the group is processed without a branch per output and only the store is predicated.
struct TcOutS {
    uint32_t p_lo, p_hi, mu, off;
};

// One output, written so that it costs about twenty instructions: the planes are paired with shift-adds, joined by one
// (two for 7 and 8 planes) wide multiply-add, the quotient estimate is one high multiply, and the two subtractions, the
// choice between r and r - p (sign of the difference: r < 2p < 2^62) and the predicated store are spelled out in PTX so
// that no branch and no 64-bit compare is generated. Same value as tc_reduce / tc_reduce_dev (bconv_tc_plan.h).
template <int NB, bool ALWAYS = false>
__device__ __forceinline__ void tc_output(const uint32_t *c, const uint4 m, uint64_t *__restrict__ out_n) {
    constexpr int SH = 8 * NB - 17;
    const uint32_t x0 = c[0] + (c[1] << 8), x1 = c[2] + (c[3] << 8);
    uint32_t vl, vh, vq;  // V mod 2^64 as two words; V >> SH
    if constexpr (NB <= 6) {
        const uint32_t x2 = NB == 4 ? 0u : (NB == 5 ? c[4] : c[4] + (c[5] << 8));
        const uint64_t v = (uint64_t)x1 * 65536u + (((uint64_t)x2 << 32) | x0);
        vl = (uint32_t)v, vh = (uint32_t)(v >> 32);
        vq = __funnelshift_r(vl, vh, SH);
    } else {
        const uint32_t x2 = c[4] + (c[5] << 8), x3 = NB == 7 ? c[6] : c[6] + (c[7] << 8);
        const uint64_t a = (uint64_t)x1 * 65536u + x0, b = (uint64_t)x3 * 65536u + x2;
        const uint64_t mid = (a >> 32) + b;
        vl = (uint32_t)a, vh = (uint32_t)mid;
        vq = __funnelshift_r((uint32_t)mid, (uint32_t)(mid >> 32), SH - 32);
    }
    const uint32_t qhat = __umulhi(vq, m.z);
    const uint64_t qp = (uint64_t)qhat * m.x;
    const uint32_t ql = (uint32_t)qp, qh = (uint32_t)(qp >> 32) + qhat * m.y;
    uint32_t rl, rh;
    // plain asm (no volatile): independent outputs of a group may be interleaved by the scheduler
    asm("{\n\t"
        ".reg .u32 tl, th;\n\t"
        ".reg .pred pn;\n\t"
        "sub.cc.u32 %0, %2, %4;\n\t"
        "subc.u32 %1, %3, %5;\n\t"
        "sub.cc.u32 tl, %0, %6;\n\t"
        "subc.u32 th, %1, %7;\n\t"
        "setp.lt.s32 pn, th, 0;\n\t"
        "selp.u32 %0, %0, tl, pn;\n\t"
        "selp.u32 %1, %1, th, pn;\n\t"
        "}\n"
        : "=&r"(rl), "=&r"(rh)
        : "r"(vl), "r"(vh), "r"(ql), "r"(qh), "r"(m.x), "r"(m.y));
    if constexpr (ALWAYS) {
        asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(out_n + m.w), "r"(rl), "r"(rh) : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred pv;\n\t"
            "setp.ne.u32 pv, %3, 0xFFFFFFFF;\n\t"
            "@pv st.global.v2.u32 [%0], {%1, %2};\n\t"
            "}\n" ::"l"(out_n + m.w),
            "r"(rl), "r"(rh), "r"(m.w)
            : "memory");
    }
}

// NV = number of outputs the group holds (0: not known at compile time, every slot is processed and the store of an empty
// one is predicated off)
template <int NB, int NV = 0>
__device__ __forceinline__ void tc_group_lean(const uint32_t (&c)[16], uint32_t mo_smem, uint64_t *__restrict__ out_n) {
    constexpr int OPG = NV ? NV : 16 / NB;
#pragma unroll
    for (int o = 0; o < OPG; o++) {
        uint4 m;
        // the records do not change while a job's tiles are reduced: the load may move freely
        asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(m.x), "=r"(m.y), "=r"(m.z), "=r"(m.w) : "r"(mo_smem + 16 * o));
        tc_output<NB, NV != 0>(&c[o * NB], m, out_n);
    }
}

// grid = (N / 128, jobs); dynamic shared memory >= TC_SMEM_BYTES (the launcher asks for more, so that the CTAs
// resident on one SM can never want more than its 512 TMEM columns and the allocation never has to wait)
template <int WG>
__global__ void __launch_bounds__(128 * WG) bconv_tc_kernel(const uint64_t *__restrict__ in, uint64_t *__restrict__ out,
                                                            const uint64_t *__restrict__ copy_src, const TcJob *__restrict__ jobs,
                                                            const TcGroup *__restrict__ groups, const uint8_t *__restrict__ images, uint32_t N,
                                                            uint32_t *err) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t *sA = tc_smem, *sB = tc_smem + TC_SMEM_A;
    uint64_t *bar = reinterpret_cast<uint64_t *>(tc_smem + TC_SMEM_CTRL);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tc_smem + TC_SMEM_CTRL + 8);
    const TcJob job = jobs[blockIdx.y];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n0 = blockIdx.x * 128;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"(job.alloc_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // B: the ready-made byte image of this job
    {
        const int4 *src = reinterpret_cast<const int4 *>(images + job.img_off);
        int4 *dst = reinterpret_cast<int4 *>(sB);
        for (uint32_t i = tid; i < job.n_groups * 64; i += 128 * WG) dst[i] = __ldg(src + i);
    }
    // A: row = coefficient, the 8 bytes of input limb i at k = 8 i .. 8 i + 7 (two limbs per 16-byte store)
    {
        const uint32_t r = tid & 127, part = tid >> 7;
        constexpr int PAIRS = 4 / WG;
        const bool copy = copy_src != nullptr && job.copy_dst_slot0 != 0xFFFFFFFFu;
#pragma unroll
        for (int pp = 0; pp < PAIRS; pp++) {
            const uint32_t i = 2 * (part * PAIRS + pp);
            uint64_t v[2] = {0, 0};
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (i + h < job.ni) {
                    const size_t off = (size_t)(job.in_slot0 + i + h) * N + n0 + r;
                    v[h] = in[off];
                    if (copy) out[(size_t)(job.copy_dst_slot0 + i + h) * N + n0 + r] = copy_src[off];
                }
            }
            *reinterpret_cast<ulonglong2 *>(sA + (r >> 3) * 512 + (i >> 1) * 128 + (r & 7) * 16) = make_ulonglong2(v[0], v[1]);
        }
    }
    // generic-proxy writes of A and B become visible to the tensor core's (async-proxy) reads
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) {
        const uint64_t adesc = tc_desc(tc_smem_u32(sA)), bdesc = tc_desc(tc_smem_u32(sB));
        // D s32, A and B u8, both K-major, N = 16 * groups, M = 128
        const uint32_t idesc = (2u << 4) | (((16u * job.n_groups) >> 3) << 17) | ((128u >> 4) << 24);
        tc_mma_i8(tmem, adesc, bdesc, idesc, 0u);
        tc_mma_i8(tmem, adesc + (256u >> 4), bdesc + (256u >> 4), idesc, 1u);  // k = 32..63: two core matrices further
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem_u32(bar)) : "memory");
    }
    // bounded wait for the accumulators
    uint32_t done = 0;
    for (uint32_t it = 0; it < TC_WAIT_LIMIT && !done; it++) {
        asm volatile(
            "{\n\t"
            ".reg .pred P1;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, P1;\n\t"
            "}\n"
            : "=r"(done)
            : "r"(tc_smem_u32(bar)), "r"(0u)
            : "memory");
    }
    const bool ok = __all_sync(0xFFFFFFFFu, done != 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const uint32_t wq = warp & 3, wg = warp >> 2;
        const uint32_t n = n0 + wq * 32 + lane;
        const uint32_t lane_base = tmem + ((wq * 32u) << 16);
        for (uint32_t g = wg; g < job.n_groups; g += WG) {
            uint32_t c[16];
            tc_ld16(lane_base + g * 16, c);
            const TcGroup *G = groups + job.grp_off + g;
            const uint2 hdr = __ldg(reinterpret_cast<const uint2 *>(G));
            switch (hdr.x) {
                case 4: tc_group_outputs<4>(c, G, hdr.y, out, N, n); break;
                case 5: tc_group_outputs<5>(c, G, hdr.y, out, N, n); break;
                case 6: tc_group_outputs<6>(c, G, hdr.y, out, N, n); break;
                case 7: tc_group_outputs<7>(c, G, hdr.y, out, N, n); break;
                default: tc_group_outputs<8>(c, G, hdr.y, out, N, n); break;
            }
        }
    } else if (lane == 0) {
        atomicExch(err, 1u);  // the MMA never signalled: outputs of this tile are not written
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(job.alloc_cols) : "memory");
}


// ================================================================================================
// Persistent form: a CTA stays on its SM and walks over work items (job, tile), job-major, with stride gridDim.x.
// The job's B image and group table stay in shared memory until the job changes; the next item's A tile is fetched
// with cp.async into the second A buffer while the current tile's accumulators are reduced and stored, so global
// latency, the MMA and the epilogue overlap inside one CTA (and across the CTAs sharing the SM). TMEM is allocated
// once per CTA. One mbarrier, used with alternating phase parity, signals each tile's MMA pair.
// ================================================================================================
constexpr uint32_t TCP_SMEM_A0 = 0, TCP_SMEM_A1 = TC_SMEM_A, TCP_SMEM_B = 2 * TC_SMEM_A, TCP_SMEM_GRP = TCP_SMEM_B + TC_SMEM_B;
constexpr uint32_t TCP_SMEM_CTRL = TCP_SMEM_GRP + 16 * 4 * 16 + 64;  // 16 groups x 4 output records, then one byte count per group
constexpr uint32_t TCP_SMEM_BYTES = TCP_SMEM_CTRL + 32;

__device__ __forceinline__ void tc_cp_async8(uint32_t smem_dst, const void *gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void tc_cp_async16(uint32_t smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}

// the rows of A for tile `tile` of `job`: 8 bytes per (coefficient, input limb), zeros for limbs the job does not have
// A batch of conversions in one launch: set b reads input limb slot s at s * (in_lm1 + 1) + b * in_bs and writes output limb
// slot s at s * (out_lm1 + 1) + b * out_bs (batch-major and limb-major buffers as for the transforms, ntt_kernels.cuh)
struct TcBatch {
    uint32_t batch, in_lm1, in_bs, out_lm1, out_bs;
    uint32_t serial_ld;  // 1: wait for every TMEM load before reducing it (no second register set in flight)
};

template <int WG>
__device__ __forceinline__ void tcp_fetch_a(uint8_t *sA, const uint64_t *__restrict__ in, const TcJob &job, uint32_t N, uint32_t tile, uint32_t b,
                                            const TcBatch &tb) {
    const uint32_t tid = threadIdx.x, r = tid & 127, part = tid >> 7;
    constexpr int LIMBS = 8 / WG;
#pragma unroll
    for (int j = 0; j < LIMBS; j++) {
        const uint32_t i = part * LIMBS + j;
        uint8_t *dst = sA + (r >> 3) * 512 + (i >> 1) * 128 + (r & 7) * 16 + (i & 1) * 8;
        if (i < job.ni) {
            const size_t slot = (size_t)(job.in_slot0 + i * (job.in_stride1 + 1)) * (tb.in_lm1 + 1) + (size_t)b * tb.in_bs;
            tc_cp_async8(tc_smem_u32(dst), in + slot * N + (size_t)tile * 128 + r);
        } else {
            *reinterpret_cast<uint64_t *>(dst) = 0;
        }
    }
}

template <int WG>
__global__ void __launch_bounds__(128 * WG) bconv_tc_persist(const uint64_t *__restrict__ in, uint64_t *__restrict__ out,
                                                             const uint64_t *__restrict__ copy_src, const TcJob *__restrict__ jobs,
                                                             const TcGroup *__restrict__ groups, const uint8_t *__restrict__ images, uint32_t N,
                                                             uint32_t n_jobs, uint32_t alloc_cols, uint32_t *err, const TcBatch tb) {
    extern __shared__ __align__(1024) uint8_t tc_smem[];
    uint8_t *sB = tc_smem + TCP_SMEM_B;
    TcOutS *sOut = reinterpret_cast<TcOutS *>(tc_smem + TCP_SMEM_GRP);              // [16][4]
    uint32_t *sNb = reinterpret_cast<uint32_t *>(tc_smem + TCP_SMEM_GRP + 16 * 4 * 16);  // [16]
    uint64_t *bar = reinterpret_cast<uint64_t *>(tc_smem + TCP_SMEM_CTRL);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tc_smem + TCP_SMEM_CTRL + 8);
    constexpr uint32_t THREADS = 128 * WG;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // items: job-major, then set of the batch, then tile (N is a power of two)
    const uint32_t tiles = N >> 7, tile_mask = tiles - 1, log_tiles = 31 - __clz(tiles), per_job = tb.batch << log_tiles, total = n_jobs * per_job;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"(alloc_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(tc_smem_u32(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    uint32_t item = blockIdx.x, cur = 0, phase = 0, loaded_job = 0xFFFFFFFFu;
    bool ok = true;
    TcJob job{};
    if (item < total) {
        job = jobs[item / per_job];
        tcp_fetch_a<WG>(tc_smem + TCP_SMEM_A0, in, job, N, item & tile_mask, (item % per_job) >> log_tiles, tb);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t wq = warp & 3, wg = warp >> 2;
    const uint32_t lane_base = tmem + ((wq * 32u) << 16);

    while (item < total && ok) {
        const uint32_t jb = item / per_job, tile = item & tile_mask, bset = (item - jb * per_job) >> log_tiles;
        if (jb != loaded_job) {
            // a new job: its B image and group table (the MMA that read the old image has completed: every thread
            // waited for it before the previous epilogue, and the barrier at the end of that iteration has passed)
            job = jobs[jb];
            const uint8_t *img = images + job.img_off;
            for (uint32_t i = tid; i < job.n_groups * 64; i += THREADS) tc_cp_async16(tc_smem_u32(sB + 16 * i), img + 16 * i);
            asm volatile("cp.async.commit_group;" ::: "memory");
            // output records in the epilogue's form (nobody reads the old ones any more: see above)
            if (tid < job.n_groups * 4) {
                const TcGroup *G = groups + job.grp_off + (tid >> 2);
                const uint32_t o = tid & 3;
                const uint2 hdr = __ldg(reinterpret_cast<const uint2 *>(G));
                TcOutS rec{1u, 0u, 0u, 0xFFFFFFFFu};
                if (o < hdr.y) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(&G->o[o]));
                    rec = TcOutS{raw.x, raw.y, raw.z, raw.w * (tb.out_lm1 + 1) * N};
                }
                sOut[tid] = rec;
                if (o == 0) sNb[tid >> 2] = hdr.x * 8 + hdr.y;  // bytes per output, outputs in the group
            }
            loaded_job = jb;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint8_t *sA = tc_smem + (cur ? TCP_SMEM_A1 : TCP_SMEM_A0);
        if (tid == 0) {
            const uint64_t adesc = tc_desc(tc_smem_u32(sA)), bdesc = tc_desc(tc_smem_u32(sB));
            const uint32_t idesc = (2u << 4) | (((16u * job.n_groups) >> 3) << 17) | ((128u >> 4) << 24);
            tc_mma_i8(tmem, adesc, bdesc, idesc, 0u);
            tc_mma_i8(tmem, adesc + (256u >> 4), bdesc + (256u >> 4), idesc, 1u);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tc_smem_u32(bar)) : "memory");
        }
        // next item's rows of A into the other buffer (its last reader, the MMA of the previous iteration, is done)
        const uint32_t next = item + gridDim.x;
        if (next < total) {
            const uint32_t njb = next / per_job, nb = (next - njb * per_job) >> log_tiles;
            if (njb == jb) {
                tcp_fetch_a<WG>(tc_smem + (cur ? TCP_SMEM_A0 : TCP_SMEM_A1), in, job, N, next & tile_mask, nb, tb);
            } else {
                const TcJob nj = jobs[njb];
                tcp_fetch_a<WG>(tc_smem + (cur ? TCP_SMEM_A0 : TCP_SMEM_A1), in, nj, N, next & tile_mask, nb, tb);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        // ModUp: the digit's own limbs travel from the NTT-form input to the output buffer (single set only)
        if (copy_src != nullptr && job.copy_dst_slot0 != 0xFFFFFFFFu) {
            const uint32_t r = tid & 127, part = tid >> 7;
            for (uint32_t i = part; i < job.ni; i += WG)
                out[(size_t)(job.copy_dst_slot0 + i) * N + (size_t)tile * 128 + r] = copy_src[(size_t)(job.in_slot0 + i) * N + (size_t)tile * 128 + r];
        }
        // bounded wait for the accumulators
        uint32_t done = 0;
        for (uint32_t it = 0; it < TC_WAIT_LIMIT && !done; it++) {
            asm volatile(
                "{\n\t"
                ".reg .pred P1;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
                "selp.b32 %0, 1, 0, P1;\n\t"
                "}\n"
                : "=r"(done)
                : "r"(tc_smem_u32(bar)), "r"(phase)
                : "memory");
        }
        phase ^= 1u;
        ok = __all_sync(0xFFFFFFFFu, done != 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            uint64_t *out_n = out + (size_t)bset * tb.out_bs * N + (tile * 128 + wq * 32 + lane);
            // (dealing single outputs instead of whole groups over the warpgroups evens the work but triples the TMEM loads:
            // measured 56 against 37 us per key switch)
            auto reduce_group = [&](const uint32_t (&c)[16], uint32_t g) {
                const uint32_t mo = tc_smem_u32(sOut + 4 * g);
                // one case per (bytes per output, outputs in the group): no slot is processed in vain and no store is predicated
                switch (sNb[g]) {
                    case 4 * 8 + 1: tc_group_lean<4, 1>(c, mo, out_n); break;
                    case 4 * 8 + 2: tc_group_lean<4, 2>(c, mo, out_n); break;
                    case 4 * 8 + 3: tc_group_lean<4, 3>(c, mo, out_n); break;
                    case 4 * 8 + 4: tc_group_lean<4, 4>(c, mo, out_n); break;
                    case 5 * 8 + 1: tc_group_lean<5, 1>(c, mo, out_n); break;
                    case 5 * 8 + 2: tc_group_lean<5, 2>(c, mo, out_n); break;
                    case 5 * 8 + 3: tc_group_lean<5, 3>(c, mo, out_n); break;
                    case 6 * 8 + 1: tc_group_lean<6, 1>(c, mo, out_n); break;
                    case 6 * 8 + 2: tc_group_lean<6, 2>(c, mo, out_n); break;
                    case 7 * 8 + 1: tc_group_lean<7, 1>(c, mo, out_n); break;
                    case 7 * 8 + 2: tc_group_lean<7, 2>(c, mo, out_n); break;
                    case 8 * 8 + 1: tc_group_lean<8, 1>(c, mo, out_n); break;
                    case 8 * 8 + 2: tc_group_lean<8, 2>(c, mo, out_n); break;
                    default: break;  // an empty group: the planner makes none
                }
            };
            // two register sets: the next group's planes travel from TMEM while this one is reduced
            uint32_t ca[16], cb[16];
            uint32_t g = wg;
            if (tb.serial_ld) {
                for (; g < job.n_groups; g += WG) {
                    tc_ld16(lane_base + g * 16, ca);
                    reduce_group(ca, g);
                }
            } else {
                if (g < job.n_groups) tc_ld16_nowait(lane_base + g * 16, ca);
                while (g < job.n_groups) {
                    tc_wait_ld(ca);
                    uint32_t gn = g + WG;
                    if (gn < job.n_groups) tc_ld16_nowait(lane_base + gn * 16, cb);
                    reduce_group(ca, g);
                    g = gn;
                    if (g >= job.n_groups) break;
                    tc_wait_ld(cb);
                    gn = g + WG;
                    if (gn < job.n_groups) tc_ld16_nowait(lane_base + gn * 16, ca);
                    reduce_group(cb, g);
                    g = gn;
                }
            }
        } else if (lane == 0) {
            atomicExch(err, 1u);  // the MMA never signalled: this CTA stops, its remaining tiles are not written
        }
        // a CTA whose wait ran out must stop as a whole: make the outcome uniform over the CTA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        ok = __syncthreads_and(ok);
        cur ^= 1u;
        item = next;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(alloc_cols) : "memory");
}

}  // namespace b2
