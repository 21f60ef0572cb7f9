// modarith.cuh - 64-bit modular arithmetic for RNS limbs on sm_100a.
//
// All kernels keep residues as uint64 and use the primes' Shoup / Barrett constants. Inside a
// transform values are kept lazily in [0,4q) (forward) or [0,2q) (inverse); every kernel's
// final store is canonical, i.e. in [0,q). That is the only property the reference's kernels
// guarantee too (include/uintmodmath.cuh:96-136, 207-215; include/butterfly.cuh:17-71), so
// outputs are bit-identical although the butterfly schedule differs.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b2 {

// {w, floor(w * 2^64 / q)}
struct __align__(16) W2 {
    uint64_t w, ws;
};

__device__ __forceinline__ W2 ldg_w2(const W2 *p) {
    ulonglong2 v = __ldg(reinterpret_cast<const ulonglong2 *>(p));
    return W2{v.x, v.y};
}

// x * w mod q in [0, 2q) for any 64-bit x (Shoup / Harvey)
__device__ __forceinline__ uint64_t mul_shoup_lazy(uint64_t x, W2 w, uint64_t q) {
    uint64_t h = __umul64hi(x, w.ws);
    return x * w.w - h * q;
}

__device__ __forceinline__ uint64_t csub(uint64_t x, uint64_t q) { return x >= q ? x - q : x; }

__device__ __forceinline__ uint64_t mul_shoup(uint64_t x, W2 w, uint64_t q) { return csub(mul_shoup_lazy(x, w, q), q); }

__device__ __forceinline__ uint64_t add_mod(uint64_t a, uint64_t b, uint64_t q) { return csub(a + b, q); }
__device__ __forceinline__ uint64_t sub_mod(uint64_t a, uint64_t b, uint64_t q) { return a >= b ? a - b : a + q - b; }

// Forward (Cooley-Tukey) lazy butterfly: x,y in [0,4q) -> x,y in [0,4q)
__device__ __forceinline__ void ct_bfly(uint64_t &x, uint64_t &y, W2 w, uint64_t q, uint64_t q2) {
    uint64_t a = csub(x, q2);
    uint64_t t = mul_shoup_lazy(y, w, q);
    x = a + t;
    y = a - t + q2;
}

// Inverse (Gentleman-Sande) lazy butterfly: x,y in [0,2q) -> x,y in [0,2q)
__device__ __forceinline__ void gs_bfly(uint64_t &x, uint64_t &y, W2 w, uint64_t q, uint64_t q2) {
    uint64_t s = x + y;
    uint64_t d = x - y + q2;
    x = csub(s, q2);
    y = mul_shoup_lazy(d, w, q);
}

struct u128 {
    uint64_t lo, hi;
};

__device__ __forceinline__ void mac128(u128 &acc, uint64_t a, uint64_t b) {
    uint64_t lo = a * b, hi = __umul64hi(a, b);
    acc.lo += lo;
    acc.hi += hi + (acc.lo < lo);
}

// Barrett reduction of a 128-bit value with ratio = floor(2^128 / q) = {r0, r1}; result in [0,q)
__device__ __forceinline__ uint64_t barrett128(u128 x, uint64_t q, uint64_t r0, uint64_t r1) {
    uint64_t carry = __umul64hi(x.lo, r0);
    uint64_t t_lo = x.lo * r1, t_hi = __umul64hi(x.lo, r1);
    uint64_t s1 = t_lo + carry;
    uint64_t c1 = s1 < carry;
    uint64_t t3 = t_hi + c1;
    uint64_t u_lo = x.hi * r0, u_hi = __umul64hi(x.hi, r0);
    uint64_t s2 = s1 + u_lo;
    uint64_t c2 = s2 < u_lo;
    uint64_t qhat = x.hi * r1 + t3 + u_hi + c2;
    uint64_t r = x.lo - qhat * q;
    return csub(r, q);
}

// x mod q for a 64-bit x, with r1 = high word of floor(2^128 / q)
__device__ __forceinline__ uint64_t barrett64(uint64_t x, uint64_t q, uint64_t r1) {
    uint64_t qhat = __umul64hi(x, r1);
    return csub(x - qhat * q, q);
}

}  // namespace b2
