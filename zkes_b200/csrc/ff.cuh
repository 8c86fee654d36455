// 256-bit Montgomery arithmetic on 8 x 32-bit limbs for BN254 Fr (scalars) and Fq (coordinates).
//
// Replaces the arkworks Fp256 arithmetic the reference takes from ark-ff / ark-bn254
// (every + - * in src/crypto/sumcheck/linear_prover.rs and src/util/poly.rs).  The in-memory
// form is the same as arkworks': little-endian limbs of a*R mod p with R = 2^256.
//
// Device code is PTX carry chains (mad.lo.cc / madc.hi.cc pairs that ptxas fuses into 32x32+64
// wide multiply-adds).  A carry flag never crosses an asm statement: every chain is one
// statement.  The same functions compile for the host with plain 64-bit C so the algorithms
// built on the chains can be unit-tested without a GPU.
#pragma once
#include <cstdint>
#include <cstddef>

#if defined(__CUDACC__)
#define ZK_HD __host__ __device__ __forceinline__
#define ZK_D __device__ __forceinline__
#else
#define ZK_HD inline
#define ZK_D inline
#endif

namespace zk {

// ------------------------------------------------------------------------------------------
// Carry-chain primitives.  acc[] indices are constant after unrolling so everything stays in
// registers.

// (acc[2k+1]:acc[2k]) += x_k * y for k = 0..3 as one carry chain; returns the carry out of acc[7].
ZK_HD uint32_t madwide4_c(uint32_t* acc, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t y) {
#ifdef __CUDA_ARCH__
  uint32_t c;
  asm("mad.lo.cc.u32   %0, %9,  %13, %0;\n\t"
      "madc.hi.cc.u32  %1, %9,  %13, %1;\n\t"
      "madc.lo.cc.u32  %2, %10, %13, %2;\n\t"
      "madc.hi.cc.u32  %3, %10, %13, %3;\n\t"
      "madc.lo.cc.u32  %4, %11, %13, %4;\n\t"
      "madc.hi.cc.u32  %5, %11, %13, %5;\n\t"
      "madc.lo.cc.u32  %6, %12, %13, %6;\n\t"
      "madc.hi.cc.u32  %7, %12, %13, %7;\n\t"
      "addc.u32        %8, 0, 0;"
      : "+r"(acc[0]), "+r"(acc[1]), "+r"(acc[2]), "+r"(acc[3]), "+r"(acc[4]), "+r"(acc[5]), "+r"(acc[6]),
        "+r"(acc[7]), "=r"(c)
      : "r"(x0), "r"(x1), "r"(x2), "r"(x3), "r"(y));
  return c;
#else
  const uint32_t x[4] = {x0, x1, x2, x3};
  uint64_t carry = 0;
  for (int k = 0; k < 4; k++) {
    uint64_t p = (uint64_t)x[k] * y;
    uint64_t lo = (uint64_t)acc[2 * k] + (uint32_t)p + carry;
    acc[2 * k] = (uint32_t)lo;
    uint64_t hi = (uint64_t)acc[2 * k + 1] + (p >> 32) + (lo >> 32);
    acc[2 * k + 1] = (uint32_t)hi;
    carry = hi >> 32;
  }
  return (uint32_t)carry;
#endif
}

// Same chain when the caller has proved that nothing is carried out of acc[7].
ZK_HD void madwide4(uint32_t* acc, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t y) {
#ifdef __CUDA_ARCH__
  asm("mad.lo.cc.u32   %0, %8,  %12, %0;\n\t"
      "madc.hi.cc.u32  %1, %8,  %12, %1;\n\t"
      "madc.lo.cc.u32  %2, %9,  %12, %2;\n\t"
      "madc.hi.cc.u32  %3, %9,  %12, %3;\n\t"
      "madc.lo.cc.u32  %4, %10, %12, %4;\n\t"
      "madc.hi.cc.u32  %5, %10, %12, %5;\n\t"
      "madc.lo.cc.u32  %6, %11, %12, %6;\n\t"
      "madc.hi.u32     %7, %11, %12, %7;"
      : "+r"(acc[0]), "+r"(acc[1]), "+r"(acc[2]), "+r"(acc[3]), "+r"(acc[4]), "+r"(acc[5]), "+r"(acc[6]),
        "+r"(acc[7])
      : "r"(x0), "r"(x1), "r"(x2), "r"(x3), "r"(y));
#else
  (void)madwide4_c(acc, x0, x1, x2, x3, y);
#endif
}

// acc[0..7] += t (single limb), ripple through all eight limbs; the caller has proved no carry out.
ZK_HD void add_limb8(uint32_t* acc, uint32_t t) {
#ifdef __CUDA_ARCH__
  asm("add.cc.u32  %0, %0, %8;\n\t"
      "addc.cc.u32 %1, %1, 0;\n\t"
      "addc.cc.u32 %2, %2, 0;\n\t"
      "addc.cc.u32 %3, %3, 0;\n\t"
      "addc.cc.u32 %4, %4, 0;\n\t"
      "addc.cc.u32 %5, %5, 0;\n\t"
      "addc.cc.u32 %6, %6, 0;\n\t"
      "addc.u32    %7, %7, 0;"
      : "+r"(acc[0]), "+r"(acc[1]), "+r"(acc[2]), "+r"(acc[3]), "+r"(acc[4]), "+r"(acc[5]), "+r"(acc[6]),
        "+r"(acc[7])
      : "r"(t));
#else
  uint64_t c = t;
  for (int k = 0; k < 8; k++) {
    c += acc[k];
    acc[k] = (uint32_t)c;
    c >>= 32;
  }
#endif
}

// acc[0..8] += t (single limb) rippling through nine limbs; the caller has proved no carry out.
ZK_HD void add_limb9(uint32_t* acc, uint32_t t) {
#ifdef __CUDA_ARCH__
  asm("add.cc.u32  %0, %0, %9;\n\t"
      "addc.cc.u32 %1, %1, 0;\n\t"
      "addc.cc.u32 %2, %2, 0;\n\t"
      "addc.cc.u32 %3, %3, 0;\n\t"
      "addc.cc.u32 %4, %4, 0;\n\t"
      "addc.cc.u32 %5, %5, 0;\n\t"
      "addc.cc.u32 %6, %6, 0;\n\t"
      "addc.cc.u32 %7, %7, 0;\n\t"
      "addc.u32    %8, %8, 0;"
      : "+r"(acc[0]), "+r"(acc[1]), "+r"(acc[2]), "+r"(acc[3]), "+r"(acc[4]), "+r"(acc[5]), "+r"(acc[6]),
        "+r"(acc[7]), "+r"(acc[8])
      : "r"(t));
#else
  uint64_t c = t;
  for (int k = 0; k < 9; k++) {
    c += acc[k];
    acc[k] = (uint32_t)c;
    c >>= 32;
  }
#endif
}

// r = a + b over 8 limbs, returns the carry out.
ZK_HD uint32_t add8(uint32_t* r, const uint32_t* a, const uint32_t* b) {
#ifdef __CUDA_ARCH__
  uint32_t c;
  asm("add.cc.u32  %0, %9,  %17;\n\t"
      "addc.cc.u32 %1, %10, %18;\n\t"
      "addc.cc.u32 %2, %11, %19;\n\t"
      "addc.cc.u32 %3, %12, %20;\n\t"
      "addc.cc.u32 %4, %13, %21;\n\t"
      "addc.cc.u32 %5, %14, %22;\n\t"
      "addc.cc.u32 %6, %15, %23;\n\t"
      "addc.cc.u32 %7, %16, %24;\n\t"
      "addc.u32    %8, 0, 0;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(c)
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(b[0]),
        "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]));
  return c;
#else
  uint64_t c = 0;
  uint32_t t[8];
  for (int k = 0; k < 8; k++) {
    c += (uint64_t)a[k] + b[k];
    t[k] = (uint32_t)c;
    c >>= 32;
  }
  for (int k = 0; k < 8; k++) r[k] = t[k];
  return (uint32_t)c;
#endif
}

// r = a - b over 8 limbs, returns 1 when a < b (borrow), else 0.
ZK_HD uint32_t sub8(uint32_t* r, const uint32_t* a, const uint32_t* b) {
#ifdef __CUDA_ARCH__
  uint32_t c;
  asm("sub.cc.u32  %0, %9,  %17;\n\t"
      "subc.cc.u32 %1, %10, %18;\n\t"
      "subc.cc.u32 %2, %11, %19;\n\t"
      "subc.cc.u32 %3, %12, %20;\n\t"
      "subc.cc.u32 %4, %13, %21;\n\t"
      "subc.cc.u32 %5, %14, %22;\n\t"
      "subc.cc.u32 %6, %15, %23;\n\t"
      "subc.cc.u32 %7, %16, %24;\n\t"
      "subc.u32    %8, 0, 0;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(c)
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(b[0]),
        "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]), "r"(b[6]), "r"(b[7]));
  return c & 1u;
#else
  int64_t c = 0;
  uint32_t t[8];
  for (int k = 0; k < 8; k++) {
    c += (int64_t)a[k] - (int64_t)b[k];
    t[k] = (uint32_t)c;
    c >>= 32;  // arithmetic shift keeps the borrow as -1
  }
  for (int k = 0; k < 8; k++) r[k] = t[k];
  return c ? 1u : 0u;
#endif
}

// ------------------------------------------------------------------------------------------
// Field parameters.  mod(i), r2(i), one(i) return limb i; loops over them are fully unrolled
// so the values become immediates.

struct FrParams {  // BN254 scalar field
  static ZK_HD constexpr uint32_t mod(int i) {
    constexpr uint32_t m[8] = {0xf0000001u, 0x43e1f593u, 0x79b97091u, 0x2833e848u,
                               0x8181585du, 0xb85045b6u, 0xe131a029u, 0x30644e72u};
    return m[i];
  }
  static constexpr uint32_t inv = 0xefffffffu;  // -mod^-1 mod 2^32
  static ZK_HD constexpr uint32_t r2(int i) {   // R^2 mod p
    constexpr uint32_t m[8] = {0xae216da7u, 0x1bb8e645u, 0xe35c59e3u, 0x53fe3ab1u,
                               0x53bb8085u, 0x8c49833du, 0x7f4e44a5u, 0x0216d0b1u};
    return m[i];
  }
  static ZK_HD constexpr uint32_t one(int i) {  // R mod p
    constexpr uint32_t m[8] = {0x4ffffffbu, 0xac96341cu, 0x9f60cd29u, 0x36fc7695u,
                               0x7879462eu, 0x666ea36fu, 0x9a07df2fu, 0x0e0a77c1u};
    return m[i];
  }
  static ZK_HD constexpr uint32_t r3(int i) {  // R^3 mod p
    constexpr uint32_t m[8] = {0xb4bf0040u, 0x5e94d8e1u, 0x1cfbb6b8u, 0x2a489cbeu,
                               0xa19fcfedu, 0x893cc664u, 0x7fcc657cu, 0x0cf8594bu};
    return m[i];
  }
};

struct FqParams {  // BN254 base field
  static ZK_HD constexpr uint32_t mod(int i) {
    constexpr uint32_t m[8] = {0xd87cfd47u, 0x3c208c16u, 0x6871ca8du, 0x97816a91u,
                               0x8181585du, 0xb85045b6u, 0xe131a029u, 0x30644e72u};
    return m[i];
  }
  static constexpr uint32_t inv = 0xe4866389u;
  static ZK_HD constexpr uint32_t r2(int i) {
    constexpr uint32_t m[8] = {0x538afa89u, 0xf32cfc5bu, 0xd44501fbu, 0xb5e71911u,
                               0x0a417ff6u, 0x47ab1effu, 0xcab8351fu, 0x06d89f71u};
    return m[i];
  }
  static ZK_HD constexpr uint32_t one(int i) {
    constexpr uint32_t m[8] = {0xc58f0d9du, 0xd35d438du, 0xf5c70b3du, 0x0a78eb28u,
                               0x7879462cu, 0x666ea36fu, 0x9a07df2fu, 0x0e0a77c1u};
    return m[i];
  }
  static ZK_HD constexpr uint32_t r3(int i) {
    constexpr uint32_t m[8] = {0xda1530dfu, 0xb1cd6dafu, 0xa7283db6u, 0x62f210e6u,
                               0x0ada0afbu, 0xef7f0b0cu, 0x2d592544u, 0x20fd6e90u};
    return m[i];
  }
};

// ------------------------------------------------------------------------------------------
template <class P>
struct alignas(16) Fp {
  uint32_t v[8];

  static ZK_HD Fp zero() {
    Fp r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = 0;
    return r;
  }
  static ZK_HD Fp one() {
    Fp r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = P::one(i);
    return r;
  }
  static ZK_HD Fp modulus() {
    Fp r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = P::mod(i);
    return r;
  }
  static ZK_HD Fp r2() {
    Fp r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = P::r2(i);
    return r;
  }
  static ZK_HD Fp r3() {
    Fp r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.v[i] = P::r3(i);
    return r;
  }
  ZK_HD bool is_zero() const {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) o |= v[i];
    return o == 0;
  }
  ZK_HD bool operator==(const Fp& b) const {
    uint32_t o = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) o |= v[i] ^ b.v[i];
    return o == 0;
  }
  ZK_HD bool operator!=(const Fp& b) const { return !(*this == b); }
};

// r = (a < mod) ? a : a - mod, for a < 2*mod (carry = the 257th bit of a).
template <class P>
ZK_HD void final_sub(uint32_t* a, uint32_t carry) {
  uint32_t d[8], m[8];
#pragma unroll
  for (int i = 0; i < 8; i++) m[i] = P::mod(i);
  uint32_t borrow = sub8(d, a, m);
  // keep the difference when it did not borrow, or when the sum had overflowed 2^256
  bool take = (borrow == 0) | (carry != 0);
#pragma unroll
  for (int i = 0; i < 8; i++) a[i] = take ? d[i] : a[i];
}

template <class P>
ZK_HD Fp<P> add(const Fp<P>& a, const Fp<P>& b) {
  Fp<P> r;
  uint32_t c = add8(r.v, a.v, b.v);
  final_sub<P>(r.v, c);
  return r;
}

template <class P>
ZK_HD Fp<P> sub(const Fp<P>& a, const Fp<P>& b) {
  Fp<P> r;
  uint32_t borrow = sub8(r.v, a.v, b.v);
  uint32_t m[8], t[8];
#pragma unroll
  for (int i = 0; i < 8; i++) m[i] = borrow ? P::mod(i) : 0u;
  (void)add8(t, r.v, m);
#pragma unroll
  for (int i = 0; i < 8; i++) r.v[i] = t[i];
  return r;
}

template <class P>
ZK_HD Fp<P> neg(const Fp<P>& a) {
  return sub(Fp<P>::zero(), a);
}

template <class P>
ZK_HD Fp<P> dbl(const Fp<P>& a) {
  return add(a, a);
}

// Montgomery product a*b/R mod p.  `a` must be < p; `b` may be any 256-bit value.
//
// Operand scanning with two accumulators: E holds the 64-bit columns that start at even
// limbs, O the columns that start at odd limbs (O is offset by one limb), so every row of
// partial products is a chain of non-overlapping 32x32+64 multiply-adds.  After the
// reduction row the low limb of E is zero; dividing by 2^32 turns the odd columns into the
// even ones and vice versa, so the two arrays swap roles instead of shifting.
// Bounds: the running value E + 2^32*O stays below a + p, and below 2^32 (a + p) inside a
// row, so O fits 8 limbs and E needs one extra limb (e8) only inside a row.
template <class P>
ZK_HD Fp<P> mul(const Fp<P>& a, const Fp<P>& b) {
  uint32_t E[8], O[8];
#pragma unroll
  for (int i = 0; i < 8; i++) E[i] = O[i] = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t bi = b.v[i];
    uint32_t e8 = madwide4_c(E, a.v[0], a.v[2], a.v[4], a.v[6], bi);
    madwide4(O, a.v[1], a.v[3], a.v[5], a.v[7], bi);
    const uint32_t m = E[0] * P::inv;
    e8 += madwide4_c(E, P::mod(0), P::mod(2), P::mod(4), P::mod(6), m);
    madwide4(O, P::mod(1), P::mod(3), P::mod(5), P::mod(7), m);
    // divide by 2^32: new even = O + E[1]; new odd = E >> 64
    add_limb8(O, E[1]);
    uint32_t T[8];
#pragma unroll
    for (int k = 0; k < 6; k++) T[k] = E[k + 2];
    T[6] = e8;
    T[7] = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
      E[k] = O[k];
      O[k] = T[k];
    }
  }
  // value = E + 2^32 * O  (< 2p < 2^256)
  Fp<P> r;
  uint32_t S[8];
  S[0] = 0;
#pragma unroll
  for (int k = 1; k < 8; k++) S[k] = O[k - 1];
  (void)add8(r.v, E, S);
  final_sub<P>(r.v, 0);
  return r;
}

// Multiplication by a value that is fixed for a whole launch (a round challenge).
//
// For a fixed x the table holds c[j] = x * 2^(32 j + 64) mod p as plain integers.  Then for any
// d in Montgomery form, sum_j d_j c[j] = 2^64 * (x d) (mod p) needs 8 rows of 8 multiply-adds
// and no 512-bit intermediate; two Montgomery rounds remove the factor 2^64 and bring the
// 291-bit sum below 2^227 + p, so one conditional subtraction completes it: 82 multiply-adds
// against 136 for a general product.  The result is x*d in Montgomery form (d's own factor R).
template <class P>
struct FixedMul {
  uint32_t c[8][8];
};

// Build the table from x in Montgomery form (host or device).
template <class P>
ZK_HD FixedMul<P> make_fixed_mul(const Fp<P>& x_mont) {
  FixedMul<P> t;
  Fp<P> two64 = Fp<P>::zero();
  two64.v[2] = 1;
  Fp<P> two32 = Fp<P>::zero();
  two32.v[1] = 1;
  const Fp<P> step = to_mont(two32);  // 2^32 * R
  Fp<P> cur = mul(x_mont, two64);     // x * 2^64 as a plain integer mod p
  for (int j = 0; j < 8; j++) {
    for (int k = 0; k < 8; k++) t.c[j][k] = cur.v[k];
    cur = mul(cur, step);             // times 2^32
  }
  return t;
}

template <class P>
ZK_HD Fp<P> mul_fixed(const FixedMul<P>& t, const Fp<P>& d) {
  uint32_t E[9], O[9];
#pragma unroll
  for (int i = 0; i < 9; i++) E[i] = O[i] = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    E[8] += madwide4_c(E, t.c[j][0], t.c[j][2], t.c[j][4], t.c[j][6], d.v[j]);
    O[8] += madwide4_c(O, t.c[j][1], t.c[j][3], t.c[j][5], t.c[j][7], d.v[j]);
  }
#pragma unroll
  for (int round = 0; round < 2; round++) {
    const uint32_t m = E[0] * P::inv;
    E[8] += madwide4_c(E, P::mod(0), P::mod(2), P::mod(4), P::mod(6), m);
    O[8] += madwide4_c(O, P::mod(1), P::mod(3), P::mod(5), P::mod(7), m);
    // divide by 2^32: new even = O + E[1] (nine limbs), new odd = E >> 64
    add_limb9(O, E[1]);
    uint32_t T[9];
#pragma unroll
    for (int k = 0; k < 7; k++) T[k] = E[k + 2];
    T[7] = 0;
    T[8] = 0;
#pragma unroll
    for (int k = 0; k < 9; k++) {
      E[k] = O[k];
      O[k] = T[k];
    }
  }
  // value = E + 2^32 * O < 2^227 + p
  Fp<P> r;
  uint32_t S[8];
  S[0] = 0;
#pragma unroll
  for (int k = 1; k < 8; k++) S[k] = O[k - 1];
  (void)add8(r.v, E, S);
  final_sub<P>(r.v, 0);
  return r;
}

// t0 * d0 + t1 * d1 + t2 * d2 for three launch-constant multipliers in one accumulation: the
// three 291-bit row sums share the accumulators and one pair of Montgomery rounds, 210
// multiply-adds in all.  The d's may be any 256-bit values (unreduced differences).
template <class P>
ZK_HD Fp<P> mul_fixed3(const FixedMul<P>& t0, const uint32_t* d0, const FixedMul<P>& t1, const uint32_t* d1,
                       const FixedMul<P>& t2, const uint32_t* d2) {
  uint32_t E[9], O[9];
#pragma unroll
  for (int i = 0; i < 9; i++) E[i] = O[i] = 0;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    E[8] += madwide4_c(E, t0.c[j][0], t0.c[j][2], t0.c[j][4], t0.c[j][6], d0[j]);
    O[8] += madwide4_c(O, t0.c[j][1], t0.c[j][3], t0.c[j][5], t0.c[j][7], d0[j]);
    E[8] += madwide4_c(E, t1.c[j][0], t1.c[j][2], t1.c[j][4], t1.c[j][6], d1[j]);
    O[8] += madwide4_c(O, t1.c[j][1], t1.c[j][3], t1.c[j][5], t1.c[j][7], d1[j]);
    E[8] += madwide4_c(E, t2.c[j][0], t2.c[j][2], t2.c[j][4], t2.c[j][6], d2[j]);
    O[8] += madwide4_c(O, t2.c[j][1], t2.c[j][3], t2.c[j][5], t2.c[j][7], d2[j]);
  }
#pragma unroll
  for (int round = 0; round < 2; round++) {
    const uint32_t m = E[0] * P::inv;
    E[8] += madwide4_c(E, P::mod(0), P::mod(2), P::mod(4), P::mod(6), m);
    O[8] += madwide4_c(O, P::mod(1), P::mod(3), P::mod(5), P::mod(7), m);
    add_limb9(O, E[1]);
    uint32_t T[9];
#pragma unroll
    for (int k = 0; k < 7; k++) T[k] = E[k + 2];
    T[7] = 0;
    T[8] = 0;
#pragma unroll
    for (int k = 0; k < 9; k++) {
      E[k] = O[k];
      O[k] = T[k];
    }
  }
  // value = E + 2^32 * O < 3 * 2^225 + p < 2p
  Fp<P> r;
  uint32_t S[8];
  S[0] = 0;
#pragma unroll
  for (int k = 1; k < 8; k++) S[k] = O[k - 1];
  (void)add8(r.v, E, S);
  final_sub<P>(r.v, 0);
  return r;
}

// a + p - b without the conditional correction: any value congruent to a - b below 2p.
template <class P>
ZK_HD void sub_lazy(uint32_t* out, const Fp<P>& a, const Fp<P>& b) {
  uint32_t m[8], t[8];
#pragma unroll
  for (int i = 0; i < 8; i++) m[i] = P::mod(i);
  (void)add8(t, a.v, m);
  (void)sub8(out, t, b.v);
}

template <class P>
ZK_HD Fp<P> sqr(const Fp<P>& a) {
  return mul(a, a);
}

// 512-bit integer used for lazily reduced sums of products.
struct Wide {
  uint32_t v[16];
};

// Full 512-bit product of two 256-bit integers (no reduction).
// Even/odd column accumulators over 16 limbs; rows in increasing order so the limb that
// receives a row's carry has not been written before.
ZK_HD void mul_wide(Wide& out, const uint32_t* a, const uint32_t* b) {
  uint32_t E[16], O[16];  // O[k] sits at limb position k+1
#pragma unroll
  for (int i = 0; i < 16; i++) E[i] = O[i] = 0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    if ((i & 1) == 0) {
      E[i + 8] = madwide4_c(E + i, a[0], a[2], a[4], a[6], b[i]);
      madwide4(O + i, a[1], a[3], a[5], a[7], b[i]);  // top carry is zero: value < 2^(32(i+9))
    } else {
      O[i + 7] = madwide4_c(O + i - 1, a[0], a[2], a[4], a[6], b[i]);
      madwide4(E + i + 1, a[1], a[3], a[5], a[7], b[i]);
    }
  }
  // out = E + (O << 32)
  uint32_t S[8];
  S[0] = 0;
#pragma unroll
  for (int k = 1; k < 8; k++) S[k] = O[k - 1];
  uint32_t c = add8(out.v, E, S);
  // upper half with carry-in: fold the carry into the first addend limb chain
  uint32_t S2[8];
#pragma unroll
  for (int k = 0; k < 8; k++) S2[k] = O[k + 7];
  uint32_t hi[8];
#pragma unroll
  for (int k = 0; k < 8; k++) hi[k] = E[k + 8];
  add_limb8(hi, c);  // E's upper half + carry cannot overflow: the product fits 512 bits
  (void)add8(out.v + 8, hi, S2);
}

// acc += w over 16 limbs (caller keeps acc below 2^512).
ZK_HD void wide_add(Wide& acc, const Wide& w) {
  uint32_t c = add8(acc.v, acc.v, w.v);
  uint32_t hi[8];
#pragma unroll
  for (int k = 0; k < 8; k++) hi[k] = w.v[k + 8];
  // hi + c cannot overflow 2^256 for the products used here (w < p^2 < 2^508)
  add_limb8(hi, c);
  (void)add8(acc.v + 8, acc.v + 8, hi);
}

// Keep acc < p * 2^256 by subtracting p from the upper half when it is >= p.
// Valid while acc < 2 * p * 2^256, i.e. after adding at most 5 products of reduced operands
// to an accumulator that was below p * 2^256 (5 p^2 < p * 2^256 for both BN254 fields).
template <class P>
ZK_HD void wide_trim(Wide& acc) {
  final_sub<P>(acc.v + 8, 0);
}
constexpr int kLazyProducts = 5;

// Montgomery reduction of T < p * 2^256: returns T / 2^256 mod p, fully reduced.
// Only the low half goes through the reduction rows: (T_lo + M p) / 2^256 <= p, and the
// upper half (< p) is added afterwards, so one conditional subtraction finishes.
template <class P>
ZK_HD Fp<P> redc(const Wide& t) {
  uint32_t E[8], O[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    E[i] = t.v[i];
    O[i] = 0;
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t m = E[0] * P::inv;
    uint32_t e8 = madwide4_c(E, P::mod(0), P::mod(2), P::mod(4), P::mod(6), m);
    madwide4(O, P::mod(1), P::mod(3), P::mod(5), P::mod(7), m);
    add_limb8(O, E[1]);
    uint32_t T[8];
#pragma unroll
    for (int k = 0; k < 6; k++) T[k] = E[k + 2];
    T[6] = e8;
    T[7] = 0;
#pragma unroll
    for (int k = 0; k < 8; k++) {
      E[k] = O[k];
      O[k] = T[k];
    }
  }
  Fp<P> r;
  uint32_t S[8], lo[8];
  S[0] = 0;
#pragma unroll
  for (int k = 1; k < 8; k++) S[k] = O[k - 1];
  (void)add8(lo, E, S);                   // <= p
  uint32_t c = add8(r.v, lo, t.v + 8);    // < 2p < 2^256
  final_sub<P>(r.v, c);
  return r;
}

// Into / out of Montgomery form.
template <class P>
ZK_HD Fp<P> to_mont(const Fp<P>& canonical) {
  return mul(Fp<P>::r2(), canonical);
}
template <class P>
ZK_HD Fp<P> from_mont(const Fp<P>& a) {
  Fp<P> o = Fp<P>::zero();
  o.v[0] = 1;
  return mul(a, o);
}

// Small unsigned integer as a field element (Montgomery form).
template <class P>
ZK_HD Fp<P> from_u32(uint32_t x) {
  Fp<P> c = Fp<P>::zero();
  c.v[0] = x;
  return to_mont(c);
}

// a^e for a 256-bit exponent given as canonical limbs (square and multiply, MSB first).
template <class P>
ZK_HD Fp<P> pow_limbs(const Fp<P>& a, const uint32_t* e) {
  Fp<P> r = Fp<P>::one();
  for (int i = 7; i >= 0; i--) {
    for (int bit = 31; bit >= 0; bit--) {
      r = sqr(r);
      if ((e[i] >> bit) & 1u) r = mul(r, a);
    }
  }
  return r;
}

// Multiplicative inverse by Fermat (0 maps to 0).
template <class P>
ZK_HD Fp<P> inverse(const Fp<P>& a) {
  uint32_t e[8];
#pragma unroll
  for (int i = 0; i < 8; i++) e[i] = P::mod(i);
  e[0] -= 2;  // both moduli end in a limb > 2
  return pow_limbs(a, e);
}

using Fr = Fp<FrParams>;
using Fq = Fp<FqParams>;

}  // namespace zk
