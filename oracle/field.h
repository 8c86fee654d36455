/* CPU oracle (TEST INFRASTRUCTURE ONLY): BN254 Fr / Fq arithmetic on 4 x 64-bit limbs.
 *
 * Restates what the reference gets from ark-ff 0.5 / ark-bn254 0.5 (not vendored with it):
 * prime-field arithmetic in Montgomery form with R = 2^256.  Written from the textbook CIOS
 * algorithm with unsigned __int128; independent of the library's 32-bit-limb device code.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may link this. */
#pragma once
#include <cstdint>
#include <cstring>

namespace orc {
typedef unsigned __int128 u128;

template <int FIELD>
struct FieldConst;
template <>
struct FieldConst<0> {  // Fr
  static constexpr uint64_t MOD[4] = {0x43e1f593f0000001ull, 0x2833e84879b97091ull, 0xb85045b68181585dull, 0x30644e72e131a029ull};
  static constexpr uint64_t INV = 0xc2e1f593efffffffull;  // -MOD^-1 mod 2^64
  static constexpr uint64_t R2[4] = {0x1bb8e645ae216da7ull, 0x53fe3ab1e35c59e3ull, 0x8c49833d53bb8085ull, 0x0216d0b17f4e44a5ull};
  static constexpr uint64_t ONE[4] = {0xac96341c4ffffffbull, 0x36fc76959f60cd29ull, 0x666ea36f7879462eull, 0x0e0a77c19a07df2full};
};
template <>
struct FieldConst<1> {  // Fq
  static constexpr uint64_t MOD[4] = {0x3c208c16d87cfd47ull, 0x97816a916871ca8dull, 0xb85045b68181585dull, 0x30644e72e131a029ull};
  static constexpr uint64_t INV = 0x87d20782e4866389ull;
  static constexpr uint64_t R2[4] = {0xf32cfc5b538afa89ull, 0xb5e71911d44501fbull, 0x47ab1eff0a417ff6ull, 0x06d89f71cab8351full};
  static constexpr uint64_t ONE[4] = {0xd35d438dc58f0d9dull, 0x0a78eb28f5c70b3dull, 0x666ea36f7879462cull, 0x0e0a77c19a07df2full};
};

template <int FIELD>
struct Fe {
  uint64_t l[4];
  typedef FieldConst<FIELD> C;

  static Fe zero() { Fe r; memset(r.l, 0, 32); return r; }
  static Fe one() { Fe r; memcpy(r.l, C::ONE, 32); return r; }
  bool is_zero() const { return (l[0] | l[1] | l[2] | l[3]) == 0; }
  bool operator==(const Fe& o) const { return !memcmp(l, o.l, 32); }
  bool operator!=(const Fe& o) const { return !(*this == o); }

  static bool geq_mod(const uint64_t* a) {
    for (int i = 3; i >= 0; i--) {
      if (a[i] > C::MOD[i]) return true;
      if (a[i] < C::MOD[i]) return false;
    }
    return true;
  }
  static void sub_mod(uint64_t* a) {
    u128 b = 0;
    for (int i = 0; i < 4; i++) {
      u128 d = (u128)a[i] - C::MOD[i] - (uint64_t)b;
      a[i] = (uint64_t)d;
      b = (d >> 64) & 1;
    }
  }
  Fe operator+(const Fe& o) const {
    Fe r;
    u128 c = 0;
    for (int i = 0; i < 4; i++) {
      c += (u128)l[i] + o.l[i];
      r.l[i] = (uint64_t)c;
      c >>= 64;
    }
    if (c || geq_mod(r.l)) sub_mod(r.l);
    return r;
  }
  Fe operator-(const Fe& o) const {
    Fe r;
    u128 b = 0;
    for (int i = 0; i < 4; i++) {
      u128 d = (u128)l[i] - o.l[i] - (uint64_t)b;
      r.l[i] = (uint64_t)d;
      b = (d >> 64) & 1;
    }
    if (b) {
      u128 c = 0;
      for (int i = 0; i < 4; i++) {
        c += (u128)r.l[i] + C::MOD[i];
        r.l[i] = (uint64_t)c;
        c >>= 64;
      }
    }
    return r;
  }
  Fe neg() const { return zero() - *this; }
  // Montgomery product (coarsely integrated operand scanning).
  Fe operator*(const Fe& o) const {
    uint64_t t[6] = {0, 0, 0, 0, 0, 0};
    for (int i = 0; i < 4; i++) {
      u128 c = 0;
      for (int j = 0; j < 4; j++) {
        c += (u128)l[j] * o.l[i] + t[j];
        t[j] = (uint64_t)c;
        c >>= 64;
      }
      c += t[4];
      t[4] = (uint64_t)c;
      t[5] = (uint64_t)(c >> 64);
      const uint64_t m = t[0] * C::INV;
      c = (u128)m * C::MOD[0] + t[0];
      c >>= 64;
      for (int j = 1; j < 4; j++) {
        c += (u128)m * C::MOD[j] + t[j];
        t[j - 1] = (uint64_t)c;
        c >>= 64;
      }
      c += t[4];
      t[3] = (uint64_t)c;
      t[4] = t[5] + (uint64_t)(c >> 64);
    }
    Fe r;
    memcpy(r.l, t, 32);
    if (t[4] || geq_mod(r.l)) sub_mod(r.l);
    return r;
  }
  // canonical integer (little-endian limbs) -> Montgomery form; any 256-bit input is reduced
  static Fe from_canonical(const uint64_t* c) {
    Fe x, r2;
    memcpy(x.l, c, 32);
    memcpy(r2.l, C::R2, 32);
    return r2 * x;
  }
  void to_canonical(uint64_t* out) const {
    Fe o = zero();
    o.l[0] = 1;
    Fe c = (*this) * o;
    memcpy(out, c.l, 32);
  }
  static Fe from_u64(uint64_t v) {
    uint64_t c[4] = {v, 0, 0, 0};
    return from_canonical(c);
  }
  Fe pow(const uint64_t* e) const {
    Fe r = one();
    for (int i = 3; i >= 0; i--)
      for (int b = 63; b >= 0; b--) {
        r = r * r;
        if ((e[i] >> b) & 1) r = r * (*this);
      }
    return r;
  }
  Fe inverse() const {  // Fermat; 0 -> 0
    uint64_t e[4];
    memcpy(e, C::MOD, 32);
    e[0] -= 2;
    return pow(e);
  }
};
typedef Fe<0> Fr;
typedef Fe<1> Fq;
}  // namespace orc
