/* CPU oracle (TEST INFRASTRUCTURE ONLY): BN254 G1 (y^2 = x^3 + 3 over Fq) and the bucket-method
 * multi-scalar multiplication.
 *
 * The reference takes both from ark-ec 0.5 (`VariableBaseMSM::msm`, called at
 * src/crypto/polycommit/kzh2.rs:640,658 and kzh3.rs:666,685,748,772), which is not vendored with it.  This
 * restates the published algorithms: Jacobian doubling (a = 0) and mixed addition from the explicit-formulas
 * literature, and the windowed bucket method as ark-ec describes it: window width c = ln(n) + 2 bits (3 below
 * 32 points), unsigned digits, 2^c - 1 buckets per window filled by mixed additions, a running-sum pass per
 * window, windows combined by c doublings each.  Scalars are used as the canonical integers they are: a
 * negative quantised weight lifted to r - |v| is a full-width scalar here, as it is for arkworks.
 * The result of an MSM is a unique group element, so any correct schedule compares equal after normalising. */
#pragma once
#include <cmath>
#include <thread>
#include <vector>
#include "field.h"

namespace orc {

struct Affine {
  Fq x, y;  // x = y = 0 encodes the point at infinity (not on the curve)
  bool is_inf() const { return x.is_zero() && y.is_zero(); }
};
struct Jac {
  Fq x, y, z;  // z = 0: infinity
  static Jac inf() { return Jac{Fq::one(), Fq::one(), Fq::zero()}; }
  bool is_inf() const { return z.is_zero(); }
};

inline Jac jac_double(const Jac& p) {  // dbl-2009-l (a = 0)
  if (p.is_inf()) return p;
  const Fq a = p.x * p.x, b = p.y * p.y, c = b * b;
  Fq d = (p.x + b) * (p.x + b) - a - c;
  d = d + d;
  const Fq e = a + a + a, f = e * e;
  Jac r;
  r.x = f - (d + d);
  Fq c8 = c + c;
  c8 = c8 + c8;
  c8 = c8 + c8;
  r.y = e * (d - r.x) - c8;
  r.z = p.y * p.z;
  r.z = r.z + r.z;
  return r;
}

inline Jac jac_add_affine(const Jac& p, const Affine& q) {  // madd-2007-bl
  if (q.is_inf()) return p;
  if (p.is_inf()) return Jac{q.x, q.y, Fq::one()};
  const Fq z1z1 = p.z * p.z, u2 = q.x * z1z1, s2 = q.y * p.z * z1z1;
  if (u2 == p.x) {
    if (s2 == p.y) return jac_double(p);
    return Jac::inf();
  }
  const Fq h = u2 - p.x, hh = h * h;
  Fq i = hh + hh;
  i = i + i;
  const Fq j = h * i;
  Fq rr = s2 - p.y;
  rr = rr + rr;
  const Fq v = p.x * i;
  Jac r;
  r.x = rr * rr - j - (v + v);
  Fq yj = p.y * j;
  yj = yj + yj;
  r.y = rr * (v - r.x) - yj;
  r.z = (p.z + h) * (p.z + h) - z1z1 - hh;
  return r;
}

inline Jac jac_add(const Jac& p, const Jac& q) {  // add-2007-bl
  if (p.is_inf()) return q;
  if (q.is_inf()) return p;
  const Fq z1z1 = p.z * p.z, z2z2 = q.z * q.z;
  const Fq u1 = p.x * z2z2, u2 = q.x * z1z1;
  const Fq s1 = p.y * q.z * z2z2, s2 = q.y * p.z * z1z1;
  if (u1 == u2) {
    if (s1 == s2) return jac_double(p);
    return Jac::inf();
  }
  const Fq h = u2 - u1;
  Fq i = h + h;
  i = i * i;
  const Fq j = h * i;
  Fq rr = s2 - s1;
  rr = rr + rr;
  const Fq v = u1 * i;
  Jac r;
  r.x = rr * rr - j - (v + v);
  Fq sj = s1 * j;
  sj = sj + sj;
  r.y = rr * (v - r.x) - sj;
  r.z = ((p.z + q.z) * (p.z + q.z) - z1z1 - z2z2) * h;
  return r;
}

inline Affine jac_to_affine(const Jac& p) {
  if (p.is_inf()) return Affine{Fq::zero(), Fq::zero()};
  const Fq zi = p.z.inverse(), zi2 = zi * zi;
  return Affine{p.x * zi2, p.y * zi2 * zi};
}

inline unsigned digit_at(const uint64_t* s, unsigned bit, unsigned c) {  // c <= 32 bits from position `bit`
  const unsigned limb = bit >> 6, off = bit & 63;
  if (limb >= 4) return 0;
  uint64_t v = s[limb] >> off;
  if (off + c > 64 && limb + 1 < 4) v |= s[limb + 1] << (64 - off);
  return (unsigned)(v & ((1ull << c) - 1));
}

// One bucket-method MSM over points [0, n): scalars are canonical little-endian integers (4 limbs each).
inline Jac msm_serial(const Affine* bases, const uint64_t* scalars, size_t n) {
  if (n == 0) return Jac::inf();
  const unsigned c = n < 32 ? 3u : (unsigned)(std::log((double)n)) + 2u;
  const unsigned windows = (254 + c - 1) / c;
  std::vector<Jac> window_sums(windows, Jac::inf());
  std::vector<Jac> buckets((size_t(1) << c) - 1);
  for (unsigned w = 0; w < windows; w++) {
    bool any = false;
    for (auto& b : buckets) b = Jac::inf();
    for (size_t i = 0; i < n; i++) {
      const unsigned d = digit_at(scalars + 4 * i, w * c, c);
      if (d) {
        buckets[d - 1] = jac_add_affine(buckets[d - 1], bases[i]);
        any = true;
      }
    }
    if (!any) continue;
    Jac running = Jac::inf(), sum = Jac::inf();
    for (size_t b = buckets.size(); b-- > 0;) {
      running = jac_add(running, buckets[b]);
      sum = jac_add(sum, running);
    }
    window_sums[w] = sum;
  }
  Jac acc = Jac::inf();
  for (unsigned w = windows; w-- > 0;) {
    for (unsigned k = 0; k < c; k++) acc = jac_double(acc);
    acc = jac_add(acc, window_sums[w]);
  }
  return acc;
}

// The same over `threads` contiguous ranges of the points, partial results added.
inline Jac msm(const Affine* bases, const uint64_t* scalars, size_t n, int threads) {
  if (threads < 1) threads = 1;
  if (n < 4096 || threads == 1) return msm_serial(bases, scalars, n);
  std::vector<Jac> part((size_t)threads, Jac::inf());
  std::vector<std::thread> th;
  const size_t chunk = (n + threads - 1) / threads;
  for (int t = 0; t < threads; t++) {
    const size_t b = std::min(n, chunk * t), e = std::min(n, chunk * (t + 1));
    th.emplace_back([=, &part] { part[t] = msm_serial(bases + b, scalars + 4 * b, e - b); });
  }
  for (auto& x : th) x.join();
  Jac acc = Jac::inf();
  for (auto& p : part) acc = jac_add(acc, p);
  return acc;
}

}  // namespace orc
