// BN254 G1 (y^2 = x^3 + 3 over Fq) point arithmetic for the MSM pipeline.
//
// Stands in for ark-ec's short-Weierstrass group law behind `P::G1::msm` (call sites
// src/crypto/polycommit/kzh2.rs:640,658 and kzh3.rs:666,685,748,772).  Bucket sums use extended
// Jacobian coordinates (X, Y, ZZ, ZZZ) with x = X/ZZ, y = Y/ZZZ and ZZ^3 = ZZZ^2: a mixed
// addition costs 8M + 2S and needs no inversion.  Formulas are the published "xyzz" ones for
// a = 0 (add-2008-s, madd-2008-s, dbl-2008-s-1, mdbl-2008-s-1).  A group element has many
// representations; results are compared after normalising to affine.
#pragma once
#include "ff.cuh"

namespace zk {

struct alignas(16) Affine {  // the point at infinity is encoded as x = y = 0
  Fq x, y;
  ZK_HD bool is_inf() const { return x.is_zero() && y.is_zero(); }
};

struct alignas(16) Xyzz {  // infinity: zz == 0
  Fq x, y, zz, zzz;
  ZK_HD bool is_inf() const { return zz.is_zero(); }
  static ZK_HD Xyzz inf() {
    Xyzz p;
    p.x = Fq::zero();
    p.y = Fq::zero();
    p.zz = Fq::zero();
    p.zzz = Fq::zero();
    return p;
  }
  static ZK_HD Xyzz from_affine(const Affine& a) {
    if (a.is_inf()) return inf();
    Xyzz p;
    p.x = a.x;
    p.y = a.y;
    p.zz = Fq::one();
    p.zzz = Fq::one();
    return p;
  }
};

struct alignas(16) Jacobian {  // x = X/Z^2, y = Y/Z^3, infinity: Z == 0
  Fq x, y, z;
};

ZK_HD Affine neg(const Affine& a) {
  Affine r;
  r.x = a.x;
  r.y = a.y.is_zero() ? a.y : sub(Fq::zero(), a.y);
  return r;
}

ZK_HD Xyzz neg(const Xyzz& a) {
  Xyzz r = a;
  r.y = sub(Fq::zero(), a.y);
  return r;
}

// 2 * (affine point), mdbl-2008-s-1.
ZK_HD Xyzz dbl_affine(const Affine& a) {
  if (a.is_inf() || a.y.is_zero()) return Xyzz::inf();
  Xyzz r;
  const Fq u = dbl(a.y), v = sqr(u), w = mul(u, v), s = mul(a.x, v);
  const Fq x2 = sqr(a.x), m = add(dbl(x2), x2);
  r.x = sub(sqr(m), dbl(s));
  r.y = sub(mul(m, sub(s, r.x)), mul(w, a.y));
  r.zz = v;
  r.zzz = w;
  return r;
}

// 2 * p, dbl-2008-s-1.
ZK_HD Xyzz dbl(const Xyzz& p) {
  if (p.is_inf() || p.y.is_zero()) return Xyzz::inf();
  Xyzz r;
  const Fq u = dbl(p.y), v = sqr(u), w = mul(u, v), s = mul(p.x, v);
  const Fq x2 = sqr(p.x), m = add(dbl(x2), x2);
  r.x = sub(sqr(m), dbl(s));
  r.y = sub(mul(m, sub(s, r.x)), mul(w, p.y));
  r.zz = mul(v, p.zz);
  r.zzz = mul(w, p.zzz);
  return r;
}

// The doubling that an addition falls into when both operands are the same point: rare, so on the
// device it is a call rather than a second copy of the formulas inside every addition (the kernels'
// code has to stay within the instruction cache).
#ifdef __CUDACC__
static __device__ __noinline__ void dbl_rare(Xyzz* r, const Xyzz* p) { *r = dbl(*p); }
static __device__ __noinline__ void dbl_affine_rare(Xyzz* r, const Affine* a) { *r = dbl_affine(*a); }
#endif

// p + (affine q), madd-2008-s with the exceptional cases handled.
ZK_HD Xyzz add_mixed(const Xyzz& p, const Affine& q) {
  if (q.is_inf()) return p;
  if (p.is_inf()) return Xyzz::from_affine(q);
  const Fq u2 = mul(q.x, p.zz), s2 = mul(q.y, p.zzz);
  const Fq pp_ = sub(u2, p.x), r_ = sub(s2, p.y);
  if (pp_.is_zero()) {
    if (!r_.is_zero()) return Xyzz::inf();
#ifdef __CUDA_ARCH__
    Xyzz d;
    dbl_affine_rare(&d, &q);
    return d;
#else
    return dbl_affine(q);
#endif
  }
  Xyzz r;
  const Fq pp = sqr(pp_), ppp = mul(pp_, pp), q_ = mul(p.x, pp);
  r.x = sub(sub(sqr(r_), ppp), dbl(q_));
  r.y = sub(mul(r_, sub(q_, r.x)), mul(p.y, ppp));
  r.zz = mul(p.zz, pp);
  r.zzz = mul(p.zzz, ppp);
  return r;
}

// p + q, add-2008-s with the exceptional cases handled.
ZK_HD Xyzz add(const Xyzz& p, const Xyzz& q) {
  if (q.is_inf()) return p;
  if (p.is_inf()) return q;
  const Fq u1 = mul(p.x, q.zz), u2 = mul(q.x, p.zz);
  const Fq s1 = mul(p.y, q.zzz), s2 = mul(q.y, p.zzz);
  const Fq pp_ = sub(u2, u1), r_ = sub(s2, s1);
  if (pp_.is_zero()) {
    if (!r_.is_zero()) return Xyzz::inf();
#ifdef __CUDA_ARCH__
    Xyzz d;
    dbl_rare(&d, &p);
    return d;
#else
    return dbl(p);
#endif
  }
  Xyzz r;
  const Fq pp = sqr(pp_), ppp = mul(pp_, pp), q_ = mul(u1, pp);
  r.x = sub(sub(sqr(r_), ppp), dbl(q_));
  r.y = sub(mul(r_, sub(q_, r.x)), mul(s1, ppp));
  r.zz = mul(mul(p.zz, q.zz), pp);
  r.zzz = mul(mul(p.zzz, q.zzz), ppp);
  return r;
}

// Same point in Jacobian form: (X*ZZ, Y*ZZZ, ZZ) since ZZ^3 = ZZZ^2.
ZK_HD Jacobian to_jacobian(const Xyzz& p) {
  Jacobian j;
  if (p.is_inf()) {
    j.x = Fq::one();
    j.y = Fq::one();
    j.z = Fq::zero();
    return j;
  }
  j.x = mul(p.x, p.zz);
  j.y = mul(p.y, p.zzz);
  j.z = p.zz;
  return j;
}

// Affine form given the inverses of zz and zzz are computed here (one field inversion).
ZK_HD Affine to_affine(const Xyzz& p) {
  Affine a;
  if (p.is_inf()) {
    a.x = Fq::zero();
    a.y = Fq::zero();
    return a;
  }
  // 1/zzz, then 1/zz = zzz^-2 * zz^2  (zz^3 = zzz^2  =>  zz^-1 = zz^2 / zzz^2)
  const Fq izzz = inverse(p.zzz);
  const Fq izz = mul(sqr(izzz), sqr(p.zz));
  a.x = mul(p.x, izz);
  a.y = mul(p.y, izzz);
  return a;
}

// One copy of the full addition / doubling per translation unit, for kernels that add in many
// places (tree reductions, running sums): operands go through memory, which costs a few per cent
// of an addition and keeps those kernels a fraction of their inlined size.
#ifdef __CUDA_ARCH__
static __device__ __noinline__ void add_to(Xyzz* acc, const Xyzz* q) { *acc = add(*acc, *q); }
static __device__ __noinline__ void dbl_in_place(Xyzz* acc) { *acc = dbl(*acc); }
#else
inline void add_to(Xyzz* acc, const Xyzz* q) { *acc = add(*acc, *q); }
inline void dbl_in_place(Xyzz* acc) { *acc = dbl(*acc); }
#endif

// k * p for a small unsigned k (double and add, MSB first).
ZK_HD Xyzz mul_small(const Xyzz& p, uint32_t k) {
  Xyzz acc = Xyzz::inf();
  int top = 31;
  while (top >= 0 && !((k >> top) & 1u)) top--;  // skip the leading zero bits
  for (int bit = top; bit >= 0; bit--) {
    dbl_in_place(&acc);
    if ((k >> bit) & 1u) add_to(&acc, &p);
  }
  return acc;
}

}  // namespace zk
