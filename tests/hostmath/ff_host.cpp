// Host build of the device field / curve arithmetic, exported for the CPU unit tests.
// The carry chains compile to their portable C form here, so the algorithms (not the PTX)
// are what these symbols exercise.
#include "../../zkes_b200/csrc/ff.cuh"
#include <cstring>
using namespace zk;

template <class P> static void ld(Fp<P>& x, const uint32_t* p) { memcpy(x.v, p, 32); }

#define DEF(name, P)                                                                         \
  extern "C" void zkh_##name##_mul(const uint32_t* a, const uint32_t* b, uint32_t* r) {      \
    Fp<P> x, y; ld(x, a); ld(y, b); Fp<P> z = mul(x, y); memcpy(r, z.v, 32); }               \
  extern "C" void zkh_##name##_add(const uint32_t* a, const uint32_t* b, uint32_t* r) {      \
    Fp<P> x, y; ld(x, a); ld(y, b); Fp<P> z = add(x, y); memcpy(r, z.v, 32); }               \
  extern "C" void zkh_##name##_sub(const uint32_t* a, const uint32_t* b, uint32_t* r) {      \
    Fp<P> x, y; ld(x, a); ld(y, b); Fp<P> z = sub(x, y); memcpy(r, z.v, 32); }               \
  extern "C" void zkh_##name##_inv(const uint32_t* a, uint32_t* r) {                         \
    Fp<P> x; ld(x, a); Fp<P> z = inverse(x); memcpy(r, z.v, 32); }                           \
  extern "C" void zkh_##name##_to_mont(const uint32_t* a, uint32_t* r) {                     \
    Fp<P> x; ld(x, a); Fp<P> z = to_mont(x); memcpy(r, z.v, 32); }                           \
  extern "C" void zkh_##name##_from_mont(const uint32_t* a, uint32_t* r) {                   \
    Fp<P> x; ld(x, a); Fp<P> z = from_mont(x); memcpy(r, z.v, 32); }                         \
  extern "C" void zkh_##name##_mul_fixed(const uint32_t* x, const uint32_t* d, uint32_t* r) {  \
    Fp<P> a, b; ld(a, x); ld(b, d); FixedMul<P> t = make_fixed_mul(a);                        \
    Fp<P> z = mul_fixed(t, b); memcpy(r, z.v, 32); }                                         \
  /* x0*(a1-a0) + x1*(a2-a0) + x2*((a3-a2)-(a1-a0)) through mul_fixed3 with lazy differences */ \
  extern "C" void zkh_##name##_fold2(const uint32_t* x, const uint32_t* a, uint32_t* r) {      \
    Fp<P> x0, x1, t[4]; ld(x0, x); ld(x1, x + 8); for (int i = 0; i < 4; i++) ld(t[i], a + 8 * i); \
    FixedMul<P> f0 = make_fixed_mul(x0), f1 = make_fixed_mul(x1), f01 = make_fixed_mul(mul(x0, x1)); \
    uint32_t d01[8], d02[8], d23[8], dd[8], m2[8], tmp[8];                                    \
    sub_lazy<P>(d01, t[1], t[0]); sub_lazy<P>(d02, t[2], t[0]); sub_lazy<P>(d23, t[3], t[2]); \
    for (int i = 0; i < 8; i++) m2[i] = P::mod(i);                                            \
    add8(tmp, d23, m2); add8(tmp, tmp, m2); sub8(dd, tmp, d01);                               \
    Fp<P> z = add(t[0], mul_fixed3(f0, d01, f1, d02, f01, dd)); memcpy(r, z.v, 32); }         \
  /* sum of n products through the lazy accumulator, trimmed every kLazyProducts */         \
  extern "C" void zkh_##name##_dot(const uint32_t* a, const uint32_t* b, int n, uint32_t* r) { \
    Wide acc; memset(&acc, 0, sizeof acc); int pending = 0;                                  \
    for (int i = 0; i < n; i++) {                                                            \
      Wide w; mul_wide(w, a + 8 * i, b + 8 * i); wide_add(acc, w);                           \
      if (++pending == kLazyProducts) { wide_trim<P>(acc); pending = 0; }                    \
    }                                                                                        \
    wide_trim<P>(acc); Fp<P> z = redc<P>(acc); memcpy(r, z.v, 32); }

DEF(fr, FrParams)
DEF(fq, FqParams)

extern "C" void zkh_mul_wide(const uint32_t* a, const uint32_t* b, uint32_t* r) {
  Wide w; mul_wide(w, a, b); memcpy(r, w.v, 64);
}

// ---- G1 group law (ec.cuh) on Montgomery-form coordinates
#include "../../zkes_b200/csrc/ec.cuh"
static Affine ld_aff(const uint32_t* p) { Affine a; memcpy(a.x.v, p, 32); memcpy(a.y.v, p + 8, 32); return a; }
static void st_aff(uint32_t* p, const Affine& a) { memcpy(p, a.x.v, 32); memcpy(p + 8, a.y.v, 32); }
// out = normalised ((((k1 * a) + b) + (k2 * c as xyzz)) doubled `dbls` times)
extern "C" void zkh_g1_combo(const uint32_t* a, uint32_t k1, const uint32_t* b, const uint32_t* c, uint32_t k2,
                             int dbls, uint32_t* out) {
  Xyzz acc = mul_small(Xyzz::from_affine(ld_aff(a)), k1);
  acc = add_mixed(acc, ld_aff(b));
  acc = add(acc, mul_small(Xyzz::from_affine(ld_aff(c)), k2));
  for (int i = 0; i < dbls; i++) acc = dbl(acc);
  st_aff(out, to_affine(acc));
}
extern "C" void zkh_g1_jacobian(const uint32_t* a, uint32_t k, uint32_t* out) {
  Jacobian j = to_jacobian(mul_small(Xyzz::from_affine(ld_aff(a)), k));
  memcpy(out, j.x.v, 32); memcpy(out + 8, j.y.v, 32); memcpy(out + 16, j.z.v, 32);
}

// ---- device-form transcript (strobe_dev.cuh) driven from a raw 200-byte state
#include "../../zkes_b200/csrc/strobe_dev.cuh"
// state: 200 bytes + pos, pos_begin, cur_flags (3 x u32).  Appends n scalars (Montgomery) under
// "round_message", draws one "challenge"; writes the challenge (Montgomery) and the new state.
extern "C" void zkh_strobe_round(uint8_t* state200, uint32_t* pos3, const uint32_t* scalars, int n, uint32_t* challenge) {
  StrobeState st;
  memcpy(st.lanes, state200, 200);
  st.pos = pos3[0]; st.pos_begin = pos3[1]; st.cur_flags = pos3[2];
  for (int i = 0; i < n; i++) {
    Fr x; memcpy(x.v, scalars + 8 * i, 32);
    transcript_append_scalar_dev(st, "round_message", 13, x);
  }
  Fr c = transcript_challenge_scalar_dev(st, "challenge", 9);
  memcpy(challenge, c.v, 32);
  memcpy(state200, st.lanes, 200);
  pos3[0] = st.pos; pos3[1] = st.pos_begin; pos3[2] = st.cur_flags;
}
