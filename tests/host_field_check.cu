// Host-only check of the 64-bit-limb inversion used for the affine form of commitments (csrc/msm.hpp) against the
// shared 32-bit-limb field code: inverse_host(a) == inverse(a), a * inverse_host(a) == 1, 0 -> 0, for both BN254 fields.
// Built and run by tests/test_host_field_cpu.py; prints "ok" and exits 0 when every case agrees.
#include "internal.hpp"
#include "msm.hpp"

#include <cstdio>
#include <cstring>

using namespace zk;

template <class F>
static int run(const char* name) {
  F a = F::one();
  int bad = 0;
  for (int i = 0; i < 400; i++) {
    a.v[i % 8] ^= 0x9e3779b9u * (uint32_t)(i + 1);
    a.v[7] &= 0x0fffffffu;  // below both moduli
    const F x = inverse(a), y = inverse_host(a);
    if (memcmp(&x, &y, sizeof(F)) != 0) bad++;
    const F one = mul(a, y);
    const F want = F::one();
    if (!a.is_zero() && memcmp(&one, &want, sizeof(F)) != 0) bad++;
  }
  // edge values: 0, 1, p - 1
  const F z = inverse_host(F::zero());
  if (!z.is_zero()) bad++;
  const F o1 = inverse_host(F::one()), w1 = F::one();
  if (memcmp(&o1, &w1, sizeof(F)) != 0) bad++;
  const F m1 = neg(F::one()), im1 = inverse_host(m1);
  if (memcmp(&im1, &m1, sizeof(F)) != 0) bad++;  // (-1)^(-1) = -1
  if (bad) printf("%s: %d mismatches\n", name, bad);
  return bad;
}

int main() {
  const int bad = run<Fq>("Fq") + run<Fr>("Fr");
  if (!bad) printf("ok\n");
  return bad ? 1 : 0;
}
