/* CPU oracle (TEST INFRASTRUCTURE ONLY): C entry points over the G1 restatement (g1.h) in the library's wire
 * form: affine points {x[4], y[4]} Montgomery mod q with zeros for infinity, scalars Fr in Montgomery form,
 * results Jacobian {X, Y, Z} Montgomery mod q. */
#include <algorithm>
#include "g1.h"

namespace orc {
extern int g_threads;
}
using namespace orc;

static std::vector<uint64_t> canonical_scalars(const uint64_t* scalars, size_t n) {
  std::vector<uint64_t> out(4 * n);
  for (size_t i = 0; i < n; i++) {
    Fr s;
    memcpy(s.l, scalars + 4 * i, 32);
    s.to_canonical(out.data() + 4 * i);
  }
  return out;
}

extern "C" {

// P::G1::msm(bases, scalars): out = sum_i scalars[i] * bases[i].
void orc_g1_msm(uint64_t n, const uint64_t* bases, const uint64_t* scalars, uint64_t* out_jac) {
  static_assert(sizeof(Affine) == 64 && sizeof(Jac) == 96, "wire layout");
  const std::vector<uint64_t> sc = canonical_scalars(scalars, n);
  const Jac r = msm(reinterpret_cast<const Affine*>(bases), sc.data(), n, g_threads);
  memcpy(out_jac, &r, 96);
}

// The d_x loop of kzh2_commit / kzh3_commit (kzh2.rs:653-660, kzh3.rs:680-687): n_rows MSMs over the same bases,
// one rayon task per row in the reference, one thread per block of rows here.
void orc_g1_msm_rows(uint64_t n_bases, uint64_t n_rows, const uint64_t* bases, const uint64_t* scalars, uint64_t* out_jac) {
  const std::vector<uint64_t> sc = canonical_scalars(scalars, n_bases * n_rows);
  int t = g_threads < 1 ? 1 : g_threads;
  std::vector<std::thread> th;
  const uint64_t chunk = (n_rows + t - 1) / t;
  for (int k = 0; k < t; k++) {
    const uint64_t b = std::min(n_rows, chunk * k), e = std::min(n_rows, chunk * (k + 1));
    th.emplace_back([=, &sc] {
      for (uint64_t r = b; r < e; r++) {
        const Jac p = msm_serial(reinterpret_cast<const Affine*>(bases), sc.data() + 4 * r * n_bases, n_bases);
        memcpy(out_jac + 12 * r, &p, 96);
      }
    });
  }
  for (auto& x : th) x.join();
}

// CurveGroup::into_affine for n Jacobian points.
void orc_g1_normalize(uint64_t n, const uint64_t* jac, uint64_t* affine_out) {
  for (uint64_t i = 0; i < n; i++) {
    Jac p;
    memcpy(&p, jac + 12 * i, 96);
    const Affine a = jac_to_affine(p);
    memcpy(affine_out + 8 * i, &a, 64);
  }
}

// k * P by double-and-add (k canonical, 4 limbs), for building test bases.
void orc_g1_mul(const uint64_t* base_affine, const uint64_t* k_canonical, uint64_t* out_jac) {
  Affine b;
  memcpy(&b, base_affine, 64);
  Jac acc = Jac::inf();
  for (int i = 255; i >= 0; i--) {
    acc = jac_double(acc);
    if ((k_canonical[i >> 6] >> (i & 63)) & 1) acc = jac_add_affine(acc, b);
  }
  memcpy(out_jac, &acc, 96);
}

}  // extern "C"
