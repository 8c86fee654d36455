// Device-resident KZH structured reference string (shared by the KZH entry points).
#pragma once
#include "msm.hpp"

struct zk_kzh_srs {
  int dims = 0;
  uint32_t n = 0, x_log = 0, y_log = 0, z_log = 0;
  zk::Affine* h[3] = {nullptr, nullptr, nullptr};  // full (2^n or this rank's slab), mid (2^(n - x_log)), low (2^z_log, KZH3)
  uint64_t count[3] = {0, 0, 0};
  int rank = 0, world = 1;      // sharded SRS: h[0] holds entries [slab_begin, slab_begin + count[0]) of the full vector
  uint64_t slab_begin = 0;
};

