// A fold entry point for hosts that must not allocate device memory.
//
// Some embedders of this library cannot call cudaMalloc at the point where they need a fold:
// a prover that has handed the whole of HBM to its own pool at start-up (a later cudaMalloc
// simply fails), or a service loop that is not allowed to hit the allocator's implicit
// device-wide synchronisation between requests.  zk_fold_lsb_static folds a device-resident
// table with caller-owned input and output and keeps its intermediate tables in the
// file-scope array below, which every GPU that loads the library holds until the process
// exits (1.5 MiB).  No zk_ctx is involved: creating one allocates.
#include "../../include/zkb200.h"
#include "ctx.hpp"

using namespace zk;

namespace {

constexpr uint32_t kStaticMaxVars = ZK_FOLD_STATIC_MAX_VARS;
constexpr size_t kPingElems = size_t(1) << (kStaticMaxVars - 1);
constexpr size_t kPongElems = size_t(1) << (kStaticMaxVars - 2);

// Intermediate tables of the k-step fold: [ping: 2^(max-1) elements][pong: 2^(max-2) elements].
static __device__ __align__(256) unsigned char g_fold_scratch[(kPingElems + kPongElems) * sizeof(Fr)];

constexpr int kMaxDevices = 64;
struct PerDevice {
  Fr* scratch = nullptr;  // device address of g_fold_scratch on this device
  int sm_count = 0;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_dev_mu;

// The array's name is only a handle in host code; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int device_setup(int device, PerDevice** out) {
  std::lock_guard<std::mutex> lk(g_dev_mu);
  PerDevice& d = g_dev[device];
  if (!d.scratch) {
    void* p = nullptr;
    ZK_CUDA(cudaGetSymbolAddress(&p, g_fold_scratch));
    int sms = 0;
    ZK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    d.sm_count = sms;
    d.scratch = reinterpret_cast<Fr*>(p);
  }
  *out = &d;
  return ZK_OK;
}

}  // namespace

extern "C" int zk_fold_lsb_static(uint32_t n, const uint64_t* evals_dev, uint32_t k, const uint64_t* point,
                                  uint64_t* out_dev, void* stream) {
  if (!evals_dev || !out_dev || (k && !point)) return fail(ZK_ERR_ARG, "fold_lsb_static: NULL argument");
  if (k > n) return fail(ZK_ERR_ARG, "invalid size of partial point");
  if (n > kStaticMaxVars)
    return fail(ZK_ERR_ARG, "fold_lsb_static: n = %u exceeds the static scratch limit of %u variables; use zk_fold_lsb",
                n, kStaticMaxVars);
  int device = 0;
  ZK_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return fail(ZK_ERR_ARG, "fold_lsb_static: device %d not supported", device);
  PerDevice* d = nullptr;
  int rc = device_setup(device, &d);
  if (rc != ZK_OK) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const uint64_t size = 1ull << n;
  const Fr* cur = reinterpret_cast<const Fr*>(evals_dev);
  Fr* out = reinterpret_cast<Fr*>(out_dev);
  if (k == 0) {
    ZK_CUDA(cudaMemcpyAsync(out, cur, size * sizeof(Fr), cudaMemcpyDeviceToDevice, s));
    return ZK_OK;
  }
  Fr* bufs[2] = {d->scratch, d->scratch + kPingElems};
  for (uint32_t i = 0; i < k; i++) {
    // step i writes 2^(n-i-1) elements: into the caller's output on the last step, otherwise
    // into ping (even steps, at most 2^(max-1)) or pong (odd steps, at most 2^(max-2))
    Fr* dst = (i + 1 == k) ? out : bufs[i & 1];
    Fr r;
    memcpy(r.v, point + 4 * (uint64_t)i, 32);
    launch_fold(cur, dst, r, size >> (i + 1), d->sm_count * 8, s);
    cur = dst;
  }
  ZK_CUDA(cudaGetLastError());
  return ZK_OK;
}
