// Allocation-free GEMV entry point: see wq_gemv_noalloc.h.  The scratch memory the split-k hand-off needs lives in a
// file-scope device array; its device address is looked up once per device, in this translation unit.
#include "wq_gemv_noalloc.h"

#include <mutex>
#include <stdio.h>

#include "wq_gemv.cuh"

namespace {

struct NoAllocScratch {
  float partials[B2_NOALLOC_SCRATCH_FLOATS];
  unsigned counters[B2_NOALLOC_MAX_ITEMS];
  int status[64];
};

// Held by every GPU that loads this library until the process exits (about 4.03 MiB).
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
NoAllocScratch* g_dev_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device ordinal

void set_err(char* err, const char* msg) {
  if (err) snprintf(err, 160, "%s", msg);
}

// The array's name is only a host-side stand-in; kernels need its device address, which differs per device.
int scratch_for_current_device(NoAllocScratch** out, char* err) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_err(err, "b2_wq_gemv_noalloc: cannot identify the current device");
    return 2;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_dev_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      set_err(err, "b2_wq_gemv_noalloc: cudaGetSymbolAddress failed for the built-in scratch array");
      return 2;
    }
    g_dev_ptr[dev] = static_cast<NoAllocScratch*>(p);
  }
  *out = g_dev_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int b2_wq_gemv_noalloc(const uint8_t* wq, int n, int k, int bits, int group, int ks, const void* x_bf16, long ldx,
                                  int m, void* y_bf16, long ldy, int* status_out, cudaStream_t stream, char* err) {
  if (!wq || !x_bf16 || !y_bf16 || n <= 0 || k <= 0 || m <= 0 || m > 32 || n % 32 || k % 128 || ks < 1 ||
      (k / 128) % ks || (bits != 2 && bits != 3 && bits != 4) || (group != 64 && group != 128)) {
    set_err(err, "b2_wq_gemv_noalloc: bad argument (n % 32, k % 128, ks | k/128, bits in 2..4, group 64|128, 1 <= m <= 32)");
    return 1;
  }
  const int rb = 2;
  const long need = b2_wq_gemv_scratch_floats(n, k, ks, rb, m);
  if (need > (long)B2_NOALLOC_SCRATCH_FLOATS || n / 32 > B2_NOALLOC_MAX_ITEMS) {
    if (err)
      snprintf(err, 160, "b2_wq_gemv_noalloc: problem needs %ld scratch floats / %d items; the built-in array holds %d / %d",
               need, n / 32, (int)B2_NOALLOC_SCRATCH_FLOATS, (int)B2_NOALLOC_MAX_ITEMS);
    return 1;
  }
  NoAllocScratch* s = nullptr;
  const int rc = scratch_for_current_device(&s, err);
  if (rc) return rc;
  // Counters and the status word must start at zero whatever an earlier (possibly failed) call left there.
  if (cudaMemsetAsync(s->counters, 0, sizeof(unsigned) * (size_t)(n / 32), stream) != cudaSuccess ||
      cudaMemsetAsync(s->status, 0, sizeof(int), stream) != cudaSuccess) {
    set_err(err, "b2_wq_gemv_noalloc: cudaMemsetAsync failed");
    return 2;
  }
  b2::WqGemvArgs a = {};
  a.wq = wq;
  a.n = n; a.k = k; a.m = m;
  a.bits = bits; a.group = group;
  a.ks = ks; a.rb = rb;
  a.vworkers = b2_wq_gemv_vworkers(n, k, ks, rb);
  a.fmax = b2_wq_gemv_fmax(n, k, ks, rb);
  a.pro = b2::PRO_PLAIN;
  a.x = static_cast<const bf16*>(x_bf16); a.ldx = ldx;
  a.epi = b2::EPI_STORE;
  a.y = static_cast<bf16*>(y_bf16); a.ldy = ldy;
  a.scratch = s->partials;
  a.counters = s->counters;
  a.status = s->status;
  const int st = b2_wq_gemv(&a, stream);
  if (st != 0) {
    set_err(err, st == 1 ? "b2_wq_gemv_noalloc: the GEMV launcher rejected the arguments (alignment of x / ldx?)"
                         : "b2_wq_gemv_noalloc: kernel launch failed");
    return st == 1 ? 1 : 2;
  }
  if (status_out &&
      cudaMemcpyAsync(status_out, s->status, sizeof(int), cudaMemcpyDeviceToDevice, stream) != cudaSuccess) {
    set_err(err, "b2_wq_gemv_noalloc: status copy failed");
    return 2;
  }
  return 0;
}
