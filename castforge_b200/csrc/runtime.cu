// Host-side runtime helpers shared by every entry point: status/last-error text and cached
// device properties.  No device code lives here.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace cfb {

static thread_local char t_last_error[512] = "";

int32_t set_error(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_last_error, sizeof t_last_error, fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64];  // zero-initialised; one slot per device ordinal
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static long long g_tunables[kTuneCount] = {0, 0, 0, 1, 0, 60, 1, 0, 0, 0, 1, 1, 1};  // a1_persist on; 60 MB of a group's tail kept in L2 and re-read first
static const char* const kTunableNames[kTuneCount] = {"a1_keep_mb", "a1_demote", "a1_merge", "a1_persist", "a1_group_mb", "a1_retain_mb", "gemv_ring", "gemv_ring_rounds", "w4_split_k", "a1_bar_sleep", "a1_tail_first", "gemm_pair", "colpar_p2p"};

long long tunable(int id) { return (id >= 0 && id < kTuneCount) ? g_tunables[id] : 0; }

}  // namespace cfb

extern "C" int32_t cfb200_tune(const char* key, int64_t value) {
  if (key)
    for (int i = 0; i < cfb::kTuneCount; ++i)
      if (strcmp(key, cfb::kTunableNames[i]) == 0) {
        cfb::g_tunables[i] = value;
        return CFB200_OK;
      }
  return cfb::set_error(CFB200_ERR_INVALID, "unknown tunable '%s'", key ? key : "(null)");
}

extern "C" int32_t cfb200_selftest_expired_wait(int32_t which, int32_t* observed_host) {
  if (!observed_host) return cfb::set_error(CFB200_ERR_INVALID, "NULL argument");
  *observed_host = 0;
  if (which == 0) return cfb::a1_expired_wait_selftest(observed_host);
  if (which >= 1 && which <= 3) return cfb::tc_expired_wait_selftest(observed_host, which - 1);
  return cfb::set_error(CFB200_ERR_INVALID, "unknown self-test %d", which);
}

extern "C" const char* cfb200_last_error(void) { return cfb::t_last_error; }
extern "C" const char* cfb200_version(void) { return "0.1.0"; }
