// Host-side status plumbing shared by every entry point of libcda_b200.so.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace cda {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return CDA_OK;
  return fail(CDA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

int device_sm_count(int device) {
  static int cached[64];
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return 148; }
  if (device >= 0 && device < 64 && cached[device] > 0) return cached[device];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 148;   // B200; only reached when no device is visible (host-only planning calls)
  }
  if (device >= 0 && device < 64) cached[device] = n;
  return n;
}

}  // namespace cda

extern "C" int cda_b200_version(void) { return CDA_B200_ABI_VERSION; }

extern "C" const char* cda_b200_last_error_string(void) { return cda::g_err; }

extern "C" int cda_b200_slot_bytes(int k_bits, int v_bits) {
  if (!cda::bits_ok(k_bits) || !cda::bits_ok(v_bits))
    return cda::fail(CDA_ERR_UNSUPPORTED, "k_bits/v_bits must be 2 or 4 (got %d/%d)", k_bits, v_bits);
  return cda::slot_bytes_for(k_bits, v_bits);
}
