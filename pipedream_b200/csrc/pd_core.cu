// Library core: error string, device checks, version query.
#include "pd_common.cuh"
#include <mutex>

static thread_local char g_err[512] = "";

void pd_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

PD_EXPORT const char* pd_last_error() { return g_err; }

PD_EXPORT int pd_abi_version() { return 1; }

static std::mutex g_dev_mu;
static int g_dev_major[64];
static int g_dev_sms[64];
static bool g_dev_known[64];

static int pd_query_device(int* major, int* sms) {
  int dev = 0;
  PD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    pd_set_error("device ordinal %d out of range", dev);
    return PD_ERR_INVALID;
  }
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (!g_dev_known[dev]) {
    int mj = 0, n = 0;
    PD_CUDA(cudaDeviceGetAttribute(&mj, cudaDevAttrComputeCapabilityMajor, dev));
    PD_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    g_dev_major[dev] = mj;
    g_dev_sms[dev] = n;
    g_dev_known[dev] = true;
  }
  *major = g_dev_major[dev];
  *sms = g_dev_sms[dev];
  return PD_OK;
}

int pd_check_device() {
  int mj = 0, n = 0;
  int rc = pd_query_device(&mj, &n);
  if (rc != PD_OK) return rc;
  if (mj != 10) {
    pd_set_error("pipedream_b200 kernels are built for sm_100a only; current device is sm_%d0", mj);
    return PD_ERR_ARCH;
  }
  return PD_OK;
}

int pd_num_sms() {
  int mj = 0, n = 0;
  if (pd_query_device(&mj, &n) != PD_OK) return 148;
  return n > 0 ? n : 148;
}

PD_EXPORT int pd_device_ok() { return pd_check_device(); }
PD_EXPORT int pd_sm_count() { return pd_num_sms(); }
