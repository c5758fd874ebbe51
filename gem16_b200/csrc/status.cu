// Status transport for the C ABI: thread-local last-error string, launch checks, device gate.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace gemb {
namespace {
thread_local char g_last_error[512] = "";
}

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
  va_end(ap);
  return code;
}

int32_t check_launch(const char* op) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return GEMB_OK;
  return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
}

namespace {
struct DeviceInfo {
  int major = -1;
  int sms = 0;
};
DeviceInfo g_info[64];
}  // namespace

static const DeviceInfo* current_info(const char* op, int32_t* rc) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = fail(GEMB_UNSUPPORTED, "%s: no usable CUDA device (%s)", op,
               e == cudaSuccess ? "device index out of range" : cudaGetErrorName(e));
    cudaGetLastError();
    return nullptr;
  }
  DeviceInfo& info = g_info[dev];
  if (info.major < 0) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      *rc = fail(GEMB_UNSUPPORTED, "%s: cannot query the CUDA device", op);
      return nullptr;
    }
    info.sms = sms;
    info.major = major;
  }
  *rc = GEMB_OK;
  return &info;
}

int32_t require_sm100(const char* op) {
  int32_t rc;
  const DeviceInfo* info = current_info(op, &rc);
  if (!info) return rc;
  if (info->major != 10)
    return fail(GEMB_UNSUPPORTED, "%s: requires an sm_100 (B200) device, found compute capability %d.x",
                op, info->major);
  return GEMB_OK;
}

int sm_count() {
  int32_t rc;
  const DeviceInfo* info = current_info("sm_count", &rc);
  return info ? info->sms : 148;
}

}  // namespace gemb

extern "C" {

const char* gemb_last_error(void) { return gemb::g_last_error; }

const char* gemb_status_name(int32_t status) {
  switch (status) {
    case GEMB_OK: return "kOk";
    case GEMB_INVALID_ARGUMENT: return "kInvalidArgument";
    case GEMB_NOT_FOUND: return "kNotFound";
    case GEMB_IO_ERROR: return "kIoError";
    case GEMB_DATA_LOSS: return "kDataLoss";
    case GEMB_UNSUPPORTED: return "kUnsupported";
    case GEMB_RESOURCE_EXHAUSTED: return "kResourceExhausted";
    case GEMB_CANCELLED: return "kCancelled";
    case GEMB_INTERNAL: return "kInternal";
    default: return "unknown";
  }
}

int32_t gemb_abi_version(void) { return 1; }

int32_t gemb_device_check(void) { return gemb::require_sm100("gemb_device_check"); }

uint64_t gemb_interleaved_scale_bytes(uint64_t rows, uint64_t contracting_elements) {
  uint64_t r = (rows + 127) / 128 * 128;
  uint64_t c = (contracting_elements / 16 + 3) / 4 * 4;
  return r * c;
}

}  // extern "C"
