// Library-level entry points of the es_b200 C ABI: version, error strings, per-device property cache.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace es_b200 {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int get_device_info(DeviceInfo* out) {
  constexpr int kMaxDevices = 64;
  static DeviceInfo cache[kMaxDevices];
  static bool valid[kMaxDevices] = {false};
  static std::mutex mu;
  int dev = 0;
  ES_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(ES_B200_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!valid[dev]) {
    DeviceInfo d;
    ES_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    ES_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    ES_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
    cache[dev] = d;
    valid[dev] = true;
  }
  *out = cache[dev];
  if (out->cc_major != 10)
    return fail(ES_B200_ERR_UNSUPPORTED_DEVICE, "es_b200 kernels are built for sm_100a only; device %d is sm_%d%d",
                dev, out->cc_major, out->cc_minor);
  return ES_B200_OK;
}

// Counts the device-side errors that es_b200_check_status has reported.  A kernel that gave up may have left the work
// counters of the call's scratch non-zero; whoever owns a scratch buffer compares this number with the one it saw when
// it last zeroed the buffer and zeroes it again when it has moved.
static std::atomic<uint64_t> g_error_epoch{0};
void note_device_error() { g_error_epoch.fetch_add(1, std::memory_order_relaxed); }

static int env_or(const char* name, int fallback) {
  const char* v = getenv(name);
  return v ? atoi(v) : fallback;
}

Tunables& tunables() {
  static Tunables t = {
      env_or("ES_B200_MM_HEAVY_MIN_ROWS", 0),      env_or("ES_B200_MM_TINY_MAX_ROWS", 0),
      env_or("ES_B200_MM_PAIR_FIRST_CLUSTERS", 32), env_or("ES_B200_MM_SPLIT_MIN_ROWS", 256),
      env_or("ES_B200_MM_STREAM_MAX_CTAS", 0),     env_or("ES_B200_MM_PAIR_MAX_CLUSTERS", 0),
      env_or("ES_B200_MM_DYNAMIC", 1),             env_or("ES_B200_MM_STREAM_LSU", 1),
      env_or("ES_B200_MM_ITEM_K_STEPS", 16), env_or("ES_B200_MM_STREAM_MID_LEAD_CTAS", -1),
  };
  return t;
}

}  // namespace es_b200

extern "C" int es_b200_set_tunable(const char* name, int value) {
  using namespace es_b200;
  ES_REQUIRE(name != nullptr, "null tunable name");
  Tunables& t = tunables();
  const struct { const char* n; int* p; } table[] = {
      {"mm_heavy_min_rows", &t.mm_heavy_min_rows},         {"mm_tiny_max_rows", &t.mm_tiny_max_rows},
      {"mm_pair_first_clusters", &t.mm_pair_first_clusters}, {"mm_split_min_rows", &t.mm_split_min_rows},
      {"mm_stream_max_ctas", &t.mm_stream_max_ctas},       {"mm_pair_max_clusters", &t.mm_pair_max_clusters},
      {"mm_dynamic", &t.mm_dynamic},                       {"mm_stream_lsu", &t.mm_stream_lsu},
      {"mm_item_k_steps", &t.mm_item_k_steps}, {"mm_stream_mid_lead_ctas", &t.mm_stream_mid_lead_ctas},
  };
  for (const auto& e : table)
    if (strcmp(e.n, name) == 0) {
      *e.p = value;
      return ES_B200_OK;
    }
  return fail(ES_B200_ERR_INVALID_ARGUMENT, "unknown tunable '%s'", name);
}

extern "C" uint64_t es_b200_error_epoch(void) { return es_b200::g_error_epoch.load(std::memory_order_relaxed); }

extern "C" const char* es_b200_version(void) { return "es_b200 0.2 (sm_100a)"; }

extern "C" const char* es_b200_last_error(void) { return es_b200::last_error_buffer(); }

extern "C" const char* es_b200_strerror(int code) {
  switch (code) {
    case ES_B200_OK: return "ok";
    case ES_B200_ERR_INVALID_ARGUMENT: return "invalid argument";
    case ES_B200_ERR_CUDA: return "CUDA error";
    case ES_B200_ERR_UNSUPPORTED_DEVICE: return "unsupported device (needs compute capability 10.x)";
    case ES_B200_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small";
    case ES_B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait timed out";
    default: return "unknown error code";
  }
}
