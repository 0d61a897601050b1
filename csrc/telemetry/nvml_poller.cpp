// Background NVML poller: one thread samples every visible GPU at a fixed interval and keeps
// the latest sample behind a mutex; the trainer reads snapshots without touching NVML itself
// (reference: nmoe/csrc/gpu.cpp:166-213).  NVML is opened with dlopen at start() so the
// library loads on machines without a driver, and every entry point is read-only: nothing
// here changes clocks, power limits or any other device setting.
#include <dlfcn.h>
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

namespace {

struct GpuSample {
  int32_t index;
  int32_t util_gpu, util_mem;
  int64_t mem_used, mem_total;
  int32_t power_mw, temp_c, sm_clock_mhz, sm_clock_max_mhz;
  uint64_t throttle_reasons;
  int64_t ecc_uncorrected;
  int64_t ts_ms;
};

typedef int (*fn_init)();
typedef int (*fn_shutdown)();
typedef int (*fn_count)(unsigned*);
typedef int (*fn_handle)(unsigned, void**);
struct NvmlUtil { unsigned gpu, memory; };
struct NvmlMem { unsigned long long total, free, used; };
typedef int (*fn_util)(void*, NvmlUtil*);
typedef int (*fn_mem)(void*, NvmlMem*);
typedef int (*fn_uint)(void*, unsigned*);
typedef int (*fn_temp)(void*, int, unsigned*);
typedef int (*fn_clock)(void*, int, unsigned*);
typedef int (*fn_u64)(void*, unsigned long long*);
typedef int (*fn_ecc)(void*, int, int, unsigned long long*);

struct Api {
  void* so = nullptr;
  fn_init init = nullptr; fn_shutdown shutdown = nullptr; fn_count count = nullptr; fn_handle handle = nullptr;
  fn_util util = nullptr; fn_mem mem = nullptr; fn_uint power = nullptr; fn_temp temp = nullptr;
  fn_clock clock = nullptr, max_clock = nullptr; fn_u64 throttle = nullptr; fn_ecc ecc = nullptr;
};

Api g_api;
std::mutex g_mu;
std::vector<GpuSample> g_latest;
std::thread g_thread;
std::atomic<bool> g_run{false};

bool load_api(const char* path) {
  g_api.so = dlopen(path && path[0] ? path : "libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!g_api.so) return false;
#define SYM(field, type, name) g_api.field = reinterpret_cast<type>(dlsym(g_api.so, name))
  SYM(init, fn_init, "nvmlInit_v2"); SYM(shutdown, fn_shutdown, "nvmlShutdown");
  SYM(count, fn_count, "nvmlDeviceGetCount_v2"); SYM(handle, fn_handle, "nvmlDeviceGetHandleByIndex_v2");
  SYM(util, fn_util, "nvmlDeviceGetUtilizationRates"); SYM(mem, fn_mem, "nvmlDeviceGetMemoryInfo");
  SYM(power, fn_uint, "nvmlDeviceGetPowerUsage"); SYM(temp, fn_temp, "nvmlDeviceGetTemperature");
  SYM(clock, fn_clock, "nvmlDeviceGetClockInfo"); SYM(max_clock, fn_clock, "nvmlDeviceGetMaxClockInfo");
  SYM(throttle, fn_u64, "nvmlDeviceGetCurrentClocksThrottleReasons");
  SYM(ecc, fn_ecc, "nvmlDeviceGetTotalEccErrors");
#undef SYM
  return g_api.init && g_api.count && g_api.handle;
}

void poll_loop(int interval_ms) {
  unsigned n = 0;
  if (g_api.count(&n) != 0) n = 0;
  std::vector<void*> handles(n, nullptr);
  for (unsigned i = 0; i < n; ++i) g_api.handle(i, &handles[i]);
  while (g_run.load()) {
    std::vector<GpuSample> cur(n);
    for (unsigned i = 0; i < n; ++i) {
      GpuSample s;
      memset(&s, 0, sizeof(s));
      s.index = static_cast<int32_t>(i);
      void* h = handles[i];
      NvmlUtil u{0, 0};
      if (g_api.util && g_api.util(h, &u) == 0) { s.util_gpu = u.gpu; s.util_mem = u.memory; }
      NvmlMem m{0, 0, 0};
      if (g_api.mem && g_api.mem(h, &m) == 0) { s.mem_used = m.used; s.mem_total = m.total; }
      unsigned v = 0;
      if (g_api.power && g_api.power(h, &v) == 0) s.power_mw = v;
      if (g_api.temp && g_api.temp(h, 0, &v) == 0) s.temp_c = v;
      if (g_api.clock && g_api.clock(h, 1, &v) == 0) s.sm_clock_mhz = v;          // 1 = SM clock domain
      if (g_api.max_clock && g_api.max_clock(h, 1, &v) == 0) s.sm_clock_max_mhz = v;
      unsigned long long r = 0;
      if (g_api.throttle && g_api.throttle(h, &r) == 0) s.throttle_reasons = r;
      if (g_api.ecc && g_api.ecc(h, 1, 0, &r) == 0) s.ecc_uncorrected = static_cast<int64_t>(r);  // uncorrected, volatile
      s.ts_ms = std::chrono::duration_cast<std::chrono::milliseconds>(
                    std::chrono::system_clock::now().time_since_epoch()).count();
      cur[i] = s;
    }
    {
      std::lock_guard<std::mutex> g(g_mu);
      g_latest.swap(cur);
    }
    for (int waited = 0; waited < interval_ms && g_run.load(); waited += 20)
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

}  // namespace

extern "C" {

// lib_path may be null/empty (default libnvidia-ml.so.1); tests pass a fake NVML library.
int nmoe_gpu_poller_start(int interval_ms, const char* lib_path) {
  if (g_run.load()) return 0;
  if (!g_api.so && !load_api(lib_path)) return -1;
  if (g_api.init() != 0) return -2;
  g_run.store(true);
  g_thread = std::thread(poll_loop, interval_ms < 20 ? 20 : interval_ms);
  return 0;
}

int nmoe_gpu_poller_stop() {
  if (!g_run.load()) return 0;
  g_run.store(false);
  if (g_thread.joinable()) g_thread.join();
  if (g_api.shutdown) g_api.shutdown();
  if (g_api.so) { dlclose(g_api.so); g_api = Api(); }
  std::lock_guard<std::mutex> g(g_mu);
  g_latest.clear();
  return 0;
}

int nmoe_gpu_poller_running() { return g_run.load() ? 1 : 0; }

// Copies up to max_gpus samples (13 int64 fields each) into out; returns the number copied.
int nmoe_gpu_poller_snapshot(int64_t* out, int max_gpus) {
  std::lock_guard<std::mutex> g(g_mu);
  int n = 0;
  for (const GpuSample& s : g_latest) {
    if (n >= max_gpus) break;
    int64_t* o = out + n * 13;
    o[0] = s.index; o[1] = s.util_gpu; o[2] = s.util_mem; o[3] = s.mem_used; o[4] = s.mem_total;
    o[5] = s.power_mw; o[6] = s.temp_c; o[7] = s.sm_clock_mhz; o[8] = s.sm_clock_max_mhz;
    o[9] = static_cast<int64_t>(s.throttle_reasons); o[10] = s.ecc_uncorrected; o[11] = s.ts_ms; o[12] = 0;
    ++n;
  }
  return n;
}

}  // extern "C"
