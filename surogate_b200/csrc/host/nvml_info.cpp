// Read-only GPU telemetry through NVML, loaded with dlopen so the host runtime has no link-time dependency on the driver.
// Only getters are resolved: nothing here can change a clock, a power limit or any other device setting.
// Reference counterpart: csrc/src/utilities/gpu_info.cpp.
#include <dlfcn.h>

#include <mutex>

#include "host_api.h"

namespace sg {

namespace {
using nvmlDevice_t = void*;
struct NvmlUtil { unsigned gpu, memory; };
struct NvmlMem { unsigned long long total, free, used; };
struct Api {
    void* lib = nullptr;
    int (*init)() = nullptr;
    int (*get_handle)(unsigned, nvmlDevice_t*) = nullptr;
    int (*name)(nvmlDevice_t, char*, unsigned) = nullptr;
    int (*clock)(nvmlDevice_t, int, unsigned*) = nullptr;
    int (*max_clock)(nvmlDevice_t, int, unsigned*) = nullptr;
    int (*power)(nvmlDevice_t, unsigned*) = nullptr;
    int (*power_limit)(nvmlDevice_t, unsigned*) = nullptr;
    int (*temp)(nvmlDevice_t, int, unsigned*) = nullptr;
    int (*util)(nvmlDevice_t, NvmlUtil*) = nullptr;
    int (*mem)(nvmlDevice_t, NvmlMem*) = nullptr;
    int (*throttle)(nvmlDevice_t, unsigned long long*) = nullptr;
    int (*pcie)(nvmlDevice_t, int, unsigned*) = nullptr;
    bool ok = false;
};
Api& api() {
    static Api a;
    static std::once_flag once;
    std::call_once(once, [] {
        a.lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
        if (!a.lib) return;
        auto sym = [&](const char* n) { return dlsym(a.lib, n); };
        a.init = reinterpret_cast<int (*)()>(sym("nvmlInit_v2"));
        a.get_handle = reinterpret_cast<int (*)(unsigned, nvmlDevice_t*)>(sym("nvmlDeviceGetHandleByIndex_v2"));
        a.name = reinterpret_cast<int (*)(nvmlDevice_t, char*, unsigned)>(sym("nvmlDeviceGetName"));
        a.clock = reinterpret_cast<int (*)(nvmlDevice_t, int, unsigned*)>(sym("nvmlDeviceGetClockInfo"));
        a.max_clock = reinterpret_cast<int (*)(nvmlDevice_t, int, unsigned*)>(sym("nvmlDeviceGetMaxClockInfo"));
        a.power = reinterpret_cast<int (*)(nvmlDevice_t, unsigned*)>(sym("nvmlDeviceGetPowerUsage"));
        a.power_limit = reinterpret_cast<int (*)(nvmlDevice_t, unsigned*)>(sym("nvmlDeviceGetEnforcedPowerLimit"));
        a.temp = reinterpret_cast<int (*)(nvmlDevice_t, int, unsigned*)>(sym("nvmlDeviceGetTemperature"));
        a.util = reinterpret_cast<int (*)(nvmlDevice_t, NvmlUtil*)>(sym("nvmlDeviceGetUtilizationRates"));
        a.mem = reinterpret_cast<int (*)(nvmlDevice_t, NvmlMem*)>(sym("nvmlDeviceGetMemoryInfo"));
        a.throttle = reinterpret_cast<int (*)(nvmlDevice_t, unsigned long long*)>(sym("nvmlDeviceGetCurrentClocksThrottleReasons"));
        a.pcie = reinterpret_cast<int (*)(nvmlDevice_t, int, unsigned*)>(sym("nvmlDeviceGetPcieThroughput"));
        a.ok = a.init && a.get_handle && a.init() == 0;
    });
    return a;
}
}  // namespace

GpuTelemetry query_gpu(int index) {
    GpuTelemetry t;
    Api& a = api();
    if (!a.ok) { t.error = a.lib ? "nvmlInit failed" : "libnvidia-ml.so.1 not found"; return t; }
    nvmlDevice_t dev = nullptr;
    if (a.get_handle(static_cast<unsigned>(index), &dev) != 0) { t.error = "no such device"; return t; }
    char name[96] = {0};
    if (a.name && a.name(dev, name, sizeof name) == 0) t.name = name;
    if (a.clock) { a.clock(dev, 1, &t.sm_clock_mhz); a.clock(dev, 2, &t.mem_clock_mhz); }  // 1 = SM, 2 = memory
    if (a.max_clock) a.max_clock(dev, 1, &t.sm_clock_max_mhz);
    if (a.power) a.power(dev, &t.power_mw);
    if (a.power_limit) a.power_limit(dev, &t.power_limit_mw);
    if (a.temp) a.temp(dev, 0, &t.temperature_c);
    NvmlUtil u{0, 0};
    if (a.util && a.util(dev, &u) == 0) { t.gpu_util = u.gpu; t.mem_util = u.memory; }
    NvmlMem m{0, 0, 0};
    if (a.mem && a.mem(dev, &m) == 0) { t.mem_used = m.used; t.mem_total = m.total; }
    if (a.throttle) a.throttle(dev, &t.throttle_reasons);
    unsigned rx = 0, tx = 0;
    if (a.pcie) { a.pcie(dev, 1, &rx); a.pcie(dev, 0, &tx); }  // 0 = TX, 1 = RX (KB/s)
    t.pcie_rx_kbs = rx;
    t.pcie_tx_kbs = tx;
    t.ok = true;
    return t;
}

}  // namespace sg
