#include "memory_manager.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

#include "mft_cuda.h"

namespace ops {

MemoryManager& MemoryManager::instance() {
    static MemoryManager m;
    return m;
}
// The reference's loops call these after every step to hand host memory back to the OS.  On the device the cache is
// what makes the next step allocation-free, so only what exceeds a high-water mark (MFT_CACHE_HIGH_WATER_MB,
// default 16 GiB) is returned to the driver.
static int64_t cache_high_water() {
    static const int64_t v = [] {
        const char* e = std::getenv("MFT_CACHE_HIGH_WATER_MB");
        return (e ? std::atoll(e) : 16384LL) << 20;
    }();
    return v;
}
void MemoryManager::force_cleanup() { mft_trim_cache(cache_high_water()); }
void MemoryManager::clear_unused_memory() { mft_trim_cache(cache_high_water()); }
size_t MemoryManager::device_bytes_in_use() const { int64_t s[6] = {0}; mft_mem_stats(s); return (size_t)s[0]; }
size_t MemoryManager::device_bytes_cached() const { int64_t s[6] = {0}; mft_mem_stats(s); return (size_t)s[1]; }
void MemoryManager::print_memory_stats() const {
    int64_t s[6] = {0};
    mft_mem_stats(s);
    std::cout << "[memory] device in use " << s[0] / (1 << 20) << " MiB, cached " << s[1] / (1 << 20) << " MiB, peak " << s[2] / (1 << 20)
              << " MiB, driver allocations " << s[3] << ", reuses " << s[4] << ", host RSS " << MemoryMonitor::get_system_memory_usage() / (1 << 20) << " MiB" << std::endl;
}

static size_t read_status_kb(const char* key) {
    FILE* f = std::fopen("/proc/self/status", "r");
    if (!f) return 0;
    char line[256];
    size_t kb = 0;
    const size_t n = std::strlen(key);
    while (std::fgets(line, sizeof line, f))
        if (std::strncmp(line, key, n) == 0) { std::sscanf(line + n, "%zu", &kb); break; }
    std::fclose(f);
    return kb;
}
size_t MemoryMonitor::get_system_memory_usage() { return read_status_kb("VmRSS:") * 1024; }
size_t MemoryMonitor::get_peak_memory_usage() { return read_status_kb("VmHWM:") * 1024; }

}  // namespace ops
