// Memory facade with the reference's entry points (core/memory_manager.h): callers keep invoking
// MemoryManager::instance().force_cleanup() etc.; behind it sits the caching device allocator of
// libmft_cuda.so, which is trimmed rather than emptied so steady-state steps never re-allocate.
#pragma once
#include <cstddef>
#include <string>

namespace ops {

class MemoryManager {
public:
    static MemoryManager& instance();
    void force_cleanup();               // returns cached device blocks to the driver
    void clear_unused_memory();
    void cleanup_dead_references() {}
    void print_memory_stats() const;
    size_t device_bytes_in_use() const;
    size_t device_bytes_cached() const;
private:
    MemoryManager() = default;
};

class MemoryMonitor {
public:
    static size_t get_system_memory_usage();   // resident set size of this process, bytes
    static size_t get_peak_memory_usage();
};

}  // namespace ops
