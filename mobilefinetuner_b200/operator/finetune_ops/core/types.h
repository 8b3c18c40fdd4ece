// Element types and device tags of the operator API (same names and values as
// the reference's core/dtype.h and core/device.h so callers compile unchanged).
#pragma once
#include <cstdint>
#include <cstring>
#include <string>

namespace ops {

enum class DType : int8_t { kFloat32 = 0, kFloat16 = 1, kBFloat16 = 2, kInt32 = 3, kInt64 = 4, kInt8 = 5, kBool = 6, kUInt8 = 7 };

struct DTypeUtils {
    static size_t size_of(DType t) {
        static const size_t sz[8] = {4, 2, 2, 4, 8, 1, 1, 1};
        const int i = static_cast<int>(t);
        return (i >= 0 && i < 8) ? sz[i] : 0;
    }
    static std::string to_string(DType t) {
        static const char* nm[8] = {"float32", "float16", "bfloat16", "int32", "int64", "int8", "bool", "uint8"};
        const int i = static_cast<int>(t);
        return (i >= 0 && i < 8) ? nm[i] : "unknown";
    }
    static bool is_floating_point(DType t) { return t == DType::kFloat32 || t == DType::kFloat16 || t == DType::kBFloat16; }
    static bool is_integer(DType t) { return t == DType::kInt32 || t == DType::kInt64 || t == DType::kInt8; }
};

constexpr DType kFloat32 = DType::kFloat32;
constexpr DType kFloat16 = DType::kFloat16;
constexpr DType kBFloat16 = DType::kBFloat16;
constexpr DType kInt32 = DType::kInt32;
constexpr DType kInt64 = DType::kInt64;
constexpr DType kInt8 = DType::kInt8;
constexpr DType kBool = DType::kBool;
constexpr DType kUInt8 = DType::kUInt8;

// bfloat16 <-> float32, round to nearest even
inline uint16_t float32_to_bf16_bits(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);   // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
inline float bf16_bits_to_float32(uint16_t b) {
    const uint32_t u = static_cast<uint32_t>(b) << 16;
    float v;
    std::memcpy(&v, &u, 4);
    return v;
}
// IEEE half <-> float32 (round to nearest even, subnormals handled)
inline float fp16_bits_to_float32(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while (!(m & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 112) << 23) | (man << 13);
    float v;
    std::memcpy(&v, &u, 4);
    return v;
}
inline uint16_t float32_to_fp16_bits(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
    uint32_t man = u & 0x7fffffu;
    if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const int shift = 14 - exp;
        uint32_t r = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return (uint16_t)(sign | r);
}

enum class DeviceType : int8_t { kCPU = 0, kCUDA = 1, kMetal = 2 };

// The device tag is nominal: callers construct tensors with kCPU and hand them to ops::, which
// run on the process's CUDA device; Tensor::device() keeps reporting what the caller passed.
class Device {
public:
    Device(DeviceType type, int index = 0) : type_(type), index_(index) {}
    DeviceType type() const { return type_; }
    int index() const { return index_; }
    bool is_cpu() const { return type_ == DeviceType::kCPU; }
    bool is_cuda() const { return type_ == DeviceType::kCUDA; }
    bool is_metal() const { return type_ == DeviceType::kMetal; }
    std::string to_string() const {
        if (type_ == DeviceType::kCPU) return "cpu";
        return std::string(type_ == DeviceType::kCUDA ? "cuda:" : "metal:") + std::to_string(index_);
    }
    bool operator==(const Device& o) const { return type_ == o.type_ && index_ == o.index_; }
    bool operator!=(const Device& o) const { return !(*this == o); }
private:
    DeviceType type_;
    int index_;
};
const Device kCPU(DeviceType::kCPU, 0);
const Device kCUDA(DeviceType::kCUDA, 0);
const Device kMetal(DeviceType::kMetal, 0);

}  // namespace ops
