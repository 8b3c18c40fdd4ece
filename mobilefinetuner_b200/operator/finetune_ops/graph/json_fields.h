// Minimal field extraction from a HuggingFace config.json (flat keys, numbers / strings / string arrays).
#pragma once
#include <filesystem>
#include <fstream>
#include <regex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace ops {
namespace detail {

inline std::string read_config_text(const std::string& path_or_dir) {
    namespace fs = std::filesystem;
    fs::path p(path_or_dir);
    if (fs::is_directory(p)) p /= "config.json";
    std::ifstream f(p);
    if (!f.is_open()) throw std::runtime_error("cannot open " + p.string());
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}
inline bool json_number(const std::string& js, const std::string& key, double* out) {
    std::smatch m;
    if (std::regex_search(js, m, std::regex("\"" + key + "\"\\s*:\\s*(-?[0-9][0-9eE\\.+-]*)"))) { *out = std::stod(m[1]); return true; }
    return false;
}
inline int json_int(const std::string& js, const std::string& key, int dflt) { double v; return json_number(js, key, &v) ? (int)v : dflt; }
inline float json_float(const std::string& js, const std::string& key, float dflt) { double v; return json_number(js, key, &v) ? (float)v : dflt; }
inline bool json_bool(const std::string& js, const std::string& key, bool dflt) {
    std::smatch m;
    return std::regex_search(js, m, std::regex("\"" + key + "\"\\s*:\\s*(true|false)")) ? m[1] == "true" : dflt;
}
inline std::string json_string(const std::string& js, const std::string& key, const std::string& dflt) {
    std::smatch m;
    return std::regex_search(js, m, std::regex("\"" + key + "\"\\s*:\\s*\"([^\"]*)\"")) ? std::string(m[1]) : dflt;
}
inline std::vector<std::string> json_string_array(const std::string& js, const std::string& key) {
    std::vector<std::string> out;
    std::smatch m;
    if (!std::regex_search(js, m, std::regex("\"" + key + "\"\\s*:\\s*\\[([^\\]]*)\\]"))) return out;
    const std::string arr = m[1];
    const std::regex item("\"([^\"]*)\"");
    for (std::sregex_iterator it(arr.begin(), arr.end(), item), end; it != end; ++it) out.push_back((*it)[1]);
    return out;
}

}  // namespace detail
}  // namespace ops
