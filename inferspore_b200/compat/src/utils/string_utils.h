// String helpers with the names the InferSpore sources use (fmtstr, vec2str,
// arr2str; reference: src/utils/string_utils.h).
#pragma once
#include <cstdio>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

// printf-style formatting into a std::string.
template <typename... Args>
inline std::string fmtstr(const std::string& format, Args... args) {
    const int needed = std::snprintf(nullptr, 0, format.c_str(), args...);
    if (needed < 0) throw std::runtime_error("fmtstr: formatting failed");
    std::string out(static_cast<size_t>(needed) + 1, '\0');
    std::snprintf(&out[0], out.size(), format.c_str(), args...);
    out.resize(static_cast<size_t>(needed));
    return out;
}

// "(a, b, c)" for a vector.
template <typename T>
inline std::string vec2str(std::vector<T> vec) {
    std::ostringstream os;
    os << "(";
    for (size_t i = 0; i < vec.size(); ++i) os << (i ? ", " : "") << vec[i];
    os << ")";
    return os.str();
}

// "(a, b, c)" for the first `size` elements of an array.
template <typename T>
inline std::string arr2str(T* arr, size_t size) {
    std::ostringstream os;
    os << "(";
    for (size_t i = 0; i < size; ++i) os << (i ? ", " : "") << arr[i];
    os << ")";
    return os.str();
}
