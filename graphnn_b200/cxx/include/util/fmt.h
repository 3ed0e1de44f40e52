// Minimal fmt::sprintf (printf-style formatting into std::string) for driver code that
// names things with it; the reference vendors a full formatting library for the same use.
#ifndef S2V_FMT_H
#define S2V_FMT_H

#include <cstdio>
#include <string>

namespace fmt
{
namespace detail
{
inline const char* arg(const std::string& s) { return s.c_str(); }
template <typename T> inline T arg(T v) { return v; }
}  // namespace detail

template <typename... Args>
inline std::string sprintf(const char* format, Args... args)
{
    const int n = std::snprintf(nullptr, 0, format, detail::arg(args)...);
    if (n <= 0) return std::string();
    std::string out((size_t)n + 1, '\0');
    std::snprintf(&out[0], out.size(), format, detail::arg(args)...);
    out.resize((size_t)n);
    return out;
}
inline std::string sprintf(const std::string& format) { return format; }
}  // namespace fmt
#endif
