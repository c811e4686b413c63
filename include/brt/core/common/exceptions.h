// BRT_ENFORCE / BRT_THROW (runtime/include/brt/core/common/common.h,
// exceptions.h): constructor-time failures are C++ exceptions; run-time failures
// are Status values.
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

namespace brt {

class BrtException : public std::runtime_error {
public:
  BrtException(const char *file, int line, const std::string &what)
      : std::runtime_error(Format(file, line, what)) {}

private:
  static std::string Format(const char *file, int line, const std::string &what) {
    std::ostringstream ss;
    ss << file << ":" << line << " " << what;
    return ss.str();
  }
};

class NotImplementedException : public std::logic_error {
public:
  explicit NotImplementedException(const std::string &what) : std::logic_error(what) {}
};

namespace detail {
inline std::string MakeMsg() { return ""; }
template <typename... Args> std::string MakeMsg(const Args &...args) {
  std::ostringstream ss;
  (ss << ... << args);
  return ss.str();
}
} // namespace detail
} // namespace brt

#define BRT_THROW(...) throw ::brt::BrtException(__FILE__, __LINE__, ::brt::detail::MakeMsg(__VA_ARGS__))

#define BRT_ENFORCE(cond, ...)                                                 \
  do {                                                                         \
    if (!(cond))                                                               \
      throw ::brt::BrtException(__FILE__, __LINE__,                            \
                                std::string("BRT_ENFORCE(" #cond ") failed. ") +\
                                    ::brt::detail::MakeMsg(__VA_ARGS__));      \
  } while (0)

#define BRT_NOT_IMPLEMENTED(...) throw ::brt::NotImplementedException(::brt::detail::MakeMsg(__VA_ARGS__))
