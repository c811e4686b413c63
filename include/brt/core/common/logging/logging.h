// A small logger behind the reference's macro names
// (runtime/include/brt/core/common/logging/macros.h: BRT_LOGS_DEFAULT(severity)).
#pragma once

#include <iostream>
#include <sstream>

namespace brt {
namespace logging {

enum class Severity { kVERBOSE = 0, kINFO = 1, kWARNING = 2, kERROR = 3, kFATAL = 4 };

class Logger {
public:
  static Severity &MinSeverity() {
    static Severity s = Severity::kWARNING; // the reference's tests run at WARNING
    return s;
  }
};

class Capture {
public:
  Capture(Severity sev, const char *file, int line) : sev_(sev) {
    static const char *names[] = {"V", "I", "W", "E", "F"};
    ss_ << "[brt " << names[(int)sev] << " " << file << ":" << line << "] ";
  }
  ~Capture() {
    if ((int)sev_ >= (int)Logger::MinSeverity())
      std::cerr << ss_.str() << std::endl;
  }
  std::ostream &Stream() { return ss_; }

private:
  Severity sev_;
  std::ostringstream ss_;
};

} // namespace logging
} // namespace brt

#define BRT_LOGS_DEFAULT(severity)                                             \
  ::brt::logging::Capture(::brt::logging::Severity::k##severity, __FILE__, __LINE__).Stream()
