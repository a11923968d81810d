// Error reporting of the host runtime: a failed check throws std::runtime_error with a composed message.
// The headers under csrc/host depend on the C++ standard library only, so the same code is compiled
// into the Python extension and into the sanitizer test binary (host_tests.cpp).
#pragma once
#include <sstream>
#include <stdexcept>
#include <string>

namespace cosmos {
namespace host {

template <typename... Args>
[[noreturn]] inline void fail(const Args&... args) {
  std::ostringstream os;
  (os << ... << args);
  throw std::runtime_error(os.str());
}

template <typename... Args>
inline void check(bool ok, const Args&... args) {
  if (!ok) fail(args...);
}

}  // namespace host
}  // namespace cosmos
