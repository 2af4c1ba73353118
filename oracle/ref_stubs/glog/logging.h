// Stand-in for glog on hosts without it: LOG(severity) << ... swallows its operands.  Test infrastructure only.
#pragma once
#include <ostream>
namespace f3d_ref_stub {
struct NullLog {
  template <typename T> NullLog &operator<<(const T &) { return *this; }
  NullLog &operator<<(std::ostream &(*)(std::ostream &)) { return *this; }
};
}  // namespace f3d_ref_stub
#define LOG(severity) ::f3d_ref_stub::NullLog()
