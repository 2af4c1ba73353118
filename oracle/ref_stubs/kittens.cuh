// Host stand-in for the ThunderKittens header the reference's hash_fns.cuh includes (the submodule is not part of the
// reference checkout).  Only what the REGISTER overloads of the hash functions touch: a shared-vector type that the
// unused shared-memory overloads name in their signatures, and laneid().  Test infrastructure only.
#pragma once
#include <stdint.h>
namespace kittens {
template <typename T, int N>
struct sv {
  T data[N * 32];
  T &operator[](int i) { return data[i]; }
  const T &operator[](int i) const { return data[i]; }
};
inline int laneid() { return 0; }
}  // namespace kittens
