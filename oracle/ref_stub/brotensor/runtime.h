// Host-only stand-in for the brotensor runtime calls common.cpp makes.  TEST INFRASTRUCTURE ONLY.
#pragma once
#include "tensor.h"
namespace brotensor {
inline void init() {}
inline void sync_all() {}
}  // namespace brotensor
