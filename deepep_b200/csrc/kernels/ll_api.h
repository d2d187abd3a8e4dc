// Low-latency (decode) dispatch/combine launchers.
#pragma once
#include "common.cuh"

namespace dep {
}  // namespace dep
