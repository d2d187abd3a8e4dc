// Fused MoE (MegaMoE) launchers.
#pragma once
#include "common.cuh"

namespace dep {
}  // namespace dep
