// Test doubles of the CUDA entry points used by Session (see fake_cuda.cpp).
#pragma once
#include <string>
#include <utility>
#include <vector>

#include "session.h"

namespace dep {
namespace fake {

void install(bool vmm_supported);                                // swap every entry of cuda_api() for a host-memory double
void restore();                                                  // back to the CUDA runtime / driver
// The (nth + 1)-th call of `entry` from now on returns `code` (a cudaError_t or CUresult value); code 0 removes the fault.
void fail(const std::string& entry, int nth, int code);
std::vector<std::pair<std::string, double>> log();               // (entry, CLOCK_MONOTONIC seconds) of every call so far
void clear();                                                    // forget the log, the call counts, the faults and leftover handles
int open_allocations();                                          // virtual-memory handles (own and imported) not yet released

}  // namespace fake
}  // namespace dep
