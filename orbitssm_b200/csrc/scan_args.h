// The scan kernels take the public argument block of include/orbit_b200.h by value.
#pragma once
#include "../../include/orbit_b200.h"

namespace orbit {
using ScanArgs = ::orbit_scan_args;
constexpr int SCAN_MAX_RANK = 8;   // largest d_ssm_in / d_ssm_out the kernels serve
}  // namespace orbit
