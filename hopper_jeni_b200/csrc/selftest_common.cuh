// Shared by the translation units of the diagnostics library (libgqa_b200_selftest.so).
#pragma once

#include "gqa_common.cuh"

namespace gqa_selftest {

// 256-byte device status area of the self tests (a fixed device array of this library, one per GPU):
// word 0 takes the report of a bounded wait that gave up, bytes 8-23 the cycle counters of the issue-rate probe.
int status_area(unsigned int** out);

}  // namespace gqa_selftest
