// Process-wide count of kernels launched by this library (what the benchmark
// reports as its own launches).
#pragma once

namespace b200c {

void note_kernel_launch(int n = 1);
unsigned long long kernel_launch_count();

} // namespace b200c
