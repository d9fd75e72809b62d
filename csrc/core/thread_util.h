// Thread placement helpers (reference: rust/thread-lib/src/lib.rs:4-16).
#pragma once

#include <string>
#include <vector>

namespace pplx {

// Pins the calling thread to one logical CPU. Throws pplx::Error on failure.
void pin_cpu(int cpu);
// CPUs the calling thread may run on.
std::vector<int> current_affinity();
void set_thread_name(const std::string& name);

}  // namespace pplx
