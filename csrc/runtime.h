// Native host-side runtime pieces: the paged-KV block allocator used by the Reasoner's
// decode path and the checkpoint reader (torch-free cores under csrc/host). Registered as torch custom
// classes so Python holds them by reference and calls cost no interpreter-level loops.
#pragma once
#include <torch/library.h>

namespace cosmos {
void register_runtime_ops(torch::Library& m);
// memory-mapped safetensors reader (safetensors_reader.cpp)
void register_safetensors(torch::Library& m);
}
