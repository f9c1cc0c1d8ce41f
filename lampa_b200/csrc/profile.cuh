// Optional per-kernel timing with CUDA events on the launching stream (off by default).
#pragma once
#include <cuda_runtime.h>

namespace lampa {

bool prof_enabled();
void prof_mark(const char* name, cudaStream_t st, bool begin);

// Brackets one kernel launch with two events when profiling is on; free otherwise.
struct ProfScope {
    const char* name;
    cudaStream_t st;
    bool on;
    ProfScope(const char* n, cudaStream_t s) : name(n), st(s), on(prof_enabled()) {
        if (on) prof_mark(name, st, true);
    }
    ~ProfScope() {
        if (on) prof_mark(name, st, false);
    }
};

}  // namespace lampa
