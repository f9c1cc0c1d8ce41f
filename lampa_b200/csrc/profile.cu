// Per-kernel CUDA-event timing for the benchmark's roofline figures.
#include "profile.cuh"

#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/lampa_b200.h"

namespace lampa {

namespace {
struct Rec { const char* name; cudaEvent_t a, b; bool closed; };
std::mutex g_mu;
bool g_on = false;
std::vector<Rec> g_recs;
}  // namespace

bool prof_enabled() { return g_on; }

void prof_mark(const char* name, cudaStream_t st, bool begin) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (begin) {
        Rec r{name, nullptr, nullptr, false};
        if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
        cudaEventRecord(r.a, st);
        g_recs.push_back(r);
    } else {
        for (size_t i = g_recs.size(); i-- > 0;)
            if (!g_recs[i].closed && g_recs[i].name == name) {
                cudaEventRecord(g_recs[i].b, st);
                g_recs[i].closed = true;
                break;
            }
    }
}

}  // namespace lampa

using namespace lampa;

extern "C" int lampa_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& r : g_recs) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    g_recs.clear();
    g_on = on != 0;
    return LAMPA_OK;
}

extern "C" int lampa_profile_read(char* names, size_t names_cap, float* total_ms, int32_t* launches,
                                  int32_t max_kernels, int32_t* n_kernels) {
    if (!names || !total_ms || !launches || !n_kernels || max_kernels <= 0) return LAMPA_ERR_ARG;
    std::lock_guard<std::mutex> lk(g_mu);
    std::map<std::string, std::pair<double, int>> agg;
    std::vector<std::string> order;
    for (auto& r : g_recs) {
        if (!r.closed) continue;
        if (cudaEventSynchronize(r.b) != cudaSuccess) return LAMPA_ERR_CUDA;
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) != cudaSuccess) return LAMPA_ERR_CUDA;
        auto it = agg.find(r.name);
        if (it == agg.end()) { agg[r.name] = {ms, 1}; order.push_back(r.name); }
        else { it->second.first += ms; it->second.second += 1; }
    }
    size_t pos = 0;
    int n = 0;
    for (auto& nm : order) {
        if (n >= max_kernels || pos + nm.size() + 2 > names_cap) break;
        std::memcpy(names + pos, nm.c_str(), nm.size());
        pos += nm.size();
        names[pos++] = '\n';
        total_ms[n] = (float)agg[nm].first;
        launches[n] = agg[nm].second;
        ++n;
    }
    names[pos] = '\0';
    *n_kernels = n;
    return LAMPA_OK;
}
