// Optional per-kernel timing with CUDA events on the launching stream.  Off by default; when
// enabled (odmkv_timing_enable(1)) the launchers bracket their dominant kernels with event pairs,
// and odmkv_timing_read sums the elapsed time per kernel name after synchronising the events.
#include "common.cuh"

#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace odmkv {

struct EventPair { cudaEvent_t a, b; };
static std::mutex g_mu;
static bool g_on = false;
static std::map<std::string, std::vector<EventPair>> g_events;
static std::vector<EventPair> g_open;   // begin() without end(), per call nesting depth 1
static std::vector<std::string> g_open_names;

bool timing_on() { return g_on; }

void timing_begin(const char *name, cudaStream_t st) {
    if (!g_on) return;
    std::lock_guard<std::mutex> lk(g_mu);
    EventPair p;
    cudaEventCreate(&p.a);
    cudaEventCreate(&p.b);
    cudaEventRecord(p.a, st);
    g_open.push_back(p);
    g_open_names.push_back(name);
}

void timing_end(cudaStream_t st) {
    if (!g_on) return;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_open.empty()) return;
    EventPair p = g_open.back();
    std::string name = g_open_names.back();
    g_open.pop_back();
    g_open_names.pop_back();
    cudaEventRecord(p.b, st);
    g_events[name].push_back(p);
}

}  // namespace odmkv

extern "C" {

void odmkv_timing_enable(int on) {
    std::lock_guard<std::mutex> lk(odmkv::g_mu);
    odmkv::g_on = on != 0;
}

// Sum of elapsed milliseconds and number of launches recorded for `kernel` since the last read;
// waits for the recorded events.  Returns 0, or a CUDA error code.
int odmkv_timing_read(const char *kernel, double *total_ms, long long *launches) {
    std::lock_guard<std::mutex> lk(odmkv::g_mu);
    double tot = 0.0;
    long long n = 0;
    auto it = odmkv::g_events.find(kernel ? kernel : "");
    if (it != odmkv::g_events.end()) {
        for (auto &p : it->second) {
            cudaError_t e = cudaEventSynchronize(p.b);
            if (e != cudaSuccess) return (int)e;
            float ms = 0.f;
            e = cudaEventElapsedTime(&ms, p.a, p.b);
            if (e != cudaSuccess) return (int)e;
            tot += ms;
            ++n;
            cudaEventDestroy(p.a);
            cudaEventDestroy(p.b);
        }
        odmkv::g_events.erase(it);
    }
    if (total_ms) *total_ms = tot;
    if (launches) *launches = n;
    return 0;
}

}  // extern "C"
