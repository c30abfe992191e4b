// Library-wide pieces of the C-ABI: version, last-error string, device peak probe.
#include <stdarg.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace splatad {

static thread_local char g_last_error[512] = "";

void set_last_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

// ---- optional per-kernel timing ---------------------------------------------------------
struct ProfRec { const char *name; cudaEvent_t a, b; };
static std::vector<ProfRec> g_prof;
static bool g_prof_on = false;

bool prof_enabled() { return g_prof_on; }

void prof_begin(const char *name, cudaStream_t st) {
    ProfRec r;
    r.name = name;
    cudaEventCreate(&r.a);
    cudaEventCreate(&r.b);
    cudaEventRecord(r.a, st);
    g_prof.push_back(r);
}

void prof_end(cudaStream_t st) { cudaEventRecord(g_prof.back().b, st); }

// FP32 FMA throughput probe: every thread runs `iters` rounds of 8 independent FMA chains.
__global__ void __launch_bounds__(256) fma_probe_kernel(float *out, int iters, float a, float b) {
    float x0 = threadIdx.x * 1e-3f, x1 = x0 + 1.f, x2 = x0 + 2.f, x3 = x0 + 3.f;
    float x4 = x0 + 4.f, x5 = x0 + 5.f, x6 = x0 + 6.f, x7 = x0 + 7.f;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            x0 = fmaf(x0, a, b); x1 = fmaf(x1, a, b); x2 = fmaf(x2, a, b); x3 = fmaf(x3, a, b);
            x4 = fmaf(x4, a, b); x5 = fmaf(x5, a, b); x6 = fmaf(x6, a, b); x7 = fmaf(x7, a, b);
        }
    }
    out[blockIdx.x * blockDim.x + threadIdx.x] = x0 + x1 + x2 + x3 + x4 + x5 + x6 + x7;
}

} // namespace splatad

using namespace splatad;

extern "C" const char *splatad_last_error(void) { return g_last_error; }

extern "C" int splatad_version(void) { return SPLATAD_B200_VERSION; }

// Launches the FMA probe: grid blocks of 256 threads, iters*128 FMAs per thread.
// flops issued = grid * 256 * iters * 128 * 2. `out` needs grid*256 floats.
extern "C" int splatad_fma_probe(float *out, int32_t grid, int32_t iters, void *stream) {
    SPL_REQUIRE(out && grid > 0 && iters > 0, SPLATAD_ERR_BAD_ARG, "fma_probe: bad argument");
    fma_probe_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(out, iters, 0.999999f, 1e-7f);
    return check_launch("fma_probe");
}

// Turns per-kernel CUDA-event timing on or off (off by default). While on, every kernel launch
// of the library is bracketed by an event pair on its stream; this creates CUDA events, so it is
// a measurement mode, not for production frames.
extern "C" int splatad_profile_enable(int32_t enable) {
    g_prof_on = enable != 0;
    return SPLATAD_OK;
}

// Waits for the recorded events, writes one line per kernel name, "name launches total_ms\n",
// into buf (NUL terminated, truncated to cap) and clears the records.
extern "C" int splatad_profile_report(char *buf, size_t cap) {
    SPL_REQUIRE(buf && cap > 0, SPLATAD_ERR_BAD_ARG, "profile_report: bad buffer");
    std::map<std::string, std::pair<int, double>> agg;
    std::vector<std::string> order;
    for (auto &r : g_prof) {
        cudaEventSynchronize(r.b);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, r.a, r.b);
        if (!agg.count(r.name)) order.push_back(r.name);
        auto &e = agg[r.name];
        e.first += 1;
        e.second += ms;
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    g_prof.clear();
    std::string out;
    char line[256];
    for (auto &nme : order) {
        snprintf(line, sizeof(line), "%s %d %.6f\n", nme.c_str(), agg[nme].first, agg[nme].second);
        out += line;
    }
    strncpy(buf, out.c_str(), cap - 1);
    buf[cap - 1] = 0;
    return SPLATAD_OK;
}
