// CUDA-event pairs around launches, summed by kernel class (engine option "profile"): what an engine's step costs per
// kind of kernel, measured on the stream it runs on.  Events are pooled and reused; reading synchronises the device.
#pragma once
#include <cuda_runtime.h>

#include <utility>
#include <vector>

namespace asd {

struct EventProfiler {
    int on = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pool;
    std::vector<std::pair<int, int>> used;   // (class, pool index)
    void reset() { used.clear(); }
    int begin(int cls, cudaStream_t s) {
        if (!on) return -1;
        if (used.size() == pool.size()) {
            cudaEvent_t a, b;
            cudaEventCreate(&a);
            cudaEventCreate(&b);
            pool.emplace_back(a, b);
        }
        const int idx = (int)used.size();
        used.emplace_back(cls, idx);
        cudaEventRecord(pool[idx].first, s);
        return idx;
    }
    void end(int idx, cudaStream_t s) {
        if (idx >= 0) cudaEventRecord(pool[idx].second, s);
    }
    // ms and launches per class since the last read; returns cudaSuccess or the failing call's error
    cudaError_t read(float* ms_by_class, int* n_by_class, int nclass) {
        cudaError_t rc = cudaDeviceSynchronize();
        if (rc != cudaSuccess) return rc;
        for (int i = 0; i < nclass; ++i) {
            ms_by_class[i] = 0.f;
            if (n_by_class) n_by_class[i] = 0;
        }
        for (auto& u : used) {
            float ms = 0.f;
            rc = cudaEventElapsedTime(&ms, pool[u.second].first, pool[u.second].second);
            if (rc != cudaSuccess) return rc;
            if (u.first < nclass) {
                ms_by_class[u.first] += ms;
                if (n_by_class) n_by_class[u.first] += 1;
            }
        }
        used.clear();
        return cudaSuccess;
    }
    ~EventProfiler() {
        for (auto& p : pool) {
            cudaEventDestroy(p.first);
            cudaEventDestroy(p.second);
        }
    }
};

struct ProfRegion {
    EventProfiler& p;
    cudaStream_t s;
    int idx;
    ProfRegion(EventProfiler& p_, int cls, cudaStream_t s_) : p(p_), s(s_), idx(p_.begin(cls, s_)) {}
    ~ProfRegion() { p.end(idx, s); }
};

}  // namespace asd
