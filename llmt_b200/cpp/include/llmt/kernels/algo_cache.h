// Record of the kernel plan used per problem (llmt algo_cache.h:18-42 caches a
// cuBLASLt algorithm per key for run-to-run determinism).  Here the plan is a
// pure function of the key, so the cache is a log: it lets a test assert that
// one problem always maps to one plan.
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <tuple>

namespace llmt::kernels {

struct AlgoKey {
    int64_t m, n, k, batch, flags, dtype, compute, scale;
    bool operator<(const AlgoKey& o) const noexcept {
        return std::tie(m, n, k, batch, flags, dtype, compute, scale) <
               std::tie(o.m, o.n, o.k, o.batch, o.flags, o.dtype, o.compute, o.scale);
    }
};

struct AlgoCache {
    std::map<AlgoKey, std::string> map;
};

}  // namespace llmt::kernels
