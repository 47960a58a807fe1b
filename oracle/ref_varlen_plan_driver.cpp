// TEST INFRASTRUCTURE ONLY. Drives the reference's own header-only planner
// (ktt_flash/varlen_plan.hpp, included from the mounted reference tree, never copied) so
// that oracle/varlen_plan.py can be checked against it and golden vectors generated.
//
// usage: varlen_plan <causal 0|1> <key_side 0|1> <n> cu_q[0..n] cu_k[0..n]
// prints: "intervals" then lo/hi per packed query, "rows" then kfirst klast a b u0 per
// tile row, or "error <message>" when the reference rejects the offsets.
#include <cstdio>
#include <cstdlib>
#include <exception>
#include <vector>

#include "varlen_plan.hpp"

int main(int argc, char** argv) {
    if (argc < 4) return 2;
    const bool causal = std::atoi(argv[1]) != 0;
    const bool key_side = std::atoi(argv[2]) != 0;
    const int n = std::atoi(argv[3]);
    if (argc != 4 + 2 * (n + 1)) return 2;
    std::vector<int64_t> cu_q, cu_k;
    for (int i = 0; i <= n; ++i) cu_q.push_back(std::atoll(argv[4 + i]));
    for (int i = 0; i <= n; ++i) cu_k.push_back(std::atoll(argv[5 + n + i]));
    namespace vl = ktt::bridge::ktt_flash::varlen;
    try {
        std::vector<int64_t> lo, hi;
        vl::intervals(cu_q, cu_k, causal, lo, hi);
        std::printf("intervals %zu\n", lo.size());
        for (size_t i = 0; i < lo.size(); ++i) std::printf("%lld %lld\n", (long long)lo[i], (long long)hi[i]);
        const vl::Plan plan = key_side ? vl::key_plan(cu_q, cu_k, causal, 0.0f) : vl::plan(cu_q, cu_k, causal, 0.0f);
        std::printf("rows %zu %u\n", plan.rows.size(), plan.tiles);
        for (const auto& r : plan.rows) std::printf("%u %u %u %u %u\n", r.kfirst, r.klast, r.a, r.b, r.u0);
    } catch (const std::exception& e) {
        std::printf("error %s\n", e.what());
    }
    return 0;
}
