// Compiles the reference-signature shim against the C ABI and exercises what needs no GPU: geometry helpers and the
// exception behaviour of the reference's operators (std::invalid_argument on unsupported geometry).
#include <cstdio>

#include "basalt_shim.hpp"

using namespace basalt::kernels;

int main() {
    int failures = 0;
    const NativeExpertLayout L = native_expert_layout(40, 40, 2048, 512);
    if (L.bytes != 1769488 || L.gu_row != 1152 || L.d_row != 288 || L.up_off != 589824 || L.down_off != 1179648) { std::puts("layout"); ++failures; }
    if (!native_expert_supported(29, 14, 7168, 2048) || native_expert_supported(40, 40, 2000, 512)) { std::puts("supported"); ++failures; }
    if (native_expert_scratch_bytes(L, 640) < (size_t) 640 * 512 * 4) { std::puts("scratch"); ++failures; }
    if (native_expert_scratch_bytes(640, 512) < native_expert_scratch_bytes(L, 640)) { std::puts("scratch bound"); ++failures; }
    RouterArgs a;
    a.n_expert = 100;   // not a multiple of 32
    bool threw = false;
    try { router(nullptr, nullptr, nullptr, 4, a, nullptr, nullptr, nullptr, nullptr); } catch (const std::invalid_argument&) { threw = true; }
    if (!threw) { std::puts("router geometry must throw"); ++failures; }
    threw = false;
    try { native_moe_combine(nullptr, nullptr, nullptr, nullptr, 2048, 10, nullptr); } catch (const std::invalid_argument&) { threw = true; }
    if (!threw) { std::puts("combine without a stream must throw"); ++failures; }
    threw = false;
    try { native_expert_layout(7, 7, 2048, 512); } catch (const std::invalid_argument&) { threw = true; }
    if (!threw) { std::puts("unknown type must throw"); ++failures; }
    route_tail_skip(nullptr, nullptr, ResidentTabs{}, 500, 4, 1, 8, nullptr, nullptr);   // out of range: a silent no-op, as in the reference
    std::printf("shim %s\n", failures ? "FAILED" : "ok");
    return failures;
}
