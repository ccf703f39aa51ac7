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
    try { native_expert_layout(9, 9, 2048, 512); } catch (const std::invalid_argument&) { threw = true; }
    if (!threw) { std::puts("unknown type must throw"); ++failures; }
    route_tail_skip(nullptr, nullptr, ResidentTabs{}, 500, 4, 1, 8, nullptr, nullptr);   // out of range: a silent no-op, as in the reference
    {
        namespace c = basalt::kernels::cpu;
        std::string err;
        const std::string b = std::to_string(L.bytes);
        const std::string text = "# experts v6: layer gu_type d_type offset blob_bytes (n_expert 4, total " + std::to_string(8 * L.bytes) +
                                 ")\n0 40 40 0 " + b + "\n1 40 40 " + std::to_string(4 * L.bytes) + " " + b + "\n";
        if (!c::expert_layout_load_text(text, 2, 512, err, 2048, 512) || c::expert_layout().n_expert != 4 ||
            c::expert_layout().blob_offset(1, 2) != 6 * L.bytes || c::expert_layout().fmt[1].down_off != L.down_off ||
            c::expert_layout().total != 8 * L.bytes || c::expert_layout().version != 6) { std::puts(("layout text: " + err).c_str()); ++failures; }
        if (c::expert_layout_load_text("# experts v8: x\n", 2, 512, err, 2048, 512) || err.find("v8") == std::string::npos) { std::puts("v8 must be refused"); ++failures; }
        if (c::expert_layout().version != 6) { std::puts("a refused text must leave the table alone"); ++failures; }
    }
    threw = false;
    try { basalt::kernels::wgemm::norm_pack((const float*) nullptr, nullptr, 1e-6f, 2048, 4, nullptr, nullptr, nullptr); } catch (const std::invalid_argument&) { threw = true; }
    if (!threw) { std::puts("norm_pack without a stream must throw"); ++failures; }
    {
        // the prompt path's host-side helpers (include/basalt/prefill/moe_fp4.hpp): sizes, runs and pieces
        namespace fp4 = basalt::prefill::fp4;
        if (fp4::token_bytes(10, 2560) != 10u * (1280 + 160) || fp4::scale_count(100, 16) != (2 + 16) * 64u || fp4::max_blocks(300, 4) != 3 + 4) { std::puts("fp4 sizes"); ++failures; }
        const int32_t bounds[6] = {0, 100, 100, 500, 520, 700};      // five experts: 100, 0, 400, 20, 180 rows
        fp4::Group g;
        g.n = 5;
        g.bounds_host = bounds;
        if (fp4::run_length(g, 0, 256) != 2 || fp4::run_length(g, 2, 256) != 1 || fp4::run_length(g, 3, 256) != 2 || fp4::run_length(g, 0, 1000) != 5) { std::puts("run_length"); ++failures; }
        fp4::Pieces pc;
        fp4::cut_pieces(bounds, 5, 200, pc);       // whole = 192: expert 2 is cut into 192 + 192 + 16
        const std::vector<int32_t> want_e = {0, 2, 2, 2, 3, 4}, want_b = {0, 100, 292, 484, 500, 520, 700}, want_g = {0, 1, 2, 3, 5, 6};
        if (pc.expert != want_e || pc.bounds != want_b || pc.group != want_g) { std::puts("cut_pieces"); ++failures; }
        threw = false;
        try { fp4::run_group(g, 256, nullptr); } catch (const std::invalid_argument&) { threw = true; }
        if (!threw) { std::puts("run_group without noted rows must throw"); ++failures; }
        threw = false;
        try { fp4::run(fp4::Product{}, nullptr); } catch (const std::logic_error&) { threw = true; }
        if (!threw) { std::puts("run(Product) must say it is not provided"); ++failures; }
    }
    std::printf("shim %s\n", failures ? "FAILED" : "ok");
    return failures;
}
