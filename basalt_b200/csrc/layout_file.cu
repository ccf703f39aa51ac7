// layout_file.cu - reading a model file's `experts.layout` text: where each layer's expert blobs start inside the
// `experts` section, their ggml types and their size.  Host code only (no launch, no device memory).
//
// Behaviour follows Basalt's expert_layout_load_text (src/kernels/cpu/expert_layout.cpp:133-203; format described in
// include/basalt/kernels/cpu/expert_layout.hpp:60-67 and docs/model-file.md:230-241):
//   "# experts vN: ... (n_expert E, total B)"   header: version N (newer than 7 refused), E replaces the caller's count
//   "layer gu_type d_type offset blob_bytes"    one line per layer; from v7 a sixth column, the up rows' type
//   other '#' lines and empty lines are skipped, columns past the ones read are ignored,
//   blob_bytes must equal the size the formats make, and layer l must start where layer l - 1's n_expert blobs end.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace bsx {
namespace {

constexpr int kNewestVersion = 7;   // v6: NVFP4 blobs end in a 16-byte scale tail; v7: up_type column

struct Cursor {
    const char* p;
    const char* end;
    void blanks() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\r' || *p == '\v' || *p == '\f')) ++p;
    }
    // one decimal integer (optionally signed), as operator>> reads one: leading blanks skipped, at least one digit
    bool integer(bool allow_sign, long long& sv, unsigned long long& uv) {
        blanks();
        bool neg = false;
        if (p < end && (*p == '-' || *p == '+')) {
            neg = *p == '-';
            ++p;
        }
        if (p >= end || *p < '0' || *p > '9') return false;
        unsigned long long v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            const unsigned d = (unsigned) (*p - '0');
            if (v > (~0ull - d) / 10) return false;
            v = v * 10 + d;
            ++p;
        }
        uv = neg ? 0ull - v : v;   // an unsigned column takes a minus sign as strtoull does (the stream extraction's rule)
        if (v > (1ull << 62)) {
            if (allow_sign) return false;
            sv = 0;
        } else {
            sv = neg ? -(long long) v : (long long) v;
        }
        return true;
    }
    bool i64(long long& v) {
        unsigned long long u;
        return integer(true, v, u);
    }
    bool u64(unsigned long long& v) {
        long long s;
        return integer(false, s, v);
    }
};

void say(char* err, size_t cap, const char* fmt, ...) __attribute__((format(printf, 3, 4)));
void say(char* err, size_t cap, const char* fmt, ...) {
    if (!err || !cap) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, cap, fmt, ap);
    va_end(ap);
}

// Block geometry of the ggml formats a model file's experts come in (values per block, bytes per block: the GGUF format's
// own constants, include/basalt/ggml/ggml_common.h) and the activation format the reference's CPU dot product pairs with each
// (0: none, so the loader refuses the type; src/kernels/cpu/native_expert.cpp:78-85).  Wider than the set this library has
// kernels for: a table must parse before anyone asks which layers can run.
enum : int { kActQ8_0 = 8, kActQ8_1 = 9, kActQ8_K = 15 };
struct Geo {
    int values, bytes, act;
};
bool ggml_geo(long long type, Geo& g) {
    switch (type) {
        case 6: g = {32, 22, kActQ8_0}; return true;     // Q5_0
        case 7: g = {32, 24, kActQ8_1}; return true;     // Q5_1
        case 8: g = {32, 34, kActQ8_0}; return true;     // Q8_0
        case 10: g = {256, 84, kActQ8_K}; return true;   // Q2_K
        case 11: g = {256, 110, kActQ8_K}; return true;  // Q3_K
        case 12: g = {256, 144, kActQ8_K}; return true;  // Q4_K
        case 13: g = {256, 176, kActQ8_K}; return true;  // Q5_K
        case 14: g = {256, 210, kActQ8_K}; return true;  // Q6_K
        case 16: g = {256, 66, kActQ8_K}; return true;   // IQ2_XXS
        case 17: g = {256, 74, kActQ8_K}; return true;   // IQ2_XS
        case 18: g = {256, 98, kActQ8_K}; return true;   // IQ3_XXS
        case 19: g = {256, 50, kActQ8_K}; return true;   // IQ1_S
        case 20: g = {32, 18, kActQ8_0}; return true;    // IQ4_NL
        case 21: g = {256, 110, kActQ8_K}; return true;  // IQ3_S
        case 22: g = {256, 82, kActQ8_K}; return true;   // IQ2_S
        case 23: g = {256, 136, kActQ8_K}; return true;  // IQ4_XS
        case 29: g = {256, 56, kActQ8_K}; return true;   // IQ1_M
        case 40: g = {64, 36, kActQ8_0}; return true;    // NVFP4
        case 42: g = {64, 18, kActQ8_0}; return true;    // Q2_0 (the engine's own 2-bit format)
        default: return false;
    }
}
int act_values(int act) { return act == kActQ8_K ? 256 : 32; }

long long leading_int(const char* p, const char* end) {   // atoll on a bounded range
    Cursor c{p, end};
    long long v = 0;
    return c.i64(v) ? v : 0;
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" int32_t bsx_layout_parse(const char* text, size_t len, int64_t n_layers, int64_t n_expert, int64_t n_embd, int64_t n_ff,
                                    float swiglu_limit, bsx_layout_row* rows, bsx_layout_info* info, char* err, size_t err_cap) {
    if (err && err_cap) err[0] = 0;
    if (!rows || !info || (!text && len)) return BSX_E_POINTER;
    if (n_layers <= 0 || n_expert < 0) {
        say(err, err_cap, "expert layout: %lld layers of %lld experts", (long long) n_layers, (long long) n_expert);
        return BSX_E_GEOMETRY;
    }
    if (len == 0) {
        say(err, err_cap, "the expert layout is empty");
        return BSX_E_GEOMETRY;
    }
    memset(info, 0, sizeof *info);
    for (int64_t l = 0; l < n_layers; ++l) {
        memset(&rows[l], 0, sizeof rows[l]);
        rows[l].offset = ~0ull;
    }
    int version = 0;
    uint64_t max_blob = 0;
    static const char kHeader[] = "# experts v";
    static const char kCount[] = "(n_expert ";
    const char* p = text;
    const char* const end = text + len;
    while (p < end) {
        const char* nl = static_cast<const char*>(memchr(p, '\n', (size_t) (end - p)));
        const char* le = nl ? nl : end;
        const size_t n = (size_t) (le - p);
        if (n == 0) {
            p = le + 1;
            continue;
        }
        if (*p == '#') {
            if (n >= sizeof kHeader - 1 && memcmp(p, kHeader, sizeof kHeader - 1) == 0) {
                version = (int) leading_int(p + sizeof kHeader - 1, le);
                if (version > kNewestVersion) {
                    say(err, err_cap, "the expert layout is v%d; this library reads up to v%d", version, kNewestVersion);
                    return BSX_E_TYPE;
                }
            }
            // the header's expert count wins over the caller's (a pruned model ships fewer experts than its geometry says)
            for (const char* q = p; q + sizeof kCount - 1 <= le; ++q)
                if (memcmp(q, kCount, sizeof kCount - 1) == 0) {
                    n_expert = leading_int(q + sizeof kCount - 1, le);
                    break;
                }
            p = le + 1;
            continue;
        }
        Cursor c{p, le};
        long long l = -1, gt = -1, dt = -1, ut = -1;
        unsigned long long off = 0, blob = 0;
        const bool five = c.i64(l) && c.i64(gt) && c.i64(dt) && c.u64(off) && c.u64(blob);
        if (!five || l < 0 || l >= n_layers || (version >= 7 && !c.i64(ut))) {
            say(err, err_cap, "expert layout: a malformed line: %.*s", (int) (n > 200 ? 200 : n), p);
            return BSX_E_GEOMETRY;
        }
        // the loader's format rules (native_fmt, src/kernels/cpu/native_expert.cpp:75-128)
        if (ut < 0) ut = gt;
        Geo gg, gu, gd;
        if (!ggml_geo(gt, gg) || !ggml_geo(ut, gu) || !ggml_geo(dt, gd)) {
            say(err, err_cap, "expert layout: layer %lld: no dot product for type %lld", l, !ggml_geo(gt, gg) ? gt : !ggml_geo(ut, gu) ? ut : dt);
            return BSX_E_TYPE;
        }
        if (gu.act != gg.act || n_embd % gu.values || (ut != gt && (gt == 40 || ut == 40 || gt == 42 || ut == 42))) {
            say(err, err_cap, "expert layout: layer %lld: gate type %lld and up type %lld cannot share one layer", l, gt, ut);
            return BSX_E_TYPE;
        }
        if (n_embd <= 0 || n_ff <= 0 || n_embd % gg.values || n_ff % gd.values || n_embd % act_values(gg.act) || n_ff % act_values(gd.act)) {
            say(err, err_cap, "expert layout: layer %lld: expert geometry is not whole blocks", l);
            return BSX_E_GEOMETRY;
        }
        if ((gt == 40) != (dt == 40)) {
            say(err, err_cap, "expert layout: layer %lld: NVFP4 gate/up and down come together (the scale tail covers all three)", l);
            return BSX_E_TYPE;
        }
        const uint64_t gu_row = (uint64_t) (n_embd / gg.values) * gg.bytes, up_row = (uint64_t) (n_embd / gu.values) * gu.bytes;
        const uint64_t d_row = (uint64_t) (n_ff / gd.values) * gd.bytes;
        const uint64_t bytes = (uint64_t) n_ff * (gu_row + up_row) + (uint64_t) n_embd * d_row + (gt == 40 ? 16 : 0);
        if (bytes != blob) {
            say(err, err_cap, "expert layout: layer %lld blob is %llu B but its formats make %llu", l, blob, (unsigned long long) bytes);
            return BSX_E_GEOMETRY;
        }
        (void) swiglu_limit;   // rides into the kernels' layout (bsx_expert_layout_init), not into the table
        rows[l].gu_type = (int32_t) gt;
        rows[l].d_type = (int32_t) dt;
        rows[l].up_type = (int32_t) ut;
        rows[l].kernels = bsx_expert_supported((int32_t) gt, (int32_t) dt, (int32_t) ut, n_embd, n_ff);
        rows[l].offset = off;
        rows[l].blob_bytes = blob;
        if (blob > max_blob) max_blob = blob;
        p = le + 1;
    }
    uint64_t at = 0;
    for (int64_t l = 0; l < n_layers; ++l) {
        if (rows[l].offset != at) {
            say(err, err_cap, "expert layout: layer %lld is missing or not contiguous", (long long) l);
            return BSX_E_GEOMETRY;
        }
        at += rows[l].blob_bytes * (uint64_t) n_expert;
    }
    info->version = version;
    info->n_layers = n_layers;
    info->n_expert = n_expert;
    info->max_blob = max_blob;
    info->total = at;
    return BSX_OK;
}
