// TEST INFRASTRUCTURE, NOT PRODUCT.  C entry points over the reference engine's own CPU code (its vendored ggml
// quantisers/dequantisers and its CPU expert-offload pool), so the Python tests and the bench's cpu_baseline leg can call
// them through ctypes.  This file is compiled together with the reference's sources, where they lie in the reference
// checkout, into oracle/_ref/libref_cpu.so by oracle/Makefile; nothing from the reference is copied into this repository.
//
// Wrapped reference interfaces:
//   ggml_get_type_traits / ggml_quantize_chunk          include/basalt/ggml/ggml.h:60-77
//   cpu::native_fmt / native_quant_act / native_quant_h  include/basalt/kernels/cpu/native_expert.hpp:44-58
//   cpu::ExpertPool::run_split_multi_native              include/basalt/kernels/cpu/pool.hpp:96-97
//   cpu::expert_layout_load_text / expert_layout         include/basalt/kernels/cpu/expert_layout.hpp:53-65
//   cpu::cpu_name / cpu_avx512_ok / cpu_avx2_ok           include/basalt/kernels/cpu/expert_layout.hpp:37-52
//   cpu::nvfp4_256_gu_rows / nvfp4_256_down_rows          include/basalt/kernels/cpu/nvfp4_avx2.hpp:10-18 (the AVX2 kernels, called
//                                                         directly so that the AVX2 path can be timed on a CPU that also has AVX-512)
#include "basalt/ggml/ggml.h"
#include "basalt/kernels/cpu/expert_layout.hpp"
#include "basalt/kernels/cpu/native_expert.hpp"
#include "basalt/kernels/cpu/nvfp4_avx2.hpp"
#include "basalt/kernels/cpu/pool.hpp"

#include <barrier>
#include <thread>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

using namespace basalt::kernels;

extern "C" {

// Bytes of one row of n values of `type` (0 when the reference build does not carry the type).
int64_t ref_row_bytes(int type, int64_t n) {
    const ggml_type_traits* t = ggml_get_type_traits((ggml_type) type);
    if (!t || n % t->blck_size) return 0;
    return (int64_t) (n / t->blck_size * t->type_size);
}

// dst <- rows x cols floats quantised by the reference quantiser; returns bytes written (0: no quantiser).
int64_t ref_quantize(int type, const float* src, void* dst, int64_t rows, int64_t cols) {
    const ggml_type_traits* t = ggml_get_type_traits((ggml_type) type);
    if (!t || !t->from_float_ref) return 0;
    return (int64_t) ggml_quantize_chunk((ggml_type) type, src, dst, 0, rows, cols);
}

// y <- n values decoded by the reference's to_float; returns 0 on success.
int ref_dequantize(int type, const void* src, float* y, int64_t n) {
    const ggml_type_traits* t = ggml_get_type_traits((ggml_type) type);
    if (!t || !t->to_float) return -1;
    t->to_float(src, y, n);
    return 0;
}

// The reference's blob geometry: out[0..6] = gu_row, d_row, up_off, down_off, bytes, tail, act_bytes; returns 0 or -1.
int ref_native_fmt(int gu_type, int d_type, int64_t n_embd, int64_t n_ff, float swiglu_limit, int64_t* out, char* err,
                   int err_len) {
    cpu::NativeFmt f;
    std::string e;
    if (!cpu::native_fmt(gu_type, d_type, n_embd, n_ff, f, e, swiglu_limit)) {
        if (err && err_len > 0) { std::strncpy(err, e.c_str(), (size_t) err_len - 1); err[err_len - 1] = 0; }
        return -1;
    }
    out[0] = (int64_t) f.gu_row; out[1] = (int64_t) f.d_row; out[2] = (int64_t) f.up_off; out[3] = (int64_t) f.down_off;
    out[4] = (int64_t) f.bytes; out[5] = (int64_t) f.tail; out[6] = (int64_t) f.act_bytes;
    return 0;
}

struct RefPool {
    cpu::ExpertPool* pool;
};

void* ref_pool_create(int n_workers) { return new RefPool{new cpu::ExpertPool(n_workers < 1 ? 1 : n_workers)}; }
void ref_pool_destroy(void* p) {
    if (!p) return;
    RefPool* rp = (RefPool*) p;
    delete rp->pool;
    delete rp;
}
int ref_pool_workers(void* p) { return ((RefPool*) p)->pool->workers(); }

// The reference's CPU expert-offload path for one layer step: `n_pairs` (token, expert) pairs grouped by the caller into
// expert-sorted rows.  blobs[e] = expert e's blob; off[E+1] = row offsets per expert; src[row] = token of that row;
// x = [T][n_embd] fp32.  Each row's unweighted expert output lands in rows_out[row][n_embd].  Experts with more than
// MAXT rows are cut into several jobs, as the engine's callers do (include/basalt/kernels/cpu/expert.hpp:74).
// Returns 0, or -1 when the reference refuses the geometry.
int ref_pool_layer(void* p, int gu_type, int d_type, int64_t n_embd, int64_t n_ff, float swiglu_limit,
                   const uint8_t* const* blobs, int n_expert, const int32_t* off, const int32_t* src, const float* x,
                   int T, float* rows_out) {
    cpu::NativeFmt f;
    std::string e;
    if (!cpu::native_fmt(gu_type, d_type, n_embd, n_ff, f, e, swiglu_limit)) return -1;
    // quantise every token's activation once (the caller's native_quant_act)
    std::vector<uint8_t> act((size_t) T * f.act_bytes);
    for (int t = 0; t < T; ++t) cpu::native_quant_act(f, x + (size_t) t * n_embd, act.data() + (size_t) t * f.act_bytes);
    std::vector<cpu::ExpertJobMulti> jobs;
    for (int ex = 0; ex < n_expert; ++ex) {
        for (int r0 = off[ex]; r0 < off[ex + 1]; r0 += cpu::MAXT) {
            cpu::ExpertJobMulti j;
            j.blob = blobs[ex];
            j.nt = off[ex + 1] - r0 < cpu::MAXT ? off[ex + 1] - r0 : cpu::MAXT;
            for (int i = 0; i < j.nt; ++i) {
                j.nact[i] = act.data() + (size_t) src[r0 + i] * f.act_bytes;
                j.out[i] = rows_out + (size_t) (r0 + i) * n_embd;
            }
            jobs.push_back(j);
        }
    }
    cpu::ExpertPool* pool = ((RefPool*) p)->pool;
    if (!jobs.empty()) pool->run_split_multi_native(f, jobs.data(), (int) jobs.size());   // batches internally
    return 0;
}

// The reference's parse of an `experts.layout` text.  Returns 1 and fills head[0..4] = version, n_expert, max_blob, total,
// n_layers and per layer rows[6 l ..] = gu_type, d_type, up_type, offset, blob_bytes, up_off; or 0 with the reason in err.
int ref_layout_load_text(const char* text, int64_t len, int64_t n_layers, int64_t n_expert, int64_t n_embd, int64_t n_ff,
                         float swiglu_limit, int64_t* head, int64_t* rows, char* err, int err_len) {
    std::string e;
    if (!cpu::expert_layout_load_text(std::string(text, (size_t) len), n_layers, n_expert, e, n_embd, n_ff, swiglu_limit)) {
        if (err && err_len > 0) { std::strncpy(err, e.c_str(), (size_t) err_len - 1); err[err_len - 1] = 0; }
        return 0;
    }
    const cpu::ExpertLayout& L = cpu::expert_layout();
    head[0] = L.version; head[1] = L.n_expert; head[2] = (int64_t) L.max_blob; head[3] = (int64_t) L.total; head[4] = L.n_layers;
    for (int64_t l = 0; l < L.n_layers; ++l) {
        const cpu::NativeFmt& f = L.fmt[(size_t) l];
        int64_t* r = rows + 6 * l;
        r[0] = f.gu_type; r[1] = f.d_type; r[2] = f.up_type; r[3] = (int64_t) L.offset[(size_t) l]; r[4] = (int64_t) L.bytes[(size_t) l];
        r[5] = (int64_t) f.up_off;
    }
    return 1;
}

// The host CPU as the reference names it, and the widest instruction set its kernels pick here: 3 = AVX-512, 2 = AVX2, 0 = neither.
int ref_cpu_info(char* name, int name_len) {
    const std::string n = cpu::cpu_name();
    if (name && name_len > 0) { std::strncpy(name, n.c_str(), (size_t) name_len - 1); name[name_len - 1] = 0; }
    return cpu::cpu_avx512_ok() ? 3 : cpu::cpu_avx2_ok() ? 2 : 0;
}

// The same layer step as ref_pool_layer for all-NVFP4 blobs with the reference's AVX2 kernels forced (nvfp4_256_*), whatever
// else the CPU has: `n_threads` threads, each taking the same slice of rows of every job (the pool's row split), gate/up
// rows first, then - after every thread has finished them - the down rows.  Returns 0, -1 on a geometry the kernels refuse.
int ref_avx2_layer(int n_threads, int64_t n_embd, int64_t n_ff, const uint8_t* const* blobs, int n_expert, const int32_t* off,
                   const int32_t* src, const float* x, int T, float* rows_out) {
    cpu::NativeFmt f;
    std::string e;
    if (!cpu::native_fmt(40, 40, n_embd, n_ff, f, e, 0.f)) return -1;
    if (!cpu::cpu_avx2_ok() || !cpu::nvfp4_256_fits((int) n_embd, (int) n_ff)) return -1;
    std::vector<uint8_t> act((size_t) T * f.act_bytes);
    for (int t = 0; t < T; ++t) cpu::native_quant_act(f, x + (size_t) t * n_embd, act.data() + (size_t) t * f.act_bytes);
    struct Job { const uint8_t* blob; int r0, nt; };
    std::vector<Job> jobs;
    for (int ex = 0; ex < n_expert; ++ex)
        for (int r0 = off[ex]; r0 < off[ex + 1]; r0 += cpu::MAXT) jobs.push_back(Job{blobs[ex], r0, off[ex + 1] - r0 < cpu::MAXT ? off[ex + 1] - r0 : cpu::MAXT});
    const int n_rows = off[n_expert];
    std::vector<float> h((size_t) n_rows * n_ff);
    std::vector<uint8_t> hq((size_t) n_rows * f.h_bytes);
    if (n_threads < 1) n_threads = 1;
    std::barrier sync(n_threads);
    auto work = [&](int tid) {
        const int g0 = (int) (n_ff * tid / n_threads), g1 = (int) (n_ff * (tid + 1) / n_threads);
        for (const Job& j : jobs) {
            const void* a[cpu::MAXT];
            float* ff[cpu::MAXT];
            for (int i = 0; i < j.nt; ++i) {
                a[i] = act.data() + (size_t) src[j.r0 + i] * f.act_bytes;
                ff[i] = h.data() + (size_t) (j.r0 + i) * n_ff;
            }
            float sg, su;
            std::memcpy(&sg, j.blob + f.bytes - 16, 4);
            std::memcpy(&su, j.blob + f.bytes - 12, 4);
            if (g1 > g0) cpu::nvfp4_256_gu_rows(j.blob, f.gu_row, f.up_off, (int) n_embd, sg, su, 0.f, a, j.nt, ff, g0, g1);
        }
        sync.arrive_and_wait();
        for (int r = tid; r < n_rows; r += n_threads) cpu::native_quant_h(f, h.data() + (size_t) r * n_ff, hq.data() + (size_t) r * f.h_bytes);
        sync.arrive_and_wait();
        const int d0 = (int) (n_embd * tid / n_threads), d1 = (int) (n_embd * (tid + 1) / n_threads);
        for (const Job& j : jobs) {
            const void* a[cpu::MAXT];
            float* out[cpu::MAXT];
            for (int i = 0; i < j.nt; ++i) {
                a[i] = hq.data() + (size_t) (j.r0 + i) * f.h_bytes;
                out[i] = rows_out + (size_t) (j.r0 + i) * n_embd;
            }
            float sd;
            std::memcpy(&sd, j.blob + f.bytes - 8, 4);
            if (d1 > d0) cpu::nvfp4_256_down_rows(j.blob + f.down_off, f.d_row, (int) n_ff, sd, a, j.nt, out, d0, d1);
        }
    };
    std::vector<std::thread> pool;
    for (int t = 1; t < n_threads; ++t) pool.emplace_back(work, t);
    work(0);
    for (std::thread& t : pool) t.join();
    return 0;
}

}  // extern "C"
