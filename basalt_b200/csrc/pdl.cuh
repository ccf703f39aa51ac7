// pdl.cuh - programmatic dependent launch for the kernels of one layer step, after the Basalt engine's own helper
// (include/basalt/kernels/pdl.hpp:20-32, used by its router at src/kernels/cuda/router.cu:59-60,223-224).
//
// Inside a PdlScope every launch made through launch_k carries cudaLaunchAttributeProgrammaticStreamSerialization: the
// kernel may be scheduled while the kernel before it on the stream is still finishing, so its launch latency and its
// prologue (barrier init, tensor-memory allocation, loads of constant weights) hide under the predecessor's tail.  Every
// kernel launched this way calls pdl_wait() before it reads anything an earlier kernel wrote and before it writes
// anything; pdl_wait() returns once the earlier kernels have completed and their writes are visible, so results are those
// of plain launches.  Outside a scope launch_k is the plain <<<>>> launch and pdl_wait() returns at once.
#pragma once
#include <cuda_runtime.h>

namespace bsx {

struct PdlState {
    bool on = false;
    int plain = 0;   // launches still to go the plain way (the first kernel of a step follows work of another kind)
    // The next launch reads nothing the kernel before it writes (its inputs were complete before that kernel started): it may run
    // beside its predecessor and wait for it only before it exits, which keeps "my completion implies my predecessors'" true for
    // the kernels after it.  Read and cleared by the launch code of the kernels that support it.
    bool late_wait = false;
};
inline PdlState& pdl_state() {
    thread_local PdlState s;
    return s;
}

class PdlScope {
public:
    explicit PdlScope(bool on, int first_plain = 1) : prev_(pdl_state()) {
        pdl_state().on = on;
        pdl_state().plain = first_plain;
    }
    ~PdlScope() { pdl_state() = prev_; }
    PdlScope(const PdlScope&) = delete;
    PdlScope& operator=(const PdlScope&) = delete;

private:
    PdlState prev_;
};

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// lets the next kernel of the stream start once every block of this grid has called it or exited (scheduling only)
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    PdlState& ps = pdl_state();
    if (ps.on) {
        if (ps.plain > 0) {
            --ps.plain;
        } else {
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = grid;
            cfg.blockDim = block;
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            (void) cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // an error stays for the caller's launch check
            return;
        }
    }
    kernel<<<grid, block, smem, stream>>>(static_cast<KArgs>(args)...);
}
#endif

}  // namespace bsx
