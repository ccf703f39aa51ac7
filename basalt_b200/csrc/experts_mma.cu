#include "experts.cuh"
namespace bsx {
int32_t experts_grouped_mma(const ExpertArgs&, cudaStream_t) { return BSX_E_TYPE; }
}
