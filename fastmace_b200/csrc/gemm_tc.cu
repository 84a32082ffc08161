// tcgen05 / TMEM 3xTF32 GEMM (placeholder until the tensor-core kernel lands: reports "unsupported" so callers use
// the SIMT kernel).

#include "gemm.cuh"

namespace fmb {

int gemm_tc(const GemmArgs&, cudaStream_t) { return FMB_ERR_UNSUPPORTED; }

}  // namespace fmb
