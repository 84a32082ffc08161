// fp32 GEMM with batch/row-strided operands, the building block of the per-irrep linears, the species-dependent
// skip, the readout-side products and the last layer of the radial MLP.
#pragma once

#include "fmb_common.cuh"

namespace fmb {

// C[r, :] (+)= A[r, :] * B for r in [0, m). Row r of A starts at a + (r / a_nm) * a_bs + (r % a_nm) * a_rs, and the
// same for C; B is [k][n] row-major with leading dimension ldb.
struct GemmArgs {
    const float* a = nullptr;
    const float* b = nullptr;
    // optional tensor-core operands: B transposed ([n][k], K contiguous) and split into tf32 hi / lo parts
    const float* bt_hi = nullptr;
    const float* bt_lo = nullptr;
    // optional: the same parts packed per (128 columns, 32 K) piece in the shared-memory operand layout (gemm_ws.cu)
    const float* b_img = nullptr;
    uint32_t* error_word = nullptr;   // device status word for bounded-wait failures
    float* c = nullptr;
    int m = 0, n = 0, k = 0;
    int a_nm = 1;
    long long a_bs = 0, a_rs = 0;
    int c_nm = 1;
    long long c_bs = 0, c_rs = 0;
    int ldb = 0;
    int accumulate = 0;
    // optional: rows at or beyond *m_limit - m_limit_offset (a device scalar, e.g. the edge count) are skipped
    const long long* m_limit = nullptr;
    long long m_limit_offset = 0;
    // optional: only batches whose species equals `select` are written (species-dependent linear)
    const int32_t* batch_species = nullptr;
    int select = -1;
};

int gemm_simt(const GemmArgs& args, cudaStream_t stream);
// tcgen05 / TMEM 3xTF32 kernel; returns FMB_ERR_UNSUPPORTED for shapes it does not take.
int gemm_tc(const GemmArgs& args, cudaStream_t stream);
// several GEMMs (at most 8) in one launch of the tensor-core kernel; FMB_ERR_UNSUPPORTED if any does not qualify
int gemm_tc_batch(const GemmArgs* list, int count, cudaStream_t stream);
// warp-specialised tensor-core kernel (weights by bulk copy from b_img); FMB_ERR_UNSUPPORTED if any does not qualify
int gemm_ws_batch(const GemmArgs* list, int count, cudaStream_t stream);
// the same through whichever kernel applies (one launch when the tensor-core kernel takes them all)
int gemm_batch(const GemmArgs* list, int count, cudaStream_t stream);
// picks gemm_tc when it applies and FMB_GEMM selects it, else gemm_simt
int gemm(const GemmArgs& args, cudaStream_t stream);
// false when FMB_GEMM=simt keeps every contraction on the FP32 pipes (A/B tests)
bool tensor_cores_enabled();

}  // namespace fmb
