// SIMT fp32 GEMM (FMA pipe) with batch/row-strided rows. 128 x 128 x 8 tiles, 256 threads, 8 x 8 register tiles,
// register-prefetched double buffering. Exact fp32 (no tensor cores): the parity baseline of the tcgen05 3xTF32 kernel.

#include "gemm.cuh"

#include <cstdlib>
#include <cstring>

namespace fmb {

namespace {

constexpr int BM = 128, BN = 128, BK = 8, THREADS = 256;

struct RowMap {
    int nm;
    long long bs, rs;
    __device__ __forceinline__ long long operator()(int r) const {
        return nm == 1 ? (long long)r * bs : (long long)(r / nm) * bs + (long long)(r % nm) * rs;
    }
};

__global__ void __launch_bounds__(THREADS)
k_gemm_simt(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, int m, int n, int k,
            RowMap amap, RowMap cmap, int ldb, int accumulate, const long long* __restrict__ m_limit,
            long long m_limit_offset, const int32_t* __restrict__ batch_species, int select) {
    if (m_limit) {
        long long lim = *m_limit - m_limit_offset;
        if (lim < m) m = lim < 0 ? 0 : (int)lim;
    }
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    if (row0 >= m) return;
    __shared__ __align__(16) float As[2][BK][BM];
    __shared__ __align__(16) float Bs[2][BK][BN];
    const int tid = threadIdx.x;
    const int a_row = tid >> 1, a_k = (tid & 1) * 4;
    const int b_k = tid >> 5, b_col = (tid & 31) * 4;
    const bool a_ok = row0 + a_row < m;
    const float* a_ptr = a + (a_ok ? amap(row0 + a_row) : 0) + a_k;
    const float* b_ptr = b + (long long)b_k * ldb + col0 + b_col;
    const int ty = tid >> 4, tx = tid & 15;   // 16 x 16 threads, each 8 rows x 8 cols (rows ty*8.., cols tx*4 and 64+tx*4)
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    float4 ra = a_ok ? *reinterpret_cast<const float4*>(a_ptr) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 rb = *reinterpret_cast<const float4*>(b_ptr);
    As[0][a_k + 0][a_row] = ra.x; As[0][a_k + 1][a_row] = ra.y; As[0][a_k + 2][a_row] = ra.z; As[0][a_k + 3][a_row] = ra.w;
    *reinterpret_cast<float4*>(&Bs[0][b_k][b_col]) = rb;
    __syncthreads();
    const int tiles = k / BK;
    for (int t = 0; t < tiles; ++t) {
        const int cur = t & 1;
        if (t + 1 < tiles) {
            ra = a_ok ? *reinterpret_cast<const float4*>(a_ptr + (t + 1) * BK) : make_float4(0.f, 0.f, 0.f, 0.f);
            rb = *reinterpret_cast<const float4*>(b_ptr + (long long)(t + 1) * BK * ldb);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][kk][ty * 8]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][kk][ty * 8 + 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[cur][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[cur][kk][64 + tx * 4]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (t + 1 < tiles) {
            const int nxt = cur ^ 1;
            As[nxt][a_k + 0][a_row] = ra.x; As[nxt][a_k + 1][a_row] = ra.y;
            As[nxt][a_k + 2][a_row] = ra.z; As[nxt][a_k + 3][a_row] = ra.w;
            *reinterpret_cast<float4*>(&Bs[nxt][b_k][b_col]) = rb;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = row0 + ty * 8 + i;
        if (r >= m) continue;
        if (batch_species && batch_species[r / cmap.nm] != select) continue;
        float* crow = c + cmap(r) + col0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float4* dst = reinterpret_cast<float4*>(crow + half * 64 + tx * 4);
            float4 v = make_float4(acc[i][half * 4 + 0], acc[i][half * 4 + 1], acc[i][half * 4 + 2], acc[i][half * 4 + 3]);
            if (accumulate) {
                const float4 old = *dst;
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            *dst = v;
        }
    }
}

}  // namespace

int gemm_simt(const GemmArgs& g, cudaStream_t stream) {
    FMB_REQUIRE(g.a && g.b && g.c, "gemm: null operand");
    FMB_REQUIRE(g.n % BN == 0 && g.k % BK == 0 && g.k >= BK, "gemm: n must be a multiple of 128 and k of 8");
    if (g.m <= 0) return FMB_OK;
    RowMap amap{g.a_nm, g.a_bs, g.a_rs}, cmap{g.c_nm, g.c_bs, g.c_rs};
    dim3 grid(g.n / BN, ceil_div(g.m, BM));
    k_gemm_simt<<<grid, THREADS, 0, stream>>>(g.a, g.b, g.c, g.m, g.n, g.k, amap, cmap, g.ldb ? g.ldb : g.n,
                                              g.accumulate, g.m_limit, g.m_limit_offset, g.batch_species, g.select);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

bool tensor_cores_enabled() { return true; }

int gemm_batch(const GemmArgs* list, int count, cudaStream_t stream) {
    int done = 0;
    while (done < count) {
        const int take = count - done < 8 ? count - done : 8;
        int rc = gemm_ws_batch(list + done, take, stream);
        if (rc == FMB_ERR_UNSUPPORTED) rc = gemm_tc_batch(list + done, take, stream);
        if (rc == FMB_ERR_UNSUPPORTED) {      // a shape neither tensor-core kernel takes
            for (int q = 0; q < take; ++q) {
                rc = gemm_simt(list[done + q], stream);
                if (rc) return rc;
            }
        } else if (rc) {
            return rc;
        }
        done += take;
    }
    return FMB_OK;
}

int gemm(const GemmArgs& g, cudaStream_t stream) {
    const int rc = gemm_tc(g, stream);
    if (rc != FMB_ERR_UNSUPPORTED) return rc;
    return gemm_simt(g, stream);
}

}  // namespace fmb
