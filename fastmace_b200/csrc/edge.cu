// Fused edge featurisation: edge vector (float64 difference, cast to fp32), real spherical harmonics l <= 3, Bessel
// basis x polynomial cutoff, and the three hidden layers of every interaction's radial MLP -- values and their
// derivative with respect to the edge length in the same pass (forward-mode), which is what the analytic force
// kernels need instead of an autograd tape.
//
// The 16 polynomials of sh16 below, their constants and their order are those of the reference's kernel
// (fastmace/kernels/triton/edge_sh.py:40-58); the gradient used by the adjoint kernels (edge_gradient.cuh) follows
// the same file's backward (:82-126).
//
// Reference: edge geometry inside ScaleShiftMACE.forward (fastmace/model/energy.py:62-100), spherical harmonics
// fastmace/kernels/triton/edge_sh.py:40-78, radial network call site fastmace/rewrites/generic/modules.py:454 with
// e3nn's FullyConnectedNet scaling (:148-150). The envelope multiplies the 8 Bessel inputs of a bias-free network, so
// an edge at or beyond the cutoff yields exactly zero weights (fastmace/model/capabilities.py:369-394).

#include "edge_gradient.cuh"
#include "gemm.cuh"
#include "stages.cuh"

namespace fmb {

namespace {

constexpr int kEdgesPerBlock = 128;
constexpr int kThreads = 128;

__device__ __forceinline__ void sh16(float x, float y, float z, float* Y) {
    const float S3 = 1.7320508075688772f, S5 = 2.23606797749979f, S56 = 0.9128709291752769f, S38 = 0.6123724356957945f;
    const float C1 = 1.7320508075688772f, C2 = 2.23606797749979f, C3 = 2.6457513110645907f;
    const float s20 = S3 * x * z;
    const float s21 = S3 * x * y;
    const float y2 = y * y;
    const float x2z2 = x * x + z * z;
    const float s22 = y2 - 0.5f * x2z2;
    const float s23 = S3 * y * z;
    const float s24 = S3 / 2.0f * (z * z - x * x);
    Y[0] = 1.0f;
    Y[1] = C1 * x; Y[2] = C1 * y; Y[3] = C1 * z;
    Y[4] = C2 * s20; Y[5] = C2 * s21; Y[6] = C2 * s22; Y[7] = C2 * s23; Y[8] = C2 * s24;
    Y[9] = C3 * (S56 * (s20 * z + s24 * x));
    Y[10] = C3 * (S5 * s20 * y);
    Y[11] = C3 * (S38 * (4.0f * y2 - x2z2) * x);
    Y[12] = C3 * (0.5f * y * (2.0f * y2 - 3.0f * x2z2));
    Y[13] = C3 * (S38 * z * (4.0f * y2 - x2z2));
    Y[14] = C3 * (S5 * s24 * y);
    Y[15] = C3 * (S56 * (s24 * z - s20 * x));
}

// act: [2][64][128] value rows then tangent rows, k-major (edge contiguous). w: [K][64] in shared memory.
// Each thread owns 8 edges x 8 outputs (te = tid / 8 edge group, tj = tid % 8 output group).
template <int K>
__device__ __forceinline__ void mlp_layer(float* __restrict__ act, const float* __restrict__ w, float silu_norm,
                                          float (&val)[8][8], float (&tan)[8][8]) {
    const int te = threadIdx.x >> 3, tj = threadIdx.x & 7;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) { val[i][j] = 0.0f; tan[i][j] = 0.0f; }
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
        const float4 v0 = *reinterpret_cast<const float4*>(&act[k * 128 + te * 8]);
        const float4 v1 = *reinterpret_cast<const float4*>(&act[k * 128 + te * 8 + 4]);
        const float4 t0 = *reinterpret_cast<const float4*>(&act[(64 + k) * 128 + te * 8]);
        const float4 t1 = *reinterpret_cast<const float4*>(&act[(64 + k) * 128 + te * 8 + 4]);
        const float4 w0 = *reinterpret_cast<const float4*>(&w[k * 64 + tj * 8]);
        const float4 w1 = *reinterpret_cast<const float4*>(&w[k * 64 + tj * 8 + 4]);
        const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const float tt[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                val[i][j] = fmaf(vv[i], ww[j], val[i][j]);
                tan[i][j] = fmaf(tt[i], ww[j], tan[i][j]);
            }
    }
    // normalised SiLU and its derivative
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float a = val[i][j];
            const float sig = 1.0f / (1.0f + expf(-a));
            val[i][j] = silu_norm * a * sig;
            tan[i][j] = silu_norm * sig * (1.0f + a * (1.0f - sig)) * tan[i][j];
        }
}

__device__ __forceinline__ void store_act(float* __restrict__ act, const float (&val)[8][8], const float (&tan)[8][8]) {
    const int te = threadIdx.x >> 3, tj = threadIdx.x & 7;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int k = tj * 8 + j;
        *reinterpret_cast<float4*>(&act[k * 128 + te * 8]) = make_float4(val[0][j], val[1][j], val[2][j], val[3][j]);
        *reinterpret_cast<float4*>(&act[k * 128 + te * 8 + 4]) = make_float4(val[4][j], val[5][j], val[6][j], val[7][j]);
        *reinterpret_cast<float4*>(&act[(64 + k) * 128 + te * 8]) = make_float4(tan[0][j], tan[1][j], tan[2][j], tan[3][j]);
        *reinterpret_cast<float4*>(&act[(64 + k) * 128 + te * 8 + 4]) = make_float4(tan[4][j], tan[5][j], tan[6][j], tan[7][j]);
    }
}

struct EdgeParams {
    int n_layers;
    int capacity;
    float r_cut;
    float silu_norm;
    double cell[9];
    const float* rad_w[FMB_MAX_LAYERS][3];
};

__global__ void __launch_bounds__(kThreads)
k_edge_features(EdgeParams p, const double* __restrict__ x, const int32_t* __restrict__ edge_index,
                const float* __restrict__ unit_shifts, const long long* __restrict__ count_ptr,
                float* __restrict__ edge_vec, float* __restrict__ edge_sh, float* __restrict__ edge_hidden) {
    extern __shared__ __align__(16) float smem[];
    float* act = smem;                       // [2][64][128]
    float* w_s = smem + 2 * 64 * 128;        // [64][64] (first layer uses [8][64])
    float* feat = w_s + 64 * 64;             // [2][8][128] Bessel x cutoff and its derivative
    const long long count = *count_ptr;
    const long long e0 = (long long)blockIdx.x * kEdgesPerBlock;
    if (e0 >= count) return;
    const int tid = threadIdx.x;
    const long long e = e0 + tid;
    const bool live = e < count;
    {
        float ef[8], def[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) { ef[k] = 0.0f; def[k] = 0.0f; }
        if (live) {
            const int s = edge_index[e], r = edge_index[p.capacity + e];
            const double u0 = unit_shifts[3 * e], u1 = unit_shifts[3 * e + 1], u2 = unit_shifts[3 * e + 2];
            double v[3];
#pragma unroll
            for (int a = 0; a < 3; ++a) {
                const double shift = u0 * p.cell[a] + u1 * p.cell[3 + a] + u2 * p.cell[6 + a];
                v[a] = (x[3 * r + a] - x[3 * s + a]) + shift;
            }
            const float vx = (float)v[0], vy = (float)v[1], vz = (float)v[2];
            const float len = sqrtf(vx * vx + vy * vy + vz * vz);
            const float inv = 1.0f / fmaxf(len, 1e-12f);
            const float ux = vx * inv, uy = vy * inv, uz = vz * inv;
            reinterpret_cast<float4*>(edge_vec)[e] = make_float4(ux, uy, uz, len);
            float Y[16];
            sh16(ux, uy, uz, Y);
            float4* ysh = reinterpret_cast<float4*>(edge_sh + 16 * e);
            ysh[0] = make_float4(Y[0], Y[1], Y[2], Y[3]);
            ysh[1] = make_float4(Y[4], Y[5], Y[6], Y[7]);
            ysh[2] = make_float4(Y[8], Y[9], Y[10], Y[11]);
            ysh[3] = make_float4(Y[12], Y[13], Y[14], Y[15]);
            if (len < p.r_cut) {
                const float rc = p.r_cut;
                const float xr = len / rc;
                const float x2 = xr * xr, x4 = x2 * x2, x5 = x4 * xr;
                // p = 5: 1 - 21 x^5 + 35 x^6 - 15 x^7 and its derivative
                const float env = 1.0f - 21.0f * x5 + 35.0f * x5 * xr - 15.0f * x5 * x2;
                const float denv = (-105.0f * x4 + 210.0f * x5 - 105.0f * x5 * xr) / rc;
                const float pref = sqrtf(2.0f / rc);
                const float inv_r = 1.0f / len;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float wk = (float)(k + 1) * 3.14159265358979323846f / rc;
                    float sn, cs;
                    sincosf(wk * len, &sn, &cs);
                    const float bes = pref * sn * inv_r;
                    const float dbes = pref * (wk * cs * inv_r - sn * inv_r * inv_r);
                    ef[k] = bes * env;
                    def[k] = dbes * env + bes * denv;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            feat[k * 128 + tid] = ef[k];
            feat[(8 + k) * 128 + tid] = def[k];
        }
    }
    float val[8][8], tan[8][8];
    const int te = tid >> 3, tj = tid & 7;
    for (int layer = 0; layer < p.n_layers; ++layer) {
        __syncthreads();
        // first layer: 8 -> 64
        for (int k = tid; k < 8 * 64; k += kThreads) w_s[k] = p.rad_w[layer][0][k];
        for (int k = tid; k < 8 * 128; k += kThreads) {
            act[k] = feat[k];
            act[64 * 128 + k] = feat[8 * 128 + k];
        }
        __syncthreads();
        mlp_layer<8>(act, w_s, p.silu_norm, val, tan);
        __syncthreads();
        store_act(act, val, tan);
        for (int hidden = 1; hidden < 3; ++hidden) {
            for (int k = tid; k < 64 * 64; k += kThreads) w_s[k] = p.rad_w[layer][hidden][k];
            __syncthreads();
            mlp_layer<64>(act, w_s, p.silu_norm, val, tan);
            __syncthreads();
            if (hidden < 2) store_act(act, val, tan);
        }
        // the third hidden layer goes to global memory: [layer][0 value / 1 tangent][edge][64]
        float* hv = edge_hidden + ((long long)(2 * layer) * p.capacity) * 64;
        float* ht = edge_hidden + ((long long)(2 * layer + 1) * p.capacity) * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long long ee = e0 + te * 8 + i;
            if (ee < count) {
                float4* dv = reinterpret_cast<float4*>(hv + ee * 64 + tj * 8);
                float4* dt = reinterpret_cast<float4*>(ht + ee * 64 + tj * 8);
                dv[0] = make_float4(val[i][0], val[i][1], val[i][2], val[i][3]);
                dv[1] = make_float4(val[i][4], val[i][5], val[i][6], val[i][7]);
                dt[0] = make_float4(tan[i][0], tan[i][1], tan[i][2], tan[i][3]);
                dt[1] = make_float4(tan[i][4], tan[i][5], tan[i][6], tan[i][7]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ tensor-core MLP
// The same kernel with the three hidden layers on the warp-level tensor-core path (mma.sync m16n8k8, 3xTF32: value
// and remainder parts of both operands, A_lo B_hi + A_hi B_lo + A_hi B_hi in fp32 accumulators). The layers are 64 wide:
// a tcgen05 tile (M = 128, one issuing thread, TMEM round trips between the layers for the SiLU) would spend its time
// on fixed costs, while here every warp owns 32 edges end to end -- activations private to the warp in shared memory
// (only __syncwarp between layers), accumulators and the SiLU in registers. Shared-memory strides are chosen so that
// the fragment loads are conflict-free (68 = 4 mod 32 for the A side, 72 = 8 mod 32 for the B side).
constexpr int kLda = 68, kLdb = 72;
constexpr int kActFloats = 32 * kLda;                       // one warp's activations (values or tangents)
constexpr int kMmaSmemFloats = 2 * 64 * kLdb + 4 * 2 * kActFloats;

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma_16x8x8(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One layer for this warp's 32 edges: cv / ct [m tile][n tile][4] = act (values / tangents) [32][K] x W [K][64].
template <int K>
__device__ __forceinline__ void layer_mma(const float* __restrict__ av, const float* __restrict__ at,
                                          const float* __restrict__ wh, const float* __restrict__ wl,
                                          float (&cv)[2][8][4], float (&ct)[2][8][4]) {
    const int lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) { cv[mt][nt][i] = 0.0f; ct[mt][nt][i] = 0.0f; }
#pragma unroll 1
    for (int k0 = 0; k0 < K; k0 += 8) {
        uint32_t vh[2][4], vl[2][4], th[2][4], tl[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int off = (gid + 8 * (i & 1) + 16 * mt) * kLda + k0 + tig + 4 * (i >> 1);
                const float v = av[off], t = at[off];
                vh[mt][i] = to_tf32(v); vl[mt][i] = to_tf32(v - __uint_as_float(vh[mt][i]));
                th[mt][i] = to_tf32(t); tl[mt][i] = to_tf32(t - __uint_as_float(th[mt][i]));
            }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int o0 = (k0 + tig) * kLdb + nt * 8 + gid, o1 = o0 + 4 * kLdb;
            const uint32_t bh0 = __float_as_uint(wh[o0]), bh1 = __float_as_uint(wh[o1]);
            const uint32_t bl0 = __float_as_uint(wl[o0]), bl1 = __float_as_uint(wl[o1]);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                mma_16x8x8(cv[mt][nt], vl[mt], bh0, bh1);
                mma_16x8x8(cv[mt][nt], vh[mt], bl0, bl1);
                mma_16x8x8(cv[mt][nt], vh[mt], bh0, bh1);
                mma_16x8x8(ct[mt][nt], tl[mt], bh0, bh1);
                mma_16x8x8(ct[mt][nt], th[mt], bl0, bl1);
                mma_16x8x8(ct[mt][nt], th[mt], bh0, bh1);
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2)
k_edge_features_mma(EdgeParams p, const double* __restrict__ x, const int32_t* __restrict__ edge_index,
                    const float* __restrict__ unit_shifts, const long long* __restrict__ count_ptr,
                    float* __restrict__ edge_vec, float* __restrict__ edge_sh, float* __restrict__ edge_hidden) {
    extern __shared__ __align__(16) float smem[];
    float* wh = smem;                          // [64][kLdb] tf32 values of the layer's weights
    float* wl = smem + 64 * kLdb;              // their tf32 remainders
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
    float* av = smem + 2 * 64 * kLdb + warp * 2 * kActFloats;   // this warp's activations [32][kLda]
    float* at = av + kActFloats;                                // and their d/dr
    const long long count = *count_ptr;
    const long long e0 = (long long)blockIdx.x * kEdgesPerBlock;
    if (e0 >= count) return;
    const long long e = e0 + tid;
    const bool live = e < count;
    float ef[8], def[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) { ef[k] = 0.0f; def[k] = 0.0f; }
    if (live) {
        const int s = edge_index[e], r = edge_index[p.capacity + e];
        const double u0 = unit_shifts[3 * e], u1 = unit_shifts[3 * e + 1], u2 = unit_shifts[3 * e + 2];
        double v[3];
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const double shift = u0 * p.cell[a] + u1 * p.cell[3 + a] + u2 * p.cell[6 + a];
            v[a] = (x[3 * r + a] - x[3 * s + a]) + shift;
        }
        const float vx = (float)v[0], vy = (float)v[1], vz = (float)v[2];
        const float len = sqrtf(vx * vx + vy * vy + vz * vz);
        const float inv = 1.0f / fmaxf(len, 1e-12f);
        const float ux = vx * inv, uy = vy * inv, uz = vz * inv;
        reinterpret_cast<float4*>(edge_vec)[e] = make_float4(ux, uy, uz, len);
        float Y[16];
        sh16(ux, uy, uz, Y);
        float4* ysh = reinterpret_cast<float4*>(edge_sh + 16 * e);
        ysh[0] = make_float4(Y[0], Y[1], Y[2], Y[3]);
        ysh[1] = make_float4(Y[4], Y[5], Y[6], Y[7]);
        ysh[2] = make_float4(Y[8], Y[9], Y[10], Y[11]);
        ysh[3] = make_float4(Y[12], Y[13], Y[14], Y[15]);
        if (len < p.r_cut) {
            const float rc = p.r_cut;
            const float xr = len / rc;
            const float x2 = xr * xr, x4 = x2 * x2, x5 = x4 * xr;
            const float env = 1.0f - 21.0f * x5 + 35.0f * x5 * xr - 15.0f * x5 * x2;
            const float denv = (-105.0f * x4 + 210.0f * x5 - 105.0f * x5 * xr) / rc;
            const float pref = sqrtf(2.0f / rc);
            const float inv_r = 1.0f / len;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float wk = (float)(k + 1) * 3.14159265358979323846f / rc;
                float sn, cs;
                sincosf(wk * len, &sn, &cs);
                const float bes = pref * sn * inv_r;
                const float dbes = pref * (wk * cs * inv_r - sn * inv_r * inv_r);
                ef[k] = bes * env;
                def[k] = dbes * env + bes * denv;
            }
        }
    }
    float cv[2][8][4], ct[2][8][4];
    for (int layer = 0; layer < p.n_layers; ++layer) {
        for (int hidden = 0; hidden < 3; ++hidden) {
            const int kk = hidden == 0 ? 8 : 64;
            __syncthreads();                        // every warp is done with the previous weights
            const float* __restrict__ wsrc = p.rad_w[layer][hidden];
            for (int q = tid; q < kk * 64; q += kThreads) {
                const float w = __ldg(wsrc + q);
                const float hi = __uint_as_float(to_tf32(w));
                const int dst = (q >> 6) * kLdb + (q & 63);
                wh[dst] = hi;
                wl[dst] = __uint_as_float(to_tf32(w - hi));
            }
            if (hidden == 0) {
                // this thread's edge is row `lane` of its warp's tile
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    av[lane * kLda + k] = ef[k];
                    at[lane * kLda + k] = def[k];
                }
            }
            __syncthreads();
            if (hidden == 0) layer_mma<8>(av, at, wh, wl, cv, ct);
            else layer_mma<64>(av, at, wh, wl, cv, ct);
            // normalised SiLU and its derivative on the accumulator fragments
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float a = cv[mt][nt][i];
                        // ex2.approx + rcp.approx: relative error of a few 1e-7 on the sigmoid, far inside the fp32
                        // tolerance of the forces, and a third of the instructions of expf and an IEEE division
                        const float sig = __fdividef(1.0f, 1.0f + __expf(-a));
                        cv[mt][nt][i] = p.silu_norm * a * sig;
                        ct[mt][nt][i] = p.silu_norm * sig * (1.0f + a * (1.0f - sig)) * ct[mt][nt][i];
                    }
            if (hidden < 2) {
                __syncwarp();                       // all lanes have read this layer's inputs
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int off = (gid + 8 * h + 16 * mt) * kLda + nt * 8 + 2 * tig;
                            *reinterpret_cast<float2*>(av + off) = make_float2(cv[mt][nt][2 * h], cv[mt][nt][2 * h + 1]);
                            *reinterpret_cast<float2*>(at + off) = make_float2(ct[mt][nt][2 * h], ct[mt][nt][2 * h + 1]);
                        }
                __syncwarp();
            }
        }
        // the third hidden layer goes to global memory: [layer][0 value / 1 tangent][edge][64]
        float* hv = edge_hidden + ((long long)(2 * layer) * p.capacity) * 64;
        float* ht = edge_hidden + ((long long)(2 * layer + 1) * p.capacity) * 64;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const long long ee = e0 + warp * 32 + gid + 8 * h + 16 * mt;
                if (ee < count) {
#pragma unroll
                    for (int nt = 0; nt < 8; ++nt) {
                        *reinterpret_cast<float2*>(hv + ee * 64 + nt * 8 + 2 * tig) =
                            make_float2(cv[mt][nt][2 * h], cv[mt][nt][2 * h + 1]);
                        *reinterpret_cast<float2*>(ht + ee * 64 + nt * 8 + 2 * tig) =
                            make_float2(ct[mt][nt][2 * h], ct[mt][nt][2 * h + 1]);
                    }
                }
            }
    }
}

// The harmonics and their gradient exactly as the edge and adjoint kernels evaluate them, on plain vectors.
__global__ void k_harmonics_probe(const float* __restrict__ vectors, const float* __restrict__ grad_sh,
                                  float* __restrict__ sh, float* __restrict__ grad_vectors, int n) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    const float vx = vectors[3 * e], vy = vectors[3 * e + 1], vz = vectors[3 * e + 2];
    const float len = sqrtf(vx * vx + vy * vy + vz * vz);
    const float inv = 1.0f / fmaxf(len, 1e-12f);
    const float ux = vx * inv, uy = vy * inv, uz = vz * inv;
    float Y[16];
    sh16(ux, uy, uz, Y);
    for (int k = 0; k < 16; ++k) sh[16 * e + k] = Y[k];
    if (grad_sh && grad_vectors) {
        float g[16], q[3];
        for (int k = 0; k < 16; ++k) g[k] = grad_sh[16 * e + k];
        edge_vector_gradient(g, 0.0f, ux, uy, uz, len, q);
        for (int a = 0; a < 3; ++a) grad_vectors[3 * e + a] = q[a];
    }
}

}  // namespace

int edge_features(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, const double* positions,
                  const long long* count, cudaStream_t stream) {
    if (!count) count = (const long long*)nl->count;
    EdgeParams p;
    p.n_layers = model->n_layers;
    p.capacity = nl->capacity;
    p.r_cut = model->r_cut;
    p.silu_norm = model->silu_norm;
    for (int k = 0; k < 9; ++k) p.cell[k] = nl->cell[k];
    for (int t = 0; t < model->n_layers; ++t)
        for (int k = 0; k < 3; ++k) p.rad_w[t][k] = model->layer[t].rad_w[k];
    const size_t smem = (size_t)(2 * 64 * 128 + 64 * 64 + 2 * 8 * 128) * sizeof(float);
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_edge_features, (int)smem));
    const int blocks = ceil_div(nl->capacity, kEdgesPerBlock);
    if (tensor_cores_enabled()) {
        const size_t smem_mma = (size_t)kMmaSmemFloats * sizeof(float);
        FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_edge_features_mma, (int)smem_mma));
        k_edge_features_mma<<<blocks, kThreads, smem_mma, stream>>>(p, positions, nl->edge_index, nl->unit_shifts,
                                                                    count, work->edge_vec,
                                                                    work->edge_sh, work->edge_hidden);
        FMB_LAUNCH_CHECK();
        return FMB_OK;
    }
    k_edge_features<<<blocks, kThreads, smem, stream>>>(p, positions, nl->edge_index, nl->unit_shifts,
                                                        count, work->edge_vec, work->edge_sh,
                                                        work->edge_hidden);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace fmb

extern "C" FMB_API int fmb_harmonics_probe(const float* vectors, const float* grad_sh, float* sh, float* grad_vectors, int n,
                                           fmb_stream_t stream) {
    FMB_REQUIRE(vectors && sh && n >= 0, "fmb_harmonics_probe: null argument");
    if (n == 0) return FMB_OK;
    fmb::k_harmonics_probe<<<fmb::ceil_div(n, 128), 128, 0, (cudaStream_t)stream>>>(vectors, grad_sh, sh, grad_vectors, n);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}
