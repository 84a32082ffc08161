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
#include "tc_common.cuh"

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

struct EdgeParams {
    int n_layers;
    int capacity;
    float r_cut;
    float silu_norm;
    double cell[9];
    const float* rad_w[FMB_MAX_LAYERS][3];
    const float* mlp_img[FMB_MAX_LAYERS];     // the same three layers as tensor-core operand images (or null)
    uint32_t* error_word;
};

// Edge vector, length and the Bessel x envelope features with their d/dr (zero at and beyond the cutoff).
struct EdgeGeometry {
    float ux, uy, uz, len;
};

__device__ __forceinline__ EdgeGeometry edge_geometry(const EdgeParams& p, const double* __restrict__ x,
                                                      const int32_t* __restrict__ edge_index,
                                                      const float* __restrict__ unit_shifts, long long e) {
    const int s = edge_index[e], r = edge_index[p.capacity + e];
    const double u0 = unit_shifts[3 * e], u1 = unit_shifts[3 * e + 1], u2 = unit_shifts[3 * e + 2];
    double v[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const double shift = u0 * p.cell[a] + u1 * p.cell[3 + a] + u2 * p.cell[6 + a];
        v[a] = (x[3 * r + a] - x[3 * s + a]) + shift;
    }
    const float vx = (float)v[0], vy = (float)v[1], vz = (float)v[2];
    EdgeGeometry g;
    g.len = sqrtf(vx * vx + vy * vy + vz * vz);
    const float inv = 1.0f / fmaxf(g.len, 1e-12f);
    g.ux = vx * inv; g.uy = vy * inv; g.uz = vz * inv;
    return g;
}

__device__ __forceinline__ void bessel_features(float len, float rc, float (&ef)[8], float (&def)[8]) {
#pragma unroll
    for (int k = 0; k < 8; ++k) { ef[k] = 0.0f; def[k] = 0.0f; }
    if (len < rc) {
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

// four of the eight (first = 0 or 4), for kernels that spread an edge's basis functions over two threads
__device__ __forceinline__ void bessel_features(float len, float rc, int first, float (&ef)[4], float (&def)[4]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) { ef[k] = 0.0f; def[k] = 0.0f; }
    if (len < rc) {
        const float xr = len / rc;
        const float x2 = xr * xr, x4 = x2 * x2, x5 = x4 * xr;
        const float env = 1.0f - 21.0f * x5 + 35.0f * x5 * xr - 15.0f * x5 * x2;
        const float denv = (-105.0f * x4 + 210.0f * x5 - 105.0f * x5 * xr) / rc;
        const float pref = sqrtf(2.0f / rc);
        const float inv_r = 1.0f / len;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float wk = (float)(first + k + 1) * 3.14159265358979323846f / rc;
            float sn, cs;
            sincosf(wk * len, &sn, &cs);
            const float bes = pref * sn * inv_r;
            const float dbes = pref * (wk * cs * inv_r - sn * inv_r * inv_r);
            ef[k] = bes * env;
            def[k] = dbes * env + bes * denv;
        }
    }
}

__device__ __forceinline__ void store_harmonics(const EdgeGeometry& g, float* __restrict__ edge_vec,
                                                float* __restrict__ edge_sh, long long e) {
    reinterpret_cast<float4*>(edge_vec)[e] = make_float4(g.ux, g.uy, g.uz, g.len);
    float Y[16];
    sh16(g.ux, g.uy, g.uz, Y);
    float4* ysh = reinterpret_cast<float4*>(edge_sh + 16 * e);
    ysh[0] = make_float4(Y[0], Y[1], Y[2], Y[3]);
    ysh[1] = make_float4(Y[4], Y[5], Y[6], Y[7]);
    ysh[2] = make_float4(Y[8], Y[9], Y[10], Y[11]);
    ysh[3] = make_float4(Y[12], Y[13], Y[14], Y[15]);
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
        const EdgeGeometry g = edge_geometry(p, x, edge_index, unit_shifts, e);
        store_harmonics(g, edge_vec, edge_sh, e);
        bessel_features(g.len, p.r_cut, ef, def);
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

// ------------------------------------------------------------------------------------------------ tcgen05 MLP
// The three hidden layers on the tcgen05 path (the warp-level mma.sync instructions above run at a fraction of the
// tensor pipe's rate on this architecture: 124 us for 62 k edges, with the pipe 46 % busy).
//
// One CTA = 64 edges = one M = 128 accumulator tile: the values and the d/dr tangents of an edge are two rows of the
// same tile, so one chain of MMAs (N = 64, 3xTF32) serves both. Rows are ordered so that a quarter of the accumulator
// lanes (the 32 lanes one warp can read) holds 16 edges' values (lanes 0-15) and the same edges' tangents (lanes
// 16-31): the SiLU needs both, and the two lanes of an edge trade halves of what they read with shuffles, so that every
// lane does the same amount of exp / reciprocal work and nothing crosses warps. Eight warps: warps w and w + 4 read
// the same lane quarter and take 32 of the 64 columns each, i.e. a thread finishes 16 columns of one edge, values
// and tangents. The activated rows go back to shared memory as the next layer's operand (tf32 value and remainder
// parts, K-major with the 128-byte swizzle); the third layer's rows leave through the same memory as whole 256-byte
// rows. The weights arrive as ready-made operand images by bulk copy while the SiLU of the layer before runs. One
// thread issues the MMAs. Every wait is bounded.
constexpr int kTcEdges = 64;
constexpr int kTcThreads = 256;
constexpr int kTcATile = 128 * 64 * 4;                 // 32 KB: [128 rows][64 k], one of the two tf32 parts
constexpr int kTcWTile = 64 * 64 * 4;                  // 16 KB: [64 outputs][64 k]
constexpr int kTcBytes = 2 * kTcATile + 2 * kTcWTile + 64 + 1024;
constexpr unsigned kTcSpin = 1u << 20;
// float offsets of the layers' images inside mlp_img: [8 -> 64] value / remainder (one K half each), then the two
// [64 -> 64] layers, value (two K halves) then remainder
constexpr int kImgFirstLo = 2048, kImgHidden = 4096, kImgHiddenStride = 8192;

__device__ __forceinline__ void store_split(uint8_t* hi_tile, uint8_t* lo_tile, int row, int k, const float4& v) {
    const float4 hi = make_float4(tc::tf32_rna(v.x), tc::tf32_rna(v.y), tc::tf32_rna(v.z), tc::tf32_rna(v.w));
    const float4 lo = make_float4(tc::tf32_rna(v.x - hi.x), tc::tf32_rna(v.y - hi.y), tc::tf32_rna(v.z - hi.z),
                                  tc::tf32_rna(v.w - hi.w));
    const uint32_t off = tc::tile_offset<128>(row, k);
    *reinterpret_cast<float4*>(hi_tile + off) = hi;
    *reinterpret_cast<float4*>(lo_tile + off) = lo;
}

__global__ void __launch_bounds__(kTcThreads, 2)
k_edge_features_tc(const __grid_constant__ EdgeParams p, const double* __restrict__ x,
                   const int32_t* __restrict__ edge_index, const float* __restrict__ unit_shifts,
                   const long long* __restrict__ count_ptr, float* __restrict__ edge_vec, float* __restrict__ edge_sh,
                   float* __restrict__ edge_hidden) {
    using namespace tc;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* a_hi = smem;
    uint8_t* a_lo = smem + kTcATile;
    uint8_t* w_buf = smem + 2 * kTcATile;                // value image, then remainder image 16 KB further
    uint64_t* bars = reinterpret_cast<uint64_t*>(w_buf + 2 * kTcWTile);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar_w = smem_u32(bars), bar_mma = bar_w + 8;

    const long long count = *count_ptr;
    const long long e0 = (long long)blockIdx.x * kTcEdges;
    if (e0 >= count) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quarter = warp & 3;                        // the 32 accumulator lanes this warp reads
    const int half = warp >> 2;                          // and the 32 columns of them it takes
    const int upper = lane >> 4;                         // 0: this lane's accumulator row holds values, 1: tangents
    const int row_v = quarter * 32 + (lane & 15), row_t = row_v + 16;
    const long long e = e0 + quarter * 16 + (lane & 15);
    const bool live = e < count;

    auto request_weights = [&](int layer, int hidden) {
        const float* img = p.mlp_img[layer];
        const uint32_t dst = smem_u32(w_buf);
        if (hidden == 0) {
            mbar_expect_tx(bar_w, 2 * 8192);
            bulk_load(dst, img, 8192, bar_w);
            bulk_load(dst + kTcWTile, img + kImgFirstLo, 8192, bar_w);
        } else {
            mbar_expect_tx(bar_w, 2 * kTcWTile);
            bulk_load(dst, img + kImgHidden + (hidden - 1) * kImgHiddenStride, 2 * kTcWTile, bar_w);
        }
    };
    if (tid == 0) {
        mbar_init(bar_w, 1);
        mbar_init(bar_mma, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        request_weights(0, 0);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), 64);
    }

    // geometry: the four threads of an edge share its vector; the two lower ones evaluate four radial basis
    // functions each, one of the upper ones the harmonics
    float ef[4] = {0.f, 0.f, 0.f, 0.f}, def[4] = {0.f, 0.f, 0.f, 0.f};
    if (live && !(upper && half)) {
        const EdgeGeometry g = edge_geometry(p, x, edge_index, unit_shifts, e);
        if (upper) store_harmonics(g, edge_vec, edge_sh, e);
        else bessel_features(g.len, p.r_cut, 4 * half, ef, def);
    }

    uint32_t w_parity = 0, mma_parity = 0;
    uint32_t tmem_base = 0;
    for (int layer = 0; layer < p.n_layers; ++layer) {
        for (int hidden = 0; hidden < 3; ++hidden) {
            if (hidden == 0 && !upper) {
                // the 8 radial features and their d/dr: K = 8, the first 32 bytes of the two rows of this edge
                store_split(a_hi, a_lo, row_v, 4 * half, make_float4(ef[0], ef[1], ef[2], ef[3]));
                store_split(a_hi, a_lo, row_t, 4 * half, make_float4(def[0], def[1], def[2], def[3]));
            }
            fence_async_smem();
            fence_before_sync();
            __syncthreads();
            fence_after_sync();
            if (layer == 0 && hidden == 0) tmem_base = *tmem_slot;
            if (tid == 0) {
                mbar_wait(bar_w, w_parity, abort_flag, kTcSpin);
                const uint32_t idesc = make_idesc<64>();
                const uint64_t da_hi = make_desc(smem_u32(a_hi)), da_lo = make_desc(smem_u32(a_lo));
                const uint64_t dw_hi = make_desc(smem_u32(w_buf)), dw_lo = make_desc(smem_u32(w_buf) + kTcWTile);
                if (hidden == 0) {
                    mma_tf32(tmem_base, da_lo, dw_hi, idesc, 0);
                    mma_tf32(tmem_base, da_hi, dw_lo, idesc, 1);
                    mma_tf32(tmem_base, da_hi, dw_hi, idesc, 1);
                } else {
#pragma unroll
                    for (int k8 = 0; k8 < 8; ++k8)
                        mma_tf32(tmem_base, da_lo + k_step<128>(k8), dw_hi + k_step<64>(k8), idesc, k8 > 0 ? 1 : 0);
#pragma unroll
                    for (int k8 = 0; k8 < 8; ++k8) mma_tf32(tmem_base, da_hi + k_step<128>(k8), dw_lo + k_step<64>(k8), idesc, 1);
#pragma unroll
                    for (int k8 = 0; k8 < 8; ++k8) mma_tf32(tmem_base, da_hi + k_step<128>(k8), dw_hi + k_step<64>(k8), idesc, 1);
                }
                mma_commit(bar_mma);
            }
            w_parity ^= 1u;
            mbar_wait(bar_mma, mma_parity, abort_flag, kTcSpin);
            mma_parity ^= 1u;
            fence_after_sync();
            if (tid == 0) {
                // the weight buffer is free: the next layer's image travels while this layer's SiLU runs
                if (hidden < 2) request_weights(layer, hidden + 1);
                else if (layer + 1 < p.n_layers) request_weights(layer + 1, 0);
            }
            // 32 columns of this lane's accumulator row: pre-activations (lower lanes) or raw tangents (upper lanes)
            float own[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(32 * half);
            {
                float v0[16], v1[16];
                tmem_load_16x2(taddr, taddr + 16, v0, v1);
#pragma unroll
                for (int i = 0; i < 16; ++i) { own[i] = v0[i]; own[16 + i] = v1[i]; }
            }
            // the lower lane finishes the first 16 of these columns, the upper lane the other 16
            float act[16], tng[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float send = upper ? own[i] : own[16 + i];
                const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
                act[i] = upper ? recv : own[i];
                tng[i] = upper ? own[16 + i] : recv;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float a = act[i];
                // ex2.approx + rcp.approx: relative error of a few 1e-7 on the sigmoid, far inside the fp32
                // tolerance of the forces
                const float sig = __fdividef(1.0f, 1.0f + __expf(-a));
                act[i] = p.silu_norm * a * sig;
                tng[i] = p.silu_norm * sig * (1.0f + a * (1.0f - sig)) * tng[i];
            }
            const int col0 = 32 * half + 16 * upper;
            if (hidden < 2) {
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    store_split(a_hi, a_lo, row_v, col0 + 4 * i4, make_float4(act[4 * i4], act[4 * i4 + 1], act[4 * i4 + 2], act[4 * i4 + 3]));
                    store_split(a_hi, a_lo, row_t, col0 + 4 * i4, make_float4(tng[4 * i4], tng[4 * i4 + 1], tng[4 * i4 + 2], tng[4 * i4 + 3]));
                }
            } else {
                // the third hidden layer goes to global memory, [layer][0 value / 1 tangent][edge][64]: staged in
                // the (now free) operand tile as plain rows [128][64] with the 16-byte slot XORed with the row, then
                // written as whole rows -- a quarter's 16 value rows are 4 KB contiguous, and so are its tangent rows
                float4* stage = reinterpret_cast<float4*>(a_hi);
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const int slot = (col0 >> 2) + i4;
                    stage[row_v * 16 + (slot ^ (row_v & 15))] = make_float4(act[4 * i4], act[4 * i4 + 1], act[4 * i4 + 2], act[4 * i4 + 3]);
                    stage[row_t * 16 + (slot ^ (row_t & 15))] = make_float4(tng[4 * i4], tng[4 * i4 + 1], tng[4 * i4 + 2], tng[4 * i4 + 3]);
                }
                __syncthreads();
                float* hv = edge_hidden + ((long long)(2 * layer) * p.capacity) * 64;
                float* ht = edge_hidden + ((long long)(2 * layer + 1) * p.capacity) * 64;
                // 2,048 float4 in all; a warp instruction moves two rows
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int row = it * 16 + (tid >> 4), slot = tid & 15;
                    const int q = row >> 5, j = row & 31;                 // quarter and lane of the row
                    const long long edge = e0 + q * 16 + (j & 15);
                    if (edge < count) {
                        float* dst = (j < 16 ? hv : ht) + edge * 64 + 4 * slot;
                        *reinterpret_cast<float4*>(dst) = stage[row * 16 + (slot ^ (row & 15))];
                    }
                }
                if (layer + 1 < p.n_layers) __syncthreads();      // the next interaction's operands go to the same tile
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        if (lane == 0 && *abort_flag && p.error_word) atomicOr(p.error_word, FMB_STATUS_TENSOR_TIMEOUT);
        __syncwarp();
        tmem_free(tmem_base, 64);
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
    p.error_word = work->status;
    bool images = model->n_layers > 0;
    for (int t = 0; t < model->n_layers; ++t) {
        p.mlp_img[t] = model->layer[t].mlp_img;
        images = images && p.mlp_img[t] != nullptr;
    }
    if (images) {
        // operand images packed: the tcgen05 kernel, 64 edges per CTA
        FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_edge_features_tc, kTcBytes));
        k_edge_features_tc<<<ceil_div(nl->capacity, kTcEdges), kTcThreads, kTcBytes, stream>>>(
            p, positions, nl->edge_index, nl->unit_shifts, count, work->edge_vec, work->edge_sh, work->edge_hidden);
        FMB_LAUNCH_CHECK();
        return FMB_OK;
    }
    const size_t smem_mma = (size_t)kMmaSmemFloats * sizeof(float);
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_edge_features_mma, (int)smem_mma));
    k_edge_features_mma<<<ceil_div(nl->capacity, kEdgesPerBlock), kThreads, smem_mma, stream>>>(
        p, positions, nl->edge_index, nl->unit_shifts, count, work->edge_vec, work->edge_sh, work->edge_hidden);
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
