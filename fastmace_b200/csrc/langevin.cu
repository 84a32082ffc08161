// ASE Langevin (NVT, fixed cell) as two fused float64 stages. Replaces Langevin.first_half / second_half
// (fastmace/integrators/langevin.py:233-263) and the Triton stage fastmace/kernels/triton/fused_integrator.py:47-133.
//
// first half:  rnd_pos = c5 sqrt(kT) eta, rnd_vel = c3 sqrt(kT) xi - c4 sqrt(kT) eta, optional centre-of-mass
//              projection, v += c1 f / m - c2 v + rnd_vel, x_old = x, x += dt v + rnd_pos, v = (x - x_old - rnd_pos) / dt
// second half: v += c1 f / m - c2 v + rnd_vel
// The noise row is selected by a device-side cursor that the second half advances, so a captured step replays with
// new noise without host involvement.

#include "fmb_common.cuh"

#include <algorithm>

namespace fmb {

namespace {

constexpr int kBlocks = 128;

// stage 1: random terms and the partial sums the projection needs: per block [sum rnd_pos (3), sum m rnd_pos (3),
// sum m rnd_vel (3), sum m]
__global__ void __launch_bounds__(256)
k_noise(fmb_langevin_t lv) {
    __shared__ double sh[8][10];
    const int n = lv.n_atoms;
    const double s = *lv.sqrt_kT;
    const long long row = (long long)(*lv.noise_cursor) * 2 * n * 3;
    const double* xi = lv.noise + row;
    const double* eta = xi + (long long)n * 3;
    double acc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    const int per_block = (n + gridDim.x - 1) / gridDim.x;
    const int begin = blockIdx.x * per_block, end = min(n, begin + per_block);
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const double m = lv.masses[i];
        const double c3 = lv.c3_unit[i] * s, c4 = lv.c4_unit[i] * s, c5 = lv.c5_unit[i] * s;
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const double e = eta[3 * i + a], x = xi[3 * i + a];
            const double rp = c5 * e;
            const double rv = c3 * x - c4 * e;
            lv.rnd_pos[3 * i + a] = rp;
            lv.rnd_vel[3 * i + a] = rv;
            acc[a] += rp;
            acc[3 + a] += rp * m;
            acc[6 + a] += rv * m;
        }
        acc[9] += m;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int q = 0; q < 10; ++q) {
        const double v = warp_sum(acc[q]);
        if (lane == 0) sh[warp][q] = v;
    }
    __syncthreads();
    if (threadIdx.x < 10) {
        double v = 0.0;
        for (int w = 0; w < 8; ++w) v += sh[w][threadIdx.x];
        lv.partial[blockIdx.x * 16 + threadIdx.x] = v;
    }
}

__global__ void __launch_bounds__(256)
k_first_half(fmb_langevin_t lv, int blocks) {
    __shared__ double tot[10];
    if (threadIdx.x < 10) {
        double v = 0.0;
        for (int b = 0; b < blocks; ++b) v += lv.partial[b * 16 + threadIdx.x];
        tot[threadIdx.x] = v;
    }
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = lv.n_atoms;
    if (i >= n) return;
    const double m = lv.masses[i];
    const double factor = sqrt((double)n / ((double)n - 1.0));
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        double rp = lv.rnd_pos[3 * i + a], rv = lv.rnd_vel[3 * i + a];
        if (lv.fix_com == 2) {          // mass-weighted projection of both terms
            rp -= tot[3 + a] / tot[9];
            rv -= tot[6 + a] / tot[9];
        } else if (lv.fix_com == 1) {   // ASE's projection
            rp = (rp - tot[a] / n) * factor;
            rv = (rv - tot[6 + a] / (m * n)) * factor;
        }
        lv.rnd_pos[3 * i + a] = rp;
        lv.rnd_vel[3 * i + a] = rv;
        double v = lv.velocities[3 * i + a];
        v += lv.c1 * lv.forces[3 * i + a] / m - lv.c2 * v + rv;
        const double x_old = lv.positions[3 * i + a];
        const double x_new = x_old + (lv.dt * v + rp);
        lv.x_old[3 * i + a] = x_old;
        lv.positions[3 * i + a] = x_new;
        lv.velocities[3 * i + a] = (x_new - x_old - rp) / lv.dt;
    }
}

__global__ void __launch_bounds__(256)
k_second_half(fmb_langevin_t lv) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0) *lv.noise_cursor_rw = *lv.noise_cursor_rw + 1;
    if (i >= lv.n_atoms) return;
    const double m = lv.masses[i];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        double v = lv.velocities[3 * i + a];
        v += lv.c1 * lv.forces[3 * i + a] / m - lv.c2 * v + lv.rnd_vel[3 * i + a];
        lv.velocities[3 * i + a] = v;
    }
}

}  // namespace

}  // namespace fmb

using namespace fmb;

extern "C" FMB_API int fmb_langevin_first_half(const fmb_langevin_t* lv, fmb_stream_t stream_) {
    FMB_REQUIRE(lv && lv->n_atoms > 1, "fmb_langevin_first_half: bad argument");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int blocks = std::min(kBlocks, ceil_div(lv->n_atoms, 256));
    k_noise<<<blocks, 256, 0, stream>>>(*lv);
    FMB_LAUNCH_CHECK();
    k_first_half<<<ceil_div(lv->n_atoms, 256), 256, 0, stream>>>(*lv, blocks);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_langevin_second_half(const fmb_langevin_t* lv, fmb_stream_t stream_) {
    FMB_REQUIRE(lv, "fmb_langevin_second_half: bad argument");
    k_second_half<<<ceil_div(lv->n_atoms, 256), 256, 0, (cudaStream_t)stream_>>>(*lv);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}
