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

// the ten sums of k_noise over this rank's atoms, in block order (a spatially decomposed run adds the ranks' sums)
__global__ void k_noise_sums(fmb_langevin_t lv, int blocks, double* __restrict__ sums) {
    if (threadIdx.x < 10) {
        double v = 0.0;
        for (int b = 0; b < blocks; ++b) v += lv.partial[b * 16 + threadIdx.x];
        sums[threadIdx.x] = v;
    }
}

// `global_sums` / `n_global`: the ten sums and the atom count of the whole system when this rank integrates a part
// of it (null / 0: the block partials of this launch and lv.n_atoms)
__global__ void __launch_bounds__(256)
k_first_half(fmb_langevin_t lv, int blocks, const double* __restrict__ global_sums, long long n_global) {
    __shared__ double tot[10];
    if (threadIdx.x < 10) {
        double v = 0.0;
        if (global_sums) v = global_sums[threadIdx.x];
        else for (int b = 0; b < blocks; ++b) v += lv.partial[b * 16 + threadIdx.x];
        tot[threadIdx.x] = v;
    }
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= lv.n_atoms) return;
    const double n = n_global > 0 ? (double)n_global : (double)lv.n_atoms;
    const double m = lv.masses[i];
    const double factor = sqrt(n / (n - 1.0));
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

// Counter-based normal deviates (Philox4x32-10 + Box-Muller in float64): one (seed, step, atom) triple always yields
// the same six numbers, so every rank of a domain-decomposed run draws identical noise without communication and
// without the host generator, whose draw of 6 N normals per step is the bottleneck beyond ~10^5 atoms.
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
    c[0] = n0; c[1] = (uint32_t)p1; c[2] = n2; c[3] = (uint32_t)p0;
}

__device__ __forceinline__ void philox(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

__device__ __forceinline__ void box_muller(uint32_t a, uint32_t b, uint32_t c, uint32_t d, double& z0, double& z1) {
    const double u1 = ((double)(((uint64_t)(a >> 5) << 26) | (uint64_t)(b >> 6)) + 0.5) * (1.0 / 9007199254740992.0);
    const double u2 = ((double)(((uint64_t)(c >> 5) << 26) | (uint64_t)(d >> 6)) + 0.5) * (1.0 / 9007199254740992.0);
    const double r = sqrt(-2.0 * log(u1));
    double sn, cs;
    sincospi(2.0 * u2, &sn, &cs);
    z0 = r * cs;
    z1 = r * sn;
}

// `ids`: the atom index the generator is keyed with (null = the position in the array), so that an atom draws the same
// numbers whichever rank integrates it
__global__ void __launch_bounds__(256)
k_device_noise(int n, unsigned long long seed, const int32_t* __restrict__ step, const int32_t* __restrict__ ids,
               double* __restrict__ row) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t key = ids ? (uint32_t)ids[i] : (uint32_t)i;
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    double z[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t c[4] = {key, (uint32_t)*step, (uint32_t)h, 0x6d616365u};
        philox(c, k0, k1);
        uint32_t e[4] = {key, (uint32_t)*step, (uint32_t)(h + 2), 0x6d616365u};
        philox(e, k0, k1);
        box_muller(c[0], c[1], c[2], c[3], z[4 * h + 0], z[4 * h + 1]);
        box_muller(e[0], e[1], e[2], e[3], z[4 * h + 2], z[4 * h + 3]);
    }
    // xi then eta, [2][n][3]
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        row[3 * i + a] = z[a];
        row[3 * (long long)n + 3 * i + a] = z[4 + a];
    }
}

}  // namespace

}  // namespace fmb

using namespace fmb;

extern "C" FMB_API int fmb_langevin_device_noise(double* noise_row, int n_atoms, unsigned long long seed,
                                                 const int32_t* step_counter, fmb_stream_t stream_) {
    FMB_REQUIRE(noise_row && step_counter && n_atoms > 0, "fmb_langevin_device_noise: bad argument");
    k_device_noise<<<ceil_div(n_atoms, 256), 256, 0, (cudaStream_t)stream_>>>(n_atoms, seed, step_counter, nullptr, noise_row);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_langevin_device_noise_ids(double* noise_row, int n_atoms, const int32_t* atom_ids,
                                                     unsigned long long seed, const int32_t* step_counter,
                                                     fmb_stream_t stream_) {
    FMB_REQUIRE(noise_row && step_counter && atom_ids && n_atoms > 0, "fmb_langevin_device_noise_ids: bad argument");
    k_device_noise<<<ceil_div(n_atoms, 256), 256, 0, (cudaStream_t)stream_>>>(n_atoms, seed, step_counter, atom_ids, noise_row);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_langevin_noise_sums(const fmb_langevin_t* lv, double* sums, fmb_stream_t stream_) {
    FMB_REQUIRE(lv && sums && lv->n_atoms > 0, "fmb_langevin_noise_sums: bad argument");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int blocks = std::min(kBlocks, ceil_div(lv->n_atoms, 256));
    k_noise<<<blocks, 256, 0, stream>>>(*lv);
    FMB_LAUNCH_CHECK();
    k_noise_sums<<<1, 32, 0, stream>>>(*lv, blocks, sums);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_langevin_first_half_global(const fmb_langevin_t* lv, const double* global_sums,
                                                      long long n_global, fmb_stream_t stream_) {
    FMB_REQUIRE(lv && global_sums && lv->n_atoms > 0 && n_global > 1, "fmb_langevin_first_half_global: bad argument");
    k_first_half<<<ceil_div(lv->n_atoms, 256), 256, 0, (cudaStream_t)stream_>>>(*lv, 0, global_sums, n_global);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_langevin_first_half(const fmb_langevin_t* lv, fmb_stream_t stream_) {
    FMB_REQUIRE(lv && lv->n_atoms > 1, "fmb_langevin_first_half: bad argument");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int blocks = std::min(kBlocks, ceil_div(lv->n_atoms, 256));
    k_noise<<<blocks, 256, 0, stream>>>(*lv);
    FMB_LAUNCH_CHECK();
    k_first_half<<<ceil_div(lv->n_atoms, 256), 256, 0, stream>>>(*lv, blocks, nullptr, 0);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_langevin_second_half(const fmb_langevin_t* lv, fmb_stream_t stream_) {
    FMB_REQUIRE(lv, "fmb_langevin_second_half: bad argument");
    k_second_half<<<ceil_div(lv->n_atoms, 256), 256, 0, (cudaStream_t)stream_>>>(*lv);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}
