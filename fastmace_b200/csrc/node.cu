// Per-atom stages: symmetric contraction (correlation 3) as a species-dependent polynomial in the 16 message
// components, readouts with their gradient, the float64 energy / virial reductions.
//
// Reference: EquivariantProductBasisBlock / SymmetricContraction of mace-torch, in the polynomial form the reference's
// generated kernels evaluate (fastmace/kernels/cuda/sc_generated.py:1-20: one block per atom, one thread per
// channel, y_C = sum_a w_a sum coef * monomial); energy contract fastmace/model/energy.py:92-99 (per-atom terms in
// model precision, reduced in float64, E0 in float64).

#include "stages.cuh"
#include "generated/symcon_generated.cuh"

namespace fmb {

namespace {

// One thread per (atom, channel); the polynomial is generated straight-line code (generated/symcon_generated.cuh):
// 16 inputs and the outputs live in registers, each coefficient is one coalesced load from the [species][term][C] table.
template <int LOUT>
__global__ void __launch_bounds__(kC)
k_symcon_forward(int n_atoms, int n_terms, const float* __restrict__ coef, const int32_t* __restrict__ species,
                 const float* __restrict__ msg, float* __restrict__ basis) {
    constexpr int OUT = SymconShape<LOUT>::kOut;
    const int a = blockIdx.x, c = threadIdx.x;
    if (a >= n_atoms) return;
    float x[kNSH], y[OUT];
#pragma unroll
    for (int k = 0; k < kNSH; ++k) x[k] = msg[((long long)a * kNSH + k) * kC + c];
#pragma unroll
    for (int k = 0; k < OUT; ++k) y[k] = 0.0f;
    symcon_forward_body<LOUT>(x, coef + (long long)species[a] * n_terms * kC + c, y);
#pragma unroll
    for (int k = 0; k < OUT; ++k) basis[((long long)a * OUT + k) * kC + c] = y[k];
}

template <int LOUT>
__global__ void __launch_bounds__(kC)
k_symcon_backward(int n_atoms, int n_terms, const float* __restrict__ coef, const int32_t* __restrict__ species,
                  const float* __restrict__ msg, const float* __restrict__ d_basis, float* __restrict__ d_msg) {
    constexpr int OUT = SymconShape<LOUT>::kOut;
    const int a = blockIdx.x, c = threadIdx.x;
    if (a >= n_atoms) return;
    float x[kNSH], dx[kNSH], g[OUT];
#pragma unroll
    for (int k = 0; k < kNSH; ++k) {
        x[k] = msg[((long long)a * kNSH + k) * kC + c];
        dx[k] = 0.0f;
    }
#pragma unroll
    for (int k = 0; k < OUT; ++k) g[k] = d_basis[((long long)a * OUT + k) * kC + c];
    symcon_backward_body<LOUT>(x, coef + (long long)species[a] * n_terms * kC + c, g, dx);
#pragma unroll
    for (int k = 0; k < kNSH; ++k) d_msg[((long long)a * kNSH + k) * kC + c] = dx[k];
}

// The same for kSymGroup atoms of one species per CTA (groups[g][0 .. kSymGroup), -1 = empty slot): a coefficient is
// loaded once and used for every atom of the group. Atoms at or beyond n_rows are skipped.
constexpr int kSymGroup = 4;

template <int LOUT, int R> struct SymconGroup;
#define FMB_SYMCON_GROUP(L_)                                                                                           \
    template <int R> struct SymconGroup<L_, R> {                                                                       \
        template <typename... A> static __device__ __forceinline__ void forward(A&&... a) {                           \
            symcon_forward_group_##L_<R>(a...);                                                                        \
        }                                                                                                              \
        template <typename... A> static __device__ __forceinline__ void backward(A&&... a) {                          \
            symcon_backward_group_##L_<R>(a...);                                                                       \
        }                                                                                                              \
    };
FMB_SYMCON_GROUP(0)
FMB_SYMCON_GROUP(1)
FMB_SYMCON_GROUP(2)

template <int LOUT>
__global__ void __launch_bounds__(kC)
k_symcon_forward_group(int n_groups, int n_rows, int n_terms, const float* __restrict__ coef,
                       const int32_t* __restrict__ species, const int32_t* __restrict__ groups,
                       const float* __restrict__ msg, float* __restrict__ basis) {
    constexpr int OUT = SymconShape<LOUT>::kOut, R = 2;       // half a group per CTA, like the adjoint
    const int c = threadIdx.x;
    int atom[R];
    int lead = -1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        atom[r] = groups[blockIdx.x * R + r];
        if (atom[r] >= n_rows) atom[r] = -1;
        if (lead < 0 && atom[r] >= 0) lead = atom[r];
    }
    if (lead < 0) return;
    float x[R][kNSH], y[R][OUT];
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int k = 0; k < kNSH; ++k) x[r][k] = atom[r] >= 0 ? msg[((long long)atom[r] * kNSH + k) * kC + c] : 0.0f;
#pragma unroll
        for (int k = 0; k < OUT; ++k) y[r][k] = 0.0f;
    }
    SymconGroup<LOUT, R>::forward(x, coef + (long long)species[lead] * n_terms * kC + c, y);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (atom[r] < 0) continue;
#pragma unroll
        for (int k = 0; k < OUT; ++k) basis[((long long)atom[r] * OUT + k) * kC + c] = y[r][k];
    }
}

// adjoint: two atoms per CTA (half a group), the registers hold x, dx and g of both
template <int LOUT>
__global__ void __launch_bounds__(kC)
k_symcon_backward_group(int n_groups, int n_rows, int n_terms, const float* __restrict__ coef,
                        const int32_t* __restrict__ species, const int32_t* __restrict__ groups,
                        const float* __restrict__ msg, const float* __restrict__ d_basis, float* __restrict__ d_msg) {
    constexpr int OUT = SymconShape<LOUT>::kOut, R = 2;
    const int c = threadIdx.x;
    int atom[R];
    int lead = -1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        atom[r] = groups[blockIdx.x * R + r];
        if (atom[r] >= n_rows) atom[r] = -1;
        if (lead < 0 && atom[r] >= 0) lead = atom[r];
    }
    if (lead < 0) return;
    float x[R][kNSH], dx[R][kNSH], g[R][OUT];
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int k = 0; k < kNSH; ++k) {
            x[r][k] = atom[r] >= 0 ? msg[((long long)atom[r] * kNSH + k) * kC + c] : 0.0f;
            dx[r][k] = 0.0f;
        }
#pragma unroll
        for (int k = 0; k < OUT; ++k) g[r][k] = atom[r] >= 0 ? d_basis[((long long)atom[r] * OUT + k) * kC + c] : 0.0f;
    }
    SymconGroup<LOUT, R>::backward(x, coef + (long long)species[lead] * n_terms * kC + c, g, dx);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (atom[r] < 0) continue;
#pragma unroll
        for (int k = 0; k < kNSH; ++k) d_msg[((long long)atom[r] * kNSH + k) * kC + c] = dx[r][k];
    }
}

// h[a][k][c] = table[species[a]][k][c]  (layer 0's species-only skip connection)
__global__ void k_fill_from_species(int n_atoms, int row, const int32_t* __restrict__ species,
                                    const float* __restrict__ table, float* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_atoms * row) return;
    const int a = (int)(i / row), k = (int)(i % row);
    out[i] = table[(long long)species[a] * row + k];
}

// One warp per atom. Non-last layers: e += h[a][0][:] . w, gradient w. Last layer: 128 -> 16 -> SiLU -> 1 with its
// gradient. The energy scale is folded in here. mode bit 0: add to node_energy instead of overwriting.
__global__ void __launch_bounds__(128)
k_readout(int n_atoms, int n_energy, int dim_first, int dim_last, int mlp_hidden, float scale, float shift, float silu_norm,
          const float* __restrict__ h_first, const float* __restrict__ h_last, const float* __restrict__ w_first,
          const float* __restrict__ w_last0, const float* __restrict__ w_last1, float* __restrict__ node_energy,
          float* __restrict__ d_h_first, float* __restrict__ d_h_last) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a = blockIdx.x * 4 + warp;
    if (a >= n_atoms) return;
    if (a >= n_energy) {
        // an atom whose energy belongs to another domain: it contributes no energy and seeds no gradient
        float* df = d_h_first + (long long)a * dim_first * kC;
        for (int k = lane; k < dim_first * kC; k += 32) df[k] = 0.0f;
        if (lane == 0) node_energy[a] = 0.0f;
        return;
    }
    // first readout (linear) and the gradient it leaves on h_first's scalars; other components start at zero
    float e = 0.0f;
    const float* hf = h_first + (long long)a * dim_first * kC;
    float* df = d_h_first + (long long)a * dim_first * kC;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int c = lane + 32 * q;
        e = fmaf(hf[c], w_first[c], e);
        df[c] = scale * w_first[c];
    }
    for (int k = kC + lane; k < dim_first * kC; k += 32) df[k] = 0.0f;
    // last readout
    const float* hl = h_last + (long long)a * dim_last * kC;
    float z[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) z[j] = 0.0f;
    float hv[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int c = lane + 32 * q;
        hv[q] = hl[c];
#pragma unroll
        for (int j = 0; j < 16; ++j) z[j] = fmaf(hv[q], w_last0[c * 16 + j], z[j]);
    }
    float dz[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float zz = warp_sum(z[j]);
        const float sig = 1.0f / (1.0f + expf(-zz));
        e += (lane == 0) ? silu_norm * zz * sig * w_last1[j] : 0.0f;
        dz[j] = scale * w_last1[j] * silu_norm * sig * (1.0f + zz * (1.0f - sig));
    }
    e = warp_sum(e);
    if (lane == 0) node_energy[a] = scale * e + shift;
    float* dl = d_h_last + (long long)a * dim_last * kC;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int c = lane + 32 * q;
        float g = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) g = fmaf(w_last0[c * 16 + j], dz[j], g);
        dl[c] = g;
    }
}

constexpr int kReduceBlocks = 256;

struct E0Table {
    double v[FMB_MAX_SPECIES];
};

// partial[b][0] = sum of node energies (+E0) of block b's atoms, partial[b][1..6] = virial components; float64.
__global__ void __launch_bounds__(256)
k_reduce_partial(int n_atoms, int n_energy, const float* __restrict__ node_energy, const int32_t* __restrict__ species,
                 E0Table e0, const float* __restrict__ atom_virial,
                 double* __restrict__ partial, const float* __restrict__ force_acc, float* __restrict__ forces) {
    __shared__ double sh[8][7];
    // the forces are minus the accumulated gradient (independent of the sums below; it saves a launch)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 3 * n_atoms; i += gridDim.x * blockDim.x) forces[i] = -force_acc[i];
    double acc[7] = {0, 0, 0, 0, 0, 0, 0};
    const int per_block = (n_atoms + gridDim.x - 1) / gridDim.x;
    const int begin = blockIdx.x * per_block, end = min(n_atoms, begin + per_block);
    for (int a = begin + threadIdx.x; a < end; a += blockDim.x) {
        if (a < n_energy) acc[0] += (double)node_energy[a] + e0.v[species[a]];
        if (atom_virial) {
#pragma unroll
            for (int q = 0; q < 6; ++q) acc[1 + q] += (double)atom_virial[6 * a + q];
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int q = 0; q < 7; ++q) {
        const double v = warp_sum(acc[q]);
        if (lane == 0) sh[warp][q] = v;
    }
    __syncthreads();
    if (threadIdx.x < 7) {
        double v = 0.0;
        for (int w = 0; w < 8; ++w) v += sh[w][threadIdx.x];
        partial[blockIdx.x * 8 + threadIdx.x] = v;
    }
}

// one warp per quantity (energy, six virial components): lane l adds blocks l, l + 32, ... in order, then a butterfly
// in fixed order -- the same sum every run
__global__ void __launch_bounds__(7 * 32)
k_reduce_final(int blocks, const double* __restrict__ partial, double inv_volume, int compute_stress,
               double* __restrict__ energy, float* __restrict__ stress, uint32_t* __restrict__ status) {
    const int q = threadIdx.x >> 5, lane = threadIdx.x & 31;
    double v = 0.0;
    for (int b = lane; b < blocks; b += 32) v += partial[b * 8 + q];
    v = warp_sum(v);
    if (lane != 0) return;
    if (q == 0) {
        *energy = v;
        if (!(v == v) || v > 1e300 || v < -1e300) atomicOr(status, FMB_STATUS_NONFINITE);
    } else if (compute_stress) {
        // order xx, yy, zz, yz, xz, xy
        const double s = v * inv_volume;
        const int idx[6][2] = {{0, 0}, {1, 1}, {2, 2}, {1, 2}, {0, 2}, {0, 1}};
        const int i = idx[q - 1][0], j = idx[q - 1][1];
        stress[3 * i + j] = (float)s;
        stress[3 * j + i] = (float)s;
    }
}

__global__ void k_commit(int n3, const float* __restrict__ forces, const double* __restrict__ energy,
                         const float* __restrict__ stress, double* __restrict__ f64, double* __restrict__ e64,
                         double* __restrict__ s64) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n3) f64[i] = (double)forces[i];
    if (i == 0) *e64 = *energy;
    if (s64 && i < 9) s64[i] = (double)stress[i];
}

}  // namespace

int symcon_forward(int n_atoms, int n_terms, int out_dim, const int32_t* terms, const float* coef,
                   const int32_t* species, const float* msg, float* basis, const int32_t* groups, int n_groups,
                   cudaStream_t stream) {
    (void)terms;
    if (n_atoms <= 0) return FMB_OK;
#define FMB_SYM(L_)                                                                                              \
    {                                                                                                            \
        FMB_REQUIRE(n_terms == SymconShape<L_>::kTerms, "symcon: coefficient table does not match the kernel"); \
        if (groups && n_groups > 0)                                                                              \
            k_symcon_forward_group<L_><<<2 * n_groups, kC, 0, stream>>>(2 * n_groups, n_atoms, n_terms, coef, species,   \
                                                                        groups, msg, basis);                     \
        else                                                                                                     \
            k_symcon_forward<L_><<<n_atoms, kC, 0, stream>>>(n_atoms, n_terms, coef, species, msg, basis);       \
    }
    if (out_dim == 1) FMB_SYM(0) else if (out_dim == 4) FMB_SYM(1) else if (out_dim == 9) FMB_SYM(2) else {
        FMB_REQUIRE(false, "symcon: unsupported output irreps");
    }
#undef FMB_SYM
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int symcon_backward(int n_atoms, int n_terms, int out_dim, const int32_t* terms, const float* coef,
                    const int32_t* species, const float* msg, const float* d_basis, float* d_msg, const int32_t* groups,
                    int n_groups, cudaStream_t stream) {
    (void)terms;
    if (n_atoms <= 0) return FMB_OK;
#define FMB_SYM(L_)                                                                                                  \
    {                                                                                                                \
        FMB_REQUIRE(n_terms == SymconShape<L_>::kTerms, "symcon: coefficient table does not match the kernel");     \
        if (groups && n_groups > 0)                                                                                  \
            k_symcon_backward_group<L_><<<2 * n_groups, kC, 0, stream>>>(2 * n_groups, n_atoms, n_terms, coef, species,  \
                                                                         groups, msg, d_basis, d_msg);               \
        else                                                                                                         \
            k_symcon_backward<L_><<<n_atoms, kC, 0, stream>>>(n_atoms, n_terms, coef, species, msg, d_basis, d_msg); \
    }
    if (out_dim == 1) FMB_SYM(0) else if (out_dim == 4) FMB_SYM(1) else if (out_dim == 9) FMB_SYM(2) else {
        FMB_REQUIRE(false, "symcon: unsupported output irreps");
    }
#undef FMB_SYM
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int fill_from_species(int n_atoms, int row, const int32_t* species, const float* table, float* out, cudaStream_t stream) {
    const long long total = (long long)n_atoms * row;
    k_fill_from_species<<<ceil_div(total, 256), 256, 0, stream>>>(n_atoms, row, species, table, out);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int readout(const fmb_model_t* m, int n_atoms, int n_energy, const float* h_first, const float* h_last,
            float* node_energy, float* d_h_first, float* d_h_last, cudaStream_t stream) {
    const int dim_first = (m->layer[0].l_out_max + 1) * (m->layer[0].l_out_max + 1);
    const int dim_last = 1;
    const float* w_last = m->layer[m->n_layers - 1].w_readout;
    k_readout<<<ceil_div(n_atoms, 4), 128, 0, stream>>>(n_atoms, n_energy, dim_first, dim_last, m->mlp_hidden, m->scale, m->shift,
                                                        m->silu_norm, h_first, h_last, m->layer[0].w_readout, w_last,
                                                        w_last + kC * 16, node_energy, d_h_first, d_h_last);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int reduce_outputs(const fmb_model_t* m, const fmb_work_t* w, int n_energy, double volume, cudaStream_t stream) {
    E0Table e0;
    for (int k = 0; k < FMB_MAX_SPECIES; ++k) e0.v[k] = m->e0[k];
    k_reduce_partial<<<kReduceBlocks, 256, 0, stream>>>(w->n_atoms, n_energy, w->node_energy, w->species, e0,
                                                        w->compute_stress ? w->atom_virial : nullptr, w->partial,
                                                        w->force_acc, w->forces);
    FMB_LAUNCH_CHECK();
    k_reduce_final<<<1, 7 * 32, 0, stream>>>(kReduceBlocks, w->partial, 1.0 / volume, w->compute_stress, w->energy, w->stress,
                                         w->status);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int commit_forces(const fmb_work_t* w, double* f64, double* e64, double* s64, cudaStream_t stream) {
    k_commit<<<ceil_div(3LL * w->n_atoms, 256), 256, 0, stream>>>(3 * w->n_atoms, w->forces, w->energy, w->stress, f64,
                                                                  e64, s64);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace fmb
