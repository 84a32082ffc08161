// Pack / unpack kernels of the halo exchange of a spatially decomposed run (one rank per GPU, each rank owns the atoms
// of one brick of the periodic cell and holds the atoms within cutoff + skin of it as halo atoms).
//
// Four exchanges per step move rows between an atom's owner and the ranks that hold it as a halo atom: positions and
// the node features x = linear_up(h1) outwards, the gradient of x and the partial forces back. A rank's halo atoms
// are ordered by owner, so whatever arrives from one peer is one contiguous block of rows: receives land in place
// (no unpack kernel on the forward exchanges) and the reverse exchanges send straight out of the halo rows (no pack
// kernel). The two kernels here cover the other ends: gathering the rows a peer asked for into the send buffer, and
// adding what came back into the owners' rows in a fixed order (no atomics, so the sums are reproducible).
//
// The reference runs one structure on one GPU (SPEC.md:70-74); its tiled backend's "receivers + edges + halo senders"
// tile (fastmace/model/tiled.py:1-26) is the structural precedent.

#include "fmb_common.cuh"

#include <algorithm>

namespace fmb {

namespace {

// out[i][:] = rows[index[i]][:], rows of `width` 4-byte words
__global__ void __launch_bounds__(256)
k_gather_rows(const uint32_t* __restrict__ rows, const int32_t* __restrict__ index, uint32_t* __restrict__ out, int n,
              int width) {
    const long long total = (long long)n * width;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(t / width), w = (int)(t - (long long)i * width);
        out[t] = rows[(long long)index[i] * width + w];
    }
}

// dst[target[t]][:] += sum over k in [ptr[t], ptr[t + 1]) of recv[source[k]][:], summed in the order of k
template <typename T>
__global__ void __launch_bounds__(128)
k_add_rows(const T* __restrict__ recv, const int32_t* __restrict__ ptr, const int32_t* __restrict__ source,
           const int32_t* __restrict__ target, T* __restrict__ dst, int n_targets, int width) {
    for (int t = blockIdx.x; t < n_targets; t += gridDim.x) {
        const int b = ptr[t], e = ptr[t + 1];
        if (b == e) continue;
        T* out = dst + (long long)(target ? target[t] : t) * width;
        for (int w = threadIdx.x; w < width; w += blockDim.x) {
            T acc = out[w];
            for (int k = b; k < e; ++k) acc += recv[(long long)source[k] * width + w];
            out[w] = acc;
        }
    }
}

// positions of the local atoms in the rank's own frame: owned atoms first (the state's positions may lie outside the
// cell: `shift` brings them into the brick), then the halo atoms as received from their owners plus the shift of
// their periodic image, everything minus the frame's origin; shift is [n_owned + n_halo][3]
__global__ void __launch_bounds__(256)
k_local_positions(const double* __restrict__ owned, int n_owned, const double* __restrict__ received,
                  const double* __restrict__ shift, int n_halo, double ox, double oy, double oz,
                  double* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_owned + n_halo) return;
    const double origin[3] = {ox, oy, oz};
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const double x = i < n_owned ? owned[3 * i + a] : received[3 * (i - n_owned) + a];
        out[3 * i + a] = __dsub_rn(__dadd_rn(x, shift[3 * i + a]), origin[a]);
    }
}

// state forces (float64) of the owned atoms from the rank's partial forces (fp32, already the negative gradient) and
// the shares that came back from the ranks holding these atoms as halo atoms, summed in a fixed order
__global__ void __launch_bounds__(256)
k_owned_forces(const float* __restrict__ local_forces, const float* __restrict__ recv, const int32_t* __restrict__ ptr,
               const int32_t* __restrict__ source, int n_owned, double* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_owned) return;
    float acc[3] = {local_forces[3 * i], local_forces[3 * i + 1], local_forces[3 * i + 2]};
    if (ptr)
        for (int k = ptr[i]; k < ptr[i + 1]; ++k) {
            const long long r = 3LL * source[k];
            acc[0] += recv[r]; acc[1] += recv[r + 1]; acc[2] += recv[r + 2];
        }
    out[3 * i] = acc[0]; out[3 * i + 1] = acc[1]; out[3 * i + 2] = acc[2];
}

}  // namespace

}  // namespace fmb

using namespace fmb;

extern "C" FMB_API int fmb_halo_gather_rows(const void* rows, const int32_t* index, void* out, int n, int row_bytes,
                                            fmb_stream_t stream) {
    FMB_REQUIRE(n >= 0 && row_bytes > 0 && row_bytes % 4 == 0, "fmb_halo_gather_rows: rows are multiples of 4 bytes");
    if (n == 0) return FMB_OK;
    FMB_REQUIRE(rows && index && out, "fmb_halo_gather_rows: null argument");
    const int width = row_bytes / 4;
    const long long total = (long long)n * width;
    const int blocks = (int)std::min<long long>((total + 255) / 256, 148 * 16);
    k_gather_rows<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint32_t*)rows, index, (uint32_t*)out, n, width);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_halo_add_rows(const float* received, const int32_t* ptr, const int32_t* source,
                                         const int32_t* target, float* dst, int n_targets, int row_floats,
                                         fmb_stream_t stream) {
    FMB_REQUIRE(n_targets >= 0 && row_floats > 0, "fmb_halo_add_rows: bad size");
    if (n_targets == 0) return FMB_OK;
    FMB_REQUIRE(received && ptr && source && dst, "fmb_halo_add_rows: null argument");
    k_add_rows<float><<<std::min(n_targets, 148 * 16), 128, 0, (cudaStream_t)stream>>>(received, ptr, source, target, dst,
                                                                                       n_targets, row_floats);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_halo_local_positions(const double* owned, int n_owned, const double* received,
                                                const double* shift, int n_halo, const double* origin, double* out,
                                                fmb_stream_t stream) {
    FMB_REQUIRE(n_owned >= 0 && n_halo >= 0 && origin && out, "fmb_halo_local_positions: bad argument");
    const int n = n_owned + n_halo;
    if (n == 0) return FMB_OK;
    FMB_REQUIRE((n_owned == 0 || owned) && (n_halo == 0 || received) && shift, "fmb_halo_local_positions: null argument");
    k_local_positions<<<ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(owned, n_owned, received, shift, n_halo,
                                                                          origin[0], origin[1], origin[2], out);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_halo_owned_forces(const float* local_forces, const float* received, const int32_t* ptr,
                                             const int32_t* source, int n_owned, double* forces64, fmb_stream_t stream) {
    FMB_REQUIRE(n_owned >= 0, "fmb_halo_owned_forces: bad size");
    if (n_owned == 0) return FMB_OK;
    FMB_REQUIRE(local_forces && forces64 && (!ptr || (received && source)), "fmb_halo_owned_forces: null argument");
    k_owned_forces<<<ceil_div(n_owned, 256), 256, 0, (cudaStream_t)stream>>>(local_forces, received, ptr, source, n_owned,
                                                                             forces64);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}
