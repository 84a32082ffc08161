// Periodic cell-list neighbour build with a Verlet skin, receiver-sorted CSR output, stable compaction to the cutoff
// and the rebuild test. Replaces SkinNeighbourList.build_gpu / compact / needs_rebuild
// (fastmace/neighbors/skin.py:421-497, 702-729, 685-693) and the screen kernels of fastmace/neighbors/pair_search.py.
//
// Design: atoms are binned in fractional slabs at least (cutoff + skin) thick; one warp per receiver walks the
// stencil of neighbouring bins (with the periodic image read off the wrap), decides every pair in float64 with the
// reference's expression, and sorts its own short row by (sender, image) in shared memory. No global sort, no
// host synchronisation; every kernel can be gated by a device flag so that a rebuild can sit inside a captured step.
//
// Float64 arithmetic uses explicit round-to-nearest multiplies and adds in the reference's order (no FMA
// contraction), so the decisions are those of the reference's element-wise expressions.

#include "fmb_common.cuh"

#include <cooperative_groups.h>

namespace fmb {

namespace {

__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }

// rows @ matrix for one row: r0 * m[0] + r1 * m[1] + r2 * m[2], left to right (skin.py:100-102)
__device__ __forceinline__ void times_3x3(double r0, double r1, double r2, const double* __restrict__ m, double* out) {
#pragma unroll
    for (int a = 0; a < 3; ++a) out[a] = add(add(mul(r0, m[a]), mul(r1, m[3 + a])), mul(r2, m[6 + a]));
}

__device__ __forceinline__ double norm2(double x, double y, double z) {
    return add(add(mul(x, x), mul(y, y)), mul(z, z));
}

struct NlConst {
    double cell[9];
    double inverse[9];
    int nbins[3];
    int reach[3];
    double reach2;     // (cutoff + skin)^2
    double cutoff2;
};

__device__ __forceinline__ void zero_bins_item(int i, int32_t* bin_count, int32_t* bin_fill, int total_bins) {
    if (i <= total_bins) bin_count[i] = 0;
    if (i < total_bins) bin_fill[i] = 0;
}

__global__ void k_zero_bins(int32_t* bin_count, int32_t* bin_fill, int total_bins, const int32_t* flag) {
    if (flag && *flag == 0) return;
    zero_bins_item(blockIdx.x * blockDim.x + threadIdx.x, bin_count, bin_fill, total_bins);
}

__device__ __forceinline__ void wrap_bin_item(const NlConst& c, int i, const double* __restrict__ x,
                                              double* __restrict__ wrapped, double* __restrict__ offsets,
                                              int32_t* __restrict__ atom_bin, int32_t* __restrict__ bin_count) {
    double p0 = x[3 * i], p1 = x[3 * i + 1], p2 = x[3 * i + 2];
    double frac[3], off[3], back[3];
    times_3x3(p0, p1, p2, c.inverse, frac);
#pragma unroll
    for (int a = 0; a < 3; ++a) off[a] = floor(frac[a]);
    times_3x3(off[0], off[1], off[2], c.cell, back);
    int b[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        wrapped[3 * i + a] = sub((a == 0 ? p0 : a == 1 ? p1 : p2), back[a]);
        offsets[3 * i + a] = off[a];
        double fw = frac[a] - off[a];
        int v = (int)(fw * (double)c.nbins[a]);
        b[a] = min(max(v, 0), c.nbins[a] - 1);
    }
    int bin = (b[0] * c.nbins[1] + b[1]) * c.nbins[2] + b[2];
    atom_bin[i] = bin;
    atomicAdd(&bin_count[bin], 1);
}

__global__ void k_wrap_bin(NlConst c, int n, const double* __restrict__ x, double* __restrict__ wrapped,
                           double* __restrict__ offsets, int32_t* __restrict__ atom_bin, int32_t* __restrict__ bin_count,
                           const int32_t* flag) {
    if (flag && *flag == 0) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) wrap_bin_item(c, i, x, wrapped, offsets, atom_bin, bin_count);
}

__device__ __forceinline__ void bin_fill_item(int i, const int32_t* __restrict__ atom_bin,
                                              const int32_t* __restrict__ bin_start, int32_t* __restrict__ bin_fill,
                                              int32_t* __restrict__ bin_atoms) {
    const int bin = atom_bin[i];
    const int slot = atomicAdd(&bin_fill[bin], 1);
    bin_atoms[bin_start[bin] + slot] = i;
}

__global__ void k_bin_fill(int n, const int32_t* __restrict__ atom_bin, const int32_t* __restrict__ bin_start,
                           int32_t* __restrict__ bin_fill, int32_t* __restrict__ bin_atoms, const int32_t* flag) {
    if (flag && *flag == 0) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) bin_fill_item(i, atom_bin, bin_start, bin_fill, bin_atoms);
}

constexpr int kWarpsPerBlock = 4;

// One warp per receiver. MODE 0: count the candidates; MODE 1: collect, sort by (sender, image) and write them.
template <int MODE>
__device__ __forceinline__ void rows_receiver(const NlConst& c, int r, int lane, unsigned long long* keys, int capacity,
                                              const double* __restrict__ wrapped, const double* __restrict__ offsets,
                                              const int32_t* __restrict__ atom_bin, const int32_t* __restrict__ bin_start,
                                              const int32_t* __restrict__ bin_atoms, int32_t* __restrict__ row_count,
                                              const int32_t* __restrict__ row_ptr, int32_t* __restrict__ cand_index,
                                              float* __restrict__ cand_shift, uint32_t* __restrict__ status) {
    const double rx = wrapped[3 * r], ry = wrapped[3 * r + 1], rz = wrapped[3 * r + 2];
    const int bin = atom_bin[r];
    const int b2 = bin % c.nbins[2], b1 = (bin / c.nbins[2]) % c.nbins[1], b0 = bin / (c.nbins[2] * c.nbins[1]);
    int found = 0;
    for (int d0 = -c.reach[0]; d0 <= c.reach[0]; ++d0) {
        const int B0 = b0 + d0;
        const int n0 = (B0 >= 0) ? B0 / c.nbins[0] : -((-B0 + c.nbins[0] - 1) / c.nbins[0]);
        const int s0 = B0 - n0 * c.nbins[0];
        for (int d1 = -c.reach[1]; d1 <= c.reach[1]; ++d1) {
            const int B1 = b1 + d1;
            const int n1 = (B1 >= 0) ? B1 / c.nbins[1] : -((-B1 + c.nbins[1] - 1) / c.nbins[1]);
            const int s1 = B1 - n1 * c.nbins[1];
            for (int d2 = -c.reach[2]; d2 <= c.reach[2]; ++d2) {
                const int B2 = b2 + d2;
                const int n2 = (B2 >= 0) ? B2 / c.nbins[2] : -((-B2 + c.nbins[2] - 1) / c.nbins[2]);
                const int s2 = B2 - n2 * c.nbins[2];
                // the sender's image sits n cells away, so the reference's image (added to r - s) is -n
                const double i0 = (double)(-n0), i1 = (double)(-n1), i2 = (double)(-n2);
                double iv[3];
                times_3x3(i0, i1, i2, c.cell, iv);
                const int sbin = (s0 * c.nbins[1] + s1) * c.nbins[2] + s2;
                const int begin = bin_start[sbin], end = bin_start[sbin + 1];
                for (int base = begin; base < end; base += 32) {
                    const int k = base + lane;
                    bool hit = false;
                    int s = 0;
                    if (k < end) {
                        s = bin_atoms[k];
                        const double vx = add(sub(rx, wrapped[3 * s]), iv[0]);
                        const double vy = add(sub(ry, wrapped[3 * s + 1]), iv[1]);
                        const double vz = add(sub(rz, wrapped[3 * s + 2]), iv[2]);
                        hit = norm2(vx, vy, vz) < c.reach2;
                        if (hit && s == r) {
                            // self pair: dropped only when the unit shift is zero (skin.py:462-463)
                            hit = !(n0 == 0 && n1 == 0 && n2 == 0);
                        }
                    }
                    const unsigned mask = __ballot_sync(0xffffffffu, hit);
                    if (MODE == 1 && hit) {
                        const int slot = found + __popc(mask & ((1u << lane) - 1u));
                        if (slot < FMB_MAX_ROW) {
                            const unsigned long long image_key =
                                ((unsigned long long)(-n0 + 128) << 16) | ((unsigned long long)(-n1 + 128) << 8) |
                                (unsigned long long)(-n2 + 128);
                            keys[slot] = ((unsigned long long)(unsigned)s << 24) | image_key;
                        }
                    }
                    found += __popc(mask);
                }
            }
        }
    }
    if (MODE == 0) {
        if (lane == 0) row_count[r] = found;
        return;
    }
    if (found > FMB_MAX_ROW) {
        if (lane == 0) atomicOr(status, FMB_STATUS_ROW_OVERFLOW);
        found = FMB_MAX_ROW;
    }
    // bitonic sort of keys[0..found) padded to a power of two
    int padded = 32;
    while (padded < found) padded <<= 1;
    for (int k = found + lane; k < padded; k += 32) keys[k] = ~0ull;
    __syncwarp();
    for (int size = 2; size <= padded; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = lane; t < (padded >> 1); t += 32) {
                const int lo = ((t / stride) * (stride << 1)) + (t % stride);
                const int hi = lo + stride;
                const bool ascending = ((lo & size) == 0);
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a > b) == ascending) {
                    keys[lo] = b;
                    keys[hi] = a;
                }
            }
            __syncwarp();
        }
    }
    const int start = row_ptr[r];
    const double or0 = offsets[3 * r], or1 = offsets[3 * r + 1], or2 = offsets[3 * r + 2];
    for (int k = lane; k < found; k += 32) {
        const int dst = start + k;
        if (dst >= capacity) break;
        const unsigned long long key = keys[k];
        const int s = (int)(key >> 24);
        const double i0 = (double)((int)((key >> 16) & 0xff) - 128);
        const double i1 = (double)((int)((key >> 8) & 0xff) - 128);
        const double i2 = (double)((int)(key & 0xff) - 128);
        cand_index[dst] = s;
        cand_index[capacity + dst] = r;
        cand_shift[3 * dst + 0] = (float)add(sub(i0, or0), offsets[3 * s]);
        cand_shift[3 * dst + 1] = (float)add(sub(i1, or1), offsets[3 * s + 1]);
        cand_shift[3 * dst + 2] = (float)add(sub(i2, or2), offsets[3 * s + 2]);
    }
}

template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_rows(NlConst c, int n, int capacity, const double* __restrict__ wrapped, const double* __restrict__ offsets,
       const int32_t* __restrict__ atom_bin, const int32_t* __restrict__ bin_start, const int32_t* __restrict__ bin_atoms,
       int32_t* __restrict__ row_count, const int32_t* __restrict__ row_ptr, int32_t* __restrict__ cand_index,
       float* __restrict__ cand_shift, uint32_t* __restrict__ status, const int32_t* flag) {
    if (flag && *flag == 0) return;
    extern __shared__ unsigned long long s_keys[];   // MODE 1: [kWarpsPerBlock][FMB_MAX_ROW]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * kWarpsPerBlock + warp;
    if (r >= n) return;
    unsigned long long* keys = MODE == 1 ? s_keys + (size_t)warp * FMB_MAX_ROW : nullptr;
    rows_receiver<MODE>(c, r, lane, keys, capacity, wrapped, offsets, atom_bin, bin_start, bin_atoms, row_count, row_ptr,
                        cand_index, cand_shift, status);
}

struct FinishArgs {
    float pad0, pad1, pad2;
    int32_t* cand_index;
    float* cand_shift;
    int32_t* edge_index;
    float* unit_shifts;
    float* shifts;
    int64_t* num_candidates;
    double* reference;
    double* build_cell;
    uint32_t* status;
};

__device__ __forceinline__ void finish_items(const NlConst& c, int n, int capacity, const int32_t* __restrict__ row_ptr,
                                             const double* __restrict__ x, const FinishArgs& f, int tid, int stride) {
    const float pad0 = f.pad0, pad1 = f.pad1, pad2 = f.pad2;
    int32_t* const cand_index = f.cand_index;
    float* const cand_shift = f.cand_shift;
    int32_t* const edge_index = f.edge_index;
    float* const unit_shifts = f.unit_shifts;
    float* const shifts = f.shifts;
    int64_t* const num_candidates = f.num_candidates;
    double* const reference = f.reference;
    double* const build_cell = f.build_cell;
    uint32_t* const status = f.status;
    const int total = row_ptr[n];
    if (tid == 0) {
        *num_candidates = total;
        if (total > capacity) atomicOr(status, FMB_STATUS_CAND_OVERFLOW);
        for (int k = 0; k < 9; ++k) build_cell[k] = c.cell[k];
    }
    double ps[3];
    times_3x3((double)pad0, (double)pad1, (double)pad2, c.cell, ps);
    for (int k = min(total, capacity) + tid; k < capacity; k += stride) {
        cand_index[k] = 0;
        cand_index[capacity + k] = 0;
        edge_index[k] = 0;
        edge_index[capacity + k] = 0;
        cand_shift[3 * k] = pad0; cand_shift[3 * k + 1] = pad1; cand_shift[3 * k + 2] = pad2;
        unit_shifts[3 * k] = pad0; unit_shifts[3 * k + 1] = pad1; unit_shifts[3 * k + 2] = pad2;
        shifts[3 * k] = (float)ps[0]; shifts[3 * k + 1] = (float)ps[1]; shifts[3 * k + 2] = (float)ps[2];
    }
    for (int k = tid; k < 3 * n; k += stride) reference[k] = x[k];
}

__global__ void k_finish_build(NlConst c, int n, int capacity, const int32_t* __restrict__ row_ptr,
                               const double* __restrict__ x, FinishArgs f, const int32_t* flag) {
    if (flag && *flag == 0) return;
    finish_items(c, n, capacity, row_ptr, x, f, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
}

// compact: MODE 0 counts the candidates of each receiver inside the cutoff; MODE 1 writes the stable partition.
template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_compact(NlConst c, int n, int capacity, const double* __restrict__ x, const int32_t* __restrict__ cand_row_ptr,
          const int32_t* __restrict__ cand_index, const float* __restrict__ cand_shift,
          int32_t* __restrict__ edge_row_count, const int32_t* __restrict__ edge_row_ptr,
          int32_t* __restrict__ edge_index, float* __restrict__ unit_shifts, float* __restrict__ shifts,
          int64_t* __restrict__ count_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * kWarpsPerBlock + warp;
    if (r >= n) return;
    const int total = min(cand_row_ptr[n], capacity);
    const int begin = min(cand_row_ptr[r], total), end = min(cand_row_ptr[r + 1], total);
    const double rx = x[3 * r], ry = x[3 * r + 1], rz = x[3 * r + 2];
    int inside_before = 0, outside_before = 0;
    int in_base = 0, out_base = 0;
    if (MODE == 1) {
        const int count = edge_row_ptr[n];
        in_base = edge_row_ptr[r];
        out_base = count + (begin - in_base);
        if (r == 0 && lane == 0) *count_out = count;
    }
    for (int base = begin; base < end; base += 32) {
        const int k = base + lane;
        bool valid = k < end, inside = false;
        int s = 0;
        float u0 = 0.f, u1 = 0.f, u2 = 0.f;
        double sh[3] = {0.0, 0.0, 0.0};
        if (valid) {
            s = cand_index[k];
            u0 = cand_shift[3 * k]; u1 = cand_shift[3 * k + 1]; u2 = cand_shift[3 * k + 2];
            times_3x3((double)u0, (double)u1, (double)u2, c.cell, sh);
            const double vx = add(sub(rx, x[3 * s]), sh[0]);
            const double vy = add(sub(ry, x[3 * s + 1]), sh[1]);
            const double vz = add(sub(rz, x[3 * s + 2]), sh[2]);
            inside = norm2(vx, vy, vz) < c.cutoff2;
        }
        const unsigned in_mask = __ballot_sync(0xffffffffu, inside);
        const unsigned out_mask = __ballot_sync(0xffffffffu, valid && !inside);
        if (MODE == 1 && valid) {
            const unsigned lt = (1u << lane) - 1u;
            const int dst = inside ? in_base + inside_before + __popc(in_mask & lt)
                                   : out_base + outside_before + __popc(out_mask & lt);
            edge_index[dst] = s;
            edge_index[capacity + dst] = r;
            unit_shifts[3 * dst] = u0; unit_shifts[3 * dst + 1] = u1; unit_shifts[3 * dst + 2] = u2;
            shifts[3 * dst] = (float)sh[0]; shifts[3 * dst + 1] = (float)sh[1]; shifts[3 * dst + 2] = (float)sh[2];
        }
        inside_before += __popc(in_mask);
        outside_before += __popc(out_mask);
    }
    if (MODE == 0 && lane == 0) edge_row_count[r] = inside_before;
}

__global__ void k_max_displacement(int n, const double* __restrict__ x, const double* __restrict__ ref,
                                   unsigned long long* __restrict__ max_bits) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    double d2 = 0.0;
    if (i < n) {
        const double dx = sub(x[3 * i], ref[3 * i]), dy = sub(x[3 * i + 1], ref[3 * i + 1]),
                     dz = sub(x[3 * i + 2], ref[3 * i + 2]);
        d2 = norm2(dx, dy, dz);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d2 = fmax(d2, __shfl_xor_sync(0xffffffffu, d2, o));
    if ((threadIdx.x & 31) == 0 && d2 > 0.0) atomicMax(max_bits, (unsigned long long)__double_as_longlong(d2));
}

__global__ void k_rebuild_flag(const unsigned long long* __restrict__ max_bits, double threshold2, int32_t* flag) {
    *flag = __longlong_as_double((long long)*max_bits) > threshold2 ? 1 : 0;
}

// The same test in one launch for lists of a few thousand atoms (one CTA walks them): the maximum is exact whatever
// the order, so the flag and the recorded maximum equal those of the three-node form above.
constexpr int kSmallTestAtoms = 8192;

__global__ void __launch_bounds__(1024)
k_rebuild_test_small(int n, const double* __restrict__ x, const double* __restrict__ ref, double threshold2,
                     unsigned long long* __restrict__ max_bits, int32_t* __restrict__ flag) {
    __shared__ double warp_max[32];
    double d2 = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const double dx = sub(x[3 * i], ref[3 * i]), dy = sub(x[3 * i + 1], ref[3 * i + 1]),
                     dz = sub(x[3 * i + 2], ref[3 * i + 2]);
        d2 = fmax(d2, norm2(dx, dy, dz));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d2 = fmax(d2, __shfl_xor_sync(0xffffffffu, d2, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = d2;
    __syncthreads();
    if (threadIdx.x < 32) {
        d2 = warp_max[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d2 = fmax(d2, __shfl_xor_sync(0xffffffffu, d2, o));
        if (threadIdx.x == 0) {
            *max_bits = d2 > 0.0 ? (unsigned long long)__double_as_longlong(d2) : 0ull;
            *flag = d2 > threshold2 ? 1 : 0;
        }
    }
}

// ---------------------------------------------------------------------------------------------- scan
__global__ void __launch_bounds__(kScanBlock)
k_scan_tiles(const int32_t* __restrict__ in, int32_t* __restrict__ out, int n, int32_t* __restrict__ tile_sums,
             const int32_t* flag, int write_total) {
    if (flag && *flag == 0) return;
    __shared__ int32_t warp_totals[32];
    const int tile = blockIdx.x;
    const int base = tile * kScanTile + threadIdx.x * kScanItems;
    int v[kScanItems];
    int sum = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        v[k] = (base + k < n) ? in[base + k] : 0;
        sum += v[k];
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) warp_totals[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = warp_totals[lane];
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        warp_totals[lane] = wi - w;   // exclusive
        if (lane == 31) {
            tile_sums[tile] = wi;
            if (write_total) out[n] = wi;     // a scan of one tile is complete here
        }
    }
    __syncthreads();
    int run = warp_totals[warp] + incl - sum;
#pragma unroll
    for (int k = 0; k < kScanItems; ++k) {
        if (base + k < n) out[base + k] = run;
        run += v[k];
    }
}

__global__ void __launch_bounds__(kScanBlock)
k_scan_sums(int32_t* __restrict__ tile_sums, int tiles, int32_t* __restrict__ out, int n, const int32_t* flag) {
    if (flag && *flag == 0) return;
    // a single block scans the tile totals serially in chunks of kScanBlock (tiles <= a few thousand)
    __shared__ int32_t buf[kScanBlock];
    __shared__ int32_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < tiles; base += kScanBlock) {
        const int i = base + threadIdx.x;
        const int v = (i < tiles) ? tile_sums[i] : 0;
        buf[threadIdx.x] = v;
        __syncthreads();
        for (int o = 1; o < kScanBlock; o <<= 1) {
            int t = (threadIdx.x >= o) ? buf[threadIdx.x - o] : 0;
            __syncthreads();
            buf[threadIdx.x] += t;
            __syncthreads();
        }
        if (i < tiles) tile_sums[i] = carry + buf[threadIdx.x] - v;
        __syncthreads();
        if (threadIdx.x == 0) carry += buf[kScanBlock - 1];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[n] = carry;
}

__global__ void k_scan_add(int32_t* __restrict__ out, int n, const int32_t* __restrict__ tile_sums, const int32_t* flag) {
    if (flag && *flag == 0) return;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] += tile_sums[i / kScanTile];
}

// ------------------------------------------------------------------------------ gated build of a small list
// The eight launches of a build as one cooperative kernel, for lists whose two scans fit one CTA (atoms and bins up to
// kSmallBuild). Inside a captured step the build is gated by the device flag; a step that does not rebuild then pays
// for one launch that reads the flag and returns instead of eight. The phases are the kernels' own bodies, separated by
// grid barriers; the result is the same list (the order inside a bin depends on the atomics as before, the rows are
// sorted afterwards).
constexpr int kSmallBuild = 4096;
constexpr int kCoopThreads = 256;

struct SmallBuildArgs {
    NlConst c;
    int n, capacity, total_bins;
    const double* x;
    double* wrapped;
    double* offsets;
    int32_t* atom_bin;
    int32_t* bin_count;
    int32_t* bin_start;
    int32_t* bin_fill;
    int32_t* bin_atoms;
    int32_t* cand_row_count;
    int32_t* cand_row_ptr;
    FinishArgs finish;
    const int32_t* flag;
};

// exclusive scan of n <= kSmallBuild values by one CTA of kCoopThreads threads, total at out[n]
__device__ void scan_by_one_cta(const int32_t* __restrict__ in, int32_t* __restrict__ out, int n) {
    constexpr int kItems = kSmallBuild / kCoopThreads;
    __shared__ int32_t warp_totals[kCoopThreads / 32];
    const int base = threadIdx.x * kItems;
    int v[kItems];
    int sum = 0;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
        v[k] = base + k < n ? in[base + k] : 0;
        sum += v[k];
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) warp_totals[warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < kCoopThreads / 32; ++w) {
        if (w < warp) before += warp_totals[w];
        total += warp_totals[w];
    }
    int run = before + incl - sum;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
        if (base + k < n) out[base + k] = run;
        run += v[k];
    }
    if (threadIdx.x == 0) out[n] = total;
    __syncthreads();
}

__global__ void __launch_bounds__(kCoopThreads)
k_build_small(const __grid_constant__ SmallBuildArgs a) {
    if (a.flag && *a.flag == 0) return;                 // the same answer in every CTA: nobody reaches a grid barrier
    extern __shared__ unsigned long long s_keys[];      // [warps of the CTA][FMB_MAX_ROW]
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    const int tid = blockIdx.x * kCoopThreads + threadIdx.x, stride = gridDim.x * kCoopThreads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first_row = blockIdx.x * (kCoopThreads / 32) + warp, row_stride = gridDim.x * (kCoopThreads / 32);
    for (int i = tid; i <= a.total_bins; i += stride) zero_bins_item(i, a.bin_count, a.bin_fill, a.total_bins);
    grid.sync();
    for (int i = tid; i < a.n; i += stride) wrap_bin_item(a.c, i, a.x, a.wrapped, a.offsets, a.atom_bin, a.bin_count);
    grid.sync();
    if (blockIdx.x == 0) scan_by_one_cta(a.bin_count, a.bin_start, a.total_bins);
    grid.sync();
    for (int i = tid; i < a.n; i += stride) bin_fill_item(i, a.atom_bin, a.bin_start, a.bin_fill, a.bin_atoms);
    grid.sync();
    for (int r = first_row; r < a.n; r += row_stride)
        rows_receiver<0>(a.c, r, lane, nullptr, a.capacity, a.wrapped, a.offsets, a.atom_bin, a.bin_start, a.bin_atoms,
                         a.cand_row_count, nullptr, nullptr, nullptr, a.finish.status);
    grid.sync();
    if (blockIdx.x == 0) scan_by_one_cta(a.cand_row_count, a.cand_row_ptr, a.n);
    grid.sync();
    for (int r = first_row; r < a.n; r += row_stride) {
        rows_receiver<1>(a.c, r, lane, s_keys + (size_t)warp * FMB_MAX_ROW, a.capacity, a.wrapped, a.offsets, a.atom_bin,
                         a.bin_start, a.bin_atoms, nullptr, a.cand_row_ptr, a.finish.cand_index, a.finish.cand_shift,
                         a.finish.status);
        __syncwarp();
    }
    grid.sync();
    finish_items(a.c, a.n, a.capacity, a.cand_row_ptr, a.x, a.finish, tid, stride);
}

NlConst make_const(const fmb_nl_t* nl) {
    NlConst c;
    for (int k = 0; k < 9; ++k) {
        c.cell[k] = nl->cell[k];
        c.inverse[k] = nl->inverse[k];
    }
    for (int a = 0; a < 3; ++a) {
        c.nbins[a] = nl->nbins[a];
        c.reach[a] = nl->reach_bins[a];
    }
    const double reach = nl->cutoff + nl->skin;
    c.reach2 = reach * reach;
    c.cutoff2 = nl->cutoff * nl->cutoff;
    return c;
}

}  // namespace

int exclusive_scan(const int32_t* in, int32_t* out, int n, int32_t* scratch, const int32_t* flag, cudaStream_t stream) {
    const int tiles = ceil_div(n, kScanTile);
    k_scan_tiles<<<tiles, kScanBlock, 0, stream>>>(in, out, n, scratch, flag, tiles == 1 ? 1 : 0);
    FMB_LAUNCH_CHECK();
    if (tiles == 1) return FMB_OK;
    k_scan_sums<<<1, kScanBlock, 0, stream>>>(scratch, tiles, out, n, flag);
    FMB_LAUNCH_CHECK();
    if (tiles > 1) {
        k_scan_add<<<ceil_div(n, 256), 256, 0, stream>>>(out, n, scratch, flag);
        FMB_LAUNCH_CHECK();
    }
    return FMB_OK;
}

}  // namespace fmb

using namespace fmb;

namespace fmb {
namespace {

FinishArgs finish_args(const fmb_nl_t* nl) {
    FinishArgs f;
    f.pad0 = nl->pad_unit_shift[0]; f.pad1 = nl->pad_unit_shift[1]; f.pad2 = nl->pad_unit_shift[2];
    f.cand_index = nl->candidate_index; f.cand_shift = nl->candidate_unit_shifts;
    f.edge_index = nl->edge_index; f.unit_shifts = nl->unit_shifts; f.shifts = nl->shifts;
    f.num_candidates = nl->num_candidates; f.reference = nl->reference_positions; f.build_cell = nl->build_cell;
    f.status = nl->status;
    return f;
}

// the gated build of a small list as one cooperative launch; FMB_ERR_UNSUPPORTED when the device cannot hold the grid
int build_small(const fmb_nl_t* nl, const double* positions, const int32_t* flag, cudaStream_t stream) {
    const size_t smem = (size_t)(kCoopThreads / 32) * FMB_MAX_ROW * sizeof(unsigned long long);
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_build_small, (int)smem));
    static int resident = 0;
    if (resident == 0) {
        int per_sm = 0, sms = 0, dev = 0, coop = 0;
        FMB_CUDA_CHECK(cudaGetDevice(&dev));
        FMB_CUDA_CHECK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        FMB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_build_small, kCoopThreads, smem) != cudaSuccess) per_sm = 0;
        resident = coop && per_sm > 0 ? per_sm * sms : -1;
    }
    if (resident < 0) return FMB_ERR_UNSUPPORTED;
    SmallBuildArgs a;
    a.c = make_const(nl);
    a.n = nl->n_atoms; a.capacity = nl->capacity; a.total_bins = nl->nbins[0] * nl->nbins[1] * nl->nbins[2];
    a.x = positions; a.wrapped = nl->wrapped; a.offsets = nl->offsets; a.atom_bin = nl->atom_bin;
    a.bin_count = nl->bin_count; a.bin_start = nl->bin_start; a.bin_fill = nl->bin_fill; a.bin_atoms = nl->bin_atoms;
    a.cand_row_count = nl->cand_row_count; a.cand_row_ptr = nl->cand_row_ptr;
    a.finish = finish_args(nl);
    a.flag = flag;
    // one warp per receiver in one pass where the device holds that many CTAs; never more than are resident together
    const int wanted = ceil_div(a.n, kCoopThreads / 32);
    const int grid = wanted < resident ? wanted : resident;
    void* args[] = {(void*)&a};
    FMB_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)k_build_small, dim3(grid), dim3(kCoopThreads), args, smem, stream));
    return FMB_OK;
}

}  // namespace
}  // namespace fmb

extern "C" FMB_API int fmb_nl_build(const fmb_nl_t* nl, const double* positions, int only_if_flag, fmb_stream_t stream_) {
    FMB_REQUIRE(nl && positions, "fmb_nl_build: null argument");
    FMB_REQUIRE(nl->n_atoms > 0 && nl->capacity > 0, "fmb_nl_build: empty list");
    for (int a = 0; a < 3; ++a)
        FMB_REQUIRE(nl->nbins[a] >= 1 && nl->reach_bins[a] >= 1 && nl->reach_bins[a] < 100, "fmb_nl_build: bad bins");
    cudaStream_t stream = (cudaStream_t)stream_;
    const NlConst c = make_const(nl);
    const int n = nl->n_atoms;
    const int total_bins = nl->nbins[0] * nl->nbins[1] * nl->nbins[2];
    const int32_t* flag = only_if_flag ? nl->rebuild_flag : nullptr;
    if (only_if_flag && n <= kSmallBuild && total_bins < kSmallBuild) {
        const int rc = build_small(nl, positions, flag, stream);
        if (rc != FMB_ERR_UNSUPPORTED) return rc;
    }
    k_zero_bins<<<ceil_div(total_bins + 1, 256), 256, 0, stream>>>(nl->bin_count, nl->bin_fill, total_bins, flag);
    FMB_LAUNCH_CHECK();
    k_wrap_bin<<<ceil_div(n, 256), 256, 0, stream>>>(c, n, positions, nl->wrapped, nl->offsets, nl->atom_bin,
                                                     nl->bin_count, flag);
    FMB_LAUNCH_CHECK();
    int rc = exclusive_scan(nl->bin_count, nl->bin_start, total_bins, nl->scan_scratch, flag, stream);
    if (rc) return rc;
    k_bin_fill<<<ceil_div(n, 256), 256, 0, stream>>>(n, nl->atom_bin, nl->bin_start, nl->bin_fill, nl->bin_atoms, flag);
    FMB_LAUNCH_CHECK();
    const int row_blocks = ceil_div(n, kWarpsPerBlock);
    k_rows<0><<<row_blocks, kWarpsPerBlock * 32, 0, stream>>>(c, n, nl->capacity, nl->wrapped, nl->offsets, nl->atom_bin,
                                                               nl->bin_start, nl->bin_atoms, nl->cand_row_count, nullptr,
                                                               nullptr, nullptr, nl->status, flag);
    FMB_LAUNCH_CHECK();
    rc = exclusive_scan(nl->cand_row_count, nl->cand_row_ptr, n, nl->scan_scratch, flag, stream);
    if (rc) return rc;
    const size_t smem = (size_t)kWarpsPerBlock * FMB_MAX_ROW * sizeof(unsigned long long);
    k_rows<1><<<row_blocks, kWarpsPerBlock * 32, smem, stream>>>(c, n, nl->capacity, nl->wrapped, nl->offsets,
                                                                  nl->atom_bin, nl->bin_start, nl->bin_atoms, nullptr,
                                                                  nl->cand_row_ptr, nl->candidate_index,
                                                                  nl->candidate_unit_shifts, nl->status, flag);
    FMB_LAUNCH_CHECK();
    k_finish_build<<<148 * 2, 256, 0, stream>>>(c, n, nl->capacity, nl->cand_row_ptr, positions, finish_args(nl), flag);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_nl_compact(const fmb_nl_t* nl, const double* positions, fmb_stream_t stream_) {
    FMB_REQUIRE(nl && positions, "fmb_nl_compact: null argument");
    cudaStream_t stream = (cudaStream_t)stream_;
    const NlConst c = make_const(nl);
    const int n = nl->n_atoms;
    const int row_blocks = ceil_div(n, kWarpsPerBlock);
    k_compact<0><<<row_blocks, kWarpsPerBlock * 32, 0, stream>>>(c, n, nl->capacity, positions, nl->cand_row_ptr,
                                                                  nl->candidate_index, nl->candidate_unit_shifts,
                                                                  nl->edge_row_count, nullptr, nullptr, nullptr, nullptr,
                                                                  nullptr);
    FMB_LAUNCH_CHECK();
    int rc = exclusive_scan(nl->edge_row_count, nl->edge_row_ptr, n, nl->scan_scratch, nullptr, stream);
    if (rc) return rc;
    k_compact<1><<<row_blocks, kWarpsPerBlock * 32, 0, stream>>>(c, n, nl->capacity, positions, nl->cand_row_ptr,
                                                                  nl->candidate_index, nl->candidate_unit_shifts, nullptr,
                                                                  nl->edge_row_ptr, nl->edge_index, nl->unit_shifts,
                                                                  nl->shifts, nl->count);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

extern "C" FMB_API int fmb_nl_needs_rebuild(const fmb_nl_t* nl, const double* positions, double fraction, fmb_stream_t stream_) {
    FMB_REQUIRE(nl && positions, "fmb_nl_needs_rebuild: null argument");
    cudaStream_t stream = (cudaStream_t)stream_;
    if (nl->n_atoms <= kSmallTestAtoms) {
        const double t = fraction * nl->skin / 2.0;
        k_rebuild_test_small<<<1, 1024, 0, stream>>>(nl->n_atoms, positions, nl->reference_positions, t * t,
                                                     (unsigned long long*)nl->max_disp2_bits, nl->rebuild_flag);
        FMB_LAUNCH_CHECK();
        return FMB_OK;
    }
    FMB_CUDA_CHECK(cudaMemsetAsync(nl->max_disp2_bits, 0, sizeof(uint64_t), stream));
    k_max_displacement<<<ceil_div(nl->n_atoms, 256), 256, 0, stream>>>(
        nl->n_atoms, positions, nl->reference_positions, (unsigned long long*)nl->max_disp2_bits);
    FMB_LAUNCH_CHECK();
    const double t = fraction * nl->skin / 2.0;
    k_rebuild_flag<<<1, 1, 0, stream>>>((const unsigned long long*)nl->max_disp2_bits, t * t, nl->rebuild_flag);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}
