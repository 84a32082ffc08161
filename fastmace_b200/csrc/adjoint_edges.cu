// Adjoint of the interactions with per-edge hand-over instead of the mirror evaluation (used when the edge list is a
// single chunk, so that per-edge buffers of the whole list fit).
//
// The mirror kernels (interaction.cu) make every receiver's CTA evaluate each of its edges twice -- as stored and in
// the opposite direction -- because that yields the sender-side gradient and the force without a scatter; the price is
// the gather of the mirror receiver's whole message-gradient row (20 KB per edge for the medium model), which makes
// that kernel L2-bandwidth bound. Here every directed edge is evaluated once, in its receiver's row, and hands over
//   * the gradient of its sender's features  dxe[e] = dE/dx_sender from this edge   ([IN][128] floats), and
//   * the gradient of its edge vector        qe[e]  = dE/dv_e                        (3 floats),
// and two light gather kernels finish the job through the mirror map e -> e' (the edge sender(e) <- receiver(e) with
// the opposite image; it exists because the neighbour list is full):
//   dE/dx_a = sum over the row of a of dxe[e'],      F_a = -(sum over the row of qe[e] - qe[e']),
//   virial_a = sum over the row of v_e (x) qe[e].
// Everything is summed in a fixed order; there are no atomics. Per edge the L2 traffic drops from 37 KB to about 14 KB
// and the coupling arithmetic halves.
//
// Replaces autograd through conv_tp + scatter_sum (fastmace/rewrites/generic/modules.py:485-486) like the mirror
// kernels; the reference's own edge-owned kernel scatters with atomicAdd (factorized_projected.cuh:258-353).

#include "stages.cuh"
#include "edge_gradient.cuh"
#include "tc_common.cuh"
#include "generated/tp_generated.cuh"

#include <cstdlib>

namespace fmb {

namespace {

template <int LIN, bool FLIP, bool NEED_DX> struct TpBackwardSel;
#define FMB_TP_BACKWARD_SEL(LIN_)                                                                                      \
    template <bool FLIP, bool NEED_DX> struct TpBackwardSel<LIN_, FLIP, NEED_DX> {                                     \
        template <typename... A> static __device__ __forceinline__ void run(A&&... a) {                               \
            tp_backward_##LIN_<FLIP, NEED_DX>(a...);                                                                   \
        }                                                                                                              \
    };
FMB_TP_BACKWARD_SEL(0)
FMB_TP_BACKWARD_SEL(1)
FMB_TP_BACKWARD_SEL(2)

constexpr int kBatch = 8;
constexpr int kAdjBatch = 16;          // edges between two CTA barriers of the streamed kernels (their 17 sums meet in shared memory)

// mirror[e] = index of the edge (sender = receiver(e), receiver = sender(e), image = -image(e)), or -1. With `slot`:
// the edges below *listed_below that stand for their pair (no opposite edge, or the lower index of the two) are listed
// in `list` and get the position as their slot (the order of the list depends on the atomics; the slots are only
// names of rows).
__global__ void k_mirror(const long long* __restrict__ count_ptr, int capacity, const int32_t* __restrict__ edge_index,
                         const float* __restrict__ unit_shifts, const int32_t* __restrict__ row_ptr,
                         int32_t* __restrict__ mirror, uint32_t* __restrict__ status,
                         const long long* __restrict__ listed_below, int32_t* __restrict__ slot,
                         int32_t* __restrict__ list, unsigned long long* __restrict__ list_count, int list_capacity) {
    const long long count = *count_ptr;
    const long long listed = slot ? *listed_below : 0;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (long long)gridDim.x * blockDim.x) {
        const int s = edge_index[e], r = edge_index[capacity + e];
        const float u0 = -unit_shifts[3 * e], u1 = -unit_shifts[3 * e + 1], u2 = -unit_shifts[3 * e + 2];
        // row s is sorted by (sender, image): first entry whose sender is >= r
        int lo = row_ptr[s], hi = row_ptr[s + 1];
        const int end = hi;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (edge_index[mid] < r) lo = mid + 1; else hi = mid;
        }
        int found = -1;
        for (int q = lo; q < end && edge_index[q] == r; ++q) {
            if (unit_shifts[3 * q] == u0 && unit_shifts[3 * q + 1] == u1 && unit_shifts[3 * q + 2] == u2) {
                found = q;
                break;
            }
        }
        mirror[e] = found;
        if (found < 0) atomicOr(status, FMB_STATUS_NO_MIRROR);
        if (slot && e < listed && (found < 0 || e < found)) {
            const unsigned long long k = atomicAdd(list_count, 1ull);
            if (k < (unsigned long long)list_capacity) {
                slot[e] = (int)k;
                list[k] = (int)e;
            } else {
                slot[e] = 0;                                   // a row that exists; the status word says it is wrong
                atomicOr(status, FMB_STATUS_PAIR_OVERFLOW);
            }
        }
    }
}

// Per-edge adjoint of the tensor product: CTA per receiver, thread per channel.
template <int LIN, int MINB>
__global__ void __launch_bounds__(kC, MINB)
k_tp_adjoint_edges(int n_atoms, int n_rows, int n_valid, long long chunk_e0, long long chunk_edges,
                   const long long* __restrict__ count_ptr, const int32_t* __restrict__ row_ptr,
                   const int32_t* __restrict__ senders, const float* __restrict__ x, const float* __restrict__ edge_sh,
                   const float* __restrict__ edge_vec, const float* __restrict__ tp_w, long long tangent_offset,
                   const float* __restrict__ d_mid, float* __restrict__ dxe, float4* __restrict__ qe) {
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    __shared__ float red[kBatch][4][18];
    const int c = threadIdx.x, warp = c >> 5, lane = c & 31;
    // this launch covers the edges [e0, e1) (a chunk of the list: tp_w holds their weights); a row that straddles two
    // chunks is simply visited by both, every edge is independent
    const long long count = *count_ptr;
    const long long e0 = chunk_e0, e1 = min(count, chunk_e0 + chunk_edges);
    if (e0 >= e1) return;
    int first = 0;
    if (e0 > 0) {
        int lo = 0, hi = n_atoms;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (row_ptr[mid + 1] > e0) hi = mid; else lo = mid + 1;
        }
        first = lo;
    }
    for (int a = first + blockIdx.x; a < n_rows; a += gridDim.x) {
        const long long rb = max((long long)row_ptr[a], e0), re = min((long long)row_ptr[a + 1], e1);
        if (rb >= e1) break;
        if (a >= n_valid) {
            // no message gradient on this receiver: its edges hand over zeros
            for (long long e = rb; e < re; ++e) {
#pragma unroll
                for (int k = 0; k < IN; ++k) dxe[(e * IN + k) * kC + c] = 0.0f;
                if (c == 0) qe[e] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            continue;
        }
        float g_a[MID];
#pragma unroll
        for (int k = 0; k < MID; ++k) g_a[k] = __ldg(d_mid + ((long long)a * MID + k) * kC + c);
        for (long long batch = rb; batch < re; batch += kBatch) {
            const int nb = (int)min((long long)kBatch, re - batch);
            for (int k = 0; k < nb; ++k) {
                const long long e = batch + k;
                const int j = senders[e];
                float Y[16], w[P], wp[P], x_j[IN], dY[16], dxj[IN];
                {
                    const float4* yp = reinterpret_cast<const float4*>(edge_sh + 16 * e);
                    const float4 y0 = __ldg(yp), y1 = __ldg(yp + 1), y2 = __ldg(yp + 2), y3 = __ldg(yp + 3);
                    Y[0] = y0.x; Y[1] = y0.y; Y[2] = y0.z; Y[3] = y0.w; Y[4] = y1.x; Y[5] = y1.y; Y[6] = y1.z; Y[7] = y1.w;
                    Y[8] = y2.x; Y[9] = y2.y; Y[10] = y2.z; Y[11] = y2.w; Y[12] = y3.x; Y[13] = y3.y; Y[14] = y3.z; Y[15] = y3.w;
                }
                const float* wr = tp_w + (e - chunk_e0) * (long long)(P * kC) + c;
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    w[p] = __ldg(wr + p * kC);
                    wp[p] = __ldg(wr + tangent_offset + p * kC);
                }
#pragma unroll
                for (int q = 0; q < IN; ++q) {
                    x_j[q] = __ldg(x + ((long long)j * IN + q) * kC + c);
                    dxj[q] = 0.0f;
                }
#pragma unroll
                for (int q = 0; q < 16; ++q) dY[q] = 0.0f;
                float dr = 0.0f;
                TpBackwardSel<LIN, false, true>::run(x_j, Y, w, wp, g_a, dY, dr, dxj);
#pragma unroll
                for (int q = 0; q < IN; ++q) dxe[(e * IN + q) * kC + c] = dxj[q];
                // 16 + 1 sums over the channels: transpose-reduce inside the warp, the four warps meet in shared memory
                {
#pragma unroll
                    for (int half = 8, bit = 16; half >= 1; half >>= 1, bit >>= 1) {
                        const bool upper = (lane & bit) != 0;
#pragma unroll
                        for (int i = 0; i < half; ++i) {
                            const float keep = upper ? dY[i + half] : dY[i];
                            const float send = upper ? dY[i] : dY[i + half];
                            dY[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                        }
                    }
                    dY[0] += __shfl_xor_sync(0xffffffffu, dY[0], 1);
                }
                dr = warp_sum(dr);
                if ((lane & 1) == 0) red[k][warp][lane >> 1] = dY[0];
                if (lane == 0) red[k][warp][16] = dr;
            }
            __syncthreads();
            if (c < nb) {
                const long long e = batch + c;
                float g[16];
#pragma unroll
                for (int q = 0; q < 16; ++q) g[q] = red[c][0][q] + red[c][1][q] + red[c][2][q] + red[c][3][q];
                const float drt = red[c][0][16] + red[c][1][16] + red[c][2][16] + red[c][3][16];
                const float4 uv = __ldg(reinterpret_cast<const float4*>(edge_vec) + e);
                float q3[3];
                edge_vector_gradient(g, drt, uv.x, uv.y, uv.z, uv.w, q3);
                qe[e] = make_float4(q3[0], q3[1], q3[2], 0.0f);
            }
            __syncthreads();
        }
    }
}

// The adjoint with every per-edge operand streamed through shared memory (whole edge list in one launch, every row
// carries a gradient) and two channels per thread on the packed FP32 pipe (fma.rn.f32x2, sm_100). The direct-load
// kernel above asks for an edge's 2 P C weights, its sender's rows and its harmonics when it gets to the edge and
// waits for them; its CTAs take whole rows (a tail of 14 % of the SM time on 1,944 atoms) and meet twice per eight
// edges. Here every CTA takes the same number of edges (an edge is independent of the others of its row), one thread
// keeps STAGES - 1 edges ahead of the consumers with bulk copies that complete on mbarriers -- per edge the weights,
// their d/dr, the sender's feature rows and the 16 harmonics -- a stage is handed back by one arrival per warp, and
// the CTA meets once per 16 edges. 64 threads per CTA: the per-channel operands, the row's message gradient and the
// partial sums are pairs. The scalar form issued 533 instructions per warp and edge for 32 channels and was bound by
// that; the pair form issues about as many for 64.
constexpr unsigned kAdjSpin = 1u << 20;

template <int LIN> struct TpBackwardPairSel;
#define FMB_TP_BACKWARD_PAIR_SEL(LIN_)                                                                                 \
    template <> struct TpBackwardPairSel<LIN_> {                                                                       \
        template <typename... A> static __device__ __forceinline__ void run(A&&... a) {                               \
            tp_backward_pair_##LIN_<false, true>(a...);                                                                \
        }                                                                                                              \
    };
FMB_TP_BACKWARD_PAIR_SEL(1)

constexpr int kPairThreads = kC / 2;

template <int LIN, int STAGES, int MINB>
__global__ void __launch_bounds__(kPairThreads, MINB)
k_tp_adjoint_pairs(int n_rows, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
                   const float* __restrict__ x, const float* __restrict__ edge_sh, const float* __restrict__ edge_vec,
                   const float* __restrict__ tp_w, long long tangent_offset, const float* __restrict__ d_mid,
                   float* __restrict__ dxe, float4* __restrict__ qe, uint32_t* __restrict__ error_word,
                   const int32_t* __restrict__ mirror, const int32_t* __restrict__ slot) {
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    constexpr int kW = P * kC;                              // floats of one edge's weights
    constexpr int kStage = 2 * kW + IN * kC + 16;           // weights, d/dr, sender rows, harmonics
    constexpr int kWarps = kPairThreads / 32;
    extern __shared__ __align__(128) float ring[];          // [STAGES][kStage]
    __shared__ uint64_t bars[2 * STAGES];
    __shared__ int abort_sh, first_row_sh;
    __shared__ float red[2][kAdjBatch][kWarps][18];
    volatile int* abort_flag = &abort_sh;
    const int c = threadIdx.x, warp = c >> 5, lane = c & 31;     // channels 2 c and 2 c + 1
    const long long total = row_ptr[n_rows];
    const long long per_cta = (total + gridDim.x - 1) / gridDim.x;
    const long long eb = (long long)blockIdx.x * per_cta, ee = min(total, eb + per_cta);
    if (eb >= ee) return;
    const uint32_t bar0 = tc::smem_u32(bars), ring0 = tc::smem_u32(ring);
    if (c == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(bar0 + 8 * s, 1);                        // full
            tc::mbar_init(bar0 + 8 * (STAGES + s), kWarps);        // empty: one arrival per warp
        }
        abort_sh = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    long long issued = eb;
    int issue_stage = 0;
    uint32_t issue_parity = 1;
    int next_sender = c == 0 ? senders[eb] : 0;
    // the row of tp_w that holds an edge's weights: its own, or with one row per pair of opposite edges the slot of
    // the lower edge of the pair
    auto row_of = [&](long long e) -> long long {
        if (!slot) return e;
        const int m = mirror[e];
        return slot[(m < 0 || e < m) ? e : (long long)m];
    };
    long long next_row = c == 0 ? row_of(eb) : 0;
    auto issue = [&]() {
        tc::mbar_wait(bar0 + 8 * (STAGES + issue_stage), issue_parity, abort_flag, kAdjSpin);
        const uint32_t full = bar0 + 8 * issue_stage;
        const uint32_t dst = ring0 + issue_stage * (kStage * 4);
        tc::mbar_expect_tx(full, kStage * 4);
        tc::bulk_load(dst, tp_w + next_row * kW, kW * 4, full);
        tc::bulk_load(dst + kW * 4, tp_w + tangent_offset + next_row * kW, kW * 4, full);
        tc::bulk_load(dst + 2 * kW * 4, x + (long long)next_sender * (IN * kC), IN * kC * 4, full);
        tc::bulk_load(dst + (2 * kW + IN * kC) * 4, edge_sh + 16 * issued, 64, full);
        ++issued;
        if (issued < ee) {
            next_sender = senders[issued];
            next_row = row_of(issued);
        }
        if (++issue_stage == STAGES) { issue_stage = 0; issue_parity ^= 1u; }
    };
    if (c == 0) {
        while (issued < ee && issued < eb + STAGES - 1) issue();
        int lo = 0, hi = n_rows - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (row_ptr[mid] <= eb) lo = mid; else hi = mid - 1;
        }
        first_row_sh = lo;
    }
    __syncthreads();
    int a = first_row_sh;
    long long row_end = row_ptr[a + 1];
    float2 g_a[MID];
#pragma unroll
    for (int k = 0; k < MID; ++k) g_a[k] = __ldg(reinterpret_cast<const float2*>(d_mid + ((long long)a * MID + k) * kC) + c);
    int stage = 0, buf = 0;
    uint32_t parity = 0;
    for (long long batch = eb; batch < ee; batch += kAdjBatch) {
        const int nb = (int)min((long long)kAdjBatch, ee - batch);
        for (int k = 0; k < nb; ++k) {
            const long long e = batch + k;
            if (e >= row_end) {
                do { ++a; row_end = row_ptr[a + 1]; } while (e >= row_end);
#pragma unroll
                for (int q = 0; q < MID; ++q)
                    g_a[q] = __ldg(reinterpret_cast<const float2*>(d_mid + ((long long)a * MID + q) * kC) + c);
            }
            if (c == 0 && issued < ee && issued < e + STAGES) issue();
            float Y[16];
            float2 w[P], wp[P], x_j[IN], dY2[16], dxj[IN];
            tc::mbar_wait(bar0 + 8 * stage, parity, abort_flag, kAdjSpin);
            {
                const float* st = ring + stage * kStage;
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    w[p] = reinterpret_cast<const float2*>(st + p * kC)[c];
                    wp[p] = reinterpret_cast<const float2*>(st + kW + p * kC)[c];
                }
#pragma unroll
                for (int q = 0; q < IN; ++q) {
                    x_j[q] = reinterpret_cast<const float2*>(st + 2 * kW + q * kC)[c];
                    dxj[q] = make_float2(0.0f, 0.0f);
                }
                const float4* yp = reinterpret_cast<const float4*>(st + 2 * kW + IN * kC);
                const float4 y0 = yp[0], y1 = yp[1], y2 = yp[2], y3 = yp[3];
                Y[0] = y0.x; Y[1] = y0.y; Y[2] = y0.z; Y[3] = y0.w; Y[4] = y1.x; Y[5] = y1.y; Y[6] = y1.z; Y[7] = y1.w;
                Y[8] = y2.x; Y[9] = y2.y; Y[10] = y2.z; Y[11] = y2.w; Y[12] = y3.x; Y[13] = y3.y; Y[14] = y3.z; Y[15] = y3.w;
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar0 + 8 * (STAGES + stage));
            if (++stage == STAGES) { stage = 0; parity ^= 1u; }
#pragma unroll
            for (int q = 0; q < 16; ++q) dY2[q] = make_float2(0.0f, 0.0f);
            float2 dr2 = make_float2(0.0f, 0.0f);
            TpBackwardPairSel<LIN>::run(x_j, Y, w, wp, g_a, dY2, dr2, dxj);
#pragma unroll
            for (int q = 0; q < IN; ++q) reinterpret_cast<float2*>(dxe + (e * IN + q) * kC)[c] = dxj[q];
            float dY[16];
#pragma unroll
            for (int q = 0; q < 16; ++q) dY[q] = dY2[q].x + dY2[q].y;
            float dr = dr2.x + dr2.y;
            {
#pragma unroll
                for (int half = 8, bit = 16; half >= 1; half >>= 1, bit >>= 1) {
                    const bool upper = (lane & bit) != 0;
#pragma unroll
                    for (int i = 0; i < half; ++i) {
                        const float keep = upper ? dY[i + half] : dY[i];
                        const float send = upper ? dY[i] : dY[i + half];
                        dY[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                    }
                }
                dY[0] += __shfl_xor_sync(0xffffffffu, dY[0], 1);
            }
            dr = warp_sum(dr);
            if ((lane & 1) == 0) red[buf][k][warp][lane >> 1] = dY[0];
            if (lane == 0) red[buf][k][warp][16] = dr;
        }
        __syncthreads();
        if (c < nb) {
            const long long e = batch + c;
            float g[16];
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                g[q] = red[buf][c][0][q];
#pragma unroll
                for (int ww = 1; ww < kWarps; ++ww) g[q] += red[buf][c][ww][q];
            }
            float drt = red[buf][c][0][16];
#pragma unroll
            for (int ww = 1; ww < kWarps; ++ww) drt += red[buf][c][ww][16];
            const float4 uv = __ldg(reinterpret_cast<const float4*>(edge_vec) + e);
            float q3[3];
            edge_vector_gradient(g, drt, uv.x, uv.y, uv.z, uv.w, q3);
            qe[e] = make_float4(q3[0], q3[1], q3[2], 0.0f);
        }
        buf ^= 1;
    }
    __syncthreads();
    if (c == 0 && abort_sh && error_word) atomicOr(error_word, FMB_STATUS_TENSOR_TIMEOUT);
}

// dE/dx_a = sum over the row of a of the hand-over of the mirror edges (rows at or beyond n_source hand over nothing)
template <int IN>
__global__ void __launch_bounds__(kC)
k_gather_dx(int n_rows, int n_source, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
            const int32_t* __restrict__ mirror, const float* __restrict__ dxe, float* __restrict__ d_x) {
    const int c = threadIdx.x;
    for (int a = blockIdx.x; a < n_rows; a += gridDim.x) {
        float acc[IN];
#pragma unroll
        for (int k = 0; k < IN; ++k) acc[k] = 0.0f;
        const long long rb = row_ptr[a], re = row_ptr[a + 1];
        // four edges at a time: their mirror indices first, then all the rows, so that the loads overlap
        for (long long e = rb; e < re; e += 4) {
            int m[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const bool live = e + q < re;
                m[q] = live ? mirror[e + q] : -1;
                if (live && senders[e + q] >= n_source) m[q] = -1;
            }
            float v[4][IN];
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int k = 0; k < IN; ++k)
                    v[q][k] = m[q] >= 0 ? __ldg(dxe + ((long long)m[q] * IN + k) * kC + c) : 0.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int k = 0; k < IN; ++k) acc[k] += v[q][k];
        }
#pragma unroll
        for (int k = 0; k < IN; ++k) d_x[((long long)a * IN + k) * kC + c] = acc[k];
    }
}

// First interaction (reassociated form), per edge: the receiver's gradient block [16][Z][64] in shared memory,
// dE/dY[lm] = sum_k dS[lm, z_j, k] hidden[k], dE/dr = sum_k hidden'[k] sum_lm dS[lm, z_j, k] Y[lm]; the edge-vector
// gradient is added to qe (rows below n_add, which the later interaction wrote) or stored. A thread takes an edge and
// four harmonics: the sums over the 64 radial features run inside the thread -- the features of 16 edges are staged in
// shared memory -- and only the four threads of an edge meet at the end, by shuffles inside a group of four lanes. (A
// thread per (feature, eight harmonics) spent 137 instructions per warp and edge on 16 FMAs per thread: channel
// reductions by shuffle and two barriers per eight edges; 72 -> 45 us.)
constexpr int kFaPass = 16;                       // edges per pass
constexpr int kFaThreads = 4 * kFaPass;
constexpr int kFaLd = kRadial + 1;                // row stride of the staged features (conflict-free across edges)

__global__ void __launch_bounds__(kFaThreads)
k_first_adjoint_rows(int n_rows, int n_valid, int n_add, int n_species, const int32_t* __restrict__ row_ptr,
                     const int32_t* __restrict__ senders, const int32_t* __restrict__ species,
                     const float* __restrict__ edge_sh, const float* __restrict__ edge_vec,
                     const float* __restrict__ hidden, const float* __restrict__ hidden_tangent,
                     const float* __restrict__ d_s, float4* __restrict__ qe) {
    __shared__ float hs[kFaPass][kFaLd], hps[kFaPass][kFaLd];
    extern __shared__ float own[];                        // [16][n_species][kFaLd]: the four harmonics groups and the
                                                          // species of a warp's edges fall into different banks
    const int c = threadIdx.x, slot = c >> 2, grp = c & 3, lane = c & 31;
    const long long row_floats = (long long)kNSH * n_species * kRadial;
    const int lm_stride = n_species * kFaLd;
    for (int a = blockIdx.x; a < n_rows; a += gridDim.x) {
        const long long rb = row_ptr[a], re = row_ptr[a + 1];
        if (a >= n_valid) {
            if (a >= n_add)
                for (long long e = rb + c; e < re; e += kFaThreads) qe[e] = make_float4(0.f, 0.f, 0.f, 0.f);
            continue;
        }
        __syncthreads();                                  // the previous row's block is no longer read
        for (int q = c; q < (int)row_floats; q += kFaThreads) own[(q >> 6) * kFaLd + (q & 63)] = __ldg(d_s + a * row_floats + q);
        for (long long batch = rb; batch < re; batch += kFaPass) {
            const int nb = (int)min((long long)kFaPass, re - batch);
            __syncthreads();                              // the previous pass is done with the staged features
            for (int q = c; q < nb * kRadial; q += kFaThreads) {
                const int el = q >> 6, k = q & 63;
                hs[el][k] = __ldg(hidden + (batch + el) * kRadial + k);
                hps[el][k] = __ldg(hidden_tangent + (batch + el) * kRadial + k);
            }
            __syncthreads();
            const bool live = slot < nb;
            const long long e = batch + (live ? slot : 0);
            float g[4] = {0.f, 0.f, 0.f, 0.f}, dr = 0.0f;
            if (live) {
                const int zj = species[senders[e]];
                const float4 y = __ldg(reinterpret_cast<const float4*>(edge_sh + 16 * e) + grp);
                const float* ds = own + (4 * grp * n_species + zj) * kFaLd;       // harmonics 4 grp .. 4 grp + 3
#pragma unroll 8
                for (int k = 0; k < kRadial; ++k) {
                    const float h = hs[slot][k], hp = hps[slot][k];
                    const float d0 = ds[k], d1 = ds[lm_stride + k], d2 = ds[2 * lm_stride + k], d3 = ds[3 * lm_stride + k];
                    g[0] = fmaf(d0, h, g[0]); g[1] = fmaf(d1, h, g[1]); g[2] = fmaf(d2, h, g[2]); g[3] = fmaf(d3, h, g[3]);
                    const float dh = fmaf(d0, y.x, fmaf(d1, y.y, fmaf(d2, y.z, d3 * y.w)));
                    dr = fmaf(dh, hp, dr);
                }
            }
            // the four threads of an edge exchange their harmonics' gradients and add up the radial one
            float all[16];
            const int base = lane & ~3;
#pragma unroll
            for (int src = 0; src < 4; ++src)
#pragma unroll
                for (int i = 0; i < 4; ++i) all[4 * src + i] = __shfl_sync(0xffffffffu, g[i], base + src);
            dr += __shfl_xor_sync(0xffffffffu, dr, 1);
            dr += __shfl_xor_sync(0xffffffffu, dr, 2);
            if (live && grp == 0) {
                const float4 uv = __ldg(reinterpret_cast<const float4*>(edge_vec) + e);
                float q3[3];
                edge_vector_gradient(all, dr, uv.x, uv.y, uv.z, uv.w, q3);
                float4 out = make_float4(q3[0], q3[1], q3[2], 0.0f);
                if (a < n_add) {
                    const float4 old = qe[e];
                    out.x += old.x; out.y += old.y; out.z += old.z;
                }
                qe[e] = out;
            }
        }
    }
}

// F_a = -(sum_row qe[e] - qe[mirror e]), virial_a = sum_row v_e (x) qe[e]; one warp per atom, lanes over its edges,
// folded with a fixed butterfly. RESTRICT: only the edges into atoms below n_valid carry a gradient -- an atom at or
// beyond it (a halo atom) has no row terms and no virial, and a mirror edge counts only if its receiver (this edge's
// sender) is below n_valid; qe and edge_vec are never read elsewhere.
template <bool RESTRICT>
__global__ void __launch_bounds__(256)
k_force_gather(int n_atoms, int n_valid, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
               const int32_t* __restrict__ mirror, const float4* __restrict__ qe, const float* __restrict__ edge_vec,
               float* __restrict__ force_acc, float* __restrict__ atom_virial) {
    const int a = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (a >= n_atoms) return;
    float f[3] = {0.f, 0.f, 0.f}, vir[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const bool own = !RESTRICT || a < n_valid;
    for (long long e = row_ptr[a] + lane; e < row_ptr[a + 1]; e += 32) {
        const float4 q = own ? qe[e] : make_float4(0.f, 0.f, 0.f, 0.f);
        int m = mirror[e];
        if (RESTRICT && senders[e] >= n_valid) m = -1;
        const float4 qm = m >= 0 ? qe[m] : make_float4(0.f, 0.f, 0.f, 0.f);
        f[0] += q.x - qm.x; f[1] += q.y - qm.y; f[2] += q.z - qm.z;
        if (own) {
            const float4 uv = __ldg(reinterpret_cast<const float4*>(edge_vec) + e);
            const float vx = uv.x * uv.w, vy = uv.y * uv.w, vz = uv.z * uv.w;
            vir[0] += vx * q.x; vir[1] += vy * q.y; vir[2] += vz * q.z;
            vir[3] += 0.5f * (vy * q.z + vz * q.y);
            vir[4] += 0.5f * (vx * q.z + vz * q.x);
            vir[5] += 0.5f * (vx * q.y + vy * q.x);
        }
    }
#pragma unroll
    for (int q = 0; q < 3; ++q) f[q] = warp_sum(f[q]);
#pragma unroll
    for (int q = 0; q < 6; ++q) vir[q] = warp_sum(vir[q]);
    if (lane == 0) {
#pragma unroll
        for (int q = 0; q < 3; ++q) force_acc[3 * (long long)a + q] = f[q];
#pragma unroll
        for (int q = 0; q < 6; ++q) atom_virial[6 * (long long)a + q] = vir[q];
    }
}

int grid_for(const void* kernel, int rows, int threads, size_t smem) {
    int per_sm = 0, sms = 148, dev = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int cap = per_sm * sms * 4;
    return rows < cap ? rows : cap;
}

}  // namespace

int mirror_map(const fmb_nl_t* nl, int32_t* mirror, uint32_t* status, const long long* listed_below, int32_t* slot,
               int32_t* list, long long* list_count, int list_capacity, cudaStream_t stream) {
    const int blocks = ceil_div(nl->capacity, 256);
    if (slot) FMB_CUDA_CHECK(cudaMemsetAsync(list_count, 0, sizeof(long long), stream));
    k_mirror<<<blocks < 1184 ? blocks : 1184, 256, 0, stream>>>((const long long*)nl->count, nl->capacity, nl->edge_index,
                                                               nl->unit_shifts, nl->edge_row_ptr, mirror, status,
                                                               listed_below, slot, list, (unsigned long long*)list_count,
                                                               list_capacity);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int tp_adjoint_edges(const EdgeAdjointArgs& t, cudaStream_t stream) {
    if (t.n_rows <= 0) return FMB_OK;
    if (t.lin == 0) {
        static const int grid_cap = grid_for((const void*)k_tp_adjoint_edges<0, 2>, 1 << 30, kC, 0);
        k_tp_adjoint_edges<0, 2><<<t.n_rows < grid_cap ? t.n_rows : grid_cap, kC, 0, stream>>>(
            t.n_atoms, t.n_rows, t.n_valid, t.chunk_e0, t.chunk_edges, t.count, t.row_ptr, t.senders, t.x, t.edge_sh, t.edge_vec,
            t.tp_w, t.tangent_offset, t.d_mid, t.dxe,
            reinterpret_cast<float4*>(t.qe));
    } else if (t.lin == 1 && t.whole_list && t.n_valid >= t.n_rows && t.chunk_e0 == 0) {
        constexpr int kStages = 3, kMinB = 4;      // measured best of 2 .. 6 stages at 2 .. 4 CTAs per SM
        constexpr int smem = kStages * (2 * TpShape<1>::kPaths * kC + TpShape<1>::kInDim * kC + 16) * 4;
        auto kernel = k_tp_adjoint_pairs<1, kStages, kMinB>;
        FMB_CUDA_CHECK(opt_in_shared_memory((const void*)kernel, smem));
        static int grid_cap = 0;
        if (grid_cap == 0) {
            int per_sm = 0, sms = 148, dev = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kPairThreads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            grid_cap = per_sm * sms;
        }
        kernel<<<grid_cap, kPairThreads, smem, stream>>>(
            t.n_rows, t.row_ptr, t.senders, t.x, t.edge_sh, t.edge_vec, t.tp_w, t.tangent_offset, t.d_mid, t.dxe,
            reinterpret_cast<float4*>(t.qe), t.error_word, t.mirror, t.slot);
    } else if (t.lin == 1) {
        // four CTAs per SM (127 registers): measured best on the 1,944-atom cell among 2 .. 6
        static const int grid_cap = grid_for((const void*)k_tp_adjoint_edges<1, 4>, 1 << 30, kC, 0);
        k_tp_adjoint_edges<1, 4><<<t.n_rows < grid_cap ? t.n_rows : grid_cap, kC, 0, stream>>>(
            t.n_atoms, t.n_rows, t.n_valid, t.chunk_e0, t.chunk_edges, t.count, t.row_ptr, t.senders, t.x, t.edge_sh,
            t.edge_vec, t.tp_w, t.tangent_offset, t.d_mid, t.dxe, reinterpret_cast<float4*>(t.qe));
    } else if (t.lin == 2) {
        static const int grid_cap = grid_for((const void*)k_tp_adjoint_edges<2, 2>, 1 << 30, kC, 0);
        k_tp_adjoint_edges<2, 2><<<t.n_rows < grid_cap ? t.n_rows : grid_cap, kC, 0, stream>>>(
            t.n_atoms, t.n_rows, t.n_valid, t.chunk_e0, t.chunk_edges, t.count, t.row_ptr, t.senders, t.x, t.edge_sh, t.edge_vec,
            t.tp_w, t.tangent_offset, t.d_mid, t.dxe,
            reinterpret_cast<float4*>(t.qe));
    } else {
        return FMB_ERR_UNSUPPORTED;
    }
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int gather_sender_gradient(const EdgeAdjointArgs& t, cudaStream_t stream) {
    const int rows = t.n_gather > 0 ? t.n_gather : t.n_rows;     // atoms that collect; the edges of [0, n_rows) hand over
    if (rows <= 0) return FMB_OK;
    const int in_dim = (t.lin + 1) * (t.lin + 1);
    const int grid = rows < 1184 ? rows : 1184;
    if (in_dim == 1) {
        k_gather_dx<1><<<grid, kC, 0, stream>>>(rows, t.n_rows, t.row_ptr, t.senders, t.mirror, t.dxe, t.d_x);
    } else if (in_dim == 4) {
        k_gather_dx<4><<<grid, kC, 0, stream>>>(rows, t.n_rows, t.row_ptr, t.senders, t.mirror, t.dxe, t.d_x);
    } else if (in_dim == 9) {
        k_gather_dx<9><<<grid, kC, 0, stream>>>(rows, t.n_rows, t.row_ptr, t.senders, t.mirror, t.dxe, t.d_x);
    } else {
        return FMB_ERR_UNSUPPORTED;
    }
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int first_adjoint_edges(const FirstArgs& f, int n_add, float* qe, cudaStream_t stream) {
    if (f.n_rows <= 0) return FMB_OK;
    const size_t smem = (size_t)f.n_species * kNSH * kFaLd * sizeof(float);
    static int grid_cap = 0;
    if (grid_cap == 0) grid_cap = grid_for((const void*)k_first_adjoint_rows, 1 << 30, kFaThreads, smem);
    k_first_adjoint_rows<<<f.n_rows < grid_cap ? f.n_rows : grid_cap, kFaThreads, smem, stream>>>(
        f.n_rows, f.n_valid, n_add, f.n_species, f.row_ptr, f.senders, f.species, f.edge_sh, f.edge_vec, f.hidden,
        f.hidden_tangent, f.d_s, reinterpret_cast<float4*>(qe));
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int force_gather(int n_atoms, int n_valid, const int32_t* row_ptr, const int32_t* senders, const int32_t* mirror,
                 const float* qe, const float* edge_vec, float* force_acc, float* atom_virial, cudaStream_t stream) {
    if (n_atoms <= 0) return FMB_OK;
    if (n_valid < n_atoms)
        k_force_gather<true><<<ceil_div(n_atoms, 8), 256, 0, stream>>>(n_atoms, n_valid, row_ptr, senders, mirror,
                                                                       reinterpret_cast<const float4*>(qe), edge_vec,
                                                                       force_acc, atom_virial);
    else
        k_force_gather<false><<<ceil_div(n_atoms, 8), 256, 0, stream>>>(n_atoms, n_valid, row_ptr, senders, mirror,
                                                                        reinterpret_cast<const float4*>(qe), edge_vec,
                                                                        force_acc, atom_virial);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace fmb
