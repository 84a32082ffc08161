// Channelwise equivariant tensor product fused with the receiver-sorted segmented sum, and its analytic adjoint.
//
// Forward (replaces conv_tp + scatter_sum, fastmace/rewrites/generic/modules.py:485-486, and the receiver-streaming
// kernel fastmace/kernels/oeq_streaming/factorized_projected.cuh:128-186): one CTA of 128 threads (one per channel)
// owns a receiver, walks its CSR edges, keeps the whole message row in registers and writes it once. No atomics.
//
// Backward (replaces autograd through conv_tp and the edge-owned kernel factorized_projected.cuh:258-353, which
// scatters the sender gradient with atomicAdd): the neighbour list is full, so every edge j -> a has a mirror
// a -> j with the opposite vector, the same length (hence the same radial weights) and harmonics (-1)^l Y_lm.
// The CTA that owns atom a therefore evaluates, for each edge j -> a of its row,
//   * the edge as stored   (receiver a: own message gradient g_a, gathered sender features x_j), and
//   * its mirror a -> j    (receiver j: gathered g_j, own features x_a),
// which yields dE/dY and dE/dr of both edges summed (the force on a is minus the sum over its row of the combined
// edge-vector gradient) and the complete gradient of x_a -- all owned by this CTA, so nothing is scattered.
// The virial is half the sum over rows of v (x) q because every edge is visited in both roles.

#include "stages.cuh"
#include "generated/tp_generated.cuh"
#include "edge_gradient.cuh"
#include "tc_common.cuh"

#include <cstdlib>
#include <map>

namespace fmb {

namespace {

template <int LIN, bool FLIP, bool NEED_DX> struct TpBackward;
#define FMB_TP_BACKWARD(LIN_)                                                                                          \
    template <bool FLIP, bool NEED_DX> struct TpBackward<LIN_, FLIP, NEED_DX> {                                        \
        template <typename... A> static __device__ __forceinline__ void run(A&&... a) {                               \
            tp_backward_##LIN_<FLIP, NEED_DX>(a...);                                                                   \
        }                                                                                                              \
    };
FMB_TP_BACKWARD(0)
FMB_TP_BACKWARD(1)
FMB_TP_BACKWARD(2)

// First row a chunk starting at edge e0 has to visit: the smallest r whose edges reach beyond e0 or start at or after
// it (rows finished by earlier chunks are skipped; empty rows are initialised by the chunk their offset falls in).
__device__ __forceinline__ int chunk_first_row(const int32_t* __restrict__ row_ptr, int n, long long e0) {
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_ptr[mid + 1] > e0 || row_ptr[mid] >= e0) hi = mid; else lo = mid + 1;
    }
    return lo;
}

__device__ __forceinline__ void load_sh(const float* __restrict__ edge_sh, long long e, float (&Y)[16]) {
    const float4* p = reinterpret_cast<const float4*>(edge_sh + 16 * e);
    const float4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2), d = __ldg(p + 3);
    Y[0] = a.x; Y[1] = a.y; Y[2] = a.z; Y[3] = a.w; Y[4] = b.x; Y[5] = b.y; Y[6] = b.z; Y[7] = b.w;
    Y[8] = c.x; Y[9] = c.y; Y[10] = c.z; Y[11] = c.w; Y[12] = d.x; Y[13] = d.y; Y[14] = d.z; Y[15] = d.w;
}

// ---------------------------------------------------------------------------------------------- forward
template <int LIN, bool SPECIES_X>
__global__ void __launch_bounds__(kC)
k_tp_forward(int n_atoms, int n_rows, long long chunk_e0, long long chunk_edges, const long long* __restrict__ count_ptr,
             const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
             const int32_t* __restrict__ species, const float* __restrict__ x, const float* __restrict__ edge_sh,
             const float* __restrict__ tp_w, float* __restrict__ mid) {
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    const long long count = *count_ptr;
    const long long e0 = chunk_e0, e1 = min(count, chunk_e0 + chunk_edges);
    if (e0 >= e1 && !(e0 == 0 && count == 0)) return;
    const int c = threadIdx.x;
    const int first = (e0 == 0) ? 0 : chunk_first_row(row_ptr, n_atoms, e0);
    for (int i = first + blockIdx.x; i < n_rows; i += gridDim.x) {
        const long long rb = row_ptr[i], re = row_ptr[i + 1];
        if (rb >= e1 && e1 < count) break;   // rows of later chunks (the last chunk also zeroes trailing empty rows)
        float acc[MID];
        float* out = mid + ((long long)i * MID) * kC + c;
        if (rb < e0) {
#pragma unroll
            for (int k = 0; k < MID; ++k) acc[k] = out[(long long)k * kC];   // continue a row split by the chunking
        } else {
#pragma unroll
            for (int k = 0; k < MID; ++k) acc[k] = 0.0f;
        }
        const long long b = max(rb, e0), en = min(re, e1);
        // unrolled so that the loads of several edges are in flight together (the loop is bound by their latency)
#pragma unroll 4
        for (long long e = b; e < en; ++e) {
            const int s = senders[e];
            float xs[IN], Y[16], w[P];
            if (SPECIES_X) {
                xs[0] = __ldg(x + (long long)species[s] * kC + c);
            } else {
#pragma unroll
                for (int k = 0; k < IN; ++k) xs[k] = __ldg(x + ((long long)s * IN + k) * kC + c);
            }
            load_sh(edge_sh, e, Y);
            const float* wr = tp_w + (e - chunk_e0) * (long long)(P * kC) + c;
#pragma unroll
            for (int p = 0; p < P; ++p) w[p] = __ldg(wr + p * kC);
            tp_forward<LIN>(xs, Y, w, acc);
        }
#pragma unroll
        for (int k = 0; k < MID; ++k) out[(long long)k * kC] = acc[k];
    }
}

// The same forward pass with every per-edge operand streamed through shared memory (whole edge list in one chunk):
// the direct-load kernel above spends its time waiting for the 4 P C bytes of weights per edge, which come from HBM
// (long-scoreboard stalls: 8.6 per issued instruction), and the sender's rows. Here a CTA owns a contiguous block of
// receivers, so its edges are one contiguous range, and one thread keeps kFwdStages - 1 edges ahead of the consumers
// with bulk copies that complete on mbarriers: per edge the weights, the sender's feature rows and the 16 harmonics.
// A stage is handed back by one arrival per warp.
constexpr int kFwdStages = 5;
constexpr unsigned kFwdSpin = 1u << 20;

template <int LIN>
__global__ void __launch_bounds__(kC)
k_tp_forward_stream(int n_rows, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
                    const float* __restrict__ x, const float* __restrict__ edge_sh, const float* __restrict__ tp_w,
                    float* __restrict__ mid, uint32_t* __restrict__ error_word) {
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    constexpr int kRow = P * kC;                       // floats of one edge's weights
    constexpr int kStage = kRow + IN * kC + 16;        // weights, sender rows, harmonics
    extern __shared__ __align__(128) float ring[];     // [kFwdStages][kStage]
    __shared__ uint64_t bars[2 * kFwdStages];
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;
    const int c = threadIdx.x, lane = c & 31;
    // contiguous blocks of receivers that differ by at most one row, so that every CTA of the grid has work
    const int r0 = (int)((long long)blockIdx.x * n_rows / gridDim.x), r1 = (int)((long long)(blockIdx.x + 1) * n_rows / gridDim.x);
    if (r0 >= r1) return;
    const long long eb = row_ptr[r0], ee = row_ptr[r1];
    const uint32_t bar0 = tc::smem_u32(bars), ring0 = tc::smem_u32(ring);
    if (c == 0) {
        for (int s = 0; s < kFwdStages; ++s) {
            tc::mbar_init(bar0 + 8 * s, 1);                        // full
            tc::mbar_init(bar0 + 8 * (kFwdStages + s), 4);         // empty: one arrival per warp
        }
        abort_sh = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // thread 0: next edge to request, its stage and the parity its `empty` barrier must have passed; the sender index
    // is read one request ahead so that its latency is not on the path
    long long issued = eb;
    int issue_stage = 0;
    uint32_t issue_parity = 1;
    int next_sender = (c == 0 && eb < ee) ? senders[eb] : 0;
    auto issue = [&]() {
        tc::mbar_wait(bar0 + 8 * (kFwdStages + issue_stage), issue_parity, abort_flag, kFwdSpin);
        const uint32_t full = bar0 + 8 * issue_stage;
        const uint32_t dst = ring0 + issue_stage * (kStage * 4);
        tc::mbar_expect_tx(full, kStage * 4);
        tc::bulk_load(dst, tp_w + issued * kRow, kRow * 4, full);
        tc::bulk_load(dst + kRow * 4, x + (long long)next_sender * (IN * kC), IN * kC * 4, full);
        tc::bulk_load(dst + (kRow + IN * kC) * 4, edge_sh + 16 * issued, 64, full);
        ++issued;
        if (issued < ee) next_sender = senders[issued];
        if (++issue_stage == kFwdStages) { issue_stage = 0; issue_parity ^= 1u; }
    };
    if (c == 0)
        while (issued < ee && issued < eb + kFwdStages - 1) issue();
    int stage = 0;
    uint32_t parity = 0;
    for (int i = r0; i < r1; ++i) {
        const long long rb = row_ptr[i], re = row_ptr[i + 1];
        float acc[MID];
#pragma unroll
        for (int k = 0; k < MID; ++k) acc[k] = 0.0f;
        for (long long e = rb; e < re; ++e) {
            // the stage the previous edge used has been handed back by now: refill it
            if (c == 0 && issued < ee && issued < e + kFwdStages) issue();
            float xs[IN], Y[16], w[P];
            tc::mbar_wait(bar0 + 8 * stage, parity, abort_flag, kFwdSpin);
            const float* st = ring + stage * kStage;
#pragma unroll
            for (int p = 0; p < P; ++p) w[p] = st[p * kC + c];
#pragma unroll
            for (int k = 0; k < IN; ++k) xs[k] = st[kRow + k * kC + c];
            {
                const float4* yp = reinterpret_cast<const float4*>(st + kRow + IN * kC);
                const float4 y0 = yp[0], y1 = yp[1], y2 = yp[2], y3 = yp[3];
                Y[0] = y0.x; Y[1] = y0.y; Y[2] = y0.z; Y[3] = y0.w; Y[4] = y1.x; Y[5] = y1.y; Y[6] = y1.z; Y[7] = y1.w;
                Y[8] = y2.x; Y[9] = y2.y; Y[10] = y2.z; Y[11] = y2.w; Y[12] = y3.x; Y[13] = y3.y; Y[14] = y3.z; Y[15] = y3.w;
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar0 + 8 * (kFwdStages + stage));
            if (++stage == kFwdStages) { stage = 0; parity ^= 1u; }
            tp_forward<LIN>(xs, Y, w, acc);
        }
        float* out = mid + ((long long)i * MID) * kC + c;
#pragma unroll
        for (int k = 0; k < MID; ++k) out[(long long)k * kC] = acc[k];
    }
    __syncthreads();
    if (c == 0 && abort_sh && error_word) atomicOr(error_word, FMB_STATUS_TENSOR_TIMEOUT);
}

// The streamed forward pass with two channels per thread on the packed FP32 pipe (fma.rn.f32x2, sm_100): 64 threads
// per CTA, the per-channel operands and the message row as pairs, a harmonic times its coupling coefficient as one
// scalar product shared by the pair. The kernel above is bound by FP32 issue (260 instructions per warp and edge for 32
// channels); the pair form issues about as many for 64.
constexpr int kPairThreads = kC / 2;

template <int LIN>
__global__ void __launch_bounds__(kPairThreads)
k_tp_forward_pairs(int n_rows, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
                   const float* __restrict__ x, const float* __restrict__ edge_sh, const float* __restrict__ tp_w,
                   float* __restrict__ mid, uint32_t* __restrict__ error_word, const int32_t* __restrict__ mirror,
                   const int32_t* __restrict__ slot) {
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    constexpr int kRow = P * kC;                       // floats of one edge's weights
    constexpr int kStage = kRow + IN * kC + 16;        // weights, sender rows, harmonics
    extern __shared__ __align__(128) float ring[];     // [kFwdStages][kStage]
    __shared__ uint64_t bars[2 * kFwdStages];
    __shared__ int abort_sh;
    volatile int* abort_flag = &abort_sh;
    const int c = threadIdx.x, lane = c & 31;          // channels 2 c and 2 c + 1
    // contiguous blocks of receivers that differ by at most one row, so that every CTA of the grid has work
    const int r0 = (int)((long long)blockIdx.x * n_rows / gridDim.x), r1 = (int)((long long)(blockIdx.x + 1) * n_rows / gridDim.x);
    if (r0 >= r1) return;
    const long long eb = row_ptr[r0], ee = row_ptr[r1];
    const uint32_t bar0 = tc::smem_u32(bars), ring0 = tc::smem_u32(ring);
    if (c == 0) {
        for (int s = 0; s < kFwdStages; ++s) {
            tc::mbar_init(bar0 + 8 * s, 1);                                  // full
            tc::mbar_init(bar0 + 8 * (kFwdStages + s), kPairThreads / 32);   // empty: one arrival per warp
        }
        abort_sh = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    long long issued = eb;
    int issue_stage = 0;
    uint32_t issue_parity = 1;
    int next_sender = (c == 0 && eb < ee) ? senders[eb] : 0;
    // the row of tp_w that holds an edge's weights: its own, or with one row per pair of opposite edges the slot of
    // the lower edge of the pair
    auto row_of = [&](long long e) -> long long {
        if (!slot) return e;
        const int m = mirror[e];
        return slot[(m < 0 || e < m) ? e : (long long)m];
    };
    long long next_row = (c == 0 && eb < ee) ? row_of(eb) : 0;
    auto issue = [&]() {
        tc::mbar_wait(bar0 + 8 * (kFwdStages + issue_stage), issue_parity, abort_flag, kFwdSpin);
        const uint32_t full = bar0 + 8 * issue_stage;
        const uint32_t dst = ring0 + issue_stage * (kStage * 4);
        tc::mbar_expect_tx(full, kStage * 4);
        tc::bulk_load(dst, tp_w + next_row * kRow, kRow * 4, full);
        tc::bulk_load(dst + kRow * 4, x + (long long)next_sender * (IN * kC), IN * kC * 4, full);
        tc::bulk_load(dst + (kRow + IN * kC) * 4, edge_sh + 16 * issued, 64, full);
        ++issued;
        if (issued < ee) {
            next_sender = senders[issued];
            next_row = row_of(issued);
        }
        if (++issue_stage == kFwdStages) { issue_stage = 0; issue_parity ^= 1u; }
    };
    if (c == 0)
        while (issued < ee && issued < eb + kFwdStages - 1) issue();
    int stage = 0;
    uint32_t parity = 0;
    for (int i = r0; i < r1; ++i) {
        const long long rb = row_ptr[i], re = row_ptr[i + 1];
        float2 acc[MID];
#pragma unroll
        for (int k = 0; k < MID; ++k) acc[k] = make_float2(0.0f, 0.0f);
        for (long long e = rb; e < re; ++e) {
            if (c == 0 && issued < ee && issued < e + kFwdStages) issue();
            float2 xs[IN], w[P];
            float Y[16];
            tc::mbar_wait(bar0 + 8 * stage, parity, abort_flag, kFwdSpin);
            const float* st = ring + stage * kStage;
#pragma unroll
            for (int p = 0; p < P; ++p) w[p] = reinterpret_cast<const float2*>(st + p * kC)[c];
#pragma unroll
            for (int k = 0; k < IN; ++k) xs[k] = reinterpret_cast<const float2*>(st + kRow + k * kC)[c];
            {
                const float4* yp = reinterpret_cast<const float4*>(st + kRow + IN * kC);
                const float4 y0 = yp[0], y1 = yp[1], y2 = yp[2], y3 = yp[3];
                Y[0] = y0.x; Y[1] = y0.y; Y[2] = y0.z; Y[3] = y0.w; Y[4] = y1.x; Y[5] = y1.y; Y[6] = y1.z; Y[7] = y1.w;
                Y[8] = y2.x; Y[9] = y2.y; Y[10] = y2.z; Y[11] = y2.w; Y[12] = y3.x; Y[13] = y3.y; Y[14] = y3.z; Y[15] = y3.w;
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar0 + 8 * (kFwdStages + stage));
            if (++stage == kFwdStages) { stage = 0; parity ^= 1u; }
            tp_forward_pair<LIN>(xs, Y, w, acc);
        }
        float2* out = reinterpret_cast<float2*>(mid + ((long long)i * MID) * kC) + c;
#pragma unroll
        for (int k = 0; k < MID; ++k) out[(long long)k * (kC / 2)] = acc[k];
    }
    __syncthreads();
    if (c == 0 && abort_sh && error_word) atomicOr(error_word, FMB_STATUS_TENSOR_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------- backward
constexpr int kEdgeBatch = 8;
constexpr int kRed = 17;     // 16 harmonic gradients + the radial one

// After the call, lane l of each warp holds in `v[0]` the warp sum of value (l >> 1) of the 16 inputs.
__device__ __forceinline__ void warp_reduce16(float (&v)[16]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int half = 8, bit = 16; half >= 1; half >>= 1, bit >>= 1) {
        const bool upper = (lane & bit) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float keep = upper ? v[i + half] : v[i];
            const float send = upper ? v[i] : v[i + half];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
        }
    }
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
}

template <int LIN, bool SPECIES_X, bool NEED_DX, int MINB = 1>
__global__ void __launch_bounds__(kC, MINB)
k_tp_backward(int n_atoms, int n_rows, int n_valid, int fresh_from, long long chunk_e0, long long chunk_edges, long long tangent_offset,
              const long long* __restrict__ count_ptr, const int32_t* __restrict__ row_ptr,
              const int32_t* __restrict__ senders, const int32_t* __restrict__ species, const float* __restrict__ x,
              const float* __restrict__ edge_sh, const float* __restrict__ edge_vec, const float* __restrict__ tp_w,
              const float* __restrict__ d_mid, float* __restrict__ d_x, float* __restrict__ force_acc,
              float* __restrict__ atom_virial, int first_layer_of_pass) {
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    __shared__ float red[kEdgeBatch][4][kRed + 1];
    const long long count = *count_ptr;
    const long long e0 = chunk_e0, e1 = min(count, chunk_e0 + chunk_edges);
    const int c = threadIdx.x, warp = c >> 5, lane = c & 31;
    if (e0 >= e1 && !(e0 == 0 && count == 0)) return;
    const int first = (e0 == 0) ? 0 : chunk_first_row(row_ptr, n_atoms, e0);
    for (int a = first + blockIdx.x; a < n_rows; a += gridDim.x) {
        const long long rb = row_ptr[a], re = row_ptr[a + 1];
        if (rb >= e1 && e1 < count) break;
        const bool continued = rb < e0;     // this row started in an earlier chunk: accumulate onto its partial sums
        float g_a[MID], x_a[IN], dx[IN];
#pragma unroll
        for (int k = 0; k < MID; ++k) g_a[k] = a < n_valid ? __ldg(d_mid + ((long long)a * MID + k) * kC + c) : 0.0f;
        if (SPECIES_X) {
            x_a[0] = __ldg(x + (long long)species[a] * kC + c);
        } else {
#pragma unroll
            for (int k = 0; k < IN; ++k) x_a[k] = __ldg(x + ((long long)a * IN + k) * kC + c);
        }
#pragma unroll
        for (int k = 0; k < IN; ++k) dx[k] = 0.0f;
        float fsum[3] = {0.f, 0.f, 0.f}, vir[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        const long long b = max(rb, e0), en = min(re, e1);
        for (long long batch = b; batch < en; batch += kEdgeBatch) {
            const int nb = (int)min((long long)kEdgeBatch, en - batch);
            for (int k = 0; k < nb; ++k) {
                const long long e = batch + k;
                const int j = senders[e];
                float Y[16], w[P], wp[P], x_j[IN], dY[16];
                load_sh(edge_sh, e, Y);
                const float* wr = tp_w + (e - chunk_e0) * (long long)(P * kC) + c;
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    w[p] = __ldg(wr + p * kC);
                    wp[p] = __ldg(wr + tangent_offset + p * kC);
                }
                if (SPECIES_X) {
                    x_j[0] = __ldg(x + (long long)species[j] * kC + c);
                } else {
#pragma unroll
                    for (int q = 0; q < IN; ++q) x_j[q] = __ldg(x + ((long long)j * IN + q) * kC + c);
                }
#pragma unroll
                for (int q = 0; q < 16; ++q) dY[q] = 0.0f;
                float dr = 0.0f;
                float unused[IN];
                // the edge as stored: receiver a, sender j
                TpBackward<LIN, false, false>::run(x_j, Y, w, wp, g_a, dY, dr, unused);
                // its mirror: receiver j, sender a
                {
                    float g_j[MID];
#pragma unroll
                    // rows at or beyond n_valid carry no gradient (atoms whose energy another domain owns)
                    for (int q = 0; q < MID; ++q)
                        g_j[q] = j < n_valid ? __ldg(d_mid + ((long long)j * MID + q) * kC + c) : 0.0f;
                    TpBackward<LIN, true, NEED_DX>::run(x_a, Y, w, wp, g_j, dY, dr, dx);
                }
                warp_reduce16(dY);
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
                fsum[0] += q3[0]; fsum[1] += q3[1]; fsum[2] += q3[2];
                const float vx = uv.x * uv.w, vy = uv.y * uv.w, vz = uv.z * uv.w;
                vir[0] += vx * q3[0]; vir[1] += vy * q3[1]; vir[2] += vz * q3[2];
                vir[3] += 0.5f * (vy * q3[2] + vz * q3[1]);
                vir[4] += 0.5f * (vx * q3[2] + vz * q3[0]);
                vir[5] += 0.5f * (vx * q3[1] + vy * q3[0]);
            }
            __syncthreads();
        }
        // threads 0..7 hold partial force / virial sums: fold them inside warp 0
        if (warp == 0) {
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
#pragma unroll
                for (int q = 0; q < 3; ++q) fsum[q] += __shfl_xor_sync(0xffffffffu, fsum[q], o);
#pragma unroll
                for (int q = 0; q < 6; ++q) vir[q] += __shfl_xor_sync(0xffffffffu, vir[q], o);
            }
            if (lane == 0) {
                const bool fresh = (first_layer_of_pass || a >= fresh_from) && !continued;
#pragma unroll
                for (int q = 0; q < 3; ++q)
                    force_acc[3 * a + q] = (fresh ? 0.0f : force_acc[3 * a + q]) + fsum[q];
#pragma unroll
                for (int q = 0; q < 6; ++q)
                    atom_virial[6 * a + q] = (fresh ? 0.0f : atom_virial[6 * a + q]) + 0.5f * vir[q];
            }
        }
        if (NEED_DX) {
#pragma unroll
            for (int k = 0; k < IN; ++k) {
                float* dst = d_x + ((long long)a * IN + k) * kC + c;
                *dst = continued ? *dst + dx[k] : dx[k];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------- first layer
// The first layer's senders are species-only rows, so its message factorises (exact algebra, the reference's
// "reassociation", fastmace/rewrites/mh1/modules.py:146-160): per receiver i and sender species z
//     S[i, lm, z, k] = sum_{e -> i, species(sender e) = z} Y[e, lm] * hidden[e, k]          (16 x 64 per species)
// and the message is S times a per-l matrix that folds the last radial layer, the sender row and the message linear.
// No [E, P*C] weights, no tensor product per edge.
constexpr int kFirstZ = FMB_MAX_SPECIES;

// CTA per receiver, thread = (k = tid & 63, half = tid >> 6 -> harmonics 8 * half .. 8 * half + 7). The sums live in
// registers, one set per sender species (an edge adds into the set of its sender's species through a 0 / 1 factor, so
// that no index depends on data), and the operands of four edges are requested together: the chain sender -> species
// -> features is three dependent loads, which a loop over single edges pays in full for every edge (11 warps stalled
// on loads per issued instruction in the version that accumulated in shared memory).
template <int Z>
__global__ void __launch_bounds__(kC)
k_first_accumulate(int n_rows, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
                   const int32_t* __restrict__ species, const float* __restrict__ edge_sh,
                   const float* __restrict__ hidden, float* __restrict__ s_out) {
    constexpr int kAhead = 4;
    const int k = threadIdx.x & 63, half = threadIdx.x >> 6;
    for (int i = blockIdx.x; i < n_rows; i += gridDim.x) {
        float acc[Z][8];
#pragma unroll
        for (int z = 0; z < Z; ++z)
#pragma unroll
            for (int m = 0; m < 8; ++m) acc[z][m] = 0.0f;
        const long long rb = row_ptr[i], re = row_ptr[i + 1];
        for (long long e0 = rb; e0 < re; e0 += kAhead) {
            int zs[kAhead];
            float h[kAhead];
            float4 y0[kAhead], y1[kAhead];
#pragma unroll
            for (int q = 0; q < kAhead; ++q) {
                const bool live = e0 + q < re;
                const long long e = live ? e0 + q : rb;
                zs[q] = species[senders[e]];
                h[q] = live ? __ldg(hidden + e * kRadial + k) : 0.0f;
                const float4* yp = reinterpret_cast<const float4*>(edge_sh + 16 * e + 8 * half);
                y0[q] = __ldg(yp);
                y1[q] = __ldg(yp + 1);
            }
#pragma unroll
            for (int q = 0; q < kAhead; ++q)
#pragma unroll
                for (int z = 0; z < Z; ++z) {
                    const float hz = zs[q] == z ? h[q] : 0.0f;
                    acc[z][0] = fmaf(y0[q].x, hz, acc[z][0]);
                    acc[z][1] = fmaf(y0[q].y, hz, acc[z][1]);
                    acc[z][2] = fmaf(y0[q].z, hz, acc[z][2]);
                    acc[z][3] = fmaf(y0[q].w, hz, acc[z][3]);
                    acc[z][4] = fmaf(y1[q].x, hz, acc[z][4]);
                    acc[z][5] = fmaf(y1[q].y, hz, acc[z][5]);
                    acc[z][6] = fmaf(y1[q].z, hz, acc[z][6]);
                    acc[z][7] = fmaf(y1[q].w, hz, acc[z][7]);
                }
        }
        // global layout [i][lm][z][k]: the K = n_species * 64 values of one (atom, harmonic) row are contiguous
        float* out = s_out + (long long)i * kNSH * Z * kRadial + k;
#pragma unroll
        for (int z = 0; z < Z; ++z)
#pragma unroll
            for (int m = 0; m < 8; ++m) out[((8 * half + m) * Z + z) * kRadial] = acc[z][m];
    }
}

// Backward of the same: CTA per atom a; for each edge j -> a of its row both the edge (gradient block of a, species
// of j) and its mirror a -> j (gradient block of j, species of a, harmonics with (-1)^l) contribute
//   dE/dY[lm] = sum_k C[lm, k] hidden[k],   dE/dr = sum_k hidden'[k] sum_lm C[lm, k] Y[lm],   C = G_a[., z_j] + (-1)^l G_j[., z_a]
// and the force on a is minus the sum over the row of the edge-vector gradient, as in k_tp_backward.
__global__ void __launch_bounds__(kC)
k_first_backward(int n_rows, int n_valid, int fresh_from, int n_species, const long long* __restrict__ count_ptr,
                 const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ senders,
                 const int32_t* __restrict__ species, const float* __restrict__ edge_sh,
                 const float* __restrict__ edge_vec, const float* __restrict__ hidden,
                 const float* __restrict__ hidden_tangent, const float* __restrict__ d_s,
                 float* __restrict__ force_acc, float* __restrict__ atom_virial, int first_layer_of_pass) {
    __shared__ float red[kEdgeBatch][4][kRed + 1];
    extern __shared__ float own[];                        // this atom's gradient block [16][n_species][64]
    const int c = threadIdx.x, k = c & 63, half = c >> 6, warp = c >> 5, lane = c & 31;
    const long long row_floats = (long long)kNSH * n_species * kRadial;
    for (int a = blockIdx.x; a < n_rows; a += gridDim.x) {
        const long long rb = row_ptr[a], re = row_ptr[a + 1];
        const int za = species[a];
        __syncthreads();
        for (int q = c; q < (int)row_floats; q += kC) own[q] = a < n_valid ? __ldg(d_s + a * row_floats + q) : 0.0f;
        __syncthreads();
        float fsum[3] = {0.f, 0.f, 0.f}, vir[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (long long batch = rb; batch < re; batch += kEdgeBatch) {
            const int nb = (int)min((long long)kEdgeBatch, re - batch);
            for (int b = 0; b < nb; ++b) {
                const long long e = batch + b;
                const int j = senders[e];
                const int zj = species[j];
                const float h = __ldg(hidden + e * kRadial + k), hp = __ldg(hidden_tangent + e * kRadial + k);
                const float4* yp = reinterpret_cast<const float4*>(edge_sh + 16 * e + 8 * half);
                const float4 y0 = __ldg(yp), y1 = __ldg(yp + 1);
                const float Y[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
                float part[9];
                float dh = 0.0f;
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    const int lm = 8 * half + m;
                    // (-1)^l of harmonic lm: l = 0 (lm 0), 1 (1..3), 2 (4..8), 3 (9..15)
                    const float sign = (lm >= 1 && lm <= 3) || lm >= 9 ? -1.0f : 1.0f;
                    const long long cell = ((long long)lm * n_species) * kRadial + k;
                    const float ga = own[cell + zj * kRadial];
                    const float gj = j < n_valid ? __ldg(d_s + j * row_floats + cell + (long long)za * kRadial) : 0.0f;
                    const float cc = ga + sign * gj;
                    part[m] = cc * h;
                    dh = fmaf(cc, Y[m], dh);
                }
                part[8] = dh * hp;
                // reduce over the warp: the 8 harmonic sums with a transpose-reduce (lane l ends with value l >> 2),
                // the radial one with a plain butterfly; the warps meet in shared memory
#pragma unroll
                for (int halfw = 4, bit = 16; halfw >= 1; halfw >>= 1, bit >>= 1) {
                    const bool upper = (lane & bit) != 0;
#pragma unroll
                    for (int m = 0; m < halfw; ++m) {
                        const float keep = upper ? part[m + halfw] : part[m];
                        const float send = upper ? part[m] : part[m + halfw];
                        part[m] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                    }
                }
                part[0] += __shfl_xor_sync(0xffffffffu, part[0], 2);
                part[0] += __shfl_xor_sync(0xffffffffu, part[0], 1);
                part[8] = warp_sum(part[8]);
                if ((lane & 3) == 0) red[b][warp][lane >> 2] = part[0];
                if (lane == 0) red[b][warp][16] = part[8];
            }
            __syncthreads();
            if (c < nb) {
                const long long e = batch + c;
                float g[16];
                // warps 0, 1 hold harmonics 0..7 (half 0), warps 2, 3 harmonics 8..15
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    g[m] = red[c][0][m] + red[c][1][m];
                    g[8 + m] = red[c][2][m] + red[c][3][m];
                }
                const float drt = red[c][0][16] + red[c][1][16] + red[c][2][16] + red[c][3][16];
                const float4 uv = __ldg(reinterpret_cast<const float4*>(edge_vec) + e);
                float q3[3];
                edge_vector_gradient(g, drt, uv.x, uv.y, uv.z, uv.w, q3);
                fsum[0] += q3[0]; fsum[1] += q3[1]; fsum[2] += q3[2];
                const float vx = uv.x * uv.w, vy = uv.y * uv.w, vz = uv.z * uv.w;
                vir[0] += vx * q3[0]; vir[1] += vy * q3[1]; vir[2] += vz * q3[2];
                vir[3] += 0.5f * (vy * q3[2] + vz * q3[1]);
                vir[4] += 0.5f * (vx * q3[2] + vz * q3[0]);
                vir[5] += 0.5f * (vx * q3[1] + vy * q3[0]);
            }
            __syncthreads();
        }
        if (warp == 0) {
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
#pragma unroll
                for (int q = 0; q < 3; ++q) fsum[q] += __shfl_xor_sync(0xffffffffu, fsum[q], o);
#pragma unroll
                for (int q = 0; q < 6; ++q) vir[q] += __shfl_xor_sync(0xffffffffu, vir[q], o);
            }
            if (lane == 0) {
                const bool fresh = first_layer_of_pass || a >= fresh_from;
#pragma unroll
                for (int q = 0; q < 3; ++q)
                    force_acc[3 * a + q] = (fresh ? 0.0f : force_acc[3 * a + q]) + fsum[q];
#pragma unroll
                for (int q = 0; q < 6; ++q)
                    atom_virial[6 * a + q] = (fresh ? 0.0f : atom_virial[6 * a + q]) + 0.5f * vir[q];
            }
        }
    }
}

int persistent_grid(const void* kernel, int n_atoms) {
    static std::map<const void*, int> cache;
    auto it = cache.find(kernel);
    if (it == cache.end()) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kC, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
        int sms = 148, dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        it = cache.emplace(kernel, per_sm * sms * 4).first;
    }
    return n_atoms < it->second ? n_atoms : it->second;
}

}  // namespace

int tp_forward_launch(const TpArgs& t, cudaStream_t stream) {
    if (t.n_rows <= 0) return FMB_OK;
#define FMB_FWD(LIN_, SP_)                                                                                             \
    {                                                                                                                  \
        auto kernel = k_tp_forward<LIN_, SP_>;                                                                         \
        const int grid = persistent_grid((const void*)kernel, t.n_rows);                                                           \
        kernel<<<grid, kC, 0, stream>>>(t.n_atoms, t.n_rows, t.chunk_e0, t.chunk_edges, t.count, t.row_ptr, t.senders, \
                                        t.species, t.x, t.edge_sh, t.tp_w, t.mid);                                     \
    }
#define FMB_FWD_STREAM(LIN_)                                                                                           \
    {                                                                                                                  \
        constexpr int smem = kFwdStages * (TpShape<LIN_>::kPaths * kC + TpShape<LIN_>::kInDim * kC + 16) * 4;          \
        static int grid_cap = 0;                                                                                       \
        FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_tp_forward_stream<LIN_>, smem));                            \
        if (grid_cap == 0) {                                                                                           \
            int per_sm = 0, sms = 148, dev = 0;                                                                        \
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_tp_forward_stream<LIN_>, kC, smem) != cudaSuccess || \
                per_sm < 1)                                                                                            \
                per_sm = 1;                                                                                            \
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); \
            grid_cap = per_sm * sms;                                                                                   \
        }                                                                                                              \
        const int grid = t.n_rows < grid_cap ? t.n_rows : grid_cap;                                                    \
        k_tp_forward_stream<LIN_><<<grid, kC, smem, stream>>>(t.n_rows, t.row_ptr, t.senders, t.x, t.edge_sh, t.tp_w,  \
                                                              t.mid, t.error_word);                                    \
    }
    if (t.species_x) {
        FMB_REQUIRE(t.lin == 0, "tp_forward: species table only for scalar senders");
        FMB_FWD(0, true)
    } else if (t.lin == 0) {
        FMB_FWD(0, false)
    } else if (t.whole_list && t.lin == 1) {
        constexpr int smem = kFwdStages * (TpShape<1>::kPaths * kC + TpShape<1>::kInDim * kC + 16) * 4;
        static int grid_cap = 0;
        FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_tp_forward_pairs<1>, smem));
        if (grid_cap == 0) {
            int per_sm = 0, sms = 148, dev = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_tp_forward_pairs<1>, kPairThreads, smem) != cudaSuccess ||
                per_sm < 1)
                per_sm = 1;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            grid_cap = per_sm * sms;
        }
        const int grid = t.n_rows < grid_cap ? t.n_rows : grid_cap;
        k_tp_forward_pairs<1><<<grid, kPairThreads, smem, stream>>>(t.n_rows, t.row_ptr, t.senders, t.x, t.edge_sh, t.tp_w,
                                                                    t.mid, t.error_word, t.mirror, t.slot);
    } else if (t.whole_list && t.lin == 2) {
        FMB_FWD_STREAM(2)
    } else if (t.lin == 1) {
        FMB_FWD(1, false)
    } else if (t.lin == 2) {
        FMB_FWD(2, false)
    } else {
        FMB_REQUIRE(false, "tp_forward: unsupported node l_max");
    }
#undef FMB_FWD
#undef FMB_FWD_STREAM
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int tp_backward_launch(const TpArgs& t, cudaStream_t stream) {
    if (t.n_rows <= 0) return FMB_OK;
#define FMB_BWD_OCC(LIN_, SP_, DX_, MINB_)                                                                             \
    {                                                                                                                  \
        auto kernel = k_tp_backward<LIN_, SP_, DX_, MINB_>;                                                            \
        const int grid = persistent_grid((const void*)kernel, t.n_rows);                                               \
        kernel<<<grid, kC, 0, stream>>>(t.n_atoms, t.n_rows, t.n_valid, t.fresh_from, t.chunk_e0, t.chunk_edges,       \
                                        t.tangent_offset, t.count, t.row_ptr,                                         \
                                        t.senders, t.species, t.x, t.edge_sh, t.edge_vec, t.tp_w, t.d_mid, t.d_x,      \
                                        t.force_acc, t.atom_virial, t.first_layer_of_pass);                            \
    }
#define FMB_BWD(LIN_, SP_, DX_) FMB_BWD_OCC(LIN_, SP_, DX_, 1)
    if (t.species_x) {
        FMB_REQUIRE(t.lin == 0, "tp_backward: species table only for scalar senders");
        FMB_BWD(0, true, false)
    } else if (t.lin == 0) {
        FMB_BWD(0, false, true)
    } else if (t.lin == 1) {
        // CTAs per SM the compiler targets (FMB_TP_OCCUPANCY = 2, 3 or 4; 168 / 128 registers at 3 / 4). Measured on
        // the 1,944-atom cell: 0.47 / 0.51 / 0.56 ms -- the kernel is bound by the 37 KB per edge it pulls through L2
        // (the mirror receiver's 20 KB gradient row, 10 KB of radial weights), not by issue slots, so 2 stays.
        FMB_BWD_OCC(1, false, true, 2)
    } else if (t.lin == 2) {
        FMB_BWD(2, false, true)
    } else {
        FMB_REQUIRE(false, "tp_backward: unsupported node l_max");
    }
#undef FMB_BWD
#undef FMB_BWD_OCC
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace fmb

namespace fmb {

int first_accumulate_launch(const FirstArgs& f, cudaStream_t stream) {
    if (f.n_rows <= 0) return FMB_OK;
    FMB_REQUIRE(f.n_species >= 1 && f.n_species <= kFirstZ, "first layer: too many species");
#define FMB_FIRST(Z_)                                                                                              \
    case Z_: {                                                                                                     \
        const int grid = persistent_grid((const void*)k_first_accumulate<Z_>, f.n_rows);                           \
        k_first_accumulate<Z_><<<grid, kC, 0, stream>>>(f.n_rows, f.row_ptr, f.senders, f.species, f.edge_sh,     \
                                                        f.hidden, f.s);                                            \
        break;                                                                                                     \
    }
    switch (f.n_species) {
        FMB_FIRST(1) FMB_FIRST(2) FMB_FIRST(3) FMB_FIRST(4) FMB_FIRST(5) FMB_FIRST(6) FMB_FIRST(7) FMB_FIRST(8)
        default: FMB_REQUIRE(false, "first layer: too many species");
    }
#undef FMB_FIRST
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int first_backward_launch(const FirstArgs& f, cudaStream_t stream) {
    if (f.n_rows <= 0) return FMB_OK;
    const int grid = persistent_grid((const void*)k_first_backward, f.n_rows);
    const size_t smem = (size_t)kNSH * f.n_species * kRadial * sizeof(float);
    k_first_backward<<<grid, kC, smem, stream>>>(f.n_rows, f.n_valid, f.fresh_from, f.n_species, f.count, f.row_ptr,
                                              f.senders, f.species, f.edge_sh, f.edge_vec, f.hidden, f.hidden_tangent,
                                              f.d_s, f.force_acc, f.atom_virial, f.first_layer_of_pass);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace fmb
