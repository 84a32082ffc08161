// Channelwise tensor product of the interactions after the first, fused with the last layer of the radial MLP: the
// per-edge weights W[e, path, channel] = hidden[e, :] . W4[:, path, channel] are produced by the tensor cores straight
// into tensor memory and consumed from there, so the [edges][paths * 128] weight matrix (5 KB per edge for ten paths)
// never exists in HBM. Replaces conv_tp + scatter_sum and the last radial linear (fastmace/rewrites/generic/
// modules.py:485-486). Forward only: the adjoint of these interactions is the per-edge hand-over kernel
// (adjoint_edges.cu) or, for lists too large for its buffers, the mirror evaluation (interaction.cu); a fused
// adjoint of this shape needs one channel reduction per path and measured three times slower than the former.
//
// One persistent CTA per SM: 8 consumer warps (two groups of 128 threads, thread = channel = TMEM lane) and one warp
// that feeds the tensor cores. A work item is a pair of receivers, one per consumer group; a round covers up to 64
// edges of each. Per round the consumers split the edges' 64 hidden radial features into tf32 hi / lo parts and write
// them as the N-side operand (K-major, 128-byte swizzle); then, path by path,
//   * bulk copies bring the path's 128 x 64 block of W4 (pre-split and pre-swizzled at packing time, 16 KB pieces)
//     through a ring of shared-memory stages,
//   * one thread issues the 3xTF32 MMAs (M = 128 channels, N = 128 edge columns, K = 64) into one of two TMEM
//     accumulators and commits to mbarriers,
//   * each consumer thread reads its lane (channel) four edge columns at a time and applies the path's coupling
//     (generated bodies, tp_paths_generated.cuh) while the tensor cores work on the next path.
// The message row of a receiver is accumulated in registers per path and stored once per round; nothing is scattered
// and there are no atomics.
//
// Every wait is bounded (tc::mbar_wait): if one gives up, the CTA raises FMB_STATUS_TENSOR_TIMEOUT, stops waiting
// everywhere, runs to its end and frees its tensor memory.

#include "stages.cuh"
#include "tc_common.cuh"
#include "edge_gradient.cuh"
#include "generated/tp_generated.cuh"
#include "generated/tp_paths_generated.cuh"

#include <type_traits>

namespace fmb {

namespace {

using namespace tc;


constexpr int kFusedThreads = 288;        // 8 consumer warps + the tensor-core warp
constexpr int kStageBytes = 16384;        // one (hi or lo) x (K half) piece of a path's weight block: 128 rows x 32
constexpr int kRoundEdges = 64;           // edge columns per consumer group and round
constexpr unsigned kSpin = 1u << 20;

struct FusedShape {
    static constexpr int kTN = 128;              // MMA N: edge columns (+ their d/dr twins)
    static constexpr int kBTile = kTN * 256;                  // bytes of the hi (or lo) N-side operand
    static constexpr int kStages = 8;
    static constexpr int kRing = 2 * kBTile;
    static constexpr int kYsh = kRing + kStages * kStageBytes;           // harmonics of the round's edges [128][16]
    static constexpr int kVec = kYsh + 128 * 64;                         // unit vector and length [128] float4
    static constexpr int kSnd = kVec + 128 * 16;                         // senders [128]
    static constexpr int kRed = kSnd + 128 * 4;                          // adjoint: [128 edges][4 warps][17]
    static constexpr int kScratch = kRed + 0; // force / virial hand-over between warps
    static constexpr int kBars = kScratch + 256;
    static constexpr int kMisc = kBars + 256;
    static constexpr int kBytes = kMisc + 16 + 1024;                     // + slack to align the base to 1024 bytes
};
static_assert(FusedShape::kBytes <= 232448, "shared memory budget");

// barrier slots
constexpr int kBarFull = 0, kBarEmpty = 8, kBarTFull = 16, kBarTEmpty = 18, kBarB = 20;

constexpr int pow2_at_least(int n) { return n <= 2 ? 2 : n <= 4 ? 4 : n <= 8 ? 8 : 16; }
constexpr int log2_of(int n) { return n == 2 ? 1 : n == 4 ? 2 : n == 8 ? 3 : 4; }

// Transpose-reduce of NP (a power of two <= 16) values over the warp: afterwards v[0] of lane l holds the warp total
// of value l >> (5 - log2 NP).
template <int NP>
__device__ __forceinline__ void warp_reduce_t(float (&v)[NP]) {
    const int lane = threadIdx.x & 31;
    int bit = 16;
#pragma unroll
    for (int half = NP / 2; half >= 1; half >>= 1, bit >>= 1) {
        const bool upper = (lane & bit) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float keep = upper ? v[i + half] : v[i];
            const float send = upper ? v[i] : v[i + half];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
        }
    }
#pragma unroll
    for (int rest = 16 >> log2_of(NP); rest >= 1; rest >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], rest);
}

// State of the thread that feeds the tensor cores: it keeps the ring of weight pieces full (bulk copies, look-ahead
// of NST pieces across paths, rounds and work items: the sequence of pieces is periodic) and issues the MMAs of one
// path at a time. Counters wrap by comparison, there is no division on this thread's critical path.
template <int TN, int NST>
struct Feeder {
    uint32_t bar0, ring0, tmem_base, idesc;
    uint64_t desc_bh, desc_bl;
    const float* image;
    volatile int* abort_flag;
    uint32_t pieces;                  // 4 * paths: pieces of one pass over the weight image
    uint32_t total;                   // pieces this CTA consumes in all
    uint32_t step = 0, load = 0;      // pieces consumed / requested
    uint32_t st = 0, ph = 0;          // stage and parity of the next piece to consume
    uint32_t lst = 0, lph = 1;        // stage to refill and the parity its `empty` barrier has to show
    uint32_t piece = 0;               // next piece to request
    uint32_t gpath = 0, ground = 0;

    __device__ __forceinline__ uint32_t bar(int slot) const { return bar0 + 8u * (uint32_t)slot; }

    __device__ __forceinline__ void top_up() {
        while (load < total && load - step < (uint32_t)NST) {
            mbar_wait(bar(kBarEmpty) + 8u * lst, lph, abort_flag, kSpin);
            const uint32_t full = bar(kBarFull) + 8u * lst;
            mbar_expect_tx(full, kStageBytes);
            bulk_load(ring0 + lst * kStageBytes, image + (size_t)piece * (kStageBytes / 4), kStageBytes, full);
            ++load;
            if (++piece == pieces) piece = 0;
            if (++lst == (uint32_t)NST) { lst = 0; lph ^= 1u; }
        }
    }

    // waits until the consumers have staged the N-side operand of the next round
    __device__ __forceinline__ void begin_round() {
        top_up();
        mbar_wait(bar(kBarB), ground & 1u, abort_flag, kSpin);
        fence_after_sync();
        ++ground;
    }

    // the 24 MMAs of one path (3xTF32: weights_lo x hidden_hi, weights_hi x hidden_lo, weights_hi x hidden_hi, per K
    // half) into accumulator gpath & 1
    __device__ __forceinline__ void path() {
        const uint32_t buf = gpath & 1u;
        mbar_wait(bar(kBarTEmpty + buf), ((gpath >> 1) & 1u) ^ 1u, abort_flag, kSpin);
        fence_after_sync();
        const uint32_t d = tmem_base + buf * TN;
#pragma unroll
        for (int s4 = 0; s4 < 4; ++s4) {
            top_up();
            mbar_wait(bar(kBarFull) + 8u * st, ph, abort_flag, kSpin);
            fence_after_sync();
            const uint64_t adesc = make_desc(ring0 + st * kStageBytes);
            const int kh = s4 >> 1;
            if ((s4 & 1) == 0) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_tf32(d, adesc + (uint64_t)(2 * k), desc_bh + k_step<TN>(4 * kh + k), idesc, (s4 == 0 && k == 0) ? 0 : 1);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_tf32(d, adesc + (uint64_t)(2 * k), desc_bl + k_step<TN>(4 * kh + k), idesc, 1);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_tf32(d, adesc + (uint64_t)(2 * k), desc_bh + k_step<TN>(4 * kh + k), idesc, 1);
            }
            mma_commit(bar(kBarEmpty) + 8u * st);
            ++step;
            if (++st == (uint32_t)NST) { st = 0; ph ^= 1u; }
        }
        mma_commit(bar(kBarTFull + buf));
        ++gpath;
    }
};

// sender rows of EB edge columns for one path: the path's input components of x (and, for the adjoint, the path's
// components of the senders' message gradient; rows at or beyond n_valid read as zero)
template <typename TP, int IN, int EB>
__device__ __forceinline__ void gather_x(const float* __restrict__ x, const int* __restrict__ snd_col, int c,
                                         float (&xn)[EB][TP::kNin]) {
#pragma unroll
    for (int q = 0; q < EB; ++q) {
        const long long j = snd_col[q];
#pragma unroll
        for (int m = 0; m < TP::kNin; ++m) xn[q][m] = __ldg(x + ((j * IN + TP::kInOff + m) * kC + c));
    }
}

// rows and rounds of work item `item` (receivers 2 item and 2 item + 1)
struct ItemRows {
    int rb[2], deg[2], rounds;
};
__device__ __forceinline__ ItemRows item_rows(const int32_t* __restrict__ row_ptr, int n_rows, int item) {
    ItemRows r;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const int i = 2 * item + g;
        if (i < n_rows) {
            r.rb[g] = row_ptr[i];
            r.deg[g] = row_ptr[i + 1] - r.rb[g];
        } else {
            r.rb[g] = 0;
            r.deg[g] = 0;
        }
    }
    const int longest = max(r.deg[0], r.deg[1]);
    r.rounds = max(1, (longest + kRoundEdges - 1) / kRoundEdges);
    return r;
}

template <int LIN>
__global__ void __launch_bounds__(kFusedThreads, 1)
k_tp_fused(const __grid_constant__ FusedArgs a) {
    using S = FusedShape;
    constexpr int P = TpShape<LIN>::kPaths, IN = TpShape<LIN>::kInDim, MID = TpShape<LIN>::kMidDim;
    constexpr int TN = S::kTN, NST = S::kStages;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* b_hi = smem;
    uint8_t* b_lo = smem + S::kBTile;
    uint8_t* ring = smem + S::kRing;
    float* ysh = reinterpret_cast<float*>(smem + S::kYsh);
    int* snd = reinterpret_cast<int*>(smem + S::kSnd);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::kMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::kMisc + 4);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int slot) { return bar0 + 8u * (uint32_t)slot; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(bar(kBarFull + s), 1);
            mbar_init(bar(kBarEmpty + s), 1);
        }
        mbar_init(bar(kBarTFull), 1);
        mbar_init(bar(kBarTFull + 1), 1);
        mbar_init(bar(kBarTEmpty), 8);
        mbar_init(bar(kBarTEmpty + 1), 8);
        mbar_init(bar(kBarB), 8);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(smem_u32(tmem_slot), 2 * TN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const int n_items = (a.n_rows + 1) >> 1;
    const int32_t* __restrict__ row_ptr = a.row_ptr;

    if (warp == 8) {
        // ------------------------------------------------------------------ tensor-core warp (one thread)
        if (lane == 0) {
            Feeder<TN, NST> feed;
            feed.bar0 = bar0; feed.ring0 = smem_u32(ring); feed.tmem_base = tmem_base; feed.idesc = make_idesc<TN>();
            feed.desc_bh = make_desc(smem_u32(b_hi)); feed.desc_bl = make_desc(smem_u32(b_lo));
            feed.image = a.image; feed.abort_flag = abort_flag; feed.pieces = 4u * P;
            uint32_t total = 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x)
                total += (uint32_t)item_rows(row_ptr, a.n_rows, item).rounds * (4u * P);
            feed.total = total;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
                const int rounds = item_rows(row_ptr, a.n_rows, item).rounds;
                for (int r = 0; r < rounds; ++r) {
                    feed.begin_round();
                    for (int p = 0; p < P; ++p) feed.path();
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ consumers: thread = channel = TMEM lane
        const int wg = tid >> 7, c = tid & 127, quadrant = warp & 3;
        const uint32_t lane_base = (uint32_t)(quadrant * 32) << 16;
        const int col0 = wg * kRoundEdges;
        uint32_t gpath = 0;
        const float* __restrict__ x = a.x;
        // staging map of the N-side operand: 64 rows x 16 float4 per sweep of the 256 threads
        const int ld_row = warp * 8 + (lane & 7), ld_q = lane >> 3;
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const ItemRows rows = item_rows(row_ptr, a.n_rows, item);
            const int i = 2 * item + wg;
            const bool row_ok = i < a.n_rows;
            for (int r = 0; r < rows.rounds; ++r) {
                const int n_g = min(max(rows.deg[wg] - r * kRoundEdges, 0), kRoundEdges);
                named_barrier(1, 256);              // every consumer is done with the previous round's tables
                if (tid < 128) {
                    const int g = tid >> 6, idx = tid & 63;
                    const bool ok = idx < rows.deg[g] - r * kRoundEdges;
                    const long long e = (long long)rows.rb[g] + r * kRoundEdges + idx;
                    snd[tid] = ok ? a.senders[e] : 0;
                }
                for (int q = tid; q < 512; q += 256) {
                    const int col = q >> 2, g = col >> 6, idx = col & 63;
                    const bool ok = idx < rows.deg[g] - r * kRoundEdges;
                    const long long e = (long long)rows.rb[g] + r * kRoundEdges + idx;
                    reinterpret_cast<float4*>(ysh)[q] =
                        ok ? __ldg(reinterpret_cast<const float4*>(a.edge_sh + 16 * e) + (q & 3)) : zero4;
                }

#pragma unroll
                for (int sweep = 0; sweep < TN / 64; ++sweep) {
                    const int row = ld_row + 64 * sweep;          // operand row: edge column, + 128 for its d/dr twin
                    const int col = row & 127, g = col >> 6, idx = col & 63;
                    const bool ok = idx < rows.deg[g] - r * kRoundEdges;
                    const long long e = (long long)rows.rb[g] + r * kRoundEdges + idx;
                    const float* src = a.hidden + e * kRadial;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 v = ok ? __ldg(reinterpret_cast<const float4*>(src) + ld_q + 4 * j) : zero4;
                        const float4 hi = make_float4(tf32_rna(v.x), tf32_rna(v.y), tf32_rna(v.z), tf32_rna(v.w));
                        const float4 lo = make_float4(tf32_rna(v.x - hi.x), tf32_rna(v.y - hi.y), tf32_rna(v.z - hi.z),
                                                      tf32_rna(v.w - hi.w));
                        const uint32_t off = tile_offset<TN>(row, (ld_q + 4 * j) * 4);
                        *reinterpret_cast<float4*>(b_hi + off) = hi;
                        *reinterpret_cast<float4*>(b_lo + off) = lo;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarB));
                named_barrier(1, 256);              // tables visible to every consumer

                auto path_fn = [&](auto tag) {
                    constexpr int p = decltype(tag)::value;
                    using TP = TpPath<LIN, p>;
                    constexpr int NI = TP::kNin, NE = TP::kNe, NO = TP::kNo;
                    const uint32_t buf = gpath & 1u;
                    const uint32_t t0 = tmem_base + lane_base + buf * TN + (uint32_t)col0;
{
                        // EB edges per batch; the next batch's sender rows are requested before this one is used, the
                        // first one before the accumulator is waited for
                        constexpr int EB = LIN == 1 ? 16 : 8;
                        float acc[NO];
#pragma unroll
                        for (int m = 0; m < NO; ++m) acc[m] = 0.0f;
                        float xn[EB][NI];
                        gather_x<TP, IN, EB>(x, snd + col0, c, xn);
                        mbar_wait(bar(kBarTFull + buf), (gpath >> 1) & 1u, abort_flag, kSpin);
                        fence_after_sync();
#pragma unroll 1
                        for (int sb = 0; sb < n_g; sb += EB) {
                            float xj[EB][NI], w[EB];
#pragma unroll
                            for (int q = 0; q < EB; ++q)
#pragma unroll
                                for (int m = 0; m < NI; ++m) xj[q][m] = xn[q][m];
                            if (sb + EB < n_g) gather_x<TP, IN, EB>(x, snd + col0 + sb + EB, c, xn);
                            tmem_load<EB>(t0 + sb, w);
#pragma unroll
                            for (int q = 0; q < EB; ++q) {
                                float Y[NE];
#pragma unroll
                                for (int m = 0; m < NE; ++m) Y[m] = ysh[(col0 + sb + q) * 16 + TP::kEdgeOff + m];
                                TP::forward(xj[q], Y, w[q], acc);
                            }
                        }
                        fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(kBarTEmpty + buf));
                        if (row_ok) {
#pragma unroll
                            for (int m = 0; m < NO; ++m) {
                                float* out = a.mid + (((long long)i * MID + TP::kSlotBase + m * TP::kSlotStride) * kC + c);
                                *out = r == 0 ? acc[m] : *out + acc[m];
                            }
                        }
                    }
                    ++gpath;
                };
#define FMB_PATH_CALL(p) path_fn(std::integral_constant<int, p>{});
                if constexpr (LIN == 1) {
                    FMB_FOR_EACH_PATH_1(FMB_PATH_CALL)
                } else {
                    FMB_FOR_EACH_PATH_2(FMB_PATH_CALL)
                }
#undef FMB_PATH_CALL


            }

        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 8) {
        __syncwarp();
        if (lane == 0 && *abort_flag && a.error_word) atomicOr(a.error_word, FMB_STATUS_TENSOR_TIMEOUT);
        tmem_free(tmem_base, 2 * TN);
    }
}

// ------------------------------------------------------------------------------------------------ weights only
// The same tensor-core pipeline used as a plain producer of the per-edge radial weights W[e][path * 128 + channel]
// (or of their d/dr, from the tangent features) for the edge-major kernels: tiles of 256 consecutive edges, the
// consumers only move accumulator columns to global memory -- lane = channel, so a warp writes 128 contiguous bytes of
// one edge row per store (a path-major layout [path][edge][128], contiguous per tile, measured slower both for this
// kernel and for its readers). The hidden features of a tile are split and staged once for all paths, the accumulator of
// path p is stored while the tensor cores work on path p + 1. HBM-write bound: 4 * paths * 128 bytes per edge.
struct WeightArgs {
    const float* hidden;          // [edges][64]
    const float* image;           // fmb_layer_t.rad_img
    float* out;                   // [edges][n_paths * 128]
    const long long* limit;       // device scalar: rows at or beyond *limit - limit_offset are skipped
    long long limit_offset;
    int rows;                     // host bound on the rows of this launch
    int n_paths;
    uint32_t* error_word;
    const int32_t* row_index;     // or null: output row r comes from hidden row row_index[r]
};

constexpr int kWeightStages = 4;
constexpr int kWeightTile = 256;
constexpr int kWeightRing = 2 * kWeightTile * 256;                    // after the hi and lo N-side operands
constexpr int kWeightBars = kWeightRing + kWeightStages * kStageBytes;
constexpr int kWeightBytes = kWeightBars + 256 + 16 + 1024;

__global__ void __launch_bounds__(kFusedThreads, 1)
k_radial_weights(const __grid_constant__ WeightArgs a) {
    constexpr int TN = kWeightTile, NST = kWeightStages;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* b_hi = smem;
    uint8_t* b_lo = smem + TN * 256;
    uint8_t* ring = smem + kWeightRing;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kWeightBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kWeightBars + 256);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kWeightBars + 260);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int slot) { return bar0 + 8u * (uint32_t)slot; };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(bar(kBarFull + s), 1);
            mbar_init(bar(kBarEmpty + s), 1);
        }
        mbar_init(bar(kBarTFull), 1);
        mbar_init(bar(kBarTFull + 1), 1);
        mbar_init(bar(kBarTEmpty), 8);
        mbar_init(bar(kBarTEmpty + 1), 8);
        mbar_init(bar(kBarB), 8);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(smem_u32(tmem_slot), 2 * TN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    long long rows = a.rows;
    if (a.limit) rows = min(rows, max(*a.limit - a.limit_offset, 0LL));
    const int n_tiles = (int)((rows + TN - 1) / TN);
    const int P = a.n_paths;

    if (warp == 8) {
        if (lane == 0) {
            Feeder<TN, NST> feed;
            feed.bar0 = bar0; feed.ring0 = smem_u32(ring); feed.tmem_base = tmem_base; feed.idesc = make_idesc<TN>();
            feed.desc_bh = make_desc(smem_u32(b_hi)); feed.desc_bl = make_desc(smem_u32(b_lo));
            feed.image = a.image; feed.abort_flag = abort_flag; feed.pieces = 4u * P;
            uint32_t total = 0;
            for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) total += 4u * P;
            feed.total = total;
            for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                feed.begin_round();
                for (int p = 0; p < P; ++p) feed.path();
            }
        }
    } else {
        const int wg = tid >> 7, c = tid & 127, quadrant = warp & 3;
        const uint32_t lane_base = (uint32_t)(quadrant * 32) << 16;
        const int ld_row = warp * 8 + (lane & 7), ld_q = lane >> 3;
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const long long ld = (long long)P * kC;
        uint32_t gpath = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) {
            const long long e0 = (long long)t * TN;
#pragma unroll
            for (int sweep = 0; sweep < TN / 64; ++sweep) {
                const int row = ld_row + 64 * sweep;
                const bool ok = e0 + row < rows;
                const long long source = a.row_index ? (ok ? (long long)a.row_index[e0 + row] : 0) : e0 + row;
                const float* src = a.hidden + source * kRadial;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 v = ok ? __ldg(reinterpret_cast<const float4*>(src) + ld_q + 4 * j) : zero4;
                    const float4 hi = make_float4(tf32_rna(v.x), tf32_rna(v.y), tf32_rna(v.z), tf32_rna(v.w));
                    const float4 lo = make_float4(tf32_rna(v.x - hi.x), tf32_rna(v.y - hi.y), tf32_rna(v.z - hi.z),
                                                  tf32_rna(v.w - hi.w));
                    const uint32_t off = tile_offset<TN>(row, (ld_q + 4 * j) * 4);
                    *reinterpret_cast<float4*>(b_hi + off) = hi;
                    *reinterpret_cast<float4*>(b_lo + off) = lo;
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarB));
            const long long eg = e0 + 128 * wg;                        // first edge of this group's 128 columns
            const int live = (int)min(128LL, max(rows - eg, 0LL));
            for (int p = 0; p < P; ++p) {
                const uint32_t buf = gpath & 1u;
                const uint32_t t0 = tmem_base + lane_base + buf * TN + 128u * (uint32_t)wg;
                mbar_wait(bar(kBarTFull + buf), (gpath >> 1) & 1u, abort_flag, kSpin);
                fence_after_sync();
                float* dst = a.out + eg * ld + (long long)p * kC + c;
                for (int sb = 0; sb < live; sb += 16) {
                    float w[16];
                    tmem_load<16>(t0 + sb, w);
#pragma unroll
                    for (int q = 0; q < 16; ++q)
                        if (sb + q < live) dst[(long long)(sb + q) * ld] = w[q];
                }
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarTEmpty + buf));
                ++gpath;
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 8) {
        __syncwarp();
        if (lane == 0 && *abort_flag && a.error_word) atomicOr(a.error_word, FMB_STATUS_TENSOR_TIMEOUT);
        tmem_free(tmem_base, 2 * TN);
    }
}

template <int LIN>
int launch_fused(const FusedArgs& f, cudaStream_t stream) {
    static int sms = 0;
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_tp_fused<LIN>, FusedShape::kBytes));
    if (sms == 0) {
        int dev = 0, count = 148;
        FMB_CUDA_CHECK(cudaGetDevice(&dev));
        FMB_CUDA_CHECK(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev));
        sms = count;
    }
    const int items = (f.n_rows + 1) / 2;
    const int grid = items < sms ? items : sms;       // one persistent CTA per SM
    k_tp_fused<LIN><<<grid, kFusedThreads, FusedShape::kBytes, stream>>>(f);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace

int radial_weights_tc(const float* hidden, const float* image, float* out, int rows, int n_paths, const long long* limit,
                      long long limit_offset, const int32_t* row_index, uint32_t* error_word, int max_ctas,
                      cudaStream_t stream) {
    if (!image || n_paths < 1) return FMB_ERR_UNSUPPORTED;
    if (rows <= 0) return FMB_OK;
    static int sms = 0;
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_radial_weights, kWeightBytes));
    if (sms == 0) {
        int dev = 0, count = 148;
        FMB_CUDA_CHECK(cudaGetDevice(&dev));
        FMB_CUDA_CHECK(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev));
        sms = count;
    }
    WeightArgs a{hidden, image, out, limit, limit_offset, rows, n_paths, error_word, row_index};
    const int tiles = (rows + kWeightTile - 1) / kWeightTile;
    const int ctas = max_ctas > 0 && max_ctas < sms ? max_ctas : sms;
    k_radial_weights<<<tiles < ctas ? tiles : ctas, kFusedThreads, kWeightBytes, stream>>>(a);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

int tp_fused_forward(const FusedArgs& f, cudaStream_t stream) {
    if (!f.image || f.lin < 1 || f.lin > 2) return FMB_ERR_UNSUPPORTED;
    if (f.n_rows <= 0) return FMB_OK;
    return f.lin == 1 ? launch_fused<1>(f, stream) : launch_fused<2>(f, stream);
}


}  // namespace fmb
