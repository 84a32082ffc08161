// Warp-specialised tcgen05 / TMEM GEMM (3xTF32) for the per-irrep linears, the species skip and the first-layer
// fold: C[r, :] (+)= A[r, :] * W with strided rows (GemmArgs), N a multiple of 128, K a multiple of 32.
//
// The first tensor-core GEMM of this library (gemm_tc.cu) stages both operands through registers with all threads and
// then issues its MMAs, so every K chunk pays a global-memory round trip in series (measured: 6,000 of the 7,500
// cycles a 64-wide chunk takes are spent waiting for the loads). Here the roles are split:
//   * the weights never pass through registers: their tf32 value / remainder parts are packed at load time into the
//     K-major 128-byte-swizzled operand layout, 32 KB per (128 columns, 32 K) piece, and one thread brings the pieces
//     in with bulk copies that complete on an mbarrier;
//   * four loader warps hold the activation rows of the next K chunk in registers while they split and store the
//     current one, so the loads of chunk k + 1 are in flight during chunk k;
//   * the same thread that issues the bulk copies issues the MMAs (M = 128 rows, N = 128, K = 8 each; 12 per chunk)
//     and commits them to the stage's `empty` barrier; after the last chunk it commits to the accumulator barrier and
//     the loader warps turn into the epilogue (strided rows, accumulate, species mask): the accumulator rows are
//     turned through shared memory so that every store instruction writes one whole row.
// One CTA computes one 128 x 128 tile of C; up to eight problems share a launch. Waits are bounded (tc::mbar_wait).
// A launch with more narrow tiles than the GPU has SMs pairs adjacent column tiles instead (128 x 256 per CTA: two
// weight pieces per stage, N = 256 per MMA): the MMA issue rate, not their width, bounds the K loop, and the activation
// rows are loaded and split once instead of twice.

#include "gemm.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <cstdlib>

namespace fmb {

namespace {

using namespace tc;

constexpr int kWsThreads = 160;          // 4 loader / epilogue warps + the control warp
constexpr int kWsMaxStages = 2;
constexpr int kWsTK = 32;                // K elements per stage
constexpr int kWsPiece = 128 * kWsTK * 4;        // 16 KB: one of the value / remainder parts of an operand stage
// A stage: A value, A remainder, then the W value and W remainder pieces -- one of each for a launch of 128-column
// tiles (64 KB), two of each where column tiles are paired (96 KB). A launch of at most one wave runs two stages per
// CTA; a larger one runs a single stage and, being small, two or three CTAs per SM, so that the tiles of what would
// be the second wave overlap the first instead of waiting for it.
constexpr int kWsTail = 256 + 1024;
constexpr unsigned kWsSpin = 1u << 20;
constexpr int kWsMaxProblems = 8;

struct WsRowMap {
    int nm;
    long long bs, rs;
    __device__ __forceinline__ long long operator()(int r) const {
        return nm == 1 ? (long long)r * bs : (long long)(r / nm) * bs + (long long)(r % nm) * rs;
    }
};

struct WsProblem {
    const float* a;
    const float* img;            // weight image: piece (n tile, k chunk) at float offset (nt * (k / 32) + kc) * 8192
    float* c;
    int m, n, k;
    WsRowMap amap, cmap;
    int accumulate;
    const long long* m_limit;
    long long m_limit_offset;
    const int32_t* batch_species;
    int select;
    int tile_begin;              // first CTA of this problem
};

struct WsBatch {
    WsProblem p[kWsMaxProblems];
    int count;
    int wide;                    // pair adjacent column tiles (128 x 256 per CTA) where a problem has two or more
    int stages;                  // operand stages per CTA (1 or 2)
    uint32_t* error_word;
};

// the loader thread's share of K chunk kc: one float4 of each of 8 rows; the 8 lanes that share a row read the whole
// 128-byte line of the chunk, so a warp instruction touches 4 full lines
__device__ __forceinline__ void ws_fetch(const float* const (&src)[8], const bool (&ok)[8], int kc, int ld_q,
                                         float4 (&out)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
        out[i] = ok[i] ? __ldg(reinterpret_cast<const float4*>(src[i] + kc * kWsTK) + ld_q) : make_float4(0.f, 0.f, 0.f, 0.f);
}

__device__ __forceinline__ void add_to_global(float* dst, const float4& v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// barrier slots: b_full[2], a_full[2], empty[2], acc
constexpr int kWsBFull = 0, kWsAFull = 2, kWsEmpty = 4, kWsAcc = 6;

__global__ void __launch_bounds__(kWsThreads, 3)
k_gemm_ws(const __grid_constant__ WsBatch batch) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int stages = batch.stages;
    const int w_pieces_launch = batch.wide ? 2 : 1;
    const uint32_t stage_bytes = (uint32_t)(2 + 2 * w_pieces_launch) * kWsPiece;
    const uint32_t w_hi_off = 2 * kWsPiece, w_lo_off = (uint32_t)(2 + w_pieces_launch) * kWsPiece;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + stages * stage_bytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int slot) { return bar0 + 8u * (uint32_t)slot; };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef FMB_GEMM_PROFILE
    const long long t_begin = clock64();
    long long t_loop = 0, t_acc = 0;
#endif

    int which = 0;
#pragma unroll
    for (int q = 1; q < kWsMaxProblems; ++q)
        if (q < batch.count && (int)blockIdx.x >= batch.p[q].tile_begin) which = q;
    // every field the loops use is copied to registers (the record is selected with a run-time index)
    const WsProblem& pr = batch.p[which];
    const float* __restrict__ a = pr.a;
    const float* __restrict__ img = pr.img;
    float* const c_out = pr.c;
    const WsRowMap amap = pr.amap, cmap = pr.cmap;
    const int accumulate = pr.accumulate, select = pr.select, k = pr.k;
    const int32_t* const batch_species = pr.batch_species;
    int m = pr.m;
    if (pr.m_limit) {
        const long long lim = *pr.m_limit - pr.m_limit_offset;
        if (lim < m) m = lim < 0 ? 0 : (int)lim;
    }
    const int n128 = pr.n >> 7;
    const int n_wide = batch.wide ? (n128 >> 1) : 0;
    const int per_row_tile = n128 - n_wide;                  // wide pairs first, then the odd narrow tile
    const int local = blockIdx.x - pr.tile_begin;
    const int row0 = (local / per_row_tile) * 128, slot = local % per_row_tile;
    const int nt = slot < n_wide ? 2 * slot : slot + n_wide;   // first 128-column tile of this CTA
    const int tn = slot < n_wide ? 256 : 128;
    if (row0 >= m) return;
    const int chunks = k / kWsTK;

    if (tid == 0) {
        for (int s = 0; s < kWsMaxStages; ++s) {
            mbar_init(bar(kWsBFull + s), 1);
            mbar_init(bar(kWsAFull + s), 4);
            mbar_init(bar(kWsEmpty + s), 1);
        }
        mbar_init(bar(kWsAcc), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t tmem_columns = batch.wide ? 256u : 128u;
    if (warp == 4) tmem_alloc(smem_u32(tmem_slot), tmem_columns);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t stage0 = smem_u32(smem);

    if (warp == 4) {
        if (lane == 0) {
            const uint32_t idesc = tn == 256 ? make_idesc<256>() : make_idesc<128>();
            const size_t piece_floats = 2 * kWsPiece / 4;      // [value 16 KB][remainder 16 KB] of one (n tile, k chunk)
            const float* pieces = img + (size_t)nt * chunks * piece_floats;
            int requested = 0;
            for (int kc = 0; kc < chunks; ++kc) {
                // keep the weight pieces of the next stages on their way
                while (requested < chunks && requested < kc + stages) {
                    const int s = requested % stages;
                    mbar_wait(bar(kWsEmpty + s), ((requested / stages) & 1) ^ 1, abort_flag, kWsSpin);
                    mbar_expect_tx(bar(kWsBFull + s), (tn >> 7) * 2 * kWsPiece);
                    const uint32_t dst = stage0 + s * stage_bytes;
                    for (int half = 0; half < (tn >> 7); ++half) {
                        const float* piece = pieces + ((size_t)half * chunks + requested) * piece_floats;
                        bulk_load(dst + w_hi_off + half * kWsPiece, piece, kWsPiece, bar(kWsBFull + s));
                        bulk_load(dst + w_lo_off + half * kWsPiece, piece + kWsPiece / 4, kWsPiece, bar(kWsBFull + s));
                    }
                    ++requested;
                }
                const int s = kc % stages;
                const uint32_t parity = (kc / stages) & 1;
                mbar_wait(bar(kWsBFull + s), parity, abort_flag, kWsSpin);
                mbar_wait(bar(kWsAFull + s), parity, abort_flag, kWsSpin);
                fence_after_sync();
                const uint32_t base = stage0 + s * stage_bytes;
                const uint64_t a_hi = make_desc(base), a_lo = make_desc(base + kWsPiece);
                const uint64_t w_hi = make_desc(base + w_hi_off), w_lo = make_desc(base + w_lo_off);
#pragma unroll
                for (int k8 = 0; k8 < 4; ++k8)
                    mma_tf32(tmem_base, a_lo + (uint64_t)(2 * k8), w_hi + (uint64_t)(2 * k8), idesc, (kc > 0 || k8 > 0) ? 1 : 0);
#pragma unroll
                for (int k8 = 0; k8 < 4; ++k8) mma_tf32(tmem_base, a_hi + (uint64_t)(2 * k8), w_lo + (uint64_t)(2 * k8), idesc, 1);
#pragma unroll
                for (int k8 = 0; k8 < 4; ++k8) mma_tf32(tmem_base, a_hi + (uint64_t)(2 * k8), w_hi + (uint64_t)(2 * k8), idesc, 1);
                mma_commit(bar(kWsEmpty + s));
            }
            mma_commit(bar(kWsAcc));
        }
    } else {
        // ------------------------------------------------------------------ loaders: a warp takes 32 rows
        const int ld_row = warp * 32 + (lane >> 3), ld_q = lane & 7;
        const float* src[8];
        bool ok[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = row0 + ld_row + 4 * i;
            ok[i] = row < m;
            src[i] = a + (ok[i] ? amap(row) : 0);
        }
        float4 next[8];
        ws_fetch(src, ok, 0, ld_q, next);
        for (int kc = 0; kc < chunks; ++kc) {
            float4 cur[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) cur[i] = next[i];
            if (kc + 1 < chunks) ws_fetch(src, ok, kc + 1, ld_q, next);
            const int s = kc % stages;
            mbar_wait(bar(kWsEmpty + s), ((kc / stages) & 1) ^ 1, abort_flag, kWsSpin);
            uint8_t* hi_tile = smem + s * stage_bytes;
            uint8_t* lo_tile = hi_tile + kWsPiece;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 v = cur[i];
                const float4 hi = make_float4(tf32_rna(v.x), tf32_rna(v.y), tf32_rna(v.z), tf32_rna(v.w));
                const float4 lo = make_float4(tf32_rna(v.x - hi.x), tf32_rna(v.y - hi.y), tf32_rna(v.z - hi.z),
                                              tf32_rna(v.w - hi.w));
                const uint32_t off = tile_offset<128>(ld_row + 4 * i, ld_q * 4);
                *reinterpret_cast<float4*>(hi_tile + off) = hi;
                *reinterpret_cast<float4*>(lo_tile + off) = lo;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kWsAFull + s));
        }
#ifdef FMB_GEMM_PROFILE
        t_loop = clock64();
#endif
        // ------------------------------------------------------------------ epilogue
        // A lane reads its row of the accumulator (lane = row in TMEM), but a row written by its lane alone makes every
        // store instruction touch 32 lines with 16 bytes each (measured 4,500 cycles for 64 KB). The warp's 32 rows go
        // through its own 16 KB of the operand stages instead (free once the accumulator barrier has completed) and
        // leave as whole 512-byte rows, one per instruction.
        const int row_base = row0 + warp * 32;
        const bool mine = row_base + lane < m && !(batch_species && batch_species[(row_base + lane) / cmap.nm] != select);
        const unsigned live = __ballot_sync(0xffffffffu, mine);             // bit rr: row rr of this warp is written
        float4* const turn = reinterpret_cast<float4*>(smem + warp * 16384);      // [32 rows][32 float4], XOR-swizzled
        float* const c_tile = c_out + nt * 128 + 4 * lane;
        const int q0 = row_base / cmap.nm, rem0 = row_base % cmap.nm;
#pragma unroll 1
        for (int c0 = 0; c0 < tn; c0 += 128) {
            if (c0 == 0) {
                mbar_wait(bar(kWsAcc), 0, abort_flag, kWsSpin);
#ifdef FMB_GEMM_PROFILE
                t_acc = clock64();
#endif
                fence_after_sync();
            }
#pragma unroll
            for (int col = 0; col < 128; col += 32) {
                float v[16], u[16];
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c0 + col);
                tmem_load_16x2(taddr, taddr + 16, v, u);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    turn[lane * 32 + (((col >> 2) + q) ^ lane)] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    turn[lane * 32 + (((col >> 2) + 4 + q) ^ lane)] = make_float4(u[4 * q], u[4 * q + 1], u[4 * q + 2], u[4 * q + 3]);
                }
            }
            __syncwarp();
            int q = q0, rem = rem0;
#pragma unroll 8
            for (int rr = 0; rr < 32; ++rr) {
                const float4 v = turn[rr * 32 + (lane ^ rr)];
                if ((live >> rr) & 1u) {
                    float* dst = c_tile + c0 + (long long)q * cmap.bs + (long long)rem * cmap.rs;
                    // accumulate: the add happens at the memory side (every element has one writer, so the sum is the
                    // same old + new as a load and a store would give, without the round trip for the old values)
                    if (accumulate) add_to_global(dst, v);
                    else *reinterpret_cast<float4*>(dst) = v;
                }
                if (++rem == cmap.nm) { rem = 0; ++q; }
            }
            __syncwarp();
        }
    }
#ifdef FMB_GEMM_PROFILE
    if (blockIdx.x == 0 && tid == 0)
        printf("gemm_ws grid %d k %d n %d acc %d | prologue+loop %lld wait_acc %lld epilogue %lld total %lld\n", (int)gridDim.x, k, pr.n,
               accumulate, t_loop - t_begin, t_acc - t_loop, clock64() - t_acc, clock64() - t_begin);
#endif
    fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        if (lane == 0 && *abort_flag && batch.error_word) atomicOr(batch.error_word, FMB_STATUS_TENSOR_TIMEOUT);
        tmem_free(tmem_base, tmem_columns);
    }
}

}  // namespace

int gemm_ws_batch(const GemmArgs* list, int count, cudaStream_t stream) {
    if (count < 1 || count > kWsMaxProblems) return FMB_ERR_UNSUPPORTED;
    WsBatch batch{};
    batch.count = count;
    batch.error_word = list[0].error_word;
    static const int sm_count = [] {
        int device = 0, sms = 148;
        if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        return sms;
    }();
    // launches of more than one wave pair adjacent column tiles (128 x 256): half the CTAs and half the A traffic
    int narrow_tiles = 0;
    for (int q = 0; q < count; ++q) narrow_tiles += ceil_div(std::max(list[q].m, 0), 128) * (list[q].n / 128);
    batch.wide = narrow_tiles > sm_count ? 1 : 0;
    // pairing is for launches whose 128-column tiles would not fit one wave even at three CTAs per SM
    if (batch.wide) {
        bool any_pair = false;
        for (int q = 0; q < count; ++q) any_pair = any_pair || list[q].n >= 256;
        if (!any_pair) batch.wide = 0;
    }
    batch.stages = narrow_tiles > sm_count ? 1 : kWsMaxStages;
    int tiles = 0;
    for (int q = 0; q < count; ++q) {
        const GemmArgs& g = list[q];
        if (!g.b_img || g.n % 128 != 0 || g.k % kWsTK != 0 || g.k < kWsTK) return FMB_ERR_UNSUPPORTED;
        FMB_REQUIRE(g.a && g.c, "gemm_ws: null operand");
        WsProblem& p = batch.p[q];
        p.a = g.a; p.img = g.b_img; p.c = g.c;
        p.m = g.m; p.n = g.n; p.k = g.k;
        p.amap = WsRowMap{g.a_nm, g.a_bs, g.a_rs};
        p.cmap = WsRowMap{g.c_nm, g.c_bs, g.c_rs};
        p.accumulate = g.accumulate;
        p.m_limit = g.m_limit; p.m_limit_offset = g.m_limit_offset;
        p.batch_species = g.batch_species; p.select = g.select;
        p.tile_begin = tiles;
        const int n128 = g.n / 128;
        tiles += ceil_div(std::max(g.m, 0), 128) * (n128 - (batch.wide ? n128 / 2 : 0));
    }
    if (tiles == 0) return FMB_OK;
    const int smem_bytes = batch.stages * (batch.wide ? 6 : 4) * kWsPiece + kWsTail;
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_gemm_ws, kWsMaxStages * 6 * kWsPiece + kWsTail));
    k_gemm_ws<<<tiles, kWsThreads, smem_bytes, stream>>>(batch);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace fmb
