// tcgen05 / TMEM GEMM in 3xTF32 split precision for sm_100a: C[M, N] (+)= A[M, K] * B[K, N] with fp32-level accuracy.
//
// Every fp32 operand is split as x = hi + lo with hi = tf32(x), lo = tf32(x - hi); the product is accumulated as
// A_lo*B_hi + A_hi*B_lo + A_hi*B_hi in the fp32 TMEM accumulator (the reference's split-precision GEMMs do the same on
// mma.sync: fastmace/kernels/cutlass/tf32x3_sm80.cu:1-24). The weights are static, so their split, transposed
// (K-major) copies are made once at packing time; the activations are split on their way into shared memory.
//
// One CTA (128 threads) owns a 128-row tile of A and walks the N tiles (64 columns each): operands sit in shared
// memory in the K-major layout with 128-byte swizzle (written by the staging stores), one elected
// thread issues tcgen05.mma (M = 128, N = 64, K = 8 per instruction), completion arrives on an mbarrier through
// tcgen05.commit, and the four warps read their TMEM lane quadrants back with tcgen05.ld for the epilogue (strided
// rows, accumulate, species mask -- the same GemmArgs contract as the SIMT kernel). Two CTAs of 8 warps fit per SM
// (96 KB shared memory, 128 TMEM columns each).
//
// Every wait is bounded: if the mbarrier does not flip within the spin limit the CTA raises the error word, skips the
// remaining work, frees its TMEM and returns.

#include "gemm.cuh"

#include <algorithm>
#include <cstdlib>

namespace fmb {

namespace {

constexpr int TM = 128;          // rows per CTA tile (UMMA M)
// UMMA N (the 64-, 128- or 256-row operand) is a template parameter: a 128x64x8 tf32 MMA occupies the tensor core for
// about as long as a 128x256x8 one (measured: ~128 cycles per instruction at N = 64), so wide tiles are what reach
// the tensor peak; narrow ones are kept for small N.
constexpr int TK = 64;           // K elements staged per chunk
constexpr int kThreads = 256;      // 8 warps: two per TMEM lane quadrant, each taking half of a tile's columns
constexpr unsigned kSpinLimit = 1u << 24;

constexpr int kTileBytesA = TM * TK * 4;   // 32 KB (one of hi / lo)
template <int TN> constexpr int smem_bytes() { return 2 * kTileBytesA + 2 * TN * TK * 4 + 64 + 1024; }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major tiles with the 128-byte swizzle the tensor core reads at full rate: a [rows][64] fp32 tile is stored as two
// K halves of [rows][32] (128-byte rows, 1024-byte groups of 8 rows); inside a row the 16-byte chunk index is XORed
// with (row mod 8). (The unswizzled interleaved layout works too, but each MMA then fetches its operands 16 bytes at
// a time: the first version of this kernel spent ~400 cycles per 128x64x8 MMA that way.)
template <int ROWS>
__device__ __forceinline__ uint32_t tile_offset(int row, int k) {
    const int half = k >> 5, chunk = (k >> 2) & 7;
    return (uint32_t)(half * (ROWS * 128) + (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4) + (k & 3) * 4);
}

// shared-memory matrix descriptor (sm_100): start address (16-byte units), stride between 8-row groups 1024 bytes,
// leading-dimension offset unused for swizzled K-major operands (1), descriptor version 1, layout 128-byte swizzle
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// descriptor increment (in 16-byte units) of K step k8 (8 elements = 32 bytes) inside a [ROWS][64] tile
template <int ROWS>
__device__ __forceinline__ uint64_t k_step(int k8) {
    return (uint64_t)(((k8 >> 2) * (ROWS * 128) + (k8 & 3) * 32) >> 4);
}

// instruction descriptor: D fp32, A and B tf32, both K-major, N = TN, M = 128
template <int TN>
__device__ __forceinline__ uint32_t make_idesc() {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}

__device__ __forceinline__ float tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

struct RowMap {
    int nm;
    long long bs, rs;
    __device__ __forceinline__ long long operator()(int r) const {
        return nm == 1 ? (long long)r * bs : (long long)(r / nm) * bs + (long long)(r % nm) * rs;
    }
};

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// One GEMM of a batched launch.
struct Problem {
    const float* a;
    const float* bt_hi;
    const float* bt_lo;
    float* c;
    int m, n, k;
    RowMap amap, cmap;
    int accumulate;
    const long long* m_limit;
    long long m_limit_offset;
    const int32_t* batch_species;
    int select;
    int n_split;        // CTAs along N per row tile
    int tile_begin;     // first CTA of this problem in the launch
};

constexpr int kMaxProblems = 8;

struct Batch {
    Problem p[kMaxProblems];
    int count;
    uint32_t* error_word;
};

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}

// Software pipeline per CTA: the operands of work item i+1 (one 64-wide K chunk of one 64-column tile) are fetched
// into registers while the tensor cores work on item i, and the accumulator of the previous column tile is read back
// and stored while the current tile's MMAs run (two TMEM accumulators of 64 columns).
//
// SWAP = true computes the same product with the roles of the tensor-core operands exchanged (C^T = B^T A^T): the
// 128-row operand is a tile of the pre-split weights (resident, K = 64 only), the 64-row operand a tile of activation
// rows, and accumulator lane = output column. A warp then stores 128 contiguous bytes of one output row per
// instruction, which is what the wide radial-weight outputs ([edges][P*C]) need; without the swap every lane would
// write into a different row.
template <bool SWAP, int TN>
__global__ void __launch_bounds__(kThreads, TN <= 64 ? 2 : 1)
k_gemm_tc(const __grid_constant__ Batch batch) {
    constexpr int kTileBytesB = TN * TK * 4;
    constexpr int kTmemCols = 2 * TN;          // two accumulators
    constexpr int kRowSteps = TN / 64;         // staging steps of the TN-row operand (64 rows per step)
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzle atoms are 1024-byte aligned
    uint8_t* a_hi = smem;
    uint8_t* a_lo = smem + kTileBytesA;
    uint8_t* b_hi = smem + 2 * kTileBytesA;
    uint8_t* b_lo = b_hi + kTileBytesB;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(b_lo + kTileBytesB);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 1);

    int which = 0;
#pragma unroll
    for (int q = 1; q < kMaxProblems; ++q)
        if (q < batch.count && (int)blockIdx.x >= batch.p[q].tile_begin) which = q;
    const Problem& pr = batch.p[which];
    int m = pr.m;
    if (pr.m_limit) {
        long long lim = *pr.m_limit - pr.m_limit_offset;
        if (lim < m) m = lim < 0 ? 0 : (int)lim;
    }
    const int local = blockIdx.x - pr.tile_begin;
    // SWAP: row0 is the first output COLUMN of this CTA's 128-wide tile and the 64-wide tiles walk output rows
    const int row0 = (local / pr.n_split) * TM;
    if (!SWAP && row0 >= m) return;
    const int n_tiles_host = SWAP ? (pr.m + TN - 1) / TN : pr.n / TN;
    const int n_tiles = SWAP ? (m + TN - 1) / TN : pr.n / TN;
    const int per = (n_tiles_host + pr.n_split - 1) / pr.n_split;
    const int nt_begin = (local % pr.n_split) * per;
    const int nt_end = min(n_tiles, nt_begin + per);
    if (nt_begin >= nt_end) return;
    const int k = pr.k, k_chunks = k / TK;
    // Everything the loops read from the problem record is copied into registers here: the record is selected with a
    // run-time index, and reading its fields in the inner loops made the first version of this kernel five times slower.
    float* const c_out = pr.c;
    const RowMap cmap = pr.cmap;
    const RowMap amap = pr.amap;
    const int accumulate = pr.accumulate;
    const int32_t* const batch_species = pr.batch_species;
    const int select = pr.select;
    const float* __restrict__ a = pr.a;
    const float* __restrict__ bt_hi = pr.bt_hi;
    const float* __restrict__ bt_lo = pr.bt_lo;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef FMB_GEMM_PROFILE
    long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long t_begin = clock64();
#define GP0() const long long gp__ = clock64()
#define GP1(slot) prof[slot] += clock64() - gp__
#else
#define GP0()
#define GP1(slot)
#endif

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(mbar)), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = make_idesc<TN>();
    const uint32_t bar = smem_u32(mbar);
    uint32_t phase = 0;
    bool failed = false;
    // descriptors of the four operand tiles
    const uint64_t desc_ah = make_desc(smem_u32(a_hi)), desc_al = make_desc(smem_u32(a_lo));
    const uint64_t desc_bh = make_desc(smem_u32(b_hi)), desc_bl = make_desc(smem_u32(b_lo));

    // staging map: 8 rows x 4 sixteen-byte quads per warp step (64-byte runs per row, conflict-free 512-byte stores)
    const int ld_row = warp * 8 + (lane & 7);     // + 64 * i
    const int ld_q = lane >> 3;                    // + 4 * j
    const bool a_resident = k_chunks == 1;

    float4 ra[TM / 64][TK / 16];
    float4 rbh[kRowSteps][TK / 16], rbl[SWAP ? 1 : kRowSteps][TK / 16];

    auto fetch_a = [&](int kc) {
#pragma unroll
        for (int i = 0; i < TM / 64; ++i) {
            const int row = ld_row + 64 * i;
            const bool ok = row0 + row < m;
            const float* src = a + (ok ? amap(row0 + row) : 0) + kc * TK;
#pragma unroll
            for (int j = 0; j < TK / 16; ++j)
                ra[i][j] = ok ? __ldg(reinterpret_cast<const float4*>(src) + ld_q + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto split_store = [&](const float4 v, uint8_t* hi_tile, uint8_t* lo_tile, uint32_t off) {
        const float4 hi = make_float4(tf32_rna(v.x), tf32_rna(v.y), tf32_rna(v.z), tf32_rna(v.w));
        const float4 lo = make_float4(tf32_rna(v.x - hi.x), tf32_rna(v.y - hi.y), tf32_rna(v.z - hi.z),
                                      tf32_rna(v.w - hi.w));
        *reinterpret_cast<float4*>(hi_tile + off) = hi;
        *reinterpret_cast<float4*>(lo_tile + off) = lo;
    };
    auto store_a = [&]() {
#pragma unroll
        for (int i = 0; i < TM / 64; ++i)
#pragma unroll
            for (int j = 0; j < TK / 16; ++j)
                split_store(ra[i][j], a_hi, a_lo, tile_offset<TM>(ld_row + 64 * i, (ld_q + 4 * j) * 4));
    };
    // SWAP: the resident 128-row tile is a block of the pre-split weights, copied as it is
    auto stage_weights_128 = [&]() {
#pragma unroll
        for (int i = 0; i < TM / 64; ++i) {
            const long long src = (long long)(row0 + ld_row + 64 * i) * k;
#pragma unroll
            for (int j = 0; j < TK / 16; ++j) {
                const uint32_t off = tile_offset<TM>(ld_row + 64 * i, (ld_q + 4 * j) * 4);
                *reinterpret_cast<float4*>(a_hi + off) = __ldg(reinterpret_cast<const float4*>(bt_hi + src) + ld_q + 4 * j);
                *reinterpret_cast<float4*>(a_lo + off) = __ldg(reinterpret_cast<const float4*>(bt_lo + src) + ld_q + 4 * j);
            }
        }
    };
    auto fetch_b = [&](int nt, int kc) {
#pragma unroll
        for (int i = 0; i < kRowSteps; ++i) {
            if (SWAP) {
                const int row = nt * TN + ld_row + 64 * i;             // an activation row (output row)
                const bool ok = row < m;
                const float* src = a + (ok ? amap(row) : 0) + kc * TK;
#pragma unroll
                for (int j = 0; j < TK / 16; ++j)
                    rbh[i][j] = ok ? __ldg(reinterpret_cast<const float4*>(src) + ld_q + 4 * j)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            } else {
                const long long src = (long long)(nt * TN + ld_row + 64 * i) * k + kc * TK;
#pragma unroll
                for (int j = 0; j < TK / 16; ++j) {
                    rbh[i][j] = __ldg(reinterpret_cast<const float4*>(bt_hi + src) + ld_q + 4 * j);
                    rbl[SWAP ? 0 : i][j] = __ldg(reinterpret_cast<const float4*>(bt_lo + src) + ld_q + 4 * j);
                }
            }
        }
    };
    auto store_b = [&]() {
#pragma unroll
        for (int i = 0; i < kRowSteps; ++i)
#pragma unroll
            for (int j = 0; j < TK / 16; ++j) {
                const uint32_t off = tile_offset<TN>(ld_row + 64 * i, (ld_q + 4 * j) * 4);
                if (SWAP) {
                    split_store(rbh[i][j], b_hi, b_lo, off);
                } else {
                    *reinterpret_cast<float4*>(b_hi + off) = rbh[i][j];
                    *reinterpret_cast<float4*>(b_lo + off) = rbl[SWAP ? 0 : i][j];
                }
            }
    };
    // Accumulator rows live one per thread (TMEM lane); warps w and w + 4 share a lane quadrant and take half of the
    // tile's columns each, 32 at a time.
    auto epilogue = [&](int nt) {
        const int quadrant = warp & 3, half = warp >> 2;
        const int row = row0 + quadrant * 32 + lane;
#pragma unroll
        for (int cc = 0; cc < TN / 64; ++cc) {
            const int col_in_tile = half * (TN / 2) + cc * 32;
            const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)((nt & 1) * TN + col_in_tile);
            uint32_t v[32];
            tmem_load_32(taddr, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (SWAP) {
                // lane = output column `row`; v[j] belongs to output row nt * TN + col_in_tile + j. Plain rows
                // (c_nm == 1, checked on the host): one pointer walks down the column with the row stride.
                const int out_row0 = nt * TN + col_in_tile;
                const long long ldc = cmap.bs;
                float* d = c_out + row + (long long)out_row0 * ldc;
                const int live = m - out_row0;          // rows of this chunk that exist
                if (accumulate) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < live) *d += __uint_as_float(v[j]);
                        d += ldc;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < live) *d = __uint_as_float(v[j]);
                        d += ldc;
                    }
                }
            } else if (row < m && !(batch_species && batch_species[row / cmap.nm] != select)) {
                float4* dst = reinterpret_cast<float4*>(c_out + cmap(row) + nt * TN + col_in_tile);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float4 o = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                           __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                    if (accumulate) {
                        const float4 old = dst[q];
                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    dst[q] = o;
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

#ifdef FMB_GEMM_PROFILE
    prof[6] = clock64() - t_begin;      // set-up: alloc, barrier, descriptors
#endif
    if (SWAP) {
        stage_weights_128();
    } else if (a_resident) {
        fetch_a(0);
        store_a();
    } else {
        fetch_a(0);
    }
    fetch_b(nt_begin, 0);
    bool in_flight = false;
    int pending_tile = -1;          // column tile whose accumulator is complete once the MMAs in flight finish
    for (int nt = nt_begin; nt < nt_end && !failed; ++nt) {
        for (int kc = 0; kc < k_chunks; ++kc) {
            if (in_flight) {
                GP0();
                if (!mbar_wait(bar, phase)) failed = true;
                phase ^= 1;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                GP1(0);
            }
            {
                GP0();
                if (!SWAP && !a_resident) store_a();
                store_b();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                GP1(1);
            }
            {
                GP0();
                const int any = __syncthreads_or(failed ? 1 : 0);
                GP1(2);
                if (any) { failed = true; break; }
            }
            if (tid == 0) {
                GP0();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + (uint32_t)((nt & 1) * TN);
#pragma unroll
                for (int term = 0; term < 3; ++term) {
                    const uint64_t aa = term == 0 ? desc_al : desc_ah;
                    const uint64_t bb = term == 1 ? desc_bl : desc_bh;
#pragma unroll
                    for (int k8 = 0; k8 < TK / 8; ++k8) {
                        const int acc = (kc > 0 || term > 0 || k8 > 0) ? 1 : 0;
                        mma_tf32(tmem_d, aa + k_step<TM>(k8), bb + k_step<TN>(k8), idesc, acc);
                    }
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                             :: "r"(bar) : "memory");
                GP1(3);
            }
            in_flight = true;
            // fetch the next item's operands while the tensor cores run
            int nkc = kc + 1, nnt = nt;
            if (nkc == k_chunks) { nkc = 0; nnt = nt + 1; }
            if (nnt < nt_end) {
                if (!SWAP && !a_resident) fetch_a(nkc);
                fetch_b(nnt, nkc);
            }
            // the previous column tile finished before this item was issued: store it now
            if (kc == 0 && pending_tile >= 0) {
                epilogue(pending_tile);
                pending_tile = -1;
            }
            if (kc == k_chunks - 1) pending_tile = nt;
        }
    }
    if (!failed && in_flight) {
        if (!mbar_wait(bar, phase)) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    if (__syncthreads_or(failed ? 1 : 0)) failed = true;
    {
        GP0();
        if (!failed && pending_tile >= 0) epilogue(pending_tile);
        GP1(5);
    }
#ifdef FMB_GEMM_PROFILE
    if (blockIdx.x == 0 && (tid == 0 || tid == 64))
        printf("gemm<%d,%d> tid %d total %lld | setup %lld wait %lld store %lld sync %lld issue %lld epilogue %lld\n", (int)SWAP, TN,
               tid, clock64() - t_begin, prof[6], prof[0], prof[1], prof[2], prof[3], prof[5]);
#endif
    if (failed && tid == 0 && batch.error_word) atomicOr(batch.error_word, FMB_STATUS_TENSOR_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}


template <bool SWAP, int TN>
int launch(const Batch& batch, int tiles, cudaStream_t stream) {
    FMB_CUDA_CHECK(opt_in_shared_memory((const void*)k_gemm_tc<SWAP, TN>, smem_bytes<TN>()));
    k_gemm_tc<SWAP, TN><<<tiles, kThreads, smem_bytes<TN>(), stream>>>(batch);
    FMB_LAUNCH_CHECK();
    return FMB_OK;
}

}  // namespace

int gemm_tc_batch(const GemmArgs* list, int count, cudaStream_t stream) {
    if (count < 1 || count > kMaxProblems) return FMB_ERR_UNSUPPORTED;
    Batch batch{};
    batch.count = count;
    batch.error_word = list[0].error_word;
    int tiles = 0, sms = 148;
    for (int q = 0; q < count; ++q) {
        const GemmArgs& g = list[q];
        if (!g.bt_hi || !g.bt_lo) return FMB_ERR_UNSUPPORTED;
        if (g.n % 64 != 0 || g.k % TK != 0 || g.k < TK) return FMB_ERR_UNSUPPORTED;
        FMB_REQUIRE(g.a && g.c, "gemm_tc: null operand");
    }
    // Wide outputs of a single K chunk (the radial weights) run with the operand roles swapped and 256 rows per MMA;
    // the others take 128-column tiles when N allows. All problems of a launch must agree.
    auto wants_swap = [](const GemmArgs& g) {
        return g.k == TK && g.n % TM == 0 && g.n >= 4 * TM && !g.batch_species && g.m >= 4 * TM && g.c_nm == 1 &&
               g.a_nm == 1;
    };
    const bool swap = wants_swap(list[0]);
    bool wide = true;
    for (int q = 0; q < count; ++q) {
        if (wants_swap(list[q]) != swap) return FMB_ERR_UNSUPPORTED;
        if (list[q].n % 128 != 0) wide = false;
    }
    const int tn = swap ? 256 : (wide ? 128 : 64);
    long long row_tiles_total = 0;
    for (int q = 0; q < count; ++q) row_tiles_total += ceil_div(std::max(list[q].m, 0), TM);
    for (int q = 0; q < count; ++q) {
        const GemmArgs& g = list[q];
        Problem& p = batch.p[q];
        p.a = g.a; p.bt_hi = g.bt_hi; p.bt_lo = g.bt_lo; p.c = g.c;
        p.m = g.m; p.n = g.n; p.k = g.k;
        p.amap = RowMap{g.a_nm, g.a_bs, g.a_rs};
        p.cmap = RowMap{g.c_nm, g.c_bs, g.c_rs};
        p.accumulate = g.accumulate;
        p.m_limit = g.m_limit; p.m_limit_offset = g.m_limit_offset;
        p.batch_species = g.batch_species; p.select = g.select;
        p.tile_begin = tiles;
        if (swap) {
            // CTA = (128-column tile, a run of about four 256-row tiles)
            const int row_tiles = ceil_div(std::max(g.m, 0), tn);
            p.n_split = std::max(1, ceil_div(row_tiles, 4));
            tiles += (g.n / TM) * p.n_split;
        } else {
            // split the column tiles over several CTAs when there are too few row tiles to fill the GPU
            const int n_tiles = g.n / tn;
            int split = (n_tiles + 4) / 5;
            if (row_tiles_total < 2 * sms) split = n_tiles;
            p.n_split = std::max(1, std::min(split, n_tiles));
            tiles += ceil_div(std::max(g.m, 0), TM) * p.n_split;
        }
    }
    if (tiles == 0) return FMB_OK;
    if (swap) return launch<true, 256>(batch, tiles, stream);
    if (tn == 128) return launch<false, 128>(batch, tiles, stream);
    return launch<false, 64>(batch, tiles, stream);
}

int gemm_tc(const GemmArgs& g, cudaStream_t stream) {
    if (g.m <= 0) return (g.bt_hi && g.bt_lo) ? FMB_OK : FMB_ERR_UNSUPPORTED;
    return gemm_tc_batch(&g, 1, stream);
}

}  // namespace fmb
