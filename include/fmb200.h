/* fmb200 -- C ABI of the B200-native MACE force path (sm_100a).
 *
 * Every entry point is extern "C", takes plain pointers and sizes, launches on the CUDA stream it is given and
 * returns an int status (FMB_OK or an FMB_ERR_* code); none throws, none allocates device memory unless its comment
 * says so: all device buffers belong to the caller (the Python host allocates them as torch tensors and passes
 * data_ptr()). Device-side failures that cannot be returned synchronously (edge capacity overflow, a neighbour row
 * longer than the sort buffer) set bits in the caller's `status` word on the device; the host reads it when it
 * chooses (the reference's "overflow flag checked before commit", fastmace/engine/graph.py:44-56,586-595).
 *
 * Each function cites the reference interface it replaces (file:line within the FastMACE tree).
 */
#ifndef FMB200_H
#define FMB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FMB_API __attribute__((visibility("default")))
#else
#define FMB_API
#endif

#define FMB_OK 0
#define FMB_ERR_ARG 1       /* bad argument (null pointer, unsupported size) */
#define FMB_ERR_CUDA 2      /* a CUDA call failed; fmb_last_error() has the text */
#define FMB_ERR_UNSUPPORTED 3

/* bits of the device status word */
#define FMB_STATUS_CAND_OVERFLOW 1u   /* more candidate pairs than `capacity` */
#define FMB_STATUS_ROW_OVERFLOW 2u    /* one receiver has more candidates than FMB_MAX_ROW */
#define FMB_STATUS_BIN_OVERFLOW 4u    /* internal: cell-list bins inconsistent */
#define FMB_STATUS_NONFINITE 8u       /* a non-finite energy was produced */
#define FMB_STATUS_TENSOR_TIMEOUT 16u /* a tensor-core kernel gave up waiting for its own MMA completion barrier */
#define FMB_STATUS_NO_MIRROR 32u      /* an edge has no opposite edge: the neighbour list is not a full list */
#define FMB_STATUS_PAIR_OVERFLOW 64u  /* more pairs of opposite edges than tp_w has rows (pair_capacity) */

#define FMB_MAX_ROW 1024              /* candidates per receiver the in-kernel sort can hold */
#define FMB_MAX_LAYERS 2
#define FMB_MAX_SPECIES 8
#define FMB_MAX_PATHS 17

typedef void* fmb_stream_t;           /* a cudaStream_t */

FMB_API int fmb_version(void);
FMB_API const char* fmb_last_error(void);
/* sizeof of the structs below, for the host binding to verify its mirror: which = 0 fmb_nl_t, 1 fmb_model_t,
 * 2 fmb_work_t, 3 fmb_langevin_t */
FMB_API int fmb_sizeof(int which);
/* kernels this library has launched (or captured into a graph) in this process so far */
FMB_API long long fmb_launch_count(void);

/* ------------------------------------------------------------------------------------------------ neighbour list
 * Replaces SkinNeighbourList (fastmace/neighbors/skin.py:164-747) with sort_receivers on and no sender groups.
 * Buffers mirror the reference's names (skin.py:606-621): candidate_index, candidate_unit_shifts, edge_index,
 * unit_shifts, shifts, count, reference_positions, build_cell; plus CSR row pointers the streaming kernels read. */
typedef struct {
    int32_t n_atoms;
    int32_t capacity;                 /* entries of every per-edge buffer */
    double cutoff;
    double skin;
    double cell[9];                   /* build cell, rows are lattice vectors */
    double inverse[9];                /* inverse of the cell */
    int32_t nbins[3];                 /* cell-list bins per axis (fractional slabs at least cutoff+skin thick) */
    int32_t reach_bins[3];            /* stencil half-width per axis */
    float pad_unit_shift[3];          /* padding pair: atom 0 and a far image (skin.py:247-252) */
    int32_t max_bin_atoms;            /* unused by the kernels (bins are walked through bin_start) */
    /* device buffers */
    double* wrapped;                  /* [n_atoms, 3] positions wrapped into the cell */
    double* offsets;                  /* [n_atoms, 3] integer cell of each atom (as double) */
    int32_t* atom_bin;                /* [n_atoms] */
    int32_t* bin_count;               /* [total_bins + 1] */
    int32_t* bin_start;               /* [total_bins + 1] exclusive scan of bin_count */
    int32_t* bin_fill;                /* [total_bins] */
    int32_t* bin_atoms;               /* [n_atoms] atoms ordered by bin */
    int32_t* cand_row_count;          /* [n_atoms + 1] */
    int32_t* cand_row_ptr;            /* [n_atoms + 1] */
    int32_t* candidate_index;         /* [2, capacity] row 0 sender, row 1 receiver */
    float* candidate_unit_shifts;     /* [capacity, 3] */
    int32_t* edge_row_count;          /* [n_atoms + 1] */
    int32_t* edge_row_ptr;            /* [n_atoms + 1] CSR over the compacted edges (by receiver) */
    int32_t* edge_index;              /* [2, capacity] */
    float* unit_shifts;               /* [capacity, 3] */
    float* shifts;                    /* [capacity, 3] */
    int64_t* count;                   /* [1] edges inside the cutoff after compact */
    int64_t* num_candidates;          /* [1] candidates of the last build */
    double* reference_positions;      /* [n_atoms, 3] */
    double* build_cell;               /* [9] */
    int32_t* scan_scratch;            /* [>= 2 * ceil(max(n_atoms, total_bins) / 4096) + 8] */
    uint64_t* max_disp2_bits;         /* [1] bit pattern of max |x - x_ref|^2 (non-negative double) */
    int32_t* rebuild_flag;            /* [1] set by fmb_nl_needs_rebuild */
    uint32_t* status;                 /* [1] FMB_STATUS_* bits */
} fmb_nl_t;

/* skin.py:421-497 (build_gpu): candidates within cutoff + skin, float64 decision, ordered by (receiver, sender,
 * image). If `only_if_flag` is nonzero every kernel returns at once unless *rebuild_flag != 0 (a rebuild inside a
 * captured step). Writes candidate_*, cand_row_ptr, num_candidates, reference_positions, build_cell. */
FMB_API int fmb_nl_build(const fmb_nl_t* nl, const double* positions, int only_if_flag, fmb_stream_t stream);
/* skin.py:702-729 (compact): stable partition, inside-cutoff first; writes edge_index, unit_shifts, shifts, count and
 * edge_row_ptr. */
FMB_API int fmb_nl_compact(const fmb_nl_t* nl, const double* positions, fmb_stream_t stream);
/* No counterpart in the reference. fmb_nl_compact for hosts that cannot hand over scratch memory (a driver whose
 * device pool is frozen once its step graphs exist, a plugin arena that forbids allocation while stepping): the
 * per-receiver counts and scan sums live in one device array inside the library (about 1 MiB per GPU, held until the
 * process exits) and nothing is allocated. nl->edge_row_count and nl->scan_scratch are ignored; everything else is as
 * for fmb_nl_compact. Lists above FMB_STATIC_COMPACT_MAX_ATOMS atoms are refused (FMB_ERR_ARG). The first call on a
 * device resolves the array's address and should be made outside stream capture. All calls on a GPU share the
 * array: run them on one stream (or order them), overlapping calls race. */
#define FMB_STATIC_COMPACT_MAX_ATOMS 262144
FMB_API int fmb_nl_compact_static(const fmb_nl_t* nl, const double* positions, fmb_stream_t stream);
/* skin.py:685-693 (needs_rebuild, fixed cell): rebuild_flag = max_i |x_i - x_ref,i|^2 > (fraction * skin / 2)^2. */
FMB_API int fmb_nl_needs_rebuild(const fmb_nl_t* nl, const double* positions, double fraction, fmb_stream_t stream);

/* ------------------------------------------------------------------------------------------------ model */
typedef struct {
    int32_t l_in_max;                 /* node irreps entering the tensor product: 0..l_in_max */
    int32_t l_out_max;                /* irreps leaving the product block */
    int32_t n_paths;
    int32_t mid_dim;                  /* components per channel of the scattered message */
    int32_t n_sc_terms;               /* polynomial terms of the symmetric contraction */
    int32_t skip_lmax;
    int32_t is_last;
    int32_t pad_;
    const float* rad_w[4];            /* radial MLP, [in][out], 1/sqrt(fan_in) folded */
    const float* x_species;           /* layer 0: linear_up(embedding) per species [n_species][C] */
    const float* sc_species;          /* layer 0: skip connection per species [n_species][out_dim][C] */
    const float* w_up;                /* [l_in_max+1][C][C], 1/sqrt(C) folded */
    const float* w_up_t;              /* transposed */
    const float* w_skip;              /* [skip_lmax+1][n_species][C][C] */
    const float* w_skip_t;
    const float* w_lin;               /* per l_out: [K = n_seg*C][C], norm and 1/avg_num_neighbors folded; l blocks
                                         concatenated in l order */
    const float* w_lin_t;             /* per l_out: [C][K] */
    const float* w_prod;              /* [l_out_max+1][C][C] */
    const float* w_prod_t;
    const int32_t* sc_terms;          /* [n_sc_terms][4]: i, j, k (unused = -1), m_out */
    const float* sc_coef;             /* [n_species][n_sc_terms][C] */
    const float* w_readout;           /* non-last: [C] (scale folded); last: [C][16] then [16] */
    /* tensor-core twins of the GEMM weights, in the order rad_w[3], w_up, w_up_t, w_skip, w_skip_t, w_lin, w_lin_t,
     * w_prod, w_prod_t: for every [K][N] block at float offset o of the array, the twin holds at offset 2 o the
     * transposed block [N][K] rounded to tf32 (hi) followed by the tf32 remainder (lo). Null = SIMT GEMM. */
    const float* tc[9];
    /* First layer only (senders are species-only rows, so the edge side reduces to 64 x 16 outer products per
     * receiver and sender species, fastmace/rewrites/mh1/modules.py:146-160): per output irrep l the matrix
     * [n_species * 64][C] = last radial layer x sender species row x message linear, l blocks concatenated; its
     * transpose [C][n_species * 64] per l; and the tensor-core twins of both. Null = evaluate the first layer like the
     * others. */
    const float* first[4];
    /* Last radial layer as the fused tensor-product kernels stream it into shared memory: for path p, K half h (32 of
     * the 64 hidden features) and part (0 = tf32 remainder, 1 = tf32 value) a 16 KB tile [128 channels][32] of
     * W4^T in the K-major 128-byte-swizzled operand layout, at float offset ((p * 2 + h) * 2 + part) * 4096.
     * Null = materialise the per-edge weights with a GEMM. */
    const float* rad_img;
    /* The tensor-core twins again, packed for bulk copies into shared memory (warp-specialised GEMM): for a [K][N]
     * block at float offset o the image starts at 2 o and holds, for column tile nt (128 columns) and K chunk kc
     * (32 rows of the block) at float offset (nt * (K / 32) + kc) * 8192, the [128][32] tile of the transposed block in
     * the K-major 128-byte-swizzled operand layout: 4,096 tf32 values, then their 4,096 tf32 remainders. Blocks whose
     * N is not a multiple of 128 or whose K is not a multiple of 32 are left zero (the other kernels take them).
     * tc_img[i] belongs to tc[i] (entry 0 unused), first_img[0 / 1] to first[2 / 3]. Null = not packed. */
    const float* tc_img[9];
    const float* first_img[2];
    /* The three hidden layers of the radial MLP (rad_w[0..2]) as operand images for the tcgen05 edge kernel: layer
     * [K][64] -> tile [64 outputs][K] of its transpose, K-major with the 128-byte swizzle in halves of 32 K (2,048
     * floats; the first layer fills 8 of the 32 columns of one half), tf32 values then tf32 remainders; float offsets
     * 0 / 2,048 (first), 4,096 / 8,192 (second), 12,288 / 16,384 (third), 20,480 floats in all. Null on any layer =
     * the warp-level tensor-core kernel evaluates the MLPs from rad_w. */
    const float* mlp_img;
} fmb_layer_t;

typedef struct {
    int32_t n_species;
    int32_t channels;                 /* 128 */
    int32_t hidden_lmax;
    int32_t n_layers;
    int32_t n_bessel;                 /* 8 */
    int32_t cutoff_p;                 /* 5 */
    int32_t radial_width;             /* 64 */
    int32_t mlp_hidden;               /* 16 */
    float r_cut;
    float scale;
    float shift;
    float silu_norm;
    double e0[FMB_MAX_SPECIES];       /* isolated-atom energies of the present species */
    fmb_layer_t layer[FMB_MAX_LAYERS];
} fmb_model_t;

/* Workspace of one force evaluation; every buffer is the caller's. Sizes in floats unless noted. */
typedef struct {
    int32_t n_atoms;
    int32_t edge_capacity;            /* entries of the per-edge buffers */
    int32_t chunk_edges;              /* edges whose tensor-product weights are resident at once */
    int32_t compute_stress;
    const int32_t* species;           /* [n_atoms] index into the present species */
    float* edge_vec;                  /* [edge_capacity][4] unit vector and length */
    float* edge_sh;                   /* [edge_capacity][16] */
    float* edge_hidden;               /* [n_layers][2][edge_capacity][64]: last hidden layer and its d/dr */
    float* tp_w;                      /* [2 * chunk_edges][max_paths * C]: weights, then their d/dr */
    float* x;                         /* [n_atoms][in_dim(1)][C] linear_up output of layer 1 */
    float* mid;                       /* [n_atoms][max mid_dim][C] scattered message (reused by both layers) */
    float* msg;                       /* [n_layers][n_atoms][16][C] */
    float* basis;                     /* [n_atoms][max out_dim][C] symmetric contraction output */
    float* h;                         /* [n_layers][n_atoms][out_dim][C] node features after each layer */
    float* d_h;                       /* [n_atoms][hidden_dim][C] gradient of h1 (and scratch for h2's) */
    float* d_basis;                   /* [n_atoms][max out_dim][C] */
    float* d_msg;                     /* [n_atoms][16][C] */
    float* d_mid;                     /* [n_atoms][max mid_dim][C] */
    float* d_x;                       /* [n_atoms][in_dim(1)][C] */
    float* node_energy;               /* [n_atoms] */
    float* atom_virial;               /* [n_atoms][6] */
    float* force_acc;                 /* [n_atoms][3] */
    double* partial;                  /* [>= 1024 * 8] block partial sums; [4096..4097] hold two int64 edge limits */
    /* outputs */
    double* energy;                   /* [1] */
    float* forces;                    /* [n_atoms][3] */
    float* stress;                    /* [9] */
    uint32_t* status;                 /* [1] */
    /* Domain decomposition (negative = every atom; 0 owned atoms is refused: such a rank has nothing to evaluate and
     * skips the call): the atoms are ordered owned | inner halo | outer halo. Atoms
     * [0, n_energy_atoms) are owned: only they contribute energy and get the last layer's rows; atoms
     * [0, n_inner_atoms) get the first layer's rows (they are senders of owned receivers); the rest only act as
     * species-only senders of the first layer. Forces come out for every atom (partial sums for halo atoms). */
    int32_t n_energy_atoms;
    int32_t n_inner_atoms;
    /* Optional per-edge hand-over buffers of the adjoint (all three or none):
     * mirror [edge_capacity] int32 (index of the opposite edge), edge_q [edge_capacity][4] (gradient of the edge vector),
     * edge_dx [edge_capacity][(hidden_lmax + 1)^2][C] (gradient of the sender's features from that edge). Null = the
     * mirror-evaluation kernels. */
    int32_t* mirror;
    float* edge_q;
    float* edge_dx;
    /* Optional, with the three above: an edge and its opposite edge have the same length, hence the same radial
     * weights, so the last interaction's weights are produced once per pair. canon_list [edge_capacity] int32 lists the
     * edges that stand for their pair (the lower index of the two), canon_count [1] int64 their number, edge_slot
     * [edge_capacity] int32 holds, for a listed edge, its row in tp_w. Written by fmb_edge_features every call. Null =
     * one row of tp_w per edge. */
    int32_t* edge_slot;
    int32_t* canon_list;
    long long* canon_count;
    /* Optional: atoms grouped four at a time by species for the symmetric contraction ([n_symcon_groups][4] atom
     * indices, -1 = empty slot; every atom exactly once; all atoms of a group have the same species). Null = one atom per
     * CTA. */
    const int32_t* symcon_groups;
    int32_t n_symcon_groups;
    /* Halo-exchange mode of a spatially decomposed run (nonzero; needs n_energy_atoms == n_inner_atoms = the owned
     * atoms and the hand-over buffers): the atoms beyond the owned ones are halo atoms that belong to other ranks.
     * Both interactions are evaluated for the owned atoms only; the halo rows of x are written by the caller
     * between phase 0 and phase 1 (fetched from their owners), the halo rows of d_x are read by the caller after
     * phase 1 (returned to their owners, whose rows receive them before phase 2), and forces come out as partial sums
     * for every local atom (the halo atoms' shares go back to their owners). */
    int32_t halo_exchange;
    /* With the pair-row fields above: the rows each half of tp_w holds when it is sized for one row per pair of
     * opposite edges (a little over edge_capacity / 2) instead of chunk_edges rows; 0 = chunk_edges rows. A list with
     * more pairs than that raises FMB_STATUS_PAIR_OVERFLOW and the rows beyond are not produced. */
    int32_t pair_capacity;
    int32_t pad_;
} fmb_work_t;

/* MACEForceField.__call__ (fastmace/model/forces.py:1127-1136,1220-1240): energy (float64), forces and stress of the
 * compacted edges in `nl` at float64 `positions`; analytic backward instead of autograd
 * (fastmace/rewrites/engine.py:122-192 for the definitions). Graph-capturable: no host synchronisation, reads the
 * edge count from the device. */
FMB_API int fmb_forces(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, const double* positions,
               fmb_stream_t stream);

/* fmb_forces in three phases for a workspace in halo-exchange mode; no counterpart in the reference, which runs one
 * structure on one GPU (SPEC.md:70-74; structural precedent: the halo senders of a tile, fastmace/model/tiled.py:1-26).
 * phase 0: edge features of the edges into owned atoms, first interaction, x = linear_up(h1) of the owned atoms;
 * phase 1: second interaction, readouts, its adjoint down to d_x of every local atom;
 * phase 2: adjoint of linear_up and of the first interaction, forces (partial sums), energy and virial of the owned
 *          atoms' edges.
 * `positions` is read by phase 0 only. Each phase is stream-ordered and graph-capturable like fmb_forces. */
FMB_API int fmb_forces_phase(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, const double* positions,
                             int phase, fmb_stream_t stream);

/* Halo-exchange helpers (no counterpart in the reference): out[i] = rows[index[i]] for rows of row_bytes bytes (a
 * multiple of 4): the rows a peer holds as halo atoms, gathered into the send buffer. */
FMB_API int fmb_halo_gather_rows(const void* rows, const int32_t* index, void* out, int n, int row_bytes,
                                 fmb_stream_t stream);
/* dst[target[t]] += sum_{k in [ptr[t], ptr[t+1])} received[source[k]], rows of row_floats floats, summed in the order
 * of k (no atomics): what the peers computed for atoms this rank owns, added into the owners' rows. target null =
 * row t itself. */
FMB_API int fmb_halo_add_rows(const float* received, const int32_t* ptr, const int32_t* source, const int32_t* target,
                              float* dst, int n_targets, int row_floats, fmb_stream_t stream);
/* out [n_owned + n_halo][3] = (owned | received) + shift - origin, float64: the rank's atoms in its own frame (shift
 * [n_owned + n_halo][3]: whole cell vectors that bring an owned atom into the brick and a halo atom to its image). */
FMB_API int fmb_halo_local_positions(const double* owned, int n_owned, const double* received, const double* shift,
                                     int n_halo, const double* origin, double* out, fmb_stream_t stream);
/* forces64[i] = local_forces[i] + sum_{k in [ptr[i], ptr[i+1])} received[source[k]] for the owned atoms (ptr null = no
 * peers): the reverse force accumulation, cast to the float64 state (fastmace/engine/graph.py:1125-1131). */
FMB_API int fmb_halo_owned_forces(const float* local_forces, const float* received, const int32_t* ptr,
                                  const int32_t* source, int n_owned, double* forces64, fmb_stream_t stream);

/* Individual stages, exported for kernel-level parity tests (same arguments as inside fmb_forces). */
FMB_API int fmb_edge_features(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, const double* positions,
                      fmb_stream_t stream);
FMB_API int fmb_forward(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, fmb_stream_t stream);
FMB_API int fmb_backward(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, fmb_stream_t stream);

/* The real spherical harmonics l <= 3 (component normalised, on v / max(|v|, 1e-12)) and, when grad_sh and
 * grad_vectors are given, the gradient of sum(grad_sh * sh) with respect to the vectors, through the same device
 * functions the edge and adjoint kernels call: fastmace/kernels/triton/edge_sh.py:40-78 (edge_sh3) and :82-126 (its
 * backward). vectors [n][3], grad_sh / sh [n][16], grad_vectors [n][3], all fp32 on the device; exported for the
 * parity test against the reference kernel's fixture. */
FMB_API int fmb_harmonics_probe(const float* vectors, const float* grad_sh, float* sh, float* grad_vectors, int n,
                                fmb_stream_t stream);

/* C[M, N] (+)= A[M, K] B[K, N] in fp32; exported for tests. impl 0: SIMT FMA kernel reading b ([K][N]); impl 1:
 * tcgen05 3xTF32 kernel reading bt_hi / bt_lo (B transposed [N][K], split in tf32 hi and lo; K and N multiples of
 * 64), status FMB_ERR_UNSUPPORTED otherwise; impl 2: the warp-specialised tcgen05 kernel, bt_hi pointing at the
 * pre-swizzled weight image (pieces of [128 columns][32 K]: 4,096 tf32 values, then their 4,096 remainders; N a
 * multiple of 128, K of 32), bt_lo unused. `status` (device word, may be null) receives FMB_STATUS_TENSOR_TIMEOUT. */
FMB_API int fmb_gemm(const float* a, const float* b, const float* bt_hi, const float* bt_lo, float* c, int m, int n,
                     int k, int accumulate, int impl, uint32_t* status, fmb_stream_t stream);

/* Per-stage CUDA-event timing of eager (not captured) force calls, the counterpart of the reference's stage
 * breakdown tool (tools/step_breakdown.py: CUDA events around each stage). Stages, in order: edge features, radial
 * weight GEMMs, tensor product forward layer 0 / layer 1, per-irrep linears, symmetric contraction forward /
 * backward, tensor product backward layer 1 / layer 0, readout + reductions. fmb_profile_read synchronises, fills
 * the milliseconds and the number of timed spans per stage since the last read, and returns the stage count. */
FMB_API int fmb_profile_enable(int on);
FMB_API int fmb_profile_read(float* ms, int* spans, int n);

/* ------------------------------------------------------------------------------------------------ Langevin
 * Replaces Langevin.first_half / second_half (fastmace/integrators/langevin.py:233-263) and the fused stage
 * (fastmace/kernels/triton/fused_integrator.py:47-133). All float64. */
typedef struct {
    int32_t n_atoms;
    int32_t fix_com;                  /* 0 off, 1 ASE projection, 2 mass-weighted projection */
    double dt;
    double c1;
    double c2;
    double* positions;                /* [n_atoms, 3] */
    double* velocities;
    const double* forces;
    const double* masses;             /* [n_atoms] */
    const double* c3_unit;            /* [n_atoms] */
    const double* c4_unit;
    const double* c5_unit;
    const double* sqrt_kT;            /* [1] */
    const double* noise;              /* [steps, 2, n_atoms, 3] drawn-ahead batch: xi then eta */
    const int32_t* noise_cursor;      /* [1] row of `noise` this step reads (device counter) */
    double* x_old;
    double* rnd_pos;
    double* rnd_vel;
    double* partial;                  /* [>= 1024 * 8] */
    int32_t* noise_cursor_rw;         /* same address as noise_cursor; incremented by the second half */
} fmb_langevin_t;

FMB_API int fmb_langevin_first_half(const fmb_langevin_t* lv, fmb_stream_t stream);
FMB_API int fmb_langevin_second_half(const fmb_langevin_t* lv, fmb_stream_t stream);
/* No counterpart in the reference (its noise is NumPy's, drawn on the host: langevin.py:224-231). Fills one noise
 * row [2][n_atoms][3] (xi, then eta) with standard normals from Philox4x32-10 keyed by `seed` and indexed by
 * (*step_counter, atom): identical on every GPU that passes the same seed and step, for domain-decomposed runs and for
 * sizes where the host draw of 6 N normals per step would limit the step. */
FMB_API int fmb_langevin_device_noise(double* noise_row, int n_atoms, unsigned long long seed,
                                      const int32_t* step_counter, fmb_stream_t stream);
/* The same generator keyed by atom_ids[i] instead of i: in a spatially decomposed run an atom draws the same numbers
 * whichever rank integrates it (atom_ids = the atoms' indices in the whole system). */
FMB_API int fmb_langevin_device_noise_ids(double* noise_row, int n_atoms, const int32_t* atom_ids, unsigned long long seed,
                                          const int32_t* step_counter, fmb_stream_t stream);
/* fmb_langevin_first_half in two parts for a rank that integrates a part of the system (no counterpart in the
 * reference): fmb_langevin_noise_sums computes the random terms of this rank's atoms and writes the ten sums the
 * centre-of-mass projection needs (sum rnd_pos [3], sum m rnd_pos [3], sum m rnd_vel [3], sum m) to `sums`; the caller
 * adds the ranks' sums; fmb_langevin_first_half_global applies the projection with the system's sums and atom count,
 * then the half kick and the drift (fastmace/integrators/langevin.py:233-257). */
FMB_API int fmb_langevin_noise_sums(const fmb_langevin_t* lv, double* sums, fmb_stream_t stream);
FMB_API int fmb_langevin_first_half_global(const fmb_langevin_t* lv, const double* global_sums, long long n_global,
                                           fmb_stream_t stream);
/* state.forces/energy/stress <- ForceOutput (fastmace/engine/graph.py:1125-1131): fp32 -> float64 copies. */
FMB_API int fmb_commit_forces(const fmb_work_t* work, double* forces64, double* energy64, double* stress64,
                      fmb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
