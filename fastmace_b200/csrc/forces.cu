// The energy / forces / stress evaluation: forward through both interaction layers, analytic backward to the edge
// vectors, float64 reductions. Replaces MACEForceField.__call__ (fastmace/model/forces.py:1127-1136,1220-1240) and the
// autograd force/virial path it runs (fastmace/rewrites/engine.py:122-192). Everything is stream-ordered and reads
// the edge count from the device, so the whole call can be captured in a CUDA graph.
//
// Tensor-product weights are materialised per chunk of `chunk_edges` edges (values in the first half of tp_w,
// d/dr in the second half); the backward pass recomputes them chunk by chunk instead of keeping them.

#include "gemm.cuh"
#include "stages.cuh"

#include <cstdlib>

#include <cmath>
#include <algorithm>
#include <vector>

namespace fmb {

namespace {

// Optional per-stage CUDA-event timing of eager (not captured) calls, for the benchmark's roofline figures.
enum Stage { kStEdge = 0, kStRadial, kStTpFwd0, kStTpFwd1, kStLinear, kStSymFwd, kStSymBwd, kStTpBwd1, kStTpBwd0,
             kStReadout, kStages };

struct StageTimer {
    bool on = false;
    struct Span { int stage; cudaEvent_t a, b; };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> pool;
    cudaEvent_t event() {
        if (!pool.empty()) { cudaEvent_t e = pool.back(); pool.pop_back(); return e; }
        cudaEvent_t e;
        cudaEventCreate(&e);
        return e;
    }
} g_timer;

struct StageScope {
    cudaStream_t stream;
    cudaEvent_t b = nullptr;
    StageScope(cudaStream_t s, int stage) : stream(s) {
        if (!g_timer.on) return;
        cudaEvent_t a = g_timer.event();
        b = g_timer.event();
        cudaEventRecord(a, stream);
        g_timer.spans.push_back({stage, a, b});
    }
    ~StageScope() {
        if (b) cudaEventRecord(b, stream);
    }
};

// A second stream per device for the radial-weight producer: its output depends only on the edge features, so it runs
// beside the first interaction's node kernels (forward) and beside the readout / product / contraction adjoints
// (backward), which are latency-bound launches of a few dozen CTAs. Created on the first eager call; captured calls
// record the fork / join as graph dependencies.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr, join_tangent = nullptr;
    // A phased force call (fmb_forces_phase) starts the producers in phase 0 and waits for them in phase 1. Several
    // ranks played on one device share this stream: their workspaces are listed, and as the stream runs in order, the
    // latest `join_tangent` stands for every producer started before it.
    std::vector<const fmb_work_t*> phased;
};

SideStream* side_stream(cudaStream_t main) {
    static SideStream per_device[16];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
    SideStream& s = per_device[dev];
    if (!s.stream) {
        cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(main, &status) != cudaSuccess || status != cudaStreamCaptureStatusNone) return nullptr;
        if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) { s.stream = nullptr; return nullptr; }
        if (cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join_tangent, cudaEventDisableTiming) != cudaSuccess) {
            s.stream = nullptr;
            return nullptr;
        }
    }
    return &s;
}

bool overlap_enabled() { return !g_timer.on; }       // the stage timers attribute time on one stream

inline int dim_of(int lmax) { return (lmax + 1) * (lmax + 1); }

// K-contiguous message layout: per output irrep l the block starts at component base[l] and holds (2l+1) rows of
// segs[l] * C values.
struct MidLayout {
    int base[4];
    int segs[4];
    int mid_dim;
};

MidLayout mid_layout(int l_in_max) {
    // paths of a node irrep set 0..l_in_max with harmonics 0..3 into 0..3, natural parity: count per output l
    MidLayout m{};
    int comp = 0;
    for (int lo = 0; lo <= 3; ++lo) {
        int segs = 0;
        for (int li = 0; li <= l_in_max; ++li)
            for (int le = 0; le <= 3; ++le)
                if (std::abs(li - le) <= lo && lo <= li + le && ((li + le + lo) % 2 == 0)) ++segs;
        m.base[lo] = comp;
        m.segs[lo] = segs;
        comp += segs * (2 * lo + 1);
    }
    m.mid_dim = comp;
    return m;
}

struct Ctx {
    const fmb_model_t* m;
    const fmb_nl_t* nl;
    const fmb_work_t* w;
    cudaStream_t stream;
    int n;               // atoms of the list
    int n0;              // atoms that get first-layer rows (owned + inner halo; = n without domain decomposition)
    int n1;              // owned atoms: last-layer rows and energy
    int hidden_dim;      // components of h after layer 0
    long long count_cap; // entries of the edge buffers
    int n_chunks;
    long long chunk;
    cudaEvent_t radial_ready = nullptr;   // set when the radial weights of this pass are being produced on the side stream
    bool exchange = false;                // halo-exchange mode: rows [n0, n) of x arrive from other ranks between phases
};

// When the whole edge list is one chunk, the last interaction's radial weights written by the forward pass are still
// in tp_w when its adjoint runs (the reassociated first layer never touches tp_w), so the adjoint only adds their d/dr.
// The forward pass then takes the unfused route (GEMM + tensor-product kernel) so that the weights exist; with more
// than one chunk the fused kernel runs instead and the adjoint recomputes both per chunk. The rows of the forward pass
// (n1) and of the adjoint (n0) must be the same prefix of the list: true without decomposition and for a rank of a
// halo-exchange run, not for the ghost-shell scheme (n1 < n0).
bool keeps_forward_weights(const Ctx& c, int layer) {
    return c.n_chunks == 1 && layer > 0 && layer == c.m->n_layers - 1 && c.m->layer[0].first[0] != nullptr &&
           c.n0 == c.n1;
}

// Per-edge hand-over adjoint (adjoint_edges.cu) instead of the mirror evaluation: the buffers exist and the first
// interaction is in its reassociated form (its per-edge kernel closes the chain).
bool edge_local_adjoint(const Ctx& c) {
    return c.w->mirror && c.w->edge_q && c.w->edge_dx && c.m->n_layers == 2 && c.m->layer[0].first[0] != nullptr;
}

float* h_of(const Ctx& c, int layer) {
    return layer == 0 ? c.w->h : c.w->h + (long long)c.n * c.hidden_dim * kC;
}
float* msg_of(const Ctx& c, int layer) { return c.w->msg + (long long)layer * c.n * kNSH * kC; }
const float* hidden_of(const Ctx& c, int layer, int tangent) {
    return c.w->edge_hidden + ((long long)(2 * layer + tangent) * c.count_cap) * kRadial;
}

// limits[0] = edges whose receiver gets first-layer rows, limits[1] = edges whose receiver is owned (the list is
// receiver-sorted, so both are prefixes); without domain decomposition both equal the edge count
__global__ void k_edge_limits(const int32_t* __restrict__ row_ptr, int n0, int n1, long long* __restrict__ limits) {
    limits[0] = row_ptr[n0];
    limits[1] = row_ptr[n1];
}

long long* edge_limits(const Ctx& c) { return reinterpret_cast<long long*>(c.w->partial + 4096); }
// every atom gets every row: both limits are the edge count itself and nothing has to be computed
bool plain_rows(const Ctx& c) { return c.n0 == c.n && c.n1 == c.n; }
const long long* edge_limit(const Ctx& c, int which) {
    return plain_rows(c) ? (const long long*)c.nl->count : edge_limits(c) + which;
}

// One row of radial weights per pair of opposite edges (they have the same length): the whole list is one chunk whose
// weights are kept, the per-edge adjoint's mirror map exists, and the kernels that read the rows by slot are the ones
// that run (node l_max 1, tensor-core producer).
bool pair_rows(const Ctx& c) {
    const int last = c.m->n_layers - 1;
    return last > 0 && keeps_forward_weights(c, last) && edge_local_adjoint(c) && c.w->edge_slot && c.w->canon_list &&
           c.w->canon_count && c.m->layer[last].l_in_max == 1 && c.m->layer[last].rad_img != nullptr;
}

// rows of each half of tp_w (values, then d/dr)
long long weight_rows(const Ctx& c) { return c.w->pair_capacity > 0 ? (long long)c.w->pair_capacity : c.chunk; }

// first .. last: 0 = values, 1 = their d/dr (second half of tp_w)
// `stream` / `max_ctas`: the producer can run on the side stream with fewer CTAs than SMs (it is one persistent CTA per
// SM with all of its shared and tensor memory, so the SMs it leaves free are what the kernels beside it run on)
int radial_weights(const Ctx& c, int layer, long long e0, int first, int last, const long long* limit,
                   cudaStream_t stream = nullptr, int max_ctas = 0) {
    const fmb_layer_t& L = c.m->layer[layer];
    long long rows = std::min<long long>(c.chunk, c.count_cap - e0);
    if (c.w->pair_capacity > 0) {
        FMB_REQUIRE(layer == c.m->n_layers - 1 && pair_rows(c),
                    "forces: tp_w is sized for one row per pair of opposite edges, which this call cannot use");
        rows = std::min<long long>(rows, c.w->pair_capacity);
    }
    if (!stream) stream = c.stream;
    StageScope scope(stream, kStRadial);
    if (L.rad_img && tensor_cores_enabled()) {
        // the fused kernels' tensor-core pipeline as a plain producer (one launch per matrix)
        const bool pairs = layer == c.m->n_layers - 1 && pair_rows(c);
        if (pairs) limit = c.w->canon_count;              // the listed edges, one row each
        bool done = true;
        for (int tangent = first; tangent <= last && done; ++tangent) {
            const int rc = radial_weights_tc(hidden_of(c, layer, tangent) + e0 * kRadial, L.rad_img,
                                             c.w->tp_w + (long long)tangent * weight_rows(c) * L.n_paths * kC, (int)rows, L.n_paths,
                                             limit, e0, pairs ? c.w->canon_list : nullptr, c.w->status, max_ctas, stream);
            if (rc == FMB_ERR_UNSUPPORTED) done = false;
            else if (rc) return rc;
        }
        if (done) return FMB_OK;
    }
    GemmArgs list[2];
    const int count = last - first + 1;
    for (int tangent = first; tangent <= last; ++tangent) {
        GemmArgs& g = list[tangent - first];
        g.a = hidden_of(c, layer, tangent) + e0 * kRadial;
        g.a_bs = kRadial;
        g.b = L.rad_w[3];
        if (L.tc[0]) {
            g.bt_hi = L.tc[0];
            g.bt_lo = L.tc[0] + (long long)kRadial * L.n_paths * kC;
        }
        g.error_word = c.w->status;
        g.c = c.w->tp_w + (long long)tangent * weight_rows(c) * L.n_paths * kC;
        g.c_bs = (long long)L.n_paths * kC;
        g.m = (int)rows;
        g.n = L.n_paths * kC;
        g.k = kRadial;
        g.m_limit = limit;
        g.m_limit_offset = e0;
    }
    return gemm_batch(list, count, stream);
}

// A group of independent per-irrep linears that go out as one launch.
struct LinearBatch {
    GemmArgs list[32];
    int count = 0;
};

// `twin`, `img`: bases of the weight array's tensor-core twin and image (or null); the block's part starts at twice its
// float offset in both
void block_linear(LinearBatch& batch, const Ctx& c, int rows, const float* in, long long in_atom, long long in_off, int k,
                  const float* base, const float* twin, const float* img, long long w_off, float* out, long long out_atom,
                  long long out_off, int n_out, int l, int accumulate, const int32_t* batch_species = nullptr,
                  int select = -1) {
    GemmArgs& g = batch.list[batch.count++];
    const int nm = 2 * l + 1;
    g.a = in + in_off;
    g.a_nm = nm; g.a_bs = in_atom; g.a_rs = k;
    g.b = base + w_off;
    if (twin) {
        g.bt_hi = twin + 2 * w_off;
        g.bt_lo = g.bt_hi + (long long)k * n_out;
    }
    if (img) g.b_img = img + 2 * w_off;
    g.error_word = c.w->status;
    g.c = out + out_off;
    g.c_nm = nm; g.c_bs = out_atom; g.c_rs = n_out;
    g.m = rows * nm; g.n = n_out; g.k = k;
    g.accumulate = accumulate;
    g.batch_species = batch_species;
    g.select = select;
}

int run_linears(const Ctx& c, LinearBatch& batch) {
    if (batch.count == 0) return FMB_OK;
    StageScope scope(c.stream, kStLinear);
    const int rc = gemm_batch(batch.list, batch.count, c.stream);
    batch.count = 0;
    return rc;
}

long long lin_weight_offset(const MidLayout& ml, int l) {
    long long off = 0;
    for (int q = 0; q < l; ++q) off += (long long)ml.segs[q] * kC * kC;
    return off;
}

#define FMB_TRY(expr)            \
    do {                         \
        const int rc__ = (expr); \
        if (rc__) return rc__;   \
    } while (0)

// x = linear_up(h_{layer-1}) for the rows this rank computes; in halo-exchange mode this closes the first phase, so that
// the rows of the halo atoms can be fetched from their owners before the tensor product reads them
void queue_linear_up(LinearBatch& lb, const Ctx& c, int layer) {
    const fmb_layer_t& L = c.m->layer[layer];
    const int in_dim = dim_of(L.l_in_max);
    const float* h_in = h_of(c, layer - 1);
    for (int l = 0; l <= L.l_in_max; ++l)
        block_linear(lb, c, c.n0, h_in, (long long)c.hidden_dim * kC, (long long)l * l * kC, kC, L.w_up, L.tc[1], L.tc_img[1],
                     (long long)l * kC * kC, c.w->x, (long long)in_dim * kC, (long long)l * l * kC, kC, l, 0);
}

int forward_layer(const Ctx& c, int layer, bool with_up = true) {
    const fmb_layer_t& L = c.m->layer[layer];
    const MidLayout ml = mid_layout(L.l_in_max);
    FMB_REQUIRE(ml.mid_dim == L.mid_dim, "forward: message layout mismatch");
    const int in_dim = dim_of(L.l_in_max), out_dim = dim_of(L.l_out_max);
    float* h_out = h_of(c, layer);
    const float* x = nullptr;
    const int rows = layer == 0 ? c.n0 : c.n1;     // atoms that get this layer's outputs
    LinearBatch lb;
    if (layer == 0) {
        FMB_TRY(fill_from_species(rows, out_dim * kC, c.w->species, L.sc_species, h_out, c.stream));
        x = L.x_species;
    } else {
        const float* h_in = h_of(c, layer - 1);
        const int h_in_dim = c.hidden_dim;
        // species-dependent skip: one row-masked GEMM per present species and irrep, each row written exactly once
        for (int l = 0; l <= L.skip_lmax; ++l)
            for (int z = 0; z < c.m->n_species; ++z)
                block_linear(lb, c, rows, h_in, (long long)h_in_dim * kC, (long long)l * l * kC, kC, L.w_skip, L.tc[3], L.tc_img[3],
                             ((long long)l * c.m->n_species + z) * kC * kC, h_out, (long long)out_dim * kC,
                             (long long)l * l * kC, kC, l, 0, c.w->species, z);
        if (with_up) queue_linear_up(lb, c, layer);
        FMB_TRY(run_linears(c, lb));
        x = c.w->x;
    }
    float* msg = msg_of(c, layer);
    const bool reassociated = layer == 0 && L.first[0] != nullptr;
    if (reassociated) {
        // outer products per receiver and sender species, then one GEMM per output irrep straight to the message
        const int nz = c.m->n_species;
        {
            FirstArgs f{};
            f.n_rows = rows; f.n_species = nz; f.count = (const long long*)c.nl->count;
            f.row_ptr = c.nl->edge_row_ptr; f.senders = c.nl->edge_index; f.species = c.w->species;
            f.edge_sh = c.w->edge_sh; f.hidden = hidden_of(c, 0, 0); f.s = c.w->mid;
            StageScope scope(c.stream, kStTpFwd0);
            FMB_TRY(first_accumulate_launch(f, c.stream));
        }
        const long long s_atom = (long long)kNSH * nz * kRadial;
        for (int l = 0; l <= 3; ++l)
            block_linear(lb, c, rows, c.w->mid, s_atom, (long long)l * l * nz * kRadial, nz * kRadial, L.first[0],
                         L.first[2], L.first_img[0], (long long)l * nz * kRadial * kC, msg, (long long)kNSH * kC,
                         (long long)l * l * kC, kC, l, 0);
        FMB_TRY(run_linears(c, lb));
    } else {
    bool fused = false;
    if (layer > 0 && L.rad_img && tensor_cores_enabled() && !keeps_forward_weights(c, layer)) {
        // last radial layer inside the tensor-product kernel: no per-edge weight matrix, one launch for all rows
        FusedArgs f{};
        f.lin = L.l_in_max; f.n_rows = rows; f.row_ptr = c.nl->edge_row_ptr; f.senders = c.nl->edge_index;
        f.x = x; f.edge_sh = c.w->edge_sh; f.hidden = hidden_of(c, layer, 0); f.image = L.rad_img; f.mid = c.w->mid;
        f.error_word = c.w->status;
        StageScope scope(c.stream, kStTpFwd1);
        const int rc = tp_fused_forward(f, c.stream);
        if (rc != FMB_ERR_UNSUPPORTED) {
            if (rc) return rc;
            fused = true;
        }
    }
    for (int k = 0; k < c.n_chunks && !fused; ++k) {
        const long long e0 = (long long)k * c.chunk;
        if (c.radial_ready && layer > 0) {
            FMB_CUDA_CHECK(cudaStreamWaitEvent(c.stream, c.radial_ready, 0));     // produced beside the first interaction
        } else {
            FMB_TRY(radial_weights(c, layer, e0, 0, 0, edge_limit(c, layer == 0 ? 0 : 1)));
        }
        TpArgs t{};
        t.lin = L.l_in_max; t.species_x = layer == 0; t.n_atoms = c.n; t.n_rows = rows;
        t.chunk_e0 = e0; t.chunk_edges = c.chunk; t.whole_list = c.n_chunks == 1; t.error_word = c.w->status;
        t.count = (const long long*)c.nl->count; t.row_ptr = c.nl->edge_row_ptr; t.senders = c.nl->edge_index;
        t.species = c.w->species; t.x = x; t.edge_sh = c.w->edge_sh; t.tp_w = c.w->tp_w; t.mid = c.w->mid;
        if (layer == c.m->n_layers - 1 && pair_rows(c)) { t.mirror = c.w->mirror; t.slot = c.w->edge_slot; }
        StageScope scope(c.stream, layer == 0 ? kStTpFwd0 : kStTpFwd1);
        FMB_TRY(tp_forward_launch(t, c.stream));
    }
    for (int l = 0; l <= 3; ++l)
        block_linear(lb, c, rows, c.w->mid, (long long)ml.mid_dim * kC, (long long)ml.base[l] * kC, ml.segs[l] * kC, L.w_lin,
                     L.tc[5], L.tc_img[5], lin_weight_offset(ml, l), msg, (long long)kNSH * kC, (long long)l * l * kC, kC, l, 0);
    FMB_TRY(run_linears(c, lb));
    }
    {
        StageScope scope(c.stream, kStSymFwd);
        FMB_TRY(symcon_forward(rows, L.n_sc_terms, out_dim, L.sc_terms, L.sc_coef, c.w->species, msg, c.w->basis,
                               c.w->symcon_groups, c.w->n_symcon_groups, c.stream));
    }
    for (int l = 0; l <= L.l_out_max; ++l)
        block_linear(lb, c, rows, c.w->basis, (long long)out_dim * kC, (long long)l * l * kC, kC, L.w_prod, L.tc[7], L.tc_img[7],
                     (long long)l * kC * kC, h_out, (long long)out_dim * kC, (long long)l * l * kC, kC, l, 1);
    FMB_TRY(run_linears(c, lb));
    return FMB_OK;
}

// d_h_out: gradient of this layer's output features [n][out_dim][C]. Produces d_x (layer >= 1) and the force / virial
// contributions; for layer >= 1 also adds the skip and linear_up terms into d_h_in.
// The adjoint of linear_up: d_h_in += d_x W_up^T for the rows this rank computes (after the halo atoms' shares of d_x
// have come back from the ranks that hold them as ghosts, in halo-exchange mode).
int backward_linear_up(const Ctx& c, int layer, float* d_h_in) {
    const fmb_layer_t& L = c.m->layer[layer];
    const int in_dim = dim_of(L.l_in_max);
    LinearBatch lb;
    for (int l = 0; l <= L.l_in_max; ++l)
        block_linear(lb, c, c.n0, c.w->d_x, (long long)in_dim * kC, (long long)l * l * kC, kC, L.w_up_t, L.tc[2], L.tc_img[2],
                     (long long)l * kC * kC, d_h_in, (long long)c.hidden_dim * kC, (long long)l * l * kC, kC, l, 1);
    return run_linears(c, lb);
}

int backward_layer(const Ctx& c, int layer, const float* d_h_out, float* d_h_in, int first_layer_of_pass,
                   bool with_up = true) {
    const fmb_layer_t& L = c.m->layer[layer];
    const MidLayout ml = mid_layout(L.l_in_max);
    const int in_dim = dim_of(L.l_in_max), out_dim = dim_of(L.l_out_max);
    const int rows = layer == 0 ? c.n0 : c.n1;     // atoms whose outputs of this layer carry a gradient
    (void)in_dim;
    LinearBatch lb;
    for (int l = 0; l <= L.l_out_max; ++l)
        block_linear(lb, c, rows, d_h_out, (long long)out_dim * kC, (long long)l * l * kC, kC, L.w_prod_t, L.tc[8], L.tc_img[8],
                     (long long)l * kC * kC, c.w->d_basis, (long long)out_dim * kC, (long long)l * l * kC, kC, l, 0);
    if (layer > 0) {
        for (int l = 0; l <= L.skip_lmax; ++l)
            for (int z = 0; z < c.m->n_species; ++z)
                block_linear(lb, c, rows, d_h_out, (long long)out_dim * kC, (long long)l * l * kC, kC, L.w_skip_t, L.tc[4], L.tc_img[4],
                             ((long long)l * c.m->n_species + z) * kC * kC, d_h_in, (long long)c.hidden_dim * kC,
                             (long long)l * l * kC, kC, l, 1, c.w->species, z);
    }
    FMB_TRY(run_linears(c, lb));
    {
        StageScope scope(c.stream, kStSymBwd);
        FMB_TRY(symcon_backward(rows, L.n_sc_terms, out_dim, L.sc_terms, L.sc_coef, c.w->species, msg_of(c, layer),
                                c.w->d_basis, c.w->d_msg, c.w->symcon_groups, c.w->n_symcon_groups, c.stream));
    }
    if (layer == 0 && L.first[0] != nullptr) {
        // reassociated first layer: gradient of the outer-product sums, then the per-edge kernel
        const int nz = c.m->n_species;
        const long long s_atom = (long long)kNSH * nz * kRadial;
        for (int l = 0; l <= 3; ++l)
            block_linear(lb, c, rows, c.w->d_msg, (long long)kNSH * kC, (long long)l * l * kC, kC, L.first[1], L.first[3], L.first_img[1],
                         (long long)l * nz * kRadial * kC, c.w->d_mid, s_atom, (long long)l * l * nz * kRadial,
                         nz * kRadial, l, 0);
        FMB_TRY(run_linears(c, lb));
        FirstArgs f{};
        // halo-exchange mode: the halo rows' edges belong to other ranks and are skipped altogether
        f.n_rows = c.exchange ? rows : c.n; f.n_valid = rows; f.fresh_from = c.n0; f.n_species = nz;
        f.count = (const long long*)c.nl->count; f.row_ptr = c.nl->edge_row_ptr; f.senders = c.nl->edge_index;
        f.species = c.w->species; f.edge_sh = c.w->edge_sh; f.edge_vec = c.w->edge_vec;
        f.hidden = hidden_of(c, 0, 0); f.hidden_tangent = hidden_of(c, 0, 1); f.d_s = c.w->d_mid;
        f.force_acc = c.w->force_acc; f.atom_virial = c.w->atom_virial; f.first_layer_of_pass = first_layer_of_pass;
        StageScope scope(c.stream, kStTpBwd0);
        if (edge_local_adjoint(c)) {
            // the later interaction has written the edge-vector gradients of the rows below n0; add this one's and
            // turn the per-edge gradients into forces and virials
            FMB_TRY(first_adjoint_edges(f, first_layer_of_pass ? 0 : c.n0, c.w->edge_q, c.stream));
            FMB_TRY(force_gather(c.n, c.exchange ? rows : c.n, c.nl->edge_row_ptr, c.nl->edge_index, c.w->mirror,
                                 c.w->edge_q, c.w->edge_vec, c.w->force_acc, c.w->atom_virial, c.stream));
            return FMB_OK;
        }
        FMB_TRY(first_backward_launch(f, c.stream));
        return FMB_OK;
    }
    for (int l = 0; l <= 3; ++l)
        block_linear(lb, c, rows, c.w->d_msg, (long long)kNSH * kC, (long long)l * l * kC, kC, L.w_lin_t, L.tc[6], L.tc_img[6],
                     lin_weight_offset(ml, l), c.w->d_mid, (long long)ml.mid_dim * kC, (long long)ml.base[l] * kC,
                     ml.segs[l] * kC, l, 0);
    FMB_TRY(run_linears(c, lb));
    if (layer > 0 && edge_local_adjoint(c)) {
        EdgeAdjointArgs t{};
        t.lin = L.l_in_max; t.n_atoms = c.n; t.n_rows = c.n0; t.n_valid = rows; t.count = (const long long*)c.nl->count;
        t.n_gather = c.exchange ? c.n : c.n0;      // halo atoms collect their shares too: they go back to their owners
        t.row_ptr = c.nl->edge_row_ptr; t.senders = c.nl->edge_index; t.mirror = c.w->mirror; t.x = c.w->x;
        t.edge_sh = c.w->edge_sh; t.edge_vec = c.w->edge_vec; t.tp_w = c.w->tp_w;
        t.tangent_offset = weight_rows(c) * L.n_paths * kC; t.d_mid = c.w->d_mid; t.dxe = c.w->edge_dx; t.qe = c.w->edge_q;
        t.d_x = c.w->d_x; t.whole_list = c.n_chunks == 1; t.error_word = c.w->status;
        if (layer == c.m->n_layers - 1 && pair_rows(c)) t.slot = c.w->edge_slot;
        for (int k = 0; k < c.n_chunks; ++k) {
            const long long e0 = (long long)k * c.chunk;
            if (c.radial_ready) {
                FMB_CUDA_CHECK(cudaStreamWaitEvent(c.stream, c.radial_ready, 0));
            } else {
                FMB_TRY(radial_weights(c, layer, e0, keeps_forward_weights(c, layer) ? 1 : 0, 1, edge_limit(c, 0)));
            }
            t.chunk_e0 = e0; t.chunk_edges = c.chunk;
            StageScope scope(c.stream, kStTpBwd1);
            FMB_TRY(tp_adjoint_edges(t, c.stream));
        }
        {
            StageScope scope(c.stream, kStTpBwd1);
            FMB_TRY(gather_sender_gradient(t, c.stream));
        }
        if (with_up) FMB_TRY(backward_linear_up(c, layer, d_h_in));
        return FMB_OK;
    }
    FMB_REQUIRE(!c.exchange, "halo-exchange mode needs the per-edge hand-over buffers (mirror, edge_q, edge_dx)");
    for (int k = 0; k < c.n_chunks; ++k) {
        const long long e0 = (long long)k * c.chunk;
        if (c.radial_ready && layer > 0) {
            FMB_CUDA_CHECK(cudaStreamWaitEvent(c.stream, c.radial_ready, 0));
        } else {
            FMB_TRY(radial_weights(c, layer, e0, keeps_forward_weights(c, layer) ? 1 : 0, 1,
                                   layer == 0 ? (const long long*)c.nl->count : edge_limit(c, 0)));
        }
        TpArgs t{};
        t.lin = L.l_in_max; t.species_x = layer == 0; t.n_atoms = c.n;
        // every atom that sends into a row with a gradient gets a force; first-layer senders are all atoms
        t.n_rows = layer == 0 ? c.n : c.n0; t.n_valid = rows; t.fresh_from = layer == 0 ? c.n0 : 0;
        t.chunk_e0 = e0; t.chunk_edges = c.chunk; t.tangent_offset = weight_rows(c) * L.n_paths * kC;
        t.count = (const long long*)c.nl->count; t.row_ptr = c.nl->edge_row_ptr; t.senders = c.nl->edge_index;
        t.species = c.w->species; t.x = layer == 0 ? L.x_species : c.w->x;
        t.edge_sh = c.w->edge_sh; t.edge_vec = c.w->edge_vec; t.tp_w = c.w->tp_w;
        t.d_mid = c.w->d_mid; t.d_x = c.w->d_x; t.force_acc = c.w->force_acc; t.atom_virial = c.w->atom_virial;
        t.first_layer_of_pass = first_layer_of_pass; t.error_word = c.w->status;
        StageScope scope(c.stream, layer == 0 ? kStTpBwd0 : kStTpBwd1);
        FMB_TRY(tp_backward_launch(t, c.stream));
    }
    if (layer > 0 && with_up) FMB_TRY(backward_linear_up(c, layer, d_h_in));
    return FMB_OK;
}

int make_ctx(Ctx& c, const fmb_model_t* m, const fmb_nl_t* nl, const fmb_work_t* w, cudaStream_t stream) {
    FMB_REQUIRE(m && nl && w, "forces: null argument");
    FMB_REQUIRE(m->channels == kC && m->n_layers == 2 && m->radial_width == kRadial && m->n_bessel == kBessel &&
                    m->cutoff_p == 5 && m->mlp_hidden == 16,
                "forces: unsupported model shape (128 channels, 2 layers, 8 Bessel, p = 5, 64-wide radial MLP)");
    FMB_REQUIRE(m->n_species >= 1 && m->n_species <= FMB_MAX_SPECIES, "forces: too many species");
    FMB_REQUIRE(w->n_atoms == nl->n_atoms && w->edge_capacity == nl->capacity, "forces: workspace / list mismatch");
    FMB_REQUIRE(w->chunk_edges > 0, "forces: chunk_edges must be positive");
    c.m = m; c.nl = nl; c.w = w; c.stream = stream;
    c.n = w->n_atoms;
    c.n1 = w->n_energy_atoms < 0 ? c.n : w->n_energy_atoms;      // negative: not restricted
    c.n0 = w->n_inner_atoms < 0 ? c.n : w->n_inner_atoms;
    FMB_REQUIRE(c.n1 > 0, "forces: no owned atoms (a rank without owned atoms skips the call)");
    FMB_REQUIRE(c.n1 <= c.n0 && c.n0 <= c.n, "forces: owned <= inner <= all atoms");
    c.exchange = w->halo_exchange != 0;
    if (c.exchange) {
        FMB_REQUIRE(c.n0 == c.n1, "halo-exchange mode: the rows of both interactions are the owned atoms");
        FMB_REQUIRE(w->mirror && w->edge_q && w->edge_dx && m->layer[0].first[0] != nullptr,
                    "halo-exchange mode needs the per-edge hand-over buffers and the reassociated first interaction");
    }
    c.hidden_dim = dim_of(m->hidden_lmax);
    c.count_cap = nl->capacity;
    c.chunk = std::min<long long>(w->chunk_edges, nl->capacity);
    c.n_chunks = ceil_div(nl->capacity, c.chunk);
    return FMB_OK;
}

double cell_volume(const fmb_nl_t* nl) {
    const double* m = nl->cell;
    return std::fabs(m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) +
                     m[2] * (m[3] * m[7] - m[4] * m[6]));
}

}  // namespace

}  // namespace fmb

using namespace fmb;

extern "C" FMB_API int fmb_edge_features(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work,
                                 const double* positions, fmb_stream_t stream) {
    FMB_REQUIRE(model && nl && work && positions, "fmb_edge_features: null argument");
    StageScope scope((cudaStream_t)stream, kStEdge);
    // halo-exchange mode: only the edges into owned atoms are evaluated on this rank (a prefix of the receiver-sorted
    // list, limits[0] = row_ptr[owned atoms])
    const long long* limit = nullptr;
    if (work->halo_exchange) {
        Ctx c;
        FMB_TRY(make_ctx(c, model, nl, work, (cudaStream_t)stream));
        k_edge_limits<<<1, 1, 0, c.stream>>>(nl->edge_row_ptr, c.n0, c.n1, edge_limits(c));
        FMB_LAUNCH_CHECK();
        limit = edge_limits(c);
    }
    const int rc = edge_features(model, nl, work, positions, limit, (cudaStream_t)stream);
    if (rc) return rc;
    // opposite-edge map for the per-edge adjoint (the compaction reorders edges every step)
    if (work->mirror && work->edge_q && work->edge_dx) {
        Ctx c;
        FMB_TRY(make_ctx(c, model, nl, work, (cudaStream_t)stream));
        const bool pairs = pair_rows(c);
        return mirror_map(nl, work->mirror, work->status, limit ? limit : (const long long*)nl->count,
                          pairs ? work->edge_slot : nullptr, work->canon_list, work->canon_count,
                          work->pair_capacity > 0 ? work->pair_capacity : nl->capacity, (cudaStream_t)stream);
    }
    return FMB_OK;
}

// Starts the radial-weight producer of the last interaction (values: which = 0, d/dr: which = 1) on the side stream
// when the pass will use kept weights (one chunk, no domain restriction); the layer code then waits for it instead of
// launching it. `tangent_too` (forward pass of a whole force call): the d/dr producer follows the value producer on the
// side stream at once and `tangent_ready` is what the adjoint waits for -- beside the forward tensor product it costs
// little, beside the adjoint's node kernels it took 120 of their SMs.
int fork_radial(Ctx& c, int which, bool tangent_too = false, cudaEvent_t* tangent_ready = nullptr) {
    const int layer = c.m->n_layers - 1;
    if (!overlap_enabled() || !keeps_forward_weights(c, layer) || !c.m->layer[layer].rad_img || !tensor_cores_enabled())
        return FMB_OK;
    SideStream* side = side_stream(c.stream);
    if (!side) return FMB_OK;
    constexpr int side_ctas = 136;      // the SMs it leaves free serve the node kernels beside it (104 .. 148 measure alike)
    FMB_CUDA_CHECK(cudaEventRecord(side->fork, c.stream));
    FMB_CUDA_CHECK(cudaStreamWaitEvent(side->stream, side->fork, 0));
    FMB_TRY(radial_weights(c, layer, 0, which, which, edge_limit(c, which == 0 ? 1 : 0), side->stream, side_ctas));
    FMB_CUDA_CHECK(cudaEventRecord(side->join, side->stream));
    c.radial_ready = side->join;
    if (tangent_too && which == 0 && tangent_ready) {
        FMB_TRY(radial_weights(c, layer, 0, 1, 1, edge_limit(c, 0), side->stream, side_ctas));
        FMB_CUDA_CHECK(cudaEventRecord(side->join_tangent, side->stream));
        *tangent_ready = side->join_tangent;
    }
    return FMB_OK;
}

namespace {

int forward_pass(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, cudaStream_t stream,
                 cudaEvent_t* tangent_ready) {
    Ctx c;
    FMB_TRY(make_ctx(c, model, nl, work, stream));
    if (!plain_rows(c)) {
        k_edge_limits<<<1, 1, 0, c.stream>>>(nl->edge_row_ptr, c.n0, c.n1, edge_limits(c));
        FMB_LAUNCH_CHECK();
    }
    FMB_TRY(fork_radial(c, 0, tangent_ready != nullptr, tangent_ready));
    FMB_TRY(forward_layer(c, 0));
    FMB_TRY(forward_layer(c, 1));
    // readout; the gradient of the last layer's scalars is parked in `basis` (free after the forward pass)
    StageScope scope(c.stream, kStReadout);
    FMB_TRY(readout(model, c.n0, c.n1, h_of(c, 0), h_of(c, 1), work->node_energy, work->d_h, work->basis, c.stream));
    return FMB_OK;
}

// `tangent_ready`: set by a forward pass of the same call that has already started the d/dr producer (the edge limits
// it wrote are still valid too)
int backward_pass(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, cudaStream_t stream,
                  cudaEvent_t tangent_ready) {
    Ctx c;
    FMB_TRY(make_ctx(c, model, nl, work, stream));
    if (tangent_ready) {
        c.radial_ready = tangent_ready;
    } else {
        if (!plain_rows(c)) {
            k_edge_limits<<<1, 1, 0, c.stream>>>(nl->edge_row_ptr, c.n0, c.n1, edge_limits(c));
            FMB_LAUNCH_CHECK();
        }
        FMB_TRY(fork_radial(c, 1));
    }
    FMB_TRY(backward_layer(c, 1, work->basis, work->d_h, 1));
    FMB_TRY(backward_layer(c, 0, work->d_h, nullptr, 0));
    StageScope scope(c.stream, kStReadout);
    FMB_TRY(reduce_outputs(model, work, c.n1, cell_volume(nl), c.stream));
    return FMB_OK;
}

}  // namespace

extern "C" FMB_API int fmb_forward(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, fmb_stream_t stream) {
    return forward_pass(model, nl, work, (cudaStream_t)stream, nullptr);
}

extern "C" FMB_API int fmb_backward(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, fmb_stream_t stream) {
    return backward_pass(model, nl, work, (cudaStream_t)stream, nullptr);
}

extern "C" FMB_API int fmb_forces_phase(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work,
                                        const double* positions, int phase, fmb_stream_t stream) {
    FMB_REQUIRE(work && work->halo_exchange, "fmb_forces_phase: the workspace is not in halo-exchange mode");
    FMB_REQUIRE(phase >= 0 && phase <= 2, "fmb_forces_phase: phase is 0, 1 or 2");
    Ctx c;
    if (phase == 0) {
        FMB_REQUIRE(positions, "fmb_forces_phase: phase 0 needs the positions");
        FMB_TRY(fmb_edge_features(model, nl, work, positions, stream));
        FMB_TRY(make_ctx(c, model, nl, work, (cudaStream_t)stream));
        // the radial weights of the second interaction and their d/dr, beside the first interaction (the edge limits
        // are in place: the edge kernel's call computed them)
        cudaEvent_t tangent = nullptr;
        FMB_TRY(fork_radial(c, 0, true, &tangent));
        if (c.radial_ready && tangent) side_stream(c.stream)->phased.push_back(work);
        c.radial_ready = nullptr;
        FMB_TRY(forward_layer(c, 0));
        LinearBatch lb;
        queue_linear_up(lb, c, 1);
        return run_linears(c, lb);
    }
    FMB_TRY(make_ctx(c, model, nl, work, (cudaStream_t)stream));
    if (phase == 1) {
        SideStream* side = side_stream(c.stream);
        bool started = false;
        bool alone = false;
        if (side) {
            auto it = std::find(side->phased.begin(), side->phased.end(), work);
            if (it != side->phased.end()) {
                started = true;
                alone = side->phased.size() == 1;
                side->phased.erase(it);
            }
        }
        if (started) c.radial_ready = alone ? side->join : side->join_tangent;
        FMB_TRY(forward_layer(c, 1, false));
        {
            StageScope scope(c.stream, kStReadout);
            FMB_TRY(readout(model, c.n0, c.n1, h_of(c, 0), h_of(c, 1), work->node_energy, work->d_h, work->basis, c.stream));
        }
        c.radial_ready = started ? side->join_tangent : nullptr;
        return backward_layer(c, 1, work->basis, work->d_h, 1, false);
    }
    FMB_TRY(backward_linear_up(c, 1, work->d_h));
    FMB_TRY(backward_layer(c, 0, work->d_h, nullptr, 0));
    StageScope scope(c.stream, kStReadout);
    return reduce_outputs(model, work, c.n1, cell_volume(nl), c.stream);
}

extern "C" FMB_API int fmb_forces(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, const double* positions,
                          fmb_stream_t stream) {
    if (work && work->halo_exchange) {
        // no other rank: the three phases back to back (the halo rows of x and d_x are then the caller's business)
        for (int phase = 0; phase < 3; ++phase) FMB_TRY(fmb_forces_phase(model, nl, work, positions, phase, stream));
        return FMB_OK;
    }
    FMB_TRY(fmb_edge_features(model, nl, work, positions, stream));
    cudaEvent_t tangent_ready = nullptr;
    FMB_TRY(forward_pass(model, nl, work, (cudaStream_t)stream, &tangent_ready));
    FMB_TRY(backward_pass(model, nl, work, (cudaStream_t)stream, tangent_ready));
    return FMB_OK;
}

extern "C" FMB_API int fmb_gemm(const float* a, const float* b, const float* bt_hi, const float* bt_lo, float* c, int m,
                                int n, int k, int accumulate, int impl, uint32_t* status, fmb_stream_t stream) {
    GemmArgs g;
    g.a = a; g.b = b; g.bt_hi = bt_hi; g.bt_lo = bt_lo; g.error_word = status; g.c = c; g.m = m; g.n = n; g.k = k;
    g.a_bs = k; g.c_bs = n; g.accumulate = accumulate;
    if (impl == 2) {
        g.b_img = bt_hi;
        return gemm_ws_batch(&g, 1, (cudaStream_t)stream);
    }
    return impl == 1 ? gemm_tc(g, (cudaStream_t)stream) : gemm_simt(g, (cudaStream_t)stream);
}

extern "C" FMB_API int fmb_commit_forces(const fmb_work_t* work, double* forces64, double* energy64, double* stress64,
                                 fmb_stream_t stream) {
    FMB_REQUIRE(work && forces64 && energy64, "fmb_commit_forces: null argument");
    return commit_forces(work, forces64, energy64, work->compute_stress ? stress64 : nullptr, (cudaStream_t)stream);
}

extern "C" FMB_API int fmb_profile_enable(int on) {
    g_timer.on = on != 0;
    return FMB_OK;
}

extern "C" FMB_API int fmb_profile_read(float* ms, int* spans, int n) {
    FMB_REQUIRE(ms && spans && n >= kStages, "fmb_profile_read: need room for every stage");
    for (int k = 0; k < n; ++k) { ms[k] = 0.0f; spans[k] = 0; }
    for (auto& span : g_timer.spans) {
        FMB_CUDA_CHECK(cudaEventSynchronize(span.b));
        float t = 0.0f;
        FMB_CUDA_CHECK(cudaEventElapsedTime(&t, span.a, span.b));
        ms[span.stage] += t;
        spans[span.stage] += 1;
        g_timer.pool.push_back(span.a);
        g_timer.pool.push_back(span.b);
    }
    g_timer.spans.clear();
    return kStages;
}
