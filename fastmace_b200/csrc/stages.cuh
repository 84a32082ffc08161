// Internal launch functions shared between the translation units of libfmb200.
#pragma once

#include "fmb_common.cuh"

namespace fmb {

// `count`: device edge count to featurise (null = the list's own count)
int edge_features(const fmb_model_t* model, const fmb_nl_t* nl, const fmb_work_t* work, const double* positions,
                  const long long* count, cudaStream_t stream);

struct TpArgs {
    int lin;
    bool species_x;
    int n_atoms;           // atoms of the list (rows of row_ptr)
    int n_rows;            // receivers this launch computes: [0, n_rows)
    int n_valid;           // backward: atoms [0, n_valid) have a message gradient, the others read as zero
    int fresh_from;        // backward: atoms at or beyond this start their force / virial sums from zero
    long long chunk_e0, chunk_edges, tangent_offset;
    bool whole_list;       // the launch covers the whole edge list (one chunk): the streaming forward kernel applies
    const long long* count;
    const int32_t* row_ptr;
    const int32_t* senders;
    const int32_t* species;
    const float* x;
    const float* edge_sh;
    const float* edge_vec;
    const float* tp_w;
    float* mid;            // forward output
    const float* d_mid;    // backward input
    float* d_x;
    float* force_acc;
    float* atom_virial;
    int first_layer_of_pass;
    uint32_t* error_word;  // device status word for bounded-wait failures of the staged kernels
    const int32_t* mirror; // with `slot`: the weights of edge e are row slot[min(e, mirror[e])] of tp_w (one row per pair)
    const int32_t* slot;
};
int tp_forward_launch(const TpArgs& t, cudaStream_t stream);
int tp_backward_launch(const TpArgs& t, cudaStream_t stream);

// Tensor product of an interaction after the first with the last radial layer fused in (tp_fused.cu): no per-edge
// weight matrix; one launch covers all rows.
struct FusedArgs {
    int lin;
    int n_rows;            // receivers [0, n_rows)
    int n_valid;           // adjoint: atoms [0, n_valid) have a message gradient, the others read as zero
    int fresh_from;        // adjoint: atoms at or beyond this start their force / virial sums from zero
    int first_layer_of_pass;
    const int32_t* row_ptr;
    const int32_t* senders;
    const float* x;                // [atoms][(lin + 1)^2][C]
    const float* edge_sh;
    const float* edge_vec;
    const float* hidden;           // [edges][64] last hidden radial layer of this interaction
    const float* hidden_tangent;   // its derivative with respect to the edge length (adjoint)
    const float* image;            // fmb_layer_t.rad_img
    float* mid;                    // forward output
    const float* d_mid;            // adjoint input
    float* d_x;
    float* force_acc;
    float* atom_virial;
    uint32_t* error_word;
};
// FMB_ERR_UNSUPPORTED when the fused kernels do not apply (no weight image, lin outside 1..2)
int tp_fused_forward(const FusedArgs& f, cudaStream_t stream);

// Per-edge radial weights (or their d/dr) [rows][n_paths * 128] = hidden [rows][64] x last radial layer, through the
// fused kernels' tensor-core pipeline (tp_fused.cu); FMB_ERR_UNSUPPORTED without the weight image.
// `row_index` (or null): output row r is computed from hidden row row_index[r]
int radial_weights_tc(const float* hidden, const float* image, float* out, int rows, int n_paths, const long long* limit,
                      long long limit_offset, const int32_t* row_index, uint32_t* error_word, int max_ctas,
                      cudaStream_t stream);

// first layer in reassociated form (outer products per receiver and sender species)
struct FirstArgs {
    int n_rows, n_valid, fresh_from, n_species;
    const long long* count;
    const int32_t* row_ptr;
    const int32_t* senders;
    const int32_t* species;
    const float* edge_sh;
    const float* edge_vec;
    const float* hidden;           // [edges][64] last hidden radial layer of the first interaction
    const float* hidden_tangent;   // its derivative with respect to the edge length
    float* s;                      // forward output [n][16][n_species][64]
    const float* d_s;              // backward input, same layout
    float* force_acc;
    float* atom_virial;
    int first_layer_of_pass;
};
int first_accumulate_launch(const FirstArgs& f, cudaStream_t stream);
int first_backward_launch(const FirstArgs& f, cudaStream_t stream);

// Adjoint with per-edge hand-over (adjoint_edges.cu)
struct EdgeAdjointArgs {
    int lin;
    int n_atoms;           // atoms of the list
    int n_rows;            // receivers [0, n_rows)
    int n_valid;           // atoms [0, n_valid) have a message gradient
    int n_gather;          // atoms [0, n_gather) collect the gradient of their own features (d_x rows)
    long long chunk_e0, chunk_edges;   // this launch covers the edges [chunk_e0, chunk_e0 + chunk_edges) below the count
    const long long* count;
    const int32_t* row_ptr;
    const int32_t* senders;
    const int32_t* mirror;
    const float* x;
    const float* edge_sh;
    const float* edge_vec;
    const float* tp_w;             // [chunk edges][paths * C] values, d/dr behind them at tangent_offset
    long long tangent_offset;
    const float* d_mid;
    float* dxe;                    // [edges][(lin + 1)^2][C]
    float* qe;                     // [edges][4]
    float* d_x;                    // [n_rows][(lin + 1)^2][C]
    bool whole_list;               // the launch covers the whole edge list (tp_w holds every edge's weights)
    uint32_t* error_word;
    const int32_t* slot;           // or null: the weights of edge e are row slot[min(e, mirror[e])] of tp_w
};
// `slot`, `list`, `list_count` (or null): the edges below *listed_below that stand for their pair
int mirror_map(const fmb_nl_t* nl, int32_t* mirror, uint32_t* status, const long long* listed_below, int32_t* slot,
               int32_t* list, long long* list_count, int list_capacity, cudaStream_t stream);
// per-edge adjoint of an interaction after the first for one chunk of edges; after the last chunk the gather of the
// sender-side gradients into d_x
int tp_adjoint_edges(const EdgeAdjointArgs& t, cudaStream_t stream);
int gather_sender_gradient(const EdgeAdjointArgs& t, cudaStream_t stream);
// first interaction: adds its edge-vector gradients to qe (rows below n_add) or stores them
int first_adjoint_edges(const FirstArgs& f, int n_add, float* qe, cudaStream_t stream);
// forces (as gradients) and per-atom virials from the per-edge gradients; only the edges into atoms [0, n_valid) carry
// a gradient (the others are read as zero, whatever qe holds for them)
int force_gather(int n_atoms, int n_valid, const int32_t* row_ptr, const int32_t* senders, const int32_t* mirror,
                 const float* qe, const float* edge_vec, float* force_acc, float* atom_virial, cudaStream_t stream);

int symcon_forward(int n_atoms, int n_terms, int out_dim, const int32_t* terms, const float* coef,
                   const int32_t* species, const float* msg, float* basis, const int32_t* groups, int n_groups,
                   cudaStream_t stream);
int symcon_backward(int n_atoms, int n_terms, int out_dim, const int32_t* terms, const float* coef,
                    const int32_t* species, const float* msg, const float* d_basis, float* d_msg, const int32_t* groups,
                    int n_groups, cudaStream_t stream);
int fill_from_species(int n_atoms, int row, const int32_t* species, const float* table, float* out, cudaStream_t stream);
int readout(const fmb_model_t* m, int n_atoms, int n_energy, const float* h_first, const float* h_last, float* node_energy,
            float* d_h_first, float* d_h_last, cudaStream_t stream);
int reduce_outputs(const fmb_model_t* m, const fmb_work_t* w, int n_energy, double volume, cudaStream_t stream);
int commit_forces(const fmb_work_t* w, double* f64, double* e64, double* s64, cudaStream_t stream);

}  // namespace fmb
