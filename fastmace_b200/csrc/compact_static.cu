// fmb_nl_compact_static: neighbour compaction for callers that cannot give the library scratch memory.
//
// fmb_nl_compact needs two scratch buffers from its caller (per-receiver counts and the scan's tile sums). Some
// hosts cannot supply them: an MD driver that has frozen its device pool once its step graphs are captured, or a
// plugin host that hands out a fixed arena and forbids any allocation while it is stepping. For them this entry
// point keeps that scratch in one file-scope device array that lives for as long as the library is loaded
// (about 1 MiB on every GPU that loads it) and allocates nothing, ever. Inputs and outputs still belong to the
// caller and are passed in the fmb_nl_t as before; its edge_row_count and scan_scratch members are ignored.
//
// Rules that follow from sharing one array:
//   * at most FMB_STATIC_COMPACT_MAX_ATOMS atoms; larger lists are refused with FMB_ERR_ARG and a message;
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress) and caches it, so make
//     that first call outside any stream capture;
//   * every call overwrites the part of the array it reads (each receiver's count is written before the scan reads
//     it, and the scan writes its tile sums before using them), so nothing has to be zeroed between calls; the
//     previous call's contents are simply left behind;
//   * two calls that overlap in time on one GPU (different streams) would share the scratch and race: keep them on
//     one stream or order them with events.

#include "fmb_common.cuh"

#include <mutex>

namespace fmb {

namespace {

constexpr int kMaxAtoms = FMB_STATIC_COMPACT_MAX_ATOMS;
constexpr int kCountWords = ((kMaxAtoms + 1 + 63) / 64) * 64;              // keeps the second region 256-byte aligned
constexpr int kScanWords = 2 * (kMaxAtoms / 4096 + 2) + 8;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) int32_t g_compact_scratch[kCountWords + kScanWords];

std::mutex g_setup_mutex;
int32_t* g_scratch_address[kMaxDevices] = {};

// The name g_compact_scratch is only a host-side handle here: kernels must be given the device address that
// cudaGetSymbolAddress returns for the device that is current.
int scratch_for_current_device(int32_t** out) {
    int device = 0;
    FMB_CUDA_CHECK(cudaGetDevice(&device));
    FMB_REQUIRE(device >= 0 && device < kMaxDevices, "fmb_nl_compact_static: device index out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        FMB_CUDA_CHECK(cudaGetSymbolAddress(&address, g_compact_scratch));
        g_scratch_address[device] = static_cast<int32_t*>(address);
    }
    *out = g_scratch_address[device];
    return FMB_OK;
}

}  // namespace

}  // namespace fmb

extern "C" FMB_API int fmb_nl_compact_static(const fmb_nl_t* nl, const double* positions, fmb_stream_t stream) {
    FMB_REQUIRE(nl && positions, "fmb_nl_compact_static: null argument");
    FMB_REQUIRE(nl->n_atoms > 0, "fmb_nl_compact_static: the list has no atoms");
    if (nl->n_atoms > fmb::kMaxAtoms) {
        fmb::set_error_text("fmb_nl_compact_static: more atoms than FMB_STATIC_COMPACT_MAX_ATOMS (262144); "
                            "use fmb_nl_compact with caller-provided scratch");
        return FMB_ERR_ARG;
    }
    int32_t* scratch = nullptr;
    const int rc = fmb::scratch_for_current_device(&scratch);
    if (rc) return rc;
    fmb_nl_t with_static = *nl;
    with_static.edge_row_count = scratch;
    with_static.scan_scratch = scratch + fmb::kCountWords;
    return fmb_nl_compact(&with_static, positions, stream);
}
