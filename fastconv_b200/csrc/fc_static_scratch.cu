// Winograd forward for callers that are not allowed to allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: a plugin running inside an engine
// whose memory budget is fixed at start-up, a real-time loop where an allocation (an implicit
// device synchronisation) is forbidden after initialisation, or a process whose allocator is
// owned by another framework.  fc_wino_forward works on caller-provided V and M workspaces, but
// those callers have nowhere to get them from.  This entry point keeps the two Winograd-domain
// workspaces in a fixed array that is part of the library image itself, so the only buffers the
// caller passes are the layer's input, its pre-transformed filter and its output.
#include "fc_internal.h"

namespace {

// 4 Mi floats = 16 MiB, resident on every GPU that loads this library until the process exits.
constexpr size_t kScratchFloats = FC_STATIC_SCRATCH_FLOATS;
static __device__ __align__(256) float g_static_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
// Device address of g_static_scratch per GPU.  In host code the name `g_static_scratch` is only a
// handle for the runtime's symbol table, never a pointer a kernel may dereference; the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
float *g_scratch_addr[kMaxDevices] = {nullptr};

int scratch_for_current_device(int device, float **out) {
    if (g_scratch_addr[device] == nullptr) {
        float *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            fc::set_error("cudaGetSymbolAddress(static scratch) failed on device %d: %s", device,
                          cudaGetErrorString(e));
            return FC_ERR_CUDA;
        }
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return FC_OK;
}

}  // namespace

extern "C" int fc_wino_forward_static_scratch(const float *d_in, const float *d_U, float *d_out,
                                              const fc_conv_desc *desc, void *stream) {
    FC_REQUIRE(d_in && d_U && d_out && desc, FC_ERR_INVALID_ARG, "NULL argument");
    fc::WinoGeom g;
    FC_PROPAGATE(fc::wino_geom(desc, &g));
    const size_t v_elems = (size_t)64 * g.tp * g.icp;
    const size_t m_elems = (size_t)64 * g.oc * g.tp;
    FC_REQUIRE(v_elems + m_elems <= kScratchFloats, FC_ERR_UNSUPPORTED,
               "layer needs %zu floats of Winograd workspace (V %zu + M %zu) but the built-in scratch holds %zu; "
               "use fc_wino_forward with caller-provided workspaces for this size",
               v_elems + m_elems, v_elems, m_elems, kScratchFloats);
    int device = -1;
    FC_CHECK_CUDA(cudaGetDevice(&device));
    FC_REQUIRE(device >= 0 && device < kMaxDevices, FC_ERR_UNSUPPORTED, "device index %d not supported", device);
    float *scratch = nullptr;
    FC_PROPAGATE(scratch_for_current_device(device, &scratch));
    float *d_V = scratch;            // [64][icp][tp]; v_elems is a multiple of 64, so M stays 256-byte aligned
    float *d_M = scratch + v_elems;  // [64][oc][tp]

    // The stage launchers only read the stream and the device index from a context.
    fc_context view;
    view.device = device;
    view.sm_count = 0;
    view.stream = (cudaStream_t)stream;
    view.slab = nullptr;
    view.d_status = nullptr;
    // Nothing in the scratch has to start at zero: the input transform writes every element of V it
    // owns, zero padding of the tile and channel axes included, and the GEMM writes every element of M
    // before the output transform reads it.  Whatever an earlier call left behind is overwritten.
    FC_PROPAGATE(fc::launch_input_transform_rowmajor(&view, d_in, d_V, g));
    FC_PROPAGATE(fc::launch_wino_gemm_ffma(&view, d_U, d_V, d_M, g));
    FC_PROPAGATE(fc::launch_output_transform(&view, d_M, d_out, g));
    return FC_OK;
}
