// Internal declarations shared by the translation units of libfastconv_b200.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <map>

#include "../../include/fastconv_b200.h"
#include "fc_arena.h"

namespace fc {

void set_error(const char *fmt, ...);
unsigned default_peer_wait_polls();  // from $FASTCONV_PEER_WAIT_MS, else five seconds' worth

#define FC_CHECK_CUDA(call)                                                                             \
    do {                                                                                                \
        cudaError_t fc_err__ = (call);                                                                  \
        if (fc_err__ != cudaSuccess) {                                                                  \
            fc::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(fc_err__), __FILE__, __LINE__); \
            return FC_ERR_CUDA;                                                                         \
        }                                                                                               \
    } while (0)

#define FC_REQUIRE(cond, status, ...)     \
    do {                                  \
        if (!(cond)) {                    \
            fc::set_error(__VA_ARGS__);   \
            return (status);              \
        }                                 \
    } while (0)

#define FC_PROPAGATE(call)               \
    do {                                 \
        int fc_st__ = (call);            \
        if (fc_st__ != FC_OK) return fc_st__; \
    } while (0)

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }
inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// Geometry of one Winograd F(6x6,3x3) layer (3x3, stride 1, symmetric padding):
// output size as the reference driver derives it (winoF63ZC/winoF63ZC.cpp:334-338).
struct WinoGeom {
    int n, ic, oc, ih, iw, pad, oh, ow, th, tw, tiles, icp, tp;
    int n_ocb, n_kb;  // boxes of the packed filter: ceil(oc/128) x ceil(ic/32)
    int ocp;          // oc rounded up to 4: row length of the FP32-mode filter layout U[p][ic][ocp]
};

// Two operand layouts, chosen by the arithmetic mode of the TensorGEMM:
//   tensor-core modes  U packed 128x32 boxes (upack_index), V[p][tp][icp]   -- K-major, what UMMA/TMA want
//   fp32 mirrored mode U[p][icp][ocp],                      V[p][icp][tp]   -- row index contiguous, so GEMM
//                      tiles reach shared memory as [k][row] with async 16-byte copies and no transposition
// M[p][oc][tp] is the same in both.
inline bool rowmajor_layout(int mode) { return mode == FC_MATH_FP32_MIRRORED; }

// The transformed filter U is stored as contiguous boxes of 128 output channels x 32 input channels
// (16 KB each, zero padded): box (p, ocb, kb) starts at ((p*n_ocb + ocb)*n_kb + kb)*4096 floats and holds
// element (oc, ic) at (oc%128)*32 + ic%32.  One box is exactly one TMA load / one shared-memory stage of
// the GEMM kernels, so the dominant weight stream reads HBM in 16 KB contiguous pieces.
constexpr int U_BOX_ROWS = 128, U_BOX_COLS = 32, U_BOX_ELEMS = U_BOX_ROWS * U_BOX_COLS;
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t upack_index(int p, int oc, int ic, int n_ocb, int n_kb) {
    return ((((size_t)p * n_ocb + (oc >> 7)) * n_kb + (ic >> 5)) * U_BOX_ROWS + (oc & 127)) * U_BOX_COLS + (ic & 31);
}

int wino_geom(const fc_conv_desc *d, WinoGeom *g);  // validates and fills

// Kernel configuration of the multiply-accumulate stage; every field 0 = let the launcher's heuristic decide.
// This is what Tuning() searches (the counterpart of the reference's ocBlock/tileBlock/icBlock and mc/nc/kc).
struct KernelCfg {
    int bm, bn;     // block rows (output channels) / columns (tiles or pixels): 64 or 128 for FFMA (Winograd also 64 x 256
                    // and 128 x 80/96/112), bn a multiple of 16 for tcgen05
    int skinny;     // FFMA TensorGEMM with <= 32 tiles: 1 = one-thread-per-channel kernel, 2 = blocked kernel
    int smem_kb;    // tcgen05 kernels: shared-memory budget of the operand ring (sets the stage count / CTAs per SM)
};

// What a layer applies to every output element before storing it: y = relu(y + bias[oc]); both parts optional.
// The bias add is one rounded fp32 addition, so a chain of layers stays reproducible bit for bit.
struct Epilogue {
    const float *bias;  // per output channel, device memory, or NULL
    int relu;
#ifdef __CUDACC__
    __device__ __forceinline__ float operator()(float v, int ch) const {
        if (bias != nullptr) v = __fadd_rn(v, __ldg(bias + ch));
        return relu ? fmaxf(v, 0.0f) : v;
    }
#endif
};
constexpr Epilogue kNoEpilogue = {nullptr, 0};

// Output buffers of the ranks of a channel-split layer, as seen from this GPU (own memory or peer-mapped).
struct PeerOuts {
    float *base[FC_MAX_PEERS];
    int count;
};

// The same for a layer that is replayed without host involvement (a CUDA graph, a persistent stream of forwards):
// the step number lives on the device.  `step` counts the forwards this rank has published; a forward with number
// s = *step + 1 stores into the buffers of parity s & 1 and, when its last block is done, writes s into flag[rank]
// of every rank and into *step.
struct ScatterPublish {
    float *base[2][FC_MAX_PEERS];  // [parity][rank]: this rank's first channel inside rank r's output buffer
    int *flags[FC_MAX_PEERS];      // rank r's flag array int[world], as seen from this GPU
    int *step;                     // this GPU's memory
    unsigned *ticket;              // this GPU's memory, zero between launches: blocks of the launch that are done
    int count, rank;
};

struct CommonSlot {
    size_t bytes;
    void *ptr;
};

}  // namespace fc

struct fc_context {
    int device;
    int sm_count;
    cudaStream_t stream;
    void *slab;
    fc::Arena arena;
    std::map<size_t, fc::CommonSlot> common;
    cudaEvent_t ev[6];
    cudaEvent_t user_ev[FC_TIMER_SLOTS];
    int *d_status;  // device word kernels with bounded waits report into
    cudaStream_t copy_in, copy_out;  // created on first use by the pipelined host forward
    unsigned peer_wait_polls;        // iteration limit of the flag waits of channel-split layers
};

// Programmatic dependent launch.  Every kernel of the forward path is launched with the
// programmatic-stream-serialization attribute and calls pdl_wait() before it touches anything its predecessor in the
// stream reads or writes; what does not depend on the predecessor (barrier set-up, TMEM allocation, streaming
// constant weights) comes before the wait.  pdl_wait() is a no-op for a plain launch.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// None of the kernels signals early: pdl_trigger() marks where the signal used to be and does nothing, so a dependent
// grid comes in when the blocks of its predecessor exit.  Measured on the VGG-16 stack
// (CUDA graph, fp32): with griddepcontrol.launch_dependents at the top of every kernel 11.15 ms at 64 images, 1.684 at 8,
// 0.400 at one; with the signal moved to where a block has only its stores left 10.96 / 1.638 / 0.392; without any signal
// 10.92 / 1.631 / 0.382; without the attribute 10.92 / 1.632 / 0.384.  A dependent's blocks that come in early hold
// registers and shared memory through the last wave of the grid they wait for.
__device__ __forceinline__ void pdl_trigger() {}

namespace fc {
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
}  // namespace fc
#endif

// kernel launchers (device pointers, context stream) ------------------------------------------
namespace fc {

// one forward of a channel-split Winograd layer whose output transform stores into every rank's buffer and publishes
// the step itself (step number and buffer parity live on the device: the launch can be replayed by a CUDA graph)
int conv_forward_scatter_publish(fc_conv *conv, const float *d_in, const ScatterPublish &pub);

int launch_filter_transform(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic);
int launch_filter_transform_rowmajor(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic);
int launch_input_transform_rowmajor(fc_context *ctx, const float *d_in, float *d_V, const WinoGeom &g);
int launch_input_transform(fc_context *ctx, const float *d_in, float *d_V, const WinoGeom &g);
int launch_output_transform(fc_context *ctx, const float *d_M, float *d_out, const WinoGeom &g,
                            const Epilogue &ep = kNoEpilogue);
// fp32 layers with at most 4 input channels and a warp's worth of tiles: the TensorGEMM inside the output transform
// (same accumulation chain, M never stored)
bool output_transform_can_fuse_gemm(const WinoGeom &g);
int launch_output_transform_fused_gemm(fc_context *ctx, const float *d_U, const float *d_V, float *d_out,
                                       const WinoGeom &g, const Epilogue &ep);
int launch_output_transform_scatter(fc_context *ctx, const float *d_M, const PeerOuts &dst, const WinoGeom &g,
                                    const Epilogue &ep = kNoEpilogue);
int launch_output_transform_scatter_publish(fc_context *ctx, const float *d_M, const ScatterPublish &dst,
                                            const WinoGeom &g, const Epilogue &ep = kNoEpilogue);
int launch_peer_publish(fc_context *ctx, int *const *flags, int world, int rank, int step);
int launch_peer_wait(fc_context *ctx, const int *flags, int world, int step);
// waits until every rank's flag has reached *d_step (this rank's own count of published forwards)
int launch_peer_wait_published(fc_context *ctx, const int *flags, int world, const int *d_step);
int launch_wino_gemm_ffma(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g,
                          const KernelCfg *cfg = nullptr);
int launch_wino_gemm_tc(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g,
                        int mode, const KernelCfg *cfg = nullptr, const float *d_scales = nullptr);
// FC_MATH_TF32_U16: whether the layer runs with accumulator rows = channels (the layout the fp16 filter is built for),
// and the one-time conversion of the packed fp32 filter to fp16 boxes + 64 per-position scales (behind the boxes)
bool wino_gemm_tc_rows_are_channels(const WinoGeom &g);
size_t filter_u16_floats(const WinoGeom &g);  // floats the fp16 boxes and the scales occupy together
int launch_filter_to_u16(fc_context *ctx, const float *d_U32, float *d_U16, const WinoGeom &g);
inline const float *filter_u16_scales(const float *d_U16, const WinoGeom &g) {
    return d_U16 + (size_t)64 * g.n_ocb * g.n_kb * U_BOX_ELEMS / 2;
}
int launch_im2col_gather(fc_context *ctx, const float *d_in, float *d_B, const fc_conv_desc &d, int oh, int ow,
                         int image);
// d_ktab: per-layer k -> (offset, u:v) table (igemm_fill_ktab), or NULL outside a planned layer
int launch_igemm_ffma(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const fc_conv_desc &d,
                      int oh, int ow, const KernelCfg *cfg = nullptr, const int *d_ktab = nullptr,
                      const Epilogue &ep = kNoEpilogue, size_t in_img_stride = 0, size_t out_img_stride = 0,
                      float *d_bmat = nullptr);
// scratch for the materialised gathered matrix of a few-pixel, long-reduction layer: K x igemm_matrix_ld floats
bool igemm_wants_matrix(const fc_conv_desc &d, int oh, int ow);
bool igemm_is_tiny(const fc_conv_desc &d, int oh, int ow);  // M, N, K <= 32: the reference's unfused scalar GEMM
size_t igemm_matrix_ld(const fc_conv_desc &d, int oh, int ow);
// group == ic: one thread per output element, reduction over the kh*kw taps only
int launch_depthwise(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out, const fc_conv_desc &d,
                     int oh, int ow, const Epilogue &ep = kNoEpilogue);
size_t igemm_ktab_entries(const fc_conv_desc &d);
void igemm_fill_ktab(const fc_conv_desc &d, int *host_pairs);  // 2 ints per entry
int launch_igemm_tc(fc_context *ctx, const float *d_in, const float *d_packed, float *d_out, const fc_conv_desc &d,
                    int oh, int ow, int mode, const KernelCfg *cfg = nullptr, const int *d_ktab = nullptr,
                    const Epilogue &ep = kNoEpilogue, size_t in_img_stride = 0, size_t out_img_stride = 0);
// direct convolution on the tensor cores (stride 1 or 2, TF32): NHWC copy of the input + shifted TMA boxes
bool direct_tc_eligible(const fc_conv_desc &d);
enum { DIRECT_VS_GATHER = 0, DIRECT_VS_WINOGRAD_TF32 = 1, DIRECT_VS_WINOGRAD_FP32 = 2 };  // what it would replace
bool direct_tc_preferred(const fc_conv_desc &d, int oh, int ow, int sm_count, int rival);
size_t direct_nhwc_elems(const fc_conv_desc &d);
size_t direct_packed_elems(const fc_conv_desc &d);
int direct_tc_launches(const fc_conv_desc &d, int oh, int ow, int sm_count, const KernelCfg *cfg, bool has_epilogue);
int launch_direct_pack_weights(fc_context *ctx, const float *d_kernel, float *d_wp, const fc_conv_desc &d);
int launch_direct_tc(fc_context *ctx, const float *d_in, float *d_nhwc, const float *d_wp, float *d_out,
                     const fc_conv_desc &d, int oh, int ow, const KernelCfg *cfg = nullptr,
                     const Epilogue &ep = kNoEpilogue);
size_t igemm_packed_elems(int oc, int K);
int launch_igemm_pack_weights(fc_context *ctx, const float *d_kernel, float *d_packed, int oc, int K);

}  // namespace fc
