// C ABI of libfastconv_b200: context + device arena, stage-level entry points, planned layers.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "fc_internal.h"

namespace fc {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

// FASTCONV_PDL=0 in the environment turns programmatic dependent launch off (plain stream order).
bool pdl_enabled() {
    static int state = -1;
    if (state < 0) {
        const char *e = getenv("FASTCONV_PDL");
        state = (e && e[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

// FASTCONV_GRAPH=0 makes a layer list replay its layers as ordinary launches instead of one CUDA graph, so that a
// profiler sees plain kernel launches.
static bool graph_enabled() {
    static int state = -1;
    if (state < 0) {
        const char *e = getenv("FASTCONV_GRAPH");
        state = (e && e[0] == '0') ? 0 : 1;
    }
    return state == 1;
}

static int check_desc(const fc_conv_desc *d) {
    FC_REQUIRE(d != nullptr, FC_ERR_INVALID_ARG, "descriptor is NULL");
    FC_REQUIRE(d->batch > 0 && d->ic > 0 && d->oc > 0 && d->ih > 0 && d->iw > 0 && d->kh > 0 && d->kw > 0,
               FC_ERR_INVALID_ARG, "descriptor has a non-positive extent");
    FC_REQUIRE(d->sh > 0 && d->sw > 0, FC_ERR_INVALID_ARG, "stride must be positive (conv_layer.h:62-63)");
    FC_REQUIRE(d->pad_left >= 0 && d->pad_right >= 0 && d->pad_top >= 0 && d->pad_bottom >= 0, FC_ERR_INVALID_ARG,
               "negative padding");
    FC_REQUIRE(d->group >= 1 && d->ic % d->group == 0 && d->oc % d->group == 0, FC_ERR_INVALID_ARG,
               "group=%d must divide the %d input and %d output channels", d->group, d->ic, d->oc);
    FC_REQUIRE(d->iw + d->pad_left + d->pad_right >= d->kw && d->ih + d->pad_top + d->pad_bottom >= d->kh,
               FC_ERR_INVALID_ARG, "kernel larger than the padded input");
    return FC_OK;
}

int wino_geom(const fc_conv_desc *d, WinoGeom *g) {
    FC_PROPAGATE(check_desc(d));
    // The reference driver ignores kh/kw/stride and assumes 3x3 s1 with one symmetric pad
    // (winoF63ZC/winoF63ZC.cpp:334-338); anything else is refused here instead of computed wrongly.
    FC_REQUIRE(d->group == 1, FC_ERR_UNSUPPORTED, "winograd F(6x6,3x3) is built for group 1, got %d", d->group);
    FC_REQUIRE(d->kh == 3 && d->kw == 3, FC_ERR_UNSUPPORTED, "winograd F(6x6,3x3) needs a 3x3 kernel, got %dx%d",
               d->kh, d->kw);
    FC_REQUIRE(d->sh == 1 && d->sw == 1, FC_ERR_UNSUPPORTED, "winograd F(6x6,3x3) needs stride 1, got %dx%d", d->sh,
               d->sw);
    FC_REQUIRE(d->pad_left == d->pad_right && d->pad_left == d->pad_top && d->pad_left == d->pad_bottom,
               FC_ERR_UNSUPPORTED, "winograd F(6x6,3x3) needs one symmetric padding value");
    g->n = d->batch; g->ic = d->ic; g->oc = d->oc; g->ih = d->ih; g->iw = d->iw; g->pad = d->pad_left;
    g->oh = d->ih + 2 * g->pad - 2;
    g->ow = d->iw + 2 * g->pad - 2;
    FC_REQUIRE(g->oh >= 1 && g->ow >= 1, FC_ERR_INVALID_ARG, "empty output");
    g->th = (g->oh + 5) / 6;
    g->tw = (g->ow + 5) / 6;
    const long long tiles = (long long)g->n * g->th * g->tw;
    FC_REQUIRE(tiles < (1ll << 30), FC_ERR_UNSUPPORTED, "too many tiles (%lld)", tiles);
    g->tiles = (int)tiles;
    g->icp = round_up(g->ic, 8);
    g->tp = round_up(g->tiles, 8);
    g->n_ocb = (g->oc + U_BOX_ROWS - 1) / U_BOX_ROWS;
    g->n_kb = (g->ic + U_BOX_COLS - 1) / U_BOX_COLS;
    g->ocp = round_up(g->oc, 4);
    return FC_OK;
}

}  // namespace fc

using namespace fc;

struct fc_conv {
    fc_context *ctx;
    fc_conv_desc desc;
    int algo, mode;
    int oh, ow;
    WinoGeom geom;
    // A large batch runs as several passes over blocks of images so that the Winograd-domain buffers V and M of
    // one pass stay in L2 between the kernel that writes them and the one that reads them (plan_passes).
    int pass_imgs;        // images per pass; == desc.batch when the layer runs in one pass
    WinoGeom pass_geom;   // geometry of a full pass
    WinoGeom tail_geom;   // geometry of the last, shorter pass (n == 0 when the batch divides evenly)
    float *d_kernel;  // raw [oc][ic*kh*kw]
    float *d_packed;  // tensor-core implicit GEMM: padded hi/lo planes of the weights
    float *d_ktab;    // fp32 implicit GEMM: int pairs (offset, u:v) per k, in a float-typed arena slot
    float *d_bmat;    // fp32 implicit GEMM of a few-pixel, long-reduction layer: the materialised gathered matrix
    float *d_nhwc;    // direct tensor-core path: the input of one forward as [n][h][w][channels padded to 32]
    float *d_wp;      // direct tensor-core path: weights as [tap][oc][channels padded to 32]
    float *d_bias;    // per-channel bias of the epilogue, or NULL
    int relu;         // epilogue: clamp at zero after the bias
    float *d_U, *d_V, *d_M;
    float *d_in, *d_out;  // staging for forward_host
    float kernel_tran_ms;
    float stage_ms[5];
    std::vector<float> round_ms;  // per-iteration totals of the most recent fc_conv_profile
    KernelCfg cfg;        // all zero = launcher heuristics; set by fc_conv_tune
    bool auto_requested;  // created with FC_ALGO_AUTO: Tuning may switch between Winograd and im2col
    bool wino_eligible;   // 3x3, stride 1, symmetric padding
    int requested_mode;   // the mode given to fc_conv_create; `mode` is the arithmetic it resolved to for this layer
};

extern "C" {

int fc_abi_version(void) { return FC_ABI_VERSION; }

const char *fc_status_string(int s) {
    switch (s) {
        case FC_OK: return "ok";
        case FC_ERR_INVALID_ARG: return "invalid argument";
        case FC_ERR_UNSUPPORTED: return "unsupported shape or mode";
        case FC_ERR_OUT_OF_MEMORY: return "out of device memory";
        case FC_ERR_CUDA: return "CUDA error";
        case FC_ERR_NO_DEVICE: return "no usable CUDA device";
        case FC_ERR_TIMEOUT: return "device-side wait timed out";
        case FC_ERR_COMM: return "multi-GPU communication error";
        default: return "unknown status";
    }
}

const char *fc_last_error(void) { return fc::g_err; }

int fc_device_count(int *count) {
    FC_REQUIRE(count != nullptr, FC_ERR_INVALID_ARG, "count is NULL");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    *count = n;
    return FC_OK;
}

// ---- context + arena -----------------------------------------------------------------------

int fc_context_create(int device, size_t arena_bytes, fc_context **out) {
    FC_REQUIRE(out != nullptr, FC_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        set_error("no CUDA device is visible; this library has no CPU path");
        return FC_ERR_NO_DEVICE;
    }
    FC_REQUIRE(device >= 0 && device < n, FC_ERR_INVALID_ARG, "device %d out of range (0..%d)", device, n - 1);
    cudaDeviceProp prop;
    FC_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
    FC_REQUIRE(prop.major == 10, FC_ERR_NO_DEVICE, "device %d is sm_%d%d; the kernels are built for sm_100a only",
               device, prop.major, prop.minor);
    FC_CHECK_CUDA(cudaSetDevice(device));
    fc_context *ctx = new (std::nothrow) fc_context();
    FC_REQUIRE(ctx != nullptr, FC_ERR_OUT_OF_MEMORY, "host allocation failed");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->slab = nullptr;
    ctx->stream = nullptr;
    ctx->d_status = nullptr;
    ctx->copy_in = ctx->copy_out = nullptr;
    ctx->peer_wait_polls = default_peer_wait_polls();
    for (auto &e : ctx->ev) e = nullptr;
    for (auto &e : ctx->user_ev) e = nullptr;
    if (arena_bytes < (1u << 20)) arena_bytes = 1u << 20;
    cudaError_t e = cudaMalloc(&ctx->slab, arena_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMalloc of the %zu-byte arena failed: %s", arena_bytes, cudaGetErrorString(e));
        delete ctx;
        return FC_ERR_OUT_OF_MEMORY;
    }
    ctx->arena.reset((uintptr_t)ctx->slab, arena_bytes);
    // from here on a failure releases what exists so far (slab, stream, events) through fc_context_destroy
    auto finish = [&]() -> int {
        FC_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        for (auto &ev : ctx->ev) FC_CHECK_CUDA(cudaEventCreate(&ev));
        for (auto &ev : ctx->user_ev) FC_CHECK_CUDA(cudaEventCreate(&ev));
        ctx->d_status = (int *)ctx->arena.alloc(256);
        FC_CHECK_CUDA(cudaMemsetAsync(ctx->d_status, 0, 256, ctx->stream));
        FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
        return FC_OK;
    };
    const int st = finish();
    if (st != FC_OK) {
        fc_context_destroy(ctx);
        return st;
    }
    *out = ctx;
    return FC_OK;
}

int fc_context_destroy(fc_context *ctx) {
    if (!ctx) return FC_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    for (auto &ev : ctx->ev)
        if (ev) cudaEventDestroy(ev);
    for (auto &ev : ctx->user_ev)
        if (ev) cudaEventDestroy(ev);
    if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->slab) cudaFree(ctx->slab);
    delete ctx;
    return FC_OK;
}

// Waits for the stream, then reads (and clears) the word kernels with bounded waits report into.
static int sync_and_check_status(fc_context *ctx) {
    int st = 0;
    FC_CHECK_CUDA(cudaMemcpyAsync(&st, ctx->d_status, sizeof st, cudaMemcpyDeviceToHost, ctx->stream));
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    if (st != 0) {
        FC_CHECK_CUDA(cudaMemsetAsync(ctx->d_status, 0, sizeof st, ctx->stream));
        FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
        set_error("a kernel gave up a bounded device-side wait (status word %d)", st);
        return FC_ERR_TIMEOUT;
    }
    return FC_OK;
}

int fc_context_synchronize(fc_context *ctx) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));  // a process may hold contexts on several GPUs
    return sync_and_check_status(ctx);
}

int fc_context_device(const fc_context *ctx, int *device) {
    FC_REQUIRE(ctx != nullptr && device != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    *device = ctx->device;
    return FC_OK;
}

int fc_context_info(const fc_context *ctx, int *sm_count, int *sm_clock_max_mhz) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    if (sm_count) *sm_count = ctx->sm_count;
    if (sm_clock_max_mhz) {
        int khz = 0;
        FC_CHECK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device));
        *sm_clock_max_mhz = khz / 1000;
    }
    return FC_OK;
}

int fc_context_stream(const fc_context *ctx, void **stream) {
    FC_REQUIRE(ctx != nullptr && stream != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    *stream = (void *)ctx->stream;
    return FC_OK;
}

int fc_arena_alloc(fc_context *ctx, size_t bytes, void **dptr) {
    FC_REQUIRE(ctx != nullptr && dptr != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    const uintptr_t p = ctx->arena.alloc(bytes);
    *dptr = (void *)p;
    FC_REQUIRE(p != 0, FC_ERR_OUT_OF_MEMORY,
               "arena exhausted: %zu bytes requested, %zu in use of %zu, largest free block %zu", bytes,
               ctx->arena.in_use(), ctx->arena.capacity(), ctx->arena.largest_free());
    return FC_OK;
}

int fc_arena_size_of(fc_context *ctx, const void *dptr, size_t *bytes) {
    FC_REQUIRE(ctx != nullptr && bytes != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    *bytes = ctx->arena.size_of((uintptr_t)dptr);
    FC_REQUIRE(*bytes != 0, FC_ERR_INVALID_ARG, "pointer %p was not allocated from this arena", dptr);
    return FC_OK;
}

int fc_arena_free(fc_context *ctx, void *dptr) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    if (dptr == nullptr) return FC_OK;
    FC_REQUIRE(ctx->arena.release((uintptr_t)dptr), FC_ERR_INVALID_ARG,
               "pointer %p was not allocated from this arena (or was freed twice)", dptr);
    return FC_OK;
}

int fc_arena_free_all(fc_context *ctx) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    ctx->arena.release_all();
    ctx->common.clear();
    ctx->d_status = (int *)ctx->arena.alloc(256);
    return FC_OK;
}

int fc_arena_stats(fc_context *ctx, size_t *capacity, size_t *in_use, size_t *peak, size_t *blocks) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    if (capacity) *capacity = ctx->arena.capacity();
    if (in_use) *in_use = ctx->arena.in_use();
    if (peak) *peak = ctx->arena.peak();
    if (blocks) *blocks = ctx->arena.blocks();
    return FC_OK;
}

int fc_arena_common_request(fc_context *ctx, size_t bytes, size_t id) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    CommonSlot &s = ctx->common[id];  // value-initialised on first use
    FC_REQUIRE(s.ptr == nullptr || bytes <= s.bytes, FC_ERR_INVALID_ARG,
               "common pool %zu is already committed with %zu bytes; free it before requesting %zu", id, s.bytes,
               bytes);
    if (bytes > s.bytes) s.bytes = bytes;
    return FC_OK;
}

int fc_arena_common_commit(fc_context *ctx) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    for (auto &kv : ctx->common) {
        if (kv.second.ptr != nullptr || kv.second.bytes == 0) continue;
        void *p = nullptr;
        FC_PROPAGATE(fc_arena_alloc(ctx, kv.second.bytes, &p));
        kv.second.ptr = p;
    }
    return FC_OK;
}

int fc_arena_common_ptr(fc_context *ctx, size_t id, void **dptr) {
    FC_REQUIRE(ctx != nullptr && dptr != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    auto it = ctx->common.find(id);
    FC_REQUIRE(it != ctx->common.end() && it->second.ptr != nullptr, FC_ERR_INVALID_ARG,
               "common pool %zu has not been requested and committed", id);
    *dptr = it->second.ptr;
    return FC_OK;
}

int fc_arena_common_free(fc_context *ctx, size_t id) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    auto it = ctx->common.find(id);
    FC_REQUIRE(it != ctx->common.end(), FC_ERR_INVALID_ARG, "common pool %zu does not exist", id);
    if (it->second.ptr) ctx->arena.release((uintptr_t)it->second.ptr);
    ctx->common.erase(it);
    return FC_OK;
}

int fc_memcpy_h2d(fc_context *ctx, void *dst, const void *src, size_t bytes) {
    FC_REQUIRE(ctx != nullptr && dst != nullptr && src != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    return FC_OK;
}

int fc_memcpy_d2h(fc_context *ctx, void *dst, const void *src, size_t bytes) {
    FC_REQUIRE(ctx != nullptr && dst != nullptr && src != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    return FC_OK;
}

int fc_memset_device(fc_context *ctx, void *dst, int value, size_t bytes) {
    FC_REQUIRE(ctx != nullptr && dst != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_CHECK_CUDA(cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return FC_OK;
}

int fc_host_alloc_pinned(size_t bytes, void **hptr) {
    FC_REQUIRE(hptr != nullptr, FC_ERR_INVALID_ARG, "hptr is NULL");
    FC_CHECK_CUDA(cudaMallocHost(hptr, bytes));
    return FC_OK;
}

int fc_host_free_pinned(void *hptr) {
    if (hptr) FC_CHECK_CUDA(cudaFreeHost(hptr));
    return FC_OK;
}

int fc_timer_record(fc_context *ctx, int slot) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    FC_REQUIRE(slot >= 0 && slot < FC_TIMER_SLOTS, FC_ERR_INVALID_ARG, "timer slot %d out of range", slot);
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_CHECK_CUDA(cudaEventRecord(ctx->user_ev[slot], ctx->stream));
    return FC_OK;
}

int fc_timer_elapsed_ms(fc_context *ctx, int a, int b, float *ms) {
    FC_REQUIRE(ctx != nullptr && ms != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(a >= 0 && a < FC_TIMER_SLOTS && b >= 0 && b < FC_TIMER_SLOTS, FC_ERR_INVALID_ARG,
               "timer slot out of range");
    FC_CHECK_CUDA(cudaEventSynchronize(ctx->user_ev[b]));
    FC_CHECK_CUDA(cudaEventElapsedTime(ms, ctx->user_ev[a], ctx->user_ev[b]));
    return FC_OK;
}

// ---- shape helpers -------------------------------------------------------------------------

int fc_conv_output_size(const fc_conv_desc *d, int *oh, int *ow) {
    FC_PROPAGATE(check_desc(d));
    FC_REQUIRE(oh != nullptr && ow != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    *ow = (d->iw + d->pad_left + d->pad_right - d->kw) / d->sw + 1;
    *oh = (d->ih + d->pad_top + d->pad_bottom - d->kh) / d->sh + 1;
    return FC_OK;
}

int fc_select_algorithm(const fc_conv_desc *d, int *algo) {
    FC_PROPAGATE(check_desc(d));
    FC_REQUIRE(algo != nullptr, FC_ERR_INVALID_ARG, "algo is NULL");
    int a = FC_ALGO_IM2COL;  // fall-back, ConvTest.cpp:329-330
    if (d->group == 1 && (d->sh > d->sw ? d->sh : d->sw) == 1) {  // grouped layers: implicit GEMM per group
        if ((d->kh > d->kw ? d->kh : d->kw) == 1) {
            a = FC_ALGO_IM2COL;  // "direct" in the reference, whose case body is empty
        } else if (d->kh == 3 && d->kw == 3 && d->pad_left == d->pad_right && d->pad_left == d->pad_top &&
                   d->pad_left == d->pad_bottom) {
            a = FC_ALGO_WINOGRAD;
        }
    }
    *algo = a;
    return FC_OK;
}

static size_t u_elems_for(const WinoGeom &g, int mode) {
    if (mode == FC_MATH_TF32_U16) return filter_u16_floats(g);
    return rowmajor_layout(mode) ? (size_t)64 * g.icp * g.ocp : (size_t)64 * g.n_ocb * g.n_kb * U_BOX_ELEMS;
}

int fc_wino_buffer_elems(const fc_conv_desc *d, int mode, size_t *u, size_t *v, size_t *m) {
    FC_REQUIRE(mode >= FC_MATH_FP32_MIRRORED && mode <= FC_MATH_TF32, FC_ERR_INVALID_ARG, "unknown math mode %d", mode);
    WinoGeom g;
    FC_PROPAGATE(wino_geom(d, &g));
    if (u) *u = u_elems_for(g, mode);
    if (v) *v = (size_t)64 * g.tp * g.icp;
    if (m) *m = (size_t)64 * g.oc * g.tp;
    return FC_OK;
}

// ---- Winograd stages -----------------------------------------------------------------------

int fc_wino_filter_transform(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic, int mode) {
    FC_REQUIRE(ctx && d_kernel && d_U, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(oc > 0 && ic > 0, FC_ERR_INVALID_ARG, "non-positive channel count");
    FC_REQUIRE(mode >= FC_MATH_FP32_MIRRORED && mode <= FC_MATH_TF32, FC_ERR_INVALID_ARG, "unknown math mode %d", mode);
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_PROPAGATE(rowmajor_layout(mode) ? launch_filter_transform_rowmajor(ctx, d_kernel, d_U, oc, ic)
                                       : launch_filter_transform(ctx, d_kernel, d_U, oc, ic));
    // One-time work, so it is synchronous: the TensorGEMM kernels request their first boxes of U before they wait for
    // their predecessor in the stream (U is constant during a forward), which is only sound once U is complete.
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    return FC_OK;
}

static int input_transform_dispatch(fc_context *ctx, const float *d_in, float *d_V, const WinoGeom &g, int mode) {
    return rowmajor_layout(mode) ? launch_input_transform_rowmajor(ctx, d_in, d_V, g)
                                 : launch_input_transform(ctx, d_in, d_V, g);
}

int fc_wino_input_transform(fc_context *ctx, const float *d_in, float *d_V, const fc_conv_desc *desc, int mode) {
    FC_REQUIRE(ctx && d_in && d_V, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(mode >= FC_MATH_FP32_MIRRORED && mode <= FC_MATH_TF32, FC_ERR_INVALID_ARG, "unknown math mode %d", mode);
    WinoGeom g;
    FC_PROPAGATE(wino_geom(desc, &g));
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    return input_transform_dispatch(ctx, d_in, d_V, g, mode);
}

static int wino_gemm_dispatch(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const WinoGeom &g,
                              int mode, const KernelCfg *cfg = nullptr) {
    switch (mode) {
        case FC_MATH_FP32_MIRRORED: return launch_wino_gemm_ffma(ctx, d_U, d_V, d_M, g, cfg);
        case FC_MATH_3XTF32:
        case FC_MATH_TF32: return launch_wino_gemm_tc(ctx, d_U, d_V, d_M, g, mode, cfg);
        case FC_MATH_TF32_U16: return launch_wino_gemm_tc(ctx, d_U, d_V, d_M, g, mode, cfg, filter_u16_scales(d_U, g));
        default: set_error("unknown math mode %d", mode); return FC_ERR_INVALID_ARG;
    }
}

int fc_wino_tensor_gemm(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const fc_conv_desc *desc,
                        int mode) {
    FC_REQUIRE(ctx && d_U && d_V && d_M, FC_ERR_INVALID_ARG, "NULL argument");
    WinoGeom g;
    FC_PROPAGATE(wino_geom(desc, &g));
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    return wino_gemm_dispatch(ctx, d_U, d_V, d_M, g, mode);
}

int fc_wino_output_transform(fc_context *ctx, const float *d_M, float *d_out, const fc_conv_desc *desc) {
    FC_REQUIRE(ctx && d_M && d_out, FC_ERR_INVALID_ARG, "NULL argument");
    WinoGeom g;
    FC_PROPAGATE(wino_geom(desc, &g));
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    return launch_output_transform(ctx, d_M, d_out, g);
}

int fc_wino_forward(fc_context *ctx, const float *d_in, const float *d_U, float *d_V, float *d_M, float *d_out,
                    const fc_conv_desc *desc, int mode, float *stage_ms) {
    FC_REQUIRE(ctx && d_in && d_U && d_V && d_M && d_out, FC_ERR_INVALID_ARG, "NULL argument");
    WinoGeom g;
    FC_PROPAGATE(wino_geom(desc, &g));
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    if (stage_ms) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[0], ctx->stream));
    FC_PROPAGATE(input_transform_dispatch(ctx, d_in, d_V, g, mode));
    if (stage_ms) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[1], ctx->stream));
    FC_PROPAGATE(wino_gemm_dispatch(ctx, d_U, d_V, d_M, g, mode));
    if (stage_ms) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[2], ctx->stream));
    FC_PROPAGATE(launch_output_transform(ctx, d_M, d_out, g));
    if (stage_ms) {
        FC_CHECK_CUDA(cudaEventRecord(ctx->ev[3], ctx->stream));
        FC_CHECK_CUDA(cudaEventSynchronize(ctx->ev[3]));
        FC_CHECK_CUDA(cudaEventElapsedTime(&stage_ms[0], ctx->ev[0], ctx->ev[1]));
        stage_ms[1] = 0.0f;
        FC_CHECK_CUDA(cudaEventElapsedTime(&stage_ms[2], ctx->ev[1], ctx->ev[2]));
        FC_CHECK_CUDA(cudaEventElapsedTime(&stage_ms[3], ctx->ev[2], ctx->ev[3]));
    }
    return FC_OK;
}

// ---- im2col / implicit GEMM ----------------------------------------------------------------

int fc_im2col_gather(fc_context *ctx, const float *d_in, float *d_gathered, const fc_conv_desc *desc, int image) {
    FC_REQUIRE(ctx && d_in && d_gathered, FC_ERR_INVALID_ARG, "NULL argument");
    int oh, ow;
    FC_PROPAGATE(fc_conv_output_size(desc, &oh, &ow));
    FC_REQUIRE(image >= 0 && image < desc->batch, FC_ERR_INVALID_ARG, "image %d outside the batch of %d", image,
               desc->batch);
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    return launch_im2col_gather(ctx, d_in, d_gathered, *desc, oh, ow, image);
}

int fc_igemm_packed_elems(int oc, int K, size_t *elems) {
    FC_REQUIRE(elems != nullptr && oc > 0 && K > 0, FC_ERR_INVALID_ARG, "bad argument");
    *elems = igemm_packed_elems(oc, K);
    return FC_OK;
}

int fc_igemm_pack_weights(fc_context *ctx, const float *d_kernel, float *d_packed, int oc, int K) {
    FC_REQUIRE(ctx && d_kernel && d_packed, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(oc > 0 && K > 0, FC_ERR_INVALID_ARG, "non-positive matrix extent");
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    return launch_igemm_pack_weights(ctx, d_kernel, d_packed, oc, K);
}

int fc_igemm_forward(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out,
                     const fc_conv_desc *desc, int mode) {
    FC_REQUIRE(ctx && d_in && d_kernel && d_out, FC_ERR_INVALID_ARG, "NULL argument");
    int oh, ow;
    FC_PROPAGATE(fc_conv_output_size(desc, &oh, &ow));
    FC_REQUIRE(desc->group == 1, FC_ERR_UNSUPPORTED, "the stage entry point computes group 1 (a planned layer takes groups)");
    FC_REQUIRE((long long)desc->batch * oh * ow < (1ll << 31) && (long long)desc->ic * desc->kh * desc->kw < (1ll << 31),
               FC_ERR_UNSUPPORTED, "GEMM extent exceeds 32-bit indexing");
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    switch (mode) {
        case FC_MATH_FP32_MIRRORED: return launch_igemm_ffma(ctx, d_in, d_kernel, d_out, *desc, oh, ow);
        case FC_MATH_3XTF32:
        case FC_MATH_TF32: return launch_igemm_tc(ctx, d_in, d_kernel, d_out, *desc, oh, ow, mode);
        default: set_error("unknown math mode %d", mode); return FC_ERR_INVALID_ARG;
    }
}

// ---- planned layer --------------------------------------------------------------------------

static void conv_release(fc_conv *c) {
    fc_context *ctx = c->ctx;
    float *bufs[] = {c->d_kernel, c->d_packed, c->d_ktab, c->d_bmat, c->d_nhwc, c->d_wp, c->d_bias, c->d_U, c->d_V, c->d_M,
                     c->d_in, c->d_out};
    for (float *b : bufs)
        if (b) ctx->arena.release((uintptr_t)b);
    delete c;
}

static int grab(fc_context *ctx, float **p, size_t elems) {
    if (*p) return FC_OK;
    void *q = nullptr;
    int st = fc_arena_alloc(ctx, elems * sizeof(float), &q);
    *p = (float *)q;
    return st;
}

static void drop(fc_context *ctx, float **p) {
    if (*p) ctx->arena.release((uintptr_t)*p);
    *p = nullptr;
}

// One group of a (possibly grouped) layer as a convolution of its own: ic/group input and oc/group output channels.
static fc_conv_desc group_desc(const fc_conv *c) {
    fc_conv_desc d = c->desc;
    d.ic /= d.group;
    d.oc /= d.group;
    d.group = 1;
    return d;
}

// Optional L2 blocking over the batch.  Unblocked, V and M go out to HBM and come back: 2*(V+M) bytes of traffic that
// the layer's own bytes (input, weights, output) do not contain.  With P passes over blocks of images V and M of a pass
// can stay in L2, at the price of reading the transformed filter P times and of P times as many, smaller launches.
// FASTCONV_L2_BUDGET_MB is the part of L2 that V and M of one pass may occupy.  It is OFF (0) by default: measured on
// the batch-64 VGG-16 stack, a 48 MB budget was 1.2x (TF32) to 1.4x (fp32) SLOWER than one pass, because a pass of one
// or two images runs the three kernels in their latency-bound regime.
static size_t l2_budget_bytes() {  // read at every layer creation, so a caller can change it between layers
    const char *e = getenv("FASTCONV_L2_BUDGET_MB");
    long long mb = e ? atoll(e) : 0;
    if (mb < 0) mb = 0;
    return (size_t)mb << 20;
}

static int plan_passes(fc_conv *c) {
    const WinoGeom &g = c->geom;
    c->pass_imgs = g.n;
    c->pass_geom = g;
    memset(&c->tail_geom, 0, sizeof c->tail_geom);
    const size_t budget = l2_budget_bytes();
    const size_t per_img = (size_t)256 * g.th * g.tw * (g.icp + g.oc);  // V + M bytes of one image
    const size_t vm = per_img * g.n, u = (size_t)256 * g.icp * g.oc;
    if (budget == 0 || g.n == 1 || vm <= budget) return FC_OK;
    int imgs = (int)(budget / per_img);
    if (imgs < 1) imgs = 1;
    const int passes = (g.n + imgs - 1) / imgs;
    if ((size_t)(passes - 1) * u >= 2 * vm) return FC_OK;  // re-reading the filter would cost more than it saves
    imgs = (g.n + passes - 1) / passes;  // even out the passes
    fc_conv_desc d = c->desc;
    d.batch = imgs;
    FC_PROPAGATE(wino_geom(&d, &c->pass_geom));
    c->pass_imgs = imgs;
    if (g.n % imgs) {
        d.batch = g.n % imgs;
        FC_PROPAGATE(wino_geom(&d, &c->tail_geom));
    }
    return FC_OK;
}

static int conv_passes(const fc_conv *c) { return (c->desc.batch + c->pass_imgs - 1) / c->pass_imgs; }

// Workspaces and one-time weight re-layout of one algorithm (idempotent): Winograd gets U/V/M and the
// filter transform, the tensor-core implicit GEMM gets the packed hi/lo weight planes, the fp32 implicit
// GEMM its k -> (offset, u:v) decode table.
static int conv_prepare(fc_conv *c, int algo) {
    fc_context *ctx = c->ctx;
    const fc_conv_desc &d = c->desc;
    int st = FC_OK;
    bool timed = false;
    std::vector<int> ktab;  // host copy of the decode table; must outlive the asynchronous upload below
    if (algo == FC_ALGO_WINOGRAD) {
        st = plan_passes(c);
        if (st != FC_OK) return st;
        const WinoGeom &g = c->pass_geom;  // V and M hold one pass
        const bool fresh = c->d_U == nullptr;
        st = grab(ctx, &c->d_U, u_elems_for(g, c->mode));
        if (st == FC_OK) st = grab(ctx, &c->d_V, (size_t)64 * g.tp * g.icp);
        if (st == FC_OK) st = grab(ctx, &c->d_M, (size_t)64 * g.oc * g.tp);
        if (st == FC_OK && fresh) {
            cudaEventRecord(ctx->ev[0], ctx->stream);
            if (c->mode == FC_MATH_TF32_U16) {  // the packed fp32 filter into a scratch allocation, then its fp16 copy
                float *tmp = nullptr;
                st = grab(ctx, &tmp, u_elems_for(g, FC_MATH_TF32));
                if (st == FC_OK) st = launch_filter_transform(ctx, c->d_kernel, tmp, g.oc, g.ic);
                if (st == FC_OK) st = launch_filter_to_u16(ctx, tmp, c->d_U, g);
                cudaStreamSynchronize(ctx->stream);
                drop(ctx, &tmp);
            } else {
                st = rowmajor_layout(c->mode) ? launch_filter_transform_rowmajor(ctx, c->d_kernel, c->d_U, g.oc, g.ic)
                                              : launch_filter_transform(ctx, c->d_kernel, c->d_U, g.oc, g.ic);
            }
            cudaEventRecord(ctx->ev[1], ctx->stream);
            timed = true;
        }
    } else if (algo == FC_ALGO_DIRECT) {
        const bool fresh = c->d_wp == nullptr;
        st = grab(ctx, &c->d_wp, direct_packed_elems(d));
        if (st == FC_OK) st = grab(ctx, &c->d_nhwc, direct_nhwc_elems(d));
        if (st == FC_OK && fresh) {
            cudaEventRecord(ctx->ev[0], ctx->stream);
            st = launch_direct_pack_weights(ctx, c->d_kernel, c->d_wp, d);
            cudaEventRecord(ctx->ev[1], ctx->stream);
            timed = true;
        }
    } else if (d.group > 1 && d.group == d.ic) {
        // depthwise: one plain fp32 kernel over the raw weights in every mode, nothing to prepare
    } else if (c->mode != FC_MATH_FP32_MIRRORED) {
        const bool fresh = c->d_packed == nullptr;
        const fc_conv_desc gd = group_desc(c);
        const int K = gd.ic * gd.kh * gd.kw;
        const size_t per_group = igemm_packed_elems(gd.oc, K);
        st = grab(ctx, &c->d_packed, per_group * d.group);
        if (st == FC_OK && fresh) {
            cudaEventRecord(ctx->ev[0], ctx->stream);
            for (int g = 0; g < d.group && st == FC_OK; ++g)
                st = launch_igemm_pack_weights(ctx, c->d_kernel + (size_t)g * gd.oc * K, c->d_packed + g * per_group, gd.oc, K);
            cudaEventRecord(ctx->ev[1], ctx->stream);
            timed = true;
        }
    }
    const bool gathers = algo == FC_ALGO_IM2COL;  // the implicit GEMMs; Winograd and the direct path index nothing
    if (st == FC_OK && gathers && c->d_ktab == nullptr && !(d.group > 1 && d.group == d.ic)) {
        // every implicit GEMM reads the k decode table
        FC_REQUIRE((long long)d.ic * d.ih * d.iw < (1ll << 31) && d.kh < 0x4000 && d.kw < 0x4000, FC_ERR_UNSUPPORTED,
                   "image or kernel too large for the 32-bit decode table");
        const fc_conv_desc gd = group_desc(c);  // offsets are relative to the group's first channel
        const size_t entries = igemm_ktab_entries(gd);
        ktab.resize(2 * entries);
        igemm_fill_ktab(gd, ktab.data());
        st = grab(ctx, &c->d_ktab, 2 * entries);
        if (st == FC_OK) {
            cudaError_t ce = cudaMemcpyAsync(c->d_ktab, ktab.data(), 2 * entries * sizeof(int), cudaMemcpyHostToDevice,
                                             ctx->stream);
            if (ce != cudaSuccess) {
                set_error("decode table upload failed: %s", cudaGetErrorString(ce));
                st = FC_ERR_CUDA;
            }
        }
    }
    if (st == FC_OK && gathers && c->d_bmat == nullptr && igemm_wants_matrix(d, c->oh, c->ow))
        st = grab(ctx, &c->d_bmat, (size_t)d.ic * d.kh * d.kw * igemm_matrix_ld(d, c->oh, c->ow));
    if (st != FC_OK) return st;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        set_error("weight re-layout failed: %s", cudaGetErrorString(e));
        return FC_ERR_CUDA;
    }
    if (timed) cudaEventElapsedTime(&c->kernel_tran_ms, ctx->ev[0], ctx->ev[1]);
    return FC_OK;
}

int fc_resolve_plan(const fc_conv_desc *desc, int algo, int mode, int sm_count, int *algo_out, int *mode_out) {
    FC_REQUIRE(desc && algo_out && mode_out, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(mode >= FC_MATH_FP32_MIRRORED && mode <= FC_MATH_TF32_U16, FC_ERR_INVALID_ARG, "unknown math mode %d",
               mode);
    FC_REQUIRE(algo >= FC_ALGO_AUTO && algo <= FC_ALGO_WINOGRAD, FC_ERR_INVALID_ARG, "unknown algorithm %d", algo);
    int oh, ow;
    FC_PROPAGATE(fc_conv_output_size(desc, &oh, &ow));
    const bool auto_requested = algo == FC_ALGO_AUTO;
    if (algo == FC_ALGO_AUTO) FC_PROPAGATE(fc_select_algorithm(desc, &algo));
    const int sms = sm_count > 0 ? sm_count : 148;
    if (mode == FC_MATH_TF32) {
        // The mode stands for a tolerance (rel-L2 <= 3e-3), and one TF32 pass through F(6x6,3x3) misses it (6.4e-3).  A
        // layer headed for Winograd takes the direct tensor-core kernel, or stays on Winograd in the split 3xTF32
        // arithmetic where that kernel cannot run (and whenever Winograd was asked for by name); every other layer is
        // inside the tolerance with one pass.  Where `auto` may choose between the direct kernel and the gathering one,
        // it takes the faster (Tuning() still measures all of them).
        if (algo == FC_ALGO_WINOGRAD) {
            if (auto_requested && direct_tc_preferred(*desc, oh, ow, sms, DIRECT_VS_WINOGRAD_FP32))
                algo = FC_ALGO_DIRECT;
            else
                mode = FC_MATH_3XTF32;
        } else if (auto_requested && direct_tc_preferred(*desc, oh, ow, sms, DIRECT_VS_GATHER)) {
            algo = FC_ALGO_DIRECT;
        }
    } else if (mode == FC_MATH_TF32_UNBOUNDED || mode == FC_MATH_TF32_U16) {
        // one TF32 pass everywhere; `auto` takes the direct kernel where the measured crossovers favour it
        const bool u16 = mode == FC_MATH_TF32_U16;
        mode = FC_MATH_TF32;
        if (auto_requested &&
            direct_tc_preferred(*desc, oh, ow, sms, algo == FC_ALGO_WINOGRAD ? DIRECT_VS_WINOGRAD_TF32 : DIRECT_VS_GATHER))
            algo = FC_ALGO_DIRECT;
        // the fp16 filter: Winograd layers whose accumulator rows are channels (more than 64 of them, under 128 tiles)
        if (u16 && algo == FC_ALGO_WINOGRAD) {
            WinoGeom g;
            if (wino_geom(desc, &g) == FC_OK && wino_gemm_tc_rows_are_channels(g)) mode = FC_MATH_TF32_U16;
        }
    }
    // The split arithmetic stands for rel-L2 <= 1e-5, which the fp32 kernels meet with room to spare (they are
    // bit-identical to the reference).  With at most 64 input channels the reduction is too short to pay for the
    // tensor-core kernel's operand splitting: on every such layer measured (1, 8 and 64 images; 3 -> 64 @224 0.40
    // against 1.75 ms, 64 -> 64 @224 1.92 against 2.14 ms, 64 -> 128 @112 0.77 against 0.89 ms at 64 images) the FFMA
    // path is the faster one, so the accuracy mode runs it there.  $FASTCONV_3XTF32_MIN_IC moves the border (0: never).
    if (mode == FC_MATH_3XTF32 && algo == FC_ALGO_WINOGRAD) {
        const char *e = getenv("FASTCONV_3XTF32_MIN_IC");
        const int min_ic = e ? atoi(e) : 65;
        if (desc->ic < min_ic) mode = FC_MATH_FP32_MIRRORED;
    }
    // the direct tensor-core kernel is a TF32 kernel for ungrouped layers of stride 1 or 2; anything else asked for as
    // "direct" runs as the implicit GEMM (the reference's own case for the name is empty)
    if (algo == FC_ALGO_DIRECT && !(mode == FC_MATH_TF32 && direct_tc_eligible(*desc))) algo = FC_ALGO_IM2COL;
    *algo_out = algo;
    *mode_out = mode;
    return FC_OK;
}

int fc_conv_create(fc_context *ctx, const fc_conv_desc *desc, int algo, int mode, const float *h_kernel,
                   fc_conv **out) {
    FC_REQUIRE(ctx && desc && h_kernel && out, FC_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    const bool auto_requested = algo == FC_ALGO_AUTO;
    const int requested_mode = mode;
    FC_PROPAGATE(fc_resolve_plan(desc, algo, mode, ctx->sm_count, &algo, &mode));
    int oh, ow;
    FC_PROPAGATE(fc_conv_output_size(desc, &oh, &ow));
    int auto_pick = FC_ALGO_IM2COL;
    fc_select_algorithm(desc, &auto_pick);
    const bool wino_eligible = auto_pick == FC_ALGO_WINOGRAD;
    WinoGeom g;
    memset(&g, 0, sizeof g);
    if (algo == FC_ALGO_WINOGRAD || wino_eligible) FC_PROPAGATE(wino_geom(desc, &g));
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));

    fc_conv *c = new (std::nothrow) fc_conv();
    FC_REQUIRE(c != nullptr, FC_ERR_OUT_OF_MEMORY, "host allocation failed");
    c->ctx = ctx; c->desc = *desc; c->algo = algo; c->mode = mode; c->oh = oh; c->ow = ow; c->geom = g;
    c->auto_requested = auto_requested;
    c->wino_eligible = wino_eligible;
    c->requested_mode = requested_mode;

    const size_t k_elems = (size_t)desc->oc * (desc->ic / desc->group) * desc->kh * desc->kw;  // [oc][ic/group][kh][kw]
    const size_t in_elems = (size_t)desc->batch * desc->ic * desc->ih * desc->iw;
    const size_t out_elems = (size_t)desc->batch * desc->oc * oh * ow;
    int st = grab(ctx, &c->d_kernel, k_elems);
    if (st == FC_OK) st = grab(ctx, &c->d_in, in_elems);
    if (st == FC_OK) st = grab(ctx, &c->d_out, out_elems);
    if (st == FC_OK) {
        cudaError_t e = cudaMemcpyAsync(c->d_kernel, h_kernel, k_elems * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) {
            set_error("kernel upload failed: %s", cudaGetErrorString(e));
            st = FC_ERR_CUDA;
        }
    }
    if (st == FC_OK) st = conv_prepare(c, algo);
    if (st != FC_OK) {
        cudaStreamSynchronize(ctx->stream);
        conv_release(c);
        return st;
    }
    *out = c;
    return FC_OK;
}

int fc_conv_destroy(fc_conv *c) {
    if (!c) return FC_OK;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    conv_release(c);
    return FC_OK;
}

int fc_conv_math_mode(const fc_conv *c, int *mode) {
    FC_REQUIRE(c && mode, FC_ERR_INVALID_ARG, "NULL argument");
    *mode = c->mode;
    return FC_OK;
}

int fc_conv_algorithm(const fc_conv *c, int *algo) {
    FC_REQUIRE(c && algo, FC_ERR_INVALID_ARG, "NULL argument");
    *algo = c->algo;
    return FC_OK;
}

// Which implicit GEMM a layer runs.  The fp32 mode always takes the FFMA kernels.  A tensor-core mode states the
// precision the caller tolerates, not a unit: for short reductions the tcgen05 kernel's fixed cost (TMEM allocation,
// barriers, the gather's look-ahead) exceeds the whole FFMA kernel, whose exact fp32 result is inside any tensor-core
// tolerance.  Measured at batch 1 (ResNet-50 1x1 layers): K = 64..256 -> FFMA 6-18 us against 10-25 us; from K = 512 on
// the tensor cores win in TF32, from K = 1024 on in 3xTF32 (three MMAs and a split pass per k-step).  Tuning() decides by measurement (cfg.skinny 1 = FFMA, 2 = tcgen05).
//
// 3xTF32 stands for rel-L2 <= 1e-5.  The tensor core's fp32 accumulate rounds toward zero, which adds a bias of about
// 7e-9 per reduction step to a sum kept in TMEM (measured 1.4e-5 at K = 2048, 3.2e-5 at K = 4608); the implicit GEMM
// keeps its whole reduction there, so from K = 1024 on the mode runs the FFMA kernel, whose result is the reference's
// bit for bit.  (The Winograd GEMM takes its sum over into registers every 128 channels instead: fc_gemm_tc.cu.)
constexpr long long IGEMM_3XTF32_MAX_K = 1024;

static bool igemm_on_fp32_pipe(const fc_conv *c) {
    if (c->mode == FC_MATH_FP32_MIRRORED) return true;
    const fc_conv_desc gd = group_desc(c);
    const long long K = (long long)gd.ic * gd.kh * gd.kw;
    if (c->mode == FC_MATH_3XTF32 && K > IGEMM_3XTF32_MAX_K) return true;
    if (c->cfg.skinny == 1) return true;
    if (c->cfg.skinny == 2 || c->cfg.bn || c->cfg.smem_kb) return false;
    const long long flops = 2ll * gd.batch * gd.oc * K * c->oh * c->ow;
    return K <= (c->mode == FC_MATH_3XTF32 ? 512 : 256) && flops <= 500000000ll;  // short reduction AND a small problem
}

static int direct_launches(const fc_conv *c) {
    return direct_tc_launches(c->desc, c->oh, c->ow, c->ctx->sm_count > 0 ? c->ctx->sm_count : 148, &c->cfg,
                              c->d_bias != nullptr || c->relu);
}

// kernel launches of one forward of an implicit-GEMM layer
static int igemm_launches(const fc_conv *c) {
    if (c->desc.group > 1) return c->desc.group == c->desc.ic ? 1 : c->desc.group;
    const bool tile_kernel = c->cfg.skinny != 2;  // the matrix is written only ahead of the table-driven kernel
    return c->d_bmat != nullptr && igemm_on_fp32_pipe(c) && tile_kernel ? 2 : 1;
}

// fp32 layers with at most 4 input channels run the TensorGEMM inside the output transform (two kernels, M never
// stored); $FASTCONV_FUSE_SMALL_IC=0 keeps the three-kernel form for comparison.
static bool wino_pass_fuses_gemm(const fc_conv *c, const WinoGeom &g) {
    static int enabled = -1;
    if (enabled < 0) {
        const char *e = getenv("FASTCONV_FUSE_SMALL_IC");
        enabled = e && atoi(e) == 0 ? 0 : 1;
    }
    return enabled && c->mode == FC_MATH_FP32_MIRRORED && output_transform_can_fuse_gemm(g);
}

static int wino_launches(const fc_conv *c) {
    const int passes = conv_passes(c);
    int n = 0;
    for (int p = 0; p < passes; ++p) {
        const bool tail = (p + 1) * c->pass_imgs > c->desc.batch;
        n += wino_pass_fuses_gemm(c, tail ? c->tail_geom : c->pass_geom) ? 2 : 3;
    }
    return n;
}

// One pass of a Winograd layer: images [pass*pass_imgs, ...) of the batch through the three kernels.
static int wino_enqueue_pass(fc_conv *c, int pass, const float *d_in, float *d_out, bool timed) {
    fc_context *ctx = c->ctx;
    const int img0 = pass * c->pass_imgs;
    const bool tail = img0 + c->pass_imgs > c->desc.batch;
    const WinoGeom &g = tail ? c->tail_geom : c->pass_geom;
    const float *in = d_in + (size_t)img0 * g.ic * g.ih * g.iw;
    float *out = d_out + (size_t)img0 * g.oc * g.oh * g.ow;
    if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[0], ctx->stream));
    FC_PROPAGATE(input_transform_dispatch(ctx, in, c->d_V, g, c->mode));
    if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[1], ctx->stream));
    if (wino_pass_fuses_gemm(c, g)) {  // no TensorGEMM stage of its own: its time shows under the output transform
        if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[2], ctx->stream));
        FC_PROPAGATE(launch_output_transform_fused_gemm(ctx, c->d_U, c->d_V, out, g, Epilogue{c->d_bias, c->relu}));
        if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[3], ctx->stream));
        return FC_OK;
    }
    FC_PROPAGATE(wino_gemm_dispatch(ctx, c->d_U, c->d_V, c->d_M, g, c->mode, &c->cfg));
    if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[2], ctx->stream));
    FC_PROPAGATE(launch_output_transform(ctx, c->d_M, out, g, Epilogue{c->d_bias, c->relu}));
    if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[3], ctx->stream));
    return FC_OK;
}

// `timed` records the stage events of an im2col layer or of a one-pass Winograd layer (fc_conv_profile walks the
// passes of a split layer itself).
static int conv_enqueue(fc_conv *c, const float *d_in, float *d_out, bool timed) {
    fc_context *ctx = c->ctx;
    if (c->algo == FC_ALGO_WINOGRAD) {
        const int passes = conv_passes(c);
        for (int p = 0; p < passes; ++p) FC_PROPAGATE(wino_enqueue_pass(c, p, d_in, d_out, timed && passes == 1));
        return FC_OK;
    }
    if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[0], ctx->stream));
    if (timed) FC_CHECK_CUDA(cudaEventRecord(ctx->ev[1], ctx->stream));  // the gather is fused: no separate stage
    int st = FC_OK;
    const fc_conv_desc &full = c->desc;
    if (c->algo == FC_ALGO_DIRECT) {
        FC_PROPAGATE(launch_direct_tc(ctx, d_in, c->d_nhwc, c->d_wp, d_out, full, c->oh, c->ow, &c->cfg,
                                      Epilogue{c->d_bias, c->relu}));
        if (timed) {
            FC_CHECK_CUDA(cudaEventRecord(ctx->ev[2], ctx->stream));
            FC_CHECK_CUDA(cudaEventRecord(ctx->ev[3], ctx->stream));
        }
        return FC_OK;
    }
    if (full.group > 1 && full.group == full.ic) {  // depthwise: every output channel reads one input channel
        st = launch_depthwise(ctx, d_in, c->d_kernel, d_out, full, c->oh, c->ow, Epilogue{c->d_bias, c->relu});
    } else {
        // a grouped layer is `group` independent convolutions over channel slices of the same tensors
        const fc_conv_desc gd = group_desc(c);
        const size_t Kg = (size_t)gd.ic * gd.kh * gd.kw;
        const size_t in_stride = (size_t)full.ic * full.ih * full.iw, out_stride = (size_t)full.oc * c->oh * c->ow;
        const bool fp32_pipe = igemm_on_fp32_pipe(c);
        for (int g = 0; g < full.group && st == FC_OK; ++g) {
            const float *in_g = d_in + (size_t)g * gd.ic * gd.ih * gd.iw;
            float *out_g = d_out + (size_t)g * gd.oc * c->oh * c->ow;
            const Epilogue ep{c->d_bias ? c->d_bias + (size_t)g * gd.oc : nullptr, c->relu};
            if (fp32_pipe)
                st = launch_igemm_ffma(ctx, in_g, c->d_kernel + (size_t)g * gd.oc * Kg, out_g, gd, c->oh, c->ow, &c->cfg,
                                       reinterpret_cast<const int *>(c->d_ktab), ep, in_stride, out_stride, c->d_bmat);
            else
                st = launch_igemm_tc(ctx, in_g, c->d_packed + (size_t)g * igemm_packed_elems(gd.oc, (int)Kg), out_g, gd,
                                     c->oh, c->ow, c->mode, &c->cfg, reinterpret_cast<const int *>(c->d_ktab), ep,
                                     in_stride, out_stride);
        }
    }
    FC_PROPAGATE(st);
    if (timed) {
        FC_CHECK_CUDA(cudaEventRecord(ctx->ev[2], ctx->stream));
        FC_CHECK_CUDA(cudaEventRecord(ctx->ev[3], ctx->stream));
    }
    return FC_OK;
}

int fc_conv_set_epilogue(fc_conv *c, const float *h_bias, int relu) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));  // no forward of this layer is in flight while its epilogue changes
    if (h_bias != nullptr) {
        FC_PROPAGATE(grab(ctx, &c->d_bias, (size_t)c->desc.oc));
        FC_CHECK_CUDA(cudaMemcpyAsync(c->d_bias, h_bias, (size_t)c->desc.oc * sizeof(float), cudaMemcpyHostToDevice,
                                      ctx->stream));
        FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    } else {
        drop(ctx, &c->d_bias);
    }
    c->relu = relu ? 1 : 0;
    return FC_OK;
}

int fc_conv_forward_device(fc_conv *c, const float *d_in, float *d_out) {
    FC_REQUIRE(c && d_in && d_out, FC_ERR_INVALID_ARG, "NULL argument");
    FC_CHECK_CUDA(cudaSetDevice(c->ctx->device));
    return conv_enqueue(c, d_in, d_out, false);
}

int fc_conv_forward_scatter(fc_conv *c, const float *d_in, float *const *outs, int *const *flags, int world, int rank,
                            int k0, int oc_total, int step) {
    FC_REQUIRE(c && d_in && outs && flags, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(world >= 1 && world <= FC_MAX_PEERS && rank >= 0 && rank < world, FC_ERR_INVALID_ARG,
               "rank %d of %d outside the supported 1..%d ranks", rank, world, FC_MAX_PEERS);
    FC_REQUIRE(c->algo == FC_ALGO_WINOGRAD, FC_ERR_UNSUPPORTED, "the channel-split forward is built for Winograd layers");
    FC_REQUIRE(c->desc.batch == 1, FC_ERR_UNSUPPORTED, "the channel-split forward takes one image (batch %d)", c->desc.batch);
    FC_REQUIRE(k0 >= 0 && k0 + c->desc.oc <= oc_total, FC_ERR_INVALID_ARG, "slab [%d, %d) outside %d channels", k0,
               k0 + c->desc.oc, oc_total);
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    const WinoGeom &g = c->geom;
    PeerOuts dst;
    memset(&dst, 0, sizeof dst);
    dst.count = world;
    for (int r = 0; r < world; ++r) {
        FC_REQUIRE(outs[r] && flags[r], FC_ERR_INVALID_ARG, "rank %d has a NULL buffer", r);
        dst.base[r] = outs[r] + (size_t)k0 * g.oh * g.ow;
    }
    FC_PROPAGATE(input_transform_dispatch(ctx, d_in, c->d_V, g, c->mode));
    FC_PROPAGATE(wino_gemm_dispatch(ctx, c->d_U, c->d_V, c->d_M, g, c->mode, &c->cfg));
    FC_PROPAGATE(launch_output_transform_scatter(ctx, c->d_M, dst, g, Epilogue{c->d_bias, c->relu}));
    return launch_peer_publish(ctx, flags, world, rank, step);
}

}  // extern "C"

int fc::conv_forward_scatter_publish(fc_conv *c, const float *d_in, const ScatterPublish &pub) {
    FC_REQUIRE(c && d_in, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(c->algo == FC_ALGO_WINOGRAD && c->desc.batch == 1, FC_ERR_UNSUPPORTED,
               "the channel-split forward is built for single-image Winograd layers");
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    const WinoGeom &g = c->geom;
    FC_PROPAGATE(input_transform_dispatch(ctx, d_in, c->d_V, g, c->mode));
    FC_PROPAGATE(wino_gemm_dispatch(ctx, c->d_U, c->d_V, c->d_M, g, c->mode, &c->cfg));
    return launch_output_transform_scatter_publish(ctx, c->d_M, pub, g, Epilogue{c->d_bias, c->relu});
}

extern "C" {

int fc_conv_forward_host(fc_conv *c, const float *h_in, float *h_out) {
    FC_REQUIRE(c && h_in && h_out, FC_ERR_INVALID_ARG, "NULL argument");
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    const size_t in_bytes = (size_t)c->desc.batch * c->desc.ic * c->desc.ih * c->desc.iw * sizeof(float);
    const size_t out_bytes = (size_t)c->desc.batch * c->desc.oc * c->oh * c->ow * sizeof(float);
    FC_CHECK_CUDA(cudaMemcpyAsync(c->d_in, h_in, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    FC_PROPAGATE(conv_enqueue(c, c->d_in, c->d_out, false));
    FC_CHECK_CUDA(cudaMemcpyAsync(h_out, c->d_out, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    // every mode: the skinny fp32 TensorGEMM and all tensor-core kernels have bounded waits that report into the status word
    return sync_and_check_status(ctx);
}

int fc_conv_device_buffers(fc_conv *c, float **d_in, float **d_out) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    if (d_in) *d_in = c->d_in;
    if (d_out) *d_out = c->d_out;
    return FC_OK;
}

int fc_conv_time_device(fc_conv *c, const float *d_in, float *d_out, int warmup, int iters, float *ms_per_iter) {
    FC_REQUIRE(c && d_in && d_out && ms_per_iter, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(iters > 0 && warmup >= 0, FC_ERR_INVALID_ARG, "iters must be positive");
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    for (int i = 0; i < warmup; ++i) FC_PROPAGATE(conv_enqueue(c, d_in, d_out, false));
    FC_CHECK_CUDA(cudaEventRecord(ctx->ev[4], ctx->stream));
    for (int i = 0; i < iters; ++i) FC_PROPAGATE(conv_enqueue(c, d_in, d_out, false));
    FC_CHECK_CUDA(cudaEventRecord(ctx->ev[5], ctx->stream));
    FC_CHECK_CUDA(cudaEventSynchronize(ctx->ev[5]));
    float ms = 0.f;
    FC_CHECK_CUDA(cudaEventElapsedTime(&ms, ctx->ev[4], ctx->ev[5]));
    *ms_per_iter = ms / iters;
    return FC_OK;
}

int fc_conv_profile(fc_conv *c, const float *d_in, float *d_out, int iters, float stage_ms[5]) {
    FC_REQUIRE(c && d_in && d_out && stage_ms, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(iters > 0, FC_ERR_INVALID_ARG, "iters must be positive");
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    double acc[5] = {0, 0, 0, 0, 0};
    const int passes = c->algo == FC_ALGO_WINOGRAD ? conv_passes(c) : 1;
    c->round_ms.clear();
    for (int i = 0; i < iters; ++i) {
        const double before = acc[4];
        for (int p = 0; p < passes; ++p) {
            if (passes == 1)
                FC_PROPAGATE(conv_enqueue(c, d_in, d_out, true));
            else
                FC_PROPAGATE(wino_enqueue_pass(c, p, d_in, d_out, true));
            FC_CHECK_CUDA(cudaEventSynchronize(ctx->ev[3]));
            float a = 0, b = 0, d = 0, t = 0;
            FC_CHECK_CUDA(cudaEventElapsedTime(&a, ctx->ev[0], ctx->ev[1]));
            FC_CHECK_CUDA(cudaEventElapsedTime(&b, ctx->ev[1], ctx->ev[2]));
            FC_CHECK_CUDA(cudaEventElapsedTime(&d, ctx->ev[2], ctx->ev[3]));
            FC_CHECK_CUDA(cudaEventElapsedTime(&t, ctx->ev[0], ctx->ev[3]));
            acc[0] += a; acc[2] += b; acc[3] += d; acc[4] += t;
        }
        c->round_ms.push_back((float)(acc[4] - before));
    }
    stage_ms[0] = (float)(acc[0] / iters);
    stage_ms[1] = c->kernel_tran_ms;
    stage_ms[2] = (float)(acc[2] / iters);
    stage_ms[3] = (float)(acc[3] / iters);
    stage_ms[4] = (float)(acc[4] / iters);
    memcpy(c->stage_ms, stage_ms, sizeof c->stage_ms);
    return FC_OK;
}

int fc_conv_round_times(const fc_conv *c, float *ms, int capacity, int *count) {
    FC_REQUIRE(c != nullptr && count != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(capacity == 0 || ms != nullptr, FC_ERR_INVALID_ARG, "ms is NULL");
    *count = (int)c->round_ms.size();
    for (int i = 0; i < capacity && i < *count; ++i) ms[i] = c->round_ms[i];
    return FC_OK;
}

int fc_conv_work(const fc_conv *c, double *direct_flops, double *algo_flops, double *algo_bytes, double *min_bytes) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    const fc_conv_desc &d = c->desc;
    const double icg = (double)d.ic / d.group, taps = (double)d.kh * d.kw;
    const double direct = 2.0 * d.batch * d.oc * icg * taps * c->oh * c->ow;
    const double in = (double)d.batch * d.ic * d.ih * d.iw, out = (double)d.batch * d.oc * c->oh * c->ow;
    const double filt = (double)d.oc * icg * taps;
    const bool wino = c->algo == FC_ALGO_WINOGRAD;
    if (direct_flops) *direct_flops = direct;
    if (algo_flops) *algo_flops = wino ? 2.0 * 64 * c->geom.tiles * d.ic * d.oc : direct;
    if (algo_bytes) *algo_bytes = 4.0 * (in + (wino ? 64.0 * d.ic * d.oc : filt) + out);
    if (min_bytes) *min_bytes = 4.0 * (in + filt + out);
    return FC_OK;
}

// ---- Tuning() -------------------------------------------------------------------------------
// The reference tunes by exhaustive timing: every (ocBlock, tileBlock, icBlock, loop order) point runs
// `iterations` forwards and the fastest is kept (convLayer/winoF63ConvZC.cpp:25-174); the im2col layer
// keeps its best (mc, nc, kc, ...) in an append-only text log keyed by the GEMM shape
// (convLayer/im2colConv.cpp:66-92, 202-222, 261-283).  Same scheme here over the GPU kernels'
// configurations, timed with CUDA events; with FC_ALGO_AUTO on a Winograd-eligible layer the
// Winograd-vs-im2col choice itself is made from the measured times.  The log lives at
// $FASTCONV_TUNING_LOG or ./gemm_log/b200_tuning_log.

struct TuneCandidate {
    int algo;
    KernelCfg cfg;
};

static int time_current(fc_conv *c, int iters, float *ms) {
    fc_context *ctx = c->ctx;
    for (int i = 0; i < 2; ++i) FC_PROPAGATE(conv_enqueue(c, c->d_in, c->d_out, false));
    FC_CHECK_CUDA(cudaEventRecord(ctx->ev[4], ctx->stream));
    for (int i = 0; i < iters; ++i) FC_PROPAGATE(conv_enqueue(c, c->d_in, c->d_out, false));
    FC_CHECK_CUDA(cudaEventRecord(ctx->ev[5], ctx->stream));
    FC_PROPAGATE(sync_and_check_status(ctx));
    FC_CHECK_CUDA(cudaEventElapsedTime(ms, ctx->ev[4], ctx->ev[5]));
    *ms /= iters;
    return FC_OK;
}

static const char *algo_label(int algo) {
    return algo == FC_ALGO_WINOGRAD ? "winograd" : algo == FC_ALGO_DIRECT ? "direct" : "im2col";
}

static void enumerate_candidates(const fc_conv *c, int algo, std::vector<TuneCandidate> *out) {
    auto push = [&](int bm, int bn, int skinny, int smem_kb) {
        TuneCandidate t;
        t.algo = algo;
        t.cfg.bm = bm; t.cfg.bn = bn; t.cfg.skinny = skinny; t.cfg.smem_kb = smem_kb;
        out->push_back(t);
    };
    const int ffma_tiles[4][2] = {{128, 128}, {128, 64}, {64, 128}, {64, 64}};
    if (algo == FC_ALGO_DIRECT) {  // the ring's size and the width of the channel blocks
        push(0, 0, 0, 0);
        push(0, 0, 0, 104);
        push(0, 0, 0, 200);
        push(0, 128, 0, 0);  // channel blocks of 128 (two CTAs per SM) or 256 (one)
        push(0, 256, 0, 0);
        return;
    }
    const fc_conv_desc gd = group_desc(c);
    const bool ffma_only = c->mode == FC_MATH_FP32_MIRRORED ||  // ... or a 3xTF32 implicit GEMM too long for TMEM accumulation
                           (algo == FC_ALGO_IM2COL && c->mode == FC_MATH_3XTF32 &&
                            (long long)gd.ic * gd.kh * gd.kw > IGEMM_3XTF32_MAX_K);
    if (ffma_only) {
        if (algo == FC_ALGO_WINOGRAD) push(0, 0, 0, 0);  // the launcher's own choice (it alone mixes block widths in one launch)
        if (algo == FC_ALGO_WINOGRAD && (c->pass_imgs ? c->pass_geom : c->geom).tiles <= 32) push(0, 0, 1, 0);
        if (algo == FC_ALGO_IM2COL) {  // table-driven kernel in its eight block shapes
            const int small_tiles[5][2] = {{64, 64}, {32, 64}, {32, 32}, {16, 32}, {8, 32}};
            for (auto &t : ffma_tiles)
                if (t[0] * t[1] > 64 * 64) push(t[0], t[1], 1, 0);
            for (auto &t : small_tiles) push(t[0], t[1], 1, 0);
        }
        for (auto &t : ffma_tiles) push(t[0], t[1], 2, 0);
        if (algo == FC_ALGO_WINOGRAD && c->desc.oc > 64)  // block widths between 64 and 128 tiles
            for (int bn : {80, 96, 112}) push(128, bn, 2, 0);
        if (algo == FC_ALGO_WINOGRAD && c->desc.oc <= 64) push(64, 256, 2, 0);  // 4 channels x 16 tiles per thread
    } else {
        const int widths[5] = {32, 64, 96, 128, 256};
        const int budgets[3] = {72, 104, 200};
        for (int w : widths)
            for (int b : budgets) push(0, w, algo == FC_ALGO_IM2COL ? 2 : 0, b);
        if (algo == FC_ALGO_IM2COL) {  // and the FFMA kernel, which wins on short reductions
            const int small_tiles[5][2] = {{64, 64}, {32, 64}, {32, 32}, {16, 32}, {8, 32}};
            for (auto &t : small_tiles) push(t[0], t[1], 1, 0);
        }
    }
}

static const char *tuning_log_path() {
    const char *e = getenv("FASTCONV_TUNING_LOG");
    return e && e[0] ? e : "./gemm_log/b200_tuning_log";
}

// one log line: 17 key integers, then algo, bm, bn, skinny, smem_kb and the time in microseconds
static void tuning_key(const fc_conv *c, int key[17]) {
    const fc_conv_desc &d = c->desc;
    const int k[17] = {c->ctx->sm_count, c->auto_requested ? FC_ALGO_AUTO : c->algo, c->requested_mode, d.batch, d.ic, d.ih, d.iw,
                       d.oc, d.kh, d.kw, d.sh, d.sw, d.pad_left, d.pad_right, d.pad_top, d.pad_bottom, d.group};
    memcpy(key, k, sizeof k);
}

static bool tuning_log_lookup(const fc_conv *c, TuneCandidate *hit, float *us) {
    FILE *f = fopen(tuning_log_path(), "r");
    if (!f) return false;
    int key[17], row[17], v[5];
    tuning_key(c, key);
    bool found = false;
    char line[512];
    while (fgets(line, sizeof line, f)) {
        int n = 0, off = 0, pos = 0;
        bool ok = true;
        for (int i = 0; i < 17 && ok; ++i) ok = sscanf(line + pos, "%d,%n", &row[i], &off) == 1 && (pos += off, true);
        for (int i = 0; i < 5 && ok; ++i) ok = sscanf(line + pos, "%d,%n", &v[i], &off) == 1 && (pos += off, true);
        float t = 0;
        if (!ok || sscanf(line + pos, "%f%n", &t, &n) != 1) continue;
        if (memcmp(row, key, sizeof key) != 0) continue;
        hit->algo = v[0];
        hit->cfg.bm = v[1]; hit->cfg.bn = v[2]; hit->cfg.skinny = v[3]; hit->cfg.smem_kb = v[4];
        *us = t;
        found = true;  // keep scanning: the last matching line wins
    }
    fclose(f);
    return found;
}

static void tuning_log_append(const fc_conv *c, const TuneCandidate &best, float us) {
    const char *path = tuning_log_path();
    if (strcmp(path, "./gemm_log/b200_tuning_log") == 0) {
        if (system("mkdir -p ./gemm_log") != 0) return;
    }
    FILE *f = fopen(path, "a");
    if (!f) return;
    int key[17];
    tuning_key(c, key);
    for (int i = 0; i < 17; ++i) fprintf(f, "%d,", key[i]);
    fprintf(f, "%d,%d,%d,%d,%d,%.3f\n", best.algo, best.cfg.bm, best.cfg.bn, best.cfg.skinny, best.cfg.smem_kb, us);
    fclose(f);
}

int fc_conv_tune(fc_conv *c, int iters, int verbose) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(iters > 0, FC_ERR_INVALID_ARG, "iters must be positive");
    fc_context *ctx = c->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));

    TuneCandidate cached;
    float cached_us = 0;
    if (tuning_log_lookup(c, &cached, &cached_us)) {
        if (verbose) printf("log entry exists.\n");
        if (cached.algo != c->algo) FC_PROPAGATE(conv_prepare(c, cached.algo));
        c->algo = cached.algo;
        c->cfg = cached.cfg;
        return FC_OK;
    }
    if (verbose) printf("log entry doesn't exist.\n");

    std::vector<TuneCandidate> cands;
    enumerate_candidates(c, c->algo, &cands);
    // (a layer planned for the TF32 tolerance that runs in one pass must not be moved onto the Winograd path, which
    // misses that tolerance in one pass)
    if (c->auto_requested && c->wino_eligible && !(c->requested_mode == FC_MATH_TF32 && c->mode == FC_MATH_TF32)) {
        const int other = c->algo == FC_ALGO_WINOGRAD ? FC_ALGO_IM2COL : FC_ALGO_WINOGRAD;
        if (conv_prepare(c, other) == FC_OK) enumerate_candidates(c, other, &cands);
    }
    if (c->auto_requested && c->mode == FC_MATH_TF32 && direct_tc_eligible(c->desc) && c->algo != FC_ALGO_DIRECT &&
        conv_prepare(c, FC_ALGO_DIRECT) == FC_OK)
        enumerate_candidates(c, FC_ALGO_DIRECT, &cands);
    if (c->auto_requested && c->algo == FC_ALGO_DIRECT && !c->wino_eligible && conv_prepare(c, FC_ALGO_IM2COL) == FC_OK)
        enumerate_candidates(c, FC_ALGO_IM2COL, &cands);  // `auto` chose the direct kernel over the gathering one: time both
    const int start_algo = c->algo;
    const KernelCfg start_cfg = c->cfg;
    TuneCandidate best;
    best.algo = start_algo;
    best.cfg = start_cfg;
    float best_ms = 1e30f;
    for (const TuneCandidate &t : cands) {
        c->algo = t.algo;
        c->cfg = t.cfg;
        float ms = 0;
        const int st = time_current(c, iters, &ms);
        if (st == FC_ERR_UNSUPPORTED || st == FC_ERR_INVALID_ARG) continue;  // configuration does not fit this shape
        if (st != FC_OK) {
            c->algo = start_algo;
            c->cfg = start_cfg;
            return st;
        }
        if (verbose)
            printf("algo=%s bm=%d bn=%d skinny=%d smem=%dKB time=%.3f\n", algo_label(t.algo),
                   t.cfg.bm, t.cfg.bn, t.cfg.skinny, t.cfg.smem_kb, ms);
        if (ms < best_ms) {
            best_ms = ms;
            best = t;
        }
    }
    c->algo = best.algo;
    c->cfg = best.cfg;
    // the losers' workspaces go back to the arena
    if (best.algo != FC_ALGO_WINOGRAD) { drop(ctx, &c->d_U); drop(ctx, &c->d_V); drop(ctx, &c->d_M); }
    if (best.algo != FC_ALGO_IM2COL) { drop(ctx, &c->d_packed); drop(ctx, &c->d_ktab); drop(ctx, &c->d_bmat); }
    if (best.algo != FC_ALGO_DIRECT) { drop(ctx, &c->d_nhwc); drop(ctx, &c->d_wp); }
    if (verbose)
        printf("Best Config: (%d %d %d) algo=%s bm=%d bn=%d skinny=%d smem=%dKB time=%.3f\n", c->desc.ic, c->desc.oc,
               c->desc.iw, algo_label(best.algo), best.cfg.bm, best.cfg.bn,
               best.cfg.skinny, best.cfg.smem_kb, best_ms);
    if (best_ms < 1e29f) tuning_log_append(c, best, best_ms * 1e3f);
    return FC_OK;
}

int fc_conv_set_kernel_config(fc_conv *c, int bm, int bn, int variant, int smem_kb) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    FC_REQUIRE(bm >= 0 && bn >= 0 && variant >= 0 && variant <= 2 && smem_kb >= 0 && smem_kb <= 227, FC_ERR_INVALID_ARG,
               "kernel configuration (%d, %d, %d, %d) out of range", bm, bn, variant, smem_kb);
    c->cfg.bm = bm; c->cfg.bn = bn; c->cfg.skinny = variant; c->cfg.smem_kb = smem_kb;
    return FC_OK;
}

int fc_conv_get_kernel_config(const fc_conv *c, int *bm, int *bn, int *variant, int *smem_kb) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    if (bm) *bm = c->cfg.bm;
    if (bn) *bn = c->cfg.bn;
    if (variant) *variant = c->cfg.skinny;
    if (smem_kb) *smem_kb = c->cfg.smem_kb;
    return FC_OK;
}

int fc_conv_launches_per_forward(const fc_conv *c, int *launches) {
    FC_REQUIRE(c && launches, FC_ERR_INVALID_ARG, "NULL argument");
    *launches = c->algo == FC_ALGO_WINOGRAD ? wino_launches(c) : c->algo == FC_ALGO_DIRECT ? direct_launches(c) : igemm_launches(c);
    return FC_OK;
}

// ---- layer list (CUDA graph over several layers) ----------------------------------------------

struct fc_layer_list {
    fc_context *ctx;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    int launches;
    std::vector<fc_conv *> convs;
    std::vector<const float *> d_ins;
    std::vector<float *> d_outs;
    std::vector<cudaEvent_t> uploaded, computed;  // per layer, for the pipelined host forward
};

int fc_layer_list_create(fc_context *ctx, fc_conv *const *convs, const float *const *d_ins, float *const *d_outs,
                         int count, fc_layer_list **out) {
    FC_REQUIRE(ctx && convs && d_ins && d_outs && out, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(count > 0, FC_ERR_INVALID_ARG, "empty layer list");
    *out = nullptr;
    int launches = 0;
    for (int i = 0; i < count; ++i) {
        FC_REQUIRE(convs[i] && d_ins[i] && d_outs[i], FC_ERR_INVALID_ARG, "layer %d has a NULL member", i);
        FC_REQUIRE(convs[i]->ctx == ctx, FC_ERR_INVALID_ARG, "layer %d belongs to another context", i);
        launches += convs[i]->algo == FC_ALGO_WINOGRAD ? wino_launches(convs[i])
                    : convs[i]->algo == FC_ALGO_DIRECT ? direct_launches(convs[i]) : igemm_launches(convs[i]);
    }
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    // one eager pass first: kernel attributes are set and any error shows up outside the capture
    for (int i = 0; i < count; ++i) FC_PROPAGATE(conv_enqueue(convs[i], d_ins[i], d_outs[i], false));
    FC_PROPAGATE(sync_and_check_status(ctx));

    fc_layer_list *l = new (std::nothrow) fc_layer_list();
    FC_REQUIRE(l != nullptr, FC_ERR_OUT_OF_MEMORY, "host allocation failed");
    l->ctx = ctx;
    l->graph = nullptr;
    l->exec = nullptr;
    l->launches = launches;
    l->convs.assign(convs, convs + count);
    l->d_ins.assign(d_ins, d_ins + count);
    l->d_outs.assign(d_outs, d_outs + count);
    if (!graph_enabled()) {
        *out = l;
        return FC_OK;
    }
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    int st = FC_OK;
    if (e == cudaSuccess) {
        for (int i = 0; i < count && st == FC_OK; ++i) st = conv_enqueue(convs[i], d_ins[i], d_outs[i], false);
        e = cudaStreamEndCapture(ctx->stream, &l->graph);  // always end the capture, even after a failed enqueue
    }
    if (e == cudaSuccess && st == FC_OK) e = cudaGraphInstantiate(&l->exec, l->graph, 0);
    if (e != cudaSuccess || st != FC_OK) {
        if (e != cudaSuccess) set_error("capturing the layer list failed: %s", cudaGetErrorString(e));
        if (l->graph) cudaGraphDestroy(l->graph);
        delete l;
        cudaGetLastError();
        return e != cudaSuccess ? FC_ERR_CUDA : st;
    }
    *out = l;
    return FC_OK;
}

int fc_layer_list_forward(fc_layer_list *l) {
    FC_REQUIRE(l != nullptr, FC_ERR_INVALID_ARG, "list is NULL");
    if (l->exec == nullptr) {  // FASTCONV_GRAPH=0
        for (size_t i = 0; i < l->convs.size(); ++i) FC_PROPAGATE(conv_enqueue(l->convs[i], l->d_ins[i], l->d_outs[i], false));
        return FC_OK;
    }
    FC_CHECK_CUDA(cudaGraphLaunch(l->exec, l->ctx->stream));
    return FC_OK;
}

int fc_layer_list_forward_host(fc_layer_list *l, const float *const *h_ins, float *const *h_outs) {
    FC_REQUIRE(l && h_ins && h_outs, FC_ERR_INVALID_ARG, "NULL argument");
    fc_context *ctx = l->ctx;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    if (!ctx->copy_in) FC_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
    if (!ctx->copy_out) FC_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    const size_t n = l->convs.size();
    while (l->uploaded.size() < n) {
        cudaEvent_t a, b;
        FC_CHECK_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        FC_CHECK_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        l->uploaded.push_back(a);
        l->computed.push_back(b);
    }
    for (size_t i = 0; i < n; ++i) {
        fc_conv *c = l->convs[i];
        // a NULL host pointer means "chained": the layer reads what an earlier layer of the list wrote on the device
        // (or leaves its output there for a later one), so nothing is copied on that side
        float *din = const_cast<float *>(l->d_ins[i]);
        float *dout = l->d_outs[i];
        const size_t in_bytes = (size_t)c->desc.batch * c->desc.ic * c->desc.ih * c->desc.iw * sizeof(float);
        const size_t out_bytes = (size_t)c->desc.batch * c->desc.oc * c->oh * c->ow * sizeof(float);
        if (h_ins[i] != nullptr) {
            FC_CHECK_CUDA(cudaMemcpyAsync(din, h_ins[i], in_bytes, cudaMemcpyHostToDevice, ctx->copy_in));
            FC_CHECK_CUDA(cudaEventRecord(l->uploaded[i], ctx->copy_in));
            FC_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, l->uploaded[i], 0));
        }
        FC_PROPAGATE(conv_enqueue(c, din, dout, false));
        if (h_outs[i] != nullptr) {
            FC_CHECK_CUDA(cudaEventRecord(l->computed[i], ctx->stream));
            FC_CHECK_CUDA(cudaStreamWaitEvent(ctx->copy_out, l->computed[i], 0));
            FC_CHECK_CUDA(cudaMemcpyAsync(h_outs[i], dout, out_bytes, cudaMemcpyDeviceToHost, ctx->copy_out));
        }
    }
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->copy_out));
    return sync_and_check_status(ctx);
}

int fc_layer_list_launches(const fc_layer_list *l, int *n) {
    FC_REQUIRE(l && n, FC_ERR_INVALID_ARG, "NULL argument");
    *n = l->launches;
    return FC_OK;
}

int fc_layer_list_destroy(fc_layer_list *l) {
    if (!l) return FC_OK;
    cudaStreamSynchronize(l->ctx->stream);
    if (l->exec) cudaGraphExecDestroy(l->exec);
    if (l->graph) cudaGraphDestroy(l->graph);
    for (cudaEvent_t e : l->uploaded) cudaEventDestroy(e);
    for (cudaEvent_t e : l->computed) cudaEventDestroy(e);
    delete l;
    return FC_OK;
}

float fc_diff(const float *a, const float *b, int len) {
    int num = 0;
    double dif = 0.0;
    for (int i = 0; i < len; ++i) {
        const float err = fabsf(a[i] - b[i]);
        if (err > 1e-5f) {
            dif += err;
            ++num;
        }
    }
    return num == 0 ? 0.0f : (float)(dif / num);
}

}  // extern "C"
