// Peer-memory plumbing of the channel-split (K-sharded) layer: one process per GPU, every rank's output and
// flag buffers exported with CUDA IPC and mapped by the other ranks, so that a kernel of one GPU can store
// into the buffers of the others over NVLink.  The reference is a single-process CPU program: nothing here
// mirrors a reference interface.
//
// Protocol of one forward (step s, monotonically increasing):
//   1. the output transform of rank r stores its channel slab into the output buffer of every rank;
//   2. a one-warp kernel, launched after it in the same stream (so all of those stores are complete),
//      writes s into flags[r] of every rank;
//   3. a one-warp kernel on every rank polls its own flag array until all ranks have published s.
// No kernel of one GPU waits for a kernel of the SAME GPU, the wait of step 3 has an iteration limit and
// reports FC_ERR_TIMEOUT through the context status word instead of spinning forever, and only plain stores
// and loads cross NVLink (no switch-side reduction or replication objects, nothing that needs a peer to stay alive).
#include "fc_internal.h"

#include <cstdlib>
#include <cstring>

namespace fc {

namespace {

struct FlagPtrs {
    int *p[FC_MAX_PEERS];
};

__global__ void peer_publish_kernel(FlagPtrs flags, int world, int rank, int step) {
    const int r = threadIdx.x;
    if (r < world) {
        __threadfence_system();
        *reinterpret_cast<volatile int *>(flags.p[r] + rank) = step;
        __threadfence_system();
    }
}

// How long a wait polls before it gives up: fc_context_set_wait_limit_ms, initially $FASTCONV_PEER_WAIT_MS
// milliseconds (default 5000), at about 250 ns per poll.  Generous on purpose: ranks may be seconds apart at start-up (module loading, one rank still planning or
// tuning); the limit exists so that a rank whose peer has died returns an error instead of spinning for ever.  After
// a timeout the gathered output buffer is undefined.
constexpr long long POLLS_PER_MS = 4000;

__global__ void peer_wait_kernel(const int *flags, int world, int step, const int *d_step, unsigned polls, int *status) {
    const int r = threadIdx.x;
    if (r >= world) return;
    if (d_step != nullptr) step = *reinterpret_cast<const volatile int *>(d_step);  // this rank's own published count
    const volatile int *f = flags + r;
    for (unsigned i = 0; i < polls; ++i) {
        if (*f - step >= 0) {  // difference, so that a wrapped counter still compares
            __threadfence_system();
            return;
        }
        __nanosleep(200);
    }
    atomicExch(status, (int)FC_ERR_TIMEOUT);
}

}  // namespace

unsigned default_peer_wait_polls() {
    const char *e = getenv("FASTCONV_PEER_WAIT_MS");
    long long ms = e ? atoll(e) : 5000;
    if (ms < 1) ms = 1;
    if (ms > 600000) ms = 600000;
    return (unsigned)(ms * POLLS_PER_MS);
}

int launch_peer_publish(fc_context *ctx, int *const *flags, int world, int rank, int step) {
    FlagPtrs f;
    memset(&f, 0, sizeof f);
    for (int r = 0; r < world; ++r) f.p[r] = flags[r];
    // an ordinary launch (no programmatic overlap): it must not start before the stores of the transform are done
    peer_publish_kernel<<<1, 32, 0, ctx->stream>>>(f, world, rank, step);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

int launch_peer_wait(fc_context *ctx, const int *flags, int world, int step) {
    peer_wait_kernel<<<1, 32, 0, ctx->stream>>>(flags, world, step, nullptr, ctx->peer_wait_polls, ctx->d_status);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

int launch_peer_wait_published(fc_context *ctx, const int *flags, int world, const int *d_step) {
    // an ordinary launch: it starts after the scatter kernel before it has completed, *d_step included
    peer_wait_kernel<<<1, 32, 0, ctx->stream>>>(flags, world, 0, d_step, ctx->peer_wait_polls, ctx->d_status);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc

using namespace fc;

extern "C" {

int fc_peer_export(fc_context *ctx, const void *dptr, unsigned char handle[FC_PEER_HANDLE_BYTES], size_t *offset) {
    FC_REQUIRE(ctx && dptr && handle && offset, FC_ERR_INVALID_ARG, "NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == FC_PEER_HANDLE_BYTES, "IPC handle size");
    const char *base = static_cast<const char *>(ctx->slab), *p = static_cast<const char *>(dptr);
    FC_REQUIRE(p >= base && p < base + ctx->arena.capacity(), FC_ERR_INVALID_ARG,
               "pointer %p does not belong to the context's arena", dptr);
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    FC_CHECK_CUDA(cudaIpcGetMemHandle(&h, ctx->slab));
    memcpy(handle, &h, sizeof h);
    *offset = (size_t)(p - base);
    return FC_OK;
}

int fc_peer_open(fc_context *ctx, const unsigned char handle[FC_PEER_HANDLE_BYTES], void **base) {
    FC_REQUIRE(ctx && handle && base, FC_ERR_INVALID_ARG, "NULL argument");
    *base = nullptr;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    cudaError_t e = cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        set_error("cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return FC_ERR_COMM;
    }
    return FC_OK;
}

int fc_peer_close(fc_context *ctx, void *base) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    if (!base) return FC_OK;
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    FC_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
    cudaError_t e = cudaIpcCloseMemHandle(base);
    if (e != cudaSuccess) {
        set_error("cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return FC_ERR_COMM;
    }
    return FC_OK;
}

int fc_context_set_wait_limit_ms(fc_context *ctx, int ms) {
    FC_REQUIRE(ctx != nullptr, FC_ERR_INVALID_ARG, "context is NULL");
    FC_REQUIRE(ms >= 1 && ms <= 600000, FC_ERR_INVALID_ARG, "wait limit of %d ms outside 1..600000", ms);
    ctx->peer_wait_polls = (unsigned)(ms * POLLS_PER_MS);
    return FC_OK;
}

int fc_peer_wait(fc_context *ctx, const int *d_flags, int world, int step) {
    FC_REQUIRE(ctx && d_flags, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(world >= 1 && world <= FC_MAX_PEERS, FC_ERR_INVALID_ARG, "world %d outside 1..%d", world, FC_MAX_PEERS);
    FC_CHECK_CUDA(cudaSetDevice(ctx->device));
    return launch_peer_wait(ctx, d_flags, world, step);
}

}  // extern "C"
