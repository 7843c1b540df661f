// Several GPUs behind the C ABI: a communicator over the GPUs of one machine and layers sharded over it.
//
// The reference is a single-process CPU program; its only parallelism is the OpenMP split of the output-channel
// loop (winoF63ZC/winoF63ZC.cpp:1486-1544).  The two partitionings here are the ones the path offers naturally:
//   batch     images are independent: rank r runs the layer on images [b0, b1), no collective in the data path;
//   channels  output channels are independent: rank r owns channels [k0, k1) of a single-image layer, i.e. keeps
//             only its slice of the transformed filter (the dominant stream), reads the whole input, and its slab
//             of the NCHW output is contiguous.  The slabs are gathered either by the output transform itself
//             (stores into every rank's buffer over NVLink, step flags, bounded wait: fc_peer.cu) or by NCCL.
// The reduction over input channels is never split, so sharded == unsharded bit for bit.
//
// A communicator drives its ranks in one of two ways: ONE process that owns every GPU (fc_comm_init_all; the
// harness's -g N), or one process per GPU started by a launcher (fc_comm_init_env: RANK / WORLD_SIZE / LOCAL_RANK).
// In both the entry points act on the ranks local to the calling process.  NCCL is looked up at run time
// (libnccl.so.2), so the library loads on machines without it; a single process without the NCCL gather never
// needs it.
#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "fc_internal.h"

namespace fc {
namespace {

// ---- NCCL, resolved with dlopen -----------------------------------------------------------------
struct NcclId { char internal[128]; };
typedef void *NcclComm;
struct NcclApi {
    void *so;
    int (*GetUniqueId)(NcclId *);
    int (*CommInitRank)(NcclComm *, int, NcclId, int);
    int (*CommInitAll)(NcclComm *, int, const int *);
    int (*CommDestroy)(NcclComm);
    int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t);
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t);
    int (*Broadcast)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t);
    int (*GroupStart)();
    int (*GroupEnd)();
    const char *(*GetErrorString)(int);
};
constexpr int kNcclChar = 0, kNcclFloat = 7, kNcclDouble = 8, kNcclMax = 2;

int nccl_api(NcclApi **out) {
    static NcclApi api;
    static int state = 0;  // 0 = not tried, 1 = loaded, -1 = failed
    if (state == 0) {
        const char *name = getenv("FASTCONV_NCCL_LIB");
        api.so = dlopen(name && name[0] ? name : "libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        state = -1;
        if (api.so) {
            bool ok = true;
            auto sym = [&](const char *n) {
                void *p = dlsym(api.so, n);
                if (!p) ok = false;
                return p;
            };
            api.GetUniqueId = (int (*)(NcclId *))sym("ncclGetUniqueId");
            api.CommInitRank = (int (*)(NcclComm *, int, NcclId, int))sym("ncclCommInitRank");
            api.CommInitAll = (int (*)(NcclComm *, int, const int *))sym("ncclCommInitAll");
            api.CommDestroy = (int (*)(NcclComm))sym("ncclCommDestroy");
            api.AllGather = (int (*)(const void *, void *, size_t, int, NcclComm, cudaStream_t))sym("ncclAllGather");
            api.AllReduce = (int (*)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t))sym("ncclAllReduce");
            api.Broadcast = (int (*)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t))sym("ncclBroadcast");
            api.GroupStart = (int (*)())sym("ncclGroupStart");
            api.GroupEnd = (int (*)())sym("ncclGroupEnd");
            api.GetErrorString = (const char *(*)(int))sym("ncclGetErrorString");
            if (ok) state = 1;
        }
    }
    FC_REQUIRE(state == 1, FC_ERR_COMM, "NCCL (libnccl.so.2, or $FASTCONV_NCCL_LIB) could not be loaded: %s",
               dlerror() ? dlerror() : "a symbol is missing");
    *out = &api;
    return FC_OK;
}

#define FC_CHECK_NCCL(api, call)                                                                   \
    do {                                                                                           \
        int fc_nr__ = (call);                                                                      \
        if (fc_nr__ != 0) {                                                                        \
            fc::set_error("%s failed: %s (%s:%d)", #call, (api)->GetErrorString(fc_nr__), __FILE__, __LINE__); \
            return FC_ERR_COMM;                                                                    \
        }                                                                                          \
    } while (0)

}  // namespace
}  // namespace fc

using namespace fc;

struct fc_comm {
    int world, first_rank;
    bool one_process;                // this process owns every rank
    std::vector<fc_context *> ctx;   // local ranks, in rank order
    std::vector<NcclComm> nccl;      // one per local rank, created when first needed (or at init for several processes)
    // peer_base[l][r]: base of rank r's arena as local rank l sees it (own arena, a peer-enabled pointer of this
    // process, or an IPC mapping); empty until a channel-split layer with the peer gather asks for it
    std::vector<std::vector<char *>> peer_base;
    std::vector<std::vector<void *>> ipc_opened;  // mappings to close, per local rank
    bool peer_access_ok;
};

struct ShardPart {
    fc_conv *conv;        // NULL when the rank owns nothing (more ranks than images)
    int rank, local;      // world rank and index among this process's ranks
    int begin, end;       // images or output channels of this rank
    float *d_in, *d_out;  // batch split: the layer's own staging buffers.  Channel split: d_in only
    float *out[2];        // channel split: two whole-output buffers that alternate by step
    int *flags;           // channel split: int[world] step flags, then the step counter and the ticket
    int *step;
    unsigned *ticket;
    ScatterPublish pub;
    cudaEvent_t ev0, ev1;
};

struct fc_sharded_conv {
    fc_comm *comm;
    fc_conv_desc whole;
    int shard, gather, oh, ow;
    long long host_step;  // forwards enqueued so far (the device keeps its own count for the peer gather)
    std::vector<ShardPart> parts;
};

namespace {

int comm_ensure_nccl(fc_comm *c) {
    if (!c->nccl.empty()) return FC_OK;
    NcclApi *api;
    FC_PROPAGATE(nccl_api(&api));
    FC_REQUIRE(c->one_process, FC_ERR_COMM, "the communicator of a multi-process job is created at fc_comm_init_env");
    std::vector<int> devs;
    for (fc_context *x : c->ctx) devs.push_back(x->device);
    c->nccl.assign(c->ctx.size(), nullptr);
    FC_CHECK_NCCL(api, api->CommInitAll(c->nccl.data(), (int)devs.size(), devs.data()));
    return FC_OK;
}

// Small blobs of every rank to every rank, through host memory: mine = one blob per local rank, all = one per rank.
int comm_allgather_bytes(fc_comm *c, const void *mine, void *all, size_t bytes) {
    const int nlocal = (int)c->ctx.size();
    if (c->one_process) {
        memcpy(all, mine, bytes * nlocal);
        return FC_OK;
    }
    NcclApi *api;
    FC_PROPAGATE(nccl_api(&api));
    fc_context *x = c->ctx[0];
    FC_CHECK_CUDA(cudaSetDevice(x->device));
    void *d = nullptr;
    FC_PROPAGATE(fc_arena_alloc(x, bytes * (c->world + 1), &d));
    char *send = (char *)d, *recv = send + bytes;
    int st = FC_OK;
    auto run = [&]() -> int {
        FC_CHECK_CUDA(cudaMemcpyAsync(send, mine, bytes, cudaMemcpyHostToDevice, x->stream));
        FC_CHECK_NCCL(api, api->AllGather(send, recv, bytes, kNcclChar, c->nccl[0], x->stream));
        FC_CHECK_CUDA(cudaMemcpyAsync(all, recv, bytes * c->world, cudaMemcpyDeviceToHost, x->stream));
        FC_CHECK_CUDA(cudaStreamSynchronize(x->stream));
        return FC_OK;
    };
    st = run();
    fc_arena_free(x, d);
    return st;
}

// Makes every rank's arena addressable from every local rank (peer pointers inside one process, CUDA IPC between
// processes).
int comm_map_peers(fc_comm *c) {
    if (!c->peer_base.empty()) return FC_OK;
    const int nlocal = (int)c->ctx.size();
    FC_REQUIRE(c->world <= FC_MAX_PEERS, FC_ERR_UNSUPPORTED, "the peer gather takes at most %d ranks", FC_MAX_PEERS);
    std::vector<std::vector<char *>> base(nlocal, std::vector<char *>(c->world, nullptr));
    c->ipc_opened.assign(nlocal, std::vector<void *>());
    if (c->one_process) {
        FC_REQUIRE(c->peer_access_ok, FC_ERR_COMM, "these GPUs cannot address each other's memory (no peer access)");
        for (int l = 0; l < nlocal; ++l)
            for (int r = 0; r < c->world; ++r) base[l][r] = (char *)c->ctx[r]->slab;
    } else {
        std::vector<unsigned char> mine(FC_PEER_HANDLE_BYTES), all((size_t)FC_PEER_HANDLE_BYTES * c->world);
        size_t off = 0;
        FC_PROPAGATE(fc_peer_export(c->ctx[0], c->ctx[0]->slab, mine.data(), &off));
        FC_PROPAGATE(comm_allgather_bytes(c, mine.data(), all.data(), FC_PEER_HANDLE_BYTES));
        for (int r = 0; r < c->world; ++r) {
            if (r == c->first_rank) {
                base[0][r] = (char *)c->ctx[0]->slab;
                continue;
            }
            void *b = nullptr;
            FC_PROPAGATE(fc_peer_open(c->ctx[0], all.data() + (size_t)r * FC_PEER_HANDLE_BYTES, &b));
            c->ipc_opened[0].push_back(b);
            base[0][r] = (char *)b;
        }
    }
    c->peer_base.swap(base);
    return FC_OK;
}

int comm_sync_streams(fc_comm *c) {
    int st = FC_OK;
    for (fc_context *x : c->ctx) {
        const int s = fc_context_synchronize(x);
        if (s != FC_OK && st == FC_OK) st = s;
    }
    return st;
}

}  // namespace

extern "C" {

int fc_shard_range(int total, int world, int rank, int *begin, int *end) {
    FC_REQUIRE(begin && end, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(world >= 1 && rank >= 0 && rank < world && total >= 0, FC_ERR_INVALID_ARG, "bad rank %d of %d or extent %d",
               rank, world, total);
    const int base = total / world, extra = total % world;
    *begin = rank * base + (rank < extra ? rank : extra);
    *end = *begin + base + (rank < extra ? 1 : 0);
    return FC_OK;
}

int fc_comm_init_all(int ndev, const int *devices, size_t arena_bytes, fc_comm **out) {
    FC_REQUIRE(out != nullptr, FC_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    int have = 0;
    fc_device_count(&have);
    FC_REQUIRE(have > 0, FC_ERR_NO_DEVICE, "no CUDA device is visible; this library has no CPU path");
    FC_REQUIRE(ndev >= 1 && ndev <= have, FC_ERR_INVALID_ARG, "%d GPUs asked for, %d visible", ndev, have);
    fc_comm *c = new (std::nothrow) fc_comm();
    FC_REQUIRE(c != nullptr, FC_ERR_OUT_OF_MEMORY, "host allocation failed");
    c->world = ndev;
    c->first_rank = 0;
    c->one_process = true;
    c->peer_access_ok = true;
    for (int i = 0; i < ndev; ++i) {
        fc_context *x = nullptr;
        const int st = fc_context_create(devices ? devices[i] : i, arena_bytes, &x);
        if (st != FC_OK) {
            fc_comm_destroy(c);
            return st;
        }
        c->ctx.push_back(x);
    }
    for (int i = 0; i < ndev; ++i)
        for (int j = 0; j < ndev; ++j) {
            if (i == j) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, c->ctx[i]->device, c->ctx[j]->device);
            if (!can) {
                c->peer_access_ok = false;
                continue;
            }
            cudaSetDevice(c->ctx[i]->device);
            const cudaError_t e = cudaDeviceEnablePeerAccess(c->ctx[j]->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) c->peer_access_ok = false;
            cudaGetLastError();
        }
    *out = c;
    return FC_OK;
}

int fc_comm_init_env(int device, size_t arena_bytes, fc_comm **out) {
    FC_REQUIRE(out != nullptr, FC_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    auto env_int = [](const char *name, int fallback) {
        const char *e = getenv(name);
        return e && e[0] ? atoi(e) : fallback;
    };
    const int world = env_int("WORLD_SIZE", 1), rank = env_int("RANK", 0);
    if (device < 0) device = env_int("LOCAL_RANK", 0);
    FC_REQUIRE(world >= 1 && rank >= 0 && rank < world, FC_ERR_INVALID_ARG, "RANK=%d outside WORLD_SIZE=%d", rank, world);
    fc_comm *c = new (std::nothrow) fc_comm();
    FC_REQUIRE(c != nullptr, FC_ERR_OUT_OF_MEMORY, "host allocation failed");
    c->world = world;
    c->first_rank = rank;
    c->one_process = world == 1;
    c->peer_access_ok = true;
    fc_context *x = nullptr;
    int st = fc_context_create(device, arena_bytes, &x);
    if (st != FC_OK) {
        delete c;
        return st;
    }
    c->ctx.push_back(x);
    if (world == 1) {
        *out = c;
        return FC_OK;
    }
    // Rendezvous: rank 0 writes the NCCL id to a file that the other ranks of the same launch wait for.  The name is
    // $FASTCONV_COMM_ID_FILE, else built from what the ranks of one launch share: the launcher's process id and
    // MASTER_PORT.  One machine only, which is all this library drives.
    auto body = [&]() -> int {
        NcclApi *api;
        FC_PROPAGATE(nccl_api(&api));
        std::string path;
        const char *given = getenv("FASTCONV_COMM_ID_FILE");
        if (given && given[0]) {
            path = given;
        } else {
            const char *port = getenv("MASTER_PORT"), *run = getenv("TORCHELASTIC_RUN_ID");
            path = std::string("/tmp/fastconv_comm_") + std::to_string((long long)getppid()) + "_" + (port ? port : "0") +
                   "_" + (run ? run : "none") + ".id";
        }
        NcclId id;
        memset(&id, 0, sizeof id);
        if (rank == 0) {
            FC_CHECK_NCCL(api, api->GetUniqueId(&id));
            const std::string tmp = path + ".tmp";
            FILE *f = fopen(tmp.c_str(), "wb");
            FC_REQUIRE(f != nullptr, FC_ERR_COMM, "cannot write the rendezvous file %s", tmp.c_str());
            const size_t n = fwrite(&id, 1, sizeof id, f);
            fclose(f);
            FC_REQUIRE(n == sizeof id && rename(tmp.c_str(), path.c_str()) == 0, FC_ERR_COMM,
                       "cannot publish the rendezvous file %s", path.c_str());
        } else {
            const int limit_ms = env_int("FASTCONV_COMM_TIMEOUT_MS", 120000);
            bool got = false;
            for (int waited = 0; waited < limit_ms && !got; waited += 20) {
                FILE *f = fopen(path.c_str(), "rb");
                if (f) {
                    got = fread(&id, 1, sizeof id, f) == sizeof id;
                    fclose(f);
                }
                if (!got) usleep(20000);
            }
            FC_REQUIRE(got, FC_ERR_COMM, "rank %d waited %d ms for the rendezvous file %s of rank 0", rank, limit_ms,
                       path.c_str());
        }
        FC_CHECK_CUDA(cudaSetDevice(x->device));
        c->nccl.assign(1, nullptr);
        FC_CHECK_NCCL(api, api->CommInitRank(&c->nccl[0], world, id, rank));  // returns once every rank has joined
        if (rank == 0) unlink(path.c_str());
        return FC_OK;
    };
    st = body();
    if (st != FC_OK) {
        c->nccl.clear();
        fc_comm_destroy(c);
        return st;
    }
    *out = c;
    return FC_OK;
}

int fc_comm_size(const fc_comm *c, int *world, int *local_count, int *first_rank) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "communicator is NULL");
    if (world) *world = c->world;
    if (local_count) *local_count = (int)c->ctx.size();
    if (first_rank) *first_rank = c->first_rank;
    return FC_OK;
}

int fc_comm_context(fc_comm *c, int local_index, fc_context **ctx) {
    FC_REQUIRE(c && ctx, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(local_index >= 0 && local_index < (int)c->ctx.size(), FC_ERR_INVALID_ARG, "local rank %d of %zu", local_index,
               c->ctx.size());
    *ctx = c->ctx[local_index];
    return FC_OK;
}

int fc_comm_barrier(fc_comm *c) {
    FC_REQUIRE(c != nullptr, FC_ERR_INVALID_ARG, "communicator is NULL");
    FC_PROPAGATE(comm_sync_streams(c));
    if (c->one_process) return FC_OK;
    double v = 0.0;
    return fc_comm_allreduce_max(c, &v);
}

int fc_comm_allreduce_max(fc_comm *c, double *values) {
    FC_REQUIRE(c && values, FC_ERR_INVALID_ARG, "NULL argument");
    const int nlocal = (int)c->ctx.size();
    double m = values[0];
    for (int i = 1; i < nlocal; ++i) m = values[i] > m ? values[i] : m;
    if (!c->one_process) {
        NcclApi *api;
        FC_PROPAGATE(nccl_api(&api));
        fc_context *x = c->ctx[0];
        FC_CHECK_CUDA(cudaSetDevice(x->device));
        void *d = nullptr;
        FC_PROPAGATE(fc_arena_alloc(x, 256, &d));
        auto run = [&]() -> int {
            FC_CHECK_CUDA(cudaMemcpyAsync(d, &m, sizeof m, cudaMemcpyHostToDevice, x->stream));
            FC_CHECK_NCCL(api, api->AllReduce(d, d, 1, kNcclDouble, kNcclMax, c->nccl[0], x->stream));
            FC_CHECK_CUDA(cudaMemcpyAsync(&m, d, sizeof m, cudaMemcpyDeviceToHost, x->stream));
            FC_CHECK_CUDA(cudaStreamSynchronize(x->stream));
            return FC_OK;
        };
        const int st = run();
        fc_arena_free(x, d);
        FC_PROPAGATE(st);
    }
    for (int i = 0; i < nlocal; ++i) values[i] = m;
    return FC_OK;
}

int fc_comm_allgather(fc_comm *c, const void *mine, void *all, size_t bytes) {
    FC_REQUIRE(c && mine && all && bytes > 0, FC_ERR_INVALID_ARG, "bad argument");
    return comm_allgather_bytes(c, mine, all, bytes);
}

int fc_comm_destroy(fc_comm *c) {
    if (!c) return FC_OK;
    // an exporter must not free memory that a peer still maps: everyone stops, unmaps, and only then frees
    const bool joined = !c->nccl.empty() || c->one_process;
    if (joined && !c->ctx.empty()) fc_comm_barrier(c);
    for (size_t l = 0; l < c->ipc_opened.size(); ++l)
        for (void *b : c->ipc_opened[l]) fc_peer_close(c->ctx[l], b);
    if (joined && !c->ctx.empty() && !c->ipc_opened.empty()) fc_comm_barrier(c);
    NcclApi *api = nullptr;
    if (!c->nccl.empty() && nccl_api(&api) == FC_OK)
        for (size_t i = 0; i < c->nccl.size(); ++i)
            if (c->nccl[i]) {
                cudaSetDevice(c->ctx[i]->device);
                api->CommDestroy(c->nccl[i]);
            }
    for (fc_context *x : c->ctx) fc_context_destroy(x);
    delete c;
    return FC_OK;
}

// ---- a layer sharded over the communicator ------------------------------------------------------

static void sharded_release(fc_sharded_conv *s, bool all_ranks_arrive) {
    fc_comm *c = s->comm;
    // no rank may still be storing into buffers that are about to go back to the arena
    if (all_ranks_arrive && s->shard == FC_SHARD_CHANNELS) fc_comm_barrier(c);
    for (ShardPart &p : s->parts) {
        fc_context *x = c->ctx[p.local];
        cudaSetDevice(x->device);
        if (p.conv) fc_conv_destroy(p.conv);
        for (float *b : p.out)
            if (b) fc_arena_free(x, b);
        if (p.flags) fc_arena_free(x, p.flags);
        if (p.ev0) cudaEventDestroy(p.ev0);
        if (p.ev1) cudaEventDestroy(p.ev1);
    }
    delete s;
}

int fc_sharded_conv_destroy(fc_sharded_conv *s) {
    if (s) sharded_release(s, true);
    return FC_OK;
}

int fc_sharded_conv_create(fc_comm *c, const fc_conv_desc *whole, int algo, int mode, int shard, int gather,
                           const float *h_kernel, fc_sharded_conv **out) {
    FC_REQUIRE(c && whole && h_kernel && out, FC_ERR_INVALID_ARG, "NULL argument");
    *out = nullptr;
    FC_REQUIRE(shard == FC_SHARD_BATCH || shard == FC_SHARD_CHANNELS, FC_ERR_INVALID_ARG, "unknown partitioning %d", shard);
    FC_REQUIRE(gather == FC_GATHER_PEER || gather == FC_GATHER_NCCL, FC_ERR_INVALID_ARG, "unknown gather %d", gather);
    int oh, ow;
    FC_PROPAGATE(fc_conv_output_size(whole, &oh, &ow));
    if (shard == FC_SHARD_CHANNELS) {
        FC_REQUIRE(whole->batch == 1, FC_ERR_UNSUPPORTED, "the channel split takes one image (batch %d)", whole->batch);
        FC_REQUIRE(whole->group == 1, FC_ERR_UNSUPPORTED, "the channel split takes ungrouped layers");
        FC_REQUIRE(whole->oc >= c->world, FC_ERR_UNSUPPORTED, "%d output channels for %d ranks", whole->oc, c->world);
        if (gather == FC_GATHER_PEER) FC_PROPAGATE(comm_map_peers(c));
        if (gather == FC_GATHER_NCCL) FC_PROPAGATE(comm_ensure_nccl(c));
    }
    fc_sharded_conv *s = new (std::nothrow) fc_sharded_conv();
    FC_REQUIRE(s != nullptr, FC_ERR_OUT_OF_MEMORY, "host allocation failed");
    s->comm = c;
    s->whole = *whole;
    s->shard = shard;
    s->gather = gather;
    s->oh = oh;
    s->ow = ow;
    s->host_step = 0;
    const int nlocal = (int)c->ctx.size();
    const size_t out_elems = (size_t)whole->oc * oh * ow;  // one image
    const size_t k_per_oc = (size_t)(whole->ic / whole->group) * whole->kh * whole->kw;
    auto fail = [&](int st) {  // a local failure: the other ranks are not waited for
        sharded_release(s, false);
        return st;
    };
    for (int l = 0; l < nlocal; ++l) {
        ShardPart p;
        memset(&p, 0, sizeof p);
        p.local = l;
        p.rank = c->first_rank + l;
        fc_context *x = c->ctx[l];
        fc_shard_range(shard == FC_SHARD_BATCH ? whole->batch : whole->oc, c->world, p.rank, &p.begin, &p.end);
        s->parts.push_back(p);
        ShardPart &q = s->parts.back();
        if (cudaSetDevice(x->device) != cudaSuccess || cudaEventCreate(&q.ev0) != cudaSuccess ||
            cudaEventCreate(&q.ev1) != cudaSuccess) {
            set_error("event creation failed on device %d", x->device);
            return fail(FC_ERR_CUDA);
        }
        if (q.end == q.begin) continue;  // more ranks than images
        fc_conv_desc d = *whole;
        const float *w = h_kernel;
        if (shard == FC_SHARD_BATCH) {
            d.batch = q.end - q.begin;
        } else {
            d.oc = q.end - q.begin;
            w = h_kernel + (size_t)q.begin * k_per_oc;
        }
        int st = fc_conv_create(x, &d, algo, mode, w, &q.conv);
        if (st != FC_OK) return fail(st);
        fc_conv_device_buffers(q.conv, &q.d_in, &q.d_out);
        if (shard == FC_SHARD_CHANNELS) {
            int a = 0;
            fc_conv_algorithm(q.conv, &a);
            if (gather == FC_GATHER_PEER && a != FC_ALGO_WINOGRAD) {
                set_error("the peer gather is built into the Winograd output transform; this layer resolved to algorithm %d "
                          "(use the NCCL gather)", a);
                return fail(FC_ERR_UNSUPPORTED);
            }
            void *b = nullptr;
            for (int i = 0; i < 2; ++i) {
                st = fc_arena_alloc(x, out_elems * sizeof(float), &b);
                if (st != FC_OK) return fail(st);
                q.out[i] = (float *)b;
            }
            st = fc_arena_alloc(x, 256, &b);
            if (st != FC_OK) return fail(st);
            q.flags = (int *)b;
            q.step = q.flags + FC_MAX_PEERS;
            q.ticket = (unsigned *)(q.flags + FC_MAX_PEERS + 1);
            if (cudaMemsetAsync(q.flags, 0, 256, x->stream) != cudaSuccess || cudaStreamSynchronize(x->stream) != cudaSuccess) {
                set_error("clearing the step flags failed");
                return fail(FC_ERR_CUDA);
            }
        }
    }
    if (shard == FC_SHARD_CHANNELS && gather == FC_GATHER_PEER) {
        // every rank learns where the others keep their two output buffers and their flags (offsets into the arenas)
        struct Offsets { unsigned long long out[2], flags; };
        std::vector<Offsets> mine(nlocal), all(c->world);
        for (int l = 0; l < nlocal; ++l) {
            const ShardPart &q = s->parts[l];
            const char *base = (const char *)c->ctx[l]->slab;
            mine[l].out[0] = (unsigned long long)((const char *)q.out[0] - base);
            mine[l].out[1] = (unsigned long long)((const char *)q.out[1] - base);
            mine[l].flags = (unsigned long long)((const char *)q.flags - base);
        }
        int st = comm_allgather_bytes(c, mine.data(), all.data(), sizeof(Offsets));
        if (st != FC_OK) return fail(st);
        for (int l = 0; l < nlocal; ++l) {
            ShardPart &q = s->parts[l];
            memset(&q.pub, 0, sizeof q.pub);
            q.pub.count = c->world;
            q.pub.rank = q.rank;
            q.pub.step = q.step;
            q.pub.ticket = q.ticket;
            for (int r = 0; r < c->world; ++r) {
                char *b = c->peer_base[l][r];
                for (int i = 0; i < 2; ++i) q.pub.base[i][r] = (float *)(b + all[r].out[i]) + (size_t)q.begin * oh * ow;
                q.pub.flags[r] = (int *)(b + all[r].flags);
            }
        }
        // nobody publishes before everybody's flags are cleared and known
        st = fc_comm_barrier(c);
        if (st != FC_OK) return fail(st);
    }
    *out = s;
    return FC_OK;
}

int fc_sharded_conv_part(fc_sharded_conv *s, int local_index, fc_conv **conv, float **d_in, float **d_out, int *begin,
                         int *end) {
    FC_REQUIRE(s != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    FC_REQUIRE(local_index >= 0 && local_index < (int)s->parts.size(), FC_ERR_INVALID_ARG, "local rank %d of %zu",
               local_index, s->parts.size());
    const ShardPart &p = s->parts[local_index];
    if (conv) *conv = p.conv;
    if (d_in) *d_in = p.d_in;
    if (d_out) *d_out = s->shard == FC_SHARD_BATCH ? p.d_out : p.out[s->host_step & 1];
    if (begin) *begin = p.begin;
    if (end) *end = p.end;
    return FC_OK;
}

int fc_sharded_conv_upload(fc_sharded_conv *s, const float *h_in) {
    FC_REQUIRE(s && h_in, FC_ERR_INVALID_ARG, "NULL argument");
    fc_comm *c = s->comm;
    const fc_conv_desc &w = s->whole;
    const size_t img = (size_t)w.ic * w.ih * w.iw;
    const int first = s->parts.empty() ? 0 : s->parts[0].begin;
    for (ShardPart &p : s->parts) {
        if (!p.conv) continue;
        fc_context *x = c->ctx[p.local];
        FC_CHECK_CUDA(cudaSetDevice(x->device));
        // batch split: h_in holds the images of this process's ranks back to back; channel split: the one image
        const float *src = s->shard == FC_SHARD_BATCH ? h_in + (size_t)(p.begin - first) * img : h_in;
        const size_t n = s->shard == FC_SHARD_BATCH ? (size_t)(p.end - p.begin) * img : img;
        FC_CHECK_CUDA(cudaMemcpyAsync(p.d_in, src, n * sizeof(float), cudaMemcpyHostToDevice, x->stream));
    }
    return comm_sync_streams(c);
}

int fc_sharded_conv_forward(fc_sharded_conv *s) {
    FC_REQUIRE(s != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    fc_comm *c = s->comm;
    if (s->shard == FC_SHARD_BATCH) {
        for (ShardPart &p : s->parts)
            if (p.conv) FC_PROPAGATE(fc_conv_forward_device(p.conv, p.d_in, p.d_out));
        return FC_OK;
    }
    s->host_step += 1;
    const int which = (int)(s->host_step & 1);
    const size_t page = (size_t)s->oh * s->ow;
    if (s->gather == FC_GATHER_PEER) {
        for (ShardPart &p : s->parts) FC_PROPAGATE(conv_forward_scatter_publish(p.conv, p.d_in, p.pub));
        return FC_OK;
    }
    NcclApi *api;
    FC_PROPAGATE(nccl_api(&api));
    for (ShardPart &p : s->parts)
        FC_PROPAGATE(fc_conv_forward_device(p.conv, p.d_in, p.out[which] + (size_t)p.begin * page));
    const bool even = s->whole.oc % c->world == 0;
    FC_CHECK_NCCL(api, api->GroupStart());
    for (ShardPart &p : s->parts) {
        fc_context *x = c->ctx[p.local];
        if (even) {  // the slab is a contiguous, equal-sized piece of the NCHW output: one in-place all-gather
            const size_t count = (size_t)(p.end - p.begin) * page;
            FC_CHECK_NCCL(api, api->AllGather(p.out[which] + (size_t)p.begin * page, p.out[which], count, kNcclFloat,
                                              c->nccl[p.local], x->stream));
        } else {
            for (int r = 0; r < c->world; ++r) {
                int b, e;
                fc_shard_range(s->whole.oc, c->world, r, &b, &e);
                float *at = p.out[which] + (size_t)b * page;
                FC_CHECK_NCCL(api, api->Broadcast(at, at, (size_t)(e - b) * page, kNcclFloat, r, c->nccl[p.local], x->stream));
            }
        }
    }
    FC_CHECK_NCCL(api, api->GroupEnd());
    return FC_OK;
}

int fc_sharded_conv_wait(fc_sharded_conv *s) {
    FC_REQUIRE(s != nullptr, FC_ERR_INVALID_ARG, "layer is NULL");
    if (s->shard != FC_SHARD_CHANNELS || s->gather != FC_GATHER_PEER) return FC_OK;  // stream order is enough
    for (ShardPart &p : s->parts) {
        FC_CHECK_CUDA(cudaSetDevice(s->comm->ctx[p.local]->device));  // one process may drive several GPUs
        FC_PROPAGATE(launch_peer_wait_published(s->comm->ctx[p.local], p.flags, s->comm->world, p.step));
    }
    return FC_OK;
}

int fc_sharded_conv_download(fc_sharded_conv *s, float *h_out) {
    FC_REQUIRE(s && h_out, FC_ERR_INVALID_ARG, "NULL argument");
    fc_comm *c = s->comm;
    const fc_conv_desc &w = s->whole;
    const size_t img = (size_t)w.oc * s->oh * s->ow;
    if (s->shard == FC_SHARD_CHANNELS) {  // every rank holds the whole output; the first local one delivers it
        ShardPart &p = s->parts[0];
        fc_context *x = c->ctx[p.local];
        FC_CHECK_CUDA(cudaSetDevice(x->device));
        long long step = s->host_step;
        if (s->gather == FC_GATHER_PEER) {  // the device keeps the count (a graph may have replayed the layer)
            int dev_step = 0;
            FC_CHECK_CUDA(cudaMemcpyAsync(&dev_step, p.step, sizeof dev_step, cudaMemcpyDeviceToHost, x->stream));
            FC_CHECK_CUDA(cudaStreamSynchronize(x->stream));
            step = dev_step;
        }
        FC_CHECK_CUDA(cudaMemcpyAsync(h_out, p.out[step & 1], img * sizeof(float), cudaMemcpyDeviceToHost, x->stream));
        return comm_sync_streams(c);
    }
    const int first = s->parts.empty() ? 0 : s->parts[0].begin;
    for (ShardPart &p : s->parts) {
        if (!p.conv) continue;
        fc_context *x = c->ctx[p.local];
        FC_CHECK_CUDA(cudaSetDevice(x->device));
        FC_CHECK_CUDA(cudaMemcpyAsync(h_out + (size_t)(p.begin - first) * img, p.d_out, (size_t)(p.end - p.begin) * img * sizeof(float),
                                      cudaMemcpyDeviceToHost, x->stream));
    }
    return comm_sync_streams(c);
}

int fc_sharded_conv_forward_host(fc_sharded_conv *s, const float *h_in, float *h_out) {
    FC_PROPAGATE(fc_sharded_conv_upload(s, h_in));
    FC_PROPAGATE(fc_sharded_conv_forward(s));
    FC_PROPAGATE(fc_sharded_conv_wait(s));
    return fc_sharded_conv_download(s, h_out);
}

int fc_sharded_conv_time_device(fc_sharded_conv *s, int warmup, int iters, float *ms_per_iter) {
    FC_REQUIRE(s && ms_per_iter, FC_ERR_INVALID_ARG, "NULL argument");
    FC_REQUIRE(iters > 0 && warmup >= 0, FC_ERR_INVALID_ARG, "iters must be positive");
    fc_comm *c = s->comm;
    for (int i = 0; i < warmup; ++i) {
        FC_PROPAGATE(fc_sharded_conv_forward(s));
        FC_PROPAGATE(fc_sharded_conv_wait(s));
    }
    FC_PROPAGATE(fc_comm_barrier(c));
    for (ShardPart &p : s->parts) {
        FC_CHECK_CUDA(cudaSetDevice(c->ctx[p.local]->device));
        FC_CHECK_CUDA(cudaEventRecord(p.ev0, c->ctx[p.local]->stream));
    }
    for (int i = 0; i < iters; ++i) {
        FC_PROPAGATE(fc_sharded_conv_forward(s));
        FC_PROPAGATE(fc_sharded_conv_wait(s));
    }
    for (ShardPart &p : s->parts) {
        FC_CHECK_CUDA(cudaSetDevice(c->ctx[p.local]->device));
        FC_CHECK_CUDA(cudaEventRecord(p.ev1, c->ctx[p.local]->stream));
    }
    FC_PROPAGATE(comm_sync_streams(c));
    std::vector<double> ms(s->parts.size(), 0.0);
    for (size_t i = 0; i < s->parts.size(); ++i) {
        float t = 0.f;
        FC_CHECK_CUDA(cudaEventElapsedTime(&t, s->parts[i].ev0, s->parts[i].ev1));
        ms[i] = t / iters;
    }
    FC_PROPAGATE(fc_comm_allreduce_max(c, ms.data()));  // the slowest rank is the time of the job
    *ms_per_iter = (float)ms[0];
    return FC_OK;
}

}  // extern "C"
