/*
 * fastconv_b200 -- C ABI of the B200 (sm_100a) convolution-layer hot path.
 *
 * This is the drop-in boundary: everything FastConv's operator classes
 * (ConvWinoF63ZCLayer, ConvIm2colLayer) call below their Init()/Forward()
 * is replaced by the entry points declared here.  Plain C types only; device
 * buffers are raw pointers obtained from the arena functions (or any CUDA
 * allocation of the caller's).  Each declaration cites the reference
 * interface it replaces as path:line inside the FastConv tree.
 *
 * Conventions
 *   - every function returns FC_OK (0) or a negative fc_status; on failure
 *     fc_last_error() holds a message for the calling thread.
 *   - tensors are fp32 NCHW: input [n][ic][ih][iw], kernel [oc][ic][kh][kw],
 *     output [n][oc][oh][ow]; oh/ow follow conv_layer.h:68-69.
 *   - a context is bound to one GPU and one stream; it is not re-entrant
 *     (the reference layers are not either: shared workspaces).
 *   - there is no CPU fallback: without a usable GPU fc_context_create fails.
 */
#ifndef FASTCONV_B200_H_
#define FASTCONV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FC_ABI_VERSION 1

typedef enum fc_status {
    FC_OK = 0,
    FC_ERR_INVALID_ARG = -1,   /* NULL operand, non-positive size, bad enum            */
    FC_ERR_UNSUPPORTED = -2,   /* shape the requested algorithm cannot compute          */
    FC_ERR_OUT_OF_MEMORY = -3, /* arena exhausted or cudaMalloc failed                   */
    FC_ERR_CUDA = -4,          /* a CUDA runtime / driver call failed                    */
    FC_ERR_NO_DEVICE = -5,     /* no CUDA device, or not compute capability 10.x         */
    FC_ERR_TIMEOUT = -6,       /* a bounded device-side wait gave up (kernel reported)   */
    FC_ERR_COMM = -7           /* multi-GPU setup / exchange failed                      */
} fc_status;

/* Same numbering as nnp_convolution_algorithm, utility/helper.h:94-103. */
typedef enum fc_algorithm {
    FC_ALGO_AUTO = 0,
    FC_ALGO_DIRECT = 1, /* the reference's case is empty (ConvTest.cpp:369-371); here: direct convolution on the tensor
                           cores for ungrouped layers of stride 1 or 2 in FC_MATH_TF32, the implicit-GEMM kernel for anything else */
    FC_ALGO_IM2COL = 2,
    FC_ALGO_WINOGRAD = 3
} fc_algorithm;

/* Arithmetic of the multiply-accumulate stage. */
typedef enum fc_math_mode {
    FC_MATH_FP32_MIRRORED = 0, /* FFMA, one fused multiply-add per reduction step in ascending order:
                                  bit-identical to the reference's accumulation chain            */
    FC_MATH_3XTF32 = 1,        /* tcgen05 tensor cores, hi/lo TF32 split, fp32 accumulate: rel-L2 <= 1e-5.  The stage
                                  entry points run exactly that; a planned Winograd layer of at most 64 input channels
                                  runs the fp32 kernels instead (exact, and faster on so short a reduction;
                                  $FASTCONV_3XTF32_MIN_IC moves the border), fc_conv_math_mode says which       */
    FC_MATH_TF32 = 2,          /* tcgen05 tensor cores, one TF32 pass per reduction step.  The stage entry points
                                  (fc_wino_*, fc_igemm_*) run exactly that.  For a planned layer (fc_conv_create) the
                                  mode stands for its tolerance, rel-L2 <= 3e-3 against the fp32 result: one TF32 pass
                                  through F(6x6,3x3) measures 6.4e-3, so a Winograd-eligible layer runs the direct
                                  tensor-core kernel in TF32 or, where that cannot run or Winograd was asked for by
                                  name, the Winograd path in FC_MATH_3XTF32; every other layer runs in one TF32 pass.
                                  fc_conv_math_mode reports the arithmetic the layer was planned with.             */
    FC_MATH_TF32_U16 = 4,      /* fc_conv_create only; a reduced-precision mode outside every stated tolerance, like
                                  FC_MATH_TF32_UNBOUNDED (same 6.4e-3 on Winograd layers): the transformed filter of a
                                  Winograd layer is STORED as fp16 (TF32's own 11-bit significand) scaled per position by
                                  a power of two, which halves the stream that bounds single-image layers with many
                                  channels; it is expanded in shared memory and multiplied in one TF32 pass.  Layers it
                                  does not fit (at most 64 output channels, 128 tiles or more, other algorithms) run as
                                  in FC_MATH_TF32_UNBOUNDED; fc_conv_math_mode tells which.                          */
    FC_MATH_TF32_UNBOUNDED = 3 /* fc_conv_create only: one TF32 pass on every path, F(6x6,3x3) included, whatever the
                                  error (6.4e-3 rel-L2 on Winograd layers).  Faster than FC_MATH_TF32 on layers with
                                  many channels at small batch; outside the stated tolerance, hence the extra name. */
} fc_math_mode;

typedef struct fc_conv_desc {
    int32_t batch; /* images; the reference is batch 1 (no N anywhere in conv_layer.h:121-148) */
    int32_t ic, ih, iw;
    int32_t oc, kh, kw;
    int32_t sh, sw;
    int32_t pad_left, pad_right, pad_top, pad_bottom;
    int32_t group; /* parsed but unused by every reference path (conv_layer.h:27).  Here: must divide ic and oc;
                    * group > 1 runs the implicit GEMM once per group (weights [oc][ic/group][kh][kw]), group == ic a
                    * depthwise kernel; the Winograd stages and the stage-level implicit GEMM take group 1 only */
} fc_conv_desc;

typedef struct fc_context fc_context; /* one GPU + stream + device arena */
typedef struct fc_conv fc_conv;       /* one planned layer: weights, workspaces, kernels */

/* ---- library ------------------------------------------------------------- */
int fc_abi_version(void);
const char *fc_status_string(int status);
const char *fc_last_error(void);
int fc_device_count(int *count);

/* ---- context + device arena ----------------------------------------------
 * Replaces the host allocators of utility/mempool.h:23-71 (CommonMemPool::
 * Request/Alloc/GetPtr/Free, PrivateMemPool::Alloc/GetSize/Free/FreeAll/
 * PrintStats) and _mm_malloc/_mm_free (utility/common.cpp:26-49): one
 * cudaMalloc'd slab per context, sub-allocated with 256-byte alignment. */
int fc_context_create(int device, size_t arena_bytes, fc_context **out);
int fc_context_destroy(fc_context *ctx);
int fc_context_synchronize(fc_context *ctx);
int fc_context_device(const fc_context *ctx, int *device);
/* What a roofline needs to know about the GPU behind a context: the number of SMs and the maximum SM clock in MHz
 * (FP32 pipe peak = sm_count * 128 lanes * 2 flop * clock).  No reference counterpart; its nearest relative is
 * get_cache_info, utility/common.cpp:56-181, which reads the cache sizes the reference's tuner blocks for. */
int fc_context_info(const fc_context *ctx, int *sm_count, int *sm_clock_max_mhz);
/* the context's cudaStream_t, for callers that enqueue their own work in order with the library's */
int fc_context_stream(const fc_context *ctx, void **stream);
/* PrivateMemPool::Alloc / GetSize / Free / FreeAll / PrintStats */
int fc_arena_alloc(fc_context *ctx, size_t bytes, void **dptr);
int fc_arena_size_of(fc_context *ctx, const void *dptr, size_t *bytes);
int fc_arena_free(fc_context *ctx, void *dptr);
int fc_arena_free_all(fc_context *ctx);
int fc_arena_stats(fc_context *ctx, size_t *capacity, size_t *in_use, size_t *peak, size_t *blocks);
/* CommonMemPool::Request(size,id) / Alloc() / GetPtr(ptr,id) / Free(id): shared scratch, the
 * requests under one id are max-reduced and materialised by commit. */
int fc_arena_common_request(fc_context *ctx, size_t bytes, size_t id);
int fc_arena_common_commit(fc_context *ctx);
int fc_arena_common_ptr(fc_context *ctx, size_t id, void **dptr);
int fc_arena_common_free(fc_context *ctx, size_t id);
/* host<->device copies on the context's stream (synchronous on return) and pinned host memory */
int fc_memcpy_h2d(fc_context *ctx, void *dst_device, const void *src_host, size_t bytes);
int fc_memcpy_d2h(fc_context *ctx, void *dst_host, const void *src_device, size_t bytes);
int fc_memset_device(fc_context *ctx, void *dst_device, int value, size_t bytes);
int fc_host_alloc_pinned(size_t bytes, void **hptr);
int fc_host_free_pinned(void *hptr);

/* device-time stopwatch on the context stream: what the reference's Timer (utility/helper.h:66-80,
 * CLOCK_MONOTONIC around each stage) becomes on a GPU.  `slot` is 0..FC_TIMER_SLOTS-1. */
#define FC_TIMER_SLOTS 16
int fc_timer_record(fc_context *ctx, int slot);
int fc_timer_elapsed_ms(fc_context *ctx, int start_slot, int stop_slot, float *ms);

/* ---- shape helpers -------------------------------------------------------- */
/* oh/ow as conv_layer.h:68-69 / ConvTest.cpp:344-347 */
int fc_conv_output_size(const fc_conv_desc *desc, int *oh, int *ow);
/* select_algorithm, ConvTest.cpp:318-331 -- except that 1x1 stride-1 ("direct", an empty case in
 * the reference) resolves to FC_ALGO_IM2COL so that something runs. */
int fc_select_algorithm(const fc_conv_desc *desc, int *algo);
/* What fc_conv_create plans for (desc, algo, mode) on a GPU with sm_count SMs (0 = 148): FC_ALGO_AUTO resolved --
 * select_algorithm as above, then, in the TF32 modes, the direct tensor-core kernel where the measured crossovers
 * favour it -- and the planned-layer meaning of FC_MATH_TF32 / FC_MATH_TF32_UNBOUNDED resolved to the arithmetic that
 * runs (FC_MATH_TF32 or FC_MATH_3XTF32).  Needs no GPU.  The reference
 * has one arithmetic and a shape-only choice (ConvTest.cpp:318-331); this is that choice with the mode added. */
int fc_resolve_plan(const fc_conv_desc *desc, int algo, int mode, int sm_count, int *algo_out, int *mode_out);
/* element counts (floats) of the Winograd-domain buffers for a descriptor */
int fc_wino_buffer_elems(const fc_conv_desc *desc, int mode, size_t *u_elems, size_t *v_elems, size_t *m_elems);

/* ---- Winograd F(6x6,3x3) stages -------------------------------------------
 * Device-pointer entry points, one per stage of winoF63_v1_single / _multi
 * (winoF63ZC/winoF63ZC.h:5-9).  icp = ic rounded up to 8, tp = tiles rounded up to 8, ocp = oc
 * rounded up to 4; padding is zero; position p = col*8 + row of the 8x8 transformed tile.
 * M is [64][oc][tp] in every mode.  The operand layouts follow the arithmetic mode that will
 * multiply them, so `mode` must be the same for the transforms and the GEMM of one layer:
 *   FC_MATH_FP32_MIRRORED  U[64][icp][ocp], V[64][icp][tp]  (row index contiguous: GEMM tiles reach
 *                          shared memory with plain 16-byte async copies, no transposition)
 *   FC_MATH_3XTF32 / TF32  V[64][tp][icp] (K-major, what UMMA and TMA boxes want) and U in contiguous
 *                          boxes of 128 output channels x 32 input channels: with n_ocb = ceil(oc/128),
 *                          n_kb = ceil(ic/32), box (p, ocb, kb) starts at ((p*n_ocb + ocb)*n_kb + kb)*4096
 *                          floats and element (oc, ic) sits at (oc%128)*32 + ic%32 inside it -- one
 *                          box is one TMA load of the GEMM.
 * fc_wino_buffer_elems gives the float counts. */
/* offline_kernel_transform_v1, winoF63ZC/winoF63ZC.h:14 (winoF63ZC.cpp:242-322).  Synchronous: d_U is complete on
 * return.  The forward entry points below read U before they wait for earlier work of the stream, so a caller that
 * fills d_U by other means must have finished doing so before it enqueues a forward. */
int fc_wino_filter_transform(fc_context *ctx, const float *d_kernel, float *d_U, int oc, int ic, int mode);
/* input transform stage, winoF63ZC/winoF63ZC.cpp:512-813 */
int fc_wino_input_transform(fc_context *ctx, const float *d_in, float *d_V, const fc_conv_desc *desc, int mode);
/* TensorGEMM stage, winoF63ZC/winoF63ZC.cpp:818-860 + winoF63ZC/TensorGEMMZC.cpp */
int fc_wino_tensor_gemm(fc_context *ctx, const float *d_U, const float *d_V, float *d_M, const fc_conv_desc *desc,
                        int mode);
/* output transform stage, winoF63ZC/winoF63ZC.cpp:869-973 */
int fc_wino_output_transform(fc_context *ctx, const float *d_M, float *d_out, const fc_conv_desc *desc);
/* whole forward with a pre-transformed filter: winoF63_v1_single(...), winoF63ZC/winoF63ZC.h:5-6.
 * stage_ms (may be NULL) receives InputTran, KernelTran (0: one-time), TensorGEMM, OutputTran
 * device milliseconds -- the four Timer& of the reference signature. */
int fc_wino_forward(fc_context *ctx, const float *d_in, const float *d_U, float *d_V, float *d_M, float *d_out,
                    const fc_conv_desc *desc, int mode, float *stage_ms);

/* No counterpart in the reference (its layers malloc their workspaces in Init,
 * convLayer/winoF63ConvZC.cpp:193-201).  Same computation as fc_wino_forward in
 * FC_MATH_FP32_MIRRORED mode, for callers that may not allocate device memory -- a plugin inside
 * an engine with a fixed memory budget, a loop that must not synchronise the device after start-up,
 * a process whose allocator belongs to another framework.  The V and M workspaces live in a
 * FC_STATIC_SCRATCH_FLOATS-float (16 MiB) array built into the library, which every GPU that loads
 * the library holds until the process exits; the call makes no cudaMalloc / cudaFree and needs no
 * fc_context.  It runs on the CURRENT device, on `stream` (a cudaStream_t, NULL = default stream),
 * asynchronously.  Limits and rules:
 *   - 64*tp*icp + 64*oc*tp floats must fit in the array, else FC_ERR_UNSUPPORTED (e.g. 256->256@56
 *     and 512->512@28 at batch 1 fit, 128->128@112 does not);
 *   - the first call on each device looks up the array's device address: make that call before
 *     starting any stream capture;
 *   - all calls share the one array: two calls that can overlap on the GPU (different streams,
 *     or different host threads) race -- serialise them. */
#define FC_STATIC_SCRATCH_FLOATS (4u << 20)
int fc_wino_forward_static_scratch(const float *d_in, const float *d_U, float *d_out, const fc_conv_desc *desc,
                                   void *stream); /* d_U: fc_wino_filter_transform(..., FC_MATH_FP32_MIRRORED) */

/* ---- im2col / implicit GEMM ------------------------------------------------ */
/* ConvIm2colLayer::im2col(), convLayer/im2colConv.cpp:285-309: materialises the gathered matrix
 * [ic*kh*kw][oh*ow] of image `image` for inspection; the forward path never builds it. */
int fc_im2col_gather(fc_context *ctx, const float *d_in, float *d_gathered, const fc_conv_desc *desc, int image);
/* pack_a_v2, im2col/gemm_pack.cpp:192-238: one-time re-layout of the weight matrix A[oc][K] for the
 * tensor-core kernel -- rows padded to a multiple of 32 floats, stored as two planes hi = tf32(a) and
 * lo = a - hi.  fc_igemm_packed_elems gives the float count of the packed buffer. */
int fc_igemm_packed_elems(int oc, int K, size_t *elems);
int fc_igemm_pack_weights(fc_context *ctx, const float *d_kernel, float *d_packed, int oc, int K);
/* ConvIm2colLayer::im2col_v1() + sgemm(), convLayer/im2colConv.cpp:311-398: gather fused into the
 * GEMM's operand producer.  In FC_MATH_FP32_MIRRORED mode d_kernel is the raw [oc][ic*kh*kw] matrix
 * (A, lda = K); in the tensor-core modes it is the buffer written by fc_igemm_pack_weights. */
int fc_igemm_forward(fc_context *ctx, const float *d_in, const float *d_kernel, float *d_out,
                     const fc_conv_desc *desc, int mode);

/* ---- planned layer ---------------------------------------------------------
 * What ConvLayer's constructor + Init() do (conv_layer.h:27-80,
 * convLayer/winoF63ConvZC.cpp:176-213, convLayer/im2colConv.cpp:224-235):
 * deep-copies the kernel to the device, sizes and allocates workspaces from
 * the context's arena, runs the one-time filter transform. */
int fc_conv_create(fc_context *ctx, const fc_conv_desc *desc, int algo, int mode, const float *h_kernel,
                   fc_conv **out);
int fc_conv_destroy(fc_conv *conv);
int fc_conv_algorithm(const fc_conv *conv, int *algo);
/* The arithmetic the layer runs in: the mode given to fc_conv_create, or what FC_MATH_TF32 / FC_MATH_TF32_UNBOUNDED
 * resolved to for this layer (FC_MATH_TF32 or FC_MATH_3XTF32).  No reference counterpart: the reference computes in
 * fp32 only. */
int fc_conv_math_mode(const fc_conv *conv, int *mode);
/* Epilogue of the layer: every output element becomes relu(y + bias[oc]) before it is stored (both
 * parts optional: h_bias NULL = no bias, relu 0 = no clamp).  The reference carries a bias operand
 * (bias_term / bias_data, conv_layer.h:46-48,72-77) that only its general naive layer adds
 * (convLayer/naiveConv_wudu.h:78, one value per output ELEMENT); its Winograd and im2col layers ignore
 * it and have no activation.  Here the bias is one value per output CHANNEL (`oc` floats, copied),
 * added with one rounded fp32 addition, which is what lets consecutive layers of a network run
 * device to device (fc_layer_list with layer i's output as layer i+1's input) with nothing between
 * them.  Not to be called while a forward of the layer is in flight; a layer list that captured the
 * layer must be rebuilt afterwards. */
int fc_conv_set_epilogue(fc_conv *conv, const float *h_bias, int relu);
/* Forward() on device-resident tensors, asynchronous on the context stream */
int fc_conv_forward_device(fc_conv *conv, const float *d_in, float *d_out);
/* Forward() from / to host memory: H2D copy, kernels, D2H copy, synchronous */
int fc_conv_forward_host(fc_conv *conv, const float *h_in, float *h_out);
/* device buffers owned by the layer (input / output staging used by forward_host) */
int fc_conv_device_buffers(fc_conv *conv, float **d_in, float **d_out);
/* `iters` back-to-back forwards timed with CUDA events on the context stream (the reference's
 * `-i` loop, convLayer/winoF63ConvZC.cpp:227-247); ms_per_iter is the mean. */
int fc_conv_time_device(fc_conv *conv, const float *d_in, float *d_out, int warmup, int iters, float *ms_per_iter);
/* per-stage device milliseconds of the most recent fc_conv_profile call:
 * [0] InputTran / Im2colTran, [1] KernelTran (one-time, measured at create), [2] TensorGEMM / Gemm,
 * [3] OutputTran, [4] Total  (labels of convLayer/winoF63ConvZC.cpp:249-253, im2colConv.cpp:254-256) */
int fc_conv_profile(fc_conv *conv, const float *d_in, float *d_out, int iters, float stage_ms[5]);
/* Per-iteration device milliseconds of the most recent fc_conv_profile call: the "round time:" line the reference
 * prints inside its -i loop (convLayer/winoF63ConvZC.cpp:227-247).  At most `capacity` values are written; *count
 * receives how many iterations were recorded. */
int fc_conv_round_times(const fc_conv *conv, float *ms, int capacity, int *count);
/* Algorithmic work of one forward in the algorithm the layer runs, for throughput and roofline lines:
 *   direct_flops  2*N*K*C/group*R*S*OH*OW (what the reference's benchmark scripts count)
 *   algo_flops    Winograd: 2*64*T*C*K with T the tile count including overhang; otherwise direct_flops
 *   algo_bytes    4*(input + filter as the kernels read it (64*C*K for Winograd, C*K*R*S otherwise) + output)
 *   min_bytes     4*(input + raw filter + output)
 * Any pointer may be NULL. */
int fc_conv_work(const fc_conv *conv, double *direct_flops, double *algo_flops, double *algo_bytes, double *min_bytes);
/* Tuning(): picks the kernel configuration (and, for FC_ALGO_AUTO, the algorithm) from measured
 * device time (convLayer/winoF63ConvZC.cpp:25-174, convLayer/im2colConv.cpp:261-283). */
int fc_conv_tune(fc_conv *conv, int iters, int verbose);
/* The kernel configuration fixed by hand instead of by Tuning(): what the blocking arguments of the reference
 * constructors are to its layers (mc, nc, kc, row_batch, col_batch of ConvIm2colLayer, convLayer/im2colConv.h:16-18;
 * the members ocBlock / tileBlock / icBlock that ConvWinoF63ZCLayer::Tuning assigns, convLayer/winoF63ConvZC.cpp:151-161).
 * Every field 0 = the launcher's heuristic.  bm x bn: block of output channels x tiles or pixels (FFMA kernels: 64 or
 * 128 each for Winograd, also 64x256 and 128x80/96/112; 128x128 ... 8x32 for the table-driven implicit GEMM; tcgen05 kernels: bn = accumulator
 * width, a multiple of 16 up to 256).  variant: 1 / 2 select between the two kernels a path has (Winograd fp32 with
 * at most 32 tiles: 1 = the few-tile kernel, 2 = the blocked one; implicit GEMM: 1 = table-driven FFMA kernel,
 * 2 = the 16x16-thread FFMA kernel in fp32 mode and the tcgen05 kernel in the tensor-core modes).  smem_kb: size of
 * the operand ring of the tcgen05 kernels.  A combination the layer's kernels do not offer is reported by the next
 * forward (FC_ERR_INVALID_ARG / FC_ERR_UNSUPPORTED).  A layer list that captured the layer must be rebuilt. */
int fc_conv_set_kernel_config(fc_conv *conv, int bm, int bn, int variant, int smem_kb);
int fc_conv_get_kernel_config(const fc_conv *conv, int *bm, int *bn, int *variant, int *smem_kb);
/* number of kernel launches one forward issues (for launch accounting) */
int fc_conv_launches_per_forward(const fc_conv *conv, int *launches);

/* ---- layer list -------------------------------------------------------------
 * The reference benchmarks a network as a shell loop over its layers (run_vgg16.sh:5-13,
 * run_resnet50.sh:10-30: one process per layer).  A layer list plays the same list in one
 * process: the forwards of `count` planned layers, each on its own device input/output, captured
 * once into a CUDA graph so that one call replays all of their kernels without per-kernel launch
 * cost.  The layers must belong to `ctx` and outlive the list. */
typedef struct fc_layer_list fc_layer_list;
int fc_layer_list_create(fc_context *ctx, fc_conv *const *convs, const float *const *d_ins, float *const *d_outs,
                         int count, fc_layer_list **out);
int fc_layer_list_forward(fc_layer_list *list);
/* The same list from / to HOST memory (pinned buffers recommended): layer i's input upload, its
 * kernels and its output download run on three streams chained by events, so the PCIe traffic of
 * neighbouring layers overlaps in both directions with the kernels.  h_ins[i] == NULL skips the upload
 * (the layer reads what is already at its device input, e.g. the output of layer i-1 in a chained
 * list), h_outs[i] == NULL skips the download.  Synchronous on return. */
int fc_layer_list_forward_host(fc_layer_list *list, const float *const *h_ins, float *const *h_outs);
int fc_layer_list_launches(const fc_layer_list *list, int *kernel_launches);
int fc_layer_list_destroy(fc_layer_list *list);

/* ---- channel-split layer over several GPUs ----------------------------------
 * No counterpart in the reference, which is a single-process CPU program; its closest relative is
 * the OpenMP split of the output-channel loop (winoF63ZC/winoF63ZC.cpp:1486-1544).  One process per
 * GPU; rank r owns output channels [k0, k1) of a single-image layer (a fc_conv created from that
 * slice of the weights).  The ranks export their full-size output buffers and a small flag array
 * with fc_peer_export, exchange the handles by any means (the Python host uses torch.distributed)
 * and map each other's with fc_peer_open.  fc_conv_forward_scatter then runs the layer with an
 * output transform that stores the slab into EVERY rank's buffer (plain stores over NVLink) and
 * publishes `step` in flag[rank] of every rank; fc_peer_wait enqueues a bounded wait until all
 * ranks have published `step`, after which this rank's buffer holds the whole [oc_total][oh][ow]
 * output.  `step` must grow by one per forward; a caller that lets ranks run ahead of each other
 * alternates between two output buffers.  A wait that gives up reports FC_ERR_TIMEOUT at the next
 * fc_context_synchronize; the gathered output is then undefined.  The limit is fc_context_set_wait_limit_ms
 * (initially $FASTCONV_PEER_WAIT_MS, else 5000 ms: ranks may be seconds apart while one of them still plans or tunes). */
#define FC_MAX_PEERS 8
#define FC_PEER_HANDLE_BYTES 64
/* handle of the context's arena allocation and the offset of `dptr` inside it */
int fc_peer_export(fc_context *ctx, const void *dptr, unsigned char handle[FC_PEER_HANDLE_BYTES], size_t *offset);
/* maps a peer's arena into this process; *base + offset is the peer's `dptr` as this GPU sees it */
int fc_peer_open(fc_context *ctx, const unsigned char handle[FC_PEER_HANDLE_BYTES], void **base);
int fc_peer_close(fc_context *ctx, void *base);
/* outs[r]: rank r's [oc_total][oh][ow] buffer, flags[r]: rank r's int[world] array, both as seen
 * from this GPU (index `rank` is local memory).  k0 = first output channel of this rank's slab. */
int fc_conv_forward_scatter(fc_conv *conv, const float *d_in, float *const *outs, int *const *flags, int world,
                            int rank, int k0, int oc_total, int step);
int fc_peer_wait(fc_context *ctx, const int *d_flags, int world, int step);
int fc_context_set_wait_limit_ms(fc_context *ctx, int ms);

/* ---- several GPUs of one machine ------------------------------------------------
 * No counterpart in the reference either (same nearest relative: the OpenMP split over output channels,
 * winoF63ZC/winoF63ZC.cpp:1486-1544, whose threads share one address space as the GPUs here share NVLink).
 * A communicator owns one context per local rank.  Two ways to run:
 *   fc_comm_init_all   ONE process drives `ndev` GPUs (devices[] or 0..ndev-1); ranks = positions in that list.
 *   fc_comm_init_env   one process per GPU under a launcher: RANK, WORLD_SIZE, LOCAL_RANK (device < 0 = LOCAL_RANK)
 *                      and MASTER_PORT are read from the environment; rank 0 hands the NCCL id to the others through
 *                      a file under /tmp named after the launcher's process id and the port (or $FASTCONV_COMM_ID_FILE).
 * Every entry point acts on the ranks local to the calling process; with several processes all of them must make
 * the same calls in the same order.  NCCL is loaded at run time (libnccl.so.2 or $FASTCONV_NCCL_LIB) and only
 * where it is needed: several processes, or the NCCL gather. */
typedef struct fc_comm fc_comm;
int fc_comm_init_all(int ndev, const int *devices, size_t arena_bytes, fc_comm **out);
int fc_comm_init_env(int device, size_t arena_bytes, fc_comm **out);
/* every sharded layer of the communicator must be destroyed first */
int fc_comm_destroy(fc_comm *comm);
int fc_comm_size(const fc_comm *comm, int *world, int *local_count, int *first_rank);
int fc_comm_context(fc_comm *comm, int local_index, fc_context **ctx);
/* all device work of every rank complete and every rank arrived */
int fc_comm_barrier(fc_comm *comm);
/* values[local_count] in; each replaced by the maximum over all ranks (how a job's time is taken: the slowest rank) */
int fc_comm_allreduce_max(fc_comm *comm, double *values);
/* `bytes` of every rank to every rank through host memory (small records: timings, handles): mine = one record per
 * local rank, all = one per rank of the world, in rank order */
int fc_comm_allgather(fc_comm *comm, const void *mine, void *all, size_t bytes);
/* balanced contiguous split of range(total): the first total % world ranks get one item more */
int fc_shard_range(int total, int world, int rank, int *begin, int *end);

/* A layer sharded over the communicator.
 *   FC_SHARD_BATCH     rank r runs images [b0, b1) of desc->batch; full weights on every rank; NO collective.
 *   FC_SHARD_CHANNELS  single image; rank r owns output channels [k0, k1): its slice of the weights only, the whole
 *                      input, and afterwards every rank holds the whole output.  gather = FC_GATHER_PEER: the Winograd
 *                      output transform stores each result into every rank's buffer over NVLink and its last block
 *                      publishes a step number (one kernel, no collective launch; fc_sharded_conv_wait enqueues the
 *                      bounded wait for the other ranks' slabs).  FC_GATHER_NCCL: one ncclAllGather after the layer.
 * The reduction over input channels is never split: the result is bit-equal to the unsharded layer's.
 * h_kernel is the whole layer's [oc][ic/group][kh][kw].  Host tensors of upload / download / forward_host:
 *   batch split    the images of THIS process's ranks back to back (the whole batch when one process owns all ranks)
 *   channel split  the one input image; the whole [oc][oh][ow] output (delivered by the first local rank)
 * forward / wait are asynchronous on the ranks' streams; two output buffers alternate from forward to forward, so a
 * rank that is one forward ahead never overwrites what a peer still reads.  The peer gather keeps its step number
 * on the device: a captured forward can be replayed. */
enum { FC_SHARD_BATCH = 0, FC_SHARD_CHANNELS = 1 };
enum { FC_GATHER_PEER = 0, FC_GATHER_NCCL = 1 };
typedef struct fc_sharded_conv fc_sharded_conv;
int fc_sharded_conv_create(fc_comm *comm, const fc_conv_desc *desc, int algo, int mode, int shard, int gather,
                           const float *h_kernel, fc_sharded_conv **out);
int fc_sharded_conv_destroy(fc_sharded_conv *sc);
/* the planned layer of one local rank (NULL when the rank owns nothing), its device input / current output and its
 * range of images or channels; any pointer may be NULL */
int fc_sharded_conv_part(fc_sharded_conv *sc, int local_index, fc_conv **conv, float **d_in, float **d_out, int *begin,
                         int *end);
int fc_sharded_conv_upload(fc_sharded_conv *sc, const float *h_in);
int fc_sharded_conv_forward(fc_sharded_conv *sc);
int fc_sharded_conv_wait(fc_sharded_conv *sc);
int fc_sharded_conv_download(fc_sharded_conv *sc, float *h_out);
int fc_sharded_conv_forward_host(fc_sharded_conv *sc, const float *h_in, float *h_out);
/* `iters` forwards (+ waits) timed with CUDA events on every rank's stream after a barrier; the result is the
 * maximum over all ranks of the mean per forward */
int fc_sharded_conv_time_device(fc_sharded_conv *sc, int warmup, int iters, float *ms_per_iter);

/* ---- error metrics on the host ---------------------------------------------- */
/* diff(), utility/helper.cpp:74-89: mean |a-b| over the elements with |a-b| > 1e-5 */
float fc_diff(const float *a, const float *b, int len);

#ifdef __cplusplus
}
#endif
#endif /* FASTCONV_B200_H_ */
