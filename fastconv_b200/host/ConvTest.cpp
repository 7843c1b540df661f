// ConvTest -- single-layer convolution harness with the reference's command line (ConvTest.cpp:73-90):
//
//   winograd_dev -ic C -oc K -is H W -ks KH KW [-a auto|direct|im2col|winograd] [-ts online|offline]
//                [-s SH SW] [-ip P] [-tn tuning|no_tuning] [-t THREADS] [-i ITERS]
//
// It builds ONE layer, fills input and kernel with pseudo-random values, runs the naive host convolution
// as the self-check reference, then Tuning()/Init()/Forward() of the selected layer class on the GPU and
// prints the reference's header, per-stage timing lines and "The difference is".  Differences from the
// reference harness, all deliberate:
//   * `-a auto` on a 1x1 stride-1 layer runs the implicit-GEMM layer (the reference's `direct` case is
//     empty, ConvTest.cpp:369-371, so nothing ran);
//   * `-a direct` runs ConvDirectLayer: the direct tensor-core kernel for layers of stride 1 or 2 with `-m tf32`, the
//     implicit GEMM otherwise;
//   * the self-check honours kernel size, stride and padding (the reference always checks against a
//     3x3 / pad 1 naive layer, ConvTest.cpp:360) and also covers the im2col path;
//   * optional additions: -n/--batch, -m/--math fp32|3xtf32|tf32|tf32-unbounded|tf32-u16, -seed N (the reference seeds from
//     the clock), -nc/--no-check, -dev INDEX, and for several GPUs of one machine driven by this one process
//     -g/--gpus N with -shard batch|k (images or output channels split over the GPUs) and -gather peer|nccl.
//     -t is accepted and only sizes the host self-check;
//   * after the reference's lines: one "Throughput:" line and one machine-readable JSON line per layer.
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <algorithm>

#include "conv_layer.h"
#include "convLayer/directConv.h"
#include "convLayer/im2colConv.h"
#include "convLayer/naiveConv.h"
#include "convLayer/winoF63ConvZC.h"
#include "utility/helper.h"

struct options {
    size_t input_channels;
    size_t output_channels;
    struct nnp_size input_size;
    size_t input_padding;
    struct nnp_size kernel_size;
    struct nnp_size output_subsampling;
    enum nnp_convolution_algorithm algorithm;
    enum nnp_convolution_transform_strategy transform_strategy;
    enum nnp_convolution_tuning_strategy tuning_strategy;
    size_t threads;
    size_t iterations;
    // additions
    size_t batch;
    int math_mode;
    long seed;
    bool check;
    int device;  // CUDA device index of a one-GPU run
    int gpus;    // number of GPUs (ranks) of a sharded run
    int shard;   // FC_SHARD_BATCH or FC_SHARD_CHANNELS
    int gather;  // FC_GATHER_PEER or FC_GATHER_NCCL
};

static void print_options_help(const char *program_name) {
    printf("%s parameters...\n"
           "Required parameters:\n"
           "  -ic  --input-channels     The number of input channels\n"
           "  -oc  --output-channels    The number of output channels\n"
           "  -is  --input-size         Input height and width\n"
           "  -ks  --kernel-size        Kernel height and width\n"
           "Optional parameters:\n"
           "  -a   --algorithm          The algorithm (auto, direct, im2col, or winograd) for computing convolution (default: auto)\n"
           "  -ts  --transform-strategy The transformation strategy (online, or offline) for kernel transformation (default: online)\n"
           "  -s   --output-subsampling The size of a output subsampling region, AKA stride (default: 1x1)\n"
           "  -ip  --input-padding      Implicit input padding (default: 1)\n"
           "  -tn  --tuning             whether to tuning (default: no_tuning)\n"
           "  -t   --threads            The number of threads (default: 1)\n"
           "  -i   --iterations         # iterations (default: 10)\n"
           "GPU additions:\n"
           "  -n   --batch              Images per forward (default: 1)\n"
           "  -m   --math               fp32 (bit-identical accumulation), 3xtf32, tf32 (within 3e-3), tf32-unbounded or tf32-u16 (default: fp32)\n"
           "  -seed                     Seed of the input/kernel generator (default: from the clock)\n"
           "  -nc  --no-check           Skip the naive host convolution and the difference line\n"
           "  -dev --device             CUDA device index of a one-GPU run (default: 0)\n"
           "  -g   --gpus               Number of GPUs the layer is sharded over (default: 1)\n"
           "  -shard                    batch (images split, no collective) or k (output channels split; one image) (default: batch)\n"
           "  -gather                   with -shard k: peer (stores of the output transform over NVLink) or nccl (default: peer)\n",
           program_name);
}

static void fail(const char *fmt, const char *arg) {
    fprintf(stderr, "Error: ");
    fprintf(stderr, fmt, arg);
    fprintf(stderr, "\n");
    exit(EXIT_FAILURE);
}

static size_t parse_positive(const char *text, const char *what, bool allow_zero = false) {
    size_t v = 0;
    if (sscanf(text, "%zu", &v) != 1) fail("can not parse %s as an unsigned integer", text);
    if (v == 0 && !allow_zero) {
        fprintf(stderr, "Error: invalid value %s for %s: positive value expected\n", text, what);
        exit(EXIT_FAILURE);
    }
    return v;
}

static bool is_flag(const char *arg, const char *long_name, const char *short_name) {
    return strcmp(arg, long_name) == 0 || strcmp(arg, short_name) == 0;
}

static struct options parse_options(int argc, char **argv) {
    struct options o;
    memset(&o, 0, sizeof o);
    o.input_padding = 1;
    o.output_subsampling.width = o.output_subsampling.height = 1;
    o.algorithm = nnp_convolution_algorithm_auto;
    o.transform_strategy = nnp_convolution_transform_strategy_online;
    o.tuning_strategy = nnp_convolution_tuning_strategy_no_tuning;
    o.threads = 1;
    o.iterations = 10;
    o.batch = 1;
    o.math_mode = FC_MATH_FP32_MIRRORED;
    o.seed = -1;
    o.check = true;
    o.device = 0;
    o.gpus = 1;
    o.shard = FC_SHARD_BATCH;
    o.gather = FC_GATHER_PEER;

    for (int i = 1; i < argc; ++i) {
        const char *a = argv[i];
        const int left = argc - i - 1;  // arguments after the flag
        if (is_flag(a, "--help", "-h")) {
            print_options_help(argv[0]);
            exit(EXIT_SUCCESS);
        } else if (is_flag(a, "--no-check", "-nc")) {
            o.check = false;
        } else if (is_flag(a, "--input-size", "-is") || is_flag(a, "--kernel-size", "-ks") ||
                   is_flag(a, "--output-subsampling", "-s")) {
            if (left < 2) fail("expected two values after %s", a);
            struct nnp_size sz;
            sz.height = parse_positive(argv[i + 1], "the height");
            sz.width = parse_positive(argv[i + 2], "the width");
            if (a[1] == 'i' || strcmp(a, "--input-size") == 0) o.input_size = sz;
            else if (a[1] == 'k' || strcmp(a, "--kernel-size") == 0) o.kernel_size = sz;
            else o.output_subsampling = sz;
            i += 2;
        } else {
            if (left < 1) fail("expected a value after %s", a);
            const char *v = argv[++i];
            if (is_flag(a, "--input-channels", "-ic")) o.input_channels = parse_positive(v, "the number of input channels");
            else if (is_flag(a, "--output-channels", "-oc")) o.output_channels = parse_positive(v, "the number of output channels");
            else if (is_flag(a, "--input-padding", "-ip")) o.input_padding = parse_positive(v, "the padding", true);
            else if (is_flag(a, "--threads", "-t")) o.threads = parse_positive(v, "the number of threads");
            else if (is_flag(a, "--iterations", "-i")) o.iterations = parse_positive(v, "the number of iterations");
            else if (is_flag(a, "--batch", "-n")) o.batch = parse_positive(v, "the batch size");
            else if (is_flag(a, "--device", "-dev")) o.device = (int)parse_positive(v, "the GPU index", true);
            else if (is_flag(a, "--gpus", "-g")) o.gpus = (int)parse_positive(v, "the number of GPUs");
            else if (is_flag(a, "--shard", "-shard")) {
                if (strcmp(v, "batch") == 0) o.shard = FC_SHARD_BATCH;
                else if (strcmp(v, "k") == 0) o.shard = FC_SHARD_CHANNELS;
                else fail("invalid partitioning %s", v);
            } else if (is_flag(a, "--gather", "-gather")) {
                if (strcmp(v, "peer") == 0) o.gather = FC_GATHER_PEER;
                else if (strcmp(v, "nccl") == 0) o.gather = FC_GATHER_NCCL;
                else fail("invalid gather %s", v);
            }
            else if (strcmp(a, "-seed") == 0 || strcmp(a, "--seed") == 0) o.seed = (long)parse_positive(v, "the seed", true);
            else if (is_flag(a, "--algorithm", "-a")) {
                if (strcmp(v, "auto") == 0) o.algorithm = nnp_convolution_algorithm_auto;
                else if (strcmp(v, "direct") == 0) o.algorithm = nnp_convolution_algorithm_direct;
                else if (strcmp(v, "im2col") == 0) o.algorithm = nnp_convolution_algorithm_im2col;
                else if (strcmp(v, "winograd") == 0) o.algorithm = nnp_convolution_algorithm_winograd;
                else fail("invalid convolution algorithm name %s", v);
            } else if (is_flag(a, "--transform-strategy", "-ts")) {
                if (strcmp(v, "online") == 0) o.transform_strategy = nnp_convolution_transform_strategy_online;
                else if (strcmp(v, "offline") == 0) o.transform_strategy = nnp_convolution_transform_strategy_offline;
                else fail("invalid trasnformation strategy name %s", v);
            } else if (is_flag(a, "--tuning", "-tn")) {
                if (strcmp(v, "no_tuning") == 0) o.tuning_strategy = nnp_convolution_tuning_strategy_no_tuning;
                else if (strcmp(v, "tuning") == 0) o.tuning_strategy = nnp_convolution_tuning_strategy_grid_search;
                else fail("invalid tuning name %s", v);
            } else if (is_flag(a, "--math", "-m")) {
                if (strcmp(v, "fp32") == 0) o.math_mode = FC_MATH_FP32_MIRRORED;
                else if (strcmp(v, "3xtf32") == 0) o.math_mode = FC_MATH_3XTF32;
                else if (strcmp(v, "tf32") == 0) o.math_mode = FC_MATH_TF32;
                else if (strcmp(v, "tf32-unbounded") == 0) o.math_mode = FC_MATH_TF32_UNBOUNDED;
                else if (strcmp(v, "tf32-u16") == 0) o.math_mode = FC_MATH_TF32_U16;
                else fail("invalid math mode %s", v);
            } else {
                fprintf(stderr, "Error: unknown argument '%s'\n", a);
                print_options_help(argv[0]);
                exit(EXIT_FAILURE);
            }
        }
    }
    const char *missing = NULL;
    if (o.input_channels == 0) missing = "the number of input channels is not specified";
    else if (o.output_channels == 0) missing = "the number of output channels is not specified";
    else if (o.input_size.width == 0) missing = "the input size is not specified";
    else if (o.kernel_size.width == 0) missing = "the kernel size is not specified";
    if (missing) {
        fprintf(stderr, "Error: %s\n", missing);
        print_options_help(argv[0]);
        exit(EXIT_FAILURE);
    }
    return o;
}

// input in [0,256), kernel in [0,1): the value ranges of the reference generators (ConvTest.cpp:18-46)
static void fillTestInput(float *target, size_t count) {
    for (size_t i = 0; i < count; ++i) target[i] = (float)(256 * (rand() / (double)RAND_MAX));
}
static void fillTestKernel(float *target, size_t count) {
    for (size_t i = 0; i < count; ++i) target[i] = (float)(1.0 * rand() / (double)RAND_MAX);
}

// select_algorithm of ConvTest.cpp:318-331 (with 1x1 stride 1 resolved to the implicit GEMM); with -m tf32 or
// tf32-unbounded the library may answer "direct" for layers where its tensor-core kernel is the faster or the only
// accurate-enough TF32 path.
static enum nnp_convolution_algorithm select_algorithm(const fc_conv_desc &d, int math_mode) {
    int a = FC_ALGO_IM2COL, m = math_mode;
    if (fc_resolve_plan(&d, FC_ALGO_AUTO, math_mode, 0, &a, &m) != FC_OK) fc_select_algorithm(&d, &a);
    return (enum nnp_convolution_algorithm)a;
}

static const char *algorithm_name(int a) {
    return a == FC_ALGO_WINOGRAD ? "winograd" : a == FC_ALGO_DIRECT ? "direct" : "im2col";
}
static const char *math_name(int m) {
    return m == FC_MATH_3XTF32 ? "3xtf32" : m == FC_MATH_TF32 ? "tf32" : m == FC_MATH_TF32_U16 ? "tf32-u16" : "fp32";
}

// One JSON line per layer: what ran, how long it took, and how far that is from the layer's roofline -- the slower of
// its algorithmic flops at the arithmetic peak of the mode and its algorithmic bytes at the HBM bandwidth.  Peaks: FP32
// = SMs x 128 lanes x 2 x the maximum SM clock; TF32 = $FASTCONV_TF32_TFLOPS, else 759.9 (a library GEMM of 8192^3 on a
// B200), a third of it for 3xTF32; HBM = $FASTCONV_HBM_GBS, else 6538.3 (a device-to-device copy on a B200).
static void print_json_line(fc_context *ctx, fc_conv *conv, const fc_conv_desc &d, double ms, int gpus, const char *shard) {
    double direct = 0, flops = 0, bytes = 0, min_bytes = 0;
    int algo = 0, mode = 0, sms = 148, mhz = 1965;
    fc_conv_work(conv, &direct, &flops, &bytes, &min_bytes);
    fc_conv_algorithm(conv, &algo);
    fc_conv_math_mode(conv, &mode);
    fc_context_info(ctx, &sms, &mhz);
    const char *e_tf32 = getenv("FASTCONV_TF32_TFLOPS"), *e_hbm = getenv("FASTCONV_HBM_GBS");
    const double tf32 = e_tf32 ? atof(e_tf32) : 759.9, hbm = e_hbm ? atof(e_hbm) : 6538.3;
    const double fp32 = sms * 128.0 * 2.0 * mhz * 1e-6;
    const double peak = mode == FC_MATH_FP32_MIRRORED ? fp32 : mode == FC_MATH_3XTF32 ? tf32 / 3.0 : tf32;
    // a sharded layer: `conv` is one rank's share, and every rank has its own peaks
    const double t_flop = flops / (peak * 1e12) * 1e3, t_hbm = bytes / (hbm * 1e9) * 1e3;
    const double roof = t_flop > t_hbm ? t_flop : t_hbm;
    const double whole = 2.0 * d.batch * d.oc * (double)(d.ic / d.group) * d.kh * d.kw *
                         (double)((d.ih + d.pad_top + d.pad_bottom - d.kh) / d.sh + 1) *
                         (double)((d.iw + d.pad_left + d.pad_right - d.kw) / d.sw + 1);
    printf("{\"layer\": \"%d->%d@%dx%d %dx%ds%d\", \"batch\": %d, \"gpus\": %d, \"shard\": \"%s\", \"algo\": \"%s\", "
           "\"math\": \"%s\", \"ms\": %.6f, \"gflops_direct_equiv\": %.1f, \"roofline_ms\": %.6f, "
           "\"frac_of_roofline\": %.4f, \"bound\": \"%s\", \"peak_tflops\": %.1f, \"hbm_gbs\": %.1f}\n",
           d.ic, d.oc, d.ih, d.iw, d.kh, d.kw, d.sh, d.batch, gpus, shard, algorithm_name(algo), math_name(mode), ms,
           whole / (ms * 1e-3) / 1e9, roof, roof / ms, t_flop > t_hbm ? "math" : "hbm", peak, hbm);
}

void ConvLayer::print_json(const fc_conv_desc &d) {
    if (conv) print_json_line(ctx, conv, d, stage_ms[4], 1, "none");
}

// -g N: the layer sharded over N GPUs that this process drives (fc_comm_init_all, fc_sharded_conv_*).
static int run_sharded(const struct options &options, const fc_conv_desc &d, int oh, int ow, float *test_input,
                       float *test_kernel, float *ref) {
    fc_comm *comm = NULL;
    const size_t act = ((size_t)d.batch * d.ic * d.ih * d.iw + (size_t)d.batch * d.oc * oh * ow) * sizeof(float);
    const size_t wts = (size_t)d.ic * d.oc * d.kh * d.kw * sizeof(float);
    const size_t tiles = (size_t)d.batch * ((oh + 5) / 6) * ((ow + 5) / 6) + 8;
    const size_t wino = 64 * sizeof(float) * ((size_t)(d.oc + 8) * (d.ic + 8) + tiles * (d.ic + 8) + tiles * (d.oc + 8));
    if (fc_comm_init_all(options.gpus, NULL, 2 * (act + 8 * wts + wino) + (256u << 20), &comm) != FC_OK) {
        fprintf(stderr, "Error: %s\n", fc_last_error());
        return EXIT_FAILURE;
    }
    fc_sharded_conv *sc = NULL;
    const int algo = options.algorithm == nnp_convolution_algorithm_auto ? FC_ALGO_AUTO : (int)options.algorithm;
    if (fc_sharded_conv_create(comm, &d, algo, options.math_mode, options.shard, options.gather, test_kernel, &sc) != FC_OK) {
        fprintf(stderr, "Error: %s\n", fc_last_error());
        fc_comm_destroy(comm);
        return EXIT_FAILURE;
    }
    fc_conv *part = NULL;
    fc_sharded_conv_part(sc, 0, &part, NULL, NULL, NULL, NULL);
    int ran = FC_ALGO_IM2COL;
    if (part) fc_conv_algorithm(part, &ran);
    printf("Algorithm: %s\n", ran == FC_ALGO_WINOGRAD ? "winograd F63" : algorithm_name(ran));
    printf("Sharding: %s over %d GPUs%s\n", options.shard == FC_SHARD_BATCH ? "images" : "output channels", options.gpus,
           options.shard == FC_SHARD_BATCH ? ", no collective"
                                           : options.gather == FC_GATHER_PEER ? ", gathered by the output transform's stores"
                                                                              : ", NCCL all-gather");
    const size_t out_elems = (size_t)d.batch * d.oc * oh * ow;
    float *out = (float *)malloc(out_elems * sizeof(float));
    float ms = 0.f;
    if (fc_sharded_conv_forward_host(sc, test_input, out) != FC_OK ||
        fc_sharded_conv_time_device(sc, 2, options.iterations > 0 ? (int)options.iterations : 1, &ms) != FC_OK) {
        fprintf(stderr, "Error: %s\n", fc_last_error());
        return EXIT_FAILURE;
    }
    printf("Total time: %lfms\n", (double)ms);
    if (ref != NULL) diff(ref, out, (int)out_elems);
    const double flops = 2.0 * d.batch * d.oc * d.ic * d.kh * d.kw * oh * ow;
    printf("Throughput: %.1f GFLOP/s (direct-equivalent, %.6f ms per forward)\n", flops / (ms * 1e-3) / 1e9, ms);
    fc_context *ctx0 = NULL;
    fc_comm_context(comm, 0, &ctx0);
    if (part) print_json_line(ctx0, part, d, ms, options.gpus, options.shard == FC_SHARD_BATCH ? "batch" : "k");
    free(out);
    fc_sharded_conv_destroy(sc);
    fc_comm_destroy(comm);
    return 0;
}

int main(int argc, char *argv[]) {
    struct options options = parse_options(argc, argv);
    srand(options.seed >= 0 ? (unsigned)options.seed : (unsigned)time(NULL));

    const size_t ic = options.input_channels, oc = options.output_channels, pad = options.input_padding;
    const struct nnp_size in = options.input_size, ks = options.kernel_size, st = options.output_subsampling;
    fc_conv_desc d = {(int)options.batch, (int)ic, (int)in.height, (int)in.width, (int)oc, (int)ks.height, (int)ks.width,
                      (int)st.height, (int)st.width, (int)pad, (int)pad, (int)pad, (int)pad, 1};
    int oh = 0, ow = 0;
    if (fc_conv_output_size(&d, &oh, &ow) != FC_OK) {
        fprintf(stderr, "Error: %s\n", fc_last_error());
        return EXIT_FAILURE;
    }

    printf("Input channels: %zu\n", ic);
    printf("Output channels: %zu\n", oc);
    printf("Input: %zux%zu with implicit padding %zu\n", in.height, in.width, pad);
    printf("Kernel: %zux%zu\n", ks.height, ks.width);
    printf("Subsampling: %zux%zu\n", st.height, st.width);

    const size_t in_elems = options.batch * ic * in.height * in.width, k_elems = oc * ic * ks.height * ks.width;
    float *test_input = (float *)malloc(sizeof(float) * in_elems);
    float *test_kernel = (float *)malloc(sizeof(float) * (k_elems + 16));
    fillTestInput(test_input, in_elems);
    fillTestKernel(test_kernel, k_elems);

    if (options.algorithm == nnp_convolution_algorithm_auto) options.algorithm = select_algorithm(d, options.math_mode);

    if (fastconv_default_context() == NULL && options.device != 0 && options.gpus == 1) {
        fc_context *ctx = NULL;
        if (fc_context_create(options.device, (size_t)8 << 30, &ctx) != FC_OK) {
            fprintf(stderr, "Error: %s\n", fc_last_error());
            return EXIT_FAILURE;
        }
        fastconv_default_context() = ctx;
    }

    ConvNaiveLayer *conv_reference = NULL;
    if (options.check) {
        conv_reference = new ConvNaiveLayer(test_input, test_kernel, NULL, NULL, ic, in.height, in.width, oc, ks.height,
                                            ks.width, st.height, st.width, pad, pad, pad, pad);
        conv_reference->set_batch(options.batch);
        conv_reference->Forward();
    }
    float *ref = conv_reference ? conv_reference->output_data : NULL;

    if (options.gpus > 1) {
        const int rc = run_sharded(options, d, oh, ow, test_input, test_kernel, ref);
        delete conv_reference;
        free(test_input);
        free(test_kernel);
        return rc;
    }

    ConvLayer *conv = NULL;
    if (options.algorithm == nnp_convolution_algorithm_winograd)
        conv = new ConvWinoF63ZCLayer(test_input, test_kernel, NULL, ref, ic, in.height, in.width, oc, ks.height, ks.width,
                                      st.height, st.width, pad, pad, pad, pad, 1, false, options.threads,
                                      options.iterations);
    else if (options.algorithm == nnp_convolution_algorithm_direct)
        conv = new ConvDirectLayer(test_input, test_kernel, NULL, ref, ic, in.height, in.width, oc, ks.height, ks.width,
                                   st.height, st.width, pad, pad, pad, pad, 1, false, options.threads,
                                   options.iterations);
    else
        conv = new ConvIm2colLayer(test_input, test_kernel, NULL, ref, ic, in.height, in.width, oc, ks.height, ks.width,
                                   st.height, st.width, pad, pad, pad, pad, 1, false, options.threads,
                                   options.iterations);
    conv->set_batch(options.batch);
    conv->set_math_mode(options.math_mode);
    if (options.tuning_strategy != nnp_convolution_tuning_strategy_no_tuning) conv->Tuning();
    conv->Init();
    conv->Forward();

    const float *ms = conv->stage_milliseconds();
    const double flops = 2.0 * options.batch * oc * ic * ks.height * ks.width * oh * ow;
    printf("Throughput: %.1f GFLOP/s (direct-equivalent, %.6f ms per forward)\n", flops / (ms[4] * 1e-3) / 1e9, ms[4]);
    conv->print_json(d);

    delete conv;
    delete conv_reference;
    free(test_input);
    free(test_kernel);
    fc_context_destroy(fastconv_default_context());
    fastconv_default_context() = NULL;
    return 0;
}
