// Direct convolution on the 5th-generation tensor cores for layers of stride 1 or 2 (`-a direct`; the reference parses
// the name but its case is empty, ConvTest.cpp:369-371).
//
//   out[n][oc][y][x] = sum_{u,v} sum_c  W[oc][c][u][v] * in[n][c][sh*y + u - pad_t][sw*x + v - pad_l]
//
// is kh*kw GEMMs that accumulate into ONE accumulator: for every (u,v) the second operand is the input shifted
// by (u,v).  With the input in NHWC (channels innermost, padded to a multiple of 32) a shifted patch of
// bh x bw pixels x 32 channels is one 4-D TMA box whose innermost coordinate is the channel block -- always 16-byte
// aligned, whatever the shift -- and whose rows (one pixel = 128 bytes) land in shared memory exactly as a K-major,
// 128-byte-swizzled UMMA operand of 128 rows.  Pixels outside the image are the box's out-of-range elements and read as
// zero: the padding costs nothing and no im2col index is ever computed.  A stride of 2 is the tensor map's element
// stride along x and y (the box spans twice the pixels, the copy takes every second one).  The weights, re-laid
// out once as Wp[u*kw+v][oc][c], are the other K-major operand.
//
//   nchw_to_nhwc_kernel     one pass over the input per forward (the layer keeps the reference's NCHW at its boundary)
//   direct_tc_kernel        persistent; a work item = one patch of 128 output pixels x a block of <= 256 channels
//     warp 0      TMA producer: per k-block (u,v, 32 channels) one 4-D box of the input and one 3-D box of Wp
//     warp 1      tcgen05.mma kind::tf32, M = 128 pixels, N = channel block, two TMEM accumulators
//     warps 2..5  epilogue: tcgen05.ld (lane = pixel), bias/ReLU, NCHW stores (a warp writes runs of bw pixels)
//   fold_taps_kernel        replaces the layout pass when ic*kh*kw <= 32: the taps become channels of a 1x1 layer
//   bias_relu_kernel        epilogue of a small layer whose reduction was shared by several work items (make_plan)
//
// There is no Winograd transform in the way, so single-pass TF32 keeps its plain accuracy (rel-L2 3e-4..8e-4 against
// 6.4e-3 through F(6x6,3x3)).  Every mbarrier wait is bounded as in the other tensor-core kernels.
#include "fc_tc_common.cuh"

namespace fc {

namespace {

using namespace tc;

struct DirectParams {
    float *out;
    int *status;
    Epilogue ep;
    int oc, oh, ow;
    int bh, bw, n_px, n_py;  // patch shape (bh * bw = 128) and patches per image along x and y
    int bn, n_oc_items;      // channel block (multiple of 16, <= 128) and blocks per layer
    int num_kb, taps, kw;    // 32-channel blocks per tap, kh*kw, kw
    int pad_t, pad_l, sh, sw;
    int stages, acc_cols, n_items;
    int b_bytes;
    int ksplit, kb_per_split;  // the taps*num_kb k-blocks of an output block are shared by ksplit work items
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// channel block fastest: CTAs next to each other read the same input patch
__device__ __forceinline__ void item_coords(const DirectParams &P, int item, int &img, int &y0, int &x0, int &oc0,
                                            int &k_lo, int &k_hi) {
    const int part = item % P.ksplit;  // which share of the reduction
    item /= P.ksplit;
    k_lo = part * P.kb_per_split;
    k_hi = min(P.taps * P.num_kb, k_lo + P.kb_per_split);
    oc0 = (item % P.n_oc_items) * P.bn;
    int patch = item / P.n_oc_items;
    x0 = (patch % P.n_px) * P.bw;
    patch /= P.n_px;
    y0 = (patch % P.n_py) * P.bh;
    img = patch / P.n_py;
}

__global__ void __launch_bounds__(TC_THREADS) direct_tc_kernel(const __grid_constant__ CUtensorMap tmX,
                                                              const __grid_constant__ CUtensorMap tmW,
                                                              const DirectParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[8] empty[8] acc_full[2] acc_empty[2]
    const int S = P.stages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 20);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t ring = (smem_u32(smem_raw) + 512 + 1023) & ~1023u;
    const uint32_t stage_bytes = A_BYTES + (uint32_t)P.b_bytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto bar_full = [&](int s) { return smem_u32(bars + s); };
    auto bar_empty = [&](int s) { return smem_u32(bars + 8 + s); };
    auto bar_acc_full = [&](int a) { return smem_u32(bars + 16 + a); };
    auto bar_acc_empty = [&](int a) { return smem_u32(bars + 18 + a); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)(2 * P.acc_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            pdl_wait();  // the NHWC copy of the input is written by the kernel launched just before
            int g = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x) {
                int img, y0, x0, oc0, k_lo, k_hi;
                item_coords(P, item, img, y0, x0, oc0, k_lo, k_hi);
                for (int k = k_lo; k < k_hi; ++k, ++g) {
                    const int tap = k / P.num_kb, kb = k - tap * P.num_kb;
                    const int u = tap / P.kw, v = tap - u * P.kw;
                    const int s = g % S;
                    const uint32_t ph = (uint32_t)(g / S) & 1u;
                    ok = mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, P.status);
                    if (!ok) break;
                    const uint32_t dst = ring + s * stage_bytes;
                    mbar_expect_tx(bar_full(s), stage_bytes);
                    // innermost coordinate = channel block (a multiple of 32 floats); x and y may be negative or
                    // past the image: those pixels read as zero
                    tma_load_4d(dst, &tmX, bar_full(s), kb * BK, x0 * P.sw + v - P.pad_l, y0 * P.sh + u - P.pad_t, img);
                    tma_load_3d(dst + A_BYTES, &tmW, bar_full(s), kb * BK, oc0, tap);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_tf32(BM, P.bn);
            int g = 0, it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
                ok = mbar_wait(bar_acc_empty(acc), acc_ph ^ 1u, abort_flag, P.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * P.acc_cols);
                int img, y0, x0, oc0, k_lo, k_hi;
                item_coords(P, item, img, y0, x0, oc0, k_lo, k_hi);
                const int kb_per_item = k_hi - k_lo;
                for (int kb = 0; kb < kb_per_item; ++kb, ++g) {
                    const int s = g % S;
                    const uint32_t ph = (uint32_t)(g / S) & 1u;
                    ok = mbar_wait(bar_full(s), ph, abort_flag, P.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a = ring + s * stage_bytes, b = a + A_BYTES;
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ++ks) {
                        const uint32_t koff = ks * 32;  // 8 tf32 = 32 bytes further along K inside the swizzle span
                        tc_mma_tf32(d_tmem, umma_desc_k_sw128(a + koff), umma_desc_k_sw128(b + koff), idesc,
                                    (kb == 0 && ks == 0) ? 0u : 1u);
                    }
                    tc_commit(bar_empty(s));
                }
                if (ok) tc_commit(bar_acc_full(acc));
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 ----------------
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        const int r = q * 32 + lane, py = r / P.bw, px = r - py * P.bw;
        int it = 0;
        bool ok = true, waited = false;
        for (int item = blockIdx.x; item < P.n_items && ok; item += gridDim.x, ++it) {
            int img, y0, x0, oc0, k_lo, k_hi;
            item_coords(P, item, img, y0, x0, oc0, k_lo, k_hi);
            if (!waited) {  // the output may still be read by whatever consumed the forward before this one
                pdl_wait();
                waited = true;
            }
            const int acc = it & 1;
            const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
            ok = mbar_wait(bar_acc_full(acc), acc_ph, abort_flag, P.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * P.acc_cols);
            const int y = y0 + py, x = x0 + px;
            const bool inside = y < P.oh && x < P.ow;
            const size_t plane = (size_t)P.oh * P.ow;
            float *dst = P.out + ((size_t)img * P.oc + oc0) * plane + (size_t)y * P.ow + x;
            for (int c0 = 0; c0 < P.bn; c0 += 16) {
                float va[16];
                tc_ld16(t_addr + (uint32_t)c0, va);
                if (c0 + 16 >= P.bn) {  // last columns read: the MMA warp may overwrite this accumulator
                    tc_fence_before();
                    mbar_arrive(bar_acc_empty(acc));
                }
                if (inside && P.ksplit == 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (oc0 + c0 + j < P.oc) dst[(size_t)(c0 + j) * plane] = P.ep(va[j], oc0 + c0 + j);
                } else if (inside) {  // a share of the reduction: added into the zeroed output (no epilogue then)
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (oc0 + c0 + j < P.oc) atomicAdd(dst + (size_t)(c0 + j) * plane, va[j]);
                }
            }
        }
    }

    if (*abort_flag) {
        // give copies that are still in flight time to land before the CTA's shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)(2 * P.acc_cols))
                     : "memory");
    }
}

// in[n][C][HW] -> out[n][HW][Cp], channels C..Cp-1 written as zeros.  32 x 32 tiles through shared memory: reads run
// along HW, writes along the channels, both as whole 128-byte lines.
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const float *__restrict__ in, float *__restrict__ out, int C,
                                                          int Cp, int HW) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const size_t img = blockIdx.z;
    pdl_trigger();
    pdl_wait();  // the input may be the previous layer's output; the NHWC buffer may still be read by an earlier forward
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i, p = p0 + tx;
        tile[ty + 8 * i][tx] = (c < C && p < HW) ? __ldg(in + (img * C + c) * HW + p) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = p0 + ty + 8 * i;
        if (p < HW) out[(img * HW + p) * Cp + c0 + tx] = tile[tx][ty + 8 * i];
    }
}

// out[n][oc][plane] <- relu(out + bias[oc]): the epilogue of a layer whose reduction was shared by several work items
__global__ void __launch_bounds__(256) bias_relu_kernel(float *__restrict__ out, Epilogue ep, int oc, int plane,
                                                       size_t total) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = ep(out[i], (int)((i / plane) % oc));
}

// W[oc][ic][kh][kw] -> Wp[tap = u*kw + v][oc][icp], channels ic..icp-1 zero
__global__ void direct_pack_weights_kernel(const float *__restrict__ w, float *__restrict__ wp, int oc, int ic, int icp,
                                           int taps) {
    const size_t total = (size_t)taps * oc * icp;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(idx % icp);
        const size_t rest = idx / icp;
        const int o = (int)(rest % oc), tap = (int)(rest / oc);
        wp[idx] = c < ic ? __ldg(w + ((size_t)o * ic + c) * taps + tap) : 0.0f;
    }
}

// A layer whose whole reduction fits one k-block (ic*kh*kw <= 32: the 3-channel first layer of a network) would
// spend kh*kw k-blocks of 32 channels on 3 real ones.  For it the layout pass writes the taps next to each other
// instead -- F[n][y][x][k], k = (c*kh + u)*kw + v as in a row of W, zero for pixels outside the image and for
// k >= ic*kh*kw -- and the convolution becomes a 1x1 layer over 32 channels: one k-block per patch instead of kh*kw.
__global__ void __launch_bounds__(256) fold_taps_kernel(const float *__restrict__ in, float *__restrict__ out, int ic,
                                                       int ih, int iw, int kh, int kw, int pad_t, int pad_l, int oh,
                                                       int ow) {
    // one block per output row: the ic*kh input rows it needs (at most 32 of them), padded left and right with zeros,
    // are staged in shared memory with coalesced reads; a warp then writes the 32 floats of one pixel per step
    extern __shared__ float rows[];  // [ic*kh][ow + kw - 1]
    const int y = blockIdx.x % oh, img = blockIdx.x / oh;
    const int wrow = ow + kw - 1, nrows = ic * kh;
    pdl_trigger();
    pdl_wait();
    for (int idx = threadIdx.x; idx < nrows * wrow; idx += 256) {
        const int r = idx / wrow, xs = idx - r * wrow;
        const int c = r / kh, u = r - c * kh;
        const int yy = y + u - pad_t, xx = xs - pad_l;
        rows[idx] = (yy >= 0 && yy < ih && xx >= 0 && xx < iw) ? __ldg(in + (((size_t)img * ic + c) * ih + yy) * iw + xx) : 0.0f;
    }
    __syncthreads();
    const int k = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int r = k / kw, v = k - r * kw;  // r = c*kh + u
    const bool real = r < nrows;
    const float *src = rows + (real ? r * wrow + v : 0);
    float *dst = out + ((size_t)blockIdx.x * ow) * 32 + k;
    for (int x = w; x < ow; x += 8) dst[(size_t)x * 32] = real ? src[x] : 0.0f;
}

// NHWC input as a 4-D tensor (channel, x, y, image), box = 32 channels x bw x bh x 1, 128-byte swizzle, zero fill.
// A strided layer reads every sw-th column and sh-th row: the box spans bw*sw x bh*sh elements and the map's element
// strides make the copy take one in sw (sh) of them, so the landed tile is the same 128 pixels x 32 channels.
int make_map_nhwc(CUtensorMap *map, const float *base, int icp, int iw, int ih, int n, int bw, int bh, int sw, int sh) {
    EncodeTiledFn enc;
    FC_PROPAGATE(get_encoder(&enc));
    cuuint64_t dims[4] = {(cuuint64_t)icp, (cuuint64_t)iw, (cuuint64_t)ih, (cuuint64_t)n};
    cuuint64_t strides[3] = {(cuuint64_t)icp * 4, (cuuint64_t)icp * iw * 4, (cuuint64_t)icp * iw * ih * 4};
    cuuint32_t box[4] = {BK, (cuuint32_t)(bw * sw), (cuuint32_t)(bh * sh), 1};
    cuuint32_t estr[4] = {1, (cuuint32_t)sw, (cuuint32_t)sh, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FC_REQUIRE(r == CUDA_SUCCESS, FC_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (icp %d iw %d ih %d n %d box %dx%d)",
               (int)r, icp, iw, ih, n, bw, bh);
    return FC_OK;
}

}  // namespace

static bool folds_taps(const fc_conv_desc &d) {  // ... and the staged rows of one output row fit shared memory
    const long long row_floats = (long long)d.ic * d.kh * (d.iw + d.pad_left + d.pad_right);
    return d.sh == 1 && d.sw == 1 && d.kh * d.kw > 1 && d.ic * d.kh * d.kw <= BK && row_floats * 4 <= 160 * 1024 &&
           (long long)d.batch * (d.ih + d.pad_top + d.pad_bottom) < (1ll << 31);
}

bool direct_tc_eligible(const fc_conv_desc &d) {
    return d.sh >= 1 && d.sh <= 2 && d.sw >= 1 && d.sw <= 2 && d.group == 1 && d.iw <= (1 << 20) && d.ih <= (1 << 20);
}

// patch of 128 output pixels: the shape that wastes the fewest pixels, the widest one among equals (longer runs in
// the output rows)
static void direct_patch_shape(int oh, int ow, int *bh, int *bw) {
    const int shapes[6][2] = {{1, 128}, {2, 64}, {4, 32}, {8, 16}, {16, 8}, {32, 4}};
    size_t best = ~(size_t)0;
    for (const auto &s : shapes) {
        const size_t covered = (size_t)round_up(oh, s[0]) * round_up(ow, s[1]);
        if (covered < best) { best = covered; *bh = s[0]; *bw = s[1]; }
    }
}

// Whether `-a auto` should take this kernel instead of its rival.  From per-layer timings of the VGG-16 and ResNet-50
// layers at batch 1, 2, 8 and 64 on a B200:
//  * against Winograd in TF32 (3x3 stride 1) the kernel does 2.25x the multiplications but moves no V and M, so it
//    wins where the channels are few -- ic*oc/(ic+oc) up to about 100 (128 -> 256 yes, 256 -> 256 a tie) -- provided the
//    layer has a work item for every SM, or so few channels (up to about 48) that the transforms dominate anyway.
//    Small layers (at most 8 patches and no more 64-channel output blocks than SMs: 28x28 maps and below of one
//    image; with 16 patches -- 14x14 at batch 8 -- Winograd is 1.6x faster again) share their reduction among the SMs and then run within 0.8x to 1.15x of Winograd; they take this kernel
//    too, because single-pass TF32 through F(6x6,3x3) misses the 3e-3 that the mode stands for and this kernel does not;
//  * against the gathering kernel (1x1 layers, stride-2 layers) it wins by 1.3x to 4x from 50 MFLOP on.  Not with a
//    handful of channels and taps that do not fold (the 7x7 stride-2 stem: 3 real channels in every 32-wide k-block,
//    0.69 against 0.57 ms at batch 64);
//  * against the bit-exact fp32 Winograd path (the alternative when single-pass TF32 through Winograd is not
//    accurate enough) it wins on every VGG-16 and ResNet-50 layer at every batch size measured (1.3x to 2.4x).
bool direct_tc_preferred(const fc_conv_desc &d, int oh, int ow, int sm_count, int rival) {
    if (!direct_tc_eligible(d)) return false;
    if (rival == DIRECT_VS_WINOGRAD_FP32) return true;
    int bh = 8, bw = 16;
    direct_patch_shape(oh, ow, &bh, &bw);
    const double patches = (double)ceil_div(oh, bh) * ceil_div(ow, bw) * d.batch;
    const double items = patches * ceil_div(d.oc, 128);
    if (rival == DIRECT_VS_WINOGRAD_TF32) {
        const double h = (double)d.ic * d.oc / (d.ic + d.oc);
        if (patches <= 8 && patches * ceil_div(d.oc, 64) <= sm_count) return true;
        return h <= 100.0 && (items >= sm_count || h <= 48.0);
    }
    const double flops = 2.0 * d.batch * d.oc * d.ic * d.kh * d.kw * oh * ow;
    return flops >= 5e7 && (d.ic >= 16 || folds_taps(d));
}

size_t direct_nhwc_elems(const fc_conv_desc &d) {
    if (folds_taps(d)) {  // one 32-float pixel per OUTPUT position
        const int oh = d.ih + d.pad_top + d.pad_bottom - d.kh + 1, ow = d.iw + d.pad_left + d.pad_right - d.kw + 1;
        return (size_t)d.batch * oh * ow * BK;
    }
    return (size_t)d.batch * d.ih * d.iw * round_up(d.ic, BK);
}

size_t direct_packed_elems(const fc_conv_desc &d) {
    return folds_taps(d) ? (size_t)d.oc * BK : (size_t)d.kh * d.kw * d.oc * round_up(d.ic, BK);
}

// How a layer (taps already folded where they fold) is cut into work items.
struct DirectPlan {
    int bh, bw, n_px, n_py;   // patch of 128 output pixels and patches per image
    int n_oc_items, bn;       // channel blocks
    int ksplit, kb_per_split; // shares of the reduction per output block, k-blocks per share
    long long blocks;         // output blocks = patches x channel blocks
};

static DirectPlan make_plan(const fc_conv_desc &d, int oh, int ow, int sm_count, const KernelCfg *cfg) {
    DirectPlan p;
    p.bh = 8; p.bw = 16;
    direct_patch_shape(oh, ow, &p.bh, &p.bw);
    p.n_px = (int)ceil_div(ow, p.bw);
    p.n_py = (int)ceil_div(oh, p.bh);
    const size_t patches = (size_t)p.n_px * p.n_py * d.batch;
    // Channel blocks of up to 128, or of up to 256: then one CTA per SM holds all of TMEM and moves a quarter less
    // operand bytes per flop.  Measured on the VGG-16 layers with 256 and 512 channels: 447 -> 472 and 481 -> 504
    // TFLOP/s at batch 64, but 4 % slower at batch 8 where a 256-wide block leaves under two work items per SM.
    int max_bn = d.oc >= 256 && patches * ceil_div(d.oc, 256) >= 4 * (size_t)sm_count ? 256 : 128;
    // Fewer work items than SMs: channel blocks of 64 put the layer on more SMs (the pixels are then fetched once per
    // block more, which idle SMs do for free).  cfg.bn = 128 or 256 (Tuning()) overrides.
    while (max_bn > 64 && patches * ceil_div(d.oc, max_bn) < (size_t)sm_count) max_bn /= 2;
    if (cfg && (cfg->bn == 128 || cfg->bn == 256)) max_bn = cfg->bn;
    p.n_oc_items = (int)ceil_div(d.oc, max_bn);
    p.bn = round_up((int)ceil_div(d.oc, p.n_oc_items), 16);  // balanced blocks of channels
    p.blocks = (long long)patches * p.n_oc_items;
    // Still no more output blocks than SMs (the 28x28 and 14x14 layers of one image, every ResNet-50 layer at batch 1):
    // an SM pulls its operands at some 50 GB/s, so a long reduction on a few SMs is bound by that.  The reduction is
    // then shared by several work items (two CTAs per SM in all, at least four k-blocks each) that add their partial
    // sums into the zeroed output; a bias or ReLU follows in a pass of its own.  The order of the additions, hence
    // the last bits of the result, may differ from run to run.  512 -> 512 at 14x14, one image: 0.064 -> 0.0145 ms.
    const int kb_total = d.kh * d.kw * (round_up(d.ic, BK) / BK);
    p.ksplit = 1;
    if (p.blocks <= sm_count && kb_total >= 8) {
        int want = (int)(2 * sm_count / p.blocks);
        if (want > kb_total / 4) want = kb_total / 4;
        if (want > 1) p.ksplit = want;
    }
    p.kb_per_split = (int)ceil_div(kb_total, p.ksplit);
    p.ksplit = (int)ceil_div(kb_total, p.kb_per_split);
    return p;
}

// the layer as the tensor-core kernel sees it: a 1x1, unpadded layer over 32 channels when the taps fold
static fc_conv_desc kernel_view(const fc_conv_desc &full, int oh, int ow) {
    fc_conv_desc d = full;
    if (folds_taps(full)) {
        d.ic = BK; d.ih = oh; d.iw = ow; d.kh = d.kw = 1;
        d.pad_left = d.pad_right = d.pad_top = d.pad_bottom = 0;
    }
    return d;
}

// kernel launches of one forward: the layout pass, the tensor-core kernel, and the bias/ReLU pass of a shared reduction
int direct_tc_launches(const fc_conv_desc &full, int oh, int ow, int sm_count, const KernelCfg *cfg, bool has_epilogue) {
    const DirectPlan p = make_plan(kernel_view(full, oh, ow), oh, ow, sm_count, cfg);
    return 2 + (p.ksplit > 1 && has_epilogue ? 1 : 0);
}

int launch_direct_pack_weights(fc_context *ctx, const float *d_kernel, float *d_wp, const fc_conv_desc &d) {
    // folded taps: a row of W (ic*kh*kw floats) padded to 32 is the one tap of a 1x1 layer over 32 channels
    const bool fold = folds_taps(d);
    const int ic = fold ? d.ic * d.kh * d.kw : d.ic, taps = fold ? 1 : d.kh * d.kw;
    const int icp = round_up(ic, BK);
    const size_t total = direct_packed_elems(d);
    const unsigned blocks = (unsigned)(ceil_div(total, 256) > 4096 ? 4096 : ceil_div(total, 256));
    direct_pack_weights_kernel<<<blocks, 256, 0, ctx->stream>>>(d_kernel, d_wp, d.oc, ic, icp, taps);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

int launch_direct_tc(fc_context *ctx, const float *d_in, float *d_nhwc, const float *d_wp, float *d_out,
                     const fc_conv_desc &full, int oh, int ow, const KernelCfg *cfg, const Epilogue &ep) {
    FC_REQUIRE(direct_tc_eligible(full), FC_ERR_UNSUPPORTED, "the direct tensor-core path takes ungrouped layers of stride 1 or 2");
    FC_REQUIRE(ctx->d_status != nullptr, FC_ERR_INVALID_ARG, "the tensor-core kernels need a context with a status word");
    fc_conv_desc d = full;
    if (folds_taps(full)) {
        const size_t smem = (size_t)full.ic * full.kh * (ow + full.kw - 1) * sizeof(float);
        FC_CHECK_CUDA(cudaFuncSetAttribute(fold_taps_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FC_CHECK_CUDA(launch_pdl(fold_taps_kernel, dim3((unsigned)(full.batch * oh)), dim3(256), smem, ctx->stream, d_in,
                                 d_nhwc, full.ic, full.ih, full.iw, full.kh, full.kw, full.pad_top, full.pad_left, oh, ow));
        d = kernel_view(full, oh, ow);  // from here on: a 1x1, unpadded layer over the 32 folded channels
    }
    const int icp = round_up(d.ic, BK), hw = d.ih * d.iw;
    if (!folds_taps(full)) {
        dim3 grid((unsigned)ceil_div(hw, 32), (unsigned)(icp / 32), (unsigned)d.batch), block(256);
        FC_CHECK_CUDA(launch_pdl(nchw_to_nhwc_kernel, grid, block, 0, ctx->stream, d_in, d_nhwc, d.ic, icp, hw));
    }
    const DirectPlan plan = make_plan(d, oh, ow, ctx->sm_count, cfg);
    const int bh = plan.bh, bw = plan.bw;
    const bool late_epilogue = plan.ksplit > 1 && (ep.bias != nullptr || ep.relu);
    DirectParams P;
    P.out = d_out;
    P.status = ctx->d_status;
    P.ep = late_epilogue ? kNoEpilogue : ep;
    P.oc = d.oc; P.oh = oh; P.ow = ow;
    P.bh = bh; P.bw = bw;
    P.n_px = plan.n_px; P.n_py = plan.n_py;
    P.n_oc_items = plan.n_oc_items;
    P.bn = plan.bn;
    P.num_kb = icp / BK;
    P.taps = d.kh * d.kw;
    P.kw = d.kw;
    P.pad_t = d.pad_top; P.pad_l = d.pad_left;
    P.sh = d.sh; P.sw = d.sw;
    P.acc_cols = pow2_at_least(P.bn, 32);
    P.b_bytes = P.bn * BK * 4;
    P.ksplit = plan.ksplit;
    P.kb_per_split = plan.kb_per_split;
    const long long blocks = plan.blocks;
    if (P.ksplit > 1)
        FC_CHECK_CUDA(cudaMemsetAsync(d_out, 0, (size_t)d.batch * d.oc * oh * ow * sizeof(float), ctx->stream));
    const long long items = blocks * P.ksplit;
    FC_REQUIRE(items < (1ll << 31), FC_ERR_UNSUPPORTED, "too many work items");
    P.n_items = (int)items;
    const size_t stage_bytes = (size_t)A_BYTES + P.b_bytes;
    const bool two_per_sm = P.n_items > ctx->sm_count && 2 * P.acc_cols <= 256;
    const size_t budget = cfg && cfg->smem_kb ? (size_t)cfg->smem_kb * 1024 : (two_per_sm ? 104 * 1024 : 200 * 1024);
    int stages = (int)(budget / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages < 2) stages = 2;
    P.stages = stages;
    const size_t smem = 512 + 1024 + stages * stage_bytes;
    const int per_sm = (2 * P.acc_cols > 256 || smem > 113 * 1024) ? 1 : 2;
    int ctas = ctx->sm_count * per_sm;
    if (ctas > P.n_items) ctas = P.n_items;

    CUtensorMap tmX, tmW;
    FC_PROPAGATE(make_map_nhwc(&tmX, d_nhwc, icp, d.iw, d.ih, d.batch, bw, bh, d.sw, d.sh));
    FC_PROPAGATE(make_map_3d(&tmW, d_wp, icp, d.oc, P.taps, P.bn));
    FC_CHECK_CUDA(cudaFuncSetAttribute(direct_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    FC_CHECK_CUDA(launch_pdl(direct_tc_kernel, dim3((unsigned)ctas), dim3(TC_THREADS), smem, ctx->stream, tmX, tmW, P));
    if (late_epilogue) {
        const size_t total = (size_t)d.batch * d.oc * oh * ow;
        const unsigned nb = (unsigned)(ceil_div(total, 256) > (size_t)ctx->sm_count * 8 ? (size_t)ctx->sm_count * 8 : ceil_div(total, 256));
        FC_CHECK_CUDA(launch_pdl(bias_relu_kernel, dim3(nb), dim3(256), 0, ctx->stream, d_out, ep, d.oc, oh * ow, total));
    }
    return FC_OK;
}

}  // namespace fc
