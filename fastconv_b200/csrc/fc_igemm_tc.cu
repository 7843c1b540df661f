// Implicit-GEMM convolution on tcgen05 tensor cores: the im2col matrix is never built.
//
//   out[img][oc][pixel] = sum_k A[oc][k] * B[k][pixel],   k = (ic*kh + u)*kw + v
//
// A (the weights, K-major) is re-laid out once per layer by pack_weights_kernel into rows of
// Kp = roundup(K, 32) floats -- the job of the reference's pack_a_v2 (im2col/gemm_pack.cpp:192-238) --
// as two planes hi = tf32(a) and lo = a - hi, so TMA boxes can stream either or both.
// B is the reference's gathered matrix (ConvIm2colLayer::im2col, convLayer/im2colConv.cpp:285-309):
// four producer warps compute the same index map on the fly, zero-fill the padding and write the
// 32(k) x BN(pixel) slab straight into shared memory in the K-major 128-byte-swizzled form the UMMA
// descriptor expects (and its lo part in 3xTF32 mode), then hand it to the MMA warp over an mbarrier.
//
//   warp 0      TMA producer for A        warp 1   TMEM owner + MMA issuer
//   warps 2..9  B gather producers (a thread owns a pixel row and one half of the 32 k-steps of a stage);
//   warps 2..5  then run the epilogue (tcgen05.ld -> global)
#include "fc_tc_common.cuh"

namespace fc {

namespace {

using namespace tc;

struct IgemmTcParams {
    const float *in;
    float *out;
    int *status;
    int ic, ih, iw, oc, kh, kw, sh, sw, pad_l, pad_t, oh, ow;
    int K, num_kb, bn, stages, tmem_cols;
    int splits, kb_per_split;  // split-K over blockIdx.z: split s reduces k-blocks [s*kb_per_split, ...)
    const int2 *ktab;          // per-layer k -> (offset, u:v) table padded to 32 entries, or NULL
    Epilogue ep;               // applied by the epilogue warps; never together with split-K
    long long in_img_stride, out_img_stride;  // elements between images (whole tensors for one group of a grouped layer)
};

__global__ void pack_weights_kernel(const float *__restrict__ kernel, float *__restrict__ packed, int oc, int K,
                                    int Kp) {
    const size_t total = (size_t)oc * Kp;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(idx % Kp);
        const size_t r = idx / Kp;
        const float a = k < K ? kernel[r * K + k] : 0.0f;
        const float hi = to_tf32(a);
        packed[idx] = hi;
        packed[total + idx] = a - hi;
    }
}

constexpr int IG_THREADS = TC_THREADS + 128;  // 2 + 8 warps

template <bool kSplit>
__global__ void __launch_bounds__(IG_THREADS) igemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                              const IgemmTcParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full_a[8], full_b[8], empty[8], tmem_full
    const int S = P.stages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 25);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t ring = (smem_u32(smem_raw) + 512 + 1023) & ~1023u;
    uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    const uint32_t b_bytes = (uint32_t)P.bn * BK * 4;
    const uint32_t part_bytes = A_BYTES + b_bytes;
    const uint32_t stage_bytes = part_bytes * (kSplit ? 2 : 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int img = blockIdx.z / P.splits, split = blockIdx.z % P.splits;
    const int oc0 = blockIdx.y * BM, pix0 = blockIdx.x * P.bn;
    const int ohw = P.oh * P.ow;
    const int kb0 = split * P.kb_per_split;
    const int kb1 = min(P.num_kb, kb0 + P.kb_per_split);  // this CTA reduces k-blocks [kb0, kb1)
    if (kb0 >= kb1) return;  // rounding can leave the last split empty (uniform for the whole CTA)

    auto bar_full_a = [&](int s) { return smem_u32(bars + s); };
    auto bar_full_b = [&](int s) { return smem_u32(bars + 8 + s); };
    auto bar_empty = [&](int s) { return smem_u32(bars + 16 + s); };
    const uint32_t bar_tmem_full = smem_u32(bars + 24);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full_a(s), 1);
            mbar_init(bar_full_b(s), 256);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar_tmem_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)P.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer for the weights ----------------
        if (lane == 0) {
            for (int kb = kb0; kb < kb1; ++kb) {
                const int s = (kb - kb0) % S;
                const uint32_t ph = (uint32_t)((kb - kb0) / S) & 1u;
                if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, P.status)) break;
                const uint32_t a_dst = ring + s * stage_bytes;
                mbar_expect_tx(bar_full_a(s), kSplit ? 2 * A_BYTES : A_BYTES);
                tma_load_3d(a_dst, &tmA, bar_full_a(s), kb * BK, oc0, 0);
                if (kSplit) tma_load_3d(a_dst + part_bytes, &tmA, bar_full_a(s), kb * BK, oc0, 1);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_tf32(BM, P.bn);
            for (int kb = kb0; kb < kb1; ++kb) {
                const int s = (kb - kb0) % S;
                const uint32_t ph = (uint32_t)((kb - kb0) / S) & 1u;
                if (!mbar_wait(bar_full_a(s), ph, abort_flag, P.status)) break;
                if (!mbar_wait(bar_full_b(s), ph, abort_flag, P.status)) break;
                tc_fence_after();
                const uint32_t a_hi = ring + s * stage_bytes, b_hi = a_hi + A_BYTES;
                const uint32_t a_lo = a_hi + part_bytes, b_lo = a_lo + A_BYTES;
#pragma unroll
                for (int ks = 0; ks < BK / 8; ++ks) {
                    const uint32_t koff = ks * 32;
                    const uint32_t first = (kb == kb0 && ks == 0) ? 0u : 1u;
                    if (kSplit) {
                        tc_mma_tf32(tmem_base, umma_desc_k_sw128(a_lo + koff), umma_desc_k_sw128(b_hi + koff), idesc, first);
                        tc_mma_tf32(tmem_base, umma_desc_k_sw128(a_hi + koff), umma_desc_k_sw128(b_lo + koff), idesc, 1u);
                        tc_mma_tf32(tmem_base, umma_desc_k_sw128(a_hi + koff), umma_desc_k_sw128(b_hi + koff), idesc, 1u);
                    } else {
                        tc_mma_tf32(tmem_base, umma_desc_k_sw128(a_hi + koff), umma_desc_k_sw128(b_hi + koff), idesc, first);
                    }
                }
                tc_commit(bar_empty(s));
            }
            tc_commit(bar_tmem_full);
        }
    } else {
        // ---------------- gather producers, then epilogue ----------------
        // The gather is asynchronous: a thread issues 4-byte cp.async copies (zero fill outside the image) for its
        // pixel rows of k-block `it` straight to their swizzled place, commits them as one group, and only then
        // finishes k-block it-LAG (waits for that group, splits hi/lo in place for 3xTF32, hands the slab to the MMA
        // warp).  So LAG k-blocks of loads are in flight per thread and global latency is not on the critical path.
        const int gt = (threadIdx.x - 64) & 127;   // pixel row of the slab (and gt + 128 when bn > 128)
        const int kh0 = ((threadIdx.x - 64) >> 7) * (BK / 2);  // this thread gathers k-steps [kh0, kh0 + 16) of a stage
        const int khw = P.kh * P.kw;
        const float *img_ptr = P.in + (size_t)img * P.in_img_stride;
        const int lag = S > 2 ? 2 : S - 1;
        // k -> (element offset, u:v): from the layer's table when there is one (padded to a multiple of 32 entries),
        // else by division; past the reduction a row far below the image, so the copy zero-fills
        auto decode = [&](int k, bool wanted) -> int2 {
            int2 e = make_int2(0, 0x4000 << 16);
            if (!wanted) return e;
            if (P.ktab != nullptr) return __ldg(P.ktab + k);
            if (k < P.K) {
                const int c = k / khw, r2 = k - c * khw;
                const int u = r2 / P.kw, v = r2 - u * P.kw;
                e = make_int2((c * P.ih + u) * P.iw + v, (u << 16) | v);
            }
            return e;
        };
        int2 next_dec = decode(kb0 * BK + lane, true);
        bool ok = true;
        for (int it = kb0; it < kb1 + lag && ok; ++it) {
            if (it < kb1) {
                const int s = (it - kb0) % S;
                const uint32_t ph = (uint32_t)((it - kb0) / S) & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, P.status));  // warp-uniform
                if (!ok) break;
                // lane l of every warp holds the decode of k = it*32 + l (fetched during the previous iteration, so the
                // table read is not waited for here); the values travel by shuffle below
                const int off_mine = next_dec.x, uv_mine = next_dec.y;
                next_dec = decode((it + 1) * BK + lane, it + 1 < kb1);
                const uint32_t b_hi = ring + s * stage_bytes + A_BYTES;
                // a thread owns pixel rows n = gt, gt+128, ... of the slab (bn <= 256); every lane runs the loop
                // and its shuffles, lanes past the slab only skip the copies
                for (int nb = 0; nb < P.bn; nb += 128) {
                    const int n = nb + gt;
                    const bool n_ok = n < P.bn;
                    const int pix = pix0 + n;
                    const bool pix_ok = n_ok && pix < ohw;
                    const int oi = pix_ok ? pix / P.ow : 0, oj = pix_ok ? pix - oi * P.ow : 0;
                    const int base_row = oi * P.sh - P.pad_t, base_col = oj * P.sw - P.pad_l;
                    const float *pix_ptr = img_ptr + (ptrdiff_t)base_row * P.iw + base_col;
                    const uint32_t row_off = (uint32_t)(n >> 3) * 1024u + (uint32_t)(n & 7) * 128u;
                    const uint32_t sw = (uint32_t)(n & 7);
#pragma unroll 8
                    for (int kk = kh0; kk < kh0 + BK / 2; ++kk) {
                        const int off = __shfl_sync(0xffffffffu, off_mine, kk);
                        const int uv = __shfl_sync(0xffffffffu, uv_mine, kk);
                        const int row = base_row + (uv >> 16), col = base_col + (uv & 0xffff);
                        const bool in_img = pix_ok && (unsigned)row < (unsigned)P.ih && (unsigned)col < (unsigned)P.iw;
                        // K-major, 128-byte swizzle: 16-byte chunk index XOR row-in-group
                        const uint32_t o = row_off + ((((uint32_t)kk >> 2) ^ sw) << 4) + ((uint32_t)kk & 3u) * 4u;
                        if (n_ok) {
                            const float *src = in_img ? pix_ptr + off : P.in;
                            const int bytes = in_img ? 4 : 0;  // 0 source bytes: the destination is zero-filled
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(b_hi + o), "l"(src), "r"(bytes)
                                         : "memory");
                        }
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");  // one group per iteration, empty ones in the tail
            const int done = it - lag;
            if (done >= kb0) {
                if (lag == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
                else if (lag == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
                else asm volatile("cp.async.wait_group 0;" ::: "memory");
                const int sd = (done - kb0) % S;
                if (kSplit) {  // this thread's rows only: hi = tf32(x) stays in place, lo = x - hi goes to the lo slab
                    uint8_t *b_hi = ring_ptr + sd * stage_bytes + A_BYTES;
                    uint8_t *b_lo = b_hi + part_bytes;
                    for (int n = gt; n < P.bn; n += 128) {
                        const uint32_t row_off = (uint32_t)(n >> 3) * 1024u + (uint32_t)(n & 7) * 128u;
#pragma unroll
                        for (int c = kh0 / 4; c < kh0 / 4 + 4; ++c) {  // the four 16-byte chunks this thread copied
                            const uint32_t at = row_off + (((uint32_t)c ^ (uint32_t)(n & 7)) << 4);
                            float4 x = *reinterpret_cast<const float4 *>(b_hi + at);
                            float4 h = make_float4(to_tf32(x.x), to_tf32(x.y), to_tf32(x.z), to_tf32(x.w));
                            *reinterpret_cast<float4 *>(b_hi + at) = h;
                            *reinterpret_cast<float4 *>(b_lo + at) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(bar_full_b(sd));
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // nothing of this thread is in flight past this point
        if (warp < 6 && mbar_wait(bar_tmem_full, 0u, abort_flag, P.status)) {
            tc_fence_after();
            const int q = warp & 3;
            const int row = oc0 + q * 32 + lane;
            float *dst = P.out + (size_t)img * P.out_img_stride + (size_t)row * ohw + pix0;
            for (int c0 = 0; c0 < P.bn; c0 += 16) {
                float v[16];
                tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                if (row < P.oc) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (pix0 + c0 + j < ohw) {
                            if (P.splits > 1) atomicAdd(dst + c0 + j, v[j]);  // partial sum of this K range
                            else dst[c0 + j] = P.ep(v[j], row);
                        }
                }
            }
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P.tmem_cols)
                     : "memory");
    }
}

}  // namespace

size_t igemm_packed_elems(int oc, int K) { return (size_t)2 * oc * round_up(K, tc::BK); }

int launch_igemm_pack_weights(fc_context *ctx, const float *d_kernel, float *d_packed, int oc, int K) {
    const int Kp = round_up(K, tc::BK);
    const size_t total = (size_t)oc * Kp;
    const unsigned blocks = (unsigned)(ceil_div(total, 256) > 148 * 16 ? 148 * 16 : ceil_div(total, 256));
    pack_weights_kernel<<<blocks, 256, 0, ctx->stream>>>(d_kernel, d_packed, oc, K, Kp);
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

int launch_igemm_tc(fc_context *ctx, const float *d_in, const float *d_packed, float *d_out, const fc_conv_desc &d,
                    int oh, int ow, int mode, const KernelCfg *cfg, const int *d_ktab, const Epilogue &ep,
                    size_t in_img_stride, size_t out_img_stride) {
    using namespace tc;
    const bool split = mode == FC_MATH_3XTF32;
    const int K = d.ic * d.kh * d.kw, Kp = round_up(K, BK);
    const int ohw = oh * ow;
    const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int num_kb = Kp / BK;
    // Filling the machine with a small problem: split K first (a split re-reads nothing: every CTA still streams its
    // own part of the weights once), and only then narrow the pixel blocks (every extra block column re-reads the
    // weights of its row).  Tuning() showed the opposite order losing 15-20 % on the strided 3x3 ResNet layers.
    const bool may_split = ep.bias == nullptr && !ep.relu;  // bias and ReLU act on the complete sum only
    auto plan = [&](int max_bn, int *bn_out, int *n_blk_out, int *splits_out) -> size_t {
        const int n_blk = (ohw + max_bn - 1) / max_bn;
        const int bn = round_up((ohw + n_blk - 1) / n_blk, 16);
        const size_t base = (size_t)n_blk * ceil_div(d.oc, BM) * d.batch;
        int splits = 1;
        while (may_split && base * splits * 2 <= (size_t)sms && num_kb / (splits * 2) >= 4 &&
               (size_t)d.batch * splits * 2 <= 65535)
            splits *= 2;
        *bn_out = bn; *n_blk_out = n_blk; *splits_out = splits;
        return base * splits;
    };
    int bn, n_blk, splits;
    int max_bn = cfg && cfg->bn >= 16 && cfg->bn <= 256 ? cfg->bn : 128;
    size_t n_ctas = plan(max_bn, &bn, &n_blk, &splits);
    if (!(cfg && cfg->bn))
        while (max_bn > 32 && 2 * n_ctas < (size_t)sms) {
            max_bn /= 2;
            n_ctas = plan(max_bn, &bn, &n_blk, &splits);
        }
    IgemmTcParams P;
    P.in = d_in; P.out = d_out; P.status = ctx->d_status;
    P.ic = d.ic; P.ih = d.ih; P.iw = d.iw; P.oc = d.oc; P.kh = d.kh; P.kw = d.kw; P.sh = d.sh; P.sw = d.sw;
    P.pad_l = d.pad_left; P.pad_t = d.pad_top; P.oh = oh; P.ow = ow;
    P.K = K; P.num_kb = num_kb; P.bn = bn; P.tmem_cols = pow2_at_least(bn, 32);
    P.splits = splits;
    P.ktab = reinterpret_cast<const int2 *>(d_ktab);
    P.ep = ep;
    P.in_img_stride = in_img_stride ? (long long)in_img_stride : (long long)d.ic * d.ih * d.iw;
    P.out_img_stride = out_img_stride ? (long long)out_img_stride : (long long)d.oc * ohw;
    P.kb_per_split = (num_kb + splits - 1) / splits;
    const size_t stage_bytes = (size_t)(A_BYTES + bn * BK * 4) * (split ? 2 : 1);
    const size_t budget = cfg && cfg->smem_kb ? (size_t)cfg->smem_kb * 1024
                                              : (n_ctas > (size_t)ctx->sm_count ? 104 * 1024 : 200 * 1024);
    int stages = (int)(budget / stage_bytes);
    if (stages > 8) stages = 8;
    if (stages > P.kb_per_split) stages = P.kb_per_split;
    if (stages < 2) stages = 2;
    P.stages = stages;
    const size_t smem = 512 + 1024 + stages * stage_bytes;
    FC_REQUIRE(smem <= 227 * 1024, FC_ERR_UNSUPPORTED, "pixel block of %d does not fit the shared-memory ring", bn);

    CUtensorMap tmA;  // [2 planes][oc][Kp]
    FC_PROPAGATE(make_map_3d(&tmA, d_packed, Kp, d.oc, 2, BM));
    dim3 grid((unsigned)n_blk, (unsigned)ceil_div(d.oc, BM), (unsigned)(d.batch * splits)), block(IG_THREADS);
    if (splits > 1) {  // the K ranges add their partial sums into a zeroed output (this launch's channels only)
        if (P.out_img_stride == (long long)d.oc * ohw) {
            FC_CHECK_CUDA(cudaMemsetAsync(d_out, 0, (size_t)d.batch * d.oc * ohw * sizeof(float), ctx->stream));
        } else {
            FC_CHECK_CUDA(cudaMemset2DAsync(d_out, (size_t)P.out_img_stride * sizeof(float), 0,
                                            (size_t)d.oc * ohw * sizeof(float), (size_t)d.batch, ctx->stream));
        }
    }
    if (split) {
        FC_CHECK_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        igemm_tc_kernel<true><<<grid, block, smem, ctx->stream>>>(tmA, P);
    } else {
        FC_CHECK_CUDA(cudaFuncSetAttribute(igemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        igemm_tc_kernel<false><<<grid, block, smem, ctx->stream>>>(tmA, P);
    }
    FC_CHECK_CUDA(cudaGetLastError());
    return FC_OK;
}

}  // namespace fc
