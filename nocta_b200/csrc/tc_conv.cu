// Halo-resident tensor-core kernels for stride-1 convolutions with filters up to 3 x 3 (plain TF32 mode), sm_100a:
// TMA-fed tcgen05.mma (kind::tf32), accumulators in tensor memory, inline PTX.
//
// An implicit-GEMM convolution that streams one operand tile per filter tap re-reads the same pixels for every tap.  The
// kernels here load a pixel tile WITH its halo once and address every tap inside it by moving the start address of the
// shared-memory matrix descriptor: the swizzle of a TMA-written tile is a function of the absolute shared-memory
// address, so a descriptor may start at any 128-byte pixel row and use any stride between its 8-row groups (K-major
// operands) or 4-row atoms (MN-major operands, 32-byte swizzle atoms).
//
// What bounds these kernels is not operand delivery but MMA ISSUE: measured on B200, one thread issues a tcgen05.mma with
// fresh descriptors every 65 - 80 cycles at best, a barrier test costs it another ~180 cycles, while the tensor pipe needs
// 128 cycles for M = 128, N = 256, 64 for N = 128 and 48 for N = 64 (K = 8).  MMAs into ONE accumulator must come from one
// thread to stay ordered, but different accumulators can be issued by different warps.  So: one barrier round trip covers
// as many filter taps as leave two weight stages in shared memory (a filter row of 128-row weight tiles, five taps of 64-row
// ones), and wherever a tile has several accumulators they get an issuing warp each.
//
//   convh_kernel<false>  forward / input gradient, output channels on M (weights = A, streamed one filter row per
//                        stage), 8 x <=32 pixels of one image on N (halo = B).  One MMA of N = 8 * rows per k-step, one
//                        issuing warp.  Used from 128 output channels on.  Eight epilogue warps (two per quarter of the
//                        accumulator's lanes): one warp per scheduler executes dependent epilogue code at a few cycles
//                        per instruction, which bounded the kernel as soon as the epilogue did more than store.  Its
//                        epilogue can also sum, per channel, what the backward pass of a BatchNorm+ReLU that produced
//                        this convolution's input needs (see nc_cuda_offer_batchnorm_backward_sums_f32).
//   convh_kernel<false, 0, true>  the same for images of exactly 16 rows: two images per tile, each with its own issuing
//                        warp (N = 128) and half of the accumulator's columns.
//   convh_kernel<true>   the same convolution with the roles swapped for layers with at most 96 output channels: 8 x 16
//                        pixels on M (halo = A), all output channels on N (weights = B).  An MMA costs
//                        max(N / 2, operand bytes / 128, ~46) cycles whatever M is, so 64 channels on M run at half
//                        rate while 128 pixels on M with N = 64 run at two thirds.  The two 8 x 16 blocks of a tile have
//                        their own accumulators and issuing warps; up to 64 channels a second pair of warps takes
//                        k-steps 2 and 3 into accumulators of its own, which the epilogue adds.  The epilogue transposes
//                        each 32 pixel x 32 channel block through shared memory so that a warp stores whole lines.
//   dwh_kernel<false>    weight gradient for Cin % 128 == 0: A = dY tile (128 output channels, MN-major), B = x halo
//                        tile (128 input channels, MN-major); one filter row per work item, the kW taps of the row are kW
//                        MMAs per 8-pixel k-step against the same two tiles (B start moved by kw pixel rows) into kW
//                        accumulators, each with its own issuing warp.  dY and x cross from L2 to shared memory kH times
//                        instead of kH * kW times, as a few large copies per stage.
//   dwh_kernel<true>     weight gradient for narrower inputs: A = ONE 32-channel x halo chunk addressed with a leading
//                        byte offset of one pixel row, so the four 32-row chunks of M are the same channels shifted by
//                        0..3 pixels = the kW taps of a filter row (kW = 3: three quarters of M useful); B = dY tile;
//                        one accumulator and one issuing warp per filter row, all kH * kW taps per work item.
//
// Pixel tiles may hang over the image edge: TMA zero-fills what it loads there (which is also the padding) and the
// epilogues mask what they store.  No cluster launch and no multicast: each CTA loads its own tiles.  Every mbarrier
// wait is bounded; on expiry the kernel records a code in the device error word, drains, frees its TMEM and returns.
#include "tc_gemm.cuh"
#include "tc_ptx.cuh"
#include "../../include/nocta_cuda.h"

namespace tc {

namespace {
constexpr int kBM = 128;
constexpr int kWTileBytes = 128 * 128;  // one weight stage: up to 128 rows of 32 floats
constexpr int kConvhWStages = 12;       // ring slots available; a launch uses as many as fit into the 96 KB weight region
constexpr int kTW = 8, kTH = 32;        // pixel tile of the convolution kernels
constexpr int kMaxDynSmem = 227 * 1024 - 2048;

__device__ __forceinline__ uint32_t idesc_tf32(uint32_t M, uint32_t N, bool a_mn, bool b_mn) {
    // D = f32, A = B = tf32, operand majors, N / 8, M / 16
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
}  // namespace

// ------------------------------------------------------------------------------------------
// convh_kernel
// ------------------------------------------------------------------------------------------
struct ConvhParams {
    float* D;
    int ldd;
    const float* bias;
    int M;                 // output channels
    int Ho, Wo;
    int tiles_w, tiles_h;  // pixel tiles per image
    int tiles_px;          // pixel tiles in total (images * tiles_h * tiles_w)
    int tiles_m;           // 128-channel tiles (1 when the pixels are on M)
    int kH, kW, pad;
    int cchunks;           // 32-channel chunks of the input channels
    int wrows;             // rows per tap in the packed weights
    int wbox_bytes;        // bytes one weight copy delivers
    int wstages;           // weight ring depth: slots of wslot_bytes in the 96 KB weight region
    int wslot_bytes;       // one slot holds `tps` taps (one mbarrier round trip per 4 * tps MMAs)
    int pitch;             // halo line pitch in pixels
    int halo_bytes, halo_stride;
    int half_rows;         // DUAL: halo lines per image (the tile holds two images of 16 rows, one above the other)
    int tps;               // filter taps per weight stage, in (kh, kw) order; the last stage of a chunk may hold fewer
    double* stat;          // non-null: per CTA and channel (sum, sum of squares) of the output it wrote, [gridDim.x][M][2]
    // non-null bnx: the output is the upstream gradient g of a BatchNorm+ReLU with input bnx (same shape and strides as D);
    // stat then receives (sum of g', sum of g' * xhat), g' = g where gamma * xhat + beta > 0 and 0 elsewhere
    const float* bnx;
    const float* bn_mean;
    const float* bn_var;
    const float* bn_gamma;
    const float* bn_beta;
    float bn_eps;
    unsigned int* err;
};

// PXM: pixels on M.  NCH: output channels / 32 (PXM only; 0 otherwise).  DUAL (channels on M only): images of 16 rows, two
// per tile.  The output of an image pair is one run of 32 pixel rows, so everything but the halo load and the MMA issue sees
// a 32-row image; the halo box spans two images (each with its own padding lines), and because the second image's lines do
// not continue the first one's at the stride of a pixel row, each image half (N = 128) has its own issuing warp and its own
// half of the accumulator's columns - which is also what keeps the pipe busy with N = 128 MMAs.
template <bool PXM, int NCH, bool DUAL = false>
__global__ void __launch_bounds__(PXM ? 288 : (DUAL ? 352 : 320), 1)
convh_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const ConvhParams p) {
    constexpr int WSMAX = kConvhWStages;
    // MMA-issuing warps.  Channels on M: one.  Pixels on M: one per 8 x 16 pixel block of the tile, and with at most 64
    // output channels a second pair that takes k-steps 2 and 3 of every tap into accumulators of its own (added by the
    // epilogue): the short N <= 64 MMAs need four issuing threads to keep the tensor pipe busy.
    constexpr int KSPLIT = (PXM && NCH <= 2) ? 2 : 1;
    constexpr int NISS = PXM ? 2 * KSPLIT : (DUAL ? 2 : 1);
    const int WS = p.wstages;
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t bar_hfull[2];
    __shared__ __align__(8) uint64_t bar_hempty[2];
    __shared__ __align__(8) uint64_t bar_wfull[WSMAX];
    __shared__ __align__(8) uint64_t bar_wempty[WSMAX];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ double stat_sh[PXM ? 4 * NCH * 32 * 2 : 1];
    __shared__ __align__(16) float stat_tile[PXM ? 4 : 1][PXM ? 32 : 1][PXM ? 36 : 1];   // per epilogue warp: 32 pixels x 32 channels, transposed between the accumulator (lane = pixel) and the store (lane = channel)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t halo_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    const uint32_t w_base = halo_base + 2u * (uint32_t)p.halo_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; s++) {
            mbar_init(smem_u32(&bar_hfull[s]), 1);
            mbar_init(smem_u32(&bar_hempty[s]), NISS);     // one arrival per MMA-issuing warp
            mbar_init(smem_u32(&bar_acc_full[s]), NISS);
            mbar_init(smem_u32(&bar_acc_empty[s]), PXM ? 128 : 256);   // channels on M: two epilogue warps per lane quarter
        }
        for (int s = 0; s < WS; s++) {
            mbar_init(smem_u32(&bar_wfull[s]), 1);
            mbar_init(smem_u32(&bar_wempty[s]), NISS);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abortp = &abort_flag;
    const int total_tiles = p.tiles_px * p.tiles_m;  // t -> (pixel tile fastest, then channel tile)
    const int ntaps = p.kH * p.kW;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer: halo boxes (one chunk ahead) and weight tiles ----------------
            int ht = blockIdx.x, hcc = 0;   // cursor of the next halo to request
            uint32_t hcount = 0;
            bool ok = true;
            auto issue_halo = [&]() {
                if (ht >= total_tiles || !ok) return;
                const uint32_t slot = hcount & 1u;
                if (!mbar_wait(smem_u32(&bar_hempty[slot]), ((hcount >> 1) & 1u) ^ 1u, p.err, 0x600u + slot, abortp)) { ok = false; return; }
                const int pt = ht % p.tiles_px;
                const int tw = pt % p.tiles_w, tt = pt / p.tiles_w;
                const int th = tt % p.tiles_h, n = tt / p.tiles_h;
                const uint32_t full = smem_u32(&bar_hfull[slot]);
                mbar_expect_tx(full, (uint32_t)p.halo_bytes);
                tma_4d(halo_base + slot * (uint32_t)p.halo_stride, &tmX, hcc * 32, tw * kTW - p.pad, th * kTH - p.pad, DUAL ? 2 * n : n, full);
                hcount++;
                if (++hcc == p.cchunks) { hcc = 0; ht += gridDim.x; }
            };
            int s = 0;
            uint32_t ph = 0;
            issue_halo();
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int m0 = (t / p.tiles_px) * (PXM ? NCH * 32 : kBM);
                for (int cc = 0; cc < p.cchunks && ok; cc++) {
                    int wrow = m0;
                    for (int t0 = 0; t0 < ntaps && ok; t0 += p.tps) {
                        if (t0 == (ntaps > p.tps ? p.tps : 0)) issue_halo();   // the next chunk's halo, once this chunk is under way
                        if (!ok) break;
                        const int nt = (ntaps - t0) < p.tps ? (ntaps - t0) : p.tps;
                        if (!mbar_wait(smem_u32(&bar_wempty[s]), ph ^ 1u, p.err, 0x100u + s, abortp)) { ok = false; break; }
                        const uint32_t full = smem_u32(&bar_wfull[s]);
                        mbar_expect_tx(full, (uint32_t)(nt * p.wbox_bytes));
                        for (int i = 0; i < nt; i++, wrow += p.wrows)
                            tma_2d(w_base + (uint32_t)(s * p.wslot_bytes + i * p.wbox_bytes), &tmW, cc * 32, wrow, full);
                        if (++s == WS) { s = 0; ph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1 || (PXM && warp >= 6) || (DUAL && warp == 10)) {
        // ---------------- MMA issuers.  MMAs into one accumulator must come from one thread to stay ordered, and one
        // thread issues an MMA with fresh descriptors only every hundred-odd cycles; with the pixels on M the two
        // 8 x 16 pixel blocks of a tile have their own accumulators, so warp 1 issues the upper block and warp 6 the
        // lower one.  With the channels on M there is one accumulator and warp 1 issues alone.  The whole warp runs
        // the loop, lane 0 issues.
        const int issuer = warp == 1 ? 0 : (DUAL ? 1 : warp - 5);   // 0..3
        const int iss = issuer & 1, khalf = issuer >> 1;  // pixel block, half of the k-steps
        if (issuer < NISS) {
            const uint32_t leader = lane == 0 ? 1u : 0u;
            const uint64_t dw0 = smem_desc(w_base, 16u, 1024u, 2u);                      // weight tile: K-major, dense 8-row groups
            const uint64_t dh0 = smem_desc(halo_base, 16u, (uint32_t)p.pitch * 128u, 2u);  // halo: 8-row groups one halo line apart
            const uint32_t idesc_px = idesc_tf32(128u, (uint32_t)(NCH * 32), false, false);
            // this issuer's 8 x 16 pixel block (pixels on M), or its image of the pair (DUAL)
            const uint64_t sub_off = (uint64_t)(((uint32_t)((DUAL ? p.half_rows : 16) * iss * p.pitch) * 128u) >> 4);
            int s = 0;
            uint32_t ph = 0, tile_iter = 0, hcount = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, tile_iter++) {
                const uint32_t ab = tile_iter & 1u;
                const int th = ((t % p.tiles_px) / p.tiles_w) % p.tiles_h;
                const int rows = (p.Ho - th * kTH) < kTH ? (p.Ho - th * kTH) : kTH;
                const uint32_t idesc_ch = idesc_tf32(128u, DUAL ? 128u : (uint32_t)(8 * ((rows + 1) & ~1)), false, false);
                const bool active = !PXM || rows > 16 * iss;   // a short tile has no lower block: that issuer only keeps the barriers moving
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_acc_empty[ab]), ((tile_iter >> 1) & 1u) ^ 1u, p.err, 0x500u + ab, abortp));
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + ab * 256u + (uint32_t)(PXM ? khalf * 128 + iss * NCH * 32 : (DUAL ? iss * 128 : 0));
                uint32_t acc_started = 0u;   // the first MMA of a tile overwrites the accumulator
                for (int cc = 0; cc < p.cchunks && ok; cc++, hcount++) {
                    const uint32_t slot = hcount & 1u;
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_hfull[slot]), (hcount >> 1) & 1u, p.err, 0x700u + slot, abortp));
                    if (!ok) break;
                    const uint64_t dhs = dh0 + sub_off + (uint64_t)((slot * (uint32_t)p.halo_stride) >> 4);
                    uint64_t dh_row = dhs;   // first pixel of filter row kh in this issuer's part of the halo
                    int kw = 0;
                    for (int t0 = 0; t0 < ntaps; t0 += p.tps) {
                        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_wfull[s]), ph, p.err, 0x200u + s, abortp));
                        if (!ok) break;
                        tc_fence_after();
                        const int nt = (ntaps - t0) < p.tps ? (ntaps - t0) : p.tps;
                        uint64_t dw = dw0 + (uint64_t)(((uint32_t)s * (uint32_t)p.wslot_bytes) >> 4);
                        for (int i = 0; i < nt; i++, dw += (uint64_t)((uint32_t)p.wbox_bytes >> 4)) {
                            if (active) {
                                const uint64_t dh = dh_row + (uint64_t)(uint32_t)(kw * 8);   // one halo pixel = 128 bytes = 8 units
#pragma unroll
                                for (int k2 = 0; k2 < 4 / KSPLIT; k2++) {
                                    const int ks = khalf * (4 / KSPLIT) + k2;
                                    const uint32_t accum = acc_started | (uint32_t)(k2 != 0);
                                    if (PXM) umma_tf32_w(acc, dh + (uint64_t)(ks * 2), dw + (uint64_t)(ks * 2), idesc_px, accum, leader);
                                    else umma_tf32_w(acc, dw + (uint64_t)(ks * 2), dh + (uint64_t)(ks * 2), idesc_ch, accum, leader);
                                }
                                acc_started = 1u;
                            }
                            if (++kw == p.kW) { kw = 0; dh_row += (uint64_t)((uint32_t)p.pitch * 8u); }
                        }
                        umma_commit_w(smem_u32(&bar_wempty[s]), leader);
                        if (++s == WS) { s = 0; ph ^= 1u; }
                    }
                    if (ok) umma_commit_w(smem_u32(&bar_hempty[slot]), leader);
                }
                if (ok) umma_commit_w(smem_u32(&bar_acc_full[ab]), leader);
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int q = warp & 3;
        const int r = q * 32 + lane;
        uint32_t tile_iter = 0;
        bool ok = true;
        if (!PXM) {
            // Eight warps: two per quarter of the accumulator's lanes, `half` 0 takes the even 32-column chunks of a tile and
            // `half` 1 the odd ones.  One warp per scheduler executes this dependent code at a few cycles per instruction;
            // with four warps the epilogue of a tile took longer than its MMAs once anything was added to the plain store.
            const int half = (warp - 2) >> 2;
            // lane = output channel, column = pixel.  Output statistics: a thread owns channel m0 + r of every tile it
            // sees, so it keeps one running pair per channel tile and writes it once (slab = this CTA):
            // stat[2 * blockIdx.x + half][M][2].  Slots of channel tiles this CTA never visits must read zero.
            double ssum = 0.0, ssq = 0.0;
            int stat_m0 = -1;
            double* const stat_slab = p.stat ? p.stat + (size_t)(2 * blockIdx.x + half) * p.M * 2 : nullptr;
            if (p.stat)
                for (int mt = 0; mt < p.tiles_m; mt++)
                    if (mt * kBM + r < p.M) {
                        double* sd = stat_slab + (size_t)(mt * kBM + r) * 2;
                        sd[0] = 0.0; sd[1] = 0.0;
                    }
            // 128-byte lines (pixel x 32-channel segment) of a tile's part of the BatchNorm input, spread over the 256 threads
            auto prefetch_tile = [&](int tn) {
                const int pt = tn % p.tiles_px, m0 = (tn / p.tiles_px) * kBM;
                const int tw = pt % p.tiles_w, tt = pt / p.tiles_w;
                const int th = tt % p.tiles_h, n = tt / p.tiles_h;
                const int rows = (p.Ho - th * kTH) < kTH ? (p.Ho - th * kTH) : kTH;
                const int wlim = p.Wo - tw * kTW;
                const float* tb = p.bnx + (((long long)n * p.Ho + th * kTH) * p.Wo + tw * kTW) * p.ldd + m0;
                const int segs = (p.M - m0 + 31) / 32 < 4 ? (p.M - m0 + 31) / 32 : 4;
                for (int L = half * 128 + r; L < rows * 32; L += 256) {
                    const int seg = L & 3, px = L >> 2, hh = px >> 3, j = px & 7;
                    if (j < wlim && seg < segs) prefetch_l2(tb + ((long long)hh * p.Wo + j) * p.ldd + seg * 32);
                }
            };
            for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, tile_iter++) {
                const int pt = t % p.tiles_px, m0 = (t / p.tiles_px) * kBM;
                if (p.stat && m0 != stat_m0) {
                    if (stat_m0 >= 0 && stat_m0 + r < p.M) {
                        double* sd = stat_slab + (size_t)(stat_m0 + r) * 2;
                        sd[0] = ssum; sd[1] = ssq;
                    }
                    ssum = 0.0; ssq = 0.0; stat_m0 = m0;
                }
                const int tw = pt % p.tiles_w, tt = pt / p.tiles_w;
                const int th = tt % p.tiles_h, n = tt / p.tiles_h;
                const int rows = (p.Ho - th * kTH) < kTH ? (p.Ho - th * kTH) : kTH;   // image rows this tile holds
                const int wlim = p.Wo - tw * kTW;                                     // columns j < wlim are inside the image
                const int nchunks = (8 * rows + 31) / 32;                             // 32-column chunks of the tile
                const int first_c0 = half * 32;                                       // this warp: chunks half, half + 2, ...
                const int last_c0 = (nchunks - 1 - half) >= 0 ? (half + 2 * ((nchunks - 1 - half) / 2)) * 32 : -1;   // -1: none
                const uint32_t ab = tile_iter & 1u;
                const int co = m0 + r;
                const bool co_ok = co < p.M;
                const float bv = (co_ok && p.bias) ? p.bias[co] : 0.f;
                // first pixel of the tile; a column chunk of 32 = 4 image rows x 8 pixels
                float* tile_dst = p.D + (((long long)n * p.Ho + th * kTH) * p.Wo + tw * kTW) * p.ldd + co;
                const int line = p.Wo * p.ldd;  // elements between image rows (< 2^31 checked by the host)
                const bool bn = p.bnx != nullptr;
                const float* tile_bsrc = bn ? p.bnx + (tile_dst - p.D) : nullptr;
                float mu = 0.f, is = 1.f, ga = 1.f, be = 0.f;
                // BatchNorm input of one column chunk (4 image rows x 8 pixels of this thread's channel)
                auto load_bn = [&](int c0, float* xb) {
                    const int h4 = c0 >> 3;
                    const float* bsrc = tile_bsrc + (long long)h4 * line;
                    if (!co_ok) return;
                    if (wlim >= 8 && h4 + 4 <= rows) {
#pragma unroll
                        for (int hh = 0; hh < 4; hh++)
#pragma unroll
                            for (int j = 0; j < 8; j++) xb[hh * 8 + j] = __ldg(bsrc + hh * line + j * p.ldd);
                    } else {
#pragma unroll
                        for (int hh = 0; hh < 4; hh++)
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                xb[hh * 8 + j] = (h4 + hh < rows && j < wlim) ? __ldg(bsrc + hh * line + j * p.ldd) : 0.f;
                    }
                };
                float xb[32];
                if (bn) {
                    // The BatchNorm input of the NEXT tile of this CTA is requested into L2 now, a whole tile ahead of its use
                    // (the loads of the epilogue are few per SM: from DRAM their latency would bound the kernel), and the first
                    // chunk of this tile is loaded while its MMAs still run.
                    if (t == (int)blockIdx.x) prefetch_tile(t);
                    if (t + (int)gridDim.x < total_tiles) prefetch_tile(t + (int)gridDim.x);
                    if (co_ok) {
                        mu = p.bn_mean[co];
                        is = rsqrtf(p.bn_var[co] + p.bn_eps);
                        if (p.bn_gamma) ga = p.bn_gamma[co];
                        if (p.bn_beta) be = p.bn_beta[co];
                    }
                    if (last_c0 >= 0) load_bn(first_c0, xb);
                }
                ok = mbar_wait(smem_u32(&bar_acc_full[ab]), (tile_iter >> 1) & 1u, p.err, 0x400u + ab, abortp);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + ab * 256u + ((uint32_t)(q * 32) << 16);
                if (last_c0 < 0) {   // a tile of at most four image rows has no odd chunk: only release the accumulator
                    tc_fence_before();
                    mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                }
#pragma unroll 1
                for (int c0 = first_c0; c0 <= last_c0; c0 += 64) {
                    uint32_t v[32];
                    tmem_ld32(acc + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (c0 == last_c0) {
                        tc_fence_before();
                        mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                    }
                    if (!co_ok) continue;
                    const int h4 = c0 >> 3;
                    float* dst = tile_dst + (long long)h4 * line;
                    float fs = 0.f, fq = 0.f;
                    if (bn) {
                        // gradient of a BatchNorm+ReLU output: sums of g' and g' * xhat against the BatchNorm's input, whose
                        // next chunk is requested before this one is used
                        const bool full = wlim >= 8 && h4 + 4 <= rows;
                        float xn[32];
                        if (c0 < last_c0) load_bn(c0 + 64, xn);
                        if (full) {
#pragma unroll
                            for (int hh = 0; hh < 4; hh++) {
#pragma unroll
                                for (int j = 0; j < 8; j++) {
                                    const float o = __uint_as_float(v[hh * 8 + j]) + bv;
                                    dst[j * p.ldd] = o;
                                    const float xh = (xb[hh * 8 + j] - mu) * is;
                                    const float g = ((ga * xh + be) > 0.f) ? o : 0.f;
                                    fs += g;
                                    fq = fmaf(g, xh, fq);
                                }
                                dst += line;
                            }
                        } else {
#pragma unroll
                            for (int hh = 0; hh < 4; hh++) {
#pragma unroll
                                for (int j = 0; j < 8; j++)
                                    if (h4 + hh < rows && j < wlim) {
                                        const float o = __uint_as_float(v[hh * 8 + j]) + bv;
                                        dst[j * p.ldd] = o;
                                        const float xh = (xb[hh * 8 + j] - mu) * is;
                                        const float g = ((ga * xh + be) > 0.f) ? o : 0.f;
                                        fs += g;
                                        fq = fmaf(g, xh, fq);
                                    }
                                dst += line;
                            }
                        }
                        if (c0 < last_c0) {
#pragma unroll
                            for (int j = 0; j < 32; j++) xb[j] = xn[j];
                        }
                    } else if (wlim >= 8 && h4 + 4 <= rows) {
#pragma unroll
                        for (int hh = 0; hh < 4; hh++) {
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const float o = __uint_as_float(v[hh * 8 + j]) + bv;
                                dst[j * p.ldd] = o;
                                fs += o;
                                fq = fmaf(o, o, fq);
                            }
                            dst += line;
                        }
                    } else {
#pragma unroll
                        for (int hh = 0; hh < 4; hh++) {
                            if (h4 + hh < rows) {
#pragma unroll
                                for (int j = 0; j < 8; j++)
                                    if (j < wlim) {
                                        const float o = __uint_as_float(v[hh * 8 + j]) + bv;
                                        dst[j * p.ldd] = o;
                                        fs += o;
                                        fq = fmaf(o, o, fq);
                                    }
                            }
                            dst += line;
                        }
                    }
                    ssum += (double)fs;
                    ssq += (double)fq;
                }
            }
            if (p.stat && stat_m0 >= 0 && stat_m0 + r < p.M) {
                double* sd = stat_slab + (size_t)(stat_m0 + r) * 2;
                sd[0] = ssum; sd[1] = ssq;
            }
        } else {
            // lane = pixel (8 wide x 16 high block, two blocks per tile), column = output channel: a thread stores runs
            // of 32 consecutive channels of its pixel.  Output statistics: each warp transposes its 32 pixel x 32 channel
            // block through shared memory so that lane c sums channel c over the 32 pixels, keeps running sums per
            // channel chunk over all tiles of the CTA, and the four warps are combined once at the end.
            constexpr int NCHS = NCH > 0 ? NCH : 1;
            double fs[NCHS], fq[NCHS];
#pragma unroll
            for (int c = 0; c < NCHS; c++) { fs[c] = 0.0; fq[c] = 0.0; }
            const bool want_stat = p.stat != nullptr;
            const int wq = warp - 2;   // 0..3: this warp's tile in shared memory
            int stat_m0 = -1;
            auto flush_stats = [&](int m0) {
                // the four warps through shared memory, in a fixed order
                asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
                for (int ch = 0; ch < NCH; ch++) {
                    stat_sh[((wq * NCHS + ch) * 32 + lane) * 2] = fs[ch];
                    stat_sh[((wq * NCHS + ch) * 32 + lane) * 2 + 1] = fq[ch];
                    fs[ch] = 0.0; fq[ch] = 0.0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int c = threadIdx.x - 64; c < NCH * 32; c += 128) {
                    double a = 0.0, b = 0.0;
                    for (int k = 0; k < 4; k++) { a += stat_sh[((k * NCHS + c / 32) * 32 + (c & 31)) * 2]; b += stat_sh[((k * NCHS + c / 32) * 32 + (c & 31)) * 2 + 1]; }
                    double* sd = p.stat + ((size_t)blockIdx.x * p.M + m0 + c) * 2;
                    sd[0] = a; sd[1] = b;
                }
            };
            if (want_stat)   // slots of channel tiles this CTA never visits must read zero
                for (int c = threadIdx.x - 64; c < p.M; c += 128) {
                    double* sd = p.stat + ((size_t)blockIdx.x * p.M + c) * 2;
                    sd[0] = 0.0; sd[1] = 0.0;
                }
            for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, tile_iter++) {
                const int pt = t % p.tiles_px, m0 = (t / p.tiles_px) * (NCH * 32);
                if (want_stat && m0 != stat_m0) {   // the tile walk visits the channel tiles one after the other
                    if (stat_m0 >= 0) flush_stats(stat_m0);
                    stat_m0 = m0;
                }
                const int tw = pt % p.tiles_w, tt = pt / p.tiles_w;
                const int th = tt % p.tiles_h, n = tt / p.tiles_h;
                const int rows = (p.Ho - th * kTH) < kTH ? (p.Ho - th * kTH) : kTH;
                const int nsub = rows > 16 ? 2 : 1;
                const uint32_t ab = tile_iter & 1u;
                ok = mbar_wait(smem_u32(&bar_acc_full[ab]), (tile_iter >> 1) & 1u, p.err, 0x400u + ab, abortp);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + ab * 256u + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
                for (int sub = 0; sub < nsub; sub++) {
#pragma unroll
                    for (int ch = 0; ch < NCH; ch++) {
                        uint32_t v[32];
                        tmem_ld32(acc + (uint32_t)(sub * NCH * 32 + ch * 32), v);
                        tmem_ld_wait();
                        if (KSPLIT == 2) {
                            uint32_t u[32];
                            tmem_ld32(acc + (uint32_t)(128 + sub * NCH * 32 + ch * 32), u);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                        }
                        if (sub == nsub - 1 && ch == NCH - 1) {
                            tc_fence_before();
                            mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                        }
                        // Transposed through the warp's tile: a thread holds 32 channels of ONE pixel, and storing them as they
                        // are would make every store instruction touch 32 different 128-byte lines (the rate of such requests, not
                        // the bytes, then bounds the epilogue).  After the transposition lane c holds channel c, and for one pixel
                        // the warp stores one whole line.
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o;
                            o.x = __uint_as_float(v[j]);     o.y = __uint_as_float(v[j + 1]);
                            o.z = __uint_as_float(v[j + 2]); o.w = __uint_as_float(v[j + 3]);
                            if (p.bias) {
                                const float4 b4 = *reinterpret_cast<const float4*>(p.bias + m0 + ch * 32 + j);
                                o.x += b4.x; o.y += b4.y; o.z += b4.z; o.w += b4.w;
                            }
                            *reinterpret_cast<float4*>(&stat_tile[wq][lane][j]) = o;
                        }
                        __syncwarp();
                        {
                            // the warp's 32 pixels: 4 image rows x 8 columns starting at (h0, w0)
                            const int w0 = tw * kTW, h0 = th * kTH + sub * 16 + q * 4;
                            const int wlim = p.Wo - w0, hlim = p.Ho - h0;
                            float* pb = p.D + (((long long)n * p.Ho + h0) * p.Wo + w0) * p.ldd + m0 + ch * 32 + lane;
                            const int rowstep = p.Wo * p.ldd;
                            float a = 0.f, b = 0.f;
                            if (wlim >= 8 && hlim >= 4 && !want_stat) {
#pragma unroll
                                for (int k = 0; k < 32; k++) pb[(k >> 3) * rowstep + (k & 7) * p.ldd] = stat_tile[wq][k][lane];
                            } else if (wlim >= 8 && hlim >= 4) {
#pragma unroll
                                for (int k = 0; k < 32; k++) {
                                    const float o = stat_tile[wq][k][lane];
                                    pb[(k >> 3) * rowstep + (k & 7) * p.ldd] = o;
                                    a += o;
                                    b = fmaf(o, o, b);
                                }
                            } else {
#pragma unroll
                                for (int k = 0; k < 32; k++)
                                    if ((k & 7) < wlim && (k >> 3) < hlim) {
                                        const float o = stat_tile[wq][k][lane];
                                        pb[(k >> 3) * rowstep + (k & 7) * p.ldd] = o;
                                        a += o;
                                        b = fmaf(o, o, b);
                                    }
                            }
                            fs[ch] += (double)a;
                            fq[ch] += (double)b;
                        }
                        __syncwarp();
                    }
                }
            }
            if (want_stat && stat_m0 >= 0) flush_stats(stat_m0);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // A wait expired somewhere: give copies still in flight time to land before the shared memory is released.
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// dwh_kernel
// ------------------------------------------------------------------------------------------
struct DwhParams {
    float* partial;        // [splits][Cout][kH * kW * Cin]
    int Cout, Cin, kH, kW, pad;
    int TW, R, PW;         // pixel tile: TW pixels x R image rows per stage; x halo line pitch PW = TW + kW - 1
    int tiles_w, hblocks;  // pixel tiles per image row, row blocks per image
    int units_total;       // images * hblocks * tiles_w
    int units_per_split, splits;
    int items;             // work items per split
    int cigs;              // groups of input-channel chunks (item dimension)
    int G;                 // SHIFT: 32-channel chunks of x per item (1 or 2)
    int ncol;              // MMA N
    int a_stride, b_stride;  // bytes between the chunk copies of an operand inside a stage (multiples of 1024)
    int a_bytes, b_bytes;    // bytes one chunk copy delivers
    int stage_bytes, stages;
    int nissue;            // MMA-issuing warps: one per accumulator column block (kW of them, or kH when SHIFT)
    unsigned int* err;
};

constexpr int kDwhMaxStages = 8;

// SHIFT = false: A = dY (128 output channels), B = x halo (128 input channels), work item = (channel tile, input
//                channel group, filter row kh), accumulator kw at column kw * 128.
// SHIFT = true:  A = x halo chunk with LBO = one pixel row (M = 4 shifts x 32 channels), B = dY (ncol output channels),
//                work item = (output channel tile, group of G input chunks), accumulator (g, kh) at column (g * kH + kh) * ncol.
template <bool SHIFT>
__global__ void __launch_bounds__(256, 1)
dwh_kernel(const __grid_constant__ CUtensorMap tmDy, const __grid_constant__ CUtensorMap tmX, const DwhParams p) {
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t bar_full[kDwhMaxStages];
    __shared__ __align__(8) uint64_t bar_empty[kDwhMaxStages];
    __shared__ __align__(8) uint64_t bar_acc_full;
    __shared__ __align__(8) uint64_t bar_acc_empty;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    const int STAGES = p.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), (uint32_t)p.nissue);
        }
        mbar_init(smem_u32(&bar_acc_full), (uint32_t)p.nissue);
        mbar_init(smem_u32(&bar_acc_empty), 128);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abortp = &abort_flag;
    const int total_work = p.items * p.splits;   // w -> (item fastest, then split): CTAs that run together share pixels
    const int ksteps_w = p.TW >> 3;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer ----------------
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
                const int item = w % p.items, z = w / p.items;
                int co0, ci0, kh0, nA, nB;
                if (!SHIFT) {
                    kh0 = item % p.kH;
                    const int t2 = item / p.kH;
                    ci0 = (t2 % p.cigs) * 128;
                    co0 = (t2 / p.cigs) * 128;
                    nA = (p.Cout - co0) >= 128 ? 4 : (p.Cout - co0) / 32;
                    nB = 4;
                } else {
                    kh0 = 0;
                    const int cig = item % p.cigs;
                    ci0 = cig * p.G * 32;
                    co0 = (item / p.cigs) * p.ncol;
                    nA = (p.Cin / 32 - cig * p.G) < p.G ? (p.Cin / 32 - cig * p.G) : p.G;
                    nB = p.ncol / 32;
                }
                const uint32_t bytes = (uint32_t)(nA * p.a_bytes + nB * p.b_bytes);
                const int u0 = z * p.units_per_split;
                const int u1 = (u0 + p.units_per_split) < p.units_total ? (u0 + p.units_per_split) : p.units_total;
                int tw = u0 % p.tiles_w, t3 = u0 / p.tiles_w;
                int hb = t3 % p.hblocks, n = t3 / p.hblocks;
                for (int u = u0; u < u1; u++) {
                    if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, p.err, 0x900u + s, abortp)) { ok = false; break; }
                    const uint32_t full = smem_u32(&bar_full[s]);
                    mbar_expect_tx(full, bytes);
                    const uint32_t a_dst = tiles_base + (uint32_t)s * (uint32_t)p.stage_bytes;
                    const uint32_t b_dst = a_dst + (uint32_t)(SHIFT ? p.G : 4) * (uint32_t)p.a_stride;
                    const int w0 = tw * p.TW, h0 = hb * p.R;
                    if (!SHIFT) {
                        for (int c = 0; c < nA; c++) tma_4d(a_dst + (uint32_t)(c * p.a_stride), &tmDy, co0 + 32 * c, w0, h0, n, full);
                        for (int c = 0; c < nB; c++) tma_4d(b_dst + (uint32_t)(c * p.b_stride), &tmX, ci0 + 32 * c, w0 - p.pad, h0 + kh0 - p.pad, n, full);
                    } else {
                        for (int c = 0; c < nA; c++) tma_4d(a_dst + (uint32_t)(c * p.a_stride), &tmX, ci0 + 32 * c, w0 - p.pad, h0 - p.pad, n, full);
                        for (int c = 0; c < nB; c++) tma_4d(b_dst + (uint32_t)(c * p.b_stride), &tmDy, co0 + 32 * c, w0, h0, n, full);
                    }
                    if (++tw == p.tiles_w) { tw = 0; if (++hb == p.hblocks) { hb = 0; n++; } }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1 || warp >= 6) {
        // ---------------- MMA issuers: warps 1, 6, 7; each owns one accumulator block (a filter column kw, or a filter
        // row kh when SHIFT).  MMAs into one accumulator must come from one thread to stay ordered; different
        // accumulators may be issued in parallel, which is what keeps the tensor pipe fed: one thread issues an MMA
        // with fresh descriptors only every hundred-odd cycles, more than an N <= 128 MMA takes.  The whole warp runs
        // the loop, lane 0 issues.
        const int iss = warp == 1 ? 0 : warp - 5;
        if (iss < p.nissue) {
            const uint32_t leader = lane == 0 ? 1u : 0u;
            // MN-major operands: rows are reduction indices (pixels), 128 B = 32 channels each; 4-row swizzle atoms 512 B
            // apart along the reduction (SBO), 32-channel chunks LBO apart; a k-step is 8 consecutive pixel rows.
            const uint32_t idesc = idesc_tf32(128u, (uint32_t)p.ncol, true, true);
            // Every value below is derived from kernel parameters, the block index and warp-wide votes only, and every
            // branch condition is the same in all lanes: the loop is provably warp-uniform.
            const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
            const uint64_t dA0 = smem_desc(tiles_base, SHIFT ? 128u : (uint32_t)p.a_stride, 512u, 1u);
            const uint64_t dB0 = smem_desc(tiles_base + (uint32_t)(SHIFT ? p.G : 4) * (uint32_t)p.a_stride, (uint32_t)p.b_stride, 512u, 1u);
            const uint32_t a_hi = (uint32_t)(dA0 >> 32), b_hi = (uint32_t)(dB0 >> 32);
            const uint32_t a_lo0 = (uint32_t)dA0, b_lo0 = (uint32_t)dB0;
            const uint32_t stage_units = (uint32_t)p.stage_bytes >> 4;   // descriptor start addresses count 16-byte units
            const uint32_t a_row = SHIFT ? (uint32_t)p.PW * 8u : (uint32_t)p.TW * 8u;   // one image row of the A tile
            const uint32_t b_row = SHIFT ? (uint32_t)p.TW * 8u : (uint32_t)p.PW * 8u;
            int s = 0;
            uint32_t ph = 0, work_iter = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, work_iter++) {
                const int item = w % p.items, z = w / p.items;
                int nA = 1;
                if (SHIFT) {
                    const int cig = item % p.cigs;
                    nA = (p.Cin / 32 - cig * p.G) < p.G ? (p.Cin / 32 - cig * p.G) : p.G;
                }
                const int u0 = z * p.units_per_split;
                const int u1 = (u0 + p.units_per_split) < p.units_total ? (u0 + p.units_per_split) : p.units_total;
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_acc_empty), (work_iter & 1u) ^ 1u, p.err, 0xA00u, abortp));
                if (!ok) break;
                tc_fence_after();
                uint32_t accum = 0u;
                for (int u = u0; u < u1; u++) {
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_full[s]), ph, p.err, 0xB00u + s, abortp));
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t a_r = a_lo0 + (uint32_t)s * stage_units, b_r = b_lo0 + (uint32_t)s * stage_units;
                    for (int r = 0; r < p.R; r++, a_r += a_row, b_r += b_row) {
                        uint32_t a_k = a_r, b_k = b_r;
                        for (int wk = 0; wk < ksteps_w; wk++, a_k += 64u, b_k += 64u) {   // 8 pixel rows of 128 B
                            if (!SHIFT) {
                                // this issuer's filter column: B start moved by `iss` pixel rows, accumulator block `iss`
                                umma_tf32_w(tmem_u + (uint32_t)(iss * 128), ((uint64_t)a_hi << 32) | a_k,
                                            ((uint64_t)b_hi << 32) | (b_k + (uint32_t)(iss * 8)), idesc, accum, leader);
                            } else {
                                // this issuer's filter row: A start moved by `iss` halo lines, accumulators (g, iss)
                                const uint64_t db = ((uint64_t)b_hi << 32) | b_k;
                                uint32_t a_g = a_k + (uint32_t)iss * a_row, acc = tmem_u + (uint32_t)(iss * p.ncol);
                                for (int g = 0; g < nA; g++, a_g += (uint32_t)p.a_stride >> 4, acc += (uint32_t)(p.kH * p.ncol))
                                    umma_tf32_w(acc, ((uint64_t)a_hi << 32) | a_g, db, idesc, accum, leader);
                            }
                            accum = 1u;
                        }
                    }
                    umma_commit_w(smem_u32(&bar_empty[s]), leader);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit_w(smem_u32(&bar_acc_full), leader);
            }
        }
    } else {
        // ---------------- epilogue: accumulators -> partial[z] ----------------
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const int ntaps = p.kH * p.kW;
        const size_t row_len = (size_t)ntaps * p.Cin;
        uint32_t work_iter = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total_work; w += gridDim.x, work_iter++) {
            const int item = w % p.items, z = w / p.items;
            ok = mbar_wait(smem_u32(&bar_acc_full), work_iter & 1u, p.err, 0xC00u, abortp);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16);
            float* pz = p.partial + (size_t)z * p.Cout * row_len;
            if (!SHIFT) {
                const int kh0 = item % p.kH;
                const int t2 = item / p.kH;
                const int ci0 = (t2 % p.cigs) * 128, co = (t2 / p.cigs) * 128 + r;
                const bool co_ok = co < p.Cout;
                for (int kw = 0; kw < p.kW; kw++) {
                    float* dst = pz + (size_t)co * row_len + (size_t)(kh0 * p.kW + kw) * p.Cin + ci0;
#pragma unroll 1
                    for (int c0 = 0; c0 < 128; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(acc + (uint32_t)(kw * 128 + c0), v);
                        tmem_ld_wait();
                        if (co_ok) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(dst + c0 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                                       __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        }
                    }
                }
            } else {
                // lane r = (pixel shift kw = q, input channel lane); columns = output channels
                const int cig = item % p.cigs;
                const int co0 = (item / p.cigs) * p.ncol;
                const int nA = (p.Cin / 32 - cig * p.G) < p.G ? (p.Cin / 32 - cig * p.G) : p.G;
                if (q < p.kW) {
                    for (int g = 0; g < nA; g++) {
                        const int ci = (cig * p.G + g) * 32 + lane;
                        for (int kh = 0; kh < p.kH; kh++) {
                            float* dst = pz + (size_t)co0 * row_len + (size_t)(kh * p.kW + q) * p.Cin + ci;
#pragma unroll 1
                            for (int c0 = 0; c0 < p.ncol; c0 += 32) {
                                uint32_t v[32];
                                tmem_ld32(acc + (uint32_t)((g * p.kH + kh) * p.ncol + c0), v);
                                tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 32; j++) dst[(size_t)(c0 + j) * row_len] = __uint_as_float(v[j]);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_acc_empty));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
template <bool PXM, int NCH, bool DUAL = false>
static int convh_launch(const CUtensorMap& tw, const CUtensorMap& tx, ConvhParams& p, int smem, double flops, cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        NCC_TRY(cudaFuncSetAttribute(convh_kernel<PXM, NCH, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     2 * 46 * 1024 + 6 * kWTileBytes + 1024));
        attr_set = true;
    }
    const long long total = (long long)p.tiles_px * p.tiles_m;
    const int sms = ncc::sm_count();
    const unsigned grid = (unsigned)(total < sms ? total : sms);
    const long long rows = (long long)(p.tiles_px / (p.tiles_w * p.tiles_h)) * p.Ho * p.Wo;
    // an input-gradient call whose output feeds an announced BatchNorm+ReLU backward sums for it on the way out
    const ncc::BnFold* fold = ncc::bn_fold_active();
    const unsigned slabs = PXM ? grid : 2 * grid;   // channels on M: two epilogue warps per channel, each with sums of its own
    // (channels-on-M kernel only: its eight epilogue warps absorb the extra work; with the pixels on M the four epilogue warps
    // are the slower side of a tile already and the sums cost more there than the reduction they replace)
    if (!PXM && fold && fold->C == p.M && fold->rows == rows && p.ldd == p.M && !p.bias) {
        p.stat = ncc::bn_fold_buffer(slabs, p.M, st);
        if (p.stat) {
            p.bnx = fold->x; p.bn_mean = fold->mean; p.bn_var = fold->var; p.bn_gamma = fold->gamma; p.bn_beta = fold->beta;
            p.bn_eps = fold->eps;
        }
    } else if (ncc::conv_stats_wanted()) {
        p.stat = ncc::conv_stats_buffer(slabs, p.M, st);
    }
    {
        ncc::ProfScope prof(ncc::prof_role(), flops, st, true);
        convh_kernel<PXM, NCH, DUAL><<<grid, PXM ? (NCH <= 2 ? 288 : 224) : (DUAL ? 352 : 320), smem, st>>>(tw, tx, p);
    }
    NCC_COUNT_LAUNCH();
    if (p.bnx) ncc::bn_fold_publish(p.D, (int)slabs, p.stat);
    else if (p.stat) ncc::conv_stats_publish(p.D, p.M, rows, (int)slabs, p.stat);
    return ncc::launch_status("convh_kernel");
}

int conv_halo_nhwc(float* y, const float* x, const float* wpacked, const float* bias, int N, int H, int W, int Cin, int Cout,
                   int kH, int kW, int pad, int mode, cudaStream_t st) {
    const int Ho = H + 2 * pad - kH + 1, Wo = W + 2 * pad - kW + 1;
    if (mode != NC_CUDA_MATH_TF32) return NC_CUDA_ERR_UNSUPPORTED;   // no operand-conversion stage in this kernel
    if (kH < 1 || kW < 1 || kH > 3 || kW > 3 || Ho <= 0 || Wo <= 0) return NC_CUDA_ERR_UNSUPPORTED;
    if ((Cin % 32) || (Cout % 4) || Cout < 16) return NC_CUDA_ERR_UNSUPPORTED;
    if ((long long)N * Ho * Wo * Cout >= 0x7fffffffLL) return NC_CUDA_ERR_UNSUPPORTED;
    // Tiles are 8 pixels wide and up to 32 high.  With the channels on M one thread issues all MMAs of a tile, which
    // only keeps the tensor pipe busy with N = 8 * rows = 256.  Images of exactly 16 rows go two to a tile (DUAL, channels on
    // M only); other images lower than 24 rows run faster on the per-tap kernel, whose 256-pixel boxes span several images.
    const bool dual = Ho == 16 && (N % 2 == 0) && !(Cout % 32 == 0 && Cout <= 96);
    if (Ho < 24 && !dual) return NC_CUDA_ERR_UNSUPPORTED;
    // Pixels on M for up to 96 output channels (measured on the 64-channel 64 x 64 layer at batch 256: 447 against 344
    // TFLOP/s with the channels on M); from 128 channels on, channels on M with N = 256 pixels is the faster shape
    // (698 against 636 TFLOP/s on the 128-channel 32 x 32 layer).
    const int ncol = Cout;
    const bool pxm = (Cout % 32 == 0) && Cout <= 96 && (bias == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15u) == 0) &&
                     (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
    CUtensorMap tw, tx;
    unsigned long long wd[2] = {(unsigned long long)Cin, (unsigned long long)kH * kW * Cout};
    unsigned long long ws[1] = {(unsigned long long)Cin};
    unsigned wb[2] = {32, (unsigned)(pxm ? ncol : 128)};
    if (!make_map(&tw, wpacked, 2, wd, ws, wb, false)) return NC_CUDA_ERR_UNSUPPORTED;
    unsigned long long dims[4] = {(unsigned long long)Cin, (unsigned long long)W, (unsigned long long)H, (unsigned long long)N};
    unsigned long long str[3] = {(unsigned long long)Cin, (unsigned long long)W * Cin, (unsigned long long)H * W * Cin};
    unsigned box[4] = {32, (unsigned)(kTW + kW - 1), (unsigned)(dual ? Ho + kH - 1 : kTH + kH - 1), dual ? 2u : 1u};
    if (!make_map(&tx, x, 4, dims, str, box, false)) return NC_CUDA_ERR_UNSUPPORTED;
    ConvhParams p = {};
    p.D = y; p.ldd = Cout; p.bias = bias; p.M = Cout;
    p.Ho = dual ? 2 * Ho : Ho; p.Wo = Wo;   // DUAL: N / 2 "images" of 32 rows as far as the output is concerned
    p.tiles_w = (Wo + kTW - 1) / kTW; p.tiles_h = (p.Ho + kTH - 1) / kTH;
    p.tiles_px = (dual ? N / 2 : N) * p.tiles_w * p.tiles_h;
    p.half_rows = Ho + kH - 1;
    p.tiles_m = pxm ? Cout / ncol : (Cout + kBM - 1) / kBM;
    p.kH = kH; p.kW = kW; p.pad = pad;
    p.cchunks = Cin / 32;
    p.wrows = Cout;
    p.wbox_bytes = (pxm ? ncol : 128) * 128;
    // Taps per weight stage: as many as leave two stages in the 96 KB weight region, spread evenly over the stages of a
    // chunk.  Every stage costs each issuing warp a barrier round trip of ~200 cycles during which it issues nothing, so
    // two large stages beat four small ones (64 channels, 64 x 64: five taps per stage 487 / 499 TFLOP/s against 447 / 467
    // with three); 128-row weight tiles (channels on M) fit three taps, a filter row, as before.
    {
        const int ntaps = kH * kW;
        int fit = (3 * kWTileBytes) / p.wbox_bytes;
        if (fit > ntaps) fit = ntaps;
        if (fit < 1) fit = 1;
        const int per_chunk = (ntaps + fit - 1) / fit;
        p.tps = (ntaps + per_chunk - 1) / per_chunk;
    }
    p.wslot_bytes = (p.tps * p.wbox_bytes + 1023) & ~1023;
    p.wstages = 6 * kWTileBytes / p.wslot_bytes;
    if (p.wstages > kConvhWStages) p.wstages = kConvhWStages;
    p.pitch = kTW + kW - 1;
    p.halo_bytes = p.pitch * (dual ? 2 * (Ho + kH - 1) : kTH + kH - 1) * 128;
    p.halo_stride = (p.halo_bytes + 1023) & ~1023;
    p.err = ncc::device_error_word();
    const int smem = 2 * p.halo_stride + 6 * kWTileBytes + 1024;
    const double flops = 2.0 * N * Ho * Wo * (double)Cout * Cin * kH * kW;
    if (pxm) {
        switch (ncol / 32) {
            case 1: return convh_launch<true, 1>(tw, tx, p, smem, flops, st);
            case 2: return convh_launch<true, 2>(tw, tx, p, smem, flops, st);
            case 3: return convh_launch<true, 3>(tw, tx, p, smem, flops, st);
        }
    }
    if (dual) return convh_launch<false, 0, true>(tw, tx, p, smem, flops, st);
    return convh_launch<false, 0>(tw, tx, p, smem, flops, st);
}

// Pixel tile of the weight-gradient kernels: TW pixels (a multiple of 8, at most 64) by R image rows per stage, chosen
// to waste the fewest tensor-core cycles on pixels beyond the image edge while at least `min_stages` stages fit.
static bool pick_dw_tile(int Wo, int Ho, int kW, int halo_rows, int nchunk_dy, int nchunk_x, int min_stages, int* TW, int* R,
                         int* stage_bytes, int* a_stride_dy, int* b_stride_x) {
    double best = -1.0;
    for (int tw = 8; tw <= 64; tw += 8) {
        const int tiles_w = (Wo + tw - 1) / tw;
        for (int r = 1; r <= 8; r *= 2) {
            if (tw * r > 256 || (r > 1 && r > Ho)) continue;
            const int dy_stride = ((tw * r * 128) + 1023) & ~1023;
            const int x_stride = (((tw + kW - 1) * (r + halo_rows) * 128 + 256) + 1023) & ~1023;   // + two rows: the unused shifts read past the last line
            const int sb = nchunk_dy * dy_stride + nchunk_x * x_stride;
            if (sb * min_stages > kMaxDynSmem - 1024) continue;
            const int hblocks = (Ho + r - 1) / r;
            const double useful = (double)Wo * Ho / ((double)tiles_w * tw * hblocks * r);
            // prefer useful pixels, then stages of up to 128 pixels (fewer barrier round trips: measured 6 % on the 56 x 56
            // layer, 56 x 2 against 8 x 8 pixels per stage) weighed against the halo lines read again per stage
            const int px = tw * r;
            const double score = useful * 1000.0 - (double)(r + halo_rows) / r * 10.0 + (px < 128 ? px : 128) * 0.2 + px * 1e-3;
            if (score > best) { best = score; *TW = tw; *R = r; *stage_bytes = sb; *a_stride_dy = dy_stride; *b_stride_x = x_stride; }
        }
    }
    return best >= 0.0;
}

int conv_dw_halo_nhwc(float* dW, const float* dy, const float* x, int N, int H, int W, int Cin, int Cout, int kH, int kW, int pad,
                      int mode, cudaStream_t st) {
    const int Ho = H + 2 * pad - kH + 1, Wo = W + 2 * pad - kW + 1;
    if (mode != NC_CUDA_MATH_TF32) return NC_CUDA_ERR_UNSUPPORTED;
    if (kH < 1 || kW < 2 || kH > 3 || kW > 3 || Ho <= 0 || Wo <= 0) return NC_CUDA_ERR_UNSUPPORTED;
    if ((Cin % 32) || (Cout % 32)) return NC_CUDA_ERR_UNSUPPORTED;
    if ((long long)N * Ho * Wo < 4096) return NC_CUDA_ERR_UNSUPPORTED;   // too few pixels to split over the GPU
    const bool shift = (Cin % 128) != 0;
    DwhParams p = {};
    p.Cout = Cout; p.Cin = Cin; p.kH = kH; p.kW = kW; p.pad = pad;
    int dy_stride = 0, x_stride = 0;
    if (!shift) {
        p.ncol = 128; p.G = 4;
        p.cigs = Cin / 128;
        p.items = ((Cout + 127) / 128) * p.cigs * kH;
        if (!pick_dw_tile(Wo, Ho, kW, 0, 4, 4, 3, &p.TW, &p.R, &p.stage_bytes, &dy_stride, &x_stride)) return NC_CUDA_ERR_UNSUPPORTED;
        p.a_stride = dy_stride; p.b_stride = x_stride;
    } else {
        // one accumulator per (input chunk, filter row): kH * G * ncol <= 512 columns
        p.ncol = Cout >= 128 ? 128 : Cout;            // Cout % 32 == 0: 32, 64, 96 or 128
        if (Cout > 128 && Cout % 128) return NC_CUDA_ERR_UNSUPPORTED;
        p.G = (kH * 2 * p.ncol <= 512 && Cin >= 64) ? 2 : 1;
        p.cigs = (Cin / 32 + p.G - 1) / p.G;
        p.items = (Cout / p.ncol) * p.cigs;
        // two large stages beat three smaller ones here (measured: 64 -> 64 at 64 x 64 184 -> 173 us, 64 -> 128 at 32 x 32
        // 83 -> 75 us; the other variant loses 10 % with two): three issuing warps stop at every stage barrier together
        if (!pick_dw_tile(Wo, Ho, kW, kH - 1, p.ncol / 32, p.G, 2, &p.TW, &p.R, &p.stage_bytes, &dy_stride, &x_stride)) return NC_CUDA_ERR_UNSUPPORTED;
        p.a_stride = x_stride; p.b_stride = dy_stride;
    }
    p.PW = p.TW + kW - 1;
    p.nissue = shift ? kH : kW;
    p.tiles_w = (Wo + p.TW - 1) / p.TW;
    p.hblocks = (Ho + p.R - 1) / p.R;
    p.units_total = N * p.hblocks * p.tiles_w;
    const int dy_bytes = p.TW * p.R * 128, x_bytes = p.PW * (p.R + (shift ? kH - 1 : 0)) * 128;
    p.a_bytes = shift ? x_bytes : dy_bytes;
    p.b_bytes = shift ? dy_bytes : x_bytes;
    p.stages = (kMaxDynSmem - 1024) / p.stage_bytes;
    if (p.stages > kDwhMaxStages) p.stages = kDwhMaxStages;
    if (p.stages < 2) return NC_CUDA_ERR_UNSUPPORTED;
    const int sms = ncc::sm_count();
    int splits = sms / p.items;
    if (splits < 1) splits = 1;
    if (splits > p.units_total / 4) splits = p.units_total / 4 > 0 ? p.units_total / 4 : 1;
    p.units_per_split = (p.units_total + splits - 1) / splits;
    p.splits = (p.units_total + p.units_per_split - 1) / p.units_per_split;
    const size_t partial_bytes = sizeof(float) * (size_t)p.splits * Cout * kH * kW * Cin;
    if (partial_bytes > (size_t)512 << 20) return NC_CUDA_ERR_UNSUPPORTED;
    p.partial = (float*)ncc::scratch(2, partial_bytes, st);
    if (!p.partial) return NC_CUDA_ERR_RUNTIME;
    p.err = ncc::device_error_word();
    CUtensorMap tdy, tx;
    {
        unsigned long long dims[4] = {(unsigned long long)Cout, (unsigned long long)Wo, (unsigned long long)Ho, (unsigned long long)N};
        unsigned long long str[3] = {(unsigned long long)Cout, (unsigned long long)Wo * Cout, (unsigned long long)Ho * Wo * Cout};
        unsigned box[4] = {32, (unsigned)p.TW, (unsigned)p.R, 1};
        if (!make_map(&tdy, dy, 4, dims, str, box, true)) return NC_CUDA_ERR_UNSUPPORTED;
        unsigned long long xd[4] = {(unsigned long long)Cin, (unsigned long long)W, (unsigned long long)H, (unsigned long long)N};
        unsigned long long xs[3] = {(unsigned long long)Cin, (unsigned long long)W * Cin, (unsigned long long)H * W * Cin};
        unsigned xbox[4] = {32, (unsigned)p.PW, (unsigned)(p.R + (shift ? kH - 1 : 0)), 1};
        if (!make_map(&tx, x, 4, xd, xs, xbox, true)) return NC_CUDA_ERR_UNSUPPORTED;
    }
    const int smem = p.stages * p.stage_bytes + 1024;
    const long long total = (long long)p.items * p.splits;
    const unsigned grid = (unsigned)(total < sms ? total : sms);
    const double flops = 2.0 * N * Ho * Wo * (double)Cout * Cin * kH * kW;
    static bool attr_set[2] = {false, false};
    if (!attr_set[shift ? 1 : 0]) {
        if (shift) NCC_TRY(cudaFuncSetAttribute(dwh_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
        else NCC_TRY(cudaFuncSetAttribute(dwh_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
        attr_set[shift ? 1 : 0] = true;
    }
    {
        ncc::ProfScope prof(ncc::prof_role(), flops, st, true);
        if (shift) dwh_kernel<true><<<grid, 256, smem, st>>>(tdy, tx, p);
        else dwh_kernel<false><<<grid, 256, smem, st>>>(tdy, tx, p);
    }
    NCC_COUNT_LAUNCH();
    const int rc = ncc::launch_status("dwh_kernel");
    if (rc) return rc;
    return dw_reduce(dW, p.partial, p.splits, Cout, Cin, kH, kW, st);
}

}  // namespace tc
