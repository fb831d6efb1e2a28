// Tensor-core contractions for sm_100a: TMA-fed, tcgen05.mma (kind::tf32) with the accumulator in
// tensor memory, written with inline PTX.  tc_kernel serves four problem kinds; the halo-resident convolution and
// weight-gradient kernels, which take the stride-1 filters up to 3 x 3 in plain TF32 mode, live in tc_conv.cu.
//
//   GEMM   D(M,N) = A * B^T        either operand K-major or MN-major in memory
//   CONV   channels-last implicit GEMM, stride 1: rows = 128 output pixels (a w x h x n box),
//          cols = output channels, reduction = (kh, kw, 32-channel chunk).  The activation tile of
//          one reduction step is ONE 4-D TMA box at shifted (w, h) coordinates; out-of-bounds
//          elements are zero-filled by TMA, which is the padding.  Used for forward and, with
//          flipped / channel-transposed weights, for dX.
//   CONVT  the same convolution with the operand roles swapped: rows = 128 output channels (the weight
//          tile is the A operand), cols = 256 output pixels (one 4-D TMA box is the B operand).  A
//          tcgen05.mma (kind::tf32, one CTA) takes max(N / 2, operand bytes / 128, about 46) cycles
//          whatever M is, so M = 128 with N >= 128 is the full-rate shape; with pixels on N that holds
//          for any channel count >= 128, while few channels on N (N = 64: 48 cycles) would not.
//   DW     weight gradient: rows = output channels, cols = (kh, kw, ci), reduction = 32-pixel
//          boxes; both operands MN-major; split over the reduction with an ordered second stage.
//
// CTA = 6 warps (kernels with an MN-major operand add up to five more TMA-issuing warps): warp 0 issues TMA, warp 1
// allocates TMEM and issues MMAs (one lane), warps 2-5
// convert operands in shared memory when the math mode asks for it (round-to-nearest TF32, or the
// hi/lo split of 3xTF32) and then run the epilogue (tcgen05.ld -> registers -> global).
// Every mbarrier wait is bounded: on expiry the kernel records a code in the device error word,
// drains, frees its TMEM and returns.
//
// No cluster launch and no multicast anywhere: each CTA loads its own tiles.
#include "tc_gemm.cuh"
#include "tc_ptx.cuh"
#include "../../include/nocta_cuda.h"

namespace tc {

enum { KIND_GEMM = 0, KIND_CONV = 1, KIND_DW = 2, KIND_CONVT = 3 };

struct TcParams {
    int kind;
    int M, N;              // logical output extent (store masks)
    int num_k_tiles;       // reduction tiles in total
    int k_tiles_per_split; // reduction tiles per blockIdx.z
    float* D;
    long long ldd;
    const float* bias;
    float alpha, beta;
    float* partial;        // non-null: raw accumulators go to partial[z][M][N]
    // pixel-box geometry (CONV: 128-pixel output box; DW: 32-pixel reduction box)
    int bw, bh, bn;
    int tiles_w, tiles_h;
    int Ho, Wo, Nimg;
    int kW, pad;
    int cchunks;           // CONV: 32-channel chunks of the reduction channels
    int wrows;             // CONV: rows per (kh,kw) block of the packed weights (= output channels)
    int Cin;               // DW: input channels (column index -> (shift, ci))
    int lbw, lbh;                  // CONVT: log2 of the pixel box width / height
    int tiles_m, tiles_n, splits;  // persistent tile walk
    int stages;                    // operand ring depth
    double* stat;                  // CONVT, non-null: per CTA and channel (sum, sum of squares) of the output it wrote, [gridDim.x][M][2]
    unsigned int* err;
    double flops;                  // host only: algorithmic FLOPs of the launch, for the profiling scope
};

// ------------------------------------------------------------------------------------------
// The kernel
// ------------------------------------------------------------------------------------------
constexpr int BM = 128;
constexpr int BK = 32;                 // 32 floats = one 128-byte swizzle row
constexpr int A_BYTES = BM * BK * 4;   // 16 KB
constexpr int CHUNK_BYTES = 32 * BK * 4;  // one 32 x 32 MN-major chunk: 4 KB
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 196 * 1024;  // one persistent CTA per SM

template <int BN, int MODE>
struct TileCfg {
    static constexpr int B_BYTES = BN * BK * 4;
    static constexpr int OPER_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGE_BYTES = OPER_BYTES * (MODE == 2 ? 2 : 1);
    static constexpr int STAGES_RAW = kSmemBudget / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > kMaxStages ? kMaxStages : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // + alignment slack
    static constexpr int ACC_COLS = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);
    // 3xTF32 spreads the reduction over several accumulators (round-robin per k-step) and adds them
    // in FP32 in the epilogue: the tensor core's own accumulation is the largest error term left in
    // that mode and it grows with the number of additions into one accumulator.
    static constexpr int NACC = MODE == 2 ? (512 / ACC_COLS > 4 ? 4 : 512 / ACC_COLS) : 1;
    // plain TF32 keeps two accumulator buffers so the epilogue of one tile overlaps the MMAs of the next;
    // the converting modes use the epilogue warps during the main loop, so one buffer is enough there
    static constexpr int NBUF = MODE == 0 ? 2 : 1;
    static constexpr int TMEM_COLS = ACC_COLS * NACC * NBUF;
};

// MN-major operands arrive as one copy per 32-wide chunk (up to 12 per stage) and a thread spends on the
// order of a hundred cycles per copy it issues, so those kernels run extra producer warps (warps 6..,
// lane 0 each): up to two producers share the A chunks and up to four the B chunks, round-robin.  Every
// producer waits for the ring slot itself and arms the stage barrier with its own byte count.
template <bool A_MN, bool B_MN, int BN>
struct ProdCfg {
    static constexpr bool MULTI = A_MN || B_MN;
    static constexpr int NA_OWNERS = !MULTI ? 1 : (A_MN ? 2 : 1);
    static constexpr int NB_OWNERS = !MULTI ? 0 : (B_MN ? (BN / 32 < 4 ? BN / 32 : 4) : 1);
    static constexpr int NPROD = MULTI ? NA_OWNERS + NB_OWNERS : 1;
    static constexpr int THREADS = 192 + 32 * (NPROD - 1);
};

template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(352, 1)
tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcParams p) {
    using Cfg = TileCfg<BN, MODE>;
    constexpr int NBUF = Cfg::NBUF;  // accumulator buffers in tensor memory (2 = epilogue overlaps the next tile)
    const int STAGES = p.stages;
    extern __shared__ uint8_t dyn_smem[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages];
    __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
    __shared__ __align__(8) uint64_t bar_conv[kMaxStages];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles_base = (smem_u32(dyn_smem) + 1023u) & ~1023u;
    uint8_t* tiles_generic = dyn_smem + (tiles_base - smem_u32(dyn_smem));

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(&bar_full[s]), (uint32_t)ProdCfg<A_MN, B_MN, BN>::NPROD);
            mbar_init(smem_u32(&bar_empty[s]), 1);
            mbar_init(smem_u32(&bar_conv[s]), 128);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 128);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"((uint32_t)Cfg::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abortp = &abort_flag;

    // Persistent CTA: walks output tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...
    // t -> (n_tile fastest, then m_tile, then reduction split z).
    const int total_tiles = p.tiles_m * p.tiles_n * p.splits;

    if (ProdCfg<A_MN, B_MN, BN>::MULTI && (warp == 0 || warp >= 6)) {
        // ------------------------------ TMA producers (MN-major operands) ------------------------------
        if (lane == 0) {
            using PC = ProdCfg<A_MN, B_MN, BN>;
            const int me = warp == 0 ? 0 : warp - 5;  // producer index
            const bool forA = me < PC::NA_OWNERS;
            const int own = forA ? me : me - PC::NA_OWNERS;         // first chunk this producer owns
            const int step = forA ? PC::NA_OWNERS : PC::NB_OWNERS;  // and the stride to its next one
            constexpr int NACH = A_MN ? BM / 32 : 1;  // copies of operand A per stage
            constexpr int NBCH = B_MN ? BN / 32 : 1;  // copies of operand B per stage
            // 32-wide chunks that lie entirely beyond the matrix edge (rows >= M, columns >= N) are not copied at
            // all: their accumulator rows / columns are never stored, and skipping them saves issue slots and
            // shared-memory writes (Cout = 64 fills only two of the four A chunks).
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int n_tile = t % p.tiles_n, r_ = t / p.tiles_n, m_tile = r_ % p.tiles_m, z = r_ / p.tiles_m;
                const int kt_begin = z * p.k_tiles_per_split;
                int kt_end = kt_begin + p.k_tiles_per_split;
                if (kt_end > p.num_k_tiles) kt_end = p.num_k_tiles;
                const int m0 = m_tile * BM, n0 = n_tile * BN;
                const int edge = forA ? p.M - m0 : p.N - n0;  // chunks starting at or beyond it are skipped
                int my_n = 0;                                 // copies this producer issues per stage of this tile
                for (int c = own; c < (forA ? NACH : NBCH); c += step) my_n += (32 * c < edge) ? 1 : 0;
                const bool chunked = forA ? A_MN : B_MN;
                const uint32_t my_bytes = chunked ? (uint32_t)my_n * CHUNK_BYTES : (forA ? (uint32_t)A_BYTES : (uint32_t)Cfg::B_BYTES);
                int dtw = 0, dth = 0, dtn = 0;
                // DW: (first channel, tap) of this producer's B chunks
                int ci0[4] = {0, 0, 0, 0}, dkh[4] = {0, 0, 0, 0}, dkw[4] = {0, 0, 0, 0};
                if (p.kind == KIND_DW) {
                    dtw = kt_begin % p.tiles_w;
                    const int tt = kt_begin / p.tiles_w;
                    dth = tt % p.tiles_h; dtn = tt / p.tiles_h;
                    if (!forA) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int col = n0 + 32 * (own + i * step);
                            const int sh = col / p.Cin;
                            ci0[i] = col - sh * p.Cin;
                            dkh[i] = sh / p.kW; dkw[i] = sh - dkh[i] * p.kW;
                        }
                    }
                }
                for (int kt = kt_begin; kt < kt_end; kt++) {
                    if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, p.err, 0x100u + s, abortp)) { ok = false; break; }
                    const uint32_t full = smem_u32(&bar_full[s]);
                    const uint32_t a_dst = tiles_base + (uint32_t)s * Cfg::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_BYTES;
                    if (my_bytes == 0) {
                        mbar_arrive(full);
                    } else {
                        mbar_expect_tx(full, my_bytes);
                        if (p.kind == KIND_GEMM) {
                            const int k0 = kt * BK;
                            if (forA) {
                                if (!A_MN) tma_2d(a_dst, &tmA, k0, m0, full);
                                else {
#pragma unroll
                                    for (int i = 0; i < 4; i++) {
                                        const int c = own + i * step;
                                        if (c < NACH && 32 * c < edge) tma_2d(a_dst + c * CHUNK_BYTES, &tmA, m0 + 32 * c, k0, full);
                                    }
                                }
                            } else if (!B_MN) {
                                tma_2d(b_dst, &tmB, k0, n0, full);
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const int c = own + i * step;
                                    if (c < NBCH && 32 * c < edge) tma_2d(b_dst + c * CHUNK_BYTES, &tmB, n0 + 32 * c, k0, full);
                                }
                            }
                        } else {  // KIND_DW (both operands MN-major)
                            const int w0 = dtw * p.bw, h0 = dth * p.bh, nn0 = dtn * p.bn;
                            if (forA) {
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const int c = own + i * step;
                                    if (c < NACH && 32 * c < edge) tma_4d(a_dst + c * CHUNK_BYTES, &tmA, m0 + 32 * c, w0, h0, nn0, full);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const int c = own + i * step;
                                    if (c < NBCH && 32 * c < edge) tma_4d(b_dst + c * CHUNK_BYTES, &tmB, ci0[i], w0 + dkw[i] - p.pad, h0 + dkh[i] - p.pad, nn0, full);
                                }
                            }
                        }
                    }
                    if (p.kind == KIND_DW) {
                        if (++dtw == p.tiles_w) { dtw = 0; if (++dth == p.tiles_h) { dth = 0; dtn++; } }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            // One thread feeds the whole CTA, so its loop is kept free of divisions and runtime modulo:
            // ring slot / phase, filter tap and channel chunk are running counters.
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int n_tile = t % p.tiles_n, r_ = t / p.tiles_n, m_tile = r_ % p.tiles_m, z = r_ / p.tiles_m;
                const int kt_begin = z * p.k_tiles_per_split;
                int kt_end = kt_begin + p.k_tiles_per_split;
                if (kt_end > p.num_k_tiles) kt_end = p.num_k_tiles;
                const int m0 = m_tile * BM, n0 = n_tile * BN;
                // pixel box of this tile (CONV: the m tile, CONVT: the n tile)
                int pw0 = 0, ph0 = 0, pn0 = 0;
                if (p.kind == KIND_CONV || p.kind == KIND_CONVT) {
                    const int pt = p.kind == KIND_CONV ? m_tile : n_tile;
                    const int tw = pt % p.tiles_w, tt = pt / p.tiles_w;
                    pw0 = tw * p.bw; ph0 = (tt % p.tiles_h) * p.bh; pn0 = (tt / p.tiles_h) * p.bn;
                }
                // running decomposition of kt: CONV/CONVT (tap kh,kw ; chunk cc), DW (box tw,th,tn)
                int cc = 0, kh = 0, kw = 0, shift = 0, dtw = 0, dth = 0, dtn = 0, dw_ci0 = 0, dw_kh0 = 0, dw_kw0 = 0;
                if (p.kind == KIND_CONV || p.kind == KIND_CONVT) {
                    shift = kt_begin / p.cchunks; cc = kt_begin - shift * p.cchunks;
                    kh = shift / p.kW; kw = shift - kh * p.kW;
                } else if (p.kind == KIND_DW) {
                    dtw = kt_begin % p.tiles_w;
                    const int tt = kt_begin / p.tiles_w;
                    dth = tt % p.tiles_h; dtn = tt / p.tiles_h;
                    const int dshift = n0 / p.Cin;
                    dw_ci0 = n0 - dshift * p.Cin;
                    dw_kh0 = dshift / p.kW; dw_kw0 = dshift - dw_kh0 * p.kW;
                }
                for (int kt = kt_begin; kt < kt_end; kt++) {
                    if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, p.err, 0x100u + s, abortp)) { ok = false; break; }
                    const uint32_t full = smem_u32(&bar_full[s]);
                    mbar_expect_tx(full, (uint32_t)Cfg::OPER_BYTES);
                    const uint32_t a_dst = tiles_base + (uint32_t)s * Cfg::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_BYTES;
                    if (p.kind == KIND_GEMM) {
                        const int k0 = kt * BK;
                        if (!A_MN) {
                            tma_2d(a_dst, &tmA, k0, m0, full);
                        } else {
#pragma unroll
                            for (int c = 0; c < BM / 32; c++) tma_2d(a_dst + c * CHUNK_BYTES, &tmA, m0 + 32 * c, k0, full);
                        }
                        if (!B_MN) {
                            tma_2d(b_dst, &tmB, k0, n0, full);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 32; c++) tma_2d(b_dst + c * CHUNK_BYTES, &tmB, n0 + 32 * c, k0, full);
                        }
                    } else if (p.kind == KIND_CONV) {
                        tma_4d(a_dst, &tmA, cc * 32, pw0 + kw - p.pad, ph0 + kh - p.pad, pn0, full);
                        tma_2d(b_dst, &tmB, cc * 32, shift * p.wrows + n0, full);
                    } else if (p.kind == KIND_CONVT) {
                        tma_2d(a_dst, &tmA, cc * 32, shift * p.wrows + m0, full);
                        tma_4d(b_dst, &tmB, cc * 32, pw0 + kw - p.pad, ph0 + kh - p.pad, pn0, full);
                    } else {
                        const int w0 = dtw * p.bw, h0 = dth * p.bh, nn0 = dtn * p.bn;
#pragma unroll
                        for (int c = 0; c < BM / 32; c++) tma_4d(a_dst + c * CHUNK_BYTES, &tmA, m0 + 32 * c, w0, h0, nn0, full);
                        // column chunk c covers columns n0 + 32c .. : (tap, ci0) advance by 32 channels per chunk
                        int ci0 = dw_ci0, dkh = dw_kh0, dkw = dw_kw0;
#pragma unroll
                        for (int c = 0; c < BN / 32; c++) {
                            tma_4d(b_dst + c * CHUNK_BYTES, &tmB, ci0, w0 + dkw - p.pad, h0 + dkh - p.pad, nn0, full);
                            ci0 += 32;
                            if (ci0 >= p.Cin) { ci0 = 0; if (++dkw == p.kW) { dkw = 0; dkh++; } }
                        }
                        if (++dtw == p.tiles_w) { dtw = 0; if (++dth == p.tiles_h) { dth = 0; dtn++; } }
                    }
                    if (p.kind == KIND_CONV || p.kind == KIND_CONVT) {
                        if (++cc == p.cchunks) { cc = 0; shift++; if (++kw == p.kW) { kw = 0; kh++; } }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            // instruction descriptor: D = f32, A = B = tf32, majors, N, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // K-major: 8-row groups 1024 B apart (SBO); a k-step of 8 floats advances 32 B inside the swizzle row.
            // MN-major: rows are reduction indices, 128 B (32 elements of M/N) each; the swizzle atom is
            // 4 rows (SBO = 512 B between atoms along k), 32-element chunks are CHUNK_BYTES apart (LBO);
            // a k-step of 8 rows advances 1024 B.
            const uint32_t lbo_a = A_MN ? CHUNK_BYTES : 16u, sbo_a = A_MN ? 512u : 1024u;
            const uint32_t lbo_b = B_MN ? CHUNK_BYTES : 16u, sbo_b = B_MN ? 512u : 1024u;
            const uint32_t lay_a = A_MN ? 1u : 2u, lay_b = B_MN ? 1u : 2u;
            const uint32_t kstep_a = A_MN ? 1024u : 32u, kstep_b = B_MN ? 1024u : 32u;
            // descriptors are built once; a ring slot or k-step only moves the 14-bit start-address field
            const uint64_t da0 = smem_desc(tiles_base, lbo_a, sbo_a, lay_a);
            const uint64_t db0 = smem_desc(tiles_base + A_BYTES, lbo_b, sbo_b, lay_b);
            int s = 0;
            uint32_t ph = 0, tile_iter = 0;
            bool ok = true;
            // A barrier test takes this thread well over a hundred cycles before its result can be used, about as long as
            // issuing two MMAs.  The state of the NEXT stage's barrier is therefore requested before this stage's MMAs
            // are issued and only looked at afterwards: with the producers ahead it is already set, and the wait at
            // the top of the next round is skipped.
            bool known_ready = false;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, tile_iter++) {
                const int z = (t / p.tiles_n) / p.tiles_m;
                const int kt_begin = z * p.k_tiles_per_split;
                int kt_end = kt_begin + p.k_tiles_per_split;
                if (kt_end > p.num_k_tiles) kt_end = p.num_k_tiles;
                const int nk = kt_end - kt_begin;
                const uint32_t ab = tile_iter % NBUF;
                // wait until the epilogue has drained this accumulator buffer (first use passes at once)
                if (!mbar_wait(smem_u32(&bar_acc_empty[ab]), ((tile_iter / NBUF) & 1u) ^ 1u, p.err, 0x500u + ab, abortp)) { ok = false; break; }
                tc_fence_after();
                const uint32_t acc_base = tmem_base + ab * (uint32_t)(Cfg::NACC * Cfg::ACC_COLS);
                for (int i = 0; i < nk; i++) {
                    const uint32_t ready = MODE == 0 ? smem_u32(&bar_full[s]) : smem_u32(&bar_conv[s]);
                    if (!known_ready && !mbar_wait(ready, ph, p.err, 0x200u + s, abortp)) { ok = false; break; }
                    tc_fence_after();
                    {
                        const int s1 = (s + 1 == STAGES) ? 0 : s + 1;
                        const uint32_t ph1 = (s + 1 == STAGES) ? (ph ^ 1u) : ph;
                        known_ready = mbar_test(MODE == 0 ? smem_u32(&bar_full[s1]) : smem_u32(&bar_conv[s1]), ph1);
                    }
                    const uint64_t soff = (uint64_t)(((uint32_t)s * (uint32_t)Cfg::STAGE_BYTES) >> 4);
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ks++) {
                        const uint64_t da = da0 + soff + (uint64_t)((ks * kstep_a) >> 4);
                        const uint64_t db = db0 + soff + (uint64_t)((ks * kstep_b) >> 4);
                        if (MODE == 2) {
                            // accumulator (ks % NACC); small cross terms first, then the main product
                            const uint32_t acc = acc_base + (uint32_t)((ks % Cfg::NACC) * Cfg::ACC_COLS);
                            const bool first = (i == 0) && (ks < Cfg::NACC);
                            const uint64_t da_lo = da + (uint64_t)(Cfg::OPER_BYTES >> 4);
                            const uint64_t db_lo = db + (uint64_t)(Cfg::OPER_BYTES >> 4);
                            umma_tf32(acc, da_lo, db, idesc, first ? 0u : 1u);
                            umma_tf32(acc, da, db_lo, idesc, 1u);
                            umma_tf32(acc, da, db, idesc, 1u);
                        } else {
                            umma_tf32(acc_base, da, db, idesc, (uint32_t)((i | ks) != 0));
                        }
                    }
                    umma_commit(smem_u32(&bar_empty[s]));
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(smem_u32(&bar_acc_full[ab]));
            }
        }
    } else if (warp < 6) {
        // ------------------------------ converter + epilogue warps ------------------------------
        const int te = threadIdx.x - 64;  // 0..127
        const int q = warp & 3;           // TMEM lane quadrant this warp may read
        const int r = q * 32 + lane;
        int s = 0;
        uint32_t ph = 0, tile_iter = 0;
        bool ok = true;
        // CONVT output statistics: one running pair per channel tile, written once per CTA (see convh_kernel)
        double ssum = 0.0, ssq = 0.0;
        int stat_m0 = -1;
        if (p.kind == KIND_CONVT && p.stat)
            for (int mt = 0; mt < p.tiles_m; mt++)
                if (mt * BM + r < p.M) {
                    double* sd = p.stat + ((size_t)blockIdx.x * p.M + mt * BM + r) * 2;
                    sd[0] = 0.0; sd[1] = 0.0;
                }
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, tile_iter++) {
            const int n_tile = t % p.tiles_n, r_ = t / p.tiles_n, m_tile = r_ % p.tiles_m, z = r_ / p.tiles_m;
            const int kt_begin = z * p.k_tiles_per_split;
            int kt_end = kt_begin + p.k_tiles_per_split;
            if (kt_end > p.num_k_tiles) kt_end = p.num_k_tiles;
            const int nk = kt_end - kt_begin;
            const int m0 = m_tile * BM, n0 = n_tile * BN;
            if (p.kind == KIND_CONVT && p.stat && m0 != stat_m0) {
                if (stat_m0 >= 0 && stat_m0 + r < p.M) {
                    double* sd = p.stat + ((size_t)blockIdx.x * p.M + stat_m0 + r) * 2;
                    sd[0] = ssum; sd[1] = ssq;
                }
                ssum = 0.0; ssq = 0.0; stat_m0 = m0;
            }
            if (MODE != 0) {
                constexpr int NV = Cfg::OPER_BYTES / 16;
                for (int i = 0; i < nk && ok; i++) {
                    if (!mbar_wait(smem_u32(&bar_full[s]), ph, p.err, 0x300u + s, abortp)) { ok = false; break; }
                    float4* buf = reinterpret_cast<float4*>(tiles_generic + (size_t)s * Cfg::STAGE_BYTES);
                    float4* lo = reinterpret_cast<float4*>(tiles_generic + (size_t)s * Cfg::STAGE_BYTES + Cfg::OPER_BYTES);
                    for (int j = te; j < NV; j += 128) {
                        float4 v = buf[j];
                        float4 h = make_float4(ncc::round_tf32(v.x), ncc::round_tf32(v.y), ncc::round_tf32(v.z), ncc::round_tf32(v.w));
                        buf[j] = h;
                        if (MODE == 2)
                            lo[j] = make_float4(ncc::round_tf32(v.x - h.x), ncc::round_tf32(v.y - h.y),
                                                ncc::round_tf32(v.z - h.z), ncc::round_tf32(v.w - h.w));
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(smem_u32(&bar_conv[s]));
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            const uint32_t ab = tile_iter % NBUF;
            if (ok) ok = mbar_wait(smem_u32(&bar_acc_full[ab]), (tile_iter / NBUF) & 1u, p.err, 0x400u + ab, abortp);
            // all 32 lanes of a warp must agree before the aligned tcgen05.ld
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc_base = tmem_base + ab * (uint32_t)(Cfg::NACC * Cfg::ACC_COLS);
            if (p.kind == KIND_CONVT) {
                // lane = output channel, column = pixel of the box; channels-last store: for one column the
                // 32 lanes of a warp write 32 consecutive floats
                const int co = m0 + r;
                const bool co_ok = co < p.M;
                const float bv = (co_ok && p.bias) ? p.bias[co] : 0.f;
                const int tw = n_tile % p.tiles_w, tt = n_tile / p.tiles_w;
                const int pw0 = tw * p.bw, ph0 = (tt % p.tiles_h) * p.bh, pn0 = (tt / p.tiles_h) * p.bn;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    float fs = 0.f, fq = 0.f;  // output statistics over the pixels of this chunk that exist
                    uint32_t v[32];
                    tmem_ld32(acc_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (Cfg::NACC > 1) {
#pragma unroll 1
                        for (int a = 1; a < Cfg::NACC; a++) {
                            uint32_t u[32];
                            tmem_ld32(acc_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * Cfg::ACC_COLS + c0), u);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                        }
                    }
                    if (c0 + 32 >= BN) {
                        tc_fence_before();
                        mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                    }
                    // the 32 columns of a chunk are runs of consecutive w inside one image row: the 64-bit
                    // address is formed once per run, each store then adds a small constant multiple of ldd
                    const int ldd = (int)p.ldd;
                    if (p.bw >= 32) {
                        const int w = pw0 + (c0 & (p.bw - 1));
                        const int h = ph0 + ((c0 >> p.lbw) & (p.bh - 1));
                        const int n = pn0 + (c0 >> (p.lbw + p.lbh));
                        if (co_ok && h < p.Ho && n < p.Nimg) {
                            float* dst = p.D + (((long long)n * p.Ho + h) * p.Wo + w) * p.ldd + co;
                            const int lim = p.Wo - w;  // columns j < lim are inside the image
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < lim) {
                                    const float o = __uint_as_float(v[j]) + bv;
                                    dst[j * ldd] = o;
                                    if (p.stat) { fs += o; fq = fmaf(o, o, fq); }
                                }
                        }
                    } else {
#pragma unroll
                        for (int j0 = 0; j0 < 32; j0 += 8) {  // bw is 8 or 16: runs of 8 never cross a row
                            const int pj = c0 + j0;
                            const int w = pw0 + (pj & (p.bw - 1));
                            const int h = ph0 + ((pj >> p.lbw) & (p.bh - 1));
                            const int n = pn0 + (pj >> (p.lbw + p.lbh));
                            if (co_ok && h < p.Ho && n < p.Nimg) {
                                float* dst = p.D + (((long long)n * p.Ho + h) * p.Wo + w) * p.ldd + co;
                                const int lim = p.Wo - w;
#pragma unroll
                                for (int j = 0; j < 8; j++)
                                    if (j < lim) {
                                        const float o = __uint_as_float(v[j0 + j]) + bv;
                                        dst[j * ldd] = o;
                                        if (p.stat) { fs += o; fq = fmaf(o, o, fq); }
                                    }
                            }
                        }
                    }
                    ssum += (double)fs;
                    ssq += (double)fq;
                }
                continue;
            }
            // where does this row go?
            long long row_off = -1;
            if (p.kind == KIND_CONV) {
                const int tw = m_tile % p.tiles_w, tt = m_tile / p.tiles_w;
                const int cw0 = tw * p.bw, ch0 = (tt % p.tiles_h) * p.bh, cn0 = (tt / p.tiles_h) * p.bn;
                const int iw = r % p.bw, t2 = r / p.bw, ih = t2 % p.bh, in_ = t2 / p.bh;
                const int w = cw0 + iw, h = ch0 + ih, n = cn0 + in_;
                if (w < p.Wo && h < p.Ho && n < p.Nimg) row_off = (((long long)n * p.Ho + h) * p.Wo + w) * p.ldd;
            } else {
                const int m = m0 + r;
                if (m < p.M) row_off = p.partial ? ((long long)z * p.M + m) * p.N : (long long)m * p.ldd;
            }
            float* base = p.partial ? p.partial : p.D;
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) &&
                                (((p.partial ? (long long)p.N : p.ldd) & 3) == 0);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= p.N) break;  // uniform across the CTA
                uint32_t v[32];
                tmem_ld32(acc_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
                tmem_ld_wait();
                if (Cfg::NACC > 1) {
#pragma unroll 1
                    for (int a = 1; a < Cfg::NACC; a++) {
                        uint32_t u[32];
                        tmem_ld32(acc_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * Cfg::ACC_COLS + c0), u);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(u[j]));
                    }
                }
                if (c0 + 32 >= BN || n0 + c0 + 32 >= p.N) {
                    // last chunk read: the accumulator buffer may be overwritten by the tile after next
                    tc_fence_before();
                    mbar_arrive(smem_u32(&bar_acc_empty[ab]));
                }
                if (row_off < 0) continue;
                float* dst = base + row_off + n0 + c0;
                const int ncols = (p.N - (n0 + c0)) < 32 ? (p.N - (n0 + c0)) : 32;
                if (p.partial) {
                    if (vec_ok && ncols == 32) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                              __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (j < ncols) dst[j] = __uint_as_float(v[j]);
                    }
                } else {
                    const float* bias = p.bias ? p.bias + n0 + c0 : nullptr;
                    if (vec_ok && ncols == 32) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float4 o = make_float4(p.alpha * __uint_as_float(v[j]), p.alpha * __uint_as_float(v[j + 1]),
                                                   p.alpha * __uint_as_float(v[j + 2]), p.alpha * __uint_as_float(v[j + 3]));
                            if (p.beta != 0.f) {
                                float4 old = *reinterpret_cast<const float4*>(dst + j);
                                o.x += p.beta * old.x; o.y += p.beta * old.y; o.z += p.beta * old.z; o.w += p.beta * old.w;
                            }
                            if (bias) { o.x += bias[j]; o.y += bias[j + 1]; o.z += bias[j + 2]; o.w += bias[j + 3]; }
                            *reinterpret_cast<float4*>(dst + j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            if (j < ncols) {
                                float o = p.alpha * __uint_as_float(v[j]);
                                if (p.beta != 0.f) o += p.beta * dst[j];
                                if (bias) o += bias[j];
                                dst[j] = o;
                            }
                        }
                    }
                }
            }
        }
        if (p.kind == KIND_CONVT && p.stat && stat_m0 >= 0 && stat_m0 + r < p.M) {
            double* sd = p.stat + ((size_t)blockIdx.x * p.M + stat_m0 + r) * 2;
            sd[0] = ssum; sd[1] = ssq;
        }
    }

    // ------------------------------ teardown ------------------------------
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // A wait expired somewhere: give copies still in flight time to land before the CTA's
        // shared memory is released.
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// Second stages and weight packing
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) splitk_reduce_kernel(float* __restrict__ D, long long ldd, const float* __restrict__ partial,
                                                            int splits, int M, int N, const float* __restrict__ bias,
                                                            float alpha, float beta) {
    const size_t total = (size_t)M * N, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        double acc = 0.0;   // the splits are combined in double, in order: no rounding that grows with their number
        int z = 0;
        for (; z + 8 <= splits; z += 8) {   // eight loads requested before the first one is added
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) v[k] = partial[(size_t)(z + k) * total + i];
#pragma unroll
            for (int k = 0; k < 8; k++) acc += (double)v[k];
        }
        for (; z < splits; z++) acc += (double)partial[(size_t)z * total + i];
        const int m = (int)(i / N), n = (int)(i % N);
        float* d = D + (size_t)m * ldd + n;
        float o = alpha * (float)acc;
        if (beta != 0.f) o += beta * *d;
        if (bias) o += bias[n];
        *d = o;
    }
}

// partial[z][co][(kh*kW+kw)*Cin + ci]  ->  dW[co][ci][kh][kw].  Threads walk the SOURCE order (coalesced reads of every split;
// walking the destination order reads with a stride of Cin floats, eight times the sectors), eight splits are requested
// before the first one is added, and only the single write per element is scattered.
__global__ void __launch_bounds__(256) dw_reduce_kernel(float* __restrict__ dW, const float* __restrict__ partial, int splits,
                                                        int Cout, int Cin, int kH, int kW) {
    const int T = kH * kW;
    const size_t total = (size_t)Cout * Cin * T, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t src = (size_t)blockIdx.x * blockDim.x + threadIdx.x; src < total; src += stride) {
        double acc = 0.0;
        int z = 0;
        for (; z + 8 <= splits; z += 8) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 8; k++) v[k] = partial[(size_t)(z + k) * total + src];
#pragma unroll
            for (int k = 0; k < 8; k++) acc += (double)v[k];
        }
        for (; z < splits; z++) acc += (double)partial[(size_t)z * total + src];
        const int ci = (int)(src % Cin);
        const size_t r = src / Cin;
        const int tap = (int)(r % T);
        const size_t co = r / T;
        dW[(co * Cin + ci) * T + tap] = (float)acc;
    }
}

template <bool DX>
__global__ void __launch_bounds__(256) pack_weights_kernel(float* __restrict__ wp, const float* __restrict__ w, int Cout, int Cin,
                                                           int kH, int kW, int round) {
    const size_t total = (size_t)Cout * Cin * kH * kW, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t r = i;
        int kh, kw, co, ci;
        if (!DX) {  // dst (kh, kw, co, ci)
            ci = r % Cin; r /= Cin; co = r % Cout; r /= Cout; kw = r % kW; kh = (int)(r / kW);
        } else {    // dst (kh', kw', ci, co), source taps flipped
            co = r % Cout; r /= Cout; ci = r % Cin; r /= Cin; kw = r % kW; kh = (int)(r / kW);
            kh = kH - 1 - kh; kw = kW - 1 - kw;
        }
        float v = w[(((size_t)co * Cin + ci) * kH + kh) * kW + kw];
        wp[i] = round ? ncc::round_tf32(v) : v;
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
template <int BN, bool A_MN, bool B_MN, int MODE>
static int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p_in, dim3 tiles, cudaStream_t st) {
    using Cfg = TileCfg<BN, MODE>;
    TcParams p = p_in;
    p.tiles_n = (int)tiles.x; p.tiles_m = (int)tiles.y; p.splits = (int)tiles.z;
    p.stages = Cfg::STAGES;
    const long long total = (long long)tiles.x * tiles.y * tiles.z;
    const int sms = ncc::sm_count();
    dim3 grid((unsigned)(total < sms ? total : sms), 1, 1);
    static bool attr_set = false;
    auto kern = tc_kernel<BN, A_MN, B_MN, MODE>;
    if (!attr_set) {
        NCC_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set = true;
    }
    {
        ncc::ProfScope prof(ncc::prof_role(), p.flops, st, true);
        kern<<<grid, ProdCfg<A_MN, B_MN, BN>::THREADS, Cfg::SMEM_BYTES, st>>>(ta, tb, p);
    }
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("tc_kernel");
}

template <int BN, bool A_MN, bool B_MN>
static int launch_mode(int mode, const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p, dim3 grid, cudaStream_t st) {
    switch (mode) {
        case NC_CUDA_MATH_TF32: return launch_one<BN, A_MN, B_MN, 0>(ta, tb, p, grid, st);
        case NC_CUDA_MATH_TF32_RNA: return launch_one<BN, A_MN, B_MN, 1>(ta, tb, p, grid, st);
        case NC_CUDA_MATH_3XTF32: return launch_one<BN, A_MN, B_MN, 2>(ta, tb, p, grid, st);
    }
    return ncc::set_status(NC_CUDA_ERR_ARG, "tc: unknown math mode %d", mode);
}

template <bool A_MN, bool B_MN>
static int launch_bn(int bn, int mode, const CUtensorMap& ta, const CUtensorMap& tb, const TcParams& p, dim3 grid, cudaStream_t st) {
    switch (bn) {
        case 64: return launch_mode<64, A_MN, B_MN>(mode, ta, tb, p, grid, st);
        case 128: return launch_mode<128, A_MN, B_MN>(mode, ta, tb, p, grid, st);
        case 256: return launch_mode<256, A_MN, B_MN>(mode, ta, tb, p, grid, st);
    }
    return ncc::set_status(NC_CUDA_ERR_ARG, "tc: unsupported tile width %d", bn);
}

// 3xTF32 prefers 128-column tiles: four accumulators fit in tensor memory instead of two.
static int pick_bn(int N, int mode = 0) { return N <= 64 ? 64 : ((N <= 128 || mode == NC_CUDA_MATH_3XTF32) ? 128 : 256); }

// splits over the reduction so that about one wave of CTAs exists; each split keeps >= 4 tiles
static void pick_splits(int tiles, int nk, int* splits, int* kps) {
    int s = 1;
    const int sms = ncc::sm_count();
    if (tiles * 2 <= sms && nk >= 8) {
        s = sms / tiles;
        if (s > nk / 4) s = nk / 4;
        if (s < 1) s = 1;
    }
    int per = (nk + s - 1) / s;
    *kps = per;
    *splits = (nk + per - 1) / per;
}

int gemm(float* D, int ldd, const float* A, int lda, bool a_mn, const float* B, int ldb, bool b_mn, int M, int N, int K,
         const float* bias, float alpha, float beta, int mode, cudaStream_t st) {
    // rows beyond M inside the 128-row tile are zero-filled by TMA and never stored; tiny problems stay on the SIMT kernel
    if (M < 32 || N < 16 || K < 32 || (long long)M * N * K < (1ll << 22)) return NC_CUDA_ERR_UNSUPPORTED;
    if ((lda & 3) || (ldb & 3)) return NC_CUDA_ERR_UNSUPPORTED;
    const int bn = pick_bn(N, mode);
    CUtensorMap ta, tb;
    {
        unsigned long long dims[2], str[1];
        unsigned box[2];
        if (!a_mn) { dims[0] = K; dims[1] = M; str[0] = lda; box[0] = 32; box[1] = 128; }
        else       { dims[0] = M; dims[1] = K; str[0] = lda; box[0] = 32; box[1] = 32; }
        if (!make_map(&ta, A, 2, dims, str, box, a_mn)) return NC_CUDA_ERR_UNSUPPORTED;
        if (!b_mn) { dims[0] = K; dims[1] = N; str[0] = ldb; box[0] = 32; box[1] = (unsigned)bn; }
        else       { dims[0] = N; dims[1] = K; str[0] = ldb; box[0] = 32; box[1] = 32; }
        if (!make_map(&tb, B, 2, dims, str, box, b_mn)) return NC_CUDA_ERR_UNSUPPORTED;
    }
    TcParams p = {};
    p.kind = KIND_GEMM;
    p.M = M; p.N = N;
    p.num_k_tiles = (K + BK - 1) / BK;
    p.D = D; p.ldd = ldd; p.bias = bias; p.alpha = alpha; p.beta = beta;
    p.err = ncc::device_error_word();
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
    int splits, kps;
    pick_splits(tiles_m * tiles_n, p.num_k_tiles, &splits, &kps);
    p.k_tiles_per_split = kps;
    if (splits > 1) {
        p.partial = (float*)ncc::scratch(2, sizeof(float) * (size_t)splits * M * N, st);
        if (!p.partial) return NC_CUDA_ERR_RUNTIME;
    }
    dim3 grid(tiles_n, tiles_m, splits);
    p.flops = 2.0 * M * (double)N * K;
    int rc;
    if (!a_mn && !b_mn) rc = launch_bn<false, false>(bn, mode, ta, tb, p, grid, st);
    else if (!a_mn && b_mn) rc = launch_bn<false, true>(bn, mode, ta, tb, p, grid, st);
    else if (a_mn && !b_mn) rc = launch_bn<true, false>(bn, mode, ta, tb, p, grid, st);
    else rc = launch_bn<true, true>(bn, mode, ta, tb, p, grid, st);
    if (rc) return rc;
    if (splits > 1) {
        splitk_reduce_kernel<<<ncc::grid_for((long long)M * N, 256), 256, 0, st>>>(D, ldd, p.partial, splits, M, N, bias, alpha, beta);
        NCC_COUNT_LAUNCH();
        return ncc::launch_status("splitk_reduce");
    }
    return NC_CUDA_OK;
}

// Pixel box (bw, bh, bn) with bw*bh*bn == pixels that wastes the fewest rows for this image size.
static void pick_box(int pixels, int Wd, int Hd, int Nd, int* bw, int* bh, int* bn, int min_w = 1) {
    long long best = -1;
    for (int w = min_w; w <= pixels; w *= 2)
        for (int h = 1; w * h <= pixels; h *= 2) {
            int n = pixels / (w * h);
            if (w * h * n != pixels || w > 256 || h > 256 || n > 256) continue;
            long long cover = (long long)((Wd + w - 1) / w) * w * ((Hd + h - 1) / h) * h * ((Nd + n - 1) / n) * n;
            // prefer less waste, then wider rows (longer contiguous runs), then fewer images per box
            if (best < 0 || cover < best || (cover == best && (w > *bw || (w == *bw && n < *bn)))) {
                best = cover; *bw = w; *bh = h; *bn = n;
            }
        }
}

int conv_nhwc(float* y, const float* x, const float* wpacked, const float* bias, int N, int H, int W, int Cin, int Cout,
              int kH, int kW, int pad, int mode, cudaStream_t st) {
    const int Ho = H + 2 * pad - kH + 1, Wo = W + 2 * pad - kW + 1;
    if (Ho <= 0 || Wo <= 0) return NC_CUDA_ERR_UNSUPPORTED;
    if ((Cin & 3) || (Cout & 3) || Cin < 16 || Cout < 16) return NC_CUDA_ERR_UNSUPPORTED;
    if ((long long)N * Ho * Wo < 128) return NC_CUDA_ERR_UNSUPPORTED;
    {
        const int rc = conv_halo_nhwc(y, x, wpacked, bias, N, H, W, Cin, Cout, kH, kW, pad, mode, st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    if ((long long)N * Ho * Wo >= 1024 && kH * kW * Cout >= 128) {
        // pixels on the N side (256 per tile), channels on the M side
        int bw = 1, bh = 1, bnn = 1;
        pick_box(256, Wo, Ho, N, &bw, &bh, &bnn, 8);
        CUtensorMap ta, tb;
        unsigned long long wd[2] = {(unsigned long long)Cin, (unsigned long long)kH * kW * Cout};
        unsigned long long ws[1] = {(unsigned long long)Cin};
        unsigned wb[2] = {32, 128};
        if (!make_map(&ta, wpacked, 2, wd, ws, wb, false)) return NC_CUDA_ERR_UNSUPPORTED;
        unsigned long long dims[4] = {(unsigned long long)Cin, (unsigned long long)W, (unsigned long long)H, (unsigned long long)N};
        unsigned long long str[3] = {(unsigned long long)Cin, (unsigned long long)W * Cin, (unsigned long long)H * W * Cin};
        unsigned box[4] = {32, (unsigned)bw, (unsigned)bh, (unsigned)bnn};
        if (!make_map(&tb, x, 4, dims, str, box, false)) return NC_CUDA_ERR_UNSUPPORTED;
        TcParams p = {};
        p.kind = KIND_CONVT;
        p.M = Cout;
        p.cchunks = (Cin + 31) / 32;
        p.num_k_tiles = kH * kW * p.cchunks;
        p.k_tiles_per_split = p.num_k_tiles;
        p.D = y; p.ldd = Cout; p.bias = bias; p.alpha = 1.f; p.beta = 0.f;
        p.bw = bw; p.bh = bh; p.bn = bnn;
        for (p.lbw = 0; (1 << p.lbw) < bw; p.lbw++) {}
        for (p.lbh = 0; (1 << p.lbh) < bh; p.lbh++) {}
        p.tiles_w = (Wo + bw - 1) / bw; p.tiles_h = (Ho + bh - 1) / bh;
        p.Ho = Ho; p.Wo = Wo; p.Nimg = N;
        p.kW = kW; p.pad = pad; p.wrows = Cout;
        p.err = ncc::device_error_word();
        const long long tiles_px = (long long)p.tiles_w * p.tiles_h * ((N + bnn - 1) / bnn);
        p.N = (int)(tiles_px * 256 < 0x7fffffffLL ? tiles_px * 256 : 0x7fffffff);
        dim3 tiles((unsigned)tiles_px, (unsigned)((Cout + BM - 1) / BM), 1);
        p.flops = 2.0 * N * Ho * Wo * (double)Cout * Cin * kH * kW;
        // launch_one uses min(tiles, SMs) persistent CTAs: one statistics slab per CTA
        const long long total_tiles = (long long)tiles.x * tiles.y;
        const int n_ctas = (int)(total_tiles < ncc::sm_count() ? total_tiles : ncc::sm_count());
        if (ncc::conv_stats_wanted()) p.stat = ncc::conv_stats_buffer((size_t)n_ctas, Cout, st);
        const int rc = launch_mode<256, false, false>(mode, ta, tb, p, tiles, st);
        if (rc == NC_CUDA_OK && p.stat) ncc::conv_stats_publish(y, Cout, (long long)N * Ho * Wo, n_ctas, p.stat);
        return rc;
    }
    const int bn_cols = pick_bn(Cout, mode);
    int bw = 1, bh = 1, bnn = 1;
    pick_box(128, Wo, Ho, N, &bw, &bh, &bnn);
    CUtensorMap ta, tb;
    {
        unsigned long long dims[4] = {(unsigned long long)Cin, (unsigned long long)W, (unsigned long long)H, (unsigned long long)N};
        unsigned long long str[3] = {(unsigned long long)Cin, (unsigned long long)W * Cin, (unsigned long long)H * W * Cin};
        unsigned box[4] = {32, (unsigned)bw, (unsigned)bh, (unsigned)bnn};
        if (!make_map(&ta, x, 4, dims, str, box, false)) return NC_CUDA_ERR_UNSUPPORTED;
        unsigned long long wd[2] = {(unsigned long long)Cin, (unsigned long long)kH * kW * Cout};
        unsigned long long ws[1] = {(unsigned long long)Cin};
        unsigned wb[2] = {32, (unsigned)bn_cols};
        if (!make_map(&tb, wpacked, 2, wd, ws, wb, false)) return NC_CUDA_ERR_UNSUPPORTED;
    }
    TcParams p = {};
    p.kind = KIND_CONV;
    p.M = N * Ho * Wo; p.N = Cout;
    p.cchunks = (Cin + 31) / 32;
    p.num_k_tiles = kH * kW * p.cchunks;
    p.k_tiles_per_split = p.num_k_tiles;
    p.D = y; p.ldd = Cout; p.bias = bias; p.alpha = 1.f; p.beta = 0.f;
    p.bw = bw; p.bh = bh; p.bn = bnn;
    p.tiles_w = (Wo + bw - 1) / bw; p.tiles_h = (Ho + bh - 1) / bh;
    p.Ho = Ho; p.Wo = Wo; p.Nimg = N;
    p.kW = kW; p.pad = pad; p.wrows = Cout;
    p.err = ncc::device_error_word();
    const long long tiles_m = (long long)p.tiles_w * p.tiles_h * ((N + bnn - 1) / bnn);
    dim3 grid((Cout + bn_cols - 1) / bn_cols, (unsigned)tiles_m, 1);
    p.flops = 2.0 * N * Ho * Wo * (double)Cout * Cin * kH * kW;
    return launch_bn<false, false>(bn_cols, mode, ta, tb, p, grid, st);
}

int conv_dw_nhwc(float* dW, const float* dy, const float* x, int N, int H, int W, int Cin, int Cout, int kH, int kW, int pad,
                 int mode, cudaStream_t st) {
    const int Ho = H + 2 * pad - kH + 1, Wo = W + 2 * pad - kW + 1;
    if (Ho <= 0 || Wo <= 0) return NC_CUDA_ERR_UNSUPPORTED;
    if ((Cin & 31) || (Cout & 3) || Cout < 32) return NC_CUDA_ERR_UNSUPPORTED;
    {
        const int rc = conv_dw_halo_nhwc(dW, dy, x, N, H, W, Cin, Cout, kH, kW, pad, mode, st);
        if (rc != NC_CUDA_ERR_UNSUPPORTED) return rc;
    }
    const int Ncols = kH * kW * Cin;
    // column tile: whole filter rows when they fit in 256 columns, else 256 / 128 / 64
    int bn_cols;
    if (kW * Cin <= 256 && (kW * Cin) % 32 == 0 && (kW * Cin == 64 || kW * Cin == 128 || kW * Cin == 192 || kW * Cin == 256)) bn_cols = kW * Cin;
    else bn_cols = pick_bn(Ncols);
    int bw = 1, bh = 1, bnn = 1;
    pick_box(32, Wo, Ho, N, &bw, &bh, &bnn);
    CUtensorMap ta, tb;
    {
        unsigned long long dims[4] = {(unsigned long long)Cout, (unsigned long long)Wo, (unsigned long long)Ho, (unsigned long long)N};
        unsigned long long str[3] = {(unsigned long long)Cout, (unsigned long long)Wo * Cout, (unsigned long long)Ho * Wo * Cout};
        unsigned box[4] = {32, (unsigned)bw, (unsigned)bh, (unsigned)bnn};
        if (!make_map(&ta, dy, 4, dims, str, box, true)) return NC_CUDA_ERR_UNSUPPORTED;
        unsigned long long xd[4] = {(unsigned long long)Cin, (unsigned long long)W, (unsigned long long)H, (unsigned long long)N};
        unsigned long long xs[3] = {(unsigned long long)Cin, (unsigned long long)W * Cin, (unsigned long long)H * W * Cin};
        if (!make_map(&tb, x, 4, xd, xs, box, true)) return NC_CUDA_ERR_UNSUPPORTED;
    }
    TcParams p = {};
    p.kind = KIND_DW;
    p.M = Cout; p.N = Ncols;
    p.bw = bw; p.bh = bh; p.bn = bnn;
    p.tiles_w = (Wo + bw - 1) / bw; p.tiles_h = (Ho + bh - 1) / bh;
    p.Ho = Ho; p.Wo = Wo; p.Nimg = N;
    p.kW = kW; p.pad = pad; p.Cin = Cin;
    p.num_k_tiles = p.tiles_w * p.tiles_h * ((N + bnn - 1) / bnn);
    p.alpha = 1.f;
    p.err = ncc::device_error_word();
    const int tiles_m = (Cout + BM - 1) / BM, tiles_n = (Ncols + bn_cols - 1) / bn_cols;
    int splits, kps;
    pick_splits(tiles_m * tiles_n, p.num_k_tiles, &splits, &kps);
    p.k_tiles_per_split = kps;
    p.partial = (float*)ncc::scratch(2, sizeof(float) * (size_t)splits * Cout * Ncols, st);
    if (!p.partial) return NC_CUDA_ERR_RUNTIME;
    dim3 grid(tiles_n, tiles_m, splits);
    p.flops = 2.0 * N * Ho * Wo * (double)Cout * Cin * kH * kW;
    int rc;
    if (bn_cols == 192) rc = launch_mode<192, true, true>(mode, ta, tb, p, grid, st);
    else rc = launch_bn<true, true>(bn_cols, mode, ta, tb, p, grid, st);
    if (rc) return rc;
    return dw_reduce(dW, p.partial, splits, Cout, Cin, kH, kW, st);
}

int dw_reduce(float* dW, const float* partial, int splits, int Cout, int Cin, int kH, int kW, cudaStream_t st) {
    dw_reduce_kernel<<<ncc::grid_for((long long)Cout * Cin * kH * kW, 256), 256, 0, st>>>(dW, partial, splits, Cout, Cin, kH, kW);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("dw_reduce");
}

int pack_weights_fwd(float* wp, const float* w, int Cout, int Cin, int kH, int kW, bool round, cudaStream_t st) {
    pack_weights_kernel<false><<<ncc::grid_for((long long)Cout * Cin * kH * kW, 256), 256, 0, st>>>(wp, w, Cout, Cin, kH, kW, round ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("pack_weights_fwd");
}
int pack_weights_dx(float* wp, const float* w, int Cout, int Cin, int kH, int kW, bool round, cudaStream_t st) {
    pack_weights_kernel<true><<<ncc::grid_for((long long)Cout * Cin * kH * kW, 256), 256, 0, st>>>(wp, w, Cout, Cin, kH, kW, round ? 1 : 0);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status("pack_weights_dx");
}

}  // namespace tc
