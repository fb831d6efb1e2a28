// FP32 CUDA-core tiled GEMM with pluggable operand loaders: the exact-arithmetic path for shapes
// the tensor-core kernels cannot tile (tiny or unaligned channel counts, odd leading dimensions)
// and the device-side cross-check for them.  64x64 output tile per CTA, 4x4 per thread, BK = 16,
// optional split over the reduction dimension (blockIdx.z) with the epilogue functor deciding
// where partial sums go.
#pragma once
#include "nc_common.cuh"

namespace simt {

constexpr int TM = 64, TN = 64, TK = 16, PADN = 4;

// LA(m, k) / LB(n, k) return the operand element (0 outside the logical matrix is the loader's job
// only for conv padding; the kernel itself masks m >= M, n >= N, k >= k_end).
// A_KFAST / B_KFAST: consecutive threads walk k (true) or m/n (false) when filling the tile, chosen
// by the host so global loads coalesce along the contiguous index.
template <bool A_KFAST, bool B_KFAST, class LA, class LB, class EP>
__global__ void __launch_bounds__(256) gemm_kernel(int M, int N, int K, int k_per_split, LA la, LB lb, EP ep) {
    __shared__ __align__(16) float As[TK][TM + PADN];
    __shared__ __align__(16) float Bs[TK][TN + PADN];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN, z = blockIdx.z;
    const int kb = z * k_per_split;
    int ke = kb + k_per_split;
    if (ke > K) ke = K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int k0 = kb; k0 < ke; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int e = tid + 256 * i;
            int kk, mm;
            if (A_KFAST) { kk = e & (TK - 1); mm = e / TK; } else { mm = e & (TM - 1); kk = e / TM; }
            float v = 0.f;
            if (m0 + mm < M && k0 + kk < ke) v = la(m0 + mm, k0 + kk);
            As[kk][mm] = v;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int e = tid + 256 * i;
            int kk, nn;
            if (B_KFAST) { kk = e & (TK - 1); nn = e / TK; } else { nn = e & (TN - 1); kk = e / TN; }
            float v = 0.f;
            if (n0 + nn < N && k0 + kk < ke) v = lb(n0 + nn, k0 + kk);
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk++) {
            float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int n = n0 + tx * 4 + j;
            if (n < N) ep(z, m, n, acc[i][j]);
        }
    }
}

template <bool A_KFAST, bool B_KFAST, class LA, class LB, class EP>
inline int launch(int M, int N, int K, int splits, LA la, LB lb, EP ep, cudaStream_t st, const char* what) {
    if (M <= 0 || N <= 0) return NC_CUDA_OK;
    if (splits < 1) splits = 1;
    int kps = (K + splits - 1) / splits;
    kps = ((kps + TK - 1) / TK) * TK;
    if (kps < TK) kps = TK;
    splits = K > 0 ? (K + kps - 1) / kps : 1;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, splits);
    if (grid.y > 65535 || grid.z > 65535)
        return ncc::set_status(NC_CUDA_ERR_UNSUPPORTED, "%s: grid too large for the SIMT path", what);
    gemm_kernel<A_KFAST, B_KFAST><<<grid, 256, 0, st>>>(M, N, K, kps, la, lb, ep);
    NCC_COUNT_LAUNCH();
    return ncc::launch_status(what);
}

// number of reduction splits that actually get launched for (K, requested)
inline int effective_splits(int K, int splits) {
    if (splits < 1) splits = 1;
    int kps = (K + splits - 1) / splits;
    kps = ((kps + TK - 1) / TK) * TK;
    if (kps < TK) kps = TK;
    return K > 0 ? (K + kps - 1) / kps : 1;
}

}  // namespace simt
